// Internal C++ launch interface between the engine (engine.cu / abi.cu) and
// the kernel files.  Nothing here is exported from the shared library; the
// exported C ABI is declared in include/sd3_b200.h.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sd3 {

typedef __nv_bfloat16 bf16;

// status codes returned by launchers (negative = error); mirrored in the C ABI
enum : int {
  ST_OK = 0,
  ST_INVALID_ARG = -1,
  ST_UNSUPPORTED = -2,
  ST_CUDA_ERROR = -3,
  ST_DEVICE_TIMEOUT = -4,
  ST_NOT_READY = -5,
};

void set_last_error(const char* fmt, ...);
const char* get_last_error();
int check_cuda(cudaError_t e, const char* what);
int after_launch(const char* kernel_name);
long launch_count(int reset);

// ----------------------------------------------------------------------------
// tcgen05 GEMM:  acc[m, n] = sum_k A[m, k] * W[n, k]   (A: M x K row-major,
// W: N x K row-major, i.e. both operands K-major), fp32 accumulation in TMEM,
// followed by one of the fused epilogues below.
// ----------------------------------------------------------------------------
enum GemmEpi : int {
  EPI_BIAS = 0,        // out = acc + bias
  EPI_BIAS_GELU = 1,   // out = gelu_tanh(acc + bias)
  EPI_GATE_RESID = 2,  // out = resid + gate[b, n] * (acc + bias)         (fp32 out)
  EPI_QKV_NORM = 3,    // out = per-head RMSNorm on the q and k column ranges of (acc + bias)
  EPI_ADD_TABLE = 4,   // out = acc + bias + table[m % rows_in, n]         (fp32 out)
  EPI_UNPATCHIFY = 5,  // out[b, c, 2r+ph, 2s+pw] = acc + bias, n = ph*(p*C) + pw*C + c
};

struct GemmEpilogue {
  int mode = EPI_BIAS;
  const float* bias = nullptr;  // [N] or null
  void* out = nullptr;
  int out_f32 = 0;              // 0: bf16 output, 1: fp32 output
  int out_e4m3 = 0;             // with out_f32 == 0: one e4m3 byte per element (N % 64 == 0), the
                                // operand of a following FP8 GEMM; BIAS and BIAS_GELU modes only
  long ldo = 0;                 // output leading dimension in elements
  // Row remap: GEMM row m belongs to sample b = m / rows_in and is written to
  // output row b * rows_out + row_off + (m % rows_in).  rows_in = 0 means no remap.
  int rows_in = 0, rows_out = 0, row_off = 0;
  // EPI_GATE_RESID
  const float* gate = nullptr;  // gate[b * gate_stride + n]
  long gate_stride = 0;
  const float* resid = nullptr;  // same indexing as out; may alias out
  // EPI_QKV_NORM (head_dim 64): columns [0, qk_cols) are normalised; the first
  // half with wq, the second half with wk.  Either weight may be null (-> 1).
  const float* wq = nullptr;
  const float* wk = nullptr;
  int qk_cols = 0;
  float eps = 1e-6f;
  int do_norm = 1;
  // EPI_QKV_NORM, optional head-group layout (hg_groups > 1): the output is
  // (hg_groups, hg_rows, 3, E / hg_groups) -- slab g holds the q, k and v columns of the heads
  // of group g for every row -- instead of (rows, 3E); the send layout of a head all-to-all.
  int hg_groups = 0;
  long hg_rows = 0;
  // EPI_ADD_TABLE
  const float* table = nullptr;  // (rows_in, N) fp32
  // EPI_UNPATCHIFY
  int up_w = 0;      // patches per image row
  int up_h = 0;      // patches per image column
  int up_cin = 0;    // latent channels
  int up_patch = 0;  // patch size
  // output scale applied to the accumulator before bias (FP8 dequantisation)
  float alpha = 1.0f;
};

// dtype tags for A/W operands
enum : int { OPERAND_BF16 = 0, OPERAND_E4M3 = 1 };

int launch_gemm(const void* A, long lda, const void* W, long ldw, int operand_dtype, int M, int N,
                int K, const GemmEpilogue& epi, int* dev_status, cudaStream_t stream);

// One operand set of a grouped launch: acc = A (M x K) * W^T (N x K), then epi.
struct GemmProblem {
  const void* A = nullptr;
  long lda = 0;
  const void* W = nullptr;
  long ldw = 0;
  int M = 0;
  GemmEpilogue epi;
};
// Two GEMMs of the same N, K, operand type and epilogue kind as ONE launch when the CTA-pair
// kernel covers both (the second problem's tiles run in the tail of the first's); otherwise
// two launches.  Used for the image-stream GEMM of a block and its small context-stream twin.
int launch_gemm_grouped(const GemmProblem& a, const GemmProblem& b, int operand_dtype, int N, int K,
                        int* dev_status, cudaStream_t stream);

// ----------------------------------------------------------------------------
// Flash-style attention on tcgen05 (head_dim 64, bf16, non-causal).
// qkv: (B, T, 3*E) bf16 with q | k | v column blocks, head h at columns h*64.
// Output row t of sample b goes to out_c[(b*Tc + t), :] for t < Tc, otherwise
// to out_x[(b*(T-Tc) + t - Tc), :]; out_c may be null (context rows dropped).
// ----------------------------------------------------------------------------
// out_e4m3: out_c / out_x receive one e4m3 byte per element (rows E bytes apart) instead of bf16.
// scratch (optional, 16-byte aligned, attention_scratch_bytes(B, T, NH) bytes, which is 0 for
// shapes that fill the machine anyway): lets launches with too few CTAs split the keys of a
// query tile over several CTAs and merge the partial results.  score_bound (optional): an upper
// bound on |q . k| for every query and key, 0 if unknown; a bound of at most 80 / (scale log2 e)
// lets the softmax run without a running maximum.
int launch_attention_bf16(const bf16* qkv, int B, int T, int NH, int Tc, bf16* out_c, bf16* out_x,
                          float scale, int* dev_status, cudaStream_t stream, int out_e4m3 = 0,
                          void* scratch = nullptr, size_t scratch_bytes = 0, float score_bound = 0.0f);
size_t attention_scratch_bytes(int B, int T, int NH);

// Generic SIMT attention (any head_dim <= 128, fp32 or bf16 in, fp32 math).
// q: row (b*T + t) at base + row*ld + h*D; k, v: row (b*L + j) at base + row*ldk + h*D
// (L keys per sample; L <= 0 means L = T, ldk <= 0 means ldk = ld).  out rows split like above.
int launch_attention_simt(const void* q, const void* k, const void* v, long ld, int in_f32, int B,
                          int T, int NH, int D, int Tc, void* out_c, void* out_x, long ldo,
                          int out_f32, float scale, cudaStream_t stream, int L = 0, long ldk = 0);

// ----------------------------------------------------------------------------
// Memory-bound kernels
// ----------------------------------------------------------------------------
// LayerNorm (no affine) + up to two modulations:  out_i = LN(x) * (1 + scale_i[b]) + shift_i[b]
// x: (B*T, E) fp32.  shift/scale: [b * mod_stride + e].  out: bf16 (out_f32 = 0), fp32 (1) or
// e4m3 converted as is (2).
int launch_ln_modulate(const float* x, int B, int T, int E, float eps, const float* shift1,
                       const float* scale1, void* out1, const float* shift2, const float* scale2,
                       void* out2, long mod_stride, int out_f32, cudaStream_t stream);

// Skinny linear for M = B <= 64 rows:  out[b, n] = act_out(sum_k in[b,k] W[n,k] + bias[n] + add[b,n])
// W is (N, K) row-major, bf16 or fp32 (w_f32).  act: 0 none, 1 SiLU.
int launch_skinny_linear(const float* in, long ld_in, const void* W, int w_f32, const float* bias,
                         const float* add, long ld_add, float* out, long ld_out, int B, int N,
                         int K, int act_out, cudaStream_t stream);

// emb[b, i] = cos(t_b f_i), emb[b, half + i] = sin(t_b f_i), f_i = exp(-ln(1e4) i / half)
int launch_sinusoidal(const float* t, float* out, int B, int dim, cudaStream_t stream);

// 2-D sin-cos position table for an (h, w) patch grid centre-cropped from a
// (pmax, pmax) grid; table (h*w, E) fp32, evaluated in double precision.
int launch_pos_table(float* table, int h, int w, int E, int pmax, int base_size,
                     cudaStream_t stream);

// latent (B, C, H, W) fp32/bf16 -> patches (B*h*w, C*p*p) bf16 or fp32, k = c*p*p + ph*p + pw
int launch_patchify(const void* latent, int in_f32, void* out, int out_f32, int B, int C, int H,
                    int W, int p, cudaStream_t stream);

// generic conv2d (square stride, zero padding), in/out (B,C,H,W) fp32 or bf16, weights/bias fp32
int launch_conv2d_direct(const void* in, int io_f32, const float* w, const float* bias, void* out, int B, int C,
                         int H, int W, int O, int kh, int kw, int stride, int pad, cudaStream_t stream);

// element-wise casts / transposes used by weight packing and the per-op API
int launch_cast_f32_to_bf16(const float* in, bf16* out, long n, cudaStream_t stream);
// e4m3 operand = saturate(in * inv_scale) (round to nearest even); n % 4 == 0.
int launch_quantize_e4m3(const void* in, int in_f32, void* out, long n, float inv_scale,
                         cudaStream_t stream);
// *out = max |in[i]| (fp32, device memory)
int launch_absmax(const void* in, int in_f32, long n, float* out, cudaStream_t stream);
int launch_cast_bf16_to_f32(const bf16* in, float* out, long n, cudaStream_t stream);
// in: (R, C) row-major of in dtype -> out: (C, R) row-major of out dtype
int launch_transpose(const void* in, int in_f32, void* out, int out_f32, int R, int C,
                     cudaStream_t stream);
// per-head RMSNorm in place on rows of width ncols_total; heads of width D
// starting at column col0, nheads of them; x fp32 or bf16
int launch_rmsnorm_heads(void* x, int x_f32, long ld, long rows, int col0, int nheads, int D,
                         const float* w, float eps, cudaStream_t stream);

// fp32 SIMT GEMM with the same epilogues (exact mode and odd shapes)
int launch_gemm_f32(const float* A, long lda, const float* W /* (N,K) */, long ldw, int M, int N,
                    int K, const GemmEpilogue& epi, cudaStream_t stream);

}  // namespace sd3

/*
 * sd3_b200.h -- C ABI of libsd3_b200.so: the SD3.5-medium MMDiT-X denoiser
 * forward for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers and sizes, returns 0 on success or a
 * negative SD3_ERR_* code, never exits the process and never throws.  Unless
 * stated otherwise pointers are DEVICE pointers, `stream` is a cudaStream_t
 * passed as void*, and work is only enqueued (no synchronisation).  After a
 * failure sd3_last_error() returns a human-readable message (thread-local).
 *
 * The library is what the `custom_modules` torch extension (modules.cpp next
 * to this tree) binds; each declaration names the function of the reference
 * project (MichelHUANGGit/SD3.c, paths relative to its root) it stands in for.
 *
 * Conventions
 *   - "bf16" buffers hold __nv_bfloat16, "f32" buffers float.
 *   - dtype tags: SD3_DTYPE_F32 = 0, SD3_DTYPE_BF16 = 1.
 *   - packed weights are (out_features, in_features) row-major ("N x K",
 *     K contiguous); the reference boundary hands weights as (in, out), see
 *     sd3_pack_weight().
 */
#ifndef SD3_B200_H_
#define SD3_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SD3_API __attribute__((visibility("default")))
#else
#define SD3_API
#endif

#define SD3_OK 0
#define SD3_ERR_INVALID_ARG (-1)
#define SD3_ERR_UNSUPPORTED (-2)
#define SD3_ERR_CUDA (-3)
#define SD3_ERR_DEVICE_TIMEOUT (-4)
#define SD3_ERR_NOT_READY (-5)

#define SD3_DTYPE_F32 0
#define SD3_DTYPE_BF16 1

/* precision modes of a model */
#define SD3_PRECISION_BF16 0 /* bf16 tensor-core operands, fp32 accumulation / residual streams */
#define SD3_PRECISION_F32 1  /* exact fp32 arithmetic (parity mode for fp32 tensors) */
#define SD3_PRECISION_FP8 2  /* bf16 mode with the block GEMMs on e4m3 operands (one scale per weight matrix) */

/* epilogues of sd3_linear */
#define SD3_ACT_NONE 0
#define SD3_ACT_GELU_TANH 1

SD3_API int sd3_abi_version(void);
SD3_API const char* sd3_last_error(void);

/* Reads and clears the per-device status word that kernels set when one of
 * their bounded waits ran out (0 = healthy).  Synchronises the device.  The
 * reference has no counterpart: its kernels cannot time out and its host
 * code exits on CUDA errors (cuda/dit.cu:96,460,690,738). */
SD3_API int sd3_device_status(int* status_out);

/* ------------------------------------------------------------------------- */
/* Per-operator entry points                                                  */
/* ------------------------------------------------------------------------- */

/* out[m, n] = act(sum_k x[m,k] w[n,k] + bias[n]); x (M,K) bf16, w (N,K) bf16,
 * bias (N) f32 or NULL, out (M,N) bf16 or f32 (out_dtype).  tcgen05 GEMM.
 * Replaces launch_linear (cuda/dit.cu:683-756, cuBLASLt TF32, optional
 * GELU epilogue) and the CPU `linear` (modules.cpp:475-490). */
SD3_API int sd3_linear(const void* x_bf16, const void* w_nk_bf16, const float* bias, void* out,
               int out_dtype, int M, int N, int K, int act, void* stream);

/* The same contraction on e4m3 operands (tcgen05 kind::f8f6f4, fp32
 * accumulation): out = act(scale * sum_k x[m,k] w[n,k] + bias[n]), x (M,K) and
 * w (N,K) one byte per element, scale = the product of the two operands'
 * quantisation scales.  K must be a multiple of 16.  The reference has no
 * reduced-precision path; this is the FP8 variant of launch_linear
 * (cuda/dit.cu:683-756). */
SD3_API int sd3_linear_e4m3(const void* x_e4m3, const void* w_nk_e4m3, const float* bias, void* out,
                    int out_dtype, int M, int N, int K, float scale, int act, void* stream);

/* out[i] = e4m3(saturate(in[i] / scale)), round to nearest even; in f32 or bf16
 * (in_dtype), n a multiple of 4.  Producer of sd3_linear_e4m3 operands. */
SD3_API int sd3_quantize_e4m3(const void* in, int in_dtype, void* out_e4m3, long n, float scale,
                      void* stream);

/* Same contraction in exact fp32 arithmetic (SIMT); x, w, out are f32.
 * Replaces the CPU `linear` (modules.cpp:475-490) for fp32 tensors. */
SD3_API int sd3_linear_f32(const float* x, const float* w_nk, const float* bias, float* out, int M, int N,
                   int K, int act, void* stream);

/* resid[m, n] += gate[m / rows_per_sample, n] * (sum_k x[m,k] w[n,k] + bias[n]).
 * x (M,K) bf16, w (N,K) bf16, resid (M,N) f32 in place, gate rows gate_stride
 * floats apart.  Replaces launch_linear followed by gate_multiply_residual_add
 * (cuda/dit.cu:655-680, 862-903) / gating_mechanism + add
 * (modules.cpp:1223-1236, 513-518). */
SD3_API int sd3_linear_gate_residual(const void* x_bf16, const void* w_nk_bf16, const float* bias,
                             const float* gate, long gate_stride, int rows_per_sample,
                             float* resid, int M, int N, int K, void* stream);

/* Two sd3_linear / sd3_linear_gate_residual calls of the same N, K, activation and output
 * type as ONE launch: the tiles of the second problem run in the tail of the first's, so a
 * small GEMM (the 333-row context stream next to the image stream of the same block:
 * context_mlp / latent_mlp, context_attn_Wout / latent_attn_Wout, cuda/dit.cu:825-903) costs
 * no launch and no part-filled wave of its own.  Falls back to two launches where the
 * CTA-pair kernel does not cover both shapes.  Each problem has its own operands, weights,
 * bias (gate, residual) and row count. */
SD3_API int sd3_linear_pair(const void* x0_bf16, const void* w0_nk_bf16, const float* bias0, void* out0, int M0,
                            const void* x1_bf16, const void* w1_nk_bf16, const float* bias1, void* out1, int M1,
                            int out_dtype, int N, int K, int act, void* stream);
SD3_API int sd3_linear_gate_residual_pair(const void* x0_bf16, const void* w0_nk_bf16, const float* bias0,
                                          const float* gate0, int rows_per_sample0, float* resid0, int M0,
                                          const void* x1_bf16, const void* w1_nk_bf16, const float* bias1,
                                          const float* gate1, int rows_per_sample1, float* resid1, int M1,
                                          long gate_stride, int N, int K, void* stream);

/* QKV projection with fused per-head RMSNorm of q and k (head_dim 64) and the
 * token concatenation: row m = (b, t) of x goes to row b*T_total + row_offset
 * + t of qkv_out (B, T_total, 3E) bf16.  wq/wk are the (64,) RMSNorm weights
 * or NULL.  Replaces launch_linear + rmsnorm_key_query_kernel2 +
 * fused_concat_permute (cuda/dit.cu:825-860, 384-515) / partial_linear x3 +
 * rmsnorm_group + concatenate_along_tokens (modules.cpp:1391-1427). */
SD3_API int sd3_qkv_project(const void* x_bf16, const void* w_nk_bf16, const float* bias, const float* wq,
                    const float* wk, float eps, void* qkv_out_bf16, int B, int T_in, int T_total,
                    int row_offset, int E, void* stream);

/* QKV projection for sequence-parallel attention: out = per-head RMSNorm(x W^T + b) as in
 * sd3_qkv_project, for `rows` rows with K input features and q|k|v blocks of E_out columns
 * each (head_dim 64), written in head-group layout (head_groups, rows, 3, E_out/head_groups):
 * slab g holds the q, k and v columns of the heads of group g for every row, which is the
 * send buffer of the all-to-all that turns "my tokens x all heads" into "all tokens x my
 * heads" (head_groups = 1 gives the plain (rows, 3 E_out) layout).  K may differ from E_out,
 * so the same call projects replicated rows onto one rank's heads with a sliced weight.
 * Math: latent_to_qkv / context_to_qkv + RMSNorm, module_tests/modules.py:272-297; the
 * reference has no distributed path. */
SD3_API int sd3_qkv_project_groups(const void* x_bf16, const void* w_nk_bf16, const float* bias,
                                   const float* wq, const float* wk, float eps, void* out_bf16, int rows,
                                   int E_out, int K, int head_groups, void* stream);

/* Non-causal multi-head attention, head_dim 64, over the packed qkv buffer
 * (B, T, 3E) bf16.  Rows t < Tc of each sample are written to out_c (B, Tc, E)
 * (skipped when NULL), the others to out_x (B, T - Tc, E); both bf16.
 * Replaces mha_cuda + scale_softmax_kernel2 + fused_unpermute_split
 * (cuda/dit.cu:612-652, 548-608, 518-545) / multihead_attention +
 * split_along_tokens (modules.cpp:766-831, 1268-1294). */
SD3_API int sd3_attention(const void* qkv_bf16, int B, int T, int num_heads, int Tc, void* out_c_bf16,
                  void* out_x_bf16, float scale, void* stream);

/* sd3_attention with a scratch buffer.  Launches with too few (sample, head, query tile)
 * units to fill the GPU -- one long sequence with few heads, as on a rank of a
 * sequence-parallel run -- split the keys of every query tile over several CTAs and merge the
 * partial results; that needs sd3_attention_scratch_bytes(B, T, num_heads) bytes of scratch
 * (16-byte aligned; 0 for shapes that fill the GPU anyway, and then scratch may be null).
 * Same result as sd3_attention up to the rounding of the merge (fp32).  Replaces the same
 * reference code as sd3_attention. */
SD3_API long sd3_attention_scratch_bytes(int B, int T, int num_heads);
SD3_API int sd3_attention_ws(const void* qkv_bf16, int B, int T, int num_heads, int Tc, void* out_c_bf16,
                             void* out_x_bf16, float scale, void* scratch, long scratch_bytes, void* stream);

/* sd3_attention_ws for callers that know an upper bound on |q . k| over every query and key of
 * the call (score_bound, in raw dot-product units; 0 = unknown).  After the q/k RMSNorm of the
 * model (module_tests/modules.py:286-297) every head vector is x_hat * weight with
 * |x_hat|^2 <= head_dim, so score_bound = 64 * max_d |wq_d * wk_d| (times 1.01 for the bf16
 * rounding of q and k) holds for any input.  If score_bound * scale * log2(e) <= 80, the
 * softmax is evaluated as 2^(s c) / sum 2^(s c) without a running maximum -- identical in exact
 * arithmetic, no overflow or underflow possible within the bound, fewer instructions per score;
 * otherwise, and for score_bound <= 0, this is sd3_attention_ws.  A bound that does not hold
 * gives undefined results (inf / NaN), never a device fault.  scratch may be null.
 * scale == 0: the queries already carry scale * log2(e) (a score is its own exp2 argument);
 * score_bound is then a bound on those scores.  Accepted by sd3_attention and
 * sd3_attention_ws too. */
SD3_API int sd3_attention_bounded(const void* qkv_bf16, int B, int T, int num_heads, int Tc, void* out_c_bf16,
                                  void* out_x_bf16, float scale, float score_bound, void* scratch,
                                  long scratch_bytes, void* stream);

/* Generic attention in fp32 arithmetic for any head_dim <= 128: q, k, v are
 * (B, Tq|Tk, num_heads*head_dim) row-major with leading dimension ld elements,
 * dtype in_dtype; out (B, Tq, num_heads*head_dim) of out_dtype.  Stand-in for
 * `mha` (modules.cpp:901-918) on CUDA tensors. */
SD3_API int sd3_attention_generic(const void* q, const void* k, const void* v, long ld, int in_dtype,
                          int B, int T, int num_heads, int head_dim, void* out, long ldo,
                          int out_dtype, float scale, void* stream);

/* Attention with separate query and key lengths (fp32 arithmetic, head_dim <= 128):
 * q (B, Tq, heads*head_dim) with leading dimension ldq, k and v (B, Tk, heads*head_dim)
 * with leading dimension ldkv; out (B, Tq, heads*head_dim).  `mha` with L != T
 * (modules.cpp:901-918, module_tests/attention.py:51-83). */
SD3_API int sd3_cross_attention(const void* q, const void* k, const void* v, long ldq, long ldkv, int in_dtype,
                                int B, int Tq, int Tk, int num_heads, int head_dim, void* out, long ldo,
                                int out_dtype, float scale, void* stream);

/* Stand-alone 2-D convolution with square stride and zero padding: x (B,C,H,W) and out
 * (B,O,Ho,Wo) of io_dtype, weights (O,C,kh,kw) and bias (O) fp32; Ho = (H + 2 padding - kh) /
 * stride + 1.  Off the denoiser's path (its patch embedding is sd3_patch_embed); replaces
 * conv2d (modules.cpp:1037-1062) for the general shapes of module_tests/conv2d.py. */
SD3_API int sd3_conv2d(const void* x, int io_dtype, const float* w_f32, const float* bias, void* out, int B,
                       int C, int H, int W, int O, int kh, int kw, int stride, int padding, void* stream);

/* out_i = LayerNorm(x; eps, no affine) * (1 + scale_i[b]) + shift_i[b] for one
 * or two modulations (out2/shift2/scale2 NULL for one).  x (B*T, E) f32; the
 * modulation vectors are f32 rows mod_stride floats apart; outputs bf16 or f32.
 * Replaces layernorm_forward_kernel6 + scale_and_shift3 (cuda/dit.cu:17-99,
 * 357-381) / layernorm + scale_and_shift (modules.cpp:10-49, 1207-1221). */
SD3_API int sd3_layernorm_modulate(const float* x, int B, int T, int E, float eps, const float* shift1,
                           const float* scale1, void* out1, const float* shift2,
                           const float* scale2, void* out2, long mod_stride, int out_dtype,
                           void* stream);

/* out[b, n] = act(sum_k in[b,k] w[n,k] + bias[n] + add[b,n]) for a handful of
 * rows (the conditioning MLPs and every block's AdaLN projection in one
 * launch).  in/out/add f32, w (N,K) of w_dtype, act: 0 none, 1 SiLU.
 * Replaces launch_partial_linear (cuda/dit.cu:305-354, one 128x128-tiled SGEMM
 * launch per AdaLN chunk) / partial_linear + mlp (modules.cpp:492-511, 1120-1127). */
SD3_API int sd3_skinny_linear(const float* in, long ld_in, const void* w_nk, int w_dtype,
                      const float* bias, const float* add, long ld_add, float* out, long ld_out,
                      int B, int N, int K, int act, void* stream);

/* Sinusoidal timestep embedding, (B,) f32 -> (B, dim) f32, cos half first.
 * Replaces sinusoidal_embedding (modules.cpp:920-944). */
SD3_API int sd3_sinusoidal_embedding(const float* t, float* out, int B, int dim, void* stream);

/* 2-D sin-cos position table of an (h, w) patch grid centre-cropped from a
 * (pos_max, pos_max) grid, (h*w, E) f32.  Replaces positional_embedding2D +
 * crop_positional_embedding2D (modules.cpp:946-995). */
SD3_API int sd3_pos_embed_table(float* table, int h, int w, int E, int pos_max, int base_size,
                        void* stream);

/* Self-test of the device-side timeout path: launches a kernel whose only work is a
 * bounded wait (limit_us microseconds) on a barrier nobody arrives on.  After
 * the stream has drained, sd3_device_status reports code 199 once and clears
 * it; calls made afterwards are unaffected.  No counterpart in the reference,
 * which exits the process on CUDA errors (cuda/dit.cu:96,460,690,738). */
SD3_API int sd3_selftest_wait_timeout(int limit_us, void* stream);

/* Patch embedding: x[b, r*w+s, :] = conv(latent; kernel=stride=patch)[b,:,r,s]
 * + bias + pos_table[r*w+s, :].  latent (B,C,H,W) of io_dtype, w_nk bf16
 * (E, C*p*p), out (B*h*w, E) f32; scratch holds B*h*w*C*p*p bf16.
 * Replaces PatchEmbedding (modules.cpp:1093-1117). */
SD3_API int sd3_patch_embed(const void* latent, int io_dtype, const void* w_nk_bf16, const float* bias,
                    const float* pos_table, float* out, void* scratch_bf16, int B, int C, int H,
                    int W, int patch, int E, void* stream);

/* Patch embedding without any allocation and without a caller-provided
 * scratch buffer.  It has no counterpart in the reference (whose
 * PatchEmbedding, modules.cpp:1093-1117, allocates its temporaries with new[]).
 *
 * Who needs it: callers that cannot call cudaMalloc at the point where they
 * run the operator -- latency-critical serving loops (cudaMalloc and cudaFree
 * synchronise the whole device), hosts that fix the memory budget when the
 * library is loaded, and code that runs where the allocator must not be
 * entered at all.
 *
 * Same arguments and result as sd3_patch_embed minus `scratch`: the gathered
 * patches go to a fixed array of SD3_STATIC_PATCH_ELEMS bf16 elements (8 MiB)
 * that is part of the library image on every GPU that loads it.  Calls with
 * B * (H/patch) * (W/patch) * C * patch * patch above that limit fail with
 * SD3_ERR_UNSUPPORTED.  The array is shared by all calls on a device and keeps
 * the previous call's contents (none of which is read before being rewritten);
 * calls whose GPU work overlaps race on it and must be serialised by the
 * caller.  The first call on a device resolves the array's device address;
 * issue that first call before any stream capture.  No cudaMalloc, cudaFree
 * or allocating library routine is called.  A bounded device wait that runs
 * out during such a call is recorded in a word next to the array, which
 * sd3_device_status reads and clears along with the ordinary status word. */
#define SD3_STATIC_PATCH_ELEMS (4L * 1024 * 1024)
SD3_API int sd3_patch_embed_static(const void* latent, int io_dtype, const void* w_nk_bf16,
                                   const float* bias, const float* pos_table, float* out, int B,
                                   int C, int H, int W, int patch, int E, void* stream);

/* (R, C) row-major of in_dtype -> (C, R) row-major of out_dtype.  Turns a
 * boundary weight (in, out) into the packed (out, in) form. */
SD3_API int sd3_pack_weight(const void* w_in_out, int in_dtype, void* w_nk, int out_dtype, int in_features,
                    int out_features, void* stream);

/* element-wise dtype conversion of n elements */
SD3_API int sd3_cast(const void* in, int in_dtype, void* out, int out_dtype, long n, void* stream);

/* In-place RMSNorm over `nheads` consecutive groups of `head_dim` columns
 * starting at column col0 of every row.  Replaces rmsnorm_group
 * (modules.cpp:192-198) for head sizes the fused epilogue does not cover. */
SD3_API int sd3_rmsnorm_heads(void* x, int dtype, long ld, long rows, int col0, int nheads, int head_dim,
                      const float* w, float eps, void* stream);

/* ------------------------------------------------------------------------- */
/* Model-level entry points                                                   */
/* ------------------------------------------------------------------------- */

typedef struct sd3_model sd3_model;

typedef struct sd3_config {
  int num_layers;
  uint64_t dual_attention_mask; /* bit l set: layer l has the extra image-only attention */
  int pooled_dim;
  int captions_dim;
  int in_channels;
  int emb_dim;
  int attn_heads;
  int mlp_expand;
  int patch_size;
  int pos_embed_max_size;
  int base_height;
  int use_qk_norm;
  int last_discards_context; /* 1 for a full model; for a lone block: its discard_context flag */
  int precision;             /* SD3_PRECISION_* */
  int block_only;            /* 1: only transformer.* parameters are required */
} sd3_config;

/* Creates an empty model on the current device.  Host-side allocation only. */
SD3_API int sd3_model_create(const sd3_config* cfg, sd3_model** out);
SD3_API void sd3_model_destroy(sd3_model* m);

/* Registers one parameter under its reference name (the named_parameters()
 * key of module_tests/modules.py, e.g. "transformer.3.latent_to_qkv.weight").
 * 2-D weights arrive in the reference's boundary layout (in, out)
 * (module_tests/DiT.py:25-31); they are transposed / converted into the
 * packed arena here.  dev_ptr is borrowed only for the duration of the call.
 * Unknown names are rejected; missing names are reported by finalize.
 * Replaces the get_ptr lambda of DiT_forward (modules.cpp:1625-1631). */
SD3_API int sd3_model_set_param(sd3_model* m, const char* name, const void* dev_ptr, int dtype, int ndim,
                        const int64_t* shape, void* stream);

/* Checks that every parameter the configuration needs was provided.  Writes
 * the number of missing parameters to *missing (details via sd3_last_error).
 * Synchronises the device: it waits for the parameter copies, derives from the
 * q/k RMSNorm weights the bound on the attention scores of every block (which
 * selects the softmax mode of sd3_attention_bounded inside the forward) and,
 * in FP8 mode, quantises the block weights.  Call it again after a later
 * sd3_model_set_param. */
SD3_API int sd3_model_finalize(sd3_model* m, int* missing);

/* Allocates (or grows) the activation workspace for the given problem size.
 * The only place device memory for activations is allocated. */
SD3_API int sd3_model_reserve(sd3_model* m, int B, int Tc, int H, int W);

/* Full denoiser forward.  pooled (B, pooled_dim), captions (B, Tc,
 * captions_dim), latent (B, C, H, W), out (B, C, H, W) of io_dtype;
 * timesteps (B,) f32.  Replaces DiT_forward (modules.cpp:1605-1780); math of
 * MMDiT.forward (module_tests/modules.py:397-425). */
SD3_API int sd3_dit_forward(sd3_model* m, const void* pooled, const void* captions, const void* latent,
                    const float* timesteps, void* out, int io_dtype, int B, int Tc, int H, int W,
                    void* stream);

/* One MMDiT / MMDiT-X block in place on the fp32 streams c (B, Tc, E) and
 * x (B, Tx, E) with conditioning y (B, E) (all f32).  Replaces
 * DiT_block_forward_cuda / dit_block_cuda (cuda/dit.cu:768-1061) and
 * dit_block (modules.cpp:1340-1505). */
SD3_API int sd3_block_forward(sd3_model* m, int layer, const float* y, float* c, float* x, int B, int Tc,
                      int Tx, void* stream);

/* One sampling-loop update after a denoiser call on the stacked batch
 * [conditional; unconditional]: v = v_u + guidance (v_c - v_u),
 * x_state += dsigma * v (fp32 master copy, half_elems elements), and the new
 * latent is written to BOTH halves of x_stacked (2 * half_elems elements of
 * io_dtype) so it is the next step's model input.  v_stacked is the denoiser
 * output for x_stacked.  The reference has no sampler (README.md:1-7); this is
 * the caller next to DiT_forward. */
SD3_API int sd3_cfg_euler_step(float* x_state, void* x_stacked, const void* v_stacked, int io_dtype,
                               long half_elems, float guidance, float dsigma, void* stream);

/* Number of kernels this library launched since the last call with reset != 0
 * (process-wide counter, for benchmarks). */
SD3_API long sd3_launch_count(int reset);

#ifdef __cplusplus
}
#endif
#endif /* SD3_B200_H_ */

// extern "C" per-operator entry points of libsd3_b200.so (declared in
// include/sd3_b200.h).  Thin argument checks, then the launchers of kernels.h.
#include <mutex>

#include "../../include/sd3_b200.h"
#include "kernels.h"

namespace sd3 {

// One status word per device, allocated on first use and kept for the life of
// the process.  Kernels write a DEV_TIMEOUT_* code there when a wait runs out.
int* static_status_word_if_resolved();

int* device_status_word() {
  static int* words[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!words[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, sizeof(int)) != cudaSuccess) {
      cudaFree(p);
      return nullptr;
    }
    words[dev] = p;
  }
  return words[dev];
}

}  // namespace sd3

using namespace sd3;

namespace {
inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
inline bool dtype_ok(int d) { return d == SD3_DTYPE_F32 || d == SD3_DTYPE_BF16; }
}  // namespace

extern "C" {

int sd3_abi_version(void) { return 1; }

const char* sd3_last_error(void) { return get_last_error(); }

long sd3_launch_count(int reset) { return launch_count(reset); }

int sd3_device_status(int* status_out) {
  if (!status_out) return SD3_ERR_INVALID_ARG;
  int* w = device_status_word();
  if (!w) {
    set_last_error("device status word unavailable");
    return SD3_ERR_CUDA;
  }
  int rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  if (rc) return rc;
  rc = check_cuda(cudaMemcpy(status_out, w, sizeof(int), cudaMemcpyDeviceToHost), "status read");
  if (rc) return rc;
  if (*status_out != 0) {
    set_last_error("a kernel gave up a bounded wait (device status %d)", *status_out);
    return check_cuda(cudaMemset(w, 0, sizeof(int)), "status clear");
  }
  // the allocation-free entry point records into a word of its own
  if (int* ws = static_status_word_if_resolved()) {
    rc = check_cuda(cudaMemcpy(status_out, ws, sizeof(int), cudaMemcpyDeviceToHost), "status read");
    if (rc) return rc;
    if (*status_out != 0) {
      set_last_error("a kernel gave up a bounded wait (device status %d)", *status_out);
      return check_cuda(cudaMemset(ws, 0, sizeof(int)), "status clear");
    }
  }
  return SD3_OK;
}

int sd3_linear(const void* x, const void* w, const float* bias, void* out, int out_dtype, int M,
               int N, int K, int act, void* stream) {
  if (!dtype_ok(out_dtype) || (act != SD3_ACT_NONE && act != SD3_ACT_GELU_TANH)) {
    set_last_error("sd3_linear: bad out_dtype %d or act %d", out_dtype, act);
    return SD3_ERR_INVALID_ARG;
  }
  GemmEpilogue e;
  e.mode = act == SD3_ACT_GELU_TANH ? EPI_BIAS_GELU : EPI_BIAS;
  e.bias = bias;
  e.out = out;
  e.out_f32 = out_dtype == SD3_DTYPE_F32;
  e.ldo = N;
  return launch_gemm(x, K, w, K, OPERAND_BF16, M, N, K, e, device_status_word(), S(stream));
}

int sd3_linear_e4m3(const void* x, const void* w, const float* bias, void* out, int out_dtype, int M,
                    int N, int K, float scale, int act, void* stream) {
  if (!dtype_ok(out_dtype) || (act != SD3_ACT_NONE && act != SD3_ACT_GELU_TANH)) {
    set_last_error("sd3_linear_e4m3: bad out_dtype %d or act %d", out_dtype, act);
    return SD3_ERR_INVALID_ARG;
  }
  GemmEpilogue e;
  e.mode = act == SD3_ACT_GELU_TANH ? EPI_BIAS_GELU : EPI_BIAS;
  e.bias = bias;
  e.out = out;
  e.out_f32 = out_dtype == SD3_DTYPE_F32;
  e.ldo = N;
  e.alpha = scale;
  return launch_gemm(x, K, w, K, OPERAND_E4M3, M, N, K, e, device_status_word(), S(stream));
}

int sd3_quantize_e4m3(const void* in, int in_dtype, void* out, long n, float scale, void* stream) {
  if (!dtype_ok(in_dtype) || !(scale > 0.f)) {
    set_last_error("sd3_quantize_e4m3: bad dtype %d or scale %g", in_dtype, static_cast<double>(scale));
    return SD3_ERR_INVALID_ARG;
  }
  return launch_quantize_e4m3(in, in_dtype == SD3_DTYPE_F32, out, n, 1.0f / scale, S(stream));
}

int sd3_linear_f32(const float* x, const float* w, const float* bias, float* out, int M, int N,
                   int K, int act, void* stream) {
  if (act != SD3_ACT_NONE && act != SD3_ACT_GELU_TANH) {
    set_last_error("sd3_linear_f32: bad act %d", act);
    return SD3_ERR_INVALID_ARG;
  }
  GemmEpilogue e;
  e.mode = act == SD3_ACT_GELU_TANH ? EPI_BIAS_GELU : EPI_BIAS;
  e.bias = bias;
  e.out = out;
  e.out_f32 = 1;
  e.ldo = N;
  return launch_gemm_f32(x, K, w, K, M, N, K, e, S(stream));
}

int sd3_linear_gate_residual(const void* x, const void* w, const float* bias, const float* gate,
                             long gate_stride, int rows_per_sample, float* resid, int M, int N,
                             int K, void* stream) {
  if (rows_per_sample <= 0) {
    set_last_error("sd3_linear_gate_residual: rows_per_sample must be positive");
    return SD3_ERR_INVALID_ARG;
  }
  GemmEpilogue e;
  e.mode = EPI_GATE_RESID;
  e.bias = bias;
  e.out = resid;
  e.resid = resid;
  e.out_f32 = 1;
  e.ldo = N;
  e.gate = gate;
  e.gate_stride = gate_stride;
  e.rows_in = rows_per_sample;
  e.rows_out = rows_per_sample;
  e.row_off = 0;
  return launch_gemm(x, K, w, K, OPERAND_BF16, M, N, K, e, device_status_word(), S(stream));
}

int sd3_linear_pair(const void* x0, const void* w0, const float* bias0, void* out0, int M0, const void* x1,
                    const void* w1, const float* bias1, void* out1, int M1, int out_dtype, int N, int K, int act,
                    void* stream) {
  if (!dtype_ok(out_dtype) || (act != SD3_ACT_NONE && act != SD3_ACT_GELU_TANH) || M0 <= 0 || M1 <= 0) {
    set_last_error("sd3_linear_pair: bad out_dtype %d, act %d or row counts %d, %d", out_dtype, act, M0, M1);
    return SD3_ERR_INVALID_ARG;
  }
  GemmProblem p[2];
  const void* xs[2] = {x0, x1};
  const void* ws[2] = {w0, w1};
  const float* bs[2] = {bias0, bias1};
  void* outs[2] = {out0, out1};
  const int Ms[2] = {M0, M1};
  for (int i = 0; i < 2; ++i) {
    p[i].A = xs[i]; p[i].lda = K; p[i].W = ws[i]; p[i].ldw = K; p[i].M = Ms[i];
    p[i].epi.mode = act == SD3_ACT_GELU_TANH ? EPI_BIAS_GELU : EPI_BIAS;
    p[i].epi.bias = bs[i];
    p[i].epi.out = outs[i];
    p[i].epi.out_f32 = out_dtype == SD3_DTYPE_F32;
    p[i].epi.ldo = N;
  }
  return launch_gemm_grouped(p[0], p[1], OPERAND_BF16, N, K, device_status_word(), S(stream));
}

int sd3_linear_gate_residual_pair(const void* x0, const void* w0, const float* bias0, const float* gate0,
                                  int rows_per_sample0, float* resid0, int M0, const void* x1, const void* w1,
                                  const float* bias1, const float* gate1, int rows_per_sample1, float* resid1,
                                  int M1, long gate_stride, int N, int K, void* stream) {
  if (rows_per_sample0 <= 0 || rows_per_sample1 <= 0 || M0 <= 0 || M1 <= 0) {
    set_last_error("sd3_linear_gate_residual_pair: row counts must be positive");
    return SD3_ERR_INVALID_ARG;
  }
  GemmProblem p[2];
  const void* xs[2] = {x0, x1};
  const void* ws[2] = {w0, w1};
  const float* bs[2] = {bias0, bias1};
  const float* gs[2] = {gate0, gate1};
  float* rs[2] = {resid0, resid1};
  const int Ms[2] = {M0, M1};
  const int rps[2] = {rows_per_sample0, rows_per_sample1};
  for (int i = 0; i < 2; ++i) {
    p[i].A = xs[i]; p[i].lda = K; p[i].W = ws[i]; p[i].ldw = K; p[i].M = Ms[i];
    GemmEpilogue& e = p[i].epi;
    e.mode = EPI_GATE_RESID;
    e.bias = bs[i];
    e.out = rs[i];
    e.resid = rs[i];
    e.out_f32 = 1;
    e.ldo = N;
    e.gate = gs[i];
    e.gate_stride = gate_stride;
    e.rows_in = rps[i];
    e.rows_out = rps[i];
    e.row_off = 0;
  }
  return launch_gemm_grouped(p[0], p[1], OPERAND_BF16, N, K, device_status_word(), S(stream));
}

int sd3_qkv_project(const void* x, const void* w, const float* bias, const float* wq,
                    const float* wk, float eps, void* qkv_out, int B, int T_in, int T_total,
                    int row_offset, int E, void* stream) {
  if (B <= 0 || T_in <= 0 || row_offset < 0 || row_offset + T_in > T_total || E <= 0 || E % 64) {
    set_last_error("sd3_qkv_project: invalid shape (T_in %d off %d T_total %d E %d)", T_in,
                   row_offset, T_total, E);
    return SD3_ERR_INVALID_ARG;
  }
  GemmEpilogue e;
  e.mode = EPI_QKV_NORM;
  e.bias = bias;
  e.out = qkv_out;
  e.out_f32 = 0;
  e.ldo = 3L * E;
  e.rows_in = T_in;
  e.rows_out = T_total;
  e.row_off = row_offset;
  e.wq = wq;
  e.wk = wk;
  e.qk_cols = 2 * E;
  e.eps = eps;
  e.do_norm = (wq || wk) ? 1 : 0;
  return launch_gemm(x, E, w, E, OPERAND_BF16, B * T_in, 3 * E, E, e, device_status_word(),
                     S(stream));
}

int sd3_qkv_project_groups(const void* x, const void* w, const float* bias, const float* wq,
                           const float* wk, float eps, void* out, int rows, int E_out, int K, int head_groups,
                           void* stream) {
  if (rows <= 0 || E_out <= 0 || K <= 0 || head_groups < 1 || E_out % (64 * head_groups) || K % 8) {
    set_last_error("sd3_qkv_project_groups: invalid shape (rows %d E_out %d K %d groups %d)", rows, E_out, K,
                   head_groups);
    return SD3_ERR_INVALID_ARG;
  }
  GemmEpilogue e;
  e.mode = EPI_QKV_NORM;
  e.bias = bias;
  e.out = out;
  e.out_f32 = 0;
  e.ldo = 3L * E_out;
  e.rows_in = rows;
  e.rows_out = rows;
  e.row_off = 0;
  e.wq = wq;
  e.wk = wk;
  e.qk_cols = 2 * E_out;
  e.eps = eps;
  e.do_norm = (wq || wk) ? 1 : 0;
  e.hg_groups = head_groups;
  e.hg_rows = rows;
  return launch_gemm(x, K, w, K, OPERAND_BF16, rows, 3 * E_out, K, e, device_status_word(), S(stream));
}

int sd3_attention(const void* qkv, int B, int T, int num_heads, int Tc, void* out_c, void* out_x,
                  float scale, void* stream) {
  return launch_attention_bf16(static_cast<const bf16*>(qkv), B, T, num_heads, Tc,
                               static_cast<bf16*>(out_c), static_cast<bf16*>(out_x), scale,
                               device_status_word(), S(stream));
}

long sd3_attention_scratch_bytes(int B, int T, int num_heads) {
  return static_cast<long>(attention_scratch_bytes(B, T, num_heads));
}

int sd3_attention_ws(const void* qkv, int B, int T, int num_heads, int Tc, void* out_c, void* out_x, float scale,
                     void* scratch, long scratch_bytes, void* stream) {
  return launch_attention_bf16(static_cast<const bf16*>(qkv), B, T, num_heads, Tc, static_cast<bf16*>(out_c),
                               static_cast<bf16*>(out_x), scale, device_status_word(), S(stream), 0, scratch,
                               scratch_bytes > 0 ? static_cast<size_t>(scratch_bytes) : 0);
}

int sd3_attention_bounded(const void* qkv, int B, int T, int num_heads, int Tc, void* out_c, void* out_x,
                          float scale, float score_bound, void* scratch, long scratch_bytes, void* stream) {
  return launch_attention_bf16(static_cast<const bf16*>(qkv), B, T, num_heads, Tc, static_cast<bf16*>(out_c),
                               static_cast<bf16*>(out_x), scale, device_status_word(), S(stream), 0, scratch,
                               scratch_bytes > 0 ? static_cast<size_t>(scratch_bytes) : 0, score_bound);
}

int sd3_attention_generic(const void* q, const void* k, const void* v, long ld, int in_dtype,
                          int B, int T, int num_heads, int head_dim, void* out, long ldo,
                          int out_dtype, float scale, void* stream) {
  if (!dtype_ok(in_dtype) || !dtype_ok(out_dtype)) {
    set_last_error("sd3_attention_generic: bad dtype");
    return SD3_ERR_INVALID_ARG;
  }
  return launch_attention_simt(q, k, v, ld, in_dtype == SD3_DTYPE_F32, B, T, num_heads, head_dim,
                               0, nullptr, out, ldo, out_dtype == SD3_DTYPE_F32, scale, S(stream));
}

int sd3_cross_attention(const void* q, const void* k, const void* v, long ldq, long ldkv, int in_dtype, int B,
                        int Tq, int Tk, int num_heads, int head_dim, void* out, long ldo, int out_dtype, float scale,
                        void* stream) {
  if (!dtype_ok(in_dtype) || !dtype_ok(out_dtype) || Tk <= 0) {
    set_last_error("sd3_cross_attention: bad dtype or key count");
    return SD3_ERR_INVALID_ARG;
  }
  return launch_attention_simt(q, k, v, ldq, in_dtype == SD3_DTYPE_F32, B, Tq, num_heads, head_dim, 0, nullptr, out,
                               ldo, out_dtype == SD3_DTYPE_F32, scale, S(stream), Tk, ldkv);
}

int sd3_conv2d(const void* x, int io_dtype, const float* w_f32, const float* bias, void* out, int B, int C, int H,
               int W, int O, int kh, int kw, int stride, int padding, void* stream) {
  if (!dtype_ok(io_dtype)) {
    set_last_error("sd3_conv2d: bad io_dtype %d", io_dtype);
    return SD3_ERR_INVALID_ARG;
  }
  return launch_conv2d_direct(x, io_dtype == SD3_DTYPE_F32, w_f32, bias, out, B, C, H, W, O, kh, kw, stride, padding,
                              S(stream));
}

int sd3_layernorm_modulate(const float* x, int B, int T, int E, float eps, const float* shift1,
                           const float* scale1, void* out1, const float* shift2,
                           const float* scale2, void* out2, long mod_stride, int out_dtype,
                           void* stream) {
  if (!dtype_ok(out_dtype)) {
    set_last_error("sd3_layernorm_modulate: bad out_dtype %d", out_dtype);
    return SD3_ERR_INVALID_ARG;
  }
  return launch_ln_modulate(x, B, T, E, eps, shift1, scale1, out1, shift2, scale2, out2,
                            mod_stride, out_dtype == SD3_DTYPE_F32, S(stream));
}

int sd3_skinny_linear(const float* in, long ld_in, const void* w, int w_dtype, const float* bias,
                      const float* add, long ld_add, float* out, long ld_out, int B, int N, int K,
                      int act, void* stream) {
  if (!dtype_ok(w_dtype) || (act != 0 && act != 1)) {
    set_last_error("sd3_skinny_linear: bad w_dtype %d or act %d", w_dtype, act);
    return SD3_ERR_INVALID_ARG;
  }
  return launch_skinny_linear(in, ld_in, w, w_dtype == SD3_DTYPE_F32, bias, add, ld_add, out,
                              ld_out, B, N, K, act, S(stream));
}

int sd3_sinusoidal_embedding(const float* t, float* out, int B, int dim, void* stream) {
  return launch_sinusoidal(t, out, B, dim, S(stream));
}

int sd3_pos_embed_table(float* table, int h, int w, int E, int pos_max, int base_size,
                        void* stream) {
  return launch_pos_table(table, h, w, E, pos_max, base_size, S(stream));
}

int sd3_patch_embed(const void* latent, int io_dtype, const void* w, const float* bias,
                    const float* pos_table, float* out, void* scratch, int B, int C, int H, int W,
                    int patch, int E, void* stream) {
  if (!dtype_ok(io_dtype) || !scratch || !pos_table || patch <= 0 || H % patch || W % patch) {
    set_last_error("sd3_patch_embed: invalid argument");
    return SD3_ERR_INVALID_ARG;
  }
  const int hp = H / patch, wp = W / patch, Kp = C * patch * patch;
  int rc = launch_patchify(latent, io_dtype == SD3_DTYPE_F32, scratch, 0, B, C, H, W, patch,
                           S(stream));
  if (rc) return rc;
  GemmEpilogue e;
  e.mode = EPI_ADD_TABLE;
  e.bias = bias;
  e.out = out;
  e.out_f32 = 1;
  e.ldo = E;
  e.rows_in = hp * wp;
  e.rows_out = hp * wp;
  e.table = pos_table;
  return launch_gemm(scratch, Kp, w, Kp, OPERAND_BF16, B * hp * wp, E, Kp, e,
                     device_status_word(), S(stream));
}

int sd3_pack_weight(const void* w_in_out, int in_dtype, void* w_nk, int out_dtype, int in_features,
                    int out_features, void* stream) {
  if (!dtype_ok(in_dtype) || !dtype_ok(out_dtype)) {
    set_last_error("sd3_pack_weight: bad dtype");
    return SD3_ERR_INVALID_ARG;
  }
  return launch_transpose(w_in_out, in_dtype == SD3_DTYPE_F32, w_nk, out_dtype == SD3_DTYPE_F32,
                          in_features, out_features, S(stream));
}

int sd3_cast(const void* in, int in_dtype, void* out, int out_dtype, long n, void* stream) {
  if (!in || !out || n < 0 || !dtype_ok(in_dtype) || !dtype_ok(out_dtype)) {
    set_last_error("sd3_cast: invalid argument");
    return SD3_ERR_INVALID_ARG;
  }
  if (in_dtype == out_dtype)
    return check_cuda(cudaMemcpyAsync(out, in, n * (in_dtype == SD3_DTYPE_F32 ? 4 : 2),
                                      cudaMemcpyDeviceToDevice, S(stream)),
                      "sd3_cast copy");
  if (in_dtype == SD3_DTYPE_F32)
    return launch_cast_f32_to_bf16(static_cast<const float*>(in), static_cast<bf16*>(out), n,
                                   S(stream));
  return launch_cast_bf16_to_f32(static_cast<const bf16*>(in), static_cast<float*>(out), n,
                                 S(stream));
}

int sd3_rmsnorm_heads(void* x, int dtype, long ld, long rows, int col0, int nheads, int head_dim,
                      const float* w, float eps, void* stream) {
  if (!dtype_ok(dtype)) {
    set_last_error("sd3_rmsnorm_heads: bad dtype");
    return SD3_ERR_INVALID_ARG;
  }
  return launch_rmsnorm_heads(x, dtype == SD3_DTYPE_F32, ld, rows, col0, nheads, head_dim, w, eps,
                              S(stream));
}

}  // extern "C"

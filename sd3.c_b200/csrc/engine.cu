// Model-level part of the C ABI: parameter packing, the activation workspace
// and the launch sequences of one MMDiT(-X) block and of the full denoiser.
//
// Math follows MM_DiT_Block.forward / MMDiT.forward of the reference's PyTorch
// modules (module_tests/modules.py:255-355, 397-425); the host-side structure
// replaces dit_block_cuda / DiT_block_forward_cuda (cuda/dit.cu:768-1061, 17
// cudaMalloc + 17 cudaFree and fresh cuBLAS handles per call) and DiT_forward
// (modules.cpp:1605-1780): weights are packed once, activations live in one
// arena that is only (re)allocated by sd3_model_reserve, every launch goes to
// the caller's stream, nothing synchronises.
//
// Per block the launch sequence is
//   LN+modulate(c) | LN+modulate(x) (both modulations of a dual block at once)
//   QKV GEMM(c), QKV GEMM(x)  -> packed (B, Tc+Tx, 3E), RMSNorm fused, context rows first
//   joint attention           -> o_c, o_x
//   out-proj GEMM(c), (x)     -> gate * (.) + residual fused, fp32 streams in place
//   [dual] QKV GEMM(x2), attention over image tokens, out-proj GEMM with gate2
//   LN+modulate(x), MLP1 GEMM (+GELU-tanh), MLP2 GEMM (+gate, +residual); same for c
#include <math.h>
#include <algorithm>
#include <cmath>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/sd3_b200.h"
#include "kernels.h"

namespace sd3 {

int* device_status_word();

namespace {

struct Linear {
  void* w = nullptr;   // packed (N, K), bf16 or f32 depending on the model precision
  float* b = nullptr;  // (N,) f32
  int N = 0, K = 0;
  // FP8 mode: the same matrix as e4m3 = round(w / wscale), wscale = max|w| / 448
  void* w8 = nullptr;
  float wscale = 1.0f;
  bool w8_stale = false;  // w was rewritten after w8 was formed: requantise at the next finalize
};

struct LayerW {
  Linear c_qkv, c_out, c_mlp1, c_mlp2;
  Linear x_qkv, x_out, x_mlp1, x_mlp2;
  Linear d_qkv, d_out;
  float *c_wq = nullptr, *c_wk = nullptr, *x_wq = nullptr, *x_wk = nullptr, *d_wq = nullptr,
        *d_wk = nullptr;
  // upper bounds on |q . k| of the joint and the image-only attention, from the RMSNorm weights of
  // q and k (0: none, the attention keeps its running maximum); set by sd3_model_finalize
  float joint_bound = 0.f, dual_bound = 0.f;
  // Copies of the query RMSNorm weights multiplied by softmax_scale * log2(e) (set with the
  // bounds): the QKV epilogue then leaves q pre-scaled, a score is its own exp2 argument and the
  // attention kernel saves the multiply; joint_bound / dual_bound are in those units then.
  float *c_wq_s = nullptr, *x_wq_s = nullptr, *d_wq_s = nullptr;
  long c_mod_off = 0, x_mod_off = 0;  // column offsets into the concatenated AdaLN output
  int c_chunks = 0, x_chunks = 0;
  bool dual = false, last = false;
};

struct Workspace {
  void* base = nullptr;
  size_t bytes = 0;
  int B = 0, Tc = 0, Tx = 0;
  // f32
  float *temb, *th, *tout, *ph, *y, *mod, *c, *x, *pooled_f32;
  // activation-dtype buffers (bf16, or f32 in the exact mode)
  void *cap_in, *patches, *h_c, *h_x, *h_x2, *qkv, *qkv2, *o_c, *o_x, *o_x2, *hid_x, *hid_c;
  bf16* y_bf = nullptr;  // conditioning vector as a GEMM operand
  void* a8 = nullptr;    // FP8 mode: e4m3 copy of the current GEMM's left operand
  void* attn_scratch = nullptr;  // partial results of key-split attention launches (small batches, long sequences)
  size_t attn_scratch_bytes = 0;
  // position table cache
  float* pos = nullptr;
  int pos_h = 0, pos_w = 0;
};

}  // namespace

}  // namespace sd3

using namespace sd3;

struct sd3_model {
  sd3_config cfg;
  int E = 0, NH = 0, D = 0, F = 0, Kp = 0, Nout = 0;
  bool f32 = false;
  bool fp8 = false;  // bf16 everywhere except the block GEMMs, which take e4m3 operands
  std::vector<LayerW> layers;
  Linear t1, t2, p1, p2, cap, patch, fin;
  void* ada_w = nullptr;  // (ada_total, E)
  float* ada_b = nullptr;  // (ada_total,)
  long ada_total = 0, fin_mod_off = 0;
  std::map<std::string, bool> seen;
  std::vector<std::string> required;
  std::vector<void*> owned;
  Workspace ws;
  float* pos_store = nullptr;
  size_t pos_store_elems = 0;
  int* status = nullptr;
  float* amax_scratch = nullptr;  // one float for the weight quantiser
  bool finalized = false;

  size_t wbytes() const { return f32 ? 4 : 2; }
};

namespace {

inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }

int dev_alloc(sd3_model* m, void** p, size_t bytes) {
  cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
  if (e != cudaSuccess) {
    set_last_error("cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    return ST_CUDA_ERROR;
  }
  m->owned.push_back(*p);
  return ST_OK;
}

// weight given as (in, out) of dtype -> packed (out, in) at dst (model precision)
int pack_linear_weight(sd3_model* m, const void* src, int dtype, int in_f, int out_f, void* dst,
                       cudaStream_t st) {
  return launch_transpose(src, dtype == SD3_DTYPE_F32, dst, m->f32, in_f, out_f, st);
}

int copy_to_f32(const void* src, int dtype, float* dst, long n, cudaStream_t st) {
  if (dtype == SD3_DTYPE_F32)
    return check_cuda(cudaMemcpyAsync(dst, src, n * 4, cudaMemcpyDeviceToDevice, st), "param copy");
  return launch_cast_bf16_to_f32(static_cast<const bf16*>(src), dst, n, st);
}

struct Slot {
  Linear* lin = nullptr;   // weight/bias of a linear
  float** vec = nullptr;   // a plain f32 vector (RMSNorm weight)
  long ada_off = -1;       // >= 0: rows [ada_off, ada_off + n) of the AdaLN matrix
  int ada_rows = 0;
  int N = 0, K = 0;        // expected out/in features
  bool conv = false;       // 4-D conv weight, already (out, in*p*p)
};

bool find_slot(sd3_model* m, const std::string& name, Slot* s, bool* is_bias) {
  const sd3_config& c = m->cfg;
  const int E = m->E;
  std::string base = name;
  *is_bias = false;
  auto ends_with = [](const std::string& a, const char* suf) {
    const size_t n = strlen(suf);
    return a.size() >= n && a.compare(a.size() - n, n, suf) == 0;
  };
  if (ends_with(name, ".weight")) base = name.substr(0, name.size() - 7);
  else if (ends_with(name, ".bias")) { base = name.substr(0, name.size() - 5); *is_bias = true; }
  else return false;

  auto lin = [&](Linear* l, int N, int K) { s->lin = l; s->N = N; s->K = K; return true; };
  if (base == "timestep_mlp.0") return lin(&m->t1, E, 256);
  if (base == "timestep_mlp.2") return lin(&m->t2, E, E);
  if (base == "pooled_mlp.0") return lin(&m->p1, E, c.pooled_dim);
  if (base == "pooled_mlp.2") return lin(&m->p2, E, E);
  if (base == "captions_linear") return lin(&m->cap, E, c.captions_dim);
  if (base == "linear_out") return lin(&m->fin, m->Nout, E);
  if (base == "to_patch.conv") { s->conv = true; return lin(&m->patch, E, m->Kp); }
  if (base == "ada_ln_out.linear") {
    s->ada_off = m->fin_mod_off; s->ada_rows = 2 * E; s->N = 2 * E; s->K = E;
    return true;
  }
  const std::string pre = "transformer.";
  if (base.compare(0, pre.size(), pre) != 0) return false;
  const size_t dot = base.find('.', pre.size());
  if (dot == std::string::npos) return false;
  int l = -1;
  try { l = std::stoi(base.substr(pre.size(), dot - pre.size())); } catch (...) { return false; }
  if (l < 0 || l >= c.num_layers) return false;
  LayerW& L = m->layers[l];
  const std::string sub = base.substr(dot + 1);
  const int F = m->F, D = m->D;
  auto vec = [&](float** v) { s->vec = v; s->N = D; return !*is_bias; };
  if (sub == "context_ada_lnorm.linear") {
    s->ada_off = L.c_mod_off; s->ada_rows = L.c_chunks * E; s->N = s->ada_rows; s->K = E; return true;
  }
  if (sub == "latent_ada_lnorm.linear") {
    s->ada_off = L.x_mod_off; s->ada_rows = L.x_chunks * E; s->N = s->ada_rows; s->K = E; return true;
  }
  if (sub == "context_to_qkv") return lin(&L.c_qkv, 3 * E, E);
  if (sub == "latent_to_qkv") return lin(&L.x_qkv, 3 * E, E);
  if (sub == "latent_attn_Wout") return lin(&L.x_out, E, E);
  if (sub == "latent_mlp.lin1") return lin(&L.x_mlp1, F, E);
  if (sub == "latent_mlp.lin2") return lin(&L.x_mlp2, E, F);
  if (sub == "context_rmsnorm_key") return vec(&L.c_wk);
  if (sub == "context_rmsnorm_query") return vec(&L.c_wq);
  if (sub == "latent_rmsnorm_key") return vec(&L.x_wk);
  if (sub == "latent_rmsnorm_query") return vec(&L.x_wq);
  if (!L.last) {
    if (sub == "context_attn_Wout") return lin(&L.c_out, E, E);
    if (sub == "context_mlp.lin1") return lin(&L.c_mlp1, F, E);
    if (sub == "context_mlp.lin2") return lin(&L.c_mlp2, E, F);
  }
  if (L.dual) {
    if (sub == "latent_dual_to_qkv") return lin(&L.d_qkv, 3 * E, E);
    if (sub == "latent_dual_attn_Wout") return lin(&L.d_out, E, E);
    if (sub == "latent_dual_rmsnorm_key") return vec(&L.d_wk);
    if (sub == "latent_dual_rmsnorm_query") return vec(&L.d_wq);
  }
  return false;
}

void build_required(sd3_model* m) {
  const sd3_config& c = m->cfg;
  auto wb = [&](const std::string& b) {
    m->required.push_back(b + ".weight");
    m->required.push_back(b + ".bias");
  };
  if (!c.block_only) {
    wb("timestep_mlp.0"); wb("timestep_mlp.2"); wb("pooled_mlp.0"); wb("pooled_mlp.2");
    wb("captions_linear"); wb("to_patch.conv"); wb("ada_ln_out.linear"); wb("linear_out");
  }
  for (int l = 0; l < c.num_layers; ++l) {
    const LayerW& L = m->layers[l];
    const std::string p = "transformer." + std::to_string(l) + ".";
    wb(p + "context_ada_lnorm.linear"); wb(p + "context_to_qkv");
    wb(p + "latent_ada_lnorm.linear"); wb(p + "latent_to_qkv");
    wb(p + "latent_attn_Wout"); wb(p + "latent_mlp.lin1"); wb(p + "latent_mlp.lin2");
    if (!L.last) { wb(p + "context_attn_Wout"); wb(p + "context_mlp.lin1"); wb(p + "context_mlp.lin2"); }
    if (L.dual) { wb(p + "latent_dual_to_qkv"); wb(p + "latent_dual_attn_Wout"); }
    if (c.use_qk_norm) {
      m->required.push_back(p + "context_rmsnorm_key.weight");
      m->required.push_back(p + "context_rmsnorm_query.weight");
      m->required.push_back(p + "latent_rmsnorm_key.weight");
      m->required.push_back(p + "latent_rmsnorm_query.weight");
      if (L.dual) {
        m->required.push_back(p + "latent_dual_rmsnorm_key.weight");
        m->required.push_back(p + "latent_dual_rmsnorm_query.weight");
      }
    }
  }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int reserve_ws(sd3_model* m, int B, int Tc, int Tx) {
  Workspace& w = m->ws;
  if (w.base && B <= w.B && Tc <= w.Tc && Tx <= w.Tx) return ST_OK;
  if (w.base) {
    cudaError_t e = cudaFree(w.base);
    w.base = nullptr;
    if (e != cudaSuccess) return check_cuda(e, "cudaFree(workspace)");
  }
  const sd3_config& c = m->cfg;
  const size_t E = m->E, F = m->F, T = static_cast<size_t>(Tc) + Tx, ab = m->wbytes();
  const size_t nB = B, nTc = static_cast<size_t>(B) * Tc, nTx = static_cast<size_t>(B) * Tx;
  struct Item { void** p; size_t bytes; };
  std::vector<Item> items = {
      {(void**)&w.temb, nB * 256 * 4}, {(void**)&w.th, nB * E * 4}, {(void**)&w.tout, nB * E * 4},
      {(void**)&w.ph, nB * E * 4}, {(void**)&w.y, nB * E * 4}, {(void**)&w.y_bf, nB * E * 2},
      {(void**)&w.mod, nB * static_cast<size_t>(m->ada_total) * 4},
      {(void**)&w.c, nTc * E * 4}, {(void**)&w.x, nTx * E * 4},
      {(void**)&w.pooled_f32, nB * static_cast<size_t>(c.pooled_dim > 0 ? c.pooled_dim : 1) * 4},
      {&w.cap_in, nTc * static_cast<size_t>(c.captions_dim > 0 ? c.captions_dim : 1) * ab},
      {&w.patches, nTx * static_cast<size_t>(m->Kp > 0 ? m->Kp : 1) * ab},
      {&w.h_c, nTc * E * ab}, {&w.h_x, nTx * E * ab}, {&w.h_x2, nTx * E * ab},
      {&w.qkv, nB * T * 3 * E * ab}, {&w.qkv2, nTx * 3 * E * ab},
      {&w.o_c, nTc * E * ab}, {&w.o_x, nTx * E * ab}, {&w.o_x2, nTx * E * ab},
      {&w.hid_x, nTx * F * ab}, {&w.hid_c, nTc * F * ab},
      {&w.a8, m->fp8 ? (nTx > nTc ? nTx : nTc) * F : 16},
      {&w.attn_scratch, 16},
  };
  // key-split attention (head_dim 64 tensor-core path): the larger need of the joint and the image-only call
  w.attn_scratch_bytes = 0;
  if (!m->f32 && m->D == 64) {
    const size_t a = attention_scratch_bytes(B, static_cast<int>(T), m->NH);
    const size_t b2 = attention_scratch_bytes(B, Tx, m->NH);
    w.attn_scratch_bytes = a > b2 ? a : b2;
    if (w.attn_scratch_bytes > 0) items.back().bytes = w.attn_scratch_bytes;
  }
  size_t total = 0;
  for (auto& it : items) total += align_up(it.bytes, 256);
  void* base = nullptr;
  cudaError_t e = cudaMalloc(&base, total);
  if (e != cudaSuccess) {
    set_last_error("workspace cudaMalloc(%zu bytes) failed: %s", total, cudaGetErrorString(e));
    w.B = w.Tc = w.Tx = 0;
    return ST_CUDA_ERROR;
  }
  size_t off = 0;
  for (auto& it : items) {
    *it.p = static_cast<char*>(base) + off;
    off += align_up(it.bytes, 256);
  }
  w.base = base; w.bytes = total; w.B = B; w.Tc = Tc; w.Tx = Tx;
  return ST_OK;
}

// a_e4m3: A already holds e4m3 bytes (FP8 mode: written by ln_modulate, the GELU
// epilogue or a conversion pass)
int run_linear(sd3_model* m, const Linear& L, const void* A, int M, const GemmEpilogue& e,
               cudaStream_t st, bool a_e4m3 = false) {
  if (!L.w) {
    set_last_error("a required weight is missing (N %d K %d)", L.N, L.K);
    return ST_NOT_READY;
  }
  GemmEpilogue ee = e;
  if (!ee.bias) ee.bias = L.b;
  if (m->f32)
    return launch_gemm_f32(static_cast<const float*>(A), L.K, static_cast<const float*>(L.w), L.K,
                           M, L.N, L.K, ee, st);
  if (m->fp8 && L.w8) {
    // e4m3 x e4m3: the bf16 operand is converted as is (scale 1: LayerNorm
    // outputs, attention outputs and GELU outputs sit well inside e4m3's range and
    // the conversion saturates), the weight's scale is undone in the epilogue.
    const void* a8 = A;
    if (!a_e4m3) {
      int rc = launch_quantize_e4m3(A, 0, m->ws.a8, static_cast<long>(M) * L.K, 1.0f, st);
      if (rc) return rc;
      a8 = m->ws.a8;
    }
    ee.alpha = L.wscale;
    return launch_gemm(a8, L.K, L.w8, L.K, OPERAND_E4M3, M, L.N, L.K, ee, m->status, st);
  }
  if (a_e4m3) {
    set_last_error("an e4m3 operand reached a GEMM without e4m3 weights (N %d K %d)", L.N, L.K);
    return ST_UNSUPPORTED;
  }
  return launch_gemm(A, L.K, L.w, L.K, OPERAND_BF16, M, L.N, L.K, ee, m->status, st);
}

// Two linears of the same shape class (the image-stream GEMM and its context-stream twin) as
// one grouped launch where the tensor-core path takes both; otherwise one after the other.
int run_linear_pair(sd3_model* m, const Linear& La, const void* Aa, int Ma, const GemmEpilogue& ea, bool a8a,
                    const Linear& Lb, const void* Ab, int Mb, const GemmEpilogue& eb, bool a8b, cudaStream_t st) {
  const bool fp8a = m->fp8 && La.w8 && a8a, fp8b = m->fp8 && Lb.w8 && a8b;
  const bool plain_a = !(m->fp8 && La.w8) && !a8a, plain_b = !(m->fp8 && Lb.w8) && !a8b;
  const bool same_kind = (fp8a && fp8b) || (plain_a && plain_b);
  if (m->f32 || !La.w || !Lb.w || La.N != Lb.N || La.K != Lb.K || !same_kind) {
    int rc = run_linear(m, La, Aa, Ma, ea, st, a8a);
    if (rc) return rc;
    return run_linear(m, Lb, Ab, Mb, eb, st, a8b);
  }
  GemmProblem pa, pb;
  pa.A = Aa; pa.lda = La.K; pa.W = fp8a ? La.w8 : La.w; pa.ldw = La.K; pa.M = Ma; pa.epi = ea;
  pb.A = Ab; pb.lda = Lb.K; pb.W = fp8b ? Lb.w8 : Lb.w; pb.ldw = Lb.K; pb.M = Mb; pb.epi = eb;
  if (!pa.epi.bias) pa.epi.bias = La.b;
  if (!pb.epi.bias) pb.epi.bias = Lb.b;
  if (fp8a) { pa.epi.alpha = La.wscale; pb.epi.alpha = Lb.wscale; }
  return launch_gemm_grouped(pa, pb, fp8a ? OPERAND_E4M3 : OPERAND_BF16, La.N, La.K, m->status, st);
}

// QKV projection of `T_in` tokens per sample into rows [row_off, row_off+T_in)
// of each sample of the packed (B, T_total, 3E) buffer, q/k RMSNorm included.
int run_qkv(sd3_model* m, const Linear& L, const void* h, void* qkv, int B, int T_in, int T_total,
            int row_off, const float* wq, const float* wk, cudaStream_t st, bool h_e4m3 = false) {
  const int E = m->E;
  const bool norm = m->cfg.use_qk_norm && (wq || wk);
  const bool fused = !m->f32 && m->D == 64;
  GemmEpilogue e;
  e.mode = EPI_QKV_NORM;
  e.out = qkv;
  e.out_f32 = m->f32;
  e.ldo = 3L * E;
  e.rows_in = T_in; e.rows_out = T_total; e.row_off = row_off;
  e.wq = wq; e.wk = wk; e.qk_cols = 2 * E; e.eps = 1e-6f;
  e.do_norm = (fused && norm) ? 1 : 0;
  if (!fused) e.qk_cols = 0;
  int rc = run_linear(m, L, h, B * T_in, e, st, h_e4m3);
  if (rc || fused || !norm) return rc;
  const size_t ab = m->wbytes();
  for (int b = 0; b < B; ++b) {
    char* rows = static_cast<char*>(qkv) + (static_cast<size_t>(b) * T_total + row_off) * 3 * E * ab;
    rc = launch_rmsnorm_heads(rows, m->f32, 3L * E, T_in, 0, m->NH, m->D, wq, 1e-6f, st);
    if (rc) return rc;
    rc = launch_rmsnorm_heads(rows, m->f32, 3L * E, T_in, E, m->NH, m->D, wk, 1e-6f, st);
    if (rc) return rc;
  }
  return ST_OK;
}

// out_e4m3 (FP8 mode, head_dim 64 only): the outputs feed FP8 out-projections
int run_attention(sd3_model* m, const void* qkv, int B, int T, int Tc, void* o_c, void* o_x,
                  cudaStream_t st, bool out_e4m3 = false, float score_bound = 0.f, bool prescaled = false) {
  // prescaled: q already carries scale * log2(e) (only set up for the bf16 kernel)
  const float scale = prescaled ? 0.0f : 1.0f / sqrtf(static_cast<float>(m->D));
  if (!m->f32 && m->D == 64)
    return launch_attention_bf16(static_cast<const bf16*>(qkv), B, T, m->NH, Tc,
                                 static_cast<bf16*>(o_c), static_cast<bf16*>(o_x), scale, m->status,
                                 st, out_e4m3 ? 1 : 0, m->ws.attn_scratch_bytes ? m->ws.attn_scratch : nullptr,
                                 m->ws.attn_scratch_bytes, score_bound);
  if (out_e4m3) {
    set_last_error("e4m3 attention output needs head_dim 64");
    return ST_UNSUPPORTED;
  }
  const size_t ab = m->wbytes();
  const char* q = static_cast<const char*>(qkv);
  return launch_attention_simt(q, q + m->E * ab, q + 2 * m->E * ab, 3L * m->E, m->f32, B, T, m->NH,
                               m->D, Tc, o_c, o_x, m->E, m->f32, scale, st);
}

int run_gate_resid(sd3_model* m, const Linear& L, const void* A, int B, int Tseg, const float* gate,
                   long mod_stride, float* resid, cudaStream_t st, bool a_e4m3 = false) {
  GemmEpilogue e;
  e.mode = EPI_GATE_RESID;
  e.out = resid; e.resid = resid; e.out_f32 = 1; e.ldo = L.N;
  e.gate = gate; e.gate_stride = mod_stride;
  e.rows_in = Tseg; e.rows_out = Tseg; e.row_off = 0;
  return run_linear(m, L, A, B * Tseg, e, st, a_e4m3);
}

// hid_e4m3 (out): whether the hidden activations were written as e4m3
int run_mlp1(sd3_model* m, const Linear& L, const Linear& next, const void* A, int M, void* hid,
             cudaStream_t st, bool a_e4m3, bool* hid_e4m3) {
  GemmEpilogue e;
  e.mode = EPI_BIAS_GELU;
  e.out = hid; e.out_f32 = m->f32; e.ldo = L.N;
  *hid_e4m3 = m->fp8 && L.w8 && next.w8 && L.N % 64 == 0;
  e.out_e4m3 = *hid_e4m3 ? 1 : 0;
  return run_linear(m, L, A, M, e, st, a_e4m3);
}

GemmEpilogue qkv_epilogue(sd3_model* m, void* qkv, int T_in, int T_total, int row_off, const float* wq,
                          const float* wk) {
  GemmEpilogue e;
  e.mode = EPI_QKV_NORM;
  e.out = qkv;
  e.out_f32 = 0;
  e.ldo = 3L * m->E;
  e.rows_in = T_in; e.rows_out = T_total; e.row_off = row_off;
  e.wq = wq; e.wk = wk; e.qk_cols = 2 * m->E; e.eps = 1e-6f;
  e.do_norm = (m->cfg.use_qk_norm && (wq || wk)) ? 1 : 0;
  return e;
}

GemmEpilogue gate_epilogue(const Linear& L, int Tseg, const float* gate, long mod_stride, float* resid) {
  GemmEpilogue e;
  e.mode = EPI_GATE_RESID;
  e.out = resid; e.resid = resid; e.out_f32 = 1; e.ldo = L.N;
  e.gate = gate; e.gate_stride = mod_stride;
  e.rows_in = Tseg; e.rows_out = Tseg; e.row_off = 0;
  return e;
}

int block_body(sd3_model* m, int l, float* c, float* x, int B, int Tc, int Tx, const float* mod,
               long ms, cudaStream_t st) {
  const LayerW& L = m->layers[l];
  Workspace& w = m->ws;
  const int E = m->E, T = Tc + Tx;
  const float* cm = mod + L.c_mod_off;
  const float* xm = mod + L.x_mod_off;
  const float *c_shift_a, *c_scale_a, *c_gate_a = nullptr, *c_shift_m = nullptr, *c_scale_m = nullptr,
              *c_gate_m = nullptr;
  if (!L.last) {
    c_shift_a = cm; c_scale_a = cm + E; c_gate_a = cm + 2 * E;
    c_shift_m = cm + 3 * E; c_scale_m = cm + 4 * E; c_gate_m = cm + 5 * E;
  } else {
    c_scale_a = cm; c_shift_a = cm + E;  // the last block's context AdaLN is (scale, shift)
  }
  const float *x_shift_a = xm, *x_scale_a = xm + E, *x_gate_a = xm + 2 * E, *x_shift_m = xm + 3 * E,
              *x_scale_m = xm + 4 * E, *x_gate_m = xm + 5 * E;
  const float *x_shift_2 = xm + 6 * E, *x_scale_2 = xm + 7 * E, *x_gate_2 = xm + 8 * E;
  int rc;
#define SD3_TRY(expr) do { rc = (expr); if (rc) return rc; } while (0)
  // FP8 mode: LayerNorm writes the e4m3 operand of the following GEMM directly when
  // that GEMM (and, for the dual output, its twin) has e4m3 weights.
  const bool c8a = m->fp8 && L.c_qkv.w8, x8a = m->fp8 && L.x_qkv.w8 && (!L.dual || L.d_qkv.w8);
  const bool c8m = m->fp8 && L.c_mlp1.w8, x8m = m->fp8 && L.x_mlp1.w8;
  auto ln_out = [&](bool e4m3) { return m->f32 ? 1 : (e4m3 ? 2 : 0); };
  // pre-attention LayerNorm + modulate
  SD3_TRY(launch_ln_modulate(c, B, Tc, E, 1e-6f, c_shift_a, c_scale_a, w.h_c, nullptr, nullptr,
                             nullptr, ms, ln_out(c8a), st));
  if (L.dual)
    SD3_TRY(launch_ln_modulate(x, B, Tx, E, 1e-6f, x_shift_a, x_scale_a, w.h_x, x_shift_2, x_scale_2,
                               w.h_x2, ms, ln_out(x8a), st));
  else
    SD3_TRY(launch_ln_modulate(x, B, Tx, E, 1e-6f, x_shift_a, x_scale_a, w.h_x, nullptr, nullptr,
                               nullptr, ms, ln_out(x8a), st));
  // QKV (context rows first, then image rows) and joint attention
  // the tensor-core path (bf16 / FP8 modes, head_dim 64): image and context GEMMs of a kind share a launch
  const bool grouped = !m->f32 && m->D == 64;
  // q pre-scaled by softmax_scale * log2(e) through its norm weight (both streams or neither)
  const bool pre_j = L.c_wq_s != nullptr && L.x_wq_s != nullptr;
  const float* c_wq = pre_j ? L.c_wq_s : L.c_wq;
  const float* x_wq = pre_j ? L.x_wq_s : L.x_wq;
  if (grouped) {
    SD3_TRY(run_linear_pair(m, L.x_qkv, w.h_x, B * Tx, qkv_epilogue(m, w.qkv, Tx, T, Tc, x_wq, L.x_wk), x8a,
                            L.c_qkv, w.h_c, B * Tc, qkv_epilogue(m, w.qkv, Tc, T, 0, c_wq, L.c_wk), c8a, st));
  } else {
    SD3_TRY(run_qkv(m, L.c_qkv, w.h_c, w.qkv, B, Tc, T, 0, c_wq, L.c_wk, st, c8a));
    SD3_TRY(run_qkv(m, L.x_qkv, w.h_x, w.qkv, B, Tx, T, Tc, x_wq, L.x_wk, st, x8a));
  }
  // FP8 mode: both out-projections of the joint attention must take e4m3 for the
  // kernel to write it (one flag for both outputs)
  const bool o8 = m->fp8 && m->D == 64 && L.x_out.w8 && (L.last || L.c_out.w8);
  SD3_TRY(run_attention(m, w.qkv, B, T, Tc, L.last ? nullptr : w.o_c, w.o_x, st, o8, L.joint_bound, pre_j));
  if (grouped && !L.last) {
    SD3_TRY(run_linear_pair(m, L.x_out, w.o_x, B * Tx, gate_epilogue(L.x_out, Tx, x_gate_a, ms, x), o8,
                            L.c_out, w.o_c, B * Tc, gate_epilogue(L.c_out, Tc, c_gate_a, ms, c), o8, st));
  } else {
    if (!L.last) SD3_TRY(run_gate_resid(m, L.c_out, w.o_c, B, Tc, c_gate_a, ms, c, st, o8));
    SD3_TRY(run_gate_resid(m, L.x_out, w.o_x, B, Tx, x_gate_a, ms, x, st, o8));
  }
  if (L.dual) {
    const bool pre_d = L.d_wq_s != nullptr;
    SD3_TRY(run_qkv(m, L.d_qkv, w.h_x2, w.qkv2, B, Tx, Tx, 0, pre_d ? L.d_wq_s : L.d_wq, L.d_wk, st, x8a));
    const bool o8d = m->fp8 && m->D == 64 && L.d_out.w8;
    SD3_TRY(run_attention(m, w.qkv2, B, Tx, 0, nullptr, w.o_x2, st, o8d, L.dual_bound, pre_d));
    SD3_TRY(run_gate_resid(m, L.d_out, w.o_x2, B, Tx, x_gate_2, ms, x, st, o8d));
  }
  // MLPs of both streams: LayerNorm + modulate each, then the two first linears (GELU-tanh) and
  // the two second linears (gate + residual), each pair as one grouped launch
  SD3_TRY(launch_ln_modulate(x, B, Tx, E, 1e-6f, x_shift_m, x_scale_m, w.h_x, nullptr, nullptr,
                             nullptr, ms, ln_out(x8m), st));
  if (!L.last)
    SD3_TRY(launch_ln_modulate(c, B, Tc, E, 1e-6f, c_shift_m, c_scale_m, w.h_c, nullptr, nullptr,
                               nullptr, ms, ln_out(c8m), st));
  if (grouped && !L.last) {
    const bool hx8 = m->fp8 && L.x_mlp1.w8 && L.x_mlp2.w8 && L.x_mlp1.N % 64 == 0;
    const bool hc8 = m->fp8 && L.c_mlp1.w8 && L.c_mlp2.w8 && L.c_mlp1.N % 64 == 0;
    GemmEpilogue ex, ec;
    ex.mode = EPI_BIAS_GELU; ex.out = w.hid_x; ex.out_f32 = 0; ex.ldo = L.x_mlp1.N; ex.out_e4m3 = hx8 ? 1 : 0;
    ec.mode = EPI_BIAS_GELU; ec.out = w.hid_c; ec.out_f32 = 0; ec.ldo = L.c_mlp1.N; ec.out_e4m3 = hc8 ? 1 : 0;
    SD3_TRY(run_linear_pair(m, L.x_mlp1, w.h_x, B * Tx, ex, x8m, L.c_mlp1, w.h_c, B * Tc, ec, c8m, st));
    SD3_TRY(run_linear_pair(m, L.x_mlp2, w.hid_x, B * Tx, gate_epilogue(L.x_mlp2, Tx, x_gate_m, ms, x), hx8,
                            L.c_mlp2, w.hid_c, B * Tc, gate_epilogue(L.c_mlp2, Tc, c_gate_m, ms, c), hc8, st));
  } else {
    bool hid8 = false;
    SD3_TRY(run_mlp1(m, L.x_mlp1, L.x_mlp2, w.h_x, B * Tx, w.hid_x, st, x8m, &hid8));
    SD3_TRY(run_gate_resid(m, L.x_mlp2, w.hid_x, B, Tx, x_gate_m, ms, x, st, hid8));
    if (!L.last) {
      SD3_TRY(run_mlp1(m, L.c_mlp1, L.c_mlp2, w.h_c, B * Tc, w.hid_c, st, c8m, &hid8));
      SD3_TRY(run_gate_resid(m, L.c_mlp2, w.hid_c, B, Tc, c_gate_m, ms, c, st, hid8));
    }
  }
#undef SD3_TRY
  return ST_OK;
}

// FP8 mode: every block GEMM weight gets an e4m3 twin with one scale per matrix.
int quantize_block_weights(sd3_model* m) {
  int rc = check_cuda(cudaDeviceSynchronize(), "parameter copies");  // whatever stream packed them
  if (rc) return rc;
  if (!m->amax_scratch) {
    rc = dev_alloc(m, reinterpret_cast<void**>(&m->amax_scratch), 4);
    if (rc) return rc;
  }
  float* d_amax = m->amax_scratch;
  for (LayerW& Lw : m->layers) {
    Linear* all[] = {&Lw.c_qkv, &Lw.c_out, &Lw.c_mlp1, &Lw.c_mlp2, &Lw.x_qkv,
                     &Lw.x_out, &Lw.x_mlp1, &Lw.x_mlp2, &Lw.d_qkv, &Lw.d_out};
    for (Linear* L : all) {
      if (!L->w || (L->w8 && !L->w8_stale)) continue;
      const long n = static_cast<long>(L->N) * L->K;
      if (n % 4 || L->K % 16) continue;  // stays bf16
      rc = launch_absmax(L->w, 0, n, d_amax, nullptr);
      if (rc) return rc;
      float amax = 0.f;
      rc = check_cuda(cudaMemcpy(&amax, d_amax, 4, cudaMemcpyDeviceToHost), "read absmax");
      if (rc) return rc;
      if (!(amax > 0.f)) amax = 1.0f;
      L->wscale = amax / 448.0f;
      if (!L->w8) {  // a rewritten weight keeps its e4m3 buffer (same shape)
        rc = dev_alloc(m, &L->w8, static_cast<size_t>(n));
        if (rc) return rc;
      }
      rc = launch_quantize_e4m3(L->w, 0, L->w8, n, 1.0f / L->wscale, nullptr);
      if (rc) return rc;
      L->w8_stale = false;
    }
  }
  return check_cuda(cudaDeviceSynchronize(), "quantize weights");
}

// After the per-head RMSNorm (module_tests/modules.py:286-297: x / sqrt(mean(x^2) + eps) * w) a
// head vector is x_hat * w with |x_hat|^2 <= D, whatever the input; so |q . k| = |sum_d x_d y_d wq_d wk_d|
// <= D max_d |wq_d wk_d| for every query and key of an attention (context and image streams share
// the joint attention: element-wise maxima of their weights).  1 % on top covers the bf16 rounding
// of q and k.
// Where the bound is small enough for the attention kernel's bounded softmax, the query norm
// weights also get a copy multiplied by softmax_scale * log2(e): q leaves the QKV epilogue
// pre-scaled (one rounding to bf16, as before) and the bound is stored in those units.
int compute_score_bounds(sd3_model* m) {
  for (LayerW& L : m->layers) L.joint_bound = L.dual_bound = 0.f;
  if (!m->cfg.use_qk_norm || m->f32 || m->D != 64) return ST_OK;
  int rc = check_cuda(cudaDeviceSynchronize(), "parameter copies");
  if (rc) return rc;
  std::vector<float> h(m->D);
  bool ok = true;
  // |w| of a norm weight, element-wise maximum over the streams that share an attention
  auto absmax_into = [&](const float* w, std::vector<float>& acc) {
    if (!w || cudaMemcpy(h.data(), w, sizeof(float) * m->D, cudaMemcpyDeviceToHost) != cudaSuccess) {
      ok = false;
      return;
    }
    for (int d = 0; d < m->D; ++d) {
      if (!std::isfinite(h[d])) ok = false;
      acc[d] = std::max(acc[d], std::fabs(h[d]));
    }
  };
  // sum_d x_d y_d a_d with |x|^2 = |y|^2 = D is at most D max_d a_d: the bound needs the largest
  // PRODUCT |wq_d wk_d|, not the product of the largest weights
  auto pair_bound = [&](const std::vector<float>& q, const std::vector<float>& k) {
    float a = 0.f;
    for (int d = 0; d < m->D; ++d) a = std::max(a, q[d] * k[d]);
    return a;
  };
  // the bounded softmax takes exp2 arguments of at most 80: a looser bound would not be used,
  // and then q stays unscaled and the attention keeps its running maximum
  const float c = 1.4426950408889634f / sqrtf(static_cast<float>(m->D));
  auto scaled_copy = [&](const float* w, float** dst) -> int {
    if (cudaMemcpy(h.data(), w, sizeof(float) * m->D, cudaMemcpyDeviceToHost) != cudaSuccess)
      return check_cuda(cudaGetLastError(), "read norm weight");
    for (float& v : h) v *= c;
    if (!*dst) {
      int r = dev_alloc(m, reinterpret_cast<void**>(dst), sizeof(float) * m->D);
      if (r) return r;
    }
    return check_cuda(cudaMemcpy(*dst, h.data(), sizeof(float) * m->D, cudaMemcpyHostToDevice), "write norm weight");
  };
  for (LayerW& L : m->layers) {
    ok = true;
    std::vector<float> q(m->D, 0.f), k(m->D, 0.f);
    absmax_into(L.c_wq, q); absmax_into(L.x_wq, q);
    absmax_into(L.c_wk, k); absmax_into(L.x_wk, k);
    const float jb = 1.01f * m->D * pair_bound(q, k) * c;
    if (ok && jb > 0.f && jb <= 80.0f) {
      if ((rc = scaled_copy(L.c_wq, &L.c_wq_s)) || (rc = scaled_copy(L.x_wq, &L.x_wq_s))) return rc;
      L.joint_bound = jb;
    } else {
      L.c_wq_s = L.x_wq_s = nullptr;  // (a buffer from an earlier finalize stays owned by the model)
    }
    if (L.dual) {
      ok = true;
      std::vector<float> q2(m->D, 0.f), k2(m->D, 0.f);
      absmax_into(L.d_wq, q2);
      absmax_into(L.d_wk, k2);
      const float db = 1.01f * m->D * pair_bound(q2, k2) * c;
      if (ok && db > 0.f && db <= 80.0f) {
        if ((rc = scaled_copy(L.d_wq, &L.d_wq_s))) return rc;
        L.dual_bound = db;
      } else {
        L.d_wq_s = nullptr;
      }
    }
  }
  return ST_OK;
}

}  // namespace

extern "C" {

int sd3_model_create(const sd3_config* cfg, sd3_model** out) {
  if (!cfg || !out) return SD3_ERR_INVALID_ARG;
  if (cfg->num_layers <= 0 || cfg->num_layers > 64 || cfg->emb_dim <= 0 || cfg->attn_heads <= 0 ||
      cfg->emb_dim % cfg->attn_heads || cfg->mlp_expand <= 0 || cfg->emb_dim % 8) {
    set_last_error("sd3_model_create: invalid configuration (layers %d emb %d heads %d)",
                   cfg->num_layers, cfg->emb_dim, cfg->attn_heads);
    return SD3_ERR_INVALID_ARG;
  }
  if (cfg->precision != SD3_PRECISION_BF16 && cfg->precision != SD3_PRECISION_F32 &&
      cfg->precision != SD3_PRECISION_FP8) {
    set_last_error("sd3_model_create: precision %d not available", cfg->precision);
    return SD3_ERR_UNSUPPORTED;
  }
  if (!cfg->block_only &&
      (cfg->patch_size <= 0 || cfg->in_channels <= 0 || cfg->pooled_dim <= 0 ||
       cfg->captions_dim <= 0 || cfg->pos_embed_max_size <= 0 || cfg->base_height <= 0 ||
       cfg->pooled_dim % 8 || cfg->captions_dim % 8 ||
       (cfg->in_channels * cfg->patch_size * cfg->patch_size) % 8)) {
    set_last_error("sd3_model_create: invalid embedding configuration");
    return SD3_ERR_INVALID_ARG;
  }
  sd3_model* m = new sd3_model();
  m->cfg = *cfg;
  m->E = cfg->emb_dim;
  m->NH = cfg->attn_heads;
  m->D = m->E / m->NH;
  m->F = m->E * cfg->mlp_expand;
  m->Kp = cfg->block_only ? 0 : cfg->in_channels * cfg->patch_size * cfg->patch_size;
  m->Nout = m->Kp;
  m->f32 = cfg->precision == SD3_PRECISION_F32;
  m->fp8 = cfg->precision == SD3_PRECISION_FP8;
  if (m->D > 128) {
    set_last_error("sd3_model_create: head_dim %d > 128 unsupported", m->D);
    delete m;
    return SD3_ERR_UNSUPPORTED;
  }
  m->layers.resize(cfg->num_layers);
  long off = 0;
  for (int l = 0; l < cfg->num_layers; ++l) {
    LayerW& L = m->layers[l];
    L.last = cfg->last_discards_context && (l == cfg->num_layers - 1);
    L.dual = ((cfg->dual_attention_mask >> l) & 1ull) != 0;
    L.c_chunks = L.last ? 2 : 6;
    L.x_chunks = L.dual ? 9 : 6;
    L.c_mod_off = off; off += static_cast<long>(L.c_chunks) * m->E;
    L.x_mod_off = off; off += static_cast<long>(L.x_chunks) * m->E;
  }
  m->fin_mod_off = off;
  if (!cfg->block_only) off += 2L * m->E;
  m->ada_total = off;
  m->status = device_status_word();
  int rc = dev_alloc(m, &m->ada_w, static_cast<size_t>(off) * m->E * m->wbytes());
  if (!rc) rc = dev_alloc(m, reinterpret_cast<void**>(&m->ada_b), static_cast<size_t>(off) * 4);
  if (!rc) rc = check_cuda(cudaMemset(m->ada_b, 0, static_cast<size_t>(off) * 4), "memset");
  if (rc) {
    sd3_model_destroy(m);
    return rc;
  }
  build_required(m);
  *out = m;
  return SD3_OK;
}

void sd3_model_destroy(sd3_model* m) {
  if (!m) return;
  for (void* p : m->owned) cudaFree(p);
  if (m->ws.base) cudaFree(m->ws.base);
  if (m->pos_store) cudaFree(m->pos_store);
  delete m;
}

int sd3_model_set_param(sd3_model* m, const char* name, const void* dev_ptr, int dtype, int ndim,
                        const int64_t* shape, void* stream) {
  if (!m || !name || !dev_ptr || !shape || ndim < 1 || ndim > 4 ||
      (dtype != SD3_DTYPE_F32 && dtype != SD3_DTYPE_BF16)) {
    set_last_error("sd3_model_set_param: invalid argument");
    return SD3_ERR_INVALID_ARG;
  }
  Slot s;
  bool is_bias = false;
  if (!find_slot(m, name, &s, &is_bias)) {
    set_last_error("sd3_model_set_param: unknown or inapplicable parameter '%s'", name);
    return SD3_ERR_INVALID_ARG;
  }
  cudaStream_t st = S(stream);
  long numel = 1;
  for (int i = 0; i < ndim; ++i) numel *= shape[i];
  int rc = ST_OK;
  if (s.vec) {
    if (numel != s.N) {
      set_last_error("parameter '%s': expected %d elements, got %ld", name, s.N, numel);
      return SD3_ERR_INVALID_ARG;
    }
    if (!*s.vec) rc = dev_alloc(m, reinterpret_cast<void**>(s.vec), numel * 4);
    if (!rc) rc = copy_to_f32(dev_ptr, dtype, *s.vec, numel, st);
  } else if (is_bias) {
    if (numel != s.N) {
      set_last_error("parameter '%s': expected %d elements, got %ld", name, s.N, numel);
      return SD3_ERR_INVALID_ARG;
    }
    float* dst = nullptr;
    if (s.ada_off >= 0) {
      dst = m->ada_b + s.ada_off;
    } else {
      if (!s.lin->b) rc = dev_alloc(m, reinterpret_cast<void**>(&s.lin->b), numel * 4);
      dst = s.lin->b;
    }
    if (!rc) rc = copy_to_f32(dev_ptr, dtype, dst, numel, st);
  } else {
    // weight: (in, out) for linears, (out, in, p, p) for the patch conv
    bool ok;
    if (s.conv) ok = ndim == 4 && shape[0] == s.N && shape[1] * shape[2] * shape[3] == s.K;
    else ok = ndim == 2 && shape[0] == s.K && shape[1] == s.N;
    if (!ok) {
      set_last_error("parameter '%s': unexpected shape (expected in %d, out %d)", name, s.K, s.N);
      return SD3_ERR_INVALID_ARG;
    }
    void* dst = nullptr;
    if (s.ada_off >= 0) {
      dst = static_cast<char*>(m->ada_w) + static_cast<size_t>(s.ada_off) * m->E * m->wbytes();
    } else {
      if (!s.lin->w) rc = dev_alloc(m, &s.lin->w, static_cast<size_t>(numel) * m->wbytes());
      dst = s.lin->w;
      s.lin->N = s.N;
      s.lin->K = s.K;
      if (s.lin->w8) s.lin->w8_stale = true;
    }
    if (!rc) {
      if (s.conv) {
        if ((dtype == SD3_DTYPE_F32) == m->f32)
          rc = check_cuda(cudaMemcpyAsync(dst, dev_ptr, numel * m->wbytes(),
                                          cudaMemcpyDeviceToDevice, st), "conv weight copy");
        else if (dtype == SD3_DTYPE_F32)
          rc = launch_cast_f32_to_bf16(static_cast<const float*>(dev_ptr), static_cast<bf16*>(dst),
                                       numel, st);
        else
          rc = launch_cast_bf16_to_f32(static_cast<const bf16*>(dev_ptr), static_cast<float*>(dst),
                                       numel, st);
      } else {
        rc = pack_linear_weight(m, dev_ptr, dtype, s.K, s.N, dst, st);
      }
    }
  }
  if (rc) return rc;
  m->seen[name] = true;
  m->finalized = false;
  return SD3_OK;
}

int sd3_model_finalize(sd3_model* m, int* missing) {
  if (!m) return SD3_ERR_INVALID_ARG;
  int n = 0;
  std::string first;
  for (const auto& r : m->required) {
    if (!m->seen.count(r)) {
      if (n == 0) first = r;
      ++n;
    }
  }
  if (missing) *missing = n;
  if (n) {
    set_last_error("%d required parameter(s) missing, first: %s", n, first.c_str());
    return SD3_ERR_NOT_READY;
  }
  if (m->fp8 && !m->finalized) {
    int rc = quantize_block_weights(m);
    if (rc) return rc;
  }
  if (!m->finalized) {
    int rc = compute_score_bounds(m);
    if (rc) return rc;
  }
  m->finalized = true;
  return SD3_OK;
}

int sd3_model_reserve(sd3_model* m, int B, int Tc, int H, int W) {
  if (!m || B <= 0 || Tc <= 0 || H <= 0 || W <= 0) {
    set_last_error("sd3_model_reserve: invalid argument");
    return SD3_ERR_INVALID_ARG;
  }
  const int p = m->cfg.patch_size > 0 ? m->cfg.patch_size : 1;
  return reserve_ws(m, B, Tc, (H / p) * (W / p));
}

int sd3_block_forward(sd3_model* m, int layer, const float* y, float* c, float* x, int B, int Tc,
                      int Tx, void* stream) {
  if (!m || !y || !c || !x || layer < 0 || layer >= m->cfg.num_layers || B <= 0 || Tc <= 0 ||
      Tx <= 0) {
    set_last_error("sd3_block_forward: invalid argument");
    return SD3_ERR_INVALID_ARG;
  }
  if (!m->finalized) {
    set_last_error("sd3_block_forward: model not finalized");
    return SD3_ERR_NOT_READY;
  }
  int rc = reserve_ws(m, B, Tc, Tx);
  if (rc) return rc;
  cudaStream_t st = S(stream);
  const LayerW& L = m->layers[layer];
  // this layer's AdaLN vectors: rows [c_mod_off, x_mod_off + x_chunks*E) of the matrix
  const long lo = L.c_mod_off, n = static_cast<long>(L.c_chunks + L.x_chunks) * m->E;
  rc = launch_skinny_linear(y, m->E,
                            static_cast<char*>(m->ada_w) + static_cast<size_t>(lo) * m->E * m->wbytes(),
                            m->f32, m->ada_b + lo, nullptr, 0, m->ws.mod + lo, m->ada_total, B,
                            static_cast<int>(n), m->E, 0, st);
  if (rc) return rc;
  return block_body(m, layer, c, x, B, Tc, Tx, m->ws.mod, m->ada_total, st);
}

int sd3_dit_forward(sd3_model* m, const void* pooled, const void* captions, const void* latent,
                    const float* timesteps, void* out, int io_dtype, int B, int Tc, int H, int W,
                    void* stream) {
  if (!m || !pooled || !captions || !latent || !timesteps || !out || B <= 0 || Tc <= 0 ||
      (io_dtype != SD3_DTYPE_F32 && io_dtype != SD3_DTYPE_BF16)) {
    set_last_error("sd3_dit_forward: invalid argument");
    return SD3_ERR_INVALID_ARG;
  }
  if (m->cfg.block_only || !m->finalized) {
    set_last_error("sd3_dit_forward: model is block-only or not finalized");
    return SD3_ERR_NOT_READY;
  }
  const sd3_config& c = m->cfg;
  const int p = c.patch_size;
  if (H % p || W % p || H / p > c.pos_embed_max_size || W / p > c.pos_embed_max_size) {
    set_last_error("sd3_dit_forward: latent %dx%d does not fit patch %d / position grid %d", H, W, p,
                   c.pos_embed_max_size);
    return SD3_ERR_INVALID_ARG;
  }
  const int hp = H / p, wp = W / p, Tx = hp * wp, E = m->E;
  int rc = reserve_ws(m, B, Tc, Tx);
  if (rc) return rc;
  Workspace& w = m->ws;
  cudaStream_t st = S(stream);
  const bool io_f32 = io_dtype == SD3_DTYPE_F32;
#define SD3_TRY(expr) do { rc = (expr); if (rc) return rc; } while (0)
  // position table (cached per grid size)
  if (w.pos_h != hp || w.pos_w != wp || !m->pos_store) {
    const size_t need = static_cast<size_t>(Tx) * E;
    if (need > m->pos_store_elems) {
      if (m->pos_store) cudaFree(m->pos_store);
      m->pos_store = nullptr;
      SD3_TRY(check_cuda(cudaMalloc(&m->pos_store, need * 4), "cudaMalloc(pos table)"));
      m->pos_store_elems = need;
    }
    SD3_TRY(launch_pos_table(m->pos_store, hp, wp, E, c.pos_embed_max_size, c.base_height / p, st));
    w.pos_h = hp; w.pos_w = wp;
  }
  // conditioning vector y = silu(timestep_mlp(emb(t)) + pooled_mlp(pooled))
  const float* pooled32 = static_cast<const float*>(pooled);
  if (!io_f32) {
    SD3_TRY(launch_cast_bf16_to_f32(static_cast<const bf16*>(pooled), w.pooled_f32,
                                    static_cast<long>(B) * c.pooled_dim, st));
    pooled32 = w.pooled_f32;
  }
  SD3_TRY(launch_sinusoidal(timesteps, w.temb, B, 256, st));
  SD3_TRY(launch_skinny_linear(w.temb, 256, m->t1.w, m->f32, m->t1.b, nullptr, 0, w.th, E, B, E, 256, 1, st));
  SD3_TRY(launch_skinny_linear(w.th, E, m->t2.w, m->f32, m->t2.b, nullptr, 0, w.tout, E, B, E, E, 0, st));
  SD3_TRY(launch_skinny_linear(pooled32, c.pooled_dim, m->p1.w, m->f32, m->p1.b, nullptr, 0, w.ph, E, B, E, c.pooled_dim, 1, st));
  SD3_TRY(launch_skinny_linear(w.ph, E, m->p2.w, m->f32, m->p2.b, w.tout, E, w.y, E, B, E, E, 1, st));
  // every AdaLN vector of every block and of the final layer in one launch
  if (!m->f32 && m->ada_total % 64 == 0 && E % 64 == 0) {
    // As a tensor-core GEMM with M = batch: out (B, ada_total) = y W^T + b.  Only B
    // of the 128 rows of each MMA carry data, but the tensor pipe has the room
    // and TMA streams the 1.5 GB of weights at HBM speed, which the SIMT kernel
    // (8 warps per SM at its register count) does not.
    SD3_TRY(launch_cast_f32_to_bf16(w.y, w.y_bf, static_cast<long>(B) * E, st));
    GemmEpilogue e;
    e.mode = EPI_BIAS;
    e.bias = m->ada_b;
    e.out = w.mod;
    e.out_f32 = 1;
    e.ldo = m->ada_total;
    SD3_TRY(launch_gemm(w.y_bf, E, m->ada_w, E, OPERAND_BF16, B, static_cast<int>(m->ada_total), E, e,
                        m->status, st));
  } else {
    SD3_TRY(launch_skinny_linear(w.y, E, m->ada_w, m->f32, m->ada_b, nullptr, 0, w.mod, m->ada_total, B,
                                 static_cast<int>(m->ada_total), E, 0, st));
  }
  // context stream c = captions W + b
  {
    const void* cap_in = captions;
    const long n = static_cast<long>(B) * Tc * c.captions_dim;
    if (io_f32 != m->f32) {
      if (io_f32) SD3_TRY(launch_cast_f32_to_bf16(static_cast<const float*>(captions), static_cast<bf16*>(w.cap_in), n, st));
      else SD3_TRY(launch_cast_bf16_to_f32(static_cast<const bf16*>(captions), static_cast<float*>(w.cap_in), n, st));
      cap_in = w.cap_in;
    }
    GemmEpilogue e;
    e.mode = EPI_BIAS; e.out = w.c; e.out_f32 = 1; e.ldo = E;
    SD3_TRY(run_linear(m, m->cap, cap_in, B * Tc, e, st));
  }
  // image stream x = patch conv + bias + position table
  {
    SD3_TRY(launch_patchify(latent, io_f32, w.patches, m->f32, B, c.in_channels, H, W, p, st));
    GemmEpilogue e;
    e.mode = EPI_ADD_TABLE; e.out = w.x; e.out_f32 = 1; e.ldo = E;
    e.rows_in = Tx; e.rows_out = Tx; e.table = m->pos_store;
    SD3_TRY(run_linear(m, m->patch, w.patches, B * Tx, e, st));
  }
  for (int l = 0; l < c.num_layers; ++l)
    SD3_TRY(block_body(m, l, w.c, w.x, B, Tc, Tx, w.mod, m->ada_total, st));
  // final layer: LN(eps 1e-5) * (1 + scale) + shift with chunks (scale, shift), linear, unpatchify
  {
    const float* fm = w.mod + m->fin_mod_off;
    SD3_TRY(launch_ln_modulate(w.x, B, Tx, E, 1e-5f, fm + E, fm, w.h_x, nullptr, nullptr, nullptr,
                               m->ada_total, m->f32, st));
    GemmEpilogue e;
    e.mode = EPI_UNPATCHIFY; e.out = out; e.out_f32 = io_f32; e.ldo = m->Nout;
    e.rows_in = Tx; e.rows_out = Tx;
    e.up_w = wp; e.up_h = hp; e.up_cin = c.in_channels; e.up_patch = p;
    SD3_TRY(run_linear(m, m->fin, w.h_x, B * Tx, e, st));
  }
#undef SD3_TRY
  return SD3_OK;
}

}  // extern "C"

// `custom_modules`: drop-in torch extension with the entry points of the
// reference's modules.cpp (PYBIND11_MODULE at modules.cpp:1789-1815) for the
// denoiser forward path, running on CUDA tensors through libsd3_b200.so.
//
// This file is host glue only: it validates tensors, picks the precision mode
// from the tensor dtype (float32 -> exact fp32 kernels, bfloat16 -> tcgen05
// bf16 kernels), hands raw pointers to the C ABI (include/sd3_b200.h) on the
// current torch stream and allocates outputs with torch.  There is no CPU
// path: CPU tensors are rejected with an error.
//
// Same names and positional signatures as the reference:
//   DiT            modules.cpp:1605-1613   (reference: CPU only)
//   Dit_block      modules.cpp:1508-1514
//   DiT_block_cuda cuda/dit.cu:919-925
//   linear :538, layer_norm :51, rms_norm :200, conv2d :1065,
//   sinusoidal_embedding :920, positional_embedding :997, mha :901, mlp :1167
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../include/sd3_b200.h"

namespace {

using torch::Tensor;
typedef std::unordered_map<std::string, Tensor> ParamDict;

void ok(int rc, const char* what) {
  TORCH_CHECK(rc == 0, what, " failed (", rc, "): ", sd3_last_error());
}

void* stream() { return static_cast<void*>(at::cuda::getCurrentCUDAStream().stream()); }

int tag(const Tensor& t) {
  TORCH_CHECK(t.scalar_type() == torch::kFloat32 || t.scalar_type() == torch::kBFloat16,
              "custom_modules: float32 or bfloat16 tensors expected, got ", t.scalar_type());
  return t.scalar_type() == torch::kFloat32 ? SD3_DTYPE_F32 : SD3_DTYPE_BF16;
}

Tensor dev(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), "custom_modules: '", name,
              "' must be a CUDA tensor (this build has no CPU path)");
  return t.contiguous();
}

// ---------------------------------------------------------------------------
// model cache: one packed model per (configuration, parameter identity)
// ---------------------------------------------------------------------------
struct ModelHolder {
  sd3_model* m = nullptr;
  ~ModelHolder() { if (m) sd3_model_destroy(m); }
};

struct CacheEntry {
  std::string key;
  std::shared_ptr<ModelHolder> model;
  // The parameter tensors the model was packed from.  The key identifies them by storage
  // address and version counter; holding them keeps those storages alive, so an address in a
  // key can never be that of a newer tensor that reused freed memory (in-place writes bump the
  // version counter and miss the cache as they should).
  std::vector<Tensor> keep;
};

std::mutex g_mu;
std::vector<CacheEntry> g_cache;  // small LRU

std::string make_key(const sd3_config& c, const ParamDict& params, int device) {
  std::string k;
  k.reserve(64 + params.size() * 24);
  auto add = [&k](uint64_t v) { k.append(reinterpret_cast<const char*>(&v), sizeof(v)); };
  add(c.num_layers); add(c.dual_attention_mask); add(c.pooled_dim); add(c.captions_dim);
  add(c.in_channels); add(c.emb_dim); add(c.attn_heads); add(c.mlp_expand); add(c.patch_size);
  add(c.pos_embed_max_size); add(c.base_height); add(c.use_qk_norm); add(c.last_discards_context);
  add(c.precision); add(c.block_only); add(static_cast<uint64_t>(device));
  // order-independent digest of (name, storage address, version counter)
  uint64_t acc = 0;
  for (const auto& kv : params) {
    uint64_t h = std::hash<std::string>()(kv.first);
    h ^= reinterpret_cast<uint64_t>(kv.second.data_ptr()) * 0x9E3779B97F4A7C15ull;
    h ^= static_cast<uint64_t>(kv.second._version()) * 0xC2B2AE3D27D4EB4Full;
    acc += h * 0xD6E8FEB86659FD93ull;
  }
  add(acc); add(params.size());
  return k;
}

std::shared_ptr<ModelHolder> get_model(const sd3_config& cfg, const ParamDict& params,
                                       const std::string& prefix, int device) {
  const std::string key = make_key(cfg, params, device);
  std::lock_guard<std::mutex> lock(g_mu);
  for (size_t i = 0; i < g_cache.size(); ++i) {
    if (g_cache[i].key == key) {
      CacheEntry e = g_cache[i];
      g_cache.erase(g_cache.begin() + i);
      g_cache.push_back(e);
      return e.model;
    }
  }
  auto holder = std::make_shared<ModelHolder>();
  ok(sd3_model_create(&cfg, &holder->m), "sd3_model_create");
  for (const auto& kv : params) {
    Tensor t = dev(kv.second, kv.first.c_str());
    std::vector<int64_t> shape(t.sizes().begin(), t.sizes().end());
    const std::string name = prefix + kv.first;
    ok(sd3_model_set_param(holder->m, name.c_str(), t.data_ptr(), tag(t), static_cast<int>(shape.size()),
                           shape.data(), stream()),
       "sd3_model_set_param");
  }
  int missing = 0;
  ok(sd3_model_finalize(holder->m, &missing), "sd3_model_finalize");
  if (g_cache.size() >= 4) g_cache.erase(g_cache.begin());
  std::vector<Tensor> keep;
  keep.reserve(params.size());
  for (const auto& kv : params) keep.push_back(kv.second);
  g_cache.push_back({key, holder, std::move(keep)});
  return holder;
}

int precision_of(const Tensor& t) {
  return t.scalar_type() == torch::kFloat32 ? SD3_PRECISION_F32 : SD3_PRECISION_BF16;
}

// ---------------------------------------------------------------------------
// model-level entry points
// ---------------------------------------------------------------------------
Tensor DiT_forward(Tensor& pooled_captions, Tensor& captions, Tensor& latent_vector,
                   Tensor& timesteps, ParamDict& params, int num_layers,
                   std::unordered_set<int> dual_attention_layers, int pooled_dim, int captions_dim,
                   int C_in, int emb_dim, int attn_heads, int mlp_expand, int patch_size,
                   int pos_embed_max_size, int base_height, bool use_qk_norm) {
  Tensor latent = dev(latent_vector, "latent_vector");
  c10::cuda::CUDAGuard guard(latent.device());
  const auto dt = latent.scalar_type();
  Tensor pooled = dev(pooled_captions, "pooled_captions").to(dt);
  Tensor caps = dev(captions, "captions").to(dt);
  Tensor t32 = dev(timesteps, "timesteps").to(torch::kFloat32);
  TORCH_CHECK(latent.dim() == 4 && caps.dim() == 3 && pooled.dim() == 2 && t32.dim() == 1,
              "DiT: expected latent (B,C,H,W), captions (B,Tc,D), pooled (B,P), timesteps (B,)");
  const int B = latent.size(0), H = latent.size(2), W = latent.size(3), Tc = caps.size(1);
  TORCH_CHECK(latent.size(1) == C_in && caps.size(2) == captions_dim &&
              pooled.size(1) == pooled_dim && caps.size(0) == B && pooled.size(0) == B &&
              t32.size(0) == B, "DiT: tensor shapes do not match the given dimensions");
  sd3_config cfg{};
  cfg.num_layers = num_layers;
  for (int l : dual_attention_layers) {
    TORCH_CHECK(l >= 0 && l < 64, "DiT: dual attention layer index out of range");
    cfg.dual_attention_mask |= (1ull << l);
  }
  cfg.pooled_dim = pooled_dim; cfg.captions_dim = captions_dim; cfg.in_channels = C_in;
  cfg.emb_dim = emb_dim; cfg.attn_heads = attn_heads; cfg.mlp_expand = mlp_expand;
  cfg.patch_size = patch_size; cfg.pos_embed_max_size = pos_embed_max_size;
  cfg.base_height = base_height; cfg.use_qk_norm = use_qk_norm;
  cfg.last_discards_context = 1; cfg.precision = precision_of(latent); cfg.block_only = 0;
  auto model = get_model(cfg, params, "", latent.get_device());
  Tensor out = torch::empty_like(latent);
  ok(sd3_dit_forward(model->m, pooled.data_ptr(), caps.data_ptr(), latent.data_ptr(),
                     t32.data_ptr<float>(), out.data_ptr(), tag(latent), B, Tc, H, W, stream()),
     "sd3_dit_forward");
  return out;
}

// In place on context_embeddings and latent_vector, like the reference
// (modules.cpp:1602, cuda/dit.cu:1060); returns the same tensor objects.
std::vector<Tensor> DiT_block_forward_cuda(Tensor& temp_embeddings, Tensor& context_embeddings,
                                           Tensor& latent_vector, ParamDict& params, int B, int Tc,
                                           int Tx, int emb_dim, int attn_heads, int mlp_expand,
                                           bool use_dual_attention, bool use_qk_norm,
                                           bool discard_context) {
  TORCH_CHECK(latent_vector.is_cuda() && context_embeddings.is_cuda() && temp_embeddings.is_cuda(),
              "Dit_block: CUDA tensors required (this build has no CPU path)");
  c10::cuda::CUDAGuard guard(latent_vector.device());
  TORCH_CHECK(latent_vector.is_contiguous() && context_embeddings.is_contiguous(),
              "Dit_block: c and x must be contiguous (they are updated in place)");
  TORCH_CHECK(latent_vector.numel() == (int64_t)B * Tx * emb_dim &&
              context_embeddings.numel() == (int64_t)B * Tc * emb_dim &&
              temp_embeddings.numel() == (int64_t)B * emb_dim, "Dit_block: shape mismatch");
  sd3_config cfg{};
  cfg.num_layers = 1;
  cfg.dual_attention_mask = use_dual_attention ? 1 : 0;
  cfg.emb_dim = emb_dim; cfg.attn_heads = attn_heads; cfg.mlp_expand = mlp_expand;
  cfg.use_qk_norm = use_qk_norm; cfg.last_discards_context = discard_context;
  cfg.precision = precision_of(latent_vector); cfg.block_only = 1;
  auto model = get_model(cfg, params, "transformer.0.", latent_vector.get_device());
  // the fp32 residual streams live in the caller's tensors when they are float32
  const bool f32 = latent_vector.scalar_type() == torch::kFloat32;
  Tensor y = temp_embeddings.to(torch::kFloat32).contiguous();
  Tensor c = f32 ? context_embeddings : context_embeddings.to(torch::kFloat32);
  Tensor x = f32 ? latent_vector : latent_vector.to(torch::kFloat32);
  ok(sd3_block_forward(model->m, 0, y.data_ptr<float>(), c.data_ptr<float>(), x.data_ptr<float>(),
                       B, Tc, Tx, stream()),
     "sd3_block_forward");
  if (!f32) {
    context_embeddings.copy_(c);
    latent_vector.copy_(x);
  }
  return {context_embeddings, latent_vector};
}

// ---------------------------------------------------------------------------
// per-operator entry points
// ---------------------------------------------------------------------------
Tensor pack(const Tensor& w_in_out, torch::ScalarType dt) {
  Tensor w = dev(w_in_out, "weight");
  TORCH_CHECK(w.dim() == 2, "weight must be (C_in, C_out)");
  Tensor out = torch::empty({w.size(1), w.size(0)}, w.options().dtype(dt));
  ok(sd3_pack_weight(w.data_ptr(), tag(w), out.data_ptr(), dt == torch::kFloat32 ? 0 : 1,
                     (int)w.size(0), (int)w.size(1), stream()),
     "sd3_pack_weight");
  return out;
}

Tensor bias_f32(const Tensor& b, int64_t n) {
  Tensor r = dev(b, "bias").to(torch::kFloat32).contiguous();
  TORCH_CHECK(r.numel() == n, "bias size mismatch");
  return r;
}

Tensor linear_impl(const Tensor& x_in, const Tensor& W, const Tensor& b, int act) {
  Tensor x = dev(x_in, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t K = x.size(-1), N = W.size(1), M = x.numel() / K;
  TORCH_CHECK(W.size(0) == K, "linear: weight must be (C_in, C_out)");
  std::vector<int64_t> oshape(x.sizes().begin(), x.sizes().end());
  oshape.back() = N;
  Tensor bias = bias_f32(b, N);
  Tensor out = torch::empty(oshape, x.options());
  if (x.scalar_type() == torch::kFloat32) {
    Tensor w = pack(W, torch::kFloat32);
    ok(sd3_linear_f32(x.data_ptr<float>(), w.data_ptr<float>(), bias.data_ptr<float>(),
                      out.data_ptr<float>(), (int)M, (int)N, (int)K, act, stream()),
       "sd3_linear_f32");
  } else {
    tag(x);
    Tensor w = pack(W, torch::kBFloat16);
    ok(sd3_linear(x.data_ptr(), w.data_ptr(), bias.data_ptr<float>(), out.data_ptr(), SD3_DTYPE_BF16,
                  (int)M, (int)N, (int)K, act, stream()),
       "sd3_linear");
  }
  return out;
}

Tensor Linear_forward(Tensor& x, Tensor& W, Tensor& b) { return linear_impl(x, W, b, SD3_ACT_NONE); }

// mlp(x, W1, b1, W2, b2, activation, B, C_in, C_hid, C_out) -- "gelu_tanh" only
Tensor MLP(Tensor& x, Tensor& W1, Tensor& b1, Tensor& W2, Tensor& b2, std::string activation, int B,
           int C_in, int C_hid, int C_out) {
  TORCH_CHECK(activation == "gelu_tanh" || activation == "gelu",
              "mlp: only the GELU-tanh MLP of the DiT blocks is provided (got '", activation, "')");
  TORCH_CHECK(W1.size(0) == C_in && W1.size(1) == C_hid && W2.size(1) == C_out, "mlp: shape mismatch");
  Tensor h = linear_impl(x, W1, b1, SD3_ACT_GELU_TANH);
  return linear_impl(h, W2, b2, SD3_ACT_NONE);
}

// layer_norm(x (B,T,C), w, b, eps, save_for_backward) -> [out]
std::vector<Tensor> LayerNorm_forward(Tensor& x_in, Tensor& w, Tensor& b, float eps,
                                      bool save_for_backward) {
  TORCH_CHECK(!save_for_backward, "layer_norm: forward only (no statistics are saved)");
  Tensor x = dev(x_in, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t C = x.size(-1), rows = x.numel() / C;
  Tensor x32 = x.to(torch::kFloat32).contiguous();
  // LN(x) * w + b == LN(x) * (1 + (w - 1)) + b
  Tensor scale = (dev(w, "w").to(torch::kFloat32) - 1.0).contiguous();
  Tensor shift = dev(b, "b").to(torch::kFloat32).contiguous();
  Tensor out = torch::empty_like(x);
  ok(sd3_layernorm_modulate(x32.data_ptr<float>(), 1, (int)rows, (int)C, eps, shift.data_ptr<float>(),
                            scale.data_ptr<float>(), out.data_ptr(), nullptr, nullptr, nullptr, 0,
                            tag(out), stream()),
     "sd3_layernorm_modulate");
  return {out};
}

// rms_norm(x (..., C), w (C,), eps, save_for_backward) -> [out]
std::vector<Tensor> RMSNorm_forward(Tensor& x_in, Tensor& w, float eps, bool save_for_backward) {
  TORCH_CHECK(!save_for_backward, "rms_norm: forward only");
  Tensor x = dev(x_in, "x").clone();
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t C = x.size(-1), rows = x.numel() / C;
  Tensor wf = dev(w, "w").to(torch::kFloat32).contiguous();
  ok(sd3_rmsnorm_heads(x.data_ptr(), tag(x), C, rows, 0, 1, (int)C, wf.data_ptr<float>(), eps, stream()),
     "sd3_rmsnorm_heads");
  return {x};
}

// conv2d(x (B,C,H,W), kernel (O,I,kh,kw), bias, stride, padding): the patch-embedding form
// (kernel == stride, padding 0) runs as gather + tensor-core GEMM, every other shape through the
// stand-alone convolution kernel
Tensor conv2d_forward(Tensor& x_in, Tensor& kernel, Tensor& bias, int stride, int padding) {
  Tensor x = dev(x_in, "x");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor k = dev(kernel, "kernel");
  TORCH_CHECK(x.dim() == 4 && k.dim() == 4, "conv2d: (B,C,H,W) input and (O,I,kh,kw) kernel expected");
  TORCH_CHECK(k.size(1) == x.size(1), "conv2d: kernel and input channel counts differ");
  TORCH_CHECK(stride > 0 && padding >= 0, "conv2d: stride must be positive and padding non-negative");
  const int B = x.size(0), C = x.size(1), H = x.size(2), W = x.size(3), O = k.size(0), p = stride;
  Tensor bf = bias_f32(bias, O);
  const bool patch_form = padding == 0 && k.size(2) == stride && k.size(3) == stride && H % p == 0 && W % p == 0 &&
                          (C * p * p) % 8 == 0 && O % 8 == 0;
  if (!patch_form) {
    const int kh = k.size(2), kw = k.size(3);
    TORCH_CHECK(H + 2 * padding >= kh && W + 2 * padding >= kw, "conv2d: kernel larger than the padded input");
    const int Ho = (H + 2 * padding - kh) / stride + 1, Wo = (W + 2 * padding - kw) / stride + 1;
    Tensor wf = k.to(torch::kFloat32).contiguous();
    Tensor out = torch::empty({B, O, Ho, Wo}, x.options());
    ok(sd3_conv2d(x.data_ptr(), tag(x), wf.data_ptr<float>(), bf.data_ptr<float>(), out.data_ptr(), B, C, H, W, O,
                  kh, kw, stride, padding, stream()),
       "sd3_conv2d");
    return out;
  }
  const int hp = H / p, wp = W / p, Kp = C * p * p;
  Tensor zero_table = torch::zeros({(int64_t)hp * wp, O}, x.options().dtype(torch::kFloat32));
  Tensor tokens = torch::empty({(int64_t)B * hp * wp, O}, x.options().dtype(torch::kFloat32));
  Tensor w16 = k.reshape({O, Kp}).to(torch::kBFloat16).contiguous();
  Tensor scratch = torch::empty({(int64_t)B * hp * wp, Kp}, x.options().dtype(torch::kBFloat16));
  ok(sd3_patch_embed(x.data_ptr(), tag(x), w16.data_ptr(), bf.data_ptr<float>(),
                     zero_table.data_ptr<float>(), tokens.data_ptr<float>(), scratch.data_ptr(), B, C,
                     H, W, p, O, stream()),
     "sd3_patch_embed");
  return tokens.view({B, hp, wp, O}).permute({0, 3, 1, 2}).contiguous().to(x.scalar_type());
}

Tensor sinusoidal_embedding(Tensor& t_in, int emb_dim) {
  Tensor t = dev(t_in, "t").to(torch::kFloat32).contiguous();
  c10::cuda::CUDAGuard guard(t.device());
  Tensor out = torch::empty({t.size(0), emb_dim}, t.options());
  ok(sd3_sinusoidal_embedding(t.data_ptr<float>(), out.data_ptr<float>(), (int)t.size(0), emb_dim,
                              stream()),
     "sd3_sinusoidal_embedding");
  return out;
}

// positional_embedding(emb_dim, height, width, base_size) -> (height*width, emb_dim), on the current device
Tensor positional_embedding2D_forward(int emb_dim, int height, int width, int base_size) {
  TORCH_CHECK(height == width, "positional_embedding: square grids only (as the reference builds them)");
  Tensor out = torch::empty({(int64_t)height * width, emb_dim},
                            torch::TensorOptions().dtype(torch::kFloat32).device(torch::kCUDA));
  ok(sd3_pos_embed_table(out.data_ptr<float>(), height, width, emb_dim, height, base_size, stream()),
     "sd3_pos_embed_table");
  return out;
}

// mha(Q (B,T,C), K (B,L,C), V (B,L,C), num_heads) -> (B,T,C); L may differ from T
Tensor mha(Tensor& Q, Tensor& K, Tensor& V, int num_heads) {
  Tensor q = dev(Q, "Q"), k = dev(K, "K"), v = dev(V, "V");
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.sizes() == k.sizes() && k.size(0) == q.size(0) &&
                  k.size(2) == q.size(2) && k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(),
              "mha: Q (B,T,C) and K, V (B,L,C) of one dtype expected");
  const int B = q.size(0), T = q.size(1), C = q.size(2), L = k.size(1);
  TORCH_CHECK(C % num_heads == 0, "mha: C must be divisible by num_heads");
  const int D = C / num_heads;
  TORCH_CHECK(D <= 128, "mha: head_dim above 128 is not provided");
  Tensor out = torch::empty_like(q);
  if (L != T) {
    ok(sd3_cross_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), C, C, tag(q), B, T, L, num_heads, D,
                           out.data_ptr(), C, tag(out), 1.0f / std::sqrt((float)D), stream()),
       "sd3_cross_attention");
    return out;
  }
  if (q.scalar_type() == torch::kBFloat16 && D == 64) {
    Tensor qkv = torch::cat({q, k, v}, 2).contiguous();
    ok(sd3_attention(qkv.data_ptr(), B, T, num_heads, 0, nullptr, out.data_ptr(),
                     1.0f / std::sqrt((float)D), stream()),
       "sd3_attention");
  } else {
    ok(sd3_attention_generic(q.data_ptr(), k.data_ptr(), v.data_ptr(), C, tag(q), B, T, num_heads, D,
                             out.data_ptr(), C, tag(out), 1.0f / std::sqrt((float)D), stream()),
       "sd3_attention_generic");
  }
  return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("layer_norm", &LayerNorm_forward, "LayerNorm forward");
  m.def("rms_norm", &RMSNorm_forward, "RMSNorm forward");
  m.def("linear", &Linear_forward, "Linear forward");
  m.def("conv2d", &conv2d_forward, "Conv2d forward (patch embedding form)");
  m.def("sinusoidal_embedding", &sinusoidal_embedding, "Temporal sinusoidal embeddings");
  m.def("positional_embedding", &positional_embedding2D_forward, "2D positional embeddings");
  m.def("mha", &mha, "multi-head self attention");
  m.def("mlp", &MLP, "MLP");
  m.def("Dit_block", &DiT_block_forward_cuda, "Stable diffusion's DiT block");
  m.def("DiT", &DiT_forward, "SD3.5 medium");
  m.def("DiT_block_cuda", &DiT_block_forward_cuda, "Stable diffusion's DiT block (CUDA tensors)");
}

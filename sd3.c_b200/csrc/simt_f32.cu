// Exact-fp32 SIMT kernels: a shared-memory tiled FFMA GEMM with the same fused
// epilogues as the tcgen05 GEMM, and a generic attention kernel for any head
// size up to 128.  They serve the fp32 parity mode (fp32 tensors in, results
// within 1e-4 of the fp32 PyTorch modules) and shapes the tensor-core kernels
// do not cover (head_dim != 64).  Speed is secondary here; the arithmetic is
// plain fp32 FMA with fp32 accumulation.
//
// Reference counterparts: linear / partial_linear (modules.cpp:475-511) and
// multihead_attention (modules.cpp:766-831).
#include "kernels.h"
#include "ptx.cuh"

namespace sd3 {

namespace {

constexpr int SG_BM = 64, SG_BN = 64, SG_BK = 16;

__device__ __forceinline__ float gelu_tanh_exact(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}

template <bool OUT_F32>
__device__ __forceinline__ void epilogue_scalar(float acc, int m, int n, int N,
                                                const GemmEpilogue& e) {
  int b = 0, t_in = m;
  long orow = m;
  if (e.rows_in > 0) {
    b = m / e.rows_in;
    t_in = m - b * e.rows_in;
    orow = static_cast<long>(b) * e.rows_out + e.row_off + t_in;
  }
  float v = acc * e.alpha + (e.bias ? e.bias[n] : 0.f);
  long idx = orow * e.ldo + n;
  switch (e.mode) {
    case EPI_BIAS_GELU:
      v = gelu_tanh_exact(v);
      break;
    case EPI_GATE_RESID:
      v = e.resid[idx] + e.gate[static_cast<long>(b) * e.gate_stride + n] * v;
      break;
    case EPI_ADD_TABLE:
      v += e.table[static_cast<long>(t_in) * N + n];
      break;
    case EPI_UNPATCHIFY: {
      const int p = e.up_patch, C = e.up_cin;
      const int s = t_in % e.up_w, r = t_in / e.up_w;
      const long Wpix = static_cast<long>(e.up_w) * p, Hpix = static_cast<long>(e.up_h) * p;
      const int c = n % C, pw = (n / C) % p, ph = n / (C * p);
      idx = ((static_cast<long>(b) * C + c) * Hpix + (r * p + ph)) * Wpix + (s * p + pw);
      break;
    }
    default:
      break;
  }
  if constexpr (OUT_F32)
    static_cast<float*>(e.out)[idx] = v;
  else
    static_cast<bf16*>(e.out)[idx] = __float2bfloat16(v);
}

template <bool OUT_F32>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, long lda, const float* __restrict__ W, long ldw, int M,
                int N, int K, const GemmEpilogue e) {
  __shared__ float As[SG_BK][SG_BM + 4];
  __shared__ float Ws[SG_BK][SG_BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // each thread loads 4 elements of the A tile and 4 of the W tile per step
  const int lr = tid >> 2;        // 0..63 row within tile
  const int lk = (tid & 3) * 4;   // 0,4,8,12
  for (int k0 = 0; k0 < K; k0 += SG_BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + j][lr] = (am < M && k < K) ? A[static_cast<long>(am) * lda + k] : 0.f;
      Ws[lk + j][lr] = (wn < N && k < K) ? W[static_cast<long>(wn) * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SG_BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) epilogue_scalar<OUT_F32>(acc[i][j], m, n, N, e);
    }
  }
}

// ----------------------------------------------------------------------------
// Generic attention: one warp per (sample, head, query).  Lanes split the keys,
// each keeps its own online-softmax state and a D-wide partial output; the 32
// partial states are merged with shuffles at the end.
// ----------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <> __device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_as_float<bf16>(const bf16* p) { return __bfloat162float(*p); }

template <typename IT, typename OT, int DV>  // DV = ceil(D / 32) values of q per lane
__global__ void __launch_bounds__(128)
attention_simt_kernel(const IT* __restrict__ q, const IT* __restrict__ k, const IT* __restrict__ v,
                      long ld, long ldk, int B, int T, int L, int NH, int D, int Tc, OT* __restrict__ out_c,
                      OT* __restrict__ out_x, long ldo, float scale) {
  extern __shared__ float sq[];  // per warp: D floats of the scaled query
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long unit = static_cast<long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  const long total = static_cast<long>(B) * NH * T;
  if (unit >= total) return;
  const int t = static_cast<int>(unit % T);
  const int h = static_cast<int>((unit / T) % NH);
  const int b = static_cast<int>(unit / (static_cast<long>(T) * NH));
  float* myq = sq + warp * D;
  const IT* qp = q + (static_cast<long>(b) * T + t) * ld + h * D;
  for (int i = lane; i < D; i += 32) myq[i] = ld_as_float(qp + i) * scale;
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float o[DV * 32];
#pragma unroll
  for (int i = 0; i < DV * 32; ++i) o[i] = 0.f;
  for (int j = lane; j < L; j += 32) {  // L keys per sample (== T for self-attention)
    const IT* kp = k + (static_cast<long>(b) * L + j) * ldk + h * D;
    const IT* vp = v + (static_cast<long>(b) * L + j) * ldk + h * D;
    float s = 0.f;
    for (int i = 0; i < D; ++i) s = fmaf(myq[i], ld_as_float(kp + i), s);
    const float m_new = fmaxf(m, s);
    const float alpha = expf(m - m_new);  // 0 on the first key (m = -inf)
    const float p = expf(s - m_new);
    l = l * alpha + p;
#pragma unroll
    for (int i = 0; i < DV * 32; ++i)
      if (i < D) o[i] = fmaf(p, ld_as_float(vp + i), o[i] * alpha);
    m = m_new;
  }
  // merge the 32 lane states
  const float m_all = warp_max(m);
  const float f = (m == -INFINITY) ? 0.f : expf(m - m_all);
  const float l_all = warp_sum(l * f);
  const float inv = 1.0f / l_all;
  OT* dst = nullptr;
  if (t < Tc) {
    if (out_c) dst = out_c + (static_cast<long>(b) * Tc + t) * ldo + h * D;
  } else {
    dst = out_x + (static_cast<long>(b) * (T - Tc) + (t - Tc)) * ldo + h * D;
  }
#pragma unroll
  for (int i = 0; i < DV * 32; ++i) {
    if (i < D) {
      const float tot = warp_sum(o[i] * f) * inv;
      if (dst && lane == (i & 31)) {
        if constexpr (sizeof(OT) == 4)
          reinterpret_cast<float*>(dst)[i] = tot;
        else
          reinterpret_cast<bf16*>(dst)[i] = __float2bfloat16(tot);
      }
    }
  }
}

template <typename IT, typename OT>
int launch_attn_inst(const void* q, const void* k, const void* v, long ld, long ldk, int B, int T, int L, int NH,
                     int D, int Tc, void* out_c, void* out_x, long ldo, float scale,
                     cudaStream_t stream) {
  const long total = static_cast<long>(B) * NH * T;
  const int wpb = 4;
  const unsigned grid = static_cast<unsigned>((total + wpb - 1) / wpb);
  const size_t smem = static_cast<size_t>(wpb) * D * sizeof(float);
  if (D <= 32)
    attention_simt_kernel<IT, OT, 1><<<grid, wpb * 32, smem, stream>>>(
        (const IT*)q, (const IT*)k, (const IT*)v, ld, ldk, B, T, L, NH, D, Tc, (OT*)out_c, (OT*)out_x, ldo, scale);
  else if (D <= 64)
    attention_simt_kernel<IT, OT, 2><<<grid, wpb * 32, smem, stream>>>(
        (const IT*)q, (const IT*)k, (const IT*)v, ld, ldk, B, T, L, NH, D, Tc, (OT*)out_c, (OT*)out_x, ldo, scale);
  else
    attention_simt_kernel<IT, OT, 4><<<grid, wpb * 32, smem, stream>>>(
        (const IT*)q, (const IT*)k, (const IT*)v, ld, ldk, B, T, L, NH, D, Tc, (OT*)out_c, (OT*)out_x, ldo, scale);
  return after_launch("attention_simt_kernel");
}

}  // namespace

int launch_gemm_f32(const float* A, long lda, const float* W, long ldw, int M, int N, int K,
                    const GemmEpilogue& epi, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || !A || !W || !epi.out) {
    set_last_error("gemm_f32: invalid argument (M %d N %d K %d)", M, N, K);
    return ST_INVALID_ARG;
  }
  if (epi.mode == EPI_GATE_RESID && (!epi.gate || !epi.resid)) {
    set_last_error("gemm_f32: gate/residual epilogue needs gate and resid pointers");
    return ST_INVALID_ARG;
  }
  const dim3 grid((N + SG_BN - 1) / SG_BN, (M + SG_BM - 1) / SG_BM);
  if (epi.out_f32)
    gemm_f32_kernel<true><<<grid, 256, 0, stream>>>(A, lda, W, ldw, M, N, K, epi);
  else
    gemm_f32_kernel<false><<<grid, 256, 0, stream>>>(A, lda, W, ldw, M, N, K, epi);
  return after_launch("gemm_f32_kernel");
}

int launch_attention_simt(const void* q, const void* k, const void* v, long ld, int in_f32, int B,
                          int T, int NH, int D, int Tc, void* out_c, void* out_x, long ldo,
                          int out_f32, float scale, cudaStream_t stream, int L, long ldk) {
  if (L <= 0) L = T;
  if (ldk <= 0) ldk = ld;
  if (!q || !k || !v || !out_x || B <= 0 || T <= 0 || NH <= 0 || D <= 0 || D > 128 || Tc < 0 ||
      Tc > T) {
    set_last_error("attention_generic: invalid argument (head_dim %d must be <= 128)", D);
    return ST_INVALID_ARG;
  }
  if (in_f32 && out_f32)
    return launch_attn_inst<float, float>(q, k, v, ld, ldk, B, T, L, NH, D, Tc, out_c, out_x, ldo, scale, stream);
  if (in_f32)
    return launch_attn_inst<float, bf16>(q, k, v, ld, ldk, B, T, L, NH, D, Tc, out_c, out_x, ldo, scale, stream);
  if (out_f32)
    return launch_attn_inst<bf16, float>(q, k, v, ld, ldk, B, T, L, NH, D, Tc, out_c, out_x, ldo, scale, stream);
  return launch_attn_inst<bf16, bf16>(q, k, v, ld, ldk, B, T, L, NH, D, Tc, out_c, out_x, ldo, scale, stream);
}

}  // namespace sd3

// Fused epilogues shared by the tcgen05 GEMM kernels (one-CTA and CTA-pair
// variants): bias / GELU-tanh / gate+residual / per-head QK-RMSNorm with token
// re-mapping / position-table add / unpatchify, applied to accumulator rows read
// from TMEM (one output row per thread).
#pragma once
#include "kernels.h"
#include "ptx.cuh"

namespace sd3 {
namespace gemm_detail {

constexpr int EPI_WARPS = 8;

struct GemmArgs {
  int M, N, K;       // K in elements
  int k_blocks;      // ceil(K / elements per stage)
  int tiles_m, tiles_n;
  GemmEpilogue epi;
  int* status;
};

__device__ __forceinline__ float gelu_tanh_f(float x) {
  // 0.5 x (1 + tanh(u)),  u = sqrt(2/pi) (x + 0.044715 x^3); one MUFU op per element
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}

template <bool OUT_F32>
__device__ __forceinline__ void store8(void* out, long idx, const float (&o)[8]) {
  if constexpr (OUT_F32) {
    float4* p = reinterpret_cast<float4*>(static_cast<float*>(out) + idx);
    p[0] = make_float4(o[0], o[1], o[2], o[3]);
    p[1] = make_float4(o[4], o[5], o[6], o[7]);
  } else {
    uint4 u;
    u.x = pack_bf16x2(o[0], o[1]);
    u.y = pack_bf16x2(o[2], o[3]);
    u.z = pack_bf16x2(o[4], o[5]);
    u.w = pack_bf16x2(o[6], o[7]);
    *reinterpret_cast<uint4*>(static_cast<bf16*>(out) + idx) = u;
  }
}

__device__ __forceinline__ void load8(const float* p, float (&o)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
  o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}

// Epilogue for 64 consecutive accumulator columns of one row.
template <int EPI, bool OUT_F32>
__device__ __forceinline__ void epilogue_64(float (&v)[64], int m, int n_base,
                                            const GemmArgs& g) {
  const GemmEpilogue& e = g.epi;
  const int N = g.N;
  int b = 0;
  long orow = m;
  int t_in = m;
  if (e.rows_in > 0) {
    b = m / e.rows_in;
    t_in = m - b * e.rows_in;
    orow = static_cast<long>(b) * e.rows_out + e.row_off + t_in;
  }
  // bias (and dequantisation scale)
#pragma unroll
  for (int gi = 0; gi < 8; ++gi) {
    const int n = n_base + gi * 8;
    if (n < N) {
      float bb[8];
      if (e.bias) {
        load8(e.bias + n, bb);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) bb[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) v[gi * 8 + j] = fmaf(v[gi * 8 + j], e.alpha, bb[j]);
    }
  }
  if constexpr (EPI == EPI_QKV_NORM) {
    if (e.do_norm && n_base < e.qk_cols) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 64; ++j) ss = fmaf(v[j], v[j], ss);
      const float r = rsqrtf(ss * (1.0f / 64.0f) + e.eps);
      const float* w = (n_base < (e.qk_cols >> 1)) ? e.wq : e.wk;
#pragma unroll
      for (int gi = 0; gi < 8; ++gi) {
        float ww[8];
        if (w) {
          load8(w + gi * 8, ww);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) ww[j] = 1.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) v[gi * 8 + j] = v[gi * 8 + j] * r * ww[j];
      }
    }
  }
  if constexpr (EPI == EPI_UNPATCHIFY) {
    // m = (b, r, s) over the patch grid; n = ph * (p * C) + pw * C + c
    const int p = e.up_patch, C = e.up_cin;
    const int s = t_in % e.up_w, r = t_in / e.up_w;
    const long Wpix = static_cast<long>(e.up_w) * p, Hpix = static_cast<long>(e.up_h) * p;
    for (int j = 0; j < 64; ++j) {
      const int n = n_base + j;
      if (n >= N) break;
      const int c = n % C;
      const int pw = (n / C) % p;
      const int ph = n / (C * p);
      const long idx = ((static_cast<long>(b) * C + c) * Hpix + (r * p + ph)) * Wpix + (s * p + pw);
      if constexpr (OUT_F32)
        static_cast<float*>(e.out)[idx] = v[j];
      else
        static_cast<bf16*>(e.out)[idx] = __float2bfloat16(v[j]);
    }
    return;
  }
#pragma unroll
  for (int gi = 0; gi < 8; ++gi) {
    const int n = n_base + gi * 8;
    if (n >= N) break;
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = v[gi * 8 + j];
    if constexpr (EPI == EPI_BIAS_GELU) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = gelu_tanh_f(o[j]);
    } else if constexpr (EPI == EPI_GATE_RESID) {
      float gg[8], rr[8];
      load8(e.gate + static_cast<long>(b) * e.gate_stride + n, gg);
      const float4* rp = reinterpret_cast<const float4*>(e.resid + orow * e.ldo + n);
      const float4 r0 = rp[0], r1 = rp[1];
      rr[0] = r0.x; rr[1] = r0.y; rr[2] = r0.z; rr[3] = r0.w;
      rr[4] = r1.x; rr[5] = r1.y; rr[6] = r1.z; rr[7] = r1.w;
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = fmaf(gg[j], o[j], rr[j]);
    } else if constexpr (EPI == EPI_ADD_TABLE) {
      float tt[8];
      load8(e.table + static_cast<long>(t_in) * N + n, tt);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] += tt[j];
    }
    store8<OUT_F32>(e.out, orow * e.ldo + n, o);
  }
}

// Residual row segment of 32 columns into registers (issued early so that the
// DRAM/L2 latency overlaps the main loop or the previous sub-chunk).
__device__ __forceinline__ void load_resid32(const float* p, int n_base, int N, float4 (&rr)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (n_base + i * 4 < N) {
      asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(rr[i].x), "=f"(rr[i].y), "=f"(rr[i].z), "=f"(rr[i].w)
                   : "l"(p + i * 4));
    }
  }
}

// out = resid + gate[b] * (acc * alpha + bias) on 32 columns of one row
__device__ __forceinline__ void epilogue_gate32(const uint32_t (&acc)[32], const float4 (&rr)[8],
                                                float* out_row, const float* gate_row, int n_base,
                                                const GemmArgs& g) {
  const GemmEpilogue& e = g.epi;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int n = n_base + i * 4;
    if (n < g.N) {
      const float4 gg = __ldg(reinterpret_cast<const float4*>(gate_row + n));
      float4 bb = make_float4(0.f, 0.f, 0.f, 0.f);
      if (e.bias) bb = __ldg(reinterpret_cast<const float4*>(e.bias + n));
      float4 o;
      o.x = fmaf(gg.x, fmaf(__uint_as_float(acc[4 * i + 0]), e.alpha, bb.x), rr[i].x);
      o.y = fmaf(gg.y, fmaf(__uint_as_float(acc[4 * i + 1]), e.alpha, bb.y), rr[i].y);
      o.z = fmaf(gg.z, fmaf(__uint_as_float(acc[4 * i + 2]), e.alpha, bb.z), rr[i].z);
      o.w = fmaf(gg.w, fmaf(__uint_as_float(acc[4 * i + 3]), e.alpha, bb.w), rr[i].w);
      *reinterpret_cast<float4*>(out_row + n) = o;
    }
  }
}


// Drains this warp's share of one accumulator tile (rows = TMEM lanes of the
// warp's quadrant, columns [half * BN/2, (half+1) * BN/2)) through the epilogue.
// t_row: TMEM address of the accumulator (lane quadrant and column base applied);
// m: global output row of this thread; n0: first output column of the tile.
// Waits for the accumulator on tfull_bar; returns false if that wait gave up.
template <int BN, int EPI, bool OUT_F32>
__device__ __forceinline__ bool drain_tile(uint32_t t_row, int m, int n0, int half, const GemmArgs& g,
                                           uint64_t* tfull_bar, uint32_t phase, const WaitCtx& wc) {
  constexpr int COLS_PER_WARP = BN / 2;
  if constexpr (EPI == EPI_GATE_RESID) {
    // 32 columns at a time; the residual of sub-chunk i+1 is requested before
    // sub-chunk i is processed, the first one before the accumulator is even
    // complete.
    constexpr int NSUB = COLS_PER_WARP / 32;
    const GemmEpilogue& e = g.epi;
    const bool valid = m < g.M;
    const int mm = valid ? m : 0;
    const int b = mm / e.rows_in;
    float* out_row = static_cast<float*>(e.out) + static_cast<long>(mm) * e.ldo;
    const float* res_row = e.resid + static_cast<long>(mm) * e.ldo;
    const float* gate_row = e.gate + static_cast<long>(b) * e.gate_stride;
    const int nw = n0 + half * COLS_PER_WARP;
    float4 rr[8], rn[8];
    if (valid) load_resid32(res_row + nw, nw, g.N, rr);
    if (!mbar_wait(tfull_bar, phase, wc, DEV_TIMEOUT_TMEM_FULL)) return false;
    tc_fence_after_sync();
#pragma unroll
    for (int sub = 0; sub < NSUB; ++sub) {
      const int n_base = nw + sub * 32;
      if (sub + 1 < NSUB && valid) load_resid32(res_row + n_base + 32, n_base + 32, g.N, rn);
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_row + half * COLS_PER_WARP + sub * 32, r);
      tmem_wait_ld();
      if (valid && n_base < g.N) epilogue_gate32(r, rr, out_row, gate_row, n_base, g);
      if (sub + 1 < NSUB) {
#pragma unroll
        for (int i = 0; i < 8; ++i) rr[i] = rn[i];
      }
    }
  } else {
    if (!mbar_wait(tfull_bar, phase, wc, DEV_TIMEOUT_TMEM_FULL)) return false;
    tc_fence_after_sync();
    constexpr int CHUNKS = COLS_PER_WARP >= 64 ? COLS_PER_WARP / 64 : 1;
    const bool active = COLS_PER_WARP >= 64 || half == 0;  // BN = 64: one chunk, first half only
    const int c_first = COLS_PER_WARP >= 64 ? half * CHUNKS : 0;
#pragma unroll 1
    for (int ci = 0; ci < CHUNKS; ++ci) {
      const int c = c_first + ci;
      const int n_base = n0 + c * 64;
      if (!active || n_base >= g.N) break;  // warp-uniform
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(t_row + c * 64, r0);
      tmem_ld_32x32b_x32(t_row + c * 64 + 32, r1);
      tmem_wait_ld();
      float v[64];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        v[j] = __uint_as_float(r0[j]);
        v[32 + j] = __uint_as_float(r1[j]);
      }
      if (m < g.M) epilogue_64<EPI, OUT_F32>(v, m, n_base, g);
    }
  }
  return true;
}

}  // namespace gemm_detail
}  // namespace sd3

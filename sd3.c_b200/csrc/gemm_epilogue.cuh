// Fused epilogues shared by the tcgen05 GEMM kernels (one-CTA and CTA-pair
// variants): bias / GELU-tanh / gate+residual / per-head QK-RMSNorm with token
// re-mapping / position-table add / unpatchify, applied to accumulator rows read
// from TMEM (one output row per thread).
//
// Two things keep these epilogues off the critical path: every per-column
// parameter a chunk needs (bias, gate, residual) is requested in one batch
// BEFORE the accumulator load is waited for, so one memory latency is exposed
// per chunk instead of one per 8 columns; and rows are written with 32-byte
// stores (a full sector per thread) whenever the output is 32-byte aligned.
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
  int wide_store;    // output rows are 32-byte aligned at every 16-column (bf16) / 8-column (f32) group
  int tma_store;     // CTA-pair kernel: bf16 output leaves through shared memory and a TMA store
  int* status;
};

__device__ __forceinline__ float gelu_tanh_f(float x) {
  // 0.5 x (1 + tanh(u)),  u = sqrt(2/pi) (x + 0.044715 x^3); one MUFU op per element
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}

__device__ __forceinline__ void st_global_32B(void* p, uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t a4, uint32_t a5, uint32_t a6,
                                              uint32_t a7) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a0),
               "r"(a1), "r"(a2), "r"(a3), "r"(a4), "r"(a5), "r"(a6), "r"(a7)
               : "memory");
}

// 16 consecutive output values of one row
template <bool OUT_F32>
__device__ __forceinline__ void store16(void* out, long idx, const float* o, bool wide) {
  if constexpr (OUT_F32) {
    float* p = static_cast<float*>(out) + idx;
    if (wide) {
      st_global_32B(p, __float_as_uint(o[0]), __float_as_uint(o[1]), __float_as_uint(o[2]),
                    __float_as_uint(o[3]), __float_as_uint(o[4]), __float_as_uint(o[5]),
                    __float_as_uint(o[6]), __float_as_uint(o[7]));
      st_global_32B(p + 8, __float_as_uint(o[8]), __float_as_uint(o[9]), __float_as_uint(o[10]),
                    __float_as_uint(o[11]), __float_as_uint(o[12]), __float_as_uint(o[13]),
                    __float_as_uint(o[14]), __float_as_uint(o[15]));
    } else {
      float4* q = reinterpret_cast<float4*>(p);
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
    }
  } else {
    bf16* p = static_cast<bf16*>(out) + idx;
    uint32_t u[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) u[i] = pack_bf16x2(o[2 * i], o[2 * i + 1]);
    if (wide) {
      st_global_32B(p, u[0], u[1], u[2], u[3], u[4], u[5], u[6], u[7]);
    } else {
      uint4* q = reinterpret_cast<uint4*>(p);
      q[0] = make_uint4(u[0], u[1], u[2], u[3]);
      q[1] = make_uint4(u[4], u[5], u[6], u[7]);
    }
  }
}

// 8 consecutive output values (16-byte stores); used for ragged N
template <bool OUT_F32>
__device__ __forceinline__ void store8(void* out, long idx, const float* o) {
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

// `count` groups of 4 floats starting at p into dst (zeros past column N)
template <int GROUPS>
__device__ __forceinline__ void load_f4_batch(const float* p, int n_base, int N, float (&dst)[GROUPS * 4]) {
#pragma unroll
  for (int i = 0; i < GROUPS; ++i) {
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p != nullptr && n_base + i * 4 < N) t = __ldg(reinterpret_cast<const float4*>(p + n_base) + i);
    dst[4 * i] = t.x; dst[4 * i + 1] = t.y; dst[4 * i + 2] = t.z; dst[4 * i + 3] = t.w;
  }
}

// same, through ordinary (coherent) loads: for data this kernel also writes
template <int GROUPS>
__device__ __forceinline__ void load_f4_batch_rw(const float* p, int n_base, int N, float (&dst)[GROUPS * 4]) {
#pragma unroll
  for (int i = 0; i < GROUPS; ++i) {
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
    if (n_base + i * 4 < N) t = *(reinterpret_cast<const float4*>(p + n_base) + i);
    dst[4 * i] = t.x; dst[4 * i + 1] = t.y; dst[4 * i + 2] = t.z; dst[4 * i + 3] = t.w;
  }
}

struct RowMap {
  int b;      // sample index of the row
  int t_in;   // row within the sample (GEMM side)
  long orow;  // output row
};

__device__ __forceinline__ RowMap map_row(int m, const GemmEpilogue& e) {
  RowMap r;
  r.b = 0;
  r.t_in = m;
  r.orow = m;
  if (e.rows_in > 0) {
    r.b = m / e.rows_in;
    r.t_in = m - r.b * e.rows_in;
    r.orow = static_cast<long>(r.b) * e.rows_out + e.row_off + r.t_in;
  }
  return r;
}

// Epilogue for 64 consecutive accumulator columns of one row; v already holds
// acc * alpha + bias.
// stage / tmO (both or neither): 4 KiB of 1024-byte aligned shared memory private to the
// warp and the tensor map of the bf16 output.  With them the warp's 32 rows x 64 columns
// leave as ONE TMA store (rows in the 128-byte swizzle, 16-byte chunk c of row r at chunk
// c ^ (r & 7)) instead of 128 32-byte register stores; orow0 is the output row of lane 0.
template <int EPI, bool OUT_F32>
__device__ __forceinline__ void epilogue_64(float (&v)[64], const RowMap& rm, int n_base,
                                            const GemmArgs& g, uint8_t* stage = nullptr,
                                            const void* tmO = nullptr, long orow0 = 0) {
  const GemmEpilogue& e = g.epi;
  const int N = g.N;
  if constexpr (EPI == EPI_QKV_NORM) {
    if (e.do_norm && n_base < e.qk_cols) {
      const float* w = (n_base < (e.qk_cols >> 1)) ? e.wq : e.wk;
      float ww[64];
      if (w) {
        load_f4_batch<16>(w, 0, 64, ww);  // in flight while the statistic is formed
      } else {
#pragma unroll
        for (int j = 0; j < 64; ++j) ww[j] = 1.f;
      }
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
      for (int j = 0; j < 64; j += 4) {
        s0 = fmaf(v[j], v[j], s0);
        s1 = fmaf(v[j + 1], v[j + 1], s1);
        s2 = fmaf(v[j + 2], v[j + 2], s2);
        s3 = fmaf(v[j + 3], v[j + 3], s3);
      }
      const float r = rsqrtf(((s0 + s1) + (s2 + s3)) * (1.0f / 64.0f) + e.eps);
#pragma unroll
      for (int j = 0; j < 64; ++j) v[j] = v[j] * r * ww[j];
    }
  }
  if constexpr (EPI == EPI_UNPATCHIFY) {
    // m = (b, r, s) over the patch grid; n = ph * (p * C) + pw * C + c
    const int p = e.up_patch, C = e.up_cin;
    const int s = rm.t_in % e.up_w, r = rm.t_in / e.up_w;
    const long Wpix = static_cast<long>(e.up_w) * p, Hpix = static_cast<long>(e.up_h) * p;
    for (int j = 0; j < 64; ++j) {
      const int n = n_base + j;
      if (n >= N) break;
      const int c = n % C;
      const int pw = (n / C) % p;
      const int ph = n / (C * p);
      const long idx = ((static_cast<long>(rm.b) * C + c) * Hpix + (r * p + ph)) * Wpix + (s * p + pw);
      if constexpr (OUT_F32)
        static_cast<float*>(e.out)[idx] = v[j];
      else
        static_cast<bf16*>(e.out)[idx] = __float2bfloat16(v[j]);
    }
    return;
  }
  if constexpr (EPI == EPI_BIAS_GELU) {
#pragma unroll
    for (int j = 0; j < 64; ++j) v[j] = gelu_tanh_f(v[j]);
  }
  if constexpr (EPI == EPI_ADD_TABLE) {
    float tt[64];
    load_f4_batch<16>(e.table + static_cast<long>(rm.t_in) * N, n_base, N, tt);
#pragma unroll
    for (int j = 0; j < 64; ++j) v[j] += tt[j];
  }
  if constexpr (!OUT_F32 && (EPI == EPI_BIAS || EPI == EPI_BIAS_GELU || EPI == EPI_QKV_NORM)) {
    if (stage != nullptr && !e.out_e4m3) {  // warp-uniform
      const int lane = threadIdx.x & 31;
      if (lane == 0) bulk_wait_group_read0();  // the previous store of this warp has read the buffer
      __syncwarp();
      uint8_t* my_row = stage + lane * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(my_row + ((c ^ (lane & 7)) << 4)) =
            make_uint4(pack_bf16x2(v[8 * c], v[8 * c + 1]), pack_bf16x2(v[8 * c + 2], v[8 * c + 3]),
                       pack_bf16x2(v[8 * c + 4], v[8 * c + 5]), pack_bf16x2(v[8 * c + 6], v[8 * c + 7]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(tmO, stage, n_base, static_cast<int>(orow0));
        bulk_commit_group();
      }
      return;
    }
  }
  long base = rm.orow * e.ldo + n_base;  // element offset of this thread's 64 values
  if constexpr (EPI == EPI_QKV_NORM) {
    if (e.hg_groups > 1) {  // head-group layout: a 64-column chunk is one head and stays contiguous
      const int Eo = e.qk_cols >> 1, Eh = Eo / e.hg_groups;
      const int part = n_base / Eo, e0 = n_base - part * Eo, grp = e0 / Eh;
      base = (static_cast<long>(grp) * e.hg_rows + rm.orow) * (3L * Eh) + part * Eh + (e0 - grp * Eh);
    }
  }
  if constexpr (!OUT_F32 && (EPI == EPI_BIAS || EPI == EPI_BIAS_GELU)) {
    if (e.out_e4m3) {  // 64 bytes per thread; N % 64 == 0 is checked at launch
      uint4* q = reinterpret_cast<uint4*>(static_cast<uint8_t*>(e.out) + base);
#pragma unroll
      for (int gi = 0; gi < 4; ++gi) {
        const float* o = &v[gi * 16];
        q[gi] = make_uint4(pack_e4m3x4(o[0], o[1], o[2], o[3]), pack_e4m3x4(o[4], o[5], o[6], o[7]),
                           pack_e4m3x4(o[8], o[9], o[10], o[11]), pack_e4m3x4(o[12], o[13], o[14], o[15]));
      }
      return;
    }
  }
  if (n_base + 64 <= N) {
#pragma unroll
    for (int gi = 0; gi < 4; ++gi)
      store16<OUT_F32>(e.out, base + gi * 16, &v[gi * 16], g.wide_store != 0);
  } else {
#pragma unroll
    for (int gi = 0; gi < 8; ++gi) {
      const int n = n_base + gi * 8;
      if (n < N) store8<OUT_F32>(e.out, base + gi * 8, &v[gi * 8]);
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
                                           uint64_t* tfull_bar, uint32_t phase, const WaitCtx& wc,
                                           uint8_t* stage = nullptr, const void* tmO = nullptr) {
  constexpr int COLS_PER_WARP = BN / 2;
  const GemmEpilogue& e = g.epi;
  const bool valid = m < g.M;
  const RowMap rm = map_row(valid ? m : 0, e);
  if constexpr (EPI == EPI_GATE_RESID) {
    // 32 columns at a time.  Residual, gate and bias of sub-chunk i+1 are
    // requested before sub-chunk i is processed; those of the first one before
    // the accumulator is even complete.
    constexpr int NSUB = COLS_PER_WARP / 32;
    float* out_row = static_cast<float*>(e.out) + rm.orow * e.ldo;
    const float* res_row = e.resid + rm.orow * e.ldo;
    const float* gate_row = e.gate + static_cast<long>(rm.b) * e.gate_stride;
    const int nw = n0 + half * COLS_PER_WARP;
    float rr[32], gg[32], bb[32];
    if (valid) {
      load_f4_batch_rw<8>(res_row, nw, g.N, rr);
      load_f4_batch<8>(gate_row, nw, g.N, gg);
      load_f4_batch<8>(e.bias, nw, g.N, bb);
    }
    if (!mbar_wait_warp(tfull_bar, phase, wc, DEV_TIMEOUT_TMEM_FULL)) return false;
    tc_fence_after_sync();
#pragma unroll
    for (int sub = 0; sub < NSUB; ++sub) {
      const int n_base = nw + sub * 32;
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_row + half * COLS_PER_WARP + sub * 32, r);
      tmem_wait_ld();
      float o[32];
#pragma unroll
      for (int j = 0; j < 32; ++j)
        o[j] = fmaf(gg[j], fmaf(__uint_as_float(r[j]), e.alpha, bb[j]), rr[j]);
      if (sub + 1 < NSUB && valid) {  // next sub-chunk's parameters, in flight during the stores
        load_f4_batch_rw<8>(res_row, n_base + 32, g.N, rr);
        load_f4_batch<8>(gate_row, n_base + 32, g.N, gg);
        load_f4_batch<8>(e.bias, n_base + 32, g.N, bb);
      }
      if (valid && n_base < g.N) {
        if (n_base + 32 <= g.N) {
          store16<true>(out_row, n_base, &o[0], g.wide_store != 0);
          store16<true>(out_row, n_base + 16, &o[16], g.wide_store != 0);
        } else {
#pragma unroll
          for (int gi = 0; gi < 4; ++gi)
            if (n_base + gi * 8 < g.N) store8<true>(out_row, n_base + gi * 8, &o[gi * 8]);
        }
      }
    }
  } else {
    constexpr int CHUNKS = COLS_PER_WARP >= 64 ? COLS_PER_WARP / 64 : 1;
    const bool active = COLS_PER_WARP >= 64 || half == 0;  // BN = 64: one chunk, first half only
    const int c_first = COLS_PER_WARP >= 64 ? half * CHUNKS : 0;
    float bb[64];
    if (active) load_f4_batch<16>(e.bias, n0 + c_first * 64, g.N, bb);
    if (!mbar_wait_warp(tfull_bar, phase, wc, DEV_TIMEOUT_TMEM_FULL)) return false;
    tc_fence_after_sync();
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
        v[j] = fmaf(__uint_as_float(r0[j]), e.alpha, bb[j]);
        v[32 + j] = fmaf(__uint_as_float(r1[j]), e.alpha, bb[32 + j]);
      }
      if (stage != nullptr) {
        // whole warp valid or not at all (M % 32 == 0 is a condition of this path)
        if (valid) epilogue_64<EPI, OUT_F32>(v, rm, n_base, g, stage, tmO, rm.orow - (threadIdx.x & 31));
      } else if (valid) {
        epilogue_64<EPI, OUT_F32>(v, rm, n_base, g);
      }
      if (ci + 1 < CHUNKS) load_f4_batch<16>(e.bias, n_base + 64, g.N, bb);  // next chunk's bias
    }
  }
  return true;
}


// Gate + residual epilogue of the CTA-pair kernel through a TMA reduction:
// resid += gate * (acc * alpha + bias) with the addition done at L2
// (cp.reduce.async.bulk.tensor ... add.f32).  The SM neither reads the residual
// nor stores it from registers: measured on the register path, those two made
// the out-projection (K = 1536) 1.35x slower than its main loop.  A warp parks
// 32 rows x 32 columns of increments in its 4 KiB of shared memory (128-byte
// rows in the 128-byte swizzle the tensor map expects: 16-byte chunk c of row r
// sits at chunk c ^ (r & 7), which also makes the row-per-thread writes
// conflict-free) and lane 0 issues one reduction for the box.  Requires
// out == resid.  `stage` is 1024-byte aligned.  m_w0: first row of this warp.
template <int BN>
__device__ __forceinline__ bool drain_tile_gate_reduce(uint32_t t_row, int m_w0, int n0, int half,
                                                       const GemmArgs& g, const void* tmR,
                                                       uint64_t* tfull_bar, uint32_t phase,
                                                       const WaitCtx& wc, uint8_t* stage) {
  constexpr int CPW = BN / 2, NSUB = CPW / 32;
  const GemmEpilogue& e = g.epi;
  const int lane = threadIdx.x & 31;
  const int m = m_w0 + lane;
  const int b = (m < g.M ? m : g.M - 1) / e.rows_in;
  const float* gate_row = e.gate + static_cast<long>(b) * e.gate_stride;
  const int nw = n0 + half * CPW;
  float gg[32], bb[32];
  load_f4_batch<8>(gate_row, nw, g.N, gg);
  load_f4_batch<8>(e.bias, nw, g.N, bb);
  if (!mbar_wait_warp(tfull_bar, phase, wc, DEV_TIMEOUT_TMEM_FULL)) return false;
  tc_fence_after_sync();
  uint8_t* my_row = stage + lane * 128;
#pragma unroll
  for (int sub = 0; sub < NSUB; ++sub) {
    const int n_base = nw + sub * 32;
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_row + half * CPW + sub * 32, r);
    tmem_wait_ld();
    float d[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) d[j] = gg[j] * fmaf(__uint_as_float(r[j]), e.alpha, bb[j]);
    if (sub + 1 < NSUB) {
      load_f4_batch<8>(gate_row, n_base + 32, g.N, gg);
      load_f4_batch<8>(e.bias, n_base + 32, g.N, bb);
    }
    // the previous reduction of this warp must have read the buffer
    if (sub > 0 && lane == 0) bulk_wait_group_read0();
    __syncwarp();
#pragma unroll
    for (int c = 0; c < 8; ++c)
      *reinterpret_cast<float4*>(my_row + ((c ^ (lane & 7)) << 4)) =
          make_float4(d[4 * c], d[4 * c + 1], d[4 * c + 2], d[4 * c + 3]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && m_w0 < g.M) {
      tma_reduce_add_2d(tmR, stage, n_base, m_w0);
      bulk_commit_group();
    }
  }
  // the buffer is reused by this warp's next tile
  if (lane == 0) bulk_wait_group_read0();
  __syncwarp();
  return true;
}

}  // namespace gemm_detail
}  // namespace sd3

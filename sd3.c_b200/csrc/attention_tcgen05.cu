// Flash-style attention for head_dim 64 on tcgen05 / TMEM (bf16 operands, fp32
// softmax and accumulation, non-causal, no mask), used for the joint
// context||image attention of every block and the image-only attention of the
// dual blocks.
//
// One CTA owns a 128-query tile of one (sample, head); two CTAs are resident
// per SM.  Warp 0 streams K and V tiles (128 keys per stage) with TMA from the
// packed (B, T, 3E) q|k|v buffer.  The keys are consumed in sub-tiles of 64:
// warp 1 issues S_t = Q K_t^T into one of three 64-column TMEM buffers, two
// sub-tiles ahead of the softmax, so the four softmax warps (one query row per
// thread, TMEM lane == row) normally find their scores ready.  They turn S_t
// into P_t = exp2(S c - m c) in place (bf16, two per TMEM column, over the
// first 32 columns of the same buffer), and warp 1 then issues O += P_t V_t
// with P read from TMEM and V from shared memory in MN-major form.  The T x T
// score matrix never exists in memory.
//
// Two independent CTAs per SM matter: the exponentials are the scarce resource
// at head_dim 64 (one MUFU op per 256 tensor FLOP), each softmax warp runs a
// serial chain (scores ready, TMEM load, row max, exponentials, store,
// hand-off), and two CTAs that drift apart fill each other's gaps.  Variants
// with one larger CTA per SM (two query tiles sharing K/V, 128-key score
// tiles) were measured slower because their two pipelines fall into lockstep.
//
// Replaces mha_cuda (cuda/dit.cu:612-652: two cublasSgemmStridedBatched calls
// around scale_softmax_kernel2, cuda/dit.cu:548-608, over materialised T x T
// matrices) and the layout kernels fused_concat_permute /
// fused_unpermute_split (cuda/dit.cu:475-545): the epilogue writes (B, T, E)
// rows straight into the context and image output buffers.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include <vector>

#include "kernels.h"
#include "ptx.cuh"

namespace sd3 {

int encode_tmap_3d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t d0, uint64_t d1,
                   uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0,
                   uint32_t box1, uint32_t box2);

namespace {

constexpr int AT_BM = 128;      // queries per CTA
constexpr int AT_BN = 128;      // keys per shared-memory stage
constexpr int AT_SUB = 64;      // keys per score sub-tile
constexpr int AT_D = 64;        // head dim
constexpr int AT_STAGES = 2;    // K/V ring depth
constexpr int AT_TILE_BYTES = AT_BN * AT_D * 2;  // 16 KiB
constexpr int AT_SUB_BYTES = AT_SUB * AT_D * 2;  // 8 KiB
constexpr int AT_THREADS = 192;
constexpr int AT_TMEM_COLS = 256;
constexpr int AT_NBUF = 3;      // score buffers of 64 fp32 columns: [0,64), [64,128), [128,192)
constexpr int AT_S_COL = 0;
constexpr int AT_O_COL = 192;   // O: 64 fp32 columns
constexpr int AT_SMEM_BYTES = (1 + 2 * AT_STAGES) * AT_TILE_BYTES + 256 + 1024;

struct AttnArgs {
  int B, T, NH, Tc, E;
  bf16* out_c;
  bf16* out_x;
  float scale_log2e;
  int out_e4m3;  // outputs are e4m3 bytes (operand of an FP8 out-projection) instead of bf16
  int* status;
  long long* probe;  // diagnostics (SD3_ATTN_PROBE=1): 8 counters per CTA, else null
};

// O *= alpha for this thread's query row (64 fp32 columns in TMEM).  Rare (the
// running maximum has to move by more than 2^8), so it is kept out of line: its
// 16 extra live registers and its code would otherwise weigh on the hot loop.
__device__ __noinline__ void rescale_o(uint32_t o_tmem, float alpha) {
  tc_fence_after_sync();
  uint32_t o0[16];
#pragma unroll 1
  for (int part = 0; part < 4; ++part) {
    tmem_ld_32x32b_x16(o_tmem + 16 * part, o0);
    tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < 16; ++i) o0[i] = __float_as_uint(__uint_as_float(o0[i]) * alpha);
    tmem_st_32x32b_x16(o_tmem + 16 * part, o0);
  }
}

// Cycle counters are compiled in only in the PROBE instantiation: even behind a
// runtime flag they cost the softmax loop about a tenth of its throughput.
#define ATX_PROBING (PROBE && a.probe != nullptr)
#define ATX_CLK() ((PROBE && a.probe) ? clock64() : 0ll)

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <bool PROBE>
__global__ void __launch_bounds__(AT_THREADS, 2)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tmQKV, const AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;
  uint8_t* k_smem = smem + AT_TILE_BYTES;
  uint8_t* v_smem = k_smem + AT_STAGES * AT_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + AT_STAGES * AT_TILE_BYTES);
  uint64_t* q_full = bars;                  // 1
  uint64_t* k_full = bars + 1;              // AT_STAGES
  uint64_t* v_full = k_full + AT_STAGES;    // AT_STAGES
  uint64_t* k_empty = v_full + AT_STAGES;   // AT_STAGES
  uint64_t* v_empty = k_empty + AT_STAGES;  // AT_STAGES
  uint64_t* s_full = v_empty + AT_STAGES;   // AT_NBUF (one per score buffer)
  uint64_t* p_ready = s_full + AT_NBUF;     // AT_NBUF
  uint64_t* pv_done = p_ready + AT_NBUF;    // 2: products of even / odd sub-tiles
  uint64_t* o_full = pv_done + 2;           // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * AT_BM;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int T = a.T;
  const int nkv = (T + AT_BN - 1) / AT_BN;    // shared-memory stages to stream
  const int nsub = (T + AT_SUB - 1) / AT_SUB;  // score sub-tiles

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < AT_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < AT_NBUF; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_ready[s], 4);
    }
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
    mbar_init(o_full, 1);
    *s_abort = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQKV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, AT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx wc{s_abort, a.status};

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, AT_TILE_BYTES);
      tma_load_3d(q_smem, &tmQKV, q_full, h * AT_D, q0, b);
    }
    __syncwarp();
    for (int j = 0; j < nkv; ++j) {
      const int st = j % AT_STAGES;
      const uint32_t ph = (j / AT_STAGES) & 1;
      if (!mbar_wait(&k_empty[st], ph ^ 1, wc, DEV_TIMEOUT_ATTN_KV)) break;
      if (lane == 0) {
        mbar_expect_tx(&k_full[st], AT_TILE_BYTES);
        tma_load_3d(k_smem + st * AT_TILE_BYTES, &tmQKV, &k_full[st], a.E + h * AT_D, j * AT_BN, b);
      }
      __syncwarp();
      if (!mbar_wait(&v_empty[st], ph ^ 1, wc, DEV_TIMEOUT_ATTN_KV)) break;
      if (lane == 0) {
        mbar_expect_tx(&v_full[st], AT_TILE_BYTES);
        tma_load_3d(v_smem + st * AT_TILE_BYTES, &tmQKV, &v_full[st], 2 * a.E + h * AT_D,
                    j * AT_BN, b);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    constexpr uint32_t IDESC_S = make_idesc(1, 1, AT_BM, AT_SUB, 0, 0);  // Q K^T, both K-major
    constexpr uint32_t IDESC_O = make_idesc(1, 1, AT_BM, AT_D, 0, 1);    // P V, V is MN-major
    const uint32_t o_tmem = tmem_base + AT_O_COL;
    const uint64_t q_desc = make_smem_desc_sw128(smem_u32(q_smem), 16, 1024);

    // S_u = Q K_u^T for sub-tile u into score buffer (u & 1); releases the K
    // stage after its second half (or after the last sub-tile).
    auto issue_s = [&](int u, bool k_ready) -> bool {
      const int j = u >> 1, st = j % AT_STAGES;
      if ((u & 1) == 0 && !k_ready) {
        if (!mbar_wait(&k_full[st], (j / AT_STAGES) & 1, wc, DEV_TIMEOUT_ATTN_KV)) return false;
      }
      tc_fence_after_sync();
      const uint32_t s_tmem = tmem_base + AT_S_COL + (u % AT_NBUF) * AT_SUB;
      const uint64_t k_desc = make_smem_desc_sw128(
          smem_u32(k_smem + st * AT_TILE_BYTES + (u & 1) * AT_SUB_BYTES), 16, 1024);
#pragma unroll
      for (int k = 0; k < AT_D / 16; ++k)
        mma_f16_ss(s_tmem, q_desc + 2 * k, k_desc + 2 * k, IDESC_S, k != 0);
      mma_commit(&s_full[u % AT_NBUF]);
      if ((u & 1) == 1 || u == nsub - 1) mma_commit(&k_empty[st]);
      return true;
    };

    if (lane == 0) {  // a single thread runs the whole issue loop
      bool ok = mbar_wait(q_full, 0, wc, DEV_TIMEOUT_ATTN_Q);
      if (ok) ok = issue_s(0, false);
      if (ok && nsub > 1) ok = issue_s(1, false);
      long long w_p = 0, w_si = 0, w_pv = 0;
      const long long t_mma0 = ATX_CLK();
      for (int t = 0; t < nsub && ok; ++t) {
        const int j = t >> 1, st = j % AT_STAGES;
        // S_{t+2} does not depend on P_t: its buffer, (t+2) % 3, held P_{t-1},
        // whose product was issued in the previous iteration (the tensor pipe
        // executes in issue order).  Issue it first so the scores stay two
        // sub-tiles ahead of the softmax.
        const long long cs0 = ATX_CLK();
        if (t + 2 < nsub) {
          ok = issue_s(t + 2, false);
          if (!ok) break;
        }
        if (ATX_PROBING) w_si += clock64() - cs0;
        uint32_t v_ready = 1;
        if ((t & 1) == 0) v_ready = mbar_test_wait(&v_full[st], (j / AT_STAGES) & 1);
        // O += P_t V_t
        const long long cp0 = ATX_CLK();
        if (!mbar_wait(&p_ready[t % AT_NBUF], (t / AT_NBUF) & 1, wc, DEV_TIMEOUT_ATTN_P)) break;
        if (ATX_PROBING) w_p += clock64() - cp0;
        if (!v_ready) {
          if (!mbar_wait(&v_full[st], (j / AT_STAGES) & 1, wc, DEV_TIMEOUT_ATTN_KV)) break;
        }
        const long long cv0 = ATX_CLK();
        tc_fence_after_sync();
        const uint32_t p_tmem = tmem_base + AT_S_COL + (t % AT_NBUF) * AT_SUB;
        const uint64_t v_desc = make_smem_desc_sw128(
            smem_u32(v_smem + st * AT_TILE_BYTES + (t & 1) * AT_SUB_BYTES), 1024, 1024);
#pragma unroll
        for (int k = 0; k < AT_SUB / 16; ++k) {
          // 16 keys: 8 TMEM columns of packed bf16 pairs; 16 rows of V (128 B each)
          mma_f16_ts(o_tmem, p_tmem + 8 * k, v_desc + static_cast<uint64_t>((k * 16 * 128) >> 4),
                     IDESC_O, (t | k) != 0);
        }
        mma_commit(&pv_done[t & 1]);
        if ((t & 1) == 1 || t == nsub - 1) mma_commit(&v_empty[st]);
        if (t == nsub - 1) mma_commit(o_full);
        if (ATX_PROBING) w_pv += clock64() - cv0;
      }
      if (ATX_PROBING) {
        const long cta = (static_cast<long>(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        a.probe[cta * 12 + 0] = clock64() - t_mma0;
        a.probe[cta * 12 + 1] = w_p;
        a.probe[cta * 12 + 8] = w_si;
        a.probe[cta * 12 + 9] = w_pv;
      }
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t o_tmem = lane_base + AT_O_COL;
    const float c = a.scale_log2e;
    float m_used = -INFINITY;  // running max (raw score units) the exponentials refer to
    float l = 0.f;
    bool ok = true;
    bool fetched = false;  // scores of sub-tile t already requested from TMEM
    uint32_t r0[32], r1[32];
    long long w_s = 0, w_ld = 0, t_math = 0, w_st = 0, n_miss = 0;
    const long long t_sm0 = ATX_CLK();
    for (int t = 0; t < nsub; ++t) {
      const uint32_t s_tmem = lane_base + AT_S_COL + (t % AT_NBUF) * AT_SUB;
      const long long c0 = ATX_CLK();
      if (!fetched) {
        ++n_miss;
        if (!mbar_wait_warp(&s_full[t % AT_NBUF], (t / AT_NBUF) & 1, wc, DEV_TIMEOUT_ATTN_S)) { ok = false; break; }
        tc_fence_after_sync();
        tmem_ld_32x32b_x32(s_tmem, r0);
        tmem_ld_32x32b_x32(s_tmem + 32, r1);
      }
      const long long c1 = ATX_CLK();
      tmem_wait_ld();
      const long long c2 = ATX_CLK();
      const int kv0 = t * AT_SUB;
      if (kv0 + AT_SUB > T) {  // ragged last sub-tile: keys >= T do not exist
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (kv0 + i >= T) r0[i] = 0xff800000u;  // -inf
          if (kv0 + 32 + i >= T) r1[i] = 0xff800000u;
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        mx0 = max3(mx0, __uint_as_float(r0[i]), __uint_as_float(r0[i + 1]));
        mx1 = max3(mx1, __uint_as_float(r1[i]), __uint_as_float(r1[i + 1]));
      }
      const float mx = fmaxf(mx0, mx1);
      if (t == 0) {
        m_used = mx;
      } else {
        // Rescale O only when the maximum moved by more than 2^8 in the exp2
        // domain; otherwise keep exponentiating against the older maximum.
        const bool need = (mx - m_used) * c > 8.0f;
        if (__any_sync(0xffffffffu, need)) {
          float alpha = 1.0f;
          if (need) {
            alpha = ex2_approx((m_used - mx) * c);
            m_used = mx;
            l *= alpha;
          }
          // P_{t-1} V_{t-1} must have landed in O before O is rescaled; the
          // product of this sub-tile is only issued after p_ready below.
          if (!mbar_wait_warp(&pv_done[(t - 1) & 1], ((t - 1) >> 1) & 1, wc, DEV_TIMEOUT_ATTN_O)) { ok = false; break; }
          rescale_o(o_tmem, alpha);
        }
      }
      const float mc = m_used * c;
      // P = exp2(S c - m c), packed to bf16 pairs over the first 32 columns of the buffer
      float ls0 = 0.f, ls1 = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p0 = ex2_approx(fmaf(__uint_as_float(r0[2 * i]), c, -mc));
        const float p1 = ex2_approx(fmaf(__uint_as_float(r0[2 * i + 1]), c, -mc));
        const float p2 = ex2_approx(fmaf(__uint_as_float(r1[2 * i]), c, -mc));
        const float p3 = ex2_approx(fmaf(__uint_as_float(r1[2 * i + 1]), c, -mc));
        ls0 += p0 + p1;
        ls1 += p2 + p3;
        pk[i] = pack_bf16x2(p0, p1);
        pk[16 + i] = pack_bf16x2(p2, p3);
      }
      tmem_st_32x32b_x32(s_tmem, pk);
      l += ls0 + ls1;
      const long long c3 = ATX_CLK();
      // If the next scores are already there (they normally are: S is issued one
      // sub-tile ahead), request them now so the TMEM load overlaps the hand-off.
      fetched = false;
      if (t + 1 < nsub) {
        uint32_t rdy = 0;
        if (lane == 0) rdy = mbar_test_wait(&s_full[(t + 1) % AT_NBUF], ((t + 1) / AT_NBUF) & 1);
        rdy = __shfl_sync(0xffffffffu, rdy, 0);
        if (rdy) {
          tc_fence_after_sync();
          const uint32_t s_next = lane_base + AT_S_COL + ((t + 1) % AT_NBUF) * AT_SUB;
          tmem_ld_32x32b_x32(s_next, r0);
          tmem_ld_32x32b_x32(s_next + 32, r1);
          fetched = true;
        }
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t % AT_NBUF]);
      if (ATX_PROBING) {
        w_s += c1 - c0;
        w_ld += c2 - c1;
        t_math += c3 - c2;
        w_st += clock64() - c3;
      }
    }
    if (ATX_PROBING && warp == 2 && lane == 0) {
      const long cta = (static_cast<long>(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
      a.probe[cta * 12 + 2] = clock64() - t_sm0;
      a.probe[cta * 12 + 3] = w_s;
      a.probe[cta * 12 + 4] = w_ld;
      a.probe[cta * 12 + 5] = t_math;
      a.probe[cta * 12 + 6] = w_st;
      a.probe[cta * 12 + 7] = n_miss;
    }
    if (ok && mbar_wait_warp(o_full, 0, wc, DEV_TIMEOUT_ATTN_O)) {
      tc_fence_after_sync();
      uint32_t o0[32], o1[32];
      tmem_ld_32x32b_x32(o_tmem, o0);
      tmem_ld_32x32b_x32(o_tmem + 32, o1);
      tmem_wait_ld();
      const int t = q0 + row;
      if (t < T) {
        const float inv = 1.0f / l;
        bf16* dst = nullptr;
        long off = -1;  // element offset of this row's 64 values in out_c / out_x
        if (t < a.Tc) {
          if (a.out_c) off = (static_cast<long>(b) * a.Tc + t) * a.E + h * AT_D;
        } else {
          off = (static_cast<long>(b) * (T - a.Tc) + (t - a.Tc)) * a.E + h * AT_D;
        }
        if (off >= 0 && a.out_e4m3) {
          uint4* d4 = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(t < a.Tc ? a.out_c : a.out_x) + off);
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            uint4 u, w;
            u.x = pack_e4m3x4(__uint_as_float(o0[16 * i + 0]) * inv, __uint_as_float(o0[16 * i + 1]) * inv,
                              __uint_as_float(o0[16 * i + 2]) * inv, __uint_as_float(o0[16 * i + 3]) * inv);
            u.y = pack_e4m3x4(__uint_as_float(o0[16 * i + 4]) * inv, __uint_as_float(o0[16 * i + 5]) * inv,
                              __uint_as_float(o0[16 * i + 6]) * inv, __uint_as_float(o0[16 * i + 7]) * inv);
            u.z = pack_e4m3x4(__uint_as_float(o0[16 * i + 8]) * inv, __uint_as_float(o0[16 * i + 9]) * inv,
                              __uint_as_float(o0[16 * i + 10]) * inv, __uint_as_float(o0[16 * i + 11]) * inv);
            u.w = pack_e4m3x4(__uint_as_float(o0[16 * i + 12]) * inv, __uint_as_float(o0[16 * i + 13]) * inv,
                              __uint_as_float(o0[16 * i + 14]) * inv, __uint_as_float(o0[16 * i + 15]) * inv);
            w.x = pack_e4m3x4(__uint_as_float(o1[16 * i + 0]) * inv, __uint_as_float(o1[16 * i + 1]) * inv,
                              __uint_as_float(o1[16 * i + 2]) * inv, __uint_as_float(o1[16 * i + 3]) * inv);
            w.y = pack_e4m3x4(__uint_as_float(o1[16 * i + 4]) * inv, __uint_as_float(o1[16 * i + 5]) * inv,
                              __uint_as_float(o1[16 * i + 6]) * inv, __uint_as_float(o1[16 * i + 7]) * inv);
            w.z = pack_e4m3x4(__uint_as_float(o1[16 * i + 8]) * inv, __uint_as_float(o1[16 * i + 9]) * inv,
                              __uint_as_float(o1[16 * i + 10]) * inv, __uint_as_float(o1[16 * i + 11]) * inv);
            w.w = pack_e4m3x4(__uint_as_float(o1[16 * i + 12]) * inv, __uint_as_float(o1[16 * i + 13]) * inv,
                              __uint_as_float(o1[16 * i + 14]) * inv, __uint_as_float(o1[16 * i + 15]) * inv);
            d4[i] = u;
            d4[2 + i] = w;
          }
        } else if (off >= 0) {
          dst = (t < a.Tc ? a.out_c : a.out_x) + off;
        }
        if (dst) {
          uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(o0[8 * i + 0]) * inv, __uint_as_float(o0[8 * i + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(o0[8 * i + 2]) * inv, __uint_as_float(o0[8 * i + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(o0[8 * i + 4]) * inv, __uint_as_float(o0[8 * i + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(o0[8 * i + 6]) * inv, __uint_as_float(o0[8 * i + 7]) * inv);
            d4[i] = u;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(o1[8 * i + 0]) * inv, __uint_as_float(o1[8 * i + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(o1[8 * i + 2]) * inv, __uint_as_float(o1[8 * i + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(o1[8 * i + 4]) * inv, __uint_as_float(o1[8 * i + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(o1[8 * i + 6]) * inv, __uint_as_float(o1[8 * i + 7]) * inv);
            d4[4 + i] = u;
          }
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*s_abort) drain_after_abort();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, AT_TMEM_COLS);
  }
}

}  // namespace

int launch_attention_bf16(const bf16* qkv, int B, int T, int NH, int Tc, bf16* out_c, bf16* out_x,
                          float scale, int* dev_status, cudaStream_t stream, int out_e4m3) {
  if (!qkv || !out_x || B <= 0 || T <= 0 || NH <= 0 || Tc < 0 || Tc > T ||
      (reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(out_x) & 15) ||
      (reinterpret_cast<uintptr_t>(out_c) & 15)) {
    set_last_error("attention: invalid argument (B %d T %d NH %d Tc %d)", B, T, NH, Tc);
    return ST_INVALID_ARG;
  }
  if (B > 65535 || NH > 65535) {
    set_last_error("attention: B and NH must each be <= 65535");
    return ST_UNSUPPORTED;
  }
  const int E = NH * AT_D;
  CUtensorMap tm;
  int rc = encode_tmap_3d(&tm, qkv, 2, 3ull * E, (uint64_t)T, (uint64_t)B, 3ull * E * 2,
                          (uint64_t)T * 3ull * E * 2, AT_D, AT_BN, 1);
  if (rc) return rc;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_tcgen05_kernel<true>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_BYTES);
    if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(attention)");
    attr_done[dev] = true;
  }
  AttnArgs a;
  a.B = B; a.T = T; a.NH = NH; a.Tc = Tc; a.E = E;
  a.out_c = out_c; a.out_x = out_x;
  a.scale_log2e = scale * 1.4426950408889634f;
  a.out_e4m3 = out_e4m3;
  a.status = dev_status;
  a.probe = nullptr;
  const dim3 grid((T + AT_BM - 1) / AT_BM, NH, B);
  // Diagnostic: SD3_ATTN_PROBE=1 makes every launch synchronous and prints where
  // the MMA thread and a softmax warp spent their cycles (averages over CTAs).
  static const bool probing = []() {
    const char* v = getenv("SD3_ATTN_PROBE");
    return v && v[0] == '1';
  }();
  const long nctas = static_cast<long>(grid.x) * grid.y * grid.z;
  if (probing && dev_status) {
    if (cudaMalloc(&a.probe, sizeof(long long) * 12 * nctas) != cudaSuccess) a.probe = nullptr;
    if (a.probe) cudaMemset(a.probe, 0, sizeof(long long) * 12 * nctas);
  }
  if (a.probe)
    attention_tcgen05_kernel<true><<<grid, AT_THREADS, AT_SMEM_BYTES, stream>>>(tm, a);
  else
    attention_tcgen05_kernel<false><<<grid, AT_THREADS, AT_SMEM_BYTES, stream>>>(tm, a);
  const int lrc = after_launch("attention_tcgen05_kernel");
  if (a.probe) {
    std::vector<long long> hbuf(12 * nctas);
    cudaStreamSynchronize(stream);
    cudaMemcpy(hbuf.data(), a.probe, hbuf.size() * sizeof(long long), cudaMemcpyDeviceToHost);
    cudaFree(a.probe);
    double sum[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    for (long cidx = 0; cidx < nctas; ++cidx)
      for (int i = 0; i < 12; ++i) sum[i] += static_cast<double>(hbuf[cidx * 12 + i]);
    const int nsub = (T + AT_SUB - 1) / AT_SUB;
    fprintf(stderr,
            "[attention probe] B %d T %d NH %d (%d sub-tiles): per sub-tile: mma thread %.0f clk (waiting P %.0f, issuing S %.0f, issuing PV %.0f); "
            "softmax warp %.0f clk: wait S %.0f, wait TMEM load %.0f, math %.0f, store+handoff %.0f; "
            "scores not prefetched in %.1f%% of sub-tiles\n",
            B, T, NH, nsub, sum[0] / nctas / nsub, sum[1] / nctas / nsub, sum[8] / nctas / nsub,
            sum[9] / nctas / nsub, sum[2] / nctas / nsub,
            sum[3] / nctas / nsub, sum[4] / nctas / nsub, sum[5] / nctas / nsub, sum[6] / nctas / nsub,
            100.0 * sum[7] / nctas / nsub);
  }
  return lrc;
}

}  // namespace sd3

// Flash-style attention for head_dim 64 on tcgen05 / TMEM (bf16 operands, fp32
// softmax and accumulation, non-causal, no mask), used for the joint
// context||image attention of every block and the image-only attention of the
// dual blocks.
//
// One CTA owns a 128-query tile of one (sample, head); two CTAs are resident
// per SM (256 TMEM columns each).  Warp 0 streams K and V tiles of 128 keys with
// TMA from the packed (B, T, 3E) q|k|v buffer; one thread of warp 1 issues the
// MMAs; four softmax warps own one query row per thread (TMEM lane == row).
// Per 128-key tile:
//   S = Q K^T        four MMAs of N = 128 into 128 fp32 TMEM columns,
//   P = exp2(S c - m c)  as packed bf16 pairs into 64 TMEM columns of its own,
//   O += P V         eight MMAs with P read from TMEM and V from shared memory
//                    in MN-major form (no transpose of V anywhere).
// The T x T score matrix never exists in memory.
//
// What the structure is built around (cycle-stamped traces of the issue loops):
//  * A tcgen05.mma or tcgen05.commit holds the issuing thread 50-100 cycles and
//    a satisfied mbarrier test about 60.  With 64-key hand-offs the single issue
//    thread needed ~1700 cycles per 64 keys and was the bottleneck; with one
//    hand-off per 128 keys (12 MMAs, 2 commits, 4 waits) it idles half the time.
//  * An mbarrier hop costs ~140 cycles and the completion of a committed MMA
//    group ~240 cycles after its last cycle of math, so every dependency between
//    the roles is given a tile of slack: a softmax warp pulls the scores of tile
//    j into registers and releases the score buffer at once, so S_{j+1} is
//    issued ~a tile before it is needed; P has columns of its own, so the
//    products of tile j run under the softmax of tile j+1; barrier phases that
//    will be needed later are TESTED early and the test's result consumed when
//    it is needed (the common case never blocks).
//  * The exponentials are the scarce resource at head_dim 64 (one MUFU op per
//    256 tensor FLOP; 16 per clock per SM).  Two softmax warps share an SM
//    sub-partition, and the unit only stays busy if each spends most of its time
//    in exponentials: the softmax is online per 64-key HALF tile, the second
//    half's scores are only loaded once the first half has been packed (150
//    registers, no spills: with all 128 scores live ptxas spilled and the step
//    was 6 % slower), every eighth exponential is evaluated as a polynomial on
//    the FMA pipe, and the multiply-subtract / row-sum pairs use the packed
//    f32x2 instructions.
//  * Three instantiations.  <false, false>: the online softmax above, for any input.
//    <true, *>: the caller gives a bound on |q . k| (SD3.5 normalises q and k per head, so
//    64 max_d |wq_d wk_d| bounds every score whatever the input); when the exp2 argument can
//    not exceed 80 in magnitude, P = 2^(s c) needs no running maximum at all -- no row
//    maximum, vote, branch or rescale -- and three of every eight PAIRS of exponentials go to
//    the FMA pipe as packed polynomials.  <true, true>: the queries were also multiplied by
//    scale log2(e) where they were formed, so a score is its own exp2 argument.  The kernel's
//    time follows its instruction count (no pipe is saturated; two warps per sub-partition
//    are bound by their own dependent-issue latency): -17 % warp instructions, -14 % time.
//
// Replaces mha_cuda (cuda/dit.cu:612-652: two cublasSgemmStridedBatched calls
// around scale_softmax_kernel2, cuda/dit.cu:548-608, over materialised T x T
// matrices) and the layout kernels fused_concat_permute /
// fused_unpermute_split (cuda/dit.cu:475-545): the epilogue writes (B, T, E)
// rows straight into the context and image output buffers.
#include <cuda.h>

#include <cmath>
#include <mutex>

#include "kernels.h"
#include "ptx.cuh"

namespace sd3 {

int device_sm_count();
int encode_tmap_3d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t d0, uint64_t d1,
                   uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0,
                   uint32_t box1, uint32_t box2);

namespace {

constexpr int AT_BM = 128;      // queries per CTA
constexpr int AT_BN = 128;      // keys per stage, per score tile and per hand-off
constexpr int AT_D = 64;        // head dim
constexpr int AT_STAGES = 2;    // K/V ring depth
constexpr int AT_TILE_BYTES = AT_BN * AT_D * 2;  // 16 KiB
constexpr int AT_THREADS = 192;
constexpr int AT_TMEM_COLS = 256;
constexpr int AT_S_COL = 0;     // scores of one 128-key tile: 128 fp32 columns
constexpr int AT_P_COL = 128;   // exp2 of the scores as bf16 pairs: 64 columns (keys 2c, 2c+1 in column c)
constexpr int AT_O_COL = 192;   // O: 64 fp32 columns
constexpr int AT_POLY_EVERY = 4;  // of every 4 pairs of exponentials, one element goes to the FMA pipe
constexpr int AT_POLY_PAIRS = 0x49;  // bounded mode: pairs 0, 3 and 6 of every 8 go to the FMA pipe whole
constexpr float AT_BOUND_MAX = 80.0f;  // largest |score| scale log2(e) the bounded mode accepts
constexpr int AT_SMEM_BYTES = (1 + 2 * AT_STAGES) * AT_TILE_BYTES + 256 + 1024;

struct AttnArgs {
  int B, T, NH, Tc, E;
  bf16* out_c;
  bf16* out_x;
  float scale_log2e;
  int out_e4m3;  // outputs are e4m3 bytes (operand of an FP8 out-projection) instead of bf16
  int* status;
  // Key split (launches with too few CTAs to fill the machine): kv_split CTAs share a query
  // tile, each takes a contiguous range of the key tiles and leaves its unnormalised output
  // row (64 fp32), its running maximum and its row sum in part_o / part_ml; a merge kernel
  // combines them.  kv_split == 1: the CTA normalises and writes the output itself.
  int kv_split;
  float* part_o;   // (B, NH, kv_split, T, 64)
  float* part_ml;  // (B, NH, kv_split, T, 2): maximum (raw score units), row sum
};

// O *= alpha for this thread's query row (64 fp32 columns in TMEM).  Rare (the
// running maximum has to move by more than 2^8), so it is kept out of line.
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
  tmem_wait_st();
}

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

// exp2 on the FMA pipe: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by a
// degree-3 polynomial (relative error ~1e-4, below bf16 resolution), exponent
// added as an integer.  Inputs below -125 give a denormal-sized result.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -125.0f);
  const float t = x + 12582912.0f;  // 1.5 * 2^23: the low mantissa bits now hold round(x)
  const float f = x - (t - 12582912.0f);
  float p = fmaf(f, 0.0558011f, 0.2402265f);
  p = fmaf(p, f, 0.6931472f);
  p = fmaf(p, f, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

// lane 0 arrives; a predicated instruction instead of a divergent branch
__device__ __forceinline__ void mbar_arrive_lane0(uint64_t* bar, int lane) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.eq.s32 p, %1, 0;\n\t"
      "@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t"
      "}\n" ::"r"(smem_u32(bar)), "r"(lane)
      : "memory");
}
// `pre` is the result of an earlier mbar_test_wait of the same phase by every lane
// (one broadcast read, warp-uniform result); blocks only if that test failed.
__device__ __forceinline__ bool mbar_wait_pre(uint32_t pre, uint64_t* bar, uint32_t parity, const WaitCtx& w,
                                              int code) {
  if (pre != 0) return true;
  return mbar_wait_warp(bar, parity, w, code);
}

// keys >= T of a ragged last tile do not exist: their scores become -inf
__device__ __forceinline__ void mask_cols(uint32_t (&r)[32], int key0, int T) {
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (key0 + i >= T) r[i] = 0xff800000u;
}

// maximum of 64 scores: eight independent chains of 3-input maxima, then a tree
__device__ __forceinline__ float max_of2(const uint32_t (&a)[32], const uint32_t (&b)[32]) {
  float m[8];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    m[q] = fmaxf(__uint_as_float(a[8 * q]), __uint_as_float(a[8 * q + 1]));
    m[4 + q] = fmaxf(__uint_as_float(b[8 * q]), __uint_as_float(b[8 * q + 1]));
#pragma unroll
    for (int i = 2; i < 8; i += 2) {
      m[q] = max3(m[q], __uint_as_float(a[8 * q + i]), __uint_as_float(a[8 * q + i + 1]));
      m[4 + q] = max3(m[4 + q], __uint_as_float(b[8 * q + i]), __uint_as_float(b[8 * q + i + 1]));
    }
  }
  return fmaxf(max3(m[0], m[1], m[2]), max3(max3(m[3], m[4], m[5]), m[6], m[7]));
}

// p *= alpha on 32 packed bf16 pairs (rare path: the maximum moved after these were formed)
__device__ __forceinline__ void scale_packed(uint32_t (&r)[32], float alpha) {
  const __nv_bfloat162 a2 = __float2bfloat162_rn(alpha);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&r[i]);
    v = __hmul2(v, a2);
    r[i] = *reinterpret_cast<uint32_t*>(&v);
  }
}

// r[i] = bf16x2(exp2(r[2i] c + nmc), exp2(r[2i+1] c + nmc)) for i < 16, in place (word i
// is written after scores 2i and 2i+1 were read); the exponentials are added into acc.
__device__ __forceinline__ void exp_pack(uint32_t (&r)[32], float c, float nmc, float2& acc) {
  const float2 c2 = make_float2(c, c), n2 = make_float2(nmc, nmc);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), c2, n2);
    float2 p;
    p.x = ex2_approx(x.x);
    p.y = (i % AT_POLY_EVERY == 0) ? ex2_poly(x.y) : ex2_approx(x.y);
    acc = __fadd2_rn(acc, p);
    r[i] = pack_bf16x2(p.x, p.y);
  }
}

// 2^(s c) for a pair of scores on the FMA pipe with packed f32x2 instructions: n = round(s c)
// by the magic-number add, f = s c - n in [-0.5, 0.5], the same degree-3 polynomial, exponent
// added as an integer.  Needs |s c| < 2^22 and a finite result (the bounded mode guarantees
// |s c| <= AT_BOUND_MAX); six packed FMAs and two integer operations per pair.
template <bool UNIT>  // UNIT: c == 1, the scores are exp2 arguments already
__device__ __forceinline__ float2 ex2_poly2(float2 s, float2 c2) {
  const float2 magic = make_float2(12582912.0f, 12582912.0f);
  const float2 t = UNIT ? __fadd2_rn(s, magic) : __ffma2_rn(s, c2, magic);
  const float2 nn = __ffma2_rn(t, make_float2(-1.0f, -1.0f), magic);  // -round(s c)
  const float2 f = UNIT ? __fadd2_rn(s, nn) : __ffma2_rn(s, c2, nn);
  float2 p = __ffma2_rn(f, make_float2(0.0558011f, 0.0558011f), make_float2(0.2402265f, 0.2402265f));
  p = __ffma2_rn(p, f, make_float2(0.6931472f, 0.6931472f));
  p = __ffma2_rn(p, f, make_float2(1.0f, 1.0f));
  p.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  p.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  return p;
}

// Bounded mode: r[i] = bf16x2(2^(r[2i] c), 2^(r[2i+1] c)) for i < 16, in place, no maximum
// subtracted; the exponentials are added into acc.  POLY: three pairs of every eight go to the
// FMA pipe (a microbenchmark of this loop: 7.2 clk per warp-wide element against 8.2 with every
// exponential on the MUFU unit; 2/8 the same, 4/8 slower).  Without POLY a score of -inf (a
// masked key) gives exactly 0.
template <bool POLY, bool UNIT>
__device__ __forceinline__ void exp2_pack(uint32_t (&r)[32], float c, float2& acc) {
  const float2 c2 = make_float2(c, c);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 s = make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
    float2 p;
    if (POLY && ((AT_POLY_PAIRS >> (i % 8)) & 1)) {
      p = ex2_poly2<UNIT>(s, c2);
    } else {
      const float2 x = UNIT ? s : __fmul2_rn(s, c2);
      p.x = ex2_approx(x.x);
      p.y = ex2_approx(x.y);
    }
    acc = __fadd2_rn(acc, p);
    r[i] = pack_bf16x2(p.x, p.y);
  }
}

// BOUNDED: the caller guarantees |q . k| scale log2(e) <= AT_BOUND_MAX for every query and key
// (the engine derives it from the RMSNorm weights of q and k), so 2^(s c) can neither overflow
// nor vanish in fp32 / bf16 and the softmax needs no running maximum: no row maximum, no vote,
// no rescaling of O; P = 2^(s c) and the row sum normalise the output exactly as before
// (softmax is invariant to the subtracted constant).
// UNIT (bounded mode only): the queries were multiplied by scale log2(e) where they were formed
// (the engine folds the factor into the RMSNorm weight of q), so a score is its own exp2
// argument: one packed multiply per pair of scores less (measured: 4 % of the kernel).
template <bool BOUNDED, bool UNIT>
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
  uint64_t* s_full = v_full + AT_STAGES;    // AT_STAGES: scores of the tile in this stage complete (its K is free)
  uint64_t* pv_done = s_full + AT_STAGES;   // AT_STAGES: products of the tile in this stage complete (V, P free; O quiescent)
  uint64_t* s_free = pv_done + AT_STAGES;   // 1: scores pulled into registers (4 arrivals)
  uint64_t* p_ready = s_free + 1;           // 1: P of the tile stored (4 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_ready + 1);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x % a.kv_split;  // which share of the keys
  const int q0 = (blockIdx.x / a.kv_split) * AT_BM;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int T = a.T;
  const int nkv_all = (T + AT_BN - 1) / AT_BN;
  const int jt0 = static_cast<int>(static_cast<long>(nkv_all) * split / a.kv_split);  // first key tile of this CTA
  const int nkv = static_cast<int>(static_cast<long>(nkv_all) * (split + 1) / a.kv_split) - jt0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < AT_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&pv_done[s], 1);
    }
    mbar_init(s_free, 4);
    mbar_init(p_ready, 4);
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
      for (int j = 0; j < nkv; ++j) {
        const int st = j % AT_STAGES;
        const uint32_t prev = ((j / AT_STAGES) + 1) & 1;  // parity of this stage's previous use
        // K of tile j - STAGES is free once its scores are complete
        if (j >= AT_STAGES && !mbar_wait(&s_full[st], prev, wc, DEV_TIMEOUT_ATTN_KV)) break;
        mbar_expect_tx(&k_full[st], AT_TILE_BYTES);
        tma_load_3d(k_smem + st * AT_TILE_BYTES, &tmQKV, &k_full[st], a.E + h * AT_D, (jt0 + j) * AT_BN, b);
        // V of tile j - STAGES is free once its products are complete
        if (j >= AT_STAGES && !mbar_wait(&pv_done[st], prev, wc, DEV_TIMEOUT_ATTN_KV)) break;
        mbar_expect_tx(&v_full[st], AT_TILE_BYTES);
        tma_load_3d(v_smem + st * AT_TILE_BYTES, &tmQKV, &v_full[st], 2 * a.E + h * AT_D, (jt0 + j) * AT_BN, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    constexpr uint32_t IDESC_S = make_idesc(1, 1, AT_BM, AT_BN, 0, 0);  // Q K^T, both K-major, N = 128
    constexpr uint32_t IDESC_O = make_idesc(1, 1, AT_BM, AT_D, 0, 1);   // P V, V is MN-major
    const uint32_t s_tmem = tmem_base + AT_S_COL;
    const uint32_t p_tmem = tmem_base + AT_P_COL;
    const uint32_t o_tmem = tmem_base + AT_O_COL;
    const uint64_t q_desc = make_smem_desc_sw128(smem_u32(q_smem), 16, 1024);
    if (lane == 0) {  // a single thread runs the whole issue loop
      bool ok = mbar_wait(q_full, 0, wc, DEV_TIMEOUT_ATTN_Q);
      // iteration j issues the scores of tile j and the products of tile j - 1
      for (int j = 0; j <= nkv && ok; ++j) {
        if (j < nkv) {
          const int st = j % AT_STAGES;
          // the softmax warps have pulled the scores of tile j - 1 into registers
          if (j >= 1 && !mbar_wait(s_free, (j - 1) & 1, wc, DEV_TIMEOUT_ATTN_S)) break;
          if (!mbar_wait(&k_full[st], (j / AT_STAGES) & 1, wc, DEV_TIMEOUT_ATTN_KV)) break;
          tc_fence_after_sync();
          const uint64_t k_desc = make_smem_desc_sw128(smem_u32(k_smem + st * AT_TILE_BYTES), 16, 1024);
#pragma unroll
          for (int k = 0; k < AT_D / 16; ++k)
            mma_f16_ss(s_tmem, q_desc + 2 * k, k_desc + 2 * k, IDESC_S, k != 0);
          mma_commit(&s_full[st]);
        }
        if (j >= 1) {
          const int jj = j - 1, st = jj % AT_STAGES;
          if (!mbar_wait(&v_full[st], (jj / AT_STAGES) & 1, wc, DEV_TIMEOUT_ATTN_KV)) break;
          if (!mbar_wait(p_ready, jj & 1, wc, DEV_TIMEOUT_ATTN_P)) break;
          tc_fence_after_sync();
          const uint64_t v_desc = make_smem_desc_sw128(smem_u32(v_smem + st * AT_TILE_BYTES), 1024, 1024);
#pragma unroll
          for (int k = 0; k < AT_BN / 16; ++k)  // 16 keys: 8 columns of bf16 pairs, 16 rows of V (128 B each)
            mma_f16_ts(o_tmem, p_tmem + 8 * k, v_desc + static_cast<uint64_t>((k * 16 * 128) >> 4), IDESC_O,
                       (jj != 0 || k != 0));
          mma_commit(&pv_done[st]);
        }
      }
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t s_tmem = lane_base + AT_S_COL;
    const uint32_t p_tmem = lane_base + AT_P_COL;
    const uint32_t o_tmem = lane_base + AT_O_COL;
    const float c = a.scale_log2e;
    float m_used = BOUNDED ? 0.0f : -INFINITY;  // running max (raw score units) the exponentials refer to
    float2 l2 = make_float2(0.f, 0.f);
    bool ok = true;
    uint32_t pre_s = 0;  // early test of s_full for the coming tile
    uint32_t ra[32], rb[32], rc[32], rd[32];  // scores of keys 0..31, 32..63, 64..95, 96..127, then packed P
    for (int j = 0; j < nkv; ++j) {
      const int st = j % AT_STAGES;
      const int kv0 = (jt0 + j) * AT_BN;
      const bool ragged = kv0 + AT_BN > T;
      const int stp = (j + AT_STAGES - 1) % AT_STAGES;               // stage and parity of the
      const uint32_t parp = j >= 1 ? ((j - 1) / AT_STAGES) & 1 : 0;  // previous tile's products
      if (!mbar_wait_pre(pre_s, &s_full[st], (j / AT_STAGES) & 1, wc, DEV_TIMEOUT_ATTN_S)) { ok = false; break; }
      tc_fence_after_sync();
      // Each 64-key half is one step of the online softmax.  O is rescaled only when the
      // maximum moved by more than 2^8 in the exp2 domain; otherwise the exponentials keep
      // referring to the older maximum.  O is quiescent during the whole tile: the products
      // of this tile are issued after the hand-off at its end.
      auto half_step = [&](uint32_t (&r0)[32], uint32_t (&r1)[32], bool second) {
        const float mx = max_of2(r0, r1);
        const bool need = (mx - m_used) * c > 8.0f;  // always true in the very first half (m_used = -inf)
        if (__any_sync(0xffffffffu, need)) {
          float alpha = 1.0f;
          if (need) {
            alpha = ex2_approx((m_used - mx) * c);
            m_used = mx;
            l2.x *= alpha;
            l2.y *= alpha;
          }
          if (j >= 1 && ok) {
            ok = mbar_wait_warp(&pv_done[stp], parp, wc, DEV_TIMEOUT_ATTN_O);
            if (ok) rescale_o(o_tmem, alpha);
          }
          if (second) {  // the first half of P was formed against the older maximum
            scale_packed(ra, alpha);
            scale_packed(rb, alpha);
          }
        }
        const float nmc = -m_used * c;
        exp_pack(r0, c, nmc, l2);
        exp_pack(r1, c, nmc, l2);
      };
      tmem_ld_32x32b_x32(s_tmem, ra);
      tmem_ld_32x32b_x32(s_tmem + 32, rb);
      tmem_wait_ld();
      if (ragged) { mask_cols(ra, kv0, T); mask_cols(rb, kv0 + 32, T); }
      if (BOUNDED) {
        if (ragged) { exp2_pack<false, UNIT>(ra, c, l2); exp2_pack<false, UNIT>(rb, c, l2); }
        else { exp2_pack<true, UNIT>(ra, c, l2); exp2_pack<true, UNIT>(rb, c, l2); }
      } else {
        half_step(ra, rb, false);
      }
      // the second half is only loaded now: with all 128 scores live the kernel spills
      tmem_ld_32x32b_x32(s_tmem + 64, rc);
      tmem_ld_32x32b_x32(s_tmem + 96, rd);
      tmem_wait_ld();
      __syncwarp();
      mbar_arrive_lane0(s_free, lane);  // the score buffer can take the next tile
      if (ragged) { mask_cols(rc, kv0 + 64, T); mask_cols(rd, kv0 + 96, T); }
      uint32_t pre_pv = 1;
      if (j >= 1) pre_pv = mbar_test_wait(&pv_done[stp], parp);
      if (BOUNDED) {
        if (ragged) { exp2_pack<false, UNIT>(rc, c, l2); exp2_pack<false, UNIT>(rd, c, l2); }
        else { exp2_pack<true, UNIT>(rc, c, l2); exp2_pack<true, UNIT>(rd, c, l2); }
      } else {
        half_step(rc, rd, true);
      }
      // P is free once the products of the previous tile are complete (tested half a tile ago)
      if (j >= 1 && ok) ok = mbar_wait_pre(pre_pv, &pv_done[stp], parp, wc, DEV_TIMEOUT_ATTN_O);
      if (!ok) break;
      tmem_st_32x32b_x16(p_tmem, reinterpret_cast<uint32_t(&)[16]>(ra));
      tmem_st_32x32b_x16(p_tmem + 16, reinterpret_cast<uint32_t(&)[16]>(rb));
      tmem_st_32x32b_x16(p_tmem + 32, reinterpret_cast<uint32_t(&)[16]>(rc));
      tmem_st_32x32b_x16(p_tmem + 48, reinterpret_cast<uint32_t(&)[16]>(rd));
      pre_s = 0;
      if (j + 1 < nkv) pre_s = mbar_test_wait(&s_full[(j + 1) % AT_STAGES], ((j + 1) / AT_STAGES) & 1);
      tmem_wait_st();
      __syncwarp();
      mbar_arrive_lane0(p_ready, lane);
    }
    const float l = l2.x + l2.y;
    if (ok && mbar_wait_warp(&pv_done[(nkv - 1) % AT_STAGES], ((nkv - 1) / AT_STAGES) & 1, wc, DEV_TIMEOUT_ATTN_O)) {
      tc_fence_after_sync();
      uint32_t o0[32], o1[32];
      tmem_ld_32x32b_x32(o_tmem, o0);
      tmem_ld_32x32b_x32(o_tmem + 32, o1);
      tmem_wait_ld();
      const int t = q0 + row;
      if (t < T && a.kv_split > 1) {
        // partial result of this share of the keys; the merge kernel finishes the row
        const long prow = ((static_cast<long>(b) * a.NH + h) * a.kv_split + split) * T + t;
        float4* po = reinterpret_cast<float4*>(a.part_o + prow * AT_D);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          po[i] = make_float4(__uint_as_float(o0[4 * i]), __uint_as_float(o0[4 * i + 1]),
                              __uint_as_float(o0[4 * i + 2]), __uint_as_float(o0[4 * i + 3]));
          po[8 + i] = make_float4(__uint_as_float(o1[4 * i]), __uint_as_float(o1[4 * i + 1]),
                                  __uint_as_float(o1[4 * i + 2]), __uint_as_float(o1[4 * i + 3]));
        }
        *reinterpret_cast<float2*>(a.part_ml + prow * 2) = make_float2(m_used, l);
      } else if (t < T) {
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


// Combines the kv_split partial results of every query row: with m = max_s m_s and
// w_s = 2^((m_s - m) c), out = sum_s w_s O_s / sum_s w_s l_s.  One warp per (sample, head,
// token) row, two output columns per lane; rows go to the context / image outputs like in
// the attention kernel's own epilogue.
__global__ void __launch_bounds__(256) attention_merge_kernel(const AttnArgs a) {
  const long row = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long rows = static_cast<long>(a.B) * a.NH * a.T;
  if (row >= rows) return;
  const int t = static_cast<int>(row % a.T);
  const int h = static_cast<int>((row / a.T) % a.NH);
  const int b = static_cast<int>(row / (static_cast<long>(a.T) * a.NH));
  const long p0 = (static_cast<long>(b) * a.NH + h) * a.kv_split * a.T + t;  // split 0; splits are T rows apart
  float m = -INFINITY;
  for (int s = 0; s < a.kv_split; ++s) m = fmaxf(m, a.part_ml[(p0 + static_cast<long>(s) * a.T) * 2]);
  float2 acc = make_float2(0.f, 0.f);
  float l = 0.f;
  for (int s = 0; s < a.kv_split; ++s) {
    const long pr = p0 + static_cast<long>(s) * a.T;
    const float2 ml = *reinterpret_cast<const float2*>(a.part_ml + pr * 2);
    const float w = ex2_approx((ml.x - m) * a.scale_log2e);
    const float2 o = *reinterpret_cast<const float2*>(a.part_o + pr * AT_D + 2 * lane);
    acc.x = fmaf(w, o.x, acc.x);
    acc.y = fmaf(w, o.y, acc.y);
    l = fmaf(w, ml.y, l);
  }
  const float inv = 1.0f / l;
  long off = -1;
  if (t < a.Tc) {
    if (a.out_c) off = (static_cast<long>(b) * a.Tc + t) * a.E + h * AT_D;
  } else {
    off = (static_cast<long>(b) * (a.T - a.Tc) + (t - a.Tc)) * a.E + h * AT_D;
  }
  if (off < 0) return;
  void* base = t < a.Tc ? static_cast<void*>(a.out_c) : static_cast<void*>(a.out_x);
  if (a.out_e4m3)
    reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(base) + off)[lane] = pack_e4m3x2(acc.x * inv, acc.y * inv);
  else
    reinterpret_cast<uint32_t*>(static_cast<bf16*>(base) + off)[lane] = pack_bf16x2(acc.x * inv, acc.y * inv);
}

// Key split for a launch of `ctas` CTAs: the factor (1..4) that fills the last wave best,
// the split's merge pass discounted by 4 %, each share at least eight key tiles long.
// Only launches of less than 1.4 waves are split: measured at T = 16717, a launch of 1.33
// waves (3 heads) gains 9 % from a split, one of 2.66 waves (6 heads) loses 1 % and one of
// 5.3 waves loses 10 % -- the CTAs of a part-filled last wave have their SM to themselves and
// run faster, so wave arithmetic overstates what a split can recover.
int choose_kv_split(long ctas, int nkv) {
  const long slots = 2L * device_sm_count();
  if (ctas * 10 >= slots * 14) return 1;
  auto fill = [&](long n) { return static_cast<double>(n) / static_cast<double>(((n + slots - 1) / slots) * slots); };
  int best = 1;
  double best_fill = fill(ctas);
  for (int sp = 2; sp <= 4; ++sp) {
    if (nkv / sp < 8) break;
    const double f = 0.96 * fill(ctas * sp);
    if (f > best_fill + 0.02) { best = sp; best_fill = f; }
  }
  return best;
}

}  // namespace

size_t attention_scratch_bytes(int B, int T, int NH) {
  // what the key split chosen for this shape needs: partial outputs and (maximum, row sum) pairs
  if (B <= 0 || T <= 0 || NH <= 0) return 0;
  const int qtiles = (T + AT_BM - 1) / AT_BM, nkv = (T + AT_BN - 1) / AT_BN;
  const int sp = choose_kv_split(static_cast<long>(qtiles) * NH * B, nkv);
  return sp > 1 ? static_cast<size_t>(B) * NH * sp * T * (AT_D + 2) * sizeof(float) : 0;
}

// score_bound: an upper bound on |q . k| over every query and key of the launch, or 0 when none
// is known.  With 0 < score_bound * scale * log2(e) <= 80 the softmax runs without a running
// maximum (same result, about 12 % faster); any other value selects the online softmax.
// scale == 0: the queries already carry the factor scale * log2(e), the scores are used as exp2
// arguments directly (and score_bound is a bound on those).
int launch_attention_bf16(const bf16* qkv, int B, int T, int NH, int Tc, bf16* out_c, bf16* out_x,
                          float scale, int* dev_status, cudaStream_t stream, int out_e4m3, void* scratch,
                          size_t scratch_bytes, float score_bound) {
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
  static std::mutex attr_mutex;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64) {
    std::lock_guard<std::mutex> lock(attr_mutex);
    if (!attr_done[dev]) {
      cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<false, false>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_BYTES);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(attention_tcgen05_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 AT_SMEM_BYTES);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(attention_tcgen05_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 AT_SMEM_BYTES);
      if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(attention)");
      attr_done[dev] = true;
    }
  }
  AttnArgs a;
  a.B = B; a.T = T; a.NH = NH; a.Tc = Tc; a.E = E;
  a.out_c = out_c; a.out_x = out_x;
  const bool unit = scale == 0.0f;  // q carries scale log2(e) already
  a.scale_log2e = unit ? 1.0f : scale * 1.4426950408889634f;
  a.out_e4m3 = out_e4m3;
  a.status = dev_status;
  const int qtiles = (T + AT_BM - 1) / AT_BM, nkv = (T + AT_BN - 1) / AT_BN;
  a.kv_split = 1;
  a.part_o = nullptr;
  a.part_ml = nullptr;
  if (scratch && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0) {
    const int sp = choose_kv_split(static_cast<long>(qtiles) * NH * B, nkv);
    const size_t rows = static_cast<size_t>(B) * NH * sp * T;
    if (sp > 1 && rows * (AT_D + 2) * sizeof(float) <= scratch_bytes && static_cast<long>(qtiles) * sp <= 0x7fffffffL) {
      a.kv_split = sp;
      a.part_o = static_cast<float*>(scratch);
      a.part_ml = a.part_o + rows * AT_D;
    }
  }
  const dim3 grid(qtiles * a.kv_split, NH, B);
  const float bound_log2 = score_bound * fabsf(a.scale_log2e);
  if (score_bound > 0.0f && bound_log2 <= AT_BOUND_MAX && unit)
    attention_tcgen05_kernel<true, true><<<grid, AT_THREADS, AT_SMEM_BYTES, stream>>>(tm, a);
  else if (score_bound > 0.0f && bound_log2 <= AT_BOUND_MAX)
    attention_tcgen05_kernel<true, false><<<grid, AT_THREADS, AT_SMEM_BYTES, stream>>>(tm, a);
  else
    attention_tcgen05_kernel<false, false><<<grid, AT_THREADS, AT_SMEM_BYTES, stream>>>(tm, a);
  int lrc = after_launch("attention_tcgen05_kernel");
  if (lrc || a.kv_split == 1) return lrc;
  const long warps = static_cast<long>(B) * NH * T;
  attention_merge_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(a);
  return after_launch("attention_merge_kernel");
}

}  // namespace sd3

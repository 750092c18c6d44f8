// CTA-pair variant of the tcgen05 GEMM: two CTAs (a cluster of two on
// neighbouring SMs) cooperate on 256 x 256 (or, for problems of less than half a
// wave of those, 256 x 128) output tiles with
// tcgen05.mma.cta_group::2.  One launch can carry TWO problems of the same
// shape class (same N, K and epilogue: the image-stream GEMM of a block and its
// small context-stream twin); the persistent tile loop runs the first problem's
// tiles and then the second's, so the small one rides in the tail of the large
// one instead of being a launch of its own that fills less than a wave.
//
//   acc[m, n] = sum_k A[m, k] * W[n, k]        A: (M, K) K-major, W: (N, K) K-major
//
// Per 64-wide K block each CTA loads only its own 128 rows of A and its own
// 128-row half of the W tile (32 KiB instead of the 48 KiB a lone CTA needs
// for a 128 x 256 tile); the tensor cores of both SMs read the two W halves
// from both shared memories.  That cuts the L2 -> shared-memory traffic per
// FLOP by a third and leaves room for a six-stage ring.  The even CTA of the
// pair issues all MMAs, from TWO threads that take the ring's slots in turn: a
// tcgen05.mma holds its issuing thread for about as long as it runs, so with one
// thread the barrier test, the commit and the descriptor arithmetic of every slot
// were idle time of the tensor pipe; now they run under the other thread's MMAs
// (a turn counter in shared memory, bracketed by tcgen05 fences, keeps the MMAs
// in K order).  Completion is signalled to both CTAs with
// tcgen05.commit ... multicast::cluster.  Each CTA keeps the accumulator rows
// of its own half of M in its own TMEM (two buffers of 256 columns) and drains
// them through the same fused epilogues as the one-CTA kernel.
//
// Loads are plain tiled TMA (cta_group::2 form so the peer's transaction bytes
// can be credited to the leader's barrier); nothing here is a multicast load.
#include <cuda.h>
#include <mutex>

#include "gemm_epilogue.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace sd3 {

int encode_tmap_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner,
                   uint64_t outer, uint64_t ld_bytes, uint32_t box_inner, uint32_t box_outer);
int device_sm_count();

namespace {

using namespace gemm_detail;

constexpr int P_BM = 128;            // rows of A per CTA (256 per pair)
constexpr int P_KBYTES = 128;        // bytes of K per stage row (64 bf16)
constexpr int P_A_BYTES = P_BM * P_KBYTES;
// PBN = output columns per pair tile (256 or 128); each CTA loads PBN / 2 rows of W
__host__ __device__ constexpr int pair_b_bytes(int pbn) { return (pbn / 2) * P_KBYTES; }
__host__ __device__ constexpr int pair_stage_bytes(int pbn) { return P_A_BYTES + pair_b_bytes(pbn); }  // 32 / 24 KiB
// The epilogues that leave through shared memory (TMA reduction or TMA store) get 4 KiB per
// epilogue warp.
constexpr int P_RED_BYTES = 4096;
__host__ __device__ constexpr bool pair_stages_out(int epi, bool out_f32) {
  return epi == EPI_GATE_RESID || (!out_f32 && (epi == EPI_BIAS || epi == EPI_BIAS_GELU || epi == EPI_QKV_NORM));
}
// Six stages of 32 KiB (eight of 24 KiB), handed over in SLOTS of two (one full/empty barrier
// pair, one barrier test and one tcgen05.commit per slot instead of per stage: the issuing
// thread spent ~100 of every 680 cycles of a stage on those two).
__host__ __device__ constexpr int pair_stages(int pbn) { return pbn == 256 ? 6 : 8; }
__host__ __device__ constexpr int pair_red_bytes(int epi, bool out_f32) {
  return pair_stages_out(epi, out_f32) ? EPI_WARPS * P_RED_BYTES : 0;
}
constexpr int P_THREADS = 64 + 32 * EPI_WARPS + 32;  // + a second MMA-issuing warp
constexpr int P_MMA2_WARP = 2 + EPI_WARPS;
__host__ __device__ constexpr int pair_smem_bytes(int epi, bool out_f32, int pbn) {
  return pair_stages(pbn) * pair_stage_bytes(pbn) + pair_red_bytes(epi, out_f32) + 256 + 1024;
}

// One problem of a (possibly grouped) launch
struct PairProblem {
  CUtensorMap tmA, tmW, tmR;  // tmR: fp32 residual (gate + residual) or bf16 output (TMA store)
  GemmArgs g;
};

template <int EPI, bool OUT_F32, bool FP8, int PBN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_pair_tcgen05_kernel(const __grid_constant__ PairProblem p0, const __grid_constant__ PairProblem p1,
                         const int tiles0, const int tiles1) {
  // M = 256 across the pair; operands bf16, or e4m3 (128 K-elements per 128-byte stage row,
  // 32 per instruction: the byte arithmetic of the stages is the same)
  constexpr uint32_t IDESC = FP8 ? make_idesc(0, 0, 2 * P_BM, PBN, 0, 0) : make_idesc(1, 1, 2 * P_BM, PBN, 0, 0);
  constexpr int P_BN_HALF = PBN / 2;
  constexpr int P_STAGE_BYTES = pair_stage_bytes(PBN);
  constexpr int P_TMEM_COLS = 2 * PBN;  // two accumulators

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int P_STAGES = pair_stages(PBN);
  uint8_t* red_smem = smem + P_STAGES * P_STAGE_BYTES;  // 1024-byte aligned: stages are 32 / 24 KiB each
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES + pair_red_bytes(EPI, OUT_F32));
  uint64_t* empty_bar = full_bar + P_STAGES;
  uint64_t* tfull_bar = empty_bar + P_STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);
  volatile uint32_t* s_issued = reinterpret_cast<volatile uint32_t*>(s_abort + 1);  // slots whose MMAs have been issued

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);   // leader's expect_tx arrival; bytes of both CTAs
      mbar_init(&empty_bar[s], 1);  // one multicast commit per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 2 * EPI_WARPS);  // epilogue warps of both CTAs (leader's copy is used)
    }
    *s_abort = 0;
    *s_issued = 0;
    fence_barrier_init();
    prefetch_tmap(&p0.tmA);
    prefetch_tmap(&p0.tmW);
    if (tiles1 > 0) {
      prefetch_tmap(&p1.tmA);
      prefetch_tmap(&p1.tmW);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, P_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote signal
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx wc{s_abort, p0.g.status};

  const int num_tiles = tiles0 + tiles1;  // tiles of 256 x PBN: the first problem's, then the second's
  constexpr int NSLOT = P_STAGES / 2;     // slots of two stages
  const int KB = p0.g.k_blocks;        // the same K for both problems
  const int KS = (KB + 1) / 2;         // slots per tile (the last may hold one stage)

  if (warp == 0 && lane == 0) {
    // ------------------------------ TMA producer (both CTAs, one thread) ------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const bool second = tile >= tiles0;
      const PairProblem& pp = second ? p1 : p0;
      const int lt = second ? tile - tiles0 : tile;
      const int m0 = (lt / pp.g.tiles_n) * (2 * P_BM) + static_cast<int>(rank) * P_BM;
      const int n0 = (lt % pp.g.tiles_n) * PBN + static_cast<int>(rank) * P_BN_HALF;
      for (int ks = 0; ks < KS; ++ks) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, wc, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
        {
          const int nk = KB - 2 * ks < 2 ? KB - 2 * ks : 2;  // stages of this slot that carry data
          // all bytes of the slot (both CTAs) are credited to the leader's barrier
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], nk * 2 * P_STAGE_BYTES);
          constexpr int KEL = FP8 ? P_KBYTES : P_KBYTES / 2;  // K elements per stage
          for (int hs = 0; hs < nk; ++hs) {
            uint8_t* sa = smem + (2 * stage + hs) * P_STAGE_BYTES;
            tma_load_2d_pair(sa, &pp.tmA, bar, (2 * ks + hs) * KEL, m0);
            tma_load_2d_pair(sa + P_A_BYTES, &pp.tmW, bar, (2 * ks + hs) * KEL, n0);
          }
        }
        if (++stage == NSLOT) { stage = 0; phase ^= 1; }
      }
    }
  } else if ((warp == 1 || warp == P_MMA2_WARP) && lane == 0) {
    // ------------------------------ MMA issuers (leader only) -----------------
    // Two threads take the slots in turn: while one issues the eight MMAs of its slot the
    // other waits for the operands of the next one, and the commit and the barrier work of a
    // slot run under the other thread's MMAs.  `s_issued` hands the turn over, so the MMAs
    // reach the tensor pipe in K order.
    if (rank == 0) {
      const uint32_t me = warp == 1 ? 0u : 1u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      uint32_t slot_no = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * PBN);
        for (int ks = 0; ks < KS; ++ks) {
          if ((slot_no & 1u) == me) {
            if (ks == 0 && !mbar_wait(&tempty_bar[acc], acc_phase ^ 1, wc, DEV_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
            if (!mbar_wait(&full_bar[stage], phase, wc, DEV_TIMEOUT_FULL)) { ok = false; break; }
            {  // my turn: every earlier slot has been issued
              const uint64_t t0 = global_timer_ns();
              uint32_t it = 0;
              while (*s_issued != slot_no) {
                if (((++it) & 0x3ffu) == 0) {
                  if (*wc.s_abort) { ok = false; break; }
                  if (global_timer_ns() - t0 > SD3_WAIT_LIMIT_NS) {
                    *wc.s_abort = 1;
                    if (wc.g_status) atomicCAS(wc.g_status, 0, DEV_TIMEOUT_FULL);
                    ok = false;
                    break;
                  }
                }
              }
              if (!ok) break;
            }
            tc_fence_after_sync();
            const int nk = KB - 2 * ks < 2 ? KB - 2 * ks : 2;
            for (int hs = 0; hs < nk; ++hs) {
              const uint32_t a_addr = smem_u32(smem + (2 * stage + hs) * P_STAGE_BYTES);
              const uint64_t a_desc = make_smem_desc_sw128(a_addr, 16, 1024);
              const uint64_t b_desc = make_smem_desc_sw128(a_addr + P_A_BYTES, 16, 1024);
#pragma unroll
              for (int k = 0; k < P_KBYTES / 32; ++k) {
                const uint64_t adv = static_cast<uint64_t>((k * 32) >> 4);
                if constexpr (FP8)
                  mma_f8_ss_pair(d_tmem, a_desc + adv, b_desc + adv, IDESC, (ks | hs | k) != 0);
                else
                  mma_f16_ss_pair(d_tmem, a_desc + adv, b_desc + adv, IDESC, (ks | hs | k) != 0);
              }
            }
            tc_fence_before_sync();
            *s_issued = slot_no + 1;  // the other thread may issue the next slot
            mma_commit_pair(&empty_bar[stage], 3);          // frees the slot in both CTAs
            if (ks == KS - 1) mma_commit_pair(&tfull_bar[acc], 3);  // accumulator ready in both CTAs
          }
          ++slot_no;
          if (++stage == NSLOT) { stage = 0; phase ^= 1; }
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else if (warp >= 2 && warp < 2 + EPI_WARPS) {
    // ------------------------------ epilogue (both CTAs) ----------------------
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      const bool second = tile >= tiles0;
      const PairProblem& pp = second ? p1 : p0;
      const GemmArgs& g = pp.g;
      const int lt = second ? tile - tiles0 : tile;
      const int m0 = (lt / g.tiles_n) * (2 * P_BM) + static_cast<int>(rank) * P_BM;
      const int n0 = (lt % g.tiles_n) * PBN;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(acc * PBN);
      bool drained;
      if constexpr (EPI == EPI_GATE_RESID)
        drained = drain_tile_gate_reduce<PBN>(t_row, m0 + quad * 32, n0, half, g, &pp.tmR, &tfull_bar[acc],
                                              acc_phase, wc, red_smem + (warp - 2) * P_RED_BYTES);
      else
        drained = drain_tile<PBN, EPI, OUT_F32>(
            t_row, m0 + row, n0, half, g, &tfull_bar[acc], acc_phase, wc,
            (pair_stages_out(EPI, OUT_F32) && g.tma_store) ? red_smem + (warp - 2) * P_RED_BYTES : nullptr,
            &pp.tmR);
      if (!drained) break;
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if constexpr (pair_stages_out(EPI, OUT_F32)) {
      if (lane == 0) bulk_wait_group0();  // every reduction / store of this warp has landed
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*s_abort) drain_after_abort();
  cluster_sync_all();  // no remote arrival or multicast commit may target an exited CTA
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, P_TMEM_COLS);
  }
}

template <int EPI, bool OUT_F32, bool FP8, int PBN>
int launch_pair_inst(const PairProblem& p0, const PairProblem& p1, int tiles0, int tiles1, cudaStream_t stream) {
  auto kern = gemm_pair_tcgen05_kernel<EPI, OUT_F32, FP8, PBN>;
  constexpr int SMEM = pair_smem_bytes(EPI, OUT_F32, PBN);
  static std::mutex attr_mutex;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64) {
    std::lock_guard<std::mutex> lock(attr_mutex);
    if (!attr_done[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
      if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(gemm_pair)");
      attr_done[dev] = true;
    }
  }
  const int tiles = tiles0 + tiles1;
  const int max_pairs = device_sm_count() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, P_THREADS, SMEM, stream>>>(p0, p1, tiles0, tiles1);
  return after_launch("gemm_pair_tcgen05_kernel");
}

// the block GEMM epilogues exist for both tile widths, the others for 256 only
template <int EPI, bool OUT_F32, bool FP8>
int launch_pair_width(int pbn, const PairProblem& p0, const PairProblem& p1, int tiles0, int tiles1,
                      cudaStream_t stream) {
  constexpr bool narrow_built = (EPI == EPI_GATE_RESID && OUT_F32) ||
                                (!OUT_F32 && (EPI == EPI_BIAS || EPI == EPI_BIAS_GELU || EPI == EPI_QKV_NORM));
  if constexpr (narrow_built) {
    if (pbn == 128) return launch_pair_inst<EPI, OUT_F32, FP8, 128>(p0, p1, tiles0, tiles1, stream);
  }
  return launch_pair_inst<EPI, OUT_F32, FP8, 256>(p0, p1, tiles0, tiles1, stream);
}

bool narrow_tiles_built(const GemmEpilogue& epi) {
  if (epi.mode == EPI_GATE_RESID) return epi.out_f32 != 0;
  return !epi.out_f32 && (epi.mode == EPI_BIAS || epi.mode == EPI_BIAS_GELU || epi.mode == EPI_QKV_NORM);
}

// Tensor maps and arguments of one problem for pair tiles of width pbn.
int build_problem(PairProblem* pp, const GemmProblem& q, int operand_dtype, int N, int K, int pbn,
                  int* dev_status) {
  const bool fp8 = operand_dtype == OPERAND_E4M3;
  const int eb = fp8 ? 1 : 2, kel = P_KBYTES / eb;  // element bytes, K elements per stage
  const GemmEpilogue& epi = q.epi;
  const int M = q.M;
  GemmArgs& g = pp->g;
  g.M = M; g.N = N; g.K = K;
  g.k_blocks = (K + kel - 1) / kel;
  g.tiles_m = (M + 2 * P_BM - 1) / (2 * P_BM);
  g.tiles_n = N / pbn;
  g.epi = epi;
  g.status = dev_status;
  {
    const long esz = epi.out_f32 ? 4 : 2;
    g.wide_store = (N % 16 == 0) && ((epi.ldo * esz) % 32 == 0) &&
                   ((reinterpret_cast<uintptr_t>(epi.out) & 31) == 0);
  }
  int rc = encode_tmap_2d(&pp->tmA, q.A, eb, (uint64_t)K, (uint64_t)M, (uint64_t)q.lda * eb, kel, P_BM);
  if (rc) return rc;
  rc = encode_tmap_2d(&pp->tmW, q.W, eb, (uint64_t)K, (uint64_t)N, (uint64_t)q.ldw * eb, kel, pbn / 2);
  if (rc) return rc;
  const bool f32 = epi.out_f32 != 0;
  pp->tmR = pp->tmA;  // placeholder for the epilogues that neither reduce nor store through TMA
  if (epi.mode == EPI_GATE_RESID) {
    if (epi.out != epi.resid) {
      set_last_error("gemm_pair: gate/residual epilogue updates the residual in place (out must equal resid)");
      return ST_INVALID_ARG;
    }
    rc = encode_tmap_2d(&pp->tmR, epi.resid, 4, (uint64_t)N, (uint64_t)M, (uint64_t)epi.ldo * 4, 32, 32);
    if (rc) return rc;
  }
  // bf16 outputs leave through a TMA store when every warp's 32 rows are 32 consecutive
  // output rows that all exist
  g.tma_store = 0;
  if (!f32 && !epi.out_e4m3 && M % 32 == 0 && (epi.rows_in == 0 || epi.rows_in % 32 == 0) &&
      (epi.mode == EPI_BIAS || epi.mode == EPI_BIAS_GELU || epi.mode == EPI_QKV_NORM) && epi.hg_groups <= 1 &&
      (epi.ldo * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(epi.out) & 15) == 0) {
    // with a row remap the last sample's rows end at (samples - 1) * rows_out + row_off + rows_in
    const uint64_t extent = epi.rows_in > 0
                                ? (uint64_t)(M / epi.rows_in - 1) * epi.rows_out + epi.row_off + epi.rows_in
                                : (uint64_t)M;
    rc = encode_tmap_2d(&pp->tmR, epi.out, 2, (uint64_t)N, extent, (uint64_t)epi.ldo * 2, 64, 32);
    if (rc) return rc;
    g.tma_store = 1;
  }
  return ST_OK;
}

// 256-wide tiles, except for problems so small that even twice as many 128-wide tiles fit in one
// wave of CTA pairs.  The narrow tile needs 96 bytes of operands per clock per SM at the full MMA
// rate against 64, and its ring slots (48 KiB) are consumed in half the time of the wide tile's
// (64 KiB) while their refill takes as long: it reaches 0.5-0.6 of the MMA rate where the wide
// tile reaches 0.8.  Measured at 4096-4429 rows (1.3-1.5 waves of wide tiles, where wave
// arithmetic favours the narrow ones) the wide tiles are 15-25 % faster (N = 1536, K = 6144: 72
// against 90 us), at 2048 rows 35 %.  Only for problems of a few tiles (at most 1536 rows at N = 1536), where the
// narrow tiles put twice as many SMs to work, do they win, by 5-8 %.
int choose_tile_width(long tiles256, const GemmEpilogue& epi) {
  if (!narrow_tiles_built(epi)) return 256;
  const long pairs = device_sm_count() / 2;
  return (pairs > 0 && 2 * tiles256 <= pairs) ? 128 : 256;
}

}  // namespace

// Whether the CTA-pair kernel covers this problem (N a multiple of 256, enough rows to fill
// pair tiles, an epilogue that is instantiated for the operand type).
bool gemm_pair_supported(int operand_dtype, int M, int N, int K, const GemmEpilogue& epi) {
  (void)K;
  if (N % 256 != 0 || M < 2 * P_BM) return false;
  if (epi.mode == EPI_UNPATCHIFY) return false;
  if (operand_dtype == OPERAND_E4M3) {
    // e4m3 instantiations exist for the epilogues of the block GEMMs
    if (epi.mode == EPI_GATE_RESID) return epi.out_f32 != 0;
    return (epi.mode == EPI_QKV_NORM || epi.mode == EPI_BIAS_GELU || epi.mode == EPI_BIAS) && !epi.out_f32;
  }
  return operand_dtype == OPERAND_BF16;
}

// One or two problems (b may be null) of the same N, K, operand type and epilogue kind.
int launch_gemm_pair(const GemmProblem& a, const GemmProblem* b, int operand_dtype, int N, int K,
                     int* dev_status, cudaStream_t stream) {
  const bool fp8 = operand_dtype == OPERAND_E4M3;
  if (b && (b->epi.mode != a.epi.mode || b->epi.out_f32 != a.epi.out_f32)) {
    set_last_error("gemm_pair: grouped problems need the same epilogue kind");
    return ST_INVALID_ARG;
  }
  const long tiles256 = static_cast<long>((a.M + 255) / 256 + (b ? (b->M + 255) / 256 : 0)) * (N / 256);
  const int pbn = choose_tile_width(tiles256, a.epi);
  PairProblem p0, p1;
  int rc = build_problem(&p0, a, operand_dtype, N, K, pbn, dev_status);
  if (rc) return rc;
  int tiles1 = 0;
  if (b) {
    rc = build_problem(&p1, *b, operand_dtype, N, K, pbn, dev_status);
    if (rc) return rc;
    tiles1 = p1.g.tiles_m * p1.g.tiles_n;
  } else {
    p1 = p0;
  }
  const int tiles0 = p0.g.tiles_m * p0.g.tiles_n;
  const bool f32 = a.epi.out_f32 != 0;
  if (fp8) {
    switch (a.epi.mode) {
      case EPI_BIAS: return launch_pair_width<EPI_BIAS, false, true>(pbn, p0, p1, tiles0, tiles1, stream);
      case EPI_BIAS_GELU: return launch_pair_width<EPI_BIAS_GELU, false, true>(pbn, p0, p1, tiles0, tiles1, stream);
      case EPI_QKV_NORM: return launch_pair_width<EPI_QKV_NORM, false, true>(pbn, p0, p1, tiles0, tiles1, stream);
      case EPI_GATE_RESID: return launch_pair_width<EPI_GATE_RESID, true, true>(pbn, p0, p1, tiles0, tiles1, stream);
      default: break;
    }
    set_last_error("gemm_pair: no e4m3 instantiation for epilogue mode %d", a.epi.mode);
    return ST_UNSUPPORTED;
  }
  switch (a.epi.mode) {
    case EPI_BIAS:
      return f32 ? launch_pair_width<EPI_BIAS, true, false>(pbn, p0, p1, tiles0, tiles1, stream)
                 : launch_pair_width<EPI_BIAS, false, false>(pbn, p0, p1, tiles0, tiles1, stream);
    case EPI_BIAS_GELU:
      return f32 ? launch_pair_width<EPI_BIAS_GELU, true, false>(pbn, p0, p1, tiles0, tiles1, stream)
                 : launch_pair_width<EPI_BIAS_GELU, false, false>(pbn, p0, p1, tiles0, tiles1, stream);
    case EPI_GATE_RESID:
      if (!f32) break;
      return launch_pair_width<EPI_GATE_RESID, true, false>(pbn, p0, p1, tiles0, tiles1, stream);
    case EPI_QKV_NORM:
      return f32 ? launch_pair_width<EPI_QKV_NORM, true, false>(pbn, p0, p1, tiles0, tiles1, stream)
                 : launch_pair_width<EPI_QKV_NORM, false, false>(pbn, p0, p1, tiles0, tiles1, stream);
    case EPI_ADD_TABLE:
      if (!f32) break;
      return launch_pair_width<EPI_ADD_TABLE, true, false>(pbn, p0, p1, tiles0, tiles1, stream);
    default:
      break;
  }
  set_last_error("gemm_pair: unsupported epilogue mode %d / out_f32 %d", a.epi.mode, a.epi.out_f32);
  return ST_UNSUPPORTED;
}

}  // namespace sd3

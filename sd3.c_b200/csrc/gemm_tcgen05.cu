// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   acc[m, n] = sum_k A[m, k] * W[n, k]        A: (M, K) K-major, W: (N, K) K-major
//
// One CTA per SM walks output tiles of 128 x BN (BN = 256/128/64).  Warp 0
// feeds a ring of shared-memory stages with TMA (128-byte swizzle, 64 bf16 or
// 128 e4m3 of K per stage), warp 1 issues tcgen05.mma into one of two TMEM
// accumulators, warps 2-5 drain the other accumulator through the fused
// epilogue (bias / GELU-tanh / gate+residual / per-head QK-RMSNorm with token
// re-mapping / position-table add / unpatchify), so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Replaces the reference's cuBLASLt call (cuda/dit.cu:683-756 launch_linear),
// the SGEMM used for chunked projections (cuda/dit.cu:102-354) and the
// separate kernels the epilogues absorb: rmsnorm_key_query_kernel2
// (cuda/dit.cu:384-471), fused_concat_permute (cuda/dit.cu:475-515),
// gate_multiply_residual_add (cuda/dit.cu:655-680) and the GELU epilogue of
// mlp_cuda (cuda/dit.cu:759-765).
#include <cuda.h>
#include <cudaTypedefs.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "gemm_epilogue.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace sd3 {

namespace {

using namespace gemm_detail;

constexpr int BM = 128;
constexpr int STAGE_K_BYTES = 128;  // bytes of K per smem row == swizzle span
constexpr int A_STAGE_BYTES = BM * STAGE_K_BYTES;
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;  // TMA warp, MMA warp, epilogue warps

template <int BN>
struct GemmCfg {
  static constexpr int B_STAGE_BYTES = BN * STAGE_K_BYTES;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 /*barriers*/ + 1024 /*align*/;
};

template <int BN, int EPI, bool OUT_F32, bool FP8>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                    const GemmArgs g) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ELEMS_PER_STAGE = FP8 ? 128 : 64;  // K elements per stage
  constexpr int MMA_K_BYTES = 32;                  // 16 bf16 or 32 e4m3 per instruction
  constexpr uint32_t IDESC =
      FP8 ? make_idesc(0, 0, BM, BN, 0, 0) : make_idesc(1, 1, BM, BN, 0, 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], EPI_WARPS);
    }
    *s_abort = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx wc{s_abort, g.status};

  const int num_tiles = g.tiles_m * g.tiles_n;
  const int KB = g.k_blocks;

  if (warp == 0 && lane == 0) {
    // ------------------------------ TMA producer (one thread) ------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile / g.tiles_n) * BM;
      const int n0 = (tile % g.tiles_n) * BN;
      for (int kb = 0; kb < KB; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, wc, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
        {
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * ELEMS_PER_STAGE, m0);
          tma_load_2d(sa + A_STAGE_BYTES, &tmW, &full_bar[stage], kb * ELEMS_PER_STAGE, n0);
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------ MMA issuer (one thread) --------------------
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    bool stage_ready = false;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, wc, DEV_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
      for (int kb = 0; kb < KB; ++kb) {
        // readiness of this stage was tested while the previous stage's MMAs
        // were being issued; block only if that early test failed
        if (!stage_ready) {
          if (!mbar_wait(&full_bar[stage], phase, wc, DEV_TIMEOUT_FULL)) { ok = false; break; }
        }
        int ns = stage + 1;
        uint32_t np = phase;
        if (ns == STAGES) { ns = 0; np ^= 1; }
        const uint32_t next_ready = mbar_test_wait(&full_bar[ns], np);
        tc_fence_after_sync();
        {
          const uint32_t a_addr = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
          const uint64_t a_desc = make_smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t b_desc = make_smem_desc_sw128(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < STAGE_K_BYTES / MMA_K_BYTES; ++k) {
            const uint64_t adv = static_cast<uint64_t>((k * MMA_K_BYTES) >> 4);
            if constexpr (FP8)
              mma_f8_ss(d_tmem, a_desc + adv, b_desc + adv, IDESC, (kb | k) != 0);
            else
              mma_f16_ss(d_tmem, a_desc + adv, b_desc + adv, IDESC, (kb | k) != 0);
          }
          mma_commit(&empty_bar[stage]);
          if (kb == KB - 1) mma_commit(&tfull_bar[acc]);
        }
        stage = ns;
        phase = np;
        stage_ready = next_ready != 0;
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  } else if (warp >= 2) {
    // ------------------------------ epilogue ----------------------------------
    // Eight warps: warp w may read TMEM lanes [32 (w % 4), +32); warps 2-5 take
    // the first half of the tile's columns, warps 6-9 the second half.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int m0 = (tile / g.tiles_n) * BM;
      const int n0 = (tile % g.tiles_n) * BN;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(acc * BN);
      if (!drain_tile<BN, EPI, OUT_F32>(t_row, m0 + row, n0, half, g, &tfull_bar[acc], acc_phase, wc))
        break;
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*s_abort) drain_after_abort();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  // resolved once; the function-local static's initialisation is thread-safe
  static const PFN_cuTensorMapEncodeTiled_v12000 fn = []() -> PFN_cuTensorMapEncodeTiled_v12000 {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    return nullptr;
  }();
  return fn;
}

}  // namespace

// 2-D / 3-D tiled tensor maps with 128-byte swizzle (also used by attention).
int encode_tmap_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner,
                   uint64_t outer, uint64_t ld_bytes, uint32_t box_inner, uint32_t box_outer) {
  auto fn = get_encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled entry point not available");
    return ST_CUDA_ERROR;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 4   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled(2d) failed: %d (inner %llu outer %llu ld %llu)", (int)r,
                   (unsigned long long)inner, (unsigned long long)outer,
                   (unsigned long long)ld_bytes);
    return ST_CUDA_ERROR;
  }
  return ST_OK;
}

int encode_tmap_3d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t d0, uint64_t d1,
                   uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0,
                   uint32_t box1, uint32_t box2) {
  auto fn = get_encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled entry point not available");
    return ST_CUDA_ERROR;
  }
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt =
      elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled(3d) failed: %d", (int)r);
    return ST_CUDA_ERROR;
  }
  return ST_OK;
}

int device_sm_count() {
  static std::atomic<int> sms[64];  // zero-initialised; a racing first call computes the same value twice
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  int v = sms[dev].load(std::memory_order_acquire);
  if (v == 0) {
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    if (v <= 0) v = 1;
    sms[dev].store(v, std::memory_order_release);
  }
  return v;
}

namespace {

template <int BN, int EPI, bool OUT_F32, bool FP8>
int launch_inst(const CUtensorMap& tmA, const CUtensorMap& tmW, const GemmArgs& g,
                cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_tcgen05_kernel<BN, EPI, OUT_F32, FP8>;
  static std::mutex attr_mutex;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64) {
    std::lock_guard<std::mutex> lock(attr_mutex);
    if (!attr_done[dev]) {
      cudaError_t e =
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
      if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(gemm)");
      attr_done[dev] = true;
    }
  }
  const int tiles = g.tiles_m * g.tiles_n;
  const int grid = tiles < device_sm_count() ? tiles : device_sm_count();
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmW, g);
  return after_launch("gemm_tcgen05_kernel");
}

template <int BN, bool FP8>
int dispatch_epi(const CUtensorMap& tmA, const CUtensorMap& tmW, const GemmArgs& g,
                 cudaStream_t stream) {
  const bool f32 = g.epi.out_f32 != 0;
  switch (g.epi.mode) {
    case EPI_BIAS:
      return f32 ? launch_inst<BN, EPI_BIAS, true, FP8>(tmA, tmW, g, stream)
                 : launch_inst<BN, EPI_BIAS, false, FP8>(tmA, tmW, g, stream);
    case EPI_BIAS_GELU:
      return f32 ? launch_inst<BN, EPI_BIAS_GELU, true, FP8>(tmA, tmW, g, stream)
                 : launch_inst<BN, EPI_BIAS_GELU, false, FP8>(tmA, tmW, g, stream);
    case EPI_GATE_RESID:
      if (!f32) break;
      return launch_inst<BN, EPI_GATE_RESID, true, FP8>(tmA, tmW, g, stream);
    case EPI_QKV_NORM:
      return f32 ? launch_inst<BN, EPI_QKV_NORM, true, FP8>(tmA, tmW, g, stream)
                 : launch_inst<BN, EPI_QKV_NORM, false, FP8>(tmA, tmW, g, stream);
    case EPI_ADD_TABLE:
      if (!f32) break;
      return launch_inst<BN, EPI_ADD_TABLE, true, FP8>(tmA, tmW, g, stream);
    case EPI_UNPATCHIFY:
      return f32 ? launch_inst<BN, EPI_UNPATCHIFY, true, FP8>(tmA, tmW, g, stream)
                 : launch_inst<BN, EPI_UNPATCHIFY, false, FP8>(tmA, tmW, g, stream);
    default:
      break;
  }
  set_last_error("gemm: unsupported epilogue mode %d / out_f32 %d", g.epi.mode, g.epi.out_f32);
  return ST_UNSUPPORTED;
}

}  // namespace

bool gemm_pair_supported(int operand_dtype, int M, int N, int K, const GemmEpilogue& epi);
int launch_gemm_pair(const GemmProblem& a, const GemmProblem* b, int operand_dtype, int N, int K,
                     int* dev_status, cudaStream_t stream);

namespace {
// argument checks shared by the single and the grouped launch
int validate_gemm(const void* A, long lda, const void* W, long ldw, int operand_dtype, int M, int N, int K,
                  const GemmEpilogue& epi) {
  if (M <= 0 || N <= 0 || K <= 0 || !A || !W || !epi.out) {
    set_last_error("gemm: invalid argument (M %d N %d K %d)", M, N, K);
    return ST_INVALID_ARG;
  }
  const int eb = operand_dtype == OPERAND_E4M3 ? 1 : 2;
  if ((lda * eb) % 16 != 0 || (ldw * eb) % 16 != 0 || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(W) & 15)) {
    set_last_error("gemm: operands must be 16-byte aligned with 16-byte-multiple row pitch");
    return ST_INVALID_ARG;
  }
  if (epi.out_e4m3 && (epi.out_f32 || (epi.mode != EPI_BIAS && epi.mode != EPI_BIAS_GELU) || N % 64 != 0 ||
                       epi.ldo % 16 != 0)) {
    set_last_error("gemm: e4m3 output needs a bias or bias+GELU epilogue, N %% 64 == 0 and ldo %% 16 == 0");
    return ST_INVALID_ARG;
  }
  if (epi.mode != EPI_UNPATCHIFY) {
    const long oa = epi.out_f32 ? 4 : 8;
    if (N % 8 != 0 || epi.ldo % oa != 0 || (reinterpret_cast<uintptr_t>(epi.out) & 15)) {
      set_last_error("gemm: N must be a multiple of 8 and the output 16-byte aligned");
      return ST_INVALID_ARG;
    }
  }
  if (epi.mode == EPI_QKV_NORM && (epi.qk_cols % 128 != 0)) {
    set_last_error("gemm: QKV epilogue needs head_dim 64 (qk_cols multiple of 128)");
    return ST_INVALID_ARG;
  }
  if (epi.mode == EPI_GATE_RESID && (!epi.gate || !epi.resid)) {
    set_last_error("gemm: gate/residual epilogue needs gate and resid pointers");
    return ST_INVALID_ARG;
  }
  if (epi.mode == EPI_GATE_RESID &&
      (epi.rows_in <= 0 || epi.rows_in != epi.rows_out || epi.row_off != 0 || epi.ldo % 4 != 0 ||
       epi.gate_stride % 4 != 0)) {
    set_last_error("gemm: gate/residual epilogue needs rows_in == rows_out > 0 and no row offset");
    return ST_INVALID_ARG;
  }
  if (epi.mode == EPI_ADD_TABLE && (!epi.table || epi.rows_in <= 0)) {
    set_last_error("gemm: table epilogue needs table and rows_in");
    return ST_INVALID_ARG;
  }
  return ST_OK;
}
}  // namespace

int launch_gemm_grouped(const GemmProblem& a, const GemmProblem& b, int operand_dtype, int N, int K,
                        int* dev_status, cudaStream_t stream) {
  int rc = validate_gemm(a.A, a.lda, a.W, a.ldw, operand_dtype, a.M, N, K, a.epi);
  if (rc) return rc;
  rc = validate_gemm(b.A, b.lda, b.W, b.ldw, operand_dtype, b.M, N, K, b.epi);
  if (rc) return rc;
  if (a.epi.mode == b.epi.mode && a.epi.out_f32 == b.epi.out_f32 &&
      gemm_pair_supported(operand_dtype, a.M, N, K, a.epi) && gemm_pair_supported(operand_dtype, b.M, N, K, b.epi))
    return launch_gemm_pair(a, &b, operand_dtype, N, K, dev_status, stream);
  rc = launch_gemm(a.A, a.lda, a.W, a.ldw, operand_dtype, a.M, N, K, a.epi, dev_status, stream);
  if (rc) return rc;
  return launch_gemm(b.A, b.lda, b.W, b.ldw, operand_dtype, b.M, N, K, b.epi, dev_status, stream);
}

int launch_gemm(const void* A, long lda, const void* W, long ldw, int operand_dtype, int M, int N,
                int K, const GemmEpilogue& epi, int* dev_status, cudaStream_t stream) {
  int rcv = validate_gemm(A, lda, W, ldw, operand_dtype, M, N, K, epi);
  if (rcv) return rcv;
  const int eb = operand_dtype == OPERAND_E4M3 ? 1 : 2;
  // Large problems go to the CTA-pair kernel (256-row tiles across two SMs).
  if (gemm_pair_supported(operand_dtype, M, N, K, epi)) {
    GemmProblem q;
    q.A = A; q.lda = lda; q.W = W; q.ldw = ldw; q.M = M; q.epi = epi;
    return launch_gemm_pair(q, nullptr, operand_dtype, N, K, dev_status, stream);
  }

  const int BN = (N >= 256 && N % 256 == 0) ? 256 : (N > 64 ? 128 : 64);
  const int elems_per_stage = STAGE_K_BYTES / eb;

  GemmArgs g;
  g.M = M; g.N = N; g.K = K;
  g.k_blocks = (K + elems_per_stage - 1) / elems_per_stage;
  g.tiles_m = (M + BM - 1) / BM;
  g.tiles_n = (N + BN - 1) / BN;
  g.epi = epi;
  g.status = dev_status;
  {
    const long esz = epi.out_f32 ? 4 : 2;
    g.wide_store = (N % 16 == 0) && ((epi.ldo * esz) % 32 == 0) &&
                   ((reinterpret_cast<uintptr_t>(epi.out) & 31) == 0);
  }

  g.tma_store = 0;  // register stores in the one-CTA kernel
  CUtensorMap tmA, tmW;
  int rc = encode_tmap_2d(&tmA, A, eb, (uint64_t)K, (uint64_t)M, (uint64_t)lda * eb,
                          elems_per_stage, BM);
  if (rc) return rc;
  rc = encode_tmap_2d(&tmW, W, eb, (uint64_t)K, (uint64_t)N, (uint64_t)ldw * eb, elems_per_stage,
                      BN);
  if (rc) return rc;

  const bool fp8 = operand_dtype == OPERAND_E4M3;
  if (BN == 256)
    return fp8 ? dispatch_epi<256, true>(tmA, tmW, g, stream)
               : dispatch_epi<256, false>(tmA, tmW, g, stream);
  if (BN == 128)
    return fp8 ? dispatch_epi<128, true>(tmA, tmW, g, stream)
               : dispatch_epi<128, false>(tmA, tmW, g, stream);
  return fp8 ? dispatch_epi<64, true>(tmA, tmW, g, stream)
             : dispatch_epi<64, false>(tmA, tmW, g, stream);
}

}  // namespace sd3

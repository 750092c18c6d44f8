// sd3_patch_embed_static: the patch-embedding operator for callers that are
// not allowed to allocate device memory.
//
// sd3_patch_embed needs a scratch buffer (the gathered patches, B*h*w rows of
// C*p*p bf16) that the caller has to provide.  Some callers cannot: serving
// loops that must never hit the allocator because cudaMalloc/cudaFree
// synchronise the whole device, hosts that hand the library a fixed memory
// budget up front, and code that runs where the allocator must not be entered
// at all.  For them the scratch lives in a
// fixed array inside the library image.  Every GPU that loads the library
// carries that array until the process exits.
//
// Rules that follow from sharing one array:
//  * at most SD3_STATIC_PATCH_ELEMS patch elements per call, larger problems
//    are rejected with SD3_ERR_UNSUPPORTED;
//  * the array keeps whatever the previous call left in it.  Nothing here needs
//    zero-initialised scratch: the gather kernel overwrites every element the
//    GEMM reads before the GEMM runs (same stream);
//  * two calls whose GPU work overlaps (different streams, or different host
//    threads on one device) race on the array.  Serialise them.
//  * the first call on a device looks up the array's device address
//    (cudaGetSymbolAddress); make that first call before any stream capture.
//
// A second file-scope word next to the array receives the code of a bounded
// device wait that ran out during one of these calls; sd3_device_status reads
// and clears it together with the library's ordinary status word.
#include <mutex>

#include "../../include/sd3_b200.h"
#include "kernels.h"

namespace {

// 4 Mi bf16 elements = 8 MiB: covers batch 8 of 128x128 latents with 16
// channels and patch 2 (8 * 4096 * 64 = 2 Mi elements) twice over.
constexpr long kStaticPatchElems = SD3_STATIC_PATCH_ELEMS;
static __device__ __align__(256) __nv_bfloat16 g_patch_scratch[kStaticPatchElems];
static __device__ int g_static_status;  // zero at module load

struct StaticAddrs {
  __nv_bfloat16* scratch = nullptr;
  int* status = nullptr;
};
StaticAddrs g_addrs[64];
std::mutex g_addrs_mu;

// In host code `g_patch_scratch` is only a handle for the runtime, not an
// address a kernel may dereference; the real device address is looked up once
// per device (with that device current) and cached here.
const StaticAddrs* static_addrs_for_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    sd3::set_last_error("sd3_patch_embed_static: cannot identify the current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_addrs_mu);
  StaticAddrs& a = g_addrs[dev];
  if (!a.scratch) {
    void* p = nullptr;
    void* q = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_patch_scratch);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&q, g_static_status);
    if (e != cudaSuccess || !p || !q) {
      sd3::set_last_error("sd3_patch_embed_static: cudaGetSymbolAddress failed: %s",
                          cudaGetErrorString(e));
      return nullptr;
    }
    a.status = static_cast<int*>(q);
    a.scratch = static_cast<__nv_bfloat16*>(p);
  }
  return &a;
}

}  // namespace

namespace sd3 {
// The allocation-free entry point's status word on the current device, or null if no
// such call has been made there yet (nothing is resolved or allocated by asking).
int* static_status_word_if_resolved() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_addrs_mu);
  return g_addrs[dev].status;
}
}  // namespace sd3

extern "C" {

int sd3_patch_embed_static(const void* latent, int io_dtype, const void* w, const float* bias,
                           const float* pos_table, float* out, int B, int C, int H, int W, int patch,
                           int E, void* stream) {
  using namespace sd3;
  if (!latent || !w || !pos_table || !out || B <= 0 || C <= 0 || patch <= 0 || H <= 0 || W <= 0 ||
      H % patch || W % patch || E <= 0 ||
      (io_dtype != SD3_DTYPE_F32 && io_dtype != SD3_DTYPE_BF16)) {
    set_last_error("sd3_patch_embed_static: invalid argument");
    return SD3_ERR_INVALID_ARG;
  }
  const int hp = H / patch, wp = W / patch, Kp = C * patch * patch;
  const long need = static_cast<long>(B) * hp * wp * Kp;
  if (need > kStaticPatchElems) {
    set_last_error(
        "sd3_patch_embed_static: %ld patch elements needed, the built-in scratch holds %ld "
        "(use sd3_patch_embed with your own scratch buffer for larger inputs)",
        need, kStaticPatchElems);
    return SD3_ERR_UNSUPPORTED;
  }
  const StaticAddrs* addrs = static_addrs_for_current_device();
  if (!addrs) return SD3_ERR_CUDA;
  __nv_bfloat16* scratch = addrs->scratch;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = launch_patchify(latent, io_dtype == SD3_DTYPE_F32, scratch, 0, B, C, H, W, patch, st);
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
  // The library's ordinary status word is allocated on first use, which this entry point
  // must not do: a wait that runs out is recorded in the file-scope word instead.
  return launch_gemm(scratch, Kp, w, Kp, OPERAND_BF16, B * hp * wp, E, Kp, e, addrs->status, st);
}

}  // extern "C"

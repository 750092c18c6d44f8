// Classifier-free-guidance combine + Euler flow-matching update, fused into one
// pass over the latent.  The reference project has no sampler (its README only
// promises the architecture); this is the caller right next to the denoiser
// forward: every sampling step runs the denoiser on the stacked batch
// [conditional; unconditional] and then
//     v   = v_u + g (v_c - v_u)
//     x  <- x + (sigma_next - sigma) v
// The kernel keeps the stacked model input up to date by writing the new x
// into both halves, so the loop needs no other copy between steps.
#include "../../include/sd3_b200.h"
#include "kernels.h"

namespace sd3 {
int device_sm_count();
}

namespace {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// x_state: fp32 master copy of the latent (half elements); x2: stacked model
// input of T (2 * half elements); v: stacked velocity of T (cond half first).
template <typename T>
__global__ void cfg_euler_kernel(float* __restrict__ x_state, T* __restrict__ x2,
                                 const T* __restrict__ v, long half, float guidance, float dsigma) {
  long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (; i < half; i += stride) {
    const float vc = to_f<T>(v[i]);
    const float vu = to_f<T>(v[half + i]);
    const float xn = x_state[i] + dsigma * (vu + guidance * (vc - vu));
    x_state[i] = xn;
    const T xo = from_f<T>(xn);
    x2[i] = xo;
    x2[half + i] = xo;
  }
}

}  // namespace

extern "C" int sd3_cfg_euler_step(float* x_state, void* x_stacked, const void* v_stacked, int io_dtype,
                                  long half_elems, float guidance, float dsigma, void* stream) {
  using namespace sd3;
  if (!x_state || !x_stacked || !v_stacked || half_elems <= 0 ||
      (io_dtype != SD3_DTYPE_F32 && io_dtype != SD3_DTYPE_BF16)) {
    set_last_error("sd3_cfg_euler_step: invalid argument");
    return SD3_ERR_INVALID_ARG;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long blocks = (half_elems + 255) / 256;
  const unsigned grid = static_cast<unsigned>(blocks < sd3::device_sm_count() * 8 ? blocks : sd3::device_sm_count() * 8);
  if (io_dtype == SD3_DTYPE_F32)
    cfg_euler_kernel<float><<<grid, 256, 0, st>>>(x_state, static_cast<float*>(x_stacked),
                                                  static_cast<const float*>(v_stacked), half_elems,
                                                  guidance, dsigma);
  else
    cfg_euler_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        x_state, static_cast<__nv_bfloat16*>(x_stacked), static_cast<const __nv_bfloat16*>(v_stacked),
        half_elems, guidance, dsigma);
  return after_launch("cfg_euler_kernel");
}

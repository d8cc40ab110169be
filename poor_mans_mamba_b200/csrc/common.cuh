// Shared helpers of the sm_100a kernels: storage-type load/store (activations, weights
// and caches are float or bfloat16; all arithmetic is float), warp/block reductions and
// the C-ABI launch convention.  Every exported launcher returns a cudaError_t as int
// (0 = launched) and never synchronises or allocates.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define PMM_DTYPE_F32 0
#define PMM_DTYPE_BF16 1
#define PMM_ERR_BAD_ARGUMENT 1001  // outside the cudaError_t range that launches return

#define PMM_EXPORT extern "C" __attribute__((visibility("default")))

namespace pmm {

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block; `red` is shared memory for 32 floats.  Every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // protects `red` against a previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
// For results that are stored as bfloat16: relative error about 1e-6, three instructions' worth
// of special-function work instead of a full-precision exponential and division.
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.f + __expf(-x)); }

// v if v>20; exp(v) if v<-20; log1p(exp(v)) otherwise.
__device__ __forceinline__ float softplus_f(float v) {
  if (v > 20.f) return v;
  if (v < -20.f) return expf(v);
  return log1pf(expf(v));
}

inline int launch_status() { return static_cast<int>(cudaGetLastError()); }

// Programmatic dependent launch.  A kernel started with launch_pdl may begin while the kernel
// before it on the stream is still running; pdl_wait() inside it returns once that kernel has
// finished and its writes are visible, so everything a kernel does before pdl_wait() must not
// touch memory that other kernels write (reading constant weights is fine).
// pdl_launch_dependents() lets the next kernel of the stream start its own preamble early.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);  // errors surface in launch_status()
}

}  // namespace pmm

// Calls FN<float>(...) or FN<__nv_bfloat16>(...) by dtype code.
#define PMM_DISPATCH_DTYPE(code, S, ...)          \
  do {                                            \
    if ((code) == PMM_DTYPE_F32) {                \
      using S = float;                            \
      __VA_ARGS__;                                \
    } else if ((code) == PMM_DTYPE_BF16) {        \
      using S = __nv_bfloat16;                    \
      __VA_ARGS__;                                \
    } else {                                      \
      return PMM_ERR_BAD_ARGUMENT;                \
    }                                             \
  } while (0)

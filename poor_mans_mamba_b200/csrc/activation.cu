// SwiGLU activation on the output of the fused [gate; up] projection.
//   act[t,f] = silu(gu[t,f] * gate_mult) * gu[t,F+f]
// (reference src/ops/cuda_backend.cu:311-338: scale, silu, mul as three launches).
#include "common.cuh"

namespace pmm {

template <typename S>
__global__ void silu_mul_kernel(const S* __restrict__ gu, long long ld, float gate_mult,
                                S* __restrict__ out, int F) {
  const int t = blockIdx.x;
  const S* row = gu + static_cast<long long>(t) * ld;
  S* o = out + static_cast<size_t>(t) * F;
  for (int f = blockIdx.y * blockDim.x + threadIdx.x; f < F; f += gridDim.y * blockDim.x) {
    const float g = ldf(row + f) * gate_mult;
    stf(o + f, silu_f(g) * ldf(row + F + f));
  }
}

}  // namespace pmm

PMM_EXPORT int pmm_silu_mul(const void* gu, long long ld, float gate_mult, void* out, int T, int F,
                            int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (F <= 0) return PMM_ERR_BAD_ARGUMENT;
  int ytiles = (F + 1023) / 1024;
  if (ytiles > 64) ytiles = 64;
  dim3 grid(T, ytiles);
  PMM_DISPATCH_DTYPE(dtype, S, pmm::silu_mul_kernel<S><<<grid, 256, 0, stream>>>(
                                   static_cast<const S*>(gu), ld, gate_mult, static_cast<S*>(out), F));
  return pmm::launch_status();
}

namespace pmm {
template <typename S>
__global__ void add_row_bias_kernel(S* __restrict__ x, const float* __restrict__ bias, int D) {
  S* row = x + static_cast<size_t>(blockIdx.x) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) stf(row + i, ldf(row + i) + bias[i]);
}
}  // namespace pmm

// x[t, :] += bias for a contiguous [T, D] activation (projection biases).
PMM_EXPORT int pmm_add_row_bias(void* x, const float* bias, int T, int D, int dtype,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  PMM_DISPATCH_DTYPE(dtype, S,
                     pmm::add_row_bias_kernel<S><<<T, 256, 0, stream>>>(static_cast<S*>(x), bias, D));
  return pmm::launch_status();
}

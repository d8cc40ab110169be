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

// bfloat16, F and ld multiples of 8, 16-byte aligned rows: eight elements per thread.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, long long ld, float gate_mult,
                                       __nv_bfloat16* __restrict__ out, int F) {
  const int t = blockIdx.x;
  const __nv_bfloat16* row = gu + static_cast<long long>(t) * ld;
  __nv_bfloat16* o = out + static_cast<size_t>(t) * F;
  for (int f = (blockIdx.y * blockDim.x + threadIdx.x) * 8; f < F; f += gridDim.y * blockDim.x * 8) {
    const uint4 gv = *reinterpret_cast<const uint4*>(row + f);
    const uint4 uv = *reinterpret_cast<const uint4*>(row + F + f);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 g = __bfloat1622float2(g2[i]);
      const float2 u = __bfloat1622float2(u2[i]);
      o2[i] = __floats2bfloat162_rn(silu_fast(g.x * gate_mult) * u.x, silu_fast(g.y * gate_mult) * u.y);
    }
    *reinterpret_cast<uint4*>(o + f) = ov;
  }
}

}  // namespace pmm

PMM_EXPORT int pmm_silu_mul(const void* gu, long long ld, float gate_mult, void* out, int T, int F,
                            int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (F <= 0) return PMM_ERR_BAD_ARGUMENT;
  if (dtype == PMM_DTYPE_BF16 && F % 8 == 0 && ld % 8 == 0 &&
      reinterpret_cast<uintptr_t>(gu) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    int yt = (F / 8 + 255) / 256;
    if (yt > 64) yt = 64;
    pmm::silu_mul_bf16x8_kernel<<<dim3(T, yt), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(gu), ld, gate_mult, static_cast<__nv_bfloat16*>(out), F);
    return pmm::launch_status();
  }
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

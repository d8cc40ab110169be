// Embedding gather and the fused "residual add + RMSNorm" kernel.
//
// The residual stream is float in every mode.  Branch outputs (mixer / feed-forward
// results in the storage type) are folded into it by the same kernel that produces
// the next normalised activation, so the stream is read and written once per norm.
//
// Formulas: h[t] = mult * E[tok[t]]  (reference src/ops/gpu/embed.cu:5-16);
// y = x * (1/sqrt(mean(x^2)+eps)) * w  (reference src/ops/gpu/rms_norm.cu:6-26).
#include "common.cuh"

namespace pmm {

template <typename S>
__global__ void embed_kernel(float* __restrict__ out, const S* __restrict__ table,
                             const int* __restrict__ tokens, float mult, int D, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = tokens[t];
  const bool ok = id >= 0 && id < V;  // the host rejects such ids before launching
  if (!ok) id = 0;
  const S* row = table + static_cast<size_t>(id) * D;
  float* o = out + static_cast<size_t>(t) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = ok ? mult * ldf(row + i) : 0.f;
}

// One block per output row.  h' = (h + sa*a) + sb*b ; out = h' * rsqrt(mean(h'^2)+eps) * w.
// rows == nullptr: row r of h is updated in place and out[r] written.
// rows != nullptr: h is left untouched, out[r] is computed from row rows[r].
template <typename S>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const S* __restrict__ a, float sa,
                                   const S* __restrict__ b, float sb, const float* __restrict__ w,
                                   float eps, S* __restrict__ out, const int* __restrict__ rows,
                                   int D) {
  extern __shared__ float buf[];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = h[src + i];
    if (a) v = v + sa * ldf(a + src + i);
    if (b) v = v + sb * ldf(b + src + i);
    buf[i] = v;
    ss += v * v;
    if (!rows && (a || b)) h[src + i] = v;
  }
  if (!out) return;
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(D) + eps);
  S* o = out + static_cast<size_t>(r) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) stf(o + i, buf[i] * inv * w[i]);
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

// The same for widths that are a multiple of 4: four elements per thread and access.
template <typename S>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const S* __restrict__ a, float sa,
                                       const S* __restrict__ b, float sb, const float* __restrict__ w,
                                       float eps, S* __restrict__ out, const int* __restrict__ rows,
                                       int D) {
  extern __shared__ float buf[];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * D;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < D; i += blockDim.x * 4) {
    float4 v = ld4(h + src + i);
    if (a) {
      const float4 x = ld4(a + src + i);
      v.x += sa * x.x; v.y += sa * x.y; v.z += sa * x.z; v.w += sa * x.w;
    }
    if (b) {
      const float4 x = ld4(b + src + i);
      v.x += sb * x.x; v.y += sb * x.y; v.z += sb * x.z; v.w += sb * x.w;
    }
    *reinterpret_cast<float4*>(buf + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    if (!rows && (a || b)) st4(h + src + i, v);
  }
  if (!out) return;
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(D) + eps);
  S* o = out + static_cast<size_t>(r) * D;
  for (int i = threadIdx.x * 4; i < D; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(buf + i);
    const float4 g = ld4(w + i);
    st4(o + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
  }
}

__global__ void scale_f32_kernel(float* __restrict__ x, float s, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= s;
}

template <typename S>
__global__ void cast_scale_kernel(float* __restrict__ out, const S* __restrict__ in, float s, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = s * ldf(in + i);
}

}  // namespace pmm

PMM_EXPORT int pmm_embed(void* out, const void* table, const int* tokens, float mult, int T, int D,
                         int V, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::embed_kernel<S>, dim3(T), dim3(256), 0, stream,
                                               static_cast<float*>(out), static_cast<const S*>(table), tokens,
                                               mult, D, V));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_add_rmsnorm(void* h, const void* a, float sa, const void* b, float sb,
                               const float* w, float eps, void* out, const int* rows, int R, int D,
                               int dtype, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (out && !w) return PMM_ERR_BAD_ARGUMENT;
  const size_t smem = static_cast<size_t>(D) * sizeof(float);
  if (smem > 200 * 1024) return PMM_ERR_BAD_ARGUMENT;  // width beyond one block's shared memory
  const int threads = D >= 1024 ? 256 : 128;
  const bool vec = D % 4 == 0 && reinterpret_cast<uintptr_t>(h) % 16 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(b) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(w) % 16 == 0;
  PMM_DISPATCH_DTYPE(dtype, S, {
    auto kern = vec ? pmm::add_rmsnorm_vec_kernel<S> : pmm::add_rmsnorm_kernel<S>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    pmm::launch_pdl(kern, dim3(R), dim3(threads), smem, stream, static_cast<float*>(h), static_cast<const S*>(a), sa,
                    static_cast<const S*>(b), sb, w, eps, static_cast<S*>(out), rows, D);
  });
  return pmm::launch_status();
}

PMM_EXPORT int pmm_scale_f32(float* x, float s, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  pmm::scale_f32_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
      x, s, static_cast<size_t>(n));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_cast_scale(float* out, const void* in, float s, long long n, int dtype,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::cast_scale_kernel<S><<<static_cast<unsigned>((n + 255) / 256), 256,
                                                          0, stream>>>(
                                   out, static_cast<const S*>(in), s, static_cast<size_t>(n)));
  return pmm::launch_status();
}

// Token sampling on the device: greedy argmax (the first index wins ties, as the
// reference's host loop does, src/runtime/worker.cpp:30-59) and temperature sampling by
// the Gumbel-max rule, which draws exactly from softmax(logits / T):
//   token = argmax_i ( logits[i]/T + g_i ),  g_i = -log(-log(u_i))
// with u_i from a counter-based generator keyed by (seed, step, i), so a request's draws
// do not depend on what else is in the batch.  A row with T <= 0 is sampled greedily.
#include "common.cuh"
#include <math_constants.h>

namespace pmm {

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

__device__ __forceinline__ float gumbel_noise(unsigned long long seed, unsigned step, unsigned idx) {
  const unsigned long long key = splitmix64(seed ^ (static_cast<unsigned long long>(step) << 32 | idx));
  const unsigned long long r = splitmix64(key);
  // 24 random bits -> u strictly inside (0, 1)
  const float u = (static_cast<float>(r >> 40) + 0.5f) * (1.0f / 16777216.0f);
  return -logf(-logf(u));
}

__global__ void sample_rows_kernel(const float* __restrict__ logits, long long ld,
                                   const float* __restrict__ temperature,
                                   const long long* __restrict__ seeds,
                                   const int* __restrict__ steps, int* __restrict__ out, int V) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + static_cast<long long>(r) * ld;
  const float temp = temperature ? temperature[r] : 0.f;
  const bool greedy = !(temp > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / temp;
  const unsigned long long seed = seeds ? static_cast<unsigned long long>(seeds[r]) : 0ull;
  const unsigned step = steps ? static_cast<unsigned>(steps[r]) : 0u;
  float bv = -CUDART_INF_F;
  int bi = 0x7fffffff;
  // eight independent loads per thread and pass, so a row costs few memory round trips
  constexpr int kU = 8;
  for (int base = 0; base < V; base += kU * blockDim.x) {
    float v[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int i = base + u * blockDim.x + threadIdx.x;
      v[u] = i < V ? row[i] : -CUDART_INF_F;
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int i = base + u * blockDim.x + threadIdx.x;
      if (i >= V) continue;
      float x = v[u];
      if (!greedy) x = x * inv_t + gumbel_noise(seed, step, static_cast<unsigned>(i));
      if (x > bv || (x == bv && i < bi) || bi == 0x7fffffff) {
        bv = x;
        bi = i;
      }
    }
  }
  // warp, then block reduction; smaller index wins equal values
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    best_v[warp] = bv;
    best_i[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nwarp = blockDim.x >> 5;
    bv = lane < nwarp ? best_v[lane] : -CUDART_INF_F;
    bi = lane < nwarp ? best_i[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
  }
}

}  // namespace pmm

PMM_EXPORT int pmm_sample_rows(const float* logits, long long ld, const float* temperature,
                               const long long* seeds, const int* steps, int* out, int n_rows, int V,
                               cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0) return PMM_ERR_BAD_ARGUMENT;
  pmm::launch_pdl(pmm::sample_rows_kernel, dim3(n_rows), dim3(1024), 0, stream, logits, ld, temperature, seeds, steps,
                  out, V);
  return pmm::launch_status();
}

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

// Order-preserving map of a float onto unsigned integers (larger float -> larger integer).
__device__ __forceinline__ unsigned sample_orderable(float x) {
  const unsigned b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

constexpr int kSampleThreads = 256;
constexpr int kSampleLoads = 8;                                   // independent loads per thread and pass
constexpr int kSampleSpan = 2 * kSampleLoads * kSampleThreads;    // vocabulary entries per block: two passes

// A row is shared by ceil(V / kSampleSpan) blocks (a single block per row took 20 us for a
// vocabulary of 130,000).  A block finds the best (value, index) of its span and merges it into
// the row's 64-bit slot with atomicMax: value in the high word, ~index in the low word, so the
// larger value wins and among equal values the smaller index.  The block that takes the row's
// last ticket writes the token and leaves slot and ticket at zero for the next launch.
__global__ void __launch_bounds__(kSampleThreads)
    sample_rows_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ temperature,
                       const long long* __restrict__ seeds, const int* __restrict__ steps, int* __restrict__ out,
                       int V, unsigned long long* __restrict__ slots, int* __restrict__ tickets) {
  __shared__ float best_v[kSampleThreads / 32];
  __shared__ int best_i[kSampleThreads / 32];
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
  const int span_lo = blockIdx.y * kSampleSpan, span_hi = min(V, span_lo + kSampleSpan);
  for (int base = span_lo; base < span_hi; base += kSampleLoads * kSampleThreads) {
    float v[kSampleLoads];
#pragma unroll
    for (int u = 0; u < kSampleLoads; ++u) {
      const int i = base + u * kSampleThreads + threadIdx.x;
      v[u] = i < span_hi ? row[i] : -CUDART_INF_F;
    }
#pragma unroll
    for (int u = 0; u < kSampleLoads; ++u) {
      const int i = base + u * kSampleThreads + threadIdx.x;
      if (i >= span_hi) continue;
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
    constexpr int nwarp = kSampleThreads / 32;
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
    if (lane == 0) {
      if (gridDim.y == 1) {
        out[r] = bi == 0x7fffffff ? 0 : bi;
      } else {
        if (bi != 0x7fffffff)
          atomicMax(slots + r, (static_cast<unsigned long long>(sample_orderable(bv)) << 32) |
                                   (0xffffffffu - static_cast<unsigned>(bi)));
        __threadfence();
        if (atomicAdd(tickets + r, 1) == static_cast<int>(gridDim.y) - 1) {  // every span of the row is in
          __threadfence();
          const unsigned long long best = atomicExch(slots + r, 0ull);
          tickets[r] = 0;
          out[r] = best == 0ull ? 0 : static_cast<int>(0xffffffffu - static_cast<unsigned>(best & 0xffffffffu));
        }
      }
    }
  }
}

}  // namespace pmm

// slots (64-bit) and tickets (32-bit): one of each per row, zero before the first use and left
// zero by every launch; needed when the vocabulary is wider than one block's span (4,096).
PMM_EXPORT int pmm_sample_rows(const float* logits, long long ld, const float* temperature,
                               const long long* seeds, const int* steps, int* out, int n_rows, int V,
                               unsigned long long* slots, int* tickets, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0) return PMM_ERR_BAD_ARGUMENT;
  const int parts = (V + pmm::kSampleSpan - 1) / pmm::kSampleSpan;
  if (parts > 65535 || (parts > 1 && (!slots || !tickets))) return PMM_ERR_BAD_ARGUMENT;
  pmm::launch_pdl(pmm::sample_rows_kernel, dim3(n_rows, parts), dim3(pmm::kSampleThreads), 0, stream, logits, ld,
                  temperature, seeds, steps, out, V, slots, tickets);
  return pmm::launch_status();
}

// Paged grouped-query attention over the cache, float arithmetic (CUDA cores).
//
// One warp owns one (token, query head, key split): it walks the keys
// [max(lo, z*split_len), min(pos+1, (z+1)*split_len)) in chunks of 32 (one key per lane
// for the scores, one slice of the head dimension per lane for the value sum) with an
// online softmax.  Portions of prompts and decoded tokens are the same to it: a token at
// absolute position pos sees keys lo..pos of its own request through the block table;
// lo = pos-window+1 for a sliding window, else 0.  With one split the result is written
// normalised; with several, (max, sum, unnormalised output) go to scratch and
// flash_combine (attention_mma.cu) merges them.  This kernel is the 32-bit path and the general
// fallback of the bfloat16 path; the tensor-core kernels cover the long cases.
//
//   sc[s] = (q.K[s]) * scale;  p = exp(sc - max);  o = sum p V / sum p
// (reference src/ops/gpu/attention.cu:44-105).
#include "common.cuh"
#include <math_constants.h>

namespace pmm {

constexpr int kAttnWarps = 4;
constexpr int kAttnMaxAcc = 8;  // head_dim <= 256

__device__ __forceinline__ float dot_row(const float* __restrict__ qw, const float* __restrict__ kr, int Dh) {
  float dot = 0.f;
  for (int d = 0; d < Dh; d += 4) {
    const float4 kv = *reinterpret_cast<const float4*>(kr + d);
    dot += qw[d] * kv.x;
    dot += qw[d + 1] * kv.y;
    dot += qw[d + 2] * kv.z;
    dot += qw[d + 3] * kv.w;
  }
  return dot;
}

__device__ __forceinline__ float dot_row(const float* __restrict__ qw, const __nv_bfloat16* __restrict__ kr,
                                         int Dh) {
  float dot = 0.f;
  for (int d = 0; d < Dh; d += 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h2[i]);
      dot += qw[d + 2 * i] * f.x;
      dot += qw[d + 2 * i + 1] * f.y;
    }
  }
  return dot;
}

template <typename S>
__global__ void __launch_bounds__(kAttnWarps * 32)
    paged_attention_kernel(const S* __restrict__ q, const S* __restrict__ pool,
                           const int* __restrict__ block_table, int max_blocks,
                           const int* __restrict__ positions, const int* __restrict__ seq_of,
                           S* __restrict__ out, float* __restrict__ part_o,
                           float* __restrict__ part_ml, float scale, int window, int split_len,
                           int n_splits, int page_size, int Hq, int Hkv, int Dh) {
  extern __shared__ float qs[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int hq = blockIdx.y * kAttnWarps + warp;
  const int z = blockIdx.z;
  if (hq >= Hq) return;  // only warp-level synchronisation below
  const int hk = hq / (Hq / Hkv);
  const int pos = positions[t];
  const int* bt = block_table + static_cast<size_t>(seq_of[t]) * max_blocks;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int k_begin = max(lo, z * split_len);
  const int k_end = min(pos + 1, (z + 1) * split_len);
  const int kv_dim = Hkv * Dh;
  const long long v_plane = static_cast<long long>(page_size) * kv_dim;

  float* qw = qs + warp * Dh;
  const size_t q_off = (static_cast<size_t>(t) * Hq + hq) * Dh;
  for (int d = lane; d < Dh; d += 32) qw[d] = ldf(q + q_off + d);
  __syncwarp();

  float m = -CUDART_INF_F, l = 0.f;
  float acc[kAttnMaxAcc];
#pragma unroll
  for (int i = 0; i < kAttnMaxAcc; ++i) acc[i] = 0.f;

  for (int base = k_begin; base < k_end; base += 32) {
    const int key = base + lane;
    const bool valid = key < k_end;
    long long koff = 0;
    float sc = -CUDART_INF_F;
    if (valid) {
      const int page = bt[key / page_size];
      koff = (static_cast<long long>(page) * 2 * page_size + key % page_size) * kv_dim + hk * Dh;
      sc = dot_row(qw, pool + koff, Dh) * scale;
    }
    const float m_new = fmaxf(m, warp_max(sc));  // lane 0 is always valid, so m_new is finite
    const float p = valid ? expf(sc - m_new) : 0.f;
    const float corr = expf(m - m_new);  // first chunk: exp(-inf) = 0
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < kAttnMaxAcc; ++i) acc[i] *= corr;
    const int n_valid = min(32, k_end - base);
    for (int j = 0; j < n_valid; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long voff = __shfl_sync(0xffffffffu, koff, j) + v_plane;
#pragma unroll
      for (int i = 0; i < kAttnMaxAcc; ++i) {
        const int d = lane + 32 * i;
        if (d < Dh) acc[i] += pj * ldf(pool + voff + d);
      }
    }
    m = m_new;
  }

  if (n_splits == 1) {
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < kAttnMaxAcc; ++i) {
      const int d = lane + 32 * i;
      if (d < Dh) stf(out + q_off + d, acc[i] * inv);
    }
  } else {
    const size_t pi = (static_cast<size_t>(t) * Hq + hq) * n_splits + z;
#pragma unroll
    for (int i = 0; i < kAttnMaxAcc; ++i) {
      const int d = lane + 32 * i;
      if (d < Dh) part_o[pi * Dh + d] = acc[i];
    }
    if (lane == 0) {
      part_ml[pi * 2] = m;
      part_ml[pi * 2 + 1] = l;
    }
  }
}

}  // namespace pmm

// part_o needs T*Hq*n_splits*Dh floats and part_ml T*Hq*n_splits*2 floats when n_splits > 1.
PMM_EXPORT int pmm_paged_attention(const void* q, const void* pool, const int* block_table,
                                   int max_blocks, const int* positions, const int* seq_of,
                                   void* out, float* part_o, float* part_ml, float scale, int window,
                                   int split_len, int n_splits, int page_size, int T, int Hq,
                                   int Hkv, int Dh, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (Dh <= 0 || Dh % 16 || Dh > 32 * pmm::kAttnMaxAcc) return PMM_ERR_BAD_ARGUMENT;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || page_size <= 0 || n_splits < 1 || n_splits > 65535)
    return PMM_ERR_BAD_ARGUMENT;
  if (n_splits > 1 && (!part_o || !part_ml || split_len <= 0)) return PMM_ERR_BAD_ARGUMENT;
  if (n_splits == 1) split_len = 0x40000000;
  const int head_blocks = (Hq + pmm::kAttnWarps - 1) / pmm::kAttnWarps;
  if (head_blocks > 65535) return PMM_ERR_BAD_ARGUMENT;
  dim3 grid(T, head_blocks, n_splits);
  const size_t smem = static_cast<size_t>(pmm::kAttnWarps) * Dh * sizeof(float);
  PMM_DISPATCH_DTYPE(dtype, S, {
    pmm::paged_attention_kernel<S><<<grid, pmm::kAttnWarps * 32, smem, stream>>>(
        static_cast<const S*>(q), static_cast<const S*>(pool), block_table, max_blocks, positions,
        seq_of, static_cast<S*>(out), part_o, part_ml, scale, window, split_len, n_splits,
        page_size, Hq, Hkv, Dh);
  });
  return pmm::launch_status();
}

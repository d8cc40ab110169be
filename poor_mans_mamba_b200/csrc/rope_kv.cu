// Query/key scaling, rotate-half RoPE and the write of keys and values into cache pages.
//
// Input: column slices q/k/v of a projection buffer (row strides in elements).  Output:
// q_out [T, Hq*Dh] contiguous, and K/V rows either scattered through the request's block
// table into the layer's pages [page][2][page_size][Hkv*Dh], or (no pool given) written
// to contiguous k_out/v_out so that a position encoding defined elsewhere can run before
// the separate page write (kv_store).
//
//   x' = x*scale;  ang = float(pos) * inv_freq[i];
//   x'[i] <- x'[i] cos - x'[i+Dh/2] sin;  x'[i+Dh/2] <- x'[i+Dh/2] cos + x'[i] sin
// (reference src/ops/gpu/attention.cu:4-40; key_multiplier is part of k's scale and so
// applied before the rotation; inv_freq is a float table made by the caller).
#include "common.cuh"

namespace pmm {

template <typename S>
__global__ void qkv_rope_store_kernel(const S* __restrict__ q, long long ldq, const S* __restrict__ k,
                                      long long ldk, const S* __restrict__ v, long long ldv,
                                      float q_scale, float k_scale, float v_scale,
                                      const float* __restrict__ inv_freq,
                                      const int* __restrict__ positions,
                                      const int* __restrict__ seq_of,
                                      const int* __restrict__ block_table, int max_blocks,
                                      S* __restrict__ pool, int page_size, S* __restrict__ q_out,
                                      S* __restrict__ k_out, S* __restrict__ v_out, int Hq, int Hkv,
                                      int Dh) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const float fpos = static_cast<float>(pos);
  const int half = Dh / 2;
  const int kv_dim = Hkv * Dh;
  S* k_dst = nullptr;
  S* v_dst = nullptr;
  if (Hkv == 0) {
  } else if (pool) {
    const int page = block_table[static_cast<size_t>(seq_of[t]) * max_blocks + pos / page_size];
    const size_t base = (static_cast<size_t>(page) * 2 * page_size + pos % page_size) * kv_dim;
    k_dst = pool + base;
    v_dst = pool + base + static_cast<size_t>(page_size) * kv_dim;
  } else {
    k_dst = k_out + static_cast<size_t>(t) * kv_dim;
    v_dst = v_out + static_cast<size_t>(t) * kv_dim;
  }
  const int n_rot = (Hq + Hkv) * half;
  for (int idx = threadIdx.x; idx < n_rot; idx += blockDim.x) {
    const int head = idx / half, i = idx % half;
    const bool is_q = head < Hq;
    const S* src = is_q ? q + static_cast<long long>(t) * ldq + head * Dh
                        : k + static_cast<long long>(t) * ldk + (head - Hq) * Dh;
    const float sc = is_q ? q_scale : k_scale;
    const float x1 = ldf(src + i) * sc, x2 = ldf(src + i + half) * sc;
    float o1 = x1, o2 = x2;
    if (inv_freq) {
      const float ang = fpos * inv_freq[i];
      const float c = cosf(ang), s = sinf(ang);
      o1 = x1 * c - x2 * s;
      o2 = x2 * c + x1 * s;
    }
    S* dst = is_q ? q_out + static_cast<size_t>(t) * Hq * Dh + head * Dh : k_dst + (head - Hq) * Dh;
    stf(dst + i, o1);
    stf(dst + i + half, o2);
  }
  for (int idx = threadIdx.x; idx < kv_dim; idx += blockDim.x)
    stf(v_dst + idx, ldf(v + static_cast<long long>(t) * ldv + idx) * v_scale);
}

template <typename S>
__global__ void kv_store_kernel(const S* __restrict__ k, const S* __restrict__ v,
                                const int* __restrict__ positions, const int* __restrict__ seq_of,
                                const int* __restrict__ block_table, int max_blocks,
                                S* __restrict__ pool, int page_size, int kv_dim) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int page = block_table[static_cast<size_t>(seq_of[t]) * max_blocks + pos / page_size];
  const size_t base = (static_cast<size_t>(page) * 2 * page_size + pos % page_size) * kv_dim;
  for (int idx = threadIdx.x; idx < kv_dim; idx += blockDim.x) {
    pool[base + idx] = k[static_cast<size_t>(t) * kv_dim + idx];
    pool[base + static_cast<size_t>(page_size) * kv_dim + idx] = v[static_cast<size_t>(t) * kv_dim + idx];
  }
}

}  // namespace pmm

PMM_EXPORT int pmm_qkv_rope_store(const void* q, long long ldq, const void* k, long long ldk,
                                  const void* v, long long ldv, float q_scale, float k_scale,
                                  float v_scale, const float* inv_freq, const int* positions,
                                  const int* seq_of, const int* block_table, int max_blocks,
                                  void* pool, int page_size, void* q_out, void* k_out, void* v_out,
                                  int T, int Hq, int Hkv, int Dh, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (Dh <= 0 || Dh % 2 || Hq <= 0 || Hkv < 0) return PMM_ERR_BAD_ARGUMENT;
  // Hkv == 0: queries only (a layer that reads another layer's keys and values)
  if (Hkv > 0 && !pool && (!k_out || !v_out)) return PMM_ERR_BAD_ARGUMENT;
  if (Hkv > 0 && (!k || !v)) return PMM_ERR_BAD_ARGUMENT;
  if (Hkv == 0) pool = nullptr;
  if (pool && (!block_table || page_size <= 0)) return PMM_ERR_BAD_ARGUMENT;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::qkv_rope_store_kernel<S>, dim3(T), dim3(256), 0, stream,
                                               static_cast<const S*>(q), ldq, static_cast<const S*>(k), ldk,
                                               static_cast<const S*>(v), ldv, q_scale, k_scale, v_scale,
                                               inv_freq, positions, seq_of, block_table, max_blocks,
                                               static_cast<S*>(pool), page_size, static_cast<S*>(q_out),
                                               static_cast<S*>(k_out), static_cast<S*>(v_out), Hq, Hkv, Dh));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_kv_store(const void* k, const void* v, const int* positions, const int* seq_of,
                            const int* block_table, int max_blocks, void* pool, int page_size, int T,
                            int kv_dim, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (page_size <= 0 || kv_dim <= 0) return PMM_ERR_BAD_ARGUMENT;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::kv_store_kernel<S><<<T, 256, 0, stream>>>(
                                   static_cast<const S*>(k), static_cast<const S*>(v), positions,
                                   seq_of, block_table, max_blocks, static_cast<S*>(pool), page_size,
                                   kv_dim));
  return pmm::launch_status();
}

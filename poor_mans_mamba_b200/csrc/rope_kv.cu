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

// The same with 16-byte accesses, a warp per token: the token's Dh/2 cosines and sines are computed
// once into shared memory (not once per head), then every lane rotates runs of neighbouring pairs.  Needs Dh/2 a multiple of the vector width (8 bfloat16 / 4 float) and 16-byte aligned rows.
template <typename S>
struct RopeVec;
template <>
struct RopeVec<float> {
  static constexpr int W = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct RopeVec<__nv_bfloat16> {
  static constexpr int W = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h2[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

template <typename S>
__global__ void __launch_bounds__(256)
    qkv_rope_store_vec_kernel(const S* __restrict__ q, long long ldq, const S* __restrict__ k, long long ldk,
                              const S* __restrict__ v, long long ldv, float q_scale, float k_scale, float v_scale,
                              const float* __restrict__ inv_freq, const int* __restrict__ positions,
                              const int* __restrict__ seq_of, const int* __restrict__ block_table, int max_blocks,
                              S* __restrict__ pool, int page_size, S* __restrict__ q_out, S* __restrict__ k_out,
                              S* __restrict__ v_out, int Hq, int Hkv, int Dh, int n_tokens) {
  constexpr int W = RopeVec<S>::W;
  extern __shared__ float s_all[];  // per warp: [Dh/2] cosines, then [Dh/2] sines
  pdl_launch_dependents();
  pdl_wait();
  // one warp per token, eight tokens a block
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  float* s_cs = s_all + (threadIdx.x >> 5) * Dh;
  const int pos = positions[t];
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
  for (int i = lane; i < half; i += 32) {
    float c = 1.f, sn = 0.f;
    if (inv_freq) {
      const float ang = static_cast<float>(pos) * inv_freq[i];
      c = cosf(ang);
      sn = sinf(ang);
    }
    s_cs[i] = c;
    s_cs[half + i] = sn;
  }
  __syncwarp();
  const int runs = half / W;  // runs of W pairs per head
  for (int idx = lane; idx < (Hq + Hkv) * runs; idx += 32) {
    const int head = idx / runs, i0 = (idx % runs) * W;
    const bool is_q = head < Hq;
    const S* src = is_q ? q + static_cast<long long>(t) * ldq + head * Dh
                        : k + static_cast<long long>(t) * ldk + (head - Hq) * Dh;
    const float sc = is_q ? q_scale : k_scale;
    float x1[W], x2[W], o1[W], o2[W];
    RopeVec<S>::load(src + i0, x1);
    RopeVec<S>::load(src + i0 + half, x2);
#pragma unroll
    for (int e = 0; e < W; ++e) {
      const float a = x1[e] * sc, b = x2[e] * sc;
      const float c = s_cs[i0 + e], sn = s_cs[half + i0 + e];
      o1[e] = inv_freq ? a * c - b * sn : a;
      o2[e] = inv_freq ? b * c + a * sn : b;
    }
    S* dst = is_q ? q_out + static_cast<size_t>(t) * Hq * Dh + head * Dh : k_dst + (head - Hq) * Dh;
    RopeVec<S>::store(dst + i0, o1);
    RopeVec<S>::store(dst + i0 + half, o2);
  }
  for (int idx = lane * W; idx < kv_dim; idx += 32 * W) {
    float x[W];
    RopeVec<S>::load(v + static_cast<long long>(t) * ldv + idx, x);
#pragma unroll
    for (int e = 0; e < W; ++e) x[e] *= v_scale;
    RopeVec<S>::store(v_dst + idx, x);
  }
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
  {
    // 16-byte accesses where every row and slice allows them
    const int es = dtype == PMM_DTYPE_BF16 ? 2 : 4, w = 16 / es;
    auto ok16 = [&](const void* p, long long ld) { return reinterpret_cast<uintptr_t>(p) % 16 == 0 && (ld * es) % 16 == 0; };
    const bool vec = (Dh / 2) % w == 0 && ok16(q, ldq) && ok16(q_out, Dh) && (Hkv == 0 || (ok16(k, ldk) && ok16(v, ldv))) &&
                     ok16(pool, Dh) && ok16(k_out, Dh) && ok16(v_out, Dh) && Dh <= 1024;
    if (vec) {
      const size_t smem = 8 * static_cast<size_t>(Dh) * sizeof(float);
      PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::qkv_rope_store_vec_kernel<S>, dim3((T + 7) / 8), dim3(256), smem, stream,
                                                   static_cast<const S*>(q), ldq, static_cast<const S*>(k), ldk,
                                                   static_cast<const S*>(v), ldv, q_scale, k_scale, v_scale,
                                                   inv_freq, positions, seq_of, block_table, max_blocks,
                                                   static_cast<S*>(pool), page_size, static_cast<S*>(q_out),
                                                   static_cast<S*>(k_out), static_cast<S*>(v_out), Hq, Hkv, Dh, T));
      return pmm::launch_status();
    }
  }
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

// Paged grouped-query attention for prompt portions on the fifth-generation tensor cores
// (bfloat16 storage, float accumulate, head size 64 or 128, page sizes that are multiples of 64).
//
// One block = 128 query rows of ONE sequence and ONE key/value head (a row is a (token, query
// head of the group) pair, as in the mma.sync kernel) and one key split.  It walks its keys in
// tiles of 128:
//   S  = Q K^T     tcgen05.mma, both operands in shared memory: Q written there by the block's
//                  threads (128-byte swizzle by hand), the K tile brought by TMA straight from the
//                  cache pages (two boxes of 64 keys, each inside one page); S (128 x 128 float)
//                  lands in tensor memory;
//   P  = softmax   four warps, ONE THREAD PER ROW: tcgen05.ld of the row (twice: maximum, then
//                  exponentials), no shuffles; P goes to shared memory as bfloat16, swizzled as an
//                  mma operand, and is handed over with fence.proxy.async + mbarrier;
//   O += P V       tcgen05.mma with the V tile as an MN-major operand (rows = keys, as the cache
//                  stores them), accumulated in a second tensor-memory range over all tiles.  The
//                  running maximum that the exponentials are taken against is only raised when a
//                  row's true maximum exceeds it by more than 8 (a factor 256, harmless in
//                  bfloat16 and float); only then the accumulated O and sum are rescaled (a
//                  tensor-memory load, multiply and store by the row's thread).  The result is
//                  exact: P, the sum and O always refer to the same maximum.
// Warp roles: 0 = TMA producer (two stages for K, one for V; a tile's copy is requested the moment
// the product that read the stage before has finished), 1 = tensor-memory owner and MMA issuer
// (S of the next tile is issued as soon as the softmax threads have taken the current S into
// registers, so the tensor core works while they compute), 2..5 = softmax and output.  Head size
// 64: 96 KB of shared memory and 256 columns of tensor memory a block, two blocks per SM.  Head
// size 128: every tile is two sub-tiles of 64 head-size columns (Q, K and V each 32 KB a stage,
// 160 KB a block, O in 128 columns), one block per SM.
// With several key splits the block writes (max, sum, unnormalised output) and the last block of
// a row tile merges them, as in the mma.sync kernel.  Every mbarrier wait is bounded (status
// codes 11..15 in *status, the block then leaves its loops, waits for its copies in flight and
// frees its tensor memory).  No cluster multicast.
//   sc[s] = (q.K[s]) * scale;  p = exp(sc - max);  o = sum p V / sum p
// (reference src/ops/gpu/attention.cu:44-105), keys lo..pos per token, lo from the window.
#include "tcgen05.cuh"
#include <math_constants.h>

namespace pmm {

using bf16 = __nv_bfloat16;

constexpr int kAtM = 128;       // query rows per block
constexpr int kAtKeys = 128;    // keys per tile
constexpr int kAtBox = 64;      // keys per TMA box (inside one page)
constexpr int kAtDhBlock = 64;  // head-size columns per sub-tile (128 bytes of bfloat16)
constexpr int kAtThreads = 192;
constexpr int kAtTmemCols = 256;  // S: columns 0..127, O: columns 128..128+head size
constexpr float kAtLazy = 8.f;    // how far (log2) a row's maximum may run ahead of the one in use
constexpr int kAtBtCap = 512;
constexpr int kAtSubBytes = kAtM * kAtDhBlock * 2;  // 16 KB: 128 rows (queries or keys) x 64 head-size columns
constexpr int kAtPBytes = kAtM * kAtKeys * 2;       // 32 KB: two sub-tiles of 64 keys
constexpr size_t at_smem(int dh) {  // Q, K x 2, V (each head size / 64 sub-tiles), P
  return static_cast<size_t>(4 * (dh / kAtDhBlock)) * kAtSubBytes + kAtPBytes + 1024 /*alignment*/;
}

// kind::f16 instruction descriptors: float accumulate, bfloat16 operands, A K-major.
constexpr unsigned kAtIdescS = (1u << 4) | (1u << 7) | (1u << 10) | ((kAtKeys >> 3) << 17) | ((kAtM >> 4) << 24);               // B = K tile, K-major
constexpr unsigned kAtIdescO = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((kAtDhBlock >> 3) << 17) | ((kAtM >> 4) << 24);   // B = 64 columns of the V tile, MN-major

__device__ __forceinline__ float at_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned at_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}
// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` in a [rows][64] bfloat16 tile with the
// 128-byte swizzle that TMA and the tensor core use (8-row groups of 1024 bytes).
__device__ __forceinline__ int at_swizzled(int row, int chunk) {
  return (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4);
}

template <int DH>
__global__ void __launch_bounds__(kAtThreads, DH == 64 ? 2 : 1)
    attention_tc_kernel(const bf16* __restrict__ q, const __grid_constant__ CUtensorMap map_kv,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ positions,
                        const int* __restrict__ cu, bf16* __restrict__ out, float* __restrict__ part_o,
                        float* __restrict__ part_ml, float scale_log2, int window, int split_len, int n_splits,
                        int page_size, int n_seq, int Hq, int Hkv, int* __restrict__ split_counter,
                        int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NSUB = DH / kAtDhBlock;            // sub-tiles of 64 head-size columns
  constexpr int kAtQBytes = NSUB * kAtSubBytes;    // Q, a K stage, the V stage
  constexpr int kAtKBytes = NSUB * kAtSubBytes;
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bar_q, bar_kfull[2], bar_vfull, bar_s, bar_sfree, bar_p, bar_pv;
  __shared__ unsigned s_tmem_base;
  __shared__ int s_abort, s_last;
  __shared__ int s_bt[kAtBtCap];

  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = tiles;
  unsigned char* sK = sQ + kAtQBytes;
  unsigned char* sV = sK + 2 * kAtKBytes;
  unsigned char* sP = sV + kAtKBytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = Hq / Hkv;
  const int tpt = kAtM / G;  // tokens per tile; rows beyond tpt * G stay empty when G does not divide 128
  const int hk = blockIdx.y, z = blockIdx.z;

  // which sequence and which of its tokens this tile covers (heavy tiles first, as in the mma.sync kernel)
  const int tile_id = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  int seq = 0, acc = 0;
  for (; seq < n_seq; ++seq) {
    const int n = cu[seq + 1] - cu[seq];
    const int nt = (n + tpt - 1) / tpt;
    if (tile_id < acc + nt) break;
    acc += nt;
  }
  if (seq >= n_seq) return;
  const int tok0 = cu[seq] + (tile_id - acc) * tpt;
  const int n_tok = min(cu[seq + 1], tok0 + tpt) - tok0;
  const int n_rows = n_tok * G;
  const int* bt = block_table + static_cast<size_t>(seq) * max_blocks;
  const int pos_min = positions[tok0], pos_max = positions[tok0 + n_tok - 1];
  const int lo_all = window > 0 ? max(0, pos_min - window + 1) : 0;
  const int k_begin = max(lo_all, z * split_len);
  const int k_end = min(pos_max + 1, (z + 1) * split_len);
  const int first = (k_begin / kAtBox) * kAtBox;  // boxes start on multiples of 64 keys: inside one page
  const int n_tiles = k_end > k_begin ? (k_end - first + kAtKeys - 1) / kAtKeys : 0;
  const int bt_lo = first / page_size;
  const int n_bt = n_tiles > 0 ? (k_end - 1) / page_size - bt_lo + 1 : 0;
  const bool bt_shared = n_bt <= kAtBtCap;

  if (tid == 0) {
    mbar_init(&bar_q, 128);
    mbar_init(&bar_kfull[0], 1);
    mbar_init(&bar_kfull[1], 1);
    mbar_init(&bar_vfull, 1);
    mbar_init(&bar_s, 1);
    mbar_init(&bar_sfree, 128);
    mbar_init(&bar_p, 128);
    mbar_init(&bar_pv, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (bt_shared)
    for (int i = tid; i < n_bt; i += kAtThreads) s_bt[i] = bt[bt_lo + i];
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem_base)), "r"(kAtTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;
  auto page_of = [&](int idx) { return bt_shared ? s_bt[idx - bt_lo] : bt[idx]; };
  auto give_up = [&](int code) {
    if (!*abort_flag) atomicExch(status, code);
    s_abort = 1;
  };

  const int row = ((warp & 3) << 5) + lane;  // the tensor-memory lane a thread of warps 2..5 may read = its row

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n_tiles > 0) {
      int k_issued = 0, v_issued = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const int base = first + j * kAtKeys;
        // a box that starts beyond the keys of this block is read from the tile's first page
        // instead (any real page: its scores are masked, its values multiplied by zero)
        const int b0 = base, b1 = (base + kAtBox < k_end) ? base + kAtBox : base;
        const int r0 = page_of(b0 / page_size) * 2 * page_size + b0 % page_size;
        const int r1 = page_of(b1 / page_size) * 2 * page_size + b1 % page_size;
        // The K stage of tile j was read by S_{j-2}.  The tensor core works in issue order (S_{j-2},
        // S_{j-1}, P V_{j-2}, ...), so P V_{j-2}, which the previous round of this loop waited for
        // before it requested V_{j-1}, finished after S_{j-2}: the stage is free.
        unsigned char* kd = sK + (j & 1) * kAtKBytes;
        mbar_expect_tx(&bar_kfull[j & 1], kAtKBytes);
#pragma unroll
        for (int d = 0; d < NSUB; ++d) {  // a sub-tile = 64 head-size columns of 128 keys: two boxes of 64 keys
          tma_load_2d(kd + d * kAtSubBytes, &map_kv, hk * DH + d * kAtDhBlock, r0, &bar_kfull[j & 1]);
          tma_load_2d(kd + d * kAtSubBytes + kAtSubBytes / 2, &map_kv, hk * DH + d * kAtDhBlock, r1, &bar_kfull[j & 1]);
        }
        k_issued = j + 1;
        if (j > 0 && !mbar_wait(&bar_pv, (j - 1) & 1, abort_flag)) {  // P V_{j-1} done: the V stage is free
          give_up(12);
          break;
        }
        mbar_expect_tx(&bar_vfull, kAtKBytes);
#pragma unroll
        for (int d = 0; d < NSUB; ++d) {
          tma_load_2d(sV + d * kAtSubBytes, &map_kv, hk * DH + d * kAtDhBlock, r0 + page_size, &bar_vfull);
          tma_load_2d(sV + d * kAtSubBytes + kAtSubBytes / 2, &map_kv, hk * DH + d * kAtDhBlock, r1 + page_size, &bar_vfull);
        }
        v_issued = j + 1;
      }
      if (s_abort) {
        // copies already requested still write into this block's shared memory: wait for them
        for (int j = max(0, k_issued - 2); j < k_issued; ++j)
          for (unsigned i = 0; i < kSpinLimit && !mbar_try_wait(&bar_kfull[j & 1], (j >> 1) & 1); ++i) {
          }
        if (v_issued > 0)
          for (unsigned i = 0; i < kSpinLimit && !mbar_try_wait(&bar_vfull, (v_issued - 1) & 1); ++i) {
          }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_tiles > 0) {
      auto issue_s = [&](int j) {  // S_j = Q K_j^T
        unsigned char* kst = sK + (j & 1) * kAtKBytes;
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)  // 16 head-size columns a step, four steps a sub-tile
          umma_f16(tmem_base, umma_desc(sQ + (k >> 2) * kAtSubBytes) + 2 * (k & 3), umma_desc(kst + (k >> 2) * kAtSubBytes) + 2 * (k & 3),
                   kAtIdescS, k > 0 ? 1u : 0u);
        umma_commit(&bar_s);
      };
      bool ok = mbar_wait(&bar_q, 0, abort_flag) && mbar_wait(&bar_kfull[0], 0, abort_flag);
      if (!ok) give_up(13);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        issue_s(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          // the softmax threads hold S_j in registers: the next S may overwrite it, and the
          // tensor core works on it while they compute
          if (!mbar_wait(&bar_sfree, j & 1, abort_flag) ||
              !mbar_wait(&bar_kfull[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag)) {
            give_up(13);
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          issue_s(j + 1);
        }
        if (!mbar_wait(&bar_p, j & 1, abort_flag) || !mbar_wait(&bar_vfull, j & 1, abort_flag)) {
          give_up(14);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        {  // O += P V_j: A = P (two sub-tiles of 64 keys), B = V rows as they lie in the cache
           // (MN-major): 16 keys further = 16 rows of 128 bytes
#pragma unroll
          for (int d = 0; d < NSUB; ++d) {  // 64 head-size columns of O an instruction
            const unsigned long long v_desc = umma_desc(sV + d * kAtSubBytes);
#pragma unroll
            for (int k = 0; k < kAtKeys / 16; ++k) {
              const unsigned long long a_desc = umma_desc(sP + (k / 4) * (kAtPBytes / 2)) + 2 * (k % 4);
              umma_f16(tmem_base + kAtKeys + d * kAtDhBlock, a_desc, v_desc + ((k * 16 * 128) >> 4), kAtIdescO,
                       (j > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit(&bar_pv);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax and output (warps 2..5)
    const unsigned lane_base = tmem_base + (static_cast<unsigned>((warp & 3) * 32) << 16);
    const bool row_ok = row < n_rows;
    const int my_pos = row_ok ? positions[tok0 + row / G] : -1;
    const int my_lo = window > 0 ? max(my_pos - window + 1, k_begin) : k_begin;
    float m_run = -CUDART_INF_F, l_run = 0.f;  // the maximum in use (exponent's unit) and the sum against it
    bool alive = true;
    if (n_tiles > 0) {
      // this thread's query row -> shared memory, swizzled (rows beyond the tile are zero)
      const bf16* src = q + (static_cast<size_t>(tok0 + row / G) * Hq + hk * G + row % G) * DH;
#pragma unroll
      for (int c = 0; c < DH / 8; ++c) {
        const uint4 v = row_ok ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(sQ + (c >> 3) * kAtSubBytes + at_swizzled(row, c & 7)) = v;
      }
      fence_proxy_async();
      mbar_arrive(&bar_q);
    }
    for (int j = 0; j < n_tiles; ++j) {
      const int base = first + j * kAtKeys;
      bool ok = mbar_wait(&bar_s, j & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) give_up(15);
        alive = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      // the whole row of S into registers, then the tensor memory is free for the next S
      unsigned v[kAtKeys];
#pragma unroll
      for (int c = 0; c < kAtKeys / 32; ++c) tmem_ld32(lane_base + c * 32, v + c * 32);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      mbar_arrive(&bar_sfree);
      // a tile that every row of the block may read in full needs no mask
      const bool full = base >= k_begin && base + kAtKeys <= k_end && base + kAtKeys - 1 <= pos_min &&
                        (window <= 0 || base >= pos_max - window + 1);
      if (!full) {
#pragma unroll
        for (int e = 0; e < kAtKeys; ++e) {
          const int key = base + e;
          if (!(key <= my_pos && key >= my_lo && key < k_end)) v[e] = __float_as_uint(-CUDART_INF_F);
        }
      }
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int e = 0; e < kAtKeys; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(v[e]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;  // scale > 0
      // raise the maximum in use only when the row's maximum has run ahead of it by more than kAtLazy
      float alpha = 1.f;
      if (mx > m_run + kAtLazy || m_run == -CUDART_INF_F) {
        if (mx != -CUDART_INF_F) {
          alpha = at_ex2(m_run - mx);  // 0 for the first visible tile
          m_run = mx;
        }
      }
      const bool rescale = j > 0 && alpha != 1.f;
      if (j > 0) {
        // P V_{j-1} must have finished: it read the P tile that is written below, and it wrote O
        ok = mbar_wait(&bar_pv, (j - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) give_up(15);
          alive = false;
          break;
        }
      }
      if (__any_sync(0xffffffffu, rescale)) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) {
          unsigned ov[32];
          tmem_ld32(lane_base + kAtKeys + c * 32, ov);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
          for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
          tmem_st32(lane_base + kAtKeys + c * 32, ov);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
      }
      l_run *= alpha;
      const float mu = (m_run == -CUDART_INF_F) ? 0.f : m_run;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c8 = 0; c8 < kAtKeys / 8; ++c8) {
        float p[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          p[e] = at_ex2(fmaf(__uint_as_float(v[c8 * 8 + e]), scale_log2, -mu));  // masked: ex2(-inf) = 0
          sum4[e & 3] += p[e];
        }
        uint4 pk;
        pk.x = at_pack(p[0], p[1]);
        pk.y = at_pack(p[2], p[3]);
        pk.z = at_pack(p[4], p[5]);
        pk.w = at_pack(p[6], p[7]);
        *reinterpret_cast<uint4*>(sP + (c8 >> 3) * (kAtPBytes / 2) + at_swizzled(row, c8 & 7)) = pk;
      }
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      fence_proxy_async();
      mbar_arrive(&bar_p);
    }

    // ---- this block's result: O from tensor memory once the last product has finished
    constexpr float kLn2 = 0.6931471805599453f;
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) o[i] = 0.f;
    if (alive && n_tiles > 0) {
      bool ok = mbar_wait(&bar_pv, (n_tiles - 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) give_up(15);
        alive = false;
      } else {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) {
          unsigned ov[32];
          tmem_ld32(lane_base + kAtKeys + c * 32, ov);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
          for (int e = 0; e < 32; ++e) o[c * 32 + e] = __uint_as_float(ov[e]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      }
    }
    if (row_ok && alive && !s_abort) {
      const int t = tok0 + row / G, hq = hk * G + row % G;
      if (n_splits == 1) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        bf16* dst = out + (static_cast<size_t>(t) * Hq + hq) * DH;
#pragma unroll
        for (int c = 0; c < DH / 8; ++c) {
          uint4 pk;
          pk.x = at_pack(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv);
          pk.y = at_pack(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
          pk.z = at_pack(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv);
          pk.w = at_pack(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
          *reinterpret_cast<uint4*>(dst + c * 8) = pk;
        }
      } else {
        const size_t pi = (static_cast<size_t>(t) * Hq + hq) * n_splits + z;
        float* dst = part_o + pi * DH;
#pragma unroll
        for (int c = 0; c < DH / 4; ++c)
          *reinterpret_cast<float4*>(dst + c * 4) = make_float4(o[c * 4], o[c * 4 + 1], o[c * 4 + 2], o[c * 4 + 3]);
        *reinterpret_cast<float2*>(part_ml + pi * 2) = make_float2(m_run * kLn2, l_run);
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kAtTmemCols) : "memory");
  }

  // The block that finishes a row tile's last key split merges all of them (the counter returns
  // to zero for the next use).
  if (n_splits > 1) {
    __threadfence();
    __syncthreads();
    int* counter = split_counter + static_cast<size_t>(tile_id) * gridDim.y + hk;
    if (tid == 0) s_last = (atomicAdd(counter, 1) == n_splits - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) *counter = 0;
    constexpr int C4 = DH / 4;
    constexpr int kBatch = 8;
    for (int i = tid; i < n_rows * C4; i += kAtThreads) {
      const int r = i / C4, d = (i % C4) * 4;
      const int t = tok0 + r / G, hq = hk * G + r % G;
      const size_t orow = static_cast<size_t>(t) * Hq + hq;
      const float2* ml = reinterpret_cast<const float2*>(part_ml + orow * n_splits * 2);
      const float* po = part_o + orow * n_splits * DH + d;
      float mx = -CUDART_INF_F, tot = 0.f;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int z0 = 0; z0 < n_splits; z0 += kBatch) {
        float2 v[kBatch];
        float4 x[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const int zz = min(z0 + u, n_splits - 1);
          v[u] = __ldcg(ml + zz);
          x[u] = __ldcg(reinterpret_cast<const float4*>(po + static_cast<size_t>(zz) * DH));
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          if (z0 + u < n_splits && v[u].y > 0.f) {
            const float mn = fmaxf(mx, v[u].x);
            const float keep = expf(mx - mn), w = expf(v[u].x - mn);  // mx = -inf: keep = 0
            a.x = a.x * keep + w * x[u].x;
            a.y = a.y * keep + w * x[u].y;
            a.z = a.z * keep + w * x[u].z;
            a.w = a.w * keep + w * x[u].w;
            tot = tot * keep + w * v[u].y;
            mx = mn;
          }
        }
      }
      const float inv = tot > 0.f ? 1.f / tot : 0.f;
      uint2 packed;
      packed.x = at_pack(a.x * inv, a.y * inv);
      packed.y = at_pack(a.z * inv, a.w * inv);
      *reinterpret_cast<uint2*>(out + orow * DH + d) = packed;
    }
  }
}

}  // namespace pmm

// Whether the tcgen05 attention takes this shape: head size 64 or 128, up to 64 query heads per
// key/value head (a tile holds floor(128 / group) tokens; with a group size that does not divide
// 128 its last rows stay empty), pages that hold whole boxes of 64 keys.
PMM_EXPORT int pmm_attention_tc_supported(int Hq, int Hkv, int Dh, int page_size) {
  if (Hkv <= 0 || Hq % Hkv) return 0;
  const int G = Hq / Hkv;
  return ((Dh == 64 || Dh == 128) && G <= 64 && page_size > 0 && page_size % pmm::kAtBox == 0) ? 1 : 0;
}

// q [T, Hq*64] rotated queries; pool [n_pages + spare, 2, page_size, Hkv*64]; n_tiles = sum over
// sequences of ceil(new tokens / (128 / G)).  Several key splits need part_o / part_ml and
// split_counter (n_tiles * Hkv ints, zero between calls; at most 64 splits, split_len a multiple
// of 64).  status: one int, stays 0 unless a bounded wait gave up.
PMM_EXPORT int pmm_attention_tc(const void* q, const void* pool, long long pool_pages, const int* block_table,
                                int max_blocks, const int* positions, const int* cu, void* out, float* part_o,
                                float* part_ml, float scale, int window, int split_len, int n_splits, int page_size,
                                int n_seq, int n_tiles, int Hq, int Hkv, int Dh, int* split_counter, int* status,
                                cudaStream_t stream) {
  if (n_seq <= 0 || n_tiles <= 0) return 0;
  if (!pmm_attention_tc_supported(Hq, Hkv, Dh, page_size) || !status || !(scale > 0.f) || n_splits < 1 ||
      n_splits > 64 || Hkv > 65535 || pool_pages <= 0 || reinterpret_cast<uintptr_t>(pool) % 16 ||
      reinterpret_cast<uintptr_t>(q) % 16 || reinterpret_cast<uintptr_t>(out) % 16)
    return PMM_ERR_BAD_ARGUMENT;
  if (n_splits > 1 && (!part_o || !part_ml || !split_counter || split_len <= 0 || split_len % pmm::kAtBox))
    return PMM_ERR_BAD_ARGUMENT;
  if (n_splits == 1) split_len = 0x40000000;
  // the whole pool as a matrix [pages * 2 * page_size, Hkv * head size]; a box is 64 rows x 64 columns
  pmm::EncodeTiledFn fn = pmm::encode_tiled_fn();
  if (!fn) return PMM_ERR_BAD_ARGUMENT;
  CUtensorMap map;
  const long long kv_dim = static_cast<long long>(Hkv) * Dh;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(kv_dim), static_cast<cuuint64_t>(pool_pages * 2 * page_size)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(kv_dim) * 2};
  const cuuint32_t box[2] = {pmm::kAtDhBlock, pmm::kAtBox};
  const cuuint32_t elem[2] = {1, 1};
  if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return PMM_ERR_BAD_ARGUMENT;
  auto kern = Dh == 64 ? pmm::attention_tc_kernel<64> : pmm::attention_tc_kernel<128>;
  const size_t smem = pmm::at_smem(Dh);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(n_tiles, Hkv, n_splits);
  pmm::launch_pdl(kern, grid, dim3(pmm::kAtThreads), smem, stream,
      static_cast<const pmm::bf16*>(q), map, block_table, max_blocks, positions, cu, static_cast<pmm::bf16*>(out), part_o,
      part_ml, scale * 1.4426950408889634f, window, split_len, n_splits, page_size, n_seq, Hq, Hkv, split_counter, status);
  return pmm::launch_status();
}

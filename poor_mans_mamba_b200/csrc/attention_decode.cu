// Decode attention over the paged cache with the copy engine bringing the tiles: every sequence
// brings one token, a block = one sequence, one key/value head (its G = Hq/Hkv query heads are the
// rows of one 16-row mma tile) and one key split.
//
// The mma.sync kernel of attention_mma.cu gathers its K/V tiles with 16-byte cp.async copies: 16
// instructions per thread and tile, issued by the warps that also do the arithmetic, and at long
// contexts the issue of the copies, not the memory, bounds it.  Here a fifth warp requests each
// tile of 64 keys with one TMA box per 64 columns (the pool is one matrix [pages * 2 * page_size,
// Hkv * Dh]; a tile lies inside one page because the page size is a multiple of 64) into a ring of
// stages with a full and an empty mbarrier each, and runs ahead of the four compute warps as far
// as the ring allows.  The boxes land with the 128-byte swizzle (16-byte piece c of row r sits at
// piece c ^ (r & 7)), which is what keeps ldmatrix free of bank conflicts without padding.
// The four warps share every tile, warp w taking its keys 16w .. 16w+15 (own running maximum and
// sum, merged at the end), so a tile is used up quickly and the ring stays ahead.
//
// As in the cp.async form the block scales and rotates its query rows itself, and the block whose
// key range holds the new position rotates the new key, writes key and value into the cache page
// and patches them into its tile once that has landed (the copy may have read the page before the
// write); rows of a tile outside the block's key range are zeroed there (values of another request
// may be anything, and 0 * NaN is NaN).
//   x' = x*scale;  ang = float(pos) * inv_freq[i];
//   x'[i] <- x'[i] cos - x'[i+Dh/2] sin;  x'[i+Dh/2] <- x'[i+Dh/2] cos + x'[i] sin
//   sc[s] = (q.K[s]) * scale;  p = exp(sc - max);  o = sum p V / sum p
// (reference src/ops/gpu/attention.cu:4-40 and :44-105), keys lo..pos, lo from the window.
// Several key splits of a (sequence, head) are merged without a second launch.  Up to 16 splits run
// as one thread-block cluster: every block writes its (maximum, sum, unnormalised output) into the
// first block's shared memory and arrives on a barrier there; the first block merges and stores.
// More splits (or results too large for that buffer) go through global memory and a counter: the
// block that finishes the last split merges them.
// Every mbarrier wait is bounded; a wait that gives up writes a code (31: a tile never landed,
// 32: a stage never came free, 33: another block's result never came) to *status, and the step's
// results are discarded by the host.
#include "mma_helpers.cuh"
#include "tcgen05.cuh"
#include <math_constants.h>

namespace pmm {

constexpr int kDaKeys = 64;      // keys per tile = rows of a box
constexpr int kDaBoxCols = 64;   // columns per box: one 128-byte swizzle row
constexpr int kDaThreads = 160;  // warps 0..3 compute, warp 4 requests the tiles
constexpr int kDaBtCap = 512;    // block-table entries of the block's key range kept in shared memory

__host__ __device__ constexpr int da_stages(int dh) { return dh > 64 ? 3 : 4; }
__host__ __device__ constexpr size_t da_smem(int dh) {
  return 1024 /*alignment*/ + static_cast<size_t>(2 * da_stages(dh)) * kDaKeys * dh * 2 + 16 * (dh + 8) * 2;
}
// what the first block of a cluster receives: (splits - 1) x G rows of (Dh values, maximum, sum)
__host__ __device__ constexpr size_t da_parts_bytes(int dh, int G, int n_splits) {
  return static_cast<size_t>(n_splits - 1) * G * (dh + 2) * sizeof(float);
}
constexpr size_t kDaPartsMax = 24 * 1024;  // (the V ring is 32 KB at head size 64, 48 KB at 128)
constexpr int kDaClusterMax = 16;

struct DecodeAttnArgs {
  const bf16* q;          // [n_seq, ldq] unrotated queries
  long long ldq;
  const bf16* k;          // [n_seq, ldk] new keys, or nullptr: the cache holds them already
  long long ldk;
  const bf16* v;
  long long ldv;
  float q_scale, k_scale, v_scale;
  const float* inv_freq;  // [Dh/2], or nullptr: no rotation
  bf16* pool;             // the cache, writable
  const int* block_table;
  int max_blocks;
  const int* positions;
  bf16* out;
  float* part_o;
  float* part_ml;
  float scale_log2;
  int window, split_len, n_splits, page_size, Hq, Hkv;
  int* split_counter;
  int* status;
  int clustered;          // the key splits of a (sequence, head) are one cluster (gridDim.z blocks)
};

// Address of a shared-memory location of this block in block `rank` of the cluster.
__device__ __forceinline__ unsigned cluster_addr(unsigned smem_addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(unsigned addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}
// Arrival on a barrier of another block of the cluster; this thread's earlier writes into that
// block's shared memory are visible to whoever has waited for the barrier.
__device__ __forceinline__ void mbar_arrive_remote(unsigned cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_bar) : "memory");
}
// Bounded wait on a barrier of this block on which other blocks of the cluster arrive.
__device__ __forceinline__ bool mbar_wait_cluster(unsigned long long* bar, unsigned parity, volatile int* abort_flag) {
  for (unsigned i = 0; i < kSpinLimit; ++i) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if (abort_flag && (i & 63) == 63 && *abort_flag) return false;
  }
  return false;
}

template <int DH>
__global__ void __launch_bounds__(kDaThreads)
    decode_attention_kernel(const __grid_constant__ CUtensorMap map_kv, const DecodeAttnArgs a) {
  constexpr int KT = kDaKeys;
  constexpr int NSTAGE = da_stages(DH);
  constexpr int SUB = DH / kDaBoxCols;       // boxes per tile
  constexpr int BOX = KT * kDaBoxCols * 2;   // 8 KB
  constexpr int TILE = SUB * BOX;
  constexpr int QSTRIDE = DH + 8;
  constexpr int KS_Q = DH / 16;
  constexpr int NT_O = DH / 8;
  constexpr int HALF = DH / 2;
  constexpr int CHUNKS = DH / 8;             // 16-byte pieces per row

  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[NSTAGE], bar_empty[NSTAGE], bar_parts;
  __shared__ int s_bt[kDaBtCap];
  __shared__ __align__(16) bf16 s_new_k[DH], s_new_v[DH];
  __shared__ float s_wm[4][16], s_wl[4][16], s_M[16], s_L[16];
  __shared__ int s_abort, s_last;

  // Positions and block tables are inputs of the step, written before its first kernel: they are
  // read before the wait for the kernel before this one.
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = a.Hq / a.Hkv;
  const int seq = blockIdx.x, hk = blockIdx.y, z = blockIdx.z;
  const int kv_dim = a.Hkv * DH;
  const int page_size = a.page_size;
  const int pos = a.positions[seq];
  const int lo_all = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int k_begin = max(lo_all, z * a.split_len);
  const int k_end = min(pos + 1, (z + 1) * a.split_len);
  const int first_tile = (k_begin / KT) * KT;
  const int n_tiles = k_end > k_begin ? (k_end - first_tile + KT - 1) / KT : 0;
  const int* bt = a.block_table + static_cast<size_t>(seq) * a.max_blocks;

  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = ring;
  unsigned char* sV = ring + NSTAGE * TILE;
  bf16* sQ = reinterpret_cast<bf16*>(ring + 2 * NSTAGE * TILE);
  float* sParts = reinterpret_cast<float*>(sV);  // (clustered, in the first block, once every block's tiles are done) [split - 1][G][DH + 2]

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 4);
    }
    mbar_init(&bar_parts, 128 * (a.n_splits > 1 ? a.n_splits - 1 : 1));
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  // (clustered) every block has its barrier ready before another block arrives on it: the arrival
  // is here, the wait before the first access to the first block's shared memory
  if (a.clustered) asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");
  volatile int* abort_flag = &s_abort;
  auto give_up = [&](int code) {
    if (!*abort_flag) atomicExch(a.status, code);
    s_abort = 1;
  };
  // the new token: this block stores its key and value if its key range holds the position
  const bool stores_new = a.k != nullptr && n_tiles > 0 && pos >= k_begin && pos < k_end;

  if (warp == 4) {
    // ---------------------------------------------------------------- the tiles' requests
    // A layer that reads another layer's cache finds this step's key there: written by a kernel
    // of this step.  Otherwise the keys of earlier positions depend on nothing in this step.
    if (a.k == nullptr) pdl_wait();
    if (n_tiles > 0) {
      if (lane == 0) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<unsigned long long>(&map_kv)) : "memory");
      const int bt_lo = first_tile / page_size;
      const int n_bt = (k_end - 1) / page_size - bt_lo + 1;
      for (int i = lane; i < min(n_bt, kDaBtCap); i += 32) s_bt[i] = bt[bt_lo + i];
      __syncwarp();
      auto request = [&](int j) {  // one lane: tile j into its stage
        const int s = j % NSTAGE, base = first_tile + j * KT;
        const int idx = base / page_size - bt_lo;
        const int page = idx < kDaBtCap ? s_bt[idx] : bt[bt_lo + idx];
        const int row = page * 2 * page_size + base % page_size;
        mbar_expect_tx(&bar_full[s], 2 * TILE);
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub) {
          tma_load_2d(sK + s * TILE + sub * BOX, &map_kv, hk * DH + sub * kDaBoxCols, row, &bar_full[s]);
          tma_load_2d(sV + s * TILE + sub * BOX, &map_kv, hk * DH + sub * kDaBoxCols, row + page_size, &bar_full[s]);
        }
      };
      // the first filling: a lane per stage (a request costs its thread some hundred cycles)
      const int first = min(NSTAGE, n_tiles);
      if (lane < first) request(lane);
      int issued = first;
      for (int j = first; j < n_tiles; ++j) {
        int ok = 1;
        if (lane == 0) ok = mbar_wait(&bar_empty[j % NSTAGE], ((j / NSTAGE) & 1) ^ 1, abort_flag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0) give_up(32);
          break;
        }
        if (lane == 0) request(j);
        issued = j + 1;
      }
      if (lane == 0 && s_abort) {
        // copies already requested still write into this block's shared memory: wait for them
        for (int j = issued > NSTAGE ? issued - NSTAGE : 0; j < issued; ++j)
          for (unsigned n = 0; n < kSpinLimit && !mbar_try_wait(&bar_full[j % NSTAGE], (j / NSTAGE) & 1); ++n) {
          }
      }
    }
    return;  // (the compute warps synchronise among themselves from here on)
  }

  // ------------------------------------------------------------------ the four compute warps
  auto sync_compute = [&]() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); };
  // byte offset of 16-byte piece c (0 .. Dh/8-1) of row r inside a tile
  auto piece = [&](int r, int c) { return (c >> 3) * BOX + r * 128 + (((c & 7) ^ (r & 7)) << 4); };

  pdl_wait();  // the projections come from the kernel before this one
  if (stores_new) {
    const int page = bt[pos / page_size];
    bf16* k_dst = a.pool + (static_cast<size_t>(page) * 2 * page_size + pos % page_size) * kv_dim + hk * DH;
    bf16* v_dst = k_dst + static_cast<size_t>(page_size) * kv_dim;
    const bf16* ksrc = a.k + static_cast<long long>(seq) * a.ldk + hk * DH;
    const bf16* vsrc = a.v + static_cast<long long>(seq) * a.ldv + hk * DH;
    for (int i = tid; i < HALF; i += 128) {
      const float x1 = __bfloat162float(ksrc[i]) * a.k_scale, x2 = __bfloat162float(ksrc[i + HALF]) * a.k_scale;
      float o1 = x1, o2 = x2;
      if (a.inv_freq) {
        const float ang = static_cast<float>(pos) * a.inv_freq[i];
        const float c = cosf(ang), sn = sinf(ang);
        o1 = x1 * c - x2 * sn;
        o2 = x2 * c + x1 * sn;
      }
      const bf16 b1 = __float2bfloat16_rn(o1), b2 = __float2bfloat16_rn(o2);
      k_dst[i] = b1;
      k_dst[i + HALF] = b2;
      s_new_k[i] = b1;
      s_new_k[i + HALF] = b2;
    }
    for (int i = tid; i < DH; i += 128) {
      const bf16 b = __float2bfloat16_rn(__bfloat162float(vsrc[i]) * a.v_scale);
      v_dst[i] = b;
      s_new_v[i] = b;
    }
  }
  if (n_tiles > 0) {  // the query rows, scaled and rotated; rows beyond the group are zero
    for (int idx = tid; idx < 16 * HALF; idx += 128) {
      const int r = idx / HALF, i = idx % HALF;
      float o1 = 0.f, o2 = 0.f;
      if (r < G) {
        const bf16* src = a.q + static_cast<long long>(seq) * a.ldq + (hk * G + r) * DH;
        const float x1 = __bfloat162float(src[i]) * a.q_scale, x2 = __bfloat162float(src[i + HALF]) * a.q_scale;
        o1 = x1;
        o2 = x2;
        if (a.inv_freq) {
          const float ang = static_cast<float>(pos) * a.inv_freq[i];
          const float c = cosf(ang), sn = sinf(ang);
          o1 = x1 * c - x2 * sn;
          o2 = x2 * c + x1 * sn;
        }
      }
      sQ[r * QSTRIDE + i] = __float2bfloat16_rn(o1);
      sQ[r * QSTRIDE + i + HALF] = __float2bfloat16_rn(o2);
    }
  }
  sync_compute();

  const int r_lo = lane >> 2, r_hi = r_lo + 8;
  float m_lo = -CUDART_INF_F, m_hi = -CUDART_INF_F, l_lo = 0.f, l_hi = 0.f;  // maxima in the exponent's unit
  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  unsigned qf[KS_Q][4];
  if (n_tiles > 0) {
#pragma unroll
    for (int ks = 0; ks < KS_Q; ++ks)
      ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                  sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * QSTRIDE + ks * 16 + (lane >> 4) * 8);
  }
  // this lane's rows of the K and V fragments of the warp's 16 keys (swizzle term: row & 7 == lane & 7)
  const int row_k = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
  const int row_v = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
  const float scale_log2 = a.scale_log2;

  for (int it = 0; it < n_tiles; ++it) {
    const int s = it % NSTAGE, base = first_tile + it * KT;
    const bool landed = mbar_wait(&bar_full[s], (it / NSTAGE) & 1, abort_flag);
    if (!landed) {  // (every warp waits on the same barrier: all of them leave)
      if (lane == 0) give_up(31);
      break;
    }
    unsigned char* tK = sK + s * TILE;
    unsigned char* tV = sV + s * TILE;
    const bool last = it == n_tiles - 1;
    if (base < k_begin || base + KT > k_end || (stores_new && last)) {
      // rows outside the key range hold whatever the page holds: their values become zero (their
      // scores are masked); the new token's row comes from this block's own registers' work
      for (int idx = tid; idx < KT * CHUNKS; idx += 128) {
        const int r = idx / CHUNKS, c = idx % CHUNKS;
        if (base + r < k_begin || base + r >= k_end) *reinterpret_cast<uint4*>(tV + piece(r, c)) = make_uint4(0u, 0u, 0u, 0u);
      }
      if (stores_new && last && tid < 2 * CHUNKS) {
        const int r = pos - base, c = tid % CHUNKS;
        if (tid < CHUNKS)
          *reinterpret_cast<uint4*>(tK + piece(r, c)) = *reinterpret_cast<const uint4*>(s_new_k + c * 8);
        else
          *reinterpret_cast<uint4*>(tV + piece(r, c)) = *reinterpret_cast<const uint4*>(s_new_v + c * 8);
      }
      sync_compute();
    }

    const int kbase = base + warp * 16;
    if (kbase < k_end && kbase + 16 > k_begin) {  // some of this warp's keys are wanted
      float sc[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS_Q; ++ks) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3,
                    tK + (ks >> 2) * BOX + row_k * 128 + (((((ks & 3) << 1) + ((lane >> 3) & 1)) ^ (lane & 7)) << 4));
        mma_bf16(sc[0], qf[ks], b0, b1);
        mma_bf16(sc[1], qf[ks], b2, b3);
      }
      unsigned bv[NT_O / 2][4];  // the V fragments travel while the softmax is computed
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np)
        ldmatrix_x4_trans(bv[np][0], bv[np][1], bv[np][2], bv[np][3],
                          tV + (np >> 2) * BOX + row_v * 128 + (((((np & 3) << 1) + (lane >> 4)) ^ (lane & 7)) << 4));
      if (kbase < k_begin || kbase + 16 > k_end) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = kbase + nt * 8 + (lane & 3) * 2 + (e & 1);
            if (key < k_begin || key >= k_end) sc[nt][e] = -CUDART_INF_F;
          }
        }
      }
      float mx_lo = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
      float mx_hi = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo * scale_log2), mn_hi = fmaxf(m_hi, mx_hi * scale_log2);  // scale > 0
      const float mu_lo = (mn_lo == -CUDART_INF_F) ? 0.f : mn_lo;
      const float mu_hi = (mn_hi == -CUDART_INF_F) ? 0.f : mn_hi;
      const float al_lo = ex2_approx(m_lo - mu_lo), al_hi = ex2_approx(m_hi - mu_hi);
      m_lo = mn_lo;
      m_hi = mn_hi;
      unsigned pa[4];  // P as bfloat16 A fragment
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float p0 = ex2_approx(fmaf(sc[nt][0], scale_log2, -mu_lo));
        const float p1 = ex2_approx(fmaf(sc[nt][1], scale_log2, -mu_lo));
        const float p2 = ex2_approx(fmaf(sc[nt][2], scale_log2, -mu_hi));
        const float p3 = ex2_approx(fmaf(sc[nt][3], scale_log2, -mu_hi));
        sum_lo += p0 + p1;
        sum_hi += p2 + p3;
        pa[nt * 2] = pack_bf16(p0, p1);
        pa[nt * 2 + 1] = pack_bf16(p2, p3);
      }
      l_lo = l_lo * al_lo + sum_lo;
      l_hi = l_hi * al_hi + sum_hi;
      if (__any_sync(0xffffffffu, al_lo != 1.f || al_hi != 1.f)) {  // some row's maximum moved
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
          o[i][0] *= al_lo;
          o[i][1] *= al_lo;
          o[i][2] *= al_hi;
          o[i][3] *= al_hi;
        }
      }
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {
        mma_bf16(o[2 * np], pa, bv[np][0], bv[np][1]);
        mma_bf16(o[2 * np + 1], pa, bv[np][2], bv[np][3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&bar_empty[s]);  // this warp is done with the stage
  }
  sync_compute();  // every warp is done with the ring (it is reused below)
  if (a.clustered) {
    // Second round of the cluster barrier: this block's tiles are done (all of them have landed and
    // been used: nothing writes into its ring any more).  Behind it the first block's V ring takes
    // the other blocks' results.
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");
  }

  constexpr float kLn2 = 0.6931471805599453f;
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  // merge the four warps (each saw a quarter of the keys) through shared memory
  constexpr int SO = DH + 4;                 // padded row: rows g and g+1 fall into different banks
  float* sO = reinterpret_cast<float*>(sK);  // [4 warps][16][SO]; a gave-up block may still have copies in
  if (*abort_flag) {                         // flight into the ring: it leaves its part unwritten
    // (clustered) the first block stays until the others have sent: its shared memory must outlive their writes
    if (a.clustered && z == 0) {
      asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
      mbar_wait_cluster(&bar_parts, 0, nullptr);
    }
    return;  // (a block that gave up has arrived twice like every other: nobody waits for it)
  }
  if ((lane & 3) == 0) {
    s_wm[warp][r_lo] = m_lo;
    s_wm[warp][r_hi] = m_hi;
    s_wl[warp][r_lo] = l_lo;
    s_wl[warp][r_hi] = l_hi;
  }
  sync_compute();
  if (tid < 16) {
    float mm = -CUDART_INF_F;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_wm[w][tid]);
    const float mu = (mm == -CUDART_INF_F) ? 0.f : mm;
    float ll = 0.f;
    for (int w = 0; w < 4; ++w) ll += s_wl[w][tid] * exp2f(s_wm[w][tid] - mu);
    s_M[tid] = mm;
    s_L[tid] = ll;
  }
  sync_compute();
  {
    const float mu_lo = (s_M[r_lo] == -CUDART_INF_F) ? 0.f : s_M[r_lo];
    const float mu_hi = (s_M[r_hi] == -CUDART_INF_F) ? 0.f : s_M[r_hi];
    const float f_lo = exp2f(m_lo - mu_lo), f_hi = exp2f(m_hi - mu_hi);
    float* mine = sO + warp * 16 * SO;
#pragma unroll
    for (int nt = 0; nt < NT_O; ++nt) {
      const int d = nt * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(mine + r_lo * SO + d) = make_float2(o[nt][0] * f_lo, o[nt][1] * f_lo);
      *reinterpret_cast<float2*>(mine + r_hi * SO + d) = make_float2(o[nt][2] * f_hi, o[nt][3] * f_hi);
    }
  }
  sync_compute();
  const int n_splits = a.n_splits;
  if (a.clustered) {
    // ---- the splits of this (sequence, head) are one cluster: block z sends its part to block 0
    constexpr int PW = DH + 2;  // a row of a part: Dh values, maximum (exponent's unit), sum
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");  // every block's tiles are done
    if (z > 0) {
      const unsigned dst = cluster_addr(smem_u32(sParts), 0) + static_cast<unsigned>((z - 1) * G * PW) * 4u;
      for (int i = tid; i < G * DH; i += 128) {
        const int r = i / DH, d = i % DH;
        const float sum = (sO[r * SO + d] + sO[(16 + r) * SO + d]) + (sO[(32 + r) * SO + d] + sO[(48 + r) * SO + d]);
        st_cluster_f32(dst + static_cast<unsigned>(r * PW + d) * 4u, sum);
        if (d == 0) {
          st_cluster_f32(dst + static_cast<unsigned>(r * PW + DH) * 4u, s_M[r]);
          st_cluster_f32(dst + static_cast<unsigned>(r * PW + DH + 1) * 4u, s_L[r]);
        }
      }
      mbar_arrive_remote(cluster_addr(smem_u32(&bar_parts), 0));  // releases this thread's writes above
      return;
    }
    // block 0: its own part is in sO / s_M / s_L; the others arrive in sParts
    if (!mbar_wait_cluster(&bar_parts, 0, abort_flag)) {
      if (lane == 0) give_up(33);
      return;
    }
    for (int i = tid; i < G * (DH / 2); i += 128) {  // a thread per (row, two columns)
      const int r = i / (DH / 2), d = (i % (DH / 2)) * 2;
      float mx = s_M[r];
      for (int p = 0; p < n_splits - 1; ++p) mx = fmaxf(mx, sParts[(p * G + r) * PW + DH]);
      const float mu = (mx == -CUDART_INF_F) ? 0.f : mx;
      float w = exp2f(s_M[r] - mu);  // (-inf - 0 -> 0: a part without keys)
      float tot = w * s_L[r];
      float a0 = w * ((sO[r * SO + d] + sO[(16 + r) * SO + d]) + (sO[(32 + r) * SO + d] + sO[(48 + r) * SO + d]));
      float a1 = w * ((sO[r * SO + d + 1] + sO[(16 + r) * SO + d + 1]) + (sO[(32 + r) * SO + d + 1] + sO[(48 + r) * SO + d + 1]));
      for (int p = 0; p < n_splits - 1; ++p) {
        const float* part = sParts + (p * G + r) * PW;
        w = exp2f(part[DH] - mu);
        tot += w * part[DH + 1];
        a0 += w * part[d];
        a1 += w * part[d + 1];
      }
      const float inv = tot > 0.f ? 1.f / tot : 0.f;
      *reinterpret_cast<__nv_bfloat162*>(a.out + (static_cast<size_t>(seq) * a.Hq + hk * G + r) * DH + d) =
          __floats2bfloat162_rn(a0 * inv, a1 * inv);
    }
    return;
  }
  for (int i = tid; i < G * DH; i += 128) {
    const int r = i / DH, d = i % DH;
    const int hq = hk * G + r;
    const float sum = (sO[r * SO + d] + sO[(16 + r) * SO + d]) + (sO[(32 + r) * SO + d] + sO[(48 + r) * SO + d]);
    if (n_splits == 1) {
      const float l = s_L[r];
      a.out[(static_cast<size_t>(seq) * a.Hq + hq) * DH + d] = __float2bfloat16_rn(l > 0.f ? sum / l : 0.f);
    } else {
      const size_t pi = (static_cast<size_t>(seq) * a.Hq + hq) * n_splits + z;
      a.part_o[pi * DH + d] = sum;
      if (d == 0) {
        a.part_ml[pi * 2] = s_M[r] * kLn2;
        a.part_ml[pi * 2 + 1] = s_L[r];
      }
    }
  }
  if (n_splits == 1) return;

  // The block that finishes a (sequence, head)'s last key split merges all of them, so no second
  // launch is needed.  The counter returns to zero for the next use.
  __threadfence();
  sync_compute();
  int* counter = a.split_counter + static_cast<size_t>(seq) * gridDim.y + hk;
  if (tid == 0) s_last = (atomicAdd(counter, 1) == n_splits - 1);
  sync_compute();
  if (!s_last) return;
  __threadfence();
  if (tid == 0) *counter = 0;
  // A thread per (row, four columns) merges the splits in one pass with a running maximum,
  // sixteen splits' loads in flight at a time.
  constexpr int C4 = DH / 4;
  constexpr int kBatch = 16;
  for (int i = tid; i < G * C4; i += 128) {
    const int r = i / C4, d = (i % C4) * 4;
    const size_t rowi = static_cast<size_t>(seq) * a.Hq + hk * G + r;
    const float2* ml = reinterpret_cast<const float2*>(a.part_ml + rowi * n_splits * 2);
    const float* po = a.part_o + rowi * n_splits * DH + d;
    float mx = -CUDART_INF_F, tot = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
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
          acc.x = acc.x * keep + w * x[u].x;
          acc.y = acc.y * keep + w * x[u].y;
          acc.z = acc.z * keep + w * x[u].z;
          acc.w = acc.w * keep + w * x[u].w;
          tot = tot * keep + w * v[u].y;
          mx = mn;
        }
      }
    }
    const float inv = tot > 0.f ? 1.f / tot : 0.f;
    uint2 packed;
    packed.x = pack_bf16(acc.x * inv, acc.y * inv);
    packed.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(a.out + rowi * DH + d) = packed;
  }
}

template <int DH>
int launch_decode_attention(const CUtensorMap& map, DecodeAttnArgs a, int n_seq, cudaStream_t stream) {
  auto kern = decode_attention_kernel<DH>;
  const int G = a.Hq / a.Hkv;
  // the key splits as one cluster where they are few enough and their results fit beside the ring
  const size_t parts = a.n_splits > 1 ? (da_parts_bytes(DH, G, a.n_splits) + 15) / 16 * 16 : 0;
  a.clustered = a.n_splits > 1 && a.n_splits <= kDaClusterMax && parts <= kDaPartsMax ? 1 : 0;
  const size_t smem = da_smem(DH);  // (the results of a cluster's blocks go into the first block's idle V ring)
  static bool attrs_set = false;
  if (!attrs_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return static_cast<int>(e);
    attrs_set = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(n_seq, a.Hkv, a.n_splits);
  cfg.blockDim = dim3(kDaThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  if (a.clustered) {
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = 1;
    attrs[1].val.clusterDim.y = 1;
    attrs[1].val.clusterDim.z = a.n_splits;
    cfg.numAttrs = 2;
    // a cluster this large may not find room (shared memory, blocks of one GPC): then through the counter
    static signed char fits[kDaClusterMax + 1] = {};  // per cluster size: 0 not asked yet, 1 fits, -1 does not
    if (fits[a.n_splits] == 0) {
      int n = 0;
      const bool ok = cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n >= 1;
      if (!ok) (void)cudaGetLastError();
      fits[a.n_splits] = ok ? 1 : -1;
    }
    if (fits[a.n_splits] < 0) {
      a.clustered = 0;
      cfg.numAttrs = 1;
    }
  }
  if (!a.clustered && a.n_splits > 1 && (!a.part_o || !a.part_ml || !a.split_counter)) return PMM_ERR_BAD_ARGUMENT;
  cudaLaunchKernelEx(&cfg, kern, map, a);
  return launch_status();
}

}  // namespace pmm

// Whether pmm_decode_attention_tma takes this shape: head sizes 64 and 128, at most 16 query heads
// per key/value head, pages of a multiple of 64 positions.
PMM_EXPORT int pmm_decode_attention_tma_supported(int Hq, int Hkv, int Dh, int page_size) {
  if (Hkv <= 0 || Hq % Hkv || Hq / Hkv > 16) return 0;
  return ((Dh == 64 || Dh == 128) && page_size > 0 && page_size % pmm::kDaKeys == 0) ? 1 : 0;
}

// Decode step, every sequence one token (token t belongs to sequence t): attention straight from
// the projections, the arguments of pmm_flash_decode_attention plus the number of pages of the
// pool [pool_pages, 2, page_size, Hkv*Dh] and a status word (one int, stays 0 unless a bounded wait
// gave up).  Several key splits need part_o / part_ml and split_counter (n_seq * Hkv ints, zero
// between calls; split_len a multiple of 64, at most 64 splits).
PMM_EXPORT int pmm_decode_attention_tma(const void* q_src, long long ldq, const void* k_src, long long ldk,
                                        const void* v_src, long long ldv, float q_scale, float k_scale, float v_scale,
                                        const float* inv_freq, void* pool, long long pool_pages, const int* block_table,
                                        int max_blocks, const int* positions, void* out, float* part_o, float* part_ml,
                                        float scale, int window, int split_len, int n_splits, int page_size, int n_seq,
                                        int Hq, int Hkv, int Dh, int* split_counter, int* status, cudaStream_t stream) {
  if (n_seq <= 0) return 0;
  if (!pmm_decode_attention_tma_supported(Hq, Hkv, Dh, page_size) || !q_src || (k_src == nullptr) != (v_src == nullptr) ||
      !pool || !block_table || !positions || !out || !status || pool_pages <= 0 || !(scale > 0.f) || n_splits < 1 ||
      n_splits > 64 || Hkv > 65535 || reinterpret_cast<uintptr_t>(pool) % 16 || reinterpret_cast<uintptr_t>(out) % 8)
    return PMM_ERR_BAD_ARGUMENT;
  if (n_splits > 1 && (!part_o || !part_ml || !split_counter || split_len <= 0 || split_len % pmm::kDaKeys))
    return PMM_ERR_BAD_ARGUMENT;
  if (n_splits == 1) split_len = 0x40000000;
  // the whole pool as a matrix [pages * 2 * page_size, Hkv * head size]; a box is 64 rows x 64 columns
  pmm::EncodeTiledFn fn = pmm::encode_tiled_fn();
  if (!fn) return PMM_ERR_BAD_ARGUMENT;
  CUtensorMap map;
  const long long kv_dim = static_cast<long long>(Hkv) * Dh;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(kv_dim), static_cast<cuuint64_t>(pool_pages * 2 * page_size)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(kv_dim) * 2};
  const cuuint32_t box[2] = {pmm::kDaBoxCols, pmm::kDaKeys};
  const cuuint32_t elem[2] = {1, 1};
  if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, pool, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return PMM_ERR_BAD_ARGUMENT;
  pmm::DecodeAttnArgs a{};
  a.q = static_cast<const pmm::bf16*>(q_src);
  a.ldq = ldq;
  a.k = static_cast<const pmm::bf16*>(k_src);
  a.ldk = ldk;
  a.v = static_cast<const pmm::bf16*>(v_src);
  a.ldv = ldv;
  a.q_scale = q_scale;
  a.k_scale = k_scale;
  a.v_scale = v_scale;
  a.inv_freq = inv_freq;
  a.pool = static_cast<pmm::bf16*>(pool);
  a.block_table = block_table;
  a.max_blocks = max_blocks;
  a.positions = positions;
  a.out = static_cast<pmm::bf16*>(out);
  a.part_o = part_o;
  a.part_ml = part_ml;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.split_len = split_len;
  a.n_splits = n_splits;
  a.page_size = page_size;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.split_counter = split_counter;
  a.status = status;
  return Dh == 64 ? pmm::launch_decode_attention<64>(map, a, n_seq, stream)
                  : pmm::launch_decode_attention<128>(map, a, n_seq, stream);
}

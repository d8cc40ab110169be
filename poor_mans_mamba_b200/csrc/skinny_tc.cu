// Weight-streaming matrix product for steps of up to 64 tokens on the fifth-generation tensor cores:
//   y[T, N] = x[T, K] W[N, K]^T, bfloat16 operands, float accumulation,
// with the same epilogues as the mma.sync form for fewer tokens (skinny_gemm.cu): STORE (bfloat16),
// SWIGLU (W = [gate rows; up rows], act = silu(gate * mult) * up) and RESIDUAL (h += scale * y with
// float atomics; two products may share a launch).
// At these sizes the product is a read of W at memory speed, and what bounds a tcgen05 kernel is
// the number of instructions it issues: an instruction takes about a hundred cycles however narrow
// it is.  So the weights are the M side: A = a tile of 128 rows of W, B = x (N = the tokens, rounded
// up to 16), D = 128 lanes (rows of W) x up to 64 float columns (tokens) in tensor memory, and one
// instruction consumes 128 x 16 weights.
//
// A stage of the ring holds 64 columns of K: one box of W (64 columns x 128 rows, 16 KB; SWIGLU: 64
// gate rows and their 64 up rows) and one box of x (64 columns x the tokens, rows beyond T read as
// zero), both with the 128-byte swizzle; eight stages are in flight.  The weight boxes of the first
// filling are requested before the wait for the kernel before this one (programmatic dependent
// launch), the activations behind it.
// Work: a block takes row tiles bx, bx + gridDim.x, ... (two accumulators in turn, so the epilogue
// of a tile overlaps the products of the next) of its K slice blockIdx.y.  Where the row tiles are
// fewer than the SMs, K is cut into slices: RESIDUAL adds every slice to h with atomics; STORE and
// SWIGLU launch the slices of a tile as one thread-block cluster, whose blocks write their partial
// accumulators into the first block's shared memory (the idle ring), which adds them up and stores.
// Warps 0..3 = epilogue (a thread holds its row's outputs of all tokens), 4 = TMA producer,
// 5 = tensor-memory owner and MMA issuer.
// Every mbarrier wait is bounded: on a time-out the waiter writes a code (21..24) to *status,
// raises the block's abort flag, all roles leave their loops, the producer waits (bounded) for its
// copies in flight, the cluster barriers are still passed by every thread and the tensor memory is
// freed.  No cluster multicast.
// (reference: linear layers are cublasSgemm calls, src/ops/gpu/linear.cu:3-21.)
#include "tcgen05.cuh"
#include <algorithm>

namespace pmm {

using bf16 = __nv_bfloat16;

constexpr int kStTok = 64;      // tokens at most = columns of an accumulator
constexpr int kStRows = 128;    // rows of W per tile = lanes of the accumulator
constexpr int kStKB = 64;       // columns of K per box: one 128-byte swizzle row
constexpr int kStStages = 7;
constexpr int kStThreads = 192;
constexpr int kStTmemCols = 2 * kStTok;          // two accumulators
constexpr int kStWBox = kStRows * kStKB * 2;     // 16 KB
constexpr int kStXBox = kStTok * kStKB * 2;      // 8 KB (the box holds n_cols rows of it)
constexpr int kStStageBytes = kStWBox + kStXBox;
constexpr int kStRingBytes = kStStages * kStStageBytes;
constexpr int kStOutBytes = 32 * kStRows * 4;    // the epilogue's staging: 32 tokens x 128 rows of floats
constexpr int kStMaxSplit = 4;                   // blocks of a cluster = K slices of a STORE / SWIGLU tile
// what a block receives from the others of its cluster: (split - 1) senders x ceil(16 / split) groups
// of four tokens x 128 rows x 16 bytes, at most 24 KB (split 3 and 4)
constexpr int kStPartsBytes = 24 * 1024;
constexpr unsigned kStQuadBytes = kStRows * 16;  // a group of four tokens of a tile: 128 rows x float4
constexpr size_t kStSmem = 1024 /*alignment*/ + kStRingBytes + kStOutBytes + kStPartsBytes;
static_assert(kStSmem <= 227 * 1024, "shared memory of a block");

enum { kStStore = 0, kStSwiglu = 1, kStResidual = 2 };

// kind::f16 instruction descriptor without its N: float accumulate, bfloat16 A and B, both K-major, M = 128.
constexpr unsigned kStIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kStRows >> 4) << 24);

struct SkinnyTcArgs {
  int T, N;          // tokens, output columns (SWIGLU: F)
  int n_cols;        // T rounded up to 16: the instruction's N and the rows of the x box
  int n_problems;
  int K[2];
  int k_slice;       // columns of K per block along gridDim.y (a multiple of 64)
  int split;         // blocks per cluster along y (STORE / SWIGLU with K in slices), else 1
  float scale[2];    // RESIDUAL: factor on y; SWIGLU: gate multiplier
  bf16* y;           // STORE / SWIGLU output
  long long ldy;
  float* h_out;      // RESIDUAL target [T, N]
  int* status;
};

__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
// The address of `smem_addr` (a shared-memory address of this block) in block `rank` of the cluster.
__device__ __forceinline__ unsigned cluster_map(unsigned smem_addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// Copies `bytes` (a multiple of 16) of this block's shared memory into another block of the cluster
// (addresses there from cluster_map); the bytes count on the barrier `bar` of that block.
__device__ __forceinline__ void bulk_copy_to_cluster(unsigned dst, unsigned src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "r"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void st_red4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// Bounded wait on a barrier of this block that counts what other blocks of the cluster send.
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
// The four epilogue warps agree (a wait that gave up in one of them ends the tile loop of all).
__device__ __forceinline__ bool epilogue_warps_all(bool ok) {
  unsigned r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(r)
      : "r"(static_cast<unsigned>(ok))
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void epilogue_warps_sync() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

template <int MODE>
__global__ void __launch_bounds__(kStThreads)
    skinny_tc_kernel(const __grid_constant__ CUtensorMap map_x0, const __grid_constant__ CUtensorMap map_w0,
                     const __grid_constant__ CUtensorMap map_x1, const __grid_constant__ CUtensorMap map_w1,
                     const SkinnyTcArgs args) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[kStStages], bar_empty[kStStages], bar_acc_full[2], bar_acc_empty[2], bar_parts;
  __shared__ unsigned s_tmem_base;
  __shared__ int s_abort;
  pdl_launch_dependents();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int prob = blockIdx.z;
  const CUtensorMap* map_x = prob == 0 ? &map_x0 : &map_x1;
  const CUtensorMap* map_w = prob == 0 ? &map_w0 : &map_w1;
  const int K = args.K[prob];
  const int k0 = blockIdx.y * args.k_slice;
  const int k1 = min(K, k0 + args.k_slice);
  const int n_kb = k1 > k0 ? (k1 - k0 + kStKB - 1) / kStKB : 0;   // boxes (= stages) of this block's K slice
  constexpr int kTileCols = MODE == kStSwiglu ? kStRows / 2 : kStRows;  // output columns of a row tile
  constexpr int kSegs = kTileCols / 4;                                  // pieces of four columns per token
  const int n_tx = (args.N + kTileCols - 1) / kTileCols;
  const int my_tiles = static_cast<int>(blockIdx.x) < n_tx ? (n_tx - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;
  const int split = args.split;
  const bool clustered = split > 1;  // then every block has exactly one tile and a K slice with work
  const bool has_work = n_kb > 0 && my_tiles > 0;
  if (!has_work && !clustered) {  // the whole block: a product with a shorter K has nothing in this slice
    pdl_wait();
    return;
  }
  const int total = has_work ? my_tiles * n_kb : 0;  // fillings of ring stages
  const int n_cols = args.n_cols;
  const unsigned x_bytes = static_cast<unsigned>(n_cols) * kStKB * 2;

  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* stage_out = reinterpret_cast<float*>(ring + kStRingBytes);      // [32 tokens][128 rows]: outputs, transposed
  float4* parts = reinterpret_cast<float4*>(ring + kStRingBytes + kStOutBytes);  // what the cluster's other blocks send

  if (threadIdx.x < kStStages) {
    mbar_init(&bar_full[threadIdx.x], 1);
    mbar_init(&bar_empty[threadIdx.x], 1);
    if (threadIdx.x < 2) {
      mbar_init(&bar_acc_full[threadIdx.x], 1);
      mbar_init(&bar_acc_empty[threadIdx.x], 128);
    }
    if (threadIdx.x == 0) {
      mbar_init(&bar_parts, 1);
      s_abort = 0;
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem_base)), "r"(kStTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  // Every block of the cluster has its barriers ready before another block arrives on them or
  // writes into its shared memory: the arrival is here, the wait before the first such access.
  const int n_quads = args.n_cols >> 2;            // groups of four tokens
  const int q_per = (n_quads + split - 1) / split;   // groups per block of the cluster at most
  const unsigned rank = clustered ? cluster_rank() : 0u;
  const int my_quads = clustered ? (n_quads - static_cast<int>(rank) + split - 1) / split : 0;  // groups rank, rank + split, ...
  if (clustered) {
    if (threadIdx.x == 0) mbar_expect_tx(&bar_parts, static_cast<unsigned>((split - 1) * my_quads) * kStQuadBytes);
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");
  }
  const unsigned tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;
  auto give_up = [&](int code) {
    if (!*abort_flag) atomicExch(args.status, code);
    s_abort = 1;
  };

  // ------------------------------------------------------------------ the epilogue
  // Thread = accumulator lane = row of the tile; its registers hold that row's outputs.  They go
  // through shared memory, transposed ([token][row]), so that a thread then writes four
  // consecutive columns of one token (a warp: whole rows of the output) instead of a two-byte
  // piece in each of many rows.
  const int row = (warp & 3) * 32 + lane;
  // SWIGLU: rows 64..127 of the staged tokens hold up, rows 0..63 gate -> rows 0..63 = silu(gate * mult) * up
  auto apply_swiglu = [&](int n_tok, float mult) {
    for (int it = threadIdx.x; it < n_tok * (kStRows / 2); it += 128) {
      const int j = it / (kStRows / 2), r = it % (kStRows / 2);
      stage_out[j * kStRows + r] = silu_fast(stage_out[j * kStRows + r] * mult) * stage_out[j * kStRows + r + kStRows / 2];
    }
  };
  // writes the staged tokens: local token j is token `tok(j)` of the step
  auto write_out = [&](int n_tok, int n0, float scale, auto tok) {
    const int items = n_tok * kSegs;
#pragma unroll
    for (int u = 0; u < 32 * kSegs / 128; ++u) {  // fixed trip count: the loads of all rounds go out together
      const int it = static_cast<int>(threadIdx.x) + u * 128;
      const int j = it / kSegs, seg = it % kSegs;
      const int t = tok(j), n = n0 + seg * 4;
      if (it < items && t < args.T && n < args.N) {
        const float4 a = *reinterpret_cast<const float4*>(stage_out + j * kStRows + seg * 4);
        if (MODE == kStResidual) {
          float* dst = args.h_out + static_cast<long long>(t) * args.N + n;
          if (n + 4 <= args.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            st_red4(dst, scale * a.x, scale * a.y, scale * a.z, scale * a.w);
          } else {
            atomicAdd(dst, scale * a.x);
            if (n + 1 < args.N) atomicAdd(dst + 1, scale * a.y);
            if (n + 2 < args.N) atomicAdd(dst + 2, scale * a.z);
            if (n + 3 < args.N) atomicAdd(dst + 3, scale * a.w);
          }
        } else {
          bf16* dst = args.y + static_cast<long long>(t) * args.ldy + n;
          if (n + 4 <= args.N && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
            uint2 pack;
            *reinterpret_cast<__nv_bfloat162*>(&pack.x) = __floats2bfloat162_rn(a.x, a.y);
            *reinterpret_cast<__nv_bfloat162*>(&pack.y) = __floats2bfloat162_rn(a.z, a.w);
            *reinterpret_cast<uint2*>(dst) = pack;
          } else {
            dst[0] = __float2bfloat16_rn(a.x);
            if (n + 1 < args.N) dst[1] = __float2bfloat16_rn(a.y);
            if (n + 2 < args.N) dst[2] = __float2bfloat16_rn(a.z);
            if (n + 3 < args.N) dst[3] = __float2bfloat16_rn(a.w);
          }
        }
      }
    }
  };
  // A thread's first output address, read once while the products run: the address translation is
  // then at hand when the outputs are written (the first access of a block to a page costs it
  // several hundred nanoseconds otherwise).
  auto touch_out = [&](int n0, auto tok) {
    const int j = static_cast<int>(threadIdx.x) / kSegs, seg = static_cast<int>(threadIdx.x) % kSegs;
    const int t = tok(j), n = n0 + seg * 4;
    if (t < args.T && n < args.N) {
      unsigned dummy;
      if (MODE == kStResidual)
        asm volatile("ld.global.cg.u32 %0, [%1];\n" : "=r"(dummy) : "l"(args.h_out + static_cast<long long>(t) * args.N + n) : "memory");
      else
        asm volatile("ld.global.cg.u16 %0, [%1];\n" : "=r"(dummy) : "l"(args.y + static_cast<long long>(t) * args.ldy + n) : "memory");
    }
  };
  // one tile of a block that has all of K (or adds its slice with atomics): 32 tokens at a time
  auto finish_tile = [&](int ti, int buf) {
    const unsigned lane_base = tmem_base + (static_cast<unsigned>((warp & 3) * 32) << 16) + buf * kStTok;
    const int n0 = (static_cast<int>(blockIdx.x) + ti * static_cast<int>(gridDim.x)) * kTileCols;
    const float scale = args.scale[prob];
    for (int c0 = 0; c0 < n_cols; c0 += 32) {
      unsigned raw[32];
      tmem_ld32(lane_base + c0, raw);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      if (c0 + 32 >= n_cols) {  // the accumulator may take the tile after next
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        mbar_arrive(&bar_acc_empty[buf]);
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) stage_out[j * kStRows + row] = __uint_as_float(raw[j]);
      epilogue_warps_sync();
      if (MODE == kStSwiglu) {
        apply_swiglu(32, scale);
        epilogue_warps_sync();
      }
      write_out(32, n0, scale, [&](int j) { return c0 + j; });
      epilogue_warps_sync();  // the staging buffer is free for the next chunk or tile
    }
  };
  // The K slices of a tile, one per block of the cluster: the groups of four tokens are dealt out
  // over the blocks (group q belongs to block q mod split).  A block lays its partial sums out by
  // owner in its idle ring ([owner][group][row] float4) and sends every other block that block's
  // part with one bulk copy (into `parts` there: [sender][group][row]); then it adds what it
  // received to its own part and stores its groups.
  float4* send = reinterpret_cast<float4*>(ring);
  auto send_slices = [&]() {
    const unsigned lane_base = tmem_base + (static_cast<unsigned>((warp & 3) * 32) << 16);
    unsigned raw[kStTok];
    tmem_ld32(lane_base, raw);
    if (n_cols > 32) tmem_ld32(lane_base + 32, raw + 32);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
    int owner = 0, k = 0;  // group q = k * split + owner
#pragma unroll
    for (int q = 0; q < kStTok / 4; ++q) {
      if (q < n_quads)
        send[(owner * q_per + k) * kStRows + row] = make_float4(__uint_as_float(raw[4 * q]), __uint_as_float(raw[4 * q + 1]),
                                                                __uint_as_float(raw[4 * q + 2]), __uint_as_float(raw[4 * q + 3]));
      if (++owner == split) {
        owner = 0;
        ++k;
      }
    }
    fence_proxy_async();  // the copy engine reads what the threads wrote
    epilogue_warps_sync();
    const int o = threadIdx.x;
    if (o < split && o != static_cast<int>(rank)) {
      const int quads_o = (n_quads - o + split - 1) / split;
      const int slot = static_cast<int>(rank) < o ? static_cast<int>(rank) : static_cast<int>(rank) - 1;
      bulk_copy_to_cluster(cluster_map(smem_u32(parts), o) + static_cast<unsigned>(slot * q_per) * kStQuadBytes,
                           smem_u32(send) + static_cast<unsigned>(o * q_per) * kStQuadBytes,
                           static_cast<unsigned>(quads_o) * kStQuadBytes, cluster_map(smem_u32(&bar_parts), o));
    }
  };
  auto reduce_and_store = [&]() {
#pragma unroll
    for (int k = 0; k < kStTok / 8; ++k) {  // at most 8 groups a block (two blocks, 64 tokens)
      if (k < my_quads) {
        float4 a = send[(static_cast<int>(rank) * q_per + k) * kStRows + row];
        for (int sl = 0; sl < split - 1; ++sl) {
          const float4 b = parts[(sl * q_per + k) * kStRows + row];
          a.x += b.x;
          a.y += b.y;
          a.z += b.z;
          a.w += b.w;
        }
        stage_out[(4 * k) * kStRows + row] = a.x;
        stage_out[(4 * k + 1) * kStRows + row] = a.y;
        stage_out[(4 * k + 2) * kStRows + row] = a.z;
        stage_out[(4 * k + 3) * kStRows + row] = a.w;
      }
    }
    epilogue_warps_sync();
    const float scale = args.scale[prob];
    if (MODE == kStSwiglu) {
      apply_swiglu(4 * my_quads, scale);
      epilogue_warps_sync();
    }
    write_out(4 * my_quads, static_cast<int>(blockIdx.x) * kTileCols, scale,
              [&](int j) { return ((j >> 2) * split + static_cast<int>(rank)) * 4 + (j & 3); });
  };

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producer
    if (has_work) {
      if (lane == 0) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<unsigned long long>(map_w)) : "memory");
      if (lane == 1) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<unsigned long long>(map_x)) : "memory");
      // The weights depend on nothing an earlier kernel writes; the activations do: those of the
      // first filling of the ring are requested behind the wait for that kernel.
      const int first = min(kStStages, total);
      auto request_w = [&](int s, int ti, int kb) {  // one lane: announce the stage's bytes, request its weights
        unsigned char* stage = ring + s * kStStageBytes;
        const int n0 = (static_cast<int>(blockIdx.x) + ti * static_cast<int>(gridDim.x)) * kTileCols;
        const int kcol = k0 + kb * kStKB;
        mbar_expect_tx(&bar_full[s], kStWBox + x_bytes);
        if (MODE == kStSwiglu) {
          tma_load_2d(stage, map_w, kcol, n0, &bar_full[s]);
          tma_load_2d(stage + kStWBox / 2, map_w, kcol, args.N + n0, &bar_full[s]);
        } else {
          tma_load_2d(stage, map_w, kcol, n0, &bar_full[s]);
        }
      };
      auto request_x = [&](int s, int kb) {
        tma_load_2d(ring + s * kStStageBytes + kStWBox, map_x, k0 + kb * kStKB, 0, &bar_full[s]);
      };
      // the first filling: a lane per stage (a request costs its thread some hundred cycles)
      if (lane < first) request_w(lane, lane / n_kb, lane % n_kb);
      __syncwarp();
      pdl_wait();
      if (lane < first) request_x(lane, lane % n_kb);
      int issued = first;
      for (int i = first; i < total; ++i) {
        const int s = i % kStStages;
        int ok = 1;
        if (lane == 0) ok = mbar_wait(&bar_empty[s], ((i / kStStages) & 1) ^ 1, abort_flag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0) give_up(21);
          break;
        }
        if (lane == 0) {
          request_w(s, i / n_kb, i % n_kb);
          request_x(s, i % n_kb);
        }
        issued = i + 1;
      }
      if (lane == 0 && s_abort) {
        // copies already requested still write into this block's shared memory: wait for them
        for (int i = issued > kStStages ? issued - kStStages : 0; i < issued; ++i)
          for (unsigned n = 0; n < kSpinLimit && !mbar_try_wait(&bar_full[i % kStStages], (i / kStStages) & 1); ++n) {
          }
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    pdl_wait();
    if (lane == 0 && has_work) {
      const unsigned idesc = kStIdesc | (static_cast<unsigned>(n_cols >> 3) << 17);
      bool ok = true;
      int i = 0;
      for (int ti = 0; ti < my_tiles && ok; ++ti) {
        const int buf = ti & 1, use = ti >> 1;
        if (use > 0 && !mbar_wait(&bar_acc_empty[buf], (use - 1) & 1, abort_flag)) {  // the epilogue has taken this accumulator's last tile
          give_up(23);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        for (int kb = 0; kb < n_kb; ++kb, ++i) {
          const int s = i % kStStages;
          if (!mbar_wait(&bar_full[s], (i / kStStages) & 1, abort_flag)) {
            give_up(22);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const unsigned long long a_desc = umma_desc(ring + s * kStStageBytes);
          const unsigned long long b_desc = umma_desc(ring + s * kStStageBytes + kStWBox);
#pragma unroll
          for (int k = 0; k < kStKB / 16; ++k)  // 16 columns further inside the swizzled row: 32 bytes = 2 units
            umma_f16(tmem_base + buf * kStTok, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&bar_empty[s]);  // the stage is free once these products have read it
        }
        if (ok) umma_commit(&bar_acc_full[buf]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 0..3: lanes 0..127)
    pdl_wait();
    bool ready = has_work;
    if (has_work) {
      if (clustered)
        touch_out(static_cast<int>(blockIdx.x) * kTileCols, [&](int j) { return ((j >> 2) * split + static_cast<int>(rank)) * 4 + (j & 3); });
      else
        touch_out(static_cast<int>(blockIdx.x) * kTileCols, [&](int j) { return j; });
    }
    for (int ti = 0; ti < my_tiles && has_work; ++ti) {
      const int buf = ti & 1, use = ti >> 1;
      const bool mine = mbar_wait(&bar_acc_full[buf], use & 1, abort_flag);
      if (!epilogue_warps_all(mine)) {
        if (!mine && lane == 0) give_up(24);
        ready = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      if (clustered) break;  // finished below, with the other blocks' partial sums
      finish_tile(ti, buf);
    }
    if (clustered) {
      // (every block of the cluster is up: its barriers are ready and its shared memory is there)
      asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
      if (ready) send_slices();
      // A block that gave up sends nothing but still waits for the others' parts: its shared memory
      // must outlive their copies (and they give up on their own waits for its part).
      const bool mine = mbar_wait_cluster(&bar_parts, 0, ready ? abort_flag : nullptr);
      const bool all = epilogue_warps_all(mine && ready);
      if (ready && !mine && lane == 0) give_up(25);
      // Second round of the cluster barrier: once every block has received its parts, every
      // block's copies have read their source, and the blocks may leave.  (It orders execution
      // only, no data: a releasing arrival would wait for this thread's writes in flight.)
      asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");
      if (all) reduce_and_store();
      asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    }
  }
  if (clustered && warp >= 4) {
    __syncwarp();
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kStTmemCols) : "memory");
  }
}

// bfloat16 matrix [rows, cols] with row stride ld (elements); box = 64 columns x box_rows rows.
static bool st_make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {kStKB, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MODE>
int launch_skinny_tc(const CUtensorMap* maps, SkinnyTcArgs a, cudaStream_t stream) {
  auto kern = skinny_tc_kernel<MODE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kStSmem));
  if (e != cudaSuccess) return static_cast<int>(e);
  static int n_sm = 0;
  if (n_sm == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        n_sm <= 0)
      return PMM_ERR_BAD_ARGUMENT;
  }
  constexpr int cols_per_tile = MODE == kStSwiglu ? kStRows / 2 : kStRows;
  const int n_tx = (a.N + cols_per_tile - 1) / cols_per_tile;
  auto boxes_of = [](int k) { return (k + kStKB - 1) / kStKB; };
  int gx, gy;
  a.split = 1;
  if (MODE == kStResidual) {
    // slices of K so that (row tiles) x (slices of all products) is about one block per SM
    int boxes = 0;
    for (int p = 0; p < a.n_problems; ++p) boxes += boxes_of(a.K[p]);
    const int per_slice = std::max(1, (boxes * n_tx + n_sm - 1) / n_sm);
    a.k_slice = per_slice * kStKB;
    int busy = 0;
    for (int p = 0; p < a.n_problems; ++p) busy += (a.K[p] + a.k_slice - 1) / a.k_slice;
    gy = (std::max(a.K[0], a.K[1]) + a.k_slice - 1) / a.k_slice;
    gx = std::min(n_tx, std::max(1, n_sm / std::max(busy, 1)));
  } else {
    const int boxes = boxes_of(a.K[0]);
    int split = 1;
    if (2 * n_tx <= n_sm) split = std::max(1, std::min({kStMaxSplit, n_sm / n_tx, boxes / 2}));
    const int per_slice = (boxes + split - 1) / split;
    a.split = (boxes + per_slice - 1) / per_slice;  // no empty slice
    a.k_slice = per_slice * kStKB;
    gy = a.split;
    gx = a.split > 1 ? n_tx : std::min(n_tx, n_sm);
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(gx, gy, a.n_problems);
  cfg.blockDim = dim3(kStThreads);
  cfg.dynamicSmemBytes = kStSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.numAttrs = 1;
  if (a.split > 1) {
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = 1;
    attrs[1].val.clusterDim.y = a.split;
    attrs[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attrs;
  cudaLaunchKernelEx(&cfg, kern, maps[0], maps[1], maps[2], maps[3], a);
  return launch_status();
}

}  // namespace pmm

// Whether pmm_skinny_tc takes these sizes: 1..64 tokens, K a multiple of 8 (rows of 16-byte
// multiples) for every product.
PMM_EXPORT int pmm_skinny_tc_supported(int mode, int T, int N, int K0, int K1, long long ldx0, long long ldx1, long long ldy) {
  (void)ldy;
  if (T < 1 || T > pmm::kStTok || N < 1 || K0 < 8 || K0 % 8 || ldx0 % 8) return 0;
  if (K1 && (K1 < 8 || K1 % 8 || ldx1 % 8)) return 0;
  if (mode == pmm::kStResidual) return 1;
  if (mode != pmm::kStStore && mode != pmm::kStSwiglu) return 0;
  return K1 == 0 ? 1 : 0;
}

// mode 0 STORE (y bfloat16 [T, ldy]), 1 SWIGLU (w0 = [gate; up] rows, N = F, scale0 = gate multiplier),
// 2 RESIDUAL (h_out[T, N] += scale * y; one or two products).
// status: one int in device memory that stays 0 unless a bounded wait gave up.
PMM_EXPORT int pmm_skinny_tc(int mode, int T, int N, const void* x0, long long ldx0, const void* w0, int K0, float scale0,
                             const void* x1, long long ldx1, const void* w1, int K1, float scale1, void* y,
                             long long ldy, float* h_out, int* status, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (!x0 || !w0 || !status || !pmm_skinny_tc_supported(mode, T, N, K0, w1 ? K1 : 0, ldx0, w1 ? ldx1 : 0, ldy))
    return PMM_ERR_BAD_ARGUMENT;
  auto aligned16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (!aligned16(x0) || !aligned16(w0) || (w1 && (!x1 || !aligned16(x1) || !aligned16(w1)))) return PMM_ERR_BAD_ARGUMENT;
  if (mode == pmm::kStResidual ? !h_out : (!y || w1)) return PMM_ERR_BAD_ARGUMENT;
  pmm::SkinnyTcArgs a{};
  a.T = T;
  a.N = N;
  a.n_cols = (T + 15) / 16 * 16;
  a.n_problems = w1 ? 2 : 1;
  a.K[0] = K0;
  a.K[1] = w1 ? K1 : 0;
  a.scale[0] = scale0;
  a.scale[1] = scale1;
  a.y = static_cast<pmm::bf16*>(y);
  a.ldy = ldy;
  a.h_out = h_out;
  a.status = status;
  const int w_box_rows = mode == pmm::kStSwiglu ? pmm::kStRows / 2 : pmm::kStRows;
  const long long w_rows = mode == pmm::kStSwiglu ? 2LL * N : N;
  CUtensorMap maps[4];
  if (!pmm::st_make_map(&maps[0], x0, T, K0, ldx0, a.n_cols) || !pmm::st_make_map(&maps[1], w0, w_rows, K0, K0, w_box_rows))
    return PMM_ERR_BAD_ARGUMENT;
  if (w1) {
    if (!pmm::st_make_map(&maps[2], x1, T, K1, ldx1, a.n_cols) || !pmm::st_make_map(&maps[3], w1, w_rows, K1, K1, w_box_rows))
      return PMM_ERR_BAD_ARGUMENT;
  } else {
    maps[2] = maps[0];
    maps[3] = maps[1];
  }
  switch (mode) {
    case pmm::kStStore: return pmm::launch_skinny_tc<pmm::kStStore>(maps, a, stream);
    case pmm::kStSwiglu: return pmm::launch_skinny_tc<pmm::kStSwiglu>(maps, a, stream);
    default: return pmm::launch_skinny_tc<pmm::kStResidual>(maps, a, stream);
  }
}

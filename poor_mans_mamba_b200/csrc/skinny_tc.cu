// Weight-streaming matrix product for steps of 33..64 tokens (it takes 1..64) on the fifth-generation
// tensor cores:
//   y[T, N] = x[T, K] W[N, K]^T, bfloat16 operands, float accumulation,
// with the same epilogues as the mma.sync form for fewer tokens (skinny_gemm.cu): STORE (bfloat16),
// SWIGLU (W = [gate rows; up rows], act = silu(gate * mult) * up) and RESIDUAL (h += scale * y with
// float atomics; K may be cut into slices over blocks, and two products may share a launch).
// At these sizes the product is still a read of W at memory speed, but with mma.sync every warp
// re-reads the activations from shared memory for each tile of weights and the kernel ends up bound
// by that; here the tensor core reads both operands from shared memory itself.
//
// The tokens are the M side of the instruction: A = x (M = 128 rows of which at most 64 hold
// tokens), B = a tile of 32 rows of W, D = 128 lanes x 32 float columns in tensor memory (lane =
// token).  x of the block's K slice (at most 1,024 columns) is brought in once by TMA as boxes of
// 64 columns x 64 tokens (8 KB, 128-byte swizzle, rows beyond T read as zero) and stays; the
// instruction's rows 64..127 fall on the box of the next 64 columns (or on a spare box after the
// last), whatever is there only reaches accumulator lanes 64..127, which nobody reads.  W streams
// through a ring of 4 stages of 256 columns (4 boxes of 64 columns x 32 rows; SWIGLU: 16 gate + 16
// up rows).  A block walks the row tiles bx, bx + gridDim.x, ... with the ring running on across
// tile boundaries and two accumulators in turn, so the epilogue of a tile overlaps the products of
// the next.  Warps: 0, 1 = epilogue (tensor-memory lanes 0..63: a thread holds the 32 outputs of
// its token), 2 = TMA producer, 3 = tensor-memory owner and MMA issuer.  The first weight stages
// are requested before the wait for the kernel before this one (programmatic dependent launch).
// Every mbarrier wait is bounded: on a time-out the waiter writes a code (21..24) to *status,
// raises the block's abort flag, all roles leave their loops, the producer waits (bounded) for its
// copies in flight and the tensor memory is freed.  No cluster multicast.
// (reference: linear layers are cublasSgemm calls, src/ops/gpu/linear.cu:3-21.)
#include "tcgen05.cuh"
#include <algorithm>

namespace pmm {

using bf16 = __nv_bfloat16;

constexpr int kStTok = 64;      // tokens at most
constexpr int kStRows = 32;     // rows of W per tile = columns of the accumulator
constexpr int kStKB = 64;       // columns per box: one 128-byte swizzle row
constexpr int kStChunk = 4;     // boxes per pipeline stage
constexpr int kStStages = 4;
constexpr int kStMaxKB = 16;    // boxes of x resident: K slices of at most 1,024 columns
constexpr int kStThreads = 128;
constexpr int kStTmemCols = 64;  // two accumulators of 32 columns
constexpr int kStXBox = kStTok * kStKB * 2;    // 8 KB
constexpr int kStWBox = kStRows * kStKB * 2;   // 4 KB
constexpr int kStStageBytes = kStChunk * kStWBox;
constexpr size_t kStSmem = 1024 /*alignment*/ + static_cast<size_t>(kStMaxKB + 1) * kStXBox + static_cast<size_t>(kStStages) * kStStageBytes;

enum { kStStore = 0, kStSwiglu = 1, kStResidual = 2 };

// kind::f16 instruction descriptor: float accumulate, bfloat16 A and B, both K-major, N = 32, M = 128.
constexpr unsigned kStIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kStRows >> 3) << 17) | ((128 >> 4) << 24);

struct SkinnyTcArgs {
  int T, N;          // tokens, output columns (SWIGLU: F)
  int n_problems;
  int K[2];
  int k_slice;       // columns of K per block along gridDim.y (a multiple of 64, at most 1,024)
  float scale[2];    // RESIDUAL: factor on y; SWIGLU: gate multiplier
  bf16* y;           // STORE / SWIGLU output
  long long ldy;
  float* h_out;      // RESIDUAL target [T, N]
  int* status;
};

__device__ __forceinline__ void st_red4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(kStThreads)
    skinny_tc_kernel(const __grid_constant__ CUtensorMap map_x0, const __grid_constant__ CUtensorMap map_w0,
                     const __grid_constant__ CUtensorMap map_x1, const __grid_constant__ CUtensorMap map_w1,
                     const SkinnyTcArgs args) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bar_x, bar_full[kStStages], bar_empty[kStStages], bar_acc_full[2], bar_acc_empty[2];
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
  const int n_kb = k1 > k0 ? (k1 - k0 + kStKB - 1) / kStKB : 0;   // boxes of this block's K slice
  const int n_chunks = (n_kb + kStChunk - 1) / kStChunk;
  constexpr int kTileCols = MODE == kStSwiglu ? kStRows / 2 : kStRows;  // output columns of a row tile
  const int n_tx = (args.N + kTileCols - 1) / kTileCols;
  const int my_tiles = static_cast<int>(blockIdx.x) < n_tx ? (n_tx - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;
  if (n_kb == 0 || my_tiles == 0) {  // the whole block: a product with a shorter K has nothing in this slice
    pdl_wait();
    return;
  }
  const int total = my_tiles * n_chunks;  // copies of the weight ring

  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sX = tiles;                                   // [n_kb + 1] boxes of 8 KB
  unsigned char* sW = tiles + (kStMaxKB + 1) * kStXBox;        // [stages][4] boxes of 4 KB

  if (threadIdx.x == 0) {
    mbar_init(&bar_x, 1);
    for (int s = 0; s < kStStages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bar_acc_full[b], 1);
      mbar_init(&bar_acc_empty[b], 64);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 3) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem_base)), "r"(kStTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;
  auto give_up = [&](int code) {
    if (!*abort_flag) atomicExch(args.status, code);
    s_abort = 1;
  };
  // boxes of chunk c of a tile (the last chunk of a slice may be shorter)
  auto boxes_of = [&](int c) { return min(kStChunk, n_kb - c * kStChunk); };

  if (warp == 2) {
    // ---------------------------------------------------------------- TMA producer
    // The whole warp takes part: lane 0 waits and announces the bytes, then every lane requests one
    // box (a request costs its thread some hundred cycles; sixteen from one thread were the
    // longest part of a one-tile block's life).
    if (lane == 0) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<unsigned long long>(map_w)) : "memory");
    if (lane == 1) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<unsigned long long>(map_x)) : "memory");
    int issued = 0, ti = 0, c = 0;
    bool x_requested = false;
    for (int i = 0; i < total; ++i) {
      const int s = i % kStStages;
      int ok = 1;
      if (i >= kStStages && lane == 0) ok = mbar_wait(&bar_empty[s], ((i / kStStages) & 1) ^ 1, abort_flag) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) {
        if (lane == 0) give_up(21);
        break;
      }
      const int n0 = (static_cast<int>(blockIdx.x) + ti * static_cast<int>(gridDim.x)) * kTileCols;
      const int nb = boxes_of(c);
      if (lane == 0) mbar_expect_tx(&bar_full[s], nb * kStWBox);
      __syncwarp();
      if (MODE == kStSwiglu) {
        if (lane < 2 * nb) {  // 16 gate rows and their 16 up rows of box lane / 2
          const int bx = lane >> 1, up = lane & 1;
          tma_load_2d(sW + s * kStStageBytes + bx * kStWBox + up * (kStWBox / 2), map_w, k0 + (c * kStChunk + bx) * kStKB,
                      up * args.N + n0, &bar_full[s]);
        }
      } else if (lane < nb) {
        tma_load_2d(sW + s * kStStageBytes + lane * kStWBox, map_w, k0 + (c * kStChunk + lane) * kStKB, n0, &bar_full[s]);
      }
      issued = i + 1;
      if (++c == n_chunks) {
        c = 0;
        ++ti;
      }
      // The weights depend on nothing an earlier kernel writes; the activations do: they are
      // requested after the first filling of the ring, behind the wait for that kernel.
      if (!x_requested && (issued == kStStages || issued == total)) {
        pdl_wait();
        if (lane == 0) mbar_expect_tx(&bar_x, n_kb * kStXBox);
        __syncwarp();
        if (lane < n_kb) tma_load_2d(sX + lane * kStXBox, map_x, k0 + lane * kStKB, 0, &bar_x);
        x_requested = true;
      }
    }
    if (!x_requested) pdl_wait();
    if (lane == 0 && s_abort) {
      // copies already requested still write into this block's shared memory: wait for them
      for (int i = issued > kStStages ? issued - kStStages : 0; i < issued; ++i)
        for (unsigned n = 0; n < kSpinLimit && !mbar_try_wait(&bar_full[i % kStStages], (i / kStStages) & 1); ++n) {
        }
      if (x_requested)
        for (unsigned n = 0; n < kSpinLimit && !mbar_try_wait(&bar_x, 0); ++n) {
        }
    }
  } else if (warp == 3) {
    // ---------------------------------------------------------------- MMA issuer
    pdl_wait();
    if (lane == 0) {
      bool ok = mbar_wait(&bar_x, 0, abort_flag);
      if (!ok) give_up(22);
      int i = 0;
      for (int ti = 0; ti < my_tiles && ok; ++ti) {
        const int buf = ti & 1, use = ti >> 1;
        if (use > 0 && !mbar_wait(&bar_acc_empty[buf], (use - 1) & 1, abort_flag)) {  // the epilogue has taken this accumulator's last tile
          give_up(23);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        for (int c = 0; c < n_chunks; ++c, ++i) {
          const int s = i % kStStages;
          if (!mbar_wait(&bar_full[s], (i / kStStages) & 1, abort_flag)) {
            give_up(22);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const int nb = boxes_of(c);
          for (int b = 0; b < nb; ++b) {
            const unsigned long long a_desc = umma_desc(sX + (c * kStChunk + b) * kStXBox);
            const unsigned long long b_desc = umma_desc(sW + s * kStStageBytes + b * kStWBox);
#pragma unroll
            for (int k = 0; k < kStKB / 16; ++k)  // 16 columns further inside the swizzled row: 32 bytes = 2 units
              umma_f16(tmem_base + buf * kStRows, a_desc + 2 * k, b_desc + 2 * k, kStIdesc, (c > 0 || b > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&bar_empty[s]);  // the stage is free once these products have read it
        }
        if (ok) umma_commit(&bar_acc_full[buf]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 0, 1: tokens 0..63)
    pdl_wait();
    const int m = warp * 32 + lane;  // this thread's token = its tensor-memory lane
    const unsigned lane_base = tmem_base + (static_cast<unsigned>(warp * 32) << 16);
    const float scale = args.scale[prob];
    for (int ti = 0; ti < my_tiles; ++ti) {
      const int buf = ti & 1, use = ti >> 1;
      bool ok = mbar_wait(&bar_acc_full[buf], use & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) give_up(24);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      unsigned v[32];
      tmem_ld32(lane_base + buf * kStRows, v);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      mbar_arrive(&bar_acc_empty[buf]);
      if (m >= args.T) continue;
      const int n0 = (static_cast<int>(blockIdx.x) + ti * static_cast<int>(gridDim.x)) * kTileCols;
      const bool whole = n0 + kTileCols <= args.N;
      if (MODE == kStSwiglu) {
        bf16* dst = args.y + static_cast<long long>(m) * args.ldy + n0;
        float a[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) a[e] = silu_fast(__uint_as_float(v[e]) * scale) * __uint_as_float(v[16 + e]);
        if (whole) {
#pragma unroll
          for (int j = 0; j < 16; j += 8) {
            uint4 pack;
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pack);
#pragma unroll
            for (int e = 0; e < 4; ++e) p2[e] = __floats2bfloat162_rn(a[j + 2 * e], a[j + 2 * e + 1]);
            *reinterpret_cast<uint4*>(dst + j) = pack;
          }
        } else {
          for (int e = 0; e < 16; ++e)
            if (n0 + e < args.N) dst[e] = __float2bfloat16_rn(a[e]);
        }
      } else if (MODE == kStStore) {
        bf16* dst = args.y + static_cast<long long>(m) * args.ldy + n0;
        if (whole) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 pack;
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pack);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              p2[e] = __floats2bfloat162_rn(__uint_as_float(v[j + 2 * e]), __uint_as_float(v[j + 2 * e + 1]));
            *reinterpret_cast<uint4*>(dst + j) = pack;
          }
        } else {
          for (int e = 0; e < 32; ++e)
            if (n0 + e < args.N) dst[e] = __float2bfloat16_rn(__uint_as_float(v[e]));
        }
      } else {
        float* dst = args.h_out + static_cast<long long>(m) * args.N + n0;
        if (whole && (args.N & 3) == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            st_red4(dst + j, scale * __uint_as_float(v[j]), scale * __uint_as_float(v[j + 1]),
                    scale * __uint_as_float(v[j + 2]), scale * __uint_as_float(v[j + 3]));
        } else {
          for (int e = 0; e < 32; ++e)
            if (n0 + e < args.N) atomicAdd(dst + e, scale * __uint_as_float(v[e]));
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 3) {
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
int launch_skinny_tc(const CUtensorMap* maps, const SkinnyTcArgs& a, int k_max, cudaStream_t stream) {
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
  const int gy = (k_max + a.k_slice - 1) / a.k_slice;
  int busy = 0;  // (K slice, product) pairs that have work; one block per SM (by shared memory)
  for (int p = 0; p < a.n_problems; ++p) busy += (a.K[p] + a.k_slice - 1) / a.k_slice;
  const int gx = std::min(n_tx, std::max(1, n_sm / std::max(busy, 1)));
  launch_pdl(kern, dim3(gx, gy, a.n_problems), dim3(kStThreads), kStSmem, stream, maps[0], maps[1], maps[2], maps[3], a);
  return launch_status();
}

}  // namespace pmm

// Whether pmm_skinny_tc takes these sizes: 1..64 tokens, K a multiple of 8 (rows of 16-byte
// multiples); STORE and SWIGLU keep the whole K resident: at most 1,024 columns; outputs with
// 16-byte aligned rows.
PMM_EXPORT int pmm_skinny_tc_supported(int mode, int T, int N, int K0, int K1, long long ldx0, long long ldx1, long long ldy) {
  if (T < 1 || T > pmm::kStTok || N < 1 || K0 < 8 || K0 % 8 || ldx0 % 8) return 0;
  if (K1 && (K1 < 8 || K1 % 8 || ldx1 % 8)) return 0;
  if (mode == pmm::kStResidual) return 1;
  if (mode != pmm::kStStore && mode != pmm::kStSwiglu) return 0;
  return (K1 == 0 && K0 <= pmm::kStMaxKB * pmm::kStKB && ldy % 8 == 0) ? 1 : 0;
}

// mode 0 STORE (y bfloat16 [T, ldy]), 1 SWIGLU (w0 = [gate; up] rows, N = F, scale0 = gate multiplier),
// 2 RESIDUAL (h_out[T, N] += scale * y; one or two products; K cut into slices of at most 1,024 columns).
// status: one int in device memory that stays 0 unless a bounded wait gave up.
PMM_EXPORT int pmm_skinny_tc(int mode, int T, int N, const void* x0, long long ldx0, const void* w0, int K0, float scale0,
                             const void* x1, long long ldx1, const void* w1, int K1, float scale1, void* y,
                             long long ldy, float* h_out, int* status, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (!x0 || !w0 || !status || !pmm_skinny_tc_supported(mode, T, N, K0, w1 ? K1 : 0, ldx0, w1 ? ldx1 : 0, ldy))
    return PMM_ERR_BAD_ARGUMENT;
  auto aligned16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (!aligned16(x0) || !aligned16(w0) || (w1 && (!x1 || !aligned16(x1) || !aligned16(w1)))) return PMM_ERR_BAD_ARGUMENT;
  if (mode == pmm::kStResidual ? !h_out : (!y || !aligned16(y) || w1)) return PMM_ERR_BAD_ARGUMENT;
  pmm::SkinnyTcArgs a{};
  a.T = T;
  a.N = N;
  a.n_problems = w1 ? 2 : 1;
  a.K[0] = K0;
  a.K[1] = w1 ? K1 : 0;
  a.scale[0] = scale0;
  a.scale[1] = scale1;
  a.y = static_cast<pmm::bf16*>(y);
  a.ldy = ldy;
  a.h_out = h_out;
  a.status = status;
  const int k_max = std::max(a.K[0], a.K[1]);
  const int max_slice = pmm::kStMaxKB * pmm::kStKB;
  const int n_slices = (k_max + max_slice - 1) / max_slice;  // 1 for STORE and SWIGLU
  a.k_slice = ((k_max + n_slices - 1) / n_slices + pmm::kStKB - 1) / pmm::kStKB * pmm::kStKB;
  const int w_box_rows = mode == pmm::kStSwiglu ? pmm::kStRows / 2 : pmm::kStRows;
  const long long w_rows = mode == pmm::kStSwiglu ? 2LL * N : N;
  CUtensorMap maps[4];
  if (!pmm::st_make_map(&maps[0], x0, T, K0, ldx0, pmm::kStTok) || !pmm::st_make_map(&maps[1], w0, w_rows, K0, K0, w_box_rows))
    return PMM_ERR_BAD_ARGUMENT;
  if (w1) {
    if (!pmm::st_make_map(&maps[2], x1, T, K1, ldx1, pmm::kStTok) || !pmm::st_make_map(&maps[3], w1, w_rows, K1, K1, w_box_rows))
      return PMM_ERR_BAD_ARGUMENT;
  } else {
    maps[2] = maps[0];
    maps[3] = maps[1];
  }
  switch (mode) {
    case pmm::kStStore: return pmm::launch_skinny_tc<pmm::kStStore>(maps, a, k_max, stream);
    case pmm::kStSwiglu: return pmm::launch_skinny_tc<pmm::kStSwiglu>(maps, a, k_max, stream);
    default: return pmm::launch_skinny_tc<pmm::kStResidual>(maps, a, k_max, stream);
  }
}

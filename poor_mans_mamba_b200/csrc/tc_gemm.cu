// Blackwell tensor-core matrix product with a fused SwiGLU epilogue for prompt portions:
//   act[t, f] = silu((x W_gate^T)[t, f] * gate_mult) * (x W_up^T)[t, f]         (bfloat16 out)
// or, in plain mode, y = x W^T.  x [T, K] and W [rows, K] are bfloat16, K-major.
//
// One block computes a 256-token x 128-feature tile of act (two 128 x 256 accumulators, one per
// half of the tokens: the 128 gate columns next to their 128 up columns) with the
// fifth-generation tensor cores.  The tile is that large because operand traffic decides: a
// 256 x 256 tile needs 1 MB of operands from L2 for 134 MFLOP, half of what 128 x 256 needs, and a
// 2,048 x 4,096 product is 128 such tiles, one per SM in a single wave.
//   * operands are brought into shared memory by TMA (cp.async.bulk.tensor.2d, 128-byte
//     swizzle, out-of-range rows read as zero), three stages of 64 KB, signalled by mbarriers;
//   * one elected thread issues tcgen05.mma (M = 128, N = 256, K = 16 per instruction, two token
//     halves x four per 64-column stage) with the accumulators in tensor memory (all 512
//     columns: 128 lanes x 256 columns for each half); tcgen05.commit releases a stage back to
//     the producer and finally publishes the tile;
//   * eight epilogue warps read the accumulators with tcgen05.ld (a warp reads the 32 lanes of
//     its quarter; four warps per token half), apply the activation in float and store
//     bfloat16 rows.
// Warp roles: 0 = TMA producer, 1 = tensor-memory owner and MMA issuer, 2..9 = epilogue.
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiter records a code in
// *status, raises the block's abort flag and all roles leave their loops; the block still
// waits (bounded) for its own copies in flight and frees its tensor memory before it exits.
// No cluster multicast is used anywhere.
// (reference: gate and up are two cublasSgemm calls followed by scale, silu and mul launches,
// src/ops/cuda_backend.cu:311-338.)
#include "tcgen05.cuh"

namespace pmm {

using bf16 = __nv_bfloat16;

constexpr int kTcM = 256;        // tokens per tile: two halves of 128, one MMA row block each
constexpr int kTcMH = 128;       // rows of one MMA
constexpr int kTcN = 256;        // accumulator columns per tile
constexpr int kTcK = 64;         // K per stage: one 128-byte swizzle row of bfloat16
constexpr int kTcStages = 3;
constexpr int kTcThreads = 320;
constexpr int kTcTmemCols = 512; // both accumulators: all of an SM's tensor memory (one block per SM, by shared memory)
constexpr int kTcABytes = kTcM * kTcK * 2;  // 32 KB
constexpr int kTcBBytes = kTcN * kTcK * 2;  // 32 KB
constexpr size_t kTcSmem = static_cast<size_t>(kTcStages) * (kTcABytes + kTcBBytes) + 1024 /*alignment*/;

enum { kTcPlain = 0, kTcSwiglu = 1 };

// kind::f16 instruction descriptor: float accumulate, bfloat16 A and B, both K-major, N, M.
constexpr unsigned kTcIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kTcN >> 3) << 17) | ((kTcMH >> 4) << 24);

template <int MODE>
__global__ void __launch_bounds__(kTcThreads)
    tc_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                   bf16* __restrict__ out, long long ld_out, int T, int K, int F, float gate_mult,
                   int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[kTcStages], bar_empty[kTcStages], bar_accum;
  __shared__ unsigned s_tmem_base;
  __shared__ int s_abort;

  // 1024-byte aligned tiles (the swizzle pattern is a function of the address)
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sA = tiles;
  unsigned char* sB = tiles + kTcStages * kTcABytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * kTcM;
  const int n0 = blockIdx.y * (MODE == kTcSwiglu ? kTcN / 2 : kTcN);  // first output column
  const int k_blocks = K / kTcK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    mbar_init(&bar_accum, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {  // tensor memory for the two 128 x 256 float accumulators
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem_base)), "r"(kTcTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int issued = 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kTcStages;
        const unsigned use = kb / kTcStages;
        if (!mbar_wait(&bar_empty[s], (use & 1) ^ 1, abort_flag)) {
          if (!*abort_flag) atomicExch(status, 1);
          s_abort = 1;
          break;
        }
        mbar_expect_tx(&bar_full[s], kTcABytes + kTcBBytes);
        tma_load_2d(sA + s * kTcABytes, &map_x, kb * kTcK, m0, &bar_full[s]);                               // tokens 0..127
        tma_load_2d(sA + s * kTcABytes + kTcABytes / 2, &map_x, kb * kTcK, m0 + kTcMH, &bar_full[s]);      // tokens 128..255
        if (MODE == kTcSwiglu) {
          tma_load_2d(sB + s * kTcBBytes, &map_w, kb * kTcK, n0, &bar_full[s]);                      // gate rows
          tma_load_2d(sB + s * kTcBBytes + kTcBBytes / 2, &map_w, kb * kTcK, F + n0, &bar_full[s]);  // up rows
        } else {
          tma_load_2d(sB + s * kTcBBytes, &map_w, kb * kTcK, n0, &bar_full[s]);
          tma_load_2d(sB + s * kTcBBytes + kTcBBytes / 2, &map_w, kb * kTcK, n0 + kTcN / 2, &bar_full[s]);
        }
        issued = kb + 1;
      }
      if (s_abort) {
        // copies already requested still write into this block's shared memory: wait for them
        for (int kb = issued > kTcStages ? issued - kTcStages : 0; kb < issued; ++kb) {
          const int s = kb % kTcStages;
          for (unsigned i = 0; i < kSpinLimit && !mbar_try_wait(&bar_full[s], (kb / kTcStages) & 1); ++i) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < k_blocks && ok; ++kb) {
        const int s = kb % kTcStages;
        if (!mbar_wait(&bar_full[s], (kb / kTcStages) & 1, abort_flag)) {
          if (!*abort_flag) atomicExch(status, 2);
          s_abort = 1;
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned long long b_desc = umma_desc(sB + s * kTcBBytes);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const unsigned long long a_desc = umma_desc(sA + s * kTcABytes + half * (kTcABytes / 2));
#pragma unroll
          for (int k = 0; k < kTcK / 16; ++k) {
            // 16 columns further along K inside the swizzled row: 32 bytes = 2 units of 16 bytes
            umma_f16(tmem_base + half * kTcN, a_desc + 2 * k, b_desc + 2 * k, kTcIdesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(&bar_empty[s]);  // the stage is free once these MMAs have read it
      }
      if (ok) umma_commit(&bar_accum);  // the tile is complete once all MMAs have finished
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..9)
    const int quad = warp & 3;          // a warp may only read tensor-memory lanes 32*(warp % 4) ...
    const int mhalf = (warp - 2) >> 2;  // which token half, i.e. which accumulator
    bool ok = mbar_wait(&bar_accum, 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      if (lane == 0 && !*abort_flag) atomicExch(status, 3);
      s_abort = 1;
    } else {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int m = m0 + mhalf * kTcMH + quad * 32 + lane;  // this thread's token row
      const unsigned lane_base = tmem_base + (static_cast<unsigned>(quad * 32) << 16) + mhalf * kTcN;
      if (MODE == kTcSwiglu) {
#pragma unroll 1
        for (int c = 0; c < kTcN / 64; ++c) {
          unsigned g[32], u[32];
          tmem_ld32(lane_base + c * 32, g);
          tmem_ld32(lane_base + kTcN / 2 + c * 32, u);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          if (m < T) {
            bf16* dst = out + static_cast<long long>(m) * ld_out + n0 + c * 32;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 pack;
              __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pack);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float g0 = __uint_as_float(g[j + 2 * e]) * gate_mult, g1 = __uint_as_float(g[j + 2 * e + 1]) * gate_mult;
                p2[e] = __floats2bfloat162_rn(silu_fast(g0) * __uint_as_float(u[j + 2 * e]),
                                              silu_fast(g1) * __uint_as_float(u[j + 2 * e + 1]));
              }
              *reinterpret_cast<uint4*>(dst + j) = pack;
            }
          }
        }
      } else {
#pragma unroll 1
        for (int q = 0; q < kTcN / 32; ++q) {
          unsigned v[32];
          tmem_ld32(lane_base + q * 32, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          if (m < T) {
            bf16* dst = out + static_cast<long long>(m) * ld_out + n0 + q * 32;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 pack;
              __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pack);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                p2[e] = __floats2bfloat162_rn(__uint_as_float(v[j + 2 * e]), __uint_as_float(v[j + 2 * e + 1]));
              *reinterpret_cast<uint4*>(dst + j) = pack;
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTcTmemCols) : "memory");
  }
}

// bfloat16 matrix [rows, cols] with row stride ld (elements); box = 64 columns x box_rows rows.
inline bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {kTcK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace pmm

// Whether the tensor-core product takes these sizes: K a multiple of 64, output columns a
// multiple of 128 (SwiGLU: F) or 256 (plain), 16-byte aligned rows.
PMM_EXPORT int pmm_tc_gemm_supported(int mode, int K, int n_out, long long ldx, long long ld_out) {
  if (K <= 0 || K % pmm::kTcK || ldx % 8 || ld_out % 8) return 0;
  return mode == pmm::kTcSwiglu ? (n_out % 128 == 0) : (n_out % 256 == 0);
}

// mode 1: out[T, F] = silu((x Wg^T) * gate_mult) * (x Wu^T) with w = [Wg; Wu] ([2F, K]).
// mode 0: out[T, N] = x w^T with w [N, K].  status: one int, stays 0 unless a bounded wait gave up.
PMM_EXPORT int pmm_tc_gemm(int mode, const void* x, long long ldx, const void* w, void* out, long long ld_out, int T,
                           int K, int n_out, float gate_mult, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!pmm_tc_gemm_supported(mode, K, n_out, ldx, ld_out) || !status) return PMM_ERR_BAD_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(w) % 16 || reinterpret_cast<uintptr_t>(out) % 16)
    return PMM_ERR_BAD_ARGUMENT;
  CUtensorMap map_x, map_w;
  const long long w_rows = mode == pmm::kTcSwiglu ? 2LL * n_out : n_out;
  if (!pmm::make_map(&map_x, x, T, K, ldx, pmm::kTcMH) || !pmm::make_map(&map_w, w, w_rows, K, K, pmm::kTcN / 2))
    return PMM_ERR_BAD_ARGUMENT;
  const int cols_per_block = mode == pmm::kTcSwiglu ? pmm::kTcN / 2 : pmm::kTcN;
  dim3 grid((T + pmm::kTcM - 1) / pmm::kTcM, n_out / cols_per_block);
  cudaError_t e;
  if (mode == pmm::kTcSwiglu) {
    auto kern = pmm::tc_gemm_kernel<pmm::kTcSwiglu>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pmm::kTcSmem));
    if (e != cudaSuccess) return static_cast<int>(e);
    pmm::launch_pdl(kern, grid, dim3(pmm::kTcThreads), pmm::kTcSmem, stream, map_x, map_w, static_cast<pmm::bf16*>(out), ld_out, T,
                    K, n_out, gate_mult, status);
  } else {
    auto kern = pmm::tc_gemm_kernel<pmm::kTcPlain>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pmm::kTcSmem));
    if (e != cudaSuccess) return static_cast<int>(e);
    pmm::launch_pdl(kern, grid, dim3(pmm::kTcThreads), pmm::kTcSmem, stream, map_x, map_w, static_cast<pmm::bf16*>(out), ld_out, T,
                    K, n_out, gate_mult, status);
  }
  return pmm::launch_status();
}

// Weight-streaming matrix product for decode steps: y[M, N] = x[M, K] W[N, K]^T with few
// tokens (M <= 64) and bfloat16 weights.  Such a product is a read of W at memory speed;
// what matters is a deep copy pipeline, enough blocks, and not touching the small
// activations more than once.  So the kernel fuses what surrounds the product:
//   prologue  x = rmsnorm(h) * w  from the float32 residual stream (every block redoes it:
//             M rows from L2), or x read as bfloat16;
//   epilogue  STORE     y -> bfloat16 [M, N]
//             SWIGLU    W holds gate rows [0, F) and up rows [F, 2F):
//                       act[m, f] = silu(gate * gate_mult) * up  -> bfloat16 [M, F]
//             RESIDUAL  h[m, n] += scale * y  (float32 atomics; the K range may be split over
//                       blocks, and up to two products with their own x, W, K and scale can
//                       share one launch: the mixers' output projections).
// Tensor-core form: the weights are the 16-row MMA operand (A), the tokens the 8-column one
// (B), mma.sync m16n8k16 with float accumulation.  A block of 8 warps works on tiles of 32 weight
// rows; W arrives in chunks of 256 columns through a 5-stage cp.async pipeline (16 KB a stage);
// warps split a chunk 2 (rows) x 4 (columns) and the column quarters are added at the end.
// The grid is no larger than what is resident at once: a block prepares its activations once
// (for a wide model that is as much traffic as a tile of weights) and then walks its row tiles
// bx, bx + gridDim.x, ... with the copy pipeline running on across the tile boundaries.
// (reference: linear layers are cublasSgemm calls, src/ops/gpu/linear.cu:3-21, the
// multipliers, SiLU and adds separate launches, src/ops/cuda_backend.cu:311-338.)
#include "common.cuh"
#include <algorithm>

namespace pmm {

using bf16 = __nv_bfloat16;

constexpr int kSgRows = 32;     // weight rows per block
constexpr int kSgChunk = 256;   // columns per pipeline stage
// Pipeline stages: five for up to 32 tokens (K = 1024 is four chunks: all of a block's weights are
// requested at once); three for 33..64 tokens, whose activations take most of the shared memory.
__host__ __device__ constexpr int sg_stages(int mt) { return mt > 4 ? 3 : 5; }
constexpr int kSgWStride = kSgChunk + 8;
constexpr int kSgThreads = 256;
constexpr int kSgPieces = kSgRows * (kSgChunk / 8) / kSgThreads;  // 16-byte pieces per thread and chunk

enum { kSgStore = 0, kSgSwiglu = 1, kSgResidual = 2, kSgStoreF32 = 3 };

struct SkinnyProblem {
  const bf16* x;       // [M, ldx] activations, or nullptr when the norm prologue is used
  long long ldx;
  const float* h_in;   // [M, K] residual stream for the norm prologue
  const float* norm_w; // [K]
  float eps;
  const bf16* w;       // [N or 2F, K]
  int K;
  float scale;         // RESIDUAL: factor on y; SWIGLU: gate multiplier
};

struct SkinnyArgs {
  SkinnyProblem p[2];
  int n_problems;
  int M, N;            // tokens, output columns (SWIGLU: F)
  int k_slice;         // columns of K per block along gridDim.y (multiple of 256)
  bf16* y;             // STORE / SWIGLU output
  long long ldy;
  float* h_out;        // RESIDUAL target [M, N]
  float* y32;          // STORE_F32: y32[m, n] = y_scale * y
  float y_scale;
};

__device__ __forceinline__ void sg_cp16(void* smem, const void* gmem, bool pred) {
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void sg_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void sg_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void sg_ldm(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void sg_ldm2(unsigned& r0, unsigned& r1, const void* p) {
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(s));
}
__device__ __forceinline__ void sg_mma(float* d, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// What a block needs to know about its place: which slice of K, which product, which row tiles.
template <int MT, int MODE>
struct SkinnyBlock {
  static constexpr int MP = MT * 8;  // padded tokens
  static constexpr int kSgStages = sg_stages(MT);
  static constexpr int kTileCols = MODE == kSgSwiglu ? 16 : kSgRows;  // output columns of a row tile
  const SkinnyArgs& args;
  const SkinnyProblem& pr;
  int K, k0, k1, kx, xs, n_chunks;
  int t0, t_step, my_tiles, total;  // row tiles t0, t0 + t_step, ...; total = my_tiles * n_chunks copies
  bf16* sW;     // [stages][32][264]
  bf16* sX;     // [MP][xs]
  float* sRed;  // [3][32][MP] column quarters, then up rows
  float* sNw;   // [kx] norm weights of the slice (norm prologue)
  float* sInv;  // [MP] rsqrt(mean(h^2) + eps) of each row (norm prologue): applied to the sums in the epilogue
  const bf16* src[kSgPieces];  // this thread's pieces of chunk 0 of the block's first tile
  size_t tile_stride;          // elements of W between one of the block's tiles and the next

  __device__ SkinnyBlock(const SkinnyArgs& a, int bx, int bx_step, int by, int bz, unsigned char* smem_raw)
      : args(a), pr(a.p[bz]) {
    K = pr.K;
    k0 = by * a.k_slice;
    k1 = min(K, k0 + a.k_slice);
    kx = k0 < K ? (k1 - k0 + kSgChunk - 1) / kSgChunk * kSgChunk : 0;  // slice length, whole chunks
    xs = kx + 8;                                                       // row stride of x in shared memory
    sW = reinterpret_cast<bf16*>(smem_raw);
    sX = sW + kSgStages * kSgRows * kSgWStride;
    sRed = reinterpret_cast<float*>(sX + MP * xs);
    sNw = sRed + 3 * 32 * MP;
    sInv = sNw + kx;
    n_chunks = kx / kSgChunk;
    const int n_tx = (a.N + kTileCols - 1) / kTileCols;
    t0 = bx;
    t_step = bx_step;
    my_tiles = bx < n_tx ? (bx + bx_step < n_tx ? (n_tx - 1 - bx) / bx_step + 1 : 1) : 0;
    total = my_tiles * n_chunks;
    tile_stride = static_cast<size_t>(bx_step) * kTileCols * K;
    // every thread copies the same pieces (row r, 16-byte column c8) of every chunk
    const int tid = threadIdx.x, c8 = tid & 31, n0 = bx * kTileCols;
#pragma unroll
    for (int j = 0; j < kSgPieces; ++j) {
      const int r = (tid >> 5) + j * (kSgThreads / 32);
      // global row of W behind row r of a tile (SWIGLU: 16 gate rows, then their 16 up rows)
      const int wr = MODE == kSgSwiglu ? (r < 16 ? n0 + r : a.N + n0 + (r - 16)) : n0 + r;
      src[j] = pr.w + static_cast<size_t>(wr) * K + k0 + c8 * 8;
    }
  }

  // Chunk `chunk` of the block's tile number `ti` -> pipeline stage `stage`: a thread copies four
  // 16-byte pieces, the same ones (row r, column piece c8) of every chunk.
  __device__ __forceinline__ void load_chunk(int stage, int ti, int chunk) const {
    const int tid = threadIdx.x, c8 = tid & 31;
    const int n0 = (t0 + ti * t_step) * kTileCols;
    bf16* dst = sW + stage * kSgRows * kSgWStride + (tid >> 5) * kSgWStride + c8 * 8;
    const bool col_ok = k0 + chunk * kSgChunk + c8 * 8 < k1;
    const size_t off = ti * tile_stride + chunk * kSgChunk;
#pragma unroll
    for (int j = 0; j < kSgPieces; ++j) {
      const int r = (tid >> 5) + j * (kSgThreads / 32);
      const bool ok = col_ok && (MODE == kSgSwiglu ? n0 + (r & 15) < args.N : n0 + r < args.N);
      sg_cp16(dst + j * (kSgThreads / 32) * kSgWStride, ok ? src[j] + off : pr.w, ok);
    }
  }

  // groups 0..stages-2: the first weight chunks.  They depend on nothing that an earlier kernel
  // or phase writes, so they are requested before the wait for it.
  __device__ __forceinline__ void request_weights() const {
    int ti = 0, ch = 0;
#pragma unroll
    for (int s = 0; s < kSgStages - 1; ++s) {
      if (s < total) load_chunk(s, ti, ch);
      sg_commit();
      if (++ch == n_chunks) {
        ch = 0;
        ++ti;
      }
    }
  }

  // everything after the weights have been requested; ONE: the block has exactly one row tile
  // (known when the kernel is chosen: every size of a small model), which keeps the loop plain
  template <bool ONE>
  __device__ void run() const;
  __device__ void finish_tile(float (&acc)[MT][4], int n0) const;
};

template <int MT, int MODE>
template <bool ONE>
__device__ void SkinnyBlock<MT, MODE>::run() const {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int M = args.M;
  if (total == 0) return;
  // next group: the activations when they are read as bfloat16, else the norm weights
  if (pr.h_in == nullptr) {
    for (int i = tid; i < MP * (kx / 8); i += kSgThreads) {
      const int m = i / (kx / 8), k = k0 + (i % (kx / 8)) * 8;
      const bool ok = m < M && k < k1;
      sg_cp16(sX + m * xs + (k - k0), pr.x + (ok ? static_cast<size_t>(m) * pr.ldx + k : 0), ok);
    }
  } else {
    for (int i = tid; i < kx / 4; i += kSgThreads) {
      const int k = k0 + i * 4;
      sg_cp16(sNw + i * 4, pr.norm_w + (k < k1 ? k : 0), k < k1);
    }
  }
  sg_commit();
  // norm prologue: the products run on x' = h * w (bfloat16, rows >= M and columns >= K zero) and
  // the row's factor rsqrt(mean(h^2) + eps) multiplies the float sums in the epilogue:
  //   (h * inv * w) W^T = inv * ((h * w) W^T).
  // So a row goes to shared memory as soon as it has been read, and its statistic is reduced
  // beside that instead of standing between the read and the products.
  if (pr.h_in != nullptr) {
    // (The stream is read past L1: in a chain of products other blocks have just added to it.)
    // One warp per token, two tokens at a time, 8 float4 per lane and token in flight.
    constexpr int kV = 8;                 // float4 per lane per pass
    constexpr int kPass = kV * 32 * 4;    // 1024 columns per pass
    constexpr int kTok = MP >= 2 * (kSgThreads / 32) ? 2 : 1;  // tokens per warp and round: all warps busy, and every warp walks the loop equally often
    bool weights_in = false;
    for (int m0 = warp * kTok; m0 < MP; m0 += kTok * (kSgThreads / 32)) {
      float ss[kTok];
#pragma unroll
      for (int j = 0; j < kTok; ++j) ss[j] = 0.f;
      for (int kb = 0; kb < max(K, k0 + kx); kb += kPass) {
        float4 keep[kTok][kV];
#pragma unroll
        for (int j = 0; j < kTok; ++j) {
          const int m = m0 + j;
          const float* row = pr.h_in + static_cast<size_t>(m < M ? m : 0) * K;
#pragma unroll
          for (int i = 0; i < kV; ++i) {
            const int k = kb + (i * 32 + lane) * 4;
            keep[j][i] = (m < M && k < K) ? __ldcg(reinterpret_cast<const float4*>(row + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        if (!weights_in) {
          sg_wait<0>();     // the norm weights (and, incidentally, the first weight chunks) have landed
          __syncthreads();  // ... and everyone else's; every warp comes here once, in its first round
          weights_in = true;
        }
#pragma unroll
        for (int j = 0; j < kTok; ++j) {
          const int m = m0 + j;
#pragma unroll
          for (int i = 0; i < kV; ++i) {
            const int k = kb + (i * 32 + lane) * 4;
            float4 v = keep[j][i];
            ss[j] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            if (m >= MP || k < k0 || k >= k0 + kx) continue;
            if (k < k1) {
              const float4 w4 = *reinterpret_cast<const float4*>(sNw + (k - k0));
              v.x *= w4.x;
              v.y *= w4.y;
              v.z *= w4.z;
              v.w *= w4.w;
            } else {
              v = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            bf16* dst = sX + m * xs + (k - k0);
            *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v.x, v.y);
            *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(v.z, v.w);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < kTok; ++j) {
        const float tot = warp_sum(ss[j]);
        if (lane == 0 && m0 + j < MP) sInv[m0 + j] = 1.0f / sqrtf(tot / static_cast<float>(K) + pr.eps);
      }
    }
    if (!weights_in) {  // (a warp without a token of its own: MP < warps)
      sg_wait<0>();
      __syncthreads();
    }
  }

  const int ft = warp & 1, kh = warp >> 1;  // row half, column quarter of a chunk
  float acc[MT][4];
  int c = 0, tile_i = 0;                                                       // chunk and tile being multiplied
  int ld_tile = 0, ld_chunk = 0;                                               // ... and being requested
#pragma unroll
  for (int q = 0; q < kSgStages - 1; ++q)
    if (++ld_chunk == n_chunks) {
      ld_chunk = 0;
      ++ld_tile;
    }
  const int n_copies = ONE ? n_chunks : total;
  for (int i = 0; i < n_copies; ++i) {
    // groups committed so far: (stages-1) chunks, then x, then one per iteration; copy i and x are
    // complete when at most stages-2 of the newest groups are still in flight (for i = 0 the x
    // group is the newest, so everything must have landed)
    if (i == 0) sg_wait<0>(); else sg_wait<kSgStages - 2>();
    __syncthreads();
    if (ONE) {
      if (i + kSgStages - 1 < n_copies) load_chunk((i + kSgStages - 1) % kSgStages, 0, i + kSgStages - 1);
      sg_commit();
    } else {
      if (i + kSgStages - 1 < n_copies) load_chunk((i + kSgStages - 1) % kSgStages, ld_tile, ld_chunk);
      sg_commit();
      if (++ld_chunk == n_chunks) {
        ld_chunk = 0;
        ++ld_tile;
      }
    }
    if (ONE ? i == 0 : c == 0) {
#pragma unroll
      for (int q = 0; q < MT; ++q) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
    }
    if (ONE) c = i;
    const bf16* tW = sW + (i % kSgStages) * kSgRows * kSgWStride;
#pragma unroll
    for (int ks = 0; ks < kSgChunk / 64; ++ks) {  // this warp's quarter of the chunk: 4 steps of 16
      const int kcol = kh * (kSgChunk / 4) + ks * 16;
      unsigned a[4];
      sg_ldm(a[0], a[1], a[2], a[3], tW + (ft * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kSgWStride + kcol + (lane >> 4) * 8);
      const int kx_col = c * kSgChunk + kcol;
      if (MT == 1) {  // up to 8 tokens: one 8-column operand
        unsigned b0, b1;
        sg_ldm2(b0, b1, sX + (lane & 7) * xs + kx_col + ((lane >> 3) & 1) * 8);
        sg_mma(acc[0], a, b0, b1);
      }
#pragma unroll
      for (int np = 0; np < MT / 2; ++np) {
        unsigned b0, b1, b2, b3;
        sg_ldm(b0, b1, b2, b3, sX + (np * 16 + (lane & 7) + (lane >> 4) * 8) * xs + kx_col + ((lane >> 3) & 1) * 8);
        sg_mma(acc[2 * np], a, b0, b1);
        sg_mma(acc[2 * np + 1], a, b2, b3);
      }
    }
    if (!ONE && ++c == n_chunks) {
      c = 0;
      finish_tile(acc, (t0 + tile_i * t_step) * kTileCols);
      ++tile_i;
    }
  }
  sg_wait<0>();
  if (ONE) finish_tile(acc, t0 * kTileCols);
}

// The sums of one row tile -> their place (the next tile's copies are in flight meanwhile).
template <int MT, int MODE>
__device__ void SkinnyBlock<MT, MODE>::finish_tile(float (&acc)[MT][4], int n0) const {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int M = args.M;
  const int ft = warp & 1, kh = warp >> 1;
  __syncthreads();  // (the tile before this one has been taken out of sRed)

  // add the four column quarters: warps 2..7 hand their sums to warps 0,1
  const int g = lane >> 2, t2 = (lane & 3) * 2;
  if (kh > 0) {
    float* d = sRed + ((kh - 1) * 32 + ft * 16) * MP;
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
      d[g * MP + nt * 8 + t2] = acc[nt][0];
      d[g * MP + nt * 8 + t2 + 1] = acc[nt][1];
      d[(g + 8) * MP + nt * 8 + t2] = acc[nt][2];
      d[(g + 8) * MP + nt * 8 + t2 + 1] = acc[nt][3];
    }
  }
  __syncthreads();
  if (kh == 0) {
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const float* d = sRed + (q * 32 + ft * 16) * MP;
#pragma unroll
      for (int nt = 0; nt < MT; ++nt) {
        acc[nt][0] += d[g * MP + nt * 8 + t2];
        acc[nt][1] += d[g * MP + nt * 8 + t2 + 1];
        acc[nt][2] += d[(g + 8) * MP + nt * 8 + t2];
        acc[nt][3] += d[(g + 8) * MP + nt * 8 + t2 + 1];
      }
    }
  }

  if (MODE == kSgSwiglu) {
    __syncthreads();
    if (kh == 0 && ft == 1) {  // up rows -> shared memory
#pragma unroll
      for (int nt = 0; nt < MT; ++nt) {
        sRed[g * MP + nt * 8 + t2] = acc[nt][0];
        sRed[g * MP + nt * 8 + t2 + 1] = acc[nt][1];
        sRed[(g + 8) * MP + nt * 8 + t2] = acc[nt][2];
        sRed[(g + 8) * MP + nt * 8 + t2 + 1] = acc[nt][3];
      }
    }
    __syncthreads();
    if (kh == 0 && ft == 0) {
#pragma unroll
      for (int nt = 0; nt < MT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int f = n0 + g + (e >> 1) * 8, m = nt * 8 + t2 + (e & 1);
          if (f < args.N && m < M) {
            const float inv = pr.h_in ? sInv[m] : 1.f;  // the row's norm factor (norm prologue)
            const float up = sRed[(g + (e >> 1) * 8) * MP + m] * inv;
            args.y[static_cast<size_t>(m) * args.ldy + f] = __float2bfloat16_rn(silu_fast(acc[nt][e] * inv * pr.scale) * up);
          }
        }
      }
    }
    return;  // (of this tile)
  }

  if (kh == 0) {
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = n0 + ft * 16 + g + (e >> 1) * 8, m = nt * 8 + t2 + (e & 1);
        if (n < args.N && m < M) {
          if (MODE == kSgStore) {
            const float inv = pr.h_in ? sInv[m] : 1.f;  // the row's norm factor (norm prologue)
            args.y[static_cast<size_t>(m) * args.ldy + n] = __float2bfloat16_rn(acc[nt][e] * inv);
          } else if (MODE == kSgStoreF32) {
            args.y32[static_cast<size_t>(m) * args.ldy + n] = args.y_scale * acc[nt][e];
          } else {
            atomicAdd(args.h_out + static_cast<size_t>(m) * args.N + n, pr.scale * acc[nt][e]);
          }
        }
      }
    }
  }
}

// MT: token tiles of 8 (1, 2, 4 or 8 -> up to 8, 16, 32, 64 tokens).
template <int MT, int MODE, bool ONE>
__global__ void __launch_bounds__(kSgThreads) skinny_gemm_kernel(const SkinnyArgs args) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_launch_dependents();
  const SkinnyBlock<MT, MODE> blk(args, blockIdx.x, gridDim.x, blockIdx.y, blockIdx.z, smem_raw);
  blk.request_weights();
  pdl_wait();
  blk.template run<ONE>();
}

// ---------------------------------------------------------------------------------------------
// A chain of products in one launch: phase p+1 reads what phase p wrote (the residual stream, an
// activation), so the phases are separated by barriers over the whole grid, and every block
// requests the first weight chunks of its next phase before it waits at the barrier: the weights
// stream while the grid synchronises.  One block per SM at most (the grid never exceeds what is
// resident at once, so every block reaches every barrier); the wait is bounded all the same and
// records a status instead of spinning for ever.
constexpr int kChainPhases = 4;
constexpr int kOneTile = 0x40000000;  // tile step of a block that takes exactly one row tile
constexpr unsigned kChainSpinLimit = 1u << 24;
constexpr unsigned long long kChainPerLaunch = 4096;  // what every launch adds to the counter (> 3 * 1024 arrivals)

struct SkinnyChain {
  SkinnyArgs phase[kChainPhases];
  int mode[kChainPhases];
  int gx[kChainPhases], gy[kChainPhases], gz[kChainPhases];
  int n_phases;
  unsigned long long* counter;  // grows by kChainPerLaunch per launch, whatever its grid
  int* status;                  // set to 1 when a barrier wait gave up
};

__device__ __forceinline__ unsigned long long chain_load(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];\n" : "=l"(v) : "l"(p) : "memory");
  return v;
}

template <int MT>
__global__ void __launch_bounds__(kSgThreads) skinny_chain_kernel(const SkinnyChain ch) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ unsigned long long s_base;
  pdl_launch_dependents();
  const int G = gridDim.x;
  auto for_block = [&](int p, int v, auto&& fn) {
    const int bx = v % ch.gx[p], by = (v / ch.gx[p]) % ch.gy[p], bz = v / (ch.gx[p] * ch.gy[p]);
    switch (ch.mode[p]) {
      case kSgStore: fn(SkinnyBlock<MT, kSgStore>(ch.phase[p], bx, kOneTile, by, bz, smem_raw)); break;
      case kSgSwiglu: fn(SkinnyBlock<MT, kSgSwiglu>(ch.phase[p], bx, kOneTile, by, bz, smem_raw)); break;
      default: fn(SkinnyBlock<MT, kSgResidual>(ch.phase[p], bx, kOneTile, by, bz, smem_raw)); break;
    }
  };
  auto n_blocks = [&](int p) { return ch.gx[p] * ch.gy[p] * ch.gz[p]; };

  bool requested = false;
  if (static_cast<int>(blockIdx.x) < n_blocks(0)) {
    for_block(0, blockIdx.x, [](const auto& blk) { blk.request_weights(); });
    requested = true;
  }
  pdl_wait();
  // every launch adds kChainPerLaunch in total, so the count at the start is a multiple of it
  // (plus the arrivals of faster blocks of this launch, fewer than that)
  if (threadIdx.x == 0) s_base = chain_load(ch.counter) / kChainPerLaunch * kChainPerLaunch;
  __syncthreads();
  const unsigned long long base = s_base;

  for (int p = 0; p < ch.n_phases; ++p) {
    for (int v = blockIdx.x; v < n_blocks(p); v += G) {
      for_block(p, v, [&](const auto& blk) {
        if (!requested) blk.request_weights();
        blk.template run<true>();
      });
      requested = false;
      __syncthreads();  // shared memory is free for the next block of work
    }
    if (p + 1 < ch.n_phases) {
      if (static_cast<int>(blockIdx.x) < n_blocks(p + 1)) {
        for_block(p + 1, blockIdx.x, [](const auto& blk) { blk.request_weights(); });
        requested = true;
      }
      // barrier p: everything written so far is visible to every block afterwards
      if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(ch.counter, 1ULL);
        const unsigned long long target = base + static_cast<unsigned long long>(p + 1) * G;
        unsigned spins = 0;
        while (chain_load(ch.counter) < target) {
          if (++spins > kChainSpinLimit) {
            atomicExch(ch.status, 1);
            break;
          }
          __nanosleep(40);  // a hundred and more blocks poll one line: leave room for the arrivals
        }
        __threadfence();
      }
      __syncthreads();
    }
  }
  // Block 0 is past the last barrier, so every arrival of this launch has been counted: it adds
  // what is missing to the next multiple.
  if (blockIdx.x == 0 && threadIdx.x == 0)
    atomicAdd(ch.counter, kChainPerLaunch - static_cast<unsigned long long>(ch.n_phases - 1) * G);
}

inline size_t skinny_smem(int MP, int kx) {
  return static_cast<size_t>(sg_stages(MP / 8)) * kSgRows * kSgWStride * sizeof(bf16) +
         static_cast<size_t>(MP) * (kx + 8) * sizeof(bf16) + 3 * 32 * MP * sizeof(float) +
         static_cast<size_t>(kx + MP) * sizeof(float);
}

template <int MT, int MODE>
int launch_skinny(const SkinnyArgs& a, int k_max, cudaStream_t stream) {
  constexpr int MP = MT * 8;
  const int kx = (min(a.k_slice, k_max) + kSgChunk - 1) / kSgChunk * kSgChunk;
  const size_t smem = skinny_smem(MP, kx);
  if (smem > 220 * 1024) return PMM_ERR_BAD_ARGUMENT;
  auto kern = skinny_gemm_kernel<MT, MODE, false>;
  auto kern_one = skinny_gemm_kernel<MT, MODE, true>;
  for (auto k : {kern, kern_one}) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  // no more blocks than are resident at once; each walks the row tiles bx, bx + gridDim.x, ...
  static size_t seen_smem = ~size_t(0);
  static int slots = 0;
  if (seen_smem != smem) {
    int per_sm = 0, n_sm = 0, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kSgThreads, smem) != cudaSuccess || per_sm < 1)
      return PMM_ERR_BAD_ARGUMENT;
    slots = per_sm * n_sm;
    seen_smem = smem;
  }
  const int cols_per_tile = MODE == kSgSwiglu ? 16 : kSgRows;
  const int n_tx = (a.N + cols_per_tile - 1) / cols_per_tile;
  const int gy = (k_max + a.k_slice - 1) / a.k_slice;
  int busy = 0;  // (K slice, product) pairs that have work: a product with a shorter K leaves its last slices empty
  for (int p = 0; p < a.n_problems; ++p) busy += (a.p[p].K + a.k_slice - 1) / a.k_slice;
  const int gx = std::min(n_tx, std::max(1, slots / std::max(busy, 1)));
  dim3 grid(gx, gy, a.n_problems);
  launch_pdl(gx == n_tx ? kern_one : kern, grid, dim3(kSgThreads), smem, stream, a);
  return launch_status();
}

template <int MODE>
int dispatch_skinny(const SkinnyArgs& a, int k_max, cudaStream_t stream) {
  if (a.M <= 8) return launch_skinny<1, MODE>(a, k_max, stream);
  if (a.M <= 16) return launch_skinny<2, MODE>(a, k_max, stream);
  if (a.M <= 32) return launch_skinny<4, MODE>(a, k_max, stream);
  if (a.M <= 64) return launch_skinny<8, MODE>(a, k_max, stream);
  return PMM_ERR_BAD_ARGUMENT;
}

template <int MT>
int launch_chain(const SkinnyChain& ch, size_t smem, int grid, cudaStream_t stream) {
  auto kern = skinny_chain_kernel<MT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
  if (e != cudaSuccess) return static_cast<int>(e);
  // every block must be resident at once: the barriers wait for all of them
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kSgThreads, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (per_sm < 1) return PMM_ERR_BAD_ARGUMENT;
  launch_pdl(kern, dim3(grid), dim3(kSgThreads), smem, stream, ch);
  return launch_status();
}

}  // namespace pmm

// mode 0 STORE (y bfloat16 [M, ldy]), 1 SWIGLU (w = [gate; up] rows, N = F, scale0 = gate multiplier),
// 2 RESIDUAL (h_out[M, N] += scale * y, k_split blocks along K, one or two products).
// x0/x1: bfloat16 activations, or nullptr with h_in/norm_w/eps for the RMSNorm prologue (K0 == width of h_in).
PMM_EXPORT int pmm_skinny_gemm(int mode, int M, int N, const void* x0, long long ldx0, const float* h_in,
                               const float* norm_w, float eps, const void* w0, int K0, float scale0,
                               const void* x1, long long ldx1, const void* w1, int K1, float scale1,
                               void* y, long long ldy, float* h_out, int k_split, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K0 <= 0 || K0 % 8 || (w1 && (K1 <= 0 || K1 % 8)) || k_split < 1) return PMM_ERR_BAD_ARGUMENT;
  if ((x0 == nullptr) == (h_in == nullptr)) return PMM_ERR_BAD_ARGUMENT;
  if (mode != pmm::kSgResidual && (k_split != 1 || w1 != nullptr || !y)) return PMM_ERR_BAD_ARGUMENT;
  if (mode == pmm::kSgResidual && !h_out) return PMM_ERR_BAD_ARGUMENT;
  pmm::SkinnyArgs a{};
  a.p[0] = {static_cast<const pmm::bf16*>(x0), ldx0, h_in, norm_w, eps, static_cast<const pmm::bf16*>(w0), K0, scale0};
  a.n_problems = 1;
  int k_max = K0;
  if (w1) {
    if (!x1) return PMM_ERR_BAD_ARGUMENT;
    a.p[1] = {static_cast<const pmm::bf16*>(x1), ldx1, nullptr, nullptr, 0.f, static_cast<const pmm::bf16*>(w1), K1, scale1};
    a.n_problems = 2;
    k_max = K0 > K1 ? K0 : K1;
  }
  a.M = M;
  a.N = N;
  const int chunks = (k_max + pmm::kSgChunk - 1) / pmm::kSgChunk;
  a.k_slice = ((chunks + k_split - 1) / k_split) * pmm::kSgChunk;
  a.y = static_cast<pmm::bf16*>(y);
  a.ldy = ldy;
  a.h_out = h_out;
  switch (mode) {
    case pmm::kSgStore: return pmm::dispatch_skinny<pmm::kSgStore>(a, k_max, stream);
    case pmm::kSgSwiglu: return pmm::dispatch_skinny<pmm::kSgSwiglu>(a, k_max, stream);
    case pmm::kSgResidual: return pmm::dispatch_skinny<pmm::kSgResidual>(a, k_max, stream);
    default: return PMM_ERR_BAD_ARGUMENT;
  }
}

// y32[M, ldy] (float32) = scale * (x[M, K] W[N, K]^T) for up to 64 rows of bfloat16 activations: the
// output head of steps that ask for few rows of logits.
PMM_EXPORT int pmm_skinny_gemm_f32out(int M, int N, const void* x, long long ldx, const void* w, int K, float scale,
                                      float* y32, long long ldy, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || K % 8 || !x || !w || !y32) return PMM_ERR_BAD_ARGUMENT;
  pmm::SkinnyArgs a{};
  a.p[0] = {static_cast<const pmm::bf16*>(x), ldx, nullptr, nullptr, 0.f, static_cast<const pmm::bf16*>(w), K, 1.f};
  a.n_problems = 1;
  a.M = M;
  a.N = N;
  a.k_slice = (K + pmm::kSgChunk - 1) / pmm::kSgChunk * pmm::kSgChunk;
  a.ldy = ldy;
  a.y32 = y32;
  a.y_scale = scale;
  return pmm::dispatch_skinny<pmm::kSgStoreF32>(a, K, stream);
}

// One phase of pmm_skinny_chain: the arguments of pmm_skinny_gemm without M, k_split and stream.
struct PmmSkinnyPhase {
  int mode, N;
  const void* x0;
  long long ldx0;
  const float* h_in;
  const float* norm_w;
  float eps;
  const void* w0;
  int K0;
  float scale0;
  const void* x1;
  long long ldx1;
  const void* w1;
  int K1;
  float scale1;
  void* y;
  long long ldy;
  float* h_out;
};

// Up to 4 products in one launch, each reading what the one before it wrote, separated by
// barriers over the grid (at most 16 tokens).  `counter` (one 64-bit integer, zero at first use,
// owned by these launches) and `status` (an int that becomes 1 if a barrier wait ever gave up;
// the results of that launch are then not to be used) live in device memory.
PMM_EXPORT int pmm_skinny_chain(const PmmSkinnyPhase* phases, int n_phases, int M, unsigned long long* counter,
                                int* status, cudaStream_t stream) {
  if (M <= 0 || n_phases <= 0) return 0;
  if (n_phases > pmm::kChainPhases || M > 16 || !counter || !status) return PMM_ERR_BAD_ARGUMENT;
  static int n_sm = 0;
  if (n_sm == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0)
      return PMM_ERR_BAD_ARGUMENT;
  }
  pmm::SkinnyChain ch{};
  ch.n_phases = n_phases;
  ch.counter = counter;
  ch.status = status;
  size_t smem = 0;
  int most = 1;
  for (int p = 0; p < n_phases; ++p) {
    const PmmSkinnyPhase& ph = phases[p];
    if (ph.N <= 0 || ph.K0 <= 0 || ph.K0 % 8 || (ph.w1 && (ph.K1 <= 0 || ph.K1 % 8 || !ph.x1))) return PMM_ERR_BAD_ARGUMENT;
    if ((ph.x0 == nullptr) == (ph.h_in == nullptr)) return PMM_ERR_BAD_ARGUMENT;
    if (ph.mode != pmm::kSgResidual && (ph.w1 != nullptr || !ph.y)) return PMM_ERR_BAD_ARGUMENT;
    if (ph.mode == pmm::kSgResidual && !ph.h_out) return PMM_ERR_BAD_ARGUMENT;
    if (ph.mode < 0 || ph.mode > 2) return PMM_ERR_BAD_ARGUMENT;
    pmm::SkinnyArgs& a = ch.phase[p];
    a.p[0] = {static_cast<const pmm::bf16*>(ph.x0), ph.ldx0, ph.h_in, ph.norm_w, ph.eps,
              static_cast<const pmm::bf16*>(ph.w0), ph.K0, ph.scale0};
    a.n_problems = 1;
    int k_max = ph.K0;
    if (ph.w1) {
      a.p[1] = {static_cast<const pmm::bf16*>(ph.x1), ph.ldx1, nullptr, nullptr, 0.f,
                static_cast<const pmm::bf16*>(ph.w1), ph.K1, ph.scale1};
      a.n_problems = 2;
      k_max = ph.K0 > ph.K1 ? ph.K0 : ph.K1;
    }
    a.M = M;
    a.N = ph.N;
    a.y = static_cast<pmm::bf16*>(ph.y);
    a.ldy = ph.ldy;
    a.h_out = ph.h_out;
    const int cols = ph.mode == pmm::kSgSwiglu ? 16 : pmm::kSgRows;
    const int gx = (ph.N + cols - 1) / cols;
    const int chunks = (k_max + pmm::kSgChunk - 1) / pmm::kSgChunk;
    // only the residual add can split K over blocks; as many slices as keep the phase within one
    // block per SM (a product with the norm prologue keeps its whole rows)
    int k_split = 1;
    if (ph.mode == pmm::kSgResidual && !ph.h_in) {
      k_split = n_sm / (gx * a.n_problems);
      if (k_split < 1) k_split = 1;
      if (k_split > chunks) k_split = chunks;
    }
    a.k_slice = ((chunks + k_split - 1) / k_split) * pmm::kSgChunk;
    ch.mode[p] = ph.mode;
    ch.gx[p] = gx;
    ch.gy[p] = (k_max + a.k_slice - 1) / a.k_slice;
    ch.gz[p] = a.n_problems;
    const int kx = (a.k_slice < k_max ? a.k_slice : (k_max + pmm::kSgChunk - 1) / pmm::kSgChunk * pmm::kSgChunk);
    const size_t need = pmm::skinny_smem(16, kx);
    if (need > smem) smem = need;
    const int blocks = ch.gx[p] * ch.gy[p] * ch.gz[p];
    if (blocks > most) most = blocks;
  }
  if (smem > 220 * 1024) return PMM_ERR_BAD_ARGUMENT;
  int grid = most < n_sm ? most : n_sm;
  if (grid > 1024) grid = 1024;  // the counter arithmetic allows 3 * 1024 arrivals a launch
  return pmm::launch_chain<2>(ch, smem, grid, stream);
}

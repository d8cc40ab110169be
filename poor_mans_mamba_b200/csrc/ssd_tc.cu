// Chunked Mamba2 SSD scan for prompt portions on the fifth-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory; bfloat16 activations, float state).
//
// The recurrence  s_t = s_{t-1} exp(a_t) + delta_t B_t x_t^T ,  y_t = C_t . s_t + D x_t ,
// a_t = delta_t A  (reference src/ops/gpu/mamba2_scan.cu:11-50 walks it token by token) is
// evaluated per chunk of 128 tokens of one sequence portion.  With cs_i = a_0 + ... + a_i inside
// the chunk and S the state at the chunk's start:
//   y_i   = sum_{j<=i} (C_i.B_j) exp(cs_i-cs_j) delta_j x_j  +  exp(cs_i) (C_i . S)  +  D x_i
//   S_end = exp(cs_last) S  +  sum_j exp(cs_last-cs_j) delta_j x_j B_j^T
// Three launches:
//   1. ssd_tc_state:   one block per (chunk, 128 channels of x): the local term of S_end as ONE
//                      product  D[channel, n] = sum_j (w_j x_j[channel]) B_j[n].  Both operands are
//                      the chunk's rows as they lie in memory (tokens = the K dimension, so both
//                      are MN-major; x is scaled by w_j in shared memory after it arrives); a thread
//                      reads its channel's row of the accumulator from tensor memory and the rows
//                      go out as float.
//   2. the state pass of ssd_chunked.cu walks the chunks of a sequence in float and hands the
//      state at every chunk's start on as bfloat16.
//   3. ssd_tc_output:  one block per (chunk, head, slab of up to 64 head channels), two threads
//                      per token: G = C B^T (128 x 128, tensor memory) and Y2 = C S^T are issued
//                      together; every thread reads its row of G, applies the decay, the causal
//                      mask and delta_j and writes the row of M as a bfloat16 operand into the
//                      shared memory that held B; Y1 = M x follows (x as it lies in memory,
//                      MN-major); y = Y1 + exp(cs_i) Y2 + D x, the gate y silu(z) fused.
// All tiles are brought by 16-byte asynchronous copies into the 128-byte swizzled layout the
// tensor core reads (rows beyond a short chunk are zero-filled, so they change nothing: their
// delta is zero).  Any head size that is a multiple of 16 up to 128 and any state size that is a
// multiple of 16 up to 256 is taken.  All differences of cs are <= 0: no exponential overflows;
// delta, cs and every accumulator are float.  Every mbarrier wait is bounded (status codes
// 31..33 in *status; the block then skips its output, frees its tensor memory and returns).
#include "tcgen05.cuh"

namespace pmm {

using bf16 = __nv_bfloat16;

constexpr int kTQ = 128;        // tokens per chunk
constexpr int kTSub = 16384;    // bytes of a sub-tile of 128 rows x 128 bytes
constexpr float kLog2e = 1.4426950408889634f;

// Launches the state pass of ssd_chunked.cu for chunks of `q` tokens.
int launch_ssd_state_pass(const float* chunk_state, const float* chunk_decay, bf16* start_state, float* state,
                          const int* cu, const int* slots, int n_seq, int H, int PN, int q, int skip_single, int n_multi,
                          cudaStream_t stream);

__device__ __forceinline__ int tq_swz(int row, int chunk) {
  return (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4);
}
__device__ __forceinline__ void tq_cp16(void* smem, const void* gmem, bool pred) {
  const unsigned s = smem_u32(smem);
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void tq_cp_wait() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ float tq_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned tq_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Which (first token, length) chunk `c` is; chunk ids run over the sequences in order.  Called by
// all threads of the block (a multiple of 32, at most 1,024); `sh` is shared memory for 36 ints.
// Every thread takes sequences tid, tid + blockDim, ...: the loads of the sequence bounds go out
// together instead of one after the other (a step may hold hundreds of sequences).
__device__ __forceinline__ bool tq_locate(const int* __restrict__ cu, int n_seq, int c, int& t0, int& len, int& seq_tokens,
                                          int* sh) {
  if (n_seq <= 4) {  // few sequences: every thread walks them itself
    int acc = 0;
    for (int seq = 0; seq < n_seq; ++seq) {
      const int lo = cu[seq], hi = cu[seq + 1];
      const int nc = (hi - lo + kTQ - 1) / kTQ;
      if (c < acc + nc) {
        t0 = lo + (c - acc) * kTQ;
        len = min(kTQ, hi - t0);
        seq_tokens = hi - lo;
        return true;
      }
      acc += nc;
    }
    return false;
  }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
  if (tid == 0) sh[34] = -1;
  int base = 0;  // chunks of the sequences before this round
  for (int s0 = 0; s0 < n_seq; s0 += blockDim.x) {
    const int s = s0 + tid;
    int lo = 0, hi = 0;
    if (s < n_seq) lo = cu[s], hi = cu[s + 1];
    const int nc = (hi - lo + kTQ - 1) / kTQ;
    int incl = nc;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) sh[warp] = incl;
    __syncthreads();
    int before = base;
    for (int w = 0; w < warp; ++w) before += sh[w];
    const int first = before + incl - nc;
    if (s < n_seq && c >= first && c < first + nc) {
      sh[34] = lo + (c - first) * kTQ;
      sh[35] = hi;
      sh[33] = hi - lo;
    }
    for (int w = 0; w < n_warps; ++w) base += sh[w];
    __syncthreads();
    if (sh[34] >= 0 || base > c) break;  // the same decision in every thread
  }
  if (sh[34] < 0) return false;
  t0 = sh[34];
  len = min(kTQ, sh[35] - t0);
  seq_tokens = sh[33];
  return true;
}

// 128 consecutive threads (four warps, `t` = 0..127 the thread's token): delta_t and cs_t (inclusive
// sum of delta * A over the chunk's tokens).  Tokens >= len get delta 0.  `totals` is shared memory
// for four floats; the caller synchronises the block before anybody reads what is derived from it.
struct TqDelta {
  float delta, incl;  // of this token; incl is the sum within the thread's warp only
};
__device__ __forceinline__ TqDelta tq_delta_warp(const bf16* __restrict__ dt_raw, long long ld_dt, float dt_scale,
                                                 float shift, float A, int t0, int len, int h, int t, float* totals) {
  TqDelta r;
  r.delta = t < len ? softplus_f(__bfloat162float(dt_raw[static_cast<long long>(t0 + t) * ld_dt + h]) * dt_scale + shift) : 0.f;
  float incl = r.delta * A;
  const int lane = t & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) totals[t >> 5] = incl;
  r.incl = incl;
  return r;
}
// cs of token t once `totals` is visible: the warp's inclusive sum plus the warps before it.
__device__ __forceinline__ float tq_cs(const TqDelta& d, int t, const float* totals) {
  float cs = d.incl;
  for (int w = 0; w < (t >> 5); ++w) cs += totals[w];
  return cs;
}

__device__ __forceinline__ unsigned tq_idesc(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | (static_cast<unsigned>(n >> 3) << 17) |
         (static_cast<unsigned>(kTQ >> 4) << 24);
}

// Descriptor of an MN-major operand of more than 64 rows: atoms of 64 (MN) x 8 (K) elements with
// the 128-byte swizzle, 1,024 bytes from one group of 8 K-rows to the next (stride byte offset),
// `atom_stride` bytes from one atom of 64 MN elements to the next (leading byte offset).
__device__ __forceinline__ unsigned long long umma_desc_mn(const void* tile, unsigned atom_stride) {
  const unsigned addr = smem_u32(tile);
  const unsigned lo = ((addr & 0x3FFFFu) >> 4) | ((atom_stride >> 4) << 16);
  const unsigned hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return (static_cast<unsigned long long>(hi) << 32) | lo;
}

__device__ __forceinline__ unsigned tq_tmem_alloc(unsigned* slot, int cols, int warp) {
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  return *slot;
}
__device__ __forceinline__ void tq_tmem_free(unsigned base, int cols, int warp) {
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(base), "r"(cols) : "memory");
  }
}

// ----------------------------------------------------------------------------- phase 1
// grid (chunks, groups * slabs_per_group); a slab is 128 consecutive channels of x inside one
// group (all its heads read the same B).  512 threads: the sixteen warps share the copies and the
// scaling; warps w, w+4, w+8, w+12 read the tensor-memory lanes 32 (w % 4) .. +31 (= channels)
// and split the columns.  The block in which a head begins also writes the head's exp(cs_last)
// and, for phase 3, delta_j and cs_j log2(e) of the chunk's tokens.
constexpr int kTState = 512;

__global__ void __launch_bounds__(kTState)
    ssd_tc_state_kernel(const bf16* __restrict__ xbc, int ld_xbc, const bf16* __restrict__ dt_raw, long long ld_dt,
                        float dt_scale, const float* __restrict__ dt_shift, const float* __restrict__ a_log,
                        const int* __restrict__ cu, int n_seq, float* __restrict__ chunk_state,
                        float* __restrict__ chunk_decay, float* __restrict__ chunk_dt, int H, int P, int N, int G,
                        int slabs_per_group, int tmem_cols, int skip_single, int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bar;
  __shared__ unsigned s_tmem;
  __shared__ int s_abort;
  __shared__ float s_w[8][kTQ];      // per head of the slab: exp(cs_last - cs_j) * delta_j
  __shared__ float s_tot[8][4];      // per head: the four warps' sums of delta * A

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x;
  int t0, len;
  __shared__ int s_loc[36];
  int seq_tokens;
  if (!tq_locate(cu, n_seq, c, t0, len, seq_tokens, s_loc)) return;
  if (skip_single && seq_tokens == 1) return;  // lone tokens of a mixed step are the token-serial kernel's
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sA = tiles;                 // [128 tokens][128 channels]: two atoms of 64 channels
  unsigned char* sB = tiles + 2 * kTSub;     // [128 tokens][N]: one atom per 64 state columns
  const int I = H * P;
  const int g = blockIdx.y / slabs_per_group, slab = blockIdx.y % slabs_per_group;
  const int ch_per_group = (H / G) * P;
  const int ch0 = g * ch_per_group + slab * kTQ;
  const int n_ch = min(kTQ, ch_per_group - slab * kTQ);
  const int head0 = ch0 / P;
  const int n_heads = (ch0 + n_ch - 1) / P - head0 + 1;  // <= 8: a head has at least 16 channels

  if (len == 1) {
    // A lone token (a decoding request in a mixed step): S_local[ch][n] = delta x[ch] B[n], no product
    // worth a tensor core.  Thread = (channel, quarter of the state columns).
    if (tid < n_heads) {
      const int h = head0 + tid;
      const float d = softplus_f(__bfloat162float(dt_raw[static_cast<long long>(t0) * ld_dt + h]) * dt_scale + dt_shift[h]);
      const float a = -expf(a_log[h]) * d;
      s_w[tid][0] = d;
      if (h * P >= ch0) {
        float* dtp = chunk_dt + (static_cast<size_t>(c) * H + h) * (2 * kTQ);
        dtp[0] = d;
        dtp[kTQ] = a * kLog2e;
        chunk_decay[static_cast<size_t>(c) * H + h] = expf(a);
      }
    }
    __syncthreads();
    const int ch = tid & (kTQ - 1), quarter = tid >> 7;
    if (ch < n_ch) {
      const bf16* rowp = xbc + static_cast<size_t>(t0) * ld_xbc;
      const float xv = __bfloat162float(rowp[ch0 + ch]) * s_w[(ch0 + ch) / P - head0][0];
      const bf16* bp = rowp + I + g * N;
      float* dst = chunk_state + (static_cast<size_t>(c) * I + ch0 + ch) * N;
      for (int n = quarter * (N / 4); n < (quarter + 1) * (N / 4); n += 4) {
        const uint2 braw = *reinterpret_cast<const uint2*>(bp + n);
        const float2 b01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&braw.x));
        const float2 b23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&braw.y));
        *reinterpret_cast<float4*>(dst + n) = make_float4(xv * b01.x, xv * b01.y, xv * b23.x, xv * b23.y);
      }
    }
    return;
  }

  if (tid == 0) {
    mbar_init(&bar, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // B rows of the chunk and x of the slab's channels, as they lie in memory (rows = tokens): both
  // operands are MN-major.  x is scaled by w_j in place below.
  {
    const int cpr = N / 8;  // 16-byte pieces per row of B
    int j = tid / cpr, ck = tid % cpr;
    const int dj = kTState / cpr, dck = kTState % cpr;
    while (j < kTQ) {
      const bool ok = j < len;
      tq_cp16(sB + (ck >> 3) * kTSub + tq_swz(j, ck & 7),
              xbc + (ok ? static_cast<size_t>(t0 + j) * ld_xbc + I + g * N + ck * 8 : 0), ok);
      j += dj, ck += dck;
      if (ck >= cpr) ck -= cpr, ++j;
    }
  }
  for (int i = tid; i < kTQ * 16; i += kTState) {
    const int j = i >> 4, ck = i & 15;
    const bool ok = j < len && ck * 8 < n_ch;
    tq_cp16(sA + (ck >> 3) * kTSub + tq_swz(j, ck & 7),
            xbc + (ok ? static_cast<size_t>(t0 + j) * ld_xbc + ch0 + ck * 8 : 0), ok);
  }
  // delta and cs of every head of the slab: head hh by the 128 threads of quarter hh % 4, a token each
  const int quarter = tid >> 7, tok = tid & (kTQ - 1);
  TqDelta dl[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int hh = quarter + 4 * r;
    if (hh < n_heads) {
      const int h = head0 + hh;
      dl[r] = tq_delta_warp(dt_raw, ld_dt, dt_scale, dt_shift[h], -expf(a_log[h]), t0, len, h, tok, s_tot[hh]);
    }
  }
  const unsigned tmem_base = tq_tmem_alloc(&s_tmem, tmem_cols, warp);  // includes a __syncthreads: s_tot is visible
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int hh = quarter + 4 * r;
    if (hh < n_heads) {
      const int h = head0 + hh;
      const float cs = tq_cs(dl[r], tok, s_tot[hh]);
      const float last = (s_tot[hh][0] + s_tot[hh][1]) + (s_tot[hh][2] + s_tot[hh][3]);
      s_w[hh][tok] = expf(last - cs) * dl[r].delta;
      if (h * P >= ch0) {  // the head begins in this slab
        float* dtp = chunk_dt + (static_cast<size_t>(c) * H + h) * (2 * kTQ);
        dtp[tok] = dl[r].delta;
        dtp[kTQ + tok] = cs * kLog2e;
        if (tok == 0) chunk_decay[static_cast<size_t>(c) * H + h] = expf(last);
      }
    }
  }
  tq_cp_wait();
  __syncthreads();  // s_w
  // every thread scales the pieces of x that it copied itself
#pragma unroll 4
  for (int i = tid; i < kTQ * 16; i += kTState) {
    const int j = i >> 4, ck = i & 15;
    if (j < len && ck * 8 < n_ch) {
      uint4* cell = reinterpret_cast<uint4*>(sA + (ck >> 3) * kTSub + tq_swz(j, ck & 7));
      const uint4 raw = *cell;
      const float w = s_w[(ch0 + ck * 8) / P - head0][j];
      const unsigned rw[4] = {raw.x, raw.y, raw.z, raw.w};
      unsigned o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rw[e]));
        o[e] = tq_pack(f.x * w, f.y * w);
      }
      *cell = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  fence_proxy_async();
  __syncthreads();

  if (tid == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned long long a_desc = umma_desc_mn(sA, kTSub);
    for (int s = 0; s * 128 < N; ++s) {  // up to 128 state columns (two atoms) an instruction
      const int ncols = min(128, N - 128 * s);
      const unsigned idesc = tq_idesc(ncols, true) | (1u << 15);  // A and B both MN-major
      const unsigned long long b_desc = umma_desc_mn(sB + 2 * s * kTSub, kTSub);
#pragma unroll
      for (int k = 0; k < kTQ / 16; ++k)  // 16 tokens further = 16 rows of 128 bytes in both operands
        umma_f16(tmem_base + 128 * s, a_desc + ((k * 16 * 128) >> 4), b_desc + ((k * 16 * 128) >> 4), idesc, k > 0 ? 1u : 0u);
    }
    umma_commit(&bar);
  }
  volatile int* abort_flag = &s_abort;
  bool ok = mbar_wait(&bar, 0, abort_flag);
  ok = __all_sync(0xffffffffu, ok);
  if (!ok && lane == 0) {
    if (!*abort_flag) atomicExch(status, 31);
    s_abort = 1;
  }
  if (ok) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const int rw = warp & 3, part = warp >> 2;
    const unsigned lane_base = tmem_base + (static_cast<unsigned>(rw * 32) << 16);
    // A lane holds a channel's row; rows go out 16 columns at a time through shared memory (the
    // operand tiles are no longer read), so that a store covers whole 64-byte pieces of 8 rows.
    float* stage = reinterpret_cast<float*>(tiles) + warp * (32 * 20);  // 32 rows of 16 + 4 floats
    float* dst = chunk_state + (static_cast<size_t>(c) * I + ch0 + rw * 32) * N;
    for (int c16 = part; c16 < N / 16; c16 += 4) {
      unsigned v[16];
      tmem_ld16(lane_base + c16 * 16, v);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4)
        *reinterpret_cast<float4*>(stage + lane * 20 + q4 * 4) =
            make_float4(__uint_as_float(v[q4 * 4]), __uint_as_float(v[q4 * 4 + 1]), __uint_as_float(v[q4 * 4 + 2]),
                        __uint_as_float(v[q4 * 4 + 3]));
      __syncwarp();
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        const int r = pass * 8 + (lane >> 2);
        if (rw * 32 + r < n_ch)
          *reinterpret_cast<float4*>(dst + static_cast<size_t>(r) * N + c16 * 16 + (lane & 3) * 4) =
              *reinterpret_cast<const float4*>(stage + r * 20 + (lane & 3) * 4);
      }
      __syncwarp();
    }
  }
  tq_tmem_free(tmem_base, tmem_cols, warp);
}

// ----------------------------------------------------------------------------- phase 3
// grid (chunks, H * (P / PB)); 512 threads: threads t, t + 128, t + 256 and t + 384 share token t of
// the chunk (= tensor-memory lane t) and split its columns.  The chunk's B rows and the slab's
// start-state rows lie one after the other in shared memory as ONE K-major operand of 128 + PB
// rows, so G = C B^T and Y2 = C S^T are one product.  Tensor memory: G columns 0..127, Y2
// columns 128..128+PB, Y1 columns 192..192+PB.
constexpr int kTOut = 512;

// Calls f(row, piece) for the 16-byte pieces tid, tid + 512, ... of `rows` rows of `cpr` pieces.
template <typename F>
__device__ __forceinline__ void tq_pieces(int tid, int rows, int cpr, F f) {
  int j = tid / cpr, ck = tid % cpr;
  const int dj = kTOut / cpr, dck = kTOut % cpr;
  while (j < rows) {
    f(j, ck);
    j += dj, ck += dck;
    if (ck >= cpr) ck -= cpr, ++j;
  }
}

__global__ void __launch_bounds__(kTOut, 2)
    ssd_tc_output_kernel(const bf16* __restrict__ xbc, int ld_xbc, const float* __restrict__ chunk_dt,
                         const float* __restrict__ d_skip, const int* __restrict__ cu, int n_seq,
                         const bf16* __restrict__ start_state, bf16* __restrict__ y, int H, int P, int N, int G, int PB,
                         const bf16* __restrict__ z_raw, long long ld_z, float z_scale, const float* __restrict__ z_bias,
                         int z_vec, int skip_single, int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bar1, bar2;
  __shared__ unsigned s_tmem;
  __shared__ int s_abort;
  __shared__ float s_delta[kTQ], s_csl[kTQ];  // delta_j and cs_j * log2(e)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = tid & (kTQ - 1), part = tid >> 7, rw = warp & 3;
  const int c = blockIdx.x;
  int t0, len;
  __shared__ int s_loc[36];
  int seq_tokens;
  if (!tq_locate(cu, n_seq, c, t0, len, seq_tokens, s_loc)) return;
  if (skip_single && seq_tokens == 1) return;  // lone tokens of a mixed step are the token-serial kernel's
  const int slabs = P / PB;
  const int h = blockIdx.y / slabs, p0 = (blockIdx.y % slabs) * PB;
  const int I = H * P, g = h / (H / G);
  const int nb = (N + 63) / 64;
  const int bs_sub = (kTQ + PB) * 128;  // bytes of one 64-column block of the [B ; S] operand
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sC = tiles;                                  // [128 tokens][N], K-major; later M [128][128]
  unsigned char* sBS = sC + (nb > 2 ? nb : 2) * kTSub;        // [128 tokens + PB channels][N], K-major; later z [128][PB]
  unsigned char* sX = sBS + nb * bs_sub;                      // [128 tokens][PB], MN-major; later y, in place
  const size_t col0 = static_cast<size_t>(h) * P + p0;

  if (len == 1) {
    // A lone token: y[p] = (C.B) delta x[p] + exp(cs_0) C.S[p] + D x[p], a warp per channel.
    const float* dtp = chunk_dt + (static_cast<size_t>(c) * H + h) * (2 * kTQ);
    const float d0 = dtp[0], e0 = tq_ex2(dtp[kTQ]), Dh1 = d_skip[h];
    const bf16* rowp = xbc + static_cast<size_t>(t0) * ld_xbc;
    const bf16* bp = rowp + I + g * N;
    const bf16* cp = bp + G * N;
    float cb = 0.f;
    float cv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (lane * 8 < N) {
      const uint4 cq = *reinterpret_cast<const uint4*>(cp + lane * 8), bq = *reinterpret_cast<const uint4*>(bp + lane * 8);
      const unsigned cw[4] = {cq.x, cq.y, cq.z, cq.w}, bw[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 cf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&cw[e]));
        const float2 bf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[e]));
        cv[2 * e] = cf.x, cv[2 * e + 1] = cf.y;
        cb += cf.x * bf.x + cf.y * bf.y;
      }
    }
    cb = warp_sum(cb);
    constexpr int kW = kTOut / 32;
    for (int pbase = warp; pbase < PB; pbase += 4 * kW) {  // four channels of this warp at a time: their loads go out together
      uint4 sq[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int p = pbase + u * kW;
        sq[u] = make_uint4(0u, 0u, 0u, 0u);
        if (p < PB && lane * 8 < N)
          sq[u] = *reinterpret_cast<const uint4*>(start_state + (static_cast<size_t>(c) * I + col0 + p) * N + lane * 8);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int p = pbase + u * kW;
        if (p >= PB) break;  // the same in every lane
        const unsigned sw[4] = {sq[u].x, sq[u].y, sq[u].z, sq[u].w};
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 sf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&sw[e]));
          acc += cv[2 * e] * sf.x + cv[2 * e + 1] * sf.y;
        }
        acc = warp_sum(acc);
        if (lane == 0) {
          const float xv = __bfloat162float(rowp[col0 + p]);
          float v = cb * d0 * xv + e0 * acc + Dh1 * xv;
          if (z_raw) {
            const float zv = __bfloat162float(z_raw[static_cast<long long>(t0) * ld_z + col0 + p]);
            v *= silu_fast(zv * z_scale + (z_bias ? z_bias[col0 + p] : 0.f));
          }
          y[static_cast<size_t>(t0) * I + col0 + p] = __float2bfloat16_rn(v);
        }
      }
    }
    return;
  }

  if (tid == 0) {
    mbar_init(&bar1, 1);
    mbar_init(&bar2, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  tq_pieces(tid, kTQ, N / 8, [&](int j, int ck) {
    const bool ok = j < len;
    const size_t src = ok ? static_cast<size_t>(t0 + j) * ld_xbc + I + g * N + ck * 8 : 0;
    tq_cp16(sBS + (ck >> 3) * bs_sub + tq_swz(j, ck & 7), xbc + src, ok);
    tq_cp16(sC + (ck >> 3) * kTSub + tq_swz(j, ck & 7), xbc + src + (ok ? G * N : 0), ok);
  });
  {
    const bf16* src = start_state + (static_cast<size_t>(c) * I + col0) * N;
    tq_pieces(tid, PB, N / 8, [&](int p, int ck) {
      tq_cp16(sBS + (ck >> 3) * bs_sub + tq_swz(kTQ + p, ck & 7), src + static_cast<size_t>(p) * N + ck * 8, true);
    });
  }
  tq_pieces(tid, kTQ, PB / 8, [&](int j, int ck) {
    const bool ok = j < len;
    tq_cp16(sX + tq_swz(j, ck), xbc + (ok ? static_cast<size_t>(t0 + j) * ld_xbc + col0 + ck * 8 : 0), ok);
  });
  if (tid < kTQ) {  // delta_j and cs_j log2(e), as phase 1 left them
    const float* dtp = chunk_dt + (static_cast<size_t>(c) * H + h) * (2 * kTQ);
    s_delta[tid] = dtp[tid];
    s_csl[tid] = dtp[kTQ + tid];
  }
  const float Dh = d_skip[h];
  tq_cp_wait();
  fence_proxy_async();
  const unsigned tmem_base = tq_tmem_alloc(&s_tmem, 256, warp);  // includes the __syncthreads after the copies

  if (tid == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned idesc = tq_idesc(kTQ + PB, false);
    for (int k = 0; k < N / 16; ++k)  // [G | Y2] = C [B ; S]^T, K = the state columns
      umma_f16(tmem_base, umma_desc(sC + (k >> 2) * kTSub) + 2 * (k & 3), umma_desc(sBS + (k >> 2) * bs_sub) + 2 * (k & 3),
               idesc, k > 0 ? 1u : 0u);
    umma_commit(&bar1);
  }
  volatile int* abort_flag = &s_abort;
  const unsigned lane_base = tmem_base + (static_cast<unsigned>(rw * 32) << 16);
  bool ok = mbar_wait(&bar1, 0, abort_flag);
  ok = __all_sync(0xffffffffu, ok);
  if (!ok && lane == 0) {
    if (!*abort_flag) atomicExch(status, 32);
    s_abort = 1;
  }
  const float csl_i = s_csl[row];
  unsigned char* sZ = sBS;
  if (ok) {
    // C, B and S have been read.  The gate's inputs of the chunk come into B's place while M is made.
    if (z_raw && z_vec) {
      tq_pieces(tid, kTQ, PB / 8, [&](int j, int ck) {
        const bool in = j < len;
        tq_cp16(sZ + tq_swz(j, ck), z_raw + (in ? static_cast<long long>(t0 + j) * ld_z + col0 + ck * 8 : 0), in);
      });
    }
    // M[i][j] = G[i][j] exp(cs_i - cs_j) delta_j for j <= i, as the A operand of Y1 = M x, in C's
    // place; this thread's 32 columns
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    unsigned char* sM = sC;
    const int jc = part;
    if (jc <= rw) {  // the warp's rows reach this block of 32 columns
      unsigned v[32];
      tmem_ld32(lane_base + jc * 32, v);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        float m[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int j = jc * 32 + c8 * 8 + e;
          m[e] = j <= row ? __uint_as_float(v[c8 * 8 + e]) * tq_ex2(csl_i - s_csl[j]) * s_delta[j] : 0.f;
        }
        uint4 pk;
        pk.x = tq_pack(m[0], m[1]);
        pk.y = tq_pack(m[2], m[3]);
        pk.z = tq_pack(m[4], m[5]);
        pk.w = tq_pack(m[6], m[7]);
        const int ck = jc * 4 + c8;
        *reinterpret_cast<uint4*>(sM + (ck >> 3) * kTSub + tq_swz(row, ck & 7)) = pk;
      }
    } else {
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        const int ck = jc * 4 + c8;
        *reinterpret_cast<uint4*>(sM + (ck >> 3) * kTSub + tq_swz(row, ck & 7)) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    fence_proxy_async();
  }
  tq_cp_wait();  // the gate's inputs
  __syncthreads();
  if (tid == 0 && !s_abort) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned idesc_y1 = tq_idesc(PB, true);
    const unsigned long long x_desc = umma_desc(sX);
#pragma unroll
    for (int k = 0; k < kTQ / 16; ++k)
      umma_f16(tmem_base + 192, umma_desc(sC + (k >> 2) * kTSub) + 2 * (k & 3), x_desc + ((k * 16 * 128) >> 4), idesc_y1,
               k > 0 ? 1u : 0u);
    umma_commit(&bar2);
  }
  if (ok) {
    ok = mbar_wait(&bar2, 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok && lane == 0) {
      if (!*abort_flag) atomicExch(status, 33);
      s_abort = 1;
    }
  }
  if (ok) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const float e_i = tq_ex2(csl_i);
    const bool row_ok = row < len;
    for (int pc = part; pc < PB / 16; pc += 4) {
      unsigned y1[16], y2[16];
      tmem_ld16(lane_base + 192 + pc * 16, y1);
      tmem_ld16(lane_base + 128 + pc * 16, y2);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int ck = pc * 2 + hf;
        uint4* cell = reinterpret_cast<uint4*>(sX + tq_swz(row, ck));  // x in, y out: the product has read x
        const uint4 xq = *cell;
        const unsigned xw[4] = {xq.x, xq.y, xq.z, xq.w};
        unsigned zw[4] = {0u, 0u, 0u, 0u};
        if (z_raw) {
          if (z_vec) {
            const uint4 zq = *reinterpret_cast<const uint4*>(sZ + tq_swz(row, ck));
            zw[0] = zq.x, zw[1] = zq.y, zw[2] = zq.z, zw[3] = zq.w;
          } else if (row_ok) {  // rows of z that do not start on 16-byte boundaries
            const bf16* zp = z_raw + static_cast<long long>(t0 + row) * ld_z + col0 + ck * 8;
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2)
              zw[e2] = static_cast<unsigned>(__bfloat16_as_ushort(zp[2 * e2])) |
                       (static_cast<unsigned>(__bfloat16_as_ushort(zp[2 * e2 + 1])) << 16);
          }
        }
        unsigned out[4];
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) {
          const float2 xv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xw[e2]));
          const int e = hf * 8 + e2 * 2;
          float v0 = __uint_as_float(y1[e]) + e_i * __uint_as_float(y2[e]) + Dh * xv.x;
          float v1 = __uint_as_float(y1[e + 1]) + e_i * __uint_as_float(y2[e + 1]) + Dh * xv.y;
          if (z_raw) {  // gate fused: y * silu(z), z = z_raw * z_scale + z_bias
            const float2 zv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&zw[e2]));
            const size_t ch = col0 + ck * 8 + e2 * 2;
            v0 *= silu_fast(zv.x * z_scale + (z_bias ? z_bias[ch] : 0.f));
            v1 *= silu_fast(zv.y * z_scale + (z_bias ? z_bias[ch + 1] : 0.f));
          }
          out[e2] = tq_pack(v0, v1);
        }
        *cell = make_uint4(out[0], out[1], out[2], out[3]);
      }
    }
  }
  __syncthreads();
  if (!s_abort) {  // the finished rows go out in whole lines
    tq_pieces(tid, len, PB / 8, [&](int j, int ck) {
      *reinterpret_cast<uint4*>(y + static_cast<size_t>(t0 + j) * I + col0 + ck * 8) =
          *reinterpret_cast<const uint4*>(sX + tq_swz(j, ck));
    });
  }
  tq_tmem_free(tmem_base, 256, warp);
}

}  // namespace pmm

// Head sizes and state sizes the tcgen05 scan takes: multiples of 16, up to 128 and up to 256.
PMM_EXPORT int pmm_ssd_tc_supported(int P, int N) {
  return (P >= 16 && P <= 128 && P % 16 == 0 && N >= 16 && N <= 256 && N % 16 == 0) ? 1 : 0;
}

// xbc [T, ld_xbc] = [x | B | C] after the convolution; dt_raw [T, ld_dt]; state [slots, H, P, N]
// float.  Scratch: chunk_state n_chunks*H*P*N floats, chunk_decay n_chunks*H floats, chunk_dt
// n_chunks*H*256 floats, start_state n_chunks*H*P*N bfloat16 (16-byte aligned); n_chunks = sum over
// sequences of ceil(new tokens / 128).
// z_raw (or nullptr): the gate's input [T, ld_z], y <- y * silu(z_raw * z_scale + z_bias).
// skip_single: sequences that bring exactly one token are left alone (state and y): in a mixed step
// the token-serial kernel takes them (pmm_ssm_scan_seq with one_token = 2); n_multi is then the
// number of sequences that bring more than one token (0: not known).
// status: one int in device memory that stays 0 unless a bounded wait gave up.
PMM_EXPORT int pmm_ssd_tc(const void* xbc, int ld_xbc, const void* dt_raw, long long ld_dt, float dt_scale,
                          const float* dt_shift, const float* a_log, const float* d_skip, float* state, const int* cu,
                          const int* slots, void* y, float* chunk_state, float* chunk_decay, float* chunk_dt,
                          void* start_state, int n_seq, int n_chunks, int H, int P, int N, int G, const void* z_raw, long long ld_z,
                          float z_scale, const float* z_bias, int skip_single, int n_multi, int* status,
                          cudaStream_t stream) {
  using namespace pmm;
  if (n_seq <= 0 || n_chunks <= 0) return 0;
  if (!pmm_ssd_tc_supported(P, N) || H <= 0 || G <= 0 || H % G || n_seq > 65535 || !chunk_state || !chunk_decay ||
      !chunk_dt || !start_state || reinterpret_cast<uintptr_t>(start_state) % 16 || !status || ld_xbc % 8 ||
      reinterpret_cast<uintptr_t>(xbc) % 16 || reinterpret_cast<uintptr_t>(y) % 16)
    return PMM_ERR_BAD_ARGUMENT;
  const int z_vec = (z_raw && ld_z % 8 == 0 && reinterpret_cast<uintptr_t>(z_raw) % 16 == 0) ? 1 : 0;
  const int PB = P <= 64 ? P : (P % 64 == 0 ? 64 : (P % 48 == 0 ? 48 : (P % 32 == 0 ? 32 : 16)));
  const int nb = (N + 63) / 64;
  const int ch_per_group = (H / G) * P;
  const int slabs_per_group = (ch_per_group + kTQ - 1) / kTQ;
  if (static_cast<long long>(G) * slabs_per_group > 65535 || static_cast<long long>(H) * (P / PB) > 65535)
    return PMM_ERR_BAD_ARGUMENT;
  int tmem_cols = 32;
  while (tmem_cols < N) tmem_cols *= 2;
  const size_t smem1 = 1024 + 2 * kTSub + static_cast<size_t>(nb + (nb & 1)) * kTSub;
  const size_t smem3 = 1024 + static_cast<size_t>(nb > 2 ? nb : 2) * kTSub + static_cast<size_t>(nb) * (kTQ + PB) * 128 + kTSub;
  static size_t set1 = 0, set3 = 0;  // the opt-in to large shared memory, raised when a larger shape comes
  if (smem1 > set1) {
    cudaError_t e = cudaFuncSetAttribute(ssd_tc_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem1));
    if (e != cudaSuccess) return static_cast<int>(e);
    set1 = smem1;
  }
  if (smem3 > set3) {
    cudaError_t e = cudaFuncSetAttribute(ssd_tc_output_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem3));
    if (e != cudaSuccess) return static_cast<int>(e);
    set3 = smem3;
  }
  const bf16* xb = static_cast<const bf16*>(xbc);
  const bf16* dtb = static_cast<const bf16*>(dt_raw);
  launch_pdl(ssd_tc_state_kernel, dim3(n_chunks, G * slabs_per_group), dim3(kTState), smem1, stream, xb, ld_xbc, dtb, ld_dt,
             dt_scale, dt_shift, a_log, cu, n_seq, chunk_state, chunk_decay, chunk_dt, H, P, N, G, slabs_per_group, tmem_cols,
             skip_single, status);
  int rc = launch_ssd_state_pass(chunk_state, chunk_decay, static_cast<bf16*>(start_state), state, cu, slots, n_seq, H,
                                 P * N, kTQ, skip_single, n_multi, stream);
  if (rc != 0) return rc;
  launch_pdl(ssd_tc_output_kernel, dim3(n_chunks, H * (P / PB)), dim3(kTOut), smem3, stream, xb, ld_xbc,
             static_cast<const float*>(chunk_dt), d_skip, cu, n_seq, static_cast<const bf16*>(start_state),
             static_cast<bf16*>(y), H, P, N, G, PB, static_cast<const bf16*>(z_raw), ld_z, z_scale, z_bias, z_vec, skip_single, status);
  return launch_status();
}

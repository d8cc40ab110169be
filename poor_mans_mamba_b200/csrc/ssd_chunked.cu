// Chunked Mamba2 SSD scan for prompt portions (bfloat16 activations, float state), on
// tensor cores.  The recurrence
//   s_t = s_{t-1} * exp(a_t) + delta_t * B_t x_t^T ,   y_t = C_t . s_t + D x_t ,  a_t = delta_t * A
// is evaluated per chunk of 64 tokens of one sequence portion and one head.  With
// cs_i = a_0 + ... + a_i inside the chunk and S the state at the chunk's start:
//   y_i   = sum_{j<=i} (C_i.B_j) exp(cs_i-cs_j) delta_j x_j  +  exp(cs_i) (C_i . S)  +  D x_i
//   S_end = exp(cs_last) S  +  sum_j exp(cs_last-cs_j) delta_j B_j x_j^T
// Three launches, all parallel over chunks except the cheap middle one:
//   1. ssd_chunk_state:  local term of S_end and exp(cs_last) per (chunk, head)   -> scratch;
//                        extra blocks of the same launch form C B^T per (chunk, group), which
//                        all heads of a group share                                -> scratch
//   2. ssd_state_pass:   walks a sequence's chunks in float: start[c] <- state at the start of
//                        chunk c (the request's saved state for c = 0) as bfloat16, the form
//                        in which phase 3 multiplies it; final state -> slot (float)
//   3. ssd_chunk_output: y for every token from C, B, x and the chunk's start state
// All differences of cs are <= 0, so no exponential overflows; delta, cs and every
// accumulator are float; the start state is rounded to bfloat16 only as an MMA operand.
// Chunks are aligned to the start of the portion in this step; a portion that is cut
// elsewhere gives the same result up to rounding.  Rows beyond a short chunk are zero-filled
// (delta = 0), so they change nothing.
// (reference src/ops/gpu/mamba2_scan.cu:11-50 walks the tokens serially; the formulas above
// are that recurrence unrolled over a chunk.)
#include "common.cuh"

namespace pmm {

using bf16 = __nv_bfloat16;
constexpr int kQ = 64;  // tokens per chunk

__device__ __forceinline__ void ssd_cp_async16(void* smem, const void* gmem, bool pred) {
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void ssd_cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::);
}
__device__ __forceinline__ void ssd_ldm(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ssd_ldm_t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ssd_mma(float* d, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned ssd_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ unsigned ssd_scale2(unsigned packed, float s0, float s1) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&packed));
  return ssd_pack(f.x * s0, f.y * s1);
}

// Which (sequence, first token, length) chunk `c` is; chunk ids run over the sequences in order.
__device__ __forceinline__ bool ssd_locate(const int* __restrict__ cu, int n_seq, int c, int& seq,
                                           int& t0, int& len, int& first_chunk) {
  int acc = 0;
  for (seq = 0; seq < n_seq; ++seq) {
    const int n = cu[seq + 1] - cu[seq];
    const int nc = (n + kQ - 1) / kQ;
    if (c < acc + nc) {
      t0 = cu[seq] + (c - acc) * kQ;
      len = min(kQ, cu[seq + 1] - t0);
      first_chunk = acc;
      return true;
    }
    acc += nc;
  }
  return false;
}

// delta_j, cs_j (inclusive cumulative sum of delta_j * A) for the chunk's tokens; rows >= len: 0.
// Called by all threads; the first warp does the scan.  Ends with a __syncthreads().
__device__ __forceinline__ void ssd_delta_cumsum(const bf16* __restrict__ dt_raw, long long ld_dt,
                                                 float dt_scale, float shift, float A, int t0, int len,
                                                 int h, float* s_delta, float* s_cs) {
  const int tid = threadIdx.x;
  if (tid < 32) {
    float d0 = 0.f, d1 = 0.f;
    const int j0 = 2 * tid, j1 = 2 * tid + 1;
    if (j0 < len) d0 = softplus_f(__bfloat162float(dt_raw[static_cast<long long>(t0 + j0) * ld_dt + h]) * dt_scale + shift);
    if (j1 < len) d1 = softplus_f(__bfloat162float(dt_raw[static_cast<long long>(t0 + j1) * ld_dt + h]) * dt_scale + shift);
    const float a0 = d0 * A, a1 = d1 * A;
    const float pair = a0 + a1;
    float incl = pair;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, incl, o);
      if (tid >= o) incl += up;
    }
    const float excl = incl - pair;
    s_delta[j0] = d0;
    s_delta[j1] = d1;
    s_cs[j0] = excl + a0;
    s_cs[j1] = excl + pair;
  }
  __syncthreads();
}

// ----------------------------------------------------------------------------- phase 1
// Blocks with blockIdx.y < H: the local state of (chunk, head).  Blocks with blockIdx.y >= H:
// the products C_i . B_j of (chunk, group blockIdx.y - H), float [64][64], for phase 3.
template <int P, int N>
__global__ void __launch_bounds__(128)
    ssd_chunk_state_kernel(const bf16* __restrict__ xbc, int ld_xbc, const bf16* __restrict__ dt_raw,
                           long long ld_dt, float dt_scale, const float* __restrict__ dt_shift,
                           const float* __restrict__ a_log, const int* __restrict__ cu, int n_seq,
                           float* __restrict__ chunk_state, float* __restrict__ chunk_decay,
                           float* __restrict__ chunk_cb, int H, int G) {
  constexpr int SX = P + 8, SB = N + 8;
  constexpr int NB = N < 64 ? N : 64;  // columns of the state per work unit
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float s_delta[kQ], s_cs[kQ], s_w[kQ];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x;
  int seq, t0, len, first;
  if (!ssd_locate(cu, n_seq, c, seq, t0, len, first)) return;
  const int I = H * P;

  if (static_cast<int>(blockIdx.y) >= H) {
    const int g = blockIdx.y - H;
    bf16* sC = reinterpret_cast<bf16*>(smem_raw);
    bf16* sBg = sC + kQ * SB;
    for (int i = tid; i < kQ * (N / 8); i += 128) {
      const int r = i / (N / 8), col = i % (N / 8);
      const bool ok = r < len;
      const size_t row = ok ? static_cast<size_t>(t0 + r) * ld_xbc : 0;
      ssd_cp_async16(sBg + r * SB + col * 8, xbc + row + (ok ? I + g * N + col * 8 : 0), ok);
      ssd_cp_async16(sC + r * SB + col * 8, xbc + row + (ok ? I + G * N + g * N + col * 8 : 0), ok);
    }
    ssd_cp_async_wait_all();
    __syncthreads();
    float gacc[kQ / 8][4];
#pragma unroll
    for (int i = 0; i < kQ / 8; ++i) gacc[i][0] = gacc[i][1] = gacc[i][2] = gacc[i][3] = 0.f;
    const bf16* c_lane = sC + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SB + (lane >> 4) * 8;
    const bf16* b_lane = sBg + ((lane & 7) + (lane >> 4) * 8) * SB + ((lane >> 3) & 1) * 8;
#pragma unroll 2
    for (int ks = 0; ks < N / 16; ++ks) {
      unsigned a[4];
      ssd_ldm(a[0], a[1], a[2], a[3], c_lane + ks * 16);
#pragma unroll
      for (int np = 0; np < kQ / 16; ++np) {
        if (np <= warp) {  // only the tokens up to this warp's diagonal block are read later
          unsigned b0, b1, b2, b3;
          ssd_ldm(b0, b1, b2, b3, b_lane + np * 16 * SB + ks * 16);
          ssd_mma(gacc[2 * np], a, b0, b1);
          ssd_mma(gacc[2 * np + 1], a, b2, b3);
        }
      }
    }
    float* dst = chunk_cb + (static_cast<size_t>(c) * G + g) * kQ * kQ;
    const int i_lo = warp * 16 + (lane >> 2);
#pragma unroll
    for (int nt = 0; nt < kQ / 8; ++nt) {
      if (nt / 2 <= warp) {
        const int j = nt * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(dst + i_lo * kQ + j) = make_float2(gacc[nt][0], gacc[nt][1]);
        *reinterpret_cast<float2*>(dst + (i_lo + 8) * kQ + j) = make_float2(gacc[nt][2], gacc[nt][3]);
      }
    }
    return;
  }

  const int h = blockIdx.y;
  const int g = h / (H / G);
  bf16* sX = reinterpret_cast<bf16*>(smem_raw);
  bf16* sB = sX + kQ * SX;
  for (int i = tid; i < kQ * (P / 8); i += 128) {
    const int r = i / (P / 8), col = i % (P / 8);
    const bool ok = r < len;
    ssd_cp_async16(sX + r * SX + col * 8, xbc + (ok ? static_cast<size_t>(t0 + r) * ld_xbc + h * P + col * 8 : 0), ok);
  }
  for (int i = tid; i < kQ * (N / 8); i += 128) {
    const int r = i / (N / 8), col = i % (N / 8);
    const bool ok = r < len;
    ssd_cp_async16(sB + r * SB + col * 8, xbc + (ok ? static_cast<size_t>(t0 + r) * ld_xbc + I + g * N + col * 8 : 0), ok);
  }
  ssd_delta_cumsum(dt_raw, ld_dt, dt_scale, dt_shift[h], -expf(a_log[h]), t0, len, h, s_delta, s_cs);
  if (tid < kQ) s_w[tid] = expf(s_cs[kQ - 1] - s_cs[tid]) * s_delta[tid];
  if (tid == 0) chunk_decay[static_cast<size_t>(c) * H + h] = expf(s_cs[kQ - 1]);
  ssd_cp_async_wait_all();
  __syncthreads();
  // x_j <- w_j x_j once for the block (the product is rounded to bfloat16 as an mma operand)
  for (int i = tid; i < kQ * (P / 2); i += 128) {
    const int r = i / (P / 2), col = (i % (P / 2)) * 2;
    unsigned* px = reinterpret_cast<unsigned*>(sX + r * SX + col);
    *px = ssd_scale2(*px, s_w[r], s_w[r]);
  }
  __syncthreads();

  float* dst = chunk_state + (static_cast<size_t>(c) * H + h) * P * N;
  constexpr int UNITS = (P / 16) * (N / NB);
  for (int u = warp; u < UNITS; u += 4) {
    const int mt = u / (N / NB), nb = u % (N / NB);
    float acc[NB / 8][4];
#pragma unroll
    for (int i = 0; i < NB / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    // fragments of step ks+1 are requested before the products of step ks
    unsigned fa[2][4], fb[2][NB / 16][4];
    auto load_frag = [&](int ks) {
      // A[m = p][k = token] from sX[token][p]: transposed 8x8 loads
      ssd_ldm_t(fa[ks & 1][0], fa[ks & 1][1], fa[ks & 1][2], fa[ks & 1][3],
                sX + (ks * 16 + (lane >> 4) * 8 + (lane & 7)) * SX + mt * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
      for (int np = 0; np < NB / 16; ++np)
        ssd_ldm_t(fb[ks & 1][np][0], fb[ks & 1][np][1], fb[ks & 1][np][2], fb[ks & 1][np][3],
                  sB + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SB + nb * NB + np * 16 + (lane >> 4) * 8);
    };
    load_frag(0);
#pragma unroll
    for (int ks = 0; ks < kQ / 16; ++ks) {
      if (ks + 1 < kQ / 16) load_frag(ks + 1);
#pragma unroll
      for (int np = 0; np < NB / 16; ++np) {
        ssd_mma(acc[2 * np], fa[ks & 1], fb[ks & 1][np][0], fb[ks & 1][np][1]);
        ssd_mma(acc[2 * np + 1], fa[ks & 1], fb[ks & 1][np][2], fb[ks & 1][np][3]);
      }
    }
    const int p_lo = mt * 16 + (lane >> 2);
#pragma unroll
    for (int nt = 0; nt < NB / 8; ++nt) {
      const int n = nb * NB + nt * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(dst + static_cast<size_t>(p_lo) * N + n) = make_float2(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<float2*>(dst + static_cast<size_t>(p_lo + 8) * N + n) = make_float2(acc[nt][2], acc[nt][3]);
    }
  }
}

// ----------------------------------------------------------------------------- phase 2
// One sequence's chunks folded into its state, four state elements `e .. e+3` of head h per thread:
// the state before each chunk goes to start_state (bfloat16), the state after the last to `state`.
__device__ __forceinline__ void ssd_pass_sequence(const float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                                                  bf16* __restrict__ start_state, float* __restrict__ state, int slot, int H,
                                                  int PN, int h, int e, int first, int nc) {
  float4* sp = reinterpret_cast<float4*>(state + (static_cast<size_t>(slot) * H + h) * PN + e);
  float4 s = *sp;
  // The chain through s is short; the loads are what cost: eight chunks are requested at a time,
  // and the next eight while these are folded in, so a walk costs about one round trip to L2.
  constexpr int kAhead = 8;
  auto request = [&](float4 (&local)[kAhead], float (&decay)[kAhead], int c0) {
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      const int c = min(c0 + i, nc - 1);
      const size_t ch = static_cast<size_t>(first + c) * H + h;
      local[i] = __ldcs(reinterpret_cast<const float4*>(chunk_state + ch * PN + e));
      decay[i] = chunk_decay[ch];
    }
  };
  auto fold = [&](const float4 (&local)[kAhead], const float (&decay)[kAhead], int c0) {
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      if (c0 + i < nc) {
        const size_t ch = static_cast<size_t>(first + c0 + i) * H + h;
        uint2 packed;  // the state at the start of this chunk
        packed.x = ssd_pack(s.x, s.y);
        packed.y = ssd_pack(s.z, s.w);
        *reinterpret_cast<uint2*>(start_state + ch * PN + e) = packed;
        s.x = s.x * decay[i] + local[i].x;
        s.y = s.y * decay[i] + local[i].y;
        s.z = s.z * decay[i] + local[i].z;
        s.w = s.w * decay[i] + local[i].w;
      }
    }
  };
  float4 la[kAhead], lb[kAhead];
  float da[kAhead], db[kAhead];
  request(la, da, 0);
  for (int c0 = 0; c0 < nc; c0 += 2 * kAhead) {
    const bool second = c0 + kAhead < nc;
    if (second) request(lb, db, c0 + kAhead);
    fold(la, da, c0);
    if (second) {
      if (c0 + 2 * kAhead < nc) request(la, da, c0 + 2 * kAhead);
      fold(lb, db, c0 + kAhead);
    }
  }
  *sp = s;
}

__global__ void ssd_state_pass_kernel(const float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                                      bf16* __restrict__ start_state, float* __restrict__ state,
                                      const int* __restrict__ cu, const int* __restrict__ slots, int H, int PN, int q,
                                      int n_seq, int seqs_per_block, int skip_single) {
  pdl_launch_dependents();
  pdl_wait();
  // four state elements per thread (P*N is a multiple of 4 for every compiled pair)
  const int e = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const int h = blockIdx.y, seq0 = blockIdx.z * seqs_per_block;
  // chunks of the sequences before the block's first one: the threads share the sequences, so the
  // loads of their bounds go out together (a step may hold hundreds of sequences)
  __shared__ int s_first[32];
  int mine = 0;
  for (int s = threadIdx.x; s < seq0; s += blockDim.x) mine += (cu[s + 1] - cu[s] + q - 1) / q;  // q: tokens per chunk
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
  if ((threadIdx.x & 31) == 0) s_first[threadIdx.x >> 5] = mine;
  __syncthreads();
  int first = 0;
  for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) first += s_first[w];
  if (e >= PN) return;
  // a block takes several sequences in turn when a step holds many (mostly short) ones
  for (int seq = seq0; seq < min(n_seq, seq0 + seqs_per_block); ++seq) {
    const int n_tok = cu[seq + 1] - cu[seq];
    const int nc = (n_tok + q - 1) / q;
    if (nc <= 0) continue;
    if (!(skip_single && n_tok == 1))  // (a lone token is left to the token-serial kernel)
      ssd_pass_sequence(chunk_state, chunk_decay, start_state, state, slots[seq], H, PN, h, e, first, nc);
    first += nc;
  }
}

// The same pass for a mixed step, in which most sequences bring one token and are none of this
// pass's business (the token-serial kernel takes them): block z takes the z-th sequence that brings
// more than one token.  Every block finds it by itself: the threads read the bounds of all sequences
// at once (a run of sequences per thread), a scan over the 256 runs gives each run's place among the
// sequences with more than one token and among the chunks, and the thread whose run holds number z
// announces it.  (A block that walked the sequences in turn paid a round trip to L2 for each of the
// 32 lone ones: 33 us a layer in a step of 36 sequences, against 8 for the four that matter.)
__global__ void __launch_bounds__(256)
    ssd_state_pass_multi_kernel(const float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                                bf16* __restrict__ start_state, float* __restrict__ state, const int* __restrict__ cu,
                                const int* __restrict__ slots, int H, int PN, int q, int n_seq) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_multi[256], s_chunks[256];
  __shared__ int s_seq, s_first, s_nc;
  const int tid = threadIdx.x;
  const int per = (n_seq + 255) / 256;
  const int lo = min(n_seq, tid * per), hi = min(n_seq, lo + per);
  int multi = 0, chunks = 0;
  for (int s = lo; s < hi; ++s) {
    const int n = cu[s + 1] - cu[s];
    multi += n > 1 ? 1 : 0;
    chunks += (n + q - 1) / q;
  }
  s_multi[tid] = multi;
  s_chunks[tid] = chunks;
  if (tid == 0) s_seq = -1;
  __syncthreads();
  for (int o = 1; o < 256; o <<= 1) {  // inclusive scan over the runs
    const int a = tid >= o ? s_multi[tid - o] : 0, b = tid >= o ? s_chunks[tid - o] : 0;
    __syncthreads();
    s_multi[tid] += a;
    s_chunks[tid] += b;
    __syncthreads();
  }
  const int want = blockIdx.z;
  int m = s_multi[tid] - multi, c = s_chunks[tid] - chunks;  // before this thread's run
  if (want >= m && want < m + multi) {
    for (int s = lo; s < hi; ++s) {
      const int n = cu[s + 1] - cu[s];
      const int nc = (n + q - 1) / q;
      if (n > 1) {
        if (m == want) {
          s_seq = s;
          s_first = c;
          s_nc = nc;
        }
        ++m;
      }
      c += nc;
    }
  }
  __syncthreads();
  const int e = (blockIdx.x * blockDim.x + tid) * 4;
  if (s_seq < 0 || e >= PN) return;
  ssd_pass_sequence(chunk_state, chunk_decay, start_state, state, slots[s_seq], H, PN, blockIdx.y, e, s_first, s_nc);
}

// ----------------------------------------------------------------------------- phase 3
template <int P, int N>
__global__ void __launch_bounds__(128)
    ssd_chunk_output_kernel(const bf16* __restrict__ xbc, int ld_xbc, const bf16* __restrict__ dt_raw,
                            long long ld_dt, float dt_scale, const float* __restrict__ dt_shift,
                            const float* __restrict__ a_log, const float* __restrict__ d_skip,
                            const int* __restrict__ cu, int n_seq, const bf16* __restrict__ start_state,
                            const float* __restrict__ chunk_cb, bf16* __restrict__ y, int H, int G, const bf16* __restrict__ z_raw, long long ld_z,
                            float z_scale, const float* __restrict__ z_bias) {
  constexpr int SX = P + 8, SN = N + 8;
  constexpr int PB = P < 64 ? P : 64;  // output columns per pass
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sC = reinterpret_cast<bf16*>(smem_raw);
  bf16* sS = sC + kQ * SN;   // [P][SN] start state, bfloat16
  bf16* sX = sS + P * SN;    // [kQ][SX]
  __shared__ float s_delta[kQ], s_cs[kQ];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y;
  int seq, t0, len, first;
  if (!ssd_locate(cu, n_seq, c, seq, t0, len, first)) return;
  const int I = H * P, g = h / (H / G);

  for (int i = tid; i < kQ * (N / 8); i += 128) {
    const int r = i / (N / 8), col = i % (N / 8);
    const bool ok = r < len;
    const size_t row = ok ? static_cast<size_t>(t0 + r) * ld_xbc : 0;
    ssd_cp_async16(sC + r * SN + col * 8, xbc + row + (ok ? I + G * N + g * N + col * 8 : 0), ok);
  }
  for (int i = tid; i < kQ * (P / 8); i += 128) {
    const int r = i / (P / 8), col = i % (P / 8);
    const bool ok = r < len;
    ssd_cp_async16(sX + r * SX + col * 8, xbc + (ok ? static_cast<size_t>(t0 + r) * ld_xbc + h * P + col * 8 : 0), ok);
  }
  {
    const bf16* src = start_state + (static_cast<size_t>(c) * H + h) * P * N;
    for (int i = tid; i < P * (N / 8); i += 128) {
      const int p = i / (N / 8), col = i % (N / 8);
      ssd_cp_async16(sS + p * SN + col * 8, src + static_cast<size_t>(p) * N + col * 8, true);
    }
  }
  ssd_delta_cumsum(dt_raw, ld_dt, dt_scale, dt_shift[h], -expf(a_log[h]), t0, len, h, s_delta, s_cs);
  ssd_cp_async_wait_all();
  __syncthreads();

  const int i_lo = warp * 16 + (lane >> 2), i_hi = i_lo + 8;
  const float cs_lo = s_cs[i_lo], cs_hi = s_cs[i_hi];

  // The gate's inputs for this thread's outputs are requested now and used in the epilogue.
  constexpr int NT_Y = PB / 8;
  __nv_bfloat162 zreg[2][NT_Y];
  auto load_z = [&](int pb) {
    if (!z_raw) return;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int i = half ? i_hi : i_lo;
#pragma unroll
      for (int nt = 0; nt < NT_Y; ++nt) {
        const int p = pb * PB + nt * 8 + (lane & 3) * 2;
        zreg[half][nt] = i < len ? *reinterpret_cast<const __nv_bfloat162*>(
                                       z_raw + static_cast<long long>(t0 + i) * ld_z + h * P + p)
                                 : __floats2bfloat162_rn(0.f, 0.f);
      }
    }
  };
  load_z(0);

  // Fragment loads and mma instructions issue in program order: the fragments of step k+1 are
  // requested before the products of step k, so their latency hides behind them.
  const bf16* c_lane = sC + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SN + (lane >> 4) * 8;

  // C_i . B_j for this warp's 16 rows and the tokens up to its diagonal block, formed once per
  // (chunk, group) by phase 1 and read here in accumulator layout; then the decayed, masked,
  // delta-weighted matrix M as bfloat16 A-fragments
  unsigned mfrag[kQ / 16][4];
  {
    float gacc[kQ / 8][4];
    const float* gsrc = chunk_cb + (static_cast<size_t>(c) * G + g) * kQ * kQ;
#pragma unroll
    for (int nt = 0; nt < kQ / 8; ++nt) {
      float2 lo = make_float2(0.f, 0.f), hi = lo;
      if (nt / 2 <= warp) {
        const int j = nt * 8 + (lane & 3) * 2;
        lo = __ldg(reinterpret_cast<const float2*>(gsrc + i_lo * kQ + j));
        hi = __ldg(reinterpret_cast<const float2*>(gsrc + i_hi * kQ + j));
      }
      gacc[nt][0] = lo.x; gacc[nt][1] = lo.y; gacc[nt][2] = hi.x; gacc[nt][3] = hi.y;
    }
#pragma unroll
    for (int kk = 0; kk < kQ / 16; ++kk) {
      float m[2][4];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int nt = 2 * kk + half;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = nt * 8 + (lane & 3) * 2 + (e & 1);
          const int i = (e < 2) ? i_lo : i_hi;
          const float csi = (e < 2) ? cs_lo : cs_hi;
          // the result is rounded to bfloat16 next, so the fast exponential loses nothing
          m[half][e] = (j <= i) ? gacc[nt][e] * __expf(csi - s_cs[j]) * s_delta[j] : 0.f;
        }
      }
      mfrag[kk][0] = ssd_pack(m[0][0], m[0][1]);
      mfrag[kk][1] = ssd_pack(m[0][2], m[0][3]);
      mfrag[kk][2] = ssd_pack(m[1][0], m[1][1]);
      mfrag[kk][3] = ssd_pack(m[1][2], m[1][3]);
    }
  }

  const float e_lo = expf(cs_lo), e_hi = expf(cs_hi);
  const float Dh = d_skip[h];
#pragma unroll 1
  for (int pb = 0; pb < P / PB; ++pb) {
    float y1[PB / 8][4], y2[PB / 8][4];
#pragma unroll
    for (int i = 0; i < PB / 8; ++i) {
      y1[i][0] = y1[i][1] = y1[i][2] = y1[i][3] = 0.f;
      y2[i][0] = y2[i][1] = y2[i][2] = y2[i][3] = 0.f;
    }
    // within the chunk: M (delta x)
    {
      const bf16* x_lane = sX + ((lane & 7) + ((lane >> 3) & 1) * 8) * SX + pb * PB + (lane >> 4) * 8;
      unsigned fx[2][PB / 16][4];
      auto load_x = [&](int kk) {
#pragma unroll
        for (int np = 0; np < PB / 16; ++np)
          ssd_ldm_t(fx[kk & 1][np][0], fx[kk & 1][np][1], fx[kk & 1][np][2], fx[kk & 1][np][3],
                    x_lane + kk * 16 * SX + np * 16);
      };
      load_x(0);
#pragma unroll
      for (int kk = 0; kk < kQ / 16; ++kk) {
        if (kk <= warp) {
          if (kk + 1 < kQ / 16 && kk + 1 <= warp) load_x(kk + 1);
#pragma unroll
          for (int np = 0; np < PB / 16; ++np) {
            ssd_mma(y1[2 * np], mfrag[kk], fx[kk & 1][np][0], fx[kk & 1][np][1]);
            ssd_mma(y1[2 * np + 1], mfrag[kk], fx[kk & 1][np][2], fx[kk & 1][np][3]);
          }
        }
      }
    }
    // from before the chunk: C S^T
    {
      const bf16* s_lane = sS + (pb * PB + (lane & 7) + (lane >> 4) * 8) * SN + ((lane >> 3) & 1) * 8;
      unsigned fa[2][4], fs[2][PB / 16][4];
      auto load_s = [&](int ks) {
        ssd_ldm(fa[ks & 1][0], fa[ks & 1][1], fa[ks & 1][2], fa[ks & 1][3], c_lane + ks * 16);
#pragma unroll
        for (int np = 0; np < PB / 16; ++np)
          ssd_ldm(fs[ks & 1][np][0], fs[ks & 1][np][1], fs[ks & 1][np][2], fs[ks & 1][np][3],
                  s_lane + np * 16 * SN + ks * 16);
      };
      load_s(0);
#pragma unroll
      for (int ks = 0; ks < N / 16; ++ks) {
        if (ks + 1 < N / 16) load_s(ks + 1);
#pragma unroll
        for (int np = 0; np < PB / 16; ++np) {
          ssd_mma(y2[2 * np], fa[ks & 1], fs[ks & 1][np][0], fs[ks & 1][np][1]);
          ssd_mma(y2[2 * np + 1], fa[ks & 1], fs[ks & 1][np][2], fs[ks & 1][np][3]);
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < PB / 8; ++nt) {
      const int p = pb * PB + nt * 8 + (lane & 3) * 2;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int i = half ? i_hi : i_lo;
        if (i >= len) continue;
        const float e = half ? e_hi : e_lo;
        const float2 xv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sX + i * SX + p));
        float v0 = y1[nt][2 * half] + e * y2[nt][2 * half] + Dh * xv.x;
        float v1 = y1[nt][2 * half + 1] + e * y2[nt][2 * half + 1] + Dh * xv.y;
        if (z_raw) {  // gate fused: y * silu(z), z = z_raw * z_scale + z_bias
          const int c = h * P + p;
          const float2 zv = __bfloat1622float2(zreg[half][nt]);
          v0 *= silu_fast(zv.x * z_scale + (z_bias ? z_bias[c] : 0.f));
          v1 *= silu_fast(zv.y * z_scale + (z_bias ? z_bias[c + 1] : 0.f));
        }
        *reinterpret_cast<__nv_bfloat162*>(y + static_cast<size_t>(t0 + i) * I + h * P + p) = __floats2bfloat162_rn(v0, v1);
      }
    }
    if (pb + 1 < P / PB) load_z(pb + 1);
  }
}

// The state pass alone, for chunks of `q` tokens (the tcgen05 scan of ssd_tc.cu uses it with 128).
// n_multi: with skip_single, the number of sequences that bring more than one token (0: not known).
int launch_ssd_state_pass(const float* chunk_state, const float* chunk_decay, bf16* start_state, float* state,
                          const int* cu, const int* slots, int n_seq, int H, int PN, int q, int skip_single, int n_multi,
                          cudaStream_t stream) {
  if (PN % 4 || n_seq > 65535 || H > 65535 || q <= 0 || n_multi < 0 || n_multi > n_seq) return PMM_ERR_BAD_ARGUMENT;
  if (skip_single && n_multi > 0) {
    launch_pdl(ssd_state_pass_multi_kernel, dim3((PN / 4 + 255) / 256, H, n_multi), dim3(256), 0, stream, chunk_state, chunk_decay,
               start_state, state, cu, slots, H, PN, q, n_seq);
    return launch_status();
  }
  // about a thousand blocks: with many sequences a block takes several of them in turn
  const int per_seq = ((PN / 4 + 255) / 256) * H;
  int spb = static_cast<int>((static_cast<long long>(n_seq) * per_seq + 1023) / 1024);
  if (spb < 1) spb = 1;
  dim3 grid((PN / 4 + 255) / 256, H, (n_seq + spb - 1) / spb);
  launch_pdl(ssd_state_pass_kernel, grid, dim3(256), 0, stream, chunk_state, chunk_decay, start_state, state, cu, slots, H,
             PN, q, n_seq, spb, skip_single);
  return launch_status();
}

template <int P, int N>
int launch_ssd(const void* xbc, int ld_xbc, const void* dt_raw, long long ld_dt, float dt_scale,
               const float* dt_shift, const float* a_log, const float* d_skip, float* state,
               const int* cu, const int* slots, void* y, float* chunk_state, float* chunk_decay, bf16* start_state,
               float* chunk_cb, int n_seq, int n_chunks, int H, int G, const void* z_raw, long long ld_z, float z_scale,
               const float* z_bias, cudaStream_t stream) {
  // phase 1: x and B of a (chunk, head), or C and B of a (chunk, group)
  const size_t smem1 = static_cast<size_t>(kQ) * ((P > N ? P : N) + 8 + (N + 8)) * sizeof(bf16);
  const size_t smem3 = (static_cast<size_t>(kQ) * ((N + 8) + (P + 8)) + static_cast<size_t>(P) * (N + 8)) * sizeof(bf16);
  auto k1 = ssd_chunk_state_kernel<P, N>;
  auto k3 = ssd_chunk_output_kernel<P, N>;
  if (smem1 > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem1));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  if (smem3 > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem3));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  dim3 grid(n_chunks, H), grid1(n_chunks, H + G);
  launch_pdl(k1, grid1, dim3(128), smem1, stream, static_cast<const bf16*>(xbc), ld_xbc, static_cast<const bf16*>(dt_raw), ld_dt,
                                    dt_scale, dt_shift, a_log, cu, n_seq, chunk_state, chunk_decay, chunk_cb, H, G);
  const int PN = P * N;
  dim3 grid2((PN / 4 + 255) / 256, H, n_seq);
  launch_pdl(ssd_state_pass_kernel, grid2, dim3(256), 0, stream, chunk_state, chunk_decay, start_state, state, cu, slots, H, PN, kQ,
             n_seq, 1, 0);
  launch_pdl(k3, grid, dim3(128), smem3, stream, static_cast<const bf16*>(xbc), ld_xbc, static_cast<const bf16*>(dt_raw), ld_dt,
                                   dt_scale, dt_shift, a_log, d_skip, cu, n_seq, start_state, chunk_cb,
                                   static_cast<bf16*>(y), H, G, static_cast<const bf16*>(z_raw), ld_z, z_scale, z_bias);
  return launch_status();
}

}  // namespace pmm

// Head size / state size pairs the tensor-core scan is compiled for.
PMM_EXPORT int pmm_ssd_supported(int P, int N) {
  return ((P == 16 && N == 16) || (P == 32 && N == 32) || (P == 64 && N == 64) || (P == 64 && N == 128) ||
          (P == 64 && N == 256) || (P == 128 && N == 128) || (P == 128 && N == 256)) ? 1 : 0;
}

// Scratch: chunk_state n_chunks*H*P*N floats, chunk_decay n_chunks*H floats, start_state
// n_chunks*H*P*N bfloat16 (16-byte aligned), chunk_cb n_chunks*G*64*64 floats (8-byte aligned);
// n_chunks = sum over sequences of ceil(new tokens / 64).  bfloat16 activations only.
PMM_EXPORT int pmm_ssd_chunked(const void* xbc, int ld_xbc, const void* dt_raw, long long ld_dt,
                               float dt_scale, const float* dt_shift, const float* a_log,
                               const float* d_skip, float* state, const int* cu, const int* slots,
                               void* y, float* chunk_state, float* chunk_decay, void* start_state,
                               float* chunk_cb, int n_seq, int n_chunks, int H, int P, int N, int G, const void* z_raw, long long ld_z, float z_scale,
                               const float* z_bias, cudaStream_t stream) {
  if (n_seq <= 0 || n_chunks <= 0) return 0;
  if (!pmm_ssd_supported(P, N) || H <= 0 || G <= 0 || H % G || H > 65535 || n_seq > 65535 ||
      !chunk_state || !chunk_decay || !start_state || reinterpret_cast<uintptr_t>(start_state) % 16 ||
      !chunk_cb || reinterpret_cast<uintptr_t>(chunk_cb) % 8 || H + G > 65535)
    return PMM_ERR_BAD_ARGUMENT;
#define PMM_SSD_CASE(PP, NN)                                                                             \
  if (P == PP && N == NN)                                                                                \
    return pmm::launch_ssd<PP, NN>(xbc, ld_xbc, dt_raw, ld_dt, dt_scale, dt_shift, a_log, d_skip, state, \
                                   cu, slots, y, chunk_state, chunk_decay,                    \
                                   static_cast<pmm::bf16*>(start_state), chunk_cb, n_seq, n_chunks, H, G,  \
                                   z_raw,                                                                  \
                                   ld_z, z_scale, z_bias, stream)
  PMM_SSD_CASE(16, 16);
  PMM_SSD_CASE(32, 32);
  PMM_SSD_CASE(64, 64);
  PMM_SSD_CASE(64, 128);
  PMM_SSD_CASE(64, 256);
  PMM_SSD_CASE(128, 128);
  PMM_SSD_CASE(128, 256);
#undef PMM_SSD_CASE
  return PMM_ERR_BAD_ARGUMENT;
}

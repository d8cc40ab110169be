// Mamba2 selective-state recurrence (token-serial form) and the gate / gated RMSNorm.
//
// ssm_scan_seq walks the tokens of each sequence portion in order, starting from the
// request's saved state [slot][H][P][N] (float) and leaving the final state there.  It
// serves decode (one token per sequence), the 32-bit path and short portions; the
// chunked tensor-core scan replaces it for long bfloat16 prompts.
//
//   delta = softplus(dt_raw*dt_scale + dt_shift[h]);  dA = exp(delta * -exp(A_log[h]))
//   s[p,n] = s[p,n]*dA + (delta*B[n])*x[p];  y[p] = sum_n s[p,n]*C[n] + D[h]*x[p]
// (reference src/ops/gpu/mamba2_scan.cu:11-50; y uses the updated state; head h reads
// group h / (H/G)).
//
// Work split: one block per (p-tile of 32 rows, head, sequence); 8 threads share one
// state row, each holding NPT = ceil(N/8) state values in registers for the whole walk.
#include "common.cuh"

namespace pmm {

constexpr int kScanRows = 32;   // state rows (values of p) per block
constexpr int kScanTpr = 8;     // threads per state row

template <typename S, int NPT>
__global__ void __launch_bounds__(kScanRows* kScanTpr)
    ssm_scan_seq_kernel(const S* __restrict__ xbc, int ld_xbc, const S* __restrict__ dt_raw,
                        long long ld_dt, float dt_scale, const float* __restrict__ dt_shift,
                        const float* __restrict__ a_log, const float* __restrict__ d_skip,
                        float* __restrict__ state, const int* __restrict__ cu,
                        const int* __restrict__ slots, S* __restrict__ y, int H, int P, int N,
                        int G, const S* __restrict__ z_raw, long long ld_z, float z_scale,
                        const float* __restrict__ z_bias, int one_token) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane_n = threadIdx.x % kScanTpr;
  const int p = blockIdx.x * kScanRows + threadIdx.x / kScanTpr;
  const int h = blockIdx.y;
  const int s = blockIdx.z;
  const int t0 = cu[s], t1 = cu[s + 1];
  if (t1 <= t0) return;
  if (one_token == 2 && t1 - t0 != 1) return;  // only the lone tokens of a mixed step
  const bool row_ok = p < P;
  const int I = H * P;
  const int g = h / (H / G);
  const int off_b = I + g * N;
  const int off_c = I + G * N + g * N;
  const float A = -expf(a_log[h]);
  const float Dh = d_skip[h];
  const float shift = dt_shift[h];

  float st[NPT];
  float* srow = state + ((static_cast<size_t>(slots[s]) * H + h) * P + (row_ok ? p : 0)) * N;
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = lane_n + i * kScanTpr;
    st[i] = (row_ok && n < N) ? srow[n] : 0.f;
  }

  for (int t = t0; t < t1; ++t) {
    const S* row = xbc + static_cast<size_t>(t) * ld_xbc;
    const float delta = softplus_f(ldf(dt_raw + static_cast<long long>(t) * ld_dt + h) * dt_scale + shift);
    const float dA = expf(delta * A);
    const float xv = row_ok ? ldf(row + h * P + p) : 0.f;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = lane_n + i * kScanTpr;
      if (n < N) {
        const float bn = ldf(row + off_b + n);
        const float cn = ldf(row + off_c + n);
        st[i] = st[i] * dA + (delta * bn) * xv;
        acc += st[i] * cn;
      }
    }
#pragma unroll
    for (int o = kScanTpr / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (row_ok && lane_n == 0) {
      float yv = acc + Dh * xv;
      if (z_raw) {  // gate fused: y * silu(z), z = z_raw * z_scale + z_bias
        const int c = h * P + p;
        const float zv = ldf(z_raw + static_cast<long long>(t) * ld_z + c) * z_scale + (z_bias ? z_bias[c] : 0.f);
        yv *= silu_f(zv);
      }
      stf(y + static_cast<size_t>(t) * I + h * P + p, yv);
    }
  }

  if (row_ok) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = lane_n + i * kScanTpr;
      if (n < N) srow[n] = st[i];
    }
  }
}

// The same walk with four neighbouring state columns per thread and access: state rows move as
// 16-byte pieces (a warp touches four whole 128-byte lines per instruction), B and C as four
// values at a time.  Needs N % 4 == 0 and rows of xbc whose B and C parts start on 8-byte
// (bfloat16) / 16-byte (float) boundaries.  one_token 1: sequence s brings exactly token s (decode),
// so nothing waits for the sequence bounds.  one_token 2: only the sequences that bring exactly one
// token are walked (the lone tokens of a mixed step; the chunked scan takes the others).
__device__ __forceinline__ float4 scan_ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 scan_ld4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename S, int NV>
__global__ void __launch_bounds__(kScanRows* kScanTpr)
    ssm_scan_seq_vec_kernel(const S* __restrict__ xbc, int ld_xbc, const S* __restrict__ dt_raw,
                            long long ld_dt, float dt_scale, const float* __restrict__ dt_shift,
                            const float* __restrict__ a_log, const float* __restrict__ d_skip,
                            float* __restrict__ state, const int* __restrict__ cu,
                            const int* __restrict__ slots, S* __restrict__ y, int H, int P, int N,
                            int G, const S* __restrict__ z_raw, long long ld_z, float z_scale,
                            const float* __restrict__ z_bias, int one_token) {
  pdl_launch_dependents();
  const int lane_n = threadIdx.x % kScanTpr;
  const int p = blockIdx.x * kScanRows + threadIdx.x / kScanTpr;
  const int h = blockIdx.y;
  const int s = blockIdx.z;
  const bool row_ok = p < P;
  const int I = H * P;
  const int g = h / (H / G);
  const int off_b = I + g * N;
  const int off_c = I + G * N + g * N;
  const int n4 = N / 4;
  // constants of the head and the request's slot: inputs of the step, read before the wait
  const float A = -expf(a_log[h]);
  const float Dh = d_skip[h];
  const float shift = dt_shift[h];
  const int slot = slots[s];
  int t0 = s, t1 = s + 1;
  if (one_token != 1) {
    t0 = cu[s];
    t1 = cu[s + 1];
  }
  pdl_wait();
  if (t1 <= t0) return;
  if (one_token == 2 && t1 - t0 != 1) return;  // only the lone tokens of a mixed step

  float4 st[NV];
  float* srow = state + ((static_cast<size_t>(slot) * H + h) * P + (row_ok ? p : 0)) * N;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int q = lane_n + i * kScanTpr;
    st[i] = (row_ok && q < n4) ? scan_ld4(srow + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
  }

  for (int t = t0; t < t1; ++t) {
    const S* row = xbc + static_cast<size_t>(t) * ld_xbc;
    const float delta = softplus_f(ldf(dt_raw + static_cast<long long>(t) * ld_dt + h) * dt_scale + shift);
    const float dA = expf(delta * A);
    const float xv = row_ok ? ldf(row + h * P + p) : 0.f;
    const float dx = delta * xv;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int q = lane_n + i * kScanTpr;
      if (q < n4) {
        const float4 b = scan_ld4(row + off_b + 4 * q);
        const float4 c = scan_ld4(row + off_c + 4 * q);
        st[i].x = st[i].x * dA + (delta * b.x) * xv;
        st[i].y = st[i].y * dA + (delta * b.y) * xv;
        st[i].z = st[i].z * dA + (delta * b.z) * xv;
        st[i].w = st[i].w * dA + (delta * b.w) * xv;
        acc += st[i].x * c.x;
        acc += st[i].y * c.y;
        acc += st[i].z * c.z;
        acc += st[i].w * c.w;
      }
    }
    (void)dx;
#pragma unroll
    for (int o = kScanTpr / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (row_ok && lane_n == 0) {
      float yv = acc + Dh * xv;
      if (z_raw) {  // gate fused: y * silu(z), z = z_raw * z_scale + z_bias
        const int c = h * P + p;
        const float zv = ldf(z_raw + static_cast<long long>(t) * ld_z + c) * z_scale + (z_bias ? z_bias[c] : 0.f);
        yv *= silu_f(zv);
      }
      stf(y + static_cast<size_t>(t) * I + h * P + p, yv);
    }
  }

  if (row_ok) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int q = lane_n + i * kScanTpr;
      if (q < n4) *reinterpret_cast<float4*>(srow + 4 * q) = st[i];
    }
  }
}

// One block per (token, group).  z = z_raw*z_scale + z_bias[c].
//   no weight:            out = y * silu(z)
//   weight, gate first:   out = rmsnorm_group(y * silu(z)) * w
//   weight, norm first:   out = rmsnorm_group(y) * w * silu(z)
template <typename S>
__global__ void gated_norm_kernel(const S* __restrict__ y, const S* __restrict__ z_raw,
                                  long long ld_z, float z_scale, const float* __restrict__ z_bias,
                                  const float* __restrict__ w, float eps, int norm_before_gate,
                                  S* __restrict__ out, int I, int group_width) {
  extern __shared__ float buf[];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c0 = blockIdx.y * group_width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < group_width; i += blockDim.x) {
    const int c = c0 + i;
    const float yv = ldf(y + static_cast<size_t>(t) * I + c);
    const float zv = ldf(z_raw + static_cast<long long>(t) * ld_z + c) * z_scale + (z_bias ? z_bias[c] : 0.f);
    const float gate = silu_f(zv);
    float v;
    if (!w) {
      stf(out + static_cast<size_t>(t) * I + c, yv * gate);
      continue;
    }
    if (norm_before_gate) {
      v = yv;
      buf[group_width + i] = gate;
    } else {
      v = yv * gate;
    }
    buf[i] = v;
    ss += v * v;
  }
  if (!w) return;
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(group_width) + eps);
  for (int i = threadIdx.x; i < group_width; i += blockDim.x) {
    const int c = c0 + i;
    float v = buf[i] * inv * w[c];
    if (norm_before_gate) v *= buf[group_width + i];
    stf(out + static_cast<size_t>(t) * I + c, v);
  }
}

template <typename S>
int launch_scan(const void* xbc, int ld_xbc, const void* dt_raw, long long ld_dt, float dt_scale,
                const float* dt_shift, const float* a_log, const float* d_skip, float* state,
                const int* cu, const int* slots, void* y, int n_seq, int H, int P, int N, int G,
                const void* z_raw, long long ld_z, float z_scale, const float* z_bias, int one_token,
                cudaStream_t stream) {
  dim3 grid((P + kScanRows - 1) / kScanRows, H, n_seq);
  dim3 block(kScanRows * kScanTpr);
  const int npt = (N + kScanTpr - 1) / kScanTpr;
  // four state columns per thread where the rows allow 16-byte (state) and 4-element (B, C) accesses
  const size_t e4 = 4 * sizeof(S);
  const bool vec = N % 4 == 0 && N <= 256 && reinterpret_cast<uintptr_t>(state) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(xbc) % e4 == 0 && (static_cast<size_t>(ld_xbc) * sizeof(S)) % e4 == 0 &&
                   (static_cast<size_t>(H) * P * sizeof(S)) % e4 == 0;
  if (vec) {
    const int nv = (N / 4 + kScanTpr - 1) / kScanTpr;
#define PMM_SCANV_CASE(NV)                                                                                 \
  launch_pdl(ssm_scan_seq_vec_kernel<S, NV>, grid, block, 0, stream, static_cast<const S*>(xbc), ld_xbc,      \
             static_cast<const S*>(dt_raw), ld_dt, dt_scale, dt_shift, a_log, d_skip, state, cu, slots,     \
             static_cast<S*>(y), H, P, N, G, static_cast<const S*>(z_raw), ld_z, z_scale, z_bias, one_token)
    if (nv <= 1) PMM_SCANV_CASE(1);
    else if (nv <= 2) PMM_SCANV_CASE(2);
    else if (nv <= 4) PMM_SCANV_CASE(4);
    else PMM_SCANV_CASE(8);
#undef PMM_SCANV_CASE
    return launch_status();
  }
#define PMM_SCAN_CASE(NPT)                                                                         \
  launch_pdl(ssm_scan_seq_kernel<S, NPT>, grid, block, 0, stream, static_cast<const S*>(xbc), ld_xbc,  \
             static_cast<const S*>(dt_raw), ld_dt, dt_scale, dt_shift, a_log, d_skip, state, cu, slots, \
             static_cast<S*>(y), H, P, N, G, static_cast<const S*>(z_raw), ld_z, z_scale, z_bias, one_token)
  if (npt <= 1) PMM_SCAN_CASE(1);
  else if (npt <= 2) PMM_SCAN_CASE(2);
  else if (npt <= 4) PMM_SCAN_CASE(4);
  else if (npt <= 8) PMM_SCAN_CASE(8);
  else if (npt <= 16) PMM_SCAN_CASE(16);
  else if (npt <= 32) PMM_SCAN_CASE(32);
  else return PMM_ERR_BAD_ARGUMENT;  // d_state above 256
#undef PMM_SCAN_CASE
  return launch_status();
}

}  // namespace pmm

PMM_EXPORT int pmm_ssm_scan_seq(const void* xbc, int ld_xbc, const void* dt_raw, long long ld_dt,
                                float dt_scale, const float* dt_shift, const float* a_log,
                                const float* d_skip, float* state, const int* cu, const int* slots,
                                void* y, int n_seq, int H, int P, int N, int G, const void* z_raw,
                                long long ld_z, float z_scale, const float* z_bias, int one_token, int dtype,
                                cudaStream_t stream) {
  if (n_seq <= 0) return 0;
  if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G || H > 65535 || n_seq > 65535)
    return PMM_ERR_BAD_ARGUMENT;
  PMM_DISPATCH_DTYPE(dtype, S, return pmm::launch_scan<S>(xbc, ld_xbc, dt_raw, ld_dt, dt_scale,
                                                          dt_shift, a_log, d_skip, state, cu, slots,
                                                          y, n_seq, H, P, N, G, z_raw, ld_z, z_scale,
                                                          z_bias, one_token, stream));
  return 0;
}

PMM_EXPORT int pmm_gated_norm(const void* y, const void* z_raw, long long ld_z, float z_scale,
                              const float* z_bias, const float* w, float eps, int norm_before_gate,
                              void* out, int T, int I, int n_groups, int dtype,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_groups <= 0 || I % n_groups || n_groups > 65535) return PMM_ERR_BAD_ARGUMENT;
  const int gw = I / n_groups;
  const size_t smem = w ? static_cast<size_t>(gw) * sizeof(float) * (norm_before_gate ? 2 : 1) : 0;
  if (smem > 200 * 1024) return PMM_ERR_BAD_ARGUMENT;
  dim3 grid(T, n_groups);
  PMM_DISPATCH_DTYPE(dtype, S, {
    auto kern = pmm::gated_norm_kernel<S>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    pmm::launch_pdl(kern, grid, dim3(256), smem, stream, static_cast<const S*>(y), static_cast<const S*>(z_raw), ld_z,
                    z_scale, z_bias, w, eps, norm_before_gate, static_cast<S*>(out), I, gw);
  });
  return pmm::launch_status();
}

// Causal depthwise conv1d + SiLU over a flattened batch of sequence portions.
//
// Each token t of sequence s (local index j = t - cu[s]) convolves its own input with
// the K-1 inputs before it; inputs before the portion come from the per-request window
// [slot][K-1][C] (time-major, oldest first, float, zero for a new request).  The conv
// input is the affine image v = raw*pre_scale[c] + pre_bias[c] of a column slice of the
// input projection, so no separate "split and scale" pass exists.
//
//   a = bias[c] + sum_{k<K-1} w[c,k]*v[j-(K-1)+k] + w[c,K-1]*v[j];  y = silu(a)
// (reference src/ops/gpu/conv.cu:3-26, which walks tokens serially per channel).
//
// conv1d_fwd reads the window, conv1d_window_update writes it afterwards (separate
// launches: the first tokens of a portion must see the old window).  conv1d_decode does
// both for portions of exactly one token.
#include "common.cuh"

namespace pmm {

template <typename S>
__global__ void conv1d_fwd_kernel(const S* __restrict__ x, long long ldx,
                                  const float* __restrict__ pre_scale,
                                  const float* __restrict__ pre_bias, const float* __restrict__ w,
                                  const float* __restrict__ bias, const float* __restrict__ window,
                                  const int* __restrict__ seq_of, const int* __restrict__ cu,
                                  const int* __restrict__ slots, S* __restrict__ y, int T, int C,
                                  int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int t = blockIdx.x;
  if (c >= C || t >= T) return;
  const int s = seq_of[t];
  const int j = t - cu[s];
  const int left = K - 1;
  const float ps = pre_scale[c];
  const float pb = pre_bias ? pre_bias[c] : 0.f;
  const float* wrow = w + static_cast<size_t>(c) * K;
  const float* win = window + static_cast<size_t>(slots[s]) * left * C;
  float acc = bias ? bias[c] : 0.f;
  for (int k = 0; k < K; ++k) {
    const int jj = j - left + k;  // local index of the tap's input
    float v;
    if (jj >= 0) {
      v = ldf(x + static_cast<long long>(t - left + k) * ldx + c) * ps + pb;
    } else {
      v = win[static_cast<size_t>(left + jj) * C + c];
    }
    acc += wrow[k] * v;
  }
  stf(y + static_cast<size_t>(t) * C + c, silu_f(acc));
}

template <typename S>
__global__ void conv1d_window_update_kernel(const S* __restrict__ x, long long ldx,
                                            const float* __restrict__ pre_scale,
                                            const float* __restrict__ pre_bias,
                                            float* __restrict__ window,
                                            const int* __restrict__ cu,
                                            const int* __restrict__ slots, int n_seq, int C, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  if (c >= C || s >= n_seq) return;
  const int left = K - 1;
  const int t0 = cu[s], n_new = cu[s + 1] - t0;
  if (n_new <= 0) return;
  const float ps = pre_scale[c];
  const float pb = pre_bias ? pre_bias[c] : 0.f;
  float* win = window + static_cast<size_t>(slots[s]) * left * C;
  // New entry i holds the input with local index n_new - left + i.  Entries that stay
  // inside the old window move down; ascending i reads index n_new+i > i, never one that
  // this thread has already overwritten.
  for (int i = 0; i < left; ++i) {
    const int jj = n_new - left + i;
    float v;
    if (jj >= 0) {
      v = ldf(x + static_cast<long long>(t0 + jj) * ldx + c) * ps + pb;
    } else {
      v = win[static_cast<size_t>(left + jj) * C + c];
    }
    win[static_cast<size_t>(i) * C + c] = v;
  }
}

// Vector form for bfloat16 with 16-byte aligned rows: a thread owns 8 neighbouring channels
// and a strip of tokens.  All rows of the strip (and the K-1 before it) and the tokens' places
// in their sequences are requested before anything is computed, so the strip costs two memory
// round trips (short strips: the kernel needs many threads to hide its arithmetic); the K-1 previous inputs then slide through registers.  At the first token of a
// sequence the history comes from the request's window.
constexpr int kConvStrip = 4;

template <int K>
__global__ void __launch_bounds__(128)
    conv1d_fwd_vec_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const float* __restrict__ pre_scale,
                          const float* __restrict__ pre_bias, const float* __restrict__ w_t,
                          const float* __restrict__ bias, const float* __restrict__ window,
                          const int* __restrict__ seq_of, const int* __restrict__ cu,
                          const int* __restrict__ slots, __nv_bfloat16* __restrict__ y, int T, int C) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int L = K - 1;
  constexpr int R = kConvStrip + L;
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  const int t_begin = blockIdx.x * kConvStrip;
  if (c0 >= C || t_begin >= T) return;
  const int n_tok = min(T - t_begin, kConvStrip);

  uint4 raw[R];  // rows t_begin - L .. t_begin + strip - 1
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int t = t_begin - L + i;
    raw[i] = (t >= 0 && t < T) ? *reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * ldx + c0)
                               : make_uint4(0u, 0u, 0u, 0u);
  }
  int seq[kConvStrip], j[kConvStrip];
#pragma unroll
  for (int i = 0; i < kConvStrip; ++i) seq[i] = i < n_tok ? seq_of[t_begin + i] : 0;
#pragma unroll
  for (int i = 0; i < kConvStrip; ++i) j[i] = t_begin + i - cu[seq[i]];
  // per-channel constants as 16-byte loads (w_t is the tap-major copy [K][C] of the weights)
  float ps[8], pb[8], cb[8], wk[8][K];
  auto load8 = [&](const float* src, float* dst) {
    const float4 a = *reinterpret_cast<const float4*>(src + c0), b = *reinterpret_cast<const float4*>(src + c0 + 4);
    dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w;
    dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
  };
  load8(pre_scale, ps);
#pragma unroll
  for (int i = 0; i < 8; ++i) pb[i] = cb[i] = 0.f;
  if (pre_bias) load8(pre_bias, pb);
  if (bias) load8(bias, cb);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    float col[8];
    load8(w_t + static_cast<size_t>(k) * C, col);
#pragma unroll
    for (int i = 0; i < 8; ++i) wk[i][k] = col[i];
  }
  auto unpack = [&](const uint4& r, float* v) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h2[i]);
      v[2 * i] = f.x * ps[2 * i] + pb[2 * i];
      v[2 * i + 1] = f.y * ps[2 * i + 1] + pb[2 * i + 1];
    }
  };

  float hist[L][8];  // hist[k] = input of local index j - L + k
#pragma unroll
  for (int k = 0; k < L; ++k) unpack(raw[k], hist[k]);
#pragma unroll
  for (int i = 0; i < kConvStrip; ++i) {
    if (i < n_tok) {
      // inputs before the sequence's first token come from its window: all of them at a
      // sequence start inside the strip, the first L - j at the strip's start
      if (j[i] < L && (i == 0 || j[i] == 0)) {
        const float* win = window + static_cast<size_t>(slots[seq[i]]) * L * C;
#pragma unroll
        for (int k = 0; k < L; ++k) {
          const int q = j[i] - L + k;
          if (q < 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) hist[k][e] = win[static_cast<size_t>(L + q) * C + c0 + e];
          }
        }
      }
      float v[8];
      unpack(raw[L + i], v);
      uint4 outv;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&outv);
      float a[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float acc = cb[e];
#pragma unroll
        for (int k = 0; k < L; ++k) acc += wk[e][k] * hist[k][e];
        acc += wk[e][L] * v[e];
        a[e] = silu_fast(acc);  // rounded to bfloat16 next
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(a[2 * e], a[2 * e + 1]);
      *reinterpret_cast<uint4*>(y + static_cast<size_t>(t_begin + i) * C + c0) = outv;
#pragma unroll
      for (int k = 0; k + 1 < L; ++k)
#pragma unroll
        for (int e = 0; e < 8; ++e) hist[k][e] = hist[k + 1][e];
#pragma unroll
      for (int e = 0; e < 8; ++e) hist[L - 1][e] = v[e];
    }
  }
}

// One token per sequence: token index == sequence index.
template <typename S>
__global__ void conv1d_decode_kernel(const S* __restrict__ x, long long ldx,
                                     const float* __restrict__ pre_scale,
                                     const float* __restrict__ pre_bias, const float* __restrict__ w,
                                     const float* __restrict__ bias, float* __restrict__ window,
                                     const int* __restrict__ slots, S* __restrict__ y, int n_seq,
                                     int C, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  if (c >= C || s >= n_seq) return;
  const int left = K - 1;
  const float* wrow = w + static_cast<size_t>(c) * K;
  float* win = window + static_cast<size_t>(slots[s]) * left * C;
  const float v_new = ldf(x + static_cast<long long>(s) * ldx + c) * pre_scale[c] +
                      (pre_bias ? pre_bias[c] : 0.f);
  float acc = bias ? bias[c] : 0.f;
  for (int k = 0; k < left; ++k) {
    const float v = win[static_cast<size_t>(k) * C + c];
    acc += wrow[k] * v;
    if (k > 0) win[static_cast<size_t>(k - 1) * C + c] = v;
  }
  acc += wrow[left] * v_new;
  win[static_cast<size_t>(left - 1) * C + c] = v_new;
  stf(y + static_cast<size_t>(s) * C + c, silu_f(acc));
}

}  // namespace pmm

// w: [C][K]; w_t: the same weights tap-major [K][C], or nullptr (then the vector kernel is not used).
PMM_EXPORT int pmm_conv1d_fwd(const void* x, long long ldx, const float* pre_scale,
                              const float* pre_bias, const float* w, const float* w_t, const float* bias,
                              const float* window, const int* seq_of, const int* cu,
                              const int* slots, void* y, int T, int C, int K, int dtype,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  if (K < 2 || C <= 0 || (C + 127) / 128 > 65535) return PMM_ERR_BAD_ARGUMENT;
  auto aligned16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (dtype == PMM_DTYPE_BF16 && w_t && K >= 2 && K <= 4 && C % 8 == 0 && ldx % 8 == 0 && aligned16(x) &&
      aligned16(y) && aligned16(w_t) && aligned16(pre_scale) && aligned16(pre_bias) && aligned16(bias)) {
    dim3 vgrid((T + pmm::kConvStrip - 1) / pmm::kConvStrip, (C / 8 + 127) / 128);
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    __nv_bfloat16* yb = static_cast<__nv_bfloat16*>(y);
    if (K == 2) pmm::launch_pdl(pmm::conv1d_fwd_vec_kernel<2>, vgrid, dim3(128), 0, stream, xb, ldx, pre_scale, pre_bias, w_t, bias, window, seq_of, cu, slots, yb, T, C);
    if (K == 3) pmm::launch_pdl(pmm::conv1d_fwd_vec_kernel<3>, vgrid, dim3(128), 0, stream, xb, ldx, pre_scale, pre_bias, w_t, bias, window, seq_of, cu, slots, yb, T, C);
    if (K == 4) pmm::launch_pdl(pmm::conv1d_fwd_vec_kernel<4>, vgrid, dim3(128), 0, stream, xb, ldx, pre_scale, pre_bias, w_t, bias, window, seq_of, cu, slots, yb, T, C);
    return pmm::launch_status();
  }
  dim3 grid(T, (C + 127) / 128);
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::conv1d_fwd_kernel<S>, grid, dim3(128), 0, stream,
                                   static_cast<const S*>(x), ldx, pre_scale, pre_bias, w, bias,
                                   window, seq_of, cu, slots, static_cast<S*>(y), T, C, K));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_conv1d_window_update(const void* x, long long ldx, const float* pre_scale,
                                        const float* pre_bias, float* window, const int* cu,
                                        const int* slots, int n_seq, int C, int K, int dtype,
                                        cudaStream_t stream) {
  if (n_seq <= 0) return 0;
  if (K < 2 || C <= 0 || n_seq > 65535) return PMM_ERR_BAD_ARGUMENT;
  dim3 grid((C + 127) / 128, n_seq);
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::conv1d_window_update_kernel<S>, grid, dim3(128), 0, stream,
                                   static_cast<const S*>(x), ldx, pre_scale, pre_bias, window, cu,
                                   slots, n_seq, C, K));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_conv1d_decode(const void* x, long long ldx, const float* pre_scale,
                                 const float* pre_bias, const float* w, const float* bias,
                                 float* window, const int* slots, void* y, int n_seq, int C, int K,
                                 int dtype, cudaStream_t stream) {
  if (n_seq <= 0) return 0;
  if (K < 2 || C <= 0 || n_seq > 65535) return PMM_ERR_BAD_ARGUMENT;
  dim3 grid((C + 127) / 128, n_seq);
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::conv1d_decode_kernel<S>, grid, dim3(128), 0, stream,
                                               static_cast<const S*>(x), ldx, pre_scale, pre_bias, w, bias,
                                               window, slots, static_cast<S*>(y), n_seq, C, K));
  return pmm::launch_status();
}

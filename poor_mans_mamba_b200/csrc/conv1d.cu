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
// and walks a strip of tokens with the K-1 previous inputs in registers, so every input is
// read once (plus K-1 rows at the start of a strip).  At the first token of a sequence the
// history comes from the request's window.
constexpr int kConvStrip = 16;

template <int K>
__global__ void __launch_bounds__(128)
    conv1d_fwd_vec_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const float* __restrict__ pre_scale,
                          const float* __restrict__ pre_bias, const float* __restrict__ w,
                          const float* __restrict__ bias, const float* __restrict__ window,
                          const int* __restrict__ seq_of, const int* __restrict__ cu,
                          const int* __restrict__ slots, __nv_bfloat16* __restrict__ y, int T, int C) {
  constexpr int L = K - 1;
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  const int t_begin = blockIdx.x * kConvStrip;
  if (c0 >= C || t_begin >= T) return;
  const int t_end = min(T, t_begin + kConvStrip);
  float ps[8], pb[8], cb[8], wk[8][K];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ps[i] = pre_scale[c0 + i];
    pb[i] = pre_bias ? pre_bias[c0 + i] : 0.f;
    cb[i] = bias ? bias[c0 + i] : 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) wk[i][k] = w[static_cast<size_t>(c0 + i) * K + k];
  }
  auto load_row = [&](int t, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * ldx + c0);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h2[i]);
      v[2 * i] = f.x * ps[2 * i] + pb[2 * i];
      v[2 * i + 1] = f.y * ps[2 * i + 1] + pb[2 * i + 1];
    }
  };
  float hist[L][8];  // hist[i] = input of local index j - L + i
  int cur_seq = -1;
  for (int t = t_begin; t < t_end; ++t) {
    const int s = seq_of[t];
    const int j = t - cu[s];
    if (s != cur_seq || t == t_begin) {  // (re)build the history at a strip or sequence start
      cur_seq = s;
      const float* win = window + static_cast<size_t>(slots[s]) * L * C;
#pragma unroll
      for (int i = 0; i < L; ++i) {
        const int q = j - L + i;
        if (q >= 0) {
          load_row(t - L + i, hist[i]);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) hist[i][e] = win[static_cast<size_t>(L + q) * C + c0 + e];
        }
      }
    }
    float v[8];
    load_row(t, v);
    uint4 outv;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&outv);
    float a[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float acc = cb[e];
#pragma unroll
      for (int k = 0; k < L; ++k) acc += wk[e][k] * hist[k][e];
      acc += wk[e][L] * v[e];
      a[e] = silu_f(acc);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(a[2 * e], a[2 * e + 1]);
    *reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * C + c0) = outv;
#pragma unroll
    for (int i = 0; i + 1 < L; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) hist[i][e] = hist[i + 1][e];
#pragma unroll
    for (int e = 0; e < 8; ++e) hist[L - 1][e] = v[e];
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

PMM_EXPORT int pmm_conv1d_fwd(const void* x, long long ldx, const float* pre_scale,
                              const float* pre_bias, const float* w, const float* bias,
                              const float* window, const int* seq_of, const int* cu,
                              const int* slots, void* y, int T, int C, int K, int dtype,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  if (K < 2 || C <= 0 || (C + 127) / 128 > 65535) return PMM_ERR_BAD_ARGUMENT;
  if (dtype == PMM_DTYPE_BF16 && K >= 2 && K <= 4 && C % 8 == 0 && ldx % 8 == 0 &&
      reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0) {
    dim3 vgrid((T + pmm::kConvStrip - 1) / pmm::kConvStrip, (C / 8 + 127) / 128);
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    __nv_bfloat16* yb = static_cast<__nv_bfloat16*>(y);
    if (K == 2) pmm::conv1d_fwd_vec_kernel<2><<<vgrid, 128, 0, stream>>>(xb, ldx, pre_scale, pre_bias, w, bias, window, seq_of, cu, slots, yb, T, C);
    if (K == 3) pmm::conv1d_fwd_vec_kernel<3><<<vgrid, 128, 0, stream>>>(xb, ldx, pre_scale, pre_bias, w, bias, window, seq_of, cu, slots, yb, T, C);
    if (K == 4) pmm::conv1d_fwd_vec_kernel<4><<<vgrid, 128, 0, stream>>>(xb, ldx, pre_scale, pre_bias, w, bias, window, seq_of, cu, slots, yb, T, C);
    return pmm::launch_status();
  }
  dim3 grid(T, (C + 127) / 128);
  PMM_DISPATCH_DTYPE(dtype, S, pmm::conv1d_fwd_kernel<S><<<grid, 128, 0, stream>>>(
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
  PMM_DISPATCH_DTYPE(dtype, S, pmm::conv1d_window_update_kernel<S><<<grid, 128, 0, stream>>>(
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

// Paged grouped-query flash attention on tensor cores (bfloat16 storage, float accumulate).
//
// One block = one tile of query rows of ONE sequence and ONE key/value head, and one key
// split.  A "row" is a (token, query head of the group) pair, so the G = Hq/Hkv query
// heads that share a key/value head share every K/V tile that is fetched.  K/V tiles of 64
// keys are gathered row by row through the block table (its entries for the block's key range
// are read into shared memory first) with cp.async (16 bytes a time, zero-filled beyond the
// key range) into a ring of shared-memory stages; S = Q K^T and O += P V run on mma.sync
// m16n8k16 with ldmatrix operands, the Q fragments staying in registers; softmax is the online
// form in float (ex2 with the scale folded into the exponent).  Two shapes:
//   * tile of 64 rows, warp w owns rows 16w..16w+15 and walks all keys   (prompt portions)
//   * tile of 16 rows, tiles are fetched four at a time, each warp takes one whole tile and
//     the warps are merged at the end through shared memory              (decode: G rows)
// With several key splits the block writes (max, sum, unnormalised output) and
// flash_combine merges them; with one split it writes the normalised output.
//
//   sc[s] = (q.K[s]) * scale;  p = exp(sc - max);  o = sum p V / sum p
// (reference src/ops/gpu/attention.cu:44-105), keys lo..pos per token, lo from the window.
#include "mma_helpers.cuh"
#include <math_constants.h>

namespace pmm {

constexpr int kFlashKeys = 64;  // keys per tile

// Decode blocks walk few tiles and pay memory latency for each one they wait for: they keep
// four tiles in flight.  Prompt tiles have work to hide it behind: two tiles ahead, one where
// the rows are long and shared memory would limit the blocks per SM.
__host__ __device__ constexpr int flash_stages(int dh, bool splitw) { return splitw ? 4 : (dh > 64 ? 2 : 3); }

// Decode steps (every sequence brings exactly one token) can hand the kernel the unrotated
// projections instead of prepared queries: the block then scales and rotates its query rows
// itself, and the block whose key range holds the new position rotates the new key, writes key
// and value into the cache page and into its own shared-memory tile.
//   x' = x*scale;  ang = float(pos) * inv_freq[i];
//   x'[i] <- x'[i] cos - x'[i+Dh/2] sin;  x'[i+Dh/2] <- x'[i+Dh/2] cos + x'[i] sin
// (the formulas of the separate rotation kernel; reference src/ops/gpu/attention.cu:4-40)
struct FlashDecodeInputs {
  const bf16* q;          // [n_seq, ldq] unrotated queries, or nullptr: `q` of the kernel is ready
  long long ldq;
  const bf16* k;          // [n_seq, ldk] new keys, or nullptr: the cache holds them already
  long long ldk;
  const bf16* v;
  long long ldv;
  float q_scale, k_scale, v_scale;
  const float* inv_freq;  // [Dh/2], or nullptr: no rotation
  bf16* pool_w;           // the cache, writable
  int one_token;          // tile index == sequence index == token index
};

// MT = row tiles of 16 per warp: 1 (64 rows a block) or 2 (128 rows a block, every K/V fragment
// read from shared memory feeds two row tiles).  Decode blocks (SPLITW) have one 16-row tile.
template <int DH, bool SPLITW, int MT>
__global__ void __launch_bounds__(128)
    flash_paged_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool,
                       const int* __restrict__ block_table, int max_blocks,
                       const int* __restrict__ positions, const int* __restrict__ cu,
                       bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                       float scale_log2, int window, int split_len, int n_splits, int page_size,
                       int n_seq, int Hq, int Hkv, int* __restrict__ split_counter, FlashDecodeInputs dec) {
  static_assert(!SPLITW || MT == 1, "decode tiles have 16 rows");
  constexpr int M = SPLITW ? 16 : 64 * MT;
  constexpr int KT = kFlashKeys;
  constexpr int STRIDE = DH + 8;
  constexpr int NT_S = KT / 8;
  constexpr int KS_Q = DH / 16;
  constexpr int NT_O = DH / 8;
  constexpr int CHUNKS = DH / 8;  // 16-byte chunks per row
  constexpr int NSTAGE = flash_stages(DH, SPLITW);
  constexpr int BT_CAP = 512;  // block-table entries of this block's key range kept in shared memory

  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
  bf16* sK = sQ + M * STRIDE;
  bf16* sV = sK + NSTAGE * KT * STRIDE;
  __shared__ int s_pos[128];
  __shared__ int s_bt[BT_CAP];
  __shared__ float s_wm[4][16], s_wl[4][16], s_M[128], s_L[128];

  // Token positions, sequence bounds and block tables are inputs of the step, written before its
  // first kernel: they are read before the wait for the previous kernel, whose tail hides them.
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = Hq / Hkv;
  const int tpt = M / G;  // tokens per tile (host guarantees G <= M)
  const int hk = blockIdx.y, z = blockIdx.z;
  const int kv_dim = Hkv * DH;

  // which sequence and which of its tokens this tile covers.  Blocks start in index order and
  // a sequence's last tiles walk the most keys, so the tiles are handed out from the back.
  const int tile_id = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  int seq = 0, acc = 0, tok0, n_tok;
  if (SPLITW && dec.one_token) {
    seq = tok0 = tile_id;
    n_tok = 1;
  } else {
    for (; seq < n_seq; ++seq) {
      const int n = cu[seq + 1] - cu[seq];
      const int nt = (n + tpt - 1) / tpt;
      if (tile_id < acc + nt) break;
      acc += nt;
    }
    if (seq >= n_seq) return;
    tok0 = cu[seq] + (tile_id - acc) * tpt;
    n_tok = min(cu[seq + 1], tok0 + tpt) - tok0;
  }
  const int n_rows = n_tok * G;
  const int* bt = block_table + static_cast<size_t>(seq) * max_blocks;

  if (tid < M) s_pos[tid] = (tid < n_rows) ? positions[tok0 + tid / G] : -1;
  const int pos_min = positions[tok0], pos_max = positions[tok0 + n_tok - 1];
  const int lo_all = window > 0 ? max(0, pos_min - window + 1) : 0;
  const int k_begin = max(lo_all, z * split_len);
  const int k_end = min(pos_max + 1, (z + 1) * split_len);

  const int first_tile = (k_begin / KT) * KT;
  const int n_tiles = k_end > k_begin ? (k_end - first_tile + KT - 1) / KT : 0;

  // The block-table entries of this block's key range go to shared memory once, so that no tile
  // waits for a table entry from L2 before its copies can be issued.
  const int bt_lo = first_tile / page_size;
  const int n_bt = n_tiles > 0 ? (k_end - 1) / page_size - bt_lo + 1 : 0;
  const bool bt_shared = n_bt <= BT_CAP;
  if (bt_shared)
    for (int i = tid; i < n_bt; i += 128) s_bt[i] = bt[bt_lo + i];
  __syncthreads();
  auto page_of = [&](int idx) { return bt_shared ? s_bt[idx - bt_lo] : bt[idx]; };
  // A decode step that reads the projections itself is the only writer of the cache pages in its
  // step: the keys and values of earlier positions may be requested before the wait for the
  // kernel before this one (their latency then hides behind that kernel's tail); only the new
  // token's projections need it.  Every other form waits here: the rotation kernel before it wrote
  // queries and pages.
  const bool late_wait = SPLITW && dec.q != nullptr && dec.k != nullptr;
  if (!late_wait) pdl_wait();

  // the new token of a decode step: this block stores its key and value if its key range holds it
  const int new_pos = pos_max;
  const bool stores_new = SPLITW && dec.k != nullptr && n_tiles > 0 && new_pos >= k_begin && new_pos < k_end;
  constexpr int HALF = DH / 2;
  bf16 *k_dst = nullptr, *v_dst = nullptr, *k_sm = nullptr, *v_sm = nullptr;
  int new_tile = -1;  // the new position's tile in this block's ring (the last tile of its range)
  const bool single_round = n_tiles <= NSTAGE;  // else the ring slot is written in the tile's own round
  if (SPLITW && stores_new) {
    const int page = page_of(new_pos / page_size);
    k_dst = dec.pool_w + (static_cast<size_t>(page) * 2 * page_size + new_pos % page_size) * kv_dim + hk * DH;
    v_dst = k_dst + static_cast<size_t>(page_size) * kv_dim;
    new_tile = (new_pos - first_tile) / KT;
    k_sm = sK + (new_tile % NSTAGE) * KT * STRIDE + (new_pos - first_tile - new_tile * KT) * STRIDE;
    v_sm = sV + (new_tile % NSTAGE) * KT * STRIDE + (new_pos - first_tile - new_tile * KT) * STRIDE;
  }
  // Runs after the first tiles' copies have been requested, so that their latency covers it.
  auto prepare_decode_inputs = [&]() {
    if (SPLITW && stores_new) {
      for (int i = tid; i < HALF; i += 128) {
        const bf16* src = dec.k + static_cast<long long>(tok0) * dec.ldk + hk * DH;
        const float x1 = __bfloat162float(src[i]) * dec.k_scale, x2 = __bfloat162float(src[i + HALF]) * dec.k_scale;
        float o1 = x1, o2 = x2;
        if (dec.inv_freq) {
          const float ang = static_cast<float>(new_pos) * dec.inv_freq[i];
          const float c = cosf(ang), sn = sinf(ang);
          o1 = x1 * c - x2 * sn;
          o2 = x2 * c + x1 * sn;
        }
        const bf16 b1 = __float2bfloat16_rn(o1), b2 = __float2bfloat16_rn(o2);
        k_dst[i] = b1;
        k_dst[i + HALF] = b2;
        if (single_round) {
          k_sm[i] = b1;
          k_sm[i + HALF] = b2;
        }
      }
      for (int i = tid; i < DH; i += 128) {
        const bf16 b = __float2bfloat16_rn(__bfloat162float(dec.v[static_cast<long long>(tok0) * dec.ldv + hk * DH + i]) * dec.v_scale);
        v_dst[i] = b;
        if (single_round) v_sm[i] = b;
      }
    }
    if (SPLITW && dec.q != nullptr && n_tiles > 0) {
      for (int idx = tid; idx < M * HALF; idx += 128) {
        const int r = idx / HALF, i = idx % HALF;
        float o1 = 0.f, o2 = 0.f;
        if (r < n_rows) {
          const bf16* src = dec.q + static_cast<long long>(tok0 + r / G) * dec.ldq + (hk * G + r % G) * DH;
          const float x1 = __bfloat162float(src[i]) * dec.q_scale, x2 = __bfloat162float(src[i + HALF]) * dec.q_scale;
          o1 = x1;
          o2 = x2;
          if (dec.inv_freq) {
            const float ang = static_cast<float>(s_pos[r]) * dec.inv_freq[i];
            const float c = cosf(ang), sn = sinf(ang);
            o1 = x1 * c - x2 * sn;
            o2 = x2 * c + x1 * sn;
          }
        }
        sQ[r * STRIDE + i] = __float2bfloat16_rn(o1);
        sQ[r * STRIDE + i + HALF] = __float2bfloat16_rn(o2);
      }
    }
  };

  // Q rows -> shared memory (rows beyond the tile are zero)
  if (n_tiles > 0 && !(SPLITW && dec.q != nullptr)) {
    for (int c = tid; c < M * CHUNKS; c += 128) {
      const int r = c / CHUNKS, col = c % CHUNKS;
      const bool ok = r < n_rows;
      const size_t src = ok ? (static_cast<size_t>(tok0 + r / G) * Hq + hk * G + r % G) * DH + col * 8 : 0;
      cp_async16(sQ + r * STRIDE + col * 8, q + src, ok);
    }
  }

  // A tile of 64 keys lies inside one page when the page size is a multiple of 64: then one
  // table look-up serves the whole tile and every thread's pieces sit at fixed offsets from it.
  const bool tile_in_page = (page_size % KT) == 0;
  constexpr int RSTEP = 128 / CHUNKS;  // rows of a tile that one pass of the block covers
  constexpr int PIECES = KT / RSTEP;   // passes (row, 16-byte column) per thread and tile
  const int ld_r0 = tid / CHUNKS, ld_col = (tid % CHUNKS) * 8;
  const int ld_soff = ld_r0 * STRIDE + ld_col;
  const size_t v_off = static_cast<size_t>(page_size) * kv_dim;
  auto load_tile = [&](int stage, int base) {
    bf16* dK = sK + stage * KT * STRIDE + ld_soff;
    bf16* dV = sV + stage * KT * STRIDE + ld_soff;
    if (tile_in_page) {
      const int page = page_of(base / page_size);
      const bf16* src = pool + (static_cast<size_t>(page) * 2 * page_size + base % page_size + ld_r0) * kv_dim +
                        hk * DH + ld_col;
      const bool holds_new = SPLITW && stores_new && new_pos >= base && new_pos < base + KT;
      if (base >= k_begin && base + KT <= k_end && !holds_new) {  // every key of the tile is wanted
#pragma unroll
        for (int j = 0; j < PIECES; ++j) {
          cp_async16_all(dK + j * RSTEP * STRIDE, src + static_cast<size_t>(j * RSTEP) * kv_dim);
          cp_async16_all(dV + j * RSTEP * STRIDE, src + static_cast<size_t>(j * RSTEP) * kv_dim + v_off);
        }
      } else {
#pragma unroll
        for (int j = 0; j < PIECES; ++j) {
          const int key = base + ld_r0 + j * RSTEP;
          if (holds_new && key == new_pos) continue;  // this block writes that row itself
          const bool ok = key >= k_begin && key < k_end;
          const bf16* sj = ok ? src + static_cast<size_t>(j * RSTEP) * kv_dim : pool;
          cp_async16(dK + j * RSTEP * STRIDE, sj, ok);
          cp_async16(dV + j * RSTEP * STRIDE, ok ? sj + v_off : pool, ok);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < PIECES; ++j) {
        const int key = base + ld_r0 + j * RSTEP;
        if (SPLITW && stores_new && key == new_pos) continue;  // this block writes that row itself
        const bool ok = key >= k_begin && key < k_end;
        size_t src = 0;
        if (ok) {
          const int page = page_of(key / page_size);
          src = (static_cast<size_t>(page) * 2 * page_size + key % page_size) * kv_dim + hk * DH + ld_col;
        }
        cp_async16(dK + j * RSTEP * STRIDE, pool + src, ok);
        cp_async16(dV + j * RSTEP * STRIDE, pool + (ok ? src + v_off : 0), ok);
      }
    }
  };

  // Warp w owns rows row_base .. row_base + 16*MT - 1; in fragment layout a thread holds, of
  // each 16-row tile, row (lane/4) ["lo"] and row (lane/4 + 8) ["hi"].
  const int row_base = SPLITW ? 0 : warp * 16 * MT;
  const int r_lo = lane >> 2, r_hi = r_lo + 8;
  // running maxima are kept in the exponent's unit (score * scale * log2 e)
  float m_lo[MT], m_hi[MT], l_lo[MT], l_hi[MT];
  float o[MT][NT_O][4];
  unsigned qf[MT][KS_Q][4];  // the warp's query rows as mma A fragments, read from shared memory once
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_lo[mt] = m_hi[mt] = -CUDART_INF_F;
    l_lo[mt] = l_hi[mt] = 0.f;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;
  }
  auto load_q_fragments = [&]() {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int ks = 0; ks < KS_Q; ++ks)
        ldmatrix_x4(qf[mt][ks][0], qf[mt][ks][1], qf[mt][ks][2], qf[mt][ks][3],
                    sQ + (row_base + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + ks * 16 +
                        (lane >> 4) * 8);
  };
  const int k_lane_off = ((lane & 7) + (lane >> 4) * 8) * STRIDE + ((lane >> 3) & 1) * 8;
  const int v_lane_off = ((lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + (lane >> 4) * 8;

  // one tile of 64 keys against this warp's rows
  auto process_tile = [&](int stage, int base) {
    const bf16* tK = sK + stage * KT * STRIDE + k_lane_off;
    const bf16* tV = sV + stage * KT * STRIDE + v_lane_off;

    // S = Q K^T
    float s[MT][NT_S][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < NT_S; ++i) s[mt][i][0] = s[mt][i][1] = s[mt][i][2] = s[mt][i][3] = 0.f;
    // The fragment loads and the mma instructions issue in program order, so the K fragments of
    // step ks+1 are requested before the products of step ks: their latency hides behind them.
    unsigned bk[2][NT_S / 2][4];
    auto load_k = [&](int ks) {
#pragma unroll
      for (int np = 0; np < NT_S / 2; ++np)
        ldmatrix_x4(bk[ks & 1][np][0], bk[ks & 1][np][1], bk[ks & 1][np][2], bk[ks & 1][np][3],
                    tK + np * 16 * STRIDE + ks * 16);
    };
    load_k(0);
#pragma unroll
    for (int ks = 0; ks < KS_Q; ++ks) {
      if (ks + 1 < KS_Q) load_k(ks + 1);
#pragma unroll
      for (int np = 0; np < NT_S / 2; ++np) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16(s[mt][2 * np], qf[mt][ks], bk[ks & 1][np][0], bk[ks & 1][np][1]);
          mma_bf16(s[mt][2 * np + 1], qf[mt][ks], bk[ks & 1][np][2], bk[ks & 1][np][3]);
        }
      }
    }
    // the first V fragments travel while the softmax is computed
    unsigned bv[2][NT_O / 2][4];
    auto load_v = [&](int kk) {
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np)
        ldmatrix_x4_trans(bv[kk & 1][np][0], bv[kk & 1][np][1], bv[kk & 1][np][2], bv[kk & 1][np][3],
                          tV + kk * 16 * STRIDE + np * 16);
    };
    load_v(0);

    // mask and online softmax; the scale is applied inside the exponent (one fused multiply-add
    // per score).  A tile that every row of the block may read in full (inside the split, before
    // the first row's position, inside the last row's window) needs no mask.
    const bool full = base >= k_begin && base + KT <= k_end && base + KT - 1 <= pos_min &&
                      (window <= 0 || base >= pos_max - window + 1);  // rows beyond the tile are never written out
    unsigned pa[MT][KT / 16][4];  // P as bfloat16 A fragments
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      if (!full) {
        const int pos_lo = s_pos[row_base + mt * 16 + r_lo], pos_hi = s_pos[row_base + mt * 16 + r_hi];
#pragma unroll
        for (int nt = 0; nt < NT_S; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = base + nt * 8 + (lane & 3) * 2 + (e & 1);
            const int pos = (e < 2) ? pos_lo : pos_hi;
            const int lo = window > 0 ? max(pos - window + 1, k_begin) : k_begin;
            const bool ok = pos >= 0 && key <= pos && key >= lo && key < k_end;
            if (!ok) s[mt][nt][e] = -CUDART_INF_F;
          }
        }
      }
      float mx_lo = -CUDART_INF_F, mx_hi = -CUDART_INF_F;
#pragma unroll
      for (int nt = 0; nt < NT_S; ++nt) {
        mx_lo = fmaxf(mx_lo, fmaxf(s[mt][nt][0], s[mt][nt][1]));
        mx_hi = fmaxf(mx_hi, fmaxf(s[mt][nt][2], s[mt][nt][3]));
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo[mt], mx_lo * scale_log2), mn_hi = fmaxf(m_hi[mt], mx_hi * scale_log2);  // scale > 0
      const float mu_lo = (mn_lo == -CUDART_INF_F) ? 0.f : mn_lo;
      const float mu_hi = (mn_hi == -CUDART_INF_F) ? 0.f : mn_hi;
      const float al_lo = ex2_approx(m_lo[mt] - mu_lo), al_hi = ex2_approx(m_hi[mt] - mu_hi);
      m_lo[mt] = mn_lo;
      m_hi[mt] = mn_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int nt = 0; nt < NT_S; ++nt) {
        const float p0 = ex2_approx(fmaf(s[mt][nt][0], scale_log2, -mu_lo));
        const float p1 = ex2_approx(fmaf(s[mt][nt][1], scale_log2, -mu_lo));
        const float p2 = ex2_approx(fmaf(s[mt][nt][2], scale_log2, -mu_hi));
        const float p3 = ex2_approx(fmaf(s[mt][nt][3], scale_log2, -mu_hi));
        sum_lo += p0 + p1;
        sum_hi += p2 + p3;
        pa[mt][nt / 2][(nt & 1) * 2] = pack_bf16(p0, p1);
        pa[mt][nt / 2][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
      l_lo[mt] = l_lo[mt] * al_lo + sum_lo;
      l_hi[mt] = l_hi[mt] * al_hi + sum_hi;
      if (__any_sync(0xffffffffu, al_lo != 1.f || al_hi != 1.f)) {  // some row's maximum moved
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
          o[mt][i][0] *= al_lo;
          o[mt][i][1] *= al_lo;
          o[mt][i][2] *= al_hi;
          o[mt][i][3] *= al_hi;
        }
      }
    }

    // O += P V
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
      if (kk + 1 < KT / 16) load_v(kk + 1);
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16(o[mt][2 * np], pa[mt][kk], bv[kk & 1][np][0], bv[kk & 1][np][1]);
          mma_bf16(o[mt][2 * np + 1], pa[mt][kk], bv[kk & 1][np][2], bv[kk & 1][np][3]);
        }
      }
    }
  };

  if constexpr (SPLITW) {
    // decode: rounds of four tiles, requested together (one memory latency a round), one per warp
    for (int round0 = 0; round0 < n_tiles; round0 += NSTAGE) {
#pragma unroll
      for (int st = 0; st < NSTAGE; ++st)
        if (round0 + st < n_tiles) load_tile(st, first_tile + (round0 + st) * KT);
      if (stores_new && !single_round && new_tile >= round0 && new_tile < round0 + NSTAGE) {
        // the new key and value, read back from where this thread put them in the cache
        for (int i = tid; i < HALF; i += 128) {
          k_sm[i] = k_dst[i];
          k_sm[i + HALF] = k_dst[i + HALF];
        }
        for (int i = tid; i < DH; i += 128) v_sm[i] = v_dst[i];
      }
      cp_async_commit();  // the first group also carries the Q rows
      if (round0 == 0) {
        if (late_wait) pdl_wait();
        prepare_decode_inputs();
      }
      cp_async_wait<0>();
      __syncthreads();
      if (round0 == 0) load_q_fragments();
      if (round0 + warp < n_tiles) process_tile(warp, first_tile + (round0 + warp) * KT);
      __syncthreads();  // the tiles are overwritten by the next round
    }
  } else if (n_tiles > 0) {
    // Prompt tiles walk their keys from the last tile (the masked one on the diagonal) down to
    // the first: row tiles that start together then read different parts of the cache.
    const int last_tile = first_tile + (n_tiles - 1) * KT;
    cp_async_commit();  // group 0: the Q rows
#pragma unroll
    for (int st = 0; st < NSTAGE - 1; ++st) {
      if (st < n_tiles) load_tile(st, last_tile - st * KT);
      cp_async_commit();
    }
    cp_async_wait<NSTAGE - 1>();  // all but the newest NSTAGE-1 groups: the Q rows are there
    __syncthreads();
    load_q_fragments();
    for (int it = 0; it < n_tiles; ++it) {
      const int base = last_tile - it * KT;
      // tile groups so far: (NSTAGE-1) + it; tile `it` has landed when at most NSTAGE-2 newer ones are pending
      cp_async_wait<NSTAGE - 2>();
      __syncthreads();  // tile `it` is visible to all; everyone is done with tile it-1, whose stage is refilled now
      if (it + NSTAGE - 1 < n_tiles) load_tile((it + NSTAGE - 1) % NSTAGE, base - (NSTAGE - 1) * KT);
      cp_async_commit();
      process_tile(it % NSTAGE, base);
    }
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  if (late_wait && n_tiles == 0) pdl_wait();  // (a block without keys writes its empty part only then, too)

  constexpr float kLn2 = 0.6931471805599453f;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    l_lo[mt] += __shfl_xor_sync(0xffffffffu, l_lo[mt], 1);
    l_lo[mt] += __shfl_xor_sync(0xffffffffu, l_lo[mt], 2);
    l_hi[mt] += __shfl_xor_sync(0xffffffffu, l_hi[mt], 1);
    l_hi[mt] += __shfl_xor_sync(0xffffffffu, l_hi[mt], 2);
  }

  if constexpr (!SPLITW) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = row_base + mt * 16 + (half ? r_hi : r_lo);
        if (r >= n_rows) continue;
        const float m = half ? m_hi[mt] : m_lo[mt], l = half ? l_hi[mt] : l_lo[mt];
        const int t = tok0 + r / G, hq = hk * G + r % G;
        if (n_splits == 1) {
          const float inv = l > 0.f ? 1.f / l : 0.f;
          bf16* dst = out + (static_cast<size_t>(t) * Hq + hq) * DH;
#pragma unroll
          for (int nt = 0; nt < NT_O; ++nt) {
            const int d = nt * 8 + (lane & 3) * 2;
            *reinterpret_cast<__nv_bfloat162*>(dst + d) =
                __floats2bfloat162_rn(o[mt][nt][half * 2] * inv, o[mt][nt][half * 2 + 1] * inv);
          }
        } else {
          const size_t pi = (static_cast<size_t>(t) * Hq + hq) * n_splits + z;
          float* dst = part_o + pi * DH;
#pragma unroll
          for (int nt = 0; nt < NT_O; ++nt) {
            const int d = nt * 8 + (lane & 3) * 2;
            *reinterpret_cast<float2*>(dst + d) = make_float2(o[mt][nt][half * 2], o[mt][nt][half * 2 + 1]);
          }
          if ((lane & 3) == 0) *reinterpret_cast<float2*>(part_ml + pi * 2) = make_float2(m * kLn2, l);
        }
      }
    }
  } else {
    // merge the four warps (each saw a quarter of the tiles) through shared memory
    constexpr int SO = DH + 4;                 // padded row: rows g and g+1 fall into different banks
    float* sO = reinterpret_cast<float*>(sK);  // [4 warps][16][SO], K/V tiles are no longer needed
    if ((lane & 3) == 0) {
      s_wm[warp][r_lo] = m_lo[0];
      s_wm[warp][r_hi] = m_hi[0];
      s_wl[warp][r_lo] = l_lo[0];
      s_wl[warp][r_hi] = l_hi[0];
    }
    __syncthreads();
    if (tid < 16) {
      float mm = -CUDART_INF_F;
      for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_wm[w][tid]);
      const float mu = (mm == -CUDART_INF_F) ? 0.f : mm;
      float ll = 0.f;
      for (int w = 0; w < 4; ++w) ll += s_wl[w][tid] * exp2f(s_wm[w][tid] - mu);
      s_M[tid] = mm;
      s_L[tid] = ll;
    }
    __syncthreads();
    {
      const float mu_lo = (s_M[r_lo] == -CUDART_INF_F) ? 0.f : s_M[r_lo];
      const float mu_hi = (s_M[r_hi] == -CUDART_INF_F) ? 0.f : s_M[r_hi];
      const float f_lo = exp2f(m_lo[0] - mu_lo), f_hi = exp2f(m_hi[0] - mu_hi);
      float* mine = sO + warp * 16 * SO;
#pragma unroll
      for (int nt = 0; nt < NT_O; ++nt) {
        const int d = nt * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(mine + r_lo * SO + d) = make_float2(o[0][nt][0] * f_lo, o[0][nt][1] * f_lo);
        *reinterpret_cast<float2*>(mine + r_hi * SO + d) = make_float2(o[0][nt][2] * f_hi, o[0][nt][3] * f_hi);
      }
    }
    __syncthreads();
    for (int i = tid; i < n_rows * DH; i += 128) {
      const int r = i / DH, d = i % DH;
      const int t = tok0 + r / G, hq = hk * G + r % G;
      const float sum = (sO[r * SO + d] + sO[(16 + r) * SO + d]) + (sO[(32 + r) * SO + d] + sO[(48 + r) * SO + d]);
      if (n_splits == 1) {
        const float l = s_L[r];
        out[(static_cast<size_t>(t) * Hq + hq) * DH + d] = __float2bfloat16_rn(l > 0.f ? sum / l : 0.f);
      } else {
        const size_t pi = (static_cast<size_t>(t) * Hq + hq) * n_splits + z;
        part_o[pi * DH + d] = sum;
        if (d == 0) {
          part_ml[pi * 2] = s_M[r] * kLn2;
          part_ml[pi * 2 + 1] = s_L[r];
        }
      }
    }
  }

  // With a counter the block that finishes a tile's last key split merges all of them, so no
  // second launch is needed.  The counter returns to zero for the next use.
  if (n_splits > 1 && split_counter != nullptr) {
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    int* counter = split_counter + static_cast<size_t>(tile_id) * gridDim.y + hk;
    if (tid == 0) s_last = (atomicAdd(counter, 1) == n_splits - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) *counter = 0;
    // A thread per (row, four columns) merges the splits in one pass with a running maximum,
    // eight splits' loads in flight at a time.
    constexpr int C4 = DH / 4;
    constexpr int kBatch = 8;
    for (int i = tid; i < n_rows * C4; i += 128) {
      const int r = i / C4, d = (i % C4) * 4;
      const int t = tok0 + r / G, hq = hk * G + r % G;
      const size_t row = static_cast<size_t>(t) * Hq + hq;
      const float2* ml = reinterpret_cast<const float2*>(part_ml + row * n_splits * 2);
      const float* po = part_o + row * n_splits * DH + d;
      float mx = -CUDART_INF_F, tot = 0.f;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
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
            a.x = a.x * keep + w * x[u].x;
            a.y = a.y * keep + w * x[u].y;
            a.z = a.z * keep + w * x[u].z;
            a.w = a.w * keep + w * x[u].w;
            tot = tot * keep + w * v[u].y;
            mx = mn;
          }
        }
      }
      const float inv = tot > 0.f ? 1.f / tot : 0.f;
      uint2 packed;
      packed.x = pack_bf16(a.x * inv, a.y * inv);
      packed.y = pack_bf16(a.z * inv, a.w * inv);
      *reinterpret_cast<uint2*>(out + row * DH + d) = packed;
    }
  }
}

// One block per (token, query head): merges the partial results of the key splits.
// weights w_z = sum_z>0 ? exp(m_z - max m) : 0 are formed first, then every output element
// is a dot product over the splits with independent loads.
template <typename S>
__global__ void __launch_bounds__(128)
    flash_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                         S* __restrict__ out, int n_splits, int Dh) {
  extern __shared__ float w[];  // n_splits weights
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  const float* ml = part_ml + row * n_splits * 2;
  float mx = -CUDART_INF_F;
  for (int z = threadIdx.x; z < n_splits; z += blockDim.x)
    if (ml[2 * z + 1] > 0.f) mx = fmaxf(mx, ml[2 * z]);
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for (int i = 1; i < static_cast<int>(blockDim.x >> 5); ++i) mx = fmaxf(mx, red[i]);
  float part = 0.f;
  for (int z = threadIdx.x; z < n_splits; z += blockDim.x) {
    const float l = ml[2 * z + 1];
    const float wz = l > 0.f ? expf(ml[2 * z] - mx) : 0.f;
    w[z] = wz;
    part += wz * l;
  }
  const float total = block_sum(part, red);  // syncs: w[] is complete afterwards
  const float inv = total > 0.f ? 1.f / total : 0.f;
  const float* po = part_o + row * n_splits * Dh;
  for (int d = threadIdx.x; d < Dh; d += blockDim.x) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    int z = 0;
    for (; z + 4 <= n_splits; z += 4) {
      a0 += w[z] * po[static_cast<size_t>(z) * Dh + d];
      a1 += w[z + 1] * po[static_cast<size_t>(z + 1) * Dh + d];
      a2 += w[z + 2] * po[static_cast<size_t>(z + 2) * Dh + d];
      a3 += w[z + 3] * po[static_cast<size_t>(z + 3) * Dh + d];
    }
    for (; z < n_splits; ++z) a0 += w[z] * po[static_cast<size_t>(z) * Dh + d];
    stf(out + row * Dh + d, ((a0 + a1) + (a2 + a3)) * inv);
  }
}

template <int DH, bool SPLITW, int MT>
int launch_flash(const void* q, const void* pool, const int* block_table, int max_blocks,
                 const int* positions, const int* cu, void* out, float* part_o, float* part_ml,
                 float scale, int window, int split_len, int n_splits, int page_size, int n_seq,
                 int n_tiles, int Hq, int Hkv, int* split_counter, const FlashDecodeInputs& dec,
                 cudaStream_t stream) {
  constexpr int M = SPLITW ? 16 : 64 * MT;
  constexpr int NSTAGE = flash_stages(DH, SPLITW);
  const size_t smem = static_cast<size_t>(M + 2 * NSTAGE * kFlashKeys) * (DH + 8) * sizeof(bf16);
  auto kern = flash_paged_kernel<DH, SPLITW, MT>;
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  dim3 grid(n_tiles, Hkv, n_splits);
  launch_pdl(kern, grid, dim3(128), smem, stream, static_cast<const bf16*>(q), static_cast<const bf16*>(pool),
             block_table, max_blocks, positions, cu, static_cast<bf16*>(out), part_o, part_ml,
             scale * 1.4426950408889634f, window, split_len, n_splits, page_size, n_seq, Hq, Hkv, split_counter, dec);
  return launch_status();
}

}  // namespace pmm

// Whether the tensor-core kernel takes this shape (bfloat16 only; the caller checks the type).
PMM_EXPORT int pmm_flash_supported(int Hq, int Hkv, int Dh) {
  if (Hkv <= 0 || Hq % Hkv) return 0;
  const int G = Hq / Hkv;
  return (Dh == 16 || Dh == 32 || Dh == 64 || Dh == 128) && G <= 64 ? 1 : 0;
}

namespace pmm {
int flash_dispatch(const void* q, const void* pool, const int* block_table, int max_blocks,
                   const int* positions, const int* cu, void* out, float* part_o, float* part_ml,
                   float scale, int window, int split_len, int n_splits, int page_size, int n_seq,
                   int n_tiles, int tile_rows, int Hq, int Hkv, int Dh, int* split_counter,
                   const FlashDecodeInputs& dec, cudaStream_t stream) {
  if (n_seq <= 0 || n_tiles <= 0) return 0;
  if (!pmm_flash_supported(Hq, Hkv, Dh) || page_size <= 0 || n_splits < 1 || n_splits > 65535 ||
      Hkv > 65535)
    return PMM_ERR_BAD_ARGUMENT;
  if (tile_rows != 16 && tile_rows != 64 && tile_rows != 128) return PMM_ERR_BAD_ARGUMENT;
  if (Hq / Hkv > tile_rows || (tile_rows == 128 && Dh > 64)) return PMM_ERR_BAD_ARGUMENT;
  if (!(scale > 0.f)) return PMM_ERR_BAD_ARGUMENT;  // the maximum is taken before the scale is applied
  if (n_splits > 1 && (!part_o || !part_ml || split_len <= 0)) return PMM_ERR_BAD_ARGUMENT;
  if (split_counter && n_splits > 64) return PMM_ERR_BAD_ARGUMENT;
  if (n_splits == 1) split_len = 0x40000000;
  int rc;
#define PMM_FLASH_ARGS                                                                                  \
  q, pool, block_table, max_blocks, positions, cu, out, part_o, part_ml, scale, window, split_len,      \
      n_splits, page_size, n_seq, n_tiles, Hq, Hkv, split_counter, dec, stream
#define PMM_FLASH_CASE(DH)                                                       \
  rc = tile_rows == 16 ? launch_flash<DH, true, 1>(PMM_FLASH_ARGS)               \
                       : launch_flash<DH, false, 1>(PMM_FLASH_ARGS)
  if (tile_rows == 128) {
    switch (Dh) {
      case 16: rc = launch_flash<16, false, 2>(PMM_FLASH_ARGS); break;
      case 32: rc = launch_flash<32, false, 2>(PMM_FLASH_ARGS); break;
      case 64: rc = launch_flash<64, false, 2>(PMM_FLASH_ARGS); break;
      default: return PMM_ERR_BAD_ARGUMENT;
    }
    return rc;
  }
  switch (Dh) {
    case 16: PMM_FLASH_CASE(16); break;
    case 32: PMM_FLASH_CASE(32); break;
    case 64: PMM_FLASH_CASE(64); break;
    case 128: PMM_FLASH_CASE(128); break;
    default: return PMM_ERR_BAD_ARGUMENT;
  }
#undef PMM_FLASH_ARGS
#undef PMM_FLASH_CASE
  return rc;
}
}  // namespace pmm

// tile_rows M: 16 (every sequence brings at most 16/G tokens: decode), 64, or 128 (head sizes
// up to 64).  n_tiles: number of row tiles = sum over sequences of ceil(new tokens / (M / G)).
// split_counter: nullptr (the caller merges key splits with pmm_flash_combine), or
// n_tiles*Hkv ints that are zero between calls: then the last block of every tile merges
// its splits (at most 64 of them) and writes `out` itself.
PMM_EXPORT int pmm_flash_paged_attention(const void* q, const void* pool, const int* block_table,
                                         int max_blocks, const int* positions, const int* cu,
                                         void* out, float* part_o, float* part_ml, float scale,
                                         int window, int split_len, int n_splits, int page_size,
                                         int n_seq, int n_tiles, int tile_rows, int Hq, int Hkv, int Dh,
                                         int* split_counter, cudaStream_t stream) {
  pmm::FlashDecodeInputs dec{};
  return pmm::flash_dispatch(q, pool, block_table, max_blocks, positions, cu, out, part_o, part_ml, scale,
                             window, split_len, n_splits, page_size, n_seq, n_tiles, tile_rows, Hq, Hkv, Dh,
                             split_counter, dec, stream);
}

// Decode step, every sequence one token (token t belongs to sequence t): attention straight from
// the projections.  q_src/k_src/v_src: [n_seq, ld*] unrotated slices; queries and keys are scaled
// and rotated (inv_freq [Dh/2], or nullptr for no rotation) as the separate rotation kernel does,
// and the new key and value are written into the cache page of their position.  k_src == nullptr:
// the cache holds the new keys already (a layer that reads another layer's cache).
// Needs Hq/Hkv <= 16; positions[t] is the new token's position.
PMM_EXPORT int pmm_flash_decode_attention(const void* q_src, long long ldq, const void* k_src, long long ldk,
                                          const void* v_src, long long ldv, float q_scale, float k_scale,
                                          float v_scale, const float* inv_freq, void* pool,
                                          const int* block_table, int max_blocks, const int* positions,
                                          void* out, float* part_o, float* part_ml, float scale, int window,
                                          int split_len, int n_splits, int page_size, int n_seq, int Hq,
                                          int Hkv, int Dh, int* split_counter, cudaStream_t stream) {
  if (!q_src || (k_src == nullptr) != (v_src == nullptr) || Hkv <= 0 || Hq % Hkv || Hq / Hkv > 16)
    return PMM_ERR_BAD_ARGUMENT;
  if (n_splits > 1 && !split_counter) return PMM_ERR_BAD_ARGUMENT;  // the separate merge is not wired here
  pmm::FlashDecodeInputs dec{};
  dec.q = static_cast<const pmm::bf16*>(q_src);
  dec.ldq = ldq;
  dec.k = static_cast<const pmm::bf16*>(k_src);
  dec.ldk = ldk;
  dec.v = static_cast<const pmm::bf16*>(v_src);
  dec.ldv = ldv;
  dec.q_scale = q_scale;
  dec.k_scale = k_scale;
  dec.v_scale = v_scale;
  dec.inv_freq = inv_freq;
  dec.pool_w = static_cast<pmm::bf16*>(pool);
  dec.one_token = 1;
  return pmm::flash_dispatch(nullptr, pool, block_table, max_blocks, positions, nullptr, out, part_o, part_ml,
                             scale, window, split_len, n_splits, page_size, n_seq, n_seq, 16, Hq, Hkv, Dh,
                             split_counter, dec, stream);
}

// Merge of key splits: part_o [rows, n_splits, Dh], part_ml [rows, n_splits, 2] -> out [rows, Dh].
PMM_EXPORT int pmm_flash_combine(const float* part_o, const float* part_ml, void* out, int n_rows,
                                 int n_splits, int Dh, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (n_splits < 1 || Dh <= 0) return PMM_ERR_BAD_ARGUMENT;
  const size_t smem = static_cast<size_t>(n_splits) * sizeof(float);
  if (smem > 48 * 1024) return PMM_ERR_BAD_ARGUMENT;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::flash_combine_kernel<S>, dim3(n_rows), dim3(128), smem, stream,
                                               part_o, part_ml, static_cast<S*>(out), n_splits, Dh));
  return pmm::launch_status();
}

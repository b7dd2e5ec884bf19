// build: precise-math
// Ragged-batch kernels for decoders whose token mixers carry per-sequence state besides (or instead of) a paged key/value cache:
// short causal convolutions over time, sliding-window attention that keeps the first tokens of a sequence visible, and two
// recurrent matrix memories.  Every kernel takes its sizes as arguments and exists for 16-bit (bf16) and 32-bit activations;
// recurrent state, gates, decays, norms and softmax are always fp32.
//
// A batch is described per sequence by `seq_desc` (int4: first row of the sequence in the batch, number of new tokens, tokens
// seen before this step = position of the first new token, state slot).  State of a sequence lives in its slot of per-layer
// buffers; a sequence whose first new token has position 0 starts from zero state whatever its slot holds (slots are reused
// without being cleared).
//
//   window_qk_prepare     short convolution of the query / key projections -> values (= convolved keys) into cache plane 1,
//                         RMS norm over the whole query / key projection, interleaved rotary on the first rot_dims of every head,
//                         keys into cache plane 0
//   conv_state_update     keeps the last taps - 1 projected rows of every sequence for the next step
//   window_attention      softmax attention over the paged cache; query i sees key j <= i when i - j < window or j < keep_first
//   matrix_memory_scan    S <- a S + b k v^T, n <- a n + b k with log-space gates and a running maximum that starts at 0;
//                         o = S^T q / (max(|n . q|, exp(-m)) + 1e-6)
//   delta_prepare         short convolution + silu of q / k / v projections, unit-length q and k per head
//   delta_rule_scan       S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, one decay per head and key channel
//   tied_gate_scan        S <- diag(f) S + (1 - f) v^T; o = S^T q: the forget gate f of every key channel also sets what is written
//                         (q = silu, f = lower + (1 - lower) sigmoid, both formed from the fused projection while it is staged)
//   head_norm_gate        per-head RMS norm of the fp32 read-out, times a weight, times sigmoid(gate) when there is one, times a constant
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#include "../common/host.h"

namespace dsb {
namespace recur {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// reductions over the block; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float siluf_(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float logsigmoidf_(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// ------------------------------------------------------------------------------------------------------ short convolutions
// Value of channel c of the convolution at token i of a sequence's new tokens: sum_j w[c, j] * u(i - (taps - 1) + j), where u(ii) is
// row ii of the new tokens for ii >= 0, the kept row taps - 1 + ii of the sequence's state for ii < 0 when that position exists
// (seen + ii >= 0), and zero before the sequence's start.  `u` points at the channel in the sequence's first new row (row stride
// ld), `st` at the channel in row 0 of the kept rows (row stride st_ld).
template <typename T>
__device__ __forceinline__ float conv_at(const T* __restrict__ u, long long ld, const T* __restrict__ st, int st_ld,
                                         const float* __restrict__ w, int taps, int i, int seen) {
  float acc = 0.f;
#pragma unroll 4
  for (int j = 0; j < taps; ++j) {
    const int ii = i - (taps - 1) + j;
    // one load per tap from a pointer chosen without a branch (the current row stands in where nothing exists), so the loads of all taps
    // are in flight together
    const T* src = ii >= 0 ? u + static_cast<long long>(ii) * ld : (seen + ii >= 0 ? st + (taps - 1 + ii) * st_ld : u + static_cast<long long>(i) * ld);
    const float v = to_f(*src);
    acc = fmaf(w[j], (ii >= 0 || seen + ii >= 0) ? v : 0.f, acc);
  }
  return acc;
}

// The same for a token whose taps all lie among the new rows (i >= taps - 1: every token of a portion but its first taps - 1): no
// selection per tap, the four weights of a 4-tap filter in one load.  Same order of additions as conv_at.
template <typename T>
__device__ __forceinline__ float conv_inside(const T* __restrict__ u, long long ld, const float* __restrict__ w, int taps, int i) {
  const T* p = u + static_cast<long long>(i - (taps - 1)) * ld;
  if (taps == 4) {
    const float4 w4 = *reinterpret_cast<const float4*>(w);
    float acc = w4.x * to_f(p[0]);
    acc = fmaf(w4.y, to_f(p[ld]), acc);
    acc = fmaf(w4.z, to_f(p[2 * ld]), acc);
    return fmaf(w4.w, to_f(p[3 * ld]), acc);
  }
  float acc = 0.f;
  for (int j = 0; j < taps; ++j, p += ld) acc = fmaf(w[j], to_f(*p), acc);
  return acc;
}

// state [slots, taps - 1, st_ld], columns st_col0 .. st_col0 + C: after the step, row j holds the projected values of position
// seen + n - (taps - 1) + j.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ proj, long long ld, int col0, T* __restrict__ state, int st_ld, int st_col0,
                                         const int4* __restrict__ seq_desc, int C, int taps) {
  const int4 sd = seq_desc[blockIdx.y];
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  T* st = state + (static_cast<size_t>(sd.w) * (taps - 1)) * st_ld + st_col0 + c;
  const T* u = proj + static_cast<long long>(sd.x) * ld + col0 + c;
  for (int j = 0; j < taps - 1; ++j) {  // ascending: row j is rewritten after the only read of it (rows j + n are read, n >= 1)
    const int ii = sd.y - (taps - 1) + j;  // index among the new tokens of the position row j will hold
    if (ii >= 0) st[j * st_ld] = u[static_cast<long long>(ii) * ld];
    else if (sd.z + ii >= 0) st[j * st_ld] = st[(j + sd.y) * st_ld];
  }
}

// One block per token.  proj row = (... | q projection [H d] at q_col0 | k projection [G d] at k_col0 | ...).  Shared memory: (H + G) d
// convolved values + rot_dims sines / cosines.
template <typename T>
__global__ void window_qk_prepare_kernel(const T* __restrict__ proj, long long ld, int q_col0, int k_col0, const float* __restrict__ conv_q,
                                         const float* __restrict__ conv_k, const float* __restrict__ norm_q, const float* __restrict__ norm_k,
                                         const T* __restrict__ state, const int4* __restrict__ seq_desc, const int* __restrict__ tok_seq,
                                         const int* __restrict__ tok_pos, const int* __restrict__ block_table, int bt_stride, int block_size,
                                         T* __restrict__ cache, T* __restrict__ q_out, long long q_ld, const double* __restrict__ freq, int H,
                                         int G, int d, int taps, int rot_dims, float eps) {
  extern __shared__ float sm[];
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int nq = H * d, nk = G * d, C = nq + nk;
  float* y = sm;            // [C]: q channels then k channels
  float* cs = sm + C;       // [rot_dims / 2] cosines, then sines
  float* sn = cs + rot_dims / 2;
  const int seq = tok_seq[t], pos = tok_pos[t];
  const int4 sd = seq_desc[seq];
  const int i = t - sd.x;  // index among the sequence's new tokens
  const T* st = state + static_cast<size_t>(sd.w) * (taps - 1) * C;
  const T* u0 = proj + static_cast<long long>(sd.x) * ld;
  const int blk = block_table[static_cast<size_t>(seq) * bt_stride + pos / block_size];
  T* krow = cache + ((static_cast<size_t>(blk) * 2 + 0) * block_size + pos % block_size) * nk;
  T* vrow = cache + ((static_cast<size_t>(blk) * 2 + 1) * block_size + pos % block_size) * nk;
  float sq = 0.f, sk = 0.f;
  const bool inside = i >= taps - 1;  // (the same for the whole block)
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const bool is_q = c < nq;
    const int cc = is_q ? c : c - nq;
    const T* uc = u0 + (is_q ? q_col0 : k_col0) + cc;
    const float* wc = (is_q ? conv_q : conv_k) + static_cast<size_t>(cc) * taps;
    const float v = inside ? conv_inside(uc, ld, wc, taps, i) : conv_at(uc, ld, st + c, C, wc, taps, i, sd.z);
    y[c] = v;
    if (is_q) sq += v * v;
    else {
      sk += v * v;
      vrow[cc] = from_f<T>(v);  // the values are the keys as they leave the convolution
    }
  }
  for (int f = threadIdx.x; f < rot_dims / 2; f += blockDim.x) {
    // the angle is formed and brought into [-pi, pi] in double (a position in the thousands times a frequency near one loses the low
    // bits of a float); sine and cosine of the reduced angle are then taken in single precision
    const double ang = static_cast<double>(pos) * freq[f];
    const float red_ang = static_cast<float>(ang - 6.283185307179586476925 * rint(ang * 0.15915494309189533577));
    float s, c;
    sincosf(red_ang, &s, &c);
    cs[f] = c;
    sn[f] = s;
  }
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);  // (the barriers inside also publish y, cs, sn)
  const float inv_q = 1.f / sqrtf(sq / static_cast<float>(nq) + eps), inv_k = 1.f / sqrtf(sk / static_cast<float>(nk) + eps);
  T* qrow = q_out + static_cast<long long>(t) * q_ld;
  const int hp = (d + 1) / 2;  // pairs (2p, 2p + 1) per head; the last one of an odd head size has no second entry
  const int lg_hp = (hp & (hp - 1)) == 0 ? __ffs(hp) - 1 : -1;
  for (int pr = threadIdx.x; pr < (H + G) * hp; pr += blockDim.x) {
    const int head = lg_hp >= 0 ? pr >> lg_hp : pr / hp, within = 2 * (pr - head * hp);
    const int c = head * d + within;
    const bool is_q = c < nq, two = within + 1 < d;
    const int cc = is_q ? c : c - nq;
    const float inv = is_q ? inv_q : inv_k;
    const float* nw = is_q ? norm_q : norm_k;
    float a = y[c] * inv * nw[cc], b = two ? y[c + 1] * inv * nw[cc + 1] : 0.f;
    if (within + 1 < rot_dims) {
      const float co = cs[within >> 1], si = sn[within >> 1];
      const float ra = a * co - b * si, rb = b * co + a * si;
      a = ra;
      b = rb;
    }
    T* dst = is_q ? qrow : krow;
    dst[cc] = from_f<T>(a);
    if (two) dst[cc + 1] = from_f<T>(b);
  }
}

// ------------------------------------------------------------------------------------------------- sliding-window attention
// One block per (token, query head).  Visible keys of a query at position p: [0, min(keep, p + 1)) and [max(p - window + 1, that), p].
// They are walked in chunks of WA_CHUNK with a running maximum / sum (fp32).  cache [blocks, 2, block_size, G, d]: plane 0 keys, 1 values.
constexpr int WA_CHUNK = 256, WA_THREADS = 128;
template <typename T>
__global__ void __launch_bounds__(WA_THREADS)
window_attention_kernel(const T* __restrict__ q, long long q_ld, const T* __restrict__ cache, const int* __restrict__ tok_seq,
                        const int* __restrict__ tok_pos, const int* __restrict__ block_table, int bt_stride, int block_size, T* __restrict__ out,
                        long long out_ld, int H, int G, int d, int window, int keep, float scale, float out_scale) {
  extern __shared__ float sm[];
  __shared__ float red[33];
  __shared__ float sc[WA_CHUNK];
  __shared__ int key_row[WA_CHUNK];  // row of the key in the cache: block * 2 * block_size + slot (plane 0)
  const int t = blockIdx.x, h = blockIdx.y, g = h / (H / G);
  const int seq = tok_seq[t], pos = tok_pos[t];
  float* qs = sm;  // [d]
  float* acc = sm + d;  // [d]
  for (int c = threadIdx.x; c < d; c += WA_THREADS) {
    qs[c] = to_f(q[static_cast<long long>(t) * q_ld + h * d + c]) * scale;
    acc[c] = 0.f;
  }
  const int kept = min(keep, pos + 1);
  const int b0 = max(max(0, pos - window + 1), kept);
  const int n = kept + (pos - b0 + 1);
  const int* bt = block_table + static_cast<size_t>(seq) * bt_stride;
  const size_t row_elems = static_cast<size_t>(G) * d, plane = static_cast<size_t>(block_size) * row_elems;
  float m_run = -INFINITY, l_run = 0.f;
  __syncthreads();
  for (int x0 = 0; x0 < n; x0 += WA_CHUNK) {
    const int cn = min(WA_CHUNK, n - x0);
    float mx = -INFINITY;
    for (int x = threadIdx.x; x < cn; x += WA_THREADS) {
      const int j = (x0 + x) < kept ? (x0 + x) : b0 + (x0 + x - kept);
      const int row = bt[j / block_size] * 2 * block_size + j % block_size;
      key_row[x] = row;
      const T* kr = cache + static_cast<size_t>(row) * row_elems + g * d;
      float s = 0.f;
      for (int c = 0; c < d; ++c) s = fmaf(qs[c], to_f(kr[c]), s);
      sc[x] = s;
      mx = fmaxf(mx, s);
    }
    mx = block_max(mx, red);
    const float m_new = fmaxf(m_run, mx);
    float ls = 0.f;
    for (int x = threadIdx.x; x < cn; x += WA_THREADS) {
      const float p = expf(sc[x] - m_new);
      sc[x] = p;
      ls += p;
    }
    ls = block_sum(ls, red);
    const float corr = expf(m_run - m_new);  // 0 for the first chunk (m_run = -inf)
    l_run = l_run * corr + ls;
    m_run = m_new;
    for (int c = threadIdx.x; c < d; c += WA_THREADS) {
      float a = acc[c] * corr;
      for (int x = 0; x < cn; ++x) a = fmaf(sc[x], to_f(cache[static_cast<size_t>(key_row[x]) * row_elems + plane + g * d + c]), a);
      acc[c] = a;
    }
    __syncthreads();
  }
  const float inv = out_scale / l_run;
  for (int c = threadIdx.x; c < d; c += WA_THREADS) out[static_cast<long long>(t) * out_ld + h * d + c] = from_f<T>(acc[c] * inv);
}

// --------------------------------------------------------------------------------------------------------- recurrent scans
// A block owns SCAN_THREADS / R columns of the d x dv state of one (sequence, head) and walks the sequence's new tokens in order (the
// columns of these recurrences do not interact).  Thread (col, r) -- r varying fastest, R a power of two <= 32 -- holds rows r RPT ..
// r RPT + RPT - 1 of its column in registers (its q / k values are consecutive in shared memory: 16-byte loads); sums over rows are finished by a butterfly over the R lanes.  The state is kept in global memory in thread
// order ([column tile][column of the thread][RPT][SCAN_THREADS], opaque to everything but these kernels, coalesced).  Inputs travel in chunks of `ch` tokens
// (a power of two <= 16 with at most SCAN_PF * SCAN_THREADS staged values per array): while a chunk is consumed from shared memory the
// next one is already on its way in registers, so the walk never waits for global memory.
constexpr int SCAN_THREADS = 256, SCAN_PF = 8, SCAN_CPT = 2;  // SCAN_CPT: columns of the state per thread (staged q / k rows serve both)

// Where row i of a staged q / k / decay vector sits in its shared-memory row: thread r reads its rows r RPT .. r RPT + RPT - 1 four at a
// time, and the four-row groups of the R lanes lie side by side ([group][lane][4]) so that one 16-byte load of the R lanes covers a
// contiguous 16 R bytes (no bank conflicts; rows laid out plainly put lanes 32 bytes apart, a 4-way conflict).
template <int RPT, int R>
__device__ __forceinline__ int staged_pos(int i) {
  const int r = i / RPT, ii = i % RPT;
  return (ii >> 2) * (R * 4) + r * 4 + (ii & 3);
}

template <int R>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
  for (int o = R / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// q / k at columns q_col0 / k_col0 of proj (H x d each), v at v_col0 (H x dv); gates: pre-activations [T, 2 H] fp32 (input gate | forget
// gate) without their biases.  state_S [slots, H, tiles * RPT * SCAN_THREADS], state_n [slots, H, d], state_m [slots, H].  out fp32
// [T, H dv].  The block has one warp more than SCAN_THREADS: it walks the gate recurrence (m, the two decay factors and exp(-m) of every
// token, three exponentials each) of the NEXT chunk while the others consume the current one.
template <typename T, int RPT, int R>
__global__ void __launch_bounds__(SCAN_THREADS + 32, RPT <= 16 ? 2 : 1)
matrix_memory_scan_kernel(const T* __restrict__ proj, long long ld, int q_col0, int k_col0, int v_col0, const float* __restrict__ gates,
                          const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap, const int4* __restrict__ seq_desc,
                          float* __restrict__ state_S, float* __restrict__ state_n, float* __restrict__ state_m, float* __restrict__ out, int H, int d,
                          int dv, int ch) {
  extern __shared__ __align__(16) float sm[];
  constexpr int nthr = SCAN_THREADS, CB = nthr / R, CBT = SCAN_CPT * CB, DP = R * RPT;  // DP: a staged q / k row, padded with zeros past d
  const int4 sd = seq_desc[blockIdx.x];
  const int h = blockIdx.y, tid = threadIdx.x;
  const bool gate_warp = tid >= nthr;
  const int col0 = blockIdx.z * CBT, lc = (tid % nthr) / R, r = tid % R, col = col0 + lc;  // the thread's columns: col and col + CB
  const bool live = !gate_warp && col < dv, live2 = !gate_warp && col + CB < dv;
  const int ncol = min(CBT, dv - col0);
  // per buffer: q [ch DP] | k [ch DP] | v [ch CBT] | a [ch] | b [ch] | e [ch] | pad [ch]; then the gate warp's scratch (2 ch)
  const int buf = 2 * ch * DP + ch * CBT + 4 * ch;  // (a multiple of 4 floats: rows are read 16 bytes at a time)
  float* tmp_g = sm + 2 * buf;
  if (d != DP)
    for (int x = tid; x < 2 * buf; x += nthr + 32) sm[x] = 0.f;  // the padding of the rows stays zero from here on
  float S[RPT], S2[RPT], nn[RPT];
  float* gS = state_S + ((static_cast<size_t>(sd.w) * H + h) * gridDim.z + blockIdx.z) * SCAN_CPT * RPT * nthr;
  float* gn = state_n + (static_cast<size_t>(sd.w) * H + h) * d;
  float m = 0.f;  // followed by the gate warp only
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) S[ii] = S2[ii] = nn[ii] = 0.f;
  if (sd.z > 0) {
    if (!gate_warp) {
#pragma unroll
      for (int ii = 0; ii < RPT; ++ii) {
        S[ii] = gS[ii * nthr + tid];
        S2[ii] = gS[(RPT + ii) * nthr + tid];
        const int i = r * RPT + ii;
        nn[ii] = i < d ? gn[i] : 0.f;
      }
    } else {
      m = state_m[sd.w * H + h];
    }
  }
  const float qscale = 1.f / sqrtf(static_cast<float>(d));
  // staged value x = tid + e SCAN_THREADS of a chunk is (token x / d, channel x % d) of q and k and (token x / ncol, column x % ncol) of
  // v: shifts and masks when the sizes are powers of two, divisions otherwise
  const int lg_d = (d & (d - 1)) == 0 ? __ffs(d) - 1 : -1, lg_c = (ncol & (ncol - 1)) == 0 ? __ffs(ncol) - 1 : -1;
  auto split_qk = [&](int x, int& tok, int& c) {
    if (lg_d >= 0) { tok = x >> lg_d; c = x & (d - 1); } else { tok = x / d; c = x - tok * d; }
  };
  auto split_v = [&](int x, int& tok, int& c) {
    if (lg_c >= 0) { tok = x >> lg_c; c = x & (ncol - 1); } else { tok = x / ncol; c = x - tok * ncol; }
  };
  T pq[SCAN_PF], pk[SCAN_PF], pv[SCAN_PF];
  // the three stages of moving a chunk: global -> registers, registers -> shared buffer, gate recurrence -> shared buffer
  auto fetch = [&](int t0) {
    if (gate_warp) return;
    const int cn = min(ch, sd.y - t0);
    const T* base = proj + static_cast<long long>(sd.x + t0) * ld + h * d;
    const T* vbase = proj + static_cast<long long>(sd.x + t0) * ld + v_col0 + h * dv + col0;
#pragma unroll
    for (int e = 0; e < SCAN_PF; ++e) {
      int tok, c;
      split_qk(tid + e * nthr, tok, c);
      if (tok < cn) {
        pq[e] = base[tok * ld + c + q_col0];
        pk[e] = base[tok * ld + c + k_col0];
      }
      split_v(tid + e * nthr, tok, c);
      if (tok < cn) pv[e] = vbase[tok * ld + c];
    }
  };
  auto stage = [&](int t0, float* bq) {
    const int cn = min(ch, sd.y - t0);
    float* bk = bq + ch * DP;
    float* bv = bk + ch * DP;
    if (!gate_warp) {
#pragma unroll
      for (int e = 0; e < SCAN_PF; ++e) {
        int tok, c;
        split_qk(tid + e * nthr, tok, c);
        if (tok < cn) {
          bq[tok * DP + staged_pos<RPT, R>(c)] = to_f(pq[e]) * qscale;
          bk[tok * DP + staged_pos<RPT, R>(c)] = to_f(pk[e]);
        }
        split_v(tid + e * nthr, tok, c);
        if (tok < cn) bv[tok * CBT + c] = to_f(pv[e]);
      }
      return;
    }
    float* ga = bv + ch * CBT;
    float* gb = ga + ch;
    float* ge = gb + ch;
    const int lane = tid - nthr;
    if (lane < cn) {
      const float* gr = gates + static_cast<size_t>(sd.x + t0 + lane) * 2 * H;
      tmp_g[lane] = cap * tanhf((gr[h] + bias_i[h]) / cap);
      tmp_g[ch + lane] = logsigmoidf_(cap * tanhf((gr[H + h] + bias_f[h]) / cap));
    }
    __syncwarp();
    for (int x = 0; x < cn; ++x) {  // every lane walks the recurrence (m stays warp-uniform); lane 0 writes
      const float ig = tmp_g[x], fg = tmp_g[ch + x];
      const float m_new = fmaxf(fg + m, ig);
      const float a = expf(fg + m - m_new), b2 = expf(ig - m_new), e2 = expf(-m_new);
      m = m_new;
      if (lane == 0) {
        ga[x] = a;
        gb[x] = b2;
        ge[x] = e2;
      }
    }
    __syncwarp();
  };
  __syncthreads();  // the zeros are in place
  fetch(0);
  stage(0, sm);
  __syncthreads();
  int cur = 0;
  for (int t0 = 0; t0 < sd.y; t0 += ch, cur ^= 1) {
    const int cn = min(ch, sd.y - t0);
    const bool more = t0 + ch < sd.y;
    if (more) fetch(t0 + ch);
    if (!gate_warp) {
      const float* bq = sm + cur * buf + r * 4;
      const float* bk = bq + ch * DP;
      const float* bv = sm + cur * buf + 2 * ch * DP;
      const float* ga = bv + ch * CBT;
      const float* gb = ga + ch;
      const float* ge = gb + ch;
      float* orow = out + static_cast<size_t>(sd.x + t0) * H * dv + h * dv + col;
#pragma unroll 2
      for (int x = 0; x < cn; ++x) {
        const float a = ga[x], b2 = gb[x];
        const float v = live ? bv[x * CBT + lc] : 0.f, v2 = live2 ? bv[x * CBT + CB + lc] : 0.f;
        float po = 0.f, po2 = 0.f, pn = 0.f;
#pragma unroll
        for (int i4 = 0; i4 < RPT; i4 += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(bk + x * DP + i4 * R), q4 = *reinterpret_cast<const float4*>(bq + x * DP + i4 * R);
          const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float bk2 = b2 * kk[j];
            S[i4 + j] = fmaf(a, S[i4 + j], bk2 * v);
            S2[i4 + j] = fmaf(a, S2[i4 + j], bk2 * v2);
            nn[i4 + j] = fmaf(a, nn[i4 + j], bk2);
            po = fmaf(S[i4 + j], qq[j], po);
            po2 = fmaf(S2[i4 + j], qq[j], po2);
            pn = fmaf(nn[i4 + j], qq[j], pn);
          }
        }
        po = lanes_sum<R>(po);
        po2 = lanes_sum<R>(po2);
        pn = lanes_sum<R>(pn);
        const float den = fmaxf(fabsf(pn), ge[x]) + 1e-6f;
        if (live && r == 0) orow[static_cast<size_t>(x) * H * dv] = po / den;
        if (live2 && r == 0) orow[static_cast<size_t>(x) * H * dv + CB] = po2 / den;
      }
    }
    if (more) stage(t0 + ch, sm + (cur ^ 1) * buf);
    __syncthreads();
  }
  if (!gate_warp) {
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) {
      gS[ii * nthr + tid] = S[ii];
      gS[(RPT + ii) * nthr + tid] = S2[ii];
      const int i = r * RPT + ii;
      if (col == 0 && i < d) gn[i] = nn[ii];  // every column tile carries the same n; the first one keeps it
    }
  } else if (tid == nthr && blockIdx.z == 0) {
    state_m[sd.w * H + h] = m;
  }
}

// qn / kn fp32 [T, G d] (unit length; q already times d^-1/2), v fp32 [T, H dv], beta fp32 [T, H], decay fp32 [T, H d] (both finished by
// delta_prepare).  Head h reads q / k head h / (H / G).  out fp32 [T, H dv].
template <int RPT, int R>
__global__ void __launch_bounds__(SCAN_THREADS, RPT <= 16 ? 2 : 1)
delta_rule_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ v, const float* __restrict__ beta,
                       const float* __restrict__ decay, const int4* __restrict__ seq_desc, float* __restrict__ state_S, float* __restrict__ out,
                       int H, int G, int d, int dv, int ch) {
  extern __shared__ __align__(16) float sm[];
  constexpr int nthr = SCAN_THREADS, CB = nthr / R, CBT = SCAN_CPT * CB, DP = R * RPT;
  const int4 sd = seq_desc[blockIdx.x];
  const int h = blockIdx.y, g = h / (H / G), tid = threadIdx.x;
  const int col0 = blockIdx.z * CBT, lc = tid / R, r = tid % R, col = col0 + lc;  // the thread's columns: col and col + CB
  const bool live = col < dv, live2 = col + CB < dv;
  const int ncol = min(CBT, dv - col0);
  const int buf = 3 * ch * DP + ch * CBT + ((ch + 3) & ~3);  // q | k | decay | v | beta (a multiple of 4 floats)
  if (d != DP)
    for (int x = tid; x < 2 * buf; x += nthr) sm[x] = 0.f;  // the padding of the rows stays zero from here on
  float S[RPT], S2[RPT];
  float* gS = state_S + ((static_cast<size_t>(sd.w) * H + h) * gridDim.z + blockIdx.z) * SCAN_CPT * RPT * nthr;
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    S[ii] = sd.z > 0 ? gS[ii * nthr + tid] : 0.f;
    S2[ii] = sd.z > 0 ? gS[(RPT + ii) * nthr + tid] : 0.f;
  }
  const int lg_d = (d & (d - 1)) == 0 ? __ffs(d) - 1 : -1, lg_c = (ncol & (ncol - 1)) == 0 ? __ffs(ncol) - 1 : -1;
  auto split_qk = [&](int x, int& tok, int& c) {
    if (lg_d >= 0) { tok = x >> lg_d; c = x & (d - 1); } else { tok = x / d; c = x - tok * d; }
  };
  auto split_v = [&](int x, int& tok, int& c) {
    if (lg_c >= 0) { tok = x >> lg_c; c = x & (ncol - 1); } else { tok = x / ncol; c = x - tok * ncol; }
  };
  float pq[SCAN_PF], pk[SCAN_PF], pg[SCAN_PF], pv[SCAN_PF], pb = 0.f;
  auto fetch = [&](int t0) {
    const int cn = min(ch, sd.y - t0);
    const size_t row0 = static_cast<size_t>(sd.x + t0);
    const float *q0 = qn + row0 * G * d + g * d, *k0 = kn + row0 * G * d + g * d, *g0 = decay + row0 * H * d + h * d,
                *v0 = v + row0 * H * dv + h * dv + col0;
#pragma unroll
    for (int e = 0; e < SCAN_PF; ++e) {
      int tok, c;
      split_qk(tid + e * nthr, tok, c);
      if (tok < cn) {
        pq[e] = q0[tok * G * d + c];
        pk[e] = k0[tok * G * d + c];
        pg[e] = g0[tok * H * d + c];
      }
      split_v(tid + e * nthr, tok, c);
      if (tok < cn) pv[e] = v0[tok * H * dv + c];
    }
    if (tid < cn) pb = beta[(row0 + tid) * H + h];
  };
  auto stage = [&](int t0, float* bq) {
    const int cn = min(ch, sd.y - t0);
    float* bk = bq + ch * DP;
    float* bg = bk + ch * DP;
    float* bv = bg + ch * DP;
    float* bb = bv + ch * CBT;
#pragma unroll
    for (int e = 0; e < SCAN_PF; ++e) {
      int tok, c;
      split_qk(tid + e * nthr, tok, c);
      if (tok < cn) {
        const int pos = tok * DP + staged_pos<RPT, R>(c);
        bq[pos] = pq[e];
        bk[pos] = pk[e];
        bg[pos] = pg[e];
      }
      split_v(tid + e * nthr, tok, c);
      if (tok < cn) bv[tok * CBT + c] = pv[e];
    }
    if (tid < cn) bb[tid] = pb;
  };
  __syncthreads();  // the zeros are in place
  fetch(0);
  stage(0, sm);
  __syncthreads();
  int cur = 0;
  for (int t0 = 0; t0 < sd.y; t0 += ch, cur ^= 1) {
    const int cn = min(ch, sd.y - t0);
    const bool more = t0 + ch < sd.y;
    if (more) fetch(t0 + ch);
    const float* bq = sm + cur * buf + r * 4;
    const float* bk = bq + ch * DP;
    const float* bg = bk + ch * DP;
    const float* bv = sm + cur * buf + 3 * ch * DP;
    const float* bb = bv + ch * CBT;
    float* orow = out + static_cast<size_t>(sd.x + t0) * H * dv + h * dv + col;
    for (int x = 0; x < cn; ++x) {
      float ps = 0.f, ps2 = 0.f;
      float kk[RPT];
#pragma unroll
      for (int i4 = 0; i4 < RPT; i4 += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(bk + x * DP + i4 * R), g4 = *reinterpret_cast<const float4*>(bg + x * DP + i4 * R);
        const float gg[4] = {g4.x, g4.y, g4.z, g4.w};  // padded rows: decay 0 on a state of 0
        kk[i4] = k4.x; kk[i4 + 1] = k4.y; kk[i4 + 2] = k4.z; kk[i4 + 3] = k4.w;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          S[i4 + j] *= gg[j];
          S2[i4 + j] *= gg[j];
          ps = fmaf(S[i4 + j], kk[i4 + j], ps);
          ps2 = fmaf(S2[i4 + j], kk[i4 + j], ps2);
        }
      }
      ps = lanes_sum<R>(ps);
      ps2 = lanes_sum<R>(ps2);
      const float bx = bb[x];
      const float u = live ? bx * (bv[x * CBT + lc] - ps) : 0.f, u2 = live2 ? bx * (bv[x * CBT + CB + lc] - ps2) : 0.f;
      float po = 0.f, po2 = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < RPT; i4 += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(bq + x * DP + i4 * R);
        const float qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          S[i4 + j] = fmaf(kk[i4 + j], u, S[i4 + j]);
          S2[i4 + j] = fmaf(kk[i4 + j], u2, S2[i4 + j]);
          po = fmaf(S[i4 + j], qq[j], po);
          po2 = fmaf(S2[i4 + j], qq[j], po2);
        }
      }
      po = lanes_sum<R>(po);
      po2 = lanes_sum<R>(po2);
      if (live && r == 0) orow[static_cast<size_t>(x) * H * dv] = po;
      if (live2 && r == 0) orow[static_cast<size_t>(x) * H * dv + CB] = po2;
    }
    if (more) stage(t0 + ch, sm + (cur ^ 1) * buf);
    __syncthreads();
  }
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    gS[ii * nthr + tid] = S[ii];
    gS[(RPT + ii) * nthr + tid] = S2[ii];
  }
}

// Linear attention whose forget gate also decides what is written (no key projection): per head, with the fused projection proj [T, ld]
// holding the query pre-activations [H d] at q_col0, the gate pre-activations [H d] at f_col0 and the values [H dv] at v_col0,
//   q = silu(q_pre),  f = lower + (1 - lower) sigmoid(f_pre + f_bias),  S <- diag(f) S + (1 - f) v^T,  o = S^T q.
// The activations are formed in fp32 while a chunk is fetched; state layout, chunking and the thread mapping are those of the other scans.
template <typename T, int RPT, int R>
__global__ void __launch_bounds__(SCAN_THREADS, RPT <= 16 ? 2 : 1)
tied_gate_scan_kernel(const T* __restrict__ proj, long long ld, int q_col0, int f_col0, int v_col0, const float* __restrict__ f_bias,
                      const float* __restrict__ lower, const int4* __restrict__ seq_desc, float* __restrict__ state_S, float* __restrict__ out,
                      int H, int d, int dv, int ch) {
  extern __shared__ __align__(16) float sm[];
  constexpr int nthr = SCAN_THREADS, CB = nthr / R, CBT = SCAN_CPT * CB, DP = R * RPT;
  const int4 sd = seq_desc[blockIdx.x];
  const int h = blockIdx.y, tid = threadIdx.x;
  const int col0 = blockIdx.z * CBT, lc = tid / R, r = tid % R, col = col0 + lc;  // the thread's columns: col and col + CB
  const bool live = col < dv, live2 = col + CB < dv;
  const int ncol = min(CBT, dv - col0);
  const int buf = 2 * ch * DP + ch * CBT;  // q | f | v
  if (d != DP)
    for (int x = tid; x < 2 * buf; x += nthr) sm[x] = 0.f;  // padded rows: q = 0 (they never reach the output), f = 0
  float S[RPT], S2[RPT];
  float* gS = state_S + ((static_cast<size_t>(sd.w) * H + h) * gridDim.z + blockIdx.z) * SCAN_CPT * RPT * nthr;
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    S[ii] = sd.z > 0 ? gS[ii * nthr + tid] : 0.f;
    S2[ii] = sd.z > 0 ? gS[(RPT + ii) * nthr + tid] : 0.f;
  }
  const int lg_d = (d & (d - 1)) == 0 ? __ffs(d) - 1 : -1, lg_c = (ncol & (ncol - 1)) == 0 ? __ffs(ncol) - 1 : -1;
  auto split_qk = [&](int x, int& tok, int& c) {
    if (lg_d >= 0) { tok = x >> lg_d; c = x & (d - 1); } else { tok = x / d; c = x - tok * d; }
  };
  auto split_v = [&](int x, int& tok, int& c) {
    if (lg_c >= 0) { tok = x >> lg_c; c = x & (ncol - 1); } else { tok = x / ncol; c = x - tok * ncol; }
  };
  // fetch() only issues the loads of the next chunk (raw values, no use: the walk below runs while they are in flight); stage() turns them
  // into q and f after the walk.  A thread's element e is the same channel in every chunk, so its bias and lower bound are loaded once.
  T rq[SCAN_PF], rf[SCAN_PF], rv[SCAN_PF];
  float e_bias[SCAN_PF], e_low[SCAN_PF];
#pragma unroll
  for (int e = 0; e < SCAN_PF; ++e) {
    int tok, c;
    split_qk(tid + e * nthr, tok, c);
    e_bias[e] = tok < ch ? f_bias[h * d + c] : 0.f;
    e_low[e] = tok < ch ? lower[h * d + c] : 0.f;
  }
  auto fetch = [&](int t0) {
    const int cn = min(ch, sd.y - t0);
    const T* row0 = proj + static_cast<size_t>(sd.x + t0) * ld;
#pragma unroll
    for (int e = 0; e < SCAN_PF; ++e) {
      int tok, c;
      split_qk(tid + e * nthr, tok, c);
      if (tok < cn) {
        const T* pr = row0 + static_cast<size_t>(tok) * ld;
        rq[e] = pr[q_col0 + h * d + c];
        rf[e] = pr[f_col0 + h * d + c];
      }
      split_v(tid + e * nthr, tok, c);
      if (tok < cn) rv[e] = row0[static_cast<size_t>(tok) * ld + v_col0 + h * dv + col0 + c];
    }
  };
  auto stage = [&](int t0, float* bq) {
    const int cn = min(ch, sd.y - t0);
    float* bf = bq + ch * DP;
    float* bv = bf + ch * DP;
#pragma unroll
    for (int e = 0; e < SCAN_PF; ++e) {
      int tok, c;
      split_qk(tid + e * nthr, tok, c);
      if (tok < cn) {
        const int pos = tok * DP + staged_pos<RPT, R>(c);
        // the query's silu is a projection's activation (fast exponential and division); the gate enters the recurrence: a full-precision
        // exponential and a correctly rounded reciprocal (a true division would cost as much as the walk itself here)
        const float zq = to_f(rq[e]);
        bq[pos] = __fdividef(zq, 1.f + __expf(-zq));
        bf[pos] = e_low[e] + (1.f - e_low[e]) * __frcp_rn(1.f + expf(-(to_f(rf[e]) + e_bias[e])));
      }
      split_v(tid + e * nthr, tok, c);
      if (tok < cn) bv[tok * CBT + c] = to_f(rv[e]);
    }
  };
  __syncthreads();  // the zeros are in place
  fetch(0);
  stage(0, sm);
  __syncthreads();
  int cur = 0;
  for (int t0 = 0; t0 < sd.y; t0 += ch, cur ^= 1) {
    const int cn = min(ch, sd.y - t0);
    const bool more = t0 + ch < sd.y;
    if (more) fetch(t0 + ch);
    const float* bq = sm + cur * buf + r * 4;
    const float* bf = bq + ch * DP;
    const float* bv = sm + cur * buf + 2 * ch * DP;
    float* orow = out + static_cast<size_t>(sd.x + t0) * H * dv + h * dv + col;
    for (int x = 0; x < cn; ++x) {
      const float v1 = live ? bv[x * CBT + lc] : 0.f, v2 = live2 ? bv[x * CBT + CB + lc] : 0.f;
      float po = 0.f, po2 = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < RPT; i4 += 4) {
        const float4 f4 = *reinterpret_cast<const float4*>(bf + x * DP + i4 * R), q4 = *reinterpret_cast<const float4*>(bq + x * DP + i4 * R);
        const float ff[4] = {f4.x, f4.y, f4.z, f4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float w = 1.f - ff[j];
          S[i4 + j] = fmaf(ff[j], S[i4 + j], w * v1);
          S2[i4 + j] = fmaf(ff[j], S2[i4 + j], w * v2);
          po = fmaf(S[i4 + j], qq[j], po);
          po2 = fmaf(S2[i4 + j], qq[j], po2);
        }
      }
      po = lanes_sum<R>(po);
      po2 = lanes_sum<R>(po2);
      if (live && r == 0) orow[static_cast<size_t>(x) * H * dv] = po;
      if (live2 && r == 0) orow[static_cast<size_t>(x) * H * dv + CB] = po2;
    }
    if (more) stage(t0 + ch, sm + (cur ^ 1) * buf);
    __syncthreads();
  }
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    gS[ii * nthr + tid] = S[ii];
    gS[(RPT + ii) * nthr + tid] = S2[ii];
  }
}

// One block per token.  proj row holds the q [G d], k [G d] and v [H dv] projections at q_col0 / k_col0 / v_col0; the kept rows of the
// sequence are [taps - 1, 2 G d + H dv] (q | k | v channels).  Each goes through its short convolution and silu; q and k are then made unit
// vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times d^-1/2: a warp takes a head at a time, so the sums need no atomics.  The same
// pass finishes what else the scan reads per token: a_pre [T, H d] becomes the decay exp(-exp(A_log) softplus(a_pre + dt_bias)) and
// beta_pre [T, H] becomes sigmoid(beta_pre), both in place.  Outputs fp32.
template <typename T>
__global__ void delta_prepare_kernel(const T* __restrict__ proj, long long ld, int q_col0, int k_col0, int v_col0, const float* __restrict__ conv_q,
                                     const float* __restrict__ conv_k, const float* __restrict__ conv_v, const T* __restrict__ state,
                                     const int4* __restrict__ seq_desc, const int* __restrict__ tok_seq, float* __restrict__ qn,
                                     float* __restrict__ kn, float* __restrict__ vo, float* __restrict__ a_pre, float* __restrict__ beta_pre,
                                     const float* __restrict__ A_log, const float* __restrict__ dt_bias, int G, int H, int d, int dv, int taps) {
  extern __shared__ float sm[];
  const int t = blockIdx.x;
  const int nqk = G * d, nv = H * dv, C = 2 * nqk + nv;
  float* y = sm;  // [2 G d]: q then k
  const int4 sd = seq_desc[tok_seq[t]];
  const int i = t - sd.x;
  const T* st = state + static_cast<size_t>(sd.w) * (taps - 1) * C;
  const T* u0 = proj + static_cast<long long>(sd.x) * ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float qscale = 1.f / sqrtf(static_cast<float>(d));
  const bool inside = i >= taps - 1;  // (the same for the whole block)
  for (int hh = warp; hh < 2 * G; hh += nw) {  // head hh of (q heads | k heads)
    const int which = hh < G ? 0 : 1;
    const int c0 = hh * d;  // first channel of the head among the 2 G d
    const int col0 = (which ? k_col0 : q_col0) + (hh - which * G) * d;
    const float* w = (which ? conv_k : conv_q) + static_cast<size_t>(hh - which * G) * d * taps;
    float ss = 0.f;
    for (int c = lane; c < d; c += 32) {
      const float cv = inside ? conv_inside(u0 + col0 + c, ld, w + static_cast<size_t>(c) * taps, taps, i)
                              : conv_at(u0 + col0 + c, ld, st + c0 + c, C, w + static_cast<size_t>(c) * taps, taps, i, sd.z);
      const float val = siluf_(cv);
      y[c0 + c] = val;
      ss += val * val;
    }
    ss = warp_sum(ss);
    const float inv = (which ? 1.f : qscale) / sqrtf(ss + 1e-6f);
    float* dst = (which ? kn : qn) + static_cast<size_t>(t) * nqk + (hh - which * G) * d;
    for (int c = lane; c < d; c += 32) dst[c] = y[c0 + c] * inv;  // each lane re-reads what it wrote
  }
  for (int c = threadIdx.x; c < nv; c += blockDim.x) {
    const float cv = inside ? conv_inside(u0 + v_col0 + c, ld, conv_v + static_cast<size_t>(c) * taps, taps, i)
                            : conv_at(u0 + v_col0 + c, ld, st + 2 * nqk + c, C, conv_v + static_cast<size_t>(c) * taps, taps, i, sd.z);
    vo[static_cast<size_t>(t) * nv + c] = siluf_(cv);
  }
  for (int hh = warp; hh < H; hh += nw) {  // a warp per head: the head's rate once, no division per channel
    const float rate = expf(A_log[hh]);
    float* a = a_pre + static_cast<size_t>(t) * H * d + hh * d;
    for (int c = lane; c < d; c += 32) a[c] = expf(-rate * softplusf_(a[c] + dt_bias[hh * d + c]));
  }
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float* bp = beta_pre + static_cast<size_t>(t) * H + c;
    *bp = sigmoidf_(*bp);
  }
}

// One warp per (token, head): out[t, col0 + h dv + c] = o / sqrt(mean_c(o^2) + eps) * w[h * w_stride + c] * sigmoid(gate[t, h dv + c]) * mult
// (gate null: no gate factor)
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_stride, const T* __restrict__ gate,
                                      long long gate_ld, T* __restrict__ out, long long out_ld, int n_tokens, int H, int dv, float eps, float mult) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (gw >= n_tokens * H) return;
  const int t = gw / H, h = gw % H;
  const float* orow = o + (static_cast<size_t>(t) * H + h) * dv;
  float s = 0.f;
  for (int c = lane; c < dv; c += 32) s += orow[c] * orow[c];
  s = warp_sum(s);
  const float inv = 1.f / sqrtf(s / static_cast<float>(dv) + eps);
  const T* gr = gate ? gate + static_cast<long long>(t) * gate_ld + h * dv : nullptr;
  T* dst = out + static_cast<long long>(t) * out_ld + h * dv;
  for (int c = lane; c < dv; c += 32) dst[c] = from_f<T>(orow[c] * inv * w[h * w_stride + c] * (gr ? sigmoidf_(to_f(gr[c])) : 1.f) * mult);
}

}  // namespace recur
}  // namespace dsb

using namespace dsb;
using namespace dsb::recur;

// Lanes per column (R), rows per thread (RPT, rounded up to 8 / 16 / 32 / 64), column tiles of a d x dv state and tokens per staged
// chunk: about 8 rows per thread (a short dependent chain per token); a block of SCAN_THREADS threads then covers SCAN_THREADS / R columns.
static bool scan_shape(int d, int dv, int* R, int* RPT, int* tiles, int* chunk = nullptr) {
  if (d < 1 || dv < 1 || d > SCAN_PF * SCAN_THREADS) return false;
  static const int rows_target = [] { const char* e = getenv("DSB200_SCAN_ROWS"); const int v = e ? atoi(e) : 0; return v >= 4 && v <= 64 ? v : 8; }();
  int r = 1;
  while (r < 32 && (d + r - 1) / r > rows_target) r <<= 1;
  const int need = (d + r - 1) / r;
  int rpt = 8;
  while (rpt < need) rpt <<= 1;
  const int cols = SCAN_CPT * (SCAN_THREADS / r);  // columns per block
  *R = r;
  *RPT = rpt;
  *tiles = (dv + cols - 1) / cols;
  if (chunk) {
    int ch = 16;
    while (ch > 1 && (ch * d > SCAN_PF * SCAN_THREADS || ch * cols > SCAN_PF * SCAN_THREADS)) ch >>= 1;
    *chunk = ch;
  }
  return rpt <= 64;
}

// Floats of state_S per (slot, head) for a d x dv recurrent state (the layout is the scan kernels' own).
DSB_EXPORT long long dsb200_scan_state_floats(int d, int dv) {
  int R, RPT, tiles;
  if (!scan_shape(d, dv, &R, &RPT, &tiles)) return -1;
  return static_cast<long long>(tiles) * SCAN_CPT * RPT * SCAN_THREADS;
}

#define SCAN_DISPATCH(RPTv, Rv, CALL) \
  if (RPT == RPTv && R == Rv) { CALL(RPTv, Rv); launched = true; }
#define SCAN_DISPATCH_ROW(RPTv, CALL)                                                                                         \
  SCAN_DISPATCH(RPTv, 1, CALL) SCAN_DISPATCH(RPTv, 2, CALL) SCAN_DISPATCH(RPTv, 4, CALL) SCAN_DISPATCH(RPTv, 8, CALL)         \
  SCAN_DISPATCH(RPTv, 16, CALL) SCAN_DISPATCH(RPTv, 32, CALL)
#define SCAN_DISPATCH_ALL(CALL)                                                                                               \
  do {                                                                                                                        \
    SCAN_DISPATCH_ROW(8, CALL) SCAN_DISPATCH_ROW(16, CALL) SCAN_DISPATCH_ROW(32, CALL) SCAN_DISPATCH_ROW(64, CALL)            \
  } while (0)

// proj [T, ld] (dtype 0 = bf16, 1 = fp32) holds, per token, the projections a windowed attention mixer convolves: queries [H d] at
// column q_col0 and keys [G d] at k_col0.  Per token: short convolution (weights fp32 [channels, taps], last column = current token,
// earlier rows from the batch or from `state` [slots, taps - 1, (H + G) d]) -> the convolved keys go to plane 1 of the token's cache row
// (they are the values); RMS norm over the whole q / whole k projection with plain weights norm_q / norm_k; rotation of pairs (2i, 2i + 1)
// of the first rot_dims entries of every head by pos * freq[i] (freq: doubles on the device); q to q_out [T, q_ld], k to cache plane 0.
// cache [blocks, 2, block_size, G, d].  Call dsb200_conv_state_update afterwards.
DSB_EXPORT int dsb200_window_qk_prepare(const void* proj, long long ld, int q_col0, int k_col0, const float* conv_q, const float* conv_k,
                                        const float* norm_q, const float* norm_k, const void* state, const int* seq_desc, const int* tok_seq,
                                        const int* tok_pos, const int* block_table, int bt_stride, int block_size, void* cache, void* q_out,
                                        long long q_ld, const double* freq, int n_tokens, int H, int G, int d, int taps, int rot_dims, float eps,
                                        int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  DSB_REQUIRE(H >= 1 && G >= 1 && H % G == 0 && d >= 1 && rot_dims % 2 == 0 && rot_dims <= d && taps >= 1,
              "window_qk_prepare: heads %d / %d, head size %d, rotated %d, taps %d", H, G, d, rot_dims, taps);
  const size_t smem = (static_cast<size_t>(H + G) * d + rot_dims) * sizeof(float);
  DSB_REQUIRE(smem <= 200 * 1024, "window_qk_prepare: (H + G) d = %d does not fit shared memory", (H + G) * d);
  static const int block_env = [] { const char* e = getenv("DSB200_PREP_BLOCK"); return e ? atoi(e) : 0; }();
  // many tokens: small blocks (more tokens in flight per SM); few tokens (decode steps): many threads per token (a short chain per thread)
  const int few = min(1024, max(128, (((H + G) * d + 3) / 4 + 31) / 32 * 32));
  const int block = block_env >= 64 && block_env <= 1024 ? block_env : (n_tokens >= 512 ? 256 : few);
#define LAUNCH(T)                                                                                                                          \
  do {                                                                                                                                     \
    if (smem > 48 * 1024) DSB_CHECK_CUDA(cudaFuncSetAttribute(window_qk_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    window_qk_prepare_kernel<T><<<n_tokens, block, smem, stream>>>((const T*)proj, ld, q_col0, k_col0, conv_q, conv_k, norm_q, norm_k,     \
                                                                   (const T*)state, (const int4*)seq_desc, tok_seq, tok_pos, block_table,   \
                                                                   bt_stride, block_size, (T*)cache, (T*)q_out, q_ld, freq, H, G, d, taps,  \
                                                                   rot_dims, eps);                                                         \
  } while (0)
  if (dtype == 0) LAUNCH(bf16);
  else LAUNCH(float);
#undef LAUNCH
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// Columns st_col0 .. st_col0 + C of state [slots, taps - 1, st_ld] <- the last taps - 1 projected rows (columns col0 .. col0 + C of proj
// [T, ld]) of every sequence of the batch, older rows shifting up when the step brought fewer than taps - 1 tokens.  Run after the
// kernels that read the state.
DSB_EXPORT int dsb200_conv_state_update(const void* proj, long long ld, int col0, void* state, int st_ld, int st_col0, const int* seq_desc,
                                        int n_seqs, int C, int taps, int dtype, cudaStream_t stream) {
  if (n_seqs == 0 || taps <= 1 || C == 0) return DSB_OK;
  const dim3 grid((C + 255) / 256, n_seqs);
  if (dtype == 0) conv_state_update_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)proj, ld, col0, (bf16*)state, st_ld, st_col0, (const int4*)seq_desc, C, taps);
  else conv_state_update_kernel<float><<<grid, 256, 0, stream>>>((const float*)proj, ld, col0, (float*)state, st_ld, st_col0, (const int4*)seq_desc, C, taps);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// out[t, h d + c] = out_scale * sum_j softmax_j(scale q_h . k_j) v_j[c] over the keys j <= pos(t) of the token's sequence with
// pos - j < window or j < keep_first.  q [T, q_ld] (H heads of d), cache [blocks, 2, block_size, G, d] (plane 0 keys, 1 values), query head
// h reads key/value head h / (H / G); out [T, out_ld].  CUDA cores, fp32 scores and accumulation, any sizes; dtype 0 = bf16, 1 = fp32.
DSB_EXPORT int dsb200_window_attention(const void* q, long long q_ld, const void* cache, const int* tok_seq, const int* tok_pos,
                                       const int* block_table, int bt_stride, int block_size, void* out, long long out_ld, int n_tokens, int H,
                                       int G, int d, int window, int keep_first, float scale, float out_scale, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  DSB_REQUIRE(H % G == 0 && window >= 1 && keep_first >= 0 && d <= 4096, "window_attention: heads %d / %d, window %d, kept %d, head size %d", H, G,
              window, keep_first, d);
  const dim3 grid(n_tokens, H);
  const size_t smem = 2 * static_cast<size_t>(d) * sizeof(float);
  if (dtype == 0)
    window_attention_kernel<bf16><<<grid, WA_THREADS, smem, stream>>>((const bf16*)q, q_ld, (const bf16*)cache, tok_seq, tok_pos, block_table,
                                                                      bt_stride, block_size, (bf16*)out, out_ld, H, G, d, window, keep_first,
                                                                      scale, out_scale);
  else
    window_attention_kernel<float><<<grid, WA_THREADS, smem, stream>>>((const float*)q, q_ld, (const float*)cache, tok_seq, tok_pos, block_table,
                                                                       bt_stride, block_size, (float*)out, out_ld, H, G, d, window, keep_first,
                                                                       scale, out_scale);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// Matrix memory with exponential gating, per sequence and head, over the new tokens in order:
//   i = cap tanh((gates[t, h] + bias_i[h]) / cap),  f = logsigmoid(cap tanh((gates[t, H + h] + bias_f[h]) / cap)),
//   m' = max(f + m, i);  S <- exp(f + m - m') S + exp(i - m') k v^T;  n likewise with k;  out = S^T q / (max(|n . q|, exp(-m')) + 1e-6)
// with q = proj[q_col0 ..] * d^-1/2, k, v from proj [T, ld] (dtype 0 = bf16, 1 = fp32); gates fp32 [T, 2 H]; out fp32 [T, H dv].
// state_S [slots, H, dsb200_scan_state_floats(d, dv)], state_n [slots, H, d], state_m [slots, H], all fp32; a sequence at position 0 starts
// from zeros (m = 0).
DSB_EXPORT int dsb200_matrix_memory_scan(const void* proj, long long ld, int q_col0, int k_col0, int v_col0, const float* gates,
                                         const float* bias_i, const float* bias_f, float cap, const int* seq_desc, float* state_S,
                                         float* state_n, float* state_m, float* out, int n_seqs, int H, int d, int dv, int dtype,
                                         cudaStream_t stream) {
  if (n_seqs == 0) return DSB_OK;
  int R, RPT, tiles, ch;
  DSB_REQUIRE(scan_shape(d, dv, &R, &RPT, &tiles, &ch), "matrix_memory_scan: a %d x %d state per head is not supported", d, dv);
  const int threads = SCAN_THREADS + 32;
  const size_t smem = (2 * static_cast<size_t>(2 * ch * R * RPT + ch * SCAN_CPT * (SCAN_THREADS / R) + 4 * ch) + 2 * ch) * sizeof(float);
  DSB_REQUIRE(smem <= 200 * 1024, "matrix_memory_scan: head sizes %d / %d do not fit shared memory", d, dv);
  const dim3 grid(n_seqs, H, tiles);
  bool launched = false;
#define CALL(RPTv, Rv)                                                                                                                    \
  do {                                                                                                                                    \
    if (dtype == 0)                                                                                                                       \
    {                                                                                                                                     \
      if (smem > 48 * 1024)                                                                                                               \
        DSB_CHECK_CUDA(cudaFuncSetAttribute(matrix_memory_scan_kernel<bf16, RPTv, Rv>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      matrix_memory_scan_kernel<bf16, RPTv, Rv><<<grid, threads, smem, stream>>>((const bf16*)proj, ld, q_col0, k_col0, v_col0, gates, bias_i, \
                                                                                 bias_f, cap, (const int4*)seq_desc, state_S, state_n,    \
                                                                                 state_m, out, H, d, dv, ch);                             \
    }                                                                                                                                     \
    else                                                                                                                                  \
    {                                                                                                                                     \
      if (smem > 48 * 1024)                                                                                                               \
        DSB_CHECK_CUDA(cudaFuncSetAttribute(matrix_memory_scan_kernel<float, RPTv, Rv>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      matrix_memory_scan_kernel<float, RPTv, Rv><<<grid, threads, smem, stream>>>((const float*)proj, ld, q_col0, k_col0, v_col0, gates,      \
                                                                                  bias_i, bias_f, cap, (const int4*)seq_desc, state_S,    \
                                                                                  state_n, state_m, out, H, d, dv, ch);                   \
    }                                                                                                                                     \
  } while (0)
  SCAN_DISPATCH_ALL(CALL);
#undef CALL
  DSB_REQUIRE(launched, "matrix_memory_scan: no kernel for %d rows per thread x %d lanes", RPT, R);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// Inputs of the delta-rule scan from the fused projection proj [T, ld] (dtype 0 = bf16, 1 = fp32): q [G d] at q_col0, k [G d] at k_col0, v
// [H dv] at v_col0, each through its short convolution (weights fp32 [channels, taps]; earlier rows from the batch or from `state`
// [slots, taps - 1, 2 G d + H dv]) and silu; q and k then scaled to unit length per head (x / sqrt(sum x^2 + 1e-6)), q also by d^-1/2.
// qn, kn fp32 [T, G d]; vo fp32 [T, H dv].  In place: a_pre fp32 [T, H d] <- exp(-exp(A_log[h]) softplus(a_pre + dt_bias)) (the decays) and
// beta_pre fp32 [T, H] <- sigmoid(beta_pre).  Call dsb200_conv_state_update afterwards.
DSB_EXPORT int dsb200_delta_prepare(const void* proj, long long ld, int q_col0, int k_col0, int v_col0, const float* conv_q, const float* conv_k,
                                    const float* conv_v, const void* state, const int* seq_desc, const int* tok_seq, float* qn, float* kn,
                                    float* vo, float* a_pre, float* beta_pre, const float* A_log, const float* dt_bias, int n_tokens, int G, int H,
                                    int d, int dv, int taps, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  const size_t smem = 2 * static_cast<size_t>(G) * d * sizeof(float);
  DSB_REQUIRE(smem <= 200 * 1024, "delta_prepare: 2 G d = %d does not fit shared memory", 2 * G * d);
  static const int block_env = [] { const char* e = getenv("DSB200_PREP_BLOCK"); return e ? atoi(e) : 0; }();
  const int few = min(1024, max(128, ((2 * G * d + H * dv + 3) / 4 + 31) / 32 * 32));
  const int block = block_env >= 64 && block_env <= 1024 ? block_env : (n_tokens >= 512 ? 256 : few);
#define LAUNCH(T)                                                                                                                       \
  do {                                                                                                                                  \
    if (smem > 48 * 1024) DSB_CHECK_CUDA(cudaFuncSetAttribute(delta_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    delta_prepare_kernel<T><<<n_tokens, block, smem, stream>>>((const T*)proj, ld, q_col0, k_col0, v_col0, conv_q, conv_k, conv_v,        \
                                                               (const T*)state, (const int4*)seq_desc, tok_seq, qn, kn, vo, a_pre, beta_pre,  \
                                                               A_log, dt_bias, G, H, d, dv, taps);                                        \
  } while (0)
  if (dtype == 0) LAUNCH(bf16);
  else LAUNCH(float);
#undef LAUNCH
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// Gated delta rule with one decay per head and key channel, per sequence and head over the new tokens in order:
//   S <- diag(decay[t, h, :]) S;  u = beta[t, h] (v - S^T k);  S <- S + k u^T;  out = S^T q
// qn, kn fp32 [T, G d] (head h reads q / k head h / (H / G)), v fp32 [T, H dv], beta fp32 [T, H], decay fp32 [T, H d] (as dsb200_delta_prepare
// leaves them); out fp32 [T, H dv]; state_S [slots, H, dsb200_scan_state_floats(d, dv)] fp32; a sequence at position 0 starts from zeros.
DSB_EXPORT int dsb200_delta_rule_scan(const float* qn, const float* kn, const float* v, const float* beta, const float* decay, const int* seq_desc,
                                      float* state_S, float* out, int n_seqs, int H, int G, int d, int dv, cudaStream_t stream) {
  if (n_seqs == 0) return DSB_OK;
  int R, RPT, tiles, ch;
  DSB_REQUIRE(H % G == 0 && scan_shape(d, dv, &R, &RPT, &tiles, &ch), "delta_rule_scan: heads %d / %d, a %d x %d state per head is not supported", H, G, d,
              dv);
  const int threads = SCAN_THREADS;
  const size_t smem = 2 * static_cast<size_t>(3 * ch * R * RPT + ch * SCAN_CPT * (SCAN_THREADS / R) + ((ch + 3) & ~3)) * sizeof(float);
  DSB_REQUIRE(smem <= 200 * 1024, "delta_rule_scan: head sizes %d / %d do not fit shared memory", d, dv);
  const dim3 grid(n_seqs, H, tiles);
  bool launched = false;
#define CALL(RPTv, Rv)                                                                                                                         \
  do {                                                                                                                                         \
    if (smem > 48 * 1024)                                                                                                                      \
      DSB_CHECK_CUDA(cudaFuncSetAttribute(delta_rule_scan_kernel<RPTv, Rv>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));            \
    delta_rule_scan_kernel<RPTv, Rv><<<grid, threads, smem, stream>>>(qn, kn, v, beta, decay, (const int4*)seq_desc, state_S, out, H, G, d, dv, ch); \
  } while (0)
  SCAN_DISPATCH_ALL(CALL);
#undef CALL
  DSB_REQUIRE(launched, "delta_rule_scan: no kernel for %d rows per thread x %d lanes", RPT, R);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// Linear attention with the forget gate tied to the write strength, per sequence and head over the new tokens in order:
//   q = silu(proj[q_col0 ..]),  f = lower + (1 - lower) sigmoid(proj[f_col0 ..] + f_bias),  S <- diag(f) S + (1 - f) v^T,  out = S^T q
// proj [T, ld] (dtype 0 = bf16, 1 = fp32) with H heads of d (queries, gates) and dv (values); f_bias, lower fp32 [H d]; out fp32 [T, H dv];
// state_S [slots, H, dsb200_scan_state_floats(d, dv)] fp32; a sequence at position 0 starts from zeros.
DSB_EXPORT int dsb200_tied_gate_scan(const void* proj, long long ld, int q_col0, int f_col0, int v_col0, const float* f_bias, const float* lower,
                                     const int* seq_desc, float* state_S, float* out, int n_seqs, int H, int d, int dv, int dtype,
                                     cudaStream_t stream) {
  if (n_seqs == 0) return DSB_OK;
  int R, RPT, tiles, ch;
  DSB_REQUIRE(scan_shape(d, dv, &R, &RPT, &tiles, &ch), "tied_gate_scan: a %d x %d state per head is not supported", d, dv);
  const size_t smem = 2 * static_cast<size_t>(2 * ch * R * RPT + ch * SCAN_CPT * (SCAN_THREADS / R)) * sizeof(float);
  DSB_REQUIRE(smem <= 200 * 1024, "tied_gate_scan: head sizes %d / %d do not fit shared memory", d, dv);
  const dim3 grid(n_seqs, H, tiles);
  bool launched = false;
#define CALL_T(T, RPTv, Rv)                                                                                                                  \
  do {                                                                                                                                       \
    if (smem > 48 * 1024)                                                                                                                    \
      DSB_CHECK_CUDA(cudaFuncSetAttribute(tied_gate_scan_kernel<T, RPTv, Rv>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));      \
    tied_gate_scan_kernel<T, RPTv, Rv><<<grid, SCAN_THREADS, smem, stream>>>((const T*)proj, ld, q_col0, f_col0, v_col0, f_bias, lower,      \
                                                                             (const int4*)seq_desc, state_S, out, H, d, dv, ch);             \
  } while (0)
#define CALL(RPTv, Rv)                     \
  do {                                     \
    if (dtype == 0) CALL_T(bf16, RPTv, Rv); \
    else CALL_T(float, RPTv, Rv);          \
  } while (0)
  SCAN_DISPATCH_ALL(CALL);
#undef CALL
#undef CALL_T
  DSB_REQUIRE(launched, "tied_gate_scan: no kernel for %d rows per thread x %d lanes", RPT, R);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// out[t, h dv + c] = o[t, h, c] / sqrt(mean_c o[t, h, :]^2 + eps) * w[h * w_stride + c] * sigmoid(gate[t, h dv + c]) * mult.  o fp32
// [T, H dv]; w fp32 (w_stride = dv: one weight row per head, 0: one row shared by the heads); gate [T, gate_ld] and out [T, out_ld] in the
// activation dtype (0 = bf16, 1 = fp32).  gate may be null: mixers without an output gate.
DSB_EXPORT int dsb200_head_norm_gate(const float* o, const float* w, int w_stride, const void* gate, long long gate_ld, void* out, long long out_ld,
                                     int n_tokens, int H, int dv, float eps, float mult, int dtype, cudaStream_t stream) {
  const long long warps = static_cast<long long>(n_tokens) * H;
  if (warps == 0) return DSB_OK;
  const int wpb = 8;
  const int grid = static_cast<int>((warps + wpb - 1) / wpb);
  if (dtype == 0)
    head_norm_gate_kernel<bf16><<<grid, wpb * 32, 0, stream>>>(o, w, w_stride, (const bf16*)gate, gate_ld, (bf16*)out, out_ld, n_tokens, H, dv, eps, mult);
  else
    head_norm_gate_kernel<float><<<grid, wpb * 32, 0, stream>>>(o, w, w_stride, (const float*)gate, gate_ld, (float*)out, out_ld, n_tokens, H, dv, eps, mult);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// ------------------------------------------------------------------------------------------------------------------ minimal gated recurrence
// One number of state per channel: S <- (1 - z) S + z c with z = sigmoid(pz + bz), u = px + bx, c = u + 1/2 for u >= 0 and sigmoid(u) below;
// out = S silu(pg).  pz, px, pg are columns of the fused projection.  The update is the affine map S -> a S + b with a = 1 - z, b = z c, and
// affine maps compose, so long portions are cut into pieces of MG_PIECE rows of the BATCH (a piece may hold the end of one sequence and the
// start of the next: the first row of a sequence replaces whatever came before by the sequence's stored state, or zero at position 0):
//   mingru_scan_kernel     one thread per (sequence, channel) walks the new tokens in order (decode steps and short portions)
//   mingru_pieces_kernel   per (piece, channel): the composed map of the piece, (A, B); a sequence start inside makes A = 0
//   mingru_carry_kernel    per channel: walks the pieces, leaves the state in front of every piece
//   mingru_apply_kernel    per (piece, channel): walks the piece again from its carry, writes the outputs and, at a sequence's last row, its state
namespace dsb {
namespace recur {

constexpr int MG_PIECE = 32;

struct alignas(8) mg_bf16x4 {
  __nv_bfloat162 a, b;
};
// V neighbouring channels per thread (V = 4: every offset, stride and the width are multiples of 4 and the rows 16-byte aligned)
template <int V>
__device__ __forceinline__ void mg_load(const float* p, float* o) {
  if constexpr (V == 4) { const float4 v = *reinterpret_cast<const float4*>(p); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
  else o[0] = *p;
}
template <int V>
__device__ __forceinline__ void mg_load(const bf16* p, float* o) {
  if constexpr (V == 4) {
    const mg_bf16x4 v = *reinterpret_cast<const mg_bf16x4*>(p);
    const float2 lo = __bfloat1622float2(v.a), hi = __bfloat1622float2(v.b);
    o[0] = lo.x; o[1] = lo.y; o[2] = hi.x; o[3] = hi.y;
  } else o[0] = __bfloat162float(*p);
}
template <int V>
__device__ __forceinline__ void mg_store(float* p, const float* v) {
  if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else *p = v[0];
}
template <int V>
__device__ __forceinline__ void mg_store(bf16* p, const float* v) {
  if constexpr (V == 4) {
    mg_bf16x4 o;
    o.a = __floats2bfloat162_rn(v[0], v[1]);
    o.b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<mg_bf16x4*>(p) = o;
  } else *p = __float2bfloat16_rn(v[0]);
}
// the affine map of one token, S -> a S + b, from its gate and candidate pre-activations
template <int V>
__device__ __forceinline__ void mg_map(const float* pz, const float* px, const float* bz, const float* bx, float* a, float* b) {
#pragma unroll
  for (int e = 0; e < V; ++e) {
    const float z = sigmoidf_(pz[e] + bz[e]);
    const float u = px[e] + bx[e];
    a[e] = 1.f - z;
    b[e] = z * (u >= 0.f ? u + 0.5f : sigmoidf_(u));
  }
}
template <typename T, int V>
__device__ __forceinline__ void mg_step(const float* pz, const float* px, const float* pg, const float* bz, const float* bx, float* S,
                                        T* __restrict__ out) {
  float a[V], b[V], o[V];
  mg_map<V>(pz, px, bz, bx, a, b);
#pragma unroll
  for (int e = 0; e < V; ++e) {
    S[e] = fmaf(a[e], S[e], b[e]);
    o[e] = S[e] * siluf_(pg[e]);
  }
  mg_store<V>(out, o);
}

constexpr int MG_AHEAD = 4;  // tokens whose rows are loaded before the first of them is used: the walk is bound by load latency otherwise

template <typename T, int V>
__global__ void mingru_scan_kernel(const T* __restrict__ proj, long long ld, int z0, int x0, int g0, const float* __restrict__ zb,
                                   const float* __restrict__ xb, const int4* __restrict__ seq_desc, float* __restrict__ state,
                                   T* __restrict__ out, long long out_ld, int W) {
  const int4 sd = seq_desc[blockIdx.y];
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (c >= W) return;
  float* st = state + static_cast<size_t>(sd.w) * W + c;
  float S[V], bz[V], bx[V];
  mg_load<V>(st, S);
  if (sd.z == 0) {  // a sequence at position 0 starts from zero whatever the slot held
#pragma unroll
    for (int e = 0; e < V; ++e) S[e] = 0.f;
  }
  mg_load<V>(zb + c, bz);
  mg_load<V>(xb + c, bx);
  const T* row = proj + static_cast<long long>(sd.x) * ld + c;
  T* o = out + static_cast<long long>(sd.x) * out_ld + c;
  for (int i = 0; i < sd.y; i += MG_AHEAD) {
    float pz[MG_AHEAD][V], px[MG_AHEAD][V], pg[MG_AHEAD][V];
#pragma unroll
    for (int u = 0; u < MG_AHEAD; ++u)
      if (i + u < sd.y) {
        const T* r = row + static_cast<long long>(i + u) * ld;
        mg_load<V>(r + z0, pz[u]);
        mg_load<V>(r + x0, px[u]);
        mg_load<V>(r + g0, pg[u]);
      }
#pragma unroll
    for (int u = 0; u < MG_AHEAD; ++u)
      if (i + u < sd.y) mg_step<T, V>(pz[u], px[u], pg[u], bz, bx, S, o + static_cast<long long>(i + u) * out_ld);
  }
  mg_store<V>(st, S);
}

template <typename T, int V>
__global__ void mingru_pieces_kernel(const T* __restrict__ proj, long long ld, int z0, int x0, const float* __restrict__ zb,
                                     const float* __restrict__ xb, const int* __restrict__ tok_seq, const int4* __restrict__ seq_desc,
                                     const float* __restrict__ state, float* __restrict__ init, float* __restrict__ pa, float* __restrict__ pb,
                                     int n_tokens, int W) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (c >= W) return;
  const int p = blockIdx.y, t0 = p * MG_PIECE, t1 = min(n_tokens, t0 + MG_PIECE);
  float bz[V], bx[V], A[V], B[V];
  mg_load<V>(zb + c, bz);
  mg_load<V>(xb + c, bx);
#pragma unroll
  for (int e = 0; e < V; ++e) { A[e] = 1.f; B[e] = 0.f; }
  for (int t = t0; t < t1; t += MG_AHEAD) {
    float pz[MG_AHEAD][V], px[MG_AHEAD][V];
    int4 sd[MG_AHEAD];
    int sq[MG_AHEAD];
#pragma unroll
    for (int u = 0; u < MG_AHEAD; ++u)
      if (t + u < t1) {
        const T* r = proj + static_cast<long long>(t + u) * ld + c;
        mg_load<V>(r + z0, pz[u]);
        mg_load<V>(r + x0, px[u]);
        sq[u] = tok_seq[t + u];
        sd[u] = seq_desc[sq[u]];
      }
#pragma unroll
    for (int u = 0; u < MG_AHEAD; ++u)
      if (t + u < t1) {
        if (t + u == sd[u].x) {  // the sequence's own state replaces what came before
          mg_load<V>(state + static_cast<size_t>(sd[u].w) * W + c, B);
#pragma unroll
          for (int e = 0; e < V; ++e) { A[e] = 0.f; B[e] = sd[u].z > 0 ? B[e] : 0.f; }
          mg_store<V>(init + static_cast<size_t>(sq[u]) * W + c, B);
        }
        float a[V], b[V];
        mg_map<V>(pz[u], px[u], bz, bx, a, b);
#pragma unroll
        for (int e = 0; e < V; ++e) { A[e] *= a[e]; B[e] = fmaf(a[e], B[e], b[e]); }
      }
  }
  mg_store<V>(pa + static_cast<size_t>(p) * W + c, A);
  mg_store<V>(pb + static_cast<size_t>(p) * W + c, B);
}

__global__ void mingru_carry_kernel(const float* __restrict__ pa, float* __restrict__ pb, int n_pieces, int W) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= W) return;
  constexpr int AHEAD = 8;  // the maps of that many pieces are loaded before the first is applied (the walk itself is a chain)
  float S = 0.f;  // row 0 starts a sequence, so the first piece has A = 0
  for (int p = 0; p < n_pieces; p += AHEAD) {
    float A[AHEAD], B[AHEAD];
#pragma unroll
    for (int u = 0; u < AHEAD; ++u)
      if (p + u < n_pieces) {
        const size_t i = static_cast<size_t>(p + u) * W + c;
        A[u] = pa[i];
        B[u] = pb[i];
      }
#pragma unroll
    for (int u = 0; u < AHEAD; ++u)
      if (p + u < n_pieces) {
        pb[static_cast<size_t>(p + u) * W + c] = S;  // the state in front of piece p + u
        S = fmaf(A[u], S, B[u]);
      }
  }
}

template <typename T, int V>
__global__ void mingru_apply_kernel(const T* __restrict__ proj, long long ld, int z0, int x0, int g0, const float* __restrict__ zb,
                                    const float* __restrict__ xb, const int* __restrict__ tok_seq, const int4* __restrict__ seq_desc,
                                    float* __restrict__ state, const float* __restrict__ init, const float* __restrict__ carry,
                                    T* __restrict__ out, long long out_ld, int n_tokens, int W) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (c >= W) return;
  const int p = blockIdx.y, t0 = p * MG_PIECE, t1 = min(n_tokens, t0 + MG_PIECE);
  float bz[V], bx[V], S[V];
  mg_load<V>(zb + c, bz);
  mg_load<V>(xb + c, bx);
  mg_load<V>(carry + static_cast<size_t>(p) * W + c, S);
  for (int t = t0; t < t1; t += MG_AHEAD) {
    float pz[MG_AHEAD][V], px[MG_AHEAD][V], pg[MG_AHEAD][V];
    int4 sd[MG_AHEAD];
    int sq[MG_AHEAD];
#pragma unroll
    for (int u = 0; u < MG_AHEAD; ++u)
      if (t + u < t1) {
        const T* r = proj + static_cast<long long>(t + u) * ld + c;
        mg_load<V>(r + z0, pz[u]);
        mg_load<V>(r + x0, px[u]);
        mg_load<V>(r + g0, pg[u]);
        sq[u] = tok_seq[t + u];
        sd[u] = seq_desc[sq[u]];
      }
#pragma unroll
    for (int u = 0; u < MG_AHEAD; ++u)
      if (t + u < t1) {
        if (t + u == sd[u].x) mg_load<V>(init + static_cast<size_t>(sq[u]) * W + c, S);
        mg_step<T, V>(pz[u], px[u], pg[u], bz, bx, S, out + static_cast<long long>(t + u) * out_ld + c);
        if (t + u == sd[u].x + sd[u].y - 1) mg_store<V>(state + static_cast<size_t>(sd[u].w) * W + c, S);
      }
  }
}

}  // namespace recur
}  // namespace dsb

DSB_EXPORT long long dsb200_mingru_scratch_floats(int n_tokens, int n_seqs, int W) {
  const long long pieces = (n_tokens + dsb::recur::MG_PIECE - 1) / dsb::recur::MG_PIECE;
  return (2 * pieces + n_seqs) * static_cast<long long>(W);
}

// Minimal gated recurrence over every sequence's new tokens.  proj [T, ld] (dtype 0 = bf16, 1 = fp32) holds the gate, candidate and output-gate
// pre-activations at columns z_col0 / x_col0 / g_col0 (W each); zb, xb fp32 [W]; state fp32 [slots, W]; out [T, out_ld] in proj's dtype.
// seq_desc [n_seqs, 4] = (first row, new tokens, tokens seen before, slot); tok_seq [T].  scratch: dsb200_mingru_scratch_floats floats, used
// when `pieces` != 0 (portions cut into pieces that are walked side by side); else one thread per (sequence, channel) walks its tokens.
DSB_EXPORT int dsb200_mingru_scan(const void* proj, long long ld, int z_col0, int x_col0, int g_col0, const float* zb, const float* xb,
                                  const int* tok_seq, const int* seq_desc, float* state, void* out, long long out_ld, int n_tokens, int n_seqs, int W,
                                  int pieces, float* scratch, int dtype, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return DSB_OK;
  DSB_REQUIRE(W >= 1 && out_ld >= W && zb != nullptr && xb != nullptr && state != nullptr, "mingru_scan: width %d, output stride %lld", W, out_ld);
  const int threads = 128;
  auto mult4 = [](long long v) { return v % 4 == 0; };
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = mult4(W) && mult4(ld) && mult4(out_ld) && mult4(z_col0) && mult4(x_col0) && mult4(g_col0) && al16(proj) && al16(out) && al16(zb) && al16(xb) &&
                   al16(state) && al16(scratch);
  const int per = vec ? 4 : 1;
  const unsigned gx = static_cast<unsigned>((W / per + threads - 1) / threads);
  const unsigned gx1 = static_cast<unsigned>((W + threads - 1) / threads);
  if (!pieces) {
    const dim3 grid(gx, n_seqs);
    if (dtype == 0 && vec) mingru_scan_kernel<bf16, 4><<<grid, threads, 0, stream>>>((const bf16*)proj, ld, z_col0, x_col0, g_col0, zb, xb, (const int4*)seq_desc, state, (bf16*)out, out_ld, W);
    else if (dtype == 0) mingru_scan_kernel<bf16, 1><<<grid, threads, 0, stream>>>((const bf16*)proj, ld, z_col0, x_col0, g_col0, zb, xb, (const int4*)seq_desc, state, (bf16*)out, out_ld, W);
    else if (vec) mingru_scan_kernel<float, 4><<<grid, threads, 0, stream>>>((const float*)proj, ld, z_col0, x_col0, g_col0, zb, xb, (const int4*)seq_desc, state, (float*)out, out_ld, W);
    else mingru_scan_kernel<float, 1><<<grid, threads, 0, stream>>>((const float*)proj, ld, z_col0, x_col0, g_col0, zb, xb, (const int4*)seq_desc, state, (float*)out, out_ld, W);
    DSB_CHECK_CUDA(cudaGetLastError());
    return DSB_OK;
  }
  DSB_REQUIRE(scratch != nullptr && tok_seq != nullptr, "mingru_scan: the piecewise walk needs its scratch and the token -> sequence map");
  const int np = (n_tokens + MG_PIECE - 1) / MG_PIECE;
  float* pa = scratch;
  float* pb = pa + static_cast<size_t>(np) * W;
  float* init = pb + static_cast<size_t>(np) * W;
  const dim3 grid(gx, np);
  if (dtype == 0 && vec) mingru_pieces_kernel<bf16, 4><<<grid, threads, 0, stream>>>((const bf16*)proj, ld, z_col0, x_col0, zb, xb, tok_seq, (const int4*)seq_desc, state, init, pa, pb, n_tokens, W);
  else if (dtype == 0) mingru_pieces_kernel<bf16, 1><<<grid, threads, 0, stream>>>((const bf16*)proj, ld, z_col0, x_col0, zb, xb, tok_seq, (const int4*)seq_desc, state, init, pa, pb, n_tokens, W);
  else if (vec) mingru_pieces_kernel<float, 4><<<grid, threads, 0, stream>>>((const float*)proj, ld, z_col0, x_col0, zb, xb, tok_seq, (const int4*)seq_desc, state, init, pa, pb, n_tokens, W);
  else mingru_pieces_kernel<float, 1><<<grid, threads, 0, stream>>>((const float*)proj, ld, z_col0, x_col0, zb, xb, tok_seq, (const int4*)seq_desc, state, init, pa, pb, n_tokens, W);
  mingru_carry_kernel<<<gx1, threads, 0, stream>>>(pa, pb, np, W);
  if (dtype == 0 && vec) mingru_apply_kernel<bf16, 4><<<grid, threads, 0, stream>>>((const bf16*)proj, ld, z_col0, x_col0, g_col0, zb, xb, tok_seq, (const int4*)seq_desc, state, init, pb, (bf16*)out, out_ld, n_tokens, W);
  else if (dtype == 0) mingru_apply_kernel<bf16, 1><<<grid, threads, 0, stream>>>((const bf16*)proj, ld, z_col0, x_col0, g_col0, zb, xb, tok_seq, (const int4*)seq_desc, state, init, pb, (bf16*)out, out_ld, n_tokens, W);
  else if (vec) mingru_apply_kernel<float, 4><<<grid, threads, 0, stream>>>((const float*)proj, ld, z_col0, x_col0, g_col0, zb, xb, tok_seq, (const int4*)seq_desc, state, init, pb, (float*)out, out_ld, n_tokens, W);
  else mingru_apply_kernel<float, 1><<<grid, threads, 0, stream>>>((const float*)proj, ld, z_col0, x_col0, g_col0, zb, xb, tok_seq, (const int4*)seq_desc, state, init, pb, (float*)out, out_ld, n_tokens, W);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

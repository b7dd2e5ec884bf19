// build: precise-math
// Ragged-batch kernels for attention mixers whose heads are normed one by one and whose softmax has a sink:
//
//   head_norm_rotary_append   per token, from the fused projection: every query and key head is RMS-normed over its own entries with a weight
//                             shared by the heads, then the first rot_dims entries of the head are rotated (entry i paired with entry
//                             i + rot_dims / 2) by pos * freq[i], cosine and sine times a constant; every value head is divided by its own
//                             root mean square (no weight).  Queries leave as a tensor, keys and values go to their rows of the paged cache.
//   sink_attention            causal attention over the paged cache on CUDA cores: score = scale q . k, optionally soft-capped
//                             (cap tanh(score / cap)); weights exp(s_j) / (sink + sum_j exp(s_j)) with sink = 1 for a softmax that has
//                             one more, valueless entry of score 0, or 0 for the plain softmax.  Key and value heads may differ in size.
//
// Keys and values live in planes with their own row widths: k_cache + block * k_block_stride addresses block_size rows of G d values,
// v_cache + block * v_block_stride block_size rows of G dv values (both planes of one [blocks, 2, block_size, G, d] cache when d = dv, or
// two single-plane caches).  Every kernel takes its sizes as arguments and exists for bf16 and fp32 activations; norms, angles, scores and
// softmax are fp32 (angles are formed and reduced in double).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../common/host.h"

namespace dsb {
namespace sinkattn {

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

// One warp per (token, head slot); the H query heads, then the G key heads, then the G value heads of the token.
template <typename T>
__global__ void head_norm_rotary_append_kernel(const T* __restrict__ proj, long long ld, int q_col0, int k_col0, int v_col0,
                                               const float* __restrict__ wq, const float* __restrict__ wk, const double* __restrict__ freq,
                                               float mag, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                               const int* __restrict__ block_table, int bt_stride, int block_size, T* __restrict__ k_cache,
                                               long long k_block_stride, T* __restrict__ v_cache, long long v_block_stride, T* __restrict__ q_out,
                                               long long q_ld, int n_tokens, int H, int G, int d, int dv, int rot, float eps, int norm_v, int q_row,
                                               int k_row, int v_row) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int per_tok = H + 2 * G;
  if (gw >= n_tokens * per_tok) return;
  const int t = gw / per_tok, slot = gw % per_tok;
  const int pos = tok_pos[t];
  const T* row = proj + static_cast<long long>(t) * ld;
  long long cache_row = 0;
  if (slot >= H) cache_row = block_table[static_cast<size_t>(tok_seq[t]) * bt_stride + pos / block_size];
  const int in_block = pos % block_size;
  if (slot >= H + G) {  // a value head: its own root mean square, no weight
    const int g = slot - H - G;
    const T* src = row + v_col0 + g * dv;
    T* dst = v_cache + cache_row * v_block_stride + (static_cast<long long>(in_block) * G + g) * v_row;
    float inv = 1.f;
    if (norm_v) {
      float s = 0.f;
      for (int c = lane; c < dv; c += 32) { const float v = to_f(src[c]); s += v * v; }
      s = warp_sum(s);
      inv = 1.f / sqrtf(s / static_cast<float>(dv) + eps);
    }
    for (int c = lane; c < dv; c += 32) dst[c] = from_f<T>(to_f(src[c]) * inv);
    for (int c = dv + lane; c < v_row; c += 32) dst[c] = from_f<T>(0.f);  // rows padded to a width the tensor-core kernels take
    return;
  }
  const bool is_q = slot < H;
  const int head = is_q ? slot : slot - H;
  const T* src = row + (is_q ? q_col0 : k_col0) + head * d;
  const float* w = is_q ? wq : wk;
  T* dst = is_q ? q_out + static_cast<long long>(t) * q_ld + head * q_row
                : k_cache + cache_row * k_block_stride + (static_cast<long long>(in_block) * G + head) * k_row;
  float inv = 1.f;
  if (w != nullptr) {
    float s = 0.f;
    for (int c = lane; c < d; c += 32) { const float v = to_f(src[c]); s += v * v; }
    s = warp_sum(s);
    inv = 1.f / sqrtf(s / static_cast<float>(d) + eps);
  }
  const int half = rot >> 1;
  for (int i = lane; i < half; i += 32) {
    const float u = to_f(src[i]) * inv * (w ? w[i] : 1.f), v = to_f(src[i + half]) * inv * (w ? w[i + half] : 1.f);
    double a = static_cast<double>(pos) * freq[i];
    a -= 6.283185307179586476925 * rint(a * 0.15915494309189533576888);  // into [-pi, pi] before single precision takes over
    float sn, cs;
    sincosf(static_cast<float>(a), &sn, &cs);
    sn *= mag;
    cs *= mag;
    dst[i] = from_f<T>(u * cs - v * sn);
    dst[i + half] = from_f<T>(v * cs + u * sn);
  }
  for (int c = rot + lane; c < d; c += 32) dst[c] = from_f<T>(to_f(src[c]) * inv * (w ? w[c] : 1.f));
  for (int c = d + lane; c < (is_q ? q_row : k_row); c += 32) dst[c] = from_f<T>(0.f);  // padding: adds nothing to a score
}

// What the plain form of `sink_attention` does not have: per-head sink scores, a distance term on the scores, a mask by fixed parts of the
// sequence, and strides of their own for query / output heads and cached rows (so that one cached row can serve as key and as value).
struct SinkExtras {
  const float* sink_logit;     // [H] or null: exp(sink_logit[h]) joins the denominator (an entry without key and value)
  const float* r1;             // [H] or null: the score of key j loses r1[h] ln(1 + r2[h] (pos - j))
  const float* r2;
  int part;                    // > 0: a query at pos sees only the keys j <= pos with j / part == pos / part
  int k_row, v_row;            // elements between the heads of a cached key row / value row (>= d, dv)
  long long q_head_stride;     // elements between the heads of a query row
  long long out_head_stride;   // elements between the heads of an output row
};

// One block per (token, query head).  The visible keys first .. pos are walked in chunks of SA_CHUNK with a running maximum / sum (fp32).
constexpr int SA_CHUNK = 256, SA_THREADS = 128;
template <typename T>
__global__ void __launch_bounds__(SA_THREADS)
sink_attention_kernel(const T* __restrict__ q, long long q_ld, const T* __restrict__ k_cache, long long k_block_stride,
                      const T* __restrict__ v_cache, long long v_block_stride, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                      const int* __restrict__ block_table, int bt_stride, int block_size, T* __restrict__ out, long long out_ld, int H, int G,
                      int d, int dv, float scale, float cap, float sink, SinkExtras ex) {
  extern __shared__ float sm[];
  __shared__ float red[33];
  __shared__ float sc[SA_CHUNK];
  __shared__ int key_blk[SA_CHUNK], key_slot[SA_CHUNK];
  const int t = blockIdx.x, h = blockIdx.y, g = h / (H / G);
  const int seq = tok_seq[t], pos = tok_pos[t];
  float* qs = sm;        // [d]
  float* acc = sm + d;   // [dv]
  for (int c = threadIdx.x; c < d; c += SA_THREADS) qs[c] = to_f(q[static_cast<long long>(t) * q_ld + h * ex.q_head_stride + c]) * scale;
  for (int c = threadIdx.x; c < dv; c += SA_THREADS) acc[c] = 0.f;
  const int n = pos + 1;
  const int first = ex.part > 0 ? (pos / ex.part) * ex.part : 0;
  const int* bt = block_table + static_cast<size_t>(seq) * bt_stride;
  const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
  const float r1 = ex.r1 ? ex.r1[h] : 0.f, r2 = ex.r1 ? ex.r2[h] : 0.f;
  // a learned sink starts the running softmax as an entry of its own: maximum = its score, sum = 1, nothing accumulated
  float m_run = ex.sink_logit ? ex.sink_logit[h] : -INFINITY, l_run = ex.sink_logit ? 1.f : 0.f;
  __syncthreads();
  for (int x0 = first; x0 < n; x0 += SA_CHUNK) {
    const int cn = min(SA_CHUNK, n - x0);
    float mx = -INFINITY;
    for (int x = threadIdx.x; x < cn; x += SA_THREADS) {
      const int j = x0 + x;
      const int blk = bt[j / block_size], slot = j % block_size;
      key_blk[x] = blk;
      key_slot[x] = slot;
      const T* kr = k_cache + static_cast<long long>(blk) * k_block_stride + (static_cast<long long>(slot) * G + g) * ex.k_row;
      float s = 0.f;
      for (int c = 0; c < d; ++c) s = fmaf(qs[c], to_f(kr[c]), s);
      if (cap > 0.f) s = cap * tanhf(s * inv_cap);
      if (ex.r1) s -= r1 * log1pf(r2 * static_cast<float>(pos - j));
      sc[x] = s;
      mx = fmaxf(mx, s);
    }
    mx = block_max(mx, red);
    const float m_new = fmaxf(m_run, mx);
    float ls = 0.f;
    for (int x = threadIdx.x; x < cn; x += SA_THREADS) {
      const float p = expf(sc[x] - m_new);
      sc[x] = p;
      ls += p;
    }
    ls = block_sum(ls, red);
    const float corr = expf(m_run - m_new);  // 0 for the first chunk (m_run = -inf)
    l_run = l_run * corr + ls;
    m_run = m_new;
    for (int c = threadIdx.x; c < dv; c += SA_THREADS) {
      float a = acc[c] * corr;
      for (int x = 0; x < cn; ++x)
        a = fmaf(sc[x], to_f(v_cache[static_cast<long long>(key_blk[x]) * v_block_stride + (static_cast<long long>(key_slot[x]) * G + g) * ex.v_row + c]), a);
      acc[c] = a;
    }
    __syncthreads();
  }
  const float inv = 1.f / (l_run + sink * expf(-m_run));  // the constant sink's score is 0: exp(0 - m) in the shifted sum
  for (int c = threadIdx.x; c < dv; c += SA_THREADS) out[static_cast<long long>(t) * out_ld + h * ex.out_head_stride + c] = from_f<T>(acc[c] * inv);
}

// One warp per (token, slot).  Slots 0 .. H - 1: the rotated part (the last dr entries) of query head h, rotated in place.  Slot H: the
// low-rank row -- its first R entries RMS-normed with a weight, its last dr entries rotated -- goes to the token's row of the cache.
template <typename T>
__device__ __forceinline__ void rotate_half_row(const T* __restrict__ src, T* __restrict__ dst, int n, int rot, int pos, const double* __restrict__ freq,
                                                int lane) {
  const int half = rot >> 1;
  for (int i = lane; i < half; i += 32) {
    const float u = to_f(src[i]), v = to_f(src[i + half]);
    double a = static_cast<double>(pos) * freq[i];
    a -= 6.283185307179586476925 * rint(a * 0.15915494309189533576888);  // into [-pi, pi] before single precision takes over
    float sn, cs;
    sincosf(static_cast<float>(a), &sn, &cs);
    dst[i] = from_f<T>(u * cs - v * sn);
    dst[i + half] = from_f<T>(v * cs + u * sn);
  }
  if (dst != src)
    for (int c = rot + lane; c < n; c += 32) dst[c] = src[c];
}
template <typename T>
__global__ void latent_rotary_append_kernel(T* __restrict__ proj, long long ld, int q_col0, int kv_col0, const float* __restrict__ wkv,
                                            const double* __restrict__ freq, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                            const int* __restrict__ block_table, int bt_stride, int block_size, T* __restrict__ cache, int row_w,
                                            int n_tokens, int H, int d, int dr, int R, int rot, float eps) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (gw >= n_tokens * (H + 1)) return;
  const int t = gw / (H + 1), slot = gw % (H + 1);
  const int pos = tok_pos[t];
  T* row = proj + static_cast<long long>(t) * ld;
  if (slot < H) {
    T* v = row + q_col0 + slot * (d + dr) + d;
    rotate_half_row(v, v, dr, rot, pos, freq, lane);
    return;
  }
  const T* low = row + kv_col0;
  const long long blk = block_table[static_cast<size_t>(tok_seq[t]) * bt_stride + pos / block_size];
  T* dst = cache + (blk * block_size + pos % block_size) * row_w;
  float s = 0.f;
  for (int c = lane; c < R; c += 32) { const float v = to_f(low[c]); s += v * v; }
  s = warp_sum(s);
  const float inv = 1.f / sqrtf(s / static_cast<float>(R) + eps);
  for (int c = lane; c < R; c += 32) dst[c] = from_f<T>(to_f(low[c]) * inv * wkv[c]);
  rotate_half_row(low + R, dst + R, dr, rot, pos, freq, lane);
  for (int c = R + dr + lane; c < row_w; c += 32) dst[c] = from_f<T>(0.f);  // rows padded to a width the tensor-core kernels take
}

struct alignas(8) bf16x4 {
  __nv_bfloat162 a, b;
};
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const bf16x4 v = *reinterpret_cast<const bf16x4*>(p);
  const float2 lo = __bfloat1622float2(v.a), hi = __bfloat1622float2(v.b);
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  bf16x4 o;
  o.a = __floats2bfloat162_rn(v.x, v.y);
  o.b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<bf16x4*>(p) = o;
}

// One warp per (token, SL consecutive head slots): the H query heads, then the G key heads, then the G value heads of the token.  Every
// channel first passes a short causal convolution over the sequence (bias added to every real row; rows before this step's come from the
// state, rows before the sequence are zeros); query / key heads then get their RMS norm, value heads are mixed with another layer's values of
// the same token.  A lane owns VEC neighbouring channels at a time (VEC = 4: every size, offset and stride is a multiple of 4 and the rows
// are 16-byte aligned).  SL = 1: heads of any size; the convolved values of up to CH_REGS channels per lane stay in registers between the
// statistic and the scaling, what a wider head has beyond them is convolved a second time.  SL > 1 (heads of at most 32 VEC entries): the
// loads of all SL slots are issued before the first statistic is formed, and the token's metadata is read once for all of them -- the kernel
// is bound by the latency of its dependent loads, not by their volume.
constexpr int CH_REGS = 8;
template <typename T, int VEC, int SL>
__global__ void __launch_bounds__(256, 4)
conv_head_norm_append_kernel(const T* __restrict__ proj, long long ld, int col0, const float* __restrict__ bias, const float* __restrict__ conv_w,
                             const float* __restrict__ wq, const float* __restrict__ wk, const T* __restrict__ state,
                             const int4* __restrict__ seq_desc, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                             const int* __restrict__ block_table, int bt_stride, int block_size, T* __restrict__ k_cache, long long k_block_stride,
                             T* __restrict__ v_cache, long long v_block_stride, T* __restrict__ q_out, long long q_ld, const T* __restrict__ v_other,
                             const float* __restrict__ mix, T* __restrict__ v_own, int n_tokens, int H, int G, int d, int dv, int taps, float eps,
                             int q_row, int k_row, int v_row) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int per_tok = H + 2 * G, groups = (per_tok + SL - 1) / SL;
  if (gw >= n_tokens * groups) return;
  const int t = gw / groups, slot0 = (gw % groups) * SL;
  const int seq = tok_seq[t], pos = tok_pos[t];
  const int4 sd = seq_desc[seq];
  const int i = t - sd.x;  // index among the sequence's new tokens
  const int C = (H + G) * d + G * dv;  // convolved channels: q | k | v, as they lie in proj from col0 on and in the state rows
  const T* st = state ? state + static_cast<size_t>(sd.w) * (taps - 1) * C : nullptr;
  const long long cache_row = block_table[static_cast<size_t>(seq) * bt_stride + pos / block_size];
  const int in_block = pos % block_size;
  // rows the taps read: tap j reads the token taps - 1 - j positions back -- a row of this step, a row of the state, or nothing
  const int j0 = max(0, taps - 1 - pos);           // taps before j0 lie before the sequence's start
  const int js = min(taps, max(j0, taps - 1 - i));  // taps j0 .. js - 1 read the state, taps js .. read rows of this step
  const T* own = proj + static_cast<long long>(sd.x + i - (taps - 1)) * ld + col0;  // + j * ld: the row of tap j (j >= js)
  const T* old = st ? st + static_cast<long long>(i) * C : nullptr;               // + j * C: the state row of tap j (j < js)

  struct Slot {
    bool is_q, is_v;
    int head, n, ch0, width;
    T* dst;
  };
  auto slot_of = [&](int slot) {
    Slot o;
    o.is_q = slot < H;
    o.is_v = slot >= H + G;
    o.head = o.is_q ? slot : (o.is_v ? slot - H - G : slot - H);
    o.n = o.is_v ? dv : d;
    o.ch0 = o.is_q ? o.head * d : (o.is_v ? (H + G) * d + o.head * dv : H * d + o.head * d);
    o.width = o.is_q ? q_row : (o.is_v ? v_row : k_row);
    o.dst = o.is_q ? q_out + static_cast<long long>(t) * q_ld + o.head * q_row
                   : (o.is_v ? v_cache + cache_row * v_block_stride + (static_cast<long long>(in_block) * G + o.head) * v_row
                             : k_cache + cache_row * k_block_stride + (static_cast<long long>(in_block) * G + o.head) * k_row);
    return o;
  };
  auto conv = [&](int ch, float* y) {  // VEC channels from ch on
    if constexpr (VEC == 4) {
      const float4 b = bias ? load4(bias + ch) : make_float4(0.f, 0.f, 0.f, 0.f);
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = j0; j < taps; ++j) {
        const float4 u = j < js ? load4(old + static_cast<long long>(j) * C + ch) : load4(own + static_cast<long long>(j) * ld + ch);
        const float4 w = load4(conv_w + static_cast<size_t>(j) * C + ch);  // [taps, channels]: the lanes of a warp read one stretch
        a.x = fmaf(w.x, u.x + b.x, a.x);
        a.y = fmaf(w.y, u.y + b.y, a.y);
        a.z = fmaf(w.z, u.z + b.z, a.z);
        a.w = fmaf(w.w, u.w + b.w, a.w);
      }
      y[0] = a.x; y[1] = a.y; y[2] = a.z; y[3] = a.w;
    } else {
      const float b = bias ? bias[ch] : 0.f;
      float a = 0.f;
      for (int j = j0; j < taps; ++j) {
        const float u = to_f(j < js ? old[static_cast<long long>(j) * C + ch] : own[static_cast<long long>(j) * ld + ch]);
        a = fmaf(conv_w[static_cast<size_t>(j) * C + ch], u + b, a);
      }
      y[0] = a;
    }
  };
  auto emit = [&](const Slot& S, int c, const float* y, float inv) {  // scale (queries / keys) or mix (values) and store VEC channels from c on
    float o[VEC];
    if (S.is_v) {
      const size_t vi = static_cast<size_t>(t) * G * dv + S.head * dv + c;
      if (v_own) {
        if constexpr (VEC == 4) store4(v_own + vi, make_float4(y[0], y[1], y[2], y[3]));
        else v_own[vi] = from_f<T>(y[0]);
      }
      if (v_other) {
        const float lam = mix[0];
        if constexpr (VEC == 4) {
          const float4 w = load4(v_other + vi);
          o[0] = (1.f - lam) * y[0] + lam * w.x; o[1] = (1.f - lam) * y[1] + lam * w.y; o[2] = (1.f - lam) * y[2] + lam * w.z; o[3] = (1.f - lam) * y[3] + lam * w.w;
        } else {
          o[0] = (1.f - lam) * y[0] + lam * to_f(v_other[vi]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = y[e];
      }
    } else {
      const float* w = S.is_q ? wq : wk;
      if constexpr (VEC == 4) {
        const float4 g = load4(w + c);
        o[0] = y[0] * inv * g.x; o[1] = y[1] * inv * g.y; o[2] = y[2] * inv * g.z; o[3] = y[3] * inv * g.w;
      } else {
        o[0] = y[0] * inv * w[c];
      }
    }
    if constexpr (VEC == 4) store4(S.dst + c, make_float4(o[0], o[1], o[2], o[3]));
    else S.dst[c] = from_f<T>(o[0]);
  };

  if constexpr (SL > 1) {
    const int c = lane * VEC;
    float held[SL][VEC];
#pragma unroll
    for (int s = 0; s < SL; ++s) {
      if (slot0 + s < per_tok) {
        const Slot S = slot_of(slot0 + s);
        if (c < S.n) conv(S.ch0 + c, held[s]);
      }
    }
#pragma unroll
    for (int s = 0; s < SL; ++s) {
      if (slot0 + s < per_tok) {  // uniform over the warp
        const Slot S = slot_of(slot0 + s);
        float ss = 0.f;
        if (c < S.n) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) ss += held[s][e] * held[s][e];
        }
        float inv = 1.f;
        if (!S.is_v) {
          ss = warp_sum(ss);
          inv = 1.f / sqrtf(ss / static_cast<float>(S.n) + eps);
        }
        if (c < S.n) emit(S, c, held[s], inv);
        for (int x = S.n + lane; x < S.width; x += 32) S.dst[x] = from_f<T>(0.f);  // padding: adds nothing to a score or an output
      }
    }
  } else {
    const Slot S = slot_of(slot0);
    constexpr int GROUPS = CH_REGS / VEC;
    float held[CH_REGS];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < GROUPS; ++k) {
      const int c = (lane + 32 * k) * VEC;
      if (c < S.n) {
        conv(S.ch0 + c, held + k * VEC);
#pragma unroll
        for (int e = 0; e < VEC; ++e) ss += held[k * VEC + e] * held[k * VEC + e];
      }
    }
    for (int c = (lane + 32 * GROUPS) * VEC; c < S.n; c += 32 * VEC) {  // heads wider than the registers hold
      float y[VEC];
      conv(S.ch0 + c, y);
#pragma unroll
      for (int e = 0; e < VEC; ++e) ss += y[e] * y[e];
    }
    float inv = 1.f;
    if (!S.is_v) {
      ss = warp_sum(ss);
      inv = 1.f / sqrtf(ss / static_cast<float>(S.n) + eps);
    }
#pragma unroll
    for (int k = 0; k < GROUPS; ++k) {
      const int c = (lane + 32 * k) * VEC;
      if (c < S.n) emit(S, c, held + k * VEC, inv);
    }
    for (int c = (lane + 32 * GROUPS) * VEC; c < S.n; c += 32 * VEC) {
      float y[VEC];
      conv(S.ch0 + c, y);
      emit(S, c, y, inv);
    }
    for (int x = S.n + lane; x < S.width; x += 32) S.dst[x] = from_f<T>(0.f);  // padding: adds nothing to a score or an output
  }
}

}  // namespace sinkattn
}  // namespace dsb

using namespace dsb;
using namespace dsb::sinkattn;

// proj [T, ld] (dtype 0 = bf16, 1 = fp32) holds per token the query heads [H d] at q_col0, the key heads [G d] at k_col0 and the value heads
// [G dv] at v_col0.  Query / key heads: RMS norm over d with the weights wq / wk [d] (shared by the heads; null = no norm), then rotation
// of the first rot_dims entries (pairs (i, i + rot_dims / 2)) by pos * freq[i] (freq: rot_dims / 2 doubles on the device) with cosine and
// sine multiplied by `mag`.  Value heads: divided by their root mean square over dv when norm_v.  Queries -> q_out [T, q_ld]; keys ->
// k_cache, values -> v_cache at the token's (block, slot) (see the file header for the plane addressing).  q_row / k_row / v_row: elements
// between consecutive heads of a query row / a cached key row / a cached value row (>= d, d, dv); what lies past a head's own entries is
// written as zeros, so that heads padded to a common width of 64 / 128 can be served by the tensor-core attention kernels.
DSB_EXPORT int dsb200_head_norm_rotary_append(const void* proj, long long ld, int q_col0, int k_col0, int v_col0, const float* wq, const float* wk,
                                              const double* freq, float mag, const int* tok_seq, const int* tok_pos, const int* block_table,
                                              int bt_stride, int block_size, void* k_cache, long long k_block_stride, void* v_cache,
                                              long long v_block_stride, void* q_out, long long q_ld, int n_tokens, int H, int G, int d, int dv,
                                              int rot_dims, float eps, int norm_v, int q_row, int k_row, int v_row, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  DSB_REQUIRE(H >= 1 && G >= 1 && d >= 1 && dv >= 1 && rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= d && (rot_dims == 0 || freq != nullptr),
              "head_norm_rotary_append: heads %d / %d, head sizes %d / %d, rotated %d", H, G, d, dv, rot_dims);
  DSB_REQUIRE(q_row >= d && k_row >= d && v_row >= dv, "head_norm_rotary_append: row widths %d / %d / %d below the head sizes %d / %d", q_row, k_row, v_row, d, dv);
  const long long warps = static_cast<long long>(n_tokens) * (H + 2 * G);
  const int wpb = 8;
  const int grid = static_cast<int>((warps + wpb - 1) / wpb);
  if (dtype == 0)
    head_norm_rotary_append_kernel<bf16><<<grid, wpb * 32, 0, stream>>>((const bf16*)proj, ld, q_col0, k_col0, v_col0, wq, wk, freq, mag, tok_seq, tok_pos,
                                                                       block_table, bt_stride, block_size, (bf16*)k_cache, k_block_stride,
                                                                       (bf16*)v_cache, v_block_stride, (bf16*)q_out, q_ld, n_tokens, H, G, d, dv,
                                                                       rot_dims, eps, norm_v, q_row, k_row, v_row);
  else
    head_norm_rotary_append_kernel<float><<<grid, wpb * 32, 0, stream>>>((const float*)proj, ld, q_col0, k_col0, v_col0, wq, wk, freq, mag, tok_seq,
                                                                        tok_pos, block_table, bt_stride, block_size, (float*)k_cache, k_block_stride,
                                                                        (float*)v_cache, v_block_stride, (float*)q_out, q_ld, n_tokens, H, G, d, dv,
                                                                        rot_dims, eps, norm_v, q_row, k_row, v_row);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

static int launch_sink_attention(const void* q, long long q_ld, const void* k_cache, long long k_block_stride, const void* v_cache,
                                 long long v_block_stride, const int* tok_seq, const int* tok_pos, const int* block_table, int bt_stride,
                                 int block_size, void* out, long long out_ld, int n_tokens, int H, int G, int d, int dv, float scale, float cap,
                                 float sink, const SinkExtras& ex, int dtype, cudaStream_t stream) {
  const dim3 grid(n_tokens, H);
  const size_t smem = static_cast<size_t>(d + dv) * sizeof(float);
  if (dtype == 0)
    sink_attention_kernel<bf16><<<grid, SA_THREADS, smem, stream>>>((const bf16*)q, q_ld, (const bf16*)k_cache, k_block_stride, (const bf16*)v_cache,
                                                                    v_block_stride, tok_seq, tok_pos, block_table, bt_stride, block_size, (bf16*)out,
                                                                    out_ld, H, G, d, dv, scale, cap, sink, ex);
  else
    sink_attention_kernel<float><<<grid, SA_THREADS, smem, stream>>>((const float*)q, q_ld, (const float*)k_cache, k_block_stride,
                                                                     (const float*)v_cache, v_block_stride, tok_seq, tok_pos, block_table, bt_stride,
                                                                     block_size, (float*)out, out_ld, H, G, d, dv, scale, cap, sink, ex);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// out[t, h dv + c] = sum_j p_j v_j[c] over the keys j <= pos(t) of the token's sequence, p_j = exp(s_j) / (sink + sum_j exp(s_j)),
// s_j = scale q_h . k_j, soft-capped as cap tanh(s_j / cap) when cap > 0.  q [T, q_ld] (H heads of d); query head h reads key/value head
// h / (H / G); out [T, out_ld] (H heads of dv).  CUDA cores, fp32 scores and accumulation, any sizes; dtype 0 = bf16, 1 = fp32.
DSB_EXPORT int dsb200_sink_attention(const void* q, long long q_ld, const void* k_cache, long long k_block_stride, const void* v_cache,
                                     long long v_block_stride, const int* tok_seq, const int* tok_pos, const int* block_table, int bt_stride,
                                     int block_size, void* out, long long out_ld, int n_tokens, int H, int G, int d, int dv, float scale, float cap,
                                     float sink, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  DSB_REQUIRE(H >= 1 && G >= 1 && H % G == 0 && d >= 1 && dv >= 1 && d + dv <= 8192 && sink >= 0.f, "sink_attention: heads %d / %d, head sizes %d / %d", H, G,
              d, dv);
  const SinkExtras ex{nullptr, nullptr, nullptr, 0, d, dv, d, dv};
  return launch_sink_attention(q, q_ld, k_cache, k_block_stride, v_cache, v_block_stride, tok_seq, tok_pos, block_table, bt_stride, block_size, out,
                               out_ld, n_tokens, H, G, d, dv, scale, cap, sink, ex, dtype, stream);
}

// `sink_attention` with learned sinks, a distance term, a mask by parts and free strides:
//   sink_logit [H] (or null): exp(sink_logit[h]) joins head h's denominator;   r1, r2 [H] (or both null): s_j -= r1[h] ln(1 + r2[h] (pos - j));
//   part > 0: only the keys of the query's own part of `part` positions (counted from position 0 of the sequence) are visible;
//   q[t * q_ld + h * q_head_stride + c], out[t * out_ld + h * out_head_stride + c]; a cached key / value head starts every k_row / v_row
//   elements of its token's row (one plane may serve as keys and as values: pass it twice, with d and dv entries read from a head's start).
DSB_EXPORT int dsb200_sink_attention_ex(const void* q, long long q_ld, long long q_head_stride, const void* k_cache, long long k_block_stride, int k_row,
                                        const void* v_cache, long long v_block_stride, int v_row, const int* tok_seq, const int* tok_pos,
                                        const int* block_table, int bt_stride, int block_size, void* out, long long out_ld, long long out_head_stride,
                                        int n_tokens, int H, int G, int d, int dv, float scale, float cap, float sink, const float* sink_logit,
                                        const float* r1, const float* r2, int part, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  DSB_REQUIRE(H >= 1 && G >= 1 && H % G == 0 && d >= 1 && dv >= 1 && d + dv <= 8192 && sink >= 0.f && part >= 0 && k_row >= d && v_row >= dv &&
                  (r1 == nullptr) == (r2 == nullptr),
              "sink_attention: heads %d / %d, head sizes %d / %d, rows %d / %d, part %d", H, G, d, dv, k_row, v_row, part);
  const SinkExtras ex{sink_logit, r1, r2, part, k_row, v_row, q_head_stride, out_head_stride};
  return launch_sink_attention(q, q_ld, k_cache, k_block_stride, v_cache, v_block_stride, tok_seq, tok_pos, block_table, bt_stride, block_size, out,
                               out_ld, n_tokens, H, G, d, dv, scale, cap, sink, ex, dtype, stream);
}

// Low-rank attention with one rotated key part shared by the heads.  proj [T, ld] (dtype 0 = bf16, 1 = fp32) holds per token the H query heads
// (d plain entries, then dr entries to rotate) from q_col0 and the low-rank row (R entries, then dr entries to rotate) from kv_col0.  The
// query heads' rotated parts are rotated IN PLACE (first rot_dims of the dr entries; entry i pairs with entry i + rot_dims / 2; angle =
// pos * freq[i], freq: rot_dims / 2 doubles on the device); the first R entries of the low-rank row are RMS-normed with wkv [R] and, with the
// rotated last dr entries behind them, written to the token's row of cache [blocks, block_size, row_w] (zeros from R + dr on).
DSB_EXPORT int dsb200_latent_rotary_append(void* proj, long long ld, int q_col0, int kv_col0, const float* wkv, const double* freq, const int* tok_seq,
                                           const int* tok_pos, const int* block_table, int bt_stride, int block_size, void* cache, int row_w,
                                           int n_tokens, int H, int d, int dr, int R, int rot_dims, float eps, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  DSB_REQUIRE(H >= 1 && d >= 0 && dr >= 0 && R >= 1 && rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dr && (rot_dims == 0 || freq != nullptr) &&
                  row_w >= R + dr && wkv != nullptr,
              "latent_rotary_append: heads %d, head %d + %d, rank %d, rotated %d, row %d", H, d, dr, R, rot_dims, row_w);
  const long long warps = static_cast<long long>(n_tokens) * (H + 1);
  const int wpb = 8;
  const int grid = static_cast<int>((warps + wpb - 1) / wpb);
  if (dtype == 0)
    latent_rotary_append_kernel<bf16><<<grid, wpb * 32, 0, stream>>>((bf16*)proj, ld, q_col0, kv_col0, wkv, freq, tok_seq, tok_pos, block_table, bt_stride,
                                                                    block_size, (bf16*)cache, row_w, n_tokens, H, d, dr, R, rot_dims, eps);
  else
    latent_rotary_append_kernel<float><<<grid, wpb * 32, 0, stream>>>((float*)proj, ld, q_col0, kv_col0, wkv, freq, tok_seq, tok_pos, block_table,
                                                                     bt_stride, block_size, (float*)cache, row_w, n_tokens, H, d, dr, R, rot_dims, eps);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// Attention inputs behind a short causal convolution.  proj [T, ld] holds from col0 on the query heads [H d], the key heads [G d] and the value
// heads [G dv] of every token; bias (fp32, that many entries, or null) is added to every row before the convolution with conv_w (fp32
// [taps, channels]: y_t = sum_j w[j, :] u_(t - taps + 1 + j), zeros before the sequence's start).  state [slots, taps - 1, channels]: the last
// rows of the sequence's earlier steps, WITHOUT the bias (update it afterwards with dsb200_conv_state_update).  Query / key heads: RMS norm over
// d with wq / wk [d] shared by the heads -> q_out [T, q_ld] (head h at h * q_row) / the key plane.  Value heads: v_own (null, or [T, G dv])
// receives the convolved values; with v_other ([T, G dv]) and mix (one float on the device) the cached value is (1 - mix) v + mix v_other.
// Heads are padded with zeros to q_row / k_row / v_row entries.
DSB_EXPORT int dsb200_conv_head_norm_append(const void* proj, long long ld, int col0, const float* bias, const float* conv_w, const float* wq,
                                            const float* wk, const void* state, const int* seq_desc, const int* tok_seq, const int* tok_pos,
                                            const int* block_table, int bt_stride, int block_size, void* k_cache, long long k_block_stride,
                                            void* v_cache, long long v_block_stride, void* q_out, long long q_ld, const void* v_other,
                                            const float* mix, void* v_own, int n_tokens, int H, int G, int d, int dv, int taps, float eps, int q_row,
                                            int k_row, int v_row, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  DSB_REQUIRE(H >= 1 && G >= 1 && d >= 1 && dv >= 1 && taps >= 1 && (taps == 1 || state != nullptr) && conv_w != nullptr && wq != nullptr &&
                  wk != nullptr && (v_other == nullptr || mix != nullptr),
              "conv_head_norm_append: heads %d / %d, head sizes %d / %d, taps %d", H, G, d, dv, taps);
  DSB_REQUIRE(q_row >= d && k_row >= d && v_row >= dv, "conv_head_norm_append: row widths %d / %d / %d below the head sizes %d / %d", q_row, k_row, v_row, d, dv);
  auto mult4 = [](long long v) { return v % 4 == 0; };
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = mult4(d) && mult4(dv) && mult4(ld) && mult4(col0) && mult4(q_ld) && mult4(q_row) && mult4(k_row) && mult4(v_row) && mult4(k_block_stride) &&
                   mult4(v_block_stride) && al16(proj) && al16(bias) && al16(conv_w) && al16(wq) && al16(wk) && al16(state) && al16(k_cache) && al16(v_cache) && al16(q_out) && al16(v_other) && al16(v_own);
  // several slots per warp when a lane's first group of channels covers a head and there are enough tokens to fill the GPU all the same
  const bool many = (d > dv ? d : dv) <= (vec ? 128 : 32) && static_cast<long long>(n_tokens) * (H + 2 * G) >= 16384;
  const int sl = many ? 4 : 1;
  const long long warps = static_cast<long long>(n_tokens) * ((H + 2 * G + sl - 1) / sl);
  const int wpb = 8;
  const int grid = static_cast<int>((warps + wpb - 1) / wpb);
#define LAUNCH(T, V, S)                                                                                                                                     \
  conv_head_norm_append_kernel<T, V, S><<<grid, wpb * 32, 0, stream>>>((const T*)proj, ld, col0, bias, conv_w, wq, wk, (const T*)state, (const int4*)seq_desc, tok_seq, \
                                                                       tok_pos, block_table, bt_stride, block_size, (T*)k_cache, k_block_stride, (T*)v_cache,         \
                                                                       v_block_stride, (T*)q_out, q_ld, (const T*)v_other, mix, (T*)v_own, n_tokens, H, G, d, dv,     \
                                                                       taps, eps, q_row, k_row, v_row)
#define PICK(T)                                                  \
  do {                                                           \
    if (vec && many) LAUNCH(T, 4, 4);                            \
    else if (vec) LAUNCH(T, 4, 1);                               \
    else if (many) LAUNCH(T, 1, 4);                              \
    else LAUNCH(T, 1, 1);                                        \
  } while (0)
  if (dtype == 0) PICK(bf16);
  else PICK(float);
#undef PICK
#undef LAUNCH
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// build: precise-math
// Ragged-batch kernels for decoders that keep an fp32 residual stream, cache one low-rank latent per token instead of
// per-head keys and values, and route tokens with a grouped, bias-corrected top-k router.  Every kernel takes its sizes
// as arguments (no size is assumed to be a power of two or a multiple of a vector width) and exists for 16-bit (bf16)
// and 32-bit activations; sums, norms, softmax and router scores are always fp32.
//
//   embed_sinusoid        token table lookup + sinusoidal position vector -> fp32 residual
//   sandwich_norm         x += rms(y) * (wb + ob)   and / or   out = rms(x) * (w + o)      (one pass per token row)
//   stream_group_norm     x += y0 + y1 + y2         and / or   out = rms-in-groups(x) * w      (blocks whose sublayers share one norm)
//   latent_norm_append    plain-weight RMS norm of the query latent and of the key/value latent of every token; the
//                         key/value latent goes straight into its slot of the paged latent cache
//   latent_attention      softmax(q_abs . c) c over the paged latent cache: all heads of a token share the cached rows
//                         (keys and values are the same row), causal, split along the keys + merge
//   sigmoid_gate_mul      a *= sigmoid(g)
//   grouped_topk_gating   softmax scores (+ correction for the selection only), best `keep` of `groups` contiguous expert groups by
//                         their largest selection score, top-k of the surviving experts, weights = uncorrected scores
//   moe_scatter / moe_gather   expert-sorted copies and the weighted fp32 combine, any width
//   clamped_swish_gate    min(g, L) * sigmoid(alpha * min(g, L)) * (clamp(u, -L, L) + shift)
//   moe_gemm_rows         grouped expert GEMM on CUDA cores (fp32 accumulation) for shapes / dtypes the tensor-core
//                         grouped GEMM does not take
//   softcap               logits = cap * tanh(logits / cap)
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../common/host.h"

namespace dsb {
namespace latent {

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
// sum over the block; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // red may still be read from an earlier call
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

// ---------------------------------------------------------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_sinusoid_kernel(const long long* __restrict__ ids, const TW* __restrict__ table, const int* __restrict__ tok_pos,
                                      const double* __restrict__ freq, float* __restrict__ out, int dim, float scale) {
  const int t = blockIdx.x;
  const long long id = ids[t];
  const TW* row = table + id * dim;
  float* o = out + static_cast<size_t>(t) * dim;
  if (freq == nullptr) {  // no position vector: the table row alone starts the stream (tok_pos may be null)
    for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = to_f(row[i]) * scale;
    return;
  }
  const double p = static_cast<double>(tok_pos[t]);
  for (int i = threadIdx.x; 2 * i < dim; i += blockDim.x) {
    double s, c;
    sincos(p * freq[i], &s, &c);
    o[2 * i] = to_f(row[2 * i]) * scale + static_cast<float>(s);
    if (2 * i + 1 < dim) o[2 * i + 1] = to_f(row[2 * i + 1]) * scale + static_cast<float>(c);
  }
}

// --------------------------------------------------------------------------------------------------------------------- norms
// Row r of the fp32 residual (row rows[r] when `rows` is given; then nothing is written back to x):
//   y given:   x <- x + ym * y / sqrt(mean(y^2) + eps) * (wb + ob)
//   w given:   out <- x / sqrt(mean(x^2) + eps) * (w + o)      (and the same values unrounded into out32 when that is given)
//   plain:     out <- x                                        (the stream itself in out's dtype: blocks whose sublayers read it unnormed)
template <typename TY, typename TO>
__global__ void sandwich_norm_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ wb, float ob, float ym,
                                     const float* __restrict__ w, float o, TO* __restrict__ out, float* __restrict__ out32,
                                     const int* __restrict__ rows, int dim, float eps, int plain) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  float* xr = x + static_cast<size_t>(rows ? rows[r] : r) * dim;
  float sx = 0.f;
  if (y != nullptr) {
    const TY* yr = y + static_cast<size_t>(r) * dim;
    float sy = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float v = to_f(yr[c]);
      sy += v * v;
    }
    sy = block_sum(sy, red);
    const float inv = ym / sqrtf(sy / static_cast<float>(dim) + eps);
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float v = xr[c] + to_f(yr[c]) * inv * (wb[c] + ob);
      xr[c] = v;  // read back below by this same thread only
      sx += v * v;
    }
  } else if (w != nullptr) {
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float v = xr[c];
      sx += v * v;
    }
  }
  if (plain) {
    TO* orow = out + static_cast<size_t>(r) * dim;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) orow[c] = from_f<TO>(xr[c]);
    return;
  }
  if (w == nullptr) return;
  sx = block_sum(sx, red);
  const float inv = 1.f / sqrtf(sx / static_cast<float>(dim) + eps);
  TO* orow = out + static_cast<size_t>(r) * dim;
  float* o32 = out32 ? out32 + static_cast<size_t>(r) * dim : nullptr;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    const float v = xr[c] * inv * (w[c] + o);
    orow[c] = from_f<TO>(v);
    if (o32) o32[c] = v;
  }
}

// The same for dim % 4 == 0 and dim <= 4 * SN_MAXV * blockDim: 16-byte (fp32) / 8-byte (bf16) accesses, the row is read from global
// memory once and kept in registers between the statistics and the scaling.
constexpr int SN_MAXV = 4;
struct alignas(8) bf16x4 { __nv_bfloat162 a, b; };
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

template <typename TY, typename TO>
__global__ void sandwich_norm_vec_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ wb, float ob, float ym,
                                         const float* __restrict__ w, float o, TO* __restrict__ out, float* __restrict__ out32,
                                         const int* __restrict__ rows, int dim, float eps, int plain) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  float* xr = x + static_cast<size_t>(rows ? rows[r] : r) * dim;
  const int nv = dim >> 2;
  float4 xv[SN_MAXV];
  float sx = 0.f;
  if (y != nullptr) {
    const TY* yr = y + static_cast<size_t>(r) * dim;
    float4 yv[SN_MAXV];
    float sy = 0.f;
#pragma unroll
    for (int i = 0; i < SN_MAXV; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < nv) {
        yv[i] = load4(yr + 4 * c);
        xv[i] = load4(xr + 4 * c);
        sy += yv[i].x * yv[i].x + yv[i].y * yv[i].y + yv[i].z * yv[i].z + yv[i].w * yv[i].w;
      }
    }
    sy = block_sum(sy, red);
    const float inv = ym / sqrtf(sy / static_cast<float>(dim) + eps);
#pragma unroll
    for (int i = 0; i < SN_MAXV; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < nv) {
        const float4 g = load4(wb + 4 * c);
        xv[i].x += yv[i].x * inv * (g.x + ob);
        xv[i].y += yv[i].y * inv * (g.y + ob);
        xv[i].z += yv[i].z * inv * (g.z + ob);
        xv[i].w += yv[i].w * inv * (g.w + ob);
        store4(xr + 4 * c, xv[i]);
        sx += xv[i].x * xv[i].x + xv[i].y * xv[i].y + xv[i].z * xv[i].z + xv[i].w * xv[i].w;
      }
    }
  } else if (w != nullptr || plain) {
#pragma unroll
    for (int i = 0; i < SN_MAXV; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < nv) {
        xv[i] = load4(xr + 4 * c);
        sx += xv[i].x * xv[i].x + xv[i].y * xv[i].y + xv[i].z * xv[i].z + xv[i].w * xv[i].w;
      }
    }
  }
  TO* orow = out + static_cast<size_t>(r) * dim;
  if (plain) {
#pragma unroll
    for (int i = 0; i < SN_MAXV; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < nv) store4(orow + 4 * c, xv[i]);
    }
    return;
  }
  if (w == nullptr) return;
  sx = block_sum(sx, red);
  const float inv = 1.f / sqrtf(sx / static_cast<float>(dim) + eps);
#pragma unroll
  for (int i = 0; i < SN_MAXV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nv) {
      const float4 g = load4(w + 4 * c);
      const float4 v = make_float4(xv[i].x * inv * (g.x + o), xv[i].y * inv * (g.y + o), xv[i].z * inv * (g.z + o), xv[i].w * inv * (g.w + o));
      store4(orow + 4 * c, v);
      if (out32) store4(out32 + static_cast<size_t>(r) * dim + 4 * c, v);
    }
  }
}

// Blocks whose sublayers all read ONE norm of the stream and whose outputs are summed into it: output row r works on row src = rows[r] of the
// fp32 residual and of the branches (src = r without `rows`).  First the finished sublayers' outputs join the stream,
//   x <- x + y0 + y1 + y2        (y0, y1 in the activation dtype, y2 fp32; each may be null; the sum is fp32; written back only without `rows`),
// then, when w is given, the row is split into `groups` equal consecutive parts, each divided by its own sqrt(mean(part^2) + eps), and
// the whole multiplied by w: out in the activation dtype, out32 (optional) the same values before rounding.  The summed row is kept in
// shared memory (dim floats) between the two steps.
template <typename TY, typename TO>
__global__ void stream_group_norm_kernel(float* __restrict__ x, const TY* __restrict__ y0, const TY* __restrict__ y1, const float* __restrict__ y2,
                                         const float* __restrict__ w, TO* __restrict__ out, float* __restrict__ out32,
                                         const int* __restrict__ rows, int dim, int groups, float eps) {
  extern __shared__ float rowbuf[];
  __shared__ float red[33];
  const int r = blockIdx.x;
  const size_t so = static_cast<size_t>(rows ? rows[r] : r) * dim, o = static_cast<size_t>(r) * dim;
  const bool add = y0 != nullptr || y1 != nullptr || y2 != nullptr;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float v = x[so + c];
    if (y0) v += to_f(y0[so + c]);
    if (y1) v += to_f(y1[so + c]);
    if (y2) v += y2[so + c];
    if (add && rows == nullptr) x[so + c] = v;
    rowbuf[c] = v;  // read back below by this same thread only
  }
  if (w == nullptr) return;
  const int per = dim / groups;
  for (int g = 0; g < groups; ++g) {
    float s = 0.f;
    for (int c = threadIdx.x; c < per; c += blockDim.x) {
      const float v = rowbuf[g * per + c];
      s += v * v;
    }
    s = block_sum(s, red);
    const float inv = 1.f / sqrtf(s / static_cast<float>(per) + eps);
    for (int c = threadIdx.x; c < per; c += blockDim.x) {
      const float v = rowbuf[g * per + c] * inv * w[g * per + c];
      out[o + g * per + c] = from_f<TO>(v);
      if (out32) out32[o + g * per + c] = v;
    }
  }
}

// The same for parts that are multiples of 128 values and dim <= 4 * SN_MAXV * blockDim: 16-byte accesses, the row is read once and kept
// in registers; the 128 consecutive values a warp holds per step lie in one part, so a part's sum is a warp reduction plus one
// shared-memory add per warp and step.
constexpr int GN_MAXG = 32;
template <typename TY, typename TO>
__global__ void stream_group_norm_vec_kernel(float* __restrict__ x, const TY* __restrict__ y0, const TY* __restrict__ y1,
                                             const float* __restrict__ y2, const float* __restrict__ w, TO* __restrict__ out,
                                             float* __restrict__ out32, const int* __restrict__ rows, int dim, int groups, float eps) {
  __shared__ float gsum[GN_MAXG];
  const int r = blockIdx.x, lane = threadIdx.x & 31;
  const size_t so = static_cast<size_t>(rows ? rows[r] : r) * dim, o = static_cast<size_t>(r) * dim;
  const int nv = dim >> 2, per = dim / groups;
  const bool add = y0 != nullptr || y1 != nullptr || y2 != nullptr;
  if (threadIdx.x < groups) gsum[threadIdx.x] = 0.f;
  __syncthreads();
  float4 xv[SN_MAXV];
#pragma unroll
  for (int i = 0; i < SN_MAXV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    float s = 0.f;
    if (c < nv) {
      float4 v = load4(x + so + 4 * c);
      if (y0) { const float4 a = load4(y0 + so + 4 * c); v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w; }
      if (y1) { const float4 a = load4(y1 + so + 4 * c); v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w; }
      if (y2) { const float4 a = load4(y2 + so + 4 * c); v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w; }
      if (add && rows == nullptr) store4(x + so + 4 * c, v);
      xv[i] = v;
      s = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    if (w != nullptr) {
      s = warp_sum(s);
      const int c0 = (threadIdx.x - lane) + i * blockDim.x;  // the warp's first 4-vector of this step
      if (lane == 0 && c0 < nv) atomicAdd(&gsum[(4 * c0) / per], s);
    }
  }
  if (w == nullptr) return;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < SN_MAXV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nv) {
      const float inv = 1.f / sqrtf(gsum[(4 * c) / per] / static_cast<float>(per) + eps);
      const float4 g = load4(w + 4 * c);
      const float4 v = make_float4(xv[i].x * inv * g.x, xv[i].y * inv * g.y, xv[i].z * inv * g.z, xv[i].w * inv * g.w);
      store4(out + o + 4 * c, v);
      if (out32) store4(out32 + o + 4 * c, v);
    }
  }
}

// One warp per (token, which): which = 0 normalises lat[t, :nq] with wq into cq[t, :]; which = 1 normalises
// lat[t, nq : nq + nkv] with wkv into the token's row of the paged cache [blocks, block_size, nkv].
template <typename T>
__global__ void latent_norm_append_kernel(const T* __restrict__ lat, int ld, const float* __restrict__ wq, const float* __restrict__ wkv,
                                          T* __restrict__ cq, T* __restrict__ cache, const int* __restrict__ tok_seq,
                                          const int* __restrict__ tok_pos, const int* __restrict__ block_table, int bt_stride,
                                          int block_size, int cache_ld, int n_tokens, int nq, int nkv, float eps) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int t = gw >> 1, which = gw & 1;
  if (t >= n_tokens) return;
  const int n = which ? nkv : nq;
  if (n == 0) return;
  const T* src = lat + static_cast<size_t>(t) * ld + (which ? nq : 0);
  const float* w = which ? wkv : wq;
  T* dst;
  if (which) {
    const int pos = tok_pos[t];
    const int blk = block_table[static_cast<size_t>(tok_seq[t]) * bt_stride + pos / block_size];
    dst = cache + (static_cast<size_t>(blk) * block_size + pos % block_size) * cache_ld;
  } else {
    dst = cq + static_cast<size_t>(t) * nq;
  }
  float s = 0.f;
  for (int c = lane; c < n; c += 32) {
    const float v = to_f(src[c]);
    s += v * v;
  }
  s = warp_sum(s);
  const float inv = 1.f / sqrtf(s / static_cast<float>(n) + eps);
  for (int c = lane; c < n; c += 32) dst[c] = from_f<T>(to_f(src[c]) * inv * w[c]);
}

// ----------------------------------------------------------------------------------------------------------- latent attention
// Grid (token, split, head group of 8).  4 warps; warp w owns heads hg*8 + w and hg*8 + w + 4 and handles both in one pass, so that
// every latent value read from shared memory feeds two FMAs.  Keys come in tiles of 32 rows of the latent cache, converted to fp32 in
// shared memory (row stride R + 1); lane j scores key j of the tile, then lane l accumulates output columns l, l + 32, ...
// RI = ceil(R / 32) columns per lane.
constexpr int LA_KT = 32;
constexpr int LA_HPC = 8;  // heads per CTA

template <typename TC, typename TQ, int RI>
__global__ void __launch_bounds__(128)
latent_attention_kernel(const TQ* __restrict__ q, long long q_tok_stride, long long q_head_stride, const TC* __restrict__ cache,
                        float* __restrict__ out, long long o_tok_stride, long long o_head_stride, float* __restrict__ part_ml,
                        float* __restrict__ part_acc, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                        const int* __restrict__ block_table, int bt_stride, int block_size, int H, int R, float scale, int n_splits) {
  extern __shared__ float smem[];
  const int t = blockIdx.x, split = blockIdx.y, hg = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int RS = R + 1;
  float* q_s = smem;                       // [LA_HPC][R]
  float* c_s = q_s + LA_HPC * R;           // [LA_KT][RS]
  float* p_s = c_s + LA_KT * RS;           // [4][2][LA_KT]
  const int seq = tok_seq[t], pos = tok_pos[t];
  const int n_keys = pos + 1;
  int chunk = (n_keys + n_splits - 1) / n_splits;
  chunk = (chunk + LA_KT - 1) / LA_KT * LA_KT;
  const int k0 = split * chunk, k1 = min(n_keys, k0 + chunk);
  const int h_base = hg * LA_HPC;
  for (int i = threadIdx.x; i < LA_HPC * R; i += blockDim.x) {
    const int h = h_base + i / R, r = i % R;
    q_s[i] = h < H ? to_f(q[t * q_tok_stride + h * q_head_stride + r]) * scale : 0.f;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float acc[2][RI];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int i = 0; i < RI; ++i) acc[a][i] = 0.f;
  const int* bt = block_table + static_cast<size_t>(seq) * bt_stride;
  for (int kt = k0; kt < k1; kt += LA_KT) {
    __syncthreads();  // the previous tile is consumed (and q_s is written)
    for (int i = threadIdx.x; i < LA_KT * R; i += blockDim.x) {
      const int j = i / R, r = i % R;
      const int k = kt + j;
      float v = 0.f;
      if (k < k1) {
        const int blk = bt[k / block_size];
        v = to_f(cache[(static_cast<size_t>(blk) * block_size + k % block_size) * R + r]);
      }
      c_s[j * RS + r] = v;
    }
    __syncthreads();
    const bool valid = kt + lane < k1;
    // both heads of the warp in one pass over the tile: every latent value read from shared memory feeds two FMAs
    if (h_base + warp < H) {
      const float* q0 = q_s + warp * R;
      const float* q1 = q_s + (warp + 4) * R;  // zeros when the head does not exist
      const float* cj = c_s + lane * RS;
      float s0 = 0.f, s1 = 0.f;
      for (int r = 0; r < R; ++r) {
        const float cv = cj[r];
        s0 = fmaf(q0[r], cv, s0);
        s1 = fmaf(q1[r], cv, s1);
      }
      s0 = valid ? s0 : -INFINITY;
      s1 = valid ? s1 : -INFINITY;
      const float mn0 = fmaxf(m[0], warp_max(s0)), mn1 = fmaxf(m[1], warp_max(s1));  // finite: every tile holds a visible key
      const float p0 = valid ? expf(s0 - mn0) : 0.f, p1 = valid ? expf(s1 - mn1) : 0.f;
      const float corr0 = expf(m[0] - mn0), corr1 = expf(m[1] - mn1);  // exp(-inf) = 0 on the first tile
      l[0] = l[0] * corr0 + warp_sum(p0);
      l[1] = l[1] * corr1 + warp_sum(p1);
      m[0] = mn0;
      m[1] = mn1;
      float* pw = p_s + warp * 2 * LA_KT;  // [key][2 heads]
      pw[2 * lane] = p0;
      pw[2 * lane + 1] = p1;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < RI; ++i) {
        acc[0][i] *= corr0;
        acc[1][i] *= corr1;
      }
      for (int j = 0; j < LA_KT; ++j) {
        const float2 pj = *reinterpret_cast<const float2*>(pw + 2 * j);
        const float* crow = c_s + j * RS;
#pragma unroll
        for (int i = 0; i < RI; ++i) {
          const int r = lane + 32 * i;
          if (r < R) {
            const float cv = crow[r];
            acc[0][i] = fmaf(pj.x, cv, acc[0][i]);
            acc[1][i] = fmaf(pj.y, cv, acc[1][i]);
          }
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int h = h_base + warp + 4 * a;
    if (h >= H) continue;
    if (n_splits == 1) {
      const float inv = 1.f / l[a];
#pragma unroll
      for (int i = 0; i < RI; ++i) {
        const int r = lane + 32 * i;
        if (r < R) out[t * o_tok_stride + h * o_head_stride + r] = acc[a][i] * inv;
      }
    } else {
      const size_t slot = (static_cast<size_t>(t) * n_splits + split) * H + h;
      if (lane == 0) {
        part_ml[2 * slot] = m[a];
        part_ml[2 * slot + 1] = l[a];
      }
#pragma unroll
      for (int i = 0; i < RI; ++i) {
        const int r = lane + 32 * i;
        if (r < R) part_acc[slot * R + r] = acc[a][i];
      }
    }
  }
}

// one warp per (token, head): combine the splits' (max, sum, unnormalised output)
__global__ void latent_attention_merge_kernel(const float* __restrict__ part_ml, const float* __restrict__ part_acc, float* __restrict__ out,
                                              long long o_tok_stride, long long o_head_stride, int n_tokens, int H, int R, int n_splits) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (gw >= n_tokens * H) return;
  const int t = gw / H, h = gw % H;
  float mx = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, part_ml[2 * ((static_cast<size_t>(t) * n_splits + s) * H + h)]);
  float l = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const size_t slot = (static_cast<size_t>(t) * n_splits + s) * H + h;
    const float ms = part_ml[2 * slot];
    if (ms != -INFINITY) l += part_ml[2 * slot + 1] * expf(ms - mx);
  }
  const float inv = 1.f / l;
  for (int r = lane; r < R; r += 32) {
    float o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const size_t slot = (static_cast<size_t>(t) * n_splits + s) * H + h;
      const float ms = part_ml[2 * slot];
      if (ms != -INFINITY) o = fmaf(part_acc[slot * R + r], expf(ms - mx), o);
    }
    out[t * o_tok_stride + h * o_head_stride + r] = o * inv;
  }
}

// ---------------------------------------------------------------------------------------------------------------- elementwise
template <typename T>
__global__ void sigmoid_gate_mul_kernel(T* __restrict__ a, long long a_ld, const T* __restrict__ g, long long g_ld, int cols, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols;
    const int c = static_cast<int>(i % cols);
    const float gv = to_f(g[r * g_ld + c]);
    a[r * a_ld + c] = from_f<T>(to_f(a[r * a_ld + c]) * (1.f / (1.f + expf(-gv))));
  }
}

// out[t, h * dv + c] = a[h, t, c] * sigmoid(g[t, h * dv + c]): the per-head results of a batched GEMM ([H, T, dv], contiguous) become the
// token-major concatenation of heads, gated, in one pass.  VEC: dv % 4 == 0 and g_ld % 4 == 0.
template <typename T, bool VEC>
__global__ void gate_heads_kernel(const T* __restrict__ a, const T* __restrict__ g, long long g_ld, T* __restrict__ out, int n_tokens, int H, int dv) {
  constexpr int V = VEC ? 4 : 1;
  const int row = H * dv;
  const long long n = static_cast<long long>(n_tokens) * row / V;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * V;
    const long long t = e / row;
    const int rem = static_cast<int>(e % row), h = rem / dv, c = rem % dv;
    const T* src = a + (static_cast<long long>(h) * n_tokens + t) * dv + c;
    if constexpr (VEC) {
      const float4 av = load4(src), gv = load4(g + t * g_ld + rem);
      store4(out + e, make_float4(av.x / (1.f + expf(-gv.x)), av.y / (1.f + expf(-gv.y)), av.z / (1.f + expf(-gv.z)), av.w / (1.f + expf(-gv.w))));
    } else {
      out[e] = from_f<T>(to_f(*src) / (1.f + expf(-to_f(g[t * g_ld + rem]))));
    }
  }
}

// gu [rows, 2 F] = (gate | up) -> out [rows, F]
template <typename T>
__global__ void clamped_swish_gate_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int F, float alpha, float limit,
                                          float shift) {
  const long long n = rows * F;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / F;
    const int c = static_cast<int>(i % F);
    const float g = fminf(to_f(gu[r * 2 * F + c]), limit);
    const float u = fminf(fmaxf(to_f(gu[r * 2 * F + F + c]), -limit), limit);
    out[i] = from_f<T>(g * (1.f / (1.f + expf(-alpha * g))) * (u + shift));
  }
}

// F % 4 == 0: four outputs per thread and step
template <typename T>
__global__ void clamped_swish_gate_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int F, float alpha, float limit,
                                              float shift) {
  const int fv = F >> 2;
  const long long n = rows * fv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / fv;
    const int c = static_cast<int>(i % fv) * 4;
    const float4 g4 = load4(gu + r * 2 * F + c), u4 = load4(gu + r * 2 * F + F + c);
    const float gs[4] = {g4.x, g4.y, g4.z, g4.w}, us[4] = {u4.x, u4.y, u4.z, u4.w};
    float o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float g = fminf(gs[k], limit);
      const float u = fminf(fmaxf(us[k], -limit), limit);
      o[k] = g * (1.f / (1.f + expf(-alpha * g))) * (u + shift);
    }
    store4(out + r * F + c, make_float4(o[0], o[1], o[2], o[3]));
  }
}

// The same on column ranges: gate at column gate_col0 and up at column up_col0 of gu [rows, ld], result into out [rows, out_ld] (a view)
template <typename T>
__global__ void clamped_swish_gate_cols_kernel(const T* __restrict__ gu, long long ld, int gate_col0, int up_col0, T* __restrict__ out,
                                               long long out_ld, long long rows, int F, float alpha, float limit, float shift) {
  const long long n = rows * F;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / F;
    const int c = static_cast<int>(i % F);
    const float g = fminf(to_f(gu[r * ld + gate_col0 + c]), limit);
    const float u = fminf(fmaxf(to_f(gu[r * ld + up_col0 + c]), -limit), limit);
    out[r * out_ld + c] = from_f<T>(g * (1.f / (1.f + expf(-alpha * g))) * (u + shift));
  }
}

// ... with F, both column offsets and both row strides multiples of 4 and 16-byte (fp32) / 8-byte (bf16) aligned bases: four outputs per thread
template <typename T>
__global__ void clamped_swish_gate_cols_vec_kernel(const T* __restrict__ gu, long long ld, int gate_col0, int up_col0, T* __restrict__ out,
                                                   long long out_ld, long long rows, int F, float alpha, float limit, float shift) {
  const int fv = F >> 2;
  const long long n = rows * fv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / fv;
    const int c = static_cast<int>(i % fv) * 4;
    const float4 g4 = load4(gu + r * ld + gate_col0 + c), u4 = load4(gu + r * ld + up_col0 + c);
    const float gs[4] = {g4.x, g4.y, g4.z, g4.w}, us[4] = {u4.x, u4.y, u4.z, u4.w};
    float o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float g = fminf(gs[k], limit);
      const float u = fminf(fmaxf(us[k], -limit), limit);
      o[k] = g * (1.f / (1.f + expf(-alpha * g))) * (u + shift);
    }
    store4(out + r * out_ld + c, make_float4(o[0], o[1], o[2], o[3]));
  }
}

__global__ void softcap_kernel(float* __restrict__ x, long long ld, int cols, long long n, float cap) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float* p = x + (i / cols) * ld + (i % cols);
    *p = cap * tanhf(*p / cap);
  }
}

// ---------------------------------------------------------------------------------------------------------------------- router
// One warp per token.  Shared memory per warp: E selection scores + G group scores.  Ties go to the lower index.
__global__ void grouped_topk_gating_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int* __restrict__ expert_counts,
                                           float* __restrict__ scores, int* __restrict__ assignments, int* __restrict__ offsets, int n_tokens,
                                           int E, int K, int G, int keep, int normalize, int sigmoid_scores) {
  extern __shared__ float smem[];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok = blockIdx.x * (blockDim.x >> 5) + wib;
  if (tok >= n_tokens) return;
  float* choice = smem + static_cast<size_t>(wib) * (E + G);
  float* gsc = choice + E;
  const float* lg = logits + static_cast<size_t>(tok) * E;
  float mx = 0.f, inv = 1.f;
  if (!sigmoid_scores) {
    mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(lg[e] - mx);
    sum = warp_sum(sum);
    inv = 1.f / sum;
  }
  // score of expert e: its softmax probability, or (sigmoid_scores) 1 / (1 + exp(-logit)) on its own
  for (int e = lane; e < E; e += 32)
    choice[e] = (sigmoid_scores ? 1.f / (1.f + expf(-lg[e])) : expf(lg[e] - mx) * inv) + (correction ? correction[e] : 0.f);
  __syncwarp();
  if (G > 1 && keep < G) {
    const int per = E / G;
    for (int g = 0; g < G; ++g) {
      float v = -INFINITY;
      for (int e = lane; e < per; e += 32) v = fmaxf(v, choice[g * per + e]);
      v = warp_max(v);
      if (lane == 0) gsc[g] = v;
    }
    __syncwarp();
    // the `keep` best groups survive: group g is dropped when at least `keep` groups beat it (higher score, or equal and lower index)
    for (int g = 0; g < G; ++g) {
      int better = 0;
      const float mine = gsc[g];
      for (int o = lane; o < G; o += 32) better += (gsc[o] > mine || (gsc[o] == mine && o < g)) ? 1 : 0;
      better = static_cast<int>(warp_sum(static_cast<float>(better)) + 0.5f);
      if (better >= keep)
        for (int e = lane; e < per; e += 32) choice[g * per + e] = -INFINITY;
      __syncwarp();
    }
  }
  float top_sum = 0.f;
  float my_score = 0.f;   // lane k keeps the k-th pick
  int my_expert = -1;
  for (int k = 0; k < K; ++k) {
    float best = -INFINITY;
    int best_e = -1;
    for (int e = lane; e < E; e += 32) {
      const float v = choice[e];
      if (v > best || (best_e < 0 && v > -INFINITY)) { best = v; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (oe >= 0 && (best_e < 0 || ob > best || (ob == best && oe < best_e))) { best = ob; best_e = oe; }
    }
    float s = 0.f;
    if (best_e >= 0) {
      s = sigmoid_scores ? 1.f / (1.f + expf(-lg[best_e])) : expf(lg[best_e] - mx) * inv;
      if (lane == 0) choice[best_e] = -INFINITY;
    }
    __syncwarp();
    top_sum += s;
    if (lane == k) { my_score = s; my_expert = best_e; }
  }
  if (lane < K) {
    const int e = my_expert >= 0 ? my_expert : 0;  // fewer selectable experts than K cannot happen for valid configurations
    assignments[tok * K + lane] = e;
    scores[tok * K + lane] = normalize ? my_score / top_sum : my_score;
    offsets[tok * K + lane] = atomicAdd(&expert_counts[e], 1);
  }
}

__global__ void expert_cumsum_kernel(const int* __restrict__ counts, long long* __restrict__ cumsum, int E) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    long long s = 0;
    for (int e = 0; e < E; ++e) { s += counts[e]; cumsum[e] = s; }
  }
}

template <typename T, bool VEC>
__global__ void moe_scatter_kernel(const T* __restrict__ x, const int* __restrict__ assignments, const int* __restrict__ offsets,
                                   const long long* __restrict__ cumsum, T* __restrict__ moe_in, int* __restrict__ mapped_slots, int dim, int K,
                                   const float* __restrict__ row_scale) {
  const int t = blockIdx.x;
  for (int k = 0; k < K; ++k) {
    const int e = assignments[t * K + k];
    const long long slot = (e == 0 ? 0 : cumsum[e - 1]) + offsets[t * K + k];
    if (threadIdx.x == 0) mapped_slots[t * K + k] = static_cast<int>(slot);
    const float sc = row_scale ? row_scale[t * K + k] : 1.f;  // experts that weigh their input: the copy is scaled (in fp32, then rounded)
    if constexpr (VEC) {
      for (int c = threadIdx.x * 4; c < dim; c += blockDim.x * 4) {
        float4 v = load4(x + static_cast<size_t>(t) * dim + c);
        if (row_scale) v = make_float4(v.x * sc, v.y * sc, v.z * sc, v.w * sc);
        store4(moe_in + slot * dim + c, v);
      }
    } else {
      for (int c = threadIdx.x; c < dim; c += blockDim.x)
        moe_in[slot * dim + c] = row_scale ? from_f<T>(to_f(x[static_cast<size_t>(t) * dim + c]) * sc) : x[static_cast<size_t>(t) * dim + c];
    }
  }
}

template <typename T, bool VEC>
__global__ void moe_gather_kernel(const T* __restrict__ moe_out, const float* __restrict__ scores, const int* __restrict__ mapped_slots,
                                  float* __restrict__ out, int dim, int K, const int* __restrict__ assignments, int n_real,
                                  const float* __restrict__ identity_src) {
  const int t = blockIdx.x;
  // experts n_real and above are identity experts: their output is the token's own row of identity_src (fp32)
  if constexpr (VEC) {
    for (int c = threadIdx.x * 4; c < dim; c += blockDim.x * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < K; ++k) {
        const float s = scores ? scores[t * K + k] : 1.f;
        const bool same = assignments != nullptr && assignments[t * K + k] >= n_real;
        const float4 v = same ? load4(identity_src + static_cast<size_t>(t) * dim + c)
                              : load4(moe_out + static_cast<size_t>(mapped_slots[t * K + k]) * dim + c);
        acc.x = fmaf(s, v.x, acc.x); acc.y = fmaf(s, v.y, acc.y); acc.z = fmaf(s, v.z, acc.z); acc.w = fmaf(s, v.w, acc.w);
      }
      store4(out + static_cast<size_t>(t) * dim + c, acc);
    }
  } else {
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      float acc = 0.f;
      for (int k = 0; k < K; ++k) {
        const bool same = assignments != nullptr && assignments[t * K + k] >= n_real;
        const float v = same ? identity_src[static_cast<size_t>(t) * dim + c] : to_f(moe_out[static_cast<size_t>(mapped_slots[t * K + k]) * dim + c]);
        acc = fmaf(scores ? scores[t * K + k] : 1.f, v, acc);
      }
      out[static_cast<size_t>(t) * dim + c] = acc;
    }
  }
}

// ------------------------------------------------------------------------------------------------- grouped GEMM on CUDA cores
// out[r, n] = sum_k x[r, k] * w[e(r), n, k] for rows sorted by expert (inclusive row cumsum per expert on the device).
// Tiles of 32 rows x 64 columns that never straddle experts; tile b of the grid is located by walking the cumsum.
constexpr int GM = 32, GN = 64, GK = 16;
template <typename T>
__global__ void __launch_bounds__(256)
moe_gemm_rows_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out, const long long* __restrict__ cumsum, int E,
                     int N, int K) {
  __shared__ float xs[GK][GM + 1];
  __shared__ float ws[GK][GN + 1];
  __shared__ int s_info[3];
  if (threadIdx.x == 0) {
    int b = blockIdx.x, e = 0;
    long long start = 0;
    s_info[0] = -1;
    for (; e < E; ++e) {
      const long long end = cumsum[e];
      const int tiles = static_cast<int>((end - start + GM - 1) / GM);
      if (b < tiles) {
        s_info[0] = e;
        s_info[1] = static_cast<int>(start) + b * GM;
        s_info[2] = static_cast<int>(end);
        break;
      }
      b -= tiles;
      start = end;
    }
  }
  __syncthreads();
  const int e = s_info[0];
  if (e < 0) return;
  const int r0 = s_info[1], r_end = s_info[2], n0 = blockIdx.y * GN;
  const T* we = w + static_cast<size_t>(e) * N * K;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // thread computes rows ty*2 .. +1, columns tx*4 .. +3
  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  for (int k0 = 0; k0 < K; k0 += GK) {
    for (int i = threadIdx.x; i < GM * GK; i += 256) {
      const int r = i / GK, k = i % GK;
      xs[k][r] = (r0 + r < r_end && k0 + k < K) ? to_f(x[static_cast<size_t>(r0 + r) * K + k0 + k]) : 0.f;
    }
    for (int i = threadIdx.x; i < GN * GK; i += 256) {
      const int n = i / GK, k = i % GK;
      ws[k][n] = (n0 + n < N && k0 + k < K) ? to_f(we[static_cast<size_t>(n0 + n) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      const float a0 = xs[k][ty * 2], a1 = xs[k][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = ws[k][tx * 4 + j];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r0 + ty * 2 + i;
    if (r >= r_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[static_cast<size_t>(r) * N + n] = from_f<T>(acc[i][j]);
    }
  }
}

}  // namespace latent
}  // namespace dsb

using namespace dsb;
using namespace dsb::latent;

static inline int grid_for(long long n, int block) {
  long long g = (n + block - 1) / block;
  return static_cast<int>(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

// out[t, :] = table[ids[t], :] + sinusoid(tok_pos[t]): entry 2i = sin(p f_i), entry 2i + 1 = cos(p f_i); `freq` holds the
// ceil(dim / 2) frequencies as doubles on the device, or is null for no position vector (tok_pos is then unused).
// table_dtype: 0 = bf16, 1 = fp32.  out is fp32.  The table row is multiplied by `scale` (in fp32) before the position vector is added.
DSB_EXPORT int dsb200_embed_sinusoid(const long long* ids, const void* table, int table_dtype, const int* tok_pos, const double* freq,
                                     float* out, int n_tokens, int dim, float scale, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  if (table_dtype == 0)
    embed_sinusoid_kernel<bf16><<<n_tokens, 128, 0, stream>>>(ids, (const bf16*)table, tok_pos, freq, out, dim, scale);
  else
    embed_sinusoid_kernel<float><<<n_tokens, 128, 0, stream>>>(ids, (const float*)table, tok_pos, freq, out, dim, scale);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// Per row of the fp32 residual x [n_rows, dim] (row rows[r] when `rows` is given): if y: x += y_mult * rms_norm(y) * (wb + ob); if w:
// out = rms_norm(x) * (w + o); if plain_out (and no w): out = x.  y and out are bf16 (dtype 0) or fp32 (dtype 1); the weights are fp32.
// out32 (optional, fp32 [n_rows, dim]) receives the normed values before their rounding to out's dtype (a router that decides in fp32
// reads these).
DSB_EXPORT int dsb200_sandwich_norm(float* x, const void* y, int y_dtype, const float* wb, float ob, float y_mult, const float* w, float o,
                                    void* out, int out_dtype, float* out32, const int* rows, int n_rows, int dim, float eps, int plain_out,
                                    cudaStream_t stream) {
  if (n_rows == 0) return DSB_OK;
  DSB_REQUIRE(y == nullptr || (wb != nullptr && rows == nullptr), "sandwich_norm: a branch needs its weight and cannot be combined with a row gather");
  DSB_REQUIRE(w == nullptr || out != nullptr, "sandwich_norm: an output norm needs an output");
  DSB_REQUIRE(!plain_out || (w == nullptr && out != nullptr && out32 == nullptr), "sandwich_norm: the plain output replaces the output norm");
  int block = dim >= 1024 ? 256 : 128;
  const bool vec = dim % 4 == 0 && dim <= 4 * SN_MAXV * 512 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(wb) |
                                                                reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(out32)) & 15) == 0;
  if (vec) {  // one 4-vector per thread and step, at most SN_MAXV steps
    block = 64;
    while (block * SN_MAXV * 4 < dim) block *= 2;
  }
#define LAUNCH(TY, TO)                                                                                                              \
  do {                                                                                                                              \
    if (vec) sandwich_norm_vec_kernel<TY, TO><<<n_rows, block, 0, stream>>>(x, (const TY*)y, wb, ob, y_mult, w, o, (TO*)out, out32, rows, dim, eps, plain_out); \
    else sandwich_norm_kernel<TY, TO><<<n_rows, block, 0, stream>>>(x, (const TY*)y, wb, ob, y_mult, w, o, (TO*)out, out32, rows, dim, eps, plain_out);  \
  } while (0)
  if (y_dtype == 0 && out_dtype == 0) LAUNCH(bf16, bf16);
  else if (y_dtype == 0) LAUNCH(bf16, float);
  else if (out_dtype == 0) LAUNCH(float, bf16);
  else LAUNCH(float, float);
#undef LAUNCH
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// Output row r works on row src = rows[r] (src = r without `rows`) of the fp32 residual x and of the branches: x[src] + y0[src] + y1[src] +
// y2[src] (each branch optional; y0 and y1 in dtype y_dtype, y2 fp32) -- written back to x only without `rows` -- then, if w: out[r] = that
// row split into `groups` equal consecutive parts, each over its own root mean square (eps inside the root), times w.  out bf16
// (out_dtype 0) or fp32 (1); out32 (optional) the same values before rounding.
DSB_EXPORT int dsb200_stream_group_norm(float* x, const void* y0, const void* y1, int y_dtype, const float* y2, const float* w, void* out,
                                        int out_dtype, float* out32, const int* rows, int n_rows, int dim, int groups, float eps,
                                        cudaStream_t stream) {
  if (n_rows == 0) return DSB_OK;
  DSB_REQUIRE(groups >= 1 && dim % groups == 0, "stream_group_norm: %d values do not split into %d equal parts", dim, groups);
  DSB_REQUIRE(w == nullptr || out != nullptr, "stream_group_norm: a norm needs an output");
  const uintptr_t all = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y0) | reinterpret_cast<uintptr_t>(y1) | reinterpret_cast<uintptr_t>(y2) |
                        reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(out32);
  const bool vec = (dim / groups) % 128 == 0 && groups <= GN_MAXG && dim <= 4 * SN_MAXV * 512 && (all & 15) == 0;
  int block = dim >= 1024 ? 256 : 128;
  if (vec) {
    block = 64;
    while (block * SN_MAXV * 4 < dim) block *= 2;
  }
  const size_t smem = vec ? 0 : static_cast<size_t>(dim) * sizeof(float);
  DSB_REQUIRE(smem <= 200 * 1024, "stream_group_norm: a row of %d values does not fit shared memory", dim);
#define LAUNCH(TY, TO)                                                                                                                       \
  do {                                                                                                                                       \
    if (vec) {                                                                                                                               \
      stream_group_norm_vec_kernel<TY, TO><<<n_rows, block, 0, stream>>>(x, (const TY*)y0, (const TY*)y1, y2, w, (TO*)out, out32, rows, dim, groups, eps); \
    } else {                                                                                                                                 \
      if (smem > 48 * 1024)                                                                                                                  \
        DSB_CHECK_CUDA(cudaFuncSetAttribute(stream_group_norm_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));      \
      stream_group_norm_kernel<TY, TO><<<n_rows, block, smem, stream>>>(x, (const TY*)y0, (const TY*)y1, y2, w, (TO*)out, out32, rows, dim, groups, eps); \
    }                                                                                                                                        \
  } while (0)
  if (y_dtype == 0 && out_dtype == 0) LAUNCH(bf16, bf16);
  else if (y_dtype == 0) LAUNCH(bf16, float);
  else if (out_dtype == 0) LAUNCH(float, bf16);
  else LAUNCH(float, float);
#undef LAUNCH
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// lat [n_tokens, ld] holds (query latent [nq] | key/value latent [nkv]) of every token.  cq [n_tokens, nq] = plain-weight RMS norm
// of the first part; the RMS-normed second part is written to the token's row of cache [blocks, block_size, cache_ld] (cache_ld >= nkv:
// rows may be padded to a width the tensor-core attention takes; the padding is never written).
DSB_EXPORT int dsb200_latent_norm_append(const void* lat, int ld, const float* wq, const float* wkv, void* cq, void* cache, const int* tok_seq,
                                         const int* tok_pos, const int* block_table, int bt_stride, int block_size, int cache_ld, int n_tokens,
                                         int nq, int nkv, float eps, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  const int warps = 2 * n_tokens, wpb = 4;
  const int grid = (warps + wpb - 1) / wpb;
  if (dtype == 0)
    latent_norm_append_kernel<bf16><<<grid, wpb * 32, 0, stream>>>((const bf16*)lat, ld, wq, wkv, (bf16*)cq, (bf16*)cache, tok_seq, tok_pos,
                                                                  block_table, bt_stride, block_size, cache_ld, n_tokens, nq, nkv, eps);
  else
    latent_norm_append_kernel<float><<<grid, wpb * 32, 0, stream>>>((const float*)lat, ld, wq, wkv, (float*)cq, (float*)cache, tok_seq, tok_pos,
                                                                   block_table, bt_stride, block_size, cache_ld, n_tokens, nq, nkv, eps);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// floats of scratch `dsb200_latent_attention` needs for n_splits > 1
DSB_EXPORT long long dsb200_latent_attention_scratch_floats(int n_tokens, int H, int R, int n_splits) {
  return n_splits > 1 ? static_cast<long long>(n_tokens) * n_splits * H * (R + 2) : 0;
}

// out[t, h, :] = sum_j softmax_j(scale * q[t, h, :] . c_j) c_j over the cached latents c_0 .. c_pos(t) of the token's sequence.
// q: bf16 / fp32 (q_dtype 0 / 1) with element strides per token and head; cache [blocks, block_size, R] bf16 / fp32 (cache_dtype);
// out fp32 with element strides per token and head.  R <= 1024.
DSB_EXPORT int dsb200_latent_attention(const void* q, int q_dtype, long long q_tok_stride, long long q_head_stride, const void* cache,
                                       int cache_dtype, float* out, long long o_tok_stride, long long o_head_stride, float* scratch,
                                       const int* tok_seq, const int* tok_pos, const int* block_table, int bt_stride, int block_size,
                                       int n_tokens, int H, int R, float scale, int n_splits, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  DSB_REQUIRE(R >= 1 && R <= 1024 && H >= 1 && n_splits >= 1, "latent_attention: R=%d (1..1024) H=%d splits=%d", R, H, n_splits);
  DSB_REQUIRE(n_splits == 1 || scratch != nullptr, "latent_attention: splits need scratch");
  float* part_ml = scratch;
  float* part_acc = scratch ? scratch + static_cast<size_t>(n_tokens) * n_splits * H * 2 : nullptr;
  const dim3 grid(n_tokens, n_splits, (H + LA_HPC - 1) / LA_HPC);
  const size_t smem = (static_cast<size_t>(LA_HPC) * R + LA_KT * (R + 1) + 4 * 2 * LA_KT) * sizeof(float);
#define LAUNCH(TC, TQ, RI)                                                                                                        \
  do {                                                                                                                            \
    auto kern = latent_attention_kernel<TC, TQ, RI>;                                                                              \
    if (smem > 48 * 1024) DSB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));     \
    kern<<<grid, 128, smem, stream>>>((const TQ*)q, q_tok_stride, q_head_stride, (const TC*)cache, out, o_tok_stride, o_head_stride, \
                                      part_ml, part_acc, tok_seq, tok_pos, block_table, bt_stride, block_size, H, R, scale, n_splits); \
  } while (0)
#define BY_RI(TC, TQ)                          \
  do {                                         \
    if (R <= 32) LAUNCH(TC, TQ, 1);            \
    else if (R <= 64) LAUNCH(TC, TQ, 2);       \
    else if (R <= 128) LAUNCH(TC, TQ, 4);      \
    else if (R <= 256) LAUNCH(TC, TQ, 8);      \
    else if (R <= 512) LAUNCH(TC, TQ, 16);     \
    else LAUNCH(TC, TQ, 32);                   \
  } while (0)
  if (cache_dtype == 0 && q_dtype == 0) BY_RI(bf16, bf16);
  else if (cache_dtype == 0) BY_RI(bf16, float);
  else if (q_dtype == 0) BY_RI(float, bf16);
  else BY_RI(float, float);
#undef BY_RI
#undef LAUNCH
  DSB_CHECK_CUDA(cudaGetLastError());
  if (n_splits > 1) {
    const long long warps = static_cast<long long>(n_tokens) * H;
    latent_attention_merge_kernel<<<static_cast<int>((warps + 3) / 4), 128, 0, stream>>>(part_ml, part_acc, out, o_tok_stride, o_head_stride,
                                                                                         n_tokens, H, R, n_splits);
    DSB_CHECK_CUDA(cudaGetLastError());
  }
  return DSB_OK;
}

// a[r, c] *= sigmoid(g[r, c]) over [rows, cols] with row strides (elements).  dtype 0 = bf16, 1 = fp32.
DSB_EXPORT int dsb200_sigmoid_gate_mul(void* a, long long a_ld, const void* g, long long g_ld, long long rows, int cols, int dtype,
                                       cudaStream_t stream) {
  const long long n = rows * cols;
  if (n == 0) return DSB_OK;
  if (dtype == 0)
    sigmoid_gate_mul_kernel<bf16><<<grid_for(n, 256), 256, 0, stream>>>((bf16*)a, a_ld, (const bf16*)g, g_ld, cols, n);
  else
    sigmoid_gate_mul_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((float*)a, a_ld, (const float*)g, g_ld, cols, n);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// out [n_tokens, H * dv] = heads of a [H, n_tokens, dv] (contiguous) laid side by side per token, times sigmoid(g) with g [n_tokens, H * dv]
// at row stride g_ld (elements); g may be null (plain transposition).  dtype 0 = bf16, 1 = fp32.
DSB_EXPORT int dsb200_gate_heads(const void* a, const void* g, long long g_ld, void* out, int n_tokens, int H, int dv, int dtype,
                                 cudaStream_t stream) {
  const long long n = static_cast<long long>(n_tokens) * H * dv;
  if (n == 0) return DSB_OK;
  DSB_REQUIRE(g != nullptr, "gate_heads: a gate is required");
  const int esz = dtype == 0 ? 2 : 4;
  const bool vec = dv % 4 == 0 && g_ld % 4 == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(g) & (4 * esz - 1)) == 0;
#define LAUNCH(T, V) gate_heads_kernel<T, V><<<grid_for(n / (V ? 4 : 1), 256), 256, 0, stream>>>((const T*)a, (const T*)g, g_ld, (T*)out, n_tokens, H, dv)
  if (dtype == 0 && vec) LAUNCH(bf16, true);
  else if (dtype == 0) LAUNCH(bf16, false);
  else if (vec) LAUNCH(float, true);
  else LAUNCH(float, false);
#undef LAUNCH
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// gu [rows, 2 F] = (gate | up) -> out [rows, F] = g' * sigmoid(alpha g') * (clamp(u, -limit, limit) + shift), g' = min(g, limit)
DSB_EXPORT int dsb200_clamped_swish_gate(const void* gu, void* out, long long rows, int F, float alpha, float limit, float shift, int dtype,
                                         cudaStream_t stream) {
  const long long n = rows * F;
  if (n == 0) return DSB_OK;
  const bool vec = F % 4 == 0 && ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (vec && dtype == 0)
    clamped_swish_gate_vec_kernel<bf16><<<grid_for(n / 4, 256), 256, 0, stream>>>((const bf16*)gu, (bf16*)out, rows, F, alpha, limit, shift);
  else if (vec)
    clamped_swish_gate_vec_kernel<float><<<grid_for(n / 4, 256), 256, 0, stream>>>((const float*)gu, (float*)out, rows, F, alpha, limit, shift);
  else if (dtype == 0)
    clamped_swish_gate_kernel<bf16><<<grid_for(n, 256), 256, 0, stream>>>((const bf16*)gu, (bf16*)out, rows, F, alpha, limit, shift);
  else
    clamped_swish_gate_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((const float*)gu, (float*)out, rows, F, alpha, limit, shift);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// out[r, c] = g' * sigmoid(alpha g') * (clamp(u, -limit, limit) + shift) with g' = min(gu[r, gate_col0 + c], limit), u = gu[r, up_col0 + c], c < F:
// gate and up are column ranges of one fused projection gu [rows, ld]; out [rows, out_ld] may be a column range of a wider buffer.
DSB_EXPORT int dsb200_clamped_swish_gate_cols(const void* gu, long long ld, int gate_col0, int up_col0, void* out, long long out_ld, long long rows,
                                              int F, float alpha, float limit, float shift, int dtype, cudaStream_t stream) {
  const long long n = rows * F;
  if (n == 0) return DSB_OK;
  const int esz = dtype == 0 ? 2 : 4;
  const bool vec = F % 4 == 0 && gate_col0 % 4 == 0 && up_col0 % 4 == 0 && ld % 4 == 0 && out_ld % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) & (4 * esz - 1)) == 0;
  if (vec && dtype == 0)
    clamped_swish_gate_cols_vec_kernel<bf16><<<grid_for(n / 4, 256), 256, 0, stream>>>((const bf16*)gu, ld, gate_col0, up_col0, (bf16*)out, out_ld, rows, F,
                                                                                     alpha, limit, shift);
  else if (vec)
    clamped_swish_gate_cols_vec_kernel<float><<<grid_for(n / 4, 256), 256, 0, stream>>>((const float*)gu, ld, gate_col0, up_col0, (float*)out, out_ld, rows, F,
                                                                                      alpha, limit, shift);
  else if (dtype == 0)
    clamped_swish_gate_cols_kernel<bf16><<<grid_for(n, 256), 256, 0, stream>>>((const bf16*)gu, ld, gate_col0, up_col0, (bf16*)out, out_ld, rows, F, alpha,
                                                                              limit, shift);
  else
    clamped_swish_gate_cols_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((const float*)gu, ld, gate_col0, up_col0, (float*)out, out_ld, rows, F,
                                                                               alpha, limit, shift);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// x[r, c] = cap * tanh(x[r, c] / cap) over fp32 [rows, cols] with row stride ld
DSB_EXPORT int dsb200_softcap(float* x, long long ld, long long rows, int cols, float cap, cudaStream_t stream) {
  const long long n = rows * cols;
  if (n == 0) return DSB_OK;
  softcap_kernel<<<grid_for(n, 256), 256, 0, stream>>>(x, ld, cols, n, cap);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// Router: scores = softmax over the E logits of a token, or (sigmoid_scores) the sigmoid of every logit on its own; selection score =
// score + correction[e] (correction may be null); experts are split
// into `groups` contiguous groups of equal size, of which the `keep` with the largest maximal selection score stay selectable; the top_k
// selectable experts by selection score are assigned; their weights are the uncorrected scores (divided by their sum when
// `normalize`).  Outputs as dsb200_top_k_gating; expert_counts must be zeroed by the caller.
DSB_EXPORT int dsb200_grouped_topk_gating(const float* logits, const float* correction, int* expert_counts, float* scores, int* assignments,
                                          int* offsets, int n_tokens, int n_experts, int top_k, int groups, int keep, int normalize,
                                          int sigmoid_scores, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  DSB_REQUIRE(top_k >= 1 && top_k <= 32 && top_k <= n_experts && n_experts <= 2048, "grouped_topk_gating: k=%d (1..32), experts=%d (<=2048)",
              top_k, n_experts);
  DSB_REQUIRE(groups >= 1 && n_experts % groups == 0 && keep >= 1 && keep <= groups && keep * (n_experts / groups) >= top_k,
              "grouped_topk_gating: %d experts in %d groups, %d kept, top %d", n_experts, groups, keep, top_k);
  const int wpb = 4;
  const size_t smem = static_cast<size_t>(wpb) * (n_experts + groups) * sizeof(float);
  grouped_topk_gating_kernel<<<(n_tokens + wpb - 1) / wpb, wpb * 32, smem, stream>>>(logits, correction, expert_counts, scores, assignments,
                                                                                   offsets, n_tokens, n_experts, top_k, groups, keep, normalize, sigmoid_scores);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// Rows of x [n_tokens, dim] copied into expert-sorted order (any dim; dtype 0 = bf16, 1 = fp32); also writes the inclusive
// per-expert row cumsum and every (token, k)'s row.  row_scale (optional, fp32 [n_tokens, top_k]): copy k of token t is multiplied by
// row_scale[t, k] (routers whose weight applies to the expert's input).
DSB_EXPORT int dsb200_moe_scatter_rows(const void* x, const int* expert_counts, const int* assignments, const int* offsets,
                                       long long* expert_cumsum, void* moe_in, int* mapped_slots, int n_tokens, int n_experts, int dim,
                                       int top_k, int dtype, const float* row_scale, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  expert_cumsum_kernel<<<1, 32, 0, stream>>>(expert_counts, expert_cumsum, n_experts);
  const bool vec = dim % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(moe_in)) & 15) == 0;
#define LAUNCH(T, V) moe_scatter_kernel<T, V><<<n_tokens, 256, 0, stream>>>((const T*)x, assignments, offsets, expert_cumsum, (T*)moe_in, mapped_slots, dim, top_k, row_scale)
  if (dtype == 0 && vec) LAUNCH(bf16, true);
  else if (dtype == 0) LAUNCH(bf16, false);
  else if (vec) LAUNCH(float, true);
  else LAUNCH(float, false);
#undef LAUNCH
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// out[t, :] (fp32) = sum_k scores[t, k] * moe_out[mapped_slots[t, k], :]; scores may be null (plain sum).  With `assignments` (the chosen
// expert of every (token, k)): experts n_real and above are identity experts whose output is the token's row of identity_src (fp32
// [n_tokens, dim]) instead of a row of moe_out.
DSB_EXPORT int dsb200_moe_gather_rows(const void* moe_out, const float* scores, const int* mapped_slots, float* out, int n_tokens, int dim,
                                      int top_k, int dtype, const int* assignments, int n_real, const float* identity_src, cudaStream_t stream) {
  if (n_tokens == 0) return DSB_OK;
  DSB_REQUIRE(assignments == nullptr || identity_src != nullptr, "moe_gather_rows: identity experts need their source rows");
  const bool vec = dim % 4 == 0 && ((reinterpret_cast<uintptr_t>(moe_out) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(identity_src)) & 15) == 0;
#define LAUNCH(T, V) moe_gather_kernel<T, V><<<n_tokens, 256, 0, stream>>>((const T*)moe_out, scores, mapped_slots, out, dim, top_k, assignments, n_real, identity_src)
  if (dtype == 0 && vec) LAUNCH(bf16, true);
  else if (dtype == 0) LAUNCH(bf16, false);
  else if (vec) LAUNCH(float, true);
  else LAUNCH(float, false);
#undef LAUNCH
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// Grouped expert GEMM on CUDA cores: out[r, :] = w[expert(r)] x[r, :] for the R rows sorted by expert; x [R, K], w [E, N, K],
// out [R, N], all bf16 (dtype 0) or all fp32 (dtype 1), contiguous; fp32 accumulation.  expert_cumsum [E] int64 on the device.
DSB_EXPORT int dsb200_moe_gemm_rows(const void* x, const void* w, void* out, const long long* expert_cumsum, int R, int N, int K, int E,
                                    int dtype, cudaStream_t stream) {
  if (R == 0) return DSB_OK;
  const dim3 grid((R + GM - 1) / GM + E, (N + GN - 1) / GN);
  if (dtype == 0)
    moe_gemm_rows_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)x, (const bf16*)w, (bf16*)out, expert_cumsum, E, N, K);
  else
    moe_gemm_rows_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (const float*)w, (float*)out, expert_cumsum, E, N, K);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// ------------------------------------------------------------------------------------------- norm behind the sum, xIELU, scalar head gates
//   post_sum_norm         x <- rms(alpha x + y + y32 + bias) * w on the fp32 stream (blocks whose norm sits BEHIND the residual sum), with a
//                         copy of the new stream in the activation dtype for the sublayer that reads it next
//   xielu                 z > 0: a z^2 + z / 2;  z <= 0: b (exp(z) - 1 - z) + z / 2   (a, b read from device memory)
//   gate_heads_scalar     head-major result of a per-head batched GEMM -> token-major heads, each multiplied by the sigmoid of ONE number
namespace dsb {
namespace latent {

// One block per row.  VEC: dim % 4 == 0 and 16-byte aligned rows; the row is then walked in 4-value accesses.
template <typename TY, typename TO, bool VEC>
__global__ void post_sum_norm_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ y32, const float* __restrict__ bias,
                                     const float* __restrict__ w, TO* __restrict__ out, int dim, float alpha, float eps) {
  __shared__ float red[33];
  const size_t r = blockIdx.x;
  float* xr = x + r * dim;
  const TY* yr = y ? y + r * dim : nullptr;
  const float* zr = y32 ? y32 + r * dim : nullptr;
  TO* orow = out ? out + r * dim : nullptr;
  float ss = 0.f;
  if constexpr (VEC) {
    for (int c = 4 * threadIdx.x; c < dim; c += 4 * blockDim.x) {
      float4 s = load4(xr + c);
      s.x *= alpha; s.y *= alpha; s.z *= alpha; s.w *= alpha;
      if (yr) { const float4 v = load4(yr + c); s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w; }
      if (zr) { const float4 v = load4(zr + c); s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w; }
      if (bias) { const float4 v = load4(bias + c); s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w; }
      store4(xr + c, s);
      ss += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    }
  } else {
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      float s = alpha * xr[c];
      if (yr) s += to_f(yr[c]);
      if (zr) s += zr[c];
      if (bias) s += bias[c];
      xr[c] = s;
      ss += s * s;
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(dim) + eps);
  if constexpr (VEC) {  // every thread meets the values it wrote itself
    for (int c = 4 * threadIdx.x; c < dim; c += 4 * blockDim.x) {
      float4 s = load4(xr + c);
      const float4 g = load4(w + c);
      s.x = s.x * inv * g.x; s.y = s.y * inv * g.y; s.z = s.z * inv * g.z; s.w = s.w * inv * g.w;
      store4(xr + c, s);
      if (orow) store4(orow + c, s);
    }
  } else {
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float v = xr[c] * inv * w[c];
      xr[c] = v;
      if (orow) orow[c] = from_f<TO>(v);
    }
  }
}

// exp(z) - 1 - z for z <= 0.  A bf16 result takes the fast exponential: its absolute error (~1e-7) is below bf16's rounding of the z / 2 the
// term is added to; an fp32 result takes expm1f.
template <typename T>
__device__ __forceinline__ float xielu_tail(float z);
template <>
__device__ __forceinline__ float xielu_tail<float>(float z) { return expm1f(z) - z; }
template <>
__device__ __forceinline__ float xielu_tail<bf16>(float z) { return (__expf(z) - 1.f) - z; }
template <typename T>
__device__ __forceinline__ float xielu_one(float z, float a, float b) {
  return z > 0.f ? fmaf(a * z, z, 0.5f * z) : fmaf(b, xielu_tail<T>(z), 0.5f * z);
}

template <typename T>
__global__ void xielu_kernel(const T* __restrict__ u, long long ld, T* __restrict__ out, long long rows, int F, const float* __restrict__ coef) {
  const float a = coef[0], b = coef[1];
  const long long n = rows * F;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = from_f<T>(xielu_one<T>(to_f(u[(i / F) * ld + (i % F)]), a, b));
}
template <typename T>
__global__ void xielu_vec_kernel(const T* __restrict__ u, T* __restrict__ out, long long n4, const float* __restrict__ coef) {
  const float a = coef[0], b = coef[1];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 z = load4(u + 4 * i);
    z.x = xielu_one<T>(z.x, a, b);
    z.y = xielu_one<T>(z.y, a, b);
    z.z = xielu_one<T>(z.z, a, b);
    z.w = xielu_one<T>(z.w, a, b);
    store4(out + 4 * i, z);
  }
}

// VEC: dv % 4 == 0, out_ld % 4 == 0 and 16-byte aligned a / out: four values per thread.
template <typename T, bool VEC>
__global__ void gate_heads_scalar_kernel(const T* __restrict__ a, const T* __restrict__ g, long long g_ld, T* __restrict__ out, long long out_ld,
                                         int n_tokens, int H, int dv) {
  constexpr int V = VEC ? 4 : 1;
  const int row = H * dv;
  const long long n = static_cast<long long>(n_tokens) * row / V;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * V;
    const long long t = e / row;
    const int rem = static_cast<int>(e % row), h = rem / dv, c = rem % dv;
    const float gate = 1.f / (1.f + expf(-to_f(g[t * g_ld + h])));
    const T* src = a + (static_cast<long long>(h) * n_tokens + t) * dv + c;
    if constexpr (VEC) {
      const float4 v = load4(src);
      store4(out + t * out_ld + rem, make_float4(v.x * gate, v.y * gate, v.z * gate, v.w * gate));
    } else {
      out[t * out_ld + rem] = from_f<T>(to_f(*src) * gate);
    }
  }
}

}  // namespace latent
}  // namespace dsb

// x [rows, dim] fp32, in place: x <- s / sqrt(mean(s^2) + eps) * w with s = alpha x + y + y32 + bias; y [rows, dim] in y_dtype (0 = bf16,
// 1 = fp32), y32 [rows, dim] fp32, bias [dim] fp32 -- each may be null.  out (null, or [rows, dim] in out_dtype): the new x, rounded.
DSB_EXPORT int dsb200_post_sum_norm(float* x, const void* y, int y_dtype, const float* y32, const float* bias, const float* w, void* out, int out_dtype,
                                    long long rows, int dim, float alpha, float eps, cudaStream_t stream) {
  if (rows == 0) return DSB_OK;
  DSB_REQUIRE(x != nullptr && w != nullptr && dim >= 1, "post_sum_norm: stream / weight missing or width %d", dim);
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = dim % 8 == 0 && al(x) && al(y) && al(y32) && al(bias) && al(w) && al(out);
  const int threads = vec ? (dim >= 4096 ? 512 : (dim >= 1024 ? 256 : 128)) : 256;
  const unsigned grid = static_cast<unsigned>(rows);
#define LAUNCH(TY, TO)                                                                                                                          \
  do {                                                                                                                                          \
    if (vec) post_sum_norm_kernel<TY, TO, true><<<grid, threads, 0, stream>>>(x, (const TY*)y, y32, bias, w, (TO*)out, dim, alpha, eps);        \
    else post_sum_norm_kernel<TY, TO, false><<<grid, threads, 0, stream>>>(x, (const TY*)y, y32, bias, w, (TO*)out, dim, alpha, eps);           \
  } while (0)
  if (y_dtype == 0 && out_dtype == 0) LAUNCH(bf16, bf16);
  else if (y_dtype == 0) LAUNCH(bf16, float);
  else if (out_dtype == 0) LAUNCH(float, bf16);
  else LAUNCH(float, float);
#undef LAUNCH
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// out [rows, F] = xIELU(u [rows, ld]): z > 0: coef[0] z^2 + z / 2; z <= 0: coef[1] (exp(z) - 1 - z) + z / 2; coef: two floats on the device.
DSB_EXPORT int dsb200_xielu(const void* u, long long ld, void* out, long long rows, int F, const float* coef, int dtype, cudaStream_t stream) {
  const long long n = rows * F;
  if (n == 0) return DSB_OK;
  DSB_REQUIRE(coef != nullptr && ld >= F, "xielu: coefficients missing or row stride %lld below %d", ld, F);
  const bool vec = ld == F && n % 4 == 0 && ((reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (vec && dtype == 0) xielu_vec_kernel<bf16><<<grid_for(n / 4, 256), 256, 0, stream>>>((const bf16*)u, (bf16*)out, n / 4, coef);
  else if (vec) xielu_vec_kernel<float><<<grid_for(n / 4, 256), 256, 0, stream>>>((const float*)u, (float*)out, n / 4, coef);
  else if (dtype == 0) xielu_kernel<bf16><<<grid_for(n, 256), 256, 0, stream>>>((const bf16*)u, ld, (bf16*)out, rows, F, coef);
  else xielu_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((const float*)u, ld, (float*)out, rows, F, coef);
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

// out[t, h dv + c] = a[h, t, c] * sigmoid(g[t, h]): a [H, n_tokens, dv] contiguous, g [n_tokens, g_ld] with one number per head.
DSB_EXPORT int dsb200_gate_heads_scalar(const void* a, const void* g, long long g_ld, void* out, long long out_ld, int n_tokens, int H, int dv,
                                        int dtype, cudaStream_t stream) {
  const long long n = static_cast<long long>(n_tokens) * H * dv;
  if (n == 0) return DSB_OK;
  DSB_REQUIRE(out_ld >= static_cast<long long>(H) * dv && g_ld >= H, "gate_heads_scalar: strides %lld / %lld", out_ld, g_ld);
  const bool vec = dv % 4 == 0 && out_ld % 4 == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
#define LAUNCH(T, V) gate_heads_scalar_kernel<T, V><<<grid_for(n / (V ? 4 : 1), 256), 256, 0, stream>>>((const T*)a, (const T*)g, g_ld, (T*)out, out_ld, n_tokens, H, dv)
  if (dtype == 0 && vec) LAUNCH(bf16, true);
  else if (dtype == 0) LAUNCH(bf16, false);
  else if (vec) LAUNCH(float, true);
  else LAUNCH(float, false);
#undef LAUNCH
  DSB_CHECK_CUDA(cudaGetLastError());
  return DSB_OK;
}

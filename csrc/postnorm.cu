// Post-norm hybrid decoders (Lonulix) -- the glue that the fused projections, the paged softmax attention and the linear
// recurrences of seqmix.cu do not have yet:
//   * post_norm_join   x <- groupnorm(alpha x + gate * (y + idw x)) * w : the sublayer result (optionally with the share of
//                      identity experts, optionally times a sigmoid gate read from the fused projection) joins the scaled
//                      residual, the sum is RMS-normed in `groups` consecutive parts, and the new residual is written both
//                      as fp32 and as the operand of the next matrix product (no norm sits in front of a sublayer)
//   * latent_prep      latent attention: RMS norm of the query latent (-> operand of the query up-projection), RMS norm of
//                      the key/value latent and rotation of the shared rotary key part -> one cache row [rotary | latent]
//   * rot_heads        rotary positions on the first channels of every head of a projection -> dense query rows
//   * moe_route        softmax router with a selection-only correction, group-limited top-k and identity experts
//   * gated_cols       out = act(a) * b for two column blocks, or act(a) * per-expert weight (routed experts run as one
//                      stacked up-projection whose hidden columns are scaled by the token's weight for their expert), or both
//   * head_up_gate     a [V, C] matrix per head applied to per-head latent rows, times a sigmoid output gate
// Norms, gates, router, angles and the residual are fp32 in every mode; OT / CT (operand / cache type) is bf16 or float.
// This translation unit is compiled WITHOUT --use_fast_math (exact expf / erff / division / sqrt / sincos).
#include "kernels.h"

#include <cuda_bf16.h>

#include <cstdint>

#include "launch.cuh"

namespace b2b {
namespace {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ void stf(T* p, size_t i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, size_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoid_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float ldf_(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float ldf_(const bf16* p, size_t i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ void pdl_begin() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ float warp_sum_(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// sin and cos of position * frequency with the frequency given as a sum of two floats (flo may be 0): the fp32 product
// pos * fhi is corrected by what its rounding lost (an exact fused multiply-add) and by pos * flo, through the addition
// formulas with the small remainder r.  At position 1000 a plain fp32 product is off
// by up to 3e-5 rad, which a sharp softmax over far keys shows; this form is good to the last bits of the result.
__device__ __forceinline__ void turn_(float pos, float fhi, float flo, float* sn, float* cs) {
  const float a = __fmul_rn(pos, fhi);
  const float r = __fmaf_rn(pos, flo, __fmaf_rn(pos, fhi, -a));
  float s, c, sr, cr;
  sincosf(a, &s, &c);
  sincosf(r, &sr, &cr);
  *sn = __fmaf_rn(s, cr, c * sr);
  *cs = __fmaf_rn(c, cr, -s * sr);
}
// ------------------------------------------------------------------------------------------- post-norm join
// One warp per (row, group).  rows == nullptr: row = token, x is updated in place and h[t] written.  rows != nullptr:
// row r reads token rows[r] and only writes h[r] (the logit rows in front of the model norm).
// PT: channels of a group per lane kept in registers (Wg <= 32 * PT), 0 = any width (the sum is parked in x / recomputed).
constexpr int PNJ_WARPS = 4;
template <typename OT, int PT>
__global__ void __launch_bounds__(32 * PNJ_WARPS)
    post_norm_join_kernel(float* __restrict__ x, const int* __restrict__ rows, int n_rows, const float* __restrict__ y,
                          int ld_y, const float* __restrict__ gate, int ld_g, int off_g, const float* __restrict__ gbias,
                          const float* __restrict__ idw, float alpha, const float* __restrict__ w, int groups, float eps,
                          OT* __restrict__ h, int ld_h, int W) {
  pdl_begin();
  const long long wid = static_cast<long long>(blockIdx.x) * PNJ_WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(n_rows) * groups) return;
  const int r = static_cast<int>(wid / groups), g = static_cast<int>(wid % groups);
  const int t = rows != nullptr ? rows[r] : r;
  const int Wg = W / groups, c0 = g * Wg;
  float* xr = x + static_cast<size_t>(t) * W + c0;
  const float* yr = y != nullptr ? y + static_cast<size_t>(t) * ld_y + c0 : nullptr;
  const float* gr = gate != nullptr ? gate + static_cast<size_t>(t) * ld_g + off_g + c0 : nullptr;
  const float keep = idw != nullptr ? idw[t] : 0.f;
  auto value = [&](int c) {
    const float xv = xr[c];
    if (yr == nullptr) return alpha * xv;
    float yv = yr[c] + keep * xv;
    if (gr != nullptr) yv *= sigmoid_(gr[c] + gbias[c0 + c]);
    return alpha * xv + yv;
  };
  float ss = 0.f;
  float v[PT > 0 ? PT : 1];
  if (PT > 0) {
#pragma unroll
    for (int k = 0; k < PT; ++k) {
      const int c = lane + 32 * k;
      v[k] = c < Wg ? value(c) : 0.f;
      ss += v[k] * v[k];
    }
  } else {
    for (int c = lane; c < Wg; c += 32) {
      const float u = value(c);
      if (rows == nullptr) xr[c] = u;          // parked: the same lane reads it back below
      ss += u * u;
    }
  }
  const float rinv = 1.f / sqrtf(warp_sum_(ss) / static_cast<float>(Wg) + eps);
  OT* hr = h + static_cast<size_t>(r) * ld_h + c0;
  if (PT > 0) {
#pragma unroll
    for (int k = 0; k < PT; ++k) {
      const int c = lane + 32 * k;
      if (c < Wg) {
        const float o = v[k] * rinv * w[c0 + c];
        if (rows == nullptr) xr[c] = o;
        stf(hr, c, o);
      }
    }
  } else {
    for (int c = lane; c < Wg; c += 32) {
      const float o = (rows == nullptr ? xr[c] : value(c)) * rinv * w[c0 + c];
      if (rows == nullptr) xr[c] = o;
      stf(hr, c, o);
    }
  }
}

// Wide rows whose groups are multiples of 128 channels: one block of 256 threads per row, 16-byte accesses, NCH chunks of
// four channels per thread in registers (W <= 1024 * NCH); a warp's 128 channels lie in one group, so the group sums are
// the sums of whole warps' partial sums, added in a fixed order.
__device__ __forceinline__ void st4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(bf16* p, const float4& v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<unsigned*>(&a);
  u.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}
template <typename OT, int NCH>
__global__ void __launch_bounds__(256)
    post_norm_join_wide_kernel(float* __restrict__ x, const int* __restrict__ rows, int n_rows, const float* __restrict__ y,
                               int ld_y, const float* __restrict__ gate, int ld_g, int off_g,
                               const float* __restrict__ gbias, const float* __restrict__ idw, float alpha,
                               const float* __restrict__ w, int groups, float eps, OT* __restrict__ h, int ld_h, int W) {
  pdl_begin();
  __shared__ float part[NCH * 8];
  const int r = blockIdx.x;
  const int t = rows != nullptr ? rows[r] : r;
  const int Wg = W / groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wpg = Wg >> 7;
  float* xr = x + static_cast<size_t>(t) * W;
  const float keep = idw != nullptr ? idw[t] : 0.f;
  float4 v[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (j * 256 + threadIdx.x) * 4;
    float ss = 0.f;
    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < W) {
      const float4 xv = *reinterpret_cast<const float4*>(xr + c);
      float4 u = make_float4(alpha * xv.x, alpha * xv.y, alpha * xv.z, alpha * xv.w);
      if (y != nullptr) {
        float4 yv = *reinterpret_cast<const float4*>(y + static_cast<size_t>(t) * ld_y + c);
        yv = make_float4(yv.x + keep * xv.x, yv.y + keep * xv.y, yv.z + keep * xv.z, yv.w + keep * xv.w);
        if (gate != nullptr) {
          const float4 gv = *reinterpret_cast<const float4*>(gate + static_cast<size_t>(t) * ld_g + off_g + c);
          const float4 bv = *reinterpret_cast<const float4*>(gbias + c);
          yv = make_float4(yv.x * sigmoid_(gv.x + bv.x), yv.y * sigmoid_(gv.y + bv.y), yv.z * sigmoid_(gv.z + bv.z),
                           yv.w * sigmoid_(gv.w + bv.w));
        }
        u = make_float4(u.x + yv.x, u.y + yv.y, u.z + yv.z, u.w + yv.w);
      }
      v[j] = u;
      ss = u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
    }
    ss = warp_sum_(ss);
    if (lane == 0) part[j * 8 + warp] = ss;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (j * 256 + threadIdx.x) * 4;
    if (c >= W) continue;
    // entry e of part[] holds channels [128 e, 128 e + 128): a group is wpg consecutive entries
    const int e0 = (j * 8 + warp) / wpg * wpg;
    float tot = 0.f;
    for (int e = e0; e < e0 + wpg; ++e) tot += part[e];
    const float rinv = 1.f / sqrtf(tot / static_cast<float>(Wg) + eps);
    const float4 wv = *reinterpret_cast<const float4*>(w + c);
    const float4 o = make_float4(v[j].x * rinv * wv.x, v[j].y * rinv * wv.y, v[j].z * rinv * wv.z, v[j].w * rinv * wv.w);
    if (rows == nullptr) *reinterpret_cast<float4*>(xr + c) = o;
    st4(h + static_cast<size_t>(r) * ld_h + c, o);
  }
}

// ------------------------------------------------------------------------------------------- latent attention prep
// proj [T, ld] fp32: query latent (q_rank columns at off_q), then at off_kv the key/value latent (C columns) followed by
// the rotary key part (R columns) that all heads share.  One warp per token:
//   cq[t]            = rms(query latent) * wq                      (operand of the query up-projection)
//   k_cache[slot]    = [ rotate(rotary part) | rms(latent) * wc ]  (the only thing a token leaves in the cache)
// Rotation: channels (2i, 2i+1), 2i < rdims, turn by positions[t] * freq[i]; cos and sin are multiplied by amp.
constexpr int LAT_WARPS = 4;                  // one warp per token: a token's latents are a few hundred channels
template <typename OT, typename CT>
__global__ void __launch_bounds__(32 * LAT_WARPS)
    latent_prep_kernel(const float* __restrict__ proj, int ld, int off_q, int q_rank, int off_kv, int C, int R,
                       const float* __restrict__ wq, const float* __restrict__ wc, const float* __restrict__ freq,
                       int rdims, const int* __restrict__ positions, const int* __restrict__ slots, OT* __restrict__ cq,
                       int ld_cq, CT* __restrict__ k_cache, float eps, int T, float amp,
                       const float* __restrict__ freq_lo) {
  pdl_begin();
  const int t = blockIdx.x * LAT_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const int slot = slots[t];
  if (slot < 0) return;                               // padding row of a bucketed chunk (warp-uniform)
  const float* row = proj + static_cast<size_t>(t) * ld;
  const float* ql = row + off_q;
  const float* cl = row + off_kv;
  float sq = 0.f, sc = 0.f;
  for (int i = lane; i < q_rank; i += 32) sq += ql[i] * ql[i];
  for (int i = lane; i < C; i += 32) sc += cl[i] * cl[i];
  const float rq = 1.f / sqrtf(warp_sum_(sq) / static_cast<float>(max(q_rank, 1)) + eps);     // q_rank = 0: no query latent
  const float rc = 1.f / sqrtf(warp_sum_(sc) / static_cast<float>(C) + eps);
  for (int i = lane; i < q_rank; i += 32) stf(cq, static_cast<size_t>(t) * ld_cq + i, ql[i] * rq * wq[i]);
  CT* krow = k_cache + static_cast<size_t>(slot) * (R + C);
  for (int i = lane; i < C; i += 32) stf(krow, R + i, cl[i] * rc * wc[i]);
  const float* kr = cl + C;
  const float pos = static_cast<float>(positions[t]);
  for (int i = lane; i < rdims / 2; i += 32) {        // a lane turns whole pairs
    float sn, cs;
    turn_(pos, freq[i], freq_lo != nullptr ? freq_lo[i] : 0.f, &sn, &cs);
    sn *= amp;
    cs *= amp;
    const float u = kr[2 * i], v = kr[2 * i + 1];
    stf(krow, 2 * i, u * cs - v * sn);
    stf(krow, 2 * i + 1, v * cs + u * sn);
  }
  for (int i = rdims + lane; i < R; i += 32) stf(krow, i, kr[i]);
}

// src [T, ld] fp32 holds H heads of Dh channels at column off; dst [T, H * Dh] (dense) receives them with the rdims
// channels from channel roff of every head on turned by positions[t] * freq[pair] (pairs 2i, 2i+1) and multiplied by amp.
__global__ void rot_heads_kernel(const float* __restrict__ src, int ld, int off, float* __restrict__ dst, int H, int Dh,
                                 const float* __restrict__ freq, int rdims, const int* __restrict__ positions,
                                 const int* __restrict__ slots, int T, int roff, float amp,
                                 const float* __restrict__ freq_lo) {
  pdl_begin();
  const int n = H * Dh;
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= static_cast<long long>(T) * n) return;
  const int c = static_cast<int>(e % n), t = static_cast<int>(e / n);
  if (slots != nullptr && slots[t] < 0) return;
  const int d = c % Dh - roff;                        // channel within the rotated part of its head
  const float* row = src + static_cast<size_t>(t) * ld + off;
  float v = row[c];
  if (d >= 0 && d < rdims) {
    float sn, cs;
    turn_(static_cast<float>(positions[t]), freq[d >> 1], freq_lo != nullptr ? freq_lo[d >> 1] : 0.f, &sn, &cs);
    const float o = row[c - d + (d ^ 1)];             // the other channel of the pair (2i, 2i+1) of this head
    v = ((d & 1) ? v * cs + o * sn : v * cs - o * sn) * amp;
  }
  dst[static_cast<size_t>(t) * n + c] = v;
}

// ------------------------------------------------------------------------------------------- router
// One warp per token.  z = logits [E] (fp32, column off of proj), s = softmax(z); choice = s + corr; consecutive experts
// are bundled into `count` equal groups, a group's score is its largest choice, only experts of the `keep` best groups stay
// candidates; the `top` candidates with the largest choice are chosen (ties: the lower index); their weights are
// s / (sum of the chosen s + 1e-20) * scale (= the softmax over the chosen logits alone when scale = 1).  corr == nullptr:
// the choice is made on the logits themselves.  Experts n_real .. E - 1 are identity experts: their weights are summed into
// idw[t]; wt [T, ld_wt] receives the dense weight row of the real experts (0 = not chosen).  sel_idx / sel_w [T, top]
// (optional) list the choices in order.
__global__ void __launch_bounds__(128)
    moe_route_kernel(const float* __restrict__ proj, int ld, int off, const float* __restrict__ corr, int E, int n_real,
                     int count, int keep, int top, float scale, float* __restrict__ wt, int ld_wt,
                     float* __restrict__ idw, int* __restrict__ sel_idx, float* __restrict__ sel_w, int T) {
  pdl_begin();
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  float* s = sm + static_cast<size_t>(warp) * 4 * E;
  float* ch = s + E;
  float* gs = ch + E;          // group scores, later the list of chosen experts
  float* stay = gs + E;
  const float* z = proj + static_cast<size_t>(t) * ld + off;
  const float ninf = -__int_as_float(0x7f800000);
  float mx = ninf;
  for (int j = lane; j < E; j += 32) mx = fmaxf(mx, z[j]);
  mx = warp_max_(mx);
  float den = 0.f;
  for (int j = lane; j < E; j += 32) {
    const float e = expf(z[j] - mx);
    s[j] = e;
    den += e;
  }
  den = warp_sum_(den);
  for (int j = lane; j < E; j += 32) {
    const float p = s[j] / den;
    s[j] = p;
    ch[j] = corr != nullptr ? p + corr[j] : z[j];      // no correction: the largest logits themselves are chosen
  }
  __syncwarp();
  // warp arg-max over an array of n floats (lowest index among equals)
  auto argmax = [&](const float* a, int n) {
    float bv = ninf;
    int bi = 0x7fffffff;
    for (int j = lane; j < n; j += 32)
      if (a[j] > bv) {
        bv = a[j];
        bi = j;
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    return bi;
  };
  if (count > 1 && keep < count) {
    const int per = E / count;
    for (int g = lane; g < count; g += 32) {
      float m = ninf;
      for (int j = g * per; j < (g + 1) * per; ++j) m = fmaxf(m, ch[j]);
      gs[g] = m;
      stay[g] = 0.f;
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      const int g = argmax(gs, count);
      if (g == 0x7fffffff) break;
      if (lane == 0) {
        gs[g] = ninf;
        stay[g] = 1.f;
      }
      __syncwarp();
    }
    for (int j = lane; j < E; j += 32)
      if (stay[j / per] == 0.f) ch[j] = ninf;              // out of the arg-max for good (a zero would still beat negative candidates)
    __syncwarp();
  }
  for (int j = lane; j < n_real; j += 32) wt[static_cast<size_t>(t) * ld_wt + j] = 0.f;
  int* sel = reinterpret_cast<int*>(gs);
  float tot = 0.f;
  int n_sel = 0;
  for (int k = 0; k < top; ++k) {
    const int j = argmax(ch, E);
    if (j == 0x7fffffff) break;
    tot += s[j];
    if (lane == 0) {
      sel[k] = j;
      ch[j] = ninf;
    }
    ++n_sel;
    __syncwarp();
  }
  float keep_w = 0.f;
  for (int k = lane; k < top; k += 32) {
    const int j = k < n_sel ? sel[k] : -1;
    const float wgt = j >= 0 ? s[j] / (tot + 1e-20f) * scale : 0.f;
    if (j >= 0 && j < n_real) wt[static_cast<size_t>(t) * ld_wt + j] = wgt;
    if (j >= n_real) keep_w += wgt;
    if (sel_idx != nullptr) sel_idx[static_cast<size_t>(t) * top + k] = j;
    if (sel_w != nullptr) sel_w[static_cast<size_t>(t) * top + k] = wgt;
  }
  keep_w = warp_sum_(keep_w);
  if (lane == 0) idw[t] = keep_w;
}

// ------------------------------------------------------------------------------------------- gated columns
// out[t, c] = act(in[t, off_a + c]) * (wt == nullptr ? in[t, off_b + c] : wt[t, c / per]) for c < n.  both != 0 (with wt):
// act(a) * in[t, off_b + c] * weight, where the first `lead` columns have weight 1 and column c >= lead has
// wt[t, (c - lead) / per] (gated experts side by side behind a shared one).
// act: 0 silu, 1 exact (erf) gelu, 2 tanh gelu.  Four columns per thread when every offset allows 16-byte accesses.
__device__ __forceinline__ float act_(float z, int act) {
  if (act == 0) return z / (1.f + expf(-z));
  if (act == 1) return 0.5f * z * (1.f + erff(z * 0.70710678118654752440f));
  return 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
}
template <typename OT>
__global__ void __launch_bounds__(256)
    gated_cols_kernel(const float* __restrict__ in, int ld_in, int off_a, int off_b, const float* __restrict__ wt,
                      int ld_wt, int per, OT* __restrict__ out, int ld_out, int n, int act, int T, int both, int lead) {
  pdl_begin();
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= static_cast<long long>(T) * n) return;
  const int c = static_cast<int>(e % n);
  const size_t t = static_cast<size_t>(e / n);
  const float a = act_(in[t * ld_in + off_a + c], act);
  float b = wt != nullptr ? (c < lead ? 1.f : wt[t * ld_wt + (c - lead) / per]) : in[t * ld_in + off_b + c];
  if (both && wt != nullptr) b *= in[t * ld_in + off_b + c];
  stf(out, t * ld_out + c, a * b);
}

// four columns per thread, grid (column chunks, rows): no division per element; every offset a multiple of four
template <typename OT>
__global__ void __launch_bounds__(256)
    gated_cols_vec_kernel(const float* __restrict__ in, int ld_in, int off_a, int off_b, const float* __restrict__ wt,
                          int ld_wt, int per, OT* __restrict__ out, int ld_out, int n, int act, int both, int lead) {
  pdl_begin();
  const int c = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (c >= n) return;
  const size_t t = blockIdx.y;
  const float4 a = *reinterpret_cast<const float4*>(in + t * ld_in + off_a + c);
  float4 b;
  if (wt != nullptr) {
    const float wv = c < lead ? 1.f : wt[t * ld_wt + (c - lead) / per];      // per and lead are multiples of four: one expert for the four columns
    b = make_float4(wv, wv, wv, wv);
    if (both) {
      const float4 u = *reinterpret_cast<const float4*>(in + t * ld_in + off_b + c);
      b = make_float4(wv * u.x, wv * u.y, wv * u.z, wv * u.w);
    }
  } else {
    b = *reinterpret_cast<const float4*>(in + t * ld_in + off_b + c);
  }
  st4(out + t * ld_out + c, make_float4(act_(a.x, act) * b.x, act_(a.y, act) * b.y, act_(a.z, act) * b.z, act_(a.w, act) * b.w));
}

// ------------------------------------------------------------------------------------------- per-head up-projection
// out[t, h * V + v] = gate(t, h * V + v) * sum_c a[t, h * C + c] * U[h, v, c]: every head has its own [V, C] matrix (the
// value up-projection of latent attention, applied to the attention output taken over the latents), so this is a batch
// of H small matrix products.  gate (optional) = sigmoid of column off_g + h * V + v of an fp32 row (the output gate of the
// concatenated heads).  A block = 64 tokens x 64 value channels of one head, 256 threads with 4 x 4 outputs each, the
// latent dimension walked in slices of 16 through shared memory; fp32 accumulation.  (float32 mode and odd shapes; the
// bf16 serving mode runs the tensor-core variant below.)
template <typename OT>
__global__ void __launch_bounds__(256)
    head_up_gate_kernel(const OT* __restrict__ a, int ld_a, const OT* __restrict__ U, const float* __restrict__ gate,
                        int ld_g, int off_g, OT* __restrict__ out, int ld_out, int T, int H, int V, int C) {
  pdl_begin();
  __shared__ float As[16][64 + 4];       // [c][token]
  __shared__ float Us[16][64 + 4];       // [c][value channel]
  const int h = blockIdx.z, t0 = blockIdx.x * 64, v0 = blockIdx.y * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // tx: value channels, ty: tokens
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const OT* ah = a + static_cast<size_t>(h) * C;
  const OT* uh = U + static_cast<size_t>(h) * V * C;
  for (int c0 = 0; c0 < C; c0 += 16) {
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int r = e >> 4, c = e & 15;                          // consecutive threads walk the latent channels of a row
      const int t = t0 + r, v = v0 + r;
      float av = 0.f, uv = 0.f;
      if (c0 + c < C) {
        if (t < T) av = ldf_(ah + static_cast<size_t>(t) * ld_a, c0 + c);
        if (v < V) uv = ldf_(uh + static_cast<size_t>(v) * C, c0 + c);
      }
      As[c][r] = av;
      Us[c][r] = uv;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      float av[4], uv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[c][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) uv[j] = Us[c][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * uv[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + ty * 4 + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int v = v0 + tx * 4 + j;
      if (v >= V) continue;
      float o = acc[i][j];
      if (gate != nullptr) o *= sigmoid_(gate[static_cast<size_t>(t) * ld_g + off_g + h * V + v]);
      stf(out, static_cast<size_t>(t) * ld_out + h * V + v, o);
    }
  }
}

// bf16 operands with a latent width that is a multiple of 16: the same tile on `mma.sync.m16n8k16` tensor cores.  A block =
// 64 tokens x 64 value channels of one head, a warp = 16 tokens x 64 channels (8 accumulator tiles).  The [64, C] slices of
// the latent rows and of U are staged in shared memory with 16-byte loads, 128 latent channels at a time (row stride + 8
// elements: the fragment loads of a warp fall into 32 different banks).
__device__ __forceinline__ void mma_bf16_16816_(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
constexpr int HUG_KC = 128, HUG_KS = HUG_KC + 8;
__global__ void __launch_bounds__(128)
    head_up_gate_mma_kernel(const bf16* __restrict__ a, int ld_a, const bf16* __restrict__ U,
                            const float* __restrict__ gate, int ld_g, int off_g, bf16* __restrict__ out, int ld_out, int T,
                            int H, int V, int C) {
  pdl_begin();
  __shared__ __align__(16) bf16 stage[2 * 64 * HUG_KS];      // operand slices; the epilogue tile takes their place
  bf16* As = stage;
  bf16* Us = stage + 64 * HUG_KS;
  const int h = blockIdx.z, v0 = blockIdx.y * 64, t0 = blockIdx.x * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  float acc[8][4];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  for (int c0 = 0; c0 < C; c0 += HUG_KC) {
    const int kc = min(HUG_KC, C - c0), n8 = kc >> 3;          // (C is a multiple of 16)
    if (c0 > 0) __syncthreads();
    for (int idx = threadIdx.x; idx < 64 * n8; idx += 128) {
      const int r = idx / n8, c8 = idx - r * n8;
      uint4 av = make_uint4(0u, 0u, 0u, 0u), uv = make_uint4(0u, 0u, 0u, 0u);
      if (t0 + r < T) av = *reinterpret_cast<const uint4*>(a + static_cast<size_t>(t0 + r) * ld_a + static_cast<size_t>(h) * C + c0 + c8 * 8);
      if (v0 + r < V) uv = *reinterpret_cast<const uint4*>(U + (static_cast<size_t>(h) * V + v0 + r) * C + c0 + c8 * 8);
      *reinterpret_cast<uint4*>(As + r * HUG_KS + c8 * 8) = av;
      *reinterpret_cast<uint4*>(Us + r * HUG_KS + c8 * 8) = uv;
    }
    __syncthreads();
    const bf16* ar = As + (warp * 16 + gid) * HUG_KS + 2 * tig;
    const bf16* ur = Us + gid * HUG_KS + 2 * tig;
    for (int k0 = 0; k0 < kc; k0 += 16) {
      unsigned af[4];
      af[0] = *reinterpret_cast<const unsigned*>(ar + k0);
      af[1] = *reinterpret_cast<const unsigned*>(ar + 8 * HUG_KS + k0);
      af[2] = *reinterpret_cast<const unsigned*>(ar + k0 + 8);
      af[3] = *reinterpret_cast<const unsigned*>(ar + 8 * HUG_KS + k0 + 8);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const unsigned b0 = *reinterpret_cast<const unsigned*>(ur + nt * 8 * HUG_KS + k0);
        const unsigned b1 = *reinterpret_cast<const unsigned*>(ur + nt * 8 * HUG_KS + k0 + 8);
        mma_bf16_16816_(acc[nt], af, b0, b1);
      }
    }
  }
  // epilogue through shared memory: a warp parks its 16 x 64 tile, then walks it row by row so that the gate is read and
  // the operand written in whole 256- and 128-byte rows (a lane owns two adjacent channels; V is even)
  static_assert(sizeof(float) * 4 * 16 * (64 + 8) <= sizeof(bf16) * 2 * 64 * HUG_KS, "epilogue tile fits the staging area");
  float (*tile)[16][64 + 8] = reinterpret_cast<float (*)[16][64 + 8]>(stage);
  __syncthreads();                                   // every warp is done with the operand slices
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    *reinterpret_cast<float2*>(&tile[warp][gid][nt * 8 + 2 * tig]) = make_float2(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<float2*>(&tile[warp][gid + 8][nt * 8 + 2 * tig]) = make_float2(acc[nt][2], acc[nt][3]);
  }
  __syncwarp();
  const int v = v0 + 2 * lane;
  if (v >= V) return;
  const int rb = blockIdx.x * 64 + warp * 16;
  float2 gv[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {                      // all gate loads of the warp's rows in flight at once
    gv[i] = make_float2(0.f, 0.f);
    if (gate != nullptr && rb + i < T) {
      const float* g = gate + static_cast<size_t>(rb + i) * ld_g + off_g + h * V + v;
      gv[i] = make_float2(g[0], g[1]);
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (rb + i >= T) continue;
    float2 o = *reinterpret_cast<const float2*>(&tile[warp][i][2 * lane]);
    if (gate != nullptr) {
      o.x *= sigmoid_(gv[i].x);
      o.y *= sigmoid_(gv[i].y);
    }
    *reinterpret_cast<__nv_bfloat162*>(out + static_cast<size_t>(rb + i) * ld_out + h * V + v) = __floats2bfloat162_rn(o.x, o.y);
  }
}

inline int last_error() { return static_cast<int>(cudaGetLastError()); }

}  // namespace

int launch_head_up_gate(const void* a, int ld_a, const void* U, const float* gate, int ld_g, int off_g, void* out,
                        int ld_out, int T, int H, int V, int C, int f32, cudaStream_t s) {
  if (T <= 0 || H <= 0 || V <= 0) return 0;
  if (C <= 0 || H > 65535) return -2;
  const dim3 grid((T + 63) / 64, (V + 63) / 64, H);
  if (!f32 && C % 16 == 0 && V % 2 == 0 && ld_a % 8 == 0 && ld_out % 2 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(U) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0) {
    launch_kernel(head_up_gate_mma_kernel, grid, dim3(128), 0, s, 1u, static_cast<const bf16*>(a), ld_a,
                  static_cast<const bf16*>(U), gate, ld_g, off_g, static_cast<bf16*>(out), ld_out, T, H, V, C);
    return last_error();
  }
  if (f32)
    launch_kernel(head_up_gate_kernel<float>, grid, dim3(256), 0, s, 1u, static_cast<const float*>(a), ld_a,
                  static_cast<const float*>(U), gate, ld_g, off_g, static_cast<float*>(out), ld_out, T, H, V, C);
  else
    launch_kernel(head_up_gate_kernel<bf16>, grid, dim3(256), 0, s, 1u, static_cast<const bf16*>(a), ld_a,
                  static_cast<const bf16*>(U), gate, ld_g, off_g, static_cast<bf16*>(out), ld_out, T, H, V, C);
  return last_error();
}

int launch_post_norm_join(float* x, const int* rows, int n_rows, const float* y, int ld_y, const float* gate, int ld_g,
                          int off_g, const float* gbias, const float* idw, float alpha, const float* w, int groups,
                          float eps, void* h, int ld_h, int W, int f32, cudaStream_t s) {
  if (n_rows <= 0) return 0;
  if (groups <= 0 || W % groups != 0) return -2;
  auto al16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (W % 4 == 0 && (W / groups) % 128 == 0 && W <= 4096 && ld_y % 4 == 0 && ld_g % 4 == 0 && off_g % 4 == 0 &&
      ld_h % 4 == 0 && al16(x) && al16(y) && al16(gate) && al16(gbias) && al16(w) && al16(h)) {
    const int nch = W <= 1024 ? 1 : (W <= 2048 ? 2 : 4);
#define B2B_PNW(OT, N)                                                                                                  \
  launch_kernel(post_norm_join_wide_kernel<OT, N>, dim3(n_rows), dim3(256), 0, s, 1u, x, rows, n_rows, y, ld_y, gate, ld_g, \
                off_g, gbias, idw, alpha, w, groups, eps, static_cast<OT*>(h), ld_h, W)
    if (f32) {
      if (nch == 1) B2B_PNW(float, 1);
      else if (nch == 2) B2B_PNW(float, 2);
      else B2B_PNW(float, 4);
    } else {
      if (nch == 1) B2B_PNW(bf16, 1);
      else if (nch == 2) B2B_PNW(bf16, 2);
      else B2B_PNW(bf16, 4);
    }
#undef B2B_PNW
    return last_error();
  }
  const long long warps = static_cast<long long>(n_rows) * groups;
  const dim3 grid(static_cast<unsigned>((warps + PNJ_WARPS - 1) / PNJ_WARPS)), block(32 * PNJ_WARPS);
  const int per_lane = (W / groups + 31) / 32;
#define B2B_PNJ(OT, PT)                                                                                                 \
  launch_kernel(post_norm_join_kernel<OT, PT>, grid, block, 0, s, 1u, x, rows, n_rows, y, ld_y, gate, ld_g, off_g, gbias, \
                idw, alpha, w, groups, eps, static_cast<OT*>(h), ld_h, W)
#define B2B_PNJ_T(OT)                                                                                                   \
  if (per_lane <= 2) B2B_PNJ(OT, 2);                                                                                    \
  else if (per_lane <= 4) B2B_PNJ(OT, 4);                                                                               \
  else if (per_lane <= 8) B2B_PNJ(OT, 8);                                                                               \
  else if (per_lane <= 16) B2B_PNJ(OT, 16);                                                                             \
  else B2B_PNJ(OT, 0)
  if (f32) {
    B2B_PNJ_T(float);
  } else {
    B2B_PNJ_T(bf16);
  }
#undef B2B_PNJ_T
#undef B2B_PNJ
  return last_error();
}

int launch_latent_prep(const float* proj, int ld, int off_q, int q_rank, int off_kv, int C, int R, const float* wq,
                       const float* wc, const float* freq, int rdims, const int* positions, const int* slots, void* cq,
                       int ld_cq, void* k_cache, float eps, int T, int f32, float amp, const float* freq_lo,
                       cudaStream_t s) {
  if (T <= 0) return 0;
  if (rdims < 0 || rdims > R || rdims % 2 != 0) return -2;
  const dim3 grid((T + LAT_WARPS - 1) / LAT_WARPS), block(32 * LAT_WARPS);
  if (f32)
    launch_kernel(latent_prep_kernel<float, float>, grid, block, 0, s, 1u, proj, ld, off_q, q_rank, off_kv, C, R, wq, wc,
                  freq, rdims, positions, slots, static_cast<float*>(cq), ld_cq, static_cast<float*>(k_cache), eps, T, amp, freq_lo);
  else
    launch_kernel(latent_prep_kernel<bf16, bf16>, grid, block, 0, s, 1u, proj, ld, off_q, q_rank, off_kv, C, R, wq, wc,
                  freq, rdims, positions, slots, static_cast<bf16*>(cq), ld_cq, static_cast<bf16*>(k_cache), eps, T, amp, freq_lo);
  return last_error();
}

int launch_rot_heads(const float* src, int ld, int off, float* dst, int H, int Dh, const float* freq, int rdims,
                     const int* positions, const int* slots, int T, int roff, float amp, const float* freq_lo,
                     cudaStream_t s) {
  const long long n = static_cast<long long>(T) * H * Dh;
  if (n <= 0) return 0;
  if (roff < 0 || roff + rdims > Dh || rdims % 2 != 0) return -2;
  launch_kernel(rot_heads_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s, 1u, src, ld, off, dst, H, Dh,
                freq, rdims, positions, slots, T, roff, amp, freq_lo);
  return last_error();
}

int launch_moe_route(const float* proj, int ld, int off, const float* corr, int E, int n_real, int count, int keep,
                     int top, float scale, float* wt, int ld_wt, float* idw, int* sel_idx, float* sel_w, int T,
                     cudaStream_t s) {
  if (T <= 0) return 0;
  if (E <= 0 || n_real < 0 || n_real > E || count <= 0 || E % count != 0 || top <= 0 || top > E) return -2;
  if (corr == nullptr && count > 1 && keep < count) return -2;      // group-limited choice is defined on corrected scores
  int warps = 4;
  while (warps > 1 && static_cast<size_t>(warps) * 4 * E * sizeof(float) > 40 * 1024) warps /= 2;
  const size_t smem = static_cast<size_t>(warps) * 4 * E * sizeof(float);
  if (smem > 48 * 1024) return -2;
  launch_kernel(moe_route_kernel, dim3((T + warps - 1) / warps), dim3(32 * warps), smem, s, 1u, proj, ld, off, corr, E,
                n_real, count, keep, top, scale, wt, ld_wt, idw, sel_idx, sel_w, T);
  return last_error();
}

int launch_gated_cols(const float* in, int ld_in, int off_a, int off_b, const float* wt, int ld_wt, int per, void* out,
                      int ld_out, int n, int act, int T, int f32, int both, int lead, cudaStream_t s) {
  const long long tot = static_cast<long long>(T) * n;
  if (tot <= 0) return 0;
  if (n % 4 == 0 && ld_in % 4 == 0 && off_a % 4 == 0 && (wt != nullptr ? per % 4 == 0 && lead % 4 == 0 : off_b % 4 == 0) &&
      (!both || off_b % 4 == 0) &&
      ld_out % 4 == 0 && T <= 65535 && reinterpret_cast<uintptr_t>(in) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    const dim3 vgrid((n / 4 + 255) / 256, T);
    if (f32)
      launch_kernel(gated_cols_vec_kernel<float>, vgrid, dim3(256), 0, s, 1u, in, ld_in, off_a, off_b, wt, ld_wt, per,
                    static_cast<float*>(out), ld_out, n, act, both, lead);
    else
      launch_kernel(gated_cols_vec_kernel<bf16>, vgrid, dim3(256), 0, s, 1u, in, ld_in, off_a, off_b, wt, ld_wt, per,
                    static_cast<bf16*>(out), ld_out, n, act, both, lead);
    return last_error();
  }
  const dim3 grid(static_cast<unsigned>((tot + 255) / 256));
  if (f32)
    launch_kernel(gated_cols_kernel<float>, grid, dim3(256), 0, s, 1u, in, ld_in, off_a, off_b, wt, ld_wt, per,
                  static_cast<float*>(out), ld_out, n, act, T, both, lead);
  else
    launch_kernel(gated_cols_kernel<bf16>, grid, dim3(256), 0, s, 1u, in, ld_in, off_a, off_b, wt, ld_wt, per,
                  static_cast<bf16*>(out), ld_out, n, act, T, both, lead);
  return last_error();
}

}  // namespace b2b

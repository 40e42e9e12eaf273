// Sequence mixers of the parallel-block hybrid decoders (Repudra) and the glue around them:
//
//   * ls_join            one residual stream: x += sum_k w_k * (optionally width-normed) y_k, then the RMS norm of the
//                        next block (one gain for all coordinates, or a vector) written as the GEMM operand; optionally a
//                        second normed operand with its own weights (a norm per sublayer of a parallel block), a replace
//                        mode (the residual entering a pass of a looped range of layers) and a plain operand copy
//   * rot_attn_prep      softmax attention: RMS norm over the WHOLE q / k projection, rotary positions on the first
//                        `rdims` channels of every head (pairs 2i, 2i+1; frequencies from a table, so any scaling rule
//                        is a host matter), per-head value norm, K / V rows into the paged cache
//   * softmax_attention  causal softmax attention over the paged cache, key width != value width, grouped heads, optional
//                        window with kept first keys, optional score cap, optional sink in the denominator; an
//                        exact CUDA-core kernel (one warp per query and head, online softmax) and a tensor-core kernel
//                        for spans in the bf16 mode
//   * short_conv         causal per-channel convolution over time + silu, with the last taps-1 inputs per sequence slot
//   * mlstm_gates        the scalar part of the matrix memory (mLSTM): capped gates, running maximum, normaliser
//   * lin_scan           gated linear recurrences with an fp32 [dk, dv] state per head and sequence slot:
//                        diag-gated (GLA), delta rule with a decay per key channel, mLSTM matrix memory
//   * scan_post          per-head output norm, weight, output gate -> GEMM operand
//
// Everything the designs want in 32-bit stays in fp32: the residual, every norm, angles, attention scores and weights,
// gates, decays, step sizes, unit keys and the recurrent state.  OT / CT are the types of what feeds a matrix product
// and of the KV cache (bf16 when serving, float in the all-fp32 mode); projections arrive as fp32 GEMM outputs.
// This translation unit is compiled WITHOUT --use_fast_math (exact expf / division / sqrt / sincos).
#include "kernels.h"

#include <cuda_bf16.h>

#include <cstdint>

#include "launch.cuh"

namespace b2b {
namespace {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float ldf(const T* p, size_t i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p, size_t i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, size_t i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, size_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoid_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float silu_(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float logsigmoid_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

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
// sum over the block; every thread gets the result (sh: >= 32 floats, reusable after the call)
__device__ __forceinline__ float block_sum_(float v, float* sh) {
  v = warp_sum_(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (l < nw) ? sh[l] : 0.f;
  return warp_sum_(r);
}

// ------------------------------------------------------------------------------------------- residual join + norm
struct JoinTerm {
  const float* y;      // [rows, ld] sublayer output (null = no term)
  const float* w;      // [W] coordinate-wise scale (null = 1)
  int ld;
  int norm;            // != 0: y is divided by its root mean square over the width first
};

// x [T, W] fp32.  Token rows come from the spans (q_start, q_len) or, gathered, from `rows` (then x is not written:
// only the operand rows are wanted).  gamma: one gain (gstride 0) or W gains (gstride 1), stored as an offset from one
// when plus_one.  WPT warps per token (1: narrow models, no block barrier; LSJ_WARPS: the block is one token): pass 1
// sums the squares of the terms that are normed, pass 2 builds the new residual row (kept in shared memory) and its sum
// of squares, pass 3 writes the operand.  VEC: 16-byte accesses (W and every row stride multiples of 4).
// replace: the new residual row is the sum of the terms alone (the old row is not read).  gamma == nullptr: the operand is
// the residual row itself.  gamma2 / h2: a second normed operand of the same row (blocks whose two sublayers have a norm each).
// grid (groups of LSJ_WARPS / WPT tokens, sequences) or (groups of rows); dynamic smem LSJ_WARPS / WPT * W floats.
constexpr int LSJ_WARPS = 4;

template <bool VEC> struct Ld4;
template <> struct Ld4<true> {
  static __device__ __forceinline__ float4 ld(const float* p, int i) { return reinterpret_cast<const float4*>(p)[i]; }
  static __device__ __forceinline__ void st(float* p, int i, float4 v) { reinterpret_cast<float4*>(p)[i] = v; }
};
template <> struct Ld4<false> {          // one element per "vector": only .x is used
  static __device__ __forceinline__ float4 ld(const float* p, int i) { return make_float4(p[i], 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ void st(float* p, int i, float4 v) { p[i] = v.x; }
};
__device__ __forceinline__ void st_operand(float* h, int i, float4 v, bool vec) {
  if (vec) reinterpret_cast<float4*>(h)[i] = v;
  else h[i] = v.x;
}
__device__ __forceinline__ void st_operand(bf16* h, int i, float4 v, bool vec) {
  if (vec) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&a);
    u.y = *reinterpret_cast<unsigned*>(&b);
    reinterpret_cast<uint2*>(h)[i] = u;
  } else {
    h[i] = __float2bfloat16_rn(v.x);
  }
}

template <typename OT, bool VEC, int WPT>
__global__ void __launch_bounds__(32 * LSJ_WARPS)
    ls_join_kernel(float* __restrict__ x, const int* __restrict__ q_start, const int* __restrict__ q_len,
                   const int* __restrict__ rows, int n_rows, JoinTerm a, JoinTerm b, JoinTerm c, float eps,
                   const float* __restrict__ gamma, int gstride, int plus_one, OT* __restrict__ h, int ld_h, int W,
                   const float* __restrict__ gamma2, OT* __restrict__ h2, int ld_h2, int replace) {
  pdl_begin();
  extern __shared__ __align__(16) float sm[];
  __shared__ float red[32];
  constexpr int TPB = LSJ_WARPS / WPT, NL = 32 * WPT;       // tokens per block, threads per token
  const int grp = threadIdx.x / NL, lane = threadIdx.x % NL;
  float* xs = sm + static_cast<size_t>(grp) * ((W + 3) & ~3);
  auto total = [&](float v) { return WPT == 1 ? warp_sum_(v) : block_sum_(v, red); };
  int t, hrow;
  if (rows != nullptr) {
    hrow = blockIdx.x * TPB + grp;
    if (hrow >= n_rows) return;                              // (block-uniform when the block is one token)
    t = rows[hrow];
  } else {
    const int sq = blockIdx.y, n = q_len[sq], i = blockIdx.x * TPB + grp;
    if (i >= n) return;
    t = q_start[sq] + i;
    hrow = t;
  }
  constexpr int E = VEC ? 4 : 1;
  const int nv = W / E;
  const JoinTerm terms[3] = {a, b, c};
  const float inv_w = 1.f / static_cast<float>(W);
  float r[3] = {1.f, 1.f, 1.f};
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    if (terms[k].y == nullptr || !terms[k].norm) continue;
    const float* y = terms[k].y + static_cast<size_t>(t) * terms[k].ld;
    float ss = 0.f;
    for (int i = lane; i < nv; i += NL) {
      const float4 v = Ld4<VEC>::ld(y, i);
      ss += v.x * v.x + (VEC ? v.y * v.y + v.z * v.z + v.w * v.w : 0.f);
    }
    r[k] = 1.f / sqrtf(total(ss) * inv_w + eps);
  }
  float* xr = x + static_cast<size_t>(t) * W;
  float ss = 0.f;
  for (int i = lane; i < nv; i += NL) {
    float4 v = replace ? make_float4(0.f, 0.f, 0.f, 0.f) : Ld4<VEC>::ld(xr, i);
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      if (terms[k].y == nullptr) continue;
      float4 yv = Ld4<VEC>::ld(terms[k].y + static_cast<size_t>(t) * terms[k].ld, i);
      float4 wv = make_float4(1.f, 1.f, 1.f, 1.f);
      if (terms[k].w != nullptr) wv = Ld4<VEC>::ld(terms[k].w, i);
      v.x += yv.x * r[k] * wv.x;
      if (VEC) {
        v.y += yv.y * r[k] * wv.y;
        v.z += yv.z * r[k] * wv.z;
        v.w += yv.w * r[k] * wv.w;
      }
    }
    ss += v.x * v.x + (VEC ? v.y * v.y + v.z * v.z + v.w * v.w : 0.f);
    Ld4<VEC>::st(xs, i, v);
    if (rows == nullptr) Ld4<VEC>::st(xr, i, v);
  }
  if (h == nullptr) return;
  // gamma == nullptr: the operand is the residual row itself (no norm)
  const float tot = total(ss);                             // (the block barriers inside also order xs for WPT > 1)
  const float rn = gamma != nullptr ? 1.f / sqrtf(tot * inv_w + eps) : 1.f;
  const float one = plus_one ? 1.f : 0.f;
  const float g0 = gamma != nullptr ? gamma[0] + one : 1.f;
  OT* hr = h + static_cast<size_t>(hrow) * ld_h;
  OT* hr2 = h2 != nullptr ? h2 + static_cast<size_t>(hrow) * ld_h2 : nullptr;
  __syncwarp();
  for (int i = lane; i < nv; i += NL) {
    const float4 xv = Ld4<VEC>::ld(xs, i);
    float4 g = make_float4(g0, g0, g0, g0);
    if (gstride) {
      g = Ld4<VEC>::ld(gamma, i);
      g.x += one; g.y += one; g.z += one; g.w += one;
    }
    float4 v = xv;
    v.x *= rn * g.x; v.y *= rn * g.y; v.z *= rn * g.z; v.w *= rn * g.w;
    st_operand(hr, i, v, VEC);
    if (hr2 != nullptr) {                                  // a second norm of the same row (its own gains, always a vector)
      g = Ld4<VEC>::ld(gamma2, i);
      v = xv;
      v.x *= rn * (g.x + one); v.y *= rn * (g.y + one); v.z *= rn * (g.z + one); v.w *= rn * (g.w + one);
      st_operand(hr2, i, v, VEC);
    }
  }
}

// -------------------------------------------------------------------- softmax attention: norms, rotation, cache
// proj [T, ld] fp32 holds q (H*D) at off_q, k (G*D) at off_k, v (G*V) at off_v.  One block per token.
// freq [rdims / 2]: angle of pair i at position p = p * freq[i] (fp32 product); cos and sin are multiplied by amp.
constexpr int ROT_MAX_PAIRS = 128;      // rotated pairs per head: rdims <= 256

__device__ __forceinline__ void st_pair(float* p, size_t i, float a, float b) {
  *reinterpret_cast<float2*>(p + i) = make_float2(a, b);
}
__device__ __forceinline__ void st_pair(bf16* p, size_t i, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p + i) = __floats2bfloat162_rn(a, b);
}

// PAIRS: D is even and every row offset too, so a thread handles the two channels of a pair with 8-byte accesses
template <typename CT, bool PAIRS>
__global__ void __launch_bounds__(256)
    rot_attn_prep_kernel(const float* __restrict__ proj, int ld, int off_q, int off_k, int off_v,
                         const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ freq,
                         int rdims, float amp, const int* __restrict__ positions, const int* __restrict__ slots,
                         float* __restrict__ q_out, CT* __restrict__ k_cache, CT* __restrict__ v_cache, int H, int G,
                         int D, int V, float eps) {
  pdl_begin();
  __shared__ float red[32];
  __shared__ float cs_s[ROT_MAX_PAIRS], sn_s[ROT_MAX_PAIRS];
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;                               // padding row of a bucketed chunk (block-uniform)
  if (threadIdx.x < rdims / 2) {                      // the angles are the same for every head: once per token
    float sn, cs;
    sincosf(static_cast<float>(positions[t]) * freq[threadIdx.x], &sn, &cs);
    cs_s[threadIdx.x] = cs * amp;
    sn_s[threadIdx.x] = sn * amp;
  }
  const float* row = proj + static_cast<size_t>(t) * ld;
  const float* qr = row + off_q;
  const float* kr = row + off_k;
  const int nq = H * D, nk = G * D;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq; i += blockDim.x) sq += qr[i] * qr[i];
  for (int i = threadIdx.x; i < nk; i += blockDim.x) sk += kr[i] * kr[i];
  const float rq = 1.f / sqrtf(block_sum_(sq, red) / static_cast<float>(nq) + eps);
  const float rk = 1.f / sqrtf(block_sum_(sk, red) / static_cast<float>(nk) + eps);
  if (PAIRS) {                                                  // (the block sums above are barriers: the table is there)
    for (int pe = threadIdx.x; pe < (nq + nk) / 2; pe += blockDim.x) {
      const bool isq = 2 * pe < nq;
      const int i = isq ? 2 * pe : 2 * pe - nq;
      const float2 x = *reinterpret_cast<const float2*>((isq ? qr : kr) + i);
      const float2 w = *reinterpret_cast<const float2*>((isq ? qn : kn) + i);
      const float r = isq ? rq : rk;
      float a = x.x * r * w.x, b = x.y * r * w.y;
      const int d = i % D;
      if (d < rdims) {
        const float sn = sn_s[d >> 1], cs = cs_s[d >> 1];
        const float ra = a * cs - b * sn, rb = b * cs + a * sn;
        a = ra;
        b = rb;
      }
      if (isq) st_pair(q_out, static_cast<size_t>(t) * nq + i, a, b);
      else st_pair(k_cache, static_cast<size_t>(slot) * nk + i, a, b);
    }
  }
  for (int e = threadIdx.x; e < (PAIRS ? 0 : nq + nk); e += blockDim.x) {
    const bool isq = e < nq;
    const int i = isq ? e : e - nq;
    const float* src = isq ? qr : kr;
    const float* w = isq ? qn : kn;
    const float r = isq ? rq : rk;
    const int d = i % D;
    float v = src[i] * r * w[i];
    if (d < rdims) {
      const int io = i - d + (d ^ 1);                 // the other half of the pair (2j, 2j+1)
      const float o = src[io] * r * w[io];
      const float sn = sn_s[d >> 1], cs = cs_s[d >> 1];
      v = (d & 1) ? v * cs + o * sn : v * cs - o * sn;
    }
    if (isq) q_out[static_cast<size_t>(t) * nq + i] = v;
    else stf(k_cache, static_cast<size_t>(slot) * nk + i, v);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = warp; g < G; g += blockDim.x >> 5) {
    const float* src = row + off_v + g * V;
    float ss = 0.f;
    for (int d = lane; d < V; d += 32) ss += src[d] * src[d];
    const float r = 1.f / sqrtf(warp_sum_(ss) / static_cast<float>(V) + eps);
    CT* dst = v_cache + (static_cast<size_t>(slot) * G + g) * V;
    for (int d = lane; d < V; d += 32) stf(dst, d, src[d] * r);
  }
}

// dot product of a shared-memory fp32 vector with a cache row, 128-bit loads when the row allows it
template <typename T> __device__ __forceinline__ float dot_row(const float* q, const T* k, int n, bool vec);
template <> __device__ __forceinline__ float dot_row<float>(const float* q, const float* k, int n, bool vec) {
  float acc = 0.f;
  if (vec) {
    const float4* k4 = reinterpret_cast<const float4*>(k);
    for (int d = 0; d < n / 4; ++d) {
      const float4 v = k4[d];
      acc += q[4 * d] * v.x + q[4 * d + 1] * v.y + q[4 * d + 2] * v.z + q[4 * d + 3] * v.w;
    }
  } else {
    for (int d = 0; d < n; ++d) acc += q[d] * k[d];
  }
  return acc;
}
template <> __device__ __forceinline__ float dot_row<bf16>(const float* q, const bf16* k, int n, bool vec) {
  float acc = 0.f;
  if (vec) {
    const uint4* k8 = reinterpret_cast<const uint4*>(k);
    for (int d = 0; d < n / 8; ++d) {
      const uint4 v = k8[d];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p[j]);
        acc += q[8 * d + 2 * j] * f.x + q[8 * d + 2 * j + 1] * f.y;
      }
    }
  } else {
    for (int d = 0; d < n; ++d) acc += q[d] * __bfloat162float(k[d]);
  }
  return acc;
}

// ------------------------------------------------------------------------------------------ softmax attention
// out[t, h, :] = sum_j softmax_j(q_t . k_j * scale) v_j over the keys j <= i, and j > i - window when window > 0
// (the first keep_first keys stay visible whatever the window).  softcap > 0: score <- softcap * tanh(score / softcap).
// sink [H] (optional): exp(sink_h) joins the denominator of head h; it has no key and no value.
// Positions count from the start of the sequence: i = kv_len - q_len + index in span.  One warp per (query, head): a
// pass over 32 keys computes one score per lane, rescales the running sums, then the lanes own value channels.
// grid (query tiles of 4, heads, sequences), 128 threads, dynamic smem 4 * D floats.
constexpr int SMX_WARPS = 4;
constexpr int SMX_VR = 8;          // value channels per lane: V <= 256 (VR = 16 for wider values, V <= 512)
constexpr int SMX_MMA_MIN_Q = 16;  // spans from this length on run on the tensor-core variant (bf16 mode)
constexpr int SMX_MMA_WARPS = 4;   // warps (of 16 queries) per block of the tensor-core variant (8 measured slower:
                                   // fewer blocks, and the early warps of a tile idle at the page barriers)
constexpr int SMX_DEC_WARPS = 8;   // warps that share one (query, head) in decode steps
constexpr int SMX_DEC_MAX_Q = 2;   // spans up to this length run the decode variant

// WPQ = 1: a block holds SMX_WARPS queries, one warp each.  WPQ > 1 (decode steps and very short spans): a block is ONE
// (query, head); its WPQ warps take the 32-key passes in turn and their partial (maximum, sum, values) are merged through
// shared memory, so a long context is read by WPQ warps at once.
template <typename CT, typename OT, int WPQ, int VR = SMX_VR>
__global__ void __launch_bounds__(32 * (WPQ > 1 ? WPQ : SMX_WARPS))
    softmax_attention_kernel(const float* __restrict__ q, const CT* __restrict__ k_cache, const CT* __restrict__ v_cache,
                             OT* __restrict__ out, int ld_out, const int* __restrict__ block_table, int max_pages,
                             const int* __restrict__ q_start, const int* __restrict__ q_len,
                             const int* __restrict__ kv_len, int H, int G, int D, int V, int window, float scale, int ldv,
                             float softcap, int keep_first, const float* __restrict__ sink) {
  pdl_begin();
  extern __shared__ float qs_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.z, hd = blockIdx.y;
  const int i = WPQ > 1 ? blockIdx.x : blockIdx.x * SMX_WARPS + warp;
  const int n = q_len[s];
  if (i >= n) return;                                  // (block-uniform when WPQ > 1; no block barrier otherwise)
  const int t = q_start[s] + i;
  const int pi = kv_len[s] - n + i;
  const int lo = window > 0 ? max(0, pi - window + 1) : 0;
  const int g = hd / (H / G);
  float* qs = qs_all + (WPQ > 1 ? 0 : warp * D);
  const float* qrow = q + (static_cast<size_t>(t) * H + hd) * D;
  if (WPQ > 1) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = qrow[d] * scale;
    __syncthreads();
  } else {
    for (int d = lane; d < D; d += 32) qs[d] = qrow[d] * scale;
    __syncwarp();
  }
  const int* bt = block_table + static_cast<size_t>(s) * max_pages;
  const bool kvec = (D * sizeof(CT)) % 16 == 0;
  float acc[VR];
#pragma unroll
  for (int r = 0; r < VR; ++r) acc[r] = 0.f;
  // sink: a learned score per head that takes part in the denominator only (a key whose value is zero); it starts the
  // running maximum and sum of ONE warp of the query
  float mx = -INFINITY, den = 0.f;
  if (sink != nullptr && (WPQ == 1 || warp == 0)) {
    mx = sink[hd];
    den = 1.f;
  }
  const int stride = WPQ > 1 ? 32 * WPQ : 32;
  // visible keys: [0, kf) -- the first keep_first keys, kept in sight when the window has moved past them -- and [lo, pi]
  const int kf = min(keep_first, lo);
  for (int seg = kf > 0 ? 0 : 1; seg < 2; ++seg) {
    const int jbeg = seg == 0 ? 0 : lo, jend = seg == 0 ? kf - 1 : pi;
    for (int j0 = jbeg + (WPQ > 1 ? 32 * warp : 0); j0 <= jend; j0 += stride) {
      const int j = j0 + lane;
      float sc = -INFINITY;
      long long slot = 0;
      if (j <= jend) {
        slot = static_cast<long long>(bt[j >> 6]) * 64 + (j & 63);
        sc = dot_row<CT>(qs, k_cache + (static_cast<size_t>(slot) * G + g) * D, D, kvec);
        if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
      }
      const float nmx = fmaxf(mx, warp_max_(sc));        // finite: key j0 is always visible
      const float corr = expf(mx - nmx);                 // first pass: exp(-inf) = 0
      const float p = (j <= jend) ? expf(sc - nmx) : 0.f;
      den = den * corr + warp_sum_(p);
      mx = nmx;
#pragma unroll
      for (int r = 0; r < VR; ++r) acc[r] *= corr;
      const int cnt = min(32, jend - j0 + 1);
      for (int jj = 0; jj < cnt; ++jj) {
        const float w = __shfl_sync(0xffffffffu, p, jj);
        const long long sl = __shfl_sync(0xffffffffu, slot, jj);
        const CT* vrow = v_cache + static_cast<size_t>(sl) * ldv + g * V;
#pragma unroll
        for (int r = 0; r < VR; ++r) {
          const int d = lane + 32 * r;
          if (d < V) acc[r] += w * ldf(vrow, d);
        }
      }
    }
  }
  if (WPQ > 1) {
    // merge the warps' partial results: part[w] = (maximum, sum, values[V])
    float* part = qs_all + ((D + 3) & ~3);
    const int ps = V + 2;
    if (lane == 0) {
      part[warp * ps] = mx;
      part[warp * ps + 1] = den;
    }
#pragma unroll
    for (int r = 0; r < VR; ++r) {
      const int d = lane + 32 * r;
      if (d < V) part[warp * ps + 2 + d] = acc[r];
    }
    __syncthreads();
    if (warp != 0) return;
    float M = -INFINITY;
    for (int w = 0; w < WPQ; ++w) M = fmaxf(M, part[w * ps]);
    den = 0.f;
#pragma unroll
    for (int r = 0; r < VR; ++r) acc[r] = 0.f;
    for (int w = 0; w < WPQ; ++w) {
      const float c = expf(part[w * ps] - M);            // a warp that saw no key: exp(-inf) = 0
      den += part[w * ps + 1] * c;
#pragma unroll
      for (int r = 0; r < VR; ++r) {
        const int d = lane + 32 * r;
        if (d < V) acc[r] += part[w * ps + 2 + d] * c;
      }
    }
  }
  const float inv = 1.f / den;
#pragma unroll
  for (int r = 0; r < VR; ++r) {
    const int d = lane + 32 * r;
    if (d < V) stf(out, static_cast<size_t>(t) * ld_out + hd * V + d, acc[r] * inv);
  }
}

// ---- tensor-core variant for spans (bf16 serving mode): S = Q K^T and O = P V as m16n8k16 bf16 MMAs with fp32
// accumulators; scores, masks, running maximum and sums are fp32 on the accumulator fragments, P is rounded to bf16 only
// as the operand of the second product (so the exponentials use the 2e-7-relative hardware exp2).  A block = 64 consecutive queries of one (sequence, head), a warp = 16 of them;
// key tiles are whole KV pages (64 keys) staged in shared memory.  DT / VT: key / value width in units of 16 channels
// (zero-padded in shared memory).
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void ldsm_x2_trans(unsigned& r0, unsigned& r1, const void* p) {
  const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}

template <int DT, int VT>
__global__ void __launch_bounds__(32 * SMX_MMA_WARPS, 3)
    softmax_attention_mma_kernel(const float* __restrict__ q, const bf16* __restrict__ k_cache,
                                 const bf16* __restrict__ v_cache, bf16* __restrict__ out, int ld_out,
                                 const int* __restrict__ block_table, int max_pages, const int* __restrict__ q_start,
                                 const int* __restrict__ q_len, const int* __restrict__ kv_len, int H, int G, int D,
                                 int V, int window, float scale, int ldv, int hg, float softcap, int keep_first,
                                 const float* __restrict__ sink) {
  // hg == 1: a block = 64 consecutive queries of one head (blockIdx.y).  hg > 1 (= H / G): the hg query heads that share
  // key/value head blockIdx.y are stacked into the rows of the tile, row r = (query r / hg, head r % hg of the group), so a
  // page is staged once for all of them and a decode step of one sequence fills hg rows instead of one.
  pdl_begin();
  constexpr int DP = 16 * DT, VP = 16 * VT, KS = DP + 8, VS = VP + 8;
  __shared__ __align__(16) bf16 Ks[64 * KS];
  __shared__ __align__(16) bf16 Vs[64 * VS];
  const int s = blockIdx.z, nq = q_len[s], n = nq * hg;
  constexpr int QT = 16 * SMX_MMA_WARPS;          // rows per block
  const int ib = blockIdx.x * QT;
  if (ib >= n) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int t0 = q_start[s], pos0 = kv_len[s] - nq;
  const int g = hg > 1 ? static_cast<int>(blockIdx.y) : static_cast<int>(blockIdx.y) / (H / G);
  const int i_r0 = ib + warp * 16 + gid, i_r1 = i_r0 + 8;
  const bool ok0 = i_r0 < n, ok1 = i_r1 < n;
  // query index within the span and head of the two rows this thread holds (clamped to the block's first row when idle)
  const int rr0 = ok0 ? i_r0 : ib, rr1 = ok1 ? i_r1 : ib;
  const int qi0 = rr0 / hg, qi1 = rr1 / hg;
  const int hd0 = hg > 1 ? g * hg + rr0 % hg : static_cast<int>(blockIdx.y);
  const int hd1 = hg > 1 ? g * hg + rr1 % hg : static_cast<int>(blockIdx.y);
  const int p0 = pos0 + qi0, p1 = pos0 + qi1;
  const int lo0 = window > 0 ? max(0, p0 - window + 1) : 0, lo1 = window > 0 ? max(0, p1 - window + 1) : 0;
  const int pfirst = pos0 + ib / hg, pmax = pos0 + (min(n, ib + QT) - 1) / hg;
  const int lo_min = window > 0 ? max(0, pfirst - window + 1) : 0;
  const int wi0 = ib + warp * 16;
  const bool wact = wi0 < n;
  const int wpmin = pos0 + wi0 / hg, wpmax = pos0 + min(n - 1, wi0 + 15) / hg;
  const int wlo = window > 0 ? max(0, wpmin - window + 1) : 0;
  unsigned qa[DT][4];
  {
    const float* q0 = q + (static_cast<size_t>(t0 + qi0) * H + hd0) * D;
    const float* q1 = q + (static_cast<size_t>(t0 + qi1) * H + hd1) * D;
#pragma unroll
    for (int kk = 0; kk < DT; ++kk) {
      const int c0 = kk * 16 + 2 * tig, c1 = c0 + 8;
      const bool a = c0 < D, b = c1 < D;
      qa[kk][0] = (ok0 && a) ? pack_bf16x2(q0[c0] * scale, q0[c0 + 1] * scale) : 0u;
      qa[kk][1] = (ok1 && a) ? pack_bf16x2(q1[c0] * scale, q1[c0 + 1] * scale) : 0u;
      qa[kk][2] = (ok0 && b) ? pack_bf16x2(q0[c1] * scale, q0[c1 + 1] * scale) : 0u;
      qa[kk][3] = (ok1 && b) ? pack_bf16x2(q1[c1] * scale, q1[c1 + 1] * scale) : 0u;
    }
  }
  float oacc[2 * VT][4];
#pragma unroll
  for (int vt = 0; vt < 2 * VT; ++vt) oacc[vt][0] = oacc[vt][1] = oacc[vt][2] = oacc[vt][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  if (sink != nullptr) {                           // the sink starts the running maximum; its weight 1 sits in one lane of the quad
    m0 = sink[hd0];
    m1 = sink[hd1];
    l0 = l1 = tig == 0 ? 1.f : 0.f;
  }
  const int* bt = block_table + static_cast<size_t>(s) * max_pages;
  // pages of the kept first keys that lie in front of the window's pages, then the window's pages
  const int pg_lo = lo_min >> 6;
  const int n_pre = (window > 0 && keep_first > 0) ? min((keep_first - 1) >> 6, pg_lo - 1) + 1 : 0;
  const int n_it = n_pre + (pmax >> 6) - pg_lo + 1;
  for (int it = 0; it < n_it; ++it) {
    const int pg = it < n_pre ? it : pg_lo + it - n_pre;
    const size_t page = static_cast<size_t>(bt[pg]);
    const int kb = pg * 64;
    __syncthreads();                           // every warp is done with the previous tile
    {
      const bf16* ksrc = k_cache + (page * 64 * G + g) * D;
      const bf16* vsrc = v_cache + page * 64 * ldv + g * V;
      constexpr int KC = DP / 8, VC = VP / 8;
      for (int idx = threadIdx.x; idx < 64 * KC; idx += 32 * SMX_MMA_WARPS) {
        const int r = idx / KC, c8 = idx % KC;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (c8 * 8 < D) v = *reinterpret_cast<const uint4*>(ksrc + static_cast<size_t>(r) * G * D + c8 * 8);
        *reinterpret_cast<uint4*>(Ks + r * KS + c8 * 8) = v;
      }
      for (int idx = threadIdx.x; idx < 64 * VC; idx += 32 * SMX_MMA_WARPS) {
        const int r = idx / VC, c8 = idx % VC;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        // rows past the newest key of the block may hold anything (a page that is used again): P = 0 there, but
        // 0 * NaN would still spoil the sum, so they are staged as zeros
        if (c8 * 8 < V && kb + r <= pmax) v = *reinterpret_cast<const uint4*>(vsrc + static_cast<size_t>(r) * ldv + c8 * 8);
        *reinterpret_cast<uint4*>(Vs + r * VS + c8 * 8) = v;
      }
    }
    __syncthreads();
    if (!wact || kb > wpmax || (kb + 63 < wlo && kb >= keep_first)) continue;      // warp-uniform: no key of this page is visible to the warp
    float sc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
      const bf16* krow = Ks + (nt * 8 + gid) * KS + 2 * tig;
#pragma unroll
      for (int kk = 0; kk < DT; ++kk) {
        const unsigned b0 = *reinterpret_cast<const unsigned*>(krow + kk * 16);
        const unsigned b1 = *reinterpret_cast<const unsigned*>(krow + kk * 16 + 8);
        mma_bf16_16816(sc[nt], qa[kk], b0, b1);
      }
    }
    // masks and the running maximum of the two rows this thread holds (shared with the 3 other lanes of its quad)
    float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int j0 = kb + nt * 8 + 2 * tig, j1 = j0 + 1;
      if (softcap > 0.f) {
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[nt][e] = softcap * tanhf(sc[nt][e] / softcap);
      }
      sc[nt][0] = (ok0 && (j0 >= lo0 || j0 < keep_first) && j0 <= p0) ? sc[nt][0] : -INFINITY;
      sc[nt][1] = (ok0 && (j1 >= lo0 || j1 < keep_first) && j1 <= p0) ? sc[nt][1] : -INFINITY;
      sc[nt][2] = (ok1 && (j0 >= lo1 || j0 < keep_first) && j0 <= p1) ? sc[nt][2] : -INFINITY;
      sc[nt][3] = (ok1 && (j1 >= lo1 || j1 < keep_first) && j1 <= p1) ? sc[nt][3] : -INFINITY;
      tm0 = fmaxf(tm0, fmaxf(sc[nt][0], sc[nt][1]));
      tm1 = fmaxf(tm1, fmaxf(sc[nt][2], sc[nt][3]));
    }
    tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1));
    tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
    tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1));
    tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
    const float n0 = fmaxf(m0, tm0), n1 = fmaxf(m1, tm1);
    // a row that sees no key of this page and none before keeps maximum -inf: use 0 as the reference so no NaN appears
    const float r0 = n0 == -INFINITY ? 0.f : n0, r1 = n1 == -INFINITY ? 0.f : n1;
    const float c0 = __expf(m0 - r0), c1 = __expf(m1 - r1);
    m0 = n0;
    m1 = n1;
    float s0 = 0.f, s1 = 0.f;
    unsigned pa[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float w00 = __expf(sc[nt][0] - r0), w01 = __expf(sc[nt][1] - r0);
      const float w10 = __expf(sc[nt][2] - r1), w11 = __expf(sc[nt][3] - r1);
      s0 += w00 + w01;
      s1 += w10 + w11;
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(w00, w01);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(w10, w11);
    }
    l0 = l0 * c0 + s0;
    l1 = l1 * c1 + s1;
#pragma unroll
    for (int vt = 0; vt < 2 * VT; ++vt) {
      oacc[vt][0] *= c0;
      oacc[vt][1] *= c0;
      oacc[vt][2] *= c1;
      oacc[vt][3] *= c1;
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const bf16* vrow = Vs + (kk * 16 + (lane & 15)) * VS;
#pragma unroll
      for (int vt = 0; vt < 2 * VT; ++vt) {
        unsigned b0, b1;
        ldsm_x2_trans(b0, b1, vrow + vt * 8);
        mma_bf16_16816(oacc[vt], pa[kk], b0, b1);
      }
    }
  }
  if (!wact) return;
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = ok0 ? 1.f / l0 : 0.f, i1 = ok1 ? 1.f / l1 : 0.f;
#pragma unroll
  for (int vt = 0; vt < 2 * VT; ++vt) {
    const int col = vt * 8 + 2 * tig;
    if (col >= V) continue;
    if (ok0) {
      const size_t t = static_cast<size_t>(t0 + qi0);
      *reinterpret_cast<unsigned*>(out + t * ld_out + hd0 * V + col) = pack_bf16x2(oacc[vt][0] * i0, oacc[vt][1] * i0);
    }
    if (ok1) {
      const size_t t = static_cast<size_t>(t0 + qi1);
      *reinterpret_cast<unsigned*>(out + t * ld_out + hd1 * V + col) = pack_bf16x2(oacc[vt][2] * i1, oacc[vt][3] * i1);
    }
  }
}

// ---------------------------------------------------------------------------------------- short convolution
// y[t, c] = silu(sum_j w[c, j] * x[t - (taps-1) + j, c]) per sequence; inputs before the span come from
// tail [slots, taps-1, C] (oldest first; zeros when the span starts the sequence).  x = proj columns off .. off + C.
// grid (channel blocks, token groups, sequences); a thread walks `tpt` tokens of one channel with the window in registers.
constexpr int CONV_MAX_TAPS = 8;

__global__ void __launch_bounds__(128)
    short_conv_kernel(const float* __restrict__ x, int ld_x, int off, const float* __restrict__ w,
                      const float* __restrict__ tail, float* __restrict__ y, int ld_y, const int* __restrict__ q_start,
                      const int* __restrict__ q_len, const int* __restrict__ kv_len, const int* __restrict__ seq_slot,
                      int C, int taps, int tpt) {
  pdl_begin();
  const int s = blockIdx.z, n = q_len[s];
  const int i0 = blockIdx.y * tpt;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (i0 >= n || c >= C) return;
  const int t0 = q_start[s], pos0 = kv_len[s] - n;
  const float* tl = tail + static_cast<size_t>(seq_slot[s]) * (taps - 1) * C;
  float wr[CONV_MAX_TAPS], win[CONV_MAX_TAPS];        // win[j]: input at distance taps-1-j behind the current token
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) {
    wr[j] = j < taps ? w[static_cast<size_t>(c) * taps + j] : 0.f;
    win[j] = 0.f;
    if (j < taps - 1) {
      const int i = i0 - (taps - 1) + j;                // span index of that input
      if (i >= 0) win[j] = x[static_cast<size_t>(t0 + i) * ld_x + off + c];
      else if (pos0 > 0) win[j] = tl[static_cast<size_t>(taps - 1 + i) * C + c];
    }
  }
  const int i1 = min(n, i0 + tpt);
  for (int i = i0; i < i1; ++i) {
    const float cur = x[static_cast<size_t>(t0 + i) * ld_x + off + c];
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
      if (j < taps - 1) {
        acc += wr[j] * win[j];
        win[j] = (j + 1 < taps - 1) ? win[j + 1] : cur;
      } else if (j == taps - 1) {
        acc += wr[j] * cur;
      }
    }
    y[static_cast<size_t>(t0 + i) * ld_y + c] = silu_(acc);
  }
}

// the last taps-1 inputs of every sequence -> tail (runs after the convolution of the step has read the old tail)
__global__ void short_conv_commit_kernel(const float* __restrict__ x, int ld_x, int off, float* __restrict__ tail,
                                         const int* __restrict__ q_start, const int* __restrict__ q_len,
                                         const int* __restrict__ kv_len, const int* __restrict__ seq_slot, int C,
                                         int taps) {
  pdl_begin();
  const int s = blockIdx.y, n = q_len[s];
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (n <= 0 || c >= C) return;
  const int t0 = q_start[s], pos0 = kv_len[s] - n;
  float* tl = tail + static_cast<size_t>(seq_slot[s]) * (taps - 1) * C;
  float nv[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) {
    nv[j] = 0.f;
    if (j < taps - 1) {
      const int i = n - (taps - 1) + j;
      if (i >= 0) nv[j] = x[static_cast<size_t>(t0 + i) * ld_x + off + c];
      else if (pos0 > 0) nv[j] = tl[static_cast<size_t>(taps - 1 + i) * C + c];
    }
  }
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j)
    if (j < taps - 1) tl[static_cast<size_t>(j) * C + c] = nv[j];
}

// --------------------------------------------------------------------------------- mLSTM: gates and normaliser
// Per (sequence, head), token by token (mx starts at 0, n at zero):
//     i = cap tanh((x_i + b_i) / cap)        f = logsigmoid(cap tanh((x_f + b_f) / cap))
//     mx' = max(f + mx, i)      keep = exp(f + mx - mx')      take = exp(i - mx')      n' = keep n + take k
// aux[t, head] = (keep, take, exp(-mx'), n' . q * qscale).  The matrix part of the memory runs in lin_scan with keep
// and take; scan_post divides by max(|n . q|, exp(-mx')) + 1e-6.  One warp per (sequence, head), key channels over lanes.
// Tiles of GATE_TT tokens: the k / q rows of the next tile stream into shared memory (cp.async) while this one is worked
// on; the gates of a tile are computed by one lane per token (the tanh / log / exp arithmetic of 32 tokens at once); the
// running maximum and the normaliser walk the tokens one by one, on registers and shared memory.
constexpr int GATE_R = 8;          // key channels per lane: dk <= 256
constexpr int GATE_TT = 32;        // tokens per tile (one lane per token for the gate arithmetic)

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// grid: one warp (= block) per (sequence, head); dynamic smem 2 buffers x 2 (k, q) x GATE_TT x dk + GATE_TT x 33 floats
__global__ void __launch_bounds__(32)
    mlstm_gates_kernel(const float* __restrict__ proj, int ld, int off_q, int off_k, int off_i, int off_f,
                       const float* __restrict__ bi, const float* __restrict__ bf_, float cap, float qscale,
                       float* __restrict__ nstate, float* __restrict__ mstate, float* __restrict__ aux,
                       const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ kv_len,
                       const int* __restrict__ seq_slot, int n_seqs, int H, int dk) {
  pdl_begin();
  extern __shared__ __align__(16) float gsm[];
  const int wid = blockIdx.x, lane = threadIdx.x;
  const int s = wid / H, hd = wid % H;
  const int n = q_len[s];
  if (n <= 0) return;
  const int t0 = q_start[s], pos0 = kv_len[s] - n;
  const size_t so = static_cast<size_t>(seq_slot[s]) * H + hd;
  float* kbuf = gsm;                                    // [2][GATE_TT][dk]
  float* qbuf = gsm + 2 * GATE_TT * dk;
  float* red = gsm + 4 * GATE_TT * dk;                  // [GATE_TT][33]
  float nr[GATE_R];
#pragma unroll
  for (int r = 0; r < GATE_R; ++r) {
    const int i = lane + 32 * r;
    nr[r] = (pos0 > 0 && i < dk) ? nstate[so * dk + i] : 0.f;
  }
  float mx0 = pos0 > 0 ? mstate[so] : 0.f;
  const float b_i = bi[hd], b_f = bf_[hd], icap = 1.f / cap;
  // 16-byte copies when every row piece starts on a 16-byte boundary
  const bool v16 = ((dk | ld | off_k | off_q) & 3) == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0;
  auto fetch = [&](int tb, int buf) {
    const int nt = min(GATE_TT, n - tb);
    for (int tt = 0; tt < nt; ++tt) {
      const float* row = proj + static_cast<size_t>(t0 + tb + tt) * ld + hd * dk;
      float* kd = kbuf + (buf * GATE_TT + tt) * dk;
      float* qd = qbuf + (buf * GATE_TT + tt) * dk;
      if (v16) {
        for (int ch = 4 * lane; ch < dk; ch += 128) {
          cp_async16(kd + ch, row + off_k + ch);
          cp_async16(qd + ch, row + off_q + ch);
        }
      } else {
        for (int ch = lane; ch < dk; ch += 32) {
          cp_async4(kd + ch, row + off_k + ch);
          cp_async4(qd + ch, row + off_q + ch);
        }
      }
    }
    cp_async_commit();
  };
  const int ntiles = (n + GATE_TT - 1) / GATE_TT;
  fetch(0, 0);
  float xi = 0.f, xf = 0.f;                             // gate pre-activations of this lane's token, fetched a tile ahead
  if (lane < GATE_TT && lane < n) {
    const float* row = proj + static_cast<size_t>(t0 + lane) * ld;
    xi = row[off_i + hd];
    xf = row[off_f + hd];
  }
  for (int it = 0; it < ntiles; ++it) {
    const int tb = it * GATE_TT, nt = min(GATE_TT, n - tb), buf = it & 1;
    if (it + 1 < ntiles) fetch(tb + GATE_TT, buf ^ 1);
    else cp_async_commit();
    // gates of the tile, one lane per token
    float fg = 0.f, ig = -INFINITY;
    if (lane < nt) {
      ig = cap * tanhf((xi + b_i) * icap);
      fg = logsigmoid_(cap * tanhf((xf + b_f) * icap));
    }
    if (lane < GATE_TT && tb + GATE_TT + lane < n) {
      const float* row = proj + static_cast<size_t>(t0 + tb + GATE_TT + lane) * ld;
      xi = row[off_i + hd];
      xf = row[off_f + hd];
    }
    // running maximum mx_t = max(f_t + mx_(t-1), i_t): an add and a max per token, walked by every lane alike (the
    // exponentials are not on this chain); lane t keeps its own mx_(t-1) and mx_t
    float mt = mx0, mprev = mx0;
    {
      float run = mx0;
#pragma unroll 8
      for (int tt = 0; tt < nt; ++tt) {
        const float f_t = __shfl_sync(0xffffffffu, fg, tt), i_t = __shfl_sync(0xffffffffu, ig, tt);
        const float nxt = fmaxf(f_t + run, i_t);
        if (lane == tt) {
          mprev = run;
          mt = nxt;
        }
        run = nxt;
      }
      mx0 = run;
    }
    const float keep = expf(fg + mprev - mt), take = lane < nt ? expf(ig - mt) : 0.f;
    cp_async_wait<1>();                                 // this tile's rows have landed (the next tile's may be in flight)
    __syncwarp();
    // (unrolled: only the normaliser itself is carried from token to token, the shuffles and shared-memory loads of
    // four tokens are in flight together)
#pragma unroll 4
    for (int tt = 0; tt < nt; ++tt) {
      const float kp = __shfl_sync(0xffffffffu, keep, tt), tk = __shfl_sync(0xffffffffu, take, tt);
      const float* kr = kbuf + (buf * GATE_TT + tt) * dk;
      const float* qr = qbuf + (buf * GATE_TT + tt) * dk;
      float dot = 0.f;
#pragma unroll
      for (int r = 0; r < GATE_R; ++r) {
        const int ch = lane + 32 * r;
        if (ch < dk) {
          nr[r] = kp * nr[r] + tk * kr[ch];
          dot += nr[r] * qr[ch];
        }
      }
      red[tt * 33 + lane] = dot * qscale;
    }
    __syncwarp();
    if (lane < nt) {
      float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 32; ++j) d4[j & 3] += red[lane * 33 + j];
      const float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
      float4* a = reinterpret_cast<float4*>(aux + (static_cast<size_t>(t0 + tb + lane) * H + hd) * 4);
      *a = make_float4(keep, take, expf(-mt), dot);
    }
    __syncwarp();
  }
#pragma unroll
  for (int r = 0; r < GATE_R; ++r) {
    const int i = lane + 32 * r;
    if (i < dk) nstate[so * dk + i] = nr[r];
  }
  if (lane == 0) mstate[so] = mx0;
}

// ------------------------------------------------------------------------------------ gated linear recurrences
// Per head, state S [dk, dv] (fp32, one per sequence slot); per token with a decay d in R^dk, keys k, queries q in R^dk,
// values v in R^dv:
//     S <- diag(d) S;   u = DELTA ? beta (v - S^T k) : v;   S <- S + k u^T;   o = S^T q
// What d, k, q, beta are is the mode's business and is prepared per token by the staging warps:
//     LS_GLA    q = x_q * qscale, k = x_k, d = sigmoid(z + bias)^(1/tau)             (z = low-rank projection)
//     LS_DELTA  q = unit(x_q) * qscale, k = unit(x_k)  (x after the short convolution; head h reads q/k head h / (H/G)),
//               d = exp(-exp(A_h) softplus(z + bias)), beta = sigmoid(x_b)
//     LS_MLSTM  q = x_q * qscale, k = take * x_k, d = keep   (keep, take from mlstm_gates)
//     LS_HGRN2  q = silu(x_q), d = lo + (1 - lo) sigmoid(z + bias), k = 1 - d   (keyless: the write strength is the
//               complement of the forget gate; lo [H * dk] = hparam bounds the gate from below, z is a plain projection)
// Columns of S are independent: a block owns CB columns of one (sequence, head); LN lanes share a column group, each with
// R key channels in registers (channel of (lane l, register m) = l + LN m; dk padded to R * LN with zeros).  Spans: while
// the scan warps walk tile i (the only token-sequential work) the staging warps prepare tile i + 1 in the other half of a
// double buffer; decode steps (DEC): every span is one token, all threads stage, then scan.
enum { LS_GLA = 0, LS_DELTA = 1, LS_MLSTM = 2, LS_HGRN2 = 3 };
// staging threads of a span block (8 warps with one token each per tile measured no better than 4 with two)
__host__ __device__ constexpr int ls_stage_threads(int) { return 128; }
// state columns per thread: 2 for spans; 4 with 16-byte state accesses for decode steps (a stream over the states)
__host__ __device__ constexpr int ls_cols(bool dec) { return dec ? 4 : 2; }

struct ScanArgs {
  const float* qk;  int ld_qk, off_q, off_k;      // q / k source rows
  const float* v;   int ld_v, off_v;
  const float* z;   int ld_z, off_z;              // low-rank decay projection (GLA, DELTA)
  const float* zbias;                             // [H * dk]
  const float* hparam;                            // DELTA: A_log [H]; HGRN2: lower bound of the forget gate [H * dk]
  const float* beta; int ld_b, off_b;             // DELTA: write strength before the sigmoid
  const float* aux;                               // MLSTM: [T, H, 4]
  float qscale, inv_tau;
  float* state; float* out; int ld_out;
  const int* q_start; const int* q_len; const int* kv_len; const int* seq_slot;
  int H, G, dk, dv;
};

template <int MODE, int R, int LN, bool DEC, int CB>
__global__ void __launch_bounds__(LN* CB / ls_cols(DEC) + (DEC ? 0 : ls_stage_threads(R* LN))) lin_scan_kernel(ScanArgs a) {
  pdl_begin();
  constexpr int C = ls_cols(DEC);
  constexpr int NSCAN = LN * CB / C;
  constexpr int NSTW = DEC ? NSCAN / 32 : ls_stage_threads(R * LN) / 32;
  constexpr int DKP = R * LN;
  constexpr int EPL = (DKP + 31) / 32;
  constexpr int TPW = DEC ? 1 : (DKP <= 128 ? 2 : 1);
  constexpr int TT = NSTW * TPW;
  constexpr int NBUF = DEC ? 1 : 2;
  static_assert(NSCAN % 32 == 0, "scan threads are whole warps");
  __shared__ __align__(16) float qs[NBUF * TT * DKP];
  __shared__ __align__(16) float ks[NBUF * TT * DKP];
  __shared__ __align__(16) float ds[NBUF * TT * DKP];
  __shared__ __align__(16) float vs[NBUF * TT * CB];
  __shared__ float bs[NBUF * TT];
  const int s = blockIdx.z, hd = blockIdx.y;
  const int n = a.q_len[s];
  if (n <= 0) return;                               // (block-uniform)
  const int H = a.H, dk = a.dk, dv = a.dv;
  const int t0 = a.q_start[s];
  const int pos0 = a.kv_len[s] - n;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool scanner = DEC || tid < NSCAN;
  const bool stager = DEC || tid >= NSCAN;
  const int sw = DEC ? warp : warp - NSCAN / 32;
  const int cgp = (tid % NSCAN) / LN, l = tid % LN;
  const int c0 = blockIdx.x * CB + cgp * C;
  const int hqk = MODE == LS_DELTA ? hd / (H / a.G) : hd;
  float* S_g = a.state + (static_cast<size_t>(a.seq_slot[s]) * H + hd) * static_cast<size_t>(dk) * dv;
  const bool vec = C == 4 && (dv % 4 == 0) && (c0 + C <= dv);        // 16-byte state accesses
  float S[C][R];
  if (scanner) {
#pragma unroll
    for (int m = 0; m < R; ++m) {
      const int i = l + LN * m;
      const bool ld_ok = pos0 > 0 && i < dk;
      if (vec) {
        float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ld_ok) v4 = *reinterpret_cast<const float4*>(S_g + static_cast<size_t>(i) * dv + c0);
        const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int c = 0; c < C; ++c) S[c][m] = v[c & 3];
      } else {
#pragma unroll
        for (int c = 0; c < C; ++c) S[c][m] = (ld_ok && c0 + c < dv) ? S_g[static_cast<size_t>(i) * dv + c0 + c] : 0.f;
      }
    }
  }
  float zb[EPL], lob[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int i = lane + 32 * e;
    zb[e] = (MODE != LS_MLSTM && stager && i < dk) ? a.zbias[hd * dk + i] : 0.f;
    lob[e] = (MODE == LS_HGRN2 && stager && i < dk) ? a.hparam[hd * dk + i] : 0.f;
  }
  const float rate = MODE == LS_DELTA ? expf(a.hparam[hd]) : 0.f;
  float pq[TPW][EPL], pk[TPW][EPL], pz[TPW][EPL], pv[TPW], pb[TPW], pd[TPW];
  const int vc = blockIdx.x * CB + lane;
  auto load_tile = [&](int tb) {
#pragma unroll
    for (int tw = 0; tw < TPW; ++tw) {
      const int tt = sw * TPW + tw;
      const bool tok = tb + tt < n;
      const size_t t = static_cast<size_t>(t0 + tb + (tok ? tt : 0));
      const float* qrow = a.qk + t * a.ld_qk + hqk * dk;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const int i = lane + 32 * e;
        const bool ok = tok && i < dk;
        pq[tw][e] = ok ? qrow[a.off_q + i] : 0.f;
        pk[tw][e] = (MODE != LS_HGRN2 && ok) ? qrow[a.off_k + i] : 0.f;
        if (MODE != LS_MLSTM) pz[tw][e] = ok ? a.z[t * a.ld_z + a.off_z + hd * dk + i] : 0.f;
      }
      pv[tw] = 0.f;
      if (CB <= 32) {
        if (tok && lane < CB && vc < dv) pv[tw] = a.v[t * a.ld_v + a.off_v + hd * dv + vc];
      }
      pb[tw] = 1.f;
      pd[tw] = 1.f;
      if (MODE == LS_DELTA) pb[tw] = tok ? a.beta[t * a.ld_b + a.off_b + hd] : 0.f;
      if (MODE == LS_MLSTM) {
        const float4 g = tok ? *reinterpret_cast<const float4*>(a.aux + (t * H + hd) * 4) : make_float4(1.f, 0.f, 0.f, 0.f);
        pd[tw] = g.x;
        pb[tw] = g.y;
      }
    }
  };
  auto stage_tile = [&](int buf) {
#pragma unroll
    for (int tw = 0; tw < TPW; ++tw) {
      const int tt = buf * TT + sw * TPW + tw;
      float rq = a.qscale, rk = 1.f;
      if (MODE == LS_DELTA) {
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          sq += pq[tw][e] * pq[tw][e];
          sk += pk[tw][e] * pk[tw][e];
        }
        rq = a.qscale / sqrtf(warp_sum_(sq) + 1e-6f);
        rk = 1.f / sqrtf(warp_sum_(sk) + 1e-6f);
      }
      if (MODE == LS_MLSTM) rk = pb[tw];
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const int i = lane + 32 * e;
        if (i < DKP) {
          const bool ok = i < dk;
          float d = 1.f;
          if (MODE == LS_GLA) d = expf(logsigmoid_(pz[tw][e] + zb[e]) * a.inv_tau);
          if (MODE == LS_DELTA) d = expf(-rate * softplus_(pz[tw][e] + zb[e]));
          if (MODE == LS_MLSTM) d = pd[tw];
          if (MODE == LS_HGRN2) {
            d = lob[e] + (1.f - lob[e]) * sigmoid_(pz[tw][e] + zb[e]);
            qs[tt * DKP + i] = silu_(pq[tw][e]);
            ks[tt * DKP + i] = ok ? 1.f - d : 0.f;
          } else {
            qs[tt * DKP + i] = pq[tw][e] * rq;
            ks[tt * DKP + i] = pk[tw][e] * rk;
          }
          ds[tt * DKP + i] = ok ? d : 0.f;
        }
      }
      if (lane < CB) vs[tt * CB + lane] = pv[tw];
      if (MODE == LS_DELTA && lane == 0) bs[tt] = sigmoid_(pb[tw]);
    }
  };
  auto scan_tile = [&](int buf, int tb, int nt) {
    float po[TT][C];
#pragma unroll
    for (int tl = 0; tl < TT; ++tl) {
      if (tl >= nt) break;
      const int tt = buf * TT + tl;
      float u[C], o[C];
#pragma unroll
      for (int c = 0; c < C; ++c) {
        u[c] = vs[tt * CB + cgp * C + c];
        o[c] = 0.f;
      }
      float kr[R];
#pragma unroll
      for (int m = 0; m < R; ++m) {
        const int o1 = tt * DKP + l + LN * m;
        const float dv_ = ds[o1];
        kr[m] = ks[o1];
#pragma unroll
        for (int c = 0; c < C; ++c) S[c][m] *= dv_;
      }
      if (MODE == LS_DELTA) {
        float part[C];
#pragma unroll
        for (int c = 0; c < C; ++c) part[c] = 0.f;
#pragma unroll
        for (int m = 0; m < R; ++m)
#pragma unroll
          for (int c = 0; c < C; ++c) part[c] += kr[m] * S[c][m];
#pragma unroll
        for (int sh = 1; sh < LN; sh *= 2)
#pragma unroll
          for (int c = 0; c < C; ++c) part[c] += __shfl_xor_sync(0xffffffffu, part[c], sh);
        const float be = bs[tt];
#pragma unroll
        for (int c = 0; c < C; ++c) u[c] = be * (u[c] - part[c]);
      }
#pragma unroll
      for (int m = 0; m < R; ++m) {
        const float qv = qs[tt * DKP + l + LN * m];
#pragma unroll
        for (int c = 0; c < C; ++c) {
          S[c][m] += kr[m] * u[c];
          o[c] += S[c][m] * qv;
        }
      }
#pragma unroll
      for (int c = 0; c < C; ++c) po[tl][c] = o[c];
    }
#pragma unroll
    for (int tl = 0; tl < TT; ++tl) {
      if (tl >= nt) break;
#pragma unroll
      for (int sh = 1; sh < LN; sh *= 2)
#pragma unroll
        for (int c = 0; c < C; ++c) po[tl][c] += __shfl_xor_sync(0xffffffffu, po[tl][c], sh);
      if (l == 0) {
        float* orow = a.out + static_cast<size_t>(t0 + tb + tl) * a.ld_out + hd * dv + c0;
#pragma unroll
        for (int c = 0; c < C; ++c)
          if (c0 + c < dv) orow[c] = po[tl][c];
      }
    }
  };
  if constexpr (DEC) {
    load_tile(0);
    stage_tile(0);
    __syncthreads();
    scan_tile(0, 0, min(TT, n));
  } else {
    const int ntiles = (n + TT - 1) / TT;
    if (stager) {
      load_tile(0);
      stage_tile(0);
    }
    __syncthreads();
    for (int it = 0; it < ntiles; ++it) {
      const int tb = it * TT;
      if (scanner) {
        scan_tile(it & 1, tb, min(TT, n - tb));
      } else if (it + 1 < ntiles) {
        load_tile(tb + TT);
        stage_tile((it + 1) & 1);
      }
      __syncthreads();
    }
  }
  if (scanner) {
#pragma unroll
    for (int m = 0; m < R; ++m) {
      const int i = l + LN * m;
      if (i >= dk) continue;
      if (vec) {
        *reinterpret_cast<float4*>(S_g + static_cast<size_t>(i) * dv + c0) =
            make_float4(S[0][m], S[1 % C][m], S[2 % C][m], S[3 % C][m]);
      } else {
#pragma unroll
        for (int c = 0; c < C; ++c)
          if (c0 + c < dv) S_g[static_cast<size_t>(i) * dv + c0 + c] = S[c][m];
      }
    }
  }
}

// o [T, H*dv] fp32 -> per head: (o / den) / sqrt(mean(.^2) + eps) * weight * act(gate) -> OT.  den (aux given, mLSTM):
// max(|n.q|, exp(-mx)) + 1e-6.  weight: [dv] shared by the heads (wshared) or [H*dv].  act: 0 sigmoid, 1 silu, 2 no gate.
// One warp per (token, head).
template <typename OT>
__global__ void scan_post_kernel(const float* __restrict__ o, int ld_o, const float* __restrict__ gate, int ld_g,
                                 int off_g, const float* __restrict__ weight, int wshared, int act,
                                 const float* __restrict__ aux, OT* __restrict__ out, int ld_out, int T, int H, int dv,
                                 float eps) {
  pdl_begin();
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(T) * H) return;
  const int t = static_cast<int>(wid / H), hd = static_cast<int>(wid % H);
  const float* src = o + static_cast<size_t>(t) * ld_o + hd * dv;
  const float* grow = act == 2 ? src : gate + static_cast<size_t>(t) * ld_g + off_g + hd * dv;
  float inv = 1.f;
  if (aux != nullptr) {
    const float4 g = *reinterpret_cast<const float4*>(aux + (static_cast<size_t>(t) * H + hd) * 4);
    inv = 1.f / (fmaxf(fabsf(g.w), g.z) + 1e-6f);
  }
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) {
    const float v = src[d] * inv;
    ss += v * v;
  }
  ss = warp_sum_(ss);
  const float r = inv / sqrtf(ss / static_cast<float>(dv) + eps);
  for (int d = lane; d < dv; d += 32) {
    const float gv = act == 2 ? 1.f : (act == 1 ? silu_(grow[d]) : sigmoid_(grow[d]));
    stf(out, static_cast<size_t>(t) * ld_out + hd * dv + d, src[d] * r * weight[wshared ? d : hd * dv + d] * gv);
  }
}

inline int last_error() { return static_cast<int>(cudaGetLastError()); }

}  // namespace

// ================================================================================================ launchers
int launch_ls_join(float* x, const int* q_start, const int* q_len, const int* rows, int n_rows, int n_seqs, int max_q,
                   const float* y0, int ld0, const float* w0, int norm0, const float* y1, int ld1, const float* w1,
                   int norm1, const float* y2, int ld2, const float* w2, int norm2, float eps, const float* gamma,
                   int gstride, int plus_one, void* h, int ld_h, int W, int f32, const float* gamma2, void* h2, int ld_h2,
                   int replace, cudaStream_t s) {
  const bool wide = W > 512;                 // wide rows: the whole block works on one token
  const int tpb = wide ? 1 : LSJ_WARPS;
  dim3 grid;
  if (rows != nullptr) {
    if (n_rows <= 0) return 0;
    grid = dim3((n_rows + tpb - 1) / tpb);
  } else {
    if (n_seqs <= 0 || max_q <= 0) return 0;
    grid = dim3((max_q + tpb - 1) / tpb, n_seqs);
  }
  const JoinTerm a{y0, w0, ld0, norm0}, b{y1, w1, ld1, norm1}, c{y2, w2, ld2, norm2};
  const size_t smem = static_cast<size_t>(tpb) * ((W + 3) & ~3) * sizeof(float);
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = W % 4 == 0 && al16(x) && (y0 == nullptr || (ld0 % 4 == 0 && al16(y0))) &&
                   (y1 == nullptr || (ld1 % 4 == 0 && al16(y1))) && (y2 == nullptr || (ld2 % 4 == 0 && al16(y2))) &&
                   al16(w0) && al16(w1) && al16(w2) && (h == nullptr || (ld_h % 4 == 0 && al16(h))) &&
                   (gstride == 0 || al16(gamma)) && (h2 == nullptr || (ld_h2 % 4 == 0 && al16(h2) && al16(gamma2)));
#define B2B_LSJ1(OT, VEC, WPT)                                                                                          \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(ls_join_kernel<OT, VEC, WPT>, cudaFuncAttributeMaxDynamicSharedMemorySize,                   \
                           static_cast<int>(smem));                                                                     \
    launch_kernel(ls_join_kernel<OT, VEC, WPT>, grid, dim3(32 * LSJ_WARPS), smem, s, 1u, x, q_start, q_len, rows, n_rows, \
                  a, b, c, eps, gamma, gstride, plus_one, static_cast<OT*>(h), ld_h, W, gamma2, static_cast<OT*>(h2),    \
                  ld_h2, replace);                                                                                      \
  } while (0)
#define B2B_LSJ(OT, VEC)                                                                                                \
  do {                                                                                                                  \
    if (wide) B2B_LSJ1(OT, VEC, LSJ_WARPS);                                                                             \
    else B2B_LSJ1(OT, VEC, 1);                                                                                          \
  } while (0)
  if (f32) {
    if (vec) B2B_LSJ(float, true);
    else B2B_LSJ(float, false);
  } else {
    if (vec) B2B_LSJ(bf16, true);
    else B2B_LSJ(bf16, false);
  }
#undef B2B_LSJ
#undef B2B_LSJ1
  return last_error();
}

int launch_rot_attn_prep(const float* proj, int ld, int off_q, int off_k, int off_v, const float* qn, const float* kn,
                         const float* freq, int rdims, float amp, const int* positions, const int* slots, float* q_out,
                         void* k_cache, void* v_cache, int T, int H, int G, int D, int V, float eps, int f32,
                         cudaStream_t s) {
  if (T <= 0) return 0;
  if (rdims > D || (rdims & 1) || rdims > 2 * ROT_MAX_PAIRS) return -2;
  const bool pairs = D % 2 == 0 && ld % 2 == 0 && off_q % 2 == 0 && off_k % 2 == 0 &&
                     (reinterpret_cast<uintptr_t>(proj) & 7) == 0 && (reinterpret_cast<uintptr_t>(qn) & 7) == 0 &&
                     (reinterpret_cast<uintptr_t>(kn) & 7) == 0 && (reinterpret_cast<uintptr_t>(q_out) & 7) == 0 &&
                     (reinterpret_cast<uintptr_t>(k_cache) & 7) == 0;
#define B2B_ROT(CT, P)                                                                                                  \
  launch_kernel(rot_attn_prep_kernel<CT, P>, dim3(T), dim3(256), 0, s, 1u, proj, ld, off_q, off_k, off_v, qn, kn, freq, \
                rdims, amp, positions, slots, q_out, static_cast<CT*>(k_cache), static_cast<CT*>(v_cache), H, G, D, V, eps)
  if (f32) {
    if (pairs) B2B_ROT(float, true);
    else B2B_ROT(float, false);
  } else {
    if (pairs) B2B_ROT(bf16, true);
    else B2B_ROT(bf16, false);
  }
#undef B2B_ROT
  return last_error();
}

int launch_softmax_attention(const float* q, const void* k_cache, const void* v_cache, void* out, int ld_out,
                             const int* block_table, int max_pages, const int* q_start, const int* q_len,
                             const int* kv_len, int n_seqs, int max_q, int H, int G, int D, int V, int window,
                             float scale, int ldv, int f32, float softcap, int keep_first, const float* sink,
                             cudaStream_t s) {
  if (n_seqs <= 0 || max_q <= 0) return 0;
  if (window <= 0) keep_first = 0;          // every earlier key is visible anyway
  if (V > 64 * SMX_VR || G <= 0 || H % G != 0) return -2;
  const bool wide_v = V > 32 * SMX_VR;      // values of 257 .. 512 channels: 16 channels per lane
  if (ldv <= 0) ldv = G * V;               // values in a cache of their own; otherwise a view into wider rows
  // short spans and decode steps of grouped heads: the heads that share a key/value head become rows of the tile
  const int hg = (H / G > 1 && max_q < 16 * SMX_MMA_WARPS) ? H / G : 1;
  // (decode steps of 4 or more grouped heads too when sequences x key/value heads fill the machine: a page is staged once
  // per key/value head instead of once per query head -- 32 sequences x 8 key/value heads of 128 channels at 512 keys: 6 %
  // off the decode step; with 2 key/value heads the 64 blocks that walk their pages one by one lose to the 8-warp kernel)
  if (!f32 && (max_q * hg >= SMX_MMA_MIN_Q || (hg >= 4 && max_q <= SMX_DEC_MAX_Q && n_seqs * G >= 256)) && D % 8 == 0 && V % 8 == 0 && D <= 128 && V <= 128 && ld_out % 2 == 0 &&
      ldv % 8 == 0 && reinterpret_cast<uintptr_t>(v_cache) % 16 == 0) {
    dim3 mgrid((max_q * hg + 16 * SMX_MMA_WARPS - 1) / (16 * SMX_MMA_WARPS), hg > 1 ? G : H, n_seqs);
    const int dt = (D + 15) / 16, vt = (V + 15) / 16;
    // key / value widths in units of 16 channels, rounded up to an instantiated size
    const int dts = dt <= 2 ? 2 : (dt <= 4 ? 4 : (dt <= 6 ? 6 : 8)), vts = vt <= 2 ? 2 : (vt <= 4 ? 4 : (vt <= 5 ? 5 : (vt <= 6 ? 6 : 8)));
#define B2B_SMXMMA(A, B)                                                                                                \
  if (dts == A && vts == B)                                                                                             \
    launch_kernel(softmax_attention_mma_kernel<A, B>, dim3(mgrid), dim3(32 * SMX_MMA_WARPS), 0, s, 1u, q,                              \
                  static_cast<const bf16*>(k_cache), static_cast<const bf16*>(v_cache), static_cast<bf16*>(out), ld_out,  \
                  block_table, max_pages, q_start, q_len, kv_len, H, G, D, V, window, scale, ldv, hg, softcap, keep_first, sink);
#define B2B_SMXROW(A) B2B_SMXMMA(A, 2) B2B_SMXMMA(A, 4) B2B_SMXMMA(A, 5) B2B_SMXMMA(A, 6) B2B_SMXMMA(A, 8)
    B2B_SMXROW(2) B2B_SMXROW(4) B2B_SMXROW(6) B2B_SMXROW(8)
#undef B2B_SMXROW
#undef B2B_SMXMMA
    return last_error();
  }
#define B2B_SMX(CT, WPQ, VR_, GRID, BLOCK, SMEM)                                                                         \
  launch_kernel(softmax_attention_kernel<CT, CT, WPQ, VR_>, dim3(GRID), dim3(BLOCK), SMEM, s, 1u, q,                     \
                static_cast<const CT*>(k_cache), static_cast<const CT*>(v_cache), static_cast<CT*>(out), ld_out,        \
                block_table, max_pages, q_start, q_len, kv_len, H, G, D, V, window, scale, ldv, softcap, keep_first, sink)
#define B2B_SMX_T(WPQ, GRID, BLOCK, SMEM)                                                                               \
  if (f32) {                                                                                                            \
    if (wide_v) B2B_SMX(float, WPQ, 2 * SMX_VR, GRID, BLOCK, SMEM);                                                     \
    else B2B_SMX(float, WPQ, SMX_VR, GRID, BLOCK, SMEM);                                                                \
  } else {                                                                                                              \
    if (wide_v) B2B_SMX(bf16, WPQ, 2 * SMX_VR, GRID, BLOCK, SMEM);                                                      \
    else B2B_SMX(bf16, WPQ, SMX_VR, GRID, BLOCK, SMEM);                                                                 \
  }
  if (max_q <= SMX_DEC_MAX_Q) {
    dim3 grid(max_q, H, n_seqs);
    const size_t smem = (static_cast<size_t>((D + 3) & ~3) + SMX_DEC_WARPS * (V + 2)) * sizeof(float);
    B2B_SMX_T(SMX_DEC_WARPS, grid, 32 * SMX_DEC_WARPS, smem)
    return last_error();
  }
  dim3 grid((max_q + SMX_WARPS - 1) / SMX_WARPS, H, n_seqs);
  const size_t smem = static_cast<size_t>(SMX_WARPS) * D * sizeof(float);
  B2B_SMX_T(1, grid, 32 * SMX_WARPS, smem)
#undef B2B_SMX_T
#undef B2B_SMX
  return last_error();
}

int launch_short_conv(const float* x, int ld_x, int off, const float* w, float* tail, float* y, int ld_y,
                      const int* q_start, const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs,
                      int max_q, int C, int taps, cudaStream_t s) {
  if (n_seqs <= 0 || max_q <= 0 || C <= 0) return 0;
  if (taps < 1 || taps > CONV_MAX_TAPS) return -2;
  const int tpt = 16;
  dim3 grid((C + 127) / 128, (max_q + tpt - 1) / tpt, n_seqs);
  launch_kernel(short_conv_kernel, grid, dim3(128), 0, s, 1u, x, ld_x, off, w, static_cast<const float*>(tail), y, ld_y,
                q_start, q_len, kv_len, seq_slot, C, taps, tpt);
  if (taps > 1)
    launch_kernel(short_conv_commit_kernel, dim3((C + 127) / 128, n_seqs), dim3(128), 0, s, 1u, x, ld_x, off, tail,
                  q_start, q_len, kv_len, seq_slot, C, taps);
  return last_error();
}

int launch_mlstm_gates(const float* proj, int ld, int off_q, int off_k, int off_i, int off_f, const float* bi,
                       const float* bf_, float cap, float qscale, float* nstate, float* mstate, float* aux,
                       const int* q_start, const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs, int H,
                       int dk, cudaStream_t s) {
  if (n_seqs <= 0) return 0;
  if (dk > 32 * GATE_R) return -2;
  const size_t smem = (static_cast<size_t>(4) * GATE_TT * dk + GATE_TT * 33) * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(mlstm_gates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  launch_kernel(mlstm_gates_kernel, dim3(n_seqs * H), dim3(32), smem, s, 1u, proj, ld, off_q, off_k, off_i, off_f, bi, bf_,
                cap, qscale, nstate, mstate, aux, q_start, q_len, kv_len, seq_slot, n_seqs, H, dk);
  return last_error();
}

template <int MODE, int R, int LN, bool DEC, int CB>
static int launch_scan_cb(const ScanArgs& a, int n_seqs, cudaStream_t s) {
  dim3 grid((a.dv + CB - 1) / CB, a.H, n_seqs);
  launch_kernel(lin_scan_kernel<MODE, R, LN, DEC, CB>, grid, dim3(LN * CB / ls_cols(DEC) + (DEC ? 0 : ls_stage_threads(R * LN))), 0, s, 1u,
                a);
  return last_error();
}

template <int MODE, int R, int LN, bool DEC>
static int launch_scan_r(const ScanArgs& a, int n_seqs, cudaStream_t s) {
  if constexpr (DEC) {
    return launch_scan_cb<MODE, R, LN, true, 16>(a, n_seqs, s);
  } else {
    // the scan of a span is sequential in its tokens: its only parallelism is heads x sequences x column blocks, so
    // narrow the column blocks until about one block per SM exists
    const long long heads = static_cast<long long>(a.H) * n_seqs;
    if (a.dv > 8 && heads * ((a.dv + 31) / 32) < 120) {
      if (heads * ((a.dv + 15) / 16) >= 120 || a.dv <= 16) return launch_scan_cb<MODE, R, LN, false, 16>(a, n_seqs, s);
      return launch_scan_cb<MODE, R, LN, false, 8>(a, n_seqs, s);
    }
    return launch_scan_cb<MODE, R, LN, false, 32>(a, n_seqs, s);
  }
}

template <int MODE>
static int launch_scan_mode(const ScanArgs& a, int n_seqs, int max_q, cudaStream_t s) {
#define B2B_SCAN(R, LN)                                                                                                 \
  return max_q <= 1 ? launch_scan_r<MODE, R, LN, true>(a, n_seqs, s) : launch_scan_r<MODE, R, LN, false>(a, n_seqs, s)
  if (a.dk <= 16) B2B_SCAN(2, 8);
  if (a.dk <= 32) B2B_SCAN(4, 8);
  if (a.dk <= 64) B2B_SCAN(4, 16);
  if (a.dk <= 128) B2B_SCAN(8, 16);
  if (a.dk <= 256) B2B_SCAN(16, 16);
#undef B2B_SCAN
  return -2;
}

int launch_lin_scan(int mode, const float* qk, int ld_qk, int off_q, int off_k, const float* v, int ld_v, int off_v,
                    const float* z, int ld_z, int off_z, const float* zbias, const float* hparam, const float* beta,
                    int ld_b, int off_b, const float* aux, float qscale, float inv_tau, float* state, float* out,
                    int ld_out, const int* q_start, const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs,
                    int max_q, int H, int G, int dk, int dv, cudaStream_t s) {
  if (n_seqs <= 0) return 0;
  if (G <= 0 || H % G != 0) return -2;
  ScanArgs a{qk, ld_qk, off_q, off_k, v, ld_v, off_v, z, ld_z, off_z, zbias, hparam, beta, ld_b, off_b, aux, qscale,
             inv_tau, state, out, ld_out, q_start, q_len, kv_len, seq_slot, H, G, dk, dv};
  if (mode == LS_GLA) return launch_scan_mode<LS_GLA>(a, n_seqs, max_q, s);
  if (mode == LS_DELTA) return launch_scan_mode<LS_DELTA>(a, n_seqs, max_q, s);
  if (mode == LS_MLSTM) return launch_scan_mode<LS_MLSTM>(a, n_seqs, max_q, s);
  if (mode == LS_HGRN2) return launch_scan_mode<LS_HGRN2>(a, n_seqs, max_q, s);
  return -2;
}

int launch_scan_post(const float* o, int ld_o, const float* gate, int ld_g, int off_g, const float* weight, int wshared,
                     int act, const float* aux, void* out, int ld_out, int T, int H, int dv, float eps, int f32,
                     cudaStream_t s) {
  const long long warps = static_cast<long long>(T) * H;
  if (warps <= 0) return 0;
  const int blocks = static_cast<int>((warps + 3) / 4);
  if (f32)
    launch_kernel(scan_post_kernel<float>, dim3(blocks), dim3(128), 0, s, 1u, o, ld_o, gate, ld_g, off_g, weight, wshared,
                  act, aux, static_cast<float*>(out), ld_out, T, H, dv, eps);
  else
    launch_kernel(scan_post_kernel<bf16>, dim3(blocks), dim3(128), 0, s, 1u, o, ld_o, gate, ld_g, off_g, weight, wshared,
                  act, aux, static_cast<bf16*>(out), ld_out, T, H, dv, eps);
  return last_error();
}

}  // namespace b2b

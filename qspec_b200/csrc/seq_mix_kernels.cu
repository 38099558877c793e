// Sequence-mixer kernels, second file (include/qspec_b200_seq.h): token shift with a per-slot previous row, residual sum
// with a layer norm or unit-RMS norm of the sublayer's OUTPUT, latent (low-rank) key/value preparation with a rotary
// part, whole-projection query/key norms, sliding-window softmax attention with a per-head sink over a per-slot ring
// cache (shared by the latent and the grouped-query form), the HGRN2 gated linear recurrence with its state in
// float32, per-head output norm, and the gated per-token side input. Element type of activations and large weights:
// bfloat16 or float32; every norm, score, softmax weight, angle, gate of the recurrence and state is float32.
#include <cstdlib>
#include <cstring>
#include "seq_common.cuh"
#include "../../include/qspec_b200_seq.h"

namespace qspec {

// Pairs of elements per lane where rows allow it (even sizes and strides): 4-byte bfloat16 and 8-byte float32 loads.
template <int VEC> __device__ __forceinline__ void ld_pair(const float* p, float (&o)[2]) {
  if (VEC == 2) { const float2 t = *reinterpret_cast<const float2*>(p); o[0] = t.x; o[1] = t.y; }
  else { o[0] = *p; o[1] = 0.f; }
}
template <int VEC> __device__ __forceinline__ void ld_pair(const __nv_bfloat16* p, float (&o)[2]) {
  if (VEC == 2) { const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); o[0] = t.x; o[1] = t.y; }
  else { o[0] = __bfloat162float(*p); o[1] = 0.f; }
}

// ---- token shift --------------------------------------------------------------------------------------------------
// One CTA per token. The row before a segment's first token is the slot's saved row (buffer `phase`), zero at position
// 0; a segment's last row is saved to the other buffer, so that no CTA reads what another one of the same step writes.
template <typename T>
__global__ void __launch_bounds__(256)
token_shift_kernel(const float* __restrict__ x, const float* __restrict__ shift, float* __restrict__ prev, int slots,
                   T* __restrict__ out, const int* __restrict__ meta, int ntok, int W) {
  pdl_enter();
  const int i = blockIdx.x;
  const TokMeta m = load_meta(meta, ntok, i);
  const float* xr = x + (size_t)i * W;
  const float* pr = nullptr;
  if (i > m.seg_begin) pr = xr - W;
  else if (m.pos > 0) pr = prev + ((size_t)m.phase * slots + m.slot) * W;
  float* keep = (i == m.seg_end - 1) ? prev + ((size_t)(1 - m.phase) * slots + m.slot) * W : nullptr;
  T* orow = out + (size_t)i * W;
  for (int c = threadIdx.x; c < W; c += 256) {
    const float v = xr[c];
    const float p = pr ? pr[c] : 0.f;
    orow[c] = from_f<T>(v + (p - v) * shift[c]);
    if (keep) keep[c] = v;
  }
}

// ---- residual sum with a norm of the sublayer's output ------------------------------------------------------------
// v = sum of the parts of y (weighted); n = (v - mean) / sqrt(var + eps) * w + b (kind 0) or v / sqrt(mean(v^2) + eps) * w
// (kind 1); r = x_in + n. The row lives in shared memory between the passes; the variance is the mean of the squared
// deviations (second pass), not E[v^2] - mean^2.
template <typename T, typename YT>
__global__ void __launch_bounds__(256)
add_norm_kernel(const float* __restrict__ x_in, float* __restrict__ x_out, const YT* __restrict__ y, int y_parts,
                long long y_part_stride, long long y_tok_stride, const float* __restrict__ y_w, const float* __restrict__ w,
                const float* __restrict__ b, int kind, T* __restrict__ out, int W, float eps) {
  pdl_enter();
  extern __shared__ float sm_an[];            // row [W]
  __shared__ float red[8];
  const int i = blockIdx.x, tid = threadIdx.x;
  const YT* yr = y + (size_t)i * y_tok_stride;
  float s = 0.f;
  for (int c = tid; c < W; c += 256) {
    float v;
    if (y_parts == 1 && !y_w) {
      v = to_f(yr[c]);
    } else {
      v = 0.f;
      for (int p = 0; p < y_parts; ++p) v += (y_w ? y_w[(size_t)i * y_parts + p] : 1.0f) * to_f(yr[(size_t)p * y_part_stride + c]);
    }
    sm_an[c] = v;
    s += v;
  }
  const float inv_w = 1.0f / (float)W;
  float mean = 0.f;
  if (kind == 0) mean = block_sum_256(s, red) * inv_w;
  float q = 0.f;
  for (int c = tid; c < W; c += 256) {
    const float d = sm_an[c] - mean;
    q += d * d;
  }
  const float var = block_sum_256(q, red) * inv_w;
  const float r = 1.0f / sqrtf(var + eps);
  for (int c = tid; c < W; c += 256) {
    float v = (sm_an[c] - mean) * r * w[c];
    if (b) v += b[c];
    if (x_in) v += x_in[(size_t)i * W + c];
    if (x_out) x_out[(size_t)i * W + c] = v;
    if (out) out[(size_t)i * W + c] = from_f<T>(v);
  }
}

// ---- latent attention: norms of the low-rank projections, rotary key part, cache write ----------------------------
// Row of d: [q latent (q_rank) | kv latent (kv_rank) | shared rotary key part (rot_dim)]; the last two only when the
// layer owns a cache. One CTA per token. Cache row = position % cap: [normalised kv latent | rotated key part].
template <typename T>
__global__ void __launch_bounds__(256)
latent_prep_kernel(const T* __restrict__ d, int ld, int q_rank, int kv_rank, int rot_dim, const float* __restrict__ qn_w,
                   const float* __restrict__ kvn_w, const float* __restrict__ inv_freq, int rot_dims, int pairing, T* __restrict__ cq,
                   T* __restrict__ cache, int cap, const int* __restrict__ meta, int ntok, float eps) {
  pdl_enter();
  __shared__ float red[8];
  const int i = blockIdx.x, tid = threadIdx.x;
  const T* row = d + (size_t)i * ld;
  float ss = 0.f;
  if (q_rank > 0) {
    for (int c = tid; c < q_rank; c += 256) { const float v = to_f(row[c]); ss += v * v; }
    const float rq = 1.0f / sqrtf(block_sum_256(ss, red) / (float)q_rank + eps);
    for (int c = tid; c < q_rank; c += 256) cq[(size_t)i * q_rank + c] = from_f<T>(to_f(row[c]) * rq * qn_w[c]);
  }
  if (!cache) return;
  const int slot = meta[i], pos = meta[ntok + i];
  T* crow = cache + ((size_t)slot * cap + (pos % cap)) * (kv_rank + rot_dim);
  const T* kv = row + q_rank;
  ss = 0.f;
  for (int c = tid; c < kv_rank; c += 256) { const float v = to_f(kv[c]); ss += v * v; }
  const float rk = 1.0f / sqrtf(block_sum_256(ss, red) / (float)kv_rank + eps);
  for (int c = tid; c < kv_rank; c += 256) crow[c] = from_f<T>(to_f(kv[c]) * rk * kvn_w[c]);
  const T* kr = kv + kv_rank;
  const int half = rot_dims >> 1;
  for (int c = tid; c < half; c += 256) {
    float sn, cs;
    sincosf((float)pos * inv_freq[c], &sn, &cs);
    const int iu = pairing == QSPEC_ROTARY_INTERLEAVED ? 2 * c : c, iv = pairing == QSPEC_ROTARY_INTERLEAVED ? 2 * c + 1 : c + half;
    const float u = to_f(kr[iu]), v = to_f(kr[iv]);
    crow[kv_rank + iu] = from_f<T>(u * cs - v * sn);
    crow[kv_rank + iv] = from_f<T>(v * cs + u * sn);
  }
  for (int c = rot_dims + tid; c < rot_dim; c += 256) crow[kv_rank + c] = kr[c];
}

// Rotary positions on a slice of every head: dst[t, h, 0:n] = rotate(src[t, h, off : off + n]) in float32, the first
// rot_dims entries rotated (entry i paired with i + rot_dims / 2), the rest copied.
template <typename T>
__global__ void __launch_bounds__(128)
rotary_kernel(const T* __restrict__ src, long long src_ts, int src_hs, int off, float* __restrict__ dst, long long dst_ts, int dst_hs,
              int H, int n, int rot_dims, int pairing, const float* __restrict__ inv_freq, const int* __restrict__ meta, int ntok) {
  pdl_enter();
  const int i = blockIdx.x;
  const int pos = meta[ntok + i];
  const int half = rot_dims >> 1, rest = n - rot_dims, per = half + rest;
  for (int k = threadIdx.x; k < H * per; k += 128) {
    const int h = k / per, c = k % per;
    const T* s = src + (size_t)i * src_ts + (size_t)h * src_hs + off;
    float* o = dst + (size_t)i * dst_ts + (size_t)h * dst_hs;
    if (c < half) {
      float sn, cs;
      sincosf((float)pos * inv_freq[c], &sn, &cs);
      const int iu = pairing == QSPEC_ROTARY_INTERLEAVED ? 2 * c : c, iv = pairing == QSPEC_ROTARY_INTERLEAVED ? 2 * c + 1 : c + half;
      const float u = to_f(s[iu]), v = to_f(s[iv]);
      o[iu] = u * cs - v * sn;
      o[iv] = v * cs + u * sn;
    } else {
      o[rot_dims + c - half] = to_f(s[rot_dims + c - half]);
    }
  }
}

// ---- grouped-query attention: norm over the whole query / key projection, cache write -----------------------------
// Row of p: [q (HD) | k (GD) | v (GDV) | ...], biases already added by the projection. q -> float32 buffer, k and v ->
// ring cache rows (position % cap).
template <typename T>
__global__ void __launch_bounds__(256)
qkv_prep_kernel(const T* __restrict__ p, int ld, int HD, int GD, int GDV, const float* __restrict__ qn_w,
                const float* __restrict__ kn_w, float* __restrict__ qout, T* __restrict__ cache_k, T* __restrict__ cache_v, int cap,
                const int* __restrict__ meta, int ntok, float eps) {
  pdl_enter();
  __shared__ float red[8];
  const int i = blockIdx.x, tid = threadIdx.x;
  const T* row = p + (size_t)i * ld;
  const int slot = meta[i], pos = meta[ntok + i];
  float ss = 0.f;
  for (int c = tid; c < HD; c += 256) { const float v = to_f(row[c]); ss += v * v; }
  const float rq = 1.0f / sqrtf(block_sum_256(ss, red) / (float)HD + eps);
  for (int c = tid; c < HD; c += 256) qout[(size_t)i * HD + c] = to_f(row[c]) * rq * qn_w[c];
  const T* k = row + HD;
  ss = 0.f;
  for (int c = tid; c < GD; c += 256) { const float v = to_f(k[c]); ss += v * v; }
  const float rk = 1.0f / sqrtf(block_sum_256(ss, red) / (float)GD + eps);
  const size_t r = (size_t)slot * cap + (pos % cap);
  for (int c = tid; c < GD; c += 256) cache_k[r * GD + c] = from_f<T>(to_f(k[c]) * rk * kn_w[c]);
  const T* v = k + GD;
  for (int c = tid; c < GDV; c += 256) cache_v[r * GDV + c] = v[c];
}

// ---- sliding-window softmax attention with a sink -------------------------------------------------------------------
// One CTA of four warps per (token, query head). Query = two float32 parts (qa against key[0:DA], qb against
// key[DA:DA+DB]); keys and values are rows of a per-slot ring (row = position % cap) that already holds the step's
// own tokens. A warp takes every fourth run of four keys of the window: lanes along the rows for the dot products, an
// online softmax per warp, and the four partial results are merged in shared memory together with the sink term
// exp(sink[h]) of the denominator. Which warp takes which key depends on the token's position only, so a token's result
// does not depend on how its sequence was cut into steps or on its neighbours in the batch.
template <typename T, int NACC, int VEC>
__global__ void __launch_bounds__(128)
window_attn_kernel(const float* __restrict__ qa, long long qa_ts, long long qa_hs, int DA, const float* __restrict__ qb,
                   long long qb_ts, long long qb_hs, int DB, const T* __restrict__ kc, long long k_ss, int k_rs, int k_hs,
                   const T* __restrict__ vc, long long v_ss, int v_rs, int v_hs, int DV, const float* __restrict__ sink,
                   const T* __restrict__ gate, int gate_ld, int gate_per_head, T* __restrict__ out, const int* __restrict__ meta,
                   int ntok, int H, int G, int window, int cap, float scale) {
  pdl_enter();
  extern __shared__ float sm_wa[];            // q [DK] | acc [4][DV]
  __shared__ float s_m[4], s_l[4];
  const int i = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int DK = DA + DB;
  float* sq = sm_wa;
  float* sacc = sm_wa + ((DK + 3) & ~3);
  const int slot = meta[i], pos = meta[ntok + i];
  const int g = h / (H / G);
  for (int c = tid; c < DA; c += 128) sq[c] = qa[(size_t)i * qa_ts + (size_t)h * qa_hs + c];
  for (int c = tid; c < DB; c += 128) sq[DA + c] = qb[(size_t)i * qb_ts + (size_t)h * qb_hs + c];
  __syncthreads();
  const T* kbase = kc + (size_t)slot * k_ss + (size_t)g * k_hs;
  const T* vbase = vc + (size_t)slot * v_ss + (size_t)g * v_hs;
  const int j0 = max(0, pos - window + 1);
  float m = -INFINITY, l = 0.f;
  float acc[NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) acc[a] = 0.f;
  // a warp takes runs of KU consecutive keys (every fourth run): KU independent rows in flight per iteration
  constexpr int KU = 4;
  for (int j = j0 + warp * KU; j <= pos; j += 4 * KU) {
    const int n = min(KU, pos - j + 1);
    const T* kr[KU];
    const T* vr[KU];
#pragma unroll
    for (int u = 0; u < KU; ++u) {
      const int r = (j + (u < n ? u : 0)) % cap;
      kr[u] = kbase + (size_t)r * k_rs;
      vr[u] = vbase + (size_t)r * v_rs;
    }
    float dot[KU];
#pragma unroll
    for (int u = 0; u < KU; ++u) dot[u] = 0.f;
    for (int c = lane * VEC; c < DK; c += 32 * VEC) {
      const float q0 = sq[c], q1 = VEC == 2 ? sq[c + 1] : 0.f;
#pragma unroll
      for (int u = 0; u < KU; ++u) {
        float kv[2];
        ld_pair<VEC>(kr[u] + c, kv);
        dot[u] += q0 * kv[0];
        if (VEC == 2) dot[u] += q1 * kv[1];
      }
    }
    float mn = m;
#pragma unroll
    for (int u = 0; u < KU; ++u) {
      dot[u] = u < n ? warp_xor_sum(dot[u]) * scale : -INFINITY;
      mn = fmaxf(mn, dot[u]);
    }
    const float corr = expf(m - mn);
    float p[KU], ps = 0.f;
#pragma unroll
    for (int u = 0; u < KU; ++u) { p[u] = expf(dot[u] - mn); ps += p[u]; }
    m = mn;
    l = l * corr + ps;
#pragma unroll
    for (int a = 0; a < NACC; a += VEC) {
      const int c = lane * VEC + 32 * a;
      float s0 = 0.f, s1 = 0.f;
      if (c < DV) {
#pragma unroll
        for (int u = 0; u < KU; ++u) {
          float vv[2];
          ld_pair<VEC>(vr[u] + c, vv);
          s0 += p[u] * vv[0];
          s1 += p[u] * vv[1];
        }
      }
      acc[a] = acc[a] * corr + s0;
      if (VEC == 2) acc[a + 1] = acc[a + 1] * corr + s1;
    }
  }
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int a = 0; a < NACC; a += VEC) {
    const int c = lane * VEC + 32 * a;
    if (c < DV) {
      sacc[warp * DV + c] = acc[a];
      if (VEC == 2) sacc[warp * DV + c + 1] = acc[a + 1];
    }
  }
  __syncthreads();
  float M = sink ? sink[h] : -INFINITY;
#pragma unroll
  for (int w = 0; w < 4; ++w) M = fmaxf(M, s_m[w]);
  float f[4], L = sink ? expf(sink[h] - M) : 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    f[w] = expf(s_m[w] - M);               // a warp without keys has m = -inf: factor 0
    L += s_l[w] * f[w];
  }
  const float inv = 1.0f / L;
  for (int c = tid; c < DV; c += 128) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) o += sacc[w * DV + c] * f[w];
    o *= inv;
    if (gate) o *= 1.0f / (1.0f + expf(-to_f(gate[(size_t)i * gate_ld + (gate_per_head ? (size_t)h : (size_t)h * DV + c)])));
    out[((size_t)i * H + h) * DV + c] = from_f<T>(o);
  }
}

// ---- HGRN2 gates: q = silu(zq), f = lower + (1 - lower) sigmoid(zf + b), and 1 - f, float32, once per (token, row) -------
// gates [ntok][3][H * D]. 1 - f = (1 - lower) / (1 + e^z) is formed without the cancellation of 1 - f near f = 1.
template <typename T>
__global__ void __launch_bounds__(256)
hgrn2_gates_kernel(const T* __restrict__ p, int ld, const float* __restrict__ f_b, const float* __restrict__ lower,
                   float* __restrict__ gates, int HD, long long n) {
  pdl_enter();
  for (long long k = (long long)blockIdx.x * 256 + threadIdx.x; k < n; k += (long long)gridDim.x * 256) {
    const long long t = k / HD;
    const int c = (int)(k - t * HD);
    const T* row = p + (size_t)t * ld;
    const float zq = to_f(row[c]), z = to_f(row[HD + c]) + f_b[c], lo = lower[c];
    const float om = 1.0f / (1.0f + expf(z));             // 1 - sigmoid(z)
    float* g = gates + (size_t)t * 3 * HD + c;
    g[0] = zq / (1.0f + expf(-zq));
    g[HD] = lo + (1.0f - lo) * (1.0f - om);
    g[2 * HD] = (1.0f - lo) * om;
  }
}


// ---- scalar-decay linear attention: q = silu(zq), k = silu(zk), float32, once per (token, row); gates [ntok][2][H * D] ----
template <typename T>
__global__ void __launch_bounds__(256)
lightning_gates_kernel(const T* __restrict__ p, int ld, float* __restrict__ gates, int HD, long long n) {
  pdl_enter();
  for (long long k = (long long)blockIdx.x * 256 + threadIdx.x; k < n; k += (long long)gridDim.x * 256) {
    const long long t = k / HD;
    const int c = (int)(k - t * HD);
    const T* row = p + (size_t)t * ld;
    const float zq = to_f(row[c]), zk = to_f(row[HD + c]);
    float* g = gates + (size_t)t * 2 * HD + c;
    g[0] = zq / (1.0f + expf(-zq));
    g[HD] = zk / (1.0f + expf(-zk));
  }
}

// Unit-RMS norm over a whole row of float32 values with a weight and a sigmoid gate: out = src / rms(src) * w * sigmoid(gate).
// One CTA per row (all heads of a token are normed together).
template <typename T>
__global__ void __launch_bounds__(256)
gated_row_norm_kernel(const float* __restrict__ src, const float* __restrict__ w, const T* __restrict__ gate, int gate_ld,
                      T* __restrict__ out, int N, float eps) {
  pdl_enter();
  __shared__ float red[8];
  const int i = blockIdx.x, tid = threadIdx.x;
  const float* s = src + (size_t)i * N;
  float ss = 0.f;
  for (int c = tid; c < N; c += 256) ss += s[c] * s[c];
  const float rr = 1.0f / sqrtf(block_sum_256(ss, red) / (float)N + eps);
  for (int c = tid; c < N; c += 256) {
    const float z = to_f(gate[(size_t)i * gate_ld + c]);
    out[(size_t)i * N + c] = from_f<T>(s[c] * rr * w[c] * (1.0f / (1.0f + expf(-z))));
  }
}

// ---- residual sum with a multiplier, and the norm of the next sublayer's input ---------------------------------------
// r = x_in + mult * y_scale * (sum of weighted parts of y + weighted y2); out = r / sqrt(mean(r^2) + eps) * (w_offset + w). One CTA per
// token; the row lives in shared memory between the passes. VEC = 4: every thread takes four neighbouring columns with one
// load per operand (rows and strides on 16-byte boundaries); the parts' weights wait in shared memory.
template <typename T, typename YT, int VEC>
__global__ void __launch_bounds__(256)
residual_norm_kernel(const float* __restrict__ x_in, float* __restrict__ x_out, const YT* __restrict__ y, int y_parts,
                     long long y_part_stride, long long y_tok_stride, const float* __restrict__ y_w, const YT* __restrict__ y2,
                     const float* __restrict__ y2_w, int y2_w_stride, float mult, const float* __restrict__ w, float w_offset,
                     T* __restrict__ out, int W, float eps, const float* __restrict__ y_scale) {
  pdl_enter();
  extern __shared__ __align__(16) float sm_rn[];            // row [W]
  __shared__ float red[8];
  __shared__ float s_yw[64];
  const int i = blockIdx.x, tid = threadIdx.x;
  const YT* yr = y ? y + (size_t)i * y_tok_stride : nullptr;
  const YT* y2r = y2 ? y2 + (size_t)i * W : nullptr;
  const float w2 = (y2 && y2_w) ? y2_w[(size_t)i * y2_w_stride] : 1.0f;
  const bool weights_in_smem = y_parts <= 64;
  if (yr && weights_in_smem) {
    if (tid < y_parts) s_yw[tid] = y_w ? y_w[(size_t)i * y_parts + tid] : 1.0f;
    __syncthreads();
  }
  const float* xr = x_in + (size_t)i * W;
  float q = 0.f;
  for (int c = tid * VEC; c < W; c += 256 * VEC) {
    VecF<VEC> v;
#pragma unroll
    for (int e = 0; e < VEC; ++e) v.v[e] = 0.f;
    if (yr) {
#pragma unroll 4
      for (int p = 0; p < y_parts; ++p) {
        const float wp = weights_in_smem ? s_yw[p] : (y_w ? y_w[(size_t)i * y_parts + p] : 1.0f);
        const VecF<VEC> t = ldv<VEC>(yr + (size_t)p * y_part_stride + c);
#pragma unroll
        for (int e = 0; e < VEC; ++e) v.v[e] += wp * t.v[e];
      }
    }
    if (y2r) {
      const VecF<VEC> t = ldv<VEC>(y2r + c);
#pragma unroll
      for (int e = 0; e < VEC; ++e) v.v[e] += w2 * t.v[e];
    }
    if (y_scale) {                                          // one factor per column (a layer scale)
      const VecF<VEC> sc = ldv<VEC>(y_scale + c);
#pragma unroll
      for (int e = 0; e < VEC; ++e) v.v[e] *= sc.v[e];
    }
    VecF<VEC> r = ldv<VEC>(xr + c);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      r.v[e] += mult * v.v[e];
      q += r.v[e] * r.v[e];
    }
    if (x_out) stv<VEC>(x_out + (size_t)i * W + c, r);
    stv<VEC>(sm_rn + c, r);
  }
  if (!out) return;
  const float rr = 1.0f / sqrtf(block_sum_256(q, red) / (float)W + eps);
  for (int c = tid * VEC; c < W; c += 256 * VEC) {
    VecF<VEC> r = ldv<VEC>(sm_rn + c);
    const VecF<VEC> wv = ldv<VEC>(w + c);
#pragma unroll
    for (int e = 0; e < VEC; ++e) r.v[e] = r.v[e] * rr * (w_offset + wv.v[e]);
    stv<VEC>(out + (size_t)i * W + c, r);
  }
}

// ---- element-wise activations -------------------------------------------------------------------------------------------
__device__ __forceinline__ float act_apply(float z, int act) {
  if (act == QSPEC_ACT_GELU_ERF) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f));
  const float v = fmaxf(z, 0.f);
  return v * v;
}
template <typename T, int VEC>
__global__ void __launch_bounds__(256) act_kernel(T* __restrict__ a, long long n, int act) {
  pdl_enter();
  for (long long k = ((long long)blockIdx.x * 256 + threadIdx.x) * VEC; k < n; k += (long long)gridDim.x * 256 * VEC) {
    VecF<VEC> v = ldv<VEC>(a + k);
#pragma unroll
    for (int e = 0; e < VEC; ++e) v.v[e] = act_apply(v.v[e], act);
    stv<VEC>(a + k, v);
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ gu, int ld, T* __restrict__ out, int F, long long n) {
  pdl_enter();
  for (long long k = ((long long)blockIdx.x * 256 + threadIdx.x) * VEC; k < n; k += (long long)gridDim.x * 256 * VEC) {
    const long long t = k / F;
    const int f = (int)(k - t * F);
    const VecF<VEC> g = ldv<VEC>(gu + (size_t)t * ld + f), u = ldv<VEC>(gu + (size_t)t * ld + F + f);
    VecF<VEC> o;
#pragma unroll
    for (int e = 0; e < VEC; ++e) o.v[e] = g.v[e] / (1.0f + expf(-g.v[e])) * u.v[e];
    stv<VEC>(out + k, o);
  }
}

// ---- HGRN2: gated linear recurrence ---------------------------------------------------------------------------------
// Per head S <- diag(f) S + (1 - f) v^T, o = S^T q with f = lower + (1 - lower) sigmoid(zf + b) and q = silu(zq).
// One CTA per (segment, head, slice of 16 value columns) walks the segment's tokens in order, 16 (or 8) at a time; thread
// (row group w of 16, column c of 16) keeps rows w * NS .. of column c of the state in registers (float32). For a block of
// tokens the gates, queries (hgrn2_gates_kernel) and values are copied into shared memory (they were fetched into
// registers while the previous block was applied), then every thread applies the block's tokens to its rows, and the
// sixteen row groups' partial outputs are added per (token, column). The state is loaded from the slot at the start
// (zero at position 0) and stored at the end. o leaves un-normalised, float32.
template <typename T, int NS, int BT>
__global__ void __launch_bounds__(256)
hgrn2_scan_kernel(const T* __restrict__ p, int ld, const float* __restrict__ gates, float* __restrict__ state, float* __restrict__ o,
                  const int* __restrict__ meta, const int* __restrict__ seg_starts, int ntok, int H, int D, int DV,
                  const float* __restrict__ decay) {
  pdl_enter();
  // with a list of the segments' first rows the grid has one CTA per segment; without it, one per token, and the CTAs of
  // tokens that do not open a segment leave at once (a long prompt then pays for thousands of empty CTAs)
  const int i = seg_starts ? seg_starts[blockIdx.x] : blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * 16;
  const TokMeta mt = load_meta(meta, ntok, i);
  if (i != mt.seg_begin) return;
  constexpr int DP = 16 * NS, R = (BT * DP) / 256;           // BT tokens per block; padded rows; staged values per thread
  __shared__ __align__(16) float sq[BT][DP], sf[BT][DP], sg[BT][DP];
  __shared__ float sv[BT][16], spart[BT][16][16];
  const int tid = threadIdx.x, c = tid & 15, grp = tid >> 4;
  const int col = v0 + c;
  const bool live = col < DV;
  const int d0 = grp * NS;
  float S[NS];
  float* st = state + (((size_t)mt.slot * H + h) * D) * DV;
#pragma unroll
  for (int k = 0; k < NS; ++k) S[k] = (mt.pos > 0 && live && d0 + k < D) ? st[(size_t)(d0 + k) * DV + col] : 0.f;
  const int HD = H * D;
  const float dec = decay ? decay[h] : 1.f;
  float rq[R], rf[R], rg[R], zv = 0.f;
  auto fetch = [&](int tb) {                               // gates and values of the block's tokens into registers
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int e = tid + 256 * r, tt = e / DP, d = e % DP, t = tb + tt;
      rq[r] = 0.f; rf[r] = 1.f; rg[r] = 0.f;
      if (t < mt.seg_end && d < D) {
        if (decay) {                                          // one decay per head: gates hold [q | k] only
          const float* g = gates + (size_t)t * 2 * HD + h * D + d;
          rq[r] = g[0]; rf[r] = dec; rg[r] = g[HD];
        } else {
          const float* g = gates + (size_t)t * 3 * HD + h * D + d;
          rq[r] = g[0]; rf[r] = g[HD]; rg[r] = g[2 * HD];
        }
      }
    }
    if (tid < BT * 16) {
      const int t = tb + grp;
      zv = (t < mt.seg_end && live) ? to_f(p[(size_t)t * ld + 2 * HD + h * DV + col]) : 0.f;
      if (decay) zv = zv / (1.0f + expf(-zv));               // the scalar-decay form takes silu(v)
    }
  };
  fetch(mt.seg_begin);
  for (int tb = mt.seg_begin; tb < mt.seg_end; tb += BT) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int e = tid + 256 * r, tt = e / DP, d = e % DP;
      sq[tt][d] = rq[r]; sf[tt][d] = rf[r]; sg[tt][d] = rg[r];
    }
    if (tid < BT * 16) sv[grp][c] = zv;
    __syncthreads();
    if (tb + BT < mt.seg_end) fetch(tb + BT);
    const int nb = min(BT, mt.seg_end - tb);
    for (int tt = 0; tt < nb; ++tt) {
      const float v = sv[tt][c];
      float p0 = 0.f, p1 = 0.f;                             // two chains: the sum over rows is the long dependency
      const float4* f4 = reinterpret_cast<const float4*>(&sf[tt][d0]);
      const float4* g4 = reinterpret_cast<const float4*>(&sg[tt][d0]);
      const float4* q4 = reinterpret_cast<const float4*>(&sq[tt][d0]);
#pragma unroll
      for (int k = 0; k < NS / 4; ++k) {
        const float4 f = f4[k], gq = g4[k], q = q4[k];
        S[4 * k] = f.x * S[4 * k] + gq.x * v;             p0 += S[4 * k] * q.x;
        S[4 * k + 1] = f.y * S[4 * k + 1] + gq.y * v;     p1 += S[4 * k + 1] * q.y;
        S[4 * k + 2] = f.z * S[4 * k + 2] + gq.z * v;     p0 += S[4 * k + 2] * q.z;
        S[4 * k + 3] = f.w * S[4 * k + 3] + gq.w * v;     p1 += S[4 * k + 3] * q.w;
      }
      spart[tt][grp][c] = p0 + p1;
    }
    __syncthreads();
    if (tid < BT * 16 && grp < nb && live) {                // thread (token grp, column c) adds the sixteen row groups
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 16; ++w) s += spart[grp][w][c];
      o[(size_t)(tb + grp) * H * DV + (size_t)h * DV + col] = s;
    }
  }
  if (live) {
#pragma unroll
    for (int k = 0; k < NS; ++k)
      if (d0 + k < D) st[(size_t)(d0 + k) * DV + col] = S[k];
  }
}

// Per-head unit-RMS norm with one weight vector shared by the heads: one warp per (token, head); src float32.
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_kernel(const float* __restrict__ src, const float* __restrict__ w, T* __restrict__ out, long long rows, int DV, float eps) {
  pdl_enter();
  const long long r = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const float* s = src + r * DV;
  float ss = 0.f;
  for (int c = lane; c < DV; c += 32) ss += s[c] * s[c];
  const float rr = 1.0f / sqrtf(warp_xor_sum(ss) / (float)DV + eps);
  for (int c = lane; c < DV; c += 32) out[r * DV + c] = from_f<T>(s[c] * rr * w[c]);
}

// ---- per-token side input: g <- gelu_tanh(g) * table[id, layer part] -------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
side_gate_kernel(T* __restrict__ g, const T* __restrict__ table, const int* __restrict__ ids, int col0, int sd, int table_ld, int V,
                 long long n) {
  pdl_enter();
  for (long long k = (long long)blockIdx.x * 256 + threadIdx.x; k < n; k += (long long)gridDim.x * 256) {
    const long long t = k / sd;
    const int c = (int)(k % sd);
    int id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const float z = to_f(g[k]);
    const float ge = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    g[k] = from_f<T>(ge * to_f(table[(size_t)id * table_ld + col0 + c]));
  }
}

}  // namespace qspec

using namespace qspec;

#define MIX_DTYPE_OK(dtype) QSPEC_REQUIRE((dtype) == QSPEC_DTYPE_BF16 || (dtype) == QSPEC_DTYPE_F32, QSPEC_ERR_UNSUPPORTED, \
                                          "dtype %d: bfloat16 (1) or float32 (2) expected", (dtype))
typedef __nv_bfloat16 bf16_t;

extern "C" int qspec_seq_token_shift(const float* x, const float* shift, float* prev, int slots, void* out, const int* meta,
                                     int ntok, int W, int dtype, void* stream) {
  QSPEC_REQUIRE(x && shift && prev && out && meta, QSPEC_ERR_INVALID_ARG, "seq_token_shift: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && W > 0 && slots > 0, QSPEC_ERR_INVALID_ARG, "seq_token_shift: bad sizes");
  MIX_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(token_shift_kernel<float>, dim3(ntok), dim3(256), 0, (cudaStream_t)stream, x, shift, prev, slots, (float*)out, meta, ntok, W);
  else
    launch_pdl(token_shift_kernel<bf16_t>, dim3(ntok), dim3(256), 0, (cudaStream_t)stream, x, shift, prev, slots, (bf16_t*)out, meta, ntok, W);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T, typename YT>
static int launch_add_norm(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride, long long y_tok_stride,
                           const float* y_w, const float* w, const float* b, int kind, void* out, int ntok, int W, float eps,
                           cudaStream_t st) {
  const size_t smem = (size_t)W * sizeof(float);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(add_norm_kernel<T, YT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  launch_pdl(add_norm_kernel<T, YT>, dim3(ntok), dim3(256), smem, st, x_in, x_out, (const YT*)y, y_parts, y_part_stride, y_tok_stride,
             y_w, w, b, kind, (T*)out, W, eps);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_seq_add_norm(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride,
                                  long long y_tok_stride, const float* y_w, const float* w, const float* b, int kind, void* out,
                                  int ntok, int W, float eps, int y_dtype, int dtype, void* stream) {
  QSPEC_REQUIRE(y && w && (x_out || out), QSPEC_ERR_INVALID_ARG, "seq_add_norm: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && W > 0 && W <= 49152 && y_parts >= 1 && (kind == 0 || kind == 1), QSPEC_ERR_INVALID_ARG,
                "seq_add_norm: bad sizes (width <= 49152, kind 0 or 1)");
  MIX_DTYPE_OK(dtype);
  QSPEC_REQUIRE(y_dtype == dtype || y_dtype == QSPEC_DTYPE_F32, QSPEC_ERR_UNSUPPORTED, "seq_add_norm: y is of the activation type or float32");
  if (ntok == 0) return QSPEC_OK;
  cudaStream_t st = (cudaStream_t)stream;
#define AN_ARGS x_in, x_out, y, y_parts, y_part_stride, y_tok_stride, y_w, w, b, kind, out, ntok, W, eps, st
  if (dtype == QSPEC_DTYPE_F32) return launch_add_norm<float, float>(AN_ARGS);
  if (y_dtype == QSPEC_DTYPE_F32) return launch_add_norm<bf16_t, float>(AN_ARGS);
  return launch_add_norm<bf16_t, bf16_t>(AN_ARGS);
#undef AN_ARGS
}

extern "C" int qspec_seq_latent_prep(const void* d, int ld, int q_rank, int kv_rank, int rot_dim, const float* qn_w, const float* kvn_w,
                                     const float* inv_freq, int rot_dims, void* cq, void* cache, int cap, const int* meta, int ntok,
                                     float eps, int dtype, void* stream) {
  QSPEC_REQUIRE(q_rank > 0, QSPEC_ERR_INVALID_ARG, "seq_latent_prep: bad sizes");
  return qspec_seq_latent_prep_pairing(d, ld, q_rank, kv_rank, rot_dim, qn_w, kvn_w, inv_freq, rot_dims, QSPEC_ROTARY_HALVES, cq, cache, cap,
                                       meta, ntok, eps, dtype, stream);
}

extern "C" int qspec_seq_latent_prep_pairing(const void* d, int ld, int q_rank, int kv_rank, int rot_dim, const float* qn_w,
                                             const float* kvn_w, const float* inv_freq, int rot_dims, int pairing, void* cq, void* cache,
                                             int cap, const int* meta, int ntok, float eps, int dtype, void* stream) {
  QSPEC_REQUIRE(d && meta && (q_rank == 0 || (qn_w && cq)), QSPEC_ERR_INVALID_ARG, "seq_latent_prep: null pointer");
  QSPEC_REQUIRE(pairing == QSPEC_ROTARY_HALVES || pairing == QSPEC_ROTARY_INTERLEAVED, QSPEC_ERR_INVALID_ARG, "seq_latent_prep: unknown pairing %d", pairing);
  QSPEC_REQUIRE(!cache || (kvn_w && (inv_freq || rot_dims == 0)), QSPEC_ERR_INVALID_ARG,
                "seq_latent_prep: a cache needs the key/value norm weight and the frequencies");
  QSPEC_REQUIRE(ntok >= 0 && q_rank >= 0 && kv_rank >= 0 && rot_dim >= 0 && rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0 &&
                    cap > 0 && ld >= q_rank + (cache ? kv_rank + rot_dim : 0),
                QSPEC_ERR_INVALID_ARG, "seq_latent_prep: bad sizes");
  MIX_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(latent_prep_kernel<float>, dim3(ntok), dim3(256), 0, (cudaStream_t)stream, (const float*)d, ld, q_rank, kv_rank, rot_dim,
               qn_w, kvn_w, inv_freq, rot_dims, pairing, (float*)cq, (float*)cache, cap, meta, ntok, eps);
  else
    launch_pdl(latent_prep_kernel<bf16_t>, dim3(ntok), dim3(256), 0, (cudaStream_t)stream, (const bf16_t*)d, ld, q_rank, kv_rank, rot_dim,
               qn_w, kvn_w, inv_freq, rot_dims, pairing, (bf16_t*)cq, (bf16_t*)cache, cap, meta, ntok, eps);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_seq_rotary(const void* src, long long src_ts, int src_hs, int off, float* dst, long long dst_ts, int dst_hs, int H,
                                int n, int rot_dims, const float* inv_freq, const int* meta, int ntok, int dtype, void* stream) {
  return qspec_seq_rotary_pairing(src, src_ts, src_hs, off, dst, dst_ts, dst_hs, H, n, rot_dims, QSPEC_ROTARY_HALVES, inv_freq, meta, ntok,
                                  dtype, stream);
}

extern "C" int qspec_seq_rotary_pairing(const void* src, long long src_ts, int src_hs, int off, float* dst, long long dst_ts, int dst_hs,
                                        int H, int n, int rot_dims, int pairing, const float* inv_freq, const int* meta, int ntok,
                                        int dtype, void* stream) {
  QSPEC_REQUIRE(pairing == QSPEC_ROTARY_HALVES || pairing == QSPEC_ROTARY_INTERLEAVED, QSPEC_ERR_INVALID_ARG, "seq_rotary: unknown pairing %d", pairing);
  QSPEC_REQUIRE(src && dst && meta && (rot_dims == 0 || inv_freq), QSPEC_ERR_INVALID_ARG, "seq_rotary: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && H > 0 && n >= 0 && rot_dims >= 0 && rot_dims <= n && rot_dims % 2 == 0, QSPEC_ERR_INVALID_ARG,
                "seq_rotary: bad sizes");
  MIX_DTYPE_OK(dtype);
  if (ntok == 0 || n == 0) return QSPEC_OK;
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(rotary_kernel<float>, dim3(ntok), dim3(128), 0, (cudaStream_t)stream, (const float*)src, src_ts, src_hs, off, dst, dst_ts,
               dst_hs, H, n, rot_dims, pairing, inv_freq, meta, ntok);
  else
    launch_pdl(rotary_kernel<bf16_t>, dim3(ntok), dim3(128), 0, (cudaStream_t)stream, (const bf16_t*)src, src_ts, src_hs, off, dst, dst_ts,
               dst_hs, H, n, rot_dims, pairing, inv_freq, meta, ntok);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_seq_qkv_prep(const void* p, int ld, int HD, int GD, int GDV, const float* qn_w, const float* kn_w, float* qout,
                                  void* cache_k, void* cache_v, int cap, const int* meta, int ntok, float eps, int dtype, void* stream) {
  QSPEC_REQUIRE(p && qn_w && kn_w && qout && cache_k && cache_v && meta, QSPEC_ERR_INVALID_ARG, "seq_qkv_prep: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && HD > 0 && GD > 0 && GDV > 0 && cap > 0 && ld >= HD + GD + GDV, QSPEC_ERR_INVALID_ARG, "seq_qkv_prep: bad sizes");
  MIX_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(qkv_prep_kernel<float>, dim3(ntok), dim3(256), 0, (cudaStream_t)stream, (const float*)p, ld, HD, GD, GDV, qn_w, kn_w, qout,
               (float*)cache_k, (float*)cache_v, cap, meta, ntok, eps);
  else
    launch_pdl(qkv_prep_kernel<bf16_t>, dim3(ntok), dim3(256), 0, (cudaStream_t)stream, (const bf16_t*)p, ld, HD, GD, GDV, qn_w, kn_w, qout,
               (bf16_t*)cache_k, (bf16_t*)cache_v, cap, meta, ntok, eps);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T, int NACC, int VEC>
static int launch_window_attn(const qspec_window_attn_args* a, cudaStream_t st) {
  const int DK = a->DA + a->DB;
  const size_t smem = ((size_t)((DK + 3) & ~3) + (size_t)4 * a->DV) * sizeof(float);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(window_attn_kernel<T, NACC, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  launch_pdl(window_attn_kernel<T, NACC, VEC>, dim3(a->ntok, a->H), dim3(128), smem, st, a->qa, a->qa_tok_stride, a->qa_head_stride, a->DA,
             a->qb, a->qb_tok_stride, a->qb_head_stride, a->DB, (const T*)a->k, a->k_slot_stride, a->k_row_stride, a->k_head_stride,
             (const T*)a->v, a->v_slot_stride, a->v_row_stride, a->v_head_stride, a->DV, a->sink, (const T*)a->gate, a->gate_ld, a->gate_per_head, (T*)a->out,
             a->meta, a->ntok, a->H, a->G, a->window, a->cap, a->scale);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T, int VEC>
static int launch_window_attn_n(const qspec_window_attn_args* a, cudaStream_t st) {
  const int per = (a->DV + 31) / 32;
  if (per <= 2) return launch_window_attn<T, 2, VEC>(a, st);
  if (per <= 4) return launch_window_attn<T, 4, VEC>(a, st);
  if (per <= 8) return launch_window_attn<T, 8, VEC>(a, st);
  if (per <= 16) return launch_window_attn<T, 16, VEC>(a, st);
  return launch_window_attn<T, 32, VEC>(a, st);
}

extern "C" int qspec_seq_window_attention(const qspec_window_attn_args* a, int dtype, void* stream) {
  QSPEC_REQUIRE(a && a->qa && a->k && a->v && a->out && a->meta && (a->DB == 0 || a->qb), QSPEC_ERR_INVALID_ARG,
                "seq_window_attention: null pointer");
  QSPEC_REQUIRE(a->ntok >= 0 && a->H > 0 && a->G > 0 && a->H % a->G == 0 && a->DA > 0 && a->DB >= 0 && a->DV > 0 && a->DV <= 1024 &&
                    a->DA + a->DB <= 8192 && a->window >= 1 && a->cap >= 1 && a->H <= 65535,
                QSPEC_ERR_UNSUPPORTED, "seq_window_attention: heads %d / %d, key size %d + %d (<= 8192), value size %d (<= 1024)", a->H,
                a->G, a->DA, a->DB, a->DV);
  MIX_DTYPE_OK(dtype);
  if (a->ntok == 0) return QSPEC_OK;
  const size_t esz = dtype == QSPEC_DTYPE_F32 ? 4 : 2;
  const bool even = ((a->DA + a->DB) % 2 == 0) && (a->DV % 2 == 0) && (a->k_row_stride % 2 == 0) && (a->k_head_stride % 2 == 0) &&
                    (a->k_slot_stride % 2 == 0) && (a->v_row_stride % 2 == 0) && (a->v_head_stride % 2 == 0) && (a->v_slot_stride % 2 == 0) &&
                    ((uintptr_t)a->k % (2 * esz) == 0) && ((uintptr_t)a->v % (2 * esz) == 0);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == QSPEC_DTYPE_F32) return even ? launch_window_attn_n<float, 2>(a, st) : launch_window_attn_n<float, 1>(a, st);
  return even ? launch_window_attn_n<bf16_t, 2>(a, st) : launch_window_attn_n<bf16_t, 1>(a, st);
}

template <typename T>
static int launch_hgrn2(const void* p, int ld, const float* f_b, const float* lower, float* state, float* o, float* gates, const int* meta,
                        const int* seg_starts, int nseg, int ntok, int H, int D, int DV, cudaStream_t st, const float* decay = nullptr) {
  const long long n = (long long)ntok * H * D;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (decay) launch_pdl(lightning_gates_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, st, (const T*)p, ld, gates, H * D, n);
  else launch_pdl(hgrn2_gates_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, st, (const T*)p, ld, f_b, lower, gates, H * D, n);
  QSPEC_CHECK_LAUNCH(1);
  const dim3 grid(seg_starts ? nseg : ntok, H, (DV + 15) / 16);
#define HG_ARGS dim3(256), 0, st, (const T*)p, ld, (const float*)gates, state, o, meta, seg_starts, ntok, H, D, DV, decay
  // blocks of 16 tokens for prompt portions (fewer barriers and copies per token); 8 for decoding steps, where the state's
  // way in and out of the registers is the work and the smaller shared-memory footprint keeps more CTAs on an SM
  const bool longs = seg_starts && ntok >= 16 * nseg;
  if (D <= 64) { if (longs) launch_pdl(hgrn2_scan_kernel<T, 4, 16>, grid, HG_ARGS); else launch_pdl(hgrn2_scan_kernel<T, 4, 8>, grid, HG_ARGS); }
  else if (D <= 128) { if (longs) launch_pdl(hgrn2_scan_kernel<T, 8, 16>, grid, HG_ARGS); else launch_pdl(hgrn2_scan_kernel<T, 8, 8>, grid, HG_ARGS); }
  else launch_pdl(hgrn2_scan_kernel<T, 16, 8>, grid, HG_ARGS);
#undef HG_ARGS
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_seq_hgrn2(const void* p, int ld, const float* f_b, const float* lower, const float* norm_w, float* state,
                               float* scratch, void* out, const int* meta, const int* seg_starts, int nseg, int ntok, int H, int D,
                               int DV, float eps, int dtype, void* stream) {
  QSPEC_REQUIRE(!seg_starts || (nseg >= 1 && nseg <= ntok) || ntok == 0, QSPEC_ERR_INVALID_ARG, "seq_hgrn2: %d segments for %d tokens", nseg, ntok);
  QSPEC_REQUIRE(p && f_b && lower && norm_w && state && scratch && out && meta, QSPEC_ERR_INVALID_ARG, "seq_hgrn2: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && H > 0 && H <= 65535 && D > 0 && D <= 256 && DV > 0 && DV <= 65535 * 16 && ld >= 2 * H * D + H * DV,
                QSPEC_ERR_UNSUPPORTED, "seq_hgrn2: %d heads, key size %d (<= 256), value size %d", H, D, DV);
  MIX_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  float* gates = scratch + (size_t)ntok * H * DV;          // scratch: un-normalised outputs, then the gates
  int s = dtype == QSPEC_DTYPE_F32 ? launch_hgrn2<float>(p, ld, f_b, lower, state, scratch, gates, meta, seg_starts, nseg, ntok, H, D, DV, st)
                                   : launch_hgrn2<bf16_t>(p, ld, f_b, lower, state, scratch, gates, meta, seg_starts, nseg, ntok, H, D, DV, st);
  if (s) return s;
  const long long rows = (long long)ntok * H;
  const unsigned blocks = (unsigned)((rows + 3) / 4);
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(head_norm_kernel<float>, dim3(blocks), dim3(128), 0, st, (const float*)scratch, norm_w, (float*)out, rows, DV, eps);
  else
    launch_pdl(head_norm_kernel<bf16_t>, dim3(blocks), dim3(128), 0, st, (const float*)scratch, norm_w, (bf16_t*)out, rows, DV, eps);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_seq_side_gate(void* g, const void* table, const int* ids, int col0, int sd, int table_ld, int V, int ntok, int dtype,
                                   void* stream) {
  QSPEC_REQUIRE(g && table && ids, QSPEC_ERR_INVALID_ARG, "seq_side_gate: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && sd > 0 && col0 >= 0 && col0 + sd <= table_ld && V > 0, QSPEC_ERR_INVALID_ARG, "seq_side_gate: bad sizes");
  MIX_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  const long long n = (long long)ntok * sd;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(side_gate_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (float*)g, (const float*)table, ids, col0,
               sd, table_ld, V, n);
  else
    launch_pdl(side_gate_kernel<bf16_t>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (bf16_t*)g, (const bf16_t*)table, ids,
               col0, sd, table_ld, V, n);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T, typename YT, int VEC>
static int launch_residual_norm_v(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride, long long y_tok_stride,
                                  const float* y_w, const void* y2, const float* y2_w, int y2_w_stride, float mult, const float* w,
                                  float w_offset, void* out, int ntok, int W, float eps, const float* y_scale, cudaStream_t st) {
  const size_t smem = (size_t)W * sizeof(float);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(residual_norm_kernel<T, YT, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  launch_pdl(residual_norm_kernel<T, YT, VEC>, dim3(ntok), dim3(256), smem, st, x_in, x_out, (const YT*)y, y_parts, y_part_stride,
             y_tok_stride, y_w, (const YT*)y2, y2_w, y2_w_stride, mult, w, w_offset, (T*)out, W, eps, y_scale);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T, typename YT>
static int launch_residual_norm(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride, long long y_tok_stride,
                                const float* y_w, const void* y2, const float* y2_w, int y2_w_stride, float mult, const float* w,
                                float w_offset, void* out, int ntok, int W, float eps, const float* y_scale, cudaStream_t st) {
  // four columns per thread where every row starts on a 16-byte boundary (float32 rows; bfloat16 rows need 8 bytes)
  // QSPEC_SEQ_RESNORM=scalar keeps one column per thread and step, for comparison
  static const bool scalar = [] { const char* v = getenv("QSPEC_SEQ_RESNORM"); return v && !strcmp(v, "scalar"); }();
  const bool vec = !scalar && W % 4 == 0 && y_part_stride % 4 == 0 && y_tok_stride % 4 == 0 &&
                   (((uintptr_t)x_in | (uintptr_t)x_out | (uintptr_t)w | (uintptr_t)y_scale) & 15) == 0 &&
                   (((uintptr_t)y | (uintptr_t)y2) & (4 * sizeof(YT) - 1)) == 0 && ((uintptr_t)out & (4 * sizeof(T) - 1)) == 0;
  if (vec)
    return launch_residual_norm_v<T, YT, 4>(x_in, x_out, y, y_parts, y_part_stride, y_tok_stride, y_w, y2, y2_w, y2_w_stride, mult, w, w_offset,
                                            out, ntok, W, eps, y_scale, st);
  return launch_residual_norm_v<T, YT, 1>(x_in, x_out, y, y_parts, y_part_stride, y_tok_stride, y_w, y2, y2_w, y2_w_stride, mult, w, w_offset,
                                          out, ntok, W, eps, y_scale, st);
}

extern "C" int qspec_seq_residual_norm_scaled(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride,
                                              long long y_tok_stride, const float* y_w, const void* y2, const float* y2_w, int y2_w_stride,
                                              float mult, const float* y_scale, const float* w, float w_offset, void* out, int ntok, int W,
                                              float eps, int y_dtype, int dtype, void* stream) {
  QSPEC_REQUIRE(x_in && (x_out || out) && (!out || w), QSPEC_ERR_INVALID_ARG, "seq_residual_norm: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && W > 0 && W <= 49152 && y_parts >= 1 && y2_w_stride >= 0, QSPEC_ERR_INVALID_ARG,
                "seq_residual_norm: bad sizes (width <= 49152)");
  MIX_DTYPE_OK(dtype);
  QSPEC_REQUIRE(y_dtype == dtype || y_dtype == QSPEC_DTYPE_F32, QSPEC_ERR_UNSUPPORTED, "seq_residual_norm: y is of the activation type or float32");
  if (ntok == 0) return QSPEC_OK;
  cudaStream_t st = (cudaStream_t)stream;
#define RN_ARGS x_in, x_out, y, y_parts, y_part_stride, y_tok_stride, y_w, y2, y2_w, y2_w_stride, mult, w, w_offset, out, ntok, W, eps, y_scale, st
  if (dtype == QSPEC_DTYPE_F32) return launch_residual_norm<float, float>(RN_ARGS);
  if (y_dtype == QSPEC_DTYPE_F32) return launch_residual_norm<bf16_t, float>(RN_ARGS);
  return launch_residual_norm<bf16_t, bf16_t>(RN_ARGS);
#undef RN_ARGS
}

extern "C" int qspec_seq_residual_norm(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride,
                                       long long y_tok_stride, const float* y_w, const void* y2, const float* y2_w, int y2_w_stride,
                                       float mult, const float* w, float w_offset, void* out, int ntok, int W, float eps, int y_dtype,
                                       int dtype, void* stream) {
  return qspec_seq_residual_norm_scaled(x_in, x_out, y, y_parts, y_part_stride, y_tok_stride, y_w, y2, y2_w, y2_w_stride, mult, nullptr, w,
                                        w_offset, out, ntok, W, eps, y_dtype, dtype, stream);
}

extern "C" int qspec_seq_act(void* a, long long n, int act, int dtype, void* stream) {
  QSPEC_REQUIRE(a && n >= 0, QSPEC_ERR_INVALID_ARG, "seq_act: bad arguments");
  QSPEC_REQUIRE(act == QSPEC_ACT_RELU2 || act == QSPEC_ACT_GELU_ERF, QSPEC_ERR_INVALID_ARG, "seq_act: unknown activation %d", act);
  MIX_DTYPE_OK(dtype);
  if (n == 0) return QSPEC_OK;
  const size_t esz = dtype == QSPEC_DTYPE_F32 ? 4 : 2;
  const bool vec = n % 4 == 0 && ((uintptr_t)a & (4 * esz - 1)) == 0;
  long long blocks = (n / (vec ? 4 : 1) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == QSPEC_DTYPE_F32) {
    if (vec) launch_pdl(act_kernel<float, 4>, dim3((unsigned)blocks), dim3(256), 0, st, (float*)a, n, act);
    else launch_pdl(act_kernel<float, 1>, dim3((unsigned)blocks), dim3(256), 0, st, (float*)a, n, act);
  } else {
    if (vec) launch_pdl(act_kernel<bf16_t, 4>, dim3((unsigned)blocks), dim3(256), 0, st, (bf16_t*)a, n, act);
    else launch_pdl(act_kernel<bf16_t, 1>, dim3((unsigned)blocks), dim3(256), 0, st, (bf16_t*)a, n, act);
  }
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_seq_silu_mul(const void* gu, int ld, void* out, int ntok, int F, int dtype, void* stream) {
  QSPEC_REQUIRE(gu && out && ntok >= 0 && F > 0 && ld >= 2 * F, QSPEC_ERR_INVALID_ARG, "seq_silu_mul: bad arguments");
  MIX_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  const long long n = (long long)ntok * F;
  const size_t esz = dtype == QSPEC_DTYPE_F32 ? 4 : 2;
  const bool vec = F % 4 == 0 && ld % 4 == 0 && (((uintptr_t)gu | (uintptr_t)out) & (4 * esz - 1)) == 0;
  long long blocks = (n / (vec ? 4 : 1) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == QSPEC_DTYPE_F32) {
    if (vec) launch_pdl(silu_mul_kernel<float, 4>, dim3((unsigned)blocks), dim3(256), 0, st, (const float*)gu, ld, (float*)out, F, n);
    else launch_pdl(silu_mul_kernel<float, 1>, dim3((unsigned)blocks), dim3(256), 0, st, (const float*)gu, ld, (float*)out, F, n);
  } else {
    if (vec) launch_pdl(silu_mul_kernel<bf16_t, 4>, dim3((unsigned)blocks), dim3(256), 0, st, (const bf16_t*)gu, ld, (bf16_t*)out, F, n);
    else launch_pdl(silu_mul_kernel<bf16_t, 1>, dim3((unsigned)blocks), dim3(256), 0, st, (const bf16_t*)gu, ld, (bf16_t*)out, F, n);
  }
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_seq_lightning(const void* p, int ld, const float* decay, const float* norm_w, float* state, float* scratch, void* out,
                                   const int* meta, const int* seg_starts, int nseg, int ntok, int H, int D, int DV, float eps, int dtype,
                                   void* stream) {
  QSPEC_REQUIRE(!seg_starts || (nseg >= 1 && nseg <= ntok) || ntok == 0, QSPEC_ERR_INVALID_ARG, "seq_lightning: %d segments for %d tokens", nseg, ntok);
  QSPEC_REQUIRE(p && decay && norm_w && state && scratch && out && meta, QSPEC_ERR_INVALID_ARG, "seq_lightning: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && H > 0 && H <= 65535 && D > 0 && D <= 256 && DV > 0 && DV <= 65535 * 16 && ld >= 2 * H * D + 2 * H * DV,
                QSPEC_ERR_UNSUPPORTED, "seq_lightning: %d heads, key size %d (<= 256), value size %d", H, D, DV);
  MIX_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  float* gates = scratch + (size_t)ntok * H * DV;          // scratch: un-normalised outputs, then silu(q) and silu(k)
  int s = dtype == QSPEC_DTYPE_F32
              ? launch_hgrn2<float>(p, ld, nullptr, nullptr, state, scratch, gates, meta, seg_starts, nseg, ntok, H, D, DV, st, decay)
              : launch_hgrn2<bf16_t>(p, ld, nullptr, nullptr, state, scratch, gates, meta, seg_starts, nseg, ntok, H, D, DV, st, decay);
  if (s) return s;
  const int N = H * DV, goff = 2 * H * D + H * DV;         // the output gate's logits follow q, k and v in the row
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(gated_row_norm_kernel<float>, dim3(ntok), dim3(256), 0, st, (const float*)scratch, norm_w, (const float*)p + goff, ld,
               (float*)out, N, eps);
  else
    launch_pdl(gated_row_norm_kernel<bf16_t>, dim3(ntok), dim3(256), 0, st, (const float*)scratch, norm_w, (const bf16_t*)p + goff, ld,
               (bf16_t*)out, N, eps);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

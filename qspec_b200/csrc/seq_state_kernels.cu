// Sequence-mixer kernels, fourth file: mixers whose per-sequence state is a matrix that every token rewrites (gated delta
// rule, selective scan), short causal convolutions with an activation, grouped-query attention whose heads' weights are mixed
// after the softmax, and the clamped gated feed-forward activation. bfloat16 / float32 activations (template T); everything that
// is normed, exponentiated or carried from token to token is float32.
#include "seq_common.cuh"
#include "../../include/qspec_b200_seq.h"
#include <stdint.h>

namespace qspec {

// 4-byte asynchronous copies into shared memory (both addresses on 4-byte boundaries)
__device__ __forceinline__ void cp_async_4(float* smem_dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---- short causal convolution over time, per channel, with an activation ---------------------------------------------------
// out[t, c] = act(bias[c] + sum_j w[c, j] * in[t - taps + 1 + j, c]). Rows before the segment's first token come from the
// slot's tail (the last taps - 1 inputs of the sequence so far), rows before position 0 are zero. One thread per (token,
// channel). The CTA row of a segment's last token also writes the new tail into the other buffer, so that reading and writing
// never meet.
template <typename T, typename OT>
__global__ void __launch_bounds__(256)
conv_act_kernel(const T* __restrict__ in, int ld, const float* __restrict__ w, const float* __restrict__ bias, int taps,
                float* __restrict__ tail, int slots, OT* __restrict__ out, int out_ld, const int* __restrict__ meta, int ntok, int C,
                int act) {
  pdl_enter();
  const int i = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
  if (c >= C) return;
  const TokMeta mt = load_meta(meta, ntok, i);
  const int K1 = taps - 1;
  const int first_pos = mt.pos - (i - mt.seg_begin);              // position of the segment's first token
  const float* told = tail + ((size_t)mt.phase * slots + mt.slot) * K1 * C;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int sp = mt.pos - K1 + j;                                // source position
    float v = 0.f;
    if (sp >= first_pos) v = to_f(in[(size_t)(mt.seg_begin + sp - first_pos) * ld + c]);
    else if (sp >= 0) v = told[(size_t)(sp - (first_pos - K1)) * C + c];
    acc += w[(size_t)c * taps + j] * v;
  }
  if (act == QSPEC_CONV_ACT_SILU) acc = silu_f(acc);
  out[(size_t)i * out_ld + c] = from_f<OT>(acc);
  if (i == mt.seg_end - 1) {
    float* tnew = tail + ((size_t)(1 - mt.phase) * slots + mt.slot) * K1 * C;
    for (int r = 0; r < K1; ++r) {
      const int sp = mt.pos + 1 - K1 + r;
      float v = 0.f;
      if (sp >= first_pos) v = to_f(in[(size_t)(mt.seg_begin + sp - first_pos) * ld + c]);
      else if (sp >= 0) v = told[(size_t)(sp - (first_pos - K1)) * C + c];
      tnew[(size_t)r * C + c] = v;
    }
  }
}

// ---- gated delta rule: unit vectors, step sizes and decays -------------------------------------------------------------------
// Row t of cs (float32, in place): [q (G x D) | k (G x D) | ...]. q <- q / sqrt(sum q^2 + unit_eps) * q_mult, k likewise without
// the multiplier. gates[t] = [beta (H) | decay (H) | q.k (G)] with beta = sigmoid(b), decay = exp(-exp(A_log) softplus(a +
// dt_bias)) from ba[t] = [b (H) | a (H)], and q.k of the unit vectors. One CTA per token, one warp per query / key head.
__global__ void __launch_bounds__(128)
delta_prep_kernel(float* __restrict__ cs, int ld, const float* __restrict__ ba, const float* __restrict__ A_log,
                  const float* __restrict__ dt_bias, float* __restrict__ gates, int H, int G, int D, float unit_eps, float q_mult) {
  pdl_enter();
  const int i = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* row = cs + (size_t)i * ld;
  float* grow = gates + (size_t)i * (2 * H + G);
  for (int g = warp; g < G; g += 4) {
    float* q = row + (size_t)g * D;
    float* k = row + (size_t)(G + g) * D;
    float sq = 0.f, sk = 0.f, qk = 0.f;
    for (int c = lane; c < D; c += 32) { sq += q[c] * q[c]; sk += k[c] * k[c]; }
    const float rq = q_mult / sqrtf(warp_xor_sum(sq) + unit_eps), rk = 1.0f / sqrtf(warp_xor_sum(sk) + unit_eps);
    for (int c = lane; c < D; c += 32) {
      const float a = q[c] * rq, b = k[c] * rk;
      q[c] = a; k[c] = b;
      qk += a * b;
    }
    qk = warp_xor_sum(qk);
    if (lane == 0) grow[2 * H + g] = qk;
  }
  for (int h = tid; h < H; h += 128) {
    const float b = ba[(size_t)i * 2 * H + h], a = ba[(size_t)i * 2 * H + H + h];
    grow[h] = 1.0f / (1.0f + expf(-b));
    grow[H + h] = expf(-expf(A_log[h]) * softplus_f(a + dt_bias[h]));
  }
}

// ---- gated delta rule: the recurrence ---------------------------------------------------------------------------------------
// Per head, with S [D, DV] float32: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q. The columns of S are independent
// of one another: thread (row group rg of 8, column) keeps NS rows of one column in registers. Per token both S^T k and S^T q
// are taken from the state BEFORE the update (one reduction over the eight row groups by shuffles), and
//   u = beta (v - g (S^T k)),   o = g (S^T q) + (q.k) u,
// which is the read-out after the write. One CTA of four warps per (segment, head, 16 columns); the tokens' unit vectors, values
// and gates are copied into shared memory a block of BT tokens ahead (cp.async, two buffers). The state is read from the slot
// at the segment's start (zero at position 0) and written at its end. o leaves un-normalised, float32.
template <int NS, int BT>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ cs, int ld, const float* __restrict__ gates, float* __restrict__ state,
                  float* __restrict__ o, const int* __restrict__ meta, const int* __restrict__ seg_starts, int ntok, int H, int G,
                  int D, int DV) {
  pdl_enter();
  constexpr int DP = 8 * NS;
  __shared__ __align__(16) float sk[2][BT][DP], sq[2][BT][DP];
  __shared__ float sv[2][BT][16], sg[2][BT][4];                  // gates: beta, decay, q.k
  const int i = seg_starts[blockIdx.x], h = blockIdx.y, v0 = blockIdx.z * 16;
  const TokMeta mt = load_meta(meta, ntok, i);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rg = lane & 7, cc = warp * 4 + (lane >> 3), col = v0 + cc;
  const bool live = col < DV;
  const int d0 = rg * NS, kq = h / (H / G), GD = G * D, NG = 2 * H + G;
  float S[NS];
  float* st = state + (((size_t)mt.slot * H + h) * D) * DV;
#pragma unroll
  for (int r = 0; r < NS; ++r) S[r] = (mt.pos > 0 && live && d0 + r < D) ? st[(size_t)(d0 + r) * DV + col] : 0.f;
  // rows of the padded unit vectors beyond D stay zero in both buffers
  for (int e = tid; e < 2 * BT * DP; e += 128) { (&sk[0][0][0])[e] = 0.f; (&sq[0][0][0])[e] = 0.f; }
  __syncthreads();
  auto stage = [&](int buf, int tb) {
    const int nb = min(BT, mt.seg_end - tb);
    for (int e = tid; e < nb * D; e += 128) {
      const int tt = e / D, d = e - tt * D;
      const float* src = cs + (size_t)(tb + tt) * ld + (size_t)kq * D + d;
      cp_async_4(&sq[buf][tt][d], src);
      cp_async_4(&sk[buf][tt][d], src + GD);
    }
    for (int e = tid; e < nb * 16; e += 128) {
      const int tt = e >> 4, c = e & 15;
      if (v0 + c < DV) cp_async_4(&sv[buf][tt][c], cs + (size_t)(tb + tt) * ld + 2 * GD + (size_t)h * DV + v0 + c);
    }
    for (int e = tid; e < nb * 3; e += 128) {
      const int tt = e / 3, w = e - tt * 3;
      const float* gsrc = gates + (size_t)(tb + tt) * NG;
      cp_async_4(&sg[buf][tt][w], w == 0 ? gsrc + h : (w == 1 ? gsrc + H + h : gsrc + 2 * H + kq));
    }
    cp_async_commit();
  };
  stage(0, mt.seg_begin);
  int buf = 0;
  for (int tb = mt.seg_begin; tb < mt.seg_end; tb += BT, buf ^= 1) {
    if (tb + BT < mt.seg_end) { stage(buf ^ 1, tb + BT); cp_async_wait<1>(); } else cp_async_wait<0>();
    __syncthreads();
    const int nb = min(BT, mt.seg_end - tb);
    for (int tt = 0; tt < nb; ++tt) {
      const float4* k4 = reinterpret_cast<const float4*>(&sk[buf][tt][d0]);
      const float4* q4 = reinterpret_cast<const float4*>(&sq[buf][tt][d0]);
      float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
      float kr[NS];
#pragma unroll
      for (int r = 0; r < NS / 4; ++r) {
        const float4 k = k4[r], q = q4[r];
        kr[4 * r] = k.x; kr[4 * r + 1] = k.y; kr[4 * r + 2] = k.z; kr[4 * r + 3] = k.w;
        a0 += S[4 * r] * k.x;     b0 += S[4 * r] * q.x;
        a1 += S[4 * r + 1] * k.y; b1 += S[4 * r + 1] * q.y;
        a0 += S[4 * r + 2] * k.z; b0 += S[4 * r + 2] * q.z;
        a1 += S[4 * r + 3] * k.w; b1 += S[4 * r + 3] * q.w;
      }
      float a = a0 + a1, b = b0 + b1;
#pragma unroll
      for (int off = 1; off < 8; off <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, off);
        b += __shfl_xor_sync(0xffffffffu, b, off);
      }
      const float beta = sg[buf][tt][0], g = sg[buf][tt][1], qk = sg[buf][tt][2];
      const float v = live ? sv[buf][tt][cc] : 0.f;
      const float u = beta * (v - g * a);
#pragma unroll
      for (int r = 0; r < NS; ++r) S[r] = g * S[r] + kr[r] * u;
      if (rg == 0 && live) o[((size_t)(tb + tt) * H + h) * DV + col] = g * b + qk * u;
    }
    __syncthreads();                                             // the buffer is refilled two blocks later
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < NS; ++r)
      if (d0 + r < D) st[(size_t)(d0 + r) * DV + col] = S[r];
  }
}

// Per-head unit-RMS norm with one weight vector shared by the heads, times silu of a gate: one warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ src, const float* __restrict__ w, const T* __restrict__ gate, int gate_ld,
                      T* __restrict__ out, int ntok, int H, int DV, float eps) {
  pdl_enter();
  const long long r = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= (long long)ntok * H) return;
  const int lane = threadIdx.x & 31;
  const long long t = r / H;
  const int h = (int)(r - t * H);
  const float* s = src + r * DV;
  float ss = 0.f;
  for (int c = lane; c < DV; c += 32) ss += s[c] * s[c];
  const float rr = 1.0f / sqrtf(warp_xor_sum(ss) / (float)DV + eps);
  for (int c = lane; c < DV; c += 32) {
    float v = s[c] * rr * w[c];
    if (gate) v *= silu_f(to_f(gate[(size_t)t * gate_ld + (size_t)h * DV + c]));
    out[r * DV + c] = from_f<T>(v);
  }
}

// ---- selective scan (Mamba) ---------------------------------------------------------------------------------------------------
// Per channel c and state n: S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n; y_c = sum_n S[c, n] C_n + D_c x_c;
// out = y * silu(z). dt = softplus(dt_pre + dt_bias), A = -exp(A_log). RG neighbouring lanes share a channel, each with NS
// states in registers; their partial read-outs are added by shuffles, which is not part of the chain from token to token. One
// CTA of 128 threads per (segment, 128 / RG channels) walks the segment in blocks of BT tokens whose B, C, x and dt it first
// copies to shared memory (dt after the softplus); outputs are written per block.
template <typename T, int NS, int BT>
__global__ void __launch_bounds__(128)
mamba_scan_kernel(const T* __restrict__ x, int x_ld, const float* __restrict__ dt_pre, int dt_ld, const float* __restrict__ dt_bias,
                  const T* __restrict__ bc, int bc_ld, const T* __restrict__ z, int z_ld, const float* __restrict__ A_log,
                  const float* __restrict__ Dp, float* __restrict__ state, T* __restrict__ out, int out_ld,
                  const int* __restrict__ meta, const int* __restrict__ seg_starts, int ntok, int inner, int N, int RG) {
  pdl_enter();
  extern __shared__ __align__(16) float sm_ms[];                 // B [BT][NP] | C [BT][NP] | x [BT][CH] | dt [BT][CH] | y [BT][CH]
  const int CH = 128 / RG, NP = RG * NS;
  float* sB = sm_ms;
  float* sC = sB + BT * NP;
  float* sx = sC + BT * NP;
  float* sdt = sx + BT * CH;
  float* sy = sdt + BT * CH;
  const int i = seg_starts[blockIdx.x];
  const TokMeta mt = load_meta(meta, ntok, i);
  const int tid = threadIdx.x, rg = tid % RG, lc = tid / RG, c0 = blockIdx.y * CH, c = c0 + lc;
  const bool live = c < inner;
  const int n0 = rg * NS;
  float S[NS], A[NS];
  float* st = state + ((size_t)mt.slot * inner + (live ? c : 0)) * N;
#pragma unroll
  for (int r = 0; r < NS; ++r) {
    const bool ok = live && n0 + r < N;
    A[r] = ok ? -expf(A_log[(size_t)c * N + n0 + r]) : 0.f;
    S[r] = (ok && mt.pos > 0) ? st[n0 + r] : 0.f;
  }
  for (int tb = mt.seg_begin; tb < mt.seg_end; tb += BT) {
    const int nb = min(BT, mt.seg_end - tb);
    for (int e = tid; e < nb * NP; e += 128) {
      const int tt = e / NP, n = e - tt * NP;
      const T* row = bc + (size_t)(tb + tt) * bc_ld;
      sB[tt * NP + n] = n < N ? to_f(row[n]) : 0.f;
      sC[tt * NP + n] = n < N ? to_f(row[N + n]) : 0.f;
    }
    for (int e = tid; e < nb * CH; e += 128) {
      const int tt = e / CH, k = e - tt * CH, ch = c0 + k;
      float xv = 0.f, dv = 0.f;
      if (ch < inner) {
        xv = to_f(x[(size_t)(tb + tt) * x_ld + ch]);
        dv = softplus_f(dt_pre[(size_t)(tb + tt) * dt_ld + ch] + dt_bias[ch]);
      }
      sx[tt * CH + k] = xv;
      sdt[tt * CH + k] = dv;
    }
    __syncthreads();
    for (int tt = 0; tt < nb; ++tt) {
      const float dt = sdt[tt * CH + lc], dx = dt * sx[tt * CH + lc];
      const float4* B4 = reinterpret_cast<const float4*>(sB + tt * NP + n0);
      const float4* C4 = reinterpret_cast<const float4*>(sC + tt * NP + n0);
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int r = 0; r < NS / 4; ++r) {
        const float4 b = B4[r], cq = C4[r];
        S[4 * r] = expf(dt * A[4 * r]) * S[4 * r] + dx * b.x;             y0 += S[4 * r] * cq.x;
        S[4 * r + 1] = expf(dt * A[4 * r + 1]) * S[4 * r + 1] + dx * b.y; y1 += S[4 * r + 1] * cq.y;
        S[4 * r + 2] = expf(dt * A[4 * r + 2]) * S[4 * r + 2] + dx * b.z; y0 += S[4 * r + 2] * cq.z;
        S[4 * r + 3] = expf(dt * A[4 * r + 3]) * S[4 * r + 3] + dx * b.w; y1 += S[4 * r + 3] * cq.w;
      }
      float y = y0 + y1;
      for (int off = 1; off < RG; off <<= 1) y += __shfl_xor_sync(0xffffffffu, y, off);
      if (rg == 0) sy[tt * CH + lc] = y;
    }
    __syncthreads();
    for (int e = tid; e < nb * CH; e += 128) {
      const int tt = e / CH, k = e - tt * CH, ch = c0 + k;
      if (ch < inner) {
        const float zz = to_f(z[(size_t)(tb + tt) * z_ld + ch]);
        out[(size_t)(tb + tt) * out_ld + ch] = from_f<T>((sy[tt * CH + k] + Dp[ch] * sx[tt * CH + k]) * silu_f(zz));
      }
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < NS; ++r)
      if (n0 + r < N) st[n0 + r] = S[r];
  }
}

// ---- grouped-query attention: per-head norms, rotation, value norm and value mixing, cache write -----------------------------
// Row t of p: [q (H x D) | k (G x D) | v (G x DV)]. Per head: q, k <- unit_rms * weight (one weight vector for all heads), then
// the first rot_dims entries are rotated (entry i with entry i + rot_dims / 2, angle pos * inv_freq[i], float32). v <-
// unit_rms(v) without a weight; v_first_out receives it (float32) or, with v_first_in, v <- (1 - mix) v + mix v_first_in.
// qout [ntok, H, D] float32; cache_k[slot, pos % cap] and cache_v[slot, pos % cap] take the rows in the activation type.
// One CTA per token, a warp per head.
template <typename T>
__global__ void __launch_bounds__(128)
gqa_prep_kernel(const T* __restrict__ p, int ld, const float* __restrict__ qn_w, const float* __restrict__ kn_w,
                const float* __restrict__ inv_freq, int rot_dims, const float* __restrict__ v_first_in, float* __restrict__ v_first_out,
                const float* __restrict__ mix, float* __restrict__ qout, T* __restrict__ cache_k, T* __restrict__ cache_v, int cap,
                const int* __restrict__ meta, int ntok, int H, int G, int D, int DV, float eps, int v_norm) {
  pdl_enter();
  extern __shared__ float sm_gp[];                                // one row of max(D, DV) per warp
  const int i = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slot = meta[i], pos = meta[ntok + i];
  const int DM = max(D, DV);
  float* buf = sm_gp + warp * DM;
  const T* row = p + (size_t)i * ld;
  const int half = rot_dims / 2;
  const size_t crow = (size_t)slot * cap + (size_t)(pos % cap);
  for (int hh = warp; hh < H + G; hh += 4) {                      // query heads, then key heads
    const bool isq = hh < H;
    const T* src = row + (size_t)hh * D;
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) { const float v = to_f(src[c]); buf[c] = v; ss += v * v; }
    const float rr = 1.0f / sqrtf(warp_xor_sum(ss) / (float)D + eps);
    const float* w = isq ? qn_w : kn_w;
    __syncwarp();
    for (int c = lane; c < D; c += 32) buf[c] = buf[c] * rr * w[c];
    __syncwarp();
    float* qdst = isq ? qout + ((size_t)i * H + hh) * D : nullptr;
    T* kdst = isq ? nullptr : cache_k + (crow * G + (hh - H)) * D;
    for (int c = lane; c < D; c += 32) {
      float v = buf[c];
      if (c < 2 * half) {
        const int f = c < half ? c : c - half;
        float sn, cs;
        sincosf((float)pos * inv_freq[f], &sn, &cs);
        v = c < half ? buf[c] * cs - buf[c + half] * sn : buf[c] * cs + buf[c - half] * sn;
      }
      if (isq) qdst[c] = v; else kdst[c] = from_f<T>(v);
    }
    __syncwarp();
  }
  const float lam = (v_first_in && mix) ? mix[0] : 0.f;
  for (int g = warp; g < G; g += 4) {
    const T* src = row + (size_t)(H + G) * D + (size_t)g * DV;
    float ss = 0.f;
    for (int c = lane; c < DV; c += 32) { const float v = to_f(src[c]); buf[c] = v; ss += v * v; }
    const float rr = v_norm ? 1.0f / sqrtf(warp_xor_sum(ss) / (float)DV + eps) : 1.0f;
    T* vdst = cache_v + (crow * G + g) * DV;
    for (int c = lane; c < DV; c += 32) {
      float v = buf[c] * rr;
      const size_t fi = ((size_t)i * G + g) * DV + c;
      if (v_first_in) v = (1.0f - lam) * v + lam * v_first_in[fi];
      else if (v_first_out) v_first_out[fi] = v;
      vdst[c] = from_f<T>(v);
    }
    __syncwarp();
  }
}

// ---- softmax attention whose heads' weights are mixed after the softmax ("talking heads") ------------------------------------
// weight_g(j) = exp(s_g(j)) / (exp(sink_g) + sum_j exp(s_g(j))) for every query head g of a token; then head h uses
// sum_g talk[h, g] weight_g(j) on the values of ITS key/value head. Because the mix needs finished weights of all heads, a token
// is one CTA that makes two passes over its keys: the first finds every head's maximum and denominator, the second recomputes
// the scores of a block of BK keys, turns them into weights, mixes them through shared memory and applies them to the values.
// A warp takes the key rows of a block in turn (lanes along the row, the row's elements stay in registers for all query heads
// of the group). Which thread takes which key or output depends on nothing but the sizes, so a token's result does not depend
// on its neighbours in the batch or on how its sequence was cut.
template <typename T, int NACC, int BK>
__global__ void __launch_bounds__(256)
talking_attn_kernel(const float* __restrict__ q, const T* __restrict__ kc, long long k_ss, int k_rs, int k_hs,
                    const T* __restrict__ vc, long long v_ss, int v_rs, int v_hs, const float* __restrict__ talk,
                    const float* __restrict__ sink, T* __restrict__ out, const int* __restrict__ meta, int ntok, int H, int G, int D,
                    int DV, int window, int cap, float scale) {
  pdl_enter();
  extern __shared__ float sm_ta[];                                // q [H][D] | talk [H][H] | S [H][BK] | Wm [H][BK] | m [H] | rl [H]
  const int i = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* sq = sm_ta;
  float* stalk = sq + H * D;
  float* sS = stalk + H * H;
  float* sW = sS + H * BK;
  float* sm = sW + H * BK;
  float* srl = sm + H;
  const int slot = meta[i], pos = meta[ntok + i];
  const int rep = H / G;
  for (int e = tid; e < H * D; e += 256) sq[e] = q[(size_t)i * H * D + e] * scale;
  for (int e = tid; e < H * H; e += 256) stalk[e] = talk[e];
  for (int g = tid; g < H; g += 256) { sm[g] = sink ? sink[g] : -INFINITY; srl[g] = sink ? 1.f : 0.f; }
  __syncthreads();
  const T* kbase = kc + (size_t)slot * k_ss;
  const T* vbase = vc + (size_t)slot * v_ss;
  const int j0 = max(0, pos - window + 1);
  float acc[NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) acc[a] = 0.f;

  // scores of the keys jb .. jb + BK - 1 for all heads into sS (keys beyond pos: -inf)
  auto scores = [&](int jb) {
    for (int e = warp; e < BK * G; e += 8) {
      const int jj = e / G, kg = e - jj * G, j = jb + jj;
      if (j > pos) {
        for (int r = lane; r < rep; r += 32) sS[(kg * rep + r) * BK + jj] = -INFINITY;
        continue;
      }
      const T* kr = kbase + (size_t)(j % cap) * k_rs + (size_t)kg * k_hs;
      for (int r = 0; r < rep; ++r) {
        const float* qh = sq + (size_t)(kg * rep + r) * D;
        float dot = 0.f;
        for (int c = lane; c < D; c += 32) dot += qh[c] * to_f(kr[c]);
        dot = warp_xor_sum(dot);
        if (lane == 0) sS[(kg * rep + r) * BK + jj] = dot;
      }
    }
  };

  // pass 1: maxima and denominators
  for (int jb = j0; jb <= pos; jb += BK) {
    scores(jb);
    __syncthreads();
    for (int g = tid; g < H; g += 256) {
      float m = sm[g], l = srl[g];
      float mn = m;
      for (int jj = 0; jj < BK; ++jj) mn = fmaxf(mn, sS[g * BK + jj]);
      if (mn > -INFINITY) {
        l *= expf(m - mn);
        for (int jj = 0; jj < BK; ++jj) l += expf(sS[g * BK + jj] - mn);
      }
      sm[g] = mn; srl[g] = l;
    }
    __syncthreads();
  }
  for (int g = tid; g < H; g += 256) srl[g] = srl[g] > 0.f ? 1.0f / srl[g] : 0.f;
  __syncthreads();
  // pass 2: weights, mix, values
  for (int jb = j0; jb <= pos; jb += BK) {
    scores(jb);
    __syncthreads();
    for (int e = tid; e < H * BK; e += 256) {
      const int g = e / BK;
      sS[e] = expf(sS[e] - sm[g]) * srl[g];                       // exp(-inf) = 0 for keys beyond the token
    }
    __syncthreads();
    for (int e = tid; e < H * BK; e += 256) {
      const int h = e / BK, jj = e - h * BK;
      float s = 0.f;
      for (int g = 0; g < H; ++g) s += stalk[h * H + g] * sS[g * BK + jj];
      sW[e] = s;
    }
    __syncthreads();
    const int nk = min(BK, pos - jb + 1);
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int e = tid + 256 * a;
      if (e < H * DV) {
        const int h = e / DV, c = e - h * DV;
        const T* vcol = vbase + (size_t)(h / rep) * v_hs + c;
        const float* wr = sW + h * BK;
        float s = acc[a];
        for (int jj = 0; jj < nk; ++jj) s += wr[jj] * to_f(vcol[(size_t)((jb + jj) % cap) * v_rs]);
        acc[a] = s;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < NACC; ++a) {
    const int e = tid + 256 * a;
    if (e < H * DV) out[(size_t)i * H * DV + e] = from_f<T>(acc[a]);
  }
}

// ---- clamped gated feed-forward activation ------------------------------------------------------------------------------------
// out[t, f] = g * sigmoid(alpha g) * (u + 1) with g = min(gu[t, f], limit), u = clamp(gu[t, F + f], -limit, limit).
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
glu_clamp_kernel(const T* __restrict__ gu, int ld, T* __restrict__ out, int F, long long n, float limit, float alpha) {
  pdl_enter();
  for (long long k = ((long long)blockIdx.x * 256 + threadIdx.x) * VEC; k < n; k += (long long)gridDim.x * 256 * VEC) {
    const long long t = k / F;
    const int f = (int)(k - t * F);
    const VecF<VEC> g = ldv<VEC>(gu + (size_t)t * ld + f), u = ldv<VEC>(gu + (size_t)t * ld + F + f);
    VecF<VEC> o;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float gg = fminf(g.v[e], limit), uu = fminf(fmaxf(u.v[e], -limit), limit);
      o.v[e] = gg / (1.0f + expf(-alpha * gg)) * (uu + 1.0f);
    }
    stv<VEC>(out + k, o);
  }
}

__global__ void __launch_bounds__(256) scale_f32_kernel(float* __restrict__ a, long long n, float s) {
  pdl_enter();
  for (long long k = (long long)blockIdx.x * 256 + threadIdx.x; k < n; k += (long long)gridDim.x * 256) a[k] *= s;
}

}  // namespace qspec

using namespace qspec;
typedef __nv_bfloat16 bf16_t;
#define ST_DTYPE_OK(dtype) QSPEC_REQUIRE((dtype) == QSPEC_DTYPE_BF16 || (dtype) == QSPEC_DTYPE_F32, QSPEC_ERR_UNSUPPORTED, \
                                         "dtype %d: bfloat16 (1) or float32 (2) expected", (dtype))

extern "C" int qspec_seq_conv_act(const void* in, int ld, const float* w, const float* bias, int C, int taps, int act, float* tail,
                                  int slots, void* out, int out_ld, int out_f32, const int* meta, int ntok, int dtype, void* stream) {
  QSPEC_REQUIRE(in && w && out && meta && (tail || taps == 1), QSPEC_ERR_INVALID_ARG, "seq_conv_act: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && C > 0 && taps >= 1 && taps <= 64 && ld >= C && out_ld >= C && slots > 0, QSPEC_ERR_INVALID_ARG,
                "seq_conv_act: bad sizes");
  QSPEC_REQUIRE(act == QSPEC_CONV_ACT_NONE || act == QSPEC_CONV_ACT_SILU, QSPEC_ERR_INVALID_ARG, "seq_conv_act: unknown activation %d", act);
  ST_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  const dim3 grid(ntok, (C + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
#define CV_ARGS w, bias, taps, tail, slots
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(conv_act_kernel<float, float>, grid, dim3(256), 0, st, (const float*)in, ld, CV_ARGS, (float*)out, out_ld, meta, ntok, C, act);
  else if (out_f32)
    launch_pdl(conv_act_kernel<bf16_t, float>, grid, dim3(256), 0, st, (const bf16_t*)in, ld, CV_ARGS, (float*)out, out_ld, meta, ntok, C, act);
  else
    launch_pdl(conv_act_kernel<bf16_t, bf16_t>, grid, dim3(256), 0, st, (const bf16_t*)in, ld, CV_ARGS, (bf16_t*)out, out_ld, meta, ntok, C, act);
#undef CV_ARGS
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <int NS, int BT>
static void launch_delta_scan(const float* cs, int ld, const float* gates, float* state, float* o, const int* meta, const int* seg_starts,
                              int nseg, int ntok, int H, int G, int D, int DV, cudaStream_t st) {
  launch_pdl(delta_scan_kernel<NS, BT>, dim3(nseg, H, (DV + 15) / 16), dim3(128), 0, st, cs, ld, gates, state, o, meta, seg_starts, ntok, H,
             G, D, DV);
}

extern "C" int qspec_seq_delta_rule(float* cs, int ld, const float* ba, const float* A_log, const float* dt_bias, const float* norm_w,
                                    const void* gate, int gate_ld, float* state, float* gates, float* o, void* out, const int* meta,
                                    const int* seg_starts, int nseg, int ntok, int H, int G, int D, int DV, float unit_eps, float q_mult,
                                    float eps, int dtype, void* stream) {
  QSPEC_REQUIRE(cs && ba && A_log && dt_bias && norm_w && state && gates && o && out && meta && seg_starts, QSPEC_ERR_INVALID_ARG,
                "seq_delta_rule: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && nseg >= 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && D <= 256 && DV > 0 && ld >= 2 * G * D + H * DV,
                QSPEC_ERR_INVALID_ARG, "seq_delta_rule: bad sizes (key size <= 256, heads a multiple of the key heads)");
  ST_DTYPE_OK(dtype);
  if (ntok == 0 || nseg == 0) return QSPEC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  launch_pdl(delta_prep_kernel, dim3(ntok), dim3(128), 0, st, cs, ld, ba, A_log, dt_bias, gates, H, G, D, unit_eps, q_mult);
  QSPEC_CHECK_LAUNCH(1);
  if (D <= 32) launch_delta_scan<4, 16>(cs, ld, gates, state, o, meta, seg_starts, nseg, ntok, H, G, D, DV, st);
  else if (D <= 64) launch_delta_scan<8, 16>(cs, ld, gates, state, o, meta, seg_starts, nseg, ntok, H, G, D, DV, st);
  else if (D <= 128) launch_delta_scan<16, 16>(cs, ld, gates, state, o, meta, seg_starts, nseg, ntok, H, G, D, DV, st);
  else launch_delta_scan<32, 8>(cs, ld, gates, state, o, meta, seg_starts, nseg, ntok, H, G, D, DV, st);
  QSPEC_CHECK_LAUNCH(1);
  const long long rows = (long long)ntok * H;
  const dim3 grid((unsigned)((rows + 3) / 4));
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(head_norm_gate_kernel<float>, grid, dim3(128), 0, st, (const float*)o, norm_w, (const float*)gate, gate_ld, (float*)out, ntok, H,
               DV, eps);
  else
    launch_pdl(head_norm_gate_kernel<bf16_t>, grid, dim3(128), 0, st, (const float*)o, norm_w, (const bf16_t*)gate, gate_ld, (bf16_t*)out,
               ntok, H, DV, eps);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T, int NS>
static int launch_mamba(const void* x, int x_ld, const float* dt_pre, int dt_ld, const float* dt_bias, const void* bc, int bc_ld, const void* z,
                        int z_ld, const float* A_log, const float* Dp, float* state, void* out, int out_ld, const int* meta,
                        const int* seg_starts, int nseg, int ntok, int inner, int N, cudaStream_t st) {
  constexpr int BT = 16;
  int RG = 1;
  while (RG * NS < N) RG <<= 1;
  const int CH = 128 / RG, NP = RG * NS;
  const size_t smem = (size_t)(2 * BT * NP + 3 * BT * CH) * sizeof(float);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(mamba_scan_kernel<T, NS, BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  launch_pdl(mamba_scan_kernel<T, NS, BT>, dim3(nseg, (inner + CH - 1) / CH), dim3(128), smem, st, (const T*)x, x_ld, dt_pre, dt_ld, dt_bias,
             (const T*)bc, bc_ld, (const T*)z, z_ld, A_log, Dp, state, (T*)out, out_ld, meta, seg_starts, ntok, inner, N, RG);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_seq_selective_scan(const void* x, int x_ld, const float* dt_pre, int dt_ld, const float* dt_bias, const void* bc,
                                        int bc_ld, const void* z, int z_ld, const float* A_log, const float* D_skip, float* state,
                                        void* out, int out_ld, const int* meta, const int* seg_starts, int nseg, int ntok, int inner,
                                        int N, int dtype, void* stream) {
  QSPEC_REQUIRE(x && dt_pre && dt_bias && bc && z && A_log && D_skip && state && out && meta && seg_starts, QSPEC_ERR_INVALID_ARG,
                "seq_selective_scan: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && nseg >= 0 && inner > 0 && N > 0 && N <= 512 && bc_ld >= 2 * N, QSPEC_ERR_INVALID_ARG,
                "seq_selective_scan: bad sizes (state size <= 512)");
  ST_DTYPE_OK(dtype);
  if (ntok == 0 || nseg == 0) return QSPEC_OK;
  cudaStream_t st = (cudaStream_t)stream;
#define MS_ARGS x, x_ld, dt_pre, dt_ld, dt_bias, bc, bc_ld, z, z_ld, A_log, D_skip, state, out, out_ld, meta, seg_starts, nseg, ntok, inner, N, st
  if (dtype == QSPEC_DTYPE_F32) {
    if (N <= 4) return launch_mamba<float, 4>(MS_ARGS);
    if (N <= 8) return launch_mamba<float, 8>(MS_ARGS);
    return launch_mamba<float, 16>(MS_ARGS);
  }
  if (N <= 4) return launch_mamba<bf16_t, 4>(MS_ARGS);
  if (N <= 8) return launch_mamba<bf16_t, 8>(MS_ARGS);
  return launch_mamba<bf16_t, 16>(MS_ARGS);
#undef MS_ARGS
}

extern "C" int qspec_seq_gqa_prep(const void* p, int ld, const float* qn_w, const float* kn_w, const float* inv_freq, int rot_dims,
                                  const float* v_first_in, float* v_first_out, const float* mix, float* qout, void* cache_k,
                                  void* cache_v, int cap, const int* meta, int ntok, int H, int G, int D, int DV, float eps, int v_norm,
                                  int dtype, void* stream) {
  QSPEC_REQUIRE(p && qn_w && kn_w && qout && cache_k && cache_v && meta && (inv_freq || rot_dims == 0) && (!v_first_in || mix),
                QSPEC_ERR_INVALID_ARG, "seq_gqa_prep: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && DV > 0 && cap > 0 && rot_dims >= 0 && rot_dims % 2 == 0 &&
                rot_dims <= D && ld >= (H + G) * D + G * DV, QSPEC_ERR_INVALID_ARG, "seq_gqa_prep: bad sizes");
  ST_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  const size_t smem = (size_t)4 * (D > DV ? D : DV) * sizeof(float);
  QSPEC_REQUIRE(smem <= 48 * 1024, QSPEC_ERR_UNSUPPORTED, "seq_gqa_prep: head size above 3072");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(gqa_prep_kernel<float>, dim3(ntok), dim3(128), smem, st, (const float*)p, ld, qn_w, kn_w, inv_freq, rot_dims, v_first_in,
               v_first_out, mix, qout, (float*)cache_k, (float*)cache_v, cap, meta, ntok, H, G, D, DV, eps, v_norm);
  else
    launch_pdl(gqa_prep_kernel<bf16_t>, dim3(ntok), dim3(128), smem, st, (const bf16_t*)p, ld, qn_w, kn_w, inv_freq, rot_dims, v_first_in,
               v_first_out, mix, qout, (bf16_t*)cache_k, (bf16_t*)cache_v, cap, meta, ntok, H, G, D, DV, eps, v_norm);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T, int NACC>
static int launch_talking(const qspec_talking_attn_args* a, cudaStream_t st) {
  constexpr int BK = 32;
  const size_t smem = (size_t)(a->H * a->D + a->H * a->H + 2 * a->H * BK + 2 * a->H) * sizeof(float);
  QSPEC_REQUIRE(smem <= 200 * 1024, QSPEC_ERR_UNSUPPORTED, "seq_talking_attention: %zu bytes of shared memory for the queries and the mix", smem);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(talking_attn_kernel<T, NACC, BK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  launch_pdl(talking_attn_kernel<T, NACC, BK>, dim3(a->ntok), dim3(256), smem, st, a->q, (const T*)a->k, a->k_slot_stride, a->k_row_stride,
             a->k_head_stride, (const T*)a->v, a->v_slot_stride, a->v_row_stride, a->v_head_stride, a->talk, a->sink, (T*)a->out, a->meta,
             a->ntok, a->H, a->G, a->D, a->DV, a->window, a->cap, a->scale);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T>
static int launch_talking_n(const qspec_talking_attn_args* a, cudaStream_t st) {
  const long long n = (long long)a->H * a->DV;
  if (n <= 256) return launch_talking<T, 1>(a, st);
  if (n <= 512) return launch_talking<T, 2>(a, st);
  if (n <= 1024) return launch_talking<T, 4>(a, st);
  if (n <= 2048) return launch_talking<T, 8>(a, st);
  if (n <= 4096) return launch_talking<T, 16>(a, st);
  if (n <= 8192) return launch_talking<T, 32>(a, st);
  QSPEC_REQUIRE(n <= 16384, QSPEC_ERR_UNSUPPORTED, "seq_talking_attention: heads x value size above 16384");
  return launch_talking<T, 64>(a, st);
}

extern "C" int qspec_seq_talking_attention(const qspec_talking_attn_args* a, int dtype, void* stream) {
  QSPEC_REQUIRE(a && a->q && a->k && a->v && a->talk && a->out && a->meta, QSPEC_ERR_INVALID_ARG, "seq_talking_attention: null pointer");
  QSPEC_REQUIRE(a->ntok >= 0 && a->H > 0 && a->G > 0 && a->H % a->G == 0 && a->D > 0 && a->DV > 0 && a->window > 0 && a->cap > 0,
                QSPEC_ERR_INVALID_ARG, "seq_talking_attention: bad sizes");
  ST_DTYPE_OK(dtype);
  if (a->ntok == 0) return QSPEC_OK;
  if (dtype == QSPEC_DTYPE_F32) return launch_talking_n<float>(a, (cudaStream_t)stream);
  return launch_talking_n<bf16_t>(a, (cudaStream_t)stream);
}

extern "C" int qspec_seq_glu_clamp(const void* gu, int ld, void* out, int ntok, int F, float limit, float alpha, int dtype, void* stream) {
  QSPEC_REQUIRE(gu && out && ntok >= 0 && F > 0 && ld >= 2 * F, QSPEC_ERR_INVALID_ARG, "seq_glu_clamp: bad arguments");
  ST_DTYPE_OK(dtype);
  const long long n = (long long)ntok * F;
  if (n == 0) return QSPEC_OK;
  const size_t es = dtype == QSPEC_DTYPE_F32 ? 4 : 2;
  const bool vec = F % 4 == 0 && ld % 4 == 0 && (((uintptr_t)gu | (uintptr_t)out) & (4 * es - 1)) == 0;
  const long long per = vec ? 4 : 1;
  const unsigned blocks = (unsigned)((n / per + 255) / 256 > 4096 ? 4096 : (n / per + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == QSPEC_DTYPE_F32) {
    if (vec) launch_pdl(glu_clamp_kernel<float, 4>, dim3(blocks), dim3(256), 0, st, (const float*)gu, ld, (float*)out, F, n, limit, alpha);
    else launch_pdl(glu_clamp_kernel<float, 1>, dim3(blocks), dim3(256), 0, st, (const float*)gu, ld, (float*)out, F, n, limit, alpha);
  } else {
    if (vec) launch_pdl(glu_clamp_kernel<bf16_t, 4>, dim3(blocks), dim3(256), 0, st, (const bf16_t*)gu, ld, (bf16_t*)out, F, n, limit, alpha);
    else launch_pdl(glu_clamp_kernel<bf16_t, 1>, dim3(blocks), dim3(256), 0, st, (const bf16_t*)gu, ld, (bf16_t*)out, F, n, limit, alpha);
  }
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_seq_scale_f32(float* a, long long n, float s, void* stream) {
  QSPEC_REQUIRE(a && n >= 0, QSPEC_ERR_INVALID_ARG, "seq_scale_f32: bad arguments");
  if (n == 0) return QSPEC_OK;
  const unsigned blocks = (unsigned)((n + 255) / 256 > 4096 ? 4096 : (n + 255) / 256);
  launch_pdl(scale_f32_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, a, n, s);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

// Sequence-mixer kernels, fourth file: mixers whose per-sequence state is a matrix that every token rewrites (gated delta
// rule, selective scan), short causal convolutions with an activation, grouped-query attention whose heads' weights are mixed
// after the softmax, and the clamped gated feed-forward activation. bfloat16 / float32 activations (template T); everything that
// is normed, exponentiated or carried from token to token is float32.
#include "seq_common.cuh"
#include "../../include/qspec_b200_seq.h"
#include <stdint.h>
#include <stdlib.h>

namespace qspec {

// 4-byte asynchronous copies into shared memory (both addresses on 4-byte boundaries)
__device__ __forceinline__ void cp_async_4(float* smem_dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// 16-byte asynchronous copy into shared memory; `valid` false writes zeros and reads nothing
__device__ __forceinline__ void cp_async_16z(void* smem_dst, const void* src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src),
               "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void tk_ldmatrix_x4(uint32_t (&r)[4], const __nv_bfloat16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void tk_ldmatrix_x4_trans(uint32_t (&r)[4], const __nv_bfloat16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
// (hi, lo) split of two float32 weights: hi = bf16(w), lo = bf16(w - hi); hi + lo carries 16 mantissa bits
__device__ __forceinline__ void tk_split_bf2(float w0, float w1, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 h0 = __float2bfloat16_rn(w0), h1 = __float2bfloat16_rn(w1);
  __nv_bfloat162 hv, lv;
  hv.x = h0; hv.y = h1;
  lv = __floats2bfloat162_rn(w0 - __bfloat162float(h0), w1 - __bfloat162float(h1));
  hi = *reinterpret_cast<uint32_t*>(&hv);
  lo = *reinterpret_cast<uint32_t*>(&lv);
}
__device__ __forceinline__ void tk_mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

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
  if (i - mt.seg_begin >= K1 && taps <= 8) {                     // (uniform over the CTA) every tap lies in the step: loads without branches
    const T* src = in + (size_t)(i - K1) * ld + c;
    const float* wr = w + (size_t)c * taps;
    float v[8], ww[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int jc = j < taps ? j : 0;
      v[j] = to_f(src[(size_t)jc * ld]);
      ww[j] = j < taps ? wr[jc] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += ww[j] * v[j];
  } else
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
  // a row group's NS values sit SP apart, so that the eight groups' 16-byte reads fall on different banks
  constexpr int SP = NS >= 8 ? NS + 4 : NS, DP = 8 * SP;
  __shared__ __align__(16) float sk[2][BT][DP], sq[2][BT][DP];
  __shared__ float sv[2][BT][16];
  __shared__ __align__(16) float sg[2][BT][4];                   // gates: beta, decay, q.k
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
  // 128 / BT threads per token of the block: no division by a run-time size in the copy loops
  constexpr int TPT = 128 / BT;
  const int stt = tid / TPT, sl = tid % TPT;
  auto stage = [&](int buf, int tb) {
    const int t = tb + stt;
    if (t < mt.seg_end) {
      const float* src = cs + (size_t)t * ld + (size_t)kq * D;
      for (int d = sl, at = (sl / NS) * SP + sl % NS; d < D; d += TPT) {
        cp_async_4(&sq[buf][stt][at], src + d);
        cp_async_4(&sk[buf][stt][at], src + GD + d);
        if (TPT % NS == 0) at += (TPT / NS) * SP;                  // the step covers whole row groups
        else { const int dn = d + TPT; at = (dn / NS) * SP + dn % NS; }
      }
      const float* vsrc = cs + (size_t)t * ld + 2 * GD + (size_t)h * DV + v0;
      for (int c = sl; c < 16; c += TPT)
        if (v0 + c < DV) cp_async_4(&sv[buf][stt][c], vsrc + c);
      if (sl < 3) {
        const float* gsrc = gates + (size_t)t * NG;
        cp_async_4(&sg[buf][stt][sl], sl == 0 ? gsrc + h : (sl == 1 ? gsrc + H + h : gsrc + 2 * H + kq));
      }
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
      const float4* k4 = reinterpret_cast<const float4*>(&sk[buf][tt][rg * SP]);
      const float4* q4 = reinterpret_cast<const float4*>(&sq[buf][tt][rg * SP]);
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;   // short chains: the sums are on the token's critical path
      float kr[NS];
#pragma unroll
      for (int r = 0; r < NS / 4; ++r) {
        const float4 k = k4[r], q = q4[r];
        kr[4 * r] = k.x; kr[4 * r + 1] = k.y; kr[4 * r + 2] = k.z; kr[4 * r + 3] = k.w;
        a0 += S[4 * r] * k.x;     b0 += S[4 * r] * q.x;
        a1 += S[4 * r + 1] * k.y; b1 += S[4 * r + 1] * q.y;
        a2 += S[4 * r + 2] * k.z; b2 += S[4 * r + 2] * q.z;
        a3 += S[4 * r + 3] * k.w; b3 += S[4 * r + 3] * q.w;
      }
      float a = (a0 + a1) + (a2 + a3), b = (b0 + b1) + (b2 + b3);
#pragma unroll
      for (int off = 1; off < 8; off <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, off);
        b += __shfl_xor_sync(0xffffffffu, b, off);
      }
      const float4 gt = *reinterpret_cast<const float4*>(&sg[buf][tt][0]);
      const float beta = gt.x, g = gt.y, qk = gt.z;
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
// CTA of 128 threads per (segment, 128 / RG channels) walks the segment in blocks of BT tokens. A block's B, C, x, dt and z
// are fetched into registers while the block before it is applied, then parked in shared memory (dt after the softplus);
// outputs are written per block.
template <typename T, int NS, int RG>
__global__ void __launch_bounds__(128)
mamba_scan_kernel(const T* __restrict__ x, int x_ld, const float* __restrict__ dt_pre, int dt_ld, const float* __restrict__ dt_bias,
                  const T* __restrict__ bc, int bc_ld, const T* __restrict__ z, int z_ld, const float* __restrict__ A_log,
                  const float* __restrict__ Dp, float* __restrict__ state, T* __restrict__ out, int out_ld,
                  const int* __restrict__ meta, const int* __restrict__ seg_starts, int ntok, int inner, int N) {
  pdl_enter();
  constexpr int CH = 128 / RG, NP = RG * NS, BT = RG >= 8 ? 2 : 16 / RG;
  constexpr int XR = (BT * CH + 127) / 128, BR = (BT * NP + 127) / 128;
  __shared__ __align__(16) float sB[BT][NP], sC[BT][NP];
  __shared__ float sx[BT][CH], sdt[BT][CH], sz[BT][CH], sy[BT][CH];
  const int i = seg_starts[blockIdx.x];
  const TokMeta mt = load_meta(meta, ntok, i);
  const int tid = threadIdx.x, rg = tid % RG, lc = tid / RG, c0 = blockIdx.y * CH, c = c0 + lc;
  const bool live = c < inner;
  const int n0 = rg * NS;
  float S[NS], A[NS];
  float* st = state + ((size_t)mt.slot * inner + (live ? c : 0)) * N;
  float rx[XR], rd[XR], rz[XR], rb[BR], rc[BR];
  // every load of a block is issued before the first one is used: addresses outside the block are clamped into it rather than
  // skipped (a branch around a load would make the loads wait for one another), and what they bring is never used
  auto fetch = [&](int tb) {
#pragma unroll
    for (int r = 0; r < XR; ++r) {
      const int e = min(tid + 128 * r, BT * CH - 1), tt = e / CH, k = e % CH;
      const int t = min(tb + tt, mt.seg_end - 1), ch = min(c0 + k, inner - 1);
      rx[r] = to_f(x[(size_t)t * x_ld + ch]);
      rd[r] = dt_pre[(size_t)t * dt_ld + ch] + dt_bias[ch];
      rz[r] = to_f(z[(size_t)t * z_ld + ch]);
    }
#pragma unroll
    for (int r = 0; r < BR; ++r) {
      const int e = min(tid + 128 * r, BT * NP - 1), tt = e / NP, n = e % NP;
      const int t = min(tb + tt, mt.seg_end - 1), ns = min(n, N - 1);
      const T* row = bc + (size_t)t * bc_ld;
      const float b = to_f(row[ns]), cc = to_f(row[N + ns]);
      rb[r] = n < N ? b : 0.f;
      rc[r] = n < N ? cc : 0.f;
    }
  };
  fetch(mt.seg_begin);                                           // in flight while the state and the decay rates arrive
#pragma unroll
  for (int r = 0; r < NS; ++r) {
    const bool ok = live && n0 + r < N;
    // exp(dt A) = 2^(dt A log2 e): the rate is stored times log2 e, so that the token loop pays one multiply and one exp2
    A[r] = ok ? -expf(A_log[(size_t)c * N + n0 + r]) * 1.4426950408889634f : 0.f;
    S[r] = (ok && mt.pos > 0) ? st[n0 + r] : 0.f;
  }
  for (int tb = mt.seg_begin; tb < mt.seg_end; tb += BT) {
    const int nb = min(BT, mt.seg_end - tb);
#pragma unroll
    for (int r = 0; r < XR; ++r) {
      const int e = tid + 128 * r;
      if (e < BT * CH) {
        (&sx[0][0])[e] = rx[r];
        (&sdt[0][0])[e] = softplus_f(rd[r]);
        (&sz[0][0])[e] = rz[r];
      }
    }
#pragma unroll
    for (int r = 0; r < BR; ++r) {
      const int e = tid + 128 * r;
      if (e < BT * NP) { (&sB[0][0])[e] = rb[r]; (&sC[0][0])[e] = rc[r]; }
    }
    __syncthreads();
    if (tb + BT < mt.seg_end) fetch(tb + BT);
    for (int tt = 0; tt < nb; ++tt) {
      const float dt = sdt[tt][lc], dx = dt * sx[tt][lc];
      const float4* B4 = reinterpret_cast<const float4*>(&sB[tt][n0]);
      const float4* C4 = reinterpret_cast<const float4*>(&sC[tt][n0]);
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int r = 0; r < NS / 4; ++r) {
        const float4 b = B4[r], cq = C4[r];
        S[4 * r] = exp2f(dt * A[4 * r]) * S[4 * r] + dx * b.x;             y0 += S[4 * r] * cq.x;
        S[4 * r + 1] = exp2f(dt * A[4 * r + 1]) * S[4 * r + 1] + dx * b.y; y1 += S[4 * r + 1] * cq.y;
        S[4 * r + 2] = exp2f(dt * A[4 * r + 2]) * S[4 * r + 2] + dx * b.z; y0 += S[4 * r + 2] * cq.z;
        S[4 * r + 3] = exp2f(dt * A[4 * r + 3]) * S[4 * r + 3] + dx * b.w; y1 += S[4 * r + 3] * cq.w;
      }
      float y = y0 + y1;
#pragma unroll
      for (int off = 1; off < RG; off <<= 1) y += __shfl_xor_sync(0xffffffffu, y, off);
      if (rg == 0) sy[tt][lc] = y;
    }
    __syncthreads();
    for (int e = tid; e < nb * CH; e += 128) {
      const int tt = e / CH, k = e % CH, ch = c0 + k;
      if (ch < inner)
        out[(size_t)(tb + tt) * out_ld + ch] = from_f<T>((sy[tt][k] + Dp[ch] * sx[tt][k]) * silu_f(sz[tt][k]));
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
  extern __shared__ float sm_gp[];                                // one row of max(D, DV) per warp | cos [half] | sin [half]
  const int i = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slot = meta[i], pos = meta[ntok + i];
  const int DM = max(D, DV);
  float* buf = sm_gp + warp * DM;
  const T* row = p + (size_t)i * ld;
  const int half = rot_dims / 2;
  float* s_cos = sm_gp + 4 * DM;
  float* s_sin = s_cos + half;
  for (int f = threadIdx.x; f < half; f += 128) sincosf((float)pos * inv_freq[f], &s_sin[f], &s_cos[f]);   // once per token, for all heads
  __syncthreads();
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
        const float sn = s_sin[f], cs = s_cos[f];
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
// sum_g talk[h, g] weight_g(j) on the values of ITS key/value head. Because the mix needs finished weights of all heads, a CTA
// holds all heads of its tokens and makes two passes over the keys: the first finds every head's maximum and denominator, the
// second recomputes the scores of a block of BK keys, turns them into weights, mixes them through shared memory and applies
// them to the values. A CTA takes NQ consecutive batch rows; rows of one sequence share every key and value row that is read
// (prompt portions: NQ = 4), rows of different sequences are taken one after the other (decode-shaped batches launch NQ = 1).
//   scores   thread = (key of the block, key/value head): the key row passes through registers in 16-byte pieces and meets the
//            queries of all heads of its group and all NQ tokens (queries wait in shared memory, pre-multiplied by the scale)
//   mix      thread = (token, key, four heads): talk is kept transposed so that four heads' factors are one load
//   values   thread = (key/value head, two value columns): one value load serves the heads of the group and the NQ tokens; the
//            accumulators live in shared memory between blocks
// The block partition of the keys starts at the first key the group's first row sees, so with a full-length window every token's
// sums run in the same order however its sequence was cut. nsplit > 1 (NQ = 1 only): the CTAs of a cluster (grid y) take a
// token's key blocks in turn; they exchange their maxima and denominators after the first pass and add their partial outputs
// after the second through distributed shared memory, in rank order.
template <typename T, int REP, int NQ>
__global__ void __launch_bounds__(256)
talking_attn_kernel(const float* __restrict__ q, const T* __restrict__ kc, long long k_ss, int k_rs, int k_hs,
                    const T* __restrict__ vc, long long v_ss, int v_rs, int v_hs, const float* __restrict__ talk,
                    const float* __restrict__ sink, T* __restrict__ out, const int* __restrict__ meta, int ntok, int H, int G, int D,
                    int DV, int window, int cap, float scale, int vec_k, int vec_v, int nsplit, int tc_gc, int pv_tc) {
  pdl_enter();
  constexpr int BK = 64, KV = 16 / (int)sizeof(T);                // keys per block; elements of a 16-byte piece
  extern __shared__ __align__(16) float sm_ta[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int HP = (H + 3) & ~3, DP = (D + 3) & ~3, rep = H / G;
  // tc_gc > 0 (bfloat16, NQ = 4): the scores of both passes come from the tensor cores. The queries wait as bfloat16 rows
  // [key/value head][16 MT rows = (token, head of the group)][D + 8], the key rows of tc_gc key/value heads and one block at a time
  // as [head][key][D + 8] (cp.async); a warp takes 16 rows x 16 keys at a time with ldmatrix + mma.sync and writes float32 scores.
  // pv_tc: the value products too: the mixed weights leave shared memory as a two-term bfloat16 split (rows = the same 16-row
  // tiles), the value rows of a block come in as [head][key][DV + 8] and are read transposed; a warp owns up to eight tiles of
  // 16 rows x 16 value columns, whose sums stay in its registers over all key blocks.
  constexpr int MT = (NQ * REP + 15) / 16;
  constexpr bool TCK = sizeof(T) == 2 && NQ == 4;
  constexpr int UPW = TCK ? 8 : 1;
  const bool tc = TCK && tc_gc > 0;
  const bool pv = tc && pv_tc;
  float oacc[UPW][2][4];
  const int DQ = D + 8;
  float* sq = sm_ta;                                              // [NQ][H][DP] (CUDA-core scores only)
  float* stalk = sq + (tc ? 0 : NQ * H * DP);                     // [H][HP]: stalk[g][h] = talk[h][g]
  float* sS = stalk + H * HP;                                     // [NQ][H][BK]
  float* sW = sS + NQ * H * BK;                                   // [NQ][H][BK]
  float* sO = sW + NQ * H * BK;                                   // [NQ][H][DV]
  float* smx = sO + NQ * H * DV;                                  // [NQ][H] maxima
  float* srl = smx + NQ * H;                                      // [NQ][H] denominators, then their reciprocals
  float* spm = srl + NQ * H;                                      // [NQ][H] this CTA's own maxima / denominators, read by its cluster
  float* spl = spm + NQ * H;
  __nv_bfloat16* sQb = reinterpret_cast<__nv_bfloat16*>(spl + NQ * H);      // [G][16 MT][DQ]
  __nv_bfloat16* sKb = sQb + (size_t)G * 16 * MT * DQ;                       // [tc_gc][BK][DQ]
  const int rank = blockIdx.y;
  for (int e = tid; e < H * HP; e += 256) {
    const int g = e / HP, h = e - g * HP;
    stalk[e] = h < H ? talk[h * H + g] : 0.f;
  }
  const int row0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * NQ, rows_end = min(row0 + NQ, ntok);   // the batch's last rows see the most keys: first
  const int CP = (DV + 1) / 2, RC = (rep + REP - 1) / REP;
  int first = row0;
  while (first < rows_end) {
    // the rows first .. first + nq - 1 belong to one sequence (consecutive positions)
    const int slot = meta[first], pos0 = meta[ntok + first], seg_end = meta[3 * ntok + first];
    const int nq = min(rows_end, seg_end) - first;
    const int posl = pos0 + nq - 1;
    const int j0 = max(0, pos0 - window + 1);
    __syncthreads();                                             // the previous group is done with the shared buffers
    if (tc) {
      for (int e = tid; e < G * 16 * MT * DQ; e += 256) {
        const int c = e % DQ, t = e / DQ, rho = t % (16 * MT), kg = t / (16 * MT), a = rho / REP, r = rho % REP;
        const bool ok = c < D && a < nq && r < rep;
        sQb[e] = __float2bfloat16_rn(ok ? q[((size_t)(first + a) * H + kg * rep + r) * D + c] * scale : 0.f);
      }
    } else {
      for (int e = tid; e < nq * H * DP; e += 256) {
        const int r = e / DP, c = e - r * DP;
        sq[e] = c < D ? q[((size_t)first * H + r) * D + c] * scale : 0.f;
      }
    }
    for (int e = tid; e < nq * H; e += 256) {                    // the sink's term is counted once: by rank 0
      const bool sk = sink && rank == 0;
      smx[e] = sk ? sink[e % H] : -INFINITY;
      srl[e] = sk ? 1.f : 0.f;
    }
    for (int e = tid; e < nq * H * DV; e += 256) sO[e] = 0.f;
#pragma unroll
    for (int i = 0; i < UPW; ++i)
#pragma unroll
      for (int x = 0; x < 4; ++x) oacc[i][0][x] = oacc[i][1][x] = 0.f;
    __syncthreads();
    const T* kbase = kc + (size_t)slot * k_ss;
    const T* vbase = vc + (size_t)slot * v_ss;

    auto scores = [&](int jb) {
      if (tc) {
        const int gid = lane >> 2, tig = lane & 3, np8 = D / 8;
        for (int kg0 = 0; kg0 < G; kg0 += tc_gc) {
          const int gcn = min(tc_gc, G - kg0);
          __syncthreads();                                         // the tile's previous readers are done
          for (int e = tid; e < gcn * BK * np8; e += 256) {
            const int pc = e % np8, t = e / np8, jj = t % BK, kgl = t / BK, j = min(jb + jj, posl);
            cp_async_16z(sKb + ((size_t)(kgl * BK + jj) * DQ + pc * 8),
                         kbase + (size_t)(j < cap ? j : j % cap) * k_rs + (size_t)(kg0 + kgl) * k_hs + pc * 8, jb + jj <= posl);
          }
          cp_async_commit();
          cp_async_wait<0>();
          __syncthreads();
          for (int u = warp; u < gcn * MT * (BK / 16); u += 8) {
            const int np = u % (BK / 16), t = u / (BK / 16), mt = t % MT, kgl = t / MT, kg = kg0 + kgl;
            float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
            const __nv_bfloat16* qa = sQb + ((size_t)(kg * MT + mt) * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * DQ + 8 * (lane >> 4);
            const __nv_bfloat16* kb = sKb + ((size_t)kgl * BK + np * 16 + (lane & 7) + 8 * (lane >> 4)) * DQ + 8 * ((lane >> 3) & 1);
            for (int ks = 0; ks < D / 16; ++ks) {
              uint32_t af[4], bfr[4];
              tk_ldmatrix_x4(af, qa + ks * 16);
              tk_ldmatrix_x4(bfr, kb + ks * 16);
              tk_mma_16816(c0, af, bfr[0], bfr[1]);
              tk_mma_16816(c1, af, bfr[2], bfr[3]);
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int rho = mt * 16 + gid + 8 * half, a = rho / REP, r = rho % REP;
              if (a < nq && r < rep) {
                const int pa = pos0 + a;
                float* dst = sS + (a * H + kg * rep + r) * BK + np * 16 + 2 * tig;
#pragma unroll
                for (int x = 0; x < 4; ++x) {                       // x: (second eight keys, odd column)
                  const int jj = np * 16 + 8 * (x >> 1) + 2 * tig + (x & 1), j = jb + jj;
                  const float val = (x >> 1) ? c1[2 * half + (x & 1)] : c0[2 * half + (x & 1)];
                  dst[8 * (x >> 1) + (x & 1)] = (j <= pa && pa - j < window) ? val : -INFINITY;
                }
              }
            }
          }
        }
        return;
      }
      for (int e = tid; e < BK * G; e += 256) {
        const int kg = e / BK, jj = e - kg * BK, j = jb + jj;
        float d[NQ][REP];
#pragma unroll
        for (int a = 0; a < NQ; ++a)
#pragma unroll
          for (int r = 0; r < REP; ++r) d[a][r] = 0.f;
        for (int rc = 0; rc < RC; ++rc) {
          const int h0 = kg * rep + rc * REP, nr = min(REP, rep - rc * REP);
          if (j <= posl) {
            const T* kr = kbase + (size_t)(j % cap) * k_rs + (size_t)kg * k_hs;
            if (vec_k) {
              // 16-byte pieces of the key row, eight (then two, then one) in flight before the first is used
              auto piece = [&](const uint4& u, int c) {
                float kf[8];
                if (sizeof(T) == 2) {
                  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
                  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
                  const float2 a2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.z));
                  const float2 a3 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.w));
                  kf[0] = a0.x; kf[1] = a0.y; kf[2] = a1.x; kf[3] = a1.y; kf[4] = a2.x; kf[5] = a2.y; kf[6] = a3.x; kf[7] = a3.y;
                } else {
                  kf[0] = __uint_as_float(u.x); kf[1] = __uint_as_float(u.y); kf[2] = __uint_as_float(u.z); kf[3] = __uint_as_float(u.w);
                  kf[4] = kf[5] = kf[6] = kf[7] = 0.f;
                }
#pragma unroll
                for (int a = 0; a < NQ; ++a)
#pragma unroll
                  for (int r = 0; r < REP; ++r)
                    if (a < nq && r < nr) {
                      const float4* q4 = reinterpret_cast<const float4*>(sq + (size_t)(a * H + h0 + r) * DP + c);
#pragma unroll
                      for (int x = 0; x < KV / 4; ++x) {
                        const float4 qq = q4[x];
                        d[a][r] += qq.x * kf[4 * x] + qq.y * kf[4 * x + 1] + qq.z * kf[4 * x + 2] + qq.w * kf[4 * x + 3];
                      }
                    }
              };
              const uint4* k16 = reinterpret_cast<const uint4*>(kr);
              const int np = D / KV;
              int pc = 0;
              for (; pc + 8 <= np; pc += 8) {
                uint4 u[8];
#pragma unroll
                for (int x = 0; x < 8; ++x) u[x] = k16[pc + x];
#pragma unroll
                for (int x = 0; x < 8; ++x) piece(u[x], (pc + x) * KV);
              }
              for (; pc + 2 <= np; pc += 2) {
                const uint4 u0 = k16[pc], u1 = k16[pc + 1];
                piece(u0, pc * KV);
                piece(u1, (pc + 1) * KV);
              }
              if (pc < np) piece(k16[pc], pc * KV);
            } else {
              for (int c = 0; c < D; ++c) {
                const float kv = to_f(kr[c]);
#pragma unroll
                for (int a = 0; a < NQ; ++a)
#pragma unroll
                  for (int r = 0; r < REP; ++r)
                    if (a < nq && r < nr) d[a][r] += sq[(size_t)(a * H + h0 + r) * DP + c] * kv;
              }
            }
          }
#pragma unroll
          for (int a = 0; a < NQ; ++a)
#pragma unroll
            for (int r = 0; r < REP; ++r)
              if (a < nq && r < nr) {
                const int pa = pos0 + a;
                sS[(a * H + h0 + r) * BK + jj] = (j <= pa && pa - j < window) ? d[a][r] : -INFINITY;
                d[a][r] = 0.f;
              }
        }
      }
    };

    // pass 1: maxima and denominators, one warp per (token, head) row in turn
    for (int jb = j0 + rank * BK; jb <= posl; jb += nsplit * BK) {
      scores(jb);
      __syncthreads();
      for (int r = warp; r < nq * H; r += 8) {
        const float s0 = sS[r * BK + lane], s1 = sS[r * BK + 32 + lane];
        const float m = smx[r];
        const float mn = fmaxf(m, warp_xor_max(fmaxf(s0, s1)));
        if (mn > -INFINITY) {                                     // uniform over the warp
          const float part = warp_xor_sum(expf(s0 - mn) + expf(s1 - mn));
          if (lane == 0) { srl[r] = srl[r] * expf(m - mn) + part; smx[r] = mn; }
        }
      }
      __syncthreads();
    }
    if (nsplit > 1) {                                            // every CTA of the cluster combines all the partial pairs, in rank order
      for (int e = tid; e < nq * H; e += 256) { spm[e] = smx[e]; spl[e] = srl[e]; }
      cluster_sync_all();
      const uint32_t pm = (uint32_t)__cvta_generic_to_shared(spm), pl = (uint32_t)__cvta_generic_to_shared(spl);
      for (int e = tid; e < nq * H; e += 256) {
        float M = -INFINITY;
        for (int r = 0; r < nsplit; ++r) M = fmaxf(M, __uint_as_float(ld_dsmem_u32(mapa_shared(pm + 4u * e, (uint32_t)r))));
        float L = 0.f;
        for (int r = 0; r < nsplit; ++r) {
          const float m = __uint_as_float(ld_dsmem_u32(mapa_shared(pm + 4u * e, (uint32_t)r)));
          const float l = __uint_as_float(ld_dsmem_u32(mapa_shared(pl + 4u * e, (uint32_t)r)));
          if (m > -INFINITY) L += l * expf(m - M);
        }
        smx[e] = M; srl[e] = L;
      }
      __syncthreads();
    }
    for (int e = tid; e < nq * H; e += 256) srl[e] = srl[e] > 0.f ? 1.0f / srl[e] : 0.f;
    __syncthreads();
    // value rows of a block into the tile buffer (once the scores' products have read the key rows out of it)
    auto load_values = [&](int jb, int kg0, int gcn) {
      const int DVQ = DV + 8, np8v = DV / 8;
      for (int e = tid; e < gcn * BK * np8v; e += 256) {
        const int pc = e % np8v, t = e / np8v, jj = t % BK, kgl = t / BK, j = min(jb + jj, posl);
        cp_async_16z(sKb + ((size_t)(kgl * BK + jj) * DVQ + pc * 8),
                     vbase + (size_t)(j < cap ? j : j % cap) * v_rs + (size_t)(kg0 + kgl) * v_hs + pc * 8, jb + jj <= posl);
      }
      cp_async_commit();
    };
    const bool v_ahead = pv && tc_gc >= G;                        // one tile holds all heads: the values travel while the weights are mixed
    // pass 2: weights, mix, values
    for (int jb = j0 + rank * BK; jb <= posl; jb += nsplit * BK) {
      scores(jb);
      __syncthreads();
      if (v_ahead) load_values(jb, 0, G);
      for (int e = tid; e < nq * H * BK; e += 256) {
        const int r = e / BK;
        sS[e] = expf(sS[e] - smx[r]) * srl[r];                    // exp(-inf) = 0 for keys a row does not see
      }
      __syncthreads();
      for (int e = tid; e < nq * (HP / 4) * BK; e += 256) {
        const int jj = e % BK, t = e / BK, hc = t % (HP / 4), a = t / (HP / 4);
        float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int g = 0; g < H; ++g) {
          const float p = sS[(a * H + g) * BK + jj];
          const float4 tk = *reinterpret_cast<const float4*>(stalk + g * HP + 4 * hc);
          w.x += tk.x * p; w.y += tk.y * p; w.z += tk.z * p; w.w += tk.w * p;
        }
        const int h = 4 * hc;
        sW[(a * H + h) * BK + jj] = w.x;
        if (h + 1 < H) sW[(a * H + h + 1) * BK + jj] = w.y;
        if (h + 2 < H) sW[(a * H + h + 2) * BK + jj] = w.z;
        if (h + 3 < H) sW[(a * H + h + 3) * BK + jj] = w.w;
      }
      __syncthreads();
      const int nk = min(BK, posl - jb + 1);
      if (TCK && pv) {
        const int gid = lane >> 2, tig = lane & 3, DVQ = DV + 8, ndp = DV / 16;
        for (int kg0 = 0; kg0 < G; kg0 += tc_gc) {
          const int gcn = min(tc_gc, G - kg0);
          if (!v_ahead) {
            __syncthreads();                                       // the tile's previous readers are done
            load_values(jb, kg0, gcn);
          }
          cp_async_wait<0>();
          __syncthreads();
#pragma unroll
          for (int i = 0; i < UPW; ++i) {
            const int u = warp + 8 * i;
            if (u >= G * MT * ndp) continue;
            const int dp = u % ndp, t = u / ndp, mt = t % MT, kg = t / MT;
            if (kg < kg0 || kg >= kg0 + gcn) continue;
            const int rho0 = mt * 16 + gid, rho1 = rho0 + 8;
            const bool ok0 = rho0 / REP < nq && rho0 % REP < rep, ok1 = rho1 / REP < nq && rho1 % REP < rep;
            const float* w0 = sW + ((rho0 / REP) * H + kg * rep + rho0 % REP) * BK + 2 * tig;
            const float* w1 = sW + ((rho1 / REP) * H + kg * rep + rho1 % REP) * BK + 2 * tig;
            const __nv_bfloat16* vt = sKb + ((size_t)(kg - kg0) * BK + (lane & 7) + 8 * ((lane >> 3) & 1)) * DVQ + dp * 16 + 8 * (lane >> 4);
            const float2 zero = make_float2(0.f, 0.f);
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
              const float2 a00 = ok0 ? *reinterpret_cast<const float2*>(w0 + kk * 16) : zero;
              const float2 a01 = ok0 ? *reinterpret_cast<const float2*>(w0 + kk * 16 + 8) : zero;
              const float2 a10 = ok1 ? *reinterpret_cast<const float2*>(w1 + kk * 16) : zero;
              const float2 a11 = ok1 ? *reinterpret_cast<const float2*>(w1 + kk * 16 + 8) : zero;
              uint32_t ah[4], al[4], b[4];
              tk_split_bf2(a00.x, a00.y, ah[0], al[0]);
              tk_split_bf2(a10.x, a10.y, ah[1], al[1]);
              tk_split_bf2(a01.x, a01.y, ah[2], al[2]);
              tk_split_bf2(a11.x, a11.y, ah[3], al[3]);
              tk_ldmatrix_x4_trans(b, vt + (size_t)kk * 16 * DVQ);
              tk_mma_16816(oacc[i][0], ah, b[0], b[1]);
              tk_mma_16816(oacc[i][0], al, b[0], b[1]);
              tk_mma_16816(oacc[i][1], ah, b[2], b[3]);
              tk_mma_16816(oacc[i][1], al, b[2], b[3]);
            }
          }
        }
        __syncthreads();
        continue;
      }
      for (int e = tid; e < G * RC * CP; e += 256) {
        const int cp = e % CP, t = e / CP, rc = t % RC, kg = t / RC;
        const int c = 2 * cp, h0 = kg * rep + rc * REP, nr = min(REP, rep - rc * REP);
        const bool two = c + 1 < DV;
        float acc[NQ][REP][2];
#pragma unroll
        for (int a = 0; a < NQ; ++a)
#pragma unroll
          for (int r = 0; r < REP; ++r) {
            const bool ok = a < nq && r < nr;
            acc[a][r][0] = ok ? sO[(a * H + h0 + r) * DV + c] : 0.f;
            acc[a][r][1] = ok && two ? sO[(a * H + h0 + r) * DV + c + 1] : 0.f;
          }
        const T* vcol = vbase + (size_t)kg * v_hs + c;
        int jj = 0;
        if (vec_v && two) {
          // eight value rows in flight before the first is used; the weights of four keys are one 16-byte read
          for (; jj + 8 <= nk; jj += 8) {
            float2 vv[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              const int j = jb + jj + x;
              const T* vp = vcol + (size_t)(j < cap ? j : j % cap) * v_rs;
              if (sizeof(T) == 2) vv[x] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vp));
              else vv[x] = *reinterpret_cast<const float2*>(vp);
            }
#pragma unroll
            for (int a = 0; a < NQ; ++a)
#pragma unroll
              for (int r = 0; r < REP; ++r)
                if (a < nq && r < nr) {
                  const float4* w4 = reinterpret_cast<const float4*>(sW + (a * H + h0 + r) * BK + jj);
                  const float4 wa = w4[0], wb = w4[1];
                  acc[a][r][0] += wa.x * vv[0].x + wa.y * vv[1].x + wa.z * vv[2].x + wa.w * vv[3].x +
                                  wb.x * vv[4].x + wb.y * vv[5].x + wb.z * vv[6].x + wb.w * vv[7].x;
                  acc[a][r][1] += wa.x * vv[0].y + wa.y * vv[1].y + wa.z * vv[2].y + wa.w * vv[3].y +
                                  wb.x * vv[4].y + wb.y * vv[5].y + wb.z * vv[6].y + wb.w * vv[7].y;
                }
          }
        }
        for (; jj < nk; ++jj) {
          const int j = jb + jj;
          const T* vp = vcol + (size_t)(j < cap ? j : j % cap) * v_rs;
          const float v0 = to_f(vp[0]), v1 = two ? to_f(vp[1]) : 0.f;
#pragma unroll
          for (int a = 0; a < NQ; ++a)
#pragma unroll
            for (int r = 0; r < REP; ++r)
              if (a < nq && r < nr) {
                const float w = sW[(a * H + h0 + r) * BK + jj];
                acc[a][r][0] += w * v0;
                acc[a][r][1] += w * v1;
              }
        }
#pragma unroll
        for (int a = 0; a < NQ; ++a)
#pragma unroll
          for (int r = 0; r < REP; ++r)
            if (a < nq && r < nr) {
              sO[(a * H + h0 + r) * DV + c] = acc[a][r][0];
              if (two) sO[(a * H + h0 + r) * DV + c + 1] = acc[a][r][1];
            }
      }
      __syncthreads();
    }
    if (nsplit > 1) {                                            // CTA r adds slice r of the outputs over the ranks, in rank order
      cluster_sync_all();
      const int n = nq * H * DV, per = (n + nsplit - 1) / nsplit, e_end = min(n, (rank + 1) * per);
      const uint32_t po = (uint32_t)__cvta_generic_to_shared(sO);
      for (int e = rank * per + tid; e < e_end; e += 256) {
        float v = 0.f;
        for (int r = 0; r < nsplit; ++r) v += __uint_as_float(ld_dsmem_u32(mapa_shared(po + 4u * e, (uint32_t)r)));
        out[(size_t)first * H * DV + e] = from_f<T>(v);
      }
      cluster_sync_all();                                        // nobody leaves while its partial sums may still be read
    } else if (TCK && pv) {
      const int gid = lane >> 2, tig = lane & 3, ndp = DV / 16;
#pragma unroll
      for (int i = 0; i < UPW; ++i) {
        const int u = warp + 8 * i;
        if (u >= G * MT * ndp) continue;
        const int dp = u % ndp, t = u / ndp, mt = t % MT, kg = t / MT;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int rho = mt * 16 + gid + 8 * half, a = rho / REP, r = rho % REP;
          if (a >= nq || r >= rep) continue;
          T* orow = out + ((size_t)(first + a) * H + kg * rep + r) * DV + dp * 16 + 2 * tig;
          orow[0] = from_f<T>(oacc[i][0][2 * half]);     orow[1] = from_f<T>(oacc[i][0][2 * half + 1]);
          orow[8] = from_f<T>(oacc[i][1][2 * half]);     orow[9] = from_f<T>(oacc[i][1][2 * half + 1]);
        }
      }
    } else {
      for (int e = tid; e < nq * H * DV; e += 256) out[(size_t)first * H * DV + e] = from_f<T>(sO[e]);
    }
    first += nq;
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

template <typename T, int NS, int RG>
static int launch_mamba(const void* x, int x_ld, const float* dt_pre, int dt_ld, const float* dt_bias, const void* bc, int bc_ld, const void* z,
                        int z_ld, const float* A_log, const float* Dp, float* state, void* out, int out_ld, const int* meta,
                        const int* seg_starts, int nseg, int ntok, int inner, int N, cudaStream_t st) {
  constexpr int CH = 128 / RG;
  launch_pdl(mamba_scan_kernel<T, NS, RG>, dim3(nseg, (inner + CH - 1) / CH), dim3(128), 0, st, (const T*)x, x_ld, dt_pre, dt_ld, dt_bias,
             (const T*)bc, bc_ld, (const T*)z, z_ld, A_log, Dp, state, (T*)out, out_ld, meta, seg_starts, ntok, inner, N);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T>
static int launch_mamba_n(const void* x, int x_ld, const float* dt_pre, int dt_ld, const float* dt_bias, const void* bc, int bc_ld, const void* z,
                          int z_ld, const float* A_log, const float* Dp, float* state, void* out, int out_ld, const int* meta,
                          const int* seg_starts, int nseg, int ntok, int inner, int N, cudaStream_t st) {
#define MS_ARGS x, x_ld, dt_pre, dt_ld, dt_bias, bc, bc_ld, z, z_ld, A_log, Dp, state, out, out_ld, meta, seg_starts, nseg, ntok, inner, N, st
  // up to 16 states per thread; larger state sizes spread over 2 .. 32 neighbouring lanes
  if (N <= 4) return launch_mamba<T, 4, 1>(MS_ARGS);
  if (N <= 8) return launch_mamba<T, 8, 1>(MS_ARGS);
  if (N <= 16) return launch_mamba<T, 16, 1>(MS_ARGS);
  if (N <= 32) return launch_mamba<T, 16, 2>(MS_ARGS);
  if (N <= 64) return launch_mamba<T, 16, 4>(MS_ARGS);
  if (N <= 128) return launch_mamba<T, 16, 8>(MS_ARGS);
  if (N <= 256) return launch_mamba<T, 16, 16>(MS_ARGS);
  return launch_mamba<T, 16, 32>(MS_ARGS);
#undef MS_ARGS
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
  if (dtype == QSPEC_DTYPE_F32)
    return launch_mamba_n<float>(x, x_ld, dt_pre, dt_ld, dt_bias, bc, bc_ld, z, z_ld, A_log, D_skip, state, out, out_ld, meta, seg_starts, nseg,
                                 ntok, inner, N, st);
  return launch_mamba_n<bf16_t>(x, x_ld, dt_pre, dt_ld, dt_bias, bc, bc_ld, z, z_ld, A_log, D_skip, state, out, out_ld, meta, seg_starts, nseg,
                                ntok, inner, N, st);
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
  const size_t smem = ((size_t)4 * (D > DV ? D : DV) + rot_dims) * sizeof(float);
  QSPEC_REQUIRE(smem <= 48 * 1024, QSPEC_ERR_UNSUPPORTED, "seq_gqa_prep: head size above 2048");
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

// Shared memory of talking_attn_kernel: tc_gc > 0 replaces the float32 queries by bfloat16 query rows and a key tile.
static size_t talking_smem_bytes(const qspec_talking_attn_args* a, int nq, int rep_t, int tc_gc, int pv_tc = 0) {
  const int HP = (a->H + 3) & ~3, DP = (a->D + 3) & ~3, mt = (nq * rep_t + 15) / 16;
  size_t fl = (size_t)a->H * HP + 2 * (size_t)nq * a->H * 64 + (size_t)nq * a->H * a->DV + 4 * (size_t)nq * a->H;
  if (tc_gc <= 0) return (fl + (size_t)nq * a->H * DP) * sizeof(float);
  const int dt = pv_tc && a->DV > a->D ? a->DV : a->D;          // the tile buffer holds key rows, then value rows
  return fl * sizeof(float) + (size_t)a->G * 16 * mt * (a->D + 8) * 2 + (size_t)tc_gc * 64 * (dt + 8) * 2;
}

template <typename T, int REP, int NQ>
static int launch_talking(const qspec_talking_attn_args* a, int nsplit, int tc_gc, int pv_tc, cudaStream_t st) {
  const size_t smem = talking_smem_bytes(a, NQ, REP, tc_gc, pv_tc);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(talking_attn_kernel<T, REP, NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  // 16-byte pieces of a key row, two value columns per load: only where every row starts on such a boundary
  const size_t es = sizeof(T);
  const int kv = 16 / (int)es;
  const int vec_k = a->D % kv == 0 && a->k_row_stride % kv == 0 && a->k_head_stride % kv == 0 && a->k_slot_stride % kv == 0 &&
                    ((uintptr_t)a->k & 15) == 0;
  const int vec_v = a->v_row_stride % 2 == 0 && a->v_head_stride % 2 == 0 && a->v_slot_stride % 2 == 0 && ((uintptr_t)a->v & (2 * es - 1)) == 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a->ntok + NQ - 1) / NQ, nsplit);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (nsplit > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = nsplit;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  QSPEC_CUDA(cudaLaunchKernelEx(&cfg, talking_attn_kernel<T, REP, NQ>, a->q, (const T*)a->k, a->k_slot_stride, a->k_row_stride, a->k_head_stride,
                                (const T*)a->v, a->v_slot_stride, a->v_row_stride, a->v_head_stride, a->talk, a->sink, (T*)a->out, a->meta,
                                a->ntok, a->H, a->G, a->D, a->DV, a->window, a->cap, a->scale, vec_k, vec_v, nsplit, tc_gc, pv_tc));
  count_launch(1);
  return QSPEC_OK;
}

template <typename T>
static int launch_talking_n(const qspec_talking_attn_args* a, int rows_per_cta, cudaStream_t st) {
  // the heads of a key/value group share every key and value load: 1, 2, 4 or 8 of them per thread (more in turns)
  const int rep = a->H / a->G;
  const int rep_t = rep == 1 ? 1 : rep == 2 ? 2 : rep <= 4 ? 4 : 8;
  const size_t limit = 200 * 1024;
  const bool four = rows_per_cta >= 4 && talking_smem_bytes(a, 4, rep_t, 0) <= limit;
  QSPEC_REQUIRE(talking_smem_bytes(a, 1, rep_t, 0) <= limit, QSPEC_ERR_UNSUPPORTED,
                "seq_talking_attention: %zu bytes of shared memory for one token's heads", talking_smem_bytes(a, 1, rep_t, 0));
  // bfloat16 prompt portions whose key rows are whole 16-byte pieces take their scores from the tensor cores, with as many
  // key/value heads per key tile as shared memory holds; QSPEC_SEQ_TALK_TC=0 keeps the CUDA-core scores, for comparison
  static const bool tc_on = [] { const char* v = getenv("QSPEC_SEQ_TALK_TC"); return !(v && v[0] == '0'); }();
  int tc_gc = 0, pv_tc = 0;
  static const bool pv_on = [] { const char* v = getenv("QSPEC_SEQ_TALK_PV_TC"); return !(v && v[0] == '0'); }();
  if (sizeof(T) == 2 && rows_per_cta >= 4 && tc_on && rep <= 8 && a->D % 16 == 0 && a->k_row_stride % 8 == 0 && a->k_head_stride % 8 == 0 &&
      a->k_slot_stride % 8 == 0 && ((uintptr_t)a->k & 15) == 0) {
    // value products on the tensor cores too where the value rows are whole 16-byte pieces and eight tiles per warp hold them
    const int mt = (4 * rep_t + 15) / 16;
    pv_tc = pv_on && a->DV % 16 == 0 && a->v_row_stride % 8 == 0 && a->v_head_stride % 8 == 0 && a->v_slot_stride % 8 == 0 &&
            ((uintptr_t)a->v & 15) == 0 && a->G * mt * (a->DV / 16) <= 64;
    for (int gc = a->G < 4 ? a->G : 4; gc >= 1 && !tc_gc; gc >>= 1)
      if (talking_smem_bytes(a, 4, rep_t, gc, pv_tc) <= 224 * 1024) tc_gc = gc;
    if (!tc_gc) pv_tc = 0;
  }
  if (four || tc_gc) {
    if (rep == 1) return launch_talking<T, 1, 4>(a, 1, tc_gc, pv_tc, st);
    if (rep == 2) return launch_talking<T, 2, 4>(a, 1, tc_gc, pv_tc, st);
    if (rep <= 4) return launch_talking<T, 4, 4>(a, 1, tc_gc, pv_tc, st);
    return launch_talking<T, 8, 4>(a, 1, tc_gc, pv_tc, st);
  }
  // one row per CTA: a cluster of four CTAs shares the row's key blocks (the split is fixed, so a token's sums do not depend on
  // what else the batch holds); QSPEC_SEQ_TALK_SPLIT=1 keeps one CTA per row, for comparison
  static const int split = [] { const char* v = getenv("QSPEC_SEQ_TALK_SPLIT"); const int n = v ? atoi(v) : 4; return n >= 1 && n <= 8 ? n : 4; }();
  if (rep == 1) return launch_talking<T, 1, 1>(a, split, 0, 0, st);
  if (rep == 2) return launch_talking<T, 2, 1>(a, split, 0, 0, st);
  if (rep <= 4) return launch_talking<T, 4, 1>(a, split, 0, 0, st);
  return launch_talking<T, 8, 1>(a, split, 0, 0, st);
}

extern "C" int qspec_seq_talking_attention(const qspec_talking_attn_args* a, int rows_per_cta, int dtype, void* stream) {
  QSPEC_REQUIRE(a && a->q && a->k && a->v && a->talk && a->out && a->meta, QSPEC_ERR_INVALID_ARG, "seq_talking_attention: null pointer");
  QSPEC_REQUIRE(a->ntok >= 0 && a->H > 0 && a->G > 0 && a->H % a->G == 0 && a->D > 0 && a->DV > 0 && a->window > 0 && a->cap > 0,
                QSPEC_ERR_INVALID_ARG, "seq_talking_attention: bad sizes");
  ST_DTYPE_OK(dtype);
  if (a->ntok == 0) return QSPEC_OK;
  if (dtype == QSPEC_DTYPE_F32) return launch_talking_n<float>(a, rows_per_cta, (cudaStream_t)stream);
  return launch_talking_n<bf16_t>(a, rows_per_cta, (cudaStream_t)stream);
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

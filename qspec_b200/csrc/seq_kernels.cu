// Sequence-mixer kernels (include/qspec_b200_seq.h): norms with a zero-centred weight fused with the residual sum and a
// short causal convolution over time, per-head query/key norms, chunk-local sigmoid attention over a per-slot cache,
// router and expert feed-forward in the token-per-CTA form. Templated on the element type of activations and large
// weights (bfloat16 / float32); every reduction, exponential and the residual stream are float32 in both.
#include <cstdlib>
#include <cstring>
#include "seq_common.cuh"
#include "../../include/qspec_b200_seq.h"

namespace qspec {

// seq_mma_kernels.cu: the token form on the tensor cores; -1 if it does not take the shape
int chunk_attention_token_mma(const void* qkv, int ld, const void* ck, const void* cv, const float* bias, void* out, const int* meta,
                              int ntok, int H, int G, int D, int DV, int size, float scale, float softcap, int max_keys,
                              cudaStream_t st);

// ---- embedding ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ x,
                                                    int W, int V) {
  pdl_enter();
  const int i = blockIdx.x;
  int id = ids[i];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const T* row = table + (size_t)id * W;
  for (int c = threadIdx.x; c < W; c += 256) x[(size_t)i * W + c] = to_f(row[c]);
}

// ---- residual + post-norm + pre-norm + short convolution ------------------------------------------------------
// A CTA walks over `run` consecutive tokens of the batch. The convolution needs the normalised rows of the previous
// taps-1 tokens: rows inside the step's segment are kept in a shared-memory ring (the CTA first recomputes the taps-1
// rows in front of its run), rows before the segment come from the per-slot tail. Every thread owns the same columns in
// all rows, so the ring needs no barriers beyond those of the two row reductions. VEC = 4: 16-byte accesses (W % 4 == 0).
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
norm_conv_kernel(const float* __restrict__ x_in, float* __restrict__ x_out, const T* __restrict__ y, int y_parts,
                 long long y_part_stride, long long y_tok_stride, const float* __restrict__ y_w,
                 const float* __restrict__ post_w, const float* __restrict__ pre_w, const float* __restrict__ conv_w,
                 int taps, float* __restrict__ tail, int slots, T* __restrict__ out, const int* __restrict__ meta, int ntok,
                 int W, float eps, int run) {
  pdl_enter();
  extern __shared__ __align__(16) float sm_rows[];          // ring [rc][W]
  __shared__ float red[8];
  const int tid = threadIdx.x;
  const int i0 = blockIdx.x * run, i1 = min(i0 + run, ntok);
  const int rc = (conv_w && out) ? taps : 1, hist = rc - 1;
  const float inv_w = 1.0f / (float)W;
  const size_t tail_buf = (size_t)slots * hist * W;
  const int first_seg = meta[2 * ntok + i0];
  const int u0 = hist > 0 ? max(first_seg, i0 - hist) : i0;

  for (int u = u0; u < i1; ++u) {
    float* hrow = sm_rows + (size_t)(u % rc) * W;
    const float* xr = x_in + (size_t)u * W;
    const bool own = u >= i0;
    if (y) {
      float ss = 0.f;
      for (int c = tid * VEC; c < W; c += 256 * VEC) {
        VecF<VEC> v;
#pragma unroll
        for (int e = 0; e < VEC; ++e) v.v[e] = 0.f;
        for (int p = 0; p < y_parts; ++p) {
          const VecF<VEC> e = ldv<VEC>(y + (size_t)u * y_tok_stride + (size_t)p * y_part_stride + c);
          const float pw = y_w ? y_w[(size_t)u * y_parts + p] : 1.0f;
#pragma unroll
          for (int k = 0; k < VEC; ++k) v.v[k] += pw * e.v[k];
        }
        stv<VEC>(hrow + c, v);
#pragma unroll
        for (int k = 0; k < VEC; ++k) ss += v.v[k] * v.v[k];
      }
      const float r = 1.0f / sqrtf(block_sum_256(ss, red) * inv_w + eps);
      for (int c = tid * VEC; c < W; c += 256 * VEC) {
        const VecF<VEC> xv = ldv<VEC>(xr + c), yv = ldv<VEC>(hrow + c), pw = ldv<VEC>(post_w + c);
        VecF<VEC> v;
#pragma unroll
        for (int k = 0; k < VEC; ++k) v.v[k] = xv.v[k] + yv.v[k] * r * (1.0f + pw.v[k]);
        stv<VEC>(hrow + c, v);
        if (own) stv<VEC>(x_out + (size_t)u * W + c, v);
      }
    } else {
      for (int c = tid * VEC; c < W; c += 256 * VEC) {
        const VecF<VEC> v = ldv<VEC>(xr + c);
        stv<VEC>(hrow + c, v);
        if (own && x_out && x_out != x_in) stv<VEC>(x_out + (size_t)u * W + c, v);
      }
    }
    if (!out) continue;
    float ss = 0.f;
    for (int c = tid * VEC; c < W; c += 256 * VEC) {
      const VecF<VEC> v = ldv<VEC>(hrow + c);
#pragma unroll
      for (int k = 0; k < VEC; ++k) ss += v.v[k] * v.v[k];
    }
    const float r = 1.0f / sqrtf(block_sum_256(ss, red) * inv_w + eps);
    for (int c = tid * VEC; c < W; c += 256 * VEC) {
      VecF<VEC> v = ldv<VEC>(hrow + c);
      const VecF<VEC> pw = ldv<VEC>(pre_w + c);
#pragma unroll
      for (int k = 0; k < VEC; ++k) v.v[k] = v.v[k] * r * (1.0f + pw.v[k]);
      stv<VEC>(hrow + c, v);
    }
    if (!own) continue;
    // ---- token u: convolution over its own row and the taps-1 before it, then the tail
    const TokMeta m = load_meta(meta, ntok, u);
    const int pos_start = m.pos - (u - m.seg_begin);
    const float* tail_rd = tail ? tail + (size_t)m.phase * tail_buf + (size_t)m.slot * hist * W : nullptr;
    float* tail_wr = tail ? tail + (size_t)(1 - m.phase) * tail_buf + (size_t)m.slot * hist * W : nullptr;
    for (int c = tid * VEC; c < W; c += 256 * VEC) {
      const VecF<VEC> h0 = ldv<VEC>(hrow + c);
      VecF<VEC> v = h0;
      if (conv_w) {
        for (int j = 0; j < taps; ++j) {
          VecF<VEC> src;
          const int uu = u - j;
          if (uu >= m.seg_begin) src = ldv<VEC>(sm_rows + (size_t)(uu % rc) * W + c);
          else {
            const int pu = m.pos - j;
            if (pu >= 0 && tail_rd) src = ldv<VEC>(tail_rd + (size_t)(pu - (pos_start - hist)) * W + c);
            else {
#pragma unroll
              for (int k = 0; k < VEC; ++k) src.v[k] = 0.f;
            }
          }
#pragma unroll
          for (int k = 0; k < VEC; ++k) v.v[k] += conv_w[(size_t)(c + k) * taps + (taps - 1 - j)] * src.v[k];
        }
      }
      stv<VEC>(out + (size_t)u * W + c, v);
    }
    if (!tail_wr || hist == 0) continue;
    const int pos_end = pos_start + (m.seg_end - m.seg_begin);    // new tail row r holds position pos_end - hist + r
    const int my_row = m.pos - (pos_end - hist);
    if (my_row >= 0)
      for (int c = tid * VEC; c < W; c += 256 * VEC) stv<VEC>(tail_wr + (size_t)my_row * W + c, ldv<VEC>(hrow + c));
    if (u == m.seg_begin) {                                       // rows older than the segment are carried over
      for (int r2 = 0; r2 < hist; ++r2) {
        const int p = pos_end - hist + r2;
        if (p >= pos_start) break;
        const int ro = p - (pos_start - hist);
        for (int c = tid * VEC; c < W; c += 256 * VEC) {
          VecF<VEC> v;
#pragma unroll
          for (int k = 0; k < VEC; ++k) v.v[k] = 0.f;
          if (p >= 0) v = ldv<VEC>(tail_rd + (size_t)ro * W + c);
          stv<VEC>(tail_wr + (size_t)r2 * W + c, v);
        }
      }
    }
  }
}

// ---- the same for long prompts, in two passes ---------------------------------------------------------------------
// norm_conv_kernel walks the rows of its run one after the other, two dependent block reductions per row, and so runs at
// the latency of that chain. With many tokens the work splits into (1) norm_rows_kernel: one CTA per token, the row in
// registers through both norms, no row depends on another; normalised rows go to a float32 scratch [ntok, W]; and
// (2) conv_rows_kernel: element-wise convolution over the scratch rows (rows before the segment from the tail), output
// and tail update. Column assignment and reduction order are those of norm_conv_kernel, so both forms agree bit for bit.
template <typename T, int VEC, int NV>
__global__ void __launch_bounds__(256)
norm_rows_kernel(const float* __restrict__ x_in, float* __restrict__ x_out, const T* __restrict__ y, int y_parts,
                 long long y_part_stride, long long y_tok_stride, const float* __restrict__ y_w,
                 const float* __restrict__ post_w, const float* __restrict__ pre_w, float* __restrict__ nrm, int W, float eps) {
  pdl_enter();
  __shared__ float red[8];
  const int u = blockIdx.x, tid = threadIdx.x;
  const float inv_w = 1.0f / (float)W;
  const float* xr = x_in + (size_t)u * W;
  VecF<VEC> v[NV];
  if (y) {
    float ss = 0.f;
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      const int c = (tid + q * 256) * VEC;
#pragma unroll
      for (int e = 0; e < VEC; ++e) v[q].v[e] = 0.f;
      if (c < W) {
        for (int p = 0; p < y_parts; ++p) {
          const VecF<VEC> e = ldv<VEC>(y + (size_t)u * y_tok_stride + (size_t)p * y_part_stride + c);
          const float pw = y_w ? y_w[(size_t)u * y_parts + p] : 1.0f;
#pragma unroll
          for (int k = 0; k < VEC; ++k) v[q].v[k] += pw * e.v[k];
        }
#pragma unroll
        for (int k = 0; k < VEC; ++k) ss += v[q].v[k] * v[q].v[k];
      }
    }
    const float r = 1.0f / sqrtf(block_sum_256(ss, red) * inv_w + eps);
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      const int c = (tid + q * 256) * VEC;
      if (c < W) {
        const VecF<VEC> xv = ldv<VEC>(xr + c), pw = ldv<VEC>(post_w + c);
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[q].v[k] = xv.v[k] + v[q].v[k] * r * (1.0f + pw.v[k]);
        stv<VEC>(x_out + (size_t)u * W + c, v[q]);
      }
    }
  } else {
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      const int c = (tid + q * 256) * VEC;
      if (c < W) {
        v[q] = ldv<VEC>(xr + c);
        if (x_out && x_out != x_in) stv<VEC>(x_out + (size_t)u * W + c, v[q]);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int q = 0; q < NV; ++q)
    if ((tid + q * 256) * VEC < W) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) ss += v[q].v[k] * v[q].v[k];
    }
  const float r = 1.0f / sqrtf(block_sum_256(ss, red) * inv_w + eps);
#pragma unroll
  for (int q = 0; q < NV; ++q) {
    const int c = (tid + q * 256) * VEC;
    if (c < W) {
      const VecF<VEC> pw = ldv<VEC>(pre_w + c);
#pragma unroll
      for (int k = 0; k < VEC; ++k) v[q].v[k] = v[q].v[k] * r * (1.0f + pw.v[k]);
      stv<VEC>(nrm + (size_t)u * W + c, v[q]);
    }
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
conv_rows_kernel(const float* __restrict__ nrm, const float* __restrict__ conv_w, int taps, float* __restrict__ tail, int slots,
                 T* __restrict__ out, const int* __restrict__ meta, int ntok, int W) {
  pdl_enter();
  const int u = blockIdx.x, tid = threadIdx.x, hist = taps - 1;
  const size_t tail_buf = (size_t)slots * hist * W;
  const TokMeta m = load_meta(meta, ntok, u);
  const int pos_start = m.pos - (u - m.seg_begin);
  const float* tail_rd = tail + (size_t)m.phase * tail_buf + (size_t)m.slot * hist * W;
  float* tail_wr = tail + (size_t)(1 - m.phase) * tail_buf + (size_t)m.slot * hist * W;
  const float* hrow = nrm + (size_t)u * W;
  for (int c = tid * VEC; c < W; c += 256 * VEC) {
    VecF<VEC> v = ldv<VEC>(hrow + c);
    for (int j = 0; j < taps; ++j) {
      VecF<VEC> src;
      const int uu = u - j;
      if (uu >= m.seg_begin) src = ldv<VEC>(nrm + (size_t)uu * W + c);
      else {
        const int pu = m.pos - j;
        if (pu >= 0) src = ldv<VEC>(tail_rd + (size_t)(pu - (pos_start - hist)) * W + c);
        else {
#pragma unroll
          for (int k = 0; k < VEC; ++k) src.v[k] = 0.f;
        }
      }
#pragma unroll
      for (int k = 0; k < VEC; ++k) v.v[k] += conv_w[(size_t)(c + k) * taps + (taps - 1 - j)] * src.v[k];
    }
    stv<VEC>(out + (size_t)u * W + c, v);
  }
  const int pos_end = pos_start + (m.seg_end - m.seg_begin);      // new tail row r holds position pos_end - hist + r
  const int my_row = m.pos - (pos_end - hist);
  if (my_row >= 0)
    for (int c = tid * VEC; c < W; c += 256 * VEC) stv<VEC>(tail_wr + (size_t)my_row * W + c, ldv<VEC>(hrow + c));
  if (u == m.seg_begin) {                                         // rows older than the segment are carried over
    for (int r2 = 0; r2 < hist; ++r2) {
      const int p = pos_end - hist + r2;
      if (p >= pos_start) break;
      const int ro = p - (pos_start - hist);
      for (int c = tid * VEC; c < W; c += 256 * VEC) {
        VecF<VEC> v;
#pragma unroll
        for (int k = 0; k < VEC; ++k) v.v[k] = 0.f;
        if (p >= 0) v = ldv<VEC>(tail_rd + (size_t)ro * W + c);
        stv<VEC>(tail_wr + (size_t)r2 * W + c, v);
      }
    }
  }
}

// ---- per-head query / key norm ----------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
qk_norm_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ q_w, const float* __restrict__ k_w, int ntok, int H,
               int G, int D, float eps) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= (long long)ntok * (H + G)) return;
  const int t = (int)(row / (H + G)), hd = (int)(row % (H + G));
  T* p = qkv + (size_t)t * ld + (size_t)hd * D;               // key heads follow the query heads in the row
  const float* w = hd < H ? q_w : k_w;
  float ss = 0.f;
  for (int c = lane; c < D; c += 32) {
    const float v = to_f(p[c]);
    ss += v * v;
  }
  ss = warp_xor_sum(ss);
  const float r = 1.0f / sqrtf(ss / (float)D + eps);
  for (int c = lane; c < D; c += 32) p[c] = from_f<T>(to_f(p[c]) * r * w[c]);
}

// ---- chunk-local sigmoid attention, one CTA per (token, query head) ------------------------------------------------
__device__ __forceinline__ float capped_sigmoid_weight(float dot, float scale, float softcap, float bias) {
  float s = dot * scale;
  if (softcap > 0.f) s = softcap * tanhf(s / softcap);
  return 1.0f / (1.0f + expf(-(s + bias)));
}

// One CTA (4 warps) per (token, key/value head): the H/G query heads that share the key/value head are served together,
// so that every key and value row is fetched once per token. Keys and values go through shared memory in blocks of 32
// rows, in their storage type, one 32-bit word per lane (two bfloat16 or one float32: coalesced loads, conflict-free
// stores); the next block is fetched into registers while the current one is used. Scores: one lane per key (rows padded
// to an odd number of words); weighted sum of values: one thread per output word.
constexpr int ATT_KB = 32;       // keys per block
constexpr int ATT_CH = 4;        // 32-word column chunks per row: D, DV <= 128 words (256 bfloat16 / 128 float32)
constexpr int ATT_MAXW = 8;      // output words per thread: (H/G) * DV words <= 128 * ATT_MAXW

template <typename T> struct AttWord;
template <> struct AttWord<float> {
  static constexpr int N = 1;
  static __device__ __forceinline__ void get(uint32_t w, float& a, float& b) { a = __uint_as_float(w); b = 0.f; }
  static __device__ __forceinline__ uint32_t put(float a, float) { return __float_as_uint(a); }
};
template <> struct AttWord<__nv_bfloat16> {
  static constexpr int N = 2;
  static __device__ __forceinline__ void get(uint32_t w, float& a, float& b) {
    a = __uint_as_float(w << 16); b = __uint_as_float(w & 0xffff0000u);
  }
  static __device__ __forceinline__ uint32_t put(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

template <typename T>
__global__ void __launch_bounds__(128)
chunk_attn_kernel(const T* __restrict__ qkv, int ld, const T* __restrict__ ck, const T* __restrict__ cv,
                  const float* __restrict__ bias, T* __restrict__ out, const int* __restrict__ meta, int ntok, int H, int G,
                  int D, int DV, int size, float scale, float softcap, int nsplit) {
  pdl_enter();
  constexpr int WPE = AttWord<T>::N;
  extern __shared__ __align__(16) unsigned char sm_att_raw[];
  const int rep = H / G;
  const int kw = D / WPE, vw = DV / WPE;      // words per key / value row
  const int kst = kw | 1;                     // odd row stride: lanes that read different rows hit different banks
  float* sq = reinterpret_cast<float*>(sm_att_raw);          // [rep][D]
  float* sw = sq + rep * D;                                   // [rep][32]
  uint32_t* sk = reinterpret_cast<uint32_t*>(sw + rep * ATT_KB);   // [32][kst]
  uint32_t* sv = sk + ATT_KB * kst;                           // [32][vw]
  const int i = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const TokMeta m = load_meta(meta, ntok, i);
  const int pos_start = m.pos - (i - m.seg_begin);
  const int lo = (m.pos / size) * size;
  const int nkeys = m.pos - lo + 1;
  const int koff = H * D + g * D, voff = H * D + G * D + g * DV;
  for (int c = tid; c < rep * D; c += 128) sq[c] = to_f(qkv[(size_t)i * ld + (size_t)g * rep * D + c]);

  uint32_t pk[8][ATT_CH], pv[8][ATT_CH];     // this warp's 8 rows of the block in flight
  auto fetch = [&](int kb) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int jj = kb + warp + 4 * q;
      const bool ok = jj < nkeys;
      const int pj = lo + jj;
      const bool fresh = pj >= pos_start;
      const size_t brow = (size_t)(m.seg_begin + pj - pos_start) * ld;
      const size_t crow = (size_t)m.slot * size + jj;
      const uint32_t* kp = reinterpret_cast<const uint32_t*>(fresh ? qkv + brow + koff : ck + (crow * G + g) * D);
      const uint32_t* vp = reinterpret_cast<const uint32_t*>(fresh ? qkv + brow + voff : cv + (crow * G + g) * DV);
#pragma unroll
      for (int ch = 0; ch < ATT_CH; ++ch) {
        const int w = ch * 32 + lane;
        pk[q][ch] = (ok && w < kw) ? __ldg(kp + w) : 0u;
        pv[q][ch] = (ok && w < vw) ? __ldg(vp + w) : 0u;
      }
    }
  };
  float acc[ATT_MAXW][2];
#pragma unroll
  for (int k = 0; k < ATT_MAXW; ++k) acc[k][0] = acc[k][1] = 0.f;
  const int nout_w = rep * vw;
  // nsplit > 1: the CTAs of a cluster (grid z) take the key blocks in turn and add their partial sums at the end
  const int kstep = ATT_KB * nsplit, kb0 = ATT_KB * (int)blockIdx.z;
  if (kb0 < nkeys) fetch(kb0);
  for (int kb = kb0; kb < nkeys; kb += kstep) {
    __syncthreads();                          // the previous block has been consumed (and q is in place)
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int r = warp + 4 * q;
#pragma unroll
      for (int ch = 0; ch < ATT_CH; ++ch) {
        const int w = ch * 32 + lane;
        if (w < kw) sk[r * kst + w] = pk[q][ch];
        if (w < vw) sv[r * vw + w] = pv[q][ch];
      }
    }
    __syncthreads();
    if (kb + kstep < nkeys) fetch(kb + kstep);
    for (int hh = warp; hh < rep; hh += 4) {
      float w = 0.f;
      if (kb + lane < nkeys) {
        const uint32_t* kr = sk + lane * kst;
        const float* qr = sq + hh * D;
        float d0 = 0.f, d1 = 0.f;
        for (int c = 0; c < kw; ++c) {
          float a, b;
          AttWord<T>::get(kr[c], a, b);
          d0 += qr[c * WPE] * a;
          if (WPE == 2) d1 += qr[c * WPE + 1] * b;
        }
        w = capped_sigmoid_weight(d0 + d1, scale, softcap, bias[g * rep + hh]);
      }
      sw[hh * ATT_KB + lane] = w;
    }
    __syncthreads();
    const int nk = min(ATT_KB, nkeys - kb);
#pragma unroll
    for (int k = 0; k < ATT_MAXW; ++k) {
      const int o = tid + k * 128;
      if (o < nout_w) {
        const int hh = o / vw, dw = o - hh * vw;
        const float* wr = sw + hh * ATT_KB;
        float a0 = acc[k][0], a1 = acc[k][1];
        for (int r = 0; r < nk; ++r) {
          float a, b;
          AttWord<T>::get(sv[r * vw + dw], a, b);
          a0 += wr[r] * a;
          a1 += wr[r] * b;
        }
        acc[k][0] = a0; acc[k][1] = a1;
      }
    }
  }
  uint32_t* op = reinterpret_cast<uint32_t*>(out + (size_t)i * H * DV + (size_t)g * rep * DV);
  if (nsplit == 1) {
#pragma unroll
    for (int k = 0; k < ATT_MAXW; ++k) {
      const int o = tid + k * 128;
      if (o < nout_w) op[o] = AttWord<T>::put(acc[k][0], acc[k][1]);
    }
    return;
  }
  // Partial sums of every CTA of the cluster in its own shared memory; CTA r then adds slice r of the output words over
  // the ranks in rank order (the sum does not depend on which CTA finishes first) and stores it.
  float* sp = reinterpret_cast<float*>(sv + ATT_KB * vw);     // [nout_w][2]
#pragma unroll
  for (int k = 0; k < ATT_MAXW; ++k) {
    const int o = tid + k * 128;
    if (o < nout_w) { sp[2 * o] = acc[k][0]; sp[2 * o + 1] = acc[k][1]; }
  }
  cluster_sync_all();
  const int per = (nout_w + nsplit - 1) / nsplit;
  const int o_end = min(nout_w, ((int)blockIdx.z + 1) * per);
  const uint32_t sp_addr = (uint32_t)__cvta_generic_to_shared(sp);
  for (int o = (int)blockIdx.z * per + tid; o < o_end; o += 128) {
    float a0 = 0.f, a1 = 0.f;
    for (int r = 0; r < nsplit; ++r) {
      const uint32_t ra = mapa_shared(sp_addr + 8u * (uint32_t)o, (uint32_t)r);
      a0 += __uint_as_float(ld_dsmem_u32(ra));
      if (WPE == 2) a1 += __uint_as_float(ld_dsmem_u32(ra + 4));
    }
    op[o] = AttWord<T>::put(a0, a1);
  }
  cluster_sync_all();                          // nobody leaves while its partial sums may still be read
}

// The same for rows that cannot be read as 32-bit words (odd head sizes or leading dimensions in bfloat16): one CTA per
// (token, query head), element by element.
template <typename T>
__global__ void __launch_bounds__(128)
chunk_attn_plain_kernel(const T* __restrict__ qkv, int ld, const T* __restrict__ ck, const T* __restrict__ cv,
                        const float* __restrict__ bias, T* __restrict__ out, const int* __restrict__ meta, int ntok, int H, int G,
                        int D, int DV, int size, float scale, float softcap) {
  pdl_enter();
  extern __shared__ float sm_att[];           // q [D] | weights [size]
  float* sq = sm_att;
  float* sw = sm_att + D;
  const int i = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int g = h / (H / G);
  const TokMeta m = load_meta(meta, ntok, i);
  const int pos_start = m.pos - (i - m.seg_begin);
  const int lo = (m.pos / size) * size;
  const int nkeys = m.pos - lo + 1;
  const int koff = H * D + g * D, voff = H * D + G * D + g * DV;
  const T* qp = qkv + (size_t)i * ld + (size_t)h * D;
  for (int c = tid; c < D; c += 128) sq[c] = to_f(qp[c]);
  __syncthreads();
  const float b = bias[h];
  for (int jj = tid; jj < nkeys; jj += 128) {
    const int pj = lo + jj;
    const T* kp = pj >= pos_start ? qkv + (size_t)(m.seg_begin + pj - pos_start) * ld + koff
                                  : ck + (((size_t)m.slot * size + jj) * G + g) * D;
    float dot = 0.f;
    for (int c = 0; c < D; ++c) dot += sq[c] * to_f(kp[c]);
    sw[jj] = capped_sigmoid_weight(dot, scale, softcap, b);
  }
  __syncthreads();
  for (int d = tid; d < DV; d += 128) {
    float acc = 0.f;
    for (int jj = 0; jj < nkeys; ++jj) {
      const int pj = lo + jj;
      const T* vp = pj >= pos_start ? qkv + (size_t)(m.seg_begin + pj - pos_start) * ld + voff
                                    : cv + (((size_t)m.slot * size + jj) * G + g) * DV;
      acc += sw[jj] * to_f(vp[d]);
    }
    out[(size_t)i * H * DV + (size_t)h * DV + d] = from_f<T>(acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
cache_append_kernel(const T* __restrict__ qkv, int ld, T* __restrict__ ck, T* __restrict__ cv, const int* __restrict__ meta,
                    int ntok, int H, int G, int D, int DV, int size) {
  pdl_enter();
  const int i = blockIdx.x, tid = threadIdx.x;
  const TokMeta m = load_meta(meta, ntok, i);
  const int pos_start = m.pos - (i - m.seg_begin);
  const int last = pos_start + (m.seg_end - m.seg_begin) - 1;
  if (m.pos < (last / size) * size) return;
  const int row = m.pos % size;
  const T* kp = qkv + (size_t)i * ld + (size_t)H * D;
  const T* vp = kp + (size_t)G * D;
  T* kd = ck + ((size_t)m.slot * size + row) * G * D;
  T* vd = cv + ((size_t)m.slot * size + row) * G * DV;
  for (int c = tid; c < G * D; c += 128) kd[c] = kp[c];
  for (int c = tid; c < G * DV; c += 128) vd[c] = vp[c];
}

// ---- feed-forward pieces ----------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) relu2_kernel(T* __restrict__ a, long long n) {
  pdl_enter();
  for (long long k = (long long)blockIdx.x * 256 + threadIdx.x; k < n; k += (long long)gridDim.x * 256) {
    const float v = fmaxf(to_f(a[k]), 0.f);
    a[k] = from_f<T>(v * v);
  }
}

// Router: one CTA of 128 threads per token. Dot products by warp, then scores (softmax or sigmoid), group limits and top-k
// by one warp. The last n_extra rows of the router matrix are gate rows: their sigmoid goes to `extra`.
struct RouteOpts {
  int score_fn, n_groups, keep_groups, group_top, n_extra, extra_ld;
  float scale;
  float* extra;
};
template <typename T>
__global__ void __launch_bounds__(128)
route_kernel(const T* __restrict__ h, const float* __restrict__ rw, const float* __restrict__ corr, int* __restrict__ idx,
             float* __restrict__ weight, int W, int RE, int top, int chosen_only, RouteOpts ro) {
  pdl_enter();
  extern __shared__ float sm_rt[];            // z [R + gate rows] | choice [R] | group scores
  const int R = RE - ro.n_extra;              // the dot products cover the gate rows too; everything after them the experts only
  float* z = sm_rt;
  float* ch = sm_rt + RE;
  const int i = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const T* hp = h + (size_t)i * W;
  // four elements per lane and load where the rows allow it, four such loads in flight: the dot products are short and
  // latency-bound (router weights and the token's row both come from the L1 / L2)
  const bool vec = (W & 3) == 0 && ((uintptr_t)rw & 15) == 0 && ((uintptr_t)hp & (4 * sizeof(T) - 1)) == 0;
  if (vec) {
    // four router rows of a warp at a time (rows warp, warp + 4, warp + 8, warp + 12 of a group of 16): the token's row is
    // loaded once per step and four weight loads are in flight; every row keeps its own four partial sums, so the result
    // is the one of a row-by-row loop
    for (int r0 = warp; r0 < RE; r0 += 16) {
      float a4[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) a4[u][0] = a4[u][1] = a4[u][2] = a4[u][3] = 0.f;
#pragma unroll 2
      for (int c = lane * 4; c < W; c += 128) {
        const VecF<4> hv = ldv<4>(hp + c);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int r = r0 + 4 * u;
          if (r < RE) {
            const float4 wv = *reinterpret_cast<const float4*>(rw + (size_t)r * W + c);
            a4[u][0] += wv.x * hv.v[0]; a4[u][1] += wv.y * hv.v[1]; a4[u][2] += wv.z * hv.v[2]; a4[u][3] += wv.w * hv.v[3];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + 4 * u;
        const float acc = warp_xor_sum((a4[u][0] + a4[u][1]) + (a4[u][2] + a4[u][3]));
        if (r < RE && lane == 0) z[r] = acc;
      }
    }
  } else {
    for (int r = warp; r < RE; r += 4) {
      const float* wr = rw + (size_t)r * W;
      float acc = 0.f;
      for (int c = lane; c < W; c += 32) acc += wr[c] * to_f(hp[c]);
      acc = warp_xor_sum(acc);
      if (lane == 0) z[r] = acc;
    }
  }
  __syncthreads();
  if (warp != 0) return;
  if (chosen_only) {
    // the `top` largest logits, then a softmax over those alone (the first pick is their maximum)
    float first = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int r = lane; r < R; r += 32)
        if (z[r] > bv) { bv = z[r]; bi = r; }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (bi >= R) bi = 0;
      if (k == 0) first = bv;
      const float e = expf(bv - first);
      sum += e;
      if (lane == 0) {
        idx[(size_t)i * top + k] = bi;
        weight[(size_t)i * top + k] = e;
        z[bi] = -INFINITY;
      }
      __syncwarp();
    }
    if (lane == 0)
      for (int k = 0; k < top; ++k) weight[(size_t)i * top + k] /= sum;
    return;
  }
  for (int x = lane; x < ro.n_extra; x += 32) ro.extra[(size_t)i * ro.extra_ld + x] = 1.0f / (1.0f + expf(-z[R + x]));
  if (ro.score_fn == 1) {
    for (int r = lane; r < R; r += 32) {
      z[r] = 1.0f / (1.0f + expf(-z[r]));
      ch[r] = z[r] + (corr ? corr[r] : 0.f);
    }
  } else {
    float mx = -INFINITY;
    for (int r = lane; r < R; r += 32) mx = fmaxf(mx, z[r]);
    mx = warp_xor_max(mx);
    float sum = 0.f;
    for (int r = lane; r < R; r += 32) {
      const float e = expf(z[r] - mx);
      z[r] = e;
      sum += e;
    }
    sum = warp_xor_sum(sum);
    for (int r = lane; r < R; r += 32) {
      z[r] = z[r] / sum;
      ch[r] = z[r] + (corr ? corr[r] : 0.f);
    }
  }
  __syncwarp();
  if (ro.n_groups > 1) {
    // a group's score: the sum of its group_top largest choice scores (a lane per group); then every group counts the
    // groups ahead of it (larger score, or equal score and lower index) and drops out when keep_groups or more are
    float* gs = ch + R;
    const int size = R / ro.n_groups;
    for (int g = lane; g < ro.n_groups; g += 32) {
      const float* c = ch + g * size;
      float acc = 0.f, last = INFINITY;
      int last_i = -1;
      for (int k = 0; k < ro.group_top && k < size; ++k) {     // k-th largest: the largest entry after (last, last_i) in the order
        float bv = -INFINITY;
        int bi = -1;
        for (int e = 0; e < size; ++e) {
          const float v = c[e];
          const bool after = v < last || (v == last && e > last_i);
          if (after && (bi < 0 || v > bv)) { bv = v; bi = e; }
        }
        if (bi < 0) break;
        acc += bv;
        last = bv;
        last_i = bi;
      }
      gs[g] = acc;
    }
    __syncwarp();
    for (int g = lane; g < ro.n_groups; g += 32) {
      const float mine = gs[g];
      int ahead = 0;
      for (int o = 0; o < ro.n_groups; ++o) ahead += (gs[o] > mine || (gs[o] == mine && o < g)) ? 1 : 0;
      if (ahead >= ro.keep_groups)
        for (int e = 0; e < size; ++e) ch[g * size + e] = -INFINITY;
    }
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = lane; r < R; r += 32)
      if (ch[r] > bv) { bv = ch[r]; bi = r; }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi >= R) bi = 0;                                      // NaN scores: still a valid index
    if (lane == 0) {
      idx[(size_t)i * top + k] = bi;
      weight[(size_t)i * top + k] = z[bi] * ro.scale;
      ch[bi] = -INFINITY;
    }
    __syncwarp();
  }
}

// Expert feed-forward for few tokens: one CTA per (token, choice); a warp per output row, lanes along the reduction
// (coalesced weight rows, each read once per CTA).
template <typename T>
__global__ void __launch_bounds__(256)
expert_tokens_kernel(const T* __restrict__ h, const T* __restrict__ gate_up, const T* __restrict__ down,
                     const int* __restrict__ idx, T* __restrict__ out, int W, int F, int E, int top, float limit, int act) {
  pdl_enter();
  extern __shared__ float sm_ex[];            // h [W] | y [F]
  float* sh = sm_ex;
  float* sy = sm_ex + W;
  const int i = blockIdx.x, k = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int e = idx[(size_t)i * top + k];
  const T* hp = h + (size_t)i * W;
  T* op = out + ((size_t)i * top + k) * W;
  if (e >= E || e < 0) {
    for (int c = tid; c < W; c += 256) op[c] = hp[c];
    return;
  }
  for (int c = tid; c < W; c += 256) sh[c] = to_f(hp[c]);
  __syncthreads();
  const T* wg = gate_up + (size_t)e * (act == QSPEC_EXPERT_ACT_RELU2 ? 1 : 2) * F * W;
  const T* wu = wg + (size_t)F * W;
  if (act == QSPEC_EXPERT_ACT_RELU2) {
    for (int f = warp; f < F; f += 8) {
      float au = 0.f;
      for (int c = lane; c < W; c += 32) au += to_f(wg[(size_t)f * W + c]) * sh[c];
      au = warp_xor_sum(au);
      if (lane == 0) {
        const float u = fmaxf(to_f(from_f<T>(au)), 0.f);
        sy[f] = to_f(from_f<T>(u * u));
      }
    }
  } else
  for (int f = warp; f < F; f += 8) {
    float ag = 0.f, au = 0.f;
    for (int c = lane; c < W; c += 32) {
      ag += to_f(wg[(size_t)f * W + c]) * sh[c];
      au += to_f(wu[(size_t)f * W + c]) * sh[c];
    }
    ag = warp_xor_sum(ag);
    au = warp_xor_sum(au);
    if (lane == 0) {
      // the projections leave the matrix unit in the activation type
      if (act == QSPEC_EXPERT_ACT_SILU) {
        const float gq = to_f(from_f<T>(ag)), uq = to_f(from_f<T>(au));
        sy[f] = to_f(from_f<T>(gq / (1.0f + expf(-gq)) * uq));
      } else {
        const float gq = fminf(to_f(from_f<T>(ag)), limit);
        const float uq = fminf(fmaxf(to_f(from_f<T>(au)), -limit), limit);
        sy[f] = to_f(from_f<T>(gq * (1.0f / (1.0f + expf(-1.702f * gq))) * (uq + 1.0f)));
      }
    }
  }
  __syncthreads();
  const T* wd = down + (size_t)e * W * F;
  for (int c = warp; c < W; c += 8) {
    float acc = 0.f;
    for (int f = lane; f < F; f += 32) acc += to_f(wd[(size_t)c * F + f]) * sy[f];
    acc = warp_xor_sum(acc);
    if (lane == 0) op[c] = from_f<T>(acc);
  }
}

// ---- greedy sampling over float32 / bfloat16 logits -----------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
argmax_rows_any_kernel(const T* __restrict__ logits, int V, long long ld, long long* __restrict__ out_idx) {
  pdl_enter();
  __shared__ float sv[8];
  __shared__ int si[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* x = logits + (size_t)blockIdx.x * ld;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = tid; c < V; c += 256) {
    const float v = to_f(x[c]);
    if (v > bv) { bv = v; bi = c; }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
    out_idx[blockIdx.x] = bi < V ? bi : 0;
  }
}

}  // namespace qspec

using namespace qspec;

#define SEQ_DTYPE_OK(dtype) QSPEC_REQUIRE((dtype) == QSPEC_DTYPE_BF16 || (dtype) == QSPEC_DTYPE_F32, QSPEC_ERR_UNSUPPORTED, \
                                          "dtype %d: bfloat16 (1) or float32 (2) expected", (dtype))

extern "C" int qspec_seq_embed(const void* table, const int* ids, float* x, int ntok, int W, int V, int dtype, void* stream) {
  QSPEC_REQUIRE(table && ids && x, QSPEC_ERR_INVALID_ARG, "seq_embed: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && W > 0 && V > 0, QSPEC_ERR_INVALID_ARG, "seq_embed: bad sizes");
  SEQ_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(embed_kernel<float>, dim3(ntok), dim3(256), 0, (cudaStream_t)stream, (const float*)table, ids, x, W, V);
  else
    launch_pdl(embed_kernel<__nv_bfloat16>, dim3(ntok), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)table, ids, x, W, V);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T, int VEC>
static int launch_norm_conv(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride,
                            long long y_tok_stride, const float* y_w, const float* post_w, const float* pre_w,
                            const float* conv_w, int taps, float* tail, int slots, void* out, const int* meta, int ntok, int W,
                            float eps, cudaStream_t st) {
  const size_t smem = (size_t)taps * W * sizeof(float);
  QSPEC_REQUIRE(smem <= 200 * 1024, QSPEC_ERR_UNSUPPORTED, "seq_norm_conv: %d taps x width %d exceed shared memory", taps, W);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    QSPEC_CUDA((cudaFuncSetAttribute(norm_conv_kernel<T, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)));
    configured = smem;
  }
  // tokens per CTA: one while the batch is small (latency), a run of four once there are CTAs to spare
  const int run = ntok >= 1024 ? 4 : 1;
  launch_pdl(norm_conv_kernel<T, VEC>, dim3((ntok + run - 1) / run), dim3(256), smem, st, x_in, x_out, (const T*)y, y_parts,
             y_part_stride, y_tok_stride, y_w, post_w, pre_w, conv_w, taps, tail, slots, (T*)out, meta, ntok, W, eps, run);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T, int VEC, int NV>
static int launch_norm_rows(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride,
                            long long y_tok_stride, const float* y_w, const float* post_w, const float* pre_w,
                            const float* conv_w, int taps, float* tail, int slots, void* out, const int* meta, int ntok, int W,
                            float eps, float* scratch, cudaStream_t st) {
  launch_pdl(norm_rows_kernel<T, VEC, NV>, dim3(ntok), dim3(256), 0, st, x_in, x_out, (const T*)y, y_parts, y_part_stride,
             y_tok_stride, y_w, post_w, pre_w, scratch, W, eps);
  QSPEC_CHECK_LAUNCH(1);
  launch_pdl(conv_rows_kernel<T, VEC>, dim3(ntok), dim3(256), 0, st, (const float*)scratch, conv_w, taps, tail, slots, (T*)out, meta,
             ntok, W);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

template <typename T, int VEC>
static int launch_norm_rows_nv(int nv, const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride,
                               long long y_tok_stride, const float* y_w, const float* post_w, const float* pre_w,
                               const float* conv_w, int taps, float* tail, int slots, void* out, const int* meta, int ntok, int W,
                               float eps, float* scratch, cudaStream_t st) {
#define NR_ARGS x_in, x_out, y, y_parts, y_part_stride, y_tok_stride, y_w, post_w, pre_w, conv_w, taps, tail, slots, out, meta, ntok, W, eps, scratch, st
  if (nv <= 1) return launch_norm_rows<T, VEC, 1>(NR_ARGS);
  if (nv <= 2) return launch_norm_rows<T, VEC, 2>(NR_ARGS);
  if (nv <= 4) return launch_norm_rows<T, VEC, 4>(NR_ARGS);
  return launch_norm_rows<T, VEC, 8>(NR_ARGS);
#undef NR_ARGS
}

extern "C" int qspec_seq_norm_conv(const float* x_in, float* x_out, const void* y, int y_parts, long long y_part_stride,
                                   long long y_tok_stride, const float* y_w, const float* post_w, const float* pre_w,
                                   const float* conv_w, int taps, float* tail, int slots, void* out, const int* meta, int ntok,
                                   int W, float eps, float* scratch, int dtype, void* stream) {
  QSPEC_REQUIRE(x_in && meta, QSPEC_ERR_INVALID_ARG, "seq_norm_conv: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && W > 0 && W <= 16384, QSPEC_ERR_UNSUPPORTED, "seq_norm_conv: width %d (1..16384)", W);
  QSPEC_REQUIRE(!y || (x_out && x_out != x_in && post_w && y_parts >= 1), QSPEC_ERR_INVALID_ARG,
                "seq_norm_conv: a pending sublayer output needs its norm weight and a separate x_out");
  QSPEC_REQUIRE(!out || pre_w, QSPEC_ERR_INVALID_ARG, "seq_norm_conv: out without a norm weight");
  QSPEC_REQUIRE(out || y, QSPEC_ERR_INVALID_ARG, "seq_norm_conv: nothing to do");
  if (!conv_w) taps = 1;
  QSPEC_REQUIRE(taps >= 1 && taps <= 8, QSPEC_ERR_UNSUPPORTED, "seq_norm_conv: %d taps (1..8)", taps);
  QSPEC_REQUIRE(!conv_w || taps == 1 || (tail && slots > 0), QSPEC_ERR_INVALID_ARG, "seq_norm_conv: convolution without a tail buffer");
  SEQ_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  if (!conv_w) tail = nullptr;
  // 16-byte accesses when every row starts on a 16-byte boundary
  const bool al = W % 4 == 0 && y_part_stride % 4 == 0 && y_tok_stride % 4 == 0 &&
                  (((uintptr_t)x_in | (uintptr_t)x_out | (uintptr_t)y | (uintptr_t)out | (uintptr_t)tail | (uintptr_t)post_w |
                    (uintptr_t)pre_w) & 15) == 0;
  // long prompts with a convolution: two passes over independent rows (scratch: float32 [ntok, W]) once a row fits the
  // registers of its CTA
  const int vecw = al && ((uintptr_t)scratch & 15) == 0 ? 4 : 1;
  const int nv = (W + 256 * vecw - 1) / (256 * vecw);
  if (scratch && out && conv_w && taps > 1 && ntok >= 256 && nv <= 8) {
#define NR2_ARGS nv, x_in, x_out, y, y_parts, y_part_stride, y_tok_stride, y_w, post_w, pre_w, conv_w, taps, tail, slots, out, meta, ntok, W, eps, scratch, (cudaStream_t)stream
    if (dtype == QSPEC_DTYPE_F32) return vecw == 4 ? launch_norm_rows_nv<float, 4>(NR2_ARGS) : launch_norm_rows_nv<float, 1>(NR2_ARGS);
    return vecw == 4 ? launch_norm_rows_nv<__nv_bfloat16, 4>(NR2_ARGS) : launch_norm_rows_nv<__nv_bfloat16, 1>(NR2_ARGS);
#undef NR2_ARGS
  }
#define NC_ARGS x_in, x_out, y, y_parts, y_part_stride, y_tok_stride, y_w, post_w, pre_w, conv_w, taps, tail, slots, out, meta, ntok, W, eps, (cudaStream_t)stream
  if (dtype == QSPEC_DTYPE_F32) return al ? launch_norm_conv<float, 4>(NC_ARGS) : launch_norm_conv<float, 1>(NC_ARGS);
  return al ? launch_norm_conv<__nv_bfloat16, 4>(NC_ARGS) : launch_norm_conv<__nv_bfloat16, 1>(NC_ARGS);
#undef NC_ARGS
}

extern "C" int qspec_seq_qk_norm(void* qkv, int ld, const float* q_w, const float* k_w, int ntok, int H, int G, int D, float eps,
                                 int dtype, void* stream) {
  QSPEC_REQUIRE(qkv && q_w && k_w, QSPEC_ERR_INVALID_ARG, "seq_qk_norm: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && H > 0 && G > 0 && D > 0 && ld >= (H + G) * D, QSPEC_ERR_INVALID_ARG, "seq_qk_norm: bad sizes");
  SEQ_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  const long long rows = (long long)ntok * (H + G);
  const dim3 grid((unsigned)((rows + 3) / 4));
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(qk_norm_kernel<float>, grid, dim3(128), 0, (cudaStream_t)stream, (float*)qkv, ld, q_w, k_w, ntok, H, G, D, eps);
  else
    launch_pdl(qk_norm_kernel<__nv_bfloat16>, grid, dim3(128), 0, (cudaStream_t)stream, (__nv_bfloat16*)qkv, ld, q_w, k_w, ntok, H, G,
               D, eps);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

static int check_attn_args(const void* qkv, int ld, const void* ck, const void* cv, const int* meta, int ntok, int H, int G, int D,
                           int DV, int size, const char* what) {
  QSPEC_REQUIRE(qkv && ck && cv && meta, QSPEC_ERR_INVALID_ARG, "%s: null pointer", what);
  QSPEC_REQUIRE(ntok >= 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && DV > 0 && size > 0, QSPEC_ERR_INVALID_ARG,
                "%s: bad sizes (H %d, G %d, D %d, DV %d, chunk %d)", what, H, G, D, DV, size);
  QSPEC_REQUIRE(ld >= H * D + G * D + G * DV, QSPEC_ERR_INVALID_ARG, "%s: leading dimension %d too small", what, ld);
  return QSPEC_OK;
}

extern "C" int qspec_seq_chunk_attention(const void* qkv, int ld, const void* cache_k, const void* cache_v, const float* bias,
                                         void* out, const int* meta, int ntok, int H, int G, int D, int DV, int size, float scale,
                                         float softcap, int max_keys, int dtype, void* stream) {
  if (int s = check_attn_args(qkv, ld, cache_k, cache_v, meta, ntok, H, G, D, DV, size, "seq_chunk_attention")) return s;
  QSPEC_REQUIRE(bias && out, QSPEC_ERR_INVALID_ARG, "seq_chunk_attention: null pointer");
  SEQ_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  const int rep = H / G;
  // bfloat16 rows of head sizes 64 / 128: the tensor-core form (seq_mma_kernels.cu); QSPEC_SEQ_ATT=scalar keeps this file's
  static const bool scalar_only = [] { const char* v = getenv("QSPEC_SEQ_ATT"); return v && !strcmp(v, "scalar"); }();
  if (dtype == QSPEC_DTYPE_BF16 && !scalar_only) {
    const int s = chunk_attention_token_mma(qkv, ld, cache_k, cache_v, bias, out, meta, ntok, H, G, D, DV, size, scale, softcap,
                                            max_keys, (cudaStream_t)stream);
    if (s >= 0) return s;
  }
  const int wpe = dtype == QSPEC_DTYPE_F32 ? 1 : 2;
  const int w = dtype == QSPEC_DTYPE_F32 ? 0 : 1;
  cudaStream_t st = (cudaStream_t)stream;
  // word form: every row readable as 32-bit words, a row within ATT_CH chunks, the outputs within the per-thread budget
  const bool words = D % wpe == 0 && DV % wpe == 0 && ld % wpe == 0 && D / wpe <= 32 * ATT_CH && DV / wpe <= 32 * ATT_CH &&
                     (long long)rep * (DV / wpe) <= 128 * ATT_MAXW && (H * DV) % wpe == 0 &&
                     (((uintptr_t)qkv | (uintptr_t)cache_k | (uintptr_t)cache_v | (uintptr_t)out) & 3) == 0;
  if (words) {
    const int kst = (D / wpe) | 1;
    // Few tokens with many keys each (decoding): split the key blocks of a token over a cluster of up to 8 CTAs until
    // every SM has a few CTAs (measured at 64 tokens x 4 and x 8 key/value heads: 256 -> 512 CTAs 98 -> 55 us, 1024 CTAs
    // 63 us, 2048 CTAs 78 us -- the kernel is issue-bound, more CTAs than fill the SMs only add their fixed cost).
    // max_keys bounds the keys any token of the step sees (0: the chunk).
    const int blocks = ((max_keys > 0 ? min(max_keys, size) : size) + ATT_KB - 1) / ATT_KB;
    int nsplit = 1;
    while (nsplit < 8 && nsplit * 2 <= blocks && (long long)ntok * G * nsplit * 2 <= 1024) nsplit *= 2;
    const size_t smem = (size_t)(rep * D + rep * ATT_KB) * sizeof(float) + (size_t)ATT_KB * (kst + DV / wpe) * 4 +
                        (nsplit > 1 ? (size_t)rep * (DV / wpe) * 2 * sizeof(float) : 0);
    QSPEC_REQUIRE(smem <= 200 * 1024, QSPEC_ERR_UNSUPPORTED, "seq_chunk_attention: %d query heads of size %d per key/value head do not fit shared memory", rep, D);
    static size_t configured[2] = {0, 0};
    if (smem > 48 * 1024 && smem > configured[w]) {
      if (w == 0) QSPEC_CUDA(cudaFuncSetAttribute(chunk_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      else QSPEC_CUDA(cudaFuncSetAttribute(chunk_attn_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured[w] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ntok, G, nsplit);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (nsplit > 1) {
      attr[na].id = cudaLaunchAttributeClusterDimension;
      attr[na].val.clusterDim.x = 1;
      attr[na].val.clusterDim.y = 1;
      attr[na].val.clusterDim.z = nsplit;
      ++na;
    }
    if (pdl_enabled()) {
      attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[na].val.programmaticStreamSerializationAllowed = 1;
      ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (w == 0)
      QSPEC_CUDA(cudaLaunchKernelEx(&cfg, chunk_attn_kernel<float>, (const float*)qkv, ld, (const float*)cache_k,
                                    (const float*)cache_v, bias, (float*)out, meta, ntok, H, G, D, DV, size, scale, softcap, nsplit));
    else
      QSPEC_CUDA(cudaLaunchKernelEx(&cfg, chunk_attn_kernel<__nv_bfloat16>, (const __nv_bfloat16*)qkv, ld,
                                    (const __nv_bfloat16*)cache_k, (const __nv_bfloat16*)cache_v, bias, (__nv_bfloat16*)out, meta,
                                    ntok, H, G, D, DV, size, scale, softcap, nsplit));
    QSPEC_CHECK_LAUNCH(1);
    return QSPEC_OK;
  }
  const size_t smem = (size_t)(D + size) * sizeof(float);
  QSPEC_REQUIRE(smem <= 200 * 1024, QSPEC_ERR_UNSUPPORTED, "seq_chunk_attention: chunk of %d keys does not fit shared memory", size);
  static size_t configured_plain[2] = {0, 0};
  if (smem > 48 * 1024 && smem > configured_plain[w]) {
    if (w == 0) QSPEC_CUDA(cudaFuncSetAttribute(chunk_attn_plain_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    else QSPEC_CUDA(cudaFuncSetAttribute(chunk_attn_plain_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured_plain[w] = smem;
  }
  if (w == 0)
    launch_pdl(chunk_attn_plain_kernel<float>, dim3(ntok, H), dim3(128), smem, st, (const float*)qkv, ld, (const float*)cache_k,
               (const float*)cache_v, bias, (float*)out, meta, ntok, H, G, D, DV, size, scale, softcap);
  else
    launch_pdl(chunk_attn_plain_kernel<__nv_bfloat16>, dim3(ntok, H), dim3(128), smem, st, (const __nv_bfloat16*)qkv, ld,
               (const __nv_bfloat16*)cache_k, (const __nv_bfloat16*)cache_v, bias, (__nv_bfloat16*)out, meta, ntok, H, G, D, DV,
               size, scale, softcap);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_seq_cache_append(const void* qkv, int ld, void* cache_k, void* cache_v, const int* meta, int ntok, int H, int G,
                                      int D, int DV, int size, int dtype, void* stream) {
  if (int s = check_attn_args(qkv, ld, cache_k, cache_v, meta, ntok, H, G, D, DV, size, "seq_cache_append")) return s;
  SEQ_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(cache_append_kernel<float>, dim3(ntok), dim3(128), 0, (cudaStream_t)stream, (const float*)qkv, ld, (float*)cache_k,
               (float*)cache_v, meta, ntok, H, G, D, DV, size);
  else
    launch_pdl(cache_append_kernel<__nv_bfloat16>, dim3(ntok), dim3(128), 0, (cudaStream_t)stream, (const __nv_bfloat16*)qkv, ld,
               (__nv_bfloat16*)cache_k, (__nv_bfloat16*)cache_v, meta, ntok, H, G, D, DV, size);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_seq_relu2(void* a, long long n, int dtype, void* stream) {
  QSPEC_REQUIRE(a && n >= 0, QSPEC_ERR_INVALID_ARG, "seq_relu2: bad arguments");
  SEQ_DTYPE_OK(dtype);
  if (n == 0) return QSPEC_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(relu2_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (float*)a, n);
  else
    launch_pdl(relu2_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (__nv_bfloat16*)a, n);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

static int route_any(const void* h, const float* router_w, const float* correction, int* idx, float* weight, int ntok, int W, int R, int top,
                     int chosen_only, int dtype, void* stream, const RouteOpts* opts = nullptr) {
  RouteOpts ro = {0, 1, 1, 1, 0, 0, 1.0f, nullptr};
  if (opts) ro = *opts;
  QSPEC_REQUIRE(h && router_w && (correction || chosen_only || opts) && idx && weight, QSPEC_ERR_INVALID_ARG, "moe_route: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && W > 0 && R > 0 && R + ro.n_extra <= 1024 && top >= 1 && top <= 32 && top <= R, QSPEC_ERR_UNSUPPORTED,
                "moe_route: %d router outputs (<= 1024), top %d (<= 32)", R + ro.n_extra, top);
  QSPEC_REQUIRE(ro.n_extra >= 0 && (ro.n_extra == 0 || (ro.extra && ro.extra_ld >= ro.n_extra)), QSPEC_ERR_INVALID_ARG, "moe_route: gate rows without an output");
  QSPEC_REQUIRE(ro.n_groups >= 1 && R % ro.n_groups == 0 && ro.keep_groups >= 1 && ro.keep_groups <= ro.n_groups && ro.group_top >= 1 &&
                    top <= ro.keep_groups * (R / ro.n_groups),
                QSPEC_ERR_INVALID_ARG, "moe_route: %d groups (keep %d) of %d experts, top %d", ro.n_groups, ro.keep_groups, R, top);
  SEQ_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  const int RE = R + ro.n_extra;
  const size_t smem = (size_t)(RE + R + ro.n_groups) * sizeof(float);
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(route_kernel<float>, dim3(ntok), dim3(128), smem, (cudaStream_t)stream, (const float*)h, router_w, correction, idx,
               weight, W, RE, top, chosen_only, ro);
  else
    launch_pdl(route_kernel<__nv_bfloat16>, dim3(ntok), dim3(128), smem, (cudaStream_t)stream, (const __nv_bfloat16*)h, router_w,
               correction, idx, weight, W, RE, top, chosen_only, ro);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_moe_route_grouped(const void* h, const float* router_w, const float* correction, int* idx, float* weight, float* extra,
                                       int extra_ld, int ntok, int W, int R, int top, int score_fn, int n_groups, int keep_groups,
                                       int group_top, float scale, int n_extra, int dtype, void* stream) {
  QSPEC_REQUIRE(score_fn == 0 || score_fn == 1, QSPEC_ERR_INVALID_ARG, "moe_route_grouped: score function %d", score_fn);
  RouteOpts ro = {score_fn, n_groups < 1 ? 1 : n_groups, n_groups < 1 ? 1 : keep_groups, group_top, n_extra, extra_ld, scale, extra};
  return route_any(h, router_w, correction, idx, weight, ntok, W, R, top, 0, dtype, stream, &ro);
}

extern "C" int qspec_moe_route(const void* h, const float* router_w, const float* correction, int* idx, float* weight, int ntok, int W,
                               int R, int top, int dtype, void* stream) {
  return route_any(h, router_w, correction, idx, weight, ntok, W, R, top, 0, dtype, stream);
}

extern "C" int qspec_moe_route_chosen(const void* h, const float* router_w, int* idx, float* weight, int ntok, int W, int R, int top,
                                      int dtype, void* stream) {
  return route_any(h, router_w, nullptr, idx, weight, ntok, W, R, top, 1, dtype, stream);
}

extern "C" int qspec_moe_expert_tokens_act(const void* h, const void* gate_up, const void* down, const int* idx, void* out, int ntok, int W,
                                           int F, int E, int top, float limit, int act, int dtype, void* stream) {
  QSPEC_REQUIRE(act == QSPEC_EXPERT_ACT_GATED || act == QSPEC_EXPERT_ACT_RELU2 || act == QSPEC_EXPERT_ACT_SILU, QSPEC_ERR_INVALID_ARG,
                "moe_expert_tokens: unknown activation %d", act);
  QSPEC_REQUIRE(h && idx && out && (E == 0 || (gate_up && down)), QSPEC_ERR_INVALID_ARG, "moe_expert_tokens: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && W > 0 && F >= 0 && E >= 0 && top >= 1 && top <= 65535, QSPEC_ERR_INVALID_ARG, "moe_expert_tokens: bad sizes");
  SEQ_DTYPE_OK(dtype);
  if (ntok == 0) return QSPEC_OK;
  const size_t smem = (size_t)(W + F) * sizeof(float);
  QSPEC_REQUIRE(smem <= 200 * 1024, QSPEC_ERR_UNSUPPORTED, "moe_expert_tokens: width %d + expert size %d exceed shared memory", W, F);
  static size_t configured[2] = {0, 0};
  const int w = dtype == QSPEC_DTYPE_F32 ? 0 : 1;
  if (smem > 48 * 1024 && smem > configured[w]) {
    if (w == 0) QSPEC_CUDA(cudaFuncSetAttribute(expert_tokens_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    else QSPEC_CUDA(cudaFuncSetAttribute(expert_tokens_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[w] = smem;
  }
  if (w == 0)
    launch_pdl(expert_tokens_kernel<float>, dim3(ntok, top), dim3(256), smem, (cudaStream_t)stream, (const float*)h,
               (const float*)gate_up, (const float*)down, idx, (float*)out, W, F, E, top, limit, act);
  else
    launch_pdl(expert_tokens_kernel<__nv_bfloat16>, dim3(ntok, top), dim3(256), smem, (cudaStream_t)stream, (const __nv_bfloat16*)h,
               (const __nv_bfloat16*)gate_up, (const __nv_bfloat16*)down, idx, (__nv_bfloat16*)out, W, F, E, top, limit, act);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_moe_expert_tokens(const void* h, const void* gate_up, const void* down, const int* idx, void* out, int ntok, int W,
                                       int F, int E, int top, float limit, int dtype, void* stream) {
  return qspec_moe_expert_tokens_act(h, gate_up, down, idx, out, ntok, W, F, E, top, limit, QSPEC_EXPERT_ACT_GATED, dtype, stream);
}

extern "C" int qspec_seq_argmax_rows(const void* logits, int rows, int V, long long row_stride, long long* out_idx, int dtype,
                                     void* stream) {
  QSPEC_REQUIRE(logits && out_idx, QSPEC_ERR_INVALID_ARG, "seq_argmax_rows: null pointer");
  QSPEC_REQUIRE(rows >= 0 && V > 0 && row_stride >= V, QSPEC_ERR_INVALID_ARG, "seq_argmax_rows: bad sizes");
  SEQ_DTYPE_OK(dtype);
  if (rows == 0) return QSPEC_OK;
  if (dtype == QSPEC_DTYPE_F32)
    launch_pdl(argmax_rows_any_kernel<float>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (const float*)logits, V, row_stride, out_idx);
  else
    launch_pdl(argmax_rows_any_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)logits, V,
               row_stride, out_idx);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

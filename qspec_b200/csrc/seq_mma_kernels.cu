// Tensor-core forms of the sequence-mixer kernels (bfloat16 only; include/qspec_b200_seq.h):
//  * chunk-local sigmoid attention over 64-query tiles (prompts) and per token (decoding): warp-level mma.sync.m16n8k16
//    with float32 accumulators, like this library's other attention kernel for many sequences (seq_attention_kernel) --
//    the products are short (a chunk of keys, a handful of query heads) and their rows are gathered from two places;
//  * the grouped expert feed-forward: tcgen05.mma with the accumulator in tensor memory, operands gathered row by row
//    into the swizzled shared-memory operand layout by cp.async (the rows of an expert are scattered over the batch,
//    which is what rules out a plain TMA tile). The warp-level form of the same product is kept for comparison.
#include <cstdlib>
#include <cstring>
#include "common.cuh"
#include "../../include/qspec_b200_seq.h"

namespace qspec {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// (hi, lo) split of two float32 weights: hi = bf16(w), lo = bf16(w - hi); hi + lo carries 16 mantissa bits.
__device__ __forceinline__ void split_bf2(float w0, float w1, uint32_t& hi, uint32_t& lo) {
  const bf16 h0 = __float2bfloat16_rn(w0), h1 = __float2bfloat16_rn(w1);
  __nv_bfloat162 hv;
  hv.x = h0; hv.y = h1;
  hi = *reinterpret_cast<uint32_t*>(&hv);
  lo = pack_bf2(w0 - __bfloat162float(h0), w1 - __bfloat162float(h1));
}

// Weight of a visible key in the bfloat16 kernels: float32 throughout, with the exponentials on the special-function unit
// (ex2.approx: two units in the last place) instead of the exact library routines, which cost ~80 instructions a weight.
// tanh(u) = 1 - 2 / (e^(2u) + 1): its absolute error (~1e-7) is what the capped score carries into the sigmoid; the
// operands q and k are bfloat16 roundings (relative 4e-3), so nothing of this shows. Limits: e -> inf gives 1, e -> 0 gives -1.
__device__ __forceinline__ float capped_sigmoid_fast(float dot, float scale, float softcap, float bias) {
  float s = dot * scale;
  if (softcap > 0.f) s = softcap * (1.0f - __fdividef(2.0f, __expf(2.0f * s / softcap) + 1.0f));
  return __fdividef(1.0f, 1.0f + __expf(-(s + bias)));
}

// ---------------------------------------------------------------------------------------------------------------------
// Attention. One CTA (4 warps) per (64 consecutive batch tokens, query head). Keys come from two places:
//  * the step's own rows: batch indices [kmin, tile end), row i sees j in [lb_i, i] (lb_i = first batch row of its chunk
//    inside its segment);
//  * the cache, for rows whose chunk began before their segment: cache rows [0, nc_i) of the row's slot. Segments with
//    such rows are visited one after the other (a prompt tile has one; the caller sends decode-shaped batches elsewhere).
// Scores and weights are float32; the weights enter P.V as a two-term bfloat16 split.
// ---------------------------------------------------------------------------------------------------------------------
template <int D, int DV>
__global__ void __launch_bounds__(128)
chunk_attn_mma_kernel(const bf16* __restrict__ qkv, int ld, const bf16* __restrict__ ck, const bf16* __restrict__ cv,
                      const float* __restrict__ bias, bf16* __restrict__ out, const int* __restrict__ meta, int ntok, int H, int G,
                      int size, float scale, float softcap) {
  pdl_enter();
  constexpr int QP = D + 8, VP = 64 + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
  bf16* sK = sQ + 64 * QP;
  bf16* sVt = sK + 64 * QP;
  int* s_lb = reinterpret_cast<int*>(sVt + DV * VP);
  int* s_nc = s_lb + 64;
  int* s_sb = s_nc + 64;
  int* s_slot = s_sb + 64;
  int* s_seg = s_slot + 64;               // rows that open a cache segment
  __shared__ int s_kmin, s_nseg;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
  const int r0 = blockIdx.x * 64, h = blockIdx.y, g = h / (H / G);
  const int koff = H * D + g * D, voff = H * D + G * D + g * DV;
  if (tid == 0) { s_kmin = 0x7fffffff; s_nseg = 0; }
  __syncthreads();
  if (tid < 64) {
    const int i = r0 + tid;
    int lb = 0x7fffffff, nc = 0, sb = -1, slot = 0;
    if (i < ntok) {
      slot = meta[i];
      const int pos = meta[ntok + i];
      sb = meta[2 * ntok + i];
      const int pos_start = pos - (i - sb);
      const int lo = (pos / size) * size;
      lb = max(sb, i - (pos - lo));
      nc = lo < pos_start ? pos_start - lo : 0;
      atomicMin(&s_kmin, lb);
    }
    s_lb[tid] = lb; s_nc[tid] = nc; s_sb[tid] = sb; s_slot[tid] = slot;
  }
  // Q tile
  for (int v = tid; v < 64 * (D / 8); v += 128) {
    const int r = v / (D / 8), c = (v % (D / 8)) * 8;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (r0 + r < ntok) val = *reinterpret_cast<const uint4*>(qkv + (size_t)(r0 + r) * ld + (size_t)h * D + c);
    *reinterpret_cast<uint4*>(sQ + r * QP + c) = val;
  }
  __syncthreads();
  if (tid == 0) {                          // segments of this tile that reach into the cache, in batch order
    int n = 0, last = -1;
    for (int r = 0; r < 64; ++r)
      if (s_nc[r] > 0 && s_sb[r] != last) { s_seg[n++] = r; last = s_sb[r]; }
    s_nseg = n;
  }
  uint32_t qf[D / 16][4];
  {
    const int ra = warp * 16 + gid;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qf[ks][0] = *reinterpret_cast<const uint32_t*>(sQ + ra * QP + ks * 16 + tig * 2);
      qf[ks][1] = *reinterpret_cast<const uint32_t*>(sQ + (ra + 8) * QP + ks * 16 + tig * 2);
      qf[ks][2] = *reinterpret_cast<const uint32_t*>(sQ + ra * QP + ks * 16 + 8 + tig * 2);
      qf[ks][3] = *reinterpret_cast<const uint32_t*>(sQ + (ra + 8) * QP + ks * 16 + 8 + tig * 2);
    }
  }
  __syncthreads();
  float oacc[DV / 8][4];
#pragma unroll
  for (int nt = 0; nt < DV / 8; ++nt) oacc[nt][0] = oacc[nt][1] = oacc[nt][2] = oacc[nt][3] = 0.f;
  const float b = bias[h];
  const int rowA = warp * 16 + gid, rowB = rowA + 8;
  const int iA = r0 + rowA, iB = r0 + rowB;
  const int lbA = s_lb[rowA], lbB = s_lb[rowB];
  const int nseg = s_nseg, kmin = s_kmin;
  const int kend = min(r0 + 64, ntok);

  // source 0: the step's own rows; sources 1..nseg: cache rows of one segment each
  for (int src = 0; src <= nseg; ++src) {
    int kb0, kb1, seg_sb = -1, seg_slot = 0;
    if (src == 0) { kb0 = kmin; kb1 = kend; }
    else { const int r = s_seg[src - 1]; kb0 = 0; kb1 = s_nc[r]; seg_sb = s_sb[r]; seg_slot = s_slot[r]; }
    for (int kb = kb0; kb < kb1; kb += 64) {
      __syncthreads();                     // previous tile consumed
      for (int v = tid; v < 64 * (D / 8); v += 128) {
        const int r = v / (D / 8), c = (v % (D / 8)) * 8;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (kb + r < kb1)
          val = src == 0 ? *reinterpret_cast<const uint4*>(qkv + (size_t)(kb + r) * ld + koff + c)
                         : *reinterpret_cast<const uint4*>(ck + (((size_t)seg_slot * size + kb + r) * G + g) * D + c);
        *reinterpret_cast<uint4*>(sK + r * QP + c) = val;
      }
      for (int v = tid; v < 64 * (DV / 8); v += 128) {
        const int r = v % 64, c = (v / 64) * 8;   // consecutive threads take consecutive keys: conflict-free transposed stores
        uint4 val = make_uint4(0, 0, 0, 0);
        if (kb + r < kb1)
          val = src == 0 ? *reinterpret_cast<const uint4*>(qkv + (size_t)(kb + r) * ld + voff + c)
                         : *reinterpret_cast<const uint4*>(cv + (((size_t)seg_slot * size + kb + r) * G + g) * DV + c);
        const bf16* e = reinterpret_cast<const bf16*>(&val);
#pragma unroll
        for (int x = 0; x < 8; ++x) sVt[(c + x) * VP + r] = e[x];
      }
      __syncthreads();
      float sacc[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const bf16* kp = sK + (nt * 8 + gid) * QP + ks * 16 + tig * 2;
          mma_bf16_16816(sacc[nt], qf[ks], *reinterpret_cast<const uint32_t*>(kp), *reinterpret_cast<const uint32_t*>(kp + 8));
        }
      }
      // weights
      bool okA, okB;
      int hiA, hiB, loA, loB;                // visible key range of the two rows in this source's index space
      if (src == 0) { loA = lbA; hiA = iA; loB = lbB; hiB = iB; okA = iA < ntok; okB = iB < ntok; }
      else {
        okA = s_sb[rowA] == seg_sb && s_nc[rowA] > 0; okB = s_sb[rowB] == seg_sb && s_nc[rowB] > 0;
        loA = loB = 0; hiA = s_nc[rowA] - 1; hiB = s_nc[rowB] - 1;
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = kb + nt * 8 + tig * 2 + (e & 1);
          const bool vis = e < 2 ? (okA && j >= loA && j <= hiA) : (okB && j >= loB && j <= hiB);
          sacc[nt][e] = vis ? capped_sigmoid_fast(sacc[nt][e], scale, softcap, b) : 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t ah[4], al[4];
        split_bf2(sacc[2 * j][0], sacc[2 * j][1], ah[0], al[0]);
        split_bf2(sacc[2 * j][2], sacc[2 * j][3], ah[1], al[1]);
        split_bf2(sacc[2 * j + 1][0], sacc[2 * j + 1][1], ah[2], al[2]);
        split_bf2(sacc[2 * j + 1][2], sacc[2 * j + 1][3], ah[3], al[3]);
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
          const bf16* vp = sVt + (nt * 8 + gid) * VP + j * 16 + tig * 2;
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(vp), b1 = *reinterpret_cast<const uint32_t*>(vp + 8);
          mma_bf16_16816(oacc[nt], ah, b0, b1);
          mma_bf16_16816(oacc[nt], al, b0, b1);
        }
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < DV / 8; ++nt) {
    const int c = h * DV + nt * 8 + tig * 2;
    if (iA < ntok) *reinterpret_cast<uint32_t*>(out + (size_t)iA * H * DV + c) = pack_bf2(oacc[nt][0], oacc[nt][1]);
    if (iB < ntok) *reinterpret_cast<uint32_t*>(out + (size_t)iB * H * DV + c) = pack_bf2(oacc[nt][2], oacc[nt][3]);
  }
}

template <int D, int DV>
static int launch_attn_mma(const void* qkv, int ld, const void* ck, const void* cv, const float* bias, void* out, const int* meta,
                           int ntok, int H, int G, int size, float scale, float softcap, cudaStream_t st) {
  constexpr size_t smem = (size_t)(2 * 64 * (D + 8) + DV * 72) * sizeof(bf16) + 5 * 64 * sizeof(int);
  static bool configured = false;
  if (!configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(chunk_attn_mma_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  launch_pdl(chunk_attn_mma_kernel<D, DV>, dim3((ntok + 63) / 64, H), dim3(128), smem, st, (const bf16*)qkv, ld, (const bf16*)ck,
             (const bf16*)cv, bias, (bf16*)out, meta, ntok, H, G, size, scale, softcap);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

// ---------------------------------------------------------------------------------------------------------------------
// Attention for decode-shaped batches on the tensor cores. One CTA (4 warps) per (token, key/value head), optionally a
// cluster of CTAs per token; the rows of every product are the H/G query heads that share the key/value head (up to 16).
// A warp takes steps of 16 keys, the next step's rows in flight while it multiplies the current one: K and V rows go from
// global memory straight into the mma.sync fragments with 16-byte loads -- no shared memory, no transposes -- because
// both sums are free in the order of their terms:
//  * q.k: the 8 consecutive elements a thread loads of key n (d = 32 j + 8 tig + 0..7) serve as the B fragments of two
//    k-steps; the query fragments are read from shared memory through the same permutation of d;
//  * weights.v: a thread loads, for its four keys of a step, elements d = 64 s + 8 gid + 0..7; element t of the four
//    vectors forms the B fragment of output tile t, whose column `gid` therefore stands for d = 64 s + 8 gid + t.
// Weights are float32 and enter the second product as a two-term bfloat16 split. Partial sums of the warps are added
// through shared memory, those of the cluster's CTAs through distributed shared memory, both in a fixed order.
// ---------------------------------------------------------------------------------------------------------------------
template <int D, int DV>
__global__ void __launch_bounds__(128, 2)
chunk_attn_token_mma_kernel(const bf16* __restrict__ qkv, int ld, const bf16* __restrict__ ck, const bf16* __restrict__ cv,
                            const float* __restrict__ bias, bf16* __restrict__ out, const int* __restrict__ meta, int ntok, int H,
                            int G, int size, float scale, float softcap, int nsplit) {
  pdl_enter();
  constexpr int QS = D / 2 + 4;                           // words per query row in shared memory
  extern __shared__ __align__(16) unsigned char tk_raw[];
  const int rep = H / G;
  uint32_t* sQ = reinterpret_cast<uint32_t*>(tk_raw);     // [16][QS], rows >= rep zero
  float* sO = reinterpret_cast<float*>(sQ + 16 * QS);     // [4 warps][rep][DV]
  float* sP = sO + 4 * rep * DV;                          // [rep][DV]: this CTA's partial sums (clusters only)
  const int i = blockIdx.x, g = blockIdx.y, rank = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
  const int slot = meta[i], pos = meta[ntok + i], sb = meta[2 * ntok + i];
  const int pos_start = pos - (i - sb);
  const int lo = (pos / size) * size;
  const int nkeys = pos - lo + 1;
  const int koff = H * D + g * D, voff = H * D + G * D + g * DV;
  for (int c = tid; c < 16 * (D / 2); c += 128) {
    const int row = c / (D / 2), w = c - row * (D / 2);
    sQ[row * QS + w] = row < rep ? reinterpret_cast<const uint32_t*>(qkv + (size_t)i * ld + (size_t)(g * rep + row) * D)[w] : 0u;
  }
  __syncthreads();
  const float bias0 = gid < rep ? bias[g * rep + gid] : 0.f, bias1 = gid + 8 < rep ? bias[g * rep + gid + 8] : 0.f;
  float o[DV / 8][4];
#pragma unroll
  for (int t = 0; t < DV / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  // The warp's steps of 16 keys (step hb covers keys 16 hb ..): the rows of the next step are in flight while the current
  // one is multiplied. k[nt][j]: key 16 hb + 8 nt + gid, elements 32 j + 8 tig ..; v[q][sp]: key 16 hb + 2 tig + (q & 1) +
  // 8 (q >> 1), elements 64 sp + 8 gid ..
  struct Rows { uint4 k[2][D / 32]; uint4 v[4][DV / 64]; };
  auto fetch = [&](int hb, Rows& r) {
    const int kb = hb * 16;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int jj = kb + 8 * nt + gid;
      const bool ok = jj < nkeys;
      const int pj = lo + jj;
      const bf16* kp = (ok && pj >= pos_start) ? qkv + (size_t)(sb + pj - pos_start) * ld + koff
                                               : ck + (((size_t)slot * size + (ok ? jj : 0)) * G + g) * D;
#pragma unroll
      for (int j = 0; j < D / 32; ++j) r.k[nt][j] = ok ? __ldg(reinterpret_cast<const uint4*>(kp + 32 * j + 8 * tig)) : zero4;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int jj = kb + 2 * tig + (q & 1) + 8 * (q >> 1);
      const bool ok = jj < nkeys;
      const int pj = lo + jj;
      const bf16* vp = (ok && pj >= pos_start) ? qkv + (size_t)(sb + pj - pos_start) * ld + voff
                                               : cv + (((size_t)slot * size + (ok ? jj : 0)) * G + g) * DV;
#pragma unroll
      for (int sp = 0; sp < DV / 64; ++sp) r.v[q][sp] = ok ? __ldg(reinterpret_cast<const uint4*>(vp + 64 * sp + 8 * gid)) : zero4;
    }
  };
  const int hstep = 4 * nsplit;
  Rows cur, nxt;
  int hb = rank * 4 + warp;
  if (hb * 16 < nkeys) fetch(hb, cur);
  for (; hb * 16 < nkeys; hb += hstep) {
    const int kb = hb * 16;
    if ((hb + hstep) * 16 < nkeys) fetch(hb + hstep, nxt);
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int j = 0; j < D / 32; ++j)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int wq = 16 * j + 4 * tig + 2 * half;
        const uint32_t a[4] = {sQ[gid * QS + wq], sQ[(gid + 8) * QS + wq], sQ[gid * QS + wq + 1], sQ[(gid + 8) * QS + wq + 1]};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
          mma_bf16_16816(s[nt], a, half ? cur.k[nt][j].z : cur.k[nt][j].x, half ? cur.k[nt][j].w : cur.k[nt][j].y);
      }
    float w[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int row = gid + 8 * (c >> 1), key = kb + 8 * nt + 2 * tig + (c & 1);
        w[nt][c] = (row < rep && key < nkeys) ? capped_sigmoid_fast(s[nt][c], scale, softcap, (c >> 1) ? bias1 : bias0) : 0.f;
      }
    uint32_t ah[4], al[4];
    split_bf2(w[0][0], w[0][1], ah[0], al[0]);
    split_bf2(w[0][2], w[0][3], ah[1], al[1]);
    split_bf2(w[1][0], w[1][1], ah[2], al[2]);
    split_bf2(w[1][2], w[1][3], ah[3], al[3]);
#pragma unroll
    for (int sp = 0; sp < DV / 64; ++sp) {
      const uint32_t v0[4] = {cur.v[0][sp].x, cur.v[0][sp].y, cur.v[0][sp].z, cur.v[0][sp].w};
      const uint32_t v1[4] = {cur.v[1][sp].x, cur.v[1][sp].y, cur.v[1][sp].z, cur.v[1][sp].w};
      const uint32_t v2[4] = {cur.v[2][sp].x, cur.v[2][sp].y, cur.v[2][sp].z, cur.v[2][sp].w};
      const uint32_t v3[4] = {cur.v[3][sp].x, cur.v[3][sp].y, cur.v[3][sp].z, cur.v[3][sp].w};
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const uint32_t sel = (t & 1) ? 0x7632u : 0x5410u;
        const uint32_t b0 = __byte_perm(v0[t >> 1], v1[t >> 1], sel), b1 = __byte_perm(v2[t >> 1], v3[t >> 1], sel);
        mma_bf16_16816(o[sp * 8 + t], ah, b0, b1);
        mma_bf16_16816(o[sp * 8 + t], al, b0, b1);
      }
    }
    cur = nxt;
  }
  // this warp's sums: tile (sp, t), register c -> row gid + 8 (c >> 1), d = 64 sp + 8 (2 tig + (c & 1)) + t
#pragma unroll
  for (int sp = 0; sp < DV / 64; ++sp)
#pragma unroll
    for (int t = 0; t < 8; ++t)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int row = gid + 8 * (c >> 1);
        if (row < rep) sO[(warp * rep + row) * DV + 64 * sp + 8 * (2 * tig + (c & 1)) + t] = o[sp * 8 + t][c];
      }
  __syncthreads();
  const int nout = rep * DV;
  uint32_t* op = reinterpret_cast<uint32_t*>(out + (size_t)i * H * DV + (size_t)g * rep * DV);
  for (int e = 2 * tid; e < nout; e += 256) {
    const float a0 = ((sO[e] + sO[nout + e]) + sO[2 * nout + e]) + sO[3 * nout + e];
    const float a1 = ((sO[e + 1] + sO[nout + e + 1]) + sO[2 * nout + e + 1]) + sO[3 * nout + e + 1];
    if (nsplit == 1) op[e >> 1] = pack_bf2(a0, a1);
    else { sP[e] = a0; sP[e + 1] = a1; }
  }
  if (nsplit == 1) return;
  cluster_sync_all();
  const int words = nout >> 1, per = (words + nsplit - 1) / nsplit;
  const int w_end = min(words, (rank + 1) * per);
  const uint32_t sp_addr = (uint32_t)__cvta_generic_to_shared(sP);
  for (int wd = rank * per + tid; wd < w_end; wd += 128) {
    float a0 = 0.f, a1 = 0.f;
    for (int r = 0; r < nsplit; ++r) {
      const uint32_t ra = mapa_shared(sp_addr + 8u * (uint32_t)wd, (uint32_t)r);
      a0 += __uint_as_float(ld_dsmem_u32(ra));
      a1 += __uint_as_float(ld_dsmem_u32(ra + 4));
    }
    op[wd] = pack_bf2(a0, a1);
  }
  cluster_sync_all();                          // nobody leaves while its partial sums may still be read
}

template <int D, int DV>
static int launch_attn_token_mma(const void* qkv, int ld, const void* ck, const void* cv, const float* bias, void* out, const int* meta,
                                 int ntok, int H, int G, int size, float scale, float softcap, int max_keys, cudaStream_t st) {
  const int rep = H / G;
  const int blocks = ((max_keys > 0 ? min(max_keys, size) : size) + 31) / 32;
  // A cluster per token only while the grid would otherwise leave SMs empty: at 256 and 512 CTAs (64 tokens x 4 and 8
  // key/value heads, 544 and 1056 keys) every doubling of the CTAs made the kernel slower (32 / 42 / 58 / 82 us and
  // 105 / 125 / 157 / 233 us for 1 / 2 / 4 / 8 CTAs per token) -- the fixed chain of a CTA (table, queries, first keys,
  // the sums at the end) is what a short kernel pays for, not the blocks of one warp.
  int nsplit = 1;
  while (nsplit < 8 && 4 * nsplit < blocks && (long long)ntok * G * nsplit * 2 <= 296) nsplit *= 2;
  const size_t smem = (size_t)16 * (D / 2 + 4) * 4 + (size_t)(4 + (nsplit > 1 ? 1 : 0)) * rep * DV * sizeof(float);
  static size_t configured = 0;                          // per instantiation
  if (smem > 48 * 1024 && smem > configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(chunk_attn_token_mma_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
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
  QSPEC_CUDA(cudaLaunchKernelEx(&cfg, chunk_attn_token_mma_kernel<D, DV>, (const bf16*)qkv, ld, (const bf16*)ck, (const bf16*)cv, bias,
                                (bf16*)out, meta, ntok, H, G, size, scale, softcap, nsplit));
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

// Entry for qspec_seq_chunk_attention (seq_kernels.cu): returns -1 when the shape is not one this form takes.
int chunk_attention_token_mma(const void* qkv, int ld, const void* ck, const void* cv, const float* bias, void* out, const int* meta,
                              int ntok, int H, int G, int D, int DV, int size, float scale, float softcap, int max_keys,
                              cudaStream_t st) {
  const bool ok = H % G == 0 && H / G <= 16 && (D == 64 || D == 128) && (DV == 64 || DV == 128) && ld % 8 == 0 &&
                  (((uintptr_t)qkv | (uintptr_t)ck | (uintptr_t)cv | (uintptr_t)out) & 15) == 0;
  if (!ok) return -1;
  if (D == 64 && DV == 64) return launch_attn_token_mma<64, 64>(qkv, ld, ck, cv, bias, out, meta, ntok, H, G, size, scale, softcap, max_keys, st);
  if (D == 64) return launch_attn_token_mma<64, 128>(qkv, ld, ck, cv, bias, out, meta, ntok, H, G, size, scale, softcap, max_keys, st);
  if (DV == 64) return launch_attn_token_mma<128, 64>(qkv, ld, ck, cv, bias, out, meta, ntok, H, G, size, scale, softcap, max_keys, st);
  return launch_attn_token_mma<128, 128>(qkv, ld, ck, cv, bias, out, meta, ntok, H, G, size, scale, softcap, max_keys, st);
}

// ---------------------------------------------------------------------------------------------------------------------
// Grouped expert feed-forward. (1) moe_group_kernel sorts the (token, choice) pairs by expert and lists the 128-row tiles;
// (2) grouped_gemm_kernel<true>: [gate ; up] products of the gathered token rows, clamped-gated activation, Y rows in
// sorted order; (3) grouped_gemm_kernel<false>: down products, rows scattered back to out[token, choice]. Pairs whose
// choice is an identity expert are copied by moe_identity_kernel.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int GG_BM = 128, GG_BK = 64, GG_KP = GG_BK + 8, GG_STAGES = 3;   // rows per expert tile, k-step, padded smem row, ring depth
constexpr size_t GG_SMEM = (size_t)GG_STAGES * 2 * 128 * GG_KP * sizeof(__nv_bfloat16);

struct GroupPlan {
  int* offsets;      // [E + 1] first sorted row of every expert
  int* status;       // [1] status word at the start of the workspace: set to 1 by a CTA whose bounded wait ran out, never cleared
  int* ntiles;       // [1]
  int* tile_expert;  // [max tiles]
  int* tile_row0;    // [max tiles]
  int* perm;         // [npairs] sorted row -> pair index
};

__global__ void __launch_bounds__(1024) moe_group_kernel(const int* __restrict__ idx, int npairs, int E, GroupPlan p) {
  pdl_enter();
  extern __shared__ int s_cnt[];          // [E + 1]
  const int tid = threadIdx.x;
  for (int e = tid; e <= E; e += 1024) s_cnt[e] = 0;
  __syncthreads();
  for (int k = tid; k < npairs; k += 1024) {
    const int e = idx[k];
    if (e >= 0 && e < E) atomicAdd(&s_cnt[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int at = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      const int c = s_cnt[e];
      p.offsets[e] = at;
      for (int r = 0; r < c; r += GG_BM) { p.tile_expert[nt] = e; p.tile_row0[nt] = at + r; ++nt; }
      s_cnt[e] = at;                      // becomes the cursor
      at += c;
    }
    p.offsets[E] = at;
    *p.ntiles = nt;
  }
  __syncthreads();
  for (int k = tid; k < npairs; k += 1024) {
    const int e = idx[k];
    if (e >= 0 && e < E) p.perm[atomicAdd(&s_cnt[e], 1)] = k;
  }
}

__global__ void __launch_bounds__(128) moe_identity_kernel(const bf16* __restrict__ h, const int* __restrict__ idx, bf16* __restrict__ out,
                                                           int W, int E, int top) {
  pdl_enter();
  const int k = blockIdx.x;
  const int e = idx[k];
  if (e >= 0 && e < E) return;
  const bf16* src = h + (size_t)(k / top) * W;
  bf16* dst = out + (size_t)k * W;
  for (int c = threadIdx.x; c < W; c += 128) dst[c] = src[c];
}

// C[m, n] = sum_k A[row(m), k] * B_e[n, k] over the rows of one expert tile. 128 rows x 128 B-rows per CTA, k-steps of
// 64 through a three-stage cp.async ring, 8 warps as 2 (rows) x 4 (columns), fragments by ldmatrix. DUAL: the 128 B-rows are
// 64 gate rows and the 64 up rows of the same columns, every warp holds both for its 16 columns, and the epilogue applies
// the clamped-gated activation; otherwise 128 consecutive output columns.

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;                         // 0: the 16 bytes are zero-filled, the source is not read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

template <bool DUAL>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B, bf16* __restrict__ C, GroupPlan p, int K, int N, int top,
                    float limit) {
  pdl_enter();
  extern __shared__ __align__(16) unsigned char gg_smem[];
  bf16 (*sA)[GG_BM * GG_KP] = reinterpret_cast<bf16 (*)[GG_BM * GG_KP]>(gg_smem);
  bf16 (*sB)[128 * GG_KP] = reinterpret_cast<bf16 (*)[128 * GG_KP]>(gg_smem + (size_t)GG_STAGES * GG_BM * GG_KP * sizeof(bf16));
  __shared__ int s_row[GG_BM];
  const int tile = blockIdx.x;
  if (tile >= *p.ntiles) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
  const int wm = warp >> 2, wn = warp & 3;
  const int e = p.tile_expert[tile], m0 = p.tile_row0[tile];
  const int mend = p.offsets[e + 1];
  constexpr int BN = DUAL ? 64 : 128;                    // output columns per CTA
  const int n0 = blockIdx.y * BN;
  if (tid < GG_BM) {
    const int m = m0 + tid;
    s_row[tid] = m < mend ? p.perm[m] : -1;
  }
  __syncthreads();
  const bf16* Be = B + (size_t)e * (DUAL ? 2 : 1) * N * K;
  // this thread's four A vectors and four B vectors of a stage
  constexpr int NV = GG_BM * (GG_BK / 8) / 256, VPR = GG_BK / 8;
  const bf16* a_src[NV];
  const bf16* b_src[NV];
  bool a_ok[NV], b_ok[NV];
  int a_dst[NV], b_dst[NV];
#pragma unroll
  for (int q = 0; q < NV; ++q) {
    const int v = tid + q * 256, r = v / VPR, c = (v % VPR) * 8;
    const int pr = s_row[r];
    a_ok[q] = pr >= 0;
    a_src[q] = (DUAL ? A + (size_t)(pr < 0 ? 0 : pr / top) * K : A + (size_t)(m0 + r) * K) + c;
    if (!a_ok[q]) a_src[q] = A;
    a_dst[q] = r * GG_KP + c;
    int brow;                                            // row of B_e this smem row holds
    if (DUAL) brow = (r < 64 ? 0 : N) + n0 + (r & 63);
    else brow = n0 + r;
    b_ok[q] = (DUAL ? n0 + (r & 63) : n0 + r) < N;
    b_src[q] = b_ok[q] ? Be + (size_t)brow * K + c : Be;
    b_dst[q] = r * GG_KP + c;
  }
  auto issue = [&](int stage, int k0) {
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      const bool in_k = k0 + (((tid + q * 256) % VPR) * 8) < K;
      cp_async16(&sA[stage][a_dst[q]], a_src[q] + ((a_ok[q] && in_k) ? k0 : 0), a_ok[q] && in_k);
      cp_async16(&sB[stage][b_dst[q]], b_src[q] + ((b_ok[q] && in_k) ? k0 : 0), b_ok[q] && in_k);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  float acc[4][4][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;
  // B rows of this warp's four n-tiles (pairs of tiles are 16 consecutive rows)
  const int brow0 = DUAL ? 16 * wn : 32 * wn;            // tiles 0, 1
  const int brow1 = DUAL ? 64 + 16 * wn : 32 * wn + 16;  // tiles 2, 3
  const int nk = (K + GG_BK - 1) / GG_BK;
  // ring: stage kt lives in slot kt % 3; two stages are in flight while one is multiplied. Past the end of K the copies
  // are zero-size (nothing is read), so every iteration commits exactly one group and the wait count stays fixed.
  issue(0, 0);
  issue(1, GG_BK);
  for (int kt = 0; kt < nk; ++kt) {
    const int st = kt % GG_STAGES;
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    __syncthreads();                                     // stage kt has landed for everyone; slot (kt + 2) % 3 is free
    issue((kt + 2) % GG_STAGES, (kt + 2) * GG_BK);
#pragma unroll
    for (int ks = 0; ks < GG_BK / 16; ++ks) {
      uint32_t bfr[2][4];
      const int brl = (lane & 7) + ((lane >> 4) << 3), bcl = ks * 16 + ((lane >> 3) & 1) * 8;
      ldmatrix_x4(bfr[0], &sB[st][(brow0 + brl) * GG_KP + bcl]);
      ldmatrix_x4(bfr[1], &sB[st][(brow1 + brl) * GG_KP + bcl]);
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        uint32_t af[4];
        ldmatrix_x4(af, &sA[st][(wm * 64 + mt * 16 + (lane & 15)) * GG_KP + ks * 16 + (lane >> 4) * 8]);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) mma_bf16_16816(acc[mt][nt], af, bfr[nt >> 1][(nt & 1) * 2], bfr[nt >> 1][(nt & 1) * 2 + 1]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 64 + mt * 16 + gid + half * 8;
      const int pr = s_row[r];
      if (pr < 0) continue;
      bf16* crow = DUAL ? C + (size_t)(m0 + r) * N : C + (size_t)pr * N;
      if (DUAL) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int n = n0 + 16 * wn + nt * 8 + tig * 2;
          float v[2];
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            // projections leave the matrix unit in bfloat16, like the dense layers' products
            const float gq = fminf(__bfloat162float(__float2bfloat16_rn(acc[mt][nt][half * 2 + x])), limit);
            const float uq = fminf(fmaxf(__bfloat162float(__float2bfloat16_rn(acc[mt][nt + 2][half * 2 + x])), -limit), limit);
            v[x] = gq * (1.0f / (1.0f + expf(-1.702f * gq))) * (uq + 1.0f);
          }
          if (n + 1 < N) *reinterpret_cast<uint32_t*>(crow + n) = pack_bf2(v[0], v[1]);
          else if (n < N) crow[n] = __float2bfloat16_rn(v[0]);
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int n = n0 + 32 * wn + nt * 8 + tig * 2;
          if (n + 1 < N) *reinterpret_cast<uint32_t*>(crow + n) = pack_bf2(acc[mt][nt][half * 2], acc[mt][nt][half * 2 + 1]);
          else if (n < N) crow[n] = __float2bfloat16_rn(acc[mt][nt][half * 2]);
        }
      }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// The same product on the fifth-generation tensor cores. One CTA = 128 rows of one expert x 128 B-rows, accumulator
// [128 lanes x 128 columns] float32 in tensor memory. A and B k-steps of 64 (128 bytes per row) land in shared memory
// through the same gathering cp.async ring, laid out as the K-major 128-byte-swizzle operand layout (row r at r * 128
// bytes, 16-byte chunk c at position c ^ (r & 7); 8-row groups 1024 bytes apart), so that one elected thread multiplies a
// stage with four tcgen05.mma (M 128, N 128, K 16) whose completion (tcgen05.commit on an mbarrier) frees the slot.
// Every wait is bounded: a barrier that does not complete raises the plan's error word, and the CTA drains its copies,
// frees its tensor memory and leaves without storing.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int TC_STAGES = 3;                                               // 97 KB: two CTAs per SM
constexpr int TC_TILE_BYTES = 128 * 128;                                   // 128 rows x 64 bf16
constexpr size_t TC_SMEM = (size_t)TC_STAGES * 2 * TC_TILE_BYTES + 1024;   // + slack to start on a 1024-byte boundary
constexpr uint32_t TC_COLS = 128;                                          // tensor-memory columns of the accumulator

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t spins = 0; spins < (1u << 20); ++spins) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ bool tc_elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n" : "=r"(pred));
  return pred != 0;
}
// K-major, 128-byte swizzle: start >> 4 at [0,14), stride between 8-row groups (1024 B) >> 4 at [32,46), version 1 at
// [46,48), layout 2 at [61,64). 32 bytes further along K = + 2 in the start field.
__device__ __forceinline__ uint64_t tc_desc_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// float32 accumulator [4,6) = 1, bfloat16 A [7,10) = 1 and B [10,13) = 1, both K-major, N >> 3 at [17,23), M >> 4 at [24,29)
constexpr uint32_t TC_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(TC_IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// MODE 0: down product (rows in sorted order, output scattered to [token, choice]); 1: [gate ; up] product with the clamped
// gated activation; 2: up product alone with the squared-ReLU activation (rows gathered, output in sorted order).
template <int MODE>
__global__ void __launch_bounds__(256)
grouped_gemm_tc_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B, bf16* __restrict__ C, GroupPlan p, int K, int N, int top,
                       float limit, int act) {
  pdl_enter();
  extern __shared__ __align__(16) unsigned char tc_smem_raw[];
  __shared__ int s_row[GG_BM];
  __shared__ __align__(8) uint64_t s_bar[TC_STAGES];
  __shared__ uint32_t s_tmem;
  __shared__ volatile int s_fail;
  const int tile = blockIdx.x;
  if (tile >= *p.ntiles) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t base = (tc_smem_u32(tc_smem_raw) + 1023u) & ~1023u;      // stage s: A at base + s * 32 KB, B 16 KB after it
  const int e = p.tile_expert[tile], m0 = p.tile_row0[tile];
  const int mend = p.offsets[e + 1];
  constexpr bool DUAL = MODE == 1, GATHER = MODE != 0;
  constexpr int BN = DUAL ? 64 : 128;                    // output columns per CTA
  const int n0 = blockIdx.y * BN;
  if (tid < GG_BM) {
    const int m = m0 + tid;
    s_row[tid] = m < mend ? p.perm[m] : -1;
  }
  if (tid == 0) {
    for (int s = 0; s < TC_STAGES; ++s) tc_mbar_init(tc_smem_u32(&s_bar[s]), 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem_u32(&s_tmem)), "r"(TC_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem = s_tmem;
  const bf16* Be = B + (size_t)e * (DUAL ? 2 : 1) * N * K;
  constexpr int NV = GG_BM * (GG_BK / 8) / 256, VPR = GG_BK / 8;        // 4 vectors of A and 4 of B per thread and stage
  const bf16* a_src[NV];
  const bf16* b_src[NV];
  bool a_ok[NV], b_ok[NV];
  uint32_t dst[NV];
#pragma unroll
  for (int q = 0; q < NV; ++q) {
    const int v = tid + q * 256, r = v / VPR, c8 = v % VPR;
    const int pr = s_row[r];
    a_ok[q] = pr >= 0;
    a_src[q] = a_ok[q] ? (GATHER ? A + (size_t)(pr / top) * K : A + (size_t)(m0 + r) * K) + c8 * 8 : A;
    int brow;
    if (DUAL) brow = (r < 64 ? 0 : N) + n0 + (r & 63);
    else brow = n0 + r;
    b_ok[q] = (DUAL ? n0 + (r & 63) : n0 + r) < N;
    b_src[q] = b_ok[q] ? Be + (size_t)brow * K + c8 * 8 : Be;
    dst[q] = (uint32_t)(r * 128 + ((c8 ^ (r & 7)) << 4));
  }
  auto issue = [&](int stage, int k0) {
    const uint32_t sa = base + (uint32_t)stage * (2 * TC_TILE_BYTES), sb = sa + TC_TILE_BYTES;
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      const bool in_k = k0 + (((tid + q * 256) % VPR) * 8) < K;
      const int na = (a_ok[q] && in_k) ? 16 : 0, nb = (b_ok[q] && in_k) ? 16 : 0;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(sa + dst[q]), "l"(a_src[q] + (na ? k0 : 0)), "r"(na) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(sb + dst[q]), "l"(b_src[q] + (nb ? k0 : 0)), "r"(nb) : "memory");
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  const int nk = (K + GG_BK - 1) / GG_BK;
  // ring: k-step kt lives in slot kt % TC_STAGES; TC_STAGES - 1 steps are in flight while one is multiplied. Past the end
  // of K the copies are zero-size, so that every iteration commits exactly one group and the wait count stays fixed.
#pragma unroll
  for (int s = 0; s < TC_STAGES - 1; ++s) issue(s, s * GG_BK);
  for (int kt = 0; kt < nk; ++kt) {
    const int st = kt % TC_STAGES;
    asm volatile("cp.async.wait_group %0;\n" ::"n"(TC_STAGES - 2) : "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");     // this thread's rows, for the tensor cores' reads
    __syncthreads();                                                    // k-step kt has landed for everyone
    if (s_fail) break;                                                  // written before the barrier: uniform
    if (warp == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      if (tc_elect_one()) {
        const uint64_t ad = tc_desc_sw128(base + (uint32_t)st * (2 * TC_TILE_BYTES));
        const uint64_t bd = tc_desc_sw128(base + (uint32_t)st * (2 * TC_TILE_BYTES) + TC_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < GG_BK / 16; ++ks) tc_mma_ss(tmem, ad + 2 * ks, bd + 2 * ks, (kt | ks) ? 1u : 0u);
        tc_commit(tc_smem_u32(&s_bar[st]));
      }
      __syncwarp();
    }
    // slot (kt - 1) % TC_STAGES is refilled next: the products of k-step kt - 1 must have read it
    if (kt >= 1 && !tc_mbar_wait(tc_smem_u32(&s_bar[(kt - 1) % TC_STAGES]), (uint32_t)(((kt - 1) / TC_STAGES) & 1))) s_fail = 1;
    issue((kt + TC_STAGES - 1) % TC_STAGES, (kt + TC_STAGES - 1) * GG_BK);
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  if (!s_fail && !tc_mbar_wait(tc_smem_u32(&s_bar[(nk - 1) % TC_STAGES]), (uint32_t)(((nk - 1) / TC_STAGES) & 1))) s_fail = 1;
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  if (s_fail) {
    if (tid == 0) atomicExch(p.status, 1);
  } else {
    // warp w reads lanes 32 * (w & 3) .. + 31 (rows of the tile); the two warps of a lane quarter split the columns
    const int r = (warp & 3) * 32 + lane, half = warp >> 2;
    const int pr = s_row[r];
    const uint32_t trow = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    bf16* crow = GATHER ? C + (size_t)(m0 + r) * N : C + (size_t)(pr < 0 ? 0 : pr) * N;
    constexpr int GROUPS = DUAL ? 2 : 4;                 // groups of 16 output columns per warp
#pragma unroll
    for (int gq = 0; gq < GROUPS; ++gq) {
      const int col = half * (GROUPS * 16) + gq * 16;    // output column inside the CTA's BN
      uint32_t a[16], b[16];
      tc_ld16(trow + (uint32_t)col, a);
      if (DUAL) tc_ld16(trow + (uint32_t)(64 + col), b);
      tc_wait_ld();
      float v[16];
#pragma unroll
      for (int x = 0; x < 16; ++x) {
        if (DUAL) {
          // projections leave the matrix unit in bfloat16, like the dense layers' products
          if (act == QSPEC_EXPERT_ACT_SILU) {
            const float gv = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[x])));
            const float uv = __bfloat162float(__float2bfloat16_rn(__uint_as_float(b[x])));
            v[x] = gv / (1.0f + expf(-gv)) * uv;
          } else {
            const float gv = fminf(__bfloat162float(__float2bfloat16_rn(__uint_as_float(a[x]))), limit);
            const float uv = fminf(fmaxf(__bfloat162float(__float2bfloat16_rn(__uint_as_float(b[x]))), -limit), limit);
            v[x] = gv * (1.0f / (1.0f + expf(-1.702f * gv))) * (uv + 1.0f);
          }
        } else if (MODE == 2) {
          const float u = fmaxf(__bfloat162float(__float2bfloat16_rn(__uint_as_float(a[x]))), 0.f);
          v[x] = u * u;
        } else {
          v[x] = __uint_as_float(a[x]);
        }
      }
      const int n = n0 + col;
      if (pr >= 0) {
        if (n + 16 <= N) {
          uint4 w0, w1;
          w0.x = pack_bf2(v[0], v[1]); w0.y = pack_bf2(v[2], v[3]); w0.z = pack_bf2(v[4], v[5]); w0.w = pack_bf2(v[6], v[7]);
          w1.x = pack_bf2(v[8], v[9]); w1.y = pack_bf2(v[10], v[11]); w1.z = pack_bf2(v[12], v[13]); w1.w = pack_bf2(v[14], v[15]);
          *reinterpret_cast<uint4*>(crow + n) = w0;
          *reinterpret_cast<uint4*>(crow + n + 8) = w1;
        } else {
#pragma unroll
          for (int x = 0; x < 16; ++x)
            if (n + x < N) crow[n + x] = __float2bfloat16_rn(v[x]);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TC_COLS) : "memory");
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace qspec

using namespace qspec;

extern "C" int qspec_seq_chunk_attention_mma_supported(int H, int G, int D, int DV) {
  return H > 0 && G > 0 && H % G == 0 && (D == 64 || D == 128) && (DV == 64 || DV == 128);
}

extern "C" int qspec_seq_chunk_attention_mma(const void* qkv, int ld, const void* cache_k, const void* cache_v, const float* bias,
                                             void* out, const int* meta, int ntok, int H, int G, int D, int DV, int size,
                                             float scale, float softcap, void* stream) {
  QSPEC_REQUIRE(qkv && cache_k && cache_v && bias && out && meta, QSPEC_ERR_INVALID_ARG, "seq_chunk_attention_mma: null pointer");
  QSPEC_REQUIRE(qspec_seq_chunk_attention_mma_supported(H, G, D, DV), QSPEC_ERR_UNSUPPORTED,
                "seq_chunk_attention_mma: head sizes %d / %d (64 or 128 each)", D, DV);
  QSPEC_REQUIRE(ntok >= 0 && size > 0 && ld >= H * D + G * (D + DV) && ld % 8 == 0 && ((uintptr_t)qkv & 15) == 0 &&
                    ((uintptr_t)cache_k & 15) == 0 && ((uintptr_t)cache_v & 15) == 0,
                QSPEC_ERR_UNSUPPORTED, "seq_chunk_attention_mma: rows must be 16-byte aligned (ld %d)", ld);
  if (ntok == 0) return QSPEC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (D == 64 && DV == 64) return launch_attn_mma<64, 64>(qkv, ld, cache_k, cache_v, bias, out, meta, ntok, H, G, size, scale, softcap, st);
  if (D == 64 && DV == 128) return launch_attn_mma<64, 128>(qkv, ld, cache_k, cache_v, bias, out, meta, ntok, H, G, size, scale, softcap, st);
  if (D == 128 && DV == 64) return launch_attn_mma<128, 64>(qkv, ld, cache_k, cache_v, bias, out, meta, ntok, H, G, size, scale, softcap, st);
  return launch_attn_mma<128, 128>(qkv, ld, cache_k, cache_v, bias, out, meta, ntok, H, G, size, scale, softcap, st);
}

extern "C" int qspec_moe_expert_grouped_supported(int W, int F) { return W > 0 && F > 0 && W % 8 == 0 && F % 8 == 0; }

static size_t grouped_layout(int ntok, int top, int E, int F, size_t* off) {
  const size_t npairs = (size_t)ntok * top, max_tiles = npairs / 128 + E + 1;
  size_t at = 0;
  off[1] = at; at = align_up(at + 4, 16);                        // status word (first, wherever the rest lies)
  off[0] = at; at = align_up(at + (size_t)(E + 1) * 4, 16);      // offsets
  off[2] = at; at = align_up(at + 4, 16);                        // ntiles
  off[3] = at; at = align_up(at + max_tiles * 4, 16);            // tile_expert
  off[4] = at; at = align_up(at + max_tiles * 4, 16);            // tile_row0
  off[5] = at; at = align_up(at + npairs * 4, 16);               // perm
  off[6] = at; at = align_up(at + npairs * (size_t)F * 2, 16);   // Y
  return at;
}

extern "C" size_t qspec_moe_grouped_workspace_bytes(int ntok, int top, int E, int F) {
  size_t off[7];
  return grouped_layout(ntok > 0 ? ntok : 0, top, E, F, off);
}

extern "C" int qspec_moe_expert_grouped_act(const void* h, const void* gate_up, const void* down, const int* idx, void* out, int ntok,
                                            int W, int F, int E, int top, float limit, int act, void* workspace,
                                            size_t workspace_bytes, void* stream) {
  QSPEC_REQUIRE(act == QSPEC_EXPERT_ACT_GATED || act == QSPEC_EXPERT_ACT_RELU2 || act == QSPEC_EXPERT_ACT_SILU, QSPEC_ERR_INVALID_ARG,
                "moe_expert_grouped: unknown activation %d", act);
  QSPEC_REQUIRE(h && idx && out && workspace && (E == 0 || (gate_up && down)), QSPEC_ERR_INVALID_ARG, "moe_expert_grouped: null pointer");
  QSPEC_REQUIRE(ntok >= 0 && top >= 1 && E >= 0 && E <= 8192, QSPEC_ERR_INVALID_ARG, "moe_expert_grouped: bad sizes");
  QSPEC_REQUIRE(qspec_moe_expert_grouped_supported(W, F), QSPEC_ERR_UNSUPPORTED,
                "moe_expert_grouped: width %d and expert size %d must be multiples of 8", W, F);
  QSPEC_REQUIRE((((uintptr_t)h | (uintptr_t)gate_up | (uintptr_t)down | (uintptr_t)out | (uintptr_t)workspace) & 15) == 0,
                QSPEC_ERR_UNSUPPORTED, "moe_expert_grouped: pointers must be 16-byte aligned");
  size_t off[7];
  QSPEC_REQUIRE(workspace_bytes >= grouped_layout(ntok, top, E, F, off), QSPEC_ERR_WORKSPACE, "moe_expert_grouped: workspace too small");
  if (ntok == 0) return QSPEC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  unsigned char* ws = (unsigned char*)workspace;
  GroupPlan p;
  p.offsets = (int*)(ws + off[0]); p.status = (int*)(ws + off[1]); p.ntiles = (int*)(ws + off[2]);
  p.tile_expert = (int*)(ws + off[3]); p.tile_row0 = (int*)(ws + off[4]); p.perm = (int*)(ws + off[5]);
  bf16* Y = (bf16*)(ws + off[6]);
  const int npairs = ntok * top;
  const int max_tiles = npairs / 128 + E + 1;
  launch_pdl(moe_identity_kernel, dim3(npairs), dim3(128), 0, st, (const bf16*)h, idx, (bf16*)out, W, E, top);
  QSPEC_CHECK_LAUNCH(1);
  if (E == 0) return QSPEC_OK;
  launch_pdl(moe_group_kernel, dim3(1), dim3(1024), (size_t)(E + 1) * sizeof(int), st, idx, npairs, E, p);
  QSPEC_CHECK_LAUNCH(1);
  static bool configured = false;
  if (!configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GG_SMEM));
    QSPEC_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GG_SMEM));
    QSPEC_CUDA(cudaFuncSetAttribute(grouped_gemm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM));
    QSPEC_CUDA(cudaFuncSetAttribute(grouped_gemm_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM));
    QSPEC_CUDA(cudaFuncSetAttribute(grouped_gemm_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM));
    configured = true;
  }
  // QSPEC_SEQ_GROUPED=mma selects the warp-level (mma.sync) tiles, kept as the comparison form for timing and tests
  static const bool warp_level = [] { const char* v = getenv("QSPEC_SEQ_GROUPED"); return v && !strcmp(v, "mma"); }();
  QSPEC_REQUIRE(!warp_level || act == QSPEC_EXPERT_ACT_GATED, QSPEC_ERR_UNSUPPORTED,
                "moe_expert_grouped: the warp-level comparison form has the gated activation only");
  if (!warp_level) {
    if (act == QSPEC_EXPERT_ACT_RELU2)
      launch_pdl(grouped_gemm_tc_kernel<2>, dim3(max_tiles, (F + 127) / 128), dim3(256), TC_SMEM, st, (const bf16*)h, (const bf16*)gate_up, Y,
                 p, W, F, top, limit, act);
    else
      launch_pdl(grouped_gemm_tc_kernel<1>, dim3(max_tiles, (F + 63) / 64), dim3(256), TC_SMEM, st, (const bf16*)h, (const bf16*)gate_up, Y,
                 p, W, F, top, limit, act);
    QSPEC_CHECK_LAUNCH(1);
    launch_pdl(grouped_gemm_tc_kernel<0>, dim3(max_tiles, (W + 127) / 128), dim3(256), TC_SMEM, st, (const bf16*)Y, (const bf16*)down,
               (bf16*)out, p, F, W, top, limit, act);
    QSPEC_CHECK_LAUNCH(1);
    return QSPEC_OK;
  }
  launch_pdl(grouped_gemm_kernel<true>, dim3(max_tiles, (F + 63) / 64), dim3(256), GG_SMEM, st, (const bf16*)h, (const bf16*)gate_up, Y, p, W,
             F, top, limit);
  QSPEC_CHECK_LAUNCH(1);
  launch_pdl(grouped_gemm_kernel<false>, dim3(max_tiles, (W + 127) / 128), dim3(256), GG_SMEM, st, (const bf16*)Y, (const bf16*)down, (bf16*)out,
             p, F, W, top, limit);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

extern "C" int qspec_moe_expert_grouped(const void* h, const void* gate_up, const void* down, const int* idx, void* out, int ntok,
                                        int W, int F, int E, int top, float limit, void* workspace, size_t workspace_bytes,
                                        void* stream) {
  return qspec_moe_expert_grouped_act(h, gate_up, down, idx, out, ntok, W, F, E, top, limit, QSPEC_EXPERT_ACT_GATED, workspace,
                                      workspace_bytes, stream);
}

namespace qspec {
// ---------------------------------------------------------------------------------------------------------------------
// Sliding-window softmax attention with a sink on the tensor cores (bfloat16 keys / values in per-slot rings).
// One CTA (4 warps) per block of 16 rows; the rows of both products are either the query heads that share a key/value
// head, for one token (decode-shaped batches), or 16 consecutive batch tokens for one head (prompts). The four warps
// take every fourth step of 16 keys of the visible range, each with its own online softmax (float32 maxima and sums),
// and their partial results are merged in shared memory together with the sink term. As in the token form above, K and
// V rows go from global memory straight into the mma.sync fragments with 16-byte loads (the summation index of both
// products is permuted instead of transposing through shared memory), the next step's rows in flight while the current
// one is multiplied. A key is two parts: [0, DA) from kA (per key/value head) and [DA, DA + DB) from kB (shared by all
// heads: the rotary part of a latent cache). Weights are float32 and enter the second product as a two-term bfloat16
// split. A block of tokens may span several sequences: their key ranges are walked one after the other.
// ---------------------------------------------------------------------------------------------------------------------
struct WinMma {
  const float* q; long long q_ts, q_hs;
  const bf16* kA; long long kA_ss; int kA_rs, kA_hs;
  const bf16* kB; long long kB_ss; int kB_rs;
  const bf16* v; long long v_ss; int v_rs, v_hs;
  const float* sink; const bf16* gate; int gate_ld, gate_per_head;
  bf16* out; int out_hs; const int* meta; int ntok, H, G, window, cap; float scale; int token_rows;
};

// STREAM: key rows are loaded inside the product loop instead of a whole step ahead (long keys: the fragments of a step
// would not fit the register file); blockIdx.z selects a slice of DV value columns (values longer than DV).
template <int DA, int DB, int DV, bool STREAM>
__global__ void __launch_bounds__(128, 2) window_attn_mma_kernel(const WinMma a) {
  pdl_enter();
  constexpr int DK = DA + DB, QS = DK / 2 + 4;
  extern __shared__ __align__(16) unsigned char wm_raw[];
  uint32_t* sQ = reinterpret_cast<uint32_t*>(wm_raw);       // [16][QS]
  float* sO = reinterpret_cast<float*>(sQ + 16 * QS);        // [4 warps][16][DV]
  __shared__ float sM[4][16], sL[4][16];
  __shared__ int s_tok[16], s_head[16], s_pos[16], s_seg[16], s_slot[16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
  const int rep = a.H / a.G;
  const int kvh = a.token_rows ? (int)blockIdx.y / rep : (int)blockIdx.y;
  if (tid < 16) {
    int tok = -1, head = 0;
    if (a.token_rows) { tok = blockIdx.x * 16 + tid; head = blockIdx.y; if (tok >= a.ntok) tok = -1; }
    else if (tid < rep) { tok = blockIdx.x; head = kvh * rep + tid; }
    s_tok[tid] = tok; s_head[tid] = head;
    s_pos[tid] = tok >= 0 ? a.meta[a.ntok + tok] : -1;
    s_seg[tid] = tok >= 0 ? a.meta[2 * a.ntok + tok] : -1;
    s_slot[tid] = tok >= 0 ? a.meta[tok] : 0;
  }
  __syncthreads();
  for (int c = tid; c < 16 * (DK / 2); c += 128) {
    const int row = c / (DK / 2), w = c - row * (DK / 2);
    uint32_t val = 0u;
    if (s_tok[row] >= 0) {
      const float2 f = *reinterpret_cast<const float2*>(a.q + (size_t)s_tok[row] * a.q_ts + (size_t)s_head[row] * a.q_hs + 2 * w);
      val = pack_bf2(f.x, f.y);
    }
    sQ[row * QS + w] = val;
  }
  __syncthreads();
  const int rA = gid, rB = gid + 8;
  const int posA = s_pos[rA], posB = s_pos[rB], segA = s_seg[rA], segB = s_seg[rB];
  float o[DV / 8][4];
#pragma unroll
  for (int t = 0; t < DV / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  struct Rows { uint4 k[2][STREAM ? 1 : DK / 32]; uint4 v[4][DV / 64]; };

  int r0 = 0;
  while (r0 < 16 && s_tok[r0] >= 0) {
    // rows r0 .. r1 - 1 belong to one sequence (token rows), or all rows to the one token (head rows)
    int r1 = r0 + 1;
    while (r1 < 16 && s_tok[r1] >= 0 && s_seg[r1] == s_seg[r0]) ++r1;
    const int seg = s_seg[r0], slot = s_slot[r0];
    const int pmax = a.token_rows ? s_pos[r1 - 1] : s_pos[r0];
    const int jlo = max(0, s_pos[r0] - a.window + 1);
    const int nkeys = pmax - jlo + 1;
    const bf16* kA = a.kA + (size_t)slot * a.kA_ss + (size_t)kvh * a.kA_hs;
    const bf16* kB = DB ? a.kB + (size_t)slot * a.kB_ss : nullptr;
    const bf16* vb = a.v + (size_t)slot * a.v_ss + (size_t)kvh * a.v_hs + (size_t)blockIdx.z * DV;
    auto fetch = [&](int hb, Rows& r) {
      const int kb = hb * 16;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int jj = kb + 8 * nt + gid;
        const bool ok = jj < nkeys;
        const int row = ok ? (jlo + jj) % a.cap : 0;
        const bf16* kp = kA + (size_t)row * a.kA_rs;
#pragma unroll
        for (int j = 0; j < DA / 32; ++j) r.k[nt][j] = ok ? __ldg(reinterpret_cast<const uint4*>(kp + 32 * j + 8 * tig)) : zero4;
        if (DB) {
          const bf16* kq = kB + (size_t)row * a.kB_rs;
#pragma unroll
          for (int j = 0; j < DB / 32; ++j) r.k[nt][DA / 32 + j] = ok ? __ldg(reinterpret_cast<const uint4*>(kq + 32 * j + 8 * tig)) : zero4;
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int jj = kb + 2 * tig + (q & 1) + 8 * (q >> 1);
        const bool ok = jj < nkeys;
        const bf16* vp = vb + (size_t)(ok ? (jlo + jj) % a.cap : 0) * a.v_rs;
#pragma unroll
        for (int sp = 0; sp < DV / 64; ++sp) r.v[q][sp] = ok ? __ldg(reinterpret_cast<const uint4*>(vp + 64 * sp + 8 * gid)) : zero4;
      }
    };
    const bool inA = a.token_rows ? (segA == seg && s_tok[rA] >= 0) : rA < rep;
    const bool inB = a.token_rows ? (segB == seg && s_tok[rB] >= 0) : rB < rep;
    Rows cur, nxt;
    int hb = warp;
    if (!STREAM && hb * 16 < nkeys) fetch(hb, cur);
    for (; hb * 16 < nkeys; hb += 4) {
      const int kb = hb * 16;
      if (!STREAM && (hb + 4) * 16 < nkeys) fetch(hb + 4, nxt);
      float s[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      if (STREAM) {
        const bf16* kp[2];
        const bf16* kq[2];
        bool okk[2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int jj = kb + 8 * nt + gid;
          okk[nt] = jj < nkeys;
          const int row = okk[nt] ? (jlo + jj) % a.cap : 0;
          kp[nt] = kA + (size_t)row * a.kA_rs + 8 * tig;
          kq[nt] = DB ? kB + (size_t)row * a.kB_rs + 8 * tig : nullptr;
        }
#pragma unroll
        for (int j = 0; j < DK / 32; ++j) {
          uint4 kk[2];
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
            kk[nt] = !okk[nt] ? zero4 : __ldg(reinterpret_cast<const uint4*>(j < DA / 32 ? kp[nt] + 32 * j : kq[nt] + 32 * (j - DA / 32)));
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int wq = 16 * j + 4 * tig + 2 * half;
            const uint32_t af[4] = {sQ[gid * QS + wq], sQ[(gid + 8) * QS + wq], sQ[gid * QS + wq + 1], sQ[(gid + 8) * QS + wq + 1]};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) mma_bf16_16816(s[nt], af, half ? kk[nt].z : kk[nt].x, half ? kk[nt].w : kk[nt].y);
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {                       // this step's value rows, in flight during the softmax
          const int jj = kb + 2 * tig + (q & 1) + 8 * (q >> 1);
          const bool ok = jj < nkeys;
          const bf16* vp = vb + (size_t)(ok ? (jlo + jj) % a.cap : 0) * a.v_rs;
#pragma unroll
          for (int sp = 0; sp < DV / 64; ++sp) cur.v[q][sp] = ok ? __ldg(reinterpret_cast<const uint4*>(vp + 64 * sp + 8 * gid)) : zero4;
        }
      } else {
#pragma unroll
        for (int j = 0; j < DK / 32; ++j)
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int wq = 16 * j + 4 * tig + 2 * half;
            const uint32_t af[4] = {sQ[gid * QS + wq], sQ[(gid + 8) * QS + wq], sQ[gid * QS + wq + 1], sQ[(gid + 8) * QS + wq + 1]};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
              mma_bf16_16816(s[nt], af, half ? cur.k[nt][j].z : cur.k[nt][j].x, half ? cur.k[nt][j].w : cur.k[nt][j].y);
          }
      }
      // visible: same sequence, key position <= the row's and within its window
      float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int pj = jlo + kb + 8 * nt + 2 * tig + (c & 1);
          const int pr = (c >> 1) ? posB : posA;
          const bool vis = ((c >> 1) ? inB : inA) && pj <= pr && pr - pj < a.window && pj <= pmax;
          s[nt][c] = vis ? s[nt][c] * a.scale : -INFINITY;
          if (c >> 1) mxB = fmaxf(mxB, s[nt][c]); else mxA = fmaxf(mxA, s[nt][c]);
        }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1)); mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1)); mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);
      const float cA = nA == -INFINITY ? 1.f : __expf(mA - nA), cB = nB == -INFINITY ? 1.f : __expf(mB - nB);
      const float bA = nA == -INFINITY ? 0.f : nA, bB = nB == -INFINITY ? 0.f : nB;
      mA = nA; mB = nB;
      float w[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) w[nt][c] = __expf(s[nt][c] - ((c >> 1) ? bB : bA));      // exp(-inf) = 0 for hidden keys
      lA = lA * cA + (w[0][0] + w[0][1]) + (w[1][0] + w[1][1]);
      lB = lB * cB + (w[0][2] + w[0][3]) + (w[1][2] + w[1][3]);
#pragma unroll
      for (int t = 0; t < DV / 8; ++t) { o[t][0] *= cA; o[t][1] *= cA; o[t][2] *= cB; o[t][3] *= cB; }
      uint32_t ah[4], al[4];
      split_bf2(w[0][0], w[0][1], ah[0], al[0]);
      split_bf2(w[0][2], w[0][3], ah[1], al[1]);
      split_bf2(w[1][0], w[1][1], ah[2], al[2]);
      split_bf2(w[1][2], w[1][3], ah[3], al[3]);
#pragma unroll
      for (int sp = 0; sp < DV / 64; ++sp) {
        const uint32_t v0[4] = {cur.v[0][sp].x, cur.v[0][sp].y, cur.v[0][sp].z, cur.v[0][sp].w};
        const uint32_t v1[4] = {cur.v[1][sp].x, cur.v[1][sp].y, cur.v[1][sp].z, cur.v[1][sp].w};
        const uint32_t v2[4] = {cur.v[2][sp].x, cur.v[2][sp].y, cur.v[2][sp].z, cur.v[2][sp].w};
        const uint32_t v3[4] = {cur.v[3][sp].x, cur.v[3][sp].y, cur.v[3][sp].z, cur.v[3][sp].w};
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const uint32_t sel = (t & 1) ? 0x7632u : 0x5410u;
          const uint32_t b0 = __byte_perm(v0[t >> 1], v1[t >> 1], sel), b1 = __byte_perm(v2[t >> 1], v3[t >> 1], sel);
          mma_bf16_16816(o[sp * 8 + t], ah, b0, b1);
          mma_bf16_16816(o[sp * 8 + t], al, b0, b1);
        }
      }
      if (!STREAM) cur = nxt;
    }
    if (!a.token_rows) break;
    r0 = r1;
  }
  // the warp's sums: each thread holds a quarter of its rows' sums of weights
  lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
  if (tig == 0) { sM[warp][rA] = mA; sL[warp][rA] = lA; sM[warp][rB] = mB; sL[warp][rB] = lB; }
  // tile (sp, t), register c -> row gid + 8 (c >> 1), d = 64 sp + 8 (2 tig + (c & 1)) + t
#pragma unroll
  for (int sp = 0; sp < DV / 64; ++sp)
#pragma unroll
    for (int t = 0; t < 8; ++t)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        sO[(warp * 16 + gid + 8 * (c >> 1)) * DV + 64 * sp + 8 * (2 * tig + (c & 1)) + t] = o[sp * 8 + t][c];
  __syncthreads();
  for (int e = tid; e < 16 * DV; e += 128) {
    const int row = e / DV, d = e - row * DV;
    const int tok = s_tok[row];
    if (tok < 0) continue;
    const int head = s_head[row];
    float M = a.sink ? a.sink[head] : -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sM[w][row]);
    float L = a.sink ? __expf(a.sink[head] - M) : 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = sM[w][row] == -INFINITY ? 0.f : __expf(sM[w][row] - M);
      L += sL[w][row] * f;
      acc += sO[(w * 16 + row) * DV + d] * f;
    }
    float r = acc / L;
    if (a.gate) r *= __fdividef(1.0f, 1.0f + __expf(-__bfloat162float(a.gate[(size_t)tok * a.gate_ld + (a.gate_per_head ? (size_t)head : (size_t)head * a.out_hs + (size_t)blockIdx.z * DV + d)])));
    a.out[((size_t)tok * a.H + head) * a.out_hs + (size_t)blockIdx.z * DV + d] = __float2bfloat16_rn(r);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Absorbed latent attention for decode-shaped batches, CTA-level form: the rows of a latent cache are keys ([latent DA |
// shared rotary part 64]) and values (the latent) at once, and all heads of a token read the same rows. One CTA of 8
// warps per (token, group of up to 16 heads) walks the window in blocks of 64 keys: warp w multiplies the 16 heads'
// queries with keys 8 w .. 8 w + 7 of the block (key rows streamed through the product loop), the block's row maxima meet
// in shared memory (one running maximum per head for the whole CTA), the float32 weights go to shared memory as a
// two-term bfloat16 split, and then warp w adds the block's 64 keys into its own 64 value columns (the rows straight into
// the fragments, as above). The scores are computed once, not once per slice of value columns.
// ---------------------------------------------------------------------------------------------------------------------
template <int DA>
__global__ void __launch_bounds__(256) latent_absorbed_mma_kernel(const WinMma a, int nsplit) {
  pdl_enter();
  constexpr int DB = 64, DK = DA + DB, QS = DK / 2 + 4, NW = 8, PVW = DA / 64, PS = 36;   // PVW warps own 64 value columns each
  extern __shared__ __align__(16) unsigned char la_raw[];
  uint32_t* sQ = reinterpret_cast<uint32_t*>(la_raw);        // [16][QS]
  uint32_t* sPh = sQ + 16 * QS;                               // [16][PS] weights of the block, high terms (64 keys = 32 words)
  uint32_t* sPl = sPh + 16 * PS;                              // low terms
  float* sPart = reinterpret_cast<float*>(sPl + 16 * PS);     // clusters only: [16] maxima | [16] sums | [16][DA] value sums
  const int rank = blockIdx.z;                                // this CTA takes every nsplit-th block of 64 keys
  __shared__ float sMax[NW][16], sL[NW][16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
  const int rep = a.H / a.G, i = blockIdx.x, grp = blockIdx.y;
  const int slot = a.meta[i], pos = a.meta[a.ntok + i];
  for (int c = tid; c < 16 * (DK / 2); c += 256) {
    const int row = c / (DK / 2), w = c - row * (DK / 2);
    uint32_t val = 0u;
    if (row < rep) {
      const float2 f = *reinterpret_cast<const float2*>(a.q + (size_t)i * a.q_ts + (size_t)(grp * rep + row) * a.q_hs + 2 * w);
      val = pack_bf2(f.x, f.y);
    }
    sQ[row * QS + w] = val;
  }
  __syncthreads();
  const int jlo = max(0, pos - a.window + 1), nkeys = pos - jlo + 1;
  const bf16* kA = a.kA + (size_t)slot * a.kA_ss + (size_t)grp * a.kA_hs;
  const bf16* kB = a.kB + (size_t)slot * a.kB_ss;
  const bf16* vb = a.v + (size_t)slot * a.v_ss + (size_t)grp * a.v_hs + 64 * warp;
  const bool inA = gid < rep, inB = gid + 8 < rep;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  float o[8][4];
#pragma unroll
  for (int t = 0; t < 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
  // the key row of this thread for the next block is fetched while the current block is weighed and added: its 8-element
  // pieces for all columns stay in registers (the value accumulators of a warp are only 64 columns wide)
  uint4 kn[DK / 32];
  auto fetch_keys = [&](int kb) {
    const int jj = kb + 8 * warp + gid;
    const bool ok = jj < nkeys;
    const int row = ok ? (jlo + jj) % a.cap : 0;
    const bf16* kp = kA + (size_t)row * a.kA_rs + 8 * tig;
    const bf16* kq = kB + (size_t)row * a.kB_rs + 8 * tig;
#pragma unroll
    for (int j = 0; j < DK / 32; ++j)
      kn[j] = !ok ? zero4 : __ldg(reinterpret_cast<const uint4*>(j < DA / 32 ? kp + 32 * j : kq + 32 * (j - DA / 32)));
  };
  fetch_keys(64 * rank);
  for (int kb = 64 * rank; kb < nkeys; kb += 64 * nsplit) {
    // scores of this warp's 8 keys: thread (gid, tig) holds key kb + 8 warp + 2 tig (+1) for heads gid and gid + 8
    float s[4];
    {
      float sp[4][4];                                        // four independent chains over the key's columns
#pragma unroll
      for (int u = 0; u < 4; ++u) sp[u][0] = sp[u][1] = sp[u][2] = sp[u][3] = 0.f;
#pragma unroll
      for (int j = 0; j < DK / 32; ++j) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int wq = 16 * j + 4 * tig + 2 * half;
          const uint32_t af[4] = {sQ[gid * QS + wq], sQ[(gid + 8) * QS + wq], sQ[gid * QS + wq + 1], sQ[(gid + 8) * QS + wq + 1]};
          mma_bf16_16816(sp[(2 * j + half) & 3], af, half ? kn[j].z : kn[j].x, half ? kn[j].w : kn[j].y);
        }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) s[c] = (sp[0][c] + sp[1][c]) + (sp[2][c] + sp[3][c]);
    }
    if (kb + 64 * nsplit < nkeys) fetch_keys(kb + 64 * nsplit);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const bool vis = ((c >> 1) ? inB : inA) && kb + 8 * warp + 2 * tig + (c & 1) < nkeys;
      s[c] = vis ? s[c] * a.scale : -INFINITY;
    }
    float mxA = fmaxf(s[0], s[1]), mxB = fmaxf(s[2], s[3]);
    mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1)); mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
    mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1)); mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
    if (tig == 0) { sMax[warp][gid] = mxA; sMax[warp][gid + 8] = mxB; }
    __syncthreads();
    float nA = mA, nB = mB;
#pragma unroll
    for (int w = 0; w < NW; ++w) { nA = fmaxf(nA, sMax[w][gid]); nB = fmaxf(nB, sMax[w][gid + 8]); }
    const float cA = nA == -INFINITY ? 1.f : __expf(mA - nA), cB = nB == -INFINITY ? 1.f : __expf(mB - nB);
    const float bA = nA == -INFINITY ? 0.f : nA, bB = nB == -INFINITY ? 0.f : nB;
    mA = nA; mB = nB;
    const float w0 = __expf(s[0] - bA), w1 = __expf(s[1] - bA), w2 = __expf(s[2] - bB), w3 = __expf(s[3] - bB);
    lA = lA * cA + (w0 + w1);
    lB = lB * cB + (w2 + w3);
    uint32_t hi, lo;
    split_bf2(w0, w1, hi, lo);
    sPh[gid * PS + 4 * warp + tig] = hi; sPl[gid * PS + 4 * warp + tig] = lo;
    split_bf2(w2, w3, hi, lo);
    sPh[(gid + 8) * PS + 4 * warp + tig] = hi; sPl[(gid + 8) * PS + 4 * warp + tig] = lo;
#pragma unroll
    for (int t = 0; t < 8; ++t) { o[t][0] *= cA; o[t][1] *= cA; o[t][2] *= cB; o[t][3] *= cB; }
    __syncthreads();
    if (warp < PVW) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        if (kb + 16 * ks >= nkeys) break;
        const uint32_t ah[4] = {sPh[gid * PS + 8 * ks + tig], sPh[(gid + 8) * PS + 8 * ks + tig], sPh[gid * PS + 8 * ks + 4 + tig],
                                sPh[(gid + 8) * PS + 8 * ks + 4 + tig]};
        const uint32_t al[4] = {sPl[gid * PS + 8 * ks + tig], sPl[(gid + 8) * PS + 8 * ks + tig], sPl[gid * PS + 8 * ks + 4 + tig],
                                sPl[(gid + 8) * PS + 8 * ks + 4 + tig]};
        uint4 v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int jj = kb + 16 * ks + 2 * tig + (q & 1) + 8 * (q >> 1);
          v[q] = jj < nkeys ? __ldg(reinterpret_cast<const uint4*>(vb + (size_t)((jlo + jj) % a.cap) * a.v_rs + 8 * gid)) : zero4;
        }
        const uint32_t v0[4] = {v[0].x, v[0].y, v[0].z, v[0].w}, v1[4] = {v[1].x, v[1].y, v[1].z, v[1].w};
        const uint32_t v2[4] = {v[2].x, v[2].y, v[2].z, v[2].w}, v3[4] = {v[3].x, v[3].y, v[3].z, v[3].w};
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const uint32_t sel = (t & 1) ? 0x7632u : 0x5410u;
          const uint32_t b0 = __byte_perm(v0[t >> 1], v1[t >> 1], sel), b1 = __byte_perm(v2[t >> 1], v3[t >> 1], sel);
          mma_bf16_16816(o[t], ah, b0, b1);
          mma_bf16_16816(o[t], al, b0, b1);
        }
      }
    }
    // no barrier here: the next block's weights are written after its own first barrier, which every warp reaches only
    // after it has finished reading this block's
  }
  lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
  __syncthreads();                              // the last block's maxima have been read
  if (tig == 0) { sL[warp][gid] = lA; sL[warp][gid + 8] = lB; }
  __syncthreads();
  float LA = 0.f, LB = 0.f;
#pragma unroll
  for (int w = 0; w < NW; ++w) { LA += sL[w][gid]; LB += sL[w][gid + 8]; }
  if (nsplit > 1) {
    // partial results of this CTA into its shared memory; rank 0 merges the cluster's through distributed shared memory
    if (warp == 0 && tig == 0) { sPart[gid] = mA; sPart[gid + 8] = mB; sPart[16 + gid] = LA; sPart[16 + gid + 8] = LB; }
    if (warp < PVW) {
#pragma unroll
      for (int t = 0; t < 8; ++t)
#pragma unroll
        for (int c = 0; c < 4; ++c) sPart[32 + (gid + 8 * (c >> 1)) * DA + 64 * warp + 8 * (2 * tig + (c & 1)) + t] = o[t][c];
    }
    cluster_sync_all();
  }
  if (rank == 0 && warp < PVW) {
    const uint32_t part = (uint32_t)__cvta_generic_to_shared(sPart);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = gid + 8 * half;
      if (row >= rep) continue;
      const int head = grp * rep + row;
      const float m0 = half ? mB : mA;
      float M = a.sink ? fmaxf(m0, a.sink[head]) : m0;
      for (int r = 1; r < nsplit; ++r) M = fmaxf(M, __uint_as_float(ld_dsmem_u32(mapa_shared(part + 4u * (uint32_t)row, (uint32_t)r))));
      const float f0 = m0 == -INFINITY ? 0.f : __expf(m0 - M);
      float L = (half ? LB : LA) * f0 + (a.sink ? __expf(a.sink[head] - M) : 0.f);
      float acc[8][2];
#pragma unroll
      for (int t = 0; t < 8; ++t) { acc[t][0] = o[t][2 * half] * f0; acc[t][1] = o[t][2 * half + 1] * f0; }
      for (int r = 1; r < nsplit; ++r) {
        const float mr = __uint_as_float(ld_dsmem_u32(mapa_shared(part + 4u * (uint32_t)row, (uint32_t)r)));
        const float fr = mr == -INFINITY ? 0.f : __expf(mr - M);
        L += __uint_as_float(ld_dsmem_u32(mapa_shared(part + 4u * (uint32_t)(16 + row), (uint32_t)r))) * fr;
#pragma unroll
        for (int t = 0; t < 8; ++t)
#pragma unroll
          for (int e = 0; e < 2; ++e)
            acc[t][e] += fr * __uint_as_float(ld_dsmem_u32(
                             mapa_shared(part + 4u * (uint32_t)(32 + row * DA + 64 * warp + 8 * (2 * tig + e) + t), (uint32_t)r)));
      }
      float inv = 1.0f / L;
      // one output gate per head (a scalar commutes with the value up-projection that follows)
      if (a.gate) inv *= __fdividef(1.0f, 1.0f + __expf(-__bfloat162float(a.gate[(size_t)i * a.gate_ld + head])));
      bf16* orow = a.out + ((size_t)i * a.H + head) * a.out_hs + 64 * warp;
#pragma unroll
      for (int t = 0; t < 8; ++t)
#pragma unroll
        for (int e = 0; e < 2; ++e) orow[8 * (2 * tig + e) + t] = __float2bfloat16_rn(acc[t][e] * inv);
    }
  }
  if (nsplit > 1) cluster_sync_all();              // nobody leaves while its partial results may still be read
}

template <int DA>
static int launch_latent_absorbed(const WinMma& a, cudaStream_t st) {
  // a cluster per (token, head group) only while the grid would otherwise leave SMs empty and the window has blocks to share:
  // 64 tokens x 1 024 rows, 16 heads: 100 / 69 / 108 us with 1 / 2 / 4 CTAs per token (64 / 128 / 256 CTAs on 148 SMs)
  int nsplit = 1;
  while (nsplit < 4 && (long long)a.ntok * a.G * nsplit * 2 <= 148 && a.window >= 128 * nsplit * 2) nsplit *= 2;
  const size_t smem = (size_t)16 * ((DA + 64) / 2 + 4) * 4 + (size_t)2 * 16 * 36 * 4 + (nsplit > 1 ? (size_t)(32 + 16 * DA) * 4 : 0);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(latent_absorbed_mma_kernel<DA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.ntok, a.G, nsplit);
  cfg.blockDim = dim3(256);
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
  QSPEC_CUDA(cudaLaunchKernelEx(&cfg, latent_absorbed_mma_kernel<DA>, a, nsplit));
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

// ---------------------------------------------------------------------------------------------------------------------
// Softmax attention of one prompt portion on the tensor cores, tile form: a CTA of four warps takes 64 consecutive tokens
// of ONE sequence (rows pos0 .. pos0 + ntok - 1 of slot `slot`) and one head, and walks the visible keys in tiles of 64.
// Key tiles ([per-head part DA | shared part DB]) and value tiles arrive in shared memory by cp.async, two tiles in
// flight; ldmatrix feeds the fragments (keys as stored, values transposed), so every key / value row is read once per 64
// queries instead of once per 16. Scores, maxima, sums and weights are float32; the weights enter the second product as a
// two-term bfloat16 split taken straight from the score accumulators. Causal mask, window, sink and output gate as in
// window_attn_mma_kernel. CTAs run the longest key ranges first.
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

template <int DA, int DB, int DV, int NW>
__global__ void __launch_bounds__(32 * NW, NW == 4 ? 2 : 1) prompt_attn_mma_kernel(const WinMma a, int slot, int pos0) {
  pdl_enter();
  constexpr int DK = DA + DB, KS = DK + 8, VS = DV + 8, BM = 16 * NW, BN = 64, NT = 32 * NW, TPK = NT / BN;
  extern __shared__ __align__(16) unsigned char pa_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(pa_raw);              // [BM][KS]
  bf16* sK = sQ + BM * KS;                                 // [2][BN][KS]
  bf16* sV = sK + 2 * BN * KS;                             // [2][BN][VS]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
  const int qb = (int)gridDim.x - 1 - (int)blockIdx.x, head = blockIdx.y, kvh = head / (a.H / a.G);
  const int i0 = qb * BM;
  for (int c = tid; c < BM * (DK / 2); c += NT) {
    const int row = c / (DK / 2), w = c - row * (DK / 2), tok = i0 + row;
    uint32_t val = 0u;
    if (tok < a.ntok) {
      const float2 f = *reinterpret_cast<const float2*>(a.q + (size_t)tok * a.q_ts + (size_t)head * a.q_hs + 2 * w);
      val = pack_bf2(f.x, f.y);
    }
    *reinterpret_cast<uint32_t*>(sQ + row * KS + 2 * w) = val;
  }
  const int last = pos0 + min(i0 + BM, a.ntok) - 1;                     // last key any row of the block sees
  const int start = max(0, pos0 + i0 - a.window + 1);                    // first key the block's first row sees
  const int ntiles = (last - start + BN) / BN;
  const bf16* kA = a.kA + (size_t)slot * a.kA_ss + (size_t)kvh * a.kA_hs;
  const bf16* kB = DB ? a.kB + (size_t)slot * a.kB_ss : nullptr;
  const bf16* vb = a.v + (size_t)slot * a.v_ss + (size_t)kvh * a.v_hs;
  // TPK threads per key row: one row index (position % cap) per thread and tile, then straight runs of 16-byte pieces
  const int lkey = tid / TPK, lhalf = tid % TPK;
  auto load_tile = [&](int t, int buf) {
    const int j = start + t * BN + lkey;
    const bool ok = j <= last;
    const int row = ok ? j % a.cap : 0;
    bf16* dK = sK + ((size_t)buf * BN + lkey) * KS;
    bf16* dV = sV + ((size_t)buf * BN + lkey) * VS;
    const bf16* srcA = kA + (size_t)row * a.kA_rs;
#pragma unroll
    for (int x = 0; x < DA / 8 / TPK; ++x) {
      const int ch = lhalf * (DA / 8 / TPK) + x;
      cp_async16(dK + ch * 8, srcA + ch * 8, ok);
    }
    if (DB) {
      const bf16* srcB = kB + (size_t)row * a.kB_rs;
#pragma unroll
      for (int x = 0; x < DB / 8 / TPK; ++x) {
        const int ch = lhalf * (DB / 8 / TPK) + x;
        cp_async16(dK + DA + ch * 8, srcB + ch * 8, ok);
      }
    }
    const bf16* srcV = vb + (size_t)row * a.v_rs;
#pragma unroll
    for (int x = 0; x < DV / 8 / TPK; ++x) {
      const int ch = lhalf * (DV / 8 / TPK) + x;
      cp_async16(dV + ch * 8, srcV + ch * 8, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  load_tile(0, 0);
  __syncthreads();                                                       // the queries are in shared memory
  uint32_t qf[DK / 16][4];
#pragma unroll
  for (int ks = 0; ks < DK / 16; ++ks)
    ldmatrix_x4(qf[ks], sQ + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * KS + ks * 16 + 8 * (lane >> 4));
  float o[DV / 8][4];
#pragma unroll
  for (int t = 0; t < DV / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
  const int rowA = i0 + warp * 16 + gid, rowB = rowA + 8;
  const int posA = pos0 + rowA, posB = pos0 + rowB;
  const int wlast = pos0 + min(i0 + warp * 16 + 15, a.ntok - 1);        // last key this warp's rows see
  for (int t = 0; t < ntiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < ntiles) {
      load_tile(t + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    const int j0 = start + t * BN;
    if (j0 <= wlast) {                                                   // a tile past this warp's rows holds nothing for it
      const bf16* K = sK + (size_t)buf * BN * KS;
      const bf16* V = sV + (size_t)buf * BN * VS;
      float s[BN / 8][4];
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < DK / 16; ++ks)
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          uint32_t b[4];
          ldmatrix_x4(b, K + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * KS + ks * 16 + 8 * ((lane >> 3) & 1));
          mma_bf16_16816(s[2 * np], qf[ks], b[0], b[1]);
          mma_bf16_16816(s[2 * np + 1], qf[ks], b[2], b[3]);
        }
      float mxA = -INFINITY, mxB = -INFINITY;
      // a tile that lies wholly before the warp's first row and inside its last row's window needs no mask (most tiles)
      const int wfirst = pos0 + i0 + warp * 16;
      if (j0 + BN - 1 <= wfirst && j0 + BN - 1 <= last && (wfirst + 15) - j0 < a.window) {
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
          for (int c = 0; c < 4; ++c) s[nt][c] *= a.scale;
          mxA = fmaxf(mxA, fmaxf(s[nt][0], s[nt][1]));
          mxB = fmaxf(mxB, fmaxf(s[nt][2], s[nt][3]));
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int pj = j0 + nt * 8 + 2 * tig + (c & 1);
            const int pr = (c >> 1) ? posB : posA;
            const bool vis = pj <= pr && pr - pj < a.window && pj <= last;
            s[nt][c] = vis ? s[nt][c] * a.scale : -INFINITY;
            if (c >> 1) mxB = fmaxf(mxB, s[nt][c]); else mxA = fmaxf(mxA, s[nt][c]);
          }
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1)); mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1)); mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);
      const float cA = nA == -INFINITY ? 1.f : __expf(mA - nA), cB = nB == -INFINITY ? 1.f : __expf(mB - nB);
      const float bA = nA == -INFINITY ? 0.f : nA, bB = nB == -INFINITY ? 0.f : nB;
      mA = nA; mB = nB;
      float sumA = 0.f, sumB = 0.f;
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) {
        s[nt][0] = __expf(s[nt][0] - bA); s[nt][1] = __expf(s[nt][1] - bA);      // exp(-inf) = 0 for hidden keys
        s[nt][2] = __expf(s[nt][2] - bB); s[nt][3] = __expf(s[nt][3] - bB);
        sumA += s[nt][0] + s[nt][1];
        sumB += s[nt][2] + s[nt][3];
      }
      lA = lA * cA + sumA;
      lB = lB * cB + sumB;
      if (!__all_sync(0xffffffffu, cA == 1.f && cB == 1.f)) {            // no row of the warp met a new maximum: nothing to rescale
#pragma unroll
        for (int t2 = 0; t2 < DV / 8; ++t2) { o[t2][0] *= cA; o[t2][1] *= cA; o[t2][2] *= cB; o[t2][3] *= cB; }
      }
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        uint32_t ah[4], al[4];
        split_bf2(s[2 * kk][0], s[2 * kk][1], ah[0], al[0]);
        split_bf2(s[2 * kk][2], s[2 * kk][3], ah[1], al[1]);
        split_bf2(s[2 * kk + 1][0], s[2 * kk + 1][1], ah[2], al[2]);
        split_bf2(s[2 * kk + 1][2], s[2 * kk + 1][3], ah[3], al[3]);
#pragma unroll
        for (int dp = 0; dp < DV / 16; ++dp) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, V + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * VS + dp * 16 + 8 * (lane >> 4));
          mma_bf16_16816(o[2 * dp], ah, b[0], b[1]);
          mma_bf16_16816(o[2 * dp], al, b[0], b[1]);
          mma_bf16_16816(o[2 * dp + 1], ah, b[2], b[3]);
          mma_bf16_16816(o[2 * dp + 1], al, b[2], b[3]);
        }
      }
    }
    __syncthreads();                                                     // the buffer is free for the tile after next
  }
  lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int tok = half ? rowB : rowA;
    if (tok >= a.ntok) continue;
    const float m = half ? mB : mA, l = half ? lB : lA;
    float f = 1.f, L = l;
    if (a.sink) {
      const float M = fmaxf(m, a.sink[head]);
      f = m == -INFINITY ? 0.f : __expf(m - M);
      L = l * f + __expf(a.sink[head] - M);
    }
    float inv = L > 0.f ? f / L : 0.f;
    const bf16* gp = a.gate ? a.gate + (size_t)tok * a.gate_ld + (a.gate_per_head ? (size_t)head : (size_t)head * DV) : nullptr;
    if (gp && a.gate_per_head) inv *= __fdividef(1.0f, 1.0f + __expf(-__bfloat162float(gp[0])));
    bf16* orow = a.out + ((size_t)tok * a.H + head) * DV;
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt) {
      const int d = nt * 8 + 2 * tig;
      float v0 = o[nt][2 * half] * inv, v1 = o[nt][2 * half + 1] * inv;
      if (gp && !a.gate_per_head) {
        v0 *= __fdividef(1.0f, 1.0f + __expf(-__bfloat162float(gp[d])));
        v1 *= __fdividef(1.0f, 1.0f + __expf(-__bfloat162float(gp[d + 1])));
      }
      *reinterpret_cast<uint32_t*>(orow + d) = pack_bf2(v0, v1);
    }
  }
}

template <int DA, int DB, int DV, int NW>
static int launch_prompt_attn_w(const WinMma& a, int slot, int pos0, cudaStream_t st) {
  constexpr int BM = 16 * NW;
  constexpr size_t smem = ((size_t)(BM + 2 * 64) * (DA + DB + 8) + (size_t)2 * 64 * (DV + 8)) * sizeof(bf16);
  static bool configured = false;
  if (!configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(prompt_attn_mma_kernel<DA, DB, DV, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  launch_pdl(prompt_attn_mma_kernel<DA, DB, DV, NW>, dim3((a.ntok + BM - 1) / BM, a.H), dim3(32 * NW), smem, st, a, slot, pos0);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

// 128 tokens per CTA (eight warps, one CTA per SM) once such CTAs fill the GPU: every key / value tile then serves twice the
// queries; 64 tokens per CTA (two CTAs per SM) for shorter portions. QSPEC_SEQ_PROMPT_ROWS=64 / 128 fixes the choice.
template <int DA, int DB, int DV>
static int launch_prompt_attn(const WinMma& a, int slot, int pos0, cudaStream_t st) {
  static const int fixed = [] { const char* v = getenv("QSPEC_SEQ_PROMPT_ROWS"); return v ? atoi(v) : 0; }();
  const bool wide = fixed ? fixed == 128 : (long long)((a.ntok + 127) / 128) * a.H >= 148;
  if (wide) return launch_prompt_attn_w<DA, DB, DV, 8>(a, slot, pos0, st);
  return launch_prompt_attn_w<DA, DB, DV, 4>(a, slot, pos0, st);
}

bool prompt_mma_shape(int DA, int DB, int DV) {
  return (DA == 128 && DB == 64 && DV == 128) || (DA == 128 && DB == 0 && DV == 128) || (DA == 64 && DB == 0 && DV == 64);
}

// Entry for qspec_seq_prompt_attention_mma (below): -1 when the shape or the strides are not ones this form takes.
int prompt_attention_mma(const qspec_window_attn_args* p, const void* kB, long long kB_ss, int kB_rs, int DB, int slot, int pos0,
                         cudaStream_t st) {
  const int DA = p->DA, DV = p->DV;
  const bool ok = prompt_mma_shape(DA, DB, DV) && p->H % p->G == 0 && p->H <= 65535 && p->k_row_stride % 8 == 0 && p->k_head_stride % 8 == 0 &&
                  p->k_slot_stride % 8 == 0 && p->v_row_stride % 8 == 0 && p->v_head_stride % 8 == 0 && p->v_slot_stride % 8 == 0 &&
                  kB_rs % 8 == 0 && kB_ss % 8 == 0 && p->qa_tok_stride % 2 == 0 && p->qa_head_stride % 2 == 0 &&
                  (((uintptr_t)p->k | (uintptr_t)p->v | (uintptr_t)kB) & 15) == 0 && ((uintptr_t)p->qa & 7) == 0 && ((uintptr_t)p->out & 3) == 0;
  if (!ok) return -1;
  WinMma a;
  a.q = p->qa; a.q_ts = p->qa_tok_stride; a.q_hs = p->qa_head_stride;
  a.kA = (const bf16*)p->k; a.kA_ss = p->k_slot_stride; a.kA_rs = p->k_row_stride; a.kA_hs = p->k_head_stride;
  a.kB = (const bf16*)kB; a.kB_ss = kB_ss; a.kB_rs = kB_rs;
  a.v = (const bf16*)p->v; a.v_ss = p->v_slot_stride; a.v_rs = p->v_row_stride; a.v_hs = p->v_head_stride;
  a.sink = p->sink; a.gate = (const bf16*)p->gate; a.gate_ld = p->gate_ld; a.gate_per_head = p->gate_per_head;
  a.out = (bf16*)p->out; a.out_hs = DV; a.meta = p->meta; a.ntok = p->ntok; a.H = p->H; a.G = p->G; a.window = p->window; a.cap = p->cap;
  a.scale = p->scale; a.token_rows = 1;
  if (DB) return launch_prompt_attn<128, 64, 128>(a, slot, pos0, st);
  if (DA == 128) return launch_prompt_attn<128, 0, 128>(a, slot, pos0, st);
  return launch_prompt_attn<64, 0, 64>(a, slot, pos0, st);
}

template <int DA, int DB, int DV, bool STREAM>
static int launch_window_mma(const WinMma& a, int slices, cudaStream_t st) {
  constexpr size_t smem = (size_t)16 * ((DA + DB) / 2 + 4) * 4 + (size_t)4 * 16 * DV * sizeof(float);
  static bool configured = false;
  if (!configured) {
    QSPEC_CUDA(cudaFuncSetAttribute(window_attn_mma_kernel<DA, DB, DV, STREAM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  const dim3 grid = a.token_rows ? dim3((a.ntok + 15) / 16, a.H, slices) : dim3(a.ntok, a.G, slices);
  launch_pdl(window_attn_mma_kernel<DA, DB, DV, STREAM>, grid, dim3(128), smem, st, a);
  QSPEC_CHECK_LAUNCH(1);
  return QSPEC_OK;
}

// Shapes: per-head key part 64 or 128 with values of 64 or 128; 128 + a shared part of 64 with values of 128 (a latent
// layer's expanded form); 256 or 512 + a shared part of 64 with values of 128, 256, 384 or 512 in slices of 128 columns (a
// latent cache read in the absorbed form: key and value are the same rows).
bool window_mma_shape(int DA, int DB, int DV) {
  if (DB == 0) return (DA == 64 || DA == 128) && (DV == 64 || DV == 128);
  if (DB != 64) return false;
  if (DA == 128) return DV == 128;
  return (DA == 256 || DA == 512) && DV % 128 == 0 && DV >= 128 && DV <= 512;
}

// Entry for qspec_seq_window_attention_mma (below): -1 when the shape is not one this form takes.
int window_attention_mma(const qspec_window_attn_args* p, const void* kB, long long kB_ss, int kB_rs, int DB, int token_rows,
                         cudaStream_t st) {
  const int DA = p->DA, DV = p->DV;
  const bool ok = window_mma_shape(DA, DB, DV) && p->H % p->G == 0 && (token_rows || p->H / p->G <= 16) && p->H <= 65535 && p->G <= 65535 &&
                  p->k_row_stride % 8 == 0 && p->k_head_stride % 8 == 0 && p->k_slot_stride % 8 == 0 && p->v_row_stride % 8 == 0 &&
                  p->v_head_stride % 8 == 0 && p->v_slot_stride % 8 == 0 && kB_rs % 8 == 0 && kB_ss % 8 == 0 &&
                  p->qa_tok_stride % 2 == 0 && p->qa_head_stride % 2 == 0 &&
                  (((uintptr_t)p->k | (uintptr_t)p->v | (uintptr_t)kB) & 15) == 0 && ((uintptr_t)p->qa & 7) == 0;
  if (!ok) return -1;
  WinMma a;
  a.q = p->qa; a.q_ts = p->qa_tok_stride; a.q_hs = p->qa_head_stride;
  a.kA = (const bf16*)p->k; a.kA_ss = p->k_slot_stride; a.kA_rs = p->k_row_stride; a.kA_hs = p->k_head_stride;
  a.kB = (const bf16*)kB; a.kB_ss = kB_ss; a.kB_rs = kB_rs;
  a.v = (const bf16*)p->v; a.v_ss = p->v_slot_stride; a.v_rs = p->v_row_stride; a.v_hs = p->v_head_stride;
  a.sink = p->sink; a.gate = (const bf16*)p->gate; a.gate_ld = p->gate_ld; a.gate_per_head = p->gate_per_head;
  a.out = (bf16*)p->out; a.out_hs = DV; a.meta = p->meta; a.ntok = p->ntok; a.H = p->H; a.G = p->G; a.window = p->window; a.cap = p->cap;
  a.scale = p->scale; a.token_rows = token_rows;
  // a latent cache read in the absorbed form (keys and values are the same rows): the CTA-level kernel; QSPEC_SEQ_LATENT=sliced
  // keeps the form with one CTA per slice of 128 value columns, for comparison
  static const bool sliced = [] { const char* v = getenv("QSPEC_SEQ_LATENT"); return v && !strcmp(v, "sliced"); }();
  if (!sliced && !token_rows && DA >= 256 && DV == DA && p->v == p->k && (!p->gate || p->gate_per_head)) {
    if (DA == 512) return launch_latent_absorbed<512>(a, st);
    return launch_latent_absorbed<256>(a, st);
  }
  if (DA == 512) return launch_window_mma<512, 64, 128, true>(a, DV / 128, st);
  if (DA == 256) return launch_window_mma<256, 64, 128, true>(a, DV / 128, st);
  if (DB) return launch_window_mma<128, 64, 128, false>(a, 1, st);
  if (DA == 64 && DV == 64) return launch_window_mma<64, 0, 64, false>(a, 1, st);
  if (DA == 64) return launch_window_mma<64, 0, 128, false>(a, 1, st);
  if (DV == 64) return launch_window_mma<128, 0, 64, false>(a, 1, st);
  return launch_window_mma<128, 0, 128, false>(a, 1, st);
}
}  // namespace qspec

extern "C" int qspec_seq_window_attention_mma(const qspec_window_attn_args* args, const void* k_shared, long long k_shared_slot_stride,
                                              int k_shared_row_stride, int DB, int token_rows, void* stream) {
  QSPEC_REQUIRE(args && args->qa && args->k && args->v && args->out && args->meta && (DB == 0 || k_shared), QSPEC_ERR_INVALID_ARG,
                "seq_window_attention_mma: null pointer");
  QSPEC_REQUIRE(args->DB == 0, QSPEC_ERR_INVALID_ARG, "seq_window_attention_mma: the query is one part here (DA = the whole key size)");
  if (args->ntok == 0) return QSPEC_OK;
  qspec_window_attn_args p = *args;
  p.DA = args->DA - DB;                                   // size of the per-head key part
  const int s = qspec::window_attention_mma(&p, k_shared, k_shared_slot_stride, k_shared_row_stride, DB, token_rows, (cudaStream_t)stream);
  QSPEC_REQUIRE(s >= 0, QSPEC_ERR_UNSUPPORTED, "seq_window_attention_mma: key parts %d + %d, value size %d, or strides / alignment not taken",
                args->DA - DB, DB, args->DV);
  return s;
}

extern "C" int qspec_seq_window_attention_mma_supported(int DA, int DB, int DV, int H, int G, int token_rows) {
  return qspec::window_mma_shape(DA, DB, DV) && G > 0 && H % G == 0 && (token_rows || H / G <= 16);
}

extern "C" int qspec_seq_prompt_attention_mma(const qspec_window_attn_args* args, const void* k_shared, long long k_shared_slot_stride,
                                              int k_shared_row_stride, int DB, int slot, int pos0, void* stream) {
  QSPEC_REQUIRE(args && args->qa && args->k && args->v && args->out && (DB == 0 || k_shared), QSPEC_ERR_INVALID_ARG,
                "seq_prompt_attention_mma: null pointer");
  QSPEC_REQUIRE(args->DB == 0 && slot >= 0 && pos0 >= 0 && args->window >= 1 && args->cap >= 1, QSPEC_ERR_INVALID_ARG,
                "seq_prompt_attention_mma: the query is one part here (DA = the whole key size); slot and first position from 0");
  if (args->ntok == 0) return QSPEC_OK;
  qspec_window_attn_args p = *args;
  p.DA = args->DA - DB;
  const int s = qspec::prompt_attention_mma(&p, k_shared, k_shared_slot_stride, k_shared_row_stride, DB, slot, pos0, (cudaStream_t)stream);
  QSPEC_REQUIRE(s >= 0, QSPEC_ERR_UNSUPPORTED, "seq_prompt_attention_mma: key parts %d + %d, value size %d, or strides / alignment not taken",
                args->DA - DB, DB, args->DV);
  return s;
}

extern "C" int qspec_seq_prompt_attention_mma_supported(int DA, int DB, int DV) { return qspec::prompt_mma_shape(DA, DB, DV); }

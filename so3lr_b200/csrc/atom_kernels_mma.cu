// Per-atom dense blocks (post-attention block of every layer and the output heads, forward and reverse) with their
// contractions on the tensor cores.
//
// A CTA of 4 warps owns a tile of 64 atoms; warp w owns atoms 16w .. 16w+15 of it for every contraction (M = 16 of
// mma.sync m16n8k16), so the chain LayerNorm -> Dense -> silu -> Dense -> ... of one atom never leaves its warp.
// Activations live in shared memory feature-major ([feature][atom], row stride 65); the A fragments are split on the fly
// into FP16 hi + scaled-lo pairs, the kernels come pre-split in fragment order from global memory (L1/L2 resident, one
// 128-bit load per fragment), and every product is three MMAs (hi*hi, hi*lo, lo*hi) accumulated in FP32, which keeps
// FP32-level accuracy (the dropped lo*lo term is below 2^-22).
#include <cuda_fp16.h>

#include "kernels.h"

namespace so3lr {

namespace {

constexpr int TA = 64;     // atoms per tile
constexpr int TS = 65;     // shared-memory row stride (floats)
constexpr int NT = 128;    // threads per CTA
constexpr float kLoScale = 2048.f, kLoInv = 1.f / 2048.f;

__device__ __forceinline__ float inv_weight(int l) {
  return l == 0 ? 0.5773502691896258f : (l == 1 ? 0.4472135954999579f : (l == 2 ? 0.3779644730092272f : 0.3333333333333333f));
}
__device__ __forceinline__ void split2(float x, float y, unsigned& hi, unsigned& lo) {
  const __half2 h = __floats2half2_rn(x, y);
  const float2 hf = __half22float2(h);
  const __half2 l = __floats2half2_rn((x - hf.x) * kLoScale, (y - hf.y) * kLoScale);
  hi = *reinterpret_cast<const unsigned*>(&h);
  lo = *reinterpret_cast<const unsigned*>(&l);
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int F>
__device__ __forceinline__ void load_tile_T(float* T, const float* __restrict__ src, int row0, int n) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < TA; r += NT / 32) {
    int a = row0 + r;
#pragma unroll
    for (int c = 0; c < F / 32; ++c) {
      float v = (a < n) ? src[(size_t)a * F + lane + 32 * c] : 0.f;
      T[(lane + 32 * c) * TS + r] = v;
    }
  }
}
template <int F>
__device__ __forceinline__ void store_tile_T(float* __restrict__ dst, const float* T, int row0, int n) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < TA; r += NT / 32) {
    int a = row0 + r;
    if (a >= n) continue;
#pragma unroll
    for (int c = 0; c < F / 32; ++c) dst[(size_t)a * F + lane + 32 * c] = T[(lane + 32 * c) * TS + r];
  }
}

// Output fragment bookkeeping of a thread: acc[nt][e] is row frag_row(e) of the tile and column frag_col(nt, e).
struct Frag {
  int g, q, r0;   // r0 = first row of the warp's 16 atoms
  __device__ __forceinline__ Frag() : g((threadIdx.x & 31) >> 2), q(threadIdx.x & 3), r0(16 * (threadIdx.x >> 5)) {}
  __device__ __forceinline__ int row(int e) const { return r0 + g + 8 * (e >> 1); }
  __device__ __forceinline__ int col(int nt, int e) const { return 8 * nt + 2 * q + (e & 1); }
};

// acc[nt][e] (+)= sum_k A[row][k] * W[k][col]: A = the warp's 16 rows of the feature-major tile At (K features),
// Wf = the kernel in fragment order ([K/16][NOUT/8][32]).  ACCUM: add to the incoming acc.
// The same contraction with all output columns in one pass (one weight load in front of every three MMAs): the reverse
// dense block keeps more state live and measured faster with this form.
template <int K, int NOUT, bool ACCUM>
__device__ __forceinline__ void gemm_mma_flat(const float* At, const uint4* __restrict__ Wf, float (&acc)[NOUT / 8][4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3, r = 16 * (threadIdx.x >> 5) + g;
  float cross[NOUT / 8][4];
#pragma unroll
  for (int nt = 0; nt < NOUT / 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) { cross[nt][e] = 0.f; if (!ACCUM) acc[nt][e] = 0.f; }
#pragma unroll 1
  for (int ks = 0; ks < K / 16; ++ks) {
    const float* a = At + (16 * ks + 2 * q) * TS + r;
    unsigned ah[4], al[4];
    split2(a[0], a[TS], ah[0], al[0]);
    split2(a[8], a[TS + 8], ah[1], al[1]);
    split2(a[8 * TS], a[9 * TS], ah[2], al[2]);
    split2(a[8 * TS + 8], a[9 * TS + 8], ah[3], al[3]);
    const uint4* w = Wf + (size_t)ks * (NOUT / 8) * 32 + lane;
#pragma unroll
    for (int nt = 0; nt < NOUT / 8; ++nt) {
      const uint4 b = w[nt * 32];
      mma16816(cross[nt], ah[0], ah[1], ah[2], ah[3], b.z, b.w);
      mma16816(cross[nt], al[0], al[1], al[2], al[3], b.x, b.y);
      mma16816(acc[nt], ah[0], ah[1], ah[2], ah[3], b.x, b.y);
    }
  }
#pragma unroll
  for (int nt = 0; nt < NOUT / 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nt][e] = fmaf(cross[nt][e], kLoInv, acc[nt][e]);
}

template <int K, int NOUT, bool ACCUM>
__device__ __forceinline__ void gemm_mma(const float* At, const uint4* __restrict__ Wf, float (&acc)[NOUT / 8][4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3, r = 16 * (threadIdx.x >> 5) + g;
  // The output columns are done in groups of 64: the hi*lo cross terms need their own accumulators, and with half of them
  // live there are registers left to have a whole group's weight fragments (8 x 16 bytes per lane) in flight before the
  // first MMA of a k-step issues, instead of one load in front of every three MMAs.
  constexpr int NG = NOUT / 8 > 8 ? 8 : NOUT / 8;
#pragma unroll
  for (int n0 = 0; n0 < NOUT / 8; n0 += NG) {
    float cross[NG][4];
#pragma unroll
    for (int nt = 0; nt < NG; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) { cross[nt][e] = 0.f; if (!ACCUM) acc[n0 + nt][e] = 0.f; }
#pragma unroll 1
    for (int ks = 0; ks < K / 16; ++ks) {
      const uint4* w = Wf + ((size_t)ks * (NOUT / 8) + n0) * 32 + lane;
      uint4 b[NG];
#pragma unroll
      for (int nt = 0; nt < NG; ++nt) b[nt] = w[nt * 32];
      const float* a = At + (16 * ks + 2 * q) * TS + r;
      unsigned ah[4], al[4];
      split2(a[0], a[TS], ah[0], al[0]);
      split2(a[8], a[TS + 8], ah[1], al[1]);
      split2(a[8 * TS], a[9 * TS], ah[2], al[2]);
      split2(a[8 * TS + 8], a[9 * TS + 8], ah[3], al[3]);
#pragma unroll
      for (int nt = 0; nt < NG; ++nt) {
        mma16816(cross[nt], ah[0], ah[1], ah[2], ah[3], b[nt].z, b[nt].w);
        mma16816(cross[nt], al[0], al[1], al[2], al[3], b[nt].x, b[nt].y);
        mma16816(acc[n0 + nt], ah[0], ah[1], ah[2], ah[3], b[nt].x, b[nt].y);
      }
    }
#pragma unroll
    for (int nt = 0; nt < NG; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[n0 + nt][e] = fmaf(cross[nt][e], kLoInv, acc[n0 + nt][e]);
  }
}

// One 32 x 32 block: acc[nt][e] (+)= sum_{k<32} A[row][k0 + k] * B[k][col], B in fragment order ([2][4][32]).
template <bool ACCUM>
__device__ __forceinline__ void gemm_block32(const float* At, int k0, const uint4* __restrict__ Bf, float (&acc)[4][4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3, r = 16 * (threadIdx.x >> 5) + g;
  float cross[4][4];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) { cross[nt][e] = 0.f; if (!ACCUM) acc[nt][e] = 0.f; }
#pragma unroll
  for (int ks = 0; ks < 2; ++ks) {
    const float* a = At + (k0 + 16 * ks + 2 * q) * TS + r;
    unsigned ah[4], al[4];
    split2(a[0], a[TS], ah[0], al[0]);
    split2(a[8], a[TS + 8], ah[1], al[1]);
    split2(a[8 * TS], a[9 * TS], ah[2], al[2]);
    split2(a[8 * TS + 8], a[9 * TS + 8], ah[3], al[3]);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const uint4 b = Bf[(ks * 4 + nt) * 32 + lane];
      mma16816(cross[nt], ah[0], ah[1], ah[2], ah[3], b.z, b.w);
      mma16816(cross[nt], al[0], al[1], al[2], al[3], b.x, b.y);
      mma16816(acc[nt], ah[0], ah[1], ah[2], ah[3], b.x, b.y);
    }
  }
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nt][e] = fmaf(cross[nt][e], kLoInv, acc[nt][e]);
}

// per-row LayerNorm statistics over 128 features held feature-major in T
__device__ __forceinline__ void ln_stats(const float* T, int r, float& mean, float& rstd) {
  float s = 0.f;
  for (int k = 0; k < kF; ++k) s += T[k * TS + r];
  mean = s * (1.f / kF);
  float v = 0.f;
  for (int k = 0; k < kF; ++k) { float d = T[k * TS + r] - mean; v = fmaf(d, d, v); }
  rstd = rsqrtf(v * (1.f / kF) + kLnEps);
}

// sum over the 4 lanes that share a row (the columns of a row are spread over them)
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// post-attention block, forward:
//   x1 = LN1(xa); x2 = x1 + Dense2(silu(Dense1(silu(x1)))); [yx, gate] = Dense132([x2, inv(ev1)])
//   x3 = x2 + yx; ev2 = ev1 * (1 + gate_l); x4 = LN2(x3)
// saves z1 (hidden pre-activation), x3 and gate for the reverse pass
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NT) atom_post_fwd_mma_kernel(LayerDev L, int n, const float* __restrict__ xa,
                                                               const float* __restrict__ ev1, float* __restrict__ z1_out,
                                                               float* __restrict__ x3_out, float* __restrict__ gate_out,
                                                               float* __restrict__ x4_out, float* __restrict__ ev2_out,
                                                               const uint4* __restrict__ proj_next, float* __restrict__ qkv_next) {
  extern __shared__ float sm[];
  float* At = sm;                  // 128*TS
  float* Bt = At + kF * TS;        // 128*TS
  float* invs = Bt + kF * TS;      // 64*4
  float* gates = invs + TA * 4;    // 64*4
  const int tid = threadIdx.x;
  const int row0 = blockIdx.x * TA;
  const Frag fr;

  load_tile_T<kF>(At, xa, row0, n);
  __syncthreads();
  if (tid < TA) {
    float m, rs;
    ln_stats(At, tid, m, rs);
    for (int k = 0; k < kF; ++k) {
      float v = (At[k * TS + tid] - m) * rs * L.ln1_s[k] + L.ln1_b[k];
      At[k * TS + tid] = v;
      Bt[k * TS + tid] = silu_f(v);
    }
    int a = row0 + tid;
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    if (a < n) {
      for (int m2 = 0; m2 < kMTot; ++m2) { float e = ev1[(size_t)a * kMTot + m2]; s[degree_of(m2)] += e * e; }
    }
    for (int l = 0; l < 4; ++l) invs[tid * 4 + l] = s[l] * inv_weight(l);
  }
  __syncthreads();
  float acc[16][4];
  // hidden layer
  gemm_mma<kF, kF, false>(Bt, L.res1_f, acc);
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    const float2 b = *reinterpret_cast<const float2*>(L.res1_b + 8 * nt + 2 * fr.q);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = fr.row(e), c = fr.col(nt, e);
      const float z = acc[nt][e] + ((e & 1) ? b.y : b.x);
      if (row0 + r < n) z1_out[(size_t)(row0 + r) * kF + c] = z;
      Bt[c * TS + r] = silu_f(z);
    }
  }
  __syncwarp();
  gemm_mma<kF, kF, false>(Bt, L.res2_f, acc);
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    const float2 b = *reinterpret_cast<const float2*>(L.res2_b + 8 * nt + 2 * fr.q);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = fr.row(e), c = fr.col(nt, e);
      At[c * TS + r] += acc[nt][e] + ((e & 1) ? b.y : b.x);      // x2
    }
  }
  __syncwarp();
  // exchange: features -> features
  gemm_mma<kF, kF, false>(At, L.exxx_f, acc);
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = fr.row(e), c = fr.col(nt, e);
      const float* iv = invs + r * 4;
      const float y = acc[nt][e] + L.ex_bx[c] + iv[0] * L.ex_ix[c] + iv[1] * L.ex_ix[kF + c] + iv[2] * L.ex_ix[2 * kF + c] + iv[3] * L.ex_ix[3 * kF + c];
      const float v = At[c * TS + r] + y;
      Bt[c * TS + r] = v;
      if (row0 + r < n) x3_out[(size_t)(row0 + r) * kF + c] = v;
    }
  }
  __syncthreads();
  // gates: 4 extra output columns of the exchange layer (reads x2 in At)
  {
    int r = tid & 63, g0 = tid >> 6;
    for (int g = g0; g < 4; g += 2) {
      float s = L.ex_bg[g];
      for (int k = 0; k < kF; ++k) s = fmaf(At[k * TS + r], L.ex_xg[k * 4 + g], s);
      for (int l = 0; l < 4; ++l) s = fmaf(invs[r * 4 + l], L.ex_ig[l * 4 + g], s);
      gates[r * 4 + g] = s;
      if (row0 + r < n) gate_out[(size_t)(row0 + r) * 4 + g] = s;
    }
  }
  __syncthreads();
  if (tid < TA) {
    float m, rs;
    ln_stats(Bt, tid, m, rs);
    for (int k = 0; k < kF; ++k) Bt[k * TS + tid] = (Bt[k * TS + tid] - m) * rs * L.ln2_s[k] + L.ln2_b[k];
    int a = row0 + tid;
    if (a < n) {
      for (int m2 = 0; m2 < kMTot; ++m2) {
        float e = ev1[(size_t)a * kMTot + m2];
        ev2_out[(size_t)a * kMTot + m2] = e * (1.f + gates[tid * 4 + degree_of(m2)]);
      }
    }
  }
  __syncthreads();
  store_tile_T<kF>(x4_out, Bt, row0, n);
  // q/k/v rows of the next layer straight from the x4 tile: 5 projections x 4 heads of 32 x 32
  if (proj_next) {
#pragma unroll 1
    for (int h = 0; h < 4; ++h)
#pragma unroll 1
      for (int w = 0; w < 5; ++w) {
        float pa[4][4];
        gemm_block32<false>(Bt, 32 * h, proj_next + (size_t)(w * 4 + h) * 256, pa);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int c = w * kF + 32 * h + 8 * nt + 2 * fr.q;
          if (row0 + fr.row(0) < n) *reinterpret_cast<float2*>(qkv_next + (size_t)(row0 + fr.row(0)) * kProj + c) = make_float2(pa[nt][0], pa[nt][1]);
          if (row0 + fr.row(2) < n) *reinterpret_cast<float2*>(qkv_next + (size_t)(row0 + fr.row(2)) * kProj + c) = make_float2(pa[nt][2], pa[nt][3]);
        }
      }
  }
}

// ------------------------------------------------------------------------------------------------
// post-attention block, reverse.  in: g4 = dL/dx4, gev2 = dL/dev2 ; out: g_xa = dL/dxa, gev1 = dL/dev1
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NT) atom_post_bwd_mma_kernel(LayerDev L, int n, const float* __restrict__ xa,
                                                               const float* __restrict__ ev1, const float* __restrict__ z1,
                                                               const float* __restrict__ x3, const float* __restrict__ gate,
                                                               const float* __restrict__ g4, const float* __restrict__ gev2,
                                                               float* g_xa, float* __restrict__ gev1,
                                                               const uint4* __restrict__ projT_up, const float* __restrict__ g_qkv_up) {
  extern __shared__ float sm[];
  float* At = sm;
  float* Bt = At + kF * TS;
  float* Ct = Bt + kF * TS;
  float* ggate = Ct + kF * TS;     // 64*4
  float* ginv = ggate + TA * 4;    // 64*4
  float* rstd1 = ginv + TA * 4;    // 64
  const int tid = threadIdx.x;
  const int row0 = blockIdx.x * TA;
  const Frag fr;

  if (projT_up) {
    // cotangent of this layer's output from the layer above: skip connection (its g_xa, still in the g_xa buffer: this
    // CTA reads its rows before it overwrites them at the end) + transposed q/k/v projections of its g_qkv
    float ga[16][4];
#pragma unroll 1
    for (int w = 0; w < 5; ++w) {
      __syncthreads();
      for (int rr = threadIdx.x >> 5; rr < TA; rr += NT / 32) {
        const int a = row0 + rr, lane = threadIdx.x & 31;
#pragma unroll
        for (int c = 0; c < 4; ++c) At[(lane + 32 * c) * TS + rr] = (a < n) ? g_qkv_up[(size_t)a * kProj + w * kF + lane + 32 * c] : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        float pa[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) pa[nt][e] = w ? ga[4 * h + nt][e] : 0.f;
        gemm_block32<true>(At, 32 * h, projT_up + (size_t)(w * 4 + h) * 256, pa);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) ga[4 * h + nt][e] = pa[nt][e];
      }
    }
    __syncthreads();
    load_tile_T<kF>(Bt, g_xa, row0, n);
    __syncthreads();
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) Bt[fr.col(nt, e) * TS + fr.row(e)] += ga[nt][e];
    __syncthreads();
  } else {
    load_tile_T<kF>(Bt, g4, row0, n);
  }
  load_tile_T<kF>(At, x3, row0, n);
  load_tile_T<kF>(Ct, xa, row0, n);
  __syncthreads();
  if (tid < TA) {
    const int r = tid, a = row0 + r;
    // LayerNorm-2 reverse: Bt <- g3
    float m, rs;
    ln_stats(At, r, m, rs);
    float s1 = 0.f, s2 = 0.f;
    for (int k = 0; k < kF; ++k) {
      float xh = (At[k * TS + r] - m) * rs;
      float gy = Bt[k * TS + r] * L.ln2_s[k];
      s1 += gy; s2 = fmaf(gy, xh, s2);
    }
    s1 *= (1.f / kF); s2 *= (1.f / kF);
    for (int k = 0; k < kF; ++k) {
      float xh = (At[k * TS + r] - m) * rs;
      float gy = Bt[k * TS + r] * L.ln2_s[k];
      Bt[k * TS + r] = rs * (gy - s1 - xh * s2);
    }
    float gg[4] = {0.f, 0.f, 0.f, 0.f};
    if (a < n)
      for (int m2 = 0; m2 < kMTot; ++m2) gg[degree_of(m2)] += gev2[(size_t)a * kMTot + m2] * ev1[(size_t)a * kMTot + m2];
    for (int l = 0; l < 4; ++l) ggate[r * 4 + l] = gg[l];
    // LayerNorm-1 forward statistics: Ct <- normalised xa (no affine)
    ln_stats(Ct, r, m, rs);
    rstd1[r] = rs;
    for (int k = 0; k < kF; ++k) Ct[k * TS + r] = (Ct[k * TS + r] - m) * rs;
  }
  __syncthreads();
  // cotangent of the invariants: ginv[r][l] = sum_c g3[r][c] Wix[l][c] + sum_g ggate[r][g] Wig[l][g]
  {
    int r = tid & 63, l0 = tid >> 6;
    for (int l = l0; l < 4; l += 2) {
      float s = 0.f;
      for (int c = 0; c < kF; ++c) s = fmaf(Bt[c * TS + r], L.ex_ix[l * kF + c], s);
      for (int g = 0; g < 4; ++g) s = fmaf(ggate[r * 4 + g], L.ex_ig[l * 4 + g], s);
      ginv[r * 4 + l] = s;
    }
  }
  __syncthreads();
  float acc[16][4];
  gemm_mma_flat<kF, kF, false>(Bt, L.exxxT_f, acc);
  __syncwarp();
  // g_x2 = g3 + g3 Wxx^T + ggate Wxg^T   -> At
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = fr.row(e), c = fr.col(nt, e);
      const float* gg = ggate + r * 4;
      const float4 w = *reinterpret_cast<const float4*>(L.ex_xg + c * 4);
      At[c * TS + r] = Bt[c * TS + r] + acc[nt][e] + gg[0] * w.x + gg[1] * w.y + gg[2] * w.z + gg[3] * w.w;
    }
  }
  __syncthreads();
  if (tid < TA) {
    int a = row0 + tid;
    if (a < n)
      for (int m2 = 0; m2 < kMTot; ++m2) {
        int l = degree_of(m2);
        float e = ev1[(size_t)a * kMTot + m2];
        gev1[(size_t)a * kMTot + m2] = gev2[(size_t)a * kMTot + m2] * (1.f + gate[(size_t)a * 4 + l]) +
                                        ginv[tid * 4 + l] * 2.f * e * inv_weight(l);
      }
  }
  // residual MLP reverse
  gemm_mma_flat<kF, kF, false>(At, L.res2T_f, acc);
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = fr.row(e), c = fr.col(nt, e);
      const float z = (row0 + r < n) ? z1[(size_t)(row0 + r) * kF + c] : 0.f;
      Bt[c * TS + r] = acc[nt][e] * dsilu_f(z);
    }
  }
  __syncwarp();
  gemm_mma_flat<kF, kF, false>(Bt, L.res1T_f, acc);
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = fr.row(e), c = fr.col(nt, e);
      const float x1 = Ct[c * TS + r] * L.ln1_s[c] + L.ln1_b[c];
      At[c * TS + r] += acc[nt][e] * dsilu_f(x1);   // g_x1
    }
  }
  __syncthreads();
  if (tid < TA) {
    const int r = tid;
    float rs = rstd1[r];
    float s1 = 0.f, s2 = 0.f;
    for (int k = 0; k < kF; ++k) {
      float gy = At[k * TS + r] * L.ln1_s[k];
      s1 += gy; s2 = fmaf(gy, Ct[k * TS + r], s2);
    }
    s1 *= (1.f / kF); s2 *= (1.f / kF);
    for (int k = 0; k < kF; ++k) {
      float gy = At[k * TS + r] * L.ln1_s[k];
      At[k * TS + r] = rs * (gy - s1 - Ct[k * TS + r] * s2);
    }
  }
  __syncthreads();
  store_tile_T<kF>(g_xa, At, row0, n);
}

// ------------------------------------------------------------------------------------------------
// output heads, forward: per-atom NN energy, raw partial charge, Hirshfeld ratio
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NT) heads_fwd_mma_kernel(ModelDev M, int n, const int* __restrict__ Z, const float* __restrict__ x,
                                                           float* __restrict__ ze, float* __restrict__ zq, float* __restrict__ zh,
                                                           float* __restrict__ e_nn, float* __restrict__ q_raw,
                                                           float* __restrict__ hv /* signed Hirshfeld pre-abs value */) {
  extern __shared__ float sm[];
  float* At = sm;
  float* Bt = At + kF * TS;
  const int row0 = blockIdx.x * TA;
  const Frag fr;
  load_tile_T<kF>(At, x, row0, n);
  __syncthreads();
  float acc[16][4];
  // energy and charge heads share the structure Dense(128) -> silu -> dot
#pragma unroll 1
  for (int head = 0; head < 2; ++head) {
    const uint4* Wf = head == 0 ? M.e_reg_f : M.q_reg_f;
    const float* bias = head == 0 ? M.e_reg_b : M.q_reg_b;
    const float* fin = head == 0 ? M.e_fin_k : M.q_fin_k;
    float* zout = head == 0 ? ze : zq;
    gemm_mma<kF, kF, false>(At, Wf, acc);
    float part[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = fr.row(e), c = fr.col(nt, e);
        const float z = acc[nt][e] + bias[c];
        if (row0 + r < n) zout[(size_t)(row0 + r) * kF + c] = z;
        part[e >> 1] = fmaf(silu_f(z), fin[c], part[e >> 1]);
      }
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      const float s = quad_sum(part[h2]);
      const int a = row0 + fr.row(2 * h2);
      if (fr.q == 0 && a < n) {
        int z = Z[a];
        if (head == 0) {
          z = z < 0 ? 0 : (z >= kZEmbed ? kZEmbed - 1 : z);
          e_nn[a] = (s + M.e_fin_b) * M.e_scale[z] + M.e_offset[z];
        } else {
          z = z < 0 ? 0 : (z >= kZHead ? kZHead - 1 : z);
          q_raw[a] = s + M.q_fin_b + M.q_embed[z];
        }
      }
    }
  }
  // Hirshfeld: 128 -> 64 -> 64, then dot with the element query
  float acc8[8][4];
  gemm_mma<kF, 64, false>(At, M.h_reg_f, acc8);
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = fr.row(e), c = fr.col(nt, e);
      const float z = acc8[nt][e] + M.h_reg_b[c];
      if (row0 + r < n) zh[(size_t)(row0 + r) * 64 + c] = z;
      Bt[c * TS + r] = silu_f(z);
    }
  }
  __syncwarp();
  gemm_mma<64, 64, false>(Bt, M.h_fin_f, acc8);
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    const int a = row0 + fr.row(2 * h2);
    int z = 0;
    if (a < n) { z = Z[a]; z = z < 0 ? 0 : (z >= kZHead ? kZHead - 1 : z); }
    float s = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e1 = 0; e1 < 2; ++e1) {
        const int c = fr.col(nt, e1);
        s = fmaf(acc8[nt][2 * h2 + e1] + M.h_fin_b[c], M.h_embed1[z * 64 + c], s);
      }
    }
    s = quad_sum(s);
    if (fr.q == 0 && a < n) hv[a] = M.h_embed0[z] + s * 0.125f;
  }
}

// heads reverse: gx = dL/dx_final from cotangents of e_nn (ge), raw charge (gq) and Hirshfeld ratio (gh)
__global__ void __launch_bounds__(NT) heads_bwd_mma_kernel(ModelDev M, int n, const int* __restrict__ Z, const float* __restrict__ ze,
                                                           const float* __restrict__ zq, const float* __restrict__ zh,
                                                           const float* __restrict__ hv, const float* __restrict__ ge,
                                                           const float* __restrict__ gq, const float* __restrict__ gh,
                                                           float* __restrict__ gx) {
  extern __shared__ float sm[];
  float* At = sm;
  float* Bt = At + kF * TS;
  float* coef = Bt + kF * TS;     // 64*3 : ge*scale, gq, gh*sign/8
  int* zrow = reinterpret_cast<int*>(coef + TA * 3);
  const int tid = threadIdx.x;
  const int row0 = blockIdx.x * TA;
  const Frag fr;
  if (tid < TA) {
    int a = row0 + tid;
    float c0 = 0.f, c1 = 0.f, c2 = 0.f;
    int zz = 0;
    if (a < n) {
      int z = Z[a];
      int ze_ = z < 0 ? 0 : (z >= kZEmbed ? kZEmbed - 1 : z);
      zz = z < 0 ? 0 : (z >= kZHead ? kZHead - 1 : z);
      c0 = ge[a] * M.e_scale[ze_];
      c1 = gq[a];
      c2 = gh[a] * (hv[a] < 0.f ? -0.125f : 0.125f);
    }
    coef[tid * 3 + 0] = c0; coef[tid * 3 + 1] = c1; coef[tid * 3 + 2] = c2; zrow[tid] = zz;
  }
  __syncthreads();
  // Hirshfeld branch first: g_k[c] = c2 * embed1[z][c] -> g_sh = g_k Hfin^T -> g_zh = g_sh * dsilu(zh)
  for (int idx = tid; idx < TA * 64; idx += NT) {
    int r = idx & 63, c = idx >> 6;
    At[c * TS + r] = coef[r * 3 + 2] * M.h_embed1[zrow[r] * 64 + c];
  }
  __syncthreads();
  float acc8[8][4];
  gemm_mma<64, 64, false>(At, M.h_finT_f, acc8);
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = fr.row(e), c = fr.col(nt, e);
      const float z = (row0 + r < n) ? zh[(size_t)(row0 + r) * 64 + c] : 0.f;
      Bt[c * TS + r] = acc8[nt][e] * dsilu_f(z);
    }
  }
  __syncwarp();
  float acc[16][4];
  gemm_mma<64, kF, false>(Bt, M.h_regT_f, acc);
  __syncthreads();
  // energy branch
  for (int idx = tid; idx < TA * kF; idx += NT) {
    int r = idx & 63, c = idx >> 6;
    float z = (row0 + r < n) ? ze[(size_t)(row0 + r) * kF + c] : 0.f;
    At[c * TS + r] = coef[r * 3 + 0] * M.e_fin_k[c] * dsilu_f(z);
  }
  __syncthreads();
  gemm_mma<kF, kF, true>(At, M.e_regT_f, acc);
  __syncthreads();
  for (int idx = tid; idx < TA * kF; idx += NT) {
    int r = idx & 63, c = idx >> 6;
    float z = (row0 + r < n) ? zq[(size_t)(row0 + r) * kF + c] : 0.f;
    At[c * TS + r] = coef[r * 3 + 1] * M.q_fin_k[c] * dsilu_f(z);
  }
  __syncthreads();
  gemm_mma<kF, kF, true>(At, M.q_regT_f, acc);
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < 16; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) Bt[fr.col(nt, e) * TS + fr.row(e)] = acc[nt][e];
  __syncthreads();
  store_tile_T<kF>(gx, Bt, row0, n);
}

// ------------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------------
static constexpr size_t kSmemPostFwd = (size_t)(2 * kF * TS + 2 * TA * 4) * sizeof(float);
static constexpr size_t kSmemPostBwd = (size_t)(3 * kF * TS + 2 * TA * 4 + TA) * sizeof(float);
static constexpr size_t kSmemHeads = (size_t)(2 * kF * TS + TA * 4) * sizeof(float);

int configure_atom_mma_kernels() {
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(atom_post_fwd_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemPostFwd));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(atom_post_bwd_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemPostBwd));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(heads_fwd_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemHeads));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(heads_bwd_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemHeads));
  return kOk;
}

void launch_atom_post_fwd_mma(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, float* z1, float* x3,
                              float* gate, float* x4, float* ev2, const uint4* proj_next, float* qkv_next) {
  if (n <= 0) return;
  { atom_post_fwd_mma_kernel<<<(n + TA - 1) / TA, NT, kSmemPostFwd, s>>>(L, n, xa, ev1, z1, x3, gate, x4, ev2, proj_next, qkv_next); count_launch(); }
}
void launch_atom_post_bwd_mma(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, const float* z1,
                              const float* x3, const float* gate, const float* g4, const float* gev2, float* g_xa, float* gev1,
                              const uint4* projT_up, const float* g_qkv_up) {
  if (n <= 0) return;
  { atom_post_bwd_mma_kernel<<<(n + TA - 1) / TA, NT, kSmemPostBwd, s>>>(L, n, xa, ev1, z1, x3, gate, g4, gev2, g_xa, gev1, projT_up, g_qkv_up); count_launch(); }
}
void launch_heads_fwd_mma(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* x, float* ze, float* zq, float* zh,
                          float* e_nn, float* q_raw, float* hv) {
  if (n <= 0) return;
  { heads_fwd_mma_kernel<<<(n + TA - 1) / TA, NT, kSmemHeads, s>>>(M, n, Z, x, ze, zq, zh, e_nn, q_raw, hv); count_launch(); }
}
void launch_heads_bwd_mma(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* ze, const float* zq, const float* zh,
                          const float* hv, const float* ge, const float* gq, const float* gh, float* gx) {
  if (n <= 0) return;
  { heads_bwd_mma_kernel<<<(n + TA - 1) / TA, NT, kSmemHeads, s>>>(M, n, Z, ze, zq, zh, hv, ge, gq, gh, gx); count_launch(); }
}

}  // namespace so3lr

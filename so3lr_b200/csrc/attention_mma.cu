// Attention kernels of layers 1 and 2 (the layers with a spherical filter) with the per-edge filter contractions on the
// tensor cores.  Structure, records and phases are those of attention_sym.cu; what changes is phase B:
//
//   * groups of 16 compacted edges form the M dimension of warp-level MMAs (mma.sync m16n8k16, FP16 inputs, FP32
//     accumulation).  FP32 accuracy comes from a two-term split of both operands, x = hi + lo / 2048 with hi, lo in FP16
//     (lo is stored scaled by 2048 so that it stays in the normal range), and three MMAs per product:
//     hi*hi into one accumulator, hi*lo + lo*hi into a second one that is added with weight 1/2048.  The dropped lo*lo
//     term is below 2^-22 relative.
//   * chain per filter: z = [s, 1] * [k1w; b]   (K padded to 16, accumulator layout = A layout of the next MMA)
//                       w = silu(z) * K2        (K = 32, N = 128), written to a per-warp shared tile in edge-major rows
//                       edge loop in the "lane = 4 features" layout: radial table, logits, sums; dw replaces w in the tile
//                       dhs = dw * K2^T         (backward only; K = 128, N = 32), then silu' and the first layer
//   * the weights are converted once per CTA into fragment order (hi and scaled lo), so every B operand is one
//     conflict-free 128-bit shared load.
#include <cuda_fp16.h>

#include "kernels.h"

namespace so3lr {

namespace {

constexpr int GE = 16;                      // edges per MMA group
constexpr int kSlots = 48;                  // record slots per warp: up to 15 carried over + 32 new, rounded up to a group
constexpr int kFwRec = 36;                  // header 4 | Hermite 4 | invariants 4 | Y 24
constexpr int kBwRec = 40;
constexpr int kWS = 136;                    // row stride of the w / dw tile (floats)
constexpr int FW_WARPS = 12;
constexpr int BW_WARPS = 8;
constexpr float kInvNbar = 1.0f / kAvgNumNeighbors;
constexpr float kRc2 = kCutoffSr * kCutoffSr;
constexpr float kLoScale = 2048.f, kLoInv = 1.f / 2048.f;

__device__ __forceinline__ float invw(int l) {
  return l == 0 ? 0.5773502691896258f : (l == 1 ? 0.4472135954999579f : (l == 2 ? 0.3779644730092272f : 0.3333333333333333f));
}
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float2 ld2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st2(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
__device__ __forceinline__ float4 f4_fma(float a, float4 b, float4 c) {
  return make_float4(fmaf(a, b.x, c.x), fmaf(a, b.y, c.y), fmaf(a, b.z, c.z), fmaf(a, b.w, c.w));
}
__device__ __forceinline__ float4 f4_zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ float dot3(float4 a, float4 b, float4 c) { return a.x * b.x * c.x + a.y * b.y * c.y + a.z * b.z * c.z + a.w * b.w * c.w; }
__device__ __forceinline__ float dot2(float4 a, float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
__device__ __forceinline__ float f4_get(const float4& v, int k) { return k == 0 ? v.x : (k == 1 ? v.y : (k == 2 ? v.z : v.w)); }

// (x, y) -> FP16 pair hi and FP16 pair of the residuals scaled by 2048
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
// main += Ahi*Bhi ; cross += Ahi*Blo + Alo*Bhi   (B fragment packed as {b0hi, b1hi, b0lo, b1lo})
__device__ __forceinline__ void mma3(float (&mainc)[4], float (&cross)[4], const unsigned (&ah)[4], const unsigned (&al)[4], const uint4& b) {
  mma16816(cross, ah[0], ah[1], ah[2], ah[3], b.z, b.w);
  mma16816(cross, al[0], al[1], al[2], al[3], b.x, b.y);
  mma16816(mainc, ah[0], ah[1], ah[2], ah[3], b.x, b.y);
}

__device__ __forceinline__ void hermite_weights(float r, int& g, float4& hv, float4& hd) {
  float t = r * (1.0f / kTableH);
  g = (int)t;
  g = g > kTableGrid - 2 ? kTableGrid - 2 : g;
  t -= (float)g;
  const float t2 = t * t, t3 = t2 * t;
  hv = make_float4(1.f, t3 - 2.f * t2 + t, -2.f * t3 + 3.f * t2, t3 - t2);      // applied to (v0, h m0, v1 - v0, h m1)
  const float ih = 1.0f / kTableH;
  hd = make_float4(0.f, (3.f * t2 - 4.f * t + 1.f) * ih, (-6.f * t2 + 6.f * t) * ih, (3.f * t2 - 2.f * t) * ih);
}

__device__ __forceinline__ void invariants(const float* __restrict__ evi, const float* __restrict__ evj, float* s) {
  float d[kMTot];
#pragma unroll
  for (int c = 0; c < 6; ++c) {
    const float4 a = ld4(evj + 4 * c), b = ld4(evi + 4 * c);
    d[4 * c] = a.x - b.x; d[4 * c + 1] = a.y - b.y; d[4 * c + 2] = a.z - b.z; d[4 * c + 3] = a.w - b.w;
  }
  s[0] = s[1] = s[2] = s[3] = 0.f;
#pragma unroll
  for (int m = 0; m < kMTot; ++m) s[degree_of(m)] = fmaf(d[m], d[m], s[degree_of(m)]);
#pragma unroll
  for (int l = 0; l < 4; ++l) s[l] *= invw(l);
}

// ---- weights in fragment order (shared memory, built once per CTA) ----
// G1[f][ks 2][nt 16][lane]  : B of w = hs * K2_f,        B[k = c][n = t] = K2_f[c][t]
// G2[f][ks 8][nt 4][lane]   : B of dhs = dw * K2_f^T,    B[k = t][n = c] = K2_f[c][t]
// Z1[f][nt 4][lane]         : B of z = [s,1] * [k1w;b],  B[k][n = c], k = 0..3: k1w_f[k][c], k = 4: b_f[c]; {hi, lo} of b0 only
struct SharedWeights {
  uint4* G1;
  uint4* G2;
  uint2* Z1;
  float* kw;     // [f][4][32] + [f][32] biases, FP32 (epilogue of the second GEMM)
};
constexpr int kG1Words = 2 * 2 * 16 * 32 * 4, kG2Words = 2 * 8 * 4 * 32 * 4, kZ1Words = 2 * 4 * 32 * 2, kKwWords = 2 * 4 * 32 + 2 * 32;

template <bool WITH_G2>
__device__ __forceinline__ void build_shared_weights(const LayerDev& L, float* base, SharedWeights& W, int nthreads) {
  W.G1 = reinterpret_cast<uint4*>(base);
  W.G2 = reinterpret_cast<uint4*>(base + kG1Words);
  W.Z1 = reinterpret_cast<uint2*>(base + kG1Words + (WITH_G2 ? kG2Words : 0));
  W.kw = base + kG1Words + (WITH_G2 ? kG2Words : 0) + kZ1Words;
  for (int idx = threadIdx.x; idx < 2 * 2 * 16 * 32; idx += nthreads) {
    const int lane = idx & 31, nt = (idx >> 5) & 15, ks = (idx >> 9) & 1, f = idx >> 10;
    const int g = lane >> 2, q = lane & 3;
    const float* K2 = L.sph2_k + f * 32 * kF;
    const int c0 = 16 * ks + 2 * q, t = 8 * nt + g;
    uint4 v;
    split2(K2[c0 * kF + t], K2[(c0 + 1) * kF + t], v.x, v.z);
    split2(K2[(c0 + 8) * kF + t], K2[(c0 + 9) * kF + t], v.y, v.w);
    W.G1[idx] = v;
  }
  if (WITH_G2) {
    for (int idx = threadIdx.x; idx < 2 * 8 * 4 * 32; idx += nthreads) {
      const int lane = idx & 31, nt = (idx >> 5) & 3, ks = (idx >> 7) & 7, f = idx >> 10;
      const int g = lane >> 2, q = lane & 3;
      const float* K2 = L.sph2_k + f * 32 * kF;
      const int c = 8 * nt + g, t0 = 16 * ks + 2 * q;
      uint4 v;
      split2(K2[c * kF + t0], K2[c * kF + t0 + 1], v.x, v.z);
      split2(K2[c * kF + t0 + 8], K2[c * kF + t0 + 9], v.y, v.w);
      W.G2[idx] = v;
    }
  }
  for (int idx = threadIdx.x; idx < 2 * 4 * 32; idx += nthreads) {
    const int lane = idx & 31, nt = (idx >> 5) & 3, f = idx >> 7;
    const int g = lane >> 2, q = lane & 3;
    const int c = 8 * nt + g, k0 = 2 * q;
    auto wk = [&](int k) -> float {
      if (k < 4) return L.sph1_k[(f * 4 + k) * 32 + c];
      if (k == 4) return L.sph1_b[f * 32 + c];
      return 0.f;
    };
    uint2 v;
    split2(wk(k0), wk(k0 + 1), v.x, v.y);
    W.Z1[idx] = v;
  }
  for (int idx = threadIdx.x; idx < kKwWords; idx += nthreads) W.kw[idx] = idx < 256 ? L.sph1_k[idx] : L.sph1_b[idx - 256];
}

// Spherical filter of one group of 16 edges and one filter f: hidden pre-activations by MMA, silu, then w = hs * K2 into
// the tile (rows = edges, 128 columns).  dsl (optional) receives silu'(z) in accumulator layout [nt][4].
template <bool WITH_DERIV>
__device__ __forceinline__ void spherical_filter_mma(const SharedWeights& W, int f, const float* rec, int rec_stride, int s_off, int g0,
                                                     int lane, float* wtile, float (*dsl)[4]) {
  const int g = lane >> 2, q = lane & 3;
  // A of the first MMA: rows = edges, columns 0..3 = invariants, column 4 = 1 (bias), rest 0
  unsigned ah[4] = {0u, 0u, 0u, 0u}, al[4] = {0u, 0u, 0u, 0u};
  if (q < 2) {
    const float2 s0 = ld2(rec + (g0 + g) * rec_stride + s_off + 2 * q), s1 = ld2(rec + (g0 + g + 8) * rec_stride + s_off + 2 * q);
    split2(s0.x, s0.y, ah[0], al[0]);
    split2(s1.x, s1.y, ah[1], al[1]);
  } else if (q == 2) {
    split2(1.f, 0.f, ah[0], al[0]);
    ah[1] = ah[0]; al[1] = al[0];
  }
  unsigned hh[2][4], hl[2][4];   // A fragments of the second MMA, k-steps 0 and 1
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    float zm[4] = {0.f, 0.f, 0.f, 0.f}, zx[4] = {0.f, 0.f, 0.f, 0.f};
    const uint2 b = W.Z1[(f * 4 + nt) * 32 + lane];
    const uint4 bb = make_uint4(b.x, 0u, b.y, 0u);
    mma3(zm, zx, ah, al, bb);
    float hv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float z = fmaf(zx[k], kLoInv, zm[k]);
      const float sg = 1.f / (1.f + __expf(-z));
      hv[k] = z * sg;
      if (WITH_DERIV) dsl[nt][k] = sg * (1.f + z * (1.f - sg));
    }
    // accumulator (rows g, g+8; columns 8nt+2q, +1) = A fragment entries of k-step nt/2: (a0,a1) for even nt, (a2,a3) for odd
    const int ks = nt >> 1, o = (nt & 1) * 2;
    split2(hv[0], hv[1], hh[ks][o], hl[ks][o]);
    split2(hv[2], hv[3], hh[ks][o + 1], hl[ks][o + 1]);
  }
  // w = hs * K2_f, one head (4 n-tiles) at a time
#pragma unroll 1
  for (int h = 0; h < 4; ++h) {
    float wm[4][4], wx[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int k = 0; k < 4; ++k) { wm[n][k] = 0.f; wx[n][k] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const uint4 b = W.G1[((f * 2 + ks) * 16 + 4 * h + n) * 32 + lane];
        mma3(wm[n], wx[n], hh[ks], hl[ks], b);
      }
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      float* p = wtile + g * kWS + 32 * h + 8 * n + 2 * q;
      st2(p, make_float2(fmaf(wx[n][0], kLoInv, wm[n][0]), fmaf(wx[n][1], kLoInv, wm[n][1])));
      st2(p + 8 * kWS, make_float2(fmaf(wx[n][2], kLoInv, wm[n][2]), fmaf(wx[n][3], kLoInv, wm[n][3])));
    }
  }
}

// everything the edge loop reads from global memory for one edge and one filter
struct FwEdge { float4 hv, v0, m0, v1, m1, kf, vj; float sc; };
__device__ __forceinline__ FwEdge fw_load_edge(const float* rec, int slot, int f, int col, const float* __restrict__ table,
                                               const float* __restrict__ qkv) {
  FwEdge e;
  const float* rp = rec + slot * kFwRec;
  const float4 r0 = ld4(rp);
  e.hv = ld4(rp + 4);
  e.sc = r0.y;
  const float* p0 = table + (size_t)__float_as_int(r0.z) * 1024 + f * kF + col;
  e.v0 = ld4(p0); e.m0 = ld4(p0 + 256); e.v1 = ld4(p0 + 512); e.m1 = ld4(p0 + 768);
  const float* kj = qkv + (size_t)__float_as_int(r0.x) * kProj;
  e.kf = ld4(kj + (f ? 4 * kF : kF) + col);
  e.vj = f ? f4_zero() : ld4(kj + 2 * kF + col);
  return e;
}
struct BwEdge { float4 hv, hd, v0, m0, v1, m1, qj, kj, vj, gxj; float sc, dcn; };
__device__ __forceinline__ BwEdge bw_load_edge(const float* rec, int slot, int f, int col, const float* __restrict__ table,
                                               const float* __restrict__ qkv, const float* __restrict__ g_xa) {
  BwEdge e;
  const float* rp = rec + slot * kBwRec;
  const float4 r0 = ld4(rp);
  e.hv = ld4(rp + 4); e.hd = ld4(rp + 8);
  e.sc = r0.y; e.dcn = r0.w;
  const int j2 = __float_as_int(r0.x);
  const float* p0 = table + (size_t)__float_as_int(r0.z) * 1024 + f * kF + col;
  e.v0 = ld4(p0); e.m0 = ld4(p0 + 256); e.v1 = ld4(p0 + 512); e.m1 = ld4(p0 + 768);
  const float* kj = qkv + (size_t)j2 * kProj + f * 3 * kF;
  e.qj = ld4(kj + col); e.kj = ld4(kj + kF + col);
  if (f == 0) { e.vj = ld4(kj + 2 * kF + col); e.gxj = ld4(g_xa + (size_t)j2 * kF + col); }
  else { e.vj = f4_zero(); e.gxj = f4_zero(); }
  return e;
}

// ------------------------------------------------------------------------------------------------------------------
// forward (layers with a spherical filter)
// ------------------------------------------------------------------------------------------------------------------
constexpr int kFwWarpFloats = kSlots * kFwRec + GE * kWS;
constexpr int kFwSharedW = kG1Words + kZ1Words + kKwWords;

__global__ void __launch_bounds__(FW_WARPS * 32, 1) attn_fwd_mma_kernel(LayerDev L, int n_recv, int n, const int* __restrict__ row_ptr,
                                                                        const int* __restrict__ nbr_j, const float* __restrict__ dR,
                                                                        const float* __restrict__ qkv, const float* __restrict__ x_in,
                                                                        const float* __restrict__ ev_in, float* __restrict__ xa,
                                                                        float* __restrict__ ev1) {
  extern __shared__ float4 sm4[];
  float* sm = reinterpret_cast<float*>(sm4);
  SharedWeights W;
  build_shared_weights<false>(L, sm, W, FW_WARPS * 32);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* rec = sm + ((kFwSharedW + 3) & ~3) + warp * kFwWarpFloats;
  float* wt = rec + kSlots * kFwRec;
  const int col = 4 * lane;
  const int deg = degree_of(lane < kMTot ? lane : 0);
  for (int tile = blockIdx.x; tile * FW_WARPS < n_recv; tile += gridDim.x) {
    const int i = tile * FW_WARPS + warp;
    if (i >= n_recv) continue;
    const float* qi = qkv + (size_t)i * kProj;
    const float4 q1 = ld4(qi + col), q2 = ld4(qi + 3 * kF + col);
    float4 accx = f4_zero();
    float accev = 0.f;
    const int e0 = row_ptr[i], e1 = row_ptr[i + 1];
    int rem = 0;
    for (int eb = e0; eb < e1; eb += 32) {
      // ---- phase A ----
      const int e = eb + lane;
      const bool in = e < e1;
      const int j = in ? nbr_j[e] : -1;
      float dx = 0.f, dy = 0.f, dz = 0.f;
      if (in) { dx = dR[3 * (size_t)e]; dy = dR[3 * (size_t)e + 1]; dz = dR[3 * (size_t)e + 2]; }
      const float r2 = dx * dx + dy * dy + dz * dz;
      const bool valid = in && j >= 0 && j < n && r2 < kRc2 && r2 > 0.f;
      const unsigned mask = __ballot_sync(0xffffffffu, valid);
      const int total = rem + __popc(mask);
      const bool last = eb + 32 >= e1;
      const int nproc = last ? ((total + GE - 1) & ~(GE - 1)) : (total & ~(GE - 1));
      if (valid) {
        const int p = rem + __popc(mask & ((1u << lane) - 1u));
        const float r = sqrtf(r2), ir = 1.f / r;
        float cut, dcut;
        phys_cutoff(r, cut, dcut);
        int g; float4 hv, hd;
        hermite_weights(r, g, hv, hd);
        float s[4];
        invariants(ev_in + (size_t)i * kMTot, ev_in + (size_t)j * kMTot, s);
        float Y[kMTot];
        sph_harm_24(dx * ir, dy * ir, dz * ir, Y);
        float* rp = rec + p * kFwRec;
        st4(rp, make_float4(__int_as_float(j), cut * kInvNbar, __int_as_float(g), 0.f));
        st4(rp + 4, hv);
        st4(rp + 8, make_float4(s[0], s[1], s[2], s[3]));
#pragma unroll
        for (int c = 0; c < 6; ++c) st4(rp + 12 + 4 * c, make_float4(Y[4 * c], Y[4 * c + 1], Y[4 * c + 2], Y[4 * c + 3]));
      }
      if (total + lane < nproc) {   // padding slots of the row's last group: a harmless edge to atom i with zero weight
        float* rp = rec + (total + lane) * kFwRec;
        st4(rp, make_float4(__int_as_float(i), 0.f, __int_as_float(0), 0.f));
#pragma unroll
        for (int c = 1; c < 9; ++c) st4(rp + 4 * c, f4_zero());
      }
      __syncwarp();
      // ---- phase B ----
      for (int g0 = 0; g0 < nproc; g0 += GE) {
#pragma unroll 1
        for (int f = 0; f < 2; ++f) {
          spherical_filter_mma<false>(W, f, rec, kFwRec, 8, g0, lane, wt, nullptr);
          __syncwarp();
          const float4 qf = f ? q2 : q1;
          // loads of edge k+1 are issued before the arithmetic of edge k (the warp has few siblings to hide latency behind)
          FwEdge cur = fw_load_edge(rec, g0, f, col, L.table, qkv);
          FwEdge nx1 = fw_load_edge(rec, g0 + 1, f, col, L.table, qkv);
#pragma unroll 4
          for (int k = 0; k < GE; ++k) {
            FwEdge nx2 = nx1;                   // loads run two edges ahead of the arithmetic
            if (k + 2 < GE) nx2 = fw_load_edge(rec, g0 + k + 2, f, col, L.table, qkv);
            const float4 w = f4_fma(cur.hv.x, cur.v0, f4_fma(cur.hv.y, cur.m0, f4_fma(cur.hv.z, cur.v1, f4_fma(cur.hv.w, cur.m1, ld4(wt + k * kWS + col)))));
            const float a = group8_sum(dot3(qf, w, cur.kf)) * cur.sc;
            if (f == 0) {
              accx = f4_fma(a, cur.vj, accx);
            } else {
              const float ym = lane < kMTot ? rec[(g0 + k) * kFwRec + 12 + lane] : 0.f;
              accev = fmaf(__shfl_sync(0xffffffffu, a, 8 * deg), ym, accev);
            }
            cur = nx1; nx1 = nx2;
          }
          __syncwarp();
        }
      }
      __syncwarp();
      rem = total - nproc;
      if (rem > 0 && nproc > 0) {
        for (int q = lane; q < rem * (kFwRec / 4); q += 32) st4(rec + 4 * q, ld4(rec + nproc * kFwRec + 4 * q));
        __syncwarp();
      }
    }
    const float4 xi = ld4(x_in + (size_t)i * kF + col);
    st4(xa + (size_t)i * kF + col, make_float4(xi.x + accx.x, xi.y + accx.y, xi.z + accx.z, xi.w + accx.w));
    if (lane < kMTot) ev1[(size_t)i * kMTot + lane] = ev_in[(size_t)i * kMTot + lane] + accev;
  }
}

// ------------------------------------------------------------------------------------------------------------------
// backward (layers with a spherical filter)
// ------------------------------------------------------------------------------------------------------------------
// record fields (floats): 0 j | 1 sc | 2 table index | 3 dcut/nbar | 4-7 Hermite value weights | 8-11 derivative weights |
// 12-15 invariants, later their cotangents | 16-19 da of edge (i<-j), filter 2 | 20-23 da of edge (j<-i), filter 2 |
// 24-27 a2 (i<-j) | 28-31 a2 (j<-i) | 32-34 unit vector | 35 1/r | 36 d/dr
constexpr int kBwWarpFloats = kSlots * kBwRec + GE * kWS;
constexpr int kBwSharedW = kG1Words + kG2Words + kZ1Words + kKwWords;

__global__ void __launch_bounds__(BW_WARPS * 32, 1) attn_bwd_mma_kernel(LayerDev L, int n_recv, int n, const int* __restrict__ row_ptr,
                                                                        const int* __restrict__ nbr_j, const float* __restrict__ dR,
                                                                        const float* __restrict__ qkv, const float* __restrict__ ev_in,
                                                                        const float* __restrict__ g_xa, const float* __restrict__ gev1,
                                                                        float* __restrict__ g_qkv, float* __restrict__ gev_in,
                                                                        float* __restrict__ F, float* __restrict__ virial) {
  extern __shared__ float4 sm4[];
  float* sm = reinterpret_cast<float*>(sm4);
  SharedWeights W;
  build_shared_weights<true>(L, sm, W, BW_WARPS * 32);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* rec = sm + ((kBwSharedW + 3) & ~3) + warp * kBwWarpFloats;
  float* wt = rec + kSlots * kBwRec;
  const int col = 4 * lane, grp = lane >> 3, cg = lane & 7;
  const int g = lane >> 2, q = lane & 3;
  const int deg = degree_of(lane < kMTot ? lane : 0);
  for (int tile = blockIdx.x; tile * BW_WARPS < n_recv; tile += gridDim.x) {
    const int i = tile * BW_WARPS + warp;
    if (i >= n_recv) continue;
    const float* qi = qkv + (size_t)i * kProj;
    float4 qa = ld4(qi + col), ka = ld4(qi + kF + col), qb = ld4(qi + 3 * kF + col), kb = ld4(qi + 4 * kF + col);
    const float4 v_i = ld4(qi + 2 * kF + col);
    const float4 gx_i = ld4(g_xa + (size_t)i * kF + col);
    const float* gevi = gev1 + (size_t)i * kMTot;
    const float* evi = ev_in + (size_t)i * kMTot;
    float4 gqa = f4_zero(), gka = f4_zero(), gqb = f4_zero(), gkb = f4_zero(), gv = f4_zero();
    float gevacc = 0.f, fx = 0.f, fy = 0.f, fz = 0.f;
    const float evi_m = lane < kMTot ? evi[lane] : 0.f;
    const int e0 = row_ptr[i], e1 = row_ptr[i + 1];
    int rem = 0;
    for (int eb = e0; eb < e1; eb += 32) {
      // ---- phase A: lane = list entry ----
      const int e = eb + lane;
      const bool in = e < e1;
      const int j = in ? nbr_j[e] : -1;
      float dx = 0.f, dy = 0.f, dz = 0.f;
      if (in) { dx = dR[3 * (size_t)e]; dy = dR[3 * (size_t)e + 1]; dz = dR[3 * (size_t)e + 2]; }
      const float r2 = dx * dx + dy * dy + dz * dz;
      const bool valid = in && j >= 0 && j < n && r2 < kRc2 && r2 > 0.f;
      const unsigned mask = __ballot_sync(0xffffffffu, valid);
      const int total = rem + __popc(mask);
      const bool last = eb + 32 >= e1;
      const int nproc = last ? ((total + GE - 1) & ~(GE - 1)) : (total & ~(GE - 1));
      if (valid) {
        const int p = rem + __popc(mask & ((1u << lane) - 1u));
        const float r = sqrtf(r2), ir = 1.f / r;
        const float ux = dx * ir, uy = dy * ir, uz = dz * ir;
        float cut, dcut;
        phys_cutoff(r, cut, dcut);
        int gi; float4 hv, hd;
        hermite_weights(r, gi, hv, hd);
        float s[4];
        invariants(evi, ev_in + (size_t)j * kMTot, s);
        float Y[kMTot];
        sph_harm_24(ux, uy, uz, Y);
        float dA[4] = {0.f, 0.f, 0.f, 0.f}, dB[4] = {0.f, 0.f, 0.f, 0.f};
        const float* gevj = gev1 + (size_t)j * kMTot;
#pragma unroll
        for (int c = 0; c < 6; ++c) {
          const float4 a = ld4(gevi + 4 * c), b = ld4(gevj + 4 * c);
          dA[degree_of(4 * c)] = fmaf(a.x, Y[4 * c], dA[degree_of(4 * c)]);
          dA[degree_of(4 * c + 1)] = fmaf(a.y, Y[4 * c + 1], dA[degree_of(4 * c + 1)]);
          dA[degree_of(4 * c + 2)] = fmaf(a.z, Y[4 * c + 2], dA[degree_of(4 * c + 2)]);
          dA[degree_of(4 * c + 3)] = fmaf(a.w, Y[4 * c + 3], dA[degree_of(4 * c + 3)]);
          dB[degree_of(4 * c)] = fmaf(b.x, Y[4 * c], dB[degree_of(4 * c)]);
          dB[degree_of(4 * c + 1)] = fmaf(b.y, Y[4 * c + 1], dB[degree_of(4 * c + 1)]);
          dB[degree_of(4 * c + 2)] = fmaf(b.z, Y[4 * c + 2], dB[degree_of(4 * c + 2)]);
          dB[degree_of(4 * c + 3)] = fmaf(b.w, Y[4 * c + 3], dB[degree_of(4 * c + 3)]);
        }
        dB[0] = -dB[0]; dB[2] = -dB[2];   // Y_lm(-u) = (-1)^l Y_lm(u)
        float* rp = rec + p * kBwRec;
        st4(rp, make_float4(__int_as_float(j), cut * kInvNbar, __int_as_float(gi), dcut * kInvNbar));
        st4(rp + 4, hv);
        st4(rp + 8, hd);
        st4(rp + 12, make_float4(s[0], s[1], s[2], s[3]));
        st4(rp + 16, make_float4(dA[0], dA[1], dA[2], dA[3]));
        st4(rp + 20, make_float4(dB[0], dB[1], dB[2], dB[3]));
        st4(rp + 32, make_float4(ux, uy, uz, ir));
      }
      if (total + lane < nproc) {
        float* rp = rec + (total + lane) * kBwRec;
        st4(rp, make_float4(__int_as_float(i), 0.f, __int_as_float(0), 0.f));
#pragma unroll
        for (int c = 1; c < 9; ++c) st4(rp + 4 * c, f4_zero());
      }
      __syncwarp();
      // ---- phase B ----
      for (int g0 = 0; g0 < nproc; g0 += GE) {
        float dsp[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};   // d/d invariants of edges g0+g and g0+g+8, partial over 8 hidden units
#pragma unroll 1
        for (int f = 0; f < 2; ++f) {
          float dsl[4][4];
          spherical_filter_mma<true>(W, f, rec, kBwRec, 12, g0, lane, wt, dsl);
          __syncwarp();
          BwEdge cur = bw_load_edge(rec, g0, f, col, L.table, qkv, g_xa);
          BwEdge nx1 = bw_load_edge(rec, g0 + 1, f, col, L.table, qkv, g_xa);
          // four edges per trip (the body is large; a fully unrolled loop overflows the instruction cache)
#pragma unroll 1
          for (int k4 = 0; k4 < GE; k4 += 4) {
            float gr4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int k = k4 + u;
              BwEdge nx2 = nx1;                 // loads run two edges ahead of the arithmetic
              if (k + 2 < GE) nx2 = bw_load_edge(rec, g0 + k + 2, f, col, L.table, qkv, g_xa);
              float* rp = rec + (g0 + k) * kBwRec;
              const float sc = cur.sc, dcn = cur.dcn;
              const float4 wk = f4_fma(cur.hv.x, cur.v0, f4_fma(cur.hv.y, cur.m0, f4_fma(cur.hv.z, cur.v1, f4_fma(cur.hv.w, cur.m1, ld4(wt + k * kWS + col)))));
              const float4 td = f4_fma(cur.hd.x, cur.v0, f4_fma(cur.hd.y, cur.m0, f4_fma(cur.hd.z, cur.v1, f4_fma(cur.hd.w, cur.m1, f4_zero()))));
              const float4 qf_j = cur.qj, kf_j = cur.kj;
              const float DA = group8_sum(dot3(qa, wk, kf_j));
              const float DB = group8_sum(dot3(qf_j, wk, ka));
              float daA, daB;
              if (f == 0) {
                daA = group8_sum(dot2(gx_i, cur.vj));
                daB = group8_sum(dot2(cur.gxj, v_i));
                gv = f4_fma(sc * DB, cur.gxj, gv);
              } else {
                daA = rp[16 + grp];
                daB = rp[20 + grp];
                if (cg == 0) { rp[24 + grp] = sc * DA; rp[28 + grp] = sc * DB; }
              }
              const float dDA = sc * daA, dDB = sc * daB;
              gqa = make_float4(fmaf(dDA * wk.x, kf_j.x, gqa.x), fmaf(dDA * wk.y, kf_j.y, gqa.y), fmaf(dDA * wk.z, kf_j.z, gqa.z),
                                fmaf(dDA * wk.w, kf_j.w, gqa.w));
              gka = make_float4(fmaf(dDB * wk.x, qf_j.x, gka.x), fmaf(dDB * wk.y, qf_j.y, gka.y), fmaf(dDB * wk.z, qf_j.z, gka.z),
                                fmaf(dDB * wk.w, qf_j.w, gka.w));
              const float4 dw = make_float4(fmaf(dDA * qa.x, kf_j.x, dDB * qf_j.x * ka.x), fmaf(dDA * qa.y, kf_j.y, dDB * qf_j.y * ka.y),
                                            fmaf(dDA * qa.z, kf_j.z, dDB * qf_j.z * ka.z), fmaf(dDA * qa.w, kf_j.w, dDB * qf_j.w * ka.w));
              gr4[u] = fmaf(dcn * 0.125f, fmaf(daA, DA, daB * DB), dot2(dw, td));
              st4(wt + k * kWS + col, dw);      // the lane overwrites exactly the words it read: dw takes the place of w
              cur = nx1; nx1 = nx2;
            }
            // d/dr of the four edges: lane partials -> totals; lane (16a + 8b) ends up with edge k4 + 2a + b
            {
              float s0 = (lane & 16) ? gr4[0] : gr4[2], k0 = (lane & 16) ? gr4[2] : gr4[0];
              float s1 = (lane & 16) ? gr4[1] : gr4[3], k1 = (lane & 16) ? gr4[3] : gr4[1];
              k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
              k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
              const float s2 = (lane & 8) ? k0 : k1;
              float v = ((lane & 8) ? k1 : k0) + __shfl_xor_sync(0xffffffffu, s2, 8);
              v += __shfl_xor_sync(0xffffffffu, v, 4); v += __shfl_xor_sync(0xffffffffu, v, 2); v += __shfl_xor_sync(0xffffffffu, v, 1);
              if ((lane & 7) == 0) {
                float* gp = rec + (g0 + k4 + ((lane >> 4) & 1) * 2 + ((lane >> 3) & 1)) * kBwRec + 36;
                *gp = f ? *gp + v : v;
              }
            }
          }
          __syncwarp();
          // dhs = dw * K2_f^T (16 edges x 32 hidden units), then silu' and the first layer: d/ds_l += sum_c dz[c] k1w[l][c]
          {
            float hm[4][4], hx[4][4];
#pragma unroll
            for (int nn = 0; nn < 4; ++nn)
#pragma unroll
              for (int k = 0; k < 4; ++k) { hm[nn][k] = 0.f; hx[nn][k] = 0.f; }
#pragma unroll 2
            for (int ks = 0; ks < 8; ++ks) {
              const float* a0p = wt + g * kWS + 16 * ks + 2 * q;
              const float2 x0 = ld2(a0p), x1 = ld2(a0p + 8 * kWS), x2 = ld2(a0p + 8), x3 = ld2(a0p + 8 * kWS + 8);
              unsigned ah[4], al[4];
              split2(x0.x, x0.y, ah[0], al[0]);
              split2(x1.x, x1.y, ah[1], al[1]);
              split2(x2.x, x2.y, ah[2], al[2]);
              split2(x3.x, x3.y, ah[3], al[3]);
#pragma unroll
              for (int nn = 0; nn < 4; ++nn) {
                const uint4 b = W.G2[((f * 8 + ks) * 4 + nn) * 32 + lane];
                mma3(hm[nn], hx[nn], ah, al, b);
              }
            }
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
              const int c = 8 * nn + 2 * q;
              const float dz00 = fmaf(hx[nn][0], kLoInv, hm[nn][0]) * dsl[nn][0], dz01 = fmaf(hx[nn][1], kLoInv, hm[nn][1]) * dsl[nn][1];
              const float dz10 = fmaf(hx[nn][2], kLoInv, hm[nn][2]) * dsl[nn][2], dz11 = fmaf(hx[nn][3], kLoInv, hm[nn][3]) * dsl[nn][3];
#pragma unroll
              for (int l = 0; l < 4; ++l) {
                const float2 kw = ld2(W.kw + (f * 4 + l) * 32 + c);
                dsp[0][l] = fmaf(dz00, kw.x, fmaf(dz01, kw.y, dsp[0][l]));
                dsp[1][l] = fmaf(dz10, kw.x, fmaf(dz11, kw.y, dsp[1][l]));
              }
            }
          }
          __syncwarp();
          { float4 t = qa; qa = qb; qb = t; t = ka; ka = kb; kb = t; t = gqa; gqa = gqb; gqb = t; t = gka; gka = gkb; gkb = t; }
        }
        // complete d/d invariants over the 4 lanes of a row pair; their record slots take the cotangents
#pragma unroll
        for (int ee = 0; ee < 2; ++ee)
#pragma unroll
          for (int l = 0; l < 4; ++l) {
            float v = dsp[ee][l];
            v += __shfl_xor_sync(0xffffffffu, v, 1); v += __shfl_xor_sync(0xffffffffu, v, 2);
            dsp[ee][l] = v;
          }
        if (q == 0) {
          st4(rec + (g0 + g) * kBwRec + 12, make_float4(dsp[0][0], dsp[0][1], dsp[0][2], dsp[0][3]));
          st4(rec + (g0 + g + 8) * kBwRec + 12, make_float4(dsp[1][0], dsp[1][1], dsp[1][2], dsp[1][3]));
        }
      }
      __syncwarp();
      // ---- phase C: lane = record: angular part and the force on atom i ----
      const int ndone = nproc < total ? nproc : total;
      VirialAcc va;
      for (int slot = lane; slot < ndone; slot += 32) {
        const float* rp = rec + slot * kBwRec;
        const int j2 = __float_as_int(rp[0]);
        const float4 aA = ld4(rp + 24), aB = ld4(rp + 28), uu = ld4(rp + 32);
        const float g_r = rp[36];
        const float* gevj = gev1 + (size_t)j2 * kMTot;
        float gY[kMTot];
#pragma unroll
        for (int c = 0; c < 6; ++c) {
          const float4 a = ld4(gevi + 4 * c), b = ld4(gevj + 4 * c);
          const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
          for (int qq = 0; qq < 4; ++qq) {
            const int m = 4 * c + qq, l = degree_of(m);
            const float sgn = (l == 0 || l == 2) ? -1.f : 1.f;
            gY[m] = f4_get(aA, l) * av[qq] + sgn * f4_get(aB, l) * bv[qq];
          }
        }
        float gux, guy, guz;
        sph_harm_24_vjp(uu.x, uu.y, uu.z, gY, gux, guy, guz);
        const float gd = gux * uu.x + guy * uu.y + guz * uu.z;
        const float fsx = g_r * uu.x + (gux - gd * uu.x) * uu.w;
        const float fsy = g_r * uu.y + (guy - gd * uu.y) * uu.w;
        const float fsz = g_r * uu.z + (guz - gd * uu.z) * uu.w;
        fx += fsx; fy += fsy; fz += fsz;
        if (virial) {
          const float r = 1.f / uu.w;
          va.add(0.5f * r, uu.x, uu.y, uu.z, fsx, fsy, fsz);
        }
      }
      if (virial) va.flush_warp(virial, (size_t)i, lane);
      for (int pp = 0; pp < ndone; ++pp) {
        const float* rp = rec + pp * kBwRec;
        const int j2 = __float_as_int(rp[0]);
        if (lane < kMTot) {
          const float dev = ev_in[(size_t)j2 * kMTot + lane] - evi_m;
          gevacc = fmaf(-2.f * invw(deg) * rp[12 + deg], dev, gevacc);
        }
      }
      __syncwarp();
      rem = total - nproc;
      if (rem > 0 && nproc > 0) {
        for (int qq = lane; qq < rem * (kBwRec / 4); qq += 32) st4(rec + 4 * qq, ld4(rec + nproc * kBwRec + 4 * qq));
        __syncwarp();
      }
    }
    fx = warp_sum(fx); fy = warp_sum(fy); fz = warp_sum(fz);
    if (lane == 0) { F[3 * (size_t)i] += fx; F[3 * (size_t)i + 1] += fy; F[3 * (size_t)i + 2] += fz; }
    float* gi2 = g_qkv + (size_t)i * kProj;
    st4(gi2 + col, gqa); st4(gi2 + kF + col, gka); st4(gi2 + 2 * kF + col, gv);
    st4(gi2 + 3 * kF + col, gqb); st4(gi2 + 4 * kF + col, gkb);
    if (lane < kMTot) gev_in[(size_t)i * kMTot + lane] = gevi[lane] + gevacc;
  }
}

constexpr size_t kSmemFw = (size_t)(((kFwSharedW + 3) & ~3) + FW_WARPS * kFwWarpFloats) * sizeof(float);
constexpr size_t kSmemBw = (size_t)(((kBwSharedW + 3) & ~3) + BW_WARPS * kBwWarpFloats) * sizeof(float);
static_assert(kSmemFw <= 232448 && kSmemBw <= 232448, "shared memory budget of one CTA per SM");

}  // namespace

int configure_attention_mma_kernels() {
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemFw));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBw));
  return kOk;
}

void launch_attn_fwd_mma(cudaStream_t s, const LayerDev& L, int n_recv, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                         const float* qkv, const float* x_in, const float* ev_in, float* xa, float* ev1) {
  if (n_recv <= 0) return;
  int blocks = (n_recv + FW_WARPS - 1) / FW_WARPS;
  if (blocks > sm_count()) blocks = sm_count();
  { attn_fwd_mma_kernel<<<blocks, FW_WARPS * 32, kSmemFw, s>>>(L, n_recv, n, row_ptr, nbr_j, dR, qkv, x_in, ev_in, xa, ev1); count_launch(); }
}

void launch_attn_bwd_mma(cudaStream_t s, const LayerDev& L, int n_recv, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                         const float* qkv, const float* ev_in, const float* g_xa, const float* gev1, float* g_qkv, float* gev_in,
                         float* F, float* virial) {
  if (n_recv <= 0) return;
  int blocks = (n_recv + BW_WARPS - 1) / BW_WARPS;
  if (blocks > sm_count()) blocks = sm_count();
  { attn_bwd_mma_kernel<<<blocks, BW_WARPS * 32, kSmemBw, s>>>(L, n_recv, n, row_ptr, nbr_j, dR, qkv, ev_in, g_xa, gev1, g_qkv, gev_in, F, virial); count_launch(); }
}

}  // namespace so3lr

// Equivariant attention for the fused positions -> forces path: gather-only forward and backward kernels.
//
// One warp owns one receiver atom i and walks its row of the (symmetric) short-range list in chunks of 32 entries:
//   phase A  lane = list entry: distance test, cutoff, Hermite weights of the radial table, per-degree invariants of
//            (ev_j - ev_i), spherical harmonics; the surviving entries are compacted into per-warp shared memory
//            records.  Records that do not fill a group of 8 are carried over to the next chunk, so only the last
//            group of a row is padded.
//   phase B  lane = 4 features: groups of 8 compacted edges share one pass over the spherical-filter weights
//            (register-blocked 8 edges x 8 columns per lane), then the radial table, logits and weighted sums.
// The backward kernel uses the symmetry of the list instead of atomics: while visiting neighbour j, warp i evaluates
// both directed edges (i<-j) and (j<-i) -- they share the distance, the invariants and therefore the whole filter --
// and keeps only the gradient terms that land on atom i (q_i from the first, k_i / v_i from the second, ev_i and R_i
// from both).  Every output row is written once by its own warp: no atomics, no zero fill, bitwise reproducible.
#include "kernels.h"

namespace so3lr {

namespace {

constexpr int EB = 8;                       // edges per pass over the filter weights
constexpr int FW_WARPS = 8;
constexpr int BW_WARPS = 12;
constexpr int kSlots = 40;                  // record slots per warp: up to 7 carried over + 32 new, rounded up to a group
constexpr int kFwRec = 36;                  // floats per compacted edge record, forward: header 4 | Hermite 4 | invariants 4 | Y 24
constexpr int kBwRec = 40;                  // floats per compacted edge record, backward
constexpr int kDwS = 132;                   // row stride of the dw staging buffer
constexpr float kInvNbar = 1.0f / kAvgNumNeighbors;
constexpr float kRc2 = kCutoffSr * kCutoffSr;

__device__ __forceinline__ float invw(int l) {
  return l == 0 ? 0.5773502691896258f : (l == 1 ? 0.4472135954999579f : (l == 2 ? 0.3779644730092272f : 0.3333333333333333f));
}
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float4 f4_fma(float a, float4 b, float4 c) {
  return make_float4(fmaf(a, b.x, c.x), fmaf(a, b.y, c.y), fmaf(a, b.z, c.z), fmaf(a, b.w, c.w));
}
__device__ __forceinline__ float4 f4_zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ float dot3(float4 a, float4 b, float4 c) { return a.x * b.x * c.x + a.y * b.y * c.y + a.z * b.z * c.z + a.w * b.w * c.w; }
__device__ __forceinline__ float dot2(float4 a, float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
__device__ __forceinline__ float f4_get(const float4& v, int k) { return k == 0 ? v.x : (k == 1 ? v.y : (k == 2 ? v.z : v.w)); }

// cubic Hermite weights (value and derivative) on the table interval containing r
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

// per-degree invariants of d = ev_j - ev_i (24 components each, read with 128-bit loads)
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

// hidden layer of the spherical filter for lane c = lane and the 8 edges of a group: silu(z) (and silu'(z)) into hsg
template <bool WITH_DERIV>
__device__ __forceinline__ void hidden_layer(const float* rec, int rec_stride, int s_off, int g0, const float* k1w, float b, int lane,
                                             float* hsg) {
  float hv[EB], dv[EB];
#pragma unroll
  for (int k = 0; k < EB; ++k) {
    const float4 s = ld4(rec + (g0 + k) * rec_stride + s_off);
    const float z = fmaf(s.x, k1w[0], fmaf(s.y, k1w[1], fmaf(s.z, k1w[2], fmaf(s.w, k1w[3], b))));
    const float sg = 1.f / (1.f + __expf(-z));
    hv[k] = z * sg;
    dv[k] = sg * (1.f + z * (1.f - sg));
  }
  st4(hsg + lane * EB, make_float4(hv[0], hv[1], hv[2], hv[3]));
  st4(hsg + lane * EB + 4, make_float4(hv[4], hv[5], hv[6], hv[7]));
  if (WITH_DERIV) {
    st4(hsg + 32 * EB + lane * EB, make_float4(dv[0], dv[1], dv[2], dv[3]));
    st4(hsg + 32 * EB + lane * EB + 4, make_float4(dv[4], dv[5], dv[6], dv[7]));
  }
}

// w[k] (4 columns of this lane, 8 edges) += sum_c hs[c][k] * K2[c][col..col+3]
__device__ __forceinline__ void filter_gemm(const float* __restrict__ K2f, const float* __restrict__ hsg, int col, float4* w) {
#pragma unroll 4
  for (int c = 0; c < 32; ++c) {
    const float4 kk = ld4(K2f + c * kF + col);
    const float4 h0 = ld4(hsg + c * EB), h1 = ld4(hsg + c * EB + 4);
    w[0] = f4_fma(h0.x, kk, w[0]); w[1] = f4_fma(h0.y, kk, w[1]); w[2] = f4_fma(h0.z, kk, w[2]); w[3] = f4_fma(h0.w, kk, w[3]);
    w[4] = f4_fma(h1.x, kk, w[4]); w[5] = f4_fma(h1.y, kk, w[5]); w[6] = f4_fma(h1.z, kk, w[6]); w[7] = f4_fma(h1.w, kk, w[7]);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------------------------
constexpr int kFwWarpFloats = kSlots * kFwRec + 2 * 32 * EB;   // records | hidden activations (2 filters)

template <bool SPH>
__global__ void __launch_bounds__(FW_WARPS * 32, 2) attn_fwd_sym_kernel(LayerDev L, int n_recv, int n, const int* __restrict__ row_ptr,
                                                                        const int* __restrict__ nbr_j, const float* __restrict__ dR,
                                                                        const float* __restrict__ qkv, const float* __restrict__ x_in,
                                                                        const float* __restrict__ ev_in, float* __restrict__ xa,
                                                                        float* __restrict__ ev1) {
  extern __shared__ float4 sm4[];
  float* sm = reinterpret_cast<float*>(sm4);
  float* K2 = sm;   // [2][32][128] when SPH
  if (SPH) {
    for (int idx = threadIdx.x * 4; idx < 2 * 32 * kF; idx += FW_WARPS * 32 * 4) st4(K2 + idx, ld4(L.sph2_k + idx));
    __syncthreads();
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* rec = sm + (SPH ? 2 * 32 * kF : 0) + warp * kFwWarpFloats;
  float* hsg = rec + kSlots * kFwRec;
  const int col = 4 * lane;
  float k1w1[4] = {0.f, 0.f, 0.f, 0.f}, k1w2[4] = {0.f, 0.f, 0.f, 0.f}, b1 = 0.f, b2 = 0.f;
  if (SPH) {
#pragma unroll
    for (int k = 0; k < 4; ++k) { k1w1[k] = L.sph1_k[k * 32 + lane]; k1w2[k] = L.sph1_k[(4 + k) * 32 + lane]; }
    b1 = L.sph1_b[lane]; b2 = L.sph1_b[32 + lane];
  }
  const int deg = degree_of(lane < kMTot ? lane : 0);
  for (int tile = blockIdx.x; tile * FW_WARPS < n_recv; tile += gridDim.x) {
    const int i = tile * FW_WARPS + warp;
    if (i >= n_recv) continue;
    const float* qi = qkv + (size_t)i * kProj;
    const float4 q1 = ld4(qi + col), q2 = ld4(qi + 3 * kF + col);
    float4 accx = f4_zero();
    float accev = 0.f;
    const int e0 = row_ptr[i], e1 = row_ptr[i + 1];
    int rem = 0;   // records carried over from the previous chunk
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
      const int nproc = last ? ((total + EB - 1) & ~(EB - 1)) : (total & ~(EB - 1));
      if (valid) {
        const int p = rem + __popc(mask & ((1u << lane) - 1u));
        const float r = sqrtf(r2), ir = 1.f / r;
        float cut, dcut;
        phys_cutoff(r, cut, dcut);
        int g; float4 hv, hd;
        hermite_weights(r, g, hv, hd);
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        if (SPH) invariants(ev_in + (size_t)i * kMTot, ev_in + (size_t)j * kMTot, s);
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
      for (int g0 = 0; g0 < nproc; g0 += EB) {
        float4 w1[EB], w2[EB];
#pragma unroll
        for (int k = 0; k < EB; ++k) { w1[k] = f4_zero(); w2[k] = f4_zero(); }
        if (SPH) {
          hidden_layer<false>(rec, kFwRec, 8, g0, k1w1, b1, lane, hsg);
          hidden_layer<false>(rec, kFwRec, 8, g0, k1w2, b2, lane, hsg + 32 * EB);
          __syncwarp();
          filter_gemm(K2, hsg, col, w1);
          filter_gemm(K2 + 32 * kF, hsg + 32 * EB, col, w2);
          __syncwarp();
        }
#pragma unroll
        for (int k = 0; k < EB; ++k) {
          const float* rp = rec + (g0 + k) * kFwRec;
          const float4 r0 = ld4(rp), hv = ld4(rp + 4);
          const int j2 = __float_as_int(r0.x), g = __float_as_int(r0.z);
          const float sc = r0.y;
          const float* p0 = L.table + (size_t)g * 1024 + col;
          {
            const float4 v0 = ld4(p0), m0 = ld4(p0 + 256), v1 = ld4(p0 + 512), m1 = ld4(p0 + 768);
            w1[k] = f4_fma(hv.x, v0, f4_fma(hv.y, m0, f4_fma(hv.z, v1, f4_fma(hv.w, m1, w1[k]))));
          }
          {
            const float4 v0 = ld4(p0 + 128), m0 = ld4(p0 + 384), v1 = ld4(p0 + 640), m1 = ld4(p0 + 896);
            w2[k] = f4_fma(hv.x, v0, f4_fma(hv.y, m0, f4_fma(hv.z, v1, f4_fma(hv.w, m1, w2[k]))));
          }
          const float* kj = qkv + (size_t)j2 * kProj;
          const float4 k1 = ld4(kj + kF + col), v1 = ld4(kj + 2 * kF + col), k2 = ld4(kj + 4 * kF + col);
          const float a1 = group8_sum(dot3(q1, w1[k], k1)) * sc;
          const float a2 = group8_sum(dot3(q2, w2[k], k2)) * sc;
          accx = f4_fma(a1, v1, accx);
          const float ym = lane < kMTot ? rp[12 + lane] : 0.f;
          const float a2m = __shfl_sync(0xffffffffu, a2, 8 * deg);
          accev = fmaf(a2m, ym, accev);
        }
      }
      __syncwarp();
      // carry the records that did not fill a group over to the next chunk
      rem = total - nproc;
      if (rem > 0 && nproc > 0) {
        for (int q = lane; q < rem * (kFwRec / 4); q += 32) st4(rec + 4 * q, ld4(rec + nproc * kFwRec + 4 * q));
        __syncwarp();
      }
    }
    const float4 xi = ld4(x_in + (size_t)i * kF + col);
    st4(xa + (size_t)i * kF + col, make_float4(xi.x + accx.x, xi.y + accx.y, xi.z + accx.z, xi.w + accx.w));
    if (lane < kMTot) ev1[(size_t)i * kMTot + lane] = (SPH ? ev_in[(size_t)i * kMTot + lane] : 0.f) + accev;
  }
}

// ------------------------------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------------------------------
// record fields (floats): 0 j | 1 sc | 2 table index | 3 dcut/nbar | 4-7 Hermite value weights | 8-11 derivative weights |
// 12-15 invariants | 16-19 da of edge (i<-j), filter 2 | 20-23 da of edge (j<-i), filter 2 | 24-27 a2 (i<-j) | 28-31 a2 (j<-i) |
// 32-34 unit vector | 35 1/r | 36-39: d/d invariants (written after the group's last read of everything else) ... 36 also
// receives d/dr: the layout below keeps them apart: 36 d/dr, and d/d invariants overwrite the invariants (12-15).
constexpr int kBwWarpFloats = kSlots * kBwRec + 2 * 32 * EB + EB * kDwS;   // records | hidden (silu, silu') | dw staging

template <bool FIRST>
__global__ void __launch_bounds__(BW_WARPS * 32, 1) attn_bwd_sym_kernel(LayerDev L, int n_recv, int n, const int* __restrict__ row_ptr,
                                                                        const int* __restrict__ nbr_j, const float* __restrict__ dR,
                                                                        const float* __restrict__ qkv, const float* __restrict__ ev_in,
                                                                        const float* __restrict__ g_xa, const float* __restrict__ gev1,
                                                                        float* __restrict__ g_qkv, float* __restrict__ gev_in,
                                                                        float* __restrict__ F, float* __restrict__ virial) {
  extern __shared__ float4 sm4[];
  float* sm = reinterpret_cast<float*>(sm4);
  float* K2 = sm;                     // [2][32][128]
  float* K2T = sm + 2 * 32 * kF;      // [2][128][32]
  if (!FIRST) {
    for (int idx = threadIdx.x; idx < 2 * 32 * kF; idx += BW_WARPS * 32) {
      const float v = L.sph2_k[idx];
      K2[idx] = v;
      const int f = idx >> 12, c = (idx >> 7) & 31, t = idx & 127;
      K2T[f * 4096 + t * 32 + c] = v;
    }
    __syncthreads();
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* rec = sm + (FIRST ? 0 : 4 * 32 * kF) + warp * kBwWarpFloats;
  float* hsg = rec + kSlots * kBwRec;
  float* dwb = hsg + 2 * 32 * EB;
  const int col = 4 * lane, grp = lane >> 3;
  const int cg = lane & 7, ep = lane >> 3;      // tile of the second filter GEMM: columns 4cg..4cg+3, edges 2ep, 2ep+1
  const int deg = degree_of(lane < kMTot ? lane : 0);
  for (int tile = blockIdx.x; tile * BW_WARPS < n_recv; tile += gridDim.x) {
    const int i = tile * BW_WARPS + warp;
    if (i >= n_recv) continue;
    const float* qi = qkv + (size_t)i * kProj;
    // "a" = the filter of the current pass, "b" = the other one; swapped after each pass
    float4 qa = ld4(qi + col), ka = ld4(qi + kF + col), qb = ld4(qi + 3 * kF + col), kb = ld4(qi + 4 * kF + col);
    const float4 v_i = ld4(qi + 2 * kF + col);
    const float4 gx_i = ld4(g_xa + (size_t)i * kF + col);
    const float* gevi = gev1 + (size_t)i * kMTot;
    const float* evi = ev_in + (size_t)i * kMTot;
    float4 gqa = f4_zero(), gka = f4_zero(), gqb = f4_zero(), gkb = f4_zero(), gv = f4_zero();
    float gevacc = 0.f, fx = 0.f, fy = 0.f, fz = 0.f;
    const float evi_m = (!FIRST && lane < kMTot) ? evi[lane] : 0.f;
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
      const int nproc = last ? ((total + EB - 1) & ~(EB - 1)) : (total & ~(EB - 1));
      if (valid) {
        const int p = rem + __popc(mask & ((1u << lane) - 1u));
        const float r = sqrtf(r2), ir = 1.f / r;
        const float ux = dx * ir, uy = dy * ir, uz = dz * ir;
        float cut, dcut;
        phys_cutoff(r, cut, dcut);
        int g; float4 hv, hd;
        hermite_weights(r, g, hv, hd);
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        if (!FIRST) invariants(evi, ev_in + (size_t)j * kMTot, s);
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
        // Y_lm(-u) = (-1)^l Y_lm(u): degrees 1 and 3 change sign on the reversed edge
        dB[0] = -dB[0]; dB[2] = -dB[2];
        float* rp = rec + p * kBwRec;
        st4(rp, make_float4(__int_as_float(j), cut * kInvNbar, __int_as_float(g), dcut * kInvNbar));
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
      // ---- phase B: lane = 4 features ----
      for (int g0 = 0; g0 < nproc; g0 += EB) {
        float gr[EB];
#pragma unroll
        for (int k = 0; k < EB; ++k) gr[k] = 0.f;
        float dsp[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};   // d/d invariants, partial over this lane's 4 hidden units
#pragma unroll 1
        for (int f = 0; f < 2; ++f) {
          float4 w[EB];
#pragma unroll
          for (int k = 0; k < EB; ++k) w[k] = f4_zero();
          if (!FIRST) {
            float kw[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) kw[k] = L.sph1_k[(f * 4 + k) * 32 + lane];
            hidden_layer<true>(rec, kBwRec, 12, g0, kw, L.sph1_b[f * 32 + lane], lane, hsg);
            __syncwarp();
            filter_gemm(K2 + f * 32 * kF, hsg, col, w);
          }
#pragma unroll
          for (int k = 0; k < EB; ++k) {
            float* rp = rec + (g0 + k) * kBwRec;
            const float4 r0 = ld4(rp), hv = ld4(rp + 4), hd = ld4(rp + 8);
            const int j2 = __float_as_int(r0.x), g = __float_as_int(r0.z);
            const float sc = r0.y, dcn = r0.w;
            const float* p0 = L.table + (size_t)g * 1024 + f * kF + col;
            const float4 v0 = ld4(p0), m0 = ld4(p0 + 256), v1 = ld4(p0 + 512), m1 = ld4(p0 + 768);
            w[k] = f4_fma(hv.x, v0, f4_fma(hv.y, m0, f4_fma(hv.z, v1, f4_fma(hv.w, m1, w[k]))));
            const float4 td = f4_fma(hd.x, v0, f4_fma(hd.y, m0, f4_fma(hd.z, v1, f4_fma(hd.w, m1, f4_zero()))));
            const float* kj = qkv + (size_t)j2 * kProj + f * 3 * kF;
            const float4 qf_j = ld4(kj + col), kf_j = ld4(kj + kF + col);
            const float4 wk = w[k];
            const float DA = group8_sum(dot3(qa, wk, kf_j));
            const float DB = group8_sum(dot3(qf_j, wk, ka));
            float daA, daB;
            if (f == 0) {
              const float4 v_j = ld4(kj + 2 * kF + col);
              const float4 gx_j = ld4(g_xa + (size_t)j2 * kF + col);
              daA = group8_sum(dot2(gx_i, v_j));
              daB = group8_sum(dot2(gx_j, v_i));
              if (!FIRST) gv = f4_fma(sc * DB, gx_j, gv);
            } else {
              daA = rp[16 + grp];
              daB = rp[20 + grp];
              if (cg == 0) { rp[24 + grp] = sc * DA; rp[28 + grp] = sc * DB; }
            }
            const float dDA = sc * daA, dDB = sc * daB;
            gr[k] = fmaf(dcn * 0.125f, fmaf(daA, DA, daB * DB), gr[k]);
            if (!FIRST) {
              gqa = make_float4(fmaf(dDA * wk.x, kf_j.x, gqa.x), fmaf(dDA * wk.y, kf_j.y, gqa.y), fmaf(dDA * wk.z, kf_j.z, gqa.z),
                                fmaf(dDA * wk.w, kf_j.w, gqa.w));
              gka = make_float4(fmaf(dDB * wk.x, qf_j.x, gka.x), fmaf(dDB * wk.y, qf_j.y, gka.y), fmaf(dDB * wk.z, qf_j.z, gka.z),
                                fmaf(dDB * wk.w, qf_j.w, gka.w));
            }
            const float4 dw = make_float4(fmaf(dDA * qa.x, kf_j.x, dDB * qf_j.x * ka.x), fmaf(dDA * qa.y, kf_j.y, dDB * qf_j.y * ka.y),
                                          fmaf(dDA * qa.z, kf_j.z, dDB * qf_j.z * ka.z), fmaf(dDA * qa.w, kf_j.w, dDB * qf_j.w * ka.w));
            gr[k] += dot2(dw, td);
            if (!FIRST) st4(dwb + k * kDwS + col, dw);
          }
          if (!FIRST) {
            __syncwarp();
            // dhs[e][c] = sum_t dw[e][t] K2[c][t] for the lane's tile (2 edges x 4 hidden units)
            float4 a0 = f4_zero(), a1 = f4_zero();
            const float* kt = K2T + f * 4096 + 4 * cg;
            const float* d0 = dwb + (2 * ep) * kDwS, *d1 = dwb + (2 * ep + 1) * kDwS;
#pragma unroll 2
            for (int t4 = 0; t4 < 32; ++t4) {
              const float4 da = ld4(d0 + 4 * t4), db = ld4(d1 + 4 * t4);
              const float4 k0 = ld4(kt + (4 * t4) * 32), k1 = ld4(kt + (4 * t4 + 1) * 32), k2 = ld4(kt + (4 * t4 + 2) * 32),
                           k3 = ld4(kt + (4 * t4 + 3) * 32);
              a0 = f4_fma(da.x, k0, f4_fma(da.y, k1, f4_fma(da.z, k2, f4_fma(da.w, k3, a0))));
              a1 = f4_fma(db.x, k0, f4_fma(db.y, k1, f4_fma(db.z, k2, f4_fma(db.w, k3, a1))));
            }
            // through silu' and the first layer: d/ds_l += sum_c dz[c] k1w[l][c]
            const float* dsl = hsg + 32 * EB;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              const int c = 4 * cg + cc;
              const float dz0 = f4_get(a0, cc) * dsl[c * EB + 2 * ep], dz1 = f4_get(a1, cc) * dsl[c * EB + 2 * ep + 1];
#pragma unroll
              for (int l = 0; l < 4; ++l) {
                const float kw = L.sph1_k[(f * 4 + l) * 32 + c];
                dsp[0][l] = fmaf(dz0, kw, dsp[0][l]);
                dsp[1][l] = fmaf(dz1, kw, dsp[1][l]);
              }
            }
          }
          __syncwarp();
          // the other filter becomes the current one
          { float4 t = qa; qa = qb; qb = t; t = ka; ka = kb; kb = t; t = gqa; gqa = gqb; gqb = t; t = gka; gka = gkb; gkb = t; }
        }
        if (!FIRST) {
#pragma unroll
          for (int ee = 0; ee < 2; ++ee)
#pragma unroll
            for (int l = 0; l < 4; ++l) {
              float v = dsp[ee][l];
              v += __shfl_xor_sync(0xffffffffu, v, 1); v += __shfl_xor_sync(0xffffffffu, v, 2); v += __shfl_xor_sync(0xffffffffu, v, 4);
              dsp[ee][l] = v;
            }
          if (cg == 0) {   // all reads of the invariants of this group are done: their slots take the cotangents
            st4(rec + (g0 + 2 * ep) * kBwRec + 12, make_float4(dsp[0][0], dsp[0][1], dsp[0][2], dsp[0][3]));
            st4(rec + (g0 + 2 * ep + 1) * kBwRec + 12, make_float4(dsp[1][0], dsp[1][1], dsp[1][2], dsp[1][3]));
          }
        }
#pragma unroll
        for (int k = 0; k < EB; ++k) {
          const float v = warp_sum(gr[k]);
          if (lane == 0) rec[(g0 + k) * kBwRec + 36] = v;
        }
      }
      __syncwarp();
      // ---- phase C: lane = record: angular part and the force on atom i ----
      const int ndone = nproc < total ? nproc : total;   // processed records that are real edges
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
          for (int q = 0; q < 4; ++q) {
            const int m = 4 * c + q, l = degree_of(m);
            const float sgn = (l == 0 || l == 2) ? -1.f : 1.f;
            gY[m] = f4_get(aA, l) * av[q] + sgn * f4_get(aB, l) * bv[q];
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
      if (!FIRST) {
        // lane = component m: d/d ev_i through the invariants, - ds_l * 2 (ev_j - ev_i)_m / sqrt(2l+1)
        for (int pp = 0; pp < ndone; ++pp) {
          const float* rp = rec + pp * kBwRec;
          const int j2 = __float_as_int(rp[0]);
          if (lane < kMTot) {
            const float dev = ev_in[(size_t)j2 * kMTot + lane] - evi_m;
            gevacc = fmaf(-2.f * invw(deg) * rp[12 + deg], dev, gevacc);
          }
        }
      }
      __syncwarp();
      rem = total - nproc;
      if (rem > 0 && nproc > 0) {
        for (int q = lane; q < rem * (kBwRec / 4); q += 32) st4(rec + 4 * q, ld4(rec + nproc * kBwRec + 4 * q));
        __syncwarp();
      }
    }
    fx = warp_sum(fx); fy = warp_sum(fy); fz = warp_sum(fz);
    if (lane == 0) { F[3 * (size_t)i] += fx; F[3 * (size_t)i + 1] += fy; F[3 * (size_t)i + 2] += fz; }
    if (!FIRST) {
      float* gi = g_qkv + (size_t)i * kProj;
      st4(gi + col, gqa); st4(gi + kF + col, gka); st4(gi + 2 * kF + col, gv);
      st4(gi + 3 * kF + col, gqb); st4(gi + 4 * kF + col, gkb);
      if (lane < kMTot) gev_in[(size_t)i * kMTot + lane] = gevi[lane] + gevacc;
    }
  }
}

constexpr size_t kSmemFwSph = (size_t)(2 * 32 * kF + FW_WARPS * kFwWarpFloats) * sizeof(float);
constexpr size_t kSmemFwFirst = (size_t)(FW_WARPS * kFwWarpFloats) * sizeof(float);
constexpr size_t kSmemBw = (size_t)(4 * 32 * kF + BW_WARPS * kBwWarpFloats) * sizeof(float);
constexpr size_t kSmemBwFirst = (size_t)(BW_WARPS * kBwWarpFloats) * sizeof(float);

}  // namespace

int configure_attention_sym_kernels() {
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_sym_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemFwSph));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_sym_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemFwFirst));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_sym_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBw));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_sym_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBwFirst));
  return kOk;
}

void launch_attn_fwd_sym(cudaStream_t s, const LayerDev& L, int n_recv, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                         const float* qkv, const float* x_in, const float* ev_in, float* xa, float* ev1) {
  if (n_recv <= 0) return;
  int blocks = (n_recv + FW_WARPS - 1) / FW_WARPS;
  if (blocks > sm_count() * 2) blocks = sm_count() * 2;
  if (L.has_spherical)
    { attn_fwd_sym_kernel<true><<<blocks, FW_WARPS * 32, kSmemFwSph, s>>>(L, n_recv, n, row_ptr, nbr_j, dR, qkv, x_in, ev_in, xa, ev1); count_launch(); }
  else
    { attn_fwd_sym_kernel<false><<<blocks, FW_WARPS * 32, kSmemFwFirst, s>>>(L, n_recv, n, row_ptr, nbr_j, dR, qkv, x_in, ev_in, xa, ev1); count_launch(); }
}

void launch_attn_bwd_sym(cudaStream_t s, const LayerDev& L, int n_recv, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                         const float* qkv, const float* ev_in, const float* g_xa, const float* gev1, float* g_qkv, float* gev_in,
                         float* F, int first_layer, float* virial) {
  if (n_recv <= 0) return;
  int blocks = (n_recv + BW_WARPS - 1) / BW_WARPS;
  if (blocks > sm_count()) blocks = sm_count();
  if (first_layer)
    { attn_bwd_sym_kernel<true><<<blocks, BW_WARPS * 32, kSmemBwFirst, s>>>(L, n_recv, n, row_ptr, nbr_j, dR, qkv, ev_in, g_xa, gev1, g_qkv, gev_in, F, virial); count_launch(); }
  else
    { attn_bwd_sym_kernel<false><<<blocks, BW_WARPS * 32, kSmemBw, s>>>(L, n_recv, n, row_ptr, nbr_j, dR, qkv, ev_in, g_xa, gev1, g_qkv, gev_in, F, virial); count_launch(); }
}

}  // namespace so3lr

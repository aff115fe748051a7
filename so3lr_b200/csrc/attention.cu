// Equivariant attention of one SO3krates layer over the receiver-sorted short-range graph, forward and backward.
//
// One warp owns one receiver atom i and walks its edges.  Lane L holds features 4L..4L+3 of every 128-wide row
// (one 128-bit load per row), so head h = L / 8 lives on lanes 8h..8h+7 and a per-head dot product is a 3-step
// shuffle reduction.  The radial filters are read from an L2-resident cubic-Hermite table (value and slope per
// grid point); the spherical filter (4 -> 32 -> 128, per edge) is evaluated in registers with its second-layer
// kernel staged in shared memory.
#include "kernels.h"

namespace so3lr {

namespace {

constexpr int WARPS = 8;
constexpr float kInvNbar = 1.0f / kAvgNumNeighbors;

__device__ __forceinline__ float invw(int l) {
  return l == 0 ? 0.5773502691896258f : (l == 1 ? 0.4472135954999579f : (l == 2 ? 0.3779644730092272f : 0.3333333333333333f));
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 f4_fma(float a, float4 b, float4 c) {
  return make_float4(fmaf(a, b.x, c.x), fmaf(a, b.y, c.y), fmaf(a, b.z, c.z), fmaf(a, b.w, c.w));
}
__device__ __forceinline__ float dot3(float4 a, float4 b, float4 c) { return a.x * b.x * c.x + a.y * b.y * c.y + a.z * b.z * c.z + a.w * b.w * c.w; }
__device__ __forceinline__ float dot2(float4 a, float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }

// cubic Hermite weights on the table interval containing r
struct Hermite {
  int g;
  float h00, h10, h01, h11;       // value weights
  float d00, d10, d01, d11;       // derivative weights (already divided by the grid spacing)
};
__device__ __forceinline__ Hermite hermite_at(float r) {
  Hermite H;
  float t = r * (1.0f / kTableH);
  int g = (int)t;
  g = g > kTableGrid - 2 ? kTableGrid - 2 : g;
  t -= (float)g;
  float t2 = t * t, t3 = t2 * t;
  H.g = g;
  H.h00 = 1.f; H.h10 = t3 - 2.f * t2 + t; H.h01 = -2.f * t3 + 3.f * t2; H.h11 = t3 - t2;
  const float ih = 1.0f / kTableH;
  H.d00 = 0.f; H.d10 = (3.f * t2 - 4.f * t + 1.f) * ih; H.d01 = (-6.f * t2 + 6.f * t) * ih;
  H.d11 = (3.f * t2 - 2.f * t) * ih;
  return H;
}
// table layout per interval g: [g][4][256] = value, slope * spacing, value difference to the next knot, next slope * spacing
__device__ __forceinline__ void table_eval(const float* __restrict__ tab, const Hermite& H, int col, float4& w, float4* dw) {
  const float* p0 = tab + (size_t)H.g * 1024 + col;   // interval rows: v0, h m0, v1 - v0, h m1
  float4 v0 = ld4(p0), m0 = ld4(p0 + 256), v1 = ld4(p0 + 512), m1 = ld4(p0 + 768);
  w.x = H.h00 * v0.x + H.h10 * m0.x + H.h01 * v1.x + H.h11 * m1.x;
  w.y = H.h00 * v0.y + H.h10 * m0.y + H.h01 * v1.y + H.h11 * m1.y;
  w.z = H.h00 * v0.z + H.h10 * m0.z + H.h01 * v1.z + H.h11 * m1.z;
  w.w = H.h00 * v0.w + H.h10 * m0.w + H.h01 * v1.w + H.h11 * m1.w;
  if (dw) {
    dw->x = H.d00 * v0.x + H.d10 * m0.x + H.d01 * v1.x + H.d11 * m1.x;
    dw->y = H.d00 * v0.y + H.d10 * m0.y + H.d01 * v1.y + H.d11 * m1.y;
    dw->z = H.d00 * v0.z + H.d10 * m0.z + H.d01 * v1.z + H.d11 * m1.z;
    dw->w = H.d00 * v0.w + H.d10 * m0.w + H.d01 * v1.w + H.d11 * m1.w;
  }
}

// per-degree invariants of (ev_j - ev_i); evj is read with broadcast loads
__device__ __forceinline__ void edge_invariants(const float* evi, const float* __restrict__ evj_ptr, float* dev, float* s) {
#pragma unroll
  for (int c = 0; c < 6; ++c) {
    float4 v = ld4(evj_ptr + 4 * c);
    dev[4 * c + 0] = v.x - evi[4 * c + 0]; dev[4 * c + 1] = v.y - evi[4 * c + 1];
    dev[4 * c + 2] = v.z - evi[4 * c + 2]; dev[4 * c + 3] = v.w - evi[4 * c + 3];
  }
  s[0] = s[1] = s[2] = s[3] = 0.f;
#pragma unroll
  for (int m = 0; m < kMTot; ++m) s[degree_of(m)] = fmaf(dev[m], dev[m], s[degree_of(m)]);
#pragma unroll
  for (int l = 0; l < 4; ++l) s[l] *= invw(l);
}

template <bool SPH>
__global__ void __launch_bounds__(WARPS * 32) attn_fwd_kernel(LayerDev L, int n, const int* __restrict__ row_ptr,
                                                              const int* __restrict__ nbr_j, const float* __restrict__ dR,
                                                              const float* __restrict__ qkv, const float* __restrict__ x_in,
                                                              const float* __restrict__ ev_in, float* __restrict__ xa,
                                                              float* __restrict__ ev1) {
  extern __shared__ float sm[];
  float* K2 = sm;   // [2][32][128]
  if (SPH) {
    for (int idx = threadIdx.x * 4; idx < 2 * 32 * 128; idx += WARPS * 32 * 4) *reinterpret_cast<float4*>(K2 + idx) = ld4(L.sph2_k + idx);
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (i >= n) return;
  const int col = 4 * lane;
  const float* qi = qkv + (size_t)i * kProj;
  const float4 q1 = ld4(qi + col), q2 = ld4(qi + 3 * kF + col);
  float evi[kMTot];
  float k1w[2][4], k1b[2];
  if (SPH) {
#pragma unroll
    for (int c = 0; c < 6; ++c) {
      float4 v = ld4(ev_in + (size_t)i * kMTot + 4 * c);
      evi[4 * c] = v.x; evi[4 * c + 1] = v.y; evi[4 * c + 2] = v.z; evi[4 * c + 3] = v.w;
    }
#pragma unroll
    for (int f = 0; f < 2; ++f) {
#pragma unroll
      for (int k = 0; k < 4; ++k) k1w[f][k] = L.sph1_k[(f * 4 + k) * 32 + lane];
      k1b[f] = L.sph1_b[f * 32 + lane];
    }
  }
  float4 accx = make_float4(0.f, 0.f, 0.f, 0.f);
  float accev = 0.f;
  const int e0 = row_ptr[i], e1 = row_ptr[i + 1];
  for (int e = e0; e < e1; ++e) {
    const int j = nbr_j[e];
    const float dx = dR[3 * (size_t)e], dy = dR[3 * (size_t)e + 1], dz = dR[3 * (size_t)e + 2];
    const float r2 = dx * dx + dy * dy + dz * dz;
    if (j >= n || j < 0 || r2 >= kCutoffSr * kCutoffSr || r2 <= 0.f) continue;
    const float r = sqrtf(r2), ir = 1.f / r;
    float cut, dcut;
    phys_cutoff(r, cut, dcut);
    const Hermite H = hermite_at(r);
    float4 w1, w2;
    table_eval(L.table, H, col, w1, nullptr);
    table_eval(L.table, H, 128 + col, w2, nullptr);
    const float* kj = qkv + (size_t)j * kProj;
    const float4 k1 = ld4(kj + kF + col), v1 = ld4(kj + 2 * kF + col), k2 = ld4(kj + 4 * kF + col);
    if (SPH) {
      float dev[kMTot], s[4];
      edge_invariants(evi, ev_in + (size_t)j * kMTot, dev, s);
      float z1 = k1b[0], z2 = k1b[1];
#pragma unroll
      for (int k = 0; k < 4; ++k) { z1 = fmaf(s[k], k1w[0][k], z1); z2 = fmaf(s[k], k1w[1][k], z2); }
      const float hs1 = silu_f(z1), hs2 = silu_f(z2);
#pragma unroll 8
      for (int c = 0; c < 32; ++c) {
        float a = __shfl_sync(0xffffffffu, hs1, c), b = __shfl_sync(0xffffffffu, hs2, c);
        w1 = f4_fma(a, ld4(K2 + c * 128 + col), w1);
        w2 = f4_fma(b, ld4(K2 + 4096 + c * 128 + col), w2);
      }
    }
    const float sc = cut * kInvNbar;
    const float a1 = group8_sum(dot3(q1, w1, k1)) * sc;
    const float a2 = group8_sum(dot3(q2, w2, k2)) * sc;
    accx = f4_fma(a1, v1, accx);
    float Y[kMTot];
    sph_harm_24(dx * ir, dy * ir, dz * ir, Y);
    float ym = 0.f;
#pragma unroll
    for (int m = 0; m < kMTot; ++m) ym = (lane == m) ? Y[m] : ym;
    const float a2m = __shfl_sync(0xffffffffu, a2, 8 * degree_of(lane < kMTot ? lane : 0));
    accev = fmaf(a2m, ym, accev);
  }
  const float4 xi = ld4(x_in + (size_t)i * kF + col);
  *reinterpret_cast<float4*>(xa + (size_t)i * kF + col) = make_float4(xi.x + accx.x, xi.y + accx.y, xi.z + accx.z, xi.w + accx.w);
  if (lane < kMTot) ev1[(size_t)i * kMTot + lane] = (SPH ? ev_in[(size_t)i * kMTot + lane] : 0.f) + accev;
}

// Backward.  FIRST: first layer (no spherical filter, inputs are constants): only the edge-geometry gradient.
template <bool FIRST>
__global__ void __launch_bounds__(WARPS * 32) attn_bwd_kernel(LayerDev L, int n, const int* __restrict__ row_ptr,
                                                              const int* __restrict__ nbr_j, const float* __restrict__ dR,
                                                              const float* __restrict__ qkv, const float* __restrict__ ev_in,
                                                              const float* __restrict__ g_xa, const float* __restrict__ gev1,
                                                              float* __restrict__ g_qkv, float* __restrict__ gev_in,
                                                              float* __restrict__ g_dR, const int* __restrict__ run_if_set) {
  if (run_if_set && *run_if_set == 0) return;      // another kernel takes this launch's work
  extern __shared__ float sm[];
  float* K2 = sm;                     // [2][32][128]
  float* K2T = sm + 2 * 32 * 128;     // [2][128][32]
  float* dwbuf = sm + 4 * 32 * 128 + (threadIdx.x >> 5) * 256;   // per warp: dw1 | dw2
  if (!FIRST) {
    for (int idx = threadIdx.x; idx < 2 * 32 * 128; idx += WARPS * 32) {
      float v = L.sph2_k[idx];
      K2[idx] = v;
      int f = idx >> 12, c = (idx >> 7) & 31, ft = idx & 127;
      K2T[f * 4096 + ft * 32 + c] = v;
    }
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (i >= n) return;
  const int col = 4 * lane;
  const int grp = lane >> 3;
  const float* qi = qkv + (size_t)i * kProj;
  const float4 q1 = ld4(qi + col), q2 = ld4(qi + 3 * kF + col);
  const float4 gx = ld4(g_xa + (size_t)i * kF + col);
  float gev[kMTot];
#pragma unroll
  for (int c = 0; c < 6; ++c) {
    float4 v = ld4(gev1 + (size_t)i * kMTot + 4 * c);
    gev[4 * c] = v.x; gev[4 * c + 1] = v.y; gev[4 * c + 2] = v.z; gev[4 * c + 3] = v.w;
  }
  float evi[kMTot];
  float k1w[2][4], k1b[2];
  if (!FIRST) {
#pragma unroll
    for (int c = 0; c < 6; ++c) {
      float4 v = ld4(ev_in + (size_t)i * kMTot + 4 * c);
      evi[4 * c] = v.x; evi[4 * c + 1] = v.y; evi[4 * c + 2] = v.z; evi[4 * c + 3] = v.w;
    }
#pragma unroll
    for (int f = 0; f < 2; ++f) {
#pragma unroll
      for (int k = 0; k < 4; ++k) k1w[f][k] = L.sph1_k[(f * 4 + k) * 32 + lane];
      k1b[f] = L.sph1_b[f * 32 + lane];
    }
  }
  float4 gq1 = make_float4(0.f, 0.f, 0.f, 0.f), gq2 = gq1;
  float gevi = 0.f;   // lane m: cotangent of ev_in[i][m] from the (ev_j - ev_i) path
  const int e0 = row_ptr[i], e1 = row_ptr[i + 1];
  for (int e = e0; e < e1; ++e) {
    const int j = nbr_j[e];
    const float dx = dR[3 * (size_t)e], dy = dR[3 * (size_t)e + 1], dz = dR[3 * (size_t)e + 2];
    const float r2 = dx * dx + dy * dy + dz * dz;
    if (j >= n || j < 0 || r2 >= kCutoffSr * kCutoffSr || r2 <= 0.f) continue;
    const float r = sqrtf(r2), ir = 1.f / r;
    const float ux = dx * ir, uy = dy * ir, uz = dz * ir;
    float cut, dcut;
    phys_cutoff(r, cut, dcut);
    const Hermite H = hermite_at(r);
    float4 w1, w2, dw1r, dw2r;
    table_eval(L.table, H, col, w1, &dw1r);
    table_eval(L.table, H, 128 + col, w2, &dw2r);
    const float* kj = qkv + (size_t)j * kProj;
    const float4 k1 = ld4(kj + kF + col), v1 = ld4(kj + 2 * kF + col), k2 = ld4(kj + 4 * kF + col);
    float dev[kMTot], s[4];
    float z1 = 0.f, z2 = 0.f;
    if (!FIRST) {
      edge_invariants(evi, ev_in + (size_t)j * kMTot, dev, s);
      z1 = k1b[0]; z2 = k1b[1];
#pragma unroll
      for (int k = 0; k < 4; ++k) { z1 = fmaf(s[k], k1w[0][k], z1); z2 = fmaf(s[k], k1w[1][k], z2); }
      const float hs1 = silu_f(z1), hs2 = silu_f(z2);
#pragma unroll 8
      for (int c = 0; c < 32; ++c) {
        float a = __shfl_sync(0xffffffffu, hs1, c), b = __shfl_sync(0xffffffffu, hs2, c);
        w1 = f4_fma(a, ld4(K2 + c * 128 + col), w1);
        w2 = f4_fma(b, ld4(K2 + 4096 + c * 128 + col), w2);
      }
    }
    const float sc = cut * kInvNbar;
    const float D1 = group8_sum(dot3(q1, w1, k1));
    const float D2 = group8_sum(dot3(q2, w2, k2));
    float Y[kMTot];
    sph_harm_24(ux, uy, uz, Y);
    // cotangents of the attention coefficients (own head / own degree group)
    const float da1 = group8_sum(dot2(gx, v1));
    float da2_all[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int m = 0; m < kMTot; ++m) da2_all[degree_of(m)] = fmaf(gev[m], Y[m], da2_all[degree_of(m)]);
    const float da2 = grp == 0 ? da2_all[0] : (grp == 1 ? da2_all[1] : (grp == 2 ? da2_all[2] : da2_all[3]));
    // d/d(cutoff scale): sum over the 4 heads and 4 degrees (each group holds identical values on its 8 lanes)
    float dsc = warp_sum(da1 * D1 + da2 * D2) * 0.125f;
    float g_r = dsc * kInvNbar * dcut;
    const float dD1 = sc * da1, dD2 = sc * da2;
    // radial-filter path: dw_f = dD * q_f * k_f
    const float4 dw1 = make_float4(dD1 * q1.x * k1.x, dD1 * q1.y * k1.y, dD1 * q1.z * k1.z, dD1 * q1.w * k1.w);
    const float4 dw2 = make_float4(dD2 * q2.x * k2.x, dD2 * q2.y * k2.y, dD2 * q2.z * k2.z, dD2 * q2.w * k2.w);
    g_r += warp_sum(dot2(dw1, dw1r) + dot2(dw2, dw2r));
    // Y path: dY_m = a2_l * gev_m
    float a2l[4];
#pragma unroll
    for (int l = 0; l < 4; ++l) a2l[l] = __shfl_sync(0xffffffffu, D2, 8 * l) * sc;
    float gY[kMTot];
#pragma unroll
    for (int m = 0; m < kMTot; ++m) gY[m] = a2l[degree_of(m)] * gev[m];
    float gux, guy, guz;
    sph_harm_24_vjp(ux, uy, uz, gY, gux, guy, guz);
    const float gu_dot = gux * ux + guy * uy + guz * uz;
    const float gdx = g_r * ux + (gux - gu_dot * ux) * ir;
    const float gdy = g_r * uy + (guy - gu_dot * uy) * ir;
    const float gdz = g_r * uz + (guz - gu_dot * uz) * ir;
    if (!FIRST) {
      // receiver / sender projections
      gq1 = make_float4(fmaf(dD1 * w1.x, k1.x, gq1.x), fmaf(dD1 * w1.y, k1.y, gq1.y), fmaf(dD1 * w1.z, k1.z, gq1.z), fmaf(dD1 * w1.w, k1.w, gq1.w));
      gq2 = make_float4(fmaf(dD2 * w2.x, k2.x, gq2.x), fmaf(dD2 * w2.y, k2.y, gq2.y), fmaf(dD2 * w2.z, k2.z, gq2.z), fmaf(dD2 * w2.w, k2.w, gq2.w));
      float* gj = g_qkv + (size_t)j * kProj;
      atomicAdd(reinterpret_cast<float4*>(gj + kF + col), make_float4(dD1 * q1.x * w1.x, dD1 * q1.y * w1.y, dD1 * q1.z * w1.z, dD1 * q1.w * w1.w));
      const float a1 = D1 * sc;
      atomicAdd(reinterpret_cast<float4*>(gj + 2 * kF + col), make_float4(a1 * gx.x, a1 * gx.y, a1 * gx.z, a1 * gx.w));
      atomicAdd(reinterpret_cast<float4*>(gj + 4 * kF + col), make_float4(dD2 * q2.x * w2.x, dD2 * q2.y * w2.y, dD2 * q2.z * w2.z, dD2 * q2.w * w2.w));
      // spherical-filter path: hidden-unit cotangents dhs_c = sum_f K2[c][f] dw_f (lane c)
      __syncwarp();
      *reinterpret_cast<float4*>(dwbuf + col) = dw1;
      *reinterpret_cast<float4*>(dwbuf + 128 + col) = dw2;
      __syncwarp();
      float dh1 = 0.f, dh2 = 0.f;
#pragma unroll 4
      for (int f4 = 0; f4 < 32; ++f4) {
        float4 a = ld4(dwbuf + 4 * f4), b = ld4(dwbuf + 128 + 4 * f4);
        const float* t1 = K2T + (4 * f4) * 32 + lane;
        const float* t2 = K2T + 4096 + (4 * f4) * 32 + lane;
        dh1 = fmaf(a.x, t1[0], dh1); dh1 = fmaf(a.y, t1[32], dh1); dh1 = fmaf(a.z, t1[64], dh1); dh1 = fmaf(a.w, t1[96], dh1);
        dh2 = fmaf(b.x, t2[0], dh2); dh2 = fmaf(b.y, t2[32], dh2); dh2 = fmaf(b.z, t2[64], dh2); dh2 = fmaf(b.w, t2[96], dh2);
      }
      const float dz1 = dh1 * dsilu_f(z1), dz2 = dh2 * dsilu_f(z2);
      float ds[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) ds[k] = warp_sum(dz1 * k1w[0][k] + dz2 * k1w[1][k]);
      // d(ev_j - ev_i)_m = ds_l * 2 dev_m / sqrt(2l+1)
      float gd = 0.f;
#pragma unroll
      for (int m = 0; m < kMTot; ++m) {
        float v = ds[degree_of(m)] * 2.f * dev[m] * invw(degree_of(m));
        gd = (lane == m) ? v : gd;
      }
      if (lane < kMTot) {
        atomicAdd(gev_in + (size_t)j * kMTot + lane, gd);
        gevi -= gd;
      }
    }
    if (lane == 0) {
      g_dR[3 * (size_t)e] += gdx; g_dR[3 * (size_t)e + 1] += gdy; g_dR[3 * (size_t)e + 2] += gdz;
    }
  }
  if (!FIRST) {
    float* gi = g_qkv + (size_t)i * kProj;
    *reinterpret_cast<float4*>(gi + col) = gq1;
    *reinterpret_cast<float4*>(gi + 3 * kF + col) = gq2;
    if (lane < kMTot) atomicAdd(gev_in + (size_t)i * kMTot + lane, gevi);
  }
}

constexpr size_t kSmemFwd = (size_t)2 * 32 * 128 * sizeof(float);
constexpr size_t kSmemBwd = (size_t)(4 * 32 * 128 + WARPS * 256) * sizeof(float);

}  // namespace

int configure_attention_kernels() {
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBwd));
  return kOk;
}

void launch_attn_fwd(cudaStream_t s, const LayerDev& L, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                     const float* qkv, const float* x_in, const float* ev_in, float* xa, float* ev1) {
  if (n <= 0) return;
  int blocks = (n + WARPS - 1) / WARPS;
  if (L.has_spherical)
    { attn_fwd_kernel<true><<<blocks, WARPS * 32, kSmemFwd, s>>>(L, n, row_ptr, nbr_j, dR, qkv, x_in, ev_in, xa, ev1); count_launch(); }
  else
    { attn_fwd_kernel<false><<<blocks, WARPS * 32, 0, s>>>(L, n, row_ptr, nbr_j, dR, qkv, x_in, ev_in, xa, ev1); count_launch(); }
}

void launch_attn_bwd(cudaStream_t s, const LayerDev& L, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                     const float* qkv, const float* ev_in, const float* g_xa, const float* gev1, float* g_qkv,
                     float* gev_in, float* g_dR, int first_layer, const int* run_if_set) {
  if (n <= 0) return;
  int blocks = (n + WARPS - 1) / WARPS;
  if (first_layer)
    { attn_bwd_kernel<true><<<blocks, WARPS * 32, 0, s>>>(L, n, row_ptr, nbr_j, dR, qkv, ev_in, g_xa, gev1, g_qkv, gev_in, g_dR, nullptr); count_launch(); }
  else
    { attn_bwd_kernel<false><<<blocks, WARPS * 32, kSmemBwd, s>>>(L, n, row_ptr, nbr_j, dR, qkv, ev_in, g_xa, gev1, g_qkv, gev_in, g_dR, run_if_set); count_launch(); }
}

}  // namespace so3lr

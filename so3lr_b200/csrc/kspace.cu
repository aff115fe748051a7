// Reciprocal-space (Ewald) part of the electrostatic energy for one periodic structure: the path the reference takes when its
// energy function is called with `k_grid` and `k_smearing` (so3lr/jaxmd_utils.py:39-47,70-71; grid from
// jaxpme.kspace.get_kgrid_ewald, so3lr/cli/so3lr_md.py:1392-1428).  Published Ewald summation for Gaussian-smeared charges:
//
//   E_k = ke / (2 V) sum_{k != 0} (4 pi / k^2) exp(-s^2 k^2 / 2) |S(k)|^2 - ke sum_i q_i^2 / (sqrt(2 pi) s) - ke pi s^2 Q^2 / V,
//   S(k) = sum_i q_i exp(i k r_i),   k = 2 pi (h1 b1 + h2 b2 + h3 b3) on the FFT-frequency index grid of shape (n1, n2, n3).
//
// S(-k) = conj S(k), so one vector of every pair (k, -k) is kept with weight 2 (an index -n/2 of an even grid has no partner and
// keeps weight 1).  The kept indices are cut into tiles of 16 x 16 (h2, h3) values at one h1.  exp(i k r) factorises over the three
// indices, so a tile needs 32 sines and cosines per atom instead of 256:
//   ewald_structure_kernel  a CTA takes up to four tiles adjacent along h3 (80 table entries per atom for 1024 vectors), a thread eight
//                           vectors, and loops over a slice of the atoms staged in shared memory (4 FMAs per pair)
//   ewald_atom_kernel       thread = atom, loops over a slice of the tiles; potential phi_i and the three index-weighted sums that
//                           give the force (8 FMAs per pair)
//   ewald_finish_kernel     per atom: energy, dE/dq (it continues into the charge head's reverse pass), force
//   ewald_virial_kernel     strain derivative, added to the first atom's virial row (the rows are only ever summed)
//
// Mesh variant (mode 2; the reference's default k-space method, `coulomb_kspace_interp_nodes=4`, so3lr/potential.py:11-12): smooth
// particle-mesh Ewald (Essmann et al., J. Chem. Phys. 103, 8577 (1995)) with cubic B-splines, i.e. four mesh points per axis and atom.
//   pme_spread_kernel     charges onto the mesh Q (64 atomic adds per atom, four threads per atom)
//   cuFFT R2C             library FFT, loaded at run time (dlopen) so that the library itself has no link-time dependency on it
//   pme_influence_kernel  F(Q)(m) *= ke / V x 4 pi exp(-s^2 k^2 / 2) / k^2 x prod_d 9 / (2 + cos(2 pi m_d / n_d))^2; strain derivative
//   cuFFT C2R             the convolved potential on the mesh (unnormalised inverse transform)
//   pme_gather_kernel     phi_i and its gradient from the 64 mesh points of atom i -> the same per-atom record as the direct sum
//   ewald_finish_kernel   shared with the direct sum
#include <cufft.h>
#include <dlfcn.h>

#include <mutex>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace so3lr {

namespace {

constexpr int kTile = 16;
constexpr int kTileK = kTile * kTile;
constexpr float kTwoPi = 6.283185307179586f;

// f * h modulo 1 in [-1/2, 1/2]: the product is formed exactly inside the FMA, so the result carries the rounding of f only
__device__ __forceinline__ float phase_frac(float f, int h) {
  const float hf = (float)h;
  return fmaf(f, hf, -rintf(f * hf));
}
// exp(2 pi i x) for |x| <= 1
__device__ __forceinline__ void unit_phase(float x, float& c, float& s) {
  x -= rintf(x);
  __sincosf(kTwoPi * x, &s, &c);
}
__device__ __forceinline__ void fractional(const Cell& c, const float* __restrict__ R, int a, float& f1, float& f2, float& f3) {
  const float x = R[3 * (size_t)a], y = R[3 * (size_t)a + 1], z = R[3 * (size_t)a + 2];
  f1 = x * c.hinv[0] + y * c.hinv[3] + z * c.hinv[6];
  f2 = x * c.hinv[1] + y * c.hinv[4] + z * c.hinv[7];
  f3 = x * c.hinv[2] + y * c.hinv[5] + z * c.hinv[8];
  f1 -= floorf(f1); f2 -= floorf(f2); f3 -= floorf(f3);
}
// Cartesian k vector of an index triple: k_a = 2 pi sum_d hinv[a][d] h_d
__device__ __forceinline__ void k_vector(const Cell& c, int h1, int h2, int h3, float& kx, float& ky, float& kz) {
  kx = kTwoPi * (c.hinv[0] * h1 + c.hinv[1] * h2 + c.hinv[2] * h3);
  ky = kTwoPi * (c.hinv[3] * h1 + c.hinv[4] * h2 + c.hinv[5] * h3);
  kz = kTwoPi * (c.hinv[6] * h1 + c.hinv[7] * h2 + c.hinv[8] * h3);
}
// weight x ke / V x 4 pi exp(-s^2 k^2 / 2) / k^2
__device__ __forceinline__ float k_weight(float w, float inv_vol, float smearing, float k2) {
  return w * kKe * inv_vol * 12.566370614359172f * expf(-0.5f * smearing * smearing * k2) / k2;
}

// A group is up to four tiles that share (h1, first h2) and follow one another along h3: 16 x 64 index pairs whose phase factors need
// 16 + 64 table entries per atom.  128 threads; thread (warp w, lane l) accumulates the eight vectors h2 = w, w + 4, w + 8, w + 12 times
// h3 = l, l + 32: per atom four broadcast loads and two coalesced ones from shared memory feed 32 FMAs.
constexpr int kGroupStage = 32;            // atoms per shared-memory stage
__global__ void __launch_bounds__(128) ewald_structure_kernel(Cell cell, int n, int atoms_per_split, const float* __restrict__ R,
                                                              const float* __restrict__ q, const int4* __restrict__ tiles,
                                                              const int2* __restrict__ groups, float2* __restrict__ Sk) {
  __shared__ float2 T2[kGroupStage][kTile];        // q exp(2 pi i (f1 h1 + f2 h2)) for the group's 16 h2
  __shared__ float2 T3[kGroupStage][4 * kTile];    // exp(2 pi i f3 h3) for its 64 h3
  __shared__ float4 A[kGroupStage];                // f1 f2 f3 q
  const int2 g = groups[blockIdx.x];               // first tile, number of tiles
  const int4 t = tiles[g.x];
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int a0 = blockIdx.y * atoms_per_split;
  const int a1 = a0 + atoms_per_split < n ? a0 + atoms_per_split : n;
  float sr[8], si[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) { sr[k] = 0.f; si[k] = 0.f; }
  for (int base = a0; base < a1; base += kGroupStage) {
    __syncthreads();
    if (tid < kGroupStage) {
      const int a = base + tid;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (a < a1) {
        fractional(cell, R, a, v.x, v.y, v.z);
        v.w = q[a];
      }
      A[tid] = v;
    }
    __syncthreads();
    for (int e = tid; e < kGroupStage * 5 * kTile; e += 128) {
      const int a = e / (5 * kTile), j = e - a * (5 * kTile);
      const float4 v = A[a];
      float c, s;
      if (j < kTile) {
        unit_phase(phase_frac(v.x, t.x) + phase_frac(v.y, t.y + j), c, s);
        T2[a][j] = make_float2(v.w * c, v.w * s);
      } else {
        unit_phase(phase_frac(v.z, t.z + j - kTile), c, s);
        T3[a][j - kTile] = make_float2(c, s);
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int a = 0; a < kGroupStage; ++a) {
      const float2 w0 = T3[a][lane], w1 = T3[a][lane + 32];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 u = T2[a][w + 4 * k];
        sr[2 * k] = fmaf(u.x, w0.x, sr[2 * k]); sr[2 * k] = fmaf(-u.y, w0.y, sr[2 * k]);
        si[2 * k] = fmaf(u.x, w0.y, si[2 * k]); si[2 * k] = fmaf(u.y, w0.x, si[2 * k]);
        sr[2 * k + 1] = fmaf(u.x, w1.x, sr[2 * k + 1]); sr[2 * k + 1] = fmaf(-u.y, w1.y, sr[2 * k + 1]);
        si[2 * k + 1] = fmaf(u.x, w1.y, si[2 * k + 1]); si[2 * k + 1] = fmaf(u.y, w1.x, si[2 * k + 1]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int h3 = lane + 32 * hh, u = h3 >> 4;          // tile of the group, slot inside it
      if (u < g.y) {
        float2* out = Sk + (size_t)(g.x + u) * kTileK + (w + 4 * k) * kTile + (h3 & 15);
        atomicAdd(&out->x, sr[2 * k + hh]);
        atomicAdd(&out->y, si[2 * k + hh]);
      }
    }
}

// acc rows: phi_i, and sum_k G h_d Im[S(k) exp(-i k r_i)] for d = 1, 2, 3
__global__ void __launch_bounds__(128) ewald_atom_kernel(Cell cell, float inv_vol, float smearing, int n, int n_tiles, int tiles_per_split,
                                                         const float* __restrict__ R, const int4* __restrict__ tiles,
                                                         const float* __restrict__ wgt, const float2* __restrict__ Sk,
                                                         float* __restrict__ acc) {
  __shared__ float2 A[kTileK];               // weight x S(k) of the current tile
  const int tid = threadIdx.x;
  const int a = blockIdx.x * 128 + tid;
  float f1 = 0.f, f2 = 0.f, f3 = 0.f;
  if (a < n) fractional(cell, R, a, f1, f2, f3);
  float phi = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
  const int tile0 = blockIdx.y * tiles_per_split;
  const int tile1 = tile0 + tiles_per_split < n_tiles ? tile0 + tiles_per_split : n_tiles;
  for (int tile = tile0; tile < tile1; ++tile) {
    const int4 t = tiles[tile];
    __syncthreads();
    for (int s = tid; s < kTileK; s += 128) {
      const float w = wgt[(size_t)tile * kTileK + s];
      float2 v = make_float2(0.f, 0.f);
      if (w > 0.f) {
        float kx, ky, kz;
        k_vector(cell, t.x, t.y + (s >> 4), t.z + (s & 15), kx, ky, kz);
        const float g = k_weight(w, inv_vol, smearing, kx * kx + ky * ky + kz * kz);
        const float2 sk = Sk[(size_t)tile * kTileK + s];
        v = make_float2(g * sk.x, g * sk.y);
      }
      A[s] = v;
    }
    __syncthreads();
    float c3[kTile], s3[kTile];
#pragma unroll
    for (int j = 0; j < kTile; ++j) unit_phase(phase_frac(f3, t.z + j), c3[j], s3[j]);
    const float x1 = phase_frac(f1, t.x);
    const float h1f = (float)t.x;
#pragma unroll 1
    for (int i2 = 0; i2 < kTile; ++i2) {
      if (!((t.w >> i2) & 1)) continue;                  // no kept vector in this row of the tile
      float ur = 0.f, ui = 0.f, vr = 0.f, vi = 0.f;      // sum over h3 of A conj(T3), and of h3 A conj(T3)
#pragma unroll
      for (int j = 0; j < kTile; ++j) {
        const float2 av = A[i2 * kTile + j];
        const float pr = fmaf(av.x, c3[j], av.y * s3[j]);
        const float pi = fmaf(av.y, c3[j], -av.x * s3[j]);
        const float h3f = (float)(t.z + j);
        ur += pr; ui += pi;
        vr = fmaf(h3f, pr, vr); vi = fmaf(h3f, pi, vi);
      }
      float c, s;
      unit_phase(x1 + phase_frac(f2, t.y + i2), c, s);
      const float wr = fmaf(ur, c, ui * s);               // (u)(c - i s)
      const float wi = fmaf(ui, c, -ur * s);
      const float vim = fmaf(vi, c, -vr * s);
      phi += wr;
      d1 = fmaf(h1f, wi, d1);
      d2 = fmaf((float)(t.y + i2), wi, d2);
      d3 += vim;
    }
  }
  if (a < n) {
    float* o = acc + 4 * (size_t)a;
    atomicAdd(o, phi); atomicAdd(o + 1, d1); atomicAdd(o + 2, d2); atomicAdd(o + 3, d3);
  }
}

__global__ void __launch_bounds__(256) ewald_finish_kernel(Cell cell, float inv_vol, float smearing, int n, const float* __restrict__ q,
                                                           const float* __restrict__ total_charge, const float* __restrict__ acc,
                                                           float* __restrict__ e_coul, float* __restrict__ gq, float* __restrict__ F,
                                                           float force_sign) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= n) return;
  const float4 v = *reinterpret_cast<const float4*>(acc + 4 * (size_t)a);
  const float qa = q[a];
  const float self = kKe * 0.7978845608028654f / smearing;                                  // ke sqrt(2 / pi) / s
  const float bg = kKe * 3.141592653589793f * smearing * smearing * inv_vol * total_charge[0];
  e_coul[a] += 0.5f * qa * v.x - 0.5f * self * qa * qa - bg * qa;
  gq[a] += v.x - self * qa - 2.f * bg;
  const float s = -kTwoPi * qa * force_sign;
  float* f = F + 3 * (size_t)a;
  f[0] += s * (cell.hinv[0] * v.y + cell.hinv[1] * v.z + cell.hinv[2] * v.w);
  f[1] += s * (cell.hinv[3] * v.y + cell.hinv[4] * v.z + cell.hinv[5] * v.w);
  f[2] += s * (cell.hinv[6] * v.y + cell.hinv[7] * v.z + cell.hinv[8] * v.w);
}

// dE_k / d eps_ab = sum_k G |S|^2 / 2 (-delta_ab + 2 k_a k_b (s^2 / 2 + 1 / k^2)) + delta_ab ke pi s^2 Q^2 / V
__global__ void __launch_bounds__(kTileK) ewald_virial_kernel(Cell cell, float inv_vol, float smearing, const int4* __restrict__ tiles,
                                                              const float* __restrict__ wgt, const float2* __restrict__ Sk,
                                                              const float* __restrict__ total_charge, float* __restrict__ virial_row) {
  __shared__ float part[8][6];
  const int tid = threadIdx.x;
  const int4 t = tiles[blockIdx.x];
  const float w = wgt[(size_t)blockIdx.x * kTileK + tid];
  float v[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (w > 0.f) {
    float kx, ky, kz;
    k_vector(cell, t.x, t.y + (tid >> 4), t.z + (tid & 15), kx, ky, kz);
    const float k2 = kx * kx + ky * ky + kz * kz;
    const float2 sk = Sk[(size_t)blockIdx.x * kTileK + tid];
    const float e = 0.5f * k_weight(w, inv_vol, smearing, k2) * (sk.x * sk.x + sk.y * sk.y);
    const float m = 2.f * (0.5f * smearing * smearing + 1.f / k2);
    v[0] = e * (m * kx * kx - 1.f); v[1] = e * (m * ky * ky - 1.f); v[2] = e * (m * kz * kz - 1.f);
    v[3] = e * m * ky * kz; v[4] = e * m * kx * kz; v[5] = e * m * kx * ky;
  }
  if (blockIdx.x == 0 && tid == 0) {
    const float qt = total_charge[0];
    const float b = kKe * 3.141592653589793f * smearing * smearing * inv_vol * qt * qt;
    v[0] += b; v[1] += b; v[2] += b;
  }
#pragma unroll
  for (int c = 0; c < 6; ++c) v[c] = warp_sum(v[c]);
  if ((tid & 31) == 0)
    for (int c = 0; c < 6; ++c) part[tid >> 5][c] = v[c];
  __syncthreads();
  if (tid < 6) {
    float s = 0.f;
    for (int wp = 0; wp < kTileK / 32; ++wp) s += part[wp][tid];
    atomicAdd(virial_row + tid, s);
  }
}


// ---- mesh variant ----
// weights M4(t + j) of the mesh points m0 - j (j = 0..3) around the scaled coordinate m0 + t, and their t-derivatives
__device__ __forceinline__ void bspline4(float t, float* w, float* dw) {
  const float t2 = t * t, t3 = t2 * t, o = 1.f - t;
  w[0] = t3 * (1.f / 6.f);
  w[1] = (-3.f * t3 + 3.f * t2 + 3.f * t + 1.f) * (1.f / 6.f);
  w[2] = (3.f * t3 - 6.f * t2 + 4.f) * (1.f / 6.f);
  w[3] = o * o * o * (1.f / 6.f);
  dw[0] = 0.5f * t2;
  dw[1] = 0.5f * (-3.f * t2 + 2.f * t + 1.f);
  dw[2] = 0.5f * (3.f * t2 - 4.f * t);
  dw[3] = -0.5f * o * o;
}
__device__ __forceinline__ int wrap_index(int k, int n) { return k < 0 ? k + n : (k >= n ? k - n : k); }
// scaled coordinate of one axis: mesh point at or below it and the remainder in [0, 1)
__device__ __forceinline__ void mesh_coordinate(float f, int n, int& m0, float& t) {
  const float u = f * (float)n;
  const float fl = floorf(u);
  m0 = (int)fl;
  t = u - fl;
}
// signed frequency of a mesh index, the convention of numpy's fftfreq (n / 2 of an even n counts as -n / 2)
__device__ __forceinline__ int signed_frequency(int m, int n) { return m < (n + 1) / 2 ? m : m - n; }

__global__ void __launch_bounds__(256) pme_spread_kernel(Cell cell, int n, int n1, int n2, int n3, const float* __restrict__ R,
                                                         const float* __restrict__ q, float* __restrict__ mesh) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int a = (int)(gid >> 2), j1 = (int)(gid & 3);
  if (a >= n) return;
  float f1, f2, f3;
  fractional(cell, R, a, f1, f2, f3);
  int m1, m2, m3;
  float t1, t2, t3, w1[4], w2[4], w3[4], dw[4];
  mesh_coordinate(f1, n1, m1, t1); mesh_coordinate(f2, n2, m2, t2); mesh_coordinate(f3, n3, m3, t3);
  bspline4(t1, w1, dw); bspline4(t2, w2, dw); bspline4(t3, w3, dw);
  const float qa = q[a] * w1[j1];
  const int k1 = wrap_index(wrap_index(m1 - j1, n1), n1);
#pragma unroll
  for (int j2 = 0; j2 < 4; ++j2) {
    const int k2 = wrap_index(wrap_index(m2 - j2, n2), n2);
    float* row = mesh + ((size_t)k1 * n2 + k2) * n3;
#pragma unroll
    for (int j3 = 0; j3 < 4; ++j3) atomicAdd(row + wrap_index(wrap_index(m3 - j3, n3), n3), qa * w2[j2] * w3[j3]);
  }
}

__global__ void __launch_bounds__(256) pme_influence_kernel(Cell cell, float inv_vol, float smearing, int n1, int n2, int n3,
                                                            float2* __restrict__ fq, const float* __restrict__ total_charge,
                                                            float* __restrict__ virial_row) {
  __shared__ float part[8][6];
  const int nc = n3 / 2 + 1;
  const long long total = (long long)n1 * n2 * nc;
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  float v[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (e < total) {
    const int m3 = (int)(e % nc);
    const int m2 = (int)((e / nc) % n2);
    const int m1 = (int)(e / ((long long)nc * n2));
    float2 f = fq[e];
    float c = 0.f;
    if (m1 | m2 | m3) {
      float kx, ky, kz;
      k_vector(cell, signed_frequency(m1, n1), signed_frequency(m2, n2), signed_frequency(m3, n3), kx, ky, kz);
      const float k2 = kx * kx + ky * ky + kz * kz;
      const float b1 = 2.f + cospif(2.f * (float)m1 / (float)n1), b2 = 2.f + cospif(2.f * (float)m2 / (float)n2),
                  b3 = 2.f + cospif(2.f * (float)m3 / (float)n3);
      const float bb = b1 * b2 * b3;
      c = k_weight(1.f, inv_vol, smearing, k2) * 729.f / (bb * bb);
      if (virial_row) {
        // the stored half of the transform stands for its mirror image too, except on the planes that are their own mirror
        const float wgt = (m3 == 0 || 2 * m3 == n3) ? 1.f : 2.f;
        const float en = 0.5f * wgt * c * (f.x * f.x + f.y * f.y);
        const float m = 2.f * (0.5f * smearing * smearing + 1.f / k2);
        v[0] = en * (m * kx * kx - 1.f); v[1] = en * (m * ky * ky - 1.f); v[2] = en * (m * kz * kz - 1.f);
        v[3] = en * m * ky * kz; v[4] = en * m * kx * kz; v[5] = en * m * kx * ky;
      }
    } else if (virial_row) {
      const float qt = total_charge[0];
      const float b = kKe * 3.141592653589793f * smearing * smearing * inv_vol * qt * qt;
      v[0] = b; v[1] = b; v[2] = b;
    }
    fq[e] = make_float2(c * f.x, c * f.y);
  }
  if (!virial_row) return;
  const int tid = threadIdx.x;
#pragma unroll
  for (int k = 0; k < 6; ++k) v[k] = warp_sum(v[k]);
  if ((tid & 31) == 0)
    for (int k = 0; k < 6; ++k) part[tid >> 5][k] = v[k];
  __syncthreads();
  if (tid < 6) {
    float s = 0.f;
    for (int wp = 0; wp < 8; ++wp) s += part[wp][tid];
    if (s != 0.f) atomicAdd(virial_row + tid, s);
  }
}

__global__ void __launch_bounds__(128) pme_gather_kernel(Cell cell, int n, int n1, int n2, int n3, const float* __restrict__ R,
                                                         const float* __restrict__ mesh, float* __restrict__ acc) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= n) return;
  float f1, f2, f3;
  fractional(cell, R, a, f1, f2, f3);
  int m1, m2, m3;
  float t1, t2, t3, w1[4], w2[4], w3[4], d1[4], d2[4], d3[4];
  mesh_coordinate(f1, n1, m1, t1); mesh_coordinate(f2, n2, m2, t2); mesh_coordinate(f3, n3, m3, t3);
  bspline4(t1, w1, d1); bspline4(t2, w2, d2); bspline4(t3, w3, d3);
  int k3[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) k3[j] = wrap_index(wrap_index(m3 - j, n3), n3);
  float phi = 0.f, g1 = 0.f, g2 = 0.f, g3 = 0.f;
#pragma unroll
  for (int j1 = 0; j1 < 4; ++j1) {
    const int k1 = wrap_index(wrap_index(m1 - j1, n1), n1);
#pragma unroll
    for (int j2 = 0; j2 < 4; ++j2) {
      const int k2 = wrap_index(wrap_index(m2 - j2, n2), n2);
      const float* row = mesh + ((size_t)k1 * n2 + k2) * n3;
      float s = 0.f, sd = 0.f;       // sums over the third axis with the weights and with their derivatives
#pragma unroll
      for (int j3 = 0; j3 < 4; ++j3) {
        const float val = row[k3[j3]];
        s = fmaf(w3[j3], val, s);
        sd = fmaf(d3[j3], val, sd);
      }
      phi = fmaf(w1[j1] * w2[j2], s, phi);
      g1 = fmaf(d1[j1] * w2[j2], s, g1);
      g2 = fmaf(w1[j1] * d2[j2], s, g2);
      g3 = fmaf(w1[j1] * w2[j2], sd, g3);
    }
  }
  // the record of the direct sum: dE/dr_a = 2 pi q sum_d hinv[a][d] acc[1 + d]
  const float inv2pi = 0.15915494309189535f;
  *reinterpret_cast<float4*>(acc + 4 * (size_t)a) = make_float4(phi, g1 * (float)n1 * inv2pi, g2 * (float)n2 * inv2pi, g3 * (float)n3 * inv2pi);
}

// cuFFT entry points, resolved at run time
struct CufftApi {
  void* lib = nullptr;
  cufftResult (*plan3d)(cufftHandle*, int, int, int, cufftType) = nullptr;
  cufftResult (*set_stream)(cufftHandle, cudaStream_t) = nullptr;
  cufftResult (*exec_r2c)(cufftHandle, cufftReal*, cufftComplex*) = nullptr;
  cufftResult (*exec_c2r)(cufftHandle, cufftComplex*, cufftReal*) = nullptr;
  cufftResult (*destroy)(cufftHandle) = nullptr;
  bool ok = false;
};
CufftApi* cufft_api() {
  static CufftApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libcufft.so.11", "libcufft.so", "/usr/local/cuda/lib64/libcufft.so.11", "/usr/local/cuda/lib64/libcufft.so"};
    for (const char* nm : names) {
      api.lib = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
      if (api.lib) break;
    }
    if (!api.lib) {
      std::fprintf(stderr, "so3lr_b200: the mesh variant of the reciprocal sum needs the cuFFT library (libcufft.so.11), which could not be loaded\n");
      return;
    }
    api.plan3d = reinterpret_cast<decltype(api.plan3d)>(dlsym(api.lib, "cufftPlan3d"));
    api.set_stream = reinterpret_cast<decltype(api.set_stream)>(dlsym(api.lib, "cufftSetStream"));
    api.exec_r2c = reinterpret_cast<decltype(api.exec_r2c)>(dlsym(api.lib, "cufftExecR2C"));
    api.exec_c2r = reinterpret_cast<decltype(api.exec_c2r)>(dlsym(api.lib, "cufftExecC2R"));
    api.destroy = reinterpret_cast<decltype(api.destroy)>(dlsym(api.lib, "cufftDestroy"));
    api.ok = api.plan3d && api.set_stream && api.exec_r2c && api.exec_c2r && api.destroy;
  });
  return api.ok ? &api : nullptr;
}

}  // namespace

void kspace_free(KSpaceDev* K) {
  if (K->plans) {
    if (CufftApi* f = cufft_api()) { f->destroy(K->plan_r2c); f->destroy(K->plan_c2r); }
  }
  cudaFree(K->tiles); cudaFree(K->groups); cudaFree(K->wgt); cudaFree(K->Sk); cudaFree(K->acc); cudaFree(K->mesh); cudaFree(K->fq);
  *K = KSpaceDev{};
}

static int kspace_setup_mesh(KSpaceDev* K, int n_atoms, float smearing, int n1, int n2, int n3) {
  if (n1 < 4 || n2 < 4 || n3 < 4 || (long long)n1 * n2 * n3 > (1LL << 30)) return n1 < 4 || n2 < 4 || n3 < 4 ? kInvalidArgument : kTooLarge;
  CufftApi* f = cufft_api();
  if (!f) return kCudaError;
  K->smearing = smearing;
  K->shape[0] = n1; K->shape[1] = n2; K->shape[2] = n3;
  SO3LR_CUDA_CHECK(cudaMalloc((void**)&K->mesh, (size_t)n1 * n2 * n3 * sizeof(float)));
  SO3LR_CUDA_CHECK(cudaMalloc((void**)&K->fq, (size_t)n1 * n2 * (n3 / 2 + 1) * sizeof(float2)));
  SO3LR_CUDA_CHECK(cudaMalloc((void**)&K->acc, (size_t)n_atoms * 4 * sizeof(float)));
  if (f->plan3d(&K->plan_r2c, n1, n2, n3, CUFFT_R2C) != CUFFT_SUCCESS) return kCudaError;
  if (f->plan3d(&K->plan_c2r, n1, n2, n3, CUFFT_C2R) != CUFFT_SUCCESS) { f->destroy(K->plan_r2c); return kCudaError; }
  K->plans = true;
  K->mode = 2;
  return kOk;
}

// Tiles of the kept half of the index grid, their slot weights and the groups of the structure-factor kernel (host side)
void kspace_build_tiles(int n1, int n2, int n3, std::vector<int4>& tiles, std::vector<float>& wgt, std::vector<int2>& groups) {
  const int nn[3] = {n1, n2, n3};
  int lo[3], hi[3];
  for (int d = 0; d < 3; ++d) { lo[d] = -(nn[d] / 2); hi[d] = (nn[d] + 1) / 2 - 1; }
  auto inside = [&](int a, int b, int c) { return a >= lo[0] && a <= hi[0] && b >= lo[1] && b <= hi[1] && c >= lo[2] && c <= hi[2]; };
  // weight of an index triple: 2 for the kept member of a pair (k, -k), 0 for the other, 1 when -k is outside the grid
  auto weight = [&](int a, int b, int c) -> float {
    if (!inside(a, b, c) || (a == 0 && b == 0 && c == 0)) return 0.f;
    if (!inside(-a, -b, -c)) return 1.f;
    const bool positive = a > 0 || (a == 0 && (b > 0 || (b == 0 && c > 0)));
    return positive ? 2.f : 0.f;
  };
  for (int h1 = lo[0]; h1 <= hi[0]; ++h1)
    for (int b0 = lo[1]; b0 <= hi[1]; b0 += kTile)
      for (int c0 = lo[2]; c0 <= hi[2]; c0 += kTile) {
        float w[kTileK];
        bool any = false;
        for (int s = 0; s < kTileK; ++s) { w[s] = weight(h1, b0 + (s >> 4), c0 + (s & 15)); any |= w[s] > 0.f; }
        if (!any) continue;
        int mask = 0;                       // rows (h2) of the tile that hold a kept vector
        for (int s = 0; s < kTileK; ++s) if (w[s] > 0.f) mask |= 1 << (s >> 4);
        tiles.push_back(make_int4(h1, b0, c0, mask));
        wgt.insert(wgt.end(), w, w + kTileK);
      }
  // groups of up to four tiles that share (h1, first h2) and are adjacent along h3, runs longer than four split evenly
  for (size_t i = 0; i < tiles.size();) {
    size_t j = i + 1;
    while (j < tiles.size() && tiles[j].x == tiles[i].x && tiles[j].y == tiles[i].y && tiles[j].z == tiles[j - 1].z + kTile) ++j;
    const int run = (int)(j - i), parts = (run + 3) / 4, size = (run + parts - 1) / parts;
    for (int k = 0; k < run; k += size) groups.push_back(make_int2((int)i + k, run - k < size ? run - k : size));
    i = j;
  }
}

int kspace_setup(KSpaceDev* K, int n_atoms, int mode, float smearing, int n1, int n2, int n3) {
  kspace_free(K);
  if (!(smearing > 0.f) || n1 < 1 || n2 < 1 || n3 < 1 || n1 > 1024 || n2 > 1024 || n3 > 1024) return kInvalidArgument;
  if (mode == 2) {
    int rc = kspace_setup_mesh(K, n_atoms, smearing, n1, n2, n3);
    if (rc) kspace_free(K);
    return rc;
  }
  if (mode != 1) return kInvalidArgument;
  std::vector<int4> tiles;
  std::vector<float> wgt;
  std::vector<int2> groups;
  kspace_build_tiles(n1, n2, n3, tiles, wgt, groups);
  if (tiles.empty() || tiles.size() > (size_t)(1 << 22)) return tiles.empty() ? kInvalidArgument : kTooLarge;
  K->n_tiles = (int)tiles.size();
  K->n_groups = (int)groups.size();
  K->smearing = smearing;
  K->shape[0] = n1; K->shape[1] = n2; K->shape[2] = n3;
  SO3LR_CUDA_CHECK(cudaMalloc((void**)&K->tiles, tiles.size() * sizeof(int4)));
  SO3LR_CUDA_CHECK(cudaMalloc((void**)&K->wgt, wgt.size() * sizeof(float)));
  SO3LR_CUDA_CHECK(cudaMalloc((void**)&K->Sk, wgt.size() * sizeof(float2)));
  SO3LR_CUDA_CHECK(cudaMalloc((void**)&K->acc, (size_t)n_atoms * 4 * sizeof(float)));
  SO3LR_CUDA_CHECK(cudaMalloc((void**)&K->groups, groups.size() * sizeof(int2)));
  SO3LR_CUDA_CHECK(cudaMemcpy(K->groups, groups.data(), groups.size() * sizeof(int2), cudaMemcpyHostToDevice));
  SO3LR_CUDA_CHECK(cudaMemcpy(K->tiles, tiles.data(), tiles.size() * sizeof(int4), cudaMemcpyHostToDevice));
  SO3LR_CUDA_CHECK(cudaMemcpy(K->wgt, wgt.data(), wgt.size() * sizeof(float), cudaMemcpyHostToDevice));
  K->mode = 1;
  return kOk;
}

namespace {
float inverse_volume(const Cell& cell) {
  const float* h = cell.h;
  const double det = (double)h[0] * ((double)h[4] * h[8] - (double)h[5] * h[7]) - (double)h[1] * ((double)h[3] * h[8] - (double)h[5] * h[6]) +
                     (double)h[2] * ((double)h[3] * h[7] - (double)h[4] * h[6]);
  return (float)(1.0 / (det < 0 ? -det : det));
}
}  // namespace

// first half: the quantity that is additive over atoms -- the charge mesh (mode 2) or the structure factors (mode 1) of atoms [0, n).
// A decomposed evaluation sums it over the ranks before the second half.
int kspace_accumulate(cudaStream_t st, const KSpaceDev& K, const Cell& cell, int n, const float* R, const float* q, float** buffer,
                      long long* n_floats) {
  if ((K.mode != 1 && K.mode != 2) || !cell.periodic) return kInvalidArgument;
  if (K.mode == 2) {
    const int n1 = K.shape[0], n2 = K.shape[1], n3 = K.shape[2];
    SO3LR_CUDA_CHECK(cudaMemsetAsync(K.mesh, 0, (size_t)n1 * n2 * n3 * sizeof(float), st));
    { pme_spread_kernel<<<(unsigned)(((long long)n * 4 + 255) / 256), 256, 0, st>>>(cell, n, n1, n2, n3, R, q, K.mesh); count_launch(); }
    if (buffer) *buffer = K.mesh;
    if (n_floats) *n_floats = (long long)n1 * n2 * n3;
  } else {
    SO3LR_CUDA_CHECK(cudaMemsetAsync(K.Sk, 0, (size_t)K.n_tiles * kTileK * sizeof(float2), st));
    // groups of tiles x atom slices
    int splits = (8 * sm_count() + K.n_groups - 1) / K.n_groups;
    const int max_splits = (n + kGroupStage - 1) / kGroupStage;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    int per = (n + splits - 1) / splits;
    per = (per + kGroupStage - 1) / kGroupStage * kGroupStage;
    splits = (n + per - 1) / per;
    { ewald_structure_kernel<<<dim3(K.n_groups, splits), 128, 0, st>>>(cell, n, per, R, q, K.tiles, K.groups, K.Sk); count_launch(); }
    if (buffer) *buffer = reinterpret_cast<float*>(K.Sk);
    if (n_floats) *n_floats = 2LL * K.n_tiles * kTileK;
  }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// second half, for atoms [0, n): potential, forces and (virial_row given) the strain derivative of the whole sum
int kspace_finish(cudaStream_t st, const KSpaceDev& K, const Cell& cell, int n, const float* R, const float* q, const float* total_charge,
                  float* e_coul, float* gq, float* F, float* virial_row, float force_sign) {
  if ((K.mode != 1 && K.mode != 2) || !cell.periodic) return kInvalidArgument;
  const float inv_vol = inverse_volume(cell);
  if (K.mode == 2) {
    CufftApi* f = cufft_api();
    if (!f || !K.plans) return kCudaError;
    const int n1 = K.shape[0], n2 = K.shape[1], n3 = K.shape[2];
    if (f->set_stream(K.plan_r2c, st) != CUFFT_SUCCESS || f->set_stream(K.plan_c2r, st) != CUFFT_SUCCESS) return kCudaError;
    if (f->exec_r2c(K.plan_r2c, K.mesh, reinterpret_cast<cufftComplex*>(K.fq)) != CUFFT_SUCCESS) return kCudaError;
    const long long total = (long long)n1 * n2 * (n3 / 2 + 1);
    { pme_influence_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(cell, inv_vol, K.smearing, n1, n2, n3, K.fq, total_charge, virial_row); count_launch(); }
    if (f->exec_c2r(K.plan_c2r, reinterpret_cast<cufftComplex*>(K.fq), K.mesh) != CUFFT_SUCCESS) return kCudaError;
    { pme_gather_kernel<<<(n + 127) / 128, 128, 0, st>>>(cell, n, n1, n2, n3, R, K.mesh, K.acc); count_launch(); }
  } else {
    SO3LR_CUDA_CHECK(cudaMemsetAsync(K.acc, 0, (size_t)n * 4 * sizeof(float), st));
    // atom blocks x tile slices
    const int blocks = (n + 127) / 128;
    int ksplits = (4 * sm_count() + blocks - 1) / blocks;
    if (ksplits > K.n_tiles) ksplits = K.n_tiles;
    if (ksplits < 1) ksplits = 1;
    const int tper = (K.n_tiles + ksplits - 1) / ksplits;
    ksplits = (K.n_tiles + tper - 1) / tper;
    { ewald_atom_kernel<<<dim3(blocks, ksplits), 128, 0, st>>>(cell, inv_vol, K.smearing, n, K.n_tiles, tper, R, K.tiles, K.wgt, K.Sk, K.acc); count_launch(); }
    if (virial_row) { ewald_virial_kernel<<<K.n_tiles, kTileK, 0, st>>>(cell, inv_vol, K.smearing, K.tiles, K.wgt, K.Sk, total_charge, virial_row); count_launch(); }
  }
  { ewald_finish_kernel<<<(n + 255) / 256, 256, 0, st>>>(cell, inv_vol, K.smearing, n, q, total_charge, K.acc, e_coul, gq, F, force_sign); count_launch(); }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

int launch_ewald(cudaStream_t st, const KSpaceDev& K, const Cell& cell, int n, const float* R, const float* q, const float* total_charge,
                 float* e_coul, float* gq, float* F, float* virial_row, float force_sign) {
  int rc = kspace_accumulate(st, K, cell, n, R, q, nullptr, nullptr);
  if (rc) return rc;
  return kspace_finish(st, K, cell, n, R, q, total_charge, e_coul, gq, F, virial_row, force_sign);
}

}  // namespace so3lr

// First SO3krates layer through per-species-pair tables.
//
// The inputs of layer 0 are constants of the atom's element: x0 = embedding[Z], ev0 = 0.  Its q/k/v rows therefore
// depend on the element only and the attention logits of an edge depend on (Z_i, Z_j, r) only:
//     D_h(Z_i, Z_j, r) = sum_{t in h} q_{Z_i}[t] k_{Z_j}[t] w(r)[t],
// where w(r) is the tabulated radial filter (cubic Hermite, four rows per interval: value, slope, value difference, far
// slope).  The interpolant is linear in those rows, so contracting them with q*k once per element pair gives a table of
// 4 x 8 numbers per interval (4 heads of the invariant branch, 4 degrees of the equivariant branch) that reproduces the
// generic kernel's logits (up to the order of additions) at 128 bytes of table traffic per edge instead of 4 KB of filter
// rows plus 1.5 KB of neighbour rows.
//   forward : lane = list entry; per edge a table lookup, the cutoff, the spherical harmonics; per-element sums of the
//             invariant coefficients are combined with the element's v row at the end
//   backward: only forces leave layer 0.  Lane = list entry evaluates both directions of the edge (the list is symmetric)
//             from the per-atom contractions GV[j][element][head] = sum_{t in head} g_xa[j][t] v_element[t].
#include <algorithm>
#include <vector>

#include "kernels.h"

namespace so3lr {

namespace {

constexpr float kInvNbar = 1.0f / kAvgNumNeighbors;
constexpr float kRc2 = kCutoffSr * kCutoffSr;
constexpr int SP = kMaxTabSpecies;

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }

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

// 32 per-lane partials -> lane L holds the total of entry L
__device__ __forceinline__ float warp_transpose_reduce32(float (&v)[32], int lane) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float send = (lane & 16) ? v[i] : v[i + 16], keep = (lane & 16) ? v[i + 16] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float send = (lane & 8) ? v[i] : v[i + 8], keep = (lane & 8) ? v[i + 8] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float send = (lane & 4) ? v[i] : v[i + 4], keep = (lane & 4) ? v[i + 4] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float send = (lane & 2) ? v[i] : v[i + 2], keep = (lane & 2) ? v[i + 2] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  const float send = (lane & 1) ? v[0] : v[1], keep = (lane & 1) ? v[1] : v[0];
  return keep + __shfl_xor_sync(0xffffffffu, send, 1);
}

// table[(a * SP + b)][interval][32]: the four interval rows of the radial table (value, slope, value difference, far
// slope) contracted with q_a * k_b per head: entry 8 * row + 4 * filter + head.  Sums are formed in double precision.
__global__ void build_pair_table_kernel(const float* __restrict__ radial, const float* __restrict__ qkv_sp, int n_sp,
                                        float* __restrict__ table) {
  const int a = blockIdx.x / n_sp, b = blockIdx.x % n_sp;
  const float* qa = qkv_sp + (size_t)a * kProj;
  const float* kb = qkv_sp + (size_t)b * kProj;
  for (int idx = threadIdx.x; idx < (kTableGrid - 1) * 32; idx += blockDim.x) {
    const int iv = idx >> 5, o = idx & 31;
    const int grp = o & 3, filt = (o >> 2) & 1, row = o >> 3;
    const float* w = radial + ((size_t)iv * 4 + row) * 256 + filt * kF + 32 * grp;
    const float* q = qa + (filt ? 3 * kF : 0) + 32 * grp;
    const float* k = kb + (filt ? 4 * kF : kF) + 32 * grp;
    double s = 0.0;
    for (int t = 0; t < 32; ++t) s += (double)q[t] * (double)k[t] * (double)w[t];
    table[((size_t)(a * SP + b) * (kTableGrid - 1) + iv) * 32 + o] = (float)s;
  }
}

__global__ void __launch_bounds__(256) layer0_fwd_tab_kernel(SpeciesTables T, const float* __restrict__ embed, int n_recv, int n,
                                                             const int* __restrict__ row_ptr, const int* __restrict__ nbr_j,
                                                             const float* __restrict__ dR, const int* __restrict__ Z,
                                                             float* __restrict__ xa, float* __restrict__ ev1) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= n_recv) return;
  const int Zi = Z[i];
  const int zi = T.slot[Zi < 0 ? 0 : (Zi > 118 ? 118 : Zi)];
  float A[32], EV[32];
#pragma unroll
  for (int k = 0; k < 32; ++k) { A[k] = 0.f; EV[k] = 0.f; }
  const int e0 = row_ptr[i], e1 = row_ptr[i + 1];
  for (int e = e0 + lane; e < e1; e += 32) {
    const int j = nbr_j[e];
    const float dx = dR[3 * (size_t)e], dy = dR[3 * (size_t)e + 1], dz = dR[3 * (size_t)e + 2];
    const float r2 = dx * dx + dy * dy + dz * dz;
    if (j < 0 || j >= n || !(r2 < kRc2) || !(r2 > 0.f)) continue;
    const float r = sqrtf(r2), ir = 1.f / r;
    float cut, dcut;
    phys_cutoff(r, cut, dcut);
    const float sc = cut * kInvNbar;
    int g; float4 hv, hd;
    hermite_weights(r, g, hv, hd);
    const int Zj = Z[j];
    const int zj = T.slot[Zj < 0 ? 0 : (Zj > 118 ? 118 : Zj)];
    const float* row = T.table + ((size_t)(zi * SP + zj) * (kTableGrid - 1) + g) * 32;
    const float4 v0a = ld4(row), v0b = ld4(row + 4), m0a = ld4(row + 8), m0b = ld4(row + 12);
    const float4 v1a = ld4(row + 16), v1b = ld4(row + 20), m1a = ld4(row + 24), m1b = ld4(row + 28);   // "v1" = value difference
    float a1[4], a2[4];
    a1[0] = sc * (hv.x * v0a.x + hv.y * m0a.x + hv.z * v1a.x + hv.w * m1a.x);
    a1[1] = sc * (hv.x * v0a.y + hv.y * m0a.y + hv.z * v1a.y + hv.w * m1a.y);
    a1[2] = sc * (hv.x * v0a.z + hv.y * m0a.z + hv.z * v1a.z + hv.w * m1a.z);
    a1[3] = sc * (hv.x * v0a.w + hv.y * m0a.w + hv.z * v1a.w + hv.w * m1a.w);
    a2[0] = sc * (hv.x * v0b.x + hv.y * m0b.x + hv.z * v1b.x + hv.w * m1b.x);
    a2[1] = sc * (hv.x * v0b.y + hv.y * m0b.y + hv.z * v1b.y + hv.w * m1b.y);
    a2[2] = sc * (hv.x * v0b.z + hv.y * m0b.z + hv.z * v1b.z + hv.w * m1b.z);
    a2[3] = sc * (hv.x * v0b.w + hv.y * m0b.w + hv.z * v1b.w + hv.w * m1b.w);
#pragma unroll
    for (int z = 0; z < SP; ++z) {
      const float m = (zj == z) ? 1.f : 0.f;
#pragma unroll
      for (int h = 0; h < 4; ++h) A[4 * z + h] = fmaf(m, a1[h], A[4 * z + h]);
    }
    float Y[kMTot];
    sph_harm_24(dx * ir, dy * ir, dz * ir, Y);
#pragma unroll
    for (int m = 0; m < kMTot; ++m) EV[m] = fmaf(a2[degree_of(m)], Y[m], EV[m]);
  }
  const float At = warp_transpose_reduce32(A, lane);     // lane 4z + h: sum of a1_h over neighbours of element z
  const float Et = warp_transpose_reduce32(EV, lane);    // lane m: ev component m
  const int col = 4 * lane, hL = lane >> 3;
  float4 acc = ld4(embed + (size_t)(Zi < 0 ? 0 : (Zi >= kZEmbed ? kZEmbed - 1 : Zi)) * kF + col);
#pragma unroll
  for (int z = 0; z < SP; ++z) {
    const float c = __shfl_sync(0xffffffffu, At, 4 * z + hL);
    if (z < T.n_species) {
      const float4 v = ld4(T.v_sp + (size_t)z * kF + col);
      acc.x = fmaf(c, v.x, acc.x); acc.y = fmaf(c, v.y, acc.y); acc.z = fmaf(c, v.z, acc.z); acc.w = fmaf(c, v.w, acc.w);
    }
  }
  *reinterpret_cast<float4*>(xa + (size_t)i * kF + col) = acc;
  if (lane < kMTot) ev1[(size_t)i * kMTot + lane] = Et;
}

// GV[a][z][h] = sum_{t in head h} g_xa[a][t] * v_z[t]
__global__ void __launch_bounds__(256) layer0_gv_kernel(SpeciesTables T, int n, const float* __restrict__ g_xa, float* __restrict__ GV) {
  const int lane = threadIdx.x & 31;
  const int a = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (a >= n) return;
  const float4 g = ld4(g_xa + (size_t)a * kF + 4 * lane);
  float out = 0.f;   // lane 4z + h keeps GV[a][z][h]
#pragma unroll
  for (int z = 0; z < SP; ++z) {
    float s = 0.f;
    if (z < T.n_species) {
      const float4 v = ld4(T.v_sp + (size_t)z * kF + 4 * lane);
      s = g.x * v.x + g.y * v.y + g.z * v.z + g.w * v.w;
    }
    s = group8_sum(s);
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const float sh = __shfl_sync(0xffffffffu, s, 8 * h);
      if (lane == 4 * z + h) out = sh;
    }
  }
  GV[(size_t)a * (4 * SP) + lane] = out;
}

__global__ void __launch_bounds__(256) layer0_bwd_tab_kernel(SpeciesTables T, int n_recv, int n, const int* __restrict__ row_ptr,
                                                             const int* __restrict__ nbr_j, const float* __restrict__ dR,
                                                             const int* __restrict__ Z, const float* __restrict__ GV,
                                                             const float* __restrict__ gev1, float* __restrict__ F,
                                                             float* __restrict__ virial) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= n_recv) return;
  const int Zi = Z[i];
  const int zi = T.slot[Zi < 0 ? 0 : (Zi > 118 ? 118 : Zi)];
  const float* GVi = GV + (size_t)i * (4 * SP);
  float gevi[kMTot];
#pragma unroll
  for (int c = 0; c < 6; ++c) {
    const float4 v = ld4(gev1 + (size_t)i * kMTot + 4 * c);
    gevi[4 * c] = v.x; gevi[4 * c + 1] = v.y; gevi[4 * c + 2] = v.z; gevi[4 * c + 3] = v.w;
  }
  float fx = 0.f, fy = 0.f, fz = 0.f;
  VirialAcc va;
  const int e0 = row_ptr[i], e1 = row_ptr[i + 1];
  for (int e = e0 + lane; e < e1; e += 32) {
    const int j = nbr_j[e];
    const float dx = dR[3 * (size_t)e], dy = dR[3 * (size_t)e + 1], dz = dR[3 * (size_t)e + 2];
    const float r2 = dx * dx + dy * dy + dz * dz;
    if (j < 0 || j >= n || !(r2 < kRc2) || !(r2 > 0.f)) continue;
    const float r = sqrtf(r2), ir = 1.f / r;
    const float ux = dx * ir, uy = dy * ir, uz = dz * ir;
    float cut, dcut;
    phys_cutoff(r, cut, dcut);
    const float sc = cut * kInvNbar, dcn = dcut * kInvNbar;
    int g; float4 hv, hd;
    hermite_weights(r, g, hv, hd);
    const int Zj = Z[j];
    const int zj = T.slot[Zj < 0 ? 0 : (Zj > 118 ? 118 : Zj)];
    float Y[kMTot];
    sph_harm_24(ux, uy, uz, Y);
    const float* gevj = gev1 + (size_t)j * kMTot;
    float dA2[4] = {0.f, 0.f, 0.f, 0.f}, dB2[4] = {0.f, 0.f, 0.f, 0.f}, gj[kMTot];
#pragma unroll
    for (int c = 0; c < 6; ++c) {
      const float4 v = ld4(gevj + 4 * c);
      gj[4 * c] = v.x; gj[4 * c + 1] = v.y; gj[4 * c + 2] = v.z; gj[4 * c + 3] = v.w;
    }
#pragma unroll
    for (int m = 0; m < kMTot; ++m) {
      dA2[degree_of(m)] = fmaf(gevi[m], Y[m], dA2[degree_of(m)]);
      dB2[degree_of(m)] = fmaf(gj[m], Y[m], dB2[degree_of(m)]);
    }
    dB2[0] = -dB2[0]; dB2[2] = -dB2[2];       // Y_lm(-u) = (-1)^l Y_lm(u)
    const float4 dA1 = ld4(GVi + 4 * zj);                          // cotangents of the invariant coefficients, edge (i<-j)
    const float4 dB1 = ld4(GV + (size_t)j * (4 * SP) + 4 * zi);    // and edge (j<-i)
    float gr = 0.f, a2A[4], a2B[4];
#pragma unroll
    for (int dir = 0; dir < 2; ++dir) {
      const float* row = T.table + ((size_t)((dir ? zj : zi) * SP + (dir ? zi : zj)) * (kTableGrid - 1) + g) * 32;
      const float4 v0a = ld4(row), v0b = ld4(row + 4), m0a = ld4(row + 8), m0b = ld4(row + 12);
      const float4 v1a = ld4(row + 16), v1b = ld4(row + 20), m1a = ld4(row + 24), m1b = ld4(row + 28);
      const float4 d1 = dir ? dB1 : dA1;
      const float* d2 = dir ? dB2 : dA2;
      const float D1[4] = {hv.x * v0a.x + hv.y * m0a.x + hv.z * v1a.x + hv.w * m1a.x, hv.x * v0a.y + hv.y * m0a.y + hv.z * v1a.y + hv.w * m1a.y,
                           hv.x * v0a.z + hv.y * m0a.z + hv.z * v1a.z + hv.w * m1a.z, hv.x * v0a.w + hv.y * m0a.w + hv.z * v1a.w + hv.w * m1a.w};
      const float D2[4] = {hv.x * v0b.x + hv.y * m0b.x + hv.z * v1b.x + hv.w * m1b.x, hv.x * v0b.y + hv.y * m0b.y + hv.z * v1b.y + hv.w * m1b.y,
                           hv.x * v0b.z + hv.y * m0b.z + hv.z * v1b.z + hv.w * m1b.z, hv.x * v0b.w + hv.y * m0b.w + hv.z * v1b.w + hv.w * m1b.w};
      const float E1[4] = {hd.x * v0a.x + hd.y * m0a.x + hd.z * v1a.x + hd.w * m1a.x, hd.x * v0a.y + hd.y * m0a.y + hd.z * v1a.y + hd.w * m1a.y,
                           hd.x * v0a.z + hd.y * m0a.z + hd.z * v1a.z + hd.w * m1a.z, hd.x * v0a.w + hd.y * m0a.w + hd.z * v1a.w + hd.w * m1a.w};
      const float E2[4] = {hd.x * v0b.x + hd.y * m0b.x + hd.z * v1b.x + hd.w * m1b.x, hd.x * v0b.y + hd.y * m0b.y + hd.z * v1b.y + hd.w * m1b.y,
                           hd.x * v0b.z + hd.y * m0b.z + hd.z * v1b.z + hd.w * m1b.z, hd.x * v0b.w + hd.y * m0b.w + hd.z * v1b.w + hd.w * m1b.w};
      const float d1v[4] = {d1.x, d1.y, d1.z, d1.w};
      float dsc = 0.f, dder = 0.f;
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        dsc = fmaf(d1v[h], D1[h], fmaf(d2[h], D2[h], dsc));
        dder = fmaf(d1v[h], E1[h], fmaf(d2[h], E2[h], dder));
        if (dir == 0) a2A[h] = sc * D2[h]; else a2B[h] = sc * D2[h];
      }
      gr += dcn * dsc + sc * dder;
    }
    float gY[kMTot];
#pragma unroll
    for (int m = 0; m < kMTot; ++m) {
      const int l = degree_of(m);
      const float sgn = (l == 0 || l == 2) ? -1.f : 1.f;
      gY[m] = a2A[l] * gevi[m] + sgn * a2B[l] * gj[m];
    }
    float gux, guy, guz;
    sph_harm_24_vjp(ux, uy, uz, gY, gux, guy, guz);
    const float gd = gux * ux + guy * uy + guz * uz;
    const float fsx = gr * ux + (gux - gd * ux) * ir;
    const float fsy = gr * uy + (guy - gd * uy) * ir;
    const float fsz = gr * uz + (guz - gd * uz) * ir;
    fx += fsx; fy += fsy; fz += fsz;
    if (virial) va.add(0.5f, dx, dy, dz, fsx, fsy, fsz);
  }
  fx = warp_sum(fx); fy = warp_sum(fy); fz = warp_sum(fz);
  if (lane == 0) { F[3 * (size_t)i] += fx; F[3 * (size_t)i + 1] += fy; F[3 * (size_t)i + 2] += fz; }
  if (virial) va.flush_warp(virial, (size_t)i, lane);
}

}  // namespace

// (Re)builds the tables for the elements present in Z_host; returns kOk with T->n_species = 0 when more than
// kMaxTabSpecies elements occur (the caller then uses the generic kernels).
int species_tables_build(cudaStream_t st, const ModelDev& M, const int* Z_host, int n, SpeciesTables* T) {
  std::vector<int> sp;
  for (int a = 0; a < n; ++a) {
    int z = Z_host[a];
    z = z < 0 ? 0 : (z > 118 ? 118 : z);
    if (std::find(sp.begin(), sp.end(), z) == sp.end()) sp.push_back(z);
    if ((int)sp.size() > SP) break;
  }
  if ((int)sp.size() > SP || sp.empty()) { T->n_species = 0; return kOk; }
  std::sort(sp.begin(), sp.end());
  bool same = T->n_species == (int)sp.size();
  for (int k = 0; same && k < (int)sp.size(); ++k) same = T->species[k] == sp[k];
  if (same && T->table) return kOk;
  if (!T->table) {
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&T->table, (size_t)SP * SP * (kTableGrid - 1) * 32 * sizeof(float)));
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&T->v_sp, (size_t)SP * kF * sizeof(float)));
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&T->slot, 119 * sizeof(int)));
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&T->qkv_sp, (size_t)SP * kProj * sizeof(float)));
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&T->x_sp, (size_t)SP * kF * sizeof(float)));
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&T->z_sp, SP * sizeof(int)));
  }
  const int ns = (int)sp.size();
  int slot[119];
  for (int z = 0; z < 119; ++z) slot[z] = 0;
  for (int k = 0; k < ns; ++k) { slot[sp[k]] = k; T->species[k] = sp[k]; }
  T->n_species = ns;
  SO3LR_CUDA_CHECK(cudaMemcpyAsync(T->slot, slot, sizeof(slot), cudaMemcpyHostToDevice, st));
  SO3LR_CUDA_CHECK(cudaMemcpyAsync(T->z_sp, sp.data(), ns * sizeof(int), cudaMemcpyHostToDevice, st));
  SO3LR_CUDA_CHECK(cudaStreamSynchronize(st));   // the host arrays above go out of scope
  launch_embed(st, M, T->z_sp, ns, T->x_sp);
  launch_proj_fwd(st, M.layer[0], T->x_sp, ns, T->qkv_sp);
  SO3LR_CUDA_CHECK(cudaMemcpy2DAsync(T->v_sp, kF * sizeof(float), T->qkv_sp + 2 * kF, kProj * sizeof(float), kF * sizeof(float), ns,
                                     cudaMemcpyDeviceToDevice, st));
  { build_pair_table_kernel<<<ns * ns, 256, 0, st>>>(M.layer[0].table, T->qkv_sp, ns, T->table); count_launch(); }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

void species_tables_free(SpeciesTables* T) {
  cudaFree(T->table); cudaFree(T->v_sp); cudaFree(T->slot); cudaFree(T->qkv_sp); cudaFree(T->x_sp); cudaFree(T->z_sp);
  *T = SpeciesTables{};
}

void launch_layer0_fwd_tab(cudaStream_t s, const SpeciesTables& T, const ModelDev& M, int n_recv, int n, const int* row_ptr,
                           const int* nbr_j, const float* dR, const int* Z, float* xa, float* ev1) {
  if (n_recv <= 0) return;
  { layer0_fwd_tab_kernel<<<(n_recv + 7) / 8, 256, 0, s>>>(T, M.embed_z, n_recv, n, row_ptr, nbr_j, dR, Z, xa, ev1); count_launch(); }
}

void launch_layer0_bwd_tab(cudaStream_t s, const SpeciesTables& T, int n_recv, int n_gv, int n, const int* row_ptr, const int* nbr_j,
                           const float* dR, const int* Z, const float* g_xa, const float* gev1, float* GV, float* F, float* virial) {
  if (n_recv <= 0) return;
  { layer0_gv_kernel<<<(n_gv + 7) / 8, 256, 0, s>>>(T, n_gv, g_xa, GV); count_launch(); }
  { layer0_bwd_tab_kernel<<<(n_recv + 7) / 8, 256, 0, s>>>(T, n_recv, n, row_ptr, nbr_j, dR, Z, GV, gev1, F, virial); count_launch(); }
}

}  // namespace so3lr

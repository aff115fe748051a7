// Edge geometry + ZBL repulsion on the short-range graph, the fused long-range pair kernel (damped Coulomb +
// dispersion with analytic gradients) and the small per-graph reductions around them.
#include "kernels.h"

namespace so3lr {

namespace {

__global__ void sr_geometry_zbl_kernel(ZblParams zbl, Cell cell, int n, long long n_edges, const int* __restrict__ edge_i,
                                       const int* __restrict__ nbr_j, const int* __restrict__ Z, const float* __restrict__ R,
                                       int dR_given, float* __restrict__ dR, float* __restrict__ e_atom,
                                       float* __restrict__ g_dR, const float* __restrict__ ge, float* __restrict__ F_direct, int n_owned,
                                       float* __restrict__ virial) {
  long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_edges) return;
  const int i = edge_i[e], j = nbr_j[e];
  float dx = 0.f, dy = 0.f, dz = 0.f;
  const bool valid = i >= 0 && i < n && j >= 0 && j < n;
  if (dR_given) {
    dx = dR[3 * e]; dy = dR[3 * e + 1]; dz = dR[3 * e + 2];
  } else {
    if (valid) {
      dx = R[3 * (size_t)j] - R[3 * (size_t)i];
      dy = R[3 * (size_t)j + 1] - R[3 * (size_t)i + 1];
      dz = R[3 * (size_t)j + 2] - R[3 * (size_t)i + 2];
      min_image(cell, dx, dy, dz);
    }
    dR[3 * e] = dx; dR[3 * e + 1] = dy; dR[3 * e + 2] = dz;
  }
  float gx = 0.f, gy = 0.f, gz = 0.f;
  const float r2 = dx * dx + dy * dy + dz * dz;
  // n_owned >= 0: only the edges of owned receivers carry energy, and the receiver takes the pair's whole force
  // (the reversed edge belongs to the other atom's owner)
  if (valid && r2 > 0.f && r2 < kZblSwitchOff * kZblSwitchOff && (n_owned < 0 || i < n_owned)) {
    const float r = sqrtf(r2);
    float cut, dcut, ez, dez;
    phys_cutoff(r, cut, dcut);
    zbl_edge(zbl, r, cut, dcut, Z[i], Z[j], ez, dez);
    atomicAdd(e_atom + i, ez);
    const float s = (ge ? ge[i] : 1.f) * dez / r;
    gx = s * dx; gy = s * dy; gz = s * dz;
    if (virial) {     // every directed edge carries its own energy: dE/d eps += dR (x) g
      float* w = virial + 6 * (size_t)i;
      atomicAdd(w, dx * gx); atomicAdd(w + 1, dy * gy); atomicAdd(w + 2, dz * gz);
      atomicAdd(w + 3, dy * gz); atomicAdd(w + 4, dx * gz); atomicAdd(w + 5, dx * gy);
    }
    if (F_direct) {   // only edges shorter than 1.5 A get here: a handful per atom
      const float wi = n_owned >= 0 ? 2.f : 1.f;
      atomicAdd(F_direct + 3 * (size_t)i, wi * gx); atomicAdd(F_direct + 3 * (size_t)i + 1, wi * gy); atomicAdd(F_direct + 3 * (size_t)i + 2, wi * gz);
      if (n_owned < 0) {
        atomicAdd(F_direct + 3 * (size_t)j, -gx); atomicAdd(F_direct + 3 * (size_t)j + 1, -gy); atomicAdd(F_direct + 3 * (size_t)j + 2, -gz);
      }
    }
  }
  if (g_dR) { g_dR[3 * e] = gx; g_dR[3 * e + 1] = gy; g_dR[3 * e + 2] = gz; }
}

__global__ void force_scatter_kernel(int n, long long n_edges, const int* __restrict__ edge_i, const int* __restrict__ nbr_j,
                                     const float* __restrict__ g_dR, float* __restrict__ F) {
  long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_edges) return;
  const float gx = g_dR[3 * e], gy = g_dR[3 * e + 1], gz = g_dR[3 * e + 2];
  if (gx == 0.f && gy == 0.f && gz == 0.f) return;
  const int i = edge_i[e], j = nbr_j[e];
  if (i < 0 || i >= n || j < 0 || j >= n) return;
  // E depends on dR = R_j - R_i:  F_i = +g, F_j = -g
  atomicAdd(F + 3 * (size_t)i, gx); atomicAdd(F + 3 * (size_t)i + 1, gy); atomicAdd(F + 3 * (size_t)i + 2, gz);
  atomicAdd(F + 3 * (size_t)j, -gx); atomicAdd(F + 3 * (size_t)j + 1, -gy); atomicAdd(F + 3 * (size_t)j + 2, -gz);
}

// one warp per row i; lanes stride over the row's pairs
// Device forms of the pair terms for the long-range kernels: the same functions as coulomb_chi / dispersion_pair_fast / switching
// of pair_terms.cuh with approximate reciprocals and exponentials (rcp.approx, ex2.approx, lg2.approx: 1-2 ulp each) in place
// of IEEE divisions and libm calls, and the switch written with one exponential:
//   s(1-c) / (s(1-c) + s(c)),  s(a) = exp(-1/a)   ==   1 / (1 + E),  E = exp(1/(1-c) - 1/c)
__device__ __forceinline__ float rcp_fast(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void switching_dev(float x, float on, float off, float& f, float& df) {
  const float iw = rcp_fast(off - on);
  const float c = (x - on) * iw;
  if (c <= 0.f) { f = 1.f; df = 0.f; return; }
  if (c >= 1.f) { f = 0.f; df = 0.f; return; }
  const float ia = rcp_fast(1.f - c), ib = rcp_fast(c);
  const float t = fminf(fmaxf(ia - ib, -80.f), 80.f);
  const float E = __expf(t);
  f = rcp_fast(1.f + E);
  df = -(E * f) * (f * (ia * ia + ib * ib)) * iw;   // in this order no intermediate leaves the float range
}
__device__ __forceinline__ void coulomb_chi_dev(const LrParams& p, float r, float rinv, float& chi, float& dchi) {
  const float inv_sig = 1.f / kSigmaCoulomb;
  const float x = r * inv_sig;
  float pot = erff(x) * rinv;
  float dpot = (1.1283791670955126f * inv_sig * __expf(-x * x) - pot) * rinv;
  if (p.k_alpha > 0.f) {     // the reciprocal-space sum holds erf(r k_alpha) / r
    const float y = r * p.k_alpha;
    const float potk = erff(y) * rinv;
    pot -= potk;
    dpot -= (1.1283791670955126f * p.k_alpha * __expf(-y * y) - potk) * rinv;
  }
  if (!p.has_cutoff) { chi = pot; dchi = dpot; return; }
  float f, df;
  switching_dev(r, p.cuton, p.rc, f, df);
  chi = (pot - p.v_rc) - (1.f - f) * (r - p.rc) * p.dv_rc;
  dchi = dpot - (1.f - f) * p.dv_rc + df * (r - p.rc) * p.dv_rc;
}
// ai = alpha_free h, ci = c6_free h^2 of both atoms come precomputed per atom
__device__ __forceinline__ void dispersion_pair_dev(const LrParams& P, float r, float alf_i, float c6f_i, float hi, float alf_j, float c6f_j,
                                                    float hj, float& e, float& de_dr, float& de_dhi, float& de_dhj) {
  const float ai = alf_i * hi, aj = alf_j * hj, ci = c6f_i * hi * hi, cj = c6f_j * hj * hj;
  const float iden = rcp_fast(ai * ai * cj + aj * aj * ci);
  const float c6 = 2.f * ci * cj * ai * aj * iden;
  const float dlc6_dhi = (rcp_fast(ai) - 2.f * ai * cj * iden) * alf_i + (rcp_fast(ci) - aj * aj * iden) * 2.f * c6f_i * hi;
  const float dlc6_dhj = (rcp_fast(aj) - 2.f * aj * ci * iden) * alf_j + (rcp_fast(cj) - ai * ai * iden) * 2.f * c6f_j * hj;
  const float aij = 0.5f * (ai + aj);
  const float a17 = exp2f(__log2f(aij) * (1.f / 7.f));
  const float fs = 2.5527961000248887f;
  const float rv = fs * a17;
  const float sg = ((-0.00078893f * rv + 0.04125273f) * rv + 0.24428889f) * rv + (-0.00433008f);
  const float dsg = ((3.f * -0.00078893f) * rv + 2.f * 0.04125273f) * rv + 0.24428889f;
  const float ig = 2.f * sg * sg;
  const float kp = kDispersionScale * 2.f * 2.54f;
  const float p = kp * a17;
  const float R = r * (1.f / kBohr);
  const float R2 = R * R, p2 = p * p;
  const float R4 = R2 * R2, p4 = p2 * p2;
  const float R6 = R4 * R2, p6 = p4 * p2, R8 = R4 * R4, p8 = p4 * p4, R10 = R8 * R2, p10 = p8 * p2;
  const float i6 = rcp_fast(R6 + p6), i8 = rcp_fast(R8 + p8), i10 = rcp_fast(R10 + p10);
  const float t8 = 5.f * ig, t10 = 30.625f * ig * ig;
  const float T = i6 + t8 * i8 + t10 * i10;
  const float dT_dR = -(6.f * R4 * R * i6 * i6 + t8 * 8.f * R6 * R * i8 * i8 + t10 * 10.f * R8 * R * i10 * i10);
  const float dT_dp = -(6.f * p4 * p * i6 * i6 + t8 * 8.f * p6 * p * i8 * i8 + t10 * 10.f * p8 * p * i10 * i10);
  const float dT_dig = 5.f * i8 + 61.25f * ig * i10;
  const float dT_da17 = dT_dp * kp + dT_dig * 4.f * sg * dsg * fs;
  const float da17_dh = a17 * rcp_fast(7.f * aij) * 0.5f;
  float f = 1.f, df = 0.f;
  if (P.has_cutoff && P.has_damping) switching_dev(r, P.disp_on, P.rc, f, df);
  const float pre = -kHartree * c6;
  e = pre * T * f;
  de_dr = pre * (dT_dR * (1.f / kBohr) * f + T * df);
  de_dhi = pre * f * (T * dlc6_dhi + dT_da17 * da17_dh * alf_i);
  de_dhj = pre * f * (T * dlc6_dhj + dT_da17 * da17_dh * alf_j);
}

template <int MODE>
__global__ void __launch_bounds__(256) pair_lr_kernel(LrParams P, Cell cell, int n, const int* __restrict__ row_ptr,
                                                      const int* __restrict__ nbr_j, const int* __restrict__ Z,
                                                      const float* __restrict__ R, const float* __restrict__ q,
                                                      const float* __restrict__ h, const float* __restrict__ dR_lr,
                                                      float* __restrict__ g_dR_lr, float* __restrict__ e_atom,
                                                      float* __restrict__ F, float* __restrict__ gq, float* __restrict__ gh,
                                                      float* __restrict__ e_coul, float* __restrict__ e_disp, const float* __restrict__ ge,
                                                      float* __restrict__ virial) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= n) return;
  VirialAcc va;
  const int e0 = row_ptr[i], e1 = row_ptr[i + 1];
  if (e0 == e1) return;
  const float qi = q[i], hi = h[i];
  const int Zi = Z[i];
  const float gei = ge ? ge[i] : 1.f;
  float xi = 0.f, yi = 0.f, zi = 0.f;
  if (MODE == 0) { xi = R[3 * (size_t)i]; yi = R[3 * (size_t)i + 1]; zi = R[3 * (size_t)i + 2]; }
  float ec = 0.f, ed = 0.f, fx = 0.f, fy = 0.f, fz = 0.f, gqi = 0.f, ghi = 0.f;
  for (int e = e0 + lane; e < e1; e += 32) {
    const int j = nbr_j[e];
    float gx = 0.f, gy = 0.f, gz = 0.f;
    if (j >= 0 && j < n) {
      float dx, dy, dz;
      if (MODE == 0) {
        dx = R[3 * (size_t)j] - xi; dy = R[3 * (size_t)j + 1] - yi; dz = R[3 * (size_t)j + 2] - zi;
        min_image(cell, dx, dy, dz);
      } else {
        dx = dR_lr[3 * (size_t)e]; dy = dR_lr[3 * (size_t)e + 1]; dz = dR_lr[3 * (size_t)e + 2];
      }
      const float r2 = dx * dx + dy * dy + dz * dz;
      if (r2 > 0.f && (!P.has_cutoff || r2 < P.rc * P.rc)) {
        const float rinv = rsqrtf(r2), r = r2 * rinv;
        float chi, dchi;
        coulomb_chi_dev(P, r, rinv, chi, dchi);
        const float qj = q[j], hj = h[j];
        const float pf = P.pair_factor;
        const float kq = pf * kKe;
        const float e_c = kq * qi * qj * chi;
        float e_d, dd_dr, dd_dhi, dd_dhj;
        const int Zj = Z[j];
        dispersion_pair_dev(P, r, alpha_free(Zi), c6_free(Zi), hi, alpha_free(Zj), c6_free(Zj), hj, e_d, dd_dr, dd_dhi, dd_dhj);
        e_d *= pf; dd_dr *= pf; dd_dhi *= pf; dd_dhj *= pf;
        ec += e_c; ed += e_d;
        gqi = fmaf(kq * qj, chi, gqi);
        ghi += dd_dhi;
        atomicAdd(gq + j, gei * kq * qi * chi);
        atomicAdd(gh + j, gei * dd_dhj);
        const float de_dr = gei * (kq * qi * qj * dchi + dd_dr);
        const float s = de_dr * rinv;
        gx = s * dx; gy = s * dy; gz = s * dz;   // dE/d(dR), dR = R_j - R_i
        if (MODE == 0) {
          if (virial) va.add(1.f, dx, dy, dz, gx, gy, gz);     // every listed pair carries its own share of the energy
          fx += gx; fy += gy; fz += gz;
          atomicAdd(F + 3 * (size_t)j, -gx); atomicAdd(F + 3 * (size_t)j + 1, -gy); atomicAdd(F + 3 * (size_t)j + 2, -gz);
        }
      }
    }
    if (MODE == 1) { g_dR_lr[3 * (size_t)e] = gx; g_dR_lr[3 * (size_t)e + 1] = gy; g_dR_lr[3 * (size_t)e + 2] = gz; }
  }
  ec = warp_sum(ec); ed = warp_sum(ed); gqi = warp_sum(gqi); ghi = warp_sum(ghi);
  if (MODE == 0) { fx = warp_sum(fx); fy = warp_sum(fy); fz = warp_sum(fz); }
  if (lane == 0) {
    if (e_atom) atomicAdd(e_atom + i, ec + ed);
    if (e_coul) atomicAdd(e_coul + i, ec);
    if (e_disp) atomicAdd(e_disp + i, ed);
    atomicAdd(gq + i, gei * gqi);
    atomicAdd(gh + i, gei * ghi);
    if (MODE == 0) { atomicAdd(F + 3 * (size_t)i, fx); atomicAdd(F + 3 * (size_t)i + 1, fy); atomicAdd(F + 3 * (size_t)i + 2, fz); }
  }
  if (MODE == 0 && virial) va.flush_warp(virial, (size_t)i, lane);
}

// The single-device long-range kernel with packed operands: per atom (x, y, z, q) and (h, alpha_free, c6_free, -) so that a pair costs two
// 16-byte gathers, and a packed accumulator (Fx, Fy, Fz, dE/dq) so that the sender's share of a pair is one
// vector reduction (red.global.add.v4.f32) and one scalar one (dE/dh) instead of five scalar atomics.
__global__ void __launch_bounds__(256) pair_pack_kernel(int n, const float* __restrict__ R, const float* __restrict__ q,
                                                        const float* __restrict__ h, const int* __restrict__ Z,
                                                        float4* __restrict__ pq, float4* __restrict__ hz, float4* __restrict__ acc) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  pq[i] = make_float4(R[3 * (size_t)i], R[3 * (size_t)i + 1], R[3 * (size_t)i + 2], q[i]);
  hz[i] = make_float4(h[i], alpha_free(Z[i]), c6_free(Z[i]), 0.f);
  acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}
__global__ void __launch_bounds__(256) pair_unpack_kernel(int n, const float4* __restrict__ acc, float* __restrict__ F, float* __restrict__ gq) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float4 a = acc[i];
  F[3 * (size_t)i] += a.x; F[3 * (size_t)i + 1] += a.y; F[3 * (size_t)i + 2] += a.z;
  gq[i] += a.w;
}
__device__ __forceinline__ void red_add_f4(float4* p, float x, float y, float z, float w) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
__global__ void __launch_bounds__(256) pair_lr_packed_kernel(LrParams P, Cell cell, int n, const int* __restrict__ row_ptr,
                                                             const int* __restrict__ nbr_j, const float4* __restrict__ pq,
                                                             const float4* __restrict__ hz, float4* __restrict__ acc,
                                                             float* __restrict__ gh, float* __restrict__ e_coul,
                                                             float* __restrict__ e_disp, float* __restrict__ virial) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= n) return;
  VirialAcc va;
  const int e0 = row_ptr[i], e1 = row_ptr[i + 1];
  if (e0 == e1) return;
  const float4 pi = pq[i];
  const float4 hzi = hz[i];
  const float qi = pi.w, hi = hzi.x;
  const float pf = P.pair_factor, kq = pf * kKe, rc2 = P.rc * P.rc;
  float ec = 0.f, ed = 0.f, fx = 0.f, fy = 0.f, fz = 0.f, gqi = 0.f, ghi = 0.f;
  for (int e = e0 + lane; e < e1; e += 32) {
    const int j = nbr_j[e];
    if (j < 0 || j >= n) continue;
    const float4 pj = __ldg(pq + j);
    float dx = pj.x - pi.x, dy = pj.y - pi.y, dz = pj.z - pi.z;
    min_image(cell, dx, dy, dz);
    const float r2 = dx * dx + dy * dy + dz * dz;
    if (!(r2 > 0.f) || (P.has_cutoff && r2 >= rc2)) continue;
    const float4 hzj = __ldg(hz + j);
    const float rinv = rsqrtf(r2), r = r2 * rinv;
    float chi, dchi;
    coulomb_chi_dev(P, r, rinv, chi, dchi);
    const float qj = pj.w;
    float e_d, dd_dr, dd_dhi, dd_dhj;
    dispersion_pair_dev(P, r, hzi.y, hzi.z, hi, hzj.y, hzj.z, hzj.x, e_d, dd_dr, dd_dhi, dd_dhj);
    ec = fmaf(kq * qi * qj, chi, ec);
    ed = fmaf(pf, e_d, ed);
    gqi = fmaf(kq * qj, chi, gqi);
    ghi = fmaf(pf, dd_dhi, ghi);
    const float s = (kq * qi * qj * dchi + pf * dd_dr) * rinv;
    const float gx = s * dx, gy = s * dy, gz = s * dz;   // dE/d(dR), dR = R_j - R_i
    if (virial) va.add(1.f, dx, dy, dz, gx, gy, gz);
    fx += gx; fy += gy; fz += gz;
    red_add_f4(acc + j, -gx, -gy, -gz, kq * qi * chi);
    atomicAdd(gh + j, pf * dd_dhj);
  }
  ec = warp_sum(ec); ed = warp_sum(ed); gqi = warp_sum(gqi); ghi = warp_sum(ghi);
  fx = warp_sum(fx); fy = warp_sum(fy); fz = warp_sum(fz);
  if (lane == 0) {
    e_coul[i] += ec;     // only this warp writes the energies of row i
    e_disp[i] += ed;
    red_add_f4(acc + i, fx, fy, fz, gqi);
    atomicAdd(gh + i, ghi);
  }
  if (virial) va.flush_warp(virial, (size_t)i, lane);
}

// Owned rows of an ordered list over owned atoms and ghosts (decomposed runs; ghosts carry the larger indices, so the list
// holds every pair of two owned atoms once and every owned-ghost pair in the owned atom's row).  A pair of two owned atoms
// books its whole energy on the row atom and scatters the other end's derivatives with atomics; a pair with a ghost end books
// half of the energy and the row atom's derivatives only (the ghost's owner does the same from its side).  gq, gh and F_add
// must hold the values to add to (zeros for gq, gh) when the kernel starts.
__global__ void __launch_bounds__(256) pair_lr_owned_kernel(LrParams P, Cell cell, int n_owned, int n, const int* __restrict__ row_ptr,
                                                            const int* __restrict__ nbr_j, const int* __restrict__ Z,
                                                            const float* __restrict__ R, const float* __restrict__ q,
                                                            const float* __restrict__ h, float* __restrict__ F_add,
                                                            float* __restrict__ gq, float* __restrict__ gh, float* __restrict__ e_coul,
                                                            float* __restrict__ e_disp, float* __restrict__ virial) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= n_owned) return;
  const int e0 = row_ptr[i], e1 = row_ptr[i + 1];
  const float qi = q[i], hi = h[i];
  const float alf_i = alpha_free(Z[i]), c6f_i = c6_free(Z[i]);
  const float xi = R[3 * (size_t)i], yi = R[3 * (size_t)i + 1], zi = R[3 * (size_t)i + 2];
  float ec = 0.f, ed = 0.f, fx = 0.f, fy = 0.f, fz = 0.f, gqi = 0.f, ghi = 0.f;
  VirialAcc va;
  for (int e = e0 + lane; e < e1; e += 32) {
    const int j = nbr_j[e];
    if (j < 0 || j >= n) continue;
    float dx = R[3 * (size_t)j] - xi, dy = R[3 * (size_t)j + 1] - yi, dz = R[3 * (size_t)j + 2] - zi;
    min_image(cell, dx, dy, dz);
    const float r2 = dx * dx + dy * dy + dz * dz;
    if (!(r2 > 0.f) || (P.has_cutoff && r2 >= P.rc * P.rc)) continue;
    const float rinv = rsqrtf(r2), r = r2 * rinv;
    float chi, dchi;
    coulomb_chi_dev(P, r, rinv, chi, dchi);
    const float qj = q[j], hj = h[j];
    const int Zj = Z[j];
    float e_d, dd_dr, dd_dhi, dd_dhj;
    dispersion_pair_dev(P, r, alf_i, c6f_i, hi, alpha_free(Zj), c6_free(Zj), hj, e_d, dd_dr, dd_dhi, dd_dhj);
    const bool both = j < n_owned;
    const float w = both ? 1.f : 0.5f;                             // share of the pair energy booked on this row
    ec = fmaf(w * kKe * qi * qj, chi, ec);
    ed = fmaf(w, e_d, ed);
    gqi = fmaf(kKe * qj, chi, gqi);
    ghi += dd_dhi;
    const float s = (kKe * qi * qj * dchi + dd_dr) * rinv;   // dE_ij/d(dR), dR = R_j - R_i; F_i = +that, F_j = -that
    const float gx = s * dx, gy = s * dy, gz = s * dz;
    fx += gx; fy += gy; fz += gz;
    if (virial) va.add(w * s, dx, dy, dz, dx, dy, dz);
    if (both) {
      atomicAdd(gq + j, kKe * qi * chi);
      atomicAdd(gh + j, dd_dhj);
      atomicAdd(F_add + 3 * (size_t)j, -gx); atomicAdd(F_add + 3 * (size_t)j + 1, -gy); atomicAdd(F_add + 3 * (size_t)j + 2, -gz);
    }
  }
  ec = warp_sum(ec); ed = warp_sum(ed); gqi = warp_sum(gqi); ghi = warp_sum(ghi);
  fx = warp_sum(fx); fy = warp_sum(fy); fz = warp_sum(fz);
  if (lane == 0) {
    e_coul[i] = ec; e_disp[i] = ed;      // only this warp writes the energies of row i
    atomicAdd(gq + i, gqi); atomicAdd(gh + i, ghi);
    atomicAdd(F_add + 3 * (size_t)i, fx); atomicAdd(F_add + 3 * (size_t)i + 1, fy); atomicAdd(F_add + 3 * (size_t)i + 2, fz);
  }
  if (virial) va.flush_warp(virial, (size_t)i, lane);
}

// one CTA per graph: q = q_raw + (Q - sum q_raw) / n_g ; h = |hv|
__global__ void charge_conserve_kernel(int n_graphs, const int* __restrict__ graph_start, const float* __restrict__ q_raw,
                                       const float* __restrict__ total_charge, const float* __restrict__ hv,
                                       float* __restrict__ q, float* __restrict__ h) {
  __shared__ float red[32];
  const int g = blockIdx.x;
  const int a0 = graph_start[g], a1 = graph_start[g + 1];
  float s = 0.f;
  for (int a = a0 + threadIdx.x; a < a1; a += blockDim.x) s += q_raw[a];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  const float Q = total_charge ? total_charge[g] : 0.f;
  // the shift is applied in double: rounded to float32 first, its relative error times the atom count would show up in sum q
  const double corr = a1 > a0 ? ((double)Q - (double)red[0]) / (double)(a1 - a0) : 0.0;
  for (int a = a0 + threadIdx.x; a < a1; a += blockDim.x) {
    q[a] = (float)((double)q_raw[a] + corr);
    h[a] = fabsf(hv[a]);
  }
}

// gq_raw = gq - mean_graph(gq)
__global__ void charge_conserve_bwd_kernel(int n_graphs, const int* __restrict__ graph_start, const float* __restrict__ gq,
                                           float* __restrict__ gq_raw) {
  __shared__ float red[32];
  const int g = blockIdx.x;
  const int a0 = graph_start[g], a1 = graph_start[g + 1];
  float s = 0.f;
  for (int a = a0 + threadIdx.x; a < a1; a += blockDim.x) s += gq[a];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  const float mean = a1 > a0 ? red[0] / (float)(a1 - a0) : 0.f;
  for (int a = a0 + threadIdx.x; a < a1; a += blockDim.x) gq_raw[a] = gq[a] - mean;
}

// per-graph energy (double accumulation) and dipole sum_i q_i R_i; one CTA per graph
__global__ void graph_reduce_kernel(int n_graphs, const int* __restrict__ graph_start, const float* __restrict__ e_atom,
                                    const float* __restrict__ q, const float* __restrict__ R, double* __restrict__ e_graph,
                                    float* __restrict__ dipole) {
  __shared__ double red[4][32];
  const int g = blockIdx.x;
  const int a0 = graph_start[g], a1 = graph_start[g + 1];
  double v[4] = {0.0, 0.0, 0.0, 0.0};
  for (int a = a0 + threadIdx.x; a < a1; a += blockDim.x) {
    v[0] += (double)e_atom[a];
    if (R) {
      float qa = q[a];
      v[1] += (double)(qa * R[3 * (size_t)a]); v[2] += (double)(qa * R[3 * (size_t)a + 1]); v[3] += (double)(qa * R[3 * (size_t)a + 2]);
    }
  }
  for (int k = 0; k < 4; ++k) {
    double s = v[k];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[k][threadIdx.x >> 5] = s;
  }
  __syncthreads();
  if (threadIdx.x < 4) {
    double s = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[threadIdx.x][w];
    if (threadIdx.x == 0) e_graph[g] = s;
    else if (dipole) dipole[3 * g + threadIdx.x - 1] = (float)s;
  }
}

// ---- one structure with many atoms: the same three operations spread over many CTAs (sums in double, fixed order) ----
constexpr int kWideBlocks = 296;      // two CTAs per SM of a 148-SM part; a fixed count keeps the order of the double sums independent of the device
constexpr int kWideMinAtoms = 16384;

__device__ double block_sum_double_256(double v, double* sh) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  double s = 0.0;
  if (threadIdx.x == 0)
    for (int w = 0; w < 8; ++w) s += sh[w];
  __syncthreads();
  return s;       // valid in thread 0
}

// partials[b][0] = sum a ; with R: partials[b][1..3] = sum q R
__global__ void __launch_bounds__(256) wide_partial_kernel(int n, const float* __restrict__ a, const float* __restrict__ q,
                                                           const float* __restrict__ R, double* __restrict__ partials) {
  __shared__ double sh[8];
  double v[4] = {0.0, 0.0, 0.0, 0.0};
  for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256) {
    v[0] += (double)a[i];
    if (R) {
      const float qa = q[i];
      v[1] += (double)(qa * R[3 * (size_t)i]); v[2] += (double)(qa * R[3 * (size_t)i + 1]); v[3] += (double)(qa * R[3 * (size_t)i + 2]);
    }
  }
  for (int k = 0; k < (R ? 4 : 1); ++k) {
    const double s = block_sum_double_256(v[k], sh);
    if (threadIdx.x == 0) partials[4 * blockIdx.x + k] = s;
  }
}

__device__ double wide_total(const double* __restrict__ partials, int n_blocks, int k, double* sh) {
  // every CTA forms the same total from the same partials in the same order
  double v = 0.0;
  for (int b = threadIdx.x; b < n_blocks; b += 256) v += partials[4 * b + k];
  const double s = block_sum_double_256(v, sh);
  __shared__ double total;
  if (threadIdx.x == 0) total = s;
  __syncthreads();
  return total;
}

__global__ void __launch_bounds__(256) charge_conserve_wide_kernel(int n, const float* __restrict__ q_raw, const float* __restrict__ total_charge,
                                                                   const float* __restrict__ hv, float* __restrict__ q, float* __restrict__ h,
                                                                   const double* __restrict__ partials, int n_blocks) {
  __shared__ double sh[8];
  const float Q = total_charge ? total_charge[0] : 0.f;
  // in double: a float32 shift carries a relative error of 6e-8, which times a million atoms is a visible net charge
  const double corr = ((double)Q - wide_total(partials, n_blocks, 0, sh)) / (double)n;
  for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256) {
    q[i] = (float)((double)q_raw[i] + corr);
    h[i] = fabsf(hv[i]);
  }
}

__global__ void __launch_bounds__(256) charge_conserve_bwd_wide_kernel(int n, const float* __restrict__ gq, float* __restrict__ gq_raw,
                                                                       const double* __restrict__ partials, int n_blocks) {
  __shared__ double sh[8];
  const float mean = (float)wide_total(partials, n_blocks, 0, sh) / (float)n;
  for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256) gq_raw[i] = gq[i] - mean;
}

__global__ void __launch_bounds__(256) graph_reduce_wide_kernel(const double* __restrict__ partials, int n_blocks, int with_dipole,
                                                                double* __restrict__ e_graph, float* __restrict__ dipole) {
  __shared__ double sh[8];
  for (int k = 0; k < (with_dipole ? 4 : 1); ++k) {
    const double t = wide_total(partials, n_blocks, k, sh);
    if (threadIdx.x == 0) {
      if (k == 0) e_graph[0] = t;
      else if (dipole) dipole[k - 1] = (float)t;
    }
    __syncthreads();
  }
}

}  // namespace

void launch_sr_geometry_zbl(cudaStream_t s, const ModelDev& M, const Cell& cell, int n, long long n_edges, const int* edge_i,
                            const int* nbr_j, const int* Z, const float* R, int dR_given, float* dR, float* e_atom, float* g_dR, const float* ge,
                            float* F_direct, int n_owned, float* virial) {
  if (n_edges <= 0) return;
  unsigned blocks = (unsigned)((n_edges + 255) / 256);
  { sr_geometry_zbl_kernel<<<blocks, 256, 0, s>>>(M.zbl, cell, n, n_edges, edge_i, nbr_j, Z, R, dR_given, dR, e_atom, g_dR, ge, F_direct, n_owned, virial); count_launch(); }
}

void launch_force_scatter(cudaStream_t s, int n, long long n_edges, const int* edge_i, const int* nbr_j, const float* g_dR, float* F) {
  if (n_edges <= 0) return;
  unsigned blocks = (unsigned)((n_edges + 255) / 256);
  { force_scatter_kernel<<<blocks, 256, 0, s>>>(n, n_edges, edge_i, nbr_j, g_dR, F); count_launch(); }
}

void launch_pair_lr(cudaStream_t s, const LrParams& P, const Cell& cell, int n, const int* row_ptr, const int* nbr_j,
                    const int* Z, const float* R, const float* q, const float* h, int mode, const float* dR_lr,
                    float* g_dR_lr, float* e_atom, float* F, float* gq, float* gh, float* e_coul, float* e_disp, const float* ge,
                    float* virial) {
  if (n <= 0) return;
  int blocks = (n + 7) / 8;
  if (mode == 0)
    { pair_lr_kernel<0><<<blocks, 256, 0, s>>>(P, cell, n, row_ptr, nbr_j, Z, R, q, h, dR_lr, g_dR_lr, e_atom, F, gq, gh, e_coul, e_disp, ge, virial); count_launch(); }
  else
    { pair_lr_kernel<1><<<blocks, 256, 0, s>>>(P, cell, n, row_ptr, nbr_j, Z, R, q, h, dR_lr, g_dR_lr, e_atom, F, gq, gh, e_coul, e_disp, ge, virial); count_launch(); }
}

void launch_pair_lr_packed(cudaStream_t s, const LrParams& P, const Cell& cell, int n, const int* row_ptr, const int* nbr_j, const int* Z,
                           const float* R, const float* q, const float* h, float* pack /* 12 n floats */, float* F, float* gq, float* gh,
                           float* e_coul, float* e_disp, float* virial) {
  if (n <= 0) return;
  float4* pq = reinterpret_cast<float4*>(pack);
  float4* acc = pq + n;
  float4* hz = acc + n;
  pair_pack_kernel<<<(n + 255) / 256, 256, 0, s>>>(n, R, q, h, Z, pq, hz, acc);
  pair_lr_packed_kernel<<<(n + 7) / 8, 256, 0, s>>>(P, cell, n, row_ptr, nbr_j, pq, hz, acc, gh, e_coul, e_disp, virial);
  pair_unpack_kernel<<<(n + 255) / 256, 256, 0, s>>>(n, acc, F, gq);
  count_launch(3);
}

void launch_pair_lr_owned(cudaStream_t s, const LrParams& P, const Cell& cell, int n_owned, int n, const int* row_ptr,
                          const int* nbr_j, const int* Z, const float* R, const float* q, const float* h, float* F_add,
                          float* gq, float* gh, float* e_coul, float* e_disp, float* virial) {
  if (n_owned <= 0) return;
  cudaMemsetAsync(gq, 0, (size_t)n_owned * sizeof(float), s);
  cudaMemsetAsync(gh, 0, (size_t)n_owned * sizeof(float), s);
  { pair_lr_owned_kernel<<<(n_owned + 7) / 8, 256, 0, s>>>(P, cell, n_owned, n, row_ptr, nbr_j, Z, R, q, h, F_add, gq, gh, e_coul, e_disp, virial); count_launch(); }
}

void launch_charge_conserve(cudaStream_t s, int n_graphs, const int* graph_start, const float* q_raw,
                            const float* total_charge, const float* hv, float* q, float* h, int n_atoms, double* scratch) {
  if (n_graphs <= 0) return;
  if (n_graphs == 1 && scratch && n_atoms >= kWideMinAtoms) {
    wide_partial_kernel<<<kWideBlocks, 256, 0, s>>>(n_atoms, q_raw, nullptr, nullptr, scratch);
    charge_conserve_wide_kernel<<<kWideBlocks, 256, 0, s>>>(n_atoms, q_raw, total_charge, hv, q, h, scratch, kWideBlocks);
    count_launch(2);
    return;
  }
  { charge_conserve_kernel<<<n_graphs, 256, 0, s>>>(n_graphs, graph_start, q_raw, total_charge, hv, q, h); count_launch(); }
}
void launch_charge_conserve_bwd(cudaStream_t s, int n_graphs, const int* graph_start, const float* gq, float* gq_raw, int n_atoms,
                                double* scratch) {
  if (n_graphs <= 0) return;
  if (n_graphs == 1 && scratch && n_atoms >= kWideMinAtoms) {
    wide_partial_kernel<<<kWideBlocks, 256, 0, s>>>(n_atoms, gq, nullptr, nullptr, scratch);
    charge_conserve_bwd_wide_kernel<<<kWideBlocks, 256, 0, s>>>(n_atoms, gq, gq_raw, scratch, kWideBlocks);
    count_launch(2);
    return;
  }
  { charge_conserve_bwd_kernel<<<n_graphs, 256, 0, s>>>(n_graphs, graph_start, gq, gq_raw); count_launch(); }
}
void launch_graph_reduce(cudaStream_t s, int n_graphs, const int* graph_start, const float* e_atom, const float* q,
                         const float* R, double* e_graph, float* dipole, int n_atoms, double* scratch) {
  if (n_graphs <= 0) return;
  if (n_graphs == 1 && scratch && n_atoms >= kWideMinAtoms) {
    wide_partial_kernel<<<kWideBlocks, 256, 0, s>>>(n_atoms, e_atom, q, R, scratch);
    graph_reduce_wide_kernel<<<1, 256, 0, s>>>(scratch, kWideBlocks, R ? 1 : 0, e_graph, dipole);
    count_launch(2);
    return;
  }
  { graph_reduce_kernel<<<n_graphs, 256, 0, s>>>(n_graphs, graph_start, e_atom, q, R, e_graph, dipole); count_launch(); }
}

}  // namespace so3lr

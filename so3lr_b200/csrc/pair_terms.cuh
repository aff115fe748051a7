// Analytic pair terms of SO3LR with first derivatives: ZBL repulsion (short-range edges), erf-damped Coulomb and
// QDO-damped dispersion (long-range pairs).  All functions are host+device so the host tests can call them.
#pragma once
#include "common.cuh"

namespace so3lr {

// ---------------- forward-mode dual number with three partials (r, h_i, h_j) ----------------
struct Dual3 {
  float v, d0, d1, d2;
};
SO3LR_HD Dual3 mk(float v, float d0 = 0.f, float d1 = 0.f, float d2 = 0.f) { return Dual3{v, d0, d1, d2}; }
SO3LR_HD Dual3 operator+(Dual3 a, Dual3 b) { return mk(a.v + b.v, a.d0 + b.d0, a.d1 + b.d1, a.d2 + b.d2); }
SO3LR_HD Dual3 operator-(Dual3 a, Dual3 b) { return mk(a.v - b.v, a.d0 - b.d0, a.d1 - b.d1, a.d2 - b.d2); }
SO3LR_HD Dual3 operator*(Dual3 a, Dual3 b) {
  return mk(a.v * b.v, a.d0 * b.v + a.v * b.d0, a.d1 * b.v + a.v * b.d1, a.d2 * b.v + a.v * b.d2);
}
SO3LR_HD Dual3 operator*(float s, Dual3 a) { return mk(s * a.v, s * a.d0, s * a.d1, s * a.d2); }
SO3LR_HD Dual3 operator+(Dual3 a, float s) { return mk(a.v + s, a.d0, a.d1, a.d2); }
SO3LR_HD Dual3 operator/(Dual3 a, Dual3 b) {
  float inv = 1.f / b.v;
  float q = a.v * inv;
  return mk(q, (a.d0 - q * b.d0) * inv, (a.d1 - q * b.d1) * inv, (a.d2 - q * b.d2) * inv);
}
SO3LR_HD Dual3 dpow(Dual3 a, float p) {
  float v = powf(a.v, p);
  float g = p * v / a.v;
  return mk(v, g * a.d0, g * a.d1, g * a.d2);
}
SO3LR_HD Dual3 dpowi(Dual3 a, int n) {  // integer power by repeated multiplication
  Dual3 r = a;
  for (int k = 1; k < n; ++k) r = r * a;
  return r;
}

// Free-atom reference data (atomic units) for Z = 1..18: static polarisability and C6.  Contexts reject any other element at
// creation (so3lr_b200_system_create, so3lr_b200_dd_set_atoms), so the fall-through value is never used in an evaluation.
constexpr int kMaxZ = 18;
SO3LR_HD float alpha_free(int Z) {
  const float t[18] = {4.5f, 1.38f, 164.2f, 38.0f, 21.0f, 12.0f, 7.4f, 5.4f, 3.8f, 2.67f, 162.7f, 71.0f, 60.0f, 37.0f, 25.0f, 19.6f, 15.0f, 11.1f};
  return (Z >= 1 && Z <= 18) ? t[Z - 1] : 1.0f;
}
SO3LR_HD float c6_free(int Z) {
  const float t[18] = {6.5f, 1.46f, 1387.0f, 214.0f, 99.5f, 46.6f, 24.2f, 15.6f, 9.52f, 6.38f, 1556.0f, 627.0f, 528.0f, 305.0f, 185.0f, 134.0f, 94.6f, 64.3f};
  return (Z >= 1 && Z <= 18) ? t[Z - 1] : 1.0f;
}

struct LrParams {
  int has_cutoff;       // 0: plain erf-Coulomb and un-switched dispersion
  float rc;             // long-range cutoff
  float cuton;          // 0.45 * rc
  float v_rc, dv_rc;    // erf(rc/sigma)/rc and its derivative at rc
  int has_damping;      // dispersion switched off between rc - damping and rc
  float disp_on;        // rc - damping
  float pair_factor;    // 1 for ordered lists, 0.5 for lists holding both directions
  float k_alpha;        // 1 / (sqrt(2) s) when the reciprocal-space sum holds erf(r / (sqrt(2) s)) / r of every pair; 0: off
};

// erf-damped Coulomb kernel chi(r) (energy = ke q_i q_j chi) and d chi / d r
SO3LR_HD void coulomb_chi(const LrParams& p, float r, float& chi, float& dchi) {
  const float inv_sig = 1.f / kSigmaCoulomb;
  float x = r * inv_sig;
  float er = erff(x);
  float pot = er / r;
  float dpot = (1.1283791670955126f * inv_sig * expf(-x * x) - pot) / r;
  if (p.k_alpha > 0.f) {
    const float y = r * p.k_alpha;
    const float potk = erff(y) / r;
    pot -= potk;
    dpot -= (1.1283791670955126f * p.k_alpha * expf(-y * y) - potk) / r;
  }
  if (!p.has_cutoff) { chi = pot; dchi = dpot; return; }
  if (r >= p.rc) { chi = 0.f; dchi = 0.f; return; }
  float f, df;
  switching(r, p.cuton, p.rc, f, df);
  chi = (pot - p.v_rc) - (1.f - f) * (r - p.rc) * p.dv_rc;
  dchi = dpot - (1.f - f) * p.dv_rc + df * (r - p.rc) * p.dv_rc;
}

// Dispersion energy (eV) of one pair and its derivatives w.r.t. r (Angstrom), h_i and h_j.
SO3LR_HD void dispersion_pair(const LrParams& p, float r, int Zi, int Zj, float hi, float hj, float& e, float& de_dr,
                              float& de_dhi, float& de_dhj) {
  if (p.has_cutoff && r >= p.rc) { e = de_dr = de_dhi = de_dhj = 0.f; return; }
  Dual3 Hi = mk(hi, 0.f, 1.f, 0.f), Hj = mk(hj, 0.f, 0.f, 1.f);
  Dual3 ai = alpha_free(Zi) * Hi, aj = alpha_free(Zj) * Hj;
  Dual3 ci = c6_free(Zi) * (Hi * Hi), cj = c6_free(Zj) * (Hj * Hj);
  Dual3 aij = 0.5f * (ai + aj);
  Dual3 c6 = (2.f * (ci * cj * aj * ai)) / (ai * ai * cj + aj * aj * ci);
  Dual3 a17 = dpow(aij, 1.f / 7.f);
  const float fs = 2.5527961000248887f;   // fine_structure^(-4/21)
  Dual3 rv = fs * a17;
  Dual3 sg = ((-0.00078893f * rv + 0.04125273f) * rv + 0.24428889f) * rv + (-0.00433008f);
  Dual3 inv_gam = 2.f * (sg * sg);          // 1/gamma
  Dual3 c8 = 5.f * (inv_gam * c6);
  Dual3 c10 = 30.625f * (inv_gam * inv_gam * c6);
  Dual3 pp = (kDispersionScale * 2.f * 2.54f) * a17;
  Dual3 R = mk(r / kBohr, 1.f / kBohr, 0.f, 0.f);
  Dual3 R2 = R * R, p2 = pp * pp;
  Dual3 R6 = R2 * R2 * R2, p6 = p2 * p2 * p2;
  Dual3 R8 = R6 * R2, p8 = p6 * p2;
  Dual3 R10 = R8 * R2, p10 = p8 * p2;
  Dual3 E = c6 / (R6 + p6) + c8 / (R8 + p8) + c10 / (R10 + p10);
  E = (-kHartree) * E;
  if (p.has_cutoff && p.has_damping) {
    float f, df;
    switching(r, p.disp_on, p.rc, f, df);
    E = E * mk(f, df, 0.f, 0.f);
  }
  e = E.v; de_dr = E.d0; de_dhi = E.d1; de_dhj = E.d2;
}

// The same dispersion energy and derivatives with hand-derived partials instead of forward-mode dual numbers (about a
// quarter of the arithmetic; used by the long-range pair kernels, checked against dispersion_pair on the host).
//   E = -Hartree * c6 * T * f(r),  T = 1/(R^6+p^6) + 5 ig/(R^8+p^8) + 30.625 ig^2/(R^10+p^10),  R = r / Bohr,
//   p = 6.096 a17, ig = 2 sg^2, sg = cubic(fs * a17), a17 = ((a_i + a_j)/2)^(1/7), a = alpha_free * h, c = c6_free * h^2,
//   c6 = 2 c_i c_j a_i a_j / (a_i^2 c_j + a_j^2 c_i)
SO3LR_HD void dispersion_pair_fast(const LrParams& P, float r, int Zi, int Zj, float hi, float hj, float& e, float& de_dr,
                                   float& de_dhi, float& de_dhj) {
  if (P.has_cutoff && r >= P.rc) { e = de_dr = de_dhi = de_dhj = 0.f; return; }
  const float alf_i = alpha_free(Zi), alf_j = alpha_free(Zj), c6f_i = c6_free(Zi), c6f_j = c6_free(Zj);
  const float ai = alf_i * hi, aj = alf_j * hj, ci = c6f_i * hi * hi, cj = c6f_j * hj * hj;
  const float den = ai * ai * cj + aj * aj * ci, iden = 1.f / den;
  const float c6 = 2.f * ci * cj * ai * aj * iden;
  // d ln c6 / d h = (d ln c6/d a) alpha + (d ln c6/d c) 2 c6free h
  const float dlc6_dhi = (1.f / ai - 2.f * ai * cj * iden) * alf_i + (1.f / ci - aj * aj * iden) * 2.f * c6f_i * hi;
  const float dlc6_dhj = (1.f / aj - 2.f * aj * ci * iden) * alf_j + (1.f / cj - ai * ai * iden) * 2.f * c6f_j * hj;
  const float aij = 0.5f * (ai + aj);
#ifdef __CUDA_ARCH__
  const float a17 = exp2f(log2f(aij) * (1.f / 7.f));
#else
  const float a17 = powf(aij, 1.f / 7.f);
#endif
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
  const float i6 = 1.f / (R6 + p6), i8 = 1.f / (R8 + p8), i10 = 1.f / (R10 + p10);
  const float t8 = 5.f * ig, t10 = 30.625f * ig * ig;
  const float T = i6 + t8 * i8 + t10 * i10;
  // partials of T
  const float dT_dR = -(6.f * R4 * R * i6 * i6 + t8 * 8.f * R6 * R * i8 * i8 + t10 * 10.f * R8 * R * i10 * i10);
  const float dT_dp = -(6.f * p4 * p * i6 * i6 + t8 * 8.f * p6 * p * i8 * i8 + t10 * 10.f * p8 * p * i10 * i10);
  const float dT_dig = 5.f * i8 + 61.25f * ig * i10;
  // a17 enters through p (= kp a17) and through sg(rv = fs a17)
  const float dT_da17 = dT_dp * kp + dT_dig * 4.f * sg * dsg * fs;
  const float da17_dh = a17 / (7.f * aij) * 0.5f;          // times alpha_free of the atom
  float f = 1.f, df = 0.f;
  if (P.has_cutoff && P.has_damping) switching(r, P.disp_on, P.rc, f, df);
  const float pre = -kHartree * c6;
  e = pre * T * f;
  de_dr = pre * (dT_dR * (1.f / kBohr) * f + T * df);
  de_dhi = pre * f * (T * dlc6_dhi + dT_da17 * da17_dh * alf_i);
  de_dhj = pre * f * (T * dlc6_dhj + dT_da17 * da17_dh * alf_j);
}

struct ZblParams {
  float a[4], c[4];  // softplus-positive screening exponents and normalised weights
  float p, d;        // exponent of Z and inverse screening length scale
};

// ZBL repulsion of one directed short-range edge (half of the pair energy) and d/dr.
SO3LR_HD void zbl_edge(const ZblParams& z, float r, float cut, float dcut, int Zi, int Zj, float& e, float& de) {
  if (r >= kZblSwitchOff) { e = 0.f; de = 0.f; return; }
  float zi = (float)Zi, zj = (float)Zj;
  float s = (powf(zi, z.p) + powf(zj, z.p)) * z.d;
  float phi = 0.f, dphi = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float t = z.c[k] * expf(-z.a[k] * s * r);
    phi += t;
    dphi -= z.a[k] * s * t;
  }
  float w, dw;
  switching(r, 0.f, kZblSwitchOff, w, dw);
  float pre = 0.5f * kKe * zi * zj;
  float inv = 1.f / r;
  // e = pre * cut * phi * w / r
  e = pre * cut * phi * w * inv;
  de = pre * inv * (dcut * phi * w + cut * dphi * w + cut * phi * dw - cut * phi * w * inv);
}

}  // namespace so3lr

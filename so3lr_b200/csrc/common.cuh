// Shared device/host helpers for the SO3LR sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cmath>

#include "params.h"

#define SO3LR_HD __host__ __device__ __forceinline__
#define SO3LR_D __device__ __forceinline__

namespace so3lr {

// ---- status codes (also in include/so3lr_b200.h) ----
enum Status : int {
  kOk = 0,
  kInvalidArgument = 1,
  kCudaError = 2,
  kOverflow = 3,
  kNotFinite = 4,
  kTooLarge = 5,
};

#define SO3LR_CUDA_CHECK(expr)                                                        \
  do {                                                                                \
    cudaError_t _e = (expr);                                                          \
    if (_e != cudaSuccess) {                                                          \
      std::fprintf(stderr, "so3lr_b200: CUDA error %s at %s:%d: %s\n", #expr, __FILE__, __LINE__, \
                   cudaGetErrorString(_e));                                           \
      return kCudaError;                                                              \
    }                                                                                 \
  } while (0)

// Every kernel launch of the library is followed by count_launch(): the evaluation context whose entry point is running
// on this host thread keeps the total (so3lr_b200_system_stats).
void count_launch(int kernels = 1);

// multiprocessors of the current device (queried once per device ordinal); persistent kernels launch one CTA per SM
int sm_count();

constexpr float kCutoffSr = 4.5f;
constexpr float kAvgNumNeighbors = 13.168995780096482f;
constexpr float kLnEps = 1e-6f;
constexpr float kKe = 14.399645351950548f;
constexpr float kSigmaCoulomb = 4.0f;
constexpr float kCutonFraction = 0.45f;
constexpr float kDispersionScale = 1.2f;
constexpr float kBohr = 0.5291772105638411f;
constexpr float kHartree = 27.211386024367243f;
constexpr float kZblSwitchOff = 1.5f;
constexpr int kTableGrid = 1024;                 // radial-filter table points on [0, 4.5]
constexpr float kTableH = kCutoffSr / (kTableGrid - 1);

// Radial filters of the tiled attention kernels: 64 Chebyshev polynomials of t = kChebA * x + kChebB, x = exp(-kChebHalfGamma r),
// which maps r in [0, 4.5] onto t in [1, -1].  In this variable the filters are smooth enough that 64 terms reproduce them to
// 2e-8 and their r-derivative to 4e-6 of their largest value.
constexpr int kChebM = 64;
constexpr double kChebHalfGammaD = 0.5 * 0.9448630809783936;       // half the Bernstein decay constant (a float32 number)
constexpr double kChebX0D = 0.11932052347400147;                    // exp(-kChebHalfGammaD * 4.5)
constexpr float kChebHalfGamma = (float)kChebHalfGammaD;
constexpr float kChebA = (float)(2.0 / (1.0 - kChebX0D));
constexpr float kChebB = (float)(-(1.0 + kChebX0D) / (1.0 - kChebX0D));
constexpr int kTcImageBytes = 2 * 32768 + 4 * 8192;                 // C hi | C lo | K2 hi [2] | K2 lo [2]

SO3LR_HD int degree_of(int m) { return m < 3 ? 0 : (m < 8 ? 1 : (m < 15 ? 2 : 3)); }

SO3LR_D float silu_f(float x) { return x / (1.f + __expf(-x)); }
// d silu / dx
SO3LR_D float dsilu_f(float x) {
  float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

SO3LR_D float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Strain derivative of the energy ("virial"), dE/d eps_ab = sum over directed edges of dR_a * dE/d(dR)_b.  The gather
// kernels give every atom i the force f it receives through each of its edges (both directions of the pair), and then
// dE/d eps = 1/2 sum_i sum_j dR_ij (x) f_ij.  The sum is symmetric, so six symmetrised components are kept per atom, in
// the order xx yy zz yz xz xy.  `w` is the weight of dR (x) f for the calling kernel (1/2 in the gather kernels).
struct VirialAcc {
  float xx = 0.f, yy = 0.f, zz = 0.f, yz = 0.f, xz = 0.f, xy = 0.f;
  SO3LR_D void add(float w, float dx, float dy, float dz, float fx, float fy, float fz) {
    const float wx = w * dx, wy = w * dy, wz = w * dz;
    xx = fmaf(wx, fx, xx); yy = fmaf(wy, fy, yy); zz = fmaf(wz, fz, zz);
    yz = fmaf(0.5f * wy, fz, fmaf(0.5f * wz, fy, yz));
    xz = fmaf(0.5f * wx, fz, fmaf(0.5f * wz, fx, xz));
    xy = fmaf(0.5f * wx, fy, fmaf(0.5f * wy, fx, xy));
  }
  // all lanes of the warp that owns atom i call this; lane 0 adds the warp's total to the atom's row
  SO3LR_D void flush_warp(float* __restrict__ W, size_t i, int lane) {
    const float a = warp_sum(xx), b = warp_sum(yy), c = warp_sum(zz), d = warp_sum(yz), e = warp_sum(xz), f = warp_sum(xy);
    if (lane == 0) {
      float* w = W + 6 * i;
      w[0] += a; w[1] += b; w[2] += c; w[3] += d; w[4] += e; w[5] += f;
    }
  }
};

// sum inside aligned groups of 8 lanes
SO3LR_D float group8_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

// PhysNet cutoff 1 - 6u^5 + 15u^4 - 10u^3 and its r-derivative (u = r / rc)
SO3LR_HD void phys_cutoff(float r, float& c, float& dc) {
  const float inv = 1.f / kCutoffSr;
  float u = r * inv;
  float u2 = u * u, u3 = u2 * u;
  c = 1.f + u3 * (-10.f + u * (15.f - 6.f * u));
  dc = u2 * (-30.f + u * (60.f - 30.f * u)) * inv;
}

// smooth switch: 1 for x<=on, 0 for x>=off.  returns value and d/dx
SO3LR_HD void switching(float x, float on, float off, float& f, float& df) {
  float w = off - on;
  float c = (x - on) / w;
  if (c <= 0.f) { f = 1.f; df = 0.f; return; }
  if (c >= 1.f) { f = 0.f; df = 0.f; return; }
  // s(a) = exp(-1/a)
  float a = 1.f - c, b = c;
  float sa = expf(-1.f / a), sb = expf(-1.f / b);
  float den = sa + sb;
  f = sa / den;
  // dsa/dc = -sa/a^2 ; dsb/dc = sb/b^2
  float dsa = -sa / (a * a), dsb = sb / (b * b);
  df = (dsa * den - sa * (dsa + dsb)) / (den * den) / w;
}

// Orthonormal real spherical harmonics l=1..4 (24 values) of a unit vector, and the gradient of
// sum_m g[m] * Y[m] with respect to the (unconstrained) unit-vector components.
SO3LR_HD void sph_harm_24(float x, float y, float z, float* Y) {
  const float c1 = 0.4886025119029199f;
  Y[0] = c1 * y; Y[1] = c1 * z; Y[2] = c1 * x;
  const float a2 = 1.0925484305920792f, b2 = 0.31539156525252005f, d2 = 0.5462742152960396f;
  Y[3] = a2 * x * y; Y[4] = a2 * y * z; Y[5] = b2 * (3.f * z * z - 1.f); Y[6] = a2 * x * z; Y[7] = d2 * (x * x - y * y);
  const float a3 = 0.5900435899266435f, b3 = 2.890611442640554f, c3 = 0.4570457994644658f, d3 = 0.3731763325901154f,
              e3 = 1.445305721320277f;
  Y[8] = a3 * y * (3.f * x * x - y * y); Y[9] = b3 * x * y * z; Y[10] = c3 * y * (5.f * z * z - 1.f);
  Y[11] = d3 * (5.f * z * z * z - 3.f * z); Y[12] = c3 * x * (5.f * z * z - 1.f); Y[13] = e3 * (x * x - y * y) * z;
  Y[14] = a3 * x * (x * x - 3.f * y * y);
  const float a4 = 2.5033429417967046f, b4 = 1.7701307697799304f, c4 = 0.9461746957575601f, d4 = 0.6690465435572892f,
              e4 = 0.10578554691520431f, f4 = 0.47308734787878004f, g4 = 0.6258357354491761f;
  Y[15] = a4 * x * y * (x * x - y * y); Y[16] = b4 * y * z * (3.f * x * x - y * y);
  Y[17] = c4 * x * y * (7.f * z * z - 1.f); Y[18] = d4 * y * z * (7.f * z * z - 3.f);
  Y[19] = e4 * (35.f * z * z * z * z - 30.f * z * z + 3.f); Y[20] = d4 * x * z * (7.f * z * z - 3.f);
  Y[21] = f4 * (x * x - y * y) * (7.f * z * z - 1.f); Y[22] = b4 * x * z * (x * x - 3.f * y * y);
  Y[23] = g4 * (x * x * (x * x - 3.f * y * y) - y * y * (3.f * x * x - y * y));
}

SO3LR_HD void sph_harm_24_vjp(float x, float y, float z, const float* g, float& gx, float& gy, float& gz) {
  const float c1 = 0.4886025119029199f;
  gx = c1 * g[2]; gy = c1 * g[0]; gz = c1 * g[1];
  const float a2 = 1.0925484305920792f, b2 = 0.31539156525252005f, d2 = 0.5462742152960396f;
  gx += a2 * y * g[3] + a2 * z * g[6] + 2.f * d2 * x * g[7];
  gy += a2 * x * g[3] + a2 * z * g[4] - 2.f * d2 * y * g[7];
  gz += a2 * y * g[4] + 6.f * b2 * z * g[5] + a2 * x * g[6];
  const float a3 = 0.5900435899266435f, b3 = 2.890611442640554f, c3 = 0.4570457994644658f, d3 = 0.3731763325901154f,
              e3 = 1.445305721320277f;
  float x2 = x * x, y2 = y * y, z2 = z * z;
  gx += a3 * 6.f * x * y * g[8] + b3 * y * z * g[9] + c3 * (5.f * z2 - 1.f) * g[12] + e3 * 2.f * x * z * g[13] +
        a3 * (3.f * x2 - 3.f * y2) * g[14];
  gy += a3 * (3.f * x2 - 3.f * y2) * g[8] + b3 * x * z * g[9] + c3 * (5.f * z2 - 1.f) * g[10] - e3 * 2.f * y * z * g[13] -
        a3 * 6.f * x * y * g[14];
  gz += b3 * x * y * g[9] + c3 * 10.f * y * z * g[10] + d3 * (15.f * z2 - 3.f) * g[11] + c3 * 10.f * x * z * g[12] +
        e3 * (x2 - y2) * g[13];
  const float a4 = 2.5033429417967046f, b4 = 1.7701307697799304f, c4 = 0.9461746957575601f, d4 = 0.6690465435572892f,
              e4 = 0.10578554691520431f, f4 = 0.47308734787878004f, g4 = 0.6258357354491761f;
  // Y15 = a4 (x^3 y - x y^3)
  gx += a4 * (3.f * x2 * y - y2 * y) * g[15]; gy += a4 * (x2 * x - 3.f * x * y2) * g[15];
  // Y16 = b4 (3 x^2 y z - y^3 z)
  gx += b4 * 6.f * x * y * z * g[16]; gy += b4 * (3.f * x2 - 3.f * y2) * z * g[16]; gz += b4 * (3.f * x2 * y - y2 * y) * g[16];
  // Y17 = c4 x y (7 z^2 - 1)
  gx += c4 * y * (7.f * z2 - 1.f) * g[17]; gy += c4 * x * (7.f * z2 - 1.f) * g[17]; gz += c4 * 14.f * x * y * z * g[17];
  // Y18 = d4 y (7 z^3 - 3 z)
  gy += d4 * (7.f * z2 * z - 3.f * z) * g[18]; gz += d4 * y * (21.f * z2 - 3.f) * g[18];
  // Y19 = e4 (35 z^4 - 30 z^2 + 3)
  gz += e4 * (140.f * z2 * z - 60.f * z) * g[19];
  // Y20 = d4 x (7 z^3 - 3 z)
  gx += d4 * (7.f * z2 * z - 3.f * z) * g[20]; gz += d4 * x * (21.f * z2 - 3.f) * g[20];
  // Y21 = f4 (x^2 - y^2)(7 z^2 - 1)
  gx += f4 * 2.f * x * (7.f * z2 - 1.f) * g[21]; gy -= f4 * 2.f * y * (7.f * z2 - 1.f) * g[21];
  gz += f4 * (x2 - y2) * 14.f * z * g[21];
  // Y22 = b4 z (x^3 - 3 x y^2)
  gx += b4 * z * (3.f * x2 - 3.f * y2) * g[22]; gy -= b4 * z * 6.f * x * y * g[22]; gz += b4 * (x2 * x - 3.f * x * y2) * g[22];
  // Y23 = g4 (x^4 - 6 x^2 y^2 + y^4)
  gx += g4 * (4.f * x2 * x - 12.f * x * y2) * g[23]; gy += g4 * (4.f * y2 * y - 12.f * x2 * y) * g[23];
}

struct Cell {
  float h[9];     // rows = lattice vectors
  float hinv[9];  // inverse, so that s = dR @ hinv
  int periodic;   // 0: free space
};

// minimum-image displacement: dR - round(dR h^-1) h, the operation order of oracle.min_image.  The lattice translation is
// subtracted from dR directly (it is not rebuilt from the fractional remainder), so the result keeps the full float32
// precision of dR however many cells the two positions are apart; for an orthorhombic cell the subtraction is exact up to
// one rounding.
SO3LR_HD void min_image(const Cell& c, float& dx, float& dy, float& dz) {
  if (!c.periodic) return;
#ifdef __CUDA_ARCH__
  const float k0 = rintf(__fadd_rn(__fadd_rn(__fmul_rn(dx, c.hinv[0]), __fmul_rn(dy, c.hinv[3])), __fmul_rn(dz, c.hinv[6])));
  const float k1 = rintf(__fadd_rn(__fadd_rn(__fmul_rn(dx, c.hinv[1]), __fmul_rn(dy, c.hinv[4])), __fmul_rn(dz, c.hinv[7])));
  const float k2 = rintf(__fadd_rn(__fadd_rn(__fmul_rn(dx, c.hinv[2]), __fmul_rn(dy, c.hinv[5])), __fmul_rn(dz, c.hinv[8])));
  dx = __fsub_rn(dx, __fadd_rn(__fadd_rn(__fmul_rn(k0, c.h[0]), __fmul_rn(k1, c.h[3])), __fmul_rn(k2, c.h[6])));
  dy = __fsub_rn(dy, __fadd_rn(__fadd_rn(__fmul_rn(k0, c.h[1]), __fmul_rn(k1, c.h[4])), __fmul_rn(k2, c.h[7])));
  dz = __fsub_rn(dz, __fadd_rn(__fadd_rn(__fmul_rn(k0, c.h[2]), __fmul_rn(k1, c.h[5])), __fmul_rn(k2, c.h[8])));
#else
  const float k0 = rintf((dx * c.hinv[0] + dy * c.hinv[3]) + dz * c.hinv[6]);
  const float k1 = rintf((dx * c.hinv[1] + dy * c.hinv[4]) + dz * c.hinv[7]);
  const float k2 = rintf((dx * c.hinv[2] + dy * c.hinv[5]) + dz * c.hinv[8]);
  dx = dx - ((k0 * c.h[0] + k1 * c.h[3]) + k2 * c.h[6]);
  dy = dy - ((k0 * c.h[1] + k1 * c.h[4]) + k2 * c.h[7]);
  dz = dz - ((k0 * c.h[2] + k1 * c.h[5]) + k2 * c.h[8]);
#endif
}

SO3LR_D float dist2_rn(float dx, float dy, float dz) {
  return __fadd_rn(__fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy)), __fmul_rn(dz, dz));
}

}  // namespace so3lr

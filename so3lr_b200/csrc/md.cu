// MD step bodies that sit either side of the force evaluation: velocity Verlet halves and the Nose-Hoover chain
// thermostat (Martyna-Tuckerman-Klein propagation with a Suzuki-Yoshida factorisation), in the form
// jax_md.simulate.nvt_nose_hoover applies them (called from so3lr/cli/so3lr_md.py:1047-1075 with the chain settings of
// so3lr/cli/so3lr_md.py:1698-1707).  All state stays on the device between steps; the chain itself is a dozen doubles
// advanced by one thread, so a step costs no host round trip.
//
// Units: Angstrom, fs, amu, eV.
#include "md.h"

#include <cuda_runtime.h>

#include "common.cuh"

namespace so3lr {
namespace {
constexpr double kAccelD = 9.648533212331e-3;    // (eV/A)/amu -> A/fs^2
constexpr float kAccel = 9.648533212331e-3f;

__device__ const double kSyWeights[4][7] = {
    {1.0, 0, 0, 0, 0, 0, 0},
    {0.828981543588751, -0.657963087177502, 0.828981543588751, 0, 0, 0, 0},
    {0.2967324292201065, 0.2967324292201065, -0.186929716880426, 0.2967324292201065, 0.2967324292201065, 0, 0},
    {0.784513610477560, 0.235573213359357, -1.17767998417887, 1.31518632068391, -1.17767998417887, 0.235573213359357,
     0.784513610477560}};

__device__ double block_sum_256(double v, double* sh) {
  // fixed-order tree: the same partial sums in the same order on every launch
  const int t = threadIdx.x;
  sh[t] = v;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (t < s) sh[t] += sh[t + s];
    __syncthreads();
  }
  double r = sh[0];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(256) ke_partial_kernel(int n, const float* __restrict__ m, const float* __restrict__ V,
                                                         double* __restrict__ partials) {
  __shared__ double sh[256];
  int i = blockIdx.x * 256 + threadIdx.x;
  double k = 0.0;
  if (i < n) {
    double vx = V[3 * (size_t)i], vy = V[3 * (size_t)i + 1], vz = V[3 * (size_t)i + 2];
    k = 0.5 * (double)m[i] * (vx * vx + vy * vy + vz * vz) / kAccelD;
  }
  double s = block_sum_256(k, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

// first half of velocity Verlet, after the thermostat's momentum scaling that is waiting in chain[1]
__global__ void __launch_bounds__(256) vv_first_scaled_kernel(int n, float dt, const float* __restrict__ m, float* __restrict__ R,
                                                              float* __restrict__ V, const float* __restrict__ F,
                                                              const double* __restrict__ chain) {
  int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const float scale = chain ? (float)chain[1] : 1.0f;
  float s = 0.5f * dt * kAccel / m[i];
  for (int k = 0; k < 3; ++k) {
    float v = V[3 * (size_t)i + k] * scale + s * F[3 * (size_t)i + k];
    V[3 * (size_t)i + k] = v;
    R[3 * (size_t)i + k] += dt * v;
  }
}

// second half of velocity Verlet; also leaves each block's share of the new kinetic energy (eV)
__global__ void __launch_bounds__(256) vv_second_ke_kernel(int n, float dt, const float* __restrict__ m, float* __restrict__ V,
                                                           const float* __restrict__ F, double* __restrict__ partials) {
  __shared__ double sh[256];
  int i = blockIdx.x * 256 + threadIdx.x;
  double ke = 0.0;
  if (i < n) {
    float mi = m[i];
    float s = 0.5f * dt * kAccel / mi;
    double v2 = 0.0;
    for (int k = 0; k < 3; ++k) {
      float v = V[3 * (size_t)i + k] + s * F[3 * (size_t)i + k];
      V[3 * (size_t)i + k] = v;
      v2 += (double)v * (double)v;
    }
    ke = 0.5 * (double)mi * v2 / kAccelD;
  }
  double sum = block_sum_256(ke, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = sum;
}

__global__ void __launch_bounds__(256) scale_velocities_kernel(size_t n3, float* __restrict__ V, const double* __restrict__ chain) {
  size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i < n3) V[i] *= (float)chain[1];
}

__global__ void nhc_reset_scale_kernel(double* chain) { chain[1] = 1.0; }

__global__ void nhc_init_kernel(double* chain) {
  int t = threadIdx.x;
  if (t < kNhcStateDoubles) chain[t] = t == 1 ? 1.0 : 0.0;
}

// One factor of the chain propagator over `delta`; returns the momentum scale.  xi, p: chain positions and momenta.
__device__ double nhc_substep(int L, double* xi, double* p, const double* Q, double& ke, double delta, double kT, double dof) {
  const int M = L - 1;
  const double d2 = 0.5 * delta, d4 = 0.25 * delta, d8 = 0.125 * delta;
  if (L == 1) {
    p[0] += d4 * (2.0 * ke - dof * kT);
  } else {
    p[M] += d4 * (p[M - 1] * p[M - 1] / Q[M - 1] - kT);
    for (int m = M - 1; m > 0; --m) {
      double G = p[m - 1] * p[m - 1] / Q[m - 1] - kT;
      double s = exp(-d8 * p[m + 1] / Q[m + 1]);
      p[m] = s * (s * p[m] + d4 * G);
    }
    double s = exp(-d8 * p[1] / Q[1]);
    p[0] = s * (s * p[0] + d4 * (2.0 * ke - dof * kT));
  }
  const double scale = exp(-d2 * p[0] / Q[0]);
  ke *= scale * scale;
  for (int m = 0; m < L; ++m) xi[m] += d2 * p[m] / Q[m];
  double G = 2.0 * ke - dof * kT;
  if (L == 1) {
    p[0] += d4 * G;
  } else {
    for (int m = 0; m < M; ++m) {
      double s = exp(-d8 * p[m + 1] / Q[m + 1]);
      p[m] = s * (s * p[m] + d4 * G);
      G = p[m] * p[m] / Q[m] - kT;
    }
    p[M] += d4 * G;
  }
  return scale;
}

// Advances the chain stored at `chain` by n_half half steps (one thread); returns the product of the momentum scales.
// chain[0] (kinetic energy) follows the scaling; chain[1] is left to the caller.
__device__ double nhc_advance(double* chain, int L, int chain_steps, int sy_steps, double dt, double tau, double kT, double dof,
                              int n_half) {
  double xi[kNhcMaxChain], p[kNhcMaxChain], Q[kNhcMaxChain];
  for (int m = 0; m < L; ++m) {
    xi[m] = chain[2 + m];
    p[m] = chain[2 + kNhcMaxChain + m];
    Q[m] = kT * tau * tau * (m == 0 ? dof : 1.0);
  }
  double ke = chain[0], total = 1.0;
  const double* w = kSyWeights[sy_steps / 2];
  const double delta = dt / chain_steps;
  for (int h = 0; h < n_half; ++h)
    for (int i = 0; i < chain_steps * sy_steps; ++i) total *= nhc_substep(L, xi, p, Q, ke, delta * w[i % sy_steps], kT, dof);
  for (int m = 0; m < L; ++m) {
    chain[2 + m] = xi[m];
    chain[2 + kNhcMaxChain + m] = p[m];
  }
  chain[0] = ke;
  return total;
}

__device__ double sum_partials_256(const double* __restrict__ partials, int n_partials, double* sh) {
  double s = 0.0;
  for (int i = threadIdx.x; i < n_partials; i += 256) s += partials[i];
  return block_sum_256(s, sh);
}

// Sums the kinetic-energy partials (when given) into chain[0], then advances the chain by n_half half steps.  The
// momentum scale of those half steps is multiplied into chain[1] for the next velocity kernel to apply.
__global__ void __launch_bounds__(256) nhc_half_steps_kernel(double* chain, int L, int chain_steps, int sy_steps, double dt, double tau,
                                                             double kT, double dof, int n_half, int fresh_scale,
                                                             const double* __restrict__ partials, int n_partials) {
  __shared__ double sh[256];
  if (partials) {
    const double s = sum_partials_256(partials, n_partials, sh);
    if (threadIdx.x == 0) chain[0] = s;
  }
  if (threadIdx.x != 0) return;
  const double total = nhc_advance(chain, L, chain_steps, sy_steps, dt, tau, kT, dof, n_half);
  chain[1] = fresh_scale ? total : chain[1] * total;
}

// ---- NPT (isotropic Martyna-Tobias-Klein barostat; both chains and the box coordinate live in `state`) ----
// state: [0, 18) thermostat chain | [18, 36) barostat chain | box: [36] eps = ln(V/V0)/3, [37] p_eps, [38] c1, [39] c2,
// [40] r1, [41] r2 (the coefficients of the current step's velocity and position updates), [42] volume, [43] spare
struct NptSettings {
  int L, chain_steps, sy_steps, n_atoms;
  double dt, kT, pressure, tau_t, tau_b, V0;
};

__device__ double sinhx_x(double x) {
  const double x2 = x * x;
  return 1.0 + x2 / 6.0 + x2 * x2 / 120.0 + x2 * x2 * x2 / 5040.0 + x2 * x2 * x2 * x2 / 362880.0 + x2 * x2 * x2 * x2 * x2 / 39916800.0;
}

__device__ double npt_box_force(const NptSettings& c, double ke, double trace_virial, double eps) {
  const double alpha = 1.0 + 1.0 / c.n_atoms;
  return alpha * 2.0 * ke - trace_virial - 3.0 * c.pressure * c.V0 * exp(3.0 * eps);
}

// before the force evaluation: half steps of both chains, half kick of the box momentum, the box moves; leaves the
// coefficients of the atoms' updates.  The thermostat's momentum scale is multiplied into thermostat chain[1].
__global__ void __launch_bounds__(256) npt_pre_kernel(double* state, NptSettings c, const double* __restrict__ virial9,
                                                      const double* __restrict__ partials, int n_partials) {
  __shared__ double sh[256];
  double* tc = state;
  double* bc = state + kNhcStateDoubles;
  double* box = state + 2 * kNhcStateDoubles;
  if (partials) {
    const double s = sum_partials_256(partials, n_partials, sh);
    if (threadIdx.x == 0) tc[0] = s;
  }
  if (threadIdx.x != 0) return;
  const double W = 3.0 * (c.n_atoms + 1.0) * c.kT * c.tau_b * c.tau_b;
  const double alpha = 1.0 + 1.0 / c.n_atoms;
  double eps = box[0], p_eps = box[1];
  p_eps *= nhc_advance(bc, c.L, c.chain_steps, c.sy_steps, c.dt, c.tau_b, c.kT, 1.0, 1);
  tc[1] *= nhc_advance(tc, c.L, c.chain_steps, c.sy_steps, c.dt, c.tau_t, c.kT, 3.0 * c.n_atoms, 1);
  const double trW = virial9[0] + virial9[4] + virial9[8];
  p_eps += 0.5 * c.dt * npt_box_force(c, tc[0], trW, eps);
  const double v_eps = p_eps / W;
  const double x = alpha * v_eps * 0.5 * c.dt;
  box[2] = exp(-x);
  box[3] = 0.5 * c.dt * sinhx_x(0.5 * x) * exp(-0.5 * x);
  const double y = v_eps * c.dt;
  eps += y;
  box[4] = exp(y);
  box[5] = c.dt * exp(0.5 * y) * sinhx_x(0.5 * y);
  box[0] = eps; box[1] = p_eps;
  box[6] = c.V0 * exp(3.0 * eps);
}

// after the force evaluation and the atoms' second kick: the box's second half kick, then half steps of both chains
__global__ void __launch_bounds__(256) npt_post_kernel(double* state, NptSettings c, const double* __restrict__ virial9,
                                                       const double* __restrict__ partials, int n_partials) {
  __shared__ double sh[256];
  double* tc = state;
  double* bc = state + kNhcStateDoubles;
  double* box = state + 2 * kNhcStateDoubles;
  const double ke = sum_partials_256(partials, n_partials, sh);
  if (threadIdx.x != 0) return;
  const double W = 3.0 * (c.n_atoms + 1.0) * c.kT * c.tau_b * c.tau_b;
  double p_eps = box[1];
  const double trW = virial9[0] + virial9[4] + virial9[8];
  p_eps += 0.5 * c.dt * npt_box_force(c, ke, trW, box[0]);
  tc[0] = ke;
  bc[0] = p_eps * p_eps / (2.0 * W);
  tc[1] = nhc_advance(tc, c.L, c.chain_steps, c.sy_steps, c.dt, c.tau_t, c.kT, 3.0 * c.n_atoms, 1);
  p_eps *= nhc_advance(bc, c.L, c.chain_steps, c.sy_steps, c.dt, c.tau_b, c.kT, 1.0, 1);
  box[1] = p_eps;
}

// v <- scale_t v ; v <- c1 v + c2 a ; R <- r1 R + r2 v
__global__ void __launch_bounds__(256) npt_first_kernel(int n, const float* __restrict__ m, float* __restrict__ R, float* __restrict__ V,
                                                        const float* __restrict__ F, const double* __restrict__ state) {
  int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const double* box = state + 2 * kNhcStateDoubles;
  const float scale = (float)state[1];
  const float c1 = (float)box[2] * scale, c2 = (float)box[3] * kAccel / m[i];
  const double r1m1 = box[4] - 1.0;            // the box moves by ~1e-6 per step: keep the increment, not the factor, in float
  const float r1 = (float)r1m1, r2 = (float)box[5];
  for (int k = 0; k < 3; ++k) {
    const float v = fmaf(V[3 * (size_t)i + k], c1, c2 * F[3 * (size_t)i + k]);
    V[3 * (size_t)i + k] = v;
    const float x = R[3 * (size_t)i + k];
    R[3 * (size_t)i + k] = x + fmaf(x, r1, r2 * v);
  }
}

// v <- c1 v + c2 a, and each block's share of the kinetic energy (eV)
__global__ void __launch_bounds__(256) npt_second_kernel(int n, const float* __restrict__ m, float* __restrict__ V,
                                                         const float* __restrict__ F, const double* __restrict__ state,
                                                         double* __restrict__ partials) {
  __shared__ double sh[256];
  int i = blockIdx.x * 256 + threadIdx.x;
  const double* box = state + 2 * kNhcStateDoubles;
  double ke = 0.0;
  if (i < n) {
    const float mi = m[i];
    const float c1 = (float)box[2], c2 = (float)box[3] * kAccel / mi;
    double v2 = 0.0;
    for (int k = 0; k < 3; ++k) {
      const float v = fmaf(V[3 * (size_t)i + k], c1, c2 * F[3 * (size_t)i + k]);
      V[3 * (size_t)i + k] = v;
      v2 += (double)v * (double)v;
    }
    ke = 0.5 * (double)mi * v2 / kAccelD;
  }
  const double sum = block_sum_256(ke, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = sum;
}

__global__ void npt_init_kernel(double* state) {
  int t = threadIdx.x;
  if (t < kNptStateDoubles) state[t] = (t == 1 || t == kNhcStateDoubles + 1) ? 1.0 : 0.0;
}
}  // namespace

int nhc_settings_ok(int chain_length, int chain_steps, int sy_steps, double dt, double tau, double kT, double dof) {
  if (chain_length < 1 || chain_length > kNhcMaxChain) return 0;
  if (chain_steps < 1 || chain_steps > 64) return 0;
  if (!(sy_steps == 1 || sy_steps == 3 || sy_steps == 5 || sy_steps == 7)) return 0;
  if (!(dt > 0.0) || !(tau > 0.0) || !(kT > 0.0) || !(dof > 0.0)) return 0;
  return 1;
}

void nhc_init(cudaStream_t st, double* chain) {
  nhc_init_kernel<<<1, 32, 0, st>>>(chain);
  count_launch();
}

void nhc_half_steps(cudaStream_t st, double* chain, int L, int chain_steps, int sy_steps, double dt, double tau, double kT, double dof,
                    int n_half, int fresh_scale, const double* partials, int n_partials) {
  nhc_half_steps_kernel<<<1, 256, 0, st>>>(chain, L, chain_steps, sy_steps, dt, tau, kT, dof, n_half, fresh_scale, partials, n_partials);
  count_launch();
}

void md_kinetic_partials(cudaStream_t st, int n, const float* m, const float* V, double* partials) {
  ke_partial_kernel<<<(n + 255) / 256, 256, 0, st>>>(n, m, V, partials);
  count_launch();
}

void md_first_half(cudaStream_t st, int n, float dt, const float* m, float* R, float* V, const float* F, const double* chain) {
  vv_first_scaled_kernel<<<(n + 255) / 256, 256, 0, st>>>(n, dt, m, R, V, F, chain);
  count_launch();
}

void md_second_half(cudaStream_t st, int n, float dt, const float* m, float* V, const float* F, double* partials) {
  vv_second_ke_kernel<<<(n + 255) / 256, 256, 0, st>>>(n, dt, m, V, F, partials);
  count_launch();
}

void npt_init(cudaStream_t st, double* state) {
  npt_init_kernel<<<1, 64, 0, st>>>(state);
  count_launch();
}

static NptSettings npt_settings(const NptParams& p) {
  NptSettings c;
  c.L = p.chain_length; c.chain_steps = p.chain_steps; c.sy_steps = p.sy_steps; c.n_atoms = p.n_atoms;
  c.dt = p.dt; c.kT = p.kT; c.pressure = p.pressure; c.tau_t = p.tau_t; c.tau_b = p.tau_b; c.V0 = p.V0;
  return c;
}

void npt_pre(cudaStream_t st, double* state, const NptParams& p, const double* virial9, const double* partials, int n_partials) {
  npt_pre_kernel<<<1, 256, 0, st>>>(state, npt_settings(p), virial9, partials, n_partials);
  count_launch();
}

void npt_post(cudaStream_t st, double* state, const NptParams& p, const double* virial9, const double* partials, int n_partials) {
  npt_post_kernel<<<1, 256, 0, st>>>(state, npt_settings(p), virial9, partials, n_partials);
  count_launch();
}

void npt_first_half(cudaStream_t st, int n, const float* m, float* R, float* V, const float* F, const double* state) {
  npt_first_kernel<<<(n + 255) / 256, 256, 0, st>>>(n, m, R, V, F, state);
  count_launch();
}

void npt_second_half(cudaStream_t st, int n, const float* m, float* V, const float* F, const double* state, double* partials) {
  npt_second_kernel<<<(n + 255) / 256, 256, 0, st>>>(n, m, V, F, state, partials);
  count_launch();
}

void md_apply_scale(cudaStream_t st, int n, float* V, double* chain) {
  size_t n3 = 3 * (size_t)n;
  scale_velocities_kernel<<<(unsigned)((n3 + 255) / 256), 256, 0, st>>>(n3, V, chain);
  nhc_reset_scale_kernel<<<1, 1, 0, st>>>(chain);
  count_launch(2);
}
}  // namespace so3lr

// Launchers for the MD step bodies (velocity Verlet halves, Nose-Hoover chain).  See md.cu.
#pragma once
#include <cuda_runtime.h>

namespace so3lr {
constexpr int kNhcMaxChain = 8;
// chain state on the device: [0] kinetic energy (eV), [1] momentum scale waiting to be applied,
// [2, 2+8) chain positions, [10, 18) chain momenta (eV fs)
constexpr int kNhcStateDoubles = 2 + 2 * kNhcMaxChain;

// NPT state on the device: thermostat chain | barostat chain | box block (eps, p_eps, four step coefficients, volume, spare)
constexpr int kNptStateDoubles = 2 * kNhcStateDoubles + 8;
struct NptParams {
  int chain_length, chain_steps, sy_steps, n_atoms;
  double dt, kT, pressure, tau_t, tau_b, V0;
};
void npt_init(cudaStream_t st, double* state);
void npt_pre(cudaStream_t st, double* state, const NptParams& p, const double* virial9, const double* partials, int n_partials);
void npt_post(cudaStream_t st, double* state, const NptParams& p, const double* virial9, const double* partials, int n_partials);
void npt_first_half(cudaStream_t st, int n, const float* m, float* R, float* V, const float* F, const double* state);
void npt_second_half(cudaStream_t st, int n, const float* m, float* V, const float* F, const double* state, double* partials);

int nhc_settings_ok(int chain_length, int chain_steps, int sy_steps, double dt, double tau, double kT, double dof);
void nhc_init(cudaStream_t st, double* chain);
void nhc_half_steps(cudaStream_t st, double* chain, int chain_length, int chain_steps, int sy_steps, double dt, double tau, double kT,
                    double dof, int n_half, int fresh_scale, const double* partials, int n_partials);
void md_kinetic_partials(cudaStream_t st, int n, const float* m, const float* V, double* partials);
void md_first_half(cudaStream_t st, int n, float dt, const float* m, float* R, float* V, const float* F, const double* chain);
void md_second_half(cudaStream_t st, int n, float dt, const float* m, float* V, const float* F, double* partials);
void md_apply_scale(cudaStream_t st, int n, float* V, double* chain);
}  // namespace so3lr

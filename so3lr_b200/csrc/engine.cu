// Evaluation contexts and the C ABI of libso3lr_b200 (see include/so3lr_b200.h).
#include "../../include/so3lr_b200.h"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

#include "kernels.h"
#include "md.h"

using namespace so3lr;

struct so3lr_b200_model {
  int device = 0;
  ModelDev M{};
  std::vector<void*> owned;
};

namespace {
thread_local int64_t* tl_launch_counter = nullptr;   // the running entry point's context counter
}
namespace so3lr {
void count_launch(int kernels) {
  if (tl_launch_counter) *tl_launch_counter += kernels;
}
}  // namespace so3lr

namespace {

// first atomic number outside [1, kMaxZ] (0 -> -1 so that the result is non-zero), 0 when all are supported
int first_unsupported_element(const int32_t* Z, int n) {
  for (int a = 0; a < n; ++a)
    if (Z[a] < 1 || Z[a] > kMaxZ) return Z[a] == 0 ? -1 : Z[a];
  return 0;
}

// tracked device allocation
struct Pool {
  std::vector<void*> ptrs;
  int status = kOk;
  template <typename T>
  T* get(size_t n) {
    void* p = nullptr;
    if (n == 0) n = 1;
    if (cudaMalloc(&p, n * sizeof(T)) != cudaSuccess) { status = kCudaError; return nullptr; }
    // rows that a domain-decomposed evaluation never writes (outer ghost shells) are still read and multiplied by zero
    // cotangents: they must hold finite numbers
    if (cudaMemset(p, 0, n * sizeof(T)) != cudaSuccess) status = kCudaError;
    ptrs.push_back(p);
    return (T*)p;
  }
  void release() {
    for (void* p : ptrs) cudaFree(p);
    ptrs.clear();
  }
};

__global__ void fill_kernel(float* p, size_t n, float v) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}
__global__ void combine_energy_kernel(int n, const float* e_nn, const float* e_zbl, const float* e_c, const float* e_d, float* e_atom) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) e_atom[i] = ((e_nn[i] + e_zbl[i]) + e_c[i]) + e_d[i];
}
__global__ void moved_kernel(int n, const float* R, const float* Rref, float thr2, int* flag) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float dx = R[3 * (size_t)i] - Rref[3 * (size_t)i], dy = R[3 * (size_t)i + 1] - Rref[3 * (size_t)i + 1],
        dz = R[3 * (size_t)i + 2] - Rref[3 * (size_t)i + 2];
  float d2 = dx * dx + dy * dy + dz * dz;
  if (!(d2 <= thr2)) atomicOr(flag, (d2 != d2 || isinf(d2)) ? 2 : 1);
}
__global__ void row_ptr_from_sorted_kernel(int n, long long n_edges, const int* __restrict__ idx_i, int* __restrict__ row_ptr) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n) return;
  // first edge whose centre index is >= i
  long long lo = 0, hi = n_edges;
  while (lo < hi) {
    long long mid = (lo + hi) >> 1;
    if (idx_i[mid] < i) lo = mid + 1; else hi = mid;
  }
  row_ptr[i] = (int)lo;
}
__global__ void export_list_kernel(int n, long long count, long long capacity, const int* __restrict__ edge_i,
                                   const int* __restrict__ nbr_j, int* __restrict__ idx) {
  long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= capacity) return;
  idx[e] = e < count ? edge_i[e] : n;
  idx[capacity + e] = e < count ? nbr_j[e] : n;
}
// atoms are evaluated in a spatially sorted order: slot k holds atom perm[k]
__global__ void gather_positions_kernel(int n, const int* __restrict__ perm, const float* __restrict__ R, float* __restrict__ Rs) {
  int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const size_t a = (size_t)perm[k];
  Rs[3 * (size_t)k] = R[3 * a]; Rs[3 * (size_t)k + 1] = R[3 * a + 1]; Rs[3 * (size_t)k + 2] = R[3 * a + 2];
}
__global__ void gather_int_kernel(int n, const int* __restrict__ perm, const int* __restrict__ src, int* __restrict__ dst) {
  int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k < n) dst[k] = src[perm[k]];
}
struct UnsortArgs {
  const float* src[7];
  float* dst[7];
};
__global__ void unsort_kernel(int n, const int* __restrict__ perm, const float* __restrict__ Fs, float* __restrict__ F, UnsortArgs A) {
  int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const size_t a = (size_t)perm[k];
  F[3 * a] = Fs[3 * (size_t)k]; F[3 * a + 1] = Fs[3 * (size_t)k + 1]; F[3 * a + 2] = Fs[3 * (size_t)k + 2];
#pragma unroll
  for (int q = 0; q < 7; ++q)
    if (A.dst[q]) A.dst[q][a] = A.src[q][k];
}
__global__ void __launch_bounds__(1024) sum_to_double_kernel(int n, const float* __restrict__ a, double* __restrict__ out) {
  __shared__ double red[32];
  double v = 0.0;
  for (int k = threadIdx.x; k < n; k += blockDim.x) v += (double)a[k];
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[w];
    *out = s;
  }
}
// per-atom virial rows (xx yy zz yz xz xy) -> per-block sums in double -> the symmetric 3x3 total
__global__ void __launch_bounds__(256) virial_partial_kernel(int n, const float* __restrict__ W, double* __restrict__ partials) {
  __shared__ double sh[6][8];
  double a[6] = {0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
  for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256)
#pragma unroll
    for (int k = 0; k < 6; ++k) a[k] += (double)W[6 * (size_t)i + k];
#pragma unroll
  for (int k = 0; k < 6; ++k) {
    double v = a[k];
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) sh[k][threadIdx.x >> 5] = v;
  }
  __syncthreads();
  if (threadIdx.x < 6) {
    double v = 0.0;
    for (int w = 0; w < 8; ++w) v += sh[threadIdx.x][w];
    partials[6 * blockIdx.x + threadIdx.x] = v;
  }
}
__global__ void virial_final_kernel(int n_blocks, const double* __restrict__ partials, double* __restrict__ out9) {
  __shared__ double v[6];
  if (threadIdx.x < 6) {
    double s = 0.0;
    for (int b = 0; b < n_blocks; ++b) s += partials[6 * b + threadIdx.x];
    v[threadIdx.x] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    out9[0] = v[0]; out9[4] = v[1]; out9[8] = v[2];
    out9[5] = out9[7] = v[3]; out9[2] = out9[6] = v[4]; out9[1] = out9[3] = v[5];
  }
}
// out = a - (*sum / count): removes the mean whose numerator was summed over all ranks
__global__ void subtract_mean_kernel(int n, const float* __restrict__ a, const double* __restrict__ sum, double count,
                                     float* __restrict__ out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = a[i] - (float)(*sum / count);
}
__global__ void abs_kernel(int n, const float* __restrict__ a, float* __restrict__ out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = fabsf(a[i]);
}
// velocity Verlet halves.  units: eV, Angstrom, amu, fs -> acceleration = F/m * 9.64853321e-3 A/fs^2
constexpr float kAccel = 9.648533212331e-3f;
__global__ void vv_first_kernel(int n, float dt, const float* m, float* R, float* V, const float* F) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.5f * dt * kAccel / m[i];
  for (int k = 0; k < 3; ++k) {
    float v = V[3 * (size_t)i + k] + s * F[3 * (size_t)i + k];
    V[3 * (size_t)i + k] = v;
    R[3 * (size_t)i + k] += dt * v;
  }
}
__global__ void vv_second_kernel(int n, float dt, const float* m, float* V, const float* F) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.5f * dt * kAccel / m[i];
  for (int k = 0; k < 3; ++k) V[3 * (size_t)i + k] += s * F[3 * (size_t)i + k];
}

int make_cell(const float* cell9, Cell* c) {
  std::memset(c, 0, sizeof(Cell));
  if (!cell9) { c->periodic = 0; return kOk; }
  double h[9], inv[9];
  for (int k = 0; k < 9; ++k) h[k] = cell9[k];
  double det = h[0] * (h[4] * h[8] - h[5] * h[7]) - h[1] * (h[3] * h[8] - h[5] * h[6]) + h[2] * (h[3] * h[7] - h[4] * h[6]);
  if (!(std::fabs(det) > 1e-12) || !std::isfinite(det)) return kInvalidArgument;
  inv[0] = (h[4] * h[8] - h[5] * h[7]) / det; inv[1] = (h[2] * h[7] - h[1] * h[8]) / det; inv[2] = (h[1] * h[5] - h[2] * h[4]) / det;
  inv[3] = (h[5] * h[6] - h[3] * h[8]) / det; inv[4] = (h[0] * h[8] - h[2] * h[6]) / det; inv[5] = (h[2] * h[3] - h[0] * h[5]) / det;
  inv[6] = (h[3] * h[7] - h[4] * h[6]) / det; inv[7] = (h[1] * h[6] - h[0] * h[7]) / det; inv[8] = (h[0] * h[4] - h[1] * h[3]) / det;
  for (int k = 0; k < 9; ++k) { c->h[k] = (float)h[k]; c->hinv[k] = (float)inv[k]; }
  c->periodic = 1;
  return kOk;
}

}  // namespace

// Optional per-kernel-group timing with CUDA events on the launching stream.
// attn_fwd / attn_bwd: the kernels of the two layers with a spherical filter (one launch per layer); the first layer's
// tabulated kernels have groups of their own, so that a group's time divided by its launches is one kernel's time
enum ProfGroup { kPNlist = 0, kPGeom, kPProj, kPAttnFwd, kPPostFwd, kPHeads, kPPairLr, kPPostBwd, kPAttnBwd, kPProjBwd, kPScatter,
                 kPMisc, kPMd, kPLayer0Fwd, kPLayer0Bwd, kPKspace, kPGroups };
static const char* kProfNames[kPGroups] = {"nlist", "sr_geometry_zbl", "proj_fwd", "attn_fwd", "atom_post_fwd", "heads", "pair_lr",
                                           "atom_post_bwd", "attn_bwd", "proj_bwd", "force_scatter", "misc", "md_step",
                                           "layer0_fwd", "layer0_bwd", "kspace"};
struct Profiler {
  bool on = false;
  std::vector<cudaEvent_t> a, b;
  std::vector<int> grp;
  size_t used = 0;
  void begin(int g, cudaStream_t st) {
    if (!on) return;
    if (used == a.size()) {
      cudaEvent_t e0, e1;
      cudaEventCreate(&e0); cudaEventCreate(&e1);
      a.push_back(e0); b.push_back(e1); grp.push_back(g);
    }
    grp[used] = g;
    cudaEventRecord(a[used], st);
  }
  void end(cudaStream_t st) {
    if (!on) return;
    cudaEventRecord(b[used], st);
    ++used;
  }
  void destroy() {
    for (auto e : a) cudaEventDestroy(e);
    for (auto e : b) cudaEventDestroy(e);
    a.clear(); b.clear(); grp.clear(); used = 0;
  }
};

struct so3lr_b200_system {
  so3lr_b200_model* model = nullptr;
  // the model as this context sees it: a copy of the shared tables whose atom-embedding table is replaced by a context-owned
  // one when the structure carries a total charge or unpaired electrons (the charge / spin embeddings depend on the element,
  // the charge and the composition only); batches of several graphs get a per-atom embedding instead
  ModelDev mctx{};
  float* x0_atom = nullptr;
  Profiler prof;
  int n = 0, n_graphs = 1;
  int n_cap = 0;                 // atoms the per-atom arrays were allocated for
  int shells[4] = {0, 0, 0, 0};  // domain-decomposed evaluation: owned | + short-range ghosts | (unused) | all local atoms
  SpeciesTables sp{};            // per-element-pair tables of the first layer
  float* GV = nullptr;           // n_cap x 32 scratch of the tabulated first-layer reverse pass
  float *dd_gev2 = nullptr, *dd_gev_in = nullptr;   // ping-pong cotangents of ev between the layers of the reverse pass
  so3lr_b200_options opt{};
  Cell cell{};
  LrParams lr{};
  KSpaceDev ks{};                // reciprocal-space Coulomb part (off unless so3lr_b200_system_set_kspace switched it on)
  Cell ks_cell{};                // decomposed evaluation: the cell of the whole structure (`cell` is the rank's local one)
  bool ks_cell_set = false;
  Pool pool;
  // static inputs.  d_Z is the array the kernels read: d_Z0 (caller order) or d_Zs (sorted order)
  int *d_Z = nullptr, *d_Z0 = nullptr, *d_Zs = nullptr, *d_seg = nullptr, *d_graph_start = nullptr;
  // spatial ordering (periodic single-graph systems): slot k of every internal per-atom array holds atom d_perm[k]
  int* d_perm = nullptr;
  float *d_Rs = nullptr, *F_s = nullptr;
  bool sorted = false;
  // per-atom results in caller order (alias the internal arrays when not sorted)
  float *o_e_atom = nullptr, *o_q = nullptr, *o_h = nullptr, *o_zbl = nullptr, *o_coul = nullptr, *o_disp = nullptr;
  float *u_e_atom = nullptr, *u_q = nullptr, *u_h = nullptr, *u_zbl = nullptr, *u_coul = nullptr, *u_disp = nullptr;
  float* d_total_charge = nullptr;
  // lists
  NeighborListDev sr, lrl;
  int sr_rows = 0;               // rows of the short-range list (all atoms, or the owned ones of a decomposed evaluation)
  ValidEdges ve;                 // its entries inside the cutoff, compacted at every evaluation
  NlistWorkspace* nws = nullptr;
  float* d_Rref = nullptr;
  int* d_flag = nullptr;   // [0] skin test of the current step, [1] sticky error word of the tensor-core kernels' bounded waits,
                           // [2] graph-level call: the caller's list is not symmetric
  int* h_flag = nullptr;   // pinned copy of both
  // deferred skin test: the flags of step k are read by the host at step k + 1 (two pinned slots and an event each), so a
  // step never waits for the device; the trigger distance is lowered by `skin_margin` to cover the extra step
  bool deferred_skin = false;
  float skin_margin = 0.f;
  int* h_flag2 = nullptr;            // pinned, 2 slots x 2 ints
  cudaEvent_t flag_event[2] = {nullptr, nullptr};
  bool flag_pending[2] = {false, false};
  int flag_slot = 0;
  double* h_box = nullptr; // pinned: the box coordinate read back by the NPT step
  bool virial_fresh = false;   // virial_sum belongs to the latest evaluation
  // CUDA graph of one force evaluation between two list rebuilds (small structures are bound by the launch rate): captured at the
  // second consecutive call with the same position / force buffers, replayed until the lists are rebuilt or the buffers change
  struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    const float* R = nullptr; float* F = nullptr; int64_t stamp = -1; bool virial = false;
    int64_t launches = 0, replays = 0;
    const float* last_R = nullptr; float* last_F = nullptr; int64_t last_stamp = -1;
    bool broken = false;        // a capture failed: the context stays on plain launches
  } step_graph;
  bool have_lists = false;
  // graph-level row pointers
  int *d_rowptr_g = nullptr, *d_rowptr_lr_g = nullptr;
  // activations
  float* x[kNumLayers + 1] = {};
  float* ev[kNumLayers + 1] = {};
  float *qkv[kNumLayers] = {}, *xa[kNumLayers] = {}, *ev1[kNumLayers] = {}, *z1[kNumLayers] = {}, *x3[kNumLayers] = {},
        *gate[kNumLayers] = {};
  float *ze = nullptr, *zq = nullptr, *zh = nullptr, *e_nn = nullptr, *q_raw = nullptr, *hv = nullptr, *q = nullptr, *h = nullptr;
  float *e_atom = nullptr, *e_zbl = nullptr, *e_coul = nullptr, *e_disp = nullptr;
  float *gq = nullptr, *gh = nullptr, *gq_raw = nullptr, *ones = nullptr;
  float* pair_pack = nullptr;   // (x, y, z, q) | (Fx, Fy, Fz, dE/dq) | (h, alpha_free, c6_free, -) per atom for the packed long-range kernel
  float *g4 = nullptr, *g_xa = nullptr, *gev_a = nullptr, *gev_b = nullptr, *gev1 = nullptr, *g_qkv = nullptr;
  float* dR = nullptr;
  long long edge_cap = 0;
  float* F_int = nullptr;
  double* d_energy = nullptr;
  double* red_scratch = nullptr;   // block partials of the whole-structure sums (charge, energy, dipole)
  float* d_dipole = nullptr;
  // host staging
  float *h_R = nullptr, *h_F = nullptr, *h_q = nullptr, *h_h = nullptr, *h_dip = nullptr;
  double* h_E = nullptr;
  float* d_Rstage = nullptr;
  cudaStream_t own_stream = nullptr;
  int64_t n_rebuilds = 0, n_launches = 0;
  double* ke_partials = nullptr;   // one kinetic-energy share per block of the velocity kernels
  // strain derivative of the energy (on request): per-atom rows of six symmetrised components, block partials, 3x3 total
  bool want_virial = false;
  float* virial = nullptr;
  double* virial_partials = nullptr;
  double* virial_sum = nullptr;
  float* vir() const { return want_virial ? virial : nullptr; }
};

namespace {

// initial features of atoms [0, n): per-atom rows when the context carries them (charged batches), else the element table
int embed_atoms(so3lr_b200_system* S, cudaStream_t st, int n, float* x) {
  if (S->x0_atom) {
    SO3LR_CUDA_CHECK(cudaMemcpyAsync(x, S->x0_atom, (size_t)n * kF * sizeof(float), cudaMemcpyDeviceToDevice, st));
    return kOk;
  }
  launch_embed(st, S->mctx, S->d_Z, n, x);
  return kOk;
}

void fill(cudaStream_t s, float* p, size_t n, float v) {
  if (n == 0) return;
  if (v == 0.f) { cudaMemsetAsync(p, 0, n * sizeof(float), s); return; }
  { fill_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(p, n, v); count_launch(); }
}

int ensure_edge_buffers(so3lr_b200_system* S, long long n_edges) {
  if (n_edges <= S->edge_cap) return valid_edges_reserve(&S->ve, S->n_cap, S->edge_cap);   // row arrays exist even without edges
  long long cap = n_edges + n_edges / 4 + 1024;
  if (S->dR) cudaFree(S->dR);
  S->dR = nullptr;
  SO3LR_CUDA_CHECK(cudaMalloc((void**)&S->dR, (size_t)cap * 3 * sizeof(float)));
  S->edge_cap = cap;
  return valid_edges_reserve(&S->ve, S->n_cap, cap);
}

constexpr int kSortMinAtoms = 512;

int rebuild_lists(so3lr_b200_system* S, cudaStream_t st, const float* R_user, bool allow_sort) {
  const float r_sr = kCutoffSr + S->opt.skin;
  const float* R = R_user;
  const int nb = (S->n + 255) / 256;
  S->sorted = allow_sort && S->cell.periodic && S->n_graphs == 1 && S->n >= kSortMinAtoms;
  if (S->sorted) {
    int rc0 = spatial_order(S->nws, st, S->cell, S->n, R_user, r_sr, S->d_perm);
    if (rc0) return rc0;
    { gather_positions_kernel<<<nb, 256, 0, st>>>(S->n, S->d_perm, R_user, S->d_Rs); count_launch(); }
    { gather_int_kernel<<<nb, 256, 0, st>>>(S->n, S->d_perm, S->d_Z0, S->d_Zs); count_launch(); }
    R = S->d_Rs;
    S->d_Z = S->d_Zs;
    S->o_e_atom = S->u_e_atom; S->o_q = S->u_q; S->o_h = S->u_h; S->o_zbl = S->u_zbl; S->o_coul = S->u_coul; S->o_disp = S->u_disp;
  } else {
    S->d_Z = S->d_Z0;
    S->o_e_atom = S->e_atom; S->o_q = S->q; S->o_h = S->h; S->o_zbl = S->e_zbl; S->o_coul = S->e_coul; S->o_disp = S->e_disp;
  }
  const bool many = S->n_graphs > 1 || !S->cell.periodic;
  const int* seg = S->n_graphs > 1 ? S->d_seg : nullptr;
  const int* gs = (S->n_graphs > 1 && !S->cell.periodic) ? S->d_graph_start : nullptr;
  (void)many;
  int rc = nlist_build(S->nws, st, S->cell, S->n, R, r_sr, 0, seg, gs, &S->sr, 1, nullptr);
  if (rc) return rc;
  float r_lr;
  const int* gs_lr = gs;
  if (S->opt.cutoff_lr > 0.f) r_lr = S->opt.cutoff_lr + S->opt.skin;
  else if (S->opt.lr_list_cutoff > 0.f) r_lr = S->opt.lr_list_cutoff + S->opt.skin;
  else {
    r_lr = 1e18f;
    if (S->cell.periodic) return kInvalidArgument;   // all-pairs long range needs free space
    gs_lr = S->d_graph_start;                        // loop over the graph's atoms, no cells
  }
  rc = nlist_build(S->nws, st, S->cell, S->n, R, r_lr, S->opt.lr_both_directions ? 0 : 1, seg ? seg : (gs_lr ? S->d_seg : nullptr),
                   gs_lr, &S->lrl, 1, nullptr);
  if (rc) return rc;
  SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->d_Rref, R_user, (size_t)S->n * 3 * sizeof(float), cudaMemcpyDeviceToDevice, st));
  rc = ensure_edge_buffers(S, S->sr.count);
  if (rc) return rc;
  S->sr_rows = S->n;
  S->have_lists = true;
  S->n_rebuilds++;
  return kOk;
}

// Graph-level evaluation (displacements and lists given by the caller, gradients per edge): scatter kernels with atomics,
// valid for any list.

// Attention kernels of the layers with a spherical filter.  Default: the tiled tcgen05 kernels in both directions.
// SO3LR_B200_ATTENTION selects the earlier generations for comparison runs (all are covered by tests/test_gpu_modes.py):
// "tcf" tiled forward with the warp-per-receiver mma.sync reverse kernel, "mma" warp-per-receiver mma.sync kernels in both
// directions, "simt" FP32 shared-memory filter GEMMs.
enum AttentionMode { kAttnSimt = 0, kAttnMma = 1, kAttnTcFwd = 2, kAttnTc = 3 };
int attention_mode() {
  static const int v = [] {
    const char* e = std::getenv("SO3LR_B200_ATTENTION");
    if (e && std::strcmp(e, "simt") == 0) return (int)kAttnSimt;
    if (e && std::strcmp(e, "mma") == 0) return (int)kAttnMma;
    if (e && std::strcmp(e, "tcf") == 0) return (int)kAttnTcFwd;
    return (int)kAttnTc;
  }();
  return v;
}
bool use_mma_attention() { return attention_mode() >= kAttnMma; }
// SO3LR_B200_DENSE=simt selects the FP32 shared-memory versions of the per-atom dense blocks (see use_tc_dense below)
// SO3LR_B200_LAYER0=generic evaluates the first layer with the generic attention kernels instead of the element-pair tables
bool use_layer0_tables() {
  static const bool v = [] {
    const char* e = std::getenv("SO3LR_B200_LAYER0");
    return !(e && std::strcmp(e, "generic") == 0);
  }();
  return v;
}
bool use_mma_dense() {
  static const bool v = [] {
    const char* e = std::getenv("SO3LR_B200_DENSE");
    return !(e && std::strcmp(e, "simt") == 0);
  }();
  return v;
}
// The post-attention blocks run on the tcgen05 kernels of dense_tc.cu unless SO3LR_B200_DENSE names an earlier generation
// ("mma": mma.sync kernels, "simt": FP32 shared-memory kernels).
bool use_tc_dense() {
  static const bool v = [] {
    const char* e = std::getenv("SO3LR_B200_DENSE");
    return !(e && (std::strcmp(e, "simt") == 0 || std::strcmp(e, "mma") == 0));
  }();
  return v;
}
// With the tensor-core dense blocks the q/k/v projections ride along: the forward block also emits the next layer's
// q/k/v rows, the reverse block forms its input cotangent from the upper layer's g_xa and g_qkv.  `next` / `up` = that
// neighbouring layer (nullptr: no fusion at this end of the network).
void post_fwd_dispatch(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, float* z1, float* x3, float* gate,
                       float* x4, float* ev2, const LayerDev* next, float* qkv_next, int* err) {
  if (use_tc_dense()) launch_atom_post_fwd_tc(s, L, n, xa, ev1, z1, x3, gate, x4, ev2, next ? next->proj_u : nullptr, qkv_next, err);
  else if (use_mma_dense()) launch_atom_post_fwd_mma(s, L, n, xa, ev1, z1, x3, gate, x4, ev2, next ? next->proj_f : nullptr, qkv_next);
  else launch_atom_post_fwd(s, L, n, xa, ev1, z1, x3, gate, x4, ev2);
}
void post_bwd_dispatch(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, const float* z1, const float* x3,
                       const float* gate, const float* g4, const float* gev2, float* g_xa, float* gev1, const LayerDev* up,
                       const float* g_qkv_up, int* err) {
  if (use_tc_dense()) launch_atom_post_bwd_tc(s, L, n, xa, ev1, z1, x3, gate, g4, gev2, g_xa, gev1, up ? up->projT_u : nullptr, g_qkv_up, err);
  else if (use_mma_dense()) launch_atom_post_bwd_mma(s, L, n, xa, ev1, z1, x3, gate, g4, gev2, g_xa, gev1, up ? up->projT_f : nullptr, g_qkv_up);
  else launch_atom_post_bwd(s, L, n, xa, ev1, z1, x3, gate, g4, gev2, g_xa, gev1);
}
void heads_fwd_dispatch(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* x, float* ze, float* zq, float* zh,
                        float* e_nn, float* q_raw, float* hv, int* err) {
  if (use_tc_dense()) launch_heads_fwd_tc(s, M, n, Z, x, ze, zq, zh, e_nn, q_raw, hv, err);
  else if (use_mma_dense()) launch_heads_fwd_mma(s, M, n, Z, x, ze, zq, zh, e_nn, q_raw, hv);
  else launch_heads_fwd(s, M, n, Z, x, ze, zq, zh, e_nn, q_raw, hv);
}
void heads_bwd_dispatch(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* ze, const float* zq, const float* zh,
                        const float* hv, const float* ge, const float* gq, const float* gh, float* gx, int* err) {
  if (use_tc_dense()) launch_heads_bwd_tc(s, M, n, Z, ze, zq, zh, hv, ge, gq, gh, gx, err);
  else if (use_mma_dense()) launch_heads_bwd_mma(s, M, n, Z, ze, zq, zh, hv, ge, gq, gh, gx);
  else launch_heads_bwd(s, M, n, Z, ze, zq, zh, hv, ge, gq, gh, gx);
}
void attn_fwd_dispatch(so3lr_b200_system* S, cudaStream_t st, const LayerDev& L, int n_recv, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                       const float* qkv, const float* x_in, const float* ev_in, float* xa, float* ev1) {
  if (L.has_spherical && attention_mode() >= kAttnTcFwd) launch_attn_fwd_tc(st, L, S->ve, n_recv, qkv, x_in, ev_in, xa, ev1, S->d_flag + 1);
  else if (L.has_spherical && use_mma_attention()) launch_attn_fwd_mma(st, L, n_recv, n, row_ptr, nbr_j, dR, qkv, x_in, ev_in, xa, ev1);
  else launch_attn_fwd_sym(st, L, n_recv, n, row_ptr, nbr_j, dR, qkv, x_in, ev_in, xa, ev1);
}
void attn_bwd_dispatch(so3lr_b200_system* S, cudaStream_t st, const LayerDev& L, int n_recv, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                       const float* qkv, const float* ev_in, const float* g_xa, const float* gev1, float* g_qkv, float* gev_in, float* F,
                       int first_layer, float* virial) {
  if (!first_layer && L.has_spherical && attention_mode() == kAttnTc)
    launch_attn_bwd_tc(st, L, S->ve, n_recv, qkv, ev_in, g_xa, gev1, g_qkv, gev_in, F, virial, S->d_flag + 1);
  else if (!first_layer && L.has_spherical && use_mma_attention())
    launch_attn_bwd_mma(st, L, n_recv, n, row_ptr, nbr_j, dR, qkv, ev_in, g_xa, gev1, g_qkv, gev_in, F, virial);
  else launch_attn_bwd_sym(st, L, n_recv, n, row_ptr, nbr_j, dR, qkv, ev_in, g_xa, gev1, g_qkv, gev_in, F, first_layer, virial);
}

// SO3LR_B200_GRAPH=scatter keeps the graph-level call on the first-generation scatter kernels throughout (exact per-entry
// gradients also for lists that are symmetric)
bool graph_fast_path() {
  static const bool v = [] {
    const char* e = std::getenv("SO3LR_B200_GRAPH");
    return !(e && std::strcmp(e, "scatter") == 0);
  }();
  return v;
}

// Evaluation on caller-supplied lists and displacement vectors (receiver-sorted).  The per-atom blocks and heads are the ones of
// the fused path; the attention layers with a spherical filter run the tiled forward kernel on the entries inside the cutoff
// (it needs the rows sorted by receiver, nothing else).  The tiled reverse kernel evaluates both directions of a pair at the
// receiver, which presumes that every entry (i <- j, d) has its partner (j <- i, -d) in the list: a check kernel decides
// that on the device, and of the two reverse kernels launched per layer (tiled, scatter) the one that does not apply
// returns at once -- no host read, so the call stays enqueue-only.
int evaluate_graph(so3lr_b200_system* S, cudaStream_t st, const int* row_ptr, const int* nbr_j, const int* edge_i, long long n_edges,
                   const int* row_ptr_lr, const int* nbr_j_lr, const float* dR_in, const float* dR_lr_in, float* g_dR,
                   float* g_dR_lr_out, const float* ge, const float* positions = nullptr, float* g_positions = nullptr,
                   float* strain6 = nullptr) {
  const ModelDev& M = S->mctx;
  const int n = S->n;
  // the reciprocal-space part needs the positions and returns its own gradient; its per-atom energies are not separable, so a
  // non-uniform upstream cotangent is not supported with it
  if (S->ks.mode && (!positions || !g_positions || ge)) return kInvalidArgument;
  float* dR = const_cast<float*>(dR_in);
  const bool tiled = graph_fast_path() && attention_mode() == kAttnTc && n_edges > 0;
  int* asym = S->d_flag + 2;      // 1: some entry has no reversed partner (or the tiled path is off)
  if (tiled) {
    int rcv = valid_edges_reserve(&S->ve, S->n_cap, n_edges);
    if (rcv) return rcv;
    SO3LR_CUDA_CHECK(cudaMemsetAsync(asym, 0, sizeof(int), st));
    rcv = valid_edges_build(&S->ve, st, n, n, row_ptr, nbr_j, dR, true);
    if (rcv) return rcv;
    valid_edges_check_symmetric(S->ve, st, asym);
  }
  fill(st, S->e_zbl, n, 0.f); fill(st, S->e_coul, n, 0.f); fill(st, S->e_disp, n, 0.f);
  fill(st, S->gq, n, 0.f); fill(st, S->gh, n, 0.f);
  S->prof.begin(kPGeom, st); launch_sr_geometry_zbl(st, M, S->cell, n, n_edges, edge_i, nbr_j, S->d_Z, nullptr, 1, dR, S->e_zbl, g_dR, ge, nullptr); S->prof.end(st);
  { int rce = embed_atoms(S, st, n, S->x[0]); if (rce) return rce; }
  for (int l = 0; l < kNumLayers; ++l) {
    const LayerDev& L = M.layer[l];
    S->prof.begin(kPProj, st); launch_proj_fwd(st, L, S->x[l], n, S->qkv[l]); S->prof.end(st);
    S->prof.begin(kPAttnFwd, st);
    if (tiled && L.has_spherical) launch_attn_fwd_tc(st, L, S->ve, n, S->qkv[l], S->x[l], S->ev[l], S->xa[l], S->ev1[l], S->d_flag + 1);
    else launch_attn_fwd(st, L, n, row_ptr, nbr_j, dR, S->qkv[l], S->x[l], S->ev[l], S->xa[l], S->ev1[l]);
    S->prof.end(st);
    S->prof.begin(kPPostFwd, st);
    post_fwd_dispatch(st, L, n, S->xa[l], S->ev1[l], S->z1[l], S->x3[l], S->gate[l], S->x[l + 1], S->ev[l + 1], nullptr, nullptr, S->d_flag + 1);
    S->prof.end(st);
  }
  S->prof.begin(kPHeads, st);
  heads_fwd_dispatch(st, M, n, S->d_Z, S->x[kNumLayers], S->ze, S->zq, S->zh, S->e_nn, S->q_raw, S->hv, S->d_flag + 1);
  S->prof.end(st);
  launch_charge_conserve(st, S->n_graphs, S->d_graph_start, S->q_raw, S->d_total_charge, S->hv, S->q, S->h, S->n, S->red_scratch);
  S->prof.begin(kPPairLr, st);
  launch_pair_lr(st, S->lr, S->cell, n, row_ptr_lr, nbr_j_lr, S->d_Z, nullptr, S->q, S->h, 1, dR_lr_in, g_dR_lr_out, nullptr, nullptr, S->gq,
                 S->gh, S->e_coul, S->e_disp, ge);
  if (S->ks.mode) {
    fill(st, g_positions, (size_t)n * 3, 0.f);
    if (strain6) fill(st, strain6, 6, 0.f);
    int rck = launch_ewald(st, S->ks, S->cell, n, positions, S->q, S->d_total_charge, S->e_coul, S->gq, g_positions, strain6, -1.f);
    if (rck) return rck;
  }
  S->prof.end(st);
  { combine_energy_kernel<<<(n + 255) / 256, 256, 0, st>>>(n, S->e_nn, S->e_zbl, S->e_coul, S->e_disp, S->e_atom); count_launch(); }
  launch_charge_conserve_bwd(st, S->n_graphs, S->d_graph_start, S->gq, S->gq_raw, S->n, S->red_scratch);
  S->prof.begin(kPHeads, st);
  heads_bwd_dispatch(st, M, n, S->d_Z, S->ze, S->zq, S->zh, S->hv, ge ? ge : S->ones, S->gq_raw, S->gh, S->g4, S->d_flag + 1);
  S->prof.end(st);
  float* gev2 = S->gev_a;
  float* gev_in = S->gev_b;
  fill(st, gev2, (size_t)n * kMTot, 0.f);
  for (int l = kNumLayers - 1; l >= 0; --l) {
    const LayerDev& L = M.layer[l];
    S->prof.begin(kPPostBwd, st);
    post_bwd_dispatch(st, L, n, S->xa[l], S->ev1[l], S->z1[l], S->x3[l], S->gate[l], S->g4, gev2, S->g_xa, S->gev1, nullptr, nullptr, S->d_flag + 1);
    S->prof.end(st);
    if (l > 0) {
      SO3LR_CUDA_CHECK(cudaMemcpyAsync(gev_in, S->gev1, (size_t)n * kMTot * sizeof(float), cudaMemcpyDeviceToDevice, st));
      fill(st, S->g_qkv, (size_t)n * kProj, 0.f);
      S->prof.begin(kPAttnBwd, st);
      if (tiled && L.has_spherical) {
        int rcb = launch_attn_bwd_tc_graph(st, L, S->ve, n, S->qkv[l], S->ev[l], S->g_xa, S->gev1, S->g_qkv, gev_in, g_dR, S->d_flag + 1, asym);
        if (rcb) return rcb;
        launch_attn_bwd(st, L, n, row_ptr, nbr_j, dR, S->qkv[l], S->ev[l], S->g_xa, S->gev1, S->g_qkv, gev_in, g_dR, 0, asym);
      } else {
        launch_attn_bwd(st, L, n, row_ptr, nbr_j, dR, S->qkv[l], S->ev[l], S->g_xa, S->gev1, S->g_qkv, gev_in, g_dR, 0);
      }
      S->prof.end(st);
      // dL/dx_in = g_xa (skip connection) + projections^T
      SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->g4, S->g_xa, (size_t)n * kF * sizeof(float), cudaMemcpyDeviceToDevice, st));
      S->prof.begin(kPProjBwd, st); launch_proj_bwd(st, L, S->g_qkv, n, S->g4, 1); S->prof.end(st);
      float* t = gev2; gev2 = gev_in; gev_in = t;
    } else {
      S->prof.begin(kPAttnBwd, st); launch_attn_bwd(st, L, n, row_ptr, nbr_j, dR, S->qkv[l], S->ev[l], S->g_xa, S->gev1, nullptr, nullptr, g_dR, 1); S->prof.end(st);
    }
  }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// ---- positions -> forces (gather-only kernels on the symmetric short-range list) ----
// Atom slots are ordered by how far their features are needed: [0, n0) atoms whose energy is evaluated here ("owned"),
// [n0, n1) atoms within one interaction shell of them, [n1, n2) within two, [n2, n3) within three.  Layer l of the
// network is evaluated for the atoms that the owned atoms' energies can still see; a single-GPU evaluation has
// n0 = n1 = n2 = n3 = n.
// value and slope at the cutoff of the pair function the Coulomb term shifts: erf(r / sigma) / r, minus erf(r k_alpha) / r when the
// reciprocal-space sum holds that part
void set_coulomb_shift(LrParams& P) {
  if (!P.has_cutoff) return;
  const double rc = P.rc, sg = kSigmaCoulomb;
  double pot = std::erf(rc / sg) / rc;
  double dpot = (2.0 / std::sqrt(M_PI) / sg * std::exp(-(rc / sg) * (rc / sg)) - pot) / rc;
  if (P.k_alpha > 0.f) {
    const double a = P.k_alpha;
    const double potk = std::erf(rc * a) / rc;
    pot -= potk;
    dpot -= (2.0 / std::sqrt(M_PI) * a * std::exp(-(rc * a) * (rc * a)) - potk) / rc;
  }
  P.v_rc = (float)pot; P.dv_rc = (float)dpot;
}

// SO3LR_B200_CUDA_GRAPH=0 keeps every evaluation on plain launches
bool step_graphs_enabled() {
  static const bool v = [] {
    const char* e = std::getenv("SO3LR_B200_CUDA_GRAPH");
    return !(e && std::strcmp(e, "0") == 0);
  }();
  return v;
}
constexpr int kStepGraphMaxAtoms = 65536;   // above this a step is bound by its kernels, not by the launch rate
// the captured launches hold the cell, the pair-term constants and the buffers by value: anything that changes them drops the graph
void drop_step_graph(so3lr_b200_system* S) {
  if (S->step_graph.exec) cudaGraphExecDestroy(S->step_graph.exec);
  const bool broken = S->step_graph.broken;
  const int64_t replays = S->step_graph.replays;
  S->step_graph = so3lr_b200_system::StepGraph{};
  S->step_graph.broken = broken;
  S->step_graph.replays = replays;
}

struct Shells { int n0, n1, n2, n3; };

constexpr int kVirialBlocks = 1024;   // capacity of the block-partials buffer of the virial reduction
// sum of the per-atom virial rows of the atoms whose energy is evaluated here
void reduce_virial(so3lr_b200_system* S, cudaStream_t st, int n0) {
  int blocks = (n0 + 255) / 256;
  const int max_blocks = 4 * sm_count() < kVirialBlocks ? 4 * sm_count() : kVirialBlocks;   // four CTAs per SM, bounded by the partials buffer
  if (blocks > max_blocks) blocks = max_blocks;
  { virial_partial_kernel<<<blocks, 256, 0, st>>>(n0, S->virial, S->virial_partials); count_launch(); }
  { virial_final_kernel<<<1, 32, 0, st>>>(blocks, S->virial_partials, S->virial_sum); count_launch(); }
  S->virial_fresh = true;
}

// network forward up to the output heads: e_nn, q_raw, hv for the owned atoms; ZBL energy and force; F is zeroed first
int fused_forward(so3lr_b200_system* S, cudaStream_t st, const float* R, const Shells& c, bool owned_side_only, float* F) {
  const ModelDev& M = S->mctx;
  const int* row_ptr = S->sr.row_ptr; const int* nbr_j = S->sr.nbr_j; const int* edge_i = S->sr.edge_i;
  const int nrecv[kNumLayers] = {c.n2, c.n1, c.n0};   // receivers of layer l
  const int nsend[kNumLayers] = {c.n3, c.n2, c.n1};   // atoms whose q/k/v rows layer l reads
  fill(st, S->e_zbl, c.n0, 0.f);
  fill(st, F, (size_t)c.n3 * 3, 0.f);
  if (S->vir()) fill(st, S->virial, (size_t)c.n3 * 6, 0.f);
  S->prof.begin(kPGeom, st);
  launch_sr_geometry_zbl(st, M, S->cell, c.n3, S->sr.count, edge_i, nbr_j, S->d_Z, R, 0, S->dR, S->e_zbl, nullptr, nullptr, F,
                         owned_side_only ? c.n0 : -1, S->vir());
  if (attention_mode() >= kAttnTcFwd) {
    int rcv = valid_edges_build(&S->ve, st, S->sr_rows, c.n3, row_ptr, nbr_j, S->dR);
    if (rcv) return rcv;
  }
  S->prof.end(st);
  const bool tab0 = S->sp.n_species > 0 && use_layer0_tables();
  const bool fuse = use_mma_dense();   // q/k/v rows of layer l+1 come out of layer l's dense block
  if (!tab0) { int rce = embed_atoms(S, st, c.n3, S->x[0]); if (rce) return rce; }
  for (int l = 0; l < kNumLayers; ++l) {
    const LayerDev& L = M.layer[l];
    if (l == 0 && tab0) {
      S->prof.begin(kPLayer0Fwd, st);
      launch_layer0_fwd_tab(st, S->sp, M, nrecv[0], c.n3, row_ptr, nbr_j, S->dR, S->d_Z, S->xa[0], S->ev1[0]);
      S->prof.end(st);
    } else {
      if (!(fuse && l > 0)) { S->prof.begin(kPProj, st); launch_proj_fwd(st, L, S->x[l], nsend[l], S->qkv[l]); S->prof.end(st); }
      S->prof.begin(kPAttnFwd, st);
      attn_fwd_dispatch(S, st, L, nrecv[l], c.n3, row_ptr, nbr_j, S->dR, S->qkv[l], S->x[l], S->ev[l], S->xa[l], S->ev1[l]);
      S->prof.end(st);
    }
    S->prof.begin(kPPostFwd, st);
    const bool emit = fuse && l + 1 < kNumLayers;
    post_fwd_dispatch(st, L, nrecv[l], S->xa[l], S->ev1[l], S->z1[l], S->x3[l], S->gate[l], S->x[l + 1], S->ev[l + 1],
                      emit ? &M.layer[l + 1] : nullptr, emit ? S->qkv[l + 1] : nullptr, S->d_flag + 1);
    S->prof.end(st);
  }
  S->prof.begin(kPHeads, st);
  heads_fwd_dispatch(st, M, c.n0, S->d_Z, S->x[kNumLayers], S->ze, S->zq, S->zh, S->e_nn, S->q_raw, S->hv, S->d_flag + 1);
  S->prof.end(st);
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// reverse pass from the cotangents of the heads (gq_raw, gh on the owned atoms; d/d e_nn = 1) to the forces, added into F
int fused_backward(so3lr_b200_system* S, cudaStream_t st, const Shells& c, float* F) {
  const ModelDev& M = S->mctx;
  const int* row_ptr = S->sr.row_ptr; const int* nbr_j = S->sr.nbr_j;
  const int npost[kNumLayers] = {c.n2, c.n1, c.n0};   // atoms whose layer-l outputs carry a cotangent
  const int nattn[kNumLayers] = {c.n3, c.n2, c.n1};   // atoms that receive a cotangent through layer l's attention
  S->prof.begin(kPHeads, st);
  heads_bwd_dispatch(st, M, c.n0, S->d_Z, S->ze, S->zq, S->zh, S->hv, S->ones, S->gq_raw, S->gh, S->g4, S->d_flag + 1);
  S->prof.end(st);
  float* gev2 = S->gev_a;
  float* gev_in = S->gev_b;
  fill(st, gev2, (size_t)c.n0 * kMTot, 0.f);
  for (int l = kNumLayers - 1; l >= 0; --l) {
    const LayerDev& L = M.layer[l];
    const bool fused_in = use_mma_dense() && l + 1 < kNumLayers;   // cotangent formed from the layer above inside the block
    S->prof.begin(kPPostBwd, st);
    post_bwd_dispatch(st, L, npost[l], S->xa[l], S->ev1[l], S->z1[l], S->x3[l], S->gate[l], S->g4, gev2, S->g_xa, S->gev1,
                      fused_in ? &M.layer[l + 1] : nullptr, S->g_qkv, S->d_flag + 1);
    S->prof.end(st);
    if (c.n3 > npost[l]) {   // atoms beyond the layer's receivers have no cotangent of their own (any of them can be a neighbour)
      fill(st, S->g_xa + (size_t)npost[l] * kF, (size_t)(c.n3 - npost[l]) * kF, 0.f);
      fill(st, S->gev1 + (size_t)npost[l] * kMTot, (size_t)(c.n3 - npost[l]) * kMTot, 0.f);
    }
    S->prof.begin(l == 0 ? kPLayer0Bwd : kPAttnBwd, st);
    if (l == 0 && S->sp.n_species > 0 && use_layer0_tables())
      launch_layer0_bwd_tab(st, S->sp, nattn[0], c.n3, c.n3, row_ptr, nbr_j, S->dR, S->d_Z, S->g_xa, S->gev1, S->GV, F, S->vir());
    else
      attn_bwd_dispatch(S, st, L, nattn[l], c.n3, row_ptr, nbr_j, S->dR, S->qkv[l], S->ev[l], S->g_xa, S->gev1, S->g_qkv, gev_in, F, l == 0 ? 1 : 0,
                        S->vir());
    S->prof.end(st);
    if (l > 0) {
      if (!use_mma_dense()) {
        // dL/dx_in = g_xa (skip connection) + projections^T
        SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->g4, S->g_xa, (size_t)nattn[l] * kF * sizeof(float), cudaMemcpyDeviceToDevice, st));
        S->prof.begin(kPProjBwd, st); launch_proj_bwd(st, L, S->g_qkv, nattn[l], S->g4, 1); S->prof.end(st);
      }
      float* t = gev2; gev2 = gev_in; gev_in = t;
    }
  }
  if (S->vir()) reduce_virial(S, st, c.n0);
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// single-device evaluation: all shells coincide; long-range pairs from the ordered (or half-weight) list with scatter
int evaluate_fused(so3lr_b200_system* S, cudaStream_t st, const float* R, float* F) {
  const int n = S->n;
  const Shells c{n, n, n, n};
  int rc = fused_forward(S, st, R, c, false, F);
  if (rc) return rc;
  fill(st, S->e_coul, n, 0.f); fill(st, S->e_disp, n, 0.f); fill(st, S->gq, n, 0.f); fill(st, S->gh, n, 0.f);
  launch_charge_conserve(st, S->n_graphs, S->d_graph_start, S->q_raw, S->d_total_charge, S->hv, S->q, S->h, S->n, S->red_scratch);
  S->prof.begin(kPPairLr, st);
  launch_pair_lr_packed(st, S->lr, S->cell, n, S->lrl.row_ptr, S->lrl.nbr_j, S->d_Z, R, S->q, S->h, S->pair_pack, F, S->gq, S->gh, S->e_coul,
                        S->e_disp, S->vir());
  S->prof.end(st);
  if (S->ks.mode) {
    S->prof.begin(kPKspace, st);
    rc = launch_ewald(st, S->ks, S->cell, n, R, S->q, S->d_total_charge, S->e_coul, S->gq, F, S->vir(), 1.f);
    S->prof.end(st);
    if (rc) return rc;
  }
  { combine_energy_kernel<<<(n + 255) / 256, 256, 0, st>>>(n, S->e_nn, S->e_zbl, S->e_coul, S->e_disp, S->e_atom); count_launch(); }
  launch_charge_conserve_bwd(st, S->n_graphs, S->d_graph_start, S->gq, S->gq_raw, S->n, S->red_scratch);
  return fused_backward(S, st, c, F);
}

// Charge and spin embeddings (feature_embeddings_1 / _2 of the parameter tree; inputs total_charge / num_unpaired_electrons of
// so3lr/base_calculator.py:57-86).  Per graph and embedding: y_i = softplus(<query[Z_i], key[psi < 0]> / sqrt(128)),
// a_i = psi * y_i / sum_graph y, e_i = a_i * value[psi < 0], output e + W1^T silu(W0^T silu(e)) (bias-free residual block).
// They depend on the element, the graph's composition and psi only -- not on positions -- so they are evaluated once per
// context, on the host in double precision, and folded into the initial features: x0 = (embed[Z] + charge + spin) / sqrt(3).
// `out` receives per (graph, element) rows [n_graphs][119][128], already divided by sqrt(3); returns false when every psi is 0.
bool charge_spin_rows(const ModelDev& M, int n, const int32_t* Z, int n_graphs, const std::vector<int>& gs, const float* total_charge,
                      const float* num_unpaired, std::vector<float>* out, int* status) {
  bool any = false;
  for (int g = 0; g < n_graphs; ++g) any |= (total_charge && total_charge[g] != 0.f) || (num_unpaired && num_unpaired[g] != 0.f);
  *status = kOk;
  if (!any) return false;
  out->assign((size_t)n_graphs * kZEmbed * kF, 0.f);
  std::vector<float> q((size_t)kZEmbed * kF), k(2 * kF), v(2 * kF), r0((size_t)kF * kF), r1((size_t)kF * kF);
  auto silu = [](double x) { return x / (1.0 + std::exp(-x)); };
  for (int e = 0; e < 2; ++e) {
    const float* psi_all = e == 0 ? total_charge : num_unpaired;
    if (!psi_all) continue;
    bool used = false;
    for (int g = 0; g < n_graphs; ++g) used |= psi_all[g] != 0.f;
    if (!used) continue;
    if (cudaMemcpy(q.data(), M.cs_embed_q[e], q.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(k.data(), M.cs_embed_k[e], k.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(v.data(), M.cs_embed_v[e], v.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(r0.data(), M.cs_res0[e], r0.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(r1.data(), M.cs_res1[e], r1.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) {
      *status = kCudaError;
      return false;
    }
    for (int g = 0; g < n_graphs; ++g) {
      const double psi = psi_all[g];
      if (psi == 0.0) continue;
      const int idx = psi < 0.0 ? 1 : 0;
      double y[kZEmbed];
      bool present[kZEmbed] = {};
      for (int a = gs[g]; a < gs[g + 1]; ++a) present[Z[a]] = true;
      for (int z = 0; z < kZEmbed; ++z) {
        if (!present[z]) continue;
        double d = 0.0;
        for (int c = 0; c < kF; ++c) d += (double)q[(size_t)z * kF + c] * (double)k[idx * kF + c];
        d /= std::sqrt((double)kF);
        y[z] = d > 30.0 ? d : std::log1p(std::exp(d));
      }
      double den = 0.0;
      for (int a = gs[g]; a < gs[g + 1]; ++a) den += y[Z[a]];
      for (int z = 0; z < kZEmbed; ++z) {
        if (!present[z]) continue;
        const double a = psi * y[z] / den;
        double ev[kF], t0[kF], t1[kF];
        for (int c = 0; c < kF; ++c) ev[c] = a * (double)v[idx * kF + c];
        for (int o = 0; o < kF; ++o) {
          double acc = 0.0;
          for (int c = 0; c < kF; ++c) acc += silu(ev[c]) * (double)r0[(size_t)c * kF + o];
          t0[o] = acc;
        }
        for (int o = 0; o < kF; ++o) {
          double acc = 0.0;
          for (int c = 0; c < kF; ++c) acc += silu(t0[c]) * (double)r1[(size_t)c * kF + o];
          t1[o] = acc;
        }
        float* row = out->data() + ((size_t)g * kZEmbed + z) * kF;
        for (int c = 0; c < kF; ++c) row[c] += (float)((ev[c] + t1[c]) / std::sqrt(3.0));
      }
    }
  }
  return true;
}

}  // namespace

extern "C" {

SO3LR_B200_API int so3lr_b200_version(void) { return 100; }

SO3LR_B200_API const char* so3lr_b200_status_string(int status) {
  switch (status) {
    case kOk: return "ok";
    case kInvalidArgument: return "invalid argument";
    case kCudaError: return "CUDA error";
    case kOverflow: return "neighbor list overflow";
    case kNotFinite: return "non-finite positions";
    case kTooLarge: return "system too large";
    default: return "unknown status";
  }
}

SO3LR_B200_API int so3lr_b200_model_create(const float* blob_host, size_t n_floats, int device, so3lr_b200_model** out) {
  if (!blob_host || !out) return kInvalidArgument;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
    std::fprintf(stderr, "so3lr_b200: no CUDA device available; this library has no CPU path\n");
    return kCudaError;
  }
  if (device < 0 || device >= count) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(device));
  so3lr_b200_model* m = new so3lr_b200_model();
  m->device = device;
  int rc = build_model(blob_host, n_floats, &m->M, &m->owned);
  if (rc == kOk) rc = configure_atom_kernels();
  if (rc == kOk) rc = configure_attention_kernels();
  if (rc == kOk) rc = configure_attention_sym_kernels();
  if (rc == kOk) rc = configure_attention_mma_kernels();
  if (rc == kOk) rc = configure_attention_tc_kernels();
  if (rc == kOk) rc = configure_atom_mma_kernels();
  if (rc == kOk) rc = configure_dense_tc_kernels();
  if (rc != kOk) { so3lr_b200_model_destroy(m); return rc; }
  *out = m;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_model_destroy(so3lr_b200_model* m) {
  if (!m) return kOk;
  cudaSetDevice(m->device);
  for (void* p : m->owned) cudaFree(p);
  delete m;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_create(so3lr_b200_model* model, int n_atoms, const int32_t* Z, int n_graphs, const int32_t* graph_start,
                             const float* total_charge, const float* num_unpaired, const float* cell9,
                             const so3lr_b200_options* options, so3lr_b200_system** out) {
  if (!model || !Z || !out || !options || n_atoms <= 0 || n_graphs <= 0) return kInvalidArgument;
  if (n_atoms > 64 * 1000 * 1000) return kTooLarge;
  if (n_graphs > 1 && !graph_start) return kInvalidArgument;
  if (int bad = first_unsupported_element(Z, n_atoms)) {
    std::fprintf(stderr, "so3lr_b200: atomic number %d is outside the supported range 1..%d (free-atom polarisabilities and C6 "
                         "coefficients of the dispersion term are tabulated for these elements only)\n", bad == -1 ? 0 : bad, kMaxZ);
    return kInvalidArgument;
  }
  SO3LR_CUDA_CHECK(cudaSetDevice(model->device));
  so3lr_b200_system* S = new so3lr_b200_system();
  tl_launch_counter = &S->n_launches;
  S->model = model; S->mctx = model->M; S->n = n_atoms; S->n_cap = n_atoms; S->n_graphs = n_graphs; S->opt = *options;
  int rc = make_cell(cell9, &S->cell);
  if (rc) { delete S; return rc; }
  // long-range constants
  LrParams& P = S->lr;
  P.has_cutoff = options->cutoff_lr > 0.f;
  P.rc = options->cutoff_lr;
  P.cuton = kCutonFraction * options->cutoff_lr;
  P.has_damping = options->damping > 0.f;
  P.disp_on = options->cutoff_lr - options->damping;
  P.pair_factor = options->lr_both_directions ? 0.5f : 1.f;
  P.k_alpha = 0.f;
  set_coulomb_shift(P);
  const int n = n_atoms;
  Pool& A = S->pool;
  S->d_Z0 = A.get<int>(n); S->d_Zs = A.get<int>(n); S->d_Z = S->d_Z0; S->d_perm = A.get<int>(n);
  S->d_Rs = A.get<float>((size_t)n * 3); S->F_s = A.get<float>((size_t)n * 3);
  S->u_e_atom = A.get<float>(n); S->u_q = A.get<float>(n); S->u_h = A.get<float>(n);
  S->u_zbl = A.get<float>(n); S->u_coul = A.get<float>(n); S->u_disp = A.get<float>(n);
  S->d_seg = A.get<int>(n); S->d_graph_start = A.get<int>(n_graphs + 1);
  S->d_total_charge = A.get<float>(n_graphs);
  std::vector<int> gs(n_graphs + 1), seg(n);
  if (graph_start) { for (int g = 0; g <= n_graphs; ++g) gs[g] = graph_start[g]; }
  else { gs[0] = 0; gs[1] = n; }
  if (gs[0] != 0 || gs[n_graphs] != n) { A.release(); delete S; return kInvalidArgument; }
  for (int g = 0; g < n_graphs; ++g) {
    if (gs[g + 1] < gs[g]) { A.release(); delete S; return kInvalidArgument; }
    for (int a = gs[g]; a < gs[g + 1]; ++a) seg[a] = g;
  }
  std::vector<float> tq(n_graphs, 0.f);
  if (total_charge) for (int g = 0; g < n_graphs; ++g) tq[g] = total_charge[g];
  S->d_Rref = A.get<float>((size_t)n * 3); S->d_flag = A.get<int>(4);
  S->d_rowptr_g = A.get<int>((size_t)n + 1); S->d_rowptr_lr_g = A.get<int>((size_t)n + 1);
  for (int l = 0; l <= kNumLayers; ++l) { S->x[l] = A.get<float>((size_t)n * kF); S->ev[l] = A.get<float>((size_t)n * kMTot); }
  for (int l = 0; l < kNumLayers; ++l) {
    S->qkv[l] = A.get<float>((size_t)n * kProj); S->xa[l] = A.get<float>((size_t)n * kF); S->ev1[l] = A.get<float>((size_t)n * kMTot);
    S->z1[l] = A.get<float>((size_t)n * kF); S->x3[l] = A.get<float>((size_t)n * kF); S->gate[l] = A.get<float>((size_t)n * 4);
  }
  S->ze = A.get<float>((size_t)n * kF); S->zq = A.get<float>((size_t)n * kF); S->zh = A.get<float>((size_t)n * 64);
  S->e_nn = A.get<float>(n); S->q_raw = A.get<float>(n); S->hv = A.get<float>(n); S->q = A.get<float>(n); S->h = A.get<float>(n);
  S->e_atom = A.get<float>(n); S->e_zbl = A.get<float>(n); S->e_coul = A.get<float>(n); S->e_disp = A.get<float>(n);
  S->gq = A.get<float>(n); S->gh = A.get<float>(n); S->gq_raw = A.get<float>(n); S->ones = A.get<float>(n);
  S->pair_pack = A.get<float>((size_t)n * 12);
  S->g4 = A.get<float>((size_t)n * kF); S->g_xa = A.get<float>((size_t)n * kF);
  S->gev_a = A.get<float>((size_t)n * kMTot); S->gev_b = A.get<float>((size_t)n * kMTot); S->gev1 = A.get<float>((size_t)n * kMTot);
  S->g_qkv = A.get<float>((size_t)n * kProj);
  S->F_int = A.get<float>((size_t)n * 3);
  S->GV = A.get<float>((size_t)n * 4 * kMaxTabSpecies);
  S->d_energy = A.get<double>(n_graphs); S->d_dipole = A.get<float>((size_t)n_graphs * 3);
  S->red_scratch = A.get<double>(4 * 296);
  S->d_Rstage = A.get<float>((size_t)n * 3);
  if (A.status != kOk) { A.release(); delete S; return A.status; }
  bool ok = cudaMemcpy(S->d_Z0, Z, (size_t)n * sizeof(int), cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemcpy(S->d_seg, seg.data(), (size_t)n * sizeof(int), cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemcpy(S->d_graph_start, gs.data(), (size_t)(n_graphs + 1) * sizeof(int), cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemcpy(S->d_total_charge, tq.data(), (size_t)n_graphs * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemset(S->ev[0], 0, (size_t)n * kMTot * sizeof(float)) == cudaSuccess &&
            cudaMallocHost((void**)&S->h_flag, 2 * sizeof(int)) == cudaSuccess &&
            cudaMallocHost((void**)&S->h_R, (size_t)n * 3 * sizeof(float)) == cudaSuccess &&
            cudaMallocHost((void**)&S->h_F, (size_t)n * 3 * sizeof(float)) == cudaSuccess &&
            cudaMallocHost((void**)&S->h_q, (size_t)n * sizeof(float)) == cudaSuccess &&
            cudaMallocHost((void**)&S->h_h, (size_t)n * sizeof(float)) == cudaSuccess &&
            cudaMallocHost((void**)&S->h_dip, (size_t)n_graphs * 3 * sizeof(float)) == cudaSuccess &&
            cudaMallocHost((void**)&S->h_E, (size_t)n_graphs * sizeof(double)) == cudaSuccess &&
            cudaStreamCreateWithFlags(&S->own_stream, cudaStreamNonBlocking) == cudaSuccess;
  if (!ok) { so3lr_b200_system_destroy(S); return kCudaError; }
  fill(nullptr, S->ones, n, 1.f);
  {
    // charge / spin embeddings: per-element table for one structure, per-atom rows for a batch
    std::vector<float> rows;
    int cs_status = kOk;
    const bool charged = charge_spin_rows(model->M, n, Z, n_graphs, gs, total_charge, num_unpaired, &rows, &cs_status);
    if (cs_status != kOk) { so3lr_b200_system_destroy(S); return cs_status; }
    if (charged) {
      std::vector<float> base((size_t)kZEmbed * kF);
      if (cudaMemcpy(base.data(), model->M.embed_z, base.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) {
        so3lr_b200_system_destroy(S); return kCudaError;
      }
      if (n_graphs == 1) {
        for (size_t k = 0; k < base.size(); ++k) base[k] += rows[k];
        float* d = S->pool.get<float>(base.size());
        if (!d || cudaMemcpy(d, base.data(), base.size() * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) {
          so3lr_b200_system_destroy(S); return kCudaError;
        }
        S->mctx.embed_z = d;
      } else {
        std::vector<float> x0((size_t)n * kF);
        for (int a = 0; a < n; ++a)
          for (int c = 0; c < kF; ++c)
            x0[(size_t)a * kF + c] = base[(size_t)Z[a] * kF + c] + rows[((size_t)seg[a] * kZEmbed + Z[a]) * kF + c];
        S->x0_atom = S->pool.get<float>(x0.size());
        if (!S->x0_atom || cudaMemcpy(S->x0_atom, x0.data(), x0.size() * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) {
          so3lr_b200_system_destroy(S); return kCudaError;
        }
      }
    }
  }
  // a batch with per-atom initial features cannot use the per-element-pair tables of the first layer
  if (!S->x0_atom && species_tables_build(nullptr, S->mctx, Z, n, &S->sp) != kOk) { so3lr_b200_system_destroy(S); return kCudaError; }
  cudaDeviceSynchronize();
  S->nws = nlist_workspace_create();
  *out = S;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_destroy(so3lr_b200_system* S) {
  if (!S) return kOk;
  if (tl_launch_counter == &S->n_launches) tl_launch_counter = nullptr;
  cudaSetDevice(S->model->device);
  cudaDeviceSynchronize();
  tc_debug_print();
  dense_debug_print();
  drop_step_graph(S);
  S->pool.release();
  kspace_free(&S->ks);
  species_tables_free(&S->sp);
  S->prof.destroy();
  nlist_workspace_destroy(S->nws);
  for (NeighborListDev* L : {&S->sr, &S->lrl}) { cudaFree(L->row_ptr); cudaFree(L->nbr_j); cudaFree(L->edge_i); }
  cudaFree(S->dR);
  valid_edges_free(&S->ve);
  if (S->h_flag) cudaFreeHost(S->h_flag);
  if (S->h_flag2) cudaFreeHost(S->h_flag2);
  for (int k = 0; k < 2; ++k) if (S->flag_event[k]) cudaEventDestroy(S->flag_event[k]);
  if (S->h_box) cudaFreeHost(S->h_box);
  if (S->h_R) cudaFreeHost(S->h_R);
  if (S->h_F) cudaFreeHost(S->h_F);
  if (S->h_q) cudaFreeHost(S->h_q);
  if (S->h_h) cudaFreeHost(S->h_h);
  if (S->h_dip) cudaFreeHost(S->h_dip);
  if (S->h_E) cudaFreeHost(S->h_E);
  if (S->own_stream) cudaStreamDestroy(S->own_stream);
  delete S;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_set_cell(so3lr_b200_system* S, const float* cell9) {
  if (!S) return kInvalidArgument;
  int rc = make_cell(cell9, &S->cell);
  if (rc) return rc;
  S->have_lists = false;
  S->virial_fresh = false;
  drop_step_graph(S);
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_set_kspace(so3lr_b200_system* S, int mode, float smearing, int n1, int n2, int n3) {
  if (!S || mode < 0 || mode > 2) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  SO3LR_CUDA_CHECK(cudaDeviceSynchronize());
  S->virial_fresh = false;
  drop_step_graph(S);
  if (mode == 0) {
    kspace_free(&S->ks);
    S->lr.k_alpha = 0.f;
    set_coulomb_shift(S->lr);
    return kOk;
  }
  // one periodic structure whose pair sum is cut off: the split needs a short-ranged pair part
  if (!S->cell.periodic || S->n_graphs != 1 || !S->lr.has_cutoff || !(smearing > 0.f)) return kInvalidArgument;
  int rc = kspace_setup(&S->ks, S->n_cap, mode, smearing, n1, n2, n3);
  if (rc) {      // the context falls back to the plain truncated pair sum, consistently
    S->lr.k_alpha = 0.f;
    set_coulomb_shift(S->lr);
    return rc;
  }
  S->lr.k_alpha = (float)(1.0 / (std::sqrt(2.0) * (double)smearing));
  set_coulomb_shift(S->lr);
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_defer_skin_test(so3lr_b200_system* S, int enable, float margin) {
  if (!S || !(margin >= 0.f)) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  if (enable && !S->h_flag2) {
    SO3LR_CUDA_CHECK(cudaMallocHost((void**)&S->h_flag2, 4 * sizeof(int)));
    for (int k = 0; k < 2; ++k) SO3LR_CUDA_CHECK(cudaEventCreateWithFlags(&S->flag_event[k], cudaEventDisableTiming));
  }
  S->deferred_skin = enable != 0;
  S->skin_margin = margin;
  S->flag_pending[0] = S->flag_pending[1] = false;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_rescale_cell(so3lr_b200_system* S, const float* cell9) {
  if (!S || !cell9 || !S->cell.periodic) return kInvalidArgument;
  S->virial_fresh = false;
  drop_step_graph(S);
  return make_cell(cell9, &S->cell);
}

static int prepare_lists(so3lr_b200_system* S, cudaStream_t st, const float* R, bool allow_sort = true) {
  bool rebuild = !S->have_lists;
  if (!rebuild) {
    if (S->opt.skin <= 0.f) rebuild = true;
    else if (S->deferred_skin) {
      // this step's test goes to one pinned slot; the decision uses the other slot, written during the previous step
      const int cur = S->flag_slot, prev = cur ^ 1;
      float thr = 0.5f * S->opt.skin - S->skin_margin;
      if (thr < 0.f) thr = 0.f;
      SO3LR_CUDA_CHECK(cudaMemsetAsync(S->d_flag, 0, sizeof(int), st));
      { moved_kernel<<<(S->n + 255) / 256, 256, 0, st>>>(S->n, R, S->d_Rref, thr * thr, S->d_flag); count_launch(); }
      SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->h_flag2 + 2 * cur, S->d_flag, 2 * sizeof(int), cudaMemcpyDeviceToHost, st));
      SO3LR_CUDA_CHECK(cudaEventRecord(S->flag_event[cur], st));
      S->flag_pending[cur] = true;
      S->flag_slot = prev;
      if (S->flag_pending[prev]) {
        SO3LR_CUDA_CHECK(cudaEventSynchronize(S->flag_event[prev]));    // a whole step old: already complete in steady state
        S->flag_pending[prev] = false;
        const int* f = S->h_flag2 + 2 * prev;
        if (f[1]) {
          std::fprintf(stderr, "so3lr_b200: a bounded wait on the tensor-core pipeline ran out in an earlier evaluation\n");
          return kCudaError;
        }
        if (f[0] & 2) return kNotFinite;
        rebuild = f[0] != 0;
      }
      if (rebuild) { S->flag_pending[0] = S->flag_pending[1] = false; }
    } else {
      float thr = 0.5f * S->opt.skin;
      SO3LR_CUDA_CHECK(cudaMemsetAsync(S->d_flag, 0, sizeof(int), st));
      { moved_kernel<<<(S->n + 255) / 256, 256, 0, st>>>(S->n, R, S->d_Rref, thr * thr, S->d_flag); count_launch(); }
      SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->h_flag, S->d_flag, 2 * sizeof(int), cudaMemcpyDeviceToHost, st));
      SO3LR_CUDA_CHECK(cudaStreamSynchronize(st));
      if (S->h_flag[1]) {
        std::fprintf(stderr, "so3lr_b200: a bounded wait on the tensor-core pipeline ran out in an earlier evaluation\n");
        return kCudaError;
      }
      if (*S->h_flag & 2) return kNotFinite;
      rebuild = *S->h_flag != 0;
    }
  }
  if (rebuild) {
    S->prof.begin(kPNlist, st);
    int rc = rebuild_lists(S, st, R, allow_sort);
    S->prof.end(st);
    return rc;
  }
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_compute(so3lr_b200_system* S, void* stream, const float* R, float* F, float* e_atom, double* energy,
                              float* charges, float* hirshfeld, float* dipole) {
  if (!S || !R) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rebuilds_before = S->n_rebuilds;
  int rc = prepare_lists(S, st, R);
  if (rc) return rc;
  float* Fout = F ? F : S->F_int;
  const int n = S->n;
  // everything between the list update and the copies of the optional outputs
  auto evaluate = [&]() -> int {
    const float* R_eval = R;
    if (S->sorted) {
      { gather_positions_kernel<<<(n + 255) / 256, 256, 0, st>>>(n, S->d_perm, R, S->d_Rs); count_launch(); }
      R_eval = S->d_Rs;
    }
    int rce = evaluate_fused(S, st, R_eval, S->sorted ? S->F_s : Fout);
    if (rce) return rce;
    launch_graph_reduce(st, S->n_graphs, S->d_graph_start, S->e_atom, S->q, R_eval, S->d_energy, S->d_dipole, S->n, S->red_scratch);
    if (S->sorted) {
      UnsortArgs A{{S->e_atom, S->q, S->h, S->e_zbl, S->e_coul, S->e_disp, nullptr},
                   {S->u_e_atom, S->u_q, S->u_h, S->u_zbl, S->u_coul, S->u_disp, nullptr}};
      { unsort_kernel<<<(n + 255) / 256, 256, 0, st>>>(n, S->d_perm, S->F_s, Fout, A); count_launch(); }
    }
    return kOk;
  };
  so3lr_b200_system::StepGraph& G = S->step_graph;
  // lists unchanged by this call, a stream that can be captured, nothing in the evaluation that allocates or reads back
  const bool graph_ok = step_graphs_enabled() && !G.broken && n <= kStepGraphMaxAtoms && S->opt.skin > 0.f && !S->prof.on && !S->ks.mode &&
                        S->n_rebuilds == rebuilds_before && st != nullptr && st != cudaStreamLegacy && st != cudaStreamPerThread;
  if (graph_ok && G.exec && G.R == R && G.F == Fout && G.stamp == S->n_rebuilds && G.virial == S->want_virial) {
    SO3LR_CUDA_CHECK(cudaGraphLaunch(G.exec, st));
    S->n_launches += G.launches;
    ++G.replays;
    if (S->want_virial) S->virial_fresh = true;
  } else if (graph_ok && G.last_R == R && G.last_F == Fout && G.last_stamp == S->n_rebuilds) {
    if (G.exec) { cudaGraphExecDestroy(G.exec); G.exec = nullptr; }
    // a stream that its owner is capturing already (a runtime that records its own graphs around the call) takes plain launches
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
      cudaGetLastError();
      G.broken = true;
      rc = evaluate();
      if (rc) return rc;
    } else if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
      cudaGetLastError();
      G.broken = true;
      rc = evaluate();
      if (rc) return rc;
    } else {
      const int64_t l0 = S->n_launches;
      rc = evaluate();
      cudaGraph_t graph = nullptr;
      const cudaError_t ce = cudaStreamEndCapture(st, &graph);
      if (rc || ce != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        G.broken = true;
        if (rc) return rc;
        rc = evaluate();           // nothing ran during the failed capture
        if (rc) return rc;
      } else {
        const cudaError_t ci = cudaGraphInstantiate(&G.exec, graph, 0);
        cudaGraphDestroy(graph);
        if (ci != cudaSuccess) {
          cudaGetLastError();
          G.exec = nullptr; G.broken = true;
          rc = evaluate();
          if (rc) return rc;
        } else {
          G.R = R; G.F = Fout; G.stamp = S->n_rebuilds; G.virial = S->want_virial; G.launches = S->n_launches - l0;
          SO3LR_CUDA_CHECK(cudaGraphLaunch(G.exec, st));
        }
      }
    }
  } else {
    rc = evaluate();
    if (rc) return rc;
  }
  G.last_R = R; G.last_F = Fout; G.last_stamp = S->n_rebuilds;
  if (e_atom) SO3LR_CUDA_CHECK(cudaMemcpyAsync(e_atom, S->o_e_atom, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, st));
  if (energy) SO3LR_CUDA_CHECK(cudaMemcpyAsync(energy, S->d_energy, (size_t)S->n_graphs * sizeof(double), cudaMemcpyDeviceToDevice, st));
  if (charges) SO3LR_CUDA_CHECK(cudaMemcpyAsync(charges, S->o_q, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, st));
  if (hirshfeld) SO3LR_CUDA_CHECK(cudaMemcpyAsync(hirshfeld, S->o_h, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, st));
  if (dipole) SO3LR_CUDA_CHECK(cudaMemcpyAsync(dipole, S->d_dipole, (size_t)S->n_graphs * 3 * sizeof(float), cudaMemcpyDeviceToDevice, st));
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_graph_replays(so3lr_b200_system* S, int64_t* n_replays) {
  if (!S || !n_replays) return kInvalidArgument;
  *n_replays = S->step_graph.replays;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_compute_host(so3lr_b200_system* S, const float* R_host, float* F_host, double* E_host, float* q_host,
                                   float* h_host, float* dip_host) {
  if (!S || !R_host) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = S->own_stream;
  const int n = S->n;
  std::memcpy(S->h_R, R_host, (size_t)n * 3 * sizeof(float));
  SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->d_Rstage, S->h_R, (size_t)n * 3 * sizeof(float), cudaMemcpyHostToDevice, st));
  int rc = so3lr_b200_system_compute(S, st, S->d_Rstage, S->F_int, nullptr, nullptr, nullptr, nullptr, nullptr);
  if (rc) return rc;
  if (F_host) SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->h_F, S->F_int, (size_t)n * 3 * sizeof(float), cudaMemcpyDeviceToHost, st));
  if (E_host) SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->h_E, S->d_energy, (size_t)S->n_graphs * sizeof(double), cudaMemcpyDeviceToHost, st));
  if (q_host) SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->h_q, S->o_q, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost, st));
  if (h_host) SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->h_h, S->o_h, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost, st));
  if (dip_host) SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->h_dip, S->d_dipole, (size_t)S->n_graphs * 3 * sizeof(float), cudaMemcpyDeviceToHost, st));
  SO3LR_CUDA_CHECK(cudaStreamSynchronize(st));
  if (F_host) std::memcpy(F_host, S->h_F, (size_t)n * 3 * sizeof(float));
  if (E_host) std::memcpy(E_host, S->h_E, (size_t)S->n_graphs * sizeof(double));
  if (q_host) std::memcpy(q_host, S->h_q, (size_t)n * sizeof(float));
  if (h_host) std::memcpy(h_host, S->h_h, (size_t)n * sizeof(float));
  if (dip_host) std::memcpy(dip_host, S->h_dip, (size_t)S->n_graphs * 3 * sizeof(float));
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_aux(so3lr_b200_system* S, const float** zbl, const float** coul, const float** disp) {
  if (!S) return kInvalidArgument;
  if (zbl) *zbl = S->o_zbl ? S->o_zbl : S->e_zbl;
  if (coul) *coul = S->o_coul ? S->o_coul : S->e_coul;
  if (disp) *disp = S->o_disp ? S->o_disp : S->e_disp;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_stats(so3lr_b200_system* S, int64_t* n_rebuilds, int64_t* n_edges, int64_t* n_pairs, int64_t* n_launches) {
  if (!S) return kInvalidArgument;
  if (n_rebuilds) *n_rebuilds = S->n_rebuilds;
  if (n_edges) *n_edges = S->sr.count;
  if (n_pairs) *n_pairs = S->lrl.count;
  if (n_launches) *n_launches = S->n_launches;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_pack_rows(void* stream, int n_arrays, const float* const* arrays_dev, const int* widths, const int64_t* idx_dev,
                                        int64_t n_rows, float* buf_dev) {
  return so3lr::pack_rows(stream, n_arrays, const_cast<float* const*>(arrays_dev), widths, idx_dev, n_rows, buf_dev, false);
}
SO3LR_B200_API int so3lr_b200_unpack_rows(void* stream, int n_arrays, float* const* arrays_dev, const int* widths, const int64_t* idx_dev,
                                          int64_t n_rows, const float* buf_dev) {
  return so3lr::pack_rows(stream, n_arrays, arrays_dev, widths, idx_dev, n_rows, const_cast<float*>(buf_dev), true);
}

SO3LR_B200_API int so3lr_b200_system_valid_edges(so3lr_b200_system* S, int64_t* n_valid) {
  if (!S || !n_valid) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  *n_valid = 0;
  if (!S->ve.row_ptr || S->ve.n_rows <= 0) return kOk;
  int v = 0;
  SO3LR_CUDA_CHECK(cudaDeviceSynchronize());
  SO3LR_CUDA_CHECK(cudaMemcpy(&v, S->ve.row_ptr + S->ve.n_rows, sizeof(int), cudaMemcpyDeviceToHost));
  *n_valid = v;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_export_list(so3lr_b200_system* S, void* stream, const float* R, int which, int32_t* idx, int64_t capacity,
                                  int64_t* count_host, int* overflow_host) {
  if (!S || !R || !idx || capacity <= 0) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  S->have_lists = false;
  int rc = prepare_lists(S, st, R, false);   // lists in the caller's atom order
  if (rc) return rc;
  S->have_lists = false;                      // the next evaluation rebuilds them in its own (sorted) order
  const NeighborListDev& L = which == 0 ? S->sr : S->lrl;
  long long cnt = L.count < capacity ? L.count : capacity;
  { export_list_kernel<<<(unsigned)((capacity + 255) / 256), 256, 0, st>>>(S->n, cnt, capacity, L.edge_i, L.nbr_j, idx); count_launch(); }
  SO3LR_CUDA_CHECK(cudaStreamSynchronize(st));
  if (count_host) *count_host = L.count;
  if (overflow_host) *overflow_host = L.count > capacity ? 1 : 0;
  return kOk;
}

static int graph_eval_impl(so3lr_b200_system* S, void* stream, int64_t n_edges, const int32_t* idx_i, const int32_t* idx_j,
                           const float* edges, int64_t n_pairs, const int32_t* idx_i_lr, const int32_t* idx_j_lr,
                           const float* edges_lr, const float* g_e_atom, float* e_atom, float* g_edges, float* g_edges_lr,
                           float* charges, float* hirshfeld, const float* positions, float* g_positions, float* strain6) {
  if (!S || !idx_i || !idx_j || !edges || !g_edges || n_edges < 0 || n_pairs < 0) return kInvalidArgument;
  if (n_pairs > 0 && (!idx_i_lr || !idx_j_lr || !edges_lr || !g_edges_lr)) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int n = S->n;
  // graph-level lists are in the caller's atom order
  S->d_Z = S->d_Z0; S->sorted = false; S->have_lists = false;
  S->o_e_atom = S->e_atom; S->o_q = S->q; S->o_h = S->h; S->o_zbl = S->e_zbl; S->o_coul = S->e_coul; S->o_disp = S->e_disp;
  { row_ptr_from_sorted_kernel<<<(n + 1 + 255) / 256, 256, 0, st>>>(n, n_edges, idx_i, S->d_rowptr_g); count_launch(); }
  { row_ptr_from_sorted_kernel<<<(n + 1 + 255) / 256, 256, 0, st>>>(n, n_pairs, idx_i_lr, S->d_rowptr_lr_g); count_launch(); }
  int rc = evaluate_graph(S, st, S->d_rowptr_g, idx_j, idx_i, n_edges, S->d_rowptr_lr_g, idx_j_lr, edges, edges_lr, g_edges, g_edges_lr,
                          g_e_atom, positions, g_positions, strain6);
  if (rc) return rc;
  if (e_atom) SO3LR_CUDA_CHECK(cudaMemcpyAsync(e_atom, S->e_atom, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, st));
  if (charges) SO3LR_CUDA_CHECK(cudaMemcpyAsync(charges, S->q, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, st));
  if (hirshfeld) SO3LR_CUDA_CHECK(cudaMemcpyAsync(hirshfeld, S->h, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, st));
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_graph_eval(so3lr_b200_system* S, void* stream, int64_t n_edges, const int32_t* idx_i, const int32_t* idx_j,
                                 const float* edges, int64_t n_pairs, const int32_t* idx_i_lr, const int32_t* idx_j_lr,
                                 const float* edges_lr, const float* g_e_atom, float* e_atom, float* g_edges, float* g_edges_lr,
                                 float* charges, float* hirshfeld) {
  return graph_eval_impl(S, stream, n_edges, idx_i, idx_j, edges, n_pairs, idx_i_lr, idx_j_lr, edges_lr, g_e_atom, e_atom, g_edges, g_edges_lr,
                         charges, hirshfeld, nullptr, nullptr, nullptr);
}

SO3LR_B200_API int so3lr_b200_system_graph_eval_kspace(so3lr_b200_system* S, void* stream, int64_t n_edges, const int32_t* idx_i,
                                        const int32_t* idx_j, const float* edges, int64_t n_pairs, const int32_t* idx_i_lr,
                                        const int32_t* idx_j_lr, const float* edges_lr, const float* positions, float* e_atom,
                                        float* g_edges, float* g_edges_lr, float* g_positions, float* strain6, float* charges,
                                        float* hirshfeld) {
  if (!S || !S->ks.mode || !positions || !g_positions) return kInvalidArgument;
  return graph_eval_impl(S, stream, n_edges, idx_i, idx_j, edges, n_pairs, idx_i_lr, idx_j_lr, edges_lr, nullptr, e_atom, g_edges, g_edges_lr,
                         charges, hirshfeld, positions, g_positions, strain6);
}

SO3LR_B200_API int so3lr_b200_system_nve(so3lr_b200_system* S, void* stream, int n_steps, float dt, const float* masses, float* R, float* V,
                          float* F, double* energy) {
  if (!S || !masses || !R || !V || !F || n_steps < 0) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int n = S->n, blocks = (n + 255) / 256;
  for (int step = 0; step < n_steps; ++step) {
    S->prof.begin(kPMd, st);
    { vv_first_kernel<<<blocks, 256, 0, st>>>(n, dt, masses, R, V, F); count_launch(); }
    S->prof.end(st);
    int rc = so3lr_b200_system_compute(S, st, R, F, nullptr, step == n_steps - 1 ? energy : nullptr, nullptr, nullptr, nullptr);
    if (rc) return rc;
    S->prof.begin(kPMd, st);
    { vv_second_kernel<<<blocks, 256, 0, st>>>(n, dt, masses, V, F); count_launch(); }
    S->prof.end(st);
  }
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_enable_virial(so3lr_b200_system* S, int enable) {
  if (!S) return kInvalidArgument;
  if (S->n_graphs != 1) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  if (enable && !S->virial) {
    S->virial = S->pool.get<float>((size_t)S->n_cap * 6);
    S->virial_partials = S->pool.get<double>(6 * kVirialBlocks);
    S->virial_sum = S->pool.get<double>(9);
    if (S->pool.status != kOk) return S->pool.status;
  }
  S->want_virial = enable != 0;
  S->virial_fresh = false;
  drop_step_graph(S);
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_virial(so3lr_b200_system* S, void* stream, double* virial9_dev) {
  if (!S || !virial9_dev || !S->want_virial || !S->virial_sum) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  SO3LR_CUDA_CHECK(cudaMemcpyAsync(virial9_dev, S->virial_sum, 9 * sizeof(double), cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  return kOk;
}

SO3LR_B200_API int so3lr_b200_nhc_init(void* stream, double* chain) {
  if (!chain) return kInvalidArgument;
  tl_launch_counter = nullptr;
  nhc_init((cudaStream_t)stream, chain);
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

SO3LR_B200_API int so3lr_b200_nhc_half_steps(void* stream, double* chain, int chain_length, int chain_steps, int sy_steps, double dt,
                                             double tau, double kT, double dof, int n_half_steps, int fresh_scale,
                                             const double* ke_partials, int n_partials) {
  if (!chain || n_half_steps < 0 || (ke_partials && n_partials <= 0)) return kInvalidArgument;
  if (!nhc_settings_ok(chain_length, chain_steps, sy_steps, dt, tau, kT, dof)) return kInvalidArgument;
  tl_launch_counter = nullptr;
  nhc_half_steps((cudaStream_t)stream, chain, chain_length, chain_steps, sy_steps, dt, tau, kT, dof, n_half_steps, fresh_scale,
                 ke_partials, n_partials);
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_nvt(so3lr_b200_system* S, void* stream, int n_steps, float dt, double kT, double tau,
                                         int chain_length, int chain_steps, int sy_steps, const float* masses, float* R, float* V,
                                         float* F, double* chain, double* energy) {
  if (!S || !masses || !R || !V || !F || !chain || n_steps < 0) return kInvalidArgument;
  const int n = S->n;
  const double dof = 3.0 * (double)n;
  if (!nhc_settings_ok(chain_length, chain_steps, sy_steps, dt, tau, kT, dof)) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int blocks = (n + 255) / 256;
  if (!S->ke_partials) {
    S->ke_partials = S->pool.get<double>((size_t)(S->n_cap + 255) / 256);
    if (!S->ke_partials) return kCudaError;
  }
  if (n_steps == 0) return kOk;
  // the chain's first half step of step 0 works on the kinetic energy of the velocities as they are now
  S->prof.begin(kPMd, st);
  md_kinetic_partials(st, n, masses, V, S->ke_partials);
  nhc_half_steps(st, chain, chain_length, chain_steps, sy_steps, dt, tau, kT, dof, 1, 1, S->ke_partials, blocks);
  S->prof.end(st);
  for (int step = 0; step < n_steps; ++step) {
    S->prof.begin(kPMd, st);
    md_first_half(st, n, dt, masses, R, V, F, chain);
    S->prof.end(st);
    int rc = so3lr_b200_system_compute(S, st, R, F, nullptr, step == n_steps - 1 ? energy : nullptr, nullptr, nullptr, nullptr);
    if (rc) return rc;
    S->prof.begin(kPMd, st);
    md_second_half(st, n, dt, masses, V, F, S->ke_partials);
    // the second half step of this MD step and the first of the next act on the velocities back to back: one launch, and
    // their product is applied by the next step's first kernel
    nhc_half_steps(st, chain, chain_length, chain_steps, sy_steps, dt, tau, kT, dof, step == n_steps - 1 ? 1 : 2, 1, S->ke_partials,
                   blocks);
    if (step == n_steps - 1) md_apply_scale(st, n, V, chain);
    S->prof.end(st);
  }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

SO3LR_B200_API int so3lr_b200_npt_init(void* stream, double* state) {
  if (!state) return kInvalidArgument;
  tl_launch_counter = nullptr;
  npt_init((cudaStream_t)stream, state);
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// The two box/chain kernels of an NPT step for callers that move the atoms themselves (the decomposed driver): `virial9`
// and `kinetic_energy` (one double, eV; may be NULL in npt_pre to keep the chain's own value) are sums over all ranks.
static int npt_params_ok(int n_atoms, float dt, double kT, double pressure, double tau_t, double tau_b, int chain_length, int chain_steps,
                         int sy_steps, double V0) {
  return n_atoms > 0 && nhc_settings_ok(chain_length, chain_steps, sy_steps, dt, tau_t, kT, 3.0 * n_atoms) && tau_b > 0.0 &&
         std::isfinite(pressure) && V0 > 0.0;
}

SO3LR_B200_API int so3lr_b200_npt_pre(void* stream, double* state, int n_atoms, float dt, double kT, double pressure, double tau_t,
                                      double tau_b, int chain_length, int chain_steps, int sy_steps, double V0, const double* virial9,
                                      const double* kinetic_energy) {
  if (!state || !virial9 || !npt_params_ok(n_atoms, dt, kT, pressure, tau_t, tau_b, chain_length, chain_steps, sy_steps, V0))
    return kInvalidArgument;
  tl_launch_counter = nullptr;
  NptParams p{chain_length, chain_steps, sy_steps, n_atoms, (double)dt, kT, pressure, tau_t, tau_b, V0};
  npt_pre((cudaStream_t)stream, state, p, virial9, kinetic_energy, 1);
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

SO3LR_B200_API int so3lr_b200_npt_post(void* stream, double* state, int n_atoms, float dt, double kT, double pressure, double tau_t,
                                       double tau_b, int chain_length, int chain_steps, int sy_steps, double V0, const double* virial9,
                                       const double* kinetic_energy) {
  if (!state || !virial9 || !kinetic_energy ||
      !npt_params_ok(n_atoms, dt, kT, pressure, tau_t, tau_b, chain_length, chain_steps, sy_steps, V0))
    return kInvalidArgument;
  tl_launch_counter = nullptr;
  NptParams p{chain_length, chain_steps, sy_steps, n_atoms, (double)dt, kT, pressure, tau_t, tau_b, V0};
  npt_post((cudaStream_t)stream, state, p, virial9, kinetic_energy, 1);
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_npt(so3lr_b200_system* S, void* stream, int n_steps, float dt, double kT, double pressure,
                                         double tau_t, double tau_b, int chain_length, int chain_steps, int sy_steps,
                                         const float* masses, float* R, float* V, float* F, double* state, const float* cell0_9,
                                         float* cell_out9, double* energy) {
  if (!S || !masses || !R || !V || !F || !state || !cell0_9 || n_steps < 0) return kInvalidArgument;
  if (!S->cell.periodic || S->n_graphs != 1 || !S->want_virial) return kInvalidArgument;
  const int n = S->n;
  if (!nhc_settings_ok(chain_length, chain_steps, sy_steps, dt, tau_t, kT, 3.0 * n) || !(tau_b > 0.0) || !std::isfinite(pressure))
    return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int blocks = (n + 255) / 256;
  if (!S->ke_partials) {
    S->ke_partials = S->pool.get<double>((size_t)(S->n_cap + 255) / 256);
    if (!S->ke_partials) return kCudaError;
  }
  if (!S->h_box && cudaMallocHost((void**)&S->h_box, sizeof(double)) != cudaSuccess) return kCudaError;
  double h0[9];
  for (int k = 0; k < 9; ++k) h0[k] = cell0_9[k];
  const double V0 = std::fabs(h0[0] * (h0[4] * h0[8] - h0[5] * h0[7]) - h0[1] * (h0[3] * h0[8] - h0[5] * h0[6]) +
                              h0[2] * (h0[3] * h0[7] - h0[4] * h0[6]));
  if (!(V0 > 0.0)) return kInvalidArgument;
  NptParams p{chain_length, chain_steps, sy_steps, n, (double)dt, kT, pressure, tau_t, tau_b, V0};
  double* box = state + 2 * kNhcStateDoubles;
  float cell9[9];
  for (int step = 0; step < n_steps; ++step) {
    // the box's first half kick needs the virial of the positions as they are: the forces in F came with it
    if (!S->virial_fresh) return kInvalidArgument;
    S->prof.begin(kPMd, st);
    if (step == 0) md_kinetic_partials(st, n, masses, V, S->ke_partials);
    npt_pre(st, state, p, S->virial_sum, step == 0 ? S->ke_partials : nullptr, blocks);
    npt_first_half(st, n, masses, R, V, F, state);
    S->prof.end(st);
    // the evaluation needs the new cell on the host: one 8-byte read per step
    SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->h_box, box, sizeof(double), cudaMemcpyDeviceToHost, st));
    SO3LR_CUDA_CHECK(cudaStreamSynchronize(st));
    if (!std::isfinite(*S->h_box)) return kNotFinite;
    const double scale = std::exp(*S->h_box);
    for (int k = 0; k < 9; ++k) cell9[k] = (float)(h0[k] * scale);
    int rc = make_cell(cell9, &S->cell);     // lists stay: the skin test sees the atoms' affine motion like any other
    if (rc) return rc;
    rc = so3lr_b200_system_compute(S, st, R, F, nullptr, step == n_steps - 1 ? energy : nullptr, nullptr, nullptr, nullptr);
    if (rc) return rc;
    S->prof.begin(kPMd, st);
    npt_second_half(st, n, masses, V, F, state, S->ke_partials);
    npt_post(st, state, p, S->virial_sum, S->ke_partials, blocks);
    if (step == n_steps - 1) md_apply_scale(st, n, V, state);
    S->prof.end(st);
  }
  if (cell_out9) {
    SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->h_box, box, sizeof(double), cudaMemcpyDeviceToHost, st));
    SO3LR_CUDA_CHECK(cudaStreamSynchronize(st));
    const double scale = std::exp(*S->h_box);
    for (int k = 0; k < 9; ++k) cell_out9[k] = (float)(h0[k] * scale);
  }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// ---- domain-decomposed evaluation (one context per rank; halo exchange is the caller's job) ----
SO3LR_B200_API int so3lr_b200_dd_set_atoms(so3lr_b200_system* S, int n_local, const int32_t* shells4, const int32_t* Z_local_dev,
                                           const float* cell9) {
  if (!S || !shells4 || !Z_local_dev || n_local <= 0) return kInvalidArgument;
  if (S->n_graphs != 1) return kInvalidArgument;
  drop_step_graph(S);
  if (S->ks.mode && !S->ks_cell_set) {
    std::fprintf(stderr, "so3lr_b200: a decomposed evaluation with the reciprocal-space Coulomb sum needs so3lr_b200_dd_kspace_cell first\n");
    return kInvalidArgument;
  }
  if (S->mctx.embed_z != S->model->M.embed_z) {
    std::fprintf(stderr, "so3lr_b200: a decomposed evaluation of a charged or open-shell structure is not supported (the charge embedding "
                         "needs the composition of the whole structure)\n");
    return kInvalidArgument;
  }
  if (n_local > S->n_cap) return kTooLarge;
  if (!(shells4[0] > 0 && shells4[0] <= shells4[1] && shells4[1] <= shells4[2] && shells4[2] <= shells4[3] && shells4[3] == n_local))
    return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  int rc = make_cell(cell9, &S->cell);
  if (rc) return rc;
  S->n = n_local;
  for (int k = 0; k < 4; ++k) S->shells[k] = shells4[k];
  SO3LR_CUDA_CHECK(cudaMemcpy(S->d_Z0, Z_local_dev, (size_t)n_local * sizeof(int), cudaMemcpyDeviceToDevice));
  {
    std::vector<int> zh((size_t)n_local);
    SO3LR_CUDA_CHECK(cudaMemcpy(zh.data(), Z_local_dev, (size_t)n_local * sizeof(int), cudaMemcpyDeviceToHost));
    if (int bad = first_unsupported_element(zh.data(), n_local)) {
      std::fprintf(stderr, "so3lr_b200: atomic number %d is outside the supported range 1..%d\n", bad == -1 ? 0 : bad, kMaxZ);
      return kInvalidArgument;
    }
    rc = species_tables_build(nullptr, S->mctx, zh.data(), n_local, &S->sp);
    if (rc) return rc;
    SO3LR_CUDA_CHECK(cudaDeviceSynchronize());
  }
  const int gs[2] = {0, n_local};
  SO3LR_CUDA_CHECK(cudaMemcpy(S->d_graph_start, gs, sizeof(gs), cudaMemcpyHostToDevice));
  S->d_Z = S->d_Z0; S->sorted = false; S->have_lists = false;
  S->o_e_atom = S->e_atom; S->o_q = S->q; S->o_h = S->h; S->o_zbl = S->e_zbl; S->o_coul = S->e_coul; S->o_disp = S->e_disp;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_dd_begin(so3lr_b200_system* S, void* stream, const float* R_local_dev) {
  if (!S || !R_local_dev || S->shells[3] != S->n || S->n <= 0) return kInvalidArgument;
  if (!(S->opt.cutoff_lr > 0.f)) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int n0 = S->shells[0], n1 = S->shells[1];
  if (!S->have_lists) {
    S->prof.begin(kPNlist, st);
    // rows of the owned atoms only: every kernel of the decomposed path gathers towards an owned atom
    int rc = nlist_build(S->nws, st, S->cell, S->n, R_local_dev, kCutoffSr + S->opt.skin, 0, nullptr, nullptr, &S->sr, 1, nullptr, n0);
    if (rc) return rc;
    // ordered: ghosts carry the larger indices, so an owned row holds every owned partner once and every ghost partner
    rc = nlist_build(S->nws, st, S->cell, S->n, R_local_dev, S->opt.cutoff_lr + S->opt.skin, 1, nullptr, nullptr, &S->lrl, 1, nullptr, n0);
    if (rc) return rc;
    rc = ensure_edge_buffers(S, S->sr.count);
    if (rc) return rc;
    S->sr_rows = n0;
    S->prof.end(st);
    S->have_lists = true;
    S->n_rebuilds++;
  }
  const ModelDev& M = S->mctx;
  fill(st, S->e_zbl, n0, 0.f);
  fill(st, S->F_s, (size_t)n0 * 3, 0.f);
  if (S->vir()) fill(st, S->virial, (size_t)n0 * 6, 0.f);
  S->prof.begin(kPGeom, st);
  launch_sr_geometry_zbl(st, M, S->cell, S->n, S->sr.count, S->sr.edge_i, S->sr.nbr_j, S->d_Z, R_local_dev, 0, S->dR, S->e_zbl, nullptr, nullptr,
                         S->F_s, n0, S->vir());
  if (attention_mode() >= kAttnTcFwd) {
    int rcv = valid_edges_build(&S->ve, st, S->sr_rows, S->n, S->sr.row_ptr, S->sr.nbr_j, S->dR);
    if (rcv) return rcv;
  }
  S->prof.end(st);
  if (!(S->sp.n_species > 0 && use_layer0_tables())) launch_embed(st, M, S->d_Z, n1, S->x[0]);   // decomposed contexts are neutral
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

SO3LR_B200_API int so3lr_b200_dd_layer_forward(so3lr_b200_system* S, void* stream, int layer) {
  if (!S || layer < 0 || layer >= kNumLayers || !S->have_lists) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int n0 = S->shells[0], n1 = S->shells[1], l = layer;
  const LayerDev& L = S->mctx.layer[l];
  if (l == 0 && S->sp.n_species > 0 && use_layer0_tables()) {
    S->prof.begin(kPLayer0Fwd, st);
    launch_layer0_fwd_tab(st, S->sp, S->mctx, n0, S->n, S->sr.row_ptr, S->sr.nbr_j, S->dR, S->d_Z, S->xa[0], S->ev1[0]);
    S->prof.end(st);
  } else {
    // with the tensor-core dense blocks the owned rows of q/k/v came out of the previous layer's block; the ghost rows
    // (features just received from their owners) are projected here
    const int first = (use_mma_dense() && l > 0) ? n0 : 0;
    S->prof.begin(kPProj, st);
    launch_proj_fwd(st, L, S->x[l] + (size_t)first * kF, n1 - first, S->qkv[l] + (size_t)first * kProj);
    S->prof.end(st);
    S->prof.begin(kPAttnFwd, st);
    attn_fwd_dispatch(S, st, L, n0, S->n, S->sr.row_ptr, S->sr.nbr_j, S->dR, S->qkv[l], S->x[l], S->ev[l], S->xa[l], S->ev1[l]);
    S->prof.end(st);
  }
  const bool emit = use_mma_dense() && l + 1 < kNumLayers;
  S->prof.begin(kPPostFwd, st);
  post_fwd_dispatch(st, L, n0, S->xa[l], S->ev1[l], S->z1[l], S->x3[l], S->gate[l], S->x[l + 1], S->ev[l + 1],
                    emit ? &S->mctx.layer[l + 1] : nullptr, emit ? S->qkv[l + 1] : nullptr, S->d_flag + 1);
  S->prof.end(st);
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

SO3LR_B200_API int so3lr_b200_dd_heads(so3lr_b200_system* S, void* stream, float* q_raw_owned_dev, float* h_owned_dev) {
  if (!S || !q_raw_owned_dev || !h_owned_dev || !S->have_lists) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int n0 = S->shells[0];
  S->prof.begin(kPHeads, st);
  heads_fwd_dispatch(st, S->mctx, n0, S->d_Z, S->x[kNumLayers], S->ze, S->zq, S->zh, S->e_nn, S->q_raw, S->hv, S->d_flag + 1);
  S->prof.end(st);
  SO3LR_CUDA_CHECK(cudaMemcpyAsync(q_raw_owned_dev, S->q_raw, (size_t)n0 * sizeof(float), cudaMemcpyDeviceToDevice, st));
  { abs_kernel<<<(n0 + 255) / 256, 256, 0, st>>>(n0, S->hv, h_owned_dev); count_launch(); }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

SO3LR_B200_API int so3lr_b200_dd_pair(so3lr_b200_system* S, void* stream, const float* R_local_dev, const float* q_local_dev,
                                      const float* h_local_dev, double* gq_sum_dev) {
  if (!S || !R_local_dev || !q_local_dev || !h_local_dev || !gq_sum_dev || !S->have_lists) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int n0 = S->shells[0];
  S->prof.begin(kPPairLr, st);
  launch_pair_lr_owned(st, S->lr, S->cell, n0, S->n, S->lrl.row_ptr, S->lrl.nbr_j, S->d_Z, R_local_dev, q_local_dev, h_local_dev, S->F_s,
                       S->gq, S->gh, S->e_coul, S->e_disp, S->vir());
  S->prof.end(st);
  { sum_to_double_kernel<<<1, 1024, 0, st>>>(n0, S->gq, gq_sum_dev); count_launch(); }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

SO3LR_B200_API int so3lr_b200_dd_kspace_cell(so3lr_b200_system* S, const float* cell9_global, float total_charge) {
  if (!S || !cell9_global) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  int rc = make_cell(cell9_global, &S->ks_cell);
  if (rc) return rc;
  if (!S->ks_cell.periodic) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaMemcpy(S->d_total_charge, &total_charge, sizeof(float), cudaMemcpyHostToDevice));
  S->ks_cell_set = true;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_dd_kspace_accumulate(so3lr_b200_system* S, void* stream, const float* R_local_dev, const float* q_local_dev,
                                                   float** buffer_dev, int64_t* n_floats) {
  if (!S || !R_local_dev || !q_local_dev || !buffer_dev || !n_floats || !S->ks.mode || !S->ks_cell_set || !S->have_lists) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  long long nf = 0;
  S->prof.begin(kPKspace, st);
  int rc = kspace_accumulate(st, S->ks, S->ks_cell, S->shells[0], R_local_dev, q_local_dev, buffer_dev, &nf);
  S->prof.end(st);
  *n_floats = nf;
  return rc;
}

SO3LR_B200_API int so3lr_b200_dd_kspace_finish(so3lr_b200_system* S, void* stream, const float* R_local_dev, const float* q_local_dev,
                                               int add_strain, double* gq_sum_dev) {
  if (!S || !R_local_dev || !q_local_dev || !gq_sum_dev || !S->ks.mode || !S->ks_cell_set || !S->have_lists) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int n0 = S->shells[0];
  S->prof.begin(kPKspace, st);
  int rc = kspace_finish(st, S->ks, S->ks_cell, n0, R_local_dev, q_local_dev, S->d_total_charge, S->e_coul, S->gq, S->F_s,
                         add_strain ? S->vir() : nullptr, 1.f);
  S->prof.end(st);
  if (rc) return rc;
  { sum_to_double_kernel<<<1, 1024, 0, st>>>(n0, S->gq, gq_sum_dev); count_launch(); }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

SO3LR_B200_API int so3lr_b200_dd_heads_backward(so3lr_b200_system* S, void* stream, const double* gq_sum_all_dev, int64_t n_atoms_all,
                                                double* energy_owned_dev) {
  if (!S || !gq_sum_all_dev || n_atoms_all <= 0 || !S->have_lists) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int n0 = S->shells[0];
  { subtract_mean_kernel<<<(n0 + 255) / 256, 256, 0, st>>>(n0, S->gq, gq_sum_all_dev, (double)n_atoms_all, S->gq_raw); count_launch(); }
  { combine_energy_kernel<<<(n0 + 255) / 256, 256, 0, st>>>(n0, S->e_nn, S->e_zbl, S->e_coul, S->e_disp, S->e_atom); count_launch(); }
  if (energy_owned_dev) { sum_to_double_kernel<<<1, 1024, 0, st>>>(n0, S->e_atom, energy_owned_dev); count_launch(); }
  S->prof.begin(kPHeads, st);
  heads_bwd_dispatch(st, S->mctx, n0, S->d_Z, S->ze, S->zq, S->zh, S->hv, S->ones, S->gq_raw, S->gh, S->g4, S->d_flag + 1);
  S->prof.end(st);
  S->dd_gev2 = S->gev_a; S->dd_gev_in = S->gev_b;
  fill(st, S->dd_gev2, (size_t)n0 * kMTot, 0.f);
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// cotangents of the layer's attention outputs on the owned atoms (rows [0, n0) of the buffers 2 and 3 of dd_buffer)
SO3LR_B200_API int so3lr_b200_dd_layer_backward_post(so3lr_b200_system* S, void* stream, int layer) {
  if (!S || layer < 0 || layer >= kNumLayers || !S->have_lists || !S->dd_gev2) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int n0 = S->shells[0], l = layer;
  const bool fused_in = use_mma_dense() && l + 1 < kNumLayers;
  S->prof.begin(kPPostBwd, st);
  post_bwd_dispatch(st, S->mctx.layer[l], n0, S->xa[l], S->ev1[l], S->z1[l], S->x3[l], S->gate[l], S->g4, S->dd_gev2, S->g_xa, S->gev1,
                    fused_in ? &S->mctx.layer[l + 1] : nullptr, S->g_qkv, S->d_flag + 1);
  S->prof.end(st);
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// needs the cotangent rows of the short-range ghosts filled in by their owners
SO3LR_B200_API int so3lr_b200_dd_layer_backward_attn(so3lr_b200_system* S, void* stream, int layer) {
  if (!S || layer < 0 || layer >= kNumLayers || !S->have_lists || !S->dd_gev2) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  cudaStream_t st = (cudaStream_t)stream;
  const int n0 = S->shells[0], l = layer;
  const LayerDev& L = S->mctx.layer[l];
  S->prof.begin(l == 0 ? kPLayer0Bwd : kPAttnBwd, st);
  if (l == 0 && S->sp.n_species > 0 && use_layer0_tables())
    launch_layer0_bwd_tab(st, S->sp, n0, S->shells[1], S->n, S->sr.row_ptr, S->sr.nbr_j, S->dR, S->d_Z, S->g_xa, S->gev1, S->GV, S->F_s, S->vir());
  else
    attn_bwd_dispatch(S, st, L, n0, S->n, S->sr.row_ptr, S->sr.nbr_j, S->dR, S->qkv[l], S->ev[l], S->g_xa, S->gev1, S->g_qkv, S->dd_gev_in, S->F_s,
                      l == 0 ? 1 : 0, S->vir());
  S->prof.end(st);
  if (l == 0 && S->vir()) reduce_virial(S, st, n0);
  if (l > 0) {
    if (!use_mma_dense()) {
      SO3LR_CUDA_CHECK(cudaMemcpyAsync(S->g4, S->g_xa, (size_t)n0 * kF * sizeof(float), cudaMemcpyDeviceToDevice, st));
      S->prof.begin(kPProjBwd, st); launch_proj_bwd(st, L, S->g_qkv, n0, S->g4, 1); S->prof.end(st);
    }
    float* t = S->dd_gev2; S->dd_gev2 = S->dd_gev_in; S->dd_gev_in = t;
  }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

SO3LR_B200_API int so3lr_b200_dd_forces(so3lr_b200_system* S, void* stream, float* F_owned_dev) {
  if (!S || !F_owned_dev) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  SO3LR_CUDA_CHECK(cudaMemcpyAsync(F_owned_dev, S->F_s, (size_t)S->shells[0] * 3 * sizeof(float), cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  return kOk;
}

SO3LR_B200_API int so3lr_b200_dd_buffer(so3lr_b200_system* S, int which, int layer, float** ptr, int* row_floats) {
  if (!S || !ptr || !row_floats) return kInvalidArgument;
  switch (which) {
    case 0: if (layer < 0 || layer > kNumLayers) return kInvalidArgument; *ptr = S->x[layer]; *row_floats = kF; return kOk;
    case 1: if (layer < 0 || layer > kNumLayers) return kInvalidArgument; *ptr = S->ev[layer]; *row_floats = kMTot; return kOk;
    case 2: *ptr = S->g_xa; *row_floats = kF; return kOk;
    case 3: *ptr = S->gev1; *row_floats = kMTot; return kOk;
    default: return kInvalidArgument;
  }
}

SO3LR_B200_API int so3lr_b200_system_profile(so3lr_b200_system* S, int enable) {
  if (!S) return kInvalidArgument;
  S->prof.on = enable != 0;
  S->prof.used = 0;
  return kOk;
}

SO3LR_B200_API int so3lr_b200_system_profile_read(so3lr_b200_system* S, int max_groups, float* ms_total, int64_t* launches, const char** names) {
  if (!S || !ms_total || !launches) return kInvalidArgument;
  SO3LR_CUDA_CHECK(cudaSetDevice(S->model->device));
  tl_launch_counter = &S->n_launches;
  SO3LR_CUDA_CHECK(cudaDeviceSynchronize());
  int ng = max_groups < (int)kPGroups ? max_groups : (int)kPGroups;
  for (int g = 0; g < ng; ++g) { ms_total[g] = 0.f; launches[g] = 0; if (names) names[g] = kProfNames[g]; }
  for (size_t k = 0; k < S->prof.used; ++k) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, S->prof.a[k], S->prof.b[k]) == cudaSuccess && S->prof.grp[k] < ng) {
      ms_total[S->prof.grp[k]] += ms;
      launches[S->prof.grp[k]] += 1;
    }
  }
  S->prof.used = 0;
  return ng;
}

void so3lr_b200_host_sph_harm(float x, float y, float z, float* y24) { sph_harm_24(x, y, z, y24); }
SO3LR_B200_API void so3lr_b200_host_sph_harm_vjp(float x, float y, float z, const float* g24, float* g3) {
  sph_harm_24_vjp(x, y, z, g24, g3[0], g3[1], g3[2]);
}
SO3LR_B200_API void so3lr_b200_host_pair_terms(float r, int zi, int zj, float qi, float qj, float hi, float hj, float cutoff_lr, float damping,
                                float* out8) {
  LrParams P{};
  P.has_cutoff = cutoff_lr > 0.f; P.rc = cutoff_lr; P.cuton = kCutonFraction * cutoff_lr; P.has_damping = damping > 0.f;
  P.disp_on = cutoff_lr - damping; P.pair_factor = 1.f;
  set_coulomb_shift(P);
  float chi, dchi;
  coulomb_chi(P, r, chi, dchi);
  out8[0] = kKe * qi * qj * chi; out8[1] = kKe * qi * qj * dchi; out8[2] = kKe * qj * chi;
  dispersion_pair(P, r, zi, zj, hi, hj, out8[3], out8[4], out8[5], out8[6]);
  out8[7] = 0.f;
}
// Tile decomposition of the direct Ewald sum for an index grid (n1, n2, n3), host only.  counts4 = tiles, groups, largest group,
// groups that are not runs of adjacent tiles; weight_sum = sum of the slot weights (every non-zero index triple of the grid must be
// counted once: 2 for the kept member of a pair (k, -k), 1 for an index whose mirror image is outside the grid)
SO3LR_B200_API int so3lr_b200_host_kspace_tiles(int n1, int n2, int n3, int64_t* counts4, double* weight_sum) {
  if (!counts4 || !weight_sum || n1 < 1 || n2 < 1 || n3 < 1 || n1 > 1024 || n2 > 1024 || n3 > 1024) return kInvalidArgument;
  std::vector<int4> tiles; std::vector<float> wgt; std::vector<int2> groups;
  kspace_build_tiles(n1, n2, n3, tiles, wgt, groups);
  double sum = 0.0;
  for (float w : wgt) sum += w;
  int64_t largest = 0, bad = 0, covered = 0;
  std::vector<char> seen(tiles.size(), 0);
  for (const int2& g : groups) {
    if (g.y > largest) largest = g.y;
    for (int u = 0; u < g.y; ++u) {
      const size_t t = (size_t)g.x + u;
      if (t >= tiles.size() || seen[t]) { ++bad; continue; }
      seen[t] = 1; ++covered;
      if (u > 0 && (tiles[t].x != tiles[g.x].x || tiles[t].y != tiles[g.x].y || tiles[t].z != tiles[t - 1].z + 16)) ++bad;
    }
  }
  if (covered != (int64_t)tiles.size()) ++bad;
  // row masks agree with the weights
  for (size_t t = 0; t < tiles.size(); ++t)
    for (int r = 0; r < 16; ++r) {
      bool any = false;
      for (int c = 0; c < 16; ++c) any |= wgt[t * 256 + r * 16 + c] > 0.f;
      if (any != (((tiles[t].w >> r) & 1) != 0)) ++bad;
    }
  counts4[0] = (int64_t)tiles.size(); counts4[1] = (int64_t)groups.size(); counts4[2] = largest; counts4[3] = bad;
  *weight_sum = sum;
  return kOk;
}

// chi(r) and its derivative of the Coulomb pair function with the reciprocal-space part taken out (smearing > 0) or not (0)
SO3LR_B200_API void so3lr_b200_host_coulomb_chi(float r, float cutoff_lr, float smearing, float* out2) {
  LrParams P{};
  P.has_cutoff = cutoff_lr > 0.f; P.rc = cutoff_lr; P.cuton = kCutonFraction * cutoff_lr; P.pair_factor = 1.f;
  P.k_alpha = smearing > 0.f ? (float)(1.0 / (std::sqrt(2.0) * (double)smearing)) : 0.f;
  set_coulomb_shift(P);
  coulomb_chi(P, r, out2[0], out2[1]);
}
SO3LR_B200_API void so3lr_b200_host_dispersion_fast(float r, int zi, int zj, float hi, float hj, float cutoff_lr, float damping, float* out4) {
  LrParams P{};
  P.has_cutoff = cutoff_lr > 0.f; P.rc = cutoff_lr; P.cuton = kCutonFraction * cutoff_lr; P.has_damping = damping > 0.f;
  P.disp_on = cutoff_lr - damping; P.pair_factor = 1.f;
  dispersion_pair_fast(P, r, zi, zj, hi, hj, out4[0], out4[1], out4[2], out4[3]);
}
SO3LR_B200_API void so3lr_b200_host_zbl(const float* blob, float r, int zi, int zj, float* out2) {
  BlobOffsets O = blob_offsets();
  ZblParams z{};
  double a[4], c[4], cs = 0.0;
  auto sp = [](double x) { return x > 30 ? x : std::log1p(std::exp(x)); };
  for (int k = 0; k < 4; ++k) { a[k] = sp(blob[O.zbl[k]]); c[k] = sp(blob[O.zbl[4 + k]]); cs += c[k]; }
  for (int k = 0; k < 4; ++k) { z.a[k] = (float)a[k]; z.c[k] = (float)(c[k] / cs); }
  z.p = (float)sp(blob[O.zbl[8]]); z.d = (float)sp(blob[O.zbl[9]]);
  float cut, dcut;
  phys_cutoff(r, cut, dcut);
  if (r >= kCutoffSr) { cut = 0.f; dcut = 0.f; }
  zbl_edge(z, r, cut, dcut, zi, zj, out2[0], out2[1]);
}
SO3LR_B200_API void so3lr_b200_host_radial_filter(const float* blob, int layer, double r, double* w256, double* dw256) {
  radial_filter_reference(blob, layer, r, w256, dw256);
}
SO3LR_B200_API int so3lr_b200_list_row_total(void* stream, const int32_t* row_count_dev, int n_rows, int64_t* total_host) {
  if (!row_count_dev || !total_host || n_rows < 0) return kInvalidArgument;
  long long t = 0;
  const int rc = nlist_row_total((cudaStream_t)stream, n_rows, row_count_dev, &t);
  *total_host = t;
  return rc;
}
SO3LR_B200_API void so3lr_b200_host_radial_filter_chebyshev(const float* blob, int layer, double r, double* w256, double* dw256) {
  radial_filter_chebyshev(blob, layer, r, w256, dw256);
}

}  // extern "C"

// Launchers of the SO3LR CUDA kernels (one .cu file per group).
#pragma once
#include "model.h"

namespace so3lr {

// ---- atom_kernels.cu ----
int configure_atom_kernels();
void launch_embed(cudaStream_t s, const ModelDev& M, const int* Z, int n, float* x);
void launch_proj_fwd(cudaStream_t s, const LayerDev& L, const float* x, int n, float* qkv);
void launch_proj_bwd(cudaStream_t s, const LayerDev& L, const float* g_qkv, int n, float* gx, int accumulate);
void launch_atom_post_fwd(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, float* z1,
                          float* x3, float* gate, float* x4, float* ev2);
void launch_atom_post_bwd(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, const float* z1,
                          const float* x3, const float* gate, const float* g4, const float* gev2, float* g_xa, float* gev1);
void launch_heads_fwd(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* x, float* ze, float* zq, float* zh,
                      float* e_nn, float* q_raw, float* hv);
void launch_heads_bwd(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* ze, const float* zq, const float* zh,
                      const float* hv, const float* ge, const float* gq, const float* gh, float* gx);

// ---- atom_kernels_mma.cu: the same four blocks with their contractions as FP16-split tensor-core MMAs ----
int configure_atom_mma_kernels();
// proj_next / qkv_next (optional): also write the next layer's q/k/v rows (proj_next = that layer's proj_f).
void launch_atom_post_fwd_mma(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, float* z1, float* x3,
                              float* gate, float* x4, float* ev2, const uint4* proj_next, float* qkv_next);
// projT_up / g_qkv_up (optional): instead of reading g4, form it as (rows of g_xa left by the layer above) + the transposed
// projections (projT_up = that layer's projT_f) of that layer's g_qkv.
void launch_atom_post_bwd_mma(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, const float* z1,
                              const float* x3, const float* gate, const float* g4, const float* gev2, float* g_xa, float* gev1,
                              const uint4* projT_up, const float* g_qkv_up);
void launch_heads_fwd_mma(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* x, float* ze, float* zq, float* zh,
                          float* e_nn, float* q_raw, float* hv);
void launch_heads_bwd_mma(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* ze, const float* zq, const float* zh,
                          const float* hv, const float* ge, const float* gq, const float* gh, float* gx);

// ---- dense_tc.cu: the per-atom blocks on tcgen05 (persistent CTAs, 128-atom tiles, accumulators in tensor memory) ----
// err: device word that receives 2 when a bounded barrier wait inside a kernel ran out
int configure_dense_tc_kernels();
void dense_debug_print();   // development aid of timing builds; prints nothing otherwise
void launch_atom_post_fwd_tc(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, float* z1, float* x3, float* gate,
                             float* x4, float* ev2, const unsigned char* proj_u, float* qkv_next, int* err);
void launch_atom_post_bwd_tc(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, const float* z1, const float* x3,
                             const float* gate, const float* g4, const float* gev2, float* g_xa, float* gev1, const unsigned char* projT_u,
                             const float* g_qkv_up, int* err);

void launch_heads_fwd_tc(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* x, float* ze, float* zq, float* zh, float* e_nn,
                         float* q_raw, float* hv, int* err);
void launch_heads_bwd_tc(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* ze, const float* zq, const float* zh,
                         const float* hv, const float* ge, const float* gq, const float* gh, float* gx, int* err);

// ---- kspace.cu: reciprocal-space (Ewald) part of the electrostatic energy of one periodic structure ----
struct KSpaceDev {
  int mode = 0;            // 0 off, 1 Ewald sum over the index grid, 2 particle-mesh Ewald on a mesh of that shape
  float smearing = 0.f;    // Gaussian width s of the split erf(r / (sqrt(2) s)) / r
  int shape[3] = {0, 0, 0};
  int n_tiles = 0;
  int n_groups = 0;
  int4* tiles = nullptr;   // (h1, first h2, first h3, mask of the h2 rows that hold a kept vector) of each 16 x 16 tile of kept indices
  int2* groups = nullptr;  // (first tile, count <= 4): tiles that share (h1, first h2) and follow one another along h3
  float* wgt = nullptr;    // [n_tiles][256] 2 / 1 / 0: member of a (k, -k) pair, unpaired index, not part of the sum
  float2* Sk = nullptr;    // [n_tiles][256] structure factors
  float* acc = nullptr;    // [n_atoms][4] potential and the three index-weighted force sums
  float* mesh = nullptr;   // mode 2: [n1][n2][n3] charges, then the convolved potential
  float2* fq = nullptr;    // mode 2: [n1][n2][n3 / 2 + 1] transform of the mesh
  int plan_r2c = 0, plan_c2r = 0;   // cuFFT plans (handles)
  bool plans = false;
};
// host side of the direct sum's set-up: tiles (h1, first h2, first h3, row mask), 256 slot weights per tile, groups (first tile, count)
void kspace_build_tiles(int n1, int n2, int n3, std::vector<int4>& tiles, std::vector<float>& wgt, std::vector<int2>& groups);
int kspace_setup(KSpaceDev* K, int n_atoms, int mode, float smearing, int n1, int n2, int n3);   // allocates; call outside handlers
void kspace_free(KSpaceDev* K);
// adds to e_coul (per-atom energies), gq (dE/dq), F (force_sign = 1: forces at fixed charges; -1: the gradient) and, when given, the
// six virial components of one row
// the two halves of launch_ewald: what is additive over atoms (charge mesh or structure factors; `buffer` / `n_floats` name it), and the rest
int kspace_accumulate(cudaStream_t st, const KSpaceDev& K, const Cell& cell, int n, const float* R, const float* q, float** buffer,
                      long long* n_floats);
int kspace_finish(cudaStream_t st, const KSpaceDev& K, const Cell& cell, int n, const float* R, const float* q, const float* total_charge,
                  float* e_coul, float* gq, float* F, float* virial_row, float force_sign);
int launch_ewald(cudaStream_t st, const KSpaceDev& K, const Cell& cell, int n, const float* R, const float* q, const float* total_charge,
                 float* e_coul, float* gq, float* F, float* virial_row, float force_sign);

// ---- halo.cu: rows idx[r] of up to four row-major float arrays <-> one packed buffer [n_rows][sum of widths] ----
int pack_rows(void* stream, int n_arrays, float* const* arrays, const int* widths, const int64_t* idx, int64_t n_rows, float* buf, bool unpack);

// ---- attention.cu ----
// Short-range edges are grouped by receiver: edges row_ptr[i] .. row_ptr[i+1]-1 belong to centre i and hold the
// neighbour index nbr_j[e] and the displacement dR[e] (3 floats).  Edges with |dR| >= 4.5, |dR| == 0 or
// nbr_j >= n are padding.
int configure_attention_kernels();
void launch_attn_fwd(cudaStream_t s, const LayerDev& L, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                     const float* qkv, const float* x_in, const float* ev_in, float* xa, float* ev1);
// g_xa / gev1: cotangents of xa / ev1.  Adds into g_qkv (k,v parts by atomics; q parts stored), gev_in (atomics; the
// caller pre-loads it with gev1 for the skip connection) and g_dR (+=).  `first_layer`: only g_dR is produced.
// run_if_set (optional): the kernel of a layer with a spherical filter returns at once unless *run_if_set != 0
void launch_attn_bwd(cudaStream_t s, const LayerDev& L, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                     const float* qkv, const float* ev_in, const float* g_xa, const float* gev1, float* g_qkv,
                     float* gev_in, float* g_dR, int first_layer, const int* run_if_set = nullptr);

// ---- attention_sym.cu ----
// Gather-only kernels of the fused positions -> forces path.  They need a symmetric list (j in row i <=> i in row j with
// dR_ji = -dR_ij), which the cell-list builder guarantees.  The backward kernel writes g_qkv / gev_in rows completely
// (no pre-fill needed; gev_in includes the skip term gev1) and adds the attention part of the force on atom i to F[i].
int configure_attention_sym_kernels();
// n_recv: rows 0 .. n_recv-1 are evaluated (receivers); n: number of atoms a neighbour index may address.
void launch_attn_fwd_sym(cudaStream_t s, const LayerDev& L, int n_recv, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                         const float* qkv, const float* x_in, const float* ev_in, float* xa, float* ev1);
void launch_attn_bwd_sym(cudaStream_t s, const LayerDev& L, int n_recv, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                         const float* qkv, const float* ev_in, const float* g_xa, const float* gev1, float* g_qkv, float* gev_in,
                         float* F, int first_layer, float* virial = nullptr);

// ---- attention_mma.cu ----
// Same contracts as the *_sym launchers, for layers with a spherical filter (L.has_spherical): the per-edge filter
// contractions run as FP16-split tensor-core MMAs with FP32-level accuracy.
int configure_attention_mma_kernels();
void launch_attn_fwd_mma(cudaStream_t s, const LayerDev& L, int n_recv, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                         const float* qkv, const float* x_in, const float* ev_in, float* xa, float* ev1);
void launch_attn_bwd_mma(cudaStream_t s, const LayerDev& L, int n_recv, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                         const float* qkv, const float* ev_in, const float* g_xa, const float* gev1, float* g_qkv, float* gev_in,
                         float* F, float* virial = nullptr);

// ---- attention_tc.cu: layers with a spherical filter as CTA-tiled tcgen05 kernels ----
// Short-range list entries inside the cutoff, compacted once per evaluation and grouped by receiver: entry p of row i
// (row_ptr[i] <= p < row_ptr[i + 1]) holds the receiver i[p], the sender j[p] and d[p] = (dx, dy, dz, |dR|).
struct ValidEdges {
  int* row_ptr = nullptr;   // n_rows + 1
  int* count = nullptr;     // per-row counts (scratch of the build)
  int* i = nullptr;
  int* j = nullptr;
  float4* d = nullptr;
  int* orig = nullptr;      // position of each entry in the list it was compacted from (only when asked for)
  long long orig_cap = 0;
  void* cub_tmp = nullptr;
  size_t cub_bytes = 0;
  int row_cap = 0;
  long long capacity = 0;
  int n_rows = 0;           // rows of the latest build
};
int configure_attention_tc_kernels();
void tc_debug_print();
// (re)allocates for n_rows receivers and `capacity` entries (the capacity of the list they are compacted from)
int valid_edges_reserve(ValidEdges* V, int n_rows, long long capacity);
void valid_edges_free(ValidEdges* V);
// no host synchronisation: counts stay on the device
int valid_edges_build(ValidEdges* V, cudaStream_t s, int n_rows, int n, const int* row_ptr, const int* nbr_j, const float* dR,
                      bool want_orig = false);
// *asym = 1 when some entry (i <- j, d) has no partner (j <- i, -d) in the compacted list (the word must be zero beforehand)
void valid_edges_check_symmetric(const ValidEdges& V, cudaStream_t s, int* asym);
// The reverse kernel for caller-supplied lists: runs only while *asym == 0 and, instead of summing forces, adds to every source
// entry e (V.orig) half of the force that the pair exerts on its receiver, g[e] += (dE/d dR_e - dE/d dR_e') / 2 with e' the
// reversed entry.  For any motion of atoms or cell (dR_e' = -dR_e) that is equivalent to the per-entry gradient.  The caller
// zeroes g_qkv and presets gev_in.
int launch_attn_bwd_tc_graph(cudaStream_t s, const LayerDev& L, const ValidEdges& V, int n_recv, const float* qkv, const float* ev_in,
                             const float* g_xa, const float* gev1, float* g_qkv, float* gev_in, float* g_dR, int* err, const int* asym);
// Same results as launch_attn_fwd_sym for rows [0, n_recv).  `err` (device int) is set to 1 when a bounded wait on the
// tensor-core pipeline ran out; the outputs are then incomplete.
int launch_attn_fwd_tc(cudaStream_t s, const LayerDev& L, const ValidEdges& V, int n_recv, const float* qkv, const float* x_in,
                       const float* ev_in, float* xa, float* ev1, int* err);
// Same results as launch_attn_bwd_sym (first_layer = 0) for rows [0, n_recv): writes g_qkv and gev_in rows, adds to F (and virial).
int launch_attn_bwd_tc(cudaStream_t s, const LayerDev& L, const ValidEdges& V, int n_recv, const float* qkv, const float* ev_in,
                       const float* g_xa, const float* gev1, float* g_qkv, float* gev_in, float* F, float* virial, int* err);

// ---- layer0_tab.cu: first layer through per-element-pair tables (its inputs depend on the elements only) ----
constexpr int kMaxTabSpecies = 8;
struct SpeciesTables {
  int n_species = 0;               // 0: not available (more than kMaxTabSpecies elements): use the generic kernels
  int species[kMaxTabSpecies] = {};
  float* table = nullptr;          // [kMaxTabSpecies^2][kTableGrid][16]
  float* v_sp = nullptr;           // [species][128] value rows
  int* slot = nullptr;             // [119] atomic number -> species slot
  float* qkv_sp = nullptr;         // scratch of the build
  float* x_sp = nullptr;
  int* z_sp = nullptr;
};
int species_tables_build(cudaStream_t st, const ModelDev& M, const int* Z_host, int n, SpeciesTables* T);
void species_tables_free(SpeciesTables* T);
void launch_layer0_fwd_tab(cudaStream_t s, const SpeciesTables& T, const ModelDev& M, int n_recv, int n, const int* row_ptr,
                           const int* nbr_j, const float* dR, const int* Z, float* xa, float* ev1);
// g_xa must be valid for atoms [0, n_gv) (every possible neighbour of a receiver); GV is a scratch of n_gv x 32 floats
void launch_layer0_bwd_tab(cudaStream_t s, const SpeciesTables& T, int n_recv, int n_gv, int n, const int* row_ptr, const int* nbr_j,
                           const float* dR, const int* Z, const float* g_xa, const float* gev1, float* GV, float* F,
                           float* virial = nullptr);

// ---- pair_kernels.cu ----
// dR for every short-range edge from positions (+ minimum image), ZBL energy into e_atom[centre], ZBL gradient
// written to g_dR (initialises it) when g_dR is given, and/or added straight into the forces F_direct (F_i += g,
// F_j -= g).  With `dR_given` the displacements are inputs.
void launch_sr_geometry_zbl(cudaStream_t s, const ModelDev& M, const Cell& cell, int n, long long n_edges, const int* edge_i,
                            const int* nbr_j, const int* Z, const float* R, int dR_given, float* dR, float* e_atom, float* g_dR,
                            const float* ge, float* F_direct, int n_owned = -1, float* virial = nullptr);
// F[i] += g, F[j] -= g for every edge
void launch_force_scatter(cudaStream_t s, int n, long long n_edges, const int* edge_i, const int* nbr_j, const float* g_dR,
                          float* F);
// long-range pairs grouped by first atom (row_ptr over i).  mode 0: displacements from positions, forces accumulated;
// mode 1: displacements given (dR_lr), gradient per pair written to g_dR_lr.
void launch_pair_lr(cudaStream_t s, const LrParams& P, const Cell& cell, int n, const int* row_ptr, const int* nbr_j,
                    const int* Z, const float* R, const float* q, const float* h, int mode, const float* dR_lr,
                    float* g_dR_lr, float* e_atom, float* F, float* gq, float* gh, float* e_coul, float* e_disp,
                    const float* ge, float* virial = nullptr);
// the single-device form with packed gathers and vector reductions (pack: scratch of 12 n floats, 16-byte aligned); adds to
// F, gq, gh, e_coul, e_disp like launch_pair_lr in mode 0
void launch_pair_lr_packed(cudaStream_t s, const LrParams& P, const Cell& cell, int n, const int* row_ptr, const int* nbr_j, const int* Z,
                           const float* R, const float* q, const float* h, float* pack, float* F, float* gq, float* gh, float* e_coul,
                           float* e_disp, float* virial);
// Domain-decomposed variant: rows 0 .. n_owned-1 of an ordered list (j > i) over owned atoms and ghosts, ghosts carrying
// the larger indices.  Pairs of two owned atoms are evaluated once and scatter the partner's derivatives (atomics); pairs
// with a ghost end book half of the energy and the row atom's derivatives.  gq, gh are zeroed here and accumulated, F_add is
// added to, e_coul[i], e_disp[i] are written by the row's warp.
void launch_pair_lr_owned(cudaStream_t s, const LrParams& P, const Cell& cell, int n_owned, int n, const int* row_ptr,
                          const int* nbr_j, const int* Z, const float* R, const float* q, const float* h, float* F_add,
                          float* gq, float* gh, float* e_coul, float* e_disp, float* virial = nullptr);
// q = q_raw + (Q_g - sum_g q_raw) / n_g ; h = |hv| ; and the transposed operation for the cotangents
// (atoms of one graph are contiguous: graph g owns atoms graph_start[g] .. graph_start[g+1]-1)
// n_atoms / scratch (optional, 4 * 296 doubles): a single large structure is spread over many CTAs instead of one.
void launch_charge_conserve(cudaStream_t s, int n_graphs, const int* graph_start, const float* q_raw,
                            const float* total_charge, const float* hv, float* q, float* h, int n_atoms = 0, double* scratch = nullptr);
void launch_charge_conserve_bwd(cudaStream_t s, int n_graphs, const int* graph_start, const float* gq, float* gq_raw, int n_atoms = 0,
                                double* scratch = nullptr);
// per-graph energy (double) and dipole sums
void launch_graph_reduce(cudaStream_t s, int n_graphs, const int* graph_start, const float* e_atom, const float* q,
                         const float* R, double* e_graph, float* dipole, int n_atoms = 0, double* scratch = nullptr);

// ---- nlist.cu ----
struct NeighborListDev {
  int* row_ptr = nullptr;    // n + 1
  int row_cap = 0;           // allocated entries of row_ptr
  int* nbr_j = nullptr;      // capacity
  int* edge_i = nullptr;     // capacity
  long long capacity = 0;
  long long count = 0;       // valid after build
};
struct NlistWorkspace;       // opaque scratch (cell ids, sort buffers)
NlistWorkspace* nlist_workspace_create();
void nlist_workspace_destroy(NlistWorkspace*);
// perm[k] = index of the atom that comes k-th along a Morton curve through cells of edge >= cell_size (periodic cells
// only).  Radix sort is stable, so the order is deterministic.
int spatial_order(NlistWorkspace* ws, cudaStream_t s, const Cell& cell, int n, const float* R, float cell_size, int* perm);
// Builds rows for all i.  ordered: keep j > i only.  seg/graph_start (optional): pairs only inside one graph and the
// candidate loop runs over the graph's atoms.  Grows `out` when `allow_grow`, otherwise sets *overflow (device int).
// n_rows >= 0: only the rows of atoms 0 .. n_rows-1 are built (candidates are still all n atoms).
// 64-bit sum of per-row pair counts as the builder forms it before its 32-bit scan; kTooLarge when the CSR offsets would
// leave the int range (the builder returns the same status before it fills a single row)
int nlist_row_total(cudaStream_t s, int n, const int* row_count_dev, long long* total_host);
int nlist_build(NlistWorkspace* ws, cudaStream_t s, const Cell& cell, int n, const float* R, float r_list, int ordered,
                const int* seg, const int* graph_start, NeighborListDev* out, int allow_grow, int* d_overflow, int n_rows = -1);

}  // namespace so3lr

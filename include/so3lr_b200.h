/* so3lr_b200 -- C ABI of the B200-native SO3LR energy + force library.
 *
 * Plain pointers and sizes only; every device pointer is a CUDA device address on the device the handle was
 * created on, `stream` is a cudaStream_t passed as void*.  Every function returns an int status
 * (SO3LR_B200_OK == 0).  Nothing here falls back to the CPU: without a CUDA device the calls fail.
 *
 * "Reference" citations name files of the so3lr package (general-molecular-simulations/so3lr) whose behaviour
 * the entry point replaces.
 */
#ifndef SO3LR_B200_H_
#define SO3LR_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define SO3LR_B200_API __attribute__((visibility("default")))
#else
#define SO3LR_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
  SO3LR_B200_OK = 0,
  SO3LR_B200_INVALID_ARGUMENT = 1,
  SO3LR_B200_CUDA_ERROR = 2,
  SO3LR_B200_OVERFLOW = 3,      /* a neighbor list did not fit its fixed capacity */
  SO3LR_B200_NOT_FINITE = 4,    /* NaN / Inf positions */
  SO3LR_B200_TOO_LARGE = 5
};

typedef struct so3lr_b200_model so3lr_b200_model;     /* weights + derived tables on one device */
typedef struct so3lr_b200_system so3lr_b200_system;   /* one evaluation context: atoms, lists, workspaces */

/* Library / ABI version. */
SO3LR_B200_API int so3lr_b200_version(void);
SO3LR_B200_API const char* so3lr_b200_status_string(int status);

/* Create the model from the packed float32 parameter blob (host pointer, `n_floats` = 530238 values in the order
 * of so3lr/params/params.pkl as written by so3lr_b200/params/pack_params.py).
 * Replaces: MLFFPotentialSparse.create_from_workdir(...) in so3lr/potential.py:17-29 and
 *           load_model_from_workdir(...) in so3lr/base_calculator.py:24-33. */
SO3LR_B200_API int so3lr_b200_model_create(const float* blob_host, size_t n_floats, int device, so3lr_b200_model** out);
SO3LR_B200_API int so3lr_b200_model_destroy(so3lr_b200_model* model);

/* Options of an evaluation context.
 * cutoff_lr <= 0 : no long-range cutoff (plain erf Coulomb, unswitched dispersion; all pairs inside a graph).
 * damping   <= 0 : dispersion is not switched off before cutoff_lr.
 * lr_both_directions: 0 = each pair once, energy booked on the first atom (neighborlist_format_lr
 *   'ordered_sparse', so3lr/potential.py:22); 1 = both directions at half weight ('sparse',
 *   so3lr/base_calculator.py:31).
 * skin: extra list radius; lists are rebuilt when an atom moved more than skin/2 since the last build
 *   (dr_threshold of so3lr/jaxmd_utils.py:85). */
typedef struct so3lr_b200_options {
  float cutoff_lr;
  float damping;
  float skin;
  int lr_both_directions;
  float lr_list_cutoff;   /* radius of the long-range list when cutoff_lr <= 0; <= 0: all pairs of a graph */
} so3lr_b200_options;

/* Create a context for `n_atoms` atoms split into `n_graphs` graphs of contiguous atoms
 * (graph g owns atoms graph_start[g] .. graph_start[g+1]-1; pass n_graphs = 1 and graph_start = NULL for one
 * structure).  `atomic_numbers`, `graph_start`, `total_charge`, `num_unpaired` are host arrays (the last two may
 * be NULL = all zero).  `cell` is NULL (free space) or 9 floats, rows = lattice vectors, in Angstrom.
 * Replaces: the Graph / inputs-dict assembly of so3lr/jaxmd_utils.py:57-73 and so3lr/base_calculator.py:57-86. */
SO3LR_B200_API int so3lr_b200_system_create(so3lr_b200_model* model, int n_atoms, const int32_t* atomic_numbers, int n_graphs,
                             const int32_t* graph_start, const float* total_charge, const float* num_unpaired,
                             const float* cell, const so3lr_b200_options* options, so3lr_b200_system** out);
SO3LR_B200_API int so3lr_b200_system_destroy(so3lr_b200_system* sys);
/* New cell (NPT); forces a list rebuild on the next evaluation. */
SO3LR_B200_API int so3lr_b200_system_set_cell(so3lr_b200_system* sys, const float* cell);

/* Deferred skin test.  By default every evaluation with skin > 0 reads one flag word back from the device (has an atom
 * moved further than skin / 2 since the lists were built?) before it launches its kernels: one host wait per step.  With
 * this mode on, the flag of step k is copied to pinned memory asynchronously and read at step k + 1, so an evaluation only
 * enqueues work on the caller's stream; the trigger distance becomes skin / 2 - margin so that the lists still cover the one
 * extra step (margin >= the largest displacement of an atom in one step; 0.05 A covers a 0.5 fs step far beyond 1000 K).
 * Non-finite positions and a timed-out tensor-core wait are likewise reported by the following call.  A step that does
 * rebuild its lists still synchronises (list sizes are read back to size the buffers).
 * Replaces: the `nbrs.update` + `did_buffer_overflow` polling of so3lr/cli/so3lr_md.py:862-876,1143-1152, which XLA runs
 * inside the compiled step without a host round trip. */
SO3LR_B200_API int so3lr_b200_system_defer_skin_test(so3lr_b200_system* sys, int enable, float margin);

/* Energy + forces from positions that already live on the device (positions_dev: n_atoms x 3 float32, Cartesian,
 * Angstrom).  Outputs are device pointers and may be NULL when not wanted:
 *   forces_dev (n_atoms x 3), e_atom_dev (n_atoms), energy_dev (n_graphs doubles), charges_dev (n_atoms),
 *   hirshfeld_dev (n_atoms), dipole_dev (n_graphs x 3).
 * Work is enqueued on `stream`; the call synchronises with the stream only when a neighbor list has to be rebuilt.
 * Replaces: energy_fn + jax_md.quantity.force of so3lr/jaxmd_utils.py:130-141 (neighbor_fn.update included) and
 *           so3lr_fn of so3lr/base_calculator.py:95-122. */
SO3LR_B200_API int so3lr_b200_system_compute(so3lr_b200_system* sys, void* stream, const float* positions_dev, float* forces_dev,
                              float* e_atom_dev, double* energy_dev, float* charges_dev, float* hirshfeld_dev,
                              float* dipole_dev);

/* Same evaluation with HOST buffers: copies positions in, results out, and returns after the stream is idle.
 * This is the call a host application (ASE calculator, so3lr/ase_utils.py:7-28) makes once per step. */
SO3LR_B200_API int so3lr_b200_system_compute_host(so3lr_b200_system* sys, const float* positions_host, float* forces_host,
                                   double* energy_host, float* charges_host, float* hirshfeld_host, float* dipole_host);

/* Small structures are bound by the launch rate (about 40 launches per evaluation), so between two list rebuilds
 * so3lr_b200_system_compute replays its launches from a CUDA graph: the graph is captured at the second consecutive call with the
 * same positions / forces buffers on a stream that can be captured (not the legacy default stream) and dropped when the lists are
 * rebuilt, the cell changes or the buffers differ.  At most 65,536 atoms, skin > 0, no reciprocal-space part; SO3LR_B200_CUDA_GRAPH=0
 * in the environment keeps plain launches.  This counter tells how many evaluations were replays (tests, tuning). */
SO3LR_B200_API int so3lr_b200_system_graph_replays(so3lr_b200_system* sys, int64_t* n_replays);

/* Per-term energies of the last evaluation, per atom, device pointers valid until the next call (aux dictionary of
 * potential(graph, has_aux=True), so3lr/jaxmd_utils.py:138-139). */
SO3LR_B200_API int so3lr_b200_system_aux(so3lr_b200_system* sys, const float** zbl_dev, const float** coulomb_dev,
                          const float** dispersion_dev);

/* Counters: number of list rebuilds, current short-range edges and long-range pairs, kernels launched so far. */
SO3LR_B200_API int so3lr_b200_system_stats(so3lr_b200_system* sys, int64_t* n_rebuilds, int64_t* n_edges, int64_t* n_pairs,
                            int64_t* n_launches);
/* Short-range list entries inside the 4.5 A cutoff at the latest evaluation (the compacted list the tiled attention kernels
 * walk; the list of so3lr_b200_system_stats also holds the skin shell).  Waits for the device. */
SO3LR_B200_API int so3lr_b200_system_valid_edges(so3lr_b200_system* sys, int64_t* n_valid);

/* Copy the current neighbor lists out in jax-md layout: idx (2, capacity) int32 on the device, padded with n_atoms
 * (Sparse for the short-range list, OrderedSparse for the long-range one unless lr_both_directions).
 * which = 0: short range, 1: long range.  Sets *overflow_host when the list does not fit `capacity`.
 * Replaces: neighbor_fn.allocate / nbrs.update / nbrs.idx / nbrs.did_buffer_overflow
 *           (so3lr/jaxmd_utils.py:96-121, so3lr/cli/so3lr_md.py:862-876). */
SO3LR_B200_API int so3lr_b200_system_export_list(so3lr_b200_system* sys, void* stream, const float* positions_dev, int which,
                                  int32_t* idx_dev, int64_t capacity, int64_t* count_host, int* overflow_host);

/* Graph-level evaluation (the boundary at which the reference differentiates): displacements and index lists are
 * inputs, the outputs are per-atom energies and the gradients of sum_i g_e_atom[i] * e_atom[i] with respect to the
 * displacements.  Lists must be grouped by centre index (idx_i non-decreasing); padding entries carry index
 * n_atoms.  All pointers are device pointers; g_e_atom may be NULL (= ones).
 * When every short-range entry (i <- j, d) inside the cutoff has its partner (j <- i, -d) in the list (decided on the
 * device, no host read), both entries of a pair receive the antisymmetrised cotangent (dE/dd_e - dE/dd_e') / 2, which
 * contracts to the same forces and strain derivative for every motion of atoms or cell; otherwise, or with
 * SO3LR_B200_GRAPH=scatter in the environment, each entry receives dE/dd_e itself.  The call only enqueues work; it
 * allocates when the list is longer than any list the context has seen before.
 * Replaces: potential(graph) and its jax.grad w.r.t. graph.edges / graph.edges_lr
 *           (so3lr/jaxmd_utils.py:130-141, so3lr/graph.py:3-24). */
SO3LR_B200_API int so3lr_b200_system_graph_eval(so3lr_b200_system* sys, void* stream, int64_t n_edges, const int32_t* idx_i,
                                 const int32_t* idx_j, const float* edges, int64_t n_pairs, const int32_t* idx_i_lr,
                                 const int32_t* idx_j_lr, const float* edges_lr, const float* g_e_atom,
                                 float* e_atom_dev, float* g_edges_dev, float* g_edges_lr_dev, float* charges_dev,
                                 float* hirshfeld_dev);

/* Reciprocal-space part of the electrostatic energy (one periodic structure with a long-range cutoff).
 *   mode 1: Ewald sum over the k vectors of the FFT-frequency index grid of shape (n1, n2, n3) -- the shape of the reference's
 *           `k_grid` array as jaxpme.kspace.get_kgrid_ewald builds it;
 *   mode 2: smooth particle-mesh Ewald on a mesh of shape (n1, n2, n3) (get_kgrid_mesh), cubic B-splines = four interpolation
 *           nodes per axis (the reference's default `coulomb_kspace_interp_nodes=4`), each n >= 4; the two FFTs are cuFFT's,
 *           loaded at run time (status "CUDA error" when libcufft.so.11 cannot be loaded);
 *   mode 0: off again.
 * `smearing` is the Gaussian width (the reference's `k_smearing`, Angstrom).  While it is on, every pair of the long-range list
 * keeps only erf(r / sigma) / r - erf(r / (sqrt(2) smearing)) / r (shifted and blended towards the cutoff like the plain
 * term), and so3lr_b200_system_compute / _compute_host / the MD step bodies add
 *   ke / (2 V) sum_{k != 0} 4 pi / k^2 exp(-smearing^2 k^2 / 2) |S(k)|^2 - ke sum_i q_i^2 / (sqrt(2 pi) smearing) - ke pi smearing^2 Q^2 / V
 * with its forces, its dE/dq (which continues into the charge head's reverse pass) and its strain derivative.  The cell may change
 * afterwards (so3lr_b200_system_rescale_cell): the grid shape stays, the k vectors follow the cell.  Allocates and waits for the
 * device: call it between evaluations.  In decomposed evaluations it is driven through so3lr_b200_dd_kspace_*.
 * Replaces: the `k_grid` / `k_smearing` arguments of the reference's energy function (so3lr/jaxmd_utils.py:39-47,70-71), the
 *           grid set-up of so3lr/cli/so3lr_md.py:1392-1428 and the `coulomb_kspace_*` options of so3lr/potential.py:11-25. */
SO3LR_B200_API int so3lr_b200_system_set_kspace(so3lr_b200_system* sys, int mode, float smearing, int n1, int n2, int n3);

/* so3lr_b200_system_graph_eval for a context whose reciprocal-space part is on: `positions` (n_atoms, 3) are the Cartesian
 * positions the displacements were formed from (Graph.positions), and g_positions_dev receives the gradient of the
 * reciprocal-space energy with respect to them at fixed charges; the charges' own dependence on the geometry arrives through
 * g_edges_dev as usual.  The upstream cotangent is one for every atom (the per-atom reciprocal energies are not separable).
 * strain6_dev (may be NULL) receives the strain derivative of the reciprocal part at fixed fractional coordinates and fixed
 * charges, six symmetric components xx yy zz yz xz xy; its share that belongs to the cell alone (what a caller needs who
 * differentiates with respect to `positions` and `cell` separately, as the reference's `perturbation` does) is that minus
 * sum_i positions_i (x) g_positions_i. */
SO3LR_B200_API int so3lr_b200_system_graph_eval_kspace(so3lr_b200_system* sys, void* stream, int64_t n_edges, const int32_t* idx_i,
                                        const int32_t* idx_j, const float* edges, int64_t n_pairs, const int32_t* idx_i_lr,
                                        const int32_t* idx_j_lr, const float* edges_lr, const float* positions,
                                        float* e_atom_dev, float* g_edges_dev, float* g_edges_lr_dev, float* g_positions_dev,
                                        float* strain6_dev, float* charges_dev, float* hirshfeld_dev);

/* A velocity-Verlet (NVE) step driven by the library: positions/velocities/forces stay on the device.
 * masses_dev in amu, dt in fs, velocities in Angstrom/fs.  Runs `n_steps` steps; forces_dev must hold the forces
 * of positions_dev on entry (call so3lr_b200_system_compute first) and holds the final forces on return.
 * Replaces: the step body of jax_md.simulate.nve as driven by so3lr/cli/so3lr_md.py:1115-1152. */
SO3LR_B200_API int so3lr_b200_system_nve(so3lr_b200_system* sys, void* stream, int n_steps, float dt_fs, const float* masses_dev,
                          float* positions_dev, float* velocities_dev, float* forces_dev, double* energy_dev);

/* Strain derivative of the energy, dE/d eps_ab = sum over pairs of dR_a dE/d(dR)_b (eV; symmetric), accumulated beside the
 * forces by the same kernels when enabled (single-structure contexts only).  The stress of a periodic cell is this divided by
 * the cell volume; the pressure the reference's barostat uses is (2 KE - trace) / (3 V).  so3lr_b200_system_virial copies the
 * 3x3 matrix (row-major, 9 doubles) of the latest evaluation; for a domain-decomposed context it is the share of the
 * rank's owned atoms, to be summed over the ranks.
 * Replaces: the strain perturbation of so3lr/jaxmd_utils.py:48-51 differentiated by jax_md.quantity.stress / pressure,
 *           and the ASE calculator's stress (so3lr/ase_utils.py:10,22; tests/test_ase.py:145-172). */
SO3LR_B200_API int so3lr_b200_system_enable_virial(so3lr_b200_system* sys, int enable);
SO3LR_B200_API int so3lr_b200_system_virial(so3lr_b200_system* sys, void* stream, double* virial9_dev);

/* Nose-Hoover chain thermostat (Martyna-Tuckerman-Klein propagation, Suzuki-Yoshida factorisation), as
 * jax_md.simulate.nvt_nose_hoover applies it: half a thermostat step, velocity Verlet, half a thermostat step.
 * The chain lives in SO3LR_B200_NHC_STATE_DOUBLES doubles on the device:
 *   [0] kinetic energy the chain last saw (eV)   [1] momentum scale not yet applied to the velocities
 *   [2, 10) chain positions                       [10, 18) chain momenta (eV fs)
 * chain_length 1..8, chain_steps >= 1, sy_steps in {1, 3, 5, 7}; tau in fs, kT in eV; the chain masses are
 * kT tau^2 (times dof for the first), dof = 3 n_atoms.
 * Replaces: jax_md.simulate.nvt_nose_hoover as created in so3lr/cli/so3lr_md.py:1047-1075 with the settings of
 *           so3lr/cli/so3lr_md.py:1698-1707 (defaults so3lr/cli/so3lr_cli.py:114-116). */
#define SO3LR_B200_NHC_MAX_CHAIN 8
#define SO3LR_B200_NHC_STATE_DOUBLES 18
/* Zeroes a chain (scale = 1). */
SO3LR_B200_API int so3lr_b200_nhc_init(void* stream, double* chain_dev);
/* Advances a chain by n_half_steps half steps.  When ke_partials_dev is given, the kinetic energy is first set to the
 * sum of its n_partials entries (eV); a domain-decomposed run passes the all-reduced kinetic energy as one entry.
 * The momentum scale of the half steps is multiplied into chain_dev[1], or replaces it when fresh_scale is non-zero
 * (the velocities have taken up the previous value). */
SO3LR_B200_API int so3lr_b200_nhc_half_steps(void* stream, double* chain_dev, int chain_length, int chain_steps, int sy_steps,
                                             double dt_fs, double tau_fs, double kT, double dof, int n_half_steps,
                                             int fresh_scale, const double* ke_partials_dev, int n_partials);
/* n_steps NVT steps driven by the library, same buffers and units as so3lr_b200_system_nve.  On return the velocities
 * carry every scale (chain_dev[1] is 1) and chain_dev[0] holds their kinetic energy. */
SO3LR_B200_API int so3lr_b200_system_nvt(so3lr_b200_system* sys, void* stream, int n_steps, float dt_fs, double kT, double tau_fs,
                                         int chain_length, int chain_steps, int sy_steps, const float* masses_dev,
                                         float* positions_dev, float* velocities_dev, float* forces_dev, double* chain_dev,
                                         double* energy_dev);

/* NPT: isotropic Martyna-Tobias-Klein barostat with Nose-Hoover chains on the particles and on the box, in the form
 * jax_md.simulate.npt_nose_hoover integrates it.  The box coordinate is eps = ln(V/V0)/3 (V0 = volume of the reference cell
 * cell0), its momentum has the mass 3 (n_atoms + 1) kT tau_b^2; positions are Cartesian and scale with the box.
 * State, SO3LR_B200_NPT_STATE_DOUBLES doubles on the device: [0,18) thermostat chain, [18,36) barostat chain (layout of
 * so3lr_b200_nhc_*), [36] eps, [37] its momentum (eV fs), [38..41] coefficients of the current step, [42] volume.
 * pressure in eV/A^3 (1 bar = 6.241509074e-7).  The context must have the virial enabled and hold the evaluation of the
 * positions passed in (call so3lr_b200_system_compute after enabling it); the cell of the context follows the box, the
 * neighbor lists are kept across the rescaling and rebuilt by the skin test.  cell_out9 (host, optional) receives the
 * cell after the last step.
 * Replaces: jax_md.simulate.npt_nose_hoover as created in so3lr/cli/so3lr_md.py:1089-1107 (barostat tau = dt * nhc_baro,
 *           :1709-1711) and stepped at :1254-1282, where the box is read back with jax_md.simulate.npt_box. */
#define SO3LR_B200_NPT_STATE_DOUBLES 44
SO3LR_B200_API int so3lr_b200_npt_init(void* stream, double* state_dev);
SO3LR_B200_API int so3lr_b200_system_npt(so3lr_b200_system* sys, void* stream, int n_steps, float dt_fs, double kT, double pressure,
                                         double tau_t_fs, double tau_b_fs, int chain_length, int chain_steps, int sy_steps,
                                         const float* masses_dev, float* positions_dev, float* velocities_dev, float* forces_dev,
                                         double* state_dev, const float* cell0_9, float* cell_out9, double* energy_dev);
/* The box-and-chains part of an NPT step alone, for drivers that update the atoms themselves (the decomposed driver does):
 * npt_pre before the force evaluation (half steps of both chains, half kick of the box momentum, the box coordinate moves;
 * leaves the step's coefficients in state[38..41] and multiplies the thermostat's momentum scale into state[1]), npt_post
 * after the atoms' second kick (box half kick, chains' half steps; state[1] = the thermostat's scale).  virial9_dev and
 * kinetic_energy_dev (one double, eV) are totals over all ranks; V0 is the volume of the reference cell; n_atoms the number
 * of atoms of the whole structure.  The atoms' updates with the coefficients c1 = state[38], c2 = state[39], r1 = state[40],
 * r2 = state[41] are  v <- state[1] v;  v <- c1 v + c2 a;  R <- r1 R + r2 v  before, and  v <- c1 v + c2 a  after the
 * evaluation (a = 9.648533212331e-3 F / m). */
SO3LR_B200_API int so3lr_b200_npt_pre(void* stream, double* state_dev, int n_atoms, float dt_fs, double kT, double pressure,
                                      double tau_t_fs, double tau_b_fs, int chain_length, int chain_steps, int sy_steps, double V0,
                                      const double* virial9_dev, const double* kinetic_energy_dev);
SO3LR_B200_API int so3lr_b200_npt_post(void* stream, double* state_dev, int n_atoms, float dt_fs, double kT, double pressure,
                                       double tau_t_fs, double tau_b_fs, int chain_length, int chain_steps, int sy_steps, double V0,
                                       const double* virial9_dev, const double* kinetic_energy_dev);
/* Replaces the cell by a slightly rescaled one without discarding the neighbor lists (the caller has moved the positions
 * with the cell; the next evaluation's skin test decides about a rebuild).  so3lr_b200_system_set_cell discards them. */
SO3LR_B200_API int so3lr_b200_system_rescale_cell(so3lr_b200_system* sys, const float* cell9);

/* Domain-decomposed evaluation of one large periodic structure: every rank owns the atoms of its sub-box and holds
 * copies ("ghosts") of the atoms within the long-range list radius (12 A + skin) of it; the ghosts within one short-range
 * shell (4.5 A + skin) also carry features.  The library evaluates one rank's owned atoms layer by layer; between the
 * calls the caller moves rows between ranks (so3lr_b200/domain.py does it with NCCL send/recv):
 *   dd_begin                  lists (when invalid), ZBL, embeddings
 *   for l = 0,1,2: dd_layer_forward(l)
 *        then (l < 2) the rows of the short-range ghosts in buffers (0, l+1) and (1, l+1) are filled from their owners
 *   dd_heads                  raw partial charges and Hirshfeld ratios of the owned atoms
 *        (caller: global sum of the raw charges -> charge conservation; halo exchange of q and h to all ghosts)
 *   dd_pair                   Coulomb + dispersion of every pair that involves an owned atom (half of each pair energy is
 *                             booked here); returns the sum of dE/dq over the owned atoms
 *        (caller: sum of that number over all ranks)
 *   dd_heads_backward         energy of the owned atoms, cotangents of the final features
 *   for l = 2,1,0: dd_layer_backward_post(l)
 *        then the rows of the short-range ghosts in buffers (2) and (3) are filled from their owners
 *        dd_layer_backward_attn(l)
 *   dd_forces                 forces on the owned atoms, complete: no ghost forces exist in this scheme
 * Because the attention kernels gather both directions of every edge towards the owned atom, no rank ever computes on
 * behalf of a ghost: the work per rank is that of its owned atoms.
 * The context is created with so3lr_b200_system_create for the largest local atom count it will see (n_graphs = 1,
 * cutoff_lr > 0); dd_set_atoms installs a new local atom set and invalidates the neighbor lists.
 * Local atom order: [0, shells4[0]) owned, [shells4[0], shells4[1]) ghosts within one short-range shell of the sub-box,
 * then the remaining ghosts up to shells4[3] = n_local (shells4[2] is ignored).  `cell9` is the rank's local periodic
 * cell; along the decomposed direction it must exceed the extent of the local atoms by more than the list radius, so
 * that no pair is found through the wrap.  Z_local_dev: device int32; all other pointers are device pointers.
 * dd_buffer: device address and row length (floats) of an internal per-atom array, rows in local atom order:
 *   which 0: features x of `layer` (0..3), 1: equivariant features ev of `layer`, 2 / 3: cotangents of the current
 *   layer's attention outputs (128 / 24 floats per row).
 * Replaces: nothing in the reference (it has no multi-device path); the decomposition follows the cutoffs of
 * so3lr/potential.py:17-29 and so3lr/jaxmd_utils.py:96-121. */
SO3LR_B200_API int so3lr_b200_dd_set_atoms(so3lr_b200_system* sys, int n_local, const int32_t* shells4, const int32_t* Z_local_dev,
                                           const float* cell9);
SO3LR_B200_API int so3lr_b200_dd_begin(so3lr_b200_system* sys, void* stream, const float* R_local_dev);
SO3LR_B200_API int so3lr_b200_dd_layer_forward(so3lr_b200_system* sys, void* stream, int layer);
SO3LR_B200_API int so3lr_b200_dd_heads(so3lr_b200_system* sys, void* stream, float* q_raw_owned_dev, float* h_owned_dev);
SO3LR_B200_API int so3lr_b200_dd_pair(so3lr_b200_system* sys, void* stream, const float* R_local_dev, const float* q_local_dev,
                                      const float* h_local_dev, double* gq_sum_dev);
/* Reciprocal-space part in a decomposed evaluation (so3lr_b200_system_set_kspace on every rank's context first, with the same
 * arguments).  so3lr_b200_dd_kspace_cell gives the cell of the WHOLE structure (the context's own cell is the rank's local one)
 * and its total charge; call it again when the cell is rescaled.  Between so3lr_b200_dd_pair and so3lr_b200_dd_heads_backward:
 * _accumulate forms the owned atoms' share of the charge mesh (or of the structure factors) and names the buffer, the caller
 * sums that buffer over the ranks in place (an all-reduce of *n_floats floats: the one exchange step of this part), and _finish
 * transforms it and adds potential energies, dE/dq and forces of the owned atoms; gq_sum_dev then holds the sum of dE/dq over
 * the owned atoms including the pair part (it replaces the value so3lr_b200_dd_pair returned).  The strain derivative of the whole
 * reciprocal sum is added on the rank that passes add_strain != 0 (exactly one rank should). */
SO3LR_B200_API int so3lr_b200_dd_kspace_cell(so3lr_b200_system* sys, const float* cell9_global, float total_charge);
SO3LR_B200_API int so3lr_b200_dd_kspace_accumulate(so3lr_b200_system* sys, void* stream, const float* R_local_dev, const float* q_local_dev,
                                                   float** buffer_dev, int64_t* n_floats);
SO3LR_B200_API int so3lr_b200_dd_kspace_finish(so3lr_b200_system* sys, void* stream, const float* R_local_dev, const float* q_local_dev,
                                               int add_strain, double* gq_sum_dev);
SO3LR_B200_API int so3lr_b200_dd_heads_backward(so3lr_b200_system* sys, void* stream, const double* gq_sum_all_dev,
                                                int64_t n_atoms_all, double* energy_owned_dev);
SO3LR_B200_API int so3lr_b200_dd_layer_backward_post(so3lr_b200_system* sys, void* stream, int layer);
SO3LR_B200_API int so3lr_b200_dd_layer_backward_attn(so3lr_b200_system* sys, void* stream, int layer);
SO3LR_B200_API int so3lr_b200_dd_forces(so3lr_b200_system* sys, void* stream, float* F_owned_dev);
SO3LR_B200_API int so3lr_b200_dd_buffer(so3lr_b200_system* sys, int which, int layer, float** ptr, int* row_floats);

/* Halo packing for the exchanges between ranks: gather rows idx[r] (r < n_rows; 64-bit indices on the device) of up to four
 * row-major float arrays with `widths[t]` floats per row side by side into buf[n_rows][sum of widths], and the reverse
 * (scatter the columns of buf back into rows idx[r] of the arrays).  One launch per call on the device of the current
 * context; no counterpart in the reference (it has no multi-device path). */
SO3LR_B200_API int so3lr_b200_pack_rows(void* stream, int n_arrays, const float* const* arrays_dev, const int* widths, const int64_t* idx_dev,
                                        int64_t n_rows, float* buf_dev);
SO3LR_B200_API int so3lr_b200_unpack_rows(void* stream, int n_arrays, float* const* arrays_dev, const int* widths, const int64_t* idx_dev,
                                          int64_t n_rows, const float* buf_dev);

/* Optional timing of kernel groups with CUDA events recorded on the launching stream.  `profile(sys, 1)` starts a
 * fresh recording; `profile_read` synchronises the device, returns the number of groups and fills, per group, the
 * summed device time in ms, the number of timed launches and a static name.  No counterpart in the reference
 * (it only measures wall-clock time per MD cycle, so3lr/cli/so3lr_md.py:1813-1839). */
SO3LR_B200_API int so3lr_b200_system_profile(so3lr_b200_system* sys, int enable);
SO3LR_B200_API int so3lr_b200_system_profile_read(so3lr_b200_system* sys, int max_groups, float* ms_total, int64_t* launches,
                                                  const char** names);

/* Pair list without any device allocation.  No counterpart in the reference: it exists for callers that cannot call
 * cudaMalloc at all, such as an XLA custom-call handler (XLA's allocator already holds most of the GPU's memory, so an
 * allocation made inside the handler may fail and, if it succeeds, stalls the whole device) or a host program that
 * serves all GPU memory from its own fixed arena.  The only memory used besides the arguments is a 128 KiB scratch
 * array that is part of the library image on every GPU that loads it; that fixes the limit of
 * SO3LR_B200_NOALLOC_MAX_ATOMS atoms (larger systems return SO3LR_B200_TOO_LARGE; use
 * so3lr_b200_system_export_list for them).
 *   positions_dev: n_atoms x 3 float32 on the CURRENT device (cudaGetDevice); cell: HOST pointer to 9 floats (rows =
 *   lattice vectors, each perpendicular width >= 2 * r_cutoff) or NULL for free space; ordered = 1 keeps i < j only.
 *   idx_dev: (2, capacity) int32, pairs grouped by centre with ascending neighbour index, unused slots = n_atoms;
 *   count_dev / overflow_dev: DEVICE words that receive the number of pairs found and whether it exceeds capacity.
 * Work is only enqueued on `stream`; nothing is read back.  The first call on a device looks up the device address of
 * the scratch array (cudaGetSymbolAddress); make that first call before any stream capture begins.  The scratch is
 * shared by all calls on a device: calls whose kernels could overlap on the GPU (different streams or threads) race
 * and must be serialised by the caller.  It needs no clearing between calls. */
#define SO3LR_B200_NOALLOC_MAX_ATOMS 16384
SO3LR_B200_API int so3lr_b200_neighbor_list_noalloc(void* stream, int n_atoms, const float* positions_dev, const float* cell,
                                                    float r_cutoff, int ordered, int32_t* idx_dev, int64_t capacity,
                                                    int64_t* count_dev, int* overflow_dev);

/* Host-callable pieces of the device math, exported for the CPU tests (no GPU needed). */
/* 64-bit total of a device array of per-row pair counts, formed the way the list builder forms it ahead of its 32-bit
 * offset scan; returns SO3LR_B200_TOO_LARGE when the offsets of such a list would leave the int32 range (the builder then
 * refuses the list before filling it).  Test support for the capacity protocol of partition.neighbor_list
 * (so3lr/cli/so3lr_md.py:836-877). */
SO3LR_B200_API int so3lr_b200_list_row_total(void* stream, const int32_t* row_count_dev, int n_rows, int64_t* total_host);

SO3LR_B200_API void so3lr_b200_host_sph_harm(float x, float y, float z, float* y24);
SO3LR_B200_API void so3lr_b200_host_sph_harm_vjp(float x, float y, float z, const float* g24, float* g3);
SO3LR_B200_API void so3lr_b200_host_pair_terms(float r, int zi, int zj, float qi, float qj, float hi, float hj, float cutoff_lr,
                                float damping, float* out8);
/* out4 = dispersion energy, d/dr, d/dh_i, d/dh_j of one pair as the pair kernels evaluate it (hand-derived partials) */
/* Host-only check of the direct Ewald sum's tile decomposition for an index grid: counts4 = number of tiles, of groups, largest
 * group, inconsistencies found; weight_sum = sum of the slot weights (n1 n2 n3 - 1 when every non-zero index is counted once). */
SO3LR_B200_API int so3lr_b200_host_kspace_tiles(int n1, int n2, int n3, int64_t* counts4, double* weight_sum);
/* out2 = chi(r), d chi / d r of the Coulomb pair function; smearing > 0 takes the reciprocal-space part out of it */
SO3LR_B200_API void so3lr_b200_host_coulomb_chi(float r, float cutoff_lr, float smearing, float* out2);
SO3LR_B200_API void so3lr_b200_host_dispersion_fast(float r, int zi, int zj, float hi, float hj, float cutoff_lr, float damping,
                                                    float* out4);
SO3LR_B200_API void so3lr_b200_host_zbl(const float* blob_host, float r, int zi, int zj, float* out2);
SO3LR_B200_API void so3lr_b200_host_radial_filter(const float* blob_host, int layer, double r, double* w256, double* dw256);
/* the same filters through the 64-term Chebyshev expansion that the tiled tensor-core attention kernels contract on the fly */
SO3LR_B200_API void so3lr_b200_host_radial_filter_chebyshev(const float* blob_host, int layer, double r, double* w256, double* dw256);

#ifdef __cplusplus
}
#endif
#endif /* SO3LR_B200_H_ */

// Device-resident, kernel-ready form of the SO3LR weights (built once per handle from the packed blob).
#pragma once
#include <vector>

#include "common.cuh"
#include "pair_terms.cuh"

namespace so3lr {

struct LayerDev {
  const float* projT;   // [5][4][32 j][32 i]   forward projection  (out_i = sum_j W[h][i][j] x[h][j])
  const float* proj;    // [5][4][32 i][32 j]   as stored; used by the backward projection
  const float* table;   // [kTableGrid-1][4][256] radial filters per interval: value, h*slope, value difference, h*slope at the far knot; (w1 | w2)
  // Operand image of the tiled tensor-core attention kernels (attention_tc.cu), copied verbatim into shared memory:
  // Chebyshev coefficients of both radial filters (the tied output biases folded into the constant term) and the second
  // spherical layer, each as FP16 hi / 2048-scaled-lo pairs in 8 x 8 core-matrix order (kTcImageBytes bytes)
  const unsigned char* tc_img;
  const unsigned char* tc_img_fwd;   // the same numbers with K contiguous per output feature (forward kernel: K-major B operands)
  const float* sph1_k;  // [2][4][32]   spherical filter, first layer kernel (filter, invariant, hidden)
  const float* sph1_b;  // [2][32]
  const float* sph2_k;  // [2][32][128] second layer kernel (filter, hidden, feature); bias is folded into `table`
  const float *ln1_s, *ln1_b, *ln2_s, *ln2_b;
  const float *res1_k, *res1_kT, *res1_b, *res2_k, *res2_kT, *res2_b;   // [in][out] and transposed
  const float *ex_xx, *ex_xxT;  // [128][128] features -> features
  // the same dense kernels as tensor-core B operands: FP16 hi / scaled-lo pairs in mma.m16n8k16 fragment order,
  // [K/16][N/8][32 lanes] x {b0hi, b1hi, b0lo, b1lo} (see atom_kernels_mma.cu); "T" = transposed kernel (reverse pass)
  const uint4 *res1_f, *res1T_f, *res2_f, *res2T_f, *exxx_f, *exxxT_f;
  // q/k/v projections of this layer as 20 blocks (projection w = 0..4, head h = 0..3) of 32 x 32, fragment order
  // [w*4+h][2][4][32]: proj_f for out_i = sum_j W[i][j] x_j, projT_f for the reverse contraction over i
  const uint4 *proj_f, *projT_f;
  // B operands of the tcgen05 dense-block kernels (dense_tc.cu): FP16 hi matrix then 2048-scaled lo matrix, K contiguous,
  // element (k, n) at (k/8) * 16 N + (n/8) * 128 + (n%8) * 16 + (k%8) * 2 bytes.  res1/res2/exxx: [128 x 128] forward and
  // transposed; proj_u: five blocks of 16 KB: heads 0, 1, 2 as [K = 32 inputs of the head][N = 128 = projections 0..3, output i], the fifth
  // projection of all heads as four [32 x 32] blocks, head 3;
  // projT_u: per projection w and head h the [K = 32 outputs i][N = 32 inputs j] block (20 x 4,096 bytes)
  const unsigned char *res1_u, *res2_u, *exxx_u, *res1T_u, *res2T_u, *exxxT_u, *proj_u, *projT_u;
  const float* ex_xg;           // [128][4]   features -> gates
  const float* ex_ix;           // [4][128]   invariants -> features
  const float* ex_ig;           // [4][4]     invariants -> gates
  const float* ex_bx;           // [128]
  const float* ex_bg;           // [4]
  int has_spherical;            // layer 0 sees ev = 0: its spherical filter is a constant folded into `table`
};

struct ModelDev {
  const float* embed_z;   // [119][128], already divided by sqrt(3)
  LayerDev layer[kNumLayers];
  // energy head
  const float *e_reg_k, *e_reg_kT, *e_reg_b, *e_fin_k, *e_scale, *e_offset;
  float e_fin_b;
  // partial charge head
  const float *q_embed, *q_reg_k, *q_reg_kT, *q_reg_b, *q_fin_k;
  float q_fin_b;
  // Hirshfeld head
  const float *h_embed0, *h_embed1, *h_reg_k, *h_reg_kT, *h_reg_b, *h_fin_k, *h_fin_kT, *h_fin_b;
  const uint4 *e_reg_f, *e_regT_f, *q_reg_f, *q_regT_f, *h_reg_f, *h_regT_f, *h_fin_f, *h_finT_f;   // fragment-order copies
  const unsigned char *e_reg_u, *e_regT_u, *q_reg_u, *q_regT_u, *h_reg_u, *h_regT_u, *h_fin_u, *h_finT_u;   // tcgen05 operand images
  // charge / spin embeddings (only evaluated when a graph carries charge or unpaired electrons)
  const float *cs_embed_q[2], *cs_embed_k[2], *cs_embed_v[2], *cs_res0[2], *cs_res1[2];
  ZblParams zbl;
};

// Builds every derived array on the host (double precision where it matters) and uploads it.
// `owned` receives the device allocations so the handle can free them.
int build_model(const float* blob, size_t n_floats, ModelDev* out, std::vector<void*>* owned);

// Chebyshev expansion of the radial filters used by the tiled attention kernels: w_c(r) = sum_m coef[m][c] T_m(t(r)) with
// t = kChebA * exp(-kChebHalfGamma * r) + kChebB on r in [0, 4.5] (host evaluation in double; for tests)
void radial_filter_chebyshev(const float* blob, int layer, double r, double* w256, double* dw256);

// host helper exposed for tests: evaluate the radial-filter table entry (value, derivative) directly
void radial_filter_reference(const float* blob, int layer, double r, double* w256, double* dw256);

}  // namespace so3lr

// Offsets (in floats) into the packed SO3LR parameter blob.  The order is the one written by
// so3lr_b200/params/pack_params.py (which walks the flax tree of so3lr/params/params.pkl of the reference).
#pragma once
#include <cstddef>

namespace so3lr {

constexpr int kNumLayers = 3;
constexpr int kF = 128;        // features
constexpr int kHeads = 4;
constexpr int kHeadDim = 32;
constexpr int kMTot = 24;      // 3+5+7+9 spherical components
constexpr int kNumRbf = 32;
constexpr int kZEmbed = 119;
constexpr int kZHead = 100;
constexpr int kProj = 5 * kF;  // q1,k1,v1,q2,k2

struct ChargeSpinOffsets { size_t embed_q, embed_k, embed_v, res0, res1; };

struct LayerOffsets {
  size_t W[5];                                    // Wq1 Wk1 Wv1 Wq2 Wk2, each (4,32,32)
  size_t rad_l1_k[2], rad_l1_b[2], rad_l2_k[2], rad_l2_b[2];
  size_t sph_l1_k[2], sph_l1_b[2], sph_l2_k[2], sph_l2_b[2];
  size_t exch_k, exch_b, ln1_s, ln1_b, ln2_s, ln2_b, res1_k, res1_b, res2_k, res2_b;
};

struct BlobOffsets {
  size_t embed_z;
  ChargeSpinOffsets cs[2];
  LayerOffsets layer[kNumLayers];
  size_t e_reg_k, e_reg_b, e_fin_k, e_fin_b, e_scale, e_offset;
  size_t zbl[10];                                 // a1..a4 c1..c4 p d (raw, softplus applied at use)
  size_t q_embed, q_reg_k, q_reg_b, q_fin_k, q_fin_b;
  size_t h_embed0, h_embed1, h_reg_k, h_reg_b, h_fin_k, h_fin_b;
  size_t total;
};

inline BlobOffsets blob_offsets() {
  BlobOffsets o{};
  size_t p = 0;
  auto take = [&](size_t n) { size_t r = p; p += n; return r; };
  o.embed_z = take(kZEmbed * kF);
  for (int e = 0; e < 2; ++e) {
    o.cs[e].embed_q = take(kZEmbed * kF);
    o.cs[e].embed_k = take(2 * kF);
    o.cs[e].embed_v = take(2 * kF);
    o.cs[e].res0 = take(kF * kF);
    o.cs[e].res1 = take(kF * kF);
  }
  for (int l = 0; l < kNumLayers; ++l) {
    LayerOffsets& L = o.layer[l];
    for (int w = 0; w < 5; ++w) L.W[w] = take(kHeads * kHeadDim * kHeadDim);
    for (int f = 0; f < 2; ++f) {
      L.rad_l1_k[f] = take(kNumRbf * kF); L.rad_l1_b[f] = take(kF);
      L.rad_l2_k[f] = take(kF * kF);      L.rad_l2_b[f] = take(kF);
    }
    for (int f = 0; f < 2; ++f) {
      L.sph_l1_k[f] = take(4 * 32); L.sph_l1_b[f] = take(32);
      L.sph_l2_k[f] = take(32 * kF); L.sph_l2_b[f] = take(kF);
    }
    L.exch_k = take(132 * 132); L.exch_b = take(132);
    L.ln1_s = take(kF); L.ln1_b = take(kF); L.ln2_s = take(kF); L.ln2_b = take(kF);
    L.res1_k = take(kF * kF); L.res1_b = take(kF); L.res2_k = take(kF * kF); L.res2_b = take(kF);
  }
  o.e_reg_k = take(kF * kF); o.e_reg_b = take(kF); o.e_fin_k = take(kF); o.e_fin_b = take(1);
  o.e_scale = take(kZEmbed); o.e_offset = take(kZEmbed);
  for (int k = 0; k < 10; ++k) o.zbl[k] = take(1);
  o.q_embed = take(kZHead); o.q_reg_k = take(kF * kF); o.q_reg_b = take(kF); o.q_fin_k = take(kF); o.q_fin_b = take(1);
  o.h_embed0 = take(kZHead); o.h_embed1 = take(kZHead * 64); o.h_reg_k = take(kF * 64); o.h_reg_b = take(64);
  o.h_fin_k = take(64 * 64); o.h_fin_b = take(64);
  o.total = p;
  return o;
}

}  // namespace so3lr

// Per-atom dense blocks of the SO3krates layers and the output heads, forward and hand-written backward.
// A CTA of 128 threads owns a tile of 64 atoms.  Activations live in shared memory feature-major
// ([feature][atom], row stride 65 floats) so that one tile GEMM's output is the next one's operand;
// the 128x128 weight matrices (L2-resident, 64 KB each) are streamed through a 32-row staging buffer.
#include "kernels.h"

namespace so3lr {

namespace {

constexpr int TA = 64;     // atoms per tile
constexpr int TS = 65;     // shared-memory row stride (floats)
constexpr int NT = 128;    // threads per CTA
constexpr int WCH = 32;    // weight rows staged per chunk

__device__ __forceinline__ float inv_weight(int l) {
  return l == 0 ? 0.5773502691896258f : (l == 1 ? 0.4472135954999579f : (l == 2 ? 0.3779644730092272f : 0.3333333333333333f));
}

// global [n][F] rows row0.. -> smem T[f*TS + r]
template <int F>
__device__ __forceinline__ void load_tile_T(float* T, const float* __restrict__ src, int row0, int n) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < TA; r += NT / 32) {
    int a = row0 + r;
#pragma unroll
    for (int c = 0; c < F / 32; ++c) {
      float v = (a < n) ? src[(size_t)a * F + lane + 32 * c] : 0.f;
      T[(lane + 32 * c) * TS + r] = v;
    }
  }
}
template <int F>
__device__ __forceinline__ void store_tile_T(float* __restrict__ dst, const float* T, int row0, int n) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < TA; r += NT / 32) {
    int a = row0 + r;
    if (a >= n) continue;
#pragma unroll
    for (int c = 0; c < F / 32; ++c) dst[(size_t)a * F + lane + 32 * c] = T[(lane + 32 * c) * TS + r];
  }
}

// acc[i][j] += sum_k A[k][ty+8i] * W[k][tx+16j]   (rows ty+8i, cols tx+16j), K = rows of W, NOUT = cols
template <int K, int NOUT>
__device__ __forceinline__ void gemm_tile(const float* At, const float* __restrict__ Wg, float* Wsm, float (&acc)[8][NOUT / 16]) {
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  for (int k0 = 0; k0 < K; k0 += WCH) {
    __syncthreads();
    for (int idx = threadIdx.x * 4; idx < WCH * NOUT; idx += NT * 4) {
      *reinterpret_cast<float4*>(Wsm + idx) = *reinterpret_cast<const float4*>(Wg + (size_t)k0 * NOUT + idx);
    }
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < WCH; ++kk) {
      float a[8], b[NOUT / 16];
      const float* ap = At + (k0 + kk) * TS + ty;
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = ap[8 * i];
      const float* bp = Wsm + kk * NOUT + tx;
#pragma unroll
      for (int j = 0; j < NOUT / 16; ++j) b[j] = bp[16 * j];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < NOUT / 16; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }
}

template <int NJ>
__device__ __forceinline__ void zero_acc(float (&acc)[8][NJ]) {
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[i][j] = 0.f;
}

// per-row LayerNorm statistics over 128 features held feature-major in T
__device__ __forceinline__ void ln_stats(const float* T, int r, float& mean, float& rstd) {
  float s = 0.f;
  for (int k = 0; k < kF; ++k) s += T[k * TS + r];
  mean = s * (1.f / kF);
  float v = 0.f;
  for (int k = 0; k < kF; ++k) { float d = T[k * TS + r] - mean; v = fmaf(d, d, v); }
  rstd = rsqrtf(v * (1.f / kF) + kLnEps);
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// embedding
// ------------------------------------------------------------------------------------------------
__global__ void embed_kernel(const float* __restrict__ embed, const int* __restrict__ Z, int n, float* __restrict__ x) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)n * kF) return;
  int a = (int)(idx / kF), f = (int)(idx % kF);
  int z = Z[a];
  z = z < 0 ? 0 : (z >= kZEmbed ? kZEmbed - 1 : z);
  x[idx] = embed[z * kF + f];
}

// ------------------------------------------------------------------------------------------------
// q/k/v projections: out[n][w*128 + h*32 + i] = sum_j W[w][h][i][j] x[n][h*32 + j]
// ------------------------------------------------------------------------------------------------
constexpr int PROJ_TILE = 32;
__global__ void __launch_bounds__(640) proj_fwd_kernel(const float* __restrict__ WT, const float* __restrict__ x, int n,
                                                       float* __restrict__ out) {
  __shared__ float xs[PROJ_TILE * kF];
  const int t = threadIdx.x;            // output column 0..639
  const int wh = t >> 5, i = t & 31;    // (w*4+h), i
  const int h = wh & 3;
  float w[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) w[j] = WT[(wh * 32 + j) * 32 + i];
  for (int row0 = blockIdx.x * PROJ_TILE; row0 < n; row0 += gridDim.x * PROJ_TILE) {
    __syncthreads();
    for (int idx = t; idx < PROJ_TILE * kF; idx += 640) {
      int a = row0 + idx / kF;
      xs[idx] = a < n ? x[(size_t)row0 * kF + idx] : 0.f;
    }
    __syncthreads();
    int rows = min(PROJ_TILE, n - row0);
    for (int r = 0; r < rows; ++r) {
      const float* xr = xs + r * kF + h * 32;
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) s = fmaf(w[j], xr[j], s);
      out[(size_t)(row0 + r) * kProj + t] = s;
    }
  }
}

// gx[n][h*32+j] (+)= sum_w sum_i W[w][h][i][j] g[n][w*128+h*32+i]
__global__ void __launch_bounds__(512) proj_bwd_kernel(const float* __restrict__ W, const float* __restrict__ g, int n,
                                                       float* __restrict__ gx, int accumulate) {
  extern __shared__ float sm[];
  float* Ws = sm;                     // 20480 floats
  float* gs = sm + 5 * 4 * 32 * 32;   // PROJ_TILE * 640
  const int t = threadIdx.x;
  for (int idx = t; idx < 5 * 4 * 32 * 32; idx += 512) Ws[idx] = W[idx];
  const int c = t & 127, grp = t >> 7;   // feature column h*32+j ; atom sub-group
  const int h = c >> 5, j = c & 31;
  for (int row0 = blockIdx.x * PROJ_TILE; row0 < n; row0 += gridDim.x * PROJ_TILE) {
    __syncthreads();
    for (int idx = t; idx < PROJ_TILE * kProj; idx += 512) {
      int a = row0 + idx / kProj;
      gs[idx] = a < n ? g[(size_t)row0 * kProj + idx] : 0.f;
    }
    __syncthreads();
    for (int r = grp; r < PROJ_TILE; r += 4) {
      int a = row0 + r;
      if (a >= n) break;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 5; ++w) {
        const float* gp = gs + r * kProj + w * 128 + h * 32;
        const float* wp = Ws + ((w * 4 + h) * 32) * 32 + j;
#pragma unroll 8
        for (int i = 0; i < 32; ++i) s = fmaf(wp[i * 32], gp[i], s);
      }
      size_t o = (size_t)a * kF + c;
      gx[o] = accumulate ? gx[o] + s : s;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// post-attention block, forward:
//   x1 = LN1(xa); x2 = x1 + Dense2(silu(Dense1(silu(x1)))); [yx, gate] = Dense132([x2, inv(ev1)])
//   x3 = x2 + yx; ev2 = ev1 * (1 + gate_l); x4 = LN2(x3)
// saves z1 (hidden pre-activation), x3 and gate for the backward pass
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NT) atom_post_fwd_kernel(LayerDev L, int n, const float* __restrict__ xa,
                                                           const float* __restrict__ ev1, float* __restrict__ z1_out,
                                                           float* __restrict__ x3_out,
                                                           float* __restrict__ gate_out, float* __restrict__ x4_out,
                                                           float* __restrict__ ev2_out) {
  extern __shared__ float sm[];
  float* At = sm;                  // 128*TS
  float* Bt = At + kF * TS;        // 128*TS
  float* Wsm = Bt + kF * TS;       // WCH*128
  float* invs = Wsm + WCH * kF;    // 64*4
  float* gates = invs + TA * 4;    // 64*4
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int row0 = blockIdx.x * TA;

  load_tile_T<kF>(At, xa, row0, n);
  __syncthreads();
  if (tid < TA) {
    float m, rs;
    ln_stats(At, tid, m, rs);
    for (int k = 0; k < kF; ++k) {
      float v = (At[k * TS + tid] - m) * rs * L.ln1_s[k] + L.ln1_b[k];
      At[k * TS + tid] = v;
      Bt[k * TS + tid] = silu_f(v);
    }
    // per-degree invariants of ev1
    int a = row0 + tid;
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    if (a < n) {
      for (int m2 = 0; m2 < kMTot; ++m2) { float e = ev1[(size_t)a * kMTot + m2]; s[degree_of(m2)] += e * e; }
    }
    for (int l = 0; l < 4; ++l) invs[tid * 4 + l] = s[l] * inv_weight(l);
  }
  __syncthreads();
  float acc[8][8];
  // hidden layer
  zero_acc(acc);
  gemm_tile<kF, kF>(Bt, L.res1_k, Wsm, acc);
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int c = tx + 16 * j;
    float b = L.res1_b[c];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int r = ty + 8 * i;
      float z = acc[i][j] + b;
      if (row0 + r < n) z1_out[(size_t)(row0 + r) * kF + c] = z;
      Bt[c * TS + r] = silu_f(z);
    }
  }
  zero_acc(acc);
  gemm_tile<kF, kF>(Bt, L.res2_k, Wsm, acc);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int c = tx + 16 * j;
    float b = L.res2_b[c];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int r = ty + 8 * i;
      float v = At[c * TS + r] + acc[i][j] + b;
      At[c * TS + r] = v;
    }
  }
  // exchange: features -> features
  zero_acc(acc);
  gemm_tile<kF, kF>(At, L.ex_xx, Wsm, acc);   // first barrier inside orders the At writes above
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int c = tx + 16 * j;
    float b = L.ex_bx[c];
    float w0 = L.ex_ix[0 * kF + c], w1 = L.ex_ix[1 * kF + c], w2 = L.ex_ix[2 * kF + c], w3 = L.ex_ix[3 * kF + c];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int r = ty + 8 * i;
      const float* iv = invs + r * 4;
      float y = acc[i][j] + b + iv[0] * w0 + iv[1] * w1 + iv[2] * w2 + iv[3] * w3;
      float v = At[c * TS + r] + y;
      Bt[c * TS + r] = v;
      if (row0 + r < n) x3_out[(size_t)(row0 + r) * kF + c] = v;
    }
  }
  // gates: 4 extra output columns of the exchange layer
  {
    int r = tid & 63, g0 = tid >> 6;
    for (int g = g0; g < 4; g += 2) {
      float s = L.ex_bg[g];
      for (int k = 0; k < kF; ++k) s = fmaf(At[k * TS + r], L.ex_xg[k * 4 + g], s);
      for (int l = 0; l < 4; ++l) s = fmaf(invs[r * 4 + l], L.ex_ig[l * 4 + g], s);
      gates[r * 4 + g] = s;
      if (row0 + r < n) gate_out[(size_t)(row0 + r) * 4 + g] = s;
    }
  }
  __syncthreads();
  if (tid < TA) {
    float m, rs;
    ln_stats(Bt, tid, m, rs);
    for (int k = 0; k < kF; ++k) Bt[k * TS + tid] = (Bt[k * TS + tid] - m) * rs * L.ln2_s[k] + L.ln2_b[k];
    int a = row0 + tid;
    if (a < n) {
      for (int m2 = 0; m2 < kMTot; ++m2) {
        float e = ev1[(size_t)a * kMTot + m2];
        ev2_out[(size_t)a * kMTot + m2] = e * (1.f + gates[tid * 4 + degree_of(m2)]);
      }
    }
  }
  __syncthreads();
  store_tile_T<kF>(x4_out, Bt, row0, n);
}

// ------------------------------------------------------------------------------------------------
// post-attention block, backward.  in: g4 = dL/dx4, gev2 = dL/dev2 ; out: g_xa = dL/dxa, gev1 = dL/dev1
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NT) atom_post_bwd_kernel(LayerDev L, int n, const float* __restrict__ xa,
                                                           const float* __restrict__ ev1, const float* __restrict__ z1,
                                                           const float* __restrict__ x3, const float* __restrict__ gate,
                                                           const float* __restrict__ g4, const float* __restrict__ gev2,
                                                           float* __restrict__ g_xa, float* __restrict__ gev1) {
  extern __shared__ float sm[];
  float* At = sm;
  float* Bt = At + kF * TS;
  float* Ct = Bt + kF * TS;
  float* Wsm = Ct + kF * TS;
  float* ggate = Wsm + WCH * kF;   // 64*4
  float* ginv = ggate + TA * 4;    // 64*4
  float* rstd1 = ginv + TA * 4;    // 64
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int row0 = blockIdx.x * TA;

  load_tile_T<kF>(At, x3, row0, n);
  load_tile_T<kF>(Bt, g4, row0, n);
  load_tile_T<kF>(Ct, xa, row0, n);
  __syncthreads();
  if (tid < TA) {
    const int r = tid, a = row0 + r;
    // LayerNorm-2 backward: Bt <- g3
    float m, rs;
    ln_stats(At, r, m, rs);
    float s1 = 0.f, s2 = 0.f;
    for (int k = 0; k < kF; ++k) {
      float xh = (At[k * TS + r] - m) * rs;
      float gy = Bt[k * TS + r] * L.ln2_s[k];
      s1 += gy; s2 = fmaf(gy, xh, s2);
    }
    s1 *= (1.f / kF); s2 *= (1.f / kF);
    for (int k = 0; k < kF; ++k) {
      float xh = (At[k * TS + r] - m) * rs;
      float gy = Bt[k * TS + r] * L.ln2_s[k];
      Bt[k * TS + r] = rs * (gy - s1 - xh * s2);
    }
    // gate cotangents
    float gg[4] = {0.f, 0.f, 0.f, 0.f};
    if (a < n)
      for (int m2 = 0; m2 < kMTot; ++m2) gg[degree_of(m2)] += gev2[(size_t)a * kMTot + m2] * ev1[(size_t)a * kMTot + m2];
    for (int l = 0; l < 4; ++l) ggate[r * 4 + l] = gg[l];
    // LayerNorm-1 forward statistics: Ct <- normalised xa (no affine)
    ln_stats(Ct, r, m, rs);
    rstd1[r] = rs;
    for (int k = 0; k < kF; ++k) Ct[k * TS + r] = (Ct[k * TS + r] - m) * rs;
  }
  __syncthreads();
  // cotangent of the invariants: ginv[r][l] = sum_c g3[r][c] Wix[l][c] + sum_g ggate[r][g] Wig[l][g]
  {
    int r = tid & 63, l0 = tid >> 6;
    for (int l = l0; l < 4; l += 2) {
      float s = 0.f;
      for (int c = 0; c < kF; ++c) s = fmaf(Bt[c * TS + r], L.ex_ix[l * kF + c], s);
      for (int g = 0; g < 4; ++g) s = fmaf(ggate[r * 4 + g], L.ex_ig[l * 4 + g], s);
      ginv[r * 4 + l] = s;
    }
  }
  float acc[8][8];
  zero_acc(acc);
  gemm_tile<kF, kF>(Bt, L.ex_xxT, Wsm, acc);
  // g_x2 = g3 + g3 Wxx^T + ggate Wxg^T   -> At
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int c = tx + 16 * j;
    float w0 = L.ex_xg[c * 4 + 0], w1 = L.ex_xg[c * 4 + 1], w2 = L.ex_xg[c * 4 + 2], w3 = L.ex_xg[c * 4 + 3];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int r = ty + 8 * i;
      const float* gg = ggate + r * 4;
      At[c * TS + r] = Bt[c * TS + r] + acc[i][j] + gg[0] * w0 + gg[1] * w1 + gg[2] * w2 + gg[3] * w3;
    }
  }
  __syncthreads();
  if (tid < TA) {
    int a = row0 + tid;
    if (a < n)
      for (int m2 = 0; m2 < kMTot; ++m2) {
        int l = degree_of(m2);
        float e = ev1[(size_t)a * kMTot + m2];
        gev1[(size_t)a * kMTot + m2] = gev2[(size_t)a * kMTot + m2] * (1.f + gate[(size_t)a * 4 + l]) +
                                        ginv[tid * 4 + l] * 2.f * e * inv_weight(l);
      }
  }
  // residual MLP backward
  zero_acc(acc);
  gemm_tile<kF, kF>(At, L.res2_kT, Wsm, acc);
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int c = tx + 16 * j;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int r = ty + 8 * i;
      float z = (row0 + r < n) ? z1[(size_t)(row0 + r) * kF + c] : 0.f;
      Bt[c * TS + r] = acc[i][j] * dsilu_f(z);
    }
  }
  zero_acc(acc);
  gemm_tile<kF, kF>(Bt, L.res1_kT, Wsm, acc);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int c = tx + 16 * j;
    float s = L.ln1_s[c], b = L.ln1_b[c];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int r = ty + 8 * i;
      float x1 = Ct[c * TS + r] * s + b;
      At[c * TS + r] += acc[i][j] * dsilu_f(x1);   // g_x1
    }
  }
  __syncthreads();
  if (tid < TA) {
    const int r = tid;
    float rs = rstd1[r];
    float s1 = 0.f, s2 = 0.f;
    for (int k = 0; k < kF; ++k) {
      float gy = At[k * TS + r] * L.ln1_s[k];
      s1 += gy; s2 = fmaf(gy, Ct[k * TS + r], s2);
    }
    s1 *= (1.f / kF); s2 *= (1.f / kF);
    for (int k = 0; k < kF; ++k) {
      float gy = At[k * TS + r] * L.ln1_s[k];
      At[k * TS + r] = rs * (gy - s1 - Ct[k * TS + r] * s2);
    }
  }
  __syncthreads();
  store_tile_T<kF>(g_xa, At, row0, n);
}

// ------------------------------------------------------------------------------------------------
// output heads, forward: per-atom NN energy, raw partial charge, Hirshfeld ratio
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NT) heads_fwd_kernel(ModelDev M, int n, const int* __restrict__ Z, const float* __restrict__ x,
                                                       float* __restrict__ ze, float* __restrict__ zq, float* __restrict__ zh,
                                                       float* __restrict__ e_nn, float* __restrict__ q_raw,
                                                       float* __restrict__ hv /* signed Hirshfeld pre-abs value */) {
  extern __shared__ float sm[];
  float* At = sm;
  float* Bt = At + kF * TS;
  float* Wsm = Bt + kF * TS;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int row0 = blockIdx.x * TA;
  load_tile_T<kF>(At, x, row0, n);
  float acc[8][8];
  float part[8];
  // energy
  zero_acc(acc);
  gemm_tile<kF, kF>(At, M.e_reg_k, Wsm, acc);
#pragma unroll
  for (int i = 0; i < 8; ++i) part[i] = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int c = tx + 16 * j;
    float b = M.e_reg_b[c], w = M.e_fin_k[c];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int r = ty + 8 * i;
      float z = acc[i][j] + b;
      if (row0 + r < n) ze[(size_t)(row0 + r) * kF + c] = z;
      part[i] = fmaf(silu_f(z), w, part[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float s = part[i];
    s += __shfl_xor_sync(0xffffffffu, s, 1); s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4); s += __shfl_xor_sync(0xffffffffu, s, 8);
    int a = row0 + ty + 8 * i;
    if (tx == 0 && a < n) {
      int z = Z[a]; z = z < 0 ? 0 : (z >= kZEmbed ? kZEmbed - 1 : z);
      e_nn[a] = (s + M.e_fin_b) * M.e_scale[z] + M.e_offset[z];
    }
  }
  // charge
  zero_acc(acc);
  gemm_tile<kF, kF>(At, M.q_reg_k, Wsm, acc);
#pragma unroll
  for (int i = 0; i < 8; ++i) part[i] = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int c = tx + 16 * j;
    float b = M.q_reg_b[c], w = M.q_fin_k[c];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int r = ty + 8 * i;
      float z = acc[i][j] + b;
      if (row0 + r < n) zq[(size_t)(row0 + r) * kF + c] = z;
      part[i] = fmaf(silu_f(z), w, part[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float s = part[i];
    s += __shfl_xor_sync(0xffffffffu, s, 1); s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4); s += __shfl_xor_sync(0xffffffffu, s, 8);
    int a = row0 + ty + 8 * i;
    if (tx == 0 && a < n) {
      int z = Z[a]; z = z < 0 ? 0 : (z >= kZHead ? kZHead - 1 : z);
      q_raw[a] = s + M.q_fin_b + M.q_embed[z];
    }
  }
  // Hirshfeld: 128 -> 64 -> 64, then dot with the element query
  float acc4[8][4];
  zero_acc(acc4);
  gemm_tile<kF, 64>(At, M.h_reg_k, Wsm, acc4);
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int c = tx + 16 * j;
    float b = M.h_reg_b[c];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int r = ty + 8 * i;
      float z = acc4[i][j] + b;
      if (row0 + r < n) zh[(size_t)(row0 + r) * 64 + c] = z;
      Bt[c * TS + r] = silu_f(z);
    }
  }
  zero_acc(acc4);
  gemm_tile<64, 64>(Bt, M.h_fin_k, Wsm, acc4);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int a = row0 + ty + 8 * i;
    int z = 0;
    if (a < n) { z = Z[a]; z = z < 0 ? 0 : (z >= kZHead ? kZHead - 1 : z); }
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int c = tx + 16 * j;
      s = fmaf(acc4[i][j] + M.h_fin_b[c], M.h_embed1[z * 64 + c], s);
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1); s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4); s += __shfl_xor_sync(0xffffffffu, s, 8);
    if (tx == 0 && a < n) hv[a] = M.h_embed0[z] + s * 0.125f;
  }
}

// heads backward: gx = dL/dx_final from cotangents of e_nn (ge), raw charge (gq) and Hirshfeld ratio (gh)
__global__ void __launch_bounds__(NT) heads_bwd_kernel(ModelDev M, int n, const int* __restrict__ Z, const float* __restrict__ ze,
                                                       const float* __restrict__ zq, const float* __restrict__ zh,
                                                       const float* __restrict__ hv, const float* __restrict__ ge,
                                                       const float* __restrict__ gq, const float* __restrict__ gh,
                                                       float* __restrict__ gx) {
  extern __shared__ float sm[];
  float* At = sm;
  float* Bt = At + kF * TS;
  float* Wsm = Bt + kF * TS;
  float* coef = Wsm + WCH * kF;   // 64*3 : ge*scale, gq, gh*sign/8
  int* zrow = reinterpret_cast<int*>(coef + TA * 3);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int row0 = blockIdx.x * TA;
  if (tid < TA) {
    int a = row0 + tid;
    float c0 = 0.f, c1 = 0.f, c2 = 0.f;
    int zz = 0;
    if (a < n) {
      int z = Z[a];
      int ze_ = z < 0 ? 0 : (z >= kZEmbed ? kZEmbed - 1 : z);
      zz = z < 0 ? 0 : (z >= kZHead ? kZHead - 1 : z);
      c0 = ge[a] * M.e_scale[ze_];
      c1 = gq[a];
      c2 = gh[a] * (hv[a] < 0.f ? -0.125f : 0.125f);
    }
    coef[tid * 3 + 0] = c0; coef[tid * 3 + 1] = c1; coef[tid * 3 + 2] = c2; zrow[tid] = zz;
  }
  __syncthreads();
  // Hirshfeld branch first: g_k[c] = c2 * embed1[z][c] -> g_sh = g_k Hfin^T -> g_zh = g_sh * dsilu(zh)
  for (int idx = tid; idx < TA * 64; idx += NT) {
    int r = idx & 63, c = idx >> 6;
    At[c * TS + r] = coef[r * 3 + 2] * M.h_embed1[zrow[r] * 64 + c];
  }
  float acc4[8][4];
  zero_acc(acc4);
  gemm_tile<64, 64>(At, M.h_fin_kT, Wsm, acc4);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int c = tx + 16 * j;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int r = ty + 8 * i;
      float z = (row0 + r < n) ? zh[(size_t)(row0 + r) * 64 + c] : 0.f;
      Bt[c * TS + r] = acc4[i][j] * dsilu_f(z);
    }
  }
  float acc[8][8];
  zero_acc(acc);
  gemm_tile<64, kF>(Bt, M.h_reg_kT, Wsm, acc);
  __syncthreads();
  // energy branch
  for (int idx = tid; idx < TA * kF; idx += NT) {
    int r = idx & 63, c = idx >> 6;
    float z = (row0 + r < n) ? ze[(size_t)(row0 + r) * kF + c] : 0.f;
    At[c * TS + r] = coef[r * 3 + 0] * M.e_fin_k[c] * dsilu_f(z);
  }
  gemm_tile<kF, kF>(At, M.e_reg_kT, Wsm, acc);
  __syncthreads();
  for (int idx = tid; idx < TA * kF; idx += NT) {
    int r = idx & 63, c = idx >> 6;
    float z = (row0 + r < n) ? zq[(size_t)(row0 + r) * kF + c] : 0.f;
    At[c * TS + r] = coef[r * 3 + 1] * M.q_fin_k[c] * dsilu_f(z);
  }
  gemm_tile<kF, kF>(At, M.q_reg_kT, Wsm, acc);
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) Bt[(tx + 16 * j) * TS + ty + 8 * i] = acc[i][j];
  __syncthreads();
  store_tile_T<kF>(gx, Bt, row0, n);
}

// ------------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------------
static constexpr size_t kSmemPostFwd = (size_t)(2 * kF * TS + WCH * kF + 2 * TA * 4) * sizeof(float);
static constexpr size_t kSmemPostBwd = (size_t)(3 * kF * TS + WCH * kF + 2 * TA * 4 + TA) * sizeof(float);
static constexpr size_t kSmemHeads = (size_t)(2 * kF * TS + WCH * kF + TA * 4) * sizeof(float);
static constexpr size_t kSmemProjBwd = (size_t)(5 * 4 * 32 * 32 + PROJ_TILE * kProj) * sizeof(float);

int configure_atom_kernels() {
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(atom_post_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemPostFwd));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(atom_post_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemPostBwd));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(heads_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemHeads));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(heads_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemHeads));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(proj_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemProjBwd));
  return kOk;
}

void launch_embed(cudaStream_t s, const ModelDev& M, const int* Z, int n, float* x) {
  if (n <= 0) return;
  size_t tot = (size_t)n * kF;
  { embed_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, s>>>(M.embed_z, Z, n, x); count_launch(); }
}
void launch_proj_fwd(cudaStream_t s, const LayerDev& L, const float* x, int n, float* qkv) {
  if (n <= 0) return;
  int blocks = (n + PROJ_TILE - 1) / PROJ_TILE;
  { proj_fwd_kernel<<<blocks, 640, 0, s>>>(L.projT, x, n, qkv); count_launch(); }
}
void launch_proj_bwd(cudaStream_t s, const LayerDev& L, const float* g_qkv, int n, float* gx, int accumulate) {
  if (n <= 0) return;
  int blocks = (n + PROJ_TILE - 1) / PROJ_TILE;
  if (blocks > sm_count() * 2) blocks = sm_count() * 2;
  { proj_bwd_kernel<<<blocks, 512, kSmemProjBwd, s>>>(L.proj, g_qkv, n, gx, accumulate); count_launch(); }
}
void launch_atom_post_fwd(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, float* z1,
                          float* x3, float* gate, float* x4, float* ev2) {
  if (n <= 0) return;
  { atom_post_fwd_kernel<<<(n + TA - 1) / TA, NT, kSmemPostFwd, s>>>(L, n, xa, ev1, z1, x3, gate, x4, ev2); count_launch(); }
}
void launch_atom_post_bwd(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, const float* z1,
                          const float* x3, const float* gate, const float* g4, const float* gev2, float* g_xa, float* gev1) {
  if (n <= 0) return;
  { atom_post_bwd_kernel<<<(n + TA - 1) / TA, NT, kSmemPostBwd, s>>>(L, n, xa, ev1, z1, x3, gate, g4, gev2, g_xa, gev1); count_launch(); }
}
void launch_heads_fwd(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* x, float* ze, float* zq, float* zh,
                      float* e_nn, float* q_raw, float* hv) {
  if (n <= 0) return;
  { heads_fwd_kernel<<<(n + TA - 1) / TA, NT, kSmemHeads, s>>>(M, n, Z, x, ze, zq, zh, e_nn, q_raw, hv); count_launch(); }
}
void launch_heads_bwd(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* ze, const float* zq, const float* zh,
                      const float* hv, const float* ge, const float* gq, const float* gh, float* gx) {
  if (n <= 0) return;
  { heads_bwd_kernel<<<(n + TA - 1) / TA, NT, kSmemHeads, s>>>(M, n, Z, ze, zq, zh, hv, ge, gq, gh, gx); count_launch(); }
}

}  // namespace so3lr

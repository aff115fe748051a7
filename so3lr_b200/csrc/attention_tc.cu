// Attention kernels of layers 1 and 2 as CTA-tiled tcgen05 kernels.
//
// A tile is 128 consecutive entries of the compacted short-range edge list (entries inside the 4.5 A cutoff only, grouped
// by receiver).  Per tile and layer, both filters of all 128 edges come out of ONE chain of tcgen05.mma instructions with
// the accumulators in tensor memory:
//
//     w[e, 0:256] = Phi[e, 0:64] * C[0:64, 0:256]  +  hs_f[e, 0:32] * K2_f[0:32, 0:128]   (f = 0, 1)
//
// Phi are 64 Chebyshev polynomials of t(r) (see common.cuh): the radial filter MLPs are smooth functions of the edge length
// alone, so their 2 x 128 outputs are contracted from a 64-term expansion on the tensor cores instead of being gathered
// from a table (4 KB per edge and layer through L2 before); hs_f is the hidden layer of the spherical filter.  FP32 accuracy
// comes from the two-term FP16 split used throughout the library (x = hi + lo / 2048; products hi*hi into one accumulator,
// hi*lo + lo*hi into a second one).  Operands sit in shared memory in the 8 x 8 core-matrix order without swizzle; the
// 96 KB weight image is resident for the whole kernel.  One thread issues the MMAs; completion arrives on an mbarrier
// (tcgen05.commit); every wait is bounded and reports through an error word instead of hanging.
//
// After the MMA the filter tile is moved from tensor memory to shared memory (row = edge) and the edge loop runs in the
// "lane = 4 features" layout of the other attention kernels: sender rows are read with coalesced 512-byte loads, logits are
// 8-lane reductions.  A warp owns a run of consecutive edges and adds its partial sums to the receiver's row with vector
// reductions in global memory (a receiver's edges can span warps, tiles and CTAs).
//
// The reverse kernel forms dw in the same loop, writes it straight into shared memory as the (FP16-split) A operand of a
// second MMA chain against the SAME weight image read with the other major-ness,
//
//     [dPhi | dhs_f][e, :] = dw_f[e, 0:128] * [C_f^T | K2_f^T],
//
// and finishes the radial derivative (sum_m dPhi[e,m] T_m'(t) dt/dr) and the spherical hidden layer per edge.
#include <cuda_fp16.h>
#include <cub/cub.cuh>
#include <cstdlib>

#include "kernels.h"

namespace so3lr {

namespace {

constexpr int TE = 128;                       // edges per tile = rows of every MMA
constexpr int kLboA = 2064;                   // bytes between 8-column chunks of an A operand: 128 rows x 16 B + 16 B of padding
constexpr int kAHalf = 16 * kLboA;            // one FP16 matrix of 128 rows x 128 columns
constexpr int kWStride = 132;                 // floats per row of the filter tile
constexpr int kFwRec = 36;                    // floats per forward record: j | i | cutoff / nbar | - | Y[24] | padding (bank spread)
constexpr int kFwThreads = 512;
constexpr int kFwIssuer = 128;       // forward kernel: the thread that issues the MMAs (its own preparation is the shortest)
constexpr int kBwRec = 52;                    // floats per reverse record (48 used; 52 spreads consecutive rows over the banks)
constexpr int kBwThreads = 512;
constexpr float kInvNbar = 1.0f / kAvgNumNeighbors;
constexpr float kRc2 = kCutoffSr * kCutoffSr;
constexpr float kLoScale = 2048.f, kLoInv = 1.f / 2048.f;
constexpr int kTmemCols = 512;
constexpr int kWaitSpins = 1 << 22;

// shared-memory map (bytes)
constexpr int kOffImg = 0;                                   // weight image: C hi | C lo | K2 hi [2] | K2 lo [2]
constexpr int kOffA = kTcImageBytes;                         // A operand (hi | lo); the forward kernel reuses it as filter tile
constexpr int kARegion = TE * kWStride * 4;                  // 67584 >= 2 * kAHalf
static_assert(kARegion >= 2 * kAHalf, "A region");
constexpr int kOffFwRec = kOffA + kARegion;
constexpr int kOffFwSph = kOffFwRec + TE * kFwRec * 4;
constexpr int kOffFwMisc = kOffFwSph + 512 * 4;
constexpr int kEvStride = 28;                                // floats per staged ev row (24 used; 112 B keeps 16-byte reads conflict-free)
constexpr int kOffFwStIJ = kOffFwMisc + 64;                  // staged inputs of the next tile: (i, j) | displacement | ev rows of both atoms
constexpr int kOffFwStD = kOffFwStIJ + TE * 8;
constexpr int kOffFwStEv = kOffFwStD + TE * 16;
constexpr int kSmemFwd = kOffFwStEv + TE * 2 * kEvStride * 4;
// reverse kernel: the filter tile holds 64 edges at a time
constexpr int kOffBwW = kOffA + kARegion;
constexpr int kOffBwRec = kOffBwW + 64 * kWStride * 4;
constexpr int kOffBwSph = kOffBwRec + TE * kBwRec * 4;
constexpr int kOffBwMisc = kOffBwSph + 512 * 4;
constexpr int kSmemBwd = kOffBwMisc + 64;
static_assert(kSmemFwd <= 232448 && kSmemBwd <= 232448, "shared memory budget of one CTA per SM");

__device__ __forceinline__ float invw(int l) {
  return l == 0 ? 0.5773502691896258f : (l == 1 ? 0.4472135954999579f : (l == 2 ? 0.3779644730092272f : 0.3333333333333333f));
}
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
// float4 arithmetic as two packed operations (fma.rn.f32x2 / mul.rn.f32x2) on the halves
__device__ __forceinline__ float2 lo2(float4 v) { return make_float2(v.x, v.y); }
__device__ __forceinline__ float2 hi2(float4 v) { return make_float2(v.z, v.w); }
__device__ __forceinline__ float4 f4_fma(float a, float4 b, float4 c) {
  const float2 a2 = make_float2(a, a);
  const float2 l = __ffma2_rn(a2, lo2(b), lo2(c)), h = __ffma2_rn(a2, hi2(b), hi2(c));
  return make_float4(l.x, l.y, h.x, h.y);
}
__device__ __forceinline__ float4 f4_zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ float dot3(float4 a, float4 b, float4 c) {
  const float2 s = __ffma2_rn(__fmul2_rn(hi2(a), hi2(b)), hi2(c), __fmul2_rn(__fmul2_rn(lo2(a), lo2(b)), lo2(c)));
  return s.x + s.y;
}
__device__ __forceinline__ float dot2(float4 a, float4 b) {
  const float2 s = __ffma2_rn(hi2(a), hi2(b), __fmul2_rn(lo2(a), lo2(b)));
  return s.x + s.y;
}
__device__ __forceinline__ bool f4_nonzero(float4 a) { return a.x != 0.f || a.y != 0.f || a.z != 0.f || a.w != 0.f; }

// (x, y) -> FP16 pair hi and FP16 pair of the residuals scaled by 2048
__device__ __forceinline__ void split2(float x, float y, unsigned& hi, unsigned& lo) {
  const __half2 h = __floats2half2_rn(x, y);
  const float2 hf = __half22float2(h);
  const __half2 l = __floats2half2_rn((x - hf.x) * kLoScale, (y - hf.y) * kLoScale);
  hi = *reinterpret_cast<const unsigned*>(&h);
  lo = *reinterpret_cast<const unsigned*>(&l);
}
// eight consecutive K entries of one operand row -> one 16-byte chunk of the hi matrix and one of the lo matrix
__device__ __forceinline__ void store_chunk(unsigned char* a_hi, int chunk, int row, const float* v) {
  uint4 h, l;
  split2(v[0], v[1], h.x, l.x); split2(v[2], v[3], h.y, l.y); split2(v[4], v[5], h.z, l.z); split2(v[6], v[7], h.w, l.w);
  unsigned char* p = a_hi + chunk * kLboA + row * 16;
  *reinterpret_cast<uint4*>(p) = h;
  *reinterpret_cast<uint4*>(p + kAHalf) = l;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// instruction descriptor, kind::f16: FP16 operands, FP32 accumulator, A K-major, B K-major or MN-major, M = 128
__device__ __forceinline__ uint32_t make_idesc(int n, int b_mn_major) {
  return (1u << 4) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TE >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
  for (int it = 0; it < kWaitSpins; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n" : "=r"(ok) : "r"(mbar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// fire-and-forget vector add in global memory (no value comes back to the warp)
__device__ __forceinline__ void red_add_v4(float* p, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive FP32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int k = 0; k < 32; ++k) v[k] = __uint_as_float(r[k]);
}
// main + cross / 2048 of 32 columns (cross accumulators sit 256 columns above the main ones)
__device__ __forceinline__ void tmem_ld32_combined(uint32_t taddr, float* v) {
  uint32_t a[32], b[32];      // both loads in flight before the one wait
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%65];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]), "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]), "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31]),
        "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]), "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]), "=r"(b[16]), "=r"(b[17]), "=r"(b[18]), "=r"(b[19]), "=r"(b[20]), "=r"(b[21]), "=r"(b[22]), "=r"(b[23]), "=r"(b[24]), "=r"(b[25]), "=r"(b[26]), "=r"(b[27]), "=r"(b[28]), "=r"(b[29]), "=r"(b[30]), "=r"(b[31])
      : "r"(taddr), "r"(taddr + 256)
      : "memory");
  const float2 s2 = make_float2(kLoInv, kLoInv);
#pragma unroll
  for (int k = 0; k < 32; k += 2) {
    const float2 r = __ffma2_rn(make_float2(__uint_as_float(b[k]), __uint_as_float(b[k + 1])), s2,
                                make_float2(__uint_as_float(a[k]), __uint_as_float(a[k + 1])));
    v[k] = r.x; v[k + 1] = r.y;
  }
}

__device__ __forceinline__ void invariants(const float* __restrict__ evi, const float* __restrict__ evj, float* s) {
  float d[kMTot];
#pragma unroll
  for (int c = 0; c < 6; ++c) {
    const float4 a = ld4(evj + 4 * c), b = ld4(evi + 4 * c);
    d[4 * c] = a.x - b.x; d[4 * c + 1] = a.y - b.y; d[4 * c + 2] = a.z - b.z; d[4 * c + 3] = a.w - b.w;
  }
  s[0] = s[1] = s[2] = s[3] = 0.f;
#pragma unroll
  for (int m = 0; m < kMTot; ++m) s[degree_of(m)] = fmaf(d[m], d[m], s[degree_of(m)]);
#pragma unroll
  for (int l = 0; l < 4; ++l) s[l] *= invw(l);
}

// Column order of the Chebyshev block of the A operand: column k < 32 holds T_{2k}, column 32 + k holds T_{2k+1} (the rows of
// the coefficient image are permuted to match).  Two threads share an edge: `odd` = 0 writes the even terms (chunks 0..3),
// 1 the odd ones (chunks 4..7).  Each runs two independent recurrences of step 4, T_{m+4} = 2 T_4 T_m - T_{m-4}, so the
// dependent chain is 16 long instead of 64.
__device__ __forceinline__ void store_chebyshev_half(unsigned char* a_hi, int row, float r, bool valid, int odd) {
  const float x = expf(-kChebHalfGamma * r);
  const float t = fmaf(kChebA, x, kChebB);
  const float T2 = fmaf(2.f * t, t, -1.f), T3 = fmaf(2.f * t, T2, -t), T4x2 = 2.f * fmaf(2.f * T2, T2, -1.f);
  // chain A: m = odd, odd + 4, ...   chain B: m = odd + 2, odd + 6, ...   (prev holds T at the index 4 below cur; T_{-m} = T_m)
  float a_cur = odd ? t : 1.f, a_prev = odd ? T3 : 0.5f * T4x2;
  float b_cur = odd ? T3 : T2, b_prev = odd ? t : T2;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    float v[8];
#pragma unroll
    for (int q = 0; q < 8; q += 2) {
      v[q] = valid ? a_cur : 0.f;
      v[q + 1] = valid ? b_cur : 0.f;
      const float2 nx = __ffma2_rn(make_float2(T4x2, T4x2), make_float2(a_cur, b_cur), make_float2(-a_prev, -b_prev));
      a_prev = a_cur; a_cur = nx.x;
      b_prev = b_cur; b_cur = nx.y;
    }
    store_chunk(a_hi, 4 * odd + c, row, v);
  }
}
// hidden layer of spherical filter f into chunks 8 + 4 f .. 11 + 4 f
__device__ __forceinline__ void store_spherical_hidden_f(unsigned char* a_hi, int row, const float* s, const float* sph8, int f) {
  // sph8: per (filter, hidden unit) eight floats: the four first-layer weights, the bias, padding
#pragma unroll
  for (int c8 = 0; c8 < 4; ++c8) {
    float v[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float* p = sph8 + (f * 32 + 8 * c8 + q) * 8;
      const float4 k = ld4(p);
      const float z = fmaf(s[0], k.x, fmaf(s[1], k.y, fmaf(s[2], k.z, fmaf(s[3], k.w, p[4]))));
      v[q] = __fdividef(z, 1.f + __expf(-z));
    }
    store_chunk(a_hi, 8 + 4 * f + c8, row, v);
  }
}

// Descriptors differ only in their start-address field (bits 0..13, in units of 16 bytes): desc(addr) = base + (addr >> 4).
// The issuing thread keeps everything in registers -- shared-memory loads inside the issue loop wait behind the operand
// traffic of the MMAs already running and throttle the chain.
__device__ __forceinline__ uint64_t desc_base(uint32_t lbo, uint32_t sbo) {
  return ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | ((uint64_t)1 << 46);
}

// Forward kernel, K-major weight image (rows = output features, 8 consecutive K entries per 16 bytes; the core matrices of
// one K chunk are contiguous over the rows, the layout the tensor cores fetch fastest):
//   CT hi | CT lo : [256 features][64 terms], core (n/8, k/8) at (k/8) * 4096 + (n/8) * 128           (2 x 32 KB)
//   K2T_f hi | lo : [128 features][32 hidden], core (n/8, k/8) at (k/8) * 2048 + (n/8) * 128          (4 x 8 KB)
// w = Phi * C + hs_f * K2_f: main accumulators in TMEM columns [0, 256), cross accumulators in [256, 512)
// The Chebyshev steps (part 0) read chunks 0..7 of A only, the steps of the spherical hidden layers (part 1) chunks 8..15: part 0 is
// issued as soon as the two threads per entry that write the Chebyshev terms are through, while the other two still gather `ev`
// rows and evaluate the hidden layers.
__device__ __noinline__ void issue_forward_mma(uint32_t tmem, uint32_t a_hi, uint32_t img, int part) {
  const uint64_t da = desc_base(kLboA, 128) + (a_hi >> 4), dal = da + (kAHalf >> 4);
  const uint64_t dc = desc_base(4096, 128) + (img >> 4), dcl = dc + (32768 >> 4);
  const uint64_t dk = desc_base(2048, 128) + ((img + 65536) >> 4), dkl = dk + (16384 >> 4);
  const uint32_t id256 = make_idesc(256, 0), id128 = make_idesc(128, 0);
  // K steps 1 and 3 hold the Chebyshev terms of order 32..63 (even terms, then odd terms, 32 columns each).  Their coefficients
  // are below 2^-12 of the filter scale (the expansion converges geometrically), so their hi * lo cross terms are below 2^-23 of
  // it, like the lo * lo terms that are dropped everywhere: those steps issue the hi * hi product only.
  if (part == 0) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const uint64_t ah = da + ks * (2 * kLboA >> 4), al = dal + ks * (2 * kLboA >> 4);
      const uint64_t bh = dc + ks * (2 * 4096 >> 4), bl = dcl + ks * (2 * 4096 >> 4);
      umma(tmem, ah, bh, id256, ks > 0);
      if (ks == 1 || ks == 3) continue;
      umma(tmem + 256, ah, bl, id256, ks > 0);
      umma(tmem + 256, al, bh, id256, 1);
    }
    return;
  }
#pragma unroll
  for (int f = 0; f < 2; ++f)
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const int chunk = 8 + 4 * f + 2 * ks;
      const uint64_t ah = da + chunk * (kLboA >> 4), al = dal + chunk * (kLboA >> 4);
      const uint64_t bh = dk + (f * 8192 + ks * 2 * 2048 >> 4), bl = dkl + (f * 8192 + ks * 2 * 2048 >> 4);
      umma(tmem + 128 * f, ah, bh, id128, 1);
      umma(tmem + 256 + 128 * f, ah, bl, id128, 1);
      umma(tmem + 256 + 128 * f, al, bh, id128, 1);
    }
}

// Reverse kernel, one image for both directions, per filter f (24,576 bytes each; hi of f = 0, 1 then lo of f = 0, 1): the 96
// rows [64 Chebyshev terms | 32 hidden units] by the 128 features of the filter, core (row / 8, feature / 8) at
// (feature / 8) * 1536 + (row / 8) * 128 with the 8 features of a core row contiguous.
// Forward product (B read MN-major: N = features, K = rows): w_f = [Phi | hs_f] * [C_f ; K2_f], main accumulators in TMEM
// columns [128 f, 128 f + 128), cross 256 columns above.
constexpr int kRevImgFilter = 16 * 1536;
// part 0: the four Chebyshev steps, part 1: the two steps of the filter's hidden layer (see issue_forward_mma)
__device__ __noinline__ void issue_filter_mma(uint32_t tmem, uint32_t a_hi, uint32_t img, int f, int part) {
  const uint64_t da = desc_base(kLboA, 128) + (a_hi >> 4), dal = da + (kAHalf >> 4);
  const uint64_t db = desc_base(128, 1536) + ((img + f * kRevImgFilter) >> 4), dbl = db + (2 * kRevImgFilter >> 4);
  const uint32_t id128 = make_idesc(128, 1);
  const uint32_t d_main = tmem + 128 * f, d_cross = d_main + 256;
#pragma unroll
  for (int ks = 0; ks < 6; ++ks) {      // K = 16 rows per step: Chebyshev chunks 0..7 of A, then the two chunks pairs of hs_f
    if ((ks >= 4) != (part == 1)) continue;
    const int chunk = ks < 4 ? 2 * ks : 8 + 4 * f + 2 * (ks - 4);
    const uint64_t ah = da + chunk * (kLboA >> 4), al = dal + chunk * (kLboA >> 4);
    const uint64_t bh = db + ks * (2 * 128 >> 4), bl = dbl + ks * (2 * 128 >> 4);
    umma(d_main, ah, bh, id128, ks > 0);
    if (ks == 1 || ks == 3) continue;      // Chebyshev terms of order >= 32: no cross terms (see issue_forward_mma)
    umma(d_cross, ah, bl, id128, ks > 0);
    umma(d_cross, al, bh, id128, 1);
  }
}

// 16-warp version: warps w, w + 4, w + 8, w + 12 share a quadrant and take 32 columns each; all 128 rows
__device__ __forceinline__ void tmem_to_tile(uint32_t tmem, int f, int warp, int lane, float* wt) {
  const int q = warp & 3, col = 32 * (warp >> 2);
  float v[32];
  tmem_ld32_combined(tmem + ((uint32_t)(32 * q) << 16) + 128 * f + col, v);
  float* p = wt + (32 * q + lane) * kWStride + col;
#pragma unroll
  for (int k = 0; k < 32; k += 4) st4(p + k, make_float4(v[k], v[k + 1], v[k + 2], v[k + 3]));
}

// ------------------------------------------------------------------------------------------------------------------
// compacted edge list
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ bool edge_valid(int j, int n, float dx, float dy, float dz, float& r2) {
  r2 = dx * dx + dy * dy + dz * dz;
  return j >= 0 && j < n && r2 < kRc2 && r2 > 0.f;
}
template <bool FILL>
__global__ void __launch_bounds__(256) compact_rows_kernel(int n_rows, int n, const int* __restrict__ row_ptr, const int* __restrict__ nbr_j,
                                                           const float* __restrict__ dR, int* __restrict__ vcount,
                                                           const int* __restrict__ vrow_ptr, int* __restrict__ ve_i, int* __restrict__ ve_j,
                                                           float4* __restrict__ ve_d, int* __restrict__ ve_orig) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= n_rows) return;
  const int e0 = row_ptr[i], e1 = row_ptr[i + 1];
  int count = 0;
  const int base = FILL ? vrow_ptr[i] : 0;
  for (int eb = e0; eb < e1; eb += 32) {
    const int e = eb + lane;
    bool valid = false;
    int j = -1;
    float dx = 0.f, dy = 0.f, dz = 0.f, r2 = 0.f;
    if (e < e1) {
      j = nbr_j[e];
      dx = dR[3 * (size_t)e]; dy = dR[3 * (size_t)e + 1]; dz = dR[3 * (size_t)e + 2];
      valid = edge_valid(j, n, dx, dy, dz, r2);
    }
    const unsigned m = __ballot_sync(0xffffffffu, valid);
    if (FILL && valid) {
      const int p = base + count + __popc(m & ((1u << lane) - 1u));
      ve_i[p] = i; ve_j[p] = j;
      ve_d[p] = make_float4(dx, dy, dz, sqrtf(r2));
      if (ve_orig) ve_orig[p] = e;
    }
    count += __popc(m);
  }
  if (!FILL && lane == 0) vcount[i] = count;
}
// every compacted entry (i <- j, d) looks for (j <- i, -d) in row j; a miss sets *asym
__global__ void __launch_bounds__(256) check_symmetric_kernel(int n_rows, const int* __restrict__ vrow_ptr, const int* __restrict__ ve_i,
                                                              const int* __restrict__ ve_j, const float4* __restrict__ ve_d, int* asym) {
  const long long n_entries = vrow_ptr[n_rows];
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n_entries; e += (long long)gridDim.x * blockDim.x) {
    const int i = ve_i[e], j = ve_j[e];
    const float4 d = ve_d[e];
    const float tol = 1e-5f * d.w + 1e-6f;
    bool found = false;
    if (j >= 0 && j < n_rows) {
      for (int p = vrow_ptr[j]; p < vrow_ptr[j + 1] && !found; ++p) {
        if (ve_j[p] != i) continue;
        const float4 q = ve_d[p];
        found = fabsf(q.x + d.x) <= tol && fabsf(q.y + d.y) <= tol && fabsf(q.z + d.z) <= tol;
      }
    }
    if (!found) { atomicExch(asym, 1); return; }
  }
}
__global__ void close_scan_kernel(int n_rows, const int* __restrict__ vcount, int* __restrict__ vrow_ptr) {
  if (threadIdx.x == 0 && blockIdx.x == 0) vrow_ptr[n_rows] = n_rows > 0 ? vrow_ptr[n_rows - 1] + vcount[n_rows - 1] : 0;
}

// ------------------------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------------------------
// 16 warps.  Per tile: (1) four threads per edge prepare the A operand (geometry + Chebyshev terms 0..31 | terms 32..63 | hidden
// layer of filter 0 | of filter 1) from inputs that were staged in shared memory with cp.async during the previous tile;
// (2) one thread issues the MMA chains of the two filters (one commit each) while every warp already has the sender rows of
// its 8 edges in flight and 128 threads stage the next tile; (3) per filter: tensor memory -> shared tile, then the edge loop.
__global__ void __launch_bounds__(kFwThreads, 1) attn_fwd_tc_kernel(const unsigned char* __restrict__ img_g, const float* __restrict__ sph1_k,
                                                                    const float* __restrict__ sph1_b, int n_recv,
                                                                    const int* __restrict__ vrow_ptr, const int* __restrict__ ve_i,
                                                                    const int* __restrict__ ve_j, const float4* __restrict__ ve_d,
                                                                    const float* __restrict__ qkv, const float* __restrict__ ev_in,
                                                                    float* __restrict__ xa, float* __restrict__ ev1, int* __restrict__ err,
                                                                    long long* __restrict__ dbg) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* rec = reinterpret_cast<float*>(smem + kOffFwRec);
  float* sph = reinterpret_cast<float*>(smem + kOffFwSph);
  float* wt = reinterpret_cast<float*>(smem + kOffA);
  int* st_ij = reinterpret_cast<int*>(smem + kOffFwStIJ);
  float4* st_d = reinterpret_cast<float4*>(smem + kOffFwStD);
  float* st_ev = reinterpret_cast<float*>(smem + kOffFwStEv);
  unsigned long long* mbar_p = reinterpret_cast<unsigned long long*>(smem + kOffFwMisc);
  uint32_t* tmem_p = reinterpret_cast<uint32_t*>(smem + kOffFwMisc + 16);
  const long long n_edges = vrow_ptr[n_recv];
  const long long n_tiles = (n_edges + TE - 1) / TE;
  const long long tile0 = n_tiles * blockIdx.x / gridDim.x, tile1 = n_tiles * (blockIdx.x + 1) / gridDim.x;
  if (tile0 >= tile1) return;
  const int pad_i = ve_i[n_edges - 1];
  // inputs of one tile into the staging buffers: receiver / sender, displacement, both atoms' ev rows (threads 256..383)
  auto stage_tile = [&](long long tile) {
    if (tid < 256 || tid >= 384 || tile >= tile1) return;
    const int row = tid - 256;
    const long long e = tile * TE + row;
    int i = pad_i, j = pad_i;
    if (e < n_edges) {
      i = ve_i[e]; j = ve_j[e];
      cp_async16(st_d + row, ve_d + e);
    } else {
      st_d[row] = make_float4(1.f, 0.f, 0.f, 1.f);
    }
    st_ij[2 * row] = i; st_ij[2 * row + 1] = j;
    const float* gi = ev_in + (size_t)i * kMTot;
    const float* gj = ev_in + (size_t)j * kMTot;
    // receivers' rows in the first half of the buffer, senders' rows in the second: consecutive entries are 112 bytes apart in
    // either half, which spreads the 16-byte accesses of eight threads over all banks (interleaved, 224 bytes apart, they collide
    // in pairs)
    float* d = st_ev + row * kEvStride;
#pragma unroll
    for (int c = 0; c < 6; ++c) { cp_async16(d + 4 * c, gi + 4 * c); cp_async16(d + TE * kEvStride + 4 * c, gj + 4 * c); }
  };
  for (int k = tid; k < kTcImageBytes / 16; k += kFwThreads) reinterpret_cast<uint4*>(smem + kOffImg)[k] = reinterpret_cast<const uint4*>(img_g)[k];
  for (int k = tid; k < 512; k += kFwThreads) {      // [filter][hidden unit][w0 w1 w2 w3 b - - -]
    const int q = k & 7, c = (k >> 3) & 31, f = k >> 8;
    sph[k] = q < 4 ? sph1_k[f * 128 + q * 32 + c] : (q == 4 ? sph1_b[f * 32 + c] : 0.f);
  }
  const uint32_t mbar0 = smem_u32(mbar_p);
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar0));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_p)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  stage_tile(tile0);
  cp_async_wait_all();
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_p;
  const uint32_t a_hi = smem_u32(smem + kOffA), img = smem_u32(smem + kOffImg);
  const int col = 4 * lane;
  const int deg = degree_of(lane < kMTot ? lane : 0);
  const int k0 = 8 * warp;               // this warp's rows of the tile in the edge loop
  uint32_t parity = 0;
#ifdef SO3LR_TC_TIMING
  long long tph[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  long long tc0 = clock64();
#define TC_MARK(k) do { if (dbg && (tid & 31) == 0) { const long long c = clock64(); tph[k] += c - tc0; tc0 = c; } } while (0)
#else
#define TC_MARK(k) do { } while (0)
#endif
  for (long long tile = tile0; tile < tile1; ++tile) {
    // ---- per-edge preparation from the staged inputs ----
    {
      const int row = tid & 127, role = tid >> 7;
      const bool valid = tile * TE + row < n_edges;
      if (role < 2) {
        const float4 d = st_d[row];
        const float r = d.w;
        // the Chebyshev chunks first: once these 256 threads are through, their share of the MMA chain starts beneath the rest
        // of the preparation
        store_chebyshev_half(smem + kOffA, row, r, valid, role);
        fence_async_smem();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (tid == kFwIssuer) {
          tc_fence_after();
          issue_forward_mma(tmem, a_hi, img, 0);
        }
        if (role == 0) {
          const float ir = 1.f / r;
          float cut, dcut;
          phys_cutoff(r, cut, dcut);
          float Y[kMTot];
          sph_harm_24(d.x * ir, d.y * ir, d.z * ir, Y);
          float* rp = rec + row * kFwRec;
          st4(rp, make_float4(__int_as_float(st_ij[2 * row + 1]), __int_as_float(st_ij[2 * row]), valid ? cut * kInvNbar : 0.f, 0.f));
#pragma unroll
          for (int c = 0; c < 6; ++c) st4(rp + 4 + 4 * c, make_float4(Y[4 * c], Y[4 * c + 1], Y[4 * c + 2], Y[4 * c + 3]));
        }
      } else {
        float s[4];
        invariants(st_ev + row * kEvStride, st_ev + (TE + row) * kEvStride, s);
        store_spherical_hidden_f(smem + kOffA, row, s, sph, role - 2);
      }
    }
    TC_MARK(0);
    // sender rows of filter 0 for this warp's edges and the first receiver's query row, requested before the barrier (the indices
    // are in the staging buffer since the previous tile): the warps with the shorter preparation start their gathers while the
    // others still work, and all of them are in flight while the tensor cores run
    float4 kf[8], vj[8], qf;
    int cur_i;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const float* kj = qkv + (size_t)st_ij[2 * (k0 + u) + 1] * kProj;
      kf[u] = ld4(kj + kF + col);
      vj[u] = ld4(kj + 2 * kF + col);
    }
    cur_i = st_ij[2 * k0];
    qf = ld4(qkv + (size_t)cur_i * kProj + col);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    TC_MARK(1);
    stage_tile(tile + 1);
    bool done = true;
    if (tid == kFwIssuer) {
      tc_fence_after();
#ifdef SO3LR_TC_TIMING
      const long long q0 = clock64();
#endif
      issue_forward_mma(tmem, a_hi, img, 1);
      umma_commit(mbar0);
#ifdef SO3LR_TC_TIMING
      const long long q1 = clock64();
#endif
      done = mbar_wait(mbar0, parity);
#ifdef SO3LR_TC_TIMING
      if (dbg && blockIdx.x == 0) { dbg[9] += q1 - q0; dbg[10] += clock64() - q1; }
#endif
    }
    if (!__syncthreads_and(done)) {
      if (tid == 0) atomicExch(err, 1);
      break;
    }
    tc_fence_after();
    TC_MARK(2);
    // ---- filter 0: invariant logits, feature sums ----
    tmem_to_tile(tmem, 0, warp, lane, wt);
    tc_fence_before();
    __syncthreads();
    TC_MARK(3);
    {
      float4 accx = f4_zero();
      if (cur_i == __float_as_int(rec[(k0 + 7) * kFwRec + 1])) {      // all eight edges belong to one receiver: no flush inside
        float a[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          a[u] = group8_sum(dot3(qf, ld4(wt + (k0 + u) * kWStride + col), kf[u])) * rec[(k0 + u) * kFwRec + 2];
#pragma unroll
        for (int u = 0; u < 8; ++u) accx = f4_fma(a[u], vj[u], accx);
      } else {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float4 r0 = ld4(rec + (k0 + u) * kFwRec);
          const int iu = __float_as_int(r0.y);
          if (iu != cur_i) {
            if (f4_nonzero(accx)) red_add_v4(xa + (size_t)cur_i * kF + col, accx);
            cur_i = iu;
            accx = f4_zero();
            qf = ld4(qkv + (size_t)cur_i * kProj + col);
          }
          const float a = group8_sum(dot3(qf, ld4(wt + (k0 + u) * kWStride + col), kf[u])) * r0.z;
          accx = f4_fma(a, vj[u], accx);
        }
      }
      if (f4_nonzero(accx)) red_add_v4(xa + (size_t)cur_i * kF + col, accx);
    }
    // sender rows of filter 1: in flight across the barrier and the second tile copy
#pragma unroll
    for (int u = 0; u < 8; ++u) kf[u] = ld4(qkv + (size_t)__float_as_int(rec[(k0 + u) * kFwRec]) * kProj + 4 * kF + col);
    cur_i = __float_as_int(rec[k0 * kFwRec + 1]);
    qf = ld4(qkv + (size_t)cur_i * kProj + 3 * kF + col);
    TC_MARK(4);
    parity ^= 1;
    __syncthreads();
    TC_MARK(5);
    // ---- filter 1: equivariant logits, spherical-harmonic sums ----
    tmem_to_tile(tmem, 1, warp, lane, wt);
    tc_fence_before();
    __syncthreads();
    TC_MARK(6);
    {
      float accev = 0.f;
      if (cur_i == __float_as_int(rec[(k0 + 7) * kFwRec + 1])) {
        float a[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          a[u] = group8_sum(dot3(qf, ld4(wt + (k0 + u) * kWStride + col), kf[u])) * rec[(k0 + u) * kFwRec + 2];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float ym = lane < kMTot ? rec[(k0 + u) * kFwRec + 4 + lane] : 0.f;
          accev = fmaf(__shfl_sync(0xffffffffu, a[u], 8 * deg), ym, accev);
        }
      } else {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float4 r0 = ld4(rec + (k0 + u) * kFwRec);
          const int iu = __float_as_int(r0.y);
          if (iu != cur_i) {
            if (lane < kMTot && accev != 0.f) atomicAdd(ev1 + (size_t)cur_i * kMTot + lane, accev);
            cur_i = iu;
            accev = 0.f;
            qf = ld4(qkv + (size_t)cur_i * kProj + 3 * kF + col);
          }
          const float a = group8_sum(dot3(qf, ld4(wt + (k0 + u) * kWStride + col), kf[u])) * r0.z;
          const float ym = lane < kMTot ? rec[(k0 + u) * kFwRec + 4 + lane] : 0.f;
          accev = fmaf(__shfl_sync(0xffffffffu, a, 8 * deg), ym, accev);
        }
      }
      if (lane < kMTot && accev != 0.f) atomicAdd(ev1 + (size_t)cur_i * kMTot + lane, accev);
    }
    cp_async_wait_all();
    __syncthreads();
    TC_MARK(7);
  }
#ifdef SO3LR_TC_TIMING
  if (dbg && tid == 32 && blockIdx.x == 0) { for (int q = 0; q < 8; ++q) dbg[q] = tph[q]; dbg[8] = tile1 - tile0; }
  if (dbg && (tid & 31) == 0 && blockIdx.x == 0) { for (int q = 0; q < 8; ++q) dbg[160 + 8 * warp + q] = tph[q]; }
#endif
  cp_async_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

}  // namespace

namespace {

// ------------------------------------------------------------------------------------------------------------------
// reverse
// ------------------------------------------------------------------------------------------------------------------
// record fields (floats): 0 j | 1 i | 2 cutoff / nbar | 3 its r-derivative | 4-7 invariants | 8-11 their cotangents |
// 12-15 dA, 16-19 dB: cotangents of the equivariant logits of edge (i<-j) and (j<-i) | 20-23, 24-27 those logits x cutoff |
// 28-30 unit vector | 31 1/r | 32 d/dr | 33 r | 34 1 for a list entry, 0 for a padding row
// [dPhi | dhs_f] = dw_f * [C_f^T | K2_f^T] (the same image read K-major: N = 96 rows, K = features): main accumulators in TMEM
// columns [128 f, 128 f + 96), cross 256 columns above
__device__ __noinline__ void issue_reverse_mma(uint32_t tmem, uint32_t a_hi, uint32_t img, int f) {
  const uint64_t da = desc_base(kLboA, 128) + (a_hi >> 4), dal = da + (kAHalf >> 4);
  const uint64_t db = desc_base(1536, 128) + ((img + f * kRevImgFilter) >> 4), dbl = db + (2 * kRevImgFilter >> 4);
  const uint32_t id96 = make_idesc(96, 0);
  const uint32_t d_main = tmem + 128 * f, d_cross = d_main + 256;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {      // K = 16 features per step
    const uint64_t ah = da + ks * (2 * kLboA >> 4), al = dal + ks * (2 * kLboA >> 4);
    const uint64_t bh = db + ks * (2 * 1536 >> 4), bl = dbl + ks * (2 * 1536 >> 4);
    umma(d_main, ah, bh, id96, ks > 0);
    umma(d_cross, ah, bl, id96, ks > 0);
    umma(d_cross, al, bh, id96, 1);
  }
}

// Sender-side q / k rows of four consecutive tile rows for the reverse edge loop of filter F (lane = 4 features)
struct RevLoads {
  float4 qj[4], kj[4], qa, ka;     // senders' rows; q / k of the first row's receiver
};
template <int F>
__device__ __forceinline__ void reverse_prefetch(RevLoads& L, const float* rec, int row0, int lane, const float* __restrict__ qkv) {
  const int col = 4 * lane;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const float* pj = qkv + (size_t)__float_as_int(rec[(row0 + u) * kBwRec]) * kProj + F * 3 * kF;
    L.qj[u] = ld4(pj + col);
    L.kj[u] = ld4(pj + kF + col);
  }
  const float* pi = qkv + (size_t)__float_as_int(rec[row0 * kBwRec + 1]) * kProj + F * 3 * kF;
  L.qa = ld4(pi + col);
  L.ka = ld4(pi + kF + col);
}

// Value path of the invariant filter, split off the edge loop so that it runs while the tensor cores are busy.
// Before the loop (rows [row0, row0 + 8) of one warp): cotangents of the invariant logits of both directions of every edge,
// daA_h = <g_xa[i], v[j]>_h and daB_h = <g_xa[j], v[i]>_h, into record fields 36..39 and 40..43.
__device__ __forceinline__ void value_logit_cotangents(float* rec, int row0, int lane, const float* __restrict__ qkv,
                                                       const float* __restrict__ g_xa) {
  const int col = 4 * lane, grp = lane >> 3, cg = lane & 7;
  int cur_i = -1;
  float4 v_i = f4_zero(), gx_i = f4_zero();
#pragma unroll
  for (int k0 = 0; k0 < 8; k0 += 4) {
    float4 vj[4], gxj[4];
    int ii[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float* rp = rec + (row0 + k0 + u) * kBwRec;
      const int j = __float_as_int(rp[0]);
      ii[u] = __float_as_int(rp[1]);
      vj[u] = ld4(qkv + (size_t)j * kProj + 2 * kF + col);
      gxj[u] = ld4(g_xa + (size_t)j * kF + col);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (ii[u] != cur_i) {
        cur_i = ii[u];
        v_i = ld4(qkv + (size_t)cur_i * kProj + 2 * kF + col);
        gx_i = ld4(g_xa + (size_t)cur_i * kF + col);
      }
      const float daA = group8_sum(dot2(gx_i, vj[u])), daB = group8_sum(dot2(gxj[u], v_i));
      if (cg == 0) {
        float* rp = rec + (row0 + k0 + u) * kBwRec;
        rp[36 + grp] = daA;
        rp[40 + grp] = daB;
      }
    }
  }
}
// After the loop: cotangent of this receiver's value row, gv_i = sum_edges (cutoff x logit of edge j<-i)_h g_xa[j] (fields 44..47)
__device__ __forceinline__ void value_cotangent(const float* rec, int row0, int lane, const float* __restrict__ g_xa, float* __restrict__ g_qkv) {
  const int col = 4 * lane, grp = lane >> 3;
  float4 gxj[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) gxj[u] = ld4(g_xa + (size_t)__float_as_int(rec[(row0 + u) * kBwRec]) * kF + col);
  int cur_i = __float_as_int(rec[row0 * kBwRec + 1]);
  float4 gv = f4_zero();
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const float* rp = rec + (row0 + u) * kBwRec;
    const int i = __float_as_int(rp[1]);
    if (i != cur_i) {
      if (f4_nonzero(gv)) red_add_v4(g_qkv + (size_t)cur_i * kProj + 2 * kF + col, gv);
      cur_i = i;
      gv = f4_zero();
    }
    gv = f4_fma(rp[44 + grp], gxj[u], gv);
  }
  if (f4_nonzero(gv)) red_add_v4(g_qkv + (size_t)cur_i * kProj + 2 * kF + col, gv);
}

// Reverse edge loop of filter F over four tile rows [row0, row0 + 4) of one warp: logits of both directions of every edge,
// cotangents of this receiver's q / k rows (added to g_qkv with vector reductions when the receiver changes), dw into the
// A operand of the second MMA chain, the cutoff part of d/dr into the records.  The cotangents of the logits come from the
// records (fields 36.. for the invariant filter, 12.. for the equivariant one); cutoff x logit goes back (44.. / 20.., 24..).
template <int F>
__device__ __forceinline__ void reverse_edges4(const RevLoads& L, float* rec, const float* wt, int wrow0, int row0, unsigned char* a_hi,
                                               int lane, const float* __restrict__ qkv, float* __restrict__ g_qkv) {
  const int col = 4 * lane, grp = lane >> 3, cg = lane & 7;
  int cur_i = __float_as_int(rec[row0 * kBwRec + 1]);
  float4 qa = L.qa, ka = L.ka;
  float4 gq = f4_zero(), gk = f4_zero();
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int row = row0 + u;
    float* rp = rec + row * kBwRec;
    const float4 r0 = ld4(rp);
    const int i = __float_as_int(r0.y);
    const float sc = r0.z, dcn = r0.w;
    if (i != cur_i) {      // rare: a run of four rows mostly stays with one receiver
      {
        float* gi = g_qkv + (size_t)cur_i * kProj + F * 3 * kF + col;
        if (f4_nonzero(gq)) red_add_v4(gi, gq);
        if (f4_nonzero(gk)) red_add_v4(gi + kF, gk);
      }
      cur_i = i;
      gq = f4_zero(); gk = f4_zero();
      const float* pi = qkv + (size_t)i * kProj + F * 3 * kF;
      qa = ld4(pi + col); ka = ld4(pi + kF + col);
    }
    const float4 w = ld4(wt + (wrow0 + u) * kWStride + col);
    const float4 qj = L.qj[u], kj = L.kj[u];
    // packed FP32 arithmetic (fma.rn.f32x2) on the two halves of every float4: the products q_i k_j and q_j k_i serve both the
    // logits and dw
    const float2 w01 = make_float2(w.x, w.y), w23 = make_float2(w.z, w.w);
    const float2 pA01 = __fmul2_rn(make_float2(qa.x, qa.y), make_float2(kj.x, kj.y)), pA23 = __fmul2_rn(make_float2(qa.z, qa.w), make_float2(kj.z, kj.w));
    const float2 pB01 = __fmul2_rn(make_float2(qj.x, qj.y), make_float2(ka.x, ka.y)), pB23 = __fmul2_rn(make_float2(qj.z, qj.w), make_float2(ka.z, ka.w));
    const float2 sA = __ffma2_rn(w23, pA23, __fmul2_rn(w01, pA01)), sB = __ffma2_rn(w23, pB23, __fmul2_rn(w01, pB01));
    const float DA = group8_sum(sA.x + sA.y);
    const float DB = group8_sum(sB.x + sB.y);
    const float daA = rp[(F ? 12 : 36) + grp], daB = rp[(F ? 16 : 40) + grp];
    if (cg == 0) {
      if (F) { rp[20 + grp] = sc * DA; rp[24 + grp] = sc * DB; }
      else rp[44 + grp] = sc * DB;
    }
    const float dDA = sc * daA, dDB = sc * daB;
    const float2 a2 = make_float2(dDA, dDA), b2 = make_float2(dDB, dDB);
    {
      const float2 g01 = __ffma2_rn(a2, __fmul2_rn(w01, make_float2(kj.x, kj.y)), make_float2(gq.x, gq.y));
      const float2 g23 = __ffma2_rn(a2, __fmul2_rn(w23, make_float2(kj.z, kj.w)), make_float2(gq.z, gq.w));
      gq = make_float4(g01.x, g01.y, g23.x, g23.y);
      const float2 h01 = __ffma2_rn(b2, __fmul2_rn(w01, make_float2(qj.x, qj.y)), make_float2(gk.x, gk.y));
      const float2 h23 = __ffma2_rn(b2, __fmul2_rn(w23, make_float2(qj.z, qj.w)), make_float2(gk.z, gk.w));
      gk = make_float4(h01.x, h01.y, h23.x, h23.y);
    }
    const float2 d01 = __ffma2_rn(a2, pA01, __fmul2_rn(b2, pB01)), d23 = __ffma2_rn(a2, pA23, __fmul2_rn(b2, pB23));
    const float dw0 = d01.x, dw1 = d01.y, dw2 = d23.x, dw3 = d23.y;
    // dw as A operand of the second MMA chain: row = edge, columns 4 lane .. 4 lane + 3 of the hi and the lo matrix
    {
      uint2 h, l;
      split2(dw0, dw1, h.x, l.x); split2(dw2, dw3, h.y, l.y);
      unsigned char* p = a_hi + (lane >> 1) * kLboA + row * 16 + (lane & 1) * 8;
      *reinterpret_cast<uint2*>(p) = h;
      *reinterpret_cast<uint2*>(p + kAHalf) = l;
    }
    // cutoff part of d/dr, summed over the four heads
    float gc = dcn * fmaf(daA, DA, daB * DB);
    gc += __shfl_xor_sync(0xffffffffu, gc, 8);
    gc += __shfl_xor_sync(0xffffffffu, gc, 16);
    if (lane == 0) rp[32] += gc;
  }
  float* gi = g_qkv + (size_t)cur_i * kProj + F * 3 * kF + col;
  if (f4_nonzero(gq)) red_add_v4(gi, gq);
  if (f4_nonzero(gk)) red_add_v4(gi + kF, gk);
}

// record fields (floats): 0 j | 1 i | 2 cutoff / nbar | 3 its r-derivative | 4-7 invariants | 8-11 their cotangents |
// 12-15 dA, 16-19 dB: cotangents of the equivariant logits of edge (i<-j) and (j<-i) | 20-23, 24-27 those logits x cutoff |
// 28-30 unit vector | 31 1/r | 32 d/dr (cutoff part + even Chebyshev terms) | 33 r | 34 1 for a list entry, 0 for a padding row |
// 35 d/dr (odd Chebyshev terms) | 36-39, 40-43 cotangents of the invariant logits of edge (i<-j) and (j<-i) |
// 44-47 invariant logit of edge (j<-i) x cutoff; after the value path has read it: 44-46 angular part of the force on the receiver
//
// 16 warps.  Per tile: (1) four threads per edge prepare records and the A operand; (2) MMA chain w = Phi C + hs K2 (both filters);
// (3) per filter, in two halves of 64 rows: tensor memory -> shared tile, reverse edge loop (4 rows per warp, sender rows
// prefetched across the barriers), dw into the A operand; (4) per filter: MMA chain [dPhi | dhs] = dw [C^T | K2^T], then per
// edge the radial derivative and the spherical hidden layer (the angular part of the force is formed beneath the last chain);
// (5) force on the receiver, cotangent of ev.
// PER_ENTRY (caller-supplied lists): `F` is the gradient with respect to the source list's displacement vectors (3 floats per
// source entry, added to), `ve_orig` maps compacted entries to source entries, and the launch returns at once when *gate != 0.
template <bool PER_ENTRY>
__global__ void __launch_bounds__(kBwThreads, 1) attn_bwd_tc_kernel(const unsigned char* __restrict__ img_g, const float* __restrict__ sph1_k,
                                                                    const float* __restrict__ sph1_b, int n_recv,
                                                                    const int* __restrict__ vrow_ptr, const int* __restrict__ ve_i,
                                                                    const int* __restrict__ ve_j, const float4* __restrict__ ve_d,
                                                                    const float* __restrict__ qkv, const float* __restrict__ ev_in,
                                                                    const float* __restrict__ g_xa, const float* __restrict__ gev1,
                                                                    float* __restrict__ g_qkv, float* __restrict__ gev_in,
                                                                    float* __restrict__ F, float* __restrict__ virial,
                                                                    int* __restrict__ err, long long* __restrict__ dbg,
                                                                    const int* __restrict__ ve_orig, const int* __restrict__ gate) {
  if (PER_ENTRY && gate && *gate != 0) return;
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* rec = reinterpret_cast<float*>(smem + kOffBwRec);
  float* sph = reinterpret_cast<float*>(smem + kOffBwSph);
  float* wt = reinterpret_cast<float*>(smem + kOffBwW);
  unsigned long long* mbar_p = reinterpret_cast<unsigned long long*>(smem + kOffBwMisc);
  uint32_t* tmem_p = reinterpret_cast<uint32_t*>(smem + kOffBwMisc + 16);
  const long long n_edges = vrow_ptr[n_recv];
  const long long n_tiles = (n_edges + TE - 1) / TE;
  const long long tile0 = n_tiles * blockIdx.x / gridDim.x, tile1 = n_tiles * (blockIdx.x + 1) / gridDim.x;
  if (tile0 >= tile1) return;
  for (int k = tid; k < kTcImageBytes / 16; k += kBwThreads) reinterpret_cast<uint4*>(smem + kOffImg)[k] = reinterpret_cast<const uint4*>(img_g)[k];
  for (int k = tid; k < 512; k += kBwThreads) {      // [filter][hidden unit][w0 w1 w2 w3 b - - -]
    const int q = k & 7, c = (k >> 3) & 31, f = k >> 8;
    sph[k] = q < 4 ? sph1_k[f * 128 + q * 32 + c] : (q == 4 ? sph1_b[f * 32 + c] : 0.f);
  }
  const uint32_t mbar = smem_u32(mbar_p);
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_p)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_p;
  const uint32_t a_hi = smem_u32(smem + kOffA), img = smem_u32(smem + kOffImg);
  unsigned char* a_ptr = smem + kOffA;
  const int pad_i = ve_i[n_edges - 1];
  const int deg = degree_of(lane < kMTot ? lane : 0);
  const int quad = warp & 3;                    // TMEM lane quadrant of this warp
  const int wrow = 4 * warp;                    // this warp's 4 rows inside a 64-row half of the tile
  uint32_t parity = 0;
  bool failed = false;
#ifdef SO3LR_TC_TIMING
  long long bph[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  long long bc0 = clock64();
#define BW_MARK(k) do { if (dbg && (tid & 31) == 0) { const long long c = clock64(); bph[k] += c - bc0; bc0 = c; } } while (0)
#else
#define BW_MARK(k) do { } while (0)
#endif
  for (long long tile = tile0; tile < tile1 && !failed; ++tile) {
    float dev8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // ---- per-edge preparation ----
    {
      const int row = tid & 127, role = tid >> 7;
      const long long e = tile * TE + row;
      const bool valid = e < n_edges;
      int i = pad_i, j = pad_i;
      if (valid) { i = ve_i[e]; j = ve_j[e]; }
      float* rp = rec + row * kBwRec;
      if (role < 2) {
        float4 d = make_float4(1.f, 0.f, 0.f, 1.f);
        if (valid) d = ve_d[e];
        const float r = d.w;
        // the Chebyshev chunks first: once these 256 threads are through, the Chebyshev steps of both filters' MMA chains start
        // beneath the rest of the preparation (the gathers of the other two threads of an entry above all)
        store_chebyshev_half(a_ptr, row, r, valid, role);
        fence_async_smem();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (tid == 0) {
          tc_fence_after();
          issue_filter_mma(tmem, a_hi, img, 0, 0);
          issue_filter_mma(tmem, a_hi, img, 1, 0);
        }
        const float ir = 1.f / r;
        const float ux = d.x * ir, uy = d.y * ir, uz = d.z * ir;
        if (role == 0) {
          float cut, dcut;
          phys_cutoff(r, cut, dcut);
          st4(rp, make_float4(__int_as_float(j), __int_as_float(i), valid ? cut * kInvNbar : 0.f, valid ? dcut * kInvNbar : 0.f));
          st4(rp + 8, f4_zero());
          st4(rp + 20, f4_zero());
          st4(rp + 24, f4_zero());
          st4(rp + 28, make_float4(ux, uy, uz, ir));
          st4(rp + 32, make_float4(0.f, r, valid ? 1.f : 0.f, 0.f));
        } else {
          float Y[kMTot];
          sph_harm_24(ux, uy, uz, Y);
          float dA[4] = {0.f, 0.f, 0.f, 0.f}, dB[4] = {0.f, 0.f, 0.f, 0.f};
          const float* gevi = gev1 + (size_t)i * kMTot;
          const float* gevj = gev1 + (size_t)j * kMTot;
#pragma unroll
          for (int c = 0; c < 6; ++c) {
            const float4 a = ld4(gevi + 4 * c), b = ld4(gevj + 4 * c);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              dA[degree_of(4 * c + q)] = fmaf(av[q], Y[4 * c + q], dA[degree_of(4 * c + q)]);
              dB[degree_of(4 * c + q)] = fmaf(bv[q], Y[4 * c + q], dB[degree_of(4 * c + q)]);
            }
          }
          dB[0] = -dB[0]; dB[2] = -dB[2];   // Y_lm(-u) = (-1)^l Y_lm(u)
          st4(rp + 12, make_float4(dA[0], dA[1], dA[2], dA[3]));
          st4(rp + 16, make_float4(dB[0], dB[1], dB[2], dB[3]));
        }
      } else {
        float s[4];
        invariants(ev_in + (size_t)i * kMTot, ev_in + (size_t)j * kMTot, s);
        if (role == 2) st4(rp + 4, make_float4(s[0], s[1], s[2], s[3]));
        store_spherical_hidden_f(a_ptr, row, s, sph, role - 2);
      }
    }
    BW_MARK(0);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    BW_MARK(1);
    if (tid == 0) {
      tc_fence_after();
      issue_filter_mma(tmem, a_hi, img, 0, 1);
      issue_filter_mma(tmem, a_hi, img, 1, 1);
      umma_commit(mbar);
    }
    __syncwarp();
    // while the tensor cores run: the value path's logit cotangents (8 rows per warp), then the sender rows of the first edge run
    value_logit_cotangents(rec, 8 * warp, lane, qkv, g_xa);
    RevLoads L;
    reverse_prefetch<0>(L, rec, wrow, lane, qkv);
    bool done = true;
    if (tid == 0) done = mbar_wait(mbar, parity);     // one thread polls; the others park at the barrier below
    parity ^= 1;
    if (!__syncthreads_and(done)) { failed = true; break; }
    tc_fence_after();
    BW_MARK(2);
#pragma unroll 1
    for (int f = 0; f < 2 && !failed; ++f) {
#pragma unroll 1
      for (int hh = 0; hh < 2; ++hh) {
        if ((quad >> 1) == hh) {          // the 8 warps whose TMEM lanes hold this half: 32 columns each
          float v[32];
          const int col = 32 * (warp >> 2);
          tmem_ld32_combined(tmem + ((uint32_t)(32 * quad) << 16) + 128 * f + col, v);
          float* p = wt + (32 * (quad & 1) + lane) * kWStride + col;
#pragma unroll
          for (int k = 0; k < 32; k += 4) st4(p + k, make_float4(v[k], v[k + 1], v[k + 2], v[k + 3]));
        }
        tc_fence_before();
        __syncthreads();
        BW_MARK(3);
        if (f == 0) {
          reverse_edges4<0>(L, rec, wt, wrow, 64 * hh + wrow, a_ptr, lane, qkv, g_qkv);
          if (hh == 0) reverse_prefetch<0>(L, rec, 64 + wrow, lane, qkv);      // next run: second half of filter 0
          else reverse_prefetch<1>(L, rec, wrow, lane, qkv);                   // next run: first half of filter 1
        } else {
          reverse_edges4<1>(L, rec, wt, wrow, 64 * hh + wrow, a_ptr, lane, qkv, g_qkv);
          if (hh == 0) reverse_prefetch<1>(L, rec, 64 + wrow, lane, qkv);
        }
        BW_MARK(4);
        __syncthreads();
      }
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after();
        issue_reverse_mma(tmem, a_hi, img, f);
        umma_commit(mbar);
      }
      __syncwarp();
      if (f == 1 && lane < kMTot) {      // ev differences of this warp's 8 rows of the final flush: requested now, used after the last MMA
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float* rp = rec + (8 * warp + k) * kBwRec;
          const int j = __float_as_int(rp[0]), i = __float_as_int(rp[1]);
          dev8[k] = ev_in[(size_t)j * kMTot + lane] - ev_in[(size_t)i * kMTot + lane];
        }
      }
      if (f == 0) {
        value_cotangent(rec, 8 * warp, lane, g_xa, g_qkv);      // while the tensor cores run
      } else if (tid < 128) {
        // angular part of the force on the receiver (independent of the radial derivative that the running MMA yields); it
        // takes the record fields 44..46, which the value path has released
        float* rp = rec + tid * kBwRec;
        if (rp[34] != 0.f) {
          const int j = __float_as_int(rp[0]), i = __float_as_int(rp[1]);
          const float4 aA = ld4(rp + 20), aB = ld4(rp + 24), uu = ld4(rp + 28);
          const float* gevi = gev1 + (size_t)i * kMTot;
          const float* gevj = gev1 + (size_t)j * kMTot;
          const float aAv[4] = {aA.x, aA.y, aA.z, aA.w}, aBv[4] = {aB.x, aB.y, aB.z, aB.w};
          float gY[kMTot];
#pragma unroll
          for (int c = 0; c < 6; ++c) {
            const float4 a = ld4(gevi + 4 * c), b = ld4(gevj + 4 * c);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int m = 4 * c + q, l = degree_of(m);
              const float sgn = (l == 0 || l == 2) ? -1.f : 1.f;
              gY[m] = aAv[l] * av[q] + sgn * aBv[l] * bv[q];
            }
          }
          float gux, guy, guz;
          sph_harm_24_vjp(uu.x, uu.y, uu.z, gY, gux, guy, guz);
          const float gd = gux * uu.x + guy * uu.y + guz * uu.z;
          st4(rp + 44, make_float4((gux - gd * uu.x) * uu.w, (guy - gd * uu.y) * uu.w, (guz - gd * uu.z) * uu.w, 0.f));
        }
      }
      done = true;
      if (tid == 0) done = mbar_wait(mbar, parity);
      parity ^= 1;
      if (!__syncthreads_and(done)) { failed = true; break; }
      tc_fence_after();
      BW_MARK(5);
      // ---- per edge: radial derivative (even terms: threads 0..127, odd terms: 128..255), spherical hidden layer (all four threads of a row) ----
      {
        const int row = tid & 127, role = tid >> 7;
        float* rp = rec + row * kBwRec;
        const uint32_t lane_base = tmem + ((uint32_t)(32 * quad) << 16) + 128 * f;
        if (role < 2) {
          const float r = rp[33];
          const float x = expf(-kChebHalfGamma * r);
          const float t = fmaf(kChebA, x, kChebB), t2 = 2.f * t;
          const float dtdr = -kChebA * kChebHalfGamma * x;
          // T_m' = m U_{m-1}; columns 0..31 hold m = 2c (U of odd index), columns 32..63 hold m = 2c + 1 (U of even index);
          // both run U_{n+2} = 2 T_2 U_n - U_{n-2}
          const float T2x2 = 2.f * fmaf(t2, t, -1.f);
          float v[32];
          tmem_ld32_combined(lane_base + 32 * role, v);
          float up = role ? -1.f : -t2, uc = role ? 1.f : 0.f;      // (U_{-2}, U_0) or (U_{-3}, U_{-1})
          float acc = 0.f;
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            acc = fmaf(v[c] * (float)(2 * c + role), uc, acc);
            const float un = fmaf(T2x2, uc, -up);
            up = uc; uc = un;
          }
          rp[role ? 35 : 32] += acc * dtdr;
        }
        // spherical hidden layer, reverse: the four threads of a row take eight hidden units each and add their shares of the
        // invariants' cotangents to the record
        {
          float v[32];
          tmem_ld32_combined(lane_base + 64, v);
          const float4 s4 = ld4(rp + 4);
          float ds0 = 0.f, ds1 = 0.f, ds2 = 0.f, ds3 = 0.f;
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            const int c = 8 * role + c8;
            const float* p = sph + (f * 32 + c) * 8;
            const float4 k = ld4(p);
            const float z = fmaf(s4.x, k.x, fmaf(s4.y, k.y, fmaf(s4.z, k.z, fmaf(s4.w, k.w, p[4]))));
            const float sg = __fdividef(1.f, 1.f + __expf(-z));
            const float vc = role == 0 ? v[c8] : (role == 1 ? v[8 + c8] : (role == 2 ? v[16 + c8] : v[24 + c8]));
            const float dz = vc * sg * (1.f + z * (1.f - sg));
            ds0 = fmaf(dz, k.x, ds0); ds1 = fmaf(dz, k.y, ds1); ds2 = fmaf(dz, k.z, ds2); ds3 = fmaf(dz, k.w, ds3);
          }
          atomicAdd(rp + 8, ds0); atomicAdd(rp + 9, ds1); atomicAdd(rp + 10, ds2); atomicAdd(rp + 11, ds3);
        }
      }
      tc_fence_before();
      __syncthreads();
      BW_MARK(6);
    }
    if (failed) break;
    // ---- force on the receiver (threads 0..127; the angular part was formed under the last MMA); cotangent of ev (8 rows per warp) ----
    if (tid < 128) {
      const float* rp = rec + tid * kBwRec;
      const bool on = rp[34] != 0.f;
      const int i = on ? __float_as_int(rp[1]) : -1;
      const float4 uu = ld4(rp + 28), ang = ld4(rp + 44);
      const float g_r = rp[32] + rp[35];
      float fsx = on ? fmaf(g_r, uu.x, ang.x) : 0.f, fsy = on ? fmaf(g_r, uu.y, ang.y) : 0.f, fsz = on ? fmaf(g_r, uu.z, ang.z) : 0.f;
      if (virial && on) {
        const float hr = 0.5f * rp[33];
        const float wx = hr * uu.x, wy = hr * uu.y, wz = hr * uu.z;
        float* w = virial + 6 * (size_t)i;
        atomicAdd(w, wx * fsx); atomicAdd(w + 1, wy * fsy); atomicAdd(w + 2, wz * fsz);
        atomicAdd(w + 3, 0.5f * (wy * fsz + wz * fsy)); atomicAdd(w + 4, 0.5f * (wx * fsz + wz * fsx));
        atomicAdd(w + 5, 0.5f * (wx * fsy + wy * fsx));
      }
      if (PER_ENTRY) {
        // half of the pair's force on the receiver goes to this entry of the source list; the reversed entry, processed at the
        // other atom, receives the other half with the opposite sign
        if (on) {
          const long long e = tile * TE + tid;
          float* g = F + 3 * (size_t)ve_orig[e];
          g[0] += 0.5f * fsx; g[1] += 0.5f * fsy; g[2] += 0.5f * fsz;
        }
      } else {
      // the rows of a tile are sorted by receiver: sum each run of equal receivers inside the warp (segmented scan) and let its
      // last lane add the total, instead of up to 32 additions to one address
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float tx = __shfl_up_sync(0xffffffffu, fsx, o), ty = __shfl_up_sync(0xffffffffu, fsy, o), tz = __shfl_up_sync(0xffffffffu, fsz, o);
        const int ti = __shfl_up_sync(0xffffffffu, i, o);
        if (lane >= o && ti == i) { fsx += tx; fsy += ty; fsz += tz; }
      }
      const int inext = __shfl_down_sync(0xffffffffu, i, 1);
      if (on && (lane == 31 || inext != i)) {
        atomicAdd(F + 3 * (size_t)i, fsx); atomicAdd(F + 3 * (size_t)i + 1, fsy); atomicAdd(F + 3 * (size_t)i + 2, fsz);
      }
      }
    }
    {
      int cur_i = -1;
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float* rp = rec + (8 * warp + k) * kBwRec;
        const int i = __float_as_int(rp[1]);
        if (i != cur_i) {
          if (cur_i >= 0 && lane < kMTot && acc != 0.f) atomicAdd(gev_in + (size_t)cur_i * kMTot + lane, acc);
          cur_i = i; acc = 0.f;
        }
        if (lane < kMTot) acc = fmaf(-2.f * invw(deg) * rp[8 + deg], dev8[k], acc);
      }
      if (cur_i >= 0 && lane < kMTot && acc != 0.f) atomicAdd(gev_in + (size_t)cur_i * kMTot + lane, acc);
    }
    __syncthreads();
    BW_MARK(7);
  }
#ifdef SO3LR_TC_TIMING
  if (dbg && tid == 32 && blockIdx.x == 0) { for (int q = 0; q < 8; ++q) dbg[16 + q] = bph[q]; dbg[24] = tile1 - tile0; }
  if (dbg && (tid & 31) == 0 && blockIdx.x == 0) { for (int q = 0; q < 8; ++q) dbg[32 + 8 * warp + q] = bph[q]; }
#endif
  if (failed && tid == 0) atomicExch(err, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

}  // namespace

// ------------------------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------------------------
int configure_attention_tc_kernels() {
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFwd));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBwd));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBwd));
  return kOk;
}

int valid_edges_reserve(ValidEdges* V, int n_rows, long long capacity) {
  if (n_rows + 1 > V->row_cap) {
    if (V->row_ptr) cudaFree(V->row_ptr);
    if (V->count) cudaFree(V->count);
    V->row_ptr = nullptr; V->count = nullptr;
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&V->row_ptr, ((size_t)n_rows + 1) * sizeof(int)));
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&V->count, ((size_t)n_rows + 1) * sizeof(int)));
    V->row_cap = n_rows + 1;
    size_t need = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, need, V->count, V->row_ptr, n_rows);
    if (need > V->cub_bytes) {
      if (V->cub_tmp) cudaFree(V->cub_tmp);
      V->cub_tmp = nullptr;
      SO3LR_CUDA_CHECK(cudaMalloc(&V->cub_tmp, need));
      V->cub_bytes = need;
    }
  }
  if (capacity > V->capacity) {
    if (V->i) cudaFree(V->i);
    if (V->j) cudaFree(V->j);
    if (V->d) cudaFree(V->d);
    V->i = V->j = nullptr; V->d = nullptr;
    if (capacity < 1) capacity = 1;
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&V->i, (size_t)capacity * sizeof(int)));
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&V->j, (size_t)capacity * sizeof(int)));
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&V->d, (size_t)capacity * sizeof(float4)));
    V->capacity = capacity;
  }
  return kOk;
}

void valid_edges_free(ValidEdges* V) {
  cudaFree(V->row_ptr); cudaFree(V->count); cudaFree(V->i); cudaFree(V->j); cudaFree(V->d); cudaFree(V->orig); cudaFree(V->cub_tmp);
  *V = ValidEdges{};
}

int valid_edges_build(ValidEdges* V, cudaStream_t s, int n_rows, int n, const int* row_ptr, const int* nbr_j, const float* dR, bool want_orig) {
  if (n_rows <= 0) return kOk;
  if (n_rows + 1 > V->row_cap) return kInvalidArgument;
  if (want_orig && V->orig_cap < V->capacity) {
    if (V->orig) cudaFree(V->orig);
    V->orig = nullptr;
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&V->orig, (size_t)V->capacity * sizeof(int)));
    V->orig_cap = V->capacity;
  }
  const int blocks = (n_rows + 7) / 8;
  { compact_rows_kernel<false><<<blocks, 256, 0, s>>>(n_rows, n, row_ptr, nbr_j, dR, V->count, nullptr, nullptr, nullptr, nullptr, nullptr); count_launch(); }
  size_t tmp = V->cub_bytes;
  cub::DeviceScan::ExclusiveSum(V->cub_tmp, tmp, V->count, V->row_ptr, n_rows, s);
  count_launch(2);
  { close_scan_kernel<<<1, 32, 0, s>>>(n_rows, V->count, V->row_ptr); count_launch(); }
  { compact_rows_kernel<true><<<blocks, 256, 0, s>>>(n_rows, n, row_ptr, nbr_j, dR, nullptr, V->row_ptr, V->i, V->j, V->d, want_orig ? V->orig : nullptr); count_launch(); }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  V->n_rows = n_rows;
  return kOk;
}

// development aid: SO3LR_B200_TC_DEBUG=1 makes the forward kernel record the cycles its first CTA spends in each phase
static long long* tc_debug_buffer() {
  static long long* buf = [] {
    long long* p = nullptr;
    if (std::getenv("SO3LR_B200_TC_DEBUG")) {
      cudaMalloc((void**)&p, 288 * sizeof(long long)); cudaMemset(p, 0, 288 * sizeof(long long));
    }
    return p;
  }();
  return buf;
}
void tc_debug_print() {
  long long* d = tc_debug_buffer();
  if (!d) return;
  long long h[288];
  cudaDeviceSynchronize();
  cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  if (h[24]) std::fprintf(stderr, "tc bwd phases (cycles per tile, %lld tiles): prep %lld | sync %lld | mma1 %lld | sync+tmem->tile %lld | edge loop %lld | sync+mma2 %lld | epilogue %lld | phase C %lld\n",
               h[24], h[16] / h[24], h[17] / h[24], h[18] / h[24], h[19] / h[24], h[20] / h[24], h[21] / h[24], h[22] / h[24], h[23] / h[24]);
  if (h[24])
    for (int w = 0; w < 16; ++w) {
      std::fprintf(stderr, "  bwd warp %2d:", w);
      for (int q = 0; q < 8; ++q) std::fprintf(stderr, " %6lld", h[32 + 8 * w + q] / h[24]);
      std::fprintf(stderr, "\n");
    }
  if (h[8])
    for (int w = 0; w < 16; ++w) {
      std::fprintf(stderr, "  fwd warp %2d:", w);
      for (int q = 0; q < 8; ++q) std::fprintf(stderr, " %6lld", h[160 + 8 * w + q] / h[8]);
      std::fprintf(stderr, "\n");
    }
  std::fprintf(stderr, "tc fwd mma issue %lld wait %lld cycles per tile\n", h[9] / (h[8] ? h[8] : 1), h[10] / (h[8] ? h[8] : 1));
  std::fprintf(stderr, "tc fwd phases (cycles per tile, %lld tiles): prep %lld | sync %lld | mma+wait %lld | tmem0 %lld | loop0 %lld | sync %lld | tmem1 %lld | loop1 %lld\n",
               h[8], h[0] / (h[8] ? h[8] : 1), h[1] / (h[8] ? h[8] : 1), h[2] / (h[8] ? h[8] : 1), h[3] / (h[8] ? h[8] : 1), h[4] / (h[8] ? h[8] : 1),
               h[5] / (h[8] ? h[8] : 1), h[6] / (h[8] ? h[8] : 1), h[7] / (h[8] ? h[8] : 1));
}
int launch_attn_fwd_tc(cudaStream_t s, const LayerDev& L, const ValidEdges& V, int n_recv, const float* qkv, const float* x_in,
                       const float* ev_in, float* xa, float* ev1, int* err) {
  if (n_recv <= 0) return kOk;
  if (n_recv > V.n_rows) return kInvalidArgument;
  // the kernel adds the attention sums onto the skip connection
  SO3LR_CUDA_CHECK(cudaMemcpyAsync(xa, x_in, (size_t)n_recv * kF * sizeof(float), cudaMemcpyDeviceToDevice, s));
  SO3LR_CUDA_CHECK(cudaMemcpyAsync(ev1, ev_in, (size_t)n_recv * kMTot * sizeof(float), cudaMemcpyDeviceToDevice, s));
  { attn_fwd_tc_kernel<<<sm_count(), kFwThreads, kSmemFwd, s>>>(L.tc_img_fwd, L.sph1_k, L.sph1_b, n_recv, V.row_ptr, V.i, V.j, V.d, qkv, ev_in, xa, ev1, err, tc_debug_buffer()); count_launch(); }
  return kOk;
}

int launch_attn_bwd_tc(cudaStream_t s, const LayerDev& L, const ValidEdges& V, int n_recv, const float* qkv, const float* ev_in,
                       const float* g_xa, const float* gev1, float* g_qkv, float* gev_in, float* F, float* virial, int* err) {
  if (n_recv <= 0) return kOk;
  if (n_recv > V.n_rows) return kInvalidArgument;
  // the kernel adds into the receivers' rows: cotangents of q/k/v start at zero, that of ev at the skip term
  SO3LR_CUDA_CHECK(cudaMemsetAsync(g_qkv, 0, (size_t)n_recv * kProj * sizeof(float), s));
  SO3LR_CUDA_CHECK(cudaMemcpyAsync(gev_in, gev1, (size_t)n_recv * kMTot * sizeof(float), cudaMemcpyDeviceToDevice, s));
  { attn_bwd_tc_kernel<false><<<sm_count(), kBwThreads, kSmemBwd, s>>>(L.tc_img, L.sph1_k, L.sph1_b, n_recv, V.row_ptr, V.i, V.j, V.d, qkv, ev_in, g_xa, gev1,
                                                              g_qkv, gev_in, F, virial, err, tc_debug_buffer(), nullptr, nullptr); count_launch(); }
  return kOk;
}

int launch_attn_bwd_tc_graph(cudaStream_t s, const LayerDev& L, const ValidEdges& V, int n_recv, const float* qkv, const float* ev_in,
                             const float* g_xa, const float* gev1, float* g_qkv, float* gev_in, float* g_dR, int* err, const int* asym) {
  if (n_recv <= 0) return kOk;
  if (n_recv > V.n_rows || !V.orig) return kInvalidArgument;
  { attn_bwd_tc_kernel<true><<<sm_count(), kBwThreads, kSmemBwd, s>>>(L.tc_img, L.sph1_k, L.sph1_b, n_recv, V.row_ptr, V.i, V.j, V.d, qkv, ev_in, g_xa, gev1,
                                                             g_qkv, gev_in, g_dR, nullptr, err, nullptr, V.orig, asym); count_launch(); }
  return kOk;
}

void valid_edges_check_symmetric(const ValidEdges& V, cudaStream_t s, int* asym) {
  if (V.n_rows <= 0) return;
  { check_symmetric_kernel<<<sm_count() * 8, 256, 0, s>>>(V.n_rows, V.row_ptr, V.i, V.j, V.d, asym); count_launch(); }
}

}  // namespace so3lr

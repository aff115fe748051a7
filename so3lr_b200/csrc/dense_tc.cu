// Per-atom dense blocks (post-attention block of every layer, forward and reverse, and the output heads) on the 5th-generation
// tensor cores (tcgen05) of sm_100a.
//
// One persistent CTA of 16 warps per SM walks over tiles of 128 atoms.  Every contraction of the chain
//   LayerNorm -> Dense -> silu -> Dense -> (+) -> exchange Dense -> (+) -> LayerNorm -> q/k/v projections
// is one group of tcgen05.mma instructions with M = 128 atoms: the A operand (activations of the tile, FP16 hi + 2048-scaled
// lo, K contiguous, 8 x 8 core matrices) is written to shared memory by the epilogue of the previous contraction, the B
// operand (the layer's kernel, pre-split on the host in the same core-matrix order) arrives as one bulk asynchronous copy
// (cp.async.bulk, mbarrier completion) issued while that epilogue runs, and the FP32 accumulators live in tensor memory:
// columns [0, 256) the hi*hi products, [256, 512) the hi*lo + lo*hi cross terms (result = main + cross / 2048; the dropped
// lo*lo term is below 2^-22).  Accumulator columns that a contraction does not use hold the residual stream of the tile
// between epilogues (tcgen05.st / tcgen05.ld), so shared memory only carries operands and one FP32 staging tile.
//
// Threads t, t + 128, t + 256, t + 384 own atom row t of the tile (TMEM lane t; a warp can only reach the 32 lanes of its
// quarter) and take 32 columns each in every epilogue.  Everything that touches global memory goes through the staging
// tile with a warp per row, 16 bytes per lane; LayerNorm statistics are formed from per-thread partial sums that meet in
// shared memory.
// Every wait on an mbarrier is bounded; a wait that runs out sets the error word the host checks and the kernel carries
// on to its end (its results are then meaningless, but nothing hangs and the tensor memory is released).
#include <cuda_fp16.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "kernels.h"

namespace so3lr {

namespace {

constexpr int TM = 128;                // atoms per tile = rows of every MMA
constexpr int NTHR = 512;
constexpr int NQ = NTHR / TM;           // threads per atom row
constexpr int RPW = TM / (NTHR / 32);  // rows per warp in the warp-per-row passes
constexpr int SS = 164;                // floats per row of the staging tile (160 used; 164 spreads 16-byte row accesses over the banks)
constexpr int kALo = 32768;            // A operand: hi matrix, then lo matrix, 16 chunks (8 K entries) of 128 rows x 16 bytes
constexpr int kOffA = 0;
constexpr int kOffW = 65536;           // weight buffer (one [128 x 128] image, or slots of smaller ones)
constexpr int kWBytes = 65536;
constexpr int kOffS = kOffW + kWBytes;
constexpr int kOffStat = kOffS + TM * SS * 4;        // float2[128]: LayerNorm mean, rstd
constexpr int kOffInv = kOffStat + TM * 8;           // float4[128]: per-degree invariants (or their cotangents)
constexpr int kOffRed = kOffInv + TM * 16;           // float4[4][128]: partial sums of the column quarters
constexpr int kOffRed2 = kOffRed + NQ * TM * 16;     // float[2][4][128]: partial sums / squared deviations
constexpr int kOffMisc = kOffRed2 + 2 * NQ * TM * 4; // mbarriers, TMEM base
constexpr int kSmemDense = kOffMisc + 64;
static_assert(kSmemDense <= 232448, "shared memory budget of one CTA per SM");
constexpr float kLoScale = 2048.f, kLoInv = 1.f / 2048.f;
constexpr int kTmemCols = 512;
constexpr int kColCross = 256;         // cross accumulators
constexpr int kColX = 128;             // residual stream slot (free while N <= 128)
constexpr int kWaitSpins = 1 << 22;
constexpr int kProjBlockBytes = 16384; // [32 x 128] hi + lo, or four [32 x 32] hi + lo

__device__ __forceinline__ float inv_weight(int l) {
  return l == 0 ? 0.5773502691896258f : (l == 1 ? 0.4472135954999579f : (l == 2 ? 0.3779644730092272f : 0.3333333333333333f));
}
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void split2(float x, float y, unsigned& hi, unsigned& lo) {
  const __half2 h = __floats2half2_rn(x, y);
  const float2 hf = __half22float2(h);
  const float2 d = __fmul2_rn(__fadd2_rn(make_float2(x, y), make_float2(-hf.x, -hf.y)), make_float2(kLoScale, kLoScale));
  const __half2 l = __float22half2_rn(d);
  hi = *reinterpret_cast<const unsigned*>(&h);
  lo = *reinterpret_cast<const unsigned*>(&l);
}
// eight consecutive K entries (chunk = k / 8) of operand row `row`
__device__ __forceinline__ void a_store8(unsigned char* A, int chunk, int row, const float* v) {
  uint4 h, l;
  split2(v[0], v[1], h.x, l.x); split2(v[2], v[3], h.y, l.y); split2(v[4], v[5], h.z, l.z); split2(v[6], v[7], h.w, l.w);
  unsigned char* p = A + chunk * 2048 + row * 16;
  *reinterpret_cast<uint4*>(p) = h;
  *reinterpret_cast<uint4*>(p + kALo) = l;
}
// 32 consecutive columns starting at column c0 of operand row `row`
__device__ __forceinline__ void a_store32(unsigned char* A, int c0, int row, const float* v) {
#pragma unroll
  for (int k = 0; k < 4; ++k) a_store8(A, (c0 >> 3) + k, row, v + 8 * k);
}

// shared-memory matrix descriptor without its start address: no swizzle, lbo = bytes between core matrices along K, sbo = bytes
// between core matrices along M / N, descriptor version 1
__device__ __forceinline__ uint64_t desc_base(uint32_t lbo, uint32_t sbo) {
  return ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | ((uint64_t)1 << 46);
}
// instruction descriptor, kind::f16: FP16 operands, FP32 accumulator, both operands K-major, M = 128
__device__ __forceinline__ uint32_t make_idesc(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TM >> 4) << 24); }
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
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
// one bulk asynchronous copy global -> this CTA's shared memory (no multicast); size and both addresses multiples of 16 bytes
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem), "l"(src),
               "r"(bytes), "r"(mbar) : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// rows [row0, row0 + 128) of a row-major array with `row_bytes` bytes per atom (a multiple of 128 x threads' share): each thread
// asks for the 128-byte lines tid, tid + 512, .. of the tile
__device__ __forceinline__ void prefetch_tile(const float* base, int row_floats, int row0, int n, int tid) {
  const int rows = n - row0 < TM ? n - row0 : TM;
  if (rows <= 0) return;
  const char* p = reinterpret_cast<const char*>(base + (size_t)row0 * row_floats);
  const int lines = (rows * row_floats * 4 + 127) >> 7;
  for (int l = tid; l < lines; l += NTHR) prefetch_l2(p + ((size_t)l << 7));
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// accumulator columns c .. c+31: main + cross / 2048 (both loads in flight before the one wait)
__device__ __forceinline__ void tmem_acc32(uint32_t tlane, int c, float* v) {
  uint32_t a[32], b[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%65];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]), "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]), "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31]),
        "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]), "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]), "=r"(b[16]), "=r"(b[17]), "=r"(b[18]), "=r"(b[19]), "=r"(b[20]), "=r"(b[21]), "=r"(b[22]), "=r"(b[23]), "=r"(b[24]), "=r"(b[25]), "=r"(b[26]), "=r"(b[27]), "=r"(b[28]), "=r"(b[29]), "=r"(b[30]), "=r"(b[31])
      : "r"(tlane + c), "r"(tlane + kColCross + c)
      : "memory");
#pragma unroll
  for (int k = 0; k < 32; ++k) v[k] = fmaf(__uint_as_float(b[k]), kLoInv, __uint_as_float(a[k]));
}
// silu with the fast reciprocal (2 ulp; the operands are rounded to 22 bits right after)
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.f + __expf(-x)); }
__device__ __forceinline__ float dsilu_fast(float x) {
  const float s = __fdividef(1.f, 1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

// D[128 x n] (+)= A[:, chunks] * B: A from chunk `a_chunk0` on (2 chunks per K step of 16), B image at w_smem (hi matrix, lo
// matrix w_lo bytes above, core-matrix stride along K = 16 n bytes).  Issued by one thread; three MMAs per K step.
__device__ __noinline__ void issue_gemm(uint32_t tmem, int d_col, uint32_t a_smem, int a_chunk0, uint32_t w_smem, uint32_t w_lo, int n, int ksteps,
                                        uint32_t accumulate) {
  const uint64_t da = desc_base(2048, 128) + ((a_smem + a_chunk0 * 2048) >> 4), dal = da + (kALo >> 4);
  const uint64_t db = desc_base(16 * n, 128) + (w_smem >> 4), dbl = db + (w_lo >> 4);
  const uint32_t idesc = make_idesc(n);
  const uint32_t a_step = (2 * 2048) >> 4, b_step = (2 * 16 * n) >> 4;
#pragma unroll 1
  for (int ks = 0; ks < ksteps; ++ks) {
    const uint64_t ah = da + ks * a_step, al = dal + ks * a_step, bh = db + ks * b_step, bl = dbl + ks * b_step;
    const uint32_t acc = (ks > 0) ? 1u : accumulate;
    umma(tmem + d_col, ah, bh, idesc, acc);
    umma(tmem + kColCross + d_col, ah, bl, idesc, acc);
    umma(tmem + kColCross + d_col, al, bh, idesc, 1u);
  }
}

#ifdef SO3LR_TC_TIMING
__device__ long long g_dense_dbg[64];
#define DN_MARK(k) do { if (tid == 0 && blockIdx.x == 0) { const long long c_ = clock64(); atomicAdd((unsigned long long*)&g_dense_dbg[k], (unsigned long long)(c_ - dn_c0)); dn_c0 = c_; } } while (0)
#define DN_BEGIN() long long dn_c0 = clock64()
#define DN_TILE(k) do { if (tid == 0 && blockIdx.x == 0) atomicAdd((unsigned long long*)&g_dense_dbg[k], 1ull); } while (0)
#else
#define DN_MARK(k) do { } while (0)
#define DN_BEGIN() do { } while (0)
#define DN_TILE(k) do { } while (0)
#endif

// Bookkeeping shared by the kernels of this file.
struct Tile {
  unsigned char* sm;
  unsigned char* A;
  float* S;
  float2* stat;
  float4* inv;
  float4* red;
  float* redf;
  uint32_t mbar, mbar2, wbar, tmem, tlane;
  uint32_t mph, mph2, wph;      // phases of the two barriers (wph is only followed by thread 0)
  int tid, warp, lane, row, quarter, c0;
  bool failed;

  __device__ __forceinline__ void init(unsigned char* smem) {
    sm = smem;
    A = sm + kOffA;
    S = reinterpret_cast<float*>(sm + kOffS);
    stat = reinterpret_cast<float2*>(sm + kOffStat);
    inv = reinterpret_cast<float4*>(sm + kOffInv);
    red = reinterpret_cast<float4*>(sm + kOffRed);
    redf = reinterpret_cast<float*>(sm + kOffRed2);
    tid = threadIdx.x; warp = tid >> 5; lane = tid & 31; row = tid & 127; quarter = tid >> 7; c0 = 32 * quarter;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kOffMisc);
    uint32_t* tmem_p = reinterpret_cast<uint32_t*>(sm + kOffMisc + 32);
    mbar = smem_u32(bars); wbar = smem_u32(bars + 1); mbar2 = smem_u32(bars + 2);
    mph = 0; mph2 = 0; wph = 0; failed = false;
    if (tid == 0) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(wbar));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar2));
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
    tmem = *tmem_p;
    tlane = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
  }
  __device__ __forceinline__ void finish(int* err) {
    if (failed) atomicExch(err, 2);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  // thread 0: start the copy of a weight image into the weight buffer (the MMAs that read the bytes it replaces have completed)
  __device__ __forceinline__ void load_weights(const unsigned char* src, uint32_t bytes, uint32_t w_off = 0) {
    mbar_expect_tx(wbar, bytes);
    bulk_load(smem_u32(sm + kOffW + w_off), src, bytes, wbar);
  }
  __device__ __forceinline__ void wait_weights() {
    if (!mbar_wait(wbar, wph)) failed = true;
    wph ^= 1;
  }
  // operands written: make them visible to the tensor core, then thread 0 issues (inside `issue`) and commits
  __device__ __forceinline__ void operands_ready() {
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
  }
  __device__ __forceinline__ void wait_mma() {
    if (!mbar_wait(mbar, mph)) failed = true;
    mph ^= 1;
    tc_fence_after();
  }
  __device__ __forceinline__ void wait_mma2() {   // second accumulator set
    if (!mbar_wait(mbar2, mph2)) failed = true;
    mph2 ^= 1;
    tc_fence_after();
  }
  // LayerNorm statistics of the staging tile's rows.  Every thread holds the sum over its 32 columns; the quarters meet in
  // shared memory, then the squared deviations go the same way (two barriers, no shuffles).  Contains __syncthreads.
  __device__ __forceinline__ float part_row_sum() const {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { const float4 x = ld4(S + row * SS + c0 + 4 * k); s += (x.x + x.y) + (x.z + x.w); }
    return s;
  }
  __device__ __forceinline__ float2 row_stats(float partial_sum) {
    redf[quarter * TM + row] = partial_sum;
    __syncthreads();
    const float mean = ((redf[row] + redf[TM + row]) + (redf[2 * TM + row] + redf[3 * TM + row])) * (1.f / kF);
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float4 x = ld4(S + row * SS + c0 + 4 * k);
      const float dx = x.x - mean, dy = x.y - mean, dz = x.z - mean, dw = x.w - mean;
      q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
    }
    float* rq = redf + NQ * TM;
    rq[quarter * TM + row] = q;
    __syncthreads();
    return make_float2(mean, rsqrtf(((rq[row] + rq[TM + row]) + (rq[2 * TM + row] + rq[3 * TM + row])) * (1.f / kF) + kLnEps));
  }
  // rows of the staging tile -> global rows of `width` floats (multiple of 4, at most 128), a warp per row
  __device__ __forceinline__ void flush_rows(float* __restrict__ dst, int ld, int row0, int n, int width) {
    for (int rr = warp; rr < TM; rr += NTHR / 32) {
      const int a = row0 + rr;
      if (a < n && 4 * lane < width) st4(dst + (size_t)a * ld + 4 * lane, ld4(S + rr * SS + 4 * lane));
    }
  }
  // global rows of 128 floats -> registers (rows beyond n read as zero) -> staging tile
  __device__ __forceinline__ void fetch_rows(float4 (&v)[RPW], const float* __restrict__ src, int ld, int row0, int n) const {
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      const int a = row0 + warp + (NTHR / 32) * i;
      v[i] = a < n ? __ldg(reinterpret_cast<const float4*>(src + (size_t)a * ld) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  __device__ __forceinline__ void put_rows(const float4 (&v)[RPW]) {
#pragma unroll
    for (int i = 0; i < RPW; ++i) st4(S + (warp + (NTHR / 32) * i) * SS + 4 * lane, v[i]);
  }
  __device__ __forceinline__ void load_rows(const float* __restrict__ src, int ld, int row0, int n) {
    float4 v[RPW];
    fetch_rows(v, src, ld, row0, n);
    put_rows(v);
  }
};

// ------------------------------------------------------------------------------------------------
// post-attention block, forward:
//   x1 = LN1(xa); x2 = x1 + Dense2(silu(Dense1(silu(x1)))); [yx, gate] = Dense132([x2, inv(ev1)])
//   x3 = x2 + yx; ev2 = ev1 * (1 + gate_l); x4 = LN2(x3); q/k/v rows of the next layer from x4
// saves z1 (hidden pre-activation), x3 and gate for the reverse pass
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHR, 1) atom_post_fwd_tc_kernel(LayerDev L, int n, const float* __restrict__ xa, const float* __restrict__ ev1,
                                                                   float* __restrict__ z1_out, float* __restrict__ x3_out,
                                                                   float* __restrict__ gate_out, float* __restrict__ x4_out,
                                                                   float* __restrict__ ev2_out, const unsigned char* __restrict__ proj_u,
                                                                   float* __restrict__ qkv_next, int* err) {
  extern __shared__ __align__(1024) unsigned char smem[];
  Tile T;
  T.init(smem);
  const int tid = T.tid, warp = T.warp, lane = T.lane, row = T.row, quarter = T.quarter, c0 = T.c0;
  const uint32_t a_smem = smem_u32(T.A), w_smem = smem_u32(smem + kOffW);
  float* S = T.S;
  const int n_tiles = (n + TM - 1) / TM;
  DN_BEGIN();

  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int row0 = tile * TM;
    DN_TILE(31);
    if (tid == 0) T.load_weights(L.res1_u, 65536);
    // xa -> staging tile; per-degree invariants of ev1
    T.load_rows(xa, kF, row0, n);
    if (quarter == 3) {
      const int a = row0 + row;
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      if (a < n) {
#pragma unroll
        for (int m4 = 0; m4 < kMTot / 4; ++m4) {
          const float4 e = __ldg(reinterpret_cast<const float4*>(ev1 + (size_t)a * kMTot) + m4);
          s[degree_of(4 * m4)] += e.x * e.x; s[degree_of(4 * m4 + 1)] += e.y * e.y;
          s[degree_of(4 * m4 + 2)] += e.z * e.z; s[degree_of(4 * m4 + 3)] += e.w * e.w;
        }
      }
      T.inv[row] = make_float4(s[0] * inv_weight(0), s[1] * inv_weight(1), s[2] * inv_weight(2), s[3] * inv_weight(3));
    }
    __syncthreads();
    DN_MARK(0);
    // x1 = LN1(xa) -> residual slot; silu(x1) -> A
    {
      const float2 st = T.row_stats(T.part_row_sum());
      float v[32];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 x = ld4(S + row * SS + c0 + 4 * k);
        const float4 sc = __ldg(reinterpret_cast<const float4*>(L.ln1_s + c0) + k), bi = __ldg(reinterpret_cast<const float4*>(L.ln1_b + c0) + k);
        v[4 * k] = (x.x - st.x) * st.y * sc.x + bi.x; v[4 * k + 1] = (x.y - st.x) * st.y * sc.y + bi.y;
        v[4 * k + 2] = (x.z - st.x) * st.y * sc.z + bi.z; v[4 * k + 3] = (x.w - st.x) * st.y * sc.w + bi.w;
      }
      tmem_st32(T.tlane + kColX + c0, v);
#pragma unroll
      for (int k = 0; k < 32; ++k) v[k] = silu_fast(v[k]);
      a_store32(T.A, c0, row, v);
    }
    T.operands_ready();
    DN_MARK(1);
    if (tid == 0) {
      T.wait_weights();
      DN_MARK(2);
      tc_fence_after();
      issue_gemm(T.tmem, 0, a_smem, 0, w_smem, 32768, 128, 8, 0);
      umma_commit(T.mbar);
    }
    T.wait_mma();
    DN_MARK(3);
    if (tid == 0) T.load_weights(L.res2_u, 65536);
    // z1 = acc + b1 -> staging (saved for the reverse pass); silu(z1) -> A
    {
      float v[32];
      tmem_acc32(T.tlane, c0, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(L.res1_b + c0) + k);
        v[4 * k] += b.x; v[4 * k + 1] += b.y; v[4 * k + 2] += b.z; v[4 * k + 3] += b.w;
        st4(S + row * SS + c0 + 4 * k, make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]));
      }
#pragma unroll
      for (int k = 0; k < 32; ++k) v[k] = silu_fast(v[k]);
      a_store32(T.A, c0, row, v);
    }
    T.operands_ready();
    DN_MARK(4);
    if (tid == 0) {
      T.wait_weights();
      DN_MARK(5);
      tc_fence_after();
      issue_gemm(T.tmem, 0, a_smem, 0, w_smem, 32768, 128, 8, 0);
      umma_commit(T.mbar);
    }
    T.flush_rows(z1_out, kF, row0, n, kF);
    T.wait_mma();
    DN_MARK(6);
    if (tid == 0) T.load_weights(L.exxx_u, 65536);
    // x2 = x1 + acc + b2 -> residual slot and A; the four gate columns of the exchange layer ride along
    {
      float g0 = 0.f, g1 = 0.f, g2 = 0.f, g3 = 0.f;
      float v[32], x1[32];
      tmem_acc32(T.tlane, c0, v);
      tmem_ld32(T.tlane + kColX + c0, x1);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(L.res2_b + c0) + k);
        v[4 * k] += x1[4 * k] + b.x; v[4 * k + 1] += x1[4 * k + 1] + b.y; v[4 * k + 2] += x1[4 * k + 2] + b.z; v[4 * k + 3] += x1[4 * k + 3] + b.w;
      }
      tmem_st32(T.tlane + kColX + c0, v);
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        const float4 w = __ldg(reinterpret_cast<const float4*>(L.ex_xg) + c0 + k);
        g0 = fmaf(v[k], w.x, g0); g1 = fmaf(v[k], w.y, g1); g2 = fmaf(v[k], w.z, g2); g3 = fmaf(v[k], w.w, g3);
      }
      a_store32(T.A, c0, row, v);
      T.red[quarter * TM + row] = make_float4(g0, g1, g2, g3);
    }
    T.operands_ready();
    DN_MARK(7);
    if (tid == 0) {
      T.wait_weights();
      DN_MARK(8);
      tc_fence_after();
      issue_gemm(T.tmem, 0, a_smem, 0, w_smem, 32768, 128, 8, 0);
      umma_commit(T.mbar);
    }
    // gates and ev2 while the exchange contraction runs
    if (quarter == 3) {
      const int a = row0 + row;
      const float4 iv = T.inv[row], ga = T.red[row], gb = T.red[TM + row], gc = T.red[2 * TM + row], gd = T.red[3 * TM + row];
      float g[4] = {(ga.x + gb.x) + (gc.x + gd.x), (ga.y + gb.y) + (gc.y + gd.y), (ga.z + gb.z) + (gc.z + gd.z), (ga.w + gb.w) + (gc.w + gd.w)};
#pragma unroll
      for (int q = 0; q < 4; ++q)
        g[q] += L.ex_bg[q] + iv.x * L.ex_ig[q] + iv.y * L.ex_ig[4 + q] + iv.z * L.ex_ig[8 + q] + iv.w * L.ex_ig[12 + q];
      if (a < n) {
        st4(gate_out + (size_t)a * 4, make_float4(g[0], g[1], g[2], g[3]));
#pragma unroll
        for (int m4 = 0; m4 < kMTot / 4; ++m4) {
          float4 e = __ldg(reinterpret_cast<const float4*>(ev1 + (size_t)a * kMTot) + m4);
          e.x *= 1.f + g[degree_of(4 * m4)]; e.y *= 1.f + g[degree_of(4 * m4 + 1)];
          e.z *= 1.f + g[degree_of(4 * m4 + 2)]; e.w *= 1.f + g[degree_of(4 * m4 + 3)];
          st4(ev2_out + (size_t)a * kMTot + 4 * m4, e);
        }
      }
    }
    T.wait_mma();
    DN_MARK(9);
    if (tid == 0 && proj_u) T.load_weights(proj_u, 4 * kProjBlockBytes);
    // x3 = x2 + acc + bx + inv * Wix -> staging
    float x3_sum = 0.f;
    {
      const float4 iv = T.inv[row];
      float v[32], x2[32];
      tmem_acc32(T.tlane, c0, v);
      tmem_ld32(T.tlane + kColX + c0, x2);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(L.ex_bx + c0) + k);
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(L.ex_ix + c0) + k), w1 = __ldg(reinterpret_cast<const float4*>(L.ex_ix + kF + c0) + k);
        const float4 w2 = __ldg(reinterpret_cast<const float4*>(L.ex_ix + 2 * kF + c0) + k), w3 = __ldg(reinterpret_cast<const float4*>(L.ex_ix + 3 * kF + c0) + k);
        float4 o;
        o.x = x2[4 * k] + v[4 * k] + b.x + iv.x * w0.x + iv.y * w1.x + iv.z * w2.x + iv.w * w3.x;
        o.y = x2[4 * k + 1] + v[4 * k + 1] + b.y + iv.x * w0.y + iv.y * w1.y + iv.z * w2.y + iv.w * w3.y;
        o.z = x2[4 * k + 2] + v[4 * k + 2] + b.z + iv.x * w0.z + iv.y * w1.z + iv.z * w2.z + iv.w * w3.z;
        o.w = x2[4 * k + 3] + v[4 * k + 3] + b.w + iv.x * w0.w + iv.y * w1.w + iv.z * w2.w + iv.w * w3.w;
        st4(S + row * SS + c0 + 4 * k, o);
        x3_sum += (o.x + o.y) + (o.z + o.w);
      }
    }
    tc_fence_before();
    DN_MARK(10);
    // statistics of LayerNorm 2; x3 out
    const float2 st2 = T.row_stats(x3_sum);
    T.flush_rows(x3_out, kF, row0, n, kF);
    __syncthreads();
    DN_MARK(11);
    // x4 = LN2(x3) -> staging (in place) and A
    {
      float v[32];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 x = ld4(S + row * SS + c0 + 4 * k);
        const float4 sc = __ldg(reinterpret_cast<const float4*>(L.ln2_s + c0) + k), bi = __ldg(reinterpret_cast<const float4*>(L.ln2_b + c0) + k);
        v[4 * k] = (x.x - st2.x) * st2.y * sc.x + bi.x; v[4 * k + 1] = (x.y - st2.x) * st2.y * sc.y + bi.y;
        v[4 * k + 2] = (x.z - st2.x) * st2.y * sc.z + bi.z; v[4 * k + 3] = (x.w - st2.x) * st2.y * sc.w + bi.w;
        st4(S + row * SS + c0 + 4 * k, make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]));
      }
      if (proj_u) a_store32(T.A, c0, row, v);
    }
    T.operands_ready();
    DN_MARK(12);
    if (tile + (int)gridDim.x < n_tiles) {   // the next tile's inputs on their way into the L2
      prefetch_tile(xa, kF, (tile + gridDim.x) * TM, n, tid);
      prefetch_tile(ev1, kMTot, (tile + gridDim.x) * TM, n, tid);
    }
    if (proj_u) {
      // q/k/v rows of the next layer in five rounds: heads 0, 1, 2 ([128 x 32] x [32 x 128]: the first four projections side by
      // side), the fifth projection of all heads (four [128 x 32] x [32 x 32]), head 3.  Two accumulator sets (columns
      // [0, 128) + cross at [256, 384), and 128 columns above): the contraction of round r + 1 runs beneath the epilogue of r.
      auto issue_round = [&](int r) {
        const int set = r & 1;
        if (r == 3) {
#pragma unroll 1
          for (int h = 0; h < 4; ++h) issue_gemm(T.tmem, 128 * set + 32 * h, a_smem, 4 * h, w_smem + 3 * kProjBlockBytes + h * 4096, 2048, 32, 2, 0);
        } else {
          const int h = r < 3 ? r : 3;
          issue_gemm(T.tmem, 128 * set, a_smem, 4 * h, w_smem + (r < 3 ? r : 0) * kProjBlockBytes, kProjBlockBytes / 2, 128, 2, 0);
        }
        umma_commit(set ? T.mbar2 : T.mbar);
      };
      if (tid == 0) {
        T.wait_weights();
        tc_fence_after();
        issue_round(0);
        issue_round(1);
      }
      DN_MARK(14);
      T.flush_rows(x4_out, kF, row0, n, kF);
      DN_MARK(15);
#pragma unroll 1
      for (int r = 0; r < 5; ++r) {
        if (r & 1) T.wait_mma2(); else T.wait_mma();
        DN_MARK(16);
        if (tid == 0 && r == 0) T.load_weights(proj_u + 4 * kProjBlockBytes, kProjBlockBytes, 0);   // head 3 takes the place of head 0
        __syncthreads();   // the staging tile has been flushed by every warp
        DN_MARK(17);
        {
          float v[32];
          tmem_acc32(T.tlane, 128 * (r & 1) + c0, v);
#pragma unroll
          for (int k = 0; k < 8; ++k) st4(S + row * SS + c0 + 4 * k, make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]));
        }
        tc_fence_before();
        __syncthreads();
        DN_MARK(18);
        if (tid == 0 && r + 2 < 5) {
          if (r + 2 == 4) T.wait_weights();
          tc_fence_after();
          issue_round(r + 2);
        }
        if (r == 3) {
          T.flush_rows(qkv_next + 4 * kF, kProj, row0, n, kF);
        } else {
          const int h = r < 3 ? r : 3, r4 = lane >> 3, q = lane & 7;
          for (int g = warp; g < TM / 4; g += NTHR / 32) {
            const int rr = 4 * g + r4, a = row0 + rr;
            if (a < n) {
#pragma unroll
              for (int w = 0; w < 4; ++w) st4(qkv_next + (size_t)a * kProj + w * kF + 32 * h + 4 * q, ld4(S + rr * SS + 32 * w + 4 * q));
            }
          }
        }
        DN_MARK(19);
      }
    } else {
      T.flush_rows(x4_out, kF, row0, n, kF);
    }
    __syncthreads();   // staging tile and operand buffers are free for the next tile
    DN_MARK(13);
  }
  T.finish(err);
}


// In the warp-local passes warp w owns rows 8 w .. 8 w + 7 of the tile: lane = (r = lane & 7, ch = lane >> 3) holds the columns
// 8 (4 i + ch) .. + 7 of row 8 w + r for i = 0..3.  A warp instruction then touches one 128-byte line per row, the 16-byte
// operand chunks of a quarter warp are contiguous, and a row reduction is a per-thread sum plus two shuffles.
__device__ __forceinline__ float quad_sum_ch(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 16);
  return v;
}
__device__ __forceinline__ void ldg8(const float* __restrict__ p, float* v) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
// the same through the coherent path: for rows this kernel overwrites later on
__device__ __forceinline__ void ld8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void lds8(const float* p, float* v) {
  const float4 a = ld4(p), b = ld4(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void sts8(float* p, const float* v) {
  st4(p, make_float4(v[0], v[1], v[2], v[3]));
  st4(p + 4, make_float4(v[4], v[5], v[6], v[7]));
}
__device__ __forceinline__ int degree_start(int l) { return l == 0 ? 0 : (l == 1 ? 3 : (l == 2 ? 8 : 15)); }

// ------------------------------------------------------------------------------------------------
// post-attention block, reverse.  in: g4 = dL/dx4 (or, with projT_u: the rows of g_xa left by the layer above + the transposed
// q/k/v projections of that layer's g_qkv), gev2 = dL/dev2; out: g_xa = dL/dxa, gev1 = dL/dev1
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHR, 1) atom_post_bwd_tc_kernel(LayerDev L, int n, const float* __restrict__ xa, const float* __restrict__ ev1,
                                                                   const float* __restrict__ z1, const float* __restrict__ x3,
                                                                   const float* __restrict__ gate, const float* __restrict__ g4,
                                                                   const float* __restrict__ gev2, float* g_xa, float* __restrict__ gev1,
                                                                   const unsigned char* __restrict__ projT_u, const float* __restrict__ g_qkv_up,
                                                                   int* err) {
  extern __shared__ __align__(1024) unsigned char smem[];
  Tile T;
  T.init(smem);
  const int tid = T.tid, warp = T.warp, lane = T.lane, row = T.row, quarter = T.quarter, c0 = T.c0;
  const uint32_t a_smem = smem_u32(T.A), w_smem = smem_u32(smem + kOffW);
  unsigned char* A1 = smem + kOffS;   // second operand buffer inside the staging region (projection rounds only)
  float* S = T.S;
  const int wr = 8 * warp + (lane & 7), ch = lane >> 3;
  const int n_tiles = (n + TM - 1) / TM;
  DN_BEGIN();

  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int row0 = tile * TM;
    const int aw = row0 + wr;
    DN_TILE(63);
    if (projT_u) {
      // g4 = g_xa (skip connection of the layer above) + sum_w g_qkv[:, w] * W_w^T, block-diagonal over the heads: five rounds,
      // the operand of round w converted from global memory by each warp for its own rows while round w - 1 runs
      if (tid == 0) T.load_weights(projT_u, 4 * kProjBlockBytes);
      float sl[4][8];   // this thread's share of the slab of the coming round
      auto fetch_slab = [&](int w) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (aw < n) ldg8(g_qkv_up + (size_t)aw * kProj + w * kF + 8 * (4 * i + ch), sl[i]);
          else {
#pragma unroll
            for (int k = 0; k < 8; ++k) sl[i][k] = 0.f;
          }
        }
      };
      fetch_slab(0);
      // the rest of this tile's inputs on their way into the L2 meanwhile
      prefetch_tile(x3, kF, row0, n, tid); prefetch_tile(g_xa, kF, row0, n, tid);
      prefetch_tile(z1, kF, row0, n, tid); prefetch_tile(xa, kF, row0, n, tid);
#pragma unroll 1
      for (int w = 0; w < 5; ++w) {
        DN_MARK(40);
        if (w >= 2) { if (w & 1) T.wait_mma2(); else T.wait_mma(); }   // the MMAs that read this operand buffer have completed
        DN_MARK(41);
        if (tid == 0 && w == 2) T.load_weights(projT_u + 4 * kProjBlockBytes, kProjBlockBytes, 0);   // w = 4 takes the place of w = 0
        unsigned char* Aw = (w & 1) ? A1 : T.A;
#pragma unroll
        for (int i = 0; i < 4; ++i) a_store8(Aw, 4 * i + ch, wr, sl[i]);
        if (w < 4) fetch_slab(w + 1);
        DN_MARK(42);
        T.operands_ready();
        DN_MARK(43);
        if (tid == 0) {
          if (w == 0 || w == 4) T.wait_weights();
          DN_MARK(44);
          tc_fence_after();
#pragma unroll 1
          for (int h = 0; h < 4; ++h)
            issue_gemm(T.tmem, 32 * h, smem_u32(Aw), 4 * h, w_smem + (w < 4 ? w : 0) * kProjBlockBytes + h * 4096, 2048, 32, 2, w > 0);
          umma_commit((w & 1) ? T.mbar2 : T.mbar);
          DN_MARK(45);
        }
      }
      DN_MARK(40);
      T.wait_mma2();
      T.wait_mma();
      DN_MARK(46);
      if (tid == 0) T.load_weights(L.exxxT_u, 65536);
      {
        float v[32];
        tmem_acc32(T.tlane, c0, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) st4(S + row * SS + c0 + 4 * k, make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]));
      }
      tc_fence_before();
      __syncthreads();
      DN_MARK(47);
    } else {
      if (tid == 0) T.load_weights(L.exxxT_u, 65536);
      prefetch_tile(z1, kF, row0, n, tid); prefetch_tile(xa, kF, row0, n, tid);
    }
    DN_MARK(32);
    // LayerNorm-2 reverse (warp-local): g3 -> staging tile and A; cotangents of the gates and of the invariants; gev1 out
    {
      float xh[4][8], gy[4][8];
      // everything this phase reads from global memory is requested before the first use
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 8 * (4 * i + ch);
        if (aw < n) {
          ldg8(x3 + (size_t)aw * kF + c, xh[i]);
          if (projT_u) ld8(g_xa + (size_t)aw * kF + c, gy[i]);
          else ldg8(g4 + (size_t)aw * kF + c, gy[i]);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) { xh[i][k] = 0.f; gy[i][k] = 0.f; }
        }
      }
      const int m0 = degree_start(ch), nm = 3 + 2 * ch;   // lane (r, ch): degree l = ch of row r
      float e1[9], e2[9];
#pragma unroll
      for (int m = 0; m < 9; ++m) {
        const bool on = aw < n && m < nm;
        e2[m] = on ? __ldg(gev2 + (size_t)aw * kMTot + m0 + m) : 0.f;
        e1[m] = on ? __ldg(ev1 + (size_t)aw * kMTot + m0 + m) : 0.f;
      }
      const float gate_l = aw < n ? __ldg(gate + (size_t)aw * 4 + ch) : 0.f;
      DN_MARK(48);
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) s += xh[i][k];
      const float mean = quad_sum_ch(s) * (1.f / kF);
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) { xh[i][k] -= mean; q = fmaf(xh[i][k], xh[i][k], q); }
      const float rs = rsqrtf(quad_sum_ch(q) * (1.f / kF) + kLnEps);
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 8 * (4 * i + ch);
        float sc[8];
        ldg8(L.ln2_s + c, sc);
        if (projT_u) {
          float g[8];
          lds8(S + wr * SS + c, g);
#pragma unroll
          for (int k = 0; k < 8; ++k) gy[i][k] += g[k];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[i][k] *= rs;
          gy[i][k] *= sc[k];
          s1 += gy[i][k];
          s2 = fmaf(gy[i][k], xh[i][k], s2);
        }
      }
      s1 = quad_sum_ch(s1) * (1.f / kF);
      s2 = quad_sum_ch(s2) * (1.f / kF);
      DN_MARK(49);
      float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 8 * (4 * i + ch);
        float w0[8], w1[8], w2[8], w3[8];
        ldg8(L.ex_ix + c, w0); ldg8(L.ex_ix + kF + c, w1); ldg8(L.ex_ix + 2 * kF + c, w2); ldg8(L.ex_ix + 3 * kF + c, w3);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float g3 = rs * (gy[i][k] - s1 - xh[i][k] * s2);
          gy[i][k] = g3;
          p0 = fmaf(g3, w0[k], p0); p1 = fmaf(g3, w1[k], p1); p2 = fmaf(g3, w2[k], p2); p3 = fmaf(g3, w3[k], p3);
        }
        sts8(S + wr * SS + c, gy[i]);
        a_store8(T.A, 4 * i + ch, wr, gy[i]);
      }
      p0 = quad_sum_ch(p0); p1 = quad_sum_ch(p1); p2 = quad_sum_ch(p2); p3 = quad_sum_ch(p3);
      DN_MARK(50);
      float gg = 0.f;
#pragma unroll
      for (int m = 0; m < 9; ++m) gg = fmaf(e2[m], e1[m], gg);
      const int rl = lane & 7;
      const float gg0 = __shfl_sync(0xffffffffu, gg, rl), gg1 = __shfl_sync(0xffffffffu, gg, rl + 8);
      const float gg2 = __shfl_sync(0xffffffffu, gg, rl + 16), gg3 = __shfl_sync(0xffffffffu, gg, rl + 24);
      const float pl = ch == 0 ? p0 : (ch == 1 ? p1 : (ch == 2 ? p2 : p3));
      const float ginv = pl + gg0 * L.ex_ig[ch * 4] + gg1 * L.ex_ig[ch * 4 + 1] + gg2 * L.ex_ig[ch * 4 + 2] + gg3 * L.ex_ig[ch * 4 + 3];
      if (aw < n) {
        const float gt = 1.f + gate_l, f = 2.f * ginv * inv_weight(ch);
#pragma unroll
        for (int m = 0; m < 9; ++m)
          if (m < nm) gev1[(size_t)aw * kMTot + m0 + m] = e2[m] * gt + f * e1[m];
      }
      if (ch == 0) T.red[wr] = make_float4(gg0, gg1, gg2, gg3);
    }
    T.operands_ready();
    DN_MARK(33);
    if (tid == 0) {
      T.wait_weights();
      tc_fence_after();
      issue_gemm(T.tmem, 0, a_smem, 0, w_smem, 32768, 128, 8, 0);
      umma_commit(T.mbar);
    }
    T.wait_mma();
    DN_MARK(34);
    if (tid == 0) T.load_weights(L.res2T_u, 65536);
    // g_x2 = g3 + g3 Wxx^T + ggate Wxg^T -> residual slot and A
    {
      float v[32];
      tmem_acc32(T.tlane, c0, v);
      const float4 gg = T.red[row];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 g3 = ld4(S + row * SS + c0 + 4 * k);
        const float4 wa = __ldg(reinterpret_cast<const float4*>(L.ex_xg) + c0 + 4 * k), wb = __ldg(reinterpret_cast<const float4*>(L.ex_xg) + c0 + 4 * k + 1);
        const float4 wc = __ldg(reinterpret_cast<const float4*>(L.ex_xg) + c0 + 4 * k + 2), wd = __ldg(reinterpret_cast<const float4*>(L.ex_xg) + c0 + 4 * k + 3);
        v[4 * k] += g3.x + gg.x * wa.x + gg.y * wa.y + gg.z * wa.z + gg.w * wa.w;
        v[4 * k + 1] += g3.y + gg.x * wb.x + gg.y * wb.y + gg.z * wb.z + gg.w * wb.w;
        v[4 * k + 2] += g3.z + gg.x * wc.x + gg.y * wc.y + gg.z * wc.z + gg.w * wc.w;
        v[4 * k + 3] += g3.w + gg.x * wd.x + gg.y * wd.y + gg.z * wd.z + gg.w * wd.w;
      }
      tmem_st32(T.tlane + kColX + c0, v);
      a_store32(T.A, c0, row, v);
    }
    T.operands_ready();
    DN_MARK(35);
    if (tid == 0) {
      T.wait_weights();
      tc_fence_after();
      issue_gemm(T.tmem, 0, a_smem, 0, w_smem, 32768, 128, 8, 0);
      umma_commit(T.mbar);
    }
    T.load_rows(z1, kF, row0, n);
    T.wait_mma();
    if (tid == 0) T.load_weights(L.res1T_u, 65536);
    __syncthreads();
    DN_MARK(36);
    // residual MLP reverse, second layer: (g_x2 W2^T) * silu'(z1) -> A
    {
      float v[32];
      tmem_acc32(T.tlane, c0, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 z = ld4(S + row * SS + c0 + 4 * k);
        v[4 * k] *= dsilu_fast(z.x); v[4 * k + 1] *= dsilu_fast(z.y); v[4 * k + 2] *= dsilu_fast(z.z); v[4 * k + 3] *= dsilu_fast(z.w);
      }
      a_store32(T.A, c0, row, v);
    }
    T.operands_ready();
    DN_MARK(37);
    if (tid == 0) {
      T.wait_weights();
      tc_fence_after();
      issue_gemm(T.tmem, 0, a_smem, 0, w_smem, 32768, 128, 8, 0);
      umma_commit(T.mbar);
    }
    // normalised xa -> staging tile, 1 / std -> stat (warp-local) while the contraction runs
    {
      float x[4][8];
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (aw < n) ldg8(xa + (size_t)aw * kF + 8 * (4 * i + ch), x[i]);
        else {
#pragma unroll
          for (int k = 0; k < 8; ++k) x[i][k] = 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) s += x[i][k];
      }
      const float mean = quad_sum_ch(s) * (1.f / kF);
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) { x[i][k] -= mean; q = fmaf(x[i][k], x[i][k], q); }
      const float rs = rsqrtf(quad_sum_ch(q) * (1.f / kF) + kLnEps);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int k = 0; k < 8; ++k) x[i][k] *= rs;
        sts8(S + wr * SS + 8 * (4 * i + ch), x[i]);
      }
      if (ch == 0) T.stat[wr] = make_float2(mean, rs);
    }
    T.wait_mma();
    __syncthreads();
    DN_MARK(38);
    // g_x1 = g_x2 + (t W1^T) * silu'(x1); LayerNorm-1 reverse -> g_xa
    {
      float gy[32], xh[32];
      tmem_acc32(T.tlane, c0, gy);
      {
        float gx2[32];
        tmem_ld32(T.tlane + kColX + c0, gx2);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float4 h = ld4(S + row * SS + c0 + 4 * k);
          const float4 sc = __ldg(reinterpret_cast<const float4*>(L.ln1_s + c0) + k), bi = __ldg(reinterpret_cast<const float4*>(L.ln1_b + c0) + k);
          xh[4 * k] = h.x; xh[4 * k + 1] = h.y; xh[4 * k + 2] = h.z; xh[4 * k + 3] = h.w;
          gy[4 * k] = (gx2[4 * k] + gy[4 * k] * dsilu_fast(h.x * sc.x + bi.x)) * sc.x;
          gy[4 * k + 1] = (gx2[4 * k + 1] + gy[4 * k + 1] * dsilu_fast(h.y * sc.y + bi.y)) * sc.y;
          gy[4 * k + 2] = (gx2[4 * k + 2] + gy[4 * k + 2] * dsilu_fast(h.z * sc.z + bi.z)) * sc.z;
          gy[4 * k + 3] = (gx2[4 * k + 3] + gy[4 * k + 3] * dsilu_fast(h.w * sc.w + bi.w)) * sc.w;
        }
      }
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int k = 0; k < 32; ++k) { s1 += gy[k]; s2 = fmaf(gy[k], xh[k], s2); }
      T.redf[quarter * TM + row] = s1;
      T.redf[NQ * TM + quarter * TM + row] = s2;
      tc_fence_before();
      __syncthreads();
      const float* r2 = T.redf + NQ * TM;
      s1 = ((T.redf[row] + T.redf[TM + row]) + (T.redf[2 * TM + row] + T.redf[3 * TM + row])) * (1.f / kF);
      s2 = ((r2[row] + r2[TM + row]) + (r2[2 * TM + row] + r2[3 * TM + row])) * (1.f / kF);
      const float rs = T.stat[row].y;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        st4(S + row * SS + c0 + 4 * k, make_float4(rs * (gy[4 * k] - s1 - xh[4 * k] * s2), rs * (gy[4 * k + 1] - s1 - xh[4 * k + 1] * s2),
                                                   rs * (gy[4 * k + 2] - s1 - xh[4 * k + 2] * s2), rs * (gy[4 * k + 3] - s1 - xh[4 * k + 3] * s2)));
    }
    __syncthreads();
    T.flush_rows(g_xa, kF, row0, n, kF);
    __syncthreads();   // staging tile, operand buffers and the reduction arrays are free for the next tile
    DN_MARK(39);
  }
  T.finish(err);
}


// rows of 64 floats -> staging tile (two rows per warp instruction; rows beyond n read as zero)
__device__ __forceinline__ void load_rows64(Tile& T, const float* __restrict__ src, int row0, int n) {
  const int sub = T.lane >> 4, c = 4 * (T.lane & 15);
#pragma unroll
  for (int i = 0; i < TM / (2 * (NTHR / 32)); ++i) {
    const int rr = 2 * (T.warp + (NTHR / 32) * i) + sub, a = row0 + rr;
    const float4 v = a < n ? __ldg(reinterpret_cast<const float4*>(src + (size_t)a * 64 + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
    st4(T.S + rr * SS + c, v);
  }
}
__device__ __forceinline__ void flush_rows64(Tile& T, float* __restrict__ dst, int row0, int n) {
  const int sub = T.lane >> 4, c = 4 * (T.lane & 15);
#pragma unroll
  for (int i = 0; i < TM / (2 * (NTHR / 32)); ++i) {
    const int rr = 2 * (T.warp + (NTHR / 32) * i) + sub, a = row0 + rr;
    if (a < n) st4(dst + (size_t)a * 64 + c, ld4(T.S + rr * SS + c));
  }
}

// ------------------------------------------------------------------------------------------------
// output heads, forward: per-atom NN energy, raw partial charge, signed Hirshfeld value.
//   e = (fin_e . silu(x W_e + b_e) + c_e) scale[Z] + offset[Z];  q = fin_q . silu(x W_q + b_q) + c_q + embed_q[Z];
//   hv = embed0[Z] + ((silu(x W_h1 + b_h1) W_h2 + b_h2) . embed1[Z]) / 8
// saves the pre-activations ze, zq, zh for the reverse pass
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHR, 1) heads_fwd_tc_kernel(ModelDev M, int n, const int* __restrict__ Z, const float* __restrict__ x,
                                                               float* __restrict__ ze, float* __restrict__ zq, float* __restrict__ zh,
                                                               float* __restrict__ e_nn, float* __restrict__ q_raw, float* __restrict__ hv,
                                                               int* err) {
  extern __shared__ __align__(1024) unsigned char smem[];
  Tile T;
  T.init(smem);
  const int tid = T.tid, warp = T.warp, lane = T.lane, row = T.row, quarter = T.quarter, c0 = T.c0;
  const uint32_t a_smem = smem_u32(T.A), w_smem = smem_u32(smem + kOffW);
  float* S = T.S;
  const int wr = 8 * warp + (lane & 7), ch = lane >> 3;
  const int n_tiles = (n + TM - 1) / TM;

  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int row0 = tile * TM;
    if (tid == 0) T.load_weights(M.e_reg_u, 65536);
    {   // x -> A (warp-local)
      const int aw = row0 + wr;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v[8];
        if (aw < n) ldg8(x + (size_t)aw * kF + 8 * (4 * i + ch), v);
        else {
#pragma unroll
          for (int k = 0; k < 8; ++k) v[k] = 0.f;
        }
        a_store8(T.A, 4 * i + ch, wr, v);
      }
    }
    T.operands_ready();
    // energy and charge heads share the structure Dense(128) -> silu -> dot
#pragma unroll 1
    for (int head = 0; head < 2; ++head) {
      if (tid == 0) {
        T.wait_weights();
        tc_fence_after();
        issue_gemm(T.tmem, 0, a_smem, 0, w_smem, 32768, 128, 8, 0);
        umma_commit(T.mbar);
      }
      if (head == 1) T.flush_rows(ze, kF, row0, n, kF);      // the first head's pre-activations leave beneath the second contraction
      T.wait_mma();
      if (tid == 0) {
        if (head == 0) T.load_weights(M.q_reg_u, 65536);
        else {      // both Hirshfeld kernels: [128 x 64] at the start of the buffer, [64 x 64] 32 KB above
          mbar_expect_tx(T.wbar, 32768 + 16384);
          bulk_load(w_smem, M.h_reg_u, 32768, T.wbar);
          bulk_load(w_smem + 32768, M.h_fin_u, 16384, T.wbar);
        }
      }
      __syncthreads();      // the staging tile has been flushed by every warp
      {
        const float* bias = head == 0 ? M.e_reg_b : M.q_reg_b;
        const float* fin = head == 0 ? M.e_fin_k : M.q_fin_k;
        float v[32];
        tmem_acc32(T.tlane, c0, v);
        float part = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float4 b = __ldg(reinterpret_cast<const float4*>(bias + c0) + k), f = __ldg(reinterpret_cast<const float4*>(fin + c0) + k);
          v[4 * k] += b.x; v[4 * k + 1] += b.y; v[4 * k + 2] += b.z; v[4 * k + 3] += b.w;
          st4(S + row * SS + c0 + 4 * k, make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]));
          part = fmaf(silu_fast(v[4 * k]), f.x, fmaf(silu_fast(v[4 * k + 1]), f.y, fmaf(silu_fast(v[4 * k + 2]), f.z, fmaf(silu_fast(v[4 * k + 3]), f.w, part))));
        }
        T.redf[quarter * TM + row] = part;
      }
      tc_fence_before();
      __syncthreads();
      if (tid < TM) {
        const int a = row0 + tid;
        if (a < n) {
          const float s = (T.redf[tid] + T.redf[TM + tid]) + (T.redf[2 * TM + tid] + T.redf[3 * TM + tid]);
          int z = Z[a];
          if (head == 0) {
            z = z < 0 ? 0 : (z >= kZEmbed ? kZEmbed - 1 : z);
            e_nn[a] = (s + M.e_fin_b) * M.e_scale[z] + M.e_offset[z];
          } else {
            z = z < 0 ? 0 : (z >= kZHead ? kZHead - 1 : z);
            q_raw[a] = s + M.q_fin_b + M.q_embed[z];
          }
        }
      }
    }
    // Hirshfeld: 128 -> 64 -> 64, then the dot product with the element's query
    if (tid == 0) {
      T.wait_weights();
      tc_fence_after();
      issue_gemm(T.tmem, 0, a_smem, 0, w_smem, 16384, 64, 8, 0);
      umma_commit(T.mbar);
    }
    T.flush_rows(zq, kF, row0, n, kF);
    T.wait_mma();
    __syncthreads();
    if (quarter < 2) {
      float v[32];
      tmem_acc32(T.tlane, c0, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(M.h_reg_b + c0) + k);
        v[4 * k] += b.x; v[4 * k + 1] += b.y; v[4 * k + 2] += b.z; v[4 * k + 3] += b.w;
        st4(S + row * SS + c0 + 4 * k, make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]));
      }
#pragma unroll
      for (int k = 0; k < 32; ++k) v[k] = silu_fast(v[k]);
      a_store32(T.A, c0, row, v);
    }
    T.operands_ready();
    if (tid == 0) {
      tc_fence_after();
      issue_gemm(T.tmem, 0, a_smem, 0, w_smem + 32768, 8192, 64, 4, 0);
      umma_commit(T.mbar);
    }
    flush_rows64(T, zh, row0, n);
    T.wait_mma();
    {
      float part = 0.f;
      if (quarter < 2) {
        const int a = row0 + row;
        int z = a < n ? Z[a] : 0;
        z = z < 0 ? 0 : (z >= kZHead ? kZHead - 1 : z);
        float v[32];
        tmem_acc32(T.tlane, c0, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float4 b = __ldg(reinterpret_cast<const float4*>(M.h_fin_b + c0) + k);
          const float4 e = __ldg(reinterpret_cast<const float4*>(M.h_embed1 + (size_t)z * 64 + c0) + k);
          part = fmaf(v[4 * k] + b.x, e.x, fmaf(v[4 * k + 1] + b.y, e.y, fmaf(v[4 * k + 2] + b.z, e.z, fmaf(v[4 * k + 3] + b.w, e.w, part))));
        }
      }
      T.redf[quarter * TM + row] = part;
    }
    tc_fence_before();
    __syncthreads();
    if (tid < TM) {
      const int a = row0 + tid;
      if (a < n) {
        int z = Z[a];
        z = z < 0 ? 0 : (z >= kZHead ? kZHead - 1 : z);
        hv[a] = M.h_embed0[z] + (T.redf[tid] + T.redf[TM + tid]) * 0.125f;
      }
    }
    __syncthreads();   // staging tile, operand buffer and reduction arrays are free for the next tile
  }
  T.finish(err);
}

// ------------------------------------------------------------------------------------------------
// output heads, reverse: gx = dL/dx_final from the cotangents of e_nn (ge), of the raw charge (gq) and of the Hirshfeld ratio (gh)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHR, 1) heads_bwd_tc_kernel(ModelDev M, int n, const int* __restrict__ Z, const float* __restrict__ ze,
                                                               const float* __restrict__ zq, const float* __restrict__ zh,
                                                               const float* __restrict__ hv, const float* __restrict__ ge,
                                                               const float* __restrict__ gq, const float* __restrict__ gh,
                                                               float* __restrict__ gx, int* err) {
  extern __shared__ __align__(1024) unsigned char smem[];
  Tile T;
  T.init(smem);
  const int tid = T.tid, warp = T.warp, lane = T.lane, row = T.row, quarter = T.quarter, c0 = T.c0;
  const uint32_t a_smem = smem_u32(T.A), w_smem = smem_u32(smem + kOffW);
  unsigned char* A1 = smem + kOffS;   // second operand buffer inside the staging region
  float* S = T.S;
  const int wr = 8 * warp + (lane & 7), ch = lane >> 3;
  const int n_tiles = (n + TM - 1) / TM;

  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int row0 = tile * TM;
    const int aw = row0 + wr;
    if (tid == 0) {      // h_fin^T [64 x 64] at the start of the buffer, h_reg^T [64 x 128] 16 KB above
      mbar_expect_tx(T.wbar, 16384 + 32768);
      bulk_load(w_smem, M.h_finT_u, 16384, T.wbar);
      bulk_load(w_smem + 16384, M.h_regT_u, 32768, T.wbar);
    }
    // per-row coefficients (every lane of a row's quad computes them)
    float c_e = 0.f, c_q = 0.f, c_h = 0.f;
    int zz = 0;
    if (aw < n) {
      const int z = Z[aw];
      const int ze_ = z < 0 ? 0 : (z >= kZEmbed ? kZEmbed - 1 : z);
      zz = z < 0 ? 0 : (z >= kZHead ? kZHead - 1 : z);
      c_e = ge[aw] * M.e_scale[ze_];
      c_q = gq[aw];
      c_h = gh[aw] * (hv[aw] < 0.f ? -0.125f : 0.125f);
    }
    // Hirshfeld branch: g_k = c_h embed1[Z] -> A (K = 64: chunks 0..7, two per lane); zh -> staging tile
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float v[8];
      ldg8(M.h_embed1 + (size_t)zz * 64 + 8 * (4 * i + ch), v);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] *= c_h;
      a_store8(T.A, 4 * i + ch, wr, v);
    }
    load_rows64(T, zh, row0, n);
    T.operands_ready();
    if (tid == 0) {
      T.wait_weights();
      tc_fence_after();
      issue_gemm(T.tmem, 128, a_smem, 0, w_smem, 8192, 64, 4, 0);      // g_sh = g_k H_fin^T into columns [128, 192)
      umma_commit(T.mbar);
    }
    T.wait_mma();
    if (quarter < 2) {      // g_zh = g_sh * silu'(zh) -> A
      float v[32];
      tmem_acc32(T.tlane, 128 + c0, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 z = ld4(S + row * SS + c0 + 4 * k);
        v[4 * k] *= dsilu_fast(z.x); v[4 * k + 1] *= dsilu_fast(z.y); v[4 * k + 2] *= dsilu_fast(z.z); v[4 * k + 3] *= dsilu_fast(z.w);
      }
      a_store32(T.A, c0, row, v);
    }
    T.operands_ready();      // also: every thread is done with the staging tile, which now becomes the second operand buffer
    if (tid == 0) {
      tc_fence_after();
      issue_gemm(T.tmem, 0, a_smem, 0, w_smem + 16384, 16384, 128, 4, 0);      // gx = g_zh H_reg^T
      umma_commit(T.mbar);
    }
    // energy branch operand (warp-local): c_e fin_e silu'(ze) -> second buffer
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = 8 * (4 * i + ch);
      float v[8], f[8];
      if (aw < n) ldg8(ze + (size_t)aw * kF + c, v);
      else {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = 0.f;
      }
      ldg8(M.e_fin_k + c, f);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = c_e * f[k] * dsilu_fast(v[k]);
      a_store8(A1, 4 * i + ch, wr, v);
    }
    T.wait_mma();      // the Hirshfeld kernels have been read: their buffer takes the energy head's kernel
    if (tid == 0) T.load_weights(M.e_regT_u, 65536);
    // charge branch operand -> first buffer (its readers have completed)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = 8 * (4 * i + ch);
      float v[8], f[8];
      if (aw < n) ldg8(zq + (size_t)aw * kF + c, v);
      else {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = 0.f;
      }
      ldg8(M.q_fin_k + c, f);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = c_q * f[k] * dsilu_fast(v[k]);
      a_store8(T.A, 4 * i + ch, wr, v);
    }
    T.operands_ready();
    if (tid == 0) {
      T.wait_weights();
      tc_fence_after();
      issue_gemm(T.tmem, 0, smem_u32(A1), 0, w_smem, 32768, 128, 8, 1);      // gx += g_ze E_reg^T
      umma_commit(T.mbar);
    }
    T.wait_mma();
    if (tid == 0) {
      T.load_weights(M.q_regT_u, 65536);
      T.wait_weights();
      tc_fence_after();
      issue_gemm(T.tmem, 0, a_smem, 0, w_smem, 32768, 128, 8, 1);      // gx += g_zq Q_reg^T
      umma_commit(T.mbar);
    }
    T.wait_mma();
    {
      float v[32];
      tmem_acc32(T.tlane, c0, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) st4(S + row * SS + c0 + 4 * k, make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]));
    }
    tc_fence_before();
    __syncthreads();
    T.flush_rows(gx, kF, row0, n, kF);
    __syncthreads();   // staging tile and operand buffers are free for the next tile
  }
  T.finish(err);
}

}  // namespace

void dense_debug_print() {
#ifdef SO3LR_TC_TIMING
  long long h[64];
  cudaDeviceSynchronize();
  if (cudaMemcpyFromSymbol(h, g_dense_dbg, sizeof(h)) != cudaSuccess) return;
  for (int base = 0; base < 64; base += 32) {
    if (!h[base + 31]) continue;
    std::fprintf(stderr, "dense tc %s phases (cycles per tile, %lld tiles):", base ? "bwd" : "fwd", h[base + 31]);
    for (int k = 0; k < 24; ++k) std::fprintf(stderr, " %lld", h[base + k] / h[base + 31]);
    std::fprintf(stderr, "\n");
  }
#endif
}

int configure_dense_tc_kernels() {
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(atom_post_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDense));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(atom_post_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDense));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(heads_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDense));
  SO3LR_CUDA_CHECK(cudaFuncSetAttribute(heads_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDense));
  return kOk;
}

void launch_atom_post_fwd_tc(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, float* z1, float* x3, float* gate,
                             float* x4, float* ev2, const unsigned char* proj_u, float* qkv_next, int* err) {
  if (n <= 0) return;
  const int tiles = (n + TM - 1) / TM, grid = tiles < sm_count() ? tiles : sm_count();
  atom_post_fwd_tc_kernel<<<grid, NTHR, kSmemDense, s>>>(L, n, xa, ev1, z1, x3, gate, x4, ev2, proj_u, qkv_next, err);
  count_launch();
}

void launch_atom_post_bwd_tc(cudaStream_t s, const LayerDev& L, int n, const float* xa, const float* ev1, const float* z1, const float* x3,
                             const float* gate, const float* g4, const float* gev2, float* g_xa, float* gev1, const unsigned char* projT_u,
                             const float* g_qkv_up, int* err) {
  if (n <= 0) return;
  const int tiles = (n + TM - 1) / TM, grid = tiles < sm_count() ? tiles : sm_count();
  atom_post_bwd_tc_kernel<<<grid, NTHR, kSmemDense, s>>>(L, n, xa, ev1, z1, x3, gate, g4, gev2, g_xa, gev1, projT_u, g_qkv_up, err);
  count_launch();
}

void launch_heads_fwd_tc(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* x, float* ze, float* zq, float* zh, float* e_nn,
                         float* q_raw, float* hv, int* err) {
  if (n <= 0) return;
  const int tiles = (n + TM - 1) / TM, grid = tiles < sm_count() ? tiles : sm_count();
  heads_fwd_tc_kernel<<<grid, NTHR, kSmemDense, s>>>(M, n, Z, x, ze, zq, zh, e_nn, q_raw, hv, err);
  count_launch();
}
void launch_heads_bwd_tc(cudaStream_t s, const ModelDev& M, int n, const int* Z, const float* ze, const float* zq, const float* zh,
                         const float* hv, const float* ge, const float* gq, const float* gh, float* gx, int* err) {
  if (n <= 0) return;
  const int tiles = (n + TM - 1) / TM, grid = tiles < sm_count() ? tiles : sm_count();
  heads_bwd_tc_kernel<<<grid, NTHR, kSmemDense, s>>>(M, n, Z, ze, zq, zh, hv, ge, gq, gh, gx, err);
  count_launch();
}

}  // namespace so3lr

// Neighbor list for callers that must not allocate device memory.
//
// An XLA custom-call handler (the way so3lr's jitted `nbrs.update` would reach this library) runs while XLA's own
// allocator holds most of the GPU's memory in a pre-reserved pool, so a cudaMalloc issued from inside the handler can
// fail for lack of memory and, when it succeeds, stalls every stream of the device.  The same holds for any host
// program that hands its GPU memory out from a fixed arena.  so3lr_b200_neighbor_list_noalloc therefore builds a
// jax-md style pair list using only the caller's buffers plus one fixed scratch array that lives in the library
// image: kRowScratch below, 2 x (SO3LR_B200_NOALLOC_MAX_ATOMS + 1) int32 = 128 KiB + 8 bytes, resident on every GPU that loads
// the library until the process exits.
//
// All calls (from any thread or stream) share that array on a device: two calls whose kernels overlap on the GPU race
// on it.  Every word a call reads is written by the same call first (row counts, then their scan), so nothing has to
// be cleared between calls.
#include "../../include/so3lr_b200.h"

#include <cstring>
#include <mutex>

#include "common.cuh"

using namespace so3lr;

namespace {

constexpr int kMaxAtoms = SO3LR_B200_NOALLOC_MAX_ATOMS;
constexpr int kMaxDevices = 64;

// [0 .. kMaxAtoms] row counts, [kMaxAtoms + 1 .. 2 kMaxAtoms + 1] row starts
static __device__ __align__(256) int kRowScratch[2 * (kMaxAtoms + 1)];

// One warp per centre atom i scans all atoms j in ascending order.  FILL = false counts the row, FILL = true writes it.
template <bool FILL>
__global__ void __launch_bounds__(256) rows_all_pairs_kernel(Cell cell, int n, const float* __restrict__ R, float r2max, int ordered,
                                                             int* __restrict__ row_count, const int* __restrict__ row_start,
                                                             int* __restrict__ idx, long long capacity) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= n) return;
  const float xi = R[3 * (size_t)i], yi = R[3 * (size_t)i + 1], zi = R[3 * (size_t)i + 2];
  const long long base = FILL ? row_start[i] : 0;
  int count = 0;
  for (int j0 = 0; j0 < n; j0 += 32) {
    const int j = j0 + lane;
    bool hit = false;
    if (j < n) {
      float dx = R[3 * (size_t)j] - xi, dy = R[3 * (size_t)j + 1] - yi, dz = R[3 * (size_t)j + 2] - zi;
      min_image(cell, dx, dy, dz);
      hit = dist2_rn(dx, dy, dz) < r2max && (ordered ? j > i : j != i);
    }
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (FILL && hit) {
      const long long pos = base + count + __popc(m & ((1u << lane) - 1u));
      if (pos < capacity) { idx[pos] = i; idx[capacity + pos] = j; }
    }
    count += __popc(m);
  }
  if (!FILL && lane == 0) row_count[i] = count;
}

// Exclusive scan of n <= kMaxAtoms row counts by a single CTA of 1024 threads; also reports the total and the overflow flag.
__global__ void __launch_bounds__(1024) scan_rows_kernel(int n, const int* __restrict__ row_count, int* __restrict__ row_start,
                                                         long long capacity, long long* __restrict__ count_out,
                                                         int* __restrict__ overflow_out) {
  __shared__ long long warp_tot[32];
  __shared__ long long carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < n; base += 1024) {
    const int k = base + threadIdx.x;
    const long long v = k < n ? row_count[k] : 0;
    long long s = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      long long t = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += t;
    }
    if (lane == 31) warp_tot[warp] = s;
    __syncthreads();
    if (warp == 0) {
      long long w = warp_tot[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        long long t = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += t;
      }
      warp_tot[lane] = w;   // inclusive totals of the warps
    }
    __syncthreads();
    const long long before = carry + (warp > 0 ? warp_tot[warp - 1] : 0) + (s - v);
    if (k < n) row_start[k] = (int)(before < 2147483647LL ? before : 2147483647LL);
    __syncthreads();
    if (threadIdx.x == 0) carry += warp_tot[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    *count_out = carry;
    *overflow_out = carry > capacity ? 1 : 0;
  }
}

// slots past the last pair carry the padding index n (jax-md convention)
__global__ void pad_list_kernel(int n, const long long* __restrict__ count, long long capacity, int* __restrict__ idx) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= capacity) return;
  if (e >= *count) { idx[e] = n; idx[capacity + e] = n; }
}

std::mutex g_setup_mutex;
int* g_scratch_addr[kMaxDevices] = {};   // device address of kRowScratch, per device ordinal

// In host code `kRowScratch` is only a handle for the runtime, not a device address: the address the kernels need is
// looked up once per device, with that device current.
int scratch_for_current_device(int** out) {
  int dev = -1;
  SO3LR_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return kInvalidArgument;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[dev]) {
    int* p = nullptr;
    SO3LR_CUDA_CHECK(cudaGetSymbolAddress((void**)&p, kRowScratch));
    if (!p) return kCudaError;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return kOk;
}

}  // namespace

extern "C" SO3LR_B200_API int so3lr_b200_neighbor_list_noalloc(void* stream, int n_atoms, const float* positions_dev, const float* cell,
                                                               float r_cutoff, int ordered, int32_t* idx_dev, int64_t capacity,
                                                               int64_t* count_dev, int* overflow_dev) {
  if (!positions_dev || !idx_dev || !count_dev || !overflow_dev || n_atoms <= 0 || capacity <= 0 || !(r_cutoff > 0.f))
    return kInvalidArgument;
  if (n_atoms > kMaxAtoms) {
    std::fprintf(stderr, "so3lr_b200_neighbor_list_noalloc: %d atoms exceed the fixed scratch of %d atoms; use "
                 "so3lr_b200_system_export_list for larger systems\n", n_atoms, kMaxAtoms);
    return kTooLarge;
  }
  Cell c;
  std::memset(&c, 0, sizeof(c));
  if (cell) {
    double h[9], inv[9];
    for (int k = 0; k < 9; ++k) h[k] = cell[k];
    const double det = h[0] * (h[4] * h[8] - h[5] * h[7]) - h[1] * (h[3] * h[8] - h[5] * h[6]) + h[2] * (h[3] * h[7] - h[4] * h[6]);
    if (!(std::fabs(det) > 1e-12) || !std::isfinite(det)) return kInvalidArgument;
    inv[0] = (h[4] * h[8] - h[5] * h[7]) / det; inv[1] = (h[2] * h[7] - h[1] * h[8]) / det; inv[2] = (h[1] * h[5] - h[2] * h[4]) / det;
    inv[3] = (h[5] * h[6] - h[3] * h[8]) / det; inv[4] = (h[0] * h[8] - h[2] * h[6]) / det; inv[5] = (h[2] * h[3] - h[0] * h[5]) / det;
    inv[6] = (h[3] * h[7] - h[4] * h[6]) / det; inv[7] = (h[1] * h[6] - h[0] * h[7]) / det; inv[8] = (h[0] * h[4] - h[1] * h[3]) / det;
    for (int k = 0; k < 9; ++k) { c.h[k] = (float)h[k]; c.hinv[k] = (float)inv[k]; }
    c.periodic = 1;
    // every pair is tested at its nearest image only: that is the full list as long as no second image can fall inside the
    // cutoff, i.e. each perpendicular width of the cell (1 / |column k of the inverse|) is at least twice the cutoff
    for (int k = 0; k < 3; ++k) {
      const double width = 1.0 / std::sqrt(inv[k] * inv[k] + inv[3 + k] * inv[3 + k] + inv[6 + k] * inv[6 + k]);
      if (width < 2.0 * (double)r_cutoff) {
        std::fprintf(stderr, "so3lr_b200_neighbor_list_noalloc: perpendicular cell width %.4f A is below twice the cutoff %.4f A\n",
                     width, (double)r_cutoff);
        return kInvalidArgument;
      }
    }
  }
  int* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  int* row_count = scratch;
  int* row_start = scratch + (kMaxAtoms + 1);
  cudaStream_t st = (cudaStream_t)stream;
  const int blocks = (n_atoms + 7) / 8;
  const float r2 = r_cutoff * r_cutoff;
  long long* count_ll = reinterpret_cast<long long*>(count_dev);
  rows_all_pairs_kernel<false><<<blocks, 256, 0, st>>>(c, n_atoms, positions_dev, r2, ordered, row_count, nullptr, nullptr, 0);
  scan_rows_kernel<<<1, 1024, 0, st>>>(n_atoms, row_count, row_start, (long long)capacity, count_ll, overflow_dev);
  rows_all_pairs_kernel<true><<<blocks, 256, 0, st>>>(c, n_atoms, positions_dev, r2, ordered, nullptr, row_start, idx_dev, (long long)capacity);
  pad_list_kernel<<<(unsigned)((capacity + 255) / 256), 256, 0, st>>>(n_atoms, count_ll, (long long)capacity, idx_dev);
  count_launch(4);
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// Cell-list neighbor lists on the GPU (replaces jax_md.partition.neighbor_list for the 4.5 A and 12 A graphs).
//
// Atoms are binned into cells no smaller than the list radius, sorted by cell with a stable radix sort (so the
// row contents are deterministic), and one warp per atom scans the 27 (or fewer) surrounding cells with a
// ballot-compaction into its row.  Two passes (count, fill) with an exclusive scan in between give exact rows.
// Distances use the minimum-image convention with the float32 operation order of common.cuh::min_image and
// d2 = (dx*dx + dy*dy) + dz*dz < r*r, evaluated without fused multiply-adds.
#include "kernels.h"

#include <cub/cub.cuh>

namespace so3lr {

struct NlistWorkspace {
  int* cell_of = nullptr;      // n
  int* cell_sorted = nullptr;  // n
  int* atom_sorted = nullptr;  // n   atom indices ordered by cell
  int* atom_iota = nullptr;    // n
  int* cell_start = nullptr;   // ncell_total + 1
  float4* pos_sorted = nullptr; // n: positions in cell order, w = atom index (bit pattern)
  int* row_count = nullptr;    // n + 1
  void* cub_tmp = nullptr;
  size_t cub_bytes = 0;
  long long* d_total = nullptr;
  long long* h_total = nullptr;  // pinned
  int n_cap = 0, cell_cap = 0;
  // spatial ordering of the atoms (Morton keys of the short-range cells)
  unsigned* key = nullptr;
  unsigned* key_sorted = nullptr;
  void* sort_tmp = nullptr;
  size_t sort_bytes = 0;
  int key_cap = 0;
};

NlistWorkspace* nlist_workspace_create() { return new NlistWorkspace(); }
void nlist_workspace_destroy(NlistWorkspace* w) {
  if (!w) return;
  cudaFree(w->cell_of); cudaFree(w->cell_sorted); cudaFree(w->atom_sorted); cudaFree(w->atom_iota);
  cudaFree(w->cell_start); cudaFree(w->row_count); cudaFree(w->cub_tmp); cudaFree(w->d_total);
  cudaFree(w->key); cudaFree(w->key_sorted); cudaFree(w->sort_tmp); cudaFree(w->pos_sorted);
  if (w->h_total) cudaFreeHost(w->h_total);
  delete w;
}

namespace {

struct Grid {
  int nc[3];        // cells per dimension
  int wrap[3];      // periodic wrap in that dimension
  float lo[3];      // free space: lower corner
  float inv_w[3];   // free space: 1 / cell width
};

__device__ __forceinline__ void cell_coords(const Cell& cell, const Grid& G, float x, float y, float z, int* c) {
  if (cell.periodic) {
    float s0 = x * cell.hinv[0] + y * cell.hinv[3] + z * cell.hinv[6];
    float s1 = x * cell.hinv[1] + y * cell.hinv[4] + z * cell.hinv[7];
    float s2 = x * cell.hinv[2] + y * cell.hinv[5] + z * cell.hinv[8];
    s0 -= floorf(s0); s1 -= floorf(s1); s2 -= floorf(s2);
    c[0] = min((int)(s0 * G.nc[0]), G.nc[0] - 1);
    c[1] = min((int)(s1 * G.nc[1]), G.nc[1] - 1);
    c[2] = min((int)(s2 * G.nc[2]), G.nc[2] - 1);
  } else {
    c[0] = min(max((int)((x - G.lo[0]) * G.inv_w[0]), 0), G.nc[0] - 1);
    c[1] = min(max((int)((y - G.lo[1]) * G.inv_w[1]), 0), G.nc[1] - 1);
    c[2] = min(max((int)((z - G.lo[2]) * G.inv_w[2]), 0), G.nc[2] - 1);
  }
}

__global__ void assign_cells_kernel(Cell cell, Grid G, int n, const float* __restrict__ R, int* __restrict__ cell_of,
                                    int* __restrict__ iota) {
  int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= n) return;
  int c[3];
  cell_coords(cell, G, R[3 * (size_t)a], R[3 * (size_t)a + 1], R[3 * (size_t)a + 2], c);
  cell_of[a] = (c[2] * G.nc[1] + c[1]) * G.nc[0] + c[0];
  iota[a] = a;
}

__global__ void cell_bounds_kernel(int n, int n_cells, const int* __restrict__ cell_sorted, int* __restrict__ cell_start) {
  int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k > n) return;
  int cur = k < n ? cell_sorted[k] : n_cells;
  int prev = k > 0 ? cell_sorted[k - 1] : -1;
  for (int c = prev + 1; c <= cur; ++c) cell_start[c] = k;
}

// positions in cell order (one coalesced 16-byte load per candidate in the row kernels)
__global__ void gather_sorted_positions_kernel(int n, const float* __restrict__ R, const int* __restrict__ atom_sorted,
                                               float4* __restrict__ pos_sorted) {
  int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const int a = atom_sorted[k];
  pos_sorted[k] = make_float4(R[3 * (size_t)a], R[3 * (size_t)a + 1], R[3 * (size_t)a + 2], __int_as_float(a));
}

// FILL = false: row_count[i] = number of neighbours.  FILL = true: write rows at row_ptr[i].
template <bool FILL>
__global__ void __launch_bounds__(256) build_rows_kernel(Cell cell, Grid G, int n, const float* __restrict__ R, float r2max,
                                                         int ordered, const int* __restrict__ seg,
                                                         const float4* __restrict__ pos_sorted, const int* __restrict__ cell_start,
                                                         int* __restrict__ row_count, const int* __restrict__ row_ptr,
                                                         int* __restrict__ nbr_j, int* __restrict__ edge_i, long long capacity) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= n) return;
  const float xi = R[3 * (size_t)i], yi = R[3 * (size_t)i + 1], zi = R[3 * (size_t)i + 2];
  const int segi = seg ? seg[i] : 0;
  int ci[3];
  cell_coords(cell, G, xi, yi, zi, ci);
  long long base = FILL ? row_ptr[i] : 0;
  int count = 0;
  const int lo0 = G.nc[0] > 1 ? -1 : 0, hi0 = G.nc[0] > 1 ? 1 : 0;
  const int lo1 = G.nc[1] > 1 ? -1 : 0, hi1 = G.nc[1] > 1 ? 1 : 0;
  const int lo2 = G.nc[2] > 1 ? -1 : 0, hi2 = G.nc[2] > 1 ? 1 : 0;
  for (int d2 = lo2; d2 <= hi2; ++d2) {
    int c2 = ci[2] + d2;
    if (G.wrap[2]) c2 = (c2 + G.nc[2]) % G.nc[2]; else if (c2 < 0 || c2 >= G.nc[2]) continue;
    for (int d1 = lo1; d1 <= hi1; ++d1) {
      int c1 = ci[1] + d1;
      if (G.wrap[1]) c1 = (c1 + G.nc[1]) % G.nc[1]; else if (c1 < 0 || c1 >= G.nc[1]) continue;
      for (int d0 = lo0; d0 <= hi0; ++d0) {
        int c0 = ci[0] + d0;
        if (G.wrap[0]) c0 = (c0 + G.nc[0]) % G.nc[0]; else if (c0 < 0 || c0 >= G.nc[0]) continue;
        const int c = (c2 * G.nc[1] + c1) * G.nc[0] + c0;
        const int s0 = cell_start[c], s1 = cell_start[c + 1];
        for (int k0 = s0; k0 < s1; k0 += 32) {
          const int k = k0 + lane;
          bool hit = false;
          int j = -1;
          if (k < s1) {
            const float4 pj = pos_sorted[k];
            j = __float_as_int(pj.w);
            float dx = pj.x - xi, dy = pj.y - yi, dz = pj.z - zi;
            min_image(cell, dx, dy, dz);
            const float dd = dist2_rn(dx, dy, dz);
            hit = dd < r2max && (ordered ? j > i : j != i) && (!seg || seg[j] == segi);
          }
          const unsigned m = __ballot_sync(0xffffffffu, hit);
          if (FILL && hit) {
            long long pos = base + count + __popc(m & ((1u << lane) - 1u));
            if (pos < capacity) { nbr_j[pos] = j; edge_i[pos] = i; }
          }
          count += __popc(m);
        }
      }
    }
  }
  if (!FILL && lane == 0) row_count[i] = count;
}

// batched free-space graphs: the candidates of atom i are the atoms of its own graph
template <bool FILL>
__global__ void __launch_bounds__(256) build_rows_graph_kernel(int n, const float* __restrict__ R, float r2max, int ordered,
                                                               const int* __restrict__ seg, const int* __restrict__ graph_start,
                                                               int* __restrict__ row_count, const int* __restrict__ row_ptr,
                                                               int* __restrict__ nbr_j, int* __restrict__ edge_i, long long capacity) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= n) return;
  const float xi = R[3 * (size_t)i], yi = R[3 * (size_t)i + 1], zi = R[3 * (size_t)i + 2];
  const int g = seg[i];
  const int s0 = graph_start[g], s1 = graph_start[g + 1];
  long long base = FILL ? row_ptr[i] : 0;
  int count = 0;
  for (int k0 = s0; k0 < s1; k0 += 32) {
    const int j = k0 + lane;
    bool hit = false;
    if (j < s1) {
      float dx = R[3 * (size_t)j] - xi, dy = R[3 * (size_t)j + 1] - yi, dz = R[3 * (size_t)j + 2] - zi;
      hit = dist2_rn(dx, dy, dz) < r2max && (ordered ? j > i : j != i);
    }
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (FILL && hit) {
      long long pos = base + count + __popc(m & ((1u << lane) - 1u));
      if (pos < capacity) { nbr_j[pos] = j; edge_i[pos] = i; }
    }
    count += __popc(m);
  }
  if (!FILL && lane == 0) row_count[i] = count;
}

// 64-bit sum of the per-row counts.  The exclusive scan that follows runs in 32 bits (CSR offsets are int): this total, not
// the scan's last element, decides whether the list fits, so a sum beyond 2^31 is seen before any offset is used.
__global__ void __launch_bounds__(256) row_total_kernel(int n, const int* __restrict__ row_count, unsigned long long* __restrict__ total) {
  __shared__ unsigned long long red[8];
  unsigned long long v = 0;
  for (int k = blockIdx.x * 256 + threadIdx.x; k < n; k += gridDim.x * 256) v += (unsigned long long)(unsigned)row_count[k];
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long t = 0;
    for (int w = 0; w < 8; ++w) t += red[w];
    if (t) atomicAdd(total, t);
  }
}

__global__ void finish_scan_kernel(int n, int* __restrict__ row_ptr, const long long* __restrict__ total, long long capacity, int* overflow) {
  // row_ptr[0..n-1] hold the exclusive scan already; close it with the 64-bit total (clamped: a total beyond the int range
  // is rejected on the host before any row is filled)
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const long long t = *total;
    row_ptr[n] = t > 2147483647LL ? 2147483647 : (int)t;
    if (overflow && t > capacity) *overflow = 1;
  }
}

__global__ void clamp_rows_kernel(int n, int* __restrict__ row_ptr, long long capacity) {
  int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k <= n && (long long)row_ptr[k] > capacity) row_ptr[k] = (int)capacity;
}

__device__ __forceinline__ unsigned spread3(unsigned v) {   // 10 bits -> every third bit
  v &= 0x3ffu;
  v = (v | (v << 16)) & 0x030000ffu;
  v = (v | (v << 8)) & 0x0300f00fu;
  v = (v | (v << 4)) & 0x030c30c3u;
  v = (v | (v << 2)) & 0x09249249u;
  return v;
}
__global__ void morton_keys_kernel(Cell cell, Grid G, int n, const float* __restrict__ R, unsigned* __restrict__ key,
                                   int* __restrict__ iota) {
  int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= n) return;
  int c[3];
  cell_coords(cell, G, R[3 * (size_t)a], R[3 * (size_t)a + 1], R[3 * (size_t)a + 2], c);
  key[a] = spread3((unsigned)c[0]) | (spread3((unsigned)c[1]) << 1) | (spread3((unsigned)c[2]) << 2);
  iota[a] = a;
}

template <typename T>
int ensure(T** p, size_t n) {
  if (*p) cudaFree(*p);
  *p = nullptr;
  SO3LR_CUDA_CHECK(cudaMalloc((void**)p, n * sizeof(T)));
  return kOk;
}

}  // namespace

int nlist_row_total(cudaStream_t s, int n, const int* row_count_dev, long long* total_host) {
  unsigned long long* d = nullptr;
  SO3LR_CUDA_CHECK(cudaMalloc((void**)&d, sizeof(unsigned long long)));
  SO3LR_CUDA_CHECK(cudaMemsetAsync(d, 0, sizeof(unsigned long long), s));
  int tb = (n + 255) / 256;
  if (tb > 1024) tb = 1024;
  if (n > 0) { row_total_kernel<<<tb, 256, 0, s>>>(n, row_count_dev, d); count_launch(); }
  unsigned long long t = 0;
  cudaError_t e = cudaMemcpyAsync(&t, d, sizeof(t), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  cudaFree(d);
  if (e != cudaSuccess) return kCudaError;
  *total_host = (long long)t;
  return t > 2147483000ULL ? kTooLarge : kOk;
}

int spatial_order(NlistWorkspace* w, cudaStream_t s, const Cell& cell, int n, const float* R, float cell_size, int* perm) {
  if (n <= 0 || !cell.periodic) return kInvalidArgument;
  if (n > w->key_cap) {
    int st;
    if ((st = ensure(&w->key, n))) return st;
    if ((st = ensure(&w->key_sorted, n))) return st;
    w->key_cap = n;
  }
  if (n > w->n_cap) {
    int st;
    if ((st = ensure(&w->cell_of, n))) return st;
    if ((st = ensure(&w->cell_sorted, n))) return st;
    if ((st = ensure(&w->atom_sorted, n))) return st;
    if ((st = ensure(&w->atom_iota, n))) return st;
    if ((st = ensure(&w->row_count, (size_t)n + 1))) return st;
    if ((st = ensure(&w->pos_sorted, (size_t)n))) return st;
    w->n_cap = n;
  }
  Grid G{};
  for (int k = 0; k < 3; ++k) {
    double nx = cell.hinv[0 + k], ny = cell.hinv[3 + k], nz = cell.hinv[6 + k];
    double width = 1.0 / std::sqrt(nx * nx + ny * ny + nz * nz);
    int nc = (int)std::floor(width / (double)cell_size);
    if (nc < 1) nc = 1;
    if (nc > 1024) nc = 1024;
    G.nc[k] = nc; G.wrap[k] = 1;
  }
  { morton_keys_kernel<<<(n + 255) / 256, 256, 0, s>>>(cell, G, n, R, w->key, w->atom_iota); count_launch(); }
  size_t need = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, need, w->key, w->key_sorted, w->atom_iota, perm, n, 0, 30, s);
  if (need > w->sort_bytes) {
    if (w->sort_tmp) cudaFree(w->sort_tmp);
    w->sort_tmp = nullptr;
    SO3LR_CUDA_CHECK(cudaMalloc(&w->sort_tmp, need));
    w->sort_bytes = need;
  }
  size_t tmp = w->sort_bytes;
  cub::DeviceRadixSort::SortPairs(w->sort_tmp, tmp, w->key, w->key_sorted, w->atom_iota, perm, n, 0, 30, s);
  count_launch(6);   // histogram, prefix, four 8-bit passes
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

int nlist_build(NlistWorkspace* w, cudaStream_t s, const Cell& cell, int n, const float* R, float r_list, int ordered,
                const int* seg, const int* graph_start, NeighborListDev* out, int allow_grow, int* d_overflow, int n_rows) {
  if (n <= 0) { out->count = 0; return kOk; }
  if (n_rows < 0 || n_rows > n) n_rows = n;
  if (n > w->n_cap) {
    int st;
    if ((st = ensure(&w->cell_of, n))) return st;
    if ((st = ensure(&w->cell_sorted, n))) return st;
    if ((st = ensure(&w->atom_sorted, n))) return st;
    if ((st = ensure(&w->atom_iota, n))) return st;
    if ((st = ensure(&w->row_count, (size_t)n + 1))) return st;
    if ((st = ensure(&w->pos_sorted, (size_t)n))) return st;
    w->n_cap = n;
  }
  if (!w->d_total) {
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&w->d_total, sizeof(long long)));
    SO3LR_CUDA_CHECK(cudaMallocHost((void**)&w->h_total, sizeof(long long)));
  }
  if (n + 1 > out->row_cap) {
    if (out->row_ptr) cudaFree(out->row_ptr);
    out->row_ptr = nullptr;
    SO3LR_CUDA_CHECK(cudaMalloc((void**)&out->row_ptr, ((size_t)n + 1) * sizeof(int)));
    out->row_cap = n + 1;
  }
  const float r2max = r_list * r_list;
  const bool by_graph = graph_start != nullptr && !cell.periodic;
  Grid G{};
  int n_cells = 1;
  if (!by_graph) {
    if (cell.periodic) {
      // perpendicular widths of the cell: 1 / |column k of hinv|
      for (int k = 0; k < 3; ++k) {
        double nx = cell.hinv[0 + k], ny = cell.hinv[3 + k], nz = cell.hinv[6 + k];
        double width = 1.0 / std::sqrt(nx * nx + ny * ny + nz * nz);
        int nc = (int)std::floor(width / (double)r_list);
        if (nc < 3) nc = 1;          // fewer than 3 cells: one cell, minimum-image handles the rest
        if (nc > 1024) nc = 1024;
        G.nc[k] = nc; G.wrap[k] = 1;
      }
    } else {
      // bounding box on the host side would need a reduction; use a coarse device-free approach: the caller
      // passes free-space systems of moderate size, so read the positions back once per build.
      std::vector<float> h((size_t)n * 3);
      SO3LR_CUDA_CHECK(cudaMemcpyAsync(h.data(), R, h.size() * sizeof(float), cudaMemcpyDeviceToHost, s));
      SO3LR_CUDA_CHECK(cudaStreamSynchronize(s));
      float lo[3] = {1e30f, 1e30f, 1e30f}, hi[3] = {-1e30f, -1e30f, -1e30f};
      for (int a = 0; a < n; ++a)
        for (int k = 0; k < 3; ++k) { float v = h[3 * (size_t)a + k]; lo[k] = v < lo[k] ? v : lo[k]; hi[k] = v > hi[k] ? v : hi[k]; }
      for (int k = 0; k < 3; ++k) {
        float ext = hi[k] - lo[k];
        if (!(ext >= 0.f) || !std::isfinite(ext)) return kNotFinite;
        int nc = (int)std::floor(ext / r_list);
        if (nc < 1) nc = 1;
        if (nc > 512) nc = 512;
        G.nc[k] = nc; G.wrap[k] = 0; G.lo[k] = lo[k];
        G.inv_w[k] = nc / (ext > 0.f ? ext * 1.000001f : 1.f);
      }
    }
    n_cells = G.nc[0] * G.nc[1] * G.nc[2];
    if (n_cells + 1 > w->cell_cap) {
      int st;
      if ((st = ensure(&w->cell_start, (size_t)n_cells + 1))) return st;
      w->cell_cap = n_cells + 1;
    }
    { assign_cells_kernel<<<(n + 255) / 256, 256, 0, s>>>(cell, G, n, R, w->cell_of, w->atom_iota); count_launch(); }
    int bits = 1;
    while ((1 << bits) < n_cells && bits < 31) ++bits;
    size_t need = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, need, w->cell_of, w->cell_sorted, w->atom_iota, w->atom_sorted, n, 0, bits, s);
    size_t need2 = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, need2, w->row_count, out->row_ptr, n, s);   // sized for the largest row count
    if (need2 > need) need = need2;
    if (need > w->cub_bytes) {
      if (w->cub_tmp) cudaFree(w->cub_tmp);
      SO3LR_CUDA_CHECK(cudaMalloc(&w->cub_tmp, need));
      w->cub_bytes = need;
    }
    size_t tmp = w->cub_bytes;
    cub::DeviceRadixSort::SortPairs(w->cub_tmp, tmp, w->cell_of, w->cell_sorted, w->atom_iota, w->atom_sorted, n, 0, bits, s);
    count_launch(2 + (bits + 7) / 8);
    { cell_bounds_kernel<<<(n + 1 + 255) / 256, 256, 0, s>>>(n, n_cells, w->cell_sorted, w->cell_start); count_launch(); }
    { gather_sorted_positions_kernel<<<(n + 255) / 256, 256, 0, s>>>(n, R, w->atom_sorted, w->pos_sorted); count_launch(); }
  } else {
    size_t need = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, need, w->row_count, out->row_ptr, n, s);
    if (need > w->cub_bytes) {
      if (w->cub_tmp) cudaFree(w->cub_tmp);
      SO3LR_CUDA_CHECK(cudaMalloc(&w->cub_tmp, need));
      w->cub_bytes = need;
    }
  }
  const int blocks = (n_rows + 7) / 8;
  if (n_rows == 0) { out->count = 0; return kOk; }
  if (by_graph)
    { build_rows_graph_kernel<false><<<blocks, 256, 0, s>>>(n_rows, R, r2max, ordered, seg, graph_start, w->row_count, nullptr, nullptr, nullptr, 0); count_launch(); }
  else
    { build_rows_kernel<false><<<blocks, 256, 0, s>>>(cell, G, n_rows, R, r2max, ordered, seg, w->pos_sorted, w->cell_start,
                                                    w->row_count, nullptr, nullptr, nullptr, 0); count_launch(); }
  SO3LR_CUDA_CHECK(cudaMemsetAsync(w->d_total, 0, sizeof(long long), s));
  { int tb = (n_rows + 255) / 256; if (tb > 1024) tb = 1024;
    row_total_kernel<<<tb, 256, 0, s>>>(n_rows, w->row_count, reinterpret_cast<unsigned long long*>(w->d_total)); count_launch(); }
  size_t tmp = w->cub_bytes;
  cub::DeviceScan::ExclusiveSum(w->cub_tmp, tmp, w->row_count, out->row_ptr, n_rows, s);
  count_launch(2);
  { finish_scan_kernel<<<1, 32, 0, s>>>(n_rows, out->row_ptr, w->d_total, out->capacity, allow_grow ? nullptr : d_overflow); count_launch(); }
  SO3LR_CUDA_CHECK(cudaMemcpyAsync(w->h_total, w->d_total, sizeof(long long), cudaMemcpyDeviceToHost, s));
  SO3LR_CUDA_CHECK(cudaStreamSynchronize(s));
  const long long total = *w->h_total;
  if (total > 2147483000LL) return kTooLarge;
  if (total > out->capacity) {
    if (!allow_grow) {
      out->count = out->capacity;   // rows are truncated; the overflow flag is set on the device
    } else {
      long long cap = total + total / 4 + 1024;
      if (out->nbr_j) cudaFree(out->nbr_j);
      if (out->edge_i) cudaFree(out->edge_i);
      out->nbr_j = nullptr; out->edge_i = nullptr;
      SO3LR_CUDA_CHECK(cudaMalloc((void**)&out->nbr_j, (size_t)cap * sizeof(int)));
      SO3LR_CUDA_CHECK(cudaMalloc((void**)&out->edge_i, (size_t)cap * sizeof(int)));
      out->capacity = cap;
    }
  }
  if (total <= out->capacity) out->count = total;
  const bool truncated = total > out->capacity;
  if (by_graph)
    { build_rows_graph_kernel<true><<<blocks, 256, 0, s>>>(n_rows, R, r2max, ordered, seg, graph_start, nullptr, out->row_ptr,
                                                         out->nbr_j, out->edge_i, out->capacity); count_launch(); }
  else
    { build_rows_kernel<true><<<blocks, 256, 0, s>>>(cell, G, n_rows, R, r2max, ordered, seg, w->pos_sorted, w->cell_start, nullptr,
                                                   out->row_ptr, out->nbr_j, out->edge_i, out->capacity); count_launch(); }
  if (truncated) { clamp_rows_kernel<<<(n_rows + 1 + 255) / 256, 256, 0, s>>>(n_rows, out->row_ptr, out->capacity); count_launch(); }
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return truncated ? kOverflow : kOk;
}

}  // namespace so3lr

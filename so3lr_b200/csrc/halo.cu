// Halo packing for the exchanges between ranks of a decomposed run: the rows that travel to (arrive from) one neighbour are
// gathered from (scattered into) all per-atom arrays of the exchange by one launch.
#include <algorithm>
#include <cstdint>

#include "kernels.h"

namespace so3lr {

namespace {

struct RowPack {
  float* a[4];
  int w[4], off[5], n;
};
template <bool UNPACK>
__global__ void __launch_bounds__(256) pack_rows_kernel(RowPack P, long long n_rows, const long long* __restrict__ idx, float* buf) {
  const int W = P.off[P.n];
  const long long total = n_rows * W;
  for (long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (long long)gridDim.x * blockDim.x) {
    const long long r = id / W;
    const int c = (int)(id - r * W);
    int t = 0;
    while (t + 1 < P.n && c >= P.off[t + 1]) ++t;
    float* p = P.a[t] + (size_t)idx[r] * P.w[t] + (c - P.off[t]);
    if (UNPACK) *p = buf[id];
    else buf[id] = *p;
  }
}
}  // namespace

int pack_rows(void* stream, int n_arrays, float* const* arrays, const int* widths, const int64_t* idx, int64_t n_rows, float* buf, bool unpack) {
  if (n_arrays < 1 || n_arrays > 4 || !arrays || !widths || n_rows < 0) return kInvalidArgument;
  if (n_rows == 0) return kOk;
  if (!idx || !buf) return kInvalidArgument;
  RowPack P{};
  P.n = n_arrays;
  for (int t = 0; t < n_arrays; ++t) {
    if (!arrays[t] || widths[t] <= 0) return kInvalidArgument;
    P.a[t] = arrays[t]; P.w[t] = widths[t]; P.off[t + 1] = P.off[t] + widths[t];
  }
  const long long total = (long long)n_rows * P.off[n_arrays];
  const unsigned blocks = (unsigned)std::min<long long>((total + 255) / 256, (long long)sm_count() * 16);
  cudaStream_t st = (cudaStream_t)stream;
  if (unpack) pack_rows_kernel<true><<<blocks, 256, 0, st>>>(P, n_rows, reinterpret_cast<const long long*>(idx), buf);
  else pack_rows_kernel<false><<<blocks, 256, 0, st>>>(P, n_rows, reinterpret_cast<const long long*>(idx), buf);
  count_launch();
  SO3LR_CUDA_CHECK(cudaGetLastError());
  return kOk;
}


}  // namespace so3lr

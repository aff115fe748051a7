// Host-side preparation of the SO3LR weights: radial-filter tables, transposed kernels, ZBL constants.
#include "model.h"

#include <cuda_fp16.h>

#include <cmath>
#include <cstring>
#include <vector>

namespace so3lr {

namespace {

double softplus_d(double x) { return x > 30 ? x : std::log1p(std::exp(x)); }
double silu_d(double x) { return x / (1.0 + std::exp(-x)); }
double dsilu_d(double x) {
  double s = 1.0 / (1.0 + std::exp(-x));
  return s * (1.0 + x * (1.0 - s));
}

// the reference keeps the Bernstein decay constant as a float32 number
const double kGamma = (double)(float)0.9448630629184640;

// 32 exponential Bernstein polynomials and d/dr at distance r
void bernstein(double r, double* b, double* db) {
  const int n = kNumRbf - 1;
  double x = std::exp(-kGamma * r);
  double dx = -kGamma * x;
  double one = 1.0 - x;
  double logc = 0.0;  // log C(n,k)
  for (int k = 0; k <= n; ++k) {
    if (k > 0) logc += std::log((double)(n - k + 1)) - std::log((double)k);
    double c = std::exp(logc);
    double xk = std::pow(x, k), ok = std::pow(one, n - k);
    b[k] = c * xk * ok;
    double t1 = k > 0 ? k * std::pow(x, k - 1) * ok : 0.0;
    double t2 = (n - k) > 0 ? (n - k) * xk * std::pow(one, n - k - 1) : 0.0;
    db[k] = c * (t1 - t2) * dx;
  }
}

// w(r) and dw/dr of both radial filters of one layer, including the constant part of the spherical filter
void radial_filters(const float* blob, const BlobOffsets& O, int layer, double r, double* w, double* dw) {
  const LayerOffsets& L = O.layer[layer];
  double b[kNumRbf], db[kNumRbf];
  bernstein(r, b, db);
  for (int f = 0; f < 2; ++f) {
    const float* k1 = blob + L.rad_l1_k[f];
    const float* b1 = blob + L.rad_l1_b[f];
    const float* k2 = blob + L.rad_l2_k[f];
    const float* b2 = blob + L.rad_l2_b[f];
    double h[kF], dh[kF];
    for (int j = 0; j < kF; ++j) {
      double z = b1[j], dz = 0.0;
      for (int k = 0; k < kNumRbf; ++k) { z += b[k] * k1[k * kF + j]; dz += db[k] * k1[k * kF + j]; }
      h[j] = silu_d(z);
      dh[j] = dsilu_d(z) * dz;
    }
    const float* sb2 = blob + L.sph_l2_b[f];
    for (int j = 0; j < kF; ++j) {
      double a = (double)b2[j] + (double)sb2[j], da = 0.0;
      for (int k = 0; k < kF; ++k) { a += h[k] * k2[k * kF + j]; da += dh[k] * k2[k * kF + j]; }
      w[f * kF + j] = a;
      dw[f * kF + j] = da;
    }
    if (layer == 0) {
      // ev = 0 in the first layer: spherical filter = Dense2(silu(bias1)) (its bias2 is already added above)
      const float* sb1 = blob + L.sph_l1_b[f];
      const float* sk2 = blob + L.sph_l2_k[f];
      for (int j = 0; j < kF; ++j) {
        double a = 0.0;
        for (int c = 0; c < 32; ++c) a += silu_d(sb1[c]) * sk2[c * kF + j];
        w[f * kF + j] += a;
      }
    }
  }
}

// FP16 pair (x, y) and the pair of their residuals scaled by 2048, as the device code splits its operands
void split2_host(float x, float y, unsigned& hi, unsigned& lo) {
  const __half hx = __float2half_rn(x), hy = __float2half_rn(y);
  const __half lx = __float2half_rn((x - __half2float(hx)) * 2048.f), ly = __float2half_rn((y - __half2float(hy)) * 2048.f);
  auto bits = [](__half h) { unsigned short u; std::memcpy(&u, &h, 2); return (unsigned)u; };
  hi = bits(hx) | (bits(hy) << 16);
  lo = bits(lx) | (bits(ly) << 16);
}
// B[k][n] (K x N, row-major; transpose = read W as [N][K]) -> fragment order of mma.m16n8k16 (.col B operand)
std::vector<float> pack_fragments(const float* W, int K, int N, bool transpose) {
  std::vector<float> out((size_t)(K / 16) * (N / 8) * 32 * 4);
  auto B = [&](int k, int n) { return transpose ? W[(size_t)n * K + k] : W[(size_t)k * N + n]; };
  for (int ks = 0; ks < K / 16; ++ks)
    for (int nt = 0; nt < N / 8; ++nt)
      for (int lane = 0; lane < 32; ++lane) {
        const int g = lane >> 2, q = lane & 3, n = 8 * nt + g, k0 = 16 * ks + 2 * q;
        unsigned v[4];
        split2_host(B(k0, n), B(k0 + 1, n), v[0], v[2]);
        split2_host(B(k0 + 8, n), B(k0 + 9, n), v[1], v[3]);
        std::memcpy(&out[(((size_t)ks * (N / 8) + nt) * 32 + lane) * 4], v, 16);
      }
  return out;
}

// B[k][n] (K x N; transpose = read W as [N][K]) -> operand image of the tcgen05 dense-block kernels: hi matrix, then lo matrix,
// each with K contiguous in 8 x 8 core matrices: element (k, n) at (k/8) * 16 N + (n/8) * 128 + (n%8) * 16 + (k%8) * 2 bytes
void umma_image_append(std::vector<unsigned char>& out, const float* W, int K, int N, bool transpose) {
  const size_t half = (size_t)K * N * 2, base = out.size();
  out.resize(base + 2 * half);
  for (int k = 0; k < K; ++k)
    for (int n = 0; n < N; ++n) {
      const float v = transpose ? W[(size_t)n * K + k] : W[(size_t)k * N + n];
      unsigned short hi, lo;
      const __half h = __float2half_rn(v);
      const __half l = __float2half_rn((v - __half2float(h)) * 2048.f);
      std::memcpy(&hi, &h, 2);
      std::memcpy(&lo, &l, 2);
      const size_t off = (size_t)(k / 8) * 16 * N + (size_t)(n / 8) * 128 + (n % 8) * 16 + (k % 8) * 2;
      std::memcpy(&out[base + off], &hi, 2);
      std::memcpy(&out[base + half + off], &lo, 2);
    }
}

// Chebyshev coefficients coef[m][c] (m < kChebM, c < 256) of both radial filters of a layer in the variable
// t = A x + B, x = exp(-hg r), sampled at 256 Chebyshev-Gauss nodes (A, B, hg are the float32 constants the kernels use)
void chebyshev_coefficients(const float* blob, const BlobOffsets& O, int layer, std::vector<double>& coef) {
  const int N = 256;
  const double A = (double)kChebA, B = (double)kChebB, hg = (double)kChebHalfGamma;
  std::vector<double> w((size_t)N * 256), dw(256);
  for (int k = 0; k < N; ++k) {
    const double t = std::cos(M_PI * (k + 0.5) / N);
    const double x = (t - B) / A;
    const double r = -std::log(x) / hg;
    radial_filters(blob, O, layer, r, &w[(size_t)k * 256], dw.data());
  }
  coef.assign((size_t)kChebM * 256, 0.0);
  for (int m = 0; m < kChebM; ++m)
    for (int k = 0; k < N; ++k) {
      const double c = std::cos(M_PI * m * (k + 0.5) / N) * (m == 0 ? 1.0 : 2.0) / N;
      for (int j = 0; j < 256; ++j) coef[(size_t)m * 256 + j] += c * w[(size_t)k * 256 + j];
    }
}

// FP16 hi and 2048-scaled lo of x (the split every tensor-core operand of the library uses)
void split_half(float x, unsigned short& hi, unsigned short& lo) {
  const __half h = __float2half_rn(x);
  const __half l = __float2half_rn((x - __half2float(h)) * 2048.f);
  std::memcpy(&hi, &h, 2);
  std::memcpy(&lo, &l, 2);
}

// term held by column / row k of the Chebyshev block: even terms first, then the odd ones (the order in which the kernels
// generate the polynomials)
int cheb_term(int k) { return k < kChebM / 2 ? 2 * k : 2 * (k - kChebM / 2) + 1; }

// Forward-kernel image: B operands with K contiguous.  CT[n][k] = coefficient of term cheb_term(k) of feature n: core
// (n/8, k/8) at (k/8) * 4096 + (n/8) * 128; K2T_f[n][h]: core (n/8, h/8) at (h/8) * 2048 + (n/8) * 128.
// Layout: CT hi | CT lo (32 KB each) | K2T hi f = 0, 1 | K2T lo f = 0, 1 (8 KB each).
std::vector<float> tc_image_forward(const float* blob, const BlobOffsets& O, int layer) {
  std::vector<unsigned char> img(kTcImageBytes, 0);
  std::vector<double> coef;
  chebyshev_coefficients(blob, O, layer, coef);
  auto put = [&](size_t base_hi, size_t base_lo, size_t off, float v) {
    unsigned short hi, lo;
    split_half(v, hi, lo);
    std::memcpy(&img[base_hi + off], &hi, 2);
    std::memcpy(&img[base_lo + off], &lo, 2);
  };
  for (int k = 0; k < kChebM; ++k)
    for (int n = 0; n < 256; ++n)
      put(0, 32768, (size_t)(k / 8) * 4096 + (size_t)(n / 8) * 128 + (n % 8) * 16 + (k % 8) * 2, (float)coef[(size_t)cheb_term(k) * 256 + n]);
  const LayerOffsets& L = O.layer[layer];
  for (int f = 0; f < 2; ++f) {
    const float* K2 = blob + L.sph_l2_k[f];
    for (int h = 0; h < 32; ++h)
      for (int n = 0; n < kF; ++n)
        put(65536 + (size_t)f * 8192, 65536 + 16384 + (size_t)f * 8192, (size_t)(h / 8) * 2048 + (size_t)(n / 8) * 128 + (n % 8) * 16 + (h % 8) * 2,
            K2[h * kF + n]);
  }
  std::vector<float> out(kTcImageBytes / 4);
  std::memcpy(out.data(), img.data(), kTcImageBytes);
  return out;
}

// Operand image of the reverse attention kernel (attention_tc.cu): 8 x 8 core matrices (8 rows of 16 bytes).  Per filter f the 96
// rows [64 Chebyshev terms in the order of cheb_term | 32 hidden units of the spherical filter] by the filter's 128 features;
// core (row / 8, feature / 8) at (feature / 8) * 1536 + (row / 8) * 128.  Layout: hi f = 0 | hi f = 1 | lo f = 0 | lo f = 1.
std::vector<float> tc_image(const float* blob, const BlobOffsets& O, int layer) {
  std::vector<unsigned char> img(kTcImageBytes, 0);
  std::vector<double> coef;
  chebyshev_coefficients(blob, O, layer, coef);
  const size_t per_filter = 16 * 1536;
  static_assert(4 * 16 * 1536 == kTcImageBytes, "image size");
  const LayerOffsets& L = O.layer[layer];
  for (int f = 0; f < 2; ++f) {
    const float* K2 = blob + L.sph_l2_k[f];
    for (int row = 0; row < 96; ++row)
      for (int n = 0; n < kF; ++n) {
        const float v = row < kChebM ? (float)coef[(size_t)cheb_term(row) * 256 + f * kF + n] : K2[(row - kChebM) * kF + n];
        unsigned short hi, lo;
        split_half(v, hi, lo);
        const size_t off = (size_t)(n / 8) * 1536 + (size_t)(row / 8) * 128 + (row % 8) * 16 + (n % 8) * 2;
        std::memcpy(&img[f * per_filter + off], &hi, 2);
        std::memcpy(&img[(2 + f) * per_filter + off], &lo, 2);
      }
  }
  std::vector<float> out(kTcImageBytes / 4);
  std::memcpy(out.data(), img.data(), kTcImageBytes);
  return out;
}

struct Uploader {
  std::vector<void*>* owned;
  int status = kOk;
  const float* up(const std::vector<float>& v) {
    void* d = nullptr;
    if (cudaMalloc(&d, v.size() * sizeof(float)) != cudaSuccess) { status = kCudaError; return nullptr; }
    if (cudaMemcpy(d, v.data(), v.size() * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) { status = kCudaError; }
    owned->push_back(d);
    return (const float*)d;
  }
  const float* up(const float* p, size_t n) { return up(std::vector<float>(p, p + n)); }
  const unsigned char* up_bytes(const std::vector<unsigned char>& v) {   // cudaMalloc alignment (256 B) satisfies bulk copies
    void* d = nullptr;
    if (cudaMalloc(&d, v.size()) != cudaSuccess) { status = kCudaError; return nullptr; }
    if (cudaMemcpy(d, v.data(), v.size(), cudaMemcpyHostToDevice) != cudaSuccess) { status = kCudaError; }
    owned->push_back(d);
    return (const unsigned char*)d;
  }
  const float* upT(const float* p, int rows, int cols) {  // [rows][cols] -> [cols][rows]
    std::vector<float> t((size_t)rows * cols);
    for (int r = 0; r < rows; ++r)
      for (int c = 0; c < cols; ++c) t[(size_t)c * rows + r] = p[(size_t)r * cols + c];
    return up(t);
  }
};

}  // namespace

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] <= 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

void radial_filter_chebyshev(const float* blob, int layer, double r, double* w256, double* dw256) {
  BlobOffsets O = blob_offsets();
  std::vector<double> coef;
  chebyshev_coefficients(blob, O, layer, coef);
  const double x = std::exp(-(double)kChebHalfGamma * r), t = (double)kChebA * x + (double)kChebB;
  const double dtdr = -(double)kChebA * (double)kChebHalfGamma * x;
  std::vector<double> T(kChebM), dT(kChebM);   // dT_m/dt = m U_{m-1}
  double Um1 = 0.0, U0 = 1.0;                  // U_{-1}, U_0
  T[0] = 1.0; T[1] = t; dT[0] = 0.0; dT[1] = 1.0;
  for (int m = 2; m < kChebM; ++m) {
    T[m] = 2.0 * t * T[m - 1] - T[m - 2];
    const double U1 = 2.0 * t * U0 - Um1;      // U_{m-1}
    Um1 = U0; U0 = U1;
    dT[m] = m * U0;
  }
  for (int c = 0; c < 256; ++c) {
    double a = 0.0, b = 0.0;
    for (int m = 0; m < kChebM; ++m) { a += coef[(size_t)m * 256 + c] * T[m]; b += coef[(size_t)m * 256 + c] * dT[m]; }
    w256[c] = a; dw256[c] = b * dtdr;
  }
}

void radial_filter_reference(const float* blob, int layer, double r, double* w256, double* dw256) {
  BlobOffsets O = blob_offsets();
  radial_filters(blob, O, layer, r, w256, dw256);
}

int build_model(const float* blob, size_t n_floats, ModelDev* M, std::vector<void*>* owned) {
  BlobOffsets O = blob_offsets();
  if (n_floats != O.total) {
    std::fprintf(stderr, "so3lr_b200: parameter blob has %zu floats, expected %zu\n", n_floats, O.total);
    return kInvalidArgument;
  }
  Uploader U{owned};
  {
    std::vector<float> e(blob + O.embed_z, blob + O.embed_z + kZEmbed * kF);
    const float s = (float)(1.0 / std::sqrt(3.0));
    for (auto& v : e) v *= s;
    M->embed_z = U.up(e);
  }
  for (int e = 0; e < 2; ++e) {
    M->cs_embed_q[e] = U.up(blob + O.cs[e].embed_q, kZEmbed * kF);
    M->cs_embed_k[e] = U.up(blob + O.cs[e].embed_k, 2 * kF);
    M->cs_embed_v[e] = U.up(blob + O.cs[e].embed_v, 2 * kF);
    M->cs_res0[e] = U.up(blob + O.cs[e].res0, kF * kF);
    M->cs_res1[e] = U.up(blob + O.cs[e].res1, kF * kF);
  }
  for (int l = 0; l < kNumLayers; ++l) {
    const LayerOffsets& L = O.layer[l];
    LayerDev& D = M->layer[l];
    D.has_spherical = l > 0;
    // projections
    std::vector<float> P(5 * 4 * 32 * 32), PT(5 * 4 * 32 * 32);
    for (int w = 0; w < 5; ++w) {
      const float* W = blob + L.W[w];
      for (int h = 0; h < 4; ++h)
        for (int i = 0; i < 32; ++i)
          for (int j = 0; j < 32; ++j) {
            float v = W[(h * 32 + i) * 32 + j];
            P[((w * 4 + h) * 32 + i) * 32 + j] = v;
            PT[((w * 4 + h) * 32 + j) * 32 + i] = v;
          }
    }
    D.proj = U.up(P);
    D.projT = U.up(PT);
    {
      std::vector<float> pf, pb;
      for (int w = 0; w < 5; ++w)
        for (int h = 0; h < 4; ++h) {
          const float* W = blob + L.W[w] + (size_t)h * 32 * 32;    // [i][j]
          std::vector<float> a = pack_fragments(W, 32, 32, true);   // B[k = j][n = i] = W[i][j]
          std::vector<float> b = pack_fragments(W, 32, 32, false);  // B[k = i][n = j] = W[i][j]
          pf.insert(pf.end(), a.begin(), a.end());
          pb.insert(pb.end(), b.begin(), b.end());
        }
      D.proj_f = reinterpret_cast<const uint4*>(U.up(pf));
      D.projT_f = reinterpret_cast<const uint4*>(U.up(pb));
      // tcgen05 images: forward per head B[k = j][n = 32 w + i] = W[w][h][i][j]; reverse per (w, h) B[k = i][n = j]
      // forward: blocks of 16 KB in the order head 0 | head 1 | head 2 | k2 of all heads | head 3 (the kernel loads the first four
      // with one copy and the last one into the place of head 0 once that has been used).  Head block: [K = 32][N = 128 = the
      // first four projections side by side]; k2 block: per head [K = 32][N = 32], 4 KB each
      std::vector<unsigned char> uf, ub;
      std::vector<float> blk(32 * 128);
      auto head_block = [&](int h) {
        for (int w = 0; w < 4; ++w) {
          const float* W = blob + L.W[w] + (size_t)h * 32 * 32;
          for (int i = 0; i < 32; ++i)
            for (int j = 0; j < 32; ++j) blk[(size_t)j * 128 + 32 * w + i] = W[i * 32 + j];
        }
        umma_image_append(uf, blk.data(), 32, 128, false);
      };
      head_block(0); head_block(1); head_block(2);
      for (int h = 0; h < 4; ++h) umma_image_append(uf, blob + L.W[4] + (size_t)h * 32 * 32, 32, 32, true);   // B[k = j][n = i] = W[i][j]
      head_block(3);
      for (int w = 0; w < 5; ++w)
        for (int h = 0; h < 4; ++h) umma_image_append(ub, blob + L.W[w] + (size_t)h * 32 * 32, 32, 32, false);
      D.proj_u = U.up_bytes(uf);
      D.projT_u = U.up_bytes(ub);
    }
    // radial tables
    // per interval g (between knots g and g+1) four rows of 256: value at g, slope at g (x spacing), value difference
    // to knot g+1 (formed in double precision: the derivative of the interpolant is built from this difference, and a
    // difference of two rounded values would lose 1/spacing in accuracy), slope at g+1 (x spacing)
    std::vector<float> tab((size_t)(kTableGrid - 1) * 4 * 256);
    std::vector<double> w(256), dw(256), w1(256), dw1(256);
    radial_filters(blob, O, l, 0.0, w.data(), dw.data());
    for (int g = 0; g + 1 < kTableGrid; ++g) {
      double r1 = (double)(g + 1) * (double)kTableH;
      radial_filters(blob, O, l, r1, w1.data(), dw1.data());
      for (int j = 0; j < 256; ++j) {
        tab[((size_t)g * 4 + 0) * 256 + j] = (float)w[j];
        tab[((size_t)g * 4 + 1) * 256 + j] = (float)(dw[j] * (double)kTableH);
        tab[((size_t)g * 4 + 2) * 256 + j] = (float)(w1[j] - w[j]);
        tab[((size_t)g * 4 + 3) * 256 + j] = (float)(dw1[j] * (double)kTableH);
      }
      w.swap(w1); dw.swap(dw1);
    }
    D.table = U.up(tab);
    D.tc_img = reinterpret_cast<const unsigned char*>(U.up(tc_image(blob, O, l)));
    D.tc_img_fwd = reinterpret_cast<const unsigned char*>(U.up(tc_image_forward(blob, O, l)));
    std::vector<float> s1k(2 * 4 * 32), s1b(2 * 32), s2k(2 * 32 * 128);
    for (int f = 0; f < 2; ++f) {
      std::memcpy(&s1k[f * 128], blob + L.sph_l1_k[f], 128 * sizeof(float));
      std::memcpy(&s1b[f * 32], blob + L.sph_l1_b[f], 32 * sizeof(float));
      std::memcpy(&s2k[f * 4096], blob + L.sph_l2_k[f], 4096 * sizeof(float));
    }
    D.sph1_k = U.up(s1k); D.sph1_b = U.up(s1b); D.sph2_k = U.up(s2k);
    D.ln1_s = U.up(blob + L.ln1_s, kF); D.ln1_b = U.up(blob + L.ln1_b, kF);
    D.ln2_s = U.up(blob + L.ln2_s, kF); D.ln2_b = U.up(blob + L.ln2_b, kF);
    D.res1_k = U.up(blob + L.res1_k, kF * kF); D.res1_kT = U.upT(blob + L.res1_k, kF, kF); D.res1_b = U.up(blob + L.res1_b, kF);
    D.res2_k = U.up(blob + L.res2_k, kF * kF); D.res2_kT = U.upT(blob + L.res2_k, kF, kF); D.res2_b = U.up(blob + L.res2_b, kF);
    const float* E = blob + L.exch_k;  // [132 in][132 out]
    std::vector<float> xx(128 * 128), xg(128 * 4), ix(4 * 128), ig(16);
    for (int i = 0; i < 132; ++i)
      for (int o = 0; o < 132; ++o) {
        float v = E[i * 132 + o];
        if (i < 128 && o < 128) xx[i * 128 + o] = v;
        else if (i < 128) xg[i * 4 + (o - 128)] = v;
        else if (o < 128) ix[(i - 128) * 128 + o] = v;
        else ig[(i - 128) * 4 + (o - 128)] = v;
      }
    D.ex_xx = U.up(xx); D.ex_xxT = U.upT(xx.data(), 128, 128);
    auto frag = [&](const float* W, int K, int N, bool tr) { return reinterpret_cast<const uint4*>(U.up(pack_fragments(W, K, N, tr))); };
    D.res1_f = frag(blob + L.res1_k, kF, kF, false); D.res1T_f = frag(blob + L.res1_k, kF, kF, true);
    D.res2_f = frag(blob + L.res2_k, kF, kF, false); D.res2T_f = frag(blob + L.res2_k, kF, kF, true);
    D.exxx_f = frag(xx.data(), kF, kF, false); D.exxxT_f = frag(xx.data(), kF, kF, true);
    auto uimg = [&](const float* W, int K, int N, bool tr) { std::vector<unsigned char> b; umma_image_append(b, W, K, N, tr); return U.up_bytes(b); };
    D.res1_u = uimg(blob + L.res1_k, kF, kF, false); D.res1T_u = uimg(blob + L.res1_k, kF, kF, true);
    D.res2_u = uimg(blob + L.res2_k, kF, kF, false); D.res2T_u = uimg(blob + L.res2_k, kF, kF, true);
    D.exxx_u = uimg(xx.data(), kF, kF, false); D.exxxT_u = uimg(xx.data(), kF, kF, true);
    D.ex_xg = U.up(xg); D.ex_ix = U.up(ix); D.ex_ig = U.up(ig);
    D.ex_bx = U.up(blob + L.exch_b, 128); D.ex_bg = U.up(blob + L.exch_b + 128, 4);
  }
  M->e_reg_k = U.up(blob + O.e_reg_k, kF * kF); M->e_reg_kT = U.upT(blob + O.e_reg_k, kF, kF);
  M->e_reg_b = U.up(blob + O.e_reg_b, kF); M->e_fin_k = U.up(blob + O.e_fin_k, kF);
  M->e_fin_b = blob[O.e_fin_b];
  M->e_scale = U.up(blob + O.e_scale, kZEmbed); M->e_offset = U.up(blob + O.e_offset, kZEmbed);
  M->q_embed = U.up(blob + O.q_embed, kZHead);
  M->q_reg_k = U.up(blob + O.q_reg_k, kF * kF); M->q_reg_kT = U.upT(blob + O.q_reg_k, kF, kF);
  M->q_reg_b = U.up(blob + O.q_reg_b, kF); M->q_fin_k = U.up(blob + O.q_fin_k, kF);
  M->q_fin_b = blob[O.q_fin_b];
  M->h_embed0 = U.up(blob + O.h_embed0, kZHead); M->h_embed1 = U.up(blob + O.h_embed1, kZHead * 64);
  M->h_reg_k = U.up(blob + O.h_reg_k, kF * 64); M->h_reg_kT = U.upT(blob + O.h_reg_k, kF, 64);
  M->h_reg_b = U.up(blob + O.h_reg_b, 64);
  M->h_fin_k = U.up(blob + O.h_fin_k, 64 * 64); M->h_fin_kT = U.upT(blob + O.h_fin_k, 64, 64);
  M->h_fin_b = U.up(blob + O.h_fin_b, 64);
  {
    auto frag = [&](const float* W, int K, int N, bool tr) { return reinterpret_cast<const uint4*>(U.up(pack_fragments(W, K, N, tr))); };
    // transposed kernels: B[k][n] = W[n][k] with W stored [N_in = n][K_out = k]
    M->e_reg_f = frag(blob + O.e_reg_k, kF, kF, false); M->e_regT_f = frag(blob + O.e_reg_k, kF, kF, true);
    M->q_reg_f = frag(blob + O.q_reg_k, kF, kF, false); M->q_regT_f = frag(blob + O.q_reg_k, kF, kF, true);
    M->h_reg_f = frag(blob + O.h_reg_k, kF, 64, false); M->h_regT_f = frag(blob + O.h_reg_k, 64, kF, true);
    M->h_fin_f = frag(blob + O.h_fin_k, 64, 64, false); M->h_finT_f = frag(blob + O.h_fin_k, 64, 64, true);
    auto uimg = [&](const float* W, int K, int N, bool tr) { std::vector<unsigned char> b; umma_image_append(b, W, K, N, tr); return U.up_bytes(b); };
    M->e_reg_u = uimg(blob + O.e_reg_k, kF, kF, false); M->e_regT_u = uimg(blob + O.e_reg_k, kF, kF, true);
    M->q_reg_u = uimg(blob + O.q_reg_k, kF, kF, false); M->q_regT_u = uimg(blob + O.q_reg_k, kF, kF, true);
    M->h_reg_u = uimg(blob + O.h_reg_k, kF, 64, false); M->h_regT_u = uimg(blob + O.h_reg_k, 64, kF, true);
    M->h_fin_u = uimg(blob + O.h_fin_k, 64, 64, false); M->h_finT_u = uimg(blob + O.h_fin_k, 64, 64, true);
  }
  // ZBL constants: softplus of the raw parameters, weights normalised to one
  double a[4], c[4], cs = 0.0;
  for (int k = 0; k < 4; ++k) { a[k] = softplus_d(blob[O.zbl[k]]); c[k] = softplus_d(blob[O.zbl[4 + k]]); cs += c[k]; }
  for (int k = 0; k < 4; ++k) { M->zbl.a[k] = (float)a[k]; M->zbl.c[k] = (float)(c[k] / cs); }
  M->zbl.p = (float)softplus_d(blob[O.zbl[8]]);
  M->zbl.d = (float)softplus_d(blob[O.zbl[9]]);
  return U.status;
}

}  // namespace so3lr

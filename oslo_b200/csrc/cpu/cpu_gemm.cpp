// Host-side GEMMs for CPU inference: fp32 (C = alpha A B + beta C) and quantised uint8 x int8 -> int32 with an optional
// per-column compensation term (the "shifted activation" trick: activations are stored as u8 = s8 + 128, and
// 128 * column-sum(B) is subtracted again through `compensation`).
//
// Row-major operands, optional transposition of either one, OpenMP over row blocks of C, AVX-512 / AVX2 inner loops chosen
// at run time by function multiversioning (one binary for hosts with and without AVX-512), scalar fallback.  B is packed
// once per call into a k-major panel so the inner loop streams it with unit stride.
//
// Replaces the MKL wrappers of the reference's LightSeq subset (oslo/lightseq2/csrc/kernels/x86/gemm.cpp:10-50:
// cblas_sgemm and cblas_gemm_s8u8s32).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <immintrin.h>
#include <vector>

namespace {

constexpr int kRowBlock = 32;

// ------------------------------------------------------------------------------------------------ fp32 row update
// c[0..n) += a * b[0..n)
__attribute__((target("avx512f"))) void axpy_avx512(float* c, const float* b, float a, int n) {
  const __m512 va = _mm512_set1_ps(a);
  int j = 0;
  for (; j + 16 <= n; j += 16) _mm512_storeu_ps(c + j, _mm512_fmadd_ps(va, _mm512_loadu_ps(b + j), _mm512_loadu_ps(c + j)));
  for (; j < n; ++j) c[j] += a * b[j];
}
__attribute__((target("avx2,fma"))) void axpy_avx2(float* c, const float* b, float a, int n) {
  const __m256 va = _mm256_set1_ps(a);
  int j = 0;
  for (; j + 8 <= n; j += 8) _mm256_storeu_ps(c + j, _mm256_fmadd_ps(va, _mm256_loadu_ps(b + j), _mm256_loadu_ps(c + j)));
  for (; j < n; ++j) c[j] += a * b[j];
}
void axpy_scalar(float* c, const float* b, float a, int n) {
  for (int j = 0; j < n; ++j) c[j] += a * b[j];
}

// c[0..n) (int32) += a * b[0..n) (int8), a in [0, 255]
__attribute__((target("avx512f,avx512bw"))) void axpy_i8_avx512(int32_t* c, const int8_t* b, int32_t a, int n) {
  const __m512i va = _mm512_set1_epi32(a);
  int j = 0;
  for (; j + 16 <= n; j += 16) {
    const __m512i vb = _mm512_cvtepi8_epi32(_mm_loadu_si128(reinterpret_cast<const __m128i*>(b + j)));
    __m512i vc = _mm512_loadu_si512(reinterpret_cast<const void*>(c + j));
    vc = _mm512_add_epi32(vc, _mm512_mullo_epi32(va, vb));
    _mm512_storeu_si512(reinterpret_cast<void*>(c + j), vc);
  }
  for (; j < n; ++j) c[j] += a * b[j];
}
__attribute__((target("avx2"))) void axpy_i8_avx2(int32_t* c, const int8_t* b, int32_t a, int n) {
  const __m256i va = _mm256_set1_epi32(a);
  int j = 0;
  for (; j + 8 <= n; j += 8) {
    const __m256i vb = _mm256_cvtepi8_epi32(_mm_loadl_epi64(reinterpret_cast<const __m128i*>(b + j)));
    __m256i vc = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(c + j));
    vc = _mm256_add_epi32(vc, _mm256_mullo_epi32(va, vb));
    _mm256_storeu_si256(reinterpret_cast<__m256i*>(c + j), vc);
  }
  for (; j < n; ++j) c[j] += a * b[j];
}
void axpy_i8_scalar(int32_t* c, const int8_t* b, int32_t a, int n) {
  for (int j = 0; j < n; ++j) c[j] += a * b[j];
}

int simd_level() {
  static const int level = [] {
    __builtin_cpu_init();
    if (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw")) return 2;
    if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) return 1;
    return 0;
  }();
  return level;
}

template <typename T>
void pack_b(const T* b, long long ldb, bool transpose_b, long long k, long long n, std::vector<T>& panel) {
  // panel[kk * n + j] = B(kk, j) of the logical (k x n) matrix
  panel.resize(static_cast<size_t>(k) * n);
  if (!transpose_b) {
    for (long long kk = 0; kk < k; ++kk) std::memcpy(&panel[kk * n], b + kk * ldb, sizeof(T) * n);
  } else {
#pragma omp parallel for schedule(static)
    for (long long kk = 0; kk < k; ++kk)
      for (long long j = 0; j < n; ++j) panel[kk * n + j] = b[j * ldb + kk];
  }
}

}  // namespace

// C[m, n] = alpha * op(A)[m, k] * op(B)[k, n] + beta * C, row-major, fp32.
extern "C" int oslo_cpu_sgemm(int transpose_a, int transpose_b, long long m, long long n, long long k, float alpha, const float* a,
                              long long lda, const float* b, long long ldb, float beta, float* c, long long ldc) {
  if (m < 0 || n < 0 || k < 0 || !c || (k > 0 && (!a || !b))) return -1;
  std::vector<float> panel;
  const float* bp = b;
  long long ldp = ldb;
  if (transpose_b && k > 0) {
    pack_b(b, ldb, true, k, n, panel);
    bp = panel.data();
    ldp = n;
  }
  const int level = simd_level();
#pragma omp parallel for schedule(static)
  for (long long i0 = 0; i0 < m; i0 += kRowBlock) {
    const long long i1 = std::min(m, i0 + kRowBlock);
    for (long long i = i0; i < i1; ++i) {
      float* ci = c + i * ldc;
      if (beta == 0.f) std::memset(ci, 0, sizeof(float) * n);
      else if (beta != 1.f) for (long long j = 0; j < n; ++j) ci[j] *= beta;
    }
    for (long long kk = 0; kk < k; ++kk) {
      const float* brow = bp + kk * ldp;
      for (long long i = i0; i < i1; ++i) {
        const float av = alpha * (transpose_a ? a[kk * lda + i] : a[i * lda + kk]);
        float* ci = c + i * ldc;
        if (level == 2) axpy_avx512(ci, brow, av, static_cast<int>(n));
        else if (level == 1) axpy_avx2(ci, brow, av, static_cast<int>(n));
        else axpy_scalar(ci, brow, av, static_cast<int>(n));
      }
    }
  }
  return 0;
}

// C[m, n] (int32) = alpha * op(A)[m, k] (uint8) * op(B)[k, n] (int8) + beta * C + compensation[n] (may be null), row-major.
extern "C" int oslo_cpu_gemm_u8s8s32(int transpose_a, int transpose_b, long long m, long long n, long long k, float alpha,
                                     const uint8_t* a, long long lda, const int8_t* b, long long ldb, float beta, int32_t* c,
                                     long long ldc, const int32_t* compensation) {
  if (m < 0 || n < 0 || k < 0 || !c || (k > 0 && (!a || !b))) return -1;
  std::vector<int8_t> panel;
  const int8_t* bp = b;
  long long ldp = ldb;
  if (transpose_b && k > 0) {
    pack_b(b, ldb, true, k, n, panel);
    bp = panel.data();
    ldp = n;
  }
  const int level = simd_level();
#pragma omp parallel for schedule(static)
  for (long long i0 = 0; i0 < m; i0 += kRowBlock) {
    const long long i1 = std::min(m, i0 + kRowBlock);
    std::vector<int32_t> acc(static_cast<size_t>(n));
    for (long long i = i0; i < i1; ++i) {
      std::fill(acc.begin(), acc.end(), 0);
      for (long long kk = 0; kk < k; ++kk) {
        const int32_t av = transpose_a ? a[kk * lda + i] : a[i * lda + kk];
        if (av == 0) continue;
        const int8_t* brow = bp + kk * ldp;
        if (level == 2) axpy_i8_avx512(acc.data(), brow, av, static_cast<int>(n));
        else if (level == 1) axpy_i8_avx2(acc.data(), brow, av, static_cast<int>(n));
        else axpy_i8_scalar(acc.data(), brow, av, static_cast<int>(n));
      }
      int32_t* ci = c + i * ldc;
      for (long long j = 0; j < n; ++j) {
        float v = alpha * static_cast<float>(acc[j]);
        if (beta != 0.f) v += beta * static_cast<float>(ci[j]);
        ci[j] = static_cast<int32_t>(v < 0 ? v - 0.5f : v + 0.5f) + (compensation ? compensation[j] : 0);
      }
    }
  }
  return 0;
}

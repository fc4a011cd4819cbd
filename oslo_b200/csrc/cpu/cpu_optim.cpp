// Host-side optimizers for parameters / optimizer state kept in CPU memory (ZeRO CPU offload):
// Adam / AdamW and Adagrad over flat fp32 arrays, OpenMP over 64 Ki-element tiles, AVX-512 or AVX2 bodies chosen at
// run time (function multiversioning, so one binary runs on hosts with or without AVX-512), scalar tail.
// Optionally writes a bf16 / fp16 copy of the updated parameters into a (pinned) staging buffer in the same
// pass, which the caller then ships to the GPU with one async copy of half the bytes.
//
// Replaces oslo/torch/_C/csrc/CPUAdamBinder.cpp:19-212, includes/cpu_adam.h:20-204, CPUAdagradBinder.cpp and
// includes/simd.h of the reference (DeepSpeed-derived).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <immintrin.h>

namespace {

constexpr long long kTile = 1 << 16;

inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // NaN
  u += 0x7fffu + ((u >> 16) & 1u);  // round to nearest even
  return static_cast<uint16_t>(u >> 16);
}

inline uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = static_cast<int32_t>((x >> 23) & 0xff) - 127 + 15;
  uint32_t mant = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (mant ? 0x200u : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    mant |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t half = mant >> shift;
    const uint32_t rem = mant & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
  }
  uint32_t half = (static_cast<uint32_t>(exp) << 10) | (mant >> 13);
  const uint32_t rem = mant & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return static_cast<uint16_t>(sign | half);
}

inline void store_lowp(uint16_t* dst, int kind, long long i, float v) {
  if (dst) dst[i] = kind == 2 ? f32_to_bf16(v) : f32_to_f16(v);
}

struct AdamArgs {
  float lr, b1, b2, eps, wd, inv_bc1, inv_sqrt_bc2, grad_scale;
  int adamw;
};

inline void adam_scalar(float* p, const float* g, float* m, float* v, long long lo, long long hi, const AdamArgs& a,
                        uint16_t* lowp, int kind) {
  for (long long i = lo; i < hi; ++i) {
    float gv = g[i] * a.grad_scale;
    float pv = p[i];
    if (!a.adamw) gv += a.wd * pv;
    const float mv = a.b1 * m[i] + (1.f - a.b1) * gv;
    const float vv = a.b2 * v[i] + (1.f - a.b2) * gv * gv;
    m[i] = mv;
    v[i] = vv;
    float upd = (mv * a.inv_bc1) / (std::sqrt(vv) * a.inv_sqrt_bc2 + a.eps);
    if (a.adamw) upd += a.wd * pv;
    pv -= a.lr * upd;
    p[i] = pv;
    store_lowp(lowp, kind, i, pv);
  }
}

__attribute__((target("avx512f"))) void adam_avx512(float* p, const float* g, float* m, float* v, long long lo, long long hi,
                                                    const AdamArgs& a, uint16_t* lowp, int kind) {
  const __m512 b1 = _mm512_set1_ps(a.b1), omb1 = _mm512_set1_ps(1.f - a.b1), b2 = _mm512_set1_ps(a.b2),
               omb2 = _mm512_set1_ps(1.f - a.b2), eps = _mm512_set1_ps(a.eps), wd = _mm512_set1_ps(a.wd),
               ibc1 = _mm512_set1_ps(a.inv_bc1), isbc2 = _mm512_set1_ps(a.inv_sqrt_bc2), lr = _mm512_set1_ps(a.lr),
               gs = _mm512_set1_ps(a.grad_scale);
  long long i = lo;
  for (; i + 16 <= hi; i += 16) {
    __m512 gv = _mm512_mul_ps(_mm512_loadu_ps(g + i), gs);
    __m512 pv = _mm512_loadu_ps(p + i);
    if (!a.adamw) gv = _mm512_fmadd_ps(wd, pv, gv);
    const __m512 mv = _mm512_fmadd_ps(b1, _mm512_loadu_ps(m + i), _mm512_mul_ps(omb1, gv));
    const __m512 vv = _mm512_fmadd_ps(b2, _mm512_loadu_ps(v + i), _mm512_mul_ps(omb2, _mm512_mul_ps(gv, gv)));
    _mm512_storeu_ps(m + i, mv);
    _mm512_storeu_ps(v + i, vv);
    const __m512 denom = _mm512_fmadd_ps(_mm512_sqrt_ps(vv), isbc2, eps);
    __m512 upd = _mm512_div_ps(_mm512_mul_ps(mv, ibc1), denom);
    if (a.adamw) upd = _mm512_fmadd_ps(wd, pv, upd);
    pv = _mm512_fnmadd_ps(lr, upd, pv);
    _mm512_storeu_ps(p + i, pv);
    if (lowp) {
      alignas(64) float tmp[16];
      _mm512_store_ps(tmp, pv);
      for (int k = 0; k < 16; ++k) store_lowp(lowp, kind, i + k, tmp[k]);
    }
  }
  adam_scalar(p, g, m, v, i, hi, a, lowp, kind);
}

__attribute__((target("avx2,fma"))) void adam_avx2(float* p, const float* g, float* m, float* v, long long lo, long long hi,
                                                   const AdamArgs& a, uint16_t* lowp, int kind) {
  const __m256 b1 = _mm256_set1_ps(a.b1), omb1 = _mm256_set1_ps(1.f - a.b1), b2 = _mm256_set1_ps(a.b2),
               omb2 = _mm256_set1_ps(1.f - a.b2), eps = _mm256_set1_ps(a.eps), wd = _mm256_set1_ps(a.wd),
               ibc1 = _mm256_set1_ps(a.inv_bc1), isbc2 = _mm256_set1_ps(a.inv_sqrt_bc2), lr = _mm256_set1_ps(a.lr),
               gs = _mm256_set1_ps(a.grad_scale);
  long long i = lo;
  for (; i + 8 <= hi; i += 8) {
    __m256 gv = _mm256_mul_ps(_mm256_loadu_ps(g + i), gs);
    __m256 pv = _mm256_loadu_ps(p + i);
    if (!a.adamw) gv = _mm256_fmadd_ps(wd, pv, gv);
    const __m256 mv = _mm256_fmadd_ps(b1, _mm256_loadu_ps(m + i), _mm256_mul_ps(omb1, gv));
    const __m256 vv = _mm256_fmadd_ps(b2, _mm256_loadu_ps(v + i), _mm256_mul_ps(omb2, _mm256_mul_ps(gv, gv)));
    _mm256_storeu_ps(m + i, mv);
    _mm256_storeu_ps(v + i, vv);
    const __m256 denom = _mm256_fmadd_ps(_mm256_sqrt_ps(vv), isbc2, eps);
    __m256 upd = _mm256_div_ps(_mm256_mul_ps(mv, ibc1), denom);
    if (a.adamw) upd = _mm256_fmadd_ps(wd, pv, upd);
    pv = _mm256_fnmadd_ps(lr, upd, pv);
    _mm256_storeu_ps(p + i, pv);
    if (lowp) {
      alignas(32) float tmp[8];
      _mm256_store_ps(tmp, pv);
      for (int k = 0; k < 8; ++k) store_lowp(lowp, kind, i + k, tmp[k]);
    }
  }
  adam_scalar(p, g, m, v, i, hi, a, lowp, kind);
}

int simd_level() {
  static int level = -1;
  if (level < 0) {
    __builtin_cpu_init();
    level = __builtin_cpu_supports("avx512f") ? 2 : ((__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) ? 1 : 0);
  }
  return level;
}

}  // namespace

extern "C" int oslo_cpu_simd_level() { return simd_level(); }

// p, m, v: fp32 [n] (updated in place); g: fp32 [n].  lowp (optional): 16-bit copy of the new parameters,
// lowp_kind 1 = fp16, 2 = bf16.  bc1 / bc2: bias corrections 1 - beta^t (pass 1 to disable).
extern "C" void oslo_cpu_adam_step(float* p, const float* g, float* m, float* v, long long n, float lr, float beta1, float beta2,
                                   float eps, float weight_decay, float bc1, float bc2, float grad_scale, int adamw,
                                   uint16_t* lowp, int lowp_kind) {
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.f / bc1, 1.f / std::sqrt(bc2), grad_scale, adamw};
  const int level = simd_level();
  const long long tiles = (n + kTile - 1) / kTile;
#pragma omp parallel for schedule(static)
  for (long long t = 0; t < tiles; ++t) {
    const long long lo = t * kTile, hi = lo + kTile < n ? lo + kTile : n;
    if (level == 2) adam_avx512(p, g, m, v, lo, hi, a, lowp, lowp_kind);
    else if (level == 1) adam_avx2(p, g, m, v, lo, hi, a, lowp, lowp_kind);
    else adam_scalar(p, g, m, v, lo, hi, a, lowp, lowp_kind);
  }
}

// Adagrad: h += g^2 ; p -= lr * (g / (sqrt(h) + eps) [+ wd * p]).
extern "C" void oslo_cpu_adagrad_step(float* p, const float* g, float* h, long long n, float lr, float eps, float weight_decay,
                                      uint16_t* lowp, int lowp_kind) {
  const long long tiles = (n + kTile - 1) / kTile;
#pragma omp parallel for schedule(static)
  for (long long t = 0; t < tiles; ++t) {
    const long long lo = t * kTile, hi = lo + kTile < n ? lo + kTile : n;
#pragma omp simd
    for (long long i = lo; i < hi; ++i) {
      const float gv = g[i] + weight_decay * p[i];
      const float hv = h[i] + gv * gv;
      h[i] = hv;
      p[i] -= lr * gv / (std::sqrt(hv) + eps);
    }
    if (lowp)
      for (long long i = lo; i < hi; ++i) store_lowp(lowp, lowp_kind, i, p[i]);
  }
}

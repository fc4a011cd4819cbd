// LayerNorm / RMSNorm forward and backward for sm_100a (bf16 / fp16 / fp32).
//
// One CTA normalises one row at a time (grid-stride over rows).  Each thread keeps
// its 16-byte vectors of the row in registers, so x is read from HBM exactly once
// in forward and (x, dy) once in backward.  Statistics are fp32; the variance is
// computed around the mean from registers (two block reductions, no E[x^2]-E[x]^2
// cancellation).  Backward fuses dx with the per-CTA partial sums of dgamma/dbeta;
// a second small kernel folds the partials.
//
// Replaces apex-derived oslo/torch/_C/csrc/fused_layer_norm.cu:49-855 and lightseq2
// csrc/kernels/cuda/normalize_kernels.cu.
#include "common.cuh"

namespace oslo {

template <typename T> struct Vec8;  // 8 elements of T, 16 bytes for 2-byte types
template <> struct Vec8<__nv_bfloat16> {
  uint4 raw;
  OSLO_DEVINL void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  OSLO_DEVINL void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  OSLO_DEVINL void to_float(float* f) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f[2 * j] = __uint_as_float(w[j] << 16);
      f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
  OSLO_DEVINL void from_float(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    raw = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Vec8<__half> {
  uint4 raw;
  OSLO_DEVINL void load(const __half* p) { raw = *reinterpret_cast<const uint4*>(p); }
  OSLO_DEVINL void store(__half* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  OSLO_DEVINL void to_float(float* f) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
      f[2 * j] = __low2float(h);
      f[2 * j + 1] = __high2float(h);
    }
  }
  OSLO_DEVINL void from_float(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    raw = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Vec8<float> {
  float4 a, b;
  OSLO_DEVINL void load(const float* p) {
    a = *reinterpret_cast<const float4*>(p);
    b = *reinterpret_cast<const float4*>(p + 4);
  }
  OSLO_DEVINL void store(float* p) const {
    *reinterpret_cast<float4*>(p) = a;
    *reinterpret_cast<float4*>(p + 4) = b;
  }
  OSLO_DEVINL void to_float(float* f) const {
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  OSLO_DEVINL void from_float(const float* f) {
    a = make_float4(f[0], f[1], f[2], f[3]);
    b = make_float4(f[4], f[5], f[6], f[7]);
  }
};

template <int THREADS>
OSLO_DEVINL float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) total += scratch[w];
  return total;
}

// Two sums with ONE barrier: the scratch is double-buffered by call parity, so the write of call n + 2 cannot overtake a
// read of call n (every thread passes the barrier of call n + 1 in between, after its reads of call n).
template <int THREADS>
OSLO_DEVINL float2 block_sum2(float a, float b, float2* scratch /* [2][THREADS / 32] */, int parity) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float2* buf = scratch + parity * (THREADS / 32);
  if (lane == 0) buf[warp] = make_float2(a, b);
  __syncthreads();
  float2 total = make_float2(0.f, 0.f);
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) {
    const float2 v = buf[w];
    total.x += v.x;
    total.y += v.y;
  }
  return total;
}

// gamma / beta may be stored in T (same as x) or in fp32 ("mixed" variants of the reference).
template <typename T, typename W, int THREADS, int ITERS, bool RMS>
__global__ void __launch_bounds__(THREADS) norm_fwd_kernel(const T* __restrict__ x, const W* __restrict__ gamma,
                                                           const W* __restrict__ beta, T* __restrict__ y,
                                                           float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                           int rows, int H, float eps) {
  __shared__ float scratch[THREADS / 32];
  const int nvec = H >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + static_cast<size_t>(row) * H;
    float v[ITERS][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        Vec8<T> t;
        t.load(xr + vi * 8);
        t.to_float(v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += RMS ? v[i][j] * v[i][j] : v[i][j];
      }
    }
    float mean = 0.f, var;
    if (RMS) {
      var = block_sum<THREADS>(s, scratch) / H;
    } else {
      mean = block_sum<THREADS>(s, scratch) / H;
      float s2 = 0.f;
#pragma unroll
      for (int i = 0; i < ITERS; ++i) {
        const int vi = threadIdx.x + i * THREADS;
        if (vi < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float d = v[i][j] - mean;
            s2 += d * d;
          }
        }
      }
      var = block_sum<THREADS>(s2, scratch) / H;
    }
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
    T* yr = y + static_cast<size_t>(row) * H;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        float g[8], b[8], o[8];
        Vec8<W> t;
        if (gamma) { t.load(gamma + vi * 8); t.to_float(g); }
        if (beta) { t.load(beta + vi * 8); t.to_float(b); }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float n = (v[i][j] - mean) * rstd;
          if (gamma) n *= g[j];
          if (beta) n += b[j];
          o[j] = n;
        }
        Vec8<T> out;
        out.from_float(o);
        out.store(yr + vi * 8);
      }
    }
  }
}

// dx plus per-CTA partial column sums of dgamma / dbeta (partials: [gridDim.x, H] fp32).
template <typename T, typename W, int THREADS, int ITERS, bool RMS>
__global__ void __launch_bounds__(THREADS) norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                           const float* __restrict__ mean_in,
                                                           const float* __restrict__ rstd_in, const W* __restrict__ gamma,
                                                           T* __restrict__ dx, float* __restrict__ dgamma_part,
                                                           float* __restrict__ dbeta_part, int rows, int H) {
  __shared__ float2 scratch[2 * (THREADS / 32)];
  const int nvec = H >> 3;
  float acc_g[ITERS][8], acc_b[ITERS][8], g[ITERS][8];
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const int vi = threadIdx.x + i * THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc_g[i][j] = 0.f; acc_b[i][j] = 0.f; g[i][j] = 1.f; }
    if (gamma && vi < nvec) {
      Vec8<W> t;
      t.load(gamma + vi * 8);
      t.to_float(g[i]);
    }
  }
  // the next row's x and dy are requested before this row is reduced, so the loads overlap the barrier and the stores
  Vec8<T> nx[ITERS], nd[ITERS];
  auto fetch = [&](int row) {
    const size_t off = static_cast<size_t>(row) * H;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        nx[i].load(x + off + vi * 8);
        nd[i].load(dy + off + vi * 8);
      }
    }
  };
  if (static_cast<int>(blockIdx.x) < rows) fetch(blockIdx.x);
  int parity = 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x, parity ^= 1) {
    const size_t off = static_cast<size_t>(row) * H;
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float xh[ITERS][8], gd[ITERS][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        float d[8];
        nx[i].to_float(xh[i]);
        nd[i].to_float(d);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mean) * rstd;
          acc_g[i][j] += d[j] * xh[i][j];
          acc_b[i][j] += d[j];
          gd[i][j] = d[j] * g[i][j];
          s1 += gd[i][j];
          s2 += gd[i][j] * xh[i][j];
        }
      }
    }
    if (row + static_cast<int>(gridDim.x) < rows) fetch(row + gridDim.x);
    const float2 sums = block_sum2<THREADS>(s1, s2, scratch, parity);
    const float m2 = sums.y / H;
    const float m1 = RMS ? 0.f : sums.x / H;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (gd[i][j] - m1 - xh[i][j] * m2);
        Vec8<T> out;
        out.from_float(o);
        out.store(dx + off + vi * 8);
      }
    }
  }
  if (dgamma_part) {
    float* pg = dgamma_part + static_cast<size_t>(blockIdx.x) * H;
    float* pb = dbeta_part ? dbeta_part + static_cast<size_t>(blockIdx.x) * H : nullptr;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) {
        Vec8<float> t;
        t.from_float(acc_g[i]);
        t.store(pg + vi * 8);
        if (pb) {
          t.from_float(acc_b[i]);
          t.store(pb + vi * 8);
        }
      }
    }
  }
}

// out[c] = sum_r part[r, c]   (one or two matrices), result in W.
template <typename W>
__global__ void colsum_partials_kernel(const float* __restrict__ part_a, const float* __restrict__ part_b,
                                       W* __restrict__ out_a, W* __restrict__ out_b, int nparts, int H) {
  __shared__ float sa[16][33], sb[16][33];
  const int col = blockIdx.x * 32 + threadIdx.x;
  float a = 0.f, b = 0.f;
  if (col < H) {
    for (int r = threadIdx.y; r < nparts; r += 16) {
      a += part_a[static_cast<size_t>(r) * H + col];
      if (part_b) b += part_b[static_cast<size_t>(r) * H + col];
    }
  }
  sa[threadIdx.y][threadIdx.x] = a;
  sb[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.y == 0 && col < H) {
#pragma unroll
    for (int r = 1; r < 16; ++r) { a += sa[r][threadIdx.x]; b += sb[r][threadIdx.x]; }
    out_a[col] = static_cast<W>(a);
    if (part_b && out_b) out_b[col] = static_cast<W>(b);
  }
}

template <typename T, typename W, bool RMS>
static int norm_fwd_dispatch(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int rows,
                             int H, float eps, int num_sms, cudaStream_t st) {
  const int nvec = H / 8;
  const int grid = rows < num_sms * 16 ? rows : num_sms * 16;
#define OSLO_NF(TH, IT)                                                                                              \
  norm_fwd_kernel<T, W, TH, IT, RMS><<<grid, TH, 0, st>>>((const T*)x, (const W*)gamma, (const W*)beta, (T*)y, mean, \
                                                          rstd, rows, H, eps)
  if (nvec <= 128) OSLO_NF(128, 1);
  else if (nvec <= 256) OSLO_NF(128, 2);
  else if (nvec <= 512) OSLO_NF(128, 4);
  else if (nvec <= 1024) OSLO_NF(256, 4);
  else if (nvec <= 2048) OSLO_NF(256, 8);
  else return -1;
#undef OSLO_NF
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

template <typename T, typename W, bool RMS>
static int norm_bwd_dispatch(const void* dy, const void* x, const float* mean, const float* rstd, const void* gamma, void* dx,
                             float* pg, float* pb, int rows, int H, int grid, cudaStream_t st) {
  const int nvec = H / 8;
#define OSLO_NB(TH, IT)                                                                                         \
  norm_bwd_kernel<T, W, TH, IT, RMS><<<grid, TH, 0, st>>>((const T*)dy, (const T*)x, mean, rstd, (const W*)gamma, \
                                                          (T*)dx, pg, pb, rows, H)
  if (nvec <= 128) OSLO_NB(128, 1);
  else if (nvec <= 256) OSLO_NB(128, 2);
  else if (nvec <= 512) OSLO_NB(128, 4);
  else if (nvec <= 1024) OSLO_NB(256, 4);
  else if (nvec <= 2048) OSLO_NB(512, 4);
  else return -1;
#undef OSLO_NB
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace oslo

// dtype codes: 0 = fp32, 1 = fp16, 2 = bf16.  wdtype: dtype of gamma/beta (same as dtype, or 0 for fp32 params).
#define OSLO_DISPATCH_NORM(FN, ...)                                                                         \
  do {                                                                                                      \
    if (dtype == 0) return rms ? FN<float, float, true>(__VA_ARGS__) : FN<float, float, false>(__VA_ARGS__); \
    if (dtype == 1) {                                                                                       \
      if (wdtype == 0) return rms ? FN<__half, float, true>(__VA_ARGS__) : FN<__half, float, false>(__VA_ARGS__); \
      return rms ? FN<__half, __half, true>(__VA_ARGS__) : FN<__half, __half, false>(__VA_ARGS__);          \
    }                                                                                                       \
    if (wdtype == 0)                                                                                        \
      return rms ? FN<__nv_bfloat16, float, true>(__VA_ARGS__) : FN<__nv_bfloat16, float, false>(__VA_ARGS__); \
    return rms ? FN<__nv_bfloat16, __nv_bfloat16, true>(__VA_ARGS__)                                        \
               : FN<__nv_bfloat16, __nv_bfloat16, false>(__VA_ARGS__);                                      \
  } while (0)

// y = (x - mean) * rstd * gamma + beta  (rms != 0: y = x * rstd * gamma).  H % 8 == 0, H <= 16384.
extern "C" int oslo_norm_forward(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                                 int rows, int H, float eps, int rms, int dtype, int wdtype, int num_sms, void* stream) {
  if (rows <= 0) return 0;
  if (H % 8 || H > 16384) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OSLO_DISPATCH_NORM(oslo::norm_fwd_dispatch, x, gamma, beta, y, mean, rstd, rows, H, eps, num_sms, st);
}

// Number of partial rows the backward kernel writes (size of the scratch: 2 * parts * H floats).
extern "C" int oslo_norm_backward_parts(int rows, int num_sms) {
  const int cap = num_sms * 4;
  return rows < cap ? rows : cap;
}

// dx, and (when gamma given) dgamma / dbeta via `partials` scratch of 2 * parts * H floats.
extern "C" int oslo_norm_backward(const void* dy, const void* x, const float* mean, const float* rstd, const void* gamma,
                                  void* dx, void* dgamma, void* dbeta, float* partials, int rows, int H, int rms, int dtype,
                                  int wdtype, int num_sms, void* stream) {
  if (rows <= 0) return 0;
  if (H % 8 || H > 16384) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int parts = oslo_norm_backward_parts(rows, num_sms);
  float* pg = dgamma ? partials : nullptr;
  float* pb = (dgamma && dbeta) ? partials + static_cast<size_t>(parts) * H : nullptr;
  int rc = [&]() -> int { OSLO_DISPATCH_NORM(oslo::norm_bwd_dispatch, dy, x, mean, rstd, gamma, dx, pg, pb, rows, H, parts, st); }();
  if (rc) return rc;
  if (dgamma) {
    dim3 block(32, 16), grid((H + 31) / 32);
    if (wdtype == 0 || dtype == 0)
      oslo::colsum_partials_kernel<float><<<grid, block, 0, st>>>(pg, pb, (float*)dgamma, (float*)dbeta, parts, H);
    else if (dtype == 1)
      oslo::colsum_partials_kernel<__half><<<grid, block, 0, st>>>(pg, pb, (__half*)dgamma, (__half*)dbeta, parts, H);
    else
      oslo::colsum_partials_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(pg, pb, (__nv_bfloat16*)dgamma, (__nv_bfloat16*)dbeta, parts, H);
    if (cudaGetLastError() != cudaSuccess) return -2;
  }
  return 0;
}

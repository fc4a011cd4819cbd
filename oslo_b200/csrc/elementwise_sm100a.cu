// Bandwidth-bound fused elementwise kernels for sm_100a (bf16 / fp16 / fp32):
//   bias + GELU (tanh) fwd / bwd, SwiGLU fwd / bwd, bias + dropout + residual,
//   rotary position embedding (partial rotary, NeoX half-rotation or GPT-J
//   interleaved), scale + mask + softmax fwd / bwd, column sums (bias gradients).
// All use 16-byte accesses and grid-stride loops sized to the SM count.
//
// Replaces the TorchScript fusions in oslo/torch/nn/modules/functional.py:23-84,295-298,
// the missing scaled_masked_softmax .cu behind FusedScaleMaskSoftmaxBinder.cpp:29-127, and
// lightseq2 dropout_kernels.cu / softmax_kernels.cu / general_kernels.cu column_sum_reduce.
#include "common.cuh"

namespace oslo {

template <typename T> OSLO_DEVINL float to_f(T v);
template <> OSLO_DEVINL float to_f<float>(float v) { return v; }
template <> OSLO_DEVINL float to_f<__half>(__half v) { return __half2float(v); }
template <> OSLO_DEVINL float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> OSLO_DEVINL T from_f(float v);
template <> OSLO_DEVINL float from_f<float>(float v) { return v; }
template <> OSLO_DEVINL __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> OSLO_DEVINL __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 16-byte packet of T
template <typename T> struct Pack {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};
template <typename T> OSLO_DEVINL Pack<T> ld_pack(const T* p) {
  Pack<T> r;
  *reinterpret_cast<uint4*>(r.v) = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <typename T> OSLO_DEVINL void st_pack(T* p, const Pack<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(r.v);
}

// activation selected at run time (uniform over the launch): 0 tanh-form GELU, 1 erf-form GELU, 2 ReLU
OSLO_DEVINL float act_apply(float v, int act) {
  if (act == 0) return gelu_tanh(v);
  if (act == 1) return 0.5f * v * (1.0f + erff(v * 0.7071067811865476f));
  return fmaxf(v, 0.f);
}
OSLO_DEVINL float act_grad(float v, int act) {
  if (act == 0) return gelu_tanh_grad(v);
  if (act == 1) return 0.5f * (1.0f + erff(v * 0.7071067811865476f)) + v * 0.3989422804014327f * __expf(-0.5f * v * v);
  return v > 0.f ? 1.f : 0.f;
}

// y = act(x + bias); bias broadcast over rows (may be null). n = rows * H, H % pack == 0.
template <typename T>
__global__ void bias_gelu_fwd_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ y, size_t n, int H,
                                     int act) {
  constexpr int P = Pack<T>::N;
  const size_t nv = n / P;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    Pack<T> a = ld_pack(x + i * P), o;
    Pack<T> b;
    if (bias) b = ld_pack(bias + (i * P) % H);
#pragma unroll
    for (int j = 0; j < P; ++j) {
      float v = to_f(a.v[j]) + (bias ? to_f(b.v[j]) : 0.f);
      o.v[j] = from_f<T>(act_apply(v, act));
    }
    st_pack(y + i * P, o);
  }
}

// dx = dy * act'(x + bias)
template <typename T>
__global__ void bias_gelu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ bias,
                                     T* __restrict__ dx, size_t n, int H, int act) {
  constexpr int P = Pack<T>::N;
  const size_t nv = n / P;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    Pack<T> a = ld_pack(x + i * P), g = ld_pack(dy + i * P), o;
    Pack<T> b;
    if (bias) b = ld_pack(bias + (i * P) % H);
#pragma unroll
    for (int j = 0; j < P; ++j) {
      float v = to_f(a.v[j]) + (bias ? to_f(b.v[j]) : 0.f);
      o.v[j] = from_f<T>(to_f(g.v[j]) * act_grad(v, act));
    }
    st_pack(dx + i * P, o);
  }
}

// SwiGLU on a packed [rows, 2F] tensor (gate = [:, :F], up = [:, F:]) or two tensors (ld given).
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ y, size_t rows, int F,
                                  long long ld_in) {
  constexpr int P = Pack<T>::N;
  const int fv = F / P;
  const size_t nv = rows * fv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / fv;
    const int c = (int)(i % fv) * P;
    Pack<T> g = ld_pack(gate + r * ld_in + c), u = ld_pack(up + r * ld_in + c), o;
#pragma unroll
    for (int j = 0; j < P; ++j) {
      const float gv = to_f(g.v[j]);
      o.v[j] = from_f<T>(gv / (1.0f + __expf(-gv)) * to_f(u.v[j]));
    }
    st_pack(y + r * F + c, o);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ gate, const T* __restrict__ up,
                                  T* __restrict__ dgate, T* __restrict__ dup, size_t rows, int F, long long ld_in) {
  constexpr int P = Pack<T>::N;
  const int fv = F / P;
  const size_t nv = rows * fv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / fv;
    const int c = (int)(i % fv) * P;
    Pack<T> g = ld_pack(gate + r * ld_in + c), u = ld_pack(up + r * ld_in + c), d = ld_pack(dy + r * F + c), og, ou;
#pragma unroll
    for (int j = 0; j < P; ++j) {
      const float gv = to_f(g.v[j]), uv = to_f(u.v[j]), dv = to_f(d.v[j]);
      const float s = 1.0f / (1.0f + __expf(-gv));
      const float silu = gv * s;
      ou.v[j] = from_f<T>(dv * silu);
      og.v[j] = from_f<T>(dv * uv * (s + silu * (1.0f - s)));
    }
    st_pack(dgate + r * ld_in + c, og);
    st_pack(dup + r * ld_in + c, ou);
  }
}

// Counter-based RNG (Philox-4x32-10): the dropout mask is a pure function of (seed, offset, index),
// so backward recomputes it instead of storing a mask tensor.
OSLO_DEVINL uint4 philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// out = residual + dropout(x + bias, p) ; with grad mode: dx = dropout_mask(dy) (same seed/offset).
template <typename T, bool BWD>
__global__ void bias_dropout_add_kernel(const T* __restrict__ x, const T* __restrict__ bias, const T* __restrict__ residual,
                                        T* __restrict__ out, size_t n, int H, float p, unsigned long long seed,
                                        unsigned long long offset) {
  constexpr int P = Pack<T>::N;
  const size_t nv = n / P;
  const float scale = p < 1.f ? 1.0f / (1.0f - p) : 0.f;
  const uint32_t thresh = (uint32_t)(p * 4294967295.0);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    Pack<T> a = ld_pack(x + i * P), o, b, r;
    if (!BWD && bias) b = ld_pack(bias + (i * P) % H);
    if (!BWD && residual) r = ld_pack(residual + i * P);
    uint32_t rnd[8];
    if (p > 0.f) {
      uint4 r0 = philox4x32((uint32_t)i, (uint32_t)(i >> 32), (uint32_t)offset, (uint32_t)(offset >> 32), (uint32_t)seed,
                            (uint32_t)(seed >> 32));
      rnd[0] = r0.x; rnd[1] = r0.y; rnd[2] = r0.z; rnd[3] = r0.w;
      if (P > 4) {
        uint4 r1 = philox4x32((uint32_t)i, (uint32_t)(i >> 32) | 0x80000000u, (uint32_t)offset, (uint32_t)(offset >> 32),
                              (uint32_t)seed, (uint32_t)(seed >> 32));
        rnd[4] = r1.x; rnd[5] = r1.y; rnd[6] = r1.z; rnd[7] = r1.w;
      }
    }
#pragma unroll
    for (int j = 0; j < P; ++j) {
      float v = to_f(a.v[j]);
      if (!BWD && bias) v += to_f(b.v[j]);
      if (p > 0.f) v = (rnd[j] >= thresh) ? v * scale : 0.f;
      if (!BWD && residual) v += to_f(r.v[j]);
      o.v[j] = from_f<T>(v);
    }
    st_pack(out + i * P, o);
  }
}

// Rotary embedding in place on x[tokens, heads, head_dim] (row stride ld between tokens, head stride hs),
// rotating the first rot_dim dims of each head.  cos/sin: [seq, rot_dim/2] fp32, position = pos[token]
// (or token % seq when pos is null).  neox != 0: pairs (i, i + rot/2); else interleaved pairs (2i, 2i+1).
// sign = +1 forward, -1 backward (inverse rotation).
template <typename T>
__global__ void rope_kernel(T* __restrict__ x, const float* __restrict__ cosb, const float* __restrict__ sinb,
                            const int* __restrict__ pos, size_t tokens, int heads, int rot_dim, int seq, long long ld,
                            long long hs, int neox, float sign) {
  const int half = rot_dim / 2;
  const size_t total = tokens * heads * half;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int d = (int)(i % half);
    const size_t th = i / half;
    const int h = (int)(th % heads);
    const size_t t = th / heads;
    const int p = pos ? pos[t] : (int)(t % seq);
    const float c = cosb[(size_t)p * half + d], s = sign * sinb[(size_t)p * half + d];
    T* base = x + t * ld + h * hs;
    const int i0 = neox ? d : 2 * d, i1 = neox ? d + half : 2 * d + 1;
    const float a = to_f(base[i0]), b = to_f(base[i1]);
    base[i0] = from_f<T>(a * c - b * s);
    base[i1] = from_f<T>(b * c + a * s);
  }
}

// The same rotation for 2-byte types in the rotate-half ("neox") pairing, 16 bytes at a time: one thread takes eight
// consecutive d of one (token, head, part) and the eight partners at d + rot/2.  `parts` tensors that share the token and
// head strides and lie `ps` elements apart (q and k inside one fused QKV buffer) are rotated by one launch.
template <typename T>
__global__ void rope_vec_kernel(T* __restrict__ x, const float* __restrict__ cosb, const float* __restrict__ sinb,
                                const int* __restrict__ pos, size_t tokens, int heads, int rot_dim, int seq, long long ld,
                                long long hs, int parts, long long ps, float sign) {
  const int half = rot_dim / 2;
  const int chunks = half / 8;
  const size_t total = tokens * heads * parts * chunks;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % chunks);
    size_t r = i / chunks;
    const int part = (int)(r % parts);
    r /= parts;
    const int h = (int)(r % heads);
    const size_t t = r / heads;
    const int p = pos ? pos[t] : (int)(t % seq);
    const float4* cp = reinterpret_cast<const float4*>(cosb + (size_t)p * half + c * 8);
    const float4* sp = reinterpret_cast<const float4*>(sinb + (size_t)p * half + c * 8);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    T* base = x + t * ld + h * hs + part * ps + c * 8;
    Pack<T> a = ld_pack(base), b = ld_pack(base + half);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float av = to_f(a.v[j]), bv = to_f(b.v[j]), sj = sign * sn[j];
      a.v[j] = from_f<T>(av * cs[j] - bv * sj);
      b.v[j] = from_f<T>(bv * cs[j] + av * sj);
    }
    st_pack(base, a);
    st_pack(base + half, b);
  }
}

// Row softmax of scale * x (+ additive mask) with optional causal masking.  One warp per row.
// x: [batches, sq, sk]; mask (optional): additive fp32/T-agnostic float [mask_batches, sq or 1, sk]
// causal: key j is visible to query i iff j <= i + (sk - sq).
template <typename T>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ mask,
                                   size_t rows, int sq, int sk, float scale, int causal, int heads_per_mask, int mask_rows) {
  const int lane = threadIdx.x & 31;
  const size_t warp_global = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t row = warp_global; row < rows; row += nwarps) {
    const int qi = (int)(row % sq);
    const size_t bh = row / sq;
    const int limit = causal ? min(sk, qi + (sk - sq) + 1) : sk;
    const T* xr = x + row * sk;
    T* yr = y + row * sk;
    const float* mr = nullptr;
    if (mask) mr = mask + ((bh / heads_per_mask) * mask_rows + (mask_rows == 1 ? 0 : qi)) * (size_t)sk;
    float mx = -INFINITY;
    for (int j = lane * 8; j < limit; j += 256) {
      Pack<T> a = ld_pack(xr + j);
#pragma unroll
      for (int e = 0; e < Pack<T>::N; ++e) {
        if (j + e < limit) {
          float v = to_f(a.v[e]) * scale + (mr ? mr[j + e] : 0.f);
          mx = fmaxf(mx, v);
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (mx == -INFINITY) mx = 0.f;
    float sum = 0.f;
    for (int j = lane * 8; j < limit; j += 256) {
      Pack<T> a = ld_pack(xr + j);
#pragma unroll
      for (int e = 0; e < Pack<T>::N; ++e)
        if (j + e < limit) sum += __expf(to_f(a.v[e]) * scale + (mr ? mr[j + e] : 0.f) - mx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = sum > 0.f ? 1.0f / sum : 0.f;
    for (int j = lane * 8; j < sk; j += 256) {
      Pack<T> a = ld_pack(xr + j), o;
#pragma unroll
      for (int e = 0; e < Pack<T>::N; ++e) {
        float v = 0.f;
        if (j + e < limit) v = __expf(to_f(a.v[e]) * scale + (mr ? mr[j + e] : 0.f) - mx) * inv;
        o.v[e] = from_f<T>(v);
      }
      st_pack(yr + j, o);
    }
  }
}
// dx = scale * y * (dy - sum(dy * y)).  With sq > 0 (causal) only keys j <= query index are read from
// dy (entries beyond may be uninitialised) and dx is zero there.
template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, size_t rows, int sk,
                                   float scale, int sq) {
  const int lane = threadIdx.x & 31;
  const size_t warp_global = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t row = warp_global; row < rows; row += nwarps) {
    const int limit = sq > 0 ? min(sk, (int)(row % sq) + (sk - sq) + 1) : sk;
    const T* yr = y + row * sk;
    const T* gr = dy + row * sk;
    T* dr = dx + row * sk;
    float dot = 0.f;
    for (int j = lane * 8; j < limit; j += 256) {
      Pack<T> a = ld_pack(yr + j), g = ld_pack(gr + j);
#pragma unroll
      for (int e = 0; e < Pack<T>::N; ++e)
        if (j + e < limit) dot += to_f(a.v[e]) * to_f(g.v[e]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    for (int j = lane * 8; j < sk; j += 256) {
      Pack<T> o;
      if (j < limit) {
        Pack<T> a = ld_pack(yr + j), g = ld_pack(gr + j);
#pragma unroll
        for (int e = 0; e < Pack<T>::N; ++e)
          o.v[e] = from_f<T>(j + e < limit ? scale * to_f(a.v[e]) * (to_f(g.v[e]) - dot) : 0.f);
      } else {
#pragma unroll
        for (int e = 0; e < Pack<T>::N; ++e) o.v[e] = from_f<T>(0.f);
      }
      st_pack(dr + j, o);
    }
  }
}

// Column sums of x[rows, H] -> partial[gridDim.y, H] fp32 (second pass: colsum_partials in norm file style).
template <typename T>
__global__ void colsum_kernel(const T* __restrict__ x, float* __restrict__ partial, size_t rows, int H) {
  // block: 32 x 8 threads; each thread owns 8 consecutive columns (one 16-byte packet for 2-byte types)
  constexpr int P = Pack<T>::N;
  const int col = (blockIdx.x * 32 + threadIdx.x) * P;
  float acc[P];
#pragma unroll
  for (int j = 0; j < P; ++j) acc[j] = 0.f;
  if (col < H) {
    // four independent 16-byte loads in flight per thread
    const size_t stride = (size_t)gridDim.y * blockDim.y;
    size_t r = blockIdx.y * (size_t)blockDim.y + threadIdx.y;
    for (; r + 3 * stride < rows; r += 4 * stride) {
      Pack<T> a0 = ld_pack(x + r * H + col), a1 = ld_pack(x + (r + stride) * H + col);
      Pack<T> a2 = ld_pack(x + (r + 2 * stride) * H + col), a3 = ld_pack(x + (r + 3 * stride) * H + col);
#pragma unroll
      for (int j = 0; j < P; ++j) acc[j] += (to_f(a0.v[j]) + to_f(a1.v[j])) + (to_f(a2.v[j]) + to_f(a3.v[j]));
    }
    for (; r < rows; r += stride) {
      Pack<T> a = ld_pack(x + r * H + col);
#pragma unroll
      for (int j = 0; j < P; ++j) acc[j] += to_f(a.v[j]);
    }
  }
  __shared__ float sm[8][32 * P + 1];
#pragma unroll
  for (int j = 0; j < P; ++j) sm[threadIdx.y][threadIdx.x * P + j] = acc[j];
  __syncthreads();
  if (threadIdx.y == 0 && col < H) {
#pragma unroll
    for (int j = 0; j < P; ++j) {
      float s = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) s += sm[r][threadIdx.x * P + j];
      partial[(size_t)blockIdx.y * H + col + j] = s;
    }
  }
}
// Sum of the partial rows: block (32 columns x 8 row groups), every thread adds parts / 8 values, shared-memory fold.
template <typename T>
__global__ void colsum_finish_kernel(const float* __restrict__ partial, T* __restrict__ out, int parts, int H) {
  const int col = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (col < H)
    for (int r = threadIdx.y; r < parts; r += 8) s += partial[(size_t)r * H + col];
  __shared__ float sm[8][33];
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && col < H) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) t += sm[r][threadIdx.x];
    out[col] = from_f<T>(t);
  }
}

static inline int grid_for(size_t work_items, int threads, int num_sms) {
  size_t blocks = (work_items + threads - 1) / threads;
  size_t cap = (size_t)num_sms * 8;
  return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

}  // namespace oslo

#define OSLO_BY_DTYPE(CALL_F32, CALL_F16, CALL_BF16) \
  do {                                               \
    if (dtype == 0) { CALL_F32; }                    \
    else if (dtype == 1) { CALL_F16; }               \
    else { CALL_BF16; }                              \
  } while (0)

using namespace oslo;

extern "C" int oslo_bias_act_forward(const void* x, const void* bias, void* y, long long n, int H, int dtype, int act,
                                     int num_sms, void* stream) {
  if (n <= 0) return 0;
  if (act < 0 || act > 2) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  const int P = dtype == 0 ? 4 : 8;
  if (H % P || n % P) return -1;
  const int g = grid_for(n / P, 256, num_sms);
  OSLO_BY_DTYPE((bias_gelu_fwd_kernel<float><<<g, 256, 0, st>>>((const float*)x, (const float*)bias, (float*)y, n, H, act)),
                (bias_gelu_fwd_kernel<__half><<<g, 256, 0, st>>>((const __half*)x, (const __half*)bias, (__half*)y, n, H, act)),
                (bias_gelu_fwd_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)bias,
                                                                        (__nv_bfloat16*)y, n, H, act)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_bias_act_backward(const void* dy, const void* x, const void* bias, void* dx, long long n, int H, int dtype,
                                      int act, int num_sms, void* stream) {
  if (n <= 0) return 0;
  if (act < 0 || act > 2) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  const int P = dtype == 0 ? 4 : 8;
  if (H % P || n % P) return -1;
  const int g = grid_for(n / P, 256, num_sms);
  OSLO_BY_DTYPE((bias_gelu_bwd_kernel<float><<<g, 256, 0, st>>>((const float*)dy, (const float*)x, (const float*)bias, (float*)dx, n, H, act)),
                (bias_gelu_bwd_kernel<__half><<<g, 256, 0, st>>>((const __half*)dy, (const __half*)x, (const __half*)bias, (__half*)dx, n, H, act)),
                (bias_gelu_bwd_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                                        (const __nv_bfloat16*)bias, (__nv_bfloat16*)dx, n, H, act)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_bias_gelu_forward(const void* x, const void* bias, void* y, long long n, int H, int dtype, int num_sms,
                                      void* stream) {
  return oslo_bias_act_forward(x, bias, y, n, H, dtype, 0, num_sms, stream);
}

extern "C" int oslo_bias_gelu_backward(const void* dy, const void* x, const void* bias, void* dx, long long n, int H, int dtype,
                                       int num_sms, void* stream) {
  return oslo_bias_act_backward(dy, x, bias, dx, n, H, dtype, 0, num_sms, stream);
}

extern "C" int oslo_swiglu_forward(const void* gate, const void* up, void* y, long long rows, int F, long long ld_in, int dtype,
                                   int num_sms, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int P = dtype == 0 ? 4 : 8;
  if (F % P || ld_in % P) return -1;
  const int g = grid_for((size_t)rows * F / P, 256, num_sms);
  OSLO_BY_DTYPE((swiglu_fwd_kernel<float><<<g, 256, 0, st>>>((const float*)gate, (const float*)up, (float*)y, rows, F, ld_in)),
                (swiglu_fwd_kernel<__half><<<g, 256, 0, st>>>((const __half*)gate, (const __half*)up, (__half*)y, rows, F, ld_in)),
                (swiglu_fwd_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)gate, (const __nv_bfloat16*)up,
                                                                     (__nv_bfloat16*)y, rows, F, ld_in)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_swiglu_backward(const void* dy, const void* gate, const void* up, void* dgate, void* dup, long long rows,
                                    int F, long long ld_in, int dtype, int num_sms, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int P = dtype == 0 ? 4 : 8;
  if (F % P || ld_in % P) return -1;
  const int g = grid_for((size_t)rows * F / P, 256, num_sms);
  OSLO_BY_DTYPE((swiglu_bwd_kernel<float><<<g, 256, 0, st>>>((const float*)dy, (const float*)gate, (const float*)up, (float*)dgate, (float*)dup, rows, F, ld_in)),
                (swiglu_bwd_kernel<__half><<<g, 256, 0, st>>>((const __half*)dy, (const __half*)gate, (const __half*)up, (__half*)dgate, (__half*)dup, rows, F, ld_in)),
                (swiglu_bwd_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up,
                                                                     (__nv_bfloat16*)dgate, (__nv_bfloat16*)dup, rows, F, ld_in)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// backward != 0: out = mask(x) * scale only (bias / residual ignored).
extern "C" int oslo_bias_dropout_add(const void* x, const void* bias, const void* residual, void* out, long long n, int H,
                                     float p, unsigned long long seed, unsigned long long offset, int backward, int dtype,
                                     int num_sms, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int P = dtype == 0 ? 4 : 8;
  if (H % P || n % P) return -1;
  const int g = grid_for(n / P, 256, num_sms);
#define OSLO_BDA(T, B) bias_dropout_add_kernel<T, B><<<g, 256, 0, st>>>((const T*)x, (const T*)bias, (const T*)residual, (T*)out, n, H, p, seed, offset)
  if (backward) OSLO_BY_DTYPE(OSLO_BDA(float, true), OSLO_BDA(__half, true), OSLO_BDA(__nv_bfloat16, true));
  else OSLO_BY_DTYPE(OSLO_BDA(float, false), OSLO_BDA(__half, false), OSLO_BDA(__nv_bfloat16, false));
#undef OSLO_BDA
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_rope(void* x, const float* cosb, const float* sinb, const int* pos, long long tokens, int heads, int rot_dim,
                         int seq, long long ld, long long hs, int neox, int backward, int dtype, int num_sms, void* stream) {
  if (tokens <= 0 || rot_dim <= 0) return 0;
  if (rot_dim % 2) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  const int g = grid_for((size_t)tokens * heads * (rot_dim / 2), 256, num_sms);
  const float sign = backward ? -1.f : 1.f;
  OSLO_BY_DTYPE((rope_kernel<float><<<g, 256, 0, st>>>((float*)x, cosb, sinb, pos, tokens, heads, rot_dim, seq, ld, hs, neox, sign)),
                (rope_kernel<__half><<<g, 256, 0, st>>>((__half*)x, cosb, sinb, pos, tokens, heads, rot_dim, seq, ld, hs, neox, sign)),
                (rope_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((__nv_bfloat16*)x, cosb, sinb, pos, tokens, heads, rot_dim, seq, ld, hs, neox, sign)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// x, y: [batches * sq, sk] contiguous; sk % 8 == 0 (4 for fp32).  mask: additive fp32 or null.
// `parts` tensors `ps` elements apart (same token / head strides) in one call; the 16-byte kernel when the layout allows it.
extern "C" int oslo_rope_parts(void* x, const float* cosb, const float* sinb, const int* pos, long long tokens, int heads,
                               int rot_dim, int seq, long long ld, long long hs, int parts, long long ps, int neox, int backward,
                               int dtype, int num_sms, void* stream) {
  if (tokens <= 0 || rot_dim <= 0 || parts <= 0) return 0;
  if (rot_dim % 2) return -1;
  const int half = rot_dim / 2;
  const bool vec = dtype != 0 && neox && half % 8 == 0 && ld % 8 == 0 && hs % 8 == 0 && (parts == 1 || ps % 8 == 0) &&
                   (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(cosb) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(sinb) & 15) == 0;
  if (!vec) {
    const long long esz = dtype == 0 ? 4 : 2;
    for (int part = 0; part < parts; ++part) {
      const int rc = oslo_rope(static_cast<char*>(x) + part * ps * esz, cosb, sinb, pos, tokens, heads, rot_dim, seq, ld, hs, neox,
                               backward, dtype, num_sms, stream);
      if (rc) return rc;
    }
    return 0;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const int g = grid_for((size_t)tokens * heads * parts * (half / 8), 256, num_sms);
  const float sign = backward ? -1.f : 1.f;
  if (dtype == 1) rope_vec_kernel<__half><<<g, 256, 0, st>>>((__half*)x, cosb, sinb, pos, tokens, heads, rot_dim, seq, ld, hs, parts, ps, sign);
  else rope_vec_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((__nv_bfloat16*)x, cosb, sinb, pos, tokens, heads, rot_dim, seq, ld, hs, parts, ps, sign);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_softmax_forward(const void* x, void* y, const float* mask, long long rows, int sq, int sk, float scale,
                                    int causal, int heads_per_mask, int mask_rows, int dtype, int num_sms, void* stream) {
  if (rows <= 0) return 0;
  if (dtype == 0 || sk % 8) return -1;  // 2-byte types only; fp32 falls back to torch in Python
  cudaStream_t st = (cudaStream_t)stream;
  const int g = grid_for((size_t)rows * 32, 256, num_sms);
  if (dtype == 1)
    softmax_fwd_kernel<__half><<<g, 256, 0, st>>>((const __half*)x, (__half*)y, mask, rows, sq, sk, scale, causal, heads_per_mask, mask_rows);
  else
    softmax_fwd_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, mask, rows, sq, sk, scale, causal, heads_per_mask, mask_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_softmax_backward(const void* dy, const void* y, void* dx, long long rows, int sk, float scale, int dtype,
                                     int num_sms, void* stream) {
  if (rows <= 0) return 0;
  if (dtype == 0 || sk % 8) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  const int g = grid_for((size_t)rows * 32, 256, num_sms);
  if (dtype == 1)
    softmax_bwd_kernel<__half><<<g, 256, 0, st>>>((const __half*)dy, (const __half*)y, (__half*)dx, rows, sk, scale, 0);
  else
    softmax_bwd_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)y, (__nv_bfloat16*)dx, rows, sk, scale, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_softmax_backward_causal(const void* dy, const void* y, void* dx, long long rows, int sq, int sk, float scale,
                                            int dtype, int num_sms, void* stream) {
  if (rows <= 0) return 0;
  if (dtype == 0 || sk % 8 || sq <= 0) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  const int g = grid_for((size_t)rows * 32, 256, num_sms);
  if (dtype == 1)
    softmax_bwd_kernel<__half><<<g, 256, 0, st>>>((const __half*)dy, (const __half*)y, (__half*)dx, rows, sk, scale, sq);
  else
    softmax_bwd_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)y, (__nv_bfloat16*)dx, rows, sk, scale, sq);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Number of partial rows used by oslo_colsum (scratch = parts * H floats).
extern "C" int oslo_colsum_parts(long long rows, int num_sms) {
  long long p = (rows + 63) / 64;
  long long cap = num_sms / 2 > 0 ? num_sms / 2 : 1;  // enough blocks to fill the GPU, few enough rows for the second pass
  return (int)(p < cap ? (p ? p : 1) : cap);
}

extern "C" int oslo_colsum(const void* x, void* out, float* partial, long long rows, int H, int dtype, int num_sms, void* stream) {
  if (H <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int P = dtype == 0 ? 4 : 8;
  if (H % P) return -1;
  const int parts = oslo_colsum_parts(rows, num_sms);
  dim3 block(32, 8), grid((H / P + 31) / 32, parts);
  OSLO_BY_DTYPE((colsum_kernel<float><<<grid, block, 0, st>>>((const float*)x, partial, rows, H)),
                (colsum_kernel<__half><<<grid, block, 0, st>>>((const __half*)x, partial, rows, H)),
                (colsum_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)x, partial, rows, H)));
  const int fb = (H + 31) / 32;
  const dim3 fblock(32, 8);
  OSLO_BY_DTYPE((colsum_finish_kernel<float><<<fb, fblock, 0, st>>>(partial, (float*)out, parts, H)),
                (colsum_finish_kernel<__half><<<fb, fblock, 0, st>>>(partial, (__half*)out, parts, H)),
                (colsum_finish_kernel<__nv_bfloat16><<<fb, fblock, 0, st>>>(partial, (__nv_bfloat16*)out, parts, H)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free column sum (declared in oslo_b200_noalloc.h).  Same kernels as oslo_colsum, but the
// per-block partial sums go to a fixed array that is part of the library image instead of a buffer the
// caller allocates.  See the header for who needs this and for the rules of use.
#include "oslo_b200_noalloc.h"
#include <cstdio>
#include <mutex>

namespace {
constexpr long long kNoAllocScratchFloats = OSLO_COLSUM_NOALLOC_MAX_SCRATCH_FLOATS;
// Lives in every GPU that loads the library until the process exits (8 MiB).
static __device__ __align__(256) float g_colsum_noalloc_scratch[kNoAllocScratchFloats];

constexpr int kMaxDevices = 64;
struct NoAllocDeviceState {
  float* scratch = nullptr;  // DEVICE address of g_colsum_noalloc_scratch on that device
  int num_sms = 0;
};
NoAllocDeviceState g_noalloc_state[kMaxDevices];
std::mutex g_noalloc_mutex;

// One-time set-up for the current device.  In host code the array's name is only a handle for the
// runtime, not an address a kernel can use, so the device address is looked up once and kept.
int noalloc_setup(int dev, NoAllocDeviceState** out) {
  if (dev < 0 || dev >= kMaxDevices) return OSLO_NOALLOC_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  NoAllocDeviceState& st = g_noalloc_state[dev];
  if (st.scratch == nullptr) {
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_colsum_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      fprintf(stderr, "oslo_colsum_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return OSLO_NOALLOC_ERR_SETUP;
    }
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || sms <= 0) {
      fprintf(stderr, "oslo_colsum_noalloc: cannot read the SM count: %s\n", cudaGetErrorString(e));
      return OSLO_NOALLOC_ERR_SETUP;
    }
    st.num_sms = sms;
    st.scratch = ptr;
  }
  *out = &st;
  return 0;
}
}  // namespace

extern "C" long long oslo_colsum_noalloc_max_scratch_floats() { return kNoAllocScratchFloats; }

extern "C" int oslo_colsum_noalloc(const void* x, void* out, long long rows, int H, int dtype, void* stream) {
  if (H <= 0 || rows < 0) return 0;
  if (dtype < 0 || dtype > 2) return OSLO_NOALLOC_ERR_ARGUMENT;
  const int P = dtype == 0 ? 4 : 8;
  if (H % P) {
    fprintf(stderr, "oslo_colsum_noalloc: H = %d must be a multiple of %d for this dtype\n", H, P);
    return OSLO_NOALLOC_ERR_ARGUMENT;
  }
  // the kernels read x and write out with 16-byte vectors: refuse a misaligned pointer here, before any launch
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || x == nullptr || out == nullptr) {
    fprintf(stderr, "oslo_colsum_noalloc: x (%p) and out (%p) must be non-null and 16-byte aligned\n", x, out);
    return OSLO_NOALLOC_ERR_ARGUMENT;
  }
  if (static_cast<long long>(H) > kNoAllocScratchFloats) {
    fprintf(stderr,
            "oslo_colsum_noalloc: H = %d columns exceeds the built-in scratch of %lld floats; use oslo_colsum with a "
            "caller-provided buffer instead\n", H, kNoAllocScratchFloats);
    return OSLO_NOALLOC_ERR_TOO_LARGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return OSLO_NOALLOC_ERR_DEVICE;
  NoAllocDeviceState* st = nullptr;
  int rc = noalloc_setup(dev, &st);
  if (rc) return rc;
  // as many row partitions as oslo_colsum would use, capped so that parts * H fits the fixed array
  long long parts = oslo_colsum_parts(rows, st->num_sms);
  const long long fit = kNoAllocScratchFloats / H;
  if (parts > fit) parts = fit;
  if (parts < 1) parts = 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* partial = st->scratch;  // every (part, column) cell used below is overwritten: nothing to clear
  dim3 block(32, 8), grid((H / P + 31) / 32, static_cast<unsigned>(parts));
  OSLO_BY_DTYPE((colsum_kernel<float><<<grid, block, 0, s>>>((const float*)x, partial, rows, H)),
                (colsum_kernel<__half><<<grid, block, 0, s>>>((const __half*)x, partial, rows, H)),
                (colsum_kernel<__nv_bfloat16><<<grid, block, 0, s>>>((const __nv_bfloat16*)x, partial, rows, H)));
  const int fb = (H + 31) / 32;
  const dim3 fblock(32, 8);  // the second pass folds 8 row groups per column in shared memory
  OSLO_BY_DTYPE((colsum_finish_kernel<float><<<fb, fblock, 0, s>>>(partial, (float*)out, (int)parts, H)),
                (colsum_finish_kernel<__half><<<fb, fblock, 0, s>>>(partial, (__half*)out, (int)parts, H)),
                (colsum_finish_kernel<__nv_bfloat16><<<fb, fblock, 0, s>>>(partial, (__nv_bfloat16*)out, (int)parts, H)));
  return cudaGetLastError() == cudaSuccess ? 0 : OSLO_NOALLOC_ERR_LAUNCH;
}

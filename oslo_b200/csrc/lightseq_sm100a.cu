// LightSeq-specific kernels for sm_100a that the transformer building blocks of this library do not already cover:
//
//   oslo_ls_embedding_forward / _backward   token lookup x scale + positional row + dropout, padding rows zeroed
//                                           (oslo/lightseq2/csrc/kernels/cuda/embedding_kernels.cu:312-359, backward :420-470)
//   oslo_ls_quantize / oslo_ls_dequantize   symmetric per-tensor int8 with a clip maximum, plus the clipped-element mask
//                                           that quantisation-aware training needs (csrc/kernels/cuda/quantize_kernels.cu)
//   oslo_ls_sample                          per-row top-k / top-p (nucleus) sampling of next tokens on the device
//                                           (oslo/lightseq2/inference/kernels/transformerKernels.cc.cu ker_topk_sample /
//                                           ker_topp_sample), without sorting the vocabulary
//
// All are bandwidth-bound: 16-byte accesses, one pass (embedding, quantise) or a fixed number of counting passes over one
// row of logits held in L2 (sampling).  Dropout masks are a pure function of (seed, offset, element index) through a
// counter-based generator, so backward recomputes them instead of storing them.
#include "common.cuh"

namespace oslo {

OSLO_DEVINL uint32_t mix32(uint64_t x) {  // splitmix64 finaliser: one well-mixed 32-bit value per element index
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return static_cast<uint32_t>((x ^ (x >> 31)) >> 32);
}
OSLO_DEVINL bool keep_element(uint64_t seed, uint64_t offset, uint64_t idx, float p) {
  if (p <= 0.f) return true;
  const uint32_t r = mix32(seed ^ (offset * 0xD1342543DE82EF95ull) ^ (idx * 0x9E3779B97F4A7C15ull + offset));
  return (r >> 8) * (1.0f / 16777216.0f) >= p;
}

template <typename T> OSLO_DEVINL float lsf(T v);
template <> OSLO_DEVINL float lsf<float>(float v) { return v; }
template <> OSLO_DEVINL float lsf<__half>(__half v) { return __half2float(v); }
template <> OSLO_DEVINL float lsf<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> OSLO_DEVINL T lst(float v);
template <> OSLO_DEVINL float lst<float>(float v) { return v; }
template <> OSLO_DEVINL __half lst<__half>(float v) { return __float2half_rn(v); }
template <> OSLO_DEVINL __nv_bfloat16 lst<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// out[t, :] = keep * (emb[ids[t], :] * scale + pos[step + t % seq, :]) / (1 - p), zero for padding tokens.
// One thread handles 8 consecutive features (H % 8 == 0).
template <typename T>
__global__ void ls_embedding_fwd_kernel(const long long* __restrict__ ids, const T* __restrict__ emb, const T* __restrict__ pos,
                                        T* __restrict__ out, long long tokens, int seq, int H, int step, int pad, float scale,
                                        float p, unsigned long long seed, unsigned long long offset) {
  const long long total = tokens * (H / 8);
  const float inv = p > 0.f ? 1.0f / (1.0f - p) : 1.0f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / (H / 8);
    const int c = static_cast<int>(i - t * (H / 8)) * 8;
    const long long tok = ids[t];
    T* o = out + t * H + c;
    if (tok == pad) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = lst<T>(0.f);
      continue;
    }
    const T* e = emb + tok * H + c;
    const T* pp = pos + static_cast<long long>(step + t % seq) * H + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float v = lsf(e[j]) * scale + lsf(pp[j]);
      o[j] = lst<T>(keep_element(seed, offset, t * H + c + j, p) ? v * inv : 0.f);
    }
  }
}

// grad_emb[ids[t], :] += keep * g[t, :] * scale / (1 - p)   (fp32 accumulation buffer, atomics: tokens repeat)
template <typename T>
__global__ void ls_embedding_bwd_kernel(const long long* __restrict__ ids, const T* __restrict__ g, float* __restrict__ grad_emb,
                                        long long tokens, int H, int pad, float scale, float p, unsigned long long seed,
                                        unsigned long long offset) {
  const long long total = tokens * (H / 8);
  const float mul = scale * (p > 0.f ? 1.0f / (1.0f - p) : 1.0f);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / (H / 8);
    const int c = static_cast<int>(i - t * (H / 8)) * 8;
    const long long tok = ids[t];
    if (tok == pad) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (keep_element(seed, offset, t * H + c + j, p)) atomicAdd(grad_emb + tok * H + c + j, lsf(g[t * H + c + j]) * mul);
    }
  }
}

// q = round(clamp(x, -cmax, cmax) * 127 / cmax); clipped[i] = |x| > cmax (optional, for the straight-through gradient)
template <typename T>
__global__ void ls_quantize_kernel(const T* __restrict__ x, int8_t* __restrict__ q, uint8_t* __restrict__ clipped, long long n,
                                   float cmax) {
  const float s = 127.0f / cmax;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = lsf(x[i]);
    const float c = fminf(fmaxf(v, -cmax), cmax);
    q[i] = static_cast<int8_t>(__float2int_rn(c * s));
    if (clipped) clipped[i] = fabsf(v) > cmax ? 1 : 0;
  }
}
template <typename T>
__global__ void ls_dequantize_kernel(const int8_t* __restrict__ q, T* __restrict__ x, long long n, float cmax) {
  const float s = cmax / 127.0f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] = lst<T>(static_cast<float>(q[i]) * s);
}

// ------------------------------------------------------------------------------------------------ sampling
// Order-preserving map of a float to an unsigned key (larger float <-> larger key).
OSLO_DEVINL uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <int THREADS>
OSLO_DEVINL float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < THREADS / 32; ++w) t += red[w];
  return t;
}
template <int THREADS>
OSLO_DEVINL float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = -INFINITY;
  for (int w = 0; w < THREADS / 32; ++w) t = fmaxf(t, red[w]);
  return t;
}

// One CTA per row of logits [V].  The kept set is {i : logit_i >= threshold}; the threshold key is built bit by bit
// (32 counting passes over the row, which stays in L2) so that the set is the top_k largest logits, or, for nucleus
// sampling, the smallest set of largest logits whose probability mass reaches top_p.  A token is then drawn from the
// kept set by inverse CDF (one more pass with a block-wide running sum).  u01: one uniform number per row.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS) ls_sample_kernel(const T* __restrict__ logits, const float* __restrict__ u01,
                                                           long long* __restrict__ out, int V, int top_k, float top_p,
                                                           float inv_temperature) {
  __shared__ float red[THREADS / 32];
  __shared__ float s_scan[THREADS / 32];
  __shared__ int s_pick;
  const T* row = logits + static_cast<long long>(blockIdx.x) * V;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += THREADS) mx = fmaxf(mx, lsf(row[i]) * inv_temperature);
  mx = block_max<THREADS>(mx, red);
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += THREADS) z += __expf(lsf(row[i]) * inv_temperature - mx);
  z = block_sum<THREADS>(z, red);
  // Threshold key: the kept set is {i : key(logit_i) >= key}.  First the largest threshold that still keeps top_k
  // elements; then, inside that set (probabilities renormalised to it, as when the two filters are applied one after the
  // other), the largest threshold whose kept mass still reaches top_p.
  uint32_t key = 0;
  float base = z;  // mass that top_p refers to
  const bool use_k = top_k > 0 && top_k < V;
  const bool use_p = top_p > 0.f && top_p < 1.f;
  for (int phase = 0; phase < 2; ++phase) {
    if ((phase == 0 && !use_k) || (phase == 1 && !use_p)) continue;
    uint32_t k2 = 0;
    float kept_mass = base;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = k2 | (1u << bit);
      float cnt = 0.f, mass = 0.f;
      for (int i = threadIdx.x; i < V; i += THREADS) {
        const float l = lsf(row[i]) * inv_temperature;
        if (float_key(l) >= cand) {
          cnt += 1.f;
          mass += __expf(l - mx);
        }
      }
      cnt = block_sum<THREADS>(cnt, red);
      mass = block_sum<THREADS>(mass, red);
      const bool enough = phase == 0 ? cnt >= static_cast<float>(top_k) : mass >= top_p * base;
      if (enough) {  // the higher threshold still leaves enough candidates / probability mass
        k2 = cand;
        kept_mass = mass;
      }
    }
    key = k2 > key ? k2 : key;
    if (phase == 0) base = kept_mass;
  }
  // mass of the kept set, then inverse CDF
  float kept = 0.f;
  for (int i = threadIdx.x; i < V; i += THREADS) {
    const float l = lsf(row[i]) * inv_temperature;
    if (float_key(l) >= key) kept += __expf(l - mx);
  }
  kept = block_sum<THREADS>(kept, red);
  const float target = u01[blockIdx.x] * kept;
  if (threadIdx.x == 0) s_pick = -1;
  __syncthreads();
  float running = 0.f;  // mass of the kept elements before the current stripe (identical in every thread)
  int last_kept = -1;
  for (int base = 0; base < V; base += THREADS) {
    const int i = base + threadIdx.x;
    float pi = 0.f;
    if (i < V) {
      const float l = lsf(row[i]) * inv_temperature;
      if (float_key(l) >= key) pi = __expf(l - mx);
    }
    // inclusive scan over the block
    float v = pi;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, v, o);
      if ((threadIdx.x & 31) >= o) v += n;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 31) s_scan[threadIdx.x >> 5] = v;
    __syncthreads();
    float before = 0.f, stripe = 0.f;
    for (int w = 0; w < THREADS / 32; ++w) {
      if (w < (threadIdx.x >> 5)) before += s_scan[w];
      stripe += s_scan[w];
    }
    const float incl = running + before + v;
    if (pi > 0.f && incl >= target && incl - pi < target) atomicMax(&s_pick, i);
    if (pi > 0.f) last_kept = i;
    running += stripe;
    __syncthreads();
    if (s_pick >= 0) break;
  }
  // rounding may leave the target a hair above the total: fall back to the last kept element
  __syncthreads();
  if (s_pick < 0) {
    for (int o = 16; o > 0; o >>= 1) last_kept = max(last_kept, __shfl_xor_sync(0xffffffffu, last_kept, o));
    if ((threadIdx.x & 31) == 0 && last_kept >= 0) atomicMax(&s_pick, last_kept);
    __syncthreads();
  }
  if (threadIdx.x == 0) out[blockIdx.x] = s_pick;
}

}  // namespace oslo

#define OSLO_LS_BY_DTYPE(F32, F16, BF16) \
  switch (dtype) {                       \
    case 0: F32; break;                  \
    case 1: F16; break;                  \
    case 2: BF16; break;                 \
    default: return -1;                  \
  }

static int ls_grid(long long work, int num_sms) {
  long long b = (work + 255) / 256;
  const long long cap = static_cast<long long>(num_sms) * 8;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

// ids: [tokens] int64; emb: [vocab, H]; pos: [max_positions, H]; out: [tokens, H].  dtype 0 fp32, 1 fp16, 2 bf16.
extern "C" int oslo_ls_embedding_forward(const long long* ids, const void* emb, const void* pos, void* out, long long tokens,
                                         int seq, int H, int step, int pad, float scale, float p, unsigned long long seed,
                                         unsigned long long offset, int dtype, int num_sms, void* stream) {
  using namespace oslo;
  if (tokens <= 0) return 0;
  if (H % 8 || seq <= 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int g = ls_grid(tokens * (H / 8), num_sms);
  OSLO_LS_BY_DTYPE((ls_embedding_fwd_kernel<float><<<g, 256, 0, st>>>(ids, (const float*)emb, (const float*)pos, (float*)out, tokens, seq, H, step, pad, scale, p, seed, offset)),
                   (ls_embedding_fwd_kernel<__half><<<g, 256, 0, st>>>(ids, (const __half*)emb, (const __half*)pos, (__half*)out, tokens, seq, H, step, pad, scale, p, seed, offset)),
                   (ls_embedding_fwd_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(ids, (const __nv_bfloat16*)emb, (const __nv_bfloat16*)pos, (__nv_bfloat16*)out, tokens, seq, H, step, pad, scale, p, seed, offset)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// grad_emb: fp32 [vocab, H], accumulated into (the caller zeroes it).
extern "C" int oslo_ls_embedding_backward(const long long* ids, const void* g, float* grad_emb, long long tokens, int H, int pad,
                                          float scale, float p, unsigned long long seed, unsigned long long offset, int dtype,
                                          int num_sms, void* stream) {
  using namespace oslo;
  if (tokens <= 0) return 0;
  if (H % 8) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = ls_grid(tokens * (H / 8), num_sms);
  OSLO_LS_BY_DTYPE((ls_embedding_bwd_kernel<float><<<grid, 256, 0, st>>>(ids, (const float*)g, grad_emb, tokens, H, pad, scale, p, seed, offset)),
                   (ls_embedding_bwd_kernel<__half><<<grid, 256, 0, st>>>(ids, (const __half*)g, grad_emb, tokens, H, pad, scale, p, seed, offset)),
                   (ls_embedding_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(ids, (const __nv_bfloat16*)g, grad_emb, tokens, H, pad, scale, p, seed, offset)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_ls_quantize(const void* x, signed char* q, unsigned char* clipped, long long n, float cmax, int dtype,
                                int num_sms, void* stream) {
  using namespace oslo;
  if (n <= 0) return 0;
  if (!(cmax > 0.f)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int g = ls_grid(n, num_sms);
  OSLO_LS_BY_DTYPE((ls_quantize_kernel<float><<<g, 256, 0, st>>>((const float*)x, (int8_t*)q, clipped, n, cmax)),
                   (ls_quantize_kernel<__half><<<g, 256, 0, st>>>((const __half*)x, (int8_t*)q, clipped, n, cmax)),
                   (ls_quantize_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)x, (int8_t*)q, clipped, n, cmax)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_ls_dequantize(const signed char* q, void* x, long long n, float cmax, int dtype, int num_sms, void* stream) {
  using namespace oslo;
  if (n <= 0) return 0;
  if (!(cmax > 0.f)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int g = ls_grid(n, num_sms);
  OSLO_LS_BY_DTYPE((ls_dequantize_kernel<float><<<g, 256, 0, st>>>((const int8_t*)q, (float*)x, n, cmax)),
                   (ls_dequantize_kernel<__half><<<g, 256, 0, st>>>((const int8_t*)q, (__half*)x, n, cmax)),
                   (ls_dequantize_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const int8_t*)q, (__nv_bfloat16*)x, n, cmax)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// logits: [rows, V]; u01: [rows] uniform numbers in [0, 1); out: [rows] int64 token ids.
// top_k <= 0 and top_p >= 1 sample from the full distribution.
extern "C" int oslo_ls_sample(const void* logits, const float* u01, long long* out, int rows, int V, int top_k, float top_p,
                              float temperature, int dtype, void* stream) {
  using namespace oslo;
  if (rows <= 0) return 0;
  if (V <= 0 || !(temperature > 0.f)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float it = 1.0f / temperature;
  OSLO_LS_BY_DTYPE((ls_sample_kernel<float, 512><<<rows, 512, 0, st>>>((const float*)logits, u01, out, V, top_k, top_p, it)),
                   (ls_sample_kernel<__half, 512><<<rows, 512, 0, st>>>((const __half*)logits, u01, out, V, top_k, top_p, it)),
                   (ls_sample_kernel<__nv_bfloat16, 512><<<rows, 512, 0, st>>>((const __nv_bfloat16*)logits, u01, out, V, top_k, top_p, it)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

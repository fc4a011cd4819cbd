// Vocab-parallel cross-entropy for sm_100a.
//
// Each tensor-parallel rank holds logits [rows, V_local] for vocabulary range
// [vocab_start, vocab_start + V_local).  The loss needs three per-row scalars from
// every rank: the local max, the local sum of exp(x - local max) and the target
// logit (if the target falls in this rank's range).  Kernel 1 computes them in ONE
// pass (online softmax).  The exchange gathers `tp` triples per row; kernel 2 reads
// all triples — from a gathered local buffer, or directly from each peer's buffer
// over NVLink — combines them and writes the loss and, in place, the gradient
// (softmax - onehot) * grad_scale.  The reference performs three separate
// all-reduces and materialises an fp32 softmax (oslo/torch/nn/modules/loss.py:14-100).
#include "common.cuh"

namespace oslo {

template <typename T> OSLO_DEVINL float ce_to_f(T v);
template <> OSLO_DEVINL float ce_to_f<float>(float v) { return v; }
template <> OSLO_DEVINL float ce_to_f<__half>(__half v) { return __half2float(v); }
template <> OSLO_DEVINL float ce_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> OSLO_DEVINL T ce_from_f(float v);
template <> OSLO_DEVINL float ce_from_f<float>(float v) { return v; }
template <> OSLO_DEVINL __half ce_from_f<__half>(float v) { return __float2half_rn(v); }
template <> OSLO_DEVINL __nv_bfloat16 ce_from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

constexpr int kCeThreads = 256;

OSLO_DEVINL void online_merge(float& m, float& s, float m2, float s2) {
  const float nm = fmaxf(m, m2);
  if (nm == -INFINITY) { m = nm; s = 0.f; return; }
  s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  m = nm;
}

// stats[row] = (local max, local sum exp(x - max), target logit or 0)
template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_stats_kernel(const T* __restrict__ logits, const long long* __restrict__ target,
                                                             float* __restrict__ stats, int rows, int V, long long ld,
                                                             long long vocab_start, int valid_v) {
  __shared__ float sm_m[kCeThreads / 32], sm_s[kCeThreads / 32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* x = logits + (size_t)row * ld;
    float m = -INFINITY, s = 0.f;
    for (int j = threadIdx.x; j < valid_v; j += kCeThreads) {
      const float v = ce_to_f(x[j]);
      if (v > m) { s = s * __expf(m - v) + 1.0f; m = v; }
      else s += __expf(v - m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_merge(m, s, m2, s2);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { sm_m[threadIdx.x >> 5] = m; sm_s[threadIdx.x >> 5] = s; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < kCeThreads / 32; ++w) online_merge(m, s, sm_m[w], sm_s[w]);
      const long long t = target[row] - vocab_start;
      float tv = 0.f;
      if (t >= 0 && t < valid_v) tv = ce_to_f(x[t]);
      stats[(size_t)row * 3 + 0] = m;
      stats[(size_t)row * 3 + 1] = s;
      stats[(size_t)row * 3 + 2] = tv;
    }
  }
}

struct PeerStats {
  const float* ptr[16];  // per-rank stats buffers ([rows, 3] each); local or peer-mapped
};

// loss[row] = log(sum) + max - x_t  (0 for ignored rows); logits <- (softmax - onehot) * grad_scale[row]
// grad_scale_ptr: optional device scalar multiplied in (e.g. dloss / n_valid).
template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_loss_grad_kernel(T* __restrict__ logits, const long long* __restrict__ target,
                                                                 PeerStats peers, int tp, float* __restrict__ loss,
                                                                 int rows, int V, long long ld, long long vocab_start,
                                                                 int valid_v, long long ignore_index, float grad_scale,
                                                                 const float* __restrict__ grad_scale_ptr, int write_grad) {
  __shared__ float sh[3];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = -INFINITY, s = 0.f, tv = 0.f;
      for (int r = 0; r < tp; ++r) {
        const float* st = peers.ptr[r] + (size_t)row * 3;
        online_merge(m, s, st[0], st[1]);
        tv += st[2];
      }
      const bool ignored = target[row] == ignore_index;
      if (loss) loss[row] = ignored ? 0.f : (__logf(s) + m - tv);
      sh[0] = m;
      sh[1] = 1.0f / s;
      sh[2] = ignored ? 0.f : grad_scale * (grad_scale_ptr ? *grad_scale_ptr : 1.0f);
    }
    __syncthreads();
    if (!write_grad) continue;
    const float m = sh[0], inv = sh[1], gs = sh[2];
    T* x = logits + (size_t)row * ld;
    const long long t = target[row] - vocab_start;
    for (int j = threadIdx.x; j < V; j += kCeThreads) {
      float g = 0.f;
      if (j < valid_v) {
        g = __expf(ce_to_f(x[j]) - m) * inv;
        if (j == t) g -= 1.0f;
        g *= gs;
      }
      x[j] = ce_from_f<T>(g);
    }
  }
}

}  // namespace oslo

using namespace oslo;

// valid_v: number of real (non-padding) vocabulary columns on this rank (<= V).
extern "C" int oslo_ce_stats(const void* logits, const long long* target, float* stats, int rows, int V, long long ld,
                             long long vocab_start, int valid_v, int dtype, int num_sms, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int g = rows < num_sms * 8 ? rows : num_sms * 8;
  if (dtype == 0) ce_stats_kernel<float><<<g, kCeThreads, 0, st>>>((const float*)logits, target, stats, rows, V, ld, vocab_start, valid_v);
  else if (dtype == 1) ce_stats_kernel<__half><<<g, kCeThreads, 0, st>>>((const __half*)logits, target, stats, rows, V, ld, vocab_start, valid_v);
  else ce_stats_kernel<__nv_bfloat16><<<g, kCeThreads, 0, st>>>((const __nv_bfloat16*)logits, target, stats, rows, V, ld, vocab_start, valid_v);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// stats_ptrs: host array of `tp` device pointers (each [rows, 3] fp32).
extern "C" int oslo_ce_loss_grad(void* logits, const long long* target, const void* const* stats_ptrs, int tp, float* loss,
                                 int rows, int V, long long ld, long long vocab_start, int valid_v, long long ignore_index,
                                 float grad_scale, const float* grad_scale_ptr, int write_grad, int dtype, int num_sms,
                                 void* stream) {
  if (rows <= 0) return 0;
  if (tp > 16) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  PeerStats ps;
  for (int i = 0; i < 16; ++i) ps.ptr[i] = i < tp ? static_cast<const float*>(stats_ptrs[i]) : nullptr;
  const int g = rows < num_sms * 8 ? rows : num_sms * 8;
#define OSLO_CE(T) ce_loss_grad_kernel<T><<<g, kCeThreads, 0, st>>>((T*)logits, target, ps, tp, loss, rows, V, ld, vocab_start, valid_v, ignore_index, grad_scale, grad_scale_ptr, write_grad)
  if (dtype == 0) OSLO_CE(float);
  else if (dtype == 1) OSLO_CE(__half);
  else OSLO_CE(__nv_bfloat16);
#undef OSLO_CE
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}


// x[r, :] *= g[r] in place, 16 bytes per thread and step (the cross-entropy backward: the gradient written into the logits
// at forward time is scaled by the upstream per-token gradient).  V % 8 == 0, rows of x are `ld` elements apart.
template <bool BF16>
__global__ void row_scale_kernel(uint16_t* __restrict__ x, const float* __restrict__ g, long long rows, int V, long long ld) {
  const int vec_per_row = V / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;
    const float s = g[r];
    uint4* p = reinterpret_cast<uint4*>(x + r * ld + c);
    uint4 v = *p;
    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (BF16) {
        const float lo = __uint_as_float(w[j] << 16) * s, hi = __uint_as_float(w[j] & 0xffff0000u) * s;
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
        const __half2 o = __floats2half2_rn(__low2float(h) * s, __high2float(h) * s);
        w[j] = *reinterpret_cast<const uint32_t*>(&o);
      }
    }
    *p = v;
  }
}

extern "C" int oslo_row_scale(void* x, const float* g, long long rows, int V, long long ld, int is_bf16, int num_sms, void* stream) {
  if (rows <= 0 || V <= 0) return 0;
  if (V % 8 || ld % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
  const long long total = rows * (V / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 16LL * num_sms) blocks = 16LL * num_sms;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16) row_scale_kernel<true><<<static_cast<int>(blocks), 256, 0, st>>>(static_cast<uint16_t*>(x), g, rows, V, ld);
  else row_scale_kernel<false><<<static_cast<int>(blocks), 256, 0, st>>>(static_cast<uint16_t*>(x), g, rows, V, ld);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Multi-tensor optimizer kernels for sm_100a: Adam/AdamW, SGD, Adagrad, LAMB (two
// stages), NovoGrad, and L2 / max norms with a non-finite flag.
//
// Design: the tensor list lives in a DEVICE table (one record of pointers + numel
// per tensor) plus a block map (block -> tensor, chunk), both built once per
// optimizer and reused every step, so a whole parameter group is ONE launch no
// matter how many tensors it has.  (The reference passes the table by value in the
// kernel arguments and must split a step into launches of <= 36 tensors / 320
// blocks: oslo/torch/_C/csrc/includes/multi_tensor_apply.cuh:15-123.)
// Math is fp32; parameters/gradients may be fp32, fp16 or bf16, with an optional
// fp32 master copy.  A device-side `noop` flag (GradScaler found_inf) skips the update.
//
// Replaces oslo/torch/_C/csrc/multi_tensor_{adam,sgd,adagrad,lamb,lamb_mp,novograd,l2norm,l2norm_mp}.cu
// and lightseq2 csrc/kernels/cuda/fused_adam_kernel.cu.
#include "common.cuh"

namespace oslo {

constexpr int kMTChunk = 16384;   // elements per block
constexpr int kMTThreads = 256;

struct MTRecord {
  long long numel;
  void* ptr[5];  // meaning depends on the functor (p, g, m, v, master ...)
};

template <typename T> OSLO_DEVINL float ldf(const T* p, long long i);
template <> OSLO_DEVINL float ldf<float>(const float* p, long long i) { return p[i]; }
template <> OSLO_DEVINL float ldf<__half>(const __half* p, long long i) { return __half2float(p[i]); }
template <> OSLO_DEVINL float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> OSLO_DEVINL void stf(T* p, long long i, float v);
template <> OSLO_DEVINL void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> OSLO_DEVINL void stf<__half>(__half* p, long long i, float v) { p[i] = __float2half_rn(v); }
template <> OSLO_DEVINL void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale;
  int adamw;           // 1: decoupled weight decay, 0: L2 added to the gradient
  const float* inv_scale;  // optional device scalar multiplied into the gradient (GradScaler)
  const int* step_ptr;     // optional device step counter: bias corrections are then computed in the kernel, so a
                           // captured launch stays correct when replayed from a CUDA graph
};

// ptr: 0 = param (TP), 1 = grad (TG), 2 = exp_avg (f32), 3 = exp_avg_sq (f32), 4 = master (f32, optional)
template <typename TP, typename TG>
__global__ void __launch_bounds__(kMTThreads) mt_adam_kernel(const MTRecord* __restrict__ table, const int2* __restrict__ block_map,
                                                             AdamArgs a, const int* __restrict__ noop) {
  if (noop && *noop) return;
  const int2 bm = block_map[blockIdx.x];
  const MTRecord rec = table[bm.x];
  const long long start = (long long)bm.y * kMTChunk;
  const long long end = min(rec.numel, start + kMTChunk);
  TP* p = static_cast<TP*>(rec.ptr[0]);
  const TG* g = static_cast<const TG*>(rec.ptr[1]);
  float* m = static_cast<float*>(rec.ptr[2]);
  float* v = static_cast<float*>(rec.ptr[3]);
  float* master = static_cast<float*>(rec.ptr[4]);
  const float gs = a.grad_scale * (a.inv_scale ? *a.inv_scale : 1.0f);
  float inv_bc1 = 1.0f / a.bc1, inv_bc2 = 1.0f / a.bc2;
  if (a.step_ptr) {
    const float t = static_cast<float>(*a.step_ptr);
    inv_bc1 = 1.0f / (1.0f - powf(a.beta1, t));
    inv_bc2 = 1.0f / (1.0f - powf(a.beta2, t));
  }
  for (long long i = start + threadIdx.x; i < end; i += kMTThreads) {
    float pv = master ? master[i] : ldf<TP>(p, i);
    float gv = ldf<TG>(g, i) * gs;
    if (!a.adamw) gv += a.weight_decay * pv;
    const float mv = a.beta1 * m[i] + (1.0f - a.beta1) * gv;
    const float vv = a.beta2 * v[i] + (1.0f - a.beta2) * gv * gv;
    m[i] = mv;
    v[i] = vv;
    float upd = (mv * inv_bc1) / (sqrtf(vv * inv_bc2) + a.eps);
    if (a.adamw) upd += a.weight_decay * pv;
    pv -= a.lr * upd;
    if (master) master[i] = pv;
    stf<TP>(p, i, pv);
  }
}

struct SgdArgs {
  float lr, momentum, dampening, weight_decay, grad_scale;
  int nesterov, first_run, wd_after_momentum;
};
// ptr: 0 = param, 1 = grad, 2 = momentum buffer (f32), 4 = master (optional)
template <typename TP, typename TG>
__global__ void __launch_bounds__(kMTThreads) mt_sgd_kernel(const MTRecord* __restrict__ table, const int2* __restrict__ block_map,
                                                            SgdArgs a, const int* __restrict__ noop) {
  if (noop && *noop) return;
  const int2 bm = block_map[blockIdx.x];
  const MTRecord rec = table[bm.x];
  const long long start = (long long)bm.y * kMTChunk;
  const long long end = min(rec.numel, start + kMTChunk);
  TP* p = static_cast<TP*>(rec.ptr[0]);
  const TG* g = static_cast<const TG*>(rec.ptr[1]);
  float* buf = static_cast<float*>(rec.ptr[2]);
  float* master = static_cast<float*>(rec.ptr[4]);
  for (long long i = start + threadIdx.x; i < end; i += kMTThreads) {
    float pv = master ? master[i] : ldf<TP>(p, i);
    float gv = ldf<TG>(g, i) * a.grad_scale;
    if (a.weight_decay != 0.f && !a.wd_after_momentum) gv += a.weight_decay * pv;
    if (a.momentum != 0.f) {
      float b = a.first_run ? gv : a.momentum * buf[i] + (1.0f - a.dampening) * gv;
      buf[i] = b;
      gv = a.nesterov ? gv + a.momentum * b : b;
    }
    if (a.weight_decay != 0.f && a.wd_after_momentum) gv += a.weight_decay * pv;
    pv -= a.lr * gv;
    if (master) master[i] = pv;
    stf<TP>(p, i, pv);
  }
}

struct AdagradArgs {
  float lr, eps, weight_decay;
  int adagrad_w;
};
// ptr: 0 = param, 1 = grad, 2 = state sum (f32)
template <typename TP, typename TG>
__global__ void __launch_bounds__(kMTThreads) mt_adagrad_kernel(const MTRecord* __restrict__ table,
                                                                const int2* __restrict__ block_map, AdagradArgs a,
                                                                const int* __restrict__ noop) {
  if (noop && *noop) return;
  const int2 bm = block_map[blockIdx.x];
  const MTRecord rec = table[bm.x];
  const long long start = (long long)bm.y * kMTChunk;
  const long long end = min(rec.numel, start + kMTChunk);
  TP* p = static_cast<TP*>(rec.ptr[0]);
  const TG* g = static_cast<const TG*>(rec.ptr[1]);
  float* h = static_cast<float*>(rec.ptr[2]);
  for (long long i = start + threadIdx.x; i < end; i += kMTThreads) {
    float pv = ldf<TP>(p, i);
    float gv = ldf<TG>(g, i);
    if (!a.adagrad_w) gv += a.weight_decay * pv;
    const float hv = h[i] + gv * gv;
    h[i] = hv;
    float upd = gv / (sqrtf(hv) + a.eps);
    if (a.adagrad_w) upd += a.weight_decay * pv;
    stf<TP>(p, i, pv - a.lr * upd);
  }
}

// Sum of squares (or max |x|) per tensor and globally.  out_global[0] accumulates; out_per_tensor[t] too.
// flag is set to 1 when a non-finite value is seen.  ptr index `which` selects the tensor of the record.
template <typename T>
__global__ void __launch_bounds__(kMTThreads) mt_norm_kernel(const MTRecord* __restrict__ table, const int2* __restrict__ block_map,
                                                             int which, float* __restrict__ out_global,
                                                             float* __restrict__ out_per_tensor, int* __restrict__ flag,
                                                             int max_norm) {
  __shared__ float scratch[kMTThreads / 32];
  const int2 bm = block_map[blockIdx.x];
  const MTRecord rec = table[bm.x];
  const long long start = (long long)bm.y * kMTChunk;
  const long long end = min(rec.numel, start + kMTChunk);
  const T* x = static_cast<const T*>(rec.ptr[which]);
  float acc = 0.f;
  bool bad = false;
  for (long long i = start + threadIdx.x; i < end; i += kMTThreads) {
    const float v = ldf<T>(x, i);
    if (!isfinite(v)) bad = true;
    acc = max_norm ? fmaxf(acc, fabsf(v)) : acc + v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, acc, o);
    acc = max_norm ? fmaxf(acc, other) : acc + other;
  }
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = acc;
  if (bad && flag) *flag = 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = scratch[0];
    for (int w = 1; w < kMTThreads / 32; ++w) t = max_norm ? fmaxf(t, scratch[w]) : t + scratch[w];
    if (max_norm) {
      // values are non-negative: integer compare of the bit pattern orders them
      if (out_global) atomicMax(reinterpret_cast<int*>(out_global), __float_as_int(t));
      if (out_per_tensor) atomicMax(reinterpret_cast<int*>(out_per_tensor + bm.x), __float_as_int(t));
    } else {
      if (out_global) atomicAdd(out_global, t);
      if (out_per_tensor) atomicAdd(out_per_tensor + bm.x, t);
    }
  }
}

struct LambArgs {
  float lr, beta1, beta2, beta3, eps, weight_decay, bc1, bc2, max_grad_norm;
  int adamw, use_nvlamb;
  const float* global_grad_sumsq;  // device scalar: sum of squares of all grads
  const float* inv_scale;          // optional GradScaler inverse scale
};
// Stage 1: moments + raw update u written OVER the gradient slot of a scratch ("update") tensor.
// ptr: 0 = param, 1 = grad, 2 = m, 3 = v, 4 = update (f32, same numel)
template <typename TP, typename TG>
__global__ void __launch_bounds__(kMTThreads) mt_lamb_stage1_kernel(const MTRecord* __restrict__ table,
                                                                    const int2* __restrict__ block_map, LambArgs a,
                                                                    const int* __restrict__ noop) {
  if (noop && *noop) return;
  const int2 bm = block_map[blockIdx.x];
  const MTRecord rec = table[bm.x];
  const long long start = (long long)bm.y * kMTChunk;
  const long long end = min(rec.numel, start + kMTChunk);
  const TP* p = static_cast<const TP*>(rec.ptr[0]);
  const TG* g = static_cast<const TG*>(rec.ptr[1]);
  float* m = static_cast<float*>(rec.ptr[2]);
  float* v = static_cast<float*>(rec.ptr[3]);
  float* u = static_cast<float*>(rec.ptr[4]);
  float gnorm = sqrtf(*a.global_grad_sumsq);
  if (a.inv_scale) gnorm *= *a.inv_scale;
  const float clip = (a.max_grad_norm > 0.f && gnorm > a.max_grad_norm) ? gnorm / a.max_grad_norm : 1.0f;
  const float gs = (a.inv_scale ? *a.inv_scale : 1.0f) / clip;
  for (long long i = start + threadIdx.x; i < end; i += kMTThreads) {
    const float pv = ldf<TP>(p, i);
    float gv = ldf<TG>(g, i) * gs;
    if (!a.adamw) gv += a.weight_decay * pv;
    const float mv = a.beta1 * m[i] + a.beta3 * gv;
    const float vv = a.beta2 * v[i] + (1.0f - a.beta2) * gv * gv;
    m[i] = mv;
    v[i] = vv;
    float upd = (mv / a.bc1) / (sqrtf(vv / a.bc2) + a.eps);
    if (a.adamw) upd += a.weight_decay * pv;
    u[i] = upd;
  }
}
// Stage 2: p -= lr * ratio * u with ratio = ||p|| / ||u|| per tensor (1 when either is 0, or when
// weight decay is 0 and nvlamb is off).  ptr: 0 = param, 4 = update, [optional] 3 reused as master (f32).
template <typename TP>
__global__ void __launch_bounds__(kMTThreads) mt_lamb_stage2_kernel(const MTRecord* __restrict__ table,
                                                                    const int2* __restrict__ block_map, LambArgs a,
                                                                    const float* __restrict__ p_sumsq,
                                                                    const float* __restrict__ u_sumsq,
                                                                    const int* __restrict__ noop, int has_master_in_slot1) {
  if (noop && *noop) return;
  const int2 bm = block_map[blockIdx.x];
  const MTRecord rec = table[bm.x];
  const long long start = (long long)bm.y * kMTChunk;
  const long long end = min(rec.numel, start + kMTChunk);
  TP* p = static_cast<TP*>(rec.ptr[0]);
  const float* u = static_cast<const float*>(rec.ptr[4]);
  float ratio = 1.0f;
  if (a.use_nvlamb || a.weight_decay != 0.f) {
    const float pn = sqrtf(p_sumsq[bm.x]), un = sqrtf(u_sumsq[bm.x]);
    if (pn > 0.f && un > 0.f) ratio = pn / un;
  }
  const float step = a.lr * ratio;
  for (long long i = start + threadIdx.x; i < end; i += kMTThreads) stf<TP>(p, i, ldf<TP>(p, i) - step * u[i]);
}

struct NovoArgs {
  float lr, beta1, beta2, beta3, eps, weight_decay, bc1, bc2;
  int adamw;
  const float* second_moment;  // [num_tensors] blended per-tensor grad norms (already updated)
};
// ptr: 0 = param, 1 = grad, 2 = m
template <typename TP, typename TG>
__global__ void __launch_bounds__(kMTThreads) mt_novograd_kernel(const MTRecord* __restrict__ table,
                                                                 const int2* __restrict__ block_map, NovoArgs a,
                                                                 const int* __restrict__ noop) {
  if (noop && *noop) return;
  const int2 bm = block_map[blockIdx.x];
  const MTRecord rec = table[bm.x];
  const long long start = (long long)bm.y * kMTChunk;
  const long long end = min(rec.numel, start + kMTChunk);
  TP* p = static_cast<TP*>(rec.ptr[0]);
  const TG* g = static_cast<const TG*>(rec.ptr[1]);
  float* m = static_cast<float*>(rec.ptr[2]);
  const float denom = a.second_moment[bm.x] / a.bc2 + a.eps;
  for (long long i = start + threadIdx.x; i < end; i += kMTThreads) {
    const float pv = ldf<TP>(p, i);
    float gv = ldf<TG>(g, i) / denom;
    if (!a.adamw) gv += a.weight_decay * pv;  // L2 mode folds decay into the normalised gradient
    else gv += a.weight_decay * pv;
    const float mv = a.beta1 * m[i] + a.beta3 * gv;
    m[i] = mv;
    stf<TP>(p, i, pv - a.lr * (mv / a.bc1));
  }
}

// out[i] = in[i] * scale (dtype conversion allowed); used for unscale / cast of flat buffers.
template <typename TI, typename TO>
__global__ void scale_cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n, float scale,
                                  const float* __restrict__ dev_scale) {
  const float s = scale * (dev_scale ? *dev_scale : 1.0f);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    stf<TO>(out, i, ldf<TI>(in, i) * s);
}

}  // namespace oslo

using namespace oslo;

#define OSLO_PG_DISPATCH(KERNEL, ...)                                                                       \
  do {                                                                                                      \
    if (pdtype == 0 && gdtype == 0) KERNEL<float, float><<<nblocks, kMTThreads, 0, st>>>(__VA_ARGS__);       \
    else if (pdtype == 1 && gdtype == 1) KERNEL<__half, __half><<<nblocks, kMTThreads, 0, st>>>(__VA_ARGS__); \
    else if (pdtype == 2 && gdtype == 2) KERNEL<__nv_bfloat16, __nv_bfloat16><<<nblocks, kMTThreads, 0, st>>>(__VA_ARGS__); \
    else if (pdtype == 0 && gdtype == 1) KERNEL<float, __half><<<nblocks, kMTThreads, 0, st>>>(__VA_ARGS__);  \
    else if (pdtype == 0 && gdtype == 2) KERNEL<float, __nv_bfloat16><<<nblocks, kMTThreads, 0, st>>>(__VA_ARGS__); \
    else if (pdtype == 1 && gdtype == 0) KERNEL<__half, float><<<nblocks, kMTThreads, 0, st>>>(__VA_ARGS__);  \
    else if (pdtype == 2 && gdtype == 0) KERNEL<__nv_bfloat16, float><<<nblocks, kMTThreads, 0, st>>>(__VA_ARGS__); \
    else return -1;                                                                                         \
  } while (0)

extern "C" int oslo_mt_chunk() { return kMTChunk; }
extern "C" int oslo_mt_record_bytes() { return (int)sizeof(MTRecord); }

extern "C" int oslo_mt_adam(const void* table, const void* block_map, int nblocks, float lr, float beta1, float beta2, float eps,
                            float weight_decay, float bc1, float bc2, float grad_scale, int adamw, const float* inv_scale,
                            const int* noop, int pdtype, int gdtype, void* stream, const int* step_ptr) {
  if (nblocks <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale, adamw, inv_scale, step_ptr};
  OSLO_PG_DISPATCH(mt_adam_kernel, (const MTRecord*)table, (const int2*)block_map, a, noop);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_mt_sgd(const void* table, const void* block_map, int nblocks, float lr, float momentum, float dampening,
                           float weight_decay, float grad_scale, int nesterov, int first_run, int wd_after_momentum,
                           const int* noop, int pdtype, int gdtype, void* stream) {
  if (nblocks <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  SgdArgs a{lr, momentum, dampening, weight_decay, grad_scale, nesterov, first_run, wd_after_momentum};
  OSLO_PG_DISPATCH(mt_sgd_kernel, (const MTRecord*)table, (const int2*)block_map, a, noop);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_mt_adagrad(const void* table, const void* block_map, int nblocks, float lr, float eps, float weight_decay,
                               int adagrad_w, const int* noop, int pdtype, int gdtype, void* stream) {
  if (nblocks <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  AdagradArgs a{lr, eps, weight_decay, adagrad_w};
  OSLO_PG_DISPATCH(mt_adagrad_kernel, (const MTRecord*)table, (const int2*)block_map, a, noop);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Accumulates into out_global / out_per_tensor (caller zeroes them).  max_norm != 0: L-inf norm.
extern "C" int oslo_mt_norm(const void* table, const void* block_map, int nblocks, int which, float* out_global,
                            float* out_per_tensor, int* flag, int max_norm, int dtype, void* stream) {
  if (nblocks <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == 0) mt_norm_kernel<float><<<nblocks, kMTThreads, 0, st>>>((const MTRecord*)table, (const int2*)block_map, which, out_global, out_per_tensor, flag, max_norm);
  else if (dtype == 1) mt_norm_kernel<__half><<<nblocks, kMTThreads, 0, st>>>((const MTRecord*)table, (const int2*)block_map, which, out_global, out_per_tensor, flag, max_norm);
  else mt_norm_kernel<__nv_bfloat16><<<nblocks, kMTThreads, 0, st>>>((const MTRecord*)table, (const int2*)block_map, which, out_global, out_per_tensor, flag, max_norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_mt_lamb_stage1(const void* table, const void* block_map, int nblocks, float lr, float beta1, float beta2,
                                   float beta3, float eps, float weight_decay, float bc1, float bc2, float max_grad_norm,
                                   int adamw, int use_nvlamb, const float* global_grad_sumsq, const float* inv_scale,
                                   const int* noop, int pdtype, int gdtype, void* stream) {
  if (nblocks <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  LambArgs a{lr, beta1, beta2, beta3, eps, weight_decay, bc1, bc2, max_grad_norm, adamw, use_nvlamb, global_grad_sumsq, inv_scale};
  OSLO_PG_DISPATCH(mt_lamb_stage1_kernel, (const MTRecord*)table, (const int2*)block_map, a, noop);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_mt_lamb_stage2(const void* table, const void* block_map, int nblocks, float lr, float weight_decay,
                                   int use_nvlamb, const float* p_sumsq, const float* u_sumsq, const int* noop, int pdtype,
                                   void* stream) {
  if (nblocks <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  LambArgs a{};
  a.lr = lr; a.weight_decay = weight_decay; a.use_nvlamb = use_nvlamb;
  if (pdtype == 0) mt_lamb_stage2_kernel<float><<<nblocks, kMTThreads, 0, st>>>((const MTRecord*)table, (const int2*)block_map, a, p_sumsq, u_sumsq, noop, 0);
  else if (pdtype == 1) mt_lamb_stage2_kernel<__half><<<nblocks, kMTThreads, 0, st>>>((const MTRecord*)table, (const int2*)block_map, a, p_sumsq, u_sumsq, noop, 0);
  else mt_lamb_stage2_kernel<__nv_bfloat16><<<nblocks, kMTThreads, 0, st>>>((const MTRecord*)table, (const int2*)block_map, a, p_sumsq, u_sumsq, noop, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_mt_novograd(const void* table, const void* block_map, int nblocks, float lr, float beta1, float beta2,
                                float beta3, float eps, float weight_decay, float bc1, float bc2, int adamw,
                                const float* second_moment, const int* noop, int pdtype, int gdtype, void* stream) {
  if (nblocks <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  NovoArgs a{lr, beta1, beta2, beta3, eps, weight_decay, bc1, bc2, adamw, second_moment};
  OSLO_PG_DISPATCH(mt_novograd_kernel, (const MTRecord*)table, (const int2*)block_map, a, noop);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// dtype codes 0 fp32 / 1 fp16 / 2 bf16 for in and out.
extern "C" int oslo_scale_cast(const void* in, void* out, long long n, float scale, const float* dev_scale, int in_dtype,
                               int out_dtype, int num_sms, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  long long blocks = (n + 1023) / 1024;
  const int g = (int)(blocks < (long long)num_sms * 8 ? blocks : (long long)num_sms * 8);
#define OSLO_SC(TI, TO) scale_cast_kernel<TI, TO><<<g, 256, 0, st>>>((const TI*)in, (TO*)out, n, scale, dev_scale)
  switch (in_dtype * 3 + out_dtype) {
    case 0: OSLO_SC(float, float); break;
    case 1: OSLO_SC(float, __half); break;
    case 2: OSLO_SC(float, __nv_bfloat16); break;
    case 3: OSLO_SC(__half, float); break;
    case 4: OSLO_SC(__half, __half); break;
    case 5: OSLO_SC(__half, __nv_bfloat16); break;
    case 6: OSLO_SC(__nv_bfloat16, float); break;
    case 7: OSLO_SC(__nv_bfloat16, __half); break;
    case 8: OSLO_SC(__nv_bfloat16, __nv_bfloat16); break;
    default: return -1;
  }
#undef OSLO_SC
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ZeRO step as ONE kernel over NVLink peer memory:
//
//     reduce-scatter(gradients)  ->  cast / scale / clip  ->  AdamW on the fp32 master shard  ->  all-gather(parameters)
//
// Every rank's flat gradient buffer and flat parameter buffer live in symmetric memory.  The rank that owns elements
// [shard_start, shard_start + shard_len) PULLS those elements of every peer's gradient buffer (16-byte loads, tp of
// them in flight per thread), sums them in fp32, applies the optimizer update to its master copy and moments, and
// PUSHES the new low-precision parameters into every peer's parameter buffer with 16-byte stores.  A device-side
// barrier before (gradients final everywhere) and after (parameters landed everywhere) brackets the kernel.
//
// mode 0: only the squared norm of the reduced shard is accumulated (for global-norm clipping);
// mode 1: pull + update + push, with an optional device scalar multiplying the gradient (the clip coefficient);
// mode 2: pull once, keep the reduced, scaled fp32 gradients of the shard in `reduced` and accumulate their squared norm
//         (launched per bucket while backward is still running);
// mode 3: update from `reduced` (no second pull) with the clip coefficient, then push.
// A clip coefficient that is not finite (the global norm overflowed) makes modes 1 and 3 return without touching
// parameters or moments: the step is skipped on every rank, with no host round trip.
//
// Replaces the reference's bucket reduce + per-owner broadcasts + separate optimizer kernels
// (oslo/torch/nn/parallel/data_parallel/zero/optim/optim.py:354-634).
#include "common.cuh"

namespace oslo {

struct ZeroPeers {
  const void* grad[8];
  void* param[8];
};

struct ZeroArgs {
  float lr, beta1, beta2, eps, weight_decay, inv_bc1, inv_sqrt_bc2, grad_scale;
  int adamw, mode, world, is_bf16;
  const float* clip_coef;  // optional device scalar
  float* sumsq_out;        // optional: += sum of squares of the reduced, scaled shard
  float* reduced;          // modes 2 / 3: fp32 reduced gradients of this shard
};

OSLO_DEVINL void unpack8(const uint4& raw, bool bf16, float* f) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (bf16) { f[2 * j] = __uint_as_float(w[j] << 16); f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u); }
    else { const __half2 h = *reinterpret_cast<const __half2*>(&w[j]); f[2 * j] = __low2float(h); f[2 * j + 1] = __high2float(h); }
  }
}
OSLO_DEVINL uint4 pack8(const float* f, bool bf16) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (bf16) { const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]); w[j] = *reinterpret_cast<const uint32_t*>(&h); }
    else { const __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]); w[j] = *reinterpret_cast<const uint32_t*>(&h); }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// shard_start / shard_len in elements, both multiples of 8.
__global__ void __launch_bounds__(256) zero_step_kernel(ZeroPeers peers, float* __restrict__ master, float* __restrict__ m,
                                                       float* __restrict__ v, long long shard_start, long long shard_len,
                                                       ZeroArgs a) {
  __shared__ float red[8];
  const long long nvec = shard_len / 8;
  const bool bf16 = a.is_bf16 != 0;
  const bool updating = a.mode == 1 || a.mode == 3;
  const float coef = (updating && a.clip_coef) ? *a.clip_coef : 1.0f;
  if (updating && !(fabsf(coef) <= 3.0e38f)) return;  // NaN or infinity: skip this step
  const float gs = a.mode == 3 ? coef : a.grad_scale * coef;
  float local_sq = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long e0 = shard_start + i * 8;
    const long long off = i * 8;
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (a.mode == 3) {
      const float4 lo = *reinterpret_cast<const float4*>(a.reduced + off);
      const float4 hi = *reinterpret_cast<const float4*>(a.reduced + off + 4);
      g[0] = lo.x; g[1] = lo.y; g[2] = lo.z; g[3] = lo.w; g[4] = hi.x; g[5] = hi.y; g[6] = hi.z; g[7] = hi.w;
    } else {
      uint4 raw[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < a.world) raw[r] = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(peers.grad[r]) + e0);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < a.world) {
          float f[8];
          unpack8(raw[r], bf16, f);
#pragma unroll
          for (int j = 0; j < 8; ++j) g[j] += f[j];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      g[j] *= gs;
      local_sq += g[j] * g[j];
    }
    if (a.mode == 0) continue;
    if (a.mode == 2) {
      *reinterpret_cast<float4*>(a.reduced + off) = make_float4(g[0], g[1], g[2], g[3]);
      *reinterpret_cast<float4*>(a.reduced + off + 4) = make_float4(g[4], g[5], g[6], g[7]);
      continue;
    }
    float pnew[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float pv = master[off + j];
      float gv = g[j];
      if (!a.adamw) gv += a.weight_decay * pv;
      const float mv = a.beta1 * m[off + j] + (1.f - a.beta1) * gv;
      const float vv = a.beta2 * v[off + j] + (1.f - a.beta2) * gv * gv;
      m[off + j] = mv;
      v[off + j] = vv;
      float upd = (mv * a.inv_bc1) / (sqrtf(vv) * a.inv_sqrt_bc2 + a.eps);
      if (a.adamw) upd += a.weight_decay * pv;
      pv -= a.lr * upd;
      master[off + j] = pv;
      pnew[j] = pv;
    }
    const uint4 out = pack8(pnew, bf16);
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < a.world) *reinterpret_cast<uint4*>(static_cast<uint16_t*>(peers.param[r]) + e0) = out;
  }
  if (a.sumsq_out) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local_sq += __shfl_xor_sync(0xffffffffu, local_sq, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local_sq;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < 8; ++w) t += red[w];
      atomicAdd(a.sumsq_out, t);
    }
  }
  __threadfence_system();
}

}  // namespace oslo

// peer_grads / peer_params: host arrays of `world` device pointers to the flat 16-bit buffers.
extern "C" int oslo_zero_step(void* const* peer_grads, void* const* peer_params, float* master, float* m, float* v,
                              long long shard_start, long long shard_len, int world, int is_bf16, float lr, float beta1,
                              float beta2, float eps, float weight_decay, float bc1, float bc2, float grad_scale, int adamw,
                              int mode, const float* clip_coef, float* sumsq_out, int num_sms, void* stream,
                              float* reduced) {
  using namespace oslo;
  if (shard_len <= 0) return 0;
  if (world > 8 || shard_start % 8 || shard_len % 8) return -1;
  if ((mode == 2 || mode == 3) && (reduced == nullptr || (reinterpret_cast<uintptr_t>(reduced) & 15))) return -1;
  ZeroPeers peers;
  for (int i = 0; i < 8; ++i) {
    peers.grad[i] = i < world ? peer_grads[i] : nullptr;
    peers.param[i] = i < world ? peer_params[i] : nullptr;
  }
  ZeroArgs a{lr, beta1, beta2, eps, weight_decay, 1.f / bc1, 1.f / sqrtf(bc2), grad_scale, adamw, mode, world, is_bf16, clip_coef, sumsq_out, reduced};
  long long blocks = (shard_len / 8 + 255) / 256;
  const long long cap = (long long)num_sms * 8;
  if (blocks > cap) blocks = cap;
  zero_step_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(peers, master, m, v, shard_start, shard_len, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

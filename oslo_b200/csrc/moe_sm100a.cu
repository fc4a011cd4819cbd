// Mixture-of-experts routing kernels for sm_100a: index-based dispatch / combine and the per-expert
// position scan.  Tokens are moved by ROW INDEX (a gather of h-wide rows), never through the dense
// one-hot [tokens, experts, capacity] einsums of GShard that the reference layers use
// (oslo/torch/nn/parallel/expert_parallel/layers.py:506-509,604-608).
//
//   positions   pos[s, k] = number of earlier (token, choice) pairs routed to the same expert (rank inside the
//               expert's capacity buffer); one block per expert scans the tokens in order, first choices before
//               second choices, as GShard does.
//   dispatch    buf[slot[s, k]] = x[s]            for every kept (s, k)          (slot = expert * C + pos, or -1)
//   combine     y[s] = sum_k w[s, k] * buf[slot[s, k]]
//   and their backward passes.  With peer-mapped destination pointers the same dispatch kernel writes straight
//   into other GPUs' expert buffers (the all-to-all is then the store itself).
//
// Replaces oslo/torch/_C/csrc/expert_parallel_cuda_kernel.cu:283-558 (fp32 / fp16 only, default stream).
#include "common.cuh"

namespace oslo {

constexpr int kScanThreads = 1024;

// expert_idx: [S, K] int32 (expert chosen as k-th choice, or -1).  pos: [S, K] int32 out.  counts: [E] out.
__global__ void __launch_bounds__(kScanThreads) moe_positions_kernel(const int* __restrict__ expert_idx, int* __restrict__ pos,
                                                                    int* __restrict__ counts, int S, int K) {
  __shared__ int warp_sums[kScanThreads / 32];
  __shared__ int carry;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int k = 0; k < K; ++k) {
    for (int base = 0; base < S; base += kScanThreads) {
      const int s = base + threadIdx.x;
      const int hit = (s < S && expert_idx[s * K + k] == e) ? 1 : 0;
      int incl = hit;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (lane == 31) warp_sums[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        int w = warp_sums[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, w, o);
          if (lane >= o) w += v;
        }
        warp_sums[lane] = w;
      }
      __syncthreads();
      const int before = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - hit;
      if (hit) pos[s * K + k] = before;
      __syncthreads();
      if (threadIdx.x == kScanThreads - 1) carry += warp_sums[kScanThreads / 32 - 1];
      __syncthreads();
    }
  }
  if (threadIdx.x == 0) counts[e] = carry;
}

struct DestPtrs {
  void* p[8];  // destination buffer per expert-parallel rank (peer-mapped), or all equal for a local buffer
};

// One block per token.  slot: [S, K] (global slot = expert * C + pos, -1 = dropped).  With ep_size > 1 the slot's
// expert selects the destination rank (expert / experts_per_rank) and the row lands in that rank's buffer laid
// out [local expert][source rank][C] — the layout an all-to-all of [E, C, H] buffers would produce.
template <typename T>
__global__ void moe_dispatch_kernel(const T* __restrict__ x, DestPtrs dst, const int* __restrict__ slot, int S, int K, int H,
                                    int ep_size, int src_rank, int experts_per_rank, int C) {
  const int s = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(s) * H);
  const int nvec = H * sizeof(T) / 16;
  for (int k = 0; k < K; ++k) {
    const int sl = slot[s * K + k];
    if (sl < 0) continue;
    T* base;
    size_t row;
    if (ep_size > 1) {
      const int e = sl / C, c = sl - e * C;
      const int dest = e / experts_per_rank, le = e - dest * experts_per_rank;
      base = static_cast<T*>(dst.p[dest]);
      row = (static_cast<size_t>(le) * ep_size + src_rank) * C + c;  // [local expert][source rank][C]
    } else {
      base = static_cast<T*>(dst.p[0]);
      row = sl;
    }
    uint4* out = reinterpret_cast<uint4*>(base + row * H);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) out[v] = src[v];
  }
}

// The same dispatch seen from the destination side: one block per (expert, position) slot of THIS source; `inv` holds the
// token that owns the slot or -1.  Unowned slots are written as zeros, so the destination needs no clearing pass (and no
// barrier between that pass and the arrival of remote rows): every row of the [local expert][source][C] block that this
// source owns is written exactly once per call.
template <typename T>
__global__ void moe_dispatch_rows_kernel(const T* __restrict__ x, DestPtrs dst, const int* __restrict__ inv, int E, int H, int ep_size,
                                         int src_rank, int experts_per_rank, int C) {
  const int sl = blockIdx.x;  // e * C + c
  const int e = sl / C, c = sl - e * C;
  const int dest = e / experts_per_rank, le = e - dest * experts_per_rank;
  const size_t row = (static_cast<size_t>(le) * ep_size + src_rank) * C + c;
  uint4* out = reinterpret_cast<uint4*>(static_cast<T*>(dst.p[dest]) + row * H);
  const int nvec = H * sizeof(T) / 16;
  const int tok = inv[sl];
  if (tok >= 0) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(tok) * H);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) out[v] = src[v];
  } else {
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) out[v] = z;
  }
}

// y[s] = sum_k w[s,k] * buf[slot[s,k]]
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ buf, const float* __restrict__ w, const int* __restrict__ slot,
                                   T* __restrict__ y, int S, int K, int H) {
  const int s = blockIdx.x;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < K; ++k) {
      const int sl = slot[s * K + k];
      if (sl < 0) continue;
      const float wk = w[s * K + k];
      const T* row = buf + static_cast<size_t>(sl) * H + c;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += wk * static_cast<float>(row[j]);
    }
    T* out = y + static_cast<size_t>(s) * H + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = static_cast<T>(acc[j]);
  }
}

// dbuf[slot[s,k]] = w[s,k] * dy[s];  dw[s,k] = <dy[s], buf[slot[s,k]]>.  dbuf rows of unused slots must be zeroed
// by the caller.
template <typename T>
__global__ void moe_combine_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ buf, const float* __restrict__ w,
                                       const int* __restrict__ slot, T* __restrict__ dbuf, float* __restrict__ dw, int S,
                                       int K, int H) {
  __shared__ float red[32];
  const int s = blockIdx.x;
  for (int k = 0; k < K; ++k) {
    const int sl = slot[s * K + k];
    if (sl < 0) {
      if (threadIdx.x == 0) dw[s * K + k] = 0.f;
      continue;
    }
    const float wk = w[s * K + k];
    float dot = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      const float g = static_cast<float>(dy[static_cast<size_t>(s) * H + c]);
      dot += g * static_cast<float>(buf[static_cast<size_t>(sl) * H + c]);
      dbuf[static_cast<size_t>(sl) * H + c] = static_cast<T>(wk * g);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < (blockDim.x + 31) / 32; ++i) t += red[i];
      dw[s * K + k] = t;
    }
  }
}

// dx[s] = sum_k dbuf[slot[s,k]]  (backward of dispatch)
template <typename T>
__global__ void moe_dispatch_bwd_kernel(const T* __restrict__ dbuf, const int* __restrict__ slot, T* __restrict__ dx, int S,
                                        int K, int H) {
  const int s = blockIdx.x;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < K; ++k) {
      const int sl = slot[s * K + k];
      if (sl >= 0) acc += static_cast<float>(dbuf[static_cast<size_t>(sl) * H + c]);
    }
    dx[static_cast<size_t>(s) * H + c] = static_cast<T>(acc);
  }
}

// ---- peer-memory variants: the all-to-all of the expert buffers is done by the gather / scatter itself ----
// Expert buffers live in symmetric memory on their owner, laid out [local expert][source rank][C]; slot = expert * C +
// position as above.  `pull`: y[s] = sum_k w[s,k] * buffer_of_owner[row]  (combine forward; dispatch backward with w = 1).
struct SrcPtrs {
  const void* p[8];
};
OSLO_DEVINL size_t peer_row(int sl, int C, int experts_per_rank, int ep_size, int src_rank, int& owner) {
  const int e = sl / C, c = sl - e * C;
  owner = e / experts_per_rank;
  const int le = e - owner * experts_per_rank;
  return (static_cast<size_t>(le) * ep_size + src_rank) * C + c;
}

template <typename T>
__global__ void moe_pull_kernel(SrcPtrs src, const float* __restrict__ w, const int* __restrict__ slot, T* __restrict__ y, int S,
                                int K, int H, int ep_size, int my_rank, int experts_per_rank, int C) {
  const int s = blockIdx.x;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < K; ++k) {
      const int sl = slot[s * K + k];
      if (sl < 0) continue;
      int owner;
      const size_t row = peer_row(sl, C, experts_per_rank, ep_size, my_rank, owner);
      const float wk = w ? w[s * K + k] : 1.0f;
      const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const T*>(src.p[owner]) + row * H + c);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += wk * static_cast<float>(v[j]);
    }
    T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = static_cast<T>(acc[j]);
    *reinterpret_cast<uint4*>(y + static_cast<size_t>(s) * H + c) = *reinterpret_cast<const uint4*>(o);
  }
}

// `push scaled` (combine backward): grad_buffer_of_owner[row] = w[s,k] * dy[s]  and  dw[s,k] = <dy[s], buffer_of_owner[row]>.
template <typename T>
__global__ void moe_push_scaled_kernel(const T* __restrict__ dy, DestPtrs gdst, SrcPtrs xsrc, const float* __restrict__ w,
                                       const int* __restrict__ slot, float* __restrict__ dw, int S, int K, int H, int ep_size,
                                       int my_rank, int experts_per_rank, int C) {
  __shared__ float red[32];
  const int s = blockIdx.x;
  for (int k = 0; k < K; ++k) {
    const int sl = slot[s * K + k];
    if (sl < 0) {
      if (threadIdx.x == 0) dw[s * K + k] = 0.f;
      continue;
    }
    int owner;
    const size_t row = peer_row(sl, C, experts_per_rank, ep_size, my_rank, owner);
    const float wk = w[s * K + k];
    const T* xr = static_cast<const T*>(xsrc.p[owner]) + row * H;
    T* gr = static_cast<T*>(gdst.p[owner]) + row * H;
    float dot = 0.f;
    for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
      const uint4 graw = *reinterpret_cast<const uint4*>(dy + static_cast<size_t>(s) * H + c);
      const uint4 xraw = *reinterpret_cast<const uint4*>(xr + c);
      const T* g = reinterpret_cast<const T*>(&graw);
      const T* x = reinterpret_cast<const T*>(&xraw);
      T o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gv = static_cast<float>(g[j]);
        dot += gv * static_cast<float>(x[j]);
        o[j] = static_cast<T>(wk * gv);
      }
      *reinterpret_cast<uint4*>(gr + c) = *reinterpret_cast<const uint4*>(o);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < (blockDim.x + 31) / 32; ++i) t += red[i];
      dw[s * K + k] = t;
    }
  }
}

}  // namespace oslo

using namespace oslo;

#define OSLO_MOE_DTYPE(CALL)                                    \
  do {                                                          \
    if (dtype == 0) { using T = float; CALL; }                  \
    else if (dtype == 1) { using T = __half; CALL; }            \
    else { using T = __nv_bfloat16; CALL; }                     \
  } while (0)

extern "C" int oslo_moe_positions(const int* expert_idx, int* pos, int* counts, int S, int K, int E, void* stream) {
  if (S <= 0 || E <= 0) return 0;
  moe_positions_kernel<<<E, kScanThreads, 0, (cudaStream_t)stream>>>(expert_idx, pos, counts, S, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// dst_ptrs: host array of ep_size device pointers (ep_size = 1 for a purely local buffer [E*C, H]).
extern "C" int oslo_moe_dispatch(const void* x, void* const* dst_ptrs, int ep_size, const int* slot, int S, int K, int H,
                                 int src_rank, int experts_per_rank, int C, int dtype, void* stream) {
  if (S <= 0) return 0;
  const int esz = dtype == 0 ? 4 : 2;
  if ((H * esz) % 16 || ep_size > 8) return -1;
  DestPtrs d;
  for (int i = 0; i < 8; ++i) d.p[i] = i < ep_size ? dst_ptrs[i] : nullptr;
  OSLO_MOE_DTYPE((moe_dispatch_kernel<T><<<S, 128, 0, (cudaStream_t)stream>>>((const T*)x, d, slot, S, K, H, ep_size, src_rank,
                                                                               experts_per_rank, C)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// inv: [E * C] int, the token index that owns each slot of this source or -1; every slot row is written (zeros when unowned).
extern "C" int oslo_moe_dispatch_rows(const void* x, void* const* dst_ptrs, int ep_size, const int* inv, int E, int H, int src_rank,
                                      int experts_per_rank, int C, int dtype, void* stream) {
  if (E <= 0 || C <= 0) return 0;
  const int esz = dtype == 0 ? 4 : 2;
  if ((H * esz) % 16 || ep_size > 8 || ep_size < 1) return -1;
  DestPtrs d;
  for (int i = 0; i < 8; ++i) d.p[i] = i < ep_size ? dst_ptrs[i] : nullptr;
  OSLO_MOE_DTYPE((moe_dispatch_rows_kernel<T><<<E * C, 128, 0, (cudaStream_t)stream>>>((const T*)x, d, inv, E, H, ep_size, src_rank,
                                                                                       experts_per_rank, C)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_moe_combine(const void* buf, const float* w, const int* slot, void* y, int S, int K, int H, int dtype,
                                void* stream) {
  if (S <= 0) return 0;
  if (H % 8) return -1;
  OSLO_MOE_DTYPE((moe_combine_kernel<T><<<S, 128, 0, (cudaStream_t)stream>>>((const T*)buf, w, slot, (T*)y, S, K, H)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_moe_combine_backward(const void* dy, const void* buf, const float* w, const int* slot, void* dbuf, float* dw,
                                         int S, int K, int H, int dtype, void* stream) {
  if (S <= 0) return 0;
  OSLO_MOE_DTYPE((moe_combine_bwd_kernel<T><<<S, 256, 0, (cudaStream_t)stream>>>((const T*)dy, (const T*)buf, w, slot, (T*)dbuf, dw, S, K, H)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_moe_dispatch_backward(const void* dbuf, const int* slot, void* dx, int S, int K, int H, int dtype,
                                          void* stream) {
  if (S <= 0) return 0;
  OSLO_MOE_DTYPE((moe_dispatch_bwd_kernel<T><<<S, 256, 0, (cudaStream_t)stream>>>((const T*)dbuf, slot, (T*)dx, S, K, H)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// 16-bit types only (rows are moved as 16-byte packets of 8 elements); src_ptrs: host array of ep_size device pointers.
extern "C" int oslo_moe_pull(void* const* src_ptrs, int ep_size, const float* w, const int* slot, void* y, int S, int K, int H,
                             int my_rank, int experts_per_rank, int C, int dtype, void* stream) {
  if (S <= 0) return 0;
  if (H % 8 || ep_size > 8 || dtype == 0) return -1;
  SrcPtrs sp;
  for (int i = 0; i < 8; ++i) sp.p[i] = i < ep_size ? src_ptrs[i] : nullptr;
  if (dtype == 1)
    moe_pull_kernel<__half><<<S, 128, 0, (cudaStream_t)stream>>>(sp, w, slot, (__half*)y, S, K, H, ep_size, my_rank, experts_per_rank, C);
  else
    moe_pull_kernel<__nv_bfloat16><<<S, 128, 0, (cudaStream_t)stream>>>(sp, w, slot, (__nv_bfloat16*)y, S, K, H, ep_size, my_rank, experts_per_rank, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int oslo_moe_push_scaled(const void* dy, void* const* grad_dst_ptrs, void* const* x_src_ptrs, int ep_size, const float* w,
                                    const int* slot, float* dw, int S, int K, int H, int my_rank, int experts_per_rank, int C,
                                    int dtype, void* stream) {
  if (S <= 0) return 0;
  if (H % 8 || ep_size > 8 || dtype == 0) return -1;
  DestPtrs d;
  SrcPtrs sp;
  for (int i = 0; i < 8; ++i) {
    d.p[i] = i < ep_size ? grad_dst_ptrs[i] : nullptr;
    sp.p[i] = i < ep_size ? x_src_ptrs[i] : nullptr;
  }
  if (dtype == 1)
    moe_push_scaled_kernel<__half><<<S, 128, 0, (cudaStream_t)stream>>>((const __half*)dy, d, sp, w, slot, dw, S, K, H, ep_size, my_rank, experts_per_rank, C);
  else
    moe_push_scaled_kernel<__nv_bfloat16><<<S, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, d, sp, w, slot, dw, S, K, H, ep_size, my_rank, experts_per_rank, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

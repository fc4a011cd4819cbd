// Symmetric-memory runtime: device allocations that every rank of a group maps into its own address space
// (CUDA IPC over NVLink / NVSwitch), plus a bounded cross-GPU barrier kernel.
//
// The handles are exchanged by the Python side over the group's host (gloo) communicator.  Kernels of this
// library then read and write peer memory with plain loads / stores; nothing here uses multicast loads.
// The reference has no counterpart: all of its communication goes through torch.distributed collectives
// (oslo/torch/distributed/nn/functional.py:43-214).
#include "gemm_core.cuh"

using namespace oslo;

extern "C" int oslo_symm_alloc(unsigned long long bytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return -(int)e;
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) { cudaFree(p); return -(int)e; }
  cudaDeviceSynchronize();
  *out = p;
  return 0;
}

extern "C" int oslo_symm_free(void* p) { return -(int)cudaFree(p); }

// handle_out: 64 bytes (cudaIpcMemHandle_t)
extern "C" int oslo_ipc_get_handle(void* ptr, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return -(int)e;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

extern "C" int oslo_ipc_open_handle(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return -(int)e;
  *out = p;
  return 0;
}

extern "C" int oslo_ipc_close(void* p) { return -(int)cudaIpcCloseMemHandle(p); }

extern "C" int oslo_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }

extern "C" int oslo_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) return 0;
  return ok;
}

struct PeerFlagPtrs {
  int* p[kMaxRanks];
};

// Every rank stores `epoch` into slot [rank] of every peer's flag array, then waits (bounded) until its own
// array holds `epoch` from everyone.  One block of 32 threads.
__global__ void symm_barrier_kernel(PeerFlagPtrs peers, int* local_flags, int rank, int tp, int epoch, int* status,
                                    const int* epoch_ptr) {
  const int t = threadIdx.x;
  if (epoch_ptr) epoch = *epoch_ptr;  // device-resident epoch: the same launch can be replayed from a CUDA graph
  bool ok = true;
  if (t < tp) {
    __threadfence_system();
    st_release_sys(peers.p[t] + rank, epoch);
    ok = flag_wait_bounded(local_flags + t, epoch, nullptr, true);
  }
  if (!ok && status) atomicCAS(status, kStatusOk, kStatusPeerFlagTimeout);
  __threadfence_system();
}

extern "C" int oslo_symm_barrier(void* const* peer_flags, int* local_flags, int rank, int tp, int epoch, int* status,
                                 void* stream, const int* epoch_ptr) {
  if (tp > kMaxRanks) return -1;
  PeerFlagPtrs pf;
  for (int i = 0; i < kMaxRanks; ++i) pf.p[i] = i < tp ? static_cast<int*>(peer_flags[i]) : nullptr;
  symm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pf, local_flags, rank, tp, epoch, status, epoch_ptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}


// Final step of a reduce-scatter whose transport was the copy engine: every other rank's partial block already sits in
// slot [source] of the local slot buffer (flag [source] holds the call epoch once that copy has landed).
//     out[rows, N] = own[rows, N] + sum over sources s != rank of slots[s][rows, N]  (+ bias[N])
// Blocks wait (bounded) for the flags of all sources, then stream 16-byte vectors; sums in fp32.
__global__ void rs_fold_kernel(const uint16_t* __restrict__ own, const uint16_t* __restrict__ slots, const int* __restrict__ flags,
                               int rank, int tp, long long rows, int N, uint16_t* __restrict__ out,
                               const uint16_t* __restrict__ bias, int is_bf16, int epoch, const int* epoch_ptr, int* status) {
  __shared__ int s_ok;
  if (epoch_ptr) epoch = *epoch_ptr;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < tp && static_cast<int>(threadIdx.x) != rank &&
      !flag_wait_bounded(flags + threadIdx.x, epoch, nullptr, true)) s_ok = 0;
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0 && status) atomicCAS(status, kStatusOk, kStatusPeerFlagTimeout);
    return;
  }
  const long long slot_elems = rows * N;
  const long long nvec = slot_elems / 8;
  const int vec_per_row = N / 8;
  auto unpack = [&](const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (is_bf16) {
        f[2 * j] = __uint_as_float(w[j] << 16);
        f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
        f[2 * j] = __low2float(h);
        f[2 * j + 1] = __high2float(h);
      }
    }
  };
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8], t[8];
    unpack(*reinterpret_cast<const uint4*>(own + i * 8), acc);
    for (int s = 0; s < tp; ++s) {
      if (s == rank) continue;
      unpack(*reinterpret_cast<const uint4*>(slots + s * slot_elems + i * 8), t);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += t[j];
    }
    if (bias) {
      unpack(__ldg(reinterpret_cast<const uint4*>(bias + (i % vec_per_row) * 8)), t);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += t[j];
    }
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (is_bf16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __half2 h = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    *reinterpret_cast<uint4*>(out + i * 8) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// own, out: local [rows, N]; slots: the local slot buffer [tp, rows, N]; flags: local int[tp] written by the sources' copies.
extern "C" int oslo_rs_fold(const void* own, const void* slots, const int* flags, int rank, int tp, long long rows, int N, void* out,
                            const void* bias, int is_bf16, int epoch, const int* epoch_ptr, int* status, int num_sms, void* stream) {
  if (tp > kMaxRanks || tp < 1 || rows <= 0 || N % 8) return -1;
  const long long nvec = rows * N / 8;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 4LL * num_sms) blocks = 4LL * num_sms;
  rs_fold_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(own), static_cast<const uint16_t*>(slots), flags, rank, tp, rows, N, static_cast<uint16_t*>(out),
      static_cast<const uint16_t*>(bias), is_bf16, epoch, epoch_ptr, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

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

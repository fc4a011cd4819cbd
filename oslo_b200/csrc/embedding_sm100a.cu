// Vocab-parallel embedding lookup WITHOUT a collective: the embedding table is sharded by vocabulary rows over the
// tensor group and every shard lives in symmetric (peer-mapped) memory, so each token's row is read straight from
// the rank that owns it over NVLink.  A rank only looks up its own token shard (sequence parallelism), so the traffic
// is (tp-1)/tp of T/tp rows instead of the all-reduce / reduce-scatter of a [T, h] tensor the reference performs
// (oslo/torch/nn/modules/embedding.py:106-135).
#include "common.cuh"

namespace oslo {

struct TablePtrs {
  const void* p[8];
};

// one block per token; 16-byte loads / stores.  ids outside [0, vocab_per_rank * world) give a zero row.
__global__ void embed_pull_kernel(const long long* __restrict__ ids, TablePtrs tables, uint4* __restrict__ out, int tokens,
                                  int row_vecs, long long vocab_per_rank, int world) {
  const int t = blockIdx.x;
  if (t >= tokens) return;
  const long long id = ids[t];
  const long long owner = id / vocab_per_rank;
  uint4* dst = out + static_cast<size_t>(t) * row_vecs;
  if (id < 0 || owner >= world) {
    for (int v = threadIdx.x; v < row_vecs; v += blockDim.x) dst[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = static_cast<const uint4*>(tables.p[owner]) + static_cast<size_t>(id - owner * vocab_per_rank) * row_vecs;
  for (int v = threadIdx.x; v < row_vecs; v += blockDim.x) dst[v] = src[v];
}

}  // namespace oslo

// tables: host array of `world` device pointers to the [vocab_per_rank, H] shards; row_bytes = H * element size.
extern "C" int oslo_embed_pull(const long long* ids, void* const* tables, void* out, int tokens, int row_bytes,
                               long long vocab_per_rank, int world, void* stream) {
  using namespace oslo;
  if (tokens <= 0) return 0;
  if (world > 8 || row_bytes % 16) return -1;
  TablePtrs tp;
  for (int i = 0; i < 8; ++i) tp.p[i] = i < world ? tables[i] : nullptr;
  embed_pull_kernel<<<tokens, 128, 0, static_cast<cudaStream_t>(stream)>>>(ids, tp, static_cast<uint4*>(out), tokens, row_bytes / 16,
                                                                           vocab_per_rank, world);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

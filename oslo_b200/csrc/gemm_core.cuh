// Persistent, warp-specialised tcgen05 GEMM for sm_100a (kernel template and host helpers).
//
//   C[b] = epilogue( A[b] x B[b]^T )        A: [M, K]   B: [N, K]   C: [M, N]
//
// Either operand may be "K-major" (reduction dim contiguous, as stored by
// nn.Linear for x and W) or "MN-major" (the other dim contiguous), so forward
// (x W^T), input-gradient (dY W) and weight-gradient (dY^T x) products all run on
// the same kernel without a transposition pass.
//
// Structure of one CTA (192 threads, one CTA per SM, persistent over tiles):
//   warp 0      TMA producer: cp.async.bulk.tensor loads into a ring of
//               128-byte-swizzled shared-memory stages, completion on mbarriers;
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BLOCK_N,
//               K=16) with the accumulator in tensor memory; two accumulator
//               buffers so the epilogue of tile i overlaps the main loop of i+1;
//   warps 2-5   epilogue: tcgen05.ld the accumulator (one TMEM lane quarter per
//               warp), add bias / apply GELU / add the previous C, convert, stage
//               in swizzled shared memory and write with TMA stores.
//
// All mbarrier waits are bounded; on a timeout the kernel records a status code,
// drains, frees its tensor memory and returns.
//
// Replaces the cuBLAS calls behind F.linear / torch.matmul in the reference
// (oslo/torch/nn/modules/linear.py:73-160 and every _ops.py Matmul_* function).
#pragma once
#include "common.cuh"
#include <cstdio>
#include <mutex>

namespace oslo {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;   // 64 x 2 B = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;

struct GemmParams {
  int M, N, K, batch;
  int batch_inner;    // batch index b = outer * batch_inner + inner; each part has its own stride in the maps
  int causal;         // 0 none; 1 skip tiles entirely above the diagonal (n0 > m0 + 127);
                      // 2 reduce only k <= m0 + 127 (lower-triangular A); 3 reduce only k >= m0 (upper-triangular A^T)
  int m_blocks, n_blocks;
  int epilogue;       // 0 none, 1 +bias, 2 gelu(+bias if given), 3 multiply by gelu'(aux) (aux is an INPUT laid out like C)
  int accumulate;     // 1: C = C_old + result
  int is_bf16;        // 1 bf16, 0 fp16
  const void* bias;   // [N] in the operand dtype, or null
  void* c_ptr;        // plain pointer to C (used for accumulate)
  long long ldc;      // row stride of C in elements
  long long stride_c; // inner batch stride of C in elements
  long long stride_c_outer;  // outer batch stride of C in elements
  void* aux_ptr;      // optional second output: pre-activation (acc + bias), same layout as C
  int* status;
};

template <int BLOCK_N>
struct GemmCfg {
  static constexpr int kStageA = kBlockM * kBlockK * 2;
  static constexpr int kStageB = BLOCK_N * kBlockK * 2;
  static constexpr int kStageBytes = kStageA + kStageB;
  static constexpr int kStages = (BLOCK_N == 256) ? 4 : (BLOCK_N == 128 ? 6 : 8);
  static constexpr int kStagingBytes = 4 * 2 * 4096;  // 4 epilogue warps x 2 buffers x (32 rows x 128 B)
  static constexpr int kTmemCols = 2 * BLOCK_N;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 /*align*/ + 256 /*barriers*/;
};

OSLO_DEVINL void tile_coords(int tile, const GemmParams& p, int& b, int& mb, int& nb) {
  const int per_batch = p.m_blocks * p.n_blocks;
  b = tile / per_batch;
  int t = tile - b * per_batch;
  // groups of 8 m-blocks sweep all n-blocks, m fastest: neighbouring CTAs share B tiles in L2
  constexpr int kGroup = 8;
  const int group_size = kGroup * p.n_blocks;
  const int g = t / group_size;
  const int first_m = g * kGroup;
  const int rows = min(kGroup, p.m_blocks - first_m);
  const int r = t - g * group_size;
  mb = first_m + r % rows;
  nb = r / rows;
}


// ------------------------------------------------------------------------------------------------
// Fused collective modes.  Ranks exchange data through peer-mapped ("symmetric") buffers; flags hold
// the epoch (a per-group call counter) of the last completed hand-off, so they never need clearing.
// MODE is a bit mask: both collectives may run in one launch (all-gather of the A rows over one group, reduce-scatter
// of the result over another one: the 3-D tensor-parallel linear).
constexpr int kModePlain = 0;
constexpr int kModeAllGather = 1;      // A rows are gathered from all ranks while the GEMM runs
constexpr int kModeReduceScatter = 2;  // partial blocks are TMA-stored to their owner; the owner's own tiles add them in
constexpr int kModeGatherScatter = 3;  // both
constexpr int kMaxRanks = 8;

struct FusedParams {
  // Tile order and reduce-scatter side.  In all-gather-only launches these describe the gather group.
  int tp = 1, rank = 0;
  int shard_rows = 0;       // rows of A (AG) / of C (RS along rows) owned by one rank; a multiple of 128
  int tiles_per_shard = 0;  // output tiles per shard
  int tiles_per_chunk = 0;  // RS: output tiles per row chunk
  int epoch = 0;
  const int* epoch_ptr = nullptr;  // when set, the epoch is read from device memory (CUDA-graph replays advance it)
  int copy_ctas = 0;        // AG: CTAs [0, copy_ctas) copy, the others multiply
  int k_elems = 0;          // AG: row length of A in elements
  int chunk_rows = 0;       // rows per hand-off chunk (a multiple of 128 dividing shard_rows); one flag per chunk
  // Reduce-scatter along the COLUMNS of C (2-D / 2.5-D linears: every rank keeps all rows and one block of features).
  int rs_along_n = 0;
  int shard_cols = 0;       // columns of C owned by one rank (a multiple of the tile width)
  int n_blocks_per_shard = 0;
  int cps = 0;              // RS: row chunks per destination block
  int slot_rows = 0;        // RS: rows of one source's slot in the owner's slot buffer
  int slot_ld = 0;          // RS: row pitch of the slot buffer in elements
  // All-gather side (its own group: in a gather + scatter launch the two groups differ).
  int ag_tp = 1, ag_rank = 0;
  int ag_shard_rows = 0, ag_chunk_rows = 0;
  int ag_epoch = 0;
  const int* ag_epoch_ptr = nullptr;
  // all-gather
  const void* peer_in[kMaxRanks] = {};  // entry [ag_rank]: this rank's shard [shard_rows, K], read in place (any local memory)
  void* x_full = nullptr;               // local gathered buffer [tp * shard_rows, K] (= peer_xfull[ag_rank])
  void* peer_xfull[kMaxRanks] = {};     // every rank's gathered buffer: our shard is pushed into slot [ag_rank] of each
  int* chunk_flag = nullptr;            // local [tp * chunks_per_shard], written by the SOURCE rank: that chunk has landed
  int* peer_chunk_flag[kMaxRanks] = {}; // the same array on every rank
  int* chunk_arrive = nullptr;          // local [chunks_per_shard]: copy-CTA arrival counters for our own shard's chunks
  // reduce-scatter
  void* peer_slots[kMaxRanks] = {};     // every rank's slot buffer [tp, shard_rows, N] (slot s = rows from rank s)
  int* rs_flag = nullptr;               // local [tp * chunks_per_shard]: source p finished that chunk of our rows
  int* peer_rs_flag[kMaxRanks] = {};
  int* tile_done = nullptr;             // local [tp * chunks_per_shard]: per-chunk arrival counters
  void* rs_out = nullptr;               // local [shard_rows, N]
  const void* rs_bias = nullptr;        // optional [N]
  int* status = nullptr;
  unsigned long long* debug_times = nullptr;  // optional [8]: globaltimer stamps for tuning (null in normal use)
  // NVSwitch multicast (both null without it).  mc_xfull: the gathered buffer of this call mapped on a multicast object
  // over the group: one multimem.st delivers a piece of our shard to every rank.  mc_slots: the partial-product buffer
  // [T, N] mapped the same way: every rank stores its partial tiles LOCALLY and the owner of a row block reads the sum
  // over all ranks with multimem.ld_reduce (the switch adds in fp32).
  void* mc_xfull = nullptr;
  const void* mc_slots = nullptr;
};

// Tensor maps over every rank's slot buffer (reduce-scatter mode: the epilogue TMA-stores straight into the owner).
struct PeerMaps {
  CUtensorMap m[kMaxRanks];
};

OSLO_DEVINL int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
OSLO_DEVINL int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
OSLO_DEVINL void st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
OSLO_DEVINL void st_release_gpu(int* p, int v) { asm volatile("st.release.gpu.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
OSLO_DEVINL void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Wait (bounded, ~2 s) until *flag >= target.  abort_flag may be null.
OSLO_DEVINL bool flag_wait_bounded(const int* flag, int target, volatile int* abort_flag, bool sys_scope) {
  if ((sys_scope ? ld_acquire_sys(flag) : ld_acquire_gpu(flag)) >= target) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 1;; ++i) {
    if ((sys_scope ? ld_acquire_sys(flag) : ld_acquire_gpu(flag)) >= target) return true;
    if ((i & 0x3f) == 0) {
      if (abort_flag && *abort_flag) return false;
      if (global_timer_ns() - t0 > kWaitBudgetNs) break;
    }
    __nanosleep(64);
  }
  if (abort_flag) *abort_flag = 1;
  return false;
}

// Output tiles in shard order: AG starts with the local shard (rank, rank+1, ...), RS ends with it
// (rank+1, ..., rank), so remote traffic and compute overlap from the first tile on.
template <int MODE>
OSLO_DEVINL void fused_tile_coords(int tile, const GemmParams& p, const FusedParams& fp, int& b, int& mb, int& nb) {
  b = 0;
  const int blocks_per_chunk = fp.chunk_rows / kBlockM;
  if constexpr (MODE == kModeReduceScatter) {
    if (fp.mc_slots != nullptr) {
      // Multicast reduce-scatter: every rank walks the SAME order, row chunk by row chunk and inside a chunk owner by
      // owner, so chunk c of an owner's block is complete on all ranks at about the same time and the owners' reducer
      // CTAs pull a steady stream while the products of later chunks are still running.
      const int round = fp.tiles_per_chunk * fp.tp;
      const int c = tile / round, u = tile - c * round;
      const int shard = u / fp.tiles_per_chunk, r = u - shard * fp.tiles_per_chunk;
      mb = shard * (fp.shard_rows / kBlockM) + c * blocks_per_chunk + r % blocks_per_chunk;
      nb = r / blocks_per_chunk;
      return;
    }
  }
  if constexpr ((MODE & kModeReduceScatter) != 0) {
    // Block by block in destination order: the next rank's block first, our own block LAST (by then the other ranks'
    // partials of it have long arrived, so the tiles that finish the reduction do not wait; an order that interleaved
    // own and foreign row chunks measured slower: every skew between ranks stalled a persistent CTA).  Inside a block,
    // row chunk by row chunk, so chunks are completed, and flagged, in order.
    const int i = tile / fp.tiles_per_shard;
    const int t = tile - i * fp.tiles_per_shard;
    const int shard = (fp.rank + i + 1) % fp.tp;
    const int per_chunk = fp.tiles_per_chunk;
    const int c = t / per_chunk, r = t - c * per_chunk;
    if (fp.rs_along_n) {
      mb = c * blocks_per_chunk + r % blocks_per_chunk;
      nb = shard * fp.n_blocks_per_shard + r / blocks_per_chunk;
    } else {
      mb = shard * (fp.shard_rows / kBlockM) + c * blocks_per_chunk + r % blocks_per_chunk;
      nb = r / blocks_per_chunk;
    }
    return;
  }
  // all-gather only: the local shard first (no waiting), then row chunk by row chunk over the other ranks' shards, which
  // is the order in which every rank pushes its shard out (chunk 0 to everybody, then chunk 1 ...)
  const int blocks_per_shard = fp.shard_rows / kBlockM;
  const int n_blocks = fp.tiles_per_shard / blocks_per_shard;
  const int per_chunk = blocks_per_chunk * n_blocks;
  int shard, c, r;
  if (tile < fp.tiles_per_shard) {
    shard = fp.rank;
    c = tile / per_chunk;
    r = tile - c * per_chunk;
  } else {
    const int t = tile - fp.tiles_per_shard;
    const int per_round = per_chunk * (fp.tp - 1);  // chunk c of every other shard
    c = t / per_round;
    const int u = t - c * per_round;
    shard = (fp.rank + 1 + u / per_chunk) % fp.tp;
    r = u % per_chunk;
  }
  mb = shard * blocks_per_shard + c * blocks_per_chunk + r % blocks_per_chunk;
  nb = r / blocks_per_chunk;
}

// Reduce-scatter bookkeeping of an output tile: the rank that owns it, the row chunk inside the owner's block, and the
// index of that (owner, chunk) pair in the counter / flag arrays.
OSLO_DEVINL void rs_tile_owner(const FusedParams& fp, int m0, int n0, int& dest, int& c_in_dest) {
  if (fp.rs_along_n) {
    dest = n0 / fp.shard_cols;
    c_in_dest = m0 / fp.chunk_rows;
  } else {
    dest = m0 / fp.shard_rows;
    c_in_dest = (m0 - dest * fp.shard_rows) / fp.chunk_rows;
  }
}

// Untiled bulk copies (TMA engine, no multicast): global -> shared with mbarrier completion, shared -> global in a
// bulk group.  Addresses and sizes are multiples of 16 bytes.
OSLO_DEVINL void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
OSLO_DEVINL void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}

constexpr int kCopyPiece = 32768;  // bytes per bulk copy
constexpr int kCopyDepth = 6;      // ring slots per copy CTA (6 x 32 KiB of shared memory)
constexpr int kCopyAhead = 2;      // local loads run this many pieces ahead of the stores; the other ring slots hold
                                   // pieces whose stores are still draining (several store groups in flight)

// AG copy role: PUSH.  Reading a peer's memory is bound by the NVLink round trip (a few KB in flight per SM: measured
// ~6 GB/s per copy CTA), writing to it is not: writes are posted.  So every rank pushes ITS OWN shard into the gathered
// buffer of every rank.  One thread per copy CTA drives the TMA engine: 32 KiB pieces of the local shard go through a
// shared-memory ring (bulk load, local memory) and out again as one bulk store per destination (peers and ourselves).
// When all copy CTAs have finished the stores of a row chunk, the last one raises that chunk's flag ON EVERY
// DESTINATION; a GEMM CTA there takes the chunk as soon as the flag holds this call's epoch.
static __device__ __noinline__ void ag_copy_role(const GemmParams& p, const FusedParams& fp, uint8_t* ring, uint64_t* bars) {
  if (threadIdx.x != 0) return;
  __shared__ int s_abort;
  s_abort = 0;
  for (int i = 0; i < kCopyDepth; ++i) mbar_init(&bars[i], 1);
  fence_barrier_init();
  const int cps = fp.ag_shard_rows / fp.ag_chunk_rows;  // chunks per shard
  const long long chunk_bytes = static_cast<long long>(fp.ag_chunk_rows) * fp.k_elems * 2;
  const long long shard_bytes = chunk_bytes * cps;
  const int ppc = static_cast<int>((chunk_bytes + kCopyPiece - 1) / kCopyPiece);  // pieces per chunk
  const long long total = static_cast<long long>(cps) * ppc;                      // pieces of OUR shard
  const int owners = fp.copy_ctas < ppc ? fp.copy_ctas : ppc;                     // copy CTAs with pieces in a chunk
  const long long my_count = total > blockIdx.x ? (total - blockIdx.x + fp.copy_ctas - 1) / fp.copy_ctas : 0;
  const uint8_t* my_shard = static_cast<const uint8_t*>(fp.peer_in[fp.ag_rank]);
  bool ok = true;
  auto locate = [&](long long j, long long& off, uint32_t& bytes, int& c, bool& last_of_chunk) {
    const long long g = blockIdx.x + j * fp.copy_ctas;
    c = static_cast<int>(g / ppc);
    const long long in_chunk = (g - static_cast<long long>(c) * ppc) * kCopyPiece;
    bytes = static_cast<uint32_t>(chunk_bytes - in_chunk < kCopyPiece ? chunk_bytes - in_chunk : kCopyPiece);
    off = static_cast<long long>(c) * chunk_bytes + in_chunk;
    last_of_chunk = (g + fp.copy_ctas) / ppc != c;  // our next piece (if any) belongs to a later chunk
  };
  for (long long n = 0; n < my_count + kCopyAhead && ok; ++n) {
    if (n < my_count) {
      long long off; uint32_t bytes; int c; bool last;
      locate(n, off, bytes, c, last);
      if (!OSLO_IN_BOUNDS(off >= 0 && off + bytes <= shard_bytes && c < cps, fp.status)) { ok = false; break; }
      // slot n % depth last held piece n - depth; the store groups committed since then are pieces n - depth + 1 ..
      // n - 1 - ahead, so that many may still be pending when its own stores have finished reading the slot
      if (n >= kCopyDepth) tma_store_wait_read<kCopyDepth - 1 - kCopyAhead>();
      uint64_t* bar = &bars[n % kCopyDepth];
      mbar_arrive_expect_tx(bar, bytes);
      bulk_load(ring + (n % kCopyDepth) * kCopyPiece, my_shard + off, bytes, bar);
    }
    const long long m = n - kCopyAhead;
    if (m >= 0 && m < my_count) {
      long long off; uint32_t bytes; int c; bool last;
      locate(m, off, bytes, c, last);
      if (!mbar_wait_bounded(&bars[m % kCopyDepth], static_cast<uint32_t>((m / kCopyDepth) & 1), &s_abort)) {
        if (fp.status) atomicCAS(fp.status, kStatusOk, kStatusPeerFlagTimeout);
        ok = false;
        break;
      }
      // farthest destination first is as good as any: all links are symmetric through the switch
      for (int i = 1; i <= fp.ag_tp; ++i) {
        const int d = (fp.ag_rank + i) % fp.ag_tp;
        bulk_store(static_cast<uint8_t*>(fp.peer_xfull[d]) + fp.ag_rank * shard_bytes + off, ring + (m % kCopyDepth) * kCopyPiece, bytes);
      }
      tma_store_commit();
      if (last) {
        tma_store_wait_all();  // our pieces of this chunk have been written everywhere
        fence_proxy_async_global();
        __threadfence_system();
        const int old = atomicAdd(fp.chunk_arrive + c, 1);
        if (old == owners - 1) {
          fp.chunk_arrive[c] = 0;
          __threadfence_system();
          for (int d = 0; d < fp.ag_tp; ++d) st_release_sys(fp.peer_chunk_flag[d] + fp.ag_rank * cps + c, fp.ag_epoch);
        }
      }
    }
  }
  tma_store_wait_all();
}

OSLO_DEVINL void multimem_st_v4(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
OSLO_DEVINL uint4 multimem_ld_reduce_v4(const void* mc, bool bf16) {
  uint4 v;
  if (bf16) asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  else asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                    : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}

// AG copy role over NVSwitch multicast: all threads of the copy CTAs read our shard (local memory, 16 bytes per thread and
// step) and store each vector ONCE to the multicast address of the gathered buffer; the switch delivers it to every rank
// (ourselves included), so our links carry the shard once instead of once per peer.  Chunk flags as in the unicast role.
static __device__ __noinline__ void ag_mc_copy_role(const GemmParams& p, const FusedParams& fp) {
  constexpr int kUnroll = 16;
  const int cps = fp.ag_shard_rows / fp.ag_chunk_rows;
  const long long chunk_vecs = static_cast<long long>(fp.ag_chunk_rows) * fp.k_elems * 2 / 16;
  const uint4* src = static_cast<const uint4*>(fp.peer_in[fp.ag_rank]);
  uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(fp.mc_xfull)) + static_cast<long long>(fp.ag_rank) * cps * chunk_vecs;
  const long long stride = static_cast<long long>(fp.copy_ctas) * blockDim.x;
  for (int c = 0; c < cps; ++c) {
    const uint4* s = src + c * chunk_vecs;
    uint4* d = dst + c * chunk_vecs;
    if (!OSLO_IN_BOUNDS(static_cast<long long>(c + 1) * chunk_vecs * 16 <= static_cast<long long>(fp.ag_shard_rows) * fp.k_elems * 2,
                        fp.status)) return;
    long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + (kUnroll - 1) * stride < chunk_vecs; i += kUnroll * stride) {
      uint4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) v[u] = __ldg(s + i + u * stride);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) multimem_st_v4(d + i + u * stride, v[u]);
    }
    for (; i < chunk_vecs; i += stride) multimem_st_v4(d + i, __ldg(s + i));
    __threadfence_system();  // this thread's multicast stores are performed everywhere before the arrival below
    __syncthreads();
    if (threadIdx.x == 0) {
      const int old = atomicAdd(fp.chunk_arrive + c, 1);
      if (old == fp.copy_ctas - 1) {
        fp.chunk_arrive[c] = 0;
        __threadfence_system();
        for (int r = 0; r < fp.ag_tp; ++r) st_release_sys(fp.peer_chunk_flag[r] + fp.ag_rank * cps + c, fp.ag_epoch);
      }
    }
  }
}

// RS reduce role over NVSwitch multicast: the reducer CTAs of the rank that owns a row block wait until every rank has
// flagged row chunk c of that block (all partial tiles of the chunk are in the ranks' local partial buffers), then read
// the chunk through the multicast address with multimem.ld_reduce (one load returns the sum over all ranks, accumulated in
// fp32 inside the switch), add the bias and write the final rows.  Many independent loads per thread: the reduction is a
// round trip through the switch and only bytes in flight hide it.
static __device__ __noinline__ void rs_mc_reduce_role(const GemmParams& p, const FusedParams& fp) {
  constexpr int kUnroll = 16;
  __shared__ int s_ok;
  const int vec_per_row = p.N / 8;
  const long long chunk_vecs = static_cast<long long>(fp.chunk_rows) * vec_per_row;
  const long long stride = static_cast<long long>(fp.copy_ctas) * blockDim.x;
  const bool bf16 = p.is_bf16 != 0;
  for (int c = 0; c < fp.cps; ++c) {
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < fp.tp &&
        !flag_wait_bounded(fp.rs_flag + threadIdx.x * fp.cps + c, fp.epoch, nullptr, true)) s_ok = 0;
    __syncthreads();
    if (!s_ok) {
      if (threadIdx.x == 0 && fp.status) atomicCAS(fp.status, kStatusOk, kStatusPeerFlagTimeout);
      return;
    }
    const long long row0 = static_cast<long long>(fp.rank) * fp.shard_rows + static_cast<long long>(c) * fp.chunk_rows;
    if (!OSLO_IN_BOUNDS(row0 + fp.chunk_rows <= p.M && (c + 1) * fp.chunk_rows <= fp.shard_rows, fp.status)) return;
    const uint4* src = static_cast<const uint4*>(fp.mc_slots) + row0 * vec_per_row;       // partial buffer [T, N]
    uint4* dst = static_cast<uint4*>(fp.rs_out) + static_cast<long long>(c) * chunk_vecs;  // out [T / tp, N]
    auto finish = [&](long long i, uint4 v) {
      if (fp.rs_bias != nullptr) {
        const int col = static_cast<int>(i % vec_per_row) * 8;
        const uint4 braw = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(fp.rs_bias) + col));
        uint32_t* w = reinterpret_cast<uint32_t*>(&v);
        const uint32_t* bw = reinterpret_cast<const uint32_t*>(&braw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (bf16) {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&w[j]), b = *reinterpret_cast<const __nv_bfloat162*>(&bw[j]);
            const __nv_bfloat162 r = __floats2bfloat162_rn(__low2float(a) + __low2float(b), __high2float(a) + __high2float(b));
            w[j] = *reinterpret_cast<const uint32_t*>(&r);
          } else {
            const __half2 a = *reinterpret_cast<const __half2*>(&w[j]), b = *reinterpret_cast<const __half2*>(&bw[j]);
            const __half2 r = __floats2half2_rn(__low2float(a) + __low2float(b), __high2float(a) + __high2float(b));
            w[j] = *reinterpret_cast<const uint32_t*>(&r);
          }
        }
      }
      dst[i] = v;
    };
    long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + (kUnroll - 1) * stride < chunk_vecs; i += kUnroll * stride) {
      uint4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) v[u] = multimem_ld_reduce_v4(src + i + u * stride, bf16);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) finish(i + u * stride, v[u]);
    }
    for (; i < chunk_vecs; i += stride) finish(i, multimem_ld_reduce_v4(src + i, bf16));
  }
}

// k-block range [kb0, kb1) a tile has to reduce over, or skip = true when it has no work.
OSLO_DEVINL void tile_k_range(const GemmParams& p, int m0, int n0, int num_kb, int& kb0, int& kb1, bool& skip) {
  kb0 = 0;
  kb1 = num_kb;
  skip = false;
  if (p.causal == 1) skip = n0 > m0 + kBlockM - 1;
  else if (p.causal == 2) kb1 = min(num_kb, (m0 + kBlockM + kBlockK - 1) / kBlockK);
  else if (p.causal == 3) kb0 = min(num_kb - 1, m0 / kBlockK);
}

template <int BLOCK_N, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux,
                    const GemmParams p, const FusedParams fp_in, const __grid_constant__ PeerMaps peer_maps) {
  FusedParams fp = fp_in;
  if (MODE != kModePlain && fp.epoch_ptr) fp.epoch = *fp.epoch_ptr;
  if ((MODE & kModeAllGather) && fp.ag_epoch_ptr) fp.ag_epoch = *fp.ag_epoch_ptr;
  if constexpr ((MODE & kModeAllGather) != 0) {
    // the first fp.copy_ctas CTAs stream the peers' shards into local memory; the rest run the GEMM
    if (static_cast<int>(blockIdx.x) < fp.copy_ctas) {
      if (fp.mc_xfull != nullptr) {
        ag_mc_copy_role(p, fp);
        return;
      }
      extern __shared__ uint8_t copy_smem_raw[];
      uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(copy_smem_raw) + 1023) & ~uintptr_t(1023));
      ag_copy_role(p, fp, ring, reinterpret_cast<uint64_t*>(ring + kCopyDepth * kCopyPiece));
      return;
    }
  }
  if constexpr (MODE == kModeReduceScatter) {
    // multicast reduce-scatter: the first fp.copy_ctas CTAs pull the reduced rows of our block; the rest run the GEMM
    if (fp.mc_slots != nullptr && static_cast<int>(blockIdx.x) < fp.copy_ctas) {
      rs_mc_reduce_role(p, fp);
      return;
    }
  }
  const int cta = (MODE != kModePlain) ? static_cast<int>(blockIdx.x) - fp.copy_ctas : static_cast<int>(blockIdx.x);
  const int num_ctas = (MODE != kModePlain) ? static_cast<int>(gridDim.x) - fp.copy_ctas : static_cast<int>(gridDim.x);
  using Cfg = GemmCfg<BLOCK_N>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* staging = smem + kStages * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + Cfg::kStagingBytes);
  uint64_t* full_bar = bars;                    // [kStages]
  uint64_t* empty_bar = bars + kStages;         // [kStages]
  uint64_t* tmem_full = bars + 2 * kStages;     // [2]
  uint64_t* tmem_empty = bars + 2 * kStages + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.batch * p.m_blocks * p.n_blocks;
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int armed = 0;  // stages armed since start (capped), used to drain on abort
      int ready_shard = -1;
      (void)ready_shard;
      for (int tile = cta; tile < num_tiles && ok; tile += num_ctas) {
        int b, mb, nb;
        if constexpr (MODE == kModePlain) tile_coords(tile, p, b, mb, nb);
        else fused_tile_coords<MODE>(tile, p, fp, b, mb, nb);
        if (!OSLO_IN_BOUNDS(mb >= 0 && mb < p.m_blocks && nb >= 0 && nb < p.n_blocks && b >= 0 && b < p.batch, p.status)) {
          *abort_flag = 1;  // the other roles leave through their bounded waits
          ok = false;
          break;
        }
        const int m0 = mb * kBlockM, n0 = nb * BLOCK_N;
        const int bi = b % p.batch_inner, bo = b / p.batch_inner;
        int kb0, kb1;
        bool skip;
        tile_k_range(p, m0, n0, num_kb, kb0, kb1, skip);
        if (skip) continue;
        bool a_local = false;
        if constexpr ((MODE & kModeAllGather) != 0) {
          // rows of shard s become loadable once the copy CTAs have flagged the chunk; the own shard is read
          // straight from the symmetric input buffer through its own tensor map
          const int shard = m0 / fp.ag_shard_rows;
          const int chunk = m0 / fp.ag_chunk_rows;
          a_local = shard == fp.ag_rank;
          if (!a_local && chunk != ready_shard) {
            if (!flag_wait_bounded(fp.chunk_flag + chunk, fp.ag_epoch, abort_flag, true)) {
              ok = false;
              if (p.status) atomicCAS(p.status, kStatusOk, kStatusPeerFlagTimeout);
              break;
            }
            fence_proxy_async_global();
            ready_shard = chunk;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag)) {
            ok = false;
            if (p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutProducer);
            break;
          }
          uint8_t* sa = stage_base + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kStageA;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          const int k0 = kb * kBlockK;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < kBlockM / 64; ++c) tma_load_4d(sa + c * 8192, &tmA, &full_bar[stage], m0 + c * 64, k0, bi, bo);
          } else {
            if ((MODE & kModeAllGather) && a_local) tma_load_4d(sa, &tmAux, &full_bar[stage], k0, m0 - fp.ag_rank * fp.ag_shard_rows, bi, bo);
            else tma_load_4d(sa, &tmA, &full_bar[stage], k0, m0, bi, bo);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BLOCK_N / 64; ++c) tma_load_4d(sb + c * 8192, &tmB, &full_bar[stage], n0 + c * 64, k0, bi, bo);
          } else {
            tma_load_4d(sb, &tmB, &full_bar[stage], k0, n0, bi, bo);
          }
          if (armed < kStages) ++armed;
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // leave no bulk copy in flight: every armed stage's full barrier must flip (bounded)
        for (int s = 0; s < armed; ++s) {
          int st = (stage - 1 - s + 2 * kStages) % kStages;
          uint32_t ph = (st < stage) ? phase : (phase ^ 1);
          for (uint32_t i = 0; i < (1u << 22); ++i)
            if (mbar_try_wait(&full_bar[st], ph)) break;
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_bf16 = make_idesc_f16(kBlockM, BLOCK_N, true, A_MN, B_MN);
      constexpr uint32_t idesc_fp16 = make_idesc_f16(kBlockM, BLOCK_N, false, A_MN, B_MN);
      const uint32_t idesc = p.is_bf16 ? idesc_bf16 : idesc_fp16;
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += num_ctas) {
        int kb0 = 0, kb1 = num_kb;
        if (p.causal) {
          int b, mb, nb;
          bool skip;
          tile_coords(tile, p, b, mb, nb);
          tile_k_range(p, mb * kBlockM, nb * BLOCK_N, num_kb, kb0, kb1, skip);
          if (skip) continue;
        }
        if (!mbar_wait_bounded(&tmem_empty[buf], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BLOCK_N;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kStageA;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            // K-major: 16 elements = 32 bytes along the swizzled row; 8-row groups 1024 B apart.
            // MN-major: 16 k-rows of 128 B = 2048 B; 64-wide MN chunks 8192 B apart.
            const uint64_t da = A_MN ? make_smem_desc_sw128(sa + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma_f16(tmem_d, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[buf]);
        buf ^= 1;
        if (buf == 0) acc_phase ^= 1;
      }
      if (!ok && p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutMma);
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint8_t* my_staging = staging + (warp - 2) * 2 * 4096;
    int buf = 0;
    uint32_t acc_phase = 0;
    int sbuf = 0;
    int rs_pending = 0;
    (void)rs_pending;
    bool ok = true;
    if (MODE != kModePlain && fp.debug_times && cta == 0 && warp == 2 && lane == 0) fp.debug_times[4] = global_timer_ns();
    for (int tile = cta; tile < num_tiles && ok; tile += num_ctas) {
      int b, mb, nb;
      if constexpr (MODE == kModePlain) tile_coords(tile, p, b, mb, nb);
      else fused_tile_coords<MODE>(tile, p, fp, b, mb, nb);
      const int m0 = mb * kBlockM, n0 = nb * BLOCK_N;
      const int bi = b % p.batch_inner, bo = b / p.batch_inner;
      if (p.causal == 1 && n0 > m0 + kBlockM - 1) continue;
      if (!mbar_wait_bounded(&tmem_full[buf], acc_phase, abort_flag)) {
        ok = false;
        if (p.status && lane == 0) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BLOCK_N;
      bool rs_own = false;
      int rs_dest = 0, rs_c = 0;  // owner of this tile and row chunk inside the owner's block
      (void)rs_dest; (void)rs_c;
      if constexpr ((MODE & kModeReduceScatter) != 0) {
        // tiles of OUR block finish the reduction themselves: the other ranks' partials must have landed in our
        // slot buffer (they compute our block first, so this normally does not wait)
        rs_tile_owner(fp, m0, n0, rs_dest, rs_c);
        // with a multicast partial buffer no tile is finished here: all go to local memory and the reducer CTAs pull sums
        rs_own = fp.mc_slots == nullptr && rs_dest == fp.rank;
        if (rs_own) {
          const int cps = fp.cps;
          const int c = rs_c;
          bool got = true;
          if (lane < fp.tp && lane != fp.rank) got = flag_wait_bounded(fp.rs_flag + lane * cps + c, fp.epoch, abort_flag, true);
          got = __all_sync(0xffffffffu, got);
          if (!got) {
            ok = false;
            if (p.status && lane == 0) atomicCAS(p.status, kStatusOk, kStatusPeerFlagTimeout);
          }
        }
      }
#pragma unroll 1
      for (int chunk = 0; chunk < BLOCK_N / 64; ++chunk) {
        uint32_t r0[32], r1[32];
        __syncwarp();  // tcgen05.ld is .sync.aligned: the warp must be converged (lane 0 branches above)
        tmem_ld_32x32(taddr + chunk * 64, r0);
        tmem_ld_32x32(taddr + chunk * 64 + 32, r1);
        tmem_ld_wait();
        if (chunk == BLOCK_N / 64 - 1) {
          // accumulator fully read: hand the TMEM buffer back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
        const int col0 = n0 + chunk * 64;
        if (col0 >= p.N) continue;  // warp-uniform
        float v[64];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          v[i] = __uint_as_float(r0[i]);
          v[32 + i] = __uint_as_float(r1[i]);
        }
        if (p.bias != nullptr && (!(MODE & kModeReduceScatter) || rs_own)) {  // RS: the bias is added once, by the owner
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if (col0 + g * 8 < p.N) {
              const uint4 raw = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.bias) + col0 + g * 8));
              const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float lo, hi;
                if (p.is_bf16) {
                  lo = __uint_as_float(w[j] << 16);
                  hi = __uint_as_float(w[j] & 0xffff0000u);
                } else {
                  const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
                  lo = __low2float(h);
                  hi = __high2float(h);
                }
                v[g * 8 + 2 * j] += lo;
                v[g * 8 + 2 * j + 1] += hi;
              }
            }
          }
        }
        if (p.accumulate && row < p.M) {
          const uint16_t* cin = static_cast<const uint16_t*>(p.c_ptr) + static_cast<long long>(bi) * p.stride_c +
                                static_cast<long long>(bo) * p.stride_c_outer + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if (col0 + g * 8 < p.N) {
              const uint4 raw = *reinterpret_cast<const uint4*>(cin + g * 8);
              const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float lo, hi;
                if (p.is_bf16) {
                  lo = __uint_as_float(w[j] << 16);
                  hi = __uint_as_float(w[j] & 0xffff0000u);
                } else {
                  const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
                  lo = __low2float(h);
                  hi = __high2float(h);
                }
                v[g * 8 + 2 * j] += lo;
                v[g * 8 + 2 * j + 1] += hi;
              }
            }
          }
        }
        if constexpr ((MODE & kModeReduceScatter) != 0) {
          if (rs_own && ok) {
            const long long r_local = static_cast<long long>((fp.rs_along_n ? m0 : m0 - fp.rank * fp.shard_rows) + q * 32 + lane);
            const int c_local = fp.rs_along_n ? col0 - fp.rank * fp.shard_cols : col0;
            for (int src = 0; src < fp.tp; ++src) {
              if (src == fp.rank) continue;
              const uint16_t* sp = static_cast<const uint16_t*>(fp.peer_slots[fp.rank]) +
                                   (static_cast<long long>(src) * fp.slot_rows + r_local) * fp.slot_ld + c_local;
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                if (col0 + g * 8 < p.N) {
                  const uint4 raw = *reinterpret_cast<const uint4*>(sp + g * 8);
                  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    float lo, hi;
                    if (p.is_bf16) {
                      lo = __uint_as_float(w[j] << 16);
                      hi = __uint_as_float(w[j] & 0xffff0000u);
                    } else {
                      const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
                      lo = __low2float(h);
                      hi = __high2float(h);
                    }
                    v[g * 8 + 2 * j] += lo;
                    v[g * 8 + 2 * j + 1] += hi;
                  }
                }
              }
            }
          }
        }
        if (p.epilogue == 3 && row < p.M) {
          // multiply by gelu'(aux): aux holds a pre-activation laid out like C (the backward of a fused bias-GELU linear:
          // dPre = (dY W) * gelu'(pre) without a separate element-wise pass)
          const uint16_t* ain = static_cast<const uint16_t*>(p.aux_ptr) + static_cast<long long>(bi) * p.stride_c +
                                static_cast<long long>(bo) * p.stride_c_outer + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if (col0 + g * 8 < p.N) {
              const uint4 raw = *reinterpret_cast<const uint4*>(ain + g * 8);
              const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float lo, hi;
                if (p.is_bf16) {
                  lo = __uint_as_float(w[j] << 16);
                  hi = __uint_as_float(w[j] & 0xffff0000u);
                } else {
                  const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
                  lo = __low2float(h);
                  hi = __high2float(h);
                }
                v[g * 8 + 2 * j] *= gelu_tanh_grad(lo);
                v[g * 8 + 2 * j + 1] *= gelu_tanh_grad(hi);
              }
            }
          }
        }
        const bool want_aux = (p.aux_ptr != nullptr) && p.epilogue != 3;
        // up to two stores per chunk: optional pre-activation (aux) then the final value
        for (int pass = want_aux ? 0 : 1; pass < 2; ++pass) {
          uint8_t* sbuf_ptr = my_staging + sbuf * 4096;
          if (lane == 0) tma_store_wait_read<1>();  // the store issued two buffers ago has drained
          __syncwarp();
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            uint32_t packed[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float a0 = v[g * 8 + 2 * j], a1 = v[g * 8 + 2 * j + 1];
              if (pass == 1 && p.epilogue == 2) {
                a0 = gelu_tanh(a0);
                a1 = gelu_tanh(a1);
              }
              if (p.is_bf16) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(a0, a1);
                packed[j] = *reinterpret_cast<const uint32_t*>(&h);
              } else {
                const __half2 h = __floats2half2_rn(a0, a1);
                packed[j] = *reinterpret_cast<const uint32_t*>(&h);
              }
            }
            // 128-byte swizzle: 16-byte chunk index XOR (row mod 8)
            uint4* dst = reinterpret_cast<uint4*>(sbuf_ptr + lane * 128 + ((g ^ (lane & 7)) << 4));
            *dst = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if constexpr ((MODE & kModeReduceScatter) != 0) {
              // slot [this rank] of the rank that owns this block (a peer-mapped buffer; plain bulk store, no multicast)
              const int dest = rs_dest;
              const int r_in = fp.rs_along_n ? m0 : m0 - dest * fp.shard_rows;
              const int c_in = fp.rs_along_n ? col0 - dest * fp.shard_cols : col0;
              const int rows_in_slot = fp.rs_along_n ? p.M : fp.shard_rows;
              if (!OSLO_IN_BOUNDS(dest >= 0 && dest < fp.tp && r_in >= 0 && r_in + q * 32 < rows_in_slot && c_in >= 0 &&
                                  c_in < fp.slot_ld, fp.status)) {
                // debug builds: a tile that would leave its slot is not stored
              } else
              if (rs_own) tma_store_4d(&tmC, sbuf_ptr, c_in, r_in + q * 32, 0, 0);  // final values
              else if (fp.mc_slots != nullptr) tma_store_4d(&peer_maps.m[fp.rank], sbuf_ptr, col0, m0 + q * 32, 0, 0);  // local partial [T, N]
              else tma_store_4d(&peer_maps.m[dest], sbuf_ptr, c_in, fp.rank * fp.slot_rows + r_in + q * 32, 0, 0);
            } else {
              tma_store_4d(pass == 0 ? &tmAux : &tmC, sbuf_ptr, col0, m0 + q * 32, bi, bo);
            }
            tma_store_commit();
          }
          sbuf ^= 1;
        }
      }
      if constexpr ((MODE & kModeReduceScatter) != 0) {
        // The partial tile went into the owner's slot buffer.  Count this warp's finished quarter-tiles per row chunk
        // and publish the count when the warp moves on to another chunk (or runs out of tiles): wait for its TMA
        // stores to be complete, then one atomic; the warp that completes a chunk raises the flag on the owner,
        // whose reducer CTAs then sum the tp slots of that chunk out of their local memory.
        const int chunk = rs_dest * fp.cps + rs_c;
        const int next_tile = tile + num_ctas;
        int next_chunk = -1;
        if (next_tile < num_tiles) {
          int nb2, mb2, b2, d2, c2;
          fused_tile_coords<MODE>(next_tile, p, fp, b2, mb2, nb2);
          rs_tile_owner(fp, mb2 * kBlockM, nb2 * BLOCK_N, d2, c2);
          next_chunk = d2 * fp.cps + c2;
        }
        if (!rs_own) ++rs_pending;
        if (next_chunk != chunk && rs_pending > 0) {
          if (lane == 0) {
            tma_store_wait_all();
            fence_proxy_async_global();
            __threadfence_system();
            const int need = fp.tiles_per_chunk * 4;
            const int old = atomicAdd(fp.tile_done + chunk, rs_pending);
            if (old + rs_pending == need) {
              fp.tile_done[chunk] = 0;
              __threadfence_system();
              st_release_sys(fp.peer_rs_flag[rs_dest] + fp.rank * fp.cps + rs_c, fp.epoch);
            }
          }
          rs_pending = 0;
        }
        __syncwarp();
      }
      buf ^= 1;
      if (buf == 0) acc_phase ^= 1;
    }
    if (lane == 0) tma_store_wait_all();
    if (MODE != kModePlain && fp.debug_times && cta == 0 && warp == 2 && lane == 0) fp.debug_times[5] = global_timer_ns();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver call and needs a current context in the calling thread; worker threads
// (e.g. the autograd engine's) may not have one yet.  Re-selecting the runtime's current device binds the
// primary context to this thread.
static inline void bind_context_to_thread() {
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
}

static inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 4-D map over a [batch_outer, batch_inner, rows, cols] tensor (cols contiguous), 128-byte swizzle.
static inline int make_map(CUtensorMap* map, const void* base, int is_bf16, long long cols, long long rows, long long b_inner,
                    long long b_outer, long long row_stride_elems, long long inner_stride_elems,
                    long long outer_stride_elems, int box_cols, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)b_inner, (cuuint64_t)b_outer};
  const long long dflt = row_stride_elems * rows;
  cuuint64_t strides[3] = {(cuuint64_t)row_stride_elems * 2,
                           (cuuint64_t)(b_inner > 1 ? inner_stride_elems : dflt) * 2,
                           (cuuint64_t)(b_outer > 1 ? outer_stride_elems : dflt * b_inner) * 2};
  cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "oslo_b200: cuTensorMapEncodeTiled failed (%d): base %p dims {%llu,%llu,%llu,%llu} strides {%llu,%llu,%llu} box {%u,%u}\n",
            (int)r, base, (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
            (unsigned long long)dims[3], (unsigned long long)strides[0], (unsigned long long)strides[1],
            (unsigned long long)strides[2], box[0], box[1]);
    return -2;
  }
  return 0;
}

template <int BLOCK_N, bool A_MN, bool B_MN, int MODE = kModePlain>
static int launch(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const CUtensorMap& aux,
                  const GemmParams& p, int grid, cudaStream_t stream, const FusedParams& fp = FusedParams(),
                  const PeerMaps* peer_maps = nullptr) {
  using Cfg = GemmCfg<BLOCK_N>;
  auto kern = gemm_tcgen05_kernel<BLOCK_N, A_MN, B_MN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return -3;
    configured = true;
  }
  PeerMaps pm;
  if (peer_maps) pm = *peer_maps;
  else for (int i = 0; i < kMaxRanks; ++i) pm.m[i] = c;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(a, b, c, aux, p, fp, pm);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace oslo


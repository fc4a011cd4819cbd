// Fused compute + collective entry points for 1-D tensor parallelism with sequence parallelism:
//
//   oslo_ag_gemm   C[T, N] = all_gather(x_shard)[T, K] x B[N, K]^T, also leaving the gathered x in local memory
//   oslo_gemm_rs   out[T/tp, N] = reduce_scatter_rows( A[T, K] x B[N, K]^T )
//
// Both are ONE launch of the tcgen05 GEMM kernel in a fused mode (gemm_core.cuh):
//   * all-gather: a few CTAs PUSH this rank's shard into the gathered buffer of every rank (bulk stores to peer memory;
//     posted writes are not bound by the NVLink round trip the way remote reads are) while the remaining CTAs multiply,
//     starting with the local shard and taking each remote row chunk as soon as its source has flagged it; TMA loads
//     only ever read local memory.
//   * reduce-scatter: tiles are computed in destination order (next rank first, own rows last).  The epilogue of a
//     tile of another rank's rows TMA-stores the partial tile straight into slot [this rank] of the OWNER's slot
//     buffer (a plain bulk tensor store to peer memory) and flags each finished chunk of rows there; the epilogue of
//     a tile of our own rows adds the other ranks' partial rows (already in our slot buffer) to the accumulator and
//     stores the final result, so no separate reduction pass exists.
// All waits on peers are bounded (~2 s) and report through the status word instead of hanging.
//
// Replaces ColLinear1D / RowLinear1D = F.linear + a separate NCCL all-reduce in the reference
// (oslo/torch/nn/modules/linear.py:73-160).
#include "gemm_core.cuh"

using namespace oslo;

static int pick_block_n(int M, int N, int ctas, int max_bn) {
  const long long mb = (M + kBlockM - 1) / kBlockM;
  auto tiles = [&](int bn) { return mb * ((N + bn - 1) / bn); };
  int bn = 256;
  if (tiles(256) < ctas || N % 256 != 0 || max_bn < 256) bn = 128;
  if (N <= 64) bn = 64;
  return bn;
}

// Rows per hand-off chunk of the all-gather side: about 1024, at most 64 chunks over all shards, always a multiple of 128
// dividing the shard.  Exported so that a host-driven transport flags the same chunks the kernel waits for.
static int ag_chunk_rows(int Tl, int tp) {
  int chunk_rows = Tl;
  for (int cand = 1024; cand >= kBlockM; cand -= kBlockM) {
    if (Tl % cand == 0 && (Tl / cand) * tp <= 64) { chunk_rows = cand; break; }
  }
  return chunk_rows;
}
extern "C" int oslo_ag_chunk_rows(int Tl, int tp) { return (Tl > 0 && tp > 0 && Tl % kBlockM == 0) ? ag_chunk_rows(Tl, tp) : -1; }

#define OSLO_FUSED_LAUNCH(BN, MODE)                                                                       \
  (b_mn ? launch<BN, false, true, MODE>(ta, tb, tc, taux, p, grid, stream, fp, peer_maps_ptr)             \
        : launch<BN, false, false, MODE>(ta, tb, tc, taux, p, grid, stream, fp, peer_maps_ptr))

// x_shard: this rank's [T/tp, K] rows (any 16-byte aligned local memory).  peer_xfull / peer_chunk_flag: host arrays of
// `tp` device pointers to every rank's gathered buffer [T, K] and chunk-flag array (entry [rank] is the local one).
extern "C" int oslo_ag_gemm(const void* x_shard, void* const* peer_xfull, const void* B, void* C, const void* bias, int T, int N,
                            int K, long long ldb, int b_mn, int is_bf16, int tp, int rank, int epoch,
                            void* const* peer_chunk_flag, int* chunk_arrive, int copy_ctas, int num_sms, int* status,
                            void* stream_ptr, const int* epoch_ptr, void* mc_xfull, int external_push,
                            const void* gelu_grad_aux) {
  // gelu_grad_aux: optional [T, N] pre-activation; the product is multiplied by gelu'(aux) in the epilogue (the backward of
  // a bias-GELU linear whose incoming gradient is this product) and no bias may be given then.
  // external_push: the shards are delivered (and the chunk flags raised) by somebody else, e.g. copy-engine transfers on
  // other streams: no CTA copies, all of them multiply and take remote row chunks as their flags come up.
  // mc_xfull: the same gathered buffer through an NVSwitch multicast mapping over the group (or null): the copy CTAs then
  // store each piece of the shard once, to that address, instead of once per peer.
  if (tp > kMaxRanks || tp < 1 || T % tp) return -1;
  const int Tl = T / tp;
  if (Tl % kBlockM || N % 8 || K % 8 || ldb % 8 || (reinterpret_cast<uintptr_t>(x_shard) & 15)) return -5;
  bind_context_to_thread();
  if (external_push) {
    copy_ctas = 0;
    mc_xfull = nullptr;
  } else {
    if (copy_ctas < 1) copy_ctas = 1;
    if (copy_ctas > num_sms / 2) copy_ctas = num_sms / 2;
  }
  const int gemm_ctas_max = num_sms - copy_ctas;
  const int block_n = pick_block_n(T, N, gemm_ctas_max, 256);
  GemmParams p{};
  p.M = T; p.N = N; p.K = K; p.batch = 1; p.batch_inner = 1; p.causal = 0;
  p.m_blocks = T / kBlockM;
  p.n_blocks = (N + block_n - 1) / block_n;
  if (gelu_grad_aux && (bias || (reinterpret_cast<uintptr_t>(gelu_grad_aux) & 15))) return -5;
  p.epilogue = gelu_grad_aux ? 3 : (bias ? 1 : 0); p.accumulate = 0; p.is_bf16 = is_bf16;
  p.bias = bias; p.c_ptr = C; p.ldc = N; p.stride_c = 0; p.stride_c_outer = 0;
  p.aux_ptr = const_cast<void*>(gelu_grad_aux); p.status = status;
  FusedParams fp;
  fp.tp = tp; fp.rank = rank; fp.shard_rows = Tl; fp.epoch = epoch; fp.copy_ctas = copy_ctas; fp.k_elems = K;
  fp.tiles_per_shard = (Tl / kBlockM) * p.n_blocks;
  const int chunk_rows = ag_chunk_rows(Tl, tp);
  fp.chunk_rows = chunk_rows;
  fp.ag_tp = tp; fp.ag_rank = rank; fp.ag_shard_rows = Tl; fp.ag_chunk_rows = chunk_rows; fp.ag_epoch = epoch;
  fp.ag_epoch_ptr = epoch_ptr;
  for (int i = 0; i < tp; ++i) {
    fp.peer_xfull[i] = peer_xfull[i];
    fp.peer_chunk_flag[i] = static_cast<int*>(peer_chunk_flag[i]);
  }
  fp.peer_in[rank] = x_shard;
  void* x_full = peer_xfull[rank];
  fp.x_full = x_full;
  fp.mc_xfull = mc_xfull;
  fp.chunk_flag = static_cast<int*>(peer_chunk_flag[rank]); fp.chunk_arrive = chunk_arrive; fp.status = status; fp.epoch_ptr = epoch_ptr;
  CUtensorMap ta, tb, tc, taux;
  int rc = make_map(&ta, x_full, is_bf16, K, T, 1, 1, K, 0, 0, kBlockK, kBlockM);
  if (rc) return rc;
  rc = make_map(&taux, x_shard, is_bf16, K, Tl, 1, 1, K, 0, 0, kBlockK, kBlockM);  // local shard, read in place
  if (rc) return rc;
  if (b_mn) rc = make_map(&tb, B, is_bf16, N, K, 1, 1, ldb, 0, 0, 64, kBlockK);
  else      rc = make_map(&tb, B, is_bf16, K, N, 1, 1, ldb, 0, 0, kBlockK, block_n);
  if (rc) return rc;
  rc = make_map(&tc, C, is_bf16, N, T, 1, 1, N, 0, 0, 64, 32);
  if (rc) return rc;
  const long long total = (long long)p.m_blocks * p.n_blocks;
  const int gemm_ctas = (int)(total < gemm_ctas_max ? total : gemm_ctas_max);
  const int grid = copy_ctas + gemm_ctas;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const PeerMaps* peer_maps_ptr = nullptr;
  switch (block_n) {
    case 256: return OSLO_FUSED_LAUNCH(256, kModeAllGather);
    case 128: return OSLO_FUSED_LAUNCH(128, kModeAllGather);
    default: return OSLO_FUSED_LAUNCH(64, kModeAllGather);
  }
}

// peer_partial / peer_rs_flag: host arrays of `tp` device pointers (slot buffers [tp, T/tp, N] and flag arrays of
// tp * chunks_per_shard ints).  A: [T, K] K-major (lda), out: [T/tp, N].  addend: optional local [T, N] (see below).
extern "C" int oslo_gemm_rs(const void* A, long long lda, const void* B, long long ldb, int b_mn, void* out, const void* bias,
                            int T, int N, int K, int is_bf16, int tp, int rank, int epoch, void* const* peer_partial,
                            void* const* peer_rs_flag, int* tile_done, int reduce_ctas, int num_sms, int* status,
                            void* stream_ptr, unsigned long long* debug_times, const int* epoch_ptr, const void* addend,
                            int along_n, const void* mc_partial) {
  // mc_partial: this call's partial buffer through an NVSwitch multicast mapping over the group (or null).  With it (row
  // scatter only) every rank stores its partial tiles into its OWN buffer and `reduce_ctas` CTAs of the owner read the
  // sums with multimem.ld_reduce; without it partial tiles are stored into the owner's slots and its own tiles fold them.
  // along_n = 0: out[T/tp, N], the ROWS of the product are scattered (1-D sequence parallelism, 3-D);
  // along_n = 1: out[T, N/tp], the COLUMNS are scattered (2-D / 2.5-D SUMMA: every rank keeps its tokens).
  if (tp > kMaxRanks || tp < 1) return -1;
  if (along_n ? (N % tp != 0) : (T % tp != 0)) return -1;
  const int Tl = along_n ? T : T / tp;       // rows of one rank's output
  const int Nl = along_n ? N / tp : N;       // columns of one rank's output
  if (T % kBlockM || Tl % kBlockM || N % 8 || Nl % 8 || K % 8 || lda % 8 || ldb % 8) return -5;
  if (addend && (reinterpret_cast<uintptr_t>(addend) & 15)) return -5;
  if (along_n && bias) return -5;  // the owner-side bias is indexed by global column: add it outside in this layout
  bind_context_to_thread();
  if (along_n) mc_partial = nullptr;
  if (mc_partial) {
    if (reduce_ctas < 1) reduce_ctas = 1;
    if (reduce_ctas > num_sms / 2) reduce_ctas = num_sms / 2;
  } else {
    reduce_ctas = 0;  // the reduction is folded into the epilogue of the tiles of our own block
  }
  const int gemm_ctas_max = num_sms - reduce_ctas;
  int block_n = pick_block_n(T, N, gemm_ctas_max, 256);
  if (along_n) {
    // a tile must not straddle two owners
    while (block_n > 64 && Nl % block_n) block_n /= 2;
    if (Nl % block_n) return -5;
  }
  GemmParams p{};
  p.M = T; p.N = N; p.K = K; p.batch = 1; p.batch_inner = 1; p.causal = 0;
  p.m_blocks = T / kBlockM;
  p.n_blocks = (N + block_n - 1) / block_n;
  p.epilogue = bias ? 1 : 0; p.is_bf16 = is_bf16;
  // `addend`: a local, contiguous [T, N] partial product of this rank that is summed into every tile before it leaves
  // (two row-parallel products that feed one reduce-scatter cross NVLink once)
  p.accumulate = addend ? 1 : 0;
  p.bias = bias; p.c_ptr = addend ? const_cast<void*>(addend) : out; p.ldc = N; p.stride_c = 0; p.stride_c_outer = 0;
  p.aux_ptr = nullptr;
  p.status = status;
  FusedParams fp;
  fp.tp = tp; fp.rank = rank; fp.shard_rows = Tl; fp.epoch = epoch; fp.copy_ctas = reduce_ctas;
  fp.rs_along_n = along_n; fp.shard_cols = Nl; fp.n_blocks_per_shard = along_n ? Nl / block_n : p.n_blocks;
  fp.tiles_per_shard = (Tl / kBlockM) * fp.n_blocks_per_shard;
  int chunk_rows = Tl;  // hand-off granularity: about 512 rows, at most 64 flags in total
  for (int cand = 512; cand >= kBlockM; cand -= kBlockM) {
    if (Tl % cand == 0 && (Tl / cand) * tp <= 64) { chunk_rows = cand; break; }
  }
  if ((Tl / chunk_rows) * tp > 64) return -5;
  fp.chunk_rows = chunk_rows;
  fp.cps = Tl / chunk_rows;
  fp.slot_rows = Tl; fp.slot_ld = Nl;
  fp.tiles_per_chunk = (chunk_rows / kBlockM) * fp.n_blocks_per_shard;
  for (int i = 0; i < tp; ++i) {
    fp.peer_slots[i] = peer_partial[i];
    fp.peer_rs_flag[i] = static_cast<int*>(peer_rs_flag[i]);
  }
  fp.rs_flag = static_cast<int*>(peer_rs_flag[rank]);
  fp.tile_done = tile_done; fp.rs_out = out; fp.rs_bias = bias; fp.status = status; fp.debug_times = debug_times; fp.epoch_ptr = epoch_ptr;
  fp.mc_slots = mc_partial;
  CUtensorMap ta, tb, tc, taux;
  int rc = make_map(&ta, A, is_bf16, K, T, 1, 1, lda, 0, 0, kBlockK, kBlockM);
  if (rc) return rc;
  if (b_mn) rc = make_map(&tb, B, is_bf16, N, K, 1, 1, ldb, 0, 0, 64, kBlockK);
  else      rc = make_map(&tb, B, is_bf16, K, N, 1, 1, ldb, 0, 0, kBlockK, block_n);
  if (rc) return rc;
  // one store map per destination: rank d's slot buffer viewed [tp * Tl, Nl]; our block goes to slot [rank]
  PeerMaps maps;
  for (int d = 0; d < kMaxRanks; ++d) {
    rc = make_map(&maps.m[d], peer_partial[d < tp ? d : rank], is_bf16, Nl, (long long)tp * Tl, 1, 1, Nl, 0, 0, 64, 32);
    if (rc) return rc;
  }
  const PeerMaps* peer_maps_ptr = &maps;
  rc = make_map(&tc, out, is_bf16, Nl, Tl, 1, 1, Nl, 0, 0, 64, 32);  // final block of this rank
  if (rc) return rc;
  taux = tc;
  const long long total = (long long)p.m_blocks * p.n_blocks;
  const int gemm_ctas = (int)(total < gemm_ctas_max ? total : gemm_ctas_max);
  const int grid = reduce_ctas + gemm_ctas;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  switch (block_n) {
    case 256: return OSLO_FUSED_LAUNCH(256, kModeReduceScatter);
    case 128: return OSLO_FUSED_LAUNCH(128, kModeReduceScatter);
    default: return OSLO_FUSED_LAUNCH(64, kModeReduceScatter);
  }
}


// All-gather of the A rows over one group, GEMM, reduce-scatter of the product's rows over ANOTHER group, in one launch:
//
//     out[T/rs_tp, N] = reduce_scatter_rows_over_RS( all_gather_rows_over_AG(x_shard)[T, K] x B[N, K]^T )
//
// (the 3-D tensor-parallel linear: activations gathered over the INPUT group, partial products reduced over the OUTPUT
// group; both groups cut the token dimension into the same blocks).  The two sides keep separate flags and epochs, one
// symmetric workspace per group.  x_full receives the gathered activations for the backward pass.
extern "C" int oslo_ag_gemm_rs(const void* x_shard, void* const* peer_xfull, const void* B, long long ldb, int b_mn, void* out, int T,
                               int N, int K, int is_bf16, int ag_tp, int ag_rank, int ag_epoch, void* const* peer_chunk_flag,
                               int* chunk_arrive, const int* ag_epoch_ptr, int rs_tp, int rs_rank, int rs_epoch,
                               void* const* peer_partial, void* const* peer_rs_flag, int* tile_done, const int* rs_epoch_ptr,
                               int copy_ctas, int num_sms, int* status, void* stream_ptr) {
  if (ag_tp > kMaxRanks || rs_tp > kMaxRanks || ag_tp < 1 || rs_tp < 1 || T % ag_tp || T % rs_tp) return -1;
  if (ag_tp != rs_tp) return -1;  // both groups cut the rows into the same blocks
  const int Tl = T / rs_tp;
  if (Tl % kBlockM || N % 8 || K % 8 || ldb % 8 || (reinterpret_cast<uintptr_t>(x_shard) & 15)) return -5;
  bind_context_to_thread();
  if (copy_ctas < 1) copy_ctas = 1;
  if (copy_ctas > num_sms / 2) copy_ctas = num_sms / 2;
  const int gemm_ctas_max = num_sms - copy_ctas;
  const int block_n = pick_block_n(T, N, gemm_ctas_max, 256);
  GemmParams p{};
  p.M = T; p.N = N; p.K = K; p.batch = 1; p.batch_inner = 1; p.causal = 0;
  p.m_blocks = T / kBlockM;
  p.n_blocks = (N + block_n - 1) / block_n;
  p.epilogue = 0; p.accumulate = 0; p.is_bf16 = is_bf16;
  p.bias = nullptr; p.c_ptr = out; p.ldc = N; p.stride_c = 0; p.stride_c_outer = 0; p.aux_ptr = nullptr; p.status = status;
  FusedParams fp;
  // reduce-scatter side (also the tile order: the next rank's rows first, our own last)
  fp.tp = rs_tp; fp.rank = rs_rank; fp.shard_rows = Tl; fp.epoch = rs_epoch; fp.epoch_ptr = rs_epoch_ptr;
  fp.copy_ctas = copy_ctas; fp.k_elems = K;
  fp.n_blocks_per_shard = p.n_blocks;
  fp.tiles_per_shard = (Tl / kBlockM) * p.n_blocks;
  int chunk_rows = Tl;
  for (int cand = 512; cand >= kBlockM; cand -= kBlockM) {
    if (Tl % cand == 0 && (Tl / cand) * rs_tp <= 64) { chunk_rows = cand; break; }
  }
  if ((Tl / chunk_rows) * rs_tp > 64) return -5;
  fp.chunk_rows = chunk_rows; fp.cps = Tl / chunk_rows; fp.slot_rows = Tl; fp.slot_ld = N;
  fp.tiles_per_chunk = (chunk_rows / kBlockM) * p.n_blocks;
  for (int i = 0; i < rs_tp; ++i) {
    fp.peer_slots[i] = peer_partial[i];
    fp.peer_rs_flag[i] = static_cast<int*>(peer_rs_flag[i]);
  }
  fp.rs_flag = static_cast<int*>(peer_rs_flag[rs_rank]);
  fp.tile_done = tile_done; fp.rs_out = out; fp.status = status;
  // all-gather side: the same row blocks; every rank pushes its block to all the others, chunk by chunk
  fp.ag_tp = ag_tp; fp.ag_rank = ag_rank; fp.ag_shard_rows = Tl; fp.ag_chunk_rows = chunk_rows; fp.ag_epoch = ag_epoch;
  fp.ag_epoch_ptr = ag_epoch_ptr;
  for (int i = 0; i < ag_tp; ++i) {
    fp.peer_xfull[i] = peer_xfull[i];
    fp.peer_chunk_flag[i] = static_cast<int*>(peer_chunk_flag[i]);
  }
  fp.peer_in[ag_rank] = x_shard;
  void* x_full = peer_xfull[ag_rank];
  fp.x_full = x_full;
  fp.chunk_flag = static_cast<int*>(peer_chunk_flag[ag_rank]); fp.chunk_arrive = chunk_arrive;
  CUtensorMap ta, tb, tc, taux;
  int rc = make_map(&ta, x_full, is_bf16, K, T, 1, 1, K, 0, 0, kBlockK, kBlockM);
  if (rc) return rc;
  rc = make_map(&taux, x_shard, is_bf16, K, Tl, 1, 1, K, 0, 0, kBlockK, kBlockM);  // own shard, read in place
  if (rc) return rc;
  if (b_mn) rc = make_map(&tb, B, is_bf16, N, K, 1, 1, ldb, 0, 0, 64, kBlockK);
  else      rc = make_map(&tb, B, is_bf16, K, N, 1, 1, ldb, 0, 0, kBlockK, block_n);
  if (rc) return rc;
  PeerMaps maps;
  for (int d = 0; d < kMaxRanks; ++d) {
    rc = make_map(&maps.m[d], peer_partial[d < rs_tp ? d : rs_rank], is_bf16, N, T, 1, 1, N, 0, 0, 64, 32);
    if (rc) return rc;
  }
  const PeerMaps* peer_maps_ptr = &maps;
  rc = make_map(&tc, out, is_bf16, N, Tl, 1, 1, N, 0, 0, 64, 32);
  if (rc) return rc;
  const long long total = (long long)p.m_blocks * p.n_blocks;
  const int gemm_ctas = (int)(total < gemm_ctas_max ? total : gemm_ctas_max);
  const int grid = copy_ctas + gemm_ctas;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  switch (block_n) {
    case 256: return OSLO_FUSED_LAUNCH(256, kModeGatherScatter);
    case 128: return OSLO_FUSED_LAUNCH(128, kModeGatherScatter);
    default: return OSLO_FUSED_LAUNCH(64, kModeGatherScatter);
  }
}

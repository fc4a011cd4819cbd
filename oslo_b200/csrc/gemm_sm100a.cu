// Plain (single-GPU) entry point of the tcgen05 GEMM; the kernel lives in gemm_core.cuh.
#include "gemm_core.cuh"

// C = epilogue(A x B^T) on the tcgen05 tensor cores.
//   a_mn / b_mn : 0 = operand stored [rows = M or N, K contiguous], 1 = stored [K rows, M or N contiguous]
//   lda/ldb/ldc : row strides in elements; stride_* : batch strides in elements
//   epilogue    : 0 none, 1 bias, 2 GELU(tanh) of (acc + bias); aux (optional) receives acc + bias
//   block_n     : 0 = choose, else 64 / 128 / 256
// Returns 0 on success, negative on a host-side error.  Device-side timeouts are
// reported in *status (int32 in device memory, may be null).
extern "C" int oslo_gemm_tcgen05(const void* A, const void* B, void* C, const void* bias, void* aux, int M, int N, int K,
                                 int batch, long long lda, long long ldb, long long ldc, long long stride_a,
                                 long long stride_b, long long stride_c, int a_mn, int b_mn, int is_bf16, int epilogue,
                                 int accumulate, int block_n, int num_sms, int* status, void* stream_ptr,
                                 int batch_outer, long long ostride_a, long long ostride_b, long long ostride_c,
                                 int causal) {
  using namespace oslo;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  bind_context_to_thread();
  if (batch_outer <= 0) batch_outer = 1;
  const int b_in = batch, b_out = batch_outer;
  batch = b_in * b_out;
  if (b_out > 1 && ((ostride_a % 8) || (ostride_b % 8) || (ostride_c % 8))) return -5;
  if (causal && (M != N && causal == 1)) return -7;
  // TMA needs 16-byte aligned bases and strides
  auto bad = [](long long v) { return (v % 8) != 0; };
  if (bad(lda) || bad(ldb) || bad(ldc) || (b_in > 1 && (bad(stride_a) || bad(stride_b) || bad(stride_c))) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15) || (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) || (N % 8) ||
      (a_mn && (M % 8)) || (!a_mn && (K % 8)) || (b_mn ? 0 : (K % 8)))
    return -5;
  if (b_in == 1 && b_out == 1) batch = 1;
  if (block_n == 0) {
    const long long mb = (M + kBlockM - 1) / kBlockM;
    auto tiles = [&](int bn) { return (long long)batch * mb * ((N + bn - 1) / bn); };
    block_n = 256;
    if (tiles(256) < num_sms) block_n = 128;
    if (tiles(128) < num_sms && block_n == 128) block_n = 64;
    if (N <= 64) block_n = 64;
    else if (N <= 128 && block_n > 128) block_n = 128;
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = batch; p.batch_inner = b_in; p.causal = causal; p.stride_c_outer = ostride_c;
  p.m_blocks = (M + kBlockM - 1) / kBlockM;
  p.n_blocks = (N + block_n - 1) / block_n;
  p.epilogue = epilogue; p.accumulate = accumulate; p.is_bf16 = is_bf16;
  p.bias = bias; p.c_ptr = C; p.ldc = ldc; p.stride_c = stride_c; p.aux_ptr = aux; p.status = status;
  CUtensorMap ta, tb, tc, taux;
  int rc;
  if (a_mn) rc = make_map(&ta, A, is_bf16, M, K, b_in, b_out, lda, stride_a, ostride_a, 64, kBlockK);
  else      rc = make_map(&ta, A, is_bf16, K, M, b_in, b_out, lda, stride_a, ostride_a, kBlockK, kBlockM);
  if (rc) return rc;
  if (b_mn) rc = make_map(&tb, B, is_bf16, N, K, b_in, b_out, ldb, stride_b, ostride_b, 64, kBlockK);
  else      rc = make_map(&tb, B, is_bf16, K, N, b_in, b_out, ldb, stride_b, ostride_b, kBlockK, block_n);
  if (rc) return rc;
  rc = make_map(&tc, C, is_bf16, N, M, b_in, b_out, ldc, stride_c, ostride_c, 64, 32);
  if (rc) return rc;
  if (aux) {
    if (reinterpret_cast<uintptr_t>(aux) & 15) return -5;
    rc = make_map(&taux, aux, is_bf16, N, M, b_in, b_out, ldc, stride_c, ostride_c, 64, 32);
    if (rc) return rc;
  } else {
    taux = tc;
  }
  const long long total = (long long)p.batch * p.m_blocks * p.n_blocks;
  const int grid = (int)(total < num_sms ? total : num_sms);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
#define OSLO_LAUNCH(BN)                                                                      \
  (a_mn ? (b_mn ? launch<BN, true, true>(ta, tb, tc, taux, p, grid, stream)                   \
                : launch<BN, true, false>(ta, tb, tc, taux, p, grid, stream))                 \
        : (b_mn ? launch<BN, false, true>(ta, tb, tc, taux, p, grid, stream)                  \
                : launch<BN, false, false>(ta, tb, tc, taux, p, grid, stream)))
  switch (block_n) {
    case 256: return OSLO_LAUNCH(256);
    case 128: return OSLO_LAUNCH(128);
    case 64: return OSLO_LAUNCH(64);
    default: return -6;
  }
#undef OSLO_LAUNCH
}

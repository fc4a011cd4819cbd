// N-gram repeat blocking for beam search: for every hypothesis, ban each token that would complete an n-gram
// already present in the hypothesis (sets its log-probability to -inf).
//
// One block per hypothesis; the generated prefix is staged in shared memory, every thread owns one start position
// and compares the (n-1)-token context there with the last n-1 generated tokens.
// Replaces oslo/torch/_C/csrc/ngram_repeat_block_cuda_kernel.cu:17-77 (which launches on the default stream).
#include "common.cuh"
#include <math_constants.h>

namespace oslo {

template <typename T>
__global__ void ngram_block_kernel(const long long* __restrict__ tokens, T* __restrict__ lprobs, int max_len, int step,
                                   int vocab, int n) {
  extern __shared__ long long prefix[];
  const int row = blockIdx.x;
  const long long* t = tokens + static_cast<size_t>(row) * max_len;
  for (int i = threadIdx.x; i <= step; i += blockDim.x) prefix[i] = t[i];
  __syncthreads();
  const int ctx = n - 1;  // tokens that must match
  const int last_start = step - ctx + 1;  // the current context occupies [last_start, step]
  for (int start = threadIdx.x; start + n - 1 <= step; start += blockDim.x) {
    bool same = true;
    for (int k = 0; k < ctx; ++k) {
      if (prefix[start + k] != prefix[last_start + k]) { same = false; break; }
    }
    if (same) {
      const long long banned = prefix[start + ctx];
      if (banned >= 0 && banned < vocab) lprobs[static_cast<size_t>(row) * vocab + banned] = static_cast<T>(-CUDART_INF_F);
    }
  }
}

}  // namespace oslo

// tokens: [rows, max_len] int64 (rows = batch * beam), step = index of the last generated token,
// lprobs: [rows, vocab] in fp32 (0) / fp16 (1) / bf16 (2), modified in place.
extern "C" int oslo_ngram_repeat_block(const long long* tokens, void* lprobs, int rows, int max_len, int step, int vocab, int n,
                                       int dtype, void* stream) {
  if (rows <= 0 || n <= 0 || step + 1 < n) return 0;
  const int threads = step + 1 < 1024 ? ((step + 1 + 31) / 32 * 32) : 1024;
  const size_t smem = static_cast<size_t>(step + 1) * sizeof(long long);
  if (smem > 200 * 1024) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  using namespace oslo;
  if (dtype == 0) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(ngram_block_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ngram_block_kernel<float><<<rows, threads, smem, st>>>(tokens, (float*)lprobs, max_len, step, vocab, n);
  } else if (dtype == 1) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(ngram_block_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ngram_block_kernel<__half><<<rows, threads, smem, st>>>(tokens, (__half*)lprobs, max_len, step, vocab, n);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(ngram_block_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ngram_block_kernel<__nv_bfloat16><<<rows, threads, smem, st>>>(tokens, (__nv_bfloat16*)lprobs, max_len, step, vocab, n);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

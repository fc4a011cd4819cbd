// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
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
  int epilogue;       // 0 none, 1 +bias, 2 gelu(+bias if given), 3 reserved
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

// k-block range [kb0, kb1) a tile has to reduce over, or skip = true when it has no work.
OSLO_DEVINL void tile_k_range(const GemmParams& p, int m0, int n0, int num_kb, int& kb0, int& kb1, bool& skip) {
  kb0 = 0;
  kb1 = num_kb;
  skip = false;
  if (p.causal == 1) skip = n0 > m0 + kBlockM - 1;
  else if (p.causal == 2) kb1 = min(num_kb, (m0 + kBlockM + kBlockK - 1) / kBlockK);
  else if (p.causal == 3) kb0 = min(num_kb - 1, m0 / kBlockK);
}

template <int BLOCK_N, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux,
                    const GemmParams p) {
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
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int b, mb, nb;
        tile_coords(tile, p, b, mb, nb);
        const int m0 = mb * kBlockM, n0 = nb * BLOCK_N;
        const int bi = b % p.batch_inner, bo = b / p.batch_inner;
        int kb0, kb1;
        bool skip;
        tile_k_range(p, m0, n0, num_kb, kb0, kb1, skip);
        if (skip) continue;
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
            tma_load_4d(sa, &tmA, &full_bar[stage], k0, m0, bi, bo);
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
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
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
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int b, mb, nb;
      tile_coords(tile, p, b, mb, nb);
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
#pragma unroll 1
      for (int chunk = 0; chunk < BLOCK_N / 64; ++chunk) {
        uint32_t r0[32], r1[32];
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
        if (p.bias != nullptr) {
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
        const bool want_aux = (p.aux_ptr != nullptr);
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
            tma_store_4d(pass == 0 ? &tmAux : &tmC, sbuf_ptr, col0, m0 + q * 32, bi, bo);
            tma_store_commit();
          }
          sbuf ^= 1;
        }
      }
      buf ^= 1;
      if (buf == 0) acc_phase ^= 1;
    }
    if (lane == 0) tma_store_wait_all();
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

static EncodeTiledFn get_encode_fn() {
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
static int make_map(CUtensorMap* map, const void* base, int is_bf16, long long cols, long long rows, long long b_inner,
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
  return r == CUDA_SUCCESS ? 0 : -2;
}

template <int BLOCK_N, bool A_MN, bool B_MN>
static int launch(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const CUtensorMap& aux,
                  const GemmParams& p, int grid, cudaStream_t stream) {
  using Cfg = GemmCfg<BLOCK_N>;
  auto kern = gemm_tcgen05_kernel<BLOCK_N, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return -3;
    configured = true;
  }
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(a, b, c, aux, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace oslo

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

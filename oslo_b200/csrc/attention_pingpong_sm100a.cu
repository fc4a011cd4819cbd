// Fused attention forward for sm_100a, one pass with online softmax: two 128-row query tiles per CTA take turns on the tensor
// cores ("ping-pong"), the probabilities go back to the MMA through tensor memory, and the output accumulator is rescaled
// only when a row maximum grows by more than 2^8.
//
// One CTA handles one (batch, head, 256-query block):
//
//   warp 0      TMA producer: both Q tiles once, then K and V tiles through 2-stage rings
//   warp 1      MMA issuer.  Per key tile j and query tile t:  S_t = Q_t K_j^T (operands in shared memory, accumulator in
//               tensor memory), then O_t += P_t V_j with P_t read from tensor memory (it overwrites S_t in place as packed
//               16-bit pairs) and V_j from shared memory.  Issue order  PV_0j  QK_0(j+1)  PV_1j  QK_1(j+1)  keeps the tensor
//               pipe busy with one query tile while the softmax warps work on the other.
//   warps 2-5   softmax of query tile 0, one thread per row;  warps 6-9  the same for query tile 1.
//
// Tensor memory (512 columns): S_0 / P_0 [0,128)  S_1 / P_1 [128,256)  O_0 [256,256+HD)  O_1 [384,384+HD).
//
// Online softmax with a lazy rescale: a row keeps the maximum m it last scaled by.  When a tile's maximum exceeds m by more
// than 8 (in the log2 domain) the row's sum and its O accumulator are multiplied by 2^(m - m_new) before the tile is added;
// otherwise the exponentials are taken against the old m (they stay below 2^8, exact enough in bf16 and fp16, sums in fp32).
// The rescale is done by the softmax warp itself: it waits for the previous P V product of its tile, multiplies its 32 rows
// of O in tensor memory, and only then publishes P.  The final O / sum and the row log-sum-exp (for the backward pass) are
// written once per row.  All waits are bounded.
//
// Replaces the unfused QK^T -> mask -> softmax -> dropout -> PV chains of the reference
// (oslo/transformers/models/gpt2/modeling_gpt2.py:113-165; lightseq2 csrc/layers_new/sdpa_layer.cpp:10-66).
#include <cstdio>

#include "gemm_core.cuh"

namespace oslo {

constexpr int kPPRows = 128;        // rows of one query tile and of one key tile
constexpr int kPPThreads = 320;     // producer warp, MMA warp, 2 x 4 softmax warps
constexpr float kPPRescaleGap = 8.0f;

// 2^x on the special-function unit in one instruction (flushes denormals; 2^-inf = 0)
OSLO_DEVINL float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// max of three in one instruction
OSLO_DEVINL float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

struct AttnPPParams {
  int batch, heads, seq;
  int causal;
  float scale_log2;  // scale * log2(e)
  int is_bf16;
  float* lse;        // [batch, heads, seq] natural-log row log-sum-exp of the scaled scores
  int* status;
};

template <int HD>
struct AttnPPCfg {
  static constexpr int kHalves = HD / 64;            // 64-column swizzled halves of a [128, HD] tile
  static constexpr int kTile = kPPRows * HD * 2;      // bytes of a Q / K / V tile
  static constexpr int kSmem = 2 * kTile /*Q0 Q1*/ + 2 * kTile /*K ring*/ + 2 * kTile /*V ring*/ + 1024 + 256;
  static constexpr int kTmemCols = 512;
};

template <int HD>
__global__ void __launch_bounds__(kPPThreads, 1)
attention_fwd_pingpong_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                              const AttnPPParams p) {
  using Cfg = AttnPPCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                     // two tiles
  uint8_t* sK = sQ + 2 * Cfg::kTile;      // two stages
  uint8_t* sV = sK + 2 * Cfg::kTile;      // two stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * Cfg::kTile);
  uint64_t* q_full = bars;          // [1]
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2]  per query tile: scores of the next key tile are in tensor memory
  uint64_t* p_full = bars + 11;     // [2]  per query tile: probabilities written (4 warp arrivals)
  uint64_t* o_done = bars + 13;     // [2]  per query tile: a P V product has completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblocks = p.seq / (2 * kPPRows);
  // heavy (late) query blocks first so the causal triangle balances across the grid
  const int qb = qblocks - 1 - static_cast<int>(blockIdx.x % qblocks);
  const int bh = blockIdx.x / qblocks;
  const int h = bh % p.heads, b = bh / p.heads;
  const int q0 = qb * 2 * kPPRows;
  // key tiles seen by query tile 0 / 1 (causal: up to and including the tile's own diagonal block)
  const int nkv0 = p.causal ? 2 * qb + 1 : p.seq / kPPRows;
  const int nkv1 = p.causal ? 2 * qb + 2 : p.seq / kPPRows;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&o_done[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmO);
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
    // ---------------------------------------------------------------------------------------- TMA producer
    if (elect_one()) {
      bool ok = true;
      mbar_arrive_expect_tx(q_full, 2 * Cfg::kTile);
      for (int t = 0; t < 2; ++t)
        for (int c = 0; c < Cfg::kHalves; ++c)
          tma_load_4d(sQ + t * Cfg::kTile + c * 16384, &tmQ, q_full, c * 64, q0 + t * kPPRows, h, b);
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < nkv1 && ok; ++j) {
        if (!mbar_wait_bounded(&k_empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[st], Cfg::kTile);
        for (int c = 0; c < Cfg::kHalves; ++c)
          tma_load_4d(sK + st * Cfg::kTile + c * 16384, &tmK, &k_full[st], c * 64, j * kPPRows, h, b);
        if (!mbar_wait_bounded(&v_empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&v_full[st], Cfg::kTile);
        // MN-major operand: [k-block of 64 key rows][64-wide head-dim chunk][64 rows x 128 B]
        for (int kb = 0; kb < 2; ++kb)
          for (int c = 0; c < Cfg::kHalves; ++c)
            tma_load_4d(sV + st * Cfg::kTile + kb * (Cfg::kHalves * 8192) + c * 8192, &tmV, &v_full[st], c * 64,
                        j * kPPRows + kb * 64, h, b);
        if (++st == 2) { st = 0; ph ^= 1; }
      }
      if (!ok && p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutProducer);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc_f16(kPPRows, kPPRows, p.is_bf16 != 0, false, false);
      const uint32_t idesc_o = make_idesc_f16(kPPRows, HD, p.is_bf16 != 0, false, true);
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag);
      auto issue_s = [&](int t, int stage) {  // S_t = Q_t K^T with the K tile of `stage`
        const uint32_t q_addr = smem_u32(sQ + t * Cfg::kTile);
        const uint32_t k_addr = smem_u32(sK + stage * Cfg::kTile);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const int half = kk / 4, k = kk % 4;
          umma_f16(tmem_base + t * 128, make_smem_desc_sw128(q_addr + half * 16384 + k * 32, 16, 1024),
                   make_smem_desc_sw128(k_addr + half * 16384 + k * 32, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      // key tile 0 feeds the first scores of both query tiles
      if (ok) ok = mbar_wait_bounded(&k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        issue_s(1, 0);
        umma_commit(&k_empty[0]);
      }
      int st = 0;            // ring stage of key / value tile j
      uint32_t ph = 0;       // its phase
      for (int j = 0; j < nkv1 && ok; ++j) {
        const int nst = st ^ 1;
        const uint32_t nph = (st == 1) ? (ph ^ 1) : ph;  // phase of tile j + 1
        bool k_next_ready = false;
        if (!mbar_wait_bounded(&v_full[st], ph, abort_flag)) { ok = false; break; }
        const uint32_t v_addr = smem_u32(sV + st * Cfg::kTile);
        for (int t = 0; t < 2 && ok; ++t) {
          const int nkv = t == 0 ? nkv0 : nkv1;
          if (j >= nkv) continue;
          if (!mbar_wait_bounded(&p_full[t], static_cast<uint32_t>(j & 1), abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kPPRows / 16; ++kk) {
            const int half = kk / 4, k = kk % 4;
            umma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8,
                        make_smem_desc_sw128(v_addr + half * (Cfg::kHalves * 8192) + k * 2048, 8192, 1024), idesc_o,
                        (j > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&o_done[t]);
          if (j + 1 < nkv) {
            if (!k_next_ready) {
              if (!mbar_wait_bounded(&k_full[nst], nph, abort_flag)) { ok = false; break; }
              tc_fence_after();
              k_next_ready = true;
            }
            issue_s(t, nst);
          }
        }
        if (!ok) break;
        umma_commit(&v_empty[st]);
        if (k_next_ready) umma_commit(&k_empty[nst]);
        st = nst;
        ph = nph;
      }
      if (!ok && p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutMma);
    }
  } else {
    // -------------------------------------------------------------------------------------- softmax warps
    const int t = (warp - 2) >> 2;            // query tile of this warp group
    const int q = warp & 3;                   // tensor-memory lane quarter this warp may access
    const int row = q * 32 + lane;            // row inside the query tile
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_base + t * 128;
    const uint32_t tmem_o = tmem_base + lane_base + 256 + t * 128;
    const int nkv = t == 0 ? nkv0 : nkv1;
    const int diag_j = 2 * qb + t;            // key tile on this query tile's diagonal
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      if (!mbar_wait_bounded(&s_full[t], static_cast<uint32_t>(j & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = p.causal && j == diag_j;
      // ---- pass A: row maximum.  32 columns at a time through two register buffers (the load of the next chunk is in
      // flight while this one is reduced), four independent maxima so the reduction is not one dependent chain.
      float bm4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      {
        uint32_t ra[32], rb[32];
        __syncwarp();
        tmem_ld_32x32(tmem_s, ra);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t(&cur)[32] = (c & 1) ? rb : ra;
          uint32_t(&nxt)[32] = (c & 1) ? ra : rb;
          tmem_ld_wait();
          if (c < 3) tmem_ld_32x32(tmem_s + (c + 1) * 32, nxt);
          if (diag) {  // warp-uniform: only the tile on the diagonal pays for the mask
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i <= row) bm4[i & 3] = fmaxf(bm4[i & 3], __uint_as_float(cur[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) bm4[(i >> 1) & 3] = fmax3(bm4[(i >> 1) & 3], __uint_as_float(cur[i]), __uint_as_float(cur[i + 1]));
          }
        }
      }
      const float bm = fmaxf(fmaxf(bm4[0], bm4[1]), fmaxf(bm4[2], bm4[3])) * p.scale_log2;
      const bool grow = bm > m + kPPRescaleGap;  // always true on the first tile (m = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? bm : m;
        const float alpha = grow ? ex2_fast(m - m_new) : 1.0f;  // 0 on the first tile
        l *= alpha;
        m = m_new;
        if (j > 0) {
          // the previous P V product of this tile must have landed before its accumulator is touched
          if (!mbar_wait_bounded(&o_done[t], static_cast<uint32_t>((j - 1) & 1), abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_o + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      // ---- pass B: probabilities against the kept maximum.  The scores are read again 32 columns at a time (double
      // buffered), exponentiated, summed into four partial sums and written back packed two per 32-bit column: chunk c
      // lands in columns [16 c, 16 c + 16), always below the columns that are still to be read.
      {
        const float neg_m = -m;
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t ra[32], rb[32];
        __syncwarp();
        tmem_ld_32x32(tmem_s, ra);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t(&cur)[32] = (c & 1) ? rb : ra;
          uint32_t(&nxt)[32] = (c & 1) ? ra : rb;
          tmem_ld_wait();
          if (c < 3) tmem_ld_32x32(tmem_s + (c + 1) * 32, nxt);
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float a0 = ex2_fast(fmaf(__uint_as_float(cur[2 * i]), p.scale_log2, neg_m));
            float a1 = ex2_fast(fmaf(__uint_as_float(cur[2 * i + 1]), p.scale_log2, neg_m));
            if (diag) {
              if (c * 32 + 2 * i > row) a0 = 0.f;
              if (c * 32 + 2 * i + 1 > row) a1 = 0.f;
            }
            l4[i & 3] += a0 + a1;
            if (p.is_bf16) {
              // bf16 pair by integer arithmetic (round half up on the dropped 16 bits, then take the two high halves):
              // keeps the conversions off the special-function unit, which the exponentials already fill
              const uint32_t u0 = __float_as_uint(a0) + 0x8000u, u1 = __float_as_uint(a1) + 0x8000u;
              pk[i] = __byte_perm(u0, u1, 0x7632);
            } else {
              const __half2 hh = __floats2half2_rn(a0, a1);
              pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
            }
          }
          tmem_st_32x16(tmem_s + c * 16, pk);
        }
        l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    // epilogue: O / l -> shared (swizzled, over this tile's own Q which is no longer read) -> TMA store; log-sum-exp
    if (ok && mbar_wait_bounded(&o_done[t], static_cast<uint32_t>((nkv - 1) & 1), abort_flag)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      if (p.lse)
        p.lse[(static_cast<size_t>(b) * p.heads + h) * p.seq + q0 + t * kPPRows + row] = (m + log2f(l)) * 0.6931471805599453f;
      uint8_t* stage = sQ + t * Cfg::kTile + q * (Cfg::kHalves * 4096);  // 32 rows x (HD / 64) x 128 B per warp
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        __syncwarp();
        tmem_ld_32x32(tmem_o + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t packed[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float a0 = __uint_as_float(o[g * 8 + 2 * e]) * inv, a1 = __uint_as_float(o[g * 8 + 2 * e + 1]) * inv;
            if (p.is_bf16) { const __nv_bfloat162 hh = __floats2bfloat162_rn(a0, a1); packed[e] = *reinterpret_cast<const uint32_t*>(&hh); }
            else { const __half2 hh = __floats2half2_rn(a0, a1); packed[e] = *reinterpret_cast<const uint32_t*>(&hh); }
          }
          const int col = c * 32 + g * 8;
          const int half = col / 64, chunk = (col % 64) / 8;
          *reinterpret_cast<uint4*>(stage + half * 4096 + lane * 128 + ((chunk ^ (lane & 7)) << 4)) =
              make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        for (int half = 0; half < Cfg::kHalves; ++half)
          tma_store_4d(&tmO, stage + half * 4096, half * 64, q0 + t * kPPRows + q * 32, h, b);
        tma_store_commit();
        tma_store_wait_all();
      }
    } else if (p.status && lane == 0) {
      atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutEpilogue);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int HD>
static int launch_attention_pingpong(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
                                     const AttnPPParams& p, cudaStream_t stream) {
  using Cfg = AttnPPCfg<HD>;
  auto kern = attention_fwd_pingpong_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem) != cudaSuccess) return -3;
    configured = true;
  }
  const int grid = p.batch * p.heads * (p.seq / (2 * kPPRows));
  kern<<<grid, kPPThreads, Cfg::kSmem, stream>>>(tq, tk, tv, to, p);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    cudaFuncAttributes fa{};
    cudaFuncGetAttributes(&fa, kern);
    fprintf(stderr,
            "attention_fwd_pingpong launch refused: %s (grid %d, %d threads, %d B dynamic smem; kernel: %d regs, max %d "
            "threads / block, %zu B static smem, %d B max dynamic smem)\n",
            cudaGetErrorString(err), grid, kPPThreads, Cfg::kSmem, fa.numRegs, fa.maxThreadsPerBlock, fa.sharedSizeBytes,
            fa.maxDynamicSharedSizeBytes);
    return -(1000 + static_cast<int>(err));
  }
  return 0;
}

}  // namespace oslo

// q, k, v, o: [batch, seq, heads, head_dim] views given by element strides (token, head, batch); head_dim contiguous.
// seq % 256 == 0, head_dim in {64, 128}.  lse: [batch, heads, seq] fp32 (may be null).  Returns -5 for other shapes.
extern "C" int oslo_attention_forward_pingpong(const void* q, const void* k, const void* v, void* o, float* lse, int batch,
                                               int seq, int heads, int head_dim, long long q_tok, long long q_head,
                                               long long q_batch, long long k_tok, long long k_head, long long k_batch,
                                               long long v_tok, long long v_head, long long v_batch, long long o_tok,
                                               long long o_head, long long o_batch, float scale, int causal, int is_bf16,
                                               int* status, void* stream) {
  using namespace oslo;
  if (batch <= 0 || seq <= 0) return 0;
  if (seq % (2 * kPPRows) || (head_dim != 64 && head_dim != 128)) return -5;
  bind_context_to_thread();
  CUtensorMap tq, tk, tv, to;
  int rc = make_map(&tq, q, is_bf16, head_dim, seq, heads, batch, q_tok, q_head, q_batch, 64, kPPRows);
  if (rc) return rc;
  rc = make_map(&tk, k, is_bf16, head_dim, seq, heads, batch, k_tok, k_head, k_batch, 64, kPPRows);
  if (rc) return rc;
  rc = make_map(&tv, v, is_bf16, head_dim, seq, heads, batch, v_tok, v_head, v_batch, 64, 64);
  if (rc) return rc;
  rc = make_map(&to, o, is_bf16, head_dim, seq, heads, batch, o_tok, o_head, o_batch, 64, 32);
  if (rc) return rc;
  AttnPPParams p{batch, heads, seq, causal, scale * 1.4426950408889634f, is_bf16, lse, status};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return head_dim == 128 ? launch_attention_pingpong<128>(tq, tk, tv, to, p, st) : launch_attention_pingpong<64>(tq, tk, tv, to, p, st);
}

// Fused attention forward for sm_100a: softmax(scale * Q K^T [+ causal mask]) V without materialising the scores.
//
// One CTA handles one (batch, head, 128-query block).  Both products run on tcgen05 with accumulators in tensor
// memory; the score tile S (128 x 128 fp32) never leaves the SM:
//
//   warp 0     TMA producer: Q tile once, then K tiles (pass 1), then K and V tiles (pass 2), 2-stage rings
//   warp 1     MMA issuer: S = Q K_j^T into one of two TMEM buffers; O += P_j V_j into a third
//   warps 2-5  softmax: one thread per query row.  Pass 1 finds the row max (no exponentials); pass 2 recomputes S,
//              writes P = exp2(S - max) as bf16 into shared memory in the swizzled operand layout the MMA reads while
//              summing the row, and finally scales O by 1 / sum, stages it and stores it with TMA.
//
// Two passes over K trade one extra Q K^T product (tensor cores are idle most of the time here: the exponentials are
// the bottleneck) for never having to rescale the O accumulator in tensor memory.  The row log-sum-exp is written for
// the backward pass.  All waits are bounded.
//
// Replaces the unfused QK^T -> mask -> softmax -> dropout -> PV chains of the reference
// (oslo/transformers/models/gpt2/modeling_gpt2.py:113-165; lightseq2 csrc/layers_new/sdpa_layer.cpp:10-66).
#include "gemm_core.cuh"

namespace oslo {

constexpr int kAttBlock = 128;  // query rows per CTA and key rows per step
constexpr int kAttThreads = 192;

struct AttnParams {
  int batch, heads, seq;
  int causal;
  float scale_log2;  // scale * log2(e)
  int is_bf16;
  float* lse;        // [batch, heads, seq] natural-log row log-sum-exp of the scaled scores
  int* status;
};

template <int HD>
struct AttnCfg {
  static constexpr int kHalves = HD / 64;                 // 64-column swizzled halves of a [128, HD] tile
  static constexpr int kTile = kAttBlock * HD * 2;         // bytes of a Q / K / V tile
  static constexpr int kPBytes = kAttBlock * kAttBlock * 2;
  static constexpr int kSmem = kTile /*Q*/ + 2 * kTile /*K*/ + 2 * kTile /*V*/ + kPBytes + 1024 + 256;
  static constexpr int kTmemCols = 512;                    // S0 [0,128) S1 [128,256) O [256, 256+HD)
};

template <int HD>
__global__ void __launch_bounds__(kAttThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const AttnParams p) {
  using Cfg = AttnCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::kTile;
  uint8_t* sV = sK + 2 * Cfg::kTile;
  uint8_t* sP = sV + 2 * Cfg::kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + Cfg::kPBytes);
  uint64_t* q_full = bars;          // [1]
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2]
  uint64_t* s_empty = bars + 11;    // [2]
  uint64_t* p_full = bars + 13;     // [1]
  uint64_t* p_empty = bars + 14;    // [1]
  uint64_t* o_full = bars + 15;     // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblocks = p.seq / kAttBlock;
  // heavy (late) query blocks first so the causal triangle balances across the grid
  const int qb = qblocks - 1 - static_cast<int>(blockIdx.x % qblocks);
  const int bh = blockIdx.x / qblocks;
  const int h = bh % p.heads, b = bh / p.heads;
  const int nkv = p.causal ? qb + 1 : qblocks;
  const int q0 = qb * kAttBlock;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4); mbar_init(p_empty, 1); mbar_init(o_full, 1);
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
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    // ---------------------------------------------------------------------------------------- TMA producer
    if (elect_one()) {
      bool ok = true;
      mbar_arrive_expect_tx(q_full, Cfg::kTile);
      for (int c = 0; c < Cfg::kHalves; ++c) tma_load_4d(sQ + c * 16384, &tmQ, q_full, c * 64, q0, h, b);
      int kst = 0, vst = 0;
      uint32_t kph = 0, vph = 0;
      for (int pass = 0; pass < 2 && ok; ++pass) {
        for (int j = 0; j < nkv; ++j) {
          if (!mbar_wait_bounded(&k_empty[kst], kph ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&k_full[kst], Cfg::kTile);
          for (int c = 0; c < Cfg::kHalves; ++c)
            tma_load_4d(sK + kst * Cfg::kTile + c * 16384, &tmK, &k_full[kst], c * 64, j * kAttBlock, h, b);
          if (++kst == 2) { kst = 0; kph ^= 1; }
          if (pass == 1) {
            if (!mbar_wait_bounded(&v_empty[vst], vph ^ 1, abort_flag)) { ok = false; break; }
            mbar_arrive_expect_tx(&v_full[vst], Cfg::kTile);
            // MN-major operand: [k-block of 64 key rows][64-wide head-dim chunk][64 rows x 128 B]
            for (int kb = 0; kb < 2; ++kb)
              for (int c = 0; c < Cfg::kHalves; ++c)
                tma_load_4d(sV + vst * Cfg::kTile + kb * (Cfg::kHalves * 8192) + c * 8192, &tmV, &v_full[vst], c * 64,
                            j * kAttBlock + kb * 64, h, b);
            if (++vst == 2) { vst = 0; vph ^= 1; }
          }
        }
      }
      if (!ok && p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutProducer);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc_f16(kAttBlock, kAttBlock, p.is_bf16 != 0, false, false);
      const uint32_t idesc_o = make_idesc_f16(kAttBlock, HD, p.is_bf16 != 0, false, true);
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag);
      int kst = 0, vst = 0, sb = 0;
      uint32_t kph = 0, vph = 0, sph = 0, pph = 0;
      const uint32_t q_addr = smem_u32(sQ);
      auto issue_s = [&]() -> bool {
        if (!mbar_wait_bounded(&k_full[kst], kph, abort_flag)) return false;
        if (!mbar_wait_bounded(&s_empty[sb], sph ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + kst * Cfg::kTile);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const int half = kk / 4, k = kk % 4;
          umma_f16(tmem_base + sb * 128, make_smem_desc_sw128(q_addr + half * 16384 + k * 32, 16, 1024),
                   make_smem_desc_sw128(k_addr + half * 16384 + k * 32, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[kst]);
        umma_commit(&s_full[sb]);
        if (++kst == 2) { kst = 0; kph ^= 1; }
        if (++sb == 2) { sb = 0; sph ^= 1; }
        return true;
      };
      // pass 1: scores only
      for (int j = 0; j < nkv && ok; ++j) ok = issue_s();
      // pass 2: scores one step ahead of the P V product
      if (ok) ok = issue_s();
      for (int j = 0; j < nkv && ok; ++j) {
        if (j + 1 < nkv) ok = issue_s();
        if (!ok) break;
        if (!mbar_wait_bounded(p_full, pph, abort_flag)) { ok = false; break; }
        if (!mbar_wait_bounded(&v_full[vst], vph, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t p_addr = smem_u32(sP);
        const uint32_t v_addr = smem_u32(sV + vst * Cfg::kTile);
#pragma unroll
        for (int kk = 0; kk < kAttBlock / 16; ++kk) {
          const int half = kk / 4, k = kk % 4;
          umma_f16(tmem_o, make_smem_desc_sw128(p_addr + half * 16384 + k * 32, 16, 1024),
                   make_smem_desc_sw128(v_addr + half * (Cfg::kHalves * 8192) + k * 2048, 8192, 1024), idesc_o,
                   (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[vst]);
        umma_commit(p_empty);
        pph ^= 1;
        if (++vst == 2) { vst = 0; vph ^= 1; }
      }
      if (ok) umma_commit(o_full);
      if (!ok && p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutMma);
    }
  } else {
    // -------------------------------------------------------------------------------------- softmax warps
    const int q = warp & 3;
    const int row = q * 32 + lane;           // row inside the query block
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    float m = -INFINITY, l = 0.f;
    int sb = 0;
    uint32_t sph = 0, peph = 0;
    bool ok = true;
    // pass 1: row maximum only (the row sum is accumulated in pass 2 from the very exponentials written to P, so the
    // exponential unit is used once per score, not twice)
    for (int j = 0; j < nkv && ok; ++j) {
      if (!mbar_wait_bounded(&s_full[sb], sph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = p.causal && j == qb;
      float bm = -INFINITY;
      // the whole 128-column row in one round trip to tensor memory, then the buffer goes straight back to the MMA warp
      uint32_t r[4][32];
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(tmem_base + lane_base + sb * 128 + c * 32, r[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float t = __uint_as_float(r[c][i]);
          if (!(diag && c * 32 + i > row)) bm = fmaxf(bm, t);
        }
      }
      m = fmaxf(m, bm * p.scale_log2);
      if (++sb == 2) { sb = 0; sph ^= 1; }
    }
    // pass 2: P tiles
    for (int j = 0; j < nkv && ok; ++j) {
      if (!mbar_wait_bounded(&s_full[sb], sph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = p.causal && j == qb;
      uint32_t r[4][32];
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(tmem_base + lane_base + sb * 128 + c * 32, r[c]);
      tmem_ld_wait();
      // the scores are in registers: the S buffer can take the next product while the exponentials run
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      // P is rewritten only once the previous P V product has finished reading it (the loads above ran meanwhile)
      if (!mbar_wait_bounded(p_empty, peph ^ 1, abort_flag)) { ok = false; break; }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t packed[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i0 = g * 8 + 2 * e;
            float a0 = exp2f(__uint_as_float(r[c][i0]) * p.scale_log2 - m);
            float a1 = exp2f(__uint_as_float(r[c][i0 + 1]) * p.scale_log2 - m);
            if (diag && c * 32 + i0 > row) a0 = 0.f;
            if (diag && c * 32 + i0 + 1 > row) a1 = 0.f;
            l += a0 + a1;
            if (p.is_bf16) { const __nv_bfloat162 hh = __floats2bfloat162_rn(a0, a1); packed[e] = *reinterpret_cast<const uint32_t*>(&hh); }
            else { const __half2 hh = __floats2half2_rn(a0, a1); packed[e] = *reinterpret_cast<const uint32_t*>(&hh); }
          }
          const int col = c * 32 + g * 8;  // first of 8 columns in this 16-byte chunk
          const int half = col / 64, chunk = (col % 64) / 8;
          *reinterpret_cast<uint4*>(sP + half * 16384 + row * 128 + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      peph ^= 1;
      if (++sb == 2) { sb = 0; sph ^= 1; }
    }
    // epilogue: O / l -> shared (swizzled) -> TMA store; log-sum-exp
    if (ok && mbar_wait_bounded(o_full, 0, abort_flag)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      if (p.lse) p.lse[(static_cast<size_t>(b) * p.heads + h) * p.seq + q0 + row] = (m + log2f(l)) * 0.6931471805599453f;
      uint8_t* stage = sP + q * 8192;  // 32 rows x (HD / 64) x 128 B per warp; P is no longer needed
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32(tmem_o + lane_base + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t packed[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float a0 = __uint_as_float(r[g * 8 + 2 * e]) * inv, a1 = __uint_as_float(r[g * 8 + 2 * e + 1]) * inv;
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
        for (int half = 0; half < Cfg::kHalves; ++half) tma_store_4d(&tmO, stage + half * 4096, half * 64, q0 + q * 32, h, b);
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
static int launch_attention_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
                                const AttnParams& p, cudaStream_t stream) {
  using Cfg = AttnCfg<HD>;
  auto kern = attention_fwd_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem) != cudaSuccess) return -3;
    configured = true;
  }
  const int grid = p.batch * p.heads * (p.seq / kAttBlock);
  kern<<<grid, kAttThreads, Cfg::kSmem, stream>>>(tq, tk, tv, to, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace oslo

// q, k, v, o: [batch, seq, heads, head_dim] views given by element strides (token, head, batch); head_dim contiguous.
// seq % 128 == 0, head_dim in {64, 128}.  lse: [batch, heads, seq] fp32 (may be null).
extern "C" int oslo_attention_forward(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq,
                                      int heads, int head_dim, long long q_tok, long long q_head, long long q_batch,
                                      long long k_tok, long long k_head, long long k_batch, long long v_tok, long long v_head,
                                      long long v_batch, long long o_tok, long long o_head, long long o_batch, float scale,
                                      int causal, int is_bf16, int* status, void* stream) {
  using namespace oslo;
  if (batch <= 0 || seq <= 0) return 0;
  if (seq % kAttBlock || (head_dim != 64 && head_dim != 128)) return -5;
  bind_context_to_thread();
  CUtensorMap tq, tk, tv, to;
  int rc = make_map(&tq, q, is_bf16, head_dim, seq, heads, batch, q_tok, q_head, q_batch, 64, kAttBlock);
  if (rc) return rc;
  rc = make_map(&tk, k, is_bf16, head_dim, seq, heads, batch, k_tok, k_head, k_batch, 64, kAttBlock);
  if (rc) return rc;
  rc = make_map(&tv, v, is_bf16, head_dim, seq, heads, batch, v_tok, v_head, v_batch, 64, 64);
  if (rc) return rc;
  rc = make_map(&to, o, is_bf16, head_dim, seq, heads, batch, o_tok, o_head, o_batch, 64, 32);
  if (rc) return rc;
  AttnParams p{batch, heads, seq, causal, scale * 1.4426950408889634f, is_bf16, lse, status};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return head_dim == 128 ? launch_attention_fwd<128>(tq, tk, tv, to, p, st) : launch_attention_fwd<64>(tq, tk, tv, to, p, st);
}

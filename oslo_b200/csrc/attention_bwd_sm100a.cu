// Fused attention backward for sm_100a (no materialised score matrix).  Three kernels:
//
//   attn_delta_kernel     delta[b, h, s] = sum_d dO * O                         (row constants of the softmax gradient)
//   attn_bwd_dq_kernel    one CTA per (batch, head, 128-query block), loop over key blocks:
//                           S = Q K^T, dP = dO V^T (tcgen05, TMEM) -> P = exp(S - lse), dS = P (dP - delta) scale in
//                           registers (one thread per query row) -> dS to shared memory -> dQ += dS K
//   attn_bwd_dkv_kernel   one CTA per (batch, head, 128-key block), loop over 64-query tiles, everything transposed so
//                           that one thread owns one KEY row: S^T = K Q^T, dP^T = V dO^T -> P^T, dS^T to shared memory
//                           -> dV += P^T dO, dK += dS^T Q
//
// A [rows, 64-column] 128-byte-swizzled tile is at once a K-major operand (rows = M or N) and an MN-major operand
// (rows = K), so every tile is loaded once and used in both roles (K_j for S and for dQ; Q_i / dO_i for S^T / dP^T and
// for dK / dV).  Warp roles as in the forward kernel: warp 0 TMA, warp 1 MMA issue, warps 2-5 the element-wise math.
// All waits are bounded.
#include <cstdlib>

#include "gemm_core.cuh"

namespace oslo {

constexpr int kBwdThreads = 192;

struct AttnBwdParams {
  int batch, heads, seq;
  int causal;
  float scale, scale_log2;
  int is_bf16;
  const float* lse;    // [batch, heads, seq]
  const float* delta;  // [batch, heads, seq]
  int* status;
};

OSLO_DEVINL float ex2_approx(float x) {  // one special-function instruction; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

OSLO_DEVINL uint32_t pack2(float a, float b, bool bf16) {
  if (bf16) {
    // bf16 pair by integer arithmetic (round half away from zero on the dropped 16 bits, then the two high halves): the
    // float -> bf16 conversion instruction shares the special-function unit with the exponentials, integer adds do not
    return __byte_perm(__float_as_uint(a) + 0x8000u, __float_as_uint(b) + 0x8000u, 0x7632);
  }
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// ------------------------------------------------------------------------------------------------ delta
// one warp per (token, head) row of head_dim elements
__global__ void attn_delta_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ d_o, float* __restrict__ delta,
                                  int batch, int seq, int heads, int hd, long long o_tok, long long o_head, long long o_batch,
                                  long long g_tok, long long g_head, long long g_batch, int is_bf16) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(batch) * seq * heads;
  if (row >= total) return;
  const int h = static_cast<int>(row % heads);
  const long long t = row / heads;
  const int s = static_cast<int>(t % seq), b = static_cast<int>(t / seq);
  const uint16_t* po = o + b * o_batch + s * o_tok + h * o_head;
  const uint16_t* pg = d_o + b * g_batch + s * g_tok + h * g_head;
  float acc = 0.f;
  for (int c = lane * 2; c < hd; c += 64) {
    const uint32_t a = *reinterpret_cast<const uint32_t*>(po + c), g = *reinterpret_cast<const uint32_t*>(pg + c);
    if (is_bf16) {
      acc += __uint_as_float(a << 16) * __uint_as_float(g << 16) + __uint_as_float(a & 0xffff0000u) * __uint_as_float(g & 0xffff0000u);
    } else {
      const __half2 ha = *reinterpret_cast<const __half2*>(&a), hg = *reinterpret_cast<const __half2*>(&g);
      acc += __low2float(ha) * __low2float(hg) + __high2float(ha) * __high2float(hg);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[(static_cast<long long>(b) * heads + h) * seq + s] = acc;
}

// --------------------------------------------------------------------------------------------------- dQ
template <int HD>
struct DqCfg {
  static constexpr int kHalves = HD / 64;
  static constexpr int kTile = 128 * HD * 2;
  static constexpr int kDs = 128 * 128 * 2;
  static constexpr int kSmem = 2 * kTile /*Q, dO*/ + 4 * kTile /*K x2, V x2*/ + kDs + 1024 + 256;
};

// NG element-wise warp groups: with two, each 128-key tile is split by COLUMNS (group g takes keys [64 g, 64 g + 64)), so
// eight warps work on one tile at once and the exponentials of a tile take half as long before dQ can accumulate it.
template <int HD, int NG>
__global__ void __launch_bounds__(64 + 128 * NG, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmDQ, const AttnBwdParams p) {
  using Cfg = DqCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + Cfg::kTile;
  uint8_t* sK = sDO + Cfg::kTile;
  uint8_t* sV = sK + 2 * Cfg::kTile;
  uint8_t* sDS = sV + 2 * Cfg::kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + Cfg::kDs);
  uint64_t* qd_full = bars;       // Q and dO landed
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // S and dP computed
  uint64_t* s_empty = bars + 10;  // S and dP consumed (4 warps)
  uint64_t* ds_full = bars + 11;  // dS tile written (4 warps)
  uint64_t* ds_empty = bars + 12; // dQ product done with the dS tile
  uint64_t* dq_full = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblocks = p.seq / 128;
  const int qb = qblocks - 1 - static_cast<int>(blockIdx.x % qblocks);
  const int bh = blockIdx.x / qblocks;
  const int h = bh % p.heads, b = bh / p.heads;
  const int nkv = p.causal ? qb + 1 : qblocks;
  const int q0 = qb * 128;

  if (threadIdx.x == 0) {
    mbar_init(qd_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    mbar_init(s_full, 1); mbar_init(s_empty, 4 * NG); mbar_init(ds_full, 4 * NG); mbar_init(ds_empty, 1); mbar_init(dq_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dq = tmem_base + 256;

  if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      mbar_arrive_expect_tx(qd_full, 2 * Cfg::kTile);
      for (int c = 0; c < Cfg::kHalves; ++c) {
        tma_load_4d(sQ + c * 16384, &tmQ, qd_full, c * 64, q0, h, b);
        tma_load_4d(sDO + c * 16384, &tmDO, qd_full, c * 64, q0, h, b);
      }
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < nkv && ok; ++j) {
        if (!mbar_wait_bounded(&k_empty[st], ph ^ 1, abort_flag) || !mbar_wait_bounded(&v_empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[st], Cfg::kTile);
        mbar_arrive_expect_tx(&v_full[st], Cfg::kTile);
        for (int c = 0; c < Cfg::kHalves; ++c) {
          tma_load_4d(sK + st * Cfg::kTile + c * 16384, &tmK, &k_full[st], c * 64, j * 128, h, b);
          tma_load_4d(sV + st * Cfg::kTile + c * 16384, &tmV, &v_full[st], c * 64, j * 128, h, b);
        }
        if (++st == 2) { st = 0; ph ^= 1; }
      }
      if (!ok && p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutProducer);
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const bool bf = p.is_bf16 != 0;
      const uint32_t idesc_s = make_idesc_f16(128, 128, bf, false, false);
      const uint32_t idesc_dq = make_idesc_f16(128, HD, bf, false, true);  // B = K tile read MN-major
      bool ok = mbar_wait_bounded(qd_full, 0, abort_flag);
      int st = 0;
      uint32_t ph = 0, sph = 0, dsph = 0;
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sDO), ds_addr = smem_u32(sDS);
      int st_s = 0;          // stage of the next S / dP product (runs one key block ahead of the dQ product)
      uint32_t ph_s = 0;
      auto issue_s = [&]() -> bool {
        if (!mbar_wait_bounded(&k_full[st_s], ph_s, abort_flag) || !mbar_wait_bounded(&v_full[st_s], ph_s, abort_flag) ||
            !mbar_wait_bounded(s_empty, sph ^ 1, abort_flag))
          return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + st_s * Cfg::kTile), v_addr = smem_u32(sV + st_s * Cfg::kTile);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const int half = kk / 4, k = kk % 4;
          umma_f16(tm_s, make_smem_desc_sw128(q_addr + half * 16384 + k * 32, 16, 1024),
                   make_smem_desc_sw128(k_addr + half * 16384 + k * 32, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const int half = kk / 4, k = kk % 4;
          umma_f16(tm_dp, make_smem_desc_sw128(do_addr + half * 16384 + k * 32, 16, 1024),
                   make_smem_desc_sw128(v_addr + half * 16384 + k * 32, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[st_s]);
        umma_commit(s_full);
        sph ^= 1;
        if (++st_s == 2) { st_s = 0; ph_s ^= 1; }
        return true;
      };
      if (ok) ok = issue_s();
      for (int j = 0; j < nkv && ok; ++j) {
        // the next block's S and dP are issued as soon as the element-wise warps have taken this block's out of tensor
        // memory, so they are computed while dS of this block is still being formed
        if (j + 1 < nkv) ok = issue_s();
        if (!ok) break;
        // dQ += dS K_j once the element-wise warps have written dS
        if (!mbar_wait_bounded(ds_full, dsph, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + st * Cfg::kTile);
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk) {
          const int half = kk / 4, k = kk % 4;
          umma_f16(tm_dq, make_smem_desc_sw128(ds_addr + half * 16384 + k * 32, 16, 1024),
                   make_smem_desc_sw128(k_addr + kk * 2048, 16384, 1024), idesc_dq, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(ds_empty);
        dsph ^= 1;
        if (++st == 2) { st = 0; ph ^= 1; }
      }
      if (ok) umma_commit(dq_full);
      if (!ok && p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutMma);
    }
  } else {
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;  // which 64-column half of every tile this warp handles (NG = 2), or both (NG = 1)
    const int row = q * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const size_t stat = (static_cast<size_t>(b) * p.heads + h) * p.seq + q0 + row;
    const float lse2 = p.lse[stat] * 1.4426950408889634f;
    const float dl = p.delta[stat];
    const bool bf = p.is_bf16 != 0;
    uint32_t sph = 0, deph = 0;
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      if (!mbar_wait_bounded(s_full, sph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = p.causal && j == qb;
      // two round trips to tensor memory per tile (64 columns of S and of dP each) instead of four; the accumulators go
      // back to the MMA warp as soon as the second half is in registers, before the exponentials of that half run
#pragma unroll
      for (int hc = (NG == 2 ? grp : 0); hc < (NG == 2 ? grp + 1 : 2); ++hc) {
        uint32_t rs[2][32], rp[2][32];
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          tmem_ld_32x32(tm_s + lane_base + (hc * 2 + u) * 32, rs[u]);
          tmem_ld_32x32(tm_dp + lane_base + (hc * 2 + u) * 32, rp[u]);
        }
        tmem_ld_wait();
        if (NG == 2 || hc == 1) {  // this warp's share of the accumulators is in registers
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty);
        }
        if ((NG == 2 || hc == 0) && !mbar_wait_bounded(ds_empty, deph ^ 1, abort_flag)) {  // dS of the previous tile has been consumed
          ok = false;
        }
#pragma unroll
        for (int u2 = 0; u2 < 2; ++u2) {
          const int c = hc * 2 + u2;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t packed[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float d[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int i = g * 8 + 2 * e + u;
                float pr = ex2_approx(__uint_as_float(rs[u2][i]) * p.scale_log2 - lse2);
                if (diag && c * 32 + i > row) pr = 0.f;
                d[u] = pr * (__uint_as_float(rp[u2][i]) - dl) * p.scale;
              }
              packed[e] = pack2(d[0], d[1], bf);
            }
            const int col = c * 32 + g * 8;
            const int half = col / 64, chunk = (col % 64) / 8;
            *reinterpret_cast<uint4*>(sDS + half * 16384 + row * 128 + ((chunk ^ (row & 7)) << 4)) =
                make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
      if (!ok) break;
      sph ^= 1;
      deph ^= 1;
    }
    if (grp != 0) {
      // the first group alone writes dQ out
    } else if (ok && mbar_wait_bounded(dq_full, 0, abort_flag)) {
      tc_fence_after();
      uint8_t* stage = sDS + q * 8192;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32(tm_dq + lane_base + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t packed[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) packed[e] = pack2(__uint_as_float(r[g * 8 + 2 * e]), __uint_as_float(r[g * 8 + 2 * e + 1]), bf);
          const int col = c * 32 + g * 8;
          const int half = col / 64, chunk = (col % 64) / 8;
          *reinterpret_cast<uint4*>(stage + half * 4096 + lane * 128 + ((chunk ^ (lane & 7)) << 4)) =
              make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        for (int half = 0; half < Cfg::kHalves; ++half) tma_store_4d(&tmDQ, stage + half * 4096, half * 64, q0 + q * 32, h, b);
        tma_store_commit();
        tma_store_wait_all();
      }
    } else if (p.status && lane == 0) {
      atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutEpilogue);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace oslo

namespace oslo {

// ------------------------------------------------------------------------------------------------ dK, dV
// NG = number of element-wise warp groups (4 warps each).  With two groups consecutive query tiles go to alternating
// groups and P^T / dS^T are double-buffered in shared memory, so the exponentials of tile t + 1 run while the tensor cores
// accumulate tile t (and compute the scores of tile t + 2).
template <int HD, int NG>
struct DkvCfg {
  static constexpr int kHalves = HD / 64;
  static constexpr int kThreads = 64 + 128 * NG;
  static constexpr int kKv = 128 * HD * 2;      // K_j / V_j tile
  static constexpr int kQt = 64 * HD * 2;       // Q_i / dO_i tile of 64 query rows
  static constexpr int kPt = 128 * 64 * 2;      // P^T / dS^T tile [128 keys, 64 queries]
  static constexpr int kSmem = 2 * kKv + 4 * kQt + 2 * NG * kPt + 4096 * NG /*lse, delta per warp*/ + 1024 + 256;
};

template <int HD, int NG>
__global__ void __launch_bounds__(64 + 128 * NG, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV,
                    const AttnBwdParams p) {
  using Cfg = DkvCfg<HD, NG>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::kKv;
  uint8_t* sQ = sV + Cfg::kKv;            // [2 stages]
  uint8_t* sDO = sQ + 2 * Cfg::kQt;       // [2 stages]
  uint8_t* sP = sDO + 2 * Cfg::kQt;       // [NG stages]
  uint8_t* sDS = sP + NG * Cfg::kPt;      // [NG stages]
  float* sStat = reinterpret_cast<float*>(sDS + NG * Cfg::kPt);  // [4 NG warps][2 stages][lse 64 | delta 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sStat) + 4096 * NG);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;    // [2] Q_i and dO_i landed
  uint64_t* q_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;    // [2] S^T, dP^T computed
  uint64_t* s_empty = bars + 7;   // [2]
  uint64_t* p_full = bars + 9;    // [NG] P^T, dS^T written (4 warps)
  uint64_t* p_empty = bars + 11;  // [NG] dV, dK products done with them
  uint64_t* out_full = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = p.seq / 128;
  const int jb = static_cast<int>(blockIdx.x % kblocks);  // early key blocks (most query tiles under causality) first
  const int bh = blockIdx.x / kblocks;
  const int h = bh % p.heads, b = bh / p.heads;
  const int k0 = jb * 128;
  const int qt_first = p.causal ? jb * 2 : 0;
  const int qt_end = p.seq / 64;
  const size_t stat_base = (static_cast<size_t>(b) * p.heads + h) * p.seq;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4); }
    for (int i = 0; i < NG; ++i) { mbar_init(&p_full[i], 4); mbar_init(&p_empty[i], 1); }
    mbar_init(out_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S^T [0,64) [64,128) | dP^T [128,192) [192,256) | dV [256, 256+HD) | dK [384, 384+HD)
  const uint32_t tm_dv = tmem_base + 256, tm_dk = tmem_base + 384;

  if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      mbar_arrive_expect_tx(kv_full, 2 * Cfg::kKv);
      for (int c = 0; c < Cfg::kHalves; ++c) {
        tma_load_4d(sK + c * 16384, &tmK, kv_full, c * 64, k0, h, b);
        tma_load_4d(sV + c * 16384, &tmV, kv_full, c * 64, k0, h, b);
      }
      int st = 0;
      uint32_t ph = 0;
      for (int i = qt_first; i < qt_end && ok; ++i) {
        if (!mbar_wait_bounded(&q_empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&q_full[st], 2 * Cfg::kQt);
        for (int c = 0; c < Cfg::kHalves; ++c) {
          tma_load_4d(sQ + st * Cfg::kQt + c * 8192, &tmQ, &q_full[st], c * 64, i * 64, h, b);
          tma_load_4d(sDO + st * Cfg::kQt + c * 8192, &tmDO, &q_full[st], c * 64, i * 64, h, b);
        }
        if (++st == 2) { st = 0; ph ^= 1; }
      }
      if (!ok && p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutProducer);
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const bool bf = p.is_bf16 != 0;
      const uint32_t idesc_st = make_idesc_f16(128, 64, bf, false, false);   // S^T, dP^T: [128 keys, 64 queries]
      const uint32_t idesc_acc = make_idesc_f16(128, HD, bf, false, true);   // dV, dK: B = Q_i / dO_i read MN-major
      bool ok = mbar_wait_bounded(kv_full, 0, abort_flag);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), p_addr = smem_u32(sP), ds_addr = smem_u32(sDS);
      int st = 0, sb = 0;
      uint32_t ph = 0, sph = 0;
      const int n_tiles = qt_end - qt_first;
      auto issue_scores = [&](int stage) -> bool {
        if (!mbar_wait_bounded(&q_full[stage], ph, abort_flag) || !mbar_wait_bounded(&s_empty[sb], sph ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + stage * Cfg::kQt), do_addr = smem_u32(sDO + stage * Cfg::kQt);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const int half = kk / 4, k = kk % 4;
          umma_f16(tmem_base + sb * 64, make_smem_desc_sw128(k_addr + half * 16384 + k * 32, 16, 1024),
                   make_smem_desc_sw128(q_addr + half * 8192 + k * 32, 16, 1024), idesc_st, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const int half = kk / 4, k = kk % 4;
          umma_f16(tmem_base + 128 + sb * 64, make_smem_desc_sw128(v_addr + half * 16384 + k * 32, 16, 1024),
                   make_smem_desc_sw128(do_addr + half * 8192 + k * 32, 16, 1024), idesc_st, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[sb]);
        if (++sb == 2) { sb = 0; sph ^= 1; }
        return true;
      };
      // scores of tile t+1 are issued before the accumulation of tile t so the element-wise warps never idle
      int st_issue = 0;
      uint32_t ph_issue = 0;
      auto next_scores = [&]() -> bool {
        const uint32_t save = ph;
        ph = ph_issue;
        const bool r = issue_scores(st_issue);
        ph = save;
        if (++st_issue == 2) { st_issue = 0; ph_issue ^= 1; }
        return r;
      };
      if (ok && n_tiles > 0) ok = next_scores();
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (t + 1 < n_tiles) ok = next_scores();
        if (!ok) break;
        const int ps = t % NG;  // P^T / dS^T stage of this tile (the group that wrote it)
        if (!mbar_wait_bounded(&p_full[ps], static_cast<uint32_t>((t / NG) & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + st * Cfg::kQt), do_addr = smem_u32(sDO + st * Cfg::kQt);
#pragma unroll
        for (int kk = 0; kk < 64 / 16; ++kk) {
          umma_f16(tm_dv, make_smem_desc_sw128(p_addr + ps * Cfg::kPt + kk * 32, 16, 1024),
                   make_smem_desc_sw128(do_addr + kk * 2048, 8192, 1024), idesc_acc, (t > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 64 / 16; ++kk) {
          umma_f16(tm_dk, make_smem_desc_sw128(ds_addr + ps * Cfg::kPt + kk * 32, 16, 1024),
                   make_smem_desc_sw128(q_addr + kk * 2048, 8192, 1024), idesc_acc, (t > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&q_empty[st]);
        umma_commit(&p_empty[ps]);
        if (++st == 2) { st = 0; }
      }
      if (ok) umma_commit(out_full);
      if (!ok && p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutMma);
    }
  } else {
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;  // element-wise group: takes the tiles t with t % NG == grp
    const int row = q * 32 + lane;  // key row inside the block
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const bool bf = p.is_bf16 != 0;
    bool ok = true;
    for (int t = grp; qt_first + t < qt_end && ok; t += NG) {
      const int i = qt_first + t;
      const int sb = t & 1;                                       // tensor-memory buffer of the scores of tile t
      const uint32_t sph = static_cast<uint32_t>((t >> 1) & 1);  // its phase
      const int ps = t % NG;                                      // shared-memory stage for P^T / dS^T
      const uint32_t peph = static_cast<uint32_t>((t / NG) & 1);
      uint8_t* const sPt = sP + ps * Cfg::kPt;
      uint8_t* const sDSt = sDS + ps * Cfg::kPt;
      // row statistics of this query tile (the same for every key row): stage them through shared memory
      float* stat = sStat + ((warp - 2) * 2 + ((t / NG) & 1)) * 128;  // a private copy per warp: no barrier between warps needed
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        stat[lane + 32 * u] = p.lse[stat_base + i * 64 + lane + 32 * u] * 1.4426950408889634f;
        stat[64 + lane + 32 * u] = p.delta[stat_base + i * 64 + lane + 32 * u];
      }
      __syncwarp();
      if (!mbar_wait_bounded(&s_full[sb], sph, abort_flag) || !mbar_wait_bounded(&p_empty[ps], peph ^ 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = p.causal && (i * 64 < k0 + 128);  // some (query, key) pairs of this tile are masked
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32], rp[32];
        __syncwarp();
        tmem_ld_32x32(tmem_base + lane_base + sb * 64 + c * 32, rs);
        tmem_ld_32x32(tmem_base + 128 + lane_base + sb * 64 + c * 32, rp);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t pk_p[4], pk_d[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float pv[2], dv[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int col = c * 32 + g * 8 + 2 * e + u;  // query inside the tile
              float pr = ex2_approx(__uint_as_float(rs[g * 8 + 2 * e + u]) * p.scale_log2 - stat[col]);
              if (diag && k0 + row > i * 64 + col) pr = 0.f;
              pv[u] = pr;
              dv[u] = pr * (__uint_as_float(rp[g * 8 + 2 * e + u]) - stat[64 + col]) * p.scale;
            }
            pk_p[e] = pack2(pv[0], pv[1], bf);
            pk_d[e] = pack2(dv[0], dv[1], bf);
          }
          const int chunk = (c * 32 + g * 8) / 8;
          const int off = row * 128 + ((chunk ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(sPt + off) = make_uint4(pk_p[0], pk_p[1], pk_p[2], pk_p[3]);
          *reinterpret_cast<uint4*>(sDSt + off) = make_uint4(pk_d[0], pk_d[1], pk_d[2], pk_d[3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s_empty[sb]); mbar_arrive(&p_full[ps]); }
    }
    if (grp != 0) {
      // the first group alone writes dV and dK out (its four warps cover all 128 key rows)
    } else if (ok && mbar_wait_bounded(out_full, 0, abort_flag)) {
      tc_fence_after();
      uint8_t* stage = sQ + q * (Cfg::kHalves * 4096);  // the query-tile ring is free now
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = which == 0 ? tm_dv : tm_dk;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          __syncwarp();
          tmem_ld_32x32(src + lane_base + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t packed[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) packed[e] = pack2(__uint_as_float(r[g * 8 + 2 * e]), __uint_as_float(r[g * 8 + 2 * e + 1]), bf);
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
            tma_store_4d(which == 0 ? &tmDV : &tmDK, stage + half * 4096, half * 64, k0 + q * 32, h, b);
          tma_store_commit();
          tma_store_wait_all();
        }
        __syncwarp();
      }
    } else if (p.status && lane == 0) {
      atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutEpilogue);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <typename K>
static int set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : -3;
}

}  // namespace oslo

// q, k, v, o, d_o, dq, dk, dv: [batch, seq, heads, head_dim] views given by element strides (token, head, batch).
// lse: [batch, heads, seq] from the forward pass; delta: [batch, heads, seq] scratch written here.
// Element-wise warp groups of the dK / dV kernel: 2 by default (measured 13 % faster backward than 1);
// OSLO_B200_ATTN_BWD_GROUPS=1 sets the start value back.
static int g_dkv_groups = [] {
  const char* e = getenv("OSLO_B200_ATTN_BWD_GROUPS");
  return (e && e[0] == '1') ? 1 : 2;
}();

// Element-wise warp groups of the dQ kernel (1 or 2); OSLO_B200_ATTN_BWD_DQ_GROUPS sets the start value.
static int g_dq_groups = [] {
  const char* e = getenv("OSLO_B200_ATTN_BWD_DQ_GROUPS");
  return (e && e[0] == '2') ? 2 : 1;
}();

extern "C" int oslo_attention_backward_set_groups(int groups) {
  if (groups != 1 && groups != 2) return -1;
  g_dkv_groups = groups;
  return 0;
}

extern "C" int oslo_attention_backward_set_dq_groups(int groups) {
  if (groups != 1 && groups != 2) return -1;
  g_dq_groups = groups;
  return 0;
}

extern "C" int oslo_attention_backward(const void* q, const void* k, const void* v, const void* o, const void* d_o, void* dq,
                                       void* dk, void* dv, const float* lse, float* delta, int batch, int seq, int heads,
                                       int head_dim, const long long* strides /* 8 x (tok, head, batch) */, float scale,
                                       int causal, int is_bf16, int* status, void* stream) {
  using namespace oslo;
  if (batch <= 0 || seq <= 0) return 0;
  if (seq % 128 || (head_dim != 64 && head_dim != 128)) return -5;
  bind_context_to_thread();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto S = [&](int t, int i) { return strides[t * 3 + i]; };  // tensor order: q k v o do dq dk dv
  {
    const long long rows = static_cast<long long>(batch) * seq * heads;
    const int blocks = static_cast<int>((rows * 32 + 255) / 256);
    attn_delta_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint16_t*>(o), static_cast<const uint16_t*>(d_o), delta, batch, seq,
                                              heads, head_dim, S(3, 0), S(3, 1), S(3, 2), S(4, 0), S(4, 1), S(4, 2), is_bf16);
  }
  CUtensorMap tq128, tk128, tv128, tdo128, tdq, tq64, tdo64, tdk, tdv;
  int rc = 0;
  rc |= make_map(&tq128, q, is_bf16, head_dim, seq, heads, batch, S(0, 0), S(0, 1), S(0, 2), 64, 128);
  rc |= make_map(&tk128, k, is_bf16, head_dim, seq, heads, batch, S(1, 0), S(1, 1), S(1, 2), 64, 128);
  rc |= make_map(&tv128, v, is_bf16, head_dim, seq, heads, batch, S(2, 0), S(2, 1), S(2, 2), 64, 128);
  rc |= make_map(&tdo128, d_o, is_bf16, head_dim, seq, heads, batch, S(4, 0), S(4, 1), S(4, 2), 64, 128);
  rc |= make_map(&tq64, q, is_bf16, head_dim, seq, heads, batch, S(0, 0), S(0, 1), S(0, 2), 64, 64);
  rc |= make_map(&tdo64, d_o, is_bf16, head_dim, seq, heads, batch, S(4, 0), S(4, 1), S(4, 2), 64, 64);
  rc |= make_map(&tdq, dq, is_bf16, head_dim, seq, heads, batch, S(5, 0), S(5, 1), S(5, 2), 64, 32);
  rc |= make_map(&tdk, dk, is_bf16, head_dim, seq, heads, batch, S(6, 0), S(6, 1), S(6, 2), 64, 32);
  rc |= make_map(&tdv, dv, is_bf16, head_dim, seq, heads, batch, S(7, 0), S(7, 1), S(7, 2), 64, 32);
  if (rc) return -2;
  AttnBwdParams p{batch, heads, seq, causal, scale, scale * 1.4426950408889634f, is_bf16, lse, delta, status};
  const int grid = batch * heads * (seq / 128);
  static bool configured = false;
  if (!configured) {
    if (set_smem(attn_bwd_dq_kernel<128, 1>, DqCfg<128>::kSmem) || set_smem(attn_bwd_dq_kernel<64, 1>, DqCfg<64>::kSmem) ||
        set_smem(attn_bwd_dq_kernel<128, 2>, DqCfg<128>::kSmem) || set_smem(attn_bwd_dq_kernel<64, 2>, DqCfg<64>::kSmem) ||
        set_smem(attn_bwd_dkv_kernel<128, 1>, DkvCfg<128, 1>::kSmem) || set_smem(attn_bwd_dkv_kernel<64, 1>, DkvCfg<64, 1>::kSmem) ||
        set_smem(attn_bwd_dkv_kernel<128, 2>, DkvCfg<128, 2>::kSmem) || set_smem(attn_bwd_dkv_kernel<64, 2>, DkvCfg<64, 2>::kSmem))
      return -3;
    configured = true;
  }
  const int groups = g_dkv_groups;
  if (head_dim == 128) {
    if (groups == 2) attn_bwd_dkv_kernel<128, 2><<<grid, DkvCfg<128, 2>::kThreads, DkvCfg<128, 2>::kSmem, st>>>(tq64, tk128, tv128, tdo64, tdk, tdv, p);
    else attn_bwd_dkv_kernel<128, 1><<<grid, DkvCfg<128, 1>::kThreads, DkvCfg<128, 1>::kSmem, st>>>(tq64, tk128, tv128, tdo64, tdk, tdv, p);
    if (g_dq_groups == 2) attn_bwd_dq_kernel<128, 2><<<grid, 320, DqCfg<128>::kSmem, st>>>(tq128, tk128, tv128, tdo128, tdq, p);
    else attn_bwd_dq_kernel<128, 1><<<grid, kBwdThreads, DqCfg<128>::kSmem, st>>>(tq128, tk128, tv128, tdo128, tdq, p);
  } else {
    if (groups == 2) attn_bwd_dkv_kernel<64, 2><<<grid, DkvCfg<64, 2>::kThreads, DkvCfg<64, 2>::kSmem, st>>>(tq64, tk128, tv128, tdo64, tdk, tdv, p);
    else attn_bwd_dkv_kernel<64, 1><<<grid, DkvCfg<64, 1>::kThreads, DkvCfg<64, 1>::kSmem, st>>>(tq64, tk128, tv128, tdo64, tdk, tdv, p);
    if (g_dq_groups == 2) attn_bwd_dq_kernel<64, 2><<<grid, 320, DqCfg<64>::kSmem, st>>>(tq128, tk128, tv128, tdo128, tdq, p);
    else attn_bwd_dq_kernel<64, 1><<<grid, kBwdThreads, DqCfg<64>::kSmem, st>>>(tq128, tk128, tv128, tdo128, tdq, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

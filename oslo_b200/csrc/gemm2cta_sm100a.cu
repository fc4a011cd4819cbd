// Two-CTA tcgen05 GEMM for sm_100a: a cluster of two CTAs (one SM pair) computes one 256 x 256 tile of
//
//     C[b] = epilogue( A[b] x B[b]^T )        A: [M, K]   B: [N, K]   C: [M, N]     (bf16 / fp16 in, fp32 accumulate)
//
// with tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16).  Each CTA of the pair stages ITS OWN half of both
// operands: 128 rows of A and 128 rows of B (= 128 of the tile's 256 columns) per 64-wide k-block, 32 KiB per stage
// instead of the 48 KiB a single CTA needs for a 128 x 256 tile.  The tensor cores of both SMs read the B halves of both
// shared memories, so every B byte is loaded from global memory and read from shared memory once per 256 output rows
// instead of once per 128, which is what lets the tensor pipe stay busy.
//
// Roles per CTA (192 threads, persistent, one cluster per SM pair):
//   warp 0      TMA producer for this CTA's halves (cp.async.bulk.tensor with .cta_group::2: the bytes are counted on
//               the LEADER's "full" barrier, which only the leader arms; no multicast qualifier anywhere);
//   warp 1      leader CTA only: one elected thread issues the MMAs for the pair and commits them to the "stage empty"
//               and "accumulator full" barriers of BOTH CTAs (tcgen05.commit ... multicast::cluster);
//               in both CTAs this warp allocates / frees tensor memory (cta_group::2 needs the same warp of both);
//   warps 2-5   epilogue of this CTA's 128 rows: tcgen05.ld, bias / GELU / accumulate, swizzled staging, TMA store;
//               they hand the accumulator buffer back by arriving on the leader's "accumulator empty" barrier.
//
// Every wait is bounded; a CTA that gives up raises its abort flag, drains and still meets its partner at the closing
// cluster barrier, so tensor memory is always freed.  Operands may be K-major or MN-major, as in the one-CTA kernel
// (gemm_core.cuh), whose tensor maps and parameter block are reused.
#include "gemm_core.cuh"

namespace oslo {

constexpr int k2Stages = 6;
constexpr int k2TileM = 256;            // per cluster
constexpr int k2TileN = 256;
constexpr int k2HalfN = 128;            // B rows staged per CTA
constexpr int k2StageA = kBlockM * kBlockK * 2;   // 16 KiB
constexpr int k2StageB = k2HalfN * kBlockK * 2;   // 16 KiB
constexpr int k2StageBytes = k2StageA + k2StageB;
constexpr int k2Staging = 4 * 2 * 4096;
constexpr int k2SmemBytes = k2Stages * k2StageBytes + k2Staging + 1024 + 256;
constexpr int k2TmemCols = 512;         // two 256-column accumulator buffers

OSLO_DEVINL uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
OSLO_DEVINL void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (a variable of this CTA's shared memory) in the CTA with the given cluster rank
OSLO_DEVINL uint32_t mapa_u32(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
  return out;
}
OSLO_DEVINL void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tiled load into THIS CTA's shared memory whose bytes are counted on a barrier that may live in the partner CTA.
OSLO_DEVINL void tma_load_4d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
OSLO_DEVINL void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
OSLO_DEVINL void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
OSLO_DEVINL void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
OSLO_DEVINL void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far are done.
OSLO_DEVINL void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(static_cast<uint16_t>(3))
               : "memory");
}

OSLO_DEVINL void pair_tile_coords(int tile, int m_tiles, int n_tiles, int& b, int& mt, int& nt) {
  const int per_batch = m_tiles * n_tiles;
  b = tile / per_batch;
  const int t = tile - b * per_batch;
  constexpr int kGroup = 4;  // 4 x 256 rows sweep all column tiles: neighbouring clusters share B tiles in L2
  const int group_size = kGroup * n_tiles;
  const int g = t / group_size;
  const int first = g * kGroup;
  const int rows = min(kGroup, m_tiles - first);
  const int r = t - g * group_size;
  mt = first + r % rows;
  nt = r / rows;
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* staging = smem + k2Stages * k2StageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + k2Staging);
  uint64_t* full_bar = bars;                       // [stages]  used in the leader: bytes of both CTAs
  uint64_t* empty_bar = bars + k2Stages;           // [stages]  one per CTA, released by the leader's commits
  uint64_t* tmem_full = bars + 2 * k2Stages;       // [2]       one per CTA
  uint64_t* tmem_empty = bars + 2 * k2Stages + 2;  // [2]       used in the leader: 8 epilogue warps arrive
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * k2Stages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();  // 0 = leader
  const bool leader = cta_rank == 0;
  const int cluster_id = static_cast<int>(blockIdx.x) >> 1;
  const int num_clusters = static_cast<int>(gridDim.x) >> 1;
  const int m_tiles = (p.M + k2TileM - 1) / k2TileM;
  const int n_tiles = (p.N + k2TileN - 1) / k2TileN;
  const int num_tiles = p.batch * m_tiles * n_tiles;
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < k2Stages; ++s) {
      mbar_init(&full_bar[s], 1);   // the leader arms it with the bytes of BOTH CTAs
      mbar_init(&empty_bar[s], 1);  // one commit arrival per use
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 8);  // 4 epilogue warps of each CTA
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, k2TmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anybody touches the partner's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs, own halves)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        int b, mt, nt;
        pair_tile_coords(tile, m_tiles, n_tiles, b, mt, nt);
        const int m0 = mt * k2TileM + static_cast<int>(cta_rank) * kBlockM;   // this CTA's 128 rows of A
        const int n0 = nt * k2TileN + static_cast<int>(cta_rank) * k2HalfN;   // this CTA's 128 rows of B
        const int bi = b % p.batch_inner, bo = b / p.batch_inner;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag)) {
            ok = false;
            if (p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutProducer);
            break;
          }
          uint8_t* sa = stage_base + stage * k2StageBytes;
          uint8_t* sb = sa + k2StageA;
          // The leader's barrier counts the pair's bytes: the leader arms it (a local arrive, no fence), the partner only
          // issues loads that signal it.  The partner cannot be a phase ahead: it refills a stage only after the leader's
          // MMAs have consumed it, i.e. after this barrier's previous phase completed.  (A remote arrive with release
          // semantics here cost a cluster-scope memory barrier per k-block and halved the throughput.)
          const uint32_t bar = mapa_u32(&full_bar[stage], 0);
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * k2StageBytes);
          const int k0 = kb * kBlockK;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < kBlockM / 64; ++c) tma_load_4d_pair(sa + c * 8192, &tmA, bar, m0 + c * 64, k0, bi, bo);
          } else {
            tma_load_4d_pair(sa, &tmA, bar, k0, m0, bi, bo);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < k2HalfN / 64; ++c) tma_load_4d_pair(sb + c * 8192, &tmB, bar, n0 + c * 64, k0, bi, bo);
          } else {
            tma_load_4d_pair(sb, &tmB, bar, k0, n0, bi, bo);
          }
          if (++stage == k2Stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (leader only)
    if (leader && elect_one()) {
      constexpr uint32_t idesc_bf16 = make_idesc_f16(k2TileM, k2TileN, true, A_MN, B_MN);
      constexpr uint32_t idesc_fp16 = make_idesc_f16(k2TileM, k2TileN, false, A_MN, B_MN);
      const uint32_t idesc = p.is_bf16 ? idesc_bf16 : idesc_fp16;
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        if (!mbar_wait_bounded(&tmem_empty[buf], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * k2TileN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + stage * k2StageBytes);
          const uint32_t sb = sa + k2StageA;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(sa + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma_f16_pair(tmem_d, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage]);  // frees this stage in both CTAs
          if (++stage == k2Stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&tmem_full[buf]);  // both CTAs' epilogues may read their rows
        buf ^= 1;
        if (buf == 0) acc_phase ^= 1;
      }
      if (!ok && p.status) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutMma);
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    uint8_t* my_staging = staging + (warp - 2) * 2 * 4096;
    int buf = 0;
    uint32_t acc_phase = 0;
    int sbuf = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int b, mt, nt;
      pair_tile_coords(tile, m_tiles, n_tiles, b, mt, nt);
      const int m0 = mt * k2TileM + static_cast<int>(cta_rank) * kBlockM;
      const int n0 = nt * k2TileN;
      const int bi = b % p.batch_inner, bo = b / p.batch_inner;
      if (!mbar_wait_bounded(&tmem_full[buf], acc_phase, abort_flag)) {
        ok = false;
        if (p.status && lane == 0) atomicCAS(p.status, kStatusOk, kStatusWaitTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * k2TileN;
#pragma unroll 1
      for (int chunk = 0; chunk < k2TileN / 64; ++chunk) {
        uint32_t r0[32], r1[32];
        __syncwarp();
        tmem_ld_32x32(taddr + chunk * 64, r0);
        tmem_ld_32x32(taddr + chunk * 64 + 32, r1);
        tmem_ld_wait();
        if (chunk == k2TileN / 64 - 1) {
          // accumulator fully read: hand the buffer back to the leader's MMA thread
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(mapa_u32(&tmem_empty[buf], 0));
        }
        const int col0 = n0 + chunk * 64;
        if (col0 >= p.N || m0 >= p.M) continue;  // warp-uniform
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
        for (int pass = want_aux ? 0 : 1; pass < 2; ++pass) {
          uint8_t* sbuf_ptr = my_staging + sbuf * 4096;
          if (lane == 0) tma_store_wait_read<1>();
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
  cluster_sync_all();  // nobody frees tensor memory or leaves while the partner may still use this CTA's barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, k2TmemCols);
  }
}

template <bool A_MN, bool B_MN>
static int launch_pair(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const CUtensorMap& aux,
                       const GemmParams& p, int grid, cudaStream_t stream) {
  auto kern = gemm2cta_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, k2SmemBytes) != cudaSuccess) return -3;
    configured = true;
  }
  kern<<<grid, kGemmThreads, k2SmemBytes, stream>>>(a, b, c, aux, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace oslo

// Same contract as oslo_gemm_tcgen05 (gemm_sm100a.cu) without the causal modes; the caller picks this entry point for
// large products (at least one 256 x 256 tile per SM pair).  Returns -8 when the shape is not worth a 256-wide tile.
extern "C" int oslo_gemm_tcgen05_2cta(const void* A, const void* B, void* C, const void* bias, void* aux, int M, int N, int K,
                                      int batch, long long lda, long long ldb, long long ldc, long long stride_a,
                                      long long stride_b, long long stride_c, int a_mn, int b_mn, int is_bf16, int epilogue,
                                      int accumulate, int num_sms, int* status, void* stream_ptr, int batch_outer,
                                      long long ostride_a, long long ostride_b, long long ostride_c) {
  using namespace oslo;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  bind_context_to_thread();
  if (batch_outer <= 0) batch_outer = 1;
  const int b_in = batch, b_out = batch_outer;
  batch = b_in * b_out;
  if (b_out > 1 && ((ostride_a % 8) || (ostride_b % 8) || (ostride_c % 8))) return -5;
  auto bad = [](long long v) { return (v % 8) != 0; };
  if (bad(lda) || bad(ldb) || bad(ldc) || (b_in > 1 && (bad(stride_a) || bad(stride_b) || bad(stride_c))) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15) || (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) || (N % 8) ||
      (a_mn && (M % 8)) || (!a_mn && (K % 8)) || (b_mn ? 0 : (K % 8)))
    return -5;
  if (M < k2TileM || N < k2TileN) return -8;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = batch; p.batch_inner = b_in; p.causal = 0; p.stride_c_outer = ostride_c;
  p.m_blocks = (M + k2TileM - 1) / k2TileM;
  p.n_blocks = (N + k2TileN - 1) / k2TileN;
  p.epilogue = epilogue; p.accumulate = accumulate; p.is_bf16 = is_bf16;
  p.bias = bias; p.c_ptr = C; p.ldc = ldc; p.stride_c = stride_c; p.aux_ptr = aux; p.status = status;
  CUtensorMap ta, tb, tc, taux;
  int rc;
  if (a_mn) rc = make_map(&ta, A, is_bf16, M, K, b_in, b_out, lda, stride_a, ostride_a, 64, kBlockK);
  else      rc = make_map(&ta, A, is_bf16, K, M, b_in, b_out, lda, stride_a, ostride_a, kBlockK, kBlockM);
  if (rc) return rc;
  if (b_mn) rc = make_map(&tb, B, is_bf16, N, K, b_in, b_out, ldb, stride_b, ostride_b, 64, kBlockK);
  else      rc = make_map(&tb, B, is_bf16, K, N, b_in, b_out, ldb, stride_b, ostride_b, kBlockK, k2HalfN);
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
  long long clusters = num_sms / 2;
  if (total < clusters) clusters = total;
  const int grid = (int)clusters * 2;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  return a_mn ? (b_mn ? launch_pair<true, true>(ta, tb, tc, taux, p, grid, stream)
                      : launch_pair<true, false>(ta, tb, tc, taux, p, grid, stream))
              : (b_mn ? launch_pair<false, true>(ta, tb, tc, taux, p, grid, stream)
                      : launch_pair<false, false>(ta, tb, tc, taux, p, grid, stream));
}

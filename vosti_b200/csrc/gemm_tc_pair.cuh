// The product for many tokens on pairs of SMs (included by gemm_tc.cu, whose constants and
// epilogue it uses). A cluster of two CTAs computes a tile of 256 tokens x 256 features with
// tcgen05.mma.cta_group::2: each CTA stages its 128 tokens (A) and its 128 of the 256 features (B)
// in its own shared memory, the first CTA of the pair issues every MMA for both tensor cores,
// and each CTA's tensor memory receives the 256 columns of its own 128 tokens. Against the
// single-CTA tile (128 x 256: 48 KB of operands per k-block and SM) an SM takes in 32 KB per
// k-block, so a ring stage can hold two k-blocks and still be three stages deep: the lane that
// issues the MMAs then pays one barrier wait (about 200 cycles, even when the stage landed long
// before) and one commit per eight MMAs, 830 cycles for the 1,024 the tensor cores need, where the
// single-CTA kernel with one k-block per stage pays 610 for 512.
//
// Barriers. full[s] lives in the first CTA and counts the bytes of both CTAs' copies (the copies of
// the second CTA name it through the shared::cluster window); empty[s] and acc_full[a] exist in
// both CTAs and are signalled in both by one multicast tcgen05.commit; acc_empty[a] lives in the
// first CTA and is arrived at by the eight epilogue warps of the pair. No load uses multicast.
// Every wait is bounded; both CTAs meet at a cluster barrier before the first remote access and
// before they exit, on every path.
#pragma once

namespace pair_kernel {
constexpr int PAIR_BN = 256;                       // features per tile (128 per CTA)
constexpr int PAIR_KPS = 2;                        // k-blocks per ring stage: one wait and one commit per eight MMAs
constexpr int PAIR_STAGES = 3;
constexpr int PAIR_BLOCK_BYTES = 2 * A_BYTES;      // one k-block: 128 tokens x 64 + 128 features x 64, bf16
constexpr int PAIR_STAGE_BYTES = PAIR_KPS * PAIR_BLOCK_BYTES;
constexpr int PAIR_THREADS = 192;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t in_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols));
}
// A tile copy of this CTA whose bytes are counted by a barrier given as a shared::cluster address
// (the first CTA's): no multicast, the data lands in this CTA only.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst_smem), "l"(map), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Arrive, once all MMAs issued so far are complete, at the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3)
               : "memory");
}
}  // namespace pair_kernel

__global__ void __launch_bounds__(pair_kernel::PAIR_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ out, int tokens, int features, int k_blocks, int ld_out, int epilogue,
                    int w_tiles, unsigned* status) {
  using namespace pair_kernel;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[PAIR_STAGES];     // used in the first CTA only
  __shared__ __align__(8) uint64_t empty_bar[PAIR_STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];              // used in the first CTA only
  __shared__ uint32_t tmem_base_holder;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                       // 0: issues the MMAs
  const int pairs = gridDim.x / 2, pair = blockIdx.x / 2;
  const int m_tiles = (tokens + 2 * BM - 1) / (2 * BM), n_tiles = (features + PAIR_BN - 1) / PAIR_BN;
  const int total_tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), 8);        // four epilogue warps in each CTA of the pair
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(&tmem_base_holder), 2 * PAIR_BN);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                               // both CTAs' barriers exist before anything names them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_holder;

  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      pdl_wait();
      for (int tile = pair; tile < total_tiles && ok; tile += pairs) {
        const int m0 = (tile % m_tiles) * 2 * BM + (int)rank * BM, n0 = (tile / m_tiles) * PAIR_BN + (int)rank * BM;
        for (int kb0 = 0; kb0 < k_blocks; kb0 += PAIR_KPS, ++it) {
          const int s = it % PAIR_STAGES;
          if (it >= PAIR_STAGES && !mbar_wait(smem_u32(&empty_bar[s]), (it / PAIR_STAGES - 1) & 1, &abort_flag, status)) {
            ok = false;
            break;
          }
          const int held = k_blocks - kb0 < PAIR_KPS ? k_blocks - kb0 : PAIR_KPS;
          if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[s]), (uint32_t)(2 * held * PAIR_BLOCK_BYTES));   // both CTAs' bytes
          const uint32_t bar = in_cta(smem_u32(&full_bar[s]), 0);
          for (int q = 0; q < held; ++q) {
            const int kb = kb0 + q;
            const uint32_t dst = smem_u32(smem + s * PAIR_STAGE_BYTES + q * PAIR_BLOCK_BYTES);
            tma_load_2d_pair(dst, &map_x, kb * BK, m0, bar);
            if (w_tiles) tma_load_2d_pair(dst + A_BYTES, &map_w, 0, (kb * w_tiles + n0 / BM) * BM, bar);
            else tma_load_2d_pair(dst + A_BYTES, &map_w, kb * BK, n0, bar);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PAIR_BN >> 3) << 17) |
                                 ((uint32_t)((2 * BM) >> 4) << 24);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += pairs, ++local) {
        const uint32_t as = local & 1;
        if (local >= 2) ok = mbar_wait(smem_u32(&acc_empty[as]), ((local >> 1) - 1) & 1, &abort_flag, status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * PAIR_BN;
        for (int kb0 = 0; kb0 < k_blocks; kb0 += PAIR_KPS, ++it) {
          const int s = it % PAIR_STAGES;
          ok = mbar_wait(smem_u32(&full_bar[s]), (it / PAIR_STAGES) & 1, &abort_flag, status);
          if (!ok) break;
          tc_fence_after();
          const int held = k_blocks - kb0 < PAIR_KPS ? k_blocks - kb0 : PAIR_KPS;
#pragma unroll
          for (int q = 0; q < PAIR_KPS; ++q) {
            if (q < held) {
              const uint32_t a_addr = smem_u32(smem + s * PAIR_STAGE_BYTES + q * PAIR_BLOCK_BYTES);
              const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k)
                umma_bf16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb0 > 0 || q > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit_pair(smem_u32(&empty_bar[s]));
        }
        if (ok) umma_commit_pair(smem_u32(&acc_full[as]));
      }
    }
  } else {
    const int quarter = warp & 3;
    uint32_t local = 0;
    bool ok = true;
    pdl_wait();
    for (int tile = pair; tile < total_tiles && ok; tile += pairs, ++local) {
      const int m0 = (tile % m_tiles) * 2 * BM + (int)rank * BM, n0 = (tile / m_tiles) * PAIR_BN;
      const uint32_t as = local & 1;
      ok = mbar_wait_warp(smem_u32(&acc_full[as]), (local >> 1) & 1, &abort_flag, status);
      if (!ok) break;
      tc_fence_after();
      const int token = m0 + quarter * 32 + lane;
      const bool row_ok = token < tokens;
#pragma unroll 1
      for (int c0 = 0; c0 < PAIR_BN; c0 += 32) {
        const int f0 = n0 + c0;
        if (f0 >= features) break;
        uint32_t r[32];
        tmem_load32(tmem_base + as * PAIR_BN + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
        if (!row_ok) continue;
        store_token_columns(r, out, token, f0, features, ld_out, epilogue);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(in_cta(smem_u32(&acc_empty[as]), 0));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();                               // nothing of the peer is named after this
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * PAIR_BN);
  }
}

// Paged causal attention for prompts and portions of prompts on the 5th-generation tensor
// cores (tcgen05), head sizes 64 and 128, pages of a multiple of 16 tokens, bfloat16:
//
//   grid = (pairs of query tiles x kv heads, requests), the kv head running fastest, so that
//   CTAs start in the order of their number of key tiles, longest first, across all heads (the
//   tail of the launch is then made of the shortest ones). A CTA takes two tiles of 128 rows of
//   one request and one kv head, where a row is a (query token, query head of the group) pair, so
//   the query heads that share a kv head share its K and V tiles, and so do the two row tiles.
//   Keys are walked in tiles of 64, aligned to the absolute key index. Roles, one warpgroup each:
//     * two softmax warpgroups, one thread per row, one row tile each. A thread reads its row's
//       scores from tensor memory, does the online softmax (base 2, float32) and writes P
//       (rounded to bfloat16) to one of its group's two buffers in shared memory for the second
//       MMA, which adds to the group's running product in tensor memory; with two buffers the
//       exponentials of a tile overlap the product of the tile before. The maximum the
//       exponentials are taken against follows the true maximum lazily: only when it falls
//       behind by more than 8 (P would pass 2^8) is it raised and the running product scaled
//       down in tensor memory. At the end each thread normalises and stores its row.
//     * four loader warps: each brings 16 keys of a tile, one TMA box per 64 features of K
//       and of V straight from the page, into the tensor cores' 128-byte-swizzled layout. A tile
//       serves both row tiles, so a stage lasts twice as long as a row tile's step and three
//       stages cover the latency of the copies. The query rows come as one 4-D box per 64
//       features and row tile.
//     * four threads (one per warp) issue the MMAs: S = Q K^T (M 128, N 64) into the score
//       buffer of the row tile in tensor memory, and P V (M 128, N = head size, V read as
//       an MN-major operand straight from its [key][feature] rows) accumulating in the row
//       tile's product buffer; scores and products of each row tile have a thread each. The
//       scores of a row tile's next key tile are issued as soon as its group has read the last.
//   Registers move from the loader and MMA warpgroups to the softmax ones (setmaxnreg).
//   A row's keys are always taken in the same tiles and the same order, by one thread, whatever
//   the portion and the batch around it: its result does not depend on how the work is cut.
//
// Semantics as in attention_prefill.cu (bottom-right causal alignment, optional window,
// kernels/triton_kernels/fattn_paged.py:176-252): out = acc / l, 0 if l = 0. A box brings
// whole groups of 16 keys; keys of a group beyond the last visible one are overwritten with
// zeros in shared memory, so what unused cache slots hold never reaches the arithmetic.
#include "common.cuh"
#include "mma_util.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

namespace {

constexpr int ROWS = 128;                 // packed rows per row tile: the MMA's M
constexpr int ROW_TILES = 2;              // row tiles per CTA, one per softmax warpgroup
constexpr int KT = 64;                    // keys per tile
constexpr int GROUP_KEYS = 16;            // keys per loader warp and TMA box
constexpr int THREADS = 512;              // softmax 0, softmax 1, loaders, MMA
constexpr int MMA_WARP = 12;
constexpr float LOG2E = 1.4426950408889634f;

template <int D> __host__ __device__ constexpr int kv_stages() { return D == 128 ? 3 : 6; }   // K/V tiles in shared memory

// Byte offset of 16-byte chunk `chunk` (of 8) of row `row` inside a [rows][128 bytes] block
// with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swizzled(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                            const int* __restrict__ row_list, const int* __restrict__ cu_q,
                            const int* __restrict__ kv_len, const int* __restrict__ block_table, int max_pages,
                            int page_size, int page_shift, int num_pages, int nq, int nkv, float scale_log2,
                            int window, unsigned* status) {
  constexpr int NB = D / 64;                          // 64-element blocks of the head size
  constexpr int STAGES = kv_stages<D>();
  constexpr int Q_BYTES = NB * ROWS * 128;            // one row tile of Q
  constexpr int K_BYTES = NB * KT * 128;              // one tile of K; V the same
  constexpr int STAGE_BYTES = 2 * K_BYTES;
  constexpr int P_BYTES = ROWS * 128;                 // [128 rows][64 keys] bfloat16
  constexpr uint32_t TMEM_COLS = (2 * KT + 2 * D) <= 256 ? 256 : 512;
  constexpr uint32_t S_COL = 0, PV_COL = 2 * KT;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;                                // [row tile][NB][128 rows][128 B]
  uint8_t* kv_s = q_s + ROW_TILES * Q_BYTES;
  uint8_t* p_s = kv_s + STAGES * STAGE_BYTES;         // [row tile][2][128 rows][128 B]
  __shared__ __align__(8) uint64_t q_full, kv_full[STAGES], kv_empty[STAGES], edge_bar[KT / GROUP_KEYS];
  __shared__ __align__(8) uint64_t s_full[ROW_TILES], s_empty[ROW_TILES], p_full[ROW_TILES][2], p_empty[ROW_TILES][2];
  __shared__ uint32_t tmem_base_holder;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = row_list ? row_list[blockIdx.y] : blockIdx.y;
  const int g = blockIdx.x % nkv, pair = blockIdx.x / nkv, pairs = gridDim.x / nkv;
  const int group = nq / nkv;
  const int tokens_per_tile = ROWS / group, rows_used = tokens_per_tile * group;
  pdl_wait();
  const int q_start = cu_q[b], q_len = cu_q[b + 1] - q_start, k_len = kv_len[b];
  const int shift = k_len - q_len;
  const int token0 = (pairs - 1 - pair) * ROW_TILES * tokens_per_tile;   // the pairs with most keys start first
  if (token0 >= q_len) return;
  // keys a row tile sees: [its first row's window start, its last row's position]; the CTA walks
  // the tiles from the first tile's first key to the last tile's last key, a row tile stops at
  // its own end
  const int first_key = (window > 0 && shift + token0 - window + 1 > 0) ? shift + token0 - window + 1 : 0;
  const int tile_begin = (first_key / KT) * KT;
  int tiles_of[ROW_TILES], key_end = 0;
#pragma unroll
  for (int w = 0; w < ROW_TILES; ++w) {
    const int t0 = token0 + w * tokens_per_tile;
    const int end = t0 < q_len ? shift + min(q_len - 1, t0 + tokens_per_tile - 1) + 1 : 0;    // exclusive
    tiles_of[w] = end > tile_begin ? (end - tile_begin + KT - 1) / KT : 0;
    key_end = max(key_end, end);
  }
  const int tiles = max(tiles_of[0], tiles_of[1]);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&q_full), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&kv_full[s]), KT / GROUP_KEYS);
      mbar_init(smem_u32(&kv_empty[s]), ROW_TILES);
    }
    for (int i = 0; i < KT / GROUP_KEYS; ++i) mbar_init(smem_u32(&edge_bar[i]), 1);
    for (int i = 0; i < ROW_TILES; ++i) {
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&s_empty[i]), 4);
      for (int j = 0; j < 2; ++j) {
        mbar_init(smem_u32(&p_full[i][j]), 4);
        mbar_init(smem_u32(&p_empty[i][j]), 1);
      }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc(smem_u32(&tmem_base_holder), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_holder;
  pdl_launch_dependents();            // after the tensor memory is ours: a dependent must not take it first

  if (warp < 8) {
    // ------------------------------------------------------------ softmax and accumulation
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    const int wg = warp >> 2;                                    // its row tile
    const int r = threadIdx.x & 127;                             // row of the tile and lane of tensor memory
    const int token = token0 + wg * tokens_per_tile + r / group;
    const bool valid = r < rows_used && token < q_len;
    const int pos = valid ? shift + token : -1;                  // -1: no key is visible, nothing is written
    const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int my_tiles = wg ? tiles_of[1] : tiles_of[0];
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    // m_run is the maximum the exponentials are taken against. It follows the true running
    // maximum lazily: only when a tile's maximum exceeds it by more than RESCALE (P would pass
    // 2^RESCALE) is it raised and the running product, which stays in tensor memory, scaled down.
    constexpr float RESCALE = 8.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    const uint32_t o_tmem = lane_base + PV_COL + wg * D;

    for (int t = 0; t < my_tiles && ok; ++t) {
      const int key0 = tile_begin + t * KT;
      const int buf = t & 1;
      ok = mbar_wait(smem_u32(&s_full[wg]), t & 1, &abort_flag, status);
      if (!ok) break;
      tc_fence_after();
      uint32_t raw[2][32];
      tmem_load32_async(lane_base + S_COL + wg * KT, raw[0]);
      tmem_load32_async(lane_base + S_COL + wg * KT + 32, raw[1]);
      tmem_wait_loads();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_empty[wg]));       // the scores are in registers
      const bool masked = key0 + KT - 1 > pos || key0 < kstart;
      // the maximum is exact in any order: four independent chains, scaled once at the end
      // (scale_log2 > 0, so max(s * scale) = max(s) * scale bit for bit)
      // A row of the tile that holds no token (a lone decode token fills 1 to 16 of the 128 rows)
      // takes no part in the arithmetic: its maximum stays -inf, nothing is written to its row of
      // P, and what the product makes of that row's stale bytes is never stored.
      float part_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (!valid) {
      } else if (masked) {
#pragma unroll
        for (int i = 0; i < KT; ++i)
          if (key0 + i <= pos && key0 + i >= kstart) part_max[i & 3] = fmaxf(part_max[i & 3], __uint_as_float(raw[i >> 5][i & 31]));
      } else {
#pragma unroll
        for (int i = 0; i < KT; ++i) part_max[i & 3] = fmaxf(part_max[i & 3], __uint_as_float(raw[i >> 5][i & 31]));
      }
      const float tile_max = fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3])) * scale_log2;
      // raise the reference maximum? (always at the first visible key: m_run = -inf)
      const bool raise = tile_max > m_run + RESCALE || (m_run == -INFINITY && tile_max > -INFINITY);
      float alpha = 1.f;
      if (raise) {
        alpha = m_run == -INFINITY ? 0.f : fast_exp2(m_run - tile_max);
        m_run = tile_max;
        l_run *= alpha;
      }
      const float safe = m_run == -INFINITY ? 0.f : m_run;
      // ---- this tile's buffer of P is free once the product of the tile before the last one is
      // complete (p_empty of a buffer counts every second product, so a wait is always for the
      // barrier's current or last phase). If any row of the warp raised its maximum, the warp
      // also waits for the last product and scales its rows of the running product.
      if (t >= 2) ok = mbar_wait(smem_u32(&p_empty[wg][buf]), ((t >> 1) - 1) & 1, &abort_flag, status);
      if (t >= 1 && __any_sync(0xffffffffu, raise)) {
        ok = ok && mbar_wait(smem_u32(&p_empty[wg][buf ^ 1]), ((t - 1) >> 1) & 1, &abort_flag, status);
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t v[32];
          tmem_load32(o_tmem + c0, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_store32(o_tmem + c0, v);
        }
        tmem_wait_stores();
        tc_fence_before();
      }
      // ---- P (rounded to bfloat16) into shared memory as the A operand of the second MMA
      uint8_t* p_dst = p_s + (wg * 2 + buf) * P_BYTES;
      float part_sum[4] = {0.f, 0.f, 0.f, 0.f};         // four chains, combined in a fixed order
      if (!valid) {
      } else if (masked) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float p[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int i = 8 * c + e;
            p[e] = fast_exp2(__uint_as_float(raw[i >> 5][i & 31]) * scale_log2 - safe);
            if (!(key0 + i <= pos && key0 + i >= kstart)) p[e] = 0.f;
            part_sum[e & 3] += p[e];
          }
          *reinterpret_cast<uint4*>(p_dst + swizzled(r, c)) =
              make_uint4(pack_bf16(p[0], p[1]), pack_bf16(p[2], p[3]), pack_bf16(p[4], p[5]), pack_bf16(p[6], p[7]));
        }
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float p[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int i = 8 * c + e;
            p[e] = fast_exp2(__uint_as_float(raw[i >> 5][i & 31]) * scale_log2 - safe);
            part_sum[e & 3] += p[e];
          }
          *reinterpret_cast<uint4*>(p_dst + swizzled(r, c)) =
              make_uint4(pack_bf16(p[0], p[1]), pack_bf16(p[2], p[3]), pack_bf16(p[4], p[5]), pack_bf16(p[6], p[7]));
        }
      }
      l_run += (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_full[wg][buf]));
    }
    // ---- the last product complete means every product of the row tile is: normalise and store
    if (ok && my_tiles > 0)
      ok = mbar_wait(smem_u32(&p_empty[wg][(my_tiles - 1) & 1]), ((my_tiles - 1) >> 1) & 1, &abort_flag, status);
    tc_fence_after();
    if (my_tiles > 0) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* dst = out + ((int64_t)(q_start + token) * nq + g * group + r % group) * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t v[32];
        tmem_load32(o_tmem + c0, v);                                  // (all lanes of the warp take part)
        if (ok && valid) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float y[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = __uint_as_float(v[8 * c + e]) * inv;
            *reinterpret_cast<uint4*>(dst + c0 + 8 * c) =
                make_uint4(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]), pack_bf16(y[4], y[5]), pack_bf16(y[6], y[7]));
          }
        }
      }
    }
    tc_fence_before();
  } else if (warp < MMA_WARP) {
    // ------------------------------------------------------------ loaders
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    const int w = warp - 8;                              // keys 16 w .. 16 w + 15 of every tile
    if (w == 0 && lane == 0) {
      // Q rows: row r is token r / group, head r % group: a box [tokens][heads of the group][64]
      // per row tile (rows past the end of the tensor come as zeros and still count as bytes)
      mbar_expect_tx(smem_u32(&q_full), (uint32_t)(ROW_TILES * NB * rows_used * 128));
      for (int rt = 0; rt < ROW_TILES; ++rt)
        for (int nb = 0; nb < NB; ++nb)
          tma_load_4d(smem_u32(q_s + rt * Q_BYTES + nb * (ROWS * 128)), &map_q, 0, g * group,
                      q_start + token0 + rt * tokens_per_tile, nb, smem_u32(&q_full));
    }
    const int* table = block_table + (int64_t)b * max_pages;
    bool ok = true;
    uint32_t edges = 0;
    for (int j = 0; j < tiles && ok; ++j) {
      const int stage = j % STAGES;
      if (j >= STAGES) ok = mbar_wait(smem_u32(&kv_empty[stage]), ((j / STAGES) - 1) & 1, &abort_flag, status);
      if (!ok) break;
      const int lo = tile_begin + j * KT + w * GROUP_KEYS;
      uint8_t* dst = kv_s + stage * STAGE_BYTES + w * GROUP_KEYS * 128;     // + block * (KT * 128); V: + K_BYTES
      int row = -1;
      if (lo + GROUP_KEYS - 1 >= first_key && lo < key_end) {
        const int index = page_shift >= 0 ? lo >> page_shift : lo / page_size;
        const int page = index < max_pages ? table[index] : -1;
        if (page < 0 || page >= num_pages) raise_fault(status, VOSTI_FAULT_PAGE_RANGE);
        else row = (page * nkv + g) * page_size + (lo - index * page_size);
      }
      if (row < 0) {
        // nothing of these keys is visible: zeros, so that P = 0 meets finite values
        for (int i = lane; i < 2 * NB * GROUP_KEYS * 8; i += 32)
          *reinterpret_cast<uint4*>(dst + (i / (GROUP_KEYS * 8)) * (KT * 128) + (i % (GROUP_KEYS * 8)) * 16) = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&kv_full[stage]));
        continue;
      }
      const bool edge = lo + GROUP_KEYS > key_end;       // the box brings keys past the last visible one
      const uint32_t bar = edge ? smem_u32(&edge_bar[w]) : smem_u32(&kv_full[stage]);
      if (lane == 0) mbar_expect_tx(bar, (uint32_t)(2 * NB * GROUP_KEYS * 128));
      __syncwarp();
      if (lane < 2 * NB)
        tma_load_2d(smem_u32(dst + lane * (KT * 128)), lane < NB ? &map_k : &map_v, (lane < NB ? lane : lane - NB) * 64, row, bar);
      if (edge) {
        ok = mbar_wait(bar, edges & 1, &abort_flag, status);
        ++edges;
        const int keep = key_end - lo;                   // rows 0 .. keep-1 stay
        for (int i = lane; i < 2 * NB * GROUP_KEYS * 8; i += 32) {
          const int in_block = i % (GROUP_KEYS * 8);
          if ((in_block >> 3) >= keep)
            *reinterpret_cast<uint4*>(dst + (i / (GROUP_KEYS * 8)) * (KT * 128) + in_block * 16) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&kv_full[stage]));
      }
    }
  } else {
    // ------------------------------------------------------------ MMA issue
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (lane == 0) {
      // Four issuing threads, one per warp: scores of row tile 0, scores of row tile 1, products of
      // row tile 0, products of row tile 1. One thread alone cannot issue a tile's twelve MMAs and
      // wait on its barriers as fast as the tensor core retires them.
      const int role = warp - MMA_WARP, wg = role & 1;
      const int my_tiles = wg ? tiles_of[1] : tiles_of[0];
      constexpr uint32_t idesc_s = umma_instr_desc(ROWS, KT, false);
      constexpr uint32_t idesc_pv = umma_instr_desc(ROWS, D, true);
      // descriptors differ in their start address only: bits [0,14) in units of 16 bytes
      const uint64_t q_desc = smem_desc_sw128(smem_u32(q_s) + wg * Q_BYTES), k_desc = smem_desc_sw128(smem_u32(kv_s));
      const uint64_t v_desc = smem_desc_sw128_mn(smem_u32(kv_s) + K_BYTES, KT * 128);
      bool ok = true;
      if (role < 2) {
        // S_t = Q K_t^T into the score buffer of the row tile
        ok = mbar_wait(smem_u32(&q_full), 0, &abort_flag, status);
        for (int t = 0; t < my_tiles && ok; ++t) {
          const int stage = t % STAGES;
          ok = mbar_wait(smem_u32(&kv_full[stage]), (t / STAGES) & 1, &abort_flag, status);
          if (ok && t >= 1) ok = mbar_wait(smem_u32(&s_empty[wg]), (t - 1) & 1, &abort_flag, status);
          if (!ok) break;
          tc_fence_after();
          const uint64_t kd = k_desc + (uint64_t)((stage * STAGE_BYTES) >> 4);
#pragma unroll
          for (int kb = 0; kb < NB; ++kb)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              umma_bf16(tmem_base + S_COL + wg * KT, q_desc + (uint64_t)((kb * (ROWS * 128) + ks * 32) >> 4),
                        kd + (uint64_t)((kb * (KT * 128) + ks * 32) >> 4), idesc_s, (kb | ks) ? 1u : 0u);
          umma_commit(smem_u32(&s_full[wg]));
        }
      } else {
        // (P V) of tile t, 16 keys per MMA; V rows are [key][64 features] blocks: MN-major.
        // A stage is given back when both row tiles' products of it are complete; a row tile that
        // ends before the other one still counts itself in for the remaining tiles, each time
        // after the tile has arrived, so that it never runs a phase ahead.
        for (int t = 0; t < tiles && ok; ++t) {
          const int stage = t % STAGES;
          ok = mbar_wait(smem_u32(&kv_full[stage]), (t / STAGES) & 1, &abort_flag, status);
          if (!ok) break;
          if (t >= my_tiles) {
            mbar_arrive(smem_u32(&kv_empty[stage]));
            continue;
          }
          ok = mbar_wait(smem_u32(&p_full[wg][t & 1]), (t >> 1) & 1, &abort_flag, status);
          if (!ok) break;
          tc_fence_after();
          const uint64_t vd = v_desc + (uint64_t)((stage * STAGE_BYTES) >> 4);
          const uint64_t p_desc = smem_desc_sw128(smem_u32(p_s) + (wg * 2 + (t & 1)) * P_BYTES);
#pragma unroll
          for (int ks = 0; ks < KT / 16; ++ks)
            umma_bf16(tmem_base + PV_COL + wg * D, p_desc + (uint64_t)((ks * 32) >> 4),
                      vd + (uint64_t)((ks * 16 * 128) >> 4), idesc_pv, (t | ks) ? 1u : 0u);
          umma_commit(smem_u32(&p_empty[wg][t & 1]));
          umma_commit(smem_u32(&kv_empty[stage]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D>
constexpr size_t prefill_tc_smem_bytes() {
  return 1024 + (size_t)ROW_TILES * (D / 64) * ROWS * 128 + (size_t)kv_stages<D>() * 2 * (D / 64) * KT * 128 +
         (size_t)ROW_TILES * 2 * ROWS * 128;
}

}  // namespace

// Whether the tensor-memory kernel takes this head size and page size.
VOSTI_API int vosti_attention_prefill_tc_supported(int d, int page_size) {
  return (d == 64 || d == 128) && page_size > 0 && page_size % GROUP_KEYS == 0;
}

// Arguments and meaning as vosti_attention_prefill, plus the number of rows of q
// (tokens_total); d must be 64 or 128 and page_size a multiple of 16.
VOSTI_API int vosti_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                         const int* row_list, int count, const int* cu_q, const int* kv_len,
                                         const int* block_table, int max_pages, int page_size, int num_pages, int nq,
                                         int nkv, int d, int max_q_len, int tokens_total, float scale, int window,
                                         unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(count >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention_prefill_tc: bad head counts nq=%d nkv=%d", nq, nkv);
  VOSTI_REQUIRE(nq / nkv <= 16, "attention_prefill_tc: at most 16 query heads per kv head, got %d", nq / nkv);
  VOSTI_REQUIRE(vosti_attention_prefill_tc_supported(d, page_size),
                "attention_prefill_tc: head_dim %d must be 64 or 128 and page_size %d a multiple of 16", d, page_size);
  VOSTI_REQUIRE(max_pages > 0 && num_pages > 0 && window >= 0 && tokens_total > 0, "attention_prefill_tc: bad geometry");
  VOSTI_REQUIRE(scale > 0.f, "attention_prefill_tc: the score scale must be positive");
  VOSTI_REQUIRE(count <= 65535, "attention_prefill_tc: too many requests for one launch");
  if (count == 0 || max_q_len <= 0) return VOSTI_OK;
  const int group = nq / nkv;
  const int tokens_per_tile = ROWS / group, tokens_per_cta = ROW_TILES * tokens_per_tile;
  const int64_t cache_rows = (int64_t)num_pages * nkv * page_size;
  VOSTI_REQUIRE(cache_rows < (int64_t)1 << 31, "attention_prefill_tc: cache of %lld rows is too large", (long long)cache_rows);
  CUtensorMap map_q, map_k, map_v;
  {
    const cuuint64_t dims[4] = {64, (cuuint64_t)nq, (cuuint64_t)tokens_total, (cuuint64_t)(d / 64)};
    const cuuint64_t strides[3] = {(cuuint64_t)d * 2, (cuuint64_t)nq * d * 2, 128};
    const cuuint32_t box[4] = {64, (cuuint32_t)group, (cuuint32_t)tokens_per_tile, 1};
    VOSTI_REQUIRE(encode_tensor_map_nd(&map_q, q, 4, dims, strides, box), "attention_prefill_tc: cuTensorMapEncodeTiled failed (q)");
  }
  VOSTI_REQUIRE(cached_tensor_map(k_cache, cache_rows, d, GROUP_KEYS, &map_k) &&
                    cached_tensor_map(v_cache, cache_rows, d, GROUP_KEYS, &map_v),
                "attention_prefill_tc: cuTensorMapEncodeTiled failed (cache)");
  dim3 grid((unsigned)((max_q_len + tokens_per_cta - 1) / tokens_per_cta) * nkv, count);
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; ++page_shift) {}
#define LAUNCH_PREFILL_TC(D)                                                                                         \
  do {                                                                                                               \
    static bool configured = false;                                                                                  \
    if (!configured) {                                                                                               \
      cudaFuncSetAttribute(attention_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,             \
                           (int)prefill_tc_smem_bytes<D>());                                                         \
      configured = true;                                                                                             \
    }                                                                                                                \
    vosti_launch(attention_prefill_tc_kernel<D>, grid, dim3(THREADS), prefill_tc_smem_bytes<D>(), stream, map_q,     \
        map_k, map_v, (bf16*)out, row_list, cu_q, kv_len, block_table, max_pages, page_size, page_shift, num_pages,   \
        nq, nkv, scale * LOG2E, window, status);                                                                      \
  } while (0)
  if (d == 64) LAUNCH_PREFILL_TC(64);
  else LAUNCH_PREFILL_TC(128);
#undef LAUNCH_PREFILL_TC
  VOSTI_LAUNCH_CHECK();
}

// Paged causal attention for prompts and portions of prompts on the 5th-generation tensor
// cores (tcgen05), head sizes 64 and 128, bfloat16:
//
//   grid = (query tiles, kv heads, requests). A CTA takes 128 rows of one request and one kv
//   head, where a row is a (query token, query head of the group) pair, so the query heads
//   that share a kv head share its K and V tiles. Keys are walked in tiles of 64, aligned to
//   the absolute key index. Three roles:
//     * four loader warps gather the tile's K and V rows from the pages with cp.async into
//       shared memory in the tensor cores' 128-byte-swizzled layout (three stages);
//     * one thread issues the MMAs: S = Q K^T (M 128, N 64) into one of two score buffers in
//       tensor memory, and P V (M 128, N = head size, V read as an MN-major operand straight
//       from its [key][feature] rows) into one of two product buffers;
//     * four softmax warps, one thread per row: read the row's scores from tensor memory,
//       online softmax in base 2 and float32, write P (rounded to bfloat16) to shared memory
//       for the second MMA, and add the product tile to the row's accumulator in registers
//       (scaled by the factor of the running maximum), one tile behind the softmax.
//   The MMA of tile j+1's scores and of tile j-1's product run while tile j's softmax does.
//
// Semantics as in attention_prefill.cu (bottom-right causal alignment, optional window,
// kernels/triton_kernels/fattn_paged.py:176-252): out = acc / l, 0 if l = 0.
#include "common.cuh"
#include "mma_util.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int ROWS = 128;                 // packed rows per CTA: the MMA's M
constexpr int KT = 64;                    // keys per tile
constexpr int STAGES = 3;                 // K/V tiles in shared memory
constexpr int COMPUTE_THREADS = 128, LOADER_THREADS = 128;
constexpr int THREADS = COMPUTE_THREADS + LOADER_THREADS + 32;
constexpr int MMA_WARP = (COMPUTE_THREADS + LOADER_THREADS) / 32;
constexpr float LOG2E = 1.4426950408889634f;

// Byte offset of 16-byte chunk `chunk` (of 8) of row `row` inside a [rows][128 bytes] block
// with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swizzled(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache,
                            const bf16* __restrict__ v_cache, bf16* __restrict__ out,
                            const int* __restrict__ row_list, const int* __restrict__ cu_q,
                            const int* __restrict__ kv_len, const int* __restrict__ block_table, int max_pages,
                            int page_size, int page_shift, int num_pages, int nq, int nkv, float scale_log2,
                            int window, unsigned* status) {
  constexpr int NB = D / 64;                          // 64-element blocks of the head size
  constexpr int CHUNKS = D / 8;                       // 16-byte chunks per row
  constexpr int Q_BYTES = NB * ROWS * 128;
  constexpr int K_BYTES = NB * KT * 128;              // one tile of K; V the same
  constexpr int STAGE_BYTES = 2 * K_BYTES;
  constexpr int P_BYTES = ROWS * 128;                 // [128 rows][64 keys] bfloat16
  constexpr uint32_t TMEM_COLS = (2 * KT + 2 * D) <= 256 ? 256 : 512;
  constexpr uint32_t S_COL = 0, PV_COL = 2 * KT;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;
  uint8_t* kv_s = q_s + Q_BYTES;
  uint8_t* p_s = kv_s + STAGES * STAGE_BYTES;
  __shared__ __align__(8) uint64_t q_full, kv_full[STAGES], kv_empty[STAGES];
  __shared__ __align__(8) uint64_t s_full[2], s_empty[2], p_full[2], p_empty[2], pv_full[2], pv_empty[2];
  __shared__ uint32_t tmem_base_holder;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = row_list ? row_list[blockIdx.z] : blockIdx.z;
  const int g = blockIdx.y;
  const int group = nq / nkv;
  const int tokens_per_cta = ROWS / group, rows_used = tokens_per_cta * group;
  pdl_wait();
  const int q_start = cu_q[b], q_len = cu_q[b + 1] - q_start, k_len = kv_len[b];
  const int shift = k_len - q_len;
  const int token0 = (gridDim.x - 1 - blockIdx.x) * tokens_per_cta;   // the tiles with most keys start first
  if (token0 >= q_len) return;
  const int token_hi = min(q_len - 1, token0 + tokens_per_cta - 1);
  const int key_end = shift + token_hi + 1;                            // exclusive
  const int first_key = (window > 0 && shift + token0 - window + 1 > 0) ? shift + token0 - window + 1 : 0;
  const int tile_begin = (first_key / KT) * KT;
  const int tiles = (key_end - tile_begin + KT - 1) / KT;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&q_full), LOADER_THREADS);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&kv_full[s]), LOADER_THREADS);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&s_empty[i]), COMPUTE_THREADS / 32);
      mbar_init(smem_u32(&p_full[i]), COMPUTE_THREADS / 32);
      mbar_init(smem_u32(&p_empty[i]), 1);
      mbar_init(smem_u32(&pv_full[i]), 1);
      mbar_init(smem_u32(&pv_empty[i]), COMPUTE_THREADS / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc(smem_u32(&tmem_base_holder), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_holder;
  pdl_launch_dependents();            // after the tensor memory is ours: a dependent must not take it first

  if (warp < COMPUTE_THREADS / 32) {
    // ------------------------------------------------------------ softmax and accumulation
    const int r = threadIdx.x;                                   // row of the tile and lane of tensor memory
    const int token = token0 + r / group;
    const bool valid = r < rows_used && token < q_len;
    const int pos = valid ? shift + token : -1;                  // -1: no key is visible, nothing is written
    const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;

    // O = O * alpha + (P V) of tile i
    auto accumulate = [&](int i, float alpha) {
      const int pb = i & 1;
      ok = ok && mbar_wait(smem_u32(&pv_full[pb]), (i >> 1) & 1, &abort_flag, status);
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t v[32];
        tmem_load32(lane_base + PV_COL + pb * D + c0, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) o[c0 + j] = fmaf(o[c0 + j], alpha, __uint_as_float(v[j]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&pv_empty[pb]));
    };

    for (int j = 0; j < tiles && ok; ++j) {
      const int sb = j & 1;
      const int key0 = tile_begin + j * KT;
      ok = mbar_wait(smem_u32(&s_full[sb]), (j >> 1) & 1, &abort_flag, status);
      if (!ok) break;
      tc_fence_after();
      uint32_t raw[2][32];
      tmem_load32_async(lane_base + S_COL + sb * KT, raw[0]);
      tmem_load32_async(lane_base + S_COL + sb * KT + 32, raw[1]);
      tmem_wait_loads();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_empty[sb]));       // the scores are in registers
      const bool masked = key0 + KT - 1 > pos || key0 < kstart;
      float tile_max = -INFINITY;
      if (masked) {
#pragma unroll
        for (int i = 0; i < KT; ++i)
          if (key0 + i <= pos && key0 + i >= kstart)
            tile_max = fmaxf(tile_max, __uint_as_float(raw[i >> 5][i & 31]) * scale_log2);
      } else {
#pragma unroll
        for (int i = 0; i < KT; ++i) tile_max = fmaxf(tile_max, __uint_as_float(raw[i >> 5][i & 31]) * scale_log2);
      }
      const float m_new = fmaxf(m_run, tile_max);
      const float safe = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m_run - safe);
      m_run = m_new;
      // ---- P (rounded to bfloat16) into shared memory as the A operand of the second MMA
      if (j >= 2) ok = mbar_wait(smem_u32(&p_empty[sb]), ((j >> 1) - 1) & 1, &abort_flag, status);
      uint8_t* p_dst = p_s + sb * P_BYTES;
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float p[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int i = 8 * c + e;
          p[e] = exp2f(__uint_as_float(raw[i >> 5][i & 31]) * scale_log2 - safe);
          if (masked && !(key0 + i <= pos && key0 + i >= kstart)) p[e] = 0.f;
          sum += p[e];
        }
        *reinterpret_cast<uint4*>(p_dst + swizzled(r, c)) =
            make_uint4(pack_bf16(p[0], p[1]), pack_bf16(p[2], p[3]), pack_bf16(p[4], p[5]), pack_bf16(p[6], p[7]));
      }
      l_run = l_run * alpha + sum;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_full[sb]));
      // ---- the product of the tile before this one has had the time of this softmax
      if (j > 0) accumulate(j - 1, alpha_prev);
      alpha_prev = alpha;
    }
    if (ok) accumulate(tiles - 1, alpha_prev);
    if (ok && valid) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* dst = out + ((int64_t)(q_start + token) * nq + g * group + r % group) * D;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        uint4 v;
        v.x = pack_bf16(o[8 * c] * inv, o[8 * c + 1] * inv);
        v.y = pack_bf16(o[8 * c + 2] * inv, o[8 * c + 3] * inv);
        v.z = pack_bf16(o[8 * c + 4] * inv, o[8 * c + 5] * inv);
        v.w = pack_bf16(o[8 * c + 6] * inv, o[8 * c + 7] * inv);
        *reinterpret_cast<uint4*>(dst + 8 * c) = v;
      }
    }
  } else if (warp < MMA_WARP) {
    // ------------------------------------------------------------ loaders
    const int lt = threadIdx.x - COMPUTE_THREADS;
    // Q rows: row r is token r / group, head r % group of the group
    for (int i = lt; i < ROWS * CHUNKS; i += LOADER_THREADS) {
      const int r = i / CHUNKS, c = i % CHUNKS;
      const int token = token0 + r / group;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows_used && token < q_len)
        v = *reinterpret_cast<const uint4*>(q + ((int64_t)(q_start + token) * nq + g * group + r % group) * D + c * 8);
      *reinterpret_cast<uint4*>(q_s + (c >> 3) * (ROWS * 128) + swizzled(r, c & 7)) = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_arrive(smem_u32(&q_full));

    const int* table = block_table + (int64_t)b * max_pages;
    bool ok = true;
    auto signal = [&](int tile) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(smem_u32(&kv_full[tile % STAGES]));
    };
    for (int j = 0; j < tiles && ok; ++j) {
      if (j >= 2) {                                   // tile j-2 has landed: hand it over before waiting for room
        cp_async_wait<1>();
        signal(j - 2);
      }
      const int stage = j % STAGES;
      if (j >= STAGES) ok = mbar_wait(smem_u32(&kv_empty[stage]), ((j / STAGES) - 1) & 1, &abort_flag, status);
      if (!ok) break;
      const int key0 = tile_begin + j * KT;
      uint8_t* k_dst = kv_s + stage * STAGE_BYTES;
      uint8_t* v_dst = k_dst + K_BYTES;
#pragma unroll
      for (int i = lt; i < KT * CHUNKS; i += LOADER_THREADS) {
        const int r = i / CHUNKS, c = i % CHUNKS;
        const int key = key0 + r;
        bool live = key >= first_key && key < key_end;
        int64_t slot = 0;
        if (live) {
          const int index = page_shift >= 0 ? key >> page_shift : key / page_size;
          const int page = index < max_pages ? table[index] : -1;
          if (page < 0 || page >= num_pages) {
            raise_fault(status, VOSTI_FAULT_PAGE_RANGE);
            live = false;
          } else {
            slot = ((int64_t)page * nkv + g) * page_size + (key - index * page_size);   // row of (page, head, offset)
          }
        }
        const uint32_t offset = (c >> 3) * (KT * 128) + swizzled(r, c & 7);
        if (live) {
          cp_async16(smem_addr(k_dst + offset), k_cache + slot * D + c * 8);
          cp_async16(smem_addr(v_dst + offset), v_cache + slot * D + c * 8);
        } else {
          *reinterpret_cast<uint4*>(k_dst + offset) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(v_dst + offset) = make_uint4(0, 0, 0, 0);
        }
      }
      cp_async_commit();
    }
    if (ok) {
      if (tiles >= 2) {
        cp_async_wait<1>();
        signal(tiles - 2);
      }
      cp_async_wait<0>();
      signal(tiles - 1);
    } else {
      cp_async_wait<0>();
    }
  } else if (lane == 0) {
    // ------------------------------------------------------------ MMA issue
    constexpr uint32_t idesc_s = umma_instr_desc(ROWS, KT, false);
    constexpr uint32_t idesc_pv = umma_instr_desc(ROWS, D, true);
    bool ok = mbar_wait(smem_u32(&q_full), 0, &abort_flag, status);
    const uint32_t q_addr = smem_u32(q_s), kv_addr = smem_u32(kv_s), p_addr = smem_u32(p_s);
    for (int j = 0; j <= tiles && ok; ++j) {
      if (j < tiles) {
        // S_j = Q K_j^T
        const int stage = j % STAGES, sb = j & 1;
        ok = mbar_wait(smem_u32(&kv_full[stage]), (j / STAGES) & 1, &abort_flag, status);
        if (ok && j >= 2) ok = mbar_wait(smem_u32(&s_empty[sb]), ((j >> 1) - 1) & 1, &abort_flag, status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t k_addr = kv_addr + stage * STAGE_BYTES;
#pragma unroll
        for (int kb = 0; kb < NB; ++kb)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16(tmem_base + S_COL + sb * KT, smem_desc_sw128(q_addr + kb * (ROWS * 128) + ks * 32),
                      smem_desc_sw128(k_addr + kb * (KT * 128) + ks * 32), idesc_s, (kb | ks) ? 1u : 0u);
        umma_commit(smem_u32(&s_full[sb]));
      }
      if (j > 0) {
        // (P V) of tile j-1, 16 keys per MMA; V rows are [key][64 features] blocks: MN-major
        const int i = j - 1, stage = i % STAGES, pb = i & 1;
        ok = mbar_wait(smem_u32(&p_full[pb]), (i >> 1) & 1, &abort_flag, status);
        if (ok && i >= 2) ok = mbar_wait(smem_u32(&pv_empty[pb]), ((i >> 1) - 1) & 1, &abort_flag, status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_addr = kv_addr + stage * STAGE_BYTES + K_BYTES;
#pragma unroll
        for (int ks = 0; ks < KT / 16; ++ks)
          umma_bf16(tmem_base + PV_COL + pb * D, smem_desc_sw128(p_addr + pb * P_BYTES + ks * 32),
                    smem_desc_sw128_mn(v_addr + ks * (16 * 128), KT * 128), idesc_pv, ks ? 1u : 0u);
        umma_commit(smem_u32(&pv_full[pb]));
        umma_commit(smem_u32(&p_empty[pb]));
        umma_commit(smem_u32(&kv_empty[stage]));
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
  return 1024 + (size_t)(D / 64) * ROWS * 128 + (size_t)STAGES * 2 * (D / 64) * KT * 128 + 2 * (size_t)ROWS * 128;
}

}  // namespace

// Whether the tensor-memory kernel takes this head size.
VOSTI_API int vosti_attention_prefill_tc_supported(int d) { return d == 64 || d == 128; }

// Same arguments and meaning as vosti_attention_prefill; d must be 64 or 128.
VOSTI_API int vosti_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                         const int* row_list, int count, const int* cu_q, const int* kv_len,
                                         const int* block_table, int max_pages, int page_size, int num_pages, int nq,
                                         int nkv, int d, int max_q_len, float scale, int window, unsigned* status,
                                         cudaStream_t stream) {
  VOSTI_REQUIRE(count >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention_prefill_tc: bad head counts nq=%d nkv=%d", nq, nkv);
  VOSTI_REQUIRE(nq / nkv <= 16, "attention_prefill_tc: at most 16 query heads per kv head, got %d", nq / nkv);
  VOSTI_REQUIRE(d == 64 || d == 128, "attention_prefill_tc: head_dim %d must be 64 or 128", d);
  VOSTI_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0 && window >= 0, "attention_prefill_tc: bad cache geometry");
  VOSTI_REQUIRE(count <= 65535 && nkv <= 65535, "attention_prefill_tc: too many requests or heads for one launch");
  if (count == 0 || max_q_len <= 0) return VOSTI_OK;
  const int group = nq / nkv;
  const int tokens_per_cta = ROWS / group;
  dim3 grid((unsigned)((max_q_len + tokens_per_cta - 1) / tokens_per_cta), nkv, count);
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
    vosti_launch(attention_prefill_tc_kernel<D>, grid, dim3(THREADS), prefill_tc_smem_bytes<D>(), stream,            \
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, row_list, cu_q, kv_len, block_table,  \
        max_pages, page_size, page_shift, num_pages, nq, nkv, scale * LOG2E, window, status);                         \
  } while (0)
  if (d == 64) LAUNCH_PREFILL_TC(64);
  else LAUNCH_PREFILL_TC(128);
#undef LAUNCH_PREFILL_TC
  VOSTI_LAUNCH_CHECK();
}

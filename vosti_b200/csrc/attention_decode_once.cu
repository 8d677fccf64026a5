// The decode attention with one CTA per (token, kv head, segment), the segments of a (token, kv
// head) forming a thread-block cluster. The tile arithmetic, the merge of segments and the
// constants are those of the persistent kernel (attention_decode_common.cuh); the rule that says
// which launch takes which kernel is in attention_decode.cu.
//
// With few tokens the persistent kernel's time is mostly its ends: the producer describing the
// item to the consumers, and at the far end three trips through global memory (the partial
// record, the arrival counter, the records of the other segments). Here every warp works out
// its own share of the item from what the host wrote (position, request, page ids: lane i holds
// the cache row of the warp's tile i), so nothing is handed over inside the CTA before the first
// tiles are requested; and a segment's record goes straight into the shared memory of the
// cluster's first CTA (st.shared::cluster), which waits on an mbarrier the others arrive on and
// merges the segments in segment order with the arithmetic of merge_segments. Same formulas,
// same order of every sum as the persistent kernel at the same segment length: the same bits.
// With many tokens the CTAs run in waves (two to an SM, a new one starting where one ends), which
// measured faster than the persistent kernel's walk over its items at every batch size tried (48
// to 256 requests of 2,048 keys).
//
// Needs pages of a multiple of 16 tokens and segments of at most 4096 keys. The fused form (query
// rows and the token's own key and value from the projection's partial sums) is as in the
// persistent kernel.
#include <mutex>
#include <unordered_map>

#include "attention_decode_common.cuh"

namespace {

using namespace decode_attention;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// Every thread of every CTA of the cluster arrives once and waits once: after the wait all CTAs of
// the cluster run and what each wrote to its own shared memory before it arrived (its barriers) is
// visible to the others. The wait is put off to just before a thread's first access to another
// CTA's shared memory (or its exit), so that nobody stands still for it.
__device__ __forceinline__ void cluster_arrive_all() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_all() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// The address of this CTA's shared-memory location `addr` in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void mb_arrive_cluster(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// Bounded wait on a barrier of this CTA that other CTAs of the cluster arrive on.
__device__ __forceinline__ bool mb_wait_cluster(uint32_t bar, uint32_t parity, unsigned* status) {
  const long long start = clock64();
  while (true) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if (clock64() - start > 2000000000LL) {
      raise_fault(status, VOSTI_FAULT_WAIT_TIMEOUT);
      return false;
    }
  }
}

// A load that is issued where it stands (the compiler moves an ordinary load of read-only data
// down to its first use, which here is behind the set-up the load should overlap).
__device__ __forceinline__ int load_now(const int* p) {
  int v;
  asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}


template <int DMAX, bool EXACT, bool FUSED>
__global__ void __launch_bounds__(THREADS, DMAX <= 128 ? 2 : 1)
attention_decode_once_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                             const bf16* __restrict__ q, bf16* __restrict__ out, const int* __restrict__ token_list,
                             const int* __restrict__ positions, const int* __restrict__ request_of,
                             const int* __restrict__ block_table, int max_pages, int page_size, int page_shift,
                             int num_pages, int whole_rows, int nq, int nkv, int d_runtime, int segment_keys,
                             float scale_log2, int window, unsigned* status, const FusedProjection fused) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[CONSUMERS][RING];
  __shared__ __align__(8) uint64_t q_full, fresh_bar, records_bar;
  __shared__ volatile int abandoned;
  const int d = EXACT ? DMAX : d_runtime;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = nq / nkv;
  const int nb = (d + BOX_COLS - 1) / BOX_COLS;
  const int slot_bytes = 2 * nb * BLOCK_BYTES;
  const int q_pitch = d * 2 + 16;
  const int rec = d + 2, grec = record_floats(d);
  const int segments = (int)cluster_nctarank(), seg = (int)cluster_ctarank();
  uint8_t* ring_base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_base = ring_base + CONSUMERS * RING * slot_bytes;                          // [16][q_pitch]
  float* merge = reinterpret_cast<float*>(q_base + 16 * q_pitch);                       // [CONSUMERS][group][rec]
  bf16* fresh_kv = reinterpret_cast<bf16*>(merge + CONSUMERS * group * rec);            // [2][d]: the token's own key, value
  // [group][segments][grec]: the segments' records, used in the cluster's first CTA only
  float* records = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(fresh_kv + 2 * d) + 15) & ~uintptr_t(15));

  if (threadIdx.x == 32) {
    // the first copy of a tile would else wait for its descriptor
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
  }
  // the item: what the host wrote before the step is read at once
  const int pair = (int)blockIdx.x / segments;
  const int item = pair / nkv, g = pair % nkv;
  const int t = token_list ? load_now(token_list + item) : item;
  const int pos = load_now(positions + t), req = load_now(request_of + t);
  const int slot_of_t = (FUSED && fused.slot_mapping != nullptr) ? load_now(fused.slot_mapping + t) : -1;
  // A consumer warp's tiles are a quarter of the segment; lane i holds the page ids of tiles i and
  // i + 32. Without a window the first tile does not depend on the position, and in the fused form
  // (one token per request) the request's row of the block table is as a rule the token's index:
  // the page ids are asked for together with position and request, on that guess, and asked for
  // again if it fails.
  const int quarter = segment_keys / CONSUMERS;
  const int my_begin = seg * segment_keys + (warp - 1) * quarter;
  const bool guessed = FUSED && window == 0 && warp > 0;   // (the fused form's block table has a row per token)
  int guessed_page[2] = {-1, -1};
  if (guessed) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = lane + 32 * k;
      const int key0 = my_begin + i * TILE;
      const int index = page_shift >= 0 ? key0 >> page_shift : key0 / page_size;
      if (i * TILE < quarter && index < max_pages) guessed_page[k] = load_now(block_table + (int64_t)t * max_pages + index);
    }
  }

  if (threadIdx.x == 0) {
    abandoned = 0;
    for (int w = 0; w < CONSUMERS; ++w)
      for (int r = 0; r < RING; ++r) mb_init(smem_addr(&full_bar[w][r]), 1);
    mb_init(smem_addr(&q_full), FUSED ? CONSUMERS : 1);
    mb_init(smem_addr(&fresh_bar), 1);
    mb_init(smem_addr(&records_bar), segments);       // every CTA of the cluster arrives once, with or without a record
    mb_fence_init();
  }
  // rows of the MMA tile beyond the group stay zero
  for (int i = threadIdx.x; i < 16 * q_pitch / 16; i += THREADS) reinterpret_cast<uint4*>(q_base)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  cluster_arrive_all();
  pdl_launch_dependents();

  const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int seg_begin = seg * segment_keys, seg_end = min(seg_begin + segment_keys, pos + 1);
  const bool visible = !(seg_begin > pos || seg_end <= kstart);
  const int p_first = kstart / segment_keys, p_last = min(pos / segment_keys, segments - 1);   // the segments that hold visible keys
  const uint32_t leader_bar = map_to_rank(smem_addr(&records_bar), 0);

  if (!visible && seg != 0) {
    // nothing of this segment is visible: count the CTA in and leave
    cluster_wait_all();
    if (threadIdx.x == 0) mb_arrive_cluster(leader_bar);
    pdl_wait();                                        // (the chain of completed kernels stays unbroken)
    return;
  }
  // does the token's own key and value come with this item? (fused form, the segment of its position)
  int64_t slot = -1;
  if (FUSED && visible && pos / segment_keys == seg && fused.slot_mapping != nullptr) {
    slot = slot_of_t;
    if (slot >= fused.num_slots || slot < -1) {
      if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
      slot = -1;
    }
  }
  int rope_pos = pos;
  if (FUSED && fused.cos_table != nullptr && (pos < 0 || pos >= fused.max_positions)) {
    if (threadIdx.x == 32) raise_fault(status, VOSTI_FAULT_POSITION_RANGE);
    rope_pos = 0;
  }

  if (warp == 0) {
    // ------------------------------------------------------------ helper warp
    pdl_wait();
    if (visible && !FUSED && lane == 0) {
      mb_expect_tx(smem_addr(&q_full), (uint32_t)(group * d * 2));
      for (int row = 0; row < group; ++row)
        bulk_copy_g2s(smem_addr(q_base + row * q_pitch), q + ((int64_t)t * nq + g * group + row) * d, (uint32_t)(d * 2),
                      smem_addr(&q_full));
    }
    if (FUSED && slot >= 0) {
      const float* token_partial = fused.partial + (int64_t)t * (nq + 2 * nkv) * d;
      const int64_t cache_row = ((slot / page_size) * nkv + g) * page_size + slot % page_size;   // [pages, kv heads, page_size, d]
      head_from_partial<bf16, (DMAX + 63) / 64>(token_partial + (int64_t)(nq + g) * d, fused.splits, fused.plane, d, lane,
                                                fused.k_norm_w, fused.norm_w_is_f32, fused.eps, fused.cos_table, fused.sin_table,
                                                rope_pos, fresh_kv, fused.k_cache + cache_row * d);
      head_from_partial<bf16, (DMAX + 63) / 64>(token_partial + (int64_t)(nq + nkv + g) * d, fused.splits, fused.plane, d, lane,
                                                nullptr, 0, fused.eps, nullptr, nullptr, 0, fresh_kv + d,
                                                fused.v_cache + cache_row * d);
      __syncwarp();
      if (lane == 0) mb_arrive(smem_addr(&fresh_bar));
    }
    cluster_wait_all();
    return;
  }

  // -------------------------------------------------------------- consumers
  const int cw = warp - 1;
  const int ctid = threadIdx.x - 32;
  const bool upper_rows_live = group > 8;
  const int k_row = (lane & 7) + (lane >> 4) * 8, k_half = (lane >> 3) & 1;
  const int v_row = (lane & 7) + ((lane >> 3) & 1) * 8, v_half = lane >> 4;
  const uint32_t k_lane = k_row * 128, k_xor = (uint32_t)((k_half ^ (k_row & 7)) << 4);
  const uint32_t v_lane = v_row * 128, v_xor = (uint32_t)((v_half ^ (v_row & 7)) << 4);

  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  float o[DMAX / 8][4];
#pragma unroll
  for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  if (visible) {
    // this warp's tiles: a quarter of the segment, aligned to the key index
    const int my_end = min(my_begin + quarter, seg_end);
    const int first_tile = max(my_begin, (kstart / TILE) * TILE);
    const int tiles = my_end > first_tile ? (my_end - first_tile + TILE - 1) / TILE : 0;      // <= 64
    // cache row of each tile's first key: lane i holds tiles i and i + 32
    int rows[2] = {-1, -1};
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = lane + 32 * k;
      if (i < tiles) {
        const int key0 = first_tile + i * TILE;
        const int index = page_shift >= 0 ? key0 >> page_shift : key0 / page_size;
        int page = guessed_page[k];                    // (first_tile == my_begin when the guess was made)
        if (!guessed || req != t) page = index < max_pages ? block_table[(int64_t)req * max_pages + index] : -1;
        if (page >= 0 && page < num_pages) rows[k] = (page * nkv + g) * page_size + (key0 - index * page_size);
      }
    }
    int requested = 0;
    auto request_tile = [&]() {
      const int i = requested++;
      int row = __shfl_sync(0xffffffffu, i < 32 ? rows[0] : rows[1], i & 31);
      if (row < 0) {
        raise_fault(status, VOSTI_FAULT_PAGE_RANGE);
        row = 0;
      }
      const uint32_t ring_slot = (uint32_t)i % RING;
      const uint32_t dst = smem_addr(ring_base + (cw * RING + ring_slot) * slot_bytes);
      const uint32_t bar = smem_addr(&full_bar[cw][ring_slot]);
      if (lane == 0) {
        mb_expect_tx(bar, (uint32_t)slot_bytes);
        if (whole_rows) {
          tma_load_3d(dst, &map_k, 0, row, 0, bar);
          tma_load_3d(dst + nb * BLOCK_BYTES, &map_v, 0, row, 0, bar);
        } else {
          for (int cb = 0; cb < nb; ++cb) {
            tma_load_2d(dst + cb * BLOCK_BYTES, &map_k, cb * BOX_COLS, row, bar);
            tma_load_2d(dst + (nb + cb) * BLOCK_BYTES, &map_v, cb * BOX_COLS, row, bar);
          }
        }
      }
      __syncwarp();
    };
    // The cache rows a tile brings were written in earlier steps (fused: the token's own row is
    // replaced in shared memory); unfused, the kernel before this one wrote the newest row.
    if (!FUSED) pdl_wait();
    while (requested < min(tiles, RING)) request_tile();
    if (FUSED) {
      // this warp's share of the query rows, from the projection's partial sums
      pdl_wait();
      const float* token_partial = fused.partial + (int64_t)t * (nq + 2 * nkv) * d;
      for (int row = cw; row < group; row += CONSUMERS)
        head_from_partial<bf16, (DMAX + 63) / 64>(token_partial + (int64_t)(g * group + row) * d, fused.splits, fused.plane, d, lane,
                                                  fused.q_norm_w, fused.norm_w_is_f32, fused.eps, fused.cos_table, fused.sin_table,
                                                  rope_pos, reinterpret_cast<bf16*>(q_base + row * q_pitch), (bf16*)nullptr);
      __syncwarp();
      if (lane == 0) mb_arrive(smem_addr(&q_full));
    }
    wait_or_abandon(smem_addr(&q_full), 0, status, &abandoned);
    const uint8_t* q_s = q_base;
    constexpr bool Q_IN_REGISTERS = DMAX <= 128;
    uint32_t qa[Q_IN_REGISTERS ? DMAX / 16 : 1][4];
    if (Q_IN_REGISTERS) {
#pragma unroll
      for (int kk = 0; kk < DMAX / 16; ++kk)
        if (kk * 16 < d)
          ldmatrix_x4(qa[Q_IN_REGISTERS ? kk : 0], smem_addr(q_s + (lane & 15) * q_pitch + (kk * 16 + (lane >> 4) * 8) * 2));
    }
    for (int tile = 0; tile < tiles; ++tile) {
      const uint32_t ring_slot = (uint32_t)tile % RING;
      wait_or_abandon(smem_addr(&full_bar[cw][ring_slot]), (uint32_t)(tile / RING) & 1, status, &abandoned);
      uint8_t* tile_s = ring_base + (cw * RING + ring_slot) * slot_bytes;
      const uint32_t ks = smem_addr(tile_s), vs = ks + nb * BLOCK_BYTES;
      const int key0 = first_tile + tile * TILE;
      bool edge = false;
      if (FUSED && slot >= 0 && pos >= key0 && pos < key0 + TILE) {
        // the token's own key and value, made by the helper warp: over the row the box brought
        wait_or_abandon(smem_addr(&fresh_bar), 0, status, &abandoned);
        const int r = pos - key0;
        const uint4* src = reinterpret_cast<const uint4*>(fresh_kv);
        const int chunks = d >> 3;                     // 16-byte pieces of a row
        for (int i = lane; i < 2 * chunks; i += 32) {
          const int c = i % chunks;                    // piece of the key (i < chunks) or of the value
          uint8_t* block = tile_s + ((i < chunks ? 0 : nb) + (c >> 3)) * BLOCK_BYTES;
          *reinterpret_cast<uint4*>(block + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = src[i];
        }
        edge = true;                                   // written by threads: fence before the slot is refilled
        __syncwarp();
      }
      if (key0 < kstart || key0 + TILE - 1 > pos) {
        // a box brought keys that are masked: their V rows must not reach the MMA (0 * NaN)
        edge = true;
        uint8_t* vrows = tile_s + nb * BLOCK_BYTES;
        for (int i = lane; i < nb * TILE * 8; i += 32) {
          const int r = (i >> 3) % TILE;
          if (key0 + r < kstart || key0 + r > pos) reinterpret_cast<uint4*>(vrows)[i] = make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
      }
      attend_tile<DMAX, Q_IN_REGISTERS>(ks, vs, qa, q_s, q_pitch, d, key0, kstart, pos, scale_log2, upper_rows_live, k_lane, k_xor,
                                        v_lane, v_xor, m_row, l_row, o);
      __syncwarp();                                    // every lane is done with this slot: refill it
      if (edge) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      if (requested < tiles) request_tile();
    }
  } else {
    pdl_wait();                                        // (the first CTA of a cluster without visible keys of its own)
  }

  // ---- merge the four consumers in warp order (as the persistent kernel does)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 1);
    l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = (lane >> 2) + 8 * r;
    if (row < group) {
      float* dst = merge + ((int64_t)cw * group + row) * rec;
      if ((lane & 3) == 0) {
        dst[0] = m_row[r];
        dst[1] = l_row[r];
      }
#pragma unroll
      for (int nt = 0; nt < DMAX / 8; ++nt) {
        if (nt * 8 < d) {
          dst[2 + nt * 8 + (lane & 3) * 2] = o[nt][2 * r];
          dst[2 + nt * 8 + (lane & 3) * 2 + 1] = o[nt][2 * r + 1];
        }
      }
    }
  }
  consumer_sync();
  cluster_wait_all();
  if (visible) {
    // the segment's record into the first CTA's shared memory
    for (int row = 0; row < group; ++row) {
      float weight[CONSUMERS];
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < CONSUMERS; ++w) m = fmaxf(m, merge[((int64_t)w * group + row) * rec]);
#pragma unroll
      for (int w = 0; w < CONSUMERS; ++w) {
        const float mw = merge[((int64_t)w * group + row) * rec];
        weight[w] = mw == -INFINITY ? 0.f : fast_exp2(mw - m);
      }
      const uint32_t dst = map_to_rank(smem_addr(records + ((int64_t)row * segments + seg) * grec), 0);
      for (int c = ctid; c < rec; c += CONSUMERS * 32) {
        float value;
        if (c == 0) {
          value = m;
        } else {
          value = 0.f;
#pragma unroll
          for (int w = 0; w < CONSUMERS; ++w) value += merge[((int64_t)w * group + row) * rec + c] * weight[w];
        }
        st_cluster_f32(dst + 4u * (uint32_t)(c < 2 ? c : c + 2), value);   // the accumulator starts at float 4 of a record
      }
    }
  }
  asm volatile("fence.acq_rel.cluster;" ::: "memory");
  consumer_sync();                                     // every consumer's share of the record is on its way
  if (ctid == 0) mb_arrive_cluster(leader_bar);
  if (seg != 0) return;

  // ---- the cluster's first CTA: all segments have arrived; merge them in segment order
  if (!mb_wait_cluster(smem_addr(&records_bar), 0, status)) return;
  for (int row = cw; row < group; row += CONSUMERS)
    merge_segments<false>(records + (int64_t)row * segments * grec, out + ((int64_t)t * nq + g * group + row) * d, p_first, p_last, d);
}

// How many clusters of `cluster` CTAs with `smem` bytes each the GPU can run at once (0: none, or
// the size cannot be scheduled); asked once per (kernel, size, bytes).
template <typename Kernel>
int clusters_that_fit(Kernel kernel, int cluster, size_t smem) {
  static std::unordered_map<uint64_t, int> known;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  const uint64_t key = ((uint64_t)smem << 8) | (uint64_t)cluster;
  auto it = known.find(key);
  if (it != known.end()) return it->second;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)cluster);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = (unsigned)cluster;
  attribute[0].val.clusterDim.y = attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) {
    (void)cudaGetLastError();
    clusters = 0;
  }
  known.emplace(key, clusters);
  return clusters;
}

template <int DMAX, bool EXACT, bool FUSED>
int launch_as(const OnceLaunch& a, size_t smem) {
  auto kernel = attention_decode_once_kernel<DMAX, EXACT, FUSED>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ONCE_SMEM_CAP);
    cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    configured = true;
  }
  const dim3 grid((unsigned)((int64_t)a.count * a.nkv * a.segments));
  cudaError_t e;
  if (a.segments == 1) {
    // no cluster to form: an ordinary launch, whose CTAs are spread over all SMs first
    e = vosti_launch(kernel, grid, dim3(THREADS), smem, a.stream, a.map_k, a.map_v, a.q, a.out, a.token_list, a.positions,
                     a.request_of, a.block_table, a.max_pages, a.page_size, a.page_shift, a.num_pages, a.whole_rows, a.nq, a.nkv,
                     a.d, a.segment_keys, a.scale_log2, a.window, a.status, a.fused);
  } else {
    if (clusters_that_fit(kernel, a.segments, smem) < 1) return 0;
    e = vosti_launch_clusters(kernel, grid, dim3(THREADS), (unsigned)a.segments, smem, a.stream, a.map_k, a.map_v, a.q, a.out,
                              a.token_list, a.positions, a.request_of, a.block_table, a.max_pages, a.page_size, a.page_shift,
                              a.num_pages, a.whole_rows, a.nq, a.nkv, a.d, a.segment_keys, a.scale_log2, a.window, a.status,
                              a.fused);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    vosti_set_error("attention_decode (one CTA per item): %s", cudaGetErrorString(e));
    return -(int)e;
  }
  return 1;
}

template <int DMAX, bool EXACT>
int launch_form(const OnceLaunch& a, size_t smem) {
  return a.fused.partial != nullptr ? launch_as<DMAX, EXACT, true>(a, smem) : launch_as<DMAX, EXACT, false>(a, smem);
}

}  // namespace

namespace decode_attention {

size_t once_smem_bytes(int d, int group, int segments) {
  const size_t nb = (d + BOX_COLS - 1) / BOX_COLS;
  return 1024 + (size_t)CONSUMERS * RING * 2 * nb * BLOCK_BYTES + (size_t)16 * ((size_t)d * 2 + 16) +
         (size_t)CONSUMERS * group * (d + 2) * sizeof(float) + (size_t)2 * d * 2 + 16 +
         (size_t)segments * group * record_floats(d) * sizeof(float);
}

int launch_once(const OnceLaunch& a) {
  const int d = a.d;
  const size_t smem = once_smem_bytes(d, a.nq / a.nkv, a.segments);
  if (smem > ONCE_SMEM_CAP) return 0;
  if (d == 64) return launch_form<64, true>(a, smem);
  if (d == 128) return launch_form<128, true>(a, smem);
  if (d == 256) return launch_form<256, true>(a, smem);
  if (d < 64) return launch_form<64, false>(a, smem);
  if (d < 128) return launch_form<128, false>(a, smem);
  return launch_form<256, false>(a, smem);
}

}  // namespace decode_attention

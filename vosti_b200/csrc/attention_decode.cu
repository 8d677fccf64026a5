// Paged attention for single query tokens (decode rows and very short portions),
// bfloat16, on the tensor cores with split keys ("flash decoding"), as a persistent,
// warp-specialised kernel:
//
//   A work item is one token, one kv head with the whole group of query heads that share it
//   (they fill the MMA's 16 rows), and one segment of `segment_keys` keys counted from key 0
//   of the request. CTA c walks over the items c, c + grid, ... Warp 0 is the producer: one
//   item ahead of the consumers it describes the next item (token, position, segment), resolves
//   the block table into the cache row of every 16-key tile, and fetches the query rows; what
//   the host wrote before the step is read before the kernel waits for its predecessor. Warps
//   1..4 are the consumers: each takes a quarter of the segment and requests its own tiles by
//   TMA (one box per 16 keys of K and one of V straight from the page, 128-byte swizzle) into
//   a ring of two buffers, across item boundaries; it runs the online softmax (base 2,
//   float32) with mma.sync m16n8k16 for Q.K^T and P.V. The four are merged in warp order into
//   an unnormalised partial (max, sum, accumulator) per query head. The CTA that finishes
//   last for a (token, kv head) merges the segments in segment order and normalises; a CTA
//   counts itself in one item late, so that the wait for its own stores overlaps the next item.
//
// The segmentation depends on the key index and on the launch (its length is chosen from the
// number of tokens and the longest context, or pinned), never on the companions' contents.
// Formulas as in kernels/triton_kernels/fattn_paged.py:176-252: kv head = query head * nkv / nq,
// scale * log2(e), causal up to the token's own position, optional window, P rounded to
// bfloat16 before P.V (:246), out = acc / l (0 if l = 0).
//
// Fused form for steps in which every request brings one token: the kernel takes the QKV
// projection's unsummed K-split partial sums instead of finished query rows. The producer sums
// the splits of its item's query heads in split order, applies the per-head norm and the
// rotation (the arithmetic of qkv_post.cu, operation by operation: head_post.cuh) and puts the
// rows where the copies would have put them; for the item whose segment holds the token's own
// position it does the same for the token's key and copies its value, stores both in the cache
// for the steps to come and hands them to the consumers, which write them over the tile's row
// for that position after the tile has landed (the cache row a box brings there is not yet the
// new one). One kernel and one boundary less per layer.
//
// A box of 16 keys is read whole when pages hold a multiple of 16 tokens; the V rows of keys
// beyond the token's position (or before its window) are overwritten with zeros in shared
// memory and their scores masked, so what unused cache slots hold never reaches the
// arithmetic. Other page sizes read row by row, masked keys not at all.
#include "attention_decode_common.cuh"

namespace {

using namespace decode_attention;

struct ItemMeta {
  int t, pos, item, g, seg, kstart, request, fresh;  // t < 0: no more items; fresh: the token's own key and value come with it
};

// DMAX bounds the head size; with EXACT the head size is DMAX itself. FUSED: the query rows and
// the token's own key and value are made here from the projection's partial sums (`fused`).
template <int DMAX, bool EXACT, bool FUSED>
__global__ void __launch_bounds__(THREADS, DMAX <= 128 ? 2 : 1)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const bf16* __restrict__ q, float* __restrict__ partial, bf16* __restrict__ out,
                        int* __restrict__ arrivals, const int* __restrict__ token_list,
                        const int* __restrict__ positions, const int* __restrict__ request_of,
                        const int* __restrict__ block_table, int max_pages, int page_size, int page_shift,
                        int num_pages, int whole_pages, int whole_rows, int count, int nq, int nkv, int d_runtime,
                        int segment_keys, int max_segments, float scale_log2, int window, unsigned* status,
                        const FusedProjection fused) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[CONSUMERS][RING];
  __shared__ __align__(8) uint64_t q_full[Q_BUFFERS], q_empty[Q_BUFFERS], meta_bar[Q_BUFFERS], fresh_bar[Q_BUFFERS];
  __shared__ ItemMeta item_meta[Q_BUFFERS];
  __shared__ ItemMeta consumer_meta;       // the consumers' common copy: they all take the same decisions
  __shared__ int tile_rows[Q_BUFFERS][MAX_SEGMENT_PAGES];   // cache row of each tile's first key (whole pages)
  __shared__ int segment_pages[MAX_SEGMENT_PAGES];
  __shared__ int last_to_arrive;
  __shared__ volatile int abandoned;
  const int d = EXACT ? DMAX : d_runtime;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = nq / nkv;                       // query heads per kv head, <= 16
  const int nb = (d + BOX_COLS - 1) / BOX_COLS;     // column blocks per K or V tile
  const int slot_bytes = 2 * nb * BLOCK_BYTES;      // one ring slot: K blocks, then V blocks
  const int q_pitch = d * 2 + 16;                   // bytes per staged Q row: conflict-free ldmatrix
  const int rec = d + 2;
  uint8_t* ring_base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_base = ring_base + CONSUMERS * RING * slot_bytes;                         // [Q_BUFFERS][16][q_pitch]
  float* merge = reinterpret_cast<float*>(q_base + Q_BUFFERS * 16 * q_pitch);         // [CONSUMERS][group][rec]
  bf16* fresh_kv = reinterpret_cast<bf16*>(merge + CONSUMERS * group * rec);           // [Q_BUFFERS][2][d]: the token's own key, value

  if (threadIdx.x == 0) {
    abandoned = 0;
    for (int w = 0; w < CONSUMERS; ++w)
      for (int r = 0; r < RING; ++r) mb_init(smem_addr(&full_bar[w][r]), 1);
    for (int b = 0; b < Q_BUFFERS; ++b) {
      // fused: every consumer warp makes its share of the query rows and counts itself in
      mb_init(smem_addr(&q_full[b]), FUSED ? CONSUMERS : 1);
      mb_init(smem_addr(&fresh_bar[b]), 1);
      mb_init(smem_addr(&q_empty[b]), CONSUMERS);
      mb_init(smem_addr(&meta_bar[b]), 1);
    }
    mb_fence_init();
  }
  // rows of the MMA tile beyond the group stay zero for the whole kernel
  for (int i = threadIdx.x; i < Q_BUFFERS * 16 * q_pitch / 16; i += THREADS)
    reinterpret_cast<uint4*>(q_base)[i] = make_uint4(0, 0, 0, 0);
  if (!whole_pages)       // rows of masked keys are not loaded: what they held before must be finite
    for (int i = threadIdx.x; i < CONSUMERS * RING * slot_bytes / 16; i += THREADS)
      reinterpret_cast<uint4*>(ring_base)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  pdl_launch_dependents();
  // What the host wrote before the step (positions, requests, block tables, the token list) is
  // read at once; q and the newest cache rows come from the kernel before this one: the producer
  // waits for it before it fetches q, the consumers before they request their first tile.

  // items in segment-major order: the short last segments of the requests come last, which
  // evens out what the CTAs get
  const int pairs = count * nkv;                      // the launcher keeps pairs * max_segments below 2^31
  const int total_items = pairs * max_segments;
  const int quarter = segment_keys / CONSUMERS;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    // It describes the items to the consumers one item ahead: token, position, the cache row
    // of every tile (block table resolved) and the query rows. The consumers fetch K and V.
    uint32_t q_issued = 0;
    bool waited = false;
    const int my_items = (int)blockIdx.x < total_items ? (total_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    for (int base = 0; base < my_items; base += 32) {
      // token, position and request of 32 items at once: lane l holds item base + l
      int t_l = 0, pos_l = -1, req_l = 0;
      if (base + lane < my_items) {
        const int idx = (int)blockIdx.x + (base + lane) * (int)gridDim.x;
        const int item = (idx % pairs) / nkv;
        t_l = token_list ? token_list[item] : item;
        pos_l = positions[t_l];
        req_l = request_of[t_l];
      }
      const int n = min(32, my_items - base);
      // page ids of an item's segment, MAX_SEGMENT_PAGES / 32 per lane; -1 where none is needed
      int next_pages[MAX_SEGMENT_PAGES / 32];
      auto fetch_pages = [&](int j) {
        const int pos = __shfl_sync(0xffffffffu, pos_l, j), req = __shfl_sync(0xffffffffu, req_l, j);
        const int idx = (int)blockIdx.x + (base + j) * (int)gridDim.x;
        const int seg = idx / pairs;
        const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        const int seg_begin = seg * segment_keys;
        const int first_index = seg_begin / page_size;
        const int lo = kstart / page_size, hi = min(pos, seg_begin + segment_keys - 1) / page_size;
        const int* table = block_table + (int64_t)req * max_pages;
#pragma unroll
        for (int k = 0; k < MAX_SEGMENT_PAGES / 32; ++k) {
          const int index = first_index + lane + 32 * k;
          next_pages[k] = (index >= lo && index <= hi && index < max_pages) ? table[index] : -1;
        }
      };
      if (whole_pages) fetch_pages(0);
      for (int j = 0; j < n; ++j) {
        const int t = __shfl_sync(0xffffffffu, t_l, j), pos = __shfl_sync(0xffffffffu, pos_l, j);
        const int req = __shfl_sync(0xffffffffu, req_l, j);
        const int idx = (int)blockIdx.x + (base + j) * (int)gridDim.x;
        const int seg = idx / pairs;
        const int g = (idx % pairs) % nkv;
        const int item = (idx % pairs) / nkv;
        const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        const int seg_begin = seg * segment_keys, seg_end = min(seg_begin + segment_keys, pos + 1);
        if (whole_pages) {
          __syncwarp();
#pragma unroll
          for (int k = 0; k < MAX_SEGMENT_PAGES / 32; ++k) segment_pages[lane + 32 * k] = next_pages[k];
          __syncwarp();
          if (j + 1 < n) fetch_pages(j + 1);         // in flight while this item is described
        }
        if (seg_begin > pos || seg_end <= kstart) continue;          // nothing visible in this segment
        const uint32_t qb = q_issued % Q_BUFFERS;
        if (q_issued >= Q_BUFFERS)
          wait_or_abandon(smem_addr(&q_empty[qb]), ((q_issued / Q_BUFFERS) - 1) & 1, status, &abandoned);
        if (whole_pages) {
          const int first_index = seg_begin / page_size;
          for (int i = lane; i < segment_keys / TILE; i += 32) {
            const int key0 = seg_begin + i * TILE;
            const int index = page_shift >= 0 ? key0 >> page_shift : key0 / page_size;
            const int page = segment_pages[min(index - first_index, MAX_SEGMENT_PAGES - 1)];
            tile_rows[qb][i] = (page < 0 || page >= num_pages) ? -1 : (page * nkv + g) * page_size + (key0 - index * page_size);
          }
          __syncwarp();
        }
        // The description rests on what the host wrote before the step. The query rows (and in the
        // fused form the partial sums) come from the kernel before this one.
        if (!FUSED && !waited) {
          pdl_wait();
          waited = true;
        }
        if (!FUSED) {
          if (lane == 0) {
            // the description first: the consumers request their tiles while the query rows travel
            item_meta[qb] = ItemMeta{t, pos, item, g, seg, kstart, req, 0};
            mb_arrive(smem_addr(&meta_bar[qb]));
            mb_expect_tx(smem_addr(&q_full[qb]), (uint32_t)(group * d * 2));
            // the item's query rows are contiguous in q: the heads of one group
            for (int row = 0; row < group; ++row)
              bulk_copy_g2s(smem_addr(q_base + (qb * 16 + row) * q_pitch), q + ((int64_t)t * nq + g * group + row) * d,
                            (uint32_t)(d * 2), smem_addr(&q_full[qb]));
          }
        } else {
          // ---- fused: the consumers make the query rows from the projection's partial sums; in the
          // segment of the token's own position the producer makes the token's key and value
          int64_t slot = -1;
          if (pos / segment_keys == seg && fused.slot_mapping != nullptr) {
            slot = fused.slot_mapping[t];
            if (slot >= fused.num_slots || slot < -1) {
              if (lane == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
              slot = -1;
            }
          }
          if (lane == 0) {
            item_meta[qb] = ItemMeta{t, pos, item, g, seg, kstart, req, slot >= 0 ? 1 : 0};
            mb_arrive(smem_addr(&meta_bar[qb]));
          }
          if (slot >= 0) {
            if (!waited) {
              pdl_wait();
              waited = true;
            }
            int rope_pos = pos;
            if (fused.cos_table != nullptr && (pos < 0 || pos >= fused.max_positions)) rope_pos = 0;   // (the consumers report it)
            const float* token_partial = fused.partial + (int64_t)t * (nq + 2 * nkv) * d;
            // cache row of the slot: [pages, kv heads, page_size, d]
            const int64_t cache_row = ((slot / page_size) * nkv + g) * page_size + slot % page_size;
            bf16* mine = fresh_kv + (int64_t)qb * 2 * d;
            head_from_partial<bf16, (DMAX + 63) / 64>(token_partial + (int64_t)(nq + g) * d, fused.splits, fused.plane, d, lane, fused.k_norm_w,
                              fused.norm_w_is_f32, fused.eps, fused.cos_table, fused.sin_table, rope_pos, mine,
                              fused.k_cache + cache_row * d);
            head_from_partial<bf16, (DMAX + 63) / 64>(token_partial + (int64_t)(nq + nkv + g) * d, fused.splits, fused.plane, d, lane, nullptr, 0,
                              fused.eps, nullptr, nullptr, 0, mine + d, fused.v_cache + cache_row * d);
            __syncwarp();
            if (lane == 0) mb_arrive(smem_addr(&fresh_bar[qb]));     // key and value are in shared memory
          }
        }
        ++q_issued;
      }
    }
    // ---- no more items
    if (!waited) pdl_wait();
    const uint32_t qb = q_issued % Q_BUFFERS;
    if (q_issued >= Q_BUFFERS)
      wait_or_abandon(smem_addr(&q_empty[qb]), ((q_issued / Q_BUFFERS) - 1) & 1, status, &abandoned);
    if (lane == 0) {
      item_meta[qb] = ItemMeta{-1, 0, 0, 0, 0, 0, 0, 0};
      mb_arrive(smem_addr(&meta_bar[qb]));
    }
    return;
  }

  // -------------------------------------------------------------- consumers
  const int cw = warp - 1;
  const int ctid = threadIdx.x - 32;                 // 0..127 among the consumers
  const bool upper_rows_live = group > 8;
  // swizzled addresses of this lane's ldmatrix rows: byte (row, chunk) of a column block sits at
  // row * 128 + ((chunk ^ (row & 7)) << 4)
  const int k_row = (lane & 7) + (lane >> 4) * 8, k_half = (lane >> 3) & 1;
  const int v_row = (lane & 7) + ((lane >> 3) & 1) * 8, v_half = lane >> 4;
  const uint32_t k_lane = k_row * 128, k_xor = (uint32_t)((k_half ^ (k_row & 7)) << 4);
  const uint32_t v_lane = v_row * 128, v_xor = (uint32_t)((v_half ^ (v_row & 7)) << 4);
  // Unfused, the newest cache rows and the query rows come from the kernel before this one. Fused,
  // that kernel is the projection: the cache rows a tile brings were written in earlier steps (the
  // token's own row is replaced in shared memory), so tiles are requested at once and the warp waits
  // only before it reads the partial sums.
  bool waited = !FUSED;
  if (!FUSED) pdl_wait();
  uint32_t seen = 0, n_issued = 0, q_seen = 0;       // tiles consumed and requested by this warp, items seen
  uint32_t fresh_seen[Q_BUFFERS] = {0, 0};           // items with a fresh key and value seen so far, per buffer
  int ahead = 0;                                     // tiles of the next item already requested
  bool pending = false;                              // an item whose partials are written but not counted in
  int p_item = 0, p_g = 0, p_t = 0, p_first = 0, p_last = 0;

  // This warp's tiles of an item: first key of its first tile, and their number.
  auto my_tiles = [&](const ItemMeta& m, int& first_tile, int& tiles) {
    const int seg_begin = m.seg * segment_keys, seg_end = min(seg_begin + segment_keys, m.pos + 1);
    const int my_begin = seg_begin + cw * quarter;
    const int my_end = min(my_begin + quarter, seg_end);
    first_tile = max(my_begin, (m.kstart / TILE) * TILE);             // tiles stay aligned to the key index
    tiles = my_end > first_tile ? (my_end - first_tile + TILE - 1) / TILE : 0;
  };
  // Request the 16 keys from key0 of the item described in buffer `qslot` into the next ring slot.
  auto request_tile = [&](const ItemMeta& m, int qslot, int key0) {
    const uint32_t slot = n_issued % RING;
    const uint32_t dst = smem_addr(ring_base + (cw * RING + slot) * slot_bytes);
    const uint32_t bar = smem_addr(&full_bar[cw][slot]);
    if (whole_pages) {
      // the 16 keys lie in one page: one box for K and one for V (one per 64 columns if the
      // head size is no multiple of 64)
      int row = tile_rows[qslot][(key0 - m.seg * segment_keys) / TILE];
      if (row < 0) {
        raise_fault(status, VOSTI_FAULT_PAGE_RANGE);
        row = 0;
      }
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
    } else {
      // any page size: one box of one row per key; lanes 0-15 fetch K rows, 16-31 V rows
      const int key = key0 + (lane & 15);
      int row = -1;
      if (key >= m.kstart && key <= m.pos) {
        const int index = page_shift >= 0 ? key >> page_shift : key / page_size;
        const int page = index < max_pages ? block_table[(int64_t)m.request * max_pages + index] : -1;
        if (page < 0 || page >= num_pages) raise_fault(status, VOSTI_FAULT_PAGE_RANGE);
        else row = (page * nkv + m.g) * page_size + (key - index * page_size);
      }
      const unsigned live = __ballot_sync(0xffffffffu, row >= 0);
      if (lane == 0) mb_expect_tx(bar, (uint32_t)__popc(live) * (uint32_t)(nb * 128));
      __syncwarp();
      if (row >= 0)
        for (int cb = 0; cb < nb; ++cb)
          tma_load_2d(dst + (lane < 16 ? 0 : nb * BLOCK_BYTES) + cb * BLOCK_BYTES + (lane & 15) * 128,
                      lane < 16 ? &map_k : &map_v, cb * BOX_COLS, row, bar);
    }
    __syncwarp();
    ++n_issued;
  };
  // Count the CTA in for the pending item (thread 0; the others learn of it after the next
  // barrier); the last one to arrive merges its segments. No CTA waits for another: each
  // counts itself in after its records are visible device-wide.
  auto count_in = [&]() {
    if (ctid == 0) {
      __threadfence();
      int* counter = arrivals + (int64_t)p_item * nkv + p_g;
      const int before = atomicAdd(counter, 1);
      last_to_arrive = before == p_last - p_first;
      if (last_to_arrive) *counter = 0;               // ready for the next launch
    }
  };
  auto merge_if_last = [&]() {
    if (last_to_arrive) {
      __threadfence();
      for (int row = cw; row < group; row += CONSUMERS) {
        const int h = p_g * group + row;
        merge_segments<true>(partial + ((int64_t)p_item * nq + h) * max_segments * record_floats(d), out + ((int64_t)p_t * nq + h) * d,
                       p_first, p_last, d);
      }
    }
  };

  while (true) {
    const uint32_t qb = q_seen % Q_BUFFERS;
    if (ctid == 0) {
      wait_or_abandon(smem_addr(&meta_bar[qb]), (q_seen / Q_BUFFERS) & 1, status, &abandoned);
      consumer_meta = item_meta[qb];
    }
    consumer_sync();                                 // also: everyone is done with the previous item's merge area
    const ItemMeta meta = consumer_meta;
    if (meta.t < 0) break;
    wait_or_abandon(smem_addr(&meta_bar[qb]), (q_seen / Q_BUFFERS) & 1, status, &abandoned);
    const int pos = meta.pos, kstart = meta.kstart, seg = meta.seg, g = meta.g;
    int first_tile, tiles;
    my_tiles(meta, first_tile, tiles);
    // tiles of this item requested so far: those the previous item's tail asked for, then up to a full ring
    int requested = ahead;
    while (requested < min(tiles, RING)) request_tile(meta, qb, first_tile + (requested++) * TILE);
    ahead = 0;
    // what is known of the item after this one (its description may arrive while this one runs)
    const uint32_t nqb = (q_seen + 1) % Q_BUFFERS;
    bool next_known = false;
    ItemMeta next_meta = ItemMeta{-1, 0, 0, 0, 0, 0, 0, 0};
    int next_first = 0, next_tiles = 0;

    if (FUSED) {
      // ---- fused: this warp's share of the item's query rows, from the projection's partial sums
      int rope_pos = pos;
      if (fused.cos_table != nullptr && (pos < 0 || pos >= fused.max_positions)) {
        if (ctid == 0) raise_fault(status, VOSTI_FAULT_POSITION_RANGE);
        rope_pos = 0;
      }
      if (!waited) {
        pdl_wait();
        waited = true;
      }
      const float* token_partial = fused.partial + (int64_t)meta.t * (nq + 2 * nkv) * d;
      for (int row = cw; row < group; row += CONSUMERS)
        head_from_partial<bf16, (DMAX + 63) / 64>(token_partial + (int64_t)(g * group + row) * d, fused.splits, fused.plane, d, lane, fused.q_norm_w,
                          fused.norm_w_is_f32, fused.eps, fused.cos_table, fused.sin_table, rope_pos,
                          reinterpret_cast<bf16*>(q_base + (qb * 16 + row) * q_pitch), (bf16*)nullptr);
      __syncwarp();
      if (lane == 0) mb_arrive(smem_addr(&q_full[qb]));
    }
    // ---- Q fragments of this item into registers (up to head size 128)
    wait_or_abandon(smem_addr(&q_full[qb]), (q_seen / Q_BUFFERS) & 1, status, &abandoned);
    const uint8_t* q_s = q_base + qb * 16 * q_pitch;
    constexpr bool Q_IN_REGISTERS = DMAX <= 128;
    uint32_t qa[Q_IN_REGISTERS ? DMAX / 16 : 1][4];
    if (Q_IN_REGISTERS) {
#pragma unroll
      for (int kk = 0; kk < DMAX / 16; ++kk)
        if (kk * 16 < d)
          ldmatrix_x4(qa[Q_IN_REGISTERS ? kk : 0], smem_addr(q_s + (lane & 15) * q_pitch + (kk * 16 + (lane >> 4) * 8) * 2));
    }

    float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int tile = 0; tile < tiles; ++tile, ++seen) {
      const uint32_t slot = seen % RING;
      wait_or_abandon(smem_addr(&full_bar[cw][slot]), (seen / RING) & 1, status, &abandoned);
      const uint32_t ks = smem_addr(ring_base + (cw * RING + slot) * slot_bytes);
      const uint32_t vs = ks + nb * BLOCK_BYTES;
      const int key0 = first_tile + tile * TILE;
      bool edge = false;
      if (FUSED && meta.fresh && pos >= key0 && pos < key0 + TILE) {
        // the token's own key and value, made by the producer: over the row the box brought
        wait_or_abandon(smem_addr(&fresh_bar[qb]), fresh_seen[qb] & 1, status, &abandoned);
        const int r = pos - key0;
        const uint4* src = reinterpret_cast<const uint4*>(fresh_kv + (int64_t)qb * 2 * d);
        uint8_t* tile = ring_base + (cw * RING + slot) * slot_bytes;
        const int chunks = d >> 3;                     // 16-byte pieces of a row
        for (int i = lane; i < 2 * chunks; i += 32) {
          const int c = i % chunks;                    // piece of the key (i < chunks) or of the value
          uint8_t* block = tile + ((i < chunks ? 0 : nb) + (c >> 3)) * BLOCK_BYTES;
          *reinterpret_cast<uint4*>(block + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = src[i];
        }
        edge = true;                                   // written by threads: fence before the slot is refilled
        __syncwarp();
      }
      if (whole_pages && (key0 < kstart || key0 + TILE - 1 > pos)) {
        // a box brought keys that are masked: their V rows must not reach the MMA (0 * NaN)
        edge = true;
        uint8_t* vrows = ring_base + (cw * RING + slot) * slot_bytes + nb * BLOCK_BYTES;
        for (int i = lane; i < nb * TILE * 8; i += 32) {
          const int r = (i >> 3) % TILE;
          if (key0 + r < kstart || key0 + r > pos) reinterpret_cast<uint4*>(vrows)[i] = make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
      }

      attend_tile<DMAX, Q_IN_REGISTERS>(ks, vs, qa, q_s, q_pitch, d, key0, kstart, pos, scale_log2, upper_rows_live, k_lane, k_xor,
                                        v_lane, v_xor, m_row, l_row, o);
      __syncwarp();                                  // every lane is done with this slot: refill it
      if (edge) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      if (requested < tiles) {
        request_tile(meta, qb, first_tile + (requested++) * TILE);
      } else {
        // this item's tiles are all on their way: start on the next item's if it has been described
        if (!next_known && !abandoned && mb_try_wait(smem_addr(&meta_bar[nqb]), ((q_seen + 1) / Q_BUFFERS) & 1)) {
          next_known = true;
          next_meta = item_meta[nqb];
          if (next_meta.t >= 0) my_tiles(next_meta, next_first, next_tiles);
        }
        if (next_known && ahead < next_tiles) request_tile(next_meta, nqb, next_first + (ahead++) * TILE);
      }
    }
    // the description (and with head sizes above 128 the Q rows) of this item is not needed any more
    __syncwarp();
    if (FUSED && meta.fresh) ++fresh_seen[qb];                // (whether or not this warp had the tile of the token's position)
    if (lane == 0) mb_arrive(smem_addr(&q_empty[qb]));
    ++q_seen;

    // ---- merge the four consumers in warp order
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 1);
      l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
    }
    // the item before this one is counted in now: its stores have had an item's time to land
    if (pending) count_in();
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
    for (int row = 0; row < group; ++row) {
      // the row's maximum over the warps and each warp's weight 2^(m_w - m)
      float weight[CONSUMERS];
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < CONSUMERS; ++w) m = fmaxf(m, merge[((int64_t)w * group + row) * rec]);
#pragma unroll
      for (int w = 0; w < CONSUMERS; ++w) {
        const float mw = merge[((int64_t)w * group + row) * rec];
        weight[w] = mw == -INFINITY ? 0.f : fast_exp2(mw - m);
      }
      float* dst = partial + (((int64_t)meta.item * nq + g * group + row) * max_segments + seg) * record_floats(d);
      for (int c = ctid; c < rec; c += CONSUMERS * 32) {
        float value;
        if (c == 0) {
          value = m;
        } else {
          value = 0.f;
#pragma unroll
          for (int w = 0; w < CONSUMERS; ++w) value += merge[((int64_t)w * group + row) * rec + c] * weight[w];
        }
        dst[c < 2 ? c : c + 2] = value;                  // the accumulator starts at float 4 of a global record
      }
    }
    if (pending) merge_if_last();
    pending = true;
    p_item = meta.item; p_g = g; p_t = meta.t;
    p_first = kstart / segment_keys; p_last = pos / segment_keys;
  }
  if (!waited) pdl_wait();                           // (a CTA without items: the chain of completed kernels stays unbroken)
  if (pending) {
    consumer_sync();                                 // every consumer has written its share of the last item
    count_in();
    consumer_sync();
    merge_if_last();
  }
}

// Bytes of dynamic shared memory: ring, Q buffers, merge area, and room to align the ring.
size_t decode_smem_bytes(int d, int group) {
  const size_t nb = (d + BOX_COLS - 1) / BOX_COLS;
  return 1024 + (size_t)CONSUMERS * RING * 2 * nb * BLOCK_BYTES + (size_t)Q_BUFFERS * 16 * ((size_t)d * 2 + 16) +
         (size_t)CONSUMERS * group * (d + 2) * sizeof(float) + (size_t)Q_BUFFERS * 2 * d * 2;
}

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  return sms;
}

int ctas_per_sm(int d, int group) {
  const size_t per_sm = 228 * 1024;
  const size_t per_cta = decode_smem_bytes(d, group) + 2048;        // static arrays and the reserved kilobyte
  const int by_smem = (int)(per_sm / per_cta);
  return by_smem >= 2 ? 2 : 1;                                       // registers allow two
}

int once_ctas_per_sm(int d, int group, int segments) {
  if (once_smem_bytes(d, group, segments) > ONCE_SMEM_CAP) return 0;
  const size_t per_sm = 228 * 1024;
  const size_t per_cta = once_smem_bytes(d, group, segments) + 2048;   // static arrays and the reserved kilobyte
  const int by_smem = (int)(per_sm / per_cta);
  return by_smem >= 2 ? (d <= 128 ? 2 : 1) : by_smem;                  // registers allow two up to head size 128
}

// Keys per segment for a launch. g_pinned_segment / VOSTI_DECODE_SEGMENT fix the length; else:
//  * with pages of a multiple of 16 tokens the kernel with one CTA per item runs, with 1 to 16
//    segments per (token, kv head) (a cluster), each of the same length, a multiple of 64 up to
//    4096 keys: the count that makes waves of CTAs x (keys + a CTA's fixed cost) smallest;
//  * else (other page sizes, contexts too long for 8 segments of 4096 keys) items are spread over
//    the persistent CTAs in rounds; a round costs the segment's length plus a fixed share for
//    starting and finishing an item.
int g_pinned_segment = 0;           // vosti_set_decode_segment: 0 lets every launch choose
thread_local int g_last_kernel = 0; // which kernel this thread's last launch took: 1 persistent, 2 one CTA per item
int g_once_enabled = -1;            // vosti_set_decode_once; -1: from VOSTI_DECODE_ONCE (default on)

bool once_enabled() {
  if (g_once_enabled < 0) {
    const char* env = getenv("VOSTI_DECODE_ONCE");
    g_once_enabled = (env != nullptr && env[0] == '0') ? 0 : 1;
  }
  return g_once_enabled != 0;
}

int forced_segment_keys() {
  if (g_pinned_segment > 0) return g_pinned_segment;
  if (const char* forced = getenv("VOSTI_DECODE_SEGMENT")) {
    const int keys = atoi(forced);
    if (keys >= SEGMENT_STEP && keys <= MAX_SEGMENT && keys % SEGMENT_STEP == 0) return keys;
  }
  return 0;
}

// The segments per (token, kv head) with which the one-CTA-per-item kernel takes this launch, 0 if
// it does not. page_size 0: not known (the rule is asked for a launch shape only): pages of a
// multiple of 16 are assumed.
int once_segments(int count, int nkv, int d, int group, int max_kv_len, int page_size, int* keys_out) {
  if (!once_enabled() || (page_size > 0 && page_size % TILE != 0) || count <= 0) return 0;
  const int64_t pairs = (int64_t)count * nkv;
  const int forced = forced_segment_keys();
  // Clusters of more than 8 CTAs leave much of a GPC unused (two of them fill it), so that only a
  // few fit the GPU at once: they are for the smallest launches, and only where an SM holds two of
  // their CTAs (with one, a cluster of 14 needs 14 SMs of one GPC: measured no faster than the
  // persistent kernel, where 8 segments were 4 to 7 % faster).
  const int limit = pairs <= 8 && once_ctas_per_sm(d, group, ONCE_MAX_SEGMENTS) >= 2 ? ONCE_MAX_SEGMENTS : 8;
  // While all CTAs fit the GPU at once: as many segments as fit. Beyond that the CTAs run in waves,
  // and a launch costs about its waves times a CTA's time: its keys plus what starting and finishing
  // a CTA costs, about as much as 450 keys (fitted to batches of 20 to 256 requests of 2,048 keys:
  // one segment for most, two where one would leave the second wave nearly empty).
  const int cta_overhead = 450;
  int best = 0;
  int64_t best_cost = -1;
  for (int segments = limit; segments >= 1; --segments) {
    int keys = forced > 0 ? forced : ((max_kv_len + segments - 1) / segments + SEGMENT_STEP - 1) / SEGMENT_STEP * SEGMENT_STEP;
    if (keys < MIN_SEGMENT && forced == 0) keys = MIN_SEGMENT;
    if (keys > MAX_SEGMENT) break;                             // a warp's tiles would not fit its lanes; fewer segments are longer still
    const int needed = (max_kv_len + keys - 1) / keys;
    if (needed > segments) break;                              // (a pinned length that needs more CTAs than a cluster has)
    const int per_sm = once_ctas_per_sm(d, group, needed);
    if (per_sm < 1) continue;
    const int64_t capacity = (int64_t)sm_count() * per_sm;
    if (pairs * needed <= capacity || forced > 0) {            // one wave (or a pinned length: the same plan for every launch)
      *keys_out = keys;
      return needed;
    }
    const int64_t waves = (pairs * needed + capacity - 1) / capacity;
    const int64_t cost = waves * (keys + cta_overhead);
    if (best_cost < 0 || cost <= best_cost) {                  // ties: fewer segments
      best = needed;
      best_cost = cost;
      *keys_out = keys;
    }
  }
  return best;
}

int choose_segment_keys(int count, int nkv, int d, int group, int max_kv_len, int page_size = 0) {
  int keys = 0;
  if (once_segments(count, nkv, d, group, max_kv_len, page_size, &keys) > 0) return keys;
  const int forced = forced_segment_keys();
  if (forced > 0) return forced;
  const int64_t ctas = (int64_t)sm_count() * ctas_per_sm(d, group);
  const int64_t pairs = (int64_t)count * nkv;
  const int item_overhead = 224;       // measured: starting and finishing an item costs about as much as 220 keys
  int best = MIN_SEGMENT;
  int64_t best_cost = -1;
  for (int keys = MIN_SEGMENT; keys <= MAX_SEGMENT; keys += SEGMENT_STEP) {
    const int64_t segments = (max_kv_len + keys - 1) / keys;
    const int64_t rounds = (pairs * segments + ctas - 1) / ctas;
    const int64_t cost = rounds * (keys + item_overhead);
    if (best_cost < 0 || cost <= best_cost) {          // ties: the longer segment, fewer records
      best_cost = cost;
      best = keys;
    }
    if (segments == 1) break;
  }
  return best;
}

}  // namespace

// Pin the segment length for every later launch of this process (a multiple of 64 between 64
// and 4096), or give the choice back to the launches with 0. With a pinned length a token's
// attention is the same bits whatever else the launch holds.
VOSTI_API int vosti_set_decode_segment(int keys) {
  VOSTI_REQUIRE(keys == 0 || (keys >= SEGMENT_STEP && keys <= MAX_SEGMENT && keys % SEGMENT_STEP == 0),
                "set_decode_segment: %d is not 0 or a multiple of %d up to %d", keys, SEGMENT_STEP, MAX_SEGMENT);
  g_pinned_segment = keys;
  return VOSTI_OK;
}

// The kernel with one CTA per item on (1, the default) or off (0) for every later launch of this process.
VOSTI_API int vosti_set_decode_once(int enabled) {
  g_once_enabled = enabled ? 1 : 0;
  return VOSTI_OK;
}

// Which kernel this thread's last decode-attention launch took: 1 the persistent one, 2 the
// one with one CTA per item, 0 none yet (for tests of the rule above).
VOSTI_API int vosti_attention_decode_last_kernel() { return g_last_kernel; }

// Keys per segment, and so (max_kv_len + keys - 1) / keys partial records per token and
// head, of a launch with `count` tokens and keys up to `max_kv_len`.
VOSTI_API int vosti_attention_decode_segment_keys(int count, int nq, int nkv, int d, int max_kv_len) {
  return choose_segment_keys(count, nkv, d, nq / nkv, max_kv_len);
}

// float32 scratch elements a launch of this shape may need: count * nq * segments * (d + 4) for the
// persistent kernel's records (the kernel with one CTA per item needs none; with pages of no multiple of 16
// tokens the persistent kernel runs where the segment rule above names the other kernel's
// length, so the larger of the two is returned).
VOSTI_API int64_t vosti_attention_decode_scratch(int count, int nq, int nkv, int d, int max_kv_len) {
  const int keys = vosti_attention_decode_segment_keys(count, nq, nkv, d, max_kv_len);
  const int other = choose_segment_keys(count, nkv, d, nq / nkv, max_kv_len, 1);      // page size 1: never the other kernel's rule
  const int shorter = keys < other ? keys : other;
  return (int64_t)count * nq * ((max_kv_len + shorter - 1) / shorter) * record_floats(d);
}

// caches: bf16 [pages, kv heads, page_size, d] (a head's tokens of a page are contiguous),
// 16-byte aligned, finite in every slot of a page a live request holds.
// arrivals: int32[count * nkv], all zero before the first launch; every launch leaves it zero.
// q, out: bf16 [tokens_total, nq, d]; the kernel serves `count` tokens: those listed in
// token_list (int32[count]) or tokens 0..count-1. scratch holds the partial records of the
// launch (vosti_attention_decode_scratch elements) and may be reused by the next launch.
namespace {
int launch_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* scratch,
                  int64_t scratch_elems, int* arrivals, const int* token_list, int count, int tokens_total,
                  const int* positions, const int* request_of, const int* block_table, int max_pages,
                  int page_size, int num_pages, int nq, int nkv, int d, int max_kv_len, float scale,
                  int window, unsigned* status, cudaStream_t stream, const FusedProjection& fused) {
  VOSTI_REQUIRE(count >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention_decode: bad head counts nq=%d nkv=%d", nq, nkv);
  VOSTI_REQUIRE(nq / nkv <= 16, "attention_decode: at most 16 query heads per kv head, got %d", nq / nkv);
  VOSTI_REQUIRE(d > 0 && d % 16 == 0 && d <= 256, "attention_decode: head_dim %d must be a multiple of 16 and <= 256", d);
  VOSTI_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0 && window >= 0, "attention_decode: bad cache geometry");
  VOSTI_REQUIRE(max_kv_len > 0, "attention_decode: max_kv_len %d must be positive", max_kv_len);
  if (count == 0) return VOSTI_OK;
  const int group = nq / nkv;
  const int64_t cache_rows = (int64_t)num_pages * nkv * page_size;
  VOSTI_REQUIRE(cache_rows < (int64_t)1 << 31, "attention_decode: cache of %lld rows is too large", (long long)cache_rows);
  VOSTI_REQUIRE((reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0,
                "attention_decode: the caches must be 16-byte aligned");
  const int whole_pages = page_size % TILE == 0 ? 1 : 0;
  const int whole_rows = whole_pages && d % BOX_COLS == 0 ? 1 : 0;
  const int box_rows = whole_rows ? -TILE : whole_pages ? TILE : 1;
  CUtensorMap map_k, map_v;
  VOSTI_REQUIRE(cached_tensor_map(k_cache, cache_rows, d, box_rows, &map_k) &&
                    cached_tensor_map(v_cache, cache_rows, d, box_rows, &map_v),
                "attention_decode: cuTensorMapEncodeTiled failed");
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; ++page_shift) {}
  {
    // ---- one CTA per item: a cluster of CTAs per (token, kv head)
    int once_keys = 0;
    const int once = once_segments(count, nkv, d, group, max_kv_len, page_size, &once_keys);
    if (once > 0) {
      OnceLaunch launch;
      launch.map_k = map_k;
      launch.map_v = map_v;
      launch.q = (const bf16*)q;
      launch.out = (bf16*)out;
      launch.token_list = token_list;
      launch.positions = positions;
      launch.request_of = request_of;
      launch.block_table = block_table;
      launch.max_pages = max_pages;
      launch.page_size = page_size;
      launch.page_shift = page_shift;
      launch.num_pages = num_pages;
      launch.whole_rows = whole_rows;
      launch.count = count;
      launch.nq = nq;
      launch.nkv = nkv;
      launch.d = d;
      launch.segments = once;
      launch.segment_keys = once_keys;
      launch.scale_log2 = scale * LOG2E;
      launch.window = window;
      launch.status = status;
      launch.fused = fused;
      launch.stream = stream;
      const int launched = launch_once(launch);
      if (launched < 0) return -launched;
      if (launched > 0) {
        g_last_kernel = 2;
        return VOSTI_OK;
      }
    }
  }
  g_last_kernel = 1;
  // ---- the persistent kernel (page size 1 in the rule: never the other kernel's length)
  const int segment_keys = choose_segment_keys(count, nkv, d, group, max_kv_len, 1);
  const int segments = (max_kv_len + segment_keys - 1) / segment_keys;
  VOSTI_REQUIRE(arrivals != nullptr, "attention_decode: the arrival counters are missing");
  VOSTI_REQUIRE(scratch != nullptr && scratch_elems >= (int64_t)count * nq * segments * record_floats(d),
                "attention_decode: scratch too small");
  const size_t smem = decode_smem_bytes(d, group);
  const int64_t items = (int64_t)count * nkv * segments;
  VOSTI_REQUIRE(items < ((int64_t)1 << 30), "attention_decode: %lld work items are too many for one launch", (long long)items);
  const int64_t ctas = (int64_t)sm_count() * ctas_per_sm(d, group);
  dim3 grid((unsigned)(items < ctas ? items : ctas));
#define LAUNCH_DECODE_AS(DMAX, EXACT, FUSED)                                                                        \
  do {                                                                                                              \
    static bool configured = false;                                                                                 \
    if (!configured) {                                                                                              \
      cudaFuncSetAttribute(attention_decode_kernel<DMAX, EXACT, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)decode_smem_bytes(DMAX, 16));                                                       \
      configured = true;                                                                                            \
    }                                                                                                               \
    vosti_launch(attention_decode_kernel<DMAX, EXACT, FUSED>, grid, dim3(THREADS), smem, stream, map_k, map_v,      \
        (const bf16*)q, scratch, (bf16*)out, arrivals, token_list, positions, request_of,                          \
        block_table, max_pages, page_size, page_shift, num_pages, whole_pages, whole_rows, count, nq, nkv, d, segment_keys,     \
        segments, scale * LOG2E, window, status, fused);                                                            \
  } while (0)
#define LAUNCH_DECODE(DMAX, EXACT)                                                                                  \
  do {                                                                                                              \
    if (fused.partial != nullptr) LAUNCH_DECODE_AS(DMAX, EXACT, true);                                              \
    else LAUNCH_DECODE_AS(DMAX, EXACT, false);                                                                      \
  } while (0)
  if (d == 64) LAUNCH_DECODE(64, true);
  else if (d == 128) LAUNCH_DECODE(128, true);
  else if (d == 256) LAUNCH_DECODE(256, true);
  else if (d < 64) LAUNCH_DECODE(64, false);
  else if (d < 128) LAUNCH_DECODE(128, false);
  else LAUNCH_DECODE(256, false);
#undef LAUNCH_DECODE
#undef LAUNCH_DECODE_AS
  VOSTI_LAUNCH_CHECK();
}
}  // namespace

VOSTI_API int vosti_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* scratch,
                                     int64_t scratch_elems, int* arrivals, const int* token_list, int count, int tokens_total,
                                     const int* positions, const int* request_of, const int* block_table, int max_pages,
                                     int page_size, int num_pages, int nq, int nkv, int d, int max_kv_len, float scale,
                                     int window, unsigned* status, cudaStream_t stream) {
  FusedProjection none = {};
  return launch_decode(q, k_cache, v_cache, out, scratch, scratch_elems, arrivals, token_list, count, tokens_total, positions,
                       request_of, block_table, max_pages, page_size, num_pages, nq, nkv, d, max_kv_len, scale, window,
                       status, stream, none);
}

// The fused form: `partial` holds the QKV projection's K-split partial sums of the step's tokens
// ([splits][tokens][(nq + 2 nkv) d] float32, every request bringing one token, token i being row i);
// the kernel sums them, applies head norm and rotation, stores the new keys and values in the
// caches at slot_mapping and attends. q_norm_w / k_norm_w null: no head norm; cos / sin null: no
// rotation (float32 tables [max_positions][d / 2]). Head sizes up to 512 in steps of 16 as the
// unfused kernel; d must be even. block_table has at least `count` rows (one per request).
VOSTI_API int vosti_attention_decode_fused(const float* partial, int splits, void* k_cache, void* v_cache, void* out,
                                           float* scratch, int64_t scratch_elems, int* arrivals, int count,
                                           const int* positions, const int* request_of, const int* block_table,
                                           int max_pages, int page_size, int num_pages, int nq, int nkv, int d,
                                           int max_kv_len, float scale, int window, const void* q_norm_w,
                                           const void* k_norm_w, int norm_w_is_f32, float eps, const float* cos_table,
                                           const float* sin_table, int max_positions, const int* slot_mapping,
                                           unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(partial != nullptr && splits >= 1, "attention_decode_fused: the partial sums are missing");
  VOSTI_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "attention_decode_fused: cos and sin go together");
  VOSTI_REQUIRE(d % 2 == 0 && d / 2 <= 32 * HEAD_MAX_PAIRS, "attention_decode_fused: head_dim %d is too large", d);
  FusedProjection fused = {};
  fused.partial = partial;
  fused.splits = splits;
  fused.plane = (long long)count * (nq + 2 * nkv) * d;
  fused.q_norm_w = q_norm_w;
  fused.k_norm_w = k_norm_w;
  fused.norm_w_is_f32 = norm_w_is_f32;
  fused.eps = eps;
  fused.cos_table = cos_table;
  fused.sin_table = sin_table;
  fused.max_positions = max_positions;
  fused.slot_mapping = slot_mapping;
  fused.num_slots = (long long)num_pages * page_size;
  fused.k_cache = (bf16*)k_cache;
  fused.v_cache = (bf16*)v_cache;
  return launch_decode(nullptr, k_cache, v_cache, out, scratch, scratch_elems, arrivals, nullptr, count, count, positions,
                       request_of, block_table, max_pages, page_size, num_pages, nq, nkv, d, max_kv_len, scale, window,
                       status, stream, fused);
}


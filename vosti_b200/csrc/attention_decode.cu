// Paged attention for single query tokens (decode rows and very short portions),
// bfloat16, on the tensor cores with split keys ("flash decoding"):
//
//   grid = (segments, kv heads, tokens). One CTA takes one token, one kv head with the
//   whole group of query heads that share it (they fill the MMA's 16 rows), and one
//   segment of SEGMENT keys counted from key 0 of the request. Its four warps each take a
//   quarter of the segment (four tiles of 16 keys through two buffers: two tiles are
//   requested before any arithmetic, the others as buffers become free), run the online softmax (base 2, float32) with mma.sync m16n8k16 for
//   Q.K^T and P.V, and are merged in warp order. The CTA writes
//   an unnormalised partial (max, sum, accumulator) per query head; the CTA that finishes
//   last for a (token, kv head) merges the segments in segment order and normalises.
//
// The segmentation depends on the key index only, so a row's arithmetic does not depend
// on its batch companions. Formulas as in kernels/triton_kernels/fattn_paged.py:176-252:
// kv head = query head * nkv / nq, scale * log2(e), causal up to the token's own position,
// optional window, P rounded to bfloat16 before P.V (:246), out = acc / l (0 if l = 0).
// K and V rows are staged in shared memory by bulk copies (one per cache row, completing
// on an mbarrier per tile) straight from the pages; masked keys are never read from the cache.
#include "common.cuh"
#include "mma_util.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int TILE = 16;              // keys per MMA step
constexpr int SEGMENT = 256;          // keys per CTA
constexpr int WARP_KEYS = SEGMENT / WARPS;
constexpr int BUFFERS = 2;                     // of which this many are in shared memory at once
constexpr float LOG2E = 1.4426950408889634f;

// Partial record of one (token, query head, segment): [0] max (base-2 scores), [1] sum,
// [2 .. 2+d) accumulator.
__host__ __device__ inline int record_floats(int d) { return d + 2; }

// One warp combines the segments first..last of one (token, query head): lane s holds
// segment s's max and weight; the sums run over segments in segment order, whichever CTA
// runs this. `base` points at the head's records, `dst` at its output row.
__device__ __forceinline__ void merge_segments(const float* __restrict__ base, bf16* __restrict__ dst, int first,
                                               int last, int d) {
  const int lane = threadIdx.x & 31;
  const int rec = d + 2;
  // pass 1: the overall maximum
  float m = -INFINITY;
  for (int s0 = first; s0 <= last; s0 += 32) {
    const int s = s0 + lane;
    m = fmaxf(m, s <= last ? __ldcg(base + (int64_t)s * rec) : -INFINITY);
  }
  m = warp_max(m);
  // pass 2: weights, sum and accumulator
  float l = 0.f;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int s0 = first; s0 <= last; s0 += 32) {
    const int mine = s0 + lane;
    float w_mine = 0.f, l_mine = 0.f;
    if (mine <= last) {
      const float ms = __ldcg(base + (int64_t)mine * rec);
      if (ms != -INFINITY) {
        w_mine = fast_exp2(ms - m);
        l_mine = __ldcg(base + (int64_t)mine * rec + 1) * w_mine;
      }
    }
    const int n = min(32, last - s0 + 1);
    // segments in batches of 4: their loads are issued together, then summed in segment order
    for (int j0 = 0; j0 < n; j0 += 4) {
      float v[4][8];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const float* row = base + (int64_t)(s0 + min(j0 + b, n - 1)) * rec + 2;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = lane + 32 * i;
          v[b][i] = (c < d) ? __ldcg(row + c) : 0.f;       // other CTAs wrote these: read past L1
        }
      }
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const bool live = j0 + b < n;
        const float w = live ? __shfl_sync(0xffffffffu, w_mine, (j0 + b) & 31) : 0.f;
        l += live ? __shfl_sync(0xffffffffu, l_mine, (j0 + b) & 31) : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(v[b][i], w, acc[i]);
      }
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + 32 * i;
    if (c < d) dst[c] = __float2bfloat16_rn(acc[i] * inv);
  }
}

// DMAX bounds the head size; with EXACT the head size is DMAX itself, which turns the index
// arithmetic of the staging loops into shifts.
template <int DMAX, bool EXACT>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                        float* __restrict__ partial, bf16* __restrict__ out, int* __restrict__ arrivals,
                        const int* __restrict__ token_list,
                        const int* __restrict__ positions, const int* __restrict__ request_of,
                        const int* __restrict__ block_table, int max_pages, int page_size, int page_shift,
                        int num_pages, int nq, int nkv, int d_runtime, int max_segments, float scale_log2, int window, unsigned* status) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ __align__(8) uint64_t tile_bar[WARPS][BUFFERS];
  if ((threadIdx.x & 31) == 0) {
    for (int i = 0; i < BUFFERS; ++i) mb_init(smem_addr(&tile_bar[threadIdx.x >> 5][i]), 1);
    mb_fence_init();
  }
  __syncwarp();
  pdl_wait();
  pdl_launch_dependents();
  const int d = EXACT ? DMAX : d_runtime;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = token_list ? token_list[blockIdx.z] : blockIdx.z;
  const int g = blockIdx.y, seg = blockIdx.x;
  const int group = nq / nkv;                       // query heads per kv head, <= 16
  const int pos = positions[t];
  const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int seg_begin = seg * SEGMENT, seg_end = min(seg_begin + SEGMENT, pos + 1);
  if (seg_begin > pos || seg_end <= kstart) return;            // nothing visible in this segment
  const int* table = block_table + (int64_t)request_of[t] * max_pages;

  const int pitch = d * 2 + 16;                     // bytes per staged row: conflict-free ldmatrix
  uint8_t* q_s = smem;                              // [16][pitch]
  uint8_t* stage_base = smem + 16 * pitch + warp * (2 * BUFFERS * TILE * pitch);   // per warp: buffers x (K, V)
  const int chunks = d / 8;                         // 16-byte chunks per row

  const int my_begin = seg_begin + warp * WARP_KEYS;
  const int my_end = min(my_begin + WARP_KEYS, seg_end);
  const int first_tile = max(my_begin, (kstart / TILE) * TILE);       // tiles stay aligned to the key index
  const int tiles = my_end > first_tile ? (my_end - first_tile + TILE - 1) / TILE : 0;

  // A tile's 16 key rows and 16 value rows are fetched by one bulk copy each (lane r: key
  // row r, lane 16 + r: value row r) that signals the tile's mbarrier; rows that are not
  // visible are zero-filled and never read from the cache.
  auto issue = [&](int tile) {
    const int key0 = first_tile + tile * TILE;
    uint8_t* kdst = stage_base + (tile % BUFFERS) * (2 * TILE * pitch);
    uint8_t* vdst = kdst + TILE * pitch;
    const int row = lane & 15;
    const int key = key0 + row;
    int64_t slot = -1;
    if (key >= kstart && key <= pos) {
      const int index = page_shift >= 0 ? key >> page_shift : key / page_size;
      const int page = index < max_pages ? table[index] : -1;
      if (page < 0 || page >= num_pages) raise_fault(status, VOSTI_FAULT_PAGE_RANGE);
      else slot = ((int64_t)page * nkv + g) * page_size + (key - index * page_size);   // row of (page, head, offset)
    }
    const unsigned live = __ballot_sync(0xffffffffu, slot >= 0);
    const uint32_t bar = smem_addr(&tile_bar[warp][tile % BUFFERS]);
    if (lane == 0) mb_expect_tx(bar, (uint32_t)__popc(live) * (uint32_t)(d * 2));
    __syncwarp();
    uint8_t* dst = (lane < 16 ? kdst : vdst) + row * pitch;
    if (slot >= 0) {
      const bf16* src = (lane < 16 ? k_cache : v_cache) + slot * d;
      bulk_copy_g2s(smem_addr(dst), src, (uint32_t)(d * 2), bar);
    } else {
      for (int c = 0; c < chunks; ++c) *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(0, 0, 0, 0);
    }
  };

  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  float o[DMAX / 8][4];
#pragma unroll
  for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int tile = 0; tile < tiles && tile < BUFFERS; ++tile) issue(tile);   // the first tiles are requested at once
  // ---- Q rows of the group (rows >= group are zero)
  for (int i = threadIdx.x; i < 16 * chunks; i += WARPS * 32) {
    const int row = i / chunks, c = i % chunks;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < group) v = *reinterpret_cast<const uint4*>(q + ((int64_t)t * nq + g * group + row) * d + c * 8);
    *reinterpret_cast<uint4*>(q_s + row * pitch + c * 16) = v;
  }
  __syncthreads();                                                  // (the K/V requests above are in flight meanwhile)
  // up to head size 128 the Q fragments stay in registers for both tiles
  constexpr bool Q_IN_REGISTERS = DMAX <= 128;
  uint32_t qa[Q_IN_REGISTERS ? DMAX / 16 : 1][4];
  if (Q_IN_REGISTERS) {
#pragma unroll
    for (int kk = 0; kk < DMAX / 16; ++kk)
      if (kk * 16 < d) ldmatrix_x4(qa[Q_IN_REGISTERS ? kk : 0], smem_addr(q_s + (lane & 15) * pitch + (kk * 16 + (lane >> 4) * 8) * 2));
  }
  // rows 8..15 of the MMA tile hold query heads only if the group has more than 8
  const bool upper_rows_live = group > 8;

  for (int tile = 0; tile < tiles; ++tile) {
    mb_wait(smem_addr(&tile_bar[warp][tile % BUFFERS]), (tile / BUFFERS) & 1, status);
    __syncwarp();
    const uint8_t* ks = stage_base + (tile % BUFFERS) * (2 * TILE * pitch);
    const uint8_t* vs = ks + TILE * pitch;
    const int key0 = first_tile + tile * TILE;

    // ---- S = Q K^T for 16 keys: two 8-key column tiles
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < DMAX / 16; ++kk) {
      if (kk * 16 < d) {
        uint32_t a[4], b[4];
        // A: rows lane%16 of Q, columns kk*16 + (lane/16)*8
        if (Q_IN_REGISTERS) {
          a[0] = qa[Q_IN_REGISTERS ? kk : 0][0]; a[1] = qa[Q_IN_REGISTERS ? kk : 0][1];
          a[2] = qa[Q_IN_REGISTERS ? kk : 0][2]; a[3] = qa[Q_IN_REGISTERS ? kk : 0][3];
        } else {
          ldmatrix_x4(a, smem_addr(q_s + (lane & 15) * pitch + (kk * 16 + (lane >> 4) * 8) * 2));
        }
        // B: matrices (keys 0-7, k lo), (keys 0-7, k hi), (keys 8-15, k lo), (keys 8-15, k hi)
        ldmatrix_x4(b, smem_addr(ks + ((lane & 7) + (lane >> 4) * 8) * pitch + (kk * 16 + ((lane >> 3) & 1) * 8) * 2));
        mma_bf16(s[0], a, b[0], b[1]);
        mma_bf16(s[1], a, b[2], b[3]);
      }
    }
    // ---- online softmax (rows lane/4 and lane/4 + 8)
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        const bool visible = key >= kstart && key <= pos;
        s[nt][e] = visible ? s[nt][e] * scale_log2 : -INFINITY;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], s[nt][e]);
      }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (r == 1 && !upper_rows_live) {              // padding rows: no exponentials (warp-uniform)
        alpha[r] = 1.f;
        s[0][2] = s[0][3] = s[1][2] = s[1][3] = 0.f;
        continue;
      }
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
      const float m_new = fmaxf(m_row[r], tile_max[r]);
      const float safe = m_new == -INFINITY ? 0.f : m_new;
      alpha[r] = fast_exp2(m_row[r] - safe);
      m_row[r] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        s[nt][2 * r] = fast_exp2(s[nt][2 * r] - safe);
        s[nt][2 * r + 1] = fast_exp2(s[nt][2 * r + 1] - safe);
        sum += s[nt][2 * r] + s[nt][2 * r + 1];
      }
      l_row[r] = l_row[r] * alpha[r] + sum;          // per-thread share; reduced over the quad at the end
    }
    uint32_t p[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                     pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
    // ---- O = O * alpha + P V
#pragma unroll
    for (int nt = 0; nt < DMAX / 16; ++nt) {
      if (nt * 16 < d) {
        o[2 * nt][0] *= alpha[0]; o[2 * nt][1] *= alpha[0]; o[2 * nt][2] *= alpha[1]; o[2 * nt][3] *= alpha[1];
        o[2 * nt + 1][0] *= alpha[0]; o[2 * nt + 1][1] *= alpha[0]; o[2 * nt + 1][2] *= alpha[1]; o[2 * nt + 1][3] *= alpha[1];
        uint32_t b[4];
        // transposed: matrices (keys 0-7, cols lo), (keys 8-15, cols lo), (keys 0-7, cols hi), (keys 8-15, cols hi)
        ldmatrix_x4_trans(b, smem_addr(vs + ((lane & 7) + ((lane >> 3) & 1) * 8) * pitch + (nt * 16 + (lane >> 4) * 8) * 2));
        mma_bf16(o[2 * nt], p, b[0], b[1]);
        mma_bf16(o[2 * nt + 1], p, b[2], b[3]);
      }
    }
    if (tile + BUFFERS < tiles) {                  // this buffer is free again: fetch the tile after next
      __syncwarp();
      issue(tile + BUFFERS);
    }
  }
  // ---- merge the four warps in warp order (through the staging memory)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 1);
    l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
  }
  __syncthreads();
  float* merge = reinterpret_cast<float*>(smem + 16 * pitch);     // [WARPS][16][d + 2]
  const int rec = d + 2;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = (lane >> 2) + 8 * r;
    if (row < group) {
      float* dst = merge + ((int64_t)warp * 16 + row) * rec;
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
  __syncthreads();
  // per (row, warp): the row's maximum over the warps and this warp's weight 2^(m_w - m)
  __shared__ float row_max[16], row_weight[WARPS][16];
  if (threadIdx.x < 16 * WARPS) {
    const int row = threadIdx.x & 15, w = threadIdx.x >> 4;
    if (row < group) {
      float m = -INFINITY;
      for (int v = 0; v < WARPS; ++v) m = fmaxf(m, merge[((int64_t)v * 16 + row) * rec]);
      const float mw = merge[((int64_t)w * 16 + row) * rec];
      row_weight[w][row] = mw == -INFINITY ? 0.f : fast_exp2(mw - m);
      if (w == 0) row_max[row] = m;
    }
  }
  __syncthreads();
  for (int row = 0; row < group; ++row) {
    float* dst = partial + (((int64_t)blockIdx.z * nq + g * group + row) * max_segments + seg) * rec;
    for (int c = threadIdx.x; c < rec; c += WARPS * 32) {
      float value;
      if (c == 0) {
        value = row_max[row];
      } else {
        value = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) value += merge[((int64_t)w * 16 + row) * rec + c] * row_weight[w][row];
      }
      dst[c] = value;
    }
  }
  // ---- the CTA that finishes last for this (token, kv head) merges the segments. No CTA
  // waits for another: each counts itself in after its records are visible device-wide.
  __shared__ int last_to_arrive;
  __threadfence();
  __syncthreads();
  const int first_segment = kstart / SEGMENT, last_segment = pos / SEGMENT;
  if (threadIdx.x == 0) {
    int* counter = arrivals + (int64_t)blockIdx.z * nkv + g;
    const int before = atomicAdd(counter, 1);
    last_to_arrive = before == last_segment - first_segment;
    if (last_to_arrive) *counter = 0;               // ready for the next launch
  }
  __syncthreads();
  if (!last_to_arrive) return;
  __threadfence();
  for (int row = warp; row < group; row += WARPS) {
    const int h = g * group + row;
    merge_segments(partial + ((int64_t)blockIdx.z * nq + h) * max_segments * rec, out + ((int64_t)t * nq + h) * d,
                   first_segment, last_segment, d);
  }
}

size_t decode_smem_bytes(int d) {
  const size_t pitch = (size_t)d * 2 + 16;
  const size_t stage = 16 * pitch + (size_t)WARPS * 2 * BUFFERS * TILE * pitch;
  const size_t merge = 16 * pitch + (size_t)WARPS * 16 * (d + 2) * sizeof(float);
  return stage > merge ? stage : merge;
}

}  // namespace

// Number of key segments (and so partial records per token and head) a launch with keys
// up to `max_kv_len` uses.
VOSTI_API int vosti_attention_decode_segments(int max_kv_len) { return (max_kv_len + SEGMENT - 1) / SEGMENT; }

// float32 scratch elements needed: count * nq * segments * (d + 2).
VOSTI_API int64_t vosti_attention_decode_scratch(int count, int nq, int d, int max_kv_len) {
  return (int64_t)count * nq * vosti_attention_decode_segments(max_kv_len) * record_floats(d);
}

// caches: bf16 [pages, kv heads, page_size, d] (a head's tokens of a page are contiguous).
// arrivals: int32[count * nkv], all zero before the first launch; every launch leaves it zero.
// q, out: bf16 [tokens_total, nq, d]; the kernel serves `count` tokens: those listed in
// token_list (int32[count]) or tokens 0..count-1. scratch holds the partial records of the
// launch (vosti_attention_decode_scratch elements) and may be reused by the next launch.
VOSTI_API int vosti_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* scratch,
                                     int64_t scratch_elems, int* arrivals, const int* token_list, int count, int tokens_total,
                                     const int* positions, const int* request_of, const int* block_table, int max_pages,
                                     int page_size, int num_pages, int nq, int nkv, int d, int max_kv_len, float scale,
                                     int window, unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(count >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention_decode: bad head counts nq=%d nkv=%d", nq, nkv);
  VOSTI_REQUIRE(nq / nkv <= 16, "attention_decode: at most 16 query heads per kv head, got %d", nq / nkv);
  VOSTI_REQUIRE(d > 0 && d % 16 == 0 && d <= 256, "attention_decode: head_dim %d must be a multiple of 16 and <= 256", d);
  VOSTI_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0 && window >= 0, "attention_decode: bad cache geometry");
  if (count == 0) return VOSTI_OK;
  const int segments = vosti_attention_decode_segments(max_kv_len);
  VOSTI_REQUIRE(segments >= 1 && segments <= 65535, "attention_decode: context %d too long", max_kv_len);
  VOSTI_REQUIRE(arrivals != nullptr, "attention_decode: the arrival counters are missing");
  VOSTI_REQUIRE(scratch != nullptr && scratch_elems >= vosti_attention_decode_scratch(count, nq, d, max_kv_len),
                "attention_decode: scratch too small");
  const size_t smem = decode_smem_bytes(d);
  dim3 grid(segments, nkv, count);
  VOSTI_REQUIRE(count <= 65535, "attention_decode: too many tokens (%d) for one launch", count);
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; ++page_shift) {}
#define LAUNCH_DECODE(DMAX, EXACT)                                                                                  \
  do {                                                                                                              \
    static bool configured = false;                                                                                 \
    if (!configured) {                                                                                              \
      cudaFuncSetAttribute(attention_decode_kernel<DMAX, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                           (int)decode_smem_bytes(DMAX));                                                           \
      configured = true;                                                                                            \
    }                                                                                                               \
    vosti_launch(attention_decode_kernel<DMAX, EXACT>, grid, dim3(WARPS * 32), smem, stream,                        \
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, scratch, (bf16*)out, arrivals, token_list,      \
        positions, request_of,                                                                                      \
        block_table, max_pages, page_size, page_shift, num_pages, nq, nkv, d, segments, scale * LOG2E, window,      \
        status);                                                                                                    \
  } while (0)
  if (d == 64) LAUNCH_DECODE(64, true);
  else if (d == 128) LAUNCH_DECODE(128, true);
  else if (d == 256) LAUNCH_DECODE(256, true);
  else if (d < 64) LAUNCH_DECODE(64, false);
  else if (d < 128) LAUNCH_DECODE(128, false);
  else LAUNCH_DECODE(256, false);
#undef LAUNCH_DECODE
  VOSTI_LAUNCH_CHECK();
}

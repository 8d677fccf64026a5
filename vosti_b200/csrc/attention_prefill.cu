// Paged causal attention for prompts and portions of prompts, bfloat16, on the tensor
// cores (mma.sync m16n8k16), in the manner of flash attention:
//
//   grid = (query tiles, kv heads, requests). A CTA takes 128 rows of one request and one
//   kv head, where a row is a (query token, query head of the group) pair, so the query
//   heads that share a kv head share its K and V tiles in shared memory. Each of the eight
//   warps owns 16 rows; K/V tiles of 64 keys, aligned to the absolute key index, are staged
//   with cp.async (double-buffered) straight from the pages. Online softmax in base 2 and
//   float32; P is rounded to bfloat16 before P.V; out = acc / l.
//
// A portion's queries sit at the end of the request's keys (bottom-right causal alignment,
// kernels/triton_kernels/fattn_paged.py:177-179, 220-221): query i of q_len sees keys
// 0 .. k_len - q_len + i, or with a window only the last `window` of them. The reference's
// kernel keeps one query head per program (:481); packing the group is this design's.
#include "common.cuh"
#include "mma_util.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int KT = 64;                // keys per shared-memory tile
constexpr int KH = 32;                // keys per softmax step (two per tile): keeps the score registers few
constexpr float LOG2E = 1.4426950408889634f;

// DMAX bounds the head size; with EXACT the head size is DMAX itself (index arithmetic
// becomes shifts). page_shift >= 0: the page size is 1 << page_shift.
// MT: 16-row MMA tiles per warp.
template <int DMAX, bool EXACT, int MT>
__global__ void __launch_bounds__(WARPS * 32, (DMAX <= 128 && MT == 1) ? 2 : 1)
attention_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                         bf16* __restrict__ out, const int* __restrict__ row_list, const int* __restrict__ cu_q,
                         const int* __restrict__ kv_len, const int* __restrict__ block_table, int max_pages,
                         int page_size, int page_shift, int num_pages, int nq, int nkv, int d_runtime,
                         float scale_log2, int window, unsigned* status) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_wait();
  pdl_launch_dependents();
  constexpr int WARP_ROWS = 16 * MT, ROWS = WARPS * WARP_ROWS;
  const int d = EXACT ? DMAX : d_runtime;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = row_list ? row_list[blockIdx.z] : blockIdx.z;
  const int g = blockIdx.y;
  const int group = nq / nkv;
  const int q_start = cu_q[b], q_len = cu_q[b + 1] - q_start, k_len = kv_len[b];
  const int shift = k_len - q_len;
  const int row0 = (gridDim.x - 1 - blockIdx.x) * ROWS;    // the tiles with most keys start first
  if (row0 >= q_len * group) return;
  const int* table = block_table + (int64_t)b * max_pages;

  const int pitch = d * 2 + 16;
  const int chunks = d / 8;
  uint8_t* q_s = smem;                                   // [ROWS][pitch]
  uint8_t* kv_s = smem + ROWS * pitch;                   // 2 buffers x (K [KT][pitch], V [KT][pitch])

  // ---- Q rows: row r is token (row0 + r) / group, head (row0 + r) % group of the group
  for (int i = threadIdx.x; i < ROWS * chunks; i += WARPS * 32) {
    const int r = i / chunks, c = i % chunks;
    const int packed = row0 + r, token = packed / group;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (token < q_len)
      v = *reinterpret_cast<const uint4*>(q + ((int64_t)(q_start + token) * nq + g * group + packed % group) * d + c * 8);
    *reinterpret_cast<uint4*>(q_s + r * pitch + c * 16) = v;
  }

  // the four rows of this thread: (lane/4) + 8*r of each of the warp's two 16-row tiles
  int pos_row[MT][2], kstart_row[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int token = (row0 + warp * WARP_ROWS + mt * 16 + (lane >> 2) + 8 * r) / group;
      pos_row[mt][r] = token < q_len ? shift + token : -1;     // -1: no key is visible, nothing is written
      kstart_row[mt][r] = (window > 0 && pos_row[mt][r] - window + 1 > 0) ? pos_row[mt][r] - window + 1 : 0;
    }
  // what the whole warp sees (its 32 rows): used to skip tiles and masks
  const int warp_token_lo = (row0 + warp * WARP_ROWS) / group;
  const int warp_token_hi = (row0 + warp * WARP_ROWS + WARP_ROWS - 1) / group;
  const int warp_pos_max = warp_token_lo < q_len ? shift + min(warp_token_hi, q_len - 1) : -1;
  const int warp_pos_min = warp_token_hi < q_len ? shift + warp_token_lo : -1;       // -1: some row is padding
  const int warp_kstart_max = (window > 0 && warp_pos_max - window + 1 > 0) ? warp_pos_max - window + 1 : 0;
  const int token_lo = row0 / group, token_hi = min(q_len - 1, (row0 + ROWS - 1) / group);
  const int key_end = shift + token_hi + 1;              // exclusive
  const int first_key = (window > 0 && shift + token_lo - window + 1 > 0) ? shift + token_lo - window + 1 : 0;
  const int tile_begin = (first_key / KT) * KT;
  const int tiles = (key_end - tile_begin + KT - 1) / KT;

  auto issue = [&](int tile, int buffer) {
    const int key0 = tile_begin + tile * KT;
    uint8_t* kdst = kv_s + buffer * (2 * KT * pitch);
    uint8_t* vdst = kdst + KT * pitch;
    for (int i = threadIdx.x; i < KT * chunks; i += WARPS * 32) {
      const int r = i / chunks, c = i % chunks;
      const int key = key0 + r;
      bool valid = key >= first_key && key < key_end;
      int64_t slot = 0;
      if (valid) {
        const int index = page_shift >= 0 ? key >> page_shift : key / page_size;
        const int page = index < max_pages ? table[index] : -1;
        if (page < 0 || page >= num_pages) {
          raise_fault(status, VOSTI_FAULT_PAGE_RANGE);
          valid = false;
        } else {
          slot = ((int64_t)page * nkv + g) * page_size + (key - index * page_size);   // row of (page, head, offset)
        }
      }
      if (valid) {
        const int64_t offset = slot * d + c * 8;
        cp_async16(smem_addr(kdst + r * pitch + c * 16), k_cache + offset);
        cp_async16(smem_addr(vdst + r * pitch + c * 16), v_cache + offset);
      } else {
        *reinterpret_cast<uint4*>(kdst + r * pitch + c * 16) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(vdst + r * pitch + c * 16) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
  };

  float m_row[MT][2], l_row[MT][2];
  float o[MT][DMAX / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_row[mt][0] = m_row[mt][1] = -INFINITY;
    l_row[mt][0] = l_row[mt][1] = 0.f;
  }
  const uint8_t* q_w = q_s + warp * WARP_ROWS * pitch;

  issue(0, 0);
  for (int tile = 0; tile < tiles; ++tile) {
    const int buffer = tile & 1;
    if (tile + 1 < tiles) {
      issue(tile + 1, buffer ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint8_t* ks = kv_s + buffer * (2 * KT * pitch);
    const uint8_t* vs = ks + KT * pitch;
    const int key0 = tile_begin + tile * KT;
    // a warp whose rows see nothing of the tile skips its arithmetic
    if (key0 > warp_pos_max) {
      __syncthreads();
      continue;
    }
    const bool need_mask = key0 + KT - 1 > warp_pos_min || key0 < warp_kstart_max;

#pragma unroll 1
    for (int half = 0; half < KT / KH; ++half) {
    const int hkey0 = key0 + half * KH;
    if (hkey0 > warp_pos_max) break;
    const uint8_t* ksh = ks + half * KH * pitch;
    const uint8_t* vsh = vs + half * KH * pitch;
    // ---- S = Q K^T: 16*MT rows x KH keys per warp; a K fragment serves every row tile
    float s[MT][KH / 8][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < KH / 8; ++i) s[mt][i][0] = s[mt][i][1] = s[mt][i][2] = s[mt][i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DMAX / 16; ++kk) {
      if (kk * 16 < d) {
        uint32_t a[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          ldmatrix_x4(a[mt], smem_addr(q_w + (mt * 16 + (lane & 15)) * pitch + (kk * 16 + (lane >> 4) * 8) * 2));
#pragma unroll
        for (int j = 0; j < KH / 16; ++j) {
          uint32_t bm[4];
          ldmatrix_x4(bm, smem_addr(ksh + (j * 16 + (lane & 7) + (lane >> 4) * 8) * pitch + (kk * 16 + ((lane >> 3) & 1) * 8) * 2));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_bf16(s[mt][2 * j], a[mt], bm[0], bm[1]);
            mma_bf16(s[mt][2 * j + 1], a[mt], bm[2], bm[3]);
          }
        }
      }
    }
    // ---- mask, online softmax
    float alpha[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < KH / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = hkey0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const int r = e >> 1;
          const bool visible = !need_mask || (key <= pos_row[mt][r] && key >= kstart_row[mt][r]);
          s[mt][nt][e] = visible ? s[mt][nt][e] * scale_log2 : -INFINITY;
          tile_max[r] = fmaxf(tile_max[r], s[mt][nt][e]);
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        const float m_new = fmaxf(m_row[mt][r], tile_max[r]);
        const float safe = m_new == -INFINITY ? 0.f : m_new;
        alpha[mt][r] = exp2f(m_row[mt][r] - safe);
        m_row[mt][r] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < KH / 8; ++nt) {
          s[mt][nt][2 * r] = exp2f(s[mt][nt][2 * r] - safe);
          s[mt][nt][2 * r + 1] = exp2f(s[mt][nt][2 * r + 1] - safe);
          sum += s[mt][nt][2 * r] + s[mt][nt][2 * r + 1];
        }
        l_row[mt][r] = l_row[mt][r] * alpha[mt][r] + sum;
      }
#pragma unroll
      for (int nt = 0; nt < DMAX / 8; ++nt) {
        o[mt][nt][0] *= alpha[mt][0]; o[mt][nt][1] *= alpha[mt][0];
        o[mt][nt][2] *= alpha[mt][1]; o[mt][nt][3] *= alpha[mt][1];
      }
    }
    // ---- O += P V, 16 keys at a time; a V fragment serves both row tiles
#pragma unroll
    for (int j = 0; j < KH / 16; ++j) {
      uint32_t p[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        p[mt][0] = pack_bf16(s[mt][2 * j][0], s[mt][2 * j][1]);
        p[mt][1] = pack_bf16(s[mt][2 * j][2], s[mt][2 * j][3]);
        p[mt][2] = pack_bf16(s[mt][2 * j + 1][0], s[mt][2 * j + 1][1]);
        p[mt][3] = pack_bf16(s[mt][2 * j + 1][2], s[mt][2 * j + 1][3]);
      }
#pragma unroll
      for (int nt = 0; nt < DMAX / 16; ++nt) {
        if (nt * 16 < d) {
          uint32_t bm[4];
          ldmatrix_x4_trans(bm, smem_addr(vsh + (j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch + (nt * 16 + (lane >> 4) * 8) * 2));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_bf16(o[mt][2 * nt], p[mt], bm[0], bm[1]);
            mma_bf16(o[mt][2 * nt + 1], p[mt], bm[2], bm[3]);
          }
        }
      }
    }
    }   // halves of the tile
    __syncthreads();          // everyone is done with this buffer before it is refilled
  }

  // ---- normalise and store
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = l_row[mt][r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (pos_row[mt][r] < 0) continue;
      const int packed = row0 + warp * WARP_ROWS + mt * 16 + (lane >> 2) + 8 * r;
      const int token = packed / group, head = g * group + packed % group;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = out + ((int64_t)(q_start + token) * nq + head) * d;
#pragma unroll
      for (int nt = 0; nt < DMAX / 8; ++nt) {
        if (nt * 8 < d) {
          *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8 + (lane & 3) * 2) =
              __floats2bfloat162_rn(o[mt][nt][2 * r] * inv, o[mt][nt][2 * r + 1] * inv);
        }
      }
    }
}

int row_tiles_per_warp(int d) { return 1; }
int rows_per_cta(int d) { return WARPS * 16 * row_tiles_per_warp(d); }
size_t prefill_smem_bytes(int d) { return (size_t)(rows_per_cta(d) + 4 * KT) * ((size_t)d * 2 + 16); }

}  // namespace

// caches: bf16 [pages, kv heads, page_size, d].
// q, out: bf16 [tokens, nq, d]; serves `count` requests: those in row_list (int32[count])
// or requests 0..count-1; cu_q: int32[requests + 1]; kv_len: int32[requests];
// max_q_len: the longest portion among the served requests.
VOSTI_API int vosti_attention_prefill(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      const int* row_list, int count, const int* cu_q, const int* kv_len,
                                      const int* block_table, int max_pages, int page_size, int num_pages, int nq,
                                      int nkv, int d, int max_q_len, float scale, int window, unsigned* status,
                                      cudaStream_t stream) {
  VOSTI_REQUIRE(count >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention_prefill: bad head counts nq=%d nkv=%d", nq, nkv);
  VOSTI_REQUIRE(d > 0 && d % 16 == 0 && d <= 256, "attention_prefill: head_dim %d must be a multiple of 16 and <= 256", d);
  VOSTI_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0 && window >= 0, "attention_prefill: bad cache geometry");
  VOSTI_REQUIRE(count <= 65535 && nkv <= 65535, "attention_prefill: too many requests or heads for one launch");
  if (count == 0 || max_q_len <= 0) return VOSTI_OK;
  const int group = nq / nkv;
  const int rows = rows_per_cta(d);
  const int64_t tiles = ((int64_t)max_q_len * group + rows - 1) / rows;
  dim3 grid((unsigned)tiles, nkv, count);
  const size_t smem = prefill_smem_bytes(d);
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; ++page_shift) {}
#define LAUNCH_PREFILL(DMAX, EXACT, MT)                                                                                  \
  do {                                                                                                               \
    static bool configured = false;                                                                                  \
    if (!configured) {                                                                                               \
      cudaFuncSetAttribute(attention_prefill_kernel<DMAX, EXACT, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                           (int)prefill_smem_bytes(DMAX));                                                           \
      configured = true;                                                                                             \
    }                                                                                                                \
    vosti_launch(attention_prefill_kernel<DMAX, EXACT, MT>, grid, dim3(WARPS * 32), smem, stream,                     \
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, row_list, cu_q, kv_len, block_table,  \
        max_pages, page_size, page_shift, num_pages, nq, nkv, d, scale * LOG2E, window, status);                      \
  } while (0)
  if (d == 64) LAUNCH_PREFILL(64, true, 1);
  else if (d == 128) LAUNCH_PREFILL(128, true, 1);
  else if (d == 256) LAUNCH_PREFILL(256, true, 1);
  else if (d < 64) LAUNCH_PREFILL(64, false, 1);
  else if (d < 128) LAUNCH_PREFILL(128, false, 1);
  else LAUNCH_PREFILL(256, false, 1);
#undef LAUNCH_PREFILL
  VOSTI_LAUNCH_CHECK();
}

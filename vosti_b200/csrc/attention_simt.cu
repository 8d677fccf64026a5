// Paged causal attention on the CUDA cores, one warp per (query token, query head).
// It serves prompts, portions of prompts and single decoded tokens alike, in float32
// arithmetic for both storage types, and is the float32 path's attention.
//
// What a query sees (kernels/triton_kernels/fattn_paged.py:176-179, 220-221): keys
// 0..position of its own request (with a window w > 0 only keys > position - w); query
// head h reads kv head h * nkv / nq. Scores are scaled by scale * log2(e) and the softmax
// runs online in base 2 over key tiles (:228-246); here a tile is 32 keys aligned to the
// absolute key index, so the order of a row's arithmetic depends on its position only,
// not on how the prompt was cut or what else is in the batch. Unlike the reference's
// kernel the probabilities stay in float32 for P.V.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_D = 256;
constexpr float LOG2E = 1.4426950408889634f;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int d);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int d) {
  float s = 0.f;
  const float4* k4 = reinterpret_cast<const float4*>(k);
  for (int i = 0; i < d / 4; ++i) {
    const float4 v = k4[i];
    s = fmaf(q[4 * i + 0], v.x, s);
    s = fmaf(q[4 * i + 1], v.y, s);
    s = fmaf(q[4 * i + 2], v.z, s);
    s = fmaf(q[4 * i + 3], v.w, s);
  }
  return s;
}
template <>
__device__ __forceinline__ float dot_row<bf16>(const float* __restrict__ q, const bf16* __restrict__ k, int d) {
  float s = 0.f;
  const uint4* k8 = reinterpret_cast<const uint4*>(k);
  for (int i = 0; i < d / 8; ++i) {
    const uint4 raw = k8[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(p[j]);
      s = fmaf(q[8 * i + 2 * j], f.x, s);
      s = fmaf(q[8 * i + 2 * j + 1], f.y, s);
    }
  }
  return s;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                      T* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ request_of,
                      const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
                      int tokens, int nq, int nkv, int d, float scale_log2, int window, unsigned* status) {
  extern __shared__ float q_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t wid = (int64_t)blockIdx.x * WARPS + warp;
  if (wid >= (int64_t)tokens * nq) return;
  const int t = (int)(wid / nq), h = (int)(wid % nq);
  const int g = h * nkv / nq;
  float* qs = q_smem + warp * d;
  const T* qrow = q + ((int64_t)t * nq + h) * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_f32(qrow[i]);
  __syncwarp();

  const int b = request_of[t];
  const int pos = positions[t];
  const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* table = block_table + (int64_t)b * max_pages;

  float m = -INFINITY, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

  for (int j0 = (kstart / 32) * 32; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    bool valid = j >= kstart && j <= pos;
    int64_t slot = 0;
    float s = -INFINITY;
    if (valid) {
      const int slot_in_table = j / page_size;
      const int page = slot_in_table < max_pages ? table[slot_in_table] : -1;
      if (page < 0 || page >= num_pages) {
        raise_fault(status, VOSTI_FAULT_PAGE_RANGE);
        valid = false;
      } else {
        slot = ((int64_t)page * nkv + g) * page_size + (j % page_size);   // row of (page, head, offset)
        s = dot_row<T>(qs, k_cache + slot * d, d) * scale_log2;
      }
    }
    const float tile_max = warp_max(s);
    if (tile_max == -INFINITY) continue;  // nothing visible here: state untouched
    const float m_new = fmaxf(m, tile_max);
    const float alpha = exp2f(m - m_new);
    const float p = valid ? exp2f(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= alpha;
    const int last = min(31, pos - j0);
    for (int kk = 0; kk <= last; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const int64_t sk = __shfl_sync(0xffffffffu, slot, kk);
      if (pk == 0.f) continue;
      const T* vrow = v_cache + sk * d;
#pragma unroll
      for (int i = 0; i < MAX_D / 32; ++i) {
        const int idx = lane + 32 * i;
        if (idx < d) acc[i] = fmaf(pk, to_f32(vrow[idx]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* orow = out + ((int64_t)t * nq + h) * d;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int idx = lane + 32 * i;
    if (idx < d) orow[idx] = from_f32<T>(acc[i] * inv);
  }
}
}  // namespace

// q, out: [tokens, nq, d]; caches: [num_pages, nkv, page_size, d];
// block_table: [requests, max_pages]; positions, request_of: int32[tokens].
VOSTI_API int vosti_attention_simt(const void* q, const void* k_cache, const void* v_cache, void* out,
                                   const int* positions, const int* request_of, const int* block_table,
                                   int max_pages, int page_size, int num_pages, int tokens, int nq, int nkv,
                                   int d, float scale, int window, int is_f32, unsigned* status,
                                   cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention: bad head counts nq=%d nkv=%d", nq, nkv);
  VOSTI_REQUIRE(d > 0 && d % 16 == 0 && d <= MAX_D, "attention: head_dim %d must be a multiple of 16 and <= %d", d, MAX_D);
  VOSTI_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "attention: bad cache geometry");
  VOSTI_REQUIRE(window >= 0, "attention: window must be >= 0 (0 = all keys)");
  if (tokens == 0) return VOSTI_OK;
  const int64_t warps = (int64_t)tokens * nq;
  const int64_t blocks = (warps + WARPS - 1) / WARPS;
  VOSTI_REQUIRE(blocks <= 0x7fffffffLL, "attention: too many (token, head) pairs");
  const size_t smem = (size_t)WARPS * d * sizeof(float);
  if (is_f32)
    attention_simt_kernel<float><<<(unsigned)blocks, WARPS * 32, smem, stream>>>((const float*)q, (const float*)k_cache,
        (const float*)v_cache, (float*)out, positions, request_of, block_table, max_pages, page_size, num_pages,
        tokens, nq, nkv, d, scale * LOG2E, window, status);
  else
    attention_simt_kernel<bf16><<<(unsigned)blocks, WARPS * 32, smem, stream>>>((const bf16*)q, (const bf16*)k_cache,
        (const bf16*)v_cache, (bf16*)out, positions, request_of, block_table, max_pages, page_size, num_pages,
        tokens, nq, nkv, d, scale * LOG2E, window, status);
  VOSTI_LAUNCH_CHECK();
}

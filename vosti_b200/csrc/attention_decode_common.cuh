// What the two decode attention kernels share: the sizes of a work item, the arithmetic of one
// tile and of the merge of segments, and the arguments of the fused form. Included by
// attention_decode.cu (the persistent kernel, the rule that chooses between the two, the entry
// points) and attention_decode_once.cu (the kernel with one CTA per item).
#pragma once
#include <cstdlib>

#include "common.cuh"
#include "head_post.cuh"
#include "mma_util.cuh"
#include "tensor_map.cuh"

namespace decode_attention {


constexpr int CONSUMERS = 4;                          // consumer warps; one producer warp beside them
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr int TILE = 16;                              // keys per MMA step and per TMA box
constexpr int RING = 2;                               // K/V tile buffers per consumer warp
constexpr int Q_BUFFERS = 2;
constexpr int SEGMENT_STEP = CONSUMERS * TILE;        // 64: segment lengths are multiples of this
constexpr int MIN_SEGMENT = SEGMENT_STEP * RING;      // 128: both buffers of every warp in use
constexpr int MAX_SEGMENT = 4096;
constexpr int MAX_SEGMENT_PAGES = MAX_SEGMENT / TILE; // page ids the producer stages per item
constexpr int BOX_COLS = 64;                          // 128 bytes: the swizzle width
constexpr int BLOCK_BYTES = TILE * 128;               // one column block of a tile
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void mb_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// A wait that ran out marks the CTA as abandoned: later waits return at once, so that a fault
// costs one timeout and not one per tile, while every warp still walks through the same
// barriers (the results are garbage then and the status word says so).
__device__ __forceinline__ void wait_or_abandon(uint32_t bar, uint32_t parity, unsigned* status, volatile int* abandoned) {
  if (*abandoned) return;
  if (!mb_wait(bar, parity, status)) *abandoned = 1;
}
// A barrier among the consumer warps only (the producer never joins it).
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory"); }

// Partial record of one (token, query head, segment) in global memory: [0] max (base-2
// scores), [1] sum, [2..3] unused, [4 .. 4+d) accumulator, so that the accumulator is read as
// 16-byte words. (In shared memory a record is [max, sum, accumulator]: d + 2 floats.)
__host__ __device__ inline int record_floats(int d) { return d + 4; }

// One warp combines the segments first..last of one (token, query head): lane s holds
// segment s's max and weight; the sums run over segments in segment order, whichever CTA
// runs this. `base` points at the head's records, `dst` at its output row. A lane owns the
// columns 4 * lane .. 4 * lane + 3 (and 128 further on for head sizes above 128); the loads of
// up to BATCH segments are in flight together.
// GLOBAL: the records were written by other CTAs to global memory (read past L1); else they lie in
// this CTA's shared memory.
template <bool GLOBAL>
__device__ __forceinline__ void merge_segments(const float* __restrict__ base, bf16* __restrict__ dst, int first,
                                               int last, int d) {
  auto load2 = [](const float* p) { return GLOBAL ? __ldcg(reinterpret_cast<const float2*>(p)) : *reinterpret_cast<const float2*>(p); };
  auto load4 = [](const float* p) { return GLOBAL ? __ldcg(reinterpret_cast<const float4*>(p)) : *reinterpret_cast<const float4*>(p); };
  const int lane = threadIdx.x & 31;
  const int rec = record_floats(d);
  constexpr int BATCH = 8;
  const bool second = 4 * lane + 128 < d;               // this lane also owns columns beyond 128
  const bool owner = 4 * lane < d;
  float4 v[BATCH][2];
  // segments s0 + j0 .. s0 + j0 + BATCH - 1 (clamped to the n of this round) of the accumulator
  auto load_batch = [&](int s0, int j0, int n) {
#pragma unroll
    for (int b = 0; b < BATCH; ++b) {
      const float* row = base + (int64_t)(s0 + min(j0 + b, n - 1)) * rec + 4;
      v[b][0] = owner ? load4(row + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
      v[b][1] = second ? load4(row + 4 * lane + 128) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  // the first accumulators are requested together with the (max, sum) pairs: one trip to memory
  // instead of two when there are few segments
  load_batch(first, 0, min(32, last - first + 1));
  // pass 1: every segment's (max, sum), the first 32 segments' kept for the second pass
  float2 ml_first = make_float2(-INFINITY, 0.f);
  float m = -INFINITY;
  for (int s0 = first; s0 <= last; s0 += 32) {
    const int s = s0 + lane;
    const float2 ml = s <= last ? load2(base + (int64_t)s * rec) : make_float2(-INFINITY, 0.f);
    if (s0 == first) ml_first = ml;
    m = fmaxf(m, ml.x);
  }
  m = warp_max(m);
  // pass 2: weights, sum and accumulator
  float l = 0.f;
  float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  for (int s0 = first; s0 <= last; s0 += 32) {
    const int mine = s0 + lane;
    float w_mine = 0.f, l_mine = 0.f;
    if (mine <= last) {
      const float2 ml = s0 == first ? ml_first : load2(base + (int64_t)mine * rec);
      if (ml.x != -INFINITY) {
        w_mine = fast_exp2(ml.x - m);
        l_mine = ml.y * w_mine;
      }
    }
    const int n = min(32, last - s0 + 1);
    for (int j0 = 0; j0 < n; j0 += BATCH) {
      if (s0 != first || j0 != 0) load_batch(s0, j0, n);
#pragma unroll
      for (int b = 0; b < BATCH; ++b) {
        const bool live = j0 + b < n;
        const float w = live ? __shfl_sync(0xffffffffu, w_mine, (j0 + b) & 31) : 0.f;
        l += live ? __shfl_sync(0xffffffffu, l_mine, (j0 + b) & 31) : 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          acc[i].x = fmaf(v[b][i].x, w, acc[i].x);
          acc[i].y = fmaf(v[b][i].y, w, acc[i].y);
          acc[i].z = fmaf(v[b][i].z, w, acc[i].z);
          acc[i].w = fmaf(v[b][i].w, w, acc[i].w);
        }
      }
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  if (owner)
    *reinterpret_cast<uint2*>(dst + 4 * lane) = make_uint2(pack_bf16(acc[0].x * inv, acc[0].y * inv), pack_bf16(acc[0].z * inv, acc[0].w * inv));
  if (second)
    *reinterpret_cast<uint2*>(dst + 4 * lane + 128) = make_uint2(pack_bf16(acc[1].x * inv, acc[1].y * inv), pack_bf16(acc[1].z * inv, acc[1].w * inv));
}

// One tile of 16 keys for one warp: S = Q K^T on the tensor cores, the online softmax of the
// warp's 16 rows (base 2, float32; masked keys count as -inf), O = O * alpha + P V with P rounded
// to bfloat16. ks / vs: shared-memory addresses of the tile's K and V blocks (128-byte swizzle).
template <int DMAX, bool Q_IN_REGISTERS>
__device__ __forceinline__ void attend_tile(uint32_t ks, uint32_t vs, const uint32_t (&qa)[Q_IN_REGISTERS ? DMAX / 16 : 1][4],
                                            const uint8_t* q_s, int q_pitch, int d, int key0, int kstart, int pos,
                                            float scale_log2, bool upper_rows_live, uint32_t k_lane, uint32_t k_xor,
                                            uint32_t v_lane, uint32_t v_xor, float (&m_row)[2], float (&l_row)[2],
                                            float (&o)[DMAX / 8][4]) {
  const int lane = threadIdx.x & 31;
  // ---- S = Q K^T for 16 keys: two 8-key column tiles
  float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
  for (int kk = 0; kk < DMAX / 16; ++kk) {
    if (kk * 16 < d) {
      uint32_t a[4], b[4];
      if (Q_IN_REGISTERS) {
        a[0] = qa[Q_IN_REGISTERS ? kk : 0][0]; a[1] = qa[Q_IN_REGISTERS ? kk : 0][1];
        a[2] = qa[Q_IN_REGISTERS ? kk : 0][2]; a[3] = qa[Q_IN_REGISTERS ? kk : 0][3];
      } else {
        ldmatrix_x4(a, smem_addr(q_s + (lane & 15) * q_pitch + (kk * 16 + (lane >> 4) * 8) * 2));
      }
      // B: matrices (keys 0-7, k lo), (keys 0-7, k hi), (keys 8-15, k lo), (keys 8-15, k hi)
      ldmatrix_x4(b, ks + (kk >> 2) * BLOCK_BYTES + k_lane + ((uint32_t)((kk & 3) << 5) ^ k_xor));
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
      ldmatrix_x4_trans(b, vs + (nt >> 2) * BLOCK_BYTES + v_lane + ((uint32_t)((nt & 3) << 5) ^ v_xor));
      mma_bf16(o[2 * nt], p, b[0], b[1]);
      mma_bf16(o[2 * nt + 1], p, b[2], b[3]);
    }
  }
}

// What the fused form needs beside the attention's own arguments (partial == null: not fused).
struct FusedProjection {
  const float* partial;        // [splits][tokens][(nq + 2 nkv) d] float32
  int splits;
  long long plane;             // tokens * (nq + 2 nkv) * d
  const void* q_norm_w;        // [d] or null: no head norm
  const void* k_norm_w;
  int norm_w_is_f32;
  float eps;
  const float* cos_table;      // [max_positions][d / 2] float32 or null: no rotation
  const float* sin_table;
  int max_positions;
  const int* slot_mapping;     // [tokens] cache slot of each token's key and value, -1: none
  long long num_slots;
  bf16* k_cache;
  bf16* v_cache;
};

constexpr int ONCE_MAX_SEGMENTS = 16;     // CTAs per cluster of that kernel (above 8 it opts in to non-portable sizes)

// Everything a launch of the kernel with one CTA per item needs (attention_decode_once.cu).
struct OnceLaunch {
  CUtensorMap map_k, map_v;
  const bf16* q;
  bf16* out;
  const int* token_list;
  const int* positions;
  const int* request_of;
  const int* block_table;
  int max_pages, page_size, page_shift, num_pages, whole_rows, count, nq, nkv, d;
  int segments, segment_keys;          // CTAs per cluster and keys per segment
  float scale_log2;
  int window;
  unsigned* status;
  FusedProjection fused;               // partial == null: not fused
  cudaStream_t stream;
};

// Bytes of dynamic shared memory of that kernel with `segments` CTAs per cluster, and the most a
// CTA may ask for.
size_t once_smem_bytes(int d, int group, int segments);
constexpr size_t ONCE_SMEM_CAP = 227 * 1024 - 2048;   // an SM's share of a CTA, less the static arrays

// Launches it if a cluster of that size can be scheduled: 1 launched, 0 not (the caller runs the
// persistent kernel), negative: a CUDA error (the text is set).
int launch_once(const OnceLaunch& launch);

}  // namespace decode_attention

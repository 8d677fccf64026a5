// After the fused QKV projection, in one pass over each token's heads:
//   q heads: per-head RMSNorm (optional) -> rotation (optional) -> q_out
//   k heads: per-head RMSNorm (optional) -> rotation (optional) -> key cache slot
//   v heads: copied to the value cache slot
// Formulas: kernels/triton_kernels/qk_norm.py:40-95 (norm over head_dim with one
// weight shared by all heads, before the rotation), rope.py:78-101 (half-split pairs),
// store_kv_cache.py:75-120 (row t goes to slot_mapping[t]; slot -1 writes nothing).
// The reference rounds to bf16 between the norm and the rotation; this kernel keeps
// float32 there and rounds once at the store.
#include "common.cuh"
#include "head_post.cuh"
#include "mma_util.cuh"

namespace {
constexpr int MAX_PAIRS_PER_LANE = HEAD_MAX_PAIRS;  // head_dim <= 512

template <typename T>
__global__ void __launch_bounds__(128)
qkv_post_kernel(const T* __restrict__ qkv, const float* __restrict__ partial, int splits, int64_t plane,
                T* __restrict__ q_out, T* __restrict__ k_cache,
                T* __restrict__ v_cache, const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w,
                int norm_w_is_f32, float eps, const float* __restrict__ cos_table,
                const float* __restrict__ sin_table, int max_positions, const int* __restrict__ positions,
                const int* __restrict__ slot_mapping, int64_t num_slots, int page_size, int nq, int nkv, int d,
                unsigned* status) {
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int half = d >> 1;
  const int heads = nq + 2 * nkv;
  const int64_t in_base = (int64_t)t * heads * d;

  // Positions, slots, rotation tables and norm weights were written before the step began:
  // they are read while the projection before this kernel may still be running.
  int pos = positions ? positions[t] : 0;
  if (cos_table && (pos < 0 || pos >= max_positions)) {
    if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_POSITION_RANGE);
    pos = 0;
  }
  int64_t slot = -1;
  if (nkv > 0 && slot_mapping) {
    slot = slot_mapping[t];
    if (slot >= num_slots || slot < -1) {
      if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
      slot = -1;
    }
  }
  float cs[MAX_PAIRS_PER_LANE], sn[MAX_PAIRS_PER_LANE];
#pragma unroll
  for (int j = 0; j < MAX_PAIRS_PER_LANE; ++j) {
    const int i = lane + 32 * j;
    cs[j] = (cos_table && i < half) ? cos_table[(int64_t)pos * half + i] : 1.f;
    sn[j] = (cos_table && i < half) ? sin_table[(int64_t)pos * half + i] : 0.f;
  }
  pdl_wait();
  pdl_launch_dependents();

  for (int h = blockIdx.y * nwarps + warp; h < heads; h += gridDim.y * nwarps) {
    const T* src = qkv + in_base + (int64_t)h * d;
    const float* psrc = partial ? partial + in_base + (int64_t)h * d : nullptr;
    // element i of this head: the stored projection, or the sum of its K-split partial sums
    auto load = [&](int i) -> float {
      if (partial == nullptr) return to_f32(src[i]);
      float v = 0.f;
      for (int s = 0; s < splits; ++s) v += psrc[s * plane + i];
      return v;
    };
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    T* dst;
    if (is_q) {
      dst = q_out + ((int64_t)t * nq + h) * d;
    } else {
      if (slot < 0) continue;
      const int g = is_k ? h - nq : h - nq - nkv;
      // caches are [pages, kv heads, page_size, d]: a head's tokens of a page are contiguous
      dst = (is_k ? k_cache : v_cache) + (((slot / page_size) * nkv + g) * page_size + slot % page_size) * d;
    }
    if (partial != nullptr) {
      // from the projection's partial sums: the arithmetic the fused decode attention shares
      const bool rotated = is_q || is_k;
      head_from_partial<T>(psrc, splits, plane, d, lane, is_q ? q_norm_w : (is_k ? k_norm_w : nullptr), norm_w_is_f32, eps,
                           rotated ? cos_table : nullptr, rotated ? sin_table : nullptr, pos, dst, (T*)nullptr);
      continue;
    }
    if (!is_q && !is_k) {  // value head: plain copy
      for (int i = lane; i < d; i += 32) dst[i] = partial == nullptr ? src[i] : from_f32<T>(load(i));
      continue;
    }
    float x1[MAX_PAIRS_PER_LANE], x2[MAX_PAIRS_PER_LANE];
    float ss = 0.f;
    if (partial == nullptr) {
#pragma unroll
      for (int j = 0; j < MAX_PAIRS_PER_LANE; ++j) {
        const int i = lane + 32 * j;
        x1[j] = i < half ? to_f32(src[i]) : 0.f;
        x2[j] = i < half ? to_f32(src[i + half]) : 0.f;
      }
    } else {
      // the loads of up to four splits are issued together; the sums still run in split order
#pragma unroll
      for (int j = 0; j < MAX_PAIRS_PER_LANE; ++j) x1[j] = x2[j] = 0.f;
      constexpr int FLIGHT = 4;
      for (int s0 = 0; s0 < splits; s0 += FLIGHT) {
        float v1[FLIGHT][MAX_PAIRS_PER_LANE], v2[FLIGHT][MAX_PAIRS_PER_LANE];
#pragma unroll
        for (int f = 0; f < FLIGHT; ++f)
#pragma unroll
          for (int j = 0; j < MAX_PAIRS_PER_LANE; ++j) {
            const int i = lane + 32 * j;
            const bool live = s0 + f < splits && i < half;
            v1[f][j] = live ? psrc[(s0 + f) * plane + i] : 0.f;
            v2[f][j] = live ? psrc[(s0 + f) * plane + i + half] : 0.f;
          }
#pragma unroll
        for (int f = 0; f < FLIGHT; ++f)
          if (s0 + f < splits) {
#pragma unroll
            for (int j = 0; j < MAX_PAIRS_PER_LANE; ++j) {
              x1[j] += v1[f][j];
              x2[j] += v2[f][j];
            }
          }
      }
    }
#pragma unroll
    for (int j = 0; j < MAX_PAIRS_PER_LANE; ++j) ss += x1[j] * x1[j] + x2[j] * x2[j];
    const void* w = is_q ? q_norm_w : k_norm_w;
    float rrms = 1.f;
    if (w) rrms = rsqrtf(warp_sum(ss) / (float)d + eps);
#pragma unroll
    for (int j = 0; j < MAX_PAIRS_PER_LANE; ++j) {
      const int i = lane + 32 * j;
      if (i >= half) continue;
      float a = x1[j], b = x2[j];
      if (w) {
        a = a * rrms * load_flex(w, norm_w_is_f32, i);
        b = b * rrms * load_flex(w, norm_w_is_f32, i + half);
      }
      if (cos_table) {
        const float c = cs[j], s = sn[j];
        const float ra = a * c - b * s, rb = b * c + a * s;
        a = ra;
        b = rb;
      }
      dst[i] = from_f32<T>(a);
      dst[i + half] = from_f32<T>(b);
    }
  }
}

// The same pass for many tokens (prompts), bfloat16, head sizes 64, 128 and 256, as a stream: a
// block walks over tokens; a token's row of the projection and its rows of the rotation tables come
// by bulk copies into a ring of `stages` buffers in shared memory (what a block has in flight
// costs no registers, so four blocks to an SM keep well over 100 KB on their way), the threads
// read 16-byte words from there (D / 16 lanes share a head: 8 consecutive elements of each half per
// lane) and write 16-byte words to q and the caches. (A block per token with 2- to 8-byte words
// per lane moved 2.7 TB/s at 8,192 tokens of the 8B sizes, with 16-byte words from global memory
// into registers 3.3.)
template <int D>
__global__ void __launch_bounds__(256, 4)
qkv_post_stream_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ q_out, bf16* __restrict__ k_cache,
                       bf16* __restrict__ v_cache, const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w,
                       int norm_w_is_f32, float eps, const float* __restrict__ cos_table,
                       const float* __restrict__ sin_table, int max_positions, const int* __restrict__ positions,
                       const int* __restrict__ slot_mapping, int64_t num_slots, int page_size, int nq, int nkv, int tokens,
                       int stages, unsigned* status) {
  constexpr int HALF = D / 2, LANES_PER_HEAD = D / 16, E = 8, MAX_STAGES = 4;
  extern __shared__ __align__(16) uint8_t stream_smem[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
  __shared__ __align__(16) float wq_s[D], wk_s[D];
  const int heads = nq + 2 * nkv;
  const uint32_t row_bytes = (uint32_t)heads * D * 2, table_bytes = HALF * 4;
  const uint32_t stage_bytes = row_bytes + 2 * table_bytes;      // the row, then the cosines, then the sines
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LANES_PER_HEAD;                         // this lane's elements: sub * 8 .. sub * 8 + 7 of each half
  const int mine = (int)blockIdx.x < tokens ? (tokens - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < MAX_STAGES; ++i) mb_init(smem_addr(&full_bar[i]), 1);
    mb_fence_init();
  }
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    wq_s[i] = q_norm_w ? load_flex(q_norm_w, norm_w_is_f32, i) : 1.f;
    wk_s[i] = k_norm_w ? load_flex(k_norm_w, norm_w_is_f32, i) : 1.f;
  }
  __syncthreads();
  pdl_wait();                      // the projection comes from the kernel before this one
  pdl_launch_dependents();

  // token number i of this block, whose position is `pos`, into buffer i % stages (thread 0)
  auto token_of = [&](int i) { return (int)blockIdx.x + i * (int)gridDim.x; };
  auto position_of = [&](int i) { return (positions && i < mine) ? positions[token_of(i)] : 0; };
  auto issue = [&](int i, int pos) {
    const int t = token_of(i);
    uint8_t* stage = stream_smem + (size_t)(i % stages) * stage_bytes;
    const uint32_t bar = smem_addr(&full_bar[i % stages]);
    if (cos_table && (pos < 0 || pos >= max_positions)) {
      raise_fault(status, VOSTI_FAULT_POSITION_RANGE);
      pos = 0;
    }
    mb_expect_tx(bar, row_bytes + (cos_table ? 2 * table_bytes : 0));
    bulk_copy_g2s(smem_addr(stage), qkv + (int64_t)t * heads * D, row_bytes, bar);
    if (cos_table) {
      bulk_copy_g2s(smem_addr(stage + row_bytes), cos_table + (int64_t)pos * HALF, table_bytes, bar);
      bulk_copy_g2s(smem_addr(stage + row_bytes + table_bytes), sin_table + (int64_t)pos * HALF, table_bytes, bar);
    }
  };
  if (threadIdx.x == 0)
    for (int i = 0; i < mine && i < stages - 1; ++i) issue(i, position_of(i));
  // what the next copy and the next token's stores need is read a token ahead
  int pos_ahead = threadIdx.x == 0 ? position_of(stages - 1) : 0;
  auto slot_of = [&](int i) -> int64_t { return (nkv > 0 && slot_mapping && i < mine) ? (int64_t)slot_mapping[token_of(i)] : -1; };
  int64_t slot_ahead = slot_of(0);

  const int items = heads * LANES_PER_HEAD;                      // (head, lane of the head) pairs of a token
  for (int i = 0; i < mine; ++i) {
    const int t = token_of(i);
    // every thread is done with the buffer the next copy goes to (it held token i - 1)
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
      if (i + stages - 1 < mine) issue(i + stages - 1, pos_ahead);
      pos_ahead = position_of(i + stages);
    }
    int64_t slot = slot_ahead;
    slot_ahead = slot_of(i + 1);
    if (slot >= num_slots || slot < -1) {
      if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
      slot = -1;
    }
    const uint8_t* stage = stream_smem + (size_t)(i % stages) * stage_bytes;
    if (!mb_wait(smem_addr(&full_bar[i % stages]), (uint32_t)(i / stages) & 1, status)) return;
    const float* c_s = reinterpret_cast<const float*>(stage + row_bytes);
    const float* sn_s = c_s + HALF;
    for (int base = warp * 32; base < items; base += (int)blockDim.x) {   // (a warp's lanes stay together: shuffles below)
      const int item = base + lane;
      const bool live = item < items;
      const int h = item / LANES_PER_HEAD;
      const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
      uint4 a = make_uint4(0, 0, 0, 0), b = a;
      if (live) {
        a = *reinterpret_cast<const uint4*>(stage + ((size_t)h * D + sub * E) * 2);
        b = *reinterpret_cast<const uint4*>(stage + ((size_t)h * D + HALF + sub * E) * 2);
      }
      float x1[E], x2[E], ss = 0.f;
      const bf16* av = reinterpret_cast<const bf16*>(&a);
      const bf16* bv = reinterpret_cast<const bf16*>(&b);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        x1[e] = to_f32(av[e]);
        x2[e] = to_f32(bv[e]);
        ss += x1[e] * x1[e] + x2[e] * x2[e];
      }
      // the head's sum of squares over the lanes that share it (every lane of the warp takes part)
#pragma unroll
      for (int o = 1; o < LANES_PER_HEAD; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (!live) continue;
      bf16* dst;
      if (is_q) {
        dst = q_out + ((int64_t)t * nq + h) * D;
      } else {
        if (slot < 0) continue;
        const int g = is_k ? h - nq : h - nq - nkv;
        dst = (is_k ? k_cache : v_cache) + (((slot / page_size) * nkv + g) * page_size + slot % page_size) * D;
      }
      if (is_q || is_k) {
        const bool normed = is_q ? q_norm_w != nullptr : k_norm_w != nullptr;
        const float rrms = normed ? rsqrtf(ss / (float)D + eps) : 1.f;
        const float* w = is_q ? wq_s : wk_s;
        // this lane's eight weights of each half and its eight rotation factors, as 16-byte words
        float w1[E], w2[E], cs[E], sj[E];
#pragma unroll
        for (int v = 0; v < E / 4; ++v) {
          *reinterpret_cast<float4*>(w1 + 4 * v) = *reinterpret_cast<const float4*>(w + sub * E + 4 * v);
          *reinterpret_cast<float4*>(w2 + 4 * v) = *reinterpret_cast<const float4*>(w + HALF + sub * E + 4 * v);
          *reinterpret_cast<float4*>(cs + 4 * v) = *reinterpret_cast<const float4*>(c_s + sub * E + 4 * v);
          *reinterpret_cast<float4*>(sj + 4 * v) = *reinterpret_cast<const float4*>(sn_s + sub * E + 4 * v);
        }
        uint32_t pa[E / 2], pb[E / 2];
#pragma unroll
        for (int e = 0; e < E; e += 2) {
          float p[2], r[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            p[j] = x1[e + j];
            r[j] = x2[e + j];
            if (normed) {
              p[j] = p[j] * rrms * w1[e + j];
              r[j] = r[j] * rrms * w2[e + j];
            }
            if (cos_table) {
              const float ra = p[j] * cs[e + j] - r[j] * sj[e + j], rb = r[j] * cs[e + j] + p[j] * sj[e + j];
              p[j] = ra;
              r[j] = rb;
            }
          }
          __nv_bfloat162 va = __floats2bfloat162_rn(p[0], p[1]), vb = __floats2bfloat162_rn(r[0], r[1]);
          pa[e / 2] = *reinterpret_cast<uint32_t*>(&va);
          pb[e / 2] = *reinterpret_cast<uint32_t*>(&vb);
        }
        a = make_uint4(pa[0], pa[1], pa[2], pa[3]);
        b = make_uint4(pb[0], pb[1], pb[2], pb[3]);
      }
      *reinterpret_cast<uint4*>(dst + sub * E) = a;
      *reinterpret_cast<uint4*>(dst + HALF + sub * E) = b;
    }
  }
}

// The same pass for rotations that are not the half-split rotation of the whole head: only the
// first `rotary_dim` elements of a head are rotated (pairs (i, i + rotary_dim/2)), or the pairs
// are neighbours (2i, 2i + 1) ("interleaved"); the rest of the head passes through after the
// norm. One block per (token, head), the head in shared memory: slow and plain, for
// architectures whose position encoding asks for it (Qwen3 does not).
template <typename T>
__global__ void __launch_bounds__(128)
qkv_post_general_kernel(const T* __restrict__ qkv, const float* __restrict__ partial, int splits, int64_t plane,
                        T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                        const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int norm_w_is_f32, float eps,
                        const float* __restrict__ cos_table, const float* __restrict__ sin_table, int max_positions,
                        const int* __restrict__ positions, const int* __restrict__ slot_mapping, int64_t num_slots,
                        int page_size, int nq, int nkv, int d, int rotary_dim, int interleaved, unsigned* status) {
  __shared__ float scratch[32];
  extern __shared__ float head[];                      // d floats
  const int t = blockIdx.x, h = blockIdx.y;
  const int heads = nq + 2 * nkv;
  const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
  pdl_wait();
  pdl_launch_dependents();
  int pos = positions ? positions[t] : 0;
  if (cos_table && (pos < 0 || pos >= max_positions)) {
    if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_POSITION_RANGE);
    pos = 0;
  }
  T* dst;
  if (is_q) {
    dst = q_out + ((int64_t)t * nq + h) * d;
  } else {
    int64_t slot = slot_mapping ? slot_mapping[t] : -1;
    if (slot >= num_slots || slot < -1) {
      if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
      slot = -1;
    }
    if (slot < 0) return;
    const int g = is_k ? h - nq : h - nq - nkv;
    dst = (is_k ? k_cache : v_cache) + (((slot / page_size) * nkv + g) * page_size + slot % page_size) * d;
  }
  const int64_t at = ((int64_t)t * heads + h) * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = 0.f;
    if (partial == nullptr) v = to_f32(qkv[at + i]);
    else for (int s = 0; s < splits; ++s) v += partial[s * plane + at + i];
    head[i] = v;
    ss += v * v;
  }
  const void* w = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
  const float total = block_sum(ss, scratch);          // (also: the head is complete in shared memory)
  if (w != nullptr) {
    const float rrms = rsqrtf(total / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) head[i] = head[i] * rrms * load_flex(w, norm_w_is_f32, i);
    __syncthreads();
  }
  const bool rotated = (is_q || is_k) && cos_table != nullptr;
  const int rd = rotated ? rotary_dim : 0, half = rd >> 1;
  for (int p = threadIdx.x; p < half; p += blockDim.x) {
    const int ia = interleaved ? 2 * p : p, ib = interleaved ? 2 * p + 1 : p + half;
    const float c = cos_table[(int64_t)pos * half + p], sn = sin_table[(int64_t)pos * half + p];
    const float a = head[ia], b = head[ib];
    dst[ia] = from_f32<T>(a * c - b * sn);
    dst[ib] = from_f32<T>(b * c + a * sn);
  }
  for (int i = rd + threadIdx.x; i < d; i += blockDim.x) dst[i] = from_f32<T>(head[i]);
}
}  // namespace

// qkv: [tokens, (nq + 2*nkv) * d], or null with `partial`: float32 [splits, tokens, (nq + 2*nkv) * d],
// the K-split partial sums of the projection, summed here in split order.
// q_out: [tokens, nq * d]; caches: [pages, nkv, page_size, d] with num_slots = pages * page_size;
// slot s is (page s / page_size, offset s % page_size).
// nkv == 0: the input holds query heads only and nothing is stored.
// q_norm_w / k_norm_w null: no head norm. cos/sin null: no rotation; else float32
// tables [max_positions, rotary_dim/2]: the first rotary_dim elements of q and k heads are rotated,
// pairs (i, i + rotary_dim/2) or, with `interleaved`, (2i, 2i + 1).
VOSTI_API int vosti_qkv_post(const void* qkv, const float* partial, int splits, void* q_out, void* k_cache, void* v_cache, const void* q_norm_w,
                             const void* k_norm_w, int norm_w_is_f32, float eps, const float* cos_table,
                             const float* sin_table, int max_positions, const int* positions,
                             const int* slot_mapping, int64_t num_slots, int page_size, int tokens, int nq, int nkv, int d,
                             int rotary_dim, int interleaved, int is_f32, unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && nq > 0 && nkv >= 0 && d > 0, "qkv_post: bad sizes");
  VOSTI_REQUIRE(cos_table == nullptr || (rotary_dim > 0 && rotary_dim <= d && rotary_dim % 2 == 0),
                "qkv_post: rotary_dim %d must be even and between 2 and head_dim %d", rotary_dim, d);
  VOSTI_REQUIRE(nkv == 0 || page_size > 0, "qkv_post: page_size must be positive");
  VOSTI_REQUIRE((qkv != nullptr) != (partial != nullptr), "qkv_post: give the projection or its partial sums");
  VOSTI_REQUIRE(partial == nullptr || splits >= 1, "qkv_post: bad split count");
  const int64_t plane = (int64_t)tokens * (nq + 2 * nkv) * d;
  VOSTI_REQUIRE(d % 2 == 0 && d / 2 <= 32 * MAX_PAIRS_PER_LANE, "qkv_post: head_dim %d must be even and <= %d", d,
                64 * MAX_PAIRS_PER_LANE);
  VOSTI_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "qkv_post: cos and sin go together");
  VOSTI_REQUIRE(cos_table == nullptr || positions != nullptr, "qkv_post: rotation needs positions");
  if (tokens == 0) return VOSTI_OK;
  const int heads = nq + 2 * nkv;
  if (cos_table != nullptr && (rotary_dim != d || interleaved)) {
    VOSTI_REQUIRE(heads <= 65535, "qkv_post: too many heads for one launch");
    const dim3 grid(tokens, heads);
    const size_t smem = (size_t)d * sizeof(float);
    if (is_f32)
      vosti_launch(qkv_post_general_kernel<float>, grid, dim3(128), smem, stream, (const float*)qkv, partial, splits, plane,
                   (float*)q_out, (float*)k_cache, (float*)v_cache, q_norm_w, k_norm_w, norm_w_is_f32, eps, cos_table, sin_table,
                   max_positions, positions, slot_mapping, num_slots, page_size, nq, nkv, d, rotary_dim, interleaved, status);
    else
      vosti_launch(qkv_post_general_kernel<bf16>, grid, dim3(128), smem, stream, (const bf16*)qkv, partial, splits, plane,
                   (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, q_norm_w, k_norm_w, norm_w_is_f32, eps, cos_table, sin_table,
                   max_positions, positions, slot_mapping, num_slots, page_size, nq, nkv, d, rotary_dim, interleaved, status);
    VOSTI_LAUNCH_CHECK();
  }
  // many tokens: the streaming kernel, if two buffers of a token's row fit a block's share of an SM
  const size_t stream_stage = (size_t)heads * d * 2 + (size_t)d * 4;          // the row and its two table rows
  if (!is_f32 && partial == nullptr && tokens >= 64 && !g_vosti_fixed_order && (d == 64 || d == 128 || d == 256) &&
      2 * stream_stage <= 100 * 1024 && ((uintptr_t)qkv % 16 == 0) && ((size_t)heads * d * 2) % 16 == 0 &&
      (cos_table == nullptr || ((uintptr_t)cos_table % 16 == 0 && (uintptr_t)sin_table % 16 == 0))) {
    // four blocks to an SM where the buffers allow it; up to four buffers each
    int stages = (int)((54 * 1024) / stream_stage);
    stages = stages > 4 ? 4 : stages < 2 ? 2 : stages;
    const size_t smem = (size_t)stages * stream_stage;
    const int per_sm = smem <= 54 * 1024 ? 4 : 2;
    const int blocks = tokens < 148 * per_sm ? tokens : 148 * per_sm;
    // as many threads as share a token's (head, lane of the head) pairs evenly in whole warps
    const int items = heads * (d / 16), passes = (items + 255) / 256;
    const int threads = ((items + passes - 1) / passes + 31) / 32 * 32;
#define LAUNCH_QKV_POST_STREAM(D)                                                                                 \
    do {                                                                                                           \
      static bool configured = false;                                                                              \
      if (!configured) {                                                                                           \
        cudaFuncSetAttribute(qkv_post_stream_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);   \
        configured = true;                                                                                         \
      }                                                                                                            \
      vosti_launch(qkv_post_stream_kernel<D>, dim3(blocks), dim3(threads), smem, stream, (const bf16*)qkv, (bf16*)q_out, \
          (bf16*)k_cache, (bf16*)v_cache, q_norm_w, k_norm_w, norm_w_is_f32, eps, cos_table, sin_table,            \
          max_positions, positions, slot_mapping, num_slots, page_size, nq, nkv, tokens, stages, status);          \
    } while (0)
    if (d == 64) LAUNCH_QKV_POST_STREAM(64);
    else if (d == 128) LAUNCH_QKV_POST_STREAM(128);
    else LAUNCH_QKV_POST_STREAM(256);
#undef LAUNCH_QKV_POST_STREAM
    VOSTI_LAUNCH_CHECK();
  }
  const dim3 grid(tokens, (heads + 3) / 4);                          // a warp per (token, head)
  if (is_f32)
    vosti_launch(qkv_post_kernel<float>, grid, dim3(128), 0, stream, (const float*)qkv, partial, splits, plane, (float*)q_out, (float*)k_cache,
        (float*)v_cache, q_norm_w, k_norm_w, norm_w_is_f32, eps, cos_table, sin_table, max_positions, positions,
        slot_mapping, num_slots, page_size, nq, nkv, d, status);
  else
    vosti_launch(qkv_post_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)qkv, partial, splits, plane, (bf16*)q_out, (bf16*)k_cache,
        (bf16*)v_cache, q_norm_w, k_norm_w, norm_w_is_f32, eps, cos_table, sin_table, max_positions, positions,
        slot_mapping, num_slots, page_size, nq, nkv, d, status);
  VOSTI_LAUNCH_CHECK();
}

// The arithmetic of one head after the QKV projection, shared by qkv_post.cu and the fused
// decode attention so that both give the same bits: the head's elements are the sums of the
// projection's K-split partial sums in split order; per-head RMSNorm (optional) with float32
// statistics; half-split rotation (optional); one rounding at the store. Every product and sum
// is written with the unfused intrinsics, so that the compiler contracts nothing differently in
// the two kernels. Formulas: kernels/triton_kernels/qk_norm.py:40-95, rope.py:78-101.
#pragma once
#include "common.cuh"

constexpr int HEAD_MAX_PAIRS = 8;      // pairs (i, i + d/2) a lane holds: head_dim <= 512

// Loads that are issued where they stand: the compiler neither moves them down to their first use
// nor puts a use between them.
__device__ __forceinline__ uint32_t issue_load_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.global.b32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t issue_load_u16(const unsigned short* p) {
  unsigned short v;
  asm volatile("ld.global.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return (uint32_t)v;
}

// One warp, one head: lane l holds the pairs i = l + 32 j, j < PAIRS (the caller chooses PAIRS so
// that 64 PAIRS >= d; fewer pairs, fewer registers, the same arithmetic per element). `src` points
// at the head's first element in split 0; split s lies s * plane further on. The result goes to
// `dst` and, if given, to `dst2` as well (element i at dst[i]).
template <typename T, int PAIRS = HEAD_MAX_PAIRS>
__device__ __forceinline__ void head_from_partial(const float* __restrict__ src, int splits, long long plane, int d, int lane,
                                                  const void* __restrict__ norm_w, int norm_w_is_f32, float eps,
                                                  const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                                  int pos, T* __restrict__ dst, T* __restrict__ dst2) {
  const int half = d >> 1;
  float x1[PAIRS], x2[PAIRS];
#pragma unroll
  for (int j = 0; j < PAIRS; ++j) x1[j] = x2[j] = 0.f;
  // Norm weights and rotation factors do not depend on the sums. They are requested first and
  // looked at last (a weight stays raw bits until then), with loads that are issued where they stand,
  // so that they and the partial sums make one trip to memory together instead of several in a row.
  uint32_t w1[PAIRS], w2[PAIRS];
  float cs[PAIRS], sn[PAIRS];
#pragma unroll
  for (int j = 0; j < PAIRS; ++j) {
    const int i = lane + 32 * j;
    const bool live = i < half;
    w1[j] = w2[j] = 0u;
    cs[j] = 1.f;
    sn[j] = 0.f;
    if (live && norm_w != nullptr) {
      if (norm_w_is_f32) {
        w1[j] = issue_load_u32(reinterpret_cast<const uint32_t*>(norm_w) + i);
        w2[j] = issue_load_u32(reinterpret_cast<const uint32_t*>(norm_w) + i + half);
      } else {
        w1[j] = issue_load_u16(reinterpret_cast<const unsigned short*>(norm_w) + i);
        w2[j] = issue_load_u16(reinterpret_cast<const unsigned short*>(norm_w) + i + half);
      }
    }
    if (live && cos_table != nullptr) {
      cs[j] = __uint_as_float(issue_load_u32(reinterpret_cast<const uint32_t*>(cos_table + (long long)pos * half + i)));
      sn[j] = __uint_as_float(issue_load_u32(reinterpret_cast<const uint32_t*>(sin_table + (long long)pos * half + i)));
    }
  }
  // the loads of up to four splits (eight where a lane holds few pairs) are issued together; the
  // sums still run in split order
  constexpr int FLIGHT = PAIRS <= 2 ? 8 : 4;
  for (int s0 = 0; s0 < splits; s0 += FLIGHT) {
    float v1[FLIGHT][PAIRS], v2[FLIGHT][PAIRS];
#pragma unroll
    for (int f = 0; f < FLIGHT; ++f)
#pragma unroll
      for (int j = 0; j < PAIRS; ++j) {
        const int i = lane + 32 * j;
        const bool live = s0 + f < splits && i < half;
        v1[f][j] = live ? __uint_as_float(issue_load_u32(reinterpret_cast<const uint32_t*>(src + (s0 + f) * plane + i))) : 0.f;
        v2[f][j] = live ? __uint_as_float(issue_load_u32(reinterpret_cast<const uint32_t*>(src + (s0 + f) * plane + i + half))) : 0.f;
      }
#pragma unroll
    for (int f = 0; f < FLIGHT; ++f)
      if (s0 + f < splits) {
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) {
          x1[j] = __fadd_rn(x1[j], v1[f][j]);
          x2[j] = __fadd_rn(x2[j], v2[f][j]);
        }
      }
  }
  float rrms = 1.f;
  if (norm_w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PAIRS; ++j) ss = __fadd_rn(ss, __fadd_rn(__fmul_rn(x1[j], x1[j]), __fmul_rn(x2[j], x2[j])));
    rrms = rsqrtf(__fadd_rn(__fdiv_rn(warp_sum(ss), (float)d), eps));
  }
#pragma unroll
  for (int j = 0; j < PAIRS; ++j) {
    const int i = lane + 32 * j;
    if (i >= half) continue;
    float a = x1[j], b = x2[j];
    if (norm_w != nullptr) {
      // (a bfloat16 weight is the upper half of its float32 value)
      a = __fmul_rn(__fmul_rn(a, rrms), __uint_as_float(norm_w_is_f32 ? w1[j] : w1[j] << 16));
      b = __fmul_rn(__fmul_rn(b, rrms), __uint_as_float(norm_w_is_f32 ? w2[j] : w2[j] << 16));
    }
    if (cos_table != nullptr) {
      const float c = cs[j], sn_j = sn[j];
      const float ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn_j)), rb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn_j));
      a = ra;
      b = rb;
    }
    dst[i] = from_f32<T>(a);
    dst[i + half] = from_f32<T>(b);
    if (dst2 != nullptr) {
      dst2[i] = from_f32<T>(a);
      dst2[i + half] = from_f32<T>(b);
    }
  }
}

// The arithmetic of one head after the QKV projection, shared by qkv_post.cu and the fused
// decode attention so that both give the same bits: the head's elements are the sums of the
// projection's K-split partial sums in split order; per-head RMSNorm (optional) with float32
// statistics; half-split rotation (optional); one rounding at the store. Every product and sum
// is written with the unfused intrinsics, so that the compiler contracts nothing differently in
// the two kernels. Formulas: kernels/triton_kernels/qk_norm.py:40-95, rope.py:78-101.
#pragma once
#include "common.cuh"

constexpr int HEAD_MAX_PAIRS = 8;      // pairs (i, i + d/2) a lane holds: head_dim <= 512

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
  // the loads of up to four splits are issued together; the sums still run in split order
  constexpr int FLIGHT = 4;
  for (int s0 = 0; s0 < splits; s0 += FLIGHT) {
    float v1[FLIGHT][PAIRS], v2[FLIGHT][PAIRS];
#pragma unroll
    for (int f = 0; f < FLIGHT; ++f)
#pragma unroll
      for (int j = 0; j < PAIRS; ++j) {
        const int i = lane + 32 * j;
        const bool live = s0 + f < splits && i < half;
        v1[f][j] = live ? src[(s0 + f) * plane + i] : 0.f;
        v2[f][j] = live ? src[(s0 + f) * plane + i + half] : 0.f;
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
      a = __fmul_rn(__fmul_rn(a, rrms), load_flex(norm_w, norm_w_is_f32, i));
      b = __fmul_rn(__fmul_rn(b, rrms), load_flex(norm_w, norm_w_is_f32, i + half));
    }
    if (cos_table != nullptr) {
      const float c = cos_table[(long long)pos * half + i], sn = sin_table[(long long)pos * half + i];
      const float ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn)), rb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn));
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

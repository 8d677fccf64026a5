// Row-wise kernels: embedding gather, (residual-fused) RMSNorm, SiLU(gate)*up.
// Formulas as the reference computes them: kernels/triton_kernels/embedding.py:62-84,
// rmsnorm.py:63-93, rmsnorm_residual.py:86-125, silu_mul.py:66-87. All arithmetic in
// float32; T is the storage type of activations (float or bf16).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// With `source`, row t takes its id from values[source[t]] where source[t] >= 0: a token the
// sampler of the step before left on the device, which the host has not read yet.
// `scale` multiplies the row in float32 (1: a plain copy), for architectures that scale
// their embeddings.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const int* __restrict__ source,
                                 const int* __restrict__ values, const T* __restrict__ table,
                                 T* __restrict__ out, int hidden, int vocab, float scale, unsigned* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  if (source != nullptr && source[t] >= 0) id = values[source[t]];
  const bool bad = id < 0 || id >= vocab;
  if (bad) {
    if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_TOKEN_RANGE);
    id = 0;
  }
  const T* src = table + (int64_t)id * hidden;
  T* dst = out + (int64_t)t * hidden;
  const int bytes = hidden * (int)sizeof(T);
  if (scale != 1.f) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      dst[i] = bad ? from_f32<T>(0.f) : from_f32<T>(to_f32(src[i]) * scale);
  } else if (bytes % 16 == 0) {
    const int4* s4 = reinterpret_cast<const int4*>(src);
    int4* d4 = reinterpret_cast<int4*>(dst);
    for (int i = threadIdx.x; i < bytes / 16; i += blockDim.x) d4[i] = bad ? make_int4(0, 0, 0, 0) : s4[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = bad ? from_f32<T>(0.f) : src[i];
  }
}

VOSTI_API int vosti_embedding(const int* ids, const int* source, const int* values, const void* table, void* out,
                              int tokens, int hidden, int vocab, int is_f32, float scale, unsigned* status,
                              cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes T=%d H=%d V=%d",
                tokens, hidden, vocab);
  if (tokens == 0) return VOSTI_OK;
  if (is_f32)
    vosti_launch(embedding_kernel<float>, dim3(tokens), dim3(128), 0, stream, ids, source, values, (const float*)table, (float*)out, hidden, vocab, scale, status);
  else
    vosti_launch(embedding_kernel<bf16>, dim3(tokens), dim3(128), 0, stream, ids, source, values, (const bf16*)table, (bf16*)out, hidden, vocab, scale, status);
  VOSTI_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- RMSNorm
// One block per row. With a residual: h = x + r in float32, residual_out = round(h),
// the variance and the scaling use the unrounded h. Without: h = x.
// The row is read twice (the second read hits L1/L2) so that any width works.
template <typename T, int BLOCK>
__global__ void __launch_bounds__(BLOCK)
rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ residual, const void* __restrict__ weight,
               int weight_is_f32, T* __restrict__ out, T* __restrict__ residual_out, int width, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t base = (int64_t)blockIdx.x * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += BLOCK) {
    float h = to_f32(x[base + i]);
    if (residual) h += to_f32(residual[base + i]);
    ss += h * h;
  }
  const float total = block_sum(ss, scratch);
  const float rrms = rsqrtf(total / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += BLOCK) {
    float h = to_f32(x[base + i]);
    if (residual) h += to_f32(residual[base + i]);
    if (residual_out) residual_out[base + i] = from_f32<T>(h);
    out[base + i] = from_f32<T>(h * rrms * load_flex(weight, weight_is_f32, i));
  }
}

// The same norm for bfloat16 rows whose width is a multiple of 8 and at most BLOCK * 8 * CH:
// 16-byte accesses, and the row stays in registers between the two passes.
template <int BLOCK, int CH>
__global__ void __launch_bounds__(BLOCK)
rmsnorm_vec_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual, const void* __restrict__ weight,
                   int weight_is_f32, bf16* __restrict__ out, bf16* __restrict__ residual_out, int width, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t base = (int64_t)blockIdx.x * width;
  const int chunks = width >> 3;
  float h[CH][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int idx = threadIdx.x + c * BLOCK;
    if (idx < chunks) {
      const uint4 xv = *reinterpret_cast<const uint4*>(x + base + idx * 8);
      const bf16* xe = reinterpret_cast<const bf16*>(&xv);
      if (residual) {
        const uint4 rv = *reinterpret_cast<const uint4*>(residual + base + idx * 8);
        const bf16* re = reinterpret_cast<const bf16*>(&rv);
#pragma unroll
        for (int e = 0; e < 8; ++e) h[c][e] = to_f32(xe[e]) + to_f32(re[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) h[c][e] = to_f32(xe[e]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += h[c][e] * h[c][e];
    }
  }
  const float total = block_sum(ss, scratch);
  const float rrms = rsqrtf(total / (float)width + eps);
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int idx = threadIdx.x + c * BLOCK;
    if (idx < chunks) {
      uint4 ov, hv;
      bf16* oe = reinterpret_cast<bf16*>(&ov);
      bf16* he = reinterpret_cast<bf16*>(&hv);
      // the chunk's eight weights as 16-byte words (the weight tensor is 16-byte aligned: checked by the launcher)
      float w[8];
      if (weight_is_f32) {
        const float4 w0 = reinterpret_cast<const float4*>(weight)[idx * 2], w1 = reinterpret_cast<const float4*>(weight)[idx * 2 + 1];
        w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w; w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
      } else {
        const uint4 wv = reinterpret_cast<const uint4*>(weight)[idx];
        const bf16* we = reinterpret_cast<const bf16*>(&wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = to_f32(we[e]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        he[e] = from_f32<bf16>(h[c][e]);
        oe[e] = from_f32<bf16>(h[c][e] * rrms * w[e]);
      }
      if (residual_out) *reinterpret_cast<uint4*>(residual_out + base + idx * 8) = hv;
      *reinterpret_cast<uint4*>(out + base + idx * 8) = ov;
    }
  }
}

// `residual` may be null (plain norm). `residual_out` may be `residual` or `x` itself:
// a thread owns the same elements in both passes and reads each before it writes it.
// `out` must be a buffer of its own.
VOSTI_API int vosti_rmsnorm(const void* x, const void* residual, const void* weight, int weight_is_f32,
                            void* out, void* residual_out, int rows, int width, float eps, int is_f32,
                            cudaStream_t stream) {
  VOSTI_REQUIRE(rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", rows, width);
  VOSTI_REQUIRE(eps > 0.f, "rmsnorm: eps must be positive");
  if (rows == 0) return VOSTI_OK;
  VOSTI_REQUIRE(out != x && out != residual && out != residual_out, "rmsnorm: out must not alias another operand");
  const auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!is_f32 && width % 8 == 0 && width <= 256 * 8 * 4 && aligned(x) && aligned(residual) && aligned(out) &&
      aligned(residual_out) && aligned(weight)) {
    vosti_launch(rmsnorm_vec_kernel<256, 4>, dim3(rows), dim3(256), 0, stream, (const bf16*)x, (const bf16*)residual,
                 weight, weight_is_f32, (bf16*)out, (bf16*)residual_out, width, eps);
    VOSTI_LAUNCH_CHECK();
  }
  if (is_f32)
    vosti_launch(rmsnorm_kernel<float, 256>, dim3(rows), dim3(256), 0, stream, (const float*)x, (const float*)residual,
                 weight, weight_is_f32, (float*)out, (float*)residual_out, width, eps);
  else
    vosti_launch(rmsnorm_kernel<bf16, 256>, dim3(rows), dim3(256), 0, stream, (const bf16*)x, (const bf16*)residual,
                 weight, weight_is_f32, (bf16*)out, (bf16*)residual_out, width, eps);
  VOSTI_LAUNCH_CHECK();
}

constexpr int PREFETCH_LANES = 64;      // threads of a prefetch block that issue requests
constexpr int PREFETCH_BLOCKS = 48;     // blocks added to a launch that carries a prefetch hint

// The same norm fed by the float32 partial sums of a split-K product: x[t, i] is the sum of
// `splits` planes of [rows, width] taken in split order; it is not rounded before the add.
template <typename T, int BLOCK>
__global__ void __launch_bounds__(BLOCK)
rmsnorm_partial_kernel(const float* __restrict__ partial, int splits, int64_t plane, const T* __restrict__ residual,
                       const void* __restrict__ weight, int weight_is_f32, T* __restrict__ out,
                       T* __restrict__ residual_out, int rows, int width, float eps, VostiPrefetch ahead) {
  __shared__ float scratch[32];
  extern __shared__ float row_sum[];                       // the summed row, kept for the second pass
  if ((int)blockIdx.x >= rows) {
    // a block beyond the rows: it only asks for the next product's weights and leaves; it reads
    // nothing another kernel writes, so it does not wait for the kernel before this one
    pdl_launch_dependents();
    if (threadIdx.x < PREFETCH_LANES)
      l2_prefetch_share(ahead, (long long)((int)blockIdx.x - rows) * PREFETCH_LANES + threadIdx.x,
                        (long long)((int)gridDim.x - rows) * PREFETCH_LANES);
    return;
  }
  // the norm weights do not depend on the kernel before this one: read them while it still runs
  constexpr int PRELOAD = 4;
  float w_pre[PRELOAD];
#pragma unroll
  for (int j = 0; j < PRELOAD; ++j) {
    const int i = threadIdx.x + j * BLOCK;
    w_pre[j] = i < width ? load_flex(weight, weight_is_f32, i) : 0.f;
  }
  pdl_wait();
  pdl_launch_dependents();
  const int64_t base = (int64_t)blockIdx.x * width;
  float ss = 0.f;
  if ((width & 3) == 0) {
    // four consecutive columns per thread as one 16-byte load per split, up to eight splits in
    // flight at once; the sum over splits still runs in split order
    constexpr int FLIGHT = 8;
    for (int i = threadIdx.x * 4; i < width; i += BLOCK * 4) {
      float4 h = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s0 = 0; s0 < splits; s0 += FLIGHT) {
        float4 v[FLIGHT];
#pragma unroll
        for (int j = 0; j < FLIGHT; ++j)
          if (s0 + j < splits) v[j] = *reinterpret_cast<const float4*>(partial + (s0 + j) * plane + base + i);
#pragma unroll
        for (int j = 0; j < FLIGHT; ++j)
          if (s0 + j < splits) {
            h.x += v[j].x; h.y += v[j].y; h.z += v[j].z; h.w += v[j].w;
          }
      }
      if (residual) {
        h.x += to_f32(residual[base + i]); h.y += to_f32(residual[base + i + 1]);
        h.z += to_f32(residual[base + i + 2]); h.w += to_f32(residual[base + i + 3]);
      }
      *reinterpret_cast<float4*>(row_sum + i) = h;
      ss += h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
    }
  } else {
    constexpr int GROUP = 4;                               // elements a thread sums at once: independent loads
    for (int i0 = threadIdx.x; i0 < width; i0 += BLOCK * GROUP) {
      float h[GROUP];
#pragma unroll
      for (int j = 0; j < GROUP; ++j) h[j] = 0.f;
      for (int s = 0; s < splits; ++s) {
#pragma unroll
        for (int j = 0; j < GROUP; ++j) {
          const int i = i0 + j * BLOCK;
          if (i < width) h[j] += partial[s * plane + base + i];
        }
      }
#pragma unroll
      for (int j = 0; j < GROUP; ++j) {
        const int i = i0 + j * BLOCK;
        if (i < width) {
          if (residual) h[j] += to_f32(residual[base + i]);
          row_sum[i] = h[j];
          ss += h[j] * h[j];
        }
      }
    }
  }
  __syncthreads();                                         // the second pass reads other threads' columns
  const float total = block_sum(ss, scratch);
  const float rrms = rsqrtf(total / (float)width + eps);
#pragma unroll
  for (int j = 0; j < PRELOAD; ++j) {
    const int i = threadIdx.x + j * BLOCK;
    if (i < width) {
      const float h = row_sum[i];
      if (residual_out) residual_out[base + i] = from_f32<T>(h);
      out[base + i] = from_f32<T>(h * rrms * w_pre[j]);
    }
  }
  for (int i = threadIdx.x + PRELOAD * BLOCK; i < width; i += BLOCK) {
    const float h = row_sum[i];
    if (residual_out) residual_out[base + i] = from_f32<T>(h);
    out[base + i] = from_f32<T>(h * rrms * load_flex(weight, weight_is_f32, i));
  }
}

// partial: float32 [splits, rows, width]; residual may be null; residual_out may be residual.
VOSTI_API int vosti_rmsnorm_partial(const float* partial, int splits, const void* residual, const void* weight,
                                    int weight_is_f32, void* out, void* residual_out, int rows, int width, float eps,
                                    int is_f32, cudaStream_t stream) {
  VOSTI_REQUIRE(rows >= 0 && width > 0 && splits >= 1, "rmsnorm_partial: bad sizes rows=%d width=%d splits=%d", rows, width, splits);
  VOSTI_REQUIRE(eps > 0.f, "rmsnorm_partial: eps must be positive");
  VOSTI_REQUIRE(width <= 24576, "rmsnorm_partial: width %d does not fit the row buffer", width);
  const VostiPrefetch ahead = vosti_take_prefetch();
  if (rows == 0) return VOSTI_OK;
  VOSTI_REQUIRE(out != residual && out != residual_out, "rmsnorm_partial: out must not alias another operand");
  const int64_t plane = (int64_t)rows * width;
  const size_t smem = (size_t)width * sizeof(float);
  const dim3 grid(rows + (ahead.ptr != nullptr ? PREFETCH_BLOCKS : 0));
  if (is_f32) {
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(rmsnorm_partial_kernel<float, 1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, 24576 * 4);
      configured = true;
    }
    vosti_launch(rmsnorm_partial_kernel<float, 1024>, grid, dim3(1024), smem, stream, partial, splits, plane,
                 (const float*)residual, weight, weight_is_f32, (float*)out, (float*)residual_out, rows, width, eps, ahead);
  } else {
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(rmsnorm_partial_kernel<bf16, 1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, 24576 * 4);
      configured = true;
    }
    vosti_launch(rmsnorm_partial_kernel<bf16, 1024>, grid, dim3(1024), smem, stream, partial, splits, plane,
                 (const bf16*)residual, weight, weight_is_f32, (bf16*)out, (bf16*)residual_out, rows, width, eps, ahead);
  }
  VOSTI_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- SiLU(gate) * up
// in: [rows, 2*inter] with the gate half first; out: [rows, inter].
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int64_t rows, int inter) {
  const int64_t n = rows * inter;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / inter;
    const int c = (int)(i - r * inter);
    const float g = to_f32(gate_up[r * 2 * inter + c]);
    const float u = to_f32(gate_up[r * 2 * inter + inter + c]);
    out[i] = from_f32<T>(g * (1.f / (1.f + expf(-g))) * u);
  }
}

VOSTI_API int vosti_silu_mul(const void* gate_up, void* out, int rows, int inter, int is_f32,
                             cudaStream_t stream) {
  VOSTI_REQUIRE(rows >= 0 && inter > 0, "silu_mul: bad sizes rows=%d inter=%d", rows, inter);
  if (rows == 0) return VOSTI_OK;
  const int64_t n = (int64_t)rows * inter;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (is_f32)
    silu_mul_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, rows, inter);
  else
    silu_mul_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)gate_up, (bf16*)out, rows, inter);
  VOSTI_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- scale, bias, soft cap
// out[r, c] = cap(in[r, c] * scale + bias[c]) from a float32 product, rounded once:
// cap(y) = softcap * tanh(y / softcap) when softcap > 0, else y. `bias` may be null; `out` may
// be `in` when it is float32. This is what a projection with a bias or an output head with a
// logit scale or soft cap adds after the product; Qwen3 has none of them and never launches it.
template <typename TO>
__global__ void affine_rows_kernel(const float* in, int64_t in_stride, const void* __restrict__ bias, int bias_is_f32,
                                   TO* out, int64_t out_stride, int width, float scale, float softcap) {
  pdl_wait();
  pdl_launch_dependents();
  const float* src = in + (int64_t)blockIdx.y * in_stride;
  TO* dst = out + (int64_t)blockIdx.y * out_stride;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < width; c += gridDim.x * blockDim.x) {
    float y = src[c] * scale;
    if (bias != nullptr) y += load_flex(bias, bias_is_f32, c);
    if (softcap > 0.f) y = softcap * tanhf(y * inv_cap);
    dst[c] = from_f32<TO>(y);
  }
}

VOSTI_API int vosti_affine_rows(const float* in, int64_t in_stride, const void* bias, int bias_is_f32, void* out,
                                int64_t out_stride, int out_is_f32, int rows, int width, float scale, float softcap,
                                cudaStream_t stream) {
  VOSTI_REQUIRE(rows >= 0 && width > 0 && in_stride >= width && out_stride >= width,
                "affine_rows: bad sizes rows=%d width=%d", rows, width);
  VOSTI_REQUIRE(rows <= 65535, "affine_rows: %d rows exceed one launch", rows);
  VOSTI_REQUIRE(softcap >= 0.f && scale == scale, "affine_rows: softcap must be >= 0 and scale a number");
  VOSTI_REQUIRE(out_is_f32 || (const void*)in != out, "affine_rows: only a float32 output may overwrite its input");
  if (rows == 0) return VOSTI_OK;
  const int blocks = (width + 1023) / 1024 < 1024 ? (width + 1023) / 1024 : 1024;
  if (out_is_f32)
    vosti_launch(affine_rows_kernel<float>, dim3(blocks, rows), dim3(256), 0, stream, in, in_stride, bias, bias_is_f32,
                 (float*)out, out_stride, width, scale, softcap);
  else
    vosti_launch(affine_rows_kernel<bf16>, dim3(blocks, rows), dim3(256), 0, stream, in, in_stride, bias, bias_is_f32,
                 (bf16*)out, out_stride, width, scale, softcap);
  VOSTI_LAUNCH_CHECK();
}

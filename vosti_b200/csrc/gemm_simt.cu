// Plain matrix product on the CUDA cores with true float32 arithmetic:
//   Y[t, n] = sum_k X[row(t), k] * W[n, k]        (W in [out, in] layout, no bias)
// It is the whole float32 path's product and the fallback of the bfloat16 path for
// operand types or sizes the tensor-core kernel refuses. Each output is one thread's
// sequential fused multiply-add chain over k = 0..K-1, so a row's value never depends
// on the other rows of the launch (the reference's matmul has the same property by
// choosing tiles from (N, K) only: kernels/triton_kernels/matmul.py:33-73, 95-147).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y,
                 const int* __restrict__ row_index, int rows, int x_rows, int n, int k,
                 unsigned* status) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int lr = threadIdx.x / 4, lk = (threadIdx.x % 4) * 4;

  // source row of the X tile row this thread loads (gathered for the LM head)
  int64_t xrow = -1;
  if (m0 + lr < rows) {
    int r = row_index ? row_index[m0 + lr] : m0 + lr;
    if (r < 0 || r >= x_rows) {
      raise_fault(status, VOSTI_FAULT_ROW_RANGE);
      r = -1;
    }
    xrow = r;
  }
  const int64_t wrow = (n0 + lr < n) ? (int64_t)(n0 + lr) : -1;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < k; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int kk = k0 + lk + i;
      xs[lk + i][lr] = (xrow >= 0 && kk < k) ? to_f32(x[xrow * k + kk]) : 0.f;
      ws[lk + i][lr] = (wrow >= 0 && kk < k) ? to_f32(w[wrow * k + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = m0 + ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tx * 4 + j;
      if (c < n) y[(int64_t)r * n + c] = from_f32<TY>(acc[i][j]);
    }
  }
}

template <typename TX, typename TW, typename TY>
void launch(const void* x, const void* w, void* y, const int* row_index, int rows, int x_rows, int n,
            int k, unsigned* status, cudaStream_t stream) {
  dim3 grid((n + BN - 1) / BN, (rows + BM - 1) / BM);
  gemm_simt_kernel<TX, TW, TY><<<grid, THREADS, 0, stream>>>((const TX*)x, (const TW*)w, (TY*)y, row_index,
                                                             rows, x_rows, n, k, status);
}

}  // namespace

// x: [x_rows, k]; w: [n, k]; y: [rows, n]. With row_index (int32[rows]) row t of the
// product is taken from x[row_index[t]]; without it rows == x_rows.
VOSTI_API int vosti_gemm_simt(const void* x, const void* w, void* y, const int* row_index, int rows,
                              int x_rows, int n, int k, int x_is_f32, int w_is_f32, int y_is_f32,
                              unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(rows >= 0 && n > 0 && k > 0 && x_rows >= 0, "gemm: bad sizes rows=%d n=%d k=%d", rows, n, k);
  VOSTI_REQUIRE(row_index != nullptr || rows == x_rows, "gemm: rows != x_rows without a row index");
  if (rows == 0) return VOSTI_OK;
  VOSTI_REQUIRE((rows + BM - 1) / BM <= 65535, "gemm: too many rows (%d) for one launch", rows);
  const int code = (x_is_f32 ? 4 : 0) | (w_is_f32 ? 2 : 0) | (y_is_f32 ? 1 : 0);
  switch (code) {
    case 0: launch<bf16, bf16, bf16>(x, w, y, row_index, rows, x_rows, n, k, status, stream); break;
    case 1: launch<bf16, bf16, float>(x, w, y, row_index, rows, x_rows, n, k, status, stream); break;
    case 2: launch<bf16, float, bf16>(x, w, y, row_index, rows, x_rows, n, k, status, stream); break;
    case 3: launch<bf16, float, float>(x, w, y, row_index, rows, x_rows, n, k, status, stream); break;
    case 4: launch<float, bf16, bf16>(x, w, y, row_index, rows, x_rows, n, k, status, stream); break;
    case 5: launch<float, bf16, float>(x, w, y, row_index, rows, x_rows, n, k, status, stream); break;
    case 6: launch<float, float, bf16>(x, w, y, row_index, rows, x_rows, n, k, status, stream); break;
    default: launch<float, float, float>(x, w, y, row_index, rows, x_rows, n, k, status, stream); break;
  }
  VOSTI_LAUNCH_CHECK();
}

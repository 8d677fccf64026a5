// Sampling over float32 logits rows, one block per row.
//   temperature <= 0: greedy, the lowest index of the maximum (the reference samples
//   with torch.argmax over the row only: python/vosti_kernels/kernels.py:1088-1104).
//   temperature  > 0: weights w_i = exp((l_i - max) / T); the token is the first whose
//   inclusive cumulative weight exceeds u * total, u being a 24-bit uniform in [0,1)
//   from a counter-based generator keyed by (seed, index of the token being drawn).
// A row's result depends on its own logits, seed and index only, so it is independent of
// what else is in the batch.
// The sampler's state (temperature, seed, index of the next token) comes either as arrays with
// an entry per row, or from the per-request slots of fixed size the cache manager keeps: four
// 64-bit words per slot (temperature as float bits, seed, index of the next token to draw,
// position of the last sampled token's input), which the kernel reads by the row's slot and
// advances itself, so a decode step brings no sampler state from the host. The reference models
// its sampler as (state, logits) -> (state', token) (src/boundary/sampler.rs:7-19).
#include "common.cuh"

namespace {
constexpr int THREADS = 1024;

__device__ __forceinline__ float uniform24(unsigned long long seed, unsigned long long index) {
  unsigned long long z = seed * 0x9E3779B97F4A7C15ull + (index + 1ull) * 0xBF58476D1CE4E5B9ull;
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, int64_t row_stride, const float* __restrict__ temperature,
              const long long* __restrict__ seeds, const long long* __restrict__ counters, const int* __restrict__ slots,
              long long* __restrict__ slot_table, int num_slots, const int* __restrict__ positions,
              int* __restrict__ out, unsigned* status) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ float s_scan[THREADS + 1];
  __shared__ int s_token;
  pdl_wait();
  pdl_launch_dependents();
  const float* row = logits + (int64_t)blockIdx.x * row_stride;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // the sampler state of this row: from its slot, or from the arrays
  long long* state = nullptr;
  float temp = temperature ? temperature[blockIdx.x] : 0.f;
  unsigned long long seed = seeds ? (unsigned long long)seeds[blockIdx.x] : 0ull;
  unsigned long long index = counters ? (unsigned long long)counters[blockIdx.x] : 0ull;
  if (slots != nullptr) {
    int slot = slots[blockIdx.x];
    if (slot < 0 || slot >= num_slots) {
      if (tid == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
      temp = 0.f;
    } else {
      state = slot_table + 4ll * slot;
      temp = __int_as_float((int)(state[0] & 0xffffffffll));
      seed = (unsigned long long)state[1];
      index = (unsigned long long)state[2];
    }
  }
  __syncthreads();                       // every thread has read the state before thread 0 advances it
  if (state != nullptr && tid == 0) {
    state[2] = (long long)(index + 1ull);
    if (positions != nullptr) state[3] = positions[blockIdx.x];
  }

  // ---- maximum and its lowest index (needed by both modes)
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  auto consider = [&](float v, int i) {
    if (v > best || (v == best && i < best_i)) {
      best = v;
      best_i = i;
    }
  };
  if ((row_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
    // 16-byte loads, four of them in flight per thread
    const int quads = vocab >> 2;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    for (int q0 = tid; q0 < quads; q0 += 4 * THREADS) {
      float4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (q0 + j * THREADS < quads) v[j] = row4[q0 + j * THREADS];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int q = q0 + j * THREADS;
        if (q < quads) {
          consider(v[j].x, 4 * q);
          consider(v[j].y, 4 * q + 1);
          consider(v[j].z, 4 * q + 2);
          consider(v[j].w, 4 * q + 3);
        }
      }
    }
    for (int i = 4 * quads + tid; i < vocab; i += THREADS) consider(row[i], i);
  } else {
    for (int i = tid; i < vocab; i += THREADS) consider(row[i], i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_i;
  }
  __syncthreads();
  best = s_val[0];
  best_i = s_idx[0];
  for (int w = 1; w < THREADS / 32; ++w) {
    if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) {
      best = s_val[w];
      best_i = s_idx[w];
    }
  }
  if (!(temp > 0.f)) {
    if (tid == 0) out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
    return;
  }

  // ---- temperature: contiguous chunk per thread, fixed-order scan
  const int chunk = (vocab + THREADS - 1) / THREADS;
  const int begin = min(tid * chunk, vocab), end = min(begin + chunk, vocab);
  const float inv_t = 1.f / temp;
  float local = 0.f;
  for (int i = begin; i < end; ++i) local += expf((row[i] - best) * inv_t);
  s_scan[tid + 1] = local;
  if (tid == 0) {
    s_scan[0] = 0.f;
    s_token = vocab - 1;
  }
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    for (int i = 1; i <= THREADS; ++i) {
      run += s_scan[i];
      s_scan[i] = run;
    }
  }
  __syncthreads();
  const float total = s_scan[THREADS];
  const float u = uniform24(seed, index);
  const float target = u * total;
  const float before = s_scan[tid];
  if (target >= before && target < s_scan[tid + 1]) {
    float run = 0.f;
    for (int i = begin; i < end; ++i) {
      run += expf((row[i] - best) * inv_t);
      if (before + run > target) {
        s_token = i;
        break;
      }
    }
  }
  __syncthreads();
  if (tid == 0) out[blockIdx.x] = s_token;
}
}  // namespace

// logits: float32 [rows, vocab] with `row_stride` elements between rows; temperature:
// float32[rows] or null (all greedy); seeds, counters: int64[rows] (may be null if all greedy).
VOSTI_API int vosti_sample(const float* logits, int rows, int vocab, int64_t row_stride, const float* temperature,
                           const long long* seeds, const long long* counters, int* out, cudaStream_t stream) {
  VOSTI_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
  VOSTI_REQUIRE(temperature == nullptr || (seeds != nullptr && counters != nullptr),
                "sample: temperature sampling needs seeds and counters");
  if (rows == 0) return VOSTI_OK;
  vosti_launch(sample_kernel, dim3(rows), dim3(THREADS), 0, stream, logits, vocab, row_stride, temperature, seeds,
               counters, (const int*)nullptr, (long long*)nullptr, 0, (const int*)nullptr, out, (unsigned*)nullptr);
  VOSTI_LAUNCH_CHECK();
}

// The same with the sampler state in per-request slots: slots int32[rows] names each row's slot,
// slot_table int64[num_slots][4] = (temperature as float bits, seed, index of the next token,
// position); the kernel advances the index and, if `positions` (int32[rows]) is given, writes the
// row's position. A slot outside the table sets a fault bit and the row is sampled greedily.
VOSTI_API int vosti_sample_slots(const float* logits, int rows, int vocab, int64_t row_stride, const int* slots,
                                 long long* slot_table, int num_slots, const int* positions, int* out,
                                 unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "sample_slots: bad sizes rows=%d vocab=%d", rows, vocab);
  VOSTI_REQUIRE(slots != nullptr && slot_table != nullptr && num_slots > 0, "sample_slots: the slots or their table are missing");
  if (rows == 0) return VOSTI_OK;
  vosti_launch(sample_kernel, dim3(rows), dim3(THREADS), 0, stream, logits, vocab, row_stride, (const float*)nullptr,
               (const long long*)nullptr, (const long long*)nullptr, slots, slot_table, num_slots, positions, out, status);
  VOSTI_LAUNCH_CHECK();
}

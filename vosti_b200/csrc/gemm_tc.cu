// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05), operands staged
// in shared memory by TMA, accumulator in tensor memory:
//   Y[t, f] = sum_k X[t, k] * W[f, k]          X: [T, K], W: [F, K] (both K-major), no bias
// Up to 128 tokens, output features fill the MMA's M = 128 (one accumulator lane per
// feature) and tokens are the N side (32..128 per tile), so a decode step of a few tokens
// still uses whole instructions; K is split for enough CTAs, by a rule of the sizes only,
// and the splits are summed in split order. For more tokens see gemm_tc_wide_kernel.
//
// One CTA computes one 128 x BN tile (one K split of it): warp 0 issues the TMA loads,
// warp 1 allocates tensor memory and issues the MMAs, warps 2..5 read the accumulator
// back (tcgen05.ld) and store. Every wait on an mbarrier is bounded: after about a second
// it sets the fault bit VOSTI_FAULT_WAIT_TIMEOUT, the CTA stops issuing work, frees its
// tensor memory and returns.
//
// The reference's matmul is a Triton kernel with float32 accumulation and no split-K
// (kernels/triton_kernels/matmul.py:95-147); its SiLU(gate)*up is a second kernel
// (silu_mul.py:66-87), fused here into the epilogue.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

namespace {

constexpr int BM = 128;           // features per tile (MMA M)
constexpr int BK = 64;            // k elements per stage: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int THREADS = 192;

enum Epilogue : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_PARTIAL = 3 };

// Instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = bn.
__host__ __device__ constexpr uint32_t instr_desc(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ float silu(float g) { return g / (1.f + __expf(-g)); }

// ------------------------------------------------------------------ the kernel
template <int BN, int STAGES, int KPS>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               void* __restrict__ out, int tokens, int features, int k_blocks, int ld_out, int epilogue,
               int w_tiles, int x_rows, unsigned* status) {
  // x_rows: rows of the token box map_x brings per k-block (the tokens rounded up to 8, at most BN):
  // with few tokens the rest of the tile is never fetched; what those rows of shared memory
  // hold only reaches output columns that are not stored.
  // w_tiles > 0: the weight is stored tile by tile ([k block][feature tile][128][64], w_tiles
  // feature tiles) and map_w sees it as a matrix of 64 columns; 0: row-major [features, k]
  // KPS: k-blocks per stage of the ring. The lane that issues the MMAs pays about 200 cycles for
  // the barrier wait that follows its own commit (even when the stage landed long before), 85
  // for the commit and 95 for the loop, beside 56 per MMA: with one k-block per stage that is
  // 610 cycles per k-block, with two 416. Launches with so few CTAs that each has an SM (and its
  // shared memory) to itself, whose time is k-blocks x that cost, take two k-blocks per stage.
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int BLOCK_BYTES = A_BYTES + B_BYTES;
  constexpr int STAGE_BYTES = KPS * BLOCK_BYTES;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128-byte swizzle pattern
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_base_holder;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int splits = gridDim.z, split = blockIdx.z;
  const int kb_begin = (int)((long long)k_blocks * split / splits);
  const int kb_end = (int)((long long)k_blocks * (split + 1) / splits);
  const int my_blocks = kb_end - kb_begin;
  const int my_stages = (my_blocks + KPS - 1) / KPS;       // the last one may hold fewer k-blocks

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&accum_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_holder), BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_holder;

  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // k-blocks of stage i: i * KPS .. i * KPS + held(i) - 1 (counted from kb_begin)
      auto held = [&](int i) { return my_blocks - i * KPS < KPS ? my_blocks - i * KPS : KPS; };
      auto load_w = [&](int i, int s) {
        const uint32_t bar = smem_u32(&full_bar[s]);
        mbar_expect_tx(bar, (uint32_t)(held(i) * (A_BYTES + x_rows * BK * 2)));
        for (int q = 0; q < held(i); ++q) {
          const int kb = kb_begin + i * KPS + q;           // k offsets are multiples of 64 elements: 16-byte aligned
          const uint32_t dst = smem_u32(smem + s * STAGE_BYTES + q * BLOCK_BYTES);
          if (w_tiles) tma_load_2d(dst, &map_w, 0, (kb * w_tiles + (int)blockIdx.x) * BM, bar);
          else tma_load_2d(dst, &map_w, kb * BK, m0, bar);
        }
      };
      auto load_x = [&](int i, int s) {
        for (int q = 0; q < held(i); ++q)
          tma_load_2d(smem_u32(smem + s * STAGE_BYTES + q * BLOCK_BYTES) + A_BYTES, &map_x, (kb_begin + i * KPS + q) * BK, n0,
                      smem_u32(&full_bar[s]));
      };
      // The weight tiles of the first stages do not depend on the kernel before this one:
      // they are requested at once, the token tiles after that kernel has completed.
      const int ahead = my_stages < STAGES ? my_stages : STAGES;
      for (int i = 0; i < ahead; ++i) load_w(i, i);
      pdl_wait();
      for (int i = 0; i < ahead; ++i) load_x(i, i);
      for (int i = ahead; i < my_stages; ++i) {
        const int s = i % STAGES;
        const uint32_t round = i / STAGES;
        if (!mbar_wait(smem_u32(&empty_bar[s]), (round - 1) & 1, &abort_flag, status)) break;
        load_w(i, s);
        load_x(i, s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BN);
      bool ok = true;
      for (int i = 0; i < my_stages && ok; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(smem_u32(&full_bar[s]), (i / STAGES) & 1, &abort_flag, status);
        if (!ok) break;
        tc_fence_after();
        const int held = my_blocks - i * KPS < KPS ? my_blocks - i * KPS : KPS;
#pragma unroll
        for (int q = 0; q < KPS; ++q) {
          if (q < held) {
            const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES + q * BLOCK_BYTES);
            const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // 16 elements further along K: 32 bytes, 2 in the descriptor's 16-byte units
              umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (i > 0 || q > 0 || k > 0) ? 1u : 0u);
            }
          }
        }
        umma_commit(smem_u32(&empty_bar[s]));     // the stage is free once these MMAs have read it
      }
      if (ok) umma_commit(smem_u32(&accum_bar));  // the accumulator is complete
    }
  } else {
    // epilogue: this warp may read the 32 accumulator lanes of its quarter only
    const int quarter = warp & 3;
    pdl_wait();                                       // the output may still be read by the kernel before
    bool ok = my_blocks > 0 ? mbar_wait_warp(smem_u32(&accum_bar), 0, &abort_flag, status) : true;
    tc_fence_after();
    const int feature = m0 + quarter * 32 + lane;
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (n0 + c0 >= tokens) break;                 // uniform across the warp
        uint32_t r[32];
        if (my_blocks > 0) {
          tmem_load32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (epilogue == EPI_SWIGLU) {
          // lanes 0..15 hold gate rows, lanes 16..31 the matching up rows
          bf16* y = reinterpret_cast<bf16*>(out);
          const int out_feature = (m0 + quarter * 32) / 2 + (lane & 15);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float mine = __uint_as_float(r[j]);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
            const int t = n0 + c0 + j;
            if (lane < 16 && t < tokens && out_feature < ld_out)
              y[(int64_t)t * ld_out + out_feature] = __float2bfloat16_rn(silu(mine) * other);
          }
        } else if (feature < features) {
          if (epilogue == EPI_BF16) {
            bf16* y = reinterpret_cast<bf16*>(out);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int t = n0 + c0 + j;
              if (t < tokens) y[(int64_t)t * ld_out + feature] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
          } else {  // EPI_F32, or EPI_PARTIAL into this split's slice
            float* y = reinterpret_cast<float*>(out) + (epilogue == EPI_PARTIAL ? (int64_t)split * tokens * ld_out : 0);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int t = n0 + c0 + j;
              if (t < tokens) y[(int64_t)t * ld_out + feature] = __uint_as_float(r[j]);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    // leave time for copies that are still in flight to land before the CTA's memory goes away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, BN);
  }
}


// One token's 32 consecutive accumulator columns (features f0 .. f0 + 31) through the epilogue
// into the output: bf16, float32, or SiLU(gate) * up of 16 gate and 16 up columns.
__device__ __forceinline__ void store_token_columns(const uint32_t (&r)[32], void* __restrict__ out, int token, int f0,
                                                    int features, int ld_out, int epilogue) {
  if (epilogue == EPI_SWIGLU) {
    // columns f0..f0+15 are gate rows, f0+16..f0+31 their up rows (features % 32 == 0)
    bf16* y = reinterpret_cast<bf16*>(out) + (int64_t)token * ld_out + f0 / 2;
    uint32_t packed[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = silu(__uint_as_float(r[2 * j])) * __uint_as_float(r[16 + 2 * j]);
      const float b = silu(__uint_as_float(r[2 * j + 1])) * __uint_as_float(r[17 + 2 * j]);
      __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
      packed[j] = *reinterpret_cast<uint32_t*>(&v);
    }
    if ((ld_out & 7) == 0) {
      reinterpret_cast<uint4*>(y)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      reinterpret_cast<uint4*>(y)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) reinterpret_cast<uint32_t*>(y)[j] = packed[j];   // ld_out is even
    }
  } else if (epilogue == EPI_BF16) {
    bf16* y = reinterpret_cast<bf16*>(out) + (int64_t)token * ld_out + f0;
    if (f0 + 32 <= features && (ld_out & 7) == 0) {
#pragma unroll
      for (int v4 = 0; v4 < 4; ++v4) {
        uint32_t p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[8 * v4 + 2 * j]), __uint_as_float(r[8 * v4 + 2 * j + 1]));
          p[j] = *reinterpret_cast<uint32_t*>(&v);
        }
        reinterpret_cast<uint4*>(y)[v4] = make_uint4(p[0], p[1], p[2], p[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (f0 + j < features) y[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
    }
  } else {  // EPI_F32
    float* y = reinterpret_cast<float*>(out) + (int64_t)token * ld_out + f0;
    if (f0 + 32 <= features && (ld_out & 3) == 0) {
#pragma unroll
      for (int v4 = 0; v4 < 8; ++v4)
        reinterpret_cast<uint4*>(y)[v4] = make_uint4(r[4 * v4], r[4 * v4 + 1], r[4 * v4 + 2], r[4 * v4 + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (f0 + j < features) y[j] = __uint_as_float(r[j]);
    }
  }
}

// ------------------------------------------------------------------ the kernel for many tokens
// For more than 128 tokens the roles are swapped: 128 tokens fill the MMA's M (one
// accumulator lane per token) and 256 features are the N side, so that a thread of the
// epilogue holds consecutive features of one token and stores them as 16-byte vectors, and
// the gate and up halves of a fused SiLU*up block sit in one thread. The kernel is
// persistent (one CTA per SM walks over tiles) with two accumulators in tensor memory, so
// the epilogue of a tile runs while the next tile's MMAs are issued.
constexpr int WIDE_BN = 256;
constexpr int WIDE_STAGES = 4;
constexpr int WIDE_B_BYTES = WIDE_BN * BK * 2;
constexpr int WIDE_STAGE_BYTES = A_BYTES + WIDE_B_BYTES;

__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_wide_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ out, int tokens, int features, int k_blocks, int ld_out, int epilogue,
                    int w_tiles, unsigned* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[WIDE_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[WIDE_STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_holder;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (tokens + BM - 1) / BM, n_tiles = (features + WIDE_BN - 1) / WIDE_BN;
  const int total_tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < WIDE_STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), 4);       // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_holder), 2 * WIDE_BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_holder;

  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      pdl_wait();
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * WIDE_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % WIDE_STAGES;
          const uint32_t round = it / WIDE_STAGES;
          if (it >= WIDE_STAGES && !mbar_wait(smem_u32(&empty_bar[s]), (round - 1) & 1, &abort_flag, status)) {
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&full_bar[s]);
          mbar_expect_tx(bar, WIDE_STAGE_BYTES);
          const uint32_t a_dst = smem_u32(smem + s * WIDE_STAGE_BYTES);
          tma_load_2d(a_dst, &map_x, kb * BK, m0, bar);
          if (w_tiles) tma_load_2d(a_dst + A_BYTES, &map_w, 0, (kb * w_tiles + n0 / BM) * BM, bar);
          else tma_load_2d(a_dst + A_BYTES, &map_w, kb * BK, n0, bar);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(WIDE_BN);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
        const uint32_t as = local & 1, acc_round = local >> 1;
        if (local >= 2) ok = mbar_wait(smem_u32(&acc_empty[as]), (acc_round - 1) & 1, &abort_flag, status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * WIDE_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % WIDE_STAGES;
          ok = mbar_wait(smem_u32(&full_bar[s]), (it / WIDE_STAGES) & 1, &abort_flag, status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * WIDE_STAGE_BYTES);
          const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(smem_u32(&empty_bar[s]));
        }
        if (ok) umma_commit(smem_u32(&acc_full[as]));
      }
    }
  } else {
    const int quarter = warp & 3;
    uint32_t local = 0;
    bool ok = true;
    pdl_wait();
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
      const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * WIDE_BN;
      const uint32_t as = local & 1;
      ok = mbar_wait_warp(smem_u32(&acc_full[as]), (local >> 1) & 1, &abort_flag, status);
      if (!ok) break;
      tc_fence_after();
      const int token = m0 + quarter * 32 + lane;
      const bool row_ok = token < tokens;
#pragma unroll 1
      for (int c0 = 0; c0 < WIDE_BN; c0 += 32) {
        const int f0 = n0 + c0;
        if (f0 >= features) break;
        uint32_t r[32];
        tmem_load32(tmem_base + as * WIDE_BN + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
        if (!row_ok) continue;
        store_token_columns(r, out, token, f0, features, ld_out, epilogue);
      }
      // this warp is done reading the accumulator: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[as]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * WIDE_BN);
  }
}

#include "gemm_tc_pair.cuh"

// Sum the K splits in split order and apply the epilogue.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ out, int splits,
                                     int tokens, int features, int ld_out, int epilogue) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t plane = (int64_t)tokens * features;
  if (epilogue == EPI_SWIGLU) {
    const int64_t n = (int64_t)tokens * (features / 2);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
      const int64_t t = i / (features / 2);
      const int f = (int)(i % (features / 2));
      const int row_g = (f / 16) * 32 + (f % 16), row_u = row_g + 16;
      float g = 0.f, u = 0.f;
      for (int s = 0; s < splits; ++s) {
        g += partial[s * plane + t * features + row_g];
        u += partial[s * plane + t * features + row_u];
      }
      reinterpret_cast<bf16*>(out)[t * ld_out + f] = __float2bfloat16_rn(silu(g) * u);
    }
    return;
  }
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < plane; i += (int64_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[s * plane + i];
    const int64_t t = i / features;
    const int f = (int)(i % features);
    if (epilogue == EPI_F32)
      reinterpret_cast<float*>(out)[t * ld_out + f] = acc;
    else
      reinterpret_cast<bf16*>(out)[t * ld_out + f] = __float2bfloat16_rn(acc);
  }
}

// ------------------------------------------------------------------ host side
// Map of a row-major [rows, k] bfloat16 matrix, box [box_rows, 64], 128-byte swizzle; what
// lies outside the matrix reads as zero.
bool make_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows) {
  return encode_tensor_map_2d(map, base, rows, k, box_rows, BK);
}

struct WeightKey {
  const void* p;
  int rows, k, box;
  bool operator==(const WeightKey& o) const { return p == o.p && rows == o.rows && k == o.k && box == o.box; }
};
struct WeightKeyHash {
  size_t operator()(const WeightKey& key) const {
    return std::hash<const void*>()(key.p) ^ ((size_t)key.rows * 1000003u) ^ ((size_t)key.k << 20) ^ (size_t)key.box;
  }
};

bool weight_map(const void* w, int rows, int k, int box_rows, CUtensorMap* out) {
  static std::unordered_map<WeightKey, CUtensorMap, WeightKeyHash> cache;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  WeightKey key{w, rows, k, box_rows};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  if (cache.size() > 4096) cache.clear();
  if (!make_map(out, w, rows, k, box_rows)) return false;
  cache.emplace(key, *out);
  return true;
}

int token_tile(int tokens) { return tokens <= 32 ? 32 : tokens <= 64 ? 64 : tokens <= 128 ? 128 : 256; }

template <int BN, int STAGES, int KPS = 1>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int tokens, int features, int k_blocks, int ld_out,
           int epilogue, int splits, int w_tiles, int x_rows, unsigned* status, cudaStream_t stream) {
  constexpr size_t smem = (size_t)STAGES * KPS * (A_BYTES + BN * BK * 2) + 1024;
  static_assert(smem <= 232448, "the ring does not fit an SM's shared memory");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, KPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      vosti_set_error("gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return (int)e;
    }
    configured = true;
  }
  dim3 grid((features + BM - 1) / BM, (tokens + BN - 1) / BN, splits);
  vosti_launch(gemm_tc_kernel<BN, STAGES, KPS>, grid, dim3(THREADS), smem, stream, mw, mx, out, tokens, features, k_blocks, ld_out,
               epilogue, w_tiles, x_rows, status);
  return 0;
}

}  // namespace

// Whether the tensor-core product takes a [features, k] bfloat16 weight at all.
VOSTI_API int vosti_gemm_tc_supported(int features, int k) { return features >= 1 && k >= BK && k % 8 == 0; }

// How many K splits a product of these sizes uses (a function of the sizes only; the
// sum over splits is taken in split order). With one order of arithmetic asked for
// (vosti_set_fixed_order) no product is split: the unsplit kernels give a token the same bits
// whichever of them runs, the split ones do not. More than one split needs a float32 workspace
// of splits * tokens * features elements.
VOSTI_API int vosti_gemm_tc_splits(int tokens, int features, int k) {
  const int k_blocks = (k + BK - 1) / BK;
  const int tiles = ((features + BM - 1) / BM) * ((tokens + token_tile(tokens) - 1) / token_tile(tokens));
  if (tokens > 128 || g_vosti_fixed_order) return 1;
  int splits;
  if (token_tile(tokens) <= 64) {
    // two CTAs of this tile size fit an SM: fill both slots of every SM, never a second round
    splits = (2 * 148) / tiles;
    if (splits > k_blocks / 4) splits = k_blocks / 4;   // at least 4 k-blocks (256 elements) per split
  } else {
    if (tiles >= 96) return 1;
    splits = (148 + tiles - 1) / tiles;
    if (splits > k_blocks / 8) splits = k_blocks / 8;
  }
  if (splits > 16) splits = 16;
  return splits < 1 ? 1 : splits;
}

// x: [tokens, k] bf16; w: [features, k] bf16; epilogue 0: y bf16 [tokens, features];
// 1: y float32 [tokens, features]; 2: y bf16 [tokens, features / 2] = silu(gate) * up with
// the weight rows interleaved in blocks of 16 gate rows and their 16 up rows.
// With `defer_reduce` and more than one split the partial sums stay in the workspace
// ([splits, tokens, features] float32) for a consumer that sums them itself; y is not written.
VOSTI_API int vosti_gemm_tc(const void* x, const void* w, void* y, int tokens, int features, int k, int epilogue,
                            float* workspace, int64_t workspace_elems, int defer_reduce, int w_packed, unsigned* status,
                            cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && vosti_gemm_tc_supported(features, k), "gemm_tc: unsupported sizes F=%d K=%d", features, k);
  VOSTI_REQUIRE(epilogue >= EPI_BF16 && epilogue <= EPI_SWIGLU, "gemm_tc: unknown epilogue %d", epilogue);
  VOSTI_REQUIRE(epilogue != EPI_SWIGLU || features % 32 == 0, "gemm_tc: fused SiLU*up needs features %% 32 == 0");
  VOSTI_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_tc: operands must be 16-byte aligned");
  if (tokens == 0) return VOSTI_OK;
  const int ld_out = epilogue == EPI_SWIGLU ? features / 2 : features;
  const int k_blocks = (k + BK - 1) / BK;
  const int splits = vosti_gemm_tc_splits(tokens, features, k);
  VOSTI_REQUIRE(splits == 1 || (workspace != nullptr && workspace_elems >= (int64_t)splits * tokens * features),
                "gemm_tc: workspace too small for %d splits", splits);
  CUtensorMap mw_storage, mx;
  const CUtensorMap* mw = &mw_storage;
  // a packed weight is [k blocks][feature tiles][128][64], zero-padded to whole tiles: its
  // tensor map is that of a matrix of 64 columns
  const int w_tiles = w_packed ? (features + BM - 1) / BM : 0;
  const int w_rows = w_packed ? k_blocks * w_tiles * BM : features, w_cols = w_packed ? BK : k;
  static const bool use_pairs = [] {                 // VOSTI_GEMM_PAIR=0: the single-CTA kernel below instead
    const char* env = getenv("VOSTI_GEMM_PAIR");
    return env == nullptr || env[0] != '0';
  }();
  if (tokens > 128 && use_pairs) {
    // many tokens, two SMs per tile (cta_group::2)
    using namespace pair_kernel;
    VOSTI_REQUIRE(weight_map(w, w_rows, w_cols, BM, &mw_storage) && make_map(&mx, x, tokens, k, BM),
                  "gemm_tc: cuTensorMapEncodeTiled failed");
    constexpr size_t smem = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 1024;
    static int pair_sms = 0;
    if (pair_sms == 0) {
      int device = 0;
      cudaGetDevice(&device);
      cudaDeviceGetAttribute(&pair_sms, cudaDevAttrMultiProcessorCount, device);
      cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess || pair_sms <= 1) {
        pair_sms = 0;
        vosti_set_error("gemm_tc: cannot configure the paired kernel: %s", cudaGetErrorString(e));
        return e != cudaSuccess ? (int)e : VOSTI_UNSUPPORTED;
      }
    }
    const int tiles = ((tokens + 2 * BM - 1) / (2 * BM)) * ((features + PAIR_BN - 1) / PAIR_BN);
    const int pairs = tiles < pair_sms / 2 ? tiles : pair_sms / 2;
    vosti_launch_clusters(gemm_tc_pair_kernel, dim3(2 * pairs), dim3(PAIR_THREADS), 2, smem, stream, mx, *mw, y, tokens,
                          features, k_blocks, ld_out, epilogue, w_tiles, status);
    VOSTI_LAUNCH_CHECK();
  }
  if (tokens > 128) {
    // many tokens: persistent kernel with tokens on the M side
    VOSTI_REQUIRE(weight_map(w, w_rows, w_cols, WIDE_BN, &mw_storage) && make_map(&mx, x, tokens, k, BM),
                  "gemm_tc: cuTensorMapEncodeTiled failed");
    constexpr size_t smem = (size_t)WIDE_STAGES * WIDE_STAGE_BYTES + 1024;
    static int sms = 0;
    if (sms == 0) {
      int device = 0;
      cudaGetDevice(&device);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
      cudaError_t e = cudaFuncSetAttribute(gemm_tc_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess || sms <= 0) {
        sms = 0;
        vosti_set_error("gemm_tc: cannot configure the persistent kernel: %s", cudaGetErrorString(e));
        return e != cudaSuccess ? (int)e : VOSTI_UNSUPPORTED;
      }
    }
    const int tiles = ((tokens + BM - 1) / BM) * ((features + WIDE_BN - 1) / WIDE_BN);
    vosti_launch(gemm_tc_wide_kernel, dim3(tiles < sms ? tiles : sms), dim3(THREADS), smem, stream, mx, *mw, y, tokens,
                 features, k_blocks, ld_out, epilogue, w_tiles, status);
    VOSTI_LAUNCH_CHECK();
  }
  const int bn = token_tile(tokens);
  const int x_rows = (tokens + 7) / 8 * 8 < bn ? (tokens + 7) / 8 * 8 : bn;   // the token box: no more rows than needed
  VOSTI_REQUIRE(weight_map(w, w_rows, w_cols, BM, &mw_storage) && make_map(&mx, x, tokens, k, x_rows),
                "gemm_tc: cuTensorMapEncodeTiled failed");
  void* dst = splits > 1 ? (void*)workspace : y;
  const int epi = splits > 1 ? EPI_PARTIAL : epilogue;
  const int ld = splits > 1 ? features : ld_out;
  // no more CTAs than SMs: each has an SM's shared memory to itself and takes two k-blocks per stage
  const int64_t ctas = (int64_t)((features + BM - 1) / BM) * ((tokens + bn - 1) / bn) * splits;
  const bool lone = ctas <= 148;
#define VOSTI_GEMM_ARGS *mw, mx, dst, tokens, features, k_blocks, ld, epi, splits, w_tiles, x_rows, status, stream
  int rc;
  switch (bn) {
    case 32: rc = lone ? launch<32, 5, 2>(VOSTI_GEMM_ARGS) : launch<32, 5>(VOSTI_GEMM_ARGS); break;
    case 64: rc = lone ? launch<64, 4, 2>(VOSTI_GEMM_ARGS) : launch<64, 4>(VOSTI_GEMM_ARGS); break;
    case 128: rc = lone ? launch<128, 3, 2>(VOSTI_GEMM_ARGS) : launch<128, 6>(VOSTI_GEMM_ARGS); break;
    default: rc = launch<256, 4>(VOSTI_GEMM_ARGS); break;
  }
#undef VOSTI_GEMM_ARGS
  if (rc != 0) return rc;
  if (splits > 1 && !defer_reduce) {
    const int64_t n = (int64_t)tokens * features;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    vosti_launch(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, (const float*)workspace, y, splits, tokens,
                 features, ld_out, epilogue);
  }
  VOSTI_LAUNCH_CHECK();
}

// Sum deferred partial sums ([splits, tokens, features] float32) in split order into y
// (bf16 or float32 [tokens, features]).
VOSTI_API int vosti_splitk_reduce(const float* partial, void* y, int splits, int tokens, int features, int y_is_f32,
                                  cudaStream_t stream) {
  VOSTI_REQUIRE(splits >= 1 && tokens >= 0 && features >= 1, "splitk_reduce: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  const int64_t n = (int64_t)tokens * features;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  vosti_launch(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, partial, y, splits, tokens, features, features,
               (int)(y_is_f32 ? EPI_F32 : EPI_BF16));
  VOSTI_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ no-allocation entry point
// See no_alloc.h. The scratch of the K splits is this array instead of a caller's buffer.
#include "no_alloc.h"

static __device__ __align__(256) float g_static_scratch[VOSTI_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_static_scratch_address[MAX_DEVICES] = {};   // device address of the array, per device

// In host code the array's name is only a handle for the runtime, not an address a kernel
// can use; the device address comes from cudaGetSymbolAddress, per device.
int static_scratch(float** out) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= MAX_DEVICES) {
    vosti_set_error("gemm_tc_split_static: no usable current device (%s)", cudaGetErrorString(e));
    return e != cudaSuccess ? (int)e : VOSTI_UNSUPPORTED;
  }
  if (g_static_scratch_address[device] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      vosti_set_error("gemm_tc_split_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : VOSTI_UNSUPPORTED;
    }
    g_static_scratch_address[device] = p;
  }
  *out = g_static_scratch_address[device];
  return VOSTI_OK;
}
}  // namespace

VOSTI_API int vosti_gemm_tc_split_static(const void* x, const void* w, void* y, int tokens, int features, int k,
                                         int y_is_f32, unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(x != nullptr && w != nullptr && y != nullptr, "gemm_tc_split_static: null operand");
  VOSTI_REQUIRE(tokens >= 1 && tokens <= 128, "gemm_tc_split_static: tokens must be 1..128, got %d", tokens);
  VOSTI_REQUIRE(vosti_gemm_tc_supported(features, k), "gemm_tc_split_static: unsupported sizes F=%d K=%d", features, k);
  VOSTI_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_tc_split_static: operands must be 16-byte aligned");
  const int splits = vosti_gemm_tc_splits(tokens, features, k);
  const int64_t need = splits > 1 ? (int64_t)splits * tokens * features : 0;
  VOSTI_REQUIRE(need <= (int64_t)VOSTI_STATIC_SCRATCH_FLOATS,
                "gemm_tc_split_static: %d splits x %d tokens x %d features need %lld scratch floats, the static array "
                "holds %d", splits, tokens, features, (long long)need, VOSTI_STATIC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  const int rc_scratch = static_scratch(&scratch);
  if (rc_scratch != VOSTI_OK) return rc_scratch;
  const int epilogue = y_is_f32 ? EPI_F32 : EPI_BF16;
  const int k_blocks = (k + BK - 1) / BK;
  const int bn = token_tile(tokens);
  CUtensorMap mw, mx;                       // encoded on the stack: no cache, nothing allocated
  VOSTI_REQUIRE(make_map(&mw, w, features, k, BM) && make_map(&mx, x, tokens, k, bn),
                "gemm_tc_split_static: cuTensorMapEncodeTiled failed");
  void* dst = splits > 1 ? (void*)scratch : y;
  const int epi = splits > 1 ? EPI_PARTIAL : epilogue;
  int rc;
  switch (bn) {
    case 32: rc = launch<32, 5>(mw, mx, dst, tokens, features, k_blocks, features, epi, splits, 0, bn, status, stream); break;
    case 64: rc = launch<64, 4>(mw, mx, dst, tokens, features, k_blocks, features, epi, splits, 0, bn, status, stream); break;
    default: rc = launch<128, 6>(mw, mx, dst, tokens, features, k_blocks, features, epi, splits, 0, bn, status, stream); break;
  }
  if (rc != 0) return rc;
  if (splits > 1) {
    const int64_t n = (int64_t)tokens * features;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    vosti_launch(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, (const float*)scratch, y, splits, tokens,
                 features, features, epilogue);
  }
  VOSTI_LAUNCH_CHECK();
}

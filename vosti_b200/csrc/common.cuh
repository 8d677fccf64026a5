// Shared helpers of the sm_100a kernels: element types, conversions, fixed-order
// reductions and the device status word.
//
// Every reduction here has an order that depends only on the reduced extent and the
// block size, never on how many rows the launch carries, so a row's result does not
// depend on its batch companions (the reference states the same rule for its Triton
// kernels: tile choice from model geometry only, docs/deployment.md:44-46).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define VOSTI_API extern "C" __attribute__((visibility("default")))

// Codes a launcher returns (besides cudaError_t values, which are positive).
enum VostiStatus : int {
  VOSTI_OK = 0,
  VOSTI_BAD_ARGUMENT = -1,    // a size the kernel refuses (message via vosti_last_error)
  VOSTI_UNSUPPORTED = -2,
};

// Bits a kernel may set in the device status word (read by the host after a step).
enum VostiDeviceFault : unsigned {
  VOSTI_FAULT_TOKEN_RANGE = 1u << 0,     // token id outside the vocabulary
  VOSTI_FAULT_SLOT_RANGE = 1u << 1,      // cache slot outside the pool
  VOSTI_FAULT_PAGE_RANGE = 1u << 2,      // block-table entry outside the pool
  VOSTI_FAULT_POSITION_RANGE = 1u << 3,  // position beyond the rotation table
  VOSTI_FAULT_WAIT_TIMEOUT = 1u << 4,    // a bounded wait gave up
  VOSTI_FAULT_ROW_RANGE = 1u << 5,       // gathered row index outside the input
};

void vosti_set_error(const char* fmt, ...);
extern int g_vosti_fixed_order;   // errors.cu: one order of arithmetic however the work is cut

#define VOSTI_REQUIRE(cond, ...)            \
  do {                                      \
    if (!(cond)) {                          \
      vosti_set_error(__VA_ARGS__);         \
      return VOSTI_BAD_ARGUMENT;            \
    }                                       \
  } while (0)

#define VOSTI_LAUNCH_CHECK()                          \
  do {                                                \
    cudaError_t e__ = cudaGetLastError();             \
    if (e__ != cudaSuccess) {                         \
      vosti_set_error("%s", cudaGetErrorString(e__)); \
      return (int)e__;                                \
    }                                                 \
    return VOSTI_OK;                                  \
  } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Load element i of an array whose element type is chosen at run time
// (is_f32 != 0: float, else bf16). Used for small tensors such as norm weights,
// which stay 32-bit when the checkpoint stores them so.
__device__ __forceinline__ float load_flex(const void* p, int is_f32, int64_t i) {
  return is_f32 ? reinterpret_cast<const float*>(p)[i]
                : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed tree: xor-shuffle inside each warp, then the warp
// totals are added in warp order by every thread. `scratch` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += scratch[w];
  return total;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = -INFINITY;
  for (int w = 0; w < nwarps; ++w) total = fmaxf(total, scratch[w]);
  return total;
}

__device__ __forceinline__ void raise_fault(unsigned* status, unsigned bit) {
  if (status) atomicOr(status, bit);
}

// ---------------------------------------------------------------- dependent launches
// Kernels of the serving path are launched with programmatic stream serialization: a
// kernel may be scheduled while its predecessor in the stream is still running, runs
// whatever does not depend on the predecessor (set-up, and for the products the first
// weight tiles), and calls pdl_wait() before it touches anything the predecessor wrote or
// still reads. pdl_wait() returns once the predecessor grid has completed and its memory
// operations are visible; without the launch attribute it returns at once. Every kernel
// launched through vosti_launch must call pdl_wait() on every path before its first access
// to global memory that another kernel writes.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

int vosti_pdl_enabled();

// ---------------------------------------------------------------- weights requested ahead
// A decode step alternates between products that stream weights from HBM and short kernels
// (norms) during which HBM has little to do. The host may name the weight range the next product
// will stream (vosti_hint_prefetch); the launcher of such a short kernel takes the hint and lets
// blocks added to the launch ask for that range
// to be brought into L2 (cp.async.bulk.prefetch.L2: no destination, no completion to wait for),
// so that the product finds the start of its weights on the chip. Values never change by it.
struct VostiPrefetch {
  const char* ptr;       // 16-byte aligned, or null: nothing to ask for
  long long bytes;       // a multiple of 16
};
VostiPrefetch vosti_take_prefetch();     // the pending hint, which is cleared (errors.cu)
constexpr long long PREFETCH_PIECE = 16384;

// Worker `worker` of `workers` requests its share of the range, one piece per instruction.
__device__ __forceinline__ void l2_prefetch_share(VostiPrefetch p, long long worker, long long workers) {
  if (p.ptr == nullptr) return;
  const long long pieces = (p.bytes + PREFETCH_PIECE - 1) / PREFETCH_PIECE;
  for (long long i = worker; i < pieces; i += workers) {
    const long long at = i * PREFETCH_PIECE;
    const unsigned size = (unsigned)(p.bytes - at < PREFETCH_PIECE ? p.bytes - at : PREFETCH_PIECE);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.ptr + at), "r"(size) : "memory");
  }
}

template <typename... KArgs, typename... Args>
inline cudaError_t vosti_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = vosti_pdl_enabled() ? 1 : 0;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

// The same with thread-block clusters of `cluster` CTAs along x (the grid's x must be a multiple).
template <typename... KArgs, typename... Args>
inline cudaError_t vosti_launch_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned cluster, size_t smem,
                                         cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = vosti_pdl_enabled() ? 1 : 0;
  attribute[1].id = cudaLaunchAttributeClusterDimension;
  attribute[1].val.clusterDim.x = cluster;
  attribute[1].val.clusterDim.y = 1;
  attribute[1].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 2;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

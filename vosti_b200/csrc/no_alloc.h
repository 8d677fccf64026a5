// An entry point of the kernel library that allocates nothing.
//
// It has no counterpart in the reference project; it exists for callers of this library
// that cannot allocate device memory at the time of the call: a serving process that has
// handed every free byte of the GPU to its cache pool at start-up (a later cudaMalloc
// fails), or a host program whose device memory is owned by another allocator and that
// must not see this library reserve memory behind its back.
//
// vosti_gemm_tc_split_static computes y = x @ w^T for up to 128 tokens with the split-K
// tensor-core kernel of gemm_tc.cu. The caller passes inputs and outputs; the float32
// partial sums of the K splits, which vosti_gemm_tc takes as a caller-provided workspace,
// live in a file-scope device array of VOSTI_STATIC_SCRATCH_FLOATS floats (8 MiB) that
// every GPU loading the library holds until the process exits.
//
//  * Sizes: 1 <= tokens <= 128, and splits * tokens * features <= VOSTI_STATIC_SCRATCH_FLOATS
//    (splits = vosti_gemm_tc_splits(tokens, features, k)); anything else is refused with
//    VOSTI_BAD_ARGUMENT and a message in vosti_last_error().
//  * It calls no cudaMalloc, cudaFree or allocating library routine.
//  * The first call on a device is a set-up call: it looks up the array's device address (once
//    per device, with that device current) and raises the kernel's shared-memory limit; under
//    CUDA's default lazy module loading it is also the moment the driver places the kernel's
//    code and the 8 MiB array in device memory. The kernel exists in three widths of token
//    tile (1..32, 33..64 and 65..128 tokens), each loaded at its first use. So make one warm-up
//    call per device for each of those ranges you will use, while device memory is still
//    available, before the process hands its free memory away and before any stream capture
//    begins; every later call changes the amount of free device memory by nothing. Two threads making the first call on one device at once both
//    store the same address, which is harmless.
//  * All calls share the one array and it keeps the last call's contents. Nothing has to
//    start at zero: every partial sum the reduction reads is written by the same call. Two
//    calls that overlap on the GPU (different streams without ordering between them) race
//    on the array; order them on one stream or with events.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define VOSTI_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// x: bf16 [tokens, k]; w: bf16 [features, k]; y: bf16 or float32 [tokens, features];
// status: device word for fault bits, may be null. Returns 0, a negative VostiStatus, or a
// positive cudaError_t.
int vosti_gemm_tc_split_static(const void* x, const void* w, void* y, int tokens, int features, int k,
                               int y_is_f32, unsigned* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

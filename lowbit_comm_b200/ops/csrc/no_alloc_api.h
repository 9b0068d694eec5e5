// Allocation-free entry point.  THIS HAS NO COUNTERPART IN THE REFERENCE
// LIBRARY: it exists for callers of this library that are not allowed to
// allocate device memory at the point where they need the codec — code running
// inside a region where cudaMalloc/cudaFree are illegal or would serialise the
// device (CUDA-graph capture set-up paths, real-time inference loops, plugins
// that live inside another framework's allocator and must not touch the driver
// allocator), and plain C or ctypes callers that have no tensor library to
// allocate the intermediate payload for them.
//
// lbc_no_alloc_roundtrip does what one data-parallel rank does to a gradient
// bucket when it is alone (world size 1): error-feedback add, int8/int4 group
// quantization, decode, residual update.  The quantized payload between the two
// kernels normally lives in a caller- or framework-allocated buffer; here it
// lives in a fixed array inside the library image.
//
// What a caller must know:
//  * Limit: at most LBC_NO_ALLOC_MAX_NUMEL elements per call.  Larger inputs are
//    rejected with LBC_NO_ALLOC_TOO_LARGE; split them into group-aligned pieces.
//  * Cost: every GPU that loads the library holds LBC_NO_ALLOC_SCRATCH_BYTES of
//    device memory for this array until the process exits, used or not.
//  * First call per device: looks up the device address of the array (one
//    cudaGetSymbolAddress, with that device current).  Make the first call on a
//    device before any stream capture begins on it.
//  * The array is shared by every call on a device and keeps the previous
//    call's payload.  Each call overwrites every byte it later reads, so nothing
//    needs clearing; but two calls that can overlap on the GPU (different streams
//    without an ordering between them) race on it.  Serialise them.
//  * The call allocates nothing: no cudaMalloc/cudaFree, no allocating library
//    routine.  Inputs and outputs are the caller's.
//  * Aliasing: residual_in and residual_out may be one buffer, and out may be x.
//    But x is read through the non-coherent path (ld.global.nc) while
//    residual_out is being written, so x must not overlap residual_out (nor
//    residual_in): keep the input and the residual in separate buffers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LBC_NO_ALLOC_MAX_NUMEL (4ll * 1024 * 1024)
// worst case payload: fp32 source, groups of 16, int8 -> (16 + 4) bytes per 16 elements
#define LBC_NO_ALLOC_SCRATCH_BYTES (LBC_NO_ALLOC_MAX_NUMEL / 16 * 20)

enum {
    LBC_NO_ALLOC_OK = 0,
    LBC_NO_ALLOC_BAD_ARGUMENT = -1,
    LBC_NO_ALLOC_TOO_LARGE = -2,
    LBC_NO_ALLOC_SETUP_FAILED = -3,
    LBC_NO_ALLOC_LAUNCH_FAILED = -4,
};

// dtype: 0 fp16, 1 bf16, 2 fp32 (LbcDType); group_size 16/32/64; bit 8 or 4.
// x, out: numel elements.  residual_in / residual_out: both NULL (no error
// feedback) or both given (they may be the same buffer):
//   prepared     = T(x + residual_in)
//   out          = decode(encode(prepared))
//   residual_out = T(prepared - decoded value before rounding)
// Work is enqueued on `stream`; nothing is synchronised.  Returns one of the codes
// above; lbc_no_alloc_error_string explains them, including the CUDA error seen.
int lbc_no_alloc_roundtrip(int dtype, int group_size, int bit, const void* x, const void* residual_in, void* out,
                           void* residual_out, long long numel, cudaStream_t stream);

const char* lbc_no_alloc_error_string(int code);
long long lbc_no_alloc_max_numel(void);
long long lbc_no_alloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif

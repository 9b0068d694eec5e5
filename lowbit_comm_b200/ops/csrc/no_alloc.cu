// Allocation-free round trip (see no_alloc_api.h for the contract).  The payload
// scratch is a file-scope device array; host code must not pass the array's name
// to a kernel (on the host that name is a stand-in, not a device address), so the
// device address is fetched once per device with cudaGetSymbolAddress and cached.
#include "no_alloc_api.h"

#include <mutex>

#include "lbc_api.h"

namespace {

constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_payload_scratch[LBC_NO_ALLOC_SCRATCH_BYTES];

// The planar payload of `numel` elements is groups * (G * BIT / 8) code bytes followed by groups * sizeof(T)
// scale bytes, with no padding in between.  The array must hold it for every profile the entry point serves;
// a layout change that adds bytes (padding between the two regions, wider scales) has to show up here.
constexpr long long payload_bytes(long long numel, int group, int bit, int scale_bytes) {
    return (numel + group - 1) / group * (group * bit / 8 + scale_bytes);
}
constexpr bool scratch_holds_every_profile() {
    for (int group : {16, 32, 64})
        for (int bit : {4, 8})
            for (int scale_bytes : {2, 4})
                if (payload_bytes(LBC_NO_ALLOC_MAX_NUMEL, group, bit, scale_bytes) > LBC_NO_ALLOC_SCRATCH_BYTES)
                    return false;
    return true;
}
static_assert(scratch_holds_every_profile(), "LBC_NO_ALLOC_SCRATCH_BYTES is too small for a served profile");
static_assert(payload_bytes(LBC_NO_ALLOC_MAX_NUMEL, 16, 8, 4) == LBC_NO_ALLOC_SCRATCH_BYTES,
              "the stated worst case (fp32 source, groups of 16, 8 bit) should fill the array exactly");

std::mutex g_setup_mutex;
unsigned char* g_scratch_address[kMaxDevices] = {};
thread_local cudaError_t t_last_cuda_error = cudaSuccess;

// Device address of the scratch array on the current device; nullptr on failure.
unsigned char* scratch_for_current_device() {
    int device = -1;
    t_last_cuda_error = cudaGetDevice(&device);
    if (t_last_cuda_error != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> guard(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* address = nullptr;
        t_last_cuda_error = cudaGetSymbolAddress(&address, g_payload_scratch);
        if (t_last_cuda_error != cudaSuccess) return nullptr;
        g_scratch_address[device] = static_cast<unsigned char*>(address);
    }
    return g_scratch_address[device];
}

}  // namespace

extern "C" {

long long lbc_no_alloc_max_numel(void) { return LBC_NO_ALLOC_MAX_NUMEL; }
long long lbc_no_alloc_scratch_bytes(void) { return LBC_NO_ALLOC_SCRATCH_BYTES; }

const char* lbc_no_alloc_error_string(int code) {
    switch (code) {
        case LBC_NO_ALLOC_OK: return "ok";
        case LBC_NO_ALLOC_BAD_ARGUMENT:
            return "bad argument (dtype 0..2, group 16/32/64, bit 4/8, non-null x/out, residuals both or neither)";
        case LBC_NO_ALLOC_TOO_LARGE:
            return "numel exceeds LBC_NO_ALLOC_MAX_NUMEL (4 Mi elements): split the input into group-aligned pieces";
        case LBC_NO_ALLOC_SETUP_FAILED: return cudaGetErrorString(t_last_cuda_error);
        case LBC_NO_ALLOC_LAUNCH_FAILED: return cudaGetErrorString(t_last_cuda_error);
        default: return "unknown code";
    }
}

int lbc_no_alloc_roundtrip(int dtype, int group_size, int bit, const void* x, const void* residual_in, void* out,
                           void* residual_out, long long numel, cudaStream_t stream) {
    if (dtype < LBC_FP16 || dtype > LBC_FP32) return LBC_NO_ALLOC_BAD_ARGUMENT;
    if (group_size != 16 && group_size != 32 && group_size != 64) return LBC_NO_ALLOC_BAD_ARGUMENT;
    if (bit != 4 && bit != 8) return LBC_NO_ALLOC_BAD_ARGUMENT;
    if (numel < 0 || x == nullptr || out == nullptr) return LBC_NO_ALLOC_BAD_ARGUMENT;
    if ((residual_in == nullptr) != (residual_out == nullptr)) return LBC_NO_ALLOC_BAD_ARGUMENT;
    if (numel > LBC_NO_ALLOC_MAX_NUMEL) return LBC_NO_ALLOC_TOO_LARGE;
    if (numel == 0) return LBC_NO_ALLOC_OK;
    unsigned char* scratch = scratch_for_current_device();
    if (scratch == nullptr) return LBC_NO_ALLOC_SETUP_FAILED;

    const int64_t groups = (numel + group_size - 1) / group_size;

    LbcQuantPush q{};
    q.dtype = dtype;
    q.group_size = group_size;
    q.bit = bit;
    q.x = x;
    q.residual = residual_in;
    q.prepared_out = residual_out;   // `prepared` is parked in the residual buffer between the kernels
    q.numel = numel;
    q.mode = LBC_PUSH_BROADCAST;     // planar payload, one local destination
    q.dst[0] = scratch;
    q.num_dst = 1;
    q.layout_groups = groups;
    t_last_cuda_error = lbc_quant_push(&q, stream);
    if (t_last_cuda_error != cudaSuccess) return LBC_NO_ALLOC_LAUNCH_FAILED;

    LbcReduce r{};
    r.dtype = dtype;
    r.group_size = group_size;
    r.bit = bit;
    r.src[0] = scratch;
    r.num_src = 1;
    r.layout_groups = groups;
    r.numel = numel;
    r.scale = 1.0f;
    r.out = out;
    r.prepared = residual_out;
    r.residual_out = residual_out;
    t_last_cuda_error = lbc_reduce(&r, stream);
    if (t_last_cuda_error != cudaSuccess) return LBC_NO_ALLOC_LAUNCH_FAILED;
    return LBC_NO_ALLOC_OK;
}

}  // extern "C"

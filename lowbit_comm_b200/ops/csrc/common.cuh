// Device-side building blocks shared by every sm_100a kernel of the library:
// source-dtype traits, 128/256-bit global accesses, wire-order byte packing,
// system-scope signalling and bounded waits.
//
// Wire format facts used here (reference: csrc/quantization/quant_kernel.cuh:131-146,
// quant_pack_kernel.cu:101-144, dequant_reduce_kernel.cu:27-36): a payload word is
// as wide as the source element and holds its quantized elements most
// significant first, so inside a little-endian word the byte (int8) or nibble
// pair (int4) order is reversed.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "lbc_api.h"

namespace lbc {

constexpr int kMaxRanks = 16;
constexpr int kThreads = 256;
constexpr int kElemsPerThread = 16;  // one 16-byte vector of int8 codes per thread

// ---------------------------------------------------------------------------
// status word written by a kernel whose bounded wait ran out
// ---------------------------------------------------------------------------
struct DeviceStatus {
    unsigned int code;      // 0 = ok, 1 = wait timed out
    unsigned int phase;     // which kernel/phase gave up
    unsigned int peer;      // flag index that never arrived
    unsigned int seen;      // last value read
    unsigned int expected;  // value it waited for
    unsigned int reserved[3];
};

// ---------------------------------------------------------------------------
// dtype traits
// ---------------------------------------------------------------------------
template <typename T> struct Src;

template <> struct Src<__nv_bfloat16> {
    static constexpr int kBytes = 2;
    __device__ __forceinline__ static float up(uint16_t bits) { return __uint_as_float(uint32_t(bits) << 16); }
    __device__ __forceinline__ static uint16_t down(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }
    // two elements per 32-bit word: one conversion instruction per pair
    __device__ __forceinline__ static void up2(uint32_t w, float& lo, float& hi) {
        lo = __uint_as_float(w << 16);
        hi = __uint_as_float(w & 0xffff0000u);
    }
    __device__ __forceinline__ static uint32_t down2(float lo, float hi) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
};
template <> struct Src<__half> {
    static constexpr int kBytes = 2;
    __device__ __forceinline__ static float up(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }
    __device__ __forceinline__ static uint16_t down(float v) { return __half_as_ushort(__float2half_rn(v)); }
    __device__ __forceinline__ static void up2(uint32_t w, float& lo, float& hi) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
        lo = f.x;
        hi = f.y;
    }
    __device__ __forceinline__ static uint32_t down2(float lo, float hi) {
        const __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
};
template <> struct Src<float> {
    static constexpr int kBytes = 4;
    __device__ __forceinline__ static float up(uint32_t bits) { return __uint_as_float(bits); }
    __device__ __forceinline__ static uint32_t down(float v) { return __float_as_uint(v); }
};

// ---------------------------------------------------------------------------
// global memory accesses
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld16(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st16(void* p, uint4 v) {
    asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
struct alignas(32) U8x32 { uint32_t w[8]; };
// 256-bit accesses (sm_100+): one instruction per 32-byte sector.
__device__ __forceinline__ U8x32 ld32_stream(const void* p) {
    U8x32 v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]),
                   "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
    return v;
}
__device__ __forceinline__ U8x32 ld32(const void* p) {
    U8x32 v;
    asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]),
                   "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
    return v;
}
__device__ __forceinline__ void st32(void* p, const U8x32& v) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]),
                 "r"(v.w[2]), "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7]) : "memory");
}

// ---------------------------------------------------------------------------
// 16 source elements <-> 16 floats
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void load16(const T* base, int64_t first, int64_t numel, bool vec_ok, float (&out)[16],
                                       bool streaming) {
    if (vec_ok && first + 16 <= numel) {
        if constexpr (sizeof(T) == 2) {
            U8x32 v = streaming ? ld32_stream(base + first) : ld32(base + first);
#pragma unroll
            for (int i = 0; i < 8; ++i) Src<T>::up2(v.w[i], out[2 * i], out[2 * i + 1]);
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                U8x32 v = streaming ? ld32_stream(base + first + 8 * h) : ld32(base + first + 8 * h);
#pragma unroll
                for (int i = 0; i < 8; ++i) out[8 * h + i] = __uint_as_float(v.w[i]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int64_t at = first + i;
            if (at < numel) {
                if constexpr (sizeof(T) == 2)
                    out[i] = Src<T>::up(reinterpret_cast<const uint16_t*>(base)[at]);
                else
                    out[i] = reinterpret_cast<const float*>(base)[at];
            } else {
                out[i] = 0.0f;
            }
        }
    }
}

// Rounds to T and stores; `vals` is replaced by the rounded values (as float).
template <typename T>
__device__ __forceinline__ void round16(float (&vals)[16]) {
    if constexpr (sizeof(T) == 2) {
#pragma unroll
        for (int i = 0; i < 8; ++i) Src<T>::up2(Src<T>::down2(vals[2 * i], vals[2 * i + 1]), vals[2 * i], vals[2 * i + 1]);
    }
}

template <typename T>
__device__ __forceinline__ void store16(T* base, int64_t first, int64_t numel, bool vec_ok, const float (&vals)[16]) {
    if (vec_ok && first + 16 <= numel) {
        if constexpr (sizeof(T) == 2) {
            U8x32 v;
#pragma unroll
            for (int i = 0; i < 8; ++i) v.w[i] = Src<T>::down2(vals[2 * i], vals[2 * i + 1]);
            st32(base + first, v);
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                U8x32 v;
#pragma unroll
                for (int i = 0; i < 8; ++i) v.w[i] = __float_as_uint(vals[8 * h + i]);
                st32(base + first + 8 * h, v);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int64_t at = first + i;
            if (at < numel) {
                if constexpr (sizeof(T) == 2)
                    reinterpret_cast<uint16_t*>(base)[at] = Src<T>::down(vals[i]);
                else
                    reinterpret_cast<float*>(base)[at] = vals[i];
            }
        }
    }
}

// ---------------------------------------------------------------------------
// wire-order packing of 16 codes
// ---------------------------------------------------------------------------
// int8: natural little-endian bytes (e0 lowest) -> wire order inside each word.
template <int WordBytes>
__device__ __forceinline__ uint32_t wire_perm8(uint32_t natural) {
    return __byte_perm(natural, 0, WordBytes == 2 ? 0x2301 : 0x0123);
}

__device__ __forceinline__ int quant_rn(float v, float mul, int lim) {
    int q = __float2int_rn(v * mul);
    return max(-lim, min(lim, q));
}

// Packs 16 int8 codes (as ints in [-127,127]) into 16 wire-ordered bytes.
template <int WordBytes>
__device__ __forceinline__ uint4 pack16_i8(const int (&q)[16]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t nat = (uint32_t(q[4 * j]) & 0xffu) | ((uint32_t(q[4 * j + 1]) & 0xffu) << 8) |
                       ((uint32_t(q[4 * j + 2]) & 0xffu) << 16) | ((uint32_t(q[4 * j + 3]) & 0xffu) << 24);
        w[j] = wire_perm8<WordBytes>(nat);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Round-to-nearest-even quantization without a float->int conversion: adding
// 1.5 * 2^23 to t = v * mul leaves rint(t) in the low mantissa bits, so the low
// byte (nibble) of the result's bit pattern is the two's-complement code.  The
// product is rounded to fp32 first, exactly as rint(v * mul) would see it.
constexpr float kRoundMagic = 12582912.0f;  // bits 0x4B400000

template <int LIM>
__device__ __forceinline__ uint32_t quant_bits(float v, float mul) {
    float r = __fadd_rn(__fmul_rn(v, mul), kRoundMagic);
    r = fminf(fmaxf(r, kRoundMagic - float(LIM)), kRoundMagic + float(LIM));
    return __float_as_uint(r);
}
__device__ __forceinline__ int code_of_bits(uint32_t bits) { return int(bits) - 0x4B400000; }

// Low bytes of 16 bit patterns -> 16 wire-ordered bytes, three byte permutes per word.
template <int WordBytes>
__device__ __forceinline__ uint4 pack16_low_bytes(const uint32_t (&b)[16]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t e0 = b[4 * j], e1 = b[4 * j + 1], e2 = b[4 * j + 2], e3 = b[4 * j + 3];
        if constexpr (WordBytes == 2) {   // memory bytes: e1 e0 e3 e2
            w[j] = __byte_perm(__byte_perm(e1, e0, 0x0040), __byte_perm(e3, e2, 0x0040), 0x5410);
        } else {                          // memory bytes: e3 e2 e1 e0
            w[j] = __byte_perm(__byte_perm(e3, e2, 0x0040), __byte_perm(e1, e0, 0x0040), 0x5410);
        }
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// 16 wire-ordered int8 codes -> their values as floats: flip the sign bit of every
// byte, drop the byte into the mantissa of 2^23 and subtract 2^23 + 128 (exact).
template <int WordBytes>
__device__ __forceinline__ void unpack16_i8_fast(uint4 v, float (&out)[16]) {
    const uint32_t w[4] = {v.x ^ 0x80808080u, v.y ^ 0x80808080u, v.z ^ 0x80808080u, v.w ^ 0x80808080u};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int pos = WordBytes == 2 ? (e ^ 1) : (3 - e);
            out[4 * j + e] = __uint_as_float(__byte_perm(w[j], 0x4B000000u, 0x7540 | pos)) - 8388736.0f;
        }
    }
}

// Packs 16 int4 codes into 8 wire-ordered bytes (two 32-bit halves).
template <int WordBytes>
__device__ __forceinline__ uint2 pack16_i4(const int (&q)[16]) {
    uint32_t w[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        uint32_t nat = 0;  // byte b = (e[2b] << 4) | e[2b+1]  (big-endian byte sequence)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            uint32_t hi = uint32_t(q[8 * j + 2 * b]) & 0xfu, lo = uint32_t(q[8 * j + 2 * b + 1]) & 0xfu;
            nat |= ((hi << 4) | lo) << (8 * b);
        }
        w[j] = wire_perm8<WordBytes>(nat);
    }
    return make_uint2(w[0], w[1]);
}

template <int WordBytes>
__device__ __forceinline__ void unpack16_i8(uint4 v, float (&out)[16]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t nat = wire_perm8<WordBytes>(w[j]);  // the permutation is its own inverse
#pragma unroll
        for (int b = 0; b < 4; ++b) out[4 * j + b] = float(int(int8_t((nat >> (8 * b)) & 0xffu)));
    }
}

template <int WordBytes>
__device__ __forceinline__ void unpack16_i4(uint2 v, int (&codes)[16]) {
    const uint32_t w[2] = {v.x, v.y};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const uint32_t nat = wire_perm8<WordBytes>(w[j]);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t by = (nat >> (8 * b)) & 0xffu;
            codes[8 * j + 2 * b] = int(by >> 4);
            codes[8 * j + 2 * b + 1] = int(by & 0xfu);
        }
    }
}

__device__ __forceinline__ float int4_value(int code) { return float((code ^ 8) - 8); }

// ---------------------------------------------------------------------------
// cross-GPU signalling: release stores, acquire loads, bounded waits
// ---------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

using SignalSpec = LbcSignal;  // producer side, see lbc_api.h
using WaitSpec = LbcWait;      // consumer side, see lbc_api.h

// Returns false when the wait ran out; every thread of the block gets the same answer.
__device__ __forceinline__ bool block_wait(const WaitSpec& w) {
    if (w.flags == nullptr || w.count == 0) return true;
    __shared__ int ok;
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    if (threadIdx.x < w.count) {
        const unsigned int* f = w.flags + threadIdx.x;
        unsigned int seen = ld_acquire_sys(f);
        if (int(seen - w.epoch) < 0) {
            const unsigned long long t0 = global_ns();
            unsigned int spins = 0;
            for (;;) {
                seen = ld_acquire_sys(f);
                if (int(seen - w.epoch) >= 0) break;
                if ((++spins & 63u) == 0) {
                    volatile DeviceStatus* st = static_cast<volatile DeviceStatus*>(w.status);
                    // an earlier wait of this group already ran out: give up at once, so that the
                    // kernels queued behind a failed collective drain quickly
                    const bool failed_before = st != nullptr && st->code != 0u;
                    if (failed_before) {
                        ok = 0;
                        break;
                    }
                    if (global_ns() - t0 > w.timeout_ns) {
                        ok = 0;
                        // plain stores: the status word may live in mapped host memory, where
                        // device atomics are not guaranteed; any timed-out thread's report will do
                        if (st != nullptr) {
                            st->phase = w.phase;
                            st->peer = threadIdx.x;
                            st->seen = seen;
                            st->expected = w.epoch;
                            __threadfence_system();
                            st->code = 1u;
                            __threadfence_system();
                        }
                        break;
                    }
                }
                __nanosleep(64);
            }
        }
    }
    __syncthreads();
    return ok != 0;
}

// ---------------------------------------------------------------------------
// bulk asynchronous stores (TMA engine): shared memory -> global memory, own or a peer's.
// The copy engine moves the tile, so a back-pressured NVLink write does not stall the SM's
// load/store pipeline the way per-thread peer stores do.  No multicast, no tensor map: plain
// `cp.async.bulk` with 16-byte aligned addresses and sizes.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void fence_smem_to_async_proxy() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
                 "r"(smem_addr(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// At most one committed group may still be reading shared memory afterwards.
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// Every committed group has completed its writes.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Called by every thread after its last remote store.
// Stores through an NVLink multicast address: the switch writes the same bytes into the mapped
// region of every GPU of the multicast group (this GPU included), so one store leaves the SM
// instead of one per destination.  The data moves through .f32 registers bit for bit.
__device__ __forceinline__ void multimem_st16(void* mc_addr, uint4 v) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}
__device__ __forceinline__ void multimem_st8(void* mc_addr, uint2 v) {
    asm volatile("multimem.st.weak.global.v2.f32 [%0], {%1, %2};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y))
                 : "memory");
}

__device__ __forceinline__ void grid_signal(const SignalSpec& s) {
    if (s.num_remote <= 0) return;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned int done = atomicAdd(s.block_counter, 1u);
        if (done == gridDim.x * gridDim.y - 1) {
            *s.block_counter = 0u;
            __threadfence_system();
            for (int r = 0; r < s.num_remote; ++r) st_release_sys(s.remote_flags[r] + s.my_slot, s.epoch);
        }
    }
}

}  // namespace lbc

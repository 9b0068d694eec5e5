// Device functions shared by the codec kernels: group abs-max, alignment-agnostic payload accesses,
// scale staging and the 16-element encode / decode steps.
//
// Math parity with the reference kernels: quantization/quant_pack_kernel.cu:84-163 (the stored scale is
// rounded to the source dtype before use), quantization/dequant_reduce_kernel.cu:38-69 (scale / L decode).
#pragma once

#include "common.cuh"

namespace lbc {

template <int G>
__device__ __forceinline__ float group_max(float v) {
    constexpr int lanes = G / kElemsPerThread;
#pragma unroll
    for (int off = lanes / 2; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off, lanes));
    return v;
}

// Alignment-agnostic store of `n` bytes (n = 8 or 16) held in `v`.
__device__ __forceinline__ void store_codes(uint8_t* p, uint4 v, int n) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    if (n == 16 && (a & 15) == 0) {
        st16(p, v);
    } else if ((a & 7) == 0 && n == 8) {
        *reinterpret_cast<uint2*>(p) = make_uint2(v.x, v.y);
    } else if ((a & 3) == 0) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        for (int i = 0; i < n / 4; ++i) reinterpret_cast<uint32_t*>(p)[i] = w[i];
    } else {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        for (int i = 0; i < n / 2; ++i)
            reinterpret_cast<uint16_t*>(p)[i] = uint16_t(w[i / 2] >> (16 * (i & 1)));
    }
}

__device__ __forceinline__ uint4 load_codes(const uint8_t* p, int n) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    if (n == 16 && (a & 15) == 0) return ld16(p);
    uint32_t w[4] = {0, 0, 0, 0};
    if ((a & 3) == 0) {
        for (int i = 0; i < n / 4; ++i) w[i] = reinterpret_cast<const uint32_t*>(p)[i];
    } else {
        for (int i = 0; i < n / 2; ++i)
            w[i / 2] |= uint32_t(reinterpret_cast<const uint16_t*>(p)[i]) << (16 * (i & 1));
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T>
__device__ __forceinline__ void store_scale(uint8_t* p, float stored) {
    if constexpr (sizeof(T) == 2)
        *reinterpret_cast<uint16_t*>(p) = Src<T>::down(stored);
    else
        *reinterpret_cast<float*>(p) = stored;
}

template <typename T>
__device__ __forceinline__ float load_scale(const uint8_t* p) {
    if constexpr (sizeof(T) == 2)
        return Src<T>::up(*reinterpret_cast<const uint16_t*>(p));
    else
        return *reinterpret_cast<const float*>(p);
}

// Scales of planar payloads are written as 16-byte vectors, eight (fp32: four) groups at a
// time: one thread per group storing 2 or 4 bytes turns into one partial-sector write per
// group, which over NVLink costs a whole packet each and was measured to halve the push rate.
// The warp parks its scales in shared memory and a few lanes write them out.  Conditions
// (checked once per kernel): planar layout, layout and group offsets multiples of 8 groups,
// 16-byte aligned destinations; an 8-group unit then never straddles two shards.
struct ScaleStage {
    unsigned char bytes[kThreads / 32][32 * 4];
};

template <typename T>
__device__ __forceinline__ void park_scale(ScaleStage& stage, int group_in_warp, float stored) {
    unsigned char* slot = stage.bytes[threadIdx.x >> 5] + group_in_warp * sizeof(T);
    if constexpr (sizeof(T) == 2)
        *reinterpret_cast<uint16_t*>(slot) = Src<T>::down(stored);
    else
        *reinterpret_cast<float*>(slot) = stored;
}

__device__ __forceinline__ bool dsts_aligned16(uint8_t* const* dst, int n) {
    uintptr_t bits = 0;
    for (int d = 0; d < n; ++d) bits |= reinterpret_cast<uintptr_t>(dst[d]);
    return (bits & 15) == 0;
}

// Quantizes 16 rounded values with the group's stored scale; returns packed codes.
template <typename T, int BIT>
__device__ __forceinline__ uint4 encode16(const float (&vals)[16], float stored_scale, float (*decoded)[16]) {
    constexpr int lim = BIT == 8 ? 127 : 7;
    const float safe = fmaxf(stored_scale, 1.0e-6f);
    const float mul = float(lim) / safe;
    uint32_t b[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) b[i] = quant_bits<lim>(vals[i], mul);
    if (decoded != nullptr) {
        // this rank's own quantization error, one rounding: fma(-code, step, value)
        const float step = stored_scale / float(lim);
#pragma unroll
        for (int i = 0; i < 16; ++i) (*decoded)[i] = __fmaf_rn(-float(code_of_bits(b[i])), step, vals[i]);
    }
    if constexpr (BIT == 8) {
        return pack16_low_bytes<sizeof(T)>(b);
    } else {
        int q[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) q[i] = int(b[i]);
        const uint2 h = pack16_i4<sizeof(T)>(q);
        return make_uint4(h.x, h.y, 0, 0);
    }
}

// Unpacks 16 codes to their integer values (as floats); the caller multiplies by the step.
template <typename T, int BIT>
__device__ __forceinline__ void codes16(uint4 codes, float (&out)[16]) {
    if constexpr (BIT == 8) {
        unpack16_i8_fast<sizeof(T)>(codes, out);
    } else {
        int c[16];
        unpack16_i4<sizeof(T)>(make_uint2(codes.x, codes.y), c);
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = int4_value(c[i]);
    }
}

}  // namespace lbc

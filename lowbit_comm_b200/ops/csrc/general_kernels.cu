// General codec kernels: every combination the policy object allows that the
// production-profile kernels do not cover — top-k (1 or 2 values kept verbatim
// per group), 4-bit code-books (normal, uniform, e3m0, e2m1), stochastic
// rounding — for fp16/bf16/fp32 sources, group sizes 16/32/64, both payload
// layouts.  One kernel per (dtype, group size) with the rest as runtime
// parameters, instead of one instantiation per combination.
//
// Parity: quantization/quant_kernel.cuh:25-153 (top-k selection, scale = the
// (k+1)-th largest magnitude, selected elements zeroed), inner.cuh:9-96
// (code-book search, rounding rule, stochastic offsets), dequant_kernel.cuh
// :15-44,130-148 (decode and top-k write-back), and the fp32 twins.
// Tie-breaking between equal magnitudes: lowest index first for 16-bit
// sources, highest index first for fp32 sources.

#include <type_traits>

#include "common.cuh"
#include "lbc_api.h"

namespace lbc {

__constant__ float kCodebooks[4][16] = {
    {-1.0f, -0.815410147f, -0.655160150f, -0.510228027f, -0.375324982f, -0.246951370f, -0.122538030f, 0.0f,
     0.122538030f, 0.246951370f, 0.375324982f, 0.510228027f, 0.655160150f, 0.815410147f, 1.0f, INFINITY},
    {-1.0f, -0.85714286f, -0.71428571f, -0.57142857f, -0.42857143f, -0.28571429f, -0.14285714f, 0.0f,
     0.14285714f, 0.28571429f, 0.42857143f, 0.57142857f, 0.71428571f, 0.85714286f, 1.0f, INFINITY},
    {-1.0f, -0.5f, -0.25f, -0.125f, -0.0625f, -0.03125f, -0.015625f, 0.0f,
     0.015625f, 0.03125f, 0.0625f, 0.125f, 0.25f, 0.5f, 1.0f, INFINITY},
    {-1.0f, -0.6666666666666666f, -0.5f, -0.3333333333333333f, -0.25f, -0.16666666666666666f, -0.125f, 0.0f,
     0.125f, 0.16666666666666666f, 0.25f, 0.3333333333333333f, 0.5f, 0.6666666666666666f, 1.0f, INFINITY},
};

// Counter-based uniform in (0, 1]: a 64-bit mix of (seed, element index).
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long index) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (index + 1ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float(unsigned(z >> 40)) + 1.0f) * (1.0f / 16777216.0f);
}

struct Cand {
    float mag;
    int idx;
};

// (mag, idx) ordering: larger magnitude first; ties by index (low first unless HighWins).
template <bool HighWins>
__device__ __forceinline__ bool beats(const Cand& a, const Cand& b) {
    if (a.mag != b.mag) return a.mag > b.mag;
    return HighWins ? a.idx > b.idx : a.idx < b.idx;
}

template <bool HighWins>
__device__ __forceinline__ void insert3(Cand (&top)[3], Cand c) {
    if (beats<HighWins>(c, top[0])) {
        top[2] = top[1];
        top[1] = top[0];
        top[0] = c;
    } else if (beats<HighWins>(c, top[1])) {
        top[2] = top[1];
        top[1] = c;
    } else if (beats<HighWins>(c, top[2])) {
        top[2] = c;
    }
}

template <typename T>
__device__ __forceinline__ void store_word(uint8_t* p, uint32_t bits) {
    if constexpr (sizeof(T) == 2)
        *reinterpret_cast<uint16_t*>(p) = uint16_t(bits);
    else
        *reinterpret_cast<uint32_t*>(p) = bits;
}

template <typename T>
__device__ __forceinline__ uint32_t load_word(const uint8_t* p) {
    if constexpr (sizeof(T) == 2)
        return *reinterpret_cast<const uint16_t*>(p);
    else
        return *reinterpret_cast<const uint32_t*>(p);
}

template <typename T>
__device__ __forceinline__ uint32_t bits_of(float v) {
    return uint32_t(Src<T>::down(v));
}
template <typename T>
__device__ __forceinline__ float value_of(uint32_t bits) {
    if constexpr (sizeof(T) == 2)
        return Src<T>::up(uint16_t(bits));
    else
        return __uint_as_float(bits);
}

__device__ __forceinline__ void store_bytes(uint8_t* p, const uint32_t (&w)[4], int n) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    if ((a & 3) == 0) {
        for (int i = 0; i < n / 4; ++i) reinterpret_cast<uint32_t*>(p)[i] = w[i];
    } else {
        for (int i = 0; i < n / 2; ++i) reinterpret_cast<uint16_t*>(p)[i] = uint16_t(w[i / 2] >> (16 * (i & 1)));
    }
}
__device__ __forceinline__ void load_bytes(const uint8_t* p, uint32_t (&w)[4], int n) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    w[0] = w[1] = w[2] = w[3] = 0;
    if ((a & 3) == 0) {
        for (int i = 0; i < n / 4; ++i) w[i] = reinterpret_cast<const uint32_t*>(p)[i];
    } else {
        for (int i = 0; i < n / 2; ++i) w[i / 2] |= uint32_t(reinterpret_cast<const uint16_t*>(p)[i]) << (16 * (i & 1));
    }
}

template <typename T, int G>
__global__ void __launch_bounds__(kThreads) quant_general_kernel(const LbcQuantGeneral p) {
    constexpr int lanes = G / kElemsPerThread;
    constexpr bool kHighWins = sizeof(T) == 4;
    const int VB = G * p.bit / 8;
    const int meta_words = p.topk == 0 ? 1 : (p.topk == 1 ? 3 : 4);
    const int MB = meta_words * int(sizeof(T));
    const int CB = kElemsPerThread * p.bit / 8;
    const T* x = static_cast<const T*>(p.x);
    const T* res = static_cast<const T*>(p.residual);
    T* prep = static_cast<T*>(p.prepared_out);
    const int64_t n = p.numel;
    const int64_t num_groups = (n + G - 1) / G;
    const int64_t num_chunks = num_groups * lanes;
    const int64_t chunk_span = (num_chunks + 31) / 32 * 32;
    const bool x_vec = (reinterpret_cast<uintptr_t>(x) & 31) == 0;
    const bool r_vec = res == nullptr || (reinterpret_cast<uintptr_t>(res) & 31) == 0;
    const bool p_vec = prep == nullptr || (reinterpret_cast<uintptr_t>(prep) & 31) == 0;

    for (int64_t chunk = int64_t(blockIdx.x) * kThreads + threadIdx.x; chunk < chunk_span;
         chunk += int64_t(gridDim.x) * kThreads) {
        const bool live = chunk < num_chunks;
        const int64_t first = chunk * kElemsPerThread;
        const int64_t g = chunk / lanes;
        const int lane = int(chunk - g * lanes);
        float v[16];
        if (live) {
            load16<T>(x, first, n, x_vec, v, true);
            if (res != nullptr) {
                float r[16];
                load16<T>(res, first, n, r_vec, r, prep != res);
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] += r[i];
                round16<T>(v);
            }
            if (prep != nullptr) store16<T>(prep, first, n, p_vec, v);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.0f;
        }
        // three best (magnitude, index) candidates of the group
        Cand top[3] = {{-1.0f, -1}, {-1.0f, -1}, {-1.0f, -1}};
        if constexpr (sizeof(T) == 2) {
            // 16-bit sources: the values are exact in T, so (|v| as T bits) << 8 | (255 - index) is a 24-bit key
            // whose integer order is the order above (larger magnitude first, lower index on ties); the three
            // largest keys come out of a branch-free chain of five integer min/max per candidate.
            uint32_t k0 = 0, k1 = 0, k2 = 0;          // below every real key (an index is at most 63)
            auto put = [&](uint32_t c) {
                uint32_t t = max(k0, c);
                c = min(k0, c);
                k0 = t;
                t = max(k1, c);
                c = min(k1, c);
                k1 = t;
                k2 = max(k2, c);
            };
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                uint32_t mag_bits;      // |v| as T bits, shifted up by 8
                if constexpr (std::is_same<T, __nv_bfloat16>::value)
                    mag_bits = (__float_as_uint(v[i]) & 0x7fffffffu) >> 8;      // bf16: the high half of the fp32 pattern
                else
                    mag_bits = uint32_t(Src<T>::down(fabsf(v[i]))) << 8;
                put(mag_bits | uint32_t(255 - (lane * 16 + i)));
            }
#pragma unroll
            for (int off = lanes / 2; off > 0; off >>= 1) {
                const uint32_t o0 = __shfl_xor_sync(0xffffffffu, k0, off, lanes);
                const uint32_t o1 = __shfl_xor_sync(0xffffffffu, k1, off, lanes);
                const uint32_t o2 = __shfl_xor_sync(0xffffffffu, k2, off, lanes);
                put(o0);
                put(o1);
                put(o2);
            }
            const uint32_t keys[3] = {k0, k1, k2};
#pragma unroll
            for (int j = 0; j < 3; ++j) top[j] = Cand{Src<T>::up(uint16_t(keys[j] >> 8)), 255 - int(keys[j] & 0xffu)};
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) insert3<kHighWins>(top, Cand{fabsf(v[i]), lane * 16 + i});
#pragma unroll
            for (int off = lanes / 2; off > 0; off >>= 1) {
                Cand other[3];
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    other[j].mag = __shfl_xor_sync(0xffffffffu, top[j].mag, off, lanes);
                    other[j].idx = __shfl_xor_sync(0xffffffffu, top[j].idx, off, lanes);
                }
#pragma unroll
                for (int j = 0; j < 3; ++j) insert3<kHighWins>(top, other[j]);
            }
        }
        if (!live) continue;
        const float amax = top[p.topk].mag;  // (k+1)-th largest magnitude
        float kept[2] = {0.0f, 0.0f};
        // pull the kept values out of this lane's registers
        for (int j = 0; j < p.topk; ++j) {
            const int at = top[j].idx - lane * 16;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (i == at) { kept[j] = v[i]; v[i] = 0.0f; }
        }
        // the owning lane hands the kept value to lane 0 of the group
        for (int j = 0; j < p.topk; ++j) {
            const int owner = top[j].idx / 16;
            kept[j] = __shfl_sync(__activemask(), kept[j], (threadIdx.x & 31) - lane + owner);
        }
        float stored = amax;
        if constexpr (sizeof(T) == 2) stored = Src<T>::up(Src<T>::down(amax));
        const float safe = fmaxf(stored, 1.0e-6f);
        int q[16];
        if (p.quant_type == LBC_LINEAR) {
            const int lim = p.bit == 8 ? 127 : 7;
            const float mul = float(lim) / safe;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float t = v[i] * mul;
                if (p.stochastic) t += uniform01(p.seed, (unsigned long long)(first + i)) - 0.5f;
                q[i] = max(-lim, min(lim, __float2int_rn(t)));
            }
        } else {
            const float* table = kCodebooks[p.quant_type - 1];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float t = v[i] / safe;
                int lo = 0, hi = 14;
                while (lo < hi) {
                    const int mid = (lo + hi + 1) >> 1;
                    if (t < table[mid]) hi = mid - 1; else lo = mid;
                }
                const float gap = table[lo + 1] - table[lo];
                bool up;
                if (p.stochastic)
                    up = uniform01(p.seed, (unsigned long long)(first + i)) < (t - table[lo]) / gap;
                else
                    up = (t - table[lo]) > gap * 0.5f;
                q[i] = lo + (up ? 1 : 0);
            }
        }
        uint32_t w[4] = {0, 0, 0, 0};
        if (p.bit == 8) {
            const uint4 c = pack16_i8<sizeof(T)>(q);
            w[0] = c.x; w[1] = c.y; w[2] = c.z; w[3] = c.w;
        } else {
            const uint2 c = pack16_i4<sizeof(T)>(q);
            w[0] = c.x; w[1] = c.y;
        }
        uint32_t index_word = 0;
        if (p.topk >= 1) {
            index_word = uint32_t(top[0].idx);
            if (p.topk == 2) index_word |= uint32_t(top[1].idx) << 8;
        }
        const bool scatter = p.num_dst > 0 && p.shard_groups > 0;
        const int copies = (p.num_dst > 0 && !scatter) ? p.num_dst : 1;
        for (int d = 0; d < copies; ++d) {      // one payload, the same payload in every rank's slot, or one shard
            uint8_t* base = p.num_dst > 0 ? p.dst[d] : p.out;
            int64_t gl = g, layout = num_groups;
            if (scatter) {
                const int64_t owner = g / p.shard_groups;
                base = p.dst[owner];
                gl = g - owner * p.shard_groups;
                layout = p.shard_groups;
            }
            uint8_t* vptr;
            uint8_t* mptr;
            if (p.compact) {
                vptr = base + gl * (VB + MB);
                mptr = vptr + VB;
            } else {
                vptr = base + gl * VB;
                mptr = base + layout * VB + gl * MB;
            }
            store_bytes(vptr + lane * CB, w, CB);
            if (lane == 0) {
                store_word<T>(mptr, bits_of<T>(stored));
                if (p.topk >= 1) {
                    store_word<T>(mptr + sizeof(T), index_word);
                    store_word<T>(mptr + 2 * sizeof(T), bits_of<T>(kept[0]));
                    if (p.topk == 2) store_word<T>(mptr + 3 * sizeof(T), bits_of<T>(kept[1]));
                }
            }
        }
    }
    grid_signal(p.signal);      // no-op without destinations to notify
}

// Decodes the 16 elements of (group g, lane) of one payload into d, rounded to T, top-k values written back.
template <typename T>
__device__ __forceinline__ void decode_general_chunk(const uint8_t* src, int compact, int bit, int topk, int quant_type,
                                                     int VB, int MB, int CB, int64_t num_groups, int64_t g, int lane,
                                                     float (&d)[16]) {
    const uint8_t* vptr;
    const uint8_t* mptr;
    if (compact) {
        vptr = src + g * (VB + MB);
        mptr = vptr + VB;
    } else {
        vptr = src + g * VB;
        mptr = src + num_groups * VB + g * MB;
    }
    uint32_t w[4];
    load_bytes(vptr + lane * CB, w, CB);
    const float stored = value_of<T>(load_word<T>(mptr));
    if (quant_type == LBC_LINEAR) {
        if (bit == 8) {
            unpack16_i8<sizeof(T)>(make_uint4(w[0], w[1], w[2], w[3]), d);
            const float step = stored / 127.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) d[i] *= step;
        } else {
            int c[16];
            unpack16_i4<sizeof(T)>(make_uint2(w[0], w[1]), c);
            const float step = stored / 7.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) d[i] = int4_value(c[i]) * step;
        }
    } else {
        int c[16];
        unpack16_i4<sizeof(T)>(make_uint2(w[0], w[1]), c);
        const float* table = kCodebooks[quant_type - 1];
#pragma unroll
        for (int i = 0; i < 16; ++i) d[i] = table[c[i]] * stored;
    }
    round16<T>(d);
    if (topk >= 1) {
        const uint32_t index_word = load_word<T>(mptr + sizeof(T));
        for (int j = 0; j < topk; ++j) {
            const int at = int((index_word >> (8 * j)) & 0xffu) - lane * 16;
            if (at >= 0 && at < 16) {
                const float kept = value_of<T>(load_word<T>(mptr + (2 + j) * sizeof(T)));
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (i == at) d[i] = kept;
            }
        }
    }
}

template <typename T, int G>
__global__ void __launch_bounds__(kThreads) dequant_general_kernel(const LbcDequantGeneral p) {
    constexpr int lanes = G / kElemsPerThread;
    const int VB = G * p.bit / 8;
    const int meta_words = p.topk == 0 ? 1 : (p.topk == 1 ? 3 : 4);
    const int MB = meta_words * int(sizeof(T));
    const int CB = kElemsPerThread * p.bit / 8;
    T* out = static_cast<T*>(p.out);
    const int64_t n = p.numel;
    const int64_t num_groups = (n + G - 1) / G;
    const int64_t num_chunks = num_groups * lanes;
    const bool o_vec = (reinterpret_cast<uintptr_t>(out) & 31) == 0;
    for (int64_t chunk = int64_t(blockIdx.x) * kThreads + threadIdx.x; chunk < num_chunks;
         chunk += int64_t(gridDim.x) * kThreads) {
        const int64_t first = chunk * kElemsPerThread;
        const int64_t g = chunk / lanes;
        const int lane = int(chunk - g * lanes);
        float d[16];
        decode_general_chunk<T>(p.src, p.compact, p.bit, p.topk, p.quant_type, VB, MB, CB, num_groups, g, lane, d);
        if (p.accumulate) {
            float prev[16];
            load16<T>(out, first, n, o_vec, prev, false);
#pragma unroll
            for (int i = 0; i < 16; ++i) d[i] += prev[i];
        }
        store16<T>(out, first, n, o_vec, d);
    }
}

template <typename T, int G>
__global__ void __launch_bounds__(kThreads) reduce_general_kernel(const LbcReduceGeneral p) {
    constexpr int lanes = G / kElemsPerThread;
    if (!block_wait(p.wait)) return;      // bounded; the status word says which flag never came
    const int VB = G * p.bit / 8;
    const int meta_words = p.topk == 0 ? 1 : (p.topk == 1 ? 3 : 4);
    const int MB = meta_words * int(sizeof(T));
    const int CB = kElemsPerThread * p.bit / 8;
    T* out = static_cast<T*>(p.out);
    const T* prep = static_cast<const T*>(p.prepared);
    T* res = static_cast<T*>(p.residual_out);
    const int64_t n = p.numel;
    const int64_t num_groups = (n + G - 1) / G;
    const int64_t num_chunks = num_groups * lanes;
    const bool o_vec = (reinterpret_cast<uintptr_t>(out) & 31) == 0;
    const bool p_vec = prep == nullptr || (reinterpret_cast<uintptr_t>(prep) & 31) == 0;
    const bool r_vec = res == nullptr || (reinterpret_cast<uintptr_t>(res) & 31) == 0;
    for (int64_t chunk = int64_t(blockIdx.x) * kThreads + threadIdx.x; chunk < num_chunks;
         chunk += int64_t(gridDim.x) * kThreads) {
        const int64_t first = chunk * kElemsPerThread;
        const int64_t g = chunk / lanes;
        const int lane = int(chunk - g * lanes);
        float acc[16];
        if (p.src_shard_groups > 0) {
            // gather: the group lives in exactly one source, its owner's reduced shard
            const int64_t owner = g / p.src_shard_groups;
            decode_general_chunk<T>(p.src[owner], p.compact, p.bit, p.topk, p.quant_type, VB, MB, CB, p.src_shard_groups,
                                    g - owner * p.src_shard_groups, lane, acc);
        } else {
            const int64_t layout = p.layout_groups > 0 ? p.layout_groups : num_groups;
            decode_general_chunk<T>(p.src[0], p.compact, p.bit, p.topk, p.quant_type, VB, MB, CB, layout, g, lane, acc);
            for (int r = 1; r < p.num_src; ++r) {
                float d[16];
                decode_general_chunk<T>(p.src[r], p.compact, p.bit, p.topk, p.quant_type, VB, MB, CB, layout, g, lane, d);
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] += d[i];
                round16<T>(acc);                // the sum lives in the source dtype between payloads
            }
        }
        if (p.scale != 1.0f) {
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] *= p.scale;
            round16<T>(acc);
        }
        if (prep != nullptr) {
            float e[16];
            load16<T>(prep, first, n, p_vec, e, prep != res);
#pragma unroll
            for (int i = 0; i < 16; ++i) e[i] -= acc[i];
            store16<T>(res, first, n, r_vec, e);
        }
        store16<T>(out, first, n, o_vec, acc);
    }
}

static int general_grid(int64_t chunks, int max_blocks = 0) {
    int64_t want = (chunks + kThreads - 1) / kThreads;
    const int cap = max_blocks > 0 ? max_blocks : lbc_default_max_blocks();
    if (want < 1) want = 1;
    return int(want < cap ? want : cap);
}

template <typename T>
static cudaError_t launch_quant(const LbcQuantGeneral* p, cudaStream_t s) {
    const int64_t groups = (p->numel + p->group_size - 1) / p->group_size;
    if (groups == 0) return cudaSuccess;
    const int grid = general_grid(groups * (p->group_size / kElemsPerThread), p->max_blocks);
    switch (p->group_size) {
        case 64: quant_general_kernel<T, 64><<<grid, kThreads, 0, s>>>(*p); break;
        case 32: quant_general_kernel<T, 32><<<grid, kThreads, 0, s>>>(*p); break;
        case 16: quant_general_kernel<T, 16><<<grid, kThreads, 0, s>>>(*p); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_dequant(const LbcDequantGeneral* p, cudaStream_t s) {
    const int64_t groups = (p->numel + p->group_size - 1) / p->group_size;
    if (groups == 0) return cudaSuccess;
    const int grid = general_grid(groups * (p->group_size / kElemsPerThread));
    switch (p->group_size) {
        case 64: dequant_general_kernel<T, 64><<<grid, kThreads, 0, s>>>(*p); break;
        case 32: dequant_general_kernel<T, 32><<<grid, kThreads, 0, s>>>(*p); break;
        case 16: dequant_general_kernel<T, 16><<<grid, kThreads, 0, s>>>(*p); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_reduce_general(const LbcReduceGeneral* p, cudaStream_t s) {
    const int64_t groups = (p->numel + p->group_size - 1) / p->group_size;
    if (groups == 0) return cudaSuccess;
    const int grid = general_grid(groups * (p->group_size / kElemsPerThread), p->max_blocks);
    switch (p->group_size) {
        case 64: reduce_general_kernel<T, 64><<<grid, kThreads, 0, s>>>(*p); break;
        case 32: reduce_general_kernel<T, 32><<<grid, kThreads, 0, s>>>(*p); break;
        case 16: reduce_general_kernel<T, 16><<<grid, kThreads, 0, s>>>(*p); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

static bool general_args_ok(int bit, int topk, int quant_type) {
    if (bit != 4 && bit != 8) return false;
    if (topk < 0 || topk > 2) return false;
    if (quant_type < LBC_LINEAR || quant_type > LBC_E2M1) return false;
    if (quant_type != LBC_LINEAR && bit != 4) return false;
    return true;
}

}  // namespace lbc

extern "C" {

cudaError_t lbc_quant_general(const LbcQuantGeneral* p, cudaStream_t stream) {
    if (p == nullptr || p->numel < 0 || !lbc::general_args_ok(p->bit, p->topk, p->quant_type)) return cudaErrorInvalidValue;
    if (p->num_dst < 0 || p->num_dst > LBC_MAX_RANKS || (p->num_dst == 0 && p->out == nullptr)) return cudaErrorInvalidValue;
    if (p->shard_groups < 0) return cudaErrorInvalidValue;
    if (p->shard_groups > 0 && p->num_dst > 0) {      // every group must have an owner among the destinations
        const int64_t groups = (p->numel + p->group_size - 1) / p->group_size;
        if (groups > p->shard_groups * p->num_dst) return cudaErrorInvalidValue;
    }
    for (int d = 0; d < p->num_dst; ++d)
        if (p->dst[d] == nullptr) return cudaErrorInvalidValue;
    switch (p->dtype) {
        case LBC_BF16: return lbc::launch_quant<__nv_bfloat16>(p, stream);
        case LBC_FP16: return lbc::launch_quant<__half>(p, stream);
        case LBC_FP32: return lbc::launch_quant<float>(p, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t lbc_dequant_general(const LbcDequantGeneral* p, cudaStream_t stream) {
    if (p == nullptr || p->numel < 0 || !lbc::general_args_ok(p->bit, p->topk, p->quant_type)) return cudaErrorInvalidValue;
    switch (p->dtype) {
        case LBC_BF16: return lbc::launch_dequant<__nv_bfloat16>(p, stream);
        case LBC_FP16: return lbc::launch_dequant<__half>(p, stream);
        case LBC_FP32: return lbc::launch_dequant<float>(p, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t lbc_reduce_general(const LbcReduceGeneral* p, cudaStream_t stream) {
    if (p == nullptr || p->numel < 0 || !lbc::general_args_ok(p->bit, p->topk, p->quant_type)) return cudaErrorInvalidValue;
    if (p->num_src < 1 || p->num_src > LBC_MAX_RANKS || p->out == nullptr) return cudaErrorInvalidValue;
    if ((p->prepared == nullptr) != (p->residual_out == nullptr)) return cudaErrorInvalidValue;
    if (p->layout_groups < 0 || p->src_shard_groups < 0) return cudaErrorInvalidValue;
    {
        const int64_t groups = (p->numel + p->group_size - 1) / p->group_size;
        if (p->src_shard_groups > 0 && groups > p->src_shard_groups * p->num_src) return cudaErrorInvalidValue;
        if (p->src_shard_groups == 0 && p->layout_groups > 0 && groups > p->layout_groups) return cudaErrorInvalidValue;
    }
    for (int r = 0; r < p->num_src; ++r)
        if (p->src[r] == nullptr) return cudaErrorInvalidValue;
    switch (p->dtype) {
        case LBC_BF16: return lbc::launch_reduce_general<__nv_bfloat16>(p, stream);
        case LBC_FP16: return lbc::launch_reduce_general<__half>(p, stream);
        case LBC_FP32: return lbc::launch_reduce_general<float>(p, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // extern "C"

// Host (CPU) implementation of the wire format: plain C++17, no CUDA, no torch.
//
// Two jobs.  (1) The CPU / gloo configuration quantizes and decodes gradient
// buckets with it instead of composing a dozen torch ops per call.  (2) It is a
// second, independently written statement of the format: the tests require it
// to agree bit for bit with the torch oracle (ops/oracle.py) that the sm_100a
// kernels are checked against.
//
// Scope: deterministic rounding; int8 and int4; groups of 16, 32, 64; fp16,
// bf16 and fp32 sources; planar and compact layouts; top-k 0, 1 and 2; the
// linear code and the four 4-bit code-books.  The fused multi-payload reduce
// serves the production profile family (linear, top-k 0).  Math as in the reference's kernels
// (csrc/quantization/quant_pack_kernel.cu:25-163, dequant_kernel.cuh:15-44,
// dequant_reduce_kernel.cu:38-221): scale = group abs-max stored in the source
// dtype, q = clamp(rint(p * (L / max(s, 1e-6))), -L, L), decode q * (s / L),
// fused reduce with one fused multiply-add per payload.
//
// Build with -ffp-contract=off: every product and sum below is a separate
// fp32 rounding except the explicit fmaf.
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

namespace {

enum DType { kFP16 = 0, kBF16 = 1, kFP32 = 2 };

inline uint32_t bits_of(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}
inline float float_of(uint32_t u) {
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// ---- fp16 / bf16 <-> fp32, round to nearest even -----------------------------
inline float half_to_float(uint16_t h) {
    const uint32_t sign = uint32_t(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return float_of(sign);
        int e = -1;                       // subnormal: normalise
        do {
            ++e;
            man <<= 1;
        } while ((man & 0x400u) == 0);
        return float_of(sign | uint32_t(127 - 15 - e) << 23 | (man & 0x3FFu) << 13);
    }
    if (exp == 31) return float_of(sign | 0x7F800000u | man << 13);
    return float_of(sign | (exp + 112u) << 23 | man << 13);
}

inline uint16_t float_to_half(float f) {
    uint32_t x = bits_of(f);
    const uint16_t sign = uint16_t((x >> 16) & 0x8000u);
    x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) return uint16_t(sign | (x > 0x7F800000u ? 0x7E00u : 0x7C00u));
    if (x >= 0x477FF000u) return uint16_t(sign | 0x7C00u);       // >= 65520 rounds to infinity
    if (x < 0x38800000u) {                                      // below the smallest normal half
        if (x < 0x33000000u) return sign;                       // < 2^-25 rounds to zero
        const uint32_t shift = 126u - (x >> 23);                // 14 ... 24
        const uint32_t man = (x & 0x7FFFFFu) | 0x800000u;
        uint32_t r = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (r & 1u))) ++r;
        return uint16_t(sign | r);
    }
    uint32_t r = (x - 0x38000000u) >> 13;
    const uint32_t rem = x & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;     // may carry into the exponent: still right
    return uint16_t(sign | r);
}

inline float bf16_to_float(uint16_t b) { return float_of(uint32_t(b) << 16); }

inline uint16_t float_to_bf16(float f) {
    const uint32_t x = bits_of(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((x >> 16) | 0x0040u);   // quiet NaN
    return uint16_t((x + 0x7FFFu + ((x >> 16) & 1u)) >> 16);
}

// Groups are independent, so the loops over groups are split into contiguous ranges, one per thread.  The
// result does not depend on the split (each group is computed by the same scalar code), only the time does.
// LBC_HOST_THREADS caps the thread count (default: hardware threads, at most 8; several CPU ranks on one
// machine may want 1); tensors below 8192 groups per thread are not worth a thread.
inline int64_t host_threads_for(int64_t groups) {
    static const int64_t cap = [] {
        const char* env = std::getenv("LBC_HOST_THREADS");
        int64_t n = env != nullptr ? std::atoll(env) : int64_t(std::thread::hardware_concurrency());
        return n < 1 ? int64_t(1) : (n > 8 && env == nullptr ? int64_t(8) : n);
    }();
    const int64_t useful = groups / 8192;
    return useful < cap ? (useful < 1 ? 1 : useful) : cap;
}

template <typename Body>
void for_group_ranges(int64_t groups, Body body) {
    const int64_t threads = host_threads_for(groups);
    if (threads <= 1) {
        body(int64_t(0), groups);
        return;
    }
    const int64_t per = (groups + threads - 1) / threads;
    std::vector<std::thread> helpers;
    helpers.reserve(size_t(threads - 1));
    for (int64_t t = 1; t < threads; ++t) {
        const int64_t lo = t * per, hi = lo + per < groups ? lo + per : groups;
        if (lo < hi) helpers.emplace_back(body, lo, hi);
    }
    body(int64_t(0), per < groups ? per : groups);
    for (auto& h : helpers) h.join();
}

template <int DT> struct Src;
template <> struct Src<kFP16> {
    using T = uint16_t;
    static float up(T v) { return half_to_float(v); }
    static T down(float v) { return float_to_half(v); }
};
template <> struct Src<kBF16> {
    using T = uint16_t;
    static float up(T v) { return bf16_to_float(v); }
    static T down(float v) { return float_to_bf16(v); }
};
template <> struct Src<kFP32> {
    using T = uint32_t;
    static float up(T v) { return float_of(v); }
    static T down(float v) { return bits_of(v); }
};

struct Layout {
    int64_t groups, value_bytes, meta_bytes;
    bool compact;
    const uint8_t* values(const uint8_t* base, int64_t g) const {
        return compact ? base + g * (value_bytes + meta_bytes) : base + g * value_bytes;
    }
    const uint8_t* meta(const uint8_t* base, int64_t g) const {
        return compact ? base + g * (value_bytes + meta_bytes) + value_bytes
                       : base + groups * value_bytes + g * meta_bytes;
    }
    uint8_t* values(uint8_t* base, int64_t g) const { return const_cast<uint8_t*>(values((const uint8_t*)base, g)); }
    uint8_t* meta(uint8_t* base, int64_t g) const { return const_cast<uint8_t*>(meta((const uint8_t*)base, g)); }
};

inline Layout layout_of(int64_t numel, int group, int bit, int word, bool compact) {
    return Layout{(numel + group - 1) / group, int64_t(group) * bit / 8, int64_t(word), compact};
}

// Position of natural byte `e` of a group's value bytes: words are as wide as the source element
// and hold their bytes most-significant first.
inline int wire_pos(int e, int word) { return (e / word) * word + (word - 1 - e % word); }

inline int signed_code(const uint8_t* values, int i, int bit, int word) {
    if (bit == 8) return int(int8_t(values[wire_pos(i, word)]));
    const uint8_t byte = values[wire_pos(i / 2, word)];
    const int field = (i % 2 == 0) ? (byte >> 4) : (byte & 15);
    return field >= 8 ? field - 16 : field;
}

template <int DT>
int quantize(int group, int bit, bool compact, const void* x_, const void* res_, void* prep_, int64_t numel,
             uint8_t* out) {
    using S = Src<DT>;
    using T = typename S::T;
    const T* x = static_cast<const T*>(x_);
    const T* res = static_cast<const T*>(res_);
    T* prep = static_cast<T*>(prep_);
    const int word = int(sizeof(T));
    const Layout lay = layout_of(numel, group, bit, word, compact);
    const float lim = bit == 8 ? 127.0f : 7.0f;
    for_group_ranges(lay.groups, [=](int64_t g_lo, int64_t g_hi) {
    float p[64];
    for (int64_t g = g_lo; g < g_hi; ++g) {
        const int64_t first = g * group;
        float amax = 0.0f;
        for (int i = 0; i < group; ++i) {
            const int64_t idx = first + i;
            float v = 0.0f;
            if (idx < numel) {
                v = S::up(x[idx]);
                if (res != nullptr) v = S::up(S::down(v + S::up(res[idx])));   // prepared, rounded to T first
                if (prep != nullptr) prep[idx] = S::down(v);
            }
            p[i] = v;
            const float a = std::fabs(v);
            if (a > amax) amax = a;
        }
        const T stored = S::down(amax);                 // exact: amax is a T value
        const float safe = std::fmax(S::up(stored), 1e-6f);
        const float mul = lim / safe;
        uint8_t* values = lay.values(out, g);
        for (int i = 0; i < group; i += (bit == 8 ? 1 : 2)) {
            auto code = [&](float v) {
                float q = std::nearbyintf(v * mul);
                q = q < -lim ? -lim : (q > lim ? lim : q);
                return int(q);
            };
            if (bit == 8) {
                values[wire_pos(i, word)] = uint8_t(code(p[i]) & 255);
            } else {
                values[wire_pos(i / 2, word)] = uint8_t(((code(p[i]) & 15) << 4) | (code(p[i + 1]) & 15));
            }
        }
        std::memcpy(lay.meta(out, g), &stored, sizeof(T));
    }
    });
    return 0;
}

template <int DT>
int dequantize(int group, int bit, bool compact, const uint8_t* payload, int64_t numel, void* out_, bool accumulate) {
    using S = Src<DT>;
    using T = typename S::T;
    T* out = static_cast<T*>(out_);
    const int word = int(sizeof(T));
    const Layout lay = layout_of(numel, group, bit, word, compact);
    const float lim = bit == 8 ? 127.0f : 7.0f;
    for_group_ranges(lay.groups, [=](int64_t g_lo, int64_t g_hi) {
    for (int64_t g = g_lo; g < g_hi; ++g) {
        T stored;
        std::memcpy(&stored, lay.meta(payload, g), sizeof(T));
        const float step = S::up(stored) / lim;
        const uint8_t* values = lay.values(payload, g);
        for (int i = 0; i < group; ++i) {
            const int64_t idx = g * group + i;
            if (idx >= numel) break;
            const T y = S::down(float(signed_code(values, i, bit, word)) * step);
            out[idx] = accumulate ? S::down(S::up(out[idx]) + S::up(y)) : y;
        }
    }
    });
    return 0;
}

template <int DT>
int reduce(int group, int bit, bool compact, const uint8_t* const* payloads, int num, int64_t numel, float scale,
           void* out_, const void* prep_, void* res_out_) {
    using S = Src<DT>;
    using T = typename S::T;
    T* out = static_cast<T*>(out_);
    const T* prep = static_cast<const T*>(prep_);
    T* res_out = static_cast<T*>(res_out_);
    const int word = int(sizeof(T));
    const Layout lay = layout_of(numel, group, bit, word, compact);
    const float lim = bit == 8 ? 127.0f : 7.0f;
    for_group_ranges(lay.groups, [=](int64_t g_lo, int64_t g_hi) {
    float acc[64];
    for (int64_t g = g_lo; g < g_hi; ++g) {
        for (int i = 0; i < group; ++i) acc[i] = 0.0f;
        for (int r = 0; r < num; ++r) {
            T stored;
            std::memcpy(&stored, lay.meta(payloads[r], g), sizeof(T));
            const float step = S::up(stored) / lim;
            const uint8_t* values = lay.values(payloads[r], g);
            for (int i = 0; i < group; ++i)
                acc[i] = std::fmaf(float(signed_code(values, i, bit, word)), step, acc[i]);   // one rounding
        }
        for (int i = 0; i < group; ++i) {
            const int64_t idx = g * group + i;
            if (idx >= numel) break;
            const float y32 = acc[i] * scale;
            if (res_out != nullptr) res_out[idx] = S::down(S::up(prep[idx]) - y32);   // may alias prep
            if (out != nullptr) out[idx] = S::down(y32);
        }
    }
    });
    return 0;
}


// ---- general profiles: top-k outliers and 4-bit code-books -------------------------------------------
// Metadata words per group (each as wide as the source element): [scale] (+ [idx1 | idx2 << 8][top1][top2]).
inline int meta_words(int topk) { return topk == 0 ? 1 : (topk == 1 ? 3 : 4); }

// 15 code points in [-1, 1] plus +inf as the upper sentinel of the search (csrc/quantization/inner.cuh:9-96).
const float kCodebooks[4][16] = {
    {-1.0f, (float)-0.815410147, (float)-0.655160150, (float)-0.510228027, (float)-0.375324982, (float)-0.246951370,
     (float)-0.122538030, 0.0f, (float)0.122538030, (float)0.246951370, (float)0.375324982, (float)0.510228027,
     (float)0.655160150, (float)0.815410147, 1.0f, INFINITY},
    {-1.0f, (float)-0.85714286, (float)-0.71428571, (float)-0.57142857, (float)-0.42857143, (float)-0.28571429,
     (float)-0.14285714, 0.0f, (float)0.14285714, (float)0.28571429, (float)0.42857143, (float)0.57142857,
     (float)0.71428571, (float)0.85714286, 1.0f, INFINITY},
    {-1.0f, -0.5f, -0.25f, -0.125f, -0.0625f, -0.03125f, -0.015625f, 0.0f, 0.015625f, 0.03125f, 0.0625f, 0.125f,
     0.25f, 0.5f, 1.0f, INFINITY},
    {-1.0f, (float)-0.6666666666666666, -0.5f, (float)-0.3333333333333333, -0.25f, (float)-0.16666666666666666,
     -0.125f, 0.0f, 0.125f, (float)0.16666666666666666, 0.25f, (float)0.3333333333333333, 0.5f,
     (float)0.6666666666666666, 1.0f, INFINITY},
};

struct GeneralLayout {
    int64_t groups, value_bytes, meta_bytes;
    bool compact;
    int64_t values_at(int64_t g) const { return compact ? g * (value_bytes + meta_bytes) : g * value_bytes; }
    int64_t meta_at(int64_t g) const {
        return compact ? g * (value_bytes + meta_bytes) + value_bytes : groups * value_bytes + g * meta_bytes;
    }
};

template <int DT>
int quantize_general(int group, int bit, int topk, int quant_type, bool compact, const void* x_, const void* res_,
                     void* prep_, int64_t numel, uint8_t* out) {
    using S = Src<DT>;
    using T = typename S::T;
    const T* x = static_cast<const T*>(x_);
    const T* res = static_cast<const T*>(res_);
    T* prep = static_cast<T*>(prep_);
    const int word = int(sizeof(T));
    const GeneralLayout lay{(numel + group - 1) / group, int64_t(group) * bit / 8, int64_t(meta_words(topk)) * word,
                            compact};
    const bool last_wins = DT == kFP32;       // tie rule of the reference kernels: fp32 keeps the last maximum
    const float lim = bit == 8 ? 127.0f : 7.0f;
    T raw[64];
    float v[64];
    for (int64_t g = 0; g < lay.groups; ++g) {
        for (int i = 0; i < group; ++i) {
            const int64_t idx = g * group + i;
            T bits = S::down(0.0f);
            if (idx < numel) {
                bits = x[idx];
                if (res != nullptr) bits = S::down(S::up(x[idx]) + S::up(res[idx]));
                if (prep != nullptr) prep[idx] = bits;
            }
            raw[i] = bits;
            v[i] = S::up(bits);
        }
        int top_idx[2] = {0, 0};
        T top_val[2] = {S::down(0.0f), S::down(0.0f)};
        bool taken[64] = {false};
        for (int k = 0; k < topk; ++k) {
            int best = -1;
            float best_mag = -1.0f;
            for (int i = 0; i < group; ++i) {
                if (taken[i]) continue;
                const float mag = std::fabs(v[i]);
                if (mag > best_mag || (last_wins && mag == best_mag)) {
                    best_mag = mag;
                    best = i;
                }
            }
            taken[best] = true;
            top_idx[k] = best;
            top_val[k] = raw[best];
        }
        float amax = 0.0f;
        for (int i = 0; i < group; ++i) {
            if (taken[i]) v[i] = 0.0f;
            const float a = std::fabs(v[i]);
            if (a > amax) amax = a;
        }
        const T stored = S::down(amax);
        const float safe = std::fmax(S::up(stored), 1e-6f);
        int codes[64];
        if (quant_type == 0) {
            const float mul = lim / safe;
            for (int i = 0; i < group; ++i) {
                float q = std::nearbyintf(v[i] * mul);
                q = q < -lim ? -lim : (q > lim ? lim : q);
                codes[i] = int(q) & (bit == 8 ? 255 : 15);
            }
        } else {
            const float* table = kCodebooks[quant_type - 1];
            for (int i = 0; i < group; ++i) {
                const float t = v[i] / safe;
                int low = 0;                                   // entries of table[0..15) that are <= t, minus one
                while (low < 15 && table[low] <= t) ++low;
                low = low - 1 < 0 ? 0 : (low - 1 > 14 ? 14 : low - 1);
                const float gap = table[low + 1] - table[low];
                codes[i] = low + ((t - table[low]) > gap / 2 ? 1 : 0);
            }
        }
        uint8_t* values = out + lay.values_at(g);
        if (bit == 8) {
            for (int i = 0; i < group; ++i) values[wire_pos(i, word)] = uint8_t(codes[i]);
        } else {
            for (int i = 0; i < group; i += 2) values[wire_pos(i / 2, word)] = uint8_t((codes[i] << 4) | codes[i + 1]);
        }
        T meta[4] = {stored, T(0), T(0), T(0)};
        if (topk >= 1) {
            meta[1] = T(top_idx[0] | (topk == 2 ? top_idx[1] << 8 : 0));
            meta[2] = top_val[0];
            if (topk == 2) meta[3] = top_val[1];
        }
        std::memcpy(out + lay.meta_at(g), meta, size_t(meta_words(topk)) * sizeof(T));
    }
    return 0;
}

template <int DT>
int dequantize_general(int group, int bit, int topk, int quant_type, bool compact, const uint8_t* payload,
                       int64_t numel, void* out_, bool accumulate) {
    using S = Src<DT>;
    using T = typename S::T;
    T* out = static_cast<T*>(out_);
    const int word = int(sizeof(T));
    const GeneralLayout lay{(numel + group - 1) / group, int64_t(group) * bit / 8, int64_t(meta_words(topk)) * word,
                            compact};
    const float lim = bit == 8 ? 127.0f : 7.0f;
    for (int64_t g = 0; g < lay.groups; ++g) {
        T meta[4] = {T(0), T(0), T(0), T(0)};
        std::memcpy(meta, payload + lay.meta_at(g), size_t(meta_words(topk)) * sizeof(T));
        const float scale = S::up(meta[0]);
        const uint8_t* values = payload + lay.values_at(g);
        T decoded[64];
        for (int i = 0; i < group; ++i) {
            if (quant_type == 0) {
                decoded[i] = S::down(float(signed_code(values, i, bit, word)) * (scale / lim));
            } else {
                const uint8_t byte = values[wire_pos(i / 2, word)];
                const int code = (i % 2 == 0) ? (byte >> 4) : (byte & 15);
                decoded[i] = S::down(kCodebooks[quant_type - 1][code] * scale);
            }
        }
        const uint32_t index_word = uint32_t(meta[1]) & 0xFFFFu;
        for (int k = 0; k < topk; ++k) {
            const int pos = int((index_word >> (8 * k)) & 0xFFu);
            if (pos < group) decoded[pos] = meta[2 + k];      // outliers travel verbatim
        }
        for (int i = 0; i < group; ++i) {
            const int64_t idx = g * group + i;
            if (idx >= numel) break;
            out[idx] = accumulate ? S::down(S::up(out[idx]) + S::up(decoded[i])) : decoded[i];
        }
    }
    return 0;
}

bool bad_general(int dtype, int group, int bit, int topk, int quant_type) {
    if (dtype < 0 || dtype > 2 || (group != 16 && group != 32 && group != 64) || (bit != 8 && bit != 4)) return true;
    if (topk < 0 || topk > 2 || quant_type < 0 || quant_type > 4) return true;
    return quant_type != 0 && bit != 4;       // the code-books are 4-bit
}

bool bad_profile(int dtype, int group, int bit) {
    return dtype < 0 || dtype > 2 || (group != 16 && group != 32 && group != 64) || (bit != 8 && bit != 4);
}

}  // namespace

extern "C" {

int lbc_host_abi_version(void) { return 2; }

int lbc_host_quantize(int dtype, int group, int bit, int compact, const void* x, const void* residual,
                      void* prepared_out, int64_t numel, uint8_t* out) {
    if (bad_profile(dtype, group, bit) || numel < 0 || (numel > 0 && (x == nullptr || out == nullptr))) return 1;
    switch (dtype) {
        case kFP16: return quantize<kFP16>(group, bit, compact != 0, x, residual, prepared_out, numel, out);
        case kBF16: return quantize<kBF16>(group, bit, compact != 0, x, residual, prepared_out, numel, out);
        default: return quantize<kFP32>(group, bit, compact != 0, x, residual, prepared_out, numel, out);
    }
}

int lbc_host_dequantize(int dtype, int group, int bit, int compact, const uint8_t* payload, int64_t numel, void* out,
                        int accumulate) {
    if (bad_profile(dtype, group, bit) || numel < 0 || (numel > 0 && (payload == nullptr || out == nullptr))) return 1;
    switch (dtype) {
        case kFP16: return dequantize<kFP16>(group, bit, compact != 0, payload, numel, out, accumulate != 0);
        case kBF16: return dequantize<kBF16>(group, bit, compact != 0, payload, numel, out, accumulate != 0);
        default: return dequantize<kFP32>(group, bit, compact != 0, payload, numel, out, accumulate != 0);
    }
}

// out = T(sum_r decode_fp32(payload_r) * scale); optionally residual_out = T(float(prepared) - that fp32 value).
int lbc_host_reduce(int dtype, int group, int bit, int compact, const uint8_t* const* payloads, int num, int64_t numel,
                    float scale, void* out, const void* prepared, void* residual_out) {
    if (bad_profile(dtype, group, bit) || numel < 0 || num < 1 || payloads == nullptr) return 1;
    if ((prepared == nullptr) != (residual_out == nullptr)) return 1;
    switch (dtype) {
        case kFP16: return reduce<kFP16>(group, bit, compact != 0, payloads, num, numel, scale, out, prepared, residual_out);
        case kBF16: return reduce<kBF16>(group, bit, compact != 0, payloads, num, numel, scale, out, prepared, residual_out);
        default: return reduce<kFP32>(group, bit, compact != 0, payloads, num, numel, scale, out, prepared, residual_out);
    }
}

// General profiles (top-k 0..2; quant_type 0 linear, 1 normal, 2 uniform, 3 e3m0, 4 e2m1; deterministic rounding).
int lbc_host_quantize_general(int dtype, int group, int bit, int topk, int quant_type, int compact, const void* x,
                              const void* residual, void* prepared_out, int64_t numel, uint8_t* out) {
    if (bad_general(dtype, group, bit, topk, quant_type) || numel < 0 || (numel > 0 && (x == nullptr || out == nullptr)))
        return 1;
    switch (dtype) {
        case kFP16:
            return quantize_general<kFP16>(group, bit, topk, quant_type, compact != 0, x, residual, prepared_out, numel, out);
        case kBF16:
            return quantize_general<kBF16>(group, bit, topk, quant_type, compact != 0, x, residual, prepared_out, numel, out);
        default:
            return quantize_general<kFP32>(group, bit, topk, quant_type, compact != 0, x, residual, prepared_out, numel, out);
    }
}

int lbc_host_dequantize_general(int dtype, int group, int bit, int topk, int quant_type, int compact,
                                const uint8_t* payload, int64_t numel, void* out, int accumulate) {
    if (bad_general(dtype, group, bit, topk, quant_type) || numel < 0 ||
        (numel > 0 && (payload == nullptr || out == nullptr)))
        return 1;
    switch (dtype) {
        case kFP16:
            return dequantize_general<kFP16>(group, bit, topk, quant_type, compact != 0, payload, numel, out, accumulate != 0);
        case kBF16:
            return dequantize_general<kBF16>(group, bit, topk, quant_type, compact != 0, payload, numel, out, accumulate != 0);
        default:
            return dequantize_general<kFP32>(group, bit, topk, quant_type, compact != 0, payload, numel, out, accumulate != 0);
    }
}

// Element conversions, exported so that the tests can check them exhaustively.
float lbc_host_half_to_float(uint16_t h) { return half_to_float(h); }
uint16_t lbc_host_float_to_half(float f) { return float_to_half(f); }
uint16_t lbc_host_float_to_bf16(float f) { return float_to_bf16(f); }

}  // extern "C"

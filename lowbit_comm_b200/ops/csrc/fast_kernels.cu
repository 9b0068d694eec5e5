// Production-profile kernels (linear quantization, no top-k, nearest-even
// rounding) for sm_100a.  Two kernels cover the whole fused data path:
//
//   quant_push : [error-feedback add] -> group abs-max -> int8/int4 pack ->
//                stores into one or many destination payloads (local memory or
//                NVLink peer memory) -> release signal
//   reduce     : [bounded wait] -> dequantize R payloads -> fp32 sum -> scale ->
//                {dense output | residual update | requantize + broadcast
//                 into peer payloads + release signal}
//
// Math parity with the reference kernels: quantization/quant_pack_kernel.cu:84-163
// (prepared value and stored scale are rounded to the source dtype before use),
// quantization/dequant_reduce_kernel.cu:38-69, 150-221 (scale/127 decode, fp32
// accumulate, one rounding, residual = prepared - mean).
//
// Thread mapping: each thread owns 16 consecutive elements (one 16-byte vector
// of int8 codes, two 32-byte sectors of bf16), so a warp reads and writes fully
// coalesced 512 B / 1 KiB spans and a group of G elements is G/16 adjacent lanes.

#include "codec_device.cuh"
#include "common.cuh"
#include "lbc_api.h"

namespace lbc {

// ---------------------------------------------------------------------------
// quant_push
// ---------------------------------------------------------------------------
template <typename T, int G, int BIT>
__global__ void __launch_bounds__(kThreads, 4) quant_push_kernel(const LbcQuantPush p) {
    constexpr int lanes = G / kElemsPerThread;
    constexpr int VB = G * BIT / 8;                 // value bytes per group
    constexpr int MB = sizeof(T);                   // scale bytes per group
    constexpr int CB = kElemsPerThread * BIT / 8;   // code bytes per thread
    const T* x = static_cast<const T*>(p.x);
    const T* res = static_cast<const T*>(p.residual);
    T* prep = static_cast<T*>(p.prepared_out);
    T* lef = static_cast<T*>(p.local_ef_out);
    const int64_t n = p.numel;
    const int64_t num_groups = (n + G - 1) / G;
    const int64_t num_chunks = num_groups * lanes;  // 16-element chunks, whole groups only
    const bool x_vec = (reinterpret_cast<uintptr_t>(x) & 31) == 0;
    const bool r_vec = res == nullptr || (reinterpret_cast<uintptr_t>(res) & 31) == 0;
    const bool p_vec = prep == nullptr || (reinterpret_cast<uintptr_t>(prep) & 31) == 0;
    const bool l_vec = lef == nullptr || (reinterpret_cast<uintptr_t>(lef) & 31) == 0;

    __shared__ __align__(16) ScaleStage stage;
    const bool vec_scales = p.mode != LBC_PUSH_COMPACT_LOCAL && (p.layout_groups & 7) == 0 &&
                            (p.group_offset & 7) == 0 && (p.shard_groups & 7) == 0 && dsts_aligned16(p.dst, p.num_dst);
    const bool mcast = vec_scales && p.mode == LBC_PUSH_BROADCAST && p.mc_dst != nullptr;

    // Chunks are rounded up to a whole warp so that the shuffles stay convergent.
    const int64_t chunk_span = (num_chunks + 31) / 32 * 32;
    for (int64_t chunk = int64_t(blockIdx.x) * kThreads + threadIdx.x; chunk < chunk_span;
         chunk += int64_t(gridDim.x) * kThreads) {
        const bool live = chunk < num_chunks;
        const int64_t first = chunk * kElemsPerThread;
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
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.0f;
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
        amax = group_max<G>(amax);
        float stored = amax;
        if constexpr (sizeof(T) == 2) stored = Src<T>::up(Src<T>::down(amax));
        const int64_t g = chunk / lanes;
        const int lane = int(chunk - g * lanes);
        if (live) {
            if (prep != nullptr) store16<T>(prep, first, n, p_vec, v);
            float dq[16];
            const uint4 codes = encode16<T, BIT>(v, stored, lef != nullptr ? &dq : nullptr);
            if (lef != nullptr) store16<T>(lef, first, n, l_vec, dq);
            if (p.mode == LBC_PUSH_COMPACT_LOCAL) {
                uint8_t* rec = p.dst[0] + g * (VB + MB);
                store_codes(rec + lane * CB, codes, CB);
                if (lane == 0) store_scale<T>(rec + VB, stored);
            } else if (p.mode == LBC_PUSH_SCATTER) {
                const int64_t d = g / p.shard_groups;
                const int64_t gl = g - d * p.shard_groups;
                uint8_t* base = p.dst[d];
                store_codes(base + gl * VB + lane * CB, codes, CB);
                if (!vec_scales && lane == 0) store_scale<T>(base + p.layout_groups * VB + gl * MB, stored);
            } else {
                const int64_t gl = p.group_offset + g;
                if (mcast) {
                    if constexpr (CB == 16)
                        multimem_st16(p.mc_dst + gl * VB + lane * CB, codes);
                    else
                        multimem_st8(p.mc_dst + gl * VB + lane * CB, make_uint2(codes.x, codes.y));
                } else {
                    for (int d = 0; d < p.num_dst; ++d) {
                        uint8_t* base = p.dst[d];
                        store_codes(base + gl * VB + lane * CB, codes, CB);
                        if (!vec_scales && lane == 0) store_scale<T>(base + p.layout_groups * VB + gl * MB, stored);
                    }
                }
            }
        }
        if (vec_scales) {
            const int wlane = threadIdx.x & 31;
            if (lane == 0) park_scale<T>(stage, wlane / lanes, stored);   // dead groups park a zero
            __syncwarp();
            constexpr int groups_per_vec = 16 / MB;
            constexpr int vecs_per_warp = (32 / lanes) / groups_per_vec;
            const int64_t gv = (chunk - wlane) / lanes + int64_t(wlane) * groups_per_vec;  // first group of my vector
            if (wlane < vecs_per_warp && gv < num_groups) {
                const uint4 sv = *reinterpret_cast<const uint4*>(stage.bytes[threadIdx.x >> 5] + wlane * 16);
                if (p.mode == LBC_PUSH_SCATTER) {
                    const int64_t d = gv / p.shard_groups;
                    const int64_t gl = gv - d * p.shard_groups;
                    st16(p.dst[d] + p.layout_groups * VB + gl * MB, sv);
                } else {
                    const int64_t gl = p.group_offset + gv;
                    if (mcast) {
                        multimem_st16(p.mc_dst + p.layout_groups * VB + gl * MB, sv);
                    } else {
                        for (int d = 0; d < p.num_dst; ++d) st16(p.dst[d] + p.layout_groups * VB + gl * MB, sv);
                    }
                }
            }
            __syncwarp();
        }
    }
    grid_signal(p.signal);
}

// ---------------------------------------------------------------------------
// quant_push through the bulk-store engine (scatter and broadcast modes)
// ---------------------------------------------------------------------------
// A block quantizes one tile (256 threads x 16 elements) into shared memory, then one thread
// hands the tile's codes and scales to the copy engine, once per destination.  Two tile
// buffers alternate, so the engine drains tile i while the block quantizes tile i + 1.
// Tiles are dealt out shard-interleaved: consecutive tiles (and therefore the blocks running
// at any instant) target different ranks, and the rotation by the sender's rank keeps the W
// senders from converging on one receiver.
struct PushTile {
    unsigned char codes[2][kThreads * 16];
    unsigned char scales[2][kThreads * 4];   // up to 256 groups (G = 16) of 4-byte scales
};

template <typename T, int G, int BIT, bool kBulk>
// (16-bit sources hold the next tile's raw words in registers: three blocks per SM, two tiles in flight each)
__global__ void __launch_bounds__(kThreads, (kBulk || sizeof(T) == 2) ? 3 : 4)
quant_push_tiled_kernel(const LbcQuantPush p) {
    constexpr int lanes = G / kElemsPerThread;
    constexpr int VB = G * BIT / 8;
    constexpr int MB = sizeof(T);
    constexpr int CB = kElemsPerThread * BIT / 8;
    constexpr int tile_groups = kThreads / lanes;
    const T* x = static_cast<const T*>(p.x);
    const T* res = static_cast<const T*>(p.residual);
    T* prep = static_cast<T*>(p.prepared_out);
    T* lef = static_cast<T*>(p.local_ef_out);
    const int64_t n = p.numel;
    const int64_t num_groups = (n + G - 1) / G;
    const bool x_vec = (reinterpret_cast<uintptr_t>(x) & 31) == 0;
    const bool r_vec = res == nullptr || (reinterpret_cast<uintptr_t>(res) & 31) == 0;
    const bool p_vec = prep == nullptr || (reinterpret_cast<uintptr_t>(prep) & 31) == 0;
    const bool l_vec = lef == nullptr || (reinterpret_cast<uintptr_t>(lef) & 31) == 0;
    const bool scatter = p.mode == LBC_PUSH_SCATTER;
    // scatter: one destination per shard; broadcast: one "shard" that holds every group
    const int64_t span_groups = scatter ? p.shard_groups : (num_groups + 7) / 8 * 8;
    const int shards = scatter ? int((num_groups + p.shard_groups - 1) / p.shard_groups) : 1;
    const int64_t tiles_per_shard = (span_groups + tile_groups - 1) / tile_groups;
    const int64_t num_tiles = tiles_per_shard * shards;
    const int rot = p.signal.my_slot;   // this rank's index: staggers the senders

    // the bulk form stages whole tiles for the copy engine; the per-thread form only parks scales per warp
    __shared__ __align__(128) unsigned char tile_raw[kBulk ? sizeof(PushTile) : 16];
    PushTile& tile = *reinterpret_cast<PushTile*>(tile_raw);
    __shared__ __align__(16) unsigned char scale_buf[kBulk ? 1 : 2][kBulk ? 16 : kThreads * 4];
    int buf = 0;
    const int gl = int(threadIdx.x) / lanes;                        // my group inside a tile
    const int lane = int(threadIdx.x) - gl * lanes;
    // Where tile `vt` sits: its shard, its first group inside the shard, how many of its groups hold data,
    // and this thread's first element.
    struct Spot {
        int shard;
        int64_t gl0, live_groups, first;
    };
    auto spot_of = [&](int64_t vt) {
        Spot s;
        s.shard = int((vt + rot) % shards);
        s.gl0 = (vt / shards) * tile_groups;
        const int64_t shard_first = int64_t(s.shard) * span_groups;   // first group of the shard in the tensor
        s.live_groups = max(int64_t(0), min(int64_t(tile_groups), min(span_groups, num_groups - shard_first) - s.gl0));
        s.first = ((shard_first + s.gl0) * lanes + threadIdx.x) * kElemsPerThread;
        return s;
    };
    // 16-bit sources on 32-byte aligned tensors: the loads of tile i + 1 are issued before tile i is encoded,
    // so that every warp keeps 32 (with a residual 64) bytes per thread in flight while it computes; one
    // load per thread and tile left the memory system idle for about half of the time.  The raw words wait
    // in registers.  Everything else (fp32 sources, unaligned views, the ragged last tile) loads in place.
    constexpr bool kAhead = sizeof(T) == 2;
    const bool ahead_ok = kAhead && x_vec && r_vec;
    U8x32 raw_x, raw_r;
    bool raw_held = false;
    auto fetch = [&](const Spot& s) {
        raw_held = ahead_ok && gl < s.live_groups && s.first + 16 <= n;
        if (raw_held) {
            raw_x = ld32_stream(x + s.first);
            if (res != nullptr) raw_r = (prep != res) ? ld32_stream(res + s.first) : ld32(res + s.first);
        }
    };
    Spot here = spot_of(blockIdx.x);
    if (int64_t(blockIdx.x) < num_tiles) fetch(here);
    for (int64_t vt = blockIdx.x; vt < num_tiles; vt += gridDim.x, buf ^= 1) {
        const int shard = here.shard;
        const int64_t gl0 = here.gl0;
        const int64_t live_groups = here.live_groups;
        const bool live = gl < live_groups;
        const int64_t first = here.first;
        float v[16];
        if (live && raw_held) {
            if constexpr (kAhead) {
#pragma unroll
                for (int i = 0; i < 8; ++i) Src<T>::up2(raw_x.w[i], v[2 * i], v[2 * i + 1]);
                if (res != nullptr) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float a, b;
                        Src<T>::up2(raw_r.w[i], a, b);
                        v[2 * i] += a;
                        v[2 * i + 1] += b;
                    }
                    round16<T>(v);
                }
            }
        } else if (live) {
            load16<T>(x, first, n, x_vec, v, true);
            if (res != nullptr) {
                float r[16];
                load16<T>(res, first, n, r_vec, r, prep != res);
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] += r[i];
                round16<T>(v);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.0f;
        }
        if (vt + gridDim.x < num_tiles) {       // the next tile's loads go out before this one is encoded
            here = spot_of(vt + gridDim.x);
            fetch(here);
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
        amax = group_max<G>(amax);
        float stored = amax;
        if constexpr (sizeof(T) == 2) stored = Src<T>::up(Src<T>::down(amax));
        float dq[16];
        const uint4 codes = encode16<T, BIT>(v, stored, (live && lef != nullptr) ? &dq : nullptr);
        if (live) {
            if (prep != nullptr) store16<T>(prep, first, n, p_vec, v);
            if (lef != nullptr) store16<T>(lef, first, n, l_vec, dq);
        }
        const int64_t copy_groups = (live_groups + 7) / 8 * 8;   // layouts are padded to 8 groups
        if constexpr (kBulk) {
            // the engine may still be reading this buffer for the tile issued two iterations ago
            if (threadIdx.x == 0) bulk_wait_read_1();
            __syncthreads();
            if constexpr (BIT == 8)
                *reinterpret_cast<uint4*>(tile.codes[buf] + threadIdx.x * CB) = codes;
            else
                *reinterpret_cast<uint2*>(tile.codes[buf] + threadIdx.x * CB) = make_uint2(codes.x, codes.y);
            if (lane == 0) {
                if constexpr (sizeof(T) == 2)
                    *reinterpret_cast<uint16_t*>(tile.scales[buf] + gl * MB) = Src<T>::down(stored);
                else
                    *reinterpret_cast<float*>(tile.scales[buf] + gl * MB) = stored;
            }
            fence_smem_to_async_proxy();
            __syncthreads();
            if (threadIdx.x == 0 && live_groups > 0) {
                const uint32_t value_bytes = uint32_t(copy_groups * VB);
                const uint32_t scale_bytes = uint32_t(copy_groups * MB);
                if (scatter) {
                    uint8_t* base = p.dst[shard];
                    bulk_store(base + gl0 * VB, tile.codes[buf], value_bytes);
                    bulk_store(base + p.layout_groups * VB + gl0 * MB, tile.scales[buf], scale_bytes);
                } else {
                    const int64_t g_dst = p.group_offset + gl0;
                    for (int d = 0; d < p.num_dst; ++d) {
                        const int dd = (d + rot) % p.num_dst;
                        uint8_t* base = p.dst[dd];
                        bulk_store(base + g_dst * VB, tile.codes[buf], value_bytes);
                        bulk_store(base + p.layout_groups * VB + g_dst * MB, tile.scales[buf], scale_bytes);
                    }
                }
            }
            if (threadIdx.x == 0) bulk_commit();
        } else {
            // per-thread stores of the codes, scales gathered through shared memory into 16-byte vectors
            const int64_t g_dst = (scatter ? 0 : p.group_offset) + gl0;
            if (live) {
                if (scatter) {
                    store_codes(p.dst[shard] + (g_dst + gl) * VB + lane * CB, codes, CB);
                } else if (p.mc_dst != nullptr) {
                    if constexpr (CB == 16)
                        multimem_st16(p.mc_dst + (g_dst + gl) * VB + lane * CB, codes);
                    else
                        multimem_st8(p.mc_dst + (g_dst + gl) * VB + lane * CB, make_uint2(codes.x, codes.y));
                } else {
                    for (int d = 0; d < p.num_dst; ++d) {
                        const int dd = (d + rot) % p.num_dst;
                        store_codes(p.dst[dd] + (g_dst + gl) * VB + lane * CB, codes, CB);
                    }
                }
            }
            // scales: the block gathers the tile's scales in shared memory and its first threads write them
            // as consecutive 16-byte vectors, i.e. whole 128-byte lines (eight separate 16-byte stores from
            // eight warps were measured 15 % slower over NVLink).  Two buffers alternate, so one barrier per
            // tile is enough: a thread can only overwrite a buffer after the barrier of the tile in between,
            // which every reader of the older tile has reached by then.
            if (lane == 0) {
                if constexpr (sizeof(T) == 2)
                    *reinterpret_cast<uint16_t*>(scale_buf[buf] + gl * MB) = Src<T>::down(stored);
                else
                    *reinterpret_cast<float*>(scale_buf[buf] + gl * MB) = stored;
            }
            __syncthreads();
            if (int64_t(threadIdx.x) * 16 < copy_groups * MB) {
                const uint4 sv = *reinterpret_cast<const uint4*>(scale_buf[buf] + threadIdx.x * 16);
                const int64_t off = p.layout_groups * VB + g_dst * MB + threadIdx.x * 16;
                if (scatter) {
                    st16(p.dst[shard] + off, sv);
                } else if (p.mc_dst != nullptr) {
                    multimem_st16(p.mc_dst + off, sv);
                } else {
                    for (int d = 0; d < p.num_dst; ++d) st16(p.dst[(d + rot) % p.num_dst] + off, sv);
                }
            }
        }
    }
    if (kBulk && threadIdx.x == 0) bulk_wait_all();
    grid_signal(p.signal);
}

// ---------------------------------------------------------------------------
// reduce
// ---------------------------------------------------------------------------
template <typename T, int G, int BIT>
__global__ void __launch_bounds__(kThreads, 4) reduce_kernel(const LbcReduce p) {
    constexpr int lanes = G / kElemsPerThread;
    constexpr int VB = G * BIT / 8;
    constexpr int MB = sizeof(T);
    constexpr int CB = kElemsPerThread * BIT / 8;

    if (!block_wait(p.wait)) return;

    T* out = static_cast<T*>(p.out);
    const T* prep = static_cast<const T*>(p.prepared);
    T* rout = static_cast<T*>(p.residual_out);
    const int64_t n = p.numel;
    const int64_t num_groups = (n + G - 1) / G;
    const int64_t num_chunks = num_groups * lanes;
    const bool o_vec = out == nullptr || (reinterpret_cast<uintptr_t>(out) & 31) == 0;
    const bool p_vec = prep == nullptr || (reinterpret_cast<uintptr_t>(prep) & 31) == 0;
    const bool r_vec = rout == nullptr || (reinterpret_cast<uintptr_t>(rout) & 31) == 0;
    const int R = p.num_src;
    const int64_t rec = p.compact ? (VB + MB) : VB;
    __shared__ __align__(16) ScaleStage stage;
    const bool vec_scales = p.num_dst > 0 && (p.dst_layout_groups & 7) == 0 && (p.dst_group_offset & 7) == 0 &&
                            dsts_aligned16(p.dst, p.num_dst);
    // requantized tiles leave through the copy engine (a multicast destination takes precedence)
    const bool bulk = vec_scales && p.bulk_store != 0 && p.mc_dst == nullptr;
    // multicast: one multimem store per vector, replicated by the switch into every rank's region
    const bool mcast = vec_scales && !bulk && p.mc_dst != nullptr && (CB == 16 || CB == 8);
    __shared__ __align__(128) PushTile tile;
    int buf = 0;
    // whole warps keep the shuffles convergent; the bulk path also has block-wide barriers in the loop
    const int64_t span_unit = bulk ? kThreads : 32;
    const int64_t chunk_span = (num_chunks + span_unit - 1) / span_unit * span_unit;

    // Gather mode without destinations (the decode stage of the two-stage all-reduce): the sweep is dealt
    // out in 256-thread tiles that walk the shards round-robin, starting at shard `first_src`.  At any
    // instant the blocks of this GPU then read from all owners at once, and ranks that start at their own
    // index load every owner evenly even when they run skewed in time (gather_order 1).  gather_order 0
    // keeps the linear sweep, rotated to start at `first_src`: one owner at a time.
    const bool by_tiles = p.src_shard_groups > 0 && p.num_dst == 0 && p.group_offset == 0 && p.gather_order == 1;
    const int64_t shard_chunks = p.src_shard_groups * lanes;
    const int64_t tiles_per_shard = by_tiles ? (shard_chunks + kThreads - 1) / kThreads : 0;
    const int64_t loop_span = by_tiles ? tiles_per_shard * R * kThreads : chunk_span;
    int64_t rotation = 0;
    if (!by_tiles && p.src_shard_groups > 0 && p.first_src > 0 && p.num_dst == 0)
        rotation = (int64_t(p.first_src) * shard_chunks / 32 * 32) % chunk_span;

    for (int64_t it = int64_t(blockIdx.x) * kThreads + threadIdx.x; it < loop_span;
         it += int64_t(gridDim.x) * kThreads) {
        int64_t chunk;
        bool inside = true;
        if (by_tiles) {
            const int64_t tile = it / kThreads;                    // block-uniform
            const int64_t owner = (tile + p.first_src) % R;
            const int64_t within = (tile / R) * kThreads + threadIdx.x;
            inside = within < shard_chunks;
            chunk = owner * shard_chunks + within;
        } else {
            chunk = it + rotation;
            if (chunk >= chunk_span) chunk -= chunk_span;
        }
        const bool live = inside && chunk < num_chunks;
        const int64_t first = chunk * kElemsPerThread;
        const int64_t g = chunk / lanes;
        const int lane = int(chunk - g * lanes);
        const int64_t gs = p.group_offset + g;
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
        if (live) {
            int64_t voff = gs * rec + lane * CB;
            int64_t soff = p.compact ? gs * rec + VB : p.layout_groups * VB + gs * MB;
            int first_src = 0, last_src = R;
            if (p.src_shard_groups > 0) {
                // gather mode: the group lives in exactly one source, the owner's reduced shard,
                // which may be a peer's memory (the payload then crosses NVLink as this kernel's loads)
                const int64_t owner = gs / p.src_shard_groups;
                const int64_t gl = gs - owner * p.src_shard_groups;
                first_src = int(owner);
                last_src = first_src + 1;
                voff = gl * VB + lane * CB;
                soff = p.src_shard_groups * VB + gl * MB;
            }
#pragma unroll 4
            for (int r = first_src; r < last_src; ++r) {
                const uint8_t* base = p.src[r];
                const uint4 codes = load_codes(base + voff, CB);
                const float s = load_scale<T>(base + soff);
                // acc = fma(code, scale / L, acc): one rounding per payload, stated explicitly so
                // that the result does not depend on the compiler's contraction choices
                constexpr int lim = BIT == 8 ? 127 : 7;
                const float step = s / float(lim);
                float d[16];
                codes16<T, BIT>(codes, d);
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] = __fmaf_rn(d[i], step, acc[i]);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] *= p.scale;
            if (rout != nullptr) {
                float pv[16];
                load16<T>(prep, first, n, p_vec, pv, prep != rout);
#pragma unroll
                for (int i = 0; i < 16; ++i) pv[i] -= acc[i];
                store16<T>(rout, first, n, r_vec, pv);
            }
        }
        // y = T(sum * scale): the value every consumer sees
        round16<T>(acc);
        if (live && out != nullptr) {
            if (p.accumulate) {
                float prev[16];
                load16<T>(out, first, n, o_vec, prev, false);
#pragma unroll
                for (int i = 0; i < 16; ++i) prev[i] += acc[i];
                store16<T>(out, first, n, o_vec, prev);
            } else {
                store16<T>(out, first, n, o_vec, acc);
            }
        }
        if (p.num_dst > 0) {
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(acc[i]));
            amax = group_max<G>(amax);
            float stored = amax;
            if constexpr (sizeof(T) == 2) stored = Src<T>::up(Src<T>::down(amax));
            if (bulk) {
                // tile of this block iteration -> shared memory -> one bulk store per destination
                const uint4 codes = encode16<T, BIT>(acc, stored, nullptr);
                const int64_t g0 = (chunk - threadIdx.x) / lanes;
                const int tg = int(threadIdx.x) / lanes;
                int64_t live_groups = max(int64_t(0), min(int64_t(kThreads / lanes), num_groups - g0));
                if (threadIdx.x == 0) bulk_wait_read_1();
                __syncthreads();
                if constexpr (BIT == 8)
                    *reinterpret_cast<uint4*>(tile.codes[buf] + threadIdx.x * CB) = codes;
                else
                    *reinterpret_cast<uint2*>(tile.codes[buf] + threadIdx.x * CB) = make_uint2(codes.x, codes.y);
                if (lane == 0) {
                    if constexpr (sizeof(T) == 2)
                        *reinterpret_cast<uint16_t*>(tile.scales[buf] + tg * MB) = Src<T>::down(live ? stored : 0.0f);
                    else
                        *reinterpret_cast<float*>(tile.scales[buf] + tg * MB) = live ? stored : 0.0f;
                }
                fence_smem_to_async_proxy();
                __syncthreads();
                if (threadIdx.x == 0 && live_groups > 0) {
                    const int64_t copy_groups = (live_groups + 7) / 8 * 8;
                    const int64_t g_dst = p.dst_group_offset + g0;
                    for (int d = 0; d < p.num_dst; ++d) {
                        uint8_t* base = p.dst[(d + p.signal.my_slot) % p.num_dst];
                        bulk_store(base + g_dst * VB, tile.codes[buf], uint32_t(copy_groups * VB));
                        bulk_store(base + p.dst_layout_groups * VB + g_dst * MB, tile.scales[buf],
                                   uint32_t(copy_groups * MB));
                    }
                }
                if (threadIdx.x == 0) bulk_commit();
                buf ^= 1;
            } else if (live) {
                const uint4 codes = encode16<T, BIT>(acc, stored, nullptr);
                const int64_t gl = p.dst_group_offset + g;
                if (mcast) {
                    if constexpr (CB == 16)
                        multimem_st16(p.mc_dst + gl * VB + lane * CB, codes);
                    else
                        multimem_st8(p.mc_dst + gl * VB + lane * CB, make_uint2(codes.x, codes.y));
                } else {
                    for (int d = 0; d < p.num_dst; ++d) {
                        uint8_t* base = p.dst[d];
                        store_codes(base + gl * VB + lane * CB, codes, CB);
                        if (!vec_scales && lane == 0)
                            store_scale<T>(base + p.dst_layout_groups * VB + gl * MB, stored);
                    }
                }
            }
            if (vec_scales && !bulk) {
                const int wlane = threadIdx.x & 31;
                if (lane == 0) park_scale<T>(stage, wlane / lanes, live ? stored : 0.0f);
                __syncwarp();
                constexpr int groups_per_vec = 16 / MB;
                constexpr int vecs_per_warp = (32 / lanes) / groups_per_vec;
                const int64_t gv = (chunk - wlane) / lanes + int64_t(wlane) * groups_per_vec;
                if (wlane < vecs_per_warp && gv < num_groups) {
                    const uint4 sv = *reinterpret_cast<const uint4*>(stage.bytes[threadIdx.x >> 5] + wlane * 16);
                    const int64_t gl = p.dst_group_offset + gv;
                    if (mcast) {
                        multimem_st16(p.mc_dst + p.dst_layout_groups * VB + gl * MB, sv);
                    } else {
                        for (int d = 0; d < p.num_dst; ++d)
                            st16(p.dst[d] + p.dst_layout_groups * VB + gl * MB, sv);
                    }
                }
                __syncwarp();
            }
        }
    }
    if (bulk && threadIdx.x == 0) bulk_wait_all();
    grid_signal(p.signal);
}

// ---------------------------------------------------------------------------
// gather-decode with several tiles in flight
// ---------------------------------------------------------------------------
// The decode stage of the two-stage all-reduce, specialised: every group has exactly one source (its
// owner's reduced shard, in this GPU's arena or in a peer's), nothing is re-encoded and nothing is pushed.
// In `reduce_kernel` a thread has one 16-byte load in flight, and a load that crosses NVLink takes a few
// microseconds to come back, so the stage is bound by latency, not by the links.  Here a thread first
// issues the loads of U tiles (U x 16 bytes of codes and U scales in flight) and only then decodes them.
// The tiles are dealt as in `reduce_kernel`'s gather order 1: tile t belongs to owner (t + first_src) % R
// and covers chunks [(t / R) * 256, (t / R) * 256 + 256) of that owner's shard; neighbouring blocks read
// from neighbouring owners, so all owners are read at once whatever the grid.  Results are bit-identical to `reduce_kernel` (same decode, one rounding).
// Served: planar sources, group_offset 0, no destinations, no accumulation.
template <typename T, int G, int BIT, int U>
__global__ void __launch_bounds__(kThreads, U > 2 ? 3 : 4) gather_decode_kernel(const LbcReduce p) {
    constexpr int lanes = G / kElemsPerThread;
    constexpr int VB = G * BIT / 8;
    constexpr int MB = sizeof(T);
    constexpr int CB = kElemsPerThread * BIT / 8;
    constexpr int lim = BIT == 8 ? 127 : 7;

    if (!block_wait(p.wait)) return;

    T* out = static_cast<T*>(p.out);
    const T* prep = static_cast<const T*>(p.prepared);
    T* rout = static_cast<T*>(p.residual_out);
    const int64_t n = p.numel;
    const int64_t num_chunks = (n + G - 1) / G * lanes;
    const bool o_vec = out == nullptr || (reinterpret_cast<uintptr_t>(out) & 31) == 0;
    const bool p_vec = prep == nullptr || (reinterpret_cast<uintptr_t>(prep) & 31) == 0;
    const bool r_vec = rout == nullptr || (reinterpret_cast<uintptr_t>(rout) & 31) == 0;
    const int64_t R = p.num_src;
    const int64_t shard_chunks = p.src_shard_groups * lanes;
    const int64_t tiles_per_shard = (shard_chunks + kThreads - 1) / kThreads;
    const int64_t num_tiles = tiles_per_shard * R;
    const int64_t scale_base = p.src_shard_groups * VB;      // scales follow the codes in every shard payload

    for (int64_t t0 = blockIdx.x; t0 < num_tiles; t0 += int64_t(gridDim.x) * U) {
        uint4 codes[U];
        float step[U];
        int64_t first[U];          // first element of the chunk, -1 when this thread has nothing to do in tile j
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int64_t tile = t0 + int64_t(j) * gridDim.x;               // block-uniform
            const int64_t owner = (tile + p.first_src) % R;
            const int64_t within = (tile / R) * kThreads + threadIdx.x;     // chunk inside the owner's shard
            const int64_t chunk = owner * shard_chunks + within;
            const bool live = tile < num_tiles && within < shard_chunks && chunk < num_chunks;
            first[j] = live ? chunk * kElemsPerThread : int64_t(-1);
            codes[j] = make_uint4(0u, 0u, 0u, 0u);
            step[j] = 0.0f;
            if (live) {
                const int64_t gl = within / lanes;
                const int lane = int(within - gl * lanes);
                const uint8_t* base = p.src[owner];
                codes[j] = load_codes(base + gl * VB + lane * CB, CB);
                step[j] = load_scale<T>(base + scale_base + gl * MB);
            }
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (first[j] < 0) continue;
            float acc[16];
            codes16<T, BIT>(codes[j], acc);
            const float s = step[j] / float(lim);
            // the same two roundings as the general kernel with one source: fma(code, step, +0), then the scale
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = __fmul_rn(__fmaf_rn(acc[i], s, 0.0f), p.scale);
            if (rout != nullptr) {
                float pv[16];
                load16<T>(prep, first[j], n, p_vec, pv, prep != rout);
#pragma unroll
                for (int i = 0; i < 16; ++i) pv[i] -= acc[i];
                store16<T>(rout, first[j], n, r_vec, pv);
            }
            if (out != nullptr) store16<T>(out, first[j], n, o_vec, acc);   // store16 rounds to T
        }
    }
    grid_signal(p.signal);
}

// ---------------------------------------------------------------------------
// elementwise helpers
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads) ef_update_kernel(const T* prepared, const T* restored, T* residual,
                                                              int64_t n) {
    const bool vec = ((reinterpret_cast<uintptr_t>(prepared) | reinterpret_cast<uintptr_t>(restored) |
                       reinterpret_cast<uintptr_t>(residual)) & 31) == 0;
    const int64_t chunks = (n + 15) / 16;
    for (int64_t c = int64_t(blockIdx.x) * kThreads + threadIdx.x; c < chunks; c += int64_t(gridDim.x) * kThreads) {
        float a[16], b[16];
        load16<T>(prepared, c * 16, n, vec, a, true);
        load16<T>(restored, c * 16, n, vec, b, true);
#pragma unroll
        for (int i = 0; i < 16; ++i) a[i] -= b[i];
        store16<T>(residual, c * 16, n, vec, a);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) scale_kernel(T* x, float scale, int64_t n) {
    const bool vec = (reinterpret_cast<uintptr_t>(x) & 31) == 0;
    const int64_t chunks = (n + 15) / 16;
    for (int64_t c = int64_t(blockIdx.x) * kThreads + threadIdx.x; c < chunks; c += int64_t(gridDim.x) * kThreads) {
        float a[16];
        load16<T>(x, c * 16, n, vec, a, false);
#pragma unroll
        for (int i = 0; i < 16; ++i) a[i] *= scale;
        store16<T>(x, c * 16, n, vec, a);
    }
}

// ---------------------------------------------------------------------------
// transport helpers
// ---------------------------------------------------------------------------
struct PushBytesArgs {
    const uint8_t* src;
    int64_t nvec;  // 16-byte vectors
    uint8_t* dst[kMaxRanks];
    int num_dst;
    LbcWait wait;
    LbcSignal signal;
};

__global__ void __launch_bounds__(kThreads) push_bytes_kernel(const PushBytesArgs a) {
    if (!block_wait(a.wait)) return;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < a.nvec; i += int64_t(gridDim.x) * kThreads) {
        const uint4 v = ld16_stream(a.src + i * 16);
        for (int d = 0; d < a.num_dst; ++d) st16(a.dst[d] + i * 16, v);
    }
    grid_signal(a.signal);
}

struct WaitSignalArgs {
    LbcWait wait;
    LbcSignal signal;
};

__global__ void wait_signal_kernel(const WaitSignalArgs a) {
    if (!block_wait(a.wait)) return;
    grid_signal(a.signal);
}

// ---------------------------------------------------------------------------
// launch helpers
// ---------------------------------------------------------------------------
static int g_max_blocks = 0;

static int default_max_blocks() {
    if (g_max_blocks == 0) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        g_max_blocks = sms * 8;  // 8 resident 256-thread blocks per SM
    }
    return g_max_blocks;
}

static int grid_for(int64_t chunks, int max_blocks) {
    const int cap = max_blocks > 0 ? max_blocks : default_max_blocks();
    int64_t want = (chunks + kThreads - 1) / kThreads;
    if (want < 1) want = 1;
    return int(want < cap ? want : cap);
}

template <template <typename, int, int> class Launcher, typename P>
static cudaError_t dispatch(const P* p, cudaStream_t stream) {
#define LBC_CASE(TT, GG, BB)                                                        \
    if (p->group_size == GG && p->bit == BB) return Launcher<TT, GG, BB>::run(p, stream);
#define LBC_TYPE(TT)                                                                \
    LBC_CASE(TT, 64, 8) LBC_CASE(TT, 32, 8) LBC_CASE(TT, 16, 8)                     \
    LBC_CASE(TT, 64, 4) LBC_CASE(TT, 32, 4) LBC_CASE(TT, 16, 4)
    switch (p->dtype) {
        case LBC_BF16: LBC_TYPE(__nv_bfloat16) break;
        case LBC_FP16: LBC_TYPE(__half) break;
        case LBC_FP32: LBC_TYPE(float) break;
        default: break;
    }
#undef LBC_TYPE
#undef LBC_CASE
    return cudaErrorInvalidValue;
}

// The bulk-store kernel needs 16-byte aligned destinations and layouts padded to 8 groups;
// the collectives guarantee both, the local codec entry points (arbitrary payload tensors) do not.
// Push variants (identical payload layout, so ranks may even differ):
//   0 classic grid-stride kernel   1 shard-interleaved tiles, per-thread stores   2 tiles + bulk stores
static int g_push_variant = 1;
// Defaults from the 8 x B200 sweep (64-256 MiB): bulk stores and two blocks per SM for the
// requantize-and-broadcast stage were 4-8 % faster than per-thread stores on the full grid.
static int g_reduce_bulk = 1;
static int g_gather_order = 1;          // decode stage of the all-reduce: 1 = tiles round-robin over the owners, 0 = linear sweep
static int g_gather_prefetch = 0;       // decode stage: 0 = reduce_kernel, 2 or 4 = gather_decode_kernel with that many tiles in flight
static int g_reduce_push_blocks = 0;   // grid cap of reduce kernels that also push: 0 = two per SM, < 0 = none

static bool tiled_path_ok(const LbcQuantPush* p) {
    if (p->num_dst <= 0) return false;
    if (p->mode != LBC_PUSH_SCATTER && p->mode != LBC_PUSH_BROADCAST) return false;
    if ((p->layout_groups & 7) != 0 || (p->group_offset & 7) != 0) return false;
    if (p->mode == LBC_PUSH_SCATTER && (p->shard_groups & 7) != 0) return false;
    for (int d = 0; d < p->num_dst; ++d)
        if ((reinterpret_cast<uintptr_t>(p->dst[d]) & 15) != 0) return false;
    return true;
}

template <typename T, int G, int BIT>
struct QuantPushLauncher {
    static cudaError_t run(const LbcQuantPush* p, cudaStream_t stream) {
        const int64_t groups = (p->numel + G - 1) / G;
        if (groups == 0 && p->signal.num_remote == 0) return cudaSuccess;
        const int grid = grid_for(groups * (G / kElemsPerThread), p->max_blocks);
        const int variant = tiled_path_ok(p) ? g_push_variant : 0;
        if (variant == 2) {
            quant_push_tiled_kernel<T, G, BIT, true><<<grid, kThreads, 0, stream>>>(*p);
        } else if (variant == 1) {
            quant_push_tiled_kernel<T, G, BIT, false><<<grid, kThreads, 0, stream>>>(*p);
        } else {
            quant_push_kernel<T, G, BIT><<<grid, kThreads, 0, stream>>>(*p);
        }
        return cudaGetLastError();
    }
};

template <typename T, int G, int BIT>
struct ReduceLauncher {
    static cudaError_t run(const LbcReduce* p, cudaStream_t stream) {
        const int64_t groups = (p->numel + G - 1) / G;
        if (groups == 0 && p->signal.num_remote == 0 && p->wait.flags == nullptr) return cudaSuccess;
        int cap = p->max_blocks;
        if (p->num_dst > 1 && g_reduce_push_blocks >= 0) {   // several destinations: peers are among them
            const int push_cap = g_reduce_push_blocks > 0 ? g_reduce_push_blocks : default_max_blocks() / 4;
            if (cap == 0 || cap > push_cap) cap = push_cap;
        }
        const int grid = grid_for(groups * (G / kElemsPerThread), cap);
        LbcReduce launch = *p;
        if constexpr (BIT == 8) {
            const bool plain_gather = p->src_shard_groups > 0 && p->num_dst == 0 && p->group_offset == 0 &&
                                      p->accumulate == 0 && p->compact == 0;
            if (plain_gather && g_gather_prefetch >= 2) {
                if (g_gather_prefetch >= 4)
                    gather_decode_kernel<T, G, BIT, 4><<<grid, kThreads, 0, stream>>>(launch);
                else
                    gather_decode_kernel<T, G, BIT, 2><<<grid, kThreads, 0, stream>>>(launch);
                return cudaGetLastError();
            }
        }
        launch.gather_order = g_gather_order;
        launch.bulk_store = p->num_dst > 1 ? g_reduce_bulk : 0;   // a single (local) destination takes plain stores
        reduce_kernel<T, G, BIT><<<grid, kThreads, 0, stream>>>(launch);
        return cudaGetLastError();
    }
};

}  // namespace lbc

extern "C" {

int lbc_default_max_blocks(void) { return lbc::default_max_blocks(); }

void lbc_set_push_variant(int push_variant, int reduce_bulk, int reduce_push_blocks) {
    lbc::g_push_variant = push_variant < 0 ? 0 : (push_variant > 2 ? 2 : push_variant);
    lbc::g_reduce_bulk = reduce_bulk != 0;
    lbc::g_reduce_push_blocks = reduce_push_blocks;
}

void lbc_set_gather_order(int order) { lbc::g_gather_order = order != 0; }

void lbc_set_gather_prefetch(int tiles) { lbc::g_gather_prefetch = tiles >= 4 ? 4 : (tiles >= 2 ? 2 : 0); }

int lbc_get_gather_prefetch(void) { return lbc::g_gather_prefetch; }

cudaError_t lbc_quant_push(const LbcQuantPush* p, cudaStream_t stream) {
    if (p == nullptr || p->numel < 0 || p->num_dst < 0 || p->num_dst > LBC_MAX_RANKS) return cudaErrorInvalidValue;
    if (p->signal.num_remote < 0 || p->signal.num_remote > LBC_MAX_RANKS) return cudaErrorInvalidValue;
    if (p->mode == LBC_PUSH_SCATTER && p->shard_groups <= 0) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(p->mc_dst) & 15) != 0) return cudaErrorInvalidValue;
    if (p->mc_dst != nullptr && p->mode != LBC_PUSH_BROADCAST) return cudaErrorInvalidValue;
    return lbc::dispatch<lbc::QuantPushLauncher>(p, stream);
}

cudaError_t lbc_reduce(const LbcReduce* p, cudaStream_t stream) {
    if (p == nullptr || p->numel < 0 || p->num_src < 0 || p->num_src > LBC_MAX_RANKS) return cudaErrorInvalidValue;
    if (p->num_dst < 0 || p->num_dst > LBC_MAX_RANKS) return cudaErrorInvalidValue;
    if (p->signal.num_remote < 0 || p->signal.num_remote > LBC_MAX_RANKS) return cudaErrorInvalidValue;
    if (p->wait.count < 0 || p->wait.count > lbc::kThreads) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(p->mc_dst) & 15) != 0) return cudaErrorInvalidValue;
    if (p->src_shard_groups < 0 || (p->src_shard_groups > 0 && p->compact)) return cudaErrorInvalidValue;
    if (p->first_src < 0 || p->first_src > LBC_MAX_RANKS) return cudaErrorInvalidValue;
    if (p->src_shard_groups > 0 && p->numel > 0) {
        const int64_t groups = (p->numel + p->group_size - 1) / p->group_size;
        if ((p->group_offset + groups - 1) / p->src_shard_groups >= p->num_src) return cudaErrorInvalidValue;
    }
    return lbc::dispatch<lbc::ReduceLauncher>(p, stream);
}

cudaError_t lbc_error_feedback_update(int dtype, const void* prepared, const void* restored, void* residual,
                                      int64_t numel, cudaStream_t stream) {
    if (numel <= 0) return numel == 0 ? cudaSuccess : cudaErrorInvalidValue;
    const int grid = lbc::grid_for((numel + 15) / 16, 0);
    switch (dtype) {
        case LBC_BF16:
            lbc::ef_update_kernel<__nv_bfloat16><<<grid, lbc::kThreads, 0, stream>>>(
                static_cast<const __nv_bfloat16*>(prepared), static_cast<const __nv_bfloat16*>(restored),
                static_cast<__nv_bfloat16*>(residual), numel);
            break;
        case LBC_FP16:
            lbc::ef_update_kernel<__half><<<grid, lbc::kThreads, 0, stream>>>(
                static_cast<const __half*>(prepared), static_cast<const __half*>(restored),
                static_cast<__half*>(residual), numel);
            break;
        case LBC_FP32:
            lbc::ef_update_kernel<float><<<grid, lbc::kThreads, 0, stream>>>(
                static_cast<const float*>(prepared), static_cast<const float*>(restored),
                static_cast<float*>(residual), numel);
            break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t lbc_scale_inplace(int dtype, void* x, float scale, int64_t numel, cudaStream_t stream) {
    if (numel <= 0) return numel == 0 ? cudaSuccess : cudaErrorInvalidValue;
    const int grid = lbc::grid_for((numel + 15) / 16, 0);
    switch (dtype) {
        case LBC_BF16:
            lbc::scale_kernel<__nv_bfloat16><<<grid, lbc::kThreads, 0, stream>>>(static_cast<__nv_bfloat16*>(x), scale, numel);
            break;
        case LBC_FP16:
            lbc::scale_kernel<__half><<<grid, lbc::kThreads, 0, stream>>>(static_cast<__half*>(x), scale, numel);
            break;
        case LBC_FP32:
            lbc::scale_kernel<float><<<grid, lbc::kThreads, 0, stream>>>(static_cast<float*>(x), scale, numel);
            break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t lbc_push_bytes(const uint8_t* src, int64_t nbytes, uint8_t* const* dst, int num_dst,
                           const LbcWait* wait_before, const LbcSignal* signal, int max_blocks,
                           cudaStream_t stream) {
    if (nbytes < 0 || (nbytes & 15) != 0 || num_dst < 0 || num_dst > LBC_MAX_RANKS) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(src) & 15) != 0) return cudaErrorInvalidValue;
    lbc::PushBytesArgs a{};
    a.src = src;
    a.nvec = nbytes / 16;
    a.num_dst = num_dst;
    for (int d = 0; d < num_dst; ++d) {
        if ((reinterpret_cast<uintptr_t>(dst[d]) & 15) != 0) return cudaErrorInvalidValue;
        a.dst[d] = dst[d];
    }
    if (wait_before != nullptr) a.wait = *wait_before;
    if (signal != nullptr) a.signal = *signal;
    if (a.wait.count < 0 || a.wait.count > lbc::kThreads) return cudaErrorInvalidValue;
    const int grid = lbc::grid_for(a.nvec, max_blocks);
    lbc::push_bytes_kernel<<<grid, lbc::kThreads, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t lbc_wait_signal(const LbcWait* wait, const LbcSignal* signal, cudaStream_t stream) {
    lbc::WaitSignalArgs a{};
    if (wait != nullptr) a.wait = *wait;
    if (signal != nullptr) a.signal = *signal;
    if (a.wait.count < 0 || a.wait.count > 32) return cudaErrorInvalidValue;
    // one warp: it fits beside the resident blocks of a persistent kernel of another stream
    lbc::wait_signal_kernel<<<1, 32, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // extern "C"

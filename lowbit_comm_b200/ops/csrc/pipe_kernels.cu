// Fused compressed all-reduce for sm_100a: ONE persistent kernel per collective.
//
// Work unit: a row of 4096 elements (256 threads x 16).  Three phases, each a sweep over rows:
//   QUANT   x (+ residual) -> int8/int4 groups + scales, written into this rank's own arena
//   REDUCE  the owner of a shard pulls the row from all W ranks (bulk asynchronous loads over NVLink,
//           `cp.async.bulk` global -> shared, no multicast, no tensor map), sums it in fp32 and
//           requantizes it into its own arena (stages == 1: every rank reduces every row and writes
//           the result instead)
//   DECODE  every rank pulls the reduced row from its owner and decodes it into the output, updating
//           the error-feedback residual
// All cross-GPU traffic is loads issued by the copy engine of the SM into a ring of shared-memory
// stages (as many rows in flight per block as two blocks per SM leave room for), so neither the
// load/store pipeline nor the register file limits the bytes in flight over NVLink; flags are the
// only remote stores.
//
// Scheduling is static: block b takes rows b, b + grid, ... of every phase, so a row costs no atomics and
// no bookkeeping beyond a few integer operations, and one lane issues the loads of the row that is
// ring-depth rows ahead before the block computes the current one.  (Two dynamic schedules were built
// and measured first -- a ticket counter with a helper warp, and one with the duties shared among the
// computing warps; on a B200 both spent more time handing out rows than computing them: 2700-3300 cycles
// per row against 1000-1300 of arithmetic.)  Between phases the ranks meet through one epoch flag per
// (rank, phase): a block counts itself done on a local counter, the last block of the grid raises this
// rank's flag on every rank, and every block's first warp waits (bounded) for the flags of the ranks it
// is going to read from.  The grid must therefore be co-resident; the launcher sizes it from the
// occupancy of the kernel, and one GPU must not run two of these kernels at once.
//
// Every wait (phase flags, load completion barriers) is bounded: when it runs out the kernel records
// where in the status word, waits (bounded again) for its own loads in flight and returns.
//
// Math is identical, bit for bit, to quant_push_kernel / reduce_kernel (fast_kernels.cu).
// The reference runs the same algorithm as quantize -> NCCL all_to_all -> dequantize-reduce ->
// quantize -> NCCL all_gather -> dequantize (ccdl_comm/communication/reduce_scatter_transport.py:186-377).

#include "codec_device.cuh"
#include "common.cuh"
#include "lbc_api.h"

namespace lbc {

constexpr int kRow = kThreads * kElemsPerThread;   // 4096 elements
constexpr int kMaxRing = 8;
constexpr unsigned int kPhasePipeFlag = 8u;        // status.phase values 8..10: flag wait of QUANT/REDUCE/DECODE rows
constexpr unsigned int kPhasePipeLoad = 12u;       // status.phase: a bulk load that never completed

enum PipeKind : int { kQuant = 0, kReduce = 1, kDecode = 2 };

struct PipeItem {
    int kind;
    int shard;        // QUANT: destination shard; REDUCE: this rank's shard; DECODE: owner of the row
    int live;         // groups of the row that hold data (0: a padding row, nothing to do)
    int copy;         // live rounded up to 8 groups: what the bulk loads move
    int dense_tma;    // the dense row (x / residual / prepared) comes through the copy engine
    int gl0;          // first group of the row inside its shard
    long long first;      // first element of the row inside the tensor
    long long code_off;   // REDUCE / DECODE: arena offset of the row's codes ...
    long long scale_off;  // ... and of its scales
};

// ---------------------------------------------------------------------------
// mbarrier + bulk load helpers (shared::cta barriers, transaction counts in bytes)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned int parity) {
    unsigned int ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0u;
}
// Non-blocking look at a phase (`try_wait` may suspend the thread for a while before it answers "not yet").
__device__ __forceinline__ bool mbar_test_wait(unsigned long long* bar, unsigned int parity) {
    unsigned int ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0u;
}
// global (own or peer memory) -> this block's shared memory; completion is counted in bytes on `bar`
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, unsigned int bytes,
                                          unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
// Polling a flag with acquire loads from every waiting block slowed the whole GPU down (measured: a
// collective that takes 100 us took 3 ms); flags are polled with relaxed loads and one fence orders
// the loads that follow once the flag has been seen.
__device__ __forceinline__ unsigned int ld_relaxed_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

template <typename T>
__device__ __forceinline__ void load16_smem(const unsigned char* row, float (&out)[16]) {
    const unsigned char* p = row + threadIdx.x * (16 * sizeof(T));
    if constexpr (sizeof(T) == 2) {
        const uint4 a = *reinterpret_cast<const uint4*>(p);
        const uint4 b = *reinterpret_cast<const uint4*>(p + 16);
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) Src<T>::up2(w[i], out[2 * i], out[2 * i + 1]);
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 a = *reinterpret_cast<const uint4*>(p + 16 * q);
            out[4 * q] = __uint_as_float(a.x);
            out[4 * q + 1] = __uint_as_float(a.y);
            out[4 * q + 2] = __uint_as_float(a.z);
            out[4 * q + 3] = __uint_as_float(a.w);
        }
    }
}

template <int CB>
__device__ __forceinline__ uint4 codes_smem(const unsigned char* codes) {
    if constexpr (CB == 16) {
        return *reinterpret_cast<const uint4*>(codes + threadIdx.x * 16);
    } else {
        const uint2 h = *reinterpret_cast<const uint2*>(codes + threadIdx.x * 8);
        return make_uint4(h.x, h.y, 0u, 0u);
    }
}

template <int CB>
__device__ __forceinline__ void codes_to_global(uint8_t* dst, uint4 codes) {
    if constexpr (CB == 16)
        st16(dst, codes);
    else
        *reinterpret_cast<uint2*>(dst) = make_uint2(codes.x, codes.y);
}

// The warp's scales leave as 16-byte vectors (see ScaleStage); `group0` is the first group of the row
// inside the destination layout, `copy` the number of groups (a multiple of 8) the row may write.
template <typename T, int G>
__device__ __forceinline__ void store_row_scales(ScaleStage& stage, uint8_t* scale_base, int64_t group0, int copy,
                                                 bool live, float stored) {
    constexpr int lanes = G / kElemsPerThread;
    constexpr int MB = sizeof(T);
    constexpr int groups_per_vec = 16 / MB;
    constexpr int vecs_per_warp = (32 / lanes) / groups_per_vec;
    const int wlane = threadIdx.x & 31;
    if ((threadIdx.x % lanes) == 0) park_scale<T>(stage, wlane / lanes, live ? stored : 0.0f);
    __syncwarp();
    const int gv = int(threadIdx.x >> 5) * (32 / lanes) + wlane * groups_per_vec;   // first group of my vector in the row
    if (wlane < vecs_per_warp && gv < copy) {
        const uint4 sv = *reinterpret_cast<const uint4*>(stage.bytes[threadIdx.x >> 5] + wlane * 16);
        st16(scale_base + (group0 + gv) * MB, sv);
    }
    __syncwarp();
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <typename T, int G, int BIT>
__global__ void __launch_bounds__(kThreads, 2) pipe_allreduce_kernel(const __grid_constant__ LbcPipe p) {
    constexpr int lanes = G / kElemsPerThread;
    constexpr int VB = G * BIT / 8;
    constexpr int MB = sizeof(T);
    constexpr int CB = kElemsPerThread * BIT / 8;
    constexpr int RG = kRow / G;                        // groups per row
    constexpr int RC = RG * VB;                         // code bytes per row
    constexpr int RS = RG * MB;                         // scale bytes per row
    constexpr int SUB = (RC + RS + 127) / 128 * 128;    // one source's payload row inside a stage
    constexpr int RX = kRow * int(sizeof(T));           // a dense row
    constexpr int lim = BIT == 8 ? 127 : 7;

    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ __align__(8) unsigned long long full_bar[kMaxRing];    // a row's bytes have landed
    __shared__ __align__(8) unsigned long long empty_bar[kMaxRing];   // all eight warps have left a row
    __shared__ int s_fail;                              // a wait ran out
    __shared__ __align__(16) ScaleStage scale_stage;

    const int W = p.world, me = p.rank;
    const bool two = p.stages == 2;
    const int shards = two ? W : 1;
    const int64_t SG = p.shard_groups;
    const int64_t n = p.numel;
    const int64_t num_groups = (n + G - 1) / G;
    const int shard_rows = int((SG + RG - 1) / RG);
    const int S = p.ring_depth;
    const int stage_bytes = p.stage_bytes;
    const int wlane = threadIdx.x & 31;
    const bool first_warp = threadIdx.x < 32;

    const T* x = static_cast<const T*>(p.x);
    const T* res = static_cast<const T*>(p.residual);
    T* prep_out = static_cast<T*>(p.prepared_out);
    T* lef = static_cast<T*>(p.local_ef_out);
    const T* prep = static_cast<const T*>(p.prepared);
    T* rout = static_cast<T*>(p.residual_out);
    T* out = static_cast<T*>(p.out);
    const bool x_vec = (reinterpret_cast<uintptr_t>(x) & 31) == 0;
    const bool r_vec = res == nullptr || (reinterpret_cast<uintptr_t>(res) & 31) == 0;
    const bool po_vec = prep_out == nullptr || (reinterpret_cast<uintptr_t>(prep_out) & 31) == 0;
    const bool l_vec = lef == nullptr || (reinterpret_cast<uintptr_t>(lef) & 31) == 0;
    const bool pi_vec = prep == nullptr || (reinterpret_cast<uintptr_t>(prep) & 31) == 0;
    const bool ro_vec = rout == nullptr || (reinterpret_cast<uintptr_t>(rout) & 31) == 0;
    const bool o_vec = out == nullptr || (reinterpret_cast<uintptr_t>(out) & 31) == 0;
    // the copy engine wants 16-byte aligned sources
    const bool quant_tma_ok = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(res) & 15) == 0;
    const bool prep_tma_ok = (reinterpret_cast<uintptr_t>(prep) & 15) == 0;

    uint8_t* my_arena = p.arena[me];
    unsigned char* ctl = my_arena + p.ctl_off;
    const unsigned int* flags_quant = reinterpret_cast<const unsigned int*>(ctl + LBC_PIPE_CTL_FLAGS_QUANT);
    const unsigned int* flags_reduce = reinterpret_cast<const unsigned int*>(ctl + LBC_PIPE_CTL_FLAGS_REDUCE);
    unsigned int* done_count = reinterpret_cast<unsigned int*>(ctl + LBC_PIPE_CTL_LOCAL) + 2;   // [kind]: blocks done
    volatile DeviceStatus* status = static_cast<volatile DeviceStatus*>(p.status);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxRing; ++s) {
            mbar_init(&full_bar[s], 1u);
            mbar_init(&empty_bar[s], (unsigned int)(kThreads / 32));
        }
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    auto vload = [](const int* w) -> int { return *reinterpret_cast<const volatile int*>(w); };
    auto vstore = [](int* w, int v) { *reinterpret_cast<volatile int*>(w) = v; };

    // Position inside a phase's sweep.  A block's rows are `gridDim.x` apart, so the position is stepped with
    // a few 32-bit additions per row; nothing is divided in the row loop.
    //   QUANT : row r = shard * shard_rows + row     (a shard's rows are neighbours in memory)
    //   REDUCE: row r = row of this rank's shard
    //   DECODE: row r = row * W + k, owner (k + me) % W   (neighbouring rows come from different owners, and
    //           every rank starts its sweep at itself)
    struct Cursor {
        int shard, row, k;
    };
    const int num_groups_i = int(num_groups), SG_i = int(SG);       // group counts fit 32 bits
    auto cursor_at = [&](int kind, int r) -> Cursor {
        Cursor c;
        if (kind == kQuant) { c.shard = r / shard_rows; c.row = r - c.shard * shard_rows; c.k = 0; }
        else if (kind == kReduce) { c.shard = two ? me : 0; c.row = r; c.k = 0; }
        else { c.row = r / W; c.k = r - c.row * W; c.shard = (c.k + me) % W; }
        return c;
    };
    const int step = int(gridDim.x);
    const int step_shards = step / shard_rows, step_rows = step - step_shards * shard_rows;   // QUANT
    const int step_w_rows = step / W, step_w_k = step - step_w_rows * W;                      // DECODE
    auto advance = [&](int kind, Cursor& c) {
        if (kind == kQuant) {
            c.shard += step_shards;
            c.row += step_rows;
            if (c.row >= shard_rows) { c.row -= shard_rows; ++c.shard; }
        } else if (kind == kReduce) {
            c.row += step;
        } else {
            c.row += step_w_rows;
            c.k += step_w_k;
            if (c.k >= W) { c.k -= W; ++c.row; }
            c.shard = c.k + me;
            if (c.shard >= W) c.shard -= W;
        }
    };
    // what the computing threads need to know about a row
    auto item_at = [&](int kind, const Cursor& c) -> PipeItem {
        PipeItem it;
        it.kind = kind;
        it.shard = c.shard;
        it.gl0 = c.row * RG;
        int valid = num_groups_i - c.shard * SG_i;
        valid = valid < 0 ? 0 : (valid > SG_i ? SG_i : valid);
        int live = valid - it.gl0;
        live = live < 0 ? 0 : (live > RG ? RG : live);
        it.live = live;
        it.copy = (live + 7) / 8 * 8;
        it.first = int64_t(c.shard * SG_i + it.gl0) * G;
        // a dense row goes through the copy engine when its source is 16-byte aligned and no group of it is cut
        // by the end of the tensor; the other rows are read with plain guarded loads
        const bool whole = it.first + int64_t(live) * G <= n;
        if (kind == kQuant) it.dense_tma = (quant_tma_ok && whole) ? 1 : 0;
        else it.dense_tma = (prep != nullptr && (kind == kDecode || !two) && prep_tma_ok && whole) ? 1 : 0;
        it.code_off = it.scale_off = 0;
        return it;
    };
    // ... and what the issuing lanes need on top of that
    auto with_sources = [&](PipeItem it) -> PipeItem {
        if (it.kind != kQuant) {
            const int64_t region = it.kind == kReduce ? p.q_off + int64_t(it.shard) * p.shard_stride : p.ag_off;
            it.code_off = region + int64_t(it.gl0) * VB;
            it.scale_off = region + SG * VB + int64_t(it.gl0) * MB;
        }
        return it;
    };

    // Hands a row's loads to the copy engine (first warp; lane 0 arms the barrier, a REDUCE row spreads its
    // sources over the lanes).
    auto issue_row = [&](const PipeItem& it, int slot) {
        unsigned long long* bar = &full_bar[slot];
        unsigned char* base = ring + size_t(slot) * stage_bytes;
        if (it.live == 0) {                             // padding row: nothing to move, the barrier still turns
            if (wlane == 0) mbar_expect_tx(bar, 0u);
            return;
        }
        const unsigned int dense_bytes = it.dense_tma ? (unsigned int)(it.live) * G * sizeof(T) : 0u;
        const unsigned int code_bytes = (unsigned int)(it.copy) * VB, scale_bytes = (unsigned int)(it.copy) * MB;
        if (it.kind == kReduce) {
            if (wlane == 0) mbar_expect_tx(bar, (unsigned int)(W) * (code_bytes + scale_bytes) + dense_bytes);
            __syncwarp();
            if (wlane < W) {
                unsigned char* dst = base + wlane * SUB;
                bulk_load(dst, p.arena[wlane] + it.code_off, code_bytes, bar);
                bulk_load(dst + RC, p.arena[wlane] + it.scale_off, scale_bytes, bar);
            }
            if (wlane == 0 && it.dense_tma) bulk_load(base + W * SUB, prep + it.first, dense_bytes, bar);
        } else if (wlane == 0) {
            if (it.kind == kQuant) {
                mbar_expect_tx(bar, dense_bytes * (res != nullptr ? 2u : 1u));
                if (it.dense_tma) {
                    bulk_load(base, x + it.first, dense_bytes, bar);
                    if (res != nullptr) bulk_load(base + RX, res + it.first, dense_bytes, bar);
                }
            } else {
                const uint8_t* owner = p.arena[it.shard];
                mbar_expect_tx(bar, code_bytes + scale_bytes + dense_bytes);
                bulk_load(base, owner + it.code_off, code_bytes, bar);
                bulk_load(base + RC, owner + it.scale_off, scale_bytes, bar);
                if (it.dense_tma) bulk_load(base + SUB, prep + it.first, dense_bytes, bar);
            }
        }
        __syncwarp();
    };

    // optional cycle accounting (thread 0), per block: [0] rows  [1] waiting for a row's bytes  [2] computing
    // [3] at the barrier that ends a phase  [4] waiting for the other ranks' phase flags  [5] publishing phases
    // [6] total  [7] leaving rows and (every eighth row) handing a row to the copy engine
    const bool prof = p.profile != nullptr && threadIdx.x == 0;
    long long pc_wait = 0, pc_work = 0, pc_bar = 0, pc_flags = 0, pc_pub = 0, pc_rows = 0, pc_issue = 0;
    const long long pc_start = clock64();

    int consumed = 0;                                   // rows this block has been through: slot and parity of the ring
    bool failed = false;
    for (int kind = kQuant; kind <= kDecode && !failed; ++kind) {
        if (((p.phase_mask >> kind) & 1) == 0 || (kind == kDecode && !two)) continue;
        const int total = kind == kQuant ? shard_rows * shards : (kind == kReduce ? shard_rows : shard_rows * W);
        const int first_row = blockIdx.x;
        const int count = total > first_row ? (total - first_row + int(gridDim.x) - 1) / int(gridDim.x) : 0;
        const int consumed_at_phase_start = consumed;

        // ---- the other ranks' flags: QUANT of all ranks before REDUCE, REDUCE of all owners before DECODE ----
        if (kind != kQuant) {
            const long long pc_t0 = prof ? clock64() : 0;
            if (first_warp) {
                const unsigned int* flags = kind == kReduce ? flags_quant : flags_reduce;
                const unsigned long long t0 = global_ns();
                unsigned int spins = 0, seen = p.epoch;
                for (;;) {
                    seen = p.epoch;
                    if (wlane < W) seen = ld_relaxed_sys(flags + wlane * LBC_PIPE_FLAG_STRIDE);
                    const unsigned int late = __ballot_sync(0xffffffffu, int(seen - p.epoch) < 0);
                    if (late == 0u) break;
                    if ((++spins & 1023u) == 0) {       // the status word lives in host memory: look rarely
                        const bool failed_before = status != nullptr && status->code != 0u;
                        const bool too_long = global_ns() - t0 > p.timeout_ns;
                        if (failed_before || too_long) {
                            const int peer = __ffs(late) - 1;
                            const unsigned int peer_seen = __shfl_sync(0xffffffffu, seen, peer);
                            if (too_long && !failed_before && wlane == 0 && status != nullptr) {
                                status->phase = kPhasePipeFlag + (unsigned int)kind;
                                status->peer = (unsigned int)peer;
                                status->seen = peer_seen;
                                status->expected = p.epoch;
                                __threadfence_system();
                                status->code = 1u;
                                __threadfence_system();
                            }
                            if (wlane == 0) s_fail = 1;
                            break;
                        }
                    }
                    __nanosleep(spins < 64u ? 100 : 500);
                }
                fence_acq_rel_sys();                    // the rows behind the flags are visible from here on ...
                fence_async_global();                   // ... also to the bulk loads (another memory proxy)
            }
            __syncthreads();
            if (prof) pc_flags += clock64() - pc_t0;
            if (s_fail != 0) {
                failed = true;
                break;
            }
        }

        // ---- the sweep ----
        // S rows are in flight.  The eight warps walk the rows at their own pace: a warp waits for a row's bytes,
        // computes its 512 elements and arrives on the slot's "empty" barrier; there is no block barrier per
        // row.  Handing a row to the copy engine costs one warp several hundred cycles, so that duty rotates:
        // warp i % 8 waits until all eight have left row i and issues row i + S into the freed slot, while the
        // other seven are already at work on the rows behind it.
        Cursor here = cursor_at(kind, first_row), ahead = here;   // the row being computed, the next row to issue
        if (first_warp) {
            for (int k = 0; k < S && k < count; ++k) {
                issue_row(with_sources(item_at(kind, ahead)), (consumed + k) % S);
                advance(kind, ahead);
            }
        } else {
            for (int k = 0; k < S && k < count; ++k) advance(kind, ahead);
        }
        const int warp = threadIdx.x >> 5;
        for (int i = 0; i < count; ++i) {
            const long long pc_t0 = prof ? clock64() : 0;
            const int slot = consumed % S;
            const PipeItem it = item_at(kind, here);
            advance(kind, here);
            const unsigned char* base = ring + size_t(slot) * stage_bytes;
            const unsigned int parity = (unsigned int)(consumed / S) & 1u;
            bool arrived = mbar_try_wait(&full_bar[slot], parity);
            if (!arrived) {
                const unsigned long long t0 = global_ns();
                unsigned int spins = 0;
                while (!(arrived = mbar_try_wait(&full_bar[slot], parity))) {
                    if ((++spins & 63u) == 0 && (global_ns() - t0 > p.timeout_ns || vload(&s_fail) != 0)) break;
                }
            }
            arrived = __all_sync(0xffffffffu, arrived) != 0;   // the row's math shuffles across the whole warp
            if (!arrived) {
                if (wlane == 0 && vload(&s_fail) == 0) {
                    if (status != nullptr && status->code == 0u) {
                        status->phase = kPhasePipeLoad;
                        status->peer = (unsigned int)it.shard;
                        status->seen = (unsigned int)it.kind;
                        status->expected = p.epoch;
                        __threadfence_system();
                        status->code = 1u;
                        __threadfence_system();
                    }
                    vstore(&s_fail, 1);
                }
                break;
            }
            const long long pc_t1 = prof ? clock64() : 0;
            if (it.live != 0) {
                const int gl = int(threadIdx.x) / lanes;           // my group inside the row
                const int lane = int(threadIdx.x) - gl * lanes;
                const bool live = gl < it.live;
                const int64_t first = it.first + int64_t(threadIdx.x) * kElemsPerThread;
                if (it.kind == kQuant) {
                    float v[16];
                    if (live) {
                        if (it.dense_tma) {
                            load16_smem<T>(base, v);
                            if (res != nullptr) {
                                float r[16];
                                load16_smem<T>(base + RX, r);
#pragma unroll
                                for (int i = 0; i < 16; ++i) v[i] += r[i];
                                round16<T>(v);
                            }
                        } else {
                            load16<T>(x, first, n, x_vec, v, true);
                            if (res != nullptr) {
                                float r[16];
                                load16<T>(res, first, n, r_vec, r, prep_out != res);
#pragma unroll
                                for (int i = 0; i < 16; ++i) v[i] += r[i];
                                round16<T>(v);
                            }
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
                    float dq[16];
                    const uint4 codes = encode16<T, BIT>(v, stored, (live && lef != nullptr) ? &dq : nullptr);
                    uint8_t* payload = my_arena + p.q_off + int64_t(it.shard) * p.shard_stride;
                    if (live) {
                        if (prep_out != nullptr) store16<T>(prep_out, first, n, po_vec, v);
                        if (lef != nullptr) store16<T>(lef, first, n, l_vec, dq);
                        codes_to_global<CB>(payload + int64_t(it.gl0 + gl) * VB + lane * CB, codes);
                    }
                    store_row_scales<T, G>(scale_stage, payload + SG * VB, it.gl0, it.copy, live, stored);
                } else {
                    float acc[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
                    if (live) {
                        const int srcs = it.kind == kReduce ? W : 1;
                        for (int r = 0; r < srcs; ++r) {
                            const unsigned char* sub = base + r * SUB;
                            const uint4 codes = codes_smem<CB>(sub);
                            float s;
                            if constexpr (sizeof(T) == 2)
                                s = Src<T>::up(*reinterpret_cast<const uint16_t*>(sub + RC + gl * MB));
                            else
                                s = *reinterpret_cast<const float*>(sub + RC + gl * MB);
                            const float step = s / float(lim);
                            float d[16];
                            codes16<T, BIT>(codes, d);
#pragma unroll
                            for (int i = 0; i < 16; ++i) acc[i] = __fmaf_rn(d[i], step, acc[i]);
                        }
                        if (it.kind == kReduce) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) acc[i] *= p.scale;
                        }
                    }
                    const bool final_row = it.kind == kDecode || !two;   // writes the output and the residual
                    if (final_row) {
                        if (live) {
                            if (rout != nullptr) {
                                float pv[16];
                                if (it.dense_tma)
                                    load16_smem<T>(base + (it.kind == kReduce ? W : 1) * SUB, pv);
                                else
                                    load16<T>(prep, first, n, pi_vec, pv, prep != rout);
#pragma unroll
                                for (int i = 0; i < 16; ++i) pv[i] -= acc[i];
                                store16<T>(rout, first, n, ro_vec, pv);
                            }
                            store16<T>(out, first, n, o_vec, acc);   // rounds to T
                        }
                    } else {
                        round16<T>(acc);                              // y = T(sum * scale): what every rank will see
                        float amax = 0.0f;
#pragma unroll
                        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(acc[i]));
                        amax = group_max<G>(amax);
                        float stored = amax;
                        if constexpr (sizeof(T) == 2) stored = Src<T>::up(Src<T>::down(amax));
                        const uint4 codes = encode16<T, BIT>(acc, stored, nullptr);
                        uint8_t* payload = my_arena + p.ag_off;
                        if (live) codes_to_global<CB>(payload + int64_t(it.gl0 + gl) * VB + lane * CB, codes);
                        store_row_scales<T, G>(scale_stage, payload + SG * VB, it.gl0, it.copy, live, stored);
                    }
                }
            }
            const long long pc_t2 = prof ? clock64() : 0;
            __syncwarp();                               // this warp's stores of the row are issued
            if (wlane == 0) mbar_arrive(&empty_bar[slot]);
            if (i + S < count && warp == (i & 7)) {     // my turn: refill the slot with row i + S once all have left it
                bool freed = mbar_try_wait(&empty_bar[slot], parity);
                if (!freed) {
                    const unsigned long long t0 = global_ns();
                    unsigned int spins = 0;
                    while (!(freed = mbar_try_wait(&empty_bar[slot], parity))) {
                        if ((++spins & 63u) == 0 && (global_ns() - t0 > p.timeout_ns || vload(&s_fail) != 0)) break;
                    }
                }
                if (__all_sync(0xffffffffu, freed) == 0) {
                    if (wlane == 0) vstore(&s_fail, 1);   // a warp never left the row: its own wait says why
                    break;
                }
                issue_row(with_sources(item_at(kind, ahead)), slot);
            }
            advance(kind, ahead);
            ++consumed;
            if (prof) {
                const long long pc_t3 = clock64();
                pc_wait += pc_t1 - pc_t0; pc_work += pc_t2 - pc_t1; pc_issue += pc_t3 - pc_t2; ++pc_rows;
            }
        }
        // every warp is through with the phase's rows (or a wait ran out)
        {
            const long long pc_t0 = prof ? clock64() : 0;
            __syncthreads();
            if (prof) pc_bar += clock64() - pc_t0;
        }
        if (s_fail != 0) {
            failed = true;
            // loads may still be in flight: give them a bounded time to land before this block's shared memory is
            // handed to another block (a load from a rank that is gone never lands; nothing more can be done)
            if (threadIdx.x == 0) {
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 100000ull) __nanosleep(1000);
            }
            __syncthreads();
            break;
        }
        // `consumed` is the same in every warp again: count rows of the phase
        consumed = consumed_at_phase_start + count;
        if (failed) break;

        // ---- this block is through with the phase; the last block of the grid tells every rank ----
        if (kind == kQuant || (kind == kReduce && two)) {
            const long long pc_t0 = prof ? clock64() : 0;
            if (first_warp) {
                unsigned int prev = 0;
                if (wlane == 0) {
                    // device scope is enough here (and far cheaper than system scope): the one block that raises
                    // the flags fences at system scope after it has seen everybody's count, which orders all the
                    // rows of all blocks before the flags
                    __threadfence();
                    prev = atomicAdd(done_count + kind, 1u);
                }
                prev = __shfl_sync(0xffffffffu, prev, 0);
                if (prev == gridDim.x - 1) {
                    if (wlane == 0) {
                        done_count[kind] = 0u;          // ready for the next collective
                        __threadfence_system();
                    }
                    __syncwarp();
                    if (wlane < W) {
                        const int64_t off = p.ctl_off + (kind == kQuant ? LBC_PIPE_CTL_FLAGS_QUANT : LBC_PIPE_CTL_FLAGS_REDUCE) +
                                            int64_t(me) * LBC_PIPE_FLAG_STRIDE * 4;
                        st_release_sys(reinterpret_cast<unsigned int*>(p.arena[wlane] + off), p.epoch);
                    }
                }
            }
            if (prof) pc_pub += clock64() - pc_t0;
        }
    }
    if (prof) {
        unsigned long long* row = p.profile + size_t(blockIdx.x) * 8;
        row[0] = pc_rows; row[1] = pc_wait; row[2] = pc_work; row[3] = pc_bar; row[4] = pc_flags; row[5] = pc_pub;
        row[6] = clock64() - pc_start;
        row[7] = pc_issue;
    }
}

// One warp: raise my gate flag everywhere, then wait for everybody's.
struct PipeGateArgs {
    uint8_t* arena[LBC_MAX_RANKS];
    int world, rank;
    int64_t ctl_off;
    unsigned int epoch;
    unsigned long long timeout_ns;
    void* status;
};

__global__ void pipe_gate_kernel(const PipeGateArgs a) {
    const int64_t off = a.ctl_off + LBC_PIPE_CTL_FLAGS_GATE;
    if (int(threadIdx.x) < a.world)
        st_release_sys(reinterpret_cast<unsigned int*>(a.arena[threadIdx.x] + off) + a.rank, a.epoch);
    WaitSpec w{};
    w.flags = reinterpret_cast<const unsigned int*>(a.arena[a.rank] + off);
    w.count = a.world;
    w.epoch = a.epoch;
    w.timeout_ns = a.timeout_ns;
    w.status = a.status;
    w.phase = 11u;
    block_wait(w);
}

static int stage_bytes_for(int dtype, int group_size, int bit, int world, int stages, bool with_residual,
                           bool with_prepared) {
    const int eb = dtype == LBC_FP32 ? 4 : 2;
    const int rx = kRow * eb;
    const int rc = kRow * bit / 8;
    const int rs = (kRow / group_size) * eb;
    const int sub = (rc + rs + 127) / 128 * 128;
    int quant = rx * (with_residual ? 2 : 1);
    int reduce = world * sub + ((stages == 1 && with_prepared) ? rx : 0);
    int decode = stages == 2 ? sub + (with_prepared ? rx : 0) : 0;
    int stage = quant > reduce ? quant : reduce;
    if (decode > stage) stage = decode;
    return (stage + 127) / 128 * 128;
}

template <typename T, int G, int BIT>
struct PipeLauncher {
    static cudaError_t run(const LbcPipe* p, cudaStream_t stream) {
        static int smem_set[64] = {0};     // per device: the dynamic shared memory limit already granted
        LbcPipe launch = *p;
        launch.stage_bytes = stage_bytes_for(p->dtype, G, BIT, p->world, p->stages, p->residual != nullptr,
                                             p->prepared != nullptr);
        // as many rows in flight as two blocks per SM leave room for (the default), at least two
        int depth = p->ring_depth > 0 ? p->ring_depth : kMaxRing;
        if (depth > kMaxRing) depth = kMaxRing;
        while (depth > 2 && depth * launch.stage_bytes > 108 * 1024) --depth;
        if (depth < 2) depth = 2;
        const int smem = depth * launch.stage_bytes;
        if (smem > 220 * 1024) return cudaErrorInvalidValue;
        launch.ring_depth = depth;
        int dev = 0, sms = 148;
        cudaError_t err = cudaGetDevice(&dev);
        if (err != cudaSuccess) return err;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (dev < 64 && smem > smem_set[dev]) {
            err = cudaFuncSetAttribute(pipe_allreduce_kernel<T, G, BIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (err != cudaSuccess) return err;
            smem_set[dev] = smem;
        } else if (dev >= 64) {
            err = cudaFuncSetAttribute(pipe_allreduce_kernel<T, G, BIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (err != cudaSuccess) return err;
        }
        // The phases meet through grid-wide counters, so every block must be resident: the grid is what the
        // occupancy of this kernel allows (two blocks per SM by design), never more.
        int per_sm = 0;
        err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pipe_allreduce_kernel<T, G, BIT>, kThreads, smem);
        if (err != cudaSuccess) return err;
        if (per_sm < 1) return cudaErrorLaunchOutOfResources;
        if (per_sm > 2) per_sm = 2;
        const int64_t shard_rows = (p->shard_groups + (kRow / G) - 1) / (kRow / G);
        int64_t rows = shard_rows * p->world;          // the longest sweep (QUANT or DECODE of a two-stage call)
        if (p->stages == 1) rows = shard_rows;
        int grid = sms * per_sm;
        if (p->max_blocks > 0 && grid > p->max_blocks) grid = p->max_blocks;
        if (rows < 1) rows = 1;
        if (int64_t(grid) > rows) grid = int(rows);
        pipe_allreduce_kernel<T, G, BIT><<<grid, kThreads, smem, stream>>>(launch);
        return cudaGetLastError();
    }
};

}  // namespace lbc

extern "C" {

int lbc_pipe_stage_bytes(int dtype, int group_size, int bit, int world, int stages, int with_residual,
                         int with_prepared) {
    return lbc::stage_bytes_for(dtype, group_size, bit, world, stages, with_residual != 0, with_prepared != 0);
}

cudaError_t lbc_pipe_allreduce(const LbcPipe* p, cudaStream_t stream) {
    if (p == nullptr || p->numel < 0) return cudaErrorInvalidValue;
    if (p->world < 1 || p->world > LBC_MAX_RANKS || p->rank < 0 || p->rank >= p->world) return cudaErrorInvalidValue;
    if (p->stages != 1 && p->stages != 2) return cudaErrorInvalidValue;
    if ((p->phase_mask & ~LBC_PIPE_ALL) != 0 || p->phase_mask == 0) return cudaErrorInvalidValue;
    if (p->shard_groups <= 0 || (p->shard_groups & 7) != 0) return cudaErrorInvalidValue;
    if (p->x == nullptr || p->out == nullptr) return cudaErrorInvalidValue;
    if ((p->prepared == nullptr) != (p->residual_out == nullptr)) return cudaErrorInvalidValue;
    if (((p->q_off | p->ag_off | p->shard_stride) & 15) != 0 || (p->ctl_off & 255) != 0) return cudaErrorInvalidValue;
    const int64_t groups = (p->numel + p->group_size - 1) / p->group_size;
    const int shards = p->stages == 2 ? p->world : 1;
    if (groups > p->shard_groups * shards) return cudaErrorInvalidValue;
    const int64_t row_groups = LBC_PIPE_ROW_ELEMS / p->group_size;
    const int64_t shard_rows = (p->shard_groups + row_groups - 1) / row_groups;
    if (shard_rows * p->world >= (int64_t(1) << 31)) return cudaErrorInvalidValue;   // row indices are 32-bit
    for (int r = 0; r < p->world; ++r)
        if (p->arena[r] == nullptr || (reinterpret_cast<uintptr_t>(p->arena[r]) & 15) != 0) return cudaErrorInvalidValue;
    if (p->numel == 0) return cudaSuccess;
#define LBC_CASE(TT, GG, BB) \
    if (p->group_size == GG && p->bit == BB) return lbc::PipeLauncher<TT, GG, BB>::run(p, stream);
#define LBC_TYPE(TT) \
    LBC_CASE(TT, 64, 8) LBC_CASE(TT, 32, 8) LBC_CASE(TT, 16, 8) LBC_CASE(TT, 64, 4) LBC_CASE(TT, 32, 4) LBC_CASE(TT, 16, 4)
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

cudaError_t lbc_pipe_gate(uint8_t* const* arena, int world, int rank, int64_t ctl_off, unsigned int epoch,
                          unsigned long long timeout_ns, void* status, cudaStream_t stream) {
    if (arena == nullptr || world < 1 || world > LBC_MAX_RANKS || rank < 0 || rank >= world) return cudaErrorInvalidValue;
    lbc::PipeGateArgs a{};
    for (int r = 0; r < world; ++r) a.arena[r] = arena[r];
    a.world = world;
    a.rank = rank;
    a.ctl_off = ctl_off;
    a.epoch = epoch;
    a.timeout_ns = timeout_ns;
    a.status = status;
    lbc::pipe_gate_kernel<<<1, 32, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // extern "C"

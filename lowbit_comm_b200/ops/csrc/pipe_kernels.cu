// Pipelined compressed all-reduce for sm_100a: ONE persistent kernel per collective.
//
// Work unit: a row of 4096 elements (256 threads x 16).  Three kinds of rows:
//   QUANT   x (+ residual) -> int8/int4 groups + scales, written into this rank's own arena
//   REDUCE  the owner of a shard pulls the row from all W ranks (bulk asynchronous loads over NVLink,
//           `cp.async.bulk` global -> shared, no multicast, no tensor map), sums it in fp32 and
//           requantizes it into its own arena (stages == 1: writes the result instead)
//   DECODE  every rank pulls the reduced row from its owner and decodes it into the output, updating
//           the error-feedback residual
// All cross-GPU traffic is loads issued by the copy engine of the SM into a ring of shared-memory
// stages (3 rows in flight per block by default), so neither the load/store pipeline nor the register
// file limits the bytes in flight over NVLink; flags are the only remote stores.
//
// Scheduling: rows are handed out by a ticket counter in an order in which every row depends only on
// rows with smaller tickets (QUANT of chunk s, REDUCE of chunk s-1 and DECODE of chunk s-2 are
// interleaved row by row).  A block claims tickets in order and never blocks on a dependency while it
// still holds claimed, unprocessed rows, therefore the schedule cannot deadlock whatever the grid size
// or the number of resident blocks; HBM-bound QUANT rows, NVLink-bound REDUCE rows and DECODE rows of
// neighbouring chunks are in flight at the same time.
//
// Every wait (dependency flags, load completion barriers) is bounded: when it runs out the kernel
// records where in the status word, waits (bounded again) for its own loads in flight and returns.
//
// Math is identical, bit for bit, to quant_push_kernel / reduce_kernel (fast_kernels.cu).
// The reference runs the same algorithm as quantize -> NCCL all_to_all -> dequantize-reduce ->
// quantize -> NCCL all_gather -> dequantize (ccdl_comm/communication/reduce_scatter_transport.py:186-377).

#include "codec_device.cuh"
#include "common.cuh"
#include "lbc_api.h"

namespace lbc {

constexpr int kRow = kThreads * kElemsPerThread;   // 4096 elements
constexpr int kMaxRing = 4;
constexpr unsigned int kPhasePipeFlag = 8u;        // status.phase values 8..10: flag wait of QUANT/REDUCE/DECODE rows
constexpr unsigned int kPhasePipeLoad = 12u;       // status.phase: a bulk load that never completed

enum PipeKind : int { kQuant = 0, kReduce = 1, kDecode = 2 };

struct __align__(16) PipeItem {
    int kind;
    int chunk;
    int shard;        // QUANT: destination shard; REDUCE: this rank's shard; DECODE: owner of the row
    int live;         // groups of the row that hold data
    int copy;         // live rounded up to 8 groups: what the bulk loads move
    int dense_tma;    // the dense row (x / residual / prepared) comes through the copy engine
    int gl0;          // first group of the row inside its shard
    int pad;
    long long first;      // first element of the row inside the tensor
    long long code_off;   // REDUCE / DECODE: arena offset of the row's codes ...
    long long scale_off;  // ... and of its scales
    long long pad2;
};
static_assert(sizeof(PipeItem) == 64, "PipeItem is copied as four 16-byte vectors");

// ---------------------------------------------------------------------------
// mbarrier + bulk load helpers (shared::cta barriers, transaction counts in bytes)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
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
__global__ void __launch_bounds__(kThreads + 32, 2) pipe_allreduce_kernel(const __grid_constant__ LbcPipe p) {
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
    __shared__ __align__(8) unsigned long long full_bar[kMaxRing];
    __shared__ PipeItem meta[kMaxRing];
    __shared__ int s_tail, s_tail_refill, s_stop;       // s_stop: 1 = all rows done, 2 = a wait ran out
    __shared__ unsigned short s_ready_reduce[LBC_MAX_RANKS];   // per owner: chunks whose REDUCE flag was seen
    __shared__ __align__(16) ScaleStage scale_stage;
    // the schedule: segment s holds the QUANT rows of chunk s, the REDUCE rows of chunk s - 1 and the DECODE
    // rows of chunk s - 2 (those that exist and that this launch runs), interleaved row by row
    __shared__ long long seg_start[LBC_PIPE_MAX_CHUNKS + 3];
    // A segment opens with `seg_lead` QUANT-only super-rows: the rows behind them wait for flags that the
    // last rows of the previous segment raise, and the lead gives those stragglers time to finish while
    // every block still has work that depends on nothing.
    __shared__ int seg_lead[LBC_PIPE_MAX_CHUNKS + 3];

    const int W = p.world, me = p.rank;
    const bool two = p.stages == 2;
    const int shards = two ? W : 1;
    const int64_t SG = p.shard_groups;
    const int64_t n = p.numel;
    const int64_t num_groups = (n + G - 1) / G;
    const int64_t shard_rows = (SG + RG - 1) / RG;
    const int64_t rpc = p.rows_per_chunk;
    const int C = p.num_chunks;
    const int segs = C + (two ? 2 : 1);
    const bool run_quant = (p.phase_mask & LBC_PIPE_QUANT) != 0, run_reduce = (p.phase_mask & LBC_PIPE_REDUCE) != 0;
    const bool run_decode = two && (p.phase_mask & LBC_PIPE_DECODE) != 0;
    const int S = p.ring_depth;
    const int stage_bytes = p.stage_bytes;
    const int wlane = threadIdx.x & 31;
    const bool producer = threadIdx.x >= kThreads;      // the ninth warp

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
    unsigned int* ticket = reinterpret_cast<unsigned int*>(ctl + LBC_PIPE_CTL_LOCAL);
    unsigned int* exit_count = ticket + 1;
    unsigned int* done_count = ticket + 2;              // [2][LBC_PIPE_MAX_CHUNKS]: QUANT rows, REDUCE rows
    volatile DeviceStatus* status = static_cast<volatile DeviceStatus*>(p.status);

    auto rows_in_chunk = [&](int c) -> int64_t {
        if (c < 0 || c >= C) return 0;
        const int64_t left = shard_rows - int64_t(c) * rpc;
        return left < 0 ? 0 : (left < rpc ? left : rpc);
    };
    // kinds a segment holds and the tickets of one of its super-rows
    auto seg_kinds = [&](int sg, bool& q, bool& r, bool& d) -> int {
        q = run_quant && sg < C;
        r = run_reduce && sg >= 1 && sg - 1 < C;
        d = run_decode && sg >= 2 && sg - 2 < C;
        return (q ? shards : 0) + (r ? 1 : 0) + (d ? W : 0);
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxRing; ++s) mbar_init(&full_bar[s], 1u);
        s_tail = 0;
        s_tail_refill = 0;
        s_stop = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        long long at = 0;
        for (int sg = 0; sg < segs; ++sg) {
            bool q, r, d;
            const int per = seg_kinds(sg, q, r, d);
            int64_t rows = 0;
            if (q) rows = rows_in_chunk(sg);
            if (r && rows_in_chunk(sg - 1) > rows) rows = rows_in_chunk(sg - 1);
            if (d && rows_in_chunk(sg - 2) > rows) rows = rows_in_chunk(sg - 2);
            int lead = 0;
            if (q && (r || d)) lead = int(rows_in_chunk(sg) / 2);   // half a segment of slack
            seg_lead[sg] = lead;
            seg_start[sg] = at;
            at += rows * per + int64_t(lead) * shards;
        }
        seg_start[segs] = at;
    }
    if (threadIdx.x < LBC_MAX_RANKS) s_ready_reduce[threadIdx.x] = 0;
    __syncthreads();
    const int64_t total_tickets = seg_start[segs];
    // tickets are claimed a few at a time: one atomic per ticket on one address was most of the run time
    int batch = int(total_tickets / (int64_t(gridDim.x) * 4));
    batch = batch < 1 ? 1 : (batch > 8 ? 8 : batch);

    // ---- state of the producer warp (uniform across its lanes) ----
    int head = 0, tail = 0;                // rows consumed / rows issued (head is tracked by every thread)
    bool has_pending = false, exhausted = false, failed = false;
    PipeItem pend{};
    unsigned int ready_quant = 0;          // chunks whose QUANT flags of all ranks were seen
    int pub_chunk[2] = {-1, -1}, pub_rows[2] = {0, 0};   // finished rows not yet published: QUANT, REDUCE
    PipeItem mine{};                                      // lane i decodes ticket i of the claimed batch ...
    bool mine_valid = false;
    int batch_at = 0, batch_count = 0, pend_from = 0;     // ... and the rows are issued one after the other
    int cur_seg = 0;                                      // tickets only grow: the scan for a segment resumes here

    // Publishes finished rows of (kind, chunk): the last row of a chunk raises the chunk's flag on every rank.
    // Called by all lanes of warp 0 after a block barrier behind the rows' stores.
    auto publish = [&](int kind) {
        if (pub_rows[kind] == 0) return;
        const int c = pub_chunk[kind];
        unsigned int prev = 0;
        if (wlane == 0) {
            // device scope is enough here (and far cheaper than system scope, which cost tens of microseconds
            // per chunk when every block paid it): the one block that raises the flags fences at system scope
            // after it has seen everybody's count, which orders all the rows before the flags
            __threadfence();
            prev = atomicAdd(done_count + kind * LBC_PIPE_MAX_CHUNKS + c, (unsigned int)pub_rows[kind]);
        }
        prev = __shfl_sync(0xffffffffu, prev, 0);
        const int64_t expected = rows_in_chunk(c) * (kind == kQuant ? shards : 1);
        if (int64_t(prev) + pub_rows[kind] == expected) {
            if (wlane == 0) {
                done_count[kind * LBC_PIPE_MAX_CHUNKS + c] = 0u;   // ready for the next collective
                __threadfence_system();
            }
            __syncwarp();
            if (wlane < W) {
                const int64_t off = p.ctl_off + (kind == kQuant ? LBC_PIPE_CTL_FLAGS_QUANT : LBC_PIPE_CTL_FLAGS_REDUCE) +
                                    (int64_t(me) * LBC_PIPE_MAX_CHUNKS + c) * 4;
                st_release_sys(reinterpret_cast<unsigned int*>(p.arena[wlane] + off), p.epoch);
            }
        }
        pub_rows[kind] = 0;
        pub_chunk[kind] = -1;
    };
    auto note_done = [&](int kind, int chunk) {
        if (kind == kDecode) return;
        if (kind == kReduce && !two) return;               // one stage: nobody waits for reduced rows
        // Only a chunk's last row matters to the waiting ranks, so a block publishes its rows of a chunk once:
        // when it meets a later chunk (tickets are handed out in order: no more rows of the old one will come),
        // before it sleeps on a flag, and when it leaves.
        if (pub_chunk[kind] != chunk) publish(kind);
        pub_chunk[kind] = chunk;
        ++pub_rows[kind];
    };

    // ticket -> row; false for the empty slots of the schedule
    auto decode_ticket = [&](int64_t t, PipeItem& it) -> bool {
        while (cur_seg + 1 < segs && t >= seg_start[cur_seg + 1]) ++cur_seg;
        const int seg = cur_seg;
        bool q, r, d;
        const unsigned int per = (unsigned int)seg_kinds(seg, q, r, d);
        unsigned int rem = (unsigned int)(t - seg_start[seg]);       // a segment's tickets fit 32 bits
        const unsigned int lead = (unsigned int)seg_lead[seg], lead_tickets = lead * (unsigned int)shards;
        unsigned int j;
        int k;
        it.kind = -1;
        if (rem < lead_tickets) {                       // the QUANT-only opening of the segment
            j = rem / (unsigned int)shards;
            it.kind = kQuant; it.chunk = seg; it.shard = int(rem - j * (unsigned int)shards);
            k = 0;
        } else {
            rem -= lead_tickets;
            j = rem / per;
            k = int(rem - j * per);
        }
        if (it.kind < 0 && q) {
            if (k < shards) { it.kind = kQuant; it.chunk = seg; it.shard = k; j += lead; }
            k -= shards;
        }
        if (it.kind < 0 && r) {
            if (k == 0) { it.kind = kReduce; it.chunk = seg - 1; it.shard = two ? me : 0; }
            k -= 1;
        }
        if (it.kind < 0) { it.kind = kDecode; it.chunk = seg - 2; it.shard = (k + me) % W; }
        if (int64_t(j) >= rows_in_chunk(it.chunk)) return false;   // an empty slot of the schedule
        const int64_t row = int64_t(it.chunk) * rpc + j;
        const int64_t gl0 = row * RG;
        it.gl0 = int(gl0);
        int64_t valid = num_groups - int64_t(it.shard) * SG;
        valid = valid < 0 ? 0 : (valid > SG ? SG : valid);
        int64_t live = valid - gl0;
        live = live < 0 ? 0 : (live > RG ? RG : live);
        it.live = int(live);
        it.copy = (it.live + 7) / 8 * 8;
        it.first = (int64_t(it.shard) * SG + gl0) * G;
        // a dense row goes through the copy engine when its source is 16-byte aligned and no group of it is cut
        // by the end of the tensor; the other rows are read with plain guarded loads
        const bool whole = it.first + live * G <= n;
        if (it.kind == kQuant) {
            it.dense_tma = (quant_tma_ok && whole) ? 1 : 0;
            it.code_off = it.scale_off = 0;
        } else {
            const bool want_prep = prep != nullptr && (it.kind == kDecode || !two);
            it.dense_tma = (want_prep && prep_tma_ok && whole) ? 1 : 0;
            const int64_t region = it.kind == kReduce ? p.q_off + int64_t(it.shard) * p.shard_stride : p.ag_off;
            it.code_off = region + gl0 * VB;
            it.scale_off = region + SG * VB + gl0 * MB;
        }
        return true;
    };

    // Non-blocking look at the flags a row depends on (all lanes of warp 0).
    auto dep_ready = [&](const PipeItem& it, unsigned int& seen_out, int& peer_out) -> bool {
        if (it.kind == kQuant) return true;
        if (it.kind == kReduce) {
            if ((ready_quant >> it.chunk) & 1u) return true;
            unsigned int seen = p.epoch;
            if (wlane < W) seen = ld_relaxed_sys(flags_quant + wlane * LBC_PIPE_MAX_CHUNKS + it.chunk);
            const bool ok = int(seen - p.epoch) >= 0;
            const unsigned int late = __ballot_sync(0xffffffffu, !ok);
            if (late == 0u) {
                fence_acq_rel_sys();                   // the rows behind the flags are visible from here on ...
                fence_async_global();                  // ... also to the bulk loads (another memory proxy)
                __syncwarp();
                ready_quant |= 1u << it.chunk;
                return true;
            }
            peer_out = __ffs(late) - 1;
            seen_out = __shfl_sync(0xffffffffu, seen, peer_out);
            return false;
        }
        if ((s_ready_reduce[it.shard] >> it.chunk) & 1u) return true;
        unsigned int seen = 0;
        if (wlane == 0) seen = ld_relaxed_sys(flags_reduce + it.shard * LBC_PIPE_MAX_CHUNKS + it.chunk);
        seen = __shfl_sync(0xffffffffu, seen, 0);
        if (int(seen - p.epoch) >= 0) {
            fence_acq_rel_sys();
            fence_async_global();
            if (wlane == 0) s_ready_reduce[it.shard] |= (unsigned short)(1u << it.chunk);
            __syncwarp();
            return true;
        }
        peer_out = it.shard;
        seen_out = seen;
        return false;
    };

    // Hands the pending row's loads to the copy engine.  The row was decoded by lane `pend_from`, which also
    // issues it; only a REDUCE row, with one source per rank, spreads its loads over the lanes.
    auto issue = [&](int stage) {
        unsigned long long* bar = &full_bar[stage];
        unsigned char* base = ring + size_t(stage) * stage_bytes;
        const bool mine_turn = wlane == pend_from;
        if (pend.kind == kReduce) {
            const long long code_off = __shfl_sync(0xffffffffu, mine.code_off, pend_from);
            const long long scale_off = __shfl_sync(0xffffffffu, mine.scale_off, pend_from);
            const unsigned int code_bytes = (unsigned int)(pend.copy) * VB, scale_bytes = (unsigned int)(pend.copy) * MB;
            if (mine_turn) {
                const unsigned int prep_bytes = mine.dense_tma ? (unsigned int)(mine.live) * G * sizeof(T) : 0u;
                mbar_expect_tx(bar, (unsigned int)(W) * (code_bytes + scale_bytes) + prep_bytes);
            }
            __syncwarp();
            if (wlane < W) {
                unsigned char* dst = base + wlane * SUB;
                bulk_load(dst, p.arena[wlane] + code_off, code_bytes, bar);
                bulk_load(dst + RC, p.arena[wlane] + scale_off, scale_bytes, bar);
            }
            if (mine_turn && mine.dense_tma)
                bulk_load(base + W * SUB, prep + mine.first, (unsigned int)(mine.live) * G * sizeof(T), bar);
        } else if (mine_turn) {
            const unsigned int dense_bytes = mine.dense_tma ? (unsigned int)(mine.live) * G * sizeof(T) : 0u;
            if (mine.kind == kQuant) {
                mbar_expect_tx(bar, dense_bytes * (res != nullptr ? 2u : 1u));
                if (mine.dense_tma) {
                    bulk_load(base, x + mine.first, dense_bytes, bar);
                    if (res != nullptr) bulk_load(base + RX, res + mine.first, dense_bytes, bar);
                }
            } else {
                const unsigned int code_bytes = (unsigned int)(mine.copy) * VB, scale_bytes = (unsigned int)(mine.copy) * MB;
                const uint8_t* owner = p.arena[mine.shard];
                mbar_expect_tx(bar, code_bytes + scale_bytes + dense_bytes);
                bulk_load(base, owner + mine.code_off, code_bytes, bar);
                bulk_load(base + RC, owner + mine.scale_off, scale_bytes, bar);
                if (mine.dense_tma) bulk_load(base + SUB, prep + mine.first, dense_bytes, bar);
            }
        }
        if (mine_turn) {
            const uint4* from = reinterpret_cast<const uint4*>(&mine);
            uint4* to = reinterpret_cast<uint4*>(&meta[stage]);
            to[0] = from[0]; to[1] = from[1]; to[2] = from[2]; to[3] = from[3];
        }
        __syncwarp();
    };

    // Claims tickets and hands their loads to the copy engine until the ring is full, the schedule is used up
    // or a row's flags are not there yet.  Only with an empty ring (`may_block`) does it sleep on a flag.
    auto fill = [&](bool may_block) {
        while (!failed && tail - head < S) {
            if (!has_pending) {
                if (batch_at >= batch_count) {
                    if (exhausted) break;
                    unsigned int t = 0;
                    if (wlane == 0) t = atomicAdd(ticket, (unsigned int)batch);
                    t = __shfl_sync(0xffffffffu, t, 0);
                    if (int64_t(t) >= total_tickets) {
                        exhausted = true;
                        break;
                    }
                    const int64_t left = total_tickets - int64_t(t);
                    batch_count = left < batch ? int(left) : batch;
                    batch_at = 0;
                    // the arithmetic of a ticket is a long dependent chain: the lanes do it side by side
                    mine_valid = wlane < batch_count && decode_ticket(int64_t(t) + wlane, mine);
                }
                pend_from = batch_at++;
                const bool valid = __shfl_sync(0xffffffffu, mine_valid ? 1 : 0, pend_from) != 0;
                if (!valid) continue;
                // what every lane has to know about the row; the rest stays with the lane that decoded it
                pend.kind = __shfl_sync(0xffffffffu, mine.kind, pend_from);
                pend.chunk = __shfl_sync(0xffffffffu, mine.chunk, pend_from);
                pend.shard = __shfl_sync(0xffffffffu, mine.shard, pend_from);
                pend.live = __shfl_sync(0xffffffffu, mine.live, pend_from);
                pend.copy = __shfl_sync(0xffffffffu, mine.copy, pend_from);
                if (pend.live == 0) {              // padding row: nothing to move, but its chunk still counts it
                    note_done(pend.kind, pend.chunk);
                    continue;
                }
                has_pending = true;
            }
            unsigned int seen = 0;
            int peer = 0;
            bool ready = dep_ready(pend, seen, peer);
            if (!ready) {
                if (!may_block || tail != head) break;   // first process what this block already holds
                publish(kQuant);                   // nothing may stay unpublished while this block sleeps
                publish(kReduce);
                const unsigned long long t0 = global_ns();
                unsigned int spins = 0;
                for (;;) {
                    ready = dep_ready(pend, seen, peer);
                    if (ready) break;
                    if ((++spins & 1023u) == 0) {      // the status word lives in host memory: look rarely
                        const bool failed_before = status != nullptr && status->code != 0u;
                        const bool late = global_ns() - t0 > p.timeout_ns;
                        if (failed_before || late) {
                            if (late && !failed_before && wlane == 0 && status != nullptr) {
                                status->phase = kPhasePipeFlag + (unsigned int)pend.kind;
                                status->peer = (unsigned int)peer;
                                status->seen = seen;
                                status->expected = p.epoch;
                                __threadfence_system();
                                status->code = 1u;
                                __threadfence_system();
                            }
                            failed = true;
                            break;
                        }
                    }
                    __nanosleep(spins < 64u ? 100 : 500);
                }
                if (!ready) break;
            }
            issue(tail % S);
            ++tail;
            has_pending = false;
        }
    };
    // Ring state for the other warps.  Two words, so that nobody ever reads a word in the phase in which it
    // is written with a different meaning: `s_tail` is written while the others compute (before the row's
    // barrier) and read right after that barrier; `s_tail_refill` is written while the others wait for a
    // refill of the empty ring (between the row's barrier and the refill barrier) and read after the latter.
    auto publish_refill = [&]() {
        if (wlane == 0) {
            s_tail_refill = tail;
            if (failed) s_stop = 2;
            else if (tail == head && exhausted && !has_pending) s_stop = 1;
        }
    };

    // Warps 0..7 compute, warp 8 produces: it claims rows and issues their loads while the others work on
    // the row at the head of the ring.  One block barrier per row; a second one only when the ring ran empty.
    if (producer) {
        fill(true);
        publish_refill();
    }
    __syncthreads();
    int tail_seen = s_tail_refill, stop_seen = s_stop;
    // optional cycle accounting (one consumer thread and the producer's first lane per block):
    // [0] rows  [1] consumer: waiting for loads  [2] consumer: computing  [3] consumer: at barriers
    // [4] producer: claiming and issuing  [5] producer: asleep on flags + refills  [6] total  [7] rows issued
    const bool prof = p.profile != nullptr && (threadIdx.x == 0 || threadIdx.x == kThreads);
    long long pc_wait = 0, pc_work = 0, pc_bar = 0, pc_fill = 0, pc_refill = 0, pc_rows = 0;
    const long long pc_start = clock64();
    // leaves when a wait ran out, or when nothing is left: the producer only leaves the ring empty once the
    // schedule is used up
    while (stop_seen != 2 && head < tail_seen) {
        const int stage = head % S;
        const PipeItem it = meta[stage];
        const unsigned char* base = ring + size_t(stage) * stage_bytes;
        long long pc_t0 = prof ? clock64() : 0, pc_t1 = 0;
        if (producer) {
            fill(false);
            if (wlane == 0) s_tail = tail;
            if (prof) pc_fill += clock64() - pc_t0;
        } else {
            // ---- wait for the row's loads ----
            const unsigned int parity = (unsigned int)(head / S) & 1u;
            bool arrived = mbar_try_wait(&full_bar[stage], parity);
            if (!arrived) {
                const unsigned long long t0 = global_ns();
                unsigned int spins = 0;
                while (!(arrived = mbar_try_wait(&full_bar[stage], parity))) {
                    if ((++spins & 63u) == 0 && global_ns() - t0 > p.timeout_ns) break;
                }
            }
            arrived = __all_sync(0xffffffffu, arrived) != 0;   // the row's math shuffles across the whole warp
            if (!arrived) {
                if (status != nullptr && status->code == 0u) {
                    status->phase = kPhasePipeLoad;
                    status->peer = (unsigned int)it.shard;
                    status->seen = (unsigned int)it.kind;
                    status->expected = p.epoch;
                    __threadfence_system();
                    status->code = 1u;
                    __threadfence_system();
                }
                s_stop = 2;
            }
            if (prof) { pc_t1 = clock64(); pc_wait += pc_t1 - pc_t0; }
            if (arrived) {
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
        }
        long long pc_t2 = 0;
        if (prof) { pc_t2 = clock64(); if (!producer) pc_work += pc_t2 - pc_t1; ++pc_rows; }
        __syncthreads();                 // the stage is free again and the row's stores are issued
        if (prof) pc_bar += clock64() - pc_t2;
        stop_seen = s_stop;              // 2 if a load wait ran out in this row
        if (stop_seen == 2) break;
        ++head;
        // The producer may already be writing the next row's value into `s_tail`; whichever value a thread
        // reads, it is the count of rows issued so far or more, and "ring empty" (equal to head) can only be
        // read while the producer sits in the refill branch below, where it does not write this word.
        tail_seen = s_tail;
        if (head == tail_seen) {         // the ring ran empty: the producer claims, and may have to sleep on a flag
            const long long pc_t3 = prof ? clock64() : 0;
            if (producer) {
                note_done(it.kind, it.chunk);
                fill(true);
                publish_refill();
            }
            __syncthreads();
            if (prof) pc_refill += clock64() - pc_t3;
            tail_seen = s_tail_refill;
            stop_seen = s_stop;
        } else if (producer) {
            note_done(it.kind, it.chunk);
        }
    }

    if (stop_seen == 2) {
        // a wait ran out: give this block's loads that are still in flight a bounded chance to land,
        // then leave; the host resets the control block before the workspace is used again
        const int issued = s_tail > s_tail_refill ? s_tail : s_tail_refill;
        for (int h = head; h < issued; ++h) {
            const unsigned int parity = (unsigned int)(h / S) & 1u;
            const unsigned long long t0 = global_ns();
            while (!mbar_try_wait(&full_bar[h % S], parity)) {
                if (global_ns() - t0 > 2000000ull) break;
            }
        }
        return;
    }
    if (prof) {
        unsigned long long* row = p.profile + size_t(blockIdx.x) * 8;
        if (!producer) {
            row[0] = pc_rows; row[1] = pc_wait; row[2] = pc_work; row[3] = pc_bar; row[6] = clock64() - pc_start;
        } else {
            row[4] = pc_fill; row[5] = pc_refill; row[7] = (unsigned long long)tail;
        }
    }
    if (producer) {
        publish(kQuant);
        publish(kReduce);
        if (wlane == 0) {
            const unsigned int gone = atomicAdd(exit_count, 1u);
            if (gone == gridDim.x - 1) {               // every block has claimed its last ticket
                *ticket = 0u;
                *exit_count = 0u;
                __threadfence();
            }
        }
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
        int depth = p->ring_depth > 0 ? p->ring_depth : 3;
        if (depth > kMaxRing) depth = kMaxRing;
        while (depth > 2 && depth * launch.stage_bytes > 110 * 1024) --depth;
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
        const int per_sm = smem <= 110 * 1024 ? 2 : 1;
        const int64_t shard_rows = (p->shard_groups + (kRow / G) - 1) / (kRow / G);
        const int shards = p->stages == 2 ? p->world : 1;
        int64_t rows = shard_rows * shards * (p->stages == 2 ? 2 : 1) + shard_rows;   // upper bound of the work
        int grid = sms * per_sm;
        if (p->max_blocks > 0 && grid > p->max_blocks) grid = p->max_blocks;
        if (rows < 1) rows = 1;
        if (int64_t(grid) > rows) grid = int(rows);
        pipe_allreduce_kernel<T, G, BIT><<<grid, kThreads + 32, smem, stream>>>(launch);
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
    if (p->num_chunks < 1 || p->num_chunks > LBC_PIPE_MAX_CHUNKS || p->rows_per_chunk < 1) return cudaErrorInvalidValue;
    if (p->x == nullptr || p->out == nullptr) return cudaErrorInvalidValue;
    if ((p->prepared == nullptr) != (p->residual_out == nullptr)) return cudaErrorInvalidValue;
    if (((p->q_off | p->ag_off | p->shard_stride) & 15) != 0 || (p->ctl_off & 255) != 0) return cudaErrorInvalidValue;
    const int64_t groups = (p->numel + p->group_size - 1) / p->group_size;
    const int shards = p->stages == 2 ? p->world : 1;
    if (groups > p->shard_groups * shards) return cudaErrorInvalidValue;
    const int64_t row_groups = LBC_PIPE_ROW_ELEMS / p->group_size;
    const int64_t shard_rows = (p->shard_groups + row_groups - 1) / row_groups;
    if (int64_t(p->num_chunks) * p->rows_per_chunk < shard_rows) return cudaErrorInvalidValue;
    // tickets are 32-bit
    const int64_t per = p->stages == 2 ? 2 * p->world + 1 : 2;
    if ((p->num_chunks + 2) * p->rows_per_chunk * per >= (int64_t(1) << 31)) return cudaErrorInvalidValue;
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

// Host-callable launchers of the sm_100a kernels.  Everything here takes raw
// device pointers and a stream, so the kernels build without any torch header.
//
// Parity map (reference, csrc/): quantize_pack_kernel (quantization/
// quant_pack_kernel.cu:25-163) -> lbc_quant_push; dequant_kernel* and
// dequant_reduce*_fused kernels (quantization/dequant_kernel.cuh:62-292,
// dequant_reduce_kernel.cu:71-221) -> lbc_reduce; quant_kernel* with top-k,
// 4-bit code-books and stochastic rounding (quant_kernel.cuh:155-400) ->
// lbc_quant_general / lbc_dequant_general.  The scatter/broadcast modes, the
// signals and the bounded waits have no counterpart in the reference: there the
// payload moves through a NCCL call between kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LBC_MAX_RANKS 16

enum LbcDType { LBC_FP16 = 0, LBC_BF16 = 1, LBC_FP32 = 2 };
enum LbcQuantType { LBC_LINEAR = 0, LBC_NORMAL = 1, LBC_UNIFORM = 2, LBC_E3M0 = 3, LBC_E2M1 = 4 };
enum LbcPushMode { LBC_PUSH_BROADCAST = 0, LBC_PUSH_SCATTER = 1, LBC_PUSH_COMPACT_LOCAL = 2 };

typedef struct {
    unsigned int* remote_flags[LBC_MAX_RANKS];  // flag arrays (one per destination)
    int num_remote;                             // 0 = no signalling
    int my_slot;                                // index written inside every flag array
    unsigned int epoch;                         // value written
    unsigned int* block_counter;                // local scratch counter, zero between launches
} LbcSignal;

typedef struct {
    const unsigned int* flags;   // local flag array, NULL = no wait
    int count;                   // flags[0..count) must reach `epoch`
    unsigned int epoch;
    unsigned long long timeout_ns;
    void* status;                // LbcStatus*, device visible
    unsigned int phase;
} LbcWait;

typedef struct {
    unsigned int code, phase, peer, seen, expected, reserved[3];
} LbcStatus;

// ---- fast path: linear, top-k 0, deterministic rounding ---------------------
typedef struct {
    int dtype, group_size, bit;
    const void* x;             // T[numel]
    const void* residual;      // optional T[numel]: prepared = T(x + residual)
    void* prepared_out;        // optional T[numel]: receives `prepared` (may alias residual)
    void* local_ef_out;        // optional T[numel]: receives T(prepared - dequant(quant(prepared)))
    int64_t numel;
    int mode;                  // LbcPushMode
    uint8_t* dst[LBC_MAX_RANKS];
    int num_dst;
    int64_t shard_groups;      // scatter: groups per destination
    int64_t layout_groups;     // groups in the destination planar layout (start of the scale region)
    int64_t group_offset;      // broadcast: index of group 0 inside the destination layout
    LbcSignal signal;
    int max_blocks;            // 0 = library default
    uint8_t* mc_dst;           // broadcast only: NVLink multicast alias of dst[*] (one store reaches every rank)
} LbcQuantPush;

typedef struct {
    int dtype, group_size, bit;
    const uint8_t* src[LBC_MAX_RANKS];
    int num_src;
    int64_t layout_groups;     // groups in every source layout
    int64_t group_offset;      // first group to read inside the source layout
    int compact;               // sources use the per-group record layout
    int64_t src_shard_groups;  // > 0: gather mode, group g is read from src[g / src_shard_groups] only (every
                               // source is a planar payload of src_shard_groups groups: a peer's reduced shard)
    int first_src;             // gather mode: the sweep over the groups starts at this source's shard, so that
                               // ranks that start at their own index never read from the same peer at once
    int64_t numel;             // elements to produce
    float scale;               // applied to the fp32 sum (1/W for a mean)
    void* out;                 // optional T[numel]
    int accumulate;            // out = T(float(out) + float(T(y)))   (unfused SUM parity)
    const void* prepared;      // optional T[numel]
    void* residual_out;        // optional T[numel] = T(float(prepared) - y_fp32); may alias prepared
    uint8_t* dst[LBC_MAX_RANKS];  // optional: requantize T(y) and broadcast it (planar)
    int num_dst;
    int64_t dst_layout_groups;
    int64_t dst_group_offset;
    LbcSignal signal;
    LbcWait wait;
    int max_blocks;
    int gather_order;          // set by the launcher: 1 = gather-mode tiles walk the sources round-robin
    int bulk_store;            // set by the launcher: requantized tiles leave through bulk stores
    uint8_t* mc_dst;           // optional NVLink multicast alias of dst[*]: one multimem store reaches every rank
} LbcReduce;

cudaError_t lbc_quant_push(const LbcQuantPush* p, cudaStream_t stream);
cudaError_t lbc_reduce(const LbcReduce* p, cudaStream_t stream);

// ---- single-launch all-reduce: one persistent kernel, every NVLink byte moved by bulk loads ----------
// Every rank quantizes its tensor into its OWN arena (phase QUANT), the owner of a shard pulls that
// shard's rows from all ranks with bulk asynchronous loads, reduces and requantizes them into its own
// arena (phase REDUCE), and every rank pulls the reduced shards and decodes them (phase DECODE).  Rows of
// 4096 elements are the unit of work, dealt to the blocks statically; the ranks meet between the phases
// through one epoch flag per (rank, phase).  With stages == 1 there is one "shard" (the whole tensor),
// every rank reduces all W payloads and writes the result directly (no DECODE phase).
// The reference moves the same bytes with NCCL calls between kernels (ccdl_comm/cuda/transports/
// pipelined_ring.py:236-316); it has no counterpart of this kernel.
#define LBC_PIPE_FLAG_STRIDE 16   // u32 words between two ranks' flags (one 64-byte line per rank)
#define LBC_PIPE_ROW_ELEMS 4096
enum LbcPipePhase { LBC_PIPE_QUANT = 1, LBC_PIPE_REDUCE = 2, LBC_PIPE_DECODE = 4, LBC_PIPE_ALL = 7 };
// Control block of one workspace (same offset in every arena; zero when the arena is created):
#define LBC_PIPE_CTL_FLAGS_QUANT 0      // u32 [LBC_MAX_RANKS][LBC_PIPE_FLAG_STRIDE], word 0 of each line written by that peer
#define LBC_PIPE_CTL_FLAGS_REDUCE 1024  // u32 [LBC_MAX_RANKS][LBC_PIPE_FLAG_STRIDE], word 0 of each line written by that peer
#define LBC_PIPE_CTL_FLAGS_GATE 2048    // u32 [LBC_MAX_RANKS], written by the peers (rendezvous)
#define LBC_PIPE_CTL_LOCAL 2304         // u32 [2] reserved, then blocks done per phase: local scratch
#define LBC_PIPE_CTL_BYTES 2560

typedef struct {
    int dtype, group_size, bit;
    int world, rank;
    int stages;                 // 2 = reduce-scatter + gather, 1 = every rank reduces all payloads
    int phase_mask;             // LbcPipePhase bits; LBC_PIPE_ALL in production, single phases for one-GPU emulation
    const void* x;              // T[numel]
    void* out;                  // T[numel], may alias x
    const void* residual;       // optional T[numel]: prepared = T(x + residual)
    void* prepared_out;         // optional T[numel]: receives `prepared` (may alias residual)
    void* local_ef_out;         // optional T[numel]: receives T(prepared - dequant(quant(prepared)))
    const void* prepared;       // optional T[numel]: read by the last phase ...
    void* residual_out;         // ... which writes T(float(prepared) - result) here (may alias prepared)
    int64_t numel;
    float scale;                // applied to the fp32 sum
    uint8_t* arena[LBC_MAX_RANKS];  // base of every rank's arena (peer mappings)
    int64_t q_off;              // own quantized payload: `shards` planar payloads, `shard_stride` apart
    int64_t shard_stride;
    int64_t ag_off;             // own reduced shard, one planar payload (stages == 2)
    int64_t ctl_off;            // control block
    int64_t shard_groups;       // groups per shard, a multiple of 8
    unsigned int epoch;
    unsigned long long timeout_ns;
    void* status;               // LbcStatus*, device visible
    int max_blocks;             // 0 = two blocks per SM
    int ring_depth;             // rows in flight per block, 0 = as many as two blocks per SM leave room for (2..8)
    int stage_bytes;            // filled in by the launcher
    unsigned long long* profile;  // optional [gridDim.x][8] cycle counters (see pipe_kernels.cu), NULL = off
} LbcPipe;

cudaError_t lbc_pipe_allreduce(const LbcPipe* p, cudaStream_t stream);
// One warp: raises this rank's gate flag on every rank, then waits (bounded) for all ranks' gate flags.
// Enqueued in front of the pipelined kernel it lines the ranks up, so a rank that is ahead of its peers
// parks 32 threads instead of a grid of blocks that hold shared memory while they wait.
cudaError_t lbc_pipe_gate(uint8_t* const* arena, int world, int rank, int64_t ctl_off, unsigned int epoch,
                          unsigned long long timeout_ns, void* status, cudaStream_t stream);
// Geometry the host needs to size regions and chunks.
int lbc_pipe_stage_bytes(int dtype, int group_size, int bit, int world, int stages, int with_residual,
                         int with_prepared);

// ---- general path: top-k, 4-bit code-books, stochastic rounding --------------
typedef struct {
    int dtype, group_size, bit, topk, quant_type, stochastic, compact;
    const void* x;
    const void* residual;
    void* prepared_out;
    int64_t numel;
    uint8_t* out;
    unsigned long long seed;
    // Fused push (num_dst > 0): every piece of the payload is stored to dst[0..num_dst) instead of `out`
    // (own arena or a peer's over NVLink), and the grid raises `signal` after its last store.
    uint8_t* dst[LBC_MAX_RANKS];
    int num_dst;
    LbcSignal signal;
    int max_blocks;            // 0 = library default
    // Scatter (shard_groups > 0, with destinations): group g goes to dst[g / shard_groups] only, as group
    // g % shard_groups of a self-contained payload of shard_groups groups (a reduce-scatter's first half).
    int64_t shard_groups;
} LbcQuantGeneral;

typedef struct {
    int dtype, group_size, bit, topk, quant_type, compact;
    const uint8_t* src;
    int64_t numel;
    void* out;
    int accumulate;
} LbcDequantGeneral;

// Waits (bounded) for `wait`, then decodes src[0..num_src) group by group, sums them in the source dtype in
// source order (acc = T(acc + T(decode))), the rule of decoding one payload after the other with `accumulate`),
// applies out = T(float(acc) * scale) when scale != 1, and with `prepared` also writes
// residual_out = T(float(prepared) - float(out)).  One pass over the output for W payloads.
typedef struct {
    int dtype, group_size, bit, topk, quant_type, compact;
    const uint8_t* src[LBC_MAX_RANKS];
    int num_src;
    int64_t numel;
    void* out;
    float scale;
    const void* prepared;      // optional T[numel] (may alias residual_out)
    void* residual_out;        // optional T[numel]
    LbcWait wait;
    int max_blocks;            // 0 = library default
    int64_t layout_groups;     // groups in every source layout (planar payloads keep their scales behind that many
                               // groups of codes); 0 = the groups of `numel`
    int64_t src_shard_groups;  // > 0: gather mode, group g is read from src[g / src_shard_groups] only, as group
                               // g % src_shard_groups of a payload of src_shard_groups groups (layout_groups unused)
} LbcReduceGeneral;

cudaError_t lbc_quant_general(const LbcQuantGeneral* p, cudaStream_t stream);
cudaError_t lbc_dequant_general(const LbcDequantGeneral* p, cudaStream_t stream);
cudaError_t lbc_reduce_general(const LbcReduceGeneral* p, cudaStream_t stream);

// ---- elementwise helpers ----------------------------------------------------
// residual = T(float(prepared) - float(restored))
cudaError_t lbc_error_feedback_update(int dtype, const void* prepared, const void* restored, void* residual,
                                      int64_t numel, cudaStream_t stream);
// x = T(float(x) * scale)
cudaError_t lbc_scale_inplace(int dtype, void* x, float scale, int64_t numel, cudaStream_t stream);

// ---- transport helpers ------------------------------------------------------
// Copies `nbytes` (multiple of 16, 16-byte aligned) to every dst, then signals.
cudaError_t lbc_push_bytes(const uint8_t* src, int64_t nbytes, uint8_t* const* dst, int num_dst,
                           const LbcWait* wait_before, const LbcSignal* signal, int max_blocks,
                           cudaStream_t stream);
// Waits (bounded) for flags; optionally signals afterwards (acknowledgement).
cudaError_t lbc_wait_signal(const LbcWait* wait, const LbcSignal* signal, cudaStream_t stream);

int lbc_default_max_blocks(void);
// How quantized tiles reach their destinations: push_variant 0 classic grid-stride kernel,
// 1 shard-interleaved tiles with per-thread stores, 2 tiles handed to the bulk-store engine;
// reduce_bulk selects bulk stores for the requantize-and-broadcast stage; reduce_push_blocks caps the
// grid of that stage (0 = two blocks per SM, negative = no cap) so that every block amortises its
// closing system-scope fence.
void lbc_set_push_variant(int push_variant, int reduce_bulk, int reduce_push_blocks);
// Gather-mode decode: 1 (default) deals 256-thread tiles round-robin over the source shards, 0 sweeps linearly.
void lbc_set_gather_order(int order);
// Gather-mode decode of 8-bit planar shards: 0 (default) runs the general reduce kernel, one 16-byte load in
// flight per thread; 2 or 4 runs the specialised kernel that issues the loads of that many tiles before it
// decodes the first (same results, more bytes in flight over NVLink).  Other values round down.
void lbc_set_gather_prefetch(int tiles);
int lbc_get_gather_prefetch(void);

#ifdef __cplusplus
}
#endif

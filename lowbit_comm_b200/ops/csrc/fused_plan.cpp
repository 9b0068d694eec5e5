// Native twin of `FusedWorkspace.all_reduce` (lowbit_comm_b200/parallel/fused.py).
//
// The reference re-plans on every call (ccdl_comm/cuda/shortcut.py:18-59 builds a
// registry per call; its executors walk Python schedules per step,
// cuda/transports/pipelined_ring.py:205-282).  Here the per-call host work is a
// handful of integer operations: measured launch gaps, not kernels, dominated
// small buckets when the launches were issued from Python.
//
// Optionally (`set_chunking`; off by default because it measured slower: persistent grids of
// neighbouring chunks do not interleave) large tensors are cut into chunks that flow through the three phases on three
// streams (push on the caller's stream, reduce and gather on two side streams), so
// the NVLink-bound phases of one chunk overlap the HBM-bound phases of its
// neighbours.  Every chunk is a complete small all-reduce with its own receive
// regions and its own flag channel; a one-block gate kernel in front of every
// waiting kernel does the (bounded) waiting, so no stream can fill the GPU with
// spinning blocks.  The side streams are joined back into the caller's stream at
// the end, which keeps the region-reuse argument of the single-stream version.
//
// A one-warp gate kernel sits in front of every waiting kernel also without chunking: a rank
// that is ahead of its peers parks 32 threads instead of filling its SMs with spinning blocks.
//
// A variant that staged the payload locally and let the copy engines deliver it (peer-to-peer
// cudaMemcpyAsync on a copy stream, flags raised by a one-warp kernel behind the copies) was
// measured on 2 x B200 and dropped: with both directions busy the engines moved the payload at
// about 420 GB/s, slower than the kernels' own peer stores (about 560 GB/s), e.g. 256 MiB in
// 0.60-0.67 ms against 0.45 ms.
#include "fused_plan.h"

#include <ATen/cuda/CUDAContext.h>

#include <algorithm>
#include <stdexcept>
#include <string>
#include <vector>

#include "lbc_api.h"

namespace py = pybind11;

namespace lbc {

namespace {

constexpr int kPhaseRS = 0, kPhaseAG = 1;
constexpr int kNumPhases = 4, kFlagSlots = 16;
constexpr int64_t kAlignGroups = 8;
constexpr int kMaxChunks = 8;

int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

void check(cudaError_t err, const char* what) {
    if (err != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
}

struct Regions {        // byte offsets inside every rank's arena, for one chunk
    int64_t rs, ag, gather;
    int64_t shard_stride, gather_stride;
    int channel;
};

class FusedAllReducePlan {
  public:
    FusedAllReducePlan(int dtype, int group_size, int bit, int rank, std::vector<uintptr_t> peer_ptrs,
                       std::vector<int64_t> rs_off, int64_t rs_bytes, int64_t ag_off, int64_t ag_bytes,
                       std::vector<int64_t> gather_off, int64_t gather_bytes, std::vector<int> channels,
                       int64_t counter_offset, unsigned long long timeout_ns, uintptr_t status_device, int max_blocks,
                       int64_t max_numel)
        : dtype_(dtype), group_(group_size), bit_(bit), rank_(rank), peers_(std::move(peer_ptrs)),
          rs_off_(std::move(rs_off)), rs_bytes_(rs_bytes), ag_off_(ag_off), ag_bytes_(ag_bytes),
          gather_off_(std::move(gather_off)), gather_bytes_(gather_bytes), channels_(std::move(channels)),
          counter_offset_(counter_offset), timeout_ns_(timeout_ns), status_(status_device), max_blocks_(max_blocks),
          max_numel_(max_numel) {
        world_ = static_cast<int>(peers_.size());
        if (world_ < 1 || world_ > LBC_MAX_RANKS) throw std::invalid_argument("bad world size");
        if (rank_ < 0 || rank_ >= world_) throw std::invalid_argument("bad rank");
        if (rs_off_.size() != 2) throw std::invalid_argument("two reduce-scatter regions are required");
        if (channels_.empty()) throw std::invalid_argument("at least one flag channel is required");
        group_bytes_ = group_ * bit_ / 8 + (dtype_ == LBC_FP32 ? 4 : 2);
        elem_bytes_ = dtype_ == LBC_FP32 ? 4 : 2;
    }

    ~FusedAllReducePlan() {
        for (auto& s : side_) {
            if (s.stream != nullptr) cudaStreamDestroy(s.stream);
            if (s.done != nullptr) cudaEventDestroy(s.done);
        }
        if (start_ != nullptr) cudaEventDestroy(start_);
    }

    void set_chunking(int64_t min_chunk_bytes, int max_chunks) {
        min_chunk_bytes_ = std::max<int64_t>(min_chunk_bytes, 4096);
        max_chunks_ = std::max(1, std::min(max_chunks, std::min<int>(kMaxChunks, static_cast<int>(channels_.size()))));
    }

    // Base of the NVLink multicast mapping of the arenas (0 = none): broadcasts then leave this GPU once.
    // The requantize-and-broadcast stage of the two-stage path uses it only on request: measured on
    // 8 GPUs its multicast form was slower above 64 MiB (the replica for the sender itself also
    // arrives over NVLink, so every GPU receives W/W instead of (W-1)/W of the payload).
    void set_multicast(uintptr_t mc_base, bool in_reduce_stage) {
        mc_base_ = mc_base;
        mc_reduce_ = in_reduce_stage;
    }

    // Gather stage by peer loads (default): the decode kernel reads every rank's reduced shard from
    // that rank's memory, so the second NVLink crossing hides behind decode and error feedback.
    // Off: the reduce stage stores its shard into every rank's gather region.
    void set_pull_gather(bool on) { pull_gather_ = on; }

    // Enqueues the collective on `stream`; returns the number of kernels launched.
    int all_reduce(uintptr_t x, uintptr_t out, uintptr_t residual, int64_t numel, int stages, double scale,
                   bool update_residual, bool ef_local, unsigned int epoch, uintptr_t stream_ptr) {
        if (numel < 0 || numel > max_numel_) throw std::invalid_argument("numel exceeds the workspace capacity");
        if (numel == 0) return 0;
        if (stages == 1 && gather_off_.size() != 2) throw std::invalid_argument("this plan has no gather region");
        cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
        const int parity = static_cast<int>(epoch & 1u);
        // chunk boundaries keep every chunk's shards whole multiples of eight groups
        const int64_t unit = int64_t(group_) * kAlignGroups * world_;
        int chunks = static_cast<int>(std::min<int64_t>(max_chunks_, (numel * elem_bytes_) / min_chunk_bytes_));
        chunks = std::max(1, chunks);
        const int64_t chunk_numel = round_up(ceil_div(numel, chunks), unit);
        chunks = static_cast<int>(ceil_div(numel, chunk_numel));
        const bool piped = chunks > 1;
        cudaStream_t s_reduce = stream, s_gather = stream;
        if (piped) {
            ensure_side_streams();
            check(cudaEventRecord(start_, stream), "cudaEventRecord(start)");
            for (auto& s : side_) check(cudaStreamWaitEvent(s.stream, start_, 0), "cudaStreamWaitEvent(start)");
            s_reduce = side_[0].stream;
            s_gather = stages == 1 ? side_[0].stream : side_[1].stream;
        }
        int launches = 0;
        int64_t rs_cursor = 0, ag_cursor = 0, gather_cursor = 0;
        for (int c = 0; c < chunks; ++c) {
            const int64_t first = c * chunk_numel;
            const int64_t n = std::min(chunk_numel, numel - first);
            const int64_t groups = ceil_div(n, group_);
            const int64_t shard_groups = round_up(ceil_div(groups, world_), kAlignGroups);
            const int64_t full_groups = round_up(groups, kAlignGroups);
            Regions r;
            r.channel = channels_[c];
            r.shard_stride = round_up(shard_groups * group_bytes_, 256);
            r.gather_stride = round_up(full_groups * group_bytes_, 256);
            r.rs = rs_off_[parity] + rs_cursor;
            r.ag = ag_off_ + ag_cursor;
            r.gather = stages == 1 ? gather_off_[parity] + gather_cursor : 0;
            rs_cursor += r.shard_stride * world_;
            ag_cursor += round_up(shard_groups * world_ * group_bytes_, 256);
            gather_cursor += r.gather_stride * world_;
            if (stages != 1 && (rs_cursor > rs_bytes_ || ag_cursor > ag_bytes_))
                throw std::runtime_error("chunked regions exceed the workspace");
            if (stages == 1 && gather_cursor > gather_bytes_) throw std::runtime_error("chunked regions exceed the workspace");
            const uintptr_t off = static_cast<uintptr_t>(first) * elem_bytes_;
            grid_cap_ = max_blocks_;
            launches += one_chunk(x + off, out + off, residual == 0 ? 0 : residual + off, n, stages, scale,
                                  update_residual, ef_local, epoch, r, shard_groups, full_groups, stream, s_reduce,
                                  s_gather);
        }
        if (piped) {
            const int used = stages == 1 ? 1 : 2;
            for (int i = 0; i < used; ++i) {
                check(cudaEventRecord(side_[i].done, side_[i].stream), "cudaEventRecord(done)");
                check(cudaStreamWaitEvent(stream, side_[i].done, 0), "cudaStreamWaitEvent(done)");
            }
        }
        return launches;
    }

    // Reduce-scatter to a dense shard: rank r receives the reduced elements [r * shard_numel, (r + 1) * shard_numel)
    // in `out_shard` (shard_numel = shard_groups * group size; the caller has zeroed what lies past the tensor's
    // end).  With a residual, error feedback uses this rank's own quantization error, written back in place.
    // Three launches (quantize-and-scatter, gate, reduce), one binding crossing.
    int reduce_scatter(uintptr_t x, uintptr_t out_shard, uintptr_t residual, int64_t numel, double scale,
                       bool update_residual, unsigned int epoch, uintptr_t stream_ptr) {
        if (numel < 0 || numel > max_numel_) throw std::invalid_argument("numel exceeds the workspace capacity");
        if (numel == 0) return 0;
        cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
        const int parity = static_cast<int>(epoch & 1u);
        const int64_t groups = ceil_div(numel, group_);
        const int64_t shard_groups = round_up(ceil_div(groups, world_), kAlignGroups);
        Regions r;
        r.channel = channels_[0];
        r.shard_stride = round_up(shard_groups * group_bytes_, 256);
        r.gather_stride = 0;
        r.rs = rs_off_[parity];
        r.ag = ag_off_;
        r.gather = 0;
        if (r.shard_stride * world_ > rs_bytes_) throw std::runtime_error("shards exceed the workspace");
        grid_cap_ = max_blocks_;
        LbcQuantPush q{};
        q.dtype = dtype_;
        q.group_size = group_;
        q.bit = bit_;
        q.x = reinterpret_cast<const void*>(x);
        q.residual = reinterpret_cast<const void*>(residual);
        q.local_ef_out = (residual != 0 && update_residual) ? reinterpret_cast<void*>(residual) : nullptr;
        q.numel = numel;
        q.num_dst = world_;
        q.max_blocks = grid_cap_;
        q.mode = LBC_PUSH_SCATTER;
        q.shard_groups = shard_groups;
        q.layout_groups = shard_groups;
        for (int d = 0; d < world_; ++d)
            q.dst[d] = reinterpret_cast<uint8_t*>(peers_[d] + r.rs + rank_ * r.shard_stride);
        fill_signal(q.signal, r.channel, kPhaseRS, epoch);
        check(lbc_quant_push(&q, stream), "quant_push(scatter)");

        const int64_t shard_numel = shard_groups * group_;
        const int64_t lo = rank_ * shard_numel;
        const int64_t valid = std::max<int64_t>(0, std::min(numel, lo + shard_numel) - lo);
        LbcReduce k = base_reduce(valid, scale);
        k.num_src = world_;
        for (int s = 0; s < world_; ++s)
            k.src[s] = reinterpret_cast<const uint8_t*>(peers_[rank_] + r.rs + s * r.shard_stride);
        k.layout_groups = shard_groups;
        k.out = valid > 0 ? reinterpret_cast<void*>(out_shard) : nullptr;
        fill_wait(k.wait, r.channel, kPhaseRS, epoch);
        gate(k.wait, stream);
        check(lbc_reduce(&k, stream), "reduce(shard, dense)");
        return 3;
    }

  private:
    struct Side {
        cudaStream_t stream = nullptr;
        cudaEvent_t done = nullptr;
    };

    void ensure_side_streams() {
        if (start_ != nullptr) return;
        int lo = 0, hi = 0;
        check(cudaDeviceGetStreamPriorityRange(&lo, &hi), "cudaDeviceGetStreamPriorityRange");
        for (auto& s : side_) {
            check(cudaStreamCreateWithPriority(&s.stream, cudaStreamNonBlocking, hi), "cudaStreamCreateWithPriority");
            check(cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming), "cudaEventCreateWithFlags");
        }
        check(cudaEventCreateWithFlags(&start_, cudaEventDisableTiming), "cudaEventCreateWithFlags");
    }

    int one_chunk(uintptr_t x, uintptr_t out, uintptr_t residual, int64_t numel, int stages, double scale,
                  bool update_residual, bool ef_local, unsigned int epoch, const Regions& r, int64_t shard_groups,
                  int64_t full_groups, cudaStream_t s_push, cudaStream_t s_reduce, cudaStream_t s_gather) const {
        const bool want_ref = residual != 0 && update_residual && !ef_local;
        const bool want_local = residual != 0 && update_residual && ef_local;
        LbcQuantPush q{};
        q.dtype = dtype_;
        q.group_size = group_;
        q.bit = bit_;
        q.x = reinterpret_cast<const void*>(x);
        q.residual = reinterpret_cast<const void*>(residual);
        q.prepared_out = want_ref ? reinterpret_cast<void*>(residual) : nullptr;
        q.local_ef_out = want_local ? reinterpret_cast<void*>(residual) : nullptr;
        q.numel = numel;
        q.num_dst = world_;
        q.max_blocks = grid_cap_;
        fill_signal(q.signal, r.channel, kPhaseRS, epoch);

        if (stages == 1) {
            q.mode = LBC_PUSH_BROADCAST;
            q.layout_groups = full_groups;
            for (int d = 0; d < world_; ++d)
                q.dst[d] = reinterpret_cast<uint8_t*>(peers_[d] + r.gather + rank_ * r.gather_stride);
            if (mc_base_ != 0) q.mc_dst = reinterpret_cast<uint8_t*>(mc_base_ + r.gather + rank_ * r.gather_stride);
            check(lbc_quant_push(&q, s_push), "quant_push(broadcast)");
            LbcReduce k = base_reduce(numel, scale);
            k.num_src = world_;
            for (int s = 0; s < world_; ++s)
                k.src[s] = reinterpret_cast<const uint8_t*>(peers_[rank_] + r.gather + s * r.gather_stride);
            k.layout_groups = full_groups;
            k.out = reinterpret_cast<void*>(out);
            if (want_ref) {
                k.prepared = reinterpret_cast<const void*>(residual);
                k.residual_out = reinterpret_cast<void*>(residual);
            }
            fill_wait(k.wait, r.channel, kPhaseRS, epoch);
            gate(k.wait, s_reduce);
            check(lbc_reduce(&k, s_reduce), "reduce(one stage)");
            return 3;
        }

        q.mode = LBC_PUSH_SCATTER;
        q.shard_groups = shard_groups;
        q.layout_groups = shard_groups;
        for (int d = 0; d < world_; ++d)
            q.dst[d] = reinterpret_cast<uint8_t*>(peers_[d] + r.rs + rank_ * r.shard_stride);
        check(lbc_quant_push(&q, s_push), "quant_push(scatter)");

        const int64_t shard_numel = shard_groups * group_;
        const int64_t lo = rank_ * shard_numel;
        const int64_t valid = std::max<int64_t>(0, std::min(numel, lo + shard_numel) - lo);
        LbcReduce k2 = base_reduce(valid, scale);
        k2.num_src = world_;
        for (int s = 0; s < world_; ++s)
            k2.src[s] = reinterpret_cast<const uint8_t*>(peers_[rank_] + r.rs + s * r.shard_stride);
        k2.layout_groups = shard_groups;
        if (pull_gather_) {
            // the reduced shard stays in this rank's own gather region as a self-contained payload;
            // peers fetch it from there with the loads of their decode kernel
            k2.num_dst = 1;
            k2.dst[0] = reinterpret_cast<uint8_t*>(peers_[rank_] + r.ag);
            k2.dst_layout_groups = shard_groups;
            k2.dst_group_offset = 0;
        } else {
            k2.num_dst = world_;
            for (int d = 0; d < world_; ++d) k2.dst[d] = reinterpret_cast<uint8_t*>(peers_[d] + r.ag);
            if (mc_base_ != 0 && mc_reduce_) k2.mc_dst = reinterpret_cast<uint8_t*>(mc_base_ + r.ag);
            k2.dst_layout_groups = shard_groups * world_;
            k2.dst_group_offset = rank_ * shard_groups;
        }
        fill_signal(k2.signal, r.channel, kPhaseAG, epoch);
        fill_wait(k2.wait, r.channel, kPhaseRS, epoch);
        gate(k2.wait, s_reduce);
        check(lbc_reduce(&k2, s_reduce), "reduce(shard)");

        LbcReduce k3 = base_reduce(numel, 1.0);
        if (pull_gather_) {
            k3.num_src = world_;
            for (int s = 0; s < world_; ++s) k3.src[s] = reinterpret_cast<const uint8_t*>(peers_[s] + r.ag);
            k3.src_shard_groups = shard_groups;
            k3.first_src = rank_;
            k3.layout_groups = shard_groups;
        } else {
            k3.num_src = 1;
            k3.src[0] = reinterpret_cast<const uint8_t*>(peers_[rank_] + r.ag);
            k3.layout_groups = shard_groups * world_;
        }
        k3.out = reinterpret_cast<void*>(out);
        if (want_ref) {
            k3.prepared = reinterpret_cast<const void*>(residual);
            k3.residual_out = reinterpret_cast<void*>(residual);
        }
        fill_wait(k3.wait, r.channel, kPhaseAG, epoch);
        gate(k3.wait, s_gather);
        check(lbc_reduce(&k3, s_gather), "reduce(gather)");
        return 5;
    }


    // A one-block kernel does the (bounded) waiting, so that a rank that is ahead of its peers
    // parks 256 threads instead of filling every SM with spinning blocks while its own backward
    // pass still needs them; the reduce kernel that follows finds its flags already set.
    void gate(const LbcWait& wait, cudaStream_t stream) const {
        check(lbc_wait_signal(&wait, nullptr, stream), "wait_signal");
    }
    uintptr_t flags_addr(int rank, int channel, int phase) const {
        return peers_[rank] + static_cast<uintptr_t>((channel * kNumPhases + phase) * kFlagSlots) * 4;
    }
    void fill_signal(LbcSignal& s, int channel, int phase, unsigned int epoch) const {
        s.num_remote = world_;
        for (int d = 0; d < world_; ++d)
            s.remote_flags[d] = reinterpret_cast<unsigned int*>(flags_addr(d, channel, phase));
        s.my_slot = rank_;
        s.epoch = epoch;
        s.block_counter = reinterpret_cast<unsigned int*>(peers_[rank_] + counter_offset_ +
                                                          static_cast<uintptr_t>(channel * kNumPhases + phase) * 4);
    }
    void fill_wait(LbcWait& w, int channel, int phase, unsigned int epoch) const {
        w.flags = reinterpret_cast<const unsigned int*>(flags_addr(rank_, channel, phase));
        w.count = world_;
        w.epoch = epoch;
        w.timeout_ns = timeout_ns_;
        w.status = reinterpret_cast<void*>(status_);
        w.phase = static_cast<unsigned int>(phase);
    }
    LbcReduce base_reduce(int64_t numel, double scale) const {
        LbcReduce r{};
        r.dtype = dtype_;
        r.group_size = group_;
        r.bit = bit_;
        r.numel = numel;
        r.scale = static_cast<float>(scale);
        r.max_blocks = grid_cap_;
        return r;
    }

    int dtype_, group_, bit_, rank_, world_ = 1;
    std::vector<uintptr_t> peers_;
    std::vector<int64_t> rs_off_;
    int64_t rs_bytes_, ag_off_, ag_bytes_;
    std::vector<int64_t> gather_off_;
    int64_t gather_bytes_;
    std::vector<int> channels_;
    int64_t counter_offset_;
    unsigned long long timeout_ns_;
    uintptr_t status_;
    int max_blocks_;
    int64_t max_numel_;
    uintptr_t mc_base_ = 0;
    bool mc_reduce_ = false;
    bool pull_gather_ = true;
    int64_t group_bytes_ = 66, elem_bytes_ = 2;
    int64_t min_chunk_bytes_ = int64_t(8) << 20;
    int max_chunks_ = 1;
    mutable int grid_cap_ = 0;
    Side side_[2];
    cudaEvent_t start_ = nullptr;
};

// ---------------------------------------------------------------------------------------------
// Single-launch all-reduce: one persistent kernel per collective (pipe_kernels.cu).  The plan resolves
// the geometry (shards, rows) from the element count; regions are fixed at construction.
// ---------------------------------------------------------------------------------------------
class PipeAllReducePlan {
  public:
    PipeAllReducePlan(int dtype, int group_size, int bit, int rank, std::vector<uintptr_t> peer_ptrs, int64_t q_off,
                      int64_t q_bytes, int64_t ag_off, int64_t ag_bytes, int64_t ctl_off, unsigned long long timeout_ns,
                      uintptr_t status_device, int max_blocks, int64_t max_numel)
        : dtype_(dtype), group_(group_size), bit_(bit), rank_(rank), peers_(std::move(peer_ptrs)), q_off_(q_off),
          q_bytes_(q_bytes), ag_off_(ag_off), ag_bytes_(ag_bytes), ctl_off_(ctl_off), timeout_ns_(timeout_ns),
          status_(status_device), max_blocks_(max_blocks), max_numel_(max_numel) {
        world_ = static_cast<int>(peers_.size());
        if (world_ < 1 || world_ > LBC_MAX_RANKS) throw std::invalid_argument("bad world size");
        if (rank_ < 0 || rank_ >= world_) throw std::invalid_argument("bad rank");
        if (LBC_PIPE_ROW_ELEMS % group_ != 0) throw std::invalid_argument("group size must divide the row length");
        group_bytes_ = group_ * bit_ / 8 + (dtype_ == LBC_FP32 ? 4 : 2);
    }

    void set_ring_depth(int depth) { ring_depth_ = depth; }
    void set_max_blocks(int blocks) { max_blocks_ = blocks; }
    // Device buffer of [grid][8] 64-bit cycle counters filled by every launch (0 = off): where the blocks'
    // time goes (waiting for loads, computing, at barriers, claiming and issuing, asleep on flags).
    void set_profile_buffer(uintptr_t ptr) { profile_ = ptr; }

    // Enqueues the collective on `stream`; returns the number of kernels launched.
    int all_reduce(uintptr_t x, uintptr_t out, uintptr_t residual, int64_t numel, int stages, double scale,
                   bool update_residual, bool ef_local, unsigned int epoch, uintptr_t stream_ptr, int phase_mask,
                   bool gate) {
        if (numel < 0 || numel > max_numel_) throw std::invalid_argument("numel exceeds the workspace capacity");
        if (numel == 0) return 0;
        if (stages != 1 && stages != 2) throw std::invalid_argument("stages must be 1 or 2");
        cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
        LbcPipe p{};
        p.dtype = dtype_;
        p.group_size = group_;
        p.bit = bit_;
        p.world = world_;
        p.rank = rank_;
        p.stages = stages;
        p.phase_mask = phase_mask;
        p.x = reinterpret_cast<const void*>(x);
        p.out = reinterpret_cast<void*>(out);
        p.residual = reinterpret_cast<const void*>(residual);
        const bool want_ref = residual != 0 && update_residual && !ef_local;
        const bool want_local = residual != 0 && update_residual && ef_local;
        if (want_ref) {
            p.prepared_out = reinterpret_cast<void*>(residual);
            p.prepared = reinterpret_cast<const void*>(residual);
            p.residual_out = reinterpret_cast<void*>(residual);
        }
        if (want_local) p.local_ef_out = reinterpret_cast<void*>(residual);
        p.numel = numel;
        p.scale = static_cast<float>(scale);
        for (int r = 0; r < world_; ++r) p.arena[r] = reinterpret_cast<uint8_t*>(peers_[r]);
        const int shards = stages == 2 ? world_ : 1;
        const int64_t groups = ceil_div(numel, group_);
        p.shard_groups = round_up(ceil_div(groups, shards), kAlignGroups);
        p.shard_stride = round_up(p.shard_groups * group_bytes_, 256);
        if (p.shard_stride * shards > q_bytes_ || (stages == 2 && p.shard_groups * group_bytes_ > ag_bytes_))
            throw std::runtime_error("the pipelined workspace is too small for this tensor");
        p.q_off = q_off_;
        p.ag_off = ag_off_;
        p.ctl_off = ctl_off_;
        p.epoch = epoch;
        p.timeout_ns = timeout_ns_;
        p.status = reinterpret_cast<void*>(status_);
        p.max_blocks = max_blocks_;
        p.ring_depth = ring_depth_;
        p.profile = reinterpret_cast<unsigned long long*>(profile_);
        int launches = 0;
        if (gate && world_ > 1) {
            check(lbc_pipe_gate(p.arena, world_, rank_, ctl_off_, epoch, timeout_ns_, p.status, stream), "pipe_gate");
            ++launches;
        }
        check(lbc_pipe_allreduce(&p, stream), "pipe_allreduce");
        return launches + 1;
    }

  private:
    int dtype_, group_, bit_, rank_, world_ = 1;
    std::vector<uintptr_t> peers_;
    int64_t q_off_, q_bytes_, ag_off_, ag_bytes_, ctl_off_;
    unsigned long long timeout_ns_;
    uintptr_t status_;
    int max_blocks_;
    int64_t max_numel_;
    int64_t group_bytes_ = 66;
    int ring_depth_ = 0;
    uintptr_t profile_ = 0;
};

}  // namespace

void bind_fused_plan(py::module_& m) {
    py::class_<FusedAllReducePlan>(m, "FusedAllReducePlan")
        .def(py::init<int, int, int, int, std::vector<uintptr_t>, std::vector<int64_t>, int64_t, int64_t, int64_t,
                      std::vector<int64_t>, int64_t, std::vector<int>, int64_t, unsigned long long, uintptr_t, int,
                      int64_t>(),
             py::arg("dtype"), py::arg("group_size"), py::arg("bit"), py::arg("rank"), py::arg("peer_ptrs"),
             py::arg("rs_off"), py::arg("rs_bytes"), py::arg("ag_off"), py::arg("ag_bytes"), py::arg("gather_off"),
             py::arg("gather_bytes"), py::arg("channels"), py::arg("counter_offset"), py::arg("timeout_ns"),
             py::arg("status_device"), py::arg("max_blocks"), py::arg("max_numel"))
        .def("set_chunking", &FusedAllReducePlan::set_chunking, py::arg("min_chunk_bytes"), py::arg("max_chunks"))
        .def("set_multicast", &FusedAllReducePlan::set_multicast, py::arg("mc_base"), py::arg("in_reduce_stage") = false)
        .def("set_pull_gather", &FusedAllReducePlan::set_pull_gather, py::arg("on"))
        .def("all_reduce", &FusedAllReducePlan::all_reduce, py::arg("x"), py::arg("out"), py::arg("residual"),
             py::arg("numel"), py::arg("stages"), py::arg("scale"), py::arg("update_residual"), py::arg("ef_local"),
             py::arg("epoch"), py::arg("stream"))
        .def("reduce_scatter", &FusedAllReducePlan::reduce_scatter, py::arg("x"), py::arg("out_shard"),
             py::arg("residual"), py::arg("numel"), py::arg("scale"), py::arg("update_residual"), py::arg("epoch"),
             py::arg("stream"));
    py::class_<PipeAllReducePlan>(m, "PipeAllReducePlan")
        .def(py::init<int, int, int, int, std::vector<uintptr_t>, int64_t, int64_t, int64_t, int64_t, int64_t,
                      unsigned long long, uintptr_t, int, int64_t>(),
             py::arg("dtype"), py::arg("group_size"), py::arg("bit"), py::arg("rank"), py::arg("peer_ptrs"),
             py::arg("q_off"), py::arg("q_bytes"), py::arg("ag_off"), py::arg("ag_bytes"), py::arg("ctl_off"),
             py::arg("timeout_ns"), py::arg("status_device"), py::arg("max_blocks"), py::arg("max_numel"))
        .def("set_ring_depth", &PipeAllReducePlan::set_ring_depth, py::arg("depth"))
        .def("set_max_blocks", &PipeAllReducePlan::set_max_blocks, py::arg("blocks"))
        .def("set_profile_buffer", &PipeAllReducePlan::set_profile_buffer, py::arg("ptr"))
        .def("all_reduce", &PipeAllReducePlan::all_reduce, py::arg("x"), py::arg("out"), py::arg("residual"),
             py::arg("numel"), py::arg("stages"), py::arg("scale"), py::arg("update_residual"), py::arg("ef_local"),
             py::arg("epoch"), py::arg("stream"), py::arg("phase_mask") = static_cast<int>(LBC_PIPE_ALL),
             py::arg("gate") = false);
    // free-function form, so that callers that record and replay launches can treat it like the other launchers
    m.def("pipe_all_reduce",
          [](PipeAllReducePlan& plan, uintptr_t x, uintptr_t out, uintptr_t residual, int64_t numel, int stages,
             double scale, bool update_residual, bool ef_local, unsigned int epoch, uintptr_t stream, int phase_mask,
             bool gate) {
              return plan.all_reduce(x, out, residual, numel, stages, scale, update_residual, ef_local, epoch, stream,
                                     phase_mask, gate);
          });
    m.attr("PIPE_QUANT") = static_cast<int>(LBC_PIPE_QUANT);
    m.attr("PIPE_REDUCE") = static_cast<int>(LBC_PIPE_REDUCE);
    m.attr("PIPE_DECODE") = static_cast<int>(LBC_PIPE_DECODE);
    m.attr("PIPE_ALL") = static_cast<int>(LBC_PIPE_ALL);
    m.attr("PIPE_CTL_BYTES") = static_cast<int>(LBC_PIPE_CTL_BYTES);
    m.attr("PIPE_CTL_LOCAL") = static_cast<int>(LBC_PIPE_CTL_LOCAL);
}

}  // namespace lbc

// Native twin of `FusedWorkspace.all_reduce` (lowbit_comm_b200/parallel/fused.py).
//
// The reference re-plans on every call (ccdl_comm/cuda/shortcut.py:18-59 builds a
// registry per call; its executors walk Python schedules per step,
// cuda/transports/pipelined_ring.py:205-282).  Here the per-call host work is a
// handful of integer operations: measured launch gaps, not kernels, dominated
// small buckets when the three launches were issued from Python.
#include "fused_plan.h"

#include <ATen/cuda/CUDAContext.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "lbc_api.h"

namespace py = pybind11;

namespace lbc {

namespace {

constexpr int kPhaseRS = 0, kPhaseAG = 1;
constexpr int kNumPhases = 4, kFlagSlots = 16;
constexpr int64_t kCounterOffset = 64 * kNumPhases * kFlagSlots * 4;
constexpr int64_t kAlignGroups = 8;

int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

void check(cudaError_t err, const char* what) {
    if (err != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
}

class FusedAllReducePlan {
  public:
    FusedAllReducePlan(int dtype, int group_size, int bit, int rank, std::vector<uintptr_t> peer_ptrs,
                       std::vector<int64_t> rs_off, int64_t ag_off, std::vector<int64_t> gather_off,
                       int64_t shard_stride, int64_t gather_stride, int channel, unsigned long long timeout_ns,
                       uintptr_t status_device, int max_blocks, int64_t max_numel)
        : dtype_(dtype), group_(group_size), bit_(bit), rank_(rank), peers_(std::move(peer_ptrs)),
          rs_off_(std::move(rs_off)), ag_off_(ag_off), gather_off_(std::move(gather_off)),
          shard_stride_(shard_stride), gather_stride_(gather_stride), channel_(channel), timeout_ns_(timeout_ns),
          status_(status_device), max_blocks_(max_blocks), max_numel_(max_numel) {
        world_ = static_cast<int>(peers_.size());
        if (world_ < 1 || world_ > LBC_MAX_RANKS) throw std::invalid_argument("bad world size");
        if (rank_ < 0 || rank_ >= world_) throw std::invalid_argument("bad rank");
        if (rs_off_.size() != 2) throw std::invalid_argument("two reduce-scatter regions are required");
        value_bytes_ = group_ * bit_ / 8;
        scale_bytes_ = dtype_ == LBC_FP32 ? 4 : 2;
    }

    // Enqueues the collective on `stream`; returns the number of kernels launched.
    int all_reduce(uintptr_t x, uintptr_t out, uintptr_t residual, int64_t numel, int stages, double scale,
                   bool update_residual, bool ef_local, unsigned int epoch, uintptr_t stream_ptr) {
        if (numel < 0 || numel > max_numel_) throw std::invalid_argument("numel exceeds the workspace capacity");
        if (numel == 0) return 0;
        cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
        const int parity = static_cast<int>(epoch & 1u);
        const int64_t groups = ceil_div(numel, group_);
        int64_t shard_groups = ceil_div(groups, world_);
        shard_groups = ceil_div(shard_groups, kAlignGroups) * kAlignGroups;
        const int64_t full_groups = ceil_div(groups, kAlignGroups) * kAlignGroups;
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
        q.max_blocks = max_blocks_;
        fill_signal(q.signal, kPhaseRS, epoch);

        if (stages == 1) {
            if (gather_off_.size() != 2) throw std::invalid_argument("this plan has no gather region");
            q.mode = LBC_PUSH_BROADCAST;
            q.layout_groups = full_groups;
            for (int d = 0; d < world_; ++d)
                q.dst[d] = reinterpret_cast<uint8_t*>(peers_[d] + gather_off_[parity] + rank_ * gather_stride_);
            check(lbc_quant_push(&q, stream), "quant_push(broadcast)");
            LbcReduce r = base_reduce(numel, scale);
            r.num_src = world_;
            for (int s = 0; s < world_; ++s)
                r.src[s] = reinterpret_cast<const uint8_t*>(peers_[rank_] + gather_off_[parity] + s * gather_stride_);
            r.layout_groups = full_groups;
            r.out = reinterpret_cast<void*>(out);
            if (want_ref) {
                r.prepared = reinterpret_cast<const void*>(residual);
                r.residual_out = reinterpret_cast<void*>(residual);
            }
            fill_wait(r.wait, kPhaseRS, epoch);
            gate(r.wait, stream);
            check(lbc_reduce(&r, stream), "reduce(one stage)");
            return 3;
        }

        q.mode = LBC_PUSH_SCATTER;
        q.shard_groups = shard_groups;
        q.layout_groups = shard_groups;
        for (int d = 0; d < world_; ++d)
            q.dst[d] = reinterpret_cast<uint8_t*>(peers_[d] + rs_off_[parity] + rank_ * shard_stride_);
        check(lbc_quant_push(&q, stream), "quant_push(scatter)");

        const int64_t shard_numel = shard_groups * group_;
        const int64_t lo = rank_ * shard_numel;
        int64_t valid = (numel < lo + shard_numel ? numel : lo + shard_numel) - lo;
        if (valid < 0) valid = 0;
        LbcReduce k2 = base_reduce(valid, scale);
        k2.num_src = world_;
        for (int s = 0; s < world_; ++s)
            k2.src[s] = reinterpret_cast<const uint8_t*>(peers_[rank_] + rs_off_[parity] + s * shard_stride_);
        k2.layout_groups = shard_groups;
        k2.num_dst = world_;
        for (int d = 0; d < world_; ++d) k2.dst[d] = reinterpret_cast<uint8_t*>(peers_[d] + ag_off_);
        k2.dst_layout_groups = shard_groups * world_;
        k2.dst_group_offset = rank_ * shard_groups;
        fill_signal(k2.signal, kPhaseAG, epoch);
        fill_wait(k2.wait, kPhaseRS, epoch);
        gate(k2.wait, stream);
        check(lbc_reduce(&k2, stream), "reduce(shard)");

        LbcReduce k3 = base_reduce(numel, 1.0);
        k3.num_src = 1;
        k3.src[0] = reinterpret_cast<const uint8_t*>(peers_[rank_] + ag_off_);
        k3.layout_groups = shard_groups * world_;
        k3.out = reinterpret_cast<void*>(out);
        if (want_ref) {
            k3.prepared = reinterpret_cast<const void*>(residual);
            k3.residual_out = reinterpret_cast<void*>(residual);
        }
        fill_wait(k3.wait, kPhaseAG, epoch);
        gate(k3.wait, stream);
        check(lbc_reduce(&k3, stream), "reduce(gather)");
        return 5;
    }

  private:
    // A one-block kernel does the (bounded) waiting, so that a rank that is ahead of its peers
    // parks 256 threads instead of filling every SM with spinning blocks while its own backward
    // pass still needs them; the reduce kernel that follows finds its flags already set.
    void gate(const LbcWait& wait, cudaStream_t stream) const {
        check(lbc_wait_signal(&wait, nullptr, stream), "wait_signal");
    }
    uintptr_t flags_addr(int rank, int phase) const {
        return peers_[rank] + static_cast<uintptr_t>((channel_ * kNumPhases + phase) * kFlagSlots) * 4;
    }
    void fill_signal(LbcSignal& s, int phase, unsigned int epoch) const {
        s.num_remote = world_;
        for (int d = 0; d < world_; ++d) s.remote_flags[d] = reinterpret_cast<unsigned int*>(flags_addr(d, phase));
        s.my_slot = rank_;
        s.epoch = epoch;
        s.block_counter = reinterpret_cast<unsigned int*>(peers_[rank_] + kCounterOffset +
                                                          static_cast<uintptr_t>(channel_ * kNumPhases + phase) * 4);
    }
    void fill_wait(LbcWait& w, int phase, unsigned int epoch) const {
        w.flags = reinterpret_cast<const unsigned int*>(flags_addr(rank_, phase));
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
        r.max_blocks = max_blocks_;
        return r;
    }

    int dtype_, group_, bit_, rank_, world_ = 1;
    std::vector<uintptr_t> peers_;
    std::vector<int64_t> rs_off_;
    int64_t ag_off_;
    std::vector<int64_t> gather_off_;
    int64_t shard_stride_, gather_stride_;
    int channel_;
    unsigned long long timeout_ns_;
    uintptr_t status_;
    int max_blocks_;
    int64_t max_numel_;
    int value_bytes_ = 0, scale_bytes_ = 0;
};

}  // namespace

void bind_fused_plan(py::module_& m) {
    py::class_<FusedAllReducePlan>(m, "FusedAllReducePlan")
        .def(py::init<int, int, int, int, std::vector<uintptr_t>, std::vector<int64_t>, int64_t, std::vector<int64_t>,
                      int64_t, int64_t, int, unsigned long long, uintptr_t, int, int64_t>(),
             py::arg("dtype"), py::arg("group_size"), py::arg("bit"), py::arg("rank"), py::arg("peer_ptrs"),
             py::arg("rs_off"), py::arg("ag_off"), py::arg("gather_off"), py::arg("shard_stride"),
             py::arg("gather_stride"), py::arg("channel"), py::arg("timeout_ns"), py::arg("status_device"),
             py::arg("max_blocks"), py::arg("max_numel"))
        .def("all_reduce", &FusedAllReducePlan::all_reduce, py::arg("x"), py::arg("out"), py::arg("residual"),
             py::arg("numel"), py::arg("stages"), py::arg("scale"), py::arg("update_residual"), py::arg("ef_local"),
             py::arg("epoch"), py::arg("stream"));
}

}  // namespace lbc

// Python bindings of the sm_100a extension `_lbc_cuda`.
//
// The reference exposes its kernels as `ccdl_cuda_ops` (csrc/pybind.cpp:133-166)
// with one entry per (operation, in-place?) pair.  Here two fused launchers do
// the work (`quant_push`, `reduce`) and take raw device addresses for their
// destinations, because a destination may be another GPU's memory that no
// tensor of this process describes.  The reference's entry-point names are
// provided on top of these in lowbit_comm_b200/ops/codec.py.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <optional>
#include <string>
#include <tuple>
#include <vector>

#include "fused_plan.h"
#include "lbc_api.h"
#include "peer_memory.h"
#include "work.h"

namespace py = pybind11;

namespace {

using Ptrs = std::vector<uintptr_t>;
// (remote flag array addresses, my slot, epoch, local block counter address)
using SignalArg = std::optional<std::tuple<Ptrs, int, unsigned int, uintptr_t>>;
// (local flag array address, count, epoch, timeout ns, status device address, phase)
using WaitArg = std::optional<std::tuple<uintptr_t, int, unsigned int, unsigned long long, uintptr_t, unsigned int>>;

void cuda_check(cudaError_t err, const char* what) {
    TORCH_CHECK(err == cudaSuccess, what, ": ", cudaGetErrorString(err));
}

int dtype_code(const at::Tensor& t) {
    switch (t.scalar_type()) {
        case at::kHalf: return LBC_FP16;
        case at::kBFloat16: return LBC_BF16;
        case at::kFloat: return LBC_FP32;
        default: TORCH_CHECK(false, "unsupported source dtype ", t.scalar_type());
    }
}

void check_dense(const at::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

const void* opt_ptr(const std::optional<at::Tensor>& t, const at::Tensor& like, const char* name) {
    if (!t.has_value()) return nullptr;
    check_dense(*t, name);
    TORCH_CHECK(t->scalar_type() == like.scalar_type(), name, " must have the dtype of the input");
    TORCH_CHECK(t->numel() == like.numel(), name, " must have the input's number of elements");
    TORCH_CHECK(t->device() == like.device(), name, " must be on the input's device");
    return t->data_ptr();
}

void fill_ptrs(uint8_t** dst, int* count, const Ptrs& ptrs, const char* name) {
    TORCH_CHECK(ptrs.size() <= LBC_MAX_RANKS, name, ": at most ", LBC_MAX_RANKS, " entries");
    *count = static_cast<int>(ptrs.size());
    for (size_t i = 0; i < ptrs.size(); ++i) {
        TORCH_CHECK(ptrs[i] != 0, name, ": null address");
        dst[i] = reinterpret_cast<uint8_t*>(ptrs[i]);
    }
}

LbcSignal make_signal(const SignalArg& arg) {
    LbcSignal s{};
    if (!arg.has_value()) return s;
    const auto& [flags, slot, epoch, counter] = *arg;
    TORCH_CHECK(flags.size() <= LBC_MAX_RANKS, "signal: too many destinations");
    TORCH_CHECK(counter != 0 || flags.empty(), "signal: block counter address is required");
    s.num_remote = static_cast<int>(flags.size());
    for (size_t i = 0; i < flags.size(); ++i) s.remote_flags[i] = reinterpret_cast<unsigned int*>(flags[i]);
    s.my_slot = slot;
    s.epoch = epoch;
    s.block_counter = reinterpret_cast<unsigned int*>(counter);
    return s;
}

LbcWait make_wait(const WaitArg& arg) {
    LbcWait w{};
    if (!arg.has_value()) return w;
    const auto& [flags, count, epoch, timeout_ns, status, phase] = *arg;
    TORCH_CHECK(count >= 0 && count <= 256, "wait: count out of range");
    w.flags = reinterpret_cast<const unsigned int*>(flags);
    w.count = flags == 0 ? 0 : count;
    w.epoch = epoch;
    w.timeout_ns = timeout_ns;
    w.status = reinterpret_cast<void*>(status);
    w.phase = phase;
    return w;
}

int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---------------------------------------------------------------------------
void quant_push(const at::Tensor& x, const std::optional<at::Tensor>& residual,
                const std::optional<at::Tensor>& prepared_out, const std::optional<at::Tensor>& local_ef_out,
                const Ptrs& dst, int mode, int64_t shard_groups, int64_t layout_groups, int64_t group_offset,
                int group_size, int bit, const SignalArg& signal, int max_blocks, uintptr_t mc_dst) {
    check_dense(x, "input");
    c10::cuda::CUDAGuard guard(x.device());
    LbcQuantPush p{};
    p.dtype = dtype_code(x);
    p.group_size = group_size;
    p.bit = bit;
    p.x = x.data_ptr();
    p.residual = opt_ptr(residual, x, "residual");
    p.prepared_out = const_cast<void*>(opt_ptr(prepared_out, x, "prepared_out"));
    p.local_ef_out = const_cast<void*>(opt_ptr(local_ef_out, x, "local_ef_out"));
    p.numel = x.numel();
    p.mode = mode;
    fill_ptrs(p.dst, &p.num_dst, dst, "dst");
    const int64_t groups = ceil_div(p.numel, group_size);
    if (mode == LBC_PUSH_SCATTER) {
        TORCH_CHECK(shard_groups > 0, "scatter needs shard_groups > 0");
        TORCH_CHECK(ceil_div(groups, shard_groups) <= p.num_dst, "scatter: more shards than destinations");
        TORCH_CHECK(layout_groups >= shard_groups, "scatter: layout_groups < shard_groups");
    } else if (mode == LBC_PUSH_BROADCAST) {
        TORCH_CHECK(group_offset >= 0 && group_offset + groups <= layout_groups,
                    "broadcast: groups do not fit the destination layout");
        TORCH_CHECK(p.num_dst >= 1 || groups == 0, "broadcast needs a destination");
    } else {
        TORCH_CHECK(mode == LBC_PUSH_COMPACT_LOCAL && p.num_dst == 1, "compact mode writes one local payload");
    }
    p.shard_groups = shard_groups;
    p.layout_groups = layout_groups;
    p.group_offset = group_offset;
    p.signal = make_signal(signal);
    p.max_blocks = max_blocks;
    TORCH_CHECK(mc_dst == 0 || mode == LBC_PUSH_BROADCAST, "a multicast destination needs broadcast mode");
    p.mc_dst = reinterpret_cast<uint8_t*>(mc_dst);
    cuda_check(lbc_quant_push(&p, at::cuda::getCurrentCUDAStream()), "lbc_quant_push");
}

void reduce(const Ptrs& src, int64_t layout_groups, int64_t group_offset, bool compact, int64_t numel, int dtype,
            int group_size, int bit, double scale, const std::optional<at::Tensor>& out, bool accumulate,
            const std::optional<at::Tensor>& prepared, const std::optional<at::Tensor>& residual_out, const Ptrs& dst,
            int64_t dst_layout_groups, int64_t dst_group_offset, const SignalArg& signal, const WaitArg& wait,
            int max_blocks, uintptr_t mc_dst, int64_t src_shard_groups, int first_src) {
    LbcReduce p{};
    p.dtype = dtype;
    p.group_size = group_size;
    p.bit = bit;
    TORCH_CHECK(src.size() <= LBC_MAX_RANKS, "at most ", LBC_MAX_RANKS, " payloads per launch");
    p.num_src = static_cast<int>(src.size());
    for (size_t i = 0; i < src.size(); ++i) {
        TORCH_CHECK(src[i] != 0, "src: null address");
        p.src[i] = reinterpret_cast<const uint8_t*>(src[i]);
    }
    const int64_t groups = ceil_div(numel, group_size);
    if (src_shard_groups > 0) {
        TORCH_CHECK(!compact && numel >= 0 && group_offset >= 0, "gather mode reads planar shards");
        TORCH_CHECK(groups == 0 || (group_offset + groups - 1) / src_shard_groups < static_cast<int64_t>(src.size()),
                    "gather mode: more shards than sources");
    } else {
        TORCH_CHECK(numel >= 0 && group_offset >= 0 && group_offset + groups <= layout_groups,
                    "source groups do not fit the source layout");
    }
    p.src_shard_groups = src_shard_groups;
    p.first_src = src_shard_groups > 0 ? first_src : 0;
    p.layout_groups = layout_groups;
    p.group_offset = group_offset;
    p.compact = compact ? 1 : 0;
    p.numel = numel;
    p.scale = static_cast<float>(scale);
    auto typed = [&](const std::optional<at::Tensor>& t, const char* name) -> void* {
        if (!t.has_value()) return nullptr;
        check_dense(*t, name);
        TORCH_CHECK(dtype_code(*t) == dtype, name, " has the wrong dtype");
        TORCH_CHECK(t->numel() == numel, name, " must have numel elements");
        return t->data_ptr();
    };
    p.out = typed(out, "out");
    p.accumulate = accumulate ? 1 : 0;
    p.prepared = typed(prepared, "prepared");
    p.residual_out = typed(residual_out, "residual_out");
    TORCH_CHECK((p.prepared == nullptr) == (p.residual_out == nullptr), "prepared and residual_out go together");
    fill_ptrs(p.dst, &p.num_dst, dst, "dst");
    if (p.num_dst > 0)
        TORCH_CHECK(dst_group_offset >= 0 && dst_group_offset + groups <= dst_layout_groups,
                    "reduced groups do not fit the destination layout");
    p.dst_layout_groups = dst_layout_groups;
    p.dst_group_offset = dst_group_offset;
    p.signal = make_signal(signal);
    p.wait = make_wait(wait);
    p.max_blocks = max_blocks;
    TORCH_CHECK(mc_dst == 0 || p.num_dst > 0, "a multicast destination needs the unicast destinations too");
    p.mc_dst = reinterpret_cast<uint8_t*>(mc_dst);
    cuda_check(lbc_reduce(&p, at::cuda::getCurrentCUDAStream()), "lbc_reduce");
}

void quant_general(const at::Tensor& x, const std::optional<at::Tensor>& residual,
                   const std::optional<at::Tensor>& prepared_out, at::Tensor& out, int group_size, int bit, int topk,
                   int quant_type, bool stochastic, bool compact, uint64_t seed) {
    check_dense(x, "input");
    check_dense(out, "output");
    TORCH_CHECK(out.scalar_type() == at::kByte, "output must be uint8");
    c10::cuda::CUDAGuard guard(x.device());
    LbcQuantGeneral p{};
    p.dtype = dtype_code(x);
    p.group_size = group_size;
    p.bit = bit;
    p.topk = topk;
    p.quant_type = quant_type;
    p.stochastic = stochastic ? 1 : 0;
    p.compact = compact ? 1 : 0;
    p.x = x.data_ptr();
    p.residual = opt_ptr(residual, x, "residual");
    p.prepared_out = const_cast<void*>(opt_ptr(prepared_out, x, "prepared_out"));
    p.numel = x.numel();
    const int64_t meta_words = topk == 0 ? 1 : (topk == 1 ? 3 : 4);
    const int64_t need = ceil_div(p.numel, group_size) * (group_size * bit / 8 + meta_words * x.element_size());
    TORCH_CHECK(out.numel() == need, "output has an invalid quantized payload size: ", out.numel(), " != ", need);
    p.out = out.data_ptr<uint8_t>();
    p.seed = seed;
    cuda_check(lbc_quant_general(&p, at::cuda::getCurrentCUDAStream()), "lbc_quant_general");
}

void dequant_general(const at::Tensor& src, at::Tensor& out, int group_size, int bit, int topk, int quant_type,
                     bool compact, bool accumulate) {
    check_dense(src, "payload");
    check_dense(out, "output");
    TORCH_CHECK(src.scalar_type() == at::kByte, "payload must be uint8");
    c10::cuda::CUDAGuard guard(out.device());
    LbcDequantGeneral p{};
    p.dtype = dtype_code(out);
    p.group_size = group_size;
    p.bit = bit;
    p.topk = topk;
    p.quant_type = quant_type;
    p.compact = compact ? 1 : 0;
    p.numel = out.numel();
    const int64_t meta_words = topk == 0 ? 1 : (topk == 1 ? 3 : 4);
    const int64_t need = ceil_div(p.numel, group_size) * (group_size * bit / 8 + meta_words * out.element_size());
    TORCH_CHECK(src.numel() == need, "payload has an invalid size: ", src.numel(), " != ", need);
    p.src = src.data_ptr<uint8_t>();
    p.out = out.data_ptr();
    p.accumulate = accumulate ? 1 : 0;
    cuda_check(lbc_dequant_general(&p, at::cuda::getCurrentCUDAStream()), "lbc_dequant_general");
}

// quant_general with the stores going straight into every destination slot, and a signal at the end.
void quant_general_push(const at::Tensor& x, const std::optional<at::Tensor>& residual,
                        const std::optional<at::Tensor>& prepared_out, const Ptrs& dst, int group_size, int bit, int topk,
                        int quant_type, bool stochastic, bool compact, uint64_t seed, const SignalArg& signal,
                        int max_blocks, int64_t shard_groups) {
    check_dense(x, "input");
    TORCH_CHECK(!dst.empty(), "dst: at least one destination");
    c10::cuda::CUDAGuard guard(x.device());
    LbcQuantGeneral p{};
    p.dtype = dtype_code(x);
    p.group_size = group_size;
    p.bit = bit;
    p.topk = topk;
    p.quant_type = quant_type;
    p.stochastic = stochastic ? 1 : 0;
    p.compact = compact ? 1 : 0;
    p.x = x.data_ptr();
    p.residual = opt_ptr(residual, x, "residual");
    p.prepared_out = const_cast<void*>(opt_ptr(prepared_out, x, "prepared_out"));
    p.numel = x.numel();
    p.seed = seed;
    fill_ptrs(p.dst, &p.num_dst, dst, "dst");
    p.signal = make_signal(signal);
    p.max_blocks = max_blocks;
    p.shard_groups = shard_groups;
    cuda_check(lbc_quant_general(&p, at::cuda::getCurrentCUDAStream()), "lbc_quant_general(push)");
}

// Bounded wait, then one pass that decodes and sums every source payload, scales, and updates the residual.
void reduce_general(const Ptrs& src, at::Tensor& out, int group_size, int bit, int topk, int quant_type, bool compact,
                    double scale, const std::optional<at::Tensor>& prepared, const std::optional<at::Tensor>& residual_out,
                    const WaitArg& wait, int max_blocks, int64_t layout_groups, int64_t src_shard_groups) {
    check_dense(out, "output");
    TORCH_CHECK(prepared.has_value() == residual_out.has_value(), "prepared and residual_out come together");
    c10::cuda::CUDAGuard guard(out.device());
    LbcReduceGeneral p{};
    p.dtype = dtype_code(out);
    p.group_size = group_size;
    p.bit = bit;
    p.topk = topk;
    p.quant_type = quant_type;
    p.compact = compact ? 1 : 0;
    uint8_t* ptrs[LBC_MAX_RANKS];
    fill_ptrs(ptrs, &p.num_src, src, "src");
    for (int r = 0; r < p.num_src; ++r) p.src[r] = ptrs[r];
    p.numel = out.numel();
    p.out = out.data_ptr();
    p.scale = static_cast<float>(scale);
    p.prepared = opt_ptr(prepared, out, "prepared");
    p.residual_out = const_cast<void*>(opt_ptr(residual_out, out, "residual_out"));
    p.wait = make_wait(wait);
    p.max_blocks = max_blocks;
    p.layout_groups = layout_groups;
    p.src_shard_groups = src_shard_groups;
    cuda_check(lbc_reduce_general(&p, at::cuda::getCurrentCUDAStream()), "lbc_reduce_general");
}

void error_feedback_update(const at::Tensor& prepared, const at::Tensor& restored, at::Tensor& residual) {
    check_dense(prepared, "prepared");
    check_dense(restored, "restored");
    check_dense(residual, "residual");
    TORCH_CHECK(prepared.scalar_type() == restored.scalar_type() && prepared.scalar_type() == residual.scalar_type(),
                "prepared, restored and residual must share a dtype");
    TORCH_CHECK(prepared.numel() == restored.numel() && prepared.numel() == residual.numel(),
                "prepared, restored and residual must have the same number of elements");
    c10::cuda::CUDAGuard guard(prepared.device());
    cuda_check(lbc_error_feedback_update(dtype_code(prepared), prepared.data_ptr(), restored.data_ptr(),
                                         residual.data_ptr(), prepared.numel(), at::cuda::getCurrentCUDAStream()),
               "lbc_error_feedback_update");
}

void scale_inplace(at::Tensor& x, double scale) {
    check_dense(x, "tensor");
    c10::cuda::CUDAGuard guard(x.device());
    cuda_check(lbc_scale_inplace(dtype_code(x), x.data_ptr(), static_cast<float>(scale), x.numel(),
                                 at::cuda::getCurrentCUDAStream()),
               "lbc_scale_inplace");
}

void push_bytes(uintptr_t src, int64_t nbytes, const Ptrs& dst, const WaitArg& wait, const SignalArg& signal,
                int max_blocks) {
    uint8_t* ptrs[LBC_MAX_RANKS];
    int count = 0;
    fill_ptrs(ptrs, &count, dst, "dst");
    const LbcWait w = make_wait(wait);
    const LbcSignal s = make_signal(signal);
    cuda_check(lbc_push_bytes(reinterpret_cast<const uint8_t*>(src), nbytes, ptrs, count, &w, &s, max_blocks,
                              at::cuda::getCurrentCUDAStream()),
               "lbc_push_bytes");
}

void wait_signal(const WaitArg& wait, const SignalArg& signal) {
    const LbcWait w = make_wait(wait);
    const LbcSignal s = make_signal(signal);
    cuda_check(lbc_wait_signal(&w, &s, at::cuda::getCurrentCUDAStream()), "lbc_wait_signal");
}

at::Tensor tensor_from_address(uintptr_t ptr, int64_t nbytes, int device_index) {
    TORCH_CHECK(ptr != 0 && nbytes >= 0, "bad address or size");
    auto options = at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device_index);
    return at::from_blob(reinterpret_cast<void*>(ptr), {nbytes}, [](void*) {}, options);
}

void memset_async(uintptr_t ptr, int value, int64_t nbytes) {
    cuda_check(cudaMemsetAsync(reinterpret_cast<void*>(ptr), value, nbytes, at::cuda::getCurrentCUDAStream()),
               "cudaMemsetAsync");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "sm_100a kernels and peer-memory runtime of lowbit_comm_b200";
    m.attr("MAX_RANKS") = LBC_MAX_RANKS;
    m.attr("PUSH_BROADCAST") = static_cast<int>(LBC_PUSH_BROADCAST);
    m.attr("PUSH_SCATTER") = static_cast<int>(LBC_PUSH_SCATTER);
    m.attr("PUSH_COMPACT_LOCAL") = static_cast<int>(LBC_PUSH_COMPACT_LOCAL);
    m.attr("ARCH") = "sm_100a";

    m.def("quant_push", &quant_push, py::arg("x"), py::arg("residual"), py::arg("prepared_out"),
          py::arg("local_ef_out"), py::arg("dst"), py::arg("mode"), py::arg("shard_groups"), py::arg("layout_groups"),
          py::arg("group_offset"), py::arg("group_size"), py::arg("bit"), py::arg("signal") = py::none(),
          py::arg("max_blocks") = 0, py::arg("mc_dst") = 0);
    m.def("reduce", &reduce, py::arg("src"), py::arg("layout_groups"), py::arg("group_offset"), py::arg("compact"),
          py::arg("numel"), py::arg("dtype"), py::arg("group_size"), py::arg("bit"), py::arg("scale"), py::arg("out"),
          py::arg("accumulate"), py::arg("prepared"), py::arg("residual_out"), py::arg("dst"),
          py::arg("dst_layout_groups"), py::arg("dst_group_offset"), py::arg("signal") = py::none(),
          py::arg("wait") = py::none(), py::arg("max_blocks") = 0, py::arg("mc_dst") = 0,
          py::arg("src_shard_groups") = 0, py::arg("first_src") = 0);
    m.def("quant_general", &quant_general);
    m.def("dequant_general", &dequant_general);
    m.def("quant_general_push", &quant_general_push, py::arg("x"), py::arg("residual"), py::arg("prepared_out"),
          py::arg("dst"), py::arg("group_size"), py::arg("bit"), py::arg("topk"), py::arg("quant_type"),
          py::arg("stochastic"), py::arg("compact"), py::arg("seed"), py::arg("signal") = py::none(),
          py::arg("max_blocks") = 0, py::arg("shard_groups") = 0);
    m.def("reduce_general", &reduce_general, py::arg("src"), py::arg("out"), py::arg("group_size"), py::arg("bit"),
          py::arg("topk"), py::arg("quant_type"), py::arg("compact"), py::arg("scale"), py::arg("prepared") = py::none(),
          py::arg("residual_out") = py::none(), py::arg("wait") = py::none(), py::arg("max_blocks") = 0,
          py::arg("layout_groups") = 0, py::arg("src_shard_groups") = 0);
    m.def("error_feedback_update", &error_feedback_update);
    m.def("scale_inplace", &scale_inplace);
    m.def("push_bytes", &push_bytes, py::arg("src"), py::arg("nbytes"), py::arg("dst"), py::arg("wait") = py::none(),
          py::arg("signal") = py::none(), py::arg("max_blocks") = 0);
    m.def("wait_signal", &wait_signal, py::arg("wait") = py::none(), py::arg("signal") = py::none());
    m.def("default_max_blocks", [] { return lbc_default_max_blocks(); });
    m.def("set_push_variant",
          [](int push, bool reduce_bulk, int reduce_push_blocks) {
              lbc_set_push_variant(push, reduce_bulk ? 1 : 0, reduce_push_blocks);
          },
          py::arg("push_variant"), py::arg("reduce_bulk") = false, py::arg("reduce_push_blocks") = 0);

    m.def("set_gather_order", [](int order) { lbc_set_gather_order(order); }, py::arg("order"));
    m.def("set_gather_prefetch", [](int tiles) { lbc_set_gather_prefetch(tiles); }, py::arg("tiles"));
    m.def("get_gather_prefetch", []() { return lbc_get_gather_prefetch(); });
    m.def("arena_alloc", &lbc::arena_alloc);
    m.def("arena_free", &lbc::arena_free);
    m.def("ipc_get_handle", [](uintptr_t p) { return py::bytes(lbc::ipc_get_handle(p)); });
    m.def("ipc_open_handle", [](const py::bytes& b) { return lbc::ipc_open_handle(std::string(b)); });
    m.def("ipc_close_handle", &lbc::ipc_close_handle);
    m.def("can_access_peer", &lbc::can_access_peer);
    m.def("enable_peer_access", &lbc::enable_peer_access);
    m.def("status_alloc", [] { auto s = lbc::status_alloc(); return py::make_tuple(s.host, s.device); });
    m.def("status_free", &lbc::status_free);
    m.def("status_read", [](uintptr_t host) {
        const LbcStatus s = lbc::status_read(host);
        return py::make_tuple(s.code, s.phase, s.peer, s.seen, s.expected);
    });
    m.def("status_clear", &lbc::status_clear);
    m.def("tensor_from_address", &tensor_from_address);
    m.def("memset_async", &memset_async);

    lbc::bind_work(m);
    lbc::bind_fused_plan(m);
}

// Native completion object returned by asynchronous collectives.
//
// Role parity with the reference's CompressedWork / CudaExecutor
// (csrc/executor/compressed_work.cpp:52-226, cuda_executor.cpp:7-36): it owns
// the result, an optional transport handle, a completion event, the buffers
// that must outlive the launch and a one-shot Python callback.  The first
// `wait()` finishes the operation; concurrent waiters sleep on a condition
// variable without holding the GIL; the first error is kept and raised again by
// every later `wait()`; `query()` never runs the callback.
//
// Differences: the completion event can be a CUDA event recorded and owned here
// (`record(stream)`), `wait()` makes the *current stream* wait on it rather than
// the host, and a host-mapped status word written by bounded device waits is
// turned into an exception by `synchronize()` / `check_status()`.
#include "work.h"

#include <ATen/cuda/CUDAContext.h>
#include <cuda_runtime.h>

#include <stdexcept>

#include "peer_memory.h"

namespace lbc {

namespace {

bool py_ready(const py::object& obj) {
    if (obj.is_none()) return true;
    for (const char* name : {"is_completed", "query"}) {
        if (py::hasattr(obj, name)) return obj.attr(name)().cast<bool>();
    }
    return false;
}

void py_call_optional(const py::object& obj, const char* name) {
    if (!obj.is_none() && py::hasattr(obj, name)) obj.attr(name)();
}

}  // namespace

CompressedWork::CompressedWork(py::object result, py::object transport_work, py::object completion,
                               std::vector<py::object> resources, py::object callback, uintptr_t status_host)
    : result_(std::move(result)), transport_(std::move(transport_work)), completion_(std::move(completion)),
      resources_(std::move(resources)), callback_(std::move(callback)), status_host_(status_host) {}

CompressedWork::~CompressedWork() {
    if (event_ != nullptr) cudaEventDestroy(static_cast<cudaEvent_t>(event_));
}

void CompressedWork::record(uintptr_t stream) {
    if (event_ == nullptr) {
        cudaEvent_t ev = nullptr;
        if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess)
            throw std::runtime_error("cudaEventCreateWithFlags failed");
        event_ = ev;
        cudaGetDevice(&device_);
    }
    if (cudaEventRecord(static_cast<cudaEvent_t>(event_), reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess)
        throw std::runtime_error("cudaEventRecord failed");
}

bool CompressedWork::query() const {
    {
        std::lock_guard<std::mutex> guard(mutex_);
        if (phase_ == Phase::Done) return true;
    }
    if (!py_ready(transport_)) return false;
    if (!callback_.is_none() && !callback_ran_) return false;
    if (event_ != nullptr) return cudaEventQuery(static_cast<cudaEvent_t>(event_)) == cudaSuccess;
    return py_ready(completion_);
}

void CompressedWork::finish_locked_out() {
    // Runs with the GIL held and the mutex released, by exactly one thread.
    try {
        py_call_optional(transport_, "wait");
        if (!callback_.is_none() && !callback_ran_) {
            callback_ran_ = true;
            result_ = callback_();
        }
        if (event_ != nullptr) {
            cudaStream_t current = at::cuda::getCurrentCUDAStream(device_).stream();
            if (cudaStreamWaitEvent(current, static_cast<cudaEvent_t>(event_), 0) != cudaSuccess)
                throw std::runtime_error("cudaStreamWaitEvent failed");
        } else if (!completion_.is_none()) {
            if (py::hasattr(completion_, "wait")) completion_.attr("wait")();
            else py_call_optional(completion_, "synchronize");
        }
    } catch (py::error_already_set& err) {
        py_error_ = std::make_shared<py::error_already_set>(err);
    } catch (...) {
        cpp_error_ = std::current_exception();
    }
    resources_.clear();
    callback_ = py::none();
}

py::object CompressedWork::wait() {
    bool mine = false, self_wait = false;
    {
        py::gil_scoped_release nogil;
        std::unique_lock<std::mutex> lock(mutex_);
        if (phase_ == Phase::Idle) {
            phase_ = Phase::Running;
            runner_ = std::this_thread::get_id();
            mine = true;
        } else if (phase_ == Phase::Running && runner_ == std::this_thread::get_id()) {
            // the callback (or the transport's wait) of this very work called wait(): it would wait for itself
            self_wait = true;
        } else {
            done_cv_.wait(lock, [this] { return phase_ == Phase::Done; });
        }
    }
    if (self_wait)
        throw std::runtime_error("wait() was called by this work's own completion step; it would wait for itself");
    if (mine) {
        finish_locked_out();
        {
            py::gil_scoped_release nogil;
            std::lock_guard<std::mutex> guard(mutex_);
            phase_ = Phase::Done;
        }
        done_cv_.notify_all();
    }
    rethrow();
    return result_;
}

void CompressedWork::rethrow() const {
    if (py_error_) {
        // raise a fresh copy so that every waiter sees the same exception
        py::object type = py_error_->type(), value = py_error_->value(), trace = py_error_->trace();
        PyErr_Restore(type.inc_ref().ptr(), value.inc_ref().ptr(), trace ? trace.inc_ref().ptr() : nullptr);
        throw py::error_already_set();
    }
    if (cpp_error_) std::rethrow_exception(cpp_error_);
}

py::object CompressedWork::synchronize() {
    py::object out = wait();
    if (event_ != nullptr) {
        py::gil_scoped_release nogil;
        cudaEventSynchronize(static_cast<cudaEvent_t>(event_));
    }
    check_status();
    return out;
}

void CompressedWork::check_status() const {
    if (status_host_ == 0) return;
    const LbcStatus st = status_read(status_host_);
    if (st.code == 0) return;
    py::object exc_type = py::module_::import("lowbit_comm_b200.exceptions").attr("AsyncCommunicationError");
    py::dict info;
    info["code"] = st.code;
    info["phase"] = st.phase;
    info["peer"] = st.peer;
    info["seen"] = st.seen;
    info["expected"] = st.expected;
    py::object exc = exc_type(py::str("device wait timed out (phase {}, flag {}, saw epoch {}, expected {})")
                                  .format(st.phase, st.peer, st.seen, st.expected),
                              py::arg("status") = info);
    PyErr_SetObject(exc_type.ptr(), exc.ptr());
    throw py::error_already_set();
}

py::object CompressedWork::get_future() const {
    if (!transport_.is_none() && py::hasattr(transport_, "get_future")) return transport_.attr("get_future")();
    return py::none();
}

py::tuple CompressedWork::resources() const {
    py::tuple out(resources_.size());
    for (size_t i = 0; i < resources_.size(); ++i) out[i] = resources_[i];
    return out;
}

std::shared_ptr<CompressedWork> CudaExecutor::run(py::object result, py::object transport_work, py::object completion,
                                                  std::vector<py::object> resources, py::object callback,
                                                  uintptr_t status_host) const {
    return std::make_shared<CompressedWork>(std::move(result), std::move(transport_work), std::move(completion),
                                            std::move(resources), std::move(callback), status_host);
}

void bind_work(py::module_& m) {
    py::class_<CompressedWork, std::shared_ptr<CompressedWork>>(m, "CompressedWork")
        .def(py::init<py::object, py::object, py::object, std::vector<py::object>, py::object, uintptr_t>(),
             py::arg("result"), py::arg("transport_work") = py::none(), py::arg("completion") = py::none(),
             py::arg("resources") = std::vector<py::object>{}, py::arg("callback") = py::none(),
             py::arg("status_host") = 0)
        .def("wait", &CompressedWork::wait)
        .def("query", &CompressedWork::query)
        .def("get_future", &CompressedWork::get_future)
        .def("result", &CompressedWork::wait)
        .def("record", &CompressedWork::record, py::arg("stream"))
        .def("synchronize", &CompressedWork::synchronize)
        .def("check_status", &CompressedWork::check_status)
        .def_property_readonly("resources", &CompressedWork::resources)
        .def_property_readonly("uses_native_transport", [](const CompressedWork&) { return false; })
        .def_property_readonly("uses_native_completion", &CompressedWork::uses_native_completion);
    py::class_<CudaExecutor, std::shared_ptr<CudaExecutor>>(m, "CudaExecutor")
        .def(py::init<>())
        .def("run", &CudaExecutor::run, py::arg("result"), py::arg("transport_work") = py::none(),
             py::arg("completion") = py::none(), py::arg("resources") = std::vector<py::object>{},
             py::arg("callback") = py::none(), py::arg("status_host") = 0);
    m.def("create_cuda_executor", [] { return std::make_shared<CudaExecutor>(); });
    m.attr("NATIVE_WORK_ABI_VERSION") = 1;
}

}  // namespace lbc

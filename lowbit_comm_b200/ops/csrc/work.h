// Native asynchronous work object and its factory (see work.cpp).
#pragma once

#include <torch/extension.h>

#include <condition_variable>
#include <cstdint>
#include <exception>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace lbc {

class CompressedWork {
  public:
    CompressedWork(py::object result, py::object transport_work, py::object completion,
                   std::vector<py::object> resources, py::object callback, uintptr_t status_host);
    ~CompressedWork();
    CompressedWork(const CompressedWork&) = delete;
    CompressedWork& operator=(const CompressedWork&) = delete;

    void record(uintptr_t stream);   // record an owned CUDA event on `stream`
    bool query() const;              // never runs the callback
    py::object wait();               // current stream waits for the event
    py::object synchronize();        // wait() + host sync + status check
    void check_status() const;       // raises AsyncCommunicationError on a device time-out
    py::object get_future() const;
    py::tuple resources() const;
    bool uses_native_completion() const { return event_ != nullptr; }

  private:
    enum class Phase { Idle, Running, Done };
    void finish_locked_out();
    void rethrow() const;

    py::object result_, transport_, completion_;
    std::vector<py::object> resources_;
    py::object callback_;
    uintptr_t status_host_ = 0;
    void* event_ = nullptr;
    int device_ = 0;
    bool callback_ran_ = false;
    Phase phase_ = Phase::Idle;
    std::thread::id runner_;         // the thread inside finish_locked_out(), to refuse a wait on itself
    mutable std::mutex mutex_;
    std::condition_variable done_cv_;
    std::shared_ptr<py::error_already_set> py_error_;
    std::exception_ptr cpp_error_;
};

class CudaExecutor {
  public:
    std::shared_ptr<CompressedWork> run(py::object result, py::object transport_work, py::object completion,
                                        std::vector<py::object> resources, py::object callback,
                                        uintptr_t status_host) const;
};

void bind_work(py::module_& m);

}  // namespace lbc

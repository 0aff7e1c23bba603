// The torch.distributed front end in C++: a c10d::Backend whose collectives on CUDA tensors go
// from the dispatcher to a fused-kernel launch without entering Python.
//
// torch wraps the backend in its own C++ ProcessGroup, so dist.all_reduce / all_gather_into_tensor
// / reduce_scatter_tensor / broadcast / barrier (and with them DDP and FSDP2) reach allreduce() etc.
// below directly.  A call is planned and launched by the team's native engine (gb_engine.h) on the
// team's communication stream, ordered after the caller's stream with an event; the Work that comes
// back holds the event recorded behind the kernel: wait() makes the caller's stream wait for it and
// never blocks the host (the semantics of torch's NCCL backend).
//
// Everything else - CPU tensors, tensor lists, gather/scatter, point-to-point, compressed bridges,
// teams without an NVLink fabric - is handed to the Python process group of the same library
// (`fallback`), which implements the full surface; its Work objects are held alive here.
// Role of the reference's Python ProcessGroup (src/gpubridge/torch_backend.py).
#include <torch/extension.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/jit/python/pybind_utils.h>

#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <atomic>
#include <mutex>

#include "gb_engine.h"

namespace py = pybind11;

namespace {

int dtype_code(at::ScalarType t) {
    switch (t) {
        case at::kFloat: return 0;
        case at::kBFloat16: return 1;
        case at::kHalf: return 2;
        case at::kDouble: return 3;
        case at::kChar: return 4;
        case at::kByte: return 5;
        case at::kInt: return 6;
        case at::kLong: return 7;
        default: return -1;
    }
}

bool is_float(at::ScalarType t) {
    return t == at::kFloat || t == at::kBFloat16 || t == at::kHalf || t == at::kDouble;
}

// A collective that is in the communication stream.
class StreamWork : public c10d::Work {
 public:
    StreamWork(int rank, c10d::OpType op, std::vector<at::Tensor> outputs, c10::cuda::CUDAStream comm)
        : c10d::Work(rank, op), outputs_(std::move(outputs)), device_(comm.device()) {
        event_.record(comm);
        // A future that completes "on" the communication stream: then() callbacks and wait()
        // are ordered behind the kernel by the events the future records here.
        future_ = c10::make_intrusive<c10::ivalue::Future>(
            c10::ListType::create(c10::TensorType::get()), std::vector<c10::Device>{device_});
        c10::cuda::CUDAStreamGuard on_comm(comm);
        future_->markCompleted(c10::IValue(outputs_));
    }
    bool isCompleted() override { return event_.query(); }
    bool isSuccess() const override { return true; }
    bool wait(std::chrono::milliseconds /*timeout*/) override {
        event_.block(c10::cuda::getCurrentCUDAStream(device_.index()));
        return true;
    }
    void synchronize() override { wait(kNoTimeout); }
    void blockCurrentStream() override { wait(kNoTimeout); }
    std::vector<at::Tensor> result() override { return outputs_; }
    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }

 private:
    std::vector<at::Tensor> outputs_;
    c10::Device device_;
    at::cuda::CUDAEvent event_;
    c10::intrusive_ptr<c10::ivalue::Future> future_;
};

// A Work made by the Python group: the Python object stays alive as long as this one.
class HeldWork : public c10d::Work {
 public:
    HeldWork(int rank, py::object work) : c10d::Work(rank, c10d::OpType::UNKNOWN), work_(std::move(work)) {}
    ~HeldWork() override {
        py::gil_scoped_acquire gil;
        work_ = py::object();
    }
    bool isCompleted() override { return call<bool>("is_completed"); }
    bool isSuccess() const override { return const_cast<HeldWork*>(this)->call<bool>("is_success"); }
    bool wait(std::chrono::milliseconds timeout) override {
        py::gil_scoped_acquire gil;
        if (timeout == kNoTimeout) return work_.attr("wait")().cast<bool>();
        return work_.attr("wait")(timeout).cast<bool>();
    }
    void synchronize() override {
        py::gil_scoped_acquire gil;
        work_.attr("synchronize")();
    }
    std::vector<at::Tensor> result() override { return call<std::vector<at::Tensor>>("result"); }
    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override {
        py::gil_scoped_acquire gil;
        auto held = work_.attr("get_future")().cast<std::shared_ptr<torch::jit::PythonFutureWrapper>>();
        return held->fut;
    }

 private:
    template <typename T> T call(const char* name) {
        py::gil_scoped_acquire gil;
        return work_.attr(name)().cast<T>();
    }
    py::object work_;
};

struct NativeTeam {
    void* engine = nullptr;
    cudaStream_t stream = nullptr;         // the team's communication stream (shared with Python)
    int device = -1;
    int grid_cap = 0;
    std::vector<int> team_rank;            // group rank -> rank in the team's order
};

class GbBackend : public c10d::Backend {
 public:
    GbBackend(int rank, int size, py::object fallback)
        : c10d::Backend(rank, size), fallback_(std::move(fallback)) {}
    ~GbBackend() override {
        py::gil_scoped_acquire gil;
        fallback_ = py::object();
    }

    const std::string getBackendName() const override { return "gpubridge_native"; }

    // calls that went down the native path / to the Python group (tests and benchmarks read them)
    uint64_t nativeCalls() const { return native_calls_.load(); }
    uint64_t fallbackCalls() const { return fallback_calls_.load(); }
    void forget() {
        std::lock_guard<std::mutex> hold(lock_);
        team_ = NativeTeam();
        asked_ = false;
    }

    c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors,
                                             const c10d::AllreduceOptions& opts) override {
        int op = -1, divide = 0;
        bool floats_only = false;
        switch (opts.reduceOp.op_) {
            case c10d::ReduceOp::SUM: op = 0; break;
            case c10d::ReduceOp::AVG: op = 0; divide = getSize(); floats_only = true; break;
            case c10d::ReduceOp::MAX: op = 1; break;
            case c10d::ReduceOp::MIN: op = 2; break;
            default: break;
        }
        const NativeTeam* team = op >= 0 ? native_for(tensors) : nullptr;
        if (team != nullptr && floats_only)
            for (const auto& t : tensors) if (!is_float(t.scalar_type())) team = nullptr;
        if (team == nullptr) return via_python("allreduce", tensors, opts);
        // launches go to the team's GPU whatever device the caller has current
        c10::cuda::CUDAGuard on_device(c10::DeviceIndex(team->device));
        auto comm = enter(*team, tensors);
        for (auto& t : tensors) {
            if (t.numel() == 0) continue;
            check(gb_engine_all_reduce(team->engine, t.data_ptr(), t.data_ptr(), size_t(t.numel()),
                                       dtype_code(t.scalar_type()), op, divide, team->grid_cap, team->stream),
                  "all_reduce");
        }
        return leave(c10d::OpType::ALLREDUCE, tensors, comm);
    }

    c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor>& tensors,
                                                       const c10d::AllreduceCoalescedOptions& opts) override {
        return allreduce(tensors, opts);
    }

    c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors,
                                             const c10d::BroadcastOptions& opts) override {
        const NativeTeam* team = native_for(tensors);
        if (team == nullptr || opts.rootRank < 0 || size_t(opts.rootRank) >= team->team_rank.size())
            return via_python("broadcast", tensors, opts);
        // launches go to the team's GPU whatever device the caller has current
        c10::cuda::CUDAGuard on_device(c10::DeviceIndex(team->device));
        auto comm = enter(*team, tensors);
        for (auto& t : tensors) {
            if (t.numel() == 0) continue;
            check(gb_engine_broadcast(team->engine, t.data_ptr(), size_t(t.nbytes()),
                                      team->team_rank[size_t(opts.rootRank)], team->grid_cap, team->stream),
                  "broadcast");
        }
        return leave(c10d::OpType::BROADCAST, tensors, comm);
    }

    c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& output, at::Tensor& input,
                                                   const c10d::AllgatherOptions& opts) override {
        std::vector<at::Tensor> both{output, input};
        const NativeTeam* team = native_for(both);
        if (team == nullptr || output.scalar_type() != input.scalar_type() ||
            output.numel() != input.numel() * getSize() || !identity_order(*team)) {
            py::gil_scoped_acquire gil;
            return hold(fallback_.attr("_allgather_base")(output, input, opts));
        }
        // launches go to the team's GPU whatever device the caller has current
        c10::cuda::CUDAGuard on_device(c10::DeviceIndex(team->device));
        auto comm = enter(*team, both);
        if (input.numel() != 0)
            check(gb_engine_all_gather(team->engine, input.data_ptr(), output.data_ptr(), size_t(input.nbytes()),
                                       team->grid_cap, team->stream), "all_gather");
        std::vector<at::Tensor> outs{output};
        return leave(c10d::OpType::_ALLGATHER_BASE, outs, comm);
    }

    c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& output, at::Tensor& input,
                                                        const c10d::ReduceScatterOptions& opts) override {
        std::vector<at::Tensor> both{output, input};
        int divide = -1;
        if (opts.reduceOp.op_ == c10d::ReduceOp::SUM) divide = 0;
        else if (opts.reduceOp.op_ == c10d::ReduceOp::AVG && is_float(input.scalar_type())) divide = getSize();
        const NativeTeam* team = divide >= 0 ? native_for(both) : nullptr;
        if (team == nullptr || output.scalar_type() != input.scalar_type() ||
            input.numel() != output.numel() * getSize() || !identity_order(*team)) {
            py::gil_scoped_acquire gil;
            return hold(fallback_.attr("_reduce_scatter_base")(output, input, opts));
        }
        // launches go to the team's GPU whatever device the caller has current
        c10::cuda::CUDAGuard on_device(c10::DeviceIndex(team->device));
        auto comm = enter(*team, both);
        if (output.numel() != 0)
            check(gb_engine_reduce_scatter(team->engine, input.data_ptr(), output.data_ptr(), size_t(output.numel()),
                                           dtype_code(input.scalar_type()), divide, team->grid_cap, team->stream),
                  "reduce_scatter");
        std::vector<at::Tensor> outs{output};
        return leave(c10d::OpType::_REDUCE_SCATTER_BASE, outs, comm);
    }

    // -- the rest of the surface lives in the Python group ------------------------------------------
    c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputs,
                                             std::vector<at::Tensor>& inputs,
                                             const c10d::AllgatherOptions& opts) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("allgather")(outputs, inputs, opts));
    }
    c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(std::vector<at::Tensor>& outputs,
                                                                   std::vector<at::Tensor>& inputs,
                                                                   const c10d::AllgatherOptions& opts) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("allgather_into_tensor_coalesced")(outputs, inputs, opts));
    }
    c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outputs,
                                                  std::vector<std::vector<at::Tensor>>& inputs,
                                                  const c10d::ReduceScatterOptions& opts) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("reduce_scatter")(outputs, inputs, opts));
    }
    c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outputs,
                                                                   std::vector<at::Tensor>& inputs,
                                                                   const c10d::ReduceScatterOptions& opts) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("reduce_scatter_tensor_coalesced")(outputs, inputs, opts));
    }
    c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& outputs,
                                          std::vector<at::Tensor>& inputs, const c10d::GatherOptions& opts) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("gather")(outputs, inputs, opts));
    }
    c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& outputs,
                                           std::vector<std::vector<at::Tensor>>& inputs,
                                           const c10d::ScatterOptions& opts) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("scatter")(outputs, inputs, opts));
    }
    c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& opts) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("reduce")(tensors, opts));
    }
    c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dst, int tag) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("send")(tensors, dst, tag));
    }
    c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int src, int tag) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("recv")(tensors, src, tag));
    }
    // Refused by the library (with the reason, on every rank): let the Python group say so.
    c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& output, at::Tensor& input,
                                                 std::vector<int64_t>& output_splits,
                                                 std::vector<int64_t>& input_splits,
                                                 const c10d::AllToAllOptions& opts) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("alltoall_base")(output, input, output_splits, input_splits, opts));
    }
    c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
                                            const c10d::AllToAllOptions& opts) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("alltoall")(outputs, inputs, opts));
    }
    c10::intrusive_ptr<c10d::Work> recvAnysource(std::vector<at::Tensor>& tensors, int tag) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("recv_anysource")(tensors, tag));
    }
    c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& opts) override {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("barrier")(opts));
    }
    // Coalescing (batch_isend_irecv, coalesced collectives) is the Python group's: while a
    // batch is open every call goes there, so that it sees the whole batch.
    bool supportsCoalescing() const override { return true; }
    void startCoalescing() override {
        coalescing_.store(true);
        py::gil_scoped_acquire gil;
        fallback_.attr("_start_coalescing")(py::none());
    }
    c10::intrusive_ptr<c10d::Work> endCoalescing() override {
        coalescing_.store(false);
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr("_end_coalescing")(py::none()));
    }
    void shutdown() override {
        forget();
        py::gil_scoped_acquire gil;
        if (!fallback_.is_none()) fallback_.attr("shutdown")();
    }
    void abort() override { shutdown(); }

 private:
    template <typename Opts>
    c10::intrusive_ptr<c10d::Work> via_python(const char* name, std::vector<at::Tensor>& tensors, const Opts& opts) {
        py::gil_scoped_acquire gil;
        return hold(fallback_.attr(name)(tensors, opts));
    }

    // GIL held.
    c10::intrusive_ptr<c10d::Work> hold(py::object work) {
        fallback_calls_.fetch_add(1, std::memory_order_relaxed);
        if (work.is_none()) {       // the Python group answers None for "nothing to wait for"
            auto done = c10::make_intrusive<c10::ivalue::Future>(c10::NoneType::get());
            done->markCompleted();
            return c10d::Work::create_from_future(done);
        }
        return c10::make_intrusive<HeldWork>(getRank(), std::move(work));
    }

    // The team when every tensor can go down the native path, else null.
    const NativeTeam* native_for(const std::vector<at::Tensor>& tensors) {
        if (tensors.empty() || coalescing_.load()) return nullptr;
        for (const auto& t : tensors)
            if (!t.is_cuda() || !t.is_contiguous() || dtype_code(t.scalar_type()) < 0) return nullptr;
        {
            std::lock_guard<std::mutex> hold(lock_);
            if (!asked_) {
                // Once per group: the Python side builds the topology (a collective over the
                // store on first use) and says whether this team has an engine.
                py::gil_scoped_acquire gil;
                py::object answer = fallback_.attr("_native_team")();
                asked_ = true;
                if (!answer.is_none()) {
                    auto t = answer.cast<py::tuple>();
                    team_.engine = reinterpret_cast<void*>(t[0].cast<uintptr_t>());
                    team_.stream = reinterpret_cast<cudaStream_t>(t[1].cast<uintptr_t>());
                    team_.device = t[2].cast<int>();
                    team_.grid_cap = t[3].cast<int>();
                    team_.team_rank = t[4].cast<std::vector<int>>();
                }
            }
        }
        if (team_.engine == nullptr) return nullptr;
        for (const auto& t : tensors) if (t.get_device() != team_.device) return nullptr;
        if (gb_engine_status(team_.engine) != 0) {      // a device-side wait ran out earlier
            py::gil_scoped_acquire gil;
            fallback_.attr("_native_failed")();          // raises with the kernel's record
        }
        return &team_;
    }

    bool identity_order(const NativeTeam& team) const {
        // all_gather and reduce_scatter place slice r at team rank r: the group's order must be
        // the team's (it is, unless islands interleave the group's ranks)
        for (size_t r = 0; r < team.team_rank.size(); ++r) if (team.team_rank[r] != int(r)) return false;
        return true;
    }

    // The communication stream waits for the caller's stream; the allocator learns that the
    // tensors are in use there.
    c10::cuda::CUDAStream enter(const NativeTeam& team, const std::vector<at::Tensor>& tensors) {
        auto comm = c10::cuda::getStreamFromExternal(team.stream, c10::DeviceIndex(team.device));
        auto current = c10::cuda::getCurrentCUDAStream(c10::DeviceIndex(team.device));
        if (current != comm) {
            at::cuda::CUDAEvent ready;
            ready.record(current);
            ready.block(comm);
            for (const auto& t : tensors) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), comm);
        }
        native_calls_.fetch_add(1, std::memory_order_relaxed);
        return comm;
    }

    c10::intrusive_ptr<c10d::Work> leave(c10d::OpType op, std::vector<at::Tensor>& outputs,
                                         c10::cuda::CUDAStream comm) {
        return c10::make_intrusive<StreamWork>(getRank(), op, outputs, comm);
    }

    void check(int rc, const char* what) {
        if (rc == 0) return;
        TORCH_CHECK(false, "gpubridge_native backend: ", what, " could not be launched (",
                    rc < 0 ? "engine code " : "CUDA error ", rc, ")");
    }

    py::object fallback_;
    std::mutex lock_;
    bool asked_ = false;
    NativeTeam team_;
    std::atomic<uint64_t> native_calls_{0}, fallback_calls_{0};
    std::atomic<bool> coalescing_{false};
};

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    py::class_<GbBackend, c10d::Backend, c10::intrusive_ptr<GbBackend>>(m, "GbBackend")
        .def(py::init<int, int, py::object>(), py::arg("rank"), py::arg("size"), py::arg("fallback"))
        .def_property_readonly("native_calls", &GbBackend::nativeCalls)
        .def_property_readonly("fallback_calls", &GbBackend::fallbackCalls)
        .def("forget", &GbBackend::forget);
}

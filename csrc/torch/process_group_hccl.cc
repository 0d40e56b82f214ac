// torch.distributed backend "hccl": a c10d::Backend whose collectives are this library's C API.
//
// HCCL reaches PyTorch through torch_npu's ProcessGroupHCCL (not part of the reference repository; the reference ships only
// a usage sample, examples/03_ai_framework/01_pytorch/hccl_pytorch_allreduce_test.py:19-55). This is the equivalent for
// CUDA devices: root info travels through the c10d Store, CUDA tensors use a CUDA communicator on a dedicated stream
// (ordered after the caller's stream by an event; Work::wait() makes the caller's stream wait, never the host), CPU tensors
// use the host simulation backend so the same process group works in GPU-less tests.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>
#include <pybind11/chrono.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/extension.h>

#include <memory>
#include <mutex>

#include "hccl/hccl.h"
#include "hccl/hccl_res.h"
#include "hccl/hccl_dfx.h"

namespace {

#define HCCL_TORCH_CHECK(expr)                                                                       \
    do {                                                                                             \
        HcclResult _r = (expr);                                                                      \
        TORCH_CHECK(_r == HCCL_SUCCESS, #expr, " failed: HcclResult ", (int)_r, " (", HcclGetErrorString(_r), ")"); \
    } while (0)

HcclDataType ToHccl(at::ScalarType t)
{
    switch (t) {
        case at::kChar: return HCCL_DATA_TYPE_INT8;
        case at::kByte: case at::kBool: return HCCL_DATA_TYPE_UINT8;
        case at::kShort: return HCCL_DATA_TYPE_INT16;
        case at::kInt: return HCCL_DATA_TYPE_INT32;
        case at::kLong: return HCCL_DATA_TYPE_INT64;
        case at::kHalf: return HCCL_DATA_TYPE_FP16;
        case at::kFloat: return HCCL_DATA_TYPE_FP32;
        case at::kDouble: return HCCL_DATA_TYPE_FP64;
        case at::kBFloat16: return HCCL_DATA_TYPE_BFP16;
        case at::kFloat8_e4m3fn: return HCCL_DATA_TYPE_FP8E4M3;
        case at::kFloat8_e5m2: return HCCL_DATA_TYPE_FP8E5M2;
        default: TORCH_CHECK(false, "hccl backend: unsupported dtype ", t);
    }
}

HcclReduceOp ToHccl(const c10d::ReduceOp &op, bool *avg)
{
    *avg = false;
    switch (op.op_) {
        case c10d::ReduceOp::SUM: return HCCL_REDUCE_SUM;
        case c10d::ReduceOp::AVG: *avg = true; return HCCL_REDUCE_SUM;
        case c10d::ReduceOp::PRODUCT: return HCCL_REDUCE_PROD;
        case c10d::ReduceOp::MAX: return HCCL_REDUCE_MAX;
        case c10d::ReduceOp::MIN: return HCCL_REDUCE_MIN;
        default: TORCH_CHECK(false, "hccl backend: unsupported reduce op");
    }
}

class WorkHCCL : public c10d::Work {
public:
    WorkHCCL(c10d::OpType type, int rank, bool cuda, HcclComm comm) : c10d::Work(rank, type), cuda_(cuda), comm_(comm)
    {
        if (cuda_) C10_CUDA_CHECK(cudaEventCreateWithFlags(&event_, cudaEventDisableTiming));
    }
    ~WorkHCCL() override
    {
        if (cuda_ && event_) cudaEventDestroy(event_);
    }
    void recordEnd(cudaStream_t s) { C10_CUDA_CHECK(cudaEventRecord(event_, s)); }
    bool isCompleted() override
    {
        if (!cuda_) return done_;
        return cudaEventQuery(event_) == cudaSuccess;
    }
    bool isSuccess() const override { return true; }
    bool wait(std::chrono::milliseconds /*timeout*/ = kNoTimeout) override
    {
        if (cuda_) {
            // order the caller's current stream after the collective; the host does not block
            C10_CUDA_CHECK(cudaStreamWaitEvent(c10::cuda::getCurrentCUDAStream(), event_, 0));
        } else if (!done_) {
            HcclResult r = HcclSimStreamSynchronize(comm_);
            TORCH_CHECK(r == HCCL_SUCCESS, "hccl backend: collective failed: HcclResult ", (int)r, " (", HcclGetErrorString(r), ")");
            done_ = true;
        }
        return true;
    }
    void synchronize() override { wait(); }
    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }
    std::vector<at::Tensor> result() override { return outputs_; }
    void setOutputs(std::vector<at::Tensor> outs, cudaStream_t commStream)
    {
        outputs_ = std::move(outs);
        if (cuda_) {
            std::vector<c10::Device> devs;
            if (!outputs_.empty()) devs.push_back(outputs_[0].device());
            else devs.push_back(c10::Device(c10::kCUDA, c10::cuda::current_device()));
            future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()), devs);
            // a CUDA future records events on the current streams when it is completed: make the comm stream current
            c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(commStream, devs[0].index()));
            future_->markCompleted(c10::IValue(outputs_));
        } else {
            // host backend: point-to-point calls stay asynchronous (a send completes only when the peer receives, so
            // waiting here would deadlock two ranks that both send first); collectives complete before returning
            if (opType_ == c10d::OpType::SEND || opType_ == c10d::OpType::RECV) return;
            future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
            wait();
            future_->markCompleted(c10::IValue(outputs_));
        }
    }

private:
    bool cuda_;
    HcclComm comm_;
    cudaEvent_t event_ = nullptr;
    bool done_ = false;
    std::vector<at::Tensor> outputs_;
    c10::intrusive_ptr<c10::ivalue::Future> future_;
};

class ProcessGroupHCCL : public c10d::Backend {
public:
    ProcessGroupHCCL(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size) : c10d::Backend(rank, size), store_(store) {}
    ~ProcessGroupHCCL() override
    {
        for (auto &kv : comms_) {
            // work may still be queued on the private communication stream: let it finish before the communicator (and the
            // peer mappings its kernels use) goes away
            if (kv.second.cuda && kv.second.stream) {
                cudaSetDevice(kv.second.device);
                cudaStreamSynchronize(kv.second.stream);
            }
            if (kv.second.comm) HcclCommDestroy(kv.second.comm);
            if (kv.second.inputReady) cudaEventDestroy(kv.second.inputReady);
            if (kv.second.stream) cudaStreamDestroy(kv.second.stream);
        }
    }
    const std::string getBackendName() const override { return "hccl"; }

    struct CommEntry {
        HcclComm comm = nullptr;
        bool cuda = false;
        cudaStream_t stream = nullptr;
        cudaEvent_t inputReady = nullptr;
        int device = -1;
    };

    // One communicator per device kind, created on first use by all ranks (collective).
    CommEntry &entryFor(const at::Tensor &t)
    {
        std::lock_guard<std::mutex> lk(mu_);
        const bool cuda = t.is_cuda();
        const std::string key = cuda ? "cuda" : "cpu";
        auto it = comms_.find(key);
        if (it != comms_.end()) return it->second;
        CommEntry e;
        e.cuda = cuda;
        HcclRootInfo info;
        const std::string skey = "hccl_b200/root/" + key + "/" + std::to_string(generation_);
        if (getRank() == 0) {
            HCCL_TORCH_CHECK(HcclGetRootInfo(&info));
            std::vector<uint8_t> bytes(sizeof(info));
            memcpy(bytes.data(), &info, sizeof(info));
            store_->set(skey, bytes);
        } else {
            std::vector<uint8_t> bytes = store_->get(skey);
            TORCH_CHECK(bytes.size() == sizeof(info), "hccl backend: bad root info in store");
            memcpy(&info, bytes.data(), sizeof(info));
        }
        HcclCommConfig cfg;
        HcclCommConfigInit(&cfg);
        cfg.hcclBackend = cuda ? 2 : 1;
        if (cuda) {
            e.device = t.get_device();
            c10::cuda::CUDAGuard g(e.device);
            C10_CUDA_CHECK(cudaFree(nullptr));
            HCCL_TORCH_CHECK(HcclCommInitRootInfoConfig((uint32_t)getSize(), &info, (uint32_t)getRank(), &cfg, &e.comm));
            C10_CUDA_CHECK(cudaStreamCreateWithFlags(&e.stream, cudaStreamNonBlocking));
            C10_CUDA_CHECK(cudaEventCreateWithFlags(&e.inputReady, cudaEventDisableTiming));
            // The first CUDA communicator of the process serves the allocator hooks (unless the application attached one itself), so that
            // tensors created under hccl_b200.parallel.process_group.mem_pool() -- DistributedDataParallel's buckets, for instance --
            // are registered windows and their collectives run without staging copies.
            HcclComm attached = nullptr;
            if (HcclGetAllocatorComm(&attached) == HCCL_SUCCESS && attached == nullptr) HcclSetAllocatorComm(e.comm);
        } else {
            HCCL_TORCH_CHECK(HcclCommInitRootInfoConfig((uint32_t)getSize(), &info, (uint32_t)getRank(), &cfg, &e.comm));
        }
        return comms_.emplace(key, e).first->second;
    }

    // Runs `fn(comm, stream)` ordered after the caller's stream and returns the Work.
    template <typename F>
    c10::intrusive_ptr<c10d::Work> run(c10d::OpType type, const at::Tensor &ref, std::vector<at::Tensor> keepAlive, std::vector<at::Tensor> outputs, F &&fn)
    {
        CommEntry &e = entryFor(ref);
        auto work = c10::make_intrusive<WorkHCCL>(type, getRank(), e.cuda, e.comm);
        if (e.cuda) {
            c10::cuda::CUDAGuard g(e.device);
            cudaStream_t cur = c10::cuda::getCurrentCUDAStream(e.device);
            C10_CUDA_CHECK(cudaEventRecord(e.inputReady, cur));
            C10_CUDA_CHECK(cudaStreamWaitEvent(e.stream, e.inputReady, 0));
            auto cs = c10::cuda::getStreamFromExternal(e.stream, e.device);
            for (auto &t : keepAlive) if (t.defined() && t.is_cuda()) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), cs);
            fn(e.comm, e.stream);
            work->recordEnd(e.stream);
            work->setOutputs(std::move(outputs), e.stream);
        } else {
            fn(e.comm, nullptr);
            work->setOutputs(std::move(outputs), nullptr);
        }
        return work;
    }

    static void checkOne(const std::vector<at::Tensor> &v) { TORCH_CHECK(v.size() == 1, "hccl backend: expected exactly one tensor per call"); }
    static at::Tensor contig(const at::Tensor &t) { return t.is_contiguous() ? t : t.contiguous(); }
#include "process_group_ops.inc"

private:
    c10::intrusive_ptr<c10d::Store> store_;
    std::mutex mu_;
    std::map<std::string, CommEntry> comms_;
    int generation_ = 0;
};

c10::intrusive_ptr<c10d::Backend> createProcessGroupHCCL(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size,
                                                         const std::chrono::duration<float> & /*timeout*/)
{
    return c10::make_intrusive<ProcessGroupHCCL>(store, rank, size);
}

}  // namespace

PYBIND11_MODULE(hccl_b200_torch, m)
{
    m.doc() = "torch.distributed backend on the hccl_b200 C API";
    m.def("create_process_group", &createProcessGroupHCCL, py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout"));
}

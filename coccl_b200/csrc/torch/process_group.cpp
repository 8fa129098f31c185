// torch.distributed backend "coccl": a c10d::Backend whose all-reduce, reduce-scatter, all-gather
// and all-to-all go through the compression-aware runtime (router -> fused kernels / staged pipeline
// / native NCCL), while every other operation is delegated to an inner backend (ProcessGroupNCCL).
// The reference reaches PyTorch by preloading its libnccl.so into the trainer process
// (examples/training_scripts/train_qwen_coccl.sh:78-82); this backend is the explicit equivalent.
//
// Stream semantics follow ProcessGroupNCCL: work is enqueued on the caller's current CUDA stream and
// the returned Work is a marker (wait() is stream-ordered, it never blocks the host).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/extension.h>

#include <cstring>

#include "coccl/coccl.h"

namespace {

ncclDataType_t toNccl(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return ncclFloat32;
    case at::kHalf: return ncclFloat16;
    case at::kBFloat16: return ncclBfloat16;
    case at::kDouble: return ncclFloat64;
    case at::kInt: return ncclInt32;
    case at::kLong: return ncclInt64;
    case at::kChar: return ncclInt8;
    case at::kByte: return ncclUint8;
    case at::kBool: return ncclUint8;
    default: TORCH_CHECK(false, "coccl backend: unsupported dtype ", t);
  }
}

ncclRedOp_t toNccl(const c10d::ReduceOp& op) {
  switch (op) {
    case c10d::ReduceOp::SUM: return ncclSum;
    case c10d::ReduceOp::PRODUCT: return ncclProd;
    case c10d::ReduceOp::MIN: return ncclMin;
    case c10d::ReduceOp::MAX: return ncclMax;
    case c10d::ReduceOp::AVG: return ncclAvg;
    default: TORCH_CHECK(false, "coccl backend: unsupported reduce op");
  }
}

class MarkerWork : public c10d::Work {
 public:
  MarkerWork(int rank, c10d::OpType op, std::vector<at::Tensor> outputs)
      : c10d::Work(rank, op), outputs_(std::move(outputs)) {
    future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
    future_->markCompleted(c10::IValue(outputs_));
  }
  bool isCompleted() override { return true; }
  bool isSuccess() const override { return true; }
  bool wait(std::chrono::milliseconds) override { return true; }  // already ordered on the caller's stream
  std::vector<at::Tensor> result() override { return outputs_; }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }

 private:
  std::vector<at::Tensor> outputs_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
};

void check(ncclResult_t r, const char* what) {
  TORCH_CHECK(r == ncclSuccess, "coccl backend: ", what, " failed: ", cocclApiGetErrorString(r), " (", (int)r, ")");
}

}  // namespace

class ProcessGroupCoccl : public c10d::Backend {
 public:
  ProcessGroupCoccl(c10::intrusive_ptr<c10d::Backend> inner, c10::intrusive_ptr<c10d::Store> store, int rank, int size)
      : c10d::Backend(rank, size), inner_(std::move(inner)), store_(std::move(store)) {}

  ~ProcessGroupCoccl() override {
    if (comm_ != nullptr) cocclApiCommDestroy(comm_);
  }

  const std::string getBackendName() const override { return "coccl"; }

  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& opts) override {
    TORCH_CHECK(tensors.size() == 1, "coccl backend: one tensor per call");
    at::Tensor& t = tensors[0];
    if (!t.is_cuda() || !t.is_contiguous() || opts.reduceOp == c10d::ReduceOp::AVG) return inner_->allreduce(tensors, opts);
    ncclComm_t c = comm(t);
    check(cocclApiAllReduce(t.data_ptr(), t.data_ptr(), (size_t)t.numel(), toNccl(t.scalar_type()), toNccl(opts.reduceOp), c,
                            at::cuda::getCurrentCUDAStream(t.get_device())), "all_reduce");
    return marker(c10d::OpType::ALLREDUCE, {t});
  }

  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& out, at::Tensor& in, const c10d::ReduceScatterOptions& opts) override {
    if (!in.is_cuda() || !in.is_contiguous() || !out.is_contiguous() || opts.reduceOp == c10d::ReduceOp::AVG)
      return inner_->_reduce_scatter_base(out, in, opts);
    TORCH_CHECK(in.numel() == out.numel() * getSize(), "coccl backend: reduce_scatter size mismatch");
    ncclComm_t c = comm(in);
    check(cocclApiReduceScatter(in.data_ptr(), out.data_ptr(), (size_t)out.numel(), toNccl(in.scalar_type()), toNccl(opts.reduceOp), c,
                                at::cuda::getCurrentCUDAStream(in.get_device())), "reduce_scatter");
    return marker(c10d::OpType::_REDUCE_SCATTER_BASE, {out});
  }

  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& out, at::Tensor& in, const c10d::AllgatherOptions& opts) override {
    if (!in.is_cuda() || !in.is_contiguous() || !out.is_contiguous()) return inner_->_allgather_base(out, in, opts);
    TORCH_CHECK(out.numel() == in.numel() * getSize(), "coccl backend: all_gather size mismatch");
    ncclComm_t c = comm(in);
    check(cocclApiAllGather(in.data_ptr(), out.data_ptr(), (size_t)in.numel(), toNccl(in.scalar_type()), c,
                            at::cuda::getCurrentCUDAStream(in.get_device())), "all_gather");
    return marker(c10d::OpType::_ALLGATHER_BASE, {out});
  }

  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& out, at::Tensor& in, std::vector<int64_t>& outSplit,
                                               std::vector<int64_t>& inSplit, const c10d::AllToAllOptions& opts) override {
    if (!in.is_cuda() || !in.is_contiguous() || !out.is_contiguous() || !outSplit.empty() || !inSplit.empty() ||
        in.numel() % getSize() != 0 || in.numel() != out.numel())
      return inner_->alltoall_base(out, in, outSplit, inSplit, opts);
    ncclComm_t c = comm(in);
    check(cocclApiAllToAll(in.data_ptr(), out.data_ptr(), (size_t)in.numel() / getSize(), toNccl(in.scalar_type()), c,
                           at::cuda::getCurrentCUDAStream(in.get_device())), "all_to_all");
    return marker(c10d::OpType::ALLTOALL_BASE, {out});
  }

  // Everything else keeps its native implementation.
  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& t, const c10d::BroadcastOptions& o) override { return inner_->broadcast(t, o); }
  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor>& t, const c10d::AllreduceCoalescedOptions& o) override { return inner_->allreduce_coalesced(t, o); }
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& t, const c10d::ReduceOptions& o) override { return inner_->reduce(t, o); }
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& o, std::vector<at::Tensor>& i, const c10d::AllgatherOptions& opts) override { return inner_->allgather(o, i, opts); }
  c10::intrusive_ptr<c10d::Work> allgather_coalesced(std::vector<std::vector<at::Tensor>>& o, std::vector<at::Tensor>& i, const c10d::AllgatherOptions& opts) override { return inner_->allgather_coalesced(o, i, opts); }
  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(std::vector<at::Tensor>& o, std::vector<at::Tensor>& i, const c10d::AllgatherOptions& opts) override { return inner_->allgather_into_tensor_coalesced(o, i, opts); }
  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& o, std::vector<at::Tensor>& i, const c10d::GatherOptions& opts) override { return inner_->gather(o, i, opts); }
  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& o, std::vector<std::vector<at::Tensor>>& i, const c10d::ScatterOptions& opts) override { return inner_->scatter(o, i, opts); }
  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& o, std::vector<std::vector<at::Tensor>>& i, const c10d::ReduceScatterOptions& opts) override { return inner_->reduce_scatter(o, i, opts); }
  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& o, std::vector<at::Tensor>& i, const c10d::ReduceScatterOptions& opts) override { return inner_->reduce_scatter_tensor_coalesced(o, i, opts); }
  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor>& o, std::vector<at::Tensor>& i, const c10d::AllToAllOptions& opts) override { return inner_->alltoall(o, i, opts); }
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& t, int dst, int tag) override { return inner_->send(t, dst, tag); }
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& t, int src, int tag) override { return inner_->recv(t, src, tag); }
  c10::intrusive_ptr<c10d::Work> recvAnysource(std::vector<at::Tensor>& t, int tag) override { return inner_->recvAnysource(t, tag); }
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& o) override { return inner_->barrier(o); }
  void startCoalescing() override { inner_->startCoalescing(); }
  c10::intrusive_ptr<c10d::Work> endCoalescing() override { return inner_->endCoalescing(); }

  // Router statistics of this process: {native, compressed, deferred, lookups, fused, staged}.
  std::vector<int64_t> stats() const {
    cocclApiStats s;
    cocclApiGetStats(&s);
    return {(int64_t)s.nativeCalls, (int64_t)s.compressedCalls, (int64_t)s.deferredCalls, (int64_t)s.policyLookups,
            (int64_t)s.fusedCalls, (int64_t)s.stagedCalls};
  }

 private:
  c10::intrusive_ptr<c10d::Work> marker(c10d::OpType op, std::vector<at::Tensor> out) {
    return c10::make_intrusive<MarkerWork>(getRank(), op, std::move(out));
  }

  // The runtime's communicator is created at the first compressed-capable call: rank 0 publishes the
  // unique id through the store.
  ncclComm_t comm(const at::Tensor& t) {
    if (comm_ != nullptr) return comm_;
    c10::cuda::CUDAGuard guard(t.device());
    ncclUniqueId id;
    const std::string key = "coccl_unique_id";
    if (getRank() == 0) {
      check(cocclApiGetUniqueId(&id), "get_unique_id");
      std::vector<uint8_t> bytes(sizeof(id));
      std::memcpy(bytes.data(), &id, sizeof(id));
      store_->set(key, bytes);
    } else {
      std::vector<uint8_t> bytes = store_->get(key);
      TORCH_CHECK(bytes.size() == sizeof(id), "coccl backend: bad unique id in the store");
      std::memcpy(&id, bytes.data(), sizeof(id));
    }
    check(cocclApiCommInitRank(&comm_, getSize(), id, getRank()), "comm_init_rank");
    return comm_;
  }

  c10::intrusive_ptr<c10d::Backend> inner_;
  c10::intrusive_ptr<c10d::Store> store_;
  ncclComm_t comm_ = nullptr;
};

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  py::class_<ProcessGroupCoccl, c10d::Backend, c10::intrusive_ptr<ProcessGroupCoccl>>(m, "ProcessGroupCoccl")
      .def(py::init<c10::intrusive_ptr<c10d::Backend>, c10::intrusive_ptr<c10d::Store>, int, int>())
      .def("stats", &ProcessGroupCoccl::stats);
}

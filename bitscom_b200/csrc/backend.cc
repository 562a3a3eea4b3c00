// `lowbit` torch.distributed backend for one NVSwitch domain.
//
// ProcessGroupLowBit is a c10d::Backend.  Low-bit SUM all-reduce (bitwidth < 8) and
// low-bit reduce-scatter run as ONE fused sm_100a kernel per bucket chunk over symmetric
// memory (symm.h / fused_collectives.cu); everything else (broadcast, all-gather,
// all-to-all, send/recv, barrier, non-SUM or >= 8-bit all-reduce) is forwarded to an
// inner ProcessGroupNCCL, as in the reference
// (cpp/src/process_group_lowbit.cc:1641-1668,1779-1802).
//
// What is different from the reference's backend (cpp/src/process_group_lowbit.cc):
//   * no second raw NCCL communicator and no grouped ncclSend/ncclRecv (:543-575,
//     :776-835): peers' receive slots are written with direct NVLink stores by the kernel;
//     the IPC handles of the symmetric blocks are exchanged once through the c10d Store;
//   * no three host-synchronised phases and no progress engine (:863-966): the Work
//     holds a CUDA event, wait() orders the caller's current stream after it without
//     blocking the host, its Future completes when the result exists;
//   * residuals are keyed by (storage address, numel, dtype) of the bucket and can be
//     exported / imported for checkpointing (the reference keys by TensorImpl*, :694-725);
//   * any element count is accepted (the reference requires numel % world == 0, :702-705);
//   * timing logs and the constructor banner are off unless BITSCOM_TIMING=1.
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/chrono.h>
#include <pybind11/stl.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/ProcessGroupNCCL.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/extension.h>

#include <chrono>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <tuple>
#include <vector>

#include "symm.h"

namespace bitscom_b200 {

enum class EFMode { kNone, kLegacy, kEF21, kEF21Plus };

static EFMode parse_ef_mode(const std::string& raw, bool error_feedback) {
  std::string m;
  for (char c : raw) m.push_back((char)std::tolower((unsigned char)c));
  if (m == "auto" || m.empty()) return error_feedback ? EFMode::kLegacy : EFMode::kNone;
  if (m == "none") return EFMode::kNone;
  if (m == "legacy" || m == "ef") return EFMode::kLegacy;
  if (m == "ef21") return EFMode::kEF21;
  if (m == "ef21_plus" || m == "ef21+") return EFMode::kEF21Plus;
  TORCH_CHECK(false, "unknown error_feedback_mode '", raw, "'");
}

struct LowBitOptions {
  int bitwidth = 4;
  bool error_feedback = false;
  std::string error_feedback_mode = "auto";
  int block_size = 256;
  bool stage2_error_feedback = true;
  std::chrono::milliseconds timeout{600000};
  double kernel_timeout_ms = 30000.0;
  int64_t region_bytes = 64ll << 20;
};

static int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return 0;
    case at::kHalf: return 1;
    case at::kBFloat16: return 2;
    default: return -1;
  }
}

// The communicator as the backend and its Work objects share it: a Work may outlive the
// backend's close(), after which `comm` is null and there is no status left to read.
struct CommSlot {
  std::mutex mu;
  BcomComm* comm = nullptr;
};

// Raises if a fused kernel of this communicator gave up on one of its bounded waits.  Reads
// the host-mapped status record only: no device synchronisation.
static void raise_if_gave_up(const std::shared_ptr<CommSlot>& slot) {
  if (!slot) return;
  unsigned int st[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  {
    std::lock_guard<std::mutex> lock(slot->mu);
    if (!slot->comm) return;
    bcom_comm_status(slot->comm, st);
  }
  TORCH_CHECK(st[0] == 0, "lowbit fused collective gave up waiting: code ", st[0], ", rank ",
              st[3], " waited on peer ", st[2],
              "; the tensors of that collective are not valid");
}

// ---------------------------------------------------------------------------
// Work: a CUDA event on the communication stream
// ---------------------------------------------------------------------------
class WorkLowBit : public c10d::Work {
 public:
  WorkLowBit(int rank, c10d::OpType op, std::vector<at::Tensor> outputs,
             std::shared_ptr<CommSlot> comm, c10::DeviceIndex device)
      : c10d::Work(rank, op), outputs_(std::move(outputs)), comm_(std::move(comm)),
        device_(device) {
    future_ = c10::make_intrusive<at::ivalue::Future>(
        c10::ListType::create(c10::TensorType::get()),
        std::vector<c10::Device>{c10::Device(c10::kCUDA, device)});
  }

  // called with the communication stream current, right after the kernel was enqueued
  void mark_enqueued(const c10::cuda::CUDAStream& comm_stream) {
    done_.record(comm_stream);
    future_->markCompleted(at::IValue(outputs_));  // records its own event on comm_stream
  }

  bool isCompleted() override {
    const bool done = done_.query();
    if (done) check_status();
    return done;
  }
  bool isSuccess() const override { return true; }

  // Stream-ordered: the caller's current stream waits for the result, the host does not.  A
  // kernel that has ALREADY given up (this collective's, if it ran to its time limit before
  // the call, or an earlier one's) raises here; one that gives up later is reported by the
  // next collective, isCompleted() or synchronize().
  bool wait(std::chrono::milliseconds /*timeout*/ = kNoTimeout) override {
    done_.block(c10::cuda::getCurrentCUDAStream(device_));
    check_status();
    return true;
  }
  void synchronize() override {
    done_.synchronize();
    check_status();
  }
  bool block_current_stream() {
    done_.block(c10::cuda::getCurrentCUDAStream(device_));
    return true;
  }
  bool host_wait() {
    synchronize();
    return true;
  }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }
  std::vector<at::Tensor> result() override { return outputs_; }

 private:
  void check_status() { raise_if_gave_up(comm_); }
  std::vector<at::Tensor> outputs_;
  std::shared_ptr<CommSlot> comm_;
  c10::DeviceIndex device_;
  at::cuda::CUDAEvent done_;
  c10::intrusive_ptr<at::ivalue::Future> future_;
};

class ProcessGroupLowBit;

// Handle of the reference's three-step scheduling API
// (cpp/src/process_group_lowbit.cc:972-1085).  The fused kernel has no separate phases:
// scheduling enqueues the whole collective, launch_phase2 / launch_restore report success.
struct LowBitScheduledHandle {
  c10::intrusive_ptr<WorkLowBit> work;
  bool phase2_requested = false;
  bool restore_requested = false;
};

// ---------------------------------------------------------------------------
// the backend
// ---------------------------------------------------------------------------
class ProcessGroupLowBit : public c10d::Backend {
 public:
  ProcessGroupLowBit(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                     LowBitOptions options)
      : c10d::Backend(rank, size), store_(store), options_(std::move(options)) {
    static const int valid[] = {1, 2, 4, 8, 12, 16};
    bool ok = false;
    for (int b : valid) ok = ok || b == options_.bitwidth;
    TORCH_CHECK(ok, "bitwidth must be one of (1, 2, 4, 8, 12, 16), got ", options_.bitwidth);
    TORCH_CHECK(options_.block_size > 0, "block_size must be > 0");
    ef_mode_ = parse_ef_mode(options_.error_feedback_mode, options_.error_feedback);
    auto nccl_opts = c10d::ProcessGroupNCCL::Options::create();
    nccl_opts->timeout = options_.timeout;
    nccl_ = c10::make_intrusive<c10d::ProcessGroupNCCL>(store_, rank, size, nccl_opts);
  }

  // The destructor of the inner ProcessGroupNCCL joins its watchdog and heartbeat threads, and
  // those may need the GIL to finish (dropping the last reference of a tensor that has a
  // Python object, the stuck-GIL probe).  pybind runs this destructor with the GIL held, so
  // it is released for the teardown: torch binds its own ProcessGroupNCCL with a holder that
  // does the same.  Joining those threads with the GIL held can deadlock the process.
  ~ProcessGroupLowBit() override {
    if (Py_IsInitialized() && PyGILState_Check()) {
      pybind11::gil_scoped_release nogil;
      teardown(/*handshake_ms=*/2000);
    } else {
      teardown(/*handshake_ms=*/2000);
    }
  }

  const std::string getBackendName() const override { return "lowbit"; }

  // ---- low-bit paths ----------------------------------------------------------------
  bool stage1_ef() const { return ef_mode_ != EFMode::kNone; }
  bool stage2_ef() const {
    return options_.stage2_error_feedback && ef_mode_ == EFMode::kEF21Plus;
  }
  bool fused_ok(const at::Tensor& t) const {
    const int b = options_.bitwidth;
    return t.is_cuda() && t.is_contiguous() && dtype_code(t.scalar_type()) >= 0 &&
           (b == 1 || b == 2 || b == 4 || b == 8 || b == 12) &&
           bcom_collective_supported(dtype_code(t.scalar_type()), b, options_.block_size);
  }
  bool use_lowbit_allreduce(const at::Tensor& t, const c10d::AllreduceOptions& opts) const {
    return options_.bitwidth < 8 && opts.reduceOp == c10d::ReduceOp::SUM && getSize() > 1 &&
           fused_ok(t);
  }

  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors,
                                           const c10d::AllreduceOptions& opts) override {
    if (tensors.size() != 1 || !use_lowbit_allreduce(tensors[0], opts))
      return nccl().allreduce(tensors, opts);
    return lowbit_collective(tensors[0], tensors[0], BCOM_MODE_ALL_REDUCE,
                             c10d::OpType::ALLREDUCE);
  }

  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(
      at::Tensor& output, at::Tensor& input, const c10d::ReduceScatterOptions& opts) override {
    const bool lowbit = options_.bitwidth < 16 && opts.reduceOp == c10d::ReduceOp::SUM &&
                        getSize() > 1 && fused_ok(input) && fused_ok(output) &&
                        input.scalar_type() == output.scalar_type();
    if (!lowbit) return nccl()._reduce_scatter_base(output, input, opts);
    TORCH_CHECK(input.numel() == output.numel() * getSize(),
                "reduce_scatter: input must hold world * output elements");
    return lowbit_collective(input, output, BCOM_MODE_REDUCE_SCATTER,
                             c10d::OpType::_REDUCE_SCATTER_BASE);
  }

  c10::intrusive_ptr<c10d::Work> reduce_scatter(
      std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs,
      const c10d::ReduceScatterOptions& opts) override {
    TORCH_CHECK(outputs.size() == inputs.size(), "reduce_scatter: list sizes differ");
    const bool lowbit = outputs.size() == 1 && options_.bitwidth < 16 &&
                        opts.reduceOp == c10d::ReduceOp::SUM && getSize() > 1 &&
                        fused_ok(outputs[0]);
    if (!lowbit) return nccl().reduce_scatter(outputs, inputs, opts);
    auto& shards = inputs[0];
    TORCH_CHECK((int)shards.size() == getSize(), "reduce_scatter: need one input per rank");
    for (auto& s : shards)
      TORCH_CHECK(s.numel() == outputs[0].numel(), "reduce_scatter: shard / output size mismatch");
    std::vector<at::Tensor> flat_parts;
    for (auto& s : shards) flat_parts.push_back(s.reshape({-1}));
    at::Tensor flat = at::cat(flat_parts).contiguous();
    return lowbit_collective(flat, outputs[0], BCOM_MODE_REDUCE_SCATTER,
                             c10d::OpType::REDUCE_SCATTER);
  }

  // all-gather of quantized shards (new; the reference forwards all-gather to NCCL)
  c10::intrusive_ptr<c10d::Work> allgather_lowbit(at::Tensor& output, at::Tensor& input) {
    TORCH_CHECK(fused_ok(input) && fused_ok(output), "allgather_lowbit: unsupported tensors");
    TORCH_CHECK(output.numel() == input.numel() * getSize(),
                "allgather_lowbit: output must hold world * input elements");
    return lowbit_collective(input, output, BCOM_MODE_ALL_GATHER,
                             c10d::OpType::_ALLGATHER_BASE);
  }

  // ---- passthroughs -------------------------------------------------------------------
  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& t,
                                           const c10d::BroadcastOptions& o) override {
    return nccl().broadcast(t, o);
  }
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& t,
                                        const c10d::ReduceOptions& o) override {
    return nccl().reduce(t, o);
  }
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& out,
                                           std::vector<at::Tensor>& in,
                                           const c10d::AllgatherOptions& o) override {
    return nccl().allgather(out, in, o);
  }
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& out, at::Tensor& in,
                                                 const c10d::AllgatherOptions& o) override {
    return nccl()._allgather_base(out, in, o);
  }
  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& out, at::Tensor& in,
                                               std::vector<int64_t>& os, std::vector<int64_t>& is,
                                               const c10d::AllToAllOptions& o) override {
    return nccl().alltoall_base(out, in, os, is, o);
  }
  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor>& out,
                                          std::vector<at::Tensor>& in,
                                          const c10d::AllToAllOptions& o) override {
    return nccl().alltoall(out, in, o);
  }
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& t, int dst, int tag) override {
    return nccl().send(t, dst, tag);
  }
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& t, int src, int tag) override {
    return nccl().recv(t, src, tag);
  }
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& o) override {
    return nccl().barrier(o);
  }
  void setSequenceNumberForGroup() override {}
  uint64_t getSequenceNumberForGroup() override { return seq_; }

  // ---- scheduled-handle API ---------------------------------------------------------------
  bool progress_lowbit(bool block) {
    std::lock_guard<std::mutex> lock(mu_);
    bool all_done = true;
    for (auto it = inflight_.begin(); it != inflight_.end();) {
      if (block) (*it)->host_wait();
      if ((*it)->isCompleted()) {
        it = inflight_.erase(it);
      } else {
        all_done = false;
        ++it;
      }
    }
    return all_done;
  }

  std::shared_ptr<LowBitScheduledHandle> schedule_lowbit_allreduce(at::Tensor tensor) {
    TORCH_CHECK(getSize() > 1 && fused_ok(tensor),
                "schedule_lowbit_allreduce: tensor not eligible for the fused path");
    auto handle = std::make_shared<LowBitScheduledHandle>();
    auto work = lowbit_collective(tensor, tensor, BCOM_MODE_ALL_REDUCE, c10d::OpType::ALLREDUCE);
    handle->work = c10::static_intrusive_pointer_cast<WorkLowBit>(work);
    return handle;
  }

  // ---- residual state (checkpointing) --------------------------------------------------------
  std::vector<std::tuple<int64_t, int64_t, at::Tensor, at::Tensor>> residual_state() {
    std::lock_guard<std::mutex> lock(mu_);
    std::vector<std::tuple<int64_t, int64_t, at::Tensor, at::Tensor>> out;
    for (auto& kv : residuals_)
      out.emplace_back(std::get<0>(kv.first), std::get<1>(kv.first), kv.second.stage1,
                       kv.second.stage2);
    return out;
  }
  void clear_residuals() {
    std::lock_guard<std::mutex> lock(mu_);
    residuals_.clear();
  }
  int64_t fused_launches() const { return launches_; }
  const LowBitOptions& options() const { return options_; }

  // Orderly, collective teardown: every rank calls it after its last collective and before
  // destroy_process_group().  Releases the symmetric block with a handshake through the store
  // (wait for own kernels -> all ranks -> unmap peers -> all ranks -> free), then shuts down the
  // inner NCCL group (its communicators and helper threads): torch shuts down the
  // ProcessGroupNCCL instances it knows about, but not one that lives inside another backend.
  // Idempotent; the destructor does the same with a short handshake limit if it was not called.
  void shutdown() { teardown((int64_t)options_.timeout.count()); }

  // Releases the symmetric block only (the NCCL passthroughs keep working).
  void close_symmetric() { close_symmetric_impl((int64_t)options_.timeout.count()); }

 private:
  struct Residual {
    at::Tensor stage1, stage2;
  };
  using Key = std::tuple<int64_t, int64_t, int>;

  // All ranks reach `key` (counted through the store) or `limit_ms` passes; false on the limit.
  bool store_barrier(const std::string& key, int64_t limit_ms) {
    try {
      store_->add(key, 1);
      const auto deadline =
          std::chrono::steady_clock::now() + std::chrono::milliseconds(limit_ms);
      while (store_->add(key, 0) < getSize()) {
        if (std::chrono::steady_clock::now() >= deadline) return false;
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
      }
      return true;
    } catch (...) {  // the store is gone (its host left): treat as "peers not reachable"
      return false;
    }
  }

  void close_symmetric_impl(int64_t limit_ms) {
    std::lock_guard<std::mutex> lock(mu_);
    if (!comm_) return;
    inflight_.clear();
    const std::string prefix =
        "bitscom_b200/symm/close" + std::to_string(comm_generation_) + "/";
    c10::cuda::CUDAGuard guard(device_);
    cudaDeviceSynchronize();  // own kernels done: nothing of this rank stores into a peer
    bool everyone = store_barrier(prefix + "quiet", limit_ms);
    bcom_comm_close_peers(comm_);
    everyone = everyone && store_barrier(prefix + "unmapped", limit_ms);
    BcomComm* dead = nullptr;
    {
      std::lock_guard<std::mutex> slot_lock(slot_->mu);
      dead = slot_->comm;
      slot_->comm = nullptr;
    }
    comm_ = nullptr;
    // A peer that did not answer may still map this block: freeing it then is undefined, so
    // the block is left to the driver's process teardown instead.
    if (everyone) bcom_comm_destroy(dead);
    comm_stream_.reset();
    ++comm_generation_;
  }

  void teardown(int64_t handshake_ms) {
    close_symmetric_impl(handshake_ms);
    c10::intrusive_ptr<c10d::ProcessGroupNCCL> nccl;
    {
      std::lock_guard<std::mutex> lock(mu_);
      nccl = std::move(nccl_);
      nccl_ = nullptr;
    }
    if (nccl) {
      try {
        nccl->shutdown();
      } catch (...) {
      }
      nccl.reset();  // joins the helper threads; the caller has released the GIL
    }
  }

  c10d::ProcessGroupNCCL& nccl() const {
    TORCH_CHECK(nccl_, "lowbit backend: used after shutdown()");
    return *nccl_;
  }

  void ensure_comm(c10::DeviceIndex device) {
    if (comm_) {
      TORCH_CHECK(device == device_, "lowbit backend: one device per process group");
      return;
    }
    c10::cuda::CUDAGuard guard(device);
    device_ = device;
    TORCH_CHECK(bcom_comm_create(getRank(), getSize(), (size_t)options_.region_bytes, &comm_) == 0,
                "lowbit backend: could not allocate the symmetric block");
    {
      std::lock_guard<std::mutex> slot_lock(slot_->mu);
      slot_->comm = comm_;
    }
    std::vector<uint8_t> mine(BCOM_IPC_HANDLE_BYTES);
    TORCH_CHECK(bcom_comm_ipc_handle(comm_, mine.data()) == 0, "cudaIpcGetMemHandle failed");
    const std::string prefix = "bitscom_b200/symm/gen" + std::to_string(comm_generation_) + "/";
    store_->set(prefix + std::to_string(getRank()), mine);
    std::vector<uint8_t> all((size_t)getSize() * BCOM_IPC_HANDLE_BYTES);
    for (int r = 0; r < getSize(); ++r) {
      auto h = r == getRank() ? mine : store_->get(prefix + std::to_string(r));
      TORCH_CHECK(h.size() == BCOM_IPC_HANDLE_BYTES, "bad IPC handle from rank ", r);
      std::copy(h.begin(), h.end(), all.begin() + (size_t)r * BCOM_IPC_HANDLE_BYTES);
    }
    TORCH_CHECK(bcom_comm_open_peers(comm_, all.data()) == 0,
                "lowbit backend: cudaIpcOpenMemHandle failed (all ranks must share one node)");
    bcom_comm_set_timeout_ms(comm_, options_.kernel_timeout_ms);
    // nobody launches before everybody has mapped everybody
    const std::string ready = prefix + "ready";
    store_->add(ready, 1);
    const auto deadline = std::chrono::steady_clock::now() + options_.timeout;
    while (store_->add(ready, 0) < getSize()) {
      TORCH_CHECK(std::chrono::steady_clock::now() < deadline,
                  "lowbit backend: timed out waiting for peers to map symmetric memory");
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    comm_stream_ = std::make_unique<c10::cuda::CUDAStream>(
        c10::cuda::getStreamFromPool(/*isHighPriority=*/true, device));
  }

  Residual& residual_for(const at::Tensor& t, int64_t stage1_elems, int64_t stage2_elems) {
    const Key key{(int64_t)(uintptr_t)t.data_ptr(), t.numel(), (int)t.scalar_type()};
    auto& r = residuals_[key];
    auto opts = at::TensorOptions().dtype(at::kFloat).device(t.device());
    if (stage1_elems > 0 && (!r.stage1.defined() || r.stage1.numel() != stage1_elems))
      r.stage1 = at::zeros({stage1_elems}, opts);
    if (stage2_elems > 0 && (!r.stage2.defined() || r.stage2.numel() != stage2_elems))
      r.stage2 = at::zeros({stage2_elems}, opts);
    return r;
  }

  c10::intrusive_ptr<c10d::Work> lowbit_collective(at::Tensor& in, at::Tensor& out, int mode,
                                                   c10d::OpType op) {
    const auto device = in.device().index();
    std::lock_guard<std::mutex> lock(mu_);
    ensure_comm(device);
    raise_if_gave_up(slot_);  // an earlier kernel that gave up left partial results behind
    c10::cuda::CUDAGuard guard(device);
    const int W = getSize();
    BcomCollArgs a{};
    a.in = in.data_ptr();
    a.out = out.data_ptr();
    a.dtype = dtype_code(in.scalar_type());
    a.bits = options_.bitwidth;
    a.block = options_.block_size;
    a.mode = mode;
    a.stochastic = 0;  // the reference backend rounds to nearest (process_group_lowbit.cc:458)
    a.post_scale = 1.0f;
    a.max_ctas = 0;
    if (mode == BCOM_MODE_ALL_REDUCE) {
      a.n = in.numel();
      a.S = (a.n + W - 1) / W;
      if (stage1_ef()) {
        auto& r = residual_for(in, a.S * W, stage2_ef() ? a.S : 0);
        a.res1 = r.stage1.data_ptr<float>();
        a.res2 = stage2_ef() ? r.stage2.data_ptr<float>() : nullptr;
      }
    } else if (mode == BCOM_MODE_REDUCE_SCATTER) {
      a.S = out.numel();
      a.n = a.S * W;
    } else {
      a.S = in.numel();
      a.n = a.S * W;
    }
    if (a.n == 0) {
      auto work = c10::make_intrusive<WorkLowBit>(getRank(), op, std::vector<at::Tensor>{out},
                                                  slot_, device);
      work->mark_enqueued(c10::cuda::getCurrentCUDAStream(device));
      return work;
    }
    // order the communication stream after the producer of the tensor
    at::cuda::CUDAEvent ready;
    ready.record(c10::cuda::getCurrentCUDAStream(device));
    ready.block(*comm_stream_);
    auto work = c10::make_intrusive<WorkLowBit>(getRank(), op, std::vector<at::Tensor>{out},
                                                slot_, device);
    {
      c10::cuda::CUDAStreamGuard sguard(*comm_stream_);
      const int rc = bcom_collective(comm_, &a, (void*)comm_stream_->stream());
      TORCH_CHECK(rc == 0, "lowbit fused collective launch failed with CUDA error ", rc);
      work->mark_enqueued(*comm_stream_);
    }
    c10::cuda::CUDACachingAllocator::recordStream(in.storage().data_ptr(), *comm_stream_);
    c10::cuda::CUDACachingAllocator::recordStream(out.storage().data_ptr(), *comm_stream_);
    ++launches_;
    ++seq_;
    inflight_.push_back(work);
    if (inflight_.size() > 64) {
      for (auto it = inflight_.begin(); it != inflight_.end();)
        it = (*it)->isCompleted() ? inflight_.erase(it) : it + 1;
    }
    return work;
  }

  c10::intrusive_ptr<c10d::Store> store_;
  LowBitOptions options_;
  EFMode ef_mode_ = EFMode::kNone;
  c10::intrusive_ptr<c10d::ProcessGroupNCCL> nccl_;
  BcomComm* comm_ = nullptr;
  std::shared_ptr<CommSlot> slot_ = std::make_shared<CommSlot>();
  int comm_generation_ = 0;  // symmetric blocks created so far (store keys are per generation)
  c10::DeviceIndex device_ = -1;
  std::unique_ptr<c10::cuda::CUDAStream> comm_stream_;
  std::map<Key, Residual> residuals_;
  std::vector<c10::intrusive_ptr<WorkLowBit>> inflight_;
  std::mutex mu_;
  int64_t launches_ = 0;
  uint64_t seq_ = 0;
};

static c10::intrusive_ptr<c10d::Backend> create_backend(
    const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
    const std::chrono::milliseconds& timeout, int bitwidth, bool error_feedback,
    const std::string& error_feedback_mode, int block_size, bool stage2_error_feedback) {
  LowBitOptions o;
  o.timeout = timeout;
  o.bitwidth = bitwidth;
  o.error_feedback = error_feedback;
  o.error_feedback_mode = error_feedback_mode;
  o.block_size = block_size;
  o.stage2_error_feedback = stage2_error_feedback;
  return c10::make_intrusive<ProcessGroupLowBit>(store, rank, size, o);
}

}  // namespace bitscom_b200

namespace py = pybind11;
using namespace bitscom_b200;

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "bitscom_b200 lowbit torch.distributed backend";

  py::class_<LowBitOptions>(m, "LowBitOptions")
      .def(py::init<>())
      .def_readwrite("bitwidth", &LowBitOptions::bitwidth)
      .def_readwrite("error_feedback", &LowBitOptions::error_feedback)
      .def_readwrite("error_feedback_mode", &LowBitOptions::error_feedback_mode)
      .def_readwrite("block_size", &LowBitOptions::block_size)
      .def_readwrite("stage2_error_feedback", &LowBitOptions::stage2_error_feedback)
      .def_readwrite("timeout", &LowBitOptions::timeout)
      .def_readwrite("kernel_timeout_ms", &LowBitOptions::kernel_timeout_ms)
      .def_readwrite("region_bytes", &LowBitOptions::region_bytes);

  py::class_<LowBitScheduledHandle, std::shared_ptr<LowBitScheduledHandle>>(
      m, "LowBitScheduledHandle")
      .def("launch_phase2",
           [](LowBitScheduledHandle& h) { h.phase2_requested = true; return true; })
      .def("launch_restore",
           [](LowBitScheduledHandle& h) { h.restore_requested = true; return true; })
      .def("is_completed", [](LowBitScheduledHandle& h) { return h.work->isCompleted(); })
      .def("wait", [](LowBitScheduledHandle& h) { return h.work->host_wait(); },
           py::call_guard<py::gil_scoped_release>())
      .def("block_current_stream",
           [](LowBitScheduledHandle& h) { return h.work->block_current_stream(); });

  py::class_<ProcessGroupLowBit, c10d::Backend, c10::intrusive_ptr<ProcessGroupLowBit>>(
      m, "ProcessGroupLowBit")
      .def(py::init([](const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                       const LowBitOptions& options) {
             return c10::make_intrusive<ProcessGroupLowBit>(store, rank, size, options);
           }),
           py::arg("store"), py::arg("rank"), py::arg("size"),
           py::arg("options") = LowBitOptions())
      .def("progress_lowbit", &ProcessGroupLowBit::progress_lowbit, py::arg("block") = false,
           py::call_guard<py::gil_scoped_release>())
      .def("schedule_lowbit_allreduce", &ProcessGroupLowBit::schedule_lowbit_allreduce)
      .def("launch_scheduled_lowbit_phase2",
           [](ProcessGroupLowBit&, std::shared_ptr<LowBitScheduledHandle> h) {
             h->phase2_requested = true;
             return true;
           })
      .def("launch_scheduled_lowbit_restore",
           [](ProcessGroupLowBit&, std::shared_ptr<LowBitScheduledHandle> h) {
             h->restore_requested = true;
             return true;
           })
      .def("scheduled_lowbit_is_completed",
           [](ProcessGroupLowBit&, std::shared_ptr<LowBitScheduledHandle> h) {
             return h->work->isCompleted();
           })
      .def("scheduled_lowbit_wait",
           [](ProcessGroupLowBit&, std::shared_ptr<LowBitScheduledHandle> h) {
             return h->work->host_wait();
           },
           py::call_guard<py::gil_scoped_release>())
      .def("scheduled_lowbit_block_current_stream",
           [](ProcessGroupLowBit&, std::shared_ptr<LowBitScheduledHandle> h) {
             return h->work->block_current_stream();
           })
      .def("allgather_lowbit",
           [](ProcessGroupLowBit& pg, at::Tensor out, at::Tensor in) {
             return pg.allgather_lowbit(out, in);
           })
      .def("residual_state", &ProcessGroupLowBit::residual_state)
      .def("clear_residuals", &ProcessGroupLowBit::clear_residuals)
      .def("fused_launches", &ProcessGroupLowBit::fused_launches)
      .def("shutdown", &ProcessGroupLowBit::shutdown,
           py::call_guard<py::gil_scoped_release>())
      .def("close_symmetric", &ProcessGroupLowBit::close_symmetric,
           py::call_guard<py::gil_scoped_release>());

  m.def("create_backend", &create_backend, py::arg("store"), py::arg("rank"), py::arg("size"),
        py::arg("timeout") = std::chrono::milliseconds(600000), py::arg("bitwidth") = 4,
        py::arg("error_feedback") = false, py::arg("error_feedback_mode") = "auto",
        py::arg("block_size") = 256, py::arg("stage2_error_feedback") = true);
}

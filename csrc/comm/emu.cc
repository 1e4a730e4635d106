#include "emu.h"

#include <chrono>
#include <cstring>
#include <map>

#include "../core/log.h"

namespace amem {

static std::mutex g_mu;
static std::map<uint64_t, std::weak_ptr<EmuGroup>> g_groups;

std::shared_ptr<EmuGroup> EmuGroup::get(uint64_t comm_id, int nranks) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_groups.find(comm_id);
  if (it != g_groups.end()) {
    if (auto sp = it->second.lock()) return sp;
  }
  std::shared_ptr<EmuGroup> sp(new EmuGroup(nranks));
  g_groups[comm_id] = sp;
  return sp;
}

void EmuGroup::drop(uint64_t comm_id) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_groups.find(comm_id);
  if (it != g_groups.end() && it->second.expired()) g_groups.erase(it);
}

EmuGroup::EmuGroup(int nranks) : nranks_(nranks) {
  ready_.resize(nranks, nullptr);
  for (auto& e : ready_) cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
  cudaEventCreateWithFlags(&done_, cudaEventDisableTiming);
}

EmuGroup::~EmuGroup() {
  for (auto& e : ready_)
    if (e) cudaEventDestroy(e);
  if (done_) cudaEventDestroy(done_);
  if (dev_args_) cudaFree(dev_args_);
}

Status EmuGroup::rendezvous(int rank, int tag, const void* args, size_t arg_bytes, cudaStream_t stream, const LaunchFn& fn) {
  std::unique_lock<std::mutex> lk(mu_);
  if (arrived_ == 0) {
    tag_ = tag;
    arg_bytes_ = arg_bytes;
    host_args_.assign((size_t)nranks_ * arg_bytes, 0);
    result_ = kSuccess;
  } else if (tag != tag_ || arg_bytes != arg_bytes_) {
    result_ = fail(kInvalidUsage, "emulated ranks called different operations (tag %d vs %d)", tag, tag_);
  }
  if (arg_bytes_ == arg_bytes) memcpy(host_args_.data() + (size_t)rank * arg_bytes, args, arg_bytes);
  cudaError_t e = cudaEventRecord(ready_[rank], stream);
  if (e != cudaSuccess) result_ = fail(kCudaError, "cudaEventRecord: %s", cudaGetErrorString(e));
  uint64_t my_gen = generation_;
  if (++arrived_ == nranks_) {
    Status st = result_;
    if (st == kSuccess) {
      for (int r = 0; r < nranks_ && st == kSuccess; ++r) {
        if (r == rank) continue;
        if (cudaStreamWaitEvent(stream, ready_[r], 0) != cudaSuccess) st = fail(kCudaError, "cudaStreamWaitEvent failed");
      }
    }
    if (st == kSuccess && host_args_.size() > dev_cap_) {
      if (dev_args_) cudaFree(dev_args_);
      dev_cap_ = host_args_.size() * 2;
      if (cudaMalloc(&dev_args_, dev_cap_) != cudaSuccess) {
        dev_args_ = nullptr;
        dev_cap_ = 0;
        st = fail(kCudaError, "cudaMalloc of the emulation argument buffer failed");
      }
    }
    if (st == kSuccess) {
      // pageable source: the runtime stages the bytes before returning, host_args_ is reusable
      if (cudaMemcpyAsync(dev_args_, host_args_.data(), host_args_.size(), cudaMemcpyHostToDevice, stream) != cudaSuccess)
        st = fail(kCudaError, "argument upload failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    if (st == kSuccess) st = fn(host_args_.data(), dev_args_, stream);
    if (st == kSuccess && cudaEventRecord(done_, stream) != cudaSuccess) st = fail(kCudaError, "cudaEventRecord(done) failed");
    result_ = st;
    arrived_ = 0;
    ++generation_;
    cv_.notify_all();
    return st;
  }
  bool ok = cv_.wait_for(lk, std::chrono::milliseconds(env_long("AMEM_OP_TIMEOUT_MS", 30000)), [&] { return generation_ != my_gen; });
  if (!ok) {
    // give the slot back so a later call does not see a half-filled board
    --arrived_;
    return fail(kSystemError, "emulated rank %d waited too long for the other ranks to call the same operation", rank);
  }
  Status st = result_;
  if (st == kSuccess && cudaStreamWaitEvent(stream, done_, 0) != cudaSuccess) st = fail(kCudaError, "cudaStreamWaitEvent(done) failed");
  return st;
}

}  // namespace amem

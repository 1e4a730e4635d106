// Emulated multi-rank communicator on ONE GPU.
//
// When every rank of a communicator lives in the same process and on the same device (the
// single-GPU test-suite runs ranks as threads), the ranks' kernels must not be separate
// launches: they spin on each other's flags and nothing guarantees that two launches on one
// device run at the same time.  The ranks therefore meet here on the host; the last one to
// arrive launches ONE cooperative grid that carries all ranks (blockIdx.y = rank) and the
// other ranks' streams are made to wait for it through events.
// Reference parity: none -- the reference is tested only on eight real GPUs under mpirun (run.sh:26-30).
#pragma once
#include <cuda_runtime.h>

#include <condition_variable>
#include <functional>
#include <memory>
#include <mutex>
#include <vector>

#include "../core/status.h"

namespace amem {

class EmuGroup {
 public:
  // fn(host copy of the nranks argument blobs, the same blobs in device memory, stream)
  // launches the grid.
  using LaunchFn = std::function<Status(const void* host_args, const void* dev_args, cudaStream_t stream)>;

  static std::shared_ptr<EmuGroup> get(uint64_t comm_id, int nranks);
  static void drop(uint64_t comm_id);
  ~EmuGroup();

  // Called by each rank's thread with its own argument blob; returns once the grid has been
  // enqueued and `stream` is ordered after it.  `tag` must be equal on all ranks (it guards
  // against ranks calling different operations).
  Status rendezvous(int rank, int tag, const void* args, size_t arg_bytes, cudaStream_t stream, const LaunchFn& fn);

 private:
  EmuGroup(int nranks);
  int nranks_;
  std::mutex mu_;
  std::condition_variable cv_;
  int arrived_ = 0;
  uint64_t generation_ = 0;
  int tag_ = 0;
  Status result_ = kSuccess;
  std::vector<char> host_args_;
  size_t arg_bytes_ = 0;
  void* dev_args_ = nullptr;
  size_t dev_cap_ = 0;
  std::vector<cudaEvent_t> ready_;
  cudaEvent_t done_ = nullptr;
};

}  // namespace amem

// Device memory for the library's own use that is NOT part of a symmetric segment: work areas of
// the fused kernels, the split-K workspace of the plain GEMM, user memory from ncclMemAlloc.
// It is made with the same VMM calls as everything else and entered in the registry, so that
// ncclMemStats accounts for it and ncclPause hands it back (the reference tracks every cuMem
// allocation NCCL makes for the same reason, nccl_patch/nccl_2.27.5-1.diff:258-290).
#pragma once
#include <cstddef>
#include <cstdint>

#include "backend.h"
#include "registry.h"

namespace amem {

// `owner`: communicator id, or 0 for process-level memory (paused by ncclPause(NULL) only).
// `category`: kStateful (contents survive a pause), kScratch (contents are dead between calls),
// kResident (stays mapped through a pause).  Sizes are rounded up to the allocation granularity.
Status tracked_alloc(VmmBackend* be, uint64_t owner, int dev, size_t bytes, int category, int tag, uint64_t* va, size_t* rounded);
// Unmaps, releases, frees the address range and the host shadow, forgets the record.
Status tracked_free(VmmBackend* be, uint64_t va);

}  // namespace amem

// Type / operator dispatch shared by the CUDA launcher and the host executor.
// AMEM_DISPATCH_REDUCE(dtype, out_dtype, redop, F) expands F(TI, TO, OP) for the supported
// combination or evaluates to `return kInvalidArgument`-style handling through `F_BAD`.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "coll_args.h"

#define AMEM_DISPATCH_OP(TI, TO, redop, F)              \
  switch (redop) {                                      \
    case ::amem::kSum: case ::amem::kAvg: F(TI, TO, ::amem::kSum); break; \
    case ::amem::kProd: F(TI, TO, ::amem::kProd); break; \
    case ::amem::kMax: F(TI, TO, ::amem::kMax); break;  \
    case ::amem::kMin: F(TI, TO, ::amem::kMin); break;  \
    default: ok = false;                                \
  }

// Sets `bool ok` (must be declared by the caller) to false for unsupported combinations.
#define AMEM_DISPATCH_REDUCE(dtype, out_dtype, redop, F)                                   \
  do {                                                                                     \
    if ((dtype) == (out_dtype)) {                                                          \
      switch (dtype) {                                                                     \
        case ::amem::kI8: AMEM_DISPATCH_OP(signed char, signed char, redop, F) break;      \
        case ::amem::kU8: AMEM_DISPATCH_OP(unsigned char, unsigned char, redop, F) break;  \
        case ::amem::kI32: AMEM_DISPATCH_OP(int, int, redop, F) break;                     \
        case ::amem::kU32: AMEM_DISPATCH_OP(unsigned, unsigned, redop, F) break;           \
        case ::amem::kI64: AMEM_DISPATCH_OP(long long, long long, redop, F) break;         \
        case ::amem::kU64: AMEM_DISPATCH_OP(unsigned long long, unsigned long long, redop, F) break; \
        case ::amem::kF16: AMEM_DISPATCH_OP(__half, __half, redop, F) break;               \
        case ::amem::kF32: AMEM_DISPATCH_OP(float, float, redop, F) break;                 \
        case ::amem::kF64: AMEM_DISPATCH_OP(double, double, redop, F) break;               \
        case ::amem::kBF16: AMEM_DISPATCH_OP(__nv_bfloat16, __nv_bfloat16, redop, F) break; \
        default: ok = false;                                                               \
      }                                                                                    \
    } else if ((redop) == ::amem::kSum || (redop) == ::amem::kAvg) {                       \
      /* fused cast: sum only */                                                           \
      if ((dtype) == ::amem::kF32 && (out_dtype) == ::amem::kBF16) { F(float, __nv_bfloat16, ::amem::kSum); } \
      else if ((dtype) == ::amem::kBF16 && (out_dtype) == ::amem::kF32) { F(__nv_bfloat16, float, ::amem::kSum); } \
      else if ((dtype) == ::amem::kF32 && (out_dtype) == ::amem::kF16) { F(float, __half, ::amem::kSum); } \
      else if ((dtype) == ::amem::kF16 && (out_dtype) == ::amem::kF32) { F(__half, float, ::amem::kSum); } \
      else ok = false;                                                                     \
    } else {                                                                               \
      ok = false;                                                                          \
    }                                                                                      \
  } while (0)

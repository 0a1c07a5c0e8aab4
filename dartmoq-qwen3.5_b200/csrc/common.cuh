// Shared helpers for the libdmoq kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dmoq.h"

#define DMOQ_CHECK_ARG(cond) \
  do {                       \
    if (!(cond)) return DMOQ_EINVAL; \
  } while (0)

static inline int dmoq_launch_status() {
  return cudaPeekAtLastError() == cudaSuccess ? DMOQ_OK : DMOQ_ELAUNCH;
}

static inline int dmoq_ceil_div(int a, int b) { return (a + b - 1) / b; }

// Number of SMs of the current device, cached per process (read-only query).
int dmoq_sm_count();

// One-time kernel set-up (cudaFuncSetAttribute) is per DEVICE: a launcher keeps one flag per device ordinal.
struct DmoqOncePerDevice {
  bool done[64] = {};
  bool* slot() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return &done[dev];
  }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, bool valid) {
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }

// per-tile record written by the routing kernels
struct DmoqTile {
  int32_t expert;
  int32_t row0;
  int32_t rows;
  int32_t rank;   // member rank of the expert inside its pool
};

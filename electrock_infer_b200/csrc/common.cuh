// Shared helpers of libb200moe: error reporting, launch checks and small device utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b200moe.h"

namespace b200moe {

// Records the message returned by b200moe_last_error() on this thread and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

// Counts a kernel launch of this library (read by b200moe_kernel_launch_count()).
void note_launch();

// Called directly after every kernel launch: counts it and reports a failed launch
// (cudaGetLastError) as B200MOE_ERR_CUDA.
inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  note_launch();
  return B200MOE_OK;
}

// Number of SMs of the current device (cached per device).
int sm_count();

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Programmatic dependent launch.  Every kernel of the layer is launched with the
// programmatic-stream-serialization attribute: it may begin (block scheduling, prologue) while
// its predecessor in the stream is still draining, and must call pdl_wait() before it touches
// global memory the predecessor wrote.  pdl_launch_dependents() lets the successor do the same.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// 16-byte global load that bypasses L1 allocation: for data that is read exactly once.
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// 16-byte global store with streaming (evict-first) policy.
__device__ __forceinline__ void st_stream_16(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

}  // namespace b200moe

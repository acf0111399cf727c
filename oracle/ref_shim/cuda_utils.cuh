// Test-infrastructure shim.  The reference's MoE kernels include "cuda_utils.cuh", whose shipped
// version pulls in another vendor's runtime headers.  This file is found first on the include
// path when the unmodified reference sources are compiled with nvcc for the oracle build, and
// supplies the same names on top of the CUDA runtime: the warp width of NVIDIA GPUs, the ATen
// dispatch helpers the kernels use, and CUDA spellings of the three runtime symbols they call.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <torch/all.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <stdexcept>
#include <string>

#define WARP_SIZE 32

#define DISPATCH_FLOATING_TYPES(TYPE, NAME, ...)                                   \
  AT_DISPATCH_SWITCH(TYPE, NAME,                                                   \
                     AT_DISPATCH_CASE(at::ScalarType::Float, __VA_ARGS__)          \
                     AT_DISPATCH_CASE(at::ScalarType::Half, __VA_ARGS__)           \
                     AT_DISPATCH_CASE(at::ScalarType::BFloat16, __VA_ARGS__))

#define DISPATCH_INTEGRAL_TYPES(TYPE, NAME, ...)                                   \
  AT_DISPATCH_SWITCH(TYPE, NAME,                                                   \
                     AT_DISPATCH_CASE(at::ScalarType::Byte, __VA_ARGS__)           \
                     AT_DISPATCH_CASE(at::ScalarType::Char, __VA_ARGS__)           \
                     AT_DISPATCH_CASE(at::ScalarType::Short, __VA_ARGS__)          \
                     AT_DISPATCH_CASE(at::ScalarType::Int, __VA_ARGS__)            \
                     AT_DISPATCH_CASE(at::ScalarType::Long, __VA_ARGS__))

#define DevFuncAttribute_SET_MaxDynamicSharedMemorySize(FUNC, VAL) \
  cudaFuncSetAttribute(FUNC, cudaFuncAttributeMaxDynamicSharedMemorySize, VAL)

#define hipDeviceGetAttribute cudaDeviceGetAttribute
#define hipDeviceAttributeMaxSharedMemoryPerBlock cudaDevAttrMaxSharedMemoryPerBlock

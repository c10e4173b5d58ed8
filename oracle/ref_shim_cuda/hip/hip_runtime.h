/*
 * <hip/hip_runtime.h> for a CUDA box.  TEST INFRASTRUCTURE ONLY.
 *
 * HipGPT's src/transformer_layer.cpp and src/gpt_model.cpp are host code: they allocate, copy and
 * call launch_* functions, and use nine names of the HIP runtime.  Mapping those names onto the
 * CUDA runtime lets the two files compile, unmodified and where they lie, with g++, and run on a
 * B200 against this repository's library in place of the reference's own kernels
 * (oracle/ref_model_driver.cpp, built by oracle/Makefile into oracle/_ref/ref_model_run).
 */
#pragma once
#include <cuda_runtime.h>

typedef cudaError_t hipError_t;
#define hipSuccess cudaSuccess
#define hipGetErrorString cudaGetErrorString
#define hipMalloc cudaMalloc
#define hipFree cudaFree
#define hipMemset cudaMemset
#define hipMemcpy cudaMemcpy
#define hipMemcpyKind cudaMemcpyKind
#define hipMemcpyHostToDevice cudaMemcpyHostToDevice
#define hipMemcpyDeviceToHost cudaMemcpyDeviceToHost
#define hipMemcpyDeviceToDevice cudaMemcpyDeviceToDevice
#define hipDeviceSynchronize cudaDeviceSynchronize

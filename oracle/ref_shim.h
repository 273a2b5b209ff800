/*
 * TEST INFRASTRUCTURE ONLY — never linked into, imported by, or called from the product library.
 *
 * Host shim that lets the reference's CUDA-C kernel sources (cuda/src/ptx/<op>.cu and
 * cuda/src/ptx/headers/<family>.cuh of the reference project) compile unchanged as plain
 * C++ with g++.  The sources are compiled from where they lie in the reference checkout;
 * nothing is copied.  It is force-included (-include) in front of each reference file.
 *
 * What it supplies:
 *   - `__global__` as an empty macro, so every `extern "C" __global__ void f(...)` becomes a
 *     plain C function with the same symbol name and parameter list.
 *   - thread-local `blockIdx / threadIdx / blockDim / gridDim`, set by the launcher in
 *     ref_driver.cpp before it calls the kernel body.  All reference kernels are grid-stride
 *     loops, so launching them with blockDim = 1 and gridDim = #host-threads covers every
 *     element exactly once (ref_driver.cpp:ref_launch).
 *   - `min` / `max` / math names that CUDA provides implicitly.
 *   - `hsqrt`, which cuda_fp16.h only declares for device code (used by one f16 line in sqrt.cu).
 */
#pragma once
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <algorithm>

#define __global__
#ifndef __device__
#define __device__
#endif
#ifndef __host__
#define __host__
#endif

struct ref_dim3 {
    unsigned int x, y, z;
};
extern thread_local ref_dim3 blockIdx, threadIdx, blockDim, gridDim;

using std::max;
using std::min;

#include <cuda_fp16.h>

static inline __half hsqrt(const __half h) { return __float2half(sqrtf(__half2float(h))); }

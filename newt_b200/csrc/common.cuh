// Shared host/device helpers of the newt_b200 kernel library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#ifdef __CUDACC_RTC__
// Compiled at run time (NVRTC has no host headers): the fixed-width names and the dtype codes
// of include/newt_b200.h, spelled out.
typedef unsigned char uint8_t;
typedef unsigned short uint16_t;
typedef int int32_t;
typedef unsigned int uint32_t;
typedef long long int64_t;
typedef unsigned long long uint64_t;
typedef unsigned long long uintptr_t;
enum { NB200_F32 = 0, NB200_F16 = 1, NB200_BF16 = 2 };
#else
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/newt_b200.h"
#endif

namespace nb200 {

#ifndef __CUDACC_RTC__
// ---- host side -------------------------------------------------------------

// Records a printf-style message for nb200_last_error() on this thread and
// returns `code`, so call sites read `return fail(NB200_E_INVALID, "...")`.
int fail(int code, const char* fmt, ...);
int cuda_check(cudaError_t e, const char* what);

struct DeviceInfo {
  int device;
  int sm_count;
  int max_smem_optin;
};
// Properties of the current device (cached per device ordinal).
const DeviceInfo& device_info();

// Integer knobs set through nb200_set_tuning(); returns `dflt` when unset (0).
int tuning(const char* key, int dflt);

// How long one device-side wait may spin before the kernel gives up, in nanoseconds: the
// "wait_limit_us" knob of nb200_set_tuning(), 2 s when unset.
unsigned long long wait_limit_ns();

// Per-device status words written by kernels whose bounded waits expire.
// [0] = first error code (0 = none), [1] = detail (role / barrier / tile).
unsigned int* device_status_ptr();

// Opts `kernel` in for `smem_bytes` of dynamic shared memory, once per device and size (the
// attribute call costs microseconds; a launch-bound GEMM should not pay it every time).
int prepare_kernel(const void* kernel, int smem_bytes);

// How many clusters of the launch described by `config` fit on the device at once
// (cudaOccupancyMaxActiveClusters, remembered per device, kernel and shared-memory size).
int cluster_capacity(const void* kernel, const cudaLaunchConfig_t* config, int* clusters);

static inline int64_t cdiv64(int64_t a, int64_t b) { return (a + b - 1) / b; }
#endif  // !__CUDACC_RTC__

// ---- device side -----------------------------------------------------------

// Error codes stored in the status word.
enum : unsigned int {
  ST_OK = 0,
  ST_WAIT_TMA_FULL = 1,   // MMA warp waited for a TMA stage that never landed
  ST_WAIT_SMEM_EMPTY = 2, // TMA warp waited for a stage the MMA never released
  ST_WAIT_ACC_FULL = 3,   // epilogue waited for an accumulator never committed
  ST_WAIT_ACC_EMPTY = 4,  // MMA warp waited for an accumulator never drained
  ST_TMEM_ALLOC = 5,      // tcgen05.alloc did not succeed within the retry cap
  ST_WAIT_OTHER = 6
};

}  // namespace nb200

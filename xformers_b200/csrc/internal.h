// Host-side helpers shared by the translation units of libxfb200.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/xfb200.h"

namespace xfb {

// Per-thread message for xfb200_last_error().
char* error_buffer();
constexpr size_t kErrorBufferSize = 512;

inline int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), kErrorBufferSize, fmt, ap);
  va_end(ap);
  return code;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(XFB200_E_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return XFB200_OK;
}

inline int cuda_fail(const char* what, cudaError_t e) {
  (void)cudaGetLastError();  // do not leave the error behind for the next launch check
  return set_error(XFB200_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

constexpr int kMaxDevices = 64;
// Index of the current device, -1 if it cannot be told or is out of range.
int current_device();
// Number of SMs of the current device (cached per device).
int sm_count();

// Per-device int32 words inside the library image (device address of word 0 on the
// current device; nullptr on failure).  Layout:
//   [kWordPrefillStatus]      first code a tcgen05 prefill kernel gave up with (0 = none); kept until read
//   [kWordPrefillStatus + 1]  epoch of the launch that gave up: its remaining CTAs leave at once
//   [kWordPrefillCounters ..) work counters of the persistent prefill kernel, two per slot
//                             (next item, CTAs done); back to zero when a launch ends
//   [kWordDecodeStatus]       first code a decode kernel gave up with; [+1] unused
constexpr int kWordPrefillStatus = 0;
constexpr int kWordPrefillCounters = 2;
constexpr int kPrefillCounterSlots = 31;
constexpr int kWordDecodeStatus = kWordPrefillCounters + 2 * kPrefillCounterSlots;
constexpr int kDeviceWords = kWordDecodeStatus + 2;
int32_t* device_words();
// A non-zero number that differs from launch to launch.
uint32_t next_launch_epoch();
// True the first time it is called with this flag array while a given device is current
// (function attributes such as the dynamic shared-memory limit are per device).
bool first_use_on_device(bool (&seen)[kMaxDevices]);

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does
// not link against libcuda; nullptr if the driver does not provide it.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// Entry points implemented in other translation units.
int prefill_sm100_supported(const xfb200_prefill_params* p);
int prefill_sm100_launch(const xfb200_prefill_params* p, cudaStream_t stream);
int prefill_generic_launch(const xfb200_prefill_params* p, cudaStream_t stream);

}  // namespace xfb

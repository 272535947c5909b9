// Error reporting, device queries and the device status words shared by all entry points.
#include <atomic>

#include "internal.h"

namespace xfb {

char* error_buffer() {
  static thread_local char buf[kErrorBufferSize] = {0};
  return buf;
}

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

int sm_count() {
  static int cached[kMaxDevices] = {0};
  const int dev = current_device();
  if (dev < 0) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// The status words of the bounded waits and the work counters of the persistent
// prefill kernel live in the library image (zero when a device loads it), so no
// launch path allocates or clears anything.  In host code the array's name is
// a host-side stand-in: the device address is looked up once per device, with
// that device current.
static __device__ __align__(256) int32_t g_device_words[kDeviceWords];

int32_t* device_words() {
  static int32_t* per_device[kMaxDevices] = {nullptr};
  const int dev = current_device();
  if (dev < 0) return nullptr;
  if (per_device[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_words) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    per_device[dev] = static_cast<int32_t*>(p);
  }
  return per_device[dev];
}

uint32_t next_launch_epoch() {
  static std::atomic<uint32_t> epoch{0};
  uint32_t e = ++epoch;
  if (e == 0) e = ++epoch;  // 0 means "no launch gave up"
  return e;
}

bool first_use_on_device(bool (&seen)[kMaxDevices]) {
  const int dev = current_device();
  if (dev < 0) return true;  // unknown device: configure every time
  if (seen[dev]) return false;
  seen[dev] = true;
  return true;
}

// Reads the sticky word `first` of the current device, then clears `count`
// words from there on the same stream.
static int read_and_clear(void* stream, int first, int count, int32_t* status_out, const char* what) {
  if (status_out == nullptr) return set_error(XFB200_E_INVALID, "%s: status_out is null", what);
  int32_t* w = device_words();
  if (w == nullptr) return set_error(XFB200_E_CUDA, "%s: cannot resolve the device status words", what);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(status_out, w + first, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(w + first, 0, sizeof(int32_t) * count, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail(what, e);
  if (*status_out != 0)
    return set_error(XFB200_E_DEVICE, "%s: a kernel gave up a bounded wait (code %d); its output is not valid", what, int(*status_out));
  return XFB200_OK;
}

}  // namespace xfb

extern "C" int xfb200_abi_version(void) { return XFB200_ABI_VERSION; }
extern "C" const char* xfb200_last_error(void) { return xfb::error_buffer(); }

extern "C" int xfb200_prefill_device_status(void* stream, int32_t* status_out) {
  using namespace xfb;
  // the work counters of the persistent kernel are cleared along with the status: a launch
  // that gave up may have left them half-way
  return read_and_clear(stream, kWordPrefillStatus, kWordDecodeStatus - kWordPrefillStatus, status_out, "prefill_device_status");
}

extern "C" int xfb200_decode_device_status(void* stream, int32_t* status_out) {
  using namespace xfb;
  return read_and_clear(stream, kWordDecodeStatus, 2, status_out, "decode_device_status");
}

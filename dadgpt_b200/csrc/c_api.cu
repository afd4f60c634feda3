// Library-wide pieces of the C ABI: error text, version, the device-side status word.
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace dadattn {

namespace {
thread_local char g_error[512] = "";
constexpr int kMaxDevices = 64;
int* g_status[kMaxDevices] = {};
std::mutex g_status_mutex;
}  // namespace

char* error_buffer() { return g_error; }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return code;
}

// One 4-byte word per device, allocated the first time a kernel that can report a condition is
// launched on that device (the only allocation the library makes; it lives until exit).
int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fail(DADATTN_E_CUDA, "no current CUDA device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess || cudaMemset(p, 0, sizeof(int)) != cudaSuccess) {
      fail(DADATTN_E_CUDA, "cannot allocate the device status word: %s",
           cudaGetErrorString(cudaGetLastError()));
      return nullptr;
    }
    g_status[dev] = p;
  }
  return g_status[dev];
}

}  // namespace dadattn

using namespace dadattn;

extern "C" const char* dadattn_last_error(void) { return error_buffer(); }

extern "C" const char* dadattn_version(void) { return "dadattn 0.1 sm_100a"; }

extern "C" int dadattn_device_status(dadattn_stream_t stream) {
  int* word = device_status_word();
  if (!word) return DADATTN_E_CUDA;
  int host = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DAD_CUDA(cudaMemcpyAsync(&host, word, sizeof(int), cudaMemcpyDeviceToHost, st));
  DAD_CUDA(cudaMemsetAsync(word, 0, sizeof(int), st));
  DAD_CUDA(cudaStreamSynchronize(st));
  if (host == DADATTN_E_TIMEOUT) fail(host, "a bounded device-side wait ran out");
  else if (host == DADATTN_E_ARG) fail(host, "a kernel skipped work: sequence length outside [0, max_len)");
  else if (host != 0) fail(host, "device status %d", host);
  return host;
}


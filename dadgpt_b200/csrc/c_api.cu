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

// Two 4-byte words per device (status, and a detail for it: the source line of a wait that ran
// out), allocated the first time a kernel that can report a condition is launched on that
// device; they live until exit.
int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fail(DADATTN_E_CUDA, "no current CUDA device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 2 * sizeof(int)) != cudaSuccess || cudaMemset(p, 0, 2 * sizeof(int)) != cudaSuccess) {
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
  int host[2] = {0, 0};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DAD_CUDA(cudaMemcpyAsync(host, word, 2 * sizeof(int), cudaMemcpyDeviceToHost, st));
  DAD_CUDA(cudaMemsetAsync(word, 0, 2 * sizeof(int), st));
  DAD_CUDA(cudaStreamSynchronize(st));
  if (host[0] == DADATTN_E_TIMEOUT)
    fail(host[0], "a bounded device-side wait ran out (wait at source line %d of its kernel)", host[1]);
  else if (host[0] == DADATTN_E_ARG)
    fail(host[0], "a kernel skipped work: sequence length outside [0, max_len)");
  else if (host[0] != 0)
    fail(host[0], "device status %d", host[0]);
  return host[0];
}

// Error string, stream table and device selection.
#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <utility>

#include "common.h"

namespace sptir {

namespace {
thread_local std::string tls_error;
constexpr int kMaxDevices = 64;
std::atomic<void*> g_streams[kMaxDevices];
}  // namespace

int fail(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  tls_error = buf;
  return -1;
}

int use_device(int device_id) {
  int cur = -1;
  SPTIR_CUDA_OK(cudaGetDevice(&cur));
  if (cur != device_id) SPTIR_CUDA_OK(cudaSetDevice(device_id));
  return 0;
}

cudaStream_t stream_for(int device_id) {
  if (device_id < 0 || device_id >= kMaxDevices) return nullptr;
  return static_cast<cudaStream_t>(g_streams[device_id].load(std::memory_order_acquire));
}

namespace {
struct Scratch {
  void* ptr = nullptr;
  size_t bytes = 0;
};
std::mutex g_ws_mutex;
std::map<std::pair<int, cudaStream_t>, Scratch> g_ws;
}  // namespace

void* workspace(int device_id, cudaStream_t stream, size_t bytes) {
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  Scratch& s = g_ws[{device_id, stream}];
  if (s.bytes >= bytes && s.ptr != nullptr) return s.ptr;
  if (s.ptr != nullptr) {
    cudaFree(s.ptr);  // synchronises: nothing in flight can still use the old buffer
    s.ptr = nullptr;
    s.bytes = 0;
  }
  const size_t want = (bytes + (size_t{1} << 20) - 1) & ~((size_t{1} << 20) - 1);
  void* p = nullptr;
  const cudaError_t err = cudaMalloc(&p, want);
  if (err != cudaSuccess) {
    cudaGetLastError();  // clear the sticky-free error state of the failed allocation
    fail("workspace of %zu bytes: %s", want, cudaGetErrorString(err));
    return nullptr;
  }
  s.ptr = p;
  s.bytes = want;
  return p;
}

}  // namespace sptir

extern "C" {

const char* sparsetir_get_last_error(void) { return sptir::tls_error.c_str(); }

int sparsetir_set_stream(int device_id, void* stream) {
  if (device_id < 0 || device_id >= sptir::kMaxDevices)
    return sptir::fail("sparsetir_set_stream: device id %d out of range", device_id);
  sptir::g_streams[device_id].store(stream, std::memory_order_release);
  return 0;
}

void* sparsetir_get_stream(int device_id) { return sptir::stream_for(device_id); }

int sparsetir_version(void) { return 100; }

int sparsetir_sm_arch(void) { return 100; }

}  // extern "C"

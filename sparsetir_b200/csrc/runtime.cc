// Error string, stream table and device selection.
#include <algorithm>
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
// The stream of a (thread, device) pair, as in the reference, whose current stream is a member
// of the thread-local CUDAThreadEntry (src/runtime/cuda/cuda_device_api.cc:209-211).  A thread that
// never set one uses the process-wide default of the device.
std::atomic<void*> g_default_streams[kMaxDevices];
struct ThreadStreams {
  void* stream[kMaxDevices] = {};
  bool set[kMaxDevices] = {};
};
thread_local ThreadStreams tls_streams;
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
  if (tls_streams.set[device_id]) return static_cast<cudaStream_t>(tls_streams.stream[device_id]);
  return static_cast<cudaStream_t>(g_default_streams[device_id].load(std::memory_order_acquire));
}

namespace {
struct Scratch {
  void* ptr = nullptr;
  size_t bytes = 0;
};
std::mutex g_ws_mutex;
// [0]: plain scratch; [1]: scratch that is all zero whenever no kernel is using it
std::map<std::pair<int, cudaStream_t>, Scratch> g_ws[2];

// Grows the buffer of (device, stream) to at least `bytes`; with `zeroed`, a new buffer is cleared
// on `stream` before anything queued later can touch it.
void* grow(int kind, int device_id, cudaStream_t stream, size_t bytes) {
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  Scratch& s = g_ws[kind][{device_id, stream}];
  if (s.bytes >= bytes && s.ptr != nullptr) return s.ptr;
  if (s.ptr != nullptr) {
    cudaFree(s.ptr);  // synchronises: nothing in flight can still use the old buffer
    s.ptr = nullptr;
    s.bytes = 0;
  }
  const size_t unit = kind == 0 ? (size_t{1} << 20) : (size_t{1} << 12);
  const size_t want = (std::max<size_t>(bytes, 1) + unit - 1) & ~(unit - 1);
  void* p = nullptr;
  cudaError_t err = cudaMalloc(&p, want);
  if (err == cudaSuccess && kind == 1) {
    err = cudaMemsetAsync(p, 0, want, stream);
    if (err != cudaSuccess) cudaFree(p);
  }
  if (err != cudaSuccess) {
    cudaGetLastError();  // clear the error state of the failed call
    fail("workspace of %zu bytes: %s (reserve it before capturing a stream: "
         "sparsetir_reserve_workspace)", want, cudaGetErrorString(err));
    return nullptr;
  }
  s.ptr = p;
  s.bytes = want;
  return p;
}
}  // namespace

int peer_table(const char* fn, const void* own, int n_peers, void* const* peers, size_t align, PeerOut* out) {
  if (n_peers < 1 || n_peers > SPARSETIR_MAX_PEERS)
    return fail("%s: %d peers, expected 1 to %d", fn, n_peers, SPARSETIR_MAX_PEERS);
  if (peers == nullptr) return fail("%s: null peer table", fn);
  out->n = n_peers;
  for (int k = 0; k < n_peers; ++k) {
    if (peers[k] == nullptr) return fail("%s: peer %d is null", fn, k);
    const uintptr_t a = reinterpret_cast<uintptr_t>(peers[k]), o = reinterpret_cast<uintptr_t>(own);
    if (a % align != o % align)
      return fail("%s: peer %d is not aligned like the output itself (%zu bytes)", fn, k, align);
    out->delta[k] = static_cast<long long>(static_cast<intptr_t>(a) - static_cast<intptr_t>(o));
  }
  return 0;
}

void* workspace(int device_id, cudaStream_t stream, size_t bytes) {
  return grow(0, device_id, stream, bytes);
}

void* zeroed_workspace(int device_id, cudaStream_t stream, size_t bytes) {
  return grow(1, device_id, stream, bytes);
}

}  // namespace sptir

extern "C" {

const char* sparsetir_get_last_error(void) { return sptir::tls_error.c_str(); }

int sparsetir_set_stream(int device_id, void* stream) {
  if (device_id < 0 || device_id >= sptir::kMaxDevices)
    return sptir::fail("sparsetir_set_stream: device id %d out of range", device_id);
  sptir::tls_streams.stream[device_id] = stream;
  sptir::tls_streams.set[device_id] = true;
  return 0;
}

int sparsetir_set_default_stream(int device_id, void* stream) {
  if (device_id < 0 || device_id >= sptir::kMaxDevices)
    return sptir::fail("sparsetir_set_default_stream: device id %d out of range", device_id);
  sptir::g_default_streams[device_id].store(stream, std::memory_order_release);
  return 0;
}

int sparsetir_reserve_workspace(int device_id, void* stream, size_t scratch_bytes,
                                size_t counter_bytes) {
  if (sptir::use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (scratch_bytes > 0 && sptir::workspace(device_id, st, scratch_bytes) == nullptr) return -1;
  if (counter_bytes > 0 && sptir::zeroed_workspace(device_id, st, counter_bytes) == nullptr) return -1;
  return 0;
}

void* sparsetir_get_stream(int device_id) { return sptir::stream_for(device_id); }

int sparsetir_version(void) { return 100; }

int sparsetir_sm_arch(void) { return 100; }

}  // extern "C"

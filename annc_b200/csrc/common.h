// Shared host-side plumbing of libannc_b200: status + message, the calling
// thread's stream, host/device pointer classification, the per-thread staging
// arena and the registry of constants uploaded once.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <vector>

#include "annc_b200.h"

namespace annc {

// Records `code` and a printf-style message for annc_last_error(); returns code.
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define ANNC_CUDA(call)                                        \
  do {                                                         \
    cudaError_t annc_e_ = (call);                              \
    if (annc_e_ != cudaSuccess) return ::annc::cuda_fail(annc_e_, #call); \
  } while (0)

#define ANNC_TRY(call)                     \
  do {                                     \
    int annc_rc_ = (call);                 \
    if (annc_rc_ != ANNC_OK) return annc_rc_; \
  } while (0)

// OP_REQUIRES counterpart: the message is the reference's text.
#define ANNC_REQUIRE(cond, code, msg) \
  do {                                \
    if (!(cond)) return ::annc::fail(code, "%s", msg); \
  } while (0)

// Index of the current device, clamped to the size of the per-device caches below.  Function
// attributes, occupancy figures and symbol addresses belong to one device: code that caches them
// keeps one slot per device so that a process driving several GPUs sets each of them up.
constexpr int kMaxDevices = 64;
inline int device_slot() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0) d = 0;
  return d < kMaxDevices ? d : kMaxDevices - 1;
}

cudaStream_t current_stream();
// Events set with annc_embed_bag_set_timing_events on this thread (may be null).
void timing_events(cudaEvent_t* start, cudaEvent_t* stop);

inline int64_t numel(const annc_tensor& t) {
  int64_t n = 1;
  for (int i = 0; i < t.rank; ++i) n *= t.dims[i];
  return n;
}
size_t dtype_size(int32_t dtype);

// One entry-point invocation.  in()/out() turn caller pointers (host or device) into device
// pointers.  A host operand is given a device mirror keyed by (pointer, bytes, device) that
// persists between calls; an upload is skipped when a sampled fingerprint of the host contents
// equals the one taken when the mirror was last filled (weights and tables upload once; an
// output that comes back as the next call's input uploads not at all).  finish() copies host
// outputs back and, if anything was staged, waits.
class Call {
 public:
  Call();
  ~Call();
  int status() const { return status_; }
  cudaStream_t stream() const { return stream_; }

  // Device view of `bytes` bytes at p.  nullptr on failure (status() tells why) or when p is
  // null.  in_constant marks an operand in a weight / table position (reused under cache
  // mode 1 as well).
  const void* in(const void* p, size_t bytes);
  const void* in_constant(const void* p, size_t bytes);
  template <typename T>
  const T* in(const T* p, size_t count) {
    return static_cast<const T*>(in(static_cast<const void*>(p), count * sizeof(T)));
  }
  template <typename T>
  const T* in_constant(const T* p, size_t count) {
    return static_cast<const T*>(in_constant(static_cast<const void*>(p), count * sizeof(T)));
  }
  // Device buffer standing for output p; host outputs are copied back in finish().
  // `preload` uploads the current host contents first (for beta != 0).
  void* out(void* p, size_t bytes, bool preload = false);
  template <typename T>
  T* out(T* p, size_t count, bool preload = false) {
    return static_cast<T*>(out(static_cast<void*>(p), count * sizeof(T), preload));
  }
  // Device scratch valid until the next call of this thread on this device.
  void* scratch(size_t bytes);
  // A re-laid form (`tag`) of host operand p whose mirror is reusable: the cached buffer, or a
  // new one of out_bytes with *fresh set (the caller fills it).  nullptr when p has no reusable
  // mirror (device pointer, cache off) or memory is short: the caller then works without it.
  void* derived(const void* p, size_t bytes, int tag, size_t out_bytes, bool* fresh);
  // Small host read of possibly-device memory (synchronous).
  int read_host(const void* p, size_t bytes, void* dst);
  // True when p is device (or managed) memory.
  bool is_device(const void* p);
  // True when the call waited for its stream (then device-side error words can be read).
  bool synced() const { return synced_; }

  int finish();

 private:
  struct Pending {
    void* host;
    void* dev;
    size_t bytes;
  };
  struct Touched {
    const void* host;
    size_t bytes;
    int device;
  };
  const void* in_role(const void* p, size_t bytes, bool role_constant);
  void* mirror(const void* p, size_t bytes, bool upload, bool role_constant, bool is_output);
  cudaStream_t stream_;
  int device_;
  int status_ = ANNC_OK;
  bool staged_ = false;
  bool synced_ = false;
  bool used_scratch_ = false;
  std::vector<Pending> pending_;
  std::vector<Touched> touched_;
};

}  // namespace annc

// Status, stream, staging arena and constant registry of libannc_b200.
#include "common.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace annc {

namespace {

thread_local char g_error[512] = "";
thread_local cudaStream_t g_stream = nullptr;

struct Block {
  char* base;
  size_t cap;
  size_t used;
};

// Bump allocator over cudaMalloc'd blocks.  A call that outgrows the current
// block gets an extra block; the next call starts from one block of the
// combined size, so a steady workload settles on a single allocation.
struct Arena {
  std::vector<Block> blocks;
  ~Arena() { release(); }
  void release() {
    for (auto& b : blocks) cudaFree(b.base);
    blocks.clear();
  }
  void reset() {
    if (blocks.size() > 1) {
      size_t total = 0;
      for (auto& b : blocks) total += b.cap;
      release();
      char* p = nullptr;
      if (cudaMalloc(&p, total) == cudaSuccess) blocks.push_back({p, total, 0});
    } else if (blocks.size() == 1) {
      blocks[0].used = 0;
    }
  }
  void* alloc(size_t bytes) {
    bytes = (bytes + 255) & ~size_t(255);
    if (bytes == 0) bytes = 256;
    if (!blocks.empty()) {
      Block& b = blocks.back();
      if (b.used + bytes <= b.cap) {
        void* p = b.base + b.used;
        b.used += bytes;
        return p;
      }
    }
    size_t cap = bytes < (size_t(1) << 20) ? (size_t(1) << 20) : bytes;
    char* p = nullptr;
    if (cudaMalloc(&p, cap) != cudaSuccess) return nullptr;
    blocks.push_back({p, cap, bytes});
    return p;
  }
};

thread_local Arena g_arena;

struct Constant {
  void* dev;
  size_t bytes;
};
std::mutex g_const_mu;
std::unordered_map<const void*, Constant> g_constants;

}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(ANNC_ERR_CUDA, "CUDA error %d (%s) in %s", static_cast<int>(e),
              cudaGetErrorString(e), what);
}

cudaStream_t current_stream() { return g_stream; }

thread_local cudaEvent_t g_ev_start = nullptr, g_ev_stop = nullptr;
void timing_events(cudaEvent_t* start, cudaEvent_t* stop) {
  *start = g_ev_start;
  *stop = g_ev_stop;
}

size_t dtype_size(int32_t dtype) {
  switch (dtype) {
    case ANNC_F32:
    case ANNC_I32:
      return 4;
    case ANNC_I64:
    case ANNC_U64:
      return 8;
    case ANNC_BOOL:
      return 1;
    default:
      return 0;
  }
}

Call::Call() : stream_(g_stream) { g_arena.reset(); }
Call::~Call() {}

bool Call::is_device(const void* p) {
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (status_ == ANNC_OK) status_ = cuda_fail(e, "cudaPointerGetAttributes");
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

const void* Call::in(const void* p, size_t bytes) {
  if (p == nullptr || status_ != ANNC_OK) return nullptr;
  if (is_device(p)) return p;
  if (status_ != ANNC_OK) return nullptr;
  {
    std::lock_guard<std::mutex> lk(g_const_mu);
    auto it = g_constants.find(p);
    if (it != g_constants.end() && it->second.bytes >= bytes) return it->second.dev;
  }
  void* d = g_arena.alloc(bytes);
  if (!d) {
    status_ = fail(ANNC_ERR_CUDA, "device staging allocation of %zu bytes failed", bytes);
    return nullptr;
  }
  if (bytes) {
    cudaError_t e = cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, stream_);
    if (e != cudaSuccess) {
      status_ = cuda_fail(e, "cudaMemcpyAsync(H2D)");
      return nullptr;
    }
  }
  staged_ = true;
  return d;
}

void* Call::out(void* p, size_t bytes, bool preload) {
  if (p == nullptr || status_ != ANNC_OK) return nullptr;
  if (is_device(p)) return p;
  if (status_ != ANNC_OK) return nullptr;
  void* d = g_arena.alloc(bytes);
  if (!d) {
    status_ = fail(ANNC_ERR_CUDA, "device staging allocation of %zu bytes failed", bytes);
    return nullptr;
  }
  if (preload && bytes) {
    cudaError_t e = cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, stream_);
    if (e != cudaSuccess) {
      status_ = cuda_fail(e, "cudaMemcpyAsync(H2D)");
      return nullptr;
    }
  }
  pending_.push_back({p, d, bytes});
  staged_ = true;
  return d;
}

void* Call::scratch(size_t bytes) {
  if (status_ != ANNC_OK) return nullptr;
  void* d = g_arena.alloc(bytes);
  if (!d) status_ = fail(ANNC_ERR_CUDA, "device scratch allocation of %zu bytes failed", bytes);
  return d;
}

int Call::read_host(const void* p, size_t bytes, void* dst) {
  if (status_ != ANNC_OK) return status_;
  if (!is_device(p)) {
    if (status_ != ANNC_OK) return status_;
    memcpy(dst, p, bytes);
    return ANNC_OK;
  }
  cudaError_t e = cudaMemcpyAsync(dst, p, bytes, cudaMemcpyDeviceToHost, stream_);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream_);
  if (e != cudaSuccess) status_ = cuda_fail(e, "read_host");
  return status_;
}

int Call::finish() {
  if (status_ != ANNC_OK) return status_;
  for (auto& o : pending_) {
    if (!o.bytes) continue;
    cudaError_t e = cudaMemcpyAsync(o.host, o.dev, o.bytes, cudaMemcpyDeviceToHost, stream_);
    if (e != cudaSuccess) return status_ = cuda_fail(e, "cudaMemcpyAsync(D2H)");
  }
  pending_.clear();
  if (staged_) {
    cudaError_t e = cudaStreamSynchronize(stream_);
    if (e != cudaSuccess) return status_ = cuda_fail(e, "cudaStreamSynchronize");
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return status_ = cuda_fail(e, "kernel launch");
  return ANNC_OK;
}

}  // namespace annc

extern "C" {

const char* annc_last_error(void) { return annc::g_error; }

const char* annc_version(void) { return "annc_b200 0.1.0 sm_100a"; }

void annc_set_stream(void* s) { annc::g_stream = static_cast<cudaStream_t>(s); }
void* annc_get_stream(void) { return annc::g_stream; }

int annc_register_constant(const void* ptr, size_t bytes) {
  if (!ptr || !bytes) return annc::fail(ANNC_ERR_INVALID_ARGUMENT, "null constant");
  void* d = nullptr;
  ANNC_CUDA(cudaMalloc(&d, bytes));
  cudaError_t e = cudaMemcpy(d, ptr, bytes, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    cudaFree(d);
    return annc::cuda_fail(e, "cudaMemcpy(constant)");
  }
  std::lock_guard<std::mutex> lk(annc::g_const_mu);
  auto it = annc::g_constants.find(ptr);
  if (it != annc::g_constants.end()) cudaFree(it->second.dev);
  annc::g_constants[ptr] = {d, bytes};
  return ANNC_OK;
}

int annc_unregister_constant(const void* ptr) {
  std::lock_guard<std::mutex> lk(annc::g_const_mu);
  auto it = annc::g_constants.find(ptr);
  if (it == annc::g_constants.end()) return ANNC_ERR_INVALID_ARGUMENT;
  cudaFree(it->second.dev);
  annc::g_constants.erase(it);
  return ANNC_OK;
}

void* annc_timer_create(void) {
  cudaEvent_t e = nullptr;
  if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
  return e;
}
void annc_timer_destroy(void* ev) {
  if (ev) cudaEventDestroy(static_cast<cudaEvent_t>(ev));
}
int annc_timer_elapsed_ms(void* start, void* stop, float* ms) {
  ANNC_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(stop)));
  ANNC_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
  return ANNC_OK;
}
void annc_embed_bag_set_timing_events(void* start, void* stop) {
  annc::g_ev_start = static_cast<cudaEvent_t>(start);
  annc::g_ev_stop = static_cast<cudaEvent_t>(stop);
}

void annc_release_device_memory(void) {
  annc::g_arena.release();
  std::lock_guard<std::mutex> lk(annc::g_const_mu);
  for (auto& kv : annc::g_constants) cudaFree(kv.second.dev);
  annc::g_constants.clear();
}

}  // extern "C"

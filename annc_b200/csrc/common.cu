// Status, stream, scratch arena and the host-operand mirrors of libannc_b200.
//
// Entry points of groups (1) and (2) accept host pointers, as the reference's callers pass
// them.  Every host operand gets a device mirror keyed by (pointer, bytes, device) that
// persists between calls: callers of this ABI reuse their buffers (XLA buffer assignment, TF
// variables), so a steady workload allocates nothing.  Before an upload the host contents are
// compared, by a sampled fingerprint, with what the mirror holds; when they agree the upload is
// skipped.  That makes weights and tables upload once, and an output of one call that comes
// back as an input of the next (the host copy untouched in between) upload not at all.
#include "common.h"

#include <atomic>
#include <condition_variable>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <thread>
#include <unordered_map>

namespace annc {

namespace {

thread_local char g_error[512] = "";
thread_local cudaStream_t g_stream = nullptr;

// ---- scratch arena: bump allocator over cudaMalloc'd blocks, one per thread and device.
// Blocks are kept: a call that outgrows them adds one, reset() only rewinds.
struct Block {
  char* base;
  size_t cap;
  size_t used;
};
struct Arena {
  std::vector<Block> blocks;
  ~Arena() { release(); }
  void release() {
    for (auto& b : blocks) cudaFree(b.base);
    blocks.clear();
  }
  void reset() {
    for (auto& b : blocks) b.used = 0;
  }
  void* alloc(size_t bytes) {
    bytes = (bytes + 255) & ~size_t(255);
    if (bytes == 0) bytes = 256;
    for (auto& b : blocks) {
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
struct Arenas {
  Arena per_device[kMaxDevices];
};
thread_local Arenas g_arenas;
thread_local cudaStream_t g_last_stream[kMaxDevices] = {nullptr};
thread_local cudaEvent_t g_last_event[kMaxDevices] = {nullptr};
thread_local bool g_unsynced[kMaxDevices] = {false};

// ---- staged copies between pageable host memory and the device.
// A large operand moves through a pinned two-half bounce buffer of the calling thread: while
// the DMA of one half runs, the next chunk is copied between the caller's (pageable) buffer and
// the other half, by the caller and three helper threads (a single thread copies at about a
// fifth of what the link takes).  Small operands take the driver's own staging.
constexpr size_t kChunk = size_t(8) << 20;

class CopyPool {
 public:
  static CopyPool& get() {
    static CopyPool* p = new CopyPool();  // lives for the process: helpers never outlive it
    return *p;
  }
  // memcpy(dst, src, n) split over the helpers and the caller
  void copy(char* dst, const char* src, size_t n) {
    constexpr int kParts = kHelpers + 1;
    if (n < (size_t(1) << 20)) {
      memcpy(dst, src, n);
      return;
    }
    std::lock_guard<std::mutex> one_at_a_time(caller_mu_);
    const size_t part = ((n / kParts) + 63) & ~size_t(63);
    {
      std::lock_guard<std::mutex> lk(mu_);
      for (int i = 0; i < kHelpers; ++i) {
        const size_t off = (size_t)(i + 1) * part;
        job_[i] = {dst + off, src + off, off < n ? (off + part < n && i + 1 < kHelpers ? part : n - off) : 0};
      }
      pending_ = kHelpers;
      ++generation_;
    }
    cv_.notify_all();
    memcpy(dst, src, part < n ? part : n);
    std::unique_lock<std::mutex> lk(mu_);
    done_cv_.wait(lk, [&] { return pending_ == 0; });
  }

 private:
  static constexpr int kHelpers = 3;
  struct Job {
    char* dst;
    const char* src;
    size_t n;
  };
  CopyPool() {
    for (int i = 0; i < kHelpers; ++i) std::thread([this, i] { work(i); }).detach();
  }
  void work(int i) {
    unsigned long long seen = 0;
    for (;;) {
      Job j;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return generation_ != seen; });
        seen = generation_;
        j = job_[i];
      }
      if (j.n) memcpy(j.dst, j.src, j.n);
      {
        std::lock_guard<std::mutex> lk(mu_);
        --pending_;
      }
      done_cv_.notify_all();
    }
  }
  std::mutex mu_, caller_mu_;
  std::condition_variable cv_, done_cv_;
  Job job_[kHelpers] = {};
  int pending_ = 0;
  unsigned long long generation_ = 0;
};

struct Bounce {
  char* base = nullptr;
  cudaEvent_t ev[2] = {nullptr, nullptr};
  bool tried = false;
};
thread_local Bounce g_bounce;

bool bounce_ready() {
  Bounce& b = g_bounce;
  if (b.base) return true;
  if (b.tried) return false;
  b.tried = true;
  if (cudaHostAlloc(reinterpret_cast<void**>(&b.base), 2 * kChunk, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError();
    b.base = nullptr;
    return false;
  }
  cudaEventCreateWithFlags(&b.ev[0], cudaEventDisableTiming);
  cudaEventCreateWithFlags(&b.ev[1], cudaEventDisableTiming);
  return true;
}

cudaError_t staged_h2d(void* dev, const void* host, size_t bytes, cudaStream_t s) {
  if (bytes < kChunk / 4 || !bounce_ready())
    return cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, s);
  Bounce& b = g_bounce;
  size_t i = 0;
  for (size_t off = 0; off < bytes; off += kChunk, ++i) {
    const int h = (int)(i & 1);
    const size_t n = bytes - off < kChunk ? bytes - off : kChunk;
    cudaEventSynchronize(b.ev[h]);  // the DMA that last read this half has finished
    CopyPool::get().copy(b.base + h * kChunk, static_cast<const char*>(host) + off, n);
    cudaError_t e = cudaMemcpyAsync(static_cast<char*>(dev) + off, b.base + h * kChunk, n,
                                    cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return e;
    cudaEventRecord(b.ev[h], s);
  }
  return cudaSuccess;
}

// Returns with the host buffer complete (waits for the stream up to its last chunk).
cudaError_t staged_d2h(void* host, const void* dev, size_t bytes, cudaStream_t s) {
  if (bytes < kChunk / 4 || !bounce_ready())
    return cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, s);
  Bounce& b = g_bounce;
  size_t i = 0, prev_off = 0, prev_n = 0;
  for (size_t off = 0; off < bytes; off += kChunk, ++i) {
    const int h = (int)(i & 1);
    const size_t n = bytes - off < kChunk ? bytes - off : kChunk;
    cudaEventSynchronize(b.ev[h]);  // an earlier upload may still read this half
    cudaError_t e = cudaMemcpyAsync(b.base + h * kChunk, static_cast<const char*>(dev) + off, n,
                                    cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return e;
    cudaEventRecord(b.ev[h], s);
    if (i > 0) {  // the previous chunk has landed in the other half: move it out under this DMA
      const int ph = (int)((i - 1) & 1);
      e = cudaEventSynchronize(b.ev[ph]);
      if (e != cudaSuccess) return e;
      CopyPool::get().copy(static_cast<char*>(host) + prev_off, b.base + ph * kChunk, prev_n);
    }
    prev_off = off;
    prev_n = n;
  }
  const int lh = (int)((i - 1) & 1);
  cudaError_t e = cudaEventSynchronize(b.ev[lh]);
  if (e != cudaSuccess) return e;
  CopyPool::get().copy(static_cast<char*>(host) + prev_off, b.base + lh * kChunk, prev_n);
  return cudaSuccess;
}

// ---- mirrors
struct Key {
  const void* host;
  size_t bytes;
  int device;
  bool operator==(const Key& o) const { return host == o.host && bytes == o.bytes && device == o.device; }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    size_t h = reinterpret_cast<size_t>(k.host) * 0x9E3779B97F4A7C15ull;
    h ^= k.bytes + 0x7F4A7C15ull + (h << 6) + (h >> 2);
    return h ^ (size_t)k.device;
  }
};
struct Mirror {
  void* dev = nullptr;
  size_t bytes = 0;
  unsigned long long print = 0;  // fingerprint of the host contents the mirror holds
  bool valid = false;            // the mirror holds those contents
  bool pinned = false;           // registered with annc_register_constant: never evicted, never re-checked
  unsigned long long tick = 0;
  int users = 0;                 // calls copying into the mirror right now: not to be evicted
  cudaEvent_t ready = nullptr;   // after the last write of the mirror
  cudaEvent_t used = nullptr;    // after the last read of the mirror
  std::unordered_map<int, std::pair<void*, size_t>> derived;  // re-laid forms of a constant, by tag
};
std::mutex g_mu;
std::unordered_map<Key, Mirror, KeyHash> g_mirrors;
size_t g_mirror_bytes = 0;
size_t g_mirror_cap = size_t(24) << 30;
unsigned long long g_tick = 0;
int g_mode = 2;  // 0: no mirror reuse, 1: constants (weight positions) only, 2: every operand
std::atomic<unsigned long long> g_staged_h2d{0}, g_staged_d2h{0}, g_skipped_h2d{0};

// One 8-byte word per 4 KiB page (at most `max_samples` of them, evenly spread), the first and
// the last 64 bytes, and the length.  Operands in weight positions are sampled more thinly
// (512 words): they change when a model is reloaded, not between two steps.
unsigned long long fingerprint(const void* p, size_t bytes, size_t max_samples = 16384) {
  const unsigned char* b = static_cast<const unsigned char*>(p);
  unsigned long long h = 0xcbf29ce484222325ull ^ bytes;
  auto mix = [&](unsigned long long v) {
    h ^= v;
    h *= 0x100000001b3ull;
    h ^= h >> 29;
  };
  auto word = [&](size_t off) {
    unsigned long long v = 0;
    const size_t n = bytes - off < 8 ? bytes - off : 8;
    memcpy(&v, b + off, n);
    return v;
  };
  if (bytes <= 4096) {
    for (size_t o = 0; o < bytes; o += 8) mix(word(o));
    return h;
  }
  for (size_t o = 0; o < 64; o += 8) mix(word(o));
  for (size_t o = bytes - 64; o < bytes; o += 8) mix(word(o));
  size_t pages = bytes / 4096;
  size_t step = 4096;
  if (pages > max_samples) step = (bytes / max_samples) & ~size_t(7);
  // the sampled word moves inside its page with the page number, so that a regular pattern
  // (one changed column of a matrix) does not hide between the samples
  size_t k = 0;
  for (size_t o = 0; o + 8 <= bytes; o += step, ++k) {
    size_t at = o + ((k * 520) & 4088 & (step - 8));
    if (at + 8 > bytes) at = bytes - 8;
    mix(word(at));
  }
  return h;
}

void free_mirror(Mirror& m) {
  if (m.dev) cudaFree(m.dev);
  for (auto& d : m.derived) cudaFree(d.second.first);
  if (m.ready) cudaEventDestroy(m.ready);
  if (m.used) cudaEventDestroy(m.used);
  g_mirror_bytes -= m.bytes;
  for (auto& d : m.derived) g_mirror_bytes -= d.second.second;
}

// Drops least recently used mirrors until `need` more bytes fit under the cap (called with g_mu held).
void make_room(size_t need, const Key* keep) {
  while (g_mirror_bytes + need > g_mirror_cap && !g_mirrors.empty()) {
    auto victim = g_mirrors.end();
    for (auto it = g_mirrors.begin(); it != g_mirrors.end(); ++it) {
      if (it->second.pinned || it->second.users > 0 || (keep && it->first == *keep)) continue;
      if (victim == g_mirrors.end() || it->second.tick < victim->second.tick) victim = it;
    }
    if (victim == g_mirrors.end()) break;
    if (victim->second.used) cudaEventSynchronize(victim->second.used);
    if (victim->second.ready) cudaEventSynchronize(victim->second.ready);
    free_mirror(victim->second);
    g_mirrors.erase(victim);
  }
}

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

Call::Call() : stream_(g_stream), device_(device_slot()) {
  g_arenas.per_device[device_].reset();
  // A previous call of this thread that returned without synchronising (device pointers only)
  // may still use the arena's scratch on another stream: order this call's stream after it.
  if (g_unsynced[device_] && g_last_event[device_] && g_last_stream[device_] != stream_)
    cudaStreamWaitEvent(stream_, g_last_event[device_], 0);
}
Call::~Call() {
  if (used_scratch_ && !synced_) {
    if (!g_last_event[device_]) cudaEventCreateWithFlags(&g_last_event[device_], cudaEventDisableTiming);
    if (g_last_event[device_]) cudaEventRecord(g_last_event[device_], stream_);
    g_last_stream[device_] = stream_;
    g_unsynced[device_] = true;
  } else if (synced_) {
    g_unsynced[device_] = false;
  }
}

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

// Device mirror of host operand p.  upload: the host contents are needed on the device.
// role_constant: the operand sits in a weight / table position.
void* Call::mirror(const void* p, size_t bytes, bool upload, bool role_constant, bool is_output) {
  if (bytes == 0) bytes = 1;
  const Key key{p, bytes, device_};
  Mirror* mp = nullptr;
  bool need = false, may_reuse = false;
  unsigned long long fp = 0;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_mirrors.find(key);
    if (it == g_mirrors.end()) {
      make_room(bytes, nullptr);
      Mirror m;
      cudaError_t e = cudaMalloc(&m.dev, bytes);
      if (e != cudaSuccess) {
        cudaGetLastError();
        make_room(g_mirror_cap, nullptr);  // drop everything evictable and try once more
        e = cudaMalloc(&m.dev, bytes);
      }
      if (e != cudaSuccess) {
        cudaGetLastError();
        status_ = fail(ANNC_ERR_CUDA, "device allocation of %zu bytes for a host operand failed", bytes);
        return nullptr;
      }
      m.bytes = bytes;
      cudaEventCreateWithFlags(&m.ready, cudaEventDisableTiming);
      cudaEventCreateWithFlags(&m.used, cudaEventDisableTiming);
      g_mirror_bytes += bytes;
      it = g_mirrors.emplace(key, m).first;
    }
    Mirror& m = it->second;
    mp = &m;  // stays where it is: entries are only erased by eviction, which skips `users`
    m.tick = ++g_tick;
    may_reuse = !m.pinned && (g_mode == 2 || (g_mode == 1 && role_constant));
    if (upload) {
      need = true;
      if (m.pinned && m.valid) {
        need = false;
      } else if (may_reuse) {
        fp = fingerprint(p, bytes, role_constant ? 512 : 16384);
        need = !(m.valid && m.print == fp);
      }
      if (need) {
        ++m.users;
        // writers wait for the readers and the writer before them
        cudaStreamWaitEvent(stream_, m.used, 0);
        cudaStreamWaitEvent(stream_, m.ready, 0);
        m.valid = false;
      } else {
        cudaStreamWaitEvent(stream_, m.ready, 0);
        g_skipped_h2d += bytes;
      }
      touched_.push_back({key.host, key.bytes, key.device});
    } else if (is_output) {
      cudaStreamWaitEvent(stream_, m.used, 0);
      cudaStreamWaitEvent(stream_, m.ready, 0);
      m.valid = false;  // becomes valid again in finish(), once the host copy exists
      for (auto& d : m.derived) {
        cudaFree(d.second.first);
        g_mirror_bytes -= d.second.second;
      }
      m.derived.clear();
    }
  }
  if (need) {  // the copy itself runs outside the lock: other threads' calls go on
    const cudaError_t e = staged_h2d(mp->dev, p, bytes, stream_);
    std::lock_guard<std::mutex> lk(g_mu);
    --mp->users;
    if (e != cudaSuccess) {
      status_ = cuda_fail(e, "host-to-device copy");
      return nullptr;
    }
    cudaEventRecord(mp->ready, stream_);
    g_staged_h2d += bytes;
    mp->valid = may_reuse;
    mp->print = fp;
    for (auto& d : mp->derived) {  // re-laid forms are stale now
      cudaFree(d.second.first);
      g_mirror_bytes -= d.second.second;
    }
    mp->derived.clear();
    staged_ = true;
  }
  return mp->dev;
}

const void* Call::in(const void* p, size_t bytes) { return in_role(p, bytes, false); }
const void* Call::in_constant(const void* p, size_t bytes) { return in_role(p, bytes, true); }

const void* Call::in_role(const void* p, size_t bytes, bool role_constant) {
  if (p == nullptr || status_ != ANNC_OK) return nullptr;
  if (is_device(p)) return p;
  if (status_ != ANNC_OK) return nullptr;
  return mirror(p, bytes, true, role_constant, false);
}

void* Call::out(void* p, size_t bytes, bool preload) {
  if (p == nullptr || status_ != ANNC_OK) return nullptr;
  if (is_device(p)) return p;
  if (status_ != ANNC_OK) return nullptr;
  void* d = preload ? mirror(p, bytes, true, false, false) : mirror(p, bytes, false, false, true);
  if (!d) return nullptr;
  if (preload) {  // the call overwrites what was uploaded
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_mirrors.find(Key{p, bytes ? bytes : 1, device_});
    if (it != g_mirrors.end()) it->second.valid = false;
  }
  pending_.push_back({p, d, bytes});
  staged_ = true;
  return d;
}

void* Call::scratch(size_t bytes) {
  if (status_ != ANNC_OK) return nullptr;
  void* d = g_arenas.per_device[device_].alloc(bytes);
  if (!d) status_ = fail(ANNC_ERR_CUDA, "device scratch allocation of %zu bytes failed", bytes);
  used_scratch_ = true;
  return d;
}

// A re-laid form (`tag`) of constant host operand p, kept with its mirror: returns the cached
// device buffer, or allocates `out_bytes` and sets *fresh so that the caller fills it.
void* Call::derived(const void* p, size_t bytes, int tag, size_t out_bytes, bool* fresh) {
  *fresh = false;
  if (status_ != ANNC_OK) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_mirrors.find(Key{p, bytes ? bytes : 1, device_});
  if (it == g_mirrors.end() || !it->second.valid) return nullptr;  // not a mirrored, reusable operand
  Mirror& m = it->second;
  auto d = m.derived.find(tag);
  if (d != m.derived.end() && d->second.second == out_bytes) return d->second.first;
  make_room(out_bytes, &it->first);
  void* buf = nullptr;
  if (cudaMalloc(&buf, out_bytes) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  m.derived[tag] = {buf, out_bytes};
  g_mirror_bytes += out_bytes;
  *fresh = true;
  return buf;
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
  synced_ = true;
  return status_;
}

int Call::finish() {
  if (status_ != ANNC_OK) return status_;
  for (auto& o : pending_) {
    if (!o.bytes) continue;
    cudaError_t e = staged_d2h(o.host, o.dev, o.bytes, stream_);
    if (e != cudaSuccess) return status_ = cuda_fail(e, "device-to-host copy");
    g_staged_d2h += o.bytes;
  }
  {  // this call's reads and writes of the mirrors end here on its stream
    std::lock_guard<std::mutex> lk(g_mu);
    for (auto& k : touched_) {
      auto it = g_mirrors.find(Key{k.host, k.bytes, k.device});
      if (it != g_mirrors.end()) cudaEventRecord(it->second.used, stream_);
    }
    for (auto& o : pending_) {
      auto it = g_mirrors.find(Key{o.host, o.bytes ? o.bytes : 1, device_});
      if (it != g_mirrors.end()) cudaEventRecord(it->second.ready, stream_);
    }
  }
  if (staged_) {
    cudaError_t e = cudaStreamSynchronize(stream_);
    if (e != cudaSuccess) return status_ = cuda_fail(e, "cudaStreamSynchronize");
    synced_ = true;
    // the host copies exist now: an output mirror holds exactly what the host buffer holds
    if (g_mode == 2 && !pending_.empty()) {
      std::lock_guard<std::mutex> lk(g_mu);
      for (auto& o : pending_) {
        auto it = g_mirrors.find(Key{o.host, o.bytes ? o.bytes : 1, device_});
        if (it == g_mirrors.end() || !o.bytes) continue;
        it->second.print = fingerprint(o.host, o.bytes);
        it->second.valid = true;
      }
    }
  }
  pending_.clear();
  touched_.clear();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return status_ = cuda_fail(e, "kernel launch");
  return ANNC_OK;
}

}  // namespace annc

extern "C" {

const char* annc_last_error(void) { return annc::g_error; }

const char* annc_version(void) { return "annc_b200 0.2.0 sm_100a"; }

void annc_set_stream(void* s) { annc::g_stream = static_cast<cudaStream_t>(s); }
void* annc_get_stream(void) { return annc::g_stream; }

int annc_register_constant(const void* ptr, size_t bytes) {
  if (!ptr || !bytes) return annc::fail(ANNC_ERR_INVALID_ARGUMENT, "null constant");
  using namespace annc;
  const Key key{ptr, bytes, device_slot()};
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_mirrors.find(key);
  if (it == g_mirrors.end()) {
    Mirror m;
    ANNC_CUDA(cudaMalloc(&m.dev, bytes));
    m.bytes = bytes;
    cudaEventCreateWithFlags(&m.ready, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&m.used, cudaEventDisableTiming);
    g_mirror_bytes += bytes;
    it = g_mirrors.emplace(key, m).first;
  }
  Mirror& m = it->second;
  if (m.used) cudaEventSynchronize(m.used);
  cudaError_t e = cudaMemcpy(m.dev, ptr, bytes, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(constant)");
  g_staged_h2d += bytes;
  m.valid = true;
  m.pinned = true;
  m.print = fingerprint(ptr, bytes);
  return ANNC_OK;
}

int annc_unregister_constant(const void* ptr) {
  using namespace annc;
  std::lock_guard<std::mutex> lk(g_mu);
  const int dev = device_slot();
  for (auto it = g_mirrors.begin(); it != g_mirrors.end(); ++it) {
    if (it->first.host == ptr && it->first.device == dev && it->second.pinned) {
      cudaDeviceSynchronize();
      free_mirror(it->second);
      g_mirrors.erase(it);
      return ANNC_OK;
    }
  }
  return ANNC_ERR_INVALID_ARGUMENT;
}

int annc_set_operand_cache(int mode, size_t max_bytes) {
  if (mode < 0 || mode > 2) return annc::fail(ANNC_ERR_INVALID_ARGUMENT, "operand cache mode must be 0, 1 or 2");
  std::lock_guard<std::mutex> lk(annc::g_mu);
  annc::g_mode = mode;
  if (max_bytes) annc::g_mirror_cap = max_bytes;
  return ANNC_OK;
}

void annc_staging_counters(uint64_t* h2d_bytes, uint64_t* d2h_bytes, uint64_t* h2d_skipped_bytes) {
  if (h2d_bytes) *h2d_bytes = annc::g_staged_h2d.load();
  if (d2h_bytes) *d2h_bytes = annc::g_staged_d2h.load();
  if (h2d_skipped_bytes) *h2d_skipped_bytes = annc::g_skipped_h2d.load();
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
  using namespace annc;
  cudaDeviceSynchronize();
  for (auto& a : g_arenas.per_device) a.release();
  std::lock_guard<std::mutex> lk(g_mu);
  for (auto& kv : g_mirrors) free_mirror(kv.second);
  g_mirrors.clear();
  g_mirror_bytes = 0;
}

}  // extern "C"

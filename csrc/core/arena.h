// Caching memory arena of the C++ runtime (reference: src/common/allocator.h, src/utils/simple_mem_pool.h — a
// name-keyed buffer pool — and the NUMA allocator; here the resources are device memory and pinned host staging).
//
// Blocks are handed out from per-size free lists (sizes rounded up to 512 B below 1 MiB and to 2 MiB above), so the
// steady state of a serving loop allocates nothing: a freed block is kept and reused by the next request of its
// class.  The backend (cudaMalloc / cudaFree, cudaMallocHost / cudaFreeHost, or malloc / free in tests) is a pair of
// function pointers.  `trim()` returns cached blocks to the backend; the destructor frees everything still cached.
#pragma once
#include <cstddef>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace xft {

class Arena {
public:
  using AllocFn = void* (*)(size_t);
  using FreeFn = void (*)(void*);
  Arena(AllocFn a, FreeFn f) : alloc_(a), free_(f) {}
  ~Arena();
  Arena(const Arena&) = delete;
  Arena& operator=(const Arena&) = delete;

  void* allocate(size_t bytes);        // never returns a block smaller than asked; nullptr when the backend fails
  void release(void* p);               // back to the free list of its class (unknown pointers are ignored)
  void trim();                         // give cached blocks back to the backend
  size_t bytesInUse() const { return inUse_; }
  size_t bytesCached() const { return cached_; }
  size_t backendCalls() const { return backendCalls_; }
  static size_t roundUp(size_t bytes);

  static Arena& device();              // cudaMalloc / cudaFree on the current device
  static Arena& pinned();              // cudaMallocHost / cudaFreeHost

private:
  AllocFn alloc_;
  FreeFn free_;
  mutable std::mutex mu_;
  std::map<size_t, std::vector<void*>> free_lists_;
  std::unordered_map<void*, size_t> live_;
  size_t inUse_ = 0, cached_ = 0, backendCalls_ = 0;
};

// RAII handle
class ArenaBuf {
public:
  ArenaBuf() = default;
  ArenaBuf(Arena& a, size_t bytes) : arena_(&a), p_(a.allocate(bytes)), bytes_(bytes) {}
  ~ArenaBuf() { reset(); }
  ArenaBuf(ArenaBuf&& o) noexcept : arena_(o.arena_), p_(o.p_), bytes_(o.bytes_) { o.p_ = nullptr; }
  ArenaBuf& operator=(ArenaBuf&& o) noexcept {
    if (this != &o) { reset(); arena_ = o.arena_; p_ = o.p_; bytes_ = o.bytes_; o.p_ = nullptr; }
    return *this;
  }
  void reset() { if (p_ && arena_) arena_->release(p_); p_ = nullptr; }
  void* get() const { return p_; }
  size_t size() const { return bytes_; }
private:
  Arena* arena_ = nullptr;
  void* p_ = nullptr;
  size_t bytes_ = 0;
};

}  // namespace xft

#include "arena.h"

#include <cuda_runtime.h>

#include <cstdlib>

namespace xft {

size_t Arena::roundUp(size_t bytes) {
  if (bytes == 0) bytes = 1;
  // XFT_ARENA_EXACT=1 (sanitizer runs against the host stand-in of the device library): blocks have exactly the size
  // asked for, so an access past a buffer's end is seen instead of landing in the rounding slack
  static const bool exact = [] { const char* v = std::getenv("XFT_ARENA_EXACT"); return v && *v && *v != '0'; }();
  if (exact) return bytes;
  const size_t g = bytes < (1u << 20) ? 512 : (2u << 20);
  return (bytes + g - 1) / g * g;
}

Arena::~Arena() {
  trim();
  // blocks still in use at exit belong to objects that outlive the arena (process teardown): leave them to the OS
}

void* Arena::allocate(size_t bytes) {
  const size_t cls = roundUp(bytes);
  std::lock_guard<std::mutex> g(mu_);
  auto it = free_lists_.find(cls);
  void* p = nullptr;
  if (it != free_lists_.end() && !it->second.empty()) {
    p = it->second.back();
    it->second.pop_back();
    cached_ -= cls;
  } else {
    p = alloc_(cls);
    ++backendCalls_;
    if (!p) {
      // memory pressure: drop the cache and retry once
      for (auto& kv : free_lists_) {
        for (void* q : kv.second) free_(q);
        kv.second.clear();
      }
      cached_ = 0;
      p = alloc_(cls);
      ++backendCalls_;
      if (!p) return nullptr;
    }
  }
  live_[p] = cls;
  inUse_ += cls;
  return p;
}

void Arena::release(void* p) {
  if (!p) return;
  std::lock_guard<std::mutex> g(mu_);
  auto it = live_.find(p);
  if (it == live_.end()) return;
  const size_t cls = it->second;
  live_.erase(it);
  inUse_ -= cls;
  cached_ += cls;
  free_lists_[cls].push_back(p);
}

void Arena::trim() {
  std::lock_guard<std::mutex> g(mu_);
  for (auto& kv : free_lists_) {
    for (void* q : kv.second) free_(q);
    kv.second.clear();
  }
  cached_ = 0;
}

namespace {
void* devAlloc(size_t n) { void* p = nullptr; return cudaMalloc(&p, n) == cudaSuccess ? p : (cudaGetLastError(), nullptr); }
void devFree(void* p) { cudaFree(p); }
void* pinAlloc(size_t n) { void* p = nullptr; return cudaMallocHost(&p, n) == cudaSuccess ? p : (cudaGetLastError(), nullptr); }
void pinFree(void* p) { cudaFreeHost(p); }
}  // namespace

Arena& Arena::device() {
  static Arena* a = new Arena(devAlloc, devFree);     // leaked on purpose: outlives static destruction order
  return *a;
}
Arena& Arena::pinned() {
  static Arena* a = new Arena(pinAlloc, pinFree);
  return *a;
}

}  // namespace xft

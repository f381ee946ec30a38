// A stand-in for libnccl.so.2 for tests WITHOUT GPUs: the entry points csrc/core/comm.cc resolves with dlsym,
// working on HOST pointers between processes of one machine through a shared-memory file.  Built as a shared object by
// tests/test_cpp_runtime.py and handed to the communicator through XFT_NCCL_LIB, next to host stand-ins for the CUDA
// runtime calls (csrc/tests/comm_selftest.cc).  It implements just what the test needs: float32 / bfloat16 / uint8
// data, sum, up to 8 ranks, messages up to 4 MiB; point-to-point messages go through the sender's slot (one message per
// pair at a time, the sender waits until it is taken); a split makes a new shared-memory file per colour.
#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace {
constexpr size_t kSlot = 4u << 20;
struct Shared {
  std::atomic<int> arrived;
  std::atomic<int> generation;
  std::atomic<int> mail[64];             // [source * 8 + destination]: 1 while a message waits in the source's slot
  std::atomic<int> splits;               // how many splits this communicator has made (names of the new files)
  char pad[52];
};
struct Comm { int rank, world; Shared* sh; char* slots; size_t bytes; char name[128]; };
struct Id { char bytes[128]; };

// Waits give up after XFT_DIST_TIMEOUT_S seconds (120 when unset): a test on a loaded machine must not fail because a
// sibling process was slow, yet a lost rank must not hang it for ever.
struct Deadline {
  std::chrono::steady_clock::time_point end;
  Deadline() {
    const char* v = std::getenv("XFT_DIST_TIMEOUT_S");
    end = std::chrono::steady_clock::now() + std::chrono::seconds(v && *v ? std::max(1, std::atoi(v)) : 120);
  }
  bool passed(long spin) const { return (spin & 4095) == 4095 && std::chrono::steady_clock::now() > end; }
};

void barrier(Comm* c) {
  const int gen = c->sh->generation.load();
  if (c->sh->arrived.fetch_add(1) + 1 == c->world) {
    c->sh->arrived.store(0);
    c->sh->generation.fetch_add(1);
  } else {
    const Deadline limit;
    for (long spin = 0; c->sh->generation.load() == gen; ++spin) {
      if (limit.passed(spin)) { std::fprintf(stderr, "fake nccl: barrier timed out\n"); std::_Exit(3); }
      if ((spin & 1023) == 1023) usleep(50);
    }
  }
}
size_t elemSize(int dt) { return dt == 7 ? 4 : dt == 9 ? 2 : 1; }
float bf16ToFloat(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; std::memcpy(&f, &u, 4); return f; }
uint16_t floatToBf16(float f) { uint32_t u; std::memcpy(&u, &f, 4); u += 0x7fff + ((u >> 16) & 1); return (uint16_t)(u >> 16); }
}  // namespace

extern "C" {
int ncclGetUniqueId(Id* id) {
  std::memset(id, 0, sizeof(*id));
  std::snprintf(id->bytes, sizeof(id->bytes), "/xft_fake_nccl_%d_%ld", (int)getpid(), (long)random());
  return 0;
}
int ncclCommInitRank(void** comm, int world, Id id, int rank) {
  if (world < 1 || world > 8) return 4;
  const size_t bytes = sizeof(Shared) + (size_t)world * kSlot;
  int fd = -1;
  if (rank == 0) {
    fd = shm_open(id.bytes, O_CREAT | O_RDWR, 0600);
    if (fd < 0 || ftruncate(fd, (off_t)bytes) != 0) return 2;
  } else {
    for (int i = 0; i < 4000 && fd < 0; ++i) { fd = shm_open(id.bytes, O_RDWR, 0600); if (fd < 0) usleep(1000); }
    if (fd < 0) return 2;
    for (int i = 0; i < 4000; ++i) { off_t sz = lseek(fd, 0, SEEK_END); if ((size_t)sz >= bytes) break; usleep(1000); }
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) return 2;
  Comm* c = new Comm{rank, world, static_cast<Shared*>(p), static_cast<char*>(p) + sizeof(Shared), bytes, {0}};
  std::snprintf(c->name, sizeof(c->name), "%s", id.bytes);
  *comm = c;
  barrier(c);
  if (rank == 0) shm_unlink(id.bytes);
  return 0;
}
int ncclCommDestroy(void* comm) {
  Comm* c = static_cast<Comm*>(comm);
  munmap(c->sh, c->bytes);
  delete c;
  return 0;
}
int ncclAllReduce(const void* send, void* recv, size_t count, int dt, int op, void* comm, void*) {
  Comm* c = static_cast<Comm*>(comm);
  const size_t bytes = count * elemSize(dt);
  if (op != 0 || bytes > kSlot || (dt != 7 && dt != 9)) return 4;
  std::memcpy(c->slots + (size_t)c->rank * kSlot, send, bytes);
  barrier(c);
  for (size_t i = 0; i < count; ++i) {
    float a = 0.f;
    for (int r = 0; r < c->world; ++r) {
      const char* s = c->slots + (size_t)r * kSlot;
      a += dt == 7 ? reinterpret_cast<const float*>(s)[i] : bf16ToFloat(reinterpret_cast<const uint16_t*>(s)[i]);
    }
    if (dt == 7) static_cast<float*>(recv)[i] = a; else static_cast<uint16_t*>(recv)[i] = floatToBf16(a);
  }
  barrier(c);
  return 0;
}
int ncclAllGather(const void* send, void* recv, size_t count, int dt, void* comm, void*) {
  Comm* c = static_cast<Comm*>(comm);
  const size_t bytes = count * elemSize(dt);
  if (bytes > kSlot) return 4;
  std::memcpy(c->slots + (size_t)c->rank * kSlot, send, bytes);
  barrier(c);
  for (int r = 0; r < c->world; ++r) std::memcpy(static_cast<char*>(recv) + (size_t)r * bytes, c->slots + (size_t)r * kSlot, bytes);
  barrier(c);
  return 0;
}
int ncclBroadcast(const void* send, void* recv, size_t count, int dt, int root, void* comm, void*) {
  Comm* c = static_cast<Comm*>(comm);
  const size_t bytes = count * elemSize(dt);
  if (bytes > kSlot) return 4;
  if (c->rank == root) std::memcpy(c->slots + (size_t)root * kSlot, send, bytes);
  barrier(c);
  std::memcpy(recv, c->slots + (size_t)root * kSlot, bytes);
  barrier(c);
  return 0;
}
// point to point: the message waits in the second half of the sender's slot, so a collective in flight is not disturbed
int ncclSend(const void* send, size_t count, int dt, int peer, void* comm, void*) {
  Comm* c = static_cast<Comm*>(comm);
  const size_t bytes = count * elemSize(dt);
  if (bytes > kSlot / 2 || peer < 0 || peer >= c->world || peer == c->rank) return 4;
  std::atomic<int>& flag = c->sh->mail[c->rank * 8 + peer];
  std::memcpy(c->slots + (size_t)c->rank * kSlot + kSlot / 2, send, bytes);
  flag.store(1);
  const Deadline limit;
  for (long spin = 0; flag.load() != 0; ++spin) {
    if (limit.passed(spin)) { std::fprintf(stderr, "fake nccl: send timed out\n"); std::_Exit(3); }
    if ((spin & 1023) == 1023) usleep(50);
  }
  return 0;
}
int ncclRecv(void* recv, size_t count, int dt, int peer, void* comm, void*) {
  Comm* c = static_cast<Comm*>(comm);
  const size_t bytes = count * elemSize(dt);
  if (bytes > kSlot / 2 || peer < 0 || peer >= c->world || peer == c->rank) return 4;
  std::atomic<int>& flag = c->sh->mail[peer * 8 + c->rank];
  const Deadline limit;
  for (long spin = 0; flag.load() != 1; ++spin) {
    if (limit.passed(spin)) { std::fprintf(stderr, "fake nccl: receive timed out\n"); std::_Exit(3); }
    if ((spin & 1023) == 1023) usleep(50);
  }
  std::memcpy(recv, c->slots + (size_t)peer * kSlot + kSlot / 2, bytes);
  flag.store(0);
  return 0;
}
int ncclCommSplit(void* comm, int color, int key, void** out, void*) {
  Comm* c = static_cast<Comm*>(comm);
  // everyone publishes (colour, key), then works out its group, its rank in it and the group's file name
  int* mine = reinterpret_cast<int*>(c->slots + (size_t)c->rank * kSlot);
  mine[0] = color; mine[1] = key;
  barrier(c);
  int rank = 0, world = 0;
  for (int r = 0; r < c->world; ++r) {
    const int* o = reinterpret_cast<const int*>(c->slots + (size_t)r * kSlot);
    if (o[0] != color) continue;
    ++world;
    if (o[1] < key || (o[1] == key && r < c->rank)) ++rank;
  }
  const int serial = c->sh->splits.load();
  barrier(c);
  if (c->rank == 0) c->sh->splits.fetch_add(1);
  Id id;
  std::memset(&id, 0, sizeof(id));
  std::snprintf(id.bytes, sizeof(id.bytes), "%.90s_s%d_c%d", c->name, serial, color);
  barrier(c);
  return ncclCommInitRank(out, world, id, rank);
}
// failure handling: the stand-in can be told to report an asynchronous error; an abort just lets go of the mapping
int ncclCommGetAsyncError(void*, int* err) {
  const char* v = std::getenv("XFT_FAKE_NCCL_ASYNC_ERROR");
  *err = v && *v == '1' ? 6 : 0;
  return 0;
}
int ncclCommAbort(void* comm) { return ncclCommDestroy(comm); }
const char* ncclGetErrorString(int rc) { return rc == 0 ? "ok" : rc == 2 ? "fake nccl: shared memory" : "fake nccl: unsupported call"; }
}

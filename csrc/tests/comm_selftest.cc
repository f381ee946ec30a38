// Host-only test of the thread-rank communicator (csrc/core/comm.cc): the CUDA runtime calls and the device sum that
// comm.cc makes are replaced by host stand-ins defined here, so the turn-taking protocol itself runs on a CPU box —
// sums, gathers, broadcasts, messages between neighbours and sub-group collectives over many rounds with 1 to 8 ranks,
// no two ranks ever between operations at once; a rank that leaves early, or ranks that wait for one another, make the
// others fail instead of waiting for ever.  Built with -fsanitize=thread by
// tests/test_cpp_runtime.py.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <cstdlib>
#include <thread>
#include <vector>
#include "comm.h"
extern "C" {
cudaError_t cudaDeviceSynchronize() { return cudaSuccess; }
cudaError_t cudaMemcpyAsync(void* d, const void* s, size_t n, cudaMemcpyKind, cudaStream_t) { std::memmove(d, s, n); return cudaSuccess; }
cudaError_t cudaMemcpy(void* d, const void* s, size_t n, cudaMemcpyKind) { std::memmove(d, s, n); return cudaSuccess; }
cudaError_t cudaStreamSynchronize(cudaStream_t) { return cudaSuccess; }
// XFT_STUB_STREAM_BUSY=1: a stream whose work never finishes (what a collective looks like when a rank is lost)
cudaError_t cudaStreamQuery(cudaStream_t) { const char* v = getenv("XFT_STUB_STREAM_BUSY"); return v && *v == '1' ? cudaErrorNotReady : cudaSuccess; }
cudaError_t cudaGetDeviceCount(int* n) { *n = 1; return cudaSuccess; }
cudaError_t cudaSetDevice(int) { return cudaSuccess; }
cudaError_t cudaMalloc(void** p, size_t n) { *p = malloc(n); return cudaSuccess; }
cudaError_t cudaFree(void* p) { free(p); return cudaSuccess; }
const char* cudaGetErrorString(cudaError_t) { return "stub"; }
// "bf16" sum on host: treat as uint16 counters for the test
int xft_sum_bf16(void* dst, const void* const* srcs, int nsrc, size_t n, cudaStream_t) {
  std::vector<unsigned short> acc(n, 0);
  for (int k = 0; k < nsrc; ++k) for (size_t i = 0; i < n; ++i) acc[i] += ((const unsigned short*)srcs[k])[i];
  std::memcpy(dst, acc.data(), n * 2);
  return 0;
}
}
// process-rank mode: `comm_selftest process <rank> <world> <id file>` — one of `world` processes; the communicator is the
// NCCL one of comm.cc, talking to the stand-in library named by XFT_NCCL_LIB (csrc/tests/fake_nccl.cc)
static int processRank(int rank, int world, const char* idFile) {
  try {
    auto c = xft::makeProcessCommunicator(rank, world, idFile);
    if (!c || c->rank() != rank || c->size() != world) throw std::runtime_error("bad communicator");
    // a host broadcast larger than the staging buffer (3 pieces)
    std::vector<unsigned char> big(2500000, (unsigned char)(rank == 0 ? 0 : 0xee));
    if (rank == 0) for (size_t i = 0; i < big.size(); ++i) big[i] = (unsigned char)(i * 7 + 3);
    c->broadcastHost(big.data(), big.size());
    for (size_t i = 0; i < big.size(); i += 9973) if (big[i] != (unsigned char)(i * 7 + 3)) throw std::runtime_error("bad broadcast");
    std::vector<float> in(5, (float)(rank + 1)), out(5 * world, -1.f);
    c->allGatherF32(in.data(), out.data(), 5, nullptr);
    for (int r = 0; r < world; ++r) if (out[r * 5 + 2] != (float)(r + 1)) throw std::runtime_error("bad gather");
    std::vector<unsigned short> h(33, (unsigned short)0x3f80);          // bf16 1.0
    c->allReduceBf16(h.data(), h.size(), nullptr);
    const unsigned short want[9] = {0, 0x3f80, 0x4000, 0x4040, 0x4080, 0x40a0, 0x40c0, 0x40e0, 0x4100};   // bf16 of 0..8
    if (h[32] != want[world]) throw std::runtime_error("bad sum");
    c->barrier();
    // a ring of messages (pipeline stage boundaries), a broadcast from the last rank, and pairs made by a split
    if (world > 1) {
      std::vector<unsigned short> msg(1000, (unsigned short)(100 + rank)), got(1000, 0);
      if (rank > 0) c->recvBf16(got.data(), got.size(), rank - 1, nullptr);
      if (rank + 1 < world) c->sendBf16(msg.data(), msg.size(), rank + 1, nullptr);
      if (rank > 0 && got[999] != (unsigned short)(100 + rank - 1)) throw std::runtime_error("bad message");
      long long v = rank == world - 1 ? 4242 : -1;
      c->broadcastHost(&v, sizeof(v), world - 1);
      if (v != 4242) throw std::runtime_error("bad broadcast from the last rank");
    }
    if (world == 4) {
      auto sub = c->split(rank / 2, rank % 2);
      if (sub->size() != 2 || sub->rank() != rank % 2) throw std::runtime_error("bad split");
      std::vector<unsigned short> one(8, (unsigned short)0x3f80);
      sub->allReduceBf16(one.data(), one.size(), nullptr);
      if (one[7] != 0x4000) throw std::runtime_error("bad sum in the sub-group");
      long long v = rank % 2 == 0 ? 1000 + rank / 2 : -1;
      sub->broadcastHost(&v, sizeof(v));
      if (v != 1000 + rank / 2) throw std::runtime_error("bad broadcast in the sub-group");
    }
    std::printf("rank %d of %d ok\n", rank, world);
    return 0;
  } catch (const std::exception& e) {
    std::printf("rank %d: %s\n", rank, e.what());
    return 1;
  }
}

int main(int argc, char** argv) {
  if (argc > 4 && std::string(argv[1]) == "process") return processRank(atoi(argv[2]), atoi(argv[3]), argv[4]);
  const int n = argc > 1 ? atoi(argv[1]) : 3;
  auto comms = xft::makeThreadCommunicators(n);
  std::vector<std::thread> th;
  std::vector<int> ok(n, 0);
  static int running = 0; static bool overlap = false;
  for (int r = 0; r < n; ++r) th.emplace_back([&, r] {
    auto c = comms[r];
    try {
      c->begin();
      for (int it = 0; it < 200; ++it) {
        // only one rank may be between collectives at a time
        if (__sync_add_and_fetch(&running, 1) != 1) overlap = true;
        std::vector<unsigned short> buf(16, (unsigned short)(r + 1 + it));
        std::this_thread::yield();
        __sync_sub_and_fetch(&running, 1);
        c->allReduceBf16(buf.data(), 16, nullptr);
        unsigned short want = 0; for (int k = 0; k < n; ++k) want += (unsigned short)(k + 1 + it);
        if (buf[3] != want) throw std::runtime_error("bad sum");
        std::vector<float> in(4, (float)r), out(4 * n, -1.f);
        c->allGatherF32(in.data(), out.data(), 4, nullptr);
        for (int k = 0; k < n; ++k) if (out[k * 4 + 1] != (float)k) throw std::runtime_error("bad gather");
        long long v = r == 0 ? 777 + it : -1;
        c->broadcastHost(&v, sizeof(v));
        if (v != 777 + it) throw std::runtime_error("bad broadcast");
        c->barrier();
        // a pipeline: a message from every rank to the next one, then a broadcast from the last rank
        std::vector<unsigned short> msg(32, (unsigned short)(r * 3 + it)), got(32, 0);
        if (r > 0) c->recvBf16(got.data(), 32, r - 1, nullptr);
        if (r + 1 < n) c->sendBf16(msg.data(), 32, r + 1, nullptr);
        if (r > 0 && got[31] != (unsigned short)((r - 1) * 3 + it)) throw std::runtime_error("bad message");
        long long w = r == n - 1 ? 31 + it : -1;
        c->broadcastHost(&w, sizeof(w), n - 1);
        if (w != 31 + it) throw std::runtime_error("bad broadcast from the last rank");
      }
      if (n >= 4 && n % 2 == 0) {
        // sub-groups (the tensor-parallel group of a pipeline stage): pairs {0,1}, {2,3}, ... sum among themselves, and
        // a message crosses from each pair to the next while the world communicator stays usable
        auto sub = c->split(r / 2, r % 2);
        if (sub->size() != 2 || sub->rank() != r % 2) throw std::runtime_error("bad split");
        for (int it = 0; it < 50; ++it) {
          std::vector<unsigned short> buf(8, (unsigned short)(r + it));
          if (r >= 2) c->recvBf16(buf.data(), 8, r - 2, nullptr);
          sub->allReduceBf16(buf.data(), 8, nullptr);
          if (r + 2 < n) c->sendBf16(buf.data(), 8, r + 2, nullptr);
          c->barrier();
        }
      }
      ok[r] = 1;
    } catch (const std::exception& e) { std::printf("rank %d: %s\n", r, e.what()); }
    c->end();
  });
  for (auto& t : th) t.join();
  int good = 0; for (int r = 0; r < n; ++r) good += ok[r];
  std::printf("%d/%d ranks ok, overlap=%d\n", good, n, (int)overlap);
  // a rank that leaves early: the others must fail, not hang
  auto c2 = xft::makeThreadCommunicators(2);
  std::thread a([&] { try { c2[0]->begin(); int x = 0; c2[0]->broadcastHost(&x, 4); c2[0]->broadcastHost(&x, 4); std::printf("rank0 unexpectedly passed\n"); } catch (const std::exception& e) { std::printf("rank0 failed as expected: %s\n", e.what()); } c2[0]->end(); });
  std::thread b([&] { c2[1]->begin(); int x = 0; c2[1]->broadcastHost(&x, 4); c2[1]->end(); });
  a.join(); b.join();
  // two ranks that wait for a message from each other: both must fail, not hang
  auto c3 = xft::makeThreadCommunicators(2);
  int failed = 0;
  auto waits = [&](int r) {
    try { c3[r]->begin(); unsigned short x[4]; c3[r]->recvBf16(x, 4, 1 - r, nullptr); std::printf("rank%d unexpectedly received\n", r); }
    catch (const std::exception& e) { __sync_add_and_fetch(&failed, 1); std::printf("rank%d failed as expected: %s\n", r, e.what()); }
    c3[r]->end();
  };
  std::thread d(waits, 0), e(waits, 1);
  d.join(); e.join();
  return good == n && !overlap && failed == 2 ? 0 : 1;
}

#include "comm.h"

#include <dlfcn.h>

#include <algorithm>

#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <mutex>
#include <stdexcept>
#include <thread>

#include "kernels_c.h"

namespace xft {

namespace {

void cudaOk(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA error in ") + what + ": " + cudaGetErrorString(e));
}

int envInt(const char* name, int def) {
  const char* v = std::getenv(name);
  return v && *v ? std::atoi(v) : def;
}

// ------------------------------------------------------------------------------------------------ thread ranks
// Shared state of one group of thread ranks.  `turn` is the rank that may run; everyone else sleeps.  A collective is
// entered by the ranks in turn order; each leaves its arguments and hands the turn on; the last one to arrive performs
// the operation for all (after a device-wide synchronise, so every rank's producer kernels are complete), bumps
// `epoch` and gives the turn to the first rank.
struct ThreadGroup {
  std::mutex mu;
  std::condition_variable cv;
  int n = 0, turn = 0, arrived = 0, alive = 0;
  long long epoch = 0;
  bool broken = false;                   // a rank left in the middle of the program
  std::vector<char> gone;
  std::vector<void*> a, b;               // per-rank arguments of the collective in flight
  std::vector<cudaStream_t> streams;

  int nextAlive(int r) const {
    for (int i = 1; i <= n; ++i) { const int c = (r + i) % n; if (!gone[c]) return c; }
    return r;
  }
};

class ThreadComm : public Communicator {
public:
  ThreadComm(std::shared_ptr<ThreadGroup> g, int rank) : g_(std::move(g)), rank_(rank) {}
  ~ThreadComm() override { end(); }
  int rank() const override { return rank_; }
  int size() const override { return g_->n; }

  void begin() override {
    std::unique_lock<std::mutex> lk(g_->mu);
    g_->cv.wait(lk, [&] { return g_->turn == rank_ || g_->broken; });
    started_ = true;
  }

  void end() override {
    std::unique_lock<std::mutex> lk(g_->mu);
    if (ended_) return;
    ended_ = true;
    g_->gone[rank_] = 1;
    g_->alive--;
    if (g_->arrived > 0) g_->broken = true;          // the others are inside a collective this rank will never join
    if (g_->turn == rank_) g_->turn = g_->nextAlive(rank_);
    g_->cv.notify_all();
  }

  void allReduceBf16(void* buf, size_t n, cudaStream_t st) override {
    collective(buf, nullptr, st, [&](ThreadGroup& g) {
      std::vector<const void*> srcs(g.a.begin(), g.a.end());
      // the sum lands in rank 0's buffer, then every other rank's buffer receives a copy
      if (xft_sum_bf16(g.a[0], srcs.data(), g.n, n, st) != 0) throw std::runtime_error("xft_sum_bf16 failed");
      for (int r = 1; r < g.n; ++r) cudaOk(cudaMemcpyAsync(g.a[r], g.a[0], n * 2, cudaMemcpyDeviceToDevice, st), "all-reduce copy");
    });
  }

  void allGatherF32(const float* in, float* out, size_t n, cudaStream_t st) override {
    collective(const_cast<float*>(in), out, st, [&](ThreadGroup& g) {
      for (int dst = 0; dst < g.n; ++dst)
        for (int src = 0; src < g.n; ++src)
          cudaOk(cudaMemcpyAsync(static_cast<float*>(g.b[dst]) + (size_t)src * n, g.a[src], n * 4, cudaMemcpyDeviceToDevice, st),
                 "all-gather copy");
    });
  }

  void broadcastHost(void* data, size_t bytes) override {
    collective(data, nullptr, nullptr, [&](ThreadGroup& g) {
      for (int r = 1; r < g.n; ++r) std::memcpy(g.a[r], g.a[0], bytes);
    });
  }

  void barrier() override { collective(nullptr, nullptr, nullptr, [](ThreadGroup&) {}); }

private:
  template <class Op>
  void collective(void* a, void* b, cudaStream_t st, Op op) {
    std::unique_lock<std::mutex> lk(g_->mu);
    if (!started_ || g_->turn != rank_) throw std::runtime_error("thread rank ran out of turn (begin() not called?)");
    if (g_->broken || g_->alive != g_->n) throw std::runtime_error("a tensor-parallel rank has left");
    g_->a[rank_] = a; g_->b[rank_] = b; g_->streams[rank_] = st;
    const long long my = g_->epoch;
    if (++g_->arrived == g_->n) {
      // every rank's work up to here is on the device queue: wait for all of it, do the operation, wait for that too
      try {
        cudaOk(cudaDeviceSynchronize(), "collective (before)");
        op(*g_);
        cudaOk(cudaDeviceSynchronize(), "collective (after)");
      } catch (...) {
        g_->broken = true;               // the sleeping ranks wake up and fail too instead of waiting for ever
        g_->cv.notify_all();
        throw;
      }
      g_->arrived = 0;
      g_->epoch++;
      g_->turn = g_->nextAlive(g_->n - 1);      // the first rank runs first again
      g_->cv.notify_all();
      if (g_->turn != rank_) g_->cv.wait(lk, [&] { return g_->turn == rank_ || g_->broken; });
    } else {
      g_->turn = g_->nextAlive(rank_);
      g_->cv.notify_all();
      g_->cv.wait(lk, [&] { return (g_->epoch != my && g_->turn == rank_) || g_->broken; });
    }
    if (g_->broken) throw std::runtime_error("a tensor-parallel rank has left");
  }

  std::shared_ptr<ThreadGroup> g_;
  int rank_;
  bool started_ = false, ended_ = false;
};

}  // namespace

std::vector<std::shared_ptr<Communicator>> makeThreadCommunicators(int n) {
  if (n < 1 || n > 8) throw std::runtime_error("thread ranks: 1 to 8");
  auto g = std::make_shared<ThreadGroup>();
  g->n = g->alive = n;
  g->gone.assign(n, 0);
  g->a.assign(n, nullptr); g->b.assign(n, nullptr); g->streams.assign(n, nullptr);
  std::vector<std::shared_ptr<Communicator>> out;
  for (int r = 0; r < n; ++r) out.push_back(std::make_shared<ThreadComm>(g, r));
  return out;
}

std::pair<int, int> rankFromEnv() {
  // SINGLE_INSTANCE=1 (src/utils/environment.h): this process is a model of its own whatever launched it
  if (envInt("SINGLE_INSTANCE", 0) != 0) return {0, 1};
  static const char* pairs[][2] = {{"RANK", "WORLD_SIZE"}, {"OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE"}, {"PMI_RANK", "PMI_SIZE"}};
  for (auto& p : pairs) {
    const char* r = std::getenv(p[0]);
    const char* w = std::getenv(p[1]);
    if (r && w && *r && *w && std::atoi(w) > 0) return {std::atoi(r), std::atoi(w)};
  }
  return {0, 1};
}

// ------------------------------------------------------------------------------------------------ process ranks
namespace {

// The handful of NCCL entry points used, resolved at run time (ncclUniqueId is 128 opaque bytes; ncclDataType_t:
// ncclUint8 = 1, ncclFloat32 = 7, ncclBfloat16 = 9; ncclRedOp_t: ncclSum = 0 — stable across NCCL 2.x).
struct NcclId { char bytes[128]; };
struct NcclApi {
  void* lib = nullptr;
  int (*GetUniqueId)(NcclId*) = nullptr;
  int (*CommInitRank)(void**, int, NcclId, int) = nullptr;
  int (*CommDestroy)(void*) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;

  static NcclApi& get() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
      const char* override_path = std::getenv("XFT_NCCL_LIB");
      const char* names[] = {override_path, "libnccl.so.2", "libnccl.so"};
      for (const char* nm : names) {
        if (!nm || !*nm) continue;
        api.lib = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
        if (api.lib) break;
      }
      if (!api.lib) return;
      auto sym = [&](const char* s) { return dlsym(api.lib, s); };
      api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
      api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
      api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
      api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
      api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
      api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(sym("ncclBroadcast"));
      api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    });
    return api;
  }
  bool ok() const { return lib && GetUniqueId && CommInitRank && CommDestroy && AllReduce && AllGather && Broadcast; }
};

class NcclComm : public Communicator {
public:
  NcclComm(int rank, int world, const std::string& idFile) : rank_(rank), world_(world) {
    NcclApi& api = NcclApi::get();
    if (!api.ok()) throw std::runtime_error("tensor-parallel ranks need NCCL: libnccl.so.2 could not be loaded (XFT_NCCL_LIB names another file)");
    // one process per GPU: local rank from the launcher, else rank modulo the visible devices
    int ndev = 0;
    cudaOk(cudaGetDeviceCount(&ndev), "cudaGetDeviceCount");
    if (ndev < 1) throw std::runtime_error("no CUDA device");
    int local = envInt("LOCAL_RANK", envInt("OMPI_COMM_WORLD_LOCAL_RANK", envInt("MPI_LOCALRANKID", rank)));
    cudaOk(cudaSetDevice(local % ndev), "cudaSetDevice");
    std::string path = idFile;
    if (path.empty()) {
      const char* f = std::getenv("XFT_COMM_ID_FILE");
      path = f && *f ? f : "/tmp/xft_nccl_id." + std::to_string(envInt("MASTER_PORT", 0));
    }
    NcclId id;
    std::memset(&id, 0, sizeof(id));
    const std::string ready = path + ".ready";
    if (rank == 0) {
      check(api.GetUniqueId(&id), "ncclGetUniqueId");
      std::remove(ready.c_str());
      { std::ofstream f(path, std::ios::binary | std::ios::trunc); f.write(id.bytes, sizeof(id.bytes)); }
      { std::ofstream f(ready); f << "1"; }                    // written after the id: readers never see half an id
    } else {
      const int limit = envInt("XFT_DIST_TIMEOUT_S", 120);
      const auto t0 = std::chrono::steady_clock::now();
      for (;;) {
        std::ifstream r(ready);
        if (r.good()) {
          std::ifstream f(path, std::ios::binary);
          f.read(id.bytes, sizeof(id.bytes));
          if (f.gcount() == (std::streamsize)sizeof(id.bytes)) break;
        }
        if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > limit)
          throw std::runtime_error("rank 0's NCCL id did not arrive in " + path + " within " + std::to_string(limit) + " s");
        std::this_thread::sleep_for(std::chrono::milliseconds(50));
      }
    }
    check(api.CommInitRank(&comm_, world, id, rank), "ncclCommInitRank");
    cudaOk(cudaMalloc(&stage_, kStage), "cudaMalloc (staging)");
    barrier();
    if (rank == 0) { std::remove(ready.c_str()); std::remove(path.c_str()); }
  }
  ~NcclComm() override {
    if (stage_) cudaFree(stage_);
    if (comm_) NcclApi::get().CommDestroy(comm_);
  }
  int rank() const override { return rank_; }
  int size() const override { return world_; }
  void allReduceBf16(void* buf, size_t n, cudaStream_t st) override {
    check(NcclApi::get().AllReduce(buf, buf, n, 9 /* bf16 */, 0 /* sum */, comm_, st), "ncclAllReduce");
  }
  void allGatherF32(const float* in, float* out, size_t n, cudaStream_t st) override {
    check(NcclApi::get().AllGather(in, out, n, 7 /* fp32 */, comm_, st), "ncclAllGather");
  }
  void broadcastHost(void* data, size_t bytes) override {
    // through a device staging buffer, in pieces
    for (size_t off = 0; off < bytes; off += kStage) {
      const size_t n = std::min(kStage, bytes - off);
      if (rank_ == 0) cudaOk(cudaMemcpy(stage_, static_cast<char*>(data) + off, n, cudaMemcpyHostToDevice), "broadcast (stage in)");
      check(NcclApi::get().Broadcast(stage_, stage_, n, 1 /* uint8 */, 0, comm_, nullptr), "ncclBroadcast");
      cudaOk(cudaStreamSynchronize(nullptr), "broadcast");
      if (rank_ != 0) cudaOk(cudaMemcpy(static_cast<char*>(data) + off, stage_, n, cudaMemcpyDeviceToHost), "broadcast (stage out)");
    }
  }
  void barrier() override {
    check(NcclApi::get().AllReduce(stage_, stage_, 1, 7, 0, comm_, nullptr), "barrier");
    cudaOk(cudaStreamSynchronize(nullptr), "barrier");
  }

private:
  void check(int rc, const char* what) {
    if (rc == 0) return;
    NcclApi& api = NcclApi::get();
    throw std::runtime_error(std::string("NCCL error in ") + what + ": " + (api.GetErrorString ? api.GetErrorString(rc) : std::to_string(rc)));
  }
  static constexpr size_t kStage = 1 << 20;
  int rank_, world_;
  void* comm_ = nullptr;
  void* stage_ = nullptr;
};

}  // namespace

std::shared_ptr<Communicator> makeProcessCommunicator(int rank, int world, const std::string& idFile) {
  if (world < 2) return nullptr;
  if (rank < 0 || rank >= world) throw std::runtime_error("bad rank " + std::to_string(rank) + " of " + std::to_string(world));
  return std::make_shared<NcclComm>(rank, world, idFile);
}

}  // namespace xft

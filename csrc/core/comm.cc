#include "comm.h"

#include <dlfcn.h>

#include <algorithm>

#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <functional>
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

}  // namespace

void Communicator::waitStream(cudaStream_t st) { cudaOk(cudaStreamSynchronize(st), "cudaStreamSynchronize"); }

namespace {

// ------------------------------------------------------------------------------------------------ thread ranks
// Shared by every thread rank of one world: `turn` is the rank that may run, everyone else sleeps.  A rank that reaches
// an operation it cannot finish alone leaves its arguments and hands the turn to the next rank; when the turn comes
// back and the operation is still open, it hands the turn on again.  Whoever completes an operation (the last arriver of
// a collective, the receiver of a message) does the work — after a device-wide synchronise, so every rank's producer
// kernels are complete — and keeps running.  When the turn goes round with nobody able to go on, the program has
// deadlocked (a rank waits for an operation its partner never reaches): every waiting rank fails.
struct Sched {
  std::mutex mu;
  std::condition_variable cv;
  int n = 0, turn = 0, stalls = 0;
  bool broken = false;
  std::vector<char> gone;
  struct Mail { const void* buf = nullptr; size_t n = 0; bool posted = false; };
  std::vector<Mail> mail;                // [source * n + destination], world ranks

  int nextAlive(int r) const {
    for (int i = 1; i <= n; ++i) { const int c = (r + i) % n; if (!gone[c]) return c; }
    return r;
  }
};

// One group of ranks that runs collectives together: the world, or what split() made of it
struct Coll {
  std::vector<int> members;              // world ranks, in group order
  int arrived = 0;
  long long epoch = 0;
  std::vector<void*> a, b;               // per-member arguments of the collective in flight
  std::vector<int> color, key;           // split(): what each member asked for ...
  std::vector<std::shared_ptr<Coll>> made;   // ... and the group it got

  explicit Coll(std::vector<int> m) : members(std::move(m)) {
    const size_t n = members.size();
    a.assign(n, nullptr); b.assign(n, nullptr); color.assign(n, 0); key.assign(n, 0); made.assign(n, nullptr);
  }
};

class ThreadComm : public Communicator {
public:
  ThreadComm(std::shared_ptr<Sched> s, std::shared_ptr<Coll> c, int worldRank, bool isWorld)
      : s_(std::move(s)), c_(std::move(c)), me_(worldRank), isWorld_(isWorld), started_(!isWorld) {
    idx_ = (int)(std::find(c_->members.begin(), c_->members.end(), me_) - c_->members.begin());
  }
  ~ThreadComm() override { end(); }
  int rank() const override { return idx_; }
  int size() const override { return (int)c_->members.size(); }

  void begin() override {
    if (!isWorld_) return;
    std::unique_lock<std::mutex> lk(s_->mu);
    s_->cv.wait(lk, [&] { return s_->turn == me_ || s_->broken; });
    started_ = true;
  }

  // the rank leaves the world (a sub-group's end() is nothing: its ranks leave through the world communicator)
  void end() override {
    if (!isWorld_) return;
    std::unique_lock<std::mutex> lk(s_->mu);
    if (ended_) return;
    ended_ = true;
    s_->gone[me_] = 1;
    if (s_->turn == me_) s_->turn = s_->nextAlive(me_);
    s_->cv.notify_all();
  }

  void allReduceBf16(void* buf, size_t n, cudaStream_t st) override {
    collective(buf, nullptr, [&](Coll& g) {
      std::vector<const void*> srcs(g.a.begin(), g.a.end());
      // the sum lands in the first member's buffer, then every other member's buffer receives a copy
      if (xft_sum_bf16(g.a[0], srcs.data(), (int)g.members.size(), n, st) != 0) throw std::runtime_error("xft_sum_bf16 failed");
      for (size_t r = 1; r < g.members.size(); ++r)
        cudaOk(cudaMemcpyAsync(g.a[r], g.a[0], n * 2, cudaMemcpyDeviceToDevice, st), "all-reduce copy");
    });
  }

  void allGatherF32(const float* in, float* out, size_t n, cudaStream_t st) override {
    collective(const_cast<float*>(in), out, [&](Coll& g) {
      for (size_t dst = 0; dst < g.members.size(); ++dst)
        for (size_t src = 0; src < g.members.size(); ++src)
          cudaOk(cudaMemcpyAsync(static_cast<float*>(g.b[dst]) + src * n, g.a[src], n * 4, cudaMemcpyDeviceToDevice, st),
                 "all-gather copy");
    });
  }

  void broadcastHost(void* data, size_t bytes, int root) override {
    if (root < 0 || root >= size()) throw std::runtime_error("broadcast: bad root");
    collective(data, nullptr, [&](Coll& g) {
      for (size_t r = 0; r < g.members.size(); ++r)
        if ((int)r != root) std::memcpy(g.a[r], g.a[root], bytes);
    });
  }

  void barrier() override { collective(nullptr, nullptr, [](Coll&) {}); }

  void sendBf16(const void* buf, size_t n, int peer, cudaStream_t) override {
    std::unique_lock<std::mutex> lk(s_->mu);
    const int to = enter(peer);
    Sched::Mail& m = s_->mail[(size_t)me_ * s_->n + to];
    if (m.posted) throw std::runtime_error("send: the previous message to this rank is still waiting");
    m.buf = buf; m.n = n; m.posted = true;
    s_->stalls = 0;
    yieldUntil(lk, [&] { if (s_->gone[to]) throw std::runtime_error("a rank has left"); return !m.posted; });
  }

  void recvBf16(void* buf, size_t n, int peer, cudaStream_t st) override {
    std::unique_lock<std::mutex> lk(s_->mu);
    const int from = enter(peer);
    Sched::Mail& m = s_->mail[(size_t)from * s_->n + me_];
    yieldUntil(lk, [&] { if (!m.posted && s_->gone[from]) throw std::runtime_error("a rank has left"); return m.posted; });
    try {
      if (m.n != n) throw std::runtime_error("receive: the sender's message has another size");
      cudaOk(cudaDeviceSynchronize(), "receive (before)");
      cudaOk(cudaMemcpyAsync(buf, m.buf, n * 2, cudaMemcpyDeviceToDevice, st), "receive copy");
      cudaOk(cudaDeviceSynchronize(), "receive (after)");
    } catch (...) {
      s_->broken = true;
      s_->cv.notify_all();
      throw;
    }
    m.posted = false;                    // the sender goes on when its turn comes
    s_->stalls = 0;
  }

  std::shared_ptr<Communicator> split(int color, int key) override {
    {
      std::unique_lock<std::mutex> lk(s_->mu);
      c_->color[idx_] = color; c_->key[idx_] = key;
    }
    collective(nullptr, nullptr, [](Coll& g) {
      const int n = (int)g.members.size();
      std::vector<char> done(n, 0);
      for (int i = 0; i < n; ++i) {
        if (done[i]) continue;
        std::vector<int> grp;
        for (int j = i; j < n; ++j) if (g.color[j] == g.color[i]) grp.push_back(j);
        std::stable_sort(grp.begin(), grp.end(), [&](int x, int y) { return g.key[x] < g.key[y]; });
        std::vector<int> world;
        for (int j : grp) world.push_back(g.members[j]);
        auto made = std::make_shared<Coll>(world);
        for (int j : grp) { g.made[j] = made; done[j] = 1; }
      }
    });
    std::unique_lock<std::mutex> lk(s_->mu);
    return std::make_shared<ThreadComm>(s_, c_->made[idx_], me_, false);
  }

private:
  // common entry checks of an operation (lock held): this rank has the turn, the world is whole; returns the world rank of
  // group member `peer`
  int enter(int peer) {
    if (!started_ || s_->turn != me_) throw std::runtime_error("thread rank ran out of turn (begin() not called?)");
    if (s_->broken) throw std::runtime_error("a tensor-parallel rank has left");
    if (peer < 0 || peer >= size() || c_->members[peer] == me_) throw std::runtime_error("bad peer rank");
    return c_->members[peer];
  }
  bool membersAlive() const {
    for (int m : c_->members) if (s_->gone[m]) return false;
    return true;
  }

  // Give the turn away until `ready()` holds and the turn is back (lock held on entry and on return).
  template <class Ready>
  void yieldUntil(std::unique_lock<std::mutex>& lk, Ready ready) {
    Sched& s = *s_;
    for (;;) {
      if (s.broken) throw std::runtime_error("a tensor-parallel rank has left");
      if (s.turn == me_) {
        if (ready()) { s.stalls = 0; return; }
        const int next = s.nextAlive(me_);
        if (next == me_ || ++s.stalls > 4 * s.n + 4) {
          s.broken = true;               // nobody can go on: the sleeping ranks wake up and fail too
          s.cv.notify_all();
          throw std::runtime_error("thread ranks are waiting for one another (an operation no partner reaches)");
        }
        s.turn = next;
        s.cv.notify_all();
      }
      s.cv.wait(lk, [&] { return s.turn == me_ || s.broken; });
    }
  }

  template <class Op>
  void collective(void* a, void* b, Op op) {
    std::unique_lock<std::mutex> lk(s_->mu);
    if (!started_ || s_->turn != me_) throw std::runtime_error("thread rank ran out of turn (begin() not called?)");
    if (s_->broken || !membersAlive()) throw std::runtime_error("a tensor-parallel rank has left");
    Coll& g = *c_;
    g.a[idx_] = a; g.b[idx_] = b;
    s_->stalls = 0;
    const long long my = g.epoch;
    if (++g.arrived == (int)g.members.size()) {
      // every member's work up to here is on the device queue: wait for all of it, do the operation, wait for that too
      try {
        cudaOk(cudaDeviceSynchronize(), "collective (before)");
        op(g);
        cudaOk(cudaDeviceSynchronize(), "collective (after)");
      } catch (...) {
        s_->broken = true;               // the sleeping ranks wake up and fail too instead of waiting for ever
        s_->cv.notify_all();
        throw;
      }
      g.arrived = 0;
      g.epoch++;
      return;                            // the others go on as the turn reaches them
    }
    yieldUntil(lk, [&] {
      if (g.epoch == my && !membersAlive()) throw std::runtime_error("a tensor-parallel rank has left");
      return g.epoch != my;
    });
  }

  std::shared_ptr<Sched> s_;
  std::shared_ptr<Coll> c_;
  int me_, idx_ = 0;
  bool isWorld_, started_, ended_ = false;
};

}  // namespace

std::vector<std::shared_ptr<Communicator>> makeThreadCommunicators(int n) {
  if (n < 1 || n > 8) throw std::runtime_error("thread ranks: 1 to 8");
  auto s = std::make_shared<Sched>();
  s->n = n;
  s->gone.assign(n, 0);
  s->mail.assign((size_t)n * n, Sched::Mail());
  std::vector<int> all(n);
  for (int r = 0; r < n; ++r) all[r] = r;
  auto world = std::make_shared<Coll>(all);
  std::vector<std::shared_ptr<Communicator>> out;
  for (int r = 0; r < n; ++r) out.push_back(std::make_shared<ThreadComm>(s, world, r, true));
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
  int (*Send)(const void*, size_t, int, int, void*, cudaStream_t) = nullptr;              // pipeline stages only
  int (*Recv)(void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*CommSplit)(void*, int, int, void**, void*) = nullptr;                             // NCCL 2.18 and later
  int (*CommAbort)(void*) = nullptr;                                                      // failure handling
  int (*CommGetAsyncError)(void*, int*) = nullptr;
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
      api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
      api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
      api.CommSplit = reinterpret_cast<decltype(api.CommSplit)>(sym("ncclCommSplit"));
      api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
      api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
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
  // a communicator NCCL made out of another one (split)
  NcclComm(void* comm, int rank, int world) : rank_(rank), world_(world), comm_(comm) {
    cudaOk(cudaMalloc(&stage_, kStage), "cudaMalloc (staging)");
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
  void broadcastHost(void* data, size_t bytes, int root) override {
    // through a device staging buffer, in pieces
    for (size_t off = 0; off < bytes; off += kStage) {
      const size_t n = std::min(kStage, bytes - off);
      if (rank_ == root) cudaOk(cudaMemcpy(stage_, static_cast<char*>(data) + off, n, cudaMemcpyHostToDevice), "broadcast (stage in)");
      check(NcclApi::get().Broadcast(stage_, stage_, n, 1 /* uint8 */, root, comm_, nullptr), "ncclBroadcast");
      waitStream(nullptr);
      if (rank_ != root) cudaOk(cudaMemcpy(static_cast<char*>(data) + off, stage_, n, cudaMemcpyDeviceToHost), "broadcast (stage out)");
    }
  }
  void sendBf16(const void* buf, size_t n, int peer, cudaStream_t st) override {
    NcclApi& api = NcclApi::get();
    if (!api.Send) throw std::runtime_error("this NCCL library has no ncclSend");
    check(api.Send(buf, n, 9 /* bf16 */, peer, comm_, st), "ncclSend");
  }
  void recvBf16(void* buf, size_t n, int peer, cudaStream_t st) override {
    NcclApi& api = NcclApi::get();
    if (!api.Recv) throw std::runtime_error("this NCCL library has no ncclRecv");
    check(api.Recv(buf, n, 9 /* bf16 */, peer, comm_, st), "ncclRecv");
  }
  std::shared_ptr<Communicator> split(int color, int key) override {
    NcclApi& api = NcclApi::get();
    if (!api.CommSplit) throw std::runtime_error("pipeline stages with tensor-parallel groups need ncclCommSplit (NCCL 2.18 or later)");
    // rank and size of the new communicator: every rank tells the others its colour and key
    std::vector<float> mine = {(float)color, (float)key}, all((size_t)2 * world_);
    float* dev = static_cast<float*>(stage_);
    cudaOk(cudaMemcpy(dev, mine.data(), 8, cudaMemcpyHostToDevice), "split");
    check(api.AllGather(dev, dev + 2, 2, 7 /* fp32 */, comm_, nullptr), "ncclAllGather (split)");
    waitStream(nullptr);
    cudaOk(cudaMemcpy(all.data(), dev + 2, all.size() * 4, cudaMemcpyDeviceToHost), "split");
    int newRank = 0, newSize = 0;
    for (int r = 0; r < world_; ++r) {
      if ((int)all[2 * r] != color) continue;
      ++newSize;
      const int k = (int)all[2 * r + 1];
      if (k < key || (k == key && r < rank_)) ++newRank;
    }
    void* sub = nullptr;
    check(api.CommSplit(comm_, color, key, &sub, nullptr), "ncclCommSplit");
    return std::make_shared<NcclComm>(sub, newRank, newSize);
  }
  void barrier() override {
    check(NcclApi::get().AllReduce(stage_, stage_, 1, 7, 0, comm_, nullptr), "barrier");
    waitStream(nullptr);
  }

  // cudaStreamSynchronize with a limit: polls the stream (busily at first — a decode step's collectives take
  // microseconds — then with short sleeps) and NCCL's asynchronous error state
  void waitStream(cudaStream_t st) override {
    NcclApi& api = NcclApi::get();
    const double limit = (double)envInt("XFT_DIST_TIMEOUT_S", 1800);
    const auto t0 = std::chrono::steady_clock::now();
    for (long spin = 0;; ++spin) {
      const cudaError_t q = cudaStreamQuery(st);
      if (q == cudaSuccess) return;
      if (q != cudaErrorNotReady) cudaOk(q, "cudaStreamQuery");
      int async = 0;
      const bool bad = comm_ && api.CommGetAsyncError && (spin & 255) == 255 && api.CommGetAsyncError(comm_, &async) == 0 && async != 0;
      const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
      if (bad || waited > limit) {
        // give the communicator up: its kernels leave the device, so the process can report and end
        if (comm_ && api.CommAbort) api.CommAbort(comm_);
        comm_ = nullptr;
        throw std::runtime_error(bad ? std::string("NCCL reported an asynchronous error (a rank was lost?): ") +
                                           (api.GetErrorString ? api.GetErrorString(async) : std::to_string(async))
                                     : "a collective did not finish within " + std::to_string((long)limit) +
                                           " s (XFT_DIST_TIMEOUT_S): a rank was lost");
      }
      if (waited > 2e-3) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
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

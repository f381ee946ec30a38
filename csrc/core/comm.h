// Communication between the ranks of the C++ engine (reference: src/utils/messenger.h — reduceAdd, broadcast,
// allgatherv, the row communicator of one pipeline stage — and src/comm_helper/comm_helper.cpp; stage boundaries:
// src/models/common_decoder.h:389-391,497-498).
//
// Two implementations of one small interface:
//   * process ranks (one process per GPU, launched by mpirun / torchrun): NCCL, opened with dlopen at first use so
//     that a single-GPU program has no dependency on it; the unique id travels through a file that rank 0 writes;
//   * thread ranks (all ranks are threads of ONE process on ONE GPU): for tests and for checking a sharded load without
//     a second GPU.  The threads take turns — a rank runs alone until it reaches an operation that needs another rank
//     (a collective of its group, a send or a receive), then hands the turn on; whoever completes the operation does
//     the reduction or the copies — so kernels of different ranks never wait on one another on the device and
//     host-side caches are never touched by two threads at once.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <memory>
#include <string>
#include <vector>

namespace xft {

class Communicator {
public:
  virtual ~Communicator() {}
  virtual int rank() const = 0;
  virtual int size() const = 0;
  // buf[i] <- sum over ranks of buf[i], n bf16 values, ordered on `st`
  virtual void allReduceBf16(void* buf, size_t n, cudaStream_t st) = 0;
  // out[r * n + i] <- in[i] of rank r, n fp32 values per rank, ordered on `st`
  virtual void allGatherF32(const float* in, float* out, size_t n, cudaStream_t st) = 0;
  // host bytes of rank `root` -> every rank
  virtual void broadcastHost(void* data, size_t bytes, int root = 0) = 0;
  virtual void barrier() = 0;
  // n bf16 values to / from rank `peer` of this communicator, ordered on `st` (pipeline stage boundaries)
  virtual void sendBf16(const void* buf, size_t n, int peer, cudaStream_t st) = 0;
  virtual void recvBf16(void* buf, size_t n, int peer, cudaStream_t st) = 0;
  // Collective over all ranks: the communicator of the ranks that pass the same `color`, ordered by `key` (the tensor-
  // parallel group of one pipeline stage).
  virtual std::shared_ptr<Communicator> split(int color, int key) = 0;
  // Wait until the work queued on `st` is done.  Process ranks bound the wait: when a collective does not finish within
  // XFT_DIST_TIMEOUT_S seconds (a rank was lost) or NCCL reports an asynchronous error, the communicator is aborted and
  // std::runtime_error is thrown instead of waiting for ever.
  virtual void waitStream(cudaStream_t st);
  // thread ranks: wait for this rank's first turn / give the turn up for good (no-ops for process ranks)
  virtual void begin() {}
  virtual void end() {}
};

// Rank and world size of this process from the launcher's environment (RANK / WORLD_SIZE of torchrun,
// OMPI_COMM_WORLD_RANK / _SIZE of Open MPI, PMI_RANK / PMI_SIZE of MPICH); {0, 1} when none is set or when
// SINGLE_INSTANCE=1 asks for a model per process.
std::pair<int, int> rankFromEnv();

// NCCL communicator of `world` process ranks.  `idFile`: path through which rank 0 hands the unique id to the others
// (default: XFT_COMM_ID_FILE, else /tmp/xft_nccl_id.<MASTER_PORT or 0>).  Throws std::runtime_error when NCCL cannot be
// loaded or the id does not arrive within XFT_DIST_TIMEOUT_S seconds (default 120).
std::shared_ptr<Communicator> makeProcessCommunicator(int rank, int world, const std::string& idFile = "");

// `n` communicators whose ranks are threads of this process; hand communicator r to thread r.
std::vector<std::shared_ptr<Communicator>> makeThreadCommunicators(int n);

}  // namespace xft

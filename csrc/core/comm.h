// Communication between the tensor-parallel ranks of the C++ engine (reference: src/utils/messenger.h — reduceAdd,
// broadcast, allgatherv over oneCCL / shared memory — and src/comm_helper/comm_helper.cpp).
//
// Two implementations of one small interface:
//   * process ranks (one process per GPU, launched by mpirun / torchrun): NCCL, opened with dlopen at first use so
//     that a single-GPU program has no dependency on it; the unique id travels through a file that rank 0 writes;
//   * thread ranks (all ranks are threads of ONE process on ONE GPU): for tests and for checking a sharded load without
//     a second GPU.  The threads take turns — a rank runs alone until it reaches a collective, then hands over; the
//     last arriver does the reduction or the copies and wakes rank 0 — so kernels of different ranks never wait on
//     one another on the device and host-side caches are never touched by two threads at once.
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
  // host bytes of rank 0 -> every rank
  virtual void broadcastHost(void* data, size_t bytes) = 0;
  virtual void barrier() = 0;
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

// Environment flags, logging and the chrome-trace timeline of the C++ runtime.
// Reference: src/utils/environment.h:21-399 (Env singleton), src/utils/verbose.h, src/utils/logger.h,
// src/utils/timeline.h (RAII scopes dumped as chrome-trace JSON).  Same variable names as the Python package
// (xfastertransformer_b200/utils/flags.py) so one launch script configures both.
#pragma once
#include <cstdint>
#include <set>
#include <string>

namespace xft {

class Env {
public:
  static Env& get();
  void reload();                       // re-read the process environment (tests)

  int verbose = 0;                     // XFT_VERBOSE: 0 quiet, 1 per-step timings, 2 per-kernel notes
  int pipelineStage = 1;               // XFT_PIPELINE_STAGE
  int maxRequestNum = 1;               // XFT_MAX_REQUEST_NUM: micro-batches of one forward pass over pipeline stages
  int fakeModel = 0;                   // XFT_FAKE_MODEL: 1 zeros, 2 random N(0, 0.02)
  bool fakeLoadInfo = false;           // XFT_FAKE_LOAD_INFO
  bool timeline = false;               // XFT_TIMELINE
  std::set<std::string> timelineWhitelist;   // XFT_TIMELINE_WHITELIST (comma separated; empty = all)
  std::string debugDir;                // XFT_DEBUG_DIR
  int kvBlockSize = 64;                // XFT_KV_BLOCK_SIZE
  bool cudaGraph = true;               // XFT_CUDA_GRAPH
  int maxBatchTokens = 8192;           // XFT_MAX_BATCH_TOKENS
  double kvCacheGb = 0.0;              // XFT_KV_CACHE_GB
  int attnSplits = 0;                  // XFT_ATTN_SPLITS
  std::string engine;                  // XFT_ENGINE

private:
  Env() { reload(); }
};

enum class LogLevel { Debug = 0, Info, Warn, Error };
// printf-style; Debug and Info need XFT_VERBOSE >= 2 / >= 1, Warn and Error always print (stderr)
void log(LogLevel level, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// RAII scope of the timeline.  Records {ph:"X", name, pid, tid, ts, dur} when XFT_TIMELINE=1 (and the name passes the
// whitelist); TimeLine::dump() writes timeline_<pid>.json (or the given path) and clears the buffer.
class TimeLine {
public:
  explicit TimeLine(const char* name);
  ~TimeLine();
  TimeLine(const TimeLine&) = delete;
  TimeLine& operator=(const TimeLine&) = delete;
  static void enable(bool on);
  static size_t pending();
  static std::string dump(const std::string& path = "");
private:
  const char* name_;
  int64_t t0_ = 0;
  bool on_ = false;
};

}  // namespace xft

#include "env.h"

#include <unistd.h>

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <mutex>
#include <sstream>
#include <thread>
#include <vector>

namespace xft {
namespace {
int envInt(const char* name, int def) {
  const char* v = std::getenv(name);
  if (!v || !*v) return def;
  char* end = nullptr;
  long r = std::strtol(v, &end, 10);
  return end == v ? def : (int)r;
}
std::string envStr(const char* name) {
  const char* v = std::getenv(name);
  return v ? std::string(v) : std::string();
}
struct Event { std::string name; int64_t ts, dur; uint64_t tid; };
std::mutex g_mu;
std::vector<Event> g_events;
int g_enabled = -1;          // -1: follow the environment
int64_t nowUs() {
  return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
bool tracing() { return g_enabled < 0 ? Env::get().timeline : g_enabled != 0; }
}  // namespace

Env& Env::get() {
  static Env e;
  return e;
}

void Env::reload() {
  verbose = envInt("XFT_VERBOSE", 0);
  pipelineStage = std::max(1, envInt("XFT_PIPELINE_STAGE", 1));
  maxRequestNum = std::max(1, envInt("XFT_MAX_REQUEST_NUM", 1));
  fakeModel = envInt("XFT_FAKE_MODEL", 0);
  fakeLoadInfo = envInt("XFT_FAKE_LOAD_INFO", 0) != 0;
  timeline = envInt("XFT_TIMELINE", 0) != 0;
  timelineWhitelist.clear();
  std::stringstream ss(envStr("XFT_TIMELINE_WHITELIST"));
  for (std::string item; std::getline(ss, item, ',');) {
    const size_t b = item.find_first_not_of(" \t"), e = item.find_last_not_of(" \t");
    if (b != std::string::npos) timelineWhitelist.insert(item.substr(b, e - b + 1));
  }
  debugDir = envStr("XFT_DEBUG_DIR");
  kvBlockSize = envInt("XFT_KV_BLOCK_SIZE", 64);
  cudaGraph = envInt("XFT_CUDA_GRAPH", 1) != 0;
  maxBatchTokens = envInt("XFT_MAX_BATCH_TOKENS", 8192);
  const std::string gb = envStr("XFT_KV_CACHE_GB");
  kvCacheGb = gb.empty() ? 0.0 : std::atof(gb.c_str());
  attnSplits = envInt("XFT_ATTN_SPLITS", 0);
  engine = envStr("XFT_ENGINE");
}

void log(LogLevel level, const char* fmt, ...) {
  const int v = Env::get().verbose;
  if ((level == LogLevel::Debug && v < 2) || (level == LogLevel::Info && v < 1)) return;
  static const char* tag[] = {"debug", "info", "warn", "error"};
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  std::fprintf(stderr, "[xft %s] %s\n", tag[(int)level], buf);
}

TimeLine::TimeLine(const char* name) : name_(name) {
  if (!tracing()) return;
  const auto& wl = Env::get().timelineWhitelist;
  if (!wl.empty() && !wl.count(name)) return;
  on_ = true;
  t0_ = nowUs();
}

TimeLine::~TimeLine() {
  if (!on_) return;
  const int64_t t1 = nowUs();
  const uint64_t tid = std::hash<std::thread::id>()(std::this_thread::get_id()) & 0xffff;
  std::lock_guard<std::mutex> g(g_mu);
  g_events.push_back({name_, t0_, t1 - t0_, tid});
}

void TimeLine::enable(bool on) { g_enabled = on ? 1 : 0; }

size_t TimeLine::pending() {
  std::lock_guard<std::mutex> g(g_mu);
  return g_events.size();
}

std::string TimeLine::dump(const std::string& path) {
  std::vector<Event> ev;
  {
    std::lock_guard<std::mutex> g(g_mu);
    ev.swap(g_events);
  }
  if (ev.empty()) return "";
  const std::string file = path.empty() ? "timeline_" + std::to_string((long)getpid()) + ".json" : path;
  std::ofstream f(file);
  f << "{\"traceEvents\":[";
  for (size_t i = 0; i < ev.size(); ++i) {
    if (i) f << ",";
    f << "{\"ph\":\"X\",\"name\":\"" << ev[i].name << "\",\"pid\":" << (long)getpid() << ",\"tid\":" << ev[i].tid << ",\"ts\":" << ev[i].ts
      << ",\"dur\":" << ev[i].dur << "}";
  }
  f << "]}\n";
  return file;
}

}  // namespace xft

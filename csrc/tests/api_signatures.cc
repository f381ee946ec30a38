// Compile-only check that programs written against the reference's include/models.h keep compiling: every call form of
// its Model / AutoModel API (include/models.h:27-133) is spelled out once.  Never run; tests/test_cpp_runtime.py
// compiles it with -fsyntax-only.
#include <tuple>
#include <vector>

#include "xft/models.h"

void every_call_form(xft::Model& m, std::vector<int32_t>& flat, std::vector<std::vector<int32_t>>& ragged, SearcherConfig& cfg,
                     std::vector<int>& seqIDs, std::vector<int>& maxLens, std::vector<int32_t>& seqLens,
                     std::vector<std::vector<int>>& stopWords) {
  m.input(flat, 2);
  m.config(128, 4, 2, 1.0f, false, 2, 0, false, 1.0f, 50, 1.0f, 1.0f, stopWords);
  m.config(cfg, stopWords);
  std::vector<int> ids;
  ids = m.set_input(flat, 2, 128, 1, 1, 1.0f, false, -1, -1, true, 0.8f, 40, 0.9f, 1.1f, stopWords);
  ids = m.set_input(flat, 2, cfg);
  ids = m.set_input(ragged, cfg, stopWords);
  ids = m.set_input(ragged, 128, 1);
  ids = m.set_input(ragged, seqIDs, cfg, stopWords);
  ids = m.set_input(ragged, seqIDs);
  ids = m.set_input(ragged, seqIDs, 128);
  ids = m.set_input(flat, 2, seqIDs);
  ids = m.set_input(flat, 2, seqIDs, 128);
  ids = m.set_input(flat, 2, seqIDs, maxLens);
  ids = m.set_input(flat, seqLens, seqIDs, maxLens);
  bool done = m.isDone();
  std::tuple<float*, int, int> all = m.forward();
  std::tuple<float*, int, int> last = m.forward(false);
  std::vector<int32_t> next = m.generate();
  std::vector<int32_t> out = m.finalize();
  m.createSearcher(cfg);
  bool master = m.isMaster();
  int rank = m.getRank(), bs = m.getBatchSize(), sl = m.getSeqLen(), v = m.getVocabSize(), ml = m.getMaxSeqLen();
  SearcherConfig c2 = m.getConfig();
  m.exitSlaves();
  m.setPrefix(flat);
  m.unsetPrefix();
  bool ok = m.setStopWords(stopWords) && m.freeSeqs(seqIDs);
  (void)done; (void)all; (void)last; (void)next; (void)out; (void)master; (void)rank; (void)bs; (void)sl; (void)v; (void)ml; (void)c2; (void)ok;
}

xft::AutoModel* construct(const char* path) { return new xft::AutoModel(path, xft::DataType::bf16, xft::DataType::int8); }

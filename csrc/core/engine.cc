// Native C++ engine behind xft::Model / xft::AutoModel: loads a converted checkpoint (config.ini + .bin), keeps
// weights as bf16 [out, in] on the device, and runs the dense decoder families through the sm_100a kernels of
// libxft_b200_kernels.so with a paged KV cache.  Reference: src/models/models.cpp (driver), common_decoder.h
// (forward), decoder_block.h (weight loading), kvcache_mgr.h, sampling.cpp (greedy / stop check).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <random>
#include <stdexcept>
#include <thread>

#include "arena.h"
#include "beam.h"
#include "comm.h"
#include "dtypes.h"
#include "env.h"
#include "gptq.h"
#include "ini.h"
#include "kernels_c.h"
#include "rope_tables.h"
#include "runtime.h"
#include "xft/models.h"

namespace xft {

#define XFT_CUDA(x)                                                                                     \
  do {                                                                                                  \
    cudaError_t e_ = (x);                                                                               \
    if (e_ != cudaSuccess) throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(e_) + " at " #x); \
  } while (0)
#define XFT_K(x)                                                                          \
  do {                                                                                    \
    int rc_ = (x);                                                                        \
    if (rc_ != 0) throw std::runtime_error("kernel launch failed (" + std::to_string(rc_) + "): " #x); \
  } while (0)

namespace {

struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
  DevBuf() = default;
  explicit DevBuf(size_t n) { reset(n); }
  DevBuf(const DevBuf&) = delete;
  DevBuf& operator=(const DevBuf&) = delete;
  DevBuf(DevBuf&& o) noexcept : p(o.p), bytes(o.bytes) { o.p = nullptr; o.bytes = 0; }
  DevBuf& operator=(DevBuf&& o) noexcept { std::swap(p, o.p); std::swap(bytes, o.bytes); return *this; }
  ~DevBuf() { if (p) Arena::device().release(p); }
  // device memory comes from the caching arena: buffers that are dropped and re-created between requests
  // (scratch that grows, KV pools that are reallocated) reuse cached blocks instead of calling cudaMalloc
  void reset(size_t n) {
    if (p) { Arena::device().release(p); p = nullptr; }
    bytes = n;
    if (n) {
      p = Arena::device().allocate(n);
      if (!p) throw std::runtime_error("out of device memory allocating " + std::to_string(n) + " bytes");
    }
  }
  void ensure(size_t n) {
    // grows with a quarter of slack, except under XFT_ARENA_EXACT (see arena.cc)
    static const bool exact = [] { const char* v = std::getenv("XFT_ARENA_EXACT"); return v && *v && *v != '0'; }();
    if (n > bytes) reset(exact ? n : n + n / 4);
  }
  template <class T> T* as() const { return static_cast<T*>(p); }
};

// XFT_FAKE_MODEL (reference: src/utils/weight_util.h:76-82 zero-fills): 1 = zeros, 2 = N(0, 0.02) weights, norm gains
// of one and zero biases, so that a model of any size runs without files.  `dt`: 0 fp32, 1 fp16, 2 bf16.
std::vector<char> fakeTensor(const std::string& path, size_t bytes, int dt, int mode) {
  std::vector<char> buf(bytes, 0);
  if (mode < 2) return buf;
  const bool bias = path.find("bias") != std::string::npos;
  const bool gain = !bias && (path.find("norm") != std::string::npos);
  if (bias) return buf;
  std::mt19937 gen((uint32_t)std::hash<std::string>()(path));
  std::normal_distribution<float> nd(0.f, 0.02f);
  const size_t n = bytes / (dt == 0 ? 4 : 2);
  for (size_t i = 0; i < n; ++i) {
    const float v = gain ? 1.f : nd(gen);
    if (dt == 0) std::memcpy(buf.data() + 4 * i, &v, 4);
    else { const uint16_t h = dt == 1 ? floatToHalf(v) : floatToBf16(v); std::memcpy(buf.data() + 2 * i, &h, 2); }
  }
  return buf;
}

std::vector<char> readFile(const std::string& path, size_t expect, int dt) {
  if (const int fake = xft::Env::get().fakeModel) {
    // XFT_FAKE_LOAD_INFO: say which tensor a real load would have read here
    if (xft::Env::get().fakeLoadInfo) {
      const size_t cut = path.find_last_of('/');
      std::printf("[fake load] %s %zu bytes\n", path.substr(cut == std::string::npos ? 0 : cut + 1).c_str(), expect);
    }
    return fakeTensor(path, expect, dt, fake);
  }
  std::ifstream f(path, std::ios::binary | std::ios::ate);
  if (!f) throw std::runtime_error("cannot open " + path);
  size_t sz = (size_t)f.tellg();
  if (sz != expect) throw std::runtime_error(path + ": expected " + std::to_string(expect) + " bytes, found " + std::to_string(sz));
  std::vector<char> buf(sz);
  f.seekg(0);
  f.read(buf.data(), (std::streamsize)sz);
  return buf;
}

}  // namespace

// XFT_VERBOSE >= 1: one line per GEMM-shaped call in the reference's format (src/utils/verbose.h:24-83),
// `xft_verbose,exec,gpu,api,<kernel>,m<M>n<N>k<K>,<ms>`; the stream is synchronised on both sides of the call.
struct VerboseCall {
  cudaStream_t st;
  const char* kernel;
  int m, n, k;
  bool on;
  std::chrono::steady_clock::time_point t0;
  VerboseCall(cudaStream_t s, const char* name, int m_, int n_, int k_)
      : st(s), kernel(name), m(m_), n(n_), k(k_), on(xft::Env::get().verbose >= 1) {
    if (on) { cudaStreamSynchronize(st); t0 = std::chrono::steady_clock::now(); }
  }
  ~VerboseCall() {
    if (!on) return;
    cudaStreamSynchronize(st);
    const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    std::printf("xft_verbose,exec,gpu,api,%s,m%dn%dk%d,%.6f\n", kernel, m, n, k, ms);
  }
};

struct LayerWeights {
  DevBuf qkv, o, gateUp, down, n1, n2, qkvBias, qNorm, kNorm;
  DevBuf n1b, n2b, oBias, fc1Bias, fc2Bias;      // LayerNorm biases, output-projection bias, biases of the two-matrix MLP
  DevBuf router, expGateUp, expDown;             // mixture of experts: [E, hidden], stacked [E * 2I, hidden], [E * hidden, I]
  DevBuf expGateUpNext, expDownNext;             // hybrid weight types: the experts as the decode steps see them
  // DeepSeek e4m3 checkpoints: the experts stay e4m3 on the device (bytes in expGateUp / expDown, one fp32 scale per
  // 128 x 128 block here), the grouped GEMM expands tiles on the way to the tensor core
  DevBuf expGateUpScale, expDownScale;
  bool fp8Experts = false;
  // DeepSeek.  Attention: merged down-projection [q_lora (or heads * qk) + kv_lora + rope, hidden], its norms, the query
  // up-projection, and the per-head halves of kv_b: W_uk transposed [heads * kv_lora, nope], W_uv [heads * v, kv_lora].
  DevBuf qkvA, qANorm, qB, kvANorm, wkT, wv;
  DevBuf routerBias, sharedGateUp, sharedDown;   // correction bias [E]; shared experts as one gated MLP
  bool denseMlp = true;                          // the first layers of DeepSeek are dense
};

// A projection as the GEMMs see it: bf16 [rows, K], or per-output-channel codes (int8 [rows, K]; NF4 two codes per byte
// [rows, K / 2]) with scale / zero point per row and, for int8 activations, the per-row sum of the codes.
struct Lin {
  const void* w = nullptr;       // bf16 weights (kind 0)
  DevBuf q, scale, zero, wsum;
  int rows = 0, K = 0, pitch = 0;       // pitch: bytes from one row of codes to the next
  int kind = 0;                         // 0 bf16, 1 int8 weight-only, 2 int8 x int8 activations, 3 NF4, 4 uint4
};

// What distinguishes one dense family from another (reference: one C++ class per family under src/models, selected by
// the factory key of model_factory.h:57-114); the forward pass below reads these fields instead of being specialised.
struct FamilySpec {
  const char* name;
  bool layerNorm = false;      // LayerNorm with bias instead of RMSNorm
  int ropeStyle = 0;           // 0: pairs (i, i + rot/2); 1: pairs (2i, 2i + 1)
  double rotFrac = 1.0;        // rotary dims / head dim
  bool rope2d = false;         // ChatGLM-1: two position streams, one per half of the head
  int mlp = 0;                 // 0: gate_proj / up_proj / down_proj; 1: dense_h_to_4h + bias -> act -> dense_4h_to_h + bias;
                               // 2: merged gate‖up in dense_h_to_4h, dense_4h_to_h; 3: routed experts (Mixtral, Qwen3-MoE)
  int embedding = 0;           // 0 plain, 1 scaled by sqrt(hidden) (Gemma), 2 plus learned positions at offset 2 (OPT)
  bool lognNtk = false;        // Qwen-1: dynamic-NTK base and log-n query scale beyond the training length
  bool telechatNtk = false;    // TeleChat: NTK base from max(context, training length), table scale on long inputs
  bool residFromNorm = false;  // ChatGLM-1: residual = sqrt(2 * layers) * normalised input
  bool prefixLm = false;       // ChatGLM-1: the prompt up to its bos token attends in both directions
  int routeKind = 0;           // experts: 0 softmax over the top-k logits (Mixtral), 1 softmax then top-k, renormalised (Qwen3),
                               // 2 DeepSeek (sigmoid / softmax scores, correction bias, expert groups)
  bool mla = false;            // DeepSeek: latent attention (compressed KV cache) and shared + routed experts
};

const FamilySpec* familySpec(const std::string& type) {
  static const FamilySpec table[] = {
      {"llama"}, {"yarn_llama"}, {"qwen2"}, {"qwen3"}, {"baichuan"},
      {"gemma", false, 0, 1.0, false, 0, 1},
      {"qwen", false, 0, 1.0, false, 0, 0, true},
      {"telechat", false, 0, 1.0, false, 0, 0, false, true},
      {"chatglm2", false, 1, 0.5, false, 2},
      {"chatglm3", false, 1, 0.5, false, 2},
      {"chatglm4", false, 1, 0.5, false, 2},
      {"gpt", true, 0, 0.0, false, 1, 2},
      {"chatglm", true, 0, 0.5, true, 1, 0, false, false, true, true},
      {"mixtral", false, 0, 1.0, false, 3, 0, false, false, false, false, 0},
      {"qwen3_moe", false, 0, 1.0, false, 3, 0, false, false, false, false, 1},
      {"deepseek_moe", false, 1, 1.0, false, 3, 0, false, false, false, false, 2, true},
  };
  for (const FamilySpec& f : table)
    if (type == f.name) return &f;
  return nullptr;
}

class Engine {
public:
  Engine(const std::string& path, DataType dt, DataType kvdt, std::shared_ptr<Communicator> comm = nullptr);
  // tensor parallelism (src/layers/decoder_block.h + split_util.h): this rank holds the query heads [q0, q1) with the
  // KV heads that cover them, rows [i0, i1) of the FFN and rows [v0, v1) of the lm_head.  After these ranges are set,
  // `heads`, `kvHeads`, `inter` and `vocab` below are THIS RANK'S counts; the model's own are the ...G fields.
  // `worldComm`: every rank (arguments of rank 0, stage boundaries, the logits of the last stage); `comm`: the tensor-
  // parallel group of this pipeline stage (the same object when there is one stage; null when the group has one rank)
  std::shared_ptr<Communicator> worldComm, comm;
  int worldRank = 0, worldSize = 1;
  // pipeline stages (XFT_PIPELINE_STAGE, src/models/common_decoder.h:389-391,497-498): world = stages x tensor-parallel
  // ranks; stage s runs layers [l0, l1), receives the hidden state of stage s - 1 and hands its own to stage s + 1; the
  // last stage computes the logits and every rank receives them
  int pp = 1, ppRank = 0, l0 = 0, l1 = 0;
  int rank = 0, world = 1;
  int headsG = 0, kvHeadsG = 0, interG = 0, vocabG = 0;
  int q0 = 0, kv0 = 0, i0 = 0, v0 = 0, qOff = 0, groupG = 1, vocabPad = 0;
  // hyper-parameters
  std::string type;
  int heads = 0, kvHeads = 0, headDim = 0, hidden = 0, inter = 0, layers = 0, vocab = 0, maxPos = 0, endId = 0;
  float eps = 1e-6f, ropeTheta = 10000.f, embedScale = 1.f;
  int act = 2;   // kernel activation code: 1 relu, 2 silu, 3 gelu
  bool qkNorm = false, kvInt8 = false;
  FamilySpec spec{""};
  int rotDim = 0;              // 0: no rotary table (OPT, ALiBi Baichuan)
  int wpeRows = 0;             // OPT: rows of the learned position table
  int experts = 0, topK = 0, moeInter = 0;       // mixture of experts: count, experts per token, expert FFN width
  int sharedInterG = 0, s0 = 0;                  // DeepSeek shared experts: whole width, first column of this rank
  int e0 = 0, e1 = 0;                            // experts kept by this rank: every rank routes every token, multiplies
                                                 // the rows of its own experts, and the ranks' partial sums are added
  int wq = 0;                  // layer projections: 0 bf16, 1 weight-only int8, 2 int8 weights x int8 activations, 3 NF4, 4 uint4
  int wqNext = 0;              // hybrid types "A_B" (src/models/hybrid_model.h): A for the prompt pass, B for decode steps
  int gptq = 0;                // checkpoint holds GPTQ codes: 1 int8, 2 uint4 (0: dense tensors)
  // DeepSeek
  int qLora = 0, kvLora = 0, nope = 0, ropeD = 0, vDim = 0, firstDense = 0, sharedInter = 0, nGroup = 1, topkGroup = 1;
  float routedScale = 1.f, attnScale = 1.f;
  bool normTopk = true, sigmoidScores = true;
  int auxDt = 1;               // dtype of embeddings, head and norm gains on disk (DeepSeek keeps them in bf16)
  bool alibi = false;
  int trainLen = 0;            // Qwen-1 seq_length / TeleChat training context
  bool useDynamicNtk = true, useLognAttn = true;

  SequencePool pool;
  std::unique_ptr<BlockTables> tables;
  std::vector<int> working, cbActive;
  int prefixSeq = -1;
  std::vector<float> hostLogits;
  std::mt19937_64 rng;
  // beam search state of the current request (numBeams > 1): beam i of request r is beamSeqs[r * numBeams + i]
  std::unique_ptr<BeamSearchScorer> scorer;
  std::vector<int> beamSeqs;
  std::vector<std::vector<int32_t>> beamPrompts;

  // Runs the pending inputs of `ids`; logits land in hostLogits [rows, vocab].  Returns rows.
  int forward(const std::vector<int>& ids, bool logitsAll);
  int forwardPart(const std::vector<int>& ids, bool logitsAll, bool shareLogits);
  void ensureBlocks(int extra);
  void release(int id) { tables->free(id); pool.remove(id); }
  void attachPrefix(SequenceMeta& s);

private:
  // file [inF, outF] -> dst rows [dstRowOffset, ...) = the outputs [o0, o1) over the inputs [n0, n1) (whole tensor when
  // the ranges are left at -1), transposed to [out, in]
  void loadLinear(const std::string& file, int inF, int outF, void* dst, int dstRowOffset, int dstLd, int o0 = -1, int o1 = -1,
                  int n0 = -1, int n1 = -1);
  // elements [e0, e1) of a vector of n (all of it by default)
  DevBuf loadVector(const std::string& file, int n, bool optional = false, int dt = -1, int e0 = -1, int e1 = -1);
  void copyBlock(int src, int dst);
  std::string dir;
  int fileDt = 1;
  // DeepSeek tensor `<base>.weight.bin` ([in, out]; e4m3 with `<base>.weight_scale_inv.bin` block scales, or a float type)
  void loadDsLinear(const std::string& base, int inF, int outF, void* dst, int dstRowOffset, int dstLd, int o0 = 0, int o1 = -1,
                    int c0 = 0, int c1 = -1);
  void loadMlaLayer(const std::string& p, LayerWeights& L, int layer);
  void requantiseRows(DevBuf& w, size_t rows, int K, int kind);
  // XFT_DEBUG_DIR: the hidden state [T, hidden] at a named point of the forward pass goes to a file and a log line
  void dumpState(const std::string& name, const void* state, int T);
  long long debugStep = 0;
  void loadFp8Expert(const std::string& base, int inF, int outF, uint8_t* bytes, float* scales);
  // dense bf16 [rows, K] -> the prompt-pass form `first` and, for hybrid types, the decode form `next`; `dense` is
  // released unless a bf16 form points at it
  void quantise(DevBuf& dense, int rows, int K, Lin& first, Lin& next);
  void quantiseAs(const DevBuf& dense, int rows, int K, int kind, Lin& out);
  struct LayerLins;
  struct GptqPart { std::string base; int outF, o0, o1; };       // rows [o0, o1) of one tensor of outF outputs
  // the projections of one layer from GPTQ tensors; rows of several tensors are stacked (q‖k‖v slices, gate‖up)
  void loadGptqLayer(const std::string& p, LayerLins& first, LayerLins& next);
  void loadGptq(const std::vector<GptqPart>& parts, int inF, int n0, int n1, Lin& first, Lin& next);
  std::vector<DevBuf> gptqDense;                                  // dequantised tensors that bf16 projections point at
  // bytes of one 64-token block of one layer's K (or V) pool; the latent cache of DeepSeek has one row of
  // kv_lora_rank + rope values per token and no V pool
  size_t kvBlockBytes() const {
    return spec.mla ? (size_t)kBlock * (kvLora + ropeD) * 2 : (size_t)kvHeads * kBlock * headDim * (kvInt8 ? 1 : 2);
  }
  const float* ropeFor(int maxKv, int maxQ);      // the rotary table of this pass (NTK families keep one per base)
  DevBuf wte, wpe, lmHead, finalNorm, finalNormBias, ropeTable_, slopes_, ws, counters, status, attnCounters, partO, partMl;
  std::map<long long, DevBuf> ntkTables_;         // by round(base): Qwen-1 / TeleChat tables beyond the first
  RopeScaling ropeScaling_;
  std::vector<LayerWeights> lw;
  struct LayerLins { Lin qkv, o, gateUp, down; };
  std::vector<LayerLins> lins, linsNext;
  DevBuf actQ, actScale, actZero, actSum, guBuf;   // int8 activations + their row statistics; gate‖up before the activation
  DevBuf mQaKv, mQa, mQ, mQNope, mQRope, mQAbs, mOLat, mOHead, mTiles, mMeta, mShared;   // latent-attention activations
  std::vector<DevBuf> kc, vc, ks, vs;
  int numBlocks = 0;
  // activations
  DevBuf moeLogits, moeIdx, moeWts, moePos, moeSrc, moeRowW, moeTiles, moeMeta, moeXs, moeH1, moeYs;
  DevBuf gathered;             // logits slices of all ranks
  DevBuf dIds, dPos, dPos2, dPrefix, dQScale, dSlots, dCu, dKv, dBt, x, x2, h, qkvBuf, q, att, g, rows, logits;
  cudaStream_t st = nullptr;
  static constexpr int kBlock = 64;
  static constexpr size_t kWsBytes = 64u << 20;
};

void Engine::loadLinear(const std::string& file, int inF, int outF, void* dst, int dstRowOffset, int dstLd, int o0, int o1,
                        int n0, int n1) {
  if (o0 < 0) { o0 = 0; o1 = outF; }
  if (n0 < 0) { n0 = 0; n1 = inF; }
  auto host = readFile(dir + "/" + file, (size_t)inF * outF * dtypeSize(fileDt), fileDt);
  DevBuf tmp(host.size());
  XFT_CUDA(cudaMemcpy(tmp.p, host.data(), host.size(), cudaMemcpyHostToDevice));
  const char* src = tmp.as<char>() + ((size_t)n0 * outF + o0) * dtypeSize(fileDt);
  XFT_K(xft_transpose_to_bf16(src, fileDt, outF, n1 - n0, o1 - o0, static_cast<__nv_bfloat16*>(dst) + (size_t)dstRowOffset * dstLd,
                              dstLd, st));
  XFT_CUDA(cudaStreamSynchronize(st));
}

DevBuf Engine::loadVector(const std::string& file, int n, bool optional, int dt, int e0, int e1) {
  if (dt < 0) dt = auxDt;
  if (e0 < 0) { e0 = 0; e1 = n; }
  std::ifstream probe(dir + "/" + file, std::ios::binary);
  if (!probe) {
    if (optional) return DevBuf();
    if (!Env::get().fakeModel) throw std::runtime_error("missing " + file);
  }
  auto host = readFile(dir + "/" + file, (size_t)n * dtypeSize(dt), dt);
  const int m = e1 - e0;
  std::vector<float> f(m);
  for (int i = 0; i < m; ++i) f[i] = elemToFloat(host.data(), dt, (size_t)e0 + i);
  DevBuf d((size_t)std::max(m, 1) * 4);
  XFT_CUDA(cudaMemcpy(d.p, f.data(), (size_t)m * 4, cudaMemcpyHostToDevice));
  return d;
}

Engine::Engine(const std::string& path, DataType dt, DataType kvdt, std::shared_ptr<Communicator> c) : worldComm(std::move(c)), dir(path) {
  if (worldComm && worldComm->size() > 1) { worldRank = worldComm->rank(); worldSize = worldComm->size(); worldComm->begin(); }
  else worldComm.reset();
  pp = worldComm ? Env::get().pipelineStage : 1;
  if (pp > 1) {
    if (worldSize % pp) throw std::runtime_error("XFT_PIPELINE_STAGE does not divide the number of ranks");
    const int tp = worldSize / pp;
    ppRank = worldRank / tp;
    rank = worldRank % tp;
    world = tp;
    if (tp > 1) comm = worldComm->split(ppRank, rank);
  } else {
    comm = worldComm;
    rank = worldRank;
    world = worldSize;
  }
  Ini ini(path + "/config.ini");
  if (!ini.ok() || ini.sections().empty()) throw std::runtime_error("config.ini not found under " + path);
  type = ini.sections()[0];
  const FamilySpec* fam = familySpec(type);
  if (!fam) throw std::runtime_error("config.ini names a model type this engine does not know: [" + type + "]");
  spec = *fam;
  switch (dt) {
    case DataType::bf16: case DataType::fp16: case DataType::bf16_fp16: break;      // fp16 weights are kept as bf16
    case DataType::int8: wq = wqNext = 1; break;
    case DataType::w8a8: wq = wqNext = 2; break;
    case DataType::nf4: wq = wqNext = 3; break;
    case DataType::int4: wq = wqNext = 4; break;
    case DataType::bf16_int8: wqNext = 1; break;
    case DataType::bf16_w8a8: wqNext = 2; break;
    case DataType::bf16_nf4: wqNext = 3; break;
    case DataType::bf16_int4: wqNext = 4; break;
    case DataType::w8a8_int8: wq = 2; wqNext = 1; break;
    case DataType::w8a8_nf4: wq = 2; wqNext = 3; break;
    case DataType::w8a8_int4: wq = 2; wqNext = 4; break;
    default: throw std::runtime_error("the native C++ engine runs bf16, int8, w8a8, int4, nf4 weights and their hybrids");
  }
  kvInt8 = kvdt == DataType::int8;
  heads = (int)ini.getInt(type, "head_num");
  kvHeads = (int)ini.getInt(type, "kv_head_num", heads);
  headDim = (int)ini.getInt(type, "size_per_head");
  hidden = (int)ini.getInt(type, "hidden_size", heads * headDim);
  inter = (int)ini.getInt(type, "inter_size");
  layers = (int)ini.getInt(type, "num_layer");
  if (pp > layers) throw std::runtime_error("more pipeline stages than layers");
  { const auto lr = ppLayerRange(layers, pp, ppRank); l0 = lr.first; l1 = lr.second; }
  vocab = (int)ini.getInt(type, "vocab_size");
  maxPos = std::max<int>({(int)ini.getInt(type, "max_pos_seq_len", 0), (int)ini.getInt(type, "model_max_length", 0), 2048});
  // Baichuan-13B has no rotary table: ALiBi slopes on the attention scores (src/layers/attn_baichuan.h:33-47)
  alibi = type == "baichuan" && ini.getInt(type, "max_pos_seq_len", 0) <= 0;
  eps = (float)ini.getFloat(type, "layernorm_eps", ini.getFloat(type, "rms_norm_eps", 1e-6));
  ropeTheta = (float)ini.getFloat(type, "rope_theta", 10000.0);
  std::string rtype = ini.get(type, "rope_scaling_type", ini.get(type, "rope_type", ""));
  RopeScaling rs;
  if (type == "yarn_llama" && (rtype.empty() || rtype == "default")) rtype = "yarn";
  if (rtype == "linear" || rtype == "yarn") {
    rs.type = rtype;
    rs.factor = ini.getFloat(type, "rope_scaling_factor", ini.getFloat(type, "scaling_factor", 1.0));
    rs.originalMaxPos = (int)ini.getInt(type, "rope_scaling_original_max_position_embeddings",
                                        ini.getInt(type, "original_max_position_embeddings", 2048));
    rs.betaFast = ini.getFloat(type, "rope_scaling_beta_fast", 32.0);
    rs.betaSlow = ini.getFloat(type, "rope_scaling_beta_slow", 1.0);
    // Llama YaRN scales the table by 0.1 ln(factor) + 1 (yarn_scaled_rotary_embedding.cpp:26-84)
    if (rtype == "yarn") rs.tableScale = yarnMscale(rs.factor, 1.0);
  } else if (!rtype.empty() && rtype != "default") {
    throw std::runtime_error("rope scaling '" + rtype + "' is not supported (linear and yarn are)");
  } else if (type.rfind("chatglm", 0) == 0 && type != "chatglm") {
    // rope_ratio of the long-context GLM checkpoints multiplies the base
    ropeTheta *= (float)ini.getFloat(type, "rope_scaling_factor", ini.getFloat(type, "scaling_factor", 1.0));
  }
  ropeScaling_ = rs;
  rotDim = (alibi || spec.rotFrac <= 0.0) ? 0 : (int)(headDim * spec.rotFrac);
  if (spec.lognNtk) {
    trainLen = (int)ini.getInt(type, "seq_length", -1);
    if (trainLen <= 0) trainLen = 8192;
    useDynamicNtk = ini.getBool(type, "use_dynamic_ntk", true);
    useLognAttn = ini.getBool(type, "use_logn_attn", true);
  } else if (spec.telechatNtk) {
    trainLen = (int)ini.getInt(type, "max_pos_seq_len", 0);
    if (trainLen <= 0) trainLen = 2048;
  }
  endId = (int)ini.getInt(type, "end_id", ini.getInt(type, "start_id", 0));
  std::string a = ini.get(type, "activation_type", "silu");
  act = a.rfind("gelu", 0) == 0 ? 3 : a == "relu" ? 1 : 2;
  if (spec.mlp == 1 && act == 2) act = 3;        // the two-matrix MLP is relu (OPT) or gelu
  if (spec.mlp == 2) act = 2;                    // the merged gate‖up MLP of ChatGLM2+ is SwiGLU
  if (spec.mlp == 3) {
    experts = (int)ini.getInt(type, "sparse_experts", 0);
    topK = (int)ini.getInt(type, "num_experts_per_tok", 0);
    if (topK <= 0) topK = type == "mixtral" ? 2 : 8;
    moeInter = type == "mixtral" ? 0 : (int)ini.getInt(type, "moe_intermediate_size", 0);
    if (moeInter <= 0) moeInter = inter;
    if (experts <= 0 || topK > experts || topK > 32 || moeInter % 8 || hidden % 8)
      throw std::runtime_error("mixture of experts: sparse_experts / num_experts_per_tok / sizes are not usable");
    if (a == "swiglu") act = 2;
  }
  qkNorm = ini.getBool(type, "do_qk_norm", false);
  if (spec.embedding == 1) embedScale = std::sqrt((float)hidden);
  std::string wdt = ini.get(type, "weight_data_type", "fp16");
  fileDt = wdt == "fp32" ? 0 : wdt == "bf16" ? 2 : wdt == "fp8_e4m3" ? 3 : 1;
  if (fileDt == 3 && !spec.mla) throw std::runtime_error("fp8 checkpoints are DeepSeek checkpoints");
  auxDt = spec.mla ? 2 : fileDt;
  if (spec.mla) {
    qLora = (int)ini.getInt(type, "q_lora_rank", 0);
    kvLora = (int)ini.getInt(type, "kv_lora_rank", 512);
    nope = (int)ini.getInt(type, "qk_nope_head_dim", 128);
    ropeD = (int)ini.getInt(type, "qk_rope_head_dim", 64);
    vDim = (int)ini.getInt(type, "v_head_dim", headDim);
    firstDense = (int)ini.getInt(type, "first_k_dense_replace", 0);
    sharedInter = (int)ini.getInt(type, "dense_experts", 0) * moeInter;
    sharedInterG = sharedInter;
    nGroup = std::max(1, (int)ini.getInt(type, "n_group", 1));
    topkGroup = std::max(1, (int)ini.getInt(type, "topk_group", 1));
    routedScale = (float)ini.getFloat(type, "routed_scaling_factor", 1.0);
    normTopk = ini.getBool(type, "norm_topk_prob", true);
    const std::string sf = ini.get(type, "scoring_func", "sigmoid");
    sigmoidScores = sf.empty() || sf == "sigmoid";
    if (kvLora != 512 || ropeD != 64) throw std::runtime_error("the latent attention kernel is built for kv_lora_rank 512 + rope 64");
    if (kvInt8) throw std::runtime_error("the latent KV cache is bf16");
    if (wq || wqNext) throw std::runtime_error("quantised DeepSeek weights run through the Python API");
    if (nope % 8 || vDim % 8 || (qLora % 8) || sharedInter % 8) throw std::runtime_error("DeepSeek head sizes must be multiples of 8");
    // rotary table of the rope part only: YaRN with the model's mscale pair; softmax scale 1 / sqrt(nope + rope) times
    // (0.1 mscale_all_dim ln(factor) + 1)^2 (src/models/common_decoder.h:272-274 hard-wires factor 40)
    rs.mscale = ini.getFloat(type, "rope_scaling_mscale", 1.0);
    rs.mscaleAllDim = ini.getFloat(type, "rope_scaling_mscale_all_dim", 0.0);
    rs.tableScale = -1.0;
    ropeScaling_ = rs;
    rotDim = ropeD;
    maxPos = std::min(maxPos, 163840);
    attnScale = 1.0f / std::sqrt((float)(nope + ropeD));
    if (rs.type == "yarn" && rs.factor > 1.0) {
      const double m = 0.1 * rs.mscaleAllDim * std::log(rs.factor) + 1.0;
      attnScale = (float)(attnScale * m * m);
    }
  }
  {
    // GPTQ-converted checkpoint (llama_convert.py:335-392): per-channel codes + fp32 scales and zeros on disk
    const std::string qt = ini.get(type, "quant_qweight_data_type", "");
    if (!qt.empty()) {
      gptq = qt == "int8" ? 1 : qt == "uint4" ? 2 : 0;
      if (!gptq) throw std::runtime_error("quant_qweight_data_type must be int8 or uint4");
      if (ini.get(type, "quant_scales_data_type", "fp32") != "fp32" || ini.get(type, "quant_zeros_data_type", "fp32") != "fp32")
        throw std::runtime_error("GPTQ scales and zeros must be fp32");
      if (spec.mlp != 0 || spec.mla) throw std::runtime_error("GPTQ checkpoints exist for the llama-style families");
    }
  }
  headsG = heads; kvHeadsG = kvHeads; interG = inter; vocabG = vocab;
  groupG = std::max(headsG / std::max(kvHeadsG, 1), 1);
  if (world > 1) {
    if ((spec.mlp == 3 || spec.mla) && world > experts) throw std::runtime_error("more ranks than experts");
    if (world > headsG) throw std::runtime_error("more tensor-parallel ranks than attention heads");
    // latent attention has no KV heads to share: every rank takes a run of query heads (with their slices of the query
    // up-projection, of W_uk / W_uv and of the output projection), the latent cache is the same on every rank
    const HeadRange hr = headRange(headsG, spec.mla ? headsG : kvHeadsG, world, rank);
    q0 = hr.q0; kv0 = hr.kv0;
    heads = hr.q1 - hr.q0; kvHeads = hr.kv1 - hr.kv0;
    qOff = q0 - kv0 * groupG;                    // first local query head inside its KV group
    const auto fr = taskRange(interG, world, rank);
    i0 = fr.first; inter = fr.second - fr.first;
    const auto vr = taskRange(vocabG, world, rank);
    v0 = vr.first; vocab = vr.second - vr.first;
    for (int r = 0; r < world; ++r) { const auto x = taskRange(vocabG, world, r); vocabPad = std::max(vocabPad, x.second - x.first); }
    if (spec.mlp != 3 && (inter % 8 || (wq == 2 || wqNext == 2 ? inter % 16 : 0)))
      throw std::runtime_error("FFN slice of this rank is not a multiple of 8");
    if (spec.mla && sharedInter > 0) {
      const auto sr = taskRange(sharedInter, world, rank);
      s0 = sr.first; sharedInter = sr.second - sr.first;
      // a narrow shared expert may leave the last ranks without columns: they add nothing for it
      if (sharedInter % 8) throw std::runtime_error("shared-expert slice of this rank is not a multiple of 8");
    }
  }
  if (spec.mlp == 3 || spec.mla) {
    // expert parallelism on replicated tokens (src/layers/mlp_mixtral.h:95-187 splits every expert's columns instead):
    // whole experts per rank keep the grouped GEMMs at full width
    const auto er = expertRange(experts, world, rank);
    e0 = er.first; e1 = er.second;
  }
  if (!spec.mla && headDim != 64 && headDim != 128 && headDim != 256) throw std::runtime_error("head size must be 64, 128 or 256");

  XFT_CUDA(cudaStreamCreate(&st));
  const int qsz = heads * headDim, kvsz = kvHeads * headDim;
  // embedding (whole) and this rank's rows of the lm_head; both are stored [vocab, hidden]: convert on the host
  {
    auto host = readFile(dir + "/model.wte.bin", (size_t)vocabG * hidden * dtypeSize(auxDt), auxDt);
    std::vector<uint16_t> b((size_t)vocabG * hidden);
    for (size_t i = 0; i < b.size(); ++i) b[i] = floatToBf16(elemToFloat(host.data(), auxDt, i));
    wte.reset(b.size() * 2);
    XFT_CUDA(cudaMemcpy(wte.p, b.data(), b.size() * 2, cudaMemcpyHostToDevice));
    host = readFile(dir + "/model.lm_head.weight.bin", (size_t)vocabG * hidden * dtypeSize(auxDt), auxDt);
    const size_t nloc = (size_t)vocab * hidden, off = (size_t)v0 * hidden;
    for (size_t i = 0; i < nloc; ++i) b[i] = floatToBf16(elemToFloat(host.data(), auxDt, off + i));
    lmHead.reset(nloc * 2);
    XFT_CUDA(cudaMemcpy(lmHead.p, b.data(), nloc * 2, cudaMemcpyHostToDevice));
  }
  if (spec.embedding == 2) {
    // learned positions of OPT: max_pos_seq_len + 2 rows (the first two are never addressed by a real position)
    wpeRows = (int)ini.getInt(type, "max_pos_seq_len", 0) + 2;
    const size_t n = (size_t)wpeRows * hidden;
    auto host = readFile(dir + "/model.wpe.bin", n * dtypeSize(fileDt), fileDt);
    std::vector<uint16_t> b(n);
    for (size_t i = 0; i < n; ++i) b[i] = floatToBf16(elemToFloat(host.data(), fileDt, i));
    wpe.reset(n * 2);
    XFT_CUDA(cudaMemcpy(wpe.p, b.data(), n * 2, cudaMemcpyHostToDevice));
  }
  finalNorm = loadVector("model.final_layernorm.weight.bin", hidden);
  if (spec.layerNorm) finalNormBias = loadVector("model.final_layernorm.bias.bin", hidden);
  lw.resize(layers);
  lins.resize(layers);
  linsNext.resize(layers);
  for (int i = l0; i < l1; ++i) {
    const std::string p = "model.layers." + std::to_string(i) + ".";
    LayerWeights& L = lw[i];
    if (spec.mla) { loadMlaLayer(p, L, i); continue; }
    // merged QKV on disk: all query heads, then all key heads, then all value heads; this rank takes its query heads
    // and the KV heads that cover them.  Row-parallel projections (attention output, FFN down) take the matching
    // INPUT range; their bias is added on rank 0 only, so that the sum over ranks counts it once.
    const int qszG = headsG * headDim, kvszG = kvHeadsG * headDim, qkvG = qszG + 2 * kvszG;
    // GPTQ checkpoints hold codes instead of these dense tensors: loadGptqLayer below builds the projections from them
    auto denseLoad = [&](const std::string& file, int inF, int outF, void* dst, int dstRow, int dstLd, int o0 = -1, int o1 = -1,
                         int n0 = -1, int n1 = -1) {
      if (!gptq) loadLinear(file, inF, outF, dst, dstRow, dstLd, o0, o1, n0, n1);
    };
    const std::string qkvFile = p + "attention.query_key_value.weight.0.bin", qkvBiasFile = p + "attention.query_key_value.bias.0.bin";
    if (!gptq) L.qkv.reset((size_t)(qsz + 2 * kvsz) * hidden * 2);
    if (world == 1) {
      denseLoad(qkvFile, hidden, qkvG, L.qkv.p, 0, hidden);
      L.qkvBias = loadVector(qkvBiasFile, qkvG, true);
    } else {
      const int kOff = qszG + kv0 * headDim, vOff = qszG + kvszG + kv0 * headDim;
      denseLoad(qkvFile, hidden, qkvG, L.qkv.p, 0, hidden, q0 * headDim, q0 * headDim + qsz);
      denseLoad(qkvFile, hidden, qkvG, L.qkv.p, qsz, hidden, kOff, kOff + kvsz);
      denseLoad(qkvFile, hidden, qkvG, L.qkv.p, qsz + kvsz, hidden, vOff, vOff + kvsz);
      DevBuf bq = loadVector(qkvBiasFile, qkvG, true, -1, q0 * headDim, q0 * headDim + qsz);
      if (bq.p) {
        DevBuf bk = loadVector(qkvBiasFile, qkvG, true, -1, kOff, kOff + kvsz), bv = loadVector(qkvBiasFile, qkvG, true, -1, vOff, vOff + kvsz);
        L.qkvBias.reset((size_t)(qsz + 2 * kvsz) * 4);
        XFT_CUDA(cudaMemcpy(L.qkvBias.p, bq.p, (size_t)qsz * 4, cudaMemcpyDeviceToDevice));
        XFT_CUDA(cudaMemcpy(L.qkvBias.as<float>() + qsz, bk.p, (size_t)kvsz * 4, cudaMemcpyDeviceToDevice));
        XFT_CUDA(cudaMemcpy(L.qkvBias.as<float>() + qsz + kvsz, bv.p, (size_t)kvsz * 4, cudaMemcpyDeviceToDevice));
      }
    }
    if (!gptq) L.o.reset((size_t)hidden * qsz * 2);
    denseLoad(p + "attention.dense.weight.0.bin", qszG, hidden, L.o.p, 0, qsz, 0, hidden, q0 * headDim, q0 * headDim + qsz);
    if (rank == 0) L.oBias = loadVector(p + "attention.dense.bias.bin", hidden, true);
    if (spec.mlp == 3) {
      // router [hidden, experts] on disk -> [experts, hidden]; experts stacked: gate rows then up rows per expert, then
      // the down matrices (the layout the grouped GEMM walks, src/layers/mlp_mixtral.h:95-187 keeps one MLP object each)
      const bool mix = type == "mixtral";
      const int I = moeInter;
      L.router.reset((size_t)experts * hidden * 2);
      denseLoad(p + (mix ? "moe.gate.weight.bin" : "mlp.gate.weight.0.bin"), hidden, experts, L.router.p, 0, hidden);
      const int EL = e1 - e0;
      L.expGateUp.reset((size_t)EL * 2 * I * hidden * 2);
      L.expDown.reset((size_t)EL * hidden * I * 2);
      for (int e = e0; e < e1; ++e) {
        const std::string ep = p + (mix ? "moe.sparse_experts." : "mlp.experts.") + std::to_string(e) + ".";
        const int l = e - e0;
        denseLoad(ep + (mix ? "w1.0.bin" : "gate_proj.weight.0.bin"), hidden, I, L.expGateUp.p, l * 2 * I, hidden);
        denseLoad(ep + (mix ? "w2.0.bin" : "up_proj.weight.0.bin"), hidden, I, L.expGateUp.p, l * 2 * I + I, hidden);
        denseLoad(ep + (mix ? "w3.0.bin" : "down_proj.weight.0.bin"), I, hidden, L.expDown.p, l * hidden, I);
      }
      // quantised weight types: the experts take the VALUES of the quantised weights and stay bf16 on the device (the
      // grouped GEMM multiplies bf16), as in the Python engine; the attention projections are quantised for real.  A
      // hybrid type keeps a second stack for the decode steps.
      if (wqNext != wq) {
        const size_t gu = (size_t)EL * 2 * I * hidden * 2, dn = (size_t)EL * hidden * I * 2;
        L.expGateUpNext.reset(gu);
        L.expDownNext.reset(dn);
        XFT_CUDA(cudaMemcpy(L.expGateUpNext.p, L.expGateUp.p, gu, cudaMemcpyDeviceToDevice));
        XFT_CUDA(cudaMemcpy(L.expDownNext.p, L.expDown.p, dn, cudaMemcpyDeviceToDevice));
        if (wqNext) {
          requantiseRows(L.expGateUpNext, (size_t)EL * 2 * I, hidden, wqNext);
          requantiseRows(L.expDownNext, (size_t)EL * hidden, I, wqNext);
        }
      }
      if (wq) {
        requantiseRows(L.expGateUp, (size_t)EL * 2 * I, hidden, wq);
        requantiseRows(L.expDown, (size_t)EL * hidden, I, wq);
      }
    } else if (spec.mlp == 1) {
      if (!gptq) L.gateUp.reset((size_t)inter * hidden * 2);
      denseLoad(p + "mlp.dense_h_to_4h.weight.0.bin", hidden, interG, L.gateUp.p, 0, hidden, i0, i0 + inter);
      L.fc1Bias = loadVector(p + "mlp.dense_h_to_4h.bias.0.bin", interG, false, -1, i0, i0 + inter);
      if (rank == 0) L.fc2Bias = loadVector(p + "mlp.dense_4h_to_h.bias.bin", hidden);
    } else {
      if (!gptq) L.gateUp.reset((size_t)2 * inter * hidden * 2);
      if (spec.mlp == 2) {
        // gate rows, then up rows, in one tensor
        denseLoad(p + "mlp.dense_h_to_4h.weight.0.bin", hidden, 2 * interG, L.gateUp.p, 0, hidden, i0, i0 + inter);
        denseLoad(p + "mlp.dense_h_to_4h.weight.0.bin", hidden, 2 * interG, L.gateUp.p, inter, hidden, interG + i0, interG + i0 + inter);
      } else {
        denseLoad(p + "mlp.gate_proj.weight.0.bin", hidden, interG, L.gateUp.p, 0, hidden, i0, i0 + inter);
        denseLoad(p + "mlp.up_proj.weight.0.bin", hidden, interG, L.gateUp.p, inter, hidden, i0, i0 + inter);
      }
    }
    if (spec.mlp != 3) {
      if (!gptq) L.down.reset((size_t)hidden * inter * 2);
      denseLoad(p + (spec.mlp == 0 ? "mlp.down_proj.weight.0.bin" : "mlp.dense_4h_to_h.weight.0.bin"), interG, hidden,
                 L.down.p, 0, inter, 0, hidden, i0, i0 + inter);
    }
    L.n1 = loadVector(p + "input_layernorm.weight.bin", hidden);
    L.n2 = loadVector(p + "post_attention_layernorm.weight.bin", hidden);
    if (spec.layerNorm) {
      L.n1b = loadVector(p + "input_layernorm.bias.bin", hidden);
      L.n2b = loadVector(p + "post_attention_layernorm.bias.bin", hidden);
    }
    if (qkNorm) {
      L.qNorm = loadVector(p + "attention.q_norm.weight.bin", headDim);
      L.kNorm = loadVector(p + "attention.k_norm.weight.bin", headDim);
    }
    LayerLins& Q = lins[i];
    LayerLins& Qn = linsNext[i];
    if (gptq) { loadGptqLayer(p, Q, Qn); continue; }
    quantise(L.qkv, qsz + 2 * kvsz, hidden, Q.qkv, Qn.qkv);
    quantise(L.o, hidden, qsz, Q.o, Qn.o);
    if (spec.mlp != 3) {
      quantise(L.gateUp, spec.mlp == 1 ? inter : 2 * inter, hidden, Q.gateUp, Qn.gateUp);
      quantise(L.down, hidden, inter, Q.down, Qn.down);
    }
  }
  // rotary table [maxPos, rotDim] = cos(rotDim/2) ‖ sin(rotDim/2); the NTK families build further tables on demand
  if (rotDim > 0 && !spec.telechatNtk) {
    const std::vector<float> tab = ropeTable(maxPos, rotDim, ropeTheta, rs);
    ropeTable_.reset(tab.size() * 4);
    XFT_CUDA(cudaMemcpy(ropeTable_.p, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice));
  }
  if (alibi) {
    const std::vector<float> sl = alibiSlopes(headsG);          // this rank's heads take their own slopes
    slopes_.reset((size_t)heads * 4);
    XFT_CUDA(cudaMemcpy(slopes_.p, sl.data() + q0, (size_t)heads * 4, cudaMemcpyHostToDevice));
  }
  ws.reset(kWsBytes);
  counters.reset(8192 * 4); XFT_CUDA(cudaMemset(counters.p, 0, counters.bytes));
  attnCounters.reset(16384 * 4); XFT_CUDA(cudaMemset(attnCounters.p, 0, attnCounters.bytes));
  status.reset(16); XFT_CUDA(cudaMemset(status.p, 0, 16));
  tables.reset(new BlockTables(kBlock, 0));
  kc.resize(layers); vc.resize(layers); ks.resize(layers); vs.resize(layers);
  rng.seed((unsigned long long)std::chrono::steady_clock::now().time_since_epoch().count());
  if (Env::get().kvCacheGb > 0) {
    // XFT_KV_CACHE_GB: size the KV pools once, so that they never grow (and move) under load
    const size_t per = (size_t)(l1 - l0) * (kvBlockBytes() * (spec.mla ? 1 : 2) + (kvInt8 ? (size_t)kvHeads * kBlock * 8 : 0));
    ensureBlocks((int)std::max<size_t>(1, (size_t)(Env::get().kvCacheGb * (double)(1ull << 30)) / per));
  }
}

// Tensor dumps for debugging (reference: src/utils/debugger.h, dumpMatrix calls compiled in with -DDEBUG).  Here a run-time
// switch, with the names and the log line of the Python engine (utils/debugger.py) so that the two can be compared file
// by file: <dir>/rank<r>_step<k>_<name>.bin holds the first 64 rows as fp32, <dir>/rank<r>.log one summary line each.
void Engine::dumpState(const std::string& name, const void* state, int T) {
  const std::string& d = Env::get().debugDir;
  if (d.empty()) return;
  const int rows = std::min(T, 64);
  std::vector<uint16_t> raw((size_t)rows * hidden);
  XFT_CUDA(cudaStreamSynchronize(st));
  XFT_CUDA(cudaMemcpy(raw.data(), state, raw.size() * 2, cudaMemcpyDeviceToHost));
  std::vector<float> v(raw.size());
  double sum = 0, amax = 0;
  for (size_t i = 0; i < raw.size(); ++i) { v[i] = bf16ToFloat(raw[i]); sum += v[i]; amax = std::max(amax, (double)std::fabs(v[i])); }
  const std::string base = d + "/rank" + std::to_string(worldRank);
  {
    std::ofstream f(base + "_step" + std::to_string(debugStep) + "_" + name + ".bin", std::ios::binary | std::ios::trunc);
    if (!f) throw std::runtime_error("XFT_DEBUG_DIR: cannot write under " + d);
    f.write(reinterpret_cast<const char*>(v.data()), (std::streamsize)(v.size() * 4));
  }
  char line[512];
  std::string first;
  for (size_t i = 0; i < std::min<size_t>(6, v.size()); ++i) { char b[32]; std::snprintf(b, sizeof(b), "%s%.5g", i ? ", " : "", v[i]); first += b; }
  std::snprintf(line, sizeof(line), "step %lld %s: shape (%d, %d) dtype bf16 mean %.6g absmax %.6g first [%s]\n", debugStep, name.c_str(),
                T, hidden, raw.empty() ? 0.0 : sum / (double)raw.size(), amax, first.c_str());
  std::ofstream log(base + ".log", std::ios::app);
  log << line;
}

// Every row of a bf16 matrix [rows, K] is replaced by its quantised-and-restored value under the weight type `kind`
// (per output channel, the formulas of xft_quantize_rows: asymmetric int8, asymmetric uint4, NF4), on the host.
void Engine::requantiseRows(DevBuf& w, size_t rows, int K, int kind) {
  static const float nf4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                                0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
  const int mode = kind == 3 ? 2 : kind == 4 ? 1 : 0;
  const size_t chunk = std::max<size_t>(1, ((size_t)64 << 20) / ((size_t)K * 2));      // 64 MiB of rows at a time
  std::vector<uint16_t> host;
  for (size_t r0 = 0; r0 < rows; r0 += chunk) {
    const size_t n = std::min(chunk, rows - r0);
    host.resize(n * K);
    char* dev = static_cast<char*>(w.p) + r0 * K * 2;
    XFT_CUDA(cudaMemcpy(host.data(), dev, n * K * 2, cudaMemcpyDeviceToHost));
    // rows are independent: spread them over the host cores
    const unsigned workers = (unsigned)std::min<size_t>(std::max(1u, std::thread::hardware_concurrency()), std::max<size_t>(1, n / 64));
    auto work = [&](size_t first, size_t last) {
      std::vector<float> v(K);
      for (size_t r = first; r < last; ++r) {
        uint16_t* row = host.data() + r * K;
        float mx = -INFINITY, mn = INFINITY;
        for (int i = 0; i < K; ++i) {
          v[i] = bf16ToFloat(row[i]);
          mx = std::max(mx, mode == 2 ? std::fabs(v[i]) : v[i]);
          mn = std::min(mn, v[i]);
        }
        if (mode == 0) {
          const float sc = std::max((mx - mn) / 255.0f, 1e-10f), zp = (mx + mn) * 0.5f + 0.5f * sc;
          for (int i = 0; i < K; ++i) row[i] = floatToBf16(std::min(std::max(std::nearbyint((v[i] - zp) / sc), -128.f), 127.f) * sc + zp);
        } else if (mode == 1) {
          const float sc = std::max((mx - mn) / 15.0f, 1e-10f);
          for (int i = 0; i < K; ++i) row[i] = floatToBf16(std::min(std::max(std::nearbyint((v[i] - mn) / sc), 0.f), 15.f) * sc + mn);
        } else {
          const float sc = std::max(mx, 1e-10f);
          for (int i = 0; i < K; ++i) {
            const float xn = v[i] / sc;
            int best = 0;
            float bd = std::fabs(xn - nf4[0]);
            for (int c = 1; c < 16; ++c) { const float d = std::fabs(xn - nf4[c]); if (d < bd) { bd = d; best = c; } }
            row[i] = floatToBf16(nf4[best] * sc);
          }
        }
      }
    };
    if (workers <= 1) {
      work(0, n);
    } else {
      std::vector<std::thread> pool;
      for (unsigned w = 0; w < workers; ++w) pool.emplace_back(work, n * w / workers, n * (w + 1) / workers);
      for (auto& t : pool) t.join();
    }
    XFT_CUDA(cudaMemcpy(dev, host.data(), n * K * 2, cudaMemcpyHostToDevice));
  }
}

void Engine::loadDsLinear(const std::string& base, int inF, int outF, void* dst, int dstRowOffset, int dstLd, int o0, int o1,
                          int c0, int c1) {
  // the file holds [in, out]; the device wants rows [o0, o1) of the transpose with columns [c0, c1) (a tensor-parallel
  // slice), written at row `dstRowOffset` of a matrix whose rows are dstLd long
  if (o1 < 0) o1 = outF;
  if (c1 < 0) c1 = inF;
  const bool whole = o0 == 0 && o1 == outF && c0 == 0 && c1 == inF;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(dst) + (size_t)dstRowOffset * dstLd;
  DevBuf full;
  __nv_bfloat16* target = out;
  int targetLd = dstLd;
  if (!whole) { full.reset((size_t)outF * inF * 2); target = full.as<__nv_bfloat16>(); targetLd = inF; }
  if (fileDt != 3 || Env::get().fakeModel) {
    const int dt = fileDt == 3 ? 2 : fileDt;
    auto host = readFile(dir + "/" + base + ".weight.bin", (size_t)inF * outF * dtypeSize(dt), dt);
    DevBuf tmp(host.size());
    XFT_CUDA(cudaMemcpy(tmp.p, host.data(), host.size(), cudaMemcpyHostToDevice));
    XFT_K(xft_transpose_to_bf16(tmp.p, dt, outF, inF, outF, target, targetLd, st));
    XFT_CUDA(cudaStreamSynchronize(st));
  } else {
    // e4m3 bytes [in, out] + one fp32 scale per 128 x 128 block (deepseek_moe_convert.py:117-180): dequantise on the
    // device, then transpose like every other tensor
    const int B = 128, sr = (inF + B - 1) / B, sc = (outF + B - 1) / B;
    std::ifstream f(dir + "/" + base + ".weight.bin", std::ios::binary | std::ios::ate);
    if (!f) throw std::runtime_error("cannot open " + base + ".weight.bin");
    if ((size_t)f.tellg() != (size_t)inF * outF) throw std::runtime_error(base + ".weight.bin: unexpected size");
    std::vector<char> w((size_t)inF * outF);
    f.seekg(0);
    f.read(w.data(), (std::streamsize)w.size());
    auto scales = readFile(dir + "/" + base + ".weight_scale_inv.bin", (size_t)sr * sc * 4, 0);
    DevBuf dw(w.size()), ds(scales.size()), dense((size_t)inF * outF * 2);
    XFT_CUDA(cudaMemcpy(dw.p, w.data(), w.size(), cudaMemcpyHostToDevice));
    XFT_CUDA(cudaMemcpy(ds.p, scales.data(), scales.size(), cudaMemcpyHostToDevice));
    XFT_K(xft_fp8_block_dequant(dw.p, ds.as<float>(), inF, outF, B, dense.p, st));
    XFT_K(xft_transpose_to_bf16(dense.p, 2, outF, inF, outF, target, targetLd, st));
    XFT_CUDA(cudaStreamSynchronize(st));
  }
  if (!whole) {
    XFT_CUDA(cudaMemcpy2DAsync(out, (size_t)dstLd * 2, target + (size_t)o0 * inF + c0, (size_t)inF * 2, (size_t)(c1 - c0) * 2,
                               (size_t)(o1 - o0), cudaMemcpyDeviceToDevice, st));
    XFT_CUDA(cudaStreamSynchronize(st));
  }
}

void Engine::loadMlaLayer(const std::string& p, LayerWeights& L, int layer) {
  const int qk = nope + ropeD, H = hidden, kvw = kvLora + ropeD;
  // merged down-projection: the query part (compressed to q_lora, or this rank's heads * qk when the model has no query
  // compression) followed by compressed KV + shared rotary key (src/layers/attn_deepseek.h:78-117).  With several ranks
  // the compressed parts are computed by every rank; what follows them is split by query head.
  const int qRows = qLora > 0 ? qLora : heads * qk;
  L.qkvA.reset((size_t)(qRows + kvw) * H * 2);
  if (qLora > 0) loadDsLinear(p + "self_attn.q_a_proj", H, qLora, L.qkvA.p, 0, H);
  else loadDsLinear(p + "self_attn.q_a_proj", H, headsG * qk, L.qkvA.p, 0, H, q0 * qk, (q0 + heads) * qk);
  loadDsLinear(p + "self_attn.kv_a_proj_with_mqa", H, kvw, L.qkvA.p, qRows, H);
  if (qLora > 0) {
    L.qANorm = loadVector(p + "self_attn.q_a_layernorm.weight.bin", qLora, false, 2);
    L.qB.reset((size_t)heads * qk * qLora * 2);
    loadDsLinear(p + "self_attn.q_b_proj", qLora, headsG * qk, L.qB.p, 0, qLora, q0 * qk, (q0 + heads) * qk);
  }
  L.kvANorm = loadVector(p + "self_attn.kv_a_layernorm.weight.bin", kvLora, false, 2);
  // kv_b [kv_lora -> heads * (nope + v)] as [out, in]; per head the first `nope` rows are W_uk, the next `v` rows W_uv.
  // The absorbed form multiplies queries by W_uk^T and latent outputs by W_uv (attn_deepseek.h:408-433), so W_uk is
  // stored transposed per head and both are stacked for the per-head grouped GEMM.
  {
    DevBuf kvb((size_t)heads * (nope + vDim) * kvLora * 2);
    loadDsLinear(p + "self_attn.kv_b_proj", kvLora, headsG * (nope + vDim), kvb.p, 0, kvLora, q0 * (nope + vDim),
                 (q0 + heads) * (nope + vDim));
    L.wkT.reset((size_t)heads * kvLora * nope * 2);
    L.wv.reset((size_t)heads * vDim * kvLora * 2);
    for (int h = 0; h < heads; ++h) {
      const __nv_bfloat16* src = kvb.as<__nv_bfloat16>() + (size_t)h * (nope + vDim) * kvLora;
      XFT_K(xft_transpose_to_bf16(src, 2, kvLora, nope, kvLora, L.wkT.as<__nv_bfloat16>() + (size_t)h * kvLora * nope, nope, st));
      XFT_CUDA(cudaMemcpyAsync(L.wv.as<__nv_bfloat16>() + (size_t)h * vDim * kvLora, src + (size_t)nope * kvLora,
                               (size_t)vDim * kvLora * 2, cudaMemcpyDeviceToDevice, st));
    }
    XFT_CUDA(cudaStreamSynchronize(st));
  }
  L.o.reset((size_t)H * heads * vDim * 2);
  loadDsLinear(p + "attention.dense", headsG * vDim, H, L.o.p, 0, heads * vDim, 0, H, q0 * vDim, (q0 + heads) * vDim);
  L.n1 = loadVector(p + "input_layernorm.weight.bin", H, false, 2);
  L.n2 = loadVector(p + "post_attention_layernorm.weight.bin", H, false, 2);
  L.denseMlp = layer < firstDense;
  // a gated MLP of whole width IG of which this rank keeps columns [c, c + I)
  auto gatedMlp = [&](const std::string& base, int IG, int c, int I, DevBuf& gu, DevBuf& dn) {
    gu.reset((size_t)2 * I * H * 2);
    loadDsLinear(base + "gate_proj", H, IG, gu.p, 0, H, c, c + I);
    loadDsLinear(base + "up_proj", H, IG, gu.p, I, H, c, c + I);
    dn.reset((size_t)H * I * 2);
    loadDsLinear(base + "down_proj", IG, H, dn.p, 0, I, 0, H, c, c + I);
  };
  if (L.denseMlp) { gatedMlp(p + "mlp.", interG, i0, inter, L.gateUp, L.down); return; }
  const int E = experts, I = moeInter;
  {
    // router [hidden, experts] bf16 on disk
    auto host = readFile(dir + "/" + p + "mlp.gate.weight.bin", (size_t)H * E * 2, 2);
    DevBuf tmp(host.size());
    XFT_CUDA(cudaMemcpy(tmp.p, host.data(), host.size(), cudaMemcpyHostToDevice));
    L.router.reset((size_t)E * H * 2);
    XFT_K(xft_transpose_to_bf16(tmp.p, 2, E, H, E, L.router.p, H, st));
    XFT_CUDA(cudaStreamSynchronize(st));
  }
  L.routerBias = loadVector(p + "mlp.gate.e_score_correction_bias.bin", E, true, 2);
  if (sharedInter > 0) gatedMlp(p + "mlp.shared_experts.", sharedInterG, s0, sharedInter, L.sharedGateUp, L.sharedDown);
  const int EL = e1 - e0;
  // e4m3 files whose sizes fit the grouped e4m3 GEMM (whole 128 x 128 blocks) keep the experts in e4m3: half the bytes of
  // bf16 on the device and in every decode step (XFT_FP8_EXPERTS=0 dequantises them like the other tensors)
  const char* fp8Env = std::getenv("XFT_FP8_EXPERTS");
  L.fp8Experts = fileDt == 3 && !Env::get().fakeModel && I % 128 == 0 && H % 128 == 0 && !(fp8Env && *fp8Env == '0');
  if (L.fp8Experts) {
    const size_t guRows = (size_t)EL * 2 * I, dnRows = (size_t)EL * H;
    const int guBlocks = H / 128, dnBlocks = I / 128;                 // scale columns: blocks along the reduction
    std::vector<uint8_t> gu(guRows * H), dn(dnRows * I);
    std::vector<float> gus(guRows / 128 * guBlocks), dns(dnRows / 128 * dnBlocks);
    for (int e = e0; e < e1; ++e) {
      const std::string ep = p + "mlp.experts." + std::to_string(e) + ".";
      const size_t l = (size_t)(e - e0);
      loadFp8Expert(ep + "gate_proj", H, I, gu.data() + l * 2 * I * H, gus.data() + l * (2 * I / 128) * guBlocks);
      loadFp8Expert(ep + "up_proj", H, I, gu.data() + (l * 2 * I + I) * H, gus.data() + (l * (2 * I / 128) + I / 128) * guBlocks);
      loadFp8Expert(ep + "down_proj", I, H, dn.data() + l * H * I, dns.data() + l * (H / 128) * dnBlocks);
    }
    L.expGateUp.reset(gu.size()); L.expDown.reset(dn.size());
    L.expGateUpScale.reset(gus.size() * 4); L.expDownScale.reset(dns.size() * 4);
    XFT_CUDA(cudaMemcpy(L.expGateUp.p, gu.data(), gu.size(), cudaMemcpyHostToDevice));
    XFT_CUDA(cudaMemcpy(L.expDown.p, dn.data(), dn.size(), cudaMemcpyHostToDevice));
    XFT_CUDA(cudaMemcpy(L.expGateUpScale.p, gus.data(), gus.size() * 4, cudaMemcpyHostToDevice));
    XFT_CUDA(cudaMemcpy(L.expDownScale.p, dns.data(), dns.size() * 4, cudaMemcpyHostToDevice));
    return;
  }
  L.expGateUp.reset((size_t)EL * 2 * I * H * 2);
  L.expDown.reset((size_t)EL * H * I * 2);
  for (int e = e0; e < e1; ++e) {
    const std::string ep = p + "mlp.experts." + std::to_string(e) + ".";
    const int l = e - e0;
    loadDsLinear(ep + "gate_proj", H, I, L.expGateUp.p, l * 2 * I, H);
    loadDsLinear(ep + "up_proj", H, I, L.expGateUp.p, l * 2 * I + I, H);
    loadDsLinear(ep + "down_proj", I, H, L.expDown.p, l * H, I);
  }
}

// One expert matrix of an e4m3 checkpoint: the file holds bytes [in, out] and fp32 scales [in / 128, out / 128]; the device
// wants rows of outputs — bytes [out, in], scales [out / 128, in / 128] — written at `bytes` / `scales` (rows contiguous).
void Engine::loadFp8Expert(const std::string& base, int inF, int outF, uint8_t* bytes, float* scales) {
  std::ifstream f(dir + "/" + base + ".weight.bin", std::ios::binary | std::ios::ate);
  if (!f) throw std::runtime_error("cannot open " + base + ".weight.bin");
  if ((size_t)f.tellg() != (size_t)inF * outF) throw std::runtime_error(base + ".weight.bin: unexpected size");
  std::vector<uint8_t> w((size_t)inF * outF);
  f.seekg(0);
  f.read(reinterpret_cast<char*>(w.data()), (std::streamsize)w.size());
  constexpr int T = 64;                       // transpose in tiles: both sides stay in cache
  for (int i0 = 0; i0 < inF; i0 += T)
    for (int o0 = 0; o0 < outF; o0 += T)
      for (int i = i0; i < std::min(i0 + T, inF); ++i)
        for (int o = o0; o < std::min(o0 + T, outF); ++o) bytes[(size_t)o * inF + i] = w[(size_t)i * outF + o];
  const int sr = inF / 128, sc = outF / 128;
  auto s = readFile(dir + "/" + base + ".weight_scale_inv.bin", (size_t)sr * sc * 4, 0);
  const float* sv = reinterpret_cast<const float*>(s.data());
  for (int i = 0; i < sr; ++i)
    for (int o = 0; o < sc; ++o) scales[(size_t)o * sr + i] = sv[(size_t)i * sc + o];
}

void Engine::loadGptqLayer(const std::string& p, LayerLins& first, LayerLins& next) {
  const int qszG = headsG * headDim, kvszG = kvHeadsG * headDim, qkvG = qszG + 2 * kvszG;
  const int qsz = heads * headDim, kvsz = kvHeads * headDim;
  const int kOff = qszG + kv0 * headDim, vOff = qszG + kvszG + kv0 * headDim;
  const std::string qkv = p + "attention.query_key_value";
  loadGptq({{qkv, qkvG, q0 * headDim, q0 * headDim + qsz}, {qkv, qkvG, kOff, kOff + kvsz}, {qkv, qkvG, vOff, vOff + kvsz}}, hidden, 0,
           hidden, first.qkv, next.qkv);
  loadGptq({{p + "attention.dense", hidden, 0, hidden}}, qszG, q0 * headDim, q0 * headDim + qsz, first.o, next.o);
  loadGptq({{p + "mlp.gate_proj", interG, i0, i0 + inter}, {p + "mlp.up_proj", interG, i0, i0 + inter}}, hidden, 0, hidden,
           first.gateUp, next.gateUp);
  loadGptq({{p + "mlp.down_proj", hidden, 0, hidden}}, interG, i0, i0 + inter, first.down, next.down);
}

void Engine::loadGptq(const std::vector<GptqPart>& parts, int inF, int n0, int n1, Lin& first, Lin& next) {
  const bool u4 = gptq == 2;
  const int K = n1 - n0;
  int rows = 0;
  for (auto& pt : parts) rows += pt.o1 - pt.o0;
  if (u4 && (K % 2)) throw std::runtime_error("uint4 GPTQ tensors need an even input range");
  struct Host { std::vector<char> q; std::vector<float> s, z; };
  std::vector<Host> host(parts.size());
  for (size_t i = 0; i < parts.size(); ++i) {
    const GptqPart& pt = parts[i];
    if (u4 && (pt.outF % 2)) throw std::runtime_error("uint4 GPTQ tensors need an even output dimension");
    // (the last argument only matters for XFT_FAKE_MODEL, which has no meaning for a quantised checkpoint)
    host[i].q = readFile(dir + "/" + pt.base + ".qweight.0.bin", u4 ? (size_t)inF * pt.outF / 2 : (size_t)inF * pt.outF, 1);
    auto sb = readFile(dir + "/" + pt.base + ".scales.0.bin", (size_t)pt.outF * 4, 0);
    auto zb = readFile(dir + "/" + pt.base + ".zeros.0.bin", (size_t)pt.outF * 4, 0);
    host[i].s.resize(pt.outF); host[i].z.resize(pt.outF);
    std::memcpy(host[i].s.data(), sb.data(), sb.size());
    std::memcpy(host[i].z.data(), zb.data(), zb.size());
  }
  auto upload = [&](DevBuf& d, const void* src, size_t bytes) {
    d.reset(bytes);
    XFT_CUDA(cudaMemcpy(d.p, src, bytes, cudaMemcpyHostToDevice));
  };
  int denseAt = -1;                       // index into gptqDense of this projection's dequantised copy, made on demand
  auto build = [&](int kind, Lin& out) {
    const bool direct = (gptq == 1 && (kind == 1 || kind == 2)) || (gptq == 2 && kind == 4);
    if (direct) {
      // the stored codes are what the GEMM of this weight type reads: repack [in, out] -> [out, in] rows and keep them
      out.rows = rows; out.K = K; out.kind = kind;
      const size_t rowBytes = ((u4 ? (size_t)K / 2 : (size_t)K) + 15) / 16 * 16;
      out.pitch = (int)rowBytes;
      std::vector<uint8_t> codes((size_t)rows * rowBytes);
      std::vector<float> sc(rows), zp(rows), sums(kind == 2 ? rows : 0);
      int r = 0;
      for (size_t i = 0; i < parts.size(); ++i) {
        const GptqPart& pt = parts[i];
        const uint8_t* f = reinterpret_cast<const uint8_t*>(host[i].q.data());
        gptqRepack(f, inF, pt.outF, u4, n0, n1, pt.o0, pt.o1, (int)rowBytes, codes.data() + (size_t)r * rowBytes);
        if (kind == 2) gptqRowSums(f, inF, pt.outF, u4, n0, n1, pt.o0, pt.o1, sums.data() + r);
        std::copy(host[i].s.begin() + pt.o0, host[i].s.begin() + pt.o1, sc.begin() + r);
        std::copy(host[i].z.begin() + pt.o0, host[i].z.begin() + pt.o1, zp.begin() + r);
        r += pt.o1 - pt.o0;
      }
      upload(out.q, codes.data(), codes.size());
      upload(out.scale, sc.data(), sc.size() * 4);
      upload(out.zero, zp.data(), zp.size() * 4);
      if (kind == 2) upload(out.wsum, sums.data(), sums.size() * 4);
      return;
    }
    // another weight type was asked for: dequantise (w = q * scale + zero) and go the way of a dense checkpoint
    if (denseAt < 0) {
      std::vector<float> f32((size_t)rows * K);
      int r = 0;
      for (size_t i = 0; i < parts.size(); ++i) {
        const GptqPart& pt = parts[i];
        gptqDequant(reinterpret_cast<const uint8_t*>(host[i].q.data()), inF, pt.outF, u4, n0, n1, pt.o0, pt.o1, host[i].s.data(),
                    host[i].z.data(), f32.data() + (size_t)r * K);
        r += pt.o1 - pt.o0;
      }
      std::vector<uint16_t> b16(f32.size());
      for (size_t i = 0; i < f32.size(); ++i) b16[i] = floatToBf16(f32[i]);
      gptqDense.emplace_back();
      upload(gptqDense.back(), b16.data(), b16.size() * 2);
      denseAt = (int)gptqDense.size() - 1;
    }
    quantiseAs(gptqDense[denseAt], rows, K, kind, out);
  };
  build(wq, first);
  if (wqNext != wq) build(wqNext, next);
  if (denseAt >= 0 && wq != 0 && wqNext != 0) gptqDense.pop_back();      // no bf16 projection points at it
}

void Engine::quantise(DevBuf& dense, int rows, int K, Lin& first, Lin& next) {
  quantiseAs(dense, rows, K, wq, first);
  if (wqNext != wq) quantiseAs(dense, rows, K, wqNext, next);
  if (wq != 0 && wqNext != 0) dense.reset(0);
}

void Engine::quantiseAs(const DevBuf& dense, int rows, int K, int kind, Lin& out) {
  out.rows = rows; out.K = K; out.kind = kind;
  if (kind == 0) { out.w = dense.p; return; }
  // the quantiser of the loader (same kernel as the Python package uses): per output channel, asymmetric int8 / uint4
  // or NF4
  const bool nibbles = kind == 3 || kind == 4;
  if (nibbles && (K % 2)) throw std::runtime_error("4-bit weights need even input dimensions");
  if (kind == 2 && (K % 16)) throw std::runtime_error("w8a8 weights need input dimensions that are multiples of 16");
  // rows start on 16-byte boundaries (the GEMM reads them with TMA); codes in the padding are zero and meet
  // zero-filled activations
  const size_t rowBytes = ((nibbles ? (size_t)K / 2 : (size_t)K) + 15) / 16 * 16;
  out.pitch = (int)rowBytes;
  out.q.reset((size_t)rows * rowBytes);
  XFT_CUDA(cudaMemsetAsync(out.q.p, 0, (size_t)rows * rowBytes, st));
  out.scale.reset((size_t)rows * 4); out.zero.reset((size_t)rows * 4);
  if (kind == 2) out.wsum.reset((size_t)rows * 4);
  XFT_K(xft_quantize_rows(dense.p, 2, K, rows, K, kind == 3 ? 2 : kind == 4 ? 1 : 0, out.q.p, (long long)rowBytes,
                          out.scale.as<float>(), out.zero.as<float>(), out.wsum.as<float>(), st));
  XFT_CUDA(cudaStreamSynchronize(st));
}

const float* Engine::ropeFor(int maxKv, int maxQ) {
  if (rotDim <= 0) return nullptr;
  double theta = ropeTheta;
  if (spec.lognNtk) {
    // Qwen-1 (src/layers/rotary_embedding_qwen.cpp:33-135): contexts within the training length use the base table
    if (!useDynamicNtk || maxKv <= trainLen) return ropeTable_.as<float>();
    theta = qwenNtkTheta(ropeTheta, rotDim, maxKv, trainLen);
  } else if (spec.telechatNtk) {
    theta = telechatNtkTheta(ropeTheta, rotDim, maxKv, trainLen);
  } else {
    return ropeTable_.as<float>();
  }
  const long long key = std::llround(theta);
  auto it = ntkTables_.find(key);
  if (it == ntkTables_.end()) {
    RopeScaling rs;
    // TeleChat scales a table by 0.1 ln(input / training) + 1 when it is first built during a pass with a longer
    // input than the training length, and keeps it (src/layers/rotary_embedding_telechat.cpp:68-117)
    if (spec.telechatNtk) rs.tableScale = telechatMscale(maxQ, trainLen);
    const std::vector<float> tab = ropeTable(maxPos, rotDim, theta, rs);
    DevBuf d(tab.size() * 4);
    XFT_CUDA(cudaMemcpy(d.p, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice));
    it = ntkTables_.emplace(key, std::move(d)).first;
  }
  return it->second.as<float>();
}

void Engine::ensureBlocks(int extra) {
  auto& al = tables->allocator();
  if (al.numFree() >= extra) return;
  const int total = std::max(al.numBlocks() - al.numFree() + extra, al.numBlocks() * 3 / 2);
  const size_t per = kvBlockBytes(), sper = (size_t)kvHeads * kBlock * 4;
  for (int l = l0; l < l1; ++l) {
    DevBuf nk(per * total), nv(spec.mla ? 0 : per * total);
    // new blocks start zeroed: the TMA decode kernel reads whole tiles and masks rows past kv_len by P = 0,
    // which needs the masked V rows to be finite
    XFT_CUDA(cudaMemset(nk.as<char>() + per * numBlocks, 0, per * (total - numBlocks)));
    if (!spec.mla) XFT_CUDA(cudaMemset(nv.as<char>() + per * numBlocks, 0, per * (total - numBlocks)));
    if (numBlocks) {
      XFT_CUDA(cudaMemcpy(nk.p, kc[l].p, per * numBlocks, cudaMemcpyDeviceToDevice));
      if (!spec.mla) XFT_CUDA(cudaMemcpy(nv.p, vc[l].p, per * numBlocks, cudaMemcpyDeviceToDevice));
    }
    kc[l] = std::move(nk); vc[l] = std::move(nv);
    if (kvInt8) {
      DevBuf a(sper * total), b(sper * total);
      if (numBlocks) {
        XFT_CUDA(cudaMemcpy(a.p, ks[l].p, sper * numBlocks, cudaMemcpyDeviceToDevice));
        XFT_CUDA(cudaMemcpy(b.p, vs[l].p, sper * numBlocks, cudaMemcpyDeviceToDevice));
      }
      ks[l] = std::move(a); vs[l] = std::move(b);
    }
  }
  numBlocks = total;
  al.grow(total);
}

void Engine::copyBlock(int src, int dst) {
  const size_t per = kvBlockBytes(), sper = (size_t)kvHeads * kBlock * 4;
  for (int l = l0; l < l1; ++l) {
    XFT_CUDA(cudaMemcpyAsync(kc[l].as<char>() + per * dst, kc[l].as<char>() + per * src, per, cudaMemcpyDeviceToDevice, st));
    if (spec.mla) continue;
    XFT_CUDA(cudaMemcpyAsync(vc[l].as<char>() + per * dst, vc[l].as<char>() + per * src, per, cudaMemcpyDeviceToDevice, st));
    if (kvInt8) {
      XFT_CUDA(cudaMemcpyAsync(ks[l].as<char>() + sper * dst, ks[l].as<char>() + sper * src, sper, cudaMemcpyDeviceToDevice, st));
      XFT_CUDA(cudaMemcpyAsync(vs[l].as<char>() + sper * dst, vs[l].as<char>() + sper * src, sper, cudaMemcpyDeviceToDevice, st));
    }
  }
}

void Engine::attachPrefix(SequenceMeta& s) {
  if (prefixSeq < 0) return;
  const SequenceMeta& pre = pool.get(prefixSeq);
  const size_t n = pre.prompt.size();
  if (s.prompt.size() > n && std::equal(pre.prompt.begin(), pre.prompt.end(), s.prompt.begin())) {
    tables->fork(prefixSeq, s.id);
    s.pastLen = (int)n;
    s.pending.assign(s.prompt.begin() + n, s.prompt.end());
  }
}

// One forward pass, cut into groups of whole sequences where that is asked for (as the Python engine cuts it):
//  * XFT_MAX_BATCH_TOKENS: when the pending tokens of several sequences exceed the budget, the sequences run in groups of
//    at most that many tokens, each a ragged batch of its own, so the activation buffers stay bounded;
//  * over pipeline stages, XFT_MAX_REQUEST_NUM micro-batches: a stage hands micro-batch m on and starts on m + 1 while
//    the next stage works on m (the sends are asynchronous on the stream).
// The logits of the groups are put together in the order of the sequences; over pipeline stages the last stage collects
// them and every rank receives them once, at the end.
int Engine::forward(const std::vector<int>& seqIds, bool logitsAll) {
  std::vector<std::vector<int>> groups(1, seqIds);
  const long long cap = Env::get().maxBatchTokens;
  long long pendingTokens = 0;
  bool prompt = false;
  for (int sid : seqIds) { const size_t n = pool.get(sid).pending.size(); pendingTokens += (long long)n; prompt = prompt || n > 1; }
  if (seqIds.size() > 1 && cap > 0 && pendingTokens > cap && prompt) {
    groups.assign(1, {});
    long long n = 0;
    for (int sid : seqIds) {
      const long long mine = (long long)pool.get(sid).pending.size();
      if (!groups.back().empty() && n + mine > cap) { groups.emplace_back(); n = 0; }
      groups.back().push_back(sid);
      n += mine;
    }
  }
  const int micro = pp > 1 ? std::min<int>(Env::get().maxRequestNum, (int)seqIds.size()) : 1;
  if (groups.size() == 1 && micro > 1) {
    groups.clear();
    for (int m = 0; m < micro; ++m)
      groups.emplace_back(seqIds.begin() + seqIds.size() * m / micro, seqIds.begin() + seqIds.size() * (m + 1) / micro);
  }
  if (groups.size() == 1) return forwardPart(seqIds, logitsAll, true);
  std::vector<float> all;
  int rows = 0;
  for (const auto& g : groups) {
    const int r = forwardPart(g, logitsAll, false);
    if (ppRank == pp - 1) all.insert(all.end(), hostLogits.begin(), hostLogits.begin() + (size_t)r * vocabG);
    rows += r;
  }
  hostLogits.swap(all);
  hostLogits.resize((size_t)rows * vocabG);
  if (pp > 1) worldComm->broadcastHost(hostLogits.data(), hostLogits.size() * 4, (pp - 1) * world);
  return rows;
}

int Engine::forwardPart(const std::vector<int>& seqIds, bool logitsAll, bool shareLogits) {
  TimeLine tl("Decoder.forward");
  const auto t_begin = std::chrono::steady_clock::now();
  struct StepLog {
    const std::chrono::steady_clock::time_point t0; size_t n;
    ~StepLog() {
      if (Env::get().verbose >= 1)
        log(LogLevel::Info, "forward: %zu sequences, %.3f ms", n,
            std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count());
    }
  } step_log{t_begin, seqIds.size()};
  std::vector<int> ids, pos, pos2, prefix, slots, cu{0}, kvl, rowsel;
  bool decode = true;
  int maxQ = 0, maxKv = 0;
  for (int sid : seqIds) {
    SequenceMeta& s = pool.get(sid);
    const int n = (int)s.pending.size();
    if (n == 0) throw std::runtime_error("sequence " + std::to_string(sid) + " has no pending input");
    if (tables->len(sid) > s.pastLen) tables->truncate(sid, s.pastLen);
    ensureBlocks((s.pastLen + n + kBlock - 1) / kBlock + 1);
    auto sl = tables->append(sid, n, [&](int a, int b) { copyBlock(a, b); });
    if (spec.rope2d) {
      // ChatGLM-1 (src/models/chatglm.cpp:118-206): the position runs up to the [gMASK] / [MASK] slot and stays there
      // from the bos token on; the block position is 0 in the context and counts 1, 2, ... from bos
      const int kGmask = 130001, kMask = 130000, kBos = 130004;
      const auto& pr = s.prompt;
      auto find = [&](int tok) { auto it = std::find(pr.begin(), pr.end(), tok); return it == pr.end() ? -1 : (int)(it - pr.begin()); };
      const int bos = find(kBos);
      const int ctxLen = bos >= 0 ? bos : (int)pr.size() - 1;
      int maskPos = find(kGmask);
      if (maskPos < 0) maskPos = find(kMask);
      if (maskPos < 0) maskPos = ctxLen;
      for (int i = 0; i < n; ++i) {
        const int p = s.pastLen + i;
        pos.push_back(p < ctxLen ? p : maskPos);
        pos2.push_back(p < ctxLen ? 0 : p - ctxLen + 1);
      }
      prefix.push_back(ctxLen);
    } else {
      for (int i = 0; i < n; ++i) pos.push_back(s.pastLen + i);
    }
    for (int i = 0; i < n; ++i) { ids.push_back(s.pending[i]); slots.push_back(sl[i]); }
    cu.push_back(cu.back() + n);
    kvl.push_back(s.pastLen + n);
    if (n != 1) decode = false;
    maxQ = std::max(maxQ, n);
    maxKv = std::max(maxKv, s.pastLen + n);
    if (logitsAll) for (int i = cu[cu.size() - 2]; i < cu.back(); ++i) rowsel.push_back(i);
    else rowsel.push_back(cu.back() - 1);
    if (s.pastLen + n > maxPos || (wpeRows > 0 && s.pastLen + n > wpeRows - 2))
      throw std::runtime_error("sequence exceeds max_pos_seq_len");
  }
  const int T = (int)ids.size(), B = (int)seqIds.size(), R = (int)rowsel.size();
  size_t W = 1;
  for (int sid : seqIds) W = std::max(W, tables->table(sid).size());
  std::vector<int> bt((size_t)B * W, 0);
  for (int b = 0; b < B; ++b) { auto& t = tables->table(seqIds[b]); std::copy(t.begin(), t.end(), bt.begin() + (size_t)b * W); }
  auto up = [&](DevBuf& d, const std::vector<int>& v) {
    d.ensure(v.size() * 4 + 16);
    XFT_CUDA(cudaMemcpyAsync(d.p, v.data(), v.size() * 4, cudaMemcpyHostToDevice, st));
  };
  up(dIds, ids); up(dPos, pos); up(dSlots, slots); up(dCu, cu); up(dKv, kvl); up(dBt, bt); up(rows, rowsel);
  if (spec.rope2d) { up(dPos2, pos2); up(dPrefix, prefix); }
  const float* table = ropeFor(maxKv, maxQ);
  const float* qScale = nullptr;
  std::vector<float> qs;
  if (spec.lognNtk && useLognAttn && maxKv > trainLen) {
    // Qwen-1 log-n attention: queries beyond the training length are scaled by log(position + 1) / log(training length)
    qs.resize(pos.size());
    for (size_t i = 0; i < qs.size(); ++i) qs[i] = std::max(1.0f, std::log((float)pos[i] + 1.0f) / std::log((float)trainLen));
    dQScale.ensure(qs.size() * 4 + 16);
    XFT_CUDA(cudaMemcpyAsync(dQScale.p, qs.data(), qs.size() * 4, cudaMemcpyHostToDevice, st));
    qScale = dQScale.as<float>();
  }
  XFT_CUDA(cudaStreamSynchronize(st));   // host vectors go out of scope after this call
  const int qsz = heads * headDim, kvsz = kvHeads * headDim, qkvN = qsz + 2 * kvsz;
  x.ensure((size_t)T * hidden * 2); x2.ensure((size_t)T * hidden * 2); h.ensure((size_t)T * hidden * 2);
  qkvBuf.ensure((size_t)T * qkvN * 2); q.ensure((size_t)T * qsz * 2); att.ensure((size_t)T * qsz * 2);
  g.ensure((size_t)T * std::max(inter, 1) * 2);
  int* stp = status.as<int>();
  auto gemm = [&](const void* X, int K, const void* Wt, int wRows, void* Y, int N, int fp32, int gated, int dualOff,
                  const float* bias, const void* res, int actc, int rowsT) {
    VerboseCall v(st, "gemm_bf16", rowsT, gated ? 2 * N : N, K);
    XFT_K(xft_gemm_bf16(X, K, Wt, wRows, K, Y, N, fp32, rowsT, N, K, gated, dualOff, bias, res, N, 1.0f, actc, nullptr,
                        ws.as<float>(), kWsBytes, counters.as<int>(), 8192, stp, 0, st));
  };
  if (ppRank == 0)
    XFT_K(xft_embedding(dIds.as<int>(), wte.p, x.p, T, hidden, vocabG, embedScale, wpe.p, wpe.p ? dPos.as<int>() : nullptr, 2,
                        wpeRows, stp, st));
  const int group = groupG;
  int nsplit = 1;
  if (decode) {
    // bf16 caches run the TMA-ring kernel (64-key tiles, two CTAs per SM); int8 caches the cp.async kernel
    const int kt = !kvInt8 ? 64 : headDim == 64 ? 64 : headDim == 128 ? 32 : 16;
    const int slots = kvInt8 ? 444 : headDim <= 128 ? 296 : 148;
    const int ntiles = (maxKv + kt - 1) / kt, ctas = B * kvHeads * ((group + 15) / 16);
    nsplit = std::max(1, std::min({slots / std::max(ctas, 1), ntiles >= 16 ? ntiles / 8 : 1, 32}));
    if (ctas > 16384) nsplit = 1;
    if (nsplit > 1) { partO.ensure((size_t)B * heads * nsplit * headDim * 4); partMl.ensure((size_t)B * heads * nsplit * 8); }
  }
  const float scale = 1.0f / std::sqrt((float)headDim);
  auto norm = [&](const void* in, const DevBuf& w, const DevBuf& b, void* out, int rowsT) {
    if (spec.layerNorm) XFT_K(xft_layernorm(in, hidden, w.as<float>(), b.as<float>(), out, hidden, rowsT, hidden, eps, st));
    else XFT_K(xft_rmsnorm(in, hidden, nullptr, 0, w.as<float>(), out, hidden, nullptr, rowsT, hidden, eps, st));
  };
  // ChatGLM-1 adds sqrt(2 * layers) times the NORMALISED input instead of the block input (src/models/chatglm.cpp)
  const float resScale = spec.residFromNorm ? std::sqrt(2.0f * (float)layers) : 1.0f;
  // one layer projection in whichever form its weights have: Y[T, N] = epilogue(X[T, K] · W^T); `gated`: W holds gate rows
  // then up rows and Y = act(gate) * up
  auto lin = [&](const Lin& Wt, const void* X, void* Y, int N, int gated, const float* bias, const void* res, float rscale,
                 int actc) {
    const int K = Wt.K;
    VerboseCall v(st, Wt.kind == 0 ? "gemm_bf16" : Wt.kind == 2 ? "gemm_w8a8" : Wt.kind == 3 ? "gemm_nf4" : Wt.kind == 4 ? "gemm_int4" : "gemm_int8",
                  T, gated ? 2 * N : N, K);
    if (Wt.kind == 0) {
      XFT_K(xft_gemm_bf16(X, K, Wt.w, Wt.rows, K, Y, N, 0, T, N, K, gated, gated ? N : 0, bias, res, N, rscale, actc, nullptr,
                          ws.as<float>(), kWsBytes, counters.as<int>(), 8192, stp, 0, st));
    } else if (Wt.kind == 2) {
      // dynamic per-token int8 activations, int8 tensor-core product, corrections for both zero points in the epilogue
      actQ.ensure((size_t)T * K); actScale.ensure((size_t)T * 4); actZero.ensure((size_t)T * 4); actSum.ensure((size_t)T * 4);
      XFT_K(xft_quant_act(X, K, actQ.p, K, actScale.as<float>(), actZero.as<float>(), actSum.as<float>(), T, K, st));
      void* out = Y;
      if (gated) { guBuf.ensure((size_t)T * 2 * N * 2); out = guBuf.p; }
      const int n = gated ? 2 * N : N;
      XFT_K(xft_w8a8_gemm(actQ.p, K, Wt.q.p, Wt.pitch, out, n, 0, T, n, K, actScale.as<float>(), actZero.as<float>(),
                          actSum.as<float>(), Wt.scale.as<float>(), Wt.zero.as<float>(), Wt.wsum.as<float>(), bias,
                          gated ? nullptr : res, N, rscale, gated ? 0 : actc, ws.as<float>(), kWsBytes, counters.as<int>(), 8192,
                          stp, st));
      if (gated) XFT_K(xft_gated_act(guBuf.p, Y, T, N, actc, st));
    } else {
      const bool nf4 = Wt.kind == 3;
      const float* xsum = nullptr;
      if (!nf4) {      // an asymmetric zero point contributes zero * sum(x) per output
        actSum.ensure((size_t)T * 4);
        XFT_K(xft_row_sum(X, K, actSum.as<float>(), T, K, st));
        xsum = actSum.as<float>();
      }
      XFT_K(xft_qgemm(X, K, Wt.q.p, Wt.rows, Wt.pitch, nf4 ? 2 : Wt.kind == 4 ? 1 : 0, Y, N, 0, T, N, K, gated, gated ? N : 0,
                      Wt.scale.as<float>(), nf4 ? nullptr : Wt.zero.as<float>(), xsum, 0, bias, res, N, rscale, actc,
                      ws.as<float>(), kWsBytes, counters.as<int>(), 8192, stp, st));
    }
  };
  int moeBn = 16, moeMaxTiles = 0;
  if (spec.mlp == 3) {
    const int rowsMax = T * topK, avg = std::max(1, (rowsMax + experts - 1) / experts);
    moeBn = avg <= 16 ? 16 : avg <= 32 ? 32 : avg <= 64 ? 64 : 128;      // token tile of the grouped GEMMs
    moeMaxTiles = (rowsMax + moeBn - 1) / moeBn + experts;
    moeLogits.ensure((size_t)T * experts * 4); moeIdx.ensure((size_t)rowsMax * 4); moeWts.ensure((size_t)rowsMax * 4);
    moePos.ensure((size_t)rowsMax * 4); moeSrc.ensure((size_t)rowsMax * 4); moeRowW.ensure((size_t)rowsMax * 4);
    moeTiles.ensure((size_t)moeMaxTiles * 16); moeMeta.ensure(8);
    moeXs.ensure((size_t)rowsMax * hidden * 2); moeH1.ensure((size_t)rowsMax * moeInter * 2);
    moeYs.ensure((size_t)rowsMax * hidden * 4);
  }
  // DeepSeek: static tile table of the per-head grouped GEMMs (rows of head h are [h * T, (h + 1) * T)), split factor of
  // the latent attention at decode sizes
  int mlaTiles = 0, mlaBn = 16, mlaSplit = 1;
  if (spec.mla) {
    const int L = kvLora, qk = nope + ropeD, qRows = qLora > 0 ? qLora : heads * qk;
    mlaBn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : 128;
    std::vector<int> tiles;
    for (int hh = 0; hh < heads; ++hh)
      for (int j = 0; j < T; j += mlaBn) { tiles.push_back(hh); tiles.push_back(hh * T + j); tiles.push_back(std::min(mlaBn, T - j)); tiles.push_back(0); }
    mlaTiles = (int)tiles.size() / 4;
    const int meta[2] = {mlaTiles, heads * T};
    mTiles.ensure(tiles.size() * 4); mMeta.ensure(8);
    XFT_CUDA(cudaMemcpyAsync(mTiles.p, tiles.data(), tiles.size() * 4, cudaMemcpyHostToDevice, st));
    XFT_CUDA(cudaMemcpyAsync(mMeta.p, meta, 8, cudaMemcpyHostToDevice, st));
    XFT_CUDA(cudaStreamSynchronize(st));
    mQaKv.ensure((size_t)T * (qRows + L + ropeD) * 2); mQa.ensure((size_t)T * std::max(qLora, 8) * 2);
    mQ.ensure((size_t)T * heads * qk * 2); mQNope.ensure((size_t)heads * T * nope * 2);
    mQRope.ensure((size_t)T * heads * ropeD * 2); mQAbs.ensure((size_t)heads * T * L * 2);
    mOLat.ensure((size_t)heads * T * L * 2); mOHead.ensure((size_t)heads * T * vDim * 2);
    att.ensure((size_t)T * heads * vDim * 2);
    g.ensure((size_t)T * std::max(inter, std::max(sharedInter, 8)) * 2);
    if (sharedInter > 0) mShared.ensure((size_t)T * hidden * 4);
    if (decode) {
      const int ntiles = (maxKv + 31) / 32, ctas = T * ((heads + 15) / 16);
      mlaSplit = std::max(1, std::min({296 / std::max(ctas, 1), ntiles >= 16 ? ntiles / 8 : 1, 16}));
      if (mlaSplit > 1 && ctas <= 16384) {
        partO.ensure((size_t)ctas * mlaSplit * 16 * L * 4);
        partMl.ensure((size_t)ctas * mlaSplit * 32 * 4);
      } else {
        mlaSplit = 1;
      }
    }
  }
  auto perHead = [&](const void* X, int K, const void* Wst, int nOut, void* Y) {
    // X [heads * T, K] (rows grouped by head) x per-head weights [heads * nOut, K] -> Y [heads * T, nOut]
    XFT_K(xft_gemm_bf16_grouped(X, K, heads * T, Wst, heads * nOut, K, Y, nOut, 0, nOut, K, 0, 0, nOut, mTiles.p,
                                mMeta.as<int>(), mlaTiles, mlaBn, nullptr, 0, stp, st));
  };
  // three state buffers of T x hidden; which one plays which part rotates in the ChatGLM-1 flow
  void* cur = x.p;
  void* nxt = x2.p;
  void* hb = h.p;
  if (ppRank > 0) worldComm->recvBf16(cur, (size_t)T * hidden, worldRank - world, st);      // the state the stage before left
  const bool dbg = !Env::get().debugDir.empty();
  if (dbg) { ++debugStep; if (ppRank == 0) dumpState("embedding", cur, T); }
  auto dumpLayer = [&](int l, const char* what, const void* state) {
    if (dbg) dumpState("layer" + std::to_string(l) + "_" + what, state, T);
  };
  for (int l = l0; l < l1; ++l) {
    LayerWeights& L = lw[l];
    norm(cur, L.n1, L.n1b, hb, T);
    if (spec.mla) {
      // ---- latent attention (src/layers/attn_deepseek.h): down-projections, query up-projection, one kernel for the
      // head split + KV norm + rotary + cache append, then the absorbed form: q W_uk^T against the latent cache, the
      // latent result times W_uv, output projection
      const int Lr = kvLora, qk = nope + ropeD, qRows = qLora > 0 ? qLora : heads * qk, ldA = qRows + Lr + ropeD;
      gemm(hb, hidden, L.qkvA.p, ldA, mQaKv.p, ldA, 0, 0, 0, nullptr, nullptr, 0, T);
      const __nv_bfloat16* qPtr = mQaKv.as<__nv_bfloat16>();
      int ldq = ldA;
      if (qLora > 0) {
        XFT_K(xft_rmsnorm(mQaKv.p, ldA, nullptr, 0, L.qANorm.as<float>(), mQa.p, qLora, nullptr, T, qLora, eps, st));
        gemm(mQa.p, qLora, L.qB.p, heads * qk, mQ.p, heads * qk, 0, 0, 0, nullptr, nullptr, 0, T);
        qPtr = mQ.as<__nv_bfloat16>();
        ldq = heads * qk;
      }
      XFT_K(xft_mla_prep(qPtr, ldq, mQaKv.as<__nv_bfloat16>() + qRows, ldA, T, heads, nope, ropeD, Lr, dPos.as<int>(), table,
                         maxPos, L.kvANorm.as<float>(), eps, mQNope.p, mQRope.p, kc[l].p, (long long)numBlocks * kBlock,
                         dSlots.as<int>(), stp, 1, st));
      perHead(mQNope.p, nope, L.wkT.p, Lr, mQAbs.p);
      XFT_K(xft_mla_attention(mQAbs.p, (long long)T * Lr, Lr, mQRope.p, ropeD, (long long)heads * ropeD, mOLat.p,
                              (long long)T * Lr, Lr, kc[l].p, dBt.as<int>(), (int)W, dCu.as<int>(), dKv.as<int>(), B, T, heads,
                              kBlock, numBlocks, attnScale, mlaSplit, mlaSplit > 1 ? partO.as<float>() : nullptr,
                              mlaSplit > 1 ? partMl.as<float>() : nullptr, attnCounters.as<int>(), stp, st));
      perHead(mOLat.p, Lr, L.wv.p, vDim, mOHead.p);
      XFT_K(xft_swap_outer_dims(mOHead.p, att.p, heads, T, vDim, st));          // [heads, T, v] -> [T, heads * v]
      // row-parallel with several ranks: the residual enters on rank 0, the ranks' products are added
      gemm(att.p, heads * vDim, L.o.p, hidden, nxt, hidden, 0, 0, 0, nullptr, rank == 0 ? cur : nullptr, 0, T);
      if (comm) comm->allReduceBf16(nxt, (size_t)T * hidden, st);
      dumpLayer(l, "attn_out", nxt);
      norm(nxt, L.n2, L.n2b, hb, T);
      if (L.denseMlp) {
        gemm(hb, hidden, L.gateUp.p, 2 * inter, g.p, inter, 0, 1, inter, nullptr, nullptr, act, T);
        gemm(g.p, inter, L.down.p, hidden, cur, hidden, 0, 0, 0, nullptr, rank == 0 ? nxt : nullptr, 0, T);
        if (comm) comm->allReduceBf16(cur, (size_t)T * hidden, st);
        dumpLayer(l, "ffn_out", cur);
        continue;
      }
      // ---- shared + routed experts (src/layers/moe_deepseek.h:121-196,285-353)
      const int E = experts, k = topK, I = moeInter;
      gemm(hb, hidden, L.router.p, E, moeLogits.p, E, 1, 0, 0, nullptr, nullptr, 0, T);
      XFT_K(xft_moe_route(moeLogits.as<float>(), E, T, E, k, 2, L.routerBias.as<float>(), nGroup, topkGroup, routedScale,
                          normTopk ? 1 : 0, sigmoidScores ? 1 : 0, moeIdx.as<int>(), moeWts.as<float>(), st));
      // several ranks: rows only for this rank's experts [e0, e1), a column slice of the shared experts, sums added
      const int EL = e1 - e0;
      XFT_K(xft_moe_plan(moeIdx.as<int>(), moeWts.as<float>(), T, k, e0, e1, moeBn, moePos.as<int>(), moeSrc.as<int>(),
                         moeRowW.as<float>(), moeTiles.p, moeMeta.as<int>(), moeMaxTiles, T * k, st));
      XFT_K(xft_moe_gather(hb, hidden, moeSrc.as<int>(), moeMeta.as<int>(), moeXs.p, T * k, hidden, st));
      if (L.fp8Experts) {
        XFT_K(xft_qgemm_grouped(moeXs.p, hidden, T * k, L.expGateUp.p, EL * 2 * I, hidden, moeH1.p, I, 0, I, hidden, 1, I, 2 * I,
                                L.expGateUpScale.as<float>(), hidden / 128, moeTiles.p, moeMeta.as<int>(), moeMaxTiles, moeBn,
                                nullptr, 2, stp, st));
        XFT_K(xft_qgemm_grouped(moeH1.p, I, T * k, L.expDown.p, EL * hidden, I, moeYs.p, hidden, 1, hidden, I, 0, 0, hidden,
                                L.expDownScale.as<float>(), I / 128, moeTiles.p, moeMeta.as<int>(), moeMaxTiles, moeBn,
                                moeRowW.as<float>(), 0, stp, st));
      } else {
        XFT_K(xft_gemm_bf16_grouped(moeXs.p, hidden, T * k, L.expGateUp.p, EL * 2 * I, hidden, moeH1.p, I, 0, I, hidden, 1, I,
                                    2 * I, moeTiles.p, moeMeta.as<int>(), moeMaxTiles, moeBn, nullptr, 2, stp, st));
        XFT_K(xft_gemm_bf16_grouped(moeH1.p, I, T * k, L.expDown.p, EL * hidden, I, moeYs.p, hidden, 1, hidden, I, 0, 0, hidden,
                                    moeTiles.p, moeMeta.as<int>(), moeMaxTiles, moeBn, moeRowW.as<float>(), 0, stp, st));
      }
      const float* sharedOut = nullptr;
      if (sharedInter > 0) {
        gemm(hb, hidden, L.sharedGateUp.p, 2 * sharedInter, g.p, sharedInter, 0, 1, sharedInter, nullptr, nullptr, 2, T);
        gemm(g.p, sharedInter, L.sharedDown.p, hidden, mShared.p, hidden, 1, 0, 0, nullptr, nullptr, 0, T);
        sharedOut = mShared.as<float>();
      }
      XFT_K(xft_moe_combine(moeYs.as<float>(), moePos.as<int>(), k, sharedOut, rank == 0 ? nxt : nullptr, hidden, cur, nullptr, T,
                            hidden, st));
      if (comm) comm->allReduceBf16(cur, (size_t)T * hidden, st);
      dumpLayer(l, "ffn_out", cur);
      continue;
    }
    const LayerLins& Q = (decode && wqNext != wq) ? linsNext[l] : lins[l];
    lin(Q.qkv, hb, qkvBuf.p, qkvN, 0, L.qkvBias.as<float>(), nullptr, 1.0f, 0);
    if (spec.rope2d) {
      XFT_K(xft_qkv_rope2d_cache(qkvBuf.p, qkvN, T, heads, kvHeads, headDim, dPos.as<int>(), dPos2.as<int>(), table, rotDim,
                                 maxPos, q.p, kc[l].p, vc[l].p, ks[l].as<float>(), vs[l].as<float>(), kvInt8 ? 1 : 0, kBlock,
                                 (long long)numBlocks * kBlock, dSlots.as<int>(), stp, st));
    } else {
      XFT_K(xft_qkv_rope_cache(qkvBuf.p, qkvN, T, heads, kvHeads, headDim, dPos.as<int>(), table, rotDim, spec.ropeStyle, 0,
                               maxPos, qScale, L.qNorm.as<float>(), L.kNorm.as<float>(), eps, q.p, kc[l].p, vc[l].p,
                               ks[l].as<float>(), vs[l].as<float>(), kvInt8 ? 1 : 0, kBlock, (long long)numBlocks * kBlock,
                               dSlots.as<int>(), stp, st));
    }
    XFT_K(xft_paged_attention(q.p, att.p, kc[l].p, vc[l].p, ks[l].as<float>(), vs[l].as<float>(), dBt.as<int>(), (int)W,
                              dCu.as<int>(), dKv.as<int>(), B, maxQ, heads, kvHeads, group, qOff, headDim, kBlock, numBlocks,
                              scale, slopes_.as<float>(), spec.prefixLm ? dPrefix.as<int>() : nullptr, decode ? 1 : 0, nsplit,
                              partO.as<float>(), partMl.as<float>(), attnCounters.as<int>(), stp, st));
    // attention output projection (+ bias) + residual
    // row-parallel: every rank multiplies its slice; residual (and bias) enter on rank 0 only, then the ranks' results
    // are summed (src/layers/decoder_block.h:122-134 reduceAdd)
    lin(Q.o, att.p, nxt, hidden, 0, L.oBias.as<float>(), rank == 0 ? (spec.residFromNorm ? hb : cur) : nullptr, resScale, 0);
    if (comm) comm->allReduceBf16(nxt, (size_t)T * hidden, st);
    dumpLayer(l, "attn_out", nxt);
    // ChatGLM-1 needs the normalised state again as the residual of the MLP: it goes to `cur`, whose content (the
    // block input) is no longer needed; every other family normalises into the scratch buffer
    void* hn = spec.residFromNorm ? cur : hb;
    norm(nxt, L.n2, L.n2b, hn, T);
    if (spec.mlp == 3) {
      // router logits (fp32) -> top-k experts and weights -> rows grouped by expert -> two grouped GEMMs (the second
      // scales each row by its routing weight) -> per-token sum + residual
      const int E = experts, k = topK, I = moeInter;
      gemm(hn, hidden, L.router.p, E, moeLogits.p, E, 1, 0, 0, nullptr, nullptr, 0, T);
      XFT_K(xft_moe_route(moeLogits.as<float>(), E, T, E, k, spec.routeKind, nullptr, 1, 1, 1.0f, 1, 1, moeIdx.as<int>(),
                          moeWts.as<float>(), st));
      // with several ranks: only the pairs of this rank's experts [e0, e1) get rows; the residual enters on rank 0 and
      // the ranks' sums are added
      const int EL = e1 - e0;
      XFT_K(xft_moe_plan(moeIdx.as<int>(), moeWts.as<float>(), T, k, e0, e1, moeBn, moePos.as<int>(), moeSrc.as<int>(),
                         moeRowW.as<float>(), moeTiles.p, moeMeta.as<int>(), moeMaxTiles, T * k, st));
      XFT_K(xft_moe_gather(hn, hidden, moeSrc.as<int>(), moeMeta.as<int>(), moeXs.p, T * k, hidden, st));
      const bool nextStack = decode && wqNext != wq;
      const void* wGateUp = nextStack ? L.expGateUpNext.p : L.expGateUp.p;
      const void* wDown = nextStack ? L.expDownNext.p : L.expDown.p;
      XFT_K(xft_gemm_bf16_grouped(moeXs.p, hidden, T * k, wGateUp, EL * 2 * I, hidden, moeH1.p, I, 0, I, hidden, 1, I,
                                  2 * I, moeTiles.p, moeMeta.as<int>(), moeMaxTiles, moeBn, nullptr, act, stp, st));
      XFT_K(xft_gemm_bf16_grouped(moeH1.p, I, T * k, wDown, EL * hidden, I, moeYs.p, hidden, 1, hidden, I, 0, 0, hidden,
                                  moeTiles.p, moeMeta.as<int>(), moeMaxTiles, moeBn, moeRowW.as<float>(), 0, stp, st));
      XFT_K(xft_moe_combine(moeYs.as<float>(), moePos.as<int>(), k, nullptr, rank == 0 ? nxt : nullptr, hidden, cur, nullptr, T,
                            hidden, st));
      if (comm) comm->allReduceBf16(cur, (size_t)T * hidden, st);
      dumpLayer(l, "ffn_out", cur);
      continue;
    }
    if (spec.mlp == 1) {
      lin(Q.gateUp, hn, g.p, inter, 0, L.fc1Bias.as<float>(), nullptr, 1.0f, act);
    } else {
      lin(Q.gateUp, hn, g.p, inter, 1, nullptr, nullptr, 1.0f, act);
    }
    if (spec.residFromNorm) {
      lin(Q.down, g.p, hb, hidden, 0, L.fc2Bias.as<float>(), rank == 0 ? hn : nullptr, resScale, 0);   // into the scratch, which becomes the state
      if (comm) comm->allReduceBf16(hb, (size_t)T * hidden, st);
      std::swap(cur, hb);
    } else {
      lin(Q.down, g.p, cur, hidden, 0, L.fc2Bias.as<float>(), rank == 0 ? nxt : nullptr, resScale, 0);    // + residual, back into `cur`
      if (comm) comm->allReduceBf16(cur, (size_t)T * hidden, st);
    }
    dumpLayer(l, "ffn_out", cur);
  }
  int hs = 0;
  const bool lastStage = ppRank == pp - 1;
  if (!lastStage) {
    // hand the state to the same tensor-parallel rank of the next stage; the logits come back from the last one
    worldComm->sendBf16(cur, (size_t)T * hidden, worldRank + world, st);
    XFT_CUDA(cudaMemcpyAsync(&hs, stp, 4, cudaMemcpyDeviceToHost, st));
    worldComm->waitStream(st);
  }
  // rows that need logits -> final norm -> lm_head (fp32)
  if (lastStage) {
    for (int r = 0; r < R; ++r)
      XFT_CUDA(cudaMemcpyAsync(static_cast<char*>(nxt) + (size_t)r * hidden * 2, static_cast<char*>(cur) + (size_t)rowsel[r] * hidden * 2,
                               (size_t)hidden * 2, cudaMemcpyDeviceToDevice, st));
    norm(nxt, finalNorm, finalNormBias, hb, R);
  }
  if (!lastStage) {
  } else if (!comm) {
    logits.ensure((size_t)R * vocab * 4);
    gemm(hb, hidden, lmHead.p, vocab, logits.p, vocab, 1, 0, 0, nullptr, nullptr, 0, R);
    hostLogits.resize((size_t)R * vocab);
    XFT_CUDA(cudaMemcpyAsync(hostLogits.data(), logits.p, hostLogits.size() * 4, cudaMemcpyDeviceToHost, st));
    XFT_CUDA(cudaMemcpyAsync(&hs, stp, 4, cudaMemcpyDeviceToHost, st));
    // with ranks before this one (pipeline stages) the stream holds a receive: wait with the communicator's limit
    if (worldComm) worldComm->waitStream(st);
    else XFT_CUDA(cudaStreamSynchronize(st));
  } else {
    // vocabulary-parallel head (src/layers/dist_linear.h:49-101): this rank's rows of the lm_head give a slice of every
    // logits row; slices are padded to the widest rank's width, gathered, and put in order on the host
    const size_t per = (size_t)R * vocabPad;
    logits.ensure(per * 4);
    gathered.ensure(per * world * 4);
    XFT_CUDA(cudaMemsetAsync(logits.p, 0, per * 4, st));
    XFT_K(xft_gemm_bf16(hb, hidden, lmHead.p, vocab, hidden, logits.p, vocabPad, 1, R, vocab, hidden, 0, 0, nullptr, nullptr, 0,
                        1.0f, 0, nullptr, ws.as<float>(), kWsBytes, counters.as<int>(), 8192, stp, 0, st));
    comm->allGatherF32(logits.as<float>(), gathered.as<float>(), per, st);
    std::vector<float> all(per * world);
    XFT_CUDA(cudaMemcpyAsync(all.data(), gathered.p, all.size() * 4, cudaMemcpyDeviceToHost, st));
    XFT_CUDA(cudaMemcpyAsync(&hs, stp, 4, cudaMemcpyDeviceToHost, st));
    comm->waitStream(st);                  // the sums and the gather of this step: a lost rank ends the wait with an error
    hostLogits.resize((size_t)R * vocabG);
    for (int r = 0; r < world; ++r) {
      const auto vr = taskRange(vocabG, world, r);
      for (int row = 0; row < R; ++row)
        std::copy(all.begin() + r * per + (size_t)row * vocabPad, all.begin() + r * per + (size_t)row * vocabPad + (vr.second - vr.first),
                  hostLogits.begin() + (size_t)row * vocabG + vr.first);
    }
  }
  if (hs != 0) { cudaMemset(stp, 0, 4); throw std::runtime_error("kernel status " + std::to_string(hs)); }
  if (pp > 1 && shareLogits) {
    // every rank samples from the same logits: they travel from the first rank of the last stage
    hostLogits.resize((size_t)R * vocabG);
    worldComm->broadcastHost(hostLogits.data(), hostLogits.size() * 4, (pp - 1) * world);
  }
  for (int sid : seqIds) { SequenceMeta& s = pool.get(sid); s.pastLen += (int)s.pending.size(); s.pending.clear(); }
  return R;
}

// ----------------------------------------------------------------------------------------------------------------
Model::Model() {}
Model::~Model() {
  engine.reset();                 // buffers go back to the arena ...
  Arena::device().trim();         // ... and a destroyed model returns its memory to the device
}

void Model::load(const std::string& path, DataType dt, DataType kv, std::shared_ptr<Communicator> comm) {
  engine.reset(new Engine(path, dt, kv, std::move(comm)));
}
bool Model::isMaster() { return !engine || engine->worldRank == 0; }
int Model::getRank() { return engine ? engine->worldRank : 0; }
int Model::getWorldSize() { return engine ? engine->worldSize : 1; }
int Model::getVocabSize() { return engine->vocabG; }
int Model::getMaxSeqLen() { return engine->maxPos; }

void Model::config(int maxLen, int numBeams, int numBeamHypsToKeep, float lenPenalty, bool doEarlyStopping, int eosTokenId,
                   int padTokenId, bool doSample, float temperature, int topK, float topP, float repetitionPenalty,
                   const std::vector<std::vector<int>>& stopWordsList) {
  SearcherConfig c(maxLen, numBeams, numBeamHypsToKeep, lenPenalty, doEarlyStopping, eosTokenId, padTokenId, doSample,
                   temperature, topK, topP, repetitionPenalty);
  config(c, stopWordsList);
}
namespace {
// Tensor-parallel ranks run the same program (as the reference's ranks do under mpirun, src/models/models.cpp:202-253):
// what the caller passes on rank 0 is what every rank uses.  These helpers copy rank 0's arguments to the others.
void syncValue(Engine& e, void* p, size_t bytes) { if (e.worldComm) e.worldComm->broadcastHost(p, bytes); }
template <class T>
void syncVector(Engine& e, std::vector<T>& v) {
  if (!e.worldComm) return;
  long long n = (long long)v.size();
  syncValue(e, &n, sizeof(n));
  v.resize((size_t)n);
  if (n) syncValue(e, v.data(), (size_t)n * sizeof(T));
}
template <class T>
void syncNested(Engine& e, std::vector<std::vector<T>>& v) {
  if (!e.worldComm) return;
  std::vector<long long> lens;
  for (auto& r : v) lens.push_back((long long)r.size());
  syncVector(e, lens);
  std::vector<T> flat;
  for (auto& r : v) flat.insert(flat.end(), r.begin(), r.end());
  syncVector(e, flat);
  v.assign(lens.size(), {});
  size_t off = 0;
  for (size_t i = 0; i < lens.size(); ++i) { v[i].assign(flat.begin() + off, flat.begin() + off + lens[i]); off += (size_t)lens[i]; }
}

// beams other than beam 0 are extra sequences of the pool; the request's own sequence stays in `working`
void clearBeams(Engine& e) {
  for (size_t i = 0; i < e.beamSeqs.size(); ++i)
    if (std::find(e.working.begin(), e.working.end(), e.beamSeqs[i]) == e.working.end() && e.pool.has(e.beamSeqs[i]))
      e.release(e.beamSeqs[i]);
  e.beamSeqs.clear();
  e.beamPrompts.clear();
  e.scorer.reset();
}

// One beam-search step (src/searchers/beam_search.cpp:27-345): the first call prefills the prompts and forks every
// request into numBeams sequences that share its KV blocks; later calls run all beams, pick the next beams on the
// host and reorder the block tables (reference counts move, no KV data is copied until a shared tail block is written).
std::vector<int32_t> beamStep(Engine& e, const SearcherConfig& c) {
  const int nb = c.numBeams, bs = (int)e.working.size(), V = e.vocabG;
  std::vector<float> lp((size_t)bs * nb * V);
  if (!e.scorer) {
    e.forward(e.working, false);
    for (int r = 0; r < bs; ++r) {
      float* row = e.hostLogits.data() + (size_t)r * V;
      logSoftmaxRow(row, V);
      for (int j = 0; j < nb; ++j) std::copy(row, row + V, lp.begin() + ((size_t)r * nb + j) * V);
    }
    for (int r = 0; r < bs; ++r) {
      SequenceMeta& s = e.pool.get(e.working[r]);
      e.beamPrompts.push_back(s.prompt);
      e.beamSeqs.push_back(s.id);
      for (int j = 1; j < nb; ++j) {
        SequenceMeta& b = e.pool.create(s.prompt, s.maxLen);
        b.pastLen = s.pastLen;
        b.pending.clear();
        e.tables->fork(s.id, b.id);
        e.beamSeqs.push_back(b.id);
      }
    }
    e.scorer.reset(new BeamSearchScorer(bs, nb, c.lenPenalty, c.doEarlyStopping, c.eosTokenId, c.padTokenId, c.numBeamHypsToKeep));
    std::vector<int> promptLens;
    for (int id : e.working) promptLens.push_back((int)e.pool.get(id).prompt.size());
    e.scorer->setPromptLens(promptLens);
  } else {
    e.forward(e.beamSeqs, false);
    for (int i = 0; i < bs * nb; ++i) {
      float* row = e.hostLogits.data() + (size_t)i * V;
      logSoftmaxRow(row, V);
      std::copy(row, row + V, lp.begin() + (size_t)i * V);
    }
  }
  std::vector<int32_t> toks;
  std::vector<int> src;
  e.scorer->process(lp.data(), V, toks, src);
  // beams take over the history (block table + generated tokens) of their source beam, then append their token
  e.tables->reorder(e.beamSeqs, src);
  std::vector<std::vector<int32_t>> gen(e.beamSeqs.size());
  for (size_t i = 0; i < e.beamSeqs.size(); ++i) gen[i] = e.pool.get(e.beamSeqs[src[i]]).generated;
  bool full = false;
  for (size_t i = 0; i < e.beamSeqs.size(); ++i) {
    SequenceMeta& b = e.pool.get(e.beamSeqs[i]);
    b.generated = gen[i];
    b.stepForward(toks[i]);
    full = full || b.totalLen() >= b.maxLen;
  }
  if (e.scorer->isDone() || full)
    for (int id : e.beamSeqs) e.pool.get(id).done = true;
  return toks;
}
}  // namespace

void Model::config(SearcherConfig& c0, const std::vector<std::vector<int>>& sw0) {
  SearcherConfig c = c0;
  std::vector<std::vector<int>> sw = sw0;
  if (engine->worldComm) {
    // one seed for all ranks, or their samplers would pick different tokens
    if (c.doSample && c.seed == 0) c.seed = (unsigned long long)std::chrono::steady_clock::now().time_since_epoch().count() | 1ull;
    syncValue(*engine, &c, sizeof(c));
    syncNested(*engine, sw);
  }
  if (c.numBeams > 1 && c.doSample) throw std::runtime_error("beam search with sampling is not supported");
  configuration = c;
  if (configuration.eosTokenId == -1) configuration.eosTokenId = engine->endId;
  if (configuration.padTokenId == -1) configuration.padTokenId = configuration.eosTokenId;
  if (configuration.maxLen <= 0) configuration.maxLen = engine->maxPos;
  stopWords = cleanStopWords(sw, configuration.eosTokenId);
  if (c.seed) engine->rng.seed(c.seed);
}
bool Model::setStopWords(std::vector<std::vector<int>> sw) { stopWords = cleanStopWords(sw, configuration.eosTokenId); return true; }

void Model::input(std::vector<int32_t>& ids, int batch) {
  syncValue(*engine, &batch, sizeof(batch));
  syncVector(*engine, ids);
  if (batch <= 0 || ids.size() % batch) throw std::invalid_argument("input ids do not divide into the batch");
  clearBeams(*engine);
  for (int id : engine->working) engine->release(id);
  engine->working.clear();
  batchSize = batch;
  seqLen = (int)ids.size() / batch;
  for (int b = 0; b < batch; ++b) {
    std::vector<int32_t> p(ids.begin() + (size_t)b * seqLen, ids.begin() + (size_t)(b + 1) * seqLen);
    SequenceMeta& s = engine->pool.create(p, std::max(configuration.maxLen, seqLen + 1));
    engine->tables->add(s.id);
    engine->attachPrefix(s);
    engine->working.push_back(s.id);
  }
}

std::vector<int> Model::set_input(std::vector<int32_t>& ids, int batch, int maxLen, int numBeams, int numBeamHypsToKeep,
                                  float lenPenalty, bool doEarlyStopping, int eosTokenId, int padTokenId, bool doSample,
                                  float temperature, int topK, float topP, float repetitionPenalty,
                                  const std::vector<std::vector<int>>& sw) {
  config(maxLen, numBeams, numBeamHypsToKeep, lenPenalty, doEarlyStopping, eosTokenId, padTokenId, doSample, temperature, topK,
         topP, repetitionPenalty, sw);
  input(ids, batch);
  return engine->working;
}
std::vector<int> Model::set_input(std::vector<int32_t>& ids, int batch, SearcherConfig& c, const std::vector<std::vector<int>>& sw) {
  config(c, sw);
  input(ids, batch);
  return engine->working;
}
std::vector<int> Model::set_input(std::vector<std::vector<int32_t>>& ids, SearcherConfig& c, const std::vector<std::vector<int>>& sw) {
  config(c, sw);
  syncNested(*engine, ids);
  clearBeams(*engine);
  for (int id : engine->working) engine->release(id);
  engine->working.clear();
  batchSize = (int)ids.size();
  seqLen = 0;
  for (auto& p : ids) {
    SequenceMeta& s = engine->pool.create(p, std::max(configuration.maxLen, (int)p.size() + 1));
    engine->tables->add(s.id);
    engine->attachPrefix(s);
    engine->working.push_back(s.id);
    seqLen = std::max(seqLen, (int)p.size());
  }
  return engine->working;
}

std::vector<int> Model::set_input(std::vector<std::vector<int32_t>>& ids, std::vector<int> seqIDs, int maxLen) {
  std::vector<int> lens{maxLen};
  return cbSetInput(ids, seqIDs, lens);
}

// The one implementation behind the continuous-batching set_input overloads.  maxLens: empty = the model's limit, one
// value = the same for every new sequence, else one per new sequence (src/models/models.cpp:518-584).
std::vector<int> Model::cbSetInput(std::vector<std::vector<int32_t>>& ids, std::vector<int>& seqIDs, std::vector<int>& maxLens) {
  syncNested(*engine, ids);
  syncVector(*engine, seqIDs);
  syncVector(*engine, maxLens);
  if (!(maxLens.empty() || maxLens.size() == 1 || maxLens.size() == ids.size()))
    throw std::invalid_argument("maxLen: none, one, or one per sequence expected");
  engine->cbActive.clear();
  if (seqIDs.empty()) {
    for (size_t i = 0; i < ids.size(); ++i) {
      auto& p = ids[i];
      int m = maxLens.empty() ? -1 : maxLens.size() == 1 ? maxLens[0] : maxLens[i];
      m = m > 0 ? std::min(m, engine->maxPos) : engine->maxPos;
      SequenceMeta& s = engine->pool.create(p, std::max(m, (int)p.size() + 1));
      engine->tables->add(s.id);
      engine->attachPrefix(s);
      engine->cbActive.push_back(s.id);
    }
  } else {
    if (ids.size() != seqIDs.size()) throw std::invalid_argument("one next token per sequence id expected");
    for (size_t i = 0; i < seqIDs.size(); ++i) {
      SequenceMeta& s = engine->pool.get(seqIDs[i]);
      if (ids[i].size() != 1) throw std::invalid_argument("decode inputs carry exactly one token per sequence");
      s.generated.push_back(ids[i][0]);
      s.pending.assign(1, ids[i][0]);
      engine->cbActive.push_back(s.id);
    }
  }
  return engine->cbActive;
}
std::vector<int> Model::set_input(std::vector<int32_t>& ids, int batch, std::vector<int> seqIDs, int maxLen) {
  std::vector<int> lens{maxLen};
  return set_input(ids, batch, seqIDs, lens);
}
std::vector<int> Model::set_input(std::vector<int32_t>& ids, int batch, std::vector<int> seqIDs, const std::vector<int>& maxLen) {
  syncValue(*engine, &batch, sizeof(batch));
  syncVector(*engine, ids);
  if (batch <= 0 || ids.size() % batch) throw std::invalid_argument("input ids do not divide into the batch");
  const size_t n = ids.size() / batch;
  std::vector<std::vector<int32_t>> rows(batch);
  for (int b = 0; b < batch; ++b) rows[b].assign(ids.begin() + b * n, ids.begin() + (b + 1) * n);
  std::vector<int> lens = maxLen;
  return cbSetInput(rows, seqIDs, lens);
}
// prompts of different lengths in one flat vector (seqLens says where each ends); decode: one token per sequence id
std::vector<int> Model::set_input(std::vector<int32_t>& ids, std::vector<int32_t>& seqLens, std::vector<int> seqIDs,
                                  std::vector<int>& maxLen) {
  syncVector(*engine, ids);
  syncVector(*engine, seqLens);
  syncVector(*engine, seqIDs);
  std::vector<std::vector<int32_t>> rows;
  if (seqIDs.empty()) {
    size_t off = 0;
    for (int32_t n : seqLens) {
      if (n <= 0 || off + (size_t)n > ids.size()) throw std::invalid_argument("seqLens do not add up to the number of input ids");
      rows.emplace_back(ids.begin() + off, ids.begin() + off + n);
      off += (size_t)n;
    }
    if (off != ids.size()) throw std::invalid_argument("seqLens do not add up to the number of input ids");
  } else {
    for (int32_t t : ids) rows.push_back({t});
  }
  return cbSetInput(rows, seqIDs, maxLen);
}
// sequences of a continuous batch with a sampling configuration of their own call
std::vector<int> Model::set_input(std::vector<std::vector<int32_t>>& ids, std::vector<int> seqIDs, SearcherConfig& c,
                                  const std::vector<std::vector<int>>& sw) {
  config(c, sw);
  std::vector<int> lens{configuration.maxLen};
  return cbSetInput(ids, seqIDs, lens);
}
std::vector<int> Model::set_input(std::vector<std::vector<int32_t>>& ids, int maxLen, int numBeams, int numBeamHypsToKeep,
                                  float lenPenalty, bool doEarlyStopping, int eosTokenId, int padTokenId, bool doSample,
                                  float temperature, int topK, float topP, float repetitionPenalty,
                                  const std::vector<std::vector<int>>& sw) {
  SearcherConfig c(maxLen, numBeams, numBeamHypsToKeep, lenPenalty, doEarlyStopping, eosTokenId, padTokenId, doSample,
                   temperature, topK, topP, repetitionPenalty);
  return set_input(ids, c, sw);
}
void Model::createSearcher(SearcherConfig& c) { config(c); }

std::tuple<float*, int, int> Model::forward(bool logitsAll) {
  if (engine->cbActive.empty()) throw std::runtime_error("forward() before set_input()");
  const int rows = engine->forward(engine->cbActive, logitsAll);
  return std::make_tuple(engine->hostLogits.data(), rows, engine->vocabG);
}

// AbstractDecoder over a loaded model (reference: the decoder objects behind include/abstract_decoder.h, i.e.
// CommonDecoder::forward / reorderCache / setPrefix in src/models/common_decoder.h:295-590,771-850).
class ModelDecoder : public AbstractDecoder {
public:
  explicit ModelDecoder(Model& m) : model(m) {}

  std::tuple<float*, int, int> forward(int* ids, int64_t* dims, int step, bool logitsAll) override {
    const int rows = (int)(dims[0] * dims[1]), len = (int)dims[2];
    if (rows <= 0 || len <= 0) throw std::invalid_argument("decoder forward: empty input");
    Engine& e = *model.engine;
    if (step == 0) {
      for (int id : seqs) e.release(id);
      seqs.clear();
      std::vector<std::vector<int32_t>> prompts(rows);
      for (int r = 0; r < rows; ++r) prompts[r].assign(ids + (size_t)r * len, ids + (size_t)(r + 1) * len);
      seqs = model.set_input(prompts, std::vector<int>{}, -1);
    } else {
      if ((int)seqs.size() != rows) throw std::invalid_argument("decoder forward: batch differs from step 0");
      for (int r = 0; r < rows; ++r) {
        SequenceMeta& s = e.pool.get(seqs[r]);
        for (int i = 0; i < len; ++i) s.generated.push_back(ids[(size_t)r * len + i]);
        s.pending.assign(ids + (size_t)r * len, ids + (size_t)(r + 1) * len);
      }
    }
    e.forward(seqs, logitsAll);
    return std::make_tuple(e.hostLogits.data(), 0, e.vocabG);
  }

  std::tuple<float*, int, int> forward(const std::vector<int>& seqIDs, bool logitsAll) override {
    Engine& e = *model.engine;
    e.forward(seqIDs, logitsAll);
    return std::make_tuple(e.hostLogits.data(), 0, e.vocabG);
  }

  void reorderCache(int* idx, int size) override {
    if (size != (int)seqs.size()) throw std::invalid_argument("reorderCache: size differs from the running batch");
    Engine& e = *model.engine;
    std::vector<int> src(idx, idx + size);
    for (int v : src) if (v < 0 || v >= size) throw std::invalid_argument("reorderCache: index out of range");
    // rows take over the block tables (copy-on-write of a shared tail block) and the token history of their sources
    e.tables->reorder(seqs, src);
    std::vector<std::vector<int32_t>> gen(size);
    std::vector<int> past(size);
    for (int i = 0; i < size; ++i) { gen[i] = e.pool.get(seqs[src[i]]).generated; past[i] = e.pool.get(seqs[src[i]]).pastLen; }
    for (int i = 0; i < size; ++i) { e.pool.get(seqs[i]).generated = gen[i]; e.pool.get(seqs[i]).pastLen = past[i]; }
  }

  bool isMaster() override { return model.isMaster(); }
  int getRank() override { return model.getRank(); }
  int getEndId() override { return model.engine->endId; }
  void setPrefix(int* ids, int seqLen) override {
    std::vector<int32_t> v(ids, ids + seqLen);
    model.setPrefix(v);
  }
  void unsetPrefix() override { model.unsetPrefix(); }

  ~ModelDecoder() override {
    for (int id : seqs) model.engine->release(id);
  }

private:
  Model& model;
  std::vector<int> seqs;
};

std::unique_ptr<AbstractDecoder> makeDecoder(Model& model) { return std::unique_ptr<AbstractDecoder>(new ModelDecoder(model)); }

bool Model::isDone() {
  for (int id : engine->working) if (!engine->pool.get(id).done) return false;
  return true;
}

std::vector<int32_t> Model::generate() {
  TimeLine tl("Model.generate");
  if (engine->working.empty()) throw std::runtime_error("generate() before input()/set_input()");
  if (configuration.numBeams > 1) {
    if (isDone()) return std::vector<int32_t>((size_t)engine->working.size() * configuration.numBeams, configuration.eosTokenId);
    return beamStep(*engine, configuration);
  }
  std::vector<int> active;
  for (int id : engine->working) if (!engine->pool.get(id).done) active.push_back(id);
  std::vector<int32_t> out;
  if (!active.empty()) {
    engine->forward(active, false);
    std::uniform_real_distribution<float> uni(0.f, 1.f);
    const SearcherConfig& c = configuration;
    size_t r = 0;
    for (int id : active) {
      SequenceMeta& s = engine->pool.get(id);
      float* l = engine->hostLogits.data() + r++ * engine->vocabG;
      if (c.repetitionPenalty != 1.0f) {
        std::vector<int32_t> all(s.prompt);
        all.insert(all.end(), s.generated.begin(), s.generated.end());
        repetitionPenalty(l, engine->vocabG, all, c.repetitionPenalty);
      }
      int tok = c.doSample ? sampleTopKTopP(l, engine->vocabG, c.topK, c.topP, c.temperature, uni(engine->rng))
                           : argmaxFirst(l, engine->vocabG);
      s.stepForward(tok);
      // stop check (src/searchers/sampling.cpp:134-154): eos, or total_len + 1 >= max_len
      if (tok == c.eosTokenId || s.totalLen() >= s.maxLen || (!stopWords.empty() && matchStopWords(s.generated, stopWords)))
        s.done = true;
    }
  }
  for (int id : engine->working) {
    SequenceMeta& s = engine->pool.get(id);
    bool wasActive = std::find(active.begin(), active.end(), id) != active.end();
    out.push_back(wasActive ? s.generated.back() : configuration.eosTokenId);
  }
  return out;
}

std::vector<int32_t> Model::finalize() {
  if (Env::get().timeline) TimeLine::dump();       // as the reference: the trace is written when a request ends
  if (engine->scorer) {
    auto rows = engine->scorer->finalize(engine->beamPrompts, configuration.maxLen);
    std::vector<int32_t> flat;
    for (auto& r : rows) flat.insert(flat.end(), r.begin(), r.end());
    clearBeams(*engine);
    for (int id : engine->working) engine->release(id);
    engine->working.clear();
    return flat;
  }
  size_t w = 0;
  for (int id : engine->working) w = std::max<size_t>(w, engine->pool.get(id).totalLen());
  std::vector<int32_t> out;
  for (int id : engine->working) {
    SequenceMeta& s = engine->pool.get(id);
    out.insert(out.end(), s.prompt.begin(), s.prompt.end());
    out.insert(out.end(), s.generated.begin(), s.generated.end());
    out.insert(out.end(), w - s.totalLen(), configuration.padTokenId);
    engine->release(id);
  }
  engine->working.clear();
  return out;
}

bool Model::freeSeqs(std::vector<int>& seqIDs) {
  syncVector(*engine, seqIDs);
  for (int id : seqIDs)
    if (engine->pool.has(id)) engine->release(id);
  auto& a = engine->cbActive;
  a.erase(std::remove_if(a.begin(), a.end(), [&](int id) { return !engine->pool.has(id); }), a.end());
  return true;
}

void Model::setPrefix(std::vector<int32_t>& prefix) {
  syncVector(*engine, prefix);
  unsetPrefix();
  const int n = (int)prefix.size() / 64 * 64;      // whole blocks only: sharers never write into a shared block
  if (n == 0) return;
  std::vector<int32_t> p(prefix.begin(), prefix.begin() + n);
  SequenceMeta& s = engine->pool.create(p, n + 1);
  engine->tables->add(s.id);
  engine->forward({s.id}, false);
  engine->prefixSeq = s.id;
}
void Model::unsetPrefix() {
  if (engine->prefixSeq >= 0) { engine->release(engine->prefixSeq); engine->prefixSeq = -1; }
}

AutoModel::AutoModel(std::string modelPath, xft::DataType dataType, xft::DataType KVCacheDataType) {
  // launched as one process per GPU (mpirun, torchrun): the ranks find each other through NCCL
  const auto rw = rankFromEnv();
  load(modelPath, dataType, KVCacheDataType, rw.second > 1 ? makeProcessCommunicator(rw.first, rw.second) : nullptr);
}
AutoModel::AutoModel(std::string modelPath, xft::DataType dataType, xft::DataType KVCacheDataType,
                     std::shared_ptr<Communicator> comm) {
  load(modelPath, dataType, KVCacheDataType, std::move(comm));
}

}  // namespace xft

// Torch custom-class binding of the native C++ engine: torch.classes.xfastertransformer.AutoModel with the class and
// method names of the reference's binding (src/pytorch/pytorch_warpper.cpp:18-33, src/pytorch/auto_model.h), so
// scripts written against `torch.classes.xfastertransformer.AutoModel(path, dtype, kv_dtype)` keep working:
//
//   torch.ops.load_library(".../libxft_b200_torch.so")
//   m = torch.classes.xfastertransformer.AutoModel(path, "bf16", "fp16")
//   m.config(64, None, None, None, None, eos, pad, None, None, None, None, None, None)
//   m.input(ids);  while not m.is_done(): m.generate();  out = m.finalize()
//
// Everything below converts tensors to the std::vector arguments of xft::Model (csrc/api/xft/models.h) and back; the
// model itself runs on the GPU through the sm_100a kernel library.  Optional arguments follow the reference: None
// means "default".  One process drives one GPU, so get_rank() is 0 and every call is the master's call.
#include <torch/custom_class.h>
#include <torch/script.h>

#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "xft/models.h"

namespace {

xft::DataType parseWeightType(const std::string& s) {
  const xft::DataType dt = xft::dataTypeFromName(s.c_str());
  TORCH_CHECK(dt != xft::DataType::unknown && dt != xft::DataType::fp32, "unsupported data type '", s, "'");
  return dt;
}

xft::DataType parseKvType(const std::string& s) {
  if (s == "fp16" || s == "bf16") return xft::DataType::fp16;
  if (s == "int8") return xft::DataType::int8;
  TORCH_CHECK(false, "unsupported KV cache data type '", s, "'");
}

std::vector<int32_t> toInt32(const torch::Tensor& t) {
  torch::Tensor c = t.to(torch::kCPU, torch::kInt32).contiguous();
  std::vector<int32_t> v((size_t)c.numel());
  if (!v.empty()) std::memcpy(v.data(), c.data_ptr<int32_t>(), v.size() * sizeof(int32_t));
  return v;
}

std::vector<std::vector<int>> toStopWords(const torch::optional<std::vector<std::vector<int64_t>>>& opt) {
  std::vector<std::vector<int>> out;
  if (!opt.has_value()) return out;
  for (const auto& w : opt.value()) out.emplace_back(w.begin(), w.end());
  return out;
}

struct GenArgs {
  int maxLen, numBeams, numReturn, eos, pad, topK;
  float lenPenalty, temperature, topP, repetitionPenalty;
  bool earlyStopping, doSample;
};

GenArgs genArgs(torch::optional<int64_t> maxLength, torch::optional<int64_t> numBeams,
                torch::optional<int64_t> numReturnSequences, torch::optional<double> lenPenalty,
                torch::optional<bool> earlyStopping, torch::optional<int64_t> eos, torch::optional<int64_t> pad,
                torch::optional<bool> doSample, torch::optional<double> temperature, torch::optional<int64_t> topK,
                torch::optional<double> topP, torch::optional<double> repetitionPenalty) {
  TORCH_CHECK(maxLength.has_value(), "Make sure master's maxLen is not None.");
  GenArgs a;
  a.maxLen = (int)maxLength.value();
  a.numBeams = (int)numBeams.value_or(1);
  a.numReturn = (int)numReturnSequences.value_or(1);
  a.lenPenalty = (float)lenPenalty.value_or(1.0);
  a.earlyStopping = earlyStopping.value_or(false);
  a.eos = (int)eos.value_or(-1);
  a.pad = (int)pad.value_or(-1);
  a.doSample = doSample.value_or(false);
  a.temperature = (float)temperature.value_or(1.0);
  a.topK = (int)topK.value_or(50);
  a.topP = (float)topP.value_or(1.0);
  a.repetitionPenalty = (float)repetitionPenalty.value_or(1.0);
  return a;
}

}  // namespace

struct TorchAutoModel : torch::CustomClassHolder {
  TorchAutoModel(std::string modelPath, std::string dtype, std::string kvCacheDtype)
      : model(new xft::AutoModel(modelPath, parseWeightType(dtype), parseKvType(kvCacheDtype))) {}

  int64_t getRank() { return model->getRank(); }

  void input(torch::optional<torch::Tensor> inputIds) {
    TORCH_CHECK(inputIds.has_value(), "Make sure master's input is not None.");
    const torch::Tensor& t = inputIds.value();
    TORCH_CHECK(t.dim() == 2, "input ids must be [batch, seq_len]");
    tokenIds = toInt32(t);
    model->input(tokenIds, (int)t.size(0));
  }

  void config(torch::optional<int64_t> maxLength, torch::optional<int64_t> numBeams,
              torch::optional<int64_t> numReturnSequences, torch::optional<double> lenPenalty,
              torch::optional<bool> earlyStopping, torch::optional<int64_t> eos, torch::optional<int64_t> pad,
              torch::optional<bool> doSample, torch::optional<double> temperature, torch::optional<int64_t> topK,
              torch::optional<double> topP, torch::optional<double> repetitionPenalty,
              torch::optional<std::vector<std::vector<int64_t>>> stopWordsList) {
    const GenArgs a = genArgs(maxLength, numBeams, numReturnSequences, lenPenalty, earlyStopping, eos, pad, doSample,
                              temperature, topK, topP, repetitionPenalty);
    model->config(a.maxLen, a.numBeams, a.numReturn, a.lenPenalty, a.earlyStopping, a.eos, a.pad, a.doSample,
                  a.temperature, a.topK, a.topP, a.repetitionPenalty, toStopWords(stopWordsList));
  }

  void setInput(torch::optional<torch::Tensor> inputIds, torch::optional<int64_t> maxLength,
                torch::optional<int64_t> numBeams, torch::optional<int64_t> numReturnSequences,
                torch::optional<double> lenPenalty, torch::optional<bool> earlyStopping, torch::optional<int64_t> eos,
                torch::optional<int64_t> pad, torch::optional<bool> doSample, torch::optional<double> temperature,
                torch::optional<int64_t> topK, torch::optional<double> topP, torch::optional<double> repetitionPenalty,
                torch::optional<std::vector<std::vector<int64_t>>> stopWordsList) {
    TORCH_CHECK(inputIds.has_value(), "Make sure master's input is not None.");
    const torch::Tensor& t = inputIds.value();
    TORCH_CHECK(t.dim() == 2, "input ids must be [batch, seq_len]");
    const GenArgs a = genArgs(maxLength, numBeams, numReturnSequences, lenPenalty, earlyStopping, eos, pad, doSample,
                              temperature, topK, topP, repetitionPenalty);
    tokenIds = toInt32(t);
    model->set_input(tokenIds, (int)t.size(0), a.maxLen, a.numBeams, a.numReturn, a.lenPenalty, a.earlyStopping, a.eos,
                     a.pad, a.doSample, a.temperature, a.topK, a.topP, a.repetitionPenalty, toStopWords(stopWordsList));
  }

  // Continuous batching.  New prompts: `inputIds` is [batch, seq] (or 1-D with `seqLens` giving each prompt's length)
  // and `seqIDs` is None; a decode step: one token per listed sequence id.  Returns the sequence ids.
  torch::Tensor setInputCB(torch::optional<torch::Tensor> inputIds, torch::optional<torch::Tensor> seqLens,
                           torch::optional<torch::Tensor> seqIDs, torch::optional<torch::Tensor> maxLens) {
    TORCH_CHECK(inputIds.has_value(), "Make sure master's input is not None.");
    const torch::Tensor& t = inputIds.value();
    TORCH_CHECK(t.dim() == 1 || t.dim() == 2, "Make sure master's input is 1-D or 2-D.");
    std::vector<int32_t> flat = toInt32(t);
    std::vector<std::vector<int32_t>> rows;
    if (t.dim() == 2) {
      const int64_t b = t.size(0), s = t.size(1);
      for (int64_t i = 0; i < b; ++i) rows.emplace_back(flat.begin() + i * s, flat.begin() + (i + 1) * s);
    } else {
      TORCH_CHECK(seqLens.has_value(), "1-D input ids need seqLens");
      std::vector<int32_t> lens = toInt32(seqLens.value());
      size_t off = 0;
      for (int32_t n : lens) {
        TORCH_CHECK(off + (size_t)n <= flat.size(), "seqLens exceed the number of input ids");
        rows.emplace_back(flat.begin() + off, flat.begin() + off + n);
        off += (size_t)n;
      }
    }
    std::vector<int> ids;
    if (seqIDs.has_value()) {
      std::vector<int32_t> v = toInt32(seqIDs.value());
      ids.assign(v.begin(), v.end());
    }
    int maxLen = -1;
    if (maxLens.has_value() && maxLens.value().numel() > 0) {
      std::vector<int32_t> v = toInt32(maxLens.value());
      maxLen = *std::max_element(v.begin(), v.end());
    }
    std::vector<int> out = model->set_input(rows, ids, maxLen);
    torch::Tensor ret = torch::empty({(int64_t)out.size()}, torch::kInt64);
    for (size_t i = 0; i < out.size(); ++i) ret[i] = (int64_t)out[i];
    return ret;
  }

  bool isDone() { return model->isDone(); }

  // logits of the last position of every row: fp32 [batch, vocab]
  torch::Tensor forward(torch::Tensor inputIds) {
    TORCH_CHECK(inputIds.dim() == 2, "input ids must be [batch, seq_len]");
    tokenIds = toInt32(inputIds);
    model->input(tokenIds, (int)inputIds.size(0));
    return logits();
  }

  torch::Tensor forwardCB() { return logits(); }

  torch::Tensor generate() {
    std::vector<int32_t> next = model->generate();
    torch::Tensor ret = torch::empty({(int64_t)next.size()}, torch::kInt64);
    auto acc = ret.accessor<int64_t, 1>();
    for (size_t i = 0; i < next.size(); ++i) acc[i] = next[i];
    return ret.view({model->getBatchSize() > 0 ? (int64_t)model->getBatchSize() : (int64_t)next.size(), -1});
  }

  torch::Tensor finalize() {
    std::vector<int32_t> all = model->finalize();
    const int64_t rows = std::max(1, model->getBatchSize() * std::max(1, model->getConfig().numBeamHypsToKeep));
    torch::Tensor ret = torch::empty({(int64_t)all.size()}, torch::kInt64);
    auto acc = ret.accessor<int64_t, 1>();
    for (size_t i = 0; i < all.size(); ++i) acc[i] = all[i];
    return (all.size() % (size_t)rows == 0) ? ret.view({rows, -1}) : ret;
  }

  bool freeSeqs(torch::optional<torch::Tensor> seqIDs) {
    TORCH_CHECK(seqIDs.has_value(), "Make sure master's input is not None.");
    std::vector<int32_t> v = toInt32(seqIDs.value());
    std::vector<int> ids(v.begin(), v.end());
    return model->freeSeqs(ids);
  }

  void setPrefix(torch::optional<torch::Tensor> inputIds) {
    TORCH_CHECK(inputIds.has_value(), "Make sure master's input is not None.");
    std::vector<int32_t> ids = toInt32(inputIds.value());
    model->setPrefix(ids);
  }

  void unsetPrefix() { model->unsetPrefix(); }

 private:
  torch::Tensor logits() {
    auto [ptr, rows, vocab] = model->forward(false);
    TORCH_CHECK(ptr != nullptr, "forward() returned no logits");
    return torch::from_blob(ptr, {(int64_t)rows, (int64_t)vocab}, torch::kFloat32).clone();
  }

  std::unique_ptr<xft::AutoModel> model;
  std::vector<int32_t> tokenIds;
};

TORCH_LIBRARY(xfastertransformer, m) {
  m.class_<TorchAutoModel>("AutoModel")
      .def(torch::init<std::string, std::string, std::string>())
      .def("get_rank", &TorchAutoModel::getRank)
      .def("input", &TorchAutoModel::input)
      .def("config", &TorchAutoModel::config)
      .def("set_input", &TorchAutoModel::setInput)
      .def("set_input_cb", &TorchAutoModel::setInputCB)
      .def("is_done", &TorchAutoModel::isDone)
      .def("forward", &TorchAutoModel::forward)
      .def("forward_cb", &TorchAutoModel::forwardCB)
      .def("generate", &TorchAutoModel::generate)
      .def("finalize", &TorchAutoModel::finalize)
      .def("free_seqs", &TorchAutoModel::freeSeqs)
      .def("set_prefix", &TorchAutoModel::setPrefix)
      .def("unset_prefix", &TorchAutoModel::unsetPrefix);
}

// Runs the unmodified CPU code of AnishKamatam/tiny-inference-engine on a model folder and
// prints what the tests of this repository compare against:
//   ref_driver MODEL_DIR OUT_DIR  <  requests   (one line per request: N_NEW id id id ...)
// For every request i it writes OUT_DIR/logits_<i>.f32 (whole prompt in one step, logits of
// every row, through tests/support/sequence_runner.h) and OUT_DIR/hidden_<i>.f32 (the
// residual stream after each layer, from the model's layer hook), and then runs all
// requests together through Engine + BatchScheduler (8 tokens per step, 4-token pages,
// greedy) and writes the generated ids to OUT_DIR/greedy.txt.
#include <cstdio>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "backend/cpu/cpu_backend.h"
#include "engine/batch_scheduler.h"
#include "engine/engine.h"
#include "model/loader.h"
#include "model/qwen3.h"
#include "support/sequence_runner.h"

using namespace tie;

static void write_f32(const std::string& path, const std::vector<float>& v) {
  std::ofstream f(path, std::ios::binary);
  f.write(reinterpret_cast<const char*>(v.data()), static_cast<std::streamsize>(v.size() * sizeof(float)));
}

int main(int argc, char** argv) {
  if (argc != 3) return 2;
  const std::string out = argv[2];
  try {
    const LoadedModel weights = load_model(argv[1]);
    const ModelConfig& c = weights.config;
    CpuBackend backend(2);
    KVCacheConfig kc;
    kc.num_layers = int32_t(c.num_layers);
    kc.num_kv_heads = int32_t(c.num_kv_heads);
    kc.head_dim = int32_t(c.head_dim);
    kc.block_size = 4;
    kc.dtype = DType::F32;
    kc.budget_bytes = size_t{256} * 2 * size_t(c.num_layers * c.num_kv_heads * c.head_dim) * 4 * 4;
    PagedKVCache cache(backend, kc);
    const ServingConfig serving{8, 4};
    ModelLimits limits = model_limits(serving, PagedKVCache::blocks_for(c.max_position_embeddings, kc.block_size));
    limits.max_tokens_per_step = 256;
    limits.max_logit_rows = 256;
    Qwen3Model model(backend, weights, limits);

    std::vector<std::vector<int32_t>> prompts;
    std::vector<int32_t> new_tokens;
    for (std::string line; std::getline(std::cin, line);) {
      std::istringstream s(line);
      int32_t n = 0, id = 0;
      if (!(s >> n)) continue;
      new_tokens.push_back(n);
      prompts.emplace_back();
      while (s >> id) prompts.back().push_back(id);
    }

    for (size_t i = 0; i < prompts.size(); ++i) {
      std::vector<float> hidden;
      model.set_layer_hook([&](int, const Tensor& x) {
        hidden.insert(hidden.end(), x.data<float>(), x.data<float>() + x.numel());
      });
      test::SequenceRunner runner(model, cache);
      write_f32(out + "/logits_" + std::to_string(i) + ".f32", runner.step(prompts[i], true));
      write_f32(out + "/hidden_" + std::to_string(i) + ".f32", hidden);
    }
    model.set_layer_hook(nullptr);

    BatchSchedulerConfig sc;
    sc.serving = serving;
    sc.policy = OrderingPolicy::Fcfs;
    Engine engine(model, cache, std::make_unique<BatchScheduler>(cache, sc), serving, EngineConfig{});
    std::vector<int32_t> ids;
    for (size_t i = 0; i < prompts.size(); ++i) {
      SamplingParams p;
      p.max_tokens = new_tokens[i];
      ids.push_back(engine.add_request(prompts[i], p));
    }
    while (engine.has_work()) engine.step();
    std::ofstream g(out + "/greedy.txt");
    for (size_t i = 0; i < ids.size(); ++i) {
      const Sequence& s = engine.sequence(ids[i]);
      for (size_t t = size_t(s.prompt_len); t < s.tokens.size(); ++t) g << s.tokens[t] << (t + 1 < s.tokens.size() ? " " : "");
      g << "\n";
    }
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ref_driver: %s\n", e.what());
    return 1;
  }
  return 0;
}

// Runs the unmodified CPU code of AnishKamatam/tiny-inference-engine on a model folder and
// prints what the tests of this repository compare against:
//   ref_driver MODEL_DIR OUT_DIR PAGE TOKENS_PER_STEP SMALL_POOL_PAGES  <  requests
// (one line per request: N_NEW id id id ...). For every request i it writes
// OUT_DIR/logits_<i>.f32 (whole prompt in one step, logits of every row, through
// tests/support/sequence_runner.h) and OUT_DIR/hidden_<i>.f32 (the residual stream after each
// layer, from the model's layer hook). Then it runs all requests together, greedy, through the
// reference's Engine + BatchScheduler (first come first served, PAGE tokens a page,
// TOKENS_PER_STEP tokens a step) twice: with 256 pages -> OUT_DIR/greedy.txt, and with
// SMALL_POOL_PAGES pages and no watermark (admission may use the last free page), so few that
// it preempts -> OUT_DIR/greedy_small.txt, whose first line is "# preemptions N"
// (tests/engine/test_engine_batching.cpp:58-75 is the test this follows). The roomy run is
// timed on the host -> OUT_DIR/timing.txt (one line; a record of this machine, compared by no test).
#include <cstdio>
#include <cstdlib>
#include <chrono>
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

static KVCacheConfig cache_config(const ModelConfig& c, int32_t page, size_t pages) {
  KVCacheConfig kc;
  kc.num_layers = int32_t(c.num_layers);
  kc.num_kv_heads = int32_t(c.num_kv_heads);
  kc.head_dim = int32_t(c.head_dim);
  kc.block_size = page;
  kc.dtype = DType::F32;
  kc.budget_bytes = pages * 2 * size_t(c.num_layers * c.num_kv_heads * c.head_dim) * size_t(page) * 4;
  return kc;
}

// All requests through the reference's engine at once; returns its count of preemptions.
static int64_t run_engine(CpuBackend& backend, const LoadedModel& weights, int32_t page, size_t pages, int32_t tokens_per_step,
                          const std::vector<std::vector<int32_t>>& prompts, const std::vector<int32_t>& new_tokens,
                          const std::string& path, bool small) {
  const ModelConfig& c = weights.config;
  PagedKVCache cache(backend, cache_config(c, page, pages));
  const ServingConfig serving{tokens_per_step, 8};
  Qwen3Model model(backend, weights, model_limits(serving, PagedKVCache::blocks_for(c.max_position_embeddings, page)));
  BatchSchedulerConfig sc;
  sc.serving = serving;
  sc.policy = OrderingPolicy::Fcfs;
  if (small) sc.watermark_blocks = 0;
  Engine engine(model, cache, std::make_unique<BatchScheduler>(cache, sc), serving, EngineConfig{});
  std::vector<int32_t> ids;
  for (size_t i = 0; i < prompts.size(); ++i) {
    SamplingParams p;
    p.max_tokens = new_tokens[i];
    ids.push_back(engine.add_request(prompts[i], p));
  }
  const auto t0 = std::chrono::steady_clock::now();
  int64_t steps = 0;
  while (engine.has_work()) { engine.step(); ++steps; }
  const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  if (!small) {
    int64_t prompt_tokens = 0, generated = 0;
    for (size_t i = 0; i < prompts.size(); ++i) { prompt_tokens += int64_t(prompts[i].size()); generated += new_tokens[i]; }
    std::ofstream t(path.substr(0, path.rfind('/')) + "/timing.txt");
    t << "reference engine, CPU backend (scalar dot products, g++ -O2), all requests batched: " << steps << " steps, "
      << prompt_tokens << " prompt tokens and " << generated << " generated tokens in " << ms << " ms = "
      << double(generated) * 1e3 / ms << " generated tokens/s\n";
  }
  std::ofstream g(path);
  if (small) g << "# preemptions " << engine.stats().preemptions << "\n";
  for (size_t i = 0; i < ids.size(); ++i) {
    const Sequence& s = engine.sequence(ids[i]);
    for (size_t t = size_t(s.prompt_len); t < s.tokens.size(); ++t) g << s.tokens[t] << (t + 1 < s.tokens.size() ? " " : "");
    g << "\n";
  }
  return engine.stats().preemptions;
}

int main(int argc, char** argv) {
  if (argc != 6) return 2;
  const std::string out = argv[2];
  const int32_t page = std::atoi(argv[3]), tokens_per_step = std::atoi(argv[4]);
  const size_t small_pool = size_t(std::atoi(argv[5]));
  try {
    const LoadedModel weights = load_model(argv[1]);
    const ModelConfig& c = weights.config;
    CpuBackend backend(2);
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
    {
      PagedKVCache cache(backend, cache_config(c, 4, 256));
      ModelLimits limits = model_limits(ServingConfig{8, 4}, PagedKVCache::blocks_for(c.max_position_embeddings, 4));
      limits.max_tokens_per_step = 256;
      limits.max_logit_rows = 256;
      Qwen3Model model(backend, weights, limits);
      for (size_t i = 0; i < prompts.size(); ++i) {
        std::vector<float> hidden;
        model.set_layer_hook([&](int, const Tensor& x) {
          hidden.insert(hidden.end(), x.data<float>(), x.data<float>() + x.numel());
        });
        test::SequenceRunner runner(model, cache);
        write_f32(out + "/logits_" + std::to_string(i) + ".f32", runner.step(prompts[i], true));
        write_f32(out + "/hidden_" + std::to_string(i) + ".f32", hidden);
      }
    }
    run_engine(backend, weights, page, 256, tokens_per_step, prompts, new_tokens, out + "/greedy.txt", false);
    const int64_t preempted =
        run_engine(backend, weights, page, small_pool, tokens_per_step, prompts, new_tokens, out + "/greedy_small.txt", true);
    std::fprintf(stderr, "ref_driver: %lld preemptions with %zu pages\n", static_cast<long long>(preempted), small_pool);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ref_driver: %s\n", e.what());
    return 1;
  }
  return 0;
}

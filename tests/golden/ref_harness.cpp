// Drives the UNMODIFIED Llama4 CPU engine of kurulav1/cpi (src/engine/llama4_cpu_engine.cpp) at a tiny
// size and writes its logits after every token.  The engine's sizes are private member defaults
// (include/engine/llama4_cpu_engine.hpp:43-61), so the header is included with `private` opened.
// Built and run by make_golden.py; this file is a test fixture, not library code.
//
// usage: ref_harness MODEL_DIR OUT.f32 vocab hidden heads kv_heads head_dim layers experts expert_inter
//                    shared_inter rope_orig_max theta factor low high  tok0 tok1 ...
// It prints `forward_ms=<ms> tokens=<n>` (the wall time of the token loop alone) on standard error.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>
#include <cublas_v2.h>
#include <cublasLt.h>
#include <cuda_runtime.h>
#define private public
#include "engine/llama4_cpu_engine.hpp"
#undef private

int main(int argc, char** argv) {
  if (argc < 18) { std::fprintf(stderr, "too few arguments\n"); return 1; }
  engine::Llama4CpuEngine e;
  int a = 3;
  e.vocab_size_ = std::atoi(argv[a++]); e.hidden_ = std::atoi(argv[a++]); e.n_heads_ = std::atoi(argv[a++]);
  e.n_kv_heads_ = std::atoi(argv[a++]); e.head_dim_ = std::atoi(argv[a++]); e.n_layers_ = std::atoi(argv[a++]);
  e.n_experts_ = std::atoi(argv[a++]); e.inter_mlp_ = 2 * std::atoi(argv[a++]); e.inter_shared_ = std::atoi(argv[a++]);
  e.rope_orig_max_pos_ = std::atoi(argv[a++]); e.rope_theta_ = (float)std::atof(argv[a++]);
  e.rope_scale_ = (float)std::atof(argv[a++]); e.rope_low_freq_factor_ = (float)std::atof(argv[a++]);
  e.rope_high_freq_factor_ = (float)std::atof(argv[a++]);
  engine::EngineOptions o;
  o.model_path = argv[1];
  o.max_context = 256;
  o.verbose = false;
  e.initialize(o);
  FILE* f = std::fopen(argv[2], "wb");
  if (!f) return 2;
  std::vector<float> all;
  all.reserve((size_t)(argc - a) * e.logits_.size());
  const auto t0 = std::chrono::steady_clock::now();
  for (int i = a, pos = 0; i < argc; ++i, ++pos) {
    e.forward_token(std::atoi(argv[i]), pos);
    all.insert(all.end(), e.logits_.begin(), e.logits_.end());
  }
  const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  std::fwrite(all.data(), sizeof(float), all.size(), f);
  std::fclose(f);
  std::fprintf(stderr, "forward_ms=%.3f tokens=%d\n", ms, argc - a);
  return 0;
}

// Host-side sampling over a logits row: arg-max, temperature, top-k, top-p, min-p, repetition
// penalties.  (Role of cpp_engine/include/sampler.hpp + core/sampler.cpp; the device sampler is
// csrc/kernels/sampling.cu.)
#pragma once
#include <cstdint>
#include <random>
#include <vector>

namespace pocket {

struct HostSamplingParams {
  float temperature = 0.f;
  int top_k = 0;
  float top_p = 1.f;
  float min_p = 0.f;
  float repetition_penalty = 1.f;
  float frequency_penalty = 0.f;
  float presence_penalty = 0.f;
};

int32_t argmax(const float* logits, int n);
// `history` = tokens generated so far (for the penalties). Deterministic for a given rng state.
int32_t sample(const float* logits, int n, const HostSamplingParams& p, std::mt19937_64& rng,
               const std::vector<int32_t>& history = {});

}  // namespace pocket

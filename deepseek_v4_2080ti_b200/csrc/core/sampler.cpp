#include "sampler.hpp"

#include <algorithm>
#include <cmath>
#include <map>
#include <numeric>

namespace pocket {

int32_t argmax(const float* logits, int n) {
  int best = 0;
  for (int i = 1; i < n; ++i)
    if (logits[i] > logits[best]) best = i;
  return best;
}

int32_t sample(const float* logits, int n, const HostSamplingParams& p, std::mt19937_64& rng,
               const std::vector<int32_t>& history) {
  std::vector<float> l(logits, logits + n);
  if (!history.empty() && (p.repetition_penalty != 1.f || p.frequency_penalty != 0.f || p.presence_penalty != 0.f)) {
    std::map<int32_t, int> counts;
    for (int32_t t : history) if (t >= 0 && t < n) ++counts[t];
    for (auto& kv : counts) {
      float& v = l[kv.first];
      if (p.repetition_penalty != 1.f) v = v > 0 ? v / p.repetition_penalty : v * p.repetition_penalty;
      v -= p.frequency_penalty * kv.second + p.presence_penalty;
    }
  }
  if (p.temperature <= 1e-5f) return argmax(l.data(), n);
  std::vector<int> idx(n);
  std::iota(idx.begin(), idx.end(), 0);
  int keep = n;
  if (p.top_k > 0 && p.top_k < n) {
    keep = p.top_k;
    std::partial_sort(idx.begin(), idx.begin() + keep, idx.end(), [&](int a, int b) { return l[a] > l[b]; });
  } else {
    std::sort(idx.begin(), idx.end(), [&](int a, int b) { return l[a] > l[b]; });
  }
  const float mx = l[idx[0]];
  std::vector<double> pr(keep);
  double sum = 0;
  for (int i = 0; i < keep; ++i) { pr[i] = std::exp((l[idx[i]] - mx) / p.temperature); sum += pr[i]; }
  for (double& v : pr) v /= sum;
  if (p.min_p > 0.f) {
    const double thr = pr[0] * p.min_p;
    int k = 1;
    while (k < keep && pr[k] >= thr) ++k;
    keep = k;
  }
  if (p.top_p < 1.f) {
    double c = 0;
    int k = 0;
    while (k < keep) { c += pr[k++]; if (c >= p.top_p) break; }
    keep = std::max(1, k);
  }
  double total = 0;
  for (int i = 0; i < keep; ++i) total += pr[i];
  std::uniform_real_distribution<double> u(0.0, total);
  double r = u(rng), c = 0;
  for (int i = 0; i < keep; ++i) { c += pr[i]; if (r <= c) return idx[i]; }
  return idx[keep - 1];
}

}  // namespace pocket

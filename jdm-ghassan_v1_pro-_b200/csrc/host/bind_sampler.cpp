// Host sampler: the reference semantics in full (inference/sampler.cpp:35-257): clamped settings, repetition /
// frequency / presence penalties over a history window, n-gram ban, greedy arg-max, top-k, temperature softmax in
// double precision, min-p, top-p, renormalisation and a draw from the shared random stream.  It is the oracle for
// the device sampler and the path for settings the device kernel does not take (n-gram bans, top_k outside 2..1024).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <chrono>
#include <cmath>

#include "core.hpp"

namespace py = pybind11;
using namespace gbh;

namespace {

struct SamplingConfig {
  float temperature = 0.8f;
  int top_k = 40;
  float top_p = 0.92f;
  float min_p = 0.05f;
  float repetition_penalty = 1.12f;
  int repetition_window = 128;
  float frequency_penalty = 0.0f;
  float presence_penalty = 0.0f;
  int no_repeat_ngram = 0;
  bool greedy = false;
  bool gpu_fast_sample = true;
  u64 seed = 0;

  void validate() {
    auto fin = [](float v) { return std::isfinite(v); };
    temperature = (!fin(temperature) || temperature < 0.f) ? 0.f : std::min(temperature, 5.0f);
    top_p = (!fin(top_p) || top_p < 0.f) ? 1.0f : std::min(top_p, 1.0f);
    if (!fin(min_p) || min_p < 0.f || min_p >= 1.0f) min_p = 0.f;
    top_k = std::clamp(top_k, 0, 2048);
    repetition_penalty = (!fin(repetition_penalty) || repetition_penalty <= 0.f) ? 1.0f : std::min(repetition_penalty, 5.0f);
    frequency_penalty = fin(frequency_penalty) ? std::clamp(frequency_penalty, -5.0f, 5.0f) : 0.f;
    presence_penalty = fin(presence_penalty) ? std::clamp(presence_penalty, -5.0f, 5.0f) : 0.f;
    repetition_window = std::clamp(repetition_window, 0, 8192);
    no_repeat_ngram = std::clamp(no_repeat_ngram, 0, 8);
    if (no_repeat_ngram == 1) no_repeat_ngram = 2;
  }
};

class Sampler {
 public:
  explicit Sampler(SamplingConfig c) : cfg_(c) {
    cfg_.validate();
    reseed(c.seed != 0 ? c.seed : static_cast<u64>(std::chrono::steady_clock::now().time_since_epoch().count()));
  }
  void reseed(u64 s) { rng_.reseed(s); }
  const SamplingConfig& config() const { return cfg_; }
  void set_config(SamplingConfig c) { c.validate(); cfg_ = c; }
  float next_uniform() { return rng_.uniform(); }

  void apply_penalties(float* lg, int vocab, const std::vector<i32>& hist) const {
    const bool rep = cfg_.repetition_penalty != 1.0f, freq = cfg_.frequency_penalty != 0.f, pres = cfg_.presence_penalty != 0.f;
    if (hist.empty() || !(rep || freq || pres)) return;
    const size_t win = cfg_.repetition_window > 0 ? std::min<size_t>(hist.size(), cfg_.repetition_window) : hist.size();
    std::vector<i32> seen;
    for (size_t i = hist.size() - win; i < hist.size(); ++i)
      if (hist[i] >= 0 && hist[i] < vocab) seen.push_back(hist[i]);
    std::sort(seen.begin(), seen.end());
    for (size_t i = 0; i < seen.size();) {
      size_t j = i;
      while (j < seen.size() && seen[j] == seen[i]) ++j;
      float& l = lg[seen[i]];
      if (rep) l = l > 0.f ? l / cfg_.repetition_penalty : l * cfg_.repetition_penalty;
      if (freq) l -= cfg_.frequency_penalty * static_cast<float>(j - i);
      if (pres) l -= cfg_.presence_penalty;
      i = j;
    }
  }

  static void ban_repeated_ngrams(float* lg, int vocab, const std::vector<i32>& hist, int n) {
    if (n <= 0 || hist.size() < static_cast<size_t>(n - 1)) return;
    const size_t m = hist.size(), pre = static_cast<size_t>(n - 1);
    for (size_t i = 0; i + static_cast<size_t>(n) <= m; ++i) {
      if (!std::equal(hist.begin() + i, hist.begin() + i + pre, hist.end() - pre)) continue;
      const i32 nxt = hist[i + pre];
      if (nxt >= 0 && nxt < vocab) lg[nxt] = -1e30f;
    }
  }

  i32 sample(float* lg, int vocab, const std::vector<i32>& hist) {
    GBH_CHECK(vocab > 0, "empty vocabulary");
    apply_penalties(lg, vocab, hist);
    if (cfg_.no_repeat_ngram > 0) ban_repeated_ngrams(lg, vocab, hist, cfg_.no_repeat_ngram);
    if (cfg_.greedy || cfg_.temperature <= 0.f || cfg_.top_k == 1)
      return static_cast<i32>(std::max_element(lg, lg + vocab, [](float a, float b) { return a < b; }) - lg);
    cand_.clear();
    cand_.reserve(static_cast<size_t>(vocab));
    for (int i = 0; i < vocab; ++i) cand_.emplace_back(lg[i], i);
    const bool unfiltered = (cfg_.top_k <= 0 || cfg_.top_k >= vocab) && (cfg_.top_p <= 0.f || cfg_.top_p >= 1.f) && cfg_.min_p <= 0.f;
    if (unfiltered) {   // plain temperature sampling over the whole vocabulary, best candidate first
      const size_t best = static_cast<size_t>(std::max_element(cand_.begin(), cand_.end(), [](const auto& a, const auto& b) {
                                                return a.first < b.first; }) - cand_.begin());
      std::swap(cand_[0], cand_[best]);
      return draw(false);
    }
    int k = (cfg_.top_k > 0 && cfg_.top_k < vocab) ? cfg_.top_k : std::min(vocab, 2048);
    auto better = [](const auto& a, const auto& b) { return a.first > b.first || (a.first == b.first && a.second < b.second); };
    if (k < vocab) {
      std::partial_sort(cand_.begin(), cand_.begin() + k, cand_.end(), better);
      cand_.resize(static_cast<size_t>(k));
    } else {
      std::sort(cand_.begin(), cand_.end(), better);
    }
    return draw(true);
  }

  i32 sample_candidates(const std::vector<float>& vals, const std::vector<i32>& ids) {
    GBH_CHECK(!vals.empty() && vals.size() == ids.size(), "sample_candidates: empty set");
    cand_.clear();
    for (size_t i = 0; i < vals.size(); ++i) cand_.emplace_back(vals[i], ids[i]);
    std::sort(cand_.begin(), cand_.end(), [](const auto& a, const auto& b) {
      return a.first > b.first || (a.first == b.first && a.second < b.second); });
    return draw(true);
  }

  static double log_prob(const float* lg, int vocab, i32 token) {
    if (token < 0 || token >= vocab) return -1e30;
    const float mx = *std::max_element(lg, lg + vocab);
    double sum = 0.0;
    for (int i = 0; i < vocab; ++i) sum += std::exp(static_cast<double>(lg[i] - mx));
    return static_cast<double>(lg[token] - mx) - std::log(sum);
  }

 private:
  // cand_ is ordered best first; `filter` applies min-p / top-p
  i32 draw(bool filter) {
    if (!(cfg_.temperature > 0.f)) return cand_[0].second;
    const float inv_t = 1.0f / cfg_.temperature, mx = cand_[0].first;
    probs_.resize(cand_.size());
    double sum = 0.0;
    for (size_t i = 0; i < cand_.size(); ++i) sum += probs_[i] = std::exp(static_cast<double>((cand_[i].first - mx) * inv_t));
    if (!std::isfinite(sum) || sum <= 0.0) return cand_[0].second;
    size_t limit = cand_.size();
    if (filter) {
      for (double& p : probs_) p /= sum;
      if (cfg_.min_p > 0.f) {
        const double thresh = cfg_.min_p * probs_[0];
        size_t n = 0;
        while (n < probs_.size() && probs_[n] >= thresh) ++n;
        limit = std::max<size_t>(1, n);
      }
      if (cfg_.top_p > 0.f && cfg_.top_p < 1.0f) {
        double cum = 0.0;
        size_t n = 0;
        while (n < limit) {
          cum += probs_[n++];
          if (cum >= static_cast<double>(cfg_.top_p)) break;
        }
        limit = std::max<size_t>(1, n);
      }
      sum = 0.0;
      for (size_t i = 0; i < limit; ++i) sum += probs_[i];
    }
    const double r = static_cast<double>(rng_.uniform()) * sum;
    double acc = 0.0;
    for (size_t i = 0; i < limit; ++i) {
      acc += probs_[i];
      if (r <= acc) return cand_[i].second;
    }
    return cand_[limit - 1].second;
  }

  SamplingConfig cfg_;
  Rng rng_;
  std::vector<std::pair<float, i32>> cand_;
  std::vector<double> probs_;
};

}  // namespace

void bind_sampler(py::module_& m) {
  py::class_<SamplingConfig>(m, "SamplingConfig")
      .def(py::init<>())
      .def_readwrite("temperature", &SamplingConfig::temperature)
      .def_readwrite("top_k", &SamplingConfig::top_k)
      .def_readwrite("top_p", &SamplingConfig::top_p)
      .def_readwrite("min_p", &SamplingConfig::min_p)
      .def_readwrite("repetition_penalty", &SamplingConfig::repetition_penalty)
      .def_readwrite("repetition_window", &SamplingConfig::repetition_window)
      .def_readwrite("frequency_penalty", &SamplingConfig::frequency_penalty)
      .def_readwrite("presence_penalty", &SamplingConfig::presence_penalty)
      .def_readwrite("no_repeat_ngram", &SamplingConfig::no_repeat_ngram)
      .def_readwrite("greedy", &SamplingConfig::greedy)
      .def_readwrite("gpu_fast_sample", &SamplingConfig::gpu_fast_sample)
      .def_readwrite("seed", &SamplingConfig::seed)
      .def("validate", &SamplingConfig::validate);
  py::class_<Sampler>(m, "Sampler")
      .def(py::init<SamplingConfig>())
      .def("reseed", &Sampler::reseed)
      .def("next_uniform", &Sampler::next_uniform)
      .def_property("config", &Sampler::config, &Sampler::set_config)
      .def("sample",
           [](Sampler& s, py::array_t<float, py::array::c_style | py::array::forcecast> logits, const std::vector<i32>& hist) {
             std::vector<float> lg(logits.data(), logits.data() + logits.size());   // penalties edit a private copy
             return s.sample(lg.data(), static_cast<int>(lg.size()), hist);
           },
           py::arg("logits"), py::arg("history") = std::vector<i32>{})
      .def("sample_candidates", &Sampler::sample_candidates)
      .def_static("log_prob", [](py::array_t<float, py::array::c_style | py::array::forcecast> logits, i32 token) {
        return Sampler::log_prob(logits.data(), static_cast<int>(logits.size()), token);
      });
}

#include "stats.h"

#include <algorithm>
#include <cmath>
#include <limits>

namespace imex {
namespace {
std::vector<float> sorted(const std::vector<float> &v) {
  std::vector<float> s(v);
  std::sort(s.begin(), s.end());
  return s;
}
float at_rank(const std::vector<float> &s, size_t r) { return s[std::min(r, s.size() - 1)]; }
float sum_sq_dev(const std::vector<float> &v, float mean) {
  float acc = 0.0f;
  for (float x : v) acc += (x - mean) * (x - mean);
  return acc;
}
} // namespace

float calculateMin(const std::vector<float> &v) {
  return v.empty() ? std::numeric_limits<float>::max() : *std::min_element(v.begin(), v.end());
}

float calculateMax(const std::vector<float> &v) {
  return v.empty() ? std::numeric_limits<float>::min() : *std::max_element(v.begin(), v.end());
}

float calculateAverage(const std::vector<float> &v) {
  if (v.empty()) return 0.0f;
  float acc = 0.0f;
  for (float x : v) acc += x;
  return acc / v.size();
}

float calculateMedian(const std::vector<float> &v) {
  if (v.empty()) return 0.0f;
  const auto s = sorted(v);
  const size_t n = s.size(), r = n / 2 + 1;
  if (n % 2 == 1) return at_rank(s, r);
  return (at_rank(s, r) + at_rank(s, r - 1)) / 2;
}

float calculateVariance(const std::vector<float> &v) {
  return v.empty() ? 0.0f : sum_sq_dev(v, calculateAverage(v)) / v.size();
}

float calculateStdDev(const std::vector<float> &v) {
  return v.empty() ? 0.0f : std::sqrt(sum_sq_dev(v, calculateAverage(v)) / v.size());
}

float calculateP95(const std::vector<float> &v) {
  return v.empty() ? 0.0f : at_rank(sorted(v), static_cast<size_t>(0.95 * v.size()));
}

float calculateP5(const std::vector<float> &v) {
  return v.empty() ? 0.0f : at_rank(sorted(v), static_cast<size_t>(0.05 * v.size()));
}

float calculateMiddleThirdAverage(const std::vector<float> &v) {
  if (v.empty()) return 0.0f;
  const size_t n = v.size();
  if (n < 3) return calculateMedian(v);
  const auto s = sorted(v);
  const size_t first = n / 3, last = n - first;
  float acc = 0.0f;
  for (size_t i = first; i < last; ++i) acc += s[i];
  return acc / (last - first);
}
} // namespace imex

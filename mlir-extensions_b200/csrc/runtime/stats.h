// Timing statistics printed by the profiling loop of the runtime wrappers.
// Same definitions as the reference's
// lib/ExecutionEngine/ExecutionEngineUtils/ExecutionEngineUtils.cpp:18-150,
// including its rank conventions: the "median" is taken at sorted rank
// n/2 + 1 (one above the textbook median; for even n the mean of ranks n/2
// and n/2 + 1), P95 / P5 at rank floor(0.95 n) / floor(0.05 n), and the
// middle-third average over sorted ranks [n/3, n - n/3).  Ranks are clamped
// to n - 1, where the reference would read past the end for n <= 2.
#pragma once
#include <vector>

namespace imex {
float calculateMin(const std::vector<float> &v);
float calculateMax(const std::vector<float> &v);
float calculateAverage(const std::vector<float> &v);
float calculateMedian(const std::vector<float> &v);
float calculateStdDev(const std::vector<float> &v);
float calculateVariance(const std::vector<float> &v);
float calculateP95(const std::vector<float> &v);
float calculateP5(const std::vector<float> &v);
float calculateMiddleThirdAverage(const std::vector<float> &v);
} // namespace imex

// Shim: the metric codes of cpp/include/cuvs/distance/distance.hpp:21-67 (an interface enum; the
// rest of that header declares the pairwise-distance library and is not needed by the pins).
#pragma once
namespace cuvs::distance {
enum class DistanceType : int {
  L2Expanded = 0, L2SqrtExpanded = 1, CosineExpanded = 2, L1 = 3, L2Unexpanded = 4,
  L2SqrtUnexpanded = 5, InnerProduct = 6, Linf = 7, Canberra = 8, LpUnexpanded = 9,
  CorrelationExpanded = 10, JaccardExpanded = 11, HellingerExpanded = 12, Haversine = 13,
  BrayCurtis = 14, JensenShannon = 15, HammingUnexpanded = 16, KLDivergence = 17,
  RusselRaoExpanded = 18, DiceExpanded = 19, BitwiseHamming = 20, Precomputed = 100, CustomUDF = 101
};
}  // namespace cuvs::distance

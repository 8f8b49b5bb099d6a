/*
 * Distance-type codes of the C interface.
 * Replaces: c/include/cuvs/distance/distance.h:16-62 of the reference (same names, same values).
 * The IVF-PQ path accepts L2Expanded, L2SqrtExpanded, InnerProduct and CosineExpanded.
 */
#ifndef CUVS_B200_DISTANCE_H_
#define CUVS_B200_DISTANCE_H_
#ifdef __cplusplus
extern "C" {
#endif
typedef enum {
  L2Expanded          = 0,
  L2SqrtExpanded      = 1,
  CosineExpanded      = 2,
  L1                  = 3,
  L2Unexpanded        = 4,
  L2SqrtUnexpanded    = 5,
  InnerProduct        = 6,
  Linf                = 7,
  Canberra            = 8,
  LpUnexpanded        = 9,
  CorrelationExpanded = 10,
  JaccardExpanded     = 11,
  HellingerExpanded   = 12,
  Haversine           = 13,
  BrayCurtis          = 14,
  JensenShannon       = 15,
  HammingUnexpanded   = 16,
  KLDivergence        = 17,
  RusselRaoExpanded   = 18,
  DiceExpanded        = 19,
  BitwiseHamming      = 20,
  Precomputed         = 100
} cuvsDistanceType;
#ifdef __cplusplus
}
#endif
#endif

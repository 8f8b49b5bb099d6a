// Declarations shared between the search translation units.
#pragma once

#include "ivf_pq.hpp"

namespace cuvs::neighbors::ivf_pq {

struct scan_plan {
  uint32_t n_groups, group_threads, pqc_in_smem, pqc_bytes, group_bytes, lut_bytes, base_bytes,
    merge_bytes;
  size_t total_bytes;
};
scan_plan plan_scan(const raft::resources& res, const index<int64_t>& idx, int lut_kind, bool is_ip,
                    uint32_t k);

// Coarse stage (coarse.cu): for every query the n_probes lists with the smallest
//   score[q, l] = alpha * sum_k centers[l, k] * fq[q, k]
// sorted by (score, list id) ascending.  `scores_out` (optional) receives the selected scores.
size_t coarse_workspace_bytes(uint32_t n_queries, uint32_t n_lists, uint32_t n_probes);
void select_clusters(raft::resources& res, const float* centers, uint32_t n_lists, uint32_t dim_ext,
                     float alpha, const float* fq, uint32_t n_queries, uint32_t n_probes,
                     uint32_t* probes, float* scores_out, void* workspace, size_t workspace_bytes);

// Nearest list of every row: labels[i] = argmin_l alpha * sum_k centers[l,k] * x[i,k], ties to the
// lowest l (equals select_clusters with n_probes = 1).  `best` is scratch of n_rows * 8 bytes.
void assign_nearest(raft::resources& res, const float* centers, uint32_t n_lists, uint32_t dim_ext,
                    float alpha, const float* x_ext, uint32_t n_rows, uint32_t* labels,
                    unsigned long long* best);

}  // namespace cuvs::neighbors::ivf_pq

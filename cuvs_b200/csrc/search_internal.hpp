// Declarations shared between the search translation units.
#pragma once

#include "ivf_pq.hpp"

namespace cuvs::neighbors::ivf_pq {

struct scan_plan {
  uint32_t n_groups, group_threads, pqc_in_smem, pqc_bytes, group_bytes, lut_bytes, base_bytes,
    merge_bytes, tmem_cols, tmem_slot_off, lut_global, base_double;
  size_t total_bytes;
};
scan_plan plan_scan(const raft::resources& res, const index<int64_t>& idx, int lut_kind, bool is_ip,
                    uint32_t k);

// Coarse stage (coarse.cu): for every query the n_probes lists with the smallest
//   score[q, l] = alpha * sum_k centers[l, k] * fq[q, k]
// sorted by (score, list id) ascending.  `scores_out` (optional) receives the selected scores.
// `half_scores`: every score is rounded to half precision before the selection (fp16 coarse search).
size_t coarse_workspace_bytes(uint32_t n_queries, uint32_t n_lists, uint32_t n_probes);
void select_clusters(raft::resources& res, const float* centers, uint32_t n_lists, uint32_t dim_ext,
                     float alpha, const float* fq, uint32_t n_queries, uint32_t n_probes,
                     uint32_t* probes, float* scores_out, void* workspace, size_t workspace_bytes,
                     bool half_scores = false);

// Per row the k smallest (value, position), ascending (radix select + sort; k <= 4096).
void select_rows(raft::resources& res, const float* rows, uint32_t n_rows, uint32_t row_len, uint32_t k,
                 uint32_t* out_idx, float* out_scores);

// Tensor-core coarse stage (coarse_tc.cu): same contract and bit-identical probes as
// select_clusters; `centers_hi/lo` are the TF32 split of `centers`, `cmax` the largest row norm.
// `exact_operands`: every operand is exact in TF32 and every partial sum in fp32 (small integers):
// one product per K step, and the guard allows for no split error.
bool coarse_tc_usable(uint32_t n_lists, uint32_t n_probes, uint32_t dim_ext);
size_t coarse_tc_workspace_bytes(uint32_t n_queries, uint32_t n_lists, uint32_t dim_ext);
// Prepares `hi` / `lo` (TF32 split of the centre rows) with column `ext_col` (the |c|^2 column of L2
// metrics; >= dim_ext: none) divided by a power of two `ext_scale` close to the largest |c|, and `cmax`,
// the largest norm of a row so prepared; select_clusters_tc is given the same ext_col / ext_scale and
// multiplies the queries' entry of that column by it.  Synchronises the stream.
void prepare_tc_centers(cudaStream_t stream, const float* centers, uint32_t n_lists, uint32_t dim_ext,
                        uint32_t ext_col, float* hi, float* lo, float* cmax, float* ext_scale);
void select_clusters_tc(raft::resources& res, const float* centers, const float* centers_hi,
                        const float* centers_lo, float cmax, uint32_t n_lists, uint32_t dim_ext,
                        float alpha, const float* fq, uint32_t n_queries, uint32_t n_probes,
                        uint32_t* probes, float* scores_out, void* workspace, size_t workspace_bytes,
                        bool exact_operands = false, uint32_t ext_col = ~0u, float ext_scale = 1.0f);
void coarse_tc_status(raft::resources& res, const void* workspace, uint32_t n_queries, uint32_t n_lists,
                      uint32_t dim_ext, uint32_t* error, uint32_t* n_fallback);

// Probe selection alone (diagnostics / stage-wise tests): mode 0 = automatic, 1 = exact SIMT path,
// 2 = tensor-core path.  status[0] = error word, status[1] = queries redone exactly (mode 2).
void coarse_only(raft::resources& res, const index<int64_t>& idx, const void* queries, elem_t qtype,
                 uint32_t n_queries, uint32_t n_probes, int mode, uint32_t* probes, float* scores,
                 uint32_t* status);

// products of the TF32 split the tensor-core coarse GEMM issues per K step (1, 2 or 3)
void set_coarse_tc_products(int products);
// process-wide override used by tests: false = the tensor-core coarse GEMM streams both operands even
// where the query tile could stay resident in shared memory
void set_coarse_tc_resident(bool on);
// test hook of the bounded waits of the tensor-core coarse kernel: iterations a wait may take (0 = the
// default) and 1 + index of an operand stage left unfilled (0 = none)
void set_coarse_tc_wait_test(uint32_t spin_limit, uint32_t skip_kb);
void set_coarse_mode(int mode);  // process-wide override used by tests: 0 auto, 1 SIMT, 2 tensor core
// process-wide override used by tests: 0 = the per-subspace codebook goes to tensor memory where it
// fits, 1 = never (shared memory, else global memory)
void set_scan_codebook_home(int home);

// Nearest list of every row: labels[i] = argmin_l alpha * sum_k centers[l,k] * x[i,k], ties to the
// lowest l (equals select_clusters with n_probes = 1).  `best` is scratch of n_rows * 8 bytes.
void assign_nearest(raft::resources& res, const float* centers, uint32_t n_lists, uint32_t dim_ext,
                    float alpha, const float* x_ext, uint32_t n_rows, uint32_t* labels,
                    unsigned long long* best);

}  // namespace cuvs::neighbors::ivf_pq

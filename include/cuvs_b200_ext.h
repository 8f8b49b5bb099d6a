/*
 * Instrumentation of the IVF-PQ search path.  These entry points have no counterpart in the
 * reference; they exist so that a benchmark can report per-stage device times and the bytes the
 * code scan logically processes without guessing.  Disabled by default; when enabled, search
 * records CUDA events around its stages on the handle's stream and accumulates two counters on
 * the device.
 */
#ifndef CUVS_B200_EXT_H_
#define CUVS_B200_EXT_H_

#include "cuvs_core_c_api.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  double prep_ms;    /* query cast / pad / rotate */
  double coarse_ms;  /* probe selection */
  double sort_ms;    /* sample offsets + ordering of (query, probe) pairs by list */
  double scan_ms;    /* look-up table build + code scan + per-pair top-k (one kernel per batch) */
  double merge_ms;   /* final selection, id translation, distance post-processing */
  uint64_t batches;        /* internal batches = launches of the scan kernel */
  uint64_t pairs;          /* (query, probe) pairs scanned */
  uint64_t scan_groups;    /* sum over pairs of ceil(list size / 32) */
  uint64_t unique_groups;  /* sum over distinct probed lists, per batch, of ceil(list size / 32) */
  uint64_t launches;       /* kernels of this library launched through the handle since creation */
} cuvsB200SearchStats;

/* No counterpart in the reference: switch stage timing and counters on or off for a handle. */
CUVS_EXPORT cuvsError_t cuvsB200StatsEnable(cuvsResources_t res, bool enable);
/* No counterpart in the reference: synchronise the stream, return the accumulated figures and
 * optionally reset them. */
CUVS_EXPORT cuvsError_t cuvsB200StatsGet(cuvsResources_t res, cuvsB200SearchStats* out, bool reset);

/* No counterpart in the reference: run the probe-selection stage alone (for stage-wise checks).
 * queries f32/f16/i8/u8 [n, dim]; probes u32 [n, n_probes] (ascending by (score, list id));
 * scores f32 [n, n_probes]; mode 0 = automatic, 1 = exact SIMT path, 2 = tensor-core path;
 * status[0] = device error word (0 = none), status[1] = queries the tensor-core path had to redo
 * exactly.  Synchronises the stream. */
CUVS_EXPORT cuvsError_t cuvsB200CoarseSelect(cuvsResources_t res, void* index /* cuvsIvfPqIndex_t */,
                                             DLManagedTensor* queries, DLManagedTensor* probes,
                                             DLManagedTensor* scores, int mode, uint32_t* status);
/* No counterpart in the reference: force the probe-selection path used by cuvsIvfPqSearch in this
 * process (0 = automatic, 1 = exact SIMT path, 2 = tensor-core path where it applies; 11, 12, 13 =
 * tensor-core path with exactly 1, 2 or 3 products of the TF32 operand split per K step instead
 * of the per-handle adaptive choice; 21, 22 = as 11, 12 but with both operands streamed, no query
 * tile kept resident in shared memory). */
CUVS_EXPORT cuvsError_t cuvsB200SetCoarseMode(int mode);
/* No counterpart in the reference: where the fine-search kernel of cuvsIvfPqSearch keeps a
 * per-subspace PQ codebook in this process: 0 = tensor memory where it fits (the default),
 * 1 = never tensor memory (shared memory, else global memory), 2 = as 0 but never a kernel instantiated
 * for one exact shape, 3 = as if no look-up table fitted shared memory (tables in global memory). */
CUVS_EXPORT cuvsError_t cuvsB200SetScanCodebookHome(int home);

/* No counterpart in the reference.  Every wait inside the tensor-core probe-selection kernel is bounded;
 * when one runs out the kernel sets an error word, frees what it holds and returns, the stages behind
 * it recompute the probes of every query of that batch with the exact path, and the handle counts the
 * event.  This call returns that count (after waiting for nothing: it reports the batches whose
 * verdict has arrived; cuvsStreamSync first makes that all of them). */
CUVS_EXPORT cuvsError_t cuvsB200CoarseTimeouts(cuvsResources_t res, uint64_t* n_batches);
/* No counterpart in the reference; for tests of the above.  spin_limit: iterations (about a microsecond
 * each) a wait of that kernel may take, 0 = the default of about two seconds; skip_stage: 1 + index of
 * an operand stage of each CTA's first tile that is never filled, so that the wait for it runs out;
 * 0 = none.  Process-wide. */
CUVS_EXPORT cuvsError_t cuvsB200SetCoarseWaitTest(uint32_t spin_limit, uint32_t skip_stage);

#ifdef __cplusplus
}
#endif
#endif

// C interface: the entry points declared in include/cuvs_core_c_api.h and include/cuvs_ivf_pq.h.
//
// Mirrors c/src/core/c_api.cpp and c/src/neighbors/ivf_pq.cpp of the reference: every entry point
// runs inside translate_exceptions (c/src/core/exceptions.hpp:17-33), tensors are validated the
// way from_dlpack does (c/src/core/detail/interop.hpp:75-139) and dispatched on their dtype.
#include "../../include/cuvs_b200_ext.h"
#include "../../include/cuvs_dynamic_batching.h"
#include "../../include/cuvs_ivf_pq.h"
#include "../../include/cuvs_ivf_pq_helpers.h"
#include "../../include/cuvs_mg_ivf_pq.h"
#include "../../include/cuvs_refine.h"

#include "c_api_util.hpp"
#include "dynamic_batching.hpp"
#include "ivf_pq.hpp"
#include "search_internal.hpp"

#include <algorithm>
#include <cstring>
#include <exception>
#include <string>
#include <vector>

namespace cuvs::neighbors {
void refine_any(raft::resources& res, const void* dataset, ivf_pq::elem_t dtype, int64_t n_rows,
                uint32_t dim, const void* queries, uint32_t n_queries, const int64_t* candidates,
                uint32_t n_cand, ivf_pq::DistanceType metric, int64_t* indices, float* distances,
                uint32_t k);
}
namespace ivf_pq = cuvs::neighbors::ivf_pq;
using cuvs_b200::fail;
using index_t = ivf_pq::index<int64_t>;

namespace {
thread_local std::string g_last_error;
thread_local bool g_has_error = false;
}  // namespace
using namespace cuvs_b200::capi;

// ------------------------------------------------------------------------------------------------
// core
// ------------------------------------------------------------------------------------------------
extern "C" const char* cuvsGetLastErrorText(void) { return g_has_error ? g_last_error.c_str() : nullptr; }

extern "C" void cuvsSetLastErrorText(const char* error)
{
  if (error) {
    g_last_error = error;
    g_has_error  = true;
  } else {
    g_last_error.clear();
    g_has_error = false;
  }
}

extern "C" cuvsError_t cuvsResourcesCreate(cuvsResources_t* res)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(res != nullptr, "null output pointer");
    *res = reinterpret_cast<cuvsResources_t>(new cuvs_b200::resources());
  });
}
extern "C" cuvsError_t cuvsResourcesDestroy(cuvsResources_t res)
{
  return translate_exceptions([=] { delete reinterpret_cast<cuvs_b200::resources*>(res); });
}
extern "C" cuvsError_t cuvsStreamSet(cuvsResources_t res, cudaStream_t stream)
{
  return translate_exceptions([=] { res_of(res)->stream = stream; });
}
extern "C" cuvsError_t cuvsStreamGet(cuvsResources_t res, cudaStream_t* stream)
{
  return translate_exceptions([=] { *stream = res_of(res)->stream; });
}
extern "C" cuvsError_t cuvsStreamSync(cuvsResources_t res)
{
  return translate_exceptions([=] { res_of(res)->sync(); });
}
extern "C" cuvsError_t cuvsDeviceIdGet(cuvsResources_t res, int* device_id)
{
  return translate_exceptions([=] { *device_id = res_of(res)->device; });
}
extern "C" cuvsError_t cuvsResourcesSetWorkspacePool(cuvsResources_t res, size_t initial_size_bytes)
{
  return translate_exceptions([=] { res_of(res)->ws.reserve(initial_size_bytes); });
}
extern "C" cuvsError_t cuvsRMMAlloc(cuvsResources_t res, void** ptr, size_t bytes)
{
  return translate_exceptions([=] {
    res_of(res);
    CUDA_TRY(cudaMalloc(ptr, bytes));
  });
}
extern "C" cuvsError_t cuvsRMMFree(cuvsResources_t res, void* ptr, size_t)
{
  return translate_exceptions([=] {
    res_of(res);
    CUDA_TRY(cudaFree(ptr));
  });
}
extern "C" cuvsError_t cuvsVersionGet(uint16_t* major, uint16_t* minor, uint16_t* patch)
{
  return translate_exceptions([=] {
    *major = 26;  // the interface version mirrored (reference VERSION 26.10.00)
    *minor = 10;
    *patch = 0;
  });
}

// ------------------------------------------------------------------------------------------------
// params
// ------------------------------------------------------------------------------------------------
extern "C" cuvsError_t cuvsIvfPqIndexParamsCreate(cuvsIvfPqIndexParams_t* params)
{
  return translate_exceptions([=] {
    auto* p                           = new cuvsIvfPqIndexParams{};
    p->metric                         = L2Expanded;
    p->metric_arg                     = 2.0f;
    p->add_data_on_build              = true;
    p->n_lists                        = 1024;
    p->kmeans_n_iters                 = 20;
    p->kmeans_trainset_fraction       = 0.5;
    p->pq_bits                        = 8;
    p->pq_dim                         = 0;
    p->codebook_kind                  = CUVS_IVF_PQ_CODEBOOK_GEN_PER_SUBSPACE;
    p->force_random_rotation          = false;
    p->conservative_memory_allocation = false;
    p->max_train_points_per_pq_code   = 256;
    p->codes_layout                   = CUVS_IVF_PQ_LIST_LAYOUT_INTERLEAVED;
    *params                           = p;
  });
}
extern "C" cuvsError_t cuvsIvfPqIndexParamsDestroy(cuvsIvfPqIndexParams_t params)
{
  return translate_exceptions([=] { delete params; });
}
extern "C" cuvsError_t cuvsIvfPqSearchParamsCreate(cuvsIvfPqSearchParams_t* params)
{
  return translate_exceptions([=] {
    auto* p                     = new cuvsIvfPqSearchParams{};
    p->n_probes                 = 20;
    p->lut_dtype                = CUDA_R_32F;
    p->internal_distance_dtype  = CUDA_R_32F;
    p->coarse_search_dtype      = CUDA_R_32F;
    p->max_internal_batch_size  = 4096;
    p->preferred_shmem_carveout = 1.0;
    *params                     = p;
  });
}
extern "C" cuvsError_t cuvsIvfPqSearchParamsDestroy(cuvsIvfPqSearchParams_t params)
{
  return translate_exceptions([=] { delete params; });
}

// ------------------------------------------------------------------------------------------------
// index handle + getters
// ------------------------------------------------------------------------------------------------
extern "C" cuvsError_t cuvsIvfPqIndexCreate(cuvsIvfPqIndex_t* index)
{
  return translate_exceptions([=] { *index = new cuvsIvfPqIndex{}; });
}
extern "C" cuvsError_t cuvsIvfPqIndexDestroy(cuvsIvfPqIndex_t index)
{
  return translate_exceptions([=] {
    if (index) {
      delete reinterpret_cast<index_t*>(index->addr);
      delete index;
    }
  });
}

#define SCALAR_GETTER(NAME, EXPR)                                                  \
  extern "C" cuvsError_t NAME(cuvsIvfPqIndex_t index, int64_t* out)                \
  {                                                                                \
    return translate_exceptions([=] { *out = int64_t(index_of(index)->EXPR()); }); \
  }
SCALAR_GETTER(cuvsIvfPqIndexGetNLists, n_lists)
SCALAR_GETTER(cuvsIvfPqIndexGetDim, dim)
SCALAR_GETTER(cuvsIvfPqIndexGetSize, size)
SCALAR_GETTER(cuvsIvfPqIndexGetPqDim, pq_dim)
SCALAR_GETTER(cuvsIvfPqIndexGetPqBits, pq_bits)
SCALAR_GETTER(cuvsIvfPqIndexGetPqLen, pq_len)

namespace {
constexpr DLDataType kF32{kDLFloat, 32, 1};
constexpr DLDataType kU32{kDLUInt, 32, 1};
constexpr DLDataType kI64{kDLInt, 64, 1};
}  // namespace

extern "C" cuvsError_t cuvsIvfPqIndexGetCenters(cuvsIvfPqIndex_t index, DLManagedTensor* centers)
{
  return translate_exceptions([=] {
    auto* ix = index_of(index);
    make_view(centers, ix->centers(), kF32, {int64_t(ix->n_lists()), int64_t(ix->dim())},
              {int64_t(ix->dim_ext()), 1});
  });
}
extern "C" cuvsError_t cuvsIvfPqIndexGetCentersPadded(cuvsIvfPqIndex_t index, DLManagedTensor* centers)
{
  return translate_exceptions([=] {
    auto* ix = index_of(index);
    make_view(centers, ix->centers(), kF32, {int64_t(ix->n_lists()), int64_t(ix->dim_ext())});
  });
}
extern "C" cuvsError_t cuvsIvfPqIndexGetPqCenters(cuvsIvfPqIndex_t index, DLManagedTensor* pq_centers)
{
  return translate_exceptions([=] {
    auto* ix            = index_of(index);
    const int64_t first = ix->codebook_kind() == ivf_pq::codebook_gen::PER_SUBSPACE ? ix->pq_dim()
                                                                                     : ix->n_lists();
    make_view(pq_centers, ix->pq_centers(), kF32,
              {first, int64_t(ix->pq_len()), int64_t(ix->pq_book_size())});
  });
}
extern "C" cuvsError_t cuvsIvfPqIndexGetCentersRot(cuvsIvfPqIndex_t index, DLManagedTensor* centers_rot)
{
  return translate_exceptions([=] {
    auto* ix = index_of(index);
    make_view(centers_rot, ix->centers_rot(), kF32, {int64_t(ix->n_lists()), int64_t(ix->rot_dim())});
  });
}
extern "C" cuvsError_t cuvsIvfPqIndexGetRotationMatrix(cuvsIvfPqIndex_t index,
                                                       DLManagedTensor* rotation_matrix)
{
  return translate_exceptions([=] {
    auto* ix = index_of(index);
    make_view(rotation_matrix, ix->rotation_matrix(), kF32,
              {int64_t(ix->rot_dim()), int64_t(ix->dim())});
  });
}
extern "C" cuvsError_t cuvsIvfPqIndexGetListSizes(cuvsIvfPqIndex_t index, DLManagedTensor* list_sizes)
{
  return translate_exceptions([=] {
    auto* ix = index_of(index);
    make_view(list_sizes, ix->list_sizes(), kU32, {int64_t(ix->n_lists())});
  });
}
extern "C" cuvsError_t cuvsIvfPqIndexGetListIndices(cuvsIvfPqIndex_t index, uint32_t label,
                                                    DLManagedTensor* out_labels)
{
  return translate_exceptions([=] {
    auto* ix = index_of(index);
    CUVS_EXPECTS(label < ix->n_lists(), "label %u is out of range (n_lists = %u)", label, ix->n_lists());
    make_view(out_labels, ix->ids() + ix->host_row_offsets()[label], kI64,
              {int64_t(ix->host_list_sizes()[label])});
  });
}
extern "C" cuvsError_t cuvsIvfPqIndexUnpackContiguousListData(cuvsResources_t res,
                                                              cuvsIvfPqIndex_t index,
                                                              DLManagedTensor* out_codes,
                                                              uint32_t label, uint32_t offset)
{
  return translate_exceptions([=] {
    auto* ix   = index_of(index);
    auto* data = static_cast<uint8_t*>(checked_data(out_codes, kDLUInt, 8, 2, true, "out_codes"));
    ivf_pq::helpers::unpack_contiguous_list_data(*res_of(res), *ix, data,
                                                 uint32_t(out_codes->dl_tensor.shape[0]), label, offset);
  });
}

// ------------------------------------------------------------------------------------------------
// single-list helpers (C++ only in the reference: ivf_pq.hpp:2564-3166, namespace helpers)
// ------------------------------------------------------------------------------------------------
namespace {
const uint32_t* optional_row_indices(DLManagedTensor* t, int64_t n_rows)
{
  if (t == nullptr) { return nullptr; }
  auto* p = static_cast<const uint32_t*>(checked_data(t, kDLUInt, 32, 1, true, "in_cluster_indices"));
  CUVS_EXPECTS(t->dl_tensor.shape[0] == n_rows, "in_cluster_indices must have one entry per output row");
  return p;
}
}  // namespace

extern "C" cuvsError_t cuvsIvfPqHelpersUnpackListData(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                                      DLManagedTensor* out_codes, uint32_t label,
                                                      uint32_t offset, DLManagedTensor* in_cluster_indices)
{
  return translate_exceptions([=] {
    auto* ix   = index_of(index);
    auto* data = static_cast<uint8_t*>(checked_data(out_codes, kDLUInt, 8, 2, true, "out_codes"));
    CUVS_EXPECTS(out_codes->dl_tensor.shape[1] == int64_t(ix->pq_dim()), "out_codes must have pq_dim columns");
    const int64_t n = out_codes->dl_tensor.shape[0];
    ivf_pq::helpers::codepacker::unpack_list_data(*res_of(res), *ix, data, uint32_t(n), label, offset,
                                                  optional_row_indices(in_cluster_indices, n));
  });
}

extern "C" cuvsError_t cuvsIvfPqHelpersPackListData(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                                    DLManagedTensor* codes, uint32_t label, uint32_t offset)
{
  return translate_exceptions([=] {
    auto* ix   = index_of(index);
    auto* data = static_cast<const uint8_t*>(checked_data(codes, kDLUInt, 8, 2, true, "codes"));
    CUVS_EXPECTS(codes->dl_tensor.shape[1] == int64_t(ix->pq_dim()), "codes must have pq_dim columns");
    ivf_pq::helpers::codepacker::pack_list_data(*res_of(res), ix, data, uint32_t(codes->dl_tensor.shape[0]),
                                                label, offset);
  });
}

extern "C" cuvsError_t cuvsIvfPqHelpersPackContiguousListData(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                                              DLManagedTensor* codes, uint32_t label,
                                                              uint32_t offset)
{
  return translate_exceptions([=] {
    auto* ix   = index_of(index);
    auto* data = static_cast<const uint8_t*>(checked_data(codes, kDLUInt, 8, 2, true, "codes"));
    CUVS_EXPECTS(codes->dl_tensor.shape[1] == int64_t(cuvs_b200::ceildiv(ix->pq_dim() * ix->pq_bits(), 8u)),
                 "codes must have ceil(pq_dim * pq_bits / 8) columns");
    ivf_pq::helpers::codepacker::pack_contiguous_list_data(*res_of(res), ix, data,
                                                           uint32_t(codes->dl_tensor.shape[0]), label, offset);
  });
}

extern "C" cuvsError_t cuvsIvfPqHelpersReconstructListData(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                                           DLManagedTensor* out_vectors, uint32_t label,
                                                           uint32_t offset, DLManagedTensor* in_cluster_indices)
{
  return translate_exceptions([=] {
    auto* ix = index_of(index);
    CUVS_EXPECTS(out_vectors != nullptr, "null out_vectors");
    const DLTensor& t = out_vectors->dl_tensor;
    auto et           = elem_of_dtype(t.dtype, "out_vectors");
    void* data        = checked_data(out_vectors, t.dtype.code, t.dtype.bits, 2, true, "out_vectors");
    CUVS_EXPECTS(t.shape[1] == int64_t(ix->dim()), "out_vectors must have dim columns");
    ivf_pq::helpers::codepacker::reconstruct_list_data(*res_of(res), *ix, data, et, uint32_t(t.shape[0]), label,
                                                       offset, optional_row_indices(in_cluster_indices, t.shape[0]));
  });
}

extern "C" cuvsError_t cuvsIvfPqHelpersExtendListWithCodes(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                                           DLManagedTensor* new_codes,
                                                           DLManagedTensor* new_indices, uint32_t label,
                                                           bool contiguous)
{
  return translate_exceptions([=] {
    auto* ix   = index_of(index);
    auto* data = static_cast<const uint8_t*>(checked_data(new_codes, kDLUInt, 8, 2, true, "new_codes"));
    auto* ids  = static_cast<const int64_t*>(checked_data(new_indices, kDLInt, 64, 1, true, "new_indices"));
    const int64_t n = new_codes->dl_tensor.shape[0];
    CUVS_EXPECTS(new_indices->dl_tensor.shape[0] == n, "new_indices must have one entry per new row");
    const uint32_t cols = contiguous ? cuvs_b200::ceildiv(ix->pq_dim() * ix->pq_bits(), 8u) : ix->pq_dim();
    CUVS_EXPECTS(new_codes->dl_tensor.shape[1] == int64_t(cols), "new_codes must have %u columns", cols);
    if (contiguous) {
      ivf_pq::helpers::codepacker::extend_list_with_contiguous_codes(*res_of(res), ix, data, ids, uint32_t(n), label);
    } else {
      ivf_pq::helpers::codepacker::extend_list_with_codes(*res_of(res), ix, data, ids, uint32_t(n), label);
    }
  });
}

extern "C" cuvsError_t cuvsIvfPqHelpersExtendList(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                                  DLManagedTensor* new_vectors, DLManagedTensor* new_indices,
                                                  uint32_t label)
{
  return translate_exceptions([=] {
    auto* ix = index_of(index);
    CUVS_EXPECTS(new_vectors != nullptr, "null new_vectors");
    const DLTensor& t = new_vectors->dl_tensor;
    auto et           = elem_of_dtype(t.dtype, "new_vectors");
    void* data        = checked_data(new_vectors, t.dtype.code, t.dtype.bits, 2, true, "new_vectors");
    auto* ids = static_cast<const int64_t*>(checked_data(new_indices, kDLInt, 64, 1, true, "new_indices"));
    CUVS_EXPECTS(t.shape[1] == int64_t(ix->dim()), "new_vectors has the wrong number of columns");
    CUVS_EXPECTS(new_indices->dl_tensor.shape[0] == t.shape[0], "new_indices must have one entry per new vector");
    ivf_pq::helpers::codepacker::extend_list(*res_of(res), ix, data, et, ids, uint32_t(t.shape[0]), label);
  });
}

extern "C" cuvsError_t cuvsIvfPqHelpersEraseList(cuvsResources_t res, cuvsIvfPqIndex_t index, uint32_t label)
{
  return translate_exceptions([=] { ivf_pq::helpers::erase_list(*res_of(res), index_of(index), label); });
}

extern "C" cuvsError_t cuvsIvfPqHelpersResetIndex(cuvsResources_t res, cuvsIvfPqIndex_t index)
{
  return translate_exceptions([=] { ivf_pq::helpers::reset_index(*res_of(res), index_of(index)); });
}

// ------------------------------------------------------------------------------------------------
// build / extend / transform
// ------------------------------------------------------------------------------------------------
extern "C" cuvsError_t cuvsIvfPqBuild(cuvsResources_t res, cuvsIvfPqIndexParams_t params,
                                      DLManagedTensor* dataset_tensor, cuvsIvfPqIndex_t index)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(params != nullptr && dataset_tensor != nullptr && index != nullptr, "null argument");
    const DLTensor& t = dataset_tensor->dl_tensor;
    auto et           = elem_of_dtype(t.dtype, "dataset");
    const bool on_dev = is_device_compatible(t);
    void* data        = checked_data(dataset_tensor, t.dtype.code, t.dtype.bits, 2, on_dev, "dataset");
    auto* ix          = new index_t();
    try {
      ivf_pq::build_any(*res_of(res), convert(*params), data, et, t.shape[0], uint32_t(t.shape[1]),
                        on_dev, ix);
    } catch (...) {
      delete ix;
      throw;
    }
    delete reinterpret_cast<index_t*>(index->addr);
    index->addr       = reinterpret_cast<uintptr_t>(ix);
    index->dtype.code = t.dtype.code;
    index->dtype.bits = t.dtype.bits;
    index->dtype.lanes = 1;
  });
}

extern "C" cuvsError_t cuvsIvfPqBuildPrecomputed(cuvsResources_t res, cuvsIvfPqIndexParams_t params,
                                                 uint32_t dim, DLManagedTensor* pq_centers,
                                                 DLManagedTensor* centers, DLManagedTensor* centers_rot,
                                                 DLManagedTensor* rotation_matrix,
                                                 cuvsIvfPqIndex_t index)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(params != nullptr && index != nullptr, "null argument");
    auto* r   = res_of(res);
    auto ip   = convert(*params);
    auto* ix  = new index_t(ip.metric, ip.codebook_kind, ip.n_lists, dim, ip.pq_bits, ip.pq_dim,
                            ip.conservative_memory_allocation, ip.codes_layout);
    try {
      auto* pqc = static_cast<float*>(checked_data(pq_centers, kDLFloat, 32, 3, true, "pq_centers"));
      auto* cen = static_cast<float*>(checked_data(centers, kDLFloat, 32, 2, true, "centers"));
      auto* rot = static_cast<float*>(checked_data(centers_rot, kDLFloat, 32, 2, true, "centers_rot"));
      auto* rm  = static_cast<float*>(checked_data(rotation_matrix, kDLFloat, 32, 2, true, "rotation_matrix"));
      const auto& ps = pq_centers->dl_tensor;
      const int64_t first = ip.codebook_kind == ivf_pq::codebook_gen::PER_SUBSPACE ? ix->pq_dim() : ix->n_lists();
      CUVS_EXPECTS(ps.shape[0] == first && ps.shape[1] == ix->pq_len() && ps.shape[2] == ix->pq_book_size(),
                   "pq_centers has the wrong shape");
      CUVS_EXPECTS(centers_rot->dl_tensor.shape[0] == ix->n_lists() &&
                     centers_rot->dl_tensor.shape[1] == ix->rot_dim(),
                   "centers_rot must be [n_lists, rot_dim]");
      CUVS_EXPECTS(rotation_matrix->dl_tensor.shape[0] == ix->rot_dim() &&
                     rotation_matrix->dl_tensor.shape[1] == ix->dim(),
                   "rotation_matrix must be [rot_dim, dim]");
      const auto& cs = centers->dl_tensor;
      CUVS_EXPECTS(cs.shape[0] == ix->n_lists() && (cs.shape[1] == ix->dim() || cs.shape[1] == ix->dim_ext()),
                   "centers must be [n_lists, dim] or [n_lists, dim_ext]");
      ivf_pq::helpers::set_model(*r, ix, pqc, cen, uint32_t(cs.shape[1]), rot, rm);
    } catch (...) {
      delete ix;
      throw;
    }
    delete reinterpret_cast<index_t*>(index->addr);
    index->addr  = reinterpret_cast<uintptr_t>(ix);
    index->dtype = DLDataType{0, 0, 0};
  });
}

extern "C" cuvsError_t cuvsIvfPqExtend(cuvsResources_t res, DLManagedTensor* new_vectors,
                                       DLManagedTensor* new_indices, cuvsIvfPqIndex_t index)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(new_vectors != nullptr, "null new_vectors");
    auto* ix          = index_of(index);
    const DLTensor& t = new_vectors->dl_tensor;
    auto et           = elem_of_dtype(t.dtype, "index");
    const bool on_dev = is_device_compatible(t);
    if (new_indices) {
      CUVS_EXPECTS(on_dev == is_device_compatible(new_indices->dl_tensor),
                   "extend inputs must both either be on device memory or host memory");
    }
    if (index->dtype.code == 0 && index->dtype.bits == 0) {
      index->dtype.code = t.dtype.code;
      index->dtype.bits = t.dtype.bits;
    }
    void* data = checked_data(new_vectors, t.dtype.code, t.dtype.bits, 2, on_dev, "new_vectors");
    const int64_t* ids = nullptr;
    if (new_indices) {
      ids = static_cast<const int64_t*>(checked_data(new_indices, kDLInt, 64, 1, on_dev, "new_indices"));
      CUVS_EXPECTS(new_indices->dl_tensor.shape[0] == t.shape[0],
                   "new_indices must have one entry per new vector");
    }
    CUVS_EXPECTS(uint32_t(t.shape[1]) == ix->dim(), "new_vectors has the wrong number of columns");
    ivf_pq::extend_any(*res_of(res), data, et, t.shape[0], ids, on_dev, ix);
  });
}

extern "C" cuvsError_t cuvsIvfPqTransform(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                          DLManagedTensor* input_dataset,
                                          DLManagedTensor* output_labels,
                                          DLManagedTensor* output_dataset)
{
  return translate_exceptions([=] {
    auto* ix          = index_of(index);
    const DLTensor& t = input_dataset->dl_tensor;
    auto et           = elem_of_dtype(t.dtype, "dataset");
    void* data   = checked_data(input_dataset, t.dtype.code, t.dtype.bits, 2, true, "input_dataset");
    auto* labels = static_cast<uint32_t*>(checked_data(output_labels, kDLUInt, 32, 1, true, "output_labels"));
    auto* codes  = static_cast<uint8_t*>(checked_data(output_dataset, kDLUInt, 8, 2, true, "output_dataset"));
    CUVS_EXPECTS(uint32_t(t.shape[1]) == ix->dim(), "input_dataset has the wrong number of columns");
    CUVS_EXPECTS(output_labels->dl_tensor.shape[0] == t.shape[0] &&
                   output_dataset->dl_tensor.shape[0] == t.shape[0],
                 "outputs must have one row per input vector");
    CUVS_EXPECTS(output_dataset->dl_tensor.shape[1] ==
                   int64_t(cuvs_b200::ceildiv(ix->pq_dim() * ix->pq_bits(), 8u)),
                 "output_dataset must have ceil(pq_dim * pq_bits / 8) columns");
    ivf_pq::transform_any(*res_of(res), *ix, data, et, t.shape[0], labels, codes);
  });
}

// ------------------------------------------------------------------------------------------------
// search / serialize / deserialize
// ------------------------------------------------------------------------------------------------
namespace {
void search_entry(cuvsResources_t res, cuvsIvfPqSearchParams_t params, cuvsIvfPqIndex_t index,
                  DLManagedTensor* queries_tensor, DLManagedTensor* neighbors_tensor,
                  DLManagedTensor* distances_tensor, ivf_pq::bitset_view filter)
{
  CUVS_EXPECTS(params && queries_tensor && neighbors_tensor && distances_tensor, "null argument");
  const DLTensor& queries   = queries_tensor->dl_tensor;
  const DLTensor& neighbors = neighbors_tensor->dl_tensor;
  const DLTensor& distances = distances_tensor->dl_tensor;
  // c/src/neighbors/ivf_pq.cpp:315-325
  CUVS_EXPECTS(is_device_compatible(queries), "queries should have device compatible memory");
  CUVS_EXPECTS(is_device_compatible(neighbors), "neighbors should have device compatible memory");
  CUVS_EXPECTS(is_device_compatible(distances), "distances should have device compatible memory");
  CUVS_EXPECTS(neighbors.dtype.code == kDLInt && neighbors.dtype.bits == 64,
               "neighbors should be of type int64_t");
  CUVS_EXPECTS(distances.dtype.code == kDLFloat && distances.dtype.bits == 32,
               "distances should be of type float32");
  auto* ix = index_of(index);
  auto et  = elem_of_dtype(queries.dtype, "queries");
  void* q  = checked_data(queries_tensor, queries.dtype.code, queries.dtype.bits, 2, true, "queries");
  auto* nb = static_cast<int64_t*>(checked_data(neighbors_tensor, kDLInt, 64, 2, true, "neighbors"));
  auto* ds = static_cast<float*>(checked_data(distances_tensor, kDLFloat, 32, 2, true, "distances"));
  // ivf_pq_search.cuh:1080-1108
  CUVS_EXPECTS(queries.shape[0] == neighbors.shape[0] && queries.shape[0] == distances.shape[0],
               "Number of rows in output neighbors and distances matrices must equal the number "
               "of queries.");
  CUVS_EXPECTS(neighbors.shape[1] == distances.shape[1],
               "Number of columns in output neighbors and distances matrices must equal k");
  CUVS_EXPECTS(queries.shape[1] == int64_t(ix->dim()),
               "Number of query dimensions should equal number of dimensions in the index.");
  ivf_pq::search_params sp;
  sp.n_probes                 = params->n_probes;
  sp.lut_dtype                = params->lut_dtype;
  sp.internal_distance_dtype  = params->internal_distance_dtype;
  sp.preferred_shmem_carveout = params->preferred_shmem_carveout;
  sp.coarse_search_dtype      = params->coarse_search_dtype;
  sp.max_internal_batch_size  = params->max_internal_batch_size;
  ivf_pq::search_any(*res_of(res), sp, *ix, q, et, uint32_t(queries.shape[0]),
                     uint32_t(neighbors.shape[1]), nb, ds, nullptr, filter);
}
}  // namespace

extern "C" cuvsError_t cuvsIvfPqSearch(cuvsResources_t res, cuvsIvfPqSearchParams_t params,
                                       cuvsIvfPqIndex_t index, DLManagedTensor* queries_tensor,
                                       DLManagedTensor* neighbors_tensor,
                                       DLManagedTensor* distances_tensor)
{
  return translate_exceptions(
    [=] { search_entry(res, params, index, queries_tensor, neighbors_tensor, distances_tensor, {}); });
}

extern "C" cuvsError_t cuvsIvfPqSearchWithFilter(cuvsResources_t res, cuvsIvfPqSearchParams_t params,
                                                 cuvsIvfPqIndex_t index, DLManagedTensor* queries_tensor,
                                                 DLManagedTensor* neighbors_tensor,
                                                 DLManagedTensor* distances_tensor, cuvsFilter filter)
{
  return translate_exceptions([=] {
    ivf_pq::bitset_view view{};
    if (filter.type == BITSET) {
      auto* bt = reinterpret_cast<DLManagedTensor*>(filter.addr);
      view.bits = static_cast<const uint32_t*>(checked_data(bt, kDLUInt, 32, 1, true, "filter bitset"));
      view.n_bits = uint64_t(bt->dl_tensor.shape[0]) * 32u;
    } else {
      CUVS_EXPECTS(filter.type == NO_FILTER, "Unsupported sample filter type");
    }
    search_entry(res, params, index, queries_tensor, neighbors_tensor, distances_tensor, view);
  });
}

extern "C" cuvsError_t cuvsIvfPqSerialize(cuvsResources_t res, const char* filename,
                                          cuvsIvfPqIndex_t index)
{
  return translate_exceptions(
    [=] { ivf_pq::serialize(*res_of(res), std::string(filename), *index_of(index)); });
}

extern "C" cuvsError_t cuvsIvfPqDeserialize(cuvsResources_t res, const char* filename,
                                            cuvsIvfPqIndex_t index)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(index != nullptr && filename != nullptr, "null argument");
    auto* ix = new index_t();
    try {
      ivf_pq::deserialize(*res_of(res), std::string(filename), ix);
    } catch (...) {
      delete ix;
      throw;
    }
    delete reinterpret_cast<index_t*>(index->addr);
    index->addr = reinterpret_cast<uintptr_t>(ix);
  });
}

// ------------------------------------------------------------------------------------------------
// one-process-per-GPU list sharding
// ------------------------------------------------------------------------------------------------
extern "C" cuvsError_t cuvsMultiGpuIvfPqDistributeShard(cuvsResources_t res, const char* filename,
                                                        int rank, int n_ranks, cuvsIvfPqIndex_t index)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(index != nullptr && filename != nullptr, "null argument");
    auto* ix = new index_t();
    try {
      ivf_pq::deserialize(*res_of(res), std::string(filename), ix, rank, n_ranks);
    } catch (...) {
      delete ix;
      throw;
    }
    delete reinterpret_cast<index_t*>(index->addr);
    index->addr = reinterpret_cast<uintptr_t>(ix);
  });
}

extern "C" cuvsError_t cuvsMultiGpuIvfPqDeserializeRank(cuvsResources_t res, const char* filename, int rank,
                                                        int n_ranks, cuvsIvfPqIndex_t index, int* mode,
                                                        int64_t* id_offset)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(index && filename && mode && id_offset, "null argument");
    auto* ix = new index_t();
    try {
      ivf_pq::deserialize_mg_rank(*res_of(res), std::string(filename), rank, n_ranks, ix, mode, id_offset);
    } catch (...) {
      delete ix;
      throw;
    }
    delete reinterpret_cast<index_t*>(index->addr);
    index->addr = reinterpret_cast<uintptr_t>(ix);
  });
}

extern "C" cuvsError_t cuvsMultiGpuIvfPqSerializeRanks(cuvsResources_t res, const char* filename, int mode,
                                                       DLDataType dataset_dtype, cuvsIvfPqIndex_t* indexes,
                                                       int n_ranks)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(filename && indexes && n_ranks > 0, "null argument");
    // numpy dtype strings as raft::numpy_serializer::get_numpy_dtype<T>() spells them
    const char* ds = nullptr;
    switch (elem_of_dtype(dataset_dtype, "dataset")) {
      case ivf_pq::elem_t::f32: ds = "<f4"; break;
      case ivf_pq::elem_t::f16: ds = "<f2"; break;
      case ivf_pq::elem_t::i8: ds = "|i1"; break;
      default: ds = "|u1"; break;
    }
    std::vector<const index_t*> per_rank;
    for (int r = 0; r < n_ranks; r++) { per_rank.push_back(index_of(indexes[r])); }
    ivf_pq::serialize_mg(*res_of(res), std::string(filename), mode, ds, per_rank);
  });
}

extern "C" cuvsError_t cuvsMultiGpuIvfPqMergeParts(cuvsResources_t res, DLManagedTensor* part_distances,
                                                   DLManagedTensor* part_neighbors,
                                                   DLManagedTensor* distances, DLManagedTensor* neighbors,
                                                   bool select_min)
{
  return translate_exceptions([=] {
    // the parts may lie apart (one stride between them): e.g. views into one gathered buffer
    size_t stride_d = 0, stride_n = 0;
    auto* pd = static_cast<float*>(checked_parts(part_distances, kDLFloat, 32, "part_distances", &stride_d));
    auto* pn = static_cast<int64_t*>(checked_parts(part_neighbors, kDLInt, 64, "part_neighbors", &stride_n));
    auto* od = static_cast<float*>(checked_data(distances, kDLFloat, 32, 2, true, "distances"));
    auto* on = static_cast<int64_t*>(checked_data(neighbors, kDLInt, 64, 2, true, "neighbors"));
    const int64_t* ps = part_distances->dl_tensor.shape;
    const int64_t* ns = part_neighbors->dl_tensor.shape;
    CUVS_EXPECTS(ps[0] == ns[0] && ps[1] == ns[1] && ps[2] == ns[2],
                 "part_distances and part_neighbors must have the same shape");
    for (auto* t : {distances, neighbors}) {
      CUVS_EXPECTS(t->dl_tensor.shape[0] == ps[1] && t->dl_tensor.shape[1] == ps[2],
                   "outputs must be [n_queries, k]");
    }
    ivf_pq::detail::knn_merge_parts(*res_of(res), pd, pn, od, on, uint32_t(ps[0]), uint32_t(ps[1]),
                                    uint32_t(ps[2]), select_min, stride_d, stride_n);
  });
}

// ------------------------------------------------------------------------------------------------
// instrumentation
// ------------------------------------------------------------------------------------------------
extern "C" cuvsError_t cuvsB200StatsEnable(cuvsResources_t res, bool enable)
{
  return translate_exceptions([=] { res_of(res)->stats_enable(enable); });
}

extern "C" cuvsError_t cuvsB200StatsGet(cuvsResources_t res, cuvsB200SearchStats* out, bool reset)
{
  return translate_exceptions([=] {
    auto* r = res_of(res);
    CUVS_EXPECTS(out != nullptr, "null output");
    r->stats_resolve();
    unsigned long long h[2] = {0, 0};
    if (r->d_stats) { CUDA_TRY(cudaMemcpy(h, r->d_stats, 16, cudaMemcpyDeviceToHost)); }
    out->prep_ms       = r->stage_ms[0];
    out->coarse_ms     = r->stage_ms[1];
    out->sort_ms       = r->stage_ms[2];
    out->scan_ms       = r->stage_ms[3];
    out->merge_ms      = r->stage_ms[4];
    out->batches       = r->stat_batches;
    out->pairs         = r->stat_pairs;
    out->scan_groups   = h[0];
    out->unique_groups = h[1];
    out->launches      = r->launches;
    if (reset) {
      for (auto& v : r->stage_ms) { v = 0; }
      r->stat_batches = 0;
      r->stat_pairs   = 0;
      if (r->d_stats) { CUDA_TRY(cudaMemset(r->d_stats, 0, 16)); }
    }
  });
}

extern "C" cuvsError_t cuvsB200CoarseSelect(cuvsResources_t res, void* index_handle,
                                            DLManagedTensor* queries, DLManagedTensor* probes,
                                            DLManagedTensor* scores, int mode, uint32_t* status)
{
  return translate_exceptions([=] {
    auto* ix          = index_of(static_cast<cuvsIvfPqIndex_t>(index_handle));
    const DLTensor& q = queries->dl_tensor;
    auto et           = elem_of_dtype(q.dtype, "queries");
    void* qd   = checked_data(queries, q.dtype.code, q.dtype.bits, 2, true, "queries");
    auto* pd   = static_cast<uint32_t*>(checked_data(probes, kDLUInt, 32, 2, true, "probes"));
    auto* sd   = static_cast<float*>(checked_data(scores, kDLFloat, 32, 2, true, "scores"));
    CUVS_EXPECTS(q.shape[1] == int64_t(ix->dim()), "queries have the wrong number of columns");
    CUVS_EXPECTS(probes->dl_tensor.shape[0] == q.shape[0] && scores->dl_tensor.shape[0] == q.shape[0] &&
                   probes->dl_tensor.shape[1] == scores->dl_tensor.shape[1],
                 "probes and scores must be [n_queries, n_probes]");
    CUVS_EXPECTS(status != nullptr, "null status");
    ivf_pq::coarse_only(*res_of(res), *ix, qd, et, uint32_t(q.shape[0]),
                        uint32_t(probes->dl_tensor.shape[1]), mode, pd, sd, status);
  });
}

extern "C" cuvsError_t cuvsB200SetCoarseMode(int mode)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS((mode >= 0 && mode <= 2) || (mode >= 11 && mode <= 13) || mode == 21 || mode == 22,
                 "mode must be 0, 1, 2, 11, 12, 13, 21 or 22");
    ivf_pq::set_coarse_mode(mode);
  });
}

extern "C" cuvsError_t cuvsB200CoarseTimeouts(cuvsResources_t res, uint64_t* n_batches)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(n_batches != nullptr, "null output pointer");
    auto* r = res_of(res);
    r->adopt_tc_verdict();
    *n_batches = r->tc_timeouts;
  });
}

extern "C" cuvsError_t cuvsB200SetCoarseWaitTest(uint32_t spin_limit, uint32_t skip_stage)
{
  return translate_exceptions([=] {
    // a limit below 1000 iterations could fire on a healthy but busy GPU
    CUVS_EXPECTS(spin_limit == 0 || spin_limit >= 1000, "spin_limit must be 0 or at least 1000");
    ivf_pq::set_coarse_tc_wait_test(spin_limit, skip_stage);
  });
}

extern "C" cuvsError_t cuvsB200SetScanCodebookHome(int home)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(home >= 0 && home <= 3, "home must be 0, 1, 2 or 3");
    ivf_pq::set_scan_codebook_home(home);
  });
}

// ------------------------------------------------------------------------------------------------
// dynamic batching (C++ only in the reference: cpp/include/cuvs/neighbors/dynamic_batching.hpp)
// ------------------------------------------------------------------------------------------------
namespace db = cuvs::neighbors::dynamic_batching;

extern "C" cuvsError_t cuvsDynamicBatchingIndexParamsCreate(cuvsDynamicBatchingIndexParams_t* params)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(params != nullptr, "null argument");
    *params = new cuvsDynamicBatchingIndexParams{10, 100, 3, false};
  });
}
extern "C" cuvsError_t cuvsDynamicBatchingIndexParamsDestroy(cuvsDynamicBatchingIndexParams_t params)
{
  return translate_exceptions([=] { delete params; });
}
extern "C" cuvsError_t cuvsDynamicBatchingIndexCreate(cuvsResources_t res, cuvsDynamicBatchingIndexParams_t params,
                                                      cuvsIvfPqIndex_t upstream,
                                                      cuvsIvfPqSearchParams_t upstream_params,
                                                      cuvsDynamicBatchingIndex_t* index)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(params && upstream_params && index, "null argument");
    auto* ix = index_of(upstream);
    CUVS_EXPECTS(params->k > 0 && params->k <= ix->size(), "k must be within [1, index size]");
    db::index_params ip;
    ip.k                     = params->k;
    ip.max_batch_size        = params->max_batch_size;
    ip.n_queues              = params->n_queues;
    ip.conservative_dispatch = params->conservative_dispatch;
    ivf_pq::search_params sp;
    sp.n_probes                 = upstream_params->n_probes;
    sp.lut_dtype                = upstream_params->lut_dtype;
    sp.internal_distance_dtype  = upstream_params->internal_distance_dtype;
    sp.preferred_shmem_carveout = upstream_params->preferred_shmem_carveout;
    sp.coarse_search_dtype      = upstream_params->coarse_search_dtype;
    sp.max_internal_batch_size  = upstream_params->max_internal_batch_size;
    auto* obj = new db::index<float, int64_t>(*res_of(res), ip, *ix, sp);
    *index    = new cuvsDynamicBatchingIndex{reinterpret_cast<uintptr_t>(obj)};
  });
}
extern "C" cuvsError_t cuvsDynamicBatchingIndexDestroy(cuvsDynamicBatchingIndex_t index)
{
  return translate_exceptions([=] {
    if (index) {
      delete reinterpret_cast<db::index<float, int64_t>*>(index->addr);
      delete index;
    }
  });
}
extern "C" cuvsError_t cuvsDynamicBatchingSearch(cuvsResources_t res, cuvsDynamicBatchingIndex_t index,
                                                 double dispatch_timeout_ms, DLManagedTensor* queries,
                                                 DLManagedTensor* neighbors, DLManagedTensor* distances)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(index && index->addr && queries && neighbors && distances, "null argument");
    auto* obj = reinterpret_cast<db::index<float, int64_t>*>(index->addr);
    auto* q   = static_cast<const float*>(checked_data(queries, kDLFloat, 32, 2, true, "queries"));
    auto* nb  = static_cast<int64_t*>(checked_data(neighbors, kDLInt, 64, 2, true, "neighbors"));
    auto* ds  = static_cast<float*>(checked_data(distances, kDLFloat, 32, 2, true, "distances"));
    const int64_t n = queries->dl_tensor.shape[0];
    CUVS_EXPECTS(neighbors->dl_tensor.shape[0] == n && distances->dl_tensor.shape[0] == n,
                 "Number of rows in output neighbors and distances matrices must equal the number "
                 "of queries.");
    CUVS_EXPECTS(neighbors->dl_tensor.shape[1] == distances->dl_tensor.shape[1],
                 "Number of columns in output neighbors and distances matrices must equal k");
    db::search_params sp;
    sp.dispatch_timeout_ms = dispatch_timeout_ms;
    db::search_checked(*res_of(res), sp, *obj, q, uint32_t(n), uint32_t(queries->dl_tensor.shape[1]),
                       uint32_t(neighbors->dl_tensor.shape[1]), nb, ds);
  });
}
extern "C" cuvsError_t cuvsDynamicBatchingFailNext(cuvsDynamicBatchingIndex_t index)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(index && index->addr, "null argument");
    db::fail_next_upstream_search(*reinterpret_cast<db::index<float, int64_t>*>(index->addr));
  });
}
extern "C" cuvsError_t cuvsDynamicBatchingStats(cuvsDynamicBatchingIndex_t index, uint64_t* n_batches,
                                                uint64_t* n_rows)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(index && index->addr && n_batches && n_rows, "null argument");
    db::stats(*reinterpret_cast<db::index<float, int64_t>*>(index->addr), n_batches, n_rows);
  });
}

// ------------------------------------------------------------------------------------------------
// refine (c/src/neighbors/refine.cpp)
// ------------------------------------------------------------------------------------------------
extern "C" cuvsError_t cuvsRefine(cuvsResources_t res, DLManagedTensor* dataset, DLManagedTensor* queries,
                                  DLManagedTensor* candidates, cuvsDistanceType metric,
                                  DLManagedTensor* indices, DLManagedTensor* distances)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(dataset && queries && candidates && indices && distances, "null argument");
    const DLTensor& d = dataset->dl_tensor;
    const DLTensor& q = queries->dl_tensor;
    auto et           = elem_of_dtype(d.dtype, "dataset");
    CUVS_EXPECTS(q.dtype.code == d.dtype.code && q.dtype.bits == d.dtype.bits,
                 "dataset and queries must have the same element type");
    void* dd = checked_data(dataset, d.dtype.code, d.dtype.bits, 2, true, "dataset");
    void* qd = checked_data(queries, q.dtype.code, q.dtype.bits, 2, true, "queries");
    auto* cd = static_cast<int64_t*>(checked_data(candidates, kDLInt, 64, 2, true, "candidates"));
    auto* id = static_cast<int64_t*>(checked_data(indices, kDLInt, 64, 2, true, "indices"));
    auto* dsd = static_cast<float*>(checked_data(distances, kDLFloat, 32, 2, true, "distances"));
    CUVS_EXPECTS(q.shape[1] == d.shape[1], "dataset and queries must have the same number of columns");
    CUVS_EXPECTS(candidates->dl_tensor.shape[0] == q.shape[0] && indices->dl_tensor.shape[0] == q.shape[0] &&
                   distances->dl_tensor.shape[0] == q.shape[0],
                 "candidates, indices and distances must have one row per query");
    CUVS_EXPECTS(indices->dl_tensor.shape[1] == distances->dl_tensor.shape[1],
                 "indices and distances must have the same number of columns");
    cuvs::neighbors::refine_any(*res_of(res), dd, et, d.shape[0], uint32_t(d.shape[1]), qd,
                                uint32_t(q.shape[0]), cd, uint32_t(candidates->dl_tensor.shape[1]),
                                ivf_pq::DistanceType(int(metric)), id, dsd,
                                uint32_t(indices->dl_tensor.shape[1]));
  });
}

extern "C" cuvsError_t cuvsMultiGpuIvfPqSelectProbes(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                                     DLManagedTensor* queries, DLManagedTensor* probes)
{
  return translate_exceptions([=] {
    auto* ix          = index_of(index);
    const DLTensor& q = queries->dl_tensor;
    auto et           = elem_of_dtype(q.dtype, "queries");
    void* qd = checked_data(queries, q.dtype.code, q.dtype.bits, 2, true, "queries");
    auto* pd = static_cast<uint32_t*>(checked_data(probes, kDLUInt, 32, 2, true, "probes"));
    CUVS_EXPECTS(q.shape[1] == int64_t(ix->dim()),
                 "Number of query dimensions should equal number of dimensions in the index.");
    CUVS_EXPECTS(probes->dl_tensor.shape[0] == q.shape[0], "probes must have one row per query");
    ivf_pq::select_probes_any(*res_of(res), *ix, qd, et, uint32_t(q.shape[0]),
                              uint32_t(probes->dl_tensor.shape[1]), pd);
  });
}

extern "C" cuvsError_t cuvsMultiGpuIvfPqSearchWithProbes(cuvsResources_t res,
                                                         cuvsIvfPqSearchParams_t params,
                                                         cuvsIvfPqIndex_t index, DLManagedTensor* queries,
                                                         DLManagedTensor* probes,
                                                         DLManagedTensor* neighbors,
                                                         DLManagedTensor* distances)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(params && queries && probes && neighbors && distances, "null argument");
    auto* ix          = index_of(index);
    const DLTensor& q = queries->dl_tensor;
    auto et           = elem_of_dtype(q.dtype, "queries");
    void* qd = checked_data(queries, q.dtype.code, q.dtype.bits, 2, true, "queries");
    auto* pd = static_cast<uint32_t*>(checked_data(probes, kDLUInt, 32, 2, true, "probes"));
    auto* nb = static_cast<int64_t*>(checked_data(neighbors, kDLInt, 64, 2, true, "neighbors"));
    auto* ds = static_cast<float*>(checked_data(distances, kDLFloat, 32, 2, true, "distances"));
    CUVS_EXPECTS(q.shape[0] == neighbors->dl_tensor.shape[0] && q.shape[0] == distances->dl_tensor.shape[0] &&
                   q.shape[0] == probes->dl_tensor.shape[0],
                 "Number of rows in probes, neighbors and distances must equal the number of queries.");
    CUVS_EXPECTS(neighbors->dl_tensor.shape[1] == distances->dl_tensor.shape[1],
                 "Number of columns in output neighbors and distances matrices must equal k");
    CUVS_EXPECTS(q.shape[1] == int64_t(ix->dim()),
                 "Number of query dimensions should equal number of dimensions in the index.");
    ivf_pq::search_params sp;
    sp.n_probes                 = params->n_probes;
    sp.lut_dtype                = params->lut_dtype;
    sp.internal_distance_dtype  = params->internal_distance_dtype;
    sp.preferred_shmem_carveout = params->preferred_shmem_carveout;
    sp.coarse_search_dtype      = params->coarse_search_dtype;
    sp.max_internal_batch_size  = params->max_internal_batch_size;
    CUVS_EXPECTS(int64_t(std::min<uint32_t>(sp.n_probes, ix->n_lists())) == probes->dl_tensor.shape[1],
                 "probes must have min(n_probes, n_lists) columns");
    ivf_pq::search_any(*res_of(res), sp, *ix, qd, et, uint32_t(q.shape[0]),
                       uint32_t(neighbors->dl_tensor.shape[1]), nb, ds, pd);
  });
}

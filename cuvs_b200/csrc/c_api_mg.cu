// C interface of the multi-GPU layer: the entry points of include/cuvs_mg_ivf_pq.h (parts 1 and 2) and
// the multi-GPU resources of include/cuvs_core_c_api.h.  Mirrors c/src/neighbors/mg_ivf_pq.cpp and
// c/src/core/c_api.cpp:60-120 of the reference: same checks, same messages, host tensors for the
// single-process entries.
#include "../../include/cuvs_mg_ivf_pq.h"

#include "c_api_util.hpp"
#include "mg.hpp"

#include <cstdio>
#include <cstring>
#include <vector>

using namespace cuvs_b200::capi;
namespace mg = cuvs::neighbors::mg;

namespace {

mg::snmg_resources* clique_of(cuvsResources_t res)
{
  auto* r = res_of(res);
  CUVS_EXPECTS(r->kind == 1,
               "this call needs a multi-GPU resources handle (cuvsMultiGpuResourcesCreate)");
  return static_cast<mg::snmg_resources*>(r);
}

mg::mg_index* mg_index_of(cuvsMultiGpuIvfPqIndex_t index)
{
  CUVS_EXPECTS(index != nullptr && index->addr != 0, "the multi-GPU index handle holds no index");
  return reinterpret_cast<mg::mg_index*>(index->addr);
}

void install(cuvsMultiGpuIvfPqIndex_t index, mg::mg_index* fresh, DLDataType dtype)
{
  delete reinterpret_cast<mg::mg_index*>(index->addr);
  index->addr  = reinterpret_cast<uintptr_t>(fresh);
  index->dtype = dtype;
}

const char* numpy_dtype_string(const DLDataType& d)
{
  // as raft::numpy_serializer::get_numpy_dtype<T>() spells them
  switch (elem_of_dtype(d, "dataset")) {
    case ivf_pq::elem_t::f32: return "<f4";
    case ivf_pq::elem_t::f16: return "<f2";
    case ivf_pq::elem_t::i8: return "|i1";
    default: return "|u1";
  }
}

ivf_pq::search_params convert_search(const cuvsIvfPqSearchParams& p)
{
  ivf_pq::search_params sp;
  sp.n_probes                 = p.n_probes;
  sp.lut_dtype                = p.lut_dtype;
  sp.internal_distance_dtype  = p.internal_distance_dtype;
  sp.preferred_shmem_carveout = p.preferred_shmem_carveout;
  sp.coarse_search_dtype      = p.coarse_search_dtype;
  sp.max_internal_batch_size  = p.max_internal_batch_size;
  return sp;
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// resources
// ------------------------------------------------------------------------------------------------
extern "C" cuvsError_t cuvsMultiGpuResourcesCreate(cuvsResources_t* res)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(res != nullptr, "null output pointer");
    *res = reinterpret_cast<cuvsResources_t>(static_cast<cuvs_b200::resources*>(new mg::snmg_resources({})));
  });
}

extern "C" cuvsError_t cuvsMultiGpuResourcesCreateWithDeviceIds(cuvsResources_t* res, DLManagedTensor* device_ids)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(res != nullptr && device_ids != nullptr, "null argument");
    auto* ids = static_cast<const int32_t*>(checked_data(device_ids, kDLInt, 32, 1, false, "device_ids"));
    std::vector<int> v(ids, ids + device_ids->dl_tensor.shape[0]);
    CUVS_EXPECTS(!v.empty(), "device_ids is empty");
    *res = reinterpret_cast<cuvsResources_t>(static_cast<cuvs_b200::resources*>(new mg::snmg_resources(v)));
  });
}

extern "C" cuvsError_t cuvsMultiGpuResourcesDestroy(cuvsResources_t res)
{
  return translate_exceptions([=] { delete clique_of(res); });
}

extern "C" cuvsError_t cuvsMultiGpuResourcesSetMemoryPool(cuvsResources_t res, int percent_of_free_memory)
{
  return translate_exceptions([=] {
    auto* c = clique_of(res);
    CUVS_EXPECTS(percent_of_free_memory >= 0 && percent_of_free_memory <= 100, "percent_of_free_memory out of range");
    for (int r = 0; r < c->n_ranks(); r++) {
      int saved = 0;
      CUDA_TRY(cudaGetDevice(&saved));
      CUDA_TRY(cudaSetDevice(c->devices[size_t(r)]));
      size_t free_b = 0, total_b = 0;
      CUDA_TRY(cudaMemGetInfo(&free_b, &total_b));
      // the grow-only workspace of a rank is this engine's pool; cap the reservation at 4 GiB, far
      // beyond what a search batch needs
      const size_t want = std::min<size_t>(free_b / 100 * size_t(percent_of_free_memory), size_t(4) << 30);
      c->rank_res[size_t(r)]->ws.reserve(want);
      CUDA_TRY(cudaSetDevice(saved));
    }
  });
}

// ------------------------------------------------------------------------------------------------
// params and handles
// ------------------------------------------------------------------------------------------------
extern "C" cuvsError_t cuvsMultiGpuIvfPqIndexParamsCreate(cuvsMultiGpuIvfPqIndexParams_t* index_params)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(index_params != nullptr, "null output pointer");
    cuvsIvfPqIndexParams_t base = nullptr;
    CUVS_EXPECTS(cuvsIvfPqIndexParamsCreate(&base) == CUVS_SUCCESS, "cannot create the base parameters");
    *index_params = new cuvsMultiGpuIvfPqIndexParams{base, CUVS_NEIGHBORS_MG_SHARDED};
  });
}
extern "C" cuvsError_t cuvsMultiGpuIvfPqIndexParamsDestroy(cuvsMultiGpuIvfPqIndexParams_t index_params)
{
  return translate_exceptions([=] {
    if (index_params) {
      cuvsIvfPqIndexParamsDestroy(index_params->base_params);
      delete index_params;
    }
  });
}
extern "C" cuvsError_t cuvsMultiGpuIvfPqSearchParamsCreate(cuvsMultiGpuIvfPqSearchParams_t* params)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(params != nullptr, "null output pointer");
    cuvsIvfPqSearchParams_t base = nullptr;
    CUVS_EXPECTS(cuvsIvfPqSearchParamsCreate(&base) == CUVS_SUCCESS, "cannot create the base parameters");
    *params = new cuvsMultiGpuIvfPqSearchParams{base, CUVS_NEIGHBORS_MG_LOAD_BALANCER, CUVS_NEIGHBORS_MG_TREE_MERGE,
                                                int64_t(1) << 20};
  });
}
extern "C" cuvsError_t cuvsMultiGpuIvfPqSearchParamsDestroy(cuvsMultiGpuIvfPqSearchParams_t params)
{
  return translate_exceptions([=] {
    if (params) {
      cuvsIvfPqSearchParamsDestroy(params->base_params);
      delete params;
    }
  });
}
extern "C" cuvsError_t cuvsMultiGpuIvfPqIndexCreate(cuvsMultiGpuIvfPqIndex_t* index)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(index != nullptr, "null output pointer");
    *index = new cuvsMultiGpuIvfPqIndex{};
  });
}
extern "C" cuvsError_t cuvsMultiGpuIvfPqIndexDestroy(cuvsMultiGpuIvfPqIndex_t index)
{
  return translate_exceptions([=] {
    if (index) {
      delete reinterpret_cast<mg::mg_index*>(index->addr);
      delete index;
    }
  });
}

// ------------------------------------------------------------------------------------------------
// build / search / extend / files
// ------------------------------------------------------------------------------------------------
extern "C" cuvsError_t cuvsMultiGpuIvfPqBuild(cuvsResources_t res, cuvsMultiGpuIvfPqIndexParams_t params,
                                              DLManagedTensor* dataset_tensor, cuvsMultiGpuIvfPqIndex_t index)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(params && params->base_params && dataset_tensor && index, "null argument");
    const DLTensor& d = dataset_tensor->dl_tensor;
    CUVS_EXPECTS(is_host_compatible(d), "Multi-GPU IVF-PQ build requires dataset to have host compatible memory");
    auto et    = elem_of_dtype(d.dtype, "dataset");
    void* data = checked_data(dataset_tensor, d.dtype.code, d.dtype.bits, 2, false, "dataset");
    auto fresh = new mg::mg_index();
    try {
      mg::build(*clique_of(res), convert(*params->base_params),
                params->mode == CUVS_NEIGHBORS_MG_SHARDED ? mg::distribution_mode::SHARDED
                                                          : mg::distribution_mode::REPLICATED,
                data, et, d.shape[0], uint32_t(d.shape[1]), fresh);
    } catch (...) {
      delete fresh;
      throw;
    }
    install(index, fresh, DLDataType{d.dtype.code, d.dtype.bits, 1});
  });
}

extern "C" cuvsError_t cuvsMultiGpuIvfPqSearch(cuvsResources_t res, cuvsMultiGpuIvfPqSearchParams_t params,
                                               cuvsMultiGpuIvfPqIndex_t index, DLManagedTensor* queries_tensor,
                                               DLManagedTensor* neighbors_tensor, DLManagedTensor* distances_tensor)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(params && params->base_params && queries_tensor && neighbors_tensor && distances_tensor,
                 "null argument");
    const DLTensor& queries   = queries_tensor->dl_tensor;
    const DLTensor& neighbors = neighbors_tensor->dl_tensor;
    const DLTensor& distances = distances_tensor->dl_tensor;
    // c/src/neighbors/mg_ivf_pq.cpp:285-305
    CUVS_EXPECTS(is_host_compatible(queries), "Multi-GPU IVF-PQ search requires queries to have host compatible memory");
    CUVS_EXPECTS(is_host_compatible(neighbors),
                 "Multi-GPU IVF-PQ search requires neighbors to have host compatible memory");
    CUVS_EXPECTS(is_host_compatible(distances),
                 "Multi-GPU IVF-PQ search requires distances to have host compatible memory");
    CUVS_EXPECTS(neighbors.dtype.code == kDLInt && neighbors.dtype.bits == 64, "neighbors should be of type int64_t");
    CUVS_EXPECTS(distances.dtype.code == kDLFloat && distances.dtype.bits == 32, "distances should be of type float32");
    auto* ix = mg_index_of(index);
    CUVS_EXPECTS(queries.dtype.code == index->dtype.code && queries.dtype.bits == index->dtype.bits,
                 "type mismatch between index and queries");
    auto et  = elem_of_dtype(queries.dtype, "queries");
    void* q  = checked_data(queries_tensor, queries.dtype.code, queries.dtype.bits, 2, false, "queries");
    auto* nb = static_cast<int64_t*>(checked_data(neighbors_tensor, kDLInt, 64, 2, false, "neighbors"));
    auto* ds = static_cast<float*>(checked_data(distances_tensor, kDLFloat, 32, 2, false, "distances"));
    CUVS_EXPECTS(queries.shape[0] == neighbors.shape[0] && queries.shape[0] == distances.shape[0],
                 "Number of rows in output neighbors and distances matrices must equal the number of queries.");
    CUVS_EXPECTS(neighbors.shape[1] == distances.shape[1],
                 "Number of columns in output neighbors and distances matrices must equal k");
    CUVS_EXPECTS(!ix->parts.empty() && queries.shape[1] == int64_t(ix->parts[0]->dim()),
                 "Number of query dimensions should equal number of dimensions in the index.");
    mg::search_params sp;
    static_cast<ivf_pq::search_params&>(sp) = convert_search(*params->base_params);
    sp.search_mode      = params->search_mode == CUVS_NEIGHBORS_MG_LOAD_BALANCER ? mg::replicated_search_mode::LOAD_BALANCER
                                                                                 : mg::replicated_search_mode::ROUND_ROBIN;
    sp.merge_mode       = params->merge_mode == CUVS_NEIGHBORS_MG_TREE_MERGE ? mg::sharded_merge_mode::TREE_MERGE
                                                                             : mg::sharded_merge_mode::MERGE_ON_ROOT_RANK;
    sp.n_rows_per_batch = params->n_rows_per_batch;
    mg::search(*clique_of(res), *ix, sp, q, et, queries.shape[0], uint32_t(neighbors.shape[1]), nb, ds);
  });
}

extern "C" cuvsError_t cuvsMultiGpuIvfPqExtend(cuvsResources_t res, cuvsMultiGpuIvfPqIndex_t index,
                                               DLManagedTensor* new_vectors_tensor, DLManagedTensor* new_indices_tensor)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(new_vectors_tensor != nullptr, "null argument");
    const DLTensor& v = new_vectors_tensor->dl_tensor;
    CUVS_EXPECTS(is_host_compatible(v), "Multi-GPU IVF-PQ extend requires new_vectors to have host compatible memory");
    auto* ix = mg_index_of(index);
    CUVS_EXPECTS(v.dtype.code == index->dtype.code && v.dtype.bits == index->dtype.bits,
                 "type mismatch between index and new vectors");
    auto et    = elem_of_dtype(v.dtype, "new_vectors");
    void* data = checked_data(new_vectors_tensor, v.dtype.code, v.dtype.bits, 2, false, "new_vectors");
    const int64_t* ids = nullptr;
    if (new_indices_tensor) {
      ids = static_cast<const int64_t*>(checked_data(new_indices_tensor, kDLInt, 64, 1, false, "new_indices"));
      CUVS_EXPECTS(new_indices_tensor->dl_tensor.shape[0] == v.shape[0], "new_indices must have one entry per new vector");
    }
    CUVS_EXPECTS(!ix->parts.empty() && v.shape[1] == int64_t(ix->parts[0]->dim()),
                 "new vectors must have the dimension of the index");
    mg::extend(*clique_of(res), ix, data, et, v.shape[0], ids);
  });
}

extern "C" cuvsError_t cuvsMultiGpuIvfPqSerialize(cuvsResources_t res, cuvsMultiGpuIvfPqIndex_t index, const char* filename)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(filename != nullptr, "null argument");
    mg::serialize(*clique_of(res), *mg_index_of(index), std::string(filename), numpy_dtype_string(index->dtype));
  });
}

namespace {
// the element type recorded in the first four bytes of a multi-GPU index file
DLDataType dtype_of_mg_file(const char* filename)
{
  FILE* f = std::fopen(filename, "rb");
  CUVS_EXPECTS(f != nullptr, "Cannot open file %s", filename);
  char d[5] = {0, 0, 0, 0, 0};
  const size_t got = std::fread(d, 1, 4, f);
  std::fclose(f);
  CUVS_EXPECTS(got == 4, "Cannot read the header of %s", filename);
  const std::string s(d);
  if (s == "<f4") { return DLDataType{kDLFloat, 32, 1}; }
  if (s == "<f2") { return DLDataType{kDLFloat, 16, 1}; }
  if (s == "|i1") { return DLDataType{kDLInt, 8, 1}; }
  if (s == "|u1") { return DLDataType{kDLUInt, 8, 1}; }
  cuvs_b200::fail("Unsupported dtype string in the index file: %s", d);
}
}  // namespace

extern "C" cuvsError_t cuvsMultiGpuIvfPqDeserialize(cuvsResources_t res, const char* filename, cuvsMultiGpuIvfPqIndex_t index)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(filename != nullptr && index != nullptr, "null argument");
    const DLDataType dt = dtype_of_mg_file(filename);
    auto fresh = new mg::mg_index();
    try {
      mg::deserialize(*clique_of(res), std::string(filename), fresh);
    } catch (...) {
      delete fresh;
      throw;
    }
    install(index, fresh, dt);
  });
}

namespace {
// A single-GPU index file does not record the element type of the vectors it was built from (any of
// the four can be searched against it): the handle keeps the type it was given, fp32 when none.
void distribute_entry(cuvsResources_t res, const char* filename, cuvsMultiGpuIvfPqIndex_t index, bool by_list)
{
  CUVS_EXPECTS(filename != nullptr && index != nullptr, "null argument");
  auto fresh = new mg::mg_index();
  try {
    if (by_list) {
      mg::distribute_by_list(*clique_of(res), std::string(filename), fresh);
    } else {
      mg::distribute(*clique_of(res), std::string(filename), fresh);
    }
  } catch (...) {
    delete fresh;
    throw;
  }
  DLDataType dt = index->dtype.bits ? index->dtype : DLDataType{kDLFloat, 32, 1};
  install(index, fresh, dt);
}
}  // namespace

extern "C" cuvsError_t cuvsMultiGpuIvfPqDistribute(cuvsResources_t res, const char* filename, cuvsMultiGpuIvfPqIndex_t index)
{
  return translate_exceptions([=] { distribute_entry(res, filename, index, false); });
}
extern "C" cuvsError_t cuvsMultiGpuIvfPqDistributeByList(cuvsResources_t res, const char* filename,
                                                         cuvsMultiGpuIvfPqIndex_t index)
{
  return translate_exceptions([=] { distribute_entry(res, filename, index, true); });
}

// ------------------------------------------------------------------------------------------------
// one process per GPU
// ------------------------------------------------------------------------------------------------
extern "C" cuvsError_t cuvsMultiGpuCommIdCreate(cuvsMultiGpuCommId* id)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(id != nullptr, "null output pointer");
    mg::nccl_unique_id u;
    mg::make_unique_id(&u);
    static_assert(sizeof(u.bytes) == sizeof(id->bytes), "id size");
    std::memcpy(id->bytes, u.bytes, sizeof(u.bytes));
  });
}

extern "C" cuvsError_t cuvsMultiGpuRankCommCreate(cuvsResources_t res, const cuvsMultiGpuCommId* id, int rank, int n_ranks,
                                                  cuvsMultiGpuRankComm_t* comm)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(id != nullptr && comm != nullptr, "null argument");
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    CUVS_EXPECTS(dev == res_of(res)->device, "the device of the resources handle must be current");
    mg::nccl_unique_id u;
    std::memcpy(u.bytes, id->bytes, sizeof(u.bytes));
    *comm = reinterpret_cast<cuvsMultiGpuRankComm_t>(new mg::rank_comm(u, rank, n_ranks));
  });
}

extern "C" cuvsError_t cuvsMultiGpuRankCommAdopt(void* nccl_comm, int rank, int n_ranks, cuvsMultiGpuRankComm_t* comm)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(comm != nullptr, "null output pointer");
    *comm = reinterpret_cast<cuvsMultiGpuRankComm_t>(new mg::rank_comm(static_cast<ncclComm*>(nccl_comm), rank, n_ranks));
  });
}

extern "C" cuvsError_t cuvsMultiGpuRankCommDestroy(cuvsMultiGpuRankComm_t comm)
{
  return translate_exceptions([=] { delete reinterpret_cast<mg::rank_comm*>(comm); });
}

extern "C" cuvsError_t cuvsMultiGpuIvfPqSearchRank(cuvsResources_t res, cuvsMultiGpuRankComm_t comm,
                                                   cuvsIvfPqSearchParams_t params, cuvsIvfPqIndex_t shard,
                                                   DLManagedTensor* queries, DLManagedTensor* neighbors,
                                                   DLManagedTensor* distances)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(comm && params && queries && neighbors && distances, "null argument");
    auto* ix          = index_of(shard);
    const DLTensor& q = queries->dl_tensor;
    auto et           = elem_of_dtype(q.dtype, "queries");
    void* qd = checked_data(queries, q.dtype.code, q.dtype.bits, 2, true, "queries");
    auto* nb = static_cast<int64_t*>(checked_data(neighbors, kDLInt, 64, 2, true, "neighbors"));
    auto* ds = static_cast<float*>(checked_data(distances, kDLFloat, 32, 2, true, "distances"));
    CUVS_EXPECTS(q.shape[0] == neighbors->dl_tensor.shape[0] && q.shape[0] == distances->dl_tensor.shape[0],
                 "Number of rows in output neighbors and distances matrices must equal the number of queries.");
    CUVS_EXPECTS(neighbors->dl_tensor.shape[1] == distances->dl_tensor.shape[1],
                 "Number of columns in output neighbors and distances matrices must equal k");
    CUVS_EXPECTS(q.shape[1] == int64_t(ix->dim()),
                 "Number of query dimensions should equal number of dimensions in the index.");
    mg::search_rank(*res_of(res), *reinterpret_cast<mg::rank_comm*>(comm), convert_search(*params), *ix, qd, et,
                    uint32_t(q.shape[0]), uint32_t(neighbors->dl_tensor.shape[1]), nb, ds);
  });
}

extern "C" cuvsError_t cuvsMultiGpuRankCommStats(cuvsMultiGpuRankComm_t comm, double* stage_ms, uint64_t* batches, bool reset)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(comm && stage_ms && batches, "null argument");
    reinterpret_cast<mg::rank_comm*>(comm)->stats(stage_ms, batches, reset);
  });
}

extern "C" cuvsError_t cuvsMultiGpuRankCommSetMergeMode(cuvsMultiGpuRankComm_t comm, int mode)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(comm != nullptr, "null argument");
    CUVS_EXPECTS(mode >= 0 && mode <= 2, "mode must be 0, 1 or 2");
    reinterpret_cast<mg::rank_comm*>(comm)->set_merge_mode(mode);
  });
}

extern "C" cuvsError_t cuvsMultiGpuIvfPqListOwners(const uint32_t* list_sizes, uint32_t n_lists, int n_ranks, int32_t* owners)
{
  return translate_exceptions([=] {
    CUVS_EXPECTS(list_sizes != nullptr && owners != nullptr, "null argument");
    std::vector<uint32_t> sizes(list_sizes, list_sizes + n_lists);
    const std::vector<int> o = ivf_pq::list_owners(sizes, n_ranks);
    for (uint32_t l = 0; l < n_lists; l++) { owners[l] = o[l]; }
  });
}

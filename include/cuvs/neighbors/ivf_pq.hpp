// C++ interface of the IVF-PQ engine.
//
// Mirrors the public C++ API of the reference (cpp/include/cuvs/neighbors/ivf_pq.hpp): the same
// namespace, the same parameter structs with the same field names and defaults
// (index_params :47-151, search_params :160-213), an `index<int64_t>` with the same observers
// (:476-675), and free functions build / extend / search / serialize / deserialize.  The types the
// reference borrows from RAFT (resources, matrix views) are small local stand-ins with the same
// member names (`data_handle()`, `extent(i)`), so caller code compiles against either.
//
// Data layout in device memory (differs from the reference on purpose): instead of one allocation
// per inverted list plus pointer tables, all lists live back to back in two arenas --
//   codes : u8, list l starts at byte row_offset[l] * n_pieces * 16 and holds
//           ceil(size/32) groups of [n_pieces][32 lanes][16 bytes] (the reference's interleaved
//           layout inside a list, ivf_pq.hpp:235-296, so list payloads copy verbatim from files);
//   ids   : i64, list l starts at element row_offset[l]; slots past the list size hold -1.
// row_offset[l] is a multiple of 32.  A kernel finds a list with one load of an offset, and a
// list's bytes are contiguous and 512-byte aligned.
#pragma once

#include <cuvs/core/b200_common.hpp>

#include <cuda_fp16.h>
#include <library_types.h>  // cudaDataType_t

#include <cstdint>
#include <iosfwd>
#include <memory>
#include <string>
#include <vector>

// Everything declared here is exported from the shared library (which is otherwise built with hidden
// visibility): a C++ caller compiles against this header and links libcuvs_b200.so.
#pragma GCC visibility push(default)

namespace raft {
using resources = ::cuvs_b200::resources;

template <typename T, typename IdxT = int64_t>
struct device_matrix_view {
  T* ptr      = nullptr;
  IdxT rows   = 0;
  IdxT cols   = 0;
  T* data_handle() const { return ptr; }
  IdxT extent(int i) const { return i == 0 ? rows : cols; }
};
// host views are distinct types, so that host and device overloads can coexist as in the reference
template <typename T, typename IdxT = int64_t>
struct host_matrix_view {
  T* ptr    = nullptr;
  IdxT rows = 0;
  IdxT cols = 0;
  T* data_handle() const { return ptr; }
  IdxT extent(int i) const { return i == 0 ? rows : cols; }
};

template <typename T, typename IdxT = int64_t>
struct device_vector_view {
  T* ptr    = nullptr;
  IdxT size = 0;
  T* data_handle() const { return ptr; }
  IdxT extent(int) const { return size; }
};
template <typename T, typename IdxT = int64_t>
struct host_vector_view {
  T* ptr    = nullptr;
  IdxT size = 0;
  T* data_handle() const { return ptr; }
  IdxT extent(int) const { return size; }
};

template <typename T, typename IdxT = int64_t>
device_matrix_view<T, IdxT> make_device_matrix_view(T* p, IdxT r, IdxT c)
{
  return {p, r, c};
}
template <typename T, typename IdxT = int64_t>
host_matrix_view<T, IdxT> make_host_matrix_view(T* p, IdxT r, IdxT c)
{
  return {p, r, c};
}
template <typename T, typename IdxT = int64_t>
device_vector_view<T, IdxT> make_device_vector_view(T* p, IdxT n)
{
  return {p, n};
}
template <typename T, typename IdxT = int64_t>
host_vector_view<T, IdxT> make_host_vector_view(T* p, IdxT n)
{
  return {p, n};
}
}  // namespace raft

namespace cuvs::distance {
// cpp/include/cuvs/distance/distance.hpp:19-70 (values shared with the C enum)
enum class DistanceType : int {
  L2Expanded       = 0,
  L2SqrtExpanded   = 1,
  CosineExpanded   = 2,
  L1               = 3,
  L2Unexpanded     = 4,
  L2SqrtUnexpanded = 5,
  InnerProduct     = 6,
  Precomputed      = 100
};
}  // namespace cuvs::distance

namespace cuvs::neighbors::filtering {
// cpp/include/cuvs/neighbors/common.hpp:506-640, the part the IVF-PQ search takes
enum class FilterType { None, Bitmap, Bitset };
struct base_filter {
  virtual ~base_filter()                     = default;
  virtual FilterType get_filter_type() const = 0;
};
struct none_sample_filter : public base_filter {
  FilterType get_filter_type() const override { return FilterType::None; }
};
}  // namespace cuvs::neighbors::filtering

namespace cuvs::neighbors::ivf_pq {

using cuvs::distance::DistanceType;

enum class codebook_gen { PER_SUBSPACE = 0, PER_CLUSTER = 1 };
enum class list_layout { FLAT = 0, INTERLEAVED = 1 };

constexpr uint32_t kIndexGroupSize   = 32;  // ivf_pq.hpp:222
constexpr uint32_t kIndexGroupVecLen = 16;  // ivf_pq.hpp:224
constexpr int64_t kOutOfBoundsRecord = INT64_MAX;  // ivf_pq.hpp:231
constexpr int64_t kInvalidRecord     = -1;         // common.hpp:1634

struct index_params {
  DistanceType metric                  = DistanceType::L2Expanded;
  float metric_arg                     = 2.0f;
  bool add_data_on_build               = true;
  uint32_t n_lists                     = 1024;
  uint32_t kmeans_n_iters              = 20;
  double kmeans_trainset_fraction      = 0.5;
  uint32_t pq_bits                     = 8;
  uint32_t pq_dim                      = 0;
  codebook_gen codebook_kind           = codebook_gen::PER_SUBSPACE;
  list_layout codes_layout             = list_layout::INTERLEAVED;
  bool force_random_rotation           = false;
  bool conservative_memory_allocation  = false;
  uint32_t max_train_points_per_pq_code = 256;
};

struct search_params {
  uint32_t n_probes                      = 20;
  cudaDataType_t lut_dtype               = CUDA_R_32F;
  cudaDataType_t internal_distance_dtype = CUDA_R_32F;
  double preferred_shmem_carveout        = 1.0;
  cudaDataType_t coarse_search_dtype     = CUDA_R_32F;
  uint32_t max_internal_batch_size       = 4096;
};

// RAII device array.
template <typename T>
class dev_array {
 public:
  dev_array() = default;
  explicit dev_array(size_t n) { resize(n); }
  ~dev_array() { reset(); }
  dev_array(dev_array&& o) noexcept : p_(o.p_), n_(o.n_)
  {
    o.p_ = nullptr;
    o.n_ = 0;
  }
  dev_array& operator=(dev_array&& o) noexcept
  {
    if (this != &o) {
      reset();
      p_   = o.p_;
      n_   = o.n_;
      o.p_ = nullptr;
      o.n_ = 0;
    }
    return *this;
  }
  dev_array(const dev_array&)            = delete;
  dev_array& operator=(const dev_array&) = delete;
  void resize(size_t n)
  {
    reset();
    if (n) { CUDA_TRY(cudaMalloc(&p_, n * sizeof(T))); }
    n_ = n;
  }
  void reset()
  {
    if (p_) { cudaFree(p_); }
    p_ = nullptr;
    n_ = 0;
  }
  T* data() const { return p_; }
  size_t size() const { return n_; }

 private:
  T* p_     = nullptr;
  size_t n_ = 0;
};

template <typename IdxT>
class index;

// The index (ivf_pq.hpp:476-675).  Only IdxT = int64_t exists, as in the reference's instantiations.
template <>
class index<int64_t> {
 public:
  index() = default;
  index(DistanceType metric, codebook_gen kind, uint32_t n_lists, uint32_t dim, uint32_t pq_bits,
        uint32_t pq_dim, bool conservative_memory_allocation,
        list_layout codes_layout = list_layout::INTERLEAVED);

  // observers, same names as the reference
  DistanceType metric() const { return metric_; }
  codebook_gen codebook_kind() const { return codebook_kind_; }
  // INTERLEAVED (searchable) or FLAT: every vector's codes as one bit-packed row of
  // ceil(pq_dim * pq_bits / 8) bytes (list_spec_flat, ivf_pq.hpp:308-360; built, extended, stored and
  // unpacked, but not searched -- as in the reference)
  list_layout codes_layout() const { return layout_; }
  uint32_t bytes_per_vector() const { return cuvs_b200::ceildiv(pq_dim_ * pq_bits_, 8u); }
  // bytes one row of a list takes in the codes arena
  uint32_t list_row_bytes() const
  {
    return layout_ == list_layout::FLAT ? bytes_per_vector() : n_pieces() * kIndexGroupVecLen;
  }
  int64_t size() const { return size_; }
  uint32_t dim() const { return dim_; }
  uint32_t dim_ext() const { return cuvs_b200::round_up(dim_ + 1, 8u); }  // ivf_pq_index.cu:78-81
  uint32_t pq_bits() const { return pq_bits_; }
  uint32_t pq_dim() const { return pq_dim_; }
  uint32_t pq_len() const { return cuvs_b200::ceildiv(dim_, pq_dim_); }
  uint32_t rot_dim() const { return pq_len() * pq_dim_; }
  uint32_t pq_book_size() const { return 1u << pq_bits_; }
  uint32_t n_lists() const { return n_lists_; }
  bool conservative_memory_allocation() const { return conservative_; }
  uint32_t codes_per_piece() const { return 128u / pq_bits_; }
  uint32_t n_pieces() const { return cuvs_b200::ceildiv(pq_dim_, codes_per_piece()); }
  size_t pq_centers_size() const
  {
    return size_t(codebook_kind_ == codebook_gen::PER_SUBSPACE ? pq_dim_ : n_lists_) * pq_len() *
           pq_book_size();
  }
  static uint32_t calculate_pq_dim(uint32_t dim);  // ivf_pq_index.cu:611-622

  float* pq_centers() const { return pq_centers_.data(); }
  float* centers() const { return centers_.data(); }
  float* centers_rot() const { return centers_rot_.data(); }
  float* rotation_matrix() const { return rotation_.data(); }
  uint32_t* list_sizes() const { return list_sizes_.data(); }
  uint64_t* row_offsets() const { return row_off_.data(); }
  uint8_t* codes() const { return codes_.data(); }
  int64_t* ids() const { return ids_.data(); }
  const std::vector<uint32_t>& host_list_sizes() const { return h_list_sizes_; }
  const std::vector<uint64_t>& host_row_offsets() const { return h_row_off_; }
  // accum_sorted_sizes()[p] = total size of the p largest lists (ivf_common.cuh:255-290)
  const std::vector<int64_t>& accum_sorted_sizes() const { return accum_sorted_sizes_; }
  bool rotation_is_identity() const { return rotation_is_identity_; }
  // TF32 split of `centers` for the tensor-core coarse search, and the largest padded-row norm
  float* centers_hi() const { return centers_hi_.data(); }
  float* centers_lo() const { return centers_lo_.data(); }
  float centers_max_norm() const { return centers_max_norm_; }
  float centers_ext_scale() const { return centers_ext_scale_; }
  uint64_t total_rows_padded() const { return h_row_off_.empty() ? 0 : h_row_off_.back(); }
  // Operands of the int8 coarse search (coarse_search_dtype = CUDA_R_8I; centers_int8 and
  // rotation_matrix_int8 of cpp/src/neighbors/ivf_pq_index.cu:624-738), created on first use.  The
  // int8 values are held as fp32 numbers: every one is exact in TF32, so the tensor-core product
  // with fp32 accumulation gives the reference's int32 scores exactly.
  uint32_t dim_ext_int8() const { return cuvs_b200::round_up(dim_ + 2, 16u); }  // ivf_pq_index.cu:667
  struct int8_operands {
    const float* centers;   // [n_lists, dim_ext_int8]
    const float* rotation;  // [rot_dim, dim]
    float centers_max_norm;
  };
  int8_operands int8_coarse_operands(cudaStream_t stream) const;
  // Operands of the fp16 coarse search (coarse_search_dtype = CUDA_R_16F; the lazily cast centers of
  // cpp/src/neighbors/ivf_pq_index.cu:599-622), created on first use: the padded centers and the
  // rotation matrix rounded to half precision, held as fp32 numbers.
  struct half_operands {
    const float* centers;   // [n_lists, dim_ext]
    const float* rotation;  // [rot_dim, dim]
  };
  half_operands half_coarse_operands(cudaStream_t stream) const;

  // (Re)create the arenas for the given list sizes; contents are zero codes / -1 ids.
  void allocate_lists(const std::vector<uint32_t>& sizes, cudaStream_t stream);
  // Recompute host-side derived state after the model arrays or list sizes changed.
  void recompute_internal_state(cudaStream_t stream);

  // model arrays are public to the builder / loader
  dev_array<float> pq_centers_, centers_, centers_rot_, rotation_;
  dev_array<float> centers_hi_, centers_lo_;
  float centers_max_norm_ = 0.0f;
  float centers_ext_scale_ = 1.0f;
  mutable dev_array<float> centers_i8f_, rotation_i8f_;
  mutable dev_array<float> centers_h_, rotation_h_;
  mutable float centers_i8f_max_norm_ = 0.0f;
  dev_array<uint32_t> list_sizes_;
  dev_array<uint64_t> row_off_;
  dev_array<uint8_t> codes_;
  dev_array<int64_t> ids_;
  std::vector<uint32_t> h_list_sizes_;
  std::vector<uint64_t> h_row_off_;
  std::vector<int64_t> accum_sorted_sizes_;
  int64_t size_ = 0;

 private:
  DistanceType metric_        = DistanceType::L2Expanded;
  codebook_gen codebook_kind_ = codebook_gen::PER_SUBSPACE;
  uint32_t n_lists_ = 0, dim_ = 0, pq_bits_ = 8, pq_dim_ = 0;
  bool conservative_          = false;
  bool rotation_is_identity_  = false;
  list_layout layout_         = list_layout::INTERLEAVED;
};

// ---- free functions (ivf_pq.hpp:702-2111) -----------------------------------------------------

// Element types of datasets and queries (the reference instantiates float, half, int8_t, uint8_t).
enum class elem_t { f32 = 0, f16 = 1, i8 = 2, u8 = 3 };
inline size_t elem_size(elem_t t) { return t == elem_t::f32 ? 4 : (t == elem_t::f16 ? 2 : 1); }

// Type-erased workers behind the typed overloads below.
// `given_probes` (optional, device, [n_queries, min(n_probes, n_lists)] u32): lists to scan per
// query, replacing the coarse stage (used when probe selection is shared between GPUs).
// Bitset sample filter of the reference (cuvs::neighbors::filtering::bitset_filter<uint32_t, int64_t>,
// cpp/src/neighbors/sample_filter.cuh:162-176): vector with source id i is searched iff bit i is set.
struct bitset_view {
  const uint32_t* bits = nullptr;  // device
  uint64_t n_bits      = 0;
};
void search_any(raft::resources& res, const search_params& params, const index<int64_t>& idx,
                const void* queries, elem_t qtype, uint32_t n_queries, uint32_t k,
                int64_t* neighbors, float* distances, const uint32_t* given_probes = nullptr,
                bitset_view filter = {});
}  // namespace cuvs::neighbors::ivf_pq
namespace cuvs::neighbors::filtering {
// bitset_filter<bitset_t, index_t> (common.hpp:585-611): a view of device words, bit i = source id i
template <typename bitset_t, typename index_t>
struct bitset_filter : public base_filter {
  static_assert(sizeof(bitset_t) == 4 && sizeof(index_t) == 8, "uint32_t words and int64_t ids");
  bitset_filter(const bitset_t* device_words, uint64_t n_bits) : words_(device_words), n_bits_(n_bits) {}
  FilterType get_filter_type() const override { return FilterType::Bitset; }
  ivf_pq::bitset_view view() const { return {words_, n_bits_}; }

 private:
  const bitset_t* words_;
  uint64_t n_bits_;
};
}  // namespace cuvs::neighbors::filtering
namespace cuvs::neighbors::ivf_pq {
// Every check the search makes on its parameters before it touches the GPU (argument ranges, dtype
// pairing, a shared-memory plan for the look-up table): throws what the search would throw.
// `shard`: the index is one rank's part of a list-sharded index, which may hold fewer than k rows.
void check_search_params(const raft::resources& res, const search_params& params, const index<int64_t>& idx,
                         uint32_t k, bool shard = false);
// Probe selection alone, asynchronous on the handle's stream: probes [n_queries, n_probes] u32,
// ascending by (score, list id).
void select_probes_any(raft::resources& res, const index<int64_t>& idx, const void* queries,
                       elem_t qtype, uint32_t n_queries, uint32_t n_probes, uint32_t* probes,
                       cudaDataType_t coarse_search_dtype = CUDA_R_32F);
void build_any(raft::resources& res, const index_params& params, const void* dataset,
               elem_t dtype, int64_t n_rows, uint32_t dim, bool on_device, index<int64_t>* idx);
void extend_any(raft::resources& res, const void* new_vectors, elem_t dtype, int64_t n_rows,
                const int64_t* new_indices, bool on_device, index<int64_t>* idx);
void transform_any(raft::resources& res, const index<int64_t>& idx, const void* dataset,
                   elem_t dtype, int64_t n_rows, uint32_t* out_labels, uint8_t* out_codes);

template <typename T>
constexpr elem_t elem_of();
template <> constexpr elem_t elem_of<float>() { return elem_t::f32; }
template <> constexpr elem_t elem_of<half>() { return elem_t::f16; }
template <> constexpr elem_t elem_of<int8_t>() { return elem_t::i8; }
template <> constexpr elem_t elem_of<uint8_t>() { return elem_t::u8; }

// ivf_pq.hpp:1821-1962
template <typename T>
void search(raft::resources& res, const search_params& params, const index<int64_t>& idx,
            raft::device_matrix_view<const T, int64_t> queries,
            raft::device_matrix_view<int64_t, int64_t> neighbors,
            raft::device_matrix_view<float, int64_t> distances)
{
  CUVS_EXPECTS(queries.extent(0) == neighbors.extent(0) && queries.extent(0) == distances.extent(0),
               "Number of rows in output neighbors and distances matrices must equal the number of "
               "queries.");
  CUVS_EXPECTS(neighbors.extent(1) == distances.extent(1),
               "Number of columns in output neighbors and distances matrices must equal k");
  CUVS_EXPECTS(queries.extent(1) == idx.dim(),
               "Number of query dimensions should equal number of dimensions in the index.");
  search_any(res, params, idx, queries.data_handle(), elem_of<T>(),
             static_cast<uint32_t>(queries.extent(0)), static_cast<uint32_t>(neighbors.extent(1)),
             neighbors.data_handle(), distances.data_handle());
}

// ivf_pq.hpp:1821-1962, the overload with a sample filter: `none_sample_filter` or
// `bitset_filter<uint32_t, int64_t>` (cpp/include/cuvs/neighbors/common.hpp:506-640): the vector with
// source id i may be returned only if bit i of the bitset is set.
template <typename T>
void search(raft::resources& res, const search_params& params, const index<int64_t>& idx,
            raft::device_matrix_view<const T, int64_t> queries,
            raft::device_matrix_view<int64_t, int64_t> neighbors,
            raft::device_matrix_view<float, int64_t> distances, const filtering::base_filter& sample_filter)
{
  CUVS_EXPECTS(queries.extent(0) == neighbors.extent(0) && queries.extent(0) == distances.extent(0),
               "Number of rows in output neighbors and distances matrices must equal the number of "
               "queries.");
  CUVS_EXPECTS(neighbors.extent(1) == distances.extent(1),
               "Number of columns in output neighbors and distances matrices must equal k");
  CUVS_EXPECTS(queries.extent(1) == idx.dim(),
               "Number of query dimensions should equal number of dimensions in the index.");
  bitset_view view{};
  if (sample_filter.get_filter_type() == filtering::FilterType::Bitset) {
    view = static_cast<const filtering::bitset_filter<uint32_t, int64_t>&>(sample_filter).view();
  } else {
    CUVS_EXPECTS(sample_filter.get_filter_type() == filtering::FilterType::None, "Unsupported sample filter type");
  }
  search_any(res, params, idx, queries.data_handle(), elem_of<T>(),
             static_cast<uint32_t>(queries.extent(0)), static_cast<uint32_t>(neighbors.extent(1)),
             neighbors.data_handle(), distances.data_handle(), nullptr, view);
}

// ivf_pq.hpp:702-1262: build from a device or a host dataset, returning the index or filling one
template <typename T>
index<int64_t> build(raft::resources& res, const index_params& params,
                     raft::device_matrix_view<const T, int64_t> dataset)
{
  index<int64_t> idx;
  build_any(res, params, dataset.data_handle(), elem_of<T>(), dataset.extent(0),
            static_cast<uint32_t>(dataset.extent(1)), true, &idx);
  return idx;
}
template <typename T>
void build(raft::resources& res, const index_params& params, raft::device_matrix_view<const T, int64_t> dataset,
           index<int64_t>* idx)
{
  build_any(res, params, dataset.data_handle(), elem_of<T>(), dataset.extent(0),
            static_cast<uint32_t>(dataset.extent(1)), true, idx);
}
template <typename T>
index<int64_t> build(raft::resources& res, const index_params& params,
                     raft::host_matrix_view<const T, int64_t> dataset)
{
  index<int64_t> idx;
  build_any(res, params, dataset.data_handle(), elem_of<T>(), dataset.extent(0),
            static_cast<uint32_t>(dataset.extent(1)), false, &idx);
  return idx;
}
template <typename T>
void build(raft::resources& res, const index_params& params, raft::host_matrix_view<const T, int64_t> dataset,
           index<int64_t>* idx)
{
  build_any(res, params, dataset.data_handle(), elem_of<T>(), dataset.extent(0),
            static_cast<uint32_t>(dataset.extent(1)), false, idx);
}

// ivf_pq.hpp:1296-1780: extend in place (device or host vectors; new_indices may be null: ids continue
// from the current size)
template <typename T>
void extend(raft::resources& res, raft::device_matrix_view<const T, int64_t> new_vectors,
            const int64_t* new_indices, index<int64_t>* idx)
{
  extend_any(res, new_vectors.data_handle(), elem_of<T>(), new_vectors.extent(0), new_indices, true,
             idx);
}
template <typename T>
void extend(raft::resources& res, raft::host_matrix_view<const T, int64_t> new_vectors,
            const int64_t* new_indices, index<int64_t>* idx)
{
  extend_any(res, new_vectors.data_handle(), elem_of<T>(), new_vectors.extent(0), new_indices, false,
             idx);
}

// ivf_pq.hpp:2034-2111 (format: cpp/src/neighbors/ivf_pq/ivf_pq_serialize.cuh, version 4)
void serialize(raft::resources& res, std::ostream& os, const index<int64_t>& idx);
void serialize(raft::resources& res, const std::string& filename, const index<int64_t>& idx);
// owned(list) == false skips the payload of that list (its size becomes 0): list-sharded loading.
void deserialize(raft::resources& res, std::istream& is, index<int64_t>* idx, int shard_rank = 0,
                 int shard_count = 1);
void deserialize(raft::resources& res, const std::string& filename, index<int64_t>* idx,
                 int shard_rank = 0, int shard_count = 1);

// Multi-GPU index files of the reference (cpp/src/neighbors/mg/snmg.cuh:60-91, 780-805): dtype string,
// distribution mode (0 = REPLICATED, 1 = SHARDED by rows), number of ranks, one index stream per rank.
// One process per GPU reads its own rank's index; `id_offset` = rows held by the ranks before it
// (what the reference adds to a shard's local ids when it merges, snmg.cuh:351-355), 0 when replicated.
void deserialize_mg_rank(raft::resources& res, const std::string& filename, int rank, int n_ranks,
                         index<int64_t>* idx, int* mode, int64_t* id_offset);
void serialize_mg(raft::resources& res, const std::string& filename, int mode, const char* dtype_string,
                  const std::vector<const index<int64_t>*>& per_rank);
// the head of such a file: four bytes of dtype string, mode and number of ranks as scalar records
void serialize_mg_header(std::ostream& os, const char* dtype_string, int mode, int n_ranks);

// Which rank of a list-sharded deployment holds each list: lists are dealt in order of descending
// size (ties by list id), each to the rank holding the fewest rows so far (ties to the lowest rank),
// so that the ranks hold about the same number of rows however skewed the list sizes are.  A pure
// function of the sizes: every rank computes the same map from the header of the index file.
std::vector<int> list_owners(const std::vector<uint32_t>& list_sizes, int shard_count);
// One index stream (format version 4) out of the shards of a list-sharded index: model arrays from
// shard 0, every list from the shard that holds it.  res[r] / shards[r] live on rank r's device.
void serialize_list_sharded(const std::vector<raft::resources*>& res, std::ostream& os,
                            const std::vector<const index<int64_t>*>& shards);

namespace helpers {
// Bit-packed codes u8 [n_rows, ceil(pq_dim*pq_bits/8)] of rows [offset, offset+n_rows) of one list
// (codepacker::unpack_contiguous_list_data, cpp/src/neighbors/ivf_pq/ivf_pq_contiguous_list_data_impl.cuh).
void unpack_contiguous_list_data(raft::resources& res, const index<int64_t>& idx, uint8_t* out_codes,
                                 uint32_t n_rows, uint32_t label, uint32_t offset);
// Install precomputed model arrays (device pointers) into an empty index
// (build from precomputed centers, cpp/src/neighbors/ivf_pq/ivf_pq_build.cuh:1560-1700).
// `centers` is [n_lists, centers_cols] with centers_cols == dim (norms are computed) or dim_ext.
void set_model(raft::resources& res, index<int64_t>* idx, const float* pq_centers, const float* centers,
               uint32_t centers_cols, const float* centers_rot, const float* rotation_matrix);

// Single-list helpers of the reference (ivf_pq.hpp:2564-3128, cpp/src/neighbors/ivf_pq/
// ivf_pq_build_common.cu:30-225).  All pointers are device pointers; all calls are asynchronous on
// the handle's stream unless they change a list's size.  `in_cluster_indices`, where given, selects
// rows by their position in the list instead of the range [offset, offset + n_rows).
namespace codepacker {
using helpers::unpack_contiguous_list_data;
// Codes of list rows, one code per byte: out_codes u8 [n_rows, pq_dim].
void unpack_list_data(raft::resources& res, const index<int64_t>& idx, uint8_t* out_codes,
                      uint32_t n_rows, uint32_t label, uint32_t offset,
                      const uint32_t* in_cluster_indices = nullptr);
// Overwrite list rows [offset, offset + n_rows) with codes given one per byte, u8 [n_rows, pq_dim].
// No allocation: the rows must exist.
void pack_list_data(raft::resources& res, index<int64_t>* idx, const uint8_t* codes, uint32_t n_rows,
                    uint32_t label, uint32_t offset);
// Same with bit-packed rows, u8 [n_rows, ceil(pq_dim * pq_bits / 8)].
void pack_contiguous_list_data(raft::resources& res, index<int64_t>* idx, const uint8_t* codes,
                               uint32_t n_rows, uint32_t label, uint32_t offset);
// Decode list rows back to the input space: out [n_rows, dim] of type `out_type`
//   out[i, :] = mapping<T>( rotation^T * (pq_center(code(i, j)) + center_rot[label, j]) ).
void reconstruct_list_data(raft::resources& res, const index<int64_t>& idx, void* out_vectors,
                           elem_t out_type, uint32_t n_rows, uint32_t label, uint32_t offset,
                           const uint32_t* in_cluster_indices = nullptr);
// Append rows to one list, skipping the classification (and, with codes, the encoding):
// new_codes u8 [n_rows, pq_dim] / [n_rows, ceil(pq_dim * pq_bits / 8)], new_indices i64 [n_rows].
void extend_list_with_codes(raft::resources& res, index<int64_t>* idx, const uint8_t* new_codes,
                            const int64_t* new_indices, uint32_t n_rows, uint32_t label);
void extend_list_with_contiguous_codes(raft::resources& res, index<int64_t>* idx,
                                       const uint8_t* new_codes, const int64_t* new_indices,
                                       uint32_t n_rows, uint32_t label);
void extend_list(raft::resources& res, index<int64_t>* idx, const void* new_vectors, elem_t dtype,
                 const int64_t* new_indices, uint32_t n_rows, uint32_t label);
}  // namespace codepacker
// Remove all rows of one list / of every list (ivf_pq.hpp:3144, :3166).
void erase_list(raft::resources& res, index<int64_t>* idx, uint32_t label);
void reset_index(raft::resources& res, index<int64_t>* idx);
}  // namespace helpers

namespace detail {
// Merge `n_parts` per-part top-k lists into one (cpp/src/neighbors/detail/knn_merge_parts.cuh:24-170).
// in_* : [n_parts, n_queries, k]; out_*: [n_queries, k]; select_min picks the smallest distances.
// part_stride_*: elements between consecutive parts (0 = n_queries * k, parts back to back).
void knn_merge_parts(raft::resources& res, const float* in_dist, const int64_t* in_ids,
                     float* out_dist, int64_t* out_ids, uint32_t n_parts, uint32_t n_queries,
                     uint32_t k, bool select_min, size_t part_stride_dist = 0, size_t part_stride_ids = 0);
}  // namespace detail

}  // namespace cuvs::neighbors::ivf_pq

#pragma GCC visibility pop

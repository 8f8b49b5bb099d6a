// Helpers shared by the translation units that implement the C interface: exception translation
// (c/src/core/exceptions.hpp:17-33 of the reference), DLPack tensor validation the way the
// reference's from_dlpack does it (c/src/core/detail/interop.hpp:75-139), handle casts.
#pragma once

#include "../../include/cuvs_ivf_pq.h"

#include "ivf_pq.hpp"

#include <algorithm>
#include <exception>
#include <initializer_list>
#include <string>

namespace cuvs_b200::capi {

namespace ivf_pq = cuvs::neighbors::ivf_pq;
using cuvs_b200::fail;
using index_t = ivf_pq::index<int64_t>;

template <typename Fn>
cuvsError_t translate_exceptions(Fn&& fn)
{
  try {
    fn();
    cuvsSetLastErrorText(nullptr);
    return CUVS_SUCCESS;
  } catch (const std::exception& e) {
    cuvsSetLastErrorText(e.what());
  } catch (...) {
    cuvsSetLastErrorText("unknown exception");
  }
  return CUVS_ERROR;
}

inline bool is_device_compatible(const DLTensor& t)
{
  return t.device.device_type == kDLCUDA || t.device.device_type == kDLCUDAHost ||
         t.device.device_type == kDLCUDAManaged;
}
inline bool is_host_compatible(const DLTensor& t)
{
  return t.device.device_type == kDLCPU || t.device.device_type == kDLCUDAHost ||
         t.device.device_type == kDLCUDAManaged;
}
inline bool is_c_contiguous(const DLTensor& t)
{
  if (!t.strides) { return true; }
  int64_t expected = 1;
  for (int64_t i = t.ndim - 1; i >= 0; --i) {
    if (t.strides[i] != expected) { return false; }
    expected *= t.shape[i];
  }
  return true;
}

// from_dlpack for a row-major tensor of known dtype / rank; returns the data pointer.
inline void* checked_data(DLManagedTensor* mt, uint8_t code, uint8_t bits, int ndim, bool device,
                   const char* name)
{
  CUVS_EXPECTS(mt != nullptr, "%s: null tensor", name);
  const DLTensor& t = mt->dl_tensor;
  CUVS_EXPECTS(is_c_contiguous(t), "Expected a row-major matrix");
  CUVS_EXPECTS(code == t.dtype.code, "code mismatch between return mdspan (%i) and DLTensor (%i)",
               int(code), int(t.dtype.code));
  CUVS_EXPECTS(bits == t.dtype.bits, "bits mismatch between return mdspan (%i) and DLTensor (%i)",
               int(bits), int(t.dtype.bits));
  CUVS_EXPECTS(t.dtype.lanes == 1, "More than 1 DLTensor lanes not supported");
  if (device) {
    CUVS_EXPECTS(is_device_compatible(t), "device_type mismatch between return mdspan and DLTensor");
  } else {
    CUVS_EXPECTS(is_host_compatible(t), "device_type mismatch between return mdspan and DLTensor");
  }
  CUVS_EXPECTS(t.ndim == ndim, "ndim mismatch between return mdspan and DLTensor");
  return static_cast<char*>(t.data) + t.byte_offset;
}

// [n_parts, n, k] device tensor whose parts are row-major and may be separated by any stride
// (in elements, at least n * k); returns the data pointer and the stride between parts.
inline void* checked_parts(DLManagedTensor* mt, uint8_t code, uint8_t bits, const char* name, size_t* part_stride)
{
  CUVS_EXPECTS(mt != nullptr, "%s: null tensor", name);
  const DLTensor& t = mt->dl_tensor;
  CUVS_EXPECTS(t.ndim == 3, "ndim mismatch between return mdspan and DLTensor");
  CUVS_EXPECTS(code == t.dtype.code && bits == t.dtype.bits && t.dtype.lanes == 1,
               "%s: unexpected element type", name);
  CUVS_EXPECTS(is_device_compatible(t), "device_type mismatch between return mdspan and DLTensor");
  *part_stride = size_t(t.shape[1]) * size_t(t.shape[2]);
  if (t.strides) {
    CUVS_EXPECTS(t.strides[2] == 1 && t.strides[1] == t.shape[2] &&
                   (t.shape[0] <= 1 || t.strides[0] >= t.shape[1] * t.shape[2]),
                 "Expected row-major parts");
    if (t.shape[0] > 1) { *part_stride = size_t(t.strides[0]); }
  }
  return static_cast<char*>(t.data) + t.byte_offset;
}

inline ivf_pq::elem_t elem_of_dtype(const DLDataType& d, const char* what)
{
  if (d.code == kDLFloat && d.bits == 32) { return ivf_pq::elem_t::f32; }
  if (d.code == kDLFloat && d.bits == 16) { return ivf_pq::elem_t::f16; }
  if (d.code == kDLInt && d.bits == 8) { return ivf_pq::elem_t::i8; }
  if (d.code == kDLUInt && d.bits == 8) { return ivf_pq::elem_t::u8; }
  fail("Unsupported %s DLtensor dtype: %d and bits: %d", what, int(d.code), int(d.bits));
}

inline index_t* index_of(cuvsIvfPqIndex_t index)
{
  CUVS_EXPECTS(index != nullptr && index->addr != 0, "the index handle holds no index");
  return reinterpret_cast<index_t*>(index->addr);
}
inline cuvs_b200::resources* res_of(cuvsResources_t res)
{
  CUVS_EXPECTS(res != 0, "null resources handle");
  return reinterpret_cast<cuvs_b200::resources*>(res);
}

inline void tensor_deleter(DLManagedTensor* self)
{
  delete[] self->dl_tensor.shape;
  delete[] self->dl_tensor.strides;
  self->dl_tensor.shape   = nullptr;
  self->dl_tensor.strides = nullptr;
}

// to_dlpack for a non-owning device view (c/src/core/detail/interop.hpp:143-174)
inline void make_view(DLManagedTensor* out, void* data, DLDataType dtype, std::initializer_list<int64_t> shape,
               std::initializer_list<int64_t> strides = {})
{
  CUVS_EXPECTS(out != nullptr, "null output tensor");
  int device = 0;
  cudaGetDevice(&device);
  DLTensor& t   = out->dl_tensor;
  t.data        = data;
  t.device      = DLDevice{kDLCUDA, device};
  t.ndim        = int32_t(shape.size());
  t.dtype       = dtype;
  t.shape       = new int64_t[shape.size()];
  std::copy(shape.begin(), shape.end(), t.shape);
  t.strides = nullptr;
  if (strides.size()) {
    t.strides = new int64_t[strides.size()];
    std::copy(strides.begin(), strides.end(), t.strides);
  }
  t.byte_offset    = 0;
  out->manager_ctx = nullptr;
  out->deleter     = tensor_deleter;
}

inline ivf_pq::index_params convert(const cuvsIvfPqIndexParams& p)
{
  ivf_pq::index_params o;
  o.metric                         = ivf_pq::DistanceType(int(p.metric));
  o.metric_arg                     = p.metric_arg;
  o.add_data_on_build              = p.add_data_on_build;
  o.n_lists                        = p.n_lists;
  o.kmeans_n_iters                 = p.kmeans_n_iters;
  o.kmeans_trainset_fraction       = p.kmeans_trainset_fraction;
  o.pq_bits                        = p.pq_bits;
  o.pq_dim                         = p.pq_dim;
  o.codebook_kind                  = ivf_pq::codebook_gen(int(p.codebook_kind));
  o.force_random_rotation          = p.force_random_rotation;
  o.conservative_memory_allocation = p.conservative_memory_allocation;
  o.max_train_points_per_pq_code   = p.max_train_points_per_pq_code;
  o.codes_layout                   = ivf_pq::list_layout(int(p.codes_layout));
  return o;
}


}  // namespace cuvs_b200::capi

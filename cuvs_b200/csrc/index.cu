// Index object, arena management and the version-4 file format.
//
// File format (cpp/src/neighbors/ivf_pq/ivf_pq_serialize.cuh:41-87 writer, :124-211 reader;
// per-list records cpp/src/neighbors/ivf_list.cuh:108-176): a sequence of NumPy .npy v1.0 records.
// Scalars are 0-d arrays:  int32 version(=4), int64 n_rows, uint32 dim, uint32 pq_bits,
// uint32 pq_dim, bool conservative_memory_allocation, int32 metric, int32 codebook_kind,
// int32 codes_layout, uint32 n_lists;  then arrays pq_centers, centers, centers_rot,
// rotation_matrix (f32) and list_sizes (u32);  then per list: uint32 size and, when size > 0,
// codes u8 [ceil(size/32), n_pieces, 32, 16] and ids i64 [size].
// The reader accepts any well-formed v1.0/2.0 header and checks element size and element count
// of every record against what the format calls for.
#include "ivf_pq.hpp"
#include "search_internal.hpp"

#include <algorithm>
#include <cstring>
#include <fstream>
#include <queue>
#include <mutex>
#include <cmath>
#include <numeric>

namespace cuvs::neighbors::ivf_pq {

using cuvs_b200::ceildiv;
using cuvs_b200::round_up;

index<int64_t>::index(DistanceType metric, codebook_gen kind, uint32_t n_lists, uint32_t dim,
                      uint32_t pq_bits, uint32_t pq_dim, bool conservative, list_layout codes_layout)
  : metric_(metric),
    codebook_kind_(kind),
    n_lists_(n_lists),
    dim_(dim),
    pq_bits_(pq_bits),
    pq_dim_(pq_dim == 0 ? calculate_pq_dim(dim) : pq_dim),
    conservative_(conservative),
    layout_(codes_layout)
{
  // ivf_pq_index.cu:599-609
  CUVS_EXPECTS(pq_bits_ >= 4 && pq_bits_ <= 8,
               "`pq_bits` must be within closed range [4,8], but got %u.", pq_bits_);
  CUVS_EXPECTS((pq_bits_ * pq_dim_) % 8 == 0,
               "`pq_bits * pq_dim` must be a multiple of 8, but got %u * %u = %u.", pq_bits_,
               pq_dim_, pq_bits_ * pq_dim_);
  CUVS_EXPECTS(n_lists_ > 0 && dim_ > 0, "n_lists and dim must be positive");
  CUVS_EXPECTS(metric == DistanceType::L2Expanded || metric == DistanceType::L2SqrtExpanded ||
                 metric == DistanceType::InnerProduct || metric == DistanceType::CosineExpanded,
               "Unsupported distance type %d.", int(metric));
  pq_centers_.resize(pq_centers_size());
  centers_.resize(size_t(n_lists_) * dim_ext());
  centers_rot_.resize(size_t(n_lists_) * rot_dim());
  rotation_.resize(size_t(rot_dim()) * dim_);
  list_sizes_.resize(n_lists_);
  row_off_.resize(size_t(n_lists_) + 1);
  CUDA_TRY(cudaMemset(list_sizes_.data(), 0, size_t(n_lists_) * 4));
  CUDA_TRY(cudaMemset(row_off_.data(), 0, (size_t(n_lists_) + 1) * 8));
  h_list_sizes_.assign(n_lists_, 0);
  h_row_off_.assign(size_t(n_lists_) + 1, 0);
  accum_sorted_sizes_.assign(size_t(n_lists_) + 1, 0);
}

uint32_t index<int64_t>::calculate_pq_dim(uint32_t dim)
{
  if (dim >= 128) { dim /= 2; }
  uint32_t r = dim / 32 * 32;
  if (r > 0) { return r; }
  r = 1;
  while ((r << 1) <= dim) { r <<= 1; }
  return r;
}

__global__ void fill_i64_kernel(int64_t* p, size_t n, int64_t v)
{
  size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (i < n) { p[i] = v; }
}

// int8 image of the padded centers (ivf_pq_index.cu:661-738): components scaled by 128 and clamped;
// the squared norm x of column `dim` is spread over the m - 1 spare columns as y = round(x * 64 /
// (m - 1)) each, the rounding remainder z = (y - round(y)) * 128 goes to column `dim`.
__global__ void centers_to_int8_kernel(const float* __restrict__ centers, size_t n, uint32_t dim,
                                       uint32_t dim_ext, uint32_t dim_ext8, float* __restrict__ out)
{
  const size_t ix = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (ix >= n) { return; }
  const uint32_t col = uint32_t(ix % dim_ext8);
  const size_t row   = ix / dim_ext8;
  int8_t v;
  if (col < dim) {
    v = static_cast<int8_t>(fmaxf(-128.0f, fminf(127.0f, __fmul_rn(centers[row * dim_ext + col], 128.0f))));
  } else {
    const float x = centers[row * dim_ext + dim];
    const float c = __fdiv_rn(64.0f, static_cast<float>(dim_ext8 - dim - 1));
    const float y = fmaxf(-128.0f, fminf(127.0f, __fmul_rn(x, c)));
    const float z = fmaxf(-128.0f, fminf(127.0f, __fmul_rn(__fsub_rn(y, roundf(y)), 128.0f)));
    v             = col > dim ? static_cast<int8_t>(roundf(y)) : static_cast<int8_t>(z);
  }
  out[ix] = static_cast<float>(v);
}

// mapping<int8_t> of the rotation matrix (ivf_pq_index.cu:624-658; ann_utils.cuh:211-217).
__global__ void rotation_to_int8_kernel(const float* __restrict__ rot, size_t n, float* __restrict__ out)
{
  const size_t ix = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  // the float -> int8 mapping clamps before it converts (ann_utils.cuh:211-217): 1.0 becomes 127
  if (ix < n) {
    out[ix] = static_cast<float>(static_cast<int8_t>(fminf(fmaxf(__fmul_rn(rot[ix], 128.0f), -128.0f), 127.0f)));
  }
}

index<int64_t>::int8_operands index<int64_t>::int8_coarse_operands(cudaStream_t stream) const
{
  static std::mutex lock;  // first use may come from several searching threads at once
  std::lock_guard<std::mutex> guard(lock);
  const uint32_t d8 = dim_ext_int8();
  const size_t nc = size_t(n_lists_) * d8, nr = size_t(rot_dim()) * dim_;
  if (centers_i8f_.size() != nc || rotation_i8f_.size() != nr) {
    centers_i8f_.resize(nc);
    rotation_i8f_.resize(nr);
    centers_to_int8_kernel<<<unsigned(ceildiv<size_t>(nc, 256)), 256, 0, stream>>>(
      centers_.data(), nc, dim_, dim_ext(), d8, centers_i8f_.data());
    rotation_to_int8_kernel<<<unsigned(ceildiv<size_t>(nr, 256)), 256, 0, stream>>>(rotation_.data(), nr,
                                                                                     rotation_i8f_.data());
    CUDA_TRY(cudaGetLastError());
    std::vector<float> hc(nc);
    CUDA_TRY(cudaMemcpyAsync(hc.data(), centers_i8f_.data(), nc * 4, cudaMemcpyDeviceToHost, stream));
    CUDA_TRY(cudaStreamSynchronize(stream));  // other streams may use the arrays right after this call
    double mx = 0.0;
    for (uint32_t l = 0; l < n_lists_; l++) {
      double ss = 0.0;
      for (uint32_t k = 0; k < d8; k++) {
        const double v = hc[size_t(l) * d8 + k];
        ss += v * v;
      }
      mx = std::max(mx, ss);
    }
    centers_i8f_max_norm_ = float(std::sqrt(mx)) * 1.0001f;
  }
  return {centers_i8f_.data(), rotation_i8f_.data(), centers_i8f_max_norm_};
}

__global__ void round_to_half_kernel(const float* __restrict__ in, size_t n, float* __restrict__ out)
{
  const size_t ix = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (ix < n) { out[ix] = __half2float(__float2half_rn(in[ix])); }
}

index<int64_t>::half_operands index<int64_t>::half_coarse_operands(cudaStream_t stream) const
{
  static std::mutex lock;  // first use may come from several searching threads at once
  std::lock_guard<std::mutex> guard(lock);
  const size_t nc = size_t(n_lists_) * dim_ext(), nr = size_t(rot_dim()) * dim_;
  if (centers_h_.size() != nc || rotation_h_.size() != nr) {
    centers_h_.resize(nc);
    rotation_h_.resize(nr);
    round_to_half_kernel<<<unsigned(ceildiv<size_t>(nc, 256)), 256, 0, stream>>>(centers_.data(), nc, centers_h_.data());
    round_to_half_kernel<<<unsigned(ceildiv<size_t>(nr, 256)), 256, 0, stream>>>(rotation_.data(), nr, rotation_h_.data());
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaStreamSynchronize(stream));  // other streams may use the arrays right after this call
  }
  return {centers_h_.data(), rotation_h_.data()};
}

void index<int64_t>::allocate_lists(const std::vector<uint32_t>& sizes, cudaStream_t stream)
{
  CUVS_EXPECTS(sizes.size() == n_lists_, "list size vector has the wrong length");
  h_list_sizes_ = sizes;
  h_row_off_.assign(size_t(n_lists_) + 1, 0);
  for (uint32_t l = 0; l < n_lists_; l++) {
    h_row_off_[l + 1] = h_row_off_[l] + round_up<uint64_t>(sizes[l], kIndexGroupSize);
  }
  const uint64_t rows = h_row_off_.back();
  codes_.resize(round_up<uint64_t>(std::max<uint64_t>(rows, 32) * list_row_bytes(), 16));
  ids_.resize(std::max<uint64_t>(rows, 32));
  CUDA_TRY(cudaMemsetAsync(codes_.data(), 0, codes_.size(), stream));
  fill_i64_kernel<<<ceildiv<size_t>(ids_.size(), 256), 256, 0, stream>>>(ids_.data(), ids_.size(),
                                                                          kInvalidRecord);
  CUDA_TRY(cudaMemcpyAsync(list_sizes_.data(), h_list_sizes_.data(), size_t(n_lists_) * 4,
                           cudaMemcpyHostToDevice, stream));
  CUDA_TRY(cudaMemcpyAsync(row_off_.data(), h_row_off_.data(), (size_t(n_lists_) + 1) * 8,
                           cudaMemcpyHostToDevice, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  recompute_internal_state(stream);
}

void index<int64_t>::recompute_internal_state(cudaStream_t stream)
{
  // ivf_common.cuh:255-290: prefix sums of the list sizes sorted in descending order
  std::vector<uint32_t> sorted(h_list_sizes_);
  std::sort(sorted.begin(), sorted.end(), std::greater<uint32_t>());
  accum_sorted_sizes_.assign(size_t(n_lists_) + 1, 0);
  for (uint32_t l = 0; l < n_lists_; l++) {
    accum_sorted_sizes_[l + 1] = accum_sorted_sizes_[l] + sorted[l];
  }
  size_ = accum_sorted_sizes_.back();
  // an identity rotation lets search skip the rotation product (the result is bit-identical)
  std::vector<float> rot(size_t(rot_dim()) * dim_);
  CUDA_TRY(cudaMemcpyAsync(rot.data(), rotation_.data(), rot.size() * 4, cudaMemcpyDeviceToHost,
                           stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  bool ident = rot_dim() == dim_;
  for (uint32_t i = 0; ident && i < rot_dim(); i++) {
    for (uint32_t j = 0; j < dim_; j++) {
      if (rot[size_t(i) * dim_ + j] != (i == j ? 1.0f : 0.0f)) {
        ident = false;
        break;
      }
    }
  }
  rotation_is_identity_ = ident;
  centers_i8f_.reset();  // rebuilt from the current model on next use
  rotation_i8f_.reset();
  centers_h_.reset();
  rotation_h_.reset();
  // derived data of the tensor-core coarse search: the split centre rows with the |c|^2 column of the
  // L2 metrics rebalanced against the queries' -0.5 (the other metrics multiply that column by zero)
  const size_t nc = size_t(n_lists_) * dim_ext();
  if (centers_hi_.size() != nc) {
    centers_hi_.resize(nc);
    centers_lo_.resize(nc);
  }
  const bool norm_column = metric_ == DistanceType::L2Expanded || metric_ == DistanceType::L2SqrtExpanded;
  prepare_tc_centers(stream, centers_.data(), n_lists_, dim_ext(), norm_column ? dim_ : dim_ext(),
                     centers_hi_.data(), centers_lo_.data(), &centers_max_norm_, &centers_ext_scale_);
}

// ------------------------------------------------------------------------------------------------
// .npy framing
// ------------------------------------------------------------------------------------------------
namespace {

struct npy_header {
  char kind        = 'f';
  size_t itemsize  = 0;
  std::vector<uint64_t> shape;
  uint64_t count() const
  {
    uint64_t n = 1;
    for (auto s : shape) { n *= s; }
    return n;
  }
};

void write_header(std::ostream& os, const char* descr, const std::vector<uint64_t>& shape)
{
  std::string d = "{'descr': '";
  d += descr;
  d += "', 'fortran_order': False, 'shape': (";
  for (size_t i = 0; i < shape.size(); i++) {
    d += std::to_string(shape[i]);
    if (shape.size() == 1) {
      d += ",";
    } else if (i + 1 < shape.size()) {
      d += ", ";
    }
  }
  d += ")}";
  size_t preamble = 6 + 2 + 2 + d.size() + 1;
  size_t pad      = 64 - preamble % 64;
  std::string header = d + std::string(pad, ' ') + "\n";
  os.write("\x93NUMPY", 6);
  os.put(char(1));
  os.put(char(0));
  uint16_t hl = uint16_t(header.size());
  char b[2]   = {char(hl & 0xff), char(hl >> 8)};
  os.write(b, 2);
  os.write(header.data(), std::streamsize(header.size()));
}

template <typename T>
const char* descr_of();
template <> const char* descr_of<int32_t>() { return "<i4"; }
template <> const char* descr_of<int64_t>() { return "<i8"; }
template <> const char* descr_of<uint32_t>() { return "<u4"; }
template <> const char* descr_of<float>() { return "<f4"; }
template <> const char* descr_of<uint8_t>() { return "|u1"; }
template <> const char* descr_of<bool>() { return "|u1"; }

template <typename T>
void write_scalar(std::ostream& os, T v)
{
  write_header(os, descr_of<T>(), {});
  os.write(reinterpret_cast<const char*>(&v), sizeof(T));
}

npy_header read_header(std::istream& is)
{
  char magic[6];
  is.read(magic, 6);
  CUVS_EXPECTS(is.good() && std::memcmp(magic, "\x93NUMPY", 6) == 0,
               "ivf_pq::deserialize: bad record magic (not a serialized index?)");
  unsigned char ver[2];
  is.read(reinterpret_cast<char*>(ver), 2);
  uint32_t hlen = 0;
  if (ver[0] == 1) {
    unsigned char b[2];
    is.read(reinterpret_cast<char*>(b), 2);
    hlen = b[0] | (uint32_t(b[1]) << 8);
  } else {
    unsigned char b[4];
    is.read(reinterpret_cast<char*>(b), 4);
    hlen = b[0] | (uint32_t(b[1]) << 8) | (uint32_t(b[2]) << 16) | (uint32_t(b[3]) << 24);
  }
  CUVS_EXPECTS(is.good() && hlen > 0 && hlen < (1u << 20), "ivf_pq::deserialize: bad header length");
  std::string h(hlen, '\0');
  is.read(h.data(), hlen);
  CUVS_EXPECTS(is.good(), "ivf_pq::deserialize: truncated header");
  npy_header out;
  auto dpos = h.find("'descr'");
  CUVS_EXPECTS(dpos != std::string::npos, "ivf_pq::deserialize: header lacks descr");
  auto q1 = h.find('\'', h.find(':', dpos));
  auto q2 = h.find('\'', q1 + 1);
  CUVS_EXPECTS(q1 != std::string::npos && q2 != std::string::npos && q2 > q1 + 2,
               "ivf_pq::deserialize: malformed descr");
  std::string descr = h.substr(q1 + 1, q2 - q1 - 1);
  CUVS_EXPECTS(descr[0] == '<' || descr[0] == '|' || descr[0] == '=',
               "ivf_pq::deserialize: big-endian records are not supported");
  out.kind     = descr[1];
  out.itemsize = size_t(std::stoul(descr.substr(2)));
  auto fpos    = h.find("'fortran_order'");
  CUVS_EXPECTS(fpos != std::string::npos, "ivf_pq::deserialize: header lacks fortran_order");
  CUVS_EXPECTS(h.compare(h.find_first_not_of(" :", fpos + 15), 5, "False") == 0,
               "ivf_pq::deserialize: fortran-order records are not supported");
  auto spos = h.find("'shape'");
  CUVS_EXPECTS(spos != std::string::npos, "ivf_pq::deserialize: header lacks shape");
  auto p1 = h.find('(', spos);
  auto p2 = h.find(')', p1);
  CUVS_EXPECTS(p1 != std::string::npos && p2 != std::string::npos,
               "ivf_pq::deserialize: malformed shape");
  std::string sh = h.substr(p1 + 1, p2 - p1 - 1);
  size_t pos     = 0;
  while (pos < sh.size()) {
    while (pos < sh.size() && (sh[pos] == ' ' || sh[pos] == ',')) { pos++; }
    if (pos >= sh.size()) { break; }
    size_t end = pos;
    while (end < sh.size() && sh[end] >= '0' && sh[end] <= '9') { end++; }
    CUVS_EXPECTS(end > pos, "ivf_pq::deserialize: malformed shape");
    out.shape.push_back(std::stoull(sh.substr(pos, end - pos)));
    pos = end;
  }
  return out;
}

template <typename T>
T read_scalar(std::istream& is)
{
  npy_header h = read_header(is);
  CUVS_EXPECTS(h.itemsize == sizeof(T) && h.count() == 1,
               "ivf_pq::deserialize: scalar record has the wrong type or shape");
  T v{};
  is.read(reinterpret_cast<char*>(&v), sizeof(T));
  CUVS_EXPECTS(is.good(), "ivf_pq::deserialize: truncated scalar");
  return v;
}

// Read one array record of `count` elements of `itemsize` bytes straight into host memory.
void read_array(std::istream& is, void* dst, size_t itemsize, uint64_t count, const char* what)
{
  npy_header h = read_header(is);
  CUVS_EXPECTS(h.itemsize == itemsize && h.count() == count,
               "ivf_pq::deserialize: record `%s` has %llu elements of %zu bytes, expected %llu of %zu",
               what, (unsigned long long)h.count(), h.itemsize, (unsigned long long)count, itemsize);
  is.read(static_cast<char*>(dst), std::streamsize(itemsize * count));
  CUVS_EXPECTS(is.good(), "ivf_pq::deserialize: truncated record `%s`", what);
}

void skip_array(std::istream& is, size_t itemsize, uint64_t count, const char* what)
{
  npy_header h = read_header(is);
  CUVS_EXPECTS(h.itemsize == itemsize && h.count() == count,
               "ivf_pq::deserialize: record `%s` has an unexpected size", what);
  is.seekg(std::streamoff(itemsize * count), std::ios::cur);
  CUVS_EXPECTS(is.good(), "ivf_pq::deserialize: truncated record `%s`", what);
}

void write_device_f32(raft::resources& res, std::ostream& os, const float* dptr,
                      const std::vector<uint64_t>& shape)
{
  uint64_t n = 1;
  for (auto s : shape) { n *= s; }
  std::vector<float> h(n);
  CUDA_TRY(cudaMemcpyAsync(h.data(), dptr, n * 4, cudaMemcpyDeviceToHost, res.stream));
  res.sync();
  write_header(os, "<f4", shape);
  os.write(reinterpret_cast<const char*>(h.data()), std::streamsize(n * 4));
}

void read_device_f32(raft::resources& res, std::istream& is, float* dptr, uint64_t n,
                     const char* what)
{
  std::vector<float> h(n);
  read_array(is, h.data(), 4, n, what);
  CUDA_TRY(cudaMemcpyAsync(dptr, h.data(), n * 4, cudaMemcpyHostToDevice, res.stream));
  res.sync();
}

// cpp/src/util/serialize_validation.hpp
constexpr uint32_t kMaxIvfNLists = 1u << 24;

}  // namespace

// ------------------------------------------------------------------------------------------------
// serialize
// ------------------------------------------------------------------------------------------------
void serialize(raft::resources& res, std::ostream& os, const index<int64_t>& idx)
{
  write_scalar<int32_t>(os, 4);
  write_scalar<int64_t>(os, idx.size());
  write_scalar<uint32_t>(os, idx.dim());
  write_scalar<uint32_t>(os, idx.pq_bits());
  write_scalar<uint32_t>(os, idx.pq_dim());
  write_scalar<bool>(os, idx.conservative_memory_allocation());
  write_scalar<int32_t>(os, int32_t(idx.metric()));
  write_scalar<int32_t>(os, int32_t(idx.codebook_kind()));
  write_scalar<int32_t>(os, int32_t(idx.codes_layout()));
  write_scalar<uint32_t>(os, idx.n_lists());
  const bool flat = idx.codes_layout() == list_layout::FLAT;

  const uint64_t first = idx.codebook_kind() == codebook_gen::PER_SUBSPACE ? idx.pq_dim() : idx.n_lists();
  write_device_f32(res, os, idx.pq_centers(), {first, idx.pq_len(), idx.pq_book_size()});
  write_device_f32(res, os, idx.centers(), {idx.n_lists(), idx.dim_ext()});
  write_device_f32(res, os, idx.centers_rot(), {idx.n_lists(), idx.rot_dim()});
  write_device_f32(res, os, idx.rotation_matrix(), {idx.rot_dim(), idx.dim()});
  const auto& sizes = idx.host_list_sizes();
  write_header(os, "<u4", {idx.n_lists()});
  os.write(reinterpret_cast<const char*>(sizes.data()), std::streamsize(size_t(idx.n_lists()) * 4));

  // Lists: stage the arenas through host memory in chunks of whole lists.
  const auto& off          = idx.host_row_offsets();
  const uint64_t row_bytes = idx.list_row_bytes();
  const uint64_t chunk_rows = std::max<uint64_t>(1u << 20, 1);  // rows per staging chunk (target)
  std::vector<uint8_t> hcodes;
  std::vector<int64_t> hids;
  uint32_t l = 0;
  while (l < idx.n_lists()) {
    uint32_t l_end = l;
    while (l_end < idx.n_lists() && (l_end == l || off[l_end + 1] - off[l] <= chunk_rows)) { l_end++; }
    const uint64_t r0 = off[l], rows = off[l_end] - off[l];
    hcodes.resize(rows * row_bytes);
    hids.resize(rows);
    if (rows) {
      CUDA_TRY(cudaMemcpyAsync(hcodes.data(), idx.codes() + r0 * row_bytes, rows * row_bytes,
                               cudaMemcpyDeviceToHost, res.stream));
      CUDA_TRY(cudaMemcpyAsync(hids.data(), idx.ids() + r0, rows * 8, cudaMemcpyDeviceToHost,
                               res.stream));
      res.sync();
    }
    for (uint32_t i = l; i < l_end; i++) {
      write_scalar<uint32_t>(os, sizes[i]);
      if (sizes[i] == 0) { continue; }
      if (flat) {
        // ivf_list.cuh:108-132 with list_spec_flat: exactly `size` rows of bytes_per_vector bytes
        write_header(os, "|u1", {sizes[i], idx.bytes_per_vector()});
        os.write(reinterpret_cast<const char*>(hcodes.data() + (off[i] - r0) * row_bytes),
                 std::streamsize(uint64_t(sizes[i]) * row_bytes));
      } else {
        const uint64_t g = ceildiv<uint64_t>(sizes[i], kIndexGroupSize);
        write_header(os, "|u1", {g, idx.n_pieces(), kIndexGroupSize, kIndexGroupVecLen});
        os.write(reinterpret_cast<const char*>(hcodes.data() + (off[i] - r0) * row_bytes),
                 std::streamsize(g * kIndexGroupSize * row_bytes));
      }
      write_header(os, "<i8", {sizes[i]});
      os.write(reinterpret_cast<const char*>(hids.data() + (off[i] - r0)),
               std::streamsize(uint64_t(sizes[i]) * 8));
    }
    l = l_end;
  }
  CUVS_EXPECTS(os.good(), "Error writing the index");
}

std::vector<int> list_owners(const std::vector<uint32_t>& list_sizes, int shard_count)
{
  CUVS_EXPECTS(shard_count >= 1, "invalid number of shards %d", shard_count);
  const size_t n = list_sizes.size();
  std::vector<int> owner(n, 0);
  if (shard_count == 1) { return owner; }
  std::vector<uint32_t> order(n);
  for (size_t i = 0; i < n; i++) { order[i] = uint32_t(i); }
  std::stable_sort(order.begin(), order.end(),
                   [&](uint32_t a, uint32_t b) { return list_sizes[a] > list_sizes[b]; });
  // (rows held, rank) min-heap
  using slot = std::pair<uint64_t, int>;
  std::priority_queue<slot, std::vector<slot>, std::greater<slot>> load;
  for (int r = 0; r < shard_count; r++) { load.push({0, r}); }
  for (uint32_t l : order) {
    slot s = load.top();
    load.pop();
    owner[l] = s.second;
    // an empty list still counts as one unit so that empty lists spread evenly too
    s.first += std::max<uint32_t>(list_sizes[l], 1u);
    load.push(s);
  }
  return owner;
}

void serialize_list_sharded(const std::vector<raft::resources*>& res, std::ostream& os,
                            const std::vector<const index<int64_t>*>& shards)
{
  CUVS_EXPECTS(!shards.empty() && shards.size() == res.size(), "serialize_list_sharded: no shards");
  const index<int64_t>& m = *shards[0];
  CUVS_EXPECTS(m.codes_layout() == list_layout::INTERLEAVED, "list-sharded indexes use the INTERLEAVED layout");
  const uint32_t n_lists  = m.n_lists();
  std::vector<uint32_t> sizes(n_lists, 0);
  std::vector<int> holder(n_lists, 0);
  int64_t total = 0;
  for (size_t r = 0; r < shards.size(); r++) {
    CUVS_EXPECTS(shards[r]->n_lists() == n_lists, "serialize_list_sharded: shards of different indexes");
    const auto& hs = shards[r]->host_list_sizes();
    for (uint32_t l = 0; l < n_lists; l++) {
      if (hs[l] > 0) {
        CUVS_EXPECTS(sizes[l] == 0, "serialize_list_sharded: list %u is held by two shards", l);
        sizes[l]  = hs[l];
        holder[l] = int(r);
        total += hs[l];
      }
    }
  }
  int saved = 0;
  CUDA_TRY(cudaGetDevice(&saved));
  CUDA_TRY(cudaSetDevice(res[0]->device));
  write_scalar<int32_t>(os, 4);
  write_scalar<int64_t>(os, total);
  write_scalar<uint32_t>(os, m.dim());
  write_scalar<uint32_t>(os, m.pq_bits());
  write_scalar<uint32_t>(os, m.pq_dim());
  write_scalar<bool>(os, m.conservative_memory_allocation());
  write_scalar<int32_t>(os, int32_t(m.metric()));
  write_scalar<int32_t>(os, int32_t(m.codebook_kind()));
  write_scalar<int32_t>(os, int32_t(list_layout::INTERLEAVED));
  write_scalar<uint32_t>(os, n_lists);
  const uint64_t first = m.codebook_kind() == codebook_gen::PER_SUBSPACE ? m.pq_dim() : n_lists;
  write_device_f32(*res[0], os, m.pq_centers(), {first, m.pq_len(), m.pq_book_size()});
  write_device_f32(*res[0], os, m.centers(), {n_lists, m.dim_ext()});
  write_device_f32(*res[0], os, m.centers_rot(), {n_lists, m.rot_dim()});
  write_device_f32(*res[0], os, m.rotation_matrix(), {m.rot_dim(), m.dim()});
  write_header(os, "<u4", {n_lists});
  os.write(reinterpret_cast<const char*>(sizes.data()), std::streamsize(size_t(n_lists) * 4));
  const uint64_t row_bytes = uint64_t(m.n_pieces()) * kIndexGroupVecLen;
  std::vector<uint8_t> hcodes;
  std::vector<int64_t> hids;
  for (uint32_t l = 0; l < n_lists; l++) {
    write_scalar<uint32_t>(os, sizes[l]);
    if (sizes[l] == 0) { continue; }
    const index<int64_t>& s = *shards[holder[l]];
    const uint64_t r0       = s.host_row_offsets()[l];
    const uint64_t rows     = round_up<uint64_t>(sizes[l], kIndexGroupSize);
    hcodes.resize(rows * row_bytes);
    hids.resize(sizes[l]);
    CUDA_TRY(cudaSetDevice(res[holder[l]]->device));
    CUDA_TRY(cudaMemcpy(hcodes.data(), s.codes() + r0 * row_bytes, rows * row_bytes, cudaMemcpyDeviceToHost));
    CUDA_TRY(cudaMemcpy(hids.data(), s.ids() + r0, size_t(sizes[l]) * 8, cudaMemcpyDeviceToHost));
    write_header(os, "|u1", {rows / kIndexGroupSize, m.n_pieces(), kIndexGroupSize, kIndexGroupVecLen});
    os.write(reinterpret_cast<const char*>(hcodes.data()), std::streamsize(rows * row_bytes));
    write_header(os, "<i8", {sizes[l]});
    os.write(reinterpret_cast<const char*>(hids.data()), std::streamsize(uint64_t(sizes[l]) * 8));
  }
  CUDA_TRY(cudaSetDevice(saved));
  CUVS_EXPECTS(os.good(), "Error writing the index");
}

void serialize(raft::resources& res, const std::string& filename, const index<int64_t>& idx)
{
  std::ofstream of(filename, std::ios::out | std::ios::binary);
  CUVS_EXPECTS(bool(of), "Cannot open file %s", filename.c_str());
  serialize(res, of, idx);
  of.close();
  CUVS_EXPECTS(bool(of), "Error writing output %s", filename.c_str());
}

// ------------------------------------------------------------------------------------------------
// deserialize
// ------------------------------------------------------------------------------------------------
void deserialize(raft::resources& res, std::istream& is, index<int64_t>* out, int shard_rank,
                 int shard_count)
{
  CUVS_EXPECTS(shard_count >= 1 && shard_rank >= 0 && shard_rank < shard_count,
               "invalid shard rank %d of %d", shard_rank, shard_count);
  auto ver = read_scalar<int32_t>(is);
  CUVS_EXPECTS(ver == 4, "serialization version mismatch %d vs. %d", ver, 4);
  auto n_rows  = read_scalar<int64_t>(is);
  auto dim     = read_scalar<uint32_t>(is);
  auto pq_bits = read_scalar<uint32_t>(is);
  auto pq_dim  = read_scalar<uint32_t>(is);
  auto cma     = read_scalar<uint8_t>(is) != 0;
  auto metric  = read_scalar<int32_t>(is);
  auto kind    = read_scalar<int32_t>(is);
  auto layout  = read_scalar<int32_t>(is);
  auto n_lists = read_scalar<uint32_t>(is);

  // ivf_pq_serialize.cuh:148-174
  CUVS_EXPECTS(metric == 0 || metric == 1 || metric == 2 || metric == 6,
               "ivf_pq::deserialize: invalid metric value %d", metric);
  CUVS_EXPECTS(kind == 0 || kind == 1, "ivf_pq::deserialize: invalid codebook_gen value %d", kind);
  CUVS_EXPECTS(layout == 0 || layout == 1, "ivf_pq::deserialize: invalid list_layout value %d",
               layout);
  CUVS_EXPECTS(n_lists > 0 && n_lists <= kMaxIvfNLists,
               "ivf_pq::deserialize: n_lists=%u exceeds maximum %u", n_lists, kMaxIvfNLists);
  CUVS_EXPECTS(dim > 0 && dim <= (1u << 20) && pq_dim > 0 && pq_dim <= dim * 8u + 8u,
               "ivf_pq::deserialize: implausible dim=%u / pq_dim=%u", dim, pq_dim);
  CUVS_EXPECTS(n_rows >= 0, "ivf_pq::deserialize: negative size");

  index<int64_t> idx(DistanceType(metric), codebook_gen(kind), n_lists, dim, pq_bits, pq_dim, cma,
                     list_layout(layout));
  const bool flat = layout == int(list_layout::FLAT);
  read_device_f32(res, is, idx.pq_centers(), idx.pq_centers_size(), "pq_centers");
  read_device_f32(res, is, idx.centers(), uint64_t(n_lists) * idx.dim_ext(), "centers");
  read_device_f32(res, is, idx.centers_rot(), uint64_t(n_lists) * idx.rot_dim(), "centers_rot");
  read_device_f32(res, is, idx.rotation_matrix(), uint64_t(idx.rot_dim()) * dim, "rotation_matrix");
  std::vector<uint32_t> sizes(n_lists);
  read_array(is, sizes.data(), 4, n_lists, "list_sizes");
  uint64_t total = 0;
  for (auto s : sizes) { total += s; }
  CUVS_EXPECTS(total == uint64_t(n_rows),
               "ivf_pq::deserialize: list sizes sum to %llu but the index size is %lld",
               (unsigned long long)total, (long long)n_rows);
  std::vector<uint32_t> kept(sizes);
  if (shard_count > 1) {
    const std::vector<int> owner = list_owners(sizes, shard_count);
    for (uint32_t l = 0; l < n_lists; l++) {
      if (owner[l] != shard_rank) { kept[l] = 0; }
    }
  }
  idx.allocate_lists(kept, res.stream);

  const uint64_t row_bytes = idx.list_row_bytes();
  const auto& off          = idx.host_row_offsets();
  // Consecutive lists are consecutive in the arenas, so payloads are staged back to back and
  // flushed with one copy per arena.
  const uint64_t stage_rows = 1u << 20;
  std::vector<uint8_t> hcodes;
  std::vector<int64_t> hids;
  hcodes.reserve(stage_rows * row_bytes);
  hids.reserve(stage_rows);
  uint64_t stage_r0 = 0;
  auto flush = [&]() {
    if (hids.empty()) { return; }
    CUDA_TRY(cudaMemcpyAsync(idx.codes() + stage_r0 * row_bytes, hcodes.data(), hcodes.size(),
                             cudaMemcpyHostToDevice, res.stream));
    CUDA_TRY(cudaMemcpyAsync(idx.ids() + stage_r0, hids.data(), hids.size() * 8,
                             cudaMemcpyHostToDevice, res.stream));
    res.sync();
    stage_r0 += hids.size();
    hcodes.clear();
    hids.clear();
  };
  for (uint32_t l = 0; l < n_lists; l++) {
    auto sz = read_scalar<uint32_t>(is);
    CUVS_EXPECTS(sz == sizes[l], "ivf_pq::deserialize: list %u has size %u, header says %u", l, sz,
                 sizes[l]);
    if (sz == 0) { continue; }
    const uint64_t rows = round_up<uint64_t>(sz, kIndexGroupSize);
    // rows the record holds: whole 32-row groups (interleaved) or exactly `sz` (flat)
    const uint64_t file_rows = flat ? uint64_t(sz) : rows;
    if (kept[l] == 0) {
      skip_array(is, 1, file_rows * row_bytes, "list codes");
      skip_array(is, 8, sz, "list indices");
      continue;
    }
    CUVS_EXPECTS(stage_r0 + hids.size() == off[l], "internal error: arena offset mismatch");
    size_t c0 = hcodes.size(), i0 = hids.size();
    hcodes.resize(c0 + rows * row_bytes);
    hids.resize(i0 + rows, kInvalidRecord);
    read_array(is, hcodes.data() + c0, 1, file_rows * row_bytes, "list codes");
    read_array(is, hids.data() + i0, 8, sz, "list indices");
    if (hids.size() >= stage_rows) { flush(); }
  }
  flush();
  idx.recompute_internal_state(res.stream);
  *out = std::move(idx);
}

void deserialize(raft::resources& res, const std::string& filename, index<int64_t>* idx,
                 int shard_rank, int shard_count)
{
  std::ifstream in(filename, std::ios::in | std::ios::binary);
  CUVS_EXPECTS(bool(in), "Cannot open file %s", filename.c_str());
  deserialize(res, in, idx, shard_rank, shard_count);
}

// ------------------------------------------------------------------------------------------------
// multi-GPU index files of the reference (cpp/src/neighbors/mg/snmg.cuh:60-91 reader, :780-805 writer):
// four bytes with the numpy dtype string of the dataset type, the distribution mode and the number
// of ranks as scalar records, then one complete index stream per rank.
// ------------------------------------------------------------------------------------------------
namespace {

// Steps over one index stream; returns its size (number of vectors).
int64_t skip_index(std::istream& is)
{
  auto ver = read_scalar<int32_t>(is);
  CUVS_EXPECTS(ver == 4, "serialization version mismatch %d vs. %d", ver, 4);
  auto n_rows = read_scalar<int64_t>(is);
  read_scalar<uint32_t>(is);  // dim
  read_scalar<uint32_t>(is);  // pq_bits
  read_scalar<uint32_t>(is);  // pq_dim
  read_scalar<uint8_t>(is);   // conservative_memory_allocation
  read_scalar<int32_t>(is);   // metric
  read_scalar<int32_t>(is);   // codebook kind
  read_scalar<int32_t>(is);   // list layout
  auto n_lists = read_scalar<uint32_t>(is);
  CUVS_EXPECTS(n_lists > 0 && n_lists <= kMaxIvfNLists, "ivf_pq::deserialize: n_lists=%u exceeds maximum %u",
               n_lists, kMaxIvfNLists);
  auto skip_any = [&](const char* what) {
    npy_header h = read_header(is);
    is.seekg(std::streamoff(h.itemsize * h.count()), std::ios::cur);
    CUVS_EXPECTS(is.good(), "ivf_pq::deserialize: truncated record `%s`", what);
  };
  skip_any("pq_centers");
  skip_any("centers");
  skip_any("centers_rot");
  skip_any("rotation_matrix");
  std::vector<uint32_t> sizes(n_lists);
  read_array(is, sizes.data(), 4, n_lists, "list_sizes");
  for (uint32_t l = 0; l < n_lists; l++) {
    auto sz = read_scalar<uint32_t>(is);
    CUVS_EXPECTS(sz == sizes[l], "ivf_pq::deserialize: list %u has size %u, header says %u", l, sz, sizes[l]);
    if (sz == 0) { continue; }
    skip_any("list codes");
    skip_any("list indices");
  }
  return n_rows;
}

}  // namespace

void deserialize_mg_rank(raft::resources& res, const std::string& filename, int rank, int n_ranks,
                         index<int64_t>* idx, int* mode, int64_t* id_offset)
{
  std::ifstream is(filename, std::ios::in | std::ios::binary);
  CUVS_EXPECTS(bool(is), "Cannot open file %s", filename.c_str());
  char dtype_string[4];
  is.read(dtype_string, 4);
  CUVS_EXPECTS(is.good(), "Cannot read the header of %s", filename.c_str());
  const int m      = read_scalar<int32_t>(is);
  const int stored = read_scalar<int32_t>(is);
  CUVS_EXPECTS(m == 0 || m == 1, "multi-GPU index file: invalid distribution mode %d", m);
  // snmg.cuh:77-81
  CUVS_EXPECTS(stored == n_ranks, "Serialized index has %d ranks whereas NCCL clique has %d ranks", stored,
               n_ranks);
  CUVS_EXPECTS(rank >= 0 && rank < n_ranks, "invalid rank %d of %d", rank, n_ranks);
  int64_t offset = 0;
  for (int r = 0; r < rank; r++) { offset += skip_index(is); }
  deserialize(res, is, idx, 0, 1);
  *mode      = m;
  *id_offset = m == 1 ? offset : 0;  // SHARDED: ids are local to a rank's rows (snmg.cuh:351-355)
}

void serialize_mg_header(std::ostream& os, const char* dtype_string, int mode, int n_ranks)
{
  char d[4] = {0, 0, 0, 0};
  std::strncpy(d, dtype_string, 4);
  os.write(d, 4);
  write_scalar<int32_t>(os, mode);
  write_scalar<int32_t>(os, n_ranks);
}

void serialize_mg(raft::resources& res, const std::string& filename, int mode, const char* dtype_string,
                  const std::vector<const index<int64_t>*>& per_rank)
{
  CUVS_EXPECTS(mode == 0 || mode == 1, "invalid distribution mode %d", mode);
  std::ofstream of(filename, std::ios::out | std::ios::binary);
  CUVS_EXPECTS(bool(of), "Cannot open file %s", filename.c_str());
  serialize_mg_header(of, dtype_string, mode, int(per_rank.size()));
  for (auto* ix : per_rank) { serialize(res, of, *ix); }
  of.close();
  CUVS_EXPECTS(bool(of), "Error writing output %s", filename.c_str());
}

}  // namespace cuvs::neighbors::ivf_pq

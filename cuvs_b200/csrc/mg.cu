// Multi-GPU IVF-PQ host side: see mg.hpp for the design.  Reference semantics followed:
// cpp/src/neighbors/mg/snmg.cuh:48-91 (distribute / deserialize), :93-246 (build / extend),
// :249-561 (sharded search with merge), :563-700 (replicated search), :780-805 (serialize).
#include "mg.hpp"

#include <nccl.h>  // types and prototypes only; the library itself is bound at run time

#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>

namespace cuvs::neighbors::mg {

using namespace cuvs_b200;

// ------------------------------------------------------------------------------------------------
// NCCL, bound with dlopen so that the library has no link-time dependency on it
// ------------------------------------------------------------------------------------------------
namespace {

struct nccl_api {
  decltype(&ncclGetUniqueId) GetUniqueId     = nullptr;
  decltype(&ncclCommInitRank) CommInitRank   = nullptr;
  decltype(&ncclCommInitAll) CommInitAll     = nullptr;
  decltype(&ncclCommDestroy) CommDestroy     = nullptr;
  decltype(&ncclAllGather) AllGather         = nullptr;
  decltype(&ncclAllReduce) AllReduce         = nullptr;
  decltype(&ncclSend) Send                   = nullptr;
  decltype(&ncclRecv) Recv                   = nullptr;
  decltype(&ncclGroupStart) GroupStart       = nullptr;
  decltype(&ncclGroupEnd) GroupEnd           = nullptr;
  decltype(&ncclGetErrorString) ErrorString  = nullptr;
};

const nccl_api& nccl()
{
  static nccl_api api;
  static std::once_flag once;
  static std::string problem;
  std::call_once(once, [] {
    void* h = nullptr;
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      h = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (h) { break; }
    }
    if (!h) {
      problem = "NCCL (libnccl.so.2) could not be loaded: multi-GPU search is unavailable";
      return;
    }
    auto sym = [&](const char* n) {
      void* p = dlsym(h, n);
      if (!p) { problem = std::string("NCCL symbol not found: ") + n; }
      return p;
    };
    api.GetUniqueId  = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommInitAll  = reinterpret_cast<decltype(api.CommInitAll)>(sym("ncclCommInitAll"));
    api.CommDestroy  = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllGather    = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.AllReduce    = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.Send         = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
    api.Recv         = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
    api.GroupStart   = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd     = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.ErrorString  = reinterpret_cast<decltype(api.ErrorString)>(sym("ncclGetErrorString"));
  });
  if (!problem.empty()) { fail("%s", problem.c_str()); }
  return api;
}

#define NCCL_TRY(call)                                                                   \
  do {                                                                                   \
    ncclResult_t r__ = (call);                                                           \
    if (r__ != ncclSuccess) {                                                            \
      ::cuvs_b200::fail("NCCL error at %s:%d: %s", __FILE__, __LINE__, nccl().ErrorString(r__)); \
    }                                                                                    \
  } while (0)

struct device_guard {
  int saved = 0;
  explicit device_guard(int dev)
  {
    CUDA_TRY(cudaGetDevice(&saved));
    if (dev != saved) { CUDA_TRY(cudaSetDevice(dev)); }
  }
  ~device_guard() { cudaSetDevice(saved); }
};

bool is_min_close(ivf_pq::DistanceType m) { return m != ivf_pq::DistanceType::InnerProduct; }

__global__ void add_offset_kernel(int64_t* ids, size_t n, int64_t offset)
{
  size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  // ids of missing results (INT64_MAX) stay as they are
  if (i < n && ids[i] != ivf_pq::kOutOfBoundsRecord) { ids[i] += offset; }
}

}  // namespace

static_assert(sizeof(nccl_unique_id) == sizeof(ncclUniqueId), "ncclUniqueId is 128 bytes");

void make_unique_id(nccl_unique_id* id)
{
  ncclUniqueId u;
  NCCL_TRY(nccl().GetUniqueId(&u));
  std::memcpy(id->bytes, &u, sizeof(u));
}

// ------------------------------------------------------------------------------------------------
// rank_comm
// ------------------------------------------------------------------------------------------------
rank_comm::rank_comm(const nccl_unique_id& id, int rank, int n_ranks) : owns_(true), rank_(rank), n_ranks_(n_ranks)
{
  CUVS_EXPECTS(n_ranks >= 1 && rank >= 0 && rank < n_ranks, "invalid rank %d of %d", rank, n_ranks);
  ncclUniqueId u;
  std::memcpy(&u, id.bytes, sizeof(u));
  ncclComm_t c = nullptr;
  NCCL_TRY(nccl().CommInitRank(&c, n_ranks, u, rank));
  comm_ = c;
}

rank_comm::rank_comm(ncclComm* comm, int rank, int n_ranks) : comm_(comm), owns_(false), rank_(rank), n_ranks_(n_ranks)
{
  CUVS_EXPECTS(n_ranks >= 1 && rank >= 0 && rank < n_ranks, "invalid rank %d of %d", rank, n_ranks);
  CUVS_EXPECTS(comm != nullptr || n_ranks == 1, "null communicator");
}

rank_comm::~rank_comm()
{
  for (auto& m : pending_) {
    for (auto& e : m.e) { cudaEventDestroy(e); }
  }
  if (owns_ && comm_) { nccl().CommDestroy(comm_); }
}

void rank_comm::mark(raft::resources& res, int i)
{
  if (!res.stats_enabled) { return; }
  if (i == 0) {
    pending_.emplace_back();
    for (auto& e : pending_.back().e) { CUDA_TRY(cudaEventCreate(&e)); }
  }
  CUDA_TRY(cudaEventRecord(pending_.back().e[i], res.stream));
}

void rank_comm::stats(double ms[5], uint64_t* batches, bool reset)
{
  for (auto& m : pending_) {
    CUDA_TRY(cudaEventSynchronize(m.e[5]));
    for (int i = 0; i < 5; i++) {
      float t = 0.0f;
      CUDA_TRY(cudaEventElapsedTime(&t, m.e[i], m.e[i + 1]));
      stage_ms_[i] += t;
    }
    for (auto& e : m.e) { cudaEventDestroy(e); }
    stat_batches_++;
  }
  pending_.clear();
  for (int i = 0; i < 5; i++) { ms[i] = stage_ms_[i]; }
  *batches = stat_batches_;
  if (reset) {
    for (auto& v : stage_ms_) { v = 0; }
    stat_batches_ = 0;
  }
}

void rank_comm::reserve(uint32_t nq, uint32_t n_probes, uint32_t k)
{
  nq_       = nq;
  k_        = k;
  n_probes_ = n_probes;
  slice_    = ceildiv<uint32_t>(nq, uint32_t(n_ranks_));
  ids_bytes_   = round_up<size_t>(size_t(nq) * k * 8, 16);
  block_bytes_ = ids_bytes_ + round_up<size_t>(size_t(nq) * k * 4, 16);
  const size_t np = size_t(n_ranks_) * slice_ * n_probes;
  if (probes_.size() < np) { probes_.resize(np + np / 4); }
  const size_t nb = size_t(n_ranks_) * block_bytes_;
  if (blocks_.size() < nb) { blocks_.resize(nb + nb / 4); }
}

void* rank_comm::query_buffer(size_t bytes)
{
  if (queries_.size() < bytes) { queries_.resize(bytes + bytes / 4); }
  return queries_.data();
}
float* rank_comm::out_distances(size_t n)
{
  if (out_d_.size() < n) { out_d_.resize(n + n / 4); }
  return out_d_.data();
}
int64_t* rank_comm::out_neighbors(size_t n)
{
  if (out_i_.size() < n) { out_i_.resize(n + n / 4); }
  return out_i_.data();
}

void rank_comm::select(raft::resources& res, const ivf_pq::search_params& p, const index<int64_t>& shard,
                       const void* queries, elem_t qtype, uint32_t nq, uint32_t k)
{
  const uint32_t n_probes = std::min<uint32_t>(p.n_probes, shard.n_lists());
  CUVS_EXPECTS(n_probes > 0, "n_probes (number of clusters to probe in the search) must be positive.");
  reserve(nq, n_probes, k);
  // this rank selects the probes of its slice of the batch, straight into its slot of the gathered array
  const uint32_t lo = std::min<uint32_t>(nq, uint32_t(rank_) * slice_);
  const uint32_t hi = std::min<uint32_t>(nq, lo + slice_);
  if (hi > lo) {
    ivf_pq::select_probes_any(res, shard, static_cast<const char*>(queries) + size_t(lo) * shard.dim() * elem_size(qtype),
                              qtype, hi - lo, n_probes, probes_.data() + size_t(lo) * n_probes,
                              p.coarse_search_dtype);
  }
}

void rank_comm::gather_probes(cudaStream_t stream)
{
  if (n_ranks_ == 1) { return; }
  const size_t count = size_t(slice_) * n_probes_;
  NCCL_TRY(nccl().AllGather(probes_.data() + size_t(rank_) * count, probes_.data(), count, ncclUint32, comm_, stream));
}

void rank_comm::scan(raft::resources& res, const ivf_pq::search_params& p, const index<int64_t>& shard,
                     const void* queries, elem_t qtype, bool exchange_bounds)
{
  uint8_t* block = blocks_.data() + size_t(rank_) * block_bytes_;
  // One process per GPU: between the nearest-probe pairs and the rest the ranks min-reduce their bounds
  // on every query's k-th best score (4 bytes per query), so that each prunes like the single-GPU search.
  struct hook_guard {
    raft::resources& r;
    ~hook_guard() { r.scan_phase_hook = nullptr; }
  } guard{res};
  if (exchange_bounds && n_ranks_ > 1) {
    ncclComm* comm = comm_;
    res.scan_phase_hook = [comm](cudaStream_t stream, uint32_t* kth, uint32_t n) {
      NCCL_TRY(nccl().AllReduce(kth, kth, n, ncclUint32, ncclMin, comm, stream));
    };
  }
  ivf_pq::search_any(res, p, shard, queries, qtype, nq_, k_, reinterpret_cast<int64_t*>(block),
                     reinterpret_cast<float*>(block + ids_bytes_), probes_.data());
}

void rank_comm::search_rows(raft::resources& res, const ivf_pq::search_params& p, const index<int64_t>& part,
                            const void* queries, elem_t qtype, uint32_t nq, uint32_t k, int64_t id_offset)
{
  reserve(nq, 1, k);
  uint8_t* block = blocks_.data() + size_t(rank_) * block_bytes_;
  auto* ids      = reinterpret_cast<int64_t*>(block);
  ivf_pq::search_any(res, p, part, queries, qtype, nq, k, ids, reinterpret_cast<float*>(block + ids_bytes_));
  if (id_offset != 0) {
    const size_t n = size_t(nq) * k;
    add_offset_kernel<<<unsigned(ceildiv<size_t>(n, 256)), 256, 0, res.stream>>>(ids, n, id_offset);
    CUDA_TRY(cudaGetLastError());
    res.launches++;
  }
}

void rank_comm::gather_results(cudaStream_t stream)
{
  if (n_ranks_ == 1) { return; }
  NCCL_TRY(nccl().AllGather(blocks_.data() + size_t(rank_) * block_bytes_, blocks_.data(), block_bytes_, ncclChar,
                            comm_, stream));
}

void rank_comm::merge(raft::resources& res, bool select_min, int64_t* neighbors, float* distances)
{
  const auto* ids = reinterpret_cast<const int64_t*>(blocks_.data());
  const auto* ds  = reinterpret_cast<const float*>(blocks_.data() + ids_bytes_);
  ivf_pq::detail::knn_merge_parts(res, ds, ids, distances, neighbors, uint32_t(n_ranks_), nq_, k_, select_min,
                                  block_bytes_ / 4, block_bytes_ / 8);
}

void rank_comm::exchange_slices(cudaStream_t stream)
{
  // rows [j * slice_, ...) of this rank's block go to rank j; this rank's rows arrive from every rank
  const size_t part_ids   = round_up<size_t>(size_t(slice_) * k_ * 8, 16);
  const size_t part_bytes = part_ids + round_up<size_t>(size_t(slice_) * k_ * 4, 16);
  const size_t need       = size_t(n_ranks_) * part_bytes;
  if (parts_.size() < need) { parts_.resize(need + need / 4); }
  const uint8_t* block = blocks_.data() + size_t(rank_) * block_bytes_;
  const auto* ids      = reinterpret_cast<const int64_t*>(block);
  const auto* ds       = reinterpret_cast<const float*>(block + ids_bytes_);
  const uint32_t my_lo = std::min<uint32_t>(nq_, uint32_t(rank_) * slice_);
  const uint32_t my_n  = std::min<uint32_t>(nq_, my_lo + slice_) - my_lo;
  NCCL_TRY(nccl().GroupStart());
  for (int j = 0; j < n_ranks_; j++) {
    const uint32_t lo = std::min<uint32_t>(nq_, uint32_t(j) * slice_);
    const uint32_t n  = std::min<uint32_t>(nq_, lo + slice_) - lo;
    if (n > 0) {
      NCCL_TRY(nccl().Send(ids + size_t(lo) * k_, size_t(n) * k_, ncclInt64, j, comm_, stream));
      NCCL_TRY(nccl().Send(ds + size_t(lo) * k_, size_t(n) * k_, ncclFloat, j, comm_, stream));
    }
    if (my_n > 0) {
      uint8_t* part = parts_.data() + size_t(j) * part_bytes;
      NCCL_TRY(nccl().Recv(part, size_t(my_n) * k_, ncclInt64, j, comm_, stream));
      NCCL_TRY(nccl().Recv(part + part_ids, size_t(my_n) * k_, ncclFloat, j, comm_, stream));
    }
  }
  NCCL_TRY(nccl().GroupEnd());
}

void rank_comm::merge_slice_and_gather(raft::resources& res, bool select_min, int64_t* neighbors, float* distances)
{
  const size_t part_ids   = round_up<size_t>(size_t(slice_) * k_ * 8, 16);
  const size_t part_bytes = part_ids + round_up<size_t>(size_t(slice_) * k_ * 4, 16);
  const uint32_t my_lo    = std::min<uint32_t>(nq_, uint32_t(rank_) * slice_);
  const uint32_t my_n     = std::min<uint32_t>(nq_, my_lo + slice_) - my_lo;
  // the merged slices are gathered in place where the batch divides evenly, else through padded buffers
  const bool even   = size_t(slice_) * n_ranks_ == nq_;
  const size_t rows = size_t(slice_) * n_ranks_;
  int64_t* fin_i    = even ? neighbors : out_neighbors(rows * k_);
  float* fin_d      = even ? distances : out_distances(rows * k_);
  if (my_n > 0) {
    ivf_pq::detail::knn_merge_parts(res, reinterpret_cast<const float*>(parts_.data() + part_ids),
                                    reinterpret_cast<const int64_t*>(parts_.data()),
                                    fin_d + size_t(rank_) * slice_ * k_, fin_i + size_t(rank_) * slice_ * k_,
                                    uint32_t(n_ranks_), my_n, k_, select_min, part_bytes / 4, part_bytes / 8);
  }
  const size_t count = size_t(slice_) * k_;
  NCCL_TRY(nccl().GroupStart());
  NCCL_TRY(nccl().AllGather(fin_i + size_t(rank_) * count, fin_i, count, ncclInt64, comm_, res.stream));
  NCCL_TRY(nccl().AllGather(fin_d + size_t(rank_) * count, fin_d, count, ncclFloat, comm_, res.stream));
  NCCL_TRY(nccl().GroupEnd());
  if (!even) {
    CUDA_TRY(cudaMemcpyAsync(neighbors, fin_i, size_t(nq_) * k_ * 8, cudaMemcpyDeviceToDevice, res.stream));
    CUDA_TRY(cudaMemcpyAsync(distances, fin_d, size_t(nq_) * k_ * 4, cudaMemcpyDeviceToDevice, res.stream));
  }
}

void search_rank(raft::resources& res, rank_comm& comm, const ivf_pq::search_params& params,
                 const index<int64_t>& shard, const void* queries, elem_t qtype, uint32_t nq, uint32_t k,
                 int64_t* neighbors, float* distances)
{
  if (nq == 0) { return; }
  if (comm.n_ranks() == 1) {
    ivf_pq::search_any(res, params, shard, queries, qtype, nq, k, neighbors, distances);
    return;
  }
  comm.mark(res, 0);
  comm.select(res, params, shard, queries, qtype, nq, k);
  comm.mark(res, 1);
  comm.gather_probes(res.stream);
  comm.mark(res, 2);
  comm.scan(res, params, shard, queries, qtype, /*exchange_bounds=*/true);
  comm.mark(res, 3);
  if (comm.merge_by_slice()) {
    comm.exchange_slices(res.stream);
    comm.mark(res, 4);
    comm.merge_slice_and_gather(res, is_min_close(shard.metric()), neighbors, distances);
  } else {
    comm.gather_results(res.stream);
    comm.mark(res, 4);
    comm.merge(res, is_min_close(shard.metric()), neighbors, distances);
  }
  comm.mark(res, 5);
}

// ------------------------------------------------------------------------------------------------
// one process, all GPUs
// ------------------------------------------------------------------------------------------------
snmg_resources::snmg_resources(const std::vector<int>& device_ids)
{
  kind = 1;
  devices = device_ids;
  if (devices.empty()) {
    int n = 0;
    CUDA_TRY(cudaGetDeviceCount(&n));
    for (int d = 0; d < n; d++) { devices.push_back(d); }
  }
  CUVS_EXPECTS(!devices.empty(), "no CUDA device");
  const int n = int(devices.size());
  raw_comms.assign(size_t(n), nullptr);
  if (n > 1) {
    std::vector<ncclComm_t> c(size_t(n), nullptr);
    NCCL_TRY(nccl().CommInitAll(c.data(), n, devices.data()));
    for (int r = 0; r < n; r++) { raw_comms[size_t(r)] = c[size_t(r)]; }
  }
  for (int r = 0; r < n; r++) {
    device_guard g(devices[size_t(r)]);
    rank_res.emplace_back(new cuvs_b200::resources());
    cudaStream_t s = nullptr;
    CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    streams.push_back(s);
    rank_res.back()->stream = s;
    comms.emplace_back(new rank_comm(raw_comms[size_t(r)], r, n));
  }
}

snmg_resources::~snmg_resources()
{
  for (size_t r = 0; r < devices.size(); r++) {
    cudaSetDevice(devices[r]);
    if (r < streams.size() && streams[r]) { cudaStreamSynchronize(streams[r]); }
  }
  comms.clear();
  for (size_t r = 0; r < raw_comms.size(); r++) {
    if (raw_comms[r]) { nccl().CommDestroy(raw_comms[r]); }
  }
  for (size_t r = 0; r < devices.size(); r++) {
    cudaSetDevice(devices[r]);
    rank_res[r].reset();
    if (r < streams.size() && streams[r]) { cudaStreamDestroy(streams[r]); }
  }
  cudaSetDevice(device);
}

int64_t mg_index::size() const
{
  if (parts.empty()) { return 0; }
  if (mode == distribution_mode::REPLICATED) { return parts[0]->size(); }
  int64_t n = 0;
  for (auto& p : parts) { n += p->size(); }
  return n;
}

namespace {

// one index stream in host memory -> an index per rank (rank r keeps the lists it owns when `by_list`)
void deal_out(snmg_resources& clique, std::istream& is, bool by_list, mg_index* out)
{
  const int n = clique.n_ranks();
  out->parts.clear();
  for (int r = 0; r < n; r++) {
    device_guard g(clique.devices[size_t(r)]);
    is.clear();
    is.seekg(0);
    out->parts.emplace_back(new index<int64_t>());
    ivf_pq::deserialize(*clique.rank_res[size_t(r)], is, out->parts.back().get(), by_list ? r : 0, by_list ? n : 1);
  }
  out->id_offsets.assign(size_t(n), 0);
}

void sync_all(snmg_resources& clique)
{
  for (int r = 0; r < clique.n_ranks(); r++) {
    device_guard g(clique.devices[size_t(r)]);
    clique.rank_res[size_t(r)]->sync();
  }
}

}  // namespace

void build(snmg_resources& clique, const ivf_pq::index_params& params, distribution_mode mode,
           const void* dataset, elem_t dtype, int64_t n_rows, uint32_t dim, mg_index* out)
{
  // One global index is built on the root rank (so that every rank shares one coarse model and the
  // merged result equals a single-GPU search), written to a memory stream and dealt out.
  std::stringstream ss(std::ios::in | std::ios::out | std::ios::binary);
  {
    device_guard g(clique.devices[0]);
    index<int64_t> global;
    ivf_pq::build_any(*clique.rank_res[0], params, dataset, dtype, n_rows, dim, false, &global);
    clique.rank_res[0]->sync();
    ivf_pq::serialize(*clique.rank_res[0], ss, global);
  }
  out->mode = mode;
  out->kind = shard_kind::BY_LIST;
  deal_out(clique, ss, mode == distribution_mode::SHARDED, out);
}

void distribute(snmg_resources& clique, const std::string& filename, mg_index* out)
{
  std::ifstream is(filename, std::ios::in | std::ios::binary);
  CUVS_EXPECTS(bool(is), "Cannot open file %s", filename.c_str());
  out->mode = distribution_mode::REPLICATED;
  out->kind = shard_kind::BY_LIST;
  deal_out(clique, is, false, out);
}

void distribute_by_list(snmg_resources& clique, const std::string& filename, mg_index* out)
{
  std::ifstream is(filename, std::ios::in | std::ios::binary);
  CUVS_EXPECTS(bool(is), "Cannot open file %s", filename.c_str());
  out->mode = distribution_mode::SHARDED;
  out->kind = shard_kind::BY_LIST;
  deal_out(clique, is, true, out);
}

void deserialize(snmg_resources& clique, const std::string& filename, mg_index* out)
{
  const int n = clique.n_ranks();
  out->parts.clear();
  out->id_offsets.assign(size_t(n), 0);
  int mode = 0;
  for (int r = 0; r < n; r++) {
    device_guard g(clique.devices[size_t(r)]);
    out->parts.emplace_back(new index<int64_t>());
    int64_t off = 0;
    ivf_pq::deserialize_mg_rank(*clique.rank_res[size_t(r)], filename, r, n, out->parts.back().get(), &mode, &off);
    out->id_offsets[size_t(r)] = off;
  }
  out->mode = distribution_mode(mode);
  out->kind = shard_kind::BY_ROWS;
}

void serialize(snmg_resources& clique, const mg_index& idx, const std::string& filename, const char* dtype_string)
{
  const int n = clique.n_ranks();
  CUVS_EXPECTS(int(idx.parts.size()) == n, "the index was made for %zu ranks, the clique has %d", idx.parts.size(), n);
  std::vector<raft::resources*> res;
  std::vector<const index<int64_t>*> parts;
  for (int r = 0; r < n; r++) {
    res.push_back(clique.rank_res[size_t(r)].get());
    parts.push_back(idx.parts[size_t(r)].get());
  }
  std::ofstream of(filename, std::ios::out | std::ios::binary);
  CUVS_EXPECTS(bool(of), "Cannot open file %s", filename.c_str());
  const bool merged = idx.mode == distribution_mode::SHARDED && idx.kind == shard_kind::BY_LIST;
  ivf_pq::serialize_mg_header(of, dtype_string, merged ? int(distribution_mode::REPLICATED) : int(idx.mode), n);
  for (int r = 0; r < n; r++) {
    if (merged) {
      // a list-sharded index has no counterpart in the reference's file format (its SHARDED files hold
      // independent per-rank indexes with local ids): written as a REPLICATED file, the whole index once
      // per rank, which the reference loads and searches as such
      ivf_pq::serialize_list_sharded(res, of, parts);
    } else {
      device_guard g(clique.devices[size_t(r)]);
      ivf_pq::serialize(*res[size_t(r)], of, *parts[size_t(r)]);
    }
  }
  of.close();
  CUVS_EXPECTS(bool(of), "Error writing output %s", filename.c_str());
}

void extend(snmg_resources& clique, mg_index* idx, const void* new_vectors, elem_t dtype, int64_t n_rows,
            const int64_t* new_indices)
{
  const int n = clique.n_ranks();
  CUVS_EXPECTS(int(idx->parts.size()) == n, "the index was made for %zu ranks, the clique has %d", idx->parts.size(), n);
  if (n_rows == 0) { return; }
  const uint32_t dim  = idx->parts[0]->dim();
  const size_t row_b  = size_t(dim) * elem_size(dtype);
  const char* vectors = static_cast<const char*>(new_vectors);
  if (idx->mode == distribution_mode::REPLICATED) {
    for (int r = 0; r < n; r++) {
      device_guard g(clique.devices[size_t(r)]);
      ivf_pq::extend_any(*clique.rank_res[size_t(r)], vectors, dtype, n_rows, new_indices, false, idx->parts[size_t(r)].get());
    }
    return;
  }
  if (idx->kind == shard_kind::BY_ROWS) {
    // snmg.cuh:196-246: consecutive slices of the new rows go to consecutive ranks
    const int64_t per = ceildiv<int64_t>(n_rows, n);
    for (int r = 0; r < n; r++) {
      const int64_t off = int64_t(r) * per, cnt = std::min<int64_t>(per, n_rows - off);
      if (cnt <= 0) { continue; }
      device_guard g(clique.devices[size_t(r)]);
      ivf_pq::extend_any(*clique.rank_res[size_t(r)], vectors + size_t(off) * row_b, dtype, cnt,
                         new_indices ? new_indices + off : nullptr, false, idx->parts[size_t(r)].get());
    }
    int64_t acc = 0;
    for (int r = 0; r < n; r++) {
      idx->id_offsets[size_t(r)] = acc;
      acc += idx->parts[size_t(r)]->size();
    }
    return;
  }
  // by list: label every new row with the shared coarse model, then each rank takes the rows of its lists
  std::vector<uint32_t> labels(size_t(n_rows), 0);
  {
    device_guard g(clique.devices[0]);
    auto& res = *clique.rank_res[0];
    const size_t nr = size_t(n_rows);
    ivf_pq::dev_array<uint8_t> d_x(nr * row_b);
    ivf_pq::dev_array<uint32_t> d_l(nr);
    const size_t code_b = size_t(ceildiv<uint32_t>(idx->parts[0]->pq_dim() * idx->parts[0]->pq_bits(), 8));
    ivf_pq::dev_array<uint8_t> d_c(nr * code_b);
    CUDA_TRY(cudaMemcpyAsync(d_x.data(), vectors, size_t(n_rows) * row_b, cudaMemcpyHostToDevice, res.stream));
    ivf_pq::transform_any(res, *idx->parts[0], d_x.data(), dtype, n_rows, d_l.data(), d_c.data());
    CUDA_TRY(cudaMemcpyAsync(labels.data(), d_l.data(), size_t(n_rows) * 4, cudaMemcpyDeviceToHost, res.stream));
    res.sync();
  }
  // the owner of a list is the rank that already holds it; a list empty everywhere goes by the rule
  // of the loader applied to the current global sizes
  const uint32_t n_lists = idx->parts[0]->n_lists();
  std::vector<uint32_t> global_sizes(n_lists, 0);
  std::vector<int> owner(n_lists, -1);
  for (int r = 0; r < n; r++) {
    const auto& hs = idx->parts[size_t(r)]->host_list_sizes();
    for (uint32_t l = 0; l < n_lists; l++) {
      if (hs[l] > 0) {
        owner[l] = r;
        global_sizes[l] = hs[l];
      }
    }
  }
  const std::vector<int> by_rule = ivf_pq::list_owners(global_sizes, n);
  for (uint32_t l = 0; l < n_lists; l++) {
    if (owner[l] < 0) { owner[l] = by_rule[l]; }
  }
  const int64_t base_id = idx->size();
  for (int r = 0; r < n; r++) {
    std::vector<char> rows;
    std::vector<int64_t> ids;
    for (int64_t i = 0; i < n_rows; i++) {
      if (owner[labels[size_t(i)]] != r) { continue; }
      rows.insert(rows.end(), vectors + size_t(i) * row_b, vectors + size_t(i + 1) * row_b);
      ids.push_back(new_indices ? new_indices[i] : base_id + i);
    }
    if (ids.empty()) { continue; }
    device_guard g(clique.devices[size_t(r)]);
    ivf_pq::extend_any(*clique.rank_res[size_t(r)], rows.data(), dtype, int64_t(ids.size()), ids.data(), false,
                       idx->parts[size_t(r)].get());
  }
}

void search(snmg_resources& clique, const mg_index& idx, const search_params& params, const void* queries,
            elem_t qtype, int64_t n_queries, uint32_t k, int64_t* neighbors, float* distances)
{
  const int n = clique.n_ranks();
  CUVS_EXPECTS(int(idx.parts.size()) == n, "the index was made for %zu ranks, the clique has %d", idx.parts.size(), n);
  CUVS_EXPECTS(params.n_rows_per_batch > 0, "n_rows_per_batch must be positive");
  if (n_queries == 0) { return; }
  const uint32_t dim = idx.parts[0]->dim();
  const size_t row_b = size_t(dim) * elem_size(qtype);
  const char* q      = static_cast<const char*>(queries);
  const ivf_pq::search_params& base = params;
  const bool select_min = is_min_close(idx.parts[0]->metric());
  auto& nc = nccl();

  if (idx.mode == distribution_mode::REPLICATED) {
    // snmg.cuh:563-700: the batch is divided between the ranks (LOAD_BALANCER: every batch in n slices;
    // ROUND_ROBIN: whole batches in turn); results go straight to their place in the host arrays
    int64_t batch_no = 0;
    for (int64_t b0 = 0; b0 < n_queries; b0 += params.n_rows_per_batch, batch_no++) {
      const int64_t nb = std::min<int64_t>(params.n_rows_per_batch, n_queries - b0);
      for (int r = 0; r < n; r++) {
        int64_t lo, cnt;
        if (params.search_mode == replicated_search_mode::LOAD_BALANCER) {
          const int64_t per = ceildiv<int64_t>(nb, n);
          lo  = std::min<int64_t>(nb, int64_t(r) * per);
          cnt = std::min<int64_t>(per, nb - lo);
        } else {
          lo  = 0;
          cnt = (batch_no % n) == r ? nb : 0;
        }
        if (cnt <= 0) { continue; }
        device_guard g(clique.devices[size_t(r)]);
        auto& res = *clique.rank_res[size_t(r)];
        auto& c   = *clique.comms[size_t(r)];
        void* dq  = c.query_buffer(size_t(cnt) * row_b);
        float* dd = c.out_distances(size_t(cnt) * k);
        int64_t* di = c.out_neighbors(size_t(cnt) * k);
        CUDA_TRY(cudaMemcpyAsync(dq, q + size_t(b0 + lo) * row_b, size_t(cnt) * row_b, cudaMemcpyHostToDevice, res.stream));
        ivf_pq::search_any(res, base, *idx.parts[size_t(r)], dq, qtype, uint32_t(cnt), k, di, dd);
        CUDA_TRY(cudaMemcpyAsync(neighbors + size_t(b0 + lo) * k, di, size_t(cnt) * k * 8, cudaMemcpyDeviceToHost, res.stream));
        CUDA_TRY(cudaMemcpyAsync(distances + size_t(b0 + lo) * k, dd, size_t(cnt) * k * 4, cudaMemcpyDeviceToHost, res.stream));
      }
      sync_all(clique);
    }
    return;
  }

  for (int64_t b0 = 0; b0 < n_queries; b0 += params.n_rows_per_batch) {
    const uint32_t nb = uint32_t(std::min<int64_t>(params.n_rows_per_batch, n_queries - b0));
    std::vector<void*> dq(size_t(n), nullptr);
    // every rank needs the whole batch
    for (int r = 0; r < n; r++) {
      device_guard g(clique.devices[size_t(r)]);
      auto& res = *clique.rank_res[size_t(r)];
      dq[size_t(r)] = clique.comms[size_t(r)]->query_buffer(size_t(nb) * row_b);
      CUDA_TRY(cudaMemcpyAsync(dq[size_t(r)], q + size_t(b0) * row_b, size_t(nb) * row_b, cudaMemcpyHostToDevice, res.stream));
    }
    if (idx.kind == shard_kind::BY_LIST) {
      for (int r = 0; r < n; r++) {
        device_guard g(clique.devices[size_t(r)]);
        clique.comms[size_t(r)]->select(*clique.rank_res[size_t(r)], base, *idx.parts[size_t(r)], dq[size_t(r)], qtype, nb, k);
      }
      if (n > 1) {
        NCCL_TRY(nc.GroupStart());
        for (int r = 0; r < n; r++) { clique.comms[size_t(r)]->gather_probes(clique.streams[size_t(r)]); }
        NCCL_TRY(nc.GroupEnd());
      }
      for (int r = 0; r < n; r++) {
        device_guard g(clique.devices[size_t(r)]);
        clique.comms[size_t(r)]->scan(*clique.rank_res[size_t(r)], base, *idx.parts[size_t(r)], dq[size_t(r)], qtype);
      }
    } else {
      // snmg.cuh:249-404: every rank searches its rows for the whole batch; local ids become global
      for (int r = 0; r < n; r++) {
        device_guard g(clique.devices[size_t(r)]);
        clique.comms[size_t(r)]->search_rows(*clique.rank_res[size_t(r)], base, *idx.parts[size_t(r)], dq[size_t(r)], qtype,
                                             nb, k, idx.id_offsets[size_t(r)]);
      }
    }
    if (n > 1) {
      NCCL_TRY(nc.GroupStart());
      for (int r = 0; r < n; r++) { clique.comms[size_t(r)]->gather_results(clique.streams[size_t(r)]); }
      NCCL_TRY(nc.GroupEnd());
    }
    {
      // the root rank merges and returns the batch
      device_guard g(clique.devices[0]);
      auto& res = *clique.rank_res[0];
      auto& c   = *clique.comms[0];
      float* dd = c.out_distances(size_t(nb) * k);
      int64_t* di = c.out_neighbors(size_t(nb) * k);
      c.merge(res, select_min, di, dd);
      CUDA_TRY(cudaMemcpyAsync(neighbors + size_t(b0) * k, di, size_t(nb) * k * 8, cudaMemcpyDeviceToHost, res.stream));
      CUDA_TRY(cudaMemcpyAsync(distances + size_t(b0) * k, dd, size_t(nb) * k * 4, cudaMemcpyDeviceToHost, res.stream));
    }
    sync_all(clique);
  }
}

}  // namespace cuvs::neighbors::mg

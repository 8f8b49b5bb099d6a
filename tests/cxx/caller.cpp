// A C++ caller of the library compiled against the public header alone, the way the reference's
// benchmark wrapper uses the reference (cpp/bench/ann/src/cuvs/cuvs_ivf_pq_wrapper.h:120-235: build from
// a dataset view, search with device views, save and load by file name).  It builds an index from a
// HOST dataset, extends it, searches with and without a bitset filter, writes the index to a file,
// reads it back and checks that the search of the reloaded index returns the same bits.
// Prints "CALLER_OK" and exits 0 on success.
#include <cuvs/neighbors/ivf_pq.hpp>

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>

namespace ivf_pq = cuvs::neighbors::ivf_pq;

#define CHECK(cond)                                               \
  do {                                                            \
    if (!(cond)) {                                                \
      std::fprintf(stderr, "check failed: %s (line %d)\n", #cond, __LINE__); \
      return 1;                                                   \
    }                                                             \
  } while (0)

int main(int argc, char** argv)
{
  const std::string path = argc > 1 ? argv[1] : "/tmp/caller_index.ivfpq";
  const int64_t n = 6000, n_more = 1000, dim = 32, nq = 50, k = 10;
  std::mt19937 rng(7);
  std::normal_distribution<float> g(0.0f, 1.0f);
  std::vector<float> x(size_t(n + n_more) * dim), q(size_t(nq) * dim);
  for (auto& v : x) { v = g(rng); }
  for (int64_t i = 0; i < nq; i++) {
    for (int64_t d = 0; d < dim; d++) { q[size_t(i) * dim + d] = x[size_t(i * 7) * dim + d] + 0.01f * g(rng); }
  }

  raft::resources res;
  ivf_pq::index_params ip;
  ip.n_lists        = 32;
  ip.pq_dim         = 16;
  ip.kmeans_n_iters = 5;
  auto index = ivf_pq::build(res, ip, raft::make_host_matrix_view<const float, int64_t>(x.data(), n, dim));
  CHECK(index.size() == n && index.dim() == dim && index.pq_dim() == 16 && index.n_lists() == 32);
  // a non-empty index wants the ids of the new rows (ivf_pq_build.cuh: "You must pass data indices
  // when the index is non-empty.")
  std::vector<int64_t> more_ids(size_t(n_more), 0);
  for (int64_t i = 0; i < n_more; i++) { more_ids[size_t(i)] = n + i; }
  ivf_pq::extend(res, raft::make_host_matrix_view<const float, int64_t>(x.data() + size_t(n) * dim, n_more, dim),
                 more_ids.data(), &index);
  CHECK(index.size() == n + n_more);

  float *d_q = nullptr, *d_dist = nullptr;
  int64_t* d_nb = nullptr;
  uint32_t* d_bits = nullptr;
  CHECK(cudaMalloc(&d_q, q.size() * 4) == cudaSuccess);
  CHECK(cudaMalloc(&d_dist, size_t(nq) * k * 4) == cudaSuccess);
  CHECK(cudaMalloc(&d_nb, size_t(nq) * k * 8) == cudaSuccess);
  CHECK(cudaMemcpy(d_q, q.data(), q.size() * 4, cudaMemcpyHostToDevice) == cudaSuccess);
  auto queries   = raft::make_device_matrix_view<const float, int64_t>(d_q, nq, dim);
  auto neighbors = raft::make_device_matrix_view<int64_t, int64_t>(d_nb, nq, k);
  auto distances = raft::make_device_matrix_view<float, int64_t>(d_dist, nq, k);

  ivf_pq::search_params sp;
  sp.n_probes = 8;
  ivf_pq::search(res, sp, index, queries, neighbors, distances);
  res.sync();
  std::vector<int64_t> nb(size_t(nq) * k), nb2(nb.size());
  std::vector<float> dist(size_t(nq) * k), dist2(dist.size());
  CHECK(cudaMemcpy(nb.data(), d_nb, nb.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess);
  CHECK(cudaMemcpy(dist.data(), d_dist, dist.size() * 4, cudaMemcpyDeviceToHost) == cudaSuccess);
  int hits = 0;
  for (int64_t i = 0; i < nq; i++) {
    for (int64_t j = 0; j < k; j++) { hits += nb[size_t(i) * k + j] == i * 7; }
  }
  CHECK(hits >= nq * 8 / 10);  // a query is a slightly perturbed database vector

  // the same with a bitset filter that forbids every even id
  std::vector<uint32_t> bits((n + n_more + 31) / 32, 0xAAAAAAAAu);
  CHECK(cudaMalloc(&d_bits, bits.size() * 4) == cudaSuccess);
  CHECK(cudaMemcpy(d_bits, bits.data(), bits.size() * 4, cudaMemcpyHostToDevice) == cudaSuccess);
  cuvs::neighbors::filtering::bitset_filter<uint32_t, int64_t> filter(d_bits, uint64_t(n + n_more));
  ivf_pq::search(res, sp, index, queries, neighbors, distances, filter);
  res.sync();
  CHECK(cudaMemcpy(nb2.data(), d_nb, nb2.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess);
  for (auto id : nb2) { CHECK(id == ivf_pq::kOutOfBoundsRecord || (id & 1) == 1); }
  ivf_pq::search(res, sp, index, queries, neighbors, distances, cuvs::neighbors::filtering::none_sample_filter{});
  res.sync();
  CHECK(cudaMemcpy(nb2.data(), d_nb, nb2.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess);
  CHECK(nb2 == nb);

  // file round trip
  ivf_pq::serialize(res, path, index);
  ivf_pq::index<int64_t> back;
  ivf_pq::deserialize(res, path, &back);
  CHECK(back.size() == index.size());
  ivf_pq::search(res, sp, back, queries, neighbors, distances);
  res.sync();
  CHECK(cudaMemcpy(nb2.data(), d_nb, nb2.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess);
  CHECK(cudaMemcpy(dist2.data(), d_dist, dist2.size() * 4, cudaMemcpyDeviceToHost) == cudaSuccess);
  CHECK(nb2 == nb && dist2 == dist);

  // errors surface as exceptions with the reference's messages
  bool threw = false;
  try {
    sp.n_probes = 0;
    ivf_pq::search(res, sp, index, queries, neighbors, distances);
  } catch (const std::exception& e) {
    threw = std::string(e.what()).find("n_probes") != std::string::npos;
  }
  CHECK(threw);
  cudaFree(d_q);
  cudaFree(d_dist);
  cudaFree(d_nb);
  cudaFree(d_bits);
  std::printf("CALLER_OK\n");
  return 0;
}

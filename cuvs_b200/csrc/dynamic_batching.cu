// See dynamic_batching.hpp.
#include "dynamic_batching.hpp"

#include <chrono>
#include <condition_variable>
#include <mutex>
#include <string>
#include <vector>

namespace cuvs::neighbors::dynamic_batching {

using namespace cuvs_b200;

namespace detail {

class batch_runner {
 public:
  batch_runner(const index_params& params, const ivf_pq::index<int64_t>& upstream,
               const ivf_pq::search_params& upstream_params)
    : upstream_(upstream), sp_(upstream_params), k_(uint32_t(params.k)),
      max_batch_(uint32_t(params.max_batch_size)), dim_(upstream.dim())
  {
    CUVS_EXPECTS(params.k > 0, "dynamic batching: k must be positive");
    CUVS_EXPECTS(params.max_batch_size > 0, "dynamic batching: max_batch_size must be positive");
    CUVS_EXPECTS(params.n_queues > 0, "dynamic batching: n_queues must be positive");
    sp_.max_internal_batch_size = std::max<uint32_t>(sp_.max_internal_batch_size, max_batch_);
    {
      // everything the upstream search would refuse about its parameters is refused here, once,
      // instead of on the dispatcher thread of some later batch
      raft::resources probe;
      ivf_pq::check_search_params(probe, sp_, upstream_, k_);
    }
    queues_.resize(params.n_queues);
    for (auto& q : queues_) {
      q.res = std::make_unique<raft::resources>();
      CUDA_TRY(cudaStreamCreateWithFlags(&q.stream, cudaStreamNonBlocking));
      q.res->stream = q.stream;
      CUDA_TRY(cudaMalloc(&q.d_queries, size_t(max_batch_) * dim_ * sizeof(float)));
      CUDA_TRY(cudaMalloc(&q.d_neighbors, size_t(max_batch_) * k_ * sizeof(int64_t)));
      CUDA_TRY(cudaMalloc(&q.d_distances, size_t(max_batch_) * k_ * sizeof(float)));
    }
  }
  ~batch_runner()
  {
    for (auto& q : queues_) {
      if (q.stream) { cudaStreamSynchronize(q.stream); }
      for (auto ev : q.in_events) { cudaEventDestroy(ev); }
      for (auto ev : q.out_events) { cudaEventDestroy(ev); }
      if (q.done) { cudaEventDestroy(q.done); }
      cudaFree(q.d_queries);
      cudaFree(q.d_neighbors);
      cudaFree(q.d_distances);
      q.res.reset();
      if (q.stream) { cudaStreamDestroy(q.stream); }
    }
  }

  void search(raft::resources& res, double timeout_ms, const float* queries, uint32_t n,
              int64_t* neighbors, float* distances)
  {
    for (uint32_t r0 = 0; r0 < n; r0 += max_batch_) {
      const uint32_t rows = std::min(max_batch_, n - r0);
      submit(res, timeout_ms, queries + size_t(r0) * dim_, rows, neighbors + size_t(r0) * k_,
             distances + size_t(r0) * k_);
    }
  }

  uint64_t n_batches = 0, n_rows = 0;  // guarded by m_
  // test hook (host side): the next upstream search throws instead of running
  void fail_next()
  {
    std::lock_guard<std::mutex> lk(m_);
    fail_next_ = true;
  }
  uint32_t k() const { return k_; }
  uint32_t dim() const { return dim_; }

 private:
  enum class state { idle, open, closed, done };
  struct queue {
    std::unique_ptr<raft::resources> res;
    cudaStream_t stream   = nullptr;
    float* d_queries      = nullptr;
    int64_t* d_neighbors  = nullptr;
    float* d_distances    = nullptr;
    // everything below is guarded by the runner's mutex
    state st              = state::idle;
    uint32_t rows         = 0;   // rows reserved in the open batch
    uint32_t writers      = 0;   // contributors that have not yet recorded their input copy
    uint32_t readers      = 0;   // contributors that have not yet enqueued their result copy
    uint64_t generation   = 0;
    std::chrono::steady_clock::time_point deadline;
    std::vector<cudaEvent_t> in_events;   // input copies of the open batch
    std::vector<cudaEvent_t> out_events;  // result copies of the previous batch
    cudaEvent_t done      = nullptr;      // upstream search of the last batch (also guards d_queries)
    std::string error;                    // why the batch in flight failed (empty = it has not)
  };

  static cudaEvent_t new_event()
  {
    cudaEvent_t ev;
    CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    return ev;
  }

  void submit(raft::resources& res, double timeout_ms, const float* queries, uint32_t rows,
              int64_t* neighbors, float* distances)
  {
    std::unique_lock<std::mutex> lk(m_);
    // ---- join an open batch with room, else open one on an idle queue, else wait ----
    queue* q = nullptr;
    for (;;) {
      for (auto& c : queues_) {
        if (c.st == state::open && c.rows + rows <= max_batch_) {
          q = &c;
          break;
        }
      }
      if (!q) {
        for (auto& c : queues_) {
          if (c.st == state::idle) {
            q           = &c;
            q->st       = state::open;
            q->rows     = 0;
            q->deadline = std::chrono::steady_clock::now() +
                          std::chrono::microseconds(int64_t(std::max(0.0, timeout_ms) * 1000.0));
            break;
          }
        }
      }
      if (q) { break; }
      cv_.wait(lk);
    }
    const uint32_t offset   = q->rows;
    const bool dispatcher   = offset == 0;
    const uint64_t my_gen   = q->generation;
    cudaEvent_t prev_done   = q->done;  // the previous upstream search on this queue read d_queries
    q->rows += rows;
    q->writers++;
    q->readers++;
    if (q->rows == max_batch_) { cv_.notify_all(); }  // wakes the dispatcher of a full batch
    lk.unlock();

    // ---- this request's rows into the queue's input buffer, on the caller's stream ----
    // From here on an exception must not leave the queue's counters behind: a failure (of this
    // request's copies, or of the upstream search on the dispatcher) is recorded in the queue, the
    // protocol runs to its end so that nobody waits for a count that never arrives, and every
    // request of the failed batch reports the error.
    std::string my_error;
    cudaEvent_t in_ev = nullptr;
    try {
      if (prev_done) { CUDA_TRY(cudaStreamWaitEvent(res.stream, prev_done, 0)); }
      CUDA_TRY(cudaMemcpyAsync(q->d_queries + size_t(offset) * dim_, queries, size_t(rows) * dim_ * sizeof(float),
                               cudaMemcpyDeviceToDevice, res.stream));
      in_ev = new_event();
      CUDA_TRY(cudaEventRecord(in_ev, res.stream));
    } catch (const std::exception& e) {
      my_error = e.what();
      cudaGetLastError();
    }

    lk.lock();
    if (in_ev) { q->in_events.push_back(in_ev); }
    if (!my_error.empty() && q->error.empty()) { q->error = my_error; }
    q->writers--;
    cv_.notify_all();
    if (dispatcher) {
      // ---- close the batch when it is full or its time is up, then launch the upstream search ----
      cv_.wait_until(lk, q->deadline, [&] { return q->rows == max_batch_; });
      q->st = state::closed;
      cv_.wait(lk, [&] { return q->writers == 0; });
      const uint32_t n_rows_batch = q->rows;
      std::vector<cudaEvent_t> wait_for;
      wait_for.swap(q->in_events);
      std::vector<cudaEvent_t> prev_out;
      prev_out.swap(q->out_events);
      cudaEvent_t old_done = q->done;
      std::string err      = q->error;
      if (fail_next_ && err.empty()) {
        err        = "upstream search failed (injected by the test hook)";
        fail_next_ = false;
      }
      lk.unlock();
      cudaEvent_t done = nullptr;
      try {
        for (auto ev : prev_out) {  // results of the previous batch have left the output buffers
          CUDA_TRY(cudaStreamWaitEvent(q->stream, ev, 0));
        }
        for (auto ev : wait_for) { CUDA_TRY(cudaStreamWaitEvent(q->stream, ev, 0)); }
        if (err.empty()) {
          ivf_pq::search_any(*q->res, sp_, upstream_, q->d_queries, ivf_pq::elem_t::f32, n_rows_batch, k_,
                             q->d_neighbors, q->d_distances);
        }
        done = new_event();
        CUDA_TRY(cudaEventRecord(done, q->stream));
      } catch (const std::exception& e) {
        if (err.empty()) { err = e.what(); }
        cudaGetLastError();
      }
      for (auto ev : prev_out) { cudaEventDestroy(ev); }
      for (auto ev : wait_for) { cudaEventDestroy(ev); }
      lk.lock();
      if (done) {
        if (old_done) { cudaEventDestroy(old_done); }
        q->done = done;
      }
      q->error = err;
      q->st    = state::done;
      if (err.empty()) {
        n_batches++;
        n_rows += n_rows_batch;
      }
      cv_.notify_all();
    } else {
      cv_.wait(lk, [&] { return q->generation == my_gen && q->st == state::done; });
    }
    cudaEvent_t done        = q->done;
    std::string batch_error = q->error;
    lk.unlock();

    // ---- this request's rows of the result, on the caller's stream ----
    cudaEvent_t out_ev = nullptr;
    if (batch_error.empty()) {
      try {
        CUDA_TRY(cudaStreamWaitEvent(res.stream, done, 0));
        CUDA_TRY(cudaMemcpyAsync(neighbors, q->d_neighbors + size_t(offset) * k_, size_t(rows) * k_ * sizeof(int64_t),
                                 cudaMemcpyDeviceToDevice, res.stream));
        CUDA_TRY(cudaMemcpyAsync(distances, q->d_distances + size_t(offset) * k_, size_t(rows) * k_ * sizeof(float),
                                 cudaMemcpyDeviceToDevice, res.stream));
        out_ev = new_event();
        CUDA_TRY(cudaEventRecord(out_ev, res.stream));
      } catch (const std::exception& e) {
        batch_error = e.what();
        cudaGetLastError();
      }
    }

    lk.lock();
    if (out_ev) { q->out_events.push_back(out_ev); }
    if (--q->readers == 0) {
      q->st = state::idle;
      q->generation++;
      q->error.clear();
      cv_.notify_all();
    }
    lk.unlock();
    if (!batch_error.empty()) { fail("dynamic batching: the batch of this request failed: %s", batch_error.c_str()); }
  }

  const ivf_pq::index<int64_t>& upstream_;
  ivf_pq::search_params sp_;
  uint32_t k_, max_batch_, dim_;
  std::vector<queue> queues_;
  std::mutex m_;
  std::condition_variable cv_;
  bool fail_next_ = false;
};

}  // namespace detail

template <>
index<float, int64_t>::index(raft::resources&, const index_params& params,
                             const ivf_pq::index<int64_t>& upstream_index,
                             const ivf_pq::search_params& upstream_params)
  : runner(std::make_shared<detail::batch_runner>(params, upstream_index, upstream_params))
{
}

void search(raft::resources& res, const search_params& params, const index<float, int64_t>& idx,
            const float* queries, uint32_t n_queries, int64_t* neighbors, float* distances)
{
  CUVS_EXPECTS(idx.runner != nullptr, "dynamic batching index is not initialised");
  if (n_queries == 0) { return; }
  idx.runner->search(res, params.dispatch_timeout_ms, queries, n_queries, neighbors, distances);
}

void search_checked(raft::resources& res, const search_params& params, const index<float, int64_t>& idx,
                    const float* queries, uint32_t n_queries, uint32_t dim, uint32_t k, int64_t* neighbors,
                    float* distances)
{
  CUVS_EXPECTS(idx.runner != nullptr, "dynamic batching index is not initialised");
  CUVS_EXPECTS(dim == idx.runner->dim(),
               "Number of query dimensions should equal number of dimensions in the index.");
  CUVS_EXPECTS(k == idx.runner->k(), "k is fixed at the construction of a dynamic batching index");
  search(res, params, idx, queries, n_queries, neighbors, distances);
}

void fail_next_upstream_search(const index<float, int64_t>& idx) { idx.runner->fail_next(); }

void stats(const index<float, int64_t>& idx, uint64_t* n_batches, uint64_t* n_rows)
{
  *n_batches = idx.runner->n_batches;
  *n_rows    = idx.runner->n_rows;
}

}  // namespace cuvs::neighbors::dynamic_batching

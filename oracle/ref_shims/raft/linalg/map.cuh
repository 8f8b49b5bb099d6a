// Shim (device build only): the few RAFT pieces the reference's distance post-processing is
// written with, each with the meaning its name states: an element-wise map over a flat view,
// the unary functors mul_const_op (x * c), sqrt_op (square root), cast_op (static_cast) and
// compose_op (compose_op(f, g, h)(x) = f(g(h(x)))), a resources object that carries a stream.
#pragma once
#include <cuda_runtime.h>
#include <cmath>
#include <cstddef>
#include <stdexcept>
#include <tuple>
#include <utility>
#ifndef RAFT_FAIL
#define RAFT_FAIL(msg) throw std::runtime_error(msg)
#endif
namespace rmm {
struct cuda_stream_view {
  cudaStream_t s = nullptr;
  cuda_stream_view() = default;
  cuda_stream_view(cudaStream_t x) : s(x) {}
  operator cudaStream_t() const { return s; }
};
}  // namespace rmm
namespace raft {
struct resources {
  cudaStream_t stream = nullptr;
};
template <typename T>
struct flat_view {
  T* ptr;
  size_t n;
};
template <typename T, typename I = size_t>
flat_view<T> make_device_vector_view(T* p, I n) { return {p, size_t(n)}; }
template <typename T>
flat_view<const T> make_const_mdspan(flat_view<T> v) { return {v.ptr, v.n}; }
template <typename T>
struct mul_const_op {
  T c;
  template <typename X> __host__ __device__ auto operator()(const X& x) const { return x * c; }
};
template <typename T>
struct cast_op {
  template <typename X> __host__ __device__ T operator()(const X& x) const { return static_cast<T>(x); }
};
struct sqrt_op {
  __host__ __device__ float operator()(float x) const { return sqrtf(x); }
};
template <typename... Fs>
struct compose_op;
template <typename F>
struct compose_op<F> {
  F f;
  compose_op(F a) : f(a) {}
  template <typename X> __host__ __device__ auto operator()(const X& x) const { return f(x); }
};
template <typename F, typename... Rest>
struct compose_op<F, Rest...> {
  F f;
  compose_op<Rest...> rest;
  compose_op(F a, Rest... r) : f(a), rest(r...) {}
  template <typename X> __host__ __device__ auto operator()(const X& x) const { return f(rest(x)); }
};
template <typename... Fs>
compose_op(Fs...) -> compose_op<Fs...>;
namespace linalg {
template <typename Out, typename In, typename Op>
__global__ void map_kernel(Out* out, const In* in, size_t n, Op op)
{
  size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (i < n) { out[i] = op(in[i]); }
}
template <typename Out, typename Op, typename In>
void map(const raft::resources& res, flat_view<Out> out, Op op, flat_view<const In> in)
{
  if (out.n == 0) { return; }
  map_kernel<<<unsigned((out.n + 255) / 256), 256, 0, res.stream>>>(out.ptr, in.ptr, out.n, op);
}
}  // namespace linalg
}  // namespace raft

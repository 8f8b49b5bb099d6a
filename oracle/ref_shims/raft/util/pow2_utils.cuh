// Shim: power-of-two helpers with the meaning their names state.
#pragma once
namespace raft {
template <auto V>
struct Pow2 {
  static constexpr auto Value = V;
  template <typename T> static constexpr T div(T x) { return x / V; }
  template <typename T> static constexpr T mod(T x) { return x % V; }
  template <typename T> static constexpr T roundDown(T x) { return x - x % V; }
  template <typename T> static constexpr T roundUp(T x) { return (x + V - 1) / V * V; }
};
}  // namespace raft

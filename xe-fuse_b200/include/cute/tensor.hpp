// Minimal tuple vocabulary of the front end: the names callers of the builder API spell
// (cute::Shape, cute::Stride, cute::Int, cute::_N, make_shape, get<I>).  Shapes and strides are
// plain std::tuples; static extents are std::integral_constant-like empty types.
#pragma once

#include <cstddef>
#include <cstdint>
#include <tuple>
#include <type_traits>
#include <utility>

namespace cute {

template <int N>
struct Int {
  static constexpr int value = N;
  using value_type = int;
  constexpr operator int() const { return N; }
  constexpr int operator()() const { return N; }
};

template <int N> using C = Int<N>;

using _0 = Int<0>;    using _1 = Int<1>;     using _2 = Int<2>;     using _4 = Int<4>;
using _8 = Int<8>;    using _16 = Int<16>;   using _32 = Int<32>;   using _64 = Int<64>;
using _96 = Int<96>;  using _128 = Int<128>; using _192 = Int<192>; using _256 = Int<256>;
using _384 = Int<384>; using _512 = Int<512>; using _1024 = Int<1024>;

template <class... Ts> using tuple = std::tuple<Ts...>;
template <class... Ts> using Shape = std::tuple<Ts...>;
template <class... Ts> using Stride = std::tuple<Ts...>;
template <class... Ts> using Coord = std::tuple<Ts...>;

using std::get;

template <class... Ts>
constexpr Shape<std::decay_t<Ts>...> make_shape(Ts&&... ts) {
  return Shape<std::decay_t<Ts>...>(std::forward<Ts>(ts)...);
}
template <class... Ts>
constexpr Stride<std::decay_t<Ts>...> make_stride(Ts&&... ts) {
  return Stride<std::decay_t<Ts>...>(std::forward<Ts>(ts)...);
}
template <class... Ts>
constexpr tuple<std::decay_t<Ts>...> make_tuple(Ts&&... ts) {
  return tuple<std::decay_t<Ts>...>(std::forward<Ts>(ts)...);
}

template <class T> struct is_static : std::false_type {};
template <int N> struct is_static<Int<N>> : std::true_type {};

// Extent I of a shape as a run-time integer (static or dynamic mode alike).
template <std::size_t I, class Tuple>
constexpr std::int64_t size(Tuple const& t) {
  return static_cast<std::int64_t>(std::get<I>(t));
}

template <class Tuple>
constexpr std::size_t rank(Tuple const&) { return std::tuple_size<Tuple>::value; }

}  // namespace cute

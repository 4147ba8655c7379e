// Stand-in: make_array is only named inside member templates that the oracle never instantiates.
#pragma once
#include <cstddef>
namespace boost { namespace serialization {
template <class T> struct array_stub { T* p; std::size_t n; };
template <class T> array_stub<T> make_array(T* p, std::size_t n) { return array_stub<T>{p, n}; }
}}

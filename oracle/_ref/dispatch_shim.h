// forced-include shim for building the reference against a current torch (see oracle/build_reference.py)
#pragma once
#include <ATen/ATen.h>
namespace detail {
inline c10::ScalarType scalar_type(const at::DeprecatedTypeProperties& t) { return t.scalarType(); }
}

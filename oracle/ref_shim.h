// Force-included in front of the reference's quant_cuda sources when they are compiled, unmodified and
// where they lie, into oracle/_ref/ (see oracle/build_ref.py).  The reference was written against a
// torch whose AT_DISPATCH_* macros accepted `tensor.type()`; the installed torch only accepts a
// ScalarType there.  This overload restores the missing conversion; nothing else is changed.
#pragma once
#include <ATen/ATen.h>
#include <ATen/Dispatch.h>

namespace detail {
inline at::ScalarType scalar_type(const at::DeprecatedTypeProperties& t) { return t.scalarType(); }
}  // namespace detail

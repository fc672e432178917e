// Force-included (nvcc -include) when the reference's CUDA sources are compiled
// from where they lie.  The sources are untouched; the only incompatibility with
// current PyTorch headers is that they pass `tensor.type()` (a
// DeprecatedTypeProperties) to AT_DISPATCH_*, which now resolves the scalar type
// through ::detail::scalar_type(at::ScalarType).  This header restores the
// overload that older PyTorch shipped.  Test infrastructure only.
#pragma once
#include <ATen/ATen.h>
#include <ATen/Dispatch.h>

namespace detail {
inline at::ScalarType scalar_type(const at::DeprecatedTypeProperties& t) { return t.scalarType(); }
}  // namespace detail

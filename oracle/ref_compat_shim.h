// Test infrastructure only.  Force-included (-include) in front of the upstream
// reuse_conv sources so that they compile unmodified against torch >= 2.0:
// upstream passes `tensor.type()` (DeprecatedTypeProperties) to
// AT_DISPATCH_FLOATING_TYPES, which newer torch only accepts as a ScalarType.
#pragma once
#include <torch/extension.h>
namespace rof_ref_compat {
inline at::ScalarType scalar_type_of(at::ScalarType s) { return s; }
inline at::ScalarType scalar_type_of(const at::DeprecatedTypeProperties& t) { return t.scalarType(); }
}  // namespace rof_ref_compat
#undef AT_DISPATCH_FLOATING_TYPES
#define AT_DISPATCH_FLOATING_TYPES(TYPE, NAME, ...) \
  AT_DISPATCH_SWITCH(rof_ref_compat::scalar_type_of(TYPE), NAME, AT_DISPATCH_CASE_FLOATING_TYPES(__VA_ARGS__))

#include "fused_ops.h"

namespace pccl {
void bind_fused_ops(pybind11::module_& m) { (void)m; }
}  // namespace pccl

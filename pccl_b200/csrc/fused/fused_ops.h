// Fused compute + collective operators (tcgen05 / TMEM kernels) and their bindings.
#pragma once
#include <pybind11/pybind11.h>

namespace pccl {
void bind_fused_ops(pybind11::module_& m);
}

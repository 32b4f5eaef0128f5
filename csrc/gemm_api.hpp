// Grouped-GEMM and fused-MoE bindings (implemented in gemm_bindings.cpp).
#pragma once
#include <torch/extension.h>
namespace nep {
void bind_gemm(pybind11::module_& m);
}

// Python bindings of the hybrid-decoder kernels (stream_ops.cu, recurrent.cu, attention_window.cu).
#pragma once
#include <pybind11/pybind11.h>

namespace nrl {
void bind_hybrid(pybind11::module_& m);
}

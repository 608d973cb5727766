#include <torch/extension.h>
namespace py = pybind11;
void bind_gemm(py::module_& m) { (void)m; }

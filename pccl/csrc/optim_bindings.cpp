#include <torch/extension.h>
namespace py = pybind11;
void bind_optim(py::module_& m) { (void)m; }

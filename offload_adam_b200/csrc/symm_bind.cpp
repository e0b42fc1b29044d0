#include <torch/extension.h>
namespace py = pybind11;
void bind_symm(py::module_& m) {}

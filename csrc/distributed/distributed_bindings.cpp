// Python bindings of the native distributed layer (filled in by process_group.cpp).
#include <pybind11/pybind11.h>

namespace py = pybind11;

namespace ob {
void bind_process_group(py::module_& m);
void bind_distributed(py::module_& m) { bind_process_group(m); }
}  // namespace ob

#include <pybind11/pybind11.h>
namespace py = pybind11;
void bind_ckpt(py::module_& m);
void bind_quant(py::module_& m);
void bind_gguf(py::module_& m);
void bind_gai(py::module_& m);
void bind_formats(py::module_& m) {
  bind_ckpt(m);
  bind_quant(m);
  bind_gguf(m);
  bind_gai(m);
}

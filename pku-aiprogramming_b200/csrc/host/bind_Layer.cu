// pybind11 module `myLayer`: the attention operator in the reference's operator style
// (free functions over TinyTensor, outputs passed by reference; cf. src/bind_Layer.cpp:10-24 of
// the reference project).  The GIL is released while the GPU works.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "Layers.h"

namespace py = pybind11;

PYBIND11_MODULE(myLayer, m) {
    m.doc() = "B200 attention operator for TinyTensor";
    py::module::import("myTensor");   // the tensor classes are registered there
    m.def("AttentionForward", &AttentionForward<float>, py::call_guard<py::gil_scoped_release>(), py::arg("q"),
          py::arg("k"), py::arg("v"), py::arg("out"), py::arg("lse"), py::arg("causal") = false,
          py::arg("scale") = 0.0f);
    m.def("AttentionBackward", &AttentionBackward<float>, py::call_guard<py::gil_scoped_release>(), py::arg("q"),
          py::arg("k"), py::arg("v"), py::arg("out"), py::arg("lse"), py::arg("grad_q"), py::arg("grad_k"),
          py::arg("grad_v"), py::arg("grad_out"), py::arg("causal") = false, py::arg("scale") = 0.0f);
    m.def("AttentionForward_bf16", &AttentionForward<__nv_bfloat16>, py::call_guard<py::gil_scoped_release>(),
          py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"), py::arg("lse"), py::arg("causal") = false,
          py::arg("scale") = 0.0f);
    m.def("AttentionBackward_bf16", &AttentionBackward<__nv_bfloat16>, py::call_guard<py::gil_scoped_release>(),
          py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"), py::arg("lse"), py::arg("grad_q"),
          py::arg("grad_k"), py::arg("grad_v"), py::arg("grad_out"), py::arg("causal") = false,
          py::arg("scale") = 0.0f);
    m.def("SoftmaxForward", &SoftmaxForward<float>, py::call_guard<py::gil_scoped_release>());
    m.def("SoftmaxBackward", &SoftmaxBackward<float>, py::call_guard<py::gil_scoped_release>());
    // argument orders of the reference's FcForward / FcBackward (src/bind_Layer.cpp:12-13 there)
    m.def("FcForward", &FcForward<float>, py::call_guard<py::gil_scoped_release>());
    m.def("FcBackward", &FcBackward<float>, py::call_guard<py::gil_scoped_release>());
    m.def("FcForward_bf16", &FcForward<__nv_bfloat16>, py::call_guard<py::gil_scoped_release>());
    m.def("FcBackward_bf16", &FcBackward<__nv_bfloat16>, py::call_guard<py::gil_scoped_release>());
}

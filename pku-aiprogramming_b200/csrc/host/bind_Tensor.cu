// pybind11 module `myTensor`: Tensor_float, Tensor_double, Tensor_int with the reference's
// method list (src/bind_Tensor.cpp:15-45 of the reference project), plus Tensor_bf16.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <sstream>

#include "TinyTensor.h"

namespace py = pybind11;

template <typename T, typename C>
void add_common(C& cls) {
    using Tensor = TinyTensor<T>;
    cls.def(py::init<const std::vector<int>&, const std::string&>())
        .def(py::init<const Tensor&>())
        .def("Size", &Tensor::Size)
        .def("__add__", &Tensor::operator+, py::is_operator())
        .def("__sub__", &Tensor::operator-, py::is_operator())
        .def("__getitem__", [](const Tensor& t, int k) { return t[k]; })
        .def("get_shape", &Tensor::get_shape)
        .def("get_device", &Tensor::get_device)
        .def("flatten", &Tensor::flatten)
        .def("cpu", [](Tensor& t) -> Tensor& { return t.cpu(); }, py::return_value_policy::reference_internal)
        .def("gpu", [](Tensor& t) -> Tensor& { return t.gpu(); }, py::return_value_policy::reference_internal)
        .def("zeros", [](Tensor& t) -> Tensor& { return t.zeros(); }, py::return_value_policy::reference_internal)
        .def("ones", [](Tensor& t) -> Tensor& { return t.ones(); }, py::return_value_policy::reference_internal)
        .def("negative", [](Tensor& t) -> Tensor& { return t.negative(); }, py::return_value_policy::reference_internal)
        .def("floatks", [](Tensor& t, float k) -> Tensor& { return t.floatks(k); },
             py::return_value_policy::reference_internal)
        .def("resize", [](Tensor& t, const std::vector<int>& s) -> Tensor& { return t.resize(s); },
             py::return_value_policy::reference_internal)
        .def("ReluForward", &Tensor::ReluForward)
        .def("ReluBackward", &Tensor::ReluBackward)
        .def("SigmoidForward", &Tensor::SigmoidForward)
        .def("SigmoidBackward", &Tensor::SigmoidBackward)
        // fast path for tests and large tensors: a NumPy float32 array instead of a Python list
        .def("numpy", [](const Tensor& t) {
            std::vector<float> host = t.get_data_f32();
            std::vector<py::ssize_t> shp(t.shape.begin(), t.shape.end());
            py::array_t<float> arr(shp);
            std::copy(host.begin(), host.end(), arr.mutable_data());
            return arr;
        })
        .def("__repr__", [](const Tensor& t) {
            std::ostringstream oss;
            oss << t;
            return oss.str();
        });
}

template <typename T>
void bind_plain(py::module& m, const std::string& category) {
    using Tensor = TinyTensor<T>;
    py::class_<Tensor> cls(m, ("Tensor_" + category).c_str());
    cls.def(py::init<const std::vector<int>&, const std::string&, const std::vector<T>&>())
        .def(py::init<const py::array_t<T>&, const std::string&>())
        .def("get_data", &Tensor::get_data)
        .def("random", [](Tensor& t, T a, T b) -> Tensor& { return t.random(a, b); },
             py::return_value_policy::reference_internal)
        .def("mults", [](Tensor& t, T s) -> Tensor& { return t.mults(s); }, py::return_value_policy::reference_internal);
    add_common<T>(cls);
}

void bind_bf16(py::module& m) {
    using Tensor = TinyTensor<__nv_bfloat16>;
    py::class_<Tensor> cls(m, "Tensor_bf16");
    cls.def(py::init([](const std::vector<int>& shape, const std::string& device, const std::vector<float>& data) {
            return Tensor::from_f32(shape, device, data.data(), data.size());
        }))
        .def(py::init<const py::array_t<float>&, const std::string&>())   // float32 in, rounded to nearest even
        .def("get_data", &Tensor::get_data_f32)                          // floats out (bf16 widened exactly)
        .def("random", [](Tensor& t, float a, float b) -> Tensor& {
                return t.random(__float2bfloat16_rn(a), __float2bfloat16_rn(b));
             }, py::return_value_policy::reference_internal)
        .def("mults", [](Tensor& t, float s) -> Tensor& { return t.mults(__float2bfloat16_rn(s)); },
             py::return_value_policy::reference_internal);
    add_common<__nv_bfloat16>(cls);
}

PYBIND11_MODULE(myTensor, m) {
    m.doc() = "TinyTensor tensors with pooled device storage (float, double, int, bf16)";
    bind_plain<float>(m, "float");
    bind_plain<double>(m, "double");
    bind_plain<int>(m, "int");
    bind_bf16(m);
}

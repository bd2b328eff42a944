// pybind11 module `myTensor`: Tensor_float, Tensor_double, Tensor_int with the reference's
// method list (src/bind_Tensor.cpp:15-45 of the reference project), plus Tensor_bf16.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <ATen/dlpack.h>   // the DLPack ABI structs as shipped with torch (C header, nothing else of torch is used)

#include <cstdint>
#include <cstring>
#include <limits>
#include <sstream>

#include "TinyTensor.h"
#include "tt_attn.h"

namespace py = pybind11;

// ---- DLPack exchange -------------------------------------------------------------------------
// Export (`__dlpack__`, `__dlpack_device__`): zero-copy view of the tensor's buffer for any
// consumer of the protocol (torch.from_dlpack, np.from_dlpack for host tensors).  The capsule
// keeps the Python tensor object alive until the consumer's deleter runs, and retains the BUFFER
// (tt_buffer_retain): if the tensor is resized, moved to the other device, assigned to or used as a
// layer output of another shape meanwhile, its old block stays with the view and goes back to the
// pool only when the view's deleter has run.  Import
// (`from_dlpack`): a deep copy (device to device when the producer's data is on a GPU), because a
// TinyTensor owns its buffer.  The reference has neither; its only way out of a tensor is
// get_data() -> Python list (src/bind_Tensor.cpp:26 of the reference project).
namespace {

template <typename T> DLDataType dl_dtype();
template <> DLDataType dl_dtype<float>() { return DLDataType{kDLFloat, 32, 1}; }
template <> DLDataType dl_dtype<double>() { return DLDataType{kDLFloat, 64, 1}; }
template <> DLDataType dl_dtype<int>() { return DLDataType{kDLInt, 32, 1}; }
template <> DLDataType dl_dtype<__nv_bfloat16>() { return DLDataType{kDLBfloat, 16, 1}; }

struct DlExport {
    py::object owner;                 // keeps the TinyTensor alive
    void* retained = nullptr;         // the buffer the view shows (shared ownership until the deleter runs)
    std::vector<int64_t> shape, strides;
    DLManagedTensor managed;
};

void dl_export_deleter(DLManagedTensor* m) {
    if (!m) return;
    py::gil_scoped_acquire gil;
    auto* ex = static_cast<DlExport*>(m->manager_ctx);
    if (ex->retained) tt_buffer_release(ex->retained);
    delete ex;
}

void dl_capsule_destructor(PyObject* cap) {
    // a consumer renames the capsule to "used_dltensor"; only an unconsumed one is released here
    if (!PyCapsule_IsValid(cap, "dltensor")) return;
    auto* m = static_cast<DLManagedTensor*>(PyCapsule_GetPointer(cap, "dltensor"));
    if (m && m->deleter) m->deleter(m);
}

int device_of_pointer(const void* p) {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error("cudaPointerGetAttributes failed for a device tensor");
    }
    return attr.device;
}

template <typename T>
py::tuple dlpack_device(const TinyTensor<T>& t) {
    if (t.device == "gpu" && t.p_data) return py::make_tuple((int)kDLCUDA, device_of_pointer(t.p_data));
    if (t.device == "gpu") {
        int dev = 0;
        cudaGetDevice(&dev);
        return py::make_tuple((int)kDLCUDA, dev);
    }
    return py::make_tuple((int)kDLCPU, 0);
}

template <typename T>
py::capsule dlpack_export(py::object self, py::object /*stream*/) {
    const auto& t = self.cast<const TinyTensor<T>&>();
    auto* ex = new DlExport();
    ex->owner = self;
    ex->shape.assign(t.shape.begin(), t.shape.end());
    ex->strides.assign(t.shape.size(), 1);
    for (int i = (int)t.shape.size() - 2; i >= 0; --i) ex->strides[i] = ex->strides[i + 1] * std::max<int64_t>(ex->shape[i + 1], 1);
    DLTensor& d = ex->managed.dl_tensor;
    d.data = t.p_data;
    d.ndim = (int32_t)t.shape.size();
    d.dtype = dl_dtype<T>();
    d.shape = ex->shape.data();
    d.strides = ex->strides.data();
    d.byte_offset = 0;
    if (t.device == "gpu") {
        // tensor methods and layer calls run on the legacy default stream; make their results
        // visible to whatever stream the consumer uses
        if (cudaDeviceSynchronize() != cudaSuccess) {
            delete ex;
            throw std::runtime_error("cudaDeviceSynchronize failed before DLPack export");
        }
        int dev = 0;
        if (t.p_data) dev = device_of_pointer(t.p_data); else cudaGetDevice(&dev);
        d.device = DLDevice{kDLCUDA, dev};
    } else {
        d.device = DLDevice{kDLCPU, 0};
    }
    ex->retained = t.p_data;
    tt_buffer_retain(ex->retained);
    ex->managed.manager_ctx = ex;
    ex->managed.deleter = dl_export_deleter;
    return py::capsule(&ex->managed, "dltensor", dl_capsule_destructor);
}

template <typename T>
TinyTensor<T> dlpack_import(py::object src) {
    py::object cap_obj = py::hasattr(src, "__dlpack__") ? src.attr("__dlpack__")() : src;
    PyObject* cap = cap_obj.ptr();
    if (!PyCapsule_IsValid(cap, "dltensor"))
        throw std::invalid_argument("from_dlpack: expected an object with __dlpack__ or an unconsumed 'dltensor' capsule");
    auto* m = static_cast<DLManagedTensor*>(PyCapsule_GetPointer(cap, "dltensor"));
    const DLTensor& d = m->dl_tensor;
    const DLDataType want = dl_dtype<T>();
    auto release = [&]() {
        PyCapsule_SetName(cap, "used_dltensor");
        if (m->deleter) m->deleter(m);
    };
    std::string err;
    if (d.dtype.code != want.code || d.dtype.bits != want.bits || d.dtype.lanes != 1) err = "element type does not match this tensor class";
    const bool on_gpu = d.device.device_type == kDLCUDA || d.device.device_type == kDLCUDAManaged;
    if (!on_gpu && d.device.device_type != kDLCPU && d.device.device_type != kDLCUDAHost) err = "unsupported device type";
    std::vector<int> shape(d.ndim > 0 ? d.ndim : 0);
    int64_t expect = 1;
    for (int i = d.ndim - 1; i >= 0 && err.empty(); --i) {
        if (d.shape[i] < 0 || d.shape[i] > std::numeric_limits<int>::max()) err = "extent does not fit the int shape";
        else if (d.strides && d.shape[i] > 1 && d.strides[i] != expect) err = "only contiguous row-major data can be imported";
        shape[i] = (int)d.shape[i];
        expect *= std::max<int64_t>(d.shape[i], 1);
    }
    if (!err.empty()) {
        release();
        throw std::invalid_argument("from_dlpack: " + err);
    }
    try {
        TinyTensor<T> out(shape, on_gpu ? "gpu" : "cpu");
        if (out.size) {
            const char* from = static_cast<const char*>(d.data) + d.byte_offset;
            if (on_gpu) {
                cudaError_t e = cudaMemcpy(out.p_data, from, out.size * sizeof(T), cudaMemcpyDefault);
                if (e != cudaSuccess)
                    throw std::runtime_error(std::string("from_dlpack: copy failed: ") + cudaGetErrorString(e));
            } else {
                std::memcpy(out.p_data, from, out.size * sizeof(T));
            }
        }
        release();
        return out;
    } catch (...) {
        release();
        throw;
    }
}

}  // namespace

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
        .def("data_ptr", [](const Tensor& t) { return (std::uintptr_t)t.p_data; })
        .def("__dlpack_device__", &dlpack_device<T>)
        .def("__dlpack__", &dlpack_export<T>, py::arg("stream") = py::none())
        .def_static("from_dlpack", &dlpack_import<T>, py::arg("source"))
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

// TinyTensor<T>: the dense row-major tensor class of the TinyTensor mini-framework, rebuilt
// for this library.  Public members and method names follow the reference class
// (src/TinyTensor.h:11-76 of the reference project) so that code written against it
// compiles unchanged; what differs is underneath:
//   - device buffers come from the pooled allocator of libtt_attn (tt_alloc/tt_free) instead of
//     one cudaMalloc/cudaFree per object;
//   - move construction/assignment exist, so returning tensors by value does not deep-copy;
//   - a fourth element type, __nv_bfloat16, is supported (host <-> device conversion is
//     round-to-nearest-even);
//   - every CUDA call is checked and failures throw std::runtime_error.
// Value semantics are the reference's: copies are deep, operator[] and flatten() return
// copies, cpu()/gpu() migrate in place.
#ifndef TT_HOST_TINY_TENSOR_H
#define TT_HOST_TINY_TENSOR_H

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <iostream>
#include <string>
#include <vector>

// Element type NumPy hands over for a tensor of `Type` (bf16 has no NumPy dtype: float32 in,
// rounded to nearest even).
template <typename Type> struct TinyNumpyElem { using type = Type; };
template <> struct TinyNumpyElem<__nv_bfloat16> { using type = float; };

template <typename Type = float>
class TinyTensor {
public:
    std::vector<int> shape;
    std::string device;   // "cpu" or "gpu"
    Type* p_data;
    size_t size;

public:
    TinyTensor(const std::vector<int>& shape, const std::string& device);
    TinyTensor(const std::vector<int>& shape, const std::string& device, const std::vector<Type>& data);
    TinyTensor(const pybind11::array_t<typename TinyNumpyElem<Type>::type>& data, const std::string& device);
    TinyTensor(const TinyTensor<Type>& other);
    TinyTensor(TinyTensor<Type>&& other) noexcept;
    ~TinyTensor();

    size_t Size() const;   // product of `shape`

    TinyTensor<Type>& operator=(const TinyTensor<Type>& other);
    TinyTensor<Type>& operator=(TinyTensor<Type>&& other) noexcept;
    TinyTensor<Type> operator+(const TinyTensor<Type>& other) const;
    TinyTensor<Type> operator-(const TinyTensor<Type>& other) const;
    TinyTensor<Type> operator[](const int index) const;   // copy of slice `index` of the first dim

    std::vector<int> get_shape() const;
    std::string get_device() const;
    std::vector<Type> get_data() const;   // host copy, whatever the device
    TinyTensor<Type> flatten() const;

    TinyTensor<Type>& cpu();
    TinyTensor<Type>& gpu();

    TinyTensor<Type>& random(Type a, Type b);   // uniform in [a, b)
    TinyTensor<Type>& zeros();
    TinyTensor<Type>& ones();
    TinyTensor<Type>& negative();
    TinyTensor<Type>& mults(const Type scalar);
    TinyTensor<Type>& floatks(float k);          // fill with k
    TinyTensor<Type>& resize(const std::vector<int>& new_shape);

    TinyTensor<Type> ReluForward() const;
    TinyTensor<Type> ReluBackward(const TinyTensor<Type>& grad) const;
    TinyTensor<Type> SigmoidForward() const;
    TinyTensor<Type> SigmoidBackward(const TinyTensor<Type>& grad) const;

    template <typename T>
    friend std::ostream& operator<<(std::ostream& os, const TinyTensor<T>& tensor);

    // additions -------------------------------------------------------------------------
    // float view of the data (bf16 widened exactly), and construction from floats
    std::vector<float> get_data_f32() const;
    static TinyTensor<Type> from_f32(const std::vector<int>& shape, const std::string& device, const float* host_data,
                                     size_t count);
};

using bf16_t = __nv_bfloat16;

#endif  // TT_HOST_TINY_TENSOR_H

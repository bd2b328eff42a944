// Implementation of TinyTensor<T> (see TinyTensor.h).  Device storage is pooled (tt_alloc /
// tt_free); host storage comes from tt_host_alloc / tt_host_free.  The element-wise helpers are simple
// grid-stride kernels with 64-bit indices: they exist for API completeness, the attention
// kernels do the heavy lifting elsewhere.
#include "TinyTensor.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <random>
#include <stdexcept>
#include <typeinfo>

#include "tt_attn.h"

namespace tth {

inline void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
inline void tt_check(int rc, const char* what) {
    if (rc != TT_OK) throw std::runtime_error(std::string(what) + ": " + tt_last_error());
}

// float <-> element conversions usable on host and device
template <typename T> __host__ __device__ inline float to_f(T x) { return static_cast<float>(x); }
template <> __host__ __device__ inline float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __host__ __device__ inline T from_f(float x) { return static_cast<T>(x); }
template <> __host__ __device__ inline __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
// arithmetic in the element's natural precision (double stays double, bf16 goes through float)
template <typename T> struct Acc { using type = T; };
template <> struct Acc<__nv_bfloat16> { using type = float; };
template <typename T> __host__ __device__ inline typename Acc<T>::type widen(T x) { return static_cast<typename Acc<T>::type>(x); }
template <> __host__ __device__ inline float widen<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __host__ __device__ inline T narrow(typename Acc<T>::type x) { return static_cast<T>(x); }
template <> __host__ __device__ inline __nv_bfloat16 narrow<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

enum class UnOp { Neg, Scale, Fill, Relu, Sigmoid };
enum class BinOp { Add, Sub, ReluBwd, SigmoidBwd };

template <typename T>
__host__ __device__ inline T apply_un(UnOp op, T x, typename Acc<T>::type s) {
    using A = typename Acc<T>::type;
    A v = widen<T>(x);
    switch (op) {
        case UnOp::Neg: return narrow<T>(-v);
        case UnOp::Scale: return narrow<T>(v * s);
        case UnOp::Fill: return narrow<T>(s);
        case UnOp::Relu: return narrow<T>(v > A(0) ? v : A(0));
        case UnOp::Sigmoid: return narrow<T>(A(1.0f / (1.0f + expf(-static_cast<float>(v)))));
    }
    return x;
}
template <typename T>
__host__ __device__ inline T apply_bin(BinOp op, T a, T b) {
    using A = typename Acc<T>::type;
    A x = widen<T>(a), y = widen<T>(b);
    switch (op) {
        case BinOp::Add: return narrow<T>(x + y);
        case BinOp::Sub: return narrow<T>(x - y);
        case BinOp::ReluBwd: return narrow<T>(x > A(0) ? y : A(0));     // a = input, b = upstream grad
        case BinOp::SigmoidBwd: {
            float o = 1.0f / (1.0f + expf(-static_cast<float>(x)));
            return narrow<T>(A(o * (1.0f - o)) * y);
        }
    }
    return a;
}

template <typename T>
__global__ void unary_kernel(UnOp op, const T* in, T* out, size_t n, typename Acc<T>::type s) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = apply_un<T>(op, in[i], s);
}
template <typename T>
__global__ void binary_kernel(BinOp op, const T* a, const T* b, T* out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = apply_bin<T>(op, a[i], b[i]);
}
// counter-based uniform numbers: splitmix64 of (seed, index) -> [0,1)
__host__ __device__ inline float unit_uniform(unsigned long long seed, unsigned long long i) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (i + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}
template <typename T>
__global__ void random_kernel(T* out, size_t n, unsigned long long seed, float lo, float hi) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f<T>(lo + (hi - lo) * unit_uniform(seed, i));
}
template <typename T>
__global__ void from_f32_kernel(const float* in, T* out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f<T>(in[i]);
}

inline unsigned grid_for(size_t n) {
    size_t b = (n + 255) / 256;
    return (unsigned)std::min<size_t>(std::max<size_t>(b, 1), 148 * 16);
}

size_t count_of(const std::vector<int>& shape) {
    size_t n = 1;
    for (int d : shape) {
        if (d < 0) throw std::invalid_argument("negative extent in shape");
        n *= (size_t)d;
    }
    return n;
}
void require_device(const std::string& device) {
    if (device != "cpu" && device != "gpu") throw std::invalid_argument("Invalid device");
}
template <typename T>
T* allocate(const std::string& device, size_t n) {
    if (n == 0) return nullptr;
    void* p = nullptr;
    // host and device storage both come from the library, which keeps a buffer alive while an
    // exported view (DLPack) of it exists, whatever happens to the tensor meanwhile
    if (device == "cpu") tt_check(tt_host_alloc(n * sizeof(T), &p), "host allocation");
    else tt_check(tt_alloc(n * sizeof(T), &p), "device allocation");
    return static_cast<T*>(p);
}
template <typename T>
void release(const std::string& device, T* p) noexcept {
    if (!p) return;
    if (device == "cpu") tt_host_free(p);
    else tt_free(p);
}
// copy n elements between any two placements
template <typename T>
void copy_elems(T* dst, const std::string& dst_dev, const T* src, const std::string& src_dev, size_t n) {
    if (n == 0) return;
    if (dst_dev == "cpu" && src_dev == "cpu") {
        std::memcpy(dst, src, n * sizeof(T));
        return;
    }
    cudaMemcpyKind kind = dst_dev == "cpu" ? cudaMemcpyDeviceToHost
                          : (src_dev == "cpu" ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice);
    cuda_check(cudaMemcpy(dst, src, n * sizeof(T), kind), "tensor copy");
}
static std::atomic<unsigned long long> g_random_calls{0};

}  // namespace tth

using namespace tth;

// ------------------------------------------------------------------------------ construction
template <typename Type>
TinyTensor<Type>::TinyTensor(const std::vector<int>& shape_, const std::string& device_)
    : shape(shape_), device(device_), p_data(nullptr), size(0) {
    require_device(device);
    size = count_of(shape);
    p_data = allocate<Type>(device, size);
}

template <typename Type>
TinyTensor<Type>::TinyTensor(const std::vector<int>& shape_, const std::string& device_, const std::vector<Type>& data)
    : TinyTensor(shape_, device_) {
    if (data.size() != size) throw std::invalid_argument("data length does not match shape");
    copy_elems<Type>(p_data, device, data.data(), "cpu", size);
}

template <typename Type>
TinyTensor<Type>::TinyTensor(const pybind11::array_t<typename TinyNumpyElem<Type>::type>& data, const std::string& device_)
    : shape(), device(device_), p_data(nullptr), size(0) {
    require_device(device);
    using NpT = typename TinyNumpyElem<Type>::type;
    auto dense = pybind11::array_t<NpT, pybind11::array::c_style | pybind11::array::forcecast>::ensure(data);
    if (!dense) throw std::invalid_argument("expected a NumPy array");
    pybind11::buffer_info info = dense.request();
    for (auto d : info.shape) shape.push_back((int)d);
    if (shape.empty()) shape.push_back(1);
    size = count_of(shape);
    p_data = allocate<Type>(device, size);
    const NpT* src = static_cast<const NpT*>(info.ptr);
    if constexpr (std::is_same<Type, NpT>::value) {
        copy_elems<Type>(p_data, device, src, "cpu", size);
    } else {
        std::vector<Type> tmp(size);
        for (size_t i = 0; i < size; ++i) tmp[i] = from_f<Type>((float)src[i]);
        copy_elems<Type>(p_data, device, tmp.data(), "cpu", size);
    }
}

template <typename Type>
TinyTensor<Type>::TinyTensor(const TinyTensor<Type>& other)
    : shape(other.shape), device(other.device), p_data(nullptr), size(other.size) {
    p_data = allocate<Type>(device, size);
    copy_elems<Type>(p_data, device, other.p_data, other.device, size);
}

template <typename Type>
TinyTensor<Type>::TinyTensor(TinyTensor<Type>&& other) noexcept
    : shape(std::move(other.shape)), device(other.device), p_data(other.p_data), size(other.size) {
    other.p_data = nullptr;
    other.size = 0;
    other.shape.clear();
}

template <typename Type>
TinyTensor<Type>::~TinyTensor() {
    release<Type>(device, p_data);
    p_data = nullptr;
}

template <typename Type>
size_t TinyTensor<Type>::Size() const { return count_of(shape); }

template <typename Type>
TinyTensor<Type>& TinyTensor<Type>::operator=(const TinyTensor<Type>& other) {
    if (this == &other) return *this;
    Type* fresh = allocate<Type>(other.device, other.size);
    try {
        copy_elems<Type>(fresh, other.device, other.p_data, other.device, other.size);
    } catch (...) {
        release<Type>(other.device, fresh);
        throw;
    }
    release<Type>(device, p_data);
    shape = other.shape;
    device = other.device;
    size = other.size;
    p_data = fresh;
    return *this;
}

template <typename Type>
TinyTensor<Type>& TinyTensor<Type>::operator=(TinyTensor<Type>&& other) noexcept {
    if (this == &other) return *this;
    release<Type>(device, p_data);
    shape = std::move(other.shape);
    device = other.device;
    size = other.size;
    p_data = other.p_data;
    other.p_data = nullptr;
    other.size = 0;
    other.shape.clear();
    return *this;
}

// ------------------------------------------------------------------------------ element-wise
template <typename Type>
static TinyTensor<Type> binary(const TinyTensor<Type>& a, const TinyTensor<Type>& b, BinOp op, const char* what) {
    if (a.shape != b.shape) throw std::invalid_argument(std::string(what) + ": shapes differ");
    if (a.device != b.device) throw std::invalid_argument(std::string(what) + ": devices differ");
    TinyTensor<Type> out(a.shape, a.device);
    if (a.size == 0) return out;
    if (a.device == "cpu") {
        for (size_t i = 0; i < a.size; ++i) out.p_data[i] = apply_bin<Type>(op, a.p_data[i], b.p_data[i]);
    } else {
        binary_kernel<Type><<<grid_for(a.size), 256>>>(op, a.p_data, b.p_data, out.p_data, a.size);
        cuda_check(cudaGetLastError(), what);
        cuda_check(cudaDeviceSynchronize(), what);
    }
    return out;
}
template <typename Type>
static void unary_inplace(const TinyTensor<Type>& src, TinyTensor<Type>& dst, UnOp op, typename Acc<Type>::type s,
                          const char* what) {
    if (src.size == 0) return;
    if (src.device == "cpu") {
        for (size_t i = 0; i < src.size; ++i) dst.p_data[i] = apply_un<Type>(op, src.p_data[i], s);
    } else {
        unary_kernel<Type><<<grid_for(src.size), 256>>>(op, src.p_data, dst.p_data, src.size, s);
        cuda_check(cudaGetLastError(), what);
        cuda_check(cudaDeviceSynchronize(), what);
    }
}

template <typename Type>
TinyTensor<Type> TinyTensor<Type>::operator+(const TinyTensor<Type>& other) const {
    return binary<Type>(*this, other, BinOp::Add, "operator+");
}
template <typename Type>
TinyTensor<Type> TinyTensor<Type>::operator-(const TinyTensor<Type>& other) const {
    return binary<Type>(*this, other, BinOp::Sub, "operator-");
}

template <typename Type>
TinyTensor<Type> TinyTensor<Type>::operator[](const int index) const {
    if (shape.empty() || index < 0 || index >= shape[0]) throw std::invalid_argument("Index out of range");
    std::vector<int> sub(shape.begin() + 1, shape.end());
    if (sub.empty()) sub.push_back(1);
    TinyTensor<Type> out(sub, device);
    copy_elems<Type>(out.p_data, device, p_data + (size_t)index * out.size, device, out.size);
    return out;
}

template <typename Type>
std::vector<int> TinyTensor<Type>::get_shape() const { return shape; }
template <typename Type>
std::string TinyTensor<Type>::get_device() const { return device; }

template <typename Type>
std::vector<Type> TinyTensor<Type>::get_data() const {
    std::vector<Type> host(size);
    copy_elems<Type>(host.data(), "cpu", p_data, device, size);
    return host;
}
template <typename Type>
std::vector<float> TinyTensor<Type>::get_data_f32() const {
    std::vector<Type> raw = get_data();
    std::vector<float> out(raw.size());
    for (size_t i = 0; i < raw.size(); ++i) out[i] = to_f<Type>(raw[i]);
    return out;
}
template <typename Type>
TinyTensor<Type> TinyTensor<Type>::from_f32(const std::vector<int>& shape_, const std::string& device_,
                                            const float* host_data, size_t count) {
    TinyTensor<Type> out(shape_, device_);
    if (count != out.size) throw std::invalid_argument("data length does not match shape");
    std::vector<Type> tmp(count);
    for (size_t i = 0; i < count; ++i) tmp[i] = from_f<Type>(host_data[i]);
    copy_elems<Type>(out.p_data, out.device, tmp.data(), "cpu", count);
    return out;
}

template <typename Type>
TinyTensor<Type> TinyTensor<Type>::flatten() const {
    TinyTensor<Type> out(*this);
    out.shape = {(int)size};
    return out;
}

template <typename Type>
TinyTensor<Type>& TinyTensor<Type>::cpu() {
    if (device == "cpu") return *this;
    Type* host = allocate<Type>("cpu", size);
    try {
        copy_elems<Type>(host, "cpu", p_data, "gpu", size);
    } catch (...) {
        release<Type>("cpu", host);
        throw;
    }
    release<Type>("gpu", p_data);
    p_data = host;
    device = "cpu";
    return *this;
}
template <typename Type>
TinyTensor<Type>& TinyTensor<Type>::gpu() {
    if (device == "gpu") return *this;
    Type* dev = allocate<Type>("gpu", size);
    try {
        copy_elems<Type>(dev, "gpu", p_data, "cpu", size);
    } catch (...) {
        release<Type>("gpu", dev);
        throw;
    }
    release<Type>("cpu", p_data);
    p_data = dev;
    device = "gpu";
    return *this;
}

template <typename Type>
TinyTensor<Type>& TinyTensor<Type>::random(Type a, Type b) {
    const unsigned long long seed = 0x5EEDull * 0x100000001B3ull + g_random_calls.fetch_add(1) * 0xD1342543DE82EF95ull;
    const float lo = to_f<Type>(a), hi = to_f<Type>(b);
    if (size == 0) return *this;
    if (device == "cpu") {
        for (size_t i = 0; i < size; ++i) p_data[i] = from_f<Type>(lo + (hi - lo) * unit_uniform(seed, i));
    } else {
        random_kernel<Type><<<grid_for(size), 256>>>(p_data, size, seed, lo, hi);
        cuda_check(cudaGetLastError(), "random");
        cuda_check(cudaDeviceSynchronize(), "random");
    }
    return *this;
}
template <typename Type>
TinyTensor<Type>& TinyTensor<Type>::zeros() {
    if (size == 0) return *this;
    if (device == "cpu") std::memset(p_data, 0, size * sizeof(Type));
    else cuda_check(cudaMemset(p_data, 0, size * sizeof(Type)), "zeros");
    return *this;
}
template <typename Type>
TinyTensor<Type>& TinyTensor<Type>::ones() {
    unary_inplace<Type>(*this, *this, UnOp::Fill, typename Acc<Type>::type(1), "ones");
    return *this;
}
template <typename Type>
TinyTensor<Type>& TinyTensor<Type>::negative() {
    unary_inplace<Type>(*this, *this, UnOp::Neg, typename Acc<Type>::type(0), "negative");
    return *this;
}
template <typename Type>
TinyTensor<Type>& TinyTensor<Type>::mults(const Type scalar) {
    unary_inplace<Type>(*this, *this, UnOp::Scale, widen<Type>(scalar), "mults");
    return *this;
}
template <typename Type>
TinyTensor<Type>& TinyTensor<Type>::floatks(float k) {
    unary_inplace<Type>(*this, *this, UnOp::Fill, typename Acc<Type>::type(k), "floatks");
    return *this;
}

template <typename Type>
TinyTensor<Type>& TinyTensor<Type>::resize(const std::vector<int>& new_shape) {
    const size_t new_size = count_of(new_shape);
    if (new_size == size) {   // same element count: a pure reshape
        shape = new_shape;
        return *this;
    }
    Type* fresh = allocate<Type>(device, new_size);
    const size_t keep = std::min(size, new_size);
    try {
        copy_elems<Type>(fresh, device, p_data, device, keep);
        if (new_size > keep) {   // the reference leaves the tail uninitialised; zero it instead
            if (device == "cpu") std::memset(fresh + keep, 0, (new_size - keep) * sizeof(Type));
            else cuda_check(cudaMemset(fresh + keep, 0, (new_size - keep) * sizeof(Type)), "resize");
        }
    } catch (...) {
        release<Type>(device, fresh);
        throw;
    }
    release<Type>(device, p_data);
    p_data = fresh;
    shape = new_shape;
    size = new_size;
    return *this;
}

template <typename Type>
TinyTensor<Type> TinyTensor<Type>::ReluForward() const {
    TinyTensor<Type> out(shape, device);
    unary_inplace<Type>(*this, out, UnOp::Relu, typename Acc<Type>::type(0), "ReluForward");
    return out;
}
template <typename Type>
TinyTensor<Type> TinyTensor<Type>::ReluBackward(const TinyTensor<Type>& grad) const {
    return binary<Type>(*this, grad, BinOp::ReluBwd, "ReluBackward");
}
template <typename Type>
TinyTensor<Type> TinyTensor<Type>::SigmoidForward() const {
    TinyTensor<Type> out(shape, device);
    unary_inplace<Type>(*this, out, UnOp::Sigmoid, typename Acc<Type>::type(0), "SigmoidForward");
    return out;
}
template <typename Type>
TinyTensor<Type> TinyTensor<Type>::SigmoidBackward(const TinyTensor<Type>& grad) const {
    return binary<Type>(*this, grad, BinOp::SigmoidBwd, "SigmoidBackward");
}

template <typename Type>
std::ostream& operator<<(std::ostream& os, const TinyTensor<Type>& tensor) {
    os << "TinyTensor<" << (std::is_same<Type, __nv_bfloat16>::value ? "bf16" : typeid(Type).name()) << ">\n";
    os << "Device: " << tensor.device << "\nShape: [";
    for (size_t i = 0; i < tensor.shape.size(); ++i) os << tensor.shape[i] << (i + 1 < tensor.shape.size() ? ", " : "");
    os << "]\n";
    const std::vector<float> host = tensor.get_data_f32();
    const size_t row = tensor.shape.empty() ? 1 : (size_t)std::max(tensor.shape.back(), 1);
    const size_t limit = std::min<size_t>(host.size(), 4096);   // printing multi-GB tensors helps nobody
    for (size_t i = 0; i < limit; ++i) os << host[i] << (((i + 1) % row == 0) ? "\n" : " ");
    if (limit < host.size()) os << "... (" << host.size() - limit << " more)\n";
    return os;
}

template class TinyTensor<int>;
template class TinyTensor<float>;
template class TinyTensor<double>;
template class TinyTensor<__nv_bfloat16>;
template std::ostream& operator<<(std::ostream&, const TinyTensor<int>&);
template std::ostream& operator<<(std::ostream&, const TinyTensor<float>&);
template std::ostream& operator<<(std::ostream&, const TinyTensor<double>&);
template std::ostream& operator<<(std::ostream&, const TinyTensor<__nv_bfloat16>&);

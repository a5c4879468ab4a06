// Eager, CPU-only stand-in for the small slice of the MLX C++ API that the
// TurboQuant reference sources use (array, dtype tags, a dozen elementwise /
// reduction ops, stream tags).  TEST INFRASTRUCTURE ONLY: it exists so that the
// reference's own quantizer / dequantizer / KV-cache translation units can be
// compiled unmodified into a checker library; the product never links it.
//
// Semantics that matter for parity:
//   * every op is evaluated immediately in IEEE fp32, one rounding per op
//     (build with -ffp-contract=off, no -ffast-math);
//   * sum() accumulates sequentially, left to right, in fp32.  Real MLX leaves
//     reduction order unspecified, so this order is the definition the checker
//     and the CUDA kernels both follow for row norms.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <initializer_list>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

namespace mlx {
namespace core {

using float16_t = _Float16;

enum class DtypeTag : uint8_t { F32, F16, U8, U32, BOOL, I32 };

struct Dtype {
    DtypeTag tag;
    constexpr bool operator==(const Dtype& o) const { return tag == o.tag; }
    constexpr bool operator!=(const Dtype& o) const { return tag != o.tag; }
    size_t size() const {
        switch (tag) {
            case DtypeTag::F32: case DtypeTag::U32: case DtypeTag::I32: return 4;
            case DtypeTag::F16: return 2;
            default: return 1;
        }
    }
};

static constexpr Dtype float32{DtypeTag::F32};
static constexpr Dtype float16{DtypeTag::F16};
static constexpr Dtype uint8{DtypeTag::U8};
static constexpr Dtype uint32{DtypeTag::U32};
static constexpr Dtype int32{DtypeTag::I32};
static constexpr Dtype bool_{DtypeTag::BOOL};

using Shape = std::vector<int>;

struct Device {
    enum Kind { cpu, gpu };
    Kind kind;
    Device(Kind k = cpu) : kind(k) {}
};

struct Stream {
    int index = 0;
    Device device;
    Stream() = default;
    Stream(int i, Device d) : index(i), device(d) {}
};

inline Stream default_stream(Device d) { return Stream(0, d); }

class Primitive;

namespace allocator {
struct Buffer { void* p = nullptr; };
inline Buffer malloc(size_t n) { return Buffer{::operator new(n)}; }
}  // namespace allocator

namespace detail {
template <typename T> struct dtype_of;
template <> struct dtype_of<float> { static constexpr Dtype v = float32; };
template <> struct dtype_of<float16_t> { static constexpr Dtype v = float16; };
template <> struct dtype_of<uint8_t> { static constexpr Dtype v = uint8; };
template <> struct dtype_of<uint32_t> { static constexpr Dtype v = uint32; };
template <> struct dtype_of<int32_t> { static constexpr Dtype v = int32; };
template <> struct dtype_of<bool> { static constexpr Dtype v = bool_; };

inline double load_as_double(const uint8_t* p, Dtype dt, size_t i) {
    switch (dt.tag) {
        case DtypeTag::F32: return reinterpret_cast<const float*>(p)[i];
        case DtypeTag::F16: return static_cast<float>(reinterpret_cast<const float16_t*>(p)[i]);
        case DtypeTag::U8: return reinterpret_cast<const uint8_t*>(p)[i];
        case DtypeTag::U32: return reinterpret_cast<const uint32_t*>(p)[i];
        case DtypeTag::I32: return reinterpret_cast<const int32_t*>(p)[i];
        case DtypeTag::BOOL: return reinterpret_cast<const uint8_t*>(p)[i] ? 1.0 : 0.0;
    }
    return 0.0;
}

inline void store_from_float(uint8_t* p, Dtype dt, size_t i, float v) {
    switch (dt.tag) {
        case DtypeTag::F32: reinterpret_cast<float*>(p)[i] = v; break;
        case DtypeTag::F16: reinterpret_cast<float16_t*>(p)[i] = static_cast<float16_t>(v); break;
        case DtypeTag::U8: reinterpret_cast<uint8_t*>(p)[i] = static_cast<uint8_t>(v); break;
        case DtypeTag::U32: reinterpret_cast<uint32_t*>(p)[i] = static_cast<uint32_t>(v); break;
        case DtypeTag::I32: reinterpret_cast<int32_t*>(p)[i] = static_cast<int32_t>(v); break;
        case DtypeTag::BOOL: reinterpret_cast<uint8_t*>(p)[i] = (v != 0.0f); break;
    }
}
}  // namespace detail

class array {
public:
    // Scalar.
    array(float v) : shape_{}, dtype_(float32) {
        alloc(1);
        *reinterpret_cast<float*>(buf_->data()) = v;
    }

    // Typed pointer + shape (+ optional target dtype; converts if it differs).
    template <typename T>
    array(const T* src, Shape shape, Dtype dt = detail::dtype_of<T>::v)
        : shape_(std::move(shape)), dtype_(dt) {
        size_t n = count(shape_);
        alloc(n);
        if (dt == detail::dtype_of<T>::v) {
            if (n) std::memcpy(buf_->data(), src, n * sizeof(T));
        } else {
            for (size_t i = 0; i < n; ++i)
                detail::store_from_float(buf_->data(), dtype_, i, static_cast<float>(src[i]));
        }
    }

    // Brace list of floats with explicit shape/dtype, e.g. array({0.0f}, {1}, float32).
    array(std::initializer_list<float> vals, Shape shape, Dtype dt = float32)
        : shape_(std::move(shape)), dtype_(dt) {
        alloc(vals.size());
        size_t i = 0;
        for (float v : vals) detail::store_from_float(buf_->data(), dtype_, i++, v);
    }

    // Brace list of floats, 1-D; array({}) is the empty array.
    array(std::initializer_list<float> vals)
        : shape_{static_cast<int>(vals.size())}, dtype_(float32) {
        alloc(vals.size());
        size_t i = 0;
        for (float v : vals) reinterpret_cast<float*>(buf_->data())[i++] = v;
    }

    // Lazy node backed by a Primitive.  The shim never evaluates these: the only
    // producer is the reference's fused Metal linear, which has no CPU path.
    array(Shape shape, Dtype dt, std::shared_ptr<Primitive> prim, std::vector<array> inputs)
        : shape_(std::move(shape)), dtype_(dt), prim_(std::move(prim)) {
        (void)inputs;
        alloc(count(shape_));
    }

    // Uninitialised storage of a given shape (used by the ops below).
    static array empty(Shape shape, Dtype dt) {
        array a(0.0f);
        a.shape_ = std::move(shape);
        a.dtype_ = dt;
        a.alloc(count(a.shape_));
        return a;
    }

    template <typename T> const T* data() const { return reinterpret_cast<const T*>(buf_->data()); }
    template <typename T> T* data() { return reinterpret_cast<T*>(buf_->data()); }
    template <typename T> T item() const {
        return static_cast<T>(detail::load_as_double(buf_->data(), dtype_, 0));
    }

    const Shape& shape() const { return shape_; }
    int shape(int i) const { return shape_[i < 0 ? i + static_cast<int>(shape_.size()) : i]; }
    size_t size() const { return count(shape_); }
    size_t ndim() const { return shape_.size(); }
    Dtype dtype() const { return dtype_; }
    size_t nbytes() const { return size() * dtype_.size(); }
    bool is_lazy() const { return static_cast<bool>(prim_); }
    void set_data(allocator::Buffer b) { ::operator delete(b.p); }

    const uint8_t* raw() const { return buf_->data(); }
    uint8_t* raw() { return buf_->data(); }

    static size_t count(const Shape& s) {
        size_t n = 1;
        for (int d : s) n *= static_cast<size_t>(d);
        return n;
    }

private:
    void alloc(size_t n) { buf_ = std::make_shared<std::vector<uint8_t>>(n * dtype_.size() + 8); }

    Shape shape_;
    Dtype dtype_;
    std::shared_ptr<std::vector<uint8_t>> buf_;
    std::shared_ptr<Primitive> prim_;
};

// eval is a no-op: everything is already materialised.
template <typename... Args> inline void eval(Args&&...) {}

inline array astype(const array& a, Dtype dt) {
    if (a.dtype() == dt) return a;
    array r = array::empty(a.shape(), dt);
    size_t n = a.size();
    if (a.dtype() == float32 && dt == float16) {
        // single rounding fp32 -> fp16 (round to nearest even)
        const float* s = a.data<float>();
        float16_t* d = r.data<float16_t>();
        for (size_t i = 0; i < n; ++i) d[i] = static_cast<float16_t>(s[i]);
        return r;
    }
    for (size_t i = 0; i < n; ++i)
        detail::store_from_float(r.raw(), dt, i,
                                 static_cast<float>(detail::load_as_double(a.raw(), a.dtype(), i)));
    return r;
}

inline array reshape(const array& a, Shape shape) {
    size_t known = 1;
    int infer = -1;
    for (size_t i = 0; i < shape.size(); ++i) {
        if (shape[i] == -1) infer = static_cast<int>(i);
        else known *= static_cast<size_t>(shape[i]);
    }
    if (infer >= 0) shape[infer] = static_cast<int>(a.size() / (known ? known : 1));
    if (array::count(shape) != a.size()) throw std::invalid_argument("shim reshape: size mismatch");
    array r = array::empty(shape, a.dtype());
    if (a.nbytes()) std::memcpy(r.raw(), a.raw(), a.nbytes());
    return r;
}

namespace detail {
// Binary fp32 op with the three broadcast patterns the reference uses:
// equal shapes, one side a single element, or [rows, cols] against [rows, 1].
template <typename F>
inline array binary_f32(const array& a_in, const array& b_in, F f, Dtype out_dt = float32) {
    array a = astype(a_in, float32), b = astype(b_in, float32);
    const array& big = (a.size() >= b.size()) ? a : b;
    array r = array::empty(big.shape(), out_dt);
    size_t n = big.size();
    const float* pa = a.data<float>();
    const float* pb = b.data<float>();
    auto put = [&](size_t i, float v) {
        if (out_dt == float32) r.data<float>()[i] = v;
        else store_from_float(r.raw(), out_dt, i, v);
    };
    if (a.size() == b.size()) {
        for (size_t i = 0; i < n; ++i) put(i, f(pa[i], pb[i]));
    } else if (b.size() == 1) {
        for (size_t i = 0; i < n; ++i) put(i, f(pa[i], pb[0]));
    } else if (a.size() == 1) {
        for (size_t i = 0; i < n; ++i) put(i, f(pa[0], pb[i]));
    } else {
        const array& small = (a.size() >= b.size()) ? b : a;
        bool a_big = (&big == &a);
        if (big.ndim() != 2 || small.ndim() != 2 || small.shape(1) != 1 ||
            small.shape(0) != big.shape(0))
            throw std::invalid_argument("shim: unsupported broadcast");
        size_t rows = big.shape(0), cols = big.shape(1);
        for (size_t r0 = 0; r0 < rows; ++r0)
            for (size_t c = 0; c < cols; ++c) {
                size_t i = r0 * cols + c;
                put(i, a_big ? f(pa[i], pb[r0]) : f(pa[r0], pb[i]));
            }
    }
    return r;
}
}  // namespace detail

inline array multiply(const array& a, const array& b) {
    return detail::binary_f32(a, b, [](float x, float y) { return x * y; });
}
inline array add(const array& a, const array& b) {
    return detail::binary_f32(a, b, [](float x, float y) { return x + y; });
}
inline array subtract(const array& a, const array& b) {
    return detail::binary_f32(a, b, [](float x, float y) { return x - y; });
}
inline array divide(const array& a, const array& b) {
    return detail::binary_f32(a, b, [](float x, float y) { return x / y; });
}
inline array maximum(const array& a, const array& b) {
    return detail::binary_f32(a, b, [](float x, float y) { return x > y ? x : y; });
}
inline array less(const array& a, const array& b) {
    return detail::binary_f32(a, b, [](float x, float y) { return x < y ? 1.0f : 0.0f; }, bool_);
}
inline array greater_equal(const array& a, const array& b) {
    return detail::binary_f32(a, b, [](float x, float y) { return x >= y ? 1.0f : 0.0f; }, bool_);
}
inline array logical_and(const array& a, const array& b) {
    return detail::binary_f32(
        a, b, [](float x, float y) { return (x != 0.0f && y != 0.0f) ? 1.0f : 0.0f; }, bool_);
}

inline array sqrt(const array& a_in) {
    array a = astype(a_in, float32);
    array r = array::empty(a.shape(), float32);
    for (size_t i = 0; i < a.size(); ++i) r.data<float>()[i] = std::sqrt(a.data<float>()[i]);
    return r;
}

// Full reduction: sequential fp32.
inline array sum(const array& a_in) {
    array a = astype(a_in, float32);
    float acc = 0.0f;
    const float* p = a.data<float>();
    for (size_t i = 0; i < a.size(); ++i) acc += p[i];
    return array(acc);
}

// Reduction over the last axis of a 2-D array: sequential fp32 per row.
inline array sum(const array& a_in, const std::vector<int>& axes, bool keepdims = false) {
    array a = astype(a_in, float32);
    if (a.ndim() != 2 || axes.size() != 1 || (axes[0] != 1 && axes[0] != -1))
        throw std::invalid_argument("shim sum: only axis=1 of a 2-D array");
    int rows = a.shape(0), cols = a.shape(1);
    array r = array::empty(keepdims ? Shape{rows, 1} : Shape{rows}, float32);
    const float* p = a.data<float>();
    for (int i = 0; i < rows; ++i) {
        float acc = 0.0f;
        for (int j = 0; j < cols; ++j) acc += p[static_cast<size_t>(i) * cols + j];
        r.data<float>()[i] = acc;
    }
    return r;
}

inline array zeros(const Shape& shape, Dtype dt = float32) {
    array r = array::empty(shape, dt);
    if (r.nbytes()) std::memset(r.raw(), 0, r.nbytes());
    return r;
}
inline array zeros_like(const array& a) { return zeros(a.shape(), a.dtype()); }
inline array ones_like(const array& a) {
    array r = array::empty(a.shape(), a.dtype());
    for (size_t i = 0; i < a.size(); ++i) detail::store_from_float(r.raw(), a.dtype(), i, 1.0f);
    return r;
}

inline array take(const array& a, int index) {
    array r = array::empty({}, a.dtype());
    std::memcpy(r.raw(), a.raw() + static_cast<size_t>(index) * a.dtype().size(), a.dtype().size());
    return r;
}

inline array transpose(const array& a, const std::vector<int>& perm) {
    size_t nd = a.ndim();
    Shape out_shape(nd);
    for (size_t i = 0; i < nd; ++i) out_shape[i] = a.shape(perm[i]);
    array r = array::empty(out_shape, a.dtype());
    std::vector<size_t> in_stride(nd, 1);
    for (int i = static_cast<int>(nd) - 2; i >= 0; --i)
        in_stride[i] = in_stride[i + 1] * static_cast<size_t>(a.shape(i + 1));
    size_t es = a.dtype().size(), n = a.size();
    std::vector<int> idx(nd, 0);
    for (size_t o = 0; o < n; ++o) {
        size_t src = 0;
        for (size_t i = 0; i < nd; ++i) src += static_cast<size_t>(idx[i]) * in_stride[perm[i]];
        std::memcpy(r.raw() + o * es, a.raw() + src * es, es);
        for (int i = static_cast<int>(nd) - 1; i >= 0; --i) {
            if (++idx[i] < out_shape[i]) break;
            idx[i] = 0;
        }
    }
    return r;
}

inline array expand_dims(const array& a, int axis) {
    Shape s = a.shape();
    if (axis < 0) axis += static_cast<int>(s.size()) + 1;
    s.insert(s.begin() + axis, 1);
    return reshape(a, s);
}

}  // namespace core
}  // namespace mlx

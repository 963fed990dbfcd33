// Host reducers.  Same contract as the reference's reduce()
// (src/stdml/collective/dtype.cpp:80-165) plus bf16/f16, plus a multi-input
// form that is the oracle for the device kernels.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include <stdml/bits/collective/dtype.hpp>

namespace stdml::collective
{
float bf16_to_float(uint16_t bits)
{
    uint32_t w = static_cast<uint32_t>(bits) << 16;
    float f;
    std::memcpy(&f, &w, 4);
    return f;
}

uint16_t float_to_bf16(float x)
{
    uint32_t w;
    std::memcpy(&w, &x, 4);
    if ((w & 0x7fffffffu) > 0x7f800000u) {  // NaN: keep it a quiet NaN
        return static_cast<uint16_t>((w >> 16) | 0x0040u);
    }
    const uint32_t lsb = (w >> 16) & 1u;
    w += 0x7fffu + lsb;  // round to nearest, ties to even
    return static_cast<uint16_t>(w >> 16);
}

float f16_to_float(uint16_t h)
{
    const uint32_t sign = (static_cast<uint32_t>(h) & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t w;
    if (exp == 0) {
        if (man == 0) {
            w = sign;
        } else {  // subnormal half -> normal float
            int e = -1;
            do {
                ++e;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            w = sign | ((127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        w = sign | 0x7f800000u | (man << 13);
    } else {
        w = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &w, 4);
    return f;
}

uint16_t float_to_f16(float x)
{
    uint32_t w;
    std::memcpy(&w, &x, 4);
    const uint32_t sign = (w >> 16) & 0x8000u;
    const uint32_t absw = w & 0x7fffffffu;
    if (absw > 0x7f800000u) { return static_cast<uint16_t>(sign | 0x7e00u); }
    if (absw >= 0x47800000u) {  // >= 65536 -> inf (65520 rounds up below)
        return static_cast<uint16_t>(sign | 0x7c00u);
    }
    if (absw < 0x33000000u) {  // < 2^-25 -> 0
        return static_cast<uint16_t>(sign);
    }
    int32_t exp = static_cast<int32_t>(absw >> 23) - 127;
    uint32_t man = (absw & 0x7fffffu) | 0x800000u;
    uint32_t half;
    if (exp < -14) {  // subnormal half
        const int shift = -14 - exp + 13;  // 14..24
        const uint32_t rem = man & ((1u << shift) - 1u);
        const uint32_t halfway = 1u << (shift - 1);
        half = man >> shift;
        if (rem > halfway || (rem == halfway && (half & 1u))) { ++half; }
    } else {
        const uint32_t rem = man & 0x1fffu;
        half = (static_cast<uint32_t>(exp + 15) << 10) | ((man >> 13) & 0x3ffu);
        if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) { ++half; }
    }
    return static_cast<uint16_t>(sign | half);
}

size_t dtype_size(dtype dt)
{
    const size_t n = dtype_size_nothrow(dt);
    if (n == 0) {
        throw std::invalid_argument("dtype_size: unknown dtype " +
                                    std::to_string(static_cast<int>(dt)));
    }
    return n;
}

static const char *const k_dtype_names[dtype_count] = {
    "i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "bf16", "f16", "f32", "f64",
};

static const char *const k_op_names[reduce_op_count] = {
    "sum", "min", "max", "prod", "bit_xor",
};

const char *dtype_name(dtype dt)
{
    const int i = static_cast<int>(dt);
    return (i >= 0 && i < dtype_count) ? k_dtype_names[i] : "?";
}

const char *reduce_op_name(reduce_op op)
{
    const int i = static_cast<int>(op);
    return (i >= 0 && i < reduce_op_count) ? k_op_names[i] : "?";
}

bool parse_dtype(const std::string &s, dtype &out)
{
    for (int i = 0; i < dtype_count; ++i) {
        if (s == k_dtype_names[i]) {
            out = static_cast<dtype>(i);
            return true;
        }
    }
    return false;
}

bool parse_reduce_op(const std::string &s, reduce_op &out)
{
    for (int i = 0; i < reduce_op_count; ++i) {
        if (s == k_op_names[i]) {
            out = static_cast<reduce_op>(i);
            return true;
        }
    }
    if (s == "xor") {
        out = bit_xor;
        return true;
    }
    return false;
}

bool reduce_supported(dtype dt, reduce_op op)
{
    if (dtype_size_nothrow(dt) == 0) { return false; }
    if (op == bit_xor) { return dt <= u64; }
    return op >= sum && op <= prod;
}

namespace
{
template <typename A>
inline A apply(reduce_op op, A a, A b)
{
    switch (op) {
    case sum:
        return a + b;
    case min:
        return b < a ? b : a;
    case max:
        return a < b ? b : a;
    case prod:
        return a * b;
    default:
        return a;
    }
}

template <typename T>
inline T apply_int(reduce_op op, T a, T b)
{
    if (op == bit_xor) { return static_cast<T>(a ^ b); }
    // wrap-around arithmetic on the unsigned image: defined for every input
    using U = std::make_unsigned_t<T>;
    switch (op) {
    case sum:
        return static_cast<T>(static_cast<U>(a) + static_cast<U>(b));
    case prod:
        return static_cast<T>(static_cast<U>(a) * static_cast<U>(b));
    case min:
        return b < a ? b : a;
    case max:
        return a < b ? b : a;
    default:
        return a;
    }
}

template <typename T>
void reduce_ints(T *x, const T *y, const T *z, size_t n, reduce_op op)
{
    switch (op) {  // hoist the switch so each loop auto-vectorises
    case sum:
        for (size_t i = 0; i < n; ++i) { x[i] = apply_int<T>(sum, y[i], z[i]); }
        break;
    case min:
        for (size_t i = 0; i < n; ++i) { x[i] = apply_int<T>(min, y[i], z[i]); }
        break;
    case max:
        for (size_t i = 0; i < n; ++i) { x[i] = apply_int<T>(max, y[i], z[i]); }
        break;
    case prod:
        for (size_t i = 0; i < n; ++i) { x[i] = apply_int<T>(prod, y[i], z[i]); }
        break;
    case bit_xor:
        for (size_t i = 0; i < n; ++i) { x[i] = apply_int<T>(bit_xor, y[i], z[i]); }
        break;
    }
}

template <typename T>
void reduce_floats(T *x, const T *y, const T *z, size_t n, reduce_op op)
{
    switch (op) {
    case sum:
        for (size_t i = 0; i < n; ++i) { x[i] = y[i] + z[i]; }
        break;
    case min:
        for (size_t i = 0; i < n; ++i) { x[i] = z[i] < y[i] ? z[i] : y[i]; }
        break;
    case max:
        for (size_t i = 0; i < n; ++i) { x[i] = y[i] < z[i] ? z[i] : y[i]; }
        break;
    case prod:
        for (size_t i = 0; i < n; ++i) { x[i] = y[i] * z[i]; }
        break;
    default:
        throw std::invalid_argument("bit_xor is not defined for floating point");
    }
}

template <float (*Widen)(uint16_t), uint16_t (*Narrow)(float)>
void reduce_half(uint16_t *x, const uint16_t *y, const uint16_t *z, size_t n,
                 reduce_op op)
{
    if (op == bit_xor) {
        throw std::invalid_argument("bit_xor is not defined for floating point");
    }
    for (size_t i = 0; i < n; ++i) {
        x[i] = Narrow(apply<float>(op, Widen(y[i]), Widen(z[i])));
    }
}

template <typename T>
void many_ints(T *out, const void *const *in, size_t n, size_t count, reduce_op op)
{
    for (size_t i = 0; i < count; ++i) {
        T acc = static_cast<const T *>(in[0])[i];
        for (size_t r = 1; r < n; ++r) {
            acc = apply_int<T>(op, acc, static_cast<const T *>(in[r])[i]);
        }
        out[i] = acc;
    }
}

template <typename T>
void many_floats(T *out, const void *const *in, size_t n, size_t count,
                 reduce_op op, double scale)
{
    const bool scaled = scale != 1.0;
    const T s = static_cast<T>(scale);
    for (size_t i = 0; i < count; ++i) {
        T acc = static_cast<const T *>(in[0])[i];
        for (size_t r = 1; r < n; ++r) {
            acc = apply<T>(op, acc, static_cast<const T *>(in[r])[i]);
        }
        out[i] = scaled ? acc * s : acc;
    }
}

template <float (*Widen)(uint16_t), uint16_t (*Narrow)(float)>
void many_half(uint16_t *out, const void *const *in, size_t n, size_t count,
               reduce_op op, double scale)
{
    const bool scaled = scale != 1.0;
    const float s = static_cast<float>(scale);
    for (size_t i = 0; i < count; ++i) {
        float acc = Widen(static_cast<const uint16_t *>(in[0])[i]);
        for (size_t r = 1; r < n; ++r) {
            acc = apply<float>(op, acc, Widen(static_cast<const uint16_t *>(in[r])[i]));
        }
        out[i] = Narrow(scaled ? acc * s : acc);
    }
}
}  // namespace

void reduce(void *x, const void *y, const void *z, size_t count, dtype dt,
            reduce_op op)
{
    if (!reduce_supported(dt, op)) {
        throw std::invalid_argument(std::string("reduce: ") + reduce_op_name(op) +
                                    " is not defined for " + dtype_name(dt));
    }
#define STDML_CASE_INT(E, T)                                                   \
    case E:                                                                    \
        reduce_ints<T>(static_cast<T *>(x), static_cast<const T *>(y),         \
                       static_cast<const T *>(z), count, op);                  \
        return;
    switch (dt) {
        STDML_CASE_INT(i8, int8_t)
        STDML_CASE_INT(i16, int16_t)
        STDML_CASE_INT(i32, int32_t)
        STDML_CASE_INT(i64, int64_t)
        STDML_CASE_INT(u8, uint8_t)
        STDML_CASE_INT(u16, uint16_t)
        STDML_CASE_INT(u32, uint32_t)
        STDML_CASE_INT(u64, uint64_t)
    case bf16:
        reduce_half<bf16_to_float, float_to_bf16>(
            static_cast<uint16_t *>(x), static_cast<const uint16_t *>(y),
            static_cast<const uint16_t *>(z), count, op);
        return;
    case f16:
        reduce_half<f16_to_float, float_to_f16>(
            static_cast<uint16_t *>(x), static_cast<const uint16_t *>(y),
            static_cast<const uint16_t *>(z), count, op);
        return;
    case f32:
        reduce_floats<float>(static_cast<float *>(x), static_cast<const float *>(y),
                             static_cast<const float *>(z), count, op);
        return;
    case f64:
        reduce_floats<double>(static_cast<double *>(x),
                              static_cast<const double *>(y),
                              static_cast<const double *>(z), count, op);
        return;
    }
#undef STDML_CASE_INT
}

void scale_in_place(void *x, size_t count, dtype dt, double scale)
{
    const float s = static_cast<float>(scale);
    switch (dt) {
    case f32:
        for (size_t i = 0; i < count; ++i) { static_cast<float *>(x)[i] *= s; }
        return;
    case f64:
        for (size_t i = 0; i < count; ++i) { static_cast<double *>(x)[i] *= static_cast<double>(s); }
        return;
    case bf16:
        for (size_t i = 0; i < count; ++i) {
            uint16_t &v = static_cast<uint16_t *>(x)[i];
            v = float_to_bf16(bf16_to_float(v) * s);
        }
        return;
    case f16:
        for (size_t i = 0; i < count; ++i) {
            uint16_t &v = static_cast<uint16_t *>(x)[i];
            v = float_to_f16(f16_to_float(v) * s);
        }
        return;
    default:
        return;  // integers are not scaled (same as the device kernels)
    }
}

void reduce_many(void *out, const void *const *in, size_t n, size_t count,
                 dtype dt, reduce_op op, double scale)
{
    if (n == 0) { return; }
    if (!reduce_supported(dt, op)) {
        throw std::invalid_argument(std::string("reduce_many: ") +
                                    reduce_op_name(op) + " is not defined for " +
                                    dtype_name(dt));
    }
#define STDML_CASE_INT(E, T)                                                   \
    case E:                                                                    \
        many_ints<T>(static_cast<T *>(out), in, n, count, op);                 \
        return;
    switch (dt) {
        STDML_CASE_INT(i8, int8_t)
        STDML_CASE_INT(i16, int16_t)
        STDML_CASE_INT(i32, int32_t)
        STDML_CASE_INT(i64, int64_t)
        STDML_CASE_INT(u8, uint8_t)
        STDML_CASE_INT(u16, uint16_t)
        STDML_CASE_INT(u32, uint32_t)
        STDML_CASE_INT(u64, uint64_t)
    case bf16:
        many_half<bf16_to_float, float_to_bf16>(static_cast<uint16_t *>(out), in, n,
                                                count, op, scale);
        return;
    case f16:
        many_half<f16_to_float, float_to_f16>(static_cast<uint16_t *>(out), in, n,
                                              count, op, scale);
        return;
    case f32:
        many_floats<float>(static_cast<float *>(out), in, n, count, op, scale);
        return;
    case f64:
        many_floats<double>(static_cast<double *>(out), in, n, count, op, scale);
        return;
    }
#undef STDML_CASE_INT
}
}  // namespace stdml::collective

// Element types and reduction operators shared by the host (TCP) path and the
// device (NVLink) path.
//
// Parity: the enumerator order and names follow the reference
// (include/stdml/bits/collective/dtype.hpp:7-22 and :60-66) so that integer
// values written by user code keep their meaning.  Unlike the reference
// (src/stdml/collective/dtype.cpp:152-161, where bf16/f16 abort) the 16-bit
// float types are fully implemented here, on the host and on the device.
#pragma once
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace stdml::collective
{
enum dtype {
    i8,
    i16,
    i32,
    i64,

    u8,
    u16,
    u32,
    u64,

    bf16,
    f16,
    f32,
    f64,
};

constexpr int dtype_count = 12;

enum reduce_op {
    sum,
    min,
    max,
    prod,
    bit_xor,
};

constexpr int reduce_op_count = 5;

// Storage-only 16-bit float carriers for host code.  Arithmetic happens in
// f32; see to_float()/from_float() in dtype.cpp (round-to-nearest-even).
struct bfloat16_t {
    uint16_t bits;
};

struct float16_t {
    uint16_t bits;
};

float bf16_to_float(uint16_t bits);
uint16_t float_to_bf16(float x);
float f16_to_float(uint16_t bits);
uint16_t float_to_f16(float x);

namespace detail
{
template <typename T>
struct dtype_of;

template <>
struct dtype_of<int8_t> {
    static constexpr dtype value = i8;
};
template <>
struct dtype_of<int16_t> {
    static constexpr dtype value = i16;
};
template <>
struct dtype_of<int32_t> {
    static constexpr dtype value = i32;
};
template <>
struct dtype_of<int64_t> {
    static constexpr dtype value = i64;
};
template <>
struct dtype_of<uint8_t> {
    static constexpr dtype value = u8;
};
template <>
struct dtype_of<uint16_t> {
    static constexpr dtype value = u16;
};
template <>
struct dtype_of<uint32_t> {
    static constexpr dtype value = u32;
};
template <>
struct dtype_of<uint64_t> {
    static constexpr dtype value = u64;
};
template <>
struct dtype_of<bfloat16_t> {
    static constexpr dtype value = bf16;
};
template <>
struct dtype_of<float16_t> {
    static constexpr dtype value = f16;
};
template <>
struct dtype_of<float> {
    static constexpr dtype value = f32;
};
template <>
struct dtype_of<double> {
    static constexpr dtype value = f64;
};
// `long long` / `unsigned long long` are distinct from int64_t on LP64.
template <>
struct dtype_of<long long> {
    static constexpr dtype value = i64;
};
template <>
struct dtype_of<unsigned long long> {
    static constexpr dtype value = u64;
};
// plain `char` is what broadcast-as-bytes uses on some call sites
template <>
struct dtype_of<char> {
    static constexpr dtype value = i8;
};
}  // namespace detail

template <typename T>
constexpr dtype type()
{
    return detail::dtype_of<T>::value;
}

// Bytes per element.  Never throws for a valid enumerator (bf16/f16 -> 2).
constexpr size_t dtype_size_nothrow(dtype dt)
{
    switch (dt) {
    case i8:
    case u8:
        return 1;
    case i16:
    case u16:
    case bf16:
    case f16:
        return 2;
    case i32:
    case u32:
    case f32:
        return 4;
    case i64:
    case u64:
    case f64:
        return 8;
    }
    return 0;
}

size_t dtype_size(dtype dt);

const char *dtype_name(dtype dt);
const char *reduce_op_name(reduce_op op);
bool parse_dtype(const std::string &s, dtype &out);
bool parse_reduce_op(const std::string &s, reduce_op &out);

// true when `op` is defined for `dt` (bit_xor is integer-only, as in the
// reference where xor on float/double throws: dtype.cpp:62-78).
bool reduce_supported(dtype dt, reduce_op op);

// x[i] = y[i] op z[i] for i in [0, count).  x may alias y or z.
// 16-bit floats are widened to f32 per element, combined, and rounded back
// (round-to-nearest-even), so a chain of pairwise calls rounds at every step;
// reduce_many() below rounds once.
void reduce(void *x, const void *y, const void *z, size_t count, dtype dt,
            reduce_op op);

// out[i] = in[0][i] op in[1][i] op ... op in[n-1][i], left to right
// ("rank-ascending", the canonical order of the device kernels).  16-bit
// floats accumulate in f32 and round once; `scale` (if not 1) multiplies the
// f32/f64 accumulator before the final rounding.  Used as the CPU oracle of
// the device kernels and by the host one-shot path.
void reduce_many(void *out, const void *const *in, size_t n, size_t count,
                 dtype dt, reduce_op op, double scale = 1.0);

// x[i] *= float(scale) for floating-point dtypes; integers are left alone.
void scale_in_place(void *x, size_t count, dtype dt, double scale);
}  // namespace stdml::collective

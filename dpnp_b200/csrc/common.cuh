// Shared definitions for the sm_100a kernels and their host dispatch:
// element types, type traits, the element conversion rule, error plumbing,
// fast integer division and vector load/store helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <type_traits>

#include "../../include/dpnp_b200.h"

#define DPB_HD __host__ __device__ __forceinline__
#define DPB_D __device__ __forceinline__

namespace dpb {

// ------------------------------------------------------------------ errors
int set_error(int status, const char *fmt, ...);
void note_kernel(const char *name);  // records family name and counts one launch
void note_copy(const char *name);    // records the name of a library copy (not a kernel of ours)
int check_launch(const char *what);  // cudaGetLastError -> status

#define DPB_CUDA_TRY(expr)                                                              \
    do {                                                                                \
        cudaError_t err__ = (expr);                                                     \
        if (err__ != cudaSuccess) {                                                     \
            return ::dpb::set_error(err__ == cudaErrorMemoryAllocation ? DPB_ERR_MEMORY \
                                                                       : DPB_ERR_CUDA,  \
                                    "%s failed: %s", #expr, cudaGetErrorString(err__)); \
        }                                                                               \
    } while (0)

#define DPB_TRY(expr)                     \
    do {                                  \
        int st__ = (expr);                \
        if (st__ != DPB_OK) return st__;  \
    } while (0)

// device properties cached per device
struct DeviceProps {
    int sm_count;
    int max_smem_optin;
};
const DeviceProps &device_props();
int64_t tuning_ctas_per_sm();
bool tuning_verbose();        // log every kernel choice on stderr
bool tuning_force_generic();  // send every elementwise / reduction call to the generic strided kernels
int64_t tuning_fused_elems();  // elements per thread and register of the fused-chain interpreter

// ------------------------------------------------------------ element types

// Boolean stored as one byte; any non-zero byte reads as true (NumPy's rule,
// which the reference follows in convert_impl, include/utils/type_utils.hpp:63-114).
struct bool_t {
    unsigned char v;
    bool_t() = default;
    DPB_HD bool_t(bool b) : v(b ? 1 : 0) {}
    DPB_HD operator bool() const { return v != 0; }
};

template <class T>
struct alignas(2 * sizeof(T)) cplx {
    T re, im;
    cplx() = default;
    DPB_HD cplx(T r, T i = T(0)) : re(r), im(i) {}
};
using cfloat = cplx<float>;
using cdouble = cplx<double>;
using half_t = __half;

template <class T> struct is_cplx : std::false_type {};
template <class T> struct is_cplx<cplx<T>> : std::true_type {};
template <class T> inline constexpr bool is_cplx_v = is_cplx<T>::value;
template <class T> inline constexpr bool is_bool_v = std::is_same_v<T, bool_t>;
template <class T> inline constexpr bool is_half_v = std::is_same_v<T, half_t>;
template <class T>
inline constexpr bool is_fp_v = std::is_same_v<T, float> || std::is_same_v<T, double> || is_half_v<T>;
template <class T>
inline constexpr bool is_int_v = std::is_integral_v<T> && !std::is_same_v<T, bool>;
template <class T> inline constexpr bool is_uint_v = is_int_v<T> && std::is_unsigned_v<T>;
template <class T> inline constexpr bool is_sint_v = is_int_v<T> && std::is_signed_v<T>;

template <int TN> struct type_of;
template <> struct type_of<DPB_BOOL> { using type = bool_t; };
template <> struct type_of<DPB_INT8> { using type = int8_t; };
template <> struct type_of<DPB_UINT8> { using type = uint8_t; };
template <> struct type_of<DPB_INT16> { using type = int16_t; };
template <> struct type_of<DPB_UINT16> { using type = uint16_t; };
template <> struct type_of<DPB_INT32> { using type = int32_t; };
template <> struct type_of<DPB_UINT32> { using type = uint32_t; };
template <> struct type_of<DPB_INT64> { using type = int64_t; };
template <> struct type_of<DPB_UINT64> { using type = uint64_t; };
template <> struct type_of<DPB_HALF> { using type = half_t; };
template <> struct type_of<DPB_FLOAT> { using type = float; };
template <> struct type_of<DPB_DOUBLE> { using type = double; };
template <> struct type_of<DPB_CFLOAT> { using type = cfloat; };
template <> struct type_of<DPB_CDOUBLE> { using type = cdouble; };
template <int TN> using type_of_t = typename type_of<TN>::type;

template <class T> struct typenum_of;
#define DPB_TN(T, N) \
    template <> struct typenum_of<T> { static constexpr int value = N; };
DPB_TN(bool_t, DPB_BOOL)
DPB_TN(int8_t, DPB_INT8)
DPB_TN(uint8_t, DPB_UINT8)
DPB_TN(int16_t, DPB_INT16)
DPB_TN(uint16_t, DPB_UINT16)
DPB_TN(int32_t, DPB_INT32)
DPB_TN(uint32_t, DPB_UINT32)
DPB_TN(int64_t, DPB_INT64)
DPB_TN(uint64_t, DPB_UINT64)
DPB_TN(half_t, DPB_HALF)
DPB_TN(float, DPB_FLOAT)
DPB_TN(double, DPB_DOUBLE)
DPB_TN(cfloat, DPB_CFLOAT)
DPB_TN(cdouble, DPB_CDOUBLE)
#undef DPB_TN

inline int type_size(int tn)
{
    static const int sz[DPB_NUM_TYPES] = {1, 1, 1, 2, 2, 4, 4, 8, 8, 2, 4, 8, 8, 16};
    return (tn >= 0 && tn < DPB_NUM_TYPES) ? sz[tn] : 0;
}
inline const char *type_name(int tn)
{
    static const char *nm[DPB_NUM_TYPES] = {"bool",   "int8",   "uint8",   "int16",   "uint16",
                                            "int32",  "uint32", "int64",   "uint64",  "float16",
                                            "float32", "float64", "complex64", "complex128"};
    return (tn >= 0 && tn < DPB_NUM_TYPES) ? nm[tn] : "?";
}

// --------------------------------------------------------------- conversion
// convert<To>(from): the element conversion used by every cast-on-load and by
// copy/cast.  To bool: value != 0 (complex: either part non-zero).  From bool:
// 0 or 1.  Complex -> real keeps the real part.  Floating -> unsigned goes
// through a signed integer so that negatives wrap.  Otherwise static_cast.
template <class To, class From>
DPB_HD To convert(const From &v)
{
    if constexpr (std::is_same_v<To, From>) {
        return v;
    }
    else if constexpr (is_bool_v<To>) {
        if constexpr (is_cplx_v<From>) {
            return bool_t(v.re != 0 || v.im != 0);
        }
        else if constexpr (is_half_v<From>) {
            return bool_t(__half2float(v) != 0.0f);
        }
        else {
            return bool_t(v != From(0));
        }
    }
    else if constexpr (is_bool_v<From>) {
        if constexpr (is_cplx_v<To>) {
            using R = decltype(To{}.re);
            return To(v.v ? R(1) : R(0), R(0));
        }
        else if constexpr (is_half_v<To>) {
            return __float2half(v.v ? 1.0f : 0.0f);
        }
        else {
            return v.v ? To(1) : To(0);
        }
    }
    else if constexpr (is_cplx_v<From>) {
        if constexpr (is_cplx_v<To>) {
            using R = decltype(To{}.re);
            return To(static_cast<R>(v.re), static_cast<R>(v.im));
        }
        else {
            return convert<To>(v.re);
        }
    }
    else if constexpr (is_cplx_v<To>) {
        using R = decltype(To{}.re);
        return To(convert<R>(v), R(0));
    }
    else if constexpr (is_half_v<From>) {
        if constexpr (std::is_same_v<To, float>) return __half2float(v);
        else return convert<To>(__half2float(v));
    }
    else if constexpr (is_half_v<To>) {
        if constexpr (std::is_same_v<From, double>) return __double2half(v);
        else if constexpr (std::is_same_v<From, float>) return __float2half(v);
        else if constexpr (std::is_same_v<From, int64_t>) return __ll2half_rn(v);
        else if constexpr (std::is_same_v<From, uint64_t>) return __ull2half_rn(v);
        else if constexpr (std::is_same_v<From, uint32_t>) return __uint2half_rn(v);
        else return __int2half_rn(static_cast<int>(v));
    }
    else if constexpr (!std::is_integral_v<From> && is_uint_v<To>) {
        using I = std::conditional_t<(sizeof(To) < 4), int32_t, int64_t>;
        return (v < From(0)) ? static_cast<To>(static_cast<I>(v)) : static_cast<To>(v);
    }
    else {
        return static_cast<To>(v);
    }
}

// ------------------------------------------------------- fast index division
// Division of a 31-bit unsigned value by a fixed positive divisor with one
// 32x32->64 multiply and a shift.
struct FastDiv32 {
    uint32_t d;
    uint32_t mul;
    uint32_t shift;
    FastDiv32() = default;
    explicit FastDiv32(uint32_t divisor) : d(divisor)   // host side (no attribute: the run-time compiler rejects __host__)
    {
        uint32_t s = 0;
        while ((uint64_t(1) << s) < divisor) ++s;
        // ceil(2^(31+s) / d); fits in 32 bits because 2^(s-1) < d <= 2^s
        uint64_t p = uint64_t(1) << (31 + s);
        mul = static_cast<uint32_t>((p + divisor - 1) / divisor);
        shift = s;
    }
    DPB_HD uint32_t div(uint32_t n) const
    {
#ifdef __CUDA_ARCH__
        return static_cast<uint32_t>((static_cast<uint64_t>(n) * mul) >> 31) >> shift;
#else
        return static_cast<uint32_t>(((static_cast<uint64_t>(n) * mul) >> 31) >> shift);
#endif
    }
    DPB_HD void divmod(uint32_t n, uint32_t &q, uint32_t &r) const
    {
        q = div(n);
        r = n - q * d;
    }
};

// ------------------------------------------------------------------ vectors
template <class T, int N>
struct alignas(sizeof(T) * N) vec_t {
    T v[N];
};

// Number of elements per 16-byte access for a set of element sizes: limited by
// the widest type so that no single access exceeds 16 bytes.
template <class... Ts>
constexpr int vec_width()
{
    size_t m = 1;
    ((m = sizeof(Ts) > m ? sizeof(Ts) : m), ...);
    return static_cast<int>(16 / m);
}

template <class V>
DPB_D V load_vec(const void *p)
{
    V out;
    if constexpr (sizeof(V) == 16) {
        int4 t = __ldg(reinterpret_cast<const int4 *>(p));
        out = *reinterpret_cast<V *>(&t);
    }
    else if constexpr (sizeof(V) == 8) {
        int2 t = __ldg(reinterpret_cast<const int2 *>(p));
        out = *reinterpret_cast<V *>(&t);
    }
    else if constexpr (sizeof(V) == 4) {
        int t = __ldg(reinterpret_cast<const int *>(p));
        out = *reinterpret_cast<V *>(&t);
    }
    else if constexpr (sizeof(V) == 2) {
        short t = __ldg(reinterpret_cast<const short *>(p));
        out = *reinterpret_cast<V *>(&t);
    }
    else if constexpr (sizeof(V) == 1) {
        char t = __ldg(reinterpret_cast<const char *>(p));
        out = *reinterpret_cast<V *>(&t);
    }
    else {
        out = *reinterpret_cast<const V *>(p);
    }
    return out;
}

template <class V>
DPB_D void store_vec(void *p, const V &val)
{
    if constexpr (sizeof(V) == 16) {
        *reinterpret_cast<int4 *>(p) = *reinterpret_cast<const int4 *>(&val);
    }
    else if constexpr (sizeof(V) == 8) {
        *reinterpret_cast<int2 *>(p) = *reinterpret_cast<const int2 *>(&val);
    }
    else if constexpr (sizeof(V) == 4) {
        *reinterpret_cast<int *>(p) = *reinterpret_cast<const int *>(&val);
    }
    else if constexpr (sizeof(V) == 2) {
        *reinterpret_cast<short *>(p) = *reinterpret_cast<const short *>(&val);
    }
    else if constexpr (sizeof(V) == 1) {
        *reinterpret_cast<char *>(p) = *reinterpret_cast<const char *>(&val);
    }
    else {
        *reinterpret_cast<V *>(p) = val;
    }
}

// scalar element load through the read-only path
template <class T>
DPB_D T load_elem(const T *p)
{
    return load_vec<vec_t<T, 1>>(p).v[0];
}

#ifndef __CUDACC_RTC__
bool tuning_pdl();   // "pdl" switch: launch the streaming kernels with programmatic stream serialisation

// Launch of a kernel that begins with cudaGridDependencySynchronize(): with the attribute below the
// launch itself overlaps the tail of the kernel before it in the stream (measured on B200: 16
// back-to-back additions of 2^24 float32, 32.9 us -> 30.6 us each); the kernel still starts
// reading only after that kernel has completed and its writes are visible.
template <class... KArgs, class... Args>
inline void launch_after_previous(void (*kernel)(KArgs...), unsigned grid, unsigned block, cudaStream_t stream,
                                  Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    if (tuning_pdl()) {
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);   // an error stays in cudaGetLastError for check_launch
}

#endif

inline bool is_aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace dpb

// Counter-based random fills: element i is a pure function of (seed, i), so
// shards of one logical array can be generated independently on any device.
#include <algorithm>

#include "common.cuh"

namespace dpb {

DPB_HD uint64_t mix64(uint64_t x)
{
    // splitmix64 finaliser
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

DPB_HD uint64_t rand_bits(uint64_t seed, uint64_t index, uint64_t lane)
{
    return mix64(mix64(seed ^ (lane * 0xD6E8FEB86659FD93ull)) + index);
}

// uniform double in [0, 1) with 53 random bits
DPB_HD double unit_double(uint64_t bits) { return static_cast<double>(bits >> 11) * (1.0 / 9007199254740992.0); }

template <class T>
__global__ void uniform_kernel(T *dst, int64_t n, double lo, double hi, uint64_t seed, uint64_t first)
{
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += int64_t(gridDim.x) * blockDim.x) {
        const uint64_t bits = rand_bits(seed, first + static_cast<uint64_t>(i), 0);
        if constexpr (is_fp_v<T>) {
            const double u = unit_double(bits);
            double v = lo + (hi - lo) * u;
            if (v >= hi && hi > lo) v = lo;  // rounding must not reach the open end
            dst[i] = convert<T>(v);
        }
        else if constexpr (is_bool_v<T>) {
            dst[i] = bool_t((bits >> 63) != 0);
        }
        else {
            const uint64_t range = static_cast<uint64_t>(static_cast<int64_t>(hi) - static_cast<int64_t>(lo));
            const uint64_t r = range ? __umul64hi(bits, range) : 0;
            dst[i] = static_cast<T>(static_cast<int64_t>(lo) + static_cast<int64_t>(r));
        }
    }
}

template <class T>
__global__ void normal_kernel(T *dst, int64_t n, double mean, double stddev, uint64_t seed, uint64_t first)
{
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += int64_t(gridDim.x) * blockDim.x) {
        const uint64_t idx = first + static_cast<uint64_t>(i);
        // Box-Muller; u1 in (0, 1]
        const double u1 = 1.0 - unit_double(rand_bits(seed, idx, 1));
        const double u2 = unit_double(rand_bits(seed, idx, 2));
        const double r = sqrt(-2.0 * log(u1));
        const double z = r * cospi(2.0 * u2);
        dst[i] = convert<T>(mean + stddev * z);
    }
}



}  // namespace dpb

using namespace dpb;

#define DPB_RANDOM_SWITCH(KERNEL, ...)                                                     \
    switch (typenum) {                                                                     \
    case DPB_BOOL: KERNEL<bool_t><<<grid, 256, 0, s>>>(static_cast<bool_t *>(dst), __VA_ARGS__); break;    \
    case DPB_INT8: KERNEL<int8_t><<<grid, 256, 0, s>>>(static_cast<int8_t *>(dst), __VA_ARGS__); break;    \
    case DPB_UINT8: KERNEL<uint8_t><<<grid, 256, 0, s>>>(static_cast<uint8_t *>(dst), __VA_ARGS__); break; \
    case DPB_INT16: KERNEL<int16_t><<<grid, 256, 0, s>>>(static_cast<int16_t *>(dst), __VA_ARGS__); break; \
    case DPB_UINT16: KERNEL<uint16_t><<<grid, 256, 0, s>>>(static_cast<uint16_t *>(dst), __VA_ARGS__); break; \
    case DPB_INT32: KERNEL<int32_t><<<grid, 256, 0, s>>>(static_cast<int32_t *>(dst), __VA_ARGS__); break; \
    case DPB_UINT32: KERNEL<uint32_t><<<grid, 256, 0, s>>>(static_cast<uint32_t *>(dst), __VA_ARGS__); break; \
    case DPB_INT64: KERNEL<int64_t><<<grid, 256, 0, s>>>(static_cast<int64_t *>(dst), __VA_ARGS__); break; \
    case DPB_UINT64: KERNEL<uint64_t><<<grid, 256, 0, s>>>(static_cast<uint64_t *>(dst), __VA_ARGS__); break; \
    case DPB_HALF: KERNEL<half_t><<<grid, 256, 0, s>>>(static_cast<half_t *>(dst), __VA_ARGS__); break;    \
    case DPB_FLOAT: KERNEL<float><<<grid, 256, 0, s>>>(static_cast<float *>(dst), __VA_ARGS__); break;     \
    case DPB_DOUBLE: KERNEL<double><<<grid, 256, 0, s>>>(static_cast<double *>(dst), __VA_ARGS__); break;  \
    default: return set_error(DPB_ERR_TYPE, "random fill is not defined for %s", type_name(typenum));      \
    }

extern "C" int dpb_random_uniform(int typenum, void *dst, int64_t nelems, double lo, double hi,
                                  uint64_t seed, uint64_t first_index, void *stream)
{
    if (nelems < 0) return set_error(DPB_ERR_VALUE, "negative size");
    if (nelems == 0) return DPB_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t cap = int64_t(device_props().sm_count) * 8;
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min(cap, ceil_div(nelems, 256))));
    DPB_RANDOM_SWITCH(uniform_kernel, nelems, lo, hi, seed, first_index)
    note_kernel("random_uniform");
    return check_launch("random_uniform");
}

extern "C" int dpb_random_normal(int typenum, void *dst, int64_t nelems, double mean, double stddev,
                                 uint64_t seed, uint64_t first_index, void *stream)
{
    if (nelems < 0) return set_error(DPB_ERR_VALUE, "negative size");
    if (nelems == 0) return DPB_OK;
    if (typenum != DPB_HALF && typenum != DPB_FLOAT && typenum != DPB_DOUBLE)
        return set_error(DPB_ERR_TYPE, "normal variates need a floating-point type, got %s",
                         type_name(typenum));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t cap = int64_t(device_props().sm_count) * 8;
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min(cap, ceil_div(nelems, 256))));
    switch (typenum) {
    case DPB_HALF: normal_kernel<half_t><<<grid, 256, 0, s>>>(static_cast<half_t *>(dst), nelems, mean, stddev, seed, first_index); break;
    case DPB_FLOAT: normal_kernel<float><<<grid, 256, 0, s>>>(static_cast<float *>(dst), nelems, mean, stddev, seed, first_index); break;
    default: normal_kernel<double><<<grid, 256, 0, s>>>(static_cast<double *>(dst), nelems, mean, stddev, seed, first_index); break;
    }
    note_kernel("random_normal");
    return check_launch("random_normal");
}

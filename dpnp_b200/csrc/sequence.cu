// Linear sequences written on the device: arange-style (start, step) and linspace-style
// (start, end) fills of a contiguous array.  They replace lin_space_step_impl and
// lin_space_affine_impl (dpnp/tensor/libtensor/include/kernels/constructors.hpp:65-131,136-246).
#include "common.cuh"
#include "ew_ops.cuh"

namespace dpb {

// p[i] = start + i * step in the array's own arithmetic (integers wrap)
template <class T> __global__ void sequence_step_kernel(T *p, int64_t n, T start, T step)
{
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        if constexpr (is_half_v<T>) p[i] = __float2half(__half2float(start) + float(i) * __half2float(step));
        else if constexpr (std::is_floating_point_v<T>) p[i] = start + T(i) * step;
        else {
            using U = std::make_unsigned_t<T>;
            p[i] = static_cast<T>(static_cast<U>(static_cast<U>(start) + static_cast<U>(static_cast<U>(i) * static_cast<U>(step))));
        }
    }
}

// p[i] = start * (den - i) / den + end * i / den: the weights are computed in W (double on a
// device with 64-bit floats, constructors.hpp:217-238), rounded to T, then two fused
// multiply-adds (constructors.hpp:152-186)
template <class T, class W> __global__ void sequence_affine_kernel(T *p, int64_t n, T start, T end, int64_t den)
{
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        const W wc = W(i) / W(den);
        const W w = W(den - i) / W(den);
        if constexpr (is_half_v<T>) {
            float acc = fmaf(__half2float(start), float(w), 0.0f);
            acc = fmaf(__half2float(end), float(wc), acc);
            p[i] = __float2half(acc);
        }
        else {
            T acc = fma(start, T(w), T(0));
            acc = fma(end, T(wc), acc);
            p[i] = acc;
        }
    }
}

static int seq_grid(int64_t n)
{
    const int64_t cap = int64_t(device_props().sm_count) * 8;
    return static_cast<int>(std::max<int64_t>(1, std::min(cap, ceil_div(n, 256))));
}

}  // namespace dpb

using namespace dpb;

extern "C" int dpb_linspace_step(int typenum, void *dst, int64_t nelems, const void *start, const void *step,
                                 void *stream)
{
    if (nelems < 0) return set_error(DPB_ERR_VALUE, "negative size");
    if (nelems == 0) return DPB_OK;
    if (!dst || !start || !step) return set_error(DPB_ERR_VALUE, "null argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = seq_grid(nelems);
#define DPB_SEQ_STEP(TN, T)                                                                              \
    case TN:                                                                                             \
        sequence_step_kernel<T><<<grid, 256, 0, s>>>(static_cast<T *>(dst), nelems,                      \
                                                     *static_cast<const T *>(start), *static_cast<const T *>(step)); \
        break;
    switch (typenum) {
        DPB_SEQ_STEP(DPB_INT8, int8_t)
        DPB_SEQ_STEP(DPB_UINT8, uint8_t)
        DPB_SEQ_STEP(DPB_INT16, int16_t)
        DPB_SEQ_STEP(DPB_UINT16, uint16_t)
        DPB_SEQ_STEP(DPB_INT32, int32_t)
        DPB_SEQ_STEP(DPB_UINT32, uint32_t)
        DPB_SEQ_STEP(DPB_INT64, int64_t)
        DPB_SEQ_STEP(DPB_UINT64, uint64_t)
        DPB_SEQ_STEP(DPB_HALF, half_t)
        DPB_SEQ_STEP(DPB_FLOAT, float)
        DPB_SEQ_STEP(DPB_DOUBLE, double)
    default:
        return set_error(DPB_ERR_TYPE, "no linear-sequence kernel for type %s", type_name(typenum));
    }
#undef DPB_SEQ_STEP
    note_kernel("sequence_step");
    return check_launch("sequence_step");
}

extern "C" int dpb_linspace_affine(int typenum, void *dst, int64_t nelems, const void *start, const void *end,
                                   int include_endpoint, void *stream)
{
    if (nelems < 0) return set_error(DPB_ERR_VALUE, "negative size");
    if (nelems == 0) return DPB_OK;
    if (!dst || !start || !end) return set_error(DPB_ERR_VALUE, "null argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = seq_grid(nelems);
    int64_t den = include_endpoint ? nelems - 1 : nelems;
    if (den == 0) den = 1;
    switch (typenum) {
    case DPB_HALF:
        sequence_affine_kernel<half_t, double><<<grid, 256, 0, s>>>(static_cast<half_t *>(dst), nelems,
                                                                   *static_cast<const half_t *>(start),
                                                                   *static_cast<const half_t *>(end), den);
        break;
    case DPB_FLOAT:
        sequence_affine_kernel<float, double><<<grid, 256, 0, s>>>(static_cast<float *>(dst), nelems,
                                                                  *static_cast<const float *>(start),
                                                                  *static_cast<const float *>(end), den);
        break;
    case DPB_DOUBLE:
        sequence_affine_kernel<double, double><<<grid, 256, 0, s>>>(static_cast<double *>(dst), nelems,
                                                                    *static_cast<const double *>(start),
                                                                    *static_cast<const double *>(end), den);
        break;
    default:
        return set_error(DPB_ERR_TYPE, "linspace needs a floating-point type, got %s", type_name(typenum));
    }
    note_kernel("sequence_affine");
    return check_launch("sequence_affine");
}

// dst[0] = src[index[0]] for an index held on the device (one element of `elem_size` bytes):
// lets a search result be turned into (value, index) without a host round trip.
namespace dpb {
__global__ void take_one_kernel(const unsigned char *src, const int64_t *index, unsigned char *dst, int elem_size,
                                int64_t nelems)
{
    int64_t i = index[0];
    if (i < 0) i = 0;                 // the caller validates; never read outside the array
    if (i >= nelems) i = nelems - 1;
    if (threadIdx.x < elem_size) dst[threadIdx.x] = src[i * elem_size + threadIdx.x];
}
}  // namespace dpb

extern "C" int dpb_take_one(int typenum, const void *src, int64_t nelems, const void *index, void *dst, void *stream)
{
    if (typenum < 0 || typenum >= DPB_NUM_TYPES) return set_error(DPB_ERR_VALUE, "unknown type id");
    if (!src || !index || !dst || nelems <= 0) return set_error(DPB_ERR_VALUE, "null argument or empty array");
    take_one_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const unsigned char *>(src), static_cast<const int64_t *>(index),
        static_cast<unsigned char *>(dst), static_cast<int>(type_size(typenum)), nelems);
    note_kernel("take_one");
    return check_launch("take_one");
}

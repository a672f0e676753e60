/*
 * dpnp_b200.h -- C ABI of libdpnp_b200.so: the sm_100a data-parallel core
 * (strided elementwise engine + reduction-over-axis engine) that sits where
 * dpnp's pybind11 modules _tensor_impl / _tensor_elementwise_impl /
 * _tensor_reductions_impl sit in the reference.
 *
 * Conventions
 *  - plain pointers and sizes only; every device pointer is a CUDA device
 *    address valid on the device that is current in the calling thread;
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *    stream); all work is enqueued, nothing synchronises unless stated;
 *  - strides and offsets are in ELEMENTS, not bytes (as in usm_ndarray,
 *    dpnp/tensor/_usmarray.pxd:81-111);
 *  - every function returns a dpb_status; on failure a thread-local message
 *    is available from dpb_last_error().  No exception crosses this boundary;
 *  - there is no CPU fallback: without a CUDA device every compute entry
 *    point fails with DPB_ERR_CUDA.
 *
 * Each declaration cites the reference interface it replaces as
 * file:line relative to the root of IntelPython/dpnp.
 */
#ifndef DPNP_B200_H
#define DPNP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ types */

/* Type ids, same order as typenum_t in
 * dpnp/tensor/libtensor/include/utils/type_dispatch_building.hpp:45-62 */
typedef enum dpb_typenum {
    DPB_BOOL = 0,
    DPB_INT8 = 1,
    DPB_UINT8 = 2,
    DPB_INT16 = 3,
    DPB_UINT16 = 4,
    DPB_INT32 = 5,
    DPB_UINT32 = 6,
    DPB_INT64 = 7,
    DPB_UINT64 = 8,
    DPB_HALF = 9,
    DPB_FLOAT = 10,
    DPB_DOUBLE = 11,
    DPB_CFLOAT = 12,
    DPB_CDOUBLE = 13,
    DPB_NUM_TYPES = 14
} dpb_typenum;

/* Status codes.  The Python shim maps VALUE->ValueError, RUNTIME and CUDA->
 * RuntimeError, MEMORY->MemoryError, TYPE->TypeError, matching the exception
 * classes thrown by the reference dispatchers
 * (dpnp/tensor/libtensor/source/elementwise_functions/elementwise_functions.hpp:96-164). */
typedef enum dpb_status {
    DPB_OK = 0,
    DPB_ERR_VALUE = 1,
    DPB_ERR_RUNTIME = 2,
    DPB_ERR_CUDA = 3,
    DPB_ERR_MEMORY = 4,
    DPB_ERR_TYPE = 5
} dpb_status;

/* Contiguity / writability flags, values as in
 * dpnp/include/usm_ndarray_constants.h:32-59 */
#define DPB_FLAG_C_CONTIGUOUS 1
#define DPB_FLAG_F_CONTIGUOUS 2
#define DPB_FLAG_WRITABLE 4

/* Largest number of dimensions an array descriptor may carry, and the largest
 * number that may remain after the iteration space has been collapsed (the
 * collapsed shape and strides travel by value in kernel parameters). */
#define DPB_MAX_ND 32
#define DPB_MAX_COLLAPSED_ND 10

/* Plain-C view of an array: what dpnp4pybind11.hpp's `class usm_ndarray`
 * (dpnp/include/dpnp4pybind11.hpp:341-621) exposes to the C++ dispatchers. */
typedef struct dpb_array {
    void *data;             /* device address of element [0,...,0]            */
    int32_t nd;             /* number of dimensions, 0..DPB_MAX_ND            */
    int32_t typenum;        /* dpb_typenum                                    */
    int32_t flags;          /* DPB_FLAG_* bits                                */
    int32_t device;         /* CUDA device ordinal that owns `data`           */
    const int64_t *shape;   /* nd extents (host memory)                       */
    const int64_t *strides; /* nd strides in elements (host memory); NULL
                               means C-contiguous                             */
} dpb_array;

/* ------------------------------------------------------------- operations */

/* Unary elementwise operations (one header each under
 * dpnp/tensor/libtensor/include/kernels/elementwise_functions/). */
typedef enum dpb_unary_op {
    DPB_U_NEGATIVE = 0, /* negative.hpp */
    DPB_U_POSITIVE,     /* positive.hpp */
    DPB_U_ABS,          /* abs.hpp */
    DPB_U_EXP,          /* exp.hpp:63-133 */
    DPB_U_LOG,          /* log.hpp:60-84 */
    DPB_U_SQRT,         /* sqrt.hpp:62-84 */
    DPB_U_ERF,          /* dpnp/backend/kernels/elementwise_functions/erf.hpp:51-99 */
    DPB_U_SQUARE,       /* square.hpp */
    DPB_U_RECIPROCAL,   /* reciprocal.hpp */
    DPB_U_SIN,          /* sin.hpp */
    DPB_U_COS,          /* cos.hpp */
    DPB_U_TANH,         /* tanh.hpp */
    DPB_U_EXPM1,        /* expm1.hpp */
    DPB_U_LOG1P,        /* log1p.hpp */
    DPB_U_FLOOR,        /* floor.hpp */
    DPB_U_CEIL,         /* ceil.hpp */
    DPB_U_SIGN,         /* sign.hpp */
    DPB_U_LOGICAL_NOT,  /* logical_not.hpp */
    DPB_U_ISNAN,        /* isnan.hpp */
    DPB_U_ISFINITE,     /* isfinite.hpp */
    DPB_U_ISINF,        /* isinf.hpp */
    DPB_U_ACOS,         /* acos.hpp */
    DPB_U_ACOSH,        /* acosh.hpp */
    DPB_U_ASIN,         /* asin.hpp */
    DPB_U_ASINH,        /* asinh.hpp */
    DPB_U_ATAN,         /* atan.hpp */
    DPB_U_ATANH,        /* atanh.hpp */
    DPB_U_CBRT,         /* cbrt.hpp */
    DPB_U_COSH,         /* cosh.hpp */
    DPB_U_SINH,         /* sinh.hpp */
    DPB_U_TAN,          /* tan.hpp */
    DPB_U_EXP2,         /* exp2.hpp */
    DPB_U_LOG2,         /* log2.hpp */
    DPB_U_LOG10,        /* log10.hpp */
    DPB_U_RSQRT,        /* rsqrt.hpp */
    DPB_U_TRUNC,        /* trunc.hpp */
    DPB_U_ROUND,        /* round.hpp:70-95 (half to even) */
    DPB_U_SIGNBIT,      /* signbit.hpp */
    DPB_U_BITWISE_INVERT, /* bitwise_invert.hpp */
    DPB_U_CONJ,         /* conj.hpp */
    DPB_U_REAL,         /* real.hpp */
    DPB_U_IMAG,         /* imag.hpp */
    DPB_U_ANGLE,        /* angle.hpp */
    DPB_U_PROJ,         /* proj.hpp */
    DPB_U_NUM_OPS
} dpb_unary_op;

/* Binary elementwise operations. */
typedef enum dpb_binary_op {
    DPB_B_ADD = 0,       /* add.hpp:62-114 */
    DPB_B_SUBTRACT,      /* subtract.hpp */
    DPB_B_MULTIPLY,      /* multiply.hpp:62-105 */
    DPB_B_TRUE_DIVIDE,   /* true_divide.hpp:62-113 */
    DPB_B_MAXIMUM,       /* maximum.hpp */
    DPB_B_MINIMUM,       /* minimum.hpp */
    DPB_B_EQUAL,         /* equal.hpp */
    DPB_B_NOT_EQUAL,     /* not_equal.hpp */
    DPB_B_LESS,          /* less.hpp:60-101 */
    DPB_B_LESS_EQUAL,    /* less_equal.hpp */
    DPB_B_GREATER,       /* greater.hpp */
    DPB_B_GREATER_EQUAL, /* greater_equal.hpp */
    DPB_B_LOGICAL_AND,   /* logical_and.hpp */
    DPB_B_LOGICAL_OR,    /* logical_or.hpp */
    DPB_B_POW,           /* pow.hpp */
    DPB_B_ATAN2,         /* atan2.hpp */
    DPB_B_HYPOT,         /* hypot.hpp */
    DPB_B_COPYSIGN,      /* copysign.hpp */
    DPB_B_LOGADDEXP,     /* logaddexp.hpp, utils/math_utils.hpp:131-147 */
    DPB_B_NEXTAFTER,     /* nextafter.hpp */
    DPB_B_BITWISE_AND,   /* bitwise_and.hpp */
    DPB_B_BITWISE_OR,    /* bitwise_or.hpp */
    DPB_B_BITWISE_XOR,   /* bitwise_xor.hpp */
    DPB_B_BITWISE_LEFT_SHIFT,  /* bitwise_left_shift.hpp:88-104 */
    DPB_B_BITWISE_RIGHT_SHIFT, /* bitwise_right_shift.hpp:87-105 */
    DPB_B_FLOOR_DIVIDE,  /* floor_divide.hpp:67-90 */
    DPB_B_REMAINDER,     /* remainder.hpp:66-100 */
    DPB_B_LOGICAL_XOR,   /* logical_xor.hpp */
    DPB_B_NUM_OPS
} dpb_binary_op;

/* Reductions over trailing axes. */
typedef enum dpb_reduce_op {
    DPB_R_SUM = 0, /* source/reductions/sum.cpp */
    DPB_R_PROD,    /* source/reductions/prod.cpp */
    DPB_R_MAX,     /* source/reductions/max.cpp (NaN-propagating for fp) */
    DPB_R_MIN,     /* source/reductions/min.cpp */
    DPB_R_LOGSUMEXP, /* source/reductions/logsumexp.cpp (floating types) */
    DPB_R_HYPOT,   /* source/reductions/reduce_hypot.cpp (floating types) */
    DPB_R_NUM_OPS
} dpb_reduce_op;

/* Search reductions (index of the first extreme value, NaN counts as extreme). */
typedef enum dpb_search_op {
    DPB_S_ARGMAX = 0, /* source/reductions/argmax.cpp:76-141 */
    DPB_S_ARGMIN,     /* source/reductions/argmin.cpp */
    DPB_S_NUM_OPS
} dpb_search_op;

/* Accumulations (prefix scans) along the last axis. */
typedef enum dpb_accumulate_op {
    DPB_A_CUMSUM = 0,     /* source/accumulators/cumulative_sum.cpp */
    DPB_A_CUMPROD,        /* source/accumulators/cumulative_prod.cpp */
    DPB_A_CUMLOGSUMEXP,   /* source/accumulators/cumulative_logsumexp.cpp (floating types) */
    DPB_A_NUM_OPS
} dpb_accumulate_op;

/* -------------------------------------------------- errors and the device */

/* Message of the last failure in the calling thread ("" if none). */
const char *dpb_last_error(void);

/* Library version string. */
const char *dpb_version(void);

/* Number of CUDA devices visible (0 without a driver/GPU; never fails). */
int dpb_device_count(void);

/* Make `device` current in the calling thread (cudaSetDevice). Replaces the
 * device selection implied by a SyclQueue (dpnp/tensor/_compute_follows_data.pyx:67-160). */
/* "domain:bus:device.function" of a device (NUL-terminated, at least 16 bytes): tells two ranks
 * whether they sit on the same GPU. */
int dpb_device_pci_bus_id(int device, char *buf, int len);
int dpb_set_device(int device);
int dpb_get_device(int *device);

/* SM count and total global memory of `device`. */
int dpb_device_info(int device, int *sm_count, size_t *total_mem, int *cc_major, int *cc_minor);

/* ---------------------------------------------------------------- streams */
/* A cudaStream_t stands where the reference passes `sycl::queue` plus a
 * `depends` event list (dpnp/tensor/_elementwise_common.py:692-700); work on
 * one stream is ordered, which is what SequentialOrderManager guarantees. */

int dpb_stream_create(void **stream);
int dpb_stream_destroy(void *stream);
int dpb_stream_synchronize(void *stream);
int dpb_device_synchronize(void);

/* CUDA events, used for timing by the measurement harness. */
int dpb_event_create(void **event);
int dpb_event_destroy(void *event);
int dpb_event_record(void *event, void *stream);
int dpb_event_synchronize(void *event);
/* Work queued on `stream` after this call waits for `event` (cudaStreamWaitEvent): the explicit
 * form of the `depends` event lists of the reference's calls, needed only between two queues. */
int dpb_stream_wait_event(void *stream, void *event);
int dpb_event_elapsed_ms(void *start, void *stop, float *ms);

/* ------------------------------------------------------------- allocator */
/* Stream-ordered pool (cudaMallocAsync on the device's default mempool with a
 * raised release threshold).  Replaces dpctl.memory.MemoryUSMDevice as used by
 * dpnp/tensor/_usmarray.pyx:440-448 and sycl::malloc_device for temporaries
 * (dpnp/tensor/libtensor/include/utils/sycl_alloc_utils.hpp:107-130).
 * Returned addresses are at least 256-byte aligned.  A zero-byte request
 * returns a unique non-NULL address. */

int dpb_malloc(size_t nbytes, void *stream, void **ptr);
/* Free is ordered after all work already enqueued on `stream`; this is what
 * keep_args_alive / async_smart_free achieve with host tasks in the reference
 * (dpnp/include/dpnp4pybind11.hpp:670-736; sycl_alloc_utils.hpp:185-222). */
int dpb_free(void *ptr, void *stream);
/* Release cached memory back to the driver down to `keep_bytes`. */
int dpb_pool_trim(size_t keep_bytes);
/* Guarded blocks, a debugging aid in place of a memory checker: with the "redzones" switch on
 * (dpb_set_tuning, or DPNP_B200_REDZONES=1 in the environment) every block handed out by
 * dpb_malloc carries 512 patterned bytes in front and behind, compared with the pattern when the
 * block is freed (both by small kernels on the block's stream; nothing traps).  This call waits
 * for the device, reports how many freed blocks / bytes were found overwritten since the last
 * report, and for the first of them {user pointer, user size, offset of the byte relative to the
 * block's start}, then clears the counters.  Writes that land farther than 512 bytes from a block
 * are not seen.  No counterpart in the reference. */
int dpb_debug_redzone_report(int64_t *bad_blocks, int64_t *bad_bytes, int64_t *first3);
/* Pool counters of the current device: bytes reserved from the driver and
 * bytes handed out, now and at the high-water mark. */
int dpb_pool_stats(size_t *reserved, size_t *used, size_t *reserved_high, size_t *used_high);
/* Optional cap on live bytes handed out by dpb_malloc (0 = no cap); a request
 * that would exceed it fails with DPB_ERR_MEMORY without touching the device.
 * Used to exercise out-of-memory handling from the host. */
int dpb_pool_set_limit(size_t max_live_bytes);

/* Pinned host memory for staging (cudaHostAlloc / cudaFreeHost). */
int dpb_host_alloc(size_t nbytes, void **ptr);
int dpb_host_free(void *ptr);

/* Raw copies; kind: 0 host->device, 1 device->host, 2 device->device.
 * Replaces the memcpy fast path of copy_usm_ndarray_into_usm_ndarray
 * (dpnp/tensor/libtensor/source/copy_and_cast_usm_to_usm.cpp:147-166) and the
 * host<->USM copies of dpnp/tensor/libtensor/source/copy_numpy_ndarray_into_usm_ndarray.cpp. */
int dpb_memcpy(void *dst, const void *src, size_t nbytes, int kind, void *stream);
/* Byte-wise memset. */
int dpb_memset(void *dst, int value, size_t nbytes, void *stream);

/* ----------------------------------------- iteration-space simplification */
/* Collapse an iteration space shared by `narrays` (1..4) arrays: dimensions
 * are sorted by decreasing |stride| (the LAST array's strides are the primary
 * key), dimensions whose strides are non-positive in every array and negative
 * in at least one are reversed (offsets absorb the shift), and neighbouring
 * dimensions whose strides chain in every array are merged.
 *   shape   : in/out, nd extents
 *   strides : in/out, narrays*nd values laid out [array][dim]
 *   offsets : out, narrays element offsets to add to the base pointers
 * Returns the new number of dimensions in *nd_out.
 * Replaces simplify_iteration_space_1/_/3/_4
 * (dpnp/tensor/libtensor/source/simplify_iteration_space.cpp:51-264) and
 * simplify_iteration_{stride,two_strides,three_strides,four_strides}
 * (dpnp/tensor/libtensor/include/utils/strided_iters.hpp:363-899). */
int dpb_simplify_iteration_space(int narrays, int nd, int64_t *shape, int64_t *strides,
                                 int64_t *offsets, int *nd_out);

/* Order-preserving merge of neighbouring dimensions of one array
 * (strided_iters.hpp:945-983, compact_iteration). */
int dpb_compact_iteration(int nd, int64_t *shape, int64_t *strides, int *nd_out);

/* True (1) if the byte ranges spanned by the two arrays intersect
 * (dpnp/tensor/libtensor/include/utils/memory_overlap.hpp:52-107). */
int dpb_array_overlap(const dpb_array *a, const dpb_array *b, int *overlap);
/* True (1) if both arrays have the same pointer, type, shape and strides
 * (memory_overlap.hpp:109-151). */
int dpb_same_logical_tensors(const dpb_array *a, const dpb_array *b, int *same);

/* ------------------------------------------------------ kernel-level ABI  */
/* These take raw pointers plus element offsets, as the reference's kernel
 * function-pointer types do (typeless pointer + offset).  `shape_strides` is a
 * HOST array laid out [shape | strides of arg 1 | ... | strides of result],
 * each nd long; it is copied into kernel parameters (the reference packs it
 * into a device buffer per call, include/utils/offset_utils.hpp:93-135). */

/* out[i] = op(in[i]); replaces unary_contig_impl_fn_ptr_t
 * (include/kernels/elementwise_functions/common.hpp:693-700). */
int dpb_unary_contig(int op, int t_in, int t_out, int64_t nelems, const void *in, int64_t in_off,
                     void *out, int64_t out_off, void *stream);
/* replaces unary_strided_impl_fn_ptr_t (common.hpp:702-713). */
int dpb_unary_strided(int op, int t_in, int t_out, int64_t nelems, int nd,
                      const int64_t *shape_strides, const void *in, int64_t in_off, void *out,
                      int64_t out_off, void *stream);
/* out[i] = op(a[i], b[i]); replaces binary_contig_impl_fn_ptr_t (common.hpp:715-727). */
int dpb_binary_contig(int op, int t_a, int t_b, int t_out, int64_t nelems, const void *a,
                      int64_t a_off, const void *b, int64_t b_off, void *out, int64_t out_off,
                      void *stream);
/* replaces binary_strided_impl_fn_ptr_t (common.hpp:729-744). */
int dpb_binary_strided(int op, int t_a, int t_b, int t_out, int64_t nelems, int nd,
                       const int64_t *shape_strides, const void *a, int64_t a_off, const void *b,
                       int64_t b_off, void *out, int64_t out_off, void *stream);
/* lhs[i] = op(lhs[i], rhs[i]); replaces binary_inplace_{contig,strided}_impl_fn_ptr_t
 * (include/kernels/elementwise_functions/common_inplace.hpp). `shape_strides`
 * is [shape | rhs strides | lhs strides]. */
int dpb_binary_inplace_contig(int op, int t_rhs, int t_lhs, int64_t nelems, const void *rhs,
                              int64_t rhs_off, void *lhs, int64_t lhs_off, void *stream);
int dpb_binary_inplace_strided(int op, int t_rhs, int t_lhs, int64_t nelems, int nd,
                               const int64_t *shape_strides, const void *rhs, int64_t rhs_off,
                               void *lhs, int64_t lhs_off, void *stream);
/* dst[i] = cond[i] ? x1[i] : x2[i]; replaces where_contig_impl_fn_ptr_t and
 * where_strided_impl_fn_ptr_t (include/kernels/where.hpp:163-170,264-277).
 * `shape_strides` is [shape | cond | x1 | x2 | dst]. */
int dpb_where_contig(int t_cond, int t_val, int64_t nelems, const void *cond, const void *x1,
                     const void *x2, void *dst, void *stream);
int dpb_where_strided(int t_cond, int t_val, int64_t nelems, int nd, const int64_t *shape_strides,
                      const void *cond, int64_t cond_off, const void *x1, int64_t x1_off,
                      const void *x2, int64_t x2_off, void *dst, int64_t dst_off, void *stream);
/* dst[i] = (T_dst) src[i]; replaces copy_and_cast_contig_fn_ptr_t /
 * copy_and_cast_generic_fn_ptr_t (include/kernels/copy_and_cast.hpp:90-208,225-389). */
int dpb_copy_cast_contig(int t_src, int t_dst, int64_t nelems, const void *src, int64_t src_off,
                         void *dst, int64_t dst_off, void *stream);
int dpb_copy_cast_strided(int t_src, int t_dst, int64_t nelems, int nd,
                          const int64_t *shape_strides, const void *src, int64_t src_off, void *dst,
                          int64_t dst_off, void *stream);

/* Reduction of a C-contiguous (iter_nelems x reduction_nelems) matrix along
 * its rows: res[i] = reduce_j arg[i*reduction_nelems + j].  Replaces
 * reduction_contig_impl_fn_ptr of reduction_axis1_over_group_{temps,with_atomics}_contig_impl
 * (include/kernels/reductions.hpp:859-958,1396-1624).  Deterministic: the
 * partition of the work depends only on the sizes. */
int dpb_reduce_axis1_contig(int op, int t_in, int t_out, int64_t iter_nelems,
                            int64_t reduction_nelems, const void *arg, int64_t arg_off, void *res,
                            int64_t res_off, void *stream);
/* Reduction along the rows' index of a C-contiguous (reduction_nelems x
 * iter_nelems) matrix: res[j] = reduce_i arg[i*iter_nelems + j].  Replaces
 * reduction_axis0_over_group_{temps,with_atomics}_contig_impl (reductions.hpp:961-1046,1626-1856). */
int dpb_reduce_axis0_contig(int op, int t_in, int t_out, int64_t iter_nelems,
                            int64_t reduction_nelems, const void *arg, int64_t arg_off, void *res,
                            int64_t res_off, void *stream);
/* General case.  iter_shape_strides = [shape | arg strides | res strides]
 * (iter_nd each); red_shape_strides = [shape | arg strides] (red_nd each).
 * Replaces reduction_strided_impl_fn_ptr (reductions.hpp:740-753,1137-1394). */
int dpb_reduce_strided(int op, int t_in, int t_out, int64_t iter_nelems, int64_t reduction_nelems,
                       const void *arg, void *res, int iter_nd, const int64_t *iter_shape_strides,
                       int64_t iter_arg_off, int64_t iter_res_off, int red_nd,
                       const int64_t *red_shape_strides, int64_t red_arg_off, void *stream);
/* Same result as dpb_reduce_axis1_contig for sum, max and min over rows of int32,
 * int64, float32 or float64 (plus int32 summed into int64), but the call obtains no
 * memory from CUDA or from the pool.  It exists for callers that may not allocate while
 * they run: code hosted by a framework whose own allocator already owns the device,
 * services held to a fixed memory budget, loops whose latency must not depend on the
 * pool growing.  It has no counterpart in the reference, whose reductions always take
 * their temporaries from sycl::malloc_device.
 *
 * Long rows are split over several blocks; their partial results go to a 64 KiB array
 * that is part of the library image (one copy per GPU that loads the library, held until
 * the process exits).  With the default launch geometry the partials of any shape fit
 * (at most about 2 * SMs * 8 of them, 16 bytes each).  A reduction whose partials would
 * not fit -- rows * splits * accumulator size > 64 KiB, which takes a raised
 * "ctas_per_sm" tuning value -- is refused with DPB_ERR_VALUE and a message naming both
 * sizes; unsupported type pairs give
 * DPB_ERR_RUNTIME.  The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current); make that first call before starting
 * any stream capture.  All calls share the one array, which keeps whatever the previous
 * call left there: nothing needs clearing, because every partial is written before it is
 * read, but two calls that overlap on the GPU (different streams) race on it.  The
 * address found on the first call is remembered per device ordinal (up to 64 devices) for
 * the life of the process; a program that calls cudaDeviceReset must not use this entry
 * point afterwards. */
int dpb_reduce_axis1_contig_noalloc(int op, int t_in, int t_out, int64_t iter_nelems,
                                    int64_t reduction_nelems, const void *arg, int64_t arg_off,
                                    void *res, int64_t res_off, void *stream);
/* Search reductions; result type is always int64, the index is the C-order
 * position inside the reduced sub-space, ties resolve to the smallest index
 * and a NaN is an extreme value.  Replaces search_axis1/axis0_over_group_temps_contig_impl
 * and search_over_group_temps_strided_impl (reductions.hpp:2487-3308). */
int dpb_search_axis1_contig(int op, int t_in, int64_t iter_nelems, int64_t reduction_nelems,
                            const void *arg, int64_t arg_off, void *res, int64_t res_off,
                            void *stream);
int dpb_search_axis0_contig(int op, int t_in, int64_t iter_nelems, int64_t reduction_nelems,
                            const void *arg, int64_t arg_off, void *res, int64_t res_off,
                            void *stream);
int dpb_search_strided(int op, int t_in, int64_t iter_nelems, int64_t reduction_nelems,
                       const void *arg, void *res, int iter_nd, const int64_t *iter_shape_strides,
                       int64_t iter_arg_off, int64_t iter_res_off, int red_nd,
                       const int64_t *red_shape_strides, int64_t red_arg_off, void *stream);

/* ---------------------------------------------------- dispatch-level ABI  */
/* These take array descriptors, validate them and choose the kernel, as the
 * reference's pybind11 dispatchers do.  Error conditions and messages follow
 * the reference (ValueError for type/shape/overlap/read-only/ample-memory
 * problems, RuntimeError for an unsupported type combination). */

/* Result type of op for the given argument types, or -1 if unsupported.
 * Replaces py_unary_ufunc_result_type / py_binary_ufunc_result_type
 * (source/elementwise_functions/elementwise_functions.hpp:255-285,566-603). */
int dpb_unary_result_type(int op, int t_in);
int dpb_binary_result_type(int op, int t_a, int t_b);

/* dst = op(src).  Replaces py_unary_ufunc (elementwise_functions.hpp:76-251). */
int dpb_unary_ufunc(int op, const dpb_array *src, const dpb_array *dst, void *stream);
/* dst = op(src1, src2).  Replaces py_binary_ufunc (elementwise_functions.hpp:305-563). */
int dpb_binary_ufunc(int op, const dpb_array *src1, const dpb_array *src2, const dpb_array *dst,
                     void *stream);
/* lhs = op(lhs, rhs).  Replaces py_binary_inplace_ufunc (elementwise_functions.hpp:611-804). */
int dpb_binary_inplace_ufunc(int op, const dpb_array *lhs, const dpb_array *rhs, void *stream);
/* dst = cond ? x1 : x2.  Replaces py_where (source/where.cpp:73-245). */
int dpb_where(const dpb_array *cond, const dpb_array *x1, const dpb_array *x2, const dpb_array *dst,
              void *stream);
/* dst[...] = cast(src[...]).  Replaces copy_usm_ndarray_into_usm_ndarray
 * (source/copy_and_cast_usm_to_usm.cpp:76-...). */
int dpb_copy_array_into_array(const dpb_array *src, const dpb_array *dst, void *stream);
/* dst = src / scalar, in the type of dst.  Replaces _divide_by_scalar
 * (source/elementwise_functions/true_divide.cpp:189-246,494). */
int dpb_divide_by_scalar(const dpb_array *src, double scalar, const dpb_array *dst, void *stream);
/* Fill with a scalar given as its bit pattern in the array's type (up to 16
 * bytes).  Replaces _full_usm_ndarray / _zeros_usm_ndarray (source/full_ctor.cpp, zeros_ctor.cpp). */
int dpb_full_array(const dpb_array *dst, const void *scalar_bits, void *stream);

/* Whether op has a kernel for the (input, output) type pair.  Replaces
 * _sum_over_axis_dtype_supported etc. (source/reductions/reduction_over_axis.hpp:72-134).
 * The set is a subset of the reference's (same results; unsupported pairs are
 * cast to a temporary by the caller, dpnp/tensor/_reduction.py:250-290). */
int dpb_reduce_dtype_supported(int op, int t_in, int t_out);
/* dst = reduce(src) over the last `trailing_dims_to_reduce` axes of src; the
 * caller has permuted the reduced axes to the end and dst has the shape of
 * the leading axes.  Replaces py_reduction_over_axis / py_tree_reduction_over_axis
 * (reduction_over_axis.hpp:173-501,507-777). */
int dpb_reduction_over_axis(int op, const dpb_array *src, int trailing_dims_to_reduce,
                            const dpb_array *dst, void *stream);
/* Replaces py_search_over_axis (reduction_over_axis.hpp:780-1047). */
int dpb_search_over_axis(int op, const dpb_array *src, int trailing_dims_to_reduce,
                         const dpb_array *dst, void *stream);

/* Inclusive scan of `src` along its last axis into `dst` (same rank; same shape, or one more
 * element along the last axis when include_initial is set: position 0 then holds the
 * identity).  Any strides; src and dst may be the same array.  Replaces
 * py_accumulate_over_axis and py_accumulate_final_axis_include_initial
 * (dpnp/tensor/libtensor/source/accumulators/accumulate_over_axis.hpp:74-260,262-460) with
 * trailing_dims_to_accumulate = 1, the only value the Python layer passes
 * (dpnp/tensor/_accumulation.py:140-152). */
int dpb_accumulate_over_axis(int op, const dpb_array *src, const dpb_array *dst, int include_initial,
                             void *stream);
/* 1 if (input type, output type) has a kernel for `op`, else 0
 * (_cumsum_over_axis_dtype_supported etc.). */
int dpb_accumulate_dtype_supported(int op, int t_in, int t_out);

/* ------------------------------------------------- fused expression paths */
/* Black-Scholes call/put for n options in one pass (3 loads, 2 stores per
 * option): the expression chain of examples/example_bs.py:50-75 with every
 * intermediate rounded exactly as the op-by-op chain rounds it, so the result
 * is bit-identical to running the chain through dpb_*_ufunc.  The reference
 * has no fused path (26 ufunc launches + 2 copies). */
int dpb_black_scholes_f64(int64_t n, const double *price, const double *strike, const double *t,
                          double rate, double vol, double *call, double *put, void *stream);

/* A fused elementwise chain as a register-machine program, evaluated per element by one
 * kernel.  The reference evaluates such chains one ufunc launch at a time through
 * DPNPUnaryFunc/DPNPBinaryFunc (dpnp/dpnp_algo/dpnp_elementwise_common.py:81-235,537-739);
 * Python scalars become operands of the program instead of stride-0 arrays
 * (dpnp/tensor/_elementwise_common.py:655-659).  Every operator is the one the per-op
 * entry points use, so a program gives the bits of the op-by-op chain.
 *
 * All arrays are contiguous, hold `n` elements of the program's type (float32 or
 * float64) and do not overlap; an input flagged in `in_is_scalar` holds one element that
 * is broadcast.  Comparisons and logical operators give 1.0 / 0.0, SELECT tests != 0.
 *
 * Instruction word: op | dst << 8 | a << 16 | b << 24 | c << 32 | swap << 40.  Operands
 * a, b, c: 0..63 register, 64+i immediate i, 128+i input array i (read where it is used, so
 * inputs need no LOAD and no register), 255 the result of the previous instruction.
 * A binary instruction computes op(a, b), or op(b, a) when swap is set (so that the
 * previous result can always be given as a, where the interpreter works in place).
 * dst: a register, or 255 when only the next instruction reads the result.
 * LOAD: a = input index.  STORE: a = operand, b = output index.  SELECT: a ? b : c. */
typedef enum dpb_fused_op {
    DPB_FUSED_LOAD = 0,
    DPB_FUSED_STORE,
    DPB_FUSED_SELECT,
    DPB_FUSED_MOVE,
    DPB_FUSED_POSITIVE,
    DPB_FUSED_NEGATIVE,
    DPB_FUSED_ABS,
    DPB_FUSED_EXP,
    DPB_FUSED_LOG,
    DPB_FUSED_SQRT,
    DPB_FUSED_ERF,
    DPB_FUSED_SQUARE,
    DPB_FUSED_RECIPROCAL,
    DPB_FUSED_SIN,
    DPB_FUSED_COS,
    DPB_FUSED_TANH,
    DPB_FUSED_EXPM1,
    DPB_FUSED_LOG1P,
    DPB_FUSED_FLOOR,
    DPB_FUSED_CEIL,
    DPB_FUSED_SIGN,
    DPB_FUSED_FIRST_BINARY,
    DPB_FUSED_ADD = DPB_FUSED_FIRST_BINARY,
    DPB_FUSED_SUBTRACT,
    DPB_FUSED_MULTIPLY,
    DPB_FUSED_DIVIDE,
    DPB_FUSED_MAXIMUM,
    DPB_FUSED_MINIMUM,
    DPB_FUSED_POW,
    DPB_FUSED_LESS,
    DPB_FUSED_LESS_EQUAL,
    DPB_FUSED_GREATER,
    DPB_FUSED_GREATER_EQUAL,
    DPB_FUSED_EQUAL,
    DPB_FUSED_NOT_EQUAL,
    DPB_FUSED_LOGICAL_AND,
    DPB_FUSED_LOGICAL_OR,
    DPB_FUSED_OP_COUNT
} dpb_fused_op;

typedef struct dpb_fused_program {
    int32_t typenum;             /* DPB_FLOAT or DPB_DOUBLE */
    int32_t n_instr;             /* <= 192 */
    int32_t n_reg;               /* registers the program uses, <= 24 */
    int32_t n_imm;               /* <= 48 */
    int32_t n_in;                /* <= 12 */
    int32_t n_out;               /* <= 8 */
    const uint64_t *code;        /* host memory, n_instr words */
    const double *imm;           /* host memory; converted to the program's type */
    const void *const *in;       /* device pointers */
    const int32_t *in_is_scalar; /* may be NULL: no scalar inputs */
    void *const *out;            /* device pointers */
} dpb_fused_program;

/* Runs the program over n elements with one launch.  DPB_ERR_VALUE for a malformed
 * program (every index is checked on the host before the launch). */
int dpb_fused_elementwise(const dpb_fused_program *prog, int64_t n, void *stream);

/* The same program as a kernel of its own: written out as straight-line CUDA C++ over the operator
 * classes of the per-op kernels (one statement per instruction, registers as local variables),
 * compiled with NVRTC at first use for the current device and kept for the life of the process
 * (keyed by type, instruction words and which inputs are single elements; the immediates and the
 * pointers are arguments of the kernel).  Same results, bit for bit, as dpb_fused_elementwise and
 * as the unfused chain.  NVRTC and the driver library are loaded with dlopen at first use;
 * DPB_ERR_RUNTIME (with the compiler's log in dpb_last_error) if they are missing or the
 * compilation fails.  No counterpart in the reference, which has no fusion. */
int dpb_fused_elementwise_specialized(const dpb_fused_program *prog, int64_t n, void *stream);
/* 1 if NVRTC, the driver library, the operator headers (directory csrc next to this library) and
 * the CUDA headers are all found, else 0. */
int dpb_fused_specialize_available(void);
/* Directories searched for headers by the run-time compilation, separated by ':' (the operator
 * headers, the stand-ins of csrc/rtc, the CUDA toolkit's include directory).  NULL or "" restores
 * the default: csrc/rtc and csrc next to this library, then $DPNP_B200_CUDA_INCLUDE,
 * $CUDA_HOME/include, $CUDA_PATH/include or /usr/local/cuda/include. */
int dpb_fused_set_include_path(const char *colon_separated);
/* The generated source (NUL-terminated, cut to buf_len); *needed = bytes for all of it.  No device
 * is involved. */
int dpb_fused_specialized_source(const dpb_fused_program *prog, char *buf, int64_t buf_len, int64_t *needed);
/* Compiles the program without loading or launching it (no device needed: sm_100a is assumed when
 * there is none); *cubin_bytes = size of the device code. */
int dpb_fused_specialize_compile(const dpb_fused_program *prog, int64_t *cubin_bytes);

/* ------------------------------------------------------- device-side fill */
/* Counter-based uniform generator: element i of the output depends only on
 * (seed, i), so any shard of an array can be produced independently.
 * Floating types get lo + (hi-lo)*u with u in [0,1); integer types get
 * uniformly distributed integers in [lo, hi).  Stands in for the device-side
 * generation of dpnp.random.uniform (dpnp/random/dpnp_iface_random.py:1965-2033),
 * whose oneMKL streams are not reproducible elsewhere either. */
int dpb_random_uniform(int typenum, void *dst, int64_t nelems, double lo, double hi, uint64_t seed,
                       uint64_t first_index, void *stream);
/* Standard normal variates (Box-Muller on the same counter-based stream). */
int dpb_random_normal(int typenum, void *dst, int64_t nelems, double mean, double stddev,
                      uint64_t seed, uint64_t first_index, void *stream);

/* Linear sequences written on the device into a contiguous array of `nelems` elements.
 * `start`, `step`, `end` point to host values of the array's type.
 * dpb_linspace_step: dst[i] = start + i*step, integers wrap (lin_space_step_impl,
 * dpnp/tensor/libtensor/include/kernels/constructors.hpp:65-131; any real type).
 * dpb_linspace_affine: dst[i] = start*(den-i)/den + end*i/den with den = nelems-1 when the
 * end point is included, else nelems (lin_space_affine_impl, constructors.hpp:136-246;
 * floating types). */
int dpb_linspace_step(int typenum, void *dst, int64_t nelems, const void *start, const void *step,
                      void *stream);
int dpb_linspace_affine(int typenum, void *dst, int64_t nelems, const void *start, const void *end,
                        int include_endpoint, void *stream);

/* dst[0] = src[index[0]] with the int64 index read on the device (clamped to the array): turns the
 * result of a flattened argmax/argmin into its value without a host round trip.  The reference
 * reads such an element through usm_ndarray.__getitem__ and a device-to-host copy
 * (dpnp/tensor/_usmarray.pyx: __getitem__, _copy_utils.py:_copy_to_numpy). */
int dpb_take_one(int typenum, const void *src, int64_t nelems, const void *index, void *dst, void *stream);

/* Measurement aid for the FP64-bound fused kernels: launches SMs x blocks_per_sm blocks of 256
 * threads that each issue iters x 8 independent double-precision fused multiply-adds, and
 * reports how many were issued in all; timed by the caller with events, it gives the FP64 FMA
 * rate the device sustains.  `scratch` receives one double per thread.  No counterpart in the
 * reference. */
int dpb_probe_fp64_fma(int64_t iters, int blocks_per_sm, double *scratch, int64_t scratch_elems,
                       int64_t *fma_count, void *stream);

/* ------------------------------------------- multi-GPU: combining partials */
/* One process per GPU; arrays are sharded along their leading axis.  The reference has no
 * multi-device execution -- an array and every operation on it are tied to one queue
 * (dpnp/tensor/_compute_follows_data.pyx:67-160, dpnp/tensor/_usmarray.pyx:1113-1191) -- so
 * these entry points replace nothing; they are what a sharded reduction needs after each GPU
 * has reduced its own shard with dpb_reduction_over_axis / dpb_search_over_axis.  NCCL is
 * loaded at run time (dlopen); every call is enqueued on `stream`; no kernel of this library
 * waits on another GPU. */

/* Load NCCL from `libnccl_path` (NULL or "": the loader's default libnccl.so.2). */
int dpb_comm_load(const char *libnccl_path);
/* Version code of the loaded NCCL (ncclGetVersion). */
int dpb_comm_nccl_version(int *version);
/* 128-byte id created by rank 0 (ncclGetUniqueId); the caller hands it to the other ranks. */
int dpb_comm_unique_id(void *id128);
/* Communicator of `world` ranks on the current device (ncclCommInitRank); world == 1 needs
 * neither NCCL nor an id.  Errors: rank outside the group, missing id, NCCL failures. */
int dpb_comm_init(int rank, int world, const void *id128, void **comm);
int dpb_comm_destroy(void *comm);
int dpb_comm_info(void *comm, int *rank, int *world);
/* Peer mailboxes: where every rank's GPU can map the others' memory (one box, NVLink), the combines
 * below exchange their payloads (up to 256 KiB per rank) and fold them in ONE kernel per rank --
 * stores into the peers' mailboxes, a flag per rank, a bounded wait, the fold in rank order --
 * instead of an NCCL all-gather followed by a kernel.  Set-up, once per communicator:
 *   dpb_comm_peer_export  allocates this rank's mailbox and returns its inter-process handle
 *                         (*handle_bytes = size of a handle, 64);
 *   (the caller makes every rank's handle known to every rank: an all-gather over its host group)
 *   dpb_comm_peer_attach  maps the ranks' mailboxes from the `count` = world handles, in rank order;
 *   dpb_comm_peer_enable  switches the combines over (every rank must make the same choice, so the
 *                         caller agrees on it first: all ranks attached successfully, or none uses it).
 * A wait that runs out ("peer_polls" probes, dpb_set_tuning) makes the kernel raise an error word in
 * pinned host memory and return; every later combine of the communicator fails with
 * DPB_ERR_RUNTIME.  dpb_comm_peer_probe_wait runs that bounded wait on a flag nobody sets and
 * reports whether it gave up (*timed_out = 1): the test of the give-up path.  No counterpart in
 * the reference. */
int dpb_comm_peer_export(void *comm, void *handle, int64_t handle_capacity, int64_t *handle_bytes);
int dpb_comm_peer_attach(void *comm, const void *handles, int count);
int dpb_comm_peer_enable(void *comm, int on);
int dpb_comm_peer_probe_wait(void *comm, int64_t polls, int *timed_out, void *stream);
/* recv[r * nbytes ...] = rank r's send buffer (device memory, nbytes per rank). */
int dpb_comm_allgather(void *comm, const void *send, void *recv, int64_t nbytes, void *stream);
/* out[i] = partial_0[i] + partial_1[i] + ... in rank order, identical bits on every rank:
 * all-gather into the communicator's gather buffer, then one kernel. */
int dpb_comm_sum_ordered(void *comm, int typenum, const void *partial, void *out, int64_t count,
                         void *stream);
/* out[i] = max / min over ranks of partial_r[i], NaN propagating as in the reductions. */
int dpb_comm_extreme(void *comm, int typenum, int is_max, const void *partial, void *out,
                     int64_t count, void *stream);
/* Global argmax / argmin of a flattened sharded array.  `src` is this rank's shard (`nelems`
 * elements, may be 0), `local_index` the device int64 holding the position of its extreme
 * (result of dpb_search_over_axis), `index_offset` the flat index of the shard's first element
 * in the whole array.  Writes the winning value to `out_value` (element of `typenum`) and its
 * global flat index to `out_index` (int64), both in device memory; either may be NULL.  Rule:
 * better value; equal values -> smaller index; NaN is extreme.  A rank with an empty shard
 * takes part in the exchange and contributes nothing. */
int dpb_comm_arg_extreme(void *comm, int typenum, int is_max, const void *src, int64_t nelems,
                         const void *local_index, int64_t index_offset, void *out_value,
                         void *out_index, void *stream);

/* --------------------------------------------------------- introspection  */
/* Name of the kernel family chosen by the most recent dispatch-level call in
 * this thread ("binary_contig_vec", "strided_rows", "transpose_tile", ...),
 * and the number of kernel launches issued by this thread since the last
 * dpb_reset_launch_count(). */
const char *dpb_last_kernel(void);
int64_t dpb_launch_count(void);
void dpb_reset_launch_count(void);
/* Run-time switches; DPB_ERR_VALUE for unknown keys or values out of range.
 *   "ctas_per_sm" (1..64)              resident blocks per SM assumed when sizing grids
 *   "fused_elems_per_thread" (4 | 8)   elements per thread of the fused-chain interpreter
 *   "pdl" (0 | 1)                      contiguous elementwise kernels are launched with programmatic
 *                                      stream serialisation (the launch overlaps the previous kernel's
 *                                      tail; the kernel waits for that kernel before it reads); default 1
 *   "peer_polls" (0 .. 2^24)           probes per wait of the peer-mailbox exchange of the combines
 *                                      (default 2^24, the largest value: about half a minute -- the bound is
 *                                      there for a rank that died, not for one that is late)
 *   "scan_lookback_polls" (-1 .. 2^30) probes per wait of the single-pass scan of long rows before a
 *                                      tile gives up and is redone by the repair launches (0 makes
 *                                      every wait that is not satisfied at once give up -- a test of
 *                                      the repair path); -1 (default): long rows take the
 *                                      three-launch scan instead
 *   "verbose" (0 | 1)                  log every kernel choice on stderr; initial value from the
 *                                      environment variable DPNP_B200_VERBOSE
 *   "redzones" (0 | 1)                 guarded pool blocks, see dpb_debug_redzone_report; initial value
 *                                      from DPNP_B200_REDZONES
 *   "force_generic" (0 | 1)            route every elementwise and reduction call to the generic
 *                                      strided kernels (a debugging aid: results do not change);
 *                                      initial value from DPNP_B200_FORCE_GENERIC
 * They stand where the reference reads its environment (dpnp/config.py:32-59). */
int dpb_set_tuning(const char *key, int64_t value);

#ifdef __cplusplus
}
#endif
#endif /* DPNP_B200_H */

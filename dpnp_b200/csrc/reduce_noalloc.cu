// Row reduction that allocates nothing.
//
// Some programs that load this library are not allowed to ask CUDA for memory
// while they run: a plug-in living inside a framework that has already claimed
// the whole device for its own allocator, a service working under a fixed
// memory contract, or a loop whose timing must not depend on whether the pool
// has to grow.  For them dpb_reduce_axis1_contig_noalloc does what
// dpb_reduce_axis1_contig does for long rows split over several blocks, but
// parks the per-block partial results in a buffer that is part of the library
// image instead of one taken from the pool.
//
// The buffer is a file-scope __device__ array of kScratchBytes bytes.  Every GPU
// that loads the library holds one copy until the process exits.  Host code
// cannot use the array's name as a pointer (on the host the name only stands
// for the symbol), so the device address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and that address is what
// the kernels receive.
#include <mutex>

#include "reduce_launch.cuh"

namespace dpb {

// 64 KiB: at the default launch geometry (8 blocks per SM) a split reduction keeps at most
// about 2 * 148 * 8 partials of up to 16 bytes, i.e. under 38 KiB
constexpr size_t kScratchBytes = size_t(64) << 10;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kScratchDevices = 64;
static void *g_scratch_addr[kScratchDevices] = {};
static std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device (looked up on first use).
static int scratch_address(void **out)
{
    int dev = 0;
    DPB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kScratchDevices)
        return set_error(DPB_ERR_RUNTIME, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
        void *p = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (err != cudaSuccess || !p) {
            cudaGetLastError();
            return set_error(DPB_ERR_CUDA, "cudaGetSymbolAddress for the built-in scratch failed: %s",
                             cudaGetErrorString(err));
        }
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return DPB_OK;
}

// Same partition as the pooled path: rows shorter than 16384 elements, or enough
// rows to fill the GPU, are reduced in one pass and need no scratch at all.
template <class R>
static int reduce_rows_noalloc(int64_t nrows, int64_t L, const void *arg, void *res, cudaStream_t stream)
{
    using In = typename R::In;
    using Acc = typename R::Acc;
    const int64_t ish = nrows, isrc = L, idst = 1;
    RedMeta iter = make_meta(1, &ish, &isrc, &idst);
    const In *a = static_cast<const In *>(arg);
    if (L == 0) {
        reduce_identity_kernel<R><<<red_grid(ceil_div(nrows, 256)), 256, 0, stream>>>(
            static_cast<typename R::Out *>(res), iter, nrows);
        note_kernel("reduce_identity");
        return check_launch("reduce_identity");
    }
    int64_t nsplit = 1, chunk = L;
    const int64_t target = red_target_blocks();
    if (L > 16384 && nrows < target) {
        nsplit = std::min<int64_t>(ceil_div(target, nrows), L / 8192);
        nsplit = std::max<int64_t>(1, std::min<int64_t>(nsplit, 2048));
        chunk = ceil_div(ceil_div(L, nsplit), 1024) * 1024;
        nsplit = ceil_div(L, chunk);
    }
    if (nsplit <= 1) return launch_inner<R>(a, res, iter, nrows, L, 1, L, true, stream);

    const size_t need = static_cast<size_t>(nrows) * static_cast<size_t>(nsplit) * sizeof(Acc);
    if (need > kScratchBytes)
        return set_error(DPB_ERR_VALUE,
                         "this reduction needs %zu bytes of scratch but the built-in buffer holds %zu; "
                         "use dpb_reduce_axis1_contig (which takes scratch from the pool) instead",
                         need, kScratchBytes);
    void *scratch = nullptr;
    DPB_TRY(scratch_address(&scratch));
    // pass 1 writes every partial it will read in pass 2, so nothing has to be cleared first
    DPB_TRY(launch_inner<R>(a, scratch, iter, nrows, L, nsplit, chunk, false, stream));
    const int64_t s2 = nsplit;
    RedMeta iter2 = make_meta(1, &ish, &s2, &idst);
    return launch_inner<typename R::Stage2>(static_cast<const Acc *>(scratch), res, iter2, nrows, nsplit, 1,
                                            nsplit, true, stream);
}

}  // namespace dpb

using namespace dpb;

extern "C" int dpb_reduce_axis1_contig_noalloc(int op, int t_in, int t_out, int64_t iter_nelems,
                                               int64_t reduction_nelems, const void *arg, int64_t arg_off,
                                               void *res, int64_t res_off, void *stream)
{
    if (iter_nelems < 0 || reduction_nelems < 0) return set_error(DPB_ERR_VALUE, "negative size");
    if (iter_nelems == 0) return DPB_OK;
    if (!arg || !res) return set_error(DPB_ERR_VALUE, "null pointer");
    const char *a = static_cast<const char *>(arg) + arg_off * type_size(t_in);
    char *r = static_cast<char *>(res) + res_off * type_size(t_out);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t n = iter_nelems, L = reduction_nelems;
#define DPB_NOALLOC_CASE(OP, TI, TO, ...) \
    if (op == OP && t_in == TI && t_out == TO) return reduce_rows_noalloc<__VA_ARGS__>(n, L, a, r, s);
    DPB_NOALLOC_CASE(DPB_R_SUM, DPB_FLOAT, DPB_FLOAT, SumRed<float, float>)
    DPB_NOALLOC_CASE(DPB_R_SUM, DPB_DOUBLE, DPB_DOUBLE, SumRed<double, double>)
    DPB_NOALLOC_CASE(DPB_R_SUM, DPB_INT32, DPB_INT32, SumRed<int32_t, int32_t>)
    DPB_NOALLOC_CASE(DPB_R_SUM, DPB_INT32, DPB_INT64, SumRed<int32_t, int64_t>)
    DPB_NOALLOC_CASE(DPB_R_SUM, DPB_INT64, DPB_INT64, SumRed<int64_t, int64_t>)
    DPB_NOALLOC_CASE(DPB_R_MAX, DPB_FLOAT, DPB_FLOAT, ExtremeRed<true, float, float>)
    DPB_NOALLOC_CASE(DPB_R_MAX, DPB_DOUBLE, DPB_DOUBLE, ExtremeRed<true, double, double>)
    DPB_NOALLOC_CASE(DPB_R_MAX, DPB_INT32, DPB_INT32, ExtremeRed<true, int32_t, int32_t>)
    DPB_NOALLOC_CASE(DPB_R_MAX, DPB_INT64, DPB_INT64, ExtremeRed<true, int64_t, int64_t>)
    DPB_NOALLOC_CASE(DPB_R_MIN, DPB_FLOAT, DPB_FLOAT, ExtremeRed<false, float, float>)
    DPB_NOALLOC_CASE(DPB_R_MIN, DPB_DOUBLE, DPB_DOUBLE, ExtremeRed<false, double, double>)
    DPB_NOALLOC_CASE(DPB_R_MIN, DPB_INT32, DPB_INT32, ExtremeRed<false, int32_t, int32_t>)
    DPB_NOALLOC_CASE(DPB_R_MIN, DPB_INT64, DPB_INT64, ExtremeRed<false, int64_t, int64_t>)
#undef DPB_NOALLOC_CASE
    return set_error(DPB_ERR_RUNTIME,
                     "the allocation-free reduction covers sum/max/min of int32, int64, float32 and "
                     "float64 rows (got op %d, %s -> %s)", op, type_name(t_in), type_name(t_out));
}

// Fused Black-Scholes call/put pricing: the 26-operation elementwise chain of
// examples/example_bs.py:50-75 evaluated in registers, 3 loads and 2 stores per
// option.  Every intermediate is rounded exactly where the op-by-op chain
// rounds it (the library is compiled without multiply-add contraction), so the
// output equals the chain's bit for bit.
#include <algorithm>

#include "common.cuh"
#include "ew_erf.cuh"

namespace dpb {

DPB_D void bs_one(double P, double S, double T, double mr, double sst, double &call, double &put)
{
    const double a = log(P / S);
    const double b = T * mr;
    const double z = T * sst;
    const double c = 0.25 * z;
    const double y = 1.0 / sqrt(z);
    const double w1 = (a - b + c) * y;
    const double w2 = (a - b - c) * y;
    const double d1 = 0.5 + 0.5 * erf_f64(w1);
    const double d2 = 0.5 + 0.5 * erf_f64(w2);
    const double Se = exp(b) * S;
    const double r = P * d1 - Se * d2;
    call = r;
    put = r - P + Se;
}

constexpr int kBsThreads = 256;

// VEC doubles per 16-byte access (2, or 1 for unaligned arrays).  One access per thread and array:
// keeping 2 or 4 accesses in flight per thread was measured slower (more registers, fewer resident
// warps; the FP64 pipe is already kept busy by the warps of the other resident blocks).
template <int VEC>
__global__ void __launch_bounds__(kBsThreads)
    black_scholes_kernel(const double *__restrict__ price, const double *__restrict__ strike,
                         const double *__restrict__ t, double mr, double sst,
                         double *__restrict__ call, double *__restrict__ put, int64_t n)
{
    const int64_t nvec = n / VEC;
    const int64_t stride = int64_t(gridDim.x) * kBsThreads;
    for (int64_t v = int64_t(blockIdx.x) * kBsThreads + threadIdx.x; v < nvec; v += stride) {
        vec_t<double, VEC> p = load_vec<vec_t<double, VEC>>(price + v * VEC);
        vec_t<double, VEC> s = load_vec<vec_t<double, VEC>>(strike + v * VEC);
        vec_t<double, VEC> tt = load_vec<vec_t<double, VEC>>(t + v * VEC);
        vec_t<double, VEC> c, q;
#pragma unroll
        for (int k = 0; k < VEC; ++k) bs_one(p.v[k], s.v[k], tt.v[k], mr, sst, c.v[k], q.v[k]);
        store_vec(call + v * VEC, c);
        store_vec(put + v * VEC, q);
    }
    if (blockIdx.x == 0) {
        for (int64_t i = nvec * VEC + threadIdx.x; i < n; i += kBsThreads)
            bs_one(price[i], strike[i], t[i], mr, sst, call[i], put[i]);
    }
}

// Measures what the FP64 pipe can issue: every thread runs `iters` rounds of 8 independent
// fused multiply-adds (explicit fma(): the library is built without contraction).  The sum of
// the accumulators is stored so that nothing is optimised away.
__global__ void __launch_bounds__(256) fp64_fma_probe_kernel(int64_t iters, double seed, double *out)
{
    double a0 = seed + threadIdx.x, a1 = a0 + 1, a2 = a0 + 2, a3 = a0 + 3, a4 = a0 + 4, a5 = a0 + 5, a6 = a0 + 6,
           a7 = a0 + 7;
    const double m = 0.999999, c = 1e-9;
    for (int64_t i = 0; i < iters; ++i) {
        a0 = fma(a0, m, c);
        a1 = fma(a1, m, c);
        a2 = fma(a2, m, c);
        a3 = fma(a3, m, c);
        a4 = fma(a4, m, c);
        a5 = fma(a5, m, c);
        a6 = fma(a6, m, c);
        a7 = fma(a7, m, c);
    }
    out[int64_t(blockIdx.x) * blockDim.x + threadIdx.x] = ((a0 + a1) + (a2 + a3)) + ((a4 + a5) + (a6 + a7));
}

}  // namespace dpb

using namespace dpb;

extern "C" int dpb_probe_fp64_fma(int64_t iters, int blocks_per_sm, double *scratch, int64_t scratch_elems,
                                  int64_t *fma_count, void *stream)
{
    if (iters < 1 || blocks_per_sm < 1 || blocks_per_sm > 8 || !scratch)
        return set_error(DPB_ERR_VALUE, "dpb_probe_fp64_fma: bad arguments");
    const int64_t blocks = int64_t(device_props().sm_count) * blocks_per_sm;
    if (scratch_elems < blocks * 256) return set_error(DPB_ERR_VALUE, "dpb_probe_fp64_fma: scratch of %lld elements needed",
                                                       static_cast<long long>(blocks * 256));
    fp64_fma_probe_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(iters, 1.0, scratch);
    if (fma_count) *fma_count = blocks * 256 * iters * 8;
    note_kernel("fp64_fma_probe");
    return check_launch("fp64_fma_probe");
}

extern "C" int dpb_black_scholes_f64(int64_t n, const double *price, const double *strike,
                                     const double *t, double rate, double vol, double *call,
                                     double *put, void *stream)
{
    if (n < 0) return set_error(DPB_ERR_VALUE, "negative size");
    if (n == 0) return DPB_OK;
    if (!price || !strike || !t || !call || !put) return set_error(DPB_ERR_VALUE, "null pointer");
    const double mr = -rate;
    const double sst = vol * vol * 2;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool aligned = is_aligned(price, 16) && is_aligned(strike, 16) && is_aligned(t, 16) &&
                         is_aligned(call, 16) && is_aligned(put, 16);
    const int64_t cap = int64_t(device_props().sm_count) * tuning_ctas_per_sm();
    if (aligned) {
        const int64_t blocks = std::max<int64_t>(1, std::min(cap, ceil_div(n / 2, kBsThreads)));
        black_scholes_kernel<2><<<static_cast<int>(blocks), kBsThreads, 0, s>>>(price, strike, t, mr, sst, call, put, n);
    }
    else {
        const int64_t blocks = std::max<int64_t>(1, std::min(cap, ceil_div(n, kBsThreads)));
        black_scholes_kernel<1><<<static_cast<int>(blocks), kBsThreads, 0, s>>>(price, strike, t, mr, sst, call, put, n);
    }
    note_kernel("black_scholes_f64");
    return check_launch("black_scholes_f64");
}

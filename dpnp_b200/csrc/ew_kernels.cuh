// Elementwise engine: kernel templates and their typed launcher.
//
// A functor F describes one elementwise operation:
//   F::NIN            number of inputs (0..3)
//   F::In0/In1/In2    input element types (unused ones are char)
//   F::Out            output element type
//   Out operator()(In0[, In1[, In2]]) const
// Four kernel families serve every F:
//   ew_contig_vec / ew_contig_scalar  contiguous operands (any input may be a
//                                     broadcast scalar), 16-byte accesses when
//                                     every pointer allows it
//   ew_rows        innermost dimension unit-stride (or broadcast) in every
//                  operand, outer dimensions arbitrary
//   ew_transpose   one or more inputs contiguous along a different dimension
//                  than the output: 32x32 shared-memory tile
//   ew_generic     anything else: one element per thread-iteration, collapsed
//                  shape/strides in kernel parameters, multiply-shift division
//
// These replace the reference's Unary/Binary Contig and Strided functors and
// launchers (dpnp/tensor/libtensor/include/kernels/elementwise_functions/common.hpp:64-273,
// 302-389,398-558,779-884), the where kernels (include/kernels/where.hpp:67-313) and the
// copy/cast kernels (include/kernels/copy_and_cast.hpp:90-389).
#pragma once

#include <algorithm>

#include "common.cuh"
#include "ew_plan.h"

namespace dpb {

constexpr int kEwThreads = 256;

template <class F> struct EwPtrs {
    const void *in[3];
    void *out;
};

template <int NARR> struct StridedMeta {
    int nd;
    int64_t shape[kMaxD];
    int64_t strides[NARR][kMaxD];
    FastDiv32 div[kMaxD];
};

template <class F, class A, class B, class C>
DPB_D typename F::Out ew_apply(const F &f, A a, B b, C c)
{
    if constexpr (F::NIN == 0) return f();
    else if constexpr (F::NIN == 1) return f(a);
    else if constexpr (F::NIN == 2) return f(a, b);
    else return f(a, b, c);
}

template <class F> constexpr int ew_vec_width()
{
    if constexpr (F::NIN == 0) return vec_width<typename F::Out>();
    else if constexpr (F::NIN == 1) return vec_width<typename F::In0, typename F::Out>();
    else if constexpr (F::NIN == 2)
        return vec_width<typename F::In0, typename F::In1, typename F::Out>();
    else return vec_width<typename F::In0, typename F::In1, typename F::In2, typename F::Out>();
}

// 16-byte accesses per thread of the contiguous kernel for one streamed input: 8 unless the
// functor names its own (kUnroll)
template <class F, class = void> struct ew_unroll { static constexpr int value = 8; };
template <class F> struct ew_unroll<F, std::void_t<decltype(F::kUnroll)>> { static constexpr int value = F::kUnroll; };

// ------------------------------------------------------------- contiguous
// Tile = 256 threads x VEC elements x UNROLL vectors, one tile per block (the
// kernel keeps a stride loop so a capped grid still covers any size); the ragged
// end is handled element-wise by one block.  BMASK names, at compile time, the
// inputs that are a single broadcast element: they cost one register instead of
// a stream, which leaves room for a deeper unroll of the remaining stream.
template <class F, int VEC, int UNROLL, unsigned BMASK>
__global__ void __launch_bounds__(kEwThreads)
    ew_contig_vec_kernel(F f, EwPtrs<F> p, int64_t n)
{
    // launched with programmatic stream serialisation (launch_after_previous): the grid may be
    // set up while the previous kernel of the stream drains; nothing is read before this returns
    cudaGridDependencySynchronize();
    using In0 = typename F::In0;
    using In1 = typename F::In1;
    using In2 = typename F::In2;
    using Out = typename F::Out;
    constexpr int64_t TILE = int64_t(kEwThreads) * VEC * UNROLL;
    constexpr bool S0 = F::NIN >= 1 && !(BMASK & 1u);  // input k streams from memory
    constexpr bool S1 = F::NIN >= 2 && !(BMASK & 2u);
    constexpr bool S2 = F::NIN >= 3 && !(BMASK & 4u);
    const In0 *a = static_cast<const In0 *>(p.in[0]);
    const In1 *b = static_cast<const In1 *>(p.in[1]);
    const In2 *c = static_cast<const In2 *>(p.in[2]);
    Out *o = static_cast<Out *>(p.out);

    In0 sa{};
    In1 sb{};
    In2 sc{};
    if constexpr (F::NIN >= 1 && !S0) sa = a[0];
    if constexpr (F::NIN >= 2 && !S1) sb = b[0];
    if constexpr (F::NIN >= 3 && !S2) sc = c[0];

    const int64_t ntiles = n / TILE;
    for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const int64_t base = t * TILE + int64_t(threadIdx.x) * VEC;
        vec_t<In0, VEC> va[S0 ? UNROLL : 1];
        vec_t<In1, VEC> vb[S1 ? UNROLL : 1];
        vec_t<In2, VEC> vc[S2 ? UNROLL : 1];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t i = base + int64_t(u) * kEwThreads * VEC;
            if constexpr (S0) va[u] = load_vec<vec_t<In0, VEC>>(a + i);
            if constexpr (S1) vb[u] = load_vec<vec_t<In1, VEC>>(b + i);
            if constexpr (S2) vc[u] = load_vec<vec_t<In2, VEC>>(c + i);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t i = base + int64_t(u) * kEwThreads * VEC;
            vec_t<Out, VEC> r;
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                In0 x = sa;
                In1 y = sb;
                In2 z = sc;
                if constexpr (S0) x = va[u].v[k];
                if constexpr (S1) y = vb[u].v[k];
                if constexpr (S2) z = vc[u].v[k];
                r.v[k] = ew_apply(f, x, y, z);
            }
            store_vec(o + i, r);
        }
    }
    if (blockIdx.x == static_cast<unsigned>(ntiles % gridDim.x)) {
        for (int64_t i = ntiles * TILE + threadIdx.x; i < n; i += kEwThreads) {
            In0 x = sa;
            In1 y = sb;
            In2 z = sc;
            if constexpr (S0) x = a[i];
            if constexpr (S1) y = b[i];
            if constexpr (S2) z = c[i];
            o[i] = ew_apply(f, x, y, z);
        }
    }
}

// ------------------------------------------------------------------- rows
// The innermost collapsed dimension (length L) has stride 0 or 1 in every
// operand; `outer` describes the remaining dimensions.  A block is TX threads
// along the row times TY rows; a work item is (row group, chunk of the row).
// IB >= 0: the broadcast mask of the innermost dimension is the compile-time value IB, so a
// chunk that lies wholly inside the row issues all its loads before the first use.
template <class F, int VEC, int UNROLL, int IB>
__global__ void __launch_bounds__(kEwThreads, 5)
    ew_rows_kernel(F f, EwPtrs<F> p, StridedMeta<F::NIN + 1> outer, int64_t L, unsigned inner_bcast,
                   int64_t nrows, int tx_log2, int64_t chunks_per_row, int64_t nwork, FastDiv32 chunk_div,
                   int head)
{
    cudaGridDependencySynchronize();   // see launch_after_previous
    using In0 = typename F::In0;
    using In1 = typename F::In1;
    using In2 = typename F::In2;
    using Out = typename F::Out;
    constexpr int NARR = F::NIN + 1;
    const int TX = 1 << tx_log2;
    const int TY = kEwThreads >> tx_log2;
    const int tx = threadIdx.x & (TX - 1);
    const int ty = threadIdx.x >> tx_log2;

    for (int64_t w = blockIdx.x; w < nwork; w += gridDim.x) {
        // 31-bit multiply-shift division when the work count allows it
        const int64_t rg = (nwork < (int64_t(1) << 31)) ? int64_t(chunk_div.div(static_cast<uint32_t>(w)))
                                                         : w / chunks_per_row;
        const int64_t chunk = w - rg * chunks_per_row;
        const int64_t row = rg * TY + ty;
        if (row >= nrows) continue;
        // row -> offsets of the row start in every array
        int64_t off[NARR];
#pragma unroll
        for (int k = 0; k < NARR; ++k) off[k] = 0;
        {
            uint32_t rem = static_cast<uint32_t>(row);
            for (int d = outer.nd - 1; d >= 0; --d) {
                uint32_t q, r;
                outer.div[d].divmod(rem, q, r);
                rem = q;
#pragma unroll
                for (int k = 0; k < NARR; ++k) off[k] += int64_t(r) * outer.strides[k][d];
            }
        }
        const In0 *a = static_cast<const In0 *>(p.in[0]) + (F::NIN >= 1 ? off[0] : 0);
        const In1 *b = static_cast<const In1 *>(p.in[1]) + (F::NIN >= 2 ? off[1] : 0);
        const In2 *c = static_cast<const In2 *>(p.in[2]) + (F::NIN >= 3 ? off[2] : 0);
        Out *o = static_cast<Out *>(p.out) + off[NARR - 1];

        In0 sa{};
        In1 sb{};
        In2 sc{};
        if constexpr (F::NIN >= 1) { if (inner_bcast & 1u) sa = a[0]; }
        if constexpr (F::NIN >= 2) { if (inner_bcast & 2u) sb = b[0]; }
        if constexpr (F::NIN >= 3) { if (inner_bcast & 4u) sc = c[0]; }

        // Rows that start `VEC - head` elements past a 16-byte boundary in every operand:
        // the first `head` elements go one by one, the rest is on the vector grid.
        if (head) {
            if (chunk == 0) {
                for (int e = tx; e < head; e += TX) {
                    In0 x = sa;
                    In1 y = sb;
                    In2 z = sc;
                    if constexpr (F::NIN >= 1) { if (!(inner_bcast & 1u)) x = a[e]; }
                    if constexpr (F::NIN >= 2) { if (!(inner_bcast & 2u)) y = b[e]; }
                    if constexpr (F::NIN >= 3) { if (!(inner_bcast & 4u)) z = c[e]; }
                    o[e] = ew_apply(f, x, y, z);
                }
            }
            if constexpr (F::NIN >= 1) { if (!(inner_bcast & 1u)) a += head; }
            if constexpr (F::NIN >= 2) { if (!(inner_bcast & 2u)) b += head; }
            if constexpr (F::NIN >= 3) { if (!(inner_bcast & 4u)) c += head; }
            o += head;
        }
        const int64_t Lb = L - head;

        const int64_t v0 = chunk * (int64_t(TX) * UNROLL) + tx;  // first vector index
        if constexpr (IB >= 0) {
            constexpr bool S0 = F::NIN >= 1 && !(IB & 1), S1 = F::NIN >= 2 && !(IB & 2),
                           S2 = F::NIN >= 3 && !(IB & 4);
            if ((chunk + 1) * (int64_t(TX) * UNROLL) * VEC <= Lb) {
                vec_t<In0, VEC> va[S0 ? UNROLL : 1];
                vec_t<In1, VEC> vb[S1 ? UNROLL : 1];
                vec_t<In2, VEC> vc[S2 ? UNROLL : 1];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int64_t j = (v0 + int64_t(u) * TX) * VEC;
                    if constexpr (S0) va[u] = load_vec<vec_t<In0, VEC>>(a + j);
                    if constexpr (S1) vb[u] = load_vec<vec_t<In1, VEC>>(b + j);
                    if constexpr (S2) vc[u] = load_vec<vec_t<In2, VEC>>(c + j);
                }
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int64_t j = (v0 + int64_t(u) * TX) * VEC;
                    vec_t<Out, VEC> r;
#pragma unroll
                    for (int k = 0; k < VEC; ++k) {
                        In0 x = sa;
                        In1 y = sb;
                        In2 z = sc;
                        if constexpr (S0) x = va[u].v[k];
                        if constexpr (S1) y = vb[u].v[k];
                        if constexpr (S2) z = vc[u].v[k];
                        r.v[k] = ew_apply(f, x, y, z);
                    }
                    store_vec(o + j, r);
                }
                continue;
            }
            else {
                // the chunk that holds the end of the row: the same two phases, every vector
                // guarded, the one ragged vector element by element
                vec_t<In0, VEC> va[S0 ? UNROLL : 1];
                vec_t<In1, VEC> vb[S1 ? UNROLL : 1];
                vec_t<In2, VEC> vc[S2 ? UNROLL : 1];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int64_t j = (v0 + int64_t(u) * TX) * VEC;
                    if (j + VEC <= Lb) {
                        if constexpr (S0) va[u] = load_vec<vec_t<In0, VEC>>(a + j);
                        if constexpr (S1) vb[u] = load_vec<vec_t<In1, VEC>>(b + j);
                        if constexpr (S2) vc[u] = load_vec<vec_t<In2, VEC>>(c + j);
                    }
                }
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int64_t j = (v0 + int64_t(u) * TX) * VEC;
                    if (j + VEC <= Lb) {
                        vec_t<Out, VEC> r;
#pragma unroll
                        for (int k = 0; k < VEC; ++k) {
                            In0 x = sa;
                            In1 y = sb;
                            In2 z = sc;
                            if constexpr (S0) x = va[u].v[k];
                            if constexpr (S1) y = vb[u].v[k];
                            if constexpr (S2) z = vc[u].v[k];
                            r.v[k] = ew_apply(f, x, y, z);
                        }
                        store_vec(o + j, r);
                    }
                    else {
                        for (int64_t e = j; e < Lb; ++e) {
                            In0 x = sa;
                            In1 y = sb;
                            In2 z = sc;
                            if constexpr (S0) x = a[e];
                            if constexpr (S1) y = b[e];
                            if constexpr (S2) z = c[e];
                            o[e] = ew_apply(f, x, y, z);
                        }
                    }
                }
                continue;
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t j = (v0 + int64_t(u) * TX) * VEC;  // first element
            if (j + VEC <= Lb) {
                vec_t<In0, VEC> va;
                vec_t<In1, VEC> vb;
                vec_t<In2, VEC> vc;
                if constexpr (F::NIN >= 1) { if (!(inner_bcast & 1u)) va = load_vec<vec_t<In0, VEC>>(a + j); }
                if constexpr (F::NIN >= 2) { if (!(inner_bcast & 2u)) vb = load_vec<vec_t<In1, VEC>>(b + j); }
                if constexpr (F::NIN >= 3) { if (!(inner_bcast & 4u)) vc = load_vec<vec_t<In2, VEC>>(c + j); }
                vec_t<Out, VEC> r;
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    In0 x = sa;
                    In1 y = sb;
                    In2 z = sc;
                    if constexpr (F::NIN >= 1) { if (!(inner_bcast & 1u)) x = va.v[k]; }
                    if constexpr (F::NIN >= 2) { if (!(inner_bcast & 2u)) y = vb.v[k]; }
                    if constexpr (F::NIN >= 3) { if (!(inner_bcast & 4u)) z = vc.v[k]; }
                    r.v[k] = ew_apply(f, x, y, z);
                }
                store_vec(o + j, r);
            }
            else {
                for (int64_t e = j; e < Lb; ++e) {
                    In0 x = sa;
                    In1 y = sb;
                    In2 z = sc;
                    if constexpr (F::NIN >= 1) { if (!(inner_bcast & 1u)) x = a[e]; }
                    if constexpr (F::NIN >= 2) { if (!(inner_bcast & 2u)) y = b[e]; }
                    if constexpr (F::NIN >= 3) { if (!(inner_bcast & 4u)) z = c[e]; }
                    o[e] = ew_apply(f, x, y, z);
                }
            }
        }
    }
}

// -------------------------------------------------------------- transpose
// Dimensions: P (extent np) where the staged inputs are unit-stride, Q (extent
// nq, the last collapsed dimension) where the output is unit-stride, and the
// remaining `batch` dimensions.  A block handles one 32x32 (P x Q) tile of one
// batch entry: staged inputs are read with threads running along P and parked
// in shared memory, everything else is read with threads running along Q.
constexpr int kTile = 32;
constexpr int kTileRows = 8;  // block = 32 x 8 threads

template <class F>
__global__ void __launch_bounds__(kTile *kTileRows)
    ew_transpose_kernel(F f, EwPtrs<F> p, StridedMeta<F::NIN + 1> batch, int64_t np, int64_t nq,
                        int64_t sp0, int64_t sp1, int64_t sp2, int64_t spo, int64_t sq0, int64_t sq1,
                        int64_t sq2, int64_t sqo, unsigned staged, int64_t tiles_p, int64_t tiles_q,
                        int64_t nwork)
{
    using In0 = typename F::In0;
    using In1 = typename F::In1;
    using In2 = typename F::In2;
    using Out = typename F::Out;
    constexpr int NARR = F::NIN + 1;
    __shared__ In0 s0[F::NIN >= 1 ? kTile : 1][kTile + 1];
    __shared__ In1 s1[F::NIN >= 2 ? kTile : 1][kTile + 1];
    __shared__ In2 s2[F::NIN >= 3 ? kTile : 1][kTile + 1];

    const int tx = threadIdx.x & (kTile - 1);
    const int ty = threadIdx.x / kTile;
    const int64_t tiles_per_batch = tiles_p * tiles_q;

    for (int64_t w = blockIdx.x; w < nwork; w += gridDim.x) {
        const int64_t bi = w / tiles_per_batch;
        const int64_t tw = w - bi * tiles_per_batch;
        const int64_t tp = tw / tiles_q;
        const int64_t tq = tw - tp * tiles_q;
        const int64_t p0 = tp * kTile, q0 = tq * kTile;

        int64_t off[NARR];
#pragma unroll
        for (int k = 0; k < NARR; ++k) off[k] = 0;
        {
            uint32_t rem = static_cast<uint32_t>(bi);
            for (int d = batch.nd - 1; d >= 0; --d) {
                uint32_t q, r;
                batch.div[d].divmod(rem, q, r);
                rem = q;
#pragma unroll
                for (int k = 0; k < NARR; ++k) off[k] += int64_t(r) * batch.strides[k][d];
            }
        }
        const In0 *a = static_cast<const In0 *>(p.in[0]) + (F::NIN >= 1 ? off[0] : 0);
        const In1 *b = static_cast<const In1 *>(p.in[1]) + (F::NIN >= 2 ? off[1] : 0);
        const In2 *c = static_cast<const In2 *>(p.in[2]) + (F::NIN >= 3 ? off[2] : 0);
        Out *o = static_cast<Out *>(p.out) + off[NARR - 1];

        // stage: threads run along P (tx), rows of the tile along Q (ty + 8r)
        if (staged) {
            const int64_t pp = p0 + tx;
#pragma unroll
            for (int r = 0; r < kTile / kTileRows; ++r) {
                const int qi = ty + r * kTileRows;
                const int64_t qq = q0 + qi;
                if (pp < np && qq < nq) {
                    if constexpr (F::NIN >= 1) { if (staged & 1u) s0[qi][tx] = a[pp * sp0 + qq * sq0]; }
                    if constexpr (F::NIN >= 2) { if (staged & 2u) s1[qi][tx] = b[pp * sp1 + qq * sq1]; }
                    if constexpr (F::NIN >= 3) { if (staged & 4u) s2[qi][tx] = c[pp * sp2 + qq * sq2]; }
                }
            }
        }
        __syncthreads();
        // compute: threads run along Q (tx), rows of the tile along P (ty + 8r)
        {
            const int64_t qq = q0 + tx;
#pragma unroll
            for (int r = 0; r < kTile / kTileRows; ++r) {
                const int pi = ty + r * kTileRows;
                const int64_t pp = p0 + pi;
                if (pp < np && qq < nq) {
                    In0 x{};
                    In1 y{};
                    In2 z{};
                    if constexpr (F::NIN >= 1) x = (staged & 1u) ? s0[tx][pi] : a[pp * sp0 + qq * sq0];
                    if constexpr (F::NIN >= 2) y = (staged & 2u) ? s1[tx][pi] : b[pp * sp1 + qq * sq1];
                    if constexpr (F::NIN >= 3) z = (staged & 4u) ? s2[tx][pi] : c[pp * sp2 + qq * sq2];
                    o[pp * spo + qq * sqo] = ew_apply(f, x, y, z);
                }
            }
        }
        __syncthreads();
    }
}

// Vector form of the transpose kernel for operands of one element size (4 or 8
// bytes): the tile is T x T elements with T = 16 * VEC, staged inputs are read
// with 16-byte loads along P, every other input and the output with 16-byte
// accesses along Q.  Rows of the tile are padded by one element, which keeps the
// transposing shared-memory accesses at most 2-way conflicted.
struct TransposeStrides {
    int64_t sp[3];  // input strides along P
    int64_t sq[3];  // input strides along Q
    int64_t spo;    // output stride along P (its stride along Q is 1)
};

// Tile coordinates of work item w and the operands' batch offsets (31-bit
// multiply-shift divisions: the launcher guarantees nwork < 2^31).
struct TileDivs {
    FastDiv32 per_row;    // tiles_q
    // Work items are ordered [batch group][tile position][entry in group] with `group`
    // consecutive items per block: a block walks `group` batch entries at one tile position
    // while neighbouring blocks cover neighbouring tile positions.  (Letting one block sweep
    // neighbouring tiles instead concentrates the resident blocks on few memory channels:
    // measured 0.64 of peak against 0.95+ for this order on a 64 x 1024 x 4096 case.)
    FastDiv32 per_group;  // tiles_p * tiles_q * group
    FastDiv32 group_div;  // group
    uint32_t group;
    uint32_t nbatch;
};

// The kernel is instantiated per access pattern (STAGED / VECQ are compile-time
// bit masks over the inputs) so that the tile loop carries no run-time mode
// tests, and every per-thread address part that does not change from tile to
// tile is computed once before the loop: per tile a thread adds one 64-bit tile
// base to its precomputed offsets.  Interior tiles take a path without bounds
// tests.
// Launch bounds ask for 6 resident blocks per SM: at 32-40 registers the kernel keeps
// enough loads in flight (with 4 blocks it reached 0.77 of peak, with 6+ it reaches 0.88).
template <class F, int VEC, unsigned STAGED, unsigned VECQ>
__global__ void __launch_bounds__(kEwThreads, 6)
    ew_transpose_vec_kernel(F f, EwPtrs<F> p, StridedMeta<F::NIN + 1> batch, int64_t np, int64_t nq,
                            TransposeStrides st, TileDivs td, uint32_t nwork, int tiles_per_block)
{
    cudaGridDependencySynchronize();   // see launch_after_previous
    using In0 = typename F::In0;
    using In1 = typename F::In1;
    using Out = typename F::Out;
    constexpr int NARR = F::NIN + 1;
    constexpr int T = 16 * VEC;
    constexpr bool ST0 = (STAGED & 1u) != 0, ST1 = (STAGED & 2u) != 0;
    constexpr bool VQ0 = (VECQ & 1u) != 0, VQ1 = (VECQ & 2u) != 0;
    static_assert(F::NIN == 1 || F::NIN == 2, "one or two inputs");
    __shared__ In0 s0[ST0 ? T : 1][T + 1];
    __shared__ In1 s1[ST1 ? T : 1][T + 1];

    const int lane16 = threadIdx.x & 15;  // vector index inside a tile row
    const int row16 = threadIdx.x >> 4;   // 0..15
    // per-thread offsets relative to the tile origin, for pass r (rows row16 + 16 r)
    int64_t ld0[VEC], ld1[VEC], in0[VEC], in1[VEC], so[VEC];
#pragma unroll
    for (int r = 0; r < VEC; ++r) {
        const int64_t row = row16 + 16 * r;
        ld0[r] = lane16 * VEC + row * st.sq[0];             // staged load: vector along P, row along Q
        ld1[r] = lane16 * VEC + row * st.sq[1];
        in0[r] = row * st.sp[0] + int64_t(lane16 * VEC) * (VQ0 ? 1 : st.sq[0]);  // read along Q, row along P
        in1[r] = row * st.sp[1] + int64_t(lane16 * VEC) * (VQ1 ? 1 : st.sq[1]);
        so[r] = row * st.spo + lane16 * VEC;
    }
    const uint32_t w_begin = blockIdx.x * static_cast<uint32_t>(tiles_per_block);
    uint32_t w_end = w_begin + static_cast<uint32_t>(tiles_per_block);
    if (w_end > nwork || w_end < w_begin) w_end = nwork;

    // A block's items are `group` consecutive batch entries at one tile position: the tile
    // origin is computed for the first item; with a single batch dimension the following
    // items only advance every view by that dimension's stride.
    const In0 *a_st = nullptr, *a_in = nullptr;
    const In1 *b_st = nullptr, *b_in = nullptr;
    Out *o = nullptr;
    int64_t p0 = 0, q0 = 0;
    bool full = false, need_origin = true;
    uint32_t bi = 0;
    for (uint32_t w = w_begin; w < w_end; ++w) {
        if (need_origin) {
            uint32_t grp, rem, tw, jin, tp, tq;
            td.per_group.divmod(w, grp, rem);
            td.group_div.divmod(rem, tw, jin);
            bi = grp * td.group + jin;
            td.per_row.divmod(tw, tp, tq);
            p0 = int64_t(tp) * T;
            q0 = int64_t(tq) * T;
            int64_t off[NARR];
#pragma unroll
            for (int k = 0; k < NARR; ++k) off[k] = 0;
            uint32_t rest = bi;
            for (int d = batch.nd - 1; d >= 0; --d) {
                uint32_t q, r;
                batch.div[d].divmod(rest, q, r);
                rest = q;
#pragma unroll
                for (int k = 0; k < NARR; ++k) off[k] += int64_t(r) * batch.strides[k][d];
            }
            const In0 *a = static_cast<const In0 *>(p.in[0]) + off[0];
            const In1 *b = static_cast<const In1 *>(p.in[1]) + (F::NIN >= 2 ? off[1] : 0);
            o = static_cast<Out *>(p.out) + off[NARR - 1] + p0 * st.spo + q0;
            a_st = a + p0 + q0 * st.sq[0];              // staged view of the tile
            b_st = b + p0 + q0 * st.sq[1];
            a_in = a + p0 * st.sp[0] + q0 * st.sq[0];   // direct view of the tile
            b_in = b + p0 * st.sp[1] + q0 * st.sq[1];
            full = (p0 + T <= np) && (q0 + T <= nq);
            need_origin = batch.nd != 1;
        }
        else {
            ++bi;
            a_st += batch.strides[0][0];
            a_in += batch.strides[0][0];
            if constexpr (F::NIN >= 2) {
                b_st += batch.strides[1][0];
                b_in += batch.strides[1][0];
            }
            o += batch.strides[NARR - 1][0];
        }
        if (bi >= td.nbatch) break;  // padding of a ragged last group (uniform over the block)

        // stage: 16-byte loads along P, scattered into the transposed tile
#pragma unroll
        for (int r = 0; r < VEC; ++r) {
            const int qi = row16 + 16 * r;
            if (full || (p0 + lane16 * VEC < np && q0 + qi < nq)) {
                if constexpr (ST0) {
                    const vec_t<In0, VEC> v = load_vec<vec_t<In0, VEC>>(a_st + ld0[r]);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) s0[lane16 * VEC + e][qi] = v.v[e];
                }
                if constexpr (ST1) {
                    const vec_t<In1, VEC> v = load_vec<vec_t<In1, VEC>>(b_st + ld1[r]);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) s1[lane16 * VEC + e][qi] = v.v[e];
                }
            }
        }
        __syncthreads();
        // combine: 16-byte accesses along Q
#pragma unroll
        for (int r = 0; r < VEC; ++r) {
            const int pi = row16 + 16 * r;
            if (full || (p0 + pi < np && q0 + lane16 * VEC < nq)) {
                vec_t<In0, VEC> x;
                vec_t<In1, VEC> y;
                if constexpr (ST0) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) x.v[e] = s0[pi][lane16 * VEC + e];
                }
                else if constexpr (VQ0) x = load_vec<vec_t<In0, VEC>>(a_in + in0[r]);
                else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) x.v[e] = a_in[in0[r] + e * st.sq[0]];
                }
                if constexpr (F::NIN >= 2) {
                    if constexpr (ST1) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) y.v[e] = s1[pi][lane16 * VEC + e];
                    }
                    else if constexpr (VQ1) y = load_vec<vec_t<In1, VEC>>(b_in + in1[r]);
                    else {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) y.v[e] = b_in[in1[r] + e * st.sq[1]];
                    }
                }
                vec_t<Out, VEC> res;
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    In1 ye{};
                    if constexpr (F::NIN >= 2) ye = y.v[e];
                    res.v[e] = ew_apply(f, x.v[e], ye, char(0));
                }
                store_vec(o + so[r], res);
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------- generic
template <class F, bool IDX32, int UNROLL>
__global__ void __launch_bounds__(kEwThreads)
    ew_generic_kernel(F f, EwPtrs<F> p, StridedMeta<F::NIN + 1> m, int64_t n)
{
    using In0 = typename F::In0;
    using In1 = typename F::In1;
    using In2 = typename F::In2;
    using Out = typename F::Out;
    constexpr int NARR = F::NIN + 1;
    const int64_t block_base = int64_t(blockIdx.x) * (kEwThreads * UNROLL);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int64_t i = block_base + int64_t(u) * kEwThreads + threadIdx.x;
        if (i >= n) break;
        int64_t off[NARR];
#pragma unroll
        for (int k = 0; k < NARR; ++k) off[k] = 0;
        if constexpr (IDX32) {
            uint32_t rem = static_cast<uint32_t>(i);
            for (int d = m.nd - 1; d > 0; --d) {
                uint32_t q, r;
                m.div[d].divmod(rem, q, r);
                rem = q;
#pragma unroll
                for (int k = 0; k < NARR; ++k) off[k] += int64_t(r) * m.strides[k][d];
            }
#pragma unroll
            for (int k = 0; k < NARR; ++k) off[k] += int64_t(rem) * m.strides[k][0];
        }
        else {
            int64_t rem = i;
            for (int d = m.nd - 1; d > 0; --d) {
                const int64_t q = rem / m.shape[d];
                const int64_t r = rem - q * m.shape[d];
                rem = q;
#pragma unroll
                for (int k = 0; k < NARR; ++k) off[k] += r * m.strides[k][d];
            }
#pragma unroll
            for (int k = 0; k < NARR; ++k) off[k] += rem * m.strides[k][0];
        }
        In0 x{};
        In1 y{};
        In2 z{};
        if constexpr (F::NIN >= 1) x = static_cast<const In0 *>(p.in[0])[off[0]];
        if constexpr (F::NIN >= 2) y = static_cast<const In1 *>(p.in[1])[off[1]];
        if constexpr (F::NIN >= 3) z = static_cast<const In2 *>(p.in[2])[off[2]];
        static_cast<Out *>(p.out)[off[NARR - 1]] = ew_apply(f, x, y, z);
    }
}

// --------------------------------------------------------------- launcher

template <int NARR>
inline void fill_meta(StridedMeta<NARR> &m, const EwPlan &plan, const int *dims, int ndims,
                      const int *arr_index)
{
    m.nd = ndims;
    for (int i = 0; i < ndims; ++i) {
        const int d = dims[i];
        m.shape[i] = plan.shape[d];
        m.div[i] = FastDiv32(static_cast<uint32_t>(plan.shape[d] > 0 && plan.shape[d] < (int64_t(1) << 31)
                                                       ? plan.shape[d]
                                                       : 1));
        for (int k = 0; k < NARR; ++k) m.strides[k][i] = plan.strides[arr_index[k]][d];
    }
}

// One block per tile (the hardware scheduler balances the tail better than a
// fixed grid-stride partition); the kernels keep their stride loops, so a grid
// capped at 2^30 blocks still covers any size.
inline int ew_flat_grid(int64_t ntiles)
{
    const int64_t cap = int64_t(1) << 30;
    return static_cast<int>(ntiles < 1 ? 1 : (ntiles < cap ? ntiles : cap));
}

inline int ew_grid(int64_t nwork)
{
    const int64_t cap = int64_t(device_props().sm_count) * tuning_ctas_per_sm();
    return static_cast<int>(nwork < cap ? (nwork < 1 ? 1 : nwork) : cap);
}

// Launch functor F over the planned iteration space.  `in` holds F::NIN base
// pointers and `out` the output pointer, all already displaced by the plan's
// offsets.  The plan's array order is inputs first, output last.
template <class F>
int launch_ew(const F &f, const EwPlan &plan, const void *const *in, void *out, cudaStream_t stream)
{
    constexpr int NIN = F::NIN;
    constexpr int NARR = NIN + 1;
    using Out = typename F::Out;
    if (plan.n == 0) return DPB_OK;
    EwPtrs<F> p;
    for (int k = 0; k < 3; ++k) p.in[k] = (k < NIN) ? in[k] : nullptr;
    p.out = out;
    int arr_index[NARR];
    for (int k = 0; k < NARR; ++k) arr_index[k] = k;
    const size_t in_sizes[3] = {sizeof(typename F::In0), sizeof(typename F::In1),
                                sizeof(typename F::In2)};
    constexpr int VEC = ew_vec_width<F>();

    switch (plan.kind) {
    case EW_CONTIG: {
        bool aligned = is_aligned(out, sizeof(Out) * VEC);
        for (int k = 0; k < NIN; ++k)
            if (!(plan.bcast_mask & (1u << k))) aligned = aligned && is_aligned(in[k], in_sizes[k] * VEC);
        const unsigned m = plan.bcast_mask;
        // the vector kernel is instantiated for the broadcast patterns that occur in practice;
        // anything else (unaligned pointers, odd patterns) takes the rows kernel below
#define DPB_CONTIG_LAUNCH(U, MASK)                                                                  \
    {                                                                                               \
        const int64_t tiles = plan.n / (int64_t(kEwThreads) * VEC * (U));                           \
        launch_after_previous(ew_contig_vec_kernel<F, VEC, U, MASK>, ew_flat_grid(tiles), kEwThreads, stream, f, p, \
                              plan.n);                                                              \
        note_kernel("ew_contig_vec");                                                               \
        return check_launch("ew_contig_vec");                                                       \
    }
        if (aligned) {
            if constexpr (NIN == 0) DPB_CONTIG_LAUNCH(8, 0u)
            if constexpr (NIN == 1) {
                if (m == 0) DPB_CONTIG_LAUNCH(ew_unroll<F>::value, 0u)
            }
            if constexpr (NIN == 2) {
                if (m == 0) DPB_CONTIG_LAUNCH(4, 0u)
                if (m == 1) DPB_CONTIG_LAUNCH(8, 1u)
                if (m == 2) DPB_CONTIG_LAUNCH(8, 2u)
            }
            if constexpr (NIN == 3) {
                if (m == 0) DPB_CONTIG_LAUNCH(4, 0u)
                if (m == 2) DPB_CONTIG_LAUNCH(4, 2u)
                if (m == 4) DPB_CONTIG_LAUNCH(4, 4u)
                if (m == 6) DPB_CONTIG_LAUNCH(8, 6u)
            }
        }
#undef DPB_CONTIG_LAUNCH
        // fall through: a contiguous plan is a rows plan with no outer dimensions
    }
    case EW_ROWS: {
        const int last = plan.nd - 1;
        const int64_t L = plan.shape[last];
        int dims[kMaxD];
        for (int i = 0; i < last; ++i) dims[i] = i;
        StridedMeta<NARR> outer;
        fill_meta(outer, plan, dims, last, arr_index);
        int64_t nrows = 1;
        for (int i = 0; i < last; ++i) nrows *= plan.shape[i];
        unsigned inner_bcast = 0;
        for (int k = 0; k < NIN; ++k)
            if (plan.strides[k][last] == 0) inner_bcast |= (1u << k);
        // 16-byte accesses need row starts that sit at one common element position within
        // a 16-byte group in every unit-stride operand; rows that start off the boundary
        // take their first `head` elements one by one
        auto misalign = [](const void *ptr, size_t elem) {
            return static_cast<int>((reinterpret_cast<uintptr_t>(ptr) / elem) % VEC);
        };
        // vector accesses for the broadcast patterns that occur in practice (none; one of two
        // inputs a single value per row); anything else goes element by element
        bool aligned = VEC > 1 && (inner_bcast == 0 || (NIN == 2 && inner_bcast < 3));
        const int mis = misalign(out, sizeof(Out));
        for (int i = 0; i < last; ++i) aligned = aligned && (plan.strides[NARR - 1][i] % VEC == 0);
        for (int k = 0; k < NIN; ++k) {
            if (inner_bcast & (1u << k)) continue;
            aligned = aligned && misalign(in[k], in_sizes[k]) == mis;
            for (int i = 0; i < last; ++i) aligned = aligned && (plan.strides[k][i] % VEC == 0);
        }
        const int vec = aligned ? VEC : 1;
        const int head = aligned ? static_cast<int>(std::min<int64_t>((VEC - mis) % VEC, L)) : 0;
        constexpr int UNROLL = 4;
        const int64_t nvec = std::max<int64_t>(1, ceil_div(L - head, vec));
        int tx_log2 = 0;
        while ((1 << tx_log2) < kEwThreads && (int64_t(1) << tx_log2) * UNROLL < nvec) ++tx_log2;
        const int TX = 1 << tx_log2, TY = kEwThreads >> tx_log2;
        const int64_t chunks = ceil_div(nvec, int64_t(TX) * UNROLL);
        const int64_t nwork = ceil_div(nrows, TY) * chunks;
        const FastDiv32 chunk_div(static_cast<uint32_t>(chunks < (int64_t(1) << 31) ? chunks : 1));
#define DPB_ROWS_LAUNCH(V, MASK)                                                                    \
    launch_after_previous(ew_rows_kernel<F, V, UNROLL, MASK>, ew_flat_grid(nwork), kEwThreads, stream, \
                          f, p, outer, L, inner_bcast, nrows, tx_log2, chunks, nwork, chunk_div, head)
        if (vec > 1) {
            if (inner_bcast == 0) DPB_ROWS_LAUNCH(VEC, 0);
            else if (inner_bcast == 1) DPB_ROWS_LAUNCH(VEC, (F::NIN == 2 ? 1 : 0));
            else DPB_ROWS_LAUNCH(VEC, (F::NIN == 2 ? 2 : 0));
            note_kernel(head ? "ew_rows_vec_head" : "ew_rows_vec");
        }
        else {
            DPB_ROWS_LAUNCH(1, -1);
            note_kernel("ew_rows_scalar");
        }
#undef DPB_ROWS_LAUNCH
        return check_launch("ew_rows");
    }
    case EW_TRANSPOSE: {
        if constexpr (sizeof(typename F::In0) <= 8 && sizeof(typename F::In1) <= 8 &&
                      sizeof(typename F::In2) <= 8) {
            const int q = plan.nd - 1, pd = plan.tdim;
            int dims[kMaxD];
            int nb = 0;
            int64_t nbatch = 1;
            for (int i = 0; i < plan.nd; ++i)
                if (i != q && i != pd) {
                    dims[nb++] = i;
                    nbatch *= plan.shape[i];
                }
            StridedMeta<NARR> batch;
            fill_meta(batch, plan, dims, nb, arr_index);
            const int64_t np = plan.shape[pd], nq = plan.shape[q];
            // vector form: one or two inputs of one element size (4 or 8 bytes), every vector
            // access 16-byte aligned; instantiated per access pattern
            if constexpr ((NIN == 1 || NIN == 2) && (sizeof(Out) == 4 || sizeof(Out) == 8) &&
                          sizeof(typename F::In0) == sizeof(Out) &&
                          (NIN < 2 || sizeof(typename F::In1) == sizeof(Out))) {
                constexpr int TV = 16 / static_cast<int>(sizeof(Out));
                constexpr int T = 16 * TV;
                const int64_t tp = ceil_div(np, T), tq = ceil_div(nq, T);
                const int64_t nw = nbatch * tp * tq;
                bool ok = np % TV == 0 && nq % TV == 0 && is_aligned(out, 16) &&
                          plan.strides[NARR - 1][pd] % TV == 0 && nw < (int64_t(1) << 31);
                for (int i = 0; i < nb && ok; ++i) ok = plan.strides[NARR - 1][dims[i]] % TV == 0;
                unsigned vecq = 0;
                for (int k = 0; k < NIN && ok; ++k) {
                    bool aligned_k = is_aligned(in[k], 16);
                    for (int i = 0; i < nb; ++i) aligned_k = aligned_k && plan.strides[k][dims[i]] % TV == 0;
                    if (plan.staged_mask & (1u << k)) {
                        ok = aligned_k && plan.strides[k][q] % TV == 0;
                    }
                    else if (plan.strides[k][q] == 1 && aligned_k && plan.strides[k][pd] % TV == 0) {
                        vecq |= (1u << k);
                    }
                }
                if (ok) {
                    TransposeStrides ts;
                    for (int k = 0; k < 3; ++k) {
                        ts.sp[k] = k < NIN ? plan.strides[k][pd] : 0;
                        ts.sq[k] = k < NIN ? plan.strides[k][q] : 0;
                    }
                    ts.spo = plan.strides[NARR - 1][pd];
                    // `group` batch entries per block (fewer when that would leave under 16 blocks per SM)
                    int64_t group = std::min<int64_t>(8, nbatch);
                    while (group > 1 && ceil_div(nbatch, group) * tp * tq < int64_t(device_props().sm_count) * 16)
                        group /= 2;
                    const int tpb = static_cast<int>(group);
                    const int64_t nw_padded = ceil_div(nbatch, group) * group * tp * tq;
                    if (nw_padded >= (int64_t(1) << 31))
                        return set_error(DPB_ERR_RUNTIME, "iteration space too large for the tiled kernel");
                    const unsigned nblocks = static_cast<unsigned>(nw_padded / tpb);
                    TileDivs td;
                    td.per_row = FastDiv32(static_cast<uint32_t>(tq));
                    td.per_group = FastDiv32(static_cast<uint32_t>(tp * tq * group));
                    td.group_div = FastDiv32(static_cast<uint32_t>(group));
                    td.group = static_cast<uint32_t>(group);
                    td.nbatch = static_cast<uint32_t>(nbatch);
                    const uint32_t nw32 = static_cast<uint32_t>(nw_padded);
                    const unsigned sm = plan.staged_mask;
#define DPB_TR_LAUNCH(S, V)                                                                          \
    {                                                                                                \
        launch_after_previous(ew_transpose_vec_kernel<F, TV, S, V>, nblocks, kEwThreads, stream, f, p, batch, \
                              np, nq, ts, td, nw32, tpb);                                            \
        note_kernel("ew_transpose_vec");                                                             \
        return check_launch("ew_transpose_vec");                                                     \
    }
                    if constexpr (NIN == 1) {
                        if (sm == 1u) DPB_TR_LAUNCH(1u, 0u)
                    }
                    else {
                        if (sm == 1u && vecq == 2u) DPB_TR_LAUNCH(1u, 2u)
                        if (sm == 2u && vecq == 1u) DPB_TR_LAUNCH(2u, 1u)
                        if (sm == 3u) DPB_TR_LAUNCH(3u, 0u)
                        if (sm == 1u && vecq == 0u) DPB_TR_LAUNCH(1u, 0u)
                        if (sm == 2u && vecq == 0u) DPB_TR_LAUNCH(2u, 0u)
                    }
#undef DPB_TR_LAUNCH
                }
            }
            const int64_t tiles_p = ceil_div(np, kTile), tiles_q = ceil_div(nq, kTile);
            const int64_t nwork = nbatch * tiles_p * tiles_q;
            auto sp = [&](int k) { return k < NIN ? plan.strides[k][pd] : 0; };
            auto sq = [&](int k) { return k < NIN ? plan.strides[k][q] : 0; };
            ew_transpose_kernel<F><<<ew_grid(nwork), kTile * kTileRows, 0, stream>>>(
                f, p, batch, np, nq, sp(0), sp(1), sp(2), plan.strides[NARR - 1][pd], sq(0), sq(1),
                sq(2), plan.strides[NARR - 1][q], plan.staged_mask, tiles_p, tiles_q, nwork);
            note_kernel("ew_transpose");
            return check_launch("ew_transpose");
        }
        // element types wider than 8 bytes are not staged: fall through
    }
    case EW_GENERIC:
    default: {
        int dims[kMaxD];
        for (int i = 0; i < plan.nd; ++i) dims[i] = i;
        StridedMeta<NARR> m;
        fill_meta(m, plan, dims, plan.nd, arr_index);
        constexpr int UNROLL = 4;
        const int64_t nblocks = ceil_div(plan.n, int64_t(kEwThreads) * UNROLL);
        if (nblocks > 0x7fffffffLL)
            return set_error(DPB_ERR_RUNTIME, "iteration space too large for the strided kernel");
        if (plan.n < (int64_t(1) << 31)) {
            ew_generic_kernel<F, true, UNROLL>
                <<<static_cast<unsigned>(nblocks), kEwThreads, 0, stream>>>(f, p, m, plan.n);
            note_kernel("ew_generic32");
        }
        else {
            ew_generic_kernel<F, false, UNROLL>
                <<<static_cast<unsigned>(nblocks), kEwThreads, 0, stream>>>(f, p, m, plan.n);
            note_kernel("ew_generic64");
        }
        return check_launch("ew_generic");
    }
    }
}

}  // namespace dpb

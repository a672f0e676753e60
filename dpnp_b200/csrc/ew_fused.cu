// Fused elementwise chains: one launch evaluates a whole expression graph per element.
//
// The reference has no fusion: every ufunc call of a chain such as
// examples/example_bs.py:50-78 is one kernel that reads and writes full arrays
// (dpnp/dpnp_algo/dpnp_elementwise_common.py:81-235,537-739 calls straight into the
// per-op implementations).  Here a chain is handed over as a small register-machine
// program; the kernel interprets it with the operators of the per-op engine (the same
// device functions, so every intermediate value has the bits the unfused chain gives)
// and touches global memory only for the chain's inputs and outputs.
//
// Execution model: a block owns a tile of kFusedThreads * K consecutive elements.  A thread
// holds K elements of every virtual register in shared memory, laid out
// [register][16-byte group][thread] (bank-conflict free), plus one "accumulator" -- the result of
// the previous instruction -- in real registers, so that chains of dependent operations
// do not bounce through shared memory.  Every thread of the grid executes the same
// instruction stream: branches on the opcode are uniform.

#include <cstring>

#include "common.cuh"
#include "ew_ops.cuh"
#include "ew_erf.cuh"
#include "ew_fused.h"

namespace dpb {

constexpr int kFusedThreads = 128;


// The host turns every instruction word into one or two micro-operations whose fields the
// kernel can use as they are (operand kind resolved, shared-memory offsets multiplied out,
// the first operand always the accumulator), so the device decodes with one 16-byte load.
enum FusedKind : int32_t {
    FK_MOVE_REG = 0,   // acc <- register
    FK_MOVE_IMM,       // acc <- immediate
    FK_MOVE_IN,        // acc <- input array
    FK_STORE,          // output array <- acc (acc unchanged)
    FK_STORE_ANY,      // output array <- any operand, acc untouched (aux2 = original operand code)
    FK_SELECT,         // acc <- a ? b : c, operands by their original codes in b_off
    FK_UNARY,          // acc <- op(acc)
    FK_BIN_REG,        // acc <- op(acc, register)   (operands exchanged when swap is set)
    FK_BIN_IN,         // acc <- op(acc, input array)
    FK_BIN_ACC,        // acc <- op(acc, acc)
    FK_BIN_IMM         // acc <- op(acc, immediate)
};

struct FusedUop {
    int32_t kind_op;    // kind | op << 8 | swap << 16
    int32_t dst_off;    // register to receive acc: offset in 16-byte groups, or -1
    int32_t b_off;      // register operand: offset in 16-byte groups; SELECT: a | b << 8 | c << 16
    int32_t aux;        // immediate / input / output index
};

constexpr int kFusedMaxUops = 2 * kFusedMaxInstr;

struct FusedParams {
    int32_t n_uop;
    int32_t vector_io;                  // every array pointer is 16-byte aligned
    FusedUop uop[kFusedMaxUops];
    double imm[kFusedMaxImm];
    const void *in[kFusedMaxIn];
    int32_t in_scalar[kFusedMaxIn];     // input is one element, broadcast
    void *out[kFusedMaxOut];
};

template <class T> DPB_D T as_flag(bool_t b) { return b.v ? T(1) : T(0); }

// One decode per instruction: the opcode selects a loop over the thread's K elements.
// The first operand is in `acc`, the result replaces it.
#define DPB_FUSED_UN(CODE, EXPR)                                   \
    case CODE:                                                     \
        _Pragma("unroll") for (int k = 0; k < K; ++k) { const T x = acc[k]; acc[k] = (EXPR); } \
        break;
#define DPB_FUSED_BIN(CODE, EXPR)                                  \
    case CODE:                                                     \
        _Pragma("unroll") for (int k = 0; k < K; ++k) {            \
            const T x = SWAP ? b[k] : acc[k];                      \
            const T y = SWAP ? acc[k] : b[k];                      \
            acc[k] = (EXPR);                                       \
        }                                                          \
        break;

template <class T, int K> DPB_D void fused_unary(int op, T (&acc)[K])
{
    switch (op) {
        DPB_FUSED_UN(DPB_FUSED_NEGATIVE, NegativeOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_ABS, AbsOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_EXP, ExpOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_LOG, LogOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_SQRT, SqrtOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_ERF, ErfOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_SQUARE, SquareOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_RECIPROCAL, ReciprocalOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_SIN, SinOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_COS, CosOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_TANH, TanhOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_EXPM1, Expm1Op<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_LOG1P, Log1pOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_FLOOR, FloorOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_CEIL, CeilOp<T>::apply(x))
        DPB_FUSED_UN(DPB_FUSED_SIGN, SignOp<T>::apply(x))
    default:  // DPB_FUSED_POSITIVE, DPB_FUSED_MOVE: the value itself
        break;
    }
}

// SWAP: the accumulator holds the SECOND operand of the operator.
template <class T, int K, bool SWAP> DPB_D void fused_binary(int op, T (&acc)[K], const T (&b)[K])
{
    switch (op) {
        DPB_FUSED_BIN(DPB_FUSED_ADD, (AddOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_SUBTRACT, (SubtractOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_MULTIPLY, (MultiplyOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_DIVIDE, (TrueDivideOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_MAXIMUM, (MaximumOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_MINIMUM, (MinimumOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_POW, (PowOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_LESS, as_flag<T>(LessOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_LESS_EQUAL, as_flag<T>(LessEqualOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_GREATER, as_flag<T>(GreaterOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_GREATER_EQUAL, as_flag<T>(GreaterEqualOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_EQUAL, as_flag<T>(EqualOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_NOT_EQUAL, as_flag<T>(NotEqualOp<T, T>::apply(x, y)))
        DPB_FUSED_BIN(DPB_FUSED_LOGICAL_AND, ((x != T(0) && y != T(0)) ? T(1) : T(0)))
        DPB_FUSED_BIN(DPB_FUSED_LOGICAL_OR, ((x != T(0) || y != T(0)) ? T(1) : T(0)))
    default:
        break;
    }
}

// Second operand is one immediate for all K elements: no broadcast into registers.
#define DPB_FUSED_BINS(CODE, EXPR)                                 \
    case CODE:                                                     \
        _Pragma("unroll") for (int k = 0; k < K; ++k) {            \
            const T x = SWAP ? c : acc[k];                         \
            const T y = SWAP ? acc[k] : c;                         \
            acc[k] = (EXPR);                                       \
        }                                                          \
        break;
template <class T, int K, bool SWAP> DPB_D void fused_binary_scalar(int op, T (&acc)[K], const T c)
{
    switch (op) {
        DPB_FUSED_BINS(DPB_FUSED_ADD, (AddOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_SUBTRACT, (SubtractOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_MULTIPLY, (MultiplyOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_DIVIDE, (TrueDivideOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_MAXIMUM, (MaximumOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_MINIMUM, (MinimumOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_POW, (PowOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_LESS, as_flag<T>(LessOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_LESS_EQUAL, as_flag<T>(LessEqualOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_GREATER, as_flag<T>(GreaterOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_GREATER_EQUAL, as_flag<T>(GreaterEqualOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_EQUAL, as_flag<T>(EqualOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_NOT_EQUAL, as_flag<T>(NotEqualOp<T, T>::apply(x, y)))
        DPB_FUSED_BINS(DPB_FUSED_LOGICAL_AND, ((x != T(0) && y != T(0)) ? T(1) : T(0)))
        DPB_FUSED_BINS(DPB_FUSED_LOGICAL_OR, ((x != T(0) || y != T(0)) ? T(1) : T(0)))
    default:
        break;
    }
}
#undef DPB_FUSED_BINS
#undef DPB_FUSED_UN
#undef DPB_FUSED_BIN

// K: elements per thread and register
template <class T, int K>
__global__ void __launch_bounds__(kFusedThreads)
    ew_fused_kernel(const __grid_constant__ FusedParams prm, int64_t n)
{
    constexpr int VW = 16 / sizeof(T);  // elements per 16-byte access
    constexpr int NV = K / VW;          // 16-byte groups per thread and register
    using V = vec_t<T, VW>;
    extern __shared__ __align__(16) unsigned char fused_smem[];
    // register file: [register][group][thread] of 16-byte groups -- consecutive threads touch
    // consecutive groups, so the 128-bit accesses are conflict-free
    V *regs = reinterpret_cast<V *>(fused_smem);
    const int tid = threadIdx.x;
    const int64_t base = (int64_t(blockIdx.x) * kFusedThreads + tid) * K;  // first element of the thread
    if (base >= n) return;  // no block-wide barrier below: every thread works on its own slots
    const bool whole = base + K <= n;

    T acc[K];
#pragma unroll
    for (int k = 0; k < K; ++k) acc[k] = T(0);

    // the thread's K elements of input array i (one element broadcast, 16-byte loads, or
    // guarded element loads on the ragged tail / unaligned arrays)
    auto load_input = [&](unsigned i, T(&v)[K]) {
        const T *src = static_cast<const T *>(prm.in[i]);
        if (prm.in_scalar[i]) {
            const T c = src[0];
#pragma unroll
            for (int k = 0; k < K; ++k) v[k] = c;
        }
        else if (whole && prm.vector_io) {
#pragma unroll
            for (int k = 0; k < K; k += VW) {
                V x = load_vec<V>(src + base + k);
#pragma unroll
                for (int j = 0; j < VW; ++j) v[k + j] = x.v[j];
            }
        }
        else {
#pragma unroll
            for (int k = 0; k < K; ++k) v[k] = (base + k < n) ? src[base + k] : T(0);
        }
    };

    auto load_reg = [&](int off, T(&v)[K]) {
#pragma unroll
        for (int g = 0; g < NV; ++g) {
            const V t = regs[(off + g) * kFusedThreads + tid];
#pragma unroll
            for (int j = 0; j < VW; ++j) v[g * VW + j] = t.v[j];
        }
    };
    auto store_out = [&](int i, const T(&v)[K]) {
        T *dstp = static_cast<T *>(prm.out[i]);
        if (whole && prm.vector_io) {
#pragma unroll
            for (int k = 0; k < K; k += VW) {
                V x;
#pragma unroll
                for (int j = 0; j < VW; ++j) x.v[j] = v[k + j];
                store_vec(dstp + base + k, x);
            }
        }
        else {
#pragma unroll
            for (int k = 0; k < K; ++k)
                if (base + k < n) dstp[base + k] = v[k];
        }
    };
    // operand by its original 8-bit code (the rare paths: SELECT, stores of a non-accumulator)
    auto fetch_any = [&](unsigned x, T(&v)[K]) {
        if (x == kOpndAcc) {
#pragma unroll
            for (int k = 0; k < K; ++k) v[k] = acc[k];
        }
        else if (x >= kOpndIn) {
            load_input(x - kOpndIn, v);
        }
        else if (x >= kOpndImm) {
            const T c = static_cast<T>(prm.imm[x - kOpndImm]);
#pragma unroll
            for (int k = 0; k < K; ++k) v[k] = c;
        }
        else {
            load_reg(static_cast<int>(x) * NV, v);
        }
    };

    for (int pc = 0; pc < prm.n_uop; ++pc) {
        const FusedUop u = prm.uop[pc];
        const int kind = u.kind_op & 0xff;
        const int op = (u.kind_op >> 8) & 0xff;
        const bool swap = (u.kind_op >> 16) & 1;
        switch (kind) {
        case FK_MOVE_REG: load_reg(u.b_off, acc); break;
        case FK_MOVE_IMM: {
            const T c = static_cast<T>(prm.imm[u.aux]);
#pragma unroll
            for (int k = 0; k < K; ++k) acc[k] = c;
            break;
        }
        case FK_MOVE_IN: load_input(u.aux, acc); break;
        case FK_STORE: store_out(u.aux, acc); break;
        case FK_STORE_ANY: {
            T v[K];
            fetch_any(static_cast<unsigned>(u.b_off), v);
            store_out(u.aux, v);
            break;
        }
        case FK_SELECT: {
            T c[K], a[K], b[K];
            fetch_any(static_cast<unsigned>(u.b_off & 0xff), c);
            fetch_any(static_cast<unsigned>((u.b_off >> 8) & 0xff), a);
            fetch_any(static_cast<unsigned>((u.b_off >> 16) & 0xff), b);
#pragma unroll
            for (int k = 0; k < K; ++k) acc[k] = (c[k] != T(0)) ? a[k] : b[k];
            break;
        }
        case FK_UNARY: fused_unary<T, K>(op, acc); break;
        case FK_BIN_IMM: {
            const T c = static_cast<T>(prm.imm[u.aux]);
            if (swap) fused_binary_scalar<T, K, true>(op, acc, c);
            else fused_binary_scalar<T, K, false>(op, acc, c);
            break;
        }
        default: {  // FK_BIN_REG, FK_BIN_IN, FK_BIN_ACC
            T b[K];
            if (kind == FK_BIN_REG) load_reg(u.b_off, b);
            else if (kind == FK_BIN_IN) load_input(u.aux, b);
            else {
#pragma unroll
                for (int k = 0; k < K; ++k) b[k] = acc[k];
            }
            if (swap) fused_binary<T, K, true>(op, acc, b);
            else fused_binary<T, K, false>(op, acc, b);
            break;
        }
        }
        if (u.dst_off >= 0) {
#pragma unroll
            for (int g = 0; g < NV; ++g) {
                V t;
#pragma unroll
                for (int j = 0; j < VW; ++j) t.v[j] = acc[g * VW + j];
                regs[(u.dst_off + g) * kFusedThreads + tid] = t;
            }
        }
    }
}

namespace {

bool operand_ok(unsigned x, int n_reg, int n_imm, int n_in, bool first)
{
    if (x == kOpndAcc) return !first;
    if (x >= kOpndIn) return static_cast<int>(x - kOpndIn) < n_in;
    if (x >= kOpndImm) return static_cast<int>(x - kOpndImm) < n_imm;
    return static_cast<int>(x) < n_reg;
}

}  // namespace
}  // namespace dpb

using namespace dpb;

// Everything a launch relies on is checked here, once, on the host: the limits, the pointers and
// every index of every instruction.  `aligned`: all array pointers allow 16-byte accesses.
int dpb::fused_check_program(const dpb_fused_program *prog, int64_t n, bool *aligned_out)
{
    if (!prog) return set_error(DPB_ERR_VALUE, "fused program is null");
    if (prog->typenum != DPB_FLOAT && prog->typenum != DPB_DOUBLE)
        return set_error(DPB_ERR_TYPE, "fused programs compute in float32 or float64");
    if (prog->n_instr < 0 || prog->n_instr > kFusedMaxInstr || prog->n_imm < 0 || prog->n_imm > kFusedMaxImm ||
        prog->n_in < 0 || prog->n_in > kFusedMaxIn || prog->n_out < 0 || prog->n_out > kFusedMaxOut ||
        prog->n_reg < 0 || prog->n_reg > kFusedMaxReg)
        return set_error(DPB_ERR_VALUE, "fused program exceeds the limits of the interpreter "
                                        "(192 instructions, 48 immediates, 12 inputs, 8 outputs, 24 registers)");
    if (n < 0) return set_error(DPB_ERR_VALUE, "negative element count");
    bool aligned = true;
    for (int i = 0; i < prog->n_in; ++i) {
        if (!prog->in[i]) return set_error(DPB_ERR_VALUE, "fused program: null input pointer");
        const bool scalar = prog->in_is_scalar && prog->in_is_scalar[i];
        if (!scalar) aligned = aligned && is_aligned(prog->in[i], 16);
    }
    for (int i = 0; i < prog->n_out; ++i) {
        if (!prog->out[i]) return set_error(DPB_ERR_VALUE, "fused program: null output pointer");
        aligned = aligned && is_aligned(prog->out[i], 16);
    }
    for (int pc = 0; pc < prog->n_instr; ++pc) {
        const uint64_t w = prog->code[pc];
        const int op = static_cast<int>(w & 0xff);
        const unsigned dst = static_cast<unsigned>((w >> 8) & 0xff);
        const unsigned oa = static_cast<unsigned>((w >> 16) & 0xff);
        const unsigned ob = static_cast<unsigned>((w >> 24) & 0xff);
        const unsigned oc = static_cast<unsigned>((w >> 32) & 0xff);
        const bool first = pc == 0;
        bool ok = op >= 0 && op < DPB_FUSED_OP_COUNT;
        if (ok && op == DPB_FUSED_LOAD) ok = static_cast<int>(oa) < prog->n_in;
        else if (ok && op == DPB_FUSED_STORE)
            ok = operand_ok(oa, prog->n_reg, prog->n_imm, prog->n_in, first) && static_cast<int>(ob) < prog->n_out;
        else if (ok && op == DPB_FUSED_SELECT)
            ok = operand_ok(oa, prog->n_reg, prog->n_imm, prog->n_in, first) && operand_ok(ob, prog->n_reg, prog->n_imm, prog->n_in, first) &&
                 operand_ok(oc, prog->n_reg, prog->n_imm, prog->n_in, first);
        else if (ok && op < DPB_FUSED_FIRST_BINARY) ok = operand_ok(oa, prog->n_reg, prog->n_imm, prog->n_in, first);
        else if (ok)
            ok = operand_ok(oa, prog->n_reg, prog->n_imm, prog->n_in, first) && operand_ok(ob, prog->n_reg, prog->n_imm, prog->n_in, first);
        if (ok && op != DPB_FUSED_STORE) ok = dst == kNoDst || static_cast<int>(dst) < prog->n_reg;
        if (!ok) return set_error(DPB_ERR_VALUE, "fused program: malformed instruction");
    }
    if (aligned_out) *aligned_out = aligned;
    return DPB_OK;
}

extern "C" int dpb_fused_elementwise(const dpb_fused_program *prog, int64_t n, void *stream)
{
    bool aligned = true;
    DPB_TRY(fused_check_program(prog, n, &aligned));
    FusedParams prm;
    std::memset(&prm, 0, sizeof(prm));
    for (int i = 0; i < prog->n_in; ++i) {
        prm.in[i] = prog->in[i];
        prm.in_scalar[i] = prog->in_is_scalar ? prog->in_is_scalar[i] : 0;
    }
    for (int i = 0; i < prog->n_out; ++i) prm.out[i] = prog->out[i];
    prm.vector_io = aligned ? 1 : 0;
    for (int i = 0; i < prog->n_imm; ++i) prm.imm[i] = prog->imm[i];
    if (n == 0 || prog->n_instr == 0) return DPB_OK;
    const size_t elem = prog->typenum == DPB_DOUBLE ? 8 : 4;
    const int K = static_cast<int>(tuning_fused_elems());
    // ---- instruction words -> micro-operations
    const int NV = K / static_cast<int>(16 / elem);     // 16-byte groups per thread and register
    int nu = 0;
    auto emit = [&](int kind, int op, bool swap, int dst_off, int b_off, int aux) {
        prm.uop[nu].kind_op = kind | (op << 8) | ((swap ? 1 : 0) << 16);
        prm.uop[nu].dst_off = dst_off;
        prm.uop[nu].b_off = b_off;
        prm.uop[nu].aux = aux;
        ++nu;
    };
    // acc <- operand x (which is not the accumulator)
    auto emit_move = [&](unsigned x, int dst_off) {
        if (x >= kOpndIn) emit(FK_MOVE_IN, 0, false, dst_off, 0, static_cast<int>(x - kOpndIn));
        else if (x >= kOpndImm) emit(FK_MOVE_IMM, 0, false, dst_off, 0, static_cast<int>(x - kOpndImm));
        else emit(FK_MOVE_REG, 0, false, dst_off, static_cast<int>(x) * NV, 0);
    };
    for (int pc = 0; pc < prog->n_instr; ++pc) {
        const uint64_t w = prog->code[pc];
        const int op = static_cast<int>(w & 0xff);
        const unsigned dst = static_cast<unsigned>((w >> 8) & 0xff);
        unsigned oa = static_cast<unsigned>((w >> 16) & 0xff);
        unsigned ob = static_cast<unsigned>((w >> 24) & 0xff);
        const unsigned oc = static_cast<unsigned>((w >> 32) & 0xff);
        bool swap = (w >> 40) & 1;
        const int dst_off = (dst == kNoDst || op == DPB_FUSED_STORE) ? -1 : static_cast<int>(dst) * NV;
        if (op == DPB_FUSED_LOAD) {
            emit(FK_MOVE_IN, 0, false, dst_off, 0, static_cast<int>(oa));
        }
        else if (op == DPB_FUSED_STORE) {
            if (oa == kOpndAcc) emit(FK_STORE, 0, false, -1, 0, static_cast<int>(ob));
            else emit(FK_STORE_ANY, 0, false, -1, static_cast<int>(oa), static_cast<int>(ob));
        }
        else if (op == DPB_FUSED_SELECT) {
            emit(FK_SELECT, 0, false, dst_off, static_cast<int>(oa | (ob << 8) | (oc << 16)), 0);
        }
        else if (op < DPB_FUSED_FIRST_BINARY) {
            if (oa != kOpndAcc) emit_move(oa, -1);
            emit(FK_UNARY, op, false, dst_off, 0, 0);
        }
        else {
            if (oa != kOpndAcc && ob == kOpndAcc) {   // give the accumulator as the first operand
                const unsigned t = oa;
                oa = ob;
                ob = t;
                swap = !swap;
            }
            if (oa != kOpndAcc) emit_move(oa, -1);
            if (ob == kOpndAcc) emit(FK_BIN_ACC, op, swap, dst_off, 0, 0);
            else if (ob >= kOpndIn) emit(FK_BIN_IN, op, swap, dst_off, 0, static_cast<int>(ob - kOpndIn));
            else if (ob >= kOpndImm) emit(FK_BIN_IMM, op, swap, dst_off, 0, static_cast<int>(ob - kOpndImm));
            else emit(FK_BIN_REG, op, swap, dst_off, static_cast<int>(ob) * NV, 0);
        }
    }
    prm.n_uop = nu;
    const size_t smem = static_cast<size_t>(prog->n_reg > 0 ? prog->n_reg : 1) * K * kFusedThreads * elem;
    if (smem > device_props().max_smem_optin)
        return set_error(DPB_ERR_VALUE, "fused program: %d registers do not fit in shared memory", prog->n_reg);
    const int64_t tile = int64_t(kFusedThreads) * K;
    const int64_t blocks = (n + tile - 1) / tile;
    if (blocks > 0x7fffffff) return set_error(DPB_ERR_VALUE, "fused program: too many elements for one launch");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define DPB_FUSED_LAUNCH(T, KK)                                                                              \
    do {                                                                                                     \
        DPB_CUDA_TRY(cudaFuncSetAttribute(ew_fused_kernel<T, KK>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                          static_cast<int>(smem)));                                          \
        ew_fused_kernel<T, KK><<<static_cast<int>(blocks), kFusedThreads, smem, s>>>(prm, n);                \
    } while (0)
    if (prog->typenum == DPB_DOUBLE) {
        if (K == 8) DPB_FUSED_LAUNCH(double, 8);
        else DPB_FUSED_LAUNCH(double, 4);
    }
    else {
        if (K == 8) DPB_FUSED_LAUNCH(float, 8);
        else DPB_FUSED_LAUNCH(float, 4);
    }
#undef DPB_FUSED_LAUNCH
    note_kernel("ew_fused");
    return check_launch("ew_fused");
}

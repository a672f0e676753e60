// Fused elementwise chains, specialised: the program that ew_fused.cu interprets is written
// out as straight-line CUDA C++ -- one statement per instruction, calling the same operator
// classes (ew_ops.cuh) as the per-op kernels and the interpreter -- compiled at first use with
// the run-time compiler (NVRTC, for the architecture of the current device, without
// multiply-add contraction like the rest of the library) and kept for the life of the process.
// Every virtual register becomes a local variable, so the chain runs out of real registers with
// no dispatch at all: the kernel is the one a programmer would have written by hand for the
// chain (compare bs_fused.cu), and its results have the bits of the unfused chain.
//
// The reference has no fusion (see ew_fused.cu); nothing here has a counterpart there.
//
// NVRTC and the driver API are loaded with dlopen at first use: the library does not link
// against them, and `dpb_fused_specialize_available` says whether this path can run.  The
// operator headers are read from the directory `csrc` next to the shared library (they ship
// with the package); `csrc/rtc` holds stand-ins for the few host headers they include.
#include <dlfcn.h>
#include <sys/stat.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "ew_fused.h"

namespace dpb {
namespace {

// ------------------------------------------------------------------ the two libraries
typedef struct _nvrtcProgram *nvrtcProgram;
struct Nvrtc {
    void *handle = nullptr;
    int (*CreateProgram)(nvrtcProgram *, const char *, const char *, int, const char *const *, const char *const *);
    int (*CompileProgram)(nvrtcProgram, int, const char *const *);
    int (*DestroyProgram)(nvrtcProgram *);
    int (*GetProgramLogSize)(nvrtcProgram, size_t *);
    int (*GetProgramLog)(nvrtcProgram, char *);
    int (*GetCUBINSize)(nvrtcProgram, size_t *);
    int (*GetCUBIN)(nvrtcProgram, char *);
    const char *(*GetErrorString)(int);
};
struct Driver {
    void *handle = nullptr;
    int (*ModuleLoadData)(void **, const void *);
    int (*ModuleGetFunction)(void **, void *, const char *);
    int (*LaunchKernel)(void *, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, void *,
                        void **, void **);
    int (*GetErrorString)(int, const char **);
};

std::mutex g_mutex;
Nvrtc g_rtc;
Driver g_drv;
std::string g_load_error;
bool g_load_tried = false;
std::string g_include_override;    // dpb_fused_set_include_path

template <class F> bool sym(void *h, const char *name, F &fn)
{
    fn = reinterpret_cast<F>(dlsym(h, name));
    if (!fn) g_load_error = std::string("symbol ") + name + " not found";
    return fn != nullptr;
}

bool file_exists(const std::string &p)
{
    struct stat st;
    return stat(p.c_str(), &st) == 0;
}

// directory of this shared library
std::string library_dir()
{
    Dl_info info;
    if (!dladdr(reinterpret_cast<const void *>(&library_dir), &info) || !info.dli_fname) return ".";
    std::string p(info.dli_fname);
    const size_t slash = p.rfind('/');
    return slash == std::string::npos ? "." : p.substr(0, slash);
}

// -I directories: the operator headers, the stand-ins for host headers, the CUDA headers
std::vector<std::string> include_dirs()
{
    std::vector<std::string> dirs;
    if (!g_include_override.empty()) {
        size_t a = 0;
        while (a <= g_include_override.size()) {
            size_t b = g_include_override.find(':', a);
            if (b == std::string::npos) b = g_include_override.size();
            if (b > a) dirs.push_back(g_include_override.substr(a, b - a));
            a = b + 1;
        }
        return dirs;
    }
    const std::string csrc = library_dir() + "/csrc";
    dirs.push_back(csrc + "/rtc");
    dirs.push_back(csrc);
    for (const char *var : {"DPNP_B200_CUDA_INCLUDE", "CUDA_HOME", "CUDA_PATH"}) {
        const char *v = std::getenv(var);
        if (!v || !*v) continue;
        std::string d = std::string(v) + (std::strcmp(var, "DPNP_B200_CUDA_INCLUDE") ? "/include" : "");
        if (file_exists(d + "/cuda_fp16.h")) {
            dirs.push_back(d);
            return dirs;
        }
    }
    dirs.push_back("/usr/local/cuda/include");
    return dirs;
}

bool load_libraries()
{
    if (g_load_tried) return g_rtc.handle && g_drv.handle;
    g_load_tried = true;
    const char *named = std::getenv("DPNP_B200_NVRTC_LIB");
    std::vector<std::string> names;
    if (named && *named) names.push_back(named);
    names.insert(names.end(), {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                               "/usr/local/cuda/lib64/libnvrtc.so"});
    void *h = nullptr;
    for (const std::string &n : names)
        if ((h = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL))) break;
    if (!h) {
        g_load_error = "the run-time compiler (libnvrtc) was not found";
        return false;
    }
    Nvrtc r;
    r.handle = h;
    if (!sym(h, "nvrtcCreateProgram", r.CreateProgram) || !sym(h, "nvrtcCompileProgram", r.CompileProgram) ||
        !sym(h, "nvrtcDestroyProgram", r.DestroyProgram) || !sym(h, "nvrtcGetProgramLogSize", r.GetProgramLogSize) ||
        !sym(h, "nvrtcGetProgramLog", r.GetProgramLog) || !sym(h, "nvrtcGetCUBINSize", r.GetCUBINSize) ||
        !sym(h, "nvrtcGetCUBIN", r.GetCUBIN) || !sym(h, "nvrtcGetErrorString", r.GetErrorString))
        return false;
    g_rtc = r;
    void *d = dlopen("libcuda.so.1", RTLD_NOW | RTLD_LOCAL);
    if (!d) {
        // no driver on this machine: compiling still works (tests without a GPU), launching does not
        g_load_error = "the CUDA driver library (libcuda.so.1) was not found";
        return false;
    }
    Driver v;
    v.handle = d;
    if (!sym(d, "cuModuleLoadData", v.ModuleLoadData) || !sym(d, "cuModuleGetFunction", v.ModuleGetFunction) ||
        !sym(d, "cuLaunchKernel", v.LaunchKernel) || !sym(d, "cuGetErrorString", v.GetErrorString))
        return false;
    g_drv = v;
    return true;
}

// ------------------------------------------------------------------ source generation
const char *unary_class(int op)
{
    switch (op) {
    case DPB_FUSED_NEGATIVE: return "NegativeOp";
    case DPB_FUSED_ABS: return "AbsOp";
    case DPB_FUSED_EXP: return "ExpOp";
    case DPB_FUSED_LOG: return "LogOp";
    case DPB_FUSED_SQRT: return "SqrtOp";
    case DPB_FUSED_ERF: return "ErfOp";
    case DPB_FUSED_SQUARE: return "SquareOp";
    case DPB_FUSED_RECIPROCAL: return "ReciprocalOp";
    case DPB_FUSED_SIN: return "SinOp";
    case DPB_FUSED_COS: return "CosOp";
    case DPB_FUSED_TANH: return "TanhOp";
    case DPB_FUSED_EXPM1: return "Expm1Op";
    case DPB_FUSED_LOG1P: return "Log1pOp";
    case DPB_FUSED_FLOOR: return "FloorOp";
    case DPB_FUSED_CEIL: return "CeilOp";
    case DPB_FUSED_SIGN: return "SignOp";
    default: return nullptr;   // move, positive: the value itself
    }
}

// expression of a binary operator applied to x and y (both of type T)
std::string binary_expr(int op, const std::string &x, const std::string &y)
{
    auto call = [&](const char *cls) { return std::string(cls) + "<T, T>::apply(" + x + ", " + y + ")"; };
    auto flag = [&](const char *cls) { return "(" + call(cls) + ".v ? T(1) : T(0))"; };
    switch (op) {
    case DPB_FUSED_ADD: return call("AddOp");
    case DPB_FUSED_SUBTRACT: return call("SubtractOp");
    case DPB_FUSED_MULTIPLY: return call("MultiplyOp");
    case DPB_FUSED_DIVIDE: return call("TrueDivideOp");
    case DPB_FUSED_MAXIMUM: return call("MaximumOp");
    case DPB_FUSED_MINIMUM: return call("MinimumOp");
    case DPB_FUSED_POW: return call("PowOp");
    case DPB_FUSED_LESS: return flag("LessOp");
    case DPB_FUSED_LESS_EQUAL: return flag("LessEqualOp");
    case DPB_FUSED_GREATER: return flag("GreaterOp");
    case DPB_FUSED_GREATER_EQUAL: return flag("GreaterEqualOp");
    case DPB_FUSED_EQUAL: return flag("EqualOp");
    case DPB_FUSED_NOT_EQUAL: return flag("NotEqualOp");
    case DPB_FUSED_LOGICAL_AND: return "((" + x + " != T(0) && " + y + " != T(0)) ? T(1) : T(0))";
    default: return "((" + x + " != T(0) || " + y + " != T(0)) ? T(1) : T(0))";   // DPB_FUSED_LOGICAL_OR
    }
}

std::string operand(unsigned code)
{
    if (code == kOpndAcc) return "acc";
    if (code >= kOpndIn) return "x" + std::to_string(code - kOpndIn);
    if (code >= kOpndImm) return "c" + std::to_string(code - kOpndImm);
    return "r" + std::to_string(code);
}

// The program must have passed fused_check_program.
std::string generate_source(const dpb_fused_program *prog)
{
    const int n_in = prog->n_in, n_out = prog->n_out, n_imm = prog->n_imm;
    std::string s;
    s += "#include \"ew_ops.cuh\"\n#include \"ew_erf.cuh\"\nusing namespace dpb;\n";
    s += std::string("typedef ") + (prog->typenum == DPB_DOUBLE ? "double" : "float") + " T;\n";
    s += "constexpr int VW = 16 / sizeof(T);\ntypedef vec_t<T, VW> V;\n";
    s += "struct Args {\n    const T *in[" + std::to_string(n_in > 0 ? n_in : 1) + "];\n    T *out[" +
         std::to_string(n_out > 0 ? n_out : 1) + "];\n    double imm[" + std::to_string(n_imm > 0 ? n_imm : 1) +
         "];\n};\n\n";
    // ---- one element
    s += "// one element of the chain: x* inputs, c* scalars, r* registers, y* outputs\n";
    s += "__device__ __forceinline__ void chain(const Args &a";
    for (int i = 0; i < n_in; ++i) s += ", const T x" + std::to_string(i);
    for (int i = 0; i < n_out; ++i) s += ", T &y" + std::to_string(i);
    s += ")\n{\n";
    for (int i = 0; i < n_imm; ++i)
        s += "    const T c" + std::to_string(i) + " = static_cast<T>(a.imm[" + std::to_string(i) + "]);\n";
    if (prog->n_reg > 0) {
        s += "    T r0";
        for (int i = 1; i < prog->n_reg; ++i) s += ", r" + std::to_string(i);
        s += ";\n";
    }
    s += "    T acc = T(0);\n";
    for (int pc = 0; pc < prog->n_instr; ++pc) {
        const uint64_t w = prog->code[pc];
        const int op = static_cast<int>(w & 0xff);
        const unsigned dst = static_cast<unsigned>((w >> 8) & 0xff);
        const unsigned oa = static_cast<unsigned>((w >> 16) & 0xff);
        const unsigned ob = static_cast<unsigned>((w >> 24) & 0xff);
        const unsigned oc = static_cast<unsigned>((w >> 32) & 0xff);
        const bool swap = (w >> 40) & 1;
        std::string line;
        if (op == DPB_FUSED_STORE) {
            s += "    y" + std::to_string(ob) + " = " + operand(oa) + ";\n";
            continue;
        }
        if (op == DPB_FUSED_LOAD) line = "x" + std::to_string(oa);
        else if (op == DPB_FUSED_SELECT)
            line = "(" + operand(oa) + " != T(0)) ? " + operand(ob) + " : " + operand(oc);
        else if (op < DPB_FUSED_FIRST_BINARY) {
            const char *cls = unary_class(op);
            line = cls ? std::string(cls) + "<T>::apply(" + operand(oa) + ")" : operand(oa);
        }
        else {
            // the word may carry the operands exchanged (the interpreter wants the accumulator first)
            line = swap ? binary_expr(op, operand(ob), operand(oa)) : binary_expr(op, operand(oa), operand(ob));
        }
        s += "    acc = " + line + ";\n";
        if (dst != kNoDst) s += "    r" + std::to_string(dst) + " = acc;\n";
    }
    s += "}\n\n";
    // ---- the kernel: 16-byte accesses over a capped grid, the ragged end and unaligned arrays
    // element by element
    auto scalar = [&](int i) { return prog->in_is_scalar && prog->in_is_scalar[i]; };
    s += "extern \"C\" __global__ void __launch_bounds__(256) fused_chain(const __grid_constant__ Args a, "
         "const long long n, const int vector_io)\n{\n";
    for (int i = 0; i < n_in; ++i)
        if (scalar(i)) s += "    const T s" + std::to_string(i) + " = a.in[" + std::to_string(i) + "][0];\n";
    s += "    const long long stride = (long long)gridDim.x * 256;\n";
    s += "    const long long first = (long long)blockIdx.x * 256 + threadIdx.x;\n";
    s += "    if (vector_io) {\n        const long long nvec = n / VW;\n";
    s += "        for (long long v = first; v < nvec; v += stride) {\n";
    for (int i = 0; i < n_in; ++i)
        if (!scalar(i))
            s += "            const V vx" + std::to_string(i) + " = load_vec<V>(a.in[" + std::to_string(i) + "] + v * VW);\n";
    for (int i = 0; i < n_out; ++i) s += "            V vy" + std::to_string(i) + ";\n";
    s += "#pragma unroll\n            for (int k = 0; k < VW; ++k) {\n                chain(a";
    for (int i = 0; i < n_in; ++i)
        s += scalar(i) ? ", s" + std::to_string(i) : ", vx" + std::to_string(i) + ".v[k]";
    for (int i = 0; i < n_out; ++i) s += ", vy" + std::to_string(i) + ".v[k]";
    s += ");\n            }\n";
    for (int i = 0; i < n_out; ++i)
        s += "            store_vec(a.out[" + std::to_string(i) + "] + v * VW, vy" + std::to_string(i) + ");\n";
    s += "        }\n";
    s += "        if (blockIdx.x == 0) {\n            for (long long i = nvec * VW + threadIdx.x; i < n; i += 256) {\n";
    auto element = [&](const char *indent) {
        std::string e;
        for (int i = 0; i < n_out; ++i) e += std::string(indent) + "T y" + std::to_string(i) + ";\n";
        e += std::string(indent) + "chain(a";
        for (int i = 0; i < n_in; ++i)
            e += scalar(i) ? ", s" + std::to_string(i) : ", a.in[" + std::to_string(i) + "][i]";
        for (int i = 0; i < n_out; ++i) e += ", y" + std::to_string(i);
        e += ");\n";
        for (int i = 0; i < n_out; ++i)
            e += std::string(indent) + "a.out[" + std::to_string(i) + "][i] = y" + std::to_string(i) + ";\n";
        return e;
    };
    s += element("                ");
    s += "            }\n        }\n    }\n    else {\n        for (long long i = first; i < n; i += stride) {\n";
    s += element("            ");
    s += "        }\n    }\n}\n";
    return s;
}

// ------------------------------------------------------------------ compiled kernels
struct Compiled {
    std::vector<char> cubin;
    std::map<int, void *> function;   // device ordinal -> CUfunction (a module per device)
    std::string source;
};
std::map<std::string, Compiled> g_cache;

// what a compiled kernel depends on: type, counts, scalar inputs, the instruction words
std::string program_key(const dpb_fused_program *prog, const std::string &arch)
{
    std::string k = arch;
    const int32_t head[6] = {prog->typenum, prog->n_instr, prog->n_reg, prog->n_imm, prog->n_in, prog->n_out};
    k.append(reinterpret_cast<const char *>(head), sizeof head);
    for (int i = 0; i < prog->n_in; ++i) k.push_back(prog->in_is_scalar && prog->in_is_scalar[i] ? 1 : 0);
    k.append(reinterpret_cast<const char *>(prog->code), sizeof(uint64_t) * size_t(prog->n_instr));
    return k;
}

int compile(const dpb_fused_program *prog, const std::string &arch, Compiled &out)
{
    if (!g_rtc.handle) return set_error(DPB_ERR_RUNTIME, "fused chain: %s", g_load_error.c_str());
    out.source = generate_source(prog);
    nvrtcProgram p = nullptr;
    int rc = g_rtc.CreateProgram(&p, out.source.c_str(), "fused_chain.cu", 0, nullptr, nullptr);
    if (rc != 0) return set_error(DPB_ERR_RUNTIME, "nvrtcCreateProgram: %s", g_rtc.GetErrorString(rc));
    std::vector<std::string> opts = {"--gpu-architecture=" + arch, "--std=c++17", "--fmad=false", "-default-device"};
    for (const std::string &d : include_dirs()) opts.push_back("-I" + d);
    std::vector<const char *> argv;
    for (const std::string &o : opts) argv.push_back(o.c_str());
    rc = g_rtc.CompileProgram(p, static_cast<int>(argv.size()), argv.data());
    if (rc != 0) {
        size_t len = 0;
        g_rtc.GetProgramLogSize(p, &len);
        std::string log(len, '\0');
        if (len) g_rtc.GetProgramLog(p, &log[0]);
        g_rtc.DestroyProgram(&p);
        if (log.size() > 1500) log.resize(1500);
        return set_error(DPB_ERR_RUNTIME, "fused chain: run-time compilation failed (%s): %s", g_rtc.GetErrorString(rc),
                         log.c_str());
    }
    size_t size = 0;
    rc = g_rtc.GetCUBINSize(p, &size);
    if (rc == 0 && size > 0) {
        out.cubin.resize(size);
        rc = g_rtc.GetCUBIN(p, out.cubin.data());
    }
    g_rtc.DestroyProgram(&p);
    if (rc != 0 || size == 0) return set_error(DPB_ERR_RUNTIME, "fused chain: no device code was produced");
    return DPB_OK;
}

std::string device_arch(int *ordinal)
{
    int dev = 0, major = 0, minor = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) {
        cudaGetLastError();
        if (ordinal) *ordinal = -1;
        return "sm_100a";   // no device: compile for the architecture the library is built for
    }
    if (ordinal) *ordinal = dev;
    return "sm_" + std::to_string(major) + std::to_string(minor) + (major >= 9 ? "a" : "");
}

// compiled entry for the program (compiling it if this is the first time); g_mutex is held
int lookup(const dpb_fused_program *prog, const std::string &arch, Compiled **out)
{
    const std::string key = program_key(prog, arch);
    auto it = g_cache.find(key);
    if (it == g_cache.end()) {
        Compiled c;
        DPB_TRY(compile(prog, arch, c));
        it = g_cache.emplace(key, std::move(c)).first;
    }
    *out = &it->second;
    return DPB_OK;
}

}  // namespace
}  // namespace dpb

using namespace dpb;

extern "C" int dpb_fused_specialize_available(void)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!load_libraries()) return 0;
    const std::vector<std::string> dirs = include_dirs();
    bool ops = false, cuda = false;
    for (const std::string &d : dirs) {
        ops = ops || file_exists(d + "/ew_ops.cuh");
        cuda = cuda || file_exists(d + "/cuda_fp16.h");
    }
    return ops && cuda ? 1 : 0;
}

extern "C" int dpb_fused_set_include_path(const char *colon_separated)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    g_include_override = colon_separated ? colon_separated : "";
    return DPB_OK;
}

extern "C" int dpb_fused_specialized_source(const dpb_fused_program *prog, char *buf, int64_t buf_len, int64_t *needed)
{
    DPB_TRY(fused_check_program(prog, 0, nullptr));
    const std::string src = generate_source(prog);
    if (needed) *needed = static_cast<int64_t>(src.size()) + 1;
    if (buf && buf_len > 0) {
        const size_t n = std::min<size_t>(src.size(), static_cast<size_t>(buf_len) - 1);
        std::memcpy(buf, src.data(), n);
        buf[n] = '\0';
    }
    return DPB_OK;
}

extern "C" int dpb_fused_specialize_compile(const dpb_fused_program *prog, int64_t *cubin_bytes)
{
    DPB_TRY(fused_check_program(prog, 0, nullptr));
    std::lock_guard<std::mutex> lock(g_mutex);
    load_libraries();
    Compiled *c = nullptr;
    DPB_TRY(lookup(prog, device_arch(nullptr), &c));
    if (cubin_bytes) *cubin_bytes = static_cast<int64_t>(c->cubin.size());
    return DPB_OK;
}

extern "C" int dpb_fused_elementwise_specialized(const dpb_fused_program *prog, int64_t n, void *stream)
{
    bool aligned = true;
    DPB_TRY(fused_check_program(prog, n, &aligned));
    if (n == 0 || prog->n_instr == 0) return DPB_OK;
    void *fn = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!load_libraries()) return set_error(DPB_ERR_RUNTIME, "fused chain: %s", g_load_error.c_str());
        int dev = -1;
        const std::string arch = device_arch(&dev);
        if (dev < 0) return set_error(DPB_ERR_RUNTIME, "fused chain: no CUDA device");
        Compiled *c = nullptr;
        DPB_TRY(lookup(prog, arch, &c));
        auto it = c->function.find(dev);
        if (it == c->function.end()) {
            DPB_CUDA_TRY(cudaFree(nullptr));   // the device's primary context is current from here on
            void *module = nullptr, *f = nullptr;
            int rc = g_drv.ModuleLoadData(&module, c->cubin.data());
            if (rc == 0) rc = g_drv.ModuleGetFunction(&f, module, "fused_chain");
            if (rc != 0) {
                const char *msg = nullptr;
                g_drv.GetErrorString(rc, &msg);
                return set_error(DPB_ERR_RUNTIME, "fused chain: loading the compiled kernel failed: %s", msg ? msg : "?");
            }
            it = c->function.emplace(dev, f).first;
        }
        fn = it->second;
    }
    // the kernel's Args: in[max(n_in,1)], out[max(n_out,1)], imm[max(n_imm,1)] -- all 8-byte fields
    const int n_in = prog->n_in > 0 ? prog->n_in : 1, n_out = prog->n_out > 0 ? prog->n_out : 1;
    uint64_t args[kFusedMaxIn + kFusedMaxOut + kFusedMaxImm];
    std::memset(args, 0, sizeof args);
    for (int i = 0; i < prog->n_in; ++i) args[i] = reinterpret_cast<uint64_t>(prog->in[i]);
    for (int i = 0; i < prog->n_out; ++i) args[n_in + i] = reinterpret_cast<uint64_t>(prog->out[i]);
    for (int i = 0; i < prog->n_imm; ++i) std::memcpy(&args[n_in + n_out + i], &prog->imm[i], sizeof(double));
    const size_t elem = prog->typenum == DPB_DOUBLE ? 8 : 4;
    const int64_t vw = static_cast<int64_t>(16 / elem);
    const int64_t work = aligned ? std::max<int64_t>(1, n / vw) : n;
    const int64_t cap = int64_t(device_props().sm_count) * tuning_ctas_per_sm();
    const int64_t blocks = std::max<int64_t>(1, std::min(cap, ceil_div(work, 256)));
    long long n_arg = n;
    int vector_io = aligned ? 1 : 0;
    void *params[3] = {args, &n_arg, &vector_io};
    const int rc = g_drv.LaunchKernel(fn, static_cast<unsigned>(blocks), 1, 1, 256, 1, 1, 0, stream, params, nullptr);
    if (rc != 0) {
        const char *msg = nullptr;
        g_drv.GetErrorString(rc, &msg);
        return set_error(DPB_ERR_RUNTIME, "fused chain: launch failed: %s", msg ? msg : "?");
    }
    note_kernel("ew_fused_specialized");
    return DPB_OK;
}

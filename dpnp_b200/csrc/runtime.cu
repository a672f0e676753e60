// Host runtime of libdpnp_b200: thread-local error state, device selection,
// streams/events, the stream-ordered allocator and raw copies.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

#include "common.cuh"

namespace dpb {

static thread_local char g_err[1024] = "";
static thread_local const char *g_last_kernel = "";
static thread_local int64_t g_launches = 0;

int set_error(int status, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

// Run-time switches, read once from the environment (DPNP_B200_VERBOSE, DPNP_B200_FORCE_GENERIC;
// the reference's counterparts are the DPNP_* / SYCL_* variables of dpnp/config.py:32-59) and
// changeable through dpb_set_tuning("verbose" | "force_generic", 0 | 1).
static int env_flag(const char *name)
{
    const char *v = getenv(name);
    return (v && *v && std::strcmp(v, "0") != 0) ? 1 : 0;
}
static std::atomic<int> g_verbose{-1}, g_force_generic{-1};
bool tuning_verbose()
{
    int v = g_verbose.load(std::memory_order_relaxed);
    if (v < 0) {
        v = env_flag("DPNP_B200_VERBOSE");
        g_verbose.store(v);
    }
    return v != 0;
}
bool tuning_force_generic()
{
    int v = g_force_generic.load(std::memory_order_relaxed);
    if (v < 0) {
        v = env_flag("DPNP_B200_FORCE_GENERIC");
        g_force_generic.store(v);
    }
    return v != 0;
}

void note_kernel(const char *name)
{
    g_last_kernel = name;
    ++g_launches;
    if (tuning_verbose())
        fprintf(stderr, "[dpnp_b200] launch %lld of this thread: %s\n", static_cast<long long>(g_launches), name);
}

void note_copy(const char *name) { g_last_kernel = name; }

int check_launch(const char *what)
{
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        return set_error(DPB_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(err));
    }
    return DPB_OK;
}

static constexpr int kMaxDevices = 64;
static DeviceProps g_props[kMaxDevices];
static std::atomic<bool> g_props_ready[kMaxDevices];
static std::mutex g_props_mutex;

const DeviceProps &device_props()
{
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices) dev = 0;
    if (!g_props_ready[dev].load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_props_mutex);
        if (!g_props_ready[dev].load(std::memory_order_relaxed)) {
            int sm = 0, smem = 0;
            if (cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
                sm <= 0)
                sm = 148;
            if (cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) !=
                cudaSuccess)
                smem = 48 * 1024;
            g_props[dev].sm_count = sm;
            g_props[dev].max_smem_optin = smem;
            g_props_ready[dev].store(true, std::memory_order_release);
        }
    }
    return g_props[dev];
}

static std::atomic<int64_t> g_ctas_per_sm{8};
int64_t tuning_ctas_per_sm() { return g_ctas_per_sm.load(std::memory_order_relaxed); }
static std::atomic<int> g_pdl{1};
bool tuning_pdl() { return g_pdl.load(std::memory_order_relaxed) != 0; }
static std::atomic<int64_t> g_peer_polls{int64_t(1) << 24};
int64_t tuning_peer_polls() { return g_peer_polls.load(std::memory_order_relaxed); }
static std::atomic<int64_t> g_scan_polls{-1};
int64_t tuning_scan_lookback_polls() { return g_scan_polls.load(std::memory_order_relaxed); }
static std::atomic<int64_t> g_fused_elems{8};
int64_t tuning_fused_elems() { return g_fused_elems.load(std::memory_order_relaxed); }


// --------------------------------------------------------- guarded blocks
// A debugging aid for kernels that write where they should not (compute-sanitizer's memcheck is
// not always available): when switched on ("redzones" tuning key, DPNP_B200_REDZONES=1), every
// block of the pool gets kRedzone bytes in front and behind, filled with a pattern when the block
// is handed out and compared with it when the block comes back.  Both steps are kernels on the
// block's stream; a mismatch is counted in device memory and the first one is remembered.  Nothing
// traps: dpb_debug_redzone_report reads the counters.
constexpr size_t kRedzone = 512;
constexpr unsigned char kRedzoneByte = 0xA5;
__device__ unsigned long long g_rz_bad_bytes = 0;
__device__ unsigned long long g_rz_bad_blocks = 0;
__device__ unsigned long long g_rz_first[3] = {0, 0, 0};   // user pointer, user size, offset of the bad byte

__global__ void redzone_fill_kernel(unsigned char *base, size_t user_bytes)
{
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < kRedzone) {
        base[i] = kRedzoneByte;
        base[kRedzone + user_bytes + i] = kRedzoneByte;
    }
}

__global__ void redzone_check_kernel(const unsigned char *base, size_t user_bytes)
{
    __shared__ unsigned bad;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < 2 * kRedzone) {
        const bool front = i < kRedzone;
        const size_t at = front ? i : user_bytes + i;   // offset from base
        if (base[at] != kRedzoneByte) {
            atomicAdd(&bad, 1u);
            if (atomicAdd(&g_rz_bad_bytes, 1ull) == 0) {
                g_rz_first[0] = reinterpret_cast<unsigned long long>(base + kRedzone);
                g_rz_first[1] = user_bytes;
                // bytes before the block count as negative offsets
                g_rz_first[2] = static_cast<unsigned long long>(static_cast<long long>(at) - static_cast<long long>(kRedzone));
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && bad) atomicAdd(&g_rz_bad_blocks, 1ull);
}

static std::atomic<int> g_redzones{-1};
static bool redzones_on()
{
    int v = g_redzones.load(std::memory_order_relaxed);
    if (v < 0) {
        v = env_flag("DPNP_B200_REDZONES");
        g_redzones.store(v);
    }
    return v != 0;
}

// ------------------------------------------------------------------- pool
struct PoolState {
    std::atomic<bool> configured{false};
    std::atomic<size_t> live{0};
    std::atomic<size_t> live_high{0};
};
static PoolState g_pool[kMaxDevices];
static std::atomic<size_t> g_pool_limit{0};
static std::mutex g_pool_mutex;
// size of every live block, so that dpb_free can keep the live-byte count exact
struct BlockInfo {
    int device;
    size_t request;   // bytes taken from the pool (with the guard zones, if any)
    size_t user;      // bytes the caller asked for
    bool guarded;
};
static std::unordered_map<void *, BlockInfo> g_blocks;
static std::mutex g_blocks_mutex;

static int configure_pool(int dev)
{
    if (g_pool[dev].configured.load(std::memory_order_acquire)) return DPB_OK;
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    if (g_pool[dev].configured.load(std::memory_order_relaxed)) return DPB_OK;
    cudaMemPool_t pool;
    DPB_CUDA_TRY(cudaDeviceGetDefaultMemPool(&pool, dev));
    // Keep freed blocks cached instead of returning them to the driver at
    // every synchronisation: allocation then costs no driver call.
    uint64_t threshold = UINT64_MAX;
    DPB_CUDA_TRY(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold));
    g_pool[dev].configured.store(true, std::memory_order_release);
    return DPB_OK;
}

}  // namespace dpb

using namespace dpb;

extern "C" {

const char *dpb_last_error(void) { return g_err; }
const char *dpb_version(void) { return "dpnp_b200 0.1 (sm_100a)"; }
const char *dpb_last_kernel(void) { return g_last_kernel; }
int64_t dpb_launch_count(void) { return g_launches; }
void dpb_reset_launch_count(void) { g_launches = 0; }

int dpb_set_tuning(const char *key, int64_t value)
{
    if (key && std::strcmp(key, "ctas_per_sm") == 0 && value >= 1 && value <= 64) {
        g_ctas_per_sm.store(value);
        return DPB_OK;
    }
    if (key && std::strcmp(key, "fused_elems_per_thread") == 0 && (value == 4 || value == 8)) {
        g_fused_elems.store(value);
        return DPB_OK;
    }
    if (key && std::strcmp(key, "pdl") == 0 && (value == 0 || value == 1)) {
        g_pdl.store(static_cast<int>(value));
        return DPB_OK;
    }
    if (key && std::strcmp(key, "peer_polls") == 0 && value >= 0 && value <= (int64_t(1) << 24)) {
        g_peer_polls.store(value);
        return DPB_OK;
    }
    if (key && std::strcmp(key, "scan_lookback_polls") == 0 && value >= -1 && value <= (int64_t(1) << 30)) {
        g_scan_polls.store(value);
        return DPB_OK;
    }
    if (key && std::strcmp(key, "redzones") == 0 && (value == 0 || value == 1)) {
        g_redzones.store(static_cast<int>(value));
        return DPB_OK;
    }
    if (key && std::strcmp(key, "verbose") == 0 && (value == 0 || value == 1)) {
        g_verbose.store(static_cast<int>(value));
        return DPB_OK;
    }
    if (key && std::strcmp(key, "force_generic") == 0 && (value == 0 || value == 1)) {
        g_force_generic.store(static_cast<int>(value));
        return DPB_OK;
    }
    return set_error(DPB_ERR_VALUE, "unknown tuning key or value out of range: %s",
                     key ? key : "(null)");
}

int dpb_device_count(void)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int dpb_device_pci_bus_id(int device, char *buf, int len)
{
    if (!buf || len < 16) return set_error(DPB_ERR_VALUE, "dpb_device_pci_bus_id: a buffer of at least 16 bytes is needed");
    DPB_CUDA_TRY(cudaDeviceGetPCIBusId(buf, len, device));
    return DPB_OK;
}

int dpb_set_device(int device)
{
    DPB_CUDA_TRY(cudaSetDevice(device));
    return DPB_OK;
}

int dpb_get_device(int *device)
{
    DPB_CUDA_TRY(cudaGetDevice(device));
    return DPB_OK;
}

int dpb_device_info(int device, int *sm_count, size_t *total_mem, int *cc_major, int *cc_minor)
{
    cudaDeviceProp p;
    DPB_CUDA_TRY(cudaGetDeviceProperties(&p, device));
    if (sm_count) *sm_count = p.multiProcessorCount;
    if (total_mem) *total_mem = p.totalGlobalMem;
    if (cc_major) *cc_major = p.major;
    if (cc_minor) *cc_minor = p.minor;
    return DPB_OK;
}

int dpb_stream_create(void **stream)
{
    cudaStream_t s;
    DPB_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return DPB_OK;
}

int dpb_stream_destroy(void *stream)
{
    DPB_CUDA_TRY(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
    return DPB_OK;
}

int dpb_stream_synchronize(void *stream)
{
    DPB_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return DPB_OK;
}

int dpb_device_synchronize(void)
{
    DPB_CUDA_TRY(cudaDeviceSynchronize());
    return DPB_OK;
}

int dpb_event_create(void **event)
{
    cudaEvent_t e;
    DPB_CUDA_TRY(cudaEventCreate(&e));
    *event = e;
    return DPB_OK;
}

int dpb_event_destroy(void *event)
{
    DPB_CUDA_TRY(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
    return DPB_OK;
}

int dpb_event_record(void *event, void *stream)
{
    DPB_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
    return DPB_OK;
}

int dpb_stream_wait_event(void *stream, void *event)
{
    DPB_CUDA_TRY(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
    return DPB_OK;
}

int dpb_event_synchronize(void *event)
{
    DPB_CUDA_TRY(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
    return DPB_OK;
}

int dpb_event_elapsed_ms(void *start, void *stop, float *ms)
{
    DPB_CUDA_TRY(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start),
                                      static_cast<cudaEvent_t>(stop)));
    return DPB_OK;
}

int dpb_malloc(size_t nbytes, void *stream, void **ptr)
{
    if (!ptr) return set_error(DPB_ERR_VALUE, "dpb_malloc: null result pointer");
    *ptr = nullptr;
    const bool guarded = redzones_on();
    const size_t user = nbytes ? nbytes : 1;
    size_t request = guarded ? ((user + 15) / 16 * 16 + 2 * kRedzone) : user;
    size_t limit = g_pool_limit.load(std::memory_order_relaxed);
    if (limit && request > limit) {
        // decided before any CUDA call, so the check also works without a device
        return set_error(DPB_ERR_MEMORY,
                         "allocation of %zu bytes would exceed the pool limit of %zu bytes", request,
                         limit);
    }
    int dev = 0;
    DPB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices)
        return set_error(DPB_ERR_RUNTIME, "device ordinal %d out of range", dev);
    if (limit && g_pool[dev].live.load(std::memory_order_relaxed) + request > limit) {
        return set_error(DPB_ERR_MEMORY,
                         "allocation of %zu bytes would exceed the pool limit of %zu bytes", request,
                         limit);
    }
    DPB_TRY(configure_pool(dev));
    void *p = nullptr;
    cudaError_t err = cudaMallocAsync(&p, request, static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return set_error(err == cudaErrorMemoryAllocation ? DPB_ERR_MEMORY : DPB_ERR_CUDA,
                         "cudaMallocAsync of %zu bytes failed: %s", request,
                         cudaGetErrorString(err));
    }
    size_t now = g_pool[dev].live.fetch_add(request) + request;
    size_t high = g_pool[dev].live_high.load();
    while (now > high && !g_pool[dev].live_high.compare_exchange_weak(high, now)) {
    }
    if (guarded) {
        // the trailing zone starts right after the user's bytes, so a write one element past the end is seen
        redzone_fill_kernel<<<(kRedzone + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<unsigned char *>(p), user);
        p = static_cast<unsigned char *>(p) + kRedzone;
    }
    {
        std::lock_guard<std::mutex> lock(g_blocks_mutex);
        g_blocks[p] = BlockInfo{dev, request, user, guarded};
    }
    *ptr = p;
    return DPB_OK;
}

int dpb_free(void *ptr, void *stream)
{
    if (!ptr) return DPB_OK;
    BlockInfo info;
    {
        std::lock_guard<std::mutex> lock(g_blocks_mutex);
        auto it = g_blocks.find(ptr);
        if (it == g_blocks.end())
            return set_error(DPB_ERR_VALUE, "dpb_free: %p was not returned by dpb_malloc", ptr);
        info = it->second;
        g_pool[info.device].live.fetch_sub(info.request);
        g_blocks.erase(it);
    }
    if (info.guarded) {
        unsigned char *base = static_cast<unsigned char *>(ptr) - kRedzone;
        redzone_check_kernel<<<(2 * kRedzone + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(base, info.user);
        ptr = base;
    }
    DPB_CUDA_TRY(cudaFreeAsync(ptr, static_cast<cudaStream_t>(stream)));
    return DPB_OK;
}

int dpb_debug_redzone_report(int64_t *bad_blocks, int64_t *bad_bytes, int64_t *first3)
{
    DPB_CUDA_TRY(cudaDeviceSynchronize());
    unsigned long long blocks = 0, bytes = 0, first[3] = {0, 0, 0};
    DPB_CUDA_TRY(cudaMemcpyFromSymbol(&blocks, g_rz_bad_blocks, sizeof(blocks)));
    DPB_CUDA_TRY(cudaMemcpyFromSymbol(&bytes, g_rz_bad_bytes, sizeof(bytes)));
    DPB_CUDA_TRY(cudaMemcpyFromSymbol(first, g_rz_first, sizeof(first)));
    if (bad_blocks) *bad_blocks = static_cast<int64_t>(blocks);
    if (bad_bytes) *bad_bytes = static_cast<int64_t>(bytes);
    if (first3)
        for (int i = 0; i < 3; ++i) first3[i] = static_cast<int64_t>(first[i]);
    const unsigned long long zero[3] = {0, 0, 0};
    DPB_CUDA_TRY(cudaMemcpyToSymbol(g_rz_bad_blocks, zero, sizeof(unsigned long long)));
    DPB_CUDA_TRY(cudaMemcpyToSymbol(g_rz_bad_bytes, zero, sizeof(unsigned long long)));
    DPB_CUDA_TRY(cudaMemcpyToSymbol(g_rz_first, zero, sizeof(zero)));
    return DPB_OK;
}

int dpb_pool_trim(size_t keep_bytes)
{
    int dev = 0;
    DPB_CUDA_TRY(cudaGetDevice(&dev));
    cudaMemPool_t pool;
    DPB_CUDA_TRY(cudaDeviceGetDefaultMemPool(&pool, dev));
    DPB_CUDA_TRY(cudaMemPoolTrimTo(pool, keep_bytes));
    return DPB_OK;
}

int dpb_pool_stats(size_t *reserved, size_t *used, size_t *reserved_high, size_t *used_high)
{
    int dev = 0;
    DPB_CUDA_TRY(cudaGetDevice(&dev));
    cudaMemPool_t pool;
    DPB_CUDA_TRY(cudaDeviceGetDefaultMemPool(&pool, dev));
    uint64_t v = 0;
    if (reserved) {
        DPB_CUDA_TRY(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &v));
        *reserved = v;
    }
    if (used) {
        DPB_CUDA_TRY(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &v));
        *used = v;
    }
    if (reserved_high) {
        DPB_CUDA_TRY(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemHigh, &v));
        *reserved_high = v;
    }
    if (used_high) {
        DPB_CUDA_TRY(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemHigh, &v));
        *used_high = v;
    }
    return DPB_OK;
}

int dpb_pool_set_limit(size_t max_live_bytes)
{
    g_pool_limit.store(max_live_bytes);
    return DPB_OK;
}

int dpb_host_alloc(size_t nbytes, void **ptr)
{
    DPB_CUDA_TRY(cudaHostAlloc(ptr, nbytes ? nbytes : 1, cudaHostAllocDefault));
    return DPB_OK;
}

int dpb_host_free(void *ptr)
{
    if (!ptr) return DPB_OK;
    DPB_CUDA_TRY(cudaFreeHost(ptr));
    return DPB_OK;
}

int dpb_memcpy(void *dst, const void *src, size_t nbytes, int kind, void *stream)
{
    if (nbytes == 0) return DPB_OK;
    cudaMemcpyKind k;
    switch (kind) {
    case 0: k = cudaMemcpyHostToDevice; break;
    case 1: k = cudaMemcpyDeviceToHost; break;
    case 2: k = cudaMemcpyDeviceToDevice; break;
    default: return set_error(DPB_ERR_VALUE, "dpb_memcpy: unknown kind %d", kind);
    }
    DPB_CUDA_TRY(cudaMemcpyAsync(dst, src, nbytes, k, static_cast<cudaStream_t>(stream)));
    return DPB_OK;
}

int dpb_memset(void *dst, int value, size_t nbytes, void *stream)
{
    if (nbytes == 0) return DPB_OK;
    DPB_CUDA_TRY(cudaMemsetAsync(dst, value, nbytes, static_cast<cudaStream_t>(stream)));
    return DPB_OK;
}

}  // extern "C"

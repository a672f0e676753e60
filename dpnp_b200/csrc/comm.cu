// Combining per-GPU partial results of reductions over NVLink: one process per GPU, one NCCL
// communicator per process, loaded at run time (dlopen of libnccl.so.2) so that the library
// itself has no link-time dependency on it.
//
// The reference has no multi-device execution (an array is tied to one queue,
// dpnp/tensor/_compute_follows_data.pyx:67-160); these entry points are what a leading-axis
// sharded array needs on top of the single-device reductions:
//
//   dpb_comm_sum_ordered  all-gather of the ranks' partial sums into the communicator's gather
//                         buffer, then ONE kernel that adds the rows in rank order: every rank
//                         gets the same bits whatever order the collective moves data in
//   dpb_comm_extreme      the same with the NaN-propagating max / min of the reductions
//   dpb_comm_arg_extreme  each rank's (extreme value, global flat index of its first occurrence)
//                         is packed by a kernel, all-gathered, and a kernel on every rank picks
//                         the winner: better value, ties to the smaller index, NaN is extreme --
//                         nothing is read back to the host
//
// Everything is enqueued on the caller's stream.  The gather buffer is allocated once per
// communicator and grows only when a larger payload arrives.  No kernel here waits on another
// GPU: the only cross-GPU synchronisation is NCCL's.
#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "reduce_ops.cuh"

namespace dpb {

int64_t tuning_peer_polls();   // probes per wait of the peer exchange ("peer_polls" switch)

namespace {

// ---- the handful of NCCL entry points used, declared here (public API of libnccl.so.2)
struct NcclUniqueId {
    char internal[128];
};
typedef void *NcclComm;
enum { kNcclInt8 = 0 };
typedef int (*nccl_get_unique_id_t)(NcclUniqueId *);
typedef int (*nccl_comm_init_rank_t)(NcclComm *, int, NcclUniqueId, int);
typedef int (*nccl_comm_destroy_t)(NcclComm);
typedef int (*nccl_all_gather_t)(const void *, void *, size_t, int, NcclComm, cudaStream_t);
typedef const char *(*nccl_get_error_string_t)(int);
typedef int (*nccl_get_version_t)(int *);

struct NcclApi {
    void *handle = nullptr;
    nccl_get_unique_id_t get_unique_id = nullptr;
    nccl_comm_init_rank_t comm_init_rank = nullptr;
    nccl_comm_destroy_t comm_destroy = nullptr;
    nccl_all_gather_t all_gather = nullptr;
    nccl_get_error_string_t get_error_string = nullptr;
    nccl_get_version_t get_version = nullptr;
};
NcclApi g_nccl;
std::mutex g_nccl_mutex;

int load_nccl(const char *path)
{
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (g_nccl.handle) return DPB_OK;
    const char *names[] = {path, "libnccl.so.2", "libnccl.so"};
    void *h = nullptr;
    for (const char *n : names) {
        if (!n || !*n) continue;
        h = dlopen(n, RTLD_NOW | RTLD_LOCAL);
        if (h) break;
    }
    if (!h) return set_error(DPB_ERR_RUNTIME, "NCCL could not be loaded (%s): %s", path ? path : "libnccl.so.2", dlerror());
    NcclApi api;
    api.handle = h;
    api.get_unique_id = reinterpret_cast<nccl_get_unique_id_t>(dlsym(h, "ncclGetUniqueId"));
    api.comm_init_rank = reinterpret_cast<nccl_comm_init_rank_t>(dlsym(h, "ncclCommInitRank"));
    api.comm_destroy = reinterpret_cast<nccl_comm_destroy_t>(dlsym(h, "ncclCommDestroy"));
    api.all_gather = reinterpret_cast<nccl_all_gather_t>(dlsym(h, "ncclAllGather"));
    api.get_error_string = reinterpret_cast<nccl_get_error_string_t>(dlsym(h, "ncclGetErrorString"));
    api.get_version = reinterpret_cast<nccl_get_version_t>(dlsym(h, "ncclGetVersion"));
    if (!api.get_unique_id || !api.comm_init_rank || !api.comm_destroy || !api.all_gather || !api.get_error_string) {
        dlclose(h);
        return set_error(DPB_ERR_RUNTIME, "the NCCL library lacks an expected entry point");
    }
    g_nccl = api;
    return DPB_OK;
}

#define DPB_NCCL_TRY(expr)                                                                         \
    do {                                                                                           \
        int rc__ = (expr);                                                                         \
        if (rc__ != 0)                                                                             \
            return set_error(DPB_ERR_RUNTIME, "%s failed: %s", #expr, g_nccl.get_error_string(rc__)); \
    } while (0)

constexpr int kMaxPeers = 16;                 // ranks whose mailboxes one process maps
constexpr size_t kPeerSlotBytes = size_t(256) << 10;   // payload per rank that travels through the mailboxes
constexpr size_t kPeerFlagStride = 32;        // one flag per 32-byte sector
constexpr uint32_t kCommMagic = 0x44504243u;  // "DPBC"
constexpr int kPairBytes = 32;                // one (value, index) record: 16 value bytes, index, padding

struct Comm {
    uint32_t magic = kCommMagic;
    int rank = 0;
    int world = 1;
    int device = 0;
    NcclComm nccl = nullptr;  // null for a one-rank communicator: nothing to exchange
    void *gather = nullptr;   // world x capacity bytes
    size_t capacity = 0;      // bytes per rank
    void *pair = nullptr;     // this rank's packed (value, index) record
    // peer mailboxes (see the "peer exchange" section below)
    bool peer_on = false;
    void *box = nullptr;                  // this rank's mailbox (cudaMalloc: exported through IPC)
    void *peer_box[kMaxPeers] = {};       // every rank's mailbox as mapped into this process
    unsigned *peer_counter = nullptr;     // block counter of the exchange kernel
    unsigned *peer_error_host = nullptr;  // pinned, mapped: set by a kernel whose wait ran out
    unsigned *peer_error_dev = nullptr;   // the same word seen from the device
    unsigned epoch = 0;                   // exchanges done so far
};

Comm *as_comm(void *c)
{
    Comm *p = static_cast<Comm *>(c);
    return (p && p->magic == kCommMagic) ? p : nullptr;
}

// Room for `nbytes` per rank in the gather buffer.  Growing frees the old buffer in stream order
// (work already queued on `stream` keeps using it) and allocates the new one on the same stream.
int reserve(Comm *c, size_t nbytes, cudaStream_t stream)
{
    if (nbytes <= c->capacity) return DPB_OK;
    size_t cap = c->capacity ? c->capacity : (size_t(1) << 20);
    while (cap < nbytes) cap *= 2;
    void *p = nullptr;
    DPB_TRY(dpb_malloc(cap * static_cast<size_t>(c->world), stream, &p));
    if (c->gather) DPB_TRY(dpb_free(c->gather, stream));
    c->gather = p;
    c->capacity = cap;
    return DPB_OK;
}

// All-gather of `nbytes` per rank from `send` into the gather buffer (rank r at r * nbytes).
int gather_bytes(Comm *c, const void *send, size_t nbytes, cudaStream_t stream)
{
    DPB_TRY(reserve(c, nbytes, stream));
    if (c->world == 1 || !c->nccl) {
        DPB_CUDA_TRY(cudaMemcpyAsync(c->gather, send, nbytes, cudaMemcpyDeviceToDevice, stream));
        return DPB_OK;
    }
    DPB_NCCL_TRY(g_nccl.all_gather(send, c->gather, nbytes, kNcclInt8, c->nccl, stream));
    return DPB_OK;
}

// ---------------------------------------------------------------- kernels
// out[i] = fold over ranks r = 0..world-1, in that order, of gathered[r][i]
template <class R> __global__ void combine_rows_kernel(const typename R::In *gathered, typename R::Out *out, int64_t count, int world)
{
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    typename R::Acc acc = R::load(gathered[i], 0);
    for (int r = 1; r < world; ++r) acc = R::combine(acc, R::load(gathered[int64_t(r) * count + i], 0));
    out[i] = R::finish(acc);
}

struct PairRecord {
    unsigned char value[16];
    int64_t index;   // global flat index; negative: this rank holds no element
    int64_t pad;
};
static_assert(sizeof(PairRecord) == kPairBytes, "record layout");

template <class T> __global__ void pack_pair_kernel(const T *src, int64_t nelems, const int64_t *local_index,
                                                    int64_t index_offset, PairRecord *rec)
{
    PairRecord r;
    for (int k = 0; k < 16; ++k) r.value[k] = 0;
    r.pad = 0;
    r.index = -1;
    if (nelems > 0 && local_index) {
        const int64_t li = *local_index;
        if (li >= 0 && li < nelems) {
            const T v = src[li];
            memcpy(r.value, &v, sizeof(T));
            r.index = li + index_offset;
        }
    }
    *rec = r;
}

template <class V> __device__ bool value_has_nan(const V &v)
{
    if constexpr (is_cplx_v<V>) return v.re != v.re || v.im != v.im;
    else if constexpr (std::is_floating_point_v<V>) return v != v;
    else return false;
}

// strictly better, NaN aside: complex numbers compare by real part, then imaginary part
template <bool IS_MAX, class V> __device__ bool value_better(const V &a, const V &b)
{
    if constexpr (is_cplx_v<V>) {
        if (a.re == b.re) return IS_MAX ? a.im > b.im : a.im < b.im;
        return IS_MAX ? a.re > b.re : a.re < b.re;
    }
    else return IS_MAX ? a > b : a < b;
}

template <class V> __device__ bool value_equal(const V &a, const V &b)
{
    if constexpr (is_cplx_v<V>) return a.re == b.re && a.im == b.im;
    else return a == b;
}

// One thread walks the ranks' records: the first-occurrence rule across shards.
template <bool IS_MAX, class T> __global__ void pick_pair_kernel(const PairRecord *recs, int world, T *out_value, int64_t *out_index)
{
    using V = typename search_val<T>::type;
    bool have = false;
    T best_raw{};
    V best{};
    int64_t best_idx = -1;
    for (int r = 0; r < world; ++r) {
        const PairRecord rec = recs[r];
        if (rec.index < 0) continue;
        T raw;
        memcpy(&raw, rec.value, sizeof(T));
        V v;
        if constexpr (is_bool_v<T>) v = raw.v ? 1 : 0;
        else v = convert<V>(raw);
        bool wins;
        if (!have) wins = true;
        else {
            const bool vn = value_has_nan(v), bn = value_has_nan(best);
            if (vn || bn) wins = vn && (!bn || rec.index < best_idx);
            else if (value_equal(v, best)) wins = rec.index < best_idx;
            else wins = value_better<IS_MAX>(v, best);
        }
        if (wins) {
            have = true;
            best = v;
            best_raw = raw;
            best_idx = rec.index;
        }
    }
    if (out_value) *out_value = best_raw;
    if (out_index) *out_index = best_idx;
}

// ---------------------------------------------------------------- peer exchange
// The payloads of the combines are small (a row of partial sums, one (value, index) record), so
// their cost is latency.  Where every rank's GPU can map the others' memory (one box, NVLink), the
// exchange and the fold are ONE kernel per rank and no library call:
//   1. every block copies its share of this rank's payload into slot [set][rank] of EVERY rank's
//      mailbox (plain stores to peer memory), fences, and counts itself done; the last block to
//      finish writes the call's number into flag [set][rank] of every mailbox (release, system
//      scope);
//   2. every block waits until the flags of all ranks in its OWN mailbox carry the call's number
//      -- a bounded wait: `max_polls` probes, after which the kernel raises the communicator's
//      error word (in pinned host memory, so the host sees it without a copy) and returns;
//   3. every block folds its share of the slots in rank order (loads past L1) into the result.
// Two slot sets alternate with the call number: a rank can only be one call ahead of the slowest
// (it needs everyone's flag of call k+1 before it can start call k+2), so the set it overwrites
// is no longer being read.  The grid never exceeds one block per SM, so every block is resident
// and none waits for a block that has not started.  A mailbox is 2 sets x world slots of 256 KiB
// plus the flags; larger payloads go through NCCL.
struct PeerArgs {
    void *box[kMaxPeers];
    int rank, world, set;
    unsigned epoch;
    unsigned *counter;
    unsigned *error;
    int max_polls;
};

DPB_D char *peer_slot(const PeerArgs &a, int owner, int src)
{
    return static_cast<char *>(a.box[owner]) + (size_t(a.set) * a.world + src) * kPeerSlotBytes;
}
DPB_D unsigned *peer_flag(const PeerArgs &a, int owner, int src)
{
    return reinterpret_cast<unsigned *>(static_cast<char *>(a.box[owner]) + 2 * size_t(a.world) * kPeerSlotBytes +
                                        (size_t(a.set) * a.world + src) * kPeerFlagStride);
}
inline size_t peer_box_bytes(int world) { return 2 * size_t(world) * (kPeerSlotBytes + kPeerFlagStride); }

// Steps 1 and 2 for `nbytes` at `send`; called by all threads of all blocks.  false: the wait ran out.
DPB_D bool peer_exchange(const PeerArgs &a, const void *send, size_t nbytes)
{
    __shared__ int s_last, s_fail;
    const size_t gtid = size_t(blockIdx.x) * blockDim.x + threadIdx.x, gsize = size_t(gridDim.x) * blockDim.x;
    if (((reinterpret_cast<uintptr_t>(send) | nbytes) & 15) == 0) {
        const uint4 *src = static_cast<const uint4 *>(send);
        for (size_t i = gtid; i < nbytes / 16; i += gsize) {
            const uint4 v = src[i];
            for (int r = 0; r < a.world; ++r) reinterpret_cast<uint4 *>(peer_slot(a, r, a.rank))[i] = v;
        }
    }
    else {
        const unsigned char *src = static_cast<const unsigned char *>(send);
        for (size_t i = gtid; i < nbytes; i += gsize) {
            const unsigned char v = src[i];
            for (int r = 0; r < a.world; ++r) reinterpret_cast<unsigned char *>(peer_slot(a, r, a.rank))[i] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        s_fail = 0;
        s_last = atomicAdd(a.counter, 1u) == gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        if (threadIdx.x < a.world)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flag(a, threadIdx.x, a.rank)), "r"(a.epoch) : "memory");
        if (threadIdx.x == 0) *a.counter = 0;     // for the next call (this kernel is long done by then)
    }
    if (threadIdx.x < a.world) {
        const unsigned *f = peer_flag(a, a.rank, threadIdx.x);
        int polls = 0;
        while (true) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (v == a.epoch) break;
            if (polls >= a.max_polls) {
                s_fail = 1;
                break;
            }
            ++polls;
            if (polls > 64) __nanosleep(200);
        }
    }
    __syncthreads();
    if (s_fail) {
        if (threadIdx.x == 0) {
            *reinterpret_cast<volatile unsigned *>(a.error) = 1u;
            __threadfence_system();
        }
        return false;
    }
    return true;
}

template <class T> DPB_D T peer_load(const T *p)
{
    // past L1: the slot was written by another GPU
    if constexpr (sizeof(T) == 16) {
        const uint4 w = __ldcg(reinterpret_cast<const uint4 *>(p));
        T v;
        memcpy(&v, &w, 16);
        return v;
    }
    else if constexpr (sizeof(T) == 8) {
        const unsigned long long w = __ldcg(reinterpret_cast<const unsigned long long *>(p));
        T v;
        memcpy(&v, &w, 8);
        return v;
    }
    else if constexpr (sizeof(T) == 4) {
        const unsigned w = __ldcg(reinterpret_cast<const unsigned *>(p));
        T v;
        memcpy(&v, &w, 4);
        return v;
    }
    else if constexpr (sizeof(T) == 2) {
        const unsigned short w = __ldcg(reinterpret_cast<const unsigned short *>(p));
        T v;
        memcpy(&v, &w, 2);
        return v;
    }
    else {
        const unsigned char w = __ldcg(reinterpret_cast<const unsigned char *>(p));
        T v;
        memcpy(&v, &w, 1);
        return v;
    }
}

// exchange + fold of `count` partial results per rank, in rank order
template <class R>
__global__ void __launch_bounds__(256)
    peer_combine_kernel(PeerArgs a, const typename R::In *partial, typename R::Out *out, int64_t count)
{
    using In = typename R::In;
    if (!peer_exchange(a, partial, size_t(count) * sizeof(In))) return;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += int64_t(gridDim.x) * blockDim.x) {
        typename R::Acc acc = R::load(peer_load(reinterpret_cast<const In *>(peer_slot(a, a.rank, 0)) + i), 0);
        for (int r = 1; r < a.world; ++r)
            acc = R::combine(acc, R::load(peer_load(reinterpret_cast<const In *>(peer_slot(a, a.rank, r)) + i), 0));
        out[i] = R::finish(acc);
    }
}

// exchange of the ranks' (value, index) records; the records land in `recs` for pick_pair_kernel's rule
__global__ void __launch_bounds__(256) peer_records_kernel(PeerArgs a, const PairRecord *mine, PairRecord *recs)
{
    if (!peer_exchange(a, mine, sizeof(PairRecord))) return;
    if (threadIdx.x < a.world) {
        const uint4 *src = reinterpret_cast<const uint4 *>(peer_slot(a, a.rank, threadIdx.x));
        uint4 *dst = reinterpret_cast<uint4 *>(recs + threadIdx.x);
        dst[0] = __ldcg(src);
        dst[1] = __ldcg(src + 1);
    }
}

// a wait that nothing satisfies: the bounded wait's give-up path, for tests
__global__ void peer_probe_wait_kernel(PeerArgs a, unsigned *timed_out)
{
    const unsigned *f = peer_flag(a, a.rank, 0);
    int polls = 0;
    unsigned result = 0;
    while (true) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if (v == 0xffffffffu) break;              // never written: call numbers start at 1 and count up
        if (polls >= a.max_polls) {
            result = 1;
            break;
        }
        ++polls;
        if (polls > 64) __nanosleep(200);
    }
    *reinterpret_cast<volatile unsigned *>(timed_out) = result;
    __threadfence_system();
}

// Arguments of the next exchange; DPB_ERR_RUNTIME if an earlier one gave up.
int peer_next(Comm *c, PeerArgs &a)
{
    if (*reinterpret_cast<volatile unsigned *>(c->peer_error_host) != 0)
        return set_error(DPB_ERR_RUNTIME, "a rank did not deliver its part of an earlier exchange within the time limit; "
                                          "the communicator is unusable");
    ++c->epoch;
    for (int r = 0; r < kMaxPeers; ++r) a.box[r] = r < c->world ? c->peer_box[r] : nullptr;
    a.rank = c->rank;
    a.world = c->world;
    a.set = static_cast<int>(c->epoch & 1u);
    a.epoch = c->epoch;
    a.counter = c->peer_counter;
    a.error = c->peer_error_dev;
    a.max_polls = static_cast<int>(tuning_peer_polls());
    return DPB_OK;
}

inline bool peer_fits(const Comm *c, size_t nbytes) { return c->peer_on && c->world > 1 && nbytes <= kPeerSlotBytes; }

inline int peer_grid(size_t nbytes)
{
    const int64_t want = ceil_div(static_cast<int64_t>(nbytes), 256 * 16);
    return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, device_props().sm_count)));
}

// exchange and fold in one kernel over the peer mailboxes
template <class R> int launch_peer_combine(Comm *c, const void *partial, void *out, int64_t count, cudaStream_t s, const char *name)
{
    PeerArgs a;
    DPB_TRY(peer_next(c, a));
    peer_combine_kernel<R><<<peer_grid(size_t(count) * sizeof(typename R::In)), 256, 0, s>>>(
        a, static_cast<const typename R::In *>(partial), static_cast<typename R::Out *>(out), count);
    note_kernel(name);
    return check_launch(name);
}

template <class R> int launch_combine(Comm *c, void *out, int64_t count, cudaStream_t s, const char *name)
{
    const int threads = 256;
    const int64_t blocks = (count + threads - 1) / threads;
    if (blocks > 0x7fffffff) return set_error(DPB_ERR_VALUE, "%s: too many elements for one launch", name);
    combine_rows_kernel<R><<<static_cast<int>(blocks), threads, 0, s>>>(
        static_cast<const typename R::In *>(c->gather), static_cast<typename R::Out *>(out), count, c->world);
    note_kernel(name);
    return check_launch(name);
}

}  // namespace
}  // namespace dpb

using namespace dpb;

extern "C" {

int dpb_comm_load(const char *libnccl_path) { return load_nccl(libnccl_path); }

int dpb_comm_nccl_version(int *version)
{
    if (!g_nccl.handle) DPB_TRY(load_nccl(nullptr));
    if (!version || !g_nccl.get_version) return set_error(DPB_ERR_VALUE, "NCCL version is not available");
    DPB_NCCL_TRY(g_nccl.get_version(version));
    return DPB_OK;
}

int dpb_comm_unique_id(void *id128)
{
    if (!id128) return set_error(DPB_ERR_VALUE, "dpb_comm_unique_id: null buffer");
    if (!g_nccl.handle) DPB_TRY(load_nccl(nullptr));
    NcclUniqueId id;
    DPB_NCCL_TRY(g_nccl.get_unique_id(&id));
    std::memcpy(id128, id.internal, sizeof(id.internal));
    return DPB_OK;
}

int dpb_comm_init(int rank, int world, const void *id128, void **comm)
{
    if (!comm) return set_error(DPB_ERR_VALUE, "dpb_comm_init: null result pointer");
    *comm = nullptr;
    if (world < 1 || rank < 0 || rank >= world)
        return set_error(DPB_ERR_VALUE, "dpb_comm_init: rank %d is not in a group of %d", rank, world);
    Comm *c = new Comm();
    c->rank = rank;
    c->world = world;
    if (cudaGetDevice(&c->device) != cudaSuccess) {
        cudaGetLastError();
        delete c;
        return set_error(DPB_ERR_CUDA, "dpb_comm_init: no CUDA device is current");
    }
    if (world > 1) {
        if (!id128) {
            delete c;
            return set_error(DPB_ERR_VALUE, "dpb_comm_init: a group of %d ranks needs the unique id of rank 0", world);
        }
        int st = g_nccl.handle ? DPB_OK : load_nccl(nullptr);
        if (st != DPB_OK) {
            delete c;
            return st;
        }
        NcclUniqueId id;
        std::memcpy(id.internal, id128, sizeof(id.internal));
        const int rc = g_nccl.comm_init_rank(&c->nccl, world, id, rank);
        if (rc != 0) {
            delete c;
            return set_error(DPB_ERR_RUNTIME, "ncclCommInitRank failed: %s", g_nccl.get_error_string(rc));
        }
    }
    void *p = nullptr;
    const int st = dpb_malloc(kPairBytes, nullptr, &p);
    if (st != DPB_OK) {
        if (c->nccl) g_nccl.comm_destroy(c->nccl);
        delete c;
        return st;
    }
    cudaStreamSynchronize(nullptr);  // the record buffer is used on other streams from now on
    c->pair = p;
    *comm = c;
    return DPB_OK;
}

int dpb_comm_destroy(void *comm)
{
    Comm *c = as_comm(comm);
    if (!c) return set_error(DPB_ERR_VALUE, "not a communicator");
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    if (c->gather) dpb_free(c->gather, nullptr);
    if (c->pair) dpb_free(c->pair, nullptr);
    for (int r = 0; r < c->world && r < kMaxPeers; ++r)
        if (c->peer_box[r] && r != c->rank) cudaIpcCloseMemHandle(c->peer_box[r]);
    if (c->box) cudaFree(c->box);
    if (c->peer_counter) cudaFree(c->peer_counter);
    if (c->peer_error_host) cudaFreeHost(c->peer_error_host);
    cudaGetLastError();
    if (c->nccl) g_nccl.comm_destroy(c->nccl);
    c->magic = 0;
    delete c;
    return DPB_OK;
}

int dpb_comm_info(void *comm, int *rank, int *world)
{
    Comm *c = as_comm(comm);
    if (!c) return set_error(DPB_ERR_VALUE, "not a communicator");
    if (rank) *rank = c->rank;
    if (world) *world = c->world;
    return DPB_OK;
}

int dpb_comm_peer_export(void *comm, void *handle, int64_t handle_capacity, int64_t *handle_bytes)
{
    Comm *c = as_comm(comm);
    if (!c) return set_error(DPB_ERR_VALUE, "not a communicator");
    if (handle_bytes) *handle_bytes = static_cast<int64_t>(sizeof(cudaIpcMemHandle_t));
    if (!handle || handle_capacity < static_cast<int64_t>(sizeof(cudaIpcMemHandle_t)))
        return set_error(DPB_ERR_VALUE, "dpb_comm_peer_export: the handle needs %d bytes", int(sizeof(cudaIpcMemHandle_t)));
    if (c->world > kMaxPeers) return set_error(DPB_ERR_RUNTIME, "peer mailboxes serve at most %d ranks", kMaxPeers);
    DPB_CUDA_TRY(cudaSetDevice(c->device));
    if (!c->box) {
        // plain cudaMalloc: memory of the stream-ordered pool cannot be exported
        DPB_CUDA_TRY(cudaMalloc(&c->box, peer_box_bytes(c->world)));
        DPB_CUDA_TRY(cudaMemset(c->box, 0, peer_box_bytes(c->world)));
        DPB_CUDA_TRY(cudaMalloc(reinterpret_cast<void **>(&c->peer_counter), sizeof(unsigned)));
        DPB_CUDA_TRY(cudaMemset(c->peer_counter, 0, sizeof(unsigned)));
        DPB_CUDA_TRY(cudaHostAlloc(reinterpret_cast<void **>(&c->peer_error_host), sizeof(unsigned), cudaHostAllocMapped));
        *c->peer_error_host = 0;
        DPB_CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void **>(&c->peer_error_dev), c->peer_error_host, 0));
        DPB_CUDA_TRY(cudaDeviceSynchronize());
    }
    cudaIpcMemHandle_t h;
    DPB_CUDA_TRY(cudaIpcGetMemHandle(&h, c->box));
    std::memcpy(handle, &h, sizeof h);
    return DPB_OK;
}

int dpb_comm_peer_attach(void *comm, const void *handles, int count)
{
    Comm *c = as_comm(comm);
    if (!c) return set_error(DPB_ERR_VALUE, "not a communicator");
    if (!c->box) return set_error(DPB_ERR_VALUE, "dpb_comm_peer_attach: call dpb_comm_peer_export first");
    if (!handles || count != c->world) return set_error(DPB_ERR_VALUE, "dpb_comm_peer_attach: one handle per rank is needed");
    DPB_CUDA_TRY(cudaSetDevice(c->device));
    const cudaIpcMemHandle_t *h = static_cast<const cudaIpcMemHandle_t *>(handles);
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) {
            c->peer_box[r] = c->box;
            continue;
        }
        if (c->peer_box[r]) continue;
        cudaIpcMemHandle_t hr;
        std::memcpy(&hr, h + r, sizeof hr);
        DPB_CUDA_TRY(cudaIpcOpenMemHandle(&c->peer_box[r], hr, cudaIpcMemLazyEnablePeerAccess));
    }
    return DPB_OK;
}

int dpb_comm_peer_enable(void *comm, int on)
{
    Comm *c = as_comm(comm);
    if (!c) return set_error(DPB_ERR_VALUE, "not a communicator");
    if (on) {
        for (int r = 0; r < c->world; ++r)
            if (!c->peer_box[r]) return set_error(DPB_ERR_VALUE, "dpb_comm_peer_enable: rank %d's mailbox is not attached", r);
    }
    c->peer_on = on != 0;
    return DPB_OK;
}

int dpb_comm_peer_probe_wait(void *comm, int64_t polls, int *timed_out, void *stream)
{
    Comm *c = as_comm(comm);
    if (!c) return set_error(DPB_ERR_VALUE, "not a communicator");
    if (!c->box || !timed_out || polls < 0 || polls > (int64_t(1) << 24))
        return set_error(DPB_ERR_VALUE, "dpb_comm_peer_probe_wait: bad arguments (export the mailbox first; at most 2^24 probes)");
    PeerArgs a;
    for (int r = 0; r < kMaxPeers; ++r) a.box[r] = nullptr;
    a.box[c->rank] = c->box;
    a.rank = c->rank;
    a.world = c->world;
    a.set = 0;
    a.epoch = 0;
    a.counter = c->peer_counter;
    a.error = c->peer_error_dev;
    a.max_polls = static_cast<int>(polls);
    unsigned *word = nullptr, *word_dev = nullptr;
    DPB_CUDA_TRY(cudaHostAlloc(reinterpret_cast<void **>(&word), sizeof(unsigned), cudaHostAllocMapped));
    *word = 2;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int st = DPB_OK;
    if (cudaHostGetDevicePointer(reinterpret_cast<void **>(&word_dev), word, 0) != cudaSuccess) st = DPB_ERR_CUDA;
    if (st == DPB_OK) {
        peer_probe_wait_kernel<<<1, 1, 0, s>>>(a, word_dev);
        note_kernel("comm_peer_probe_wait");
        st = check_launch("comm_peer_probe_wait");
    }
    if (st == DPB_OK && cudaStreamSynchronize(s) != cudaSuccess) st = set_error(DPB_ERR_CUDA, "dpb_comm_peer_probe_wait: the wait kernel failed");
    *timed_out = static_cast<int>(*word);
    cudaFreeHost(word);
    return st;
}

int dpb_comm_allgather(void *comm, const void *send, void *recv, int64_t nbytes, void *stream)
{
    Comm *c = as_comm(comm);
    if (!c) return set_error(DPB_ERR_VALUE, "not a communicator");
    if (nbytes < 0 || (nbytes > 0 && (!send || !recv))) return set_error(DPB_ERR_VALUE, "dpb_comm_allgather: bad arguments");
    if (nbytes == 0) return DPB_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (c->world == 1 || !c->nccl) {
        if (send != recv) DPB_CUDA_TRY(cudaMemcpyAsync(recv, send, nbytes, cudaMemcpyDeviceToDevice, s));
        return DPB_OK;
    }
    DPB_NCCL_TRY(g_nccl.all_gather(send, recv, static_cast<size_t>(nbytes), kNcclInt8, c->nccl, s));
    return DPB_OK;
}

int dpb_comm_sum_ordered(void *comm, int typenum, const void *partial, void *out, int64_t count, void *stream)
{
    Comm *c = as_comm(comm);
    if (!c) return set_error(DPB_ERR_VALUE, "not a communicator");
    if (count < 0 || (count > 0 && (!partial || !out))) return set_error(DPB_ERR_VALUE, "dpb_comm_sum_ordered: bad arguments");
    if (count == 0) return DPB_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t nbytes = static_cast<size_t>(count) * type_size(typenum);
    if (type_size(typenum) == 0) return set_error(DPB_ERR_TYPE, "dpb_comm_sum_ordered: unknown type %d", typenum);
    const bool peer = peer_fits(c, nbytes);
    if (!peer) DPB_TRY(gather_bytes(c, partial, nbytes, s));
    switch (typenum) {
#define DPB_CASE(TN, T)                                                                               \
    case TN:                                                                                          \
        return peer ? launch_peer_combine<SumRed<T, T>>(c, partial, out, count, s, "comm_peer_sum_ordered") \
                    : launch_combine<SumRed<T, T>>(c, out, count, s, "comm_sum_ordered");
        DPB_CASE(DPB_BOOL, bool_t)
        DPB_CASE(DPB_INT8, int8_t)
        DPB_CASE(DPB_UINT8, uint8_t)
        DPB_CASE(DPB_INT16, int16_t)
        DPB_CASE(DPB_UINT16, uint16_t)
        DPB_CASE(DPB_INT32, int32_t)
        DPB_CASE(DPB_UINT32, uint32_t)
        DPB_CASE(DPB_INT64, int64_t)
        DPB_CASE(DPB_UINT64, uint64_t)
        DPB_CASE(DPB_HALF, half_t)
        DPB_CASE(DPB_FLOAT, float)
        DPB_CASE(DPB_DOUBLE, double)
        DPB_CASE(DPB_CFLOAT, cfloat)
        DPB_CASE(DPB_CDOUBLE, cdouble)
#undef DPB_CASE
    default: return set_error(DPB_ERR_TYPE, "dpb_comm_sum_ordered: unknown type %d", typenum);
    }
}

int dpb_comm_extreme(void *comm, int typenum, int is_max, const void *partial, void *out, int64_t count, void *stream)
{
    Comm *c = as_comm(comm);
    if (!c) return set_error(DPB_ERR_VALUE, "not a communicator");
    if (count < 0 || (count > 0 && (!partial || !out))) return set_error(DPB_ERR_VALUE, "dpb_comm_extreme: bad arguments");
    if (count == 0) return DPB_OK;
    if (type_size(typenum) == 0) return set_error(DPB_ERR_TYPE, "dpb_comm_extreme: unknown type %d", typenum);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool peer = peer_fits(c, static_cast<size_t>(count) * type_size(typenum));
    if (!peer) DPB_TRY(gather_bytes(c, partial, static_cast<size_t>(count) * type_size(typenum), s));
    switch (typenum) {
#define DPB_CASE(TN, T)                                                                                 \
    case TN:                                                                                            \
        if (peer)                                                                                       \
            return is_max ? launch_peer_combine<ExtremeRed<true, T, T>>(c, partial, out, count, s, "comm_peer_extreme")  \
                          : launch_peer_combine<ExtremeRed<false, T, T>>(c, partial, out, count, s, "comm_peer_extreme"); \
        return is_max ? launch_combine<ExtremeRed<true, T, T>>(c, out, count, s, "comm_extreme")        \
                      : launch_combine<ExtremeRed<false, T, T>>(c, out, count, s, "comm_extreme");
        DPB_CASE(DPB_BOOL, bool_t)
        DPB_CASE(DPB_INT8, int8_t)
        DPB_CASE(DPB_UINT8, uint8_t)
        DPB_CASE(DPB_INT16, int16_t)
        DPB_CASE(DPB_UINT16, uint16_t)
        DPB_CASE(DPB_INT32, int32_t)
        DPB_CASE(DPB_UINT32, uint32_t)
        DPB_CASE(DPB_INT64, int64_t)
        DPB_CASE(DPB_UINT64, uint64_t)
        DPB_CASE(DPB_HALF, half_t)
        DPB_CASE(DPB_FLOAT, float)
        DPB_CASE(DPB_DOUBLE, double)
        DPB_CASE(DPB_CFLOAT, cfloat)
        DPB_CASE(DPB_CDOUBLE, cdouble)
#undef DPB_CASE
    default: return set_error(DPB_ERR_TYPE, "dpb_comm_extreme: unknown type %d", typenum);
    }
}

int dpb_comm_arg_extreme(void *comm, int typenum, int is_max, const void *src, int64_t nelems,
                         const void *local_index, int64_t index_offset, void *out_value, void *out_index,
                         void *stream)
{
    Comm *c = as_comm(comm);
    if (!c) return set_error(DPB_ERR_VALUE, "not a communicator");
    if (nelems < 0 || (nelems > 0 && (!src || !local_index)))
        return set_error(DPB_ERR_VALUE, "dpb_comm_arg_extreme: bad arguments");
    if (type_size(typenum) == 0) return set_error(DPB_ERR_TYPE, "dpb_comm_arg_extreme: unknown type %d", typenum);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PairRecord *mine = static_cast<PairRecord *>(c->pair);
    const int64_t *li = static_cast<const int64_t *>(local_index);
#define DPB_CASE(TN, T)                                                                                          \
    case TN:                                                                                                     \
        pack_pair_kernel<T><<<1, 1, 0, s>>>(static_cast<const T *>(src), nelems, li, index_offset, mine);        \
        break;
    switch (typenum) {
        DPB_CASE(DPB_BOOL, bool_t)
        DPB_CASE(DPB_INT8, int8_t)
        DPB_CASE(DPB_UINT8, uint8_t)
        DPB_CASE(DPB_INT16, int16_t)
        DPB_CASE(DPB_UINT16, uint16_t)
        DPB_CASE(DPB_INT32, int32_t)
        DPB_CASE(DPB_UINT32, uint32_t)
        DPB_CASE(DPB_INT64, int64_t)
        DPB_CASE(DPB_UINT64, uint64_t)
        DPB_CASE(DPB_HALF, half_t)
        DPB_CASE(DPB_FLOAT, float)
        DPB_CASE(DPB_DOUBLE, double)
        DPB_CASE(DPB_CFLOAT, cfloat)
        DPB_CASE(DPB_CDOUBLE, cdouble)
    default: return set_error(DPB_ERR_TYPE, "dpb_comm_arg_extreme: unknown type %d", typenum);
    }
#undef DPB_CASE
    note_kernel("comm_pack_pair");
    DPB_TRY(check_launch("comm_pack_pair"));
    if (peer_fits(c, kPairBytes)) {
        DPB_TRY(reserve(c, kPairBytes, s));
        PeerArgs a;
        DPB_TRY(peer_next(c, a));
        peer_records_kernel<<<1, 256, 0, s>>>(a, mine, static_cast<PairRecord *>(c->gather));
        note_kernel("comm_peer_records");
        DPB_TRY(check_launch("comm_peer_records"));
    }
    else DPB_TRY(gather_bytes(c, mine, kPairBytes, s));
    const PairRecord *recs = static_cast<const PairRecord *>(c->gather);
    int64_t *oi = static_cast<int64_t *>(out_index);
#define DPB_CASE(TN, T)                                                                                          \
    case TN:                                                                                                     \
        if (is_max) pick_pair_kernel<true, T><<<1, 1, 0, s>>>(recs, c->world, static_cast<T *>(out_value), oi);  \
        else pick_pair_kernel<false, T><<<1, 1, 0, s>>>(recs, c->world, static_cast<T *>(out_value), oi);        \
        break;
    switch (typenum) {
        DPB_CASE(DPB_BOOL, bool_t)
        DPB_CASE(DPB_INT8, int8_t)
        DPB_CASE(DPB_UINT8, uint8_t)
        DPB_CASE(DPB_INT16, int16_t)
        DPB_CASE(DPB_UINT16, uint16_t)
        DPB_CASE(DPB_INT32, int32_t)
        DPB_CASE(DPB_UINT32, uint32_t)
        DPB_CASE(DPB_INT64, int64_t)
        DPB_CASE(DPB_UINT64, uint64_t)
        DPB_CASE(DPB_HALF, half_t)
        DPB_CASE(DPB_FLOAT, float)
        DPB_CASE(DPB_DOUBLE, double)
        DPB_CASE(DPB_CFLOAT, cfloat)
        DPB_CASE(DPB_CDOUBLE, cdouble)
    default: break;
    }
#undef DPB_CASE
    note_kernel("comm_pick_pair");
    return check_launch("comm_pick_pair");
}

}  // extern "C"

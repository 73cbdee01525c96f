// Data-parallel communication of the C ABI: one communicator over the GPUs of one box.
//
// Two services:
//  1. ag_allreduce_sum: the gradient all-reduce as a plain NCCL call (any size).  NCCL is
//     looked up at run time (the copy already loaded into the process, e.g. by PyTorch, else
//     libnccl.so.2), so the library has no link-time dependency on it.
//  2. comm_fused_update (behind ag_model_allreduce_update): for buckets of up to
//     kCapWords 4-byte words, ONE kernel per GPU that all-reduces the gradient bucket over
//     NVLink and applies the SGD update.  Every GPU owns a "symmetric" block that the other
//     GPUs of the communicator can address: directly when one process drives all GPUs (peer
//     access), through CUDA IPC handles when there is one process per GPU.  The block holds,
//     per call parity and per sending rank, one 8-byte slot for every 4-byte word of the
//     bucket: {word, sequence number}.  A thread takes four words of the local gradients,
//     writes them with their sequence number into its own rank's slots on every peer (plain
//     16-byte stores of two 8-byte elements: each slot arrives whole, so the sequence number
//     is the word's own "valid" flag and no fence or separate flag write is needed), then polls
//     its local slots of every peer until they carry this call's sequence number (bounded),
//     adds the p contributions in rank order (so all ranks compute the same bits), scales,
//     and updates its four parameters.  Slots alternate between two parities, so a rank that
//     runs ahead never overwrites what a peer still has to read.  No multicast, no bulk / TMA
//     access to peer memory.
#include <dlfcn.h>

#include <chrono>
#include <cstring>
#include <thread>
#include <vector>

#include "comm.cuh"
#include "common.cuh"

namespace ag {
namespace {

// ---- NCCL, resolved at run time -------------------------------------------------
typedef void *nccl_comm_t;
struct nccl_unique_id {
    char internal[128];
};
enum { kNcclSuccess = 0, kNcclInProgress = 7 };
enum { kNcclInt8 = 0, kNcclUint8 = 1, kNcclFloat32 = 7, kNcclBfloat16 = 9 };
enum { kNcclSum = 0 };

struct Nccl {
    void *handle = nullptr;
    int (*GetUniqueId)(nccl_unique_id *) = nullptr;
    int (*CommInitRank)(nccl_comm_t *, int, nccl_unique_id, int) = nullptr;
    int (*CommInitAll)(nccl_comm_t *, int, const int *) = nullptr;
    int (*CommDestroy)(nccl_comm_t) = nullptr;
    int (*CommAbort)(nccl_comm_t) = nullptr;
    int (*CommGetAsyncError)(nccl_comm_t, int *) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, nccl_comm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool ok = false;
};

Nccl &nccl() {
    static Nccl n;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char *name : names) {  // the copy the process already has, if any
            n.handle = dlopen(name, RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
            if (n.handle) break;
        }
        for (int i = 0; !n.handle && i < 2; ++i) n.handle = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
        if (!n.handle) return;
        bool all = true;
        auto sym = [&](const char *name) {
            void *p = dlsym(n.handle, name);
            if (!p) all = false;
            return p;
        };
        n.GetUniqueId = (decltype(n.GetUniqueId))sym("ncclGetUniqueId");
        n.CommInitRank = (decltype(n.CommInitRank))sym("ncclCommInitRank");
        n.CommInitAll = (decltype(n.CommInitAll))sym("ncclCommInitAll");
        n.CommDestroy = (decltype(n.CommDestroy))sym("ncclCommDestroy");
        n.CommAbort = (decltype(n.CommAbort))sym("ncclCommAbort");
        n.CommGetAsyncError = (decltype(n.CommGetAsyncError))sym("ncclCommGetAsyncError");
        n.AllReduce = (decltype(n.AllReduce))sym("ncclAllReduce");
        n.AllGather = (decltype(n.AllGather))sym("ncclAllGather");
        n.GroupStart = (decltype(n.GroupStart))sym("ncclGroupStart");
        n.GroupEnd = (decltype(n.GroupEnd))sym("ncclGroupEnd");
        n.GetErrorString = (decltype(n.GetErrorString))sym("ncclGetErrorString");
        n.ok = all;
    });
    return n;
}

#define AG_NCCL_TRY(expr)                                                                   \
    do {                                                                                    \
        int _r = (expr);                                                                    \
        if (_r != kNcclSuccess && _r != kNcclInProgress)                                    \
            return ::ag::fail(AG_ERR_CUDA, "%s failed: %s", #expr, nccl().GetErrorString(_r)); \
    } while (0)

}  // namespace

constexpr int kMaxRanks = 16;
constexpr size_t kCapWords = size_t(128) << 10;  // 4-byte words of the largest fused bucket (512 KiB)
// symmetric block of one rank: [2 parities][world senders][kCapWords] slots of 8 bytes
inline size_t sym_bytes(int world) { return 2 * (size_t)world * kCapWords * 8; }

}  // namespace ag

// One member GPU of a communicator, as this process sees it.
struct ag_comm_member {
    ag_device *dev = nullptr;      // the rank's device object (ordinal + stream); not owned
    ag::nccl_comm_t nccl = nullptr;
    void *sym = nullptr;           // this rank's symmetric block (owned when local)
    void *peer_sym[ag::kMaxRanks] = {};  // every rank's block as addressable from this rank
    bool opened[ag::kMaxRanks] = {};     // peer_sym[q] came from cudaIpcOpenMemHandle
    uint32_t seq = 0;              // fused calls made so far on this rank
    int clock_khz = 0;             // SM clock, looked up once (the query is slow)
};

struct ag_comm {
    int world = 0;
    bool multi_process = false;
    int my_rank = -1;              // multi-process: the one local rank
    std::vector<ag_comm_member> members;  // single process: world entries; else one
    bool fused_ready = false;
    double timeout_s = 2.0;        // bounded wait of the fused kernel and of ag_comm_wait
    ag_comm_member *member(int rank) {
        if (multi_process) return rank == my_rank ? &members[0] : nullptr;
        return rank >= 0 && rank < world ? &members[(size_t)rank] : nullptr;
    }
};

namespace ag {
namespace {

int nccl_dtype(ag_dtype t, int *out) {
    switch (t) {
        case AG_F32: *out = kNcclFloat32; return AG_OK;
        case AG_BF16: *out = kNcclBfloat16; return AG_OK;
        case AG_U8: *out = kNcclUint8; return AG_OK;
        default: return fail(AG_ERR_DTYPE, "allreduce of dtype %d is not implemented", (int)t);
    }
}

int require_nccl() {
    AG_REQUIRE(nccl().ok, AG_ERR_UNSUPPORTED,
               "NCCL (libnccl.so.2) could not be loaded: %s", dlerror() ? dlerror() : "missing symbol");
    return AG_OK;
}

// Allocates and clears the rank's symmetric block (its device must be current).
int alloc_sym(ag_comm_member &m, int world) {
    AG_CUDA_TRY(cudaDeviceGetAttribute(&m.clock_khz, cudaDevAttrClockRate, m.dev->ordinal));
    AG_CUDA_TRY(cudaMalloc(&m.sym, sym_bytes(world)));
    // sequence numbers start at 1, so cleared slots never look valid
    AG_CUDA_TRY(cudaMemsetAsync(m.sym, 0, sym_bytes(world), m.dev->stream));
    AG_CUDA_TRY(cudaStreamSynchronize(m.dev->stream));
    return AG_OK;
}

// ---- the fused kernel ---------------------------------------------------------------
struct FusedParams {
    void *peer[kMaxRanks];  // every rank's symmetric block, in rank order
    int world, rank;
    uint32_t seq;
    int64_t words;          // 4-byte words of the bucket (a multiple of 4)
    float scale;            // applied to the summed gradient unless 1
    float lr, momentum;
    int use_momentum;
    long long timeout_cycles;
    int *status;            // device status word of this rank's ag_device
};

// Two slots {word, seq} as one 16-byte access of two 8-byte elements: each element is
// written / read whole.
__device__ __forceinline__ void st_slots(void *p, uint32_t w0, uint32_t w1, uint32_t seq) {
    const unsigned long long a = ((unsigned long long)seq << 32) | w0;
    const unsigned long long b = ((unsigned long long)seq << 32) | w1;
    asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1,%2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_slots(const void *p, unsigned long long &a, unsigned long long &b) {
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

template <class T>
struct Pack {  // 16 bytes of T
    static constexpr int N = 16 / sizeof(T);
    uint4 raw;
    __device__ __forceinline__ float get(int i) const {
        if constexpr (sizeof(T) == 4) return __uint_as_float((&raw.x)[i]);
        const uint32_t w = (&raw.x)[i >> 1];
        return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
    }
    __device__ __forceinline__ void set(int i, float v) {
        if constexpr (sizeof(T) == 4) {
            (&raw.x)[i] = __float_as_uint(v);
        } else {
            __nv_bfloat16 h = __float2bfloat16_rn(v);
            const uint32_t bits = *reinterpret_cast<unsigned short *>(&h);
            uint32_t &w = (&raw.x)[i >> 1];
            w = (i & 1) ? ((w & 0x0000ffffu) | (bits << 16)) : ((w & 0xffff0000u) | bits);
        }
    }
};

template <class T>
__device__ __forceinline__ float round_to(float v) {
    return to_f32(from_f32<T>(v));
}

// grads, values, velocity: this rank's flat buckets (16-byte aligned, padded to whole 16-byte
// packs).  One thread per pack of four words.
template <class T>
__global__ void __launch_bounds__(256)
    allreduce_update_kernel(T *__restrict__ grads, T *__restrict__ values, T *__restrict__ velocity,
                            const FusedParams p) {
    constexpr int V = Pack<T>::N;
    const int64_t pack = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pack * 4 >= p.words) return;
    const int parity = (int)(p.seq & 1u);
    Pack<T> mine;
    mine.raw = reinterpret_cast<const uint4 *>(grads)[pack];
    // 1. this pack, tagged with the call's sequence number, into my slots on every peer
    const size_t my_slot = (((size_t)parity * p.world + p.rank) * kCapWords + (size_t)pack * 4) * 8;
    for (int q = 0; q < p.world; ++q) {
        if (q == p.rank) continue;
        char *dst = reinterpret_cast<char *>(p.peer[q]) + my_slot;
        st_slots(dst, mine.raw.x, mine.raw.y, p.seq);
        st_slots(dst + 16, mine.raw.z, mine.raw.w, p.seq);
    }
    // 2. the peers' packs from my own block, in rank order; each slot is valid once it carries
    //    this call's sequence number
    float sum[V];
    const long long t0 = clock64();
    for (int q = 0; q < p.world; ++q) {
        Pack<T> part;
        if (q == p.rank) {
            part = mine;
        } else {
            const char *src = reinterpret_cast<const char *>(p.peer[p.rank]) +
                              (((size_t)parity * p.world + q) * kCapWords + (size_t)pack * 4) * 8;
            unsigned long long a, b, c, d;
            for (;;) {
                ld_slots(src, a, b);
                ld_slots(src + 16, c, d);
                if ((uint32_t)(a >> 32) == p.seq && (uint32_t)(b >> 32) == p.seq &&
                    (uint32_t)(c >> 32) == p.seq && (uint32_t)(d >> 32) == p.seq)
                    break;
                if (clock64() - t0 > p.timeout_cycles) {
                    atomicCAS(p.status, 0, 150 + q);  // 150 + the rank that never arrived
                    return;                           // this pack is not updated
                }
                __nanosleep(32);
            }
            part.raw = make_uint4((uint32_t)a, (uint32_t)b, (uint32_t)c, (uint32_t)d);
        }
        if (q == 0) {
#pragma unroll
            for (int j = 0; j < V; ++j) sum[j] = part.get(j);
        } else {
            // every partial sum is rounded to T, as a reduction over T-typed buffers does
#pragma unroll
            for (int j = 0; j < V; ++j) sum[j] = round_to<T>(__fadd_rn(sum[j], part.get(j)));
        }
    }
    // 3. scale, update
    const float scale_m1 = round_to<T>(p.scale - 1.f);
    const float neg_lr = round_to<T>(-p.lr);
    Pack<T> acc, w, v;
    w.raw = reinterpret_cast<const uint4 *>(values)[pack];
    if (p.use_momentum) v.raw = reinterpret_cast<const uint4 *>(velocity)[pack];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        float g = sum[j];
        // g = (scale - 1) * g + g in T arithmetic, as the separate scaling pass computes it
        if (p.scale != 1.f) g = round_to<T>(__fadd_rn(round_to<T>(__fmul_rn(scale_m1, g)), g));
        acc.set(j, g);
        if (p.use_momentum) {
            const float vv = __fadd_rn(__fmul_rn(p.momentum, v.get(j)), g);
            v.set(j, vv);
            w.set(j, __fsub_rn(w.get(j), __fmul_rn(p.lr, vv)));
        } else {
            // w = cast_T(-lr) * g + w in T arithmetic (plain SGD goes through scaled_add)
            w.set(j, __fadd_rn(round_to<T>(__fmul_rn(neg_lr, g)), w.get(j)));
        }
    }
    reinterpret_cast<uint4 *>(grads)[pack] = acc.raw;  // the reduced, scaled gradient
    reinterpret_cast<uint4 *>(values)[pack] = w.raw;
    if (p.use_momentum) reinterpret_cast<uint4 *>(velocity)[pack] = v.raw;
}

}  // namespace

int comm_fused_update(ag_comm *comm, int rank, ag_dtype dtype, void *grads, void *values,
                      void *velocity, int64_t n, float scale, float lr, float momentum,
                      bool use_momentum) {
    AG_REQUIRE(comm != nullptr, AG_ERR_INVALID, "communicator is null");
    ag_comm_member *m = comm->member(rank);
    AG_REQUIRE(m != nullptr, AG_ERR_INVALID, "rank %d is not driven by this process", rank);
    AG_REQUIRE(comm->fused_ready, AG_ERR_UNSUPPORTED,
               "this communicator has no peer-addressable blocks (peer access unavailable)");
    AG_REQUIRE(is_float_dtype(dtype), AG_ERR_DTYPE, "fused update of dtype %d", (int)dtype);
    const size_t es = dtype_size(dtype);
    const int64_t padded = (int64_t)((n * es + 15) / 16 * 16);
    AG_REQUIRE((size_t)padded <= kCapWords * 4, AG_ERR_LIMIT,
               "bucket of %lld bytes exceeds the %zu-byte limit of the fused all-reduce; use "
               "ag_allreduce_sum and ag_model_apply_update",
               (long long)(n * es), kCapWords * 4);
    AG_REQUIRE((reinterpret_cast<uintptr_t>(grads) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(values) & 15) == 0 &&
                   (!use_momentum || (reinterpret_cast<uintptr_t>(velocity) & 15) == 0),
               AG_ERR_INVALID, "buckets must be 16-byte aligned");
    AG_ENTER(m->dev);
    FusedParams p;
    for (int q = 0; q < comm->world; ++q) p.peer[q] = m->peer_sym[q];
    p.world = comm->world;
    p.rank = rank;
    p.seq = ++m->seq;
    p.words = padded / 4;
    p.scale = scale;
    p.lr = lr;
    p.momentum = momentum;
    p.use_momentum = use_momentum ? 1 : 0;
    p.timeout_cycles = (long long)(comm->timeout_s * 1e3 * (double)m->clock_khz);
    p.status = m->dev->status_dev;
    const int64_t packs = padded / 16;
    if (packs == 0) return AG_OK;
    const unsigned ctas = (unsigned)ceil_div(packs, 256);
    if (dtype == AG_F32)
        allreduce_update_kernel<float><<<ctas, 256, 0, m->dev->stream>>>(
            (float *)grads, (float *)values, (float *)velocity, p);
    else
        allreduce_update_kernel<__nv_bfloat16><<<ctas, 256, 0, m->dev->stream>>>(
            (__nv_bfloat16 *)grads, (__nv_bfloat16 *)values, (__nv_bfloat16 *)velocity, p);
    AG_CHECK_LAUNCH();
    return AG_OK;
}

}  // namespace ag

using namespace ag;

extern "C" {

int ag_comm_unique_id(void *id_out, size_t bytes) {
    AG_REQUIRE(id_out != nullptr && bytes >= sizeof(nccl_unique_id), AG_ERR_INVALID,
               "id buffer must hold %zu bytes", sizeof(nccl_unique_id));
    AG_TRY(require_nccl());
    nccl_unique_id id;
    AG_NCCL_TRY(nccl().GetUniqueId(&id));
    memcpy(id_out, &id, sizeof(id));
    return AG_OK;
}

int ag_comm_create(ag_device *const *devs, int n, ag_comm **out) {
    AG_REQUIRE(devs && out && n >= 1 && n <= kMaxRanks, AG_ERR_INVALID,
               "1..%d devices are supported", kMaxRanks);
    *out = nullptr;
    AG_TRY(require_nccl());
    std::vector<int> ordinals;
    for (int i = 0; i < n; ++i) {
        AG_REQUIRE(devs[i] != nullptr, AG_ERR_INVALID, "device %d is null", i);
        for (int j = 0; j < i; ++j)
            AG_REQUIRE(devs[j]->ordinal != devs[i]->ordinal, AG_ERR_INVALID,
                       "GPU %d appears twice in the communicator", devs[i]->ordinal);
        ordinals.push_back(devs[i]->ordinal);
    }
    ag_comm *c = new ag_comm();
    c->world = n;
    c->members.resize((size_t)n);
    std::vector<nccl_comm_t> comms((size_t)n, nullptr);
    int r = nccl().CommInitAll(comms.data(), n, ordinals.data());
    if (r != kNcclSuccess) {
        delete c;
        return fail(AG_ERR_CUDA, "ncclCommInitAll failed: %s", nccl().GetErrorString(r));
    }
    for (int i = 0; i < n; ++i) {
        c->members[(size_t)i].dev = devs[i];
        c->members[(size_t)i].nccl = comms[(size_t)i];
    }
    // Symmetric blocks: every GPU maps every other GPU's block through peer access.
    bool peers_ok = true;
    for (int i = 0; i < n && peers_ok; ++i) {
        if (cudaSetDevice(ordinals[(size_t)i]) != cudaSuccess) { peers_ok = false; break; }
        for (int j = 0; j < n; ++j) {
            if (i == j) continue;
            int can = 0;
            cudaDeviceCanAccessPeer(&can, ordinals[(size_t)i], ordinals[(size_t)j]);
            if (!can) { peers_ok = false; break; }
            cudaError_t e = cudaDeviceEnablePeerAccess(ordinals[(size_t)j], 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else if (e != cudaSuccess) { cudaGetLastError(); peers_ok = false; break; }
        }
        if (peers_ok && alloc_sym(c->members[(size_t)i], n) != AG_OK) peers_ok = false;
    }
    if (peers_ok) {
        for (int i = 0; i < n; ++i)
            for (int j = 0; j < n; ++j) c->members[(size_t)i].peer_sym[j] = c->members[(size_t)j].sym;
        c->fused_ready = true;
    }
    *out = c;
    return AG_OK;
}

int ag_comm_create_rank(ag_device *dev, int world, int rank, const void *unique_id, size_t id_bytes,
                        ag_comm **out) {
    AG_REQUIRE(dev && out && unique_id, AG_ERR_INVALID, "null argument");
    AG_REQUIRE(id_bytes >= sizeof(nccl_unique_id), AG_ERR_INVALID, "unique id is %zu bytes",
               sizeof(nccl_unique_id));
    AG_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, AG_ERR_INVALID,
               "bad world / rank (%d / %d)", world, rank);
    *out = nullptr;
    AG_TRY(require_nccl());
    AG_ENTER(dev);
    nccl_unique_id id;
    memcpy(&id, unique_id, sizeof(id));
    nccl_comm_t nc = nullptr;
    AG_NCCL_TRY(nccl().CommInitRank(&nc, world, id, rank));
    ag_comm *c = new ag_comm();
    c->world = world;
    c->multi_process = true;
    c->my_rank = rank;
    c->members.resize(1);
    ag_comm_member &m = c->members[0];
    m.dev = dev;
    m.nccl = nc;
    *out = c;
    // Symmetric block: exchange CUDA IPC handles with an all-gather, then map the peers'.
    if (alloc_sym(m, world) != AG_OK) return AG_OK;  // plain all-reduce still works
    cudaIpcMemHandle_t mine;
    if (cudaIpcGetMemHandle(&mine, m.sym) != cudaSuccess) {
        cudaGetLastError();
        return AG_OK;
    }
    constexpr size_t H = sizeof(cudaIpcMemHandle_t);
    void *d_all = nullptr;
    AG_CUDA_TRY(cudaMalloc(&d_all, H * (size_t)world));
    AG_CUDA_TRY(cudaMemcpyAsync((char *)d_all + H * (size_t)rank, &mine, H, cudaMemcpyHostToDevice,
                                dev->stream));
    int r = nccl().AllGather((char *)d_all + H * (size_t)rank, d_all, H, kNcclInt8, nc, dev->stream);
    std::vector<cudaIpcMemHandle_t> all((size_t)world);
    cudaError_t e = cudaSuccess;
    if (r == kNcclSuccess)
        e = cudaMemcpyAsync(all.data(), d_all, H * (size_t)world, cudaMemcpyDeviceToHost, dev->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);
    cudaFree(d_all);
    if (r != kNcclSuccess || e != cudaSuccess) {
        cudaGetLastError();
        return AG_OK;
    }
    bool ok = true;
    for (int q = 0; q < world && ok; ++q) {
        if (q == rank) {
            m.peer_sym[q] = m.sym;
            continue;
        }
        void *p = nullptr;
        if (cudaIpcOpenMemHandle(&p, all[(size_t)q], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            ok = false;
            break;
        }
        m.peer_sym[q] = p;
        m.opened[q] = true;
    }
    // every rank must have mapped every block before anyone's kernel writes a flag there:
    // the all-reduce of one byte below is that barrier, and it also tells everyone whether
    // some rank failed to map
    unsigned char *d_flag = nullptr;
    AG_CUDA_TRY(cudaMalloc((void **)&d_flag, 1));
    unsigned char bad = ok ? 0 : 1;
    AG_CUDA_TRY(cudaMemcpyAsync(d_flag, &bad, 1, cudaMemcpyHostToDevice, dev->stream));
    AG_NCCL_TRY(nccl().AllReduce(d_flag, d_flag, 1, kNcclUint8, kNcclSum, nc, dev->stream));
    AG_CUDA_TRY(cudaMemcpyAsync(&bad, d_flag, 1, cudaMemcpyDeviceToHost, dev->stream));
    AG_CUDA_TRY(cudaStreamSynchronize(dev->stream));
    cudaFree(d_flag);
    c->fused_ready = bad == 0;
    return AG_OK;
}

int ag_comm_world(ag_comm *comm, int *world, int *fused_available) {
    AG_REQUIRE(comm != nullptr, AG_ERR_INVALID, "communicator is null");
    if (world) *world = comm->world;
    if (fused_available) *fused_available = comm->fused_ready ? 1 : 0;
    return AG_OK;
}

int ag_comm_set_timeout(ag_comm *comm, double seconds) {
    AG_REQUIRE(comm != nullptr && seconds > 0.0, AG_ERR_INVALID, "bad timeout");
    comm->timeout_s = seconds;
    return AG_OK;
}

int ag_allreduce_sum(ag_comm *comm, int rank, ag_dtype dtype, void *buf, int64_t n) {
    AG_REQUIRE(comm != nullptr, AG_ERR_INVALID, "communicator is null");
    ag_comm_member *m = comm->member(rank);
    AG_REQUIRE(m != nullptr, AG_ERR_INVALID, "rank %d is not driven by this process", rank);
    AG_REQUIRE(n >= 0, AG_ERR_SHAPE, "negative length");
    if (n == 0) return AG_OK;
    AG_REQUIRE(buf != nullptr, AG_ERR_INVALID, "buffer is null");
    int dt = 0;
    AG_TRY(nccl_dtype(dtype, &dt));
    AG_ENTER(m->dev);
    AG_NCCL_TRY(nccl().AllReduce(buf, buf, (size_t)n, dt, kNcclSum, m->nccl, m->dev->stream));
    return AG_OK;
}

int ag_allreduce_sum_all(ag_comm *comm, ag_dtype dtype, void *const *bufs, int64_t n) {
    AG_REQUIRE(comm != nullptr && bufs != nullptr, AG_ERR_INVALID, "null argument");
    AG_REQUIRE(!comm->multi_process, AG_ERR_INVALID,
               "this communicator drives one rank per process: use ag_allreduce_sum");
    AG_REQUIRE(n >= 0, AG_ERR_SHAPE, "negative length");
    if (n == 0) return AG_OK;
    int dt = 0;
    AG_TRY(nccl_dtype(dtype, &dt));
    AG_NCCL_TRY(nccl().GroupStart());
    int first_error = kNcclSuccess;
    for (int r = 0; r < comm->world; ++r) {
        ag_comm_member &m = comm->members[(size_t)r];
        if (!bufs[r]) { first_error = -1; continue; }
        cudaSetDevice(m.dev->ordinal);
        int e = nccl().AllReduce(bufs[r], bufs[r], (size_t)n, dt, kNcclSum, m.nccl, m.dev->stream);
        if (e != kNcclSuccess && first_error == kNcclSuccess) first_error = e;
    }
    int e = nccl().GroupEnd();
    AG_REQUIRE(first_error != -1, AG_ERR_INVALID, "a rank's buffer is null");
    AG_NCCL_TRY(first_error);
    AG_NCCL_TRY(e);
    return AG_OK;
}

int ag_comm_wait(ag_comm *comm, int rank) {
    AG_REQUIRE(comm != nullptr, AG_ERR_INVALID, "communicator is null");
    ag_comm_member *m = comm->member(rank);
    AG_REQUIRE(m != nullptr, AG_ERR_INVALID, "rank %d is not driven by this process", rank);
    AG_ENTER(m->dev);
    // Poll instead of blocking in cudaStreamSynchronize: a collective whose peer never
    // arrives would block forever; after the timeout the communicator is aborted and the
    // caller gets an error it can act on.
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        int async_err = kNcclSuccess;
        AG_NCCL_TRY(nccl().CommGetAsyncError(m->nccl, &async_err));
        if (async_err != kNcclSuccess && async_err != kNcclInProgress)
            return fail(AG_ERR_CUDA, "NCCL reported an asynchronous error: %s",
                        nccl().GetErrorString(async_err));
        cudaError_t q = cudaStreamQuery(m->dev->stream);
        if (q == cudaSuccess) break;
        if (q != cudaErrorNotReady)
            return fail(AG_ERR_CUDA, "stream error: %s", cudaGetErrorString(q));
        const double waited =
            std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        // the fused kernel's own wait ends after timeout_s and reports through the status
        // word: give it room to do so before treating the stream as stuck in a collective
        if (waited > 2.0 * comm->timeout_s + 0.5) {
            nccl().CommAbort(m->nccl);
            m->nccl = nullptr;
            return fail(AG_ERR_DEVICE_TIMEOUT,
                        "collective on rank %d did not finish within %.1f s (a peer never joined); "
                        "the communicator was aborted", rank, 2.0 * comm->timeout_s + 0.5);
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    return ag_device_wait(m->dev);  // also reports a timeout of the fused kernel's wait
}

int ag_comm_destroy(ag_comm *comm) {
    if (!comm) return AG_OK;
    for (ag_comm_member &m : comm->members) {
        if (m.dev) {
            cudaSetDevice(m.dev->ordinal);
            cudaStreamSynchronize(m.dev->stream);
        }
        for (int q = 0; q < kMaxRanks; ++q)
            if (m.opened[q] && m.peer_sym[q]) cudaIpcCloseMemHandle(m.peer_sym[q]);
        if (m.sym) cudaFree(m.sym);
        if (m.nccl && nccl().ok) nccl().CommDestroy(m.nccl);
    }
    delete comm;
    return AG_OK;
}

}  // extern "C"

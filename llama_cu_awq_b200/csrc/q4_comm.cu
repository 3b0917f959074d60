// Tensor-parallel collectives for 8-16 KB fp16 vectors: one-shot push over NVLink / NVSwitch peer memory.
// Replaces cudaAllReduce / cudaAllGather / reduce_sum_half_kernel of the reference (cuda_comm.h:144-275),
// which stage through a 128 MB buffer, two host barriers and one kernel per peer for every call.
//
// Every rank owns an inbox in its own memory: slots[2][g][Q4_COMM_MAX_GATHER_HALFS] halfs and flags[2][g] words,
// double buffered by the parity of a call counter (epoch). A call is one kernel:
//   1. store this rank's vector into slot [parity][rank] of EVERY rank's inbox (plain 128-bit peer stores),
//   2. fence, then release-store the epoch into flag [parity][rank] of every inbox,
//   3. acquire-spin (bounded) on the g local flags,
//   4. add the g local slots in rank order in fp32 (all ranks see the same order -> identical bits; the
//      reference adds in a rank-dependent order in fp16, cuda_comm.h:193-219) and write fp16.
// Parity p is reused at epoch e+2; a rank can only reach e+2 after every peer published e+1, which a peer does
// only after it finished reading its epoch-e slots, so no slot is overwritten while it is still being read.
// No host synchronisation is involved, so the call can be captured in a CUDA graph.
// Waits are bounded: after the communicator's wait limit (q4_comm_set_wait_limit_ns, default 2 s) the kernel records
// Q4_ERR_TIMEOUT in the status word and returns.
#include <chrono>
#include <dlfcn.h>
#include <mutex>
#include <string.h>
#include <thread>

#include "q4_comm_internal.h"

namespace {
constexpr unsigned long long kDefaultWaitNs = 2000ULL * 1000 * 1000;  // default bound of the flag wait: 2 s on the device's global timer
constexpr int kCommThreads = 1024;

// Messages above kWideAbove halfs are moved by kWideCtas CTAs, each with its own part of the vector, its own flags and its
// own call counter (a single CTA would need one call per 64 KB piece).
constexpr int kWideCtas = 4;        // measured on 2 GPUs at 128 / 256 KB: 4 CTAs 13.6 / 15.7 us, 8: 16.1 / 17.1, 16: 18.8 / 19.5
constexpr int kWideAbove = 32768;   // one CTA moves up to 64 KB faster (12.5 us) than several do
constexpr int kWidePad = 1;         // words between the flags of two CTAs (spreading them over cache lines changed nothing)

struct Inbox {
    uint32_t flags[2][Q4_MAX_GPUS];
    uint32_t epoch;    // local call counter
    uint32_t status;   // 0 or Q4_ERR_TIMEOUT
    uint32_t pad[14];
    uint32_t wide_flags[2][kWideCtas][Q4_MAX_GPUS * kWidePad];
    uint32_t wide_epoch[kWideCtas];
    __half slots[2][Q4_MAX_GPUS][Q4_COMM_MAX_GATHER_HALFS];
    // The wide kernel has slots of its own: its call counters are independent of the one-CTA kernel's, so the two must not
    // share a buffer (the parity argument above holds per counter).
    __half wide_slots[2][Q4_MAX_GPUS][Q4_COMM_MAX_HALFS];
    Q4LLArea ll;       // exchange area of the fused decode kernel
};

struct PeerPtrs { Inbox* p[Q4_MAX_GPUS]; };
}  // namespace

struct q4_comm_id {
    int gpu_count;
    std::mutex mu;
    Inbox* inbox[Q4_MAX_GPUS];
    int registered;
};

struct q4_comm {
    int rank, gpu_count;
    Inbox* local;
    PeerPtrs peers;
    bool imported[Q4_MAX_GPUS];  // opened through IPC (must be closed)
    q4_comm_id* id;
    unsigned long long wait_ns = kDefaultWaitNs;
    int backend = Q4_COMM_BACKEND_P2P;
    void* nccl = nullptr;        // ncclComm_t once q4_comm_nccl_init has run
};

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// mode 0: all-reduce (sum) of buf[count] in place. mode 1: all-gather, send[count] -> recv[g*count].
__global__ void __launch_bounds__(kCommThreads) comm_kernel(PeerPtrs peers, Inbox* local, int rank, int g, __half* buf, const __half* send,
                                                            int count, int mode, unsigned long long wait_ns) {
    __shared__ uint32_t s_epoch;
    griddep_wait();
    griddep_launch_dependents();
    if (threadIdx.x == 0) s_epoch = ++local->epoch;
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const int par = epoch & 1;
    const __half* src = mode == 0 ? buf : send;
    const int nvec = count >> 3;  // count is a multiple of 8
    for (int p = 0; p < g; p++) {
        uint4* dst = reinterpret_cast<uint4*>(peers.p[p]->slots[par][rank]);
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = reinterpret_cast<const uint4*>(src)[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < g) {
        st_release_sys(&peers.p[threadIdx.x]->flags[par][rank], epoch);
        unsigned long long t_start = 0;
        unsigned spins = 0;
        while (ld_acquire_sys(&local->flags[par][threadIdx.x]) != epoch) {
            if ((++spins & 255u) == 0) {
                const unsigned long long now = global_timer_ns();
                if (t_start == 0) t_start = now;
                else if (now - t_start > wait_ns) { local->status = Q4_ERR_TIMEOUT; break; }
            }
        }
    }
    __syncthreads();
    if (mode == 0) {
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] = 0.f;
            for (int r = 0; r < g; r++) {
                const uint4 v = reinterpret_cast<const uint4*>(local->slots[par][r])[i];
                const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                for (int j = 0; j < 4; j++) { const float2 f = __half22float2(h[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
            }
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int j = 0; j < 4; j++) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
            reinterpret_cast<uint4*>(buf)[i] = o;
        }
    } else {
        for (int r = 0; r < g; r++)
            for (int i = threadIdx.x; i < nvec; i += blockDim.x)
                reinterpret_cast<uint4*>(buf + (size_t)r * count)[i] = reinterpret_cast<const uint4*>(local->slots[par][r])[i];
    }
}

// The all-reduce for long vectors: CTA c owns the c-th part of the vector and runs the same protocol as comm_kernel on it
// with flags and a call counter of its own (wide_flags[.][.][c], wide_epoch[c]); CTAs never wait for one another, only for
// the same CTA of the peers, so they need not be resident together. Every CTA takes part in every call, also with an empty
// part, which keeps the counters of all ranks in step.
__global__ void __launch_bounds__(kCommThreads) comm_wide_kernel(PeerPtrs peers, Inbox* local, int rank, int g, __half* buf, int count,
                                                                 unsigned long long wait_ns) {
    __shared__ uint32_t s_epoch;
    griddep_wait();
    griddep_launch_dependents();
    const int c = blockIdx.x;
    if (threadIdx.x == 0) s_epoch = ++local->wide_epoch[c];
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const int par = epoch & 1;
    const int nvec = count >> 3;  // count is a multiple of 8
    const int per = (nvec + kWideCtas - 1) / kWideCtas;
    const int v0 = min(c * per, nvec), v1 = min(v0 + per, nvec);
    for (int p = 0; p < g; p++) {
        uint4* dst = reinterpret_cast<uint4*>(peers.p[p]->wide_slots[par][rank]);
        for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) dst[i] = reinterpret_cast<const uint4*>(buf)[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < g) {
        st_release_sys(&peers.p[threadIdx.x]->wide_flags[par][c][rank * kWidePad], epoch);
        unsigned long long t_start = 0;
        unsigned spins = 0;
        while (ld_acquire_sys(&local->wide_flags[par][c][threadIdx.x * kWidePad]) != epoch) {
            if ((++spins & 255u) == 0) {
                const unsigned long long now = global_timer_ns();
                if (t_start == 0) t_start = now;
                else if (now - t_start > wait_ns) { local->status = Q4_ERR_TIMEOUT; break; }
            }
        }
    }
    __syncthreads();
    for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] = 0.f;
        for (int r = 0; r < g; r++) {
            const uint4 v = reinterpret_cast<const uint4*>(local->wide_slots[par][r])[i];
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; j++) { const float2 f = __half22float2(h[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
        }
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; j++) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
        reinterpret_cast<uint4*>(buf)[i] = o;
    }
}

int alloc_inbox(Inbox** out) {
    Q4_CUDA_TRY(cudaMalloc((void**)out, sizeof(Inbox)));
    Q4_CUDA_TRY(cudaMemset(*out, 0, sizeof(Inbox)));
    Q4_CUDA_TRY(cudaDeviceSynchronize());
    return Q4_OK;
}

}  // namespace

int q4_comm_world(const q4_comm* c) { return c ? c->gpu_count : 1; }
int q4_comm_rank(const q4_comm* c) { return c ? c->rank : 0; }
Q4LLArea* q4_comm_ll_area(const q4_comm* c, int peer) {
    if (!c || peer < 0 || peer >= c->gpu_count || !c->peers.p[peer]) return nullptr;
    return &c->peers.p[peer]->ll;
}

extern "C" int q4_comm_id_create(q4_comm_id** id, int gpu_count) {
    if (!id || gpu_count < 1 || gpu_count > Q4_MAX_GPUS) return Q4_ERR_INVALID;
    q4_comm_id* p = new q4_comm_id();
    p->gpu_count = gpu_count;
    p->registered = 0;
    for (int i = 0; i < Q4_MAX_GPUS; i++) p->inbox[i] = nullptr;
    *id = p;
    return Q4_OK;
}

extern "C" int q4_comm_id_destroy(q4_comm_id* id) {
    delete id;
    return Q4_OK;
}

// Thread-per-GPU flavour. Every rank allocates its inbox, publishes the pointer in the shared id and waits
// (bounded) until all gpu_count ranks have done so; all ranks must therefore call this concurrently.
extern "C" int q4_comm_init_rank(q4_comm** comm, int gpu_count, q4_comm_id* id, int rank) {
    if (!comm || !id || rank < 0 || rank >= gpu_count || gpu_count != id->gpu_count) return Q4_ERR_INVALID;
    q4_comm* c = new q4_comm();
    c->rank = rank;
    c->gpu_count = gpu_count;
    c->id = id;
    for (int i = 0; i < Q4_MAX_GPUS; i++) { c->peers.p[i] = nullptr; c->imported[i] = false; }
    int dev = 0;
    Q4_CUDA_TRY(cudaGetDevice(&dev));
    for (int i = 0; i < gpu_count; i++) {
        if (i == dev) continue;
        int can = 0;
        Q4_CUDA_TRY(cudaDeviceCanAccessPeer(&can, dev, i));
        if (!can) { delete c; return Q4_ERR_CUDA; }
        cudaError_t e = cudaDeviceEnablePeerAccess(i, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
        else if (e != cudaSuccess) { q4_note_cuda_error(e, __FILE__, __LINE__); delete c; return Q4_ERR_CUDA; }
    }
    if (int e = alloc_inbox(&c->local)) { delete c; return e; }
    {
        std::lock_guard<std::mutex> lk(id->mu);
        id->inbox[rank] = c->local;
        id->registered++;
    }
    // bounded rendezvous: wait (at most 60 s of wall time) until every rank has published its inbox
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        {
            std::lock_guard<std::mutex> lk(id->mu);
            if (id->registered >= gpu_count) break;
            if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(60)) {
                id->inbox[rank] = nullptr;   // withdraw: nobody has read the table yet (readers wait for the full count)
                id->registered--;
                cudaFree(c->local);
                delete c;
                return Q4_ERR_TIMEOUT;
            }
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    for (int i = 0; i < gpu_count; i++) c->peers.p[i] = id->inbox[i];
    *comm = c;
    return Q4_OK;
}

extern "C" int q4_comm_create_local(q4_comm** comm, int gpu_count, int rank) {
    if (!comm || gpu_count < 1 || gpu_count > Q4_MAX_GPUS || rank < 0 || rank >= gpu_count) return Q4_ERR_INVALID;
    q4_comm* c = new q4_comm();
    c->rank = rank;
    c->gpu_count = gpu_count;
    c->id = nullptr;
    for (int i = 0; i < Q4_MAX_GPUS; i++) { c->peers.p[i] = nullptr; c->imported[i] = false; }
    if (int e = alloc_inbox(&c->local)) { delete c; return e; }
    c->peers.p[rank] = c->local;
    *comm = c;
    return Q4_OK;
}

extern "C" int q4_comm_export(q4_comm* comm, uint8_t handle[64]) {
    if (!comm || !handle) return Q4_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    Q4_CUDA_TRY(cudaIpcGetMemHandle(&h, comm->local));
    memcpy(handle, &h, 64);
    return Q4_OK;
}

extern "C" int q4_comm_import(q4_comm* comm, int peer, const uint8_t handle[64]) {
    if (!comm || !handle || peer < 0 || peer >= comm->gpu_count) return Q4_ERR_INVALID;
    if (peer == comm->rank) return Q4_OK;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void* p = nullptr;
    Q4_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    comm->peers.p[peer] = (Inbox*)p;
    comm->imported[peer] = true;
    return Q4_OK;
}

static int comm_launch(q4_comm* c, cudaStream_t s, __half* buf, const __half* send, int count, int mode) {
    if (!c || !buf || count <= 0 || (count & 7)) return Q4_ERR_INVALID;
    if (count > (mode == 0 ? Q4_COMM_MAX_HALFS : Q4_COMM_MAX_GATHER_HALFS)) return Q4_ERR_LIMIT;
    for (int i = 0; i < c->gpu_count; i++)
        if (!c->peers.p[i]) return Q4_ERR_INVALID;
    if (mode == 0 && count > kWideAbove) {
        Q4Launch L(dim3(kWideCtas), dim3(kCommThreads), 0, s);
        Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, comm_wide_kernel, c->peers, c->local, c->rank, c->gpu_count, buf, count, c->wait_ns));
        return Q4_OK;
    }
    Q4Launch L(dim3(1), dim3(kCommThreads), 0, s);
    Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, comm_kernel, c->peers, c->local, c->rank, c->gpu_count, buf, send, count, mode, c->wait_ns));
    return Q4_OK;
}

// ------------------------------------------------------------------------------------------------------------
// NCCL backend (the reference's -DENABLE_NCCL build: ncclAllReduce / ncclAllGather at the same call sites,
// llama2_q4.cu:474,505,534). The library is opened at run time, so that nothing here depends on it being installed;
// whichever libnccl.so.2 the process already holds (e.g. the one an ML framework loaded) is the one that is used.
// ------------------------------------------------------------------------------------------------------------
namespace {
struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, q4_nccl_id, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    bool ok = false;
};
constexpr int kNcclHalf = 6, kNcclSum = 0;   // ncclFloat16, ncclSum (nccl.h)
std::mutex g_nccl_mu;
NcclApi g_nccl;

const NcclApi* nccl_api() {
    std::lock_guard<std::mutex> lk(g_nccl_mu);
    if (!g_nccl.lib) {
        g_nccl.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!g_nccl.lib) g_nccl.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.lib) {
            g_nccl.GetUniqueId = (int (*)(void*))dlsym(g_nccl.lib, "ncclGetUniqueId");
            g_nccl.CommInitRank = (int (*)(void**, int, q4_nccl_id, int))dlsym(g_nccl.lib, "ncclCommInitRank");
            g_nccl.AllReduce = (int (*)(const void*, void*, size_t, int, int, void*, cudaStream_t))dlsym(g_nccl.lib, "ncclAllReduce");
            g_nccl.AllGather = (int (*)(const void*, void*, size_t, int, void*, cudaStream_t))dlsym(g_nccl.lib, "ncclAllGather");
            g_nccl.CommDestroy = (int (*)(void*))dlsym(g_nccl.lib, "ncclCommDestroy");
            g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.AllReduce && g_nccl.AllGather && g_nccl.CommDestroy;
        }
    }
    return g_nccl.ok ? &g_nccl : nullptr;
}
}  // namespace

extern "C" int q4_comm_nccl_available(void) { return nccl_api() ? 1 : 0; }

extern "C" int q4_comm_nccl_unique_id(q4_nccl_id* id) {
    if (!id) return Q4_ERR_INVALID;
    const NcclApi* a = nccl_api();
    if (!a) return Q4_ERR_UNSUPPORTED_SIZE;
    return a->GetUniqueId(id) == 0 ? Q4_OK : Q4_ERR_CUDA;
}

extern "C" int q4_comm_nccl_init(q4_comm* comm, const q4_nccl_id* id) {
    if (!comm || !id) return Q4_ERR_INVALID;
    const NcclApi* a = nccl_api();
    if (!a) return Q4_ERR_UNSUPPORTED_SIZE;
    if (comm->nccl) return Q4_OK;
    void* nc = nullptr;
    if (a->CommInitRank(&nc, comm->gpu_count, *id, comm->rank) != 0) return Q4_ERR_CUDA;
    comm->nccl = nc;
    return Q4_OK;
}

extern "C" int q4_comm_set_backend(q4_comm* comm, int backend) {
    if (!comm || backend < Q4_COMM_BACKEND_P2P || backend > Q4_COMM_BACKEND_AUTO) return Q4_ERR_INVALID;
    if (backend == Q4_COMM_BACKEND_NCCL && !comm->nccl) return Q4_ERR_INVALID;
    comm->backend = backend;
    return Q4_OK;
}

// Which implementation serves a message of `count` halfs. AUTO follows the measured latency table: the one-shot peer
// push for the vectors of this path (8-16 KB), NCCL for large messages when it is attached.
// Measured, us per call, peer push vs NCCL: 2 GPUs 8.7 / 9.2 at 8 KB, 9.3 / 10.1 at 16 KB, 10.2 / 10.0 at 32 KB, 12.3 / 10.3 at
// 64 KB; 4 GPUs 9.3 / 15.1 at 8 KB, 12.2 / 16.0 at 32 KB, 16.3 / 16.4 at 64 KB, 14.8 / 16.7 at 128 KB, 19.2 / 16.5 at 256 KB.
static int auto_nccl_above(int gpu_count) { return gpu_count <= 2 ? 16384 : 65536; }   // halfs: 32 KB on two GPUs, 128 KB on more
static bool use_nccl(const q4_comm* c, int count) {
    if (!c->nccl) return false;
    if (c->backend == Q4_COMM_BACKEND_NCCL) return true;
    return c->backend == Q4_COMM_BACKEND_AUTO && count > auto_nccl_above(c->gpu_count);
}

bool q4_comm_prefers_nccl(const q4_comm* c, int count) { return c && use_nccl(c, count); }

extern "C" int q4_comm_set_wait_limit_ns(q4_comm* comm, unsigned long long ns) {
    if (!comm) return Q4_ERR_INVALID;
    comm->wait_ns = ns ? ns : kDefaultWaitNs;
    return Q4_OK;
}

// After a recorded timeout the flags and the call counter of this rank are out of step with its peers': clear them.
// Every rank of the group calls this (with a host-side barrier around the calls) before the next collective.
extern "C" int q4_comm_reset(q4_comm* comm) {
    if (!comm) return Q4_ERR_INVALID;
    Q4_CUDA_TRY(cudaDeviceSynchronize());
    Q4_CUDA_TRY(cudaMemset(comm->local, 0, offsetof(Inbox, slots)));
    Q4_CUDA_TRY(cudaDeviceSynchronize());
    return Q4_OK;
}

extern "C" int q4_all_reduce(q4_comm* comm, void* stream, uint16_t* buf, int count) {
    if (comm && comm->gpu_count == 1) return Q4_OK;  // cuda_comm.h:163-171: in place, nothing to do
    if (comm && buf && count > 0 && use_nccl(comm, count))
        return nccl_api()->AllReduce(buf, buf, (size_t)count, kNcclHalf, kNcclSum, comm->nccl, (cudaStream_t)stream) == 0 ? Q4_OK : Q4_ERR_CUDA;
    return comm_launch(comm, (cudaStream_t)stream, (__half*)buf, nullptr, count, 0);
}

int q4_all_reduce_peer_push(q4_comm* comm, void* stream, uint16_t* buf, int count) {
    if (comm && comm->gpu_count == 1) return Q4_OK;
    return comm_launch(comm, (cudaStream_t)stream, (__half*)buf, nullptr, count, 0);
}

extern "C" int q4_all_gather(q4_comm* comm, void* stream, const uint16_t* send, uint16_t* recv, int sendcount) {
    if (!send) return Q4_ERR_INVALID;
    if (comm && comm->gpu_count == 1) {
        if (send != recv) Q4_CUDA_TRY(cudaMemcpyAsync(recv, send, (size_t)sendcount * 2, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
        return Q4_OK;
    }
    if (comm && recv && sendcount > 0 && use_nccl(comm, sendcount))
        return nccl_api()->AllGather(send, recv, (size_t)sendcount, kNcclHalf, comm->nccl, (cudaStream_t)stream) == 0 ? Q4_OK : Q4_ERR_CUDA;
    return comm_launch(comm, (cudaStream_t)stream, (__half*)recv, (const __half*)send, sendcount, 1);
}

extern "C" int q4_comm_status(q4_comm* comm) {
    if (!comm) return Q4_ERR_INVALID;
    uint32_t st = 0;
    Q4_CUDA_TRY(cudaMemcpy(&st, &comm->local->status, 4, cudaMemcpyDeviceToHost));
    return (int)st;
}

extern "C" int q4_comm_destroy(q4_comm* comm) {
    if (!comm) return Q4_OK;
    if (comm->nccl && nccl_api()) nccl_api()->CommDestroy(comm->nccl);
    for (int i = 0; i < comm->gpu_count; i++)
        if (comm->imported[i]) cudaIpcCloseMemHandle(comm->peers.p[i]);
    cudaFree(comm->local);
    delete comm;
    return Q4_OK;
}

#ifdef Q4_TEST_BUILD
// Test build only: makes `other`'s inbox (a second communicator of the same process and device) stand in for rank
// `peer` of `comm`. Nobody ever writes that rank's flags, so a collective on `comm` stores into valid memory, waits
// for the missing rank until the wait limit and records Q4_ERR_TIMEOUT: the time-out path exercised on one GPU.
extern "C" int q4_test_comm_set_peer(q4_comm* comm, int peer, q4_comm* other) {
    if (!comm || !other || peer < 0 || peer >= comm->gpu_count || peer == comm->rank) return Q4_ERR_INVALID;
    comm->peers.p[peer] = other->local;
    return Q4_OK;
}
#endif

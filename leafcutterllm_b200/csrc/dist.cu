// Sums over the ranks of a model cut across GPUs (one process per GPU).  The reference runs on one device and has
// nothing like this; the layer structure that is cut is rust/src/inference/engine.rs:95-116.
//
// Two ways to take a sum, chosen once at lc_dist_init:
//   NCCL            ncclAllReduce on the library's stream (libnccl.so.2 is loaded at run time with dlopen, so a single-GPU
//                   user of the library never needs it);
//   peer memory     every rank keeps its partial rows in a buffer that the other ranks have mapped (CUDA IPC).  ONE kernel
//                   per sum: it tells every peer "my rows of sum number e are written" with a flag store into the peer's
//                   memory, waits (bounded, by the global timer) until every peer has said the same, then reads all ranks'
//                   rows with plain loads over NVLink and adds them in rank order -- so every rank computes the same bits.
//                   No multicast, no library kernel ever sees a peer pointer.
// Buffer reuse: a sum's partial rows go to one of two slots, consecutive sums alternate.  A rank can start writing a slot
// again only after it finished the sum in between, which needed every peer's flag for that sum, which a peer raises only
// after it finished reading the sum before: two slots are enough.
//
// group_sum_kernel is the same arithmetic for several ranks that live in ONE process on ONE GPU (testing a cut model with a
// single GPU): one kernel over all ranks' rows, nothing waits for anything.
#include <dlfcn.h>
#include <algorithm>
#include <vector>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include "lc_kernels.h"
#include "lc_tma.cuh"

namespace lc {

namespace {

constexpr int kMaxRanks = 8;
constexpr size_t kFlagBytes = 4096;          // head of the shared buffer: one epoch word per peer
constexpr size_t kKeyBytes = 4096;           // per slot: greedy-pick keys, up to 512 sequences
constexpr size_t kPeerSumLimit = (size_t)2 << 20;  // larger sums go through NCCL

// ---- NCCL through dlopen ----
typedef struct { char internal[128]; } NcclId;
typedef void* NcclComm;
typedef int (*fn_GetUniqueId)(NcclId*);
typedef int (*fn_CommInitRank)(NcclComm*, int, NcclId, int);
typedef int (*fn_AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t);
typedef int (*fn_AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t);
typedef int (*fn_CommDestroy)(NcclComm);
typedef const char* (*fn_GetErrorString)(int);
enum { kNcclInt8 = 0, kNcclInt64 = 4, kNcclFloat32 = 7, kNcclSum = 0, kNcclMax = 2 };

struct Nccl {
    void* dl = nullptr;
    fn_GetUniqueId GetUniqueId = nullptr;
    fn_CommInitRank CommInitRank = nullptr;
    fn_AllReduce AllReduce = nullptr;
    fn_AllGather AllGather = nullptr;
    fn_CommDestroy CommDestroy = nullptr;
    fn_GetErrorString GetErrorString = nullptr;
};
Nccl g_nccl;

int32_t nccl_load() {
    if (g_nccl.dl) return LC_OK;
    const char* names[] = {getenv("LC_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        if (!n || !*n) continue;
        g_nccl.dl = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.dl) break;
    }
    LC_CHECK(g_nccl.dl != nullptr, LC_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded (%s); set LC_NCCL_LIB to its path", dlerror());
    g_nccl.GetUniqueId = (fn_GetUniqueId)dlsym(g_nccl.dl, "ncclGetUniqueId");
    g_nccl.CommInitRank = (fn_CommInitRank)dlsym(g_nccl.dl, "ncclCommInitRank");
    g_nccl.AllReduce = (fn_AllReduce)dlsym(g_nccl.dl, "ncclAllReduce");
    g_nccl.AllGather = (fn_AllGather)dlsym(g_nccl.dl, "ncclAllGather");
    g_nccl.CommDestroy = (fn_CommDestroy)dlsym(g_nccl.dl, "ncclCommDestroy");
    g_nccl.GetErrorString = (fn_GetErrorString)dlsym(g_nccl.dl, "ncclGetErrorString");
    LC_CHECK(g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.AllReduce && g_nccl.AllGather && g_nccl.CommDestroy, LC_ERR_UNSUPPORTED,
             "the NCCL library lacks an expected entry point");
    return LC_OK;
}

#define LC_NCCL(call)                                                                                         \
    do {                                                                                                      \
        int _r = (call);                                                                                      \
        if (_r != 0) {                                                                                        \
            set_error("%s failed: %s", #call, g_nccl.GetErrorString ? g_nccl.GetErrorString(_r) : "NCCL error"); \
            return LC_ERR_CUDA;                                                                               \
        }                                                                                                     \
    } while (0)

struct DistState {
    bool on = false;
    int rank = 0, world = 1, device = 0;
    NcclComm comm = nullptr;
    int want_peer = 1;
    // peer-memory path
    bool peer_ok = false;
    unsigned char* local = nullptr;     // [flags | slot 0 | slot 1 | keys 0 | keys 1]
    size_t slot_bytes = 0;
    unsigned char* peer[kMaxRanks] = {};
    unsigned* d_epoch = nullptr;        // sums taken so far (device side, so that a replayed graph keeps counting)
    unsigned* d_ticket = nullptr;
    float* plain_slot[2] = {nullptr, nullptr};  // NCCL only: ordinary device memory for the partial rows
};
DistState g_dist;

struct PeerParams {
    const unsigned char* peer[kMaxRanks];  // every rank's shared buffer as seen from here (own included)
    unsigned* flags;                       // own flag words
    unsigned* epoch;
    unsigned* ticket;
    int* error_flag;
    int rank, world;
    size_t src_off;                        // byte offset of the partial rows inside each buffer
};

__device__ __forceinline__ unsigned long long gtimer() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

// Step 1 and 2 of a sum: announce, then wait for every peer.  Returns false when the wait ran out (10 s).
__device__ __forceinline__ bool peer_barrier(const PeerParams& P, unsigned e) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (blockIdx.x == 0 && (int)threadIdx.x < P.world) {
        __threadfence_system();  // the rows the kernel ahead wrote are visible to the peers before the flag is
        unsigned* theirs = reinterpret_cast<unsigned*>(const_cast<unsigned char*>(P.peer[threadIdx.x])) + P.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(e) : "memory");
    }
    if ((int)threadIdx.x < P.world) {
        const unsigned long long t0 = gtimer();
        unsigned v = 0;
        bool ok = false;
        while (true) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(P.flags + threadIdx.x) : "memory");
            if ((int)(v - e) >= 0) { ok = true; break; }
            if (gtimer() - t0 > 10000000000ull) break;
        }
        if (!ok) s_ok = 0;
    }
    __syncthreads();
    return s_ok != 0;
}

__device__ __forceinline__ void peer_finish(const PeerParams& P, unsigned e, bool ok) {
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!ok && P.error_flag) atomicExch(P.error_flag, 3);
        const unsigned t = atomicAdd(P.ticket, 1u);
        if (t == gridDim.x - 1) {  // the last CTA of this sum: the next kernel on the stream sees the new count
            *P.ticket = 0;
            __threadfence();
            *P.epoch = e;
        }
    }
}

__global__ void __launch_bounds__(256) peer_sum_kernel(PeerParams P, float* __restrict__ dst, size_t count4) {
    const unsigned e = *P.epoch + 1;
    const bool ok = peer_barrier(P, e);
    if (ok) {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count4; i += (size_t)gridDim.x * blockDim.x) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < P.world; r++) {  // rank order: the same bits on every rank
                const float4* src = reinterpret_cast<const float4*>(P.peer[r] + P.src_off) + i;
                float4 v;
                asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(src) : "memory");
                acc.x = r ? acc.x + v.x : v.x; acc.y = r ? acc.y + v.y : v.y; acc.z = r ? acc.z + v.z : v.z; acc.w = r ? acc.w + v.w : v.w;
            }
            reinterpret_cast<float4*>(dst)[i] = acc;
        }
    }
    peer_finish(P, e, ok);
}

__global__ void __launch_bounds__(256) peer_max_kernel(PeerParams P, long long* __restrict__ dst, size_t count) {
    const unsigned e = *P.epoch + 1;
    const bool ok = peer_barrier(P, e);
    if (ok) {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
            long long best = 0;
            for (int r = 0; r < P.world; r++) {
                long long v;
                asm volatile("ld.relaxed.sys.global.s64 %0, [%1];" : "=l"(v) : "l"(reinterpret_cast<const long long*>(P.peer[r] + P.src_off) + i) : "memory");
                best = (r == 0 || v > best) ? v : best;
            }
            dst[i] = best;
        }
    }
    peer_finish(P, e, ok);
}

struct GroupPtrs { const void* src[kMaxRanks]; void* dst[kMaxRanks]; int n; };
__global__ void group_sum_kernel(GroupPtrs g, size_t count4) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count4; i += (size_t)gridDim.x * blockDim.x) {
        float4 acc = reinterpret_cast<const float4*>(g.src[0])[i];
        for (int r = 1; r < g.n; r++) {
            const float4 v = reinterpret_cast<const float4*>(g.src[r])[i];
            acc.x = acc.x + v.x; acc.y = acc.y + v.y; acc.z = acc.z + v.z; acc.w = acc.w + v.w;
        }
        for (int r = 0; r < g.n; r++) reinterpret_cast<float4*>(g.dst[r])[i] = acc;
    }
}
__global__ void group_max_kernel(GroupPtrs g, size_t count) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        long long best = reinterpret_cast<const long long*>(g.src[0])[i];
        for (int r = 1; r < g.n; r++) { const long long v = reinterpret_cast<const long long*>(g.src[r])[i]; best = v > best ? v : best; }
        for (int r = 0; r < g.n; r++) reinterpret_cast<long long*>(g.dst[r])[i] = best;
    }
}

PeerParams peer_params(size_t src_off) {
    PeerParams P{};
    for (int r = 0; r < g_dist.world; r++) P.peer[r] = g_dist.peer[r];
    P.flags = reinterpret_cast<unsigned*>(g_dist.local);
    P.epoch = g_dist.d_epoch; P.ticket = g_dist.d_ticket; P.error_flag = gemv_error_flag_dev();
    P.rank = g_dist.rank; P.world = g_dist.world; P.src_off = src_off;
    return P;
}

}  // namespace

bool dist_active() { return g_dist.on; }
int dist_rank() { return g_dist.on ? g_dist.rank : 0; }
int dist_world() { return g_dist.on ? g_dist.world : 1; }
bool dist_peer_memory() { return g_dist.on && g_dist.peer_ok; }

// Collective over the ranks: (re)creates the partial-row buffers so that each slot holds slot_bytes.
int32_t dist_reserve(size_t slot_bytes) {
    DistState& d = g_dist;
    LC_CHECK(d.on, LC_ERR_STATE, "lc_dist_init has not been called");
    slot_bytes = (slot_bytes + 255) & ~(size_t)255;
    if (slot_bytes <= d.slot_bytes) return LC_OK;
    cudaStream_t s = stream();
    LC_CUDA(cudaStreamSynchronize(s));
    for (int i = 0; i < 2; i++) { if (d.plain_slot[i]) cudaFree(d.plain_slot[i]); d.plain_slot[i] = nullptr; }
    const bool had_shared = d.local != nullptr;
    for (int r = 0; r < d.world; r++) { if (r != d.rank && d.peer[r]) cudaIpcCloseMemHandle(d.peer[r]); d.peer[r] = nullptr; }
    if (had_shared) {  // nobody frees a buffer that a peer may still have mapped: everyone closes, then everyone meets here
        long long* d_one = nullptr;
        LC_CUDA(cudaMalloc((void**)&d_one, 8));
        LC_CUDA(cudaMemsetAsync(d_one, 0, 8, s));
        LC_NCCL(g_nccl.AllReduce(d_one, d_one, 1, kNcclInt64, kNcclMax, d.comm, s));
        LC_CUDA(cudaStreamSynchronize(s));
        cudaFree(d_one);
    }
    if (d.local) { cudaFree(d.local); d.local = nullptr; }
    d.peer_ok = false;
    d.slot_bytes = slot_bytes;
    const size_t total = kFlagBytes + 2 * slot_bytes + 2 * kKeyBytes;
    int mine_ok = 0;
    cudaIpcMemHandle_t handle;
    memset(&handle, 0, sizeof(handle));
    if (d.want_peer && d.world <= kMaxRanks) {
        if (cudaMalloc((void**)&d.local, total) == cudaSuccess && cudaMemset(d.local, 0, total) == cudaSuccess &&
            cudaIpcGetMemHandle(&handle, d.local) == cudaSuccess)
            mine_ok = 1;
        (void)cudaGetLastError();
    }
    // every rank's handle and whether it has one
    struct Rec { cudaIpcMemHandle_t h; int ok; int pad[15]; };
    static_assert(sizeof(Rec) == 128, "record size");
    Rec mine; memset(&mine, 0, sizeof(mine)); mine.h = handle; mine.ok = mine_ok;
    Rec* d_recs = nullptr;
    LC_CUDA(cudaMalloc((void**)&d_recs, sizeof(Rec) * (d.world + 1)));
    LC_CUDA(cudaMemcpyAsync(d_recs + d.world, &mine, sizeof(Rec), cudaMemcpyHostToDevice, s));
    LC_NCCL(g_nccl.AllGather(d_recs + d.world, d_recs, sizeof(Rec), kNcclInt8, d.comm, s));
    std::vector<Rec> all(d.world);
    LC_CUDA(cudaMemcpyAsync(all.data(), d_recs, sizeof(Rec) * d.world, cudaMemcpyDeviceToHost, s));
    LC_CUDA(cudaStreamSynchronize(s));
    bool everyone = true;
    for (int r = 0; r < d.world; r++) everyone = everyone && all[r].ok;
    int opened = everyone ? 1 : 0;
    if (everyone) {
        for (int r = 0; r < d.world && opened; r++) {
            if (r == d.rank) { d.peer[r] = d.local; continue; }
            void* p = nullptr;
            if (cudaIpcOpenMemHandle(&p, all[r].h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { (void)cudaGetLastError(); opened = 0; break; }
            d.peer[r] = (unsigned char*)p;
        }
    }
    // all ranks must agree: the smallest of the `opened` words
    long long* d_flag = reinterpret_cast<long long*>(d_recs);
    long long v = opened;
    LC_CUDA(cudaMemcpyAsync(d_flag, &v, 8, cudaMemcpyHostToDevice, s));
    LC_NCCL(g_nccl.AllReduce(d_flag, d_flag, 1, kNcclInt64, 3 /* min */, d.comm, s));
    LC_CUDA(cudaMemcpyAsync(&v, d_flag, 8, cudaMemcpyDeviceToHost, s));
    LC_CUDA(cudaStreamSynchronize(s));
    cudaFree(d_recs);
    d.peer_ok = v == 1;
    if (!d.peer_ok) {
        for (int r = 0; r < d.world; r++) { if (r != d.rank && d.peer[r]) cudaIpcCloseMemHandle(d.peer[r]); d.peer[r] = nullptr; }
        if (d.local) { cudaFree(d.local); d.local = nullptr; }
        for (int i = 0; i < 2; i++) LC_CUDA(cudaMalloc((void**)&d.plain_slot[i], slot_bytes + kKeyBytes));
    }
    if (!d.d_epoch) {
        LC_CUDA(cudaMalloc((void**)&d.d_epoch, 8));
        LC_CUDA(cudaMemset(d.d_epoch, 0, 8));
        d.d_ticket = d.d_epoch + 1;
    }
    return LC_OK;
}

// Where a rank writes the partial rows of its next sum (i = 0, 1: consecutive sums alternate) / its greedy-pick keys.
float* dist_slot(int i) {
    DistState& d = g_dist;
    if (d.peer_ok) return reinterpret_cast<float*>(d.local + kFlagBytes + (size_t)(i & 1) * d.slot_bytes);
    return d.plain_slot[i & 1];
}
long long* dist_key_slot(int i) {
    DistState& d = g_dist;
    if (d.peer_ok) return reinterpret_cast<long long*>(d.local + kFlagBytes + 2 * d.slot_bytes + (size_t)(i & 1) * kKeyBytes);
    return reinterpret_cast<long long*>(reinterpret_cast<unsigned char*>(d.plain_slot[i & 1]) + d.slot_bytes);
}

// dst[0 .. count) = sum over the ranks of their slot `i` rows, rank order
int32_t dist_allreduce_sum(int i, float* dst, size_t count, cudaStream_t s) {
    DistState& d = g_dist;
    LC_CHECK(d.on && count * 4 <= d.slot_bytes && count % 4 == 0, LC_ERR_INVALID, "dist sum: %zu floats do not fit the reserved slot", count);
    if (d.peer_ok && count * 4 <= kPeerSumLimit) {
        PeerParams P = peer_params(kFlagBytes + (size_t)(i & 1) * d.slot_bytes);
        const unsigned grid = (unsigned)std::min<size_t>(32, (count / 4 + 255) / 256);
        peer_sum_kernel<<<grid, 256, 0, s>>>(P, dst, count / 4);
        LC_CUDA(cudaGetLastError());
        return LC_OK;
    }
    LC_NCCL(g_nccl.AllReduce(dist_slot(i), dst, count, kNcclFloat32, kNcclSum, d.comm, s));
    return LC_OK;
}

int32_t dist_allreduce_max(int i, long long* dst, size_t count, cudaStream_t s) {
    DistState& d = g_dist;
    LC_CHECK(d.on && count * 8 <= kKeyBytes, LC_ERR_INVALID, "dist max: %zu keys do not fit", count);
    if (d.peer_ok) {
        PeerParams P = peer_params(kFlagBytes + 2 * d.slot_bytes + (size_t)(i & 1) * kKeyBytes);
        peer_max_kernel<<<1, 256, 0, s>>>(P, dst, count);
        LC_CUDA(cudaGetLastError());
        return LC_OK;
    }
    LC_NCCL(g_nccl.AllReduce(dist_key_slot(i), dst, count, kNcclInt64, kNcclMax, d.comm, s));
    return LC_OK;
}

// dst = the ranks' `bytes`-byte pieces one after the other (rank order)
int32_t dist_allgather(const void* src, void* dst, size_t bytes, cudaStream_t s) {
    LC_CHECK(g_dist.on, LC_ERR_STATE, "lc_dist_init has not been called");
    LC_NCCL(g_nccl.AllGather(src, dst, bytes, kNcclInt8, g_dist.comm, s));
    return LC_OK;
}

int32_t launch_group_sum(const float* const* src, float* const* dst, int n, size_t count, cudaStream_t s) {
    LC_CHECK(n >= 1 && n <= kMaxRanks && count % 4 == 0, LC_ERR_INVALID, "group sum: %d ranks, %zu floats", n, count);
    GroupPtrs g{};
    g.n = n;
    for (int r = 0; r < n; r++) { g.src[r] = src[r]; g.dst[r] = dst[r]; }
    const unsigned grid = (unsigned)std::min<size_t>(64, (count / 4 + 255) / 256);
    group_sum_kernel<<<grid, 256, 0, s>>>(g, count / 4);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}
int32_t launch_group_max(const long long* const* src, long long* const* dst, int n, size_t count, cudaStream_t s) {
    LC_CHECK(n >= 1 && n <= kMaxRanks, LC_ERR_INVALID, "group max: %d ranks", n);
    GroupPtrs g{};
    g.n = n;
    for (int r = 0; r < n; r++) { g.src[r] = src[r]; g.dst[r] = dst[r]; }
    group_max_kernel<<<1, 256, 0, s>>>(g, count);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}

}  // namespace lc

using namespace lc;

extern "C" {

int32_t lc_dist_unique_id(void* out_id128) {
    LC_CHECK(out_id128, LC_ERR_INVALID, "lc_dist_unique_id: null output");
    LC_TRY(nccl_load());
    NcclId id;
    LC_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(out_id128, &id, sizeof(id));
    return LC_OK;
}

int32_t lc_dist_init(int32_t rank, int32_t world, const void* id128) {
    LC_CHECK(id128 && world >= 1 && rank >= 0 && rank < world, LC_ERR_INVALID, "lc_dist_init: rank %d of %d", rank, world);
    LC_CHECK(!g_dist.on, LC_ERR_STATE, "lc_dist_init was already called in this process");
    if (!have_device()) return LC_ERR_CUDA;
    LC_TRY(nccl_load());
    NcclId id;
    memcpy(&id, id128, sizeof(id));
    LC_CUDA(cudaGetDevice(&g_dist.device));
    LC_NCCL(g_nccl.CommInitRank(&g_dist.comm, world, id, rank));
    g_dist.rank = rank; g_dist.world = world; g_dist.on = true;
    if (const char* e = getenv("LC_DIST_PEER")) g_dist.want_peer = atoi(e) != 0;
    return LC_OK;
}

int32_t lc_dist_set_backend(int32_t peer_memory) {
    LC_CHECK(g_dist.slot_bytes == 0, LC_ERR_STATE, "lc_dist_set_backend must come before the first model is finalized");
    g_dist.want_peer = peer_memory ? 1 : 0;
    return LC_OK;
}

int32_t lc_dist_finalize(void) {
    DistState& d = g_dist;
    if (!d.on) return LC_OK;
    cudaStreamSynchronize(stream());
    for (int r = 0; r < d.world; r++) if (r != d.rank && d.peer[r]) cudaIpcCloseMemHandle(d.peer[r]);
    if (d.local) cudaFree(d.local);
    for (int i = 0; i < 2; i++) if (d.plain_slot[i]) cudaFree(d.plain_slot[i]);
    if (d.d_epoch) cudaFree(d.d_epoch);
    if (d.comm) g_nccl.CommDestroy(d.comm);
    d = DistState{};
    return LC_OK;
}

int32_t lc_dist_time_allreduce(size_t count, int32_t iters, float* out_us) {
    LC_CHECK(out_us && iters >= 1 && count >= 4 && count % 4 == 0, LC_ERR_INVALID, "lc_dist_time_allreduce: bad argument");
    LC_CHECK(g_dist.on, LC_ERR_STATE, "lc_dist_init has not been called");
    LC_TRY(dist_reserve(count * 4));
    cudaStream_t s = stream();
    float* dst = nullptr;
    LC_CUDA(cudaMalloc((void**)&dst, count * 4));
    for (int i = 0; i < 2; i++) LC_CUDA(cudaMemsetAsync(dist_slot(i), 0, count * 4, s));
    cudaEvent_t e0, e1;
    LC_CUDA(cudaEventCreate(&e0));
    LC_CUDA(cudaEventCreate(&e1));
    for (int i = 0; i < 4; i++) LC_TRY(dist_allreduce_sum(i, dst, count, s));
    LC_CUDA(cudaEventRecord(e0, s));
    for (int i = 0; i < iters; i++) LC_TRY(dist_allreduce_sum(i, dst, count, s));
    LC_CUDA(cudaEventRecord(e1, s));
    LC_CUDA(cudaEventSynchronize(e1));
    float ms = 0.f;
    LC_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    *out_us = ms * 1000.f / (float)iters;
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaFree(dst);
    int flag = 0;
    if (int* f = gemv_error_flag_dev()) { LC_CUDA(cudaMemcpy(&flag, f, 4, cudaMemcpyDeviceToHost)); if (flag) cudaMemset(f, 0, 4); }
    LC_CHECK(flag == 0, LC_ERR_CUDA, "a rank did not arrive at a sum within ten seconds");
    return LC_OK;
}

}  // extern "C"

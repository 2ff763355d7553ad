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
// Values per rank and sum on the peer-memory path (LC_DIST_LL_WORDS, a multiple of 1024); larger sums use NCCL.  Default 256 KiB of
// f32: there the tagged words still win (2 GPUs 9.2 against 10.7 us, 8 GPUs 20.1 against 27.4 us); at 512 KiB NCCL is ahead
// (12.6 against 11.7 us, 35.5 against 27.7 us): every rank writes its whole row, twice as wide, into every peer.
static int ll_words() {
    static const int v = [] {
        const char* e = getenv("LC_DIST_LL_WORDS");
        int w = e ? atoi(e) : 65536;
        if (w < 1024) w = 1024;
        if (w > (1 << 20)) w = 1 << 20;
        return w / 1024 * 1024;
    }();
    return v;
}
#define kLLWords (ll_words())

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
    bool setup_done = false;
    // peer-memory path
    bool peer_ok = false;
    unsigned long long* local = nullptr;    // [slot 2][source rank][kLLWords] tagged words
    unsigned long long* peer[kMaxRanks] = {};
    unsigned* d_epoch = nullptr;            // sums taken so far (device side, so that a replayed graph keeps counting)
    unsigned* d_ticket = nullptr;
};
DistState g_dist;

struct LLParams {
    unsigned long long* peer[kMaxRanks];   // every rank's buffer as seen from here (own included)
    unsigned* epoch;
    unsigned* ticket;
    int* error_flag;
    unsigned* debug;                       // 8 words written by the first wait that runs out: what it was waiting for
    unsigned long long timeout_ns;
    int rank, world;
    int row_words;                         // values per source rank in a slot
};

__device__ __forceinline__ unsigned long long gtimer() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ void st_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// One sum (or maximum of keys) over the ranks.  Every value travels as a 64-bit word: its 32 bits and, in the upper half,
// the number e of the sum it belongs to.  A rank WRITES its words into slot e & 1, row `rank`, of every rank's buffer
// (plain stores over NVLink, nothing waits for them), then polls its OWN buffer until row r of every rank r carries the
// tag e, and adds the rows in rank order.  An aligned 64-bit access is single-copy atomic, so a matching tag delivers
// the value: no flag, no fence.  push = 0: the producing kernel already wrote this rank's words (see GemvPush).
// KEYS: the values are 64-bit greedy-pick keys, sent as two words each; the result is their maximum.
template <bool KEYS>
__global__ void __launch_bounds__(256) peer_ll_kernel(LLParams P, const void* __restrict__ src, void* __restrict__ dst, size_t count, int push) {
    pdl_launch_dependents();
    // Everything ahead on the stream has finished: src is written, and the sum count is the one the previous sum left.  (A
    // gather-only launch must wait too: with small grids a whole chain of dependent kernels can be resident at once, and a
    // kernel that skipped the wait would read the count before the previous sum's kernel has moved it.)
    pdl_wait();
    const unsigned e = *P.epoch + 1; // stable for the whole kernel: only this kernel's last CTA moves it, after everyone read it
    const size_t row = (size_t)P.row_words, slot = (size_t)(e & 1u) * P.world * row;
    const size_t words = KEYS ? 2 * count : count;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
    if (push) {
        for (size_t w = tid; w < words; w += stride) {
            unsigned bits;
            if (KEYS) {
                const unsigned long long k = (unsigned long long)reinterpret_cast<const long long*>(src)[w >> 1];
                bits = (w & 1) ? (unsigned)k : (unsigned)(k >> 32);
            } else {
                bits = __float_as_uint(reinterpret_cast<const float*>(src)[w]);
            }
            const unsigned long long word = ((unsigned long long)e << 32) | bits;
            for (int r = 0; r < P.world; r++) st_sys_u64(P.peer[r] + slot + (size_t)P.rank * row + w, word);
        }
    }
    const unsigned long long* mine = P.peer[P.rank] + slot;
    bool ok = true;
    const unsigned long long t0 = gtimer();
    for (size_t i = tid; i < count; i += stride) {
        float acc = 0.f;
        long long best = 0;
        for (int r = 0; r < P.world; r++) {  // rank order: the same bits on every rank
            const unsigned long long* q = mine + (size_t)r * row + (KEYS ? 2 * i : i);
            unsigned long long a = 0, b = 0;
            for (unsigned spin = 0;; spin++) {
                a = ld_sys_u64(q);
                if (KEYS) b = ld_sys_u64(q + 1);
                if ((unsigned)(a >> 32) == e && (!KEYS || (unsigned)(b >> 32) == e)) break;
                if ((spin & 1023u) == 1023u && gtimer() - t0 > P.timeout_ns) {
                    ok = false;
                    if (P.debug && atomicCAS(P.debug, 0u, 1u) == 0u) {
                        P.debug[1] = e; P.debug[2] = (unsigned)r; P.debug[3] = (unsigned)i; P.debug[4] = (unsigned)(a >> 32);
                        P.debug[5] = (unsigned)push; P.debug[6] = KEYS ? 1u : 0u; P.debug[7] = (unsigned)count;
                    }
                    break;
                }
            }
            if (KEYS) {
                const long long k = (long long)((a << 32) | (b & 0xffffffffull));
                best = (r == 0 || k > best) ? k : best;
            } else {
                const float v = __uint_as_float((unsigned)a);
                acc = r ? acc + v : v;
            }
        }
        if (KEYS) reinterpret_cast<long long*>(dst)[i] = best;
        else reinterpret_cast<float*>(dst)[i] = acc;
    }
    if (!ok && P.error_flag) atomicExch(P.error_flag, 3);
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(P.ticket, 1u);
        if (t == gridDim.x - 1) {  // the last CTA: every CTA has read the count, the next kernel on the stream sees the new one
            *P.ticket = 0;
            __threadfence();
            *P.epoch = e;
        }
    }
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

LLParams ll_params() {
    LLParams P{};
    for (int r = 0; r < g_dist.world; r++) P.peer[r] = g_dist.peer[r];
    P.epoch = g_dist.d_epoch; P.ticket = g_dist.d_ticket; P.error_flag = gemv_error_flag_dev();
    P.debug = g_dist.d_epoch + 2;
    static const unsigned long long ms = getenv("LC_DIST_TIMEOUT_MS") ? strtoull(getenv("LC_DIST_TIMEOUT_MS"), nullptr, 10) : 10000ull;
    P.timeout_ns = ms * 1000000ull;
    P.rank = g_dist.rank; P.world = g_dist.world;
    P.row_words = kLLWords;
    return P;
}

template <bool KEYS>
int32_t launch_ll(const void* src, void* dst, size_t count, int push, cudaStream_t s) {
    LLParams P = ll_params();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)std::min<size_t>(64, (count + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    LC_CUDA(cudaLaunchKernelEx(&cfg, peer_ll_kernel<KEYS>, P, src, dst, count, push));
    return LC_OK;
}

}  // namespace

bool dist_active() { return g_dist.on; }
int dist_rank() { return g_dist.on ? g_dist.rank : 0; }
int dist_world() { return g_dist.on ? g_dist.world : 1; }
bool dist_peer_memory() { return g_dist.on && g_dist.peer_ok; }
size_t dist_peer_capacity() { return dist_peer_memory() ? (size_t)kLLWords : 0; }

// Collective over the ranks, once: the buffer of tagged words, mapped into every peer (or the agreement that it cannot be).
int32_t dist_setup() {
    DistState& d = g_dist;
    LC_CHECK(d.on, LC_ERR_STATE, "lc_dist_init has not been called");
    if (d.setup_done) return LC_OK;
    cudaStream_t s = stream();
    LC_CUDA(cudaStreamSynchronize(s));
    const size_t total = (size_t)2 * d.world * kLLWords * sizeof(unsigned long long);
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
            d.peer[r] = (unsigned long long*)p;
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
        // everyone has closed what it opened before anyone frees (the all-reduce above is behind us; one more meeting point)
        LC_CUDA(cudaMalloc((void**)&d_flag, 8));
        LC_CUDA(cudaMemsetAsync(d_flag, 0, 8, s));
        LC_NCCL(g_nccl.AllReduce(d_flag, d_flag, 1, kNcclInt64, kNcclMax, d.comm, s));
        LC_CUDA(cudaStreamSynchronize(s));
        cudaFree(d_flag);
        if (d.local) { cudaFree(d.local); d.local = nullptr; }
    }
    LC_CUDA(cudaMalloc((void**)&d.d_epoch, 40));   // sum count, ticket, 8 words of diagnostics
    LC_CUDA(cudaMemset(d.d_epoch, 0, 40));
    d.d_ticket = d.d_epoch + 1;
    d.setup_done = true;
    return LC_OK;
}

// dst[0 .. count) = sum over the ranks of their src rows, rank order.  src and dst are this rank's ordinary device memory.
int32_t dist_allreduce_sum(const float* src, float* dst, size_t count, cudaStream_t s) {
    DistState& d = g_dist;
    LC_CHECK(d.on && d.setup_done, LC_ERR_STATE, "dist sum before lc_dist_init / the model's finalize");
    if (d.peer_ok && count <= (size_t)kLLWords) return launch_ll<false>(src, dst, count, 1, s);
    LC_NCCL(g_nccl.AllReduce(src, dst, count, kNcclFloat32, kNcclSum, d.comm, s));
    return LC_OK;
}
// The second half of such a sum when the kernel that produced the rows already wrote this rank's tagged words to every rank.
int32_t dist_gather_sum(float* dst, size_t count, cudaStream_t s) {
    DistState& d = g_dist;
    LC_CHECK(d.on && d.peer_ok && count <= (size_t)kLLWords, LC_ERR_STATE, "dist gather: the peer-memory path is not set up for %zu values", count);
    return launch_ll<false>(nullptr, dst, count, 0, s);
}
// What a producing kernel needs to write its output rows as tagged words of the NEXT sum into every rank's buffer.
bool dist_push_desc(size_t count, GemvPush* out) {
    DistState& d = g_dist;
    if (!d.on || !d.peer_ok || count > (size_t)kLLWords) return false;
    for (int r = 0; r < kMaxRanks; r++) out->peer[r] = r < d.world ? d.peer[r] : nullptr;
    out->epoch = d.d_epoch; out->world = d.world; out->rank = d.rank; out->row_words = kLLWords;
    return true;
}

int32_t dist_allreduce_max(const long long* src, long long* dst, size_t count, cudaStream_t s) {
    DistState& d = g_dist;
    LC_CHECK(d.on && d.setup_done, LC_ERR_STATE, "dist max before lc_dist_init / the model's finalize");
    if (d.peer_ok && 2 * count <= (size_t)kLLWords) return launch_ll<true>(src, dst, count, 1, s);
    LC_NCCL(g_nccl.AllReduce(src, dst, count, kNcclInt64, kNcclMax, d.comm, s));
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
    LC_CHECK(!g_dist.setup_done, LC_ERR_STATE, "lc_dist_set_backend must come before the first model is finalized");
    g_dist.want_peer = peer_memory ? 1 : 0;
    return LC_OK;
}

int32_t lc_dist_info(int32_t* rank, int32_t* world, int32_t* peer_memory) {
    if (rank) *rank = dist_rank();
    if (world) *world = dist_world();
    if (peer_memory) *peer_memory = dist_peer_memory() ? 1 : 0;
    return LC_OK;
}

// Diagnostics: the record left by the first wait of a sum that ran out ([0] != 0 when there is one): sum number, the rank
// whose word was missing, the word index, the tag found there, whether the kernel also sent, whether it was a key maximum,
// the number of values.  Reading clears it.
int32_t lc_dist_debug(uint32_t* out8) {
    LC_CHECK(out8, LC_ERR_INVALID, "null output");
    memset(out8, 0, 32);
    if (!g_dist.on || !g_dist.d_epoch) return LC_OK;
    LC_CUDA(cudaMemcpy(out8, g_dist.d_epoch + 2, 32, cudaMemcpyDeviceToHost));
    LC_CUDA(cudaMemset(g_dist.d_epoch + 2, 0, 32));
    return LC_OK;
}

int32_t lc_dist_finalize(void) {
    DistState& d = g_dist;
    if (!d.on) return LC_OK;
    cudaStreamSynchronize(stream());
    for (int r = 0; r < d.world; r++) if (r != d.rank && d.peer[r]) cudaIpcCloseMemHandle(d.peer[r]);
    if (d.comm && d.local) {  // nobody frees a buffer that a peer may still have mapped: everyone closes, then everyone meets
        long long* one = nullptr;
        if (cudaMalloc((void**)&one, 8) == cudaSuccess) {
            cudaMemsetAsync(one, 0, 8, stream());
            g_nccl.AllReduce(one, one, 1, kNcclInt64, kNcclMax, d.comm, stream());
            cudaStreamSynchronize(stream());
            cudaFree(one);
        }
    }
    if (d.local) cudaFree(d.local);
    if (d.d_epoch) cudaFree(d.d_epoch);
    if (d.comm) g_nccl.CommDestroy(d.comm);
    d = DistState{};
    return LC_OK;
}

int32_t lc_dist_time_allreduce(size_t count, int32_t iters, float* out_us) {
    LC_CHECK(out_us && iters >= 1 && count >= 4 && count % 4 == 0, LC_ERR_INVALID, "lc_dist_time_allreduce: bad argument");
    LC_CHECK(g_dist.on, LC_ERR_STATE, "lc_dist_init has not been called");
    LC_TRY(dist_setup());
    cudaStream_t s = stream();
    float *src = nullptr, *dst = nullptr;
    LC_CUDA(cudaMalloc((void**)&src, count * 4));
    LC_CUDA(cudaMalloc((void**)&dst, count * 4));
    LC_CUDA(cudaMemsetAsync(src, 0, count * 4, s));
    cudaEvent_t e0, e1;
    LC_CUDA(cudaEventCreate(&e0));
    LC_CUDA(cudaEventCreate(&e1));
    for (int i = 0; i < 4; i++) LC_TRY(dist_allreduce_sum(src, dst, count, s));
    LC_CUDA(cudaEventRecord(e0, s));
    for (int i = 0; i < iters; i++) LC_TRY(dist_allreduce_sum(src, dst, count, s));
    LC_CUDA(cudaEventRecord(e1, s));
    LC_CUDA(cudaEventSynchronize(e1));
    float ms = 0.f;
    LC_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    *out_us = ms * 1000.f / (float)iters;
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaFree(src); cudaFree(dst);
    int flag = 0;
    if (int* f = gemv_error_flag_dev()) { LC_CUDA(cudaMemcpy(&flag, f, 4, cudaMemcpyDeviceToHost)); if (flag) cudaMemset(f, 0, 4); }
    LC_CHECK(flag == 0, LC_ERR_CUDA, "a rank did not arrive at a sum within ten seconds");
    return LC_OK;
}

}  // extern "C"

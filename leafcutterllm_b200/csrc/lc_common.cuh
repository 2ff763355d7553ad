// Shared host/device helpers of the library: status + error text, the
// per-device stream, checked CUDA calls, warp reductions, f16 conversions.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>
#include <string>
#include "../../include/leafcutter_b200.h"

namespace lc {

void set_error(const char* fmt, ...);
const char* get_error();

// One compute stream per device, created on first use.
cudaStream_t stream();
// Number of SMs of the current device (cached).
int sm_count();
// True when a CUDA device is usable; sets the error text otherwise.
bool have_device();

#define LC_CUDA(call)                                                                       \
    do {                                                                                    \
        cudaError_t _e = (call);                                                            \
        if (_e != cudaSuccess) {                                                            \
            lc::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return LC_ERR_CUDA;                                                             \
        }                                                                                   \
    } while (0)

#define LC_CHECK(cond, code, ...)                                                           \
    do {                                                                                    \
        if (!(cond)) {                                                                      \
            lc::set_error(__VA_ARGS__);                                                     \
            return (code);                                                                  \
        }                                                                                   \
    } while (0)

#define LC_TRY(expr)                                                                        \
    do {                                                                                    \
        int32_t _s = (expr);                                                                \
        if (_s != LC_OK) return _s;                                                         \
    } while (0)

// Geometry of a ggml block type (rust/src/model/quant.rs:186-262).
struct QuantGeom { uint32_t block_elems, block_bytes; };
bool quant_geom(uint32_t typ, QuantGeom* g);

// Device scratch that grows on demand and is reused (per device, not thread-safe:
// L1 calls are serialised by a mutex in capi).
struct DevBuf {
    void* p = nullptr;
    size_t cap = 0;
    int32_t reserve(size_t bytes);
    void release();
};

#ifdef __CUDACC__
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide sum in a fixed order (deterministic): warp shuffles, then warp 0 over the per-warp sums.
__device__ __forceinline__ float block_sum(float v, float* sh) {
    v = warp_sum(v);
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float r = (threadIdx.x < nw) ? sh[threadIdx.x] : 0.0f;
    if (w == 0) r = warp_sum(r);
    if (threadIdx.x == 0) sh[0] = r;
    __syncthreads();
    return sh[0];
}
__device__ __forceinline__ float block_max(float v, float* sh) {
    v = warp_max(v);
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float r = (threadIdx.x < nw) ? sh[threadIdx.x] : -INFINITY;
    if (w == 0) r = warp_max(r);
    if (threadIdx.x == 0) sh[0] = r;
    __syncthreads();
    return sh[0];
}

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t f2h(float f) { return __half_as_ushort(__float2half_rn(f)); }

// Activations that carry their own validity: one 64-bit word per element, f32 bits in the low half and the epoch of
// the write in the high half.  A consumer that sees the expected epoch sees the value (a naturally aligned 64-bit
// access is single-copy atomic), so a kernel can start on its input the moment the producing CTAs have written it,
// without waiting for the whole producing grid to drain.  Epochs never repeat, so stale words never match, and nothing
// ever has to be cleared.  No fences are involved: every word validates itself, and a buffer is only overwritten by a
// kernel whose own input depends -- through chains of load -> compute -> store -- on every read of the old contents.
__device__ __forceinline__ void flag_store(unsigned long long* p, float v, uint32_t epoch) {
    const unsigned long long w = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
// N (even) consecutive flagged words, polled as a batch until every epoch matches; false when the bounded poll runs out.
template <int N>
__device__ __forceinline__ bool flag_load(const unsigned long long* p, uint32_t epoch, float (&v)[N]) {
    static_assert(N % 2 == 0, "pairs of words");
    unsigned long long w[N];
    bool all = false;
    for (uint32_t it = 0; it < (1u << 20) && !all; ++it) {
#pragma unroll
        for (int i = 0; i < N; i += 2)
            asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(w[i]), "=l"(w[i + 1]) : "l"(p + i) : "memory");
        all = true;
#pragma unroll
        for (int i = 0; i < N; i++) all = all && (uint32_t)(w[i] >> 32) == epoch;
    }
#pragma unroll
    for (int i = 0; i < N; i++) v[i] = __uint_as_float((uint32_t)w[i]);
    return all;
}
// N words `stride` elements apart (word i at p + i * stride; indices >= limit are skipped and read as 0)
template <int N>
__device__ __forceinline__ bool flag_load_strided(const unsigned long long* p, int stride, int limit, uint32_t epoch, float (&v)[N]) {
    unsigned long long w[N];
    bool all = false;
    for (uint32_t it = 0; it < (1u << 20) && !all; ++it) {
#pragma unroll
        for (int i = 0; i < N; i++)
            if (i * stride < limit) asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w[i]) : "l"(p + (size_t)i * stride) : "memory");
        all = true;
#pragma unroll
        for (int i = 0; i < N; i++) all = all && (i * stride >= limit || (uint32_t)(w[i] >> 32) == epoch);
    }
#pragma unroll
    for (int i = 0; i < N; i++) v[i] = (i * stride < limit) ? __uint_as_float((uint32_t)w[i]) : 0.f;
    return all;
}
// A warp waits for 256 consecutive words by watching eight of them (the last of every 32: producers write 32 rows per
// tile), so that a kernel whose input is still being produced does not sweep its whole input through L2 over and over
// while the producers need that bandwidth for their weights.  The caller still fetches with flag_load afterwards.
__device__ __forceinline__ bool flag_watch_unit(const unsigned long long* unit_base, uint32_t epoch) {
    const int lane = threadIdx.x & 31;
    bool all = false;
    for (uint32_t it = 0; it < (1u << 20) && !all; ++it) {
        bool mine = true;
        if (lane < 8) {
            unsigned long long w;
            asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(unit_base + 32 * lane + 31) : "memory");
            mine = (uint32_t)(w >> 32) == epoch;
        }
        all = __all_sync(0xffffffffu, mine);
    }
    return all;
}
// the value of a word known to be complete
__device__ __forceinline__ float flag_value(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return __uint_as_float((uint32_t)w);
}

// Programmatic dependent launch: let the next kernel in the stream start its
// prologue now / wait until the previous kernel's memory is visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Ask the L2 cache to fetch part `part` of `nparts` of [base, base + bytes) from HBM (both 16-byte aligned).  Used by a
// kernel to pull the weights of the kernel that follows it into L2 while its own, latency-bound, work runs: the
// caller is one thread; nothing waits for the fetch and nothing is written.
__device__ __forceinline__ void l2_prefetch_part(const void* base, unsigned long long bytes, unsigned part, unsigned nparts) {
    if (base == nullptr || bytes == 0) return;
    const unsigned long long per = ((bytes + nparts - 1) / nparts + 15ull) & ~15ull;
    const unsigned long long beg = per * part;
    if (beg >= bytes) return;
    unsigned long long len = bytes - beg;
    if (len > per) len = per;
    len &= ~15ull;
    const char* a = reinterpret_cast<const char*>(base) + beg;
    for (unsigned long long off = 0; off < len; off += 16384ull) {
        const unsigned sz = (unsigned)((len - off) < 16384ull ? (len - off) : 16384ull);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a + off), "r"(sz) : "memory");
    }
}
#endif

}  // namespace lc

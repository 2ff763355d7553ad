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
// Raises a kernel's dynamic shared-memory limit once per (device, kernel): the attribute belongs to the device's copy
// of the function, so a process that drives several devices has to set it on each of them.
cudaError_t ensure_smem_limit(const void* kern, size_t bytes);

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

// Programmatic dependent launch: let the next kernel in the stream start its
// prologue now / wait until the previous kernel's memory is visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#endif

}  // namespace lc

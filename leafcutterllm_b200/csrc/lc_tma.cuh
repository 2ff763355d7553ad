// Device helpers shared by the TMA-staged GEMV kernels: mbarrier transactions with bounded waits,
// the 2-D tensor-map load, the kernel parameter block.
#pragma once
#include <cuda.h>
#include "lc_kernels.h"

namespace lc {

constexpr int kTileRows = 32;    // rows of W per TMA box (lane <-> row, or two 16-row MMA groups)
constexpr int kUnitElems = 256;  // elements of k per box

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: returns false when the phase did not complete within the spin budget.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// one probe of a phase: true when it has completed
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const void* tmap, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            smem_u32(dst)),
        "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const void* tmap, int x, int y, int z, int w, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
            smem_u32(dst)),
        "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar))
        : "memory");
}

// cpu.rs:62-64
__device__ __forceinline__ float silu_f(float v) { return v * (1.0f / (1.0f + expf(-v))); }

struct GemvParams {
    const float* x;         // [m, k]
    float* out;             // [m, n]
    const float* residual;  // or null
    const float* norm_w;    // or null
    float eps;
    int n, k, m;
    int epi;
    int* error_flag;
    GemvPush push;          // world > 0: the output rows leave as tagged words (see GemvPush)
    unsigned long long* ring = nullptr;  // diagnostics (LC_GEMV_RING): 8 wall-clock words of this launch, or null
};
// Expert grouping of one launch (device pointers; see GemvGroup): all zero for a plain product.
struct GemvGroupParams {
    const CUtensorMap* tm0;
    const CUtensorMap* tm1;
    const int32_t* cnt;
    const int32_t* list;
    const unsigned char* planes;  // [row][unit][8 sub-blocks][3 planes][32] fixed-point activations (GemvPlanes)
    const float* sxf;             // [row][unit][8]
    const float* inv2s;           // [row][unit]
    int list_stride, top_k, x_by_token;
};

// Launch with the programmatic-dependent-launch attribute (off when LC_NO_PDL is set).
bool pdl_enabled();
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

int* gemv_error_flag_dev();
constexpr size_t kMaxSmem = 227 * 1024;

// qgemv_mma.cu: Q4_K through int8 tensor-core MMAs; *launched = false when the shape does not fit.
int32_t launch_qgemv_mma_q4k(const GemvArgs& a, cudaStream_t s, bool* launched);
int32_t launch_qgemv_mma_q4k_grouped(const GemvArgs& a, cudaStream_t s, bool* launched);
// true when the single-token kernel fits shared memory for rows of k elements
bool qgemv_mma_supports(int k);
// qgemv_mma_q6k.cu: Q6_K through int8 tensor-core MMAs, up to four tokens; *launched = false when the shape does not fit.
int32_t launch_qgemv_mma_q6k(const GemvArgs& a, cudaStream_t s, bool* launched);
bool qgemv_mma_q6k_supports(const GemvArgs& a, int m);
// true when the Q5_K form of the tensor-core matrix-vector kernel fits shared memory for four tokens of k elements
bool qgemv_mma_q5k_supports4(int k);
// qgemv_kq.cu: Q5_K, Q6_K, F16 and F32, up to eight tokens, plain loads; *launched = false for other types or shapes.
int32_t launch_qgemv_kq(const GemvArgs& a, cudaStream_t s, bool* launched);

}  // namespace lc

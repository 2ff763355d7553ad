// Block dequantisation kernels (bit-exact with rust/src/kernels/mod.rs), the
// load-time weight sanity scan and the embedding row gather.
#include "lc_kernels.h"
#include "lc_quant.cuh"
#include "lc_tma.cuh"

namespace lc {

__global__ void dequant_kernel(uint32_t typ, const uint8_t* __restrict__ w, size_t n, float* __restrict__ out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = dequant_elem(typ, w, i);
}

__global__ void sanity_kernel(uint32_t typ, const uint8_t* __restrict__ w, size_t n, unsigned long long* count) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    unsigned int bad = 0;
    for (; i < n; i += stride) {
        float v = dequant_elem(typ, w, i);
        if (isnan(v) || isinf(v) || fabsf(v) > 100.0f) bad++;
    }
    for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xffffffffu, bad, o);
    if ((threadIdx.x & 31) == 0 && bad) atomicAdd(count, (unsigned long long)bad);
}

__global__ void __launch_bounds__(1024) embed_kernel(uint32_t typ, const uint8_t* __restrict__ w, size_t rows, size_t cols,
                                                     const int64_t* __restrict__ ids, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();  // the token ids may come from the kernel ahead (a decode step's advance), and `out` may still be read by it
    int t = blockIdx.x;
    int64_t id = ids[t];
    bool ok = id >= 0 && (size_t)id < rows;
    for (size_t c = threadIdx.x; c < cols; c += blockDim.x)
        out[(size_t)t * cols + c] = ok ? dequant_elem(typ, w, (size_t)id * cols + c) : 0.0f;
}

static int grid_for(size_t n, int block) {
    size_t g = (n + block - 1) / block;
    size_t cap = (size_t)sm_count() * 16;
    return (int)(g < cap ? (g ? g : 1) : cap);
}

int32_t launch_dequant(uint32_t typ, const void* w, size_t n, float* out, cudaStream_t s) {
    QuantGeom g;
    LC_CHECK(quant_geom(typ, &g), LC_ERR_UNSUPPORTED, "dequantize: unsupported ggml type %u", typ);
    if (n == 0) return LC_OK;
    dequant_kernel<<<grid_for(n, 256), 256, 0, s>>>(typ, (const uint8_t*)w, n, out);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}

int32_t launch_sanity_scan(uint32_t typ, const void* w, size_t n, unsigned long long* count, cudaStream_t s) {
    QuantGeom g;
    LC_CHECK(quant_geom(typ, &g), LC_ERR_UNSUPPORTED, "sanity scan: unsupported ggml type %u", typ);
    if (n == 0) return LC_OK;
    sanity_kernel<<<grid_for(n, 256), 256, 0, s>>>(typ, (const uint8_t*)w, n, count);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}

int32_t launch_embed(uint32_t typ, const void* w, size_t rows, size_t cols, const int64_t* ids, int n, float* out,
                     cudaStream_t s) {
    if (n <= 0) return LC_OK;
    // a row is a few thousand elements, each decoded on its own: many threads, a few elements each
    LC_CUDA(launch_pdl(embed_kernel, dim3((unsigned)n), dim3(cols >= 2048 ? 1024 : 256), 0, s, typ, (const uint8_t*)w, rows, cols, ids, out));
    return LC_OK;
}

}  // namespace lc

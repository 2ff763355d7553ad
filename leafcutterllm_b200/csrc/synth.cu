// Synthetic tensor generation on the host and on the device from the single
// source in lc_synth.h (identical bytes on both sides).
#include <vector>
#include <thread>
#include "lc_kernels.h"
#include "lc_synth.h"

namespace lc {

static bool synth_has_quantiser(uint32_t typ) {
    return typ == LC_TYPE_F32 || typ == LC_TYPE_F16 || typ == LC_TYPE_Q4_0 || typ == LC_TYPE_Q8_0 || typ == LC_TYPE_Q4_K || typ == LC_TYPE_Q5_K ||
           typ == LC_TYPE_Q6_K;
}

__global__ void synth_kernel(uint32_t typ, uint64_t seed, uint64_t name_hash, float sigma, size_t n_blocks,
                             uint32_t block_bytes, uint8_t* out) {
    size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; b < n_blocks; b += stride) lcs_synth_block(typ, seed, name_hash, sigma, b, out + b * block_bytes);
}

__global__ void synth_part_kernel(uint32_t typ, uint64_t seed, uint64_t name_hash, float sigma, size_t row_blocks, size_t row0, size_t rows,
                                  size_t blk0, size_t blks, uint32_t block_bytes, uint8_t* out) {
    const size_t total = rows * blks;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const size_t r = i / blks, c = i - r * blks;
        lcs_synth_block(typ, seed, name_hash, sigma, (row0 + r) * row_blocks + blk0 + c, out + i * block_bytes);
    }
}

int32_t launch_synth_part(uint32_t typ, uint64_t seed, uint64_t name_hash, float sigma, size_t row_blocks, size_t row0, size_t rows,
                          size_t blk0, size_t blks, void* out_dev, cudaStream_t s) {
    QuantGeom g;
    LC_CHECK(quant_geom(typ, &g), LC_ERR_UNSUPPORTED, "synth: unsupported ggml type %u", typ);
    LC_CHECK(synth_has_quantiser(typ),
             LC_ERR_UNSUPPORTED, "synth: no quantiser for ggml type %u", typ);
    LC_CHECK(blk0 + blks <= row_blocks, LC_ERR_INVALID, "synth: blocks %zu..%zu outside a row of %zu", blk0, blk0 + blks, row_blocks);
    const size_t total = rows * blks;
    if (total == 0) return LC_OK;
    size_t grid = (total + 63) / 64;
    const size_t cap = (size_t)sm_count() * 32;
    if (grid > cap) grid = cap;
    synth_part_kernel<<<(unsigned)grid, 64, 0, s>>>(typ, seed, name_hash, sigma, row_blocks, row0, rows, blk0, blks, g.block_bytes, (uint8_t*)out_dev);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}

int32_t launch_synth(uint32_t typ, uint64_t seed, uint64_t name_hash, float sigma, size_t n_elems, void* out_dev,
                     cudaStream_t s) {
    QuantGeom g;
    LC_CHECK(quant_geom(typ, &g), LC_ERR_UNSUPPORTED, "synth: unsupported ggml type %u", typ);
    LC_CHECK(synth_has_quantiser(typ),
             LC_ERR_UNSUPPORTED, "synth: no quantiser for ggml type %u", typ);
    LC_CHECK(n_elems % g.block_elems == 0, LC_ERR_INVALID, "synth: %zu elements is not a whole number of blocks", n_elems);
    size_t nb = n_elems / g.block_elems;
    if (nb == 0) return LC_OK;
    size_t grid = (nb + 63) / 64;
    size_t cap = (size_t)sm_count() * 32;
    if (grid > cap) grid = cap;
    synth_kernel<<<(unsigned)grid, 64, 0, s>>>(typ, seed, name_hash, sigma, nb, g.block_bytes, (uint8_t*)out_dev);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}

}  // namespace lc

using namespace lc;

extern "C" {

int32_t lc_synth_tensor_host(uint32_t typ, uint64_t seed, const char* name, float sigma, size_t n_elems, void* out_bytes) {
    QuantGeom g;
    LC_CHECK(name && out_bytes, LC_ERR_INVALID, "lc_synth_tensor_host: null argument");
    LC_CHECK(quant_geom(typ, &g), LC_ERR_UNSUPPORTED, "synth: unsupported ggml type %u", typ);
    LC_CHECK(synth_has_quantiser(typ),
             LC_ERR_UNSUPPORTED, "synth: no quantiser for ggml type %u", typ);
    LC_CHECK(n_elems % g.block_elems == 0, LC_ERR_INVALID, "synth: %zu elements is not a whole number of blocks", n_elems);
    size_t nb = n_elems / g.block_elems;
    uint64_t h = lcs_fnv1a(name);
    unsigned nt = std::thread::hardware_concurrency();
    if (nt == 0) nt = 1;
    if (nt > 64) nt = 64;
    if (nb < 4096) nt = 1;
    std::vector<std::thread> th;
    uint8_t* out = (uint8_t*)out_bytes;
    for (unsigned t = 0; t < nt; t++) {
        size_t b0 = nb * t / nt, b1 = nb * (t + 1) / nt;
        th.emplace_back([=]() {
            for (size_t b = b0; b < b1; b++) lcs_synth_block(typ, seed, h, sigma, b, out + b * g.block_bytes);
        });
    }
    for (auto& t : th) t.join();
    return LC_OK;
}

int32_t lc_synth_tensor_dev(uint32_t typ, uint64_t seed, const char* name, float sigma, size_t n_elems, void* out_dev) {
    LC_CHECK(name && out_dev, LC_ERR_INVALID, "lc_synth_tensor_dev: null argument");
    if (!have_device()) return LC_ERR_CUDA;
    LC_TRY(launch_synth(typ, seed, lcs_fnv1a(name), sigma, n_elems, out_dev, stream()));
    LC_CUDA(cudaStreamSynchronize(stream()));
    return LC_OK;
}

int32_t lc_synth_tokens(uint64_t seed, size_t n, int64_t vocab, int64_t* out) {
    LC_CHECK(out && vocab > 0, LC_ERR_INVALID, "lc_synth_tokens: bad argument");
    for (size_t i = 0; i < n; i++) out[i] = (int64_t)lcs_uniform_int(seed, i, (uint64_t)vocab);
    return LC_OK;
}

}  // extern "C"

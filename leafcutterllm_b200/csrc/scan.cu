// Block-scale scan of raw quantised tensors: the per-tensor body of scan_for_corruption
// (rust/src/model/loader.rs:301-422).  A block is bad when its scale -- or what the reference reads as its second
// scale -- is NaN, infinite or larger than 1e4 in magnitude.  The reference's reading rules are kept as they are,
// including the ones that do not match the ggml layouts: every type except Q6_K, Q8_K and Q8_1 is read as "f16 at
// byte 0, f16 at byte 2 when the block has 4 bytes" (loader.rs:366-381), so for Q4_0 / Q8_0 / IQ4_NL the second
// half-word is quantised data and for Q2_K / Q3_K the first one is.
//
// One thread per block, 2 - 8 header bytes out of 18 - 292: the kernel touches one 32-byte sector per block.
#include <mutex>
#include "lc_kernels.h"

namespace lc {

namespace {

enum ScanKind : int { SCAN_HALF_PAIR = 0, SCAN_Q6_K = 1, SCAN_Q8_K = 2, SCAN_Q8_1 = 3 };

__device__ __forceinline__ bool bad_scale(float v) { return isnan(v) || isinf(v) || fabsf(v) > 1e4f; }  // loader.rs:385-392
__device__ __forceinline__ float half_at(const uint8_t* p) {
    return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}
__device__ __forceinline__ float float_at(const uint8_t* p) {
    return __uint_as_float((uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24));
}

__global__ void __launch_bounds__(256) scan_scales_kernel(const uint8_t* __restrict__ raw, size_t n_blocks, uint32_t block_bytes, int kind,
                                                           unsigned long long* __restrict__ bad_out) {
    unsigned int bad = 0;
    for (size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks; b += (size_t)gridDim.x * blockDim.x) {
        const uint8_t* p = raw + b * block_bytes;
        bool is_bad;
        if (kind == SCAN_Q6_K) {
            is_bad = bad_scale(half_at(p + 208));                               // loader.rs:341-349
        } else if (kind == SCAN_Q8_K) {
            is_bad = bad_scale(float_at(p));                                    // loader.rs:350-357
        } else if (kind == SCAN_Q8_1) {
            is_bad = bad_scale(float_at(p)) || bad_scale(float_at(p + 4));      // loader.rs:358-367
        } else {
            is_bad = bad_scale(half_at(p));                                     // loader.rs:368-381
            if (block_bytes >= 4) is_bad = is_bad || bad_scale(half_at(p + 2));
        }
        bad += is_bad ? 1u : 0u;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xffffffffu, bad, o);
    if ((threadIdx.x & 31) == 0 && bad) atomicAdd(bad_out, (unsigned long long)bad);
}

}  // namespace

// Block geometry of every type code QuantType::from_u32 knows (rust/src/model/quant.rs:71-100,160-238) and how the scan
// reads its scales.  False for F32 / F16 / BF16 and unknown codes: nothing to scan (loader.rs:309-322).
bool scan_geom(uint32_t typ, uint32_t* block_elems, uint32_t* block_bytes, int* kind) {
    uint32_t e = 0, b = 0;
    int k = SCAN_HALF_PAIR;
    switch (typ) {
        case 2: e = 32; b = 18; break;                     // Q4_0
        case 3: e = 32; b = 20; break;                     // Q4_1
        case 6: e = 32; b = 22; break;                     // Q5_0
        case 7: e = 32; b = 24; break;                     // Q5_1
        case 8: e = 32; b = 34; break;                     // Q8_0
        case 9: e = 32; b = 36; k = SCAN_Q8_1; break;      // Q8_1
        case 10: e = 256; b = 84; break;                   // Q2_K
        case 11: e = 256; b = 110; break;                  // Q3_K
        case 12: e = 256; b = 144; break;                  // Q4_K
        case 13: e = 256; b = 176; break;                  // Q5_K
        case 14: e = 256; b = 210; k = SCAN_Q6_K; break;   // Q6_K
        case 15: e = 256; b = 292; k = SCAN_Q8_K; break;   // Q8_K
        case 16: e = 256; b = 66; break;                   // IQ2_XXS
        case 17: e = 256; b = 74; break;                   // IQ2_XS
        case 18: e = 256; b = 98; break;                   // IQ3_XXS
        case 19: e = 256; b = 110; break;                  // IQ3_S
        case 20: e = 32; b = 18; break;                    // IQ4_NL
        case 21: e = 256; b = 136; break;                  // IQ4_XS
        case 22: e = 256; b = 136; break;                  // IQ4_K
        case 23: e = 256; b = 162; break;                  // IQ5_0
        case 24: e = 256; b = 162; break;                  // IQ5_NL
        case 25: e = 256; b = 176; break;                  // IQ5_K
        default: return false;
    }
    *block_elems = e;
    *block_bytes = b;
    *kind = k;
    return true;
}

// counter_dev: one zeroed 64-bit word on the device; the launch adds the tensor's bad blocks to it.
int32_t launch_scan_scales(uint32_t typ, const void* raw_dev, size_t n_blocks, unsigned long long* counter_dev, cudaStream_t s) {
    uint32_t e, bb;
    int kind;
    LC_CHECK(scan_geom(typ, &e, &bb, &kind), LC_ERR_UNSUPPORTED, "block-scale scan: ggml type %u has no blocks", typ);
    if (n_blocks == 0) return LC_OK;
    size_t grid = (n_blocks + 255) / 256;
    const size_t cap = (size_t)sm_count() * 8;
    if (grid > cap) grid = cap;
    scan_scales_kernel<<<(unsigned)grid, 256, 0, s>>>((const uint8_t*)raw_dev, n_blocks, bb, kind, counter_dev);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}

}  // namespace lc

using namespace lc;

namespace {
std::mutex g_scan_mutex;
DevBuf g_scan_raw[16], g_scan_ctr[16];

int32_t scan_common(uint32_t typ, const void* host, const void* dev, size_t n_elems, uint64_t* blocks_total, uint64_t* blocks_bad) {
    LC_CHECK(blocks_total && blocks_bad, LC_ERR_INVALID, "lc_scan_blocks: null output");
    *blocks_total = 0;
    *blocks_bad = 0;
    uint32_t e, bb;
    int kind;
    if (!scan_geom(typ, &e, &bb, &kind)) return LC_OK;  // F32, F16, BF16, unknown codes: skipped by the reference
    LC_CHECK(host || dev, LC_ERR_INVALID, "lc_scan_blocks: null pointer");
    if (!have_device()) return LC_ERR_CUDA;
    std::lock_guard<std::mutex> lk(g_scan_mutex);
    int d = 0;
    LC_CUDA(cudaGetDevice(&d));
    LC_CHECK(d >= 0 && d < 16, LC_ERR_CUDA, "no current CUDA device");
    const size_t n_blocks = (n_elems + e - 1) / e;  // loader.rs:325
    LC_TRY(g_scan_ctr[d].reserve(8));
    LC_CUDA(cudaMemsetAsync(g_scan_ctr[d].p, 0, 8, stream()));
    if (host) {
        LC_TRY(g_scan_raw[d].reserve(n_blocks * bb + 1));
        if (n_blocks) LC_CUDA(cudaMemcpyAsync(g_scan_raw[d].p, host, n_blocks * bb, cudaMemcpyHostToDevice, stream()));
        dev = g_scan_raw[d].p;
    }
    LC_TRY(launch_scan_scales(typ, dev, n_blocks, (unsigned long long*)g_scan_ctr[d].p, stream()));
    unsigned long long bad = 0;
    LC_CUDA(cudaMemcpyAsync(&bad, g_scan_ctr[d].p, 8, cudaMemcpyDeviceToHost, stream()));
    LC_CUDA(cudaStreamSynchronize(stream()));
    *blocks_total = n_blocks;
    *blocks_bad = bad;
    return LC_OK;
}
}  // namespace

extern "C" {

int32_t lc_scan_blocks(uint32_t typ, const void* bytes, size_t n_elems, uint64_t* blocks_total, uint64_t* blocks_bad) {
    return scan_common(typ, bytes, nullptr, n_elems, blocks_total, blocks_bad);
}
int32_t lc_scan_blocks_dev(uint32_t typ, const void* bytes_dev, size_t n_elems, uint64_t* blocks_total, uint64_t* blocks_bad) {
    return scan_common(typ, nullptr, bytes_dev, n_elems, blocks_total, blocks_bad);
}

}  // extern "C"

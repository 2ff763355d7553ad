// Quantised matrix-vector / skinny matrix product: y[m,n] = x[m,k] . dequant(W)^T
// with W in raw GGUF block layout (rows of blocks along k), fp32 activations and
// fp32 accumulation (the reference keeps activations in f32 and dequantises the
// weight: rust/src/model/tensor.rs:107-135, rust/src/kernels/simd.rs:226-249).
//
// Main kernel (Q4_K, Q4_0, Q8_0 with k % 256 == 0):
//   * a CTA walks 32-row tiles of W; lane <-> row, warp <-> 256-element unit of k;
//   * each (tile, unit) is one 2-D TMA box [unit bytes x 32 rows] pulled into a
//     per-warp shared-memory ring (mbarrier transaction counts, bounded waits);
//   * the lane reads its row's unit from shared memory with 128-bit loads
//     (row pitch 144 B / 272 B is conflict free), decodes nibbles in registers and
//     multiplies against x held in shared memory (broadcast reads);
//   * per-row partial sums of the warps are added in warp order (deterministic).
// The weight prefetch of the first ring slots is issued before the grid
// dependency wait, so under programmatic dependent launch it overlaps the tail
// of the previous kernel.
// Fallback kernel: any type / any k, one warp per row, element-wise decode.
#include <cuda.h>
#include <cstdlib>
#include <cstring>
#include "lc_kernels.h"
#include "lc_quant.cuh"
#include "lc_tma.cuh"

namespace lc {

// ---------------------------------------------------------------------------
// tensor maps
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            (void)cudaGetLastError();
    }
    return fn;
}


static inline int unit_bytes_of(uint32_t typ) {
    switch (typ) {
        case LC_TYPE_Q4_K: return 144;
        case LC_TYPE_Q4_0: return 144;  // 8 blocks of 18 B
        case LC_TYPE_Q8_0: return 272;  // 8 blocks of 34 B
        case LC_TYPE_Q5_K: return 176;
        default: return 0;
    }
}

int32_t qweight_init(QWeight* w, uint32_t typ, const void* data_dev, int n, int k) {
    QuantGeom g;
    LC_CHECK(quant_geom(typ, &g), LC_ERR_UNSUPPORTED, "unsupported ggml type %u", typ);
    LC_CHECK(k > 0 && n > 0 && k % (int)g.block_elems == 0, LC_ERR_INVALID, "weight [%d x %d]: k is not a whole number of blocks", n, k);
    w->data = data_dev;
    w->typ = typ;
    w->n = n;
    w->k = k;
    w->row_bytes = (size_t)k / g.block_elems * g.block_bytes;
    w->has_tmap = false;
    int ub = unit_bytes_of(typ);
    static const bool no_tma = getenv("LC_NO_TMA") != nullptr;
    if (!no_tma && ub && k % kUnitElems == 0 && ((uintptr_t)data_dev % 16) == 0 && w->row_bytes % 16 == 0 && encode_fn()) {
        cuuint64_t dims[2] = {(cuuint64_t)(w->row_bytes / 4), (cuuint64_t)n};
        cuuint64_t strides[1] = {(cuuint64_t)w->row_bytes};
        cuuint32_t box[2] = {(cuuint32_t)(ub / 4), (cuuint32_t)kTileRows};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = encode_fn()((CUtensorMap*)w->tmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)data_dev, dims, strides, box,
                                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        w->has_tmap = (r == CUDA_SUCCESS);
        if (w->has_tmap) {
            cuuint32_t wide[2] = {(cuuint32_t)(ub / 4), 128u};
            r = encode_fn()((CUtensorMap*)w->tmap_wide, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)data_dev, dims, strides, wide,
                            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            w->has_tmap = (r == CUDA_SUCCESS);
        }
    }
    return LC_OK;
}

// Tensor map over an f16 key pool [rows][128 dims]: boxes of 16 rows x 64 dims (128 bytes), 128-byte swizzle, so that
// a staged page can be read with ldmatrix without bank conflicts.  false when the driver entry point is missing.
bool make_key_pool_tmap(void* out128, const void* pool, uint64_t rows) {
    if (!encode_fn() || ((uintptr_t)pool % 16) != 0) return false;
    cuuint64_t dims[2] = {128, (cuuint64_t)rows};
    cuuint64_t strides[1] = {256};
    cuuint32_t box[2] = {64, 16};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()((CUtensorMap*)out128, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (void*)pool, dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool make_act_tmap(void* out128, const void* base, uint64_t k, uint64_t rows, uint32_t box_rows) {
    // three dimensions: element, row, half (high halves, then `rows` rows further on the low halves); one box takes
    // 64 elements x box_rows rows of both halves and lands as [half][row][128 B]
    if (!encode_fn() || ((uintptr_t)base % 16) != 0 || (k * 2) % 16 != 0 || box_rows == 0 || box_rows > 256) return false;
    cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, 2};
    cuuint64_t strides[2] = {(cuuint64_t)k * 2, (cuuint64_t)k * 2 * rows};
    cuuint32_t box[3] = {64, box_rows, 2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_fn()((CUtensorMap*)out128, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, (void*)base, dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// The same activations with a fourth dimension, the 64-element chunk of k: one box takes `box_chunks` consecutive chunks
// x box_rows rows of both halves and lands as [chunk][half][row][128 B].
bool make_act_tmap_chunks(void* out128, const void* base, uint64_t k, uint64_t rows, uint32_t box_rows, uint32_t box_chunks) {
    if (!encode_fn() || ((uintptr_t)base % 16) != 0 || k % 64 != 0 || box_rows == 0 || box_rows > 256 || box_chunks == 0 || box_chunks > 256) return false;
    cuuint64_t dims[4] = {64, (cuuint64_t)rows, 2, (cuuint64_t)(k / 64)};
    cuuint64_t strides[3] = {(cuuint64_t)k * 2, (cuuint64_t)k * 2 * rows, 128};
    cuuint32_t box[4] = {64, box_rows, 2, box_chunks};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = encode_fn()((CUtensorMap*)out128, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, (void*)base, dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// ---------------------------------------------------------------------------
// per-unit dot products.  `r` = the lane's unit in registers, xs = x of this
// unit for token t at xs + t*xstride (256 floats), sx = per-32 sums of x.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float4 lds4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// four nibbles held in the low 4 bits of each byte of v -> floats
__device__ __forceinline__ void bytes_to_f4(uint32_t v, float& a, float& b, float& c, float& d) {
    a = (float)(v & 0xFFu);
    b = (float)((v >> 8) & 0xFFu);
    c = (float)((v >> 16) & 0xFFu);
    d = (float)(v >> 24);
}
__device__ __forceinline__ void sbytes_to_f4(uint32_t v, float& a, float& b, float& c, float& d) {
    a = (float)(int8_t)(v & 0xFFu);
    b = (float)(int8_t)((v >> 8) & 0xFFu);
    c = (float)(int8_t)((v >> 16) & 0xFFu);
    d = (float)(int8_t)(v >> 24);
}

template <int M>
__device__ __forceinline__ void dot_word_u(uint32_t v, const float* xs, int xstride, float2 (&acc)[M][2]) {
    float q0, q1, q2, q3;
    bytes_to_f4(v, q0, q1, q2, q3);
#pragma unroll
    for (int t = 0; t < M; t++) {
        float4 x = lds4(xs + t * xstride);
        acc[t][0] = __ffma2_rn(make_float2(q0, q1), make_float2(x.x, x.y), acc[t][0]);
        acc[t][1] = __ffma2_rn(make_float2(q2, q3), make_float2(x.z, x.w), acc[t][1]);
    }
}
template <int M>
__device__ __forceinline__ void dot_word_s(uint32_t v, const float* xs, int xstride, float2 (&acc)[M][2]) {
    float q0, q1, q2, q3;
    sbytes_to_f4(v, q0, q1, q2, q3);
#pragma unroll
    for (int t = 0; t < M; t++) {
        float4 x = lds4(xs + t * xstride);
        acc[t][0] = __ffma2_rn(make_float2(q0, q1), make_float2(x.x, x.y), acc[t][0]);
        acc[t][1] = __ffma2_rn(make_float2(q2, q3), make_float2(x.z, x.w), acc[t][1]);
    }
}
template <int M>
__device__ __forceinline__ void zero_acc(float2 (&a)[M][2]) {
#pragma unroll
    for (int t = 0; t < M; t++) a[t][0] = a[t][1] = make_float2(0.f, 0.f);
}
__device__ __forceinline__ float hsum(const float2 (&a)[2]) { return (a[0].x + a[0].y) + (a[1].x + a[1].y); }

// Q4_K unit = one super-block (rust/src/kernels/mod.rs:66-98): w = (d*sc)*q - (dmin*m).
// sum_k x_k w_k = (d*sc) * sum x_k q_k - (dmin*m) * sum x_k over each 32-element sub-block.
template <int M>
__device__ __forceinline__ void unit_dot_q4k(const uint4 (&r)[9], const float* xs, int xstride, const float* sx, int sxstride,
                                             float (&out)[M]) {
    float d = h2f((uint16_t)(r[0].x & 0xFFFFu)), dmin = h2f((uint16_t)(r[0].x >> 16));
    uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
    unpack_scales_k4(r[0].y, r[0].z, r[0].w, &sc_lo, &sc_hi, &mn_lo, &mn_hi);
#pragma unroll
    for (int g = 0; g < 4; g++) {
        uint32_t scw = (g < 2) ? sc_lo : sc_hi, mnw = (g < 2) ? mn_lo : mn_hi;
        int sh = (g & 1) * 16;
        float dl1 = d * (float)((scw >> sh) & 0xFFu), dl2 = d * (float)((scw >> (sh + 8)) & 0xFFu);
        float ml1 = dmin * (float)((mnw >> sh) & 0xFFu), ml2 = dmin * (float)((mnw >> (sh + 8)) & 0xFFu);
        float2 alo[M][2], ahi[M][2];
        zero_acc<M>(alo);
        zero_acc<M>(ahi);
        const uint32_t w[8] = {r[1 + 2 * g].x, r[1 + 2 * g].y, r[1 + 2 * g].z, r[1 + 2 * g].w,
                               r[2 + 2 * g].x, r[2 + 2 * g].y, r[2 + 2 * g].z, r[2 + 2 * g].w};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            dot_word_u<M>(w[i] & 0x0F0F0F0Fu, xs + 64 * g + 4 * i, xstride, alo);
            dot_word_u<M>((w[i] >> 4) & 0x0F0F0F0Fu, xs + 64 * g + 32 + 4 * i, xstride, ahi);
        }
#pragma unroll
        for (int t = 0; t < M; t++) {
            float s1 = sx[t * sxstride + 2 * g], s2 = sx[t * sxstride + 2 * g + 1];
            out[t] += dl1 * hsum(alo[t]) - ml1 * s1;
            out[t] += dl2 * hsum(ahi[t]) - ml2 * s2;
        }
    }
}

// byte `off` .. off+3 of the register file `r` (36 or 68 words), off known at compile time
template <int NW>
__device__ __forceinline__ uint32_t word_at(const uint32_t (&r)[NW], int off) {
    int w = off >> 2, sh = (off & 3) * 8;
    if (sh == 0) return r[w];
    return __funnelshift_r(r[w], (w + 1 < NW) ? r[w + 1] : 0u, sh);
}

// Q4_0 unit = 8 blocks of 18 B (rust/src/kernels/mod.rs:16-34): w = (q - 8) * scale,
// low nibble of byte j -> element j, high nibble -> element j + 16.
template <int M>
__device__ __forceinline__ void unit_dot_q40(const uint32_t (&r)[36], const float* xs, int xstride, float (&out)[M]) {
#pragma unroll
    for (int j = 0; j < 8; j++) {
        int off = 18 * j;
        float scale = h2f((uint16_t)(word_at<36>(r, off & ~3) >> ((off & 3) * 8)));
        float2 acc[M][2];
        zero_acc<M>(acc);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t v = word_at<36>(r, off + 2 + 4 * i);
            float q0, q1, q2, q3;
            bytes_to_f4(v & 0x0F0F0F0Fu, q0, q1, q2, q3);
            float p0, p1, p2, p3;
            bytes_to_f4((v >> 4) & 0x0F0F0F0Fu, p0, p1, p2, p3);
            q0 -= 8.f; q1 -= 8.f; q2 -= 8.f; q3 -= 8.f;
            p0 -= 8.f; p1 -= 8.f; p2 -= 8.f; p3 -= 8.f;
#pragma unroll
            for (int t = 0; t < M; t++) {
                float4 xl = lds4(xs + t * xstride + 32 * j + 4 * i);
                float4 xh = lds4(xs + t * xstride + 32 * j + 16 + 4 * i);
                acc[t][0] = __ffma2_rn(make_float2(q0, q1), make_float2(xl.x, xl.y), acc[t][0]);
                acc[t][1] = __ffma2_rn(make_float2(q2, q3), make_float2(xl.z, xl.w), acc[t][1]);
                acc[t][0] = __ffma2_rn(make_float2(p0, p1), make_float2(xh.x, xh.y), acc[t][0]);
                acc[t][1] = __ffma2_rn(make_float2(p2, p3), make_float2(xh.z, xh.w), acc[t][1]);
            }
        }
#pragma unroll
        for (int t = 0; t < M; t++) out[t] += scale * hsum(acc[t]);
    }
}

// Q8_0 unit = 8 blocks of 34 B (rust/src/kernels/mod.rs:37-51): w = q * scale.
template <int M>
__device__ __forceinline__ void unit_dot_q80(const uint32_t (&r)[68], const float* xs, int xstride, float (&out)[M]) {
#pragma unroll
    for (int j = 0; j < 8; j++) {
        int off = 34 * j;
        float scale = h2f((uint16_t)(word_at<68>(r, off & ~3) >> ((off & 3) * 8)));
        float2 acc[M][2];
        zero_acc<M>(acc);
#pragma unroll
        for (int i = 0; i < 8; i++) dot_word_s<M>(word_at<68>(r, off + 2 + 4 * i), xs + 32 * j + 4 * i, xstride, acc);
#pragma unroll
        for (int t = 0; t < M; t++) out[t] += scale * hsum(acc[t]);
    }
}

template <uint32_t TYPE> struct UnitBytes { static constexpr int v = 144; };
template <> struct UnitBytes<LC_TYPE_Q8_0> { static constexpr int v = 272; };

// ---------------------------------------------------------------------------
// the TMA-staged kernel
// ---------------------------------------------------------------------------
template <uint32_t TYPE, int M, int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32, 1)
qgemv_tma_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, GemvParams p) {
    constexpr int UB = UnitBytes<TYPE>::v;
    constexpr int STAGE_BYTES = UB * kTileRows;
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nunits = p.k / kUnitElems;
    const int ntiles = (p.n + kTileRows - 1) / kTileRows;
    const int nmat = (p.epi == EPI_SILU_MUL) ? 2 : 1;

    // shared memory carve-up
    unsigned char* stage_base = smem + (size_t)warp * STAGES * STAGE_BYTES;
    size_t off = (size_t)WARPS * STAGES * STAGE_BYTES;
    float* xs = reinterpret_cast<float*>(smem + off);            // [M][k]
    off += (size_t)M * p.k * 4;
    float* sx = reinterpret_cast<float*>(smem + off);            // [M][k/32]
    off += (size_t)M * (p.k / 32) * 4;
    float* red = reinterpret_cast<float*>(smem + off);           // [2][WARPS][M][32]
    off += (size_t)2 * WARPS * M * 32 * 4;
    float* gate_vals = reinterpret_cast<float*>(smem + off);     // [M][32]
    off += (size_t)M * 32 * 4;
    float* scratch = reinterpret_cast<float*>(smem + off);       // [32 + M]
    off += (size_t)(32 + M) * 4;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ((off + 7) & ~(size_t)7)) + warp * STAGES;

    // This warp's job list: for each of the CTA's tiles, for each matrix, the units u = warp, warp+WARPS, ...
    const int units_mine = (nunits > warp) ? (nunits - warp + WARPS - 1) / WARPS : 0;
    const int tiles_mine = (ntiles > (int)blockIdx.x) ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int jobs_per_tile = units_mine * nmat;
    const int njobs = tiles_mine * jobs_per_tile;

    auto issue = [&](int job) {
        int ti = job / jobs_per_tile, rem = job % jobs_per_tile;
        int mat = rem / units_mine, ui = rem % units_mine;
        int tile = blockIdx.x + ti * gridDim.x;
        int unit = warp + ui * WARPS;
        int st = job % STAGES;
        mbar_expect_tx(&bars[st], STAGE_BYTES);
        tma_load_2d(stage_base + (size_t)st * STAGE_BYTES, mat ? &tm1 : &tm0, unit * (UB / 4), tile * kTileRows, &bars[st]);
    };

    if (lane == 0) {
        for (int s = 0; s < STAGES; s++) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int j = 0; j < STAGES && j < njobs; j++) issue(j);  // weights do not depend on the previous kernel
    }
    pdl_launch_dependents();
    pdl_wait();  // activations of the previous kernel are visible from here on

    // ---- stage x (optionally RMS-normalised) and the per-32 sums ----
    for (int t = 0; t < M; t++) {
        float scale = 1.0f;
        if (p.norm_w) {
            float ss = 0.f;
            if (t < p.m)
                for (int i = threadIdx.x; i < p.k; i += blockDim.x) { float v = p.x[(size_t)t * p.k + i]; ss = fmaf(v, v, ss); }
            ss = warp_sum(ss);
            __syncthreads();
            if (lane == 0) scratch[warp] = ss;
            __syncthreads();
            if (warp == 0) {
                float r = (lane < WARPS) ? scratch[lane] : 0.f;
                r = warp_sum(r);
                if (lane == 0) scratch[32 + t] = 1.0f / sqrtf(r / (float)p.k + p.eps);
            }
            __syncthreads();
            scale = scratch[32 + t];
        }
        for (int i = threadIdx.x; i < p.k; i += blockDim.x) {
            float v = (t < p.m) ? p.x[(size_t)t * p.k + i] : 0.f;
            if (p.norm_w) v = (v * scale) * p.norm_w[i];
            xs[(size_t)t * p.k + i] = v;
        }
    }
    __syncthreads();
    if (TYPE == LC_TYPE_Q4_K) {
        for (int i = threadIdx.x; i < M * (p.k / 32); i += blockDim.x) {
            int t = i / (p.k / 32), b = i % (p.k / 32);
            const float* xp = xs + (size_t)t * p.k + b * 32;
            float s = 0.f;
#pragma unroll 8
            for (int e = 0; e < 32; e++) s += xp[e];
            sx[i] = s;
        }
        __syncthreads();
    }

    // ---- main loop ----
    float acc[M];
#pragma unroll
    for (int t = 0; t < M; t++) acc[t] = 0.f;
    bool ok = true;
    int job = 0;
    for (int ti = 0; ti < tiles_mine; ti++) {
        const int tile = blockIdx.x + ti * gridDim.x;
        for (int mat = 0; mat < nmat; mat++) {
            for (int ui = 0; ui < units_mine; ui++, job++) {
                const int unit = warp + ui * WARPS;
                const int st = job % STAGES;
                const uint32_t parity = (uint32_t)((job / STAGES) & 1);
                ok = ok && mbar_wait(&bars[st], parity);
                const unsigned char* src = stage_base + (size_t)st * STAGE_BYTES + lane * UB;
                if (TYPE == LC_TYPE_Q4_K) {
                    uint4 r[9];
#pragma unroll
                    for (int i = 0; i < 9; i++) r[i] = reinterpret_cast<const uint4*>(src)[i];
                    __syncwarp();
                    if (lane == 0 && job + STAGES < njobs) issue(job + STAGES);
                    unit_dot_q4k<M>(r, xs + unit * kUnitElems, p.k, sx + unit * 8, p.k / 32, acc);
                } else if (TYPE == LC_TYPE_Q4_0) {
                    uint32_t r[36];
#pragma unroll
                    for (int i = 0; i < 9; i++) {
                        uint4 v = reinterpret_cast<const uint4*>(src)[i];
                        r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
                    }
                    __syncwarp();
                    if (lane == 0 && job + STAGES < njobs) issue(job + STAGES);
                    unit_dot_q40<M>(r, xs + unit * kUnitElems, p.k, acc);
                } else {
                    uint32_t r[68];
#pragma unroll
                    for (int i = 0; i < 17; i++) {
                        uint4 v = reinterpret_cast<const uint4*>(src)[i];
                        r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
                    }
                    __syncwarp();
                    if (lane == 0 && job + STAGES < njobs) issue(job + STAGES);
                    unit_dot_q80<M>(r, xs + unit * kUnitElems, p.k, acc);
                }
            }
            // ---- cross-warp reduction of this (tile, matrix), in warp order ----
            const int seq = ti * nmat + mat;
            float* rb = red + (size_t)(seq & 1) * WARPS * M * 32;
#pragma unroll
            for (int t = 0; t < M; t++) { rb[(warp * M + t) * 32 + lane] = acc[t]; acc[t] = 0.f; }
            __syncthreads();
            if (warp < M) {
                const int t = warp;
                float y = 0.f;
#pragma unroll 4
                for (int w = 0; w < WARPS; w++) y += rb[(w * M + t) * 32 + lane];
                const int row = tile * kTileRows + lane;
                if (p.epi == EPI_SILU_MUL) {
                    if (mat == 0) {
                        gate_vals[t * 32 + lane] = y;
                    } else if (row < p.n && t < p.m) {
                        p.out[(size_t)t * p.n + row] = silu_f(gate_vals[t * 32 + lane]) * y;
                    }
                } else if (row < p.n && t < p.m) {
                    if (p.epi == EPI_ADD_RESIDUAL) y = p.residual[(size_t)t * p.n + row] + y;
                    p.out[(size_t)t * p.n + row] = y;
                }
            }
        }
    }
    if (!ok && lane == 0 && p.error_flag) atomicExch(p.error_flag, 1);
}

// ---------------------------------------------------------------------------
// fallback: any ggml type, any k.  One warp per output row, lanes stride over k.
// ---------------------------------------------------------------------------
template <int M>
__global__ void qgemv_generic_kernel(uint32_t typ, const uint8_t* __restrict__ w, const uint8_t* __restrict__ w2, GemvParams p) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scale_sh[M];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    if (p.norm_w) {
        if (warp < M) {
            float ss = 0.f;
            if (warp < p.m)
                for (int i = lane; i < p.k; i += 32) { float v = p.x[(size_t)warp * p.k + i]; ss = fmaf(v, v, ss); }
            ss = warp_sum(ss);
            if (lane == 0) scale_sh[warp] = 1.0f / sqrtf(ss / (float)p.k + p.eps);
        }
        __syncthreads();
    }
    for (int row = blockIdx.x * nwarps + warp; row < p.n; row += gridDim.x * nwarps) {
        float acc[M], acc2[M];
#pragma unroll
        for (int t = 0; t < M; t++) acc[t] = acc2[t] = 0.f;
        for (int i = lane; i < p.k; i += 32) {
            float wv = dequant_elem(typ, w, (size_t)row * p.k + i);
            float wv2 = (p.epi == EPI_SILU_MUL) ? dequant_elem(typ, w2, (size_t)row * p.k + i) : 0.f;
#pragma unroll
            for (int t = 0; t < M; t++) {
                if (t < p.m) {
                    float xv = p.x[(size_t)t * p.k + i];
                    if (p.norm_w) xv = (xv * scale_sh[t]) * p.norm_w[i];
                    acc[t] = fmaf(xv, wv, acc[t]);
                    acc2[t] = fmaf(xv, wv2, acc2[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < M; t++) {
            float y = warp_sum(acc[t]);
            float y2 = warp_sum(acc2[t]);
            if (lane == 0 && t < p.m) {
                if (p.epi == EPI_SILU_MUL) y = silu_f(y) * y2;
                else if (p.epi == EPI_ADD_RESIDUAL) y = p.residual[(size_t)t * p.n + row] + y;
                p.out[(size_t)t * p.n + row] = y;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
bool pdl_enabled() {
    static const bool on = getenv("LC_NO_PDL") == nullptr;
    return on;
}
// The word kernels raise when a bounded wait runs out.  It lives in the library image (zero when the image is loaded on a
// device), so looking it up allocates nothing: entry points that promise not to allocate can use every kernel.
static __device__ int g_error_flag_word;
static int* g_error_flag[16] = {};
int* gemv_error_flag_dev() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
    if (!g_error_flag[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_error_flag_word) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
        g_error_flag[dev] = (int*)p;
    }
    return g_error_flag[dev];
}

template <uint32_t TYPE, int M, int WARPS, int STAGES>
static size_t tma_smem_bytes(int k) {
    constexpr int UB = UnitBytes<TYPE>::v;
    size_t b = (size_t)WARPS * STAGES * UB * kTileRows;
    b += (size_t)M * k * 4 + (size_t)M * (k / 32) * 4;
    b += (size_t)2 * WARPS * M * 32 * 4 + (size_t)M * 32 * 4 + (size_t)(32 + M) * 4;
    b = (b + 7) & ~(size_t)7;
    b += (size_t)WARPS * STAGES * 8;
    return b;
}

template <uint32_t TYPE, int M, int WARPS, int STAGES>
static int32_t launch_tma_cfg(const GemvArgs& a, cudaStream_t s) {
    auto kern = qgemv_tma_kernel<TYPE, M, WARPS, STAGES>;
    size_t smem = tma_smem_bytes<TYPE, M, WARPS, STAGES>(a.w->k);
    LC_CUDA(ensure_smem_limit((const void*)kern, kMaxSmem));
    GemvParams p;
    p.x = a.x; p.out = a.out; p.residual = a.residual; p.norm_w = a.norm_w; p.eps = a.eps;
    p.n = a.w->n; p.k = a.w->k; p.m = a.m; p.epi = (int)a.epi; p.error_flag = gemv_error_flag_dev();
    int ntiles = (p.n + kTileRows - 1) / kTileRows;
    int grid = sm_count();
    if (grid > ntiles) grid = ntiles;
    const CUtensorMap* t0 = (const CUtensorMap*)a.w->tmap;
    const CUtensorMap* t1 = a.w2 ? (const CUtensorMap*)a.w2->tmap : t0;
    LC_CUDA(launch_pdl(kern, dim3(grid), dim3(WARPS * 32), smem, s, *t0, *t1, p));
    return LC_OK;
}

template <uint32_t TYPE, int M>
static int32_t launch_tma_m(const GemvArgs& a, cudaStream_t s, bool* launched) {
    *launched = true;
    int k = a.w->k;
    if constexpr (M == 1) {
        if (tma_smem_bytes<TYPE, M, 16, 3>(k) <= kMaxSmem && k <= 4096) return launch_tma_cfg<TYPE, M, 16, 3>(a, s);
        if (tma_smem_bytes<TYPE, M, 16, 2>(k) <= kMaxSmem) return launch_tma_cfg<TYPE, M, 16, 2>(a, s);
    }
    if (tma_smem_bytes<TYPE, M, 8, 2>(k) <= kMaxSmem) return launch_tma_cfg<TYPE, M, 8, 2>(a, s);
    *launched = false;
    return LC_OK;
}

template <uint32_t TYPE>
static int32_t launch_tma_type(const GemvArgs& a, int mt, cudaStream_t s, bool* launched) {
    switch (mt) {
        case 1: return launch_tma_m<TYPE, 1>(a, s, launched);
        case 2: return launch_tma_m<TYPE, 2>(a, s, launched);
        case 4: return launch_tma_m<TYPE, 4>(a, s, launched);
        default: return launch_tma_m<TYPE, 8>(a, s, launched);
    }
}

static int32_t launch_generic(const GemvArgs& a, cudaStream_t s) {
    GemvParams p;
    p.x = a.x; p.out = a.out; p.residual = a.residual; p.norm_w = a.norm_w; p.eps = a.eps;
    p.n = a.w->n; p.k = a.w->k; p.m = a.m; p.epi = (int)a.epi; p.error_flag = nullptr;
    int grid = (p.n + 7) / 8;
    int cap = sm_count() * 8;
    if (grid > cap) grid = cap;
    const uint8_t* w2 = a.w2 ? (const uint8_t*)a.w2->data : nullptr;
    LC_CUDA(launch_pdl(qgemv_generic_kernel<8>, dim3(grid), dim3(256), 0, s, a.w->typ, (const uint8_t*)a.w->data, w2, p));
    return LC_OK;
}

bool qgemv_push_supported(const GemvArgs& a) {
    static const bool force_fp32 = getenv("LC_GEMV_FP32") != nullptr;
    return a.w && !a.group && a.w->typ == LC_TYPE_Q4_K && a.w->has_tmap && a.epi != EPI_SILU_MUL && !force_fp32 && a.m >= 1 && a.m <= 8 &&
           qgemv_mma_supports(a.w->k) && ((uintptr_t)a.x % 16) == 0 && (!a.norm_w || ((uintptr_t)a.norm_w % 16) == 0);
}

static int round_m(int m) { return m <= 1 ? 1 : (m <= 2 ? 2 : (m <= 4 ? 4 : 8)); }

int32_t launch_qgemv(const GemvArgs& a, cudaStream_t s) {
    LC_CHECK(a.w && a.x && a.out, LC_ERR_INVALID, "qgemv: null argument");
    if (a.group) {  // the experts of a mixture-of-experts layer in one launch (Q4_K only)
        bool launched = false;
        LC_CHECK(a.w->typ == LC_TYPE_Q4_K && a.w->has_tmap, LC_ERR_UNSUPPORTED, "grouped qgemv: experts must be Q4_K with tensor maps");
        LC_TRY(launch_qgemv_mma_q4k_grouped(a, s, &launched));
        LC_CHECK(launched, LC_ERR_UNSUPPORTED, "grouped qgemv: rows of %d elements do not fit the kernel", a.w->k);
        return LC_OK;
    }
    LC_CHECK(a.m >= 1 && a.m <= 8, LC_ERR_INVALID, "qgemv: m=%d outside 1..8", a.m);
    if (a.epi == EPI_SILU_MUL)
        LC_CHECK(a.w2 && a.w2->n == a.w->n && a.w2->k == a.w->k && a.w2->typ == a.w->typ, LC_ERR_INVALID,
                 "qgemv: gate/up matrices differ in shape or type");
    if (a.epi == EPI_ADD_RESIDUAL) LC_CHECK(a.residual, LC_ERR_INVALID, "qgemv: residual missing");
    bool tma_ok = a.w->has_tmap && (a.epi != EPI_SILU_MUL || a.w2->has_tmap);
    static const bool force_fp32 = getenv("LC_GEMV_FP32") != nullptr;
    static const bool q5k_plain = getenv("LC_GEMV_Q5K_PLAIN") != nullptr;
    const bool f32_types = a.w->typ == LC_TYPE_Q4_K || a.w->typ == LC_TYPE_Q4_0 || a.w->typ == LC_TYPE_Q8_0;  // types qgemv_tma_kernel knows
    if (tma_ok && (a.w->typ == LC_TYPE_Q4_K || (a.w->typ == LC_TYPE_Q5_K && !q5k_plain) ||
                   ((a.w->typ == LC_TYPE_Q4_0 || a.w->typ == LC_TYPE_Q8_0) && a.w->k % kUnitElems == 0)) && !force_fp32) {
        bool launched = false;
        LC_TRY(launch_qgemv_mma_q4k(a, s, &launched));
        if (launched) return LC_OK;
    }
    LC_CHECK(a.push == nullptr, LC_ERR_STATE, "qgemv: rows cannot leave as tagged words from this kernel (qgemv_push_supported was not asked)");
    if (tma_ok && f32_types) {
        for (int mt = round_m(a.m); mt >= 1; mt >>= 1) {
            // the kernel handles mt tokens per pass; when shared memory cannot hold round_m(m) token
            // vectors the caller's m is split further below
            bool launched = false;
            if (mt < a.m) break;
            switch (a.w->typ) {
                case LC_TYPE_Q4_K: LC_TRY(launch_tma_type<LC_TYPE_Q4_K>(a, mt, s, &launched)); break;
                case LC_TYPE_Q4_0: LC_TRY(launch_tma_type<LC_TYPE_Q4_0>(a, mt, s, &launched)); break;
                case LC_TYPE_Q8_0: LC_TRY(launch_tma_type<LC_TYPE_Q8_0>(a, mt, s, &launched)); break;
                default: break;
            }
            if (launched) return LC_OK;
            break;
        }
        // shared memory too small for a.m token vectors: split the tokens
        if (a.m > 1) {
            int half = a.m / 2;
            GemvArgs lo = a, hi = a;
            lo.m = half;
            hi.m = a.m - half;
            hi.x = a.x + (size_t)half * a.w->k;
            hi.out = a.out + (size_t)half * a.w->n;
            if (a.residual) hi.residual = a.residual + (size_t)half * a.w->n;
            LC_TRY(launch_qgemv(lo, s));
            return launch_qgemv(hi, s);
        }
    }
    if (a.w->typ == LC_TYPE_Q6_K) {
        bool launched = false;
        LC_TRY(launch_qgemv_mma_q6k(a, s, &launched));
        if (launched) return LC_OK;
    }
    // Five to eight tokens of Q5_K / Q6_K (the token tiles of a prefill): two passes of the tensor-core kernels over the
    // weights are several times faster than one of the plain-load kernel, whose every row pair re-reads all tokens' activations.
    if (a.m > 4 && !a.push &&
        ((a.w->typ == LC_TYPE_Q6_K && qgemv_mma_q6k_supports(a, 4)) ||
         (a.w->typ == LC_TYPE_Q5_K && tma_ok && !q5k_plain && !force_fp32 && qgemv_mma_q5k_supports4(a.w->k) && ((uintptr_t)a.x % 16) == 0 &&
          (!a.norm_w || ((uintptr_t)a.norm_w % 16) == 0)))) {
        const int half = a.m / 2;
        GemvArgs lo = a, hi = a;
        lo.m = half;
        hi.m = a.m - half;
        hi.x = a.x + (size_t)half * a.w->k;
        hi.out = a.out + (size_t)half * a.w->n;
        if (a.residual) hi.residual = a.residual + (size_t)half * a.w->n;
        LC_TRY(launch_qgemv(lo, s));
        return launch_qgemv(hi, s);
    }
    {
        bool launched = false;
        LC_TRY(launch_qgemv_kq(a, s, &launched));  // Q5_K / Q6_K with whole 256-element blocks, F16 / F32 rows
        if (launched) return LC_OK;
    }
    return launch_generic(a, s);
}

}  // namespace lc

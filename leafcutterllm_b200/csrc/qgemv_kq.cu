// Matrix-vector products over Q5_K and Q6_K weights (rust/src/kernels/mod.rs:101-180), and over IQ4_NL and plain F16 / F32 matrices: the types a "Q4_K_M" or "Q5_K_M"
// GGUF file mixes with Q4_K (attn_v, ffn_down, output).  One warp per group of one or two output rows; a few lanes share a 256-element
// super-block, each taking the elements that live in the same 16 bytes of every plane of the block, so that a block's
// bytes are read once, in 16-byte (Q5_K) or 2-byte (Q6_K: 210-byte blocks are only 2-byte aligned) pieces, and unpacked
// with integer logic instead of one dequantisation call per element.  Per sub-block the integer quants are summed
// against x in f32 and the block's scales are applied to the sums:
//
//   Q6_K   w = d * sc[is] * (q - 32)                   ->  acc += (d * sc) * sum (q - 32) x
//   Q5_K   w = d * sc * q - dmin * m   (q has 5 bits)   ->  acc += (d * sc) * sum q x - (dmin * m) * sum x
//
// Activations are read from global memory (a token's row stays in L1); the RMS norm of the input, the residual add and
// SiLU(gate) * up are fused as in the other matrix-vector kernels.  HBM-bound work: no tensor cores.
#include "lc_kernels.h"
#include "lc_quant.cuh"
#include "lc_tma.cuh"

namespace lc {

namespace {

constexpr int kWarps = 8;

__device__ __forceinline__ uint32_t ldg16x2(const uint8_t* p) {  // four bytes from a 2-byte aligned address
    const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
    return (uint32_t)__ldg(h) | ((uint32_t)__ldg(h + 1) << 16);
}

// Sixteen x of token t starting at element e (a multiple of 16), normalised when the product fuses the RMS norm.
__device__ __forceinline__ void load_x16(const GemvParams& p, int t, int e, float scale, float (&x)[16]) {
    const float4* xp = reinterpret_cast<const float4*>(p.x + (size_t)t * p.k + e);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float4 v = __ldg(xp + i);
        x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
    }
    if (p.norm_w) {
        const float4* gp = reinterpret_cast<const float4*>(p.norm_w + e);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 g = __ldg(gp + i);
            x[4 * i] = (x[4 * i] * scale) * g.x; x[4 * i + 1] = (x[4 * i + 1] * scale) * g.y;
            x[4 * i + 2] = (x[4 * i + 2] * scale) * g.z; x[4 * i + 3] = (x[4 * i + 3] * scale) * g.w;
        }
    }
}

// Q6_K (mod.rs:145-180): lane part = (n, lh): half n of the block, l = 16 lh .. 16 lh + 15.  The four quads of those l share
// ql[64n + l] (quads 0, 2: low, high nibble), ql[64n + 32 + l] (quads 1, 3) and qh[32n + l] (two bits per quad).
// R rows at a time: the sixteen x of a quad are loaded once and used against every row's block, which divides the L1
// traffic of the activations -- five times the weight bytes with one row per warp -- by R.
template <int M, int R>
__device__ __forceinline__ void block_q6k(const uint8_t* b, size_t row_bytes, int rows_here, int part, const GemvParams& p, int e0, const float* scale,
                                          float (&acc)[R][M]) {
    const int n = part >> 1, lh = part & 1;
    uint32_t la[R][4], lb[R][4], hh[R][4];
    float dl[R][4];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const uint8_t* br = b + (size_t)min(r, rows_here - 1) * row_bytes;  // rows past the end repeat the last one; their sums are dropped
        const uint8_t* qla = br + 64 * n + 16 * lh;
        const uint8_t* qhp = br + 128 + 32 * n + 16 * lh;
#pragma unroll
        for (int i = 0; i < 4; i++) { la[r][i] = ldg16x2(qla + 4 * i); lb[r][i] = ldg16x2(qla + 32 + 4 * i); hh[r][i] = ldg16x2(qhp + 4 * i); }
        const float d = h2f(__ldg(reinterpret_cast<const uint16_t*>(br + 208)));
        const int8_t* sc = reinterpret_cast<const int8_t*>(br + 192 + 8 * n + lh);
#pragma unroll
        for (int q = 0; q < 4; q++) dl[r][q] = __fmul_rn(d, (float)__ldg(sc + 2 * q));
    }
#pragma unroll
    for (int t = 0; t < M; t++) {
        if (t >= p.m) break;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            float x[16];
            load_x16(p, t, e0 + 128 * n + 32 * q + 16 * lh, scale[t], x);
#pragma unroll
            for (int r = 0; r < R; r++) {
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const uint32_t lw = (q & 1) ? lb[r][j >> 2] : la[r][j >> 2];
                    const uint32_t byte = (lw >> (8 * (j & 3))) & 0xFFu;
                    const uint32_t lo = (q & 2) ? (byte >> 4) : (byte & 0x0Fu);
                    const uint32_t hi = (hh[r][j >> 2] >> (8 * (j & 3) + 2 * q)) & 3u;
                    s = fmaf((float)((int)(lo | (hi << 4)) - 32), x[j], s);
                }
                acc[r][t] = fmaf(dl[r][q], s, acc[r][t]);
            }
        }
    }
}

// Q5_K (mod.rs:101-142): lane part = (g, hs): 64-element group g, l = 16 hs .. 16 hs + 15.  Low nibbles of qs[32g + l] are
// sub-block 2g, high nibbles sub-block 2g + 1; bit 2g (2g + 1) of qh[l] is their fifth bit.
template <int M, int R>
__device__ __forceinline__ void block_q5k(const uint8_t* b, size_t row_bytes, int rows_here, int part, const GemvParams& p, int e0, const float* scale,
                                          float (&acc)[R][M]) {
    const int g = part >> 1, hs = part & 1;
    uint4 qs[R], qh[R];
    float dA[R], mA[R], dB[R], mB[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const uint8_t* br = b + (size_t)min(r, rows_here - 1) * row_bytes;  // rows past the end repeat the last one; their sums are dropped
        const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(br));
        qs[r] = __ldg(reinterpret_cast<const uint4*>(br + 48 + 32 * g + 16 * hs));
        qh[r] = __ldg(reinterpret_cast<const uint4*>(br + 16 + 16 * hs));
        const float d = h2f((uint16_t)(hdr.x & 0xFFFFu)), dmin = h2f((uint16_t)(hdr.x >> 16));
        uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
        unpack_scales_k4(hdr.y, hdr.z, hdr.w, &sc_lo, &sc_hi, &mn_lo, &mn_hi);
        const uint32_t scw = g < 2 ? sc_lo : sc_hi, mnw = g < 2 ? mn_lo : mn_hi;
        const int sh = (g & 1) * 16;
        dA[r] = __fmul_rn(d, (float)((scw >> sh) & 0xFFu)); mA[r] = __fmul_rn(dmin, (float)((mnw >> sh) & 0xFFu));
        dB[r] = __fmul_rn(d, (float)((scw >> (sh + 8)) & 0xFFu)); mB[r] = __fmul_rn(dmin, (float)((mnw >> (sh + 8)) & 0xFFu));
    }
#pragma unroll
    for (int t = 0; t < M; t++) {
        if (t >= p.m) break;
        float xa[16], xb[16];
        load_x16(p, t, e0 + 64 * g + 16 * hs, scale[t], xa);
        load_x16(p, t, e0 + 64 * g + 32 + 16 * hs, scale[t], xb);
        float xsa = 0.f, xsb = 0.f;
#pragma unroll
        for (int j = 0; j < 16; j++) { xsa += xa[j]; xsb += xb[j]; }
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint32_t qw[4] = {qs[r].x, qs[r].y, qs[r].z, qs[r].w}, hw[4] = {qh[r].x, qh[r].y, qh[r].z, qh[r].w};
            float sa = 0.f, sb = 0.f;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const uint32_t byte = (qw[j >> 2] >> (8 * (j & 3))) & 0xFFu;
                const uint32_t hb = (hw[j >> 2] >> (8 * (j & 3))) >> (2 * g);
                const float qa = (float)((byte & 0x0Fu) | ((hb & 1u) << 4)), qb = (float)((byte >> 4) | ((hb & 2u) << 3));
                sa = fmaf(qa, xa[j], sa);
                sb = fmaf(qb, xb[j], sb);
            }
            acc[r][t] = fmaf(dA[r], sa, acc[r][t]); acc[r][t] = fmaf(-mA[r], xsa, acc[r][t]);
            acc[r][t] = fmaf(dB[r], sb, acc[r][t]); acc[r][t] = fmaf(-mB[r], xsb, acc[r][t]);
        }
    }
}

template <uint32_t TYPE, int M>
__global__ void __launch_bounds__(kWarps * 32, 2)
qgemv_kq_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ w2, GemvParams p) {
    constexpr int LPB = TYPE == LC_TYPE_Q6_K ? 4 : 8;     // lanes per block
    constexpr int BB = TYPE == LC_TYPE_Q6_K ? 210 : 176;  // block bytes
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scale_sh[M];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (p.norm_w) {  // cpu.rs:49-60: 1 / sqrt(mean(x^2) + eps), one warp per token
        for (int t = warp; t < p.m; t += kWarps) {
            float ss = 0.f;
            for (int i = lane; i < p.k; i += 32) { const float v = p.x[(size_t)t * p.k + i]; ss = fmaf(v, v, ss); }
            ss = warp_sum(ss);
            if (lane == 0) scale_sh[t] = 1.0f / sqrtf(ss / (float)p.k + p.eps);
        }
        __syncthreads();
    }
    float scale[M];
#pragma unroll
    for (int t = 0; t < M; t++) scale[t] = (p.norm_w && t < p.m) ? scale_sh[t] : 1.f;
    const int nb = p.k / 256;
    const size_t row_bytes = (size_t)nb * BB;
    const int part = lane % LPB, bsub = lane / LPB;
    constexpr int R = M <= 2 ? 2 : 1;  // rows per warp and turn
    const int two = p.epi == EPI_SILU_MUL ? 1 : 0;
    for (int row0 = (blockIdx.x * kWarps + warp) * R; row0 < p.n; row0 += gridDim.x * kWarps * R) {
        const int rows_here = min(R, p.n - row0);
        float acc[R][M], acc2[R][M];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int t = 0; t < M; t++) acc[r][t] = acc2[r][t] = 0.f;
        for (int b0 = 0; b0 < nb; b0 += 32 / LPB) {
            const int b = b0 + bsub;
            if (b < nb) {
                const uint8_t* bp = w + (size_t)row0 * row_bytes + (size_t)b * BB;
                if (TYPE == LC_TYPE_Q6_K) block_q6k<M, R>(bp, row_bytes, rows_here, part, p, b * 256, scale, acc);
                else block_q5k<M, R>(bp, row_bytes, rows_here, part, p, b * 256, scale, acc);
                if (two) {
                    const uint8_t* bp2 = w2 + (size_t)row0 * row_bytes + (size_t)b * BB;
                    if (TYPE == LC_TYPE_Q6_K) block_q6k<M, R>(bp2, row_bytes, rows_here, part, p, b * 256, scale, acc2);
                    else block_q5k<M, R>(bp2, row_bytes, rows_here, part, p, b * 256, scale, acc2);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
#pragma unroll
            for (int t = 0; t < M; t++) {
                if (t >= p.m) break;
                float y = warp_sum(acc[r][t]);
                const float y2 = two ? warp_sum(acc2[r][t]) : 0.f;
                if (lane == 0 && r < rows_here) {
                    const int row = row0 + r;
                    if (two) y = silu_f(y) * y2;
                    else if (p.epi == EPI_ADD_RESIDUAL) y = p.residual[(size_t)t * p.n + row] + y;
                    p.out[(size_t)t * p.n + row] = y;
                }
            }
        }
    }
}

template <uint32_t TYPE, int M>
int32_t launch_kq(const GemvArgs& a, cudaStream_t s) {
    GemvParams p;
    p.x = a.x; p.out = a.out; p.residual = a.residual; p.norm_w = a.norm_w; p.eps = a.eps;
    p.n = a.w->n; p.k = a.w->k; p.m = a.m; p.epi = (int)a.epi; p.error_flag = nullptr;
    const int rows_per_cta = kWarps * (M <= 2 ? 2 : 1);
    int grid = (p.n + rows_per_cta - 1) / rows_per_cta;
    const int cap = sm_count() * 8;
    if (grid > cap) grid = cap;
    const uint8_t* w2 = a.w2 ? (const uint8_t*)a.w2->data : nullptr;
    LC_CUDA(launch_pdl(qgemv_kq_kernel<TYPE, M>, dim3(grid), dim3(kWarps * 32), 0, s, (const uint8_t*)a.w->data, w2, p));
    return LC_OK;
}

// F16 / F32 matrices (unquantised GGUF files, rust/src/model/loader.rs:213-224): one warp per row, eight weights per lane
// and load, activations from L1.  Pure streaming: 2 or 4 bytes per weight.
template <bool F32, int M>
__global__ void __launch_bounds__(kWarps * 32)
qgemv_dense_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ w2, GemvParams p) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scale_sh[M];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (p.norm_w) {
        for (int t = warp; t < p.m; t += kWarps) {
            float ss = 0.f;
            for (int i = lane; i < p.k; i += 32) { const float v = p.x[(size_t)t * p.k + i]; ss = fmaf(v, v, ss); }
            ss = warp_sum(ss);
            if (lane == 0) scale_sh[t] = 1.0f / sqrtf(ss / (float)p.k + p.eps);
        }
        __syncthreads();
    }
    float scale[M];
#pragma unroll
    for (int t = 0; t < M; t++) scale[t] = (p.norm_w && t < p.m) ? scale_sh[t] : 1.f;
    const size_t row_bytes = (size_t)p.k * (F32 ? 4 : 2);
    const int two = p.epi == EPI_SILU_MUL ? 1 : 0;
    for (int row = blockIdx.x * kWarps + warp; row < p.n; row += gridDim.x * kWarps) {
        float acc[M], acc2[M];
#pragma unroll
        for (int t = 0; t < M; t++) acc[t] = acc2[t] = 0.f;
        for (int e = lane * 8; e < p.k; e += 256) {
            float wv[8], wv2[8];
            auto load8 = [&](const uint8_t* base, float (&o)[8]) {
                if (F32) {
                    const float4 a = __ldg(reinterpret_cast<const float4*>(base + (size_t)row * row_bytes) + e / 4);
                    const float4 b = __ldg(reinterpret_cast<const float4*>(base + (size_t)row * row_bytes) + e / 4 + 1);
                    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
                } else {
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(base + (size_t)row * row_bytes) + e / 8);
                    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                    for (int j = 0; j < 4; j++) { const float2 f = __half22float2(h[j]); o[2 * j] = f.x; o[2 * j + 1] = f.y; }
                }
            };
            load8(w, wv);
            if (two) load8(w2, wv2);
#pragma unroll
            for (int t = 0; t < M; t++) {
                if (t >= p.m) break;
                const float4 xa = __ldg(reinterpret_cast<const float4*>(p.x + (size_t)t * p.k + e));
                const float4 xb = __ldg(reinterpret_cast<const float4*>(p.x + (size_t)t * p.k + e) + 1);
                float x[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                if (p.norm_w) {
                    const float4 ga = __ldg(reinterpret_cast<const float4*>(p.norm_w + e));
                    const float4 gb = __ldg(reinterpret_cast<const float4*>(p.norm_w + e) + 1);
                    const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
                    for (int j = 0; j < 8; j++) x[j] = (x[j] * scale[t]) * g[j];
                }
#pragma unroll
                for (int j = 0; j < 8; j++) { acc[t] = fmaf(x[j], wv[j], acc[t]); if (two) acc2[t] = fmaf(x[j], wv2[j], acc2[t]); }
            }
        }
#pragma unroll
        for (int t = 0; t < M; t++) {
            if (t >= p.m) break;
            float y = warp_sum(acc[t]);
            const float y2 = two ? warp_sum(acc2[t]) : 0.f;
            if (lane == 0) {
                if (two) y = silu_f(y) * y2;
                else if (p.epi == EPI_ADD_RESIDUAL) y = p.residual[(size_t)t * p.n + row] + y;
                p.out[(size_t)t * p.n + row] = y;
            }
        }
    }
}

template <bool F32, int M>
int32_t launch_dense(const GemvArgs& a, cudaStream_t s) {
    GemvParams p;
    p.x = a.x; p.out = a.out; p.residual = a.residual; p.norm_w = a.norm_w; p.eps = a.eps;
    p.n = a.w->n; p.k = a.w->k; p.m = a.m; p.epi = (int)a.epi; p.error_flag = nullptr;
    int grid = (p.n + kWarps - 1) / kWarps;
    const int cap = sm_count() * 8;
    if (grid > cap) grid = cap;
    const uint8_t* w2 = a.w2 ? (const uint8_t*)a.w2->data : nullptr;
    LC_CUDA(launch_pdl(qgemv_dense_kernel<F32, M>, dim3(grid), dim3(kWarps * 32), 0, s, (const uint8_t*)a.w->data, w2, p));
    return LC_OK;
}

// IQ4_NL (mod.rs:186-216): 18-byte blocks of 32 weights, f16 scale, nibble e & 1 of byte e >> 1 indexes the reference's
// own 16-entry table.  One warp per row, a lane per block and turn; the table sits in shared memory.
template <int M>
__global__ void __launch_bounds__(kWarps * 32)
qgemv_iq4nl_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ w2, GemvParams p) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scale_sh[M];
    __shared__ float lut[16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x < 16) {
        const float T[16] = {-1.0f, -0.6962f, -0.5251f, -0.3952f, -0.2893f, -0.1957f, -0.1107f, -0.0322f,
                             0.0322f, 0.1107f, 0.1957f, 0.2893f, 0.3952f, 0.5251f, 0.6962f, 1.0f};
        lut[threadIdx.x] = T[threadIdx.x];
    }
    if (p.norm_w) {
        for (int t = warp; t < p.m; t += kWarps) {
            float ss = 0.f;
            for (int i = lane; i < p.k; i += 32) { const float v = p.x[(size_t)t * p.k + i]; ss = fmaf(v, v, ss); }
            ss = warp_sum(ss);
            if (lane == 0) scale_sh[t] = 1.0f / sqrtf(ss / (float)p.k + p.eps);
        }
    }
    __syncthreads();
    float scale[M];
#pragma unroll
    for (int t = 0; t < M; t++) scale[t] = (p.norm_w && t < p.m) ? scale_sh[t] : 1.f;
    const int nb = p.k / 32;
    const size_t row_bytes = (size_t)nb * 18;
    const int two = p.epi == EPI_SILU_MUL ? 1 : 0;
    for (int row = blockIdx.x * kWarps + warp; row < p.n; row += gridDim.x * kWarps) {
        float acc[M], acc2[M];
#pragma unroll
        for (int t = 0; t < M; t++) acc[t] = acc2[t] = 0.f;
        for (int b = lane; b < nb; b += 32) {
            float wv[32], wv2[32];
            auto load_block = [&](const uint8_t* base, float (&o)[32]) {
                const uint8_t* bp = base + (size_t)row * row_bytes + (size_t)b * 18;
                const float sc = h2f(__ldg(reinterpret_cast<const uint16_t*>(bp)));
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t q = ldg16x2(bp + 2 + 4 * i);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint32_t byte = (q >> (8 * j)) & 0xFFu;
                        o[8 * i + 2 * j] = __fmul_rn(sc, lut[byte & 0x0Fu]);
                        o[8 * i + 2 * j + 1] = __fmul_rn(sc, lut[byte >> 4]);
                    }
                }
            };
            load_block(w, wv);
            if (two) load_block(w2, wv2);
#pragma unroll
            for (int t = 0; t < M; t++) {
                if (t >= p.m) break;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    float x[16];
                    load_x16(p, t, b * 32 + 16 * h, scale[t], x);
#pragma unroll
                    for (int j = 0; j < 16; j++) { acc[t] = fmaf(x[j], wv[16 * h + j], acc[t]); if (two) acc2[t] = fmaf(x[j], wv2[16 * h + j], acc2[t]); }
                }
            }
        }
#pragma unroll
        for (int t = 0; t < M; t++) {
            if (t >= p.m) break;
            float y = warp_sum(acc[t]);
            const float y2 = two ? warp_sum(acc2[t]) : 0.f;
            if (lane == 0) {
                if (two) y = silu_f(y) * y2;
                else if (p.epi == EPI_ADD_RESIDUAL) y = p.residual[(size_t)t * p.n + row] + y;
                p.out[(size_t)t * p.n + row] = y;
            }
        }
    }
}

template <int M>
int32_t launch_iq4nl(const GemvArgs& a, cudaStream_t s) {
    GemvParams p;
    p.x = a.x; p.out = a.out; p.residual = a.residual; p.norm_w = a.norm_w; p.eps = a.eps;
    p.n = a.w->n; p.k = a.w->k; p.m = a.m; p.epi = (int)a.epi; p.error_flag = nullptr;
    int grid = (p.n + kWarps - 1) / kWarps;
    const int cap = sm_count() * 8;
    if (grid > cap) grid = cap;
    const uint8_t* w2 = a.w2 ? (const uint8_t*)a.w2->data : nullptr;
    LC_CUDA(launch_pdl(qgemv_iq4nl_kernel<M>, dim3(grid), dim3(kWarps * 32), 0, s, (const uint8_t*)a.w->data, w2, p));
    return LC_OK;
}

}  // namespace

int32_t launch_qgemv_kq(const GemvArgs& a, cudaStream_t s, bool* launched) {
    *launched = false;
    const uint32_t typ = a.w->typ;
    const bool kq = typ == LC_TYPE_Q6_K || typ == LC_TYPE_Q5_K, dense = typ == LC_TYPE_F16 || typ == LC_TYPE_F32, iq = typ == LC_TYPE_IQ4_NL;
    if ((!kq && !dense && !iq) || a.m < 1 || a.m > 8) return LC_OK;
    if (iq && (a.w->k % 32 != 0 || a.m > 2)) return LC_OK;  // a lane holds a whole block per matrix in registers: one or two tokens
    if (kq && a.w->k % 256 != 0) return LC_OK;
    if (dense && a.w->k % 8 != 0) return LC_OK;  // rows must stay 16-byte aligned and split into groups of eight
    if (((uintptr_t)a.x % 16) != 0 || (a.norm_w && ((uintptr_t)a.norm_w % 16) != 0)) return LC_OK;
    if (((uintptr_t)a.w->data % 16) != 0 || (a.w2 && ((uintptr_t)a.w2->data % 16) != 0)) return LC_OK;
    *launched = true;
    const int mt = a.m <= 1 ? 1 : (a.m <= 2 ? 2 : (a.m <= 4 ? 4 : 8));
#define KQ(T)                                                 \
    switch (mt) {                                             \
        case 1: return launch_kq<T, 1>(a, s);                 \
        case 2: return launch_kq<T, 2>(a, s);                 \
        case 4: return launch_kq<T, 4>(a, s);                 \
        default: return launch_kq<T, 8>(a, s);                \
    }
    if (typ == LC_TYPE_Q6_K) { KQ(LC_TYPE_Q6_K) }
    if (typ == LC_TYPE_Q5_K) { KQ(LC_TYPE_Q5_K) }
#undef KQ
#define DN(F)                                                 \
    switch (mt) {                                             \
        case 1: return launch_dense<F, 1>(a, s);              \
        case 2: return launch_dense<F, 2>(a, s);              \
        case 4: return launch_dense<F, 4>(a, s);              \
        default: return launch_dense<F, 8>(a, s);             \
    }
    if (typ == LC_TYPE_F32) { DN(true) }
    if (typ == LC_TYPE_F16) { DN(false) }
#undef DN
    return mt == 1 ? launch_iq4nl<1>(a, s) : launch_iq4nl<2>(a, s);
}

}  // namespace lc

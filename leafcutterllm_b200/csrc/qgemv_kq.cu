// Matrix-vector products over Q5_K and Q6_K weights (rust/src/kernels/mod.rs:101-180): the types a "Q4_K_M" or "Q5_K_M"
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

}  // namespace

int32_t launch_qgemv_kq(const GemvArgs& a, cudaStream_t s, bool* launched) {
    *launched = false;
    const uint32_t typ = a.w->typ;
    if ((typ != LC_TYPE_Q6_K && typ != LC_TYPE_Q5_K) || a.w->k % 256 != 0 || a.m < 1 || a.m > 8) return LC_OK;
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
    KQ(LC_TYPE_Q5_K)
#undef KQ
}

}  // namespace lc

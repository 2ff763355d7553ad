// Q6_K matrix-vector product on the integer tensor cores, exact in the integer domain.
//
//   y[t, r] = sum_k x[t, k] * w[r, k],   w = d * sc[k / 16] * (q - 32)      (rust/src/kernels/mod.rs:145-180)
//
// The arithmetic of the Q4_K kernel: the activations of a 256-element unit become 24-bit fixed point in three balanced
// byte planes, the 6-bit weights are unsigned bytes, and a 16-element sub-block (one int8 scale) is one
// mma.sync m16n8k16 u8 x s8 -> s32 with 16 weight rows as A and the planes of up to two tokens as the B columns.  The
// int8 scales multiply the int32 sums as integers; d and 2^-s are applied once per unit in f32.  The offset,
//   sum_sub sc[sub] * sum_k (q - 32) P[k] = sum_sub sc[sub] * (sum_k q P[k])  -  32 * sum_sub sc[sub] * S[sub],   S = sum of P over the sub-block,
// is a product of its own: the sixteen scales of a row are the A bytes of one more MMA against the sub-block sums of
// every plane (|S| <= 2048: two balanced byte digits, two MMAs per unit), written once per unit beside the planes.
//
// Data path.  A Q6_K block has 210 bytes, so nothing of a row is 16-byte aligned and no tensor-map box describes a
// [unit x rows] tile.  A warp owns a unit of k; per 16-row tile it copies, for every row, the fourteen 16-byte pieces that
// cover the row's block (cp.async, three or two tiles in flight per warp), so that a block lies in shared memory at the
// offset its address has from a 16-byte boundary: always even, and words are read as two aligned 32-bit loads and a
// funnel shift.  Element e = 128 n + 32 j + l of a block has its low four bits in nibble j / 2 of ql[64 n + 32 (j & 1) + l]
// and its high two at bit 2 j of qh[32 n + l]; thread t of a row's four takes l = 4t .. 4t + 3 and 16 + 4t .. of every
// (n, j): twelve words per row and unit, each byte of the block read once.
#include <algorithm>
#include <cstdlib>
#include "lc_kernels.h"
#include "lc_planes.cuh"
#include "lc_quant.cuh"
#include "lc_tma.cuh"

namespace lc {

namespace {

constexpr int kUB = 210;                        // bytes of a row's 256 weights
constexpr int kRows = 16;                       // rows per tile: one MMA row group
constexpr int kPieces = 14;                     // 16-byte pieces per row and unit: the block plus its offset from a 16-byte boundary (<= 14)
constexpr int kPitch = 240;                     // bytes between the rows of a stage (60 words: eight rows start in eight different banks)
constexpr int kStageBytes = kRows * kPitch;
static_assert(2 * kPieces <= 32 && kRows % 2 == 0, "a warp instruction copies the pieces of two rows");

__device__ __forceinline__ void mma_s8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0), "r"(0), "r"(0), "r"(0));
}
__device__ __forceinline__ void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0), "r"(0), "r"(0), "r"(0));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t lds32(const unsigned char* p) { return *reinterpret_cast<const uint32_t*>(p); }
// the word at byte offset o (a multiple of 4) of a block whose start is base + (0 or 2): base is word aligned, sh = 0 or 16
__device__ __forceinline__ uint32_t block_word(const unsigned char* base, int sh, int o) {
    return __funnelshift_r(lds32(base + o), lds32(base + o + 4), sh);
}
// byte b of w, sign extended: a byte permute whose selector asks for the byte's sign in the three upper positions
__device__ __forceinline__ int sbyte(uint32_t w, int b) {
    uint32_t r;
    const uint32_t sel = ((8u | b) << 12) | ((8u | b) << 8) | ((8u | b) << 4) | (uint32_t)b;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0), "r"(sel));
    return (int)r;
}

// planes of one unit: [sub-block 8][token M][plane 3][32 bytes]
template <int M>
__device__ __forceinline__ int plane_off(int unit, int sb, int tok, int plane) {
    return ((unit * 8 + sb) * M + tok) * 96 + plane * 32;
}

// w0 / w1: the matrix (and `up` for EPI_SILU_MUL), rows of k / 256 blocks; n is a multiple of 16 and both are 16-byte aligned.
template <int M, int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32, 1)
qgemv_mma_q6k_kernel(const unsigned char* __restrict__ w0, const unsigned char* __restrict__ w1, GemvParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int NPAIR = (M + 1) / 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int nunits = p.k / kUnitElems;
    const int ntiles = p.n / kRows;
    const int nmat = (p.epi == EPI_SILU_MUL) ? 2 : 1;
    const int m_act = p.m;
    const size_t row_bytes = (size_t)nunits * kUB;
    const size_t total = (size_t)p.n * row_bytes;  // a multiple of 16: no piece that starts inside the matrix ends outside

    unsigned char* stage_base = smem + (size_t)warp * STAGES * kStageBytes;
    size_t off = (size_t)WARPS * STAGES * kStageBytes;
    unsigned char* planes = smem + off;                       // [nunits][8][M][3][32] int8
    off += (size_t)nunits * 8 * M * 96;
    unsigned char* ssum = smem + off;                         // [nunits][token pair][digit 2][column 8][sub-block 16] int8
    off += (size_t)nunits * NPAIR * 256;
    float* inv2s = reinterpret_cast<float*>(smem + off);      // [nunits][M]: 2^-s
    off += (size_t)nunits * M * 4;
    float* red = reinterpret_cast<float*>(smem + off);        // [2][WARPS][M][16]
    off += (size_t)2 * WARPS * M * kRows * 4;
    float* gate_vals = reinterpret_cast<float*>(smem + off);  // [M][16]
    off += (size_t)M * kRows * 4;
    float* scratch = reinterpret_cast<float*>(smem + off);    // [32 + M]

    const int units_mine = (nunits > warp) ? (nunits - warp + WARPS - 1) / WARPS : 0;
    const int tiles_mine = (ntiles > (int)blockIdx.x) ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int njobs = tiles_mine * nmat * units_mine;

    // byte offset of (first row of this CTA's tile ti, unit ui of this warp) in the matrix
    auto job_start = [&](int ti, int ui) -> size_t {
        return (size_t)(blockIdx.x + ti * gridDim.x) * kRows * row_bytes + (size_t)(warp + ui * WARPS) * kUB;
    };
    // producer cursor: the next job to request (all lanes; every call commits one group, an empty one past the last job,
    // so that "all but the newest STAGES - 1 groups" always means "the job about to be read")
    int pj = 0, p_ti = 0, p_mat = 0, p_ui = 0, p_st = 0;
    const int c_row = lane >= kPieces ? 1 : 0, c_piece = lane - kPieces * c_row;
    auto issue_next = [&]() {
        if (pj < njobs) {
            const unsigned char* wm = p_mat ? w1 : w0;
            const size_t b0 = job_start(p_ti, p_ui);
            // two rows per instruction: lanes 0-13 the pieces of an even row, lanes 14-27 those of the next
            if (lane < 2 * kPieces) {
                const uint32_t dst0 = smem_u32(stage_base + (size_t)p_st * kStageBytes) + (uint32_t)(c_row * kPitch + 16 * c_piece);
                size_t at = b0 + (size_t)c_row * row_bytes;
#pragma unroll
                for (int i = 0; i < kRows / 2; i++, at += 2 * row_bytes) {
                    const size_t src = (at & ~(size_t)15) + (size_t)(16 * c_piece);
                    if (src < total) cp_async16(dst0 + (uint32_t)(2 * i * kPitch), wm + src);
                }
            }
            pj++;
            if (++p_st == STAGES) p_st = 0;
            if (++p_ui == units_mine) {
                p_ui = 0;
                if (++p_mat == nmat) { p_mat = 0; ++p_ti; }
            }
        }
        cp_async_commit();
    };
    for (int j = 0; j < STAGES; j++) issue_next();  // weights do not depend on the kernel ahead
    pdl_launch_dependents();
    pdl_wait();

    // ---- RMS-norm scale per token (cpu.rs:49-60) when fused ----
    if (p.norm_w) {
        for (int tk = 0; tk < M; tk++) {
            float ss = 0.f;
            if (tk < m_act) {
                const float* xr = p.x + (size_t)tk * p.k;
                for (int i = threadIdx.x; i < p.k; i += blockDim.x) { const float v = xr[i]; ss = fmaf(v, v, ss); }
            }
            ss = warp_sum(ss);
            __syncthreads();
            if (lane == 0) scratch[warp] = ss;
            __syncthreads();
            if (warp == 0) {
                float r = (lane < WARPS) ? scratch[lane] : 0.f;
                r = warp_sum(r);
                if (lane == 0) scratch[32 + tk] = 1.0f / sqrtf(r / (float)p.k + p.eps);
            }
        }
        __syncthreads();
    }
    // ---- each warp writes the fixed-point planes of its own units ----
    for (int ui = 0; ui < units_mine; ui++) {
        const int unit = warp + ui * WARPS;
        const int e0 = unit * kUnitElems + 8 * lane;
#pragma unroll
        for (int tk = 0; tk < M; tk++) {
            float v[8];
            if (tk < m_act) {
                const float4* xp = reinterpret_cast<const float4*>(p.x + (size_t)tk * p.k + e0);
                const float4 u0 = xp[0], u1 = xp[1];
                v[0] = u0.x; v[1] = u0.y; v[2] = u0.z; v[3] = u0.w; v[4] = u1.x; v[5] = u1.y; v[6] = u1.z; v[7] = u1.w;
                if (p.norm_w) {
                    const float sc = scratch[32 + tk];
                    const float4* np = reinterpret_cast<const float4*>(p.norm_w + e0);
                    const float4 n0 = np[0], n1 = np[1];
                    const float nw[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] = (v[j] * sc) * nw[j];
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = 0.f;
            }
            unit_planes(v, lane, planes + plane_off<M>(unit, 0, tk, 0), M * 96, nullptr, inv2s + unit * M + tk);
        }
        __syncwarp();
        // the sums of every plane over the sixteen 16-element sub-blocks, as two balanced byte digits: column 3 (tk & 1) + plane
        // of pair tk / 2; columns 6 and 7 stay unread
        for (int i = lane; i < M * 3 * 16; i += 32) {
            const int tk = i / 48, pl = (i >> 4) % 3, is = i & 15;
            const uint32_t* pp = reinterpret_cast<const uint32_t*>(planes + plane_off<M>(unit, is >> 1, tk, pl) + 16 * (is & 1));
            int sum = 0;
#pragma unroll
            for (int q = 0; q < 4; q++) sum = __dp4a((int)pp[q], 0x01010101, sum);
            const int lo = (int)(signed char)sum, hi = (sum - lo) >> 8;
            unsigned char* sp = ssum + (size_t)(unit * NPAIR + (tk >> 1)) * 256 + (3 * (tk & 1) + pl) * 16 + is;
            sp[0] = (unsigned char)lo;
            sp[128] = (unsigned char)hi;
        }
    }
    __syncwarp();

    // Thread t owns C columns 2t and 2t + 1.  Columns 0-2 carry the byte planes of the pair's first token, 3-5 those of
    // its second token.  Coefficients that fold this thread's two columns into each token:
    const float cA0 = (t == 0) ? 1.f : (t == 1 ? 65536.f : 0.f), cA1 = (t == 0) ? 256.f : 0.f;
    const float cB0 = (t == 2) ? 256.f : 0.f, cB1 = (t == 1) ? 1.f : (t == 2 ? 65536.f : 0.f);
    // B fragment source of this thread: column g = lane / 4
    const int bcol_tok = (g >= 3) ? 1 : 0, bcol_pl = (g >= 3) ? g - 3 : g;

    // B fragments of a unit: per 32-element sub-block the plane bytes of elements 4t .. 4t + 3 and 16 + 4t ..
    uint32_t bf[NPAIR][8][2], bs[NPAIR][2];  // bs: the two digits of the sums of sub-blocks 4t .. 4t + 3 in this thread's column
    float isv[M];
    auto load_unit_consts = [&](int unit) {
#pragma unroll
        for (int pr = 0; pr < NPAIR; pr++) {
            const int tok = 2 * pr + bcol_tok;
            const bool colv = g < 6 && tok < M;
            const unsigned char* bp = planes + plane_off<M>(unit, 0, colv ? tok : 0, bcol_pl > 2 ? 0 : bcol_pl) + 4 * t;
#pragma unroll
            for (int sb = 0; sb < 8; sb++) {
                const uint32_t v0 = lds32(bp + sb * (M * 96)), v1 = lds32(bp + sb * (M * 96) + 16);
                bf[pr][sb][0] = colv ? v0 : 0u;
                bf[pr][sb][1] = colv ? v1 : 0u;
            }
            const unsigned char* sp = ssum + (size_t)(unit * NPAIR + pr) * 256 + (colv ? g : 0) * 16 + 4 * t;
            const uint32_t s0 = lds32(sp), s1 = lds32(sp + 128);
            bs[pr][0] = colv ? s0 : 0u;
            bs[pr][1] = colv ? s1 : 0u;
        }
#pragma unroll
        for (int tk = 0; tk < M; tk++) isv[tk] = inv2s[unit * M + tk];
    };
    const bool single_unit = units_mine == 1;
    if (single_unit) load_unit_consts(warp);

    int st = 0, seq = 0;
    for (int ti = 0; ti < tiles_mine; ti++) {
        const int tile = blockIdx.x + ti * gridDim.x;
        for (int mat = 0; mat < nmat; mat++, seq++) {
            float yacc[2][M];  // [row g / g + 8][token]: this thread's part of the row sums (the 4 threads of a row are added once per tile)
#pragma unroll
            for (int b = 0; b < 2; b++)
#pragma unroll
                for (int c = 0; c < M; c++) yacc[b][c] = 0.f;

            for (int ui = 0; ui < units_mine; ui++) {
                if (!single_unit) load_unit_consts(warp + ui * WARPS);
                cp_async_wait<STAGES - 1>();
                __syncwarp();  // every lane's pieces of this job have landed
                const unsigned char* tilep = stage_base + (size_t)st * kStageBytes;
                const size_t b0 = job_start(ti, ui);
                const uint32_t skA = (uint32_t)((b0 + (size_t)g * row_bytes) & 15), skB = (uint32_t)((b0 + (size_t)(g + 8) * row_bytes) & 15);
                const unsigned char* pa = tilep + g * kPitch + (skA & 12u);
                const unsigned char* pb = tilep + (g + 8) * kPitch + (skB & 12u);
                const int sha = (int)(skA & 2u) * 8, shb = (int)(skB & 2u) * 8;
                uint32_t scA[4], scB[4];
#pragma unroll
                for (int i = 0; i < 4; i++) { scA[i] = block_word(pa, sha, 192 + 4 * i); scB[i] = block_word(pb, shb, 192 + 4 * i); }
                const float dA = __half2float(*reinterpret_cast<const __half*>(tilep + g * kPitch + skA + 208));
                const float dB = __half2float(*reinterpret_cast<const __half*>(tilep + (g + 8) * kPitch + skB + 208));
                int acc[NPAIR][4];
#pragma unroll
                for (int pr = 0; pr < NPAIR; pr++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[pr][j] = 0;
#pragma unroll
                for (int n = 0; n < 2; n++) {
                    uint32_t qlA[4], qlB[4], qhA[2], qhB[2];
#pragma unroll
                    for (int c = 0; c < 4; c++) { qlA[c] = block_word(pa, sha, 64 * n + 16 * c + 4 * t); qlB[c] = block_word(pb, shb, 64 * n + 16 * c + 4 * t); }
#pragma unroll
                    for (int h = 0; h < 2; h++) { qhA[h] = block_word(pa, sha, 128 + 32 * n + 16 * h + 4 * t); qhB[h] = block_word(pb, shb, 128 + 32 * n + 16 * h + 4 * t); }
#pragma unroll
                    for (int j = 0; j < 4; j++) {
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const int c = (j & 1) * 2 + h;
                            const uint32_t loA = (qlA[c] >> (4 * (j >> 1))) & 0x0F0F0F0Fu, loB = (qlB[c] >> (4 * (j >> 1))) & 0x0F0F0F0Fu;
                            const uint32_t hiA = (j < 2 ? (qhA[h] << (4 - 2 * j)) : (qhA[h] >> (2 * j - 4))) & 0x30303030u;
                            const uint32_t hiB = (j < 2 ? (qhB[h] << (4 - 2 * j)) : (qhB[h] >> (2 * j - 4))) & 0x30303030u;
                            const uint32_t a0 = loA | hiA, a1 = loB | hiB;  // q, 0 .. 63
                            const int is = 8 * n + 2 * j + h;
                            const int sA = sbyte(scA[is >> 2], is & 3), sB = sbyte(scB[is >> 2], is & 3);
#pragma unroll
                            for (int pr = 0; pr < NPAIR; pr++) {
                                int cc[4];
                                mma_u8s8_k16(cc, a0, a1, bf[pr][4 * n + j][h]);
                                acc[pr][0] += sA * cc[0]; acc[pr][1] += sA * cc[1]; acc[pr][2] += sB * cc[2]; acc[pr][3] += sB * cc[3];
                            }
                        }
                    }
                }
                // ---- the offset: -32 sum_sub sc[sub] S[sub]; this thread's A bytes are the scales of sub-blocks 4t .. 4t + 3 ----
                const uint32_t sa = t == 0 ? scA[0] : (t == 1 ? scA[1] : (t == 2 ? scA[2] : scA[3]));
                const uint32_t sb_ = t == 0 ? scB[0] : (t == 1 ? scB[1] : (t == 2 ? scB[2] : scB[3]));
#pragma unroll
                for (int pr = 0; pr < NPAIR; pr++) {
                    int c0[4], c1[4];
                    mma_s8s8_k16(c0, sa, sb_, bs[pr][0]);
                    mma_s8s8_k16(c1, sa, sb_, bs[pr][1]);
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[pr][j] -= 32 * (c0[j] + 256 * c1[j]);
                }
                // ---- fold planes and scales into this thread's f32 partial row sums ----
#pragma unroll
                for (int pr = 0; pr < NPAIR; pr++) {
                    const float v0 = (float)acc[pr][0], v1 = (float)acc[pr][1], v2 = (float)acc[pr][2], v3 = (float)acc[pr][3];
#pragma unroll
                    for (int which = 0; which < 2; which++) {  // first / second token of the pair
                        const int tok = 2 * pr + which;
                        if (tok >= M) continue;
                        const float c0 = which ? cB0 : cA0, c1 = which ? cB1 : cA1;
                        yacc[0][tok] = fmaf(dA * isv[tok], c0 * v0 + c1 * v1, yacc[0][tok]);
                        yacc[1][tok] = fmaf(dB * isv[tok], c0 * v2 + c1 * v3, yacc[1][tok]);
                    }
                }
                __syncwarp();  // every lane has read the stage
                if (++st == STAGES) st = 0;
                issue_next();
            }
            // add the four threads that share a row (fixed order)
#pragma unroll
            for (int b = 0; b < 2; b++)
#pragma unroll
                for (int c = 0; c < M; c++) {
                    float v = yacc[b][c];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    yacc[b][c] = v;
                }
            // ---- cross-warp reduction of this (tile, matrix), in warp order ----
            float* rb = red + (size_t)(seq & 1) * WARPS * M * kRows;
            if (t == 0) {
#pragma unroll
                for (int tk = 0; tk < M; tk++) {
                    rb[(warp * M + tk) * kRows + g] = yacc[0][tk];
                    rb[(warp * M + tk) * kRows + g + 8] = yacc[1][tk];
                }
            }
            __syncthreads();
            if (warp < M && lane < kRows) {
                const int tk = warp;
                float y = 0.f;
#pragma unroll 4
                for (int w = 0; w < WARPS; w++) y += rb[(w * M + tk) * kRows + lane];
                const int row = tile * kRows + lane;
                bool have = false;
                if (p.epi == EPI_SILU_MUL) {
                    if (mat == 0) {
                        gate_vals[tk * kRows + lane] = y;
                    } else if (tk < m_act) {
                        y = silu_f(gate_vals[tk * kRows + lane]) * y;
                        have = true;
                    }
                } else if (tk < m_act) {
                    if (p.epi == EPI_ADD_RESIDUAL) y = p.residual[(size_t)tk * p.n + row] + y;
                    have = true;
                }
                if (have) p.out[(size_t)tk * p.n + row] = y;
            }
        }
    }
    cp_async_wait<0>();
}

template <int M, int WARPS, int STAGES>
size_t q6k_smem_bytes(int k) {
    const int nunits = k / kUnitElems;
    size_t b = (size_t)WARPS * STAGES * kStageBytes;
    b += (size_t)nunits * 8 * M * 96 + (size_t)nunits * ((M + 1) / 2) * 256 + (size_t)nunits * M * 4;
    b += (size_t)2 * WARPS * M * kRows * 4 + (size_t)M * kRows * 4 + (size_t)(32 + M) * 4;
    return b;
}

template <int M, int WARPS, int STAGES>
int32_t launch_cfg(const GemvArgs& a, cudaStream_t s) {
    auto kern = qgemv_mma_q6k_kernel<M, WARPS, STAGES>;
    const size_t smem = q6k_smem_bytes<M, WARPS, STAGES>(a.w->k);
    LC_CUDA(ensure_smem_limit((const void*)kern, kMaxSmem));
    GemvParams p;
    p.x = a.x; p.out = a.out; p.residual = a.residual; p.norm_w = a.norm_w; p.eps = a.eps;
    p.n = a.w->n; p.k = a.w->k; p.m = a.m; p.epi = (int)a.epi; p.error_flag = nullptr;
    // the same number of tiles for every CTA of the slowest wave
    const int ntiles = p.n / kRows;
    const int waves = (ntiles + sm_count() - 1) / sm_count();
    const int grid = (ntiles + waves - 1) / waves;
    const unsigned char* w0 = (const unsigned char*)a.w->data;
    const unsigned char* w1 = a.w2 ? (const unsigned char*)a.w2->data : w0;
    LC_CUDA(launch_pdl(kern, dim3(grid), dim3(WARPS * 32), smem, s, w0, w1, p));
    return LC_OK;
}

template <int M>
int32_t launch_m(const GemvArgs& a, cudaStream_t s, bool* launched) {
    const int k = a.w->k;
    *launched = true;
    if (q6k_smem_bytes<M, 16, 3>(k) <= kMaxSmem) return launch_cfg<M, 16, 3>(a, s);
    if (q6k_smem_bytes<M, 16, 2>(k) <= kMaxSmem) return launch_cfg<M, 16, 2>(a, s);
    if (q6k_smem_bytes<M, 8, 3>(k) <= kMaxSmem) return launch_cfg<M, 8, 3>(a, s);
    if (q6k_smem_bytes<M, 8, 2>(k) <= kMaxSmem) return launch_cfg<M, 8, 2>(a, s);
    *launched = false;
    return LC_OK;
}

}  // namespace

// true when launch_qgemv_mma_q6k would run these arguments with m tokens
bool qgemv_mma_q6k_supports(const GemvArgs& a, int m) {
    static const bool plain = getenv("LC_GEMV_Q6K_PLAIN") != nullptr;
    const QWeight* w = a.w;
    if (plain || !w || w->typ != LC_TYPE_Q6_K || a.group || a.push || m < 1 || m > 4) return false;
    if (w->k <= 0 || w->k % kUnitElems != 0 || w->n <= 0 || w->n % kRows != 0) return false;
    if (((uintptr_t)w->data % 16) != 0 || ((uintptr_t)a.x % 16) != 0 || (a.norm_w && ((uintptr_t)a.norm_w % 16) != 0)) return false;
    if (a.epi == EPI_SILU_MUL && (!a.w2 || ((uintptr_t)a.w2->data % 16) != 0)) return false;
    if (m <= 1) return q6k_smem_bytes<1, 8, 2>(w->k) <= kMaxSmem;
    if (m <= 2) return q6k_smem_bytes<2, 8, 2>(w->k) <= kMaxSmem;
    return q6k_smem_bytes<4, 8, 2>(w->k) <= kMaxSmem;
}

// Q6_K rows of whole 256-element blocks, a multiple of 16 rows, up to four tokens; *launched = false otherwise (the plain-load
// kernel takes those) and when LC_GEMV_Q6K_PLAIN is set.
int32_t launch_qgemv_mma_q6k(const GemvArgs& a, cudaStream_t s, bool* launched) {
    *launched = false;
    if (!qgemv_mma_q6k_supports(a, a.m)) return LC_OK;
    if (a.m <= 1) return launch_m<1>(a, s, launched);
    if (a.m <= 2) return launch_m<2>(a, s, launched);
    return launch_m<4>(a, s, launched);
}

}  // namespace lc

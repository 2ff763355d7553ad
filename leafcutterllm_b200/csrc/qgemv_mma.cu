// Q4_K matrix-vector product on the integer tensor cores, exact in the integer domain.
//
//   y[t, r] = sum_k x[t, k] * w[r, k],   w = (d * sc) * q - (dmin * m)      (rust/src/kernels/mod.rs:66-98)
//
// The reference multiplies f32 activations with the dequantised f32 weight.  Here the f32
// activations of each 256-element unit are first written as 24-bit fixed point against the
// unit's own power-of-two scale, X = round(x * 2^s), |X| < 2^23, split into three balanced
// byte planes X = P0 + 256 P1 + 65536 P2.  Then
//   sum_k x_k q_k = 2^-s * sum_p 256^p * sum_k P_p[k] q[k]
// and the inner sums are int8 x uint8 products accumulated in int32 -- mma.sync m16n8k32 with the
// 4-bit weights as the A operand (16 rows x 32 k = one Q4_K sub-block) and the planes of up to two
// tokens as the 8 B columns.  Integer arithmetic is exact and order independent; the 6-bit
// sub-block scales are applied as integer multiplies, so the only roundings are the 2^-24 fixed
// point of x (relative to the unit's largest |x|) and the final f32 conversion.
//
// Data path: the same TMA-staged [144 B x 32 rows] boxes as the f32 kernel; warp <-> unit, a thread
// holds the A fragments of rows g and g+8 (g = lane / 4) as two 32-bit shared-memory loads per
// 64-element group (bank-conflict free for the 144-byte row pitch).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include "lc_kernels.h"
#include "lc_planes.cuh"
#include "lc_quant.cuh"
#include "lc_tma.cuh"

namespace lc {

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

__device__ __forceinline__ void mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

// bytes of a row's 256 weights
__host__ __device__ constexpr int mma_unit_bytes(uint32_t typ) { return typ == LC_TYPE_Q8_0 ? 272 : (typ == LC_TYPE_Q5_K ? 176 : 144); }

__device__ __forceinline__ uint32_t lds32(const unsigned char* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ int byte_of(uint32_t w, int j) { return (int)((w >> (8 * j)) & 0xFFu); }

// planes of one unit: [sub-block 8][token M][plane 3][32 bytes]
constexpr int kGroupedSlots = 64;  // most slots one expert of a grouped launch can receive

template <int M>
__device__ __forceinline__ int plane_off(int unit, int sb, int tok, int plane) {
    return ((unit * 8 + sb) * M + tok) * 96 + plane * 32;
}

// GROUPED: one launch over the experts of a mixture-of-experts layer.  blockIdx.y = expert; the CTA reads how many
// slots the router sent to its expert (leaving at once when none), takes the expert's tensor maps from a device array and
// walks its tiles; per tile it makes one pass per M slots, re-requesting the tile's boxes (L2 hits) for the later passes,
// and writes each result row to its slot.  The activations come as fixed-point planes that gemv_planes_kernel wrote once
// for the whole launch, read per job from global memory (L2): no per-CTA norm or plane computation, and no shared memory
// that grows with k.  The plain instantiation carries none of this.
//
// TYPE = LC_TYPE_Q4_0: the same tiles (eight 18-byte blocks = 144 bytes per 256 weights), the same planes.  A block is one
// MMA: the 4 bytes a thread needs hold its low-nibble k-slots and, four bits up, its high-nibble ones (elements j and j + 16
// share byte j, rust/src/kernels/mod.rs:26-31); the block's f16 scale multiplies the plane-folded sum in f32 and the
// offset -8 d sum(x) is shared out over the four threads of a row like the min term of Q4_K.
// TYPE = LC_TYPE_Q8_0: eight 34-byte blocks = 272 bytes per 256 weights; a block is one s8 x s8 MMA (the weights are the
// signed bytes themselves, mod.rs:47-49), no offset.
// TYPE = LC_TYPE_Q5_K: a Q4_K block with the elements' fifth bits between the header and the nibbles (176 bytes; bit s of
// qh[l] belongs to element l of sub-block s, mod.rs:101-143): the A bytes are nibble | bit << 4, high nibbles moved down.
template <int M, int WARPS, int STAGES, bool GROUPED = false, uint32_t TYPE = LC_TYPE_Q4_K>
__global__ void __launch_bounds__(WARPS * 32, (WARPS <= 8 && M <= 2) ? 2 : 1)
qgemv_mma_q4k_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, GemvParams p, GemvGroupParams gp) {
    constexpr int UB = mma_unit_bytes(TYPE);  // bytes of a row's 256 weights
    const CUtensorMap* t0p = &tm0;
    const CUtensorMap* t1p = &tm1;
    int m_act = p.m;
    extern __shared__ __align__(128) unsigned char smem[];
    int* s_slot = reinterpret_cast<int*>(smem);  // GROUPED: the first 256 bytes of shared memory hold the expert's slots
    int cnt = 0, npass = 1, pass = 0;
    if constexpr (GROUPED) {
        pdl_launch_dependents();
        pdl_wait();  // the router's counts and lists and the planes come from the kernels ahead
        const int e = blockIdx.y;
        cnt = min(gp.cnt[e], min(gp.list_stride, kGroupedSlots));
        if (cnt <= 0) return;
        npass = (cnt + M - 1) / M;
        t0p = gp.tm0 + e;
        t1p = gp.tm1 + e;
        if ((int)threadIdx.x < cnt) s_slot[threadIdx.x] = gp.list[(size_t)e * gp.list_stride + threadIdx.x];
        __syncthreads();
    }
    // row of x / of out that token slot tk of this CTA reads / writes
    auto xrow = [&](int tk) -> const float* { return p.x + (size_t)tk * p.k; };
    auto orow = [&](int tk) -> size_t {
        if constexpr (GROUPED) return (size_t)s_slot[pass * M + tk] * p.n;
        else return (size_t)tk * p.n;
    };
    constexpr int RG = 2;        // 16-row MMA groups per tile
    constexpr int TR = 16 * RG;  // rows per tile
    constexpr int STAGE_BYTES = UB * TR;
    constexpr int NPAIR = (M + 1) / 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int nunits = p.k / kUnitElems;
    const int ntiles = (p.n + TR - 1) / TR;
    const int nmat = (p.epi == EPI_SILU_MUL) ? 2 : 1;

    auto gtime = [] { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; };
    unsigned long long* rg = nullptr;
    if (p.ring && threadIdx.x == 0) {
        atomicMax(p.ring + 7, gtime());  // the last CTA to start
        if (blockIdx.x == 0) { rg = p.ring; rg[0] = gtime(); rg[5] = ((unsigned long long)p.n << 32) | (unsigned)p.k; }
    }
    constexpr size_t kHead = GROUPED ? kGroupedSlots * 4 : 0;  // keeps the stages 128-byte aligned behind the slots
    unsigned char* stage_base = smem + kHead + (size_t)warp * STAGES * STAGE_BYTES;
    size_t off = kHead + (size_t)WARPS * STAGES * STAGE_BYTES;
    const int nu_s = GROUPED ? 0 : nunits;                       // GROUPED reads the planes from global memory
    unsigned char* planes = smem + off;                          // [nunits][8][M][3][32] int8
    off += (size_t)nu_s * 8 * M * 96;
    float* sxf = reinterpret_cast<float*>(smem + off);           // [nunits][M][8]: sum of x over each sub-block
    off += (size_t)nu_s * M * 8 * 4;
    float* inv2s = reinterpret_cast<float*>(smem + off);         // [nunits][M]: 2^-s
    off += (size_t)nu_s * M * 4;
    float* red = reinterpret_cast<float*>(smem + off);           // [2][WARPS][M][32]
    off += (size_t)2 * WARPS * M * 32 * 4;
    float* gate_vals = reinterpret_cast<float*>(smem + off);     // [M][32]
    off += (size_t)M * 32 * 4;
    float* scratch = reinterpret_cast<float*>(smem + off);       // [32 + M]
    off += (size_t)(32 + M) * 4;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ((off + 7) & ~(size_t)7)) + warp * STAGES;

    const int units_mine = (nunits > warp) ? (nunits - warp + WARPS - 1) / WARPS : 0;
    const int tiles_mine = (ntiles > (int)blockIdx.x) ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int njobs = tiles_mine * npass * units_mine * nmat;

    // producer cursor (lane 0): the next job to request, walked without divisions
    int pj = 0, p_ti = 0, p_pass = 0, p_mat = 0, p_ui = 0;
    auto issue_next = [&]() {
        const int st = pj & (STAGES - 1);
        mbar_expect_tx(&bars[st], STAGE_BYTES);
        tma_load_2d(stage_base + (size_t)st * STAGE_BYTES, p_mat ? t1p : t0p, (warp + p_ui * WARPS) * (UB / 4),
                    (blockIdx.x + p_ti * gridDim.x) * TR, &bars[st]);
        pj++;
        if (++p_ui == units_mine) {
            p_ui = 0;
            if (++p_mat == nmat) {
                p_mat = 0;
                if (++p_pass == npass) { p_pass = 0; ++p_ti; }
            }
        }
    };

    if (lane == 0) {
        for (int s = 0; s < STAGES; s++) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int j = 0; j < STAGES && j < njobs; j++) issue_next();  // weights do not depend on the previous kernel
    }
    // One token whose k fits one or two units per warp: each warp reads its own elements ONCE, for the sum of squares and for
    // the planes, and the gains of its first unit (weights: no dependency on the kernel ahead) are already in registers by then.
    const bool one_pass = !GROUPED && (M == 1) && p.norm_w != nullptr && nunits <= 2 * WARPS;
    float nw0[8];
    if (one_pass && warp < nunits) {
        const float4* np = reinterpret_cast<const float4*>(p.norm_w + warp * kUnitElems + 8 * lane);
        const float4 n0 = np[0], n1 = np[1];
        nw0[0] = n0.x; nw0[1] = n0.y; nw0[2] = n0.z; nw0[3] = n0.w; nw0[4] = n1.x; nw0[5] = n1.y; nw0[6] = n1.z; nw0[7] = n1.w;
    }
    if constexpr (!GROUPED) {
        pdl_launch_dependents();
        pdl_wait();
    }
    if (rg) rg[1] = gtime();
    // rows that are this rank's share of a sum over the ranks: the number of that sum (stable: the kernel ahead has finished)
    const unsigned push_e = p.push.world > 0 ? *p.push.epoch + 1u : 0u;

    // ---- RMS-norm scale per token (cpu.rs:49-60) when fused ----
    float v0[8], v1[8];
    float rms0 = 1.f;
    if (one_pass) {
        float ss = 0.f;
        if (warp < nunits) {
            const int e0 = warp * kUnitElems + 8 * lane;
            const float4* xp = reinterpret_cast<const float4*>(xrow(0) + e0);
            const float4 u0 = xp[0], u1 = xp[1];
            v0[0] = u0.x; v0[1] = u0.y; v0[2] = u0.z; v0[3] = u0.w; v0[4] = u1.x; v0[5] = u1.y; v0[6] = u1.z; v0[7] = u1.w;
#pragma unroll
            for (int j = 0; j < 8; j++) ss = fmaf(v0[j], v0[j], ss);
        }
        if (warp + WARPS < nunits) {  // the warp's second unit
            const int e0 = (warp + WARPS) * kUnitElems + 8 * lane;
            const float4* xp = reinterpret_cast<const float4*>(xrow(0) + e0);
            const float4 u0 = xp[0], u1 = xp[1];
            v1[0] = u0.x; v1[1] = u0.y; v1[2] = u0.z; v1[3] = u0.w; v1[4] = u1.x; v1[5] = u1.y; v1[6] = u1.z; v1[7] = u1.w;
#pragma unroll
            for (int j = 0; j < 8; j++) ss = fmaf(v1[j], v1[j], ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) scratch[warp] = ss;
        // No barrier here: the planes are those of x * gain, and the RMS factor -- one scalar for the whole row -- multiplies
        // the finished row sums behind the barrier of the cross-warp reduction, where every warp's part of the sum of
        // squares is visible.  A unit's power-of-two scale follows its own largest magnitude, so it does not care.
    } else if (!GROUPED && p.norm_w) {
        for (int tk = 0; tk < M; tk++) {
            float ss = 0.f;
            if (tk < m_act) {
                const float* xr = xrow(tk);
                for (int i = threadIdx.x; i < p.k; i += blockDim.x) { float v = xr[i]; ss = fmaf(v, v, ss); }
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
    for (int ui = 0; ui < (GROUPED ? 0 : units_mine); ui++) {
        const int unit = warp + ui * WARPS;
#pragma unroll
        for (int tk = 0; tk < M; tk++) {
            float v[8];
            const int e0 = unit * kUnitElems + 8 * lane;
            if (one_pass) {
                if (ui == 0) {
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] = (v0[j] * rms0) * nw0[j];
                } else {
                    const float4* np = reinterpret_cast<const float4*>(p.norm_w + e0);
                    const float4 n0 = np[0], n1 = np[1];
                    const float nw[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] = (v1[j] * rms0) * nw[j];
                }
            } else if (tk < m_act) {
                const float4* xp = reinterpret_cast<const float4*>(xrow(tk) + e0);
                float4 u0 = xp[0], u1 = xp[1];
                v[0] = u0.x; v[1] = u0.y; v[2] = u0.z; v[3] = u0.w; v[4] = u1.x; v[5] = u1.y; v[6] = u1.z; v[7] = u1.w;
                if (p.norm_w) {
                    const float sc = scratch[32 + tk];
                    const float4* np = reinterpret_cast<const float4*>(p.norm_w + e0);
                    float4 n0 = np[0], n1 = np[1];
                    const float nw[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] = (v[j] * sc) * nw[j];
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = 0.f;
            }
            unit_planes(v, lane, planes + plane_off<M>(unit, 0, tk, 0), M * 96, sxf + (unit * M + tk) * 8, inv2s + unit * M + tk);
        }
    }
    __syncwarp();
    if (rg) rg[2] = gtime();

    // Thread t owns B/C columns 2t and 2t+1.  Columns 0-2 carry the byte planes of the pair's first token,
    // 3-5 those of its second token.  Coefficients that fold this thread's two columns into each token:
    const float cA0 = (t == 0) ? 1.f : (t == 1 ? 65536.f : 0.f), cA1 = (t == 0) ? 256.f : 0.f;
    const float cB0 = (t == 2) ? 256.f : 0.f, cB1 = (t == 1) ? 1.f : (t == 2 ? 65536.f : 0.f);
    // B fragment source of this thread: column g = lane / 4
    const int bcol_tok = (g >= 3) ? 1 : 0, bcol_pl = (g >= 3) ? g - 3 : g;

    // GROUPED: row of the planes arrays that each token slot of the current pass reads (set at the start of a pass)
    int prow[M];
#pragma unroll
    for (int tk = 0; tk < M; tk++) prow[tk] = 0;
    auto load_bf = [&](int unit, uint32_t (&bf)[NPAIR][8][2]) {
#pragma unroll
        for (int pr = 0; pr < NPAIR; pr++) {
            const int tok = 2 * pr + bcol_tok;
            if constexpr (GROUPED) {
                const bool colv = g < 6 && tok < m_act;
                const int r = bcol_tok ? prow[(2 * pr + 1) < M ? 2 * pr + 1 : 0] : prow[2 * pr];
                const unsigned char* bp = gp.planes + (unsigned)(((colv ? r : 0) * nunits + unit) * 768 + (bcol_pl > 2 ? 0 : bcol_pl) * 32 + 4 * t);
#pragma unroll
                for (int sb = 0; sb < 8; sb++) {
                    const uint32_t v0 = __ldg(reinterpret_cast<const uint32_t*>(bp + sb * 96)), v1 = __ldg(reinterpret_cast<const uint32_t*>(bp + sb * 96 + 16));
                    bf[pr][sb][0] = colv ? v0 : 0u;
                    bf[pr][sb][1] = colv ? v1 : 0u;
                }
            } else {
                const bool colv = g < 6 && tok < M;
                const unsigned char* bp = planes + plane_off<M>(unit, 0, colv ? tok : 0, bcol_pl > 2 ? 0 : bcol_pl) + 4 * t;
#pragma unroll
                for (int sb = 0; sb < 8; sb++) {
                    const uint32_t v0 = lds32(bp + sb * (M * 96)), v1 = lds32(bp + sb * (M * 96) + 16);
                    bf[pr][sb][0] = colv ? v0 : 0u;
                    bf[pr][sb][1] = colv ? v1 : 0u;
                }
            }
        }
    };
    // B fragments: for each sub-block the plane bytes of k-slots 4t..4t+3 and 16+4t..; loaded once when the
    // warp owns a single unit of k, per job otherwise
    uint32_t bf[NPAIR][8][2];
    float sx2[M][2], isv[M];
    constexpr float kIsvFactor = TYPE == LC_TYPE_Q4_K ? 0.0625f : 1.0f;
    auto load_unit_consts = [&](int unit) {
        load_bf(unit, bf);
#pragma unroll
        for (int tk = 0; tk < M; tk++) {
            if constexpr (GROUPED) {
                const unsigned at = (unsigned)(prow[tk] * nunits + unit);
                const float2 sx = tk < m_act ? __ldg(reinterpret_cast<const float2*>(gp.sxf + at * 8 + 2 * t)) : make_float2(0.f, 0.f);
                sx2[tk][0] = sx.x;
                sx2[tk][1] = sx.y;
                isv[tk] = tk < m_act ? __ldg(gp.inv2s + at) * kIsvFactor : 0.f;
            } else {
                sx2[tk][0] = sxf[(unit * M + tk) * 8 + 2 * t];
                sx2[tk][1] = sxf[(unit * M + tk) * 8 + 2 * t + 1];
                isv[tk] = inv2s[unit * M + tk] * kIsvFactor;  // 2^-s and (Q4_K) the factor 16 the integer sums carry
            }
        }
    };
    const bool single_unit = !GROUPED && units_mine == 1;
    if (single_unit) load_unit_consts(warp);

    bool ok = true;
    int job = 0, seq = 0;
    for (int ti = 0; ti < tiles_mine; ti++) {
        const int tile = blockIdx.x + ti * gridDim.x;
        for (pass = 0; pass < npass; pass++) {
        if constexpr (GROUPED) {
            m_act = min(M, cnt - pass * M);
#pragma unroll
            for (int tk = 0; tk < M; tk++) {
                const int slot = s_slot[pass * M + (tk < m_act ? tk : 0)];
                prow[tk] = gp.x_by_token ? slot / gp.top_k : slot;
            }
        }
        for (int mat = 0; mat < nmat; mat++, seq++) {
            // per-thread partial row sums (the 4 threads of a row are added once per tile)
            float yacc[RG][2][M];  // [row group][row g / g+8][token]
#pragma unroll
            for (int a = 0; a < RG; a++)
#pragma unroll
                for (int b = 0; b < 2; b++)
#pragma unroll
                    for (int c = 0; c < M; c++) yacc[a][b][c] = 0.f;

            for (int ui = 0; ui < units_mine; ui++, job++) {
                const int st = job & (STAGES - 1);
                if (!single_unit) load_unit_consts(warp + ui * WARPS);
                ok = ok && mbar_wait(&bars[st], (uint32_t)((job / STAGES) & 1));
                const unsigned char* tilep = stage_base + (size_t)st * STAGE_BYTES;
                if constexpr (TYPE == LC_TYPE_Q8_0) {
#pragma unroll
                    for (int rg = 0; rg < RG; rg++) {
                        const unsigned char* rowA = tilep + (rg * 16 + g) * UB;
                        const unsigned char* rowB = rowA + 8 * UB;
#pragma unroll
                        for (int b = 0; b < 8; b++) {
                            // k-slots 4t .. 4t + 3 at 34 b + 2 + 4 t, k-slots 16 + 4t .. sixteen bytes on: word aligned for odd b
                            uint32_t a0, a1, a2, a3;
                            if (b & 1) {
                                a0 = lds32(rowA + 34 * b + 2 + 4 * t); a2 = lds32(rowA + 34 * b + 18 + 4 * t);
                                a1 = lds32(rowB + 34 * b + 2 + 4 * t); a3 = lds32(rowB + 34 * b + 18 + 4 * t);
                            } else {
                                a0 = __funnelshift_r(lds32(rowA + 34 * b + 4 * t), lds32(rowA + 34 * b + 4 + 4 * t), 16);
                                a2 = __funnelshift_r(lds32(rowA + 34 * b + 16 + 4 * t), lds32(rowA + 34 * b + 20 + 4 * t), 16);
                                a1 = __funnelshift_r(lds32(rowB + 34 * b + 4 * t), lds32(rowB + 34 * b + 4 + 4 * t), 16);
                                a3 = __funnelshift_r(lds32(rowB + 34 * b + 16 + 4 * t), lds32(rowB + 34 * b + 20 + 4 * t), 16);
                            }
                            const float dA = __half2float(*reinterpret_cast<const __half*>(rowA + 34 * b));
                            const float dB = __half2float(*reinterpret_cast<const __half*>(rowB + 34 * b));
#pragma unroll
                            for (int pr = 0; pr < NPAIR; pr++) {
                                int c[4];
                                mma_s8s8(c, a0, a1, a2, a3, bf[pr][b][0], bf[pr][b][1]);
                                const float v0 = (float)c[0], v1 = (float)c[1], v2 = (float)c[2], v3 = (float)c[3];
#pragma unroll
                                for (int which = 0; which < 2; which++) {
                                    const int tok = 2 * pr + which;
                                    if (tok >= M) continue;
                                    const float c0 = which ? cB0 : cA0, c1 = which ? cB1 : cA1;
                                    yacc[rg][0][tok] = fmaf(dA * isv[tok], c0 * v0 + c1 * v1, yacc[rg][0][tok]);
                                    yacc[rg][1][tok] = fmaf(dB * isv[tok], c0 * v2 + c1 * v3, yacc[rg][1][tok]);
                                }
                            }
                        }
                    }
                } else if constexpr (TYPE == LC_TYPE_Q4_0) {
#pragma unroll
                    for (int rg = 0; rg < RG; rg++) {
                        const unsigned char* rowA = tilep + (rg * 16 + g) * UB;
                        const unsigned char* rowB = rowA + 8 * UB;
#pragma unroll
                        for (int b = 0; b < 8; b++) {
                            // the four bytes of k-slots 4t .. 4t + 3 (low nibbles) and 16 + 4t .. (high nibbles): at 18 b + 2 + 4 t,
                            // word aligned for odd b, two bytes off for even b (two aligned words and a funnel shift)
                            uint32_t wA, wB;
                            if (b & 1) {
                                wA = lds32(rowA + 18 * b + 2 + 4 * t);
                                wB = lds32(rowB + 18 * b + 2 + 4 * t);
                            } else {
                                wA = __funnelshift_r(lds32(rowA + 18 * b + 4 * t), lds32(rowA + 18 * b + 4 + 4 * t), 16);
                                wB = __funnelshift_r(lds32(rowB + 18 * b + 4 * t), lds32(rowB + 18 * b + 4 + 4 * t), 16);
                            }
                            const float dA = __half2float(*reinterpret_cast<const __half*>(rowA + 18 * b));
                            const float dB = __half2float(*reinterpret_cast<const __half*>(rowB + 18 * b));
                            const uint32_t a0 = wA & 0x0F0F0F0Fu, a1 = wB & 0x0F0F0F0Fu, a2 = (wA >> 4) & 0x0F0F0F0Fu, a3 = (wB >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                            for (int pr = 0; pr < NPAIR; pr++) {
                                int c[4];
                                mma_u8s8(c, a0, a1, a2, a3, bf[pr][b][0], bf[pr][b][1]);
                                const float v0 = (float)c[0], v1 = (float)c[1], v2 = (float)c[2], v3 = (float)c[3];
#pragma unroll
                                for (int which = 0; which < 2; which++) {
                                    const int tok = 2 * pr + which;
                                    if (tok >= M) continue;
                                    const float c0 = which ? cB0 : cA0, c1 = which ? cB1 : cA1;
                                    yacc[rg][0][tok] = fmaf(dA * isv[tok], c0 * v0 + c1 * v1, yacc[rg][0][tok]);
                                    yacc[rg][1][tok] = fmaf(dB * isv[tok], c0 * v2 + c1 * v3, yacc[rg][1][tok]);
                                }
                            }
                            // (q - 8): this thread's share of -8 d sum(x) are blocks 2t and 2t + 1
                            if ((b >> 1) == t) {
#pragma unroll
                                for (int tok = 0; tok < M; tok++) {
                                    yacc[rg][0][tok] = fmaf(-8.0f * dA, sx2[tok][b & 1], yacc[rg][0][tok]);
                                    yacc[rg][1][tok] = fmaf(-8.0f * dB, sx2[tok][b & 1], yacc[rg][1][tok]);
                                }
                            }
                        }
                    }
                } else {
#pragma unroll
                for (int rg = 0; rg < RG; rg++) {
                    const unsigned char* rowA = tilep + (rg * 16 + g) * UB;
                    const unsigned char* rowB = rowA + 8 * UB;
                    const uint4 hA = *reinterpret_cast<const uint4*>(rowA);
                    const uint4 hB = *reinterpret_cast<const uint4*>(rowB);
                    uint32_t scA[2], mnA[2], scB[2], mnB[2];
                    unpack_scales_k4(hA.y, hA.z, hA.w, &scA[0], &scA[1], &mnA[0], &mnA[1]);
                    unpack_scales_k4(hB.y, hB.z, hB.w, &scB[0], &scB[1], &mnB[0], &mnB[1]);
                    // one int32 accumulator per C element: low-nibble products are scaled by 16*sc, high-nibble
                    // products (which carry a factor 16 because the nibble stays in place) by sc; Q5_K moves the high
                    // nibbles down to make room for the fifth bit, and both kinds are scaled by sc
                    constexpr bool Q5 = TYPE == LC_TYPE_Q5_K;
                    constexpr int QS = Q5 ? 48 : 16;  // where the nibbles start
                    uint32_t qhA0 = 0, qhA1 = 0, qhB0 = 0, qhB1 = 0;  // fifth bits of elements 4t .. 4t + 3 and 16 + 4t .. of every sub-block
                    if constexpr (Q5) {
                        qhA0 = lds32(rowA + 16 + 4 * t); qhA1 = lds32(rowA + 32 + 4 * t);
                        qhB0 = lds32(rowB + 16 + 4 * t); qhB1 = lds32(rowB + 32 + 4 * t);
                    }
                    int acc[NPAIR][4];
#pragma unroll
                    for (int pr = 0; pr < NPAIR; pr++)
#pragma unroll
                        for (int j = 0; j < 4; j++) acc[pr][j] = 0;
#pragma unroll
                    for (int grp = 0; grp < 4; grp++) {
                        const uint32_t wA0 = lds32(rowA + QS + 32 * grp + 4 * t), wA1 = lds32(rowA + QS + 16 + 32 * grp + 4 * t);
                        const uint32_t wB0 = lds32(rowB + QS + 32 * grp + 4 * t), wB1 = lds32(rowB + QS + 16 + 32 * grp + 4 * t);
                        const uint32_t swA = scA[grp >> 1], swB = scB[grp >> 1];
                        const int jl = (2 * grp) & 3;  // byte of the even sub-block in the packed scale word (0 or 2)
                        const int sAh = (int)__byte_perm(swA, 0, 0x4440 + jl + 1), sBh = (int)__byte_perm(swB, 0, 0x4440 + jl + 1);
                        int sAl, sBl;
                        uint32_t a0, a1, a2, a3, h0, h1, h2, h3;
                        if constexpr (Q5) {
                            sAl = (int)__byte_perm(swA, 0, 0x4440 + jl);
                            sBl = (int)__byte_perm(swB, 0, 0x4440 + jl);
                            // bit 2 grp (low nibbles' sub-block) and bit 2 grp + 1 (high nibbles') of every qh byte, moved to bit 4
                            auto lo5 = [&](uint32_t q) { return (grp < 2 ? (q << (4 - 2 * grp)) : (q >> (2 * grp - 4))) & 0x10101010u; };
                            auto hi5 = [&](uint32_t q) { return (grp < 2 ? (q << (3 - 2 * grp)) : (q >> (2 * grp - 3))) & 0x10101010u; };
                            a0 = (wA0 & 0x0F0F0F0Fu) | lo5(qhA0); a1 = (wB0 & 0x0F0F0F0Fu) | lo5(qhB0);
                            a2 = (wA1 & 0x0F0F0F0Fu) | lo5(qhA1); a3 = (wB1 & 0x0F0F0F0Fu) | lo5(qhB1);
                            h0 = ((wA0 >> 4) & 0x0F0F0F0Fu) | hi5(qhA0); h1 = ((wB0 >> 4) & 0x0F0F0F0Fu) | hi5(qhB0);
                            h2 = ((wA1 >> 4) & 0x0F0F0F0Fu) | hi5(qhA1); h3 = ((wB1 >> 4) & 0x0F0F0F0Fu) | hi5(qhB1);
                        } else {
                            sAl = (int)((jl ? (swA >> 12) : (swA << 4)) & 0xFF0u);
                            sBl = (int)((jl ? (swB >> 12) : (swB << 4)) & 0xFF0u);
                            a0 = wA0 & 0x0F0F0F0Fu; a1 = wB0 & 0x0F0F0F0Fu; a2 = wA1 & 0x0F0F0F0Fu; a3 = wB1 & 0x0F0F0F0Fu;
                            h0 = wA0 & 0xF0F0F0F0u; h1 = wB0 & 0xF0F0F0F0u; h2 = wA1 & 0xF0F0F0F0u; h3 = wB1 & 0xF0F0F0F0u;
                        }
#pragma unroll
                        for (int pr = 0; pr < NPAIR; pr++) {
                            int c[4];
                            mma_u8s8(c, a0, a1, a2, a3, bf[pr][2 * grp][0], bf[pr][2 * grp][1]);
                            acc[pr][0] += sAl * c[0]; acc[pr][1] += sAl * c[1]; acc[pr][2] += sBl * c[2]; acc[pr][3] += sBl * c[3];
                            mma_u8s8(c, h0, h1, h2, h3, bf[pr][2 * grp + 1][0], bf[pr][2 * grp + 1][1]);
                            acc[pr][0] += sAh * c[0]; acc[pr][1] += sAh * c[1]; acc[pr][2] += sBh * c[2]; acc[pr][3] += sBh * c[3];
                        }
                    }
                    // ---- fold planes, scales and the offset term into this thread's f32 partial row sums ----
                    const float2 ddA = __half22float2(*reinterpret_cast<const __half2*>(&hA.x));  // (d, dmin)
                    const float2 ddB = __half22float2(*reinterpret_cast<const __half2*>(&hB.x));
                    // this thread's share of sum_sb m_sb * sum_k x_k: sub-blocks 2t and 2t+1
                    const uint32_t mwA = mnA[t >> 1], mwB = mnB[t >> 1];
                    const int jm = (2 * t) & 3;
                    const float mA0 = (float)((mwA >> (8 * jm)) & 0xFFu), mA1 = (float)((mwA >> (8 * jm + 8)) & 0xFFu);
                    const float mB0 = (float)((mwB >> (8 * jm)) & 0xFFu), mB1 = (float)((mwB >> (8 * jm + 8)) & 0xFFu);
#pragma unroll
                    for (int pr = 0; pr < NPAIR; pr++) {
                        const float v0 = (float)acc[pr][0], v1 = (float)acc[pr][1], v2 = (float)acc[pr][2], v3 = (float)acc[pr][3];
#pragma unroll
                        for (int which = 0; which < 2; which++) {  // first / second token of the pair
                            const int tok = 2 * pr + which;
                            if (tok >= M) continue;
                            const float c0 = which ? cB0 : cA0, c1 = which ? cB1 : cA1;
                            const float sA = c0 * v0 + c1 * v1;
                            const float sB = c0 * v2 + c1 * v3;
                            const float mtA = mA0 * sx2[tok][0] + mA1 * sx2[tok][1];
                            const float mtB = mB0 * sx2[tok][0] + mB1 * sx2[tok][1];
                            yacc[rg][0][tok] += (ddA.x * isv[tok]) * sA - ddA.y * mtA;
                            yacc[rg][1][tok] += (ddB.x * isv[tok]) * sB - ddB.y * mtB;
                        }
                    }
                }
                }
                __syncwarp();
                if (lane == 0 && pj < njobs) issue_next();
            }
            // add the four threads that share a row (fixed order)
#pragma unroll
            for (int a = 0; a < RG; a++)
#pragma unroll
                for (int b = 0; b < 2; b++)
#pragma unroll
                    for (int c = 0; c < M; c++) {
                        float v = yacc[a][b][c];
                        v += __shfl_xor_sync(0xffffffffu, v, 1);
                        v += __shfl_xor_sync(0xffffffffu, v, 2);
                        yacc[a][b][c] = v;
                    }
            // ---- cross-warp reduction of this (tile, matrix), in warp order ----
            float* rb = red + (size_t)(seq & 1) * WARPS * M * 32;
            if (t == 0) {
#pragma unroll
                for (int rg = 0; rg < RG; rg++)
#pragma unroll
                    for (int tk = 0; tk < M; tk++) {
                        rb[(warp * M + tk) * 32 + rg * 16 + g] = yacc[rg][0][tk];
                        rb[(warp * M + tk) * 32 + rg * 16 + g + 8] = yacc[rg][1][tk];
                    }
            }
            __syncthreads();
            if (warp < M) {
                const int tk = warp;
                float y = 0.f, ssq = 0.f;
#pragma unroll 4
                for (int w = 0; w < WARPS; w++) {
                    y += rb[(w * M + tk) * 32 + lane];
                    if (one_pass) ssq += scratch[w];  // same order in every thread and CTA
                }
                if (one_pass) y *= 1.0f / sqrtf(ssq / (float)p.k + p.eps);  // cpu.rs:52-55
                const int row = lane < TR ? tile * TR + lane : p.n;  // lanes past the tile's rows hold nothing
                bool have = false;
                if (p.epi == EPI_SILU_MUL) {
                    if (mat == 0) {
                        gate_vals[tk * 32 + lane] = y;
                    } else if (row < p.n && tk < m_act) {
                        y = silu_f(gate_vals[tk * 32 + lane]) * y;
                        have = true;
                    }
                } else if (row < p.n && tk < m_act) {
                    if (p.epi == EPI_ADD_RESIDUAL) y = p.residual[orow(tk) + row] + y;
                    have = true;
                }
                if (have) {
                    if (!GROUPED && p.push.world > 0) {
                        const unsigned long long word = ((unsigned long long)push_e << 32) | (unsigned long long)__float_as_uint(y);
                        const size_t at = ((size_t)(push_e & 1u) * p.push.world + p.push.rank) * p.push.row_words + orow(tk) + row;
                        for (int r = 0; r < p.push.world; r++)
                            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.push.peer[r] + at), "l"(word) : "memory");
                    } else {
                        p.out[orow(tk) + row] = y;
                    }
                }
            }
        }
        }
    }
    if (rg) rg[3] = gtime();
    if (p.ring && threadIdx.x == 0) atomicMax(p.ring + 6, gtime());  // the last CTA to finish
    if (!ok && lane == 0 && p.error_flag) atomicExch(p.error_flag, 1);
}

// The activations of a grouped launch, once per call: row r of x (RMS-normalised with gains when norm_w is given,
// cpu.rs:49-60) as 24-bit fixed point against each 256-element unit's own power-of-two scale, split into three balanced
// byte planes, with the eight sub-block sums and 2^-s (the arithmetic of the prologue above, bit for bit).  One CTA of
// eight warps per row; a warp per unit.
__global__ void __launch_bounds__(256) gemv_planes_kernel(const float* __restrict__ x, const float* __restrict__ norm_w, float eps, int k,
                                                          unsigned char* __restrict__ planes, float* __restrict__ sxf, float* __restrict__ inv2s) {
    __shared__ float s_part[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nunits = k / kUnitElems;
    const size_t row = blockIdx.x;
    const float* xr = x + row * (size_t)k;
    pdl_launch_dependents();
    pdl_wait();
    float rms = 1.f;
    if (norm_w) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < k; i += blockDim.x) { const float v = xr[i]; ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        if (lane == 0) s_part[warp] = ss;
        __syncthreads();
        float r = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) r += s_part[w];  // every thread, same order
        rms = 1.0f / sqrtf(r / (float)k + eps);
    }
    for (int unit = warp; unit < nunits; unit += 8) {
        const int e0 = unit * kUnitElems + 8 * lane;
        const float4* xp = reinterpret_cast<const float4*>(xr + e0);
        const float4 u0 = xp[0], u1 = xp[1];
        float v[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        if (norm_w) {
            const float4* np = reinterpret_cast<const float4*>(norm_w + e0);
            const float4 n0 = np[0], n1 = np[1];
            const float nw[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = (v[j] * rms) * nw[j];
        }
        const size_t at = row * nunits + unit;
        unit_planes(v, lane, planes + at * 768, 96, sxf + at * 8, inv2s + at);
    }
}

int32_t launch_gemv_planes(const float* x, const float* norm_w, float eps, int k, int rows, const GemvPlanes& out, cudaStream_t s) {
    LC_CHECK(x && out.planes && out.sxf && out.inv2s && rows > 0 && k > 0 && k % kUnitElems == 0 && ((uintptr_t)x % 16) == 0 &&
                 (!norm_w || ((uintptr_t)norm_w % 16) == 0),
             LC_ERR_INVALID, "gemv planes: bad arguments");
    LC_CUDA(launch_pdl(gemv_planes_kernel, dim3(rows), dim3(256), 0, s, x, norm_w, eps, k, out.planes, out.sxf, out.inv2s));
    return LC_OK;
}

namespace {
unsigned long long* g_mring = nullptr;
int g_mring_seq = 0;
void dump_mring() {
    static unsigned long long h[1024 * 8];
    if (!g_mring || cudaMemcpy(h, g_mring, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return;
    fprintf(stderr, "[gemv ring] per launch slot, ns relative to CTA 0's start of the slot before:\n"
                    "  slot n k | cta0 start, last cta start | dependency met, planes done, cta0 end | last cta end\n");
    unsigned long long base = 0;
    for (int i = 0; i < 1024; i++) {
        const unsigned long long* r = h + (size_t)i * 8;
        if (!r[0]) continue;
        if (!base) base = r[0];
        fprintf(stderr, "  %4d %6llu %6llu | %7lld %7lld | %7lld %7lld %7lld | %7lld\n", i, r[5] >> 32, r[5] & 0xffffffffu, (long long)(r[0] - base),
                (long long)(r[7] - base), (long long)(r[1] - base), (long long)(r[2] - base), (long long)(r[3] - base), (long long)(r[6] - base));
        base = r[0];
    }
}
}  // namespace

template <int M, int WARPS, int STAGES>
static size_t mma_smem_bytes(int k, bool grouped = false, int unit_bytes = 144) {
    int nunits = grouped ? 0 : k / kUnitElems;
    size_t b = (size_t)WARPS * STAGES * unit_bytes * kTileRows;
    b += (size_t)nunits * 8 * M * 96 + (size_t)nunits * M * 8 * 4 + (size_t)nunits * M * 4;
    b += (size_t)2 * WARPS * M * 32 * 4 + (size_t)M * 32 * 4 + (size_t)(32 + M) * 4;
    b = (b + 7) & ~(size_t)7;
    b += (size_t)WARPS * STAGES * 8;
    return b + kGroupedSlots * 4;  // head room for the slot words of the grouped form
}

template <int M, int WARPS, int STAGES, bool GROUPED = false, uint32_t TYPE = LC_TYPE_Q4_K>
static int32_t launch_mma_cfg(const GemvArgs& a, cudaStream_t s) {
    auto kern = qgemv_mma_q4k_kernel<M, WARPS, STAGES, GROUPED, TYPE>;
    size_t smem = mma_smem_bytes<M, WARPS, STAGES>(a.w->k, GROUPED, mma_unit_bytes(TYPE));
    LC_CUDA(ensure_smem_limit((const void*)kern, kMaxSmem));
    GemvParams p;
    p.x = a.x; p.out = a.out; p.residual = a.residual; p.norm_w = a.norm_w; p.eps = a.eps;
    p.n = a.w->n; p.k = a.w->k; p.m = a.m; p.epi = (int)a.epi; p.error_flag = gemv_error_flag_dev();
    if (a.push) p.push = *a.push;
    static const bool want_ring = getenv("LC_GEMV_RING") != nullptr;
    if (want_ring) {
        if (!g_mring) {
            LC_CUDA(cudaMalloc(&g_mring, 1024 * 8 * sizeof(unsigned long long)));
            LC_CUDA(cudaMemset(g_mring, 0, 1024 * 8 * sizeof(unsigned long long)));
            atexit(dump_mring);
        }
        p.ring = g_mring + (size_t)(g_mring_seq++ % 1024) * 8;
    }
    int ntiles = (p.n + kTileRows - 1) / kTileRows;
    // CTAs per SM that fit shared memory (and, for the 8-warp shape, registers): with two per SM the
    // first CTAs of the next kernel move in while the last CTAs of this one drain
    int per_sm = (WARPS <= 8 && M <= 2 && 2 * (smem + 1024) <= kMaxSmem + 1024) ? 2 : 1;
    int grid = sm_count() * per_sm;
    if (grid > ntiles) grid = ntiles;
    const CUtensorMap* t0 = (const CUtensorMap*)a.w->tmap;
    const CUtensorMap* t1 = a.w2 ? (const CUtensorMap*)a.w2->tmap : t0;
    GemvGroupParams gp{};
    unsigned gy = 1;
    if constexpr (GROUPED) {
        const GemvGroup& g = *a.group;
        gp.tm0 = (const CUtensorMap*)g.tmaps; gp.tm1 = (const CUtensorMap*)(g.tmaps2 ? g.tmaps2 : g.tmaps);
        gp.cnt = g.counts; gp.list = g.lists; gp.list_stride = g.list_stride; gp.top_k = g.top_k; gp.x_by_token = g.x_by_token ? 1 : 0;
        gp.planes = g.planes.planes; gp.sxf = g.planes.sxf; gp.inv2s = g.planes.inv2s;
        gy = (unsigned)g.n_experts;
    }
    LC_CUDA(launch_pdl(kern, dim3(grid, gy), dim3(WARPS * 32), smem, s, *t0, *t1, p, gp));
    return LC_OK;
}

template <int M, uint32_t TYPE = LC_TYPE_Q4_K>
static int32_t launch_mma_m(const GemvArgs& a, cudaStream_t s, bool* launched) {
    *launched = true;
    int k = a.w->k;
    constexpr int ub = mma_unit_bytes(TYPE);
    if constexpr (M <= 4) {  // wider token tiles need more than 128 registers per thread: 8 warps
        if (mma_smem_bytes<M, 16, 2>(k, false, ub) <= kMaxSmem) return launch_mma_cfg<M, 16, 2, false, TYPE>(a, s);
    }
    if (mma_smem_bytes<M, 8, 2>(k, false, ub) <= kMaxSmem) return launch_mma_cfg<M, 8, 2, false, TYPE>(a, s);
    *launched = false;
    return LC_OK;
}

bool qgemv_mma_q5k_supports4(int k) {
    return k > 0 && k % kUnitElems == 0 && (mma_smem_bytes<4, 16, 2>(k, false, 176) <= kMaxSmem || mma_smem_bytes<4, 8, 2>(k, false, 176) <= kMaxSmem);
}

bool qgemv_mma_supports(int k) {
    return k > 0 && k % kUnitElems == 0 && (mma_smem_bytes<1, 16, 2>(k) <= kMaxSmem || mma_smem_bytes<1, 8, 2>(k) <= kMaxSmem);
}

// One launch over the experts of a layer (see the kernel's GROUPED note).  Token tile = the smallest of 1, 2, 4, 8 that
// holds the call's tokens; more than eight tokens make several passes per expert.
template <int M, int WARPS>
static int32_t launch_grouped_m(const GemvArgs& a, cudaStream_t s, bool* launched) {
    *launched = true;
    return launch_mma_cfg<M, WARPS, 2, true>(a, s);
}
int32_t launch_qgemv_mma_q4k_grouped(const GemvArgs& a, cudaStream_t s, bool* launched) {
    *launched = false;
    const GemvGroup* g = a.group;
    LC_CHECK(g && g->tmaps && g->counts && g->lists && g->n_experts > 0 && g->max_tokens > 0 && g->top_k > 0 && !a.residual && !a.norm_w &&
                 g->planes.planes && g->planes.sxf && g->planes.inv2s && g->list_stride <= kGroupedSlots,
             LC_ERR_INVALID, "grouped qgemv: incomplete expert group");
    // Token tile: the smallest of 1, 2, 4, 8 that holds what an expert typically receives (tokens * top_k / experts of the
    // layer); an expert with more slots than the tile makes several passes per weight tile.
    const int want = std::max(1, std::min(g->max_tokens, g->typical_tokens > 0 ? g->typical_tokens : g->max_tokens));
    if (want > 4) return launch_grouped_m<8, 8>(a, s, launched);
    if (want > 2) return launch_grouped_m<4, 16>(a, s, launched);
    if (want > 1) return launch_grouped_m<2, 16>(a, s, launched);
    return launch_grouped_m<1, 16>(a, s, launched);
}

int32_t launch_qgemv_mma_q4k(const GemvArgs& a, cudaStream_t s, bool* launched) {
    *launched = false;
    if (((uintptr_t)a.x % 16) != 0 || (a.norm_w && ((uintptr_t)a.norm_w % 16) != 0)) return LC_OK;
    if (a.w->typ == LC_TYPE_Q4_0) {
        if (a.m <= 1) return launch_mma_m<1, LC_TYPE_Q4_0>(a, s, launched);
        if (a.m <= 2) return launch_mma_m<2, LC_TYPE_Q4_0>(a, s, launched);
        if (a.m <= 4) return launch_mma_m<4, LC_TYPE_Q4_0>(a, s, launched);
        return LC_OK;  // wider token tiles of this type stay with the f32 kernel
    }
    if (a.w->typ == LC_TYPE_Q8_0) {
        if (a.m <= 1) return launch_mma_m<1, LC_TYPE_Q8_0>(a, s, launched);
        if (a.m <= 2) return launch_mma_m<2, LC_TYPE_Q8_0>(a, s, launched);
        if (a.m <= 4) return launch_mma_m<4, LC_TYPE_Q8_0>(a, s, launched);
        return LC_OK;
    }
    if (a.w->typ == LC_TYPE_Q5_K) {
        if (a.m <= 1) return launch_mma_m<1, LC_TYPE_Q5_K>(a, s, launched);
        if (a.m <= 2) return launch_mma_m<2, LC_TYPE_Q5_K>(a, s, launched);
        if (a.m <= 4) return launch_mma_m<4, LC_TYPE_Q5_K>(a, s, launched);
        return LC_OK;  // wider token tiles stay with the plain-load kernel
    }
    if (a.m <= 1) return launch_mma_m<1>(a, s, launched);
    if (a.m <= 2) return launch_mma_m<2>(a, s, launched);
    if (a.m <= 4) return launch_mma_m<4>(a, s, launched);
    if (a.m <= 6) return launch_mma_m<6>(a, s, launched);
    return launch_mma_m<8>(a, s, launched);
}

}  // namespace lc

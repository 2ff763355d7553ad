// One persistent kernel per decode step of a single sequence with Q4_K weights.
//
// A decode step is ~165 dependent phases of 1.5 - 8 us each (per layer: QKV, attention, O, gate/up, down; then
// head and argmax).  Launched as separate kernels every phase pays launch, prologue, pipeline ramp and tail, which
// is as much as the streaming itself.  Here one CTA per SM stays resident for the whole step:
//   * each warp owns a ring of TMA boxes and walks ONE job list that spans all matrix phases, so the weights of the
//     next phase stream into shared memory while the current phase drains and while the grid barrier is crossed;
//   * phases are separated by a grid barrier (monotonic 64-bit arrival counter, acquire/release, bounded spin);
//   * activations written by other CTAs are read through L2 (ld.cg), never through a possibly stale L1 line;
//   * the matrix phases are the int8 tensor-core GEMV of qgemv_mma.cu (token count 1), attention is the
//     split-context kernel of lc_attn.cuh run by four 128-thread groups per CTA.
// The kernel must be launched cooperatively (all CTAs co-resident).  A barrier or TMA wait that runs out sets the
// error flag, the CTA stops computing, keeps arriving at the remaining barriers, drains its own copies and returns.
#include <cstdlib>
#include "lc_kernels.h"
#include "lc_quant.cuh"
#include "lc_tma.cuh"
#include "lc_attn.cuh"
#include "lc_mega.h"

namespace lc {

namespace {

constexpr int kWarps = 16;
constexpr int kStages = 2;
constexpr int UB = 144;
constexpr int STAGE_BYTES = UB * kTileRows;
constexpr int kMaxUnitsPerWarp = 4;  // k <= 16 * 4 * 256 = 16384

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}
__device__ __forceinline__ uint32_t lds32(const unsigned char* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int32_t total_key(float f) {
    int32_t b = __float_as_int(f);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}

// Shared-memory layout (fixed offsets; kMaxUnits units of k at most)
constexpr int kMaxUnits = 64;
constexpr size_t OFF_RING = 0;                                                   // [kWarps][kStages][STAGE_BYTES]
constexpr size_t OFF_PLANES = OFF_RING + (size_t)kWarps * kStages * STAGE_BYTES; // [units][8][3][32]; attention scratch aliases it
constexpr size_t OFF_SXF = OFF_PLANES + (size_t)kMaxUnits * 768;                 // [units][8] f32
constexpr size_t OFF_INV2S = OFF_SXF + (size_t)kMaxUnits * 8 * 4;                // [units] f32
constexpr size_t OFF_RED = OFF_INV2S + (size_t)kMaxUnits * 4;                    // [2][kWarps][32] f32
constexpr size_t OFF_GATE = OFF_RED + 2 * kWarps * 32 * 4;                       // [32] f32
constexpr size_t OFF_SCRATCH = OFF_GATE + 32 * 4;                                // [64] f32
constexpr size_t OFF_BARS = OFF_SCRATCH + 64 * 4;                                // [kWarps][kStages] u64
constexpr size_t kMegaSmem = OFF_BARS + kWarps * kStages * 8;
static_assert(OFF_BARS % 8 == 0 && OFF_PLANES % 128 == 0, "alignment");

// producer cursor over the matrix phases of the step (lane 0 of each warp)
struct Cursor {
    int ph, ti, mat, ui;
    int tiles_mine, units_mine, nmat, tm0, tm1;
    int issued;
};

__device__ __forceinline__ void cursor_load(Cursor& c, const MegaParams& P, int warp) {
    while (c.ph < P.n_phases) {
        const MegaPhase& d = P.phases[c.ph];
        if (d.type == PH_GEMV) {
            const int ntiles = (d.n + kTileRows - 1) / kTileRows, nunits = d.k / kUnitElems;
            c.tiles_mine = (ntiles > (int)blockIdx.x) ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
            c.units_mine = (nunits > warp) ? (nunits - warp + kWarps - 1) / kWarps : 0;
            c.nmat = d.tm1 >= 0 ? 2 : 1;
            c.tm0 = d.tm0; c.tm1 = d.tm1;
            if (c.tiles_mine > 0 && c.units_mine > 0) { c.ti = c.mat = c.ui = 0; return; }
        }
        c.ph++;
    }
}

__device__ __forceinline__ void mega_issue_next(const MegaParams& P, Cursor& cur, int warp, unsigned char* stage_base, uint64_t* bars) {
    const int st = cur.issued & (kStages - 1);
    mbar_expect_tx(&bars[st], STAGE_BYTES);
    tma_load_2d(stage_base + (size_t)st * STAGE_BYTES, &P.tmaps[cur.mat ? cur.tm1 : cur.tm0], (warp + cur.ui * kWarps) * (UB / 4),
                (blockIdx.x + cur.ti * gridDim.x) * kTileRows, &bars[st]);
    cur.issued++;
    if (++cur.ui == cur.units_mine) {
        cur.ui = 0;
        if (++cur.mat == cur.nmat) {
            cur.mat = 0;
            if (++cur.ti == cur.tiles_mine) { cur.ph++; cursor_load(cur, P, warp); }
        }
    }
}

// One matrix phase: x -> fixed-point planes, then this warp's jobs of the phase.  Out of line so that the phase
// gets its own register allocation.
__device__ __noinline__ void mega_gemv_phase(const MegaParams& P, const MegaPhase& dref, Cursor& cur, int& job_ref, unsigned char* smem) {
    const MegaPhase d = dref;  // registers: the compiler cannot keep fields of a global struct across stores
    int job = job_ref;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    unsigned char* const planes = smem + OFF_PLANES;
    float* const sxf = reinterpret_cast<float*>(smem + OFF_SXF);
    float* const inv2s = reinterpret_cast<float*>(smem + OFF_INV2S);
    float* const scratch = reinterpret_cast<float*>(smem + OFF_SCRATCH);
    unsigned char* const stage_base = smem + OFF_RING + (size_t)warp * kStages * STAGE_BYTES;
    uint64_t* const bars = reinterpret_cast<uint64_t*>(smem + OFF_BARS) + warp * kStages;
    const float cA0 = (t == 0) ? 1.f : (t == 1 ? 65536.f : 0.f), cA1 = (t == 0) ? 256.f : 0.f;
    const int nunits = d.k / kUnitElems;
    const int ntiles = (d.n + kTileRows - 1) / kTileRows;
    const int tiles_mine = (ntiles > (int)blockIdx.x) ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int units_mine = (nunits > warp) ? (nunits - warp + kWarps - 1) / kWarps : 0;
    const int nmat = d.tm1 >= 0 ? 2 : 1;
    // ---- x of this warp's units into registers (through L2), RMS scale, fixed-point planes ----
    float xv[kMaxUnitsPerWarp][8];
    float ss = 0.f;
#pragma unroll
    for (int ui = 0; ui < kMaxUnitsPerWarp; ui++) {
        if (ui < units_mine) {
            const int e0 = (warp + ui * kWarps) * kUnitElems + 8 * lane;
            {
                const float4 u0 = __ldcg(reinterpret_cast<const float4*>(d.x + e0));
                const float4 u1 = __ldcg(reinterpret_cast<const float4*>(d.x + e0) + 1);
                xv[ui][0] = u0.x; xv[ui][1] = u0.y; xv[ui][2] = u0.z; xv[ui][3] = u0.w;
                xv[ui][4] = u1.x; xv[ui][5] = u1.y; xv[ui][6] = u1.z; xv[ui][7] = u1.w;
            }
#pragma unroll
            for (int j = 0; j < 8; j++) ss = fmaf(xv[ui][j], xv[ui][j], ss);
        }
    }
    float rms_scale = 1.0f;
    if (d.norm_w) {
        ss = warp_sum(ss);
        if (lane == 0) scratch[warp] = ss;
        __syncthreads();
        if (warp == 0) {
            float r = (lane < kWarps) ? scratch[lane] : 0.f;
            r = warp_sum(r);
            if (lane == 0) scratch[32] = 1.0f / sqrtf(r / (float)d.k + P.eps);
        }
        __syncthreads();
        rms_scale = scratch[32];
    }
#pragma unroll
    for (int ui = 0; ui < kMaxUnitsPerWarp; ui++) {
        if (ui < units_mine) {
            const int unit = warp + ui * kWarps;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = xv[ui][j];
            if (d.norm_w) {
                const float4* np = reinterpret_cast<const float4*>(d.norm_w + unit * kUnitElems + 8 * lane);
                const float4 n0 = np[0], n1 = np[1];
                const float nw[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = (v[j] * rms_scale) * nw[j];
            }
            float amax = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(v[j]));
            amax = warp_max(amax);
            const int ex = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 126;  // amax = f * 2^ex, f in [0.5, 1)
            const int s = max(-100, min(100, 22 - ex));
            const float up = __uint_as_float((uint32_t)(127 + s) << 23), dn = __uint_as_float((uint32_t)(127 - s) << 23);
            uint32_t pw[3][2] = {{0, 0}, {0, 0}, {0, 0}};
            int xsum = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float sv = fminf(fmaxf(v[j] * up, -4194304.f), 4194304.f);
                const int X = __float2int_rn(sv);
                xsum += X;
                const int p0 = ((X + 128) & 255) - 128;
                const int X1 = (X - p0) >> 8;
                const int p1 = ((X1 + 128) & 255) - 128;
                const int p2 = (X1 - p1) >> 8;
                pw[0][j >> 2] |= (uint32_t)(p0 & 255) << (8 * (j & 3));
                pw[1][j >> 2] |= (uint32_t)(p1 & 255) << (8 * (j & 3));
                pw[2][j >> 2] |= (uint32_t)(p2 & 255) << (8 * (j & 3));
            }
            const int sb = lane >> 2, inner = (8 * lane) & 31;
#pragma unroll
            for (int pl = 0; pl < 3; pl++)
                *reinterpret_cast<uint2*>(planes + (unit * 8 + sb) * 96 + pl * 32 + inner) = make_uint2(pw[pl][0], pw[pl][1]);
            xsum += __shfl_xor_sync(0xffffffffu, xsum, 1);
            xsum += __shfl_xor_sync(0xffffffffu, xsum, 2);
            if (t == 0) sxf[unit * 8 + sb] = (float)xsum * dn;
            if (lane == 0) inv2s[unit] = dn;
        }
    }
    __syncwarp();
    if (P.trace && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long tt;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tt));
        P.trace[4 * d.reserved + 2] = tt;
    }

    // ---- consume this phase's jobs ----
    uint32_t bf[8][2];
    float sx2[2], isv = 0.f;
    auto load_unit_consts = [&](int unit) {
        const bool colv = g < 3;
        const unsigned char* bp = planes + unit * 768 + (colv ? g : 0) * 32 + 4 * t;
#pragma unroll
        for (int sb = 0; sb < 8; sb++) {
            const uint32_t v0 = lds32(bp + sb * 96), v1 = lds32(bp + sb * 96 + 16);
            bf[sb][0] = colv ? v0 : 0u;
            bf[sb][1] = colv ? v1 : 0u;
        }
        sx2[0] = sxf[unit * 8 + 2 * t];
        sx2[1] = sxf[unit * 8 + 2 * t + 1];
        isv = inv2s[unit] * 0.0625f;
    };
    const bool single_unit = units_mine == 1;
    if (single_unit) load_unit_consts(warp);
    for (int ti = 0; ti < tiles_mine; ti++) {
        const int tile = blockIdx.x + ti * gridDim.x;
        for (int mat = 0; mat < nmat; mat++) {
            float yacc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
            for (int ui = 0; ui < units_mine; ui++, job++) {
                const int st = job & (kStages - 1);
                if (!single_unit) load_unit_consts(warp + ui * kWarps);
                if (!mbar_wait(&bars[st], (uint32_t)((job / kStages) & 1))) {
                    if (lane == 0) atomicExch(P.error_flag, 1);
                }
                if (P.trace && blockIdx.x == 0 && threadIdx.x == 0 && ti == 0 && mat == 0 && ui == 0) {
                    unsigned long long tt;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tt));
                    P.trace[4 * d.reserved + 3] = tt;
                }
                const unsigned char* tilep = stage_base + (size_t)st * STAGE_BYTES;
#pragma unroll
                for (int rg = 0; rg < 2; rg++) {
                    const unsigned char* rowA = tilep + (rg * 16 + g) * UB;
                    const unsigned char* rowB = rowA + 8 * UB;
                    const uint4 hA = *reinterpret_cast<const uint4*>(rowA);
                    const uint4 hB = *reinterpret_cast<const uint4*>(rowB);
                    uint32_t scA[2], mnA[2], scB[2], mnB[2];
                    unpack_scales_k4(hA.y, hA.z, hA.w, &scA[0], &scA[1], &mnA[0], &mnA[1]);
                    unpack_scales_k4(hB.y, hB.z, hB.w, &scB[0], &scB[1], &mnB[0], &mnB[1]);
                    int acc[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int grp = 0; grp < 4; grp++) {
                        const uint32_t wA0 = lds32(rowA + 16 + 32 * grp + 4 * t), wA1 = lds32(rowA + 32 + 32 * grp + 4 * t);
                        const uint32_t wB0 = lds32(rowB + 16 + 32 * grp + 4 * t), wB1 = lds32(rowB + 32 + 32 * grp + 4 * t);
                        const uint32_t swA = scA[grp >> 1], swB = scB[grp >> 1];
                        const int jl = (2 * grp) & 3;
                        const int sAl = (int)((jl ? (swA >> 12) : (swA << 4)) & 0xFF0u), sAh = (int)__byte_perm(swA, 0, 0x4440 + jl + 1);
                        const int sBl = (int)((jl ? (swB >> 12) : (swB << 4)) & 0xFF0u), sBh = (int)__byte_perm(swB, 0, 0x4440 + jl + 1);
                        int c[4];
                        mma_u8s8(c, wA0 & 0x0F0F0F0Fu, wB0 & 0x0F0F0F0Fu, wA1 & 0x0F0F0F0Fu, wB1 & 0x0F0F0F0Fu, bf[2 * grp][0], bf[2 * grp][1]);
                        acc[0] += sAl * c[0]; acc[1] += sAl * c[1]; acc[2] += sBl * c[2]; acc[3] += sBl * c[3];
                        mma_u8s8(c, wA0 & 0xF0F0F0F0u, wB0 & 0xF0F0F0F0u, wA1 & 0xF0F0F0F0u, wB1 & 0xF0F0F0F0u, bf[2 * grp + 1][0],
                                 bf[2 * grp + 1][1]);
                        acc[0] += sAh * c[0]; acc[1] += sAh * c[1]; acc[2] += sBh * c[2]; acc[3] += sBh * c[3];
                    }
                    const float2 ddA = __half22float2(*reinterpret_cast<const __half2*>(&hA.x));
                    const float2 ddB = __half22float2(*reinterpret_cast<const __half2*>(&hB.x));
                    const uint32_t mwA = mnA[t >> 1], mwB = mnB[t >> 1];
                    const int jm = (2 * t) & 3;
                    const float mA0 = (float)((mwA >> (8 * jm)) & 0xFFu), mA1 = (float)((mwA >> (8 * jm + 8)) & 0xFFu);
                    const float mB0 = (float)((mwB >> (8 * jm)) & 0xFFu), mB1 = (float)((mwB >> (8 * jm + 8)) & 0xFFu);
                    const float sA = cA0 * (float)acc[0] + cA1 * (float)acc[1];
                    const float sB = cA0 * (float)acc[2] + cA1 * (float)acc[3];
                    yacc[rg][0] += (ddA.x * isv) * sA - ddA.y * (mA0 * sx2[0] + mA1 * sx2[1]);
                    yacc[rg][1] += (ddB.x * isv) * sB - ddB.y * (mB0 * sx2[0] + mB1 * sx2[1]);
                }
                __syncwarp();
                if (lane == 0 && cur.ph < P.n_phases) mega_issue_next(P, cur, warp, stage_base, bars);
            }
#pragma unroll
            for (int a = 0; a < 2; a++)
#pragma unroll
                for (int b = 0; b < 2; b++) {
                    float v = yacc[a][b];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    yacc[a][b] = v;
                }
            const int seq = ti * nmat + mat;
            float* rb = reinterpret_cast<float*>(smem + OFF_RED) + (size_t)(seq & 1) * kWarps * 32;
            if (t == 0) {
#pragma unroll
                for (int rg = 0; rg < 2; rg++) {
                    rb[warp * 32 + rg * 16 + g] = yacc[rg][0];
                    rb[warp * 32 + rg * 16 + g + 8] = yacc[rg][1];
                }
            }
            __syncthreads();
            if (warp == 0) {
                float y = 0.f;
#pragma unroll 4
                for (int w = 0; w < kWarps; w++) y += rb[w * 32 + lane];
                const int row = tile * kTileRows + lane;
                if (d.epi == EPI_SILU_MUL) {
                    if (mat == 0) reinterpret_cast<float*>(smem + OFF_GATE)[lane] = y;
                    else if (row < d.n) d.out[row] = silu_f(reinterpret_cast<float*>(smem + OFF_GATE)[lane]) * y;
                } else if (row < d.n) {
                    if (d.epi == EPI_ADD_RESIDUAL) y = __ldcg(d.residual + row) + y;
                    d.out[row] = y;
                }
            }
        }
    }
    job_ref = job;
}

// Attention of one (head, split) by a 128-thread group, head_dim 128, f16 cache, at most 128 keys per split
// (attention.rs:69-113 restricted to the slice; the slices are merged in split order by the last group to finish).
// Two memory round trips: every thread owns ONE key for the scores (its 256-byte row as sixteen 128-bit loads,
// all in flight at once), then the threads split (key half, dim pair) for p.V with coalesced half2 loads.
// The token of this step is taken from k_new / v_new (rotated, rounded through f16 exactly like a cache round
// trip) and written to the cache by the first q head of its kv group.
__device__ __noinline__ void mega_attention(const AttnParams& p, int head, int split, int tid, float* sh, int bar_id) {
    constexpr int HD = 128;
    float* q_s = sh;              // [128]
    float* p_s = sh + 128;        // [128]
    float* acc_s = sh + 256;      // [2][128]
    float* red_s = sh + 512;      // [8]
    int* last_s = reinterpret_cast<int*>(sh + 520);
    const int warp = tid >> 5, lane = tid & 31;
    const int n_heads = p.n_heads;
    const KvLayout& kv = p.kv;
    const int pos = p.tok_pos[0];
    const int t_begin = split * p.chunk;
    const int t_end = min(pos + 1, t_begin + p.chunk);
    const int n = t_end - t_begin;  // <= 128 (may be <= 0: empty split)
    const int gsz = n_heads / kv.n_kv, kvh = head / gsz;
    float* pout = p.partial + ((size_t)head * p.n_splits + split) * (HD + 2);
    float m = -INFINITY, l = 0.f, a_out = 0.f;
    if (n > 0) {
        const int rp = p.tok_rope[0];
        const bool writer = (head % gsz) == 0;
        const __half* Kp = (const __half*)kv.k_pool;
        const __half* Vp = (const __half*)kv.v_pool;
        const int32_t* pt = p.page_table + (size_t)p.tok_seq[0] * p.pages_per_seq;
        // q (rotated) -> shared
        {
            float qv[1];
            load_rotated<1, HD>(p.q + head * HD, tid, rp, p.theta, qv);
            q_s[tid] = qv[0];
        }
        asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
        // ---- scores: thread tid owns key t_begin + tid ----
        float s = -INFINITY;
        const int tk = t_begin + tid;
        if (tid < n) {
            float dot = 0.f;
            if (tk == pos) {
                float kr[16];
#pragma unroll
                for (int c = 0; c < HD / 16; c++) {
                    load_rotated<16, HD>(p.k_new + kvh * HD, 16 * c, rp, p.theta, kr);
                    __half* dst = (__half*)kv.k_pool + (((size_t)pt[tk / kv.page_tokens] * kv.n_kv + kvh) * kv.page_tokens + tk % kv.page_tokens) * HD + 16 * c;
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const __half hv = __float2half_rn(kr[i]);  // cache/mod.rs:35-36, read back as cache/mod.rs:65-77
                        if (writer) dst[i] = hv;
                        dot = fmaf(q_s[16 * c + i], __half2float(hv), dot);
                    }
                }
            } else {
                const uint4* kp = reinterpret_cast<const uint4*>(Kp + (((size_t)pt[tk / kv.page_tokens] * kv.n_kv + kvh) * kv.page_tokens + tk % kv.page_tokens) * HD);
                uint4 kr[16];
#pragma unroll
                for (int c = 0; c < 16; c++) kr[c] = kp[c];
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    const __half2* h2 = reinterpret_cast<const __half2*>(&kr[c]);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float2 f = __half22float2(h2[j]);
                        dot = fmaf(q_s[8 * c + 2 * j], f.x, dot);
                        dot = fmaf(q_s[8 * c + 2 * j + 1], f.y, dot);
                    }
                }
            }
            s = dot / sqrtf((float)HD);  // attention.rs:93
        }
        // ---- softmax pieces of the slice: max, exp, sum (fixed order) ----
        float wm = warp_max(s);
        if (lane == 0) red_s[warp] = wm;
        asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
        m = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
        const float pe = (tid < n) ? expf(s - m) : 0.f;
        p_s[tid] = pe;
        const float ws = warp_sum(pe);
        if (lane == 0) red_s[4 + warp] = ws;
        asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
        l = ((red_s[4] + red_s[5]) + red_s[6]) + red_s[7];
        // ---- p.V: thread = (key half hh, dim pair j) ----
        const int hh = tid >> 6, j = tid & 63;
        float ax = 0.f, ay = 0.f;
        const int k0 = hh * 64, k1 = min(n, k0 + 64);
        // new-token value of this thread's dim pair (used instead of the cache slot at t == pos)
        float2 vnew = make_float2(0.f, 0.f);
        const bool has_new = pos >= t_begin && pos < t_end;
        if (has_new) {
            const __half h0 = __float2half_rn(__ldcg(p.v_new + kvh * HD + 2 * j));
            const __half h1 = __float2half_rn(__ldcg(p.v_new + kvh * HD + 2 * j + 1));
            vnew = make_float2(__half2float(h0), __half2float(h1));
            if (writer && hh == ((pos - t_begin) >> 6)) {
                __half* dst = (__half*)kv.v_pool + (((size_t)pt[pos / kv.page_tokens] * kv.n_kv + kvh) * kv.page_tokens + pos % kv.page_tokens) * HD + 2 * j;
                dst[0] = h0; dst[1] = h1;
            }
        }
        // loads are unconditional (clamped to the last key of the slice) so that a batch of eight is in flight together;
        // the slot of the new token may hold stale bytes, its weight is applied to vnew instead
        for (int kk = k0; kk < k1; kk += 8) {
            float2 vv[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int t2 = min(t_begin + kk + u, t_end - 1);
                const __half2 hv = *reinterpret_cast<const __half2*>(
                    Vp + (((size_t)pt[t2 / kv.page_tokens] * kv.n_kv + kvh) * kv.page_tokens + t2 % kv.page_tokens) * HD + 2 * j);
                vv[u] = __half22float2(hv);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int t2 = t_begin + kk + u;
                const bool live = kk + u < k1;
                const float pk = live ? p_s[kk + u] : 0.f;
                // a padding entry re-read the slice's last slot, which may be the new token's still unwritten row:
                // whatever bytes it holds (Inf, NaN) must not meet the zero weight
                const float2 val = (t2 == pos) ? vnew : (live ? vv[u] : make_float2(0.f, 0.f));
                ax = fmaf(pk, val.x, ax);
                ay = fmaf(pk, val.y, ay);
            }
        }
        acc_s[hh * 128 + 2 * j] = ax;
        acc_s[hh * 128 + 2 * j + 1] = ay;
        asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
        a_out = acc_s[tid] + acc_s[128 + tid];
    }
    if (p.n_splits == 1) {
        p.out[head * HD + tid] = a_out / l;
        return;
    }
    if (tid == 0) { pout[0] = m; pout[1] = l; }
    pout[2 + tid] = a_out;
    // ---- the last split of this head to finish merges all of them, in split order ----
    __threadfence();
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    if (tid == 0) *last_s = (atomicAdd(&p.counters[head], 1) == p.n_splits - 1);
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    if (!*last_s) return;
    __threadfence();
    const float* pp = p.partial + (size_t)head * p.n_splits * (HD + 2);
    float mm = -INFINITY;
    for (int sidx = 0; sidx < p.n_splits; sidx++) mm = fmaxf(mm, __ldcg(pp + (size_t)sidx * (HD + 2)));
    float ll = 0.f, a = 0.f;
    for (int sidx = 0; sidx < p.n_splits; sidx++) {
        const float* ps = pp + (size_t)sidx * (HD + 2);
        const float ms = __ldcg(ps);
        if (ms == -INFINITY) continue;  // empty split
        const float sc = expf(ms - mm);
        ll += __ldcg(ps + 1) * sc;
        a += __ldcg(ps + 2 + tid) * sc;
    }
    p.out[head * HD + tid] = a / ll;
    if (tid == 0) p.counters[head] = 0;
}

}  // namespace

__global__ void __launch_bounds__(kWarps * 32, 1) decode_mega_kernel(const __grid_constant__ MegaParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    __shared__ int sh_ok;

    unsigned char* const planes = smem + OFF_PLANES;
    float* const sxf = reinterpret_cast<float*>(smem + OFF_SXF);
    float* const inv2s = reinterpret_cast<float*>(smem + OFF_INV2S);
    float* const scratch = reinterpret_cast<float*>(smem + OFF_SCRATCH);
    unsigned char* const stage_base = smem + OFF_RING + (size_t)warp * kStages * STAGE_BYTES;
    uint64_t* const bars = reinterpret_cast<uint64_t*>(smem + OFF_BARS) + warp * kStages;

    // ---- producer: start streaming the first matrices before anything else ----
    Cursor cur;
    cur.ph = 0; cur.issued = 0;
    if (lane == 0) {
        for (int s = 0; s < kStages; s++) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        cursor_load(cur, P, warp);
        for (int j = 0; j < kStages && cur.ph < P.n_phases; j++) mega_issue_next(P, cur, warp, stage_base, bars);
    }
    __syncwarp();

    // ---- grid barrier bookkeeping: every launch adds exactly n_phases * gridDim.x arrivals ----
    const unsigned long long per_launch = (unsigned long long)P.n_phases * gridDim.x;
    unsigned long long base = 0;
    if (threadIdx.x == 0) {
        const unsigned long long v = ld_acquire_u64(P.bar);
        base = v / per_launch * per_launch;
    }
    bool alive = true;  // false after a wait ran out: stop computing, keep the barriers moving
    int job = 0;        // jobs consumed by this warp

    for (int ph = 0; ph < P.n_phases; ph++) {
        const MegaPhase& d = P.phases[ph];
        // ---- wait until every CTA has finished the previous phase ----
        if (ph > 0) {
            if (threadIdx.x == 0) {
                const unsigned long long target = base + (unsigned long long)ph * gridDim.x;
                int okv = 0;
                for (uint32_t it = 0; it < (1u << 24); ++it) {
                    if (ld_acquire_u64(P.bar) >= target) { okv = 1; break; }
                    __nanosleep(20);
                }
                sh_ok = okv;
            }
            __syncthreads();
            if (!sh_ok) {
                if (alive && threadIdx.x == 0) atomicExch(P.error_flag, 2);
                alive = false;
            }
        }
        if (P.trace && blockIdx.x == 0 && threadIdx.x == 0) {
            unsigned long long tt;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tt));
            P.trace[4 * ph] = tt;
        }
        if (alive && d.type == PH_GEMV) {
            mega_gemv_phase(P, d, cur, job, smem);
        } else if (alive && d.type == PH_ATTN) {
            AttnParams ap = P.attn;
            ap.kv.k_pool = P.k_pools[d.layer];
            ap.kv.v_pool = P.v_pools[d.layer];
            const int grp4 = warp >> 2, tid = threadIdx.x & 127;
            float* shg = reinterpret_cast<float*>(planes) + grp4 * 544;
            const int n_items = ap.n_heads * ap.n_splits;
            // items are walked in lock step by the four groups so the named barriers stay matched
            for (int it0 = blockIdx.x * 4; it0 < n_items; it0 += gridDim.x * 4) {
                const int idx = it0 + grp4;
                if (idx < n_items) {
                    const int head = idx % ap.n_heads, split = idx / ap.n_heads;
                    mega_attention(ap, head, split, tid, shg, 1 + grp4);
                }
            }
        } else if (alive && d.type == PH_EMBED) {
            // embedding row of the current token -> residual stream (engine.rs:134-144: unknown id -> zero row)
            const int64_t token = P.tokens[0];
            const bool okt = token >= 0 && token < P.embed_rows;
            for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < d.k; e += gridDim.x * blockDim.x)
                P.hidden[e] = okt ? dequant_elem(P.embed_typ, P.embed, (size_t)token * d.k + e) : 0.f;
        } else if (alive && d.type == PH_ARGMAX) {
            // greedy pick, part 1: best (key, index) of this CTA's slice (sampler.rs:6-10: last of equal maxima)
            long long best = LLONG_MIN;
            for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < P.V; i += gridDim.x * blockDim.x) {
                const long long key = ((long long)total_key(__ldcg(P.logits + i)) << 32) | (long long)(uint32_t)i;
                best = key > best ? key : best;
            }
            for (int o = 16; o > 0; o >>= 1) {
                const long long other = __shfl_xor_sync(0xffffffffu, best, o);
                best = other > best ? other : best;
            }
            long long* shk = reinterpret_cast<long long*>(scratch);
            if (lane == 0) shk[warp] = best;
            __syncthreads();
            if (warp == 0) {
                best = lane < kWarps ? shk[lane] : LLONG_MIN;
                for (int o = 16; o > 0; o >>= 1) {
                    const long long other = __shfl_xor_sync(0xffffffffu, best, o);
                    best = other > best ? other : best;
                }
                if (lane == 0) P.argmax_scratch[blockIdx.x] = best;
            }
        } else if (alive && d.type == PH_FINAL) {
            // part 2 (CTA 0): merge the per-CTA candidates, feed the token back, advance the cache position
            if (blockIdx.x == 0 && warp == 0) {
                long long best = LLONG_MIN;
                for (int i = lane; i < (int)gridDim.x; i += 32) {
                    const long long v = __ldcg(P.argmax_scratch + i);
                    best = v > best ? v : best;
                }
                for (int o = 16; o > 0; o >>= 1) {
                    const long long other = __shfl_xor_sync(0xffffffffu, best, o);
                    best = other > best ? other : best;
                }
                if (lane == 0) {
                    const int64_t nx = (int64_t)(uint32_t)(best & 0xffffffffll);
                    P.next[0] = nx;
                    P.tokens[0] = nx;
                    P.tok_pos[0] += 1;
                    if (P.rope_absolute) P.tok_rope[0] = P.tok_pos[0];
                    const int step = *P.step_ctr;
                    if (P.out_tokens) P.out_tokens[step] = nx;
                    *P.step_ctr = step + 1;
                }
            }
        }
        // ---- arrive: everything this CTA wrote in the phase is visible before the count moves ----
        __syncthreads();
        if (P.trace && blockIdx.x == 0 && threadIdx.x == 0) {
            unsigned long long tt;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tt));
            P.trace[4 * ph + 1] = tt;
        }
        if (threadIdx.x == 0) {
            __threadfence();
            atomicAdd(P.bar, 1ull);
        }
    }
    // ---- drain: copies this warp requested but never consumed (only after an aborted step) ----
    if (lane == 0) {
        for (int j = job; j < cur.issued; j++) (void)mbar_wait(&bars[j & (kStages - 1)], (uint32_t)((j / kStages) & 1));
    }
}

size_t decode_mega_smem_bytes(int max_units) {
    return max_units <= kMaxUnits ? kMegaSmem + 128 : (size_t)1 << 30;
}

int32_t launch_decode_mega(const MegaParams& P, cudaStream_t s) {
    size_t smem = decode_mega_smem_bytes(P.max_units);
    LC_CHECK(smem <= kMaxSmem, LC_ERR_UNSUPPORTED, "persistent decode kernel: %zu bytes of shared memory needed", smem);
    static bool attr_set = false;
    if (!attr_set) {
        LC_CUDA(cudaFuncSetAttribute(decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count());
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    LC_CUDA(cudaLaunchKernelEx(&cfg, decode_mega_kernel, P));
    return LC_OK;
}

}  // namespace lc

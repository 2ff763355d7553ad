// Q4_K matrix-vector product for one or two tokens on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory), exact in the integer domain.
//
//   y[t, r] = sum_k x[t, k] * w[r, k],   w = (d * sc) * q - (dmin * m)      (rust/src/kernels/mod.rs:66-98)
//
// Arithmetic is that of the mma.sync kernel next door: the f32 activations of each 256-element unit become 24-bit
// fixed point against the unit's own power-of-two scale, split into three balanced int8 planes; the 4-bit weights
// stay integers; products are accumulated in int32 per 32-element sub-block and the 6-bit sub-block scales are applied
// as integer multiplies.  What changes is who does the work.  The warp-level MMA made every thread fetch fragments,
// mask nibbles, and scale a 16x8 tile of which three columns were useful -- 640 warp instructions per 32 rows x 256 k,
// which bound the kernel by instruction issue, not by HBM.  Here:
//
//   work unit   one "block" = 128 rows x one 256-element unit = a [144 B x 128 rows] TMA box (18 KB);
//   unpack      thread r of a 128-thread group owns row r: eight 16-byte loads of packed nibbles, two masks each
//               (low nibble; high nibble left in place, carrying x16), stored with tcgen05.st as the A operand IN
//               TENSOR MEMORY (lane = row, 8 columns of 4 bytes per sub-block): the unpacked bytes never cross shared
//               memory, whose bandwidth the TMA boxes and their reads already use;
//   multiply    one thread issues eight tcgen05.mma (M=128, N=8, K=32), one per sub-block, A = those bytes (u8),
//               B = the int8 planes of x for that sub-block in shared memory (N rows = 3 planes x tokens), each into
//               its own 8 columns of tensor memory -- the accumulators never touch registers until they are final;
//   fold        thread r reads its row's 8 x 8 int32 sums with tcgen05.ld, applies the row's scales and offsets
//               (its own header, still in registers from the unpack), and adds into its f32 row sum.
//
// That is ~200 thread instructions per row and block: the kernel is bound by the TMA stream again.
//
// Work is split by blocks, not by rows: CTA c takes blocks [c*B/G, (c+1)*B/G) of the (tile, matrix, unit) order, so
// all SMs stream the same number of bytes whatever the matrix shape.  A 128-row tile whose blocks span several CTAs
// is finished by the last of them to arrive (partials in global scratch, summed in CTA order: deterministic).
#include <cstdio>
#include <cstdlib>
#include "lc_kernels.h"
#include "lc_quant.cuh"
#include "lc_tma.cuh"

namespace lc {

namespace {

constexpr int kRows = 128;                   // rows per block = MMA M
constexpr int kRawBytes = 144 * kRows;       // one TMA box
constexpr int kPlaneBytes = 8 * 256;         // B operand of one unit: 8 sub-blocks x [2 k-chunks][8 rows][16 B]
constexpr int kMaxStages = 11;

struct UmmaParams {
    GemvParams g;
    unsigned long long* partial;  // [tile][contributor][matrix][token][128] (f32 bits | valid << 32), zero between launches
    int max_contrib;
    int nslots;          // unit slots of x planes held in shared memory
    int nstages;         // raw boxes in flight
    long long* trace;    // diagnostics (LC_GEMV_TRACE): [grid][2 groups][64] SM clock stamps, or null
    unsigned long long* ring;  // diagnostics (LC_GEMV_RING): [0] launch counter, then [1024][8] wall-clock stamps per launch slot
    int ring_slot;
};

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // K-major, no swizzle: start address, leading (between the two 16-byte k chunks) and stride (between 8-row
    // groups) byte offsets in 16-byte units, descriptor version 1
    uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
// s32 accumulate, A unsigned 8-bit, B signed 8-bit, both K-major, N = 8, M = 128
constexpr uint32_t kIdesc = (2u << 4) | (0u << 7) | (1u << 10) | (1u << 17) | (8u << 24);

// D[tmem] = A[tmem] * B[smem]^T (no accumulate)
__device__ __forceinline__ void umma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t db) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%4, %4, %4, %4}, p;\n}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(db), "r"(kIdesc), "r"(zero)
        : "memory");
}
// 16 consecutive 32-bit columns of this thread's lane
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

template <int NC>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[NC]);
template <>
__device__ __forceinline__ void tmem_ld<4>(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<8>(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}

}  // namespace

// Thread roles: NG autonomous groups of 128 threads; block i of the CTA belongs to group i % NG and thread r of the
// group owns row r.  Per block a group waits for the box, unpacks it into tensor memory, meets at its own hardware
// barrier, multiplies, and folds.  A thread needs ~70 cycles to issue one tcgen05.mma whatever its shape, but threads
// issue in parallel: lane 0 of each of the group's four warps issues two of the eight sub-block products and commits
// them to the group's barrier (four arrivals); thread 0 of the group then re-requests the freed stage.
template <int M, int NG>
__global__ void __launch_bounds__(NG * 128, 1)
qgemv_umma_q4k_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, UmmaParams P) {
    constexpr int NC = (M == 1) ? 4 : 8;  // accumulator columns read per sub-block (3 planes per token)
    constexpr int GW = NG * 4;            // group warps
    constexpr int GT = NG * 128;          // group threads
    static_assert(NG == 4, "tensor memory holds four groups: 64 columns of A and 64 of accumulators each");
    constexpr int kTmemCols = 512;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const GemvParams& p = P.g;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr bool issuer_warp = false;  // every warp belongs to a group
    const int wg = tid >> 7, row = tid & 127;  // group, and the row this thread owns in every block of the group
    const int nunits = p.k / kUnitElems;
    const int nmat = (p.epi == EPI_SILU_MUL) ? 2 : 1;
    const int bpt = nunits * nmat;  // blocks per 128-row tile
    const int ntiles = (p.n + kRows - 1) / kRows;
    const long long Btot = (long long)ntiles * bpt;
    const int b_begin = (int)((long long)blockIdx.x * Btot / gridDim.x);
    const int b_end = (int)((long long)(blockIdx.x + 1) * Btot / gridDim.x);
    const int L = b_end - b_begin;
    const bool all_units = L >= nunits;  // x planes kept per unit, else per block of this CTA
    const int nslots = all_units ? nunits : L;
    const int NS = P.nstages;

    unsigned char* raw = smem;                                        // [NS][kRawBytes]   TMA boxes
    unsigned char* planes = raw + (size_t)NS * kRawBytes;             // [slots][kPlaneBytes]
    float* sxf = reinterpret_cast<float*>(planes + (size_t)P.nslots * kPlaneBytes);  // [slots][M][8] sum of x per sub-block
    float* inv2s = sxf + (size_t)P.nslots * M * 8;                    // [slots][M]        2^-s / 16
    float* red = inv2s + (size_t)P.nslots * M;                        // [2][NG][2][M][128] per segment parity, group, matrix
    float* scratch = red + 2 * NG * 2 * M * kRows;                    // [GW + M]
    uint64_t* bars = reinterpret_cast<uint64_t*>(((uintptr_t)(scratch + GW + M) + 7) & ~(uintptr_t)7);
    uint64_t* raw_full = bars;                     // [kMaxStages] a box has landed
    // A group strictly alternates "issue and commit, wait on acc_full", so no waiter can fall a phase behind.
    uint64_t* acc_full = bars + kMaxStages;        // [NG] the eight products of a block are in tensor memory (4 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + NG);
    int* flag = reinterpret_cast<int*>(tmem_slot + 1);

    int tr_n = 0;
    auto stamp = [&]() {  // first thread of each group and issuer 0
        if (P.trace && row == 0 && tr_n < 64) P.trace[((size_t)blockIdx.x * (NG + 1) + wg) * 64 + tr_n++] = clock64();
    };
    stamp();
    auto gtime = [] { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; };
    unsigned long long* rg = nullptr;
    if (P.ring && tid == 0) {
        unsigned long long* r = P.ring + 8 + (size_t)P.ring_slot * 8;
        atomicMax(r + 7, gtime());  // the last CTA to start
        if (blockIdx.x == 0) {
            rg = r;
            atomicAdd(P.ring, 1ull);
            rg[0] = gtime();
            rg[5] = ((unsigned long long)p.n << 32) | (unsigned)p.k;
        }
    }

    // refill state of a group's thread 0: the block NS after the group's current one (position in its tile, tile)
    int rq_rem = 0, rq_tile = 0;
    auto request = [&](int st, int rem, int tile) {
        const int mat = rem >= nunits ? 1 : 0, unit = rem - mat * nunits;
        mbar_expect_tx(&raw_full[st], kRawBytes);
        tma_load_2d(raw + (size_t)st * kRawBytes, mat ? &tm1 : &tm0, unit * 36, tile * kRows, &raw_full[st]);
    };

    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < NS; s++) mbar_init(&raw_full[s], 1);
            for (int g = 0; g < NG; g++) mbar_init(&acc_full[g], 4);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            int tile = b_begin / bpt, rem = b_begin - tile * bpt;
            for (int i = 0; i < NS && i < L; i++) {  // weights do not depend on the previous kernel
                request(i, rem, tile);
                if (++rem == bpt) { rem = 0; tile++; }
            }
        }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (row == 0) {  // block wg + NS, the first this thread will re-request
        const int b = b_begin + wg + NS;
        rq_tile = b / bpt;
        rq_rem = b - rq_tile * bpt;
    }
    if (tid == 1) {
        l2_prefetch_part(p.prefetch.p[0], p.prefetch.bytes[0], blockIdx.x, gridDim.x);
        l2_prefetch_part(p.prefetch.p[1], p.prefetch.bytes[1], blockIdx.x, gridDim.x);
    }
    // gains of the units this warp will quantise: they do not depend on the previous kernel either
    float nw[2][8];
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int j = 0; j < 8; j++) nw[r][j] = 1.f;
    auto unit_of_slot = [&](int s) {
        if (all_units) return s;
        const int rem = (b_begin + s) % bpt;
        return rem >= nunits ? rem - nunits : rem;
    };
    if (p.norm_w && !issuer_warp) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int s = warp + r * GW;
            if (s < nslots) {
                const float4* np = reinterpret_cast<const float4*>(p.norm_w + unit_of_slot(s) * kUnitElems + 8 * lane);
                const float4 n0 = np[0], n1 = np[1];
                nw[r][0] = n0.x; nw[r][1] = n0.y; nw[r][2] = n0.z; nw[r][3] = n0.w;
                nw[r][4] = n1.x; nw[r][5] = n1.y; nw[r][6] = n1.z; nw[r][7] = n1.w;
            }
        }
    }
    pdl_launch_dependents();
    pdl_wait();
    stamp();
    if (rg) rg[1] = gtime();

    // ---- activations -> fixed-point planes of the units this CTA meets, in the B-operand layout: per sub-block
    //      [k chunk 2][row 8][16 B], row = 3 * token + plane (the other rows hold don't-care bytes whose products land
    //      in accumulator columns nobody reads).  Warp w takes slots w, w + GW, ...; the first two are loaded before the
    //      RMS reduction so that one memory round trip covers both ----
    auto quantise = [&](int s, int tk, const float (&v)[8]) {
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(v[j]));
        amax = warp_max(amax);
        // amax = f * 2^ex with f in [0.5, 1): ex from the exponent field (zero, denormal and non-finite inputs fall into the clamp)
        const int ex = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 126;
        const int sh = max(-100, min(100, 22 - ex));  // |x| * 2^sh < 2^22
        const float up = __uint_as_float((uint32_t)(127 + sh) << 23), dn = __uint_as_float((uint32_t)(127 - sh) << 23);
        uint32_t pw[3][2] = {{0, 0}, {0, 0}, {0, 0}};
        int xsum = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float sv = v[j] * up;
            sv = fminf(fmaxf(sv, -4194304.f), 4194304.f);
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
        unsigned char* bp = planes + ((size_t)s * 8 + sb) * 256 + (inner >> 4) * 128 + (inner & 15);
#pragma unroll
        for (int pl = 0; pl < 3; pl++) *reinterpret_cast<uint2*>(bp + (3 * tk + pl) * 16) = make_uint2(pw[pl][0], pw[pl][1]);
        xsum += __shfl_xor_sync(0xffffffffu, xsum, 1);
        xsum += __shfl_xor_sync(0xffffffffu, xsum, 2);
        if ((lane & 3) == 0) sxf[((size_t)s * M + tk) * 8 + sb] = (float)xsum * dn;
        if (lane == 0) inv2s[(size_t)s * M + tk] = dn * 0.0625f;  // 2^-sh and the factor 16 the integer sums carry
    };
    auto load_x = [&](int s, int tk, float (&v)[8]) {
        const float4* xp = reinterpret_cast<const float4*>(p.x + (size_t)tk * p.k + unit_of_slot(s) * kUnitElems + 8 * lane);
        const float4 u0 = xp[0], u1 = xp[1];
        v[0] = u0.x; v[1] = u0.y; v[2] = u0.z; v[3] = u0.w; v[4] = u1.x; v[5] = u1.y; v[6] = u1.z; v[7] = u1.w;
    };
    {
        float xv[2][M][8];
        if (!issuer_warp) {
#pragma unroll
            for (int r = 0; r < 2; r++)
#pragma unroll
                for (int tk = 0; tk < M; tk++)
                    if (warp + r * GW < nslots) load_x(warp + r * GW, tk, xv[r][tk]);
        }
        float rms[M];
#pragma unroll
        for (int tk = 0; tk < M; tk++) rms[tk] = 1.f;
        if (p.norm_w) {  // cpu.rs:49-60
#pragma unroll
            for (int tk = 0; tk < M; tk++) {
                float ss = 0.f;
                if (!issuer_warp)
                    for (int i = tid; i < p.k; i += GT) { const float v = p.x[(size_t)tk * p.k + i]; ss = fmaf(v, v, ss); }
                ss = warp_sum(ss);
                if (lane == 0 && !issuer_warp) scratch[tk * GW + warp] = ss;
            }
            __syncthreads();
#pragma unroll
            for (int tk = 0; tk < M; tk++) {
                float r = 0.f;
#pragma unroll
                for (int w = 0; w < GW; w++) r += scratch[tk * GW + w];
                rms[tk] = 1.0f / sqrtf(r / (float)p.k + p.eps);
            }
        }
        if (!issuer_warp) {
#pragma unroll
            for (int r = 0; r < 2; r++)
#pragma unroll
                for (int tk = 0; tk < M; tk++)
                    if (warp + r * GW < nslots) {
                        if (p.norm_w) {
#pragma unroll
                            for (int j = 0; j < 8; j++) xv[r][tk][j] = (xv[r][tk][j] * rms[tk]) * nw[r][j];
                        }
                        quantise(warp + r * GW, tk, xv[r][tk]);
                    }
            for (int s = warp + 2 * GW; s < nslots; s += GW) {  // long per-CTA runs only
                float gw[8];
                if (p.norm_w) {
                    const float4* np = reinterpret_cast<const float4*>(p.norm_w + unit_of_slot(s) * kUnitElems + 8 * lane);
                    const float4 n0 = np[0], n1 = np[1];
                    gw[0] = n0.x; gw[1] = n0.y; gw[2] = n0.z; gw[3] = n0.w; gw[4] = n1.x; gw[5] = n1.y; gw[6] = n1.z; gw[7] = n1.w;
                }
#pragma unroll
                for (int tk = 0; tk < M; tk++) {
                    float v[8];
                    load_x(s, tk, v);
                    if (p.norm_w) {
#pragma unroll
                        for (int j = 0; j < 8; j++) v[j] = (v[j] * rms[tk]) * gw[j];
                    }
                    quantise(s, tk, v);
                }
            }
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the planes are read by the tensor core
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    stamp();
    if (rg) rg[2] = gtime();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t pl_saddr = smem_u32(planes);

    {
        // ---- the groups ----
        // tensor memory of this group: columns [128 wg, +64) the A operand, [+64, +128) the accumulators; this warp
        // reaches lanes 32 (warp % 4) ..
        const uint32_t tgrp = tmem_base + (uint32_t)(wg * 128) + ((uint32_t)((warp & 3) * 32) << 16);

        float y[2][M];
#pragma unroll
        for (int a = 0; a < 2; a++)
#pragma unroll
            for (int b = 0; b < M; b++) y[a][b] = 0.f;
        bool ok = true;
        int i = wg;                // this group's next block; its stage and the stage's phase follow without divisions
        int st = wg % NS, st_par = 0, par = 0;

        int seg = 0;
        for (int i0 = 0; i0 < L; seg++) {
            const int tile = (b_begin + i0) / bpt;
            const int i1 = min(L, (tile + 1) * bpt - b_begin);
            for (; i < i1; i += NG) {
                const int rem = (b_begin + i) - tile * bpt;
                const int mat = rem >= nunits ? 1 : 0, unit = rem - mat * nunits;
                const int slot = all_units ? unit : i;
                ok = mbar_wait(&raw_full[st], (uint32_t)st_par) && ok;
                stamp();
                const unsigned char* rp = raw + (size_t)st * kRawBytes + row * 144;
                const uint4 hdr = *reinterpret_cast<const uint4*>(rp);
                // masked nibbles -> the group's A operand: sub-block j in columns 8j.., word t of a 16-byte k chunk in column t
#pragma unroll
                for (int h = 0; h < 4; h++) {  // 64 weights = sub-blocks 2h (low nibbles) and 2h + 1 (high nibbles)
                    const uint4 q0 = *reinterpret_cast<const uint4*>(rp + 16 + 32 * h);
                    const uint4 q1 = *reinterpret_cast<const uint4*>(rp + 32 + 32 * h);
                    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                    uint32_t a[16];
#pragma unroll
                    for (int t = 0; t < 8; t++) { a[t] = w[t] & 0x0F0F0F0Fu; a[8 + t] = w[t] & 0xF0F0F0F0u; }
                    tmem_st16(tgrp + 16 * h, a);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                asm volatile("bar.sync %0, 128;" ::"r"(wg + 1) : "memory");  // the group's A operand is complete, its stage is read
                if (lane == 0) {
                    tc_fence_after();
                    const uint32_t ta = tmem_base + (uint32_t)(wg * 128);
                    const uint64_t db = umma_desc(pl_saddr + (uint32_t)(slot * kPlaneBytes), 128, 256);
#pragma unroll
                    for (int jj = 0; jj < 2; jj++) {  // sub-block j: 8 columns of A, 256 B of B (the address field counts 16-byte units)
                        const int j = 2 * (warp & 3) + jj;
                        umma_i8_ts(ta + 64 + 8 * j, ta + 8 * j, db + (uint64_t)(j * 16));
                    }
                    umma_commit(&acc_full[wg]);  // one of the group's four arrivals
                    if (row == 0 && i + NS < L) {
                        request(st, rq_rem, rq_tile);
                        rq_rem += NG;
                        while (rq_rem >= bpt) { rq_rem -= bpt; rq_tile++; }
                    }
                }
                stamp();
                if ((st += NG) >= NS) { st -= NS; st_par ^= 1; }

                // scales and offsets of this row while the tensor core works
                uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
                unpack_scales_k4(hdr.y, hdr.z, hdr.w, &sc_lo, &sc_hi, &mn_lo, &mn_hi);
                const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));  // (d, dmin)
                float mt[M];
#pragma unroll
                for (int tk = 0; tk < M; tk++) {
                    const float4 sa = *reinterpret_cast<const float4*>(sxf + ((size_t)slot * M + tk) * 8);
                    const float4 sb4 = *reinterpret_cast<const float4*>(sxf + ((size_t)slot * M + tk) * 8 + 4);
                    mt[tk] = (((float)(mn_lo & 0xFFu) * sa.x + (float)((mn_lo >> 8) & 0xFFu) * sa.y) +
                              ((float)((mn_lo >> 16) & 0xFFu) * sa.z + (float)(mn_lo >> 24) * sa.w)) +
                             (((float)(mn_hi & 0xFFu) * sb4.x + (float)((mn_hi >> 8) & 0xFFu) * sb4.y) +
                              ((float)((mn_hi >> 16) & 0xFFu) * sb4.z + (float)(mn_hi >> 24) * sb4.w));
                }

                // the eight sub-block sums of this row: scales as integer multiplies, planes and offsets in f32
                __syncwarp();
                ok = mbar_wait(&acc_full[wg], (uint32_t)par) && ok;
                par ^= 1;
                tc_fence_after();
                uint32_t c[8][NC];
#pragma unroll
                for (int j = 0; j < 8; j++) tmem_ld<NC>(tgrp + 64 + 8 * j, c[j]);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tc_fence_before();
                stamp();
                int acc[M][3];
#pragma unroll
                for (int tk = 0; tk < M; tk++) acc[tk][0] = acc[tk][1] = acc[tk][2] = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint32_t w = (j < 4) ? sc_lo : sc_hi;
                    int sc = (int)((w >> (8 * (j & 3))) & 0xFFu);
                    if ((j & 1) == 0) sc <<= 4;  // low-nibble sub-block; the high-nibble ones carry the 16 in their bytes
#pragma unroll
                    for (int tk = 0; tk < M; tk++)
#pragma unroll
                        for (int pl = 0; pl < 3; pl++) acc[tk][pl] += sc * (int)c[j][3 * tk + pl];
                }
#pragma unroll
                for (int tk = 0; tk < M; tk++) {
                    const float S = ((float)acc[tk][0] + 256.f * (float)acc[tk][1]) + 65536.f * (float)acc[tk][2];
                    const float dy = (dd.x * inv2s[(size_t)slot * M + tk]) * S - dd.y * mt[tk];
                    y[0][tk] += mat ? 0.f : dy;
                    y[1][tk] += mat ? dy : 0.f;
                }
                stamp();
            }
            if (rg) rg[3] = gtime();

            // ---- the tile's row sums: the groups in order, then across CTAs ----
            float* rb = red + (size_t)((seg & 1) * NG + wg) * (2 * M * kRows);
#pragma unroll
            for (int mt = 0; mt < 2; mt++)
#pragma unroll
                for (int tk = 0; tk < M; tk++) { rb[(mt * M + tk) * kRows + row] = y[mt][tk]; y[mt][tk] = 0.f; }
            asm volatile("bar.sync %0, %1;" ::"r"(NG + 1), "r"(GT) : "memory");
            if (wg == 0) {
                const float* r0 = red + (size_t)((seg & 1) * NG) * (2 * M * kRows);
                float v[2][M];
#pragma unroll
                for (int mt = 0; mt < 2; mt++)
#pragma unroll
                    for (int tk = 0; tk < M; tk++) {
                        float a = r0[(mt * M + tk) * kRows + row];
#pragma unroll
                        for (int g = 1; g < NG; g++) a += r0[(size_t)g * (2 * M * kRows) + (mt * M + tk) * kRows + row];
                        v[mt][tk] = a;
                    }
                const long long B0 = (long long)tile * bpt;
                const int c_first = (int)(((B0 + 1) * gridDim.x - 1) / Btot);
                const int c_last = (int)(((B0 + bpt) * gridDim.x - 1) / Btot);
                const int nc = c_last - c_first + 1;
                (void)flag;
                bool fin = true;
                if (nc > 1) {
                    // Each partial travels as one 64-bit word (f32 bits, valid = 1), so a reader that sees the flag sees
                    // the value: no fence, no counter.  The tile is finished by its FIRST CTA, which meets the tile at
                    // the end of its run of blocks while the others meet it at the start of theirs and are long done;
                    // it adds the partials in CTA order and leaves the slots cleared for the next launch.
                    unsigned long long* slots = P.partial + (size_t)tile * P.max_contrib * (2 * M * kRows);
                    const int me = (int)blockIdx.x - c_first;
                    fin = me == 0;
                    if (!fin) {
#pragma unroll
                        for (int mt = 0; mt < 2; mt++)
#pragma unroll
                            for (int tk = 0; tk < M; tk++)
                                if (mt < nmat) {
                                    const unsigned long long w = (1ull << 32) | (unsigned long long)__float_as_uint(v[mt][tk]);
                                    asm volatile("st.global.relaxed.gpu.u64 [%0], %1;" ::"l"(slots + ((size_t)me * 2 * M + mt * M + tk) * kRows + row), "l"(w) : "memory");
                                }
                    } else {
                        for (int c = 1; c < nc; c++)
#pragma unroll
                            for (int mt = 0; mt < 2; mt++)
#pragma unroll
                                for (int tk = 0; tk < M; tk++)
                                    if (mt < nmat) {
                                        unsigned long long* sp = slots + ((size_t)c * 2 * M + mt * M + tk) * kRows + row;
                                        unsigned long long w = 0;
                                        bool got = false;
                                        for (uint32_t it = 0; it < (1u << 20) && !got; ++it) {
                                            asm volatile("ld.global.relaxed.gpu.u64 %0, [%1];" : "=l"(w) : "l"(sp) : "memory");
                                            got = (w >> 32) == 1ull;
                                        }
                                        ok = ok && got;
                                        v[mt][tk] += __uint_as_float((uint32_t)w);
                                        asm volatile("st.global.relaxed.gpu.u64 [%0], %1;" ::"l"(sp), "l"(0ull) : "memory");
                                    }
                    }
                }
                const int grow = tile * kRows + row;
                if (fin && grow < p.n) {
#pragma unroll
                    for (int tk = 0; tk < M; tk++) {
                        float o = v[0][tk];
                        if (p.epi == EPI_SILU_MUL) o = silu_f(o) * v[1][tk];
                        else if (p.epi == EPI_ADD_RESIDUAL) o = p.residual[(size_t)tk * p.n + grow] + o;
                        p.out[(size_t)tk * p.n + grow] = o;
                    }
                }
            }
            i0 = i1;
            stamp();
        }
        if (!ok && row == 0 && p.error_flag) atomicExch(p.error_flag, 1);
    }
    if (rg) rg[4] = gtime();
    if (P.ring && tid == 0) atomicMax(P.ring + 8 + (size_t)P.ring_slot * 8 + 6, gtime());  // the last CTA to finish its work
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// ---------------------------------------------------------------------------
namespace {

struct UmmaScratch { DevBuf partial; };
unsigned long long* g_ring = nullptr;
void dump_ring() {
    static unsigned long long h[8 + 1024 * 8];
    if (!g_ring || cudaMemcpy(h, g_ring, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return;
    fprintf(stderr, "[gemv ring] %llu launches; per launch slot, times in ns relative to CTA 0's start of the slot before:\n"
                    "  slot n k | cta0 start, last cta start | wait done, prologue done, blocks done, cta0 end | last cta end\n", h[0]);
    unsigned long long base = 0;
    for (int i = 0; i < 1024; i++) {
        const unsigned long long* r = h + 8 + (size_t)i * 8;
        if (!r[0]) continue;
        if (!base) base = r[0];
        fprintf(stderr, "  %4d %6llu %6llu | %7lld %7lld | %7lld %7lld %7lld %7lld | %7lld\n", i, r[5] >> 32, r[5] & 0xffffffffu, (long long)(r[0] - base),
                (long long)(r[7] - base), (long long)(r[1] - base), (long long)(r[2] - base), (long long)(r[3] - base), (long long)(r[4] - base),
                (long long)(r[6] - base));
        base = r[0];
    }
}
UmmaScratch g_umma[16];

struct UmmaPlan {
    int grid, nslots, nstages, max_contrib, ntiles;
    size_t smem, partial_bytes;
    bool fits;
};

template <int M, int NG>
UmmaPlan umma_plan(int n, int k, bool two_mats) {
    UmmaPlan pl = {};
    const int nunits = k / kUnitElems, nmat = two_mats ? 2 : 1, bpt = nunits * nmat;
    pl.ntiles = (n + kRows - 1) / kRows;
    const long long Btot = (long long)pl.ntiles * bpt;
    pl.grid = (int)std::min<long long>(sm_count(), Btot);
    const int lmax = (int)((Btot + pl.grid - 1) / pl.grid);
    pl.nslots = std::min(lmax, nunits);
    size_t fixed = 1024 + (size_t)pl.nslots * kPlaneBytes + (size_t)pl.nslots * M * 9 * 4 +
                   (size_t)2 * NG * 2 * M * kRows * 4 + (size_t)(NG * 4 * M + M) * 4 + 8 + (size_t)(kMaxStages + NG) * 8 + 16;
    pl.nstages = fixed + 2 * (size_t)kRawBytes <= kMaxSmem ? (int)std::min<size_t>(kMaxStages, (kMaxSmem - fixed) / kRawBytes) : 0;
    pl.fits = pl.nstages >= 2;
    pl.smem = fixed + (size_t)pl.nstages * kRawBytes;
    pl.max_contrib = 1;
    for (int t = 0; t < pl.ntiles; t++) {
        const long long B0 = (long long)t * bpt;
        const int c_first = (int)(((B0 + 1) * pl.grid - 1) / Btot), c_last = (int)(((B0 + bpt) * pl.grid - 1) / Btot);
        pl.max_contrib = std::max(pl.max_contrib, c_last - c_first + 1);
    }
    pl.partial_bytes = (size_t)pl.ntiles * pl.max_contrib * 2 * M * kRows * sizeof(unsigned long long);
    return pl;
}

int32_t umma_reserve(int dev, size_t partial_bytes) {
    UmmaScratch& sc = g_umma[dev];
    if (sc.partial.cap >= partial_bytes) return LC_OK;
    LC_CUDA(cudaStreamSynchronize(stream()));  // no kernel may still be using the old buffer
    LC_TRY(sc.partial.reserve(partial_bytes));
    LC_CUDA(cudaMemset(sc.partial.p, 0, sc.partial.cap));  // every slot invalid; the kernel leaves them so
    if (!g_ring && getenv("LC_GEMV_RING")) {
        LC_CUDA(cudaMalloc(&g_ring, (8 + 1024 * 8) * sizeof(unsigned long long)));
        LC_CUDA(cudaMemset(g_ring, 0, (8 + 1024 * 8) * sizeof(unsigned long long)));
        atexit(dump_ring);
    }
    return LC_OK;
}

template <int M, int NG>
int32_t launch_umma_m(const GemvArgs& a, cudaStream_t s, bool* launched) {
    const UmmaPlan pl = umma_plan<M, NG>(a.w->n, a.w->k, a.epi == EPI_SILU_MUL);
    if (!pl.fits) return LC_OK;
    int dev = 0;
    LC_CUDA(cudaGetDevice(&dev));
    LC_CHECK(dev >= 0 && dev < 16, LC_ERR_INVALID, "device ordinal %d out of range", dev);
    UmmaScratch& sc = g_umma[dev];
    if (sc.partial.cap < pl.partial_bytes) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        LC_CUDA(cudaStreamIsCapturing(s, &cs));
        LC_CHECK(cs == cudaStreamCaptureStatusNone, LC_ERR_STATE,
                 "qgemv: the split-tile scratch must be reserved (qgemv_reserve_scratch) before a stream capture");
        LC_TRY(umma_reserve(dev, pl.partial_bytes));
    }
    auto kern = qgemv_umma_q4k_kernel<M, NG>;
    static bool attr_set = false;
    if (!attr_set) {
        LC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmem));
        attr_set = true;
    }
    UmmaParams P;
    GemvParams& p = P.g;
    p.x = a.x; p.out = a.out; p.residual = a.residual; p.norm_w = a.norm_w; p.eps = a.eps;
    p.n = a.w->n; p.k = a.w->k; p.m = a.m; p.epi = (int)a.epi; p.error_flag = gemv_error_flag_dev();
    p.prefetch = a.prefetch;
    P.partial = (unsigned long long*)sc.partial.p;
    P.max_contrib = pl.max_contrib;
    P.nslots = pl.nslots;
    P.nstages = pl.nstages;
    P.trace = nullptr;
    P.ring = g_ring;
    static int ring_seq = 0;
    P.ring_slot = ring_seq++ % 1024;
    static const bool want_trace = getenv("LC_GEMV_TRACE") != nullptr;
    static long long* trace_dev = nullptr;
    static int traced = 0;
    const bool tracing = want_trace && traced < 6;
    if (tracing) {
        if (!trace_dev) LC_CUDA(cudaMalloc(&trace_dev, (size_t)256 * 8 * 64 * sizeof(long long)));
        LC_CUDA(cudaMemsetAsync(trace_dev, 0, (size_t)256 * 8 * 64 * sizeof(long long), s));
        P.trace = trace_dev;
    }
    const CUtensorMap* t0 = (const CUtensorMap*)a.w->tmap_wide;
    const CUtensorMap* t1 = a.w2 ? (const CUtensorMap*)a.w2->tmap_wide : t0;
    LC_CUDA(launch_pdl(kern, dim3(pl.grid), dim3(NG * 128), pl.smem, s, *t0, *t1, P));
    if (tracing) {  // diagnostics: per-group clock stamps of three CTAs, relative to the CTA's first stamp
        traced++;
        static long long h[256 * 8 * 64];
        LC_CUDA(cudaStreamSynchronize(s));
        LC_CUDA(cudaMemcpy(h, trace_dev, sizeof(h), cudaMemcpyDeviceToHost));
        fprintf(stderr, "[gemv trace] n=%d k=%d epi=%d grid=%d stages=%d slots=%d contrib=%d\n", p.n, p.k, p.epi, pl.grid, pl.nstages,
                pl.nslots, pl.max_contrib);
        const int ctas[3] = {0, pl.grid / 2, pl.grid - 1};
        for (int ci = 0; ci < 3; ci++)
            for (int g = 0; g <= NG; g++) {
                const long long* t = h + ((size_t)ctas[ci] * (NG + 1) + g) * 64;
                fprintf(stderr, "  cta %3d group %d:", ctas[ci], g);
                for (int i = 1; i < 64 && t[i]; i++) fprintf(stderr, " %lld", t[i] - t[0]);
                fprintf(stderr, "\n");
            }
    }
    *launched = true;
    return LC_OK;
}

}  // namespace

// Makes sure no later launch for an [n x k] Q4_K matrix (m <= 2 tokens) has to allocate: call before a stream capture.
int32_t qgemv_reserve_scratch(int n, int k, bool two_mats) {
    if (k % kUnitElems != 0) return LC_OK;
    int dev = 0;
    LC_CUDA(cudaGetDevice(&dev));
    LC_CHECK(dev >= 0 && dev < 16, LC_ERR_INVALID, "device ordinal %d out of range", dev);
    const UmmaPlan pl = umma_plan<2, 4>(n, k, two_mats);  // the grid, and with it the split, does not depend on the group count
    return umma_reserve(dev, pl.partial_bytes);
}

int32_t launch_qgemv_umma_q4k(const GemvArgs& a, cudaStream_t s, bool* launched) {
    *launched = false;
    if (a.m > 2 || a.w->k % kUnitElems != 0) return LC_OK;
    if (((uintptr_t)a.x % 16) != 0 || (a.norm_w && ((uintptr_t)a.norm_w % 16) != 0)) return LC_OK;
    return a.m == 1 ? launch_umma_m<1, 4>(a, s, launched) : launch_umma_m<2, 4>(a, s, launched);
}

}  // namespace lc

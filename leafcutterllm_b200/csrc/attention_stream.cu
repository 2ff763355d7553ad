// Decode attention of ONE new token as a balanced stream over the paged f16 KV cache
// (rust/src/inference/attention.rs:69-113, rust/src/cache/mod.rs:33-77; head_dim 128, 16-token pages).
//
// The unit of work is a (kv head, page) item: one 4 KB slab of keys and one of values.  The items of the token, in
// (kv head, page) order, are cut into one contiguous run per CTA -- CTA c takes items [c*T/G, (c+1)*T/G) -- so every
// SM streams the same number of bytes whatever the context length and head count, and there is a single wave.
//
//   producer  a warp requests the run's slabs with bulk copies into a ring of stages (one mbarrier each), each lane
//             looking up its own page-table entries, starting BEFORE the kernel looks at its input: cached pages belong
//             to earlier steps.  Keys are copied row by row into a 272-byte pitch, values as one 4 KB piece;
//   consumers the other warps take the items round robin.  A warp scores the 16 keys of its page (lane = key, the two half
//             warps take the two halves of the head; with the padded pitch a 16-byte chunk of 8 consecutive keys spans
//             all banks and the query chunk is one broadcast read), updates an online softmax per query head of the kv
//             group and accumulates p.V with four dims per lane;
//   new token the warp that owns the page holding this step's position rotates k, rounds k and v through f16 exactly
//             as the cache does, patches its staged copy and stores the row into the cache;
//   merge     per (kv head) segment the warps are combined in warp order, then the CTAs that share the segment in CTA
//             order: every CTA but the segment's last publishes (max, sum, weighted V) as 64-bit words carrying a
//             valid flag; the last one collects them, writes the head's output and leaves the slots cleared.
//
// The reference's three-pass softmax and this online form agree to rounding; sums are in a fixed order, so results
// do not vary from run to run.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include "lc_kernels.h"
#include "lc_attn.cuh"
#include "lc_tma.cuh"

namespace lc {

namespace {

constexpr int kHD = 128;
constexpr int kPage = 16;
constexpr int kSlab = kPage * kHD * 2;       // bytes of one K (or V) slab in the cache
// A stage: the page's keys as two TMA boxes of 16 rows x 64 dims (128-byte rows, 128-byte swizzle: the 16-byte chunk j of
// row r sits at chunk j ^ (r & 7), which is what lets ldmatrix read 8 rows of one chunk without a bank conflict), then
// the page's values as one 4 KB piece.
constexpr int kKHalf = kPage * 128;          // one box
constexpr int kStageBytes = 2 * kSlab;
constexpr int kMaxSeg = 3;                   // kv heads a CTA's run can touch (n_kv <= SM count)
constexpr int kStateWords = 4 + kHD;         // max, sum, two pad words (16-byte alignment), weighted V

struct StreamParams {
    AttnParams a;
    unsigned long long* slots;  // polled merge: [q head][contributor][2 + kHD] words (f32 bits | valid << 32), zero between launches;
                                // ticket merge: the same room as f32 [q head][contributor][2 + kHD], then one ticket word per kv head
    int max_contrib;
    int ticket_merge;           // see the merge at the end of the kernel
    int head_cap;               // most CTAs that share one kv head's pages (0: no limit)
    int nstages;
    unsigned long long* ring;  // diagnostics (LC_ATTN_RING): [launch slot][8] wall-clock stamps, or null
    int ring_slot;
};

// Consumer warps: the per-page work is a chain of dependent shared-memory loads, shuffles and FMAs, so throughput comes
// from the number of warps in flight -- fifteen where the per-warp state of the kv group fits (with the producer warp
// a CTA of 512 threads, which leaves each thread 128 registers), seven for wide groups.
template <int GSZ>
__host__ __device__ constexpr int consumer_warps() { return GSZ <= 2 ? 15 : 7; }

template <int GSZ>
__global__ void __launch_bounds__((consumer_warps<GSZ>() + 1) * 32, 1)
attention_stream_kernel(const __grid_constant__ CUtensorMap ktm, const __grid_constant__ CUtensorMap vtm, StreamParams P) {
    constexpr int kCWarps = consumer_warps<GSZ>();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzle atoms are 1 KB
    const AttnParams& p = P.a;
    const KvLayout& kv = p.kv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = P.nstages;
    unsigned char* ring = smem;                                             // [S][kStageBytes]
    constexpr int NTc = (2 * GSZ + 7) / 8;                                  // n tiles of the score product (see below)
    float* q_s = reinterpret_cast<float*>(ring + (size_t)S * kStageBytes);  // [kMaxSeg][GSZ][kHD] rotated queries of the run's kv heads
    uint32_t* qf_s = reinterpret_cast<uint32_t*>(q_s + kMaxSeg * GSZ * kHD);  // [kMaxSeg][NTc][16][32] their B fragments, lane-major
    float* st_s = reinterpret_cast<float*>(qf_s + kMaxSeg * NTc * 16 * 32);   // [kMaxSeg][kCWarps][GSZ][kStateWords]
    float* cta_s = st_s + kMaxSeg * kCWarps * GSZ * kStateWords;            // [kMaxSeg][GSZ][kStateWords] combined over warps
    uint64_t* full = reinterpret_cast<uint64_t*>(((uintptr_t)(cta_s + kMaxSeg * GSZ * kStateWords) + 7) & ~(uintptr_t)7);  // [S]
    uint64_t* empty = full + S;                                             // [S]
    // armed[st] = how many times the producer has armed stage st.  A stage's rounds are consumed by DIFFERENT warps, and a
    // parity wait cannot tell "round r has not completed" from "round r - 1 has not completed": a warp that reached its
    // round-r item while the stage's round r - 1 data was still in flight would pass the wait and read the wrong page
    // (seen with cold caches, when copies requested together land microseconds apart).  So a consumer of round r >= 1
    // first waits until the producer says it has armed round r -- which it only does after round r - 1 was consumed.
    volatile int* armed = reinterpret_cast<volatile int*>(empty + S);       // [S]
    volatile int* s_last = armed + S;                                       // merge: this CTA took the last ticket of a head

    auto gtime = [] { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; };
    unsigned long long* rg = (P.ring && tid == 0) ? P.ring + (size_t)P.ring_slot * 16 : nullptr;
    if (rg) { atomicMax(rg + 7, gtime()); if (blockIdx.x == 0) rg[0] = gtime(); else rg = nullptr; }
    if (tid == 0) {
        for (int s = 0; s < S; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); armed[s] = 0; }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();
    if (!p.positions_settled) pdl_wait();  // the position itself may still be in flight

    // the token's items: (kv head, page), kv head major
    const int pos = p.tok_pos[0];
    const int np = pos / kPage + 1;
    const int T = kv.n_kv * np;
    // CTAs that take part: about four items each where a head has that many pages (fewer, larger shares to add up).  The
    // share per CTA never exceeds one head's pages (T / min(4, np) >= n_kv CTAs), so a run touches at most two kv heads.
    const int min_items = max(max(1, min(4, np)), P.head_cap > 0 ? (np + P.head_cap - 1) / P.head_cap : 0);
    const int G = min((int)gridDim.x, max(1, T / min_items));
    const bool active = (int)blockIdx.x < G;
    const int i_begin = active ? (int)((long long)blockIdx.x * T / G) : 0;
    const int i_end = active ? (int)((long long)(blockIdx.x + 1) * T / G) : 0;
    const int n_items = i_end - i_begin;
    const int seg0 = n_items > 0 ? i_begin / np : 0;  // first kv head of the run
    const int32_t* pt = p.page_table + (size_t)p.tok_seq[0] * p.pages_per_seq;
    bool ok = true;

    if (warp == kCWarps) {
        // ---- producer: lane i requests items i, i + 32, ... -- each needs a page-table entry from global memory, and one
        //      thread walking them one after the other made that latency, not HBM, the pace of the whole kernel ----
        // Producing lanes: min(32, S) = S (at most 26 stages fit), so that a lane's items all use one stage and a lane only
        // ever waits for the consumption of its OWN previous item: it has seen every earlier phase of that stage's
        // `empty` barrier complete, which keeps its parity waits unambiguous.  With 32 lanes over fewer stages a lane could wait for an item that a lane
        // of the same round has yet to request; lanes that need no wait can be held at the reconvergence point behind the
        // waiting ones, and then nobody requests it.
        const int PL = S < 32 ? S : 32;
        for (int i = lane; lane < PL && i < n_items; i += PL) {
            const int gi = i_begin + i;
            const int kvh = gi / np, page = gi - kvh * np;
            const int pg = pt[page];
            const int st = i % S;
            if (i >= S && !mbar_wait(&empty[st], (uint32_t)((i / S - 1) & 1))) { ok = false; break; }  // never arm a barrier that is still pending
            mbar_expect_tx(&full[st], kStageBytes);
            unsigned char* dst = ring + (size_t)st * kStageBytes;
            const int y = (pg * kv.n_kv + kvh) * kPage;  // first row of the slab in the pool seen as [rows][128]
            tma_load_2d(dst, &ktm, 0, y, &full[st]);
            tma_load_2d(dst + kKHalf, &ktm, 64, y, &full[st]);
            tma_load_2d(dst + 2 * kKHalf, &vtm, 0, y, &full[st]);
            tma_load_2d(dst + 3 * kKHalf, &vtm, 64, y, &full[st]);
            __threadfence_block();      // the arming above is visible before the count below
            armed[st] = i / S + 1;
        }
        if (!ok && p.error_flag) atomicExch(p.error_flag, 1);
        return;  // the producer takes no part in the barriers below (they count the consumer threads)
    }

    // ---- consumers ----
    pdl_wait();  // q and this step's k, v come from the projection kernel
    if (rg) rg[1] = gtime();
    const bool fused = p.k_new != nullptr;
    const int rp_of_step = fused ? p.tok_rope[0] : 0;
    // four dims of a head vector of the projection row, rotated (attention.rs:13-34)
    auto head_vec = [&](const float* plain, size_t off, float (&out4)[4]) { load_rotated<4, kHD>(plain + off, 4 * lane, rp_of_step, p.theta, out4); };
    // attention.rs:93-102: softmax(dot / sqrt(head_dim)).  Scores are kept multiplied by log2(e) so that every exponential is a
    // single ex2; the running maximum is in the same units and goes back to natural units when a warp's state is written out.
    const float sc_log2e = 1.4426950408889634f / sqrtf((float)kHD);

    // Scores run on the tensor cores: C[16 keys x 8 columns] per n tile, two columns (f16 hi and lo part of q) per query
    // head, so an n tile serves four heads and lane (row, t) of the C fragment belongs to head 4 nt + t.
    constexpr int NT = (2 * GSZ + 7) / 8;
    // p.V accumulators as C fragments of D[16 dims x 8 columns] per m tile (8 of them): this lane holds dims lane / 4 and
    // lane / 4 + 8 of each tile, columns hi / lo of head 4 nt + (lane & 3)
    float acc[NT][8][4];
    float m_own[NT], l_own[NT];  // running max and sum of head 4 nt + (lane & 3), kept by the lanes of that column
    uint32_t qf[NT][8][2];       // B fragments of the segment's queries, per n tile and 16-dim k tile
    auto reset = [&]() {
#pragma unroll
        for (int nt = 0; nt < NT; nt++) { m_own[nt] = -INFINITY; l_own[nt] = 0.f; }
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int mt = 0; mt < 8; mt++) acc[nt][mt][0] = acc[nt][mt][1] = acc[nt][mt][2] = acc[nt][mt][3] = 0.f;
    };
    reset();
    int cur_seg = -1;
    long long wait_cycles = 0;
    const long long loop0 = clock64();
    auto flush = [&](int seg) {  // this warp's state of kv head `seg` -> shared memory
        float* dst = st_s + ((size_t)(seg - seg0) * kCWarps + warp) * GSZ * kStateWords;
        {   // hi + lo columns of this lane's head: dims lane / 4 (+ 8) of every m tile
            const int t4 = lane & 3, dg = lane >> 2;
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
                if (4 * nt + t4 < GSZ) {
                    float* hd = dst + (4 * nt + t4) * kStateWords + 4;
#pragma unroll
                    for (int mt = 0; mt < 8; mt++) {
                        hd[mt * 16 + dg] = acc[nt][mt][0] + acc[nt][mt][1];
                        hd[mt * 16 + dg + 8] = acc[nt][mt][2] + acc[nt][mt][3];
                    }
                }
        }
        if (lane < 4) {  // lanes 0-3: row 0 of the C fragment, columns of heads 4 nt + lane
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
                if (4 * nt + lane < GSZ) {
                    dst[(4 * nt + lane) * kStateWords] = m_own[nt] * 0.6931471805599453f;  // back to natural-log units
                    dst[(4 * nt + lane) * kStateWords + 1] = l_own[nt];
                }
        }
    };
    // every (segment, warp) slot starts empty: a warp may meet no item of a segment
    for (int i = tid; i < kMaxSeg * kCWarps * GSZ; i += kCWarps * 32) {
        st_s[(size_t)i * kStateWords] = -INFINITY;
        st_s[(size_t)i * kStateWords + 1] = 0.f;
    }
    // ---- the queries of the run's kv heads, once per CTA: warp w stages head vector w, w + kCWarps, ... (rotated,
    //      attention.rs:13-34), then the B fragments of the score product are cut from them ----
    const int nseg_run = n_items > 0 ? (i_end - 1) / np - seg0 + 1 : 0;
    for (int hv = warp; hv < nseg_run * GSZ; hv += kCWarps) {
        const int sl = hv / GSZ, g = hv - sl * GSZ;
        float qv[4];
        head_vec(p.q, (size_t)((seg0 + sl) * GSZ + g) * kHD, qv);
        *reinterpret_cast<float4*>(q_s + (size_t)hv * kHD + 4 * lane) = make_float4(qv[0], qv[1], qv[2], qv[3]);
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kCWarps * 32) : "memory");
    // B operand of mma.m16n8k16 (16 dims x 8 columns): column 2h = f16(q of head 4 nt + h), column 2h + 1 = f16 of what
    // that rounding lost, so products with the f16 keys are exact and q keeps ~22 bits.  Lane (col = lane / 4, t = lane % 4)
    // holds column col, dims 2t, 2t+1 (register 0) and 2t+8, 2t+9 (register 1) of each 16-dim tile.
    for (int w = warp; w < nseg_run * NTc * 8; w += kCWarps) {  // one (segment, n tile, k tile) per warp and turn
        const int kt = w & 7, nt = (w >> 3) % NTc, sl = (w >> 3) / NTc;
        const int col = lane >> 2, t4 = lane & 3, hq = 4 * nt + (col >> 1);
#pragma unroll
        for (int r = 0; r < 2; r++) {
            uint32_t word = 0u;
            if (hq < GSZ) {
                const float2 x = *reinterpret_cast<const float2*>(q_s + (size_t)(sl * GSZ + hq) * kHD + kt * 16 + 2 * t4 + 8 * r);
                __half h0 = __float2half_rn(x.x), h1 = __float2half_rn(x.y);
                if (col & 1) { h0 = __float2half_rn(x.x - __half2float(h0)); h1 = __float2half_rn(x.y - __half2float(h1)); }
                const __half2 hh = __halves2half2(h0, h1);
                word = *reinterpret_cast<const uint32_t*>(&hh);
            }
            qf_s[(((size_t)sl * NTc + nt) * 16 + kt * 2 + r) * 32 + lane] = word;
        }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kCWarps * 32) : "memory");

    // this warp's items: il = warp, warp + kCWarps, ...; their kv head, page, stage and stage phase follow without divisions
    int kvh_i = n_items > 0 ? (i_begin + warp) / np : 0, page_i = n_items > 0 ? (i_begin + warp) - kvh_i * np : 0;
    int st_i = warp % S, rnd_i = warp / S;
    for (int il = warp; il < n_items; il += kCWarps) {
        const int kvh = kvh_i, page = page_i, st = st_i, rnd = rnd_i, st_par = rnd_i & 1;
        page_i += kCWarps;
        while (page_i >= np) { page_i -= np; kvh_i++; }
        st_i += kCWarps;
        while (st_i >= S) { st_i -= S; rnd_i++; }
        if (kvh != cur_seg) {
            if (cur_seg >= 0) flush(cur_seg);
            reset();
            cur_seg = kvh;
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 16; i++) qf[nt][i >> 1][i & 1] = qf_s[(((size_t)(kvh - seg0) * NTc + nt) * 16 + i) * 32 + lane];
        }
        if (rg && il == warp) rg[8] = clock64() - loop0;
        if (rnd > 0) {  // see `armed`: wait until this round of the stage has been armed (bounded)
            bool seen = false;
            for (uint32_t it = 0; it < (1u << 24) && !seen; ++it) seen = armed[st] > rnd;
            __threadfence_block();
            ok = ok && seen;
        }
        ok = mbar_wait(&full[st], (uint32_t)st_par) && ok;
        if (rg && il == warp) rg[9] = clock64() - loop0;
        unsigned char* K_b = ring + (size_t)st * kStageBytes;           // two swizzled boxes: dims 0-63, dims 64-127
        unsigned char* V_b = K_b + 2 * kKHalf;                          // values: the same two-box layout
        int nvalid = kPage;
        if (page == np - 1) {
            nvalid = pos % kPage + 1;
            if (fused) {
                // this step's token replaces the stale staged row: rotate, round through f16 (cache/mod.rs:35-36), keep in the cache
                const int r = pos % kPage;
                float kr[4];
                // in the projection row k follows the n_heads query heads and v follows the kv heads of k
                head_vec(p.k_new - (size_t)p.n_heads * kHD, (size_t)(p.n_heads + kvh) * kHD, kr);
                const float4 vr = __ldcg(reinterpret_cast<const float4*>(p.v_new + (size_t)kvh * kHD + 4 * lane));
                const __half2 k01 = __floats2half2_rn(kr[0], kr[1]), k23 = __floats2half2_rn(kr[2], kr[3]);
                const __half2 v01 = __floats2half2_rn(vr.x, vr.y), v23 = __floats2half2_rn(vr.z, vr.w);
                uint2 kw, vw;
                kw.x = *reinterpret_cast<const uint32_t*>(&k01); kw.y = *reinterpret_cast<const uint32_t*>(&k23);
                vw.x = *reinterpret_cast<const uint32_t*>(&v01); vw.y = *reinterpret_cast<const uint32_t*>(&v23);
                // dims 4 lane ..: box lane / 16, chunk (lane % 16) / 2 (swizzled by the row), 8 bytes into it for odd lanes
                *reinterpret_cast<uint2*>(K_b + (lane >> 4) * kKHalf + r * 128 + (((((lane & 15) >> 1) ^ (r & 7))) << 4) + (lane & 1) * 8) = kw;
                *reinterpret_cast<uint2*>(V_b + (lane >> 4) * kKHalf + r * 128 + (((((lane & 15) >> 1) ^ (r & 7))) << 4) + (lane & 1) * 8) = vw;
                const size_t dst = (((size_t)pt[page] * kv.n_kv + kvh) * kPage + r) * kHD + 4 * lane;
                *reinterpret_cast<uint2*>((__half*)kv.k_pool + dst) = kw;
                *reinterpret_cast<uint2*>((__half*)kv.v_pool + dst) = vw;
            }
            // value rows past this step's position hold whatever the pool held before (Inf, NaN): the tensor core would
            // multiply them with their zero weights, so they are cleared in the staged copy (a row is 128 bytes in each box)
            for (int ch = lane; ch < (kPage - nvalid) * 16; ch += 32) {
                const int rr = nvalid + (ch >> 4), cj = ch & 15;
                *reinterpret_cast<uint4*>(V_b + (cj >> 3) * kKHalf + rr * 128 + ((cj & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
        }
        {
            // ---- scores: C[16 keys x 8 columns] = K[16 x 128] . Q[128 x 8] per n tile, eight k tiles; keys through ldmatrix
            //      from the swizzled boxes (conflict free), accumulation in f32 ----
            float c[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
            const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;  // the row this lane addresses for ldmatrix
            const uint32_t lm_row = smem_u32(K_b) + (uint32_t)(lrow * 128);
#pragma unroll
            for (int kt = 0; kt < 8; kt++) {
                const int j = (kt & 3) * 2 + (lane >> 4);  // 16-byte chunk of the 128-byte row, box kt / 4
                uint32_t a0, a1, a2, a3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(lm_row + (kt >> 2) * kKHalf + ((j ^ (lrow & 7)) << 4)));
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(c[nt][0]), "+f"(c[nt][1]), "+f"(c[nt][2]), "+f"(c[nt][3])
                                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(qf[nt][kt][0]), "r"(qf[nt][kt][1]));
            }
            if (rg && il == warp) rg[10] = clock64() - loop0;
            // this lane: keys lane / 4 and lane / 4 + 8 of head 4 nt + (lane & 3) (hi + lo columns)
            const int kg = lane >> 2;
            float pe[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                // scores in units of log2(e): (dot / sqrt(head_dim)) * log2(e), so that exp() is one ex2
                const float s0 = (kg < nvalid) ? (c[nt][0] + c[nt][1]) * sc_log2e : -INFINITY;
                const float s1 = (kg + 8 < nvalid) ? (c[nt][2] + c[nt][3]) * sc_log2e : -INFINITY;
                float mx = fmaxf(s0, s1);
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const float m_new = fmaxf(m_own[nt], mx);  // finite: key 0 of every page is valid
                const float corr = exp2f(m_own[nt] - m_new);
                pe[nt][0] = exp2f(s0 - m_new);
                pe[nt][1] = exp2f(s1 - m_new);
                float ps = pe[nt][0] + pe[nt][1];
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
                l_own[nt] = l_own[nt] * corr + ps;
                m_own[nt] = m_new;
                if (__any_sync(0xffffffffu, corr != 1.f)) {  // the running maximum moved: rescale this lane's own columns
#pragma unroll
                    for (int mt = 0; mt < 8; mt++)
#pragma unroll
                        for (int i = 0; i < 4; i++) acc[nt][mt][i] *= corr;
                }
            }
            if (rg && il == warp) rg[11] = clock64() - loop0;
            // ---- p.V on the tensor cores: D[16 dims x 8 columns] += V^T[16 dims x 16 keys] . P[16 keys x 8 columns] per m tile;
            //      the weights as f16 hi / lo columns like the queries, the values transposed by ldmatrix ----
            uint32_t pf[NT][2];
            {
                const int col = lane >> 2, t4 = lane & 3, hl = col >> 1;
                const int src0 = ((2 * t4) << 2) | hl, src1 = ((2 * t4 + 1) << 2) | hl;  // lanes holding keys 2t, 2t+1 (and +8) of head hl
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    float x00 = __shfl_sync(0xffffffffu, pe[nt][0], src0), x01 = __shfl_sync(0xffffffffu, pe[nt][0], src1);
                    float x10 = __shfl_sync(0xffffffffu, pe[nt][1], src0), x11 = __shfl_sync(0xffffffffu, pe[nt][1], src1);
                    if (4 * nt + hl >= GSZ) { x00 = x01 = x10 = x11 = 0.f; }
                    __half h00 = __float2half_rn(x00), h01 = __float2half_rn(x01), h10 = __float2half_rn(x10), h11 = __float2half_rn(x11);
                    if (col & 1) {
                        h00 = __float2half_rn(x00 - __half2float(h00)); h01 = __float2half_rn(x01 - __half2float(h01));
                        h10 = __float2half_rn(x10 - __half2float(h10)); h11 = __float2half_rn(x11 - __half2float(h11));
                    }
                    const __half2 b0 = __halves2half2(h00, h01), b1 = __halves2half2(h10, h11);
                    pf[nt][0] = *reinterpret_cast<const uint32_t*>(&b0);
                    pf[nt][1] = *reinterpret_cast<const uint32_t*>(&b1);
                }
            }
            const int vkey = (lane & 7) + ((lane >> 4) & 1) * 8;  // the key row this lane addresses for the transposing ldmatrix
            const uint32_t lv_row = smem_u32(V_b) + (uint32_t)(vkey * 128);
#pragma unroll
            for (int mt = 0; mt < 8; mt++) {
                const int j = (mt & 3) * 2 + ((lane >> 3) & 1);  // dims chunk: tiles 0/2 take dims 0-7, tiles 1/3 dims 8-15 of the m tile
                uint32_t a0, a1, a2, a3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(lv_row + (mt >> 2) * kKHalf + ((j ^ (vkey & 7)) << 4)));
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(acc[nt][mt][0]), "+f"(acc[nt][mt][1]), "+f"(acc[nt][mt][2]), "+f"(acc[nt][mt][3])
                                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(pf[nt][0]), "r"(pf[nt][1]));
            }
        }
        __syncwarp();
        if (rg && il == warp) rg[12] = clock64() - loop0;
        if (rg && il == warp + kCWarps) rg[13] = clock64() - loop0;
        if (lane == 0 && il + S < n_items) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty[st])) : "memory");
    }
    if (cur_seg >= 0) flush(cur_seg);
    if (P.ring && tid == 0) atomicMax(P.ring + (size_t)P.ring_slot * 16 + 14, gtime());  // the last CTA whose warp 0 finished its items
    if (rg) { rg[2] = gtime(); rg[5] = ((unsigned long long)wait_cycles << 32) | (unsigned long long)(unsigned)(clock64() - loop0); }
    asm volatile("bar.sync 1, %0;" ::"r"(kCWarps * 32) : "memory");
    if (rg) rg[3] = gtime();

    // Two ways to add the CTAs' shares of a head, fixed per model (P.ticket_merge):
    //  * few CTAs per head (many kv heads): every CTA but the head's last publishes words that carry a valid flag and leaves;
    //    the last one polls them -- nobody pays a fence or an atomic;
    //  * many CTAs per head (one or a few kv heads per GPU, as in a model cut across GPUs): tickets, see below.
    if (!P.ticket_merge) {
        // ---- per (kv head, query head): the warps in warp order, then the CTAs that share the kv head in CTA order ----
        const int nseg = n_items > 0 ? (i_end - 1) / np - seg0 + 1 : 0;
        constexpr int kMergeGroups = kCWarps / 4;  // whole 128-thread groups among the consumers; the last warps sit the merge out
        const int hf = tid >> 7, dx = tid & 127;   // kMergeGroups (segment, query head) pairs at a time, one thread per dim
        for (int w = hf < kMergeGroups ? hf : nseg * GSZ; w < nseg * GSZ; w += kMergeGroups) {
            const int sl = w / GSZ, g = w - sl * GSZ;
            const float* ws = st_s + ((size_t)sl * kCWarps * GSZ + g) * kStateWords;  // warp 0's state; warp stride GSZ * kStateWords
            float M = -INFINITY;
    #pragma unroll
            for (int i = 0; i < kCWarps; i++) M = fmaxf(M, ws[(size_t)i * GSZ * kStateWords]);
            float L = 0.f, A = 0.f;
    #pragma unroll
            for (int i = 0; i < kCWarps; i++) {
                const float mi = ws[(size_t)i * GSZ * kStateWords];
                if (mi == -INFINITY) continue;  // the warp met no key of this head
                const float e = expf(mi - M);
                L += ws[(size_t)i * GSZ * kStateWords + 1] * e;
                A += ws[(size_t)i * GSZ * kStateWords + 4 + dx] * e;
            }
            const int seg = seg0 + sl, head = seg * GSZ + g;
            const long long first = (long long)seg * np, last = first + np - 1;
            const int c_first = (int)(((first + 1) * G - 1) / T), c_last = (int)(((last + 1) * G - 1) / T);
            const int nc = c_last - c_first + 1, me = (int)blockIdx.x - c_first;
            unsigned long long* sl_base = P.slots + (size_t)head * P.max_contrib * (2 + kHD);
            // validity tag of a slot word; the collector clears what it read
            const unsigned long long tag = 1ull;
            auto put = [&](unsigned long long* a, float v) {
                const unsigned long long wv = (tag << 32) | (unsigned long long)__float_as_uint(v);
                asm volatile("st.global.relaxed.gpu.u64 [%0], %1;" ::"l"(a), "l"(wv) : "memory");
            };
            if (nc > 1 && me != nc - 1) {
                unsigned long long* mine = sl_base + (size_t)me * (2 + kHD);
                if (dx == 0) { put(mine, M); put(mine + 1, L); }
                put(mine + 2 + dx, A);
            } else {
                // The head's LAST CTA collects the others and adds everything in CTA order.  CTAs are dispatched in index order
                // as SMs come free, so the highest index is the one most likely to have started last: when it gets here the
                // others' words are usually already in L2 and one round trip fetches them.  The three words of up to eight
                // contributors are requested together.
                constexpr int kBatch = 8;
                const float M_own = M, L_own = L, A_own = A;
                M = -INFINITY; L = 0.f; A = 0.f;
                for (int c0 = 0; c0 < nc - 1; c0 += kBatch) {
                    unsigned long long wv[kBatch][3];
                    bool all = false;
                    for (uint32_t it = 0; it < (1u << 20) && !all; ++it) {  // bounded: poll the whole batch until every word is valid
    #pragma unroll
                        for (int u = 0; u < kBatch; u++) {
                            const unsigned long long* theirs = sl_base + (size_t)min(c0 + u, nc - 2) * (2 + kHD);
                            asm volatile("ld.global.relaxed.gpu.u64 %0, [%1];" : "=l"(wv[u][0]) : "l"(theirs) : "memory");
                            asm volatile("ld.global.relaxed.gpu.u64 %0, [%1];" : "=l"(wv[u][1]) : "l"(theirs + 1) : "memory");
                            asm volatile("ld.global.relaxed.gpu.u64 %0, [%1];" : "=l"(wv[u][2]) : "l"(theirs + 2 + dx) : "memory");
                        }
                        all = true;
    #pragma unroll
                        for (int u = 0; u < kBatch; u++) all = all && (wv[u][0] >> 32) == tag && (wv[u][1] >> 32) == tag && (wv[u][2] >> 32) == tag;
                    }
                    ok = ok && all;
    #pragma unroll
                    for (int u = 0; u < kBatch; u++) {
                        if (c0 + u >= nc - 1) break;
                        const float Mc = __uint_as_float((uint32_t)wv[u][0]), Lc = __uint_as_float((uint32_t)wv[u][1]);
                        const float Ac = __uint_as_float((uint32_t)wv[u][2]);
                        const float Mn = fmaxf(M, Mc);
                        const float e0 = expf(M - Mn), e1 = expf(Mc - Mn);  // exp(-inf) = 0 for the empty start
                        A = A * e0 + Ac * e1;
                        L = L * e0 + Lc * e1;
                        M = Mn;
                    }
                }
                {   // this CTA's own share comes last
                    const float Mn = fmaxf(M, M_own);
                    const float e0 = expf(M - Mn), e1 = expf(M_own - Mn);
                    A = A * e0 + A_own * e1;
                    L = L * e0 + L_own * e1;
                    M = Mn;
                }
                if (nc > 1) {
                    for (int c = 0; c < nc - 1; c++)
                        asm volatile("st.global.relaxed.gpu.u64 [%0], %1;" ::"l"(sl_base + (size_t)c * (2 + kHD) + 2 + dx), "l"(0ull) : "memory");
                    asm volatile("bar.sync %0, 128;" ::"r"(2 + hf) : "memory");  // every thread of the pair has read the maxima and sums
                    if (dx < 2)
                        for (int c = 0; c < nc - 1; c++)
                            asm volatile("st.global.relaxed.gpu.u64 [%0], %1;" ::"l"(sl_base + (size_t)c * (2 + kHD) + dx), "l"(0ull) : "memory");
                }
                p.out[(size_t)head * kHD + dx] = A / L;
            }
        }
    } else {
        // ---- per kv head of the run: the warps in warp order; then, where several CTAs share the head, every CTA leaves its
        //      share in global memory and takes a ticket, and the CTA that takes the LAST ticket adds all shares in CTA order
        //      (so the result does not depend on who arrives last).  No polling: with one kv head per GPU (a cut model) a
        //      head spans dozens of CTAs, and a collector that polled them a few at a time paid one L2 round trip per batch. ----
        const int nseg = n_items > 0 ? (i_end - 1) / np - seg0 + 1 : 0;
        constexpr int kCThreads = kCWarps * 32;
        float* part = reinterpret_cast<float*>(P.slots);                                                   // [q head][contributor][2 + kHD]
        unsigned* tickets = reinterpret_cast<unsigned*>(P.slots) + (size_t)p.n_heads * P.max_contrib * (2 + kHD);  // [kv head], zero between launches
        for (int sl = 0; sl < nseg; sl++) {
            const int seg = seg0 + sl;
            const long long first = (long long)seg * np, last = first + np - 1;
            const int c_first = (int)(((first + 1) * G - 1) / T), c_last = (int)(((last + 1) * G - 1) / T);
            const int nc = c_last - c_first + 1, me = (int)blockIdx.x - c_first;
            for (int w = tid; w < GSZ * kHD; w += kCThreads) {
                const int g = w / kHD, dx = w - g * kHD;
                const float* ws = st_s + ((size_t)sl * kCWarps * GSZ + g) * kStateWords;  // warp 0's state; warp stride GSZ * kStateWords
                float M = -INFINITY;
    #pragma unroll
                for (int i = 0; i < kCWarps; i++) M = fmaxf(M, ws[(size_t)i * GSZ * kStateWords]);
                float L = 0.f, A = 0.f;
    #pragma unroll
                for (int i = 0; i < kCWarps; i++) {
                    const float mi = ws[(size_t)i * GSZ * kStateWords];
                    if (mi == -INFINITY) continue;  // the warp met no key of this head
                    const float e = expf(mi - M);
                    L += ws[(size_t)i * GSZ * kStateWords + 1] * e;
                    A += ws[(size_t)i * GSZ * kStateWords + 4 + dx] * e;
                }
                const int head = seg * GSZ + g;
                if (nc == 1) {
                    p.out[(size_t)head * kHD + dx] = A / L;
                } else {
                    float* mine = part + ((size_t)head * P.max_contrib + me) * (2 + kHD);
                    if (dx == 0) { mine[0] = M; mine[1] = L; }
                    mine[2 + dx] = A;
                }
            }
            if (nc > 1) {
                __threadfence();  // this CTA's share is in global memory before its ticket is
                asm volatile("bar.sync 1, %0;" ::"r"(kCThreads) : "memory");
                if (tid == 0) *s_last = atomicAdd(tickets + seg, 1u) == (unsigned)(nc - 1) ? 1 : 0;
                asm volatile("bar.sync 1, %0;" ::"r"(kCThreads) : "memory");
                if (*s_last) {
                    __threadfence();
                    // The shares' maxima and sums first, a warp per query head with its lanes over the contributors: the scale of
                    // every share and the scaled sums go to shared memory (the warps' states there are no longer needed), one
                    // lane adds the sums in CTA order.  Then every output reads its nc weighted values with independent loads.
                    // (With each thread walking maxima, sums and values of all contributors by itself the merge of 16 shares of
                    // eight heads took 14 us.)
                    float* esc = st_s;                              // [GSZ][nc]
                    float* lsc = esc + (size_t)GSZ * P.max_contrib;  // [GSZ][nc]
                    float* lsum = lsc + (size_t)GSZ * P.max_contrib; // [GSZ]
                    for (int i = tid; i < GSZ * nc; i += kCThreads) {  // every (head, share)'s maximum and sum: one round trip
                        const int g = i / nc, c = i - g * nc;
                        const float* q = part + ((size_t)(seg * GSZ + g) * P.max_contrib + c) * (2 + kHD);
                        esc[i] = __ldcg(q);
                        lsc[i] = __ldcg(q + 1);
                    }
                    asm volatile("bar.sync 1, %0;" ::"r"(kCThreads) : "memory");
                    for (int g = warp; g < GSZ; g += kCWarps) {
                        float M = -INFINITY;
                        for (int c = lane; c < nc; c += 32) M = fmaxf(M, esc[g * nc + c]);
                        M = warp_max(M);
                        for (int c = lane; c < nc; c += 32) {
                            const float e = expf(esc[g * nc + c] - M);  // exp(-inf) = 0 for a share without keys
                            esc[g * nc + c] = e;
                            lsc[g * nc + c] = lsc[g * nc + c] * e;
                        }
                        __syncwarp();
                        if (lane == 0) {
                            float L = 0.f;
                            for (int c = 0; c < nc; c++) L += lsc[g * nc + c];  // CTA order
                            lsum[g] = L;
                        }
                    }
                    asm volatile("bar.sync 1, %0;" ::"r"(kCThreads) : "memory");
                    {   // a thread's outputs together, eight shares at a time
                        constexpr int kOut = (GSZ * kHD + kCThreads - 1) / kCThreads;
                        constexpr int kB = 8;  // more in flight measured slower (16: 1.05 against 0.98 ms per 16 rank-layers of the 70B shape over 8 GPUs)
                        float A[kOut];
    #pragma unroll
                        for (int o = 0; o < kOut; o++) A[o] = 0.f;
                        for (int c0 = 0; c0 < nc; c0 += kB) {
                            float v[kOut][kB];
    #pragma unroll
                            for (int o = 0; o < kOut; o++) {
                                const int w = tid + o * kCThreads;
                                const int g = w / kHD, dx = w - g * kHD;
                                const float* base = part + (size_t)(seg * GSZ + g) * P.max_contrib * (2 + kHD) + 2 + dx;
    #pragma unroll
                                for (int u = 0; u < kB; u++)
                                    v[o][u] = (w < GSZ * kHD && c0 + u < nc) ? __ldcg(base + (size_t)(c0 + u) * (2 + kHD)) : 0.f;
                            }
    #pragma unroll
                            for (int o = 0; o < kOut; o++) {
                                const int w = tid + o * kCThreads;
                                const int g = w < GSZ * kHD ? w / kHD : 0;
    #pragma unroll
                                for (int u = 0; u < kB; u++)
                                    if (c0 + u < nc) A[o] += v[o][u] * esc[g * nc + c0 + u];  // CTA order
                            }
                        }
    #pragma unroll
                        for (int o = 0; o < kOut; o++) {
                            const int w = tid + o * kCThreads;
                            if (w < GSZ * kHD) {
                                const int g = w / kHD, dx = w - g * kHD;
                                p.out[(size_t)(seg * GSZ + g) * kHD + dx] = A[o] / lsum[g];
                            }
                        }
                    }

                    if (tid == 0) tickets[seg] = 0;  // every CTA of the head has taken its ticket: ready for the next launch
                }
                asm volatile("bar.sync 1, %0;" ::"r"(kCThreads) : "memory");
            }
        }
    }
    if (rg) rg[4] = gtime();
    if (P.ring && tid == 0) atomicMax(P.ring + (size_t)P.ring_slot * 16 + 6, gtime());
    if (!ok && lane == 0 && p.error_flag) atomicExch(p.error_flag, 1);
}

unsigned long long* g_aring = nullptr;
void dump_aring() {
    static unsigned long long h[256 * 16];
    if (!g_aring || cudaMemcpy(h, g_aring, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return;
    fprintf(stderr, "[attn ring] per launch slot (ns from CTA 0's start): last cta start | wait done, warp 0 items done, all warps done, cta0 end | last cta end\n");
    for (int i = 0; i < 256; i++) {
        const unsigned long long* r = h + (size_t)i * 16;
        if (!r[0]) continue;
        fprintf(stderr, "  %4d | %7lld | %7lld %7lld %7lld %7lld | %7lld | warp 0: %llu cycles waiting for data of %llu in its loop\n", i, (long long)(r[7] - r[0]),
                (long long)(r[1] - r[0]), (long long)(r[2] - r[0]), (long long)(r[3] - r[0]), (long long)(r[4] - r[0]), (long long)(r[6] - r[0]), r[5] >> 32,
                r[5] & 0xffffffffull);
        fprintf(stderr, "        warp 0 cycles from loop start: q %llu | item0: data %llu scores %llu softmax %llu pv %llu | item1 end %llu | last CTA's items done %lld ns\n", r[8], r[9], r[10], r[11], r[12], r[13], (long long)(r[14] - r[0]));
    }
}

int stream_max_contrib(int n_kv) { return sm_count() / n_kv + 3; }

template <int GSZ>
size_t stream_fixed_smem() {
    constexpr int kCWarps = consumer_warps<GSZ>();
    constexpr int NTc = (2 * GSZ + 7) / 8;
    return 1024 + (size_t)kMaxSeg * GSZ * kHD * 4 + (size_t)kMaxSeg * NTc * 16 * 32 * 4 + (size_t)kMaxSeg * kCWarps * GSZ * kStateWords * 4 +
           (size_t)kMaxSeg * GSZ * kStateWords * 4 + 32;
}

template <int GSZ>
int32_t launch_stream(const AttnParams& a, unsigned long long* slots, cudaStream_t s) {
    StreamParams P;
    P.a = a;
    P.max_contrib = stream_max_contrib(a.kv.n_kv);
    P.ticket_merge = P.max_contrib > 12 ? 1 : 0;  // by geometry only, so that a model never changes the slots' format
    // One kv head on this GPU (a cut model): a page costs a CTA about as much as a share costs the merge, so at most 32 CTAs share a head
    // (70B shape over 8 GPUs at 4096 keys, 16 rank-layers per step on one GPU: 1.32 ms without a limit, 1.25 / 1.24 ms with 16 / 32).
    static const int cap_env = getenv("LC_ATTN_HEAD_CAP") ? atoi(getenv("LC_ATTN_HEAD_CAP")) : 32;
    P.head_cap = cap_env;
    P.slots = slots;
    if (!g_aring && getenv("LC_ATTN_RING")) {  // diagnostics: wall-clock stamps per launch, printed at exit
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(s, &cs) == cudaSuccess && cs == cudaStreamCaptureStatusNone &&
            cudaMalloc(&g_aring, 256 * 16 * sizeof(unsigned long long)) == cudaSuccess) {
            cudaMemset(g_aring, 0, 256 * 16 * sizeof(unsigned long long));
            atexit(dump_aring);
        }
    }
    static int ring_seq = 0;
    P.ring = g_aring;
    P.ring_slot = ring_seq++ % 256;
    const size_t fixed = stream_fixed_smem<GSZ>();
    int stages = (int)((kMaxSmem - fixed) / (kStageBytes + 20));
    if (stages > 26) stages = 26;
    P.nstages = stages;
    const size_t smem = fixed + (size_t)stages * (kStageBytes + 20);
    auto kern = attention_stream_kernel<GSZ>;
    LC_CUDA(ensure_smem_limit((const void*)kern, kMaxSmem));
    CUtensorMap ktm, vtm;
    memcpy(&ktm, a.kv.k_tmap, sizeof(ktm));
    memcpy(&vtm, a.kv.v_tmap, sizeof(vtm));
    LC_CUDA(launch_pdl(kern, dim3(sm_count()), dim3((consumer_warps<GSZ>() + 1) * 32), smem, s, ktm, vtm, P));
    return LC_OK;
}

}  // namespace

size_t attention_stream_slot_bytes(int n_heads, int n_kv) {
    if (n_kv <= 0 || n_kv > sm_count() || n_heads % n_kv != 0) return 0;
    return (size_t)n_heads * stream_max_contrib(n_kv) * (2 + kHD) * sizeof(unsigned long long);
}

bool attention_stream_applies(const AttnParams& a, int n_tok) {
    const int gsz = a.kv.n_kv > 0 ? a.n_heads / a.kv.n_kv : 0;
    return a.kv.k_tmap != nullptr && a.kv.v_tmap != nullptr && n_tok == 1 && a.kv.hd == kHD && !a.kv.kv_f32 && a.kv.page_tokens == kPage && a.kv.n_kv <= sm_count() &&
           (gsz == 1 || gsz == 2 || gsz == 4 || gsz == 8);
}

int32_t launch_attention_stream(const AttnParams& a, unsigned long long* slots, cudaStream_t s) {
    switch (a.n_heads / a.kv.n_kv) {
        case 1: return launch_stream<1>(a, slots, s);
        case 2: return launch_stream<2>(a, slots, s);
        case 4: return launch_stream<4>(a, slots, s);
        default: return launch_stream<8>(a, slots, s);
    }
}

}  // namespace lc

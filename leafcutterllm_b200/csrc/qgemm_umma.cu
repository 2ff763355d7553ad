// Q4_K (and Q5_K: the kernel's UB = 176 form) weights times MANY tokens (prefill chunks, batched decode steps of five or more sequences) on the
// 5th-generation tensor cores: the dense contraction of the path (Tensor::matmul with m > 1, rust/src/tensor.rs:107-135,
// over weights that the reference dequantises per call, rust/src/model/loader.rs:213-224).
//
//   y[t, r] = sum_k x[t, k] * w[r, k],      w = d * sc * q - dmin * m       (rust/src/kernels/mod.rs:54-98)
//
// Weights stay as raw GGUF blocks in HBM; nothing dequantised is ever written back, and no weight is ever rounded: per
// 256-element unit and row the sum is regrouped as
//
//   d * sum_k (sc * q)[k] * x[t, k]  -  sum_sub (dmin * m[sub]) * sx[t, sub],       sx = sum of x over the 32-element sub-block
//
// where sc * q <= 63 * 15 is a small integer, exact in f16, and dmin * m (17 significant bits) is carried exactly by two
// f16.  Both sums run on the tensor cores with f32 accumulation; d is applied to the finished sum of each unit in f32.
// One CTA owns 128 weight rows (the M of tcgen05.mma) and up to 64 tokens, and walks k unit by unit:
//
//   producers  two threads: one requests the TMA boxes of raw blocks [144 B x 128 rows] per unit, the other per
//              64-element chunk of k the activation tile [64 x N] of f16 (128-byte rows, hardware swizzle 128B) as high
//              halves and, right behind them, low halves of the split below (one 3-D box), and per four units the tile
//              of sub-block sums;
//   unpack     two groups of 128 threads take the units in turn; thread r owns row r:
//              nibbles -> (1024 + q) as f16 by a byte permute, times sc minus 1024 sc in one HFMA2 (exact), written
//              with tcgen05.st straight into TENSOR MEMORY as the A operand (lane = row, one 32-bit column = two
//              consecutive k): 1.4 instructions per weight, and unpacked weights never cross shared memory;
//   multiply   one thread per group issues tcgen05.mma kind::f16, M=128, K=16, A from tensor memory, B from the swizzled tile.
//              Activations are x = hi + lo in f16 (2^-22 together); the high and the low tile lie one after the other,
//              so ONE instruction with N = 2 x tokens forms both products (two column ranges, added in the drain);
//              LC_GEMM_TERMS=1 keeps only the high halves (plain f16 activations, 2^-11);
//   drain      four warps of their own: when a unit's products are complete, thread r reads row r of the sums with
//              tcgen05.ld and adds d * sum into the row's f32 results, which live in its registers for the whole kernel;
//   epilogue   add the offset sums, undo the per-token power-of-two scale, then store / add the residual, or leave the
//              tile for the summing kernel (shares of k; SiLU(gate) * up).
//
// Activations are prepared by xprep_kernel: optional RMS norm (rust/src/backend/cpu.rs:49-60), a power-of-two scale per
// token that brings its largest magnitude into [0.5, 1) (so neither half leaves the f16 range), the hi/lo split, and
// the sub-block sums.  Every accumulator is written by one thread's products, in program order, and the drain adds the
// units in k order: results are deterministic.
//
// Every wait is bounded; a wait that runs out sets the library's device error flag and the CTA winds down (tensor
// memory freed, no copy left in flight).
#include <cstdio>
#include <cstdlib>
#include <cuda_fp16.h>
#include "lc_kernels.h"
#include "lc_quant.cuh"
#include "lc_tma.cuh"

namespace lc {

namespace {

constexpr int kRows = 128;     // weight rows per CTA = MMA M
constexpr int kMaxTok = 64;    // tokens per CTA (a multiple of 16)
constexpr int kMaxRaw = 4;     // raw unit boxes in flight
constexpr int kMaxB = 4;       // activation stages of two chunks each: two units in flight, and a stage always serves the same pipeline
constexpr int kUnpackGroups = 3;  // groups of four warps that take the units of k in turn
constexpr int kDrainGroups = 2;   // groups of four warps that each drain half of the tokens
constexpr int kThreads = 32 * (4 + 4 * kUnpackGroups + 4 * kDrainGroups);  // warps 0 and 3 producers, 1-2 the two issuers, then the unpack groups, then the drain
constexpr int kDRing = 8;      // units whose per-row d travel from the unpack threads to the drain at a time
constexpr int kUnitBytes = 144;  // Q4_K; a Q5_K unit has 176 (the kernel's UB)
// tensor-memory columns
constexpr uint32_t kColD = 0;            // accumulators of pipeline g at g * kColsPerPipe: [0, 2N) sum (sc q) x_hi | sum (sc q) x_lo of its unit in progress
constexpr uint32_t kColsPerPipe = 128;
constexpr uint32_t kColDmin = 256;       // [0, N): -sum dmin m sx of all units
constexpr uint32_t kColA = 320;          // four A stages of 32 columns: chunk c (64 k) of every unit goes through stage c
constexpr uint32_t kColAmin = 448;       // a stage of 8 columns per unpack group for the offset operand of the unit it works on

struct GemmParams {
    float* out;             // [T, n]
    const float* residual;  // or null
    const float* tok_scale; // [T] power of two that xprep divided token t by
    int n, k, T;
    int N;                  // tokens per CTA, padded to a multiple of 16: the box height of the activation tensor maps
    int epi;                // GemvEpilogue
    int terms;              // 3: activations as high + low halves; 1: high halves only
    int raw_stages, b_stages;
    int ksplit;             // CTAs along k per tile (gridDim.z)
    int tiles, nmat;        // row tiles per matrix; matrices (2 for EPI_SILU_MUL: blockIdx.x >= tiles works on the second)
    float* partial;         // [ksplit][nmat][T][n] f32 for the summing kernel, or null: the CTA holds the whole sum and writes `out`
    int* error_flag;
    unsigned* trace;        // diagnostics (LC_GEMM_TRACE): [7 roles][8] cycles that CTA (0, 0)'s threads spent in each kind of wait, or null
};

// ---- tcgen05 wrappers -------------------------------------------------------------------------------------------------
// Shared-memory operand descriptor, K-major, 128-byte swizzle: start address and the byte distance between 8-row groups
// in 16-byte units, descriptor version 1, layout code 2.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;                 // leading byte offset: unused with a swizzled K-major tile
    d |= (uint64_t)(1024u >> 4) << 32;      // stride byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// f32 accumulate, f16 x f16, both K-major, M = 128
__host__ __device__ constexpr uint32_t idesc_f16(int n_tok) {
    return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(n_tok >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
}
// D[tmem] (+)= A[tmem] * B[smem]^T
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- unpacking ---------------------------------------------------------------------------------------------------------
struct HdrQ4K { float d, dmin; uint32_t sc_lo, sc_hi, mn_lo, mn_hi; };
__device__ __forceinline__ void load_hdr(const unsigned char* rp, HdrQ4K& h) {
    const uint4 w = *reinterpret_cast<const uint4*>(rp);  // d, dmin, 12 scale bytes (mod.rs:66-75)
    h.d = h2f((uint16_t)(w.x & 0xFFFFu));
    h.dmin = h2f((uint16_t)(w.x >> 16));
    unpack_scales_k4(w.y, w.z, w.w, &h.sc_lo, &h.sc_hi, &h.mn_lo, &h.mn_hi);
}
// bytes b0, b1 (or b2, b3) of v, each < 64, as the f16 pair (1024 + b0, 1024 + b1): 0x64 is the high byte of 1024.0
__device__ __forceinline__ uint32_t bias_pair(uint32_t v, int upper) { return __byte_perm(v, 0x64646464u, upper ? 0x5342u : 0x5140u); }
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t h2_pair(float v) {  // (v, v) as f16x2; v is a small integer
    const __half2 h = __float2half2_rn(v);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// Chunk c of a unit = group c of mod.rs:77-96: 32 bytes whose low nibbles are elements 0..31 under sc[2c] and whose high
// nibbles are elements 32..63 under sc[2c + 1].  Column j of `col` holds (sc q) of elements 2j, 2j + 1, exact in f16:
// (1024 + q) * sc - 1024 * sc is one fused multiply-add whose exact result, at most 945, needs no rounding.
// UB = 176: a Q5_K unit (mod.rs:101-143) -- the same header, then 32 bytes whose bit s is the fifth bit of element l of
// sub-block s, then the nibbles: q < 32, (sc q) at most 1953, still exact.
template <int UB>
__device__ __forceinline__ void unpack_chunk(const unsigned char* rp, const HdrQ4K& h, int c, uint32_t (&col)[32]) {
    const uint32_t scw = c < 2 ? h.sc_lo : h.sc_hi;
    const int sh = (c & 1) * 16;
    const float fa = (float)((scw >> sh) & 0xFFu), fb = (float)((scw >> (sh + 8)) & 0xFFu);
    const uint32_t sa = h2_pair(fa), sb = h2_pair(fb), ka = h2_pair(-1024.0f * fa), kb = h2_pair(-1024.0f * fb);
    const uint4* q = reinterpret_cast<const uint4*>(rp + (UB == 176 ? 48 : 16) + 32 * c);
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const uint4 v = q[half];
        const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
        uint32_t hb[4] = {0u, 0u, 0u, 0u};
        if constexpr (UB == 176) {
            const uint4 hq = *reinterpret_cast<const uint4*>(rp + 16 + 16 * half);
            hb[0] = hq.x; hb[1] = hq.y; hb[2] = hq.z; hb[3] = hq.w;
        }
#pragma unroll
        for (int wi = 0; wi < 4; wi++) {
            uint32_t lo4 = vv[wi] & 0x0F0F0F0Fu, hi4 = (vv[wi] >> 4) & 0x0F0F0F0Fu;
            if constexpr (UB == 176) {
                lo4 |= ((hb[wi] >> (2 * c)) & 0x01010101u) << 4;
                hi4 |= ((hb[wi] >> (2 * c + 1)) & 0x01010101u) << 4;
            }
            const int j = half * 8 + wi * 2;
            col[j] = h2_fma(bias_pair(lo4, 0), sa, ka);
            col[j + 1] = h2_fma(bias_pair(lo4, 1), sa, ka);
            col[16 + j] = h2_fma(bias_pair(hi4, 0), sb, kb);
            col[16 + j + 1] = h2_fma(bias_pair(hi4, 1), sb, kb);
        }
    }
}
// The offset operand of a unit: p[i] = -dmin * m[i] has at most 17 significant bits, so hi = f16(p) and lo = f16(p - hi)
// carry it exactly (lo is a multiple of 2^-24 for any f16 dmin).  Columns 0-3: the eight hi as pairs (k' = 0..7), columns
// 4-7: the eight lo (k' = 8..15); the sums tile holds each sub-block sum at k' and k' + 8.
__device__ __forceinline__ void unpack_mins(const HdrQ4K& h, uint32_t (&col)[8]) {
    __half hi[8], lo[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float m = (float)(((i < 4 ? h.mn_lo : h.mn_hi) >> (8 * (i & 3))) & 0xFFu);
        const float pr = -h.dmin * m;
        hi[i] = __float2half_rn(pr);
        lo[i] = __float2half_rn(pr - __half2float(hi[i]));
    }
#pragma unroll
    for (int j2 = 0; j2 < 4; j2++) {
        const __half2 a = __halves2half2(hi[2 * j2], hi[2 * j2 + 1]), b = __halves2half2(lo[2 * j2], lo[2 * j2 + 1]);
        col[j2] = *reinterpret_cast<const uint32_t*>(&a);
        col[4 + j2] = *reinterpret_cast<const uint32_t*>(&b);
    }
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                 "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

}  // namespace

// One token per CTA: optional RMS norm, power-of-two scale, hi/lo split to f16, sub-block sums.
// xh: [hi rows | lo rows at lo_offset] of K f16; sx: the same for the sums, rows of K/16 f16 -- per 256-element unit the
// eight sub-block sums, twice.
// The preparation of a token's row held in shared memory.  `acc` = this thread's part of the sum of squares, accumulated
// over elements 4 * tid + 4 * blockDim * j in that order; `amax` = this thread's largest |x g| (|x| without a norm).  One
// block-wide reduction gives both the RMS scale and the row's largest magnitude (scale * max |x g|: it only picks the
// power of two that brings the row below 1, so its last-bit difference from max |(x scale) g| does not matter).
__device__ __forceinline__ void xprep_row(float* row, float acc, float amax, const float* __restrict__ norm_w, float eps, int K, int t,
                                          __half* __restrict__ xh, size_t lo_offset, __half* __restrict__ sx, size_t sx_lo_offset,
                                          float* __restrict__ tok_scale, float* sh) {
    float scale = 1.f;
    float mx;
    {   // sh: [0, 32) the warps' sums, [32, 64) their maxima
        const float ws = warp_sum(acc), wm = warp_max(amax);
        const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
        if (lane == 0) { sh[w] = ws; sh[32 + w] = wm; }
        __syncthreads();  // also: the whole row is in shared memory
        float r = (threadIdx.x < nw) ? sh[threadIdx.x] : 0.0f, rm = (threadIdx.x < nw) ? sh[32 + threadIdx.x] : 0.0f;
        if (w == 0) { r = warp_sum(r); rm = warp_max(rm); }
        __syncthreads();
        if (threadIdx.x == 0) { sh[0] = r; sh[32] = rm; }
        __syncthreads();
        if (norm_w) scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sh[0], (float)K), eps)));  // cpu.rs:52-55
        mx = sh[32] * scale;
    }
    int e = 0;
    if (mx > 0.f && mx < INFINITY) (void)frexpf(mx, &e);  // mx = f * 2^e, f in [0.5, 1)
    const float down = ldexpf(1.0f, -e);
    if (threadIdx.x == 0) tok_scale[t] = ldexpf(1.0f, e);
    __half* hi = xh + (size_t)t * K;
    __half* lo = hi + lo_offset;
    __half* sxh = sx + (size_t)t * (K / 16);
    __half* sxl = sxh + sx_lo_offset;
    // K is a multiple of 256 and a thread takes 4 consecutive elements: eight neighbouring lanes cover one sub-block,
    // and inactive lanes of the last round belong to whole sub-blocks that do not exist
    for (int i0 = 0; i0 < K; i0 += blockDim.x * 4) {
        const int i = i0 + threadIdx.x * 4;
        float part = 0.f;
        if (i < K) {
            float4 v = *reinterpret_cast<float4*>(row + i);
            if (norm_w) {
                const float4 g = *reinterpret_cast<const float4*>(norm_w + i);
                v.x = __fmul_rn(__fmul_rn(v.x, scale), g.x); v.y = __fmul_rn(__fmul_rn(v.y, scale), g.y);
                v.z = __fmul_rn(__fmul_rn(v.z, scale), g.z); v.w = __fmul_rn(__fmul_rn(v.w, scale), g.w);
            }
            const float a = v.x * down, b = v.y * down, c = v.z * down, d = v.w * down;
            const __half2 h0 = __floats2half2_rn(a, b), h1 = __floats2half2_rn(c, d);
            const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
            const __half2 l0 = __floats2half2_rn(a - f0.x, b - f0.y), l1 = __floats2half2_rn(c - f1.x, d - f1.y);
            uint2 ph, pl;
            ph.x = *reinterpret_cast<const uint32_t*>(&h0); ph.y = *reinterpret_cast<const uint32_t*>(&h1);
            pl.x = *reinterpret_cast<const uint32_t*>(&l0); pl.y = *reinterpret_cast<const uint32_t*>(&l1);
            *reinterpret_cast<uint2*>(hi + i) = ph;
            *reinterpret_cast<uint2*>(lo + i) = pl;
            // the sum of what the product will see: the two halves of every element
            const float2 g0 = __half22float2(l0), g1 = __half22float2(l1);
            part = ((f0.x + g0.x) + (f0.y + g0.y)) + ((f1.x + g1.x) + (f1.y + g1.y));
        }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        part += __shfl_xor_sync(0xffffffffu, part, 4);
        if (i < K && (threadIdx.x & 7) == 0) {
            const int sub = i >> 5, unit = sub >> 3, idx = unit * 16 + (sub & 7);
            const __half sh_ = __float2half_rn(part), sl_ = __float2half_rn(part - __half2float(sh_));
            sxh[idx] = sh_;
            sxl[idx] = sl_;
            sxh[idx + 8] = sh_;  // a second time: the offset operand pairs each sum with the high and with the low part of -dmin * m
            sxl[idx + 8] = sl_;
        }
    }
}

__global__ void __launch_bounds__(1024)
xprep_kernel(const float* __restrict__ x, const float* __restrict__ norm_w, float eps, int K, __half* __restrict__ xh,
             size_t lo_offset, __half* __restrict__ sx, size_t sx_lo_offset, float* __restrict__ tok_scale) {
    extern __shared__ float row[];
    __shared__ float sh[64];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const float* xr = x + (size_t)t * K;
    float acc = 0.f, amax = 0.f;
    for (int i = threadIdx.x * 4; i < K; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i);
        *reinterpret_cast<float4*>(row + i) = v;
        acc = fmaf(v.x, v.x, acc); acc = fmaf(v.y, v.y, acc); acc = fmaf(v.z, v.z, acc); acc = fmaf(v.w, v.w, acc);
        float4 g = make_float4(1.f, 1.f, 1.f, 1.f);
        if (norm_w) g = *reinterpret_cast<const float4*>(norm_w + i);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x * g.x), fabsf(v.y * g.y)), fmaxf(fabsf(v.z * g.z), fabsf(v.w * g.w))));  // NaN does not raise the maximum
    }
    xprep_row(row, acc, amax, norm_w, eps, K, t, xh, lo_offset, sx, sx_lo_offset, tok_scale, sh);
}

// grid = (row tiles x matrices, token tiles, shares of k).  tmw0 / tmw1: raw blocks of the matrix (and of `up` for
// EPI_SILU_MUL: CTAs past the first matrix's tiles work on the second), box = one unit x 128 rows.  tmx: the prepared
// activations [2 halves][t_cap rows][k] f16 seen in four dimensions (element, row, half, 64-element chunk), box = 64 elements
// x N rows x both halves x two chunks, 128-byte swizzle; tms: the sub-block sums [2][t_cap rows][k / 16], box = 64 x N x both halves.
//
// Roles (24 warps): warp 0 requests the activation tiles, warp 3 the raw boxes.  The units of k are multiplied by two
// pipelines in turn (unit s by pipeline s & 1: the issuing thread of warp 1 + (s & 1) and its own accumulators in tensor
// memory): one thread issues a tcgen05.mma of this shape every ~70 cycles at best, two together reach the tensor pipe's
// rate (~62 cycles per M128 N128 K16; lc_tcgen05_probe measures both).  They are unpacked by THREE groups of four warps in
// turn (unit s by group s % 3: unpacking a unit takes a group about as long as three units take the pipelines); chunk c
// of every unit goes through tensor-memory stage c, so a group works a whole unit ahead of the products.  Two groups of
// four warps only drain, half of the tokens each: thread r owns row r's f32 results of its tokens for the whole kernel,
// reads a finished unit's sums with tcgen05.ld while both pipelines already work on the next units, and writes the tile at
// the end.  The unpack threads never wait for a product, the drain never unpacks.
//
// The offset term -dmin * m needs no drain per unit: dmin * m (11 x 6 bits) is split exactly into two f16 (high part and
// remainder), the sixteen values of a unit form one K = 16 operand against the sub-block sums stored twice, and the
// products of all units accumulate in ONE set of columns, read once at the end; the two issuers take turns on it (each
// waits for the completion of the other's unit before), so the additions happen in k order.
template <int UB>
__global__ void __launch_bounds__(kThreads, 1)
qgemm_umma_q4k_kernel(const __grid_constant__ CUtensorMap tmw0, const __grid_constant__ CUtensorMap tmw1,
                      const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tms, GemmParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int mat = (int)blockIdx.x >= p.tiles ? 1 : 0, tile = (int)blockIdx.x - mat * p.tiles, tok0 = blockIdx.y * kMaxTok;
    const int N = p.N;
    // this CTA's share of k: whole groups of four units (one tile of sub-block sums), so that only its last tile can be short
    const int nquads = (p.k / kUnitElems + 3) / 4;
    const int u_begin = (int)((long long)blockIdx.z * nquads / p.ksplit) * 4;
    const int u_end = min((int)((long long)(blockIdx.z + 1) * nquads / p.ksplit) * 4, p.k / kUnitElems);
    const int nseq = u_end - u_begin;  // units are numbered from u_begin below; unit s belongs to pipeline s & 1
    const int RS = p.raw_stages;
    constexpr int BS = kMaxB;
    const bool two = p.terms == 3;
    constexpr uint32_t raw_bytes = UB * kRows;
    const uint32_t b_half = (uint32_t)N * 128u, b_bytes = 2u * b_half;

    unsigned char* bt = smem;                              // [BS][2 chunks][hi N x 128 B | lo N x 128 B], 1024-byte aligned
    unsigned char* st = bt + (size_t)BS * 2 * b_bytes;     // [2][the same for the sub-block sums of four units]
    unsigned char* raw = st + (size_t)2 * b_bytes;         // [RS][raw_bytes]
    float* dd = reinterpret_cast<float*>(raw + (size_t)RS * raw_bytes);  // [kDRing][128]: d of row r in unit s, unpack -> drain
    uint64_t* bars = reinterpret_cast<uint64_t*>(dd + kDRing * kRows);
    uint64_t* raw_full = bars;                 // [kMaxRaw] producer -> unpack (transaction bytes)
    uint64_t* raw_empty = raw_full + kMaxRaw;  // [kMaxRaw] unpack -> producer (128 arrivals)
    uint64_t* b_full = raw_empty + kMaxRaw;    // [kMaxB]   producer -> multiply
    uint64_t* b_empty = b_full + kMaxB;        // [kMaxB]   multiply (commit) -> producer
    uint64_t* s_full = b_empty + kMaxB;        // [2]       sub-block sums of four units: producer -> multiply
    uint64_t* s_empty = s_full + 2;            // [2]       multiply (the commit behind the last offset product that used them) -> producer
    // A barrier's waiter must see every phase of it: where two issuers or three unpack groups take turns, every (waiter, resource)
    // pair has a barrier of its own, so nobody ever waits for a phase two or more ahead of the last one it saw.
    uint64_t* a_full = s_empty + 2;            // [2][4]    stage c holds a chunk of a unit of pipeline g (128 arrivals) -> issuer g
    uint64_t* a_empty = a_full + 8;            // [groups][4] the products of stage c are complete (commit): the barrier of the group that fills it next
    uint64_t* am_full = a_empty + 4 * kUnpackGroups;  // [groups] the offset operand of the group's unit (128 arrivals); one stage per group
    uint64_t* am_empty = am_full + kUnpackGroups;     // [groups] its product is complete (commit)
    uint64_t* d_full = am_empty + kUnpackGroups;           // [2]       all products of a unit of pipeline g are complete (commit): the drain may read its sums,
                                               //           and the other issuer may add the next unit's offset product
    uint64_t* d_empty = d_full + 2;            // [2]       the drain has read them (128 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + 2);
    uint32_t* raw_issued = tmem_slot + 1;      // units whose raw box has been requested (a stage serves both groups in turn: see below)

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < kMaxRaw; i++) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], 128); }
        for (int i = 0; i < kMaxB; i++) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
        for (int i = 0; i < 2; i++) {
            mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 1); mbar_init(&d_full[i], 1); mbar_init(&d_empty[i], 128 * kDrainGroups);
        }
        for (int i = 0; i < kUnpackGroups; i++) { mbar_init(&am_full[i], 128); mbar_init(&am_empty[i], 1); }
        for (int i = 0; i < 8; i++) mbar_init(&a_full[i], 128);
        for (int i = 0; i < 4 * kUnpackGroups; i++) mbar_init(&a_empty[i], 1);
        *raw_issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // The kernel behind this one may be scheduled as soon as every CTA of this one runs: its CTAs take the SMs as ours leave
    // (or the idle ones at once), do their own set-up and wait for this grid's completion before they read anything.  With
    // the call behind the main loop the 64-sequence step was 0.06 ms per layer slower (the attention grid started late).
    bool ok = true;
    // diagnostics: cycles spent in each kind of wait (slot), and in the role's whole loop (slot 7)
    const bool tracing = p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    unsigned wacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const unsigned t_role0 = (unsigned)clock64();
    auto twait = [&](uint64_t* bar, uint32_t parity, int slot) -> bool {
        if (!tracing) return mbar_wait(bar, parity);
        const unsigned t0 = (unsigned)clock64();
        const bool r = mbar_wait(bar, parity);
        wacc[slot] += (unsigned)clock64() - t0;
        return r;
    };
    auto trace_out = [&](int role) {
        if (!tracing) return;
        wacc[7] = (unsigned)clock64() - t_role0;
        for (int i = 0; i < 8; i++) p.trace[role * 8 + i] = wacc[i];
    };
    // a wait whose outcome the whole warp shares: the tensor-memory instructions are warp-wide.  (One polling lane per warp
    // with a shuffle behind it, and one arrival per warp, measured slower: 44.0 vs 38.6 us at 64 tokens x 4096 x 12288.)
    auto wait_all = [&](uint64_t* bar, uint32_t parity, int slot) { return __all_sync(0xffffffffu, twait(bar, parity, slot)); };

    if (warp == 0) {
        // ---------------------------------------------------------------- producer of the activations
        // activation chunks in k order (and, with the first chunk of every four units, their sub-block sums): one
        // 3-D box brings the high and the low halves of a chunk
        if (lane == 0) {
            pdl_wait();
            const int b_total = nseq * 2;  // pairs of chunks
            for (int b_next = 0; b_next < b_total && ok; b_next++) {
                const int sb = b_next & (kMaxB - 1);
                if (!twait(&b_empty[sb], ((b_next / kMaxB) & 1) ^ 1, 0)) { ok = false; break; }
                if ((b_next & 7) == 0) {
                    const int q = b_next >> 3, ss = q & 1;
                    if (!twait(&s_empty[ss], ((q >> 1) & 1) ^ 1, 1)) { ok = false; break; }
                    mbar_expect_tx(&s_full[ss], b_bytes);
                    tma_load_3d(st + (size_t)ss * b_bytes, &tms, (u_begin / 4 + q) * 64, tok0, 0, &s_full[ss]);
                }
                mbar_expect_tx(&b_full[sb], 2 * b_bytes);
                tma_load_4d(bt + (size_t)sb * 2 * b_bytes, &tmx, 0, tok0, 0, u_begin * 4 + b_next * 2, &b_full[sb]);
            }
            trace_out(0);
        }
    } else if (warp == 3) {
        // ---------------------------------------------------------------- producer of the raw boxes, unit order
        // a thread of its own: the weights do not depend on the kernel ahead of this one, so this stream starts
        // before the wait for it
        if (lane == 0) {
            for (int s = 0; s < nseq && ok; s++) {
                const int sr = s % RS;
                if (!twait(&raw_empty[sr], ((s / RS) & 1) ^ 1, 0)) { ok = false; break; }
                mbar_expect_tx(&raw_full[sr], raw_bytes);
                tma_load_2d(raw + (size_t)sr * raw_bytes, mat ? &tmw1 : &tmw0, (u_begin + s) * (UB / 4), tile * kRows, &raw_full[sr]);
                // with an odd number of stages a stage serves the two unpack groups in turn, and a group that waited for unit
                // s before unit s - RS had landed would read that phase's parity as its own: it first waits for this count
                asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(raw_issued)), "r"((uint32_t)(s + 1)) : "memory");
            }
            trace_out(1);
        }
    } else if (warp == 1 || warp == 2) {
        // ---------------------------------------------------------------- multiply: the issuer of pipeline g
        pdl_wait();
        const int g = warp - 1;
        if (lane == 0) {
            const uint32_t idesc_main = idesc_f16(two ? 2 * N : N), idesc_min = idesc_f16(N);
            const uint32_t d_main = tmem + kColD + g * kColsPerPipe, d_min = tmem + kColDmin;
            int j = 0;
            for (int s = g; s < nseq && ok; s += 2, j++) {
                // the accumulators still hold the previous unit of this pipeline until the drain has read them
                if (j > 0 && !twait(&d_empty[g], (j - 1) & 1, 0)) { ok = false; break; }
                tc_fence_after();
                for (int c = 0; c < 4 && ok; c++) {
                    const int b_it = s * 2 + (c >> 1), sb = b_it & (kMaxB - 1);  // the pair of chunks and its stage
                    if (!(c & 1) && !twait(&b_full[sb], (b_it / kMaxB) & 1, 1)) { ok = false; break; }
                    if (!twait(&a_full[g * 4 + c], j & 1, 2)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t bdesc = umma_desc_sw128(smem_u32(bt + (size_t)(sb * 2 + (c & 1)) * b_bytes));
                    const uint32_t a_t = tmem + kColA + c * 32;
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        umma_f16_ts(d_main, a_t + ks * 8, bdesc + (uint64_t)(ks * 2), idesc_main, (uint32_t)((c | ks) != 0));
                    umma_commit(&a_empty[((s + 1) % kUnpackGroups) * 4 + c]);  // the group of the unit behind this one fills the stage next
                    if (c & 1) umma_commit(&b_empty[sb]);
                }
                if (!ok) break;
                {   // the offset term: A = the unit's sixteen halves of -dmin * m, B = this unit's 16 columns of the sums tile.
                    // One set of columns accumulates all units; the two issuers take turns, each waiting for the other's
                    // product of the unit before, so the additions happen in k order.
                    const int q = s >> 2, ss = q & 1, am = s % kUnpackGroups;
                    if (!twait(&s_full[ss], (q >> 1) & 1, 3)) { ok = false; break; }
                    // first the other issuer's unit: with it every earlier unit is complete, so the operand barrier below (which
                    // the two issuers see in turn) is in this unit's phase
                    if (s > 0 && !twait(&d_full[1 - g], ((s - 1) >> 1) & 1, 5)) { ok = false; break; }
                    if (!twait(&am_full[am], (s / kUnpackGroups) & 1, 4)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t sdesc = umma_desc_sw128(smem_u32(st + (size_t)ss * b_bytes)) + (uint64_t)((s & 3) * 2);
                    umma_f16_ts(d_min, tmem + kColAmin + am * 8, sdesc, idesc_min, (uint32_t)(s > 0));
                    if (two) umma_f16_ts(d_min, tmem + kColAmin + am * 8, sdesc + (uint64_t)(b_half >> 4), idesc_min, 1u);
                    umma_commit(&am_empty[am]);
                    if ((s & 3) == 3) umma_commit(&s_empty[ss]);  // the offset products are ordered: this one is the last on the tile
                }
                umma_commit(&d_full[g]);
            }
            trace_out(2 + g);
        }
    } else if (warp < 4 + 4 * kUnpackGroups) {
        // ---------------------------------------------------------------- unpack: group ug takes units ug, ug + kUnpackGroups, ...
        const int ug = (warp - 4) >> 2;
        const int quarter = warp & 3;                 // the tensor-memory lanes this warp may touch
        const int row = quarter * 32 + lane;          // row of the tile owned by this thread
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const bool tr = quarter == 0 && lane == 0;
        for (int s = ug; s < nseq && ok; s += kUnpackGroups) {
            const int g = s & 1;  // the unit's pipeline
            const int sr = s % RS;
            {   // the request for this unit's box has been made (see the producer)
                const unsigned t0 = (unsigned)clock64();
                uint32_t seen = 0;
                for (uint32_t it = 0; it < (1u << 24) && seen <= (uint32_t)s; ++it)
                    asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(seen) : "r"(smem_u32(raw_issued)) : "memory");
                ok = __all_sync(0xffffffffu, seen > (uint32_t)s);
                wacc[0] += (unsigned)clock64() - t0;
                if (!ok) break;
            }
            ok = wait_all(&raw_full[sr], (s / RS) & 1, 1);
            if (!ok) break;
            const unsigned char* rp = raw + (size_t)sr * raw_bytes + (size_t)row * UB;
            HdrQ4K hdr;
            load_hdr(rp, hdr);
            // the ring is deep enough: unit s + kDRing cannot be unpacked before unit s has been drained (its chunks need the
            // tensor-memory stages of unit s + kDRing - 1, ..., whose products wait for the accumulators that the drain releases)
            dd[(s & (kDRing - 1)) * kRows + row] = hdr.d;
            {   // the offset operand of this pipeline first (the header is all it needs): free once the product of the pipeline's
                // unit before has read it, which ended long ago
                uint32_t mc[8];
                unpack_mins(hdr, mc);
                ok = wait_all(&am_empty[ug], ((s / kUnpackGroups) & 1) ^ 1, 2);
                if (!ok) break;
                tc_fence_after();
                tmem_st8(tmem + lane_base + kColAmin + ug * 8, mc);
            }
            for (int c = 0; c < 4 && ok; c++) {
                // stage c still holds the unit before this one (the other group's) until that unit's products have read it; ask
                // now, look at the answer after the unpacking
                const uint32_t par = (uint32_t)(((s - 1) / kUnpackGroups) & 1);  // this group's barrier: one commit per unit it fills after the first
                bool free_now = s == 0 || mbar_test(&a_empty[ug * 4 + c], par);
                uint32_t col[32];
                unsigned tq0 = 0;
                if (tracing) tq0 = (unsigned)clock64();
                unpack_chunk<UB>(rp, hdr, c, col);
                if (tracing) { const unsigned t1 = (unsigned)clock64(); wacc[4] += t1 - tq0; tq0 = t1; }
                // the chunk before this one (the offset operand ahead of the first) has had the time of this unpacking to reach
                // tensor memory
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                if (tracing) { const unsigned t1 = (unsigned)clock64(); wacc[5] += t1 - tq0; tq0 = t1; }
                tc_fence_before();
                mbar_arrive(c > 0 ? &a_full[g * 4 + c - 1] : &am_full[ug]);
                if (tracing) { const unsigned t1 = (unsigned)clock64(); wacc[6] += t1 - tq0; tq0 = t1; }
                if (!free_now) free_now = mbar_wait(&a_empty[ug * 4 + c], par);
                ok = __all_sync(0xffffffffu, free_now);
                if (!ok) break;
                tc_fence_after();
                if (tracing) { const unsigned t1 = (unsigned)clock64(); wacc[3] += t1 - tq0; tq0 = t1; }
                const uint32_t a_t = tmem + lane_base + kColA + c * 32;
                tmem_st16(a_t, col);
                tmem_st16(a_t + 16, col + 16);
            }
            if (!ok) break;
            mbar_arrive(&raw_empty[sr]);  // this row's bytes of the unit are consumed
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            mbar_arrive(&a_full[g * 4 + 3]);
        }
        if (tr && ug < 2) trace_out(4 + ug);
    } else {
        // ---------------------------------------------------------------- drain, then epilogue
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        constexpr int kTokD = kMaxTok / kDrainGroups;                     // tokens per drain group
        const int tbase = ((warp - 4 - 4 * kUnpackGroups) >> 2) * kTokD;  // this group's first token of the tile
        float y[kTokD];
#pragma unroll
        for (int t = 0; t < kTokD; t++) y[t] = 0.f;
        pdl_wait();
        for (int s = 0; s < nseq && ok; s++) {
            const int g = s & 1, j = s >> 1;
            const uint32_t d_main = tmem + lane_base + kColD + g * kColsPerPipe;
            ok = wait_all(&d_full[g], j & 1, 0);
            if (!ok) break;
            tc_fence_after();
            const float d = dd[(s & (kDRing - 1)) * kRows + row];
#pragma unroll
            for (int t0 = 0; t0 < kTokD; t0 += 16) {
                if (tbase + t0 < N) {
                    uint32_t a[16], b[16];
                    tmem_ld16(d_main + tbase + t0, a);
                    if (two) tmem_ld16(d_main + N + tbase + t0, b);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        float v = __uint_as_float(a[i]);
                        if (two) v += __uint_as_float(b[i]);
                        y[t0 + i] = fmaf(d, v, y[t0 + i]);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&d_empty[g]);
        }
        if (quarter == 0 && lane == 0 && tbase == 0) trace_out(6);
        // the offset sums (complete: every unit's d_full followed its offset product)
        if (ok && nseq > 0) {
            const uint32_t d_min = tmem + lane_base + kColDmin;
#pragma unroll
            for (int t0 = 0; t0 < kTokD; t0 += 16) {
                if (tbase + t0 < N) {
                    uint32_t m[16];
                    tmem_ld16(d_min + tbase + t0, m);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; i++) y[t0 + i] += __uint_as_float(m[i]);
                }
            }
        }
        const int grow = tile * kRows + row;
        if (ok && grow < p.n) {
            if (p.partial) {
                // a share of k, or one of the two matrices of gate/up: the sums (scaled back per token) go to the summing kernel
                float* dst = p.partial + ((size_t)(blockIdx.z * p.nmat + mat) * p.T) * p.n;
#pragma unroll
                for (int t = 0; t < kTokD; t++) {
                    const int tok = tok0 + tbase + t;
                    if (tbase + t < N && tok < p.T) dst[(size_t)tok * p.n + grow] = y[t] * __ldg(p.tok_scale + tok);
                }
            } else {
#pragma unroll
                for (int t = 0; t < kTokD; t++) {
                    const int tok = tok0 + tbase + t;
                    if (tbase + t < N && tok < p.T) {
                        const size_t o = (size_t)tok * p.n + grow;
                        float v = y[t] * __ldg(p.tok_scale + tok);
                        if (p.epi == EPI_ADD_RESIDUAL) v = __fadd_rn(p.residual[o], v);
                        p.out[o] = v;
                    }
                }
            }
        }
    }
    if (!ok && p.error_flag) atomicExch(p.error_flag, 3);
    tc_fence_before();
    __syncthreads();
    pdl_launch_dependents();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

// Sums what the product kernel left in `partial` ([slices][T][n], slice = share of k * matrices + matrix), in slice
// order, and applies the epilogue.  With two matrices even slices belong to gate and odd ones to up.
__global__ void __launch_bounds__(256)
qgemm_reduce_kernel(const float* __restrict__ partial, int slices, size_t plane, int epi, const float* __restrict__ residual,
                    float* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= plane) return;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    for (int sl = 0; sl < slices; sl++) {
        const float4 v = *reinterpret_cast<const float4*>(partial + (size_t)sl * plane + i);
        float4& d = (epi == EPI_SILU_MUL && (sl & 1)) ? b : a;
        d.x += v.x; d.y += v.y; d.z += v.z; d.w += v.w;
    }
    if (epi == EPI_SILU_MUL) {
        a.x = __fmul_rn(silu_f(a.x), b.x); a.y = __fmul_rn(silu_f(a.y), b.y);
        a.z = __fmul_rn(silu_f(a.z), b.z); a.w = __fmul_rn(silu_f(a.w), b.w);
    } else if (epi == EPI_ADD_RESIDUAL) {
        const float4 r = *reinterpret_cast<const float4*>(residual + i);
        a.x = __fadd_rn(r.x, a.x); a.y = __fadd_rn(r.y, a.y); a.z = __fadd_rn(r.z, a.z); a.w = __fadd_rn(r.w, a.w);
    }
    *reinterpret_cast<float4*>(out + i) = a;
}

// qgemm_reduce_kernel for one token per CTA, followed by the preparation of that token's finished row as the input of the
// next product (xprep_kernel's passes on the row while it is still in shared memory).  Same sums in the same order as
// the two kernels it replaces; the block size must be the one xprep_kernel would be launched with for K = n.
__global__ void __launch_bounds__(1024)
qgemm_reduce_prep_kernel(const float* __restrict__ partial, int slices, int T, int n, int epi, const float* __restrict__ residual,
                         float* __restrict__ out, const float* __restrict__ next_norm_w, float next_eps, __half* __restrict__ xh,
                         size_t lo_offset, __half* __restrict__ sx, size_t sx_lo_offset, float* __restrict__ tok_scale) {
    extern __shared__ float row[];
    __shared__ float sh[64];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const size_t plane = (size_t)T * n;
    float acc = 0.f, amax = 0.f;
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
        const size_t idx = (size_t)t * n + i;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        for (int sl = 0; sl < slices; sl++) {
            const float4 v = *reinterpret_cast<const float4*>(partial + (size_t)sl * plane + idx);
            float4& d = (epi == EPI_SILU_MUL && (sl & 1)) ? b : a;
            d.x += v.x; d.y += v.y; d.z += v.z; d.w += v.w;
        }
        if (epi == EPI_SILU_MUL) {
            a.x = __fmul_rn(silu_f(a.x), b.x); a.y = __fmul_rn(silu_f(a.y), b.y);
            a.z = __fmul_rn(silu_f(a.z), b.z); a.w = __fmul_rn(silu_f(a.w), b.w);
        } else if (epi == EPI_ADD_RESIDUAL) {
            const float4 r = *reinterpret_cast<const float4*>(residual + idx);
            a.x = __fadd_rn(r.x, a.x); a.y = __fadd_rn(r.y, a.y); a.z = __fadd_rn(r.z, a.z); a.w = __fadd_rn(r.w, a.w);
        }
        *reinterpret_cast<float4*>(out + idx) = a;
        *reinterpret_cast<float4*>(row + i) = a;
        acc = fmaf(a.x, a.x, acc); acc = fmaf(a.y, a.y, acc); acc = fmaf(a.z, a.z, acc); acc = fmaf(a.w, a.w, acc);
        float4 g = make_float4(1.f, 1.f, 1.f, 1.f);
        if (next_norm_w) g = *reinterpret_cast<const float4*>(next_norm_w + i);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x * g.x), fabsf(a.y * g.y)), fmaxf(fabsf(a.z * g.z), fabsf(a.w * g.w))));
    }
    xprep_row(row, acc, amax, next_norm_w, next_eps, n, t, xh, lo_offset, sx, sx_lo_offset, tok_scale, sh);
}

// ---- diagnostic: what the building blocks of the kernel above cost on this GPU ----------------------------------------
// One CTA, no global-memory traffic in the timed parts; every wait bounded.  out[] (SM cycles per operation):
//   0  tcgen05.mma M128 N128 K16, A in tensor memory, one issuing thread, a commit after every four
//   1  the same with N = 256
//   2  the same (N = 128) issued by two threads at once, own accumulators each: cycles per instruction of one thread
//   3  tcgen05.commit
//   4  tcgen05.st x16 + wait::st                  5  ... + fence + arrival of 128 threads on one barrier
//   6  tcgen05.ld x16 + wait::ld                  7  tcgen05.fence::before_thread_sync     8  ...::after_thread_sync
//   9  barrier probe of a completed phase + warp vote
//   10 arrival by one thread -> a waiting thread returns (mean of eight)
//   11 / 12 / 13  unpacking one 64-element chunk of 32 rows, per warp, with 4 / 8 / 16 warps at it
__global__ void __launch_bounds__(512, 1) tcgen05_probe_kernel(double* out) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + 96 * 1024);  // [0..7] and [16..23] count 1, [8..15] count 128
    uint32_t* slot = reinterpret_cast<uint32_t*>(bars + 24);
    long long* stamp = reinterpret_cast<long long*>(slot + 4);     // [16] hop stamps
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(sm)[i] = 0x11111111u * (uint32_t)(i % 7) + (uint32_t)i;
    if (tid == 0) {
        for (int i = 0; i < 24; i++) mbar_init(&bars[i], (i >= 8 && i < 16) ? 128 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *slot;
    bool ok = true;
    constexpr int R = 64;
    if (tid == 0) {  // 0, 1, 3: one issuer
        const uint64_t bdesc = umma_desc_sw128(smem_u32(sm));
        int ph = 0;
        for (int ni = 0; ni < 2; ni++) {
            const uint32_t id = idesc_f16(ni ? 256 : 128);
            const long long t0 = clock64();
            for (int r = 0; r < R; r++) {
                umma_f16_ts(tmem, tmem + 384 + (r & 3) * 8, bdesc + (uint64_t)((r & 3) * 2), id, 1u);
                if ((r & 3) == 3) umma_commit(&bars[1 + ((r >> 2) & 3)]);
            }
            const long long t1 = clock64();
            umma_commit(&bars[0]);
            const long long t2 = clock64();
            ok = mbar_wait(&bars[0], (uint32_t)ph) && ok;
            ph ^= 1;
            out[ni] = (double)(t1 - t0) / R;
            if (ni == 0) out[3] = (double)(t2 - t1);
        }
    }
    __syncthreads();
    if ((warp == 4 || warp == 5) && lane == 0) {  // 2: two issuers at once
        const int g = warp - 4;
        const uint64_t bdesc = umma_desc_sw128(smem_u32(sm + g * 32768));
        const uint32_t id = idesc_f16(128);
        const long long t0 = clock64();
        for (int r = 0; r < R; r++) {
            umma_f16_ts(tmem + g * 128, tmem + 384 + g * 64 + (r & 3) * 8, bdesc + (uint64_t)((r & 3) * 2), id, 1u);
            if ((r & 3) == 3) umma_commit(&bars[5 + g]);
        }
        const long long t1 = clock64();
        umma_commit(&bars[16 + g]);  // every product of this thread has completed before tensor memory is written below
        ok = mbar_wait(&bars[16 + g], 0u) && ok;
        if (g == 0) out[2] = (double)(t1 - t0) / R;
    }
    __syncthreads();
    if (warp < 4) {  // 4 .. 9
        uint32_t v[16];
        for (int i = 0; i < 16; i++) v[i] = (uint32_t)(lane + i);
        const uint32_t base = tmem + ((uint32_t)(warp * 32) << 16);
        long long t0 = clock64();
        for (int r = 0; r < 32; r++) { tmem_st16(base + 448 + (r & 1) * 16, v); asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
        long long t1 = clock64();
        for (int r = 0; r < 32; r++) {
            tmem_st16(base + 448 + (r & 1) * 16, v);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            mbar_arrive(&bars[8 + (r & 7)]);
        }
        long long t2 = clock64();
        uint32_t acc = 0;
        for (int r = 0; r < 32; r++) { tmem_ld16(base + 256 + (r & 3) * 16, v); asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); acc += v[3]; }
        long long t3 = clock64();
        for (int r = 0; r < 32; r++) tc_fence_before();
        long long t4 = clock64();
        for (int r = 0; r < 32; r++) tc_fence_after();
        long long t5 = clock64();
        for (int r = 0; r < 32; r++) acc += __all_sync(0xffffffffu, mbar_test(&bars[0], 1u)) ? 1u : 0u;  // phase 1 of barrier 0 completed above
        long long t6 = clock64();
        if (tid == 0) {
            out[4] = (t1 - t0) / 32.0; out[5] = (t2 - t1) / 32.0; out[6] = (t3 - t2) / 32.0; out[7] = (t4 - t3) / 32.0; out[8] = (t5 - t4) / 32.0;
            out[9] = (t6 - t5) / 32.0;
        }
        if (acc == 0x9e3779b9u) stamp[15] = 1;  // keeps the loads' results alive
    }
    __syncthreads();
    if (warp == 2 && lane == 0) {  // 10: the arriving side
        for (int r = 0; r < 8; r++) {
            const long long t = clock64();
            while (clock64() - t < 3000) {}
            stamp[r] = clock64();
            mbar_arrive(&bars[18]);
        }
    }
    if (warp == 3 && lane == 0) {  // 10: the waiting side
        for (int r = 0; r < 8; r++) { ok = mbar_wait(&bars[18], (uint32_t)(r & 1)) && ok; stamp[8 + r] = clock64(); }
    }
    __syncthreads();
    if (tid == 0) {
        double h = 0;
        for (int r = 0; r < 8; r++) h += (double)(stamp[8 + r] - stamp[r]);
        out[10] = h / 8;
    }
    for (int nw = 4, k = 0; nw <= 16; nw *= 2, k++) {  // 11 .. 13
        __syncthreads();
        if (warp < nw) {
            const unsigned char* rp = sm + ((warp & 3) * 32 + lane) * kUnitBytes;
            uint32_t acc = 0;
            const long long t0 = clock64();
            for (int it = 0; it < 32; it++) {
                HdrQ4K hdr;
                load_hdr(rp, hdr);
                for (int c = 0; c < 4; c++) {
                    uint32_t col[32];
                    unpack_chunk<kUnitBytes>(rp, hdr, c, col);
#pragma unroll
                    for (int i = 0; i < 32; i++) acc ^= col[i];
                    asm volatile("" ::: "memory");
                }
            }
            const long long t1 = clock64();
            if (tid == 0) out[11 + k] = (double)(t1 - t0) / 128.0;
            if (acc == 0x9e3779b9u) stamp[15] = 1;  // keeps the unpacked values alive
        }
    }
    if (!ok && tid == 0) out[15] = -1.0;
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

int32_t run_tcgen05_probe(double* out16_host, cudaStream_t s) {
    double* d = nullptr;
    LC_CUDA(cudaMalloc((void**)&d, 16 * sizeof(double)));
    LC_CUDA(cudaMemsetAsync(d, 0, 16 * sizeof(double), s));
    const size_t smem = 96 * 1024 + 1024 + 1024;
    LC_CUDA(ensure_smem_limit((const void*)tcgen05_probe_kernel, smem));
    tcgen05_probe_kernel<<<1, 512, smem, s>>>(d);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(out16_host, d, 16 * sizeof(double), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFree(d);
    LC_CUDA(e);
    LC_CHECK(out16_host[15] == 0.0, LC_ERR_CUDA, "tcgen05 probe: a bounded wait ran out");
    return LC_OK;
}

// ---- host side --------------------------------------------------------------------------------------------------------
int32_t qgemm_workspace_alloc(GemmWorkspace* ws, int t_cap, int k_max) {
    LC_CHECK(ws && t_cap > 0 && k_max > 0, LC_ERR_INVALID, "qgemm workspace: bad size");
    ws->t_cap = (t_cap + 15) & ~15;
    ws->k_max = k_max;
    const size_t bytes = (size_t)2 * ws->t_cap * k_max * sizeof(__half);
    LC_CUDA(cudaMalloc(&ws->xh, bytes));
    LC_CUDA(cudaMemset(ws->xh, 0, bytes));  // rows past the tokens of a call are multiplied too (and dropped): keep them finite
    LC_CUDA(cudaMalloc(&ws->sx, bytes / 16));
    LC_CUDA(cudaMemset(ws->sx, 0, bytes / 16));
    LC_CUDA(cudaMalloc((void**)&ws->tok_scale, (size_t)ws->t_cap * sizeof(float)));
    // shares of k of the batched decode step, and the two matrices of gate/up at any number of tokens
    ws->partial_bytes = std::max((size_t)64 << 20, (size_t)2 * ws->t_cap * k_max * sizeof(float));
    LC_CUDA(cudaMalloc((void**)&ws->partial, ws->partial_bytes));
    return LC_OK;
}
void qgemm_workspace_free(GemmWorkspace* ws) {
    if (!ws) return;
    if (ws->xh) cudaFree(ws->xh);
    if (ws->sx) cudaFree(ws->sx);
    if (ws->tok_scale) cudaFree(ws->tok_scale);
    if (ws->partial) cudaFree(ws->partial);
    ws->partial = nullptr;
    ws->xh = nullptr;
    ws->sx = nullptr;
    ws->tok_scale = nullptr;
}

static int gemm_min_tokens() {
    static const int v = getenv("LC_GEMM_MIN_TOKENS") ? atoi(getenv("LC_GEMM_MIN_TOKENS")) : 5;
    return v;
}
bool qgemm_applies(const GemvArgs& a, int T, const GemmWorkspace& ws) {
    if (!a.w || !ws.xh) return false;
    if ((a.w->typ != LC_TYPE_Q4_K && a.w->typ != LC_TYPE_Q5_K) || !a.w->has_tmap || a.w->k % kUnitElems != 0) return false;
    if (a.epi == EPI_SILU_MUL && (!a.w2 || a.w2->typ != a.w->typ || !a.w2->has_tmap)) return false;
    if (T < gemm_min_tokens() || T > ws.t_cap || a.w->k > ws.k_max) return false;
    if (((uintptr_t)a.x % 16) != 0 || (a.norm_w && ((uintptr_t)a.norm_w % 16) != 0)) return false;
    return true;
}

int32_t launch_qgemm(const GemvArgs& a, const GemmWorkspace& ws, cudaStream_t s, int* launches) {
    const int T = a.m, K = a.w->k, n = a.w->n;
    LC_CHECK(qgemm_applies(a, T, ws), LC_ERR_INVALID, "qgemm: arguments outside what the kernel implements");
    if (a.epi == EPI_ADD_RESIDUAL) LC_CHECK(a.residual != nullptr, LC_ERR_INVALID, "qgemm: residual missing");
    const int terms = (getenv("LC_GEMM_TERMS") && atoi(getenv("LC_GEMM_TERMS")) == 1) ? 1 : 3;  // read per call so that a test can switch it
    // activations: [t_cap rows of high halves | t_cap rows of low halves], each row k elements of this matrix
    const size_t lo_offset = (size_t)ws.t_cap * K, sx_lo_offset = (size_t)ws.t_cap * (K / 16);
    // the summing kernel of the product before this one may have prepared exactly this input (GemvArgs::prep_next)
    const bool prepared = ws.prep_x == a.x && ws.prep_norm == a.norm_w && ws.prep_k == K && ws.prep_t == T && a.x != nullptr;
    ws.prep_x = nullptr;
    if (!prepared) {
        const size_t smem = (size_t)K * sizeof(float);
        if (smem > 48 * 1024) LC_CUDA(ensure_smem_limit((const void*)xprep_kernel, smem));
        // a token's row is short (16 - 44 KB) and its three passes are latency: many threads, one or a few float4 each
        // (64 sequences, 4 layers: 2.43 / 2.40 / 2.40 ms per step with 256 / 512 / 1024 threads)
        LC_CUDA(launch_pdl(xprep_kernel, dim3(T), dim3(K >= 4096 ? 1024 : 256), smem, s, a.x, a.norm_w, a.eps, K, (__half*)ws.xh, lo_offset, (__half*)ws.sx,
                           sx_lo_offset, ws.tok_scale));
    }
    const int N = std::min(kMaxTok, (T + 15) & ~15);
    alignas(64) CUtensorMap tmx, tms;
    LC_CHECK(make_act_tmap_chunks(&tmx, ws.xh, (uint64_t)K, (uint64_t)ws.t_cap, (uint32_t)N, 2), LC_ERR_CUDA, "qgemm: activation tensor map");
    LC_CHECK(make_act_tmap(&tms, ws.sx, (uint64_t)K / 16, (uint64_t)ws.t_cap, (uint32_t)N), LC_ERR_CUDA, "qgemm: sums tensor map");
    GemmParams p;
    p.out = a.out; p.residual = a.residual; p.tok_scale = ws.tok_scale;
    p.n = n; p.k = K; p.T = T; p.N = N; p.epi = (int)a.epi; p.terms = terms;
    const int nmat = a.epi == EPI_SILU_MUL ? 2 : 1;
    // eight activation stages (two units: a stage always serves the same pipeline); the raw boxes take what is left
    const size_t b_bytes = (size_t)2 * N * 128;
    const size_t fixed = 1024 + (size_t)(2 * kMaxB + 2) * b_bytes + (size_t)kDRing * kRows * sizeof(float) + 512;
    const bool q5 = a.w->typ == LC_TYPE_Q5_K;
    const size_t unit_bytes = q5 ? 176 : kUnitBytes;
    p.raw_stages = std::min(kMaxRaw, (int)((kMaxSmem - fixed) / (unit_bytes * kRows)));
    if (getenv("LC_GEMM_RAWSTAGES")) p.raw_stages = std::max(2, std::min(p.raw_stages, atoi(getenv("LC_GEMM_RAWSTAGES"))));
    LC_CHECK(p.raw_stages >= 2, LC_ERR_UNSUPPORTED, "qgemm: shared memory too small");
    p.b_stages = kMaxB;
    p.error_flag = gemv_error_flag_dev();
    p.trace = nullptr;
    static unsigned* d_trace = nullptr;
    const bool want_trace = getenv("LC_GEMM_TRACE") != nullptr;
    if (want_trace) {
        if (!d_trace) LC_CUDA(cudaMalloc((void**)&d_trace, 56 * sizeof(unsigned)));
        LC_CUDA(cudaMemsetAsync(d_trace, 0, 56 * sizeof(unsigned), s));
        p.trace = d_trace;
    }
    const size_t smem = fixed + (size_t)p.raw_stages * unit_bytes * kRows;
    auto kern = q5 ? qgemm_umma_q4k_kernel<176> : qgemm_umma_q4k_kernel<kUnitBytes>;
    LC_CUDA(ensure_smem_limit((const void*)kern, smem));
    const CUtensorMap* t0 = (const CUtensorMap*)a.w->tmap_wide;
    const CUtensorMap* t1 = a.w2 ? (const CUtensorMap*)a.w2->tmap_wide : t0;
    // Few tiles (a batched decode step on the square matrices): split k over several CTAs so that all SMs work; the
    // shares are summed, in a fixed order, by a small second kernel.  Cost model: waves x units per CTA, plus four
    // units' worth of prologue and epilogue per wave.  The two matrices of gate/up always meet in that kernel.
    const int tiles = (n + kRows - 1) / kRows, ttiles = (T + kMaxTok - 1) / kMaxTok, nquads = (K / kUnitElems + 3) / 4;
    int ks = 1;
    {
        const int sms = sm_count();
        long best = -1;
        for (int c = 1; c <= std::min(8, nquads); c++) {
            if (c > 1 && (size_t)c * nmat * T * n * sizeof(float) > ws.partial_bytes) break;
            if (c > 1 && (n % 4 != 0 || T > 2 * kMaxTok)) break;
            const long waves = ((long)tiles * nmat * ttiles * c + sms - 1) / sms;
            const long cost = waves * (((nquads + c - 1) / c) * 4 + 4) + (c > 1 ? 3 : 0);
            if (best < 0 || cost < best) { best = cost; ks = c; }
        }
        static const int force_gu = getenv("LC_GEMM_KSPLIT_GU") ? atoi(getenv("LC_GEMM_KSPLIT_GU")) : 0;
        static const int force = getenv("LC_GEMM_KSPLIT") ? atoi(getenv("LC_GEMM_KSPLIT")) : 0;
        int f = nmat == 2 ? force_gu : force;
        {   // per-shape override for sweeps: LC_GEMM_KS_<n>_<k>
            char name[64];
            snprintf(name, sizeof(name), "LC_GEMM_KS_%d_%d", n, K);
            if (const char* v = getenv(name)) f = atoi(v);
        }
        if (f > 0 && f <= nquads && (f == 1 || (n % 4 == 0 && (size_t)f * nmat * T * n * sizeof(float) <= ws.partial_bytes))) ks = f;
    }
    const bool summed = ks > 1 || nmat == 2;
    if (summed) LC_CHECK((size_t)ks * nmat * T * n * sizeof(float) <= ws.partial_bytes && n % 4 == 0, LC_ERR_UNSUPPORTED, "qgemm: sums buffer too small");
    p.ksplit = ks;
    p.tiles = tiles; p.nmat = nmat;
    p.partial = summed ? ws.partial : nullptr;
    dim3 grid((unsigned)(tiles * nmat), (unsigned)ttiles, (unsigned)ks);
    LC_CUDA(launch_pdl(kern, grid, dim3(kThreads), smem, s, *t0, *t1, tmx, tms, p));
    if (summed) {
        const size_t plane = (size_t)T * n;
        if (a.prep_next && n % kUnitElems == 0 && n <= ws.k_max) {
            // one CTA per token sums the shares and prepares the row for the next product, whose k is this n
            const size_t rsmem = (size_t)n * sizeof(float);
            if (rsmem > 48 * 1024) LC_CUDA(ensure_smem_limit((const void*)qgemm_reduce_prep_kernel, rsmem));
            LC_CUDA(launch_pdl(qgemm_reduce_prep_kernel, dim3(T), dim3(n >= 4096 ? 1024 : 256), rsmem, s, (const float*)ws.partial, nmat * ks, T, n,
                               (int)a.epi, a.residual, a.out, a.next_norm_w, a.next_eps, (__half*)ws.xh, (size_t)ws.t_cap * n, (__half*)ws.sx,
                               (size_t)ws.t_cap * (n / 16), ws.tok_scale));
            ws.prep_x = a.out; ws.prep_norm = a.next_norm_w; ws.prep_k = n; ws.prep_t = T;
        } else {
            LC_CUDA(launch_pdl(qgemm_reduce_kernel, dim3((unsigned)((plane / 4 + 255) / 256)), dim3(256), 0, s, (const float*)ws.partial, nmat * ks,
                               plane, (int)a.epi, a.residual, a.out));
        }
    }
    if (launches) *launches = (prepared ? 1 : 2) + (summed ? 1 : 0);
    if (want_trace) {
        unsigned h[56];
        LC_CUDA(cudaStreamSynchronize(s));
        LC_CUDA(cudaMemcpy(h, d_trace, sizeof(h), cudaMemcpyDeviceToHost));
        const char* names[7] = {"activation producer (b_empty, s_empty)", "raw producer (raw_empty)", "issuer 0 (d_empty, b_full, a_full, s_full, am_full, other issuer's unit)",
                                "issuer 1", "unpack 0 (raw requested, raw_full, am_empty, a_empty + vote | unpacking, wait::st, fence + arrive)", "unpack 1", "drain (d_full)"};
        fprintf(stderr, "[gemm waits n=%d k=%d T=%d grid %ux%ux%u] cycles of CTA 0 per kind of wait | whole loop\n", n, K, T, grid.x, grid.y, grid.z);
        for (int r = 0; r < 7; r++) {
            fprintf(stderr, "  %-62s:", names[r]);
            for (int i = 0; i < 7; i++) fprintf(stderr, " %7u", h[r * 8 + i]);
            fprintf(stderr, " | %8u\n", h[r * 8 + 7]);
        }
    }
    return LC_OK;
}

}  // namespace lc

// Causal attention of MANY new tokens (a prefill chunk) over the paged f16 KV cache on the tensor cores
// (rust/src/inference/attention.rs:69-113 at seq_len > 1: scores = q . k / sqrt(head_dim) over the keys up to the query's
// own position, softmax, weighted sum of the values; grouped-query head mapping :85).  head_dim 128, 16-token pages.
//
// A CTA of four warps takes 64 consecutive tokens of one sequence (a "tile" the host lists) and one query head; warp w owns
// query rows 16 w .. 16 w + 15.  The context is walked in tiles of 64 keys: keys and values of four pages are copied into
// shared memory with cp.async (two buffers, the next tile in flight while this one is multiplied), 128-bit chunks
// XOR-swizzled by the row so that ldmatrix reads them without bank conflicts.
//   scores   S[16 x 64] = Q[16 x 128] . K^T on mma.sync m16n8k16 (f16 in, f32 out).  The f32 queries are cut into an f16
//            high part and the f16 remainder, both multiplied: the products with the f16 keys are exact and q keeps ~22 bits.
//   softmax  online (running maximum and sum per row, kept by the four lanes that share a row), in log2 units;
//   values   O[16 x 128] += P[16 x 64] . V, the weights again as high + low halves, the values transposed by ldmatrix.
// Keys past the query's position get weight zero; value rows the cache has not written yet are zero-filled on the way in
// (their weight is zero, but 0 * NaN would not be).  Sums run in a fixed order: results do not vary from run to run.
#include "lc_kernels.h"
#include "lc_attn.cuh"
#include "lc_tma.cuh"

namespace lc {

namespace {

constexpr int kHD = 128, kPage = 16, kQT = 64, kKT = 64;
constexpr int kRowBytes = kHD * 2;                 // one key / value / query row as f16
constexpr int kTileBytes = kKT * kRowBytes;        // 16 KB
constexpr size_t kPrefillSmem = (size_t)2 * kQT * kRowBytes + 4 * kTileBytes;  // Q hi, Q lo, K x 2, V x 2 = 96 KB

__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * kRowBytes + ((chunk ^ (row & 7)) << 4)); }

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// 16 bytes global -> shared; src_bytes = 0 writes zeros instead
__device__ __forceinline__ void cp16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

__global__ void __launch_bounds__(128, 2)
attention_prefill_kernel(const float* __restrict__ q, int q_stride, float* __restrict__ out, int out_stride, KvLayout kv,
                         const PrefillTile* __restrict__ tiles, const int32_t* __restrict__ page_table, int pages_per_seq, int n_heads) {
    extern __shared__ __align__(128) unsigned char smem[];
    pdl_launch_dependents();
    pdl_wait();
    const PrefillTile tl = tiles[blockIdx.x];
    const int head = blockIdx.y, kvh = head / (n_heads / kv.n_kv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const uint32_t s_qhi = smem_u32(smem), s_qlo = s_qhi + kQT * kRowBytes, s_k = s_qlo + kQT * kRowBytes, s_v = s_k + 2 * kTileBytes;
    const int32_t* pt = page_table + (size_t)tl.seq * pages_per_seq;
    const int ctx_end = tl.pos0 + tl.n;                    // keys 0 .. ctx_end - 1 are in the cache
    const int n_kt = (ctx_end + kKT - 1) / kKT;

    auto load_kv = [&](int kt, int buf) {  // 64 keys x 16 chunks, for K and for V: 8 + 8 copies per thread
        for (int c = tid; c < kKT * 16; c += 128) {
            const int key = c >> 4, chunk = c & 15, kp = kt * kKT + key;
            const bool valid = kp < ctx_end;
            const int page = valid ? pt[kp / kPage] : 0;
            const size_t src = (((size_t)page * kv.n_kv + kvh) * kPage + (kp & (kPage - 1))) * kHD + chunk * 8;
            const uint32_t dst = (uint32_t)(buf * kTileBytes) + swz(key, chunk);
            cp16(s_k + dst, (const __half*)kv.k_pool + src, valid ? 16 : 0);
            cp16(s_v + dst, (const __half*)kv.v_pool + src, valid ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_kv(0, 0);
    // queries of the tile: f32 -> f16 high part + f16 remainder, swizzled like the keys (rows past the tile's tokens are zero)
    for (int c = tid; c < kQT * 16; c += 128) {
        const int row = c >> 4, chunk = c & 15;
        uint4 hi = make_uint4(0u, 0u, 0u, 0u), lo = hi;
        if (row < tl.n) {
            const float4* src = reinterpret_cast<const float4*>(q + (size_t)(tl.tok0 + row) * q_stride + (size_t)head * kHD + chunk * 8);
            const float4 a = src[0], b = src[1];
            const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            uint32_t h[4], l[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const __half h0 = __float2half_rn(v[2 * i]), h1 = __float2half_rn(v[2 * i + 1]);
                const __half2 hh = __halves2half2(h0, h1);
                h[i] = *reinterpret_cast<const uint32_t*>(&hh);
                l[i] = pack_h2(v[2 * i] - __half2float(h0), v[2 * i + 1] - __half2float(h1));
            }
            hi = make_uint4(h[0], h[1], h[2], h[3]);
            lo = make_uint4(l[0], l[1], l[2], l[3]);
        }
        *reinterpret_cast<uint4*>(smem + swz(row, chunk)) = hi;
        *reinterpret_cast<uint4*>(smem + kQT * kRowBytes + swz(row, chunk)) = lo;
    }

    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // rows g and g + 8 of this warp
    const float sc = 1.4426950408889634f / sqrtf((float)kHD);        // scores in log2 units: one ex2 per weight
    const int qrow0 = warp * 16;
    const int qpos[2] = {tl.pos0 + qrow0 + g, tl.pos0 + qrow0 + g + 8};
    // a warp can stop at the tile that holds its last query's position
    const int my_last_kt = min(n_kt - 1, (tl.pos0 + qrow0 + 15) / kKT);
    const int a_row = qrow0 + (lane & 7) + ((lane >> 3) & 1) * 8, a_half = lane >> 4;

    for (int kt = 0; kt < n_kt; kt++) {
        const int buf = kt & 1;
        if (kt + 1 < n_kt) load_kv(kt + 1, buf ^ 1);
        if (kt + 1 < n_kt) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // tile kt (and, the first time, the queries) is in shared memory for every warp
        if (kt <= my_last_kt) {
            const uint32_t kb = s_k + buf * kTileBytes, vb = s_v + buf * kTileBytes;
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int kp = 0; kp < 4; kp++) {  // pairs of 16-dim steps
                uint32_t qh[2][4], ql[2][4];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const uint32_t off = swz(a_row, 2 * (2 * kp + u) + a_half);
                    ldsm4(s_qhi + off, qh[u][0], qh[u][1], qh[u][2], qh[u][3]);
                    ldsm4(s_qlo + off, ql[u][0], ql[u][1], ql[u][2], ql[u][3]);
                }
#pragma unroll
                for (int nt = 0; nt < 8; nt++) {
                    uint32_t b0, b1, b2, b3;
                    ldsm4(kb + swz(8 * nt + (lane & 7), 4 * kp + (lane >> 3)), b0, b1, b2, b3);
                    mma16816(s[nt], qh[0][0], qh[0][1], qh[0][2], qh[0][3], b0, b1);
                    mma16816(s[nt], ql[0][0], ql[0][1], ql[0][2], ql[0][3], b0, b1);
                    mma16816(s[nt], qh[1][0], qh[1][1], qh[1][2], qh[1][3], b2, b3);
                    mma16816(s[nt], ql[1][0], ql[1][1], ql[1][2], ql[1][3], b2, b3);
                }
            }
            // ---- scale, causal mask, online softmax (attention.rs:93-102) ----
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int kpos = kt * kKT + 8 * nt + 2 * t4 + (i & 1);
                    const float v = (kpos <= qpos[i >> 1]) ? s[nt][i] * sc : -INFINITY;
                    s[nt][i] = v;
                    mx[i >> 1] = fmaxf(mx[i >> 1], v);
                }
            }
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);  // finite: key 0 is never past a query's position
                corr[r] = exp2f(m_run[r] - m_new);
                m_run[r] = m_new;
            }
            float ps[2] = {0.f, 0.f};
            uint32_t ph[4][4], pl[4][4];  // the weights as A fragments, high and low halves, per 16-key step
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                float pv[4];
#pragma unroll
                for (int i = 0; i < 4; i++) { pv[i] = exp2f(s[nt][i] - m_run[i >> 1]); ps[i >> 1] += pv[i]; }
                const __half h0 = __float2half_rn(pv[0]), h1 = __float2half_rn(pv[1]), h2 = __float2half_rn(pv[2]), h3 = __float2half_rn(pv[3]);
                const __half2 u01 = __halves2half2(h0, h1), u23 = __halves2half2(h2, h3);
                const int ks = nt >> 1, hs = (nt & 1) * 2;  // n tile 2 ks -> registers 0, 1; n tile 2 ks + 1 -> registers 2, 3
                ph[ks][hs] = *reinterpret_cast<const uint32_t*>(&u01);
                ph[ks][hs + 1] = *reinterpret_cast<const uint32_t*>(&u23);
                pl[ks][hs] = pack_h2(pv[0] - __half2float(h0), pv[1] - __half2float(h1));
                pl[ks][hs + 1] = pack_h2(pv[2] - __half2float(h2), pv[3] - __half2float(h3));
            }
#pragma unroll
            for (int r = 0; r < 2; r++) {
                ps[r] += __shfl_xor_sync(0xffffffffu, ps[r], 1);
                ps[r] += __shfl_xor_sync(0xffffffffu, ps[r], 2);
                l_run[r] = l_run[r] * corr[r] + ps[r];
            }
#pragma unroll
            for (int i = 0; i < 16; i++) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
            // ---- O += P . V ----
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
#pragma unroll
                for (int np = 0; np < 8; np++) {
                    uint32_t b0, b1, b2, b3;
                    const int mi = lane >> 3;
                    ldsm4t(vb + swz(16 * ks + (lane & 7) + 8 * (mi & 1), 2 * np + (mi >> 1)), b0, b1, b2, b3);
                    mma16816(o[2 * np], ph[ks][0], ph[ks][1], ph[ks][2], ph[ks][3], b0, b1);
                    mma16816(o[2 * np], pl[ks][0], pl[ks][1], pl[ks][2], pl[ks][3], b0, b1);
                    mma16816(o[2 * np + 1], ph[ks][0], ph[ks][1], ph[ks][2], ph[ks][3], b2, b3);
                    mma16816(o[2 * np + 1], pl[ks][0], pl[ks][1], pl[ks][2], pl[ks][3], b2, b3);
                }
            }
        }
        __syncthreads();  // every warp is done with buffer `buf` before the copy of tile kt + 2 lands in it
    }
    // ---- out = O / l ----
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = qrow0 + g + 8 * r;
        if (row >= tl.n) continue;
        const float inv = 1.0f / l_run[r];
        float* dst = out + (size_t)(tl.tok0 + row) * out_stride + (size_t)head * kHD + 2 * t4;
#pragma unroll
        for (int nt = 0; nt < 16; nt++) *reinterpret_cast<float2*>(dst + 8 * nt) = make_float2(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
    }
}

}  // namespace

bool attention_prefill_applies(const KvLayout& kv, int n_heads) {
    return kv.hd == kHD && !kv.kv_f32 && kv.page_tokens == kPage && kv.n_kv > 0 && n_heads % kv.n_kv == 0;
}

int32_t launch_attention_prefill(const float* q, int q_stride, float* out, int n_heads, const KvLayout& kv, const PrefillTile* tiles_dev, int n_tiles,
                                 const int32_t* page_table, int pages_per_seq, cudaStream_t s) {
    if (n_tiles <= 0) return LC_OK;
    LC_CHECK(attention_prefill_applies(kv, n_heads) && ((uintptr_t)q % 16) == 0 && q_stride % 4 == 0, LC_ERR_INVALID,
             "attention prefill: head_dim 128, f16 cache and 16-token pages only");
    LC_CUDA(ensure_smem_limit((const void*)attention_prefill_kernel, kPrefillSmem));
    LC_CUDA(launch_pdl(attention_prefill_kernel, dim3((unsigned)n_tiles, (unsigned)n_heads), dim3(128), kPrefillSmem, s, q, q_stride, out,
                       n_heads * kHD, kv, tiles_dev, page_table, pages_per_seq, n_heads));
    return LC_OK;
}

}  // namespace lc

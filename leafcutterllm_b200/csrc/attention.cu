// RoPE + paged KV-cache append, and causal grouped-query attention over the
// paged cache (rust/src/inference/attention.rs:13-118, rust/src/cache/mod.rs:33-77).
//
// Cache layout: per layer one K pool and one V pool, [page][kv_head][token in page][head_dim],
// f16 (the reference's storage type) or f32.  A (page, kv_head) slab is contiguous, so the
// keys a warp walks are 128-bit loads of consecutive addresses.
//
// Attention is split over the context: CTA (token, head, split) reduces its slice with an
// online softmax in fp32 and writes (max, sum, weighted V); the last CTA of a (token, head) to
// finish merges the splits in split order.  The reference's three-pass softmax and this one agree to rounding.
#include "lc_kernels.h"
#include "lc_attn.cuh"
#include "lc_tma.cuh"

namespace lc {

__global__ void rope_kv_append_kernel(float* __restrict__ q, float* __restrict__ k, const float* __restrict__ v, int row_stride,
                                      int n_tok, int n_heads, KvLayout kv, const int32_t* __restrict__ tok_seq,
                                      const int32_t* __restrict__ tok_pos, const int32_t* __restrict__ tok_rope,
                                      const int32_t* __restrict__ page_table, int pages_per_seq, float theta) {
    pdl_launch_dependents();
    pdl_wait();
    const int hd = kv.hd, half = hd / 2;
    const int per_tok = (n_heads + kv.n_kv) * half;
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tok * per_tok) return;
    int tok = (int)(idx / per_tok), r = (int)(idx % per_tok);
    int h = r / half, d = r % half;
    // attention.rs:16-20
    float freq = __fdiv_rn(1.0f, powf(theta, __fdiv_rn(__fmul_rn(2.0f, (float)d), (float)hd)));
    float angle = __fmul_rn((float)tok_rope[tok], freq);
    float ca = cosf(angle), sa = sinf(angle);
    if (h < n_heads) {
        float* p = q + (size_t)tok * row_stride + h * hd;
        float x1 = p[d], x2 = p[d + half];
        p[d] = __fsub_rn(__fmul_rn(x1, ca), __fmul_rn(x2, sa));
        p[d + half] = __fadd_rn(__fmul_rn(x1, sa), __fmul_rn(x2, ca));
    } else {
        int kh = h - n_heads;
        float* p = k + (size_t)tok * row_stride + kh * hd;
        const float* pv = v + (size_t)tok * row_stride + kh * hd;
        float x1 = p[d], x2 = p[d + half];
        float r1 = __fsub_rn(__fmul_rn(x1, ca), __fmul_rn(x2, sa));
        float r2 = __fadd_rn(__fmul_rn(x1, sa), __fmul_rn(x2, ca));
        p[d] = r1;
        p[d + half] = r2;
        int pos = tok_pos[tok];
        int page = page_table[(size_t)tok_seq[tok] * pages_per_seq + pos / kv.page_tokens];
        size_t base = (((size_t)page * kv.n_kv + kh) * kv.page_tokens + pos % kv.page_tokens) * hd;
        if (kv.kv_f32) {
            float* K = (float*)kv.k_pool; float* V = (float*)kv.v_pool;
            K[base + d] = r1; K[base + d + half] = r2;
            V[base + d] = pv[d]; V[base + d + half] = pv[d + half];
        } else {
            __half* K = (__half*)kv.k_pool; __half* V = (__half*)kv.v_pool;
            K[base + d] = __float2half_rn(r1); K[base + d + half] = __float2half_rn(r2);
            V[base + d] = __float2half_rn(pv[d]); V[base + d + half] = __float2half_rn(pv[d + half]);
        }
    }
}

template <int HD, bool F32>
__global__ void __launch_bounds__(kAttnWarps * 32)
attention_split_kernel(AttnParams p) {
    __shared__ float sh[8 + kAttnWarps * HD + 4];
    pdl_launch_dependents();
    pdl_wait();
    attention_item<HD, F32, 0>(p, (int)blockIdx.x, (int)blockIdx.y, (int)threadIdx.x, sh);
}

// Decode attention with the whole key/value slice of the CTA staged in shared memory by bulk copies
// (head_dim 128, f16 cache, 16-token pages).  One CTA per (token, kv head, split of 128 keys): the sixteen 4 KB
// (page, kv head) slabs of K and V are requested at once on one mbarrier -- a single memory round trip instead of one
// per pass -- and, in a fused decode step, BEFORE the grid dependency wait, because cached keys do not depend on the
// projection kernel that precedes this one.  All q heads of the kv group are then served from the staged slice.
constexpr int kStagedChunk = 128;
template <int HD>
__global__ void __launch_bounds__(kAttnWarps * 32) attention_staged_kernel(AttnParams p) {
    static_assert(HD == 128 && kAttnWarps * 32 == HD, "one thread per key and per dim");
    extern __shared__ __align__(128) unsigned char dsm[];
    __half* K_s = reinterpret_cast<__half*>(dsm);
    __half* V_s = K_s + kStagedChunk * HD;
    __shared__ __align__(16) float sh[6 * HD];  // q, p, four partial accumulators
    __shared__ __align__(8) uint64_t bar;
    const KvLayout& kv = p.kv;
    const int n_heads = p.n_heads, gsz = n_heads / kv.n_kv;
    const int tok = blockIdx.x / kv.n_kv, kvh = blockIdx.x % kv.n_kv, split = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool fused = p.k_new != nullptr;
    auto stage = [&](int pos) {
        const int t_begin = split * p.chunk, t_end = min(pos + 1, t_begin + p.chunk);
        if (tid == 0) {
            mbar_init(&bar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (t_begin < t_end) {
                const int32_t* pt = p.page_table + (size_t)p.tok_seq[tok] * p.pages_per_seq;
                const int pg0 = t_begin / 16, npg = (t_end - t_begin + 15) / 16;
                int32_t pgs[kStagedChunk / 16];
#pragma unroll
                for (int i = 0; i < kStagedChunk / 16; i++) pgs[i] = pt[pg0 + (i < npg ? i : 0)];  // all page ids in flight together
                mbar_expect_tx(&bar, (uint32_t)(npg * 2 * 16 * HD * 2));
#pragma unroll
                for (int i = 0; i < kStagedChunk / 16; i++) {
                    if (i < npg) {
                        const size_t src = ((size_t)pgs[i] * kv.n_kv + kvh) * 16 * HD;
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                         smem_u32(K_s + (size_t)i * 16 * HD)),
                                     "l"((const __half*)kv.k_pool + src), "r"(16 * HD * 2), "r"(smem_u32(&bar))
                                     : "memory");
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                         smem_u32(V_s + (size_t)i * 16 * HD)),
                                     "l"((const __half*)kv.v_pool + src), "r"(16 * HD * 2), "r"(smem_u32(&bar))
                                     : "memory");
                    }
                }
            }
        }
    };
    int pos;
    if (fused && p.positions_settled) {  // the cache holds only earlier steps' tokens: fetch before waiting for the projection kernel
        pos = p.tok_pos[tok];
        stage(pos);
        pdl_launch_dependents();
        pdl_wait();
    } else {      // the previous kernel wrote this call's keys into the cache
        pdl_launch_dependents();
        pdl_wait();
        pos = p.tok_pos[tok];
        stage(pos);
    }
    const int t_begin = split * p.chunk, t_end = min(pos + 1, t_begin + p.chunk);
    const int n = t_end - t_begin;
    __syncthreads();  // barrier initialised
    bool ok = true;
    if (n > 0) ok = mbar_wait(&bar, 0);
    const int rp = fused ? p.tok_rope[tok] : 0;
    if (n > 0 && fused && pos >= t_begin && pos < t_end) {
        // the token of this step replaces the (stale) staged slot: rotate, round through f16, keep in the cache
        const int row = pos - t_begin;
        float kr[1], vr;
        load_rotated<1, HD>(p.k_new + (size_t)tok * p.q_stride + kvh * HD, tid, rp, p.theta, kr);
        vr = __ldcg(p.v_new + (size_t)tok * p.q_stride + kvh * HD + tid);
        const __half hk = __float2half_rn(kr[0]), hv = __float2half_rn(vr);  // cache/mod.rs:35-36
        K_s[row * HD + tid] = hk;
        V_s[row * HD + tid] = hv;
        const int32_t* pt = p.page_table + (size_t)p.tok_seq[tok] * p.pages_per_seq;
        const size_t dst = (((size_t)pt[pos / 16] * kv.n_kv + kvh) * 16 + pos % 16) * HD + tid;
        ((__half*)kv.k_pool)[dst] = hk;
        ((__half*)kv.v_pool)[dst] = hv;
    }
    __syncthreads();
    // ---- compute: short dependency chains instead of an online softmax ----
    //  scores : thread t owns key t (its 256-byte row from shared memory, 16-byte chunks walked in an order rotated
    //           by t so that a quarter warp never hits one bank twice), four partial sums;
    //  softmax: one block max, one exp per key, one block sum (the three passes of attention.rs:96-102 on the slice);
    //  p.V    : warp w takes keys 32w..32w+31, lane j takes dims 4j..4j+3 (64-bit conflict-free reads), the four warps
    //           are added in warp order.
    const float inv_div = sqrtf((float)HD);  // attention.rs:93
    float* q_s = sh;                      // [128]
    float* p_s = sh + HD;                 // [128]
    float* acc_s = sh + 2 * HD;           // [4][128]
    __shared__ float red_s[8];
    __shared__ int last_s;
    for (int hq = 0; hq < gsz; hq++) {
        const int h = kvh * gsz + hq, item = tok * n_heads + h;
        float* pout = p.partial + ((size_t)item * p.n_splits + split) * (HD + 2);
        float m = -INFINITY, l = 0.f, a_out = 0.f;
        if (n > 0) {
            {
                float qv[1];
                load_rotated<1, HD>(p.q + (size_t)tok * p.q_stride + h * HD, tid, rp, p.theta, qv);
                __syncthreads();  // the previous head is done with q_s / p_s / acc_s
                q_s[tid] = qv[0];
            }
            __syncthreads();
            float sc = -INFINITY;
            if (tid < n) {
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
                const __half* krow = K_s + (size_t)tid * HD;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int c = (j + tid) & 15;
                    const uint4 kq = *reinterpret_cast<const uint4*>(krow + c * 8);
                    const float4 qa = *reinterpret_cast<const float4*>(q_s + c * 8);
                    const float4 qb = *reinterpret_cast<const float4*>(q_s + c * 8 + 4);
                    const __half2* h2 = reinterpret_cast<const __half2*>(&kq);
                    const float2 k0 = __half22float2(h2[0]), k1 = __half22float2(h2[1]), k2 = __half22float2(h2[2]), k3 = __half22float2(h2[3]);
                    d0 = fmaf(qa.x, k0.x, d0); d1 = fmaf(qa.y, k0.y, d1); d2 = fmaf(qa.z, k1.x, d2); d3 = fmaf(qa.w, k1.y, d3);
                    d0 = fmaf(qb.x, k2.x, d0); d1 = fmaf(qb.y, k2.y, d1); d2 = fmaf(qb.z, k3.x, d2); d3 = fmaf(qb.w, k3.y, d3);
                }
                sc = ((d0 + d1) + (d2 + d3)) / inv_div;
            }
            const float wm = warp_max(sc);
            if (lane == 0) red_s[warp] = wm;
            __syncthreads();
            m = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
            const float pe = (tid < n) ? expf(sc - m) : 0.f;
            p_s[tid] = pe;
            const float ws = warp_sum(pe);
            if (lane == 0) red_s[4 + warp] = ws;
            __syncthreads();
            l = ((red_s[4] + red_s[5]) + red_s[6]) + red_s[7];
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            const int kend = min(n, 32 * warp + 32);
#pragma unroll 4
            for (int k = 32 * warp; k < kend; k++) {
                const float pk = p_s[k];
                const uint2 vq = *reinterpret_cast<const uint2*>(V_s + (size_t)k * HD + 4 * lane);
                const __half2* h2 = reinterpret_cast<const __half2*>(&vq);
                const float2 v0 = __half22float2(h2[0]), v1 = __half22float2(h2[1]);
                a0 = fmaf(pk, v0.x, a0); a1 = fmaf(pk, v0.y, a1); a2 = fmaf(pk, v1.x, a2); a3 = fmaf(pk, v1.y, a3);
            }
            *reinterpret_cast<float4*>(acc_s + warp * HD + 4 * lane) = make_float4(a0, a1, a2, a3);
            __syncthreads();
            a_out = ((acc_s[tid] + acc_s[HD + tid]) + acc_s[2 * HD + tid]) + acc_s[3 * HD + tid];
        }
        if (p.n_splits == 1) {
            p.out[(size_t)item * HD + tid] = a_out / l;
            continue;
        }
        if (tid == 0) { pout[0] = m; pout[1] = l; }
        pout[2 + tid] = a_out;
        // the last split of this (token, head) to finish merges all of them, in split order
        __threadfence();
        __syncthreads();
        if (tid == 0) last_s = (atomicAdd(&p.counters[item], 1) == p.n_splits - 1);
        __syncthreads();
        if (last_s) {
            __threadfence();
            const float* pp = p.partial + (size_t)item * p.n_splits * (HD + 2);
            float mm = -INFINITY;
            for (int s2 = 0; s2 < p.n_splits; s2++) mm = fmaxf(mm, __ldcg(pp + (size_t)s2 * (HD + 2)));
            float ll = 0.f, a = 0.f;
            for (int s2 = 0; s2 < p.n_splits; s2++) {
                const float* ps = pp + (size_t)s2 * (HD + 2);
                const float ms = __ldcg(ps);
                if (ms == -INFINITY) continue;  // empty split
                const float scl = expf(ms - mm);
                ll += __ldcg(ps + 1) * scl;
                a += __ldcg(ps + 2 + tid) * scl;
            }
            p.out[(size_t)item * HD + tid] = a / ll;
            if (tid == 0) p.counters[item] = 0;
        }
    }
    if (!ok && tid == 0 && p.error_flag) atomicExch(p.error_flag, 1);
}

// ---------------------------------------------------------------------------
static bool g_attn_pdl = getenv("LC_NO_PDL") == nullptr;
template <typename... KArgs, typename... Args>
static cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_attn_pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

int32_t launch_rope_kv_append(float* q, float* k, const float* v, int row_stride, int n_tok, int n_heads, const KvLayout& kv,
                              const int32_t* tok_seq, const int32_t* tok_pos, const int32_t* tok_rope,
                              const int32_t* page_table, int pages_per_seq, float theta, cudaStream_t s) {
    if (n_tok <= 0) return LC_OK;
    long long total = (long long)n_tok * (n_heads + kv.n_kv) * (kv.hd / 2);
    unsigned grid = (unsigned)((total + 255) / 256);
    LC_CUDA(launch_k(rope_kv_append_kernel, dim3(grid), dim3(256), s, q, k, v, row_stride, n_tok, n_heads, kv, tok_seq, tok_pos,
                     tok_rope, page_table, pages_per_seq, theta));
    return LC_OK;
}

// (token, head) pairs up to which decode attention uses the split-context kernel with shared-memory staging
static int staged_pair_limit() { return sm_count() * 4; }

static void split_plan(int n_tok, int n_heads, int max_ctx, int* chunk, int* n_splits) {
    int want_ctas = sm_count() * 4;
    int base = n_tok * n_heads;
    int splits = (want_ctas + base - 1) / base;
    if (splits < 1) splits = 1;
    int ch = (max_ctx + splits - 1) / splits;
    ch = (ch + 63) / 64 * 64;
    // A batched decode step (up to 256 tokens, each over its own long context): contexts differ widely, and the CTA of the
    // longest one would run on alone at the end; 1024-key pieces keep the tail short (64 sequences: 2.66 -> 2.49 ms for 4 layers).
    if (n_tok <= 256 && ch > 1024) ch = 1024;
    *chunk = ch;
    *n_splits = (max_ctx + ch - 1) / ch;
    if (*n_splits < 1) *n_splits = 1;
}

size_t attention_scratch_bytes(int n_tok, int n_heads, int hd, int max_ctx) {
    int chunk, splits;
    split_plan(n_tok, n_heads, max_ctx, &chunk, &splits);
    size_t staged = (size_t)n_tok * n_heads * ((max_ctx + kStagedChunk - 1) / kStagedChunk) * (hd + 2) * sizeof(float);
    if (n_tok * n_heads > staged_pair_limit()) staged = 16;
    size_t plain = splits == 1 ? 16 : (size_t)n_tok * n_heads * splits * (hd + 2) * sizeof(float);
    return plain > staged ? plain : staged;
}

static bool staged_applies(const AttnParams& p, int n_tok) {
    // few tokens (decode): the split-context kernel with shared-memory staging; many tokens (prefill) keep one CTA per (token, head)
    // Up to four tokens; from eight on the pipelined split-context kernel is faster (7B shape, 8 layers, 1024 keys of context, ms per
    // step staged / split: 4 sequences 0.95 / 0.97, 8 sequences 1.47 / 1.41, 16 sequences 1.77 / 1.55; Mixtral shape, 16 sequences:
    // 17.9 / 17.1 ms per step).
    static const int lim = getenv("LC_ATTN_STAGED_TOKENS") ? atoi(getenv("LC_ATTN_STAGED_TOKENS")) : 4;
    return p.kv.hd == 128 && !p.kv.kv_f32 && p.kv.page_tokens == 16 && n_tok * p.n_heads <= staged_pair_limit() && n_tok <= lim;
}

template <int HD>
static int32_t launch_attention_hd(const AttnParams& base, int n_tok, int max_ctx, cudaStream_t s) {
    AttnParams p = base;
    if (HD == 128 && staged_applies(p, n_tok)) {
        p.chunk = kStagedChunk;
        p.n_splits = (max_ctx + kStagedChunk - 1) / kStagedChunk;
        const size_t smem = (size_t)kStagedChunk * 128 * 2 * 2;
        LC_CUDA(ensure_smem_limit((const void*)attention_staged_kernel<128>, smem));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(n_tok * p.kv.n_kv), (unsigned)p.n_splits);
        cfg.blockDim = dim3(kAttnWarps * 32);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = g_attn_pdl ? 1 : 0;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        LC_CUDA(cudaLaunchKernelEx(&cfg, attention_staged_kernel<128>, p));
        return LC_OK;
    }
    split_plan(n_tok, p.n_heads, max_ctx, &p.chunk, &p.n_splits);
    dim3 grid((unsigned)(n_tok * p.n_heads), (unsigned)p.n_splits);
    if (p.kv.kv_f32) LC_CUDA(launch_k(attention_split_kernel<HD, true>, grid, dim3(kAttnWarps * 32), s, p));
    else LC_CUDA(launch_k(attention_split_kernel<HD, false>, grid, dim3(kAttnWarps * 32), s, p));
    return LC_OK;
}

int32_t launch_attention(const float* q, int q_stride, float* out, int n_tok, int n_heads, const KvLayout& kv,
                         const int32_t* tok_seq, const int32_t* tok_pos, const int32_t* page_table, int pages_per_seq, int max_ctx,
                         void* scratch, int* counters, const AttnFusion* fuse, cudaStream_t s) {
    if (n_tok <= 0) return LC_OK;
    AttnParams p;
    p.q = q; p.q_stride = q_stride; p.out = out; p.n_heads = n_heads; p.kv = kv; p.tok_seq = tok_seq; p.tok_pos = tok_pos;
    p.page_table = page_table; p.pages_per_seq = pages_per_seq; p.chunk = 0; p.n_splits = 1; p.partial = (float*)scratch;
    p.counters = counters;
    p.k_new = fuse ? fuse->k_new : nullptr; p.v_new = fuse ? fuse->v_new : nullptr;
    p.tok_rope = fuse ? fuse->tok_rope : nullptr; p.theta = fuse ? fuse->theta : 0.f;
    p.positions_settled = (fuse && fuse->positions_settled) ? 1 : 0;
    p.error_flag = gemv_error_flag_dev();
    if (fuse && fuse->stream_slots && attention_stream_applies(p, n_tok)) return launch_attention_stream(p, fuse->stream_slots, s);
    switch (kv.hd) {
        case 32: return launch_attention_hd<32>(p, n_tok, max_ctx, s);
        case 64: return launch_attention_hd<64>(p, n_tok, max_ctx, s);
        case 128: return launch_attention_hd<128>(p, n_tok, max_ctx, s);
        case 256: return launch_attention_hd<256>(p, n_tok, max_ctx, s);
        default:
            set_error("attention: head_dim %d is not one of 32, 64, 128, 256", kv.hd);
            return LC_ERR_UNSUPPORTED;
    }
}

}  // namespace lc

// ===========================================================================
// Decode attention as a device-level operator of the C ABI
// ===========================================================================
using namespace lc;

namespace {
struct AttnOpScratch { DevBuf buf; };
AttnOpScratch g_attn_op[16];

struct AttnOpArgs {
    const float* q; const void* k_pool; const void* v_pool; const int32_t* page_table;
    int32_t n_pages, ctx_len, n_heads, n_kv, hd, page_tokens, kv_f32;
    float* out;
};

int32_t attn_op_validate(const AttnOpArgs& a, const char* who) {
    LC_CHECK(a.q && a.k_pool && a.v_pool && a.page_table && a.out, LC_ERR_INVALID, "%s: null pointer", who);
    LC_CHECK(a.n_heads > 0 && a.n_kv > 0 && a.n_heads % a.n_kv == 0, LC_ERR_INVALID, "%s: %d heads over %d kv heads", who, a.n_heads, a.n_kv);
    LC_CHECK(a.hd == 32 || a.hd == 64 || a.hd == 128 || a.hd == 256, LC_ERR_UNSUPPORTED, "%s: head_dim %d is not one of 32, 64, 128, 256", who, a.hd);
    LC_CHECK(a.page_tokens > 0 && a.ctx_len >= 1 && (int64_t)a.n_pages * a.page_tokens >= a.ctx_len, LC_ERR_INVALID,
             "%s: %d pages of %d tokens cannot hold a context of %d", who, a.n_pages, a.page_tokens, a.ctx_len);
    return LC_OK;
}

// scratch layout: [0,256): tok_seq, tok_pos   [256, 256+4*n_heads): counters   then the split partials
size_t attn_op_scratch_bytes(const AttnOpArgs& a) {
    size_t ctr = ((size_t)a.n_heads * 4 + 255) & ~(size_t)255;
    return 256 + ctr + attention_scratch_bytes(1, a.n_heads, a.hd, a.ctx_len);
}

int32_t attn_op_run(const AttnOpArgs& a, unsigned char* scratch, cudaStream_t s) {
    const int32_t meta[2] = {0, a.ctx_len - 1};
    size_t ctr = ((size_t)a.n_heads * 4 + 255) & ~(size_t)255;
    LC_CUDA(cudaMemcpyAsync(scratch, meta, sizeof(meta), cudaMemcpyHostToDevice, s));
    LC_CUDA(cudaMemsetAsync(scratch + 256, 0, ctr, s));  // the split counters must start at zero
    KvLayout kv;
    kv.k_pool = const_cast<void*>(a.k_pool); kv.v_pool = const_cast<void*>(a.v_pool);
    kv.n_kv = a.n_kv; kv.hd = a.hd; kv.page_tokens = a.page_tokens; kv.kv_f32 = a.kv_f32;
    const int32_t* meta_dev = reinterpret_cast<const int32_t*>(scratch);
    return launch_attention(a.q, a.n_heads * a.hd, a.out, 1, a.n_heads, kv, meta_dev, meta_dev + 1, a.page_table, a.n_pages, a.ctx_len,
                            scratch + 256 + ctr, reinterpret_cast<int*>(scratch + 256), nullptr, s);
}

// Scratch of lc_attention_decode_static: lives in the library image, so every GPU that loads the library
// holds this 1 MiB until the process exits.
constexpr size_t kStaticAttnScratchBytes = (size_t)1 << 20;
static __device__ __align__(256) unsigned char g_static_attn_scratch[kStaticAttnScratchBytes];
unsigned char* g_static_attn_ptr[16] = {};
}  // namespace

extern "C" {

int32_t lc_attention_decode_dev(const float* q_dev, const void* k_pool_dev, const void* v_pool_dev, const int32_t* page_table_dev,
                                int32_t n_pages, int32_t ctx_len, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                                int32_t page_tokens, int32_t kv_f32, float* out_dev) {
    if (!have_device()) return LC_ERR_CUDA;
    AttnOpArgs a{q_dev, k_pool_dev, v_pool_dev, page_table_dev, n_pages, ctx_len, n_heads, n_kv_heads, head_dim, page_tokens, kv_f32, out_dev};
    LC_TRY(attn_op_validate(a, "lc_attention_decode_dev"));
    int dev = 0;
    LC_CUDA(cudaGetDevice(&dev));
    LC_CHECK(dev >= 0 && dev < 16, LC_ERR_INVALID, "device ordinal %d out of range", dev);
    LC_TRY(g_attn_op[dev].buf.reserve(attn_op_scratch_bytes(a)));
    return attn_op_run(a, (unsigned char*)g_attn_op[dev].buf.p, stream());
}

int32_t lc_attention_decode_static(const float* q_dev, const void* k_pool_dev, const void* v_pool_dev, const int32_t* page_table_dev,
                                   int32_t n_pages, int32_t ctx_len, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                                   int32_t page_tokens, int32_t kv_f32, float* out_dev) {
    if (!have_device()) return LC_ERR_CUDA;
    AttnOpArgs a{q_dev, k_pool_dev, v_pool_dev, page_table_dev, n_pages, ctx_len, n_heads, n_kv_heads, head_dim, page_tokens, kv_f32, out_dev};
    LC_TRY(attn_op_validate(a, "lc_attention_decode_static"));
    const size_t need = attn_op_scratch_bytes(a);
    LC_CHECK(need <= kStaticAttnScratchBytes, LC_ERR_INVALID,
             "lc_attention_decode_static: this shape needs %zu bytes of split scratch, the built-in array holds %zu; use "
             "lc_attention_decode_dev for larger head counts or contexts", need, kStaticAttnScratchBytes);
    int dev = 0;
    LC_CUDA(cudaGetDevice(&dev));
    LC_CHECK(dev >= 0 && dev < 16, LC_ERR_INVALID, "device ordinal %d out of range", dev);
    if (!g_static_attn_ptr[dev]) {
        // first call on this device: resolve the device address of the array (its host-side name is only a handle)
        void* p = nullptr;
        LC_CUDA(cudaGetSymbolAddress(&p, g_static_attn_scratch));
        g_static_attn_ptr[dev] = (unsigned char*)p;
        if (!stream()) { set_error("could not create the library stream"); return LC_ERR_CUDA; }
    }
    return attn_op_run(a, g_static_attn_ptr[dev], stream());
}

}  // extern "C"

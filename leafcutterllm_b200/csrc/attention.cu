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

constexpr int kAttnWarps = 4;

struct AttnParams {
    const float* q;        // [n_tok, q_stride]: head h at q + tok*q_stride + h*hd
    int q_stride;
    float* out;            // [n_tok, n_heads*hd]
    int n_heads;
    KvLayout kv;
    const int32_t* tok_seq;
    const int32_t* tok_pos;
    const int32_t* page_table;
    int pages_per_seq;
    int chunk, n_splits;
    float* partial;        // [n_tok*n_heads][n_splits][hd+2]
    int* counters;         // [n_tok*n_heads], zero between launches
    // Decode-step fusion: every token is the only new token of its sequence.  q is rotated on load, the
    // new key/value come from k_new/v_new (rotated, rounded to the cache type exactly as a cache round
    // trip would) and are stored into the cache by the CTA that meets them.
    const float* k_new;    // null = keys and values are already in the cache and q is already rotated
    const float* v_new;
    const int32_t* tok_rope;
    float theta;
};

template <int DPL, bool F32>
__device__ __forceinline__ void load_slice(const void* pool, size_t elem_off, float (&out)[DPL]) {
    if (F32) {
        const float4* p = reinterpret_cast<const float4*>((const float*)pool + elem_off);
#pragma unroll
        for (int i = 0; i < DPL / 4; i++) { float4 v = p[i]; out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w; }
    } else {
        const uint4* p = reinterpret_cast<const uint4*>((const __half*)pool + elem_off);
#pragma unroll
        for (int i = 0; i < DPL / 8; i++) {
            uint4 v = p[i];
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; j++) { float2 f = __half22float2(h[j]); out[8 * i + 2 * j] = f.x; out[8 * i + 2 * j + 1] = f.y; }
        }
    }
}

// Dims d0 .. d0+DPL-1 of a head vector at `base`, rotated by position `rp` (attention.rs:13-34: pairs
// (d, d + hd/2), freq = 1 / theta^(2d/hd)).  rp == 0 is the identity and skips the trigonometry.
template <int DPL, int HD>
__device__ __forceinline__ void load_rotated(const float* base, int d0, int rp, float theta, float (&out)[DPL]) {
#pragma unroll
    for (int i = 0; i < DPL; i++) out[i] = base[d0 + i];
    if (rp == 0) return;
    constexpr int HALF = HD / 2;
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = d0 + i, dd = d < HALF ? d : d - HALF;
        const float freq = __fdiv_rn(1.0f, powf(theta, __fdiv_rn(__fmul_rn(2.0f, (float)dd), (float)HD)));
        const float angle = __fmul_rn((float)rp, freq);
        const float ca = cosf(angle), sa = sinf(angle);
        if (d < HALF) out[i] = __fsub_rn(__fmul_rn(base[d], ca), __fmul_rn(base[d + HALF], sa));
        else out[i] = __fadd_rn(__fmul_rn(base[d - HALF], sa), __fmul_rn(base[d], ca));
    }
}

template <int DPL, bool F32>
__device__ __forceinline__ void store_round(void* pool, size_t elem_off, float (&v)[DPL]) {
    if (F32) {
#pragma unroll
        for (int i = 0; i < DPL; i++) ((float*)pool)[elem_off + i] = v[i];
    } else {
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            __half hv = __float2half_rn(v[i]);       // cache/mod.rs:35-36
            ((__half*)pool)[elem_off + i] = hv;
            v[i] = __half2float(hv);                 // attention reads the round-tripped value (cache/mod.rs:65-77)
        }
    }
}

// One CTA per (token, head, split).  LPK lanes share a key, each holding DPL = HD / LPK dims.
template <int HD, bool F32>
__global__ void __launch_bounds__(kAttnWarps * 32)
attention_split_kernel(AttnParams p) {
    constexpr int DPL = 16 < HD / 2 ? 16 : HD / 2;
    constexpr int LPK = HD / DPL;
    constexpr int KPW = 32 / LPK;               // keys per warp per pass
    constexpr int KPI = KPW * kAttnWarps;       // keys per CTA per pass
    pdl_launch_dependents();
    pdl_wait();
    const int n_heads = p.n_heads;
    const KvLayout& kv = p.kv;
    const int tok = blockIdx.x / n_heads, h = blockIdx.x % n_heads, split = blockIdx.y;
    const int pos = p.tok_pos[tok];
    const int ctx = pos + 1;  // causal: positions 0..tok_pos (attention.rs:81-83)
    const int t_begin = split * p.chunk;
    const int t_end = min(ctx, t_begin + p.chunk);
    float* pout = p.partial + ((size_t)blockIdx.x * p.n_splits + split) * (HD + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, grp = lane / LPK, sub = lane % LPK;
    __shared__ float sm_m[kAttnWarps], sm_l[kAttnWarps];
    __shared__ float sm_acc[kAttnWarps][HD];
    __shared__ int sm_last;

    float m = -INFINITY, l = 0.f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; i++) acc[i] = 0.f;

    if (t_begin < t_end) {
        const int gsz = n_heads / kv.n_kv;
        const int kvh = h / gsz;  // attention.rs:75
        const int32_t* pt = p.page_table + (size_t)p.tok_seq[tok] * p.pages_per_seq;
        const float inv_div = sqrtf((float)HD);   // attention.rs:93: dot / sqrt(head_dim)
        const int rp = p.k_new ? p.tok_rope[tok] : 0;
        float qr[DPL];
        load_rotated<DPL, HD>(p.q + (size_t)tok * p.q_stride + h * HD, sub * DPL, rp, p.theta, qr);

        auto key_addr = [&](int t) -> size_t {
            int page = pt[t / kv.page_tokens];
            return (((size_t)page * kv.n_kv + kvh) * kv.page_tokens + t % kv.page_tokens) * HD + sub * DPL;
        };
        auto fetch = [&](int t, bool valid, float (&kr)[DPL], float (&vr)[DPL]) {
            const int tc = valid ? t : t_begin;
            if (p.k_new && valid && t == pos) {
                // the token of this step: rotate, round through the cache type, and (one head per kv group) store
                load_rotated<DPL, HD>(p.k_new + (size_t)tok * p.q_stride + kvh * HD, sub * DPL, rp, p.theta, kr);
                const float* vp = p.v_new + (size_t)tok * p.q_stride + kvh * HD + sub * DPL;
#pragma unroll
                for (int i = 0; i < DPL; i++) vr[i] = vp[i];
                if (h % gsz == 0) {
                    const size_t a = key_addr(t);
                    store_round<DPL, F32>(kv.k_pool, a, kr);
                    store_round<DPL, F32>(kv.v_pool, a, vr);
                } else if (!F32) {
#pragma unroll
                    for (int i = 0; i < DPL; i++) { kr[i] = __half2float(__float2half_rn(kr[i])); vr[i] = __half2float(__float2half_rn(vr[i])); }
                }
            } else if (p.k_new && tc == pos) {
                // a padding lane must not read the slot another CTA may be writing
#pragma unroll
                for (int i = 0; i < DPL; i++) kr[i] = vr[i] = 0.f;
            } else {
                const size_t a = key_addr(tc);
                load_slice<DPL, F32>(kv.k_pool, a, kr);
                load_slice<DPL, F32>(kv.v_pool, a, vr);
            }
        };
        auto update = [&](bool valid, const float (&kr)[DPL], const float (&vr)[DPL]) {
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < DPL; i++) dot = fmaf(qr[i], kr[i], dot);
#pragma unroll
            for (int o = 1; o < LPK; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (valid) {
                const float s = dot / inv_div;
                if (s > m) {
                    const float alpha = expf(m - s);  // exp(-inf) = 0 on the first key
                    l *= alpha;
#pragma unroll
                    for (int i = 0; i < DPL; i++) acc[i] *= alpha;
                    m = s;
                }
                const float pexp = expf(s - m);
                l += pexp;
#pragma unroll
                for (int i = 0; i < DPL; i++) acc[i] = fmaf(pexp, vr[i], acc[i]);
            }
        };

        for (int t0 = t_begin; t0 < t_end; t0 += 2 * KPI) {
            const int ta = t0 + warp * KPW + grp, tb = ta + KPI;
            const bool va = ta < t_end, vb = tb < t_end;
            float ka[DPL], vva[DPL], kb[DPL], vvb[DPL];
            fetch(ta, va, ka, vva);   // both keys' loads are in flight before the first is consumed
            fetch(tb, vb, kb, vvb);
            update(va, ka, vva);
            update(vb, kb, vvb);
        }
        // merge the key groups of the warp (lanes with equal `sub` hold the same dims), fixed order
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
            const float l2 = __shfl_xor_sync(0xffffffffu, l, o);
            const float mn = fmaxf(m, m2);
            const float a1 = (m == -INFINITY) ? 0.f : expf(m - mn);
            const float a2 = (m2 == -INFINITY) ? 0.f : expf(m2 - mn);
            l = l * a1 + l2 * a2;
#pragma unroll
            for (int i = 0; i < DPL; i++) {
                const float o2 = __shfl_xor_sync(0xffffffffu, acc[i], o);
                acc[i] = acc[i] * a1 + o2 * a2;
            }
            m = mn;
        }
    }
    // merge the warps through shared memory, in warp order
    if (grp == 0) {
        if (sub == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
        for (int i = 0; i < DPL; i++) sm_acc[warp][sub * DPL + i] = acc[i];
    }
    __syncthreads();
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; w++) mm = fmaxf(mm, sm_m[w]);
        float ll = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; w++) {
            const float sc = (sm_m[w] == -INFINITY) ? 0.f : expf(sm_m[w] - mm);
            ll += sm_l[w] * sc;
            a += sm_acc[w][d] * sc;
        }
        if (p.n_splits == 1) {
            p.out[(size_t)tok * n_heads * HD + h * HD + d] = a / ll;
        } else {
            if (d == 0) { pout[0] = mm; pout[1] = ll; }
            pout[2 + d] = a;
        }
    }
    if (p.n_splits == 1) return;
    // ---- the last split of this (token, head) to finish merges all of them, in split order ----
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(&p.counters[blockIdx.x], 1);
        sm_last = (done == p.n_splits - 1);
    }
    __syncthreads();
    if (!sm_last) return;
    __threadfence();
    const float* pp = p.partial + (size_t)blockIdx.x * p.n_splits * (HD + 2);
    float mm = -INFINITY;
    for (int s = 0; s < p.n_splits; s++) mm = fmaxf(mm, __ldcg(pp + (size_t)s * (HD + 2)));
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float ll = 0.f, a = 0.f;
        for (int s = 0; s < p.n_splits; s++) {
            const float* ps = pp + (size_t)s * (HD + 2);
            const float ms = __ldcg(ps);
            if (ms == -INFINITY) continue;  // empty split
            const float sc = expf(ms - mm);
            ll += __ldcg(ps + 1) * sc;
            a += __ldcg(ps + 2 + d) * sc;
        }
        p.out[(size_t)blockIdx.x * HD + d] = a / ll;
    }
    if (threadIdx.x == 0) p.counters[blockIdx.x] = 0;  // ready for the next launch
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

static void split_plan(int n_tok, int n_heads, int max_ctx, int* chunk, int* n_splits) {
    int want_ctas = sm_count() * 4;
    int base = n_tok * n_heads;
    int splits = (want_ctas + base - 1) / base;
    if (splits < 1) splits = 1;
    int ch = (max_ctx + splits - 1) / splits;
    ch = (ch + 63) / 64 * 64;
    *chunk = ch;
    *n_splits = (max_ctx + ch - 1) / ch;
    if (*n_splits < 1) *n_splits = 1;
}

size_t attention_scratch_bytes(int n_tok, int n_heads, int hd, int max_ctx) {
    int chunk, splits;
    split_plan(n_tok, n_heads, max_ctx, &chunk, &splits);
    if (splits == 1) return 16;
    return (size_t)n_tok * n_heads * splits * (hd + 2) * sizeof(float);
}

template <int HD>
static int32_t launch_attention_hd(const AttnParams& base, int n_tok, int max_ctx, cudaStream_t s) {
    AttnParams p = base;
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

int attention_launch_count(int n_tok, int n_heads, int max_ctx) {
    (void)n_tok; (void)n_heads; (void)max_ctx;
    return 1;
}

}  // namespace lc

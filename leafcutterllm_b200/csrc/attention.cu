// RoPE + paged KV-cache append, and causal grouped-query attention over the
// paged cache (rust/src/inference/attention.rs:13-118, rust/src/cache/mod.rs:33-77).
//
// Cache layout: per layer one K pool and one V pool, [page][kv_head][token in page][head_dim],
// f16 (the reference's storage type) or f32.  A (page, kv_head) slab is contiguous, so the
// keys a warp walks are 128-bit loads of consecutive addresses.
//
// Attention is split over the context: CTA (token, head, split) reduces its slice with an
// online softmax in fp32 and writes (max, sum, weighted V); a second kernel merges the splits
// in split order.  The reference's three-pass softmax and this one agree to rounding.
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
constexpr int kKeysPerIter = kAttnWarps * 8;  // 4 lanes per key

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

// partial layout per (token, head, split): [m, l, acc[hd]]
template <int HD, bool F32>
__global__ void __launch_bounds__(kAttnWarps * 32)
attention_split_kernel(const float* __restrict__ q, int q_stride, float* __restrict__ out, int n_heads, KvLayout kv,
                       const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos,
                       const int32_t* __restrict__ page_table, int pages_per_seq, int chunk, int n_splits,
                       float* __restrict__ partial) {
    constexpr int DPL = HD / 4;
    pdl_launch_dependents();
    pdl_wait();
    const int tok = blockIdx.x / n_heads, h = blockIdx.x % n_heads, split = blockIdx.y;
    const int ctx = tok_pos[tok] + 1;  // causal: positions 0..tok_pos (attention.rs:81-83)
    const int t_begin = split * chunk;
    const int t_end = min(ctx, t_begin + chunk);
    float* pout = partial + ((size_t)blockIdx.x * n_splits + split) * (HD + 2);
    if (t_begin >= t_end) {
        if (n_splits > 1 && threadIdx.x == 0) { pout[0] = -INFINITY; pout[1] = 0.f; }
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, grp = lane >> 2, sub = lane & 3;
    const int kvh = h / (n_heads / kv.n_kv);  // attention.rs:75
    const int32_t* pt = page_table + (size_t)tok_seq[tok] * pages_per_seq;
    const float inv_div = sqrtf((float)HD);   // attention.rs:93: dot / sqrt(head_dim)

    float qr[DPL];
    {
        const float4* qp = reinterpret_cast<const float4*>(q + (size_t)tok * q_stride + h * HD + sub * DPL);
#pragma unroll
        for (int i = 0; i < DPL / 4; i++) { float4 v = qp[i]; qr[4 * i] = v.x; qr[4 * i + 1] = v.y; qr[4 * i + 2] = v.z; qr[4 * i + 3] = v.w; }
    }
    float m = -INFINITY, l = 0.f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; i++) acc[i] = 0.f;

    for (int t0 = t_begin; t0 < t_end; t0 += kKeysPerIter) {
        int t = t0 + warp * 8 + grp;
        bool valid = t < t_end;
        int tc = valid ? t : t_begin;
        int page = pt[tc / kv.page_tokens];
        size_t base = (((size_t)page * kv.n_kv + kvh) * kv.page_tokens + tc % kv.page_tokens) * HD + sub * DPL;
        float kr[DPL], vr[DPL];
        load_slice<DPL, F32>(kv.k_pool, base, kr);
        load_slice<DPL, F32>(kv.v_pool, base, vr);
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) dot = fmaf(qr[i], kr[i], dot);
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        if (valid) {
            float s = dot / inv_div;
            if (s > m) {
                float alpha = expf(m - s);  // exp(-inf) = 0 on the first key
                l *= alpha;
#pragma unroll
                for (int i = 0; i < DPL; i++) acc[i] *= alpha;
                m = s;
            }
            float pexp = expf(s - m);
            l += pexp;
#pragma unroll
            for (int i = 0; i < DPL; i++) acc[i] = fmaf(pexp, vr[i], acc[i]);
        }
    }
    // merge the 8 key groups of the warp (lanes with equal `sub` hold the same dims)
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        float l2 = __shfl_xor_sync(0xffffffffu, l, o);
        float mn = fmaxf(m, m2);
        float a1 = (m == -INFINITY) ? 0.f : expf(m - mn);
        float a2 = (m2 == -INFINITY) ? 0.f : expf(m2 - mn);
        l = l * a1 + l2 * a2;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            float o2 = __shfl_xor_sync(0xffffffffu, acc[i], o);
            acc[i] = acc[i] * a1 + o2 * a2;
        }
        m = mn;
    }
    // merge the warps through shared memory, in warp order
    __shared__ float sm_m[kAttnWarps], sm_l[kAttnWarps];
    __shared__ float sm_acc[kAttnWarps][HD];
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
            float sc = (sm_m[w] == -INFINITY) ? 0.f : expf(sm_m[w] - mm);
            ll += sm_l[w] * sc;
            a += sm_acc[w][d] * sc;
        }
        if (n_splits == 1) {
            out[(size_t)tok * n_heads * HD + h * HD + d] = a / ll;
        } else {
            if (d == 0) { pout[0] = mm; pout[1] = ll; }
            pout[2 + d] = a;
        }
    }
}

template <int HD>
__global__ void attention_combine_kernel(const float* __restrict__ partial, int n_splits, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const float* p = partial + (size_t)blockIdx.x * n_splits * (HD + 2);
    float mm = -INFINITY;
    for (int s = 0; s < n_splits; s++) mm = fmaxf(mm, p[(size_t)s * (HD + 2)]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float ll = 0.f, a = 0.f;
        for (int s = 0; s < n_splits; s++) {
            const float* ps = p + (size_t)s * (HD + 2);
            if (ps[0] == -INFINITY) continue;  // empty split: its accumulator was never written
            float sc = expf(ps[0] - mm);
            ll += ps[1] * sc;
            a += ps[2 + d] * sc;
        }
        out[(size_t)blockIdx.x * HD + d] = a / ll;
    }
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
    ch = (ch + kKeysPerIter - 1) / kKeysPerIter * kKeysPerIter;
    if (ch < 64) ch = 64;
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
static int32_t launch_attention_hd(const float* q, int q_stride, float* out, int n_tok, int n_heads, const KvLayout& kv,
                                   const int32_t* tok_seq, const int32_t* tok_pos, const int32_t* page_table, int pages_per_seq,
                                   int max_ctx, void* scratch, cudaStream_t s) {
    int chunk, splits;
    split_plan(n_tok, n_heads, max_ctx, &chunk, &splits);
    dim3 grid((unsigned)(n_tok * n_heads), (unsigned)splits);
    if (kv.kv_f32)
        LC_CUDA(launch_k(attention_split_kernel<HD, true>, grid, dim3(kAttnWarps * 32), s, q, q_stride, out, n_heads, kv, tok_seq,
                         tok_pos, page_table, pages_per_seq, chunk, splits, (float*)scratch));
    else
        LC_CUDA(launch_k(attention_split_kernel<HD, false>, grid, dim3(kAttnWarps * 32), s, q, q_stride, out, n_heads, kv, tok_seq,
                         tok_pos, page_table, pages_per_seq, chunk, splits, (float*)scratch));
    if (splits > 1)
        LC_CUDA(launch_k(attention_combine_kernel<HD>, dim3((unsigned)(n_tok * n_heads)), dim3(HD < 128 ? HD : 128), s,
                         (const float*)scratch, splits, out));
    return LC_OK;
}

int32_t launch_attention(const float* q, int q_stride, float* out, int n_tok, int n_heads, const KvLayout& kv,
                         const int32_t* tok_seq, const int32_t* tok_pos, const int32_t* page_table, int pages_per_seq, int max_ctx,
                         void* scratch, cudaStream_t s) {
    if (n_tok <= 0) return LC_OK;
    switch (kv.hd) {
        case 32: return launch_attention_hd<32>(q, q_stride, out, n_tok, n_heads, kv, tok_seq, tok_pos, page_table, pages_per_seq, max_ctx, scratch, s);
        case 64: return launch_attention_hd<64>(q, q_stride, out, n_tok, n_heads, kv, tok_seq, tok_pos, page_table, pages_per_seq, max_ctx, scratch, s);
        case 128: return launch_attention_hd<128>(q, q_stride, out, n_tok, n_heads, kv, tok_seq, tok_pos, page_table, pages_per_seq, max_ctx, scratch, s);
        case 256: return launch_attention_hd<256>(q, q_stride, out, n_tok, n_heads, kv, tok_seq, tok_pos, page_table, pages_per_seq, max_ctx, scratch, s);
        default:
            set_error("attention: head_dim %d is not one of 32, 64, 128, 256", kv.hd);
            return LC_ERR_UNSUPPORTED;
    }
}

int attention_launch_count(int n_tok, int n_heads, int max_ctx) {
    int chunk, splits;
    split_plan(n_tok, n_heads, max_ctx, &chunk, &splits);
    return splits > 1 ? 2 : 1;
}

}  // namespace lc

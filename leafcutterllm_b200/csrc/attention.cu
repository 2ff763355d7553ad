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
#include "lc_mega.h"

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

void attention_plan(int n_tok, int n_heads, int max_ctx, int* chunk, int* n_splits) { split_plan(n_tok, n_heads, max_ctx, chunk, n_splits); }

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
// holds these 512 KiB until the process exits.
constexpr size_t kStaticAttnScratchBytes = (size_t)512 << 10;
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

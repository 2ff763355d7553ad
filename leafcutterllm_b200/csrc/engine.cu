// Model level of the C ABI: a Llama-family decoder over GGUF-quantised weights
// resident in HBM, with a paged KV cache.  Mirrors Engine / ShardEngine / KVCache
// of the reference (rust/src/inference/engine.rs, shard_engine.rs, rust/src/cache/mod.rs):
// the per-token re-dequantisation and layer streaming of engine.rs:95-97 give way
// to weights uploaded once in raw block form.
//
// One forward over T new tokens queues, per layer:
//   qgemv(Wqkv, rmsnorm fused)  -> rope + KV append -> attention (+ split merge)
//   -> qgemv(Wo, + residual) -> qgemv(Wgate|Wup, rmsnorm fused, SiLU*up) -> qgemv(Wdown, + residual)
// and at the end qgemv(head, final rmsnorm fused) on each sequence's last token and the
// greedy pick.  The single-token step of a decode loop is captured in a CUDA graph.
#include <algorithm>
#include <cstring>
#include <map>
#include <string>
#include <vector>
#include "lc_kernels.h"
#include "lc_synth.h"
#include "lc_tma.cuh"

using namespace lc;

namespace {

struct DevTensor {
    uint32_t typ = 0;
    std::vector<uint64_t> dims;
    void* dev = nullptr;   // owning pointer (null when the bytes live inside a fused buffer)
    void* view = nullptr;  // where the bytes are
    size_t nbytes = 0;
    size_t rows = 0, cols = 0;
};

struct LayerW {
    QWeight qkv, o, gate, up, down;
    QWeight q, k, v;  // used when the three cannot be fused
    bool fused_qkv = false;
    const float* attn_norm = nullptr;
    const float* ffn_norm = nullptr;
    void* fused_buf = nullptr;
    // mixture-of-experts FFN (no counterpart in the reference): f32 router [n_experts, H], the experts' three matrices,
    // and -- when every expert is Q4_K with a tensor map -- device arrays of those maps for the one-launch grouped product
    const float* router = nullptr;
    std::vector<QWeight> egate, eup, edown;
    void *tm_gate = nullptr, *tm_up = nullptr, *tm_down = nullptr;
    bool grouped_ok = false;
};

constexpr int kPrefillChunk = 512;
constexpr int kTokTile = 8;
constexpr int kMoeGroupedTokens = 64;  // calls of at most this many tokens run the experts as one grouped launch

}  // namespace

struct lc_model {
    lc_model_config cfg{};
    int device = 0;
    cudaStream_t stream = nullptr;
    std::map<std::string, DevTensor> tensors;
    bool finalized = false;
    std::vector<LayerW> layers;
    QWeight head;
    const DevTensor* embed = nullptr;
    const float* final_norm = nullptr;
    std::vector<void*> owned;  // f32 copies of norm gains etc.

    // geometry
    int H = 0, L = 0, nh = 0, nkv = 0, hd = 0, F = 0, V = 0, nqkv = 0;
    int page_tokens = 16, pages_per_seq = 0, pages_total = 0, max_seqs = 1, t_cap = 0;
    size_t kv_elt = 2;

    // KV cache
    std::vector<void*> k_pools, v_pools;  // per layer
    struct alignas(64) TmapBytes { unsigned char b[128]; };
    std::vector<TmapBytes> k_tmaps, v_tmaps;  // per layer: tensor maps over the key and value pools (f16 pools of 128-dim heads)
    bool k_tmaps_ok = false;
    std::vector<int> free_pages;
    std::vector<std::vector<int>> seq_pages;
    std::vector<int> seq_len;
    int32_t* d_page_table = nullptr;
    std::vector<int32_t> h_page_table;
    bool page_table_dirty = true;

    // step buffers
    int64_t* d_tokens = nullptr;
    int32_t *d_tok_seq = nullptr, *d_tok_pos = nullptr, *d_tok_rope = nullptr, *d_last_idx = nullptr;
    float *d_hidden = nullptr, *d_hidden2 = nullptr, *d_qkv = nullptr, *d_attn = nullptr, *d_ffn = nullptr;
    float *d_last = nullptr, *d_logits = nullptr;
    bool seeded = false;          // lc_model_set_seed: stochastic sampling allowed, draws from seeded_uniform(seed, draws++)
    uint64_t seed = 0, draws = 0;
    int64_t* d_next = nullptr;
    int64_t* d_out_tokens = nullptr;
    size_t out_tokens_cap = 0;
    int32_t* d_step_ctr = nullptr;
    unsigned long long* d_stream_slots = nullptr;  // cross-CTA merge slots of the single-token attention kernel (zero between launches)
    // mixture-of-experts scratch: the router's picks and weights per token, per-expert slot counts and lists, the slots'
    // FFN hidden rows and outputs (calls of up to kMoeGroupedTokens tokens), every expert's output plane (larger calls)
    int32_t *d_moe_sel = nullptr, *d_moe_cnt = nullptr, *d_moe_lists = nullptr;
    float *d_moe_w = nullptr, *d_moe_h = nullptr, *d_moe_y = nullptr, *d_moe_yall = nullptr;
    unsigned long long* d_moe_touched = nullptr;  // experts that received a token, summed over layers and steps since the last read
    uint64_t expert_bytes_each = 0, expert_bytes_all = 0;
    double touched_per_step = 0.0;
    void* d_attn_scratch = nullptr;
    GemmWorkspace gemm_ws;  // f16 activation halves for the many-token tensor-core product
    bool any_unfused_qkv = false;  // some layer's q/k/v differ in type
    float* d_qkv_parts = nullptr;  // then: [T][nq] | [T][nkv hd] | [T][nkv hd] before they are interleaved into d_qkv
    int* d_attn_counters = nullptr;
    size_t attn_scratch_bytes = 0;
    unsigned long long* d_sanity = nullptr;

    std::map<int, cudaGraphExec_t> decode_graphs;
    int graph_nodes = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;

    lc_counters ctr{};
    uint64_t launches_in_call = 0;

    // What the device-side per-token metadata currently describes (a decode step for these sequences at
    // these cache positions), so that consecutive one-token calls only have to send the token ids.
    bool meta_valid = false;
    std::vector<int> meta_seqs, meta_pos;
    // pinned staging for the per-step host <-> device traffic
    int64_t* pin_tokens = nullptr;
    int64_t* pin_next = nullptr;
    float* pin_logits = nullptr;
};

namespace {

// rust/src/model/arch.rs:83-96 and rust/src/model/loader.rs:173-177: engine name -> GGUF name.
std::string canonical_name(const std::string& in) {
    static const std::pair<const char*, const char*> special[] = {{"model.embed_tokens.weight", "token_embd.weight"},
                                                                 {"model.norm.weight", "output_norm.weight"},
                                                                 {"lm_head.weight", "output.weight"}};
    for (auto& p : special)
        if (in == p.first) return p.second;
    static const std::pair<const char*, const char*> layer[] = {
        {"self_attn.q_proj.weight", "attn_q.weight"},   {"self_attn.k_proj.weight", "attn_k.weight"},
        {"self_attn.v_proj.weight", "attn_v.weight"},   {"self_attn.o_proj.weight", "attn_output.weight"},
        {"mlp.gate_proj.weight", "ffn_gate.weight"},    {"mlp.up_proj.weight", "ffn_up.weight"},
        {"mlp.down_proj.weight", "ffn_down.weight"},    {"input_layernorm.weight", "attn_norm.weight"},
        {"post_attention_layernorm.weight", "ffn_norm.weight"}};
    if (in.rfind("blk.", 0) == 0) {
        size_t dot = in.find('.', 4);
        if (dot != std::string::npos) {
            std::string suffix = in.substr(dot + 1);
            for (auto& p : layer)
                if (suffix == p.first) return in.substr(0, dot + 1) + p.second;
        }
    }
    return in;
}

struct DeviceGuard {
    int prev = 0;
    bool ok = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) ok = true;
    }
    ~DeviceGuard() { if (ok) cudaSetDevice(prev); }
};

template <typename T>
int32_t dalloc(T** p, size_t count) {
    void* q = nullptr;
    cudaError_t e = cudaMalloc(&q, std::max<size_t>(count * sizeof(T), 16));
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("device allocation of %zu bytes failed: %s", count * sizeof(T), cudaGetErrorString(e));
        return LC_ERR_OOM;
    }
    *p = (T*)q;
    return LC_OK;
}

__global__ void gather_rows_kernel(const float* __restrict__ src, const int32_t* __restrict__ idx, int cols, float* __restrict__ dst) {
    pdl_launch_dependents();
    pdl_wait();
    const float* s = src + (size_t)idx[blockIdx.x] * cols;
    float* d = dst + (size_t)blockIdx.x * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) d[c] = s[c];
}

// After a greedy step: next token becomes the input of each sequence, cache positions advance,
// the token is logged.  rope_absolute: rotary position follows the cache position; otherwise it
// stays the index inside the call (0 for a one-token call, attention.rs:13-21).
__global__ void advance_kernel(const int64_t* __restrict__ next, int64_t* tokens, int32_t* tok_pos, int32_t* tok_rope, int n,
                               int rope_absolute, int64_t* out_tokens, int32_t* step_ctr) {
    pdl_launch_dependents();
    pdl_wait();
    int i = threadIdx.x;
    int step = *step_ctr;
    if (i < n) {
        tokens[i] = next[i];
        tok_pos[i] += 1;
        if (rope_absolute) tok_rope[i] = tok_pos[i];
        if (out_tokens) out_tokens[(size_t)step * n + i] = next[i];
    }
    __syncthreads();
    if (i == 0) *step_ctr = step + 1;
}

int32_t check_model(const lc_model* m, bool need_final) {
    LC_CHECK(m != nullptr, LC_ERR_INVALID, "null model handle");
    if (need_final) LC_CHECK(m->finalized, LC_ERR_STATE, "model is not finalized");
    return LC_OK;
}

int32_t ensure_pages(lc_model* m, int seq, int new_len) {
    LC_CHECK(new_len <= m->cfg.max_seq_len, LC_ERR_KV_FULL, "sequence %d would hold %d tokens, capacity is %d", seq, new_len,
             m->cfg.max_seq_len);
    int need = (new_len + m->page_tokens - 1) / m->page_tokens;
    auto& pg = m->seq_pages[seq];
    while ((int)pg.size() < need) {
        LC_CHECK(!m->free_pages.empty(), LC_ERR_KV_FULL, "KV pool exhausted (%d pages)", m->pages_total);
        int p = m->free_pages.back();
        m->free_pages.pop_back();
        m->h_page_table[(size_t)seq * m->pages_per_seq + pg.size()] = p;
        pg.push_back(p);
        m->page_table_dirty = true;
    }
    return LC_OK;
}

int32_t sync_page_table(lc_model* m) {
    if (!m->page_table_dirty) return LC_OK;
    LC_CUDA(cudaMemcpyAsync(m->d_page_table, m->h_page_table.data(), m->h_page_table.size() * 4, cudaMemcpyHostToDevice, m->stream));
    m->page_table_dirty = false;
    return LC_OK;
}

KvLayout kv_layout(const lc_model* m, int layer) {
    KvLayout kv;
    kv.k_pool = m->k_pools[layer];
    kv.v_pool = m->v_pools[layer];
    kv.n_kv = m->nkv;
    kv.hd = m->hd;
    kv.page_tokens = m->page_tokens;
    kv.kv_f32 = m->cfg.kv_dtype;
    kv.pool_pages = m->pages_total;
    kv.k_tmap = m->k_tmaps_ok ? (const void*)m->k_tmaps[layer].b : nullptr;
    kv.v_tmap = m->k_tmaps_ok ? (const void*)m->v_tmaps[layer].b : nullptr;
    return kv;
}

int32_t gemv_tiled(lc_model* m, GemvArgs a, int T, int n_out, int k_in) {
    if (qgemm_applies(a, T, m->gemm_ws)) {
        // five tokens and more: one pass over the weights on the tcgen05 tensor cores (activation split + product)
        a.m = T;
        int launches = 0;
        LC_TRY(launch_qgemm(a, m->gemm_ws, m->stream, &launches));
        m->launches_in_call += launches;
        return LC_OK;
    }
    for (int t0 = 0; t0 < T; t0 += kTokTile) {
        GemvArgs g = a;
        g.m = std::min(kTokTile, T - t0);
        g.x = a.x + (size_t)t0 * k_in;
        g.out = a.out + (size_t)t0 * n_out;
        if (a.residual) g.residual = a.residual + (size_t)t0 * n_out;
        LC_TRY(launch_qgemv(g, m->stream));
        m->launches_in_call += 1;
    }
    return LC_OK;
}

// attention_forward (attention.rs:37-118) for layer `l` on T tokens whose (normalised or raw) input is `x`.
int32_t attention_block(lc_model* m, int l, const float* x, const float* norm_w, int T, const float* residual, float* out,
                        bool decode_step) {
    LayerW& w = m->layers[l];
    GemvArgs g;
    g.x = x;
    g.norm_w = norm_w;
    g.eps = m->cfg.rms_eps;
    if (w.fused_qkv) {
        g.w = &w.qkv;
        g.out = m->d_qkv;
        // the fused output is [T, nqkv] only when every token tile writes rows of nqkv floats
        LC_TRY(gemv_tiled(m, g, T, m->nqkv, m->H));
    } else {
        // q/k/v of different types: three products.  One token writes straight into its row of d_qkv; several tokens go
        // through contiguous parts and are interleaved into the [T][nq + 2 nkv hd] rows the attention kernels expect.
        const int nq = m->nh * m->hd, nkvd = m->nkv * m->hd;
        const QWeight* ws3[3] = {&w.q, &w.k, &w.v};
        const int ns[3] = {nq, nkvd, nkvd};
        size_t part_off = 0, col_off = 0;
        for (int i = 0; i < 3; i++) {
            g.w = ws3[i];
            g.out = T == 1 ? m->d_qkv + col_off : m->d_qkv_parts + part_off;
            LC_TRY(gemv_tiled(m, g, T, ns[i], m->H));
            if (T > 1) {
                LC_CUDA(cudaMemcpy2DAsync(m->d_qkv + col_off, (size_t)m->nqkv * 4, g.out, (size_t)ns[i] * 4, (size_t)ns[i] * 4, (size_t)T,
                                          cudaMemcpyDeviceToDevice, m->stream));
                m->launches_in_call += 1;
            }
            part_off += (size_t)T * ns[i];
            col_off += ns[i];
        }
    }
    KvLayout kv = kv_layout(m, l);
    float* q = m->d_qkv;
    float* k = m->d_qkv + (size_t)m->nh * m->hd;
    float* v = k + (size_t)m->nkv * m->hd;
    if (decode_step) {
        // one new token per sequence: rotation and the cache append ride inside the attention kernel
        AttnFusion fz{k, v, m->d_tok_rope, m->cfg.rope_theta};
        fz.positions_settled = l > 0;  // the first layer of a step may run while the previous step still advances the positions
        fz.stream_slots = m->d_stream_slots;
        LC_TRY(launch_attention(q, m->nqkv, m->d_attn, T, m->nh, kv, m->d_tok_seq, m->d_tok_pos, m->d_page_table, m->pages_per_seq,
                                m->cfg.max_seq_len, m->d_attn_scratch, m->d_attn_counters, &fz, m->stream));
        m->launches_in_call += 1;
    } else {
        LC_TRY(launch_rope_kv_append(q, k, v, m->nqkv, T, m->nh, kv, m->d_tok_seq, m->d_tok_pos, m->d_tok_rope, m->d_page_table,
                                     m->pages_per_seq, m->cfg.rope_theta, m->stream));
        LC_TRY(launch_attention(q, m->nqkv, m->d_attn, T, m->nh, kv, m->d_tok_seq, m->d_tok_pos, m->d_page_table, m->pages_per_seq,
                                m->cfg.max_seq_len, m->d_attn_scratch, m->d_attn_counters, nullptr, m->stream));
        m->launches_in_call += 2;
    }
    GemvArgs o;
    o.w = &w.o;
    o.x = m->d_attn;
    o.out = out;
    if (residual) { o.residual = residual; o.epi = EPI_ADD_RESIDUAL; }
    if (residual && out == m->d_hidden2 && w.ffn_norm) {  // in a layer of the forward pass the FFN reads `out` next, through its norm
        o.prep_next = true; o.next_norm_w = w.ffn_norm; o.next_eps = m->cfg.rms_eps;
    }
    return gemv_tiled(m, o, T, m->H, m->nh * m->hd);
}

// Mixture-of-experts FFN in place of ffn_forward (moe.cu has the definition): router, then either ONE grouped launch per
// projection over the experts that received tokens (Q4_K experts, calls of up to 64 tokens), or every expert on every
// token through the ordinary products (prefill chunks, other quant types), then the weighted sum of the chosen experts.
int32_t moe_block(lc_model* m, int l, const float* x, const float* norm_w, int T, const float* residual, float* out) {
    LayerW& w = m->layers[l];
    const int E = m->cfg.n_experts, K = m->cfg.top_k;
    const bool grouped = w.grouped_ok && T <= kMoeGroupedTokens;
    MoeRouteArgs r;
    r.x = x; r.norm_w = norm_w; r.eps = m->cfg.rms_eps; r.H = m->H; r.T = T; r.w_router = w.router; r.n_experts = E; r.top_k = K;
    r.sel = m->d_moe_sel; r.wsel = m->d_moe_w;
    if (grouped) { r.counts = m->d_moe_cnt; r.lists = m->d_moe_lists; r.list_stride = kMoeGroupedTokens; r.touched = m->d_moe_touched; }
    LC_TRY(launch_moe_route(r, m->stream));
    m->launches_in_call += 1;
    if (grouped) {
        GemvGroup g1;
        g1.tmaps = w.tm_gate; g1.tmaps2 = w.tm_up; g1.counts = m->d_moe_cnt; g1.lists = m->d_moe_lists; g1.list_stride = kMoeGroupedTokens;
        g1.n_experts = E; g1.top_k = K; g1.max_tokens = T; g1.x_by_token = true;
        GemvArgs a;
        a.w = &w.egate[0]; a.w2 = &w.eup[0]; a.x = x; a.norm_w = norm_w; a.eps = m->cfg.rms_eps; a.out = m->d_moe_h; a.epi = EPI_SILU_MUL;
        a.m = std::min(T, kTokTile); a.group = &g1;
        LC_TRY(launch_qgemv(a, m->stream));
        GemvGroup g2 = g1;
        g2.tmaps = w.tm_down; g2.tmaps2 = nullptr; g2.x_by_token = false;
        GemvArgs d;
        d.w = &w.edown[0]; d.x = m->d_moe_h; d.out = m->d_moe_y; d.m = std::min(T, kTokTile); d.group = &g2;
        LC_TRY(launch_qgemv(d, m->stream));
        LC_TRY(launch_moe_combine(m->d_moe_y, m->d_moe_sel, m->d_moe_w, K, m->H, T, 0, 0, residual, out, m->stream));
        m->launches_in_call += 3;
        return LC_OK;
    }
    for (int e = 0; e < E; e++) {
        GemvArgs g;
        g.w = &w.egate[e]; g.w2 = &w.eup[e]; g.x = x; g.norm_w = norm_w; g.eps = m->cfg.rms_eps; g.out = m->d_ffn; g.epi = EPI_SILU_MUL;
        g.prep_next = true;  // the expert's down projection reads d_ffn next, without a norm
        LC_TRY(gemv_tiled(m, g, T, m->F, m->H));
        GemvArgs d;
        d.w = &w.edown[e]; d.x = m->d_ffn; d.out = m->d_moe_yall + (size_t)e * m->t_cap * m->H;
        LC_TRY(gemv_tiled(m, d, T, m->H, m->F));
    }
    LC_TRY(launch_moe_combine(m->d_moe_yall, m->d_moe_sel, m->d_moe_w, K, m->H, T, 1, (size_t)m->t_cap, residual, out, m->stream));
    m->launches_in_call += 1;
    return LC_OK;
}

// ffn_forward (engine.rs:146-164)
int32_t ffn_block(lc_model* m, int l, const float* x, const float* norm_w, int T, const float* residual, float* out,
                  bool decode_step) {
    if (m->cfg.n_experts > 0) return moe_block(m, l, x, norm_w, T, residual, out);
    LayerW& w = m->layers[l];
    GemvArgs g;
    g.w = &w.gate;
    g.w2 = &w.up;
    g.x = x;
    g.norm_w = norm_w;
    g.eps = m->cfg.rms_eps;
    g.out = m->d_ffn;
    g.epi = EPI_SILU_MUL;
    g.prep_next = true;  // the down projection reads d_ffn next, without a norm
    g.next_norm_w = nullptr;
    LC_TRY(gemv_tiled(m, g, T, m->F, m->H));
    GemvArgs d;
    d.w = &w.down;
    d.x = m->d_ffn;
    d.out = out;
    if (residual) { d.residual = residual; d.epi = EPI_ADD_RESIDUAL; }
    if (residual && out == m->d_hidden && l + 1 < m->L && m->layers[l + 1].attn_norm) {
        // the next layer's q/k/v product(s) read `out` through that layer's attention norm
        d.prep_next = true; d.next_norm_w = m->layers[l + 1].attn_norm; d.next_eps = m->cfg.rms_eps;
    }
    return gemv_tiled(m, d, T, m->H, m->F);
}

// The transformer layers (engine.rs:95-116) on T tokens described by d_tokens / d_tok_*.
int32_t run_layers(lc_model* m, int T, bool decode_step) {
    LC_TRY(launch_embed(m->embed->typ, m->embed->view, m->embed->rows, m->embed->cols, m->d_tokens, T, m->d_hidden, m->stream));
    m->launches_in_call += 1;
    for (int l = 0; l < m->L; l++) {
        LayerW& w = m->layers[l];
        LC_TRY(attention_block(m, l, m->d_hidden, w.attn_norm, T, m->d_hidden, m->d_hidden2, decode_step));
        LC_TRY(ffn_block(m, l, m->d_hidden2, w.ffn_norm, T, m->d_hidden2, m->d_hidden, decode_step));
    }
    return LC_OK;
}

// Engine::forward (engine.rs:78-132): layers, then final norm + head on n_last rows.  identity_last:
// every token is the last of its sequence (a decode step), so no gather is needed; otherwise the rows
// listed in d_last_idx are gathered.  Logits land in d_logits rows row0.., greedy picks in d_next.
int32_t forward_tokens(lc_model* m, int T, int n_last, bool identity_last, int row0) {
    LC_TRY(run_layers(m, T, identity_last));
    const float* last = m->d_hidden;
    if (!identity_last) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(n_last);
        cfg.blockDim = dim3(256);
        cfg.stream = m->stream;
        LC_CUDA(cudaLaunchKernelEx(&cfg, gather_rows_kernel, (const float*)m->d_hidden, (const int32_t*)m->d_last_idx, m->H, m->d_last));
        m->launches_in_call += 1;
        last = m->d_last;
    }
    GemvArgs h;
    h.w = &m->head;
    h.x = last;
    h.norm_w = m->final_norm;
    h.eps = m->cfg.rms_eps;
    h.out = m->d_logits + (size_t)row0 * m->V;
    LC_TRY(gemv_tiled(m, h, n_last, m->V, m->H));
    LC_TRY(launch_argmax(m->d_logits + (size_t)row0 * m->V, m->V, n_last, m->d_next + row0, m->stream));
    m->launches_in_call += 1;
    return LC_OK;
}

uint64_t algo_bytes_step(const lc_model* m, const std::vector<int>& ctx_lens) {
    uint64_t b = m->ctr.weight_bytes;  // every matrix and gain once
    if (m->cfg.n_experts > 0)          // ... but only the experts that received a token (average per layer of the last steps)
        b = b - m->expert_bytes_all + (uint64_t)(m->touched_per_step * (double)m->expert_bytes_each);
    // the embedding table is not streamed: one row per token instead
    if (m->embed) {
        bool tied = m->tensors.find("output.weight") == m->tensors.end();
        if (!tied) b -= m->embed->nbytes;
        b += (uint64_t)ctx_lens.size() * (m->embed->nbytes / std::max<size_t>(m->embed->rows, 1));
    }
    uint64_t per_tok = (uint64_t)m->L * 2 * m->nkv * m->hd * m->kv_elt;
    for (int c : ctx_lens) b += per_tok * (uint64_t)c + per_tok;  // read the context, write one token
    return b;
}

// Upload per-token metadata for a call of T tokens.
int32_t upload_meta(lc_model* m, const std::vector<int64_t>& tok, const std::vector<int32_t>& seq, const std::vector<int32_t>& pos,
                    const std::vector<int32_t>& rope, const std::vector<int32_t>& last) {
    size_t T = tok.size();
    LC_CUDA(cudaMemcpyAsync(m->d_tokens, tok.data(), T * 8, cudaMemcpyHostToDevice, m->stream));
    LC_CUDA(cudaMemcpyAsync(m->d_tok_seq, seq.data(), T * 4, cudaMemcpyHostToDevice, m->stream));
    LC_CUDA(cudaMemcpyAsync(m->d_tok_pos, pos.data(), T * 4, cudaMemcpyHostToDevice, m->stream));
    LC_CUDA(cudaMemcpyAsync(m->d_tok_rope, rope.data(), T * 4, cudaMemcpyHostToDevice, m->stream));
    if (!last.empty()) LC_CUDA(cudaMemcpyAsync(m->d_last_idx, last.data(), last.size() * 4, cudaMemcpyHostToDevice, m->stream));
    // the copies read pageable host vectors that die with the caller's frame
    LC_CUDA(cudaStreamSynchronize(m->stream));
    return LC_OK;
}

void finish_call(lc_model* m) {
    m->ctr.kernel_launches += m->launches_in_call;
    m->launches_in_call = 0;
}

}  // namespace

// A bounded wait inside a kernel ran out (TMA transaction or grid barrier): report instead of returning wrong tokens.
static int32_t check_device_flag(lc_model* m) {
    int* f = gemv_error_flag_dev();
    if (!f) return LC_OK;
    int v = 0;
    LC_CUDA(cudaMemcpyAsync(&v, f, sizeof(int), cudaMemcpyDeviceToHost, m->stream));
    LC_CUDA(cudaStreamSynchronize(m->stream));
    if (v != 0) {
        cudaMemsetAsync(f, 0, sizeof(int), m->stream);
        set_error("a device-side check failed (code %d: %s); the results of this call are not valid", v,
                  v >= 20 ? "an index outside its range" : "a bounded wait ran out");
        return LC_ERR_CUDA;
    }
    return LC_OK;
}

extern "C" {

static int32_t run_decode_steps(lc_model* m, int n_seqs, int steps);
static int32_t reserve_out_tokens(lc_model* m, size_t need);
static int32_t stage_decode_meta(lc_model* m, int n_seqs, const int32_t* seq_ids, const int64_t* toks);
static void after_decode_steps(lc_model* m, int n_seqs, const int32_t* seq_ids, int steps);

int32_t lc_model_create(const lc_model_config* cfg, lc_model** out) {
    LC_CHECK(cfg && out, LC_ERR_INVALID, "lc_model_create: null argument");
    LC_CHECK(cfg->hidden_size > 0 && cfg->num_layers > 0 && cfg->num_heads > 0 && cfg->num_kv_heads > 0 &&
                 cfg->intermediate_size > 0 && cfg->vocab_size > 0 && cfg->max_seq_len > 0,
             LC_ERR_INVALID, "lc_model_create: non-positive dimension");
    LC_CHECK(cfg->hidden_size % cfg->num_heads == 0, LC_ERR_INVALID, "hidden_size %d is not a multiple of num_heads %d",
             cfg->hidden_size, cfg->num_heads);
    LC_CHECK(cfg->num_heads % cfg->num_kv_heads == 0, LC_ERR_INVALID, "num_heads %d is not a multiple of num_kv_heads %d",
             cfg->num_heads, cfg->num_kv_heads);
    LC_CHECK(cfg->n_experts >= 0 && cfg->n_experts <= kMaxExperts, LC_ERR_INVALID, "n_experts %d outside 0..%d", cfg->n_experts, kMaxExperts);
    if (cfg->n_experts > 0)
        LC_CHECK(cfg->top_k >= 1 && cfg->top_k <= kMaxTopK && cfg->top_k <= cfg->n_experts, LC_ERR_INVALID,
                 "top_k %d outside 1..min(%d, n_experts = %d)", cfg->top_k, kMaxTopK, cfg->n_experts);
    if (!have_device()) return LC_ERR_CUDA;
    LC_CHECK(cfg->device >= 0 && cfg->device < lc_device_count(), LC_ERR_INVALID, "device %d not present", cfg->device);
    DeviceGuard dg(cfg->device);
    lc_model* m = new lc_model();
    m->cfg = *cfg;
    if (m->cfg.rms_eps == 0.0f) m->cfg.rms_eps = 1e-5f;
    if (m->cfg.max_seqs <= 0) m->cfg.max_seqs = 1;
    if (m->cfg.kv_page_tokens <= 0) m->cfg.kv_page_tokens = 16;
    m->device = cfg->device;
    m->H = cfg->hidden_size; m->L = cfg->num_layers; m->nh = cfg->num_heads; m->nkv = cfg->num_kv_heads;
    m->hd = m->H / m->nh; m->F = cfg->intermediate_size; m->V = cfg->vocab_size;
    m->nqkv = (m->nh + 2 * m->nkv) * m->hd;
    m->page_tokens = m->cfg.kv_page_tokens;
    m->max_seqs = m->cfg.max_seqs;
    m->pages_per_seq = (m->cfg.max_seq_len + m->page_tokens - 1) / m->page_tokens;
    int64_t pool = m->cfg.kv_pool_tokens > 0 ? m->cfg.kv_pool_tokens : (int64_t)m->max_seqs * m->pages_per_seq * m->page_tokens;
    m->pages_total = (int)((pool + m->page_tokens - 1) / m->page_tokens);
    m->kv_elt = m->cfg.kv_dtype ? 4 : 2;
    m->t_cap = std::max(kPrefillChunk, m->max_seqs);
    m->stream = lc::stream();
    if (!m->stream) { delete m; set_error("could not create a CUDA stream"); return LC_ERR_CUDA; }
    *out = m;
    return LC_OK;
}

static int32_t put_tensor(lc_model* m, const char* name, uint32_t typ, const uint64_t* dims, int32_t ndims, DevTensor** out_t) {
    LC_TRY(check_model(m, false));
    LC_CHECK(!m->finalized, LC_ERR_STATE, "model already finalized");
    LC_CHECK(name && dims && ndims >= 1 && ndims <= 4, LC_ERR_INVALID, "set_tensor: bad argument");
    QuantGeom g;
    LC_CHECK(quant_geom(typ, &g), LC_ERR_UNSUPPORTED, "tensor %s: unsupported ggml type %u", name, typ);
    size_t count = 1;
    for (int i = 0; i < ndims; i++) count *= dims[i];
    LC_CHECK(dims[0] % g.block_elems == 0, LC_ERR_INVALID, "tensor %s: row length %llu is not a whole number of blocks", name,
             (unsigned long long)dims[0]);
    std::string key = canonical_name(name);
    DevTensor t;
    t.typ = typ;
    t.dims.assign(dims, dims + ndims);
    t.nbytes = lc_tensor_bytes(typ, count);
    t.cols = dims[0];  // loader.rs:155: GGUF dims are fastest-first, rows = dims[1]
    t.rows = ndims >= 2 ? count / dims[0] : 1;
    auto it = m->tensors.find(key);
    if (it != m->tensors.end() && it->second.dev) cudaFree(it->second.dev);
    LC_TRY(dalloc((uint8_t**)&t.dev, t.nbytes));
    t.view = t.dev;
    m->tensors[key] = t;
    *out_t = &m->tensors[key];
    return LC_OK;
}

int32_t lc_model_set_tensor(lc_model* m, const char* name, uint32_t typ, const uint64_t* dims, int32_t ndims, const void* bytes,
                            size_t nbytes) {
    LC_TRY(check_model(m, false));
    DeviceGuard dg(m->device);
    LC_CHECK(bytes, LC_ERR_INVALID, "set_tensor: null bytes");
    DevTensor* t = nullptr;
    LC_TRY(put_tensor(m, name, typ, dims, ndims, &t));
    LC_CHECK(t->nbytes == nbytes, LC_ERR_INVALID, "tensor %s: %zu bytes given, %zu expected", name, nbytes, t->nbytes);
    LC_CUDA(cudaMemcpyAsync(t->dev, bytes, nbytes, cudaMemcpyHostToDevice, m->stream));
    LC_CUDA(cudaStreamSynchronize(m->stream));
    return LC_OK;
}

int32_t lc_model_synth_tensor(lc_model* m, const char* name, uint32_t typ, const uint64_t* dims, int32_t ndims, uint64_t seed,
                              float sigma) {
    LC_TRY(check_model(m, false));
    DeviceGuard dg(m->device);
    DevTensor* t = nullptr;
    LC_TRY(put_tensor(m, name, typ, dims, ndims, &t));
    size_t count = 1;
    for (int i = 0; i < ndims; i++) count *= dims[i];
    std::string key = canonical_name(name);
    LC_TRY(launch_synth(typ, seed, lcs_fnv1a(key.c_str()), sigma, count, t->dev, m->stream));
    LC_CUDA(cudaStreamSynchronize(m->stream));
    return LC_OK;
}

int32_t lc_model_get_tensor(lc_model* m, const char* name, void* out_bytes, size_t nbytes) {
    LC_TRY(check_model(m, false));
    DeviceGuard dg(m->device);
    LC_CHECK(name && out_bytes, LC_ERR_INVALID, "get_tensor: null argument");
    auto it = m->tensors.find(canonical_name(name));
    LC_CHECK(it != m->tensors.end(), LC_ERR_MISSING, "tensor %s was never set", name);
    LC_CHECK(it->second.nbytes == nbytes, LC_ERR_INVALID, "tensor %s holds %zu bytes, %zu requested", name, it->second.nbytes, nbytes);
    LC_CUDA(cudaMemcpyAsync(out_bytes, it->second.view, nbytes, cudaMemcpyDeviceToHost, m->stream));
    LC_CUDA(cudaStreamSynchronize(m->stream));
    return LC_OK;
}

// A gain vector as f32 on the device (norm weights are F32 in GGUF files; F16 is widened).
static int32_t gain_f32(lc_model* m, const std::string& name, int expect, const float** out) {
    auto it = m->tensors.find(name);
    LC_CHECK(it != m->tensors.end(), LC_ERR_MISSING, "missing tensor %s", name.c_str());
    DevTensor& t = it->second;
    size_t count = t.rows * t.cols;
    LC_CHECK((int)count == expect, LC_ERR_INVALID, "tensor %s has %zu elements, %d expected", name.c_str(), count, expect);
    if (t.typ == LC_TYPE_F32) { *out = (const float*)t.view; return LC_OK; }
    float* p = nullptr;
    LC_TRY(dalloc(&p, count));
    m->owned.push_back(p);
    LC_TRY(launch_dequant(t.typ, t.view, count, p, m->stream));
    *out = p;
    return LC_OK;
}

static int32_t weight_of(lc_model* m, const std::string& name, int n, int k, QWeight* w, DevTensor** tt) {
    auto it = m->tensors.find(name);
    LC_CHECK(it != m->tensors.end(), LC_ERR_MISSING, "missing tensor %s", name.c_str());
    DevTensor& t = it->second;
    LC_CHECK((int)t.rows == n && (int)t.cols == k, LC_ERR_INVALID, "tensor %s is [%zu x %zu], expected [%d x %d]", name.c_str(), t.rows,
             t.cols, n, k);
    if (tt) *tt = &t;
    return qweight_init(w, t.typ, t.view, n, k);
}

// One expert's matrix: the tensor "blk.L.expert.E.<which>.weight", or rows [e * n, (e + 1) * n) of the stacked
// three-dimensional tensor "blk.L.<which>_exps.weight" that GGUF files of mixture models carry.
static int32_t expert_weight(lc_model* m, int l, int e, const char* which, int n, int k, QWeight* w) {
    const std::string p = "blk." + std::to_string(l) + ".";
    const std::string single = p + "expert." + std::to_string(e) + "." + which + ".weight";
    if (m->tensors.count(single)) return weight_of(m, single, n, k, w, nullptr);
    const std::string stacked = p + which + "_exps.weight";
    auto it = m->tensors.find(stacked);
    LC_CHECK(it != m->tensors.end(), LC_ERR_MISSING, "missing tensor %s (or %s)", single.c_str(), stacked.c_str());
    DevTensor& t = it->second;
    LC_CHECK((int)t.cols == k && t.rows == (size_t)n * m->cfg.n_experts, LC_ERR_INVALID, "tensor %s is [%zu x %zu], expected [%d x %d] per expert",
             stacked.c_str(), t.rows, t.cols, n, k);
    QuantGeom g;
    LC_CHECK(quant_geom(t.typ, &g), LC_ERR_UNSUPPORTED, "tensor %s: unsupported type", stacked.c_str());
    const size_t row_bytes = (size_t)k / g.block_elems * g.block_bytes;
    return qweight_init(w, t.typ, (const uint8_t*)t.view + (size_t)e * n * row_bytes, n, k);
}

static int32_t finalize_experts(lc_model* m, int l) {
    LayerW& w = m->layers[l];
    const int E = m->cfg.n_experts, H = m->H, F = m->F;
    const std::string p = "blk." + std::to_string(l) + ".";
    LC_TRY(gain_f32(m, p + "ffn_gate_inp.weight", E * H, &w.router));
    w.egate.resize(E); w.eup.resize(E); w.edown.resize(E);
    bool q4k = true;
    for (int e = 0; e < E; e++) {
        LC_TRY(expert_weight(m, l, e, "ffn_gate", F, H, &w.egate[e]));
        LC_TRY(expert_weight(m, l, e, "ffn_up", F, H, &w.eup[e]));
        LC_TRY(expert_weight(m, l, e, "ffn_down", H, F, &w.edown[e]));
        LC_CHECK(w.egate[e].typ == w.eup[e].typ, LC_ERR_UNSUPPORTED, "layer %d expert %d: gate/up projections have different quant types", l, e);
        for (const QWeight* q : {&w.egate[e], &w.eup[e], &w.edown[e]}) q4k = q4k && q->typ == LC_TYPE_Q4_K && q->has_tmap;
    }
    w.grouped_ok = q4k && qgemv_mma_supports(H) && qgemv_mma_supports(F);
    if (w.grouped_ok) {
        std::vector<unsigned char> host((size_t)E * 128);
        const std::vector<QWeight>* sets[3] = {&w.egate, &w.eup, &w.edown};
        void** dst[3] = {&w.tm_gate, &w.tm_up, &w.tm_down};
        for (int i = 0; i < 3; i++) {
            for (int e = 0; e < E; e++) memcpy(&host[(size_t)e * 128], (*sets[i])[e].tmap, 128);
            LC_TRY(dalloc((uint8_t**)dst[i], host.size()));
            m->owned.push_back(*dst[i]);
            LC_CUDA(cudaMemcpyAsync(*dst[i], host.data(), host.size(), cudaMemcpyHostToDevice, m->stream));
            LC_CUDA(cudaStreamSynchronize(m->stream));
        }
    }
    uint64_t each = 0;
    for (const QWeight* q : {&w.egate[0], &w.eup[0], &w.edown[0]}) each += (uint64_t)q->n * q->row_bytes;
    m->expert_bytes_each = each;
    m->expert_bytes_all += each * E;
    return LC_OK;
}

int32_t lc_model_finalize(lc_model* m) {
    LC_TRY(check_model(m, false));
    LC_CHECK(!m->finalized, LC_ERR_STATE, "model already finalized");
    DeviceGuard dg(m->device);
    const int H = m->H, F = m->F, V = m->V, nq = m->nh * m->hd, nkvd = m->nkv * m->hd;
    m->layers.resize(m->L);
    for (int l = 0; l < m->L; l++) {
        std::string p = "blk." + std::to_string(l) + ".";
        LayerW& w = m->layers[l];
        DevTensor *tq = nullptr, *tk = nullptr, *tv = nullptr;
        LC_TRY(weight_of(m, p + "attn_q.weight", nq, H, &w.q, &tq));
        LC_TRY(weight_of(m, p + "attn_k.weight", nkvd, H, &w.k, &tk));
        LC_TRY(weight_of(m, p + "attn_v.weight", nkvd, H, &w.v, &tv));
        if (tq->typ != tk->typ || tq->typ != tv->typ) {
            // mixed files ("Q4_K_M" keeps attn_v in Q6_K): three separate products per layer
            m->any_unfused_qkv = true;
        } else {   // one [nq + 2 nkv, H] matrix so the three projections are one pass
            size_t total = tq->nbytes + tk->nbytes + tv->nbytes;
            uint8_t* buf = nullptr;
            LC_TRY(dalloc(&buf, total));
            LC_CUDA(cudaMemcpyAsync(buf, tq->view, tq->nbytes, cudaMemcpyDeviceToDevice, m->stream));
            LC_CUDA(cudaMemcpyAsync(buf + tq->nbytes, tk->view, tk->nbytes, cudaMemcpyDeviceToDevice, m->stream));
            LC_CUDA(cudaMemcpyAsync(buf + tq->nbytes + tk->nbytes, tv->view, tv->nbytes, cudaMemcpyDeviceToDevice, m->stream));
            LC_CUDA(cudaStreamSynchronize(m->stream));
            cudaFree(tq->dev); cudaFree(tk->dev); cudaFree(tv->dev);
            tq->dev = tk->dev = tv->dev = nullptr;
            tq->view = buf; tk->view = buf + tq->nbytes; tv->view = buf + tq->nbytes + tk->nbytes;
            w.fused_buf = buf;
            w.fused_qkv = true;
            LC_TRY(qweight_init(&w.qkv, tq->typ, buf, m->nqkv, H));
        }
        LC_TRY(weight_of(m, p + "attn_output.weight", H, nq, &w.o, nullptr));
        if (m->cfg.n_experts > 0) {
            LC_TRY(finalize_experts(m, l));
        } else {
            DevTensor *tg = nullptr, *tu = nullptr;
            LC_TRY(weight_of(m, p + "ffn_gate.weight", F, H, &w.gate, &tg));
            LC_TRY(weight_of(m, p + "ffn_up.weight", F, H, &w.up, &tu));
            LC_CHECK(tg->typ == tu->typ, LC_ERR_UNSUPPORTED, "layer %d: gate/up projections have different quant types", l);
            LC_TRY(weight_of(m, p + "ffn_down.weight", H, F, &w.down, nullptr));
        }
        LC_TRY(gain_f32(m, p + "attn_norm.weight", H, &w.attn_norm));
        LC_TRY(gain_f32(m, p + "ffn_norm.weight", H, &w.ffn_norm));
    }
    {
        auto it = m->tensors.find("token_embd.weight");
        LC_CHECK(it != m->tensors.end(), LC_ERR_MISSING, "missing tensor token_embd.weight");
        LC_CHECK((int)it->second.cols == H, LC_ERR_INVALID, "token_embd.weight rows are %zu wide, hidden size is %d", it->second.cols, H);
        m->embed = &it->second;
    }
    LC_TRY(gain_f32(m, "output_norm.weight", H, &m->final_norm));
    // loader.rs:192-199: tied head when output.weight is absent
    std::string head = m->tensors.count("output.weight") ? "output.weight" : "token_embd.weight";
    LC_TRY(weight_of(m, head, V, H, &m->head, nullptr));

    // weight sanity scan (loader.rs:241-249) and resident byte count
    LC_TRY(dalloc(&m->d_sanity, 1));
    LC_CUDA(cudaMemsetAsync(m->d_sanity, 0, 8, m->stream));
    uint64_t wbytes = 0;
    for (auto& kv : m->tensors) {
        DevTensor& t = kv.second;
        wbytes += t.nbytes;
        LC_TRY(launch_sanity_scan(t.typ, t.view, t.rows * t.cols, m->d_sanity, m->stream));
    }
    unsigned long long bad = 0;
    LC_CUDA(cudaMemcpyAsync(&bad, m->d_sanity, 8, cudaMemcpyDeviceToHost, m->stream));
    LC_CUDA(cudaStreamSynchronize(m->stream));
    m->ctr.sanitize_hits = bad;
    m->ctr.weight_bytes = wbytes;

    // KV pools and the page table
    size_t page_elems = (size_t)m->nkv * m->page_tokens * m->hd;
    m->k_pools.resize(m->L); m->v_pools.resize(m->L);
    for (int l = 0; l < m->L; l++) {
        LC_TRY(dalloc((uint8_t**)&m->k_pools[l], (size_t)m->pages_total * page_elems * m->kv_elt));
        LC_TRY(dalloc((uint8_t**)&m->v_pools[l], (size_t)m->pages_total * page_elems * m->kv_elt));
    }
    if (m->hd == 128 && m->cfg.kv_dtype == 0 && m->page_tokens == 16) {  // what the streaming attention kernel reads keys through
        m->k_tmaps.resize(m->L);
        m->v_tmaps.resize(m->L);
        m->k_tmaps_ok = true;
        for (int l = 0; l < m->L && m->k_tmaps_ok; l++)
            m->k_tmaps_ok = make_key_pool_tmap(m->k_tmaps[l].b, m->k_pools[l], (uint64_t)m->pages_total * m->nkv * m->page_tokens) &&
                            make_key_pool_tmap(m->v_tmaps[l].b, m->v_pools[l], (uint64_t)m->pages_total * m->nkv * m->page_tokens);
    }
    if (m->k_tmaps_ok) {
        // merge slots of the single-token attention kernel: one set per model, because a captured decode step keeps the pointer
        const size_t slot_bytes = attention_stream_slot_bytes(m->nh, m->nkv);
        if (slot_bytes) {
            LC_TRY(dalloc((uint8_t**)&m->d_stream_slots, slot_bytes));
            LC_CUDA(cudaMemsetAsync(m->d_stream_slots, 0, slot_bytes, m->stream));
        }
    }
    m->free_pages.resize(m->pages_total);
    for (int i = 0; i < m->pages_total; i++) m->free_pages[i] = m->pages_total - 1 - i;
    m->seq_pages.assign(m->max_seqs, {});
    m->seq_len.assign(m->max_seqs, 0);
    m->h_page_table.assign((size_t)m->max_seqs * m->pages_per_seq, 0);
    LC_TRY(dalloc(&m->d_page_table, m->h_page_table.size()));
    m->ctr.kv_pages_total = m->pages_total;

    // step buffers
    int T = m->t_cap;
    LC_TRY(dalloc(&m->d_tokens, T)); LC_TRY(dalloc(&m->d_tok_seq, T)); LC_TRY(dalloc(&m->d_tok_pos, T));
    LC_TRY(dalloc(&m->d_tok_rope, T)); LC_TRY(dalloc(&m->d_last_idx, T));
    LC_TRY(dalloc(&m->d_hidden, (size_t)T * H)); LC_TRY(dalloc(&m->d_hidden2, (size_t)T * H));
    LC_TRY(dalloc(&m->d_qkv, (size_t)T * m->nqkv)); LC_TRY(dalloc(&m->d_attn, (size_t)T * nq));
    LC_TRY(dalloc(&m->d_ffn, (size_t)T * F));
    LC_TRY(qgemm_workspace_alloc(&m->gemm_ws, T, std::max(std::max(H, F), nq)));
    if (m->any_unfused_qkv) LC_TRY(dalloc(&m->d_qkv_parts, (size_t)T * m->nqkv));
    if (m->cfg.n_experts > 0) {
        const int E = m->cfg.n_experts, K = m->cfg.top_k;
        LC_TRY(dalloc(&m->d_moe_sel, (size_t)T * K)); LC_TRY(dalloc(&m->d_moe_w, (size_t)T * K));
        LC_TRY(dalloc(&m->d_moe_cnt, (size_t)E)); LC_TRY(dalloc(&m->d_moe_lists, (size_t)E * kMoeGroupedTokens));
        LC_TRY(dalloc(&m->d_moe_h, (size_t)kMoeGroupedTokens * K * F)); LC_TRY(dalloc(&m->d_moe_y, (size_t)kMoeGroupedTokens * K * H));
        LC_TRY(dalloc(&m->d_moe_yall, (size_t)E * T * H));
        LC_TRY(dalloc(&m->d_moe_touched, 1));
        LC_CUDA(cudaMemsetAsync(m->d_moe_touched, 0, 8, m->stream));
    }
    LC_TRY(dalloc(&m->d_last, (size_t)m->max_seqs * H)); LC_TRY(dalloc(&m->d_logits, (size_t)m->max_seqs * V));
    LC_TRY(dalloc(&m->d_next, m->max_seqs)); LC_TRY(dalloc(&m->d_step_ctr, 1));
    size_t sc = 16;
    for (int t = 1; t <= T; t++) sc = std::max(sc, attention_scratch_bytes(t, m->nh, m->hd, m->cfg.max_seq_len));
    m->attn_scratch_bytes = sc;
    LC_TRY(dalloc((uint8_t**)&m->d_attn_scratch, sc));
    LC_TRY(dalloc(&m->d_attn_counters, (size_t)T * m->nh));
    LC_CUDA(cudaMemsetAsync(m->d_attn_counters, 0, (size_t)T * m->nh * sizeof(int), m->stream));
    LC_CUDA(cudaHostAlloc((void**)&m->pin_tokens, (size_t)m->max_seqs * 8, cudaHostAllocDefault));
    LC_CUDA(cudaHostAlloc((void**)&m->pin_next, (size_t)m->max_seqs * 8, cudaHostAllocDefault));
    LC_CUDA(cudaHostAlloc((void**)&m->pin_logits, (size_t)m->max_seqs * V * 4, cudaHostAllocDefault));
    LC_TRY(reserve_out_tokens(m, (size_t)1024 * m->max_seqs));
    LC_CUDA(cudaEventCreate(&m->ev0));
    LC_CUDA(cudaEventCreate(&m->ev1));
    LC_CUDA(cudaStreamSynchronize(m->stream));
    m->finalized = true;
    return LC_OK;
}

int32_t lc_model_destroy(lc_model* m) {
    if (!m) return LC_OK;
    DeviceGuard dg(m->device);
    cudaStreamSynchronize(m->stream);
    for (auto& g : m->decode_graphs) cudaGraphExecDestroy(g.second);
    for (auto& kv : m->tensors) if (kv.second.dev) cudaFree(kv.second.dev);
    for (auto& w : m->layers) if (w.fused_buf) cudaFree(w.fused_buf);
    for (void* p : m->owned) cudaFree(p);
    for (void* p : m->k_pools) cudaFree(p);
    for (void* p : m->v_pools) cudaFree(p);
    void* bufs[] = {m->d_moe_sel, m->d_moe_w, m->d_moe_cnt, m->d_moe_lists, m->d_moe_h, m->d_moe_y, m->d_moe_yall, m->d_moe_touched,
                    m->d_stream_slots, m->d_page_table, m->d_tokens, m->d_tok_seq, m->d_tok_pos, m->d_tok_rope, m->d_last_idx, m->d_hidden, m->d_hidden2,
                    m->d_qkv, m->d_attn, m->d_ffn, m->d_last, m->d_logits, m->d_next, m->d_out_tokens, m->d_step_ctr,
                    m->d_attn_scratch, m->d_attn_counters, m->d_sanity, m->d_qkv_parts};
    for (void* p : bufs) if (p) cudaFree(p);
    qgemm_workspace_free(&m->gemm_ws);
    if (m->pin_tokens) cudaFreeHost(m->pin_tokens);
    if (m->pin_next) cudaFreeHost(m->pin_next);
    if (m->pin_logits) cudaFreeHost(m->pin_logits);
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    delete m;
    return LC_OK;
}

int32_t lc_model_get_config(const lc_model* m, lc_model_config* out) {
    LC_TRY(check_model(m, false));
    LC_CHECK(out, LC_ERR_INVALID, "null output");
    *out = m->cfg;
    return LC_OK;
}

int32_t lc_kv_clear(lc_model* m, int32_t seq_id) {
    LC_TRY(check_model(m, true));
    LC_CHECK(seq_id >= -1 && seq_id < m->max_seqs, LC_ERR_INVALID, "sequence id %d outside 0..%d", seq_id, m->max_seqs - 1);
    for (int s = 0; s < m->max_seqs; s++) {
        if (seq_id >= 0 && s != seq_id) continue;
        for (int p : m->seq_pages[s]) m->free_pages.push_back(p);
        m->seq_pages[s].clear();
        m->seq_len[s] = 0;
    }
    m->meta_valid = false;
    return LC_OK;
}

int32_t lc_kv_memory_bytes(const lc_model* m, uint64_t* out) {
    LC_TRY(check_model(m, true));
    LC_CHECK(out, LC_ERR_INVALID, "null output");
    uint64_t tokens = 0;
    for (int v : m->seq_len) tokens += v;
    *out = tokens * (uint64_t)m->L * 2 * m->nkv * m->hd * m->kv_elt;  // cache/mod.rs:80-84
    return LC_OK;
}

int32_t lc_kv_length(const lc_model* m, int32_t seq_id, int32_t* out) {
    LC_TRY(check_model(m, true));
    LC_CHECK(out && seq_id >= 0 && seq_id < m->max_seqs, LC_ERR_INVALID, "bad sequence id %d", seq_id);
    *out = m->seq_len[seq_id];
    return LC_OK;
}

int32_t lc_forward_batch(lc_model* m, int32_t n_seqs, const int32_t* seq_ids, const int64_t* tokens, const int32_t* n_tokens,
                         float* logits_out, int64_t* next_out) {
    LC_TRY(check_model(m, true));
    LC_CHECK(n_seqs >= 1 && n_seqs <= m->max_seqs && seq_ids && tokens && n_tokens, LC_ERR_INVALID, "forward_batch: bad argument");
    DeviceGuard dg(m->device);
    int total = 0, longest = 0;
    for (int i = 0; i < n_seqs; i++) {
        LC_CHECK(seq_ids[i] >= 0 && seq_ids[i] < m->max_seqs, LC_ERR_INVALID, "sequence id %d outside 0..%d", seq_ids[i], m->max_seqs - 1);
        for (int j = 0; j < i; j++) LC_CHECK(seq_ids[j] != seq_ids[i], LC_ERR_INVALID, "sequence id %d listed twice", seq_ids[i]);
        LC_CHECK(n_tokens[i] >= 1, LC_ERR_INVALID, "sequence %d has no tokens in this call", seq_ids[i]);
        LC_TRY(ensure_pages(m, seq_ids[i], m->seq_len[seq_ids[i]] + n_tokens[i]));
        total += n_tokens[i];
        longest = std::max(longest, n_tokens[i]);
    }
    LC_TRY(sync_page_table(m));
    if (longest == 1) {
        // a decode step: token ids in (pinned staging), graph replay, picks and logits out
        LC_TRY(reserve_out_tokens(m, (size_t)n_seqs));
        LC_TRY(stage_decode_meta(m, n_seqs, seq_ids, tokens));
        LC_CUDA(cudaMemsetAsync(m->d_step_ctr, 0, 4, m->stream));
        LC_TRY(run_decode_steps(m, n_seqs, 1));
        if (logits_out) LC_CUDA(cudaMemcpyAsync(m->pin_logits, m->d_logits, (size_t)n_seqs * m->V * 4, cudaMemcpyDeviceToHost, m->stream));
        if (next_out) LC_CUDA(cudaMemcpyAsync(m->pin_next, m->d_next, (size_t)n_seqs * 8, cudaMemcpyDeviceToHost, m->stream));
        LC_CUDA(cudaStreamSynchronize(m->stream));
        if (logits_out) memcpy(logits_out, m->pin_logits, (size_t)n_seqs * m->V * 4);
        if (next_out) memcpy(next_out, m->pin_next, (size_t)n_seqs * 8);
        after_decode_steps(m, n_seqs, seq_ids, 1);
        finish_call(m);
        return check_device_flag(m);
    }
    m->meta_valid = false;
    // Rotary index = position inside the CALL (reference mode, attention.rs:13-21) or the cache position.
    if (total <= m->t_cap) {
        std::vector<int64_t> tok; std::vector<int32_t> seq, pos, rope, last;
        int off = 0;
        for (int i = 0; i < n_seqs; i++) {
            for (int t = 0; t < n_tokens[i]; t++) {
                int p = m->seq_len[seq_ids[i]] + t;
                tok.push_back(tokens[off + t]); seq.push_back(seq_ids[i]); pos.push_back(p);
                rope.push_back(m->cfg.rope_mode ? p : t);
            }
            off += n_tokens[i];
            last.push_back(off - 1);
        }
        LC_TRY(upload_meta(m, tok, seq, pos, rope, last));
        LC_TRY(forward_tokens(m, total, n_seqs, total == n_seqs, 0));
    } else {
        // long prompts: one sequence after the other, each in chunks of t_cap tokens over its growing cache
        int off = 0;
        for (int i = 0; i < n_seqs; i++) {
            for (int c0 = 0; c0 < n_tokens[i]; c0 += m->t_cap) {
                int T = std::min(m->t_cap, n_tokens[i] - c0);
                std::vector<int64_t> tok(T); std::vector<int32_t> seq(T, seq_ids[i]), pos(T), rope(T), last(1, T - 1);
                for (int t = 0; t < T; t++) {
                    tok[t] = tokens[off + c0 + t];
                    pos[t] = m->seq_len[seq_ids[i]] + c0 + t;
                    rope[t] = m->cfg.rope_mode ? pos[t] : (c0 + t);
                }
                LC_TRY(upload_meta(m, tok, seq, pos, rope, last));
                if (c0 + T == n_tokens[i]) LC_TRY(forward_tokens(m, T, 1, T == 1, i));
                else LC_TRY(run_layers(m, T, false));
            }
            off += n_tokens[i];
        }
    }
    for (int i = 0; i < n_seqs; i++) m->seq_len[seq_ids[i]] += n_tokens[i];
    if (logits_out) LC_CUDA(cudaMemcpyAsync(logits_out, m->d_logits, (size_t)n_seqs * m->V * 4, cudaMemcpyDeviceToHost, m->stream));
    if (next_out) LC_CUDA(cudaMemcpyAsync(next_out, m->d_next, (size_t)n_seqs * 8, cudaMemcpyDeviceToHost, m->stream));
    LC_CUDA(cudaStreamSynchronize(m->stream));
    m->ctr.forward_calls += 1;
    m->ctr.tokens_prefilled += total;
    uint64_t used = 0;
    for (auto& pg : m->seq_pages) used += pg.size();
    m->ctr.kv_pages_in_use = used;
    finish_call(m);
    return LC_OK;
}

int32_t lc_forward(lc_model* m, const int64_t* tokens, int32_t n, float* logits_out) {
    LC_CHECK(tokens && n >= 1 && logits_out, LC_ERR_INVALID, "lc_forward: bad argument");
    int32_t seq = 0;
    return lc_forward_batch(m, 1, &seq, tokens, &n, logits_out, nullptr);
}

// Queues `steps` greedy decode steps for the n_seqs sequences whose metadata is on the device.  The first
// step of a new batch width runs eagerly (it sets kernel attributes), then one step is captured into a
// CUDA graph that later steps replay.
static int32_t run_decode_steps(lc_model* m, int n_seqs, int steps) {
    auto one_step = [&]() -> int32_t {
        LC_TRY(forward_tokens(m, n_seqs, n_seqs, true, 0));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1);
        cfg.blockDim = dim3(std::max(32, (n_seqs + 31) / 32 * 32));
        cfg.stream = m->stream;
        LC_CUDA(cudaLaunchKernelEx(&cfg, advance_kernel, (const int64_t*)m->d_next, m->d_tokens, m->d_tok_pos, m->d_tok_rope, (int)n_seqs,
                                   (int)m->cfg.rope_mode, m->d_out_tokens, m->d_step_ctr));
        m->launches_in_call += 1;
        return LC_OK;
    };
    static const bool no_graph = getenv("LC_NO_GRAPH") != nullptr;
    cudaGraphExec_t exec = nullptr;
    int done_steps = 0;
    auto it = m->decode_graphs.find(n_seqs);
    if (it != m->decode_graphs.end()) exec = it->second;
    if (!exec && !no_graph) {
        uint64_t before = m->launches_in_call;
        LC_TRY(one_step());
        m->graph_nodes = (int)(m->launches_in_call - before);
        done_steps = 1;
        cudaGraph_t graph = nullptr;
        if (cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
            uint64_t keep = m->launches_in_call;
            int32_t st = one_step();
            m->launches_in_call = keep;
            cudaError_t e = cudaStreamEndCapture(m->stream, &graph);
            if (st == LC_OK && e == cudaSuccess && graph) {
                if (cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess) m->decode_graphs[n_seqs] = exec;
                else exec = nullptr;
            }
            if (graph) cudaGraphDestroy(graph);
        }
        (void)cudaGetLastError();
    }
    for (int s = done_steps; s < steps; s++) {
        if (exec) {
            LC_CUDA(cudaGraphLaunch(exec, m->stream));
            m->launches_in_call += m->graph_nodes;
        } else {
            LC_TRY(one_step());
        }
    }
    return LC_OK;
}

static int32_t reserve_out_tokens(lc_model* m, size_t need) {
    if (need <= m->out_tokens_cap) return LC_OK;
    if (m->d_out_tokens) cudaFree(m->d_out_tokens);
    m->d_out_tokens = nullptr;
    m->out_tokens_cap = 0;
    LC_TRY(dalloc(&m->d_out_tokens, need));
    m->out_tokens_cap = need;
    for (auto& g : m->decode_graphs) cudaGraphExecDestroy(g.second);  // the graphs bake this pointer in
    m->decode_graphs.clear();
    return LC_OK;
}

// Describes a decode step (one token per listed sequence at its current cache position) on the device.
static int32_t stage_decode_meta(lc_model* m, int n_seqs, const int32_t* seq_ids, const int64_t* toks) {
    bool same = m->meta_valid && (int)m->meta_seqs.size() == n_seqs;
    for (int i = 0; same && i < n_seqs; i++) same = m->meta_seqs[i] == seq_ids[i] && m->meta_pos[i] == m->seq_len[seq_ids[i]];
    if (same) {  // positions already advanced on the device by the previous step: only the token ids travel
        memcpy(m->pin_tokens, toks, (size_t)n_seqs * 8);
        LC_CUDA(cudaMemcpyAsync(m->d_tokens, m->pin_tokens, (size_t)n_seqs * 8, cudaMemcpyHostToDevice, m->stream));
        return LC_OK;
    }
    std::vector<int64_t> tok(toks, toks + n_seqs);
    std::vector<int32_t> seq(seq_ids, seq_ids + n_seqs), pos(n_seqs), rope(n_seqs), last(n_seqs);
    for (int i = 0; i < n_seqs; i++) {
        pos[i] = m->seq_len[seq_ids[i]];
        rope[i] = m->cfg.rope_mode ? pos[i] : 0;
        last[i] = i;
    }
    LC_TRY(upload_meta(m, tok, seq, pos, rope, last));
    m->meta_seqs.assign(seq_ids, seq_ids + n_seqs);
    m->meta_pos.assign(pos.begin(), pos.end());
    m->meta_valid = true;
    return LC_OK;
}

static void after_decode_steps(lc_model* m, int n_seqs, const int32_t* seq_ids, int steps) {
    if (m->d_moe_touched) {  // experts touched, summed over the layers of these steps (grouped calls count them; others touch all)
        unsigned long long t = 0;
        if (cudaMemcpyAsync(&t, m->d_moe_touched, 8, cudaMemcpyDeviceToHost, m->stream) == cudaSuccess &&
            cudaMemsetAsync(m->d_moe_touched, 0, 8, m->stream) == cudaSuccess && cudaStreamSynchronize(m->stream) == cudaSuccess)
            m->touched_per_step = n_seqs <= kMoeGroupedTokens && m->layers[0].grouped_ok ? (double)t / std::max(steps, 1)
                                                                                           : (double)m->L * m->cfg.n_experts;
    }
    std::vector<int> ctx;
    for (int i = 0; i < n_seqs; i++) {
        m->seq_len[seq_ids[i]] += steps;
        m->meta_pos[i] += steps;
        ctx.push_back(m->seq_len[seq_ids[i]] - 1);
    }
    m->ctr.algo_bytes_last_step = algo_bytes_step(m, ctx);
    m->ctr.tokens_decoded += (uint64_t)steps * n_seqs;
    m->ctr.forward_calls += steps;
    uint64_t used = 0;
    for (auto& pg : m->seq_pages) used += pg.size();
    m->ctr.kv_pages_in_use = used;
}

int32_t lc_decode_loop(lc_model* m, int32_t n_seqs, const int32_t* seq_ids, const int64_t* first_tokens, int32_t steps,
                       int64_t* out_tokens, float* out_ms) {
    LC_TRY(check_model(m, true));
    LC_CHECK(n_seqs >= 1 && n_seqs <= m->max_seqs && seq_ids && first_tokens && steps >= 1, LC_ERR_INVALID, "decode_loop: bad argument");
    DeviceGuard dg(m->device);
    for (int i = 0; i < n_seqs; i++) {
        LC_CHECK(seq_ids[i] >= 0 && seq_ids[i] < m->max_seqs, LC_ERR_INVALID, "sequence id %d outside 0..%d", seq_ids[i], m->max_seqs - 1);
        for (int j = 0; j < i; j++) LC_CHECK(seq_ids[j] != seq_ids[i], LC_ERR_INVALID, "sequence id %d listed twice", seq_ids[i]);
        LC_TRY(ensure_pages(m, seq_ids[i], m->seq_len[seq_ids[i]] + steps));  // pages for the whole loop up front
    }
    LC_TRY(sync_page_table(m));
    size_t need = (size_t)steps * n_seqs;
    LC_TRY(reserve_out_tokens(m, need));
    LC_TRY(stage_decode_meta(m, n_seqs, seq_ids, first_tokens));
    LC_CUDA(cudaMemsetAsync(m->d_step_ctr, 0, 4, m->stream));
    LC_CUDA(cudaEventRecord(m->ev0, m->stream));
    LC_TRY(run_decode_steps(m, n_seqs, steps));
    LC_CUDA(cudaEventRecord(m->ev1, m->stream));
    LC_CUDA(cudaEventSynchronize(m->ev1));
    float ms = 0.f;
    LC_CUDA(cudaEventElapsedTime(&ms, m->ev0, m->ev1));
    if (out_ms) *out_ms = ms;
    if (out_tokens) {
        LC_CUDA(cudaMemcpyAsync(out_tokens, m->d_out_tokens, need * 8, cudaMemcpyDeviceToHost, m->stream));
        LC_CUDA(cudaStreamSynchronize(m->stream));
    }
    after_decode_steps(m, n_seqs, seq_ids, steps);
    finish_call(m);
    return check_device_flag(m);
}

int32_t lc_model_set_seed(lc_model* m, uint64_t seed) {
    LC_TRY(check_model(m, false));
    m->seeded = true;
    m->seed = seed;
    m->draws = 0;
    return LC_OK;
}

int32_t lc_generate(lc_model* m, const int64_t* tokens, int32_t n, int32_t max_tokens, float temperature, float top_p,
                    int32_t stop_on_eos, int64_t* out_tokens, int32_t* n_out, lc_token_cb cb, void* user) {
    LC_TRY(check_model(m, true));
    LC_CHECK(tokens && n >= 1 && max_tokens >= 1 && out_tokens && n_out, LC_ERR_INVALID, "lc_generate: bad argument");
    const bool stochastic = temperature > 0.0f;
    LC_CHECK(!stochastic || m->seeded, LC_ERR_UNSUPPORTED,
             "stochastic sampling draws from an unseeded generator in the reference (rust/src/inference/sampler.rs:38-39); call "
             "lc_model_set_seed first for a seeded draw sequence, or pass temperature <= 0 for greedy");
    LC_TRY(lc_kv_clear(m, 0));  // engine.rs:52
    int32_t seq = 0;
    int64_t next = 0;
    // sample_top_p on the logits of the last forward (engine.rs:57, 69): they are still in device memory
    auto pick = [&](int64_t* tok) -> int32_t {
        if (!stochastic) return LC_OK;  // the greedy pick came back with the forward
        DeviceGuard dg(m->device);
        return sample_top_p_sync(m->d_logits, (size_t)m->V, temperature, top_p, seeded_uniform(m->seed, m->draws++), tok, m->stream);
    };
    LC_TRY(lc_forward_batch(m, 1, &seq, tokens, &n, nullptr, &next));  // engine.rs:55-57
    LC_TRY(pick(&next));
    int count = 0;
    out_tokens[count++] = next;
    if (cb) cb(next, user);
    if (!(stop_on_eos && next == 2)) {
        if (!cb && !stop_on_eos && !stochastic && max_tokens > 1) {
            // nothing observes the tokens one by one: keep the loop on the device
            LC_TRY(lc_decode_loop(m, 1, &seq, &next, max_tokens - 1, out_tokens + 1, nullptr));
            count = max_tokens;
        } else {
            for (int s = 0; s + 1 < max_tokens; s++) {  // engine.rs:65-73
                int32_t one = 1;
                int64_t cur = next;
                LC_TRY(lc_forward_batch(m, 1, &seq, &cur, &one, nullptr, &next));
                LC_TRY(pick(&next));
                out_tokens[count++] = next;
                if (cb) cb(next, user);
                if (stop_on_eos && next == 2) break;
            }
        }
    }
    *n_out = count;
    return LC_OK;
}

int32_t lc_get_counters(const lc_model* m, lc_counters* out) {
    LC_TRY(check_model(m, false));
    LC_CHECK(out, LC_ERR_INVALID, "null output");
    *out = m->ctr;
    return LC_OK;
}
int32_t lc_reset_counters(lc_model* m) {
    LC_TRY(check_model(m, false));
    uint64_t wb = m->ctr.weight_bytes, san = m->ctr.sanitize_hits, pt = m->ctr.kv_pages_total, pu = m->ctr.kv_pages_in_use;
    m->ctr = lc_counters{};
    m->ctr.weight_bytes = wb; m->ctr.sanitize_hits = san; m->ctr.kv_pages_total = pt; m->ctr.kv_pages_in_use = pu;
    return LC_OK;
}

static int32_t probe_meta(lc_model* m, int seq_tokens) {
    LC_CHECK(seq_tokens >= 1 && seq_tokens <= m->t_cap, LC_ERR_INVALID, "probe: %d tokens outside 1..%d", seq_tokens, m->t_cap);
    LC_TRY(ensure_pages(m, 0, m->seq_len[0] + seq_tokens));
    LC_TRY(sync_page_table(m));
    m->meta_valid = false;
    std::vector<int64_t> tok(seq_tokens, 0);
    std::vector<int32_t> seq(seq_tokens, 0), pos(seq_tokens), rope(seq_tokens), last;
    for (int i = 0; i < seq_tokens; i++) { pos[i] = m->seq_len[0] + i; rope[i] = m->cfg.rope_mode ? pos[i] : i; }
    return upload_meta(m, tok, seq, pos, rope, last);
}

int32_t lc_probe_attention(lc_model* m, int32_t layer, const float* normed, int32_t seq, float* out) {
    LC_TRY(check_model(m, true));
    LC_CHECK(layer >= 0 && layer < m->L && normed && out, LC_ERR_INVALID, "probe_attention: bad argument");
    DeviceGuard dg(m->device);
    LC_TRY(probe_meta(m, seq));
    LC_CUDA(cudaMemcpyAsync(m->d_hidden, normed, (size_t)seq * m->H * 4, cudaMemcpyHostToDevice, m->stream));
    LC_TRY(attention_block(m, layer, m->d_hidden, nullptr, seq, nullptr, m->d_hidden2, false));
    LC_CUDA(cudaMemcpyAsync(out, m->d_hidden2, (size_t)seq * m->H * 4, cudaMemcpyDeviceToHost, m->stream));
    LC_CUDA(cudaStreamSynchronize(m->stream));
    m->seq_len[0] += seq;
    finish_call(m);
    return LC_OK;
}

int32_t lc_probe_ffn(lc_model* m, int32_t layer, const float* x, int32_t seq, float* out) {
    LC_TRY(check_model(m, true));
    LC_CHECK(layer >= 0 && layer < m->L && x && out && seq >= 1 && seq <= m->t_cap, LC_ERR_INVALID, "probe_ffn: bad argument");
    DeviceGuard dg(m->device);
    LC_CUDA(cudaMemcpyAsync(m->d_hidden, x, (size_t)seq * m->H * 4, cudaMemcpyHostToDevice, m->stream));
    LC_TRY(ffn_block(m, layer, m->d_hidden, nullptr, seq, nullptr, m->d_hidden2, false));
    LC_CUDA(cudaMemcpyAsync(out, m->d_hidden2, (size_t)seq * m->H * 4, cudaMemcpyDeviceToHost, m->stream));
    LC_CUDA(cudaStreamSynchronize(m->stream));
    finish_call(m);
    return LC_OK;
}


}  // extern "C"

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

    // geometry: H, L, hd are the model's; nh, nkv, F, V, nqkv are THIS RANK'S part when the model is cut across ranks
    // (tp > 1: heads, kv heads, FFN rows and vocabulary rows divided by tp; experts e0 .. e0 + El - 1 of a mixture layer)
    int H = 0, L = 0, nh = 0, nkv = 0, hd = 0, F = 0, V = 0, nqkv = 0;
    int tp = 1, rank = 0, v0 = 0, e0 = 0, El = 0;
    bool use_dist = false;               // the ranks are other processes (lc_dist_init); else members lists them, or tp == 1
    std::vector<lc_model*> members;      // rank 0 of an in-process group: every rank's handle in rank order (itself first)
    lc_model* leader = nullptr;          // a rank > 0 of such a group
    float* d_part = nullptr;             // where the column-cut products leave their partial rows for the sum over the ranks
    long long* d_key = nullptr;          // greedy pick of the local vocabulary slice as (total-order key << 32 | global index)
    long long* d_key_max = nullptr;
    float* d_logits_all = nullptr;       // dist: the ranks' logit slices gathered for the host
    PrefillTile* d_tiles = nullptr;      // the call's tokens as runs of up to 64 consecutive positions of one sequence
    int n_tiles = 0;
    float* pending_dst = nullptr;        // where the next sum over the ranks has to land
    bool pending_pushed = false;         // ... and whether the product already sent its rows to the ranks
    GemvPush push_desc;
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
    GemvPlanes moe_planes_x, moe_planes_h;  // fixed-point activations of the grouped launches: the layer's input per token, the experts' hidden rows per slot
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

// Which part of a tensor rank `rank` of `tp` keeps (see the model-parallelism note of the C header).
enum { SHARD_ALL = 0, SHARD_ROWS = 1, SHARD_COLS = 2, SHARD_NONE = 3 };
struct ShardPlan { int kind = SHARD_ALL; uint64_t first = 0, count = 0; };
bool ends_with(const std::string& s, const char* suf) {
    const size_t n = strlen(suf);
    return s.size() >= n && s.compare(s.size() - n, n, suf) == 0;
}
int32_t shard_plan(const lc_model_config& c, int tp, int rank, const std::string& key, const uint64_t* dims, int ndims, ShardPlan* out) {
    ShardPlan pl;
    uint64_t total_rows = 1;
    for (int i = 1; i < ndims; i++) total_rows *= dims[i];
    pl.count = total_rows;
    *out = pl;
    if (tp <= 1) return LC_OK;
    LC_CHECK(rank >= 0 && rank < tp, LC_ERR_INVALID, "rank %d outside 0..%d", rank, tp - 1);
    const bool expert_one = key.find(".expert.") != std::string::npos;
    if (expert_one) {  // blk.L.expert.E.<proj>.weight: a whole expert, on the rank that owns it
        const size_t at = key.find(".expert.") + 8;
        const int e = atoi(key.c_str() + at), per = c.n_experts > 0 ? c.n_experts / tp : 0;
        LC_CHECK(per > 0 && c.n_experts % tp == 0, LC_ERR_INVALID, "%d experts cannot be dealt to %d ranks", c.n_experts, tp);
        if (e < rank * per || e >= (rank + 1) * per) { pl.kind = SHARD_NONE; pl.count = 0; }
        *out = pl;
        return LC_OK;
    }
    const bool rows = ends_with(key, "attn_q.weight") || ends_with(key, "attn_k.weight") || ends_with(key, "attn_v.weight") ||
                      ends_with(key, "ffn_gate.weight") || ends_with(key, "ffn_up.weight") || key == "output.weight" ||
                      ends_with(key, "ffn_gate_exps.weight") || ends_with(key, "ffn_up_exps.weight") || ends_with(key, "ffn_down_exps.weight");
    const bool cols = ends_with(key, "attn_output.weight") || ends_with(key, "ffn_down.weight");
    if (rows) {
        LC_CHECK(ndims >= 2 && total_rows % tp == 0, LC_ERR_INVALID, "tensor %s: %llu rows cannot be cut into %d equal parts", key.c_str(),
                 (unsigned long long)total_rows, tp);
        pl.kind = SHARD_ROWS; pl.count = total_rows / tp; pl.first = pl.count * rank;
    } else if (cols) {
        LC_CHECK(ndims == 2 && dims[0] % tp == 0, LC_ERR_INVALID, "tensor %s: %llu columns cannot be cut into %d equal parts", key.c_str(),
                 (unsigned long long)dims[0], tp);
        pl.kind = SHARD_COLS; pl.count = dims[0] / tp; pl.first = pl.count * rank;
    }
    *out = pl;
    return LC_OK;
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

// Where a product whose input columns are cut across the ranks writes: `out` itself for a whole model, else the rank's
// partial-row slot (the sum over the ranks, issued by the caller, then lands in `out`).
float* partial_dst(lc_model* m, float* out) {
    if (m->tp == 1) return out;
    m->pending_dst = out;
    m->pending_pushed = false;
    return m->d_part;
}
// A matrix-vector product of up to four tokens that ends in a sum over ranks in other processes can write its rows
// straight into the ranks' buffers (one NVLink trip, no kernel boundary before the transfer); the sum then only gathers.
void try_push(lc_model* m, GemvArgs* a, int T) {
    static const bool off = getenv("LC_DIST_NO_PUSH") != nullptr;  // diagnostics: every sum as its own send + gather kernel
    if (off || !m->use_dist || T > 4 || !qgemv_push_supported(*a)) return;
    if (!dist_push_desc((size_t)T * m->H, &m->push_desc)) return;
    a->push = &m->push_desc;
    m->pending_pushed = true;
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
        static const bool no_tc = getenv("LC_PREFILL_FMA") != nullptr;  // diagnostics: the one-CTA-per-(token, head) kernel for every call
        if (T >= 16 && m->n_tiles > 0 && !no_tc && attention_prefill_applies(kv, m->nh))  // a prefill chunk: tiles of 64 queries on the tensor cores
            LC_TRY(launch_attention_prefill(q, m->nqkv, m->d_attn, m->nh, kv, m->d_tiles, m->n_tiles, m->d_page_table, m->pages_per_seq, m->stream));
        else
            LC_TRY(launch_attention(q, m->nqkv, m->d_attn, T, m->nh, kv, m->d_tok_seq, m->d_tok_pos, m->d_page_table, m->pages_per_seq,
                                    m->cfg.max_seq_len, m->d_attn_scratch, m->d_attn_counters, nullptr, m->stream));
        m->launches_in_call += 2;
    }
    GemvArgs o;
    o.w = &w.o;
    o.x = m->d_attn;
    o.out = partial_dst(m, out);  // cut model: this rank's heads give a partial row; the caller sums the ranks into `out`
    if (residual && (m->tp == 1 || m->rank == 0)) { o.residual = residual; o.epi = EPI_ADD_RESIDUAL; }  // the residual enters the sum once
    if (m->tp == 1 && residual && out == m->d_hidden2 && w.ffn_norm) {  // in a layer of the forward pass the FFN reads `out` next, through its norm
        o.prep_next = true; o.next_norm_w = w.ffn_norm; o.next_eps = m->cfg.rms_eps;
    }
    o.m = T;
    if (m->tp > 1) try_push(m, &o, T);
    return gemv_tiled(m, o, T, m->H, m->nh * m->hd);
}

// Mixture-of-experts FFN in place of ffn_forward (moe.cu has the definition): router, then either ONE grouped launch per
// projection over the experts that received tokens (Q4_K experts, calls of up to 64 tokens), or every expert on every
// token through the ordinary products (prefill chunks, other quant types), then the weighted sum of the chosen experts.
int32_t moe_block(lc_model* m, int l, const float* x, const float* norm_w, int T, const float* residual, float* out) {
    LayerW& w = m->layers[l];
    const int E = m->cfg.n_experts, K = m->cfg.top_k, El = m->El, e0 = m->e0;  // this rank's experts: e0 .. e0 + El - 1
    const bool grouped = w.grouped_ok && T <= kMoeGroupedTokens;
    if (m->tp > 1 && m->rank != 0) residual = nullptr;  // the residual enters the sum over the ranks once
    out = partial_dst(m, out);
    MoeRouteArgs r;
    r.x = x; r.norm_w = norm_w; r.eps = m->cfg.rms_eps; r.H = m->H; r.T = T; r.w_router = w.router; r.n_experts = E; r.top_k = K;
    r.sel = m->d_moe_sel; r.wsel = m->d_moe_w;
    if (grouped) {
        r.counts = m->d_moe_cnt; r.lists = m->d_moe_lists; r.list_stride = kMoeGroupedTokens; r.touched = m->d_moe_touched;
        r.ticket = reinterpret_cast<unsigned*>(m->d_moe_cnt + E);  // one word behind the counts
    }
    r.local_first = e0; r.local_count = El;
    LC_TRY(launch_moe_route(r, m->stream));
    m->launches_in_call += 1;
    if (grouped) {
        GemvGroup g1;
        g1.tmaps = w.tm_gate; g1.tmaps2 = w.tm_up; g1.counts = m->d_moe_cnt + e0; g1.lists = m->d_moe_lists + (size_t)e0 * kMoeGroupedTokens;
        g1.list_stride = kMoeGroupedTokens; g1.n_experts = El; g1.top_k = K; g1.max_tokens = T; g1.x_by_token = true;
        g1.typical_tokens = (T * K + E - 1) / E;
        g1.planes = m->moe_planes_x;
        LC_TRY(launch_gemv_planes(x, norm_w, m->cfg.rms_eps, m->H, T, m->moe_planes_x, m->stream));
        GemvArgs a;
        a.w = &w.egate[0]; a.w2 = &w.eup[0]; a.x = x; a.out = m->d_moe_h; a.epi = EPI_SILU_MUL;
        a.m = std::min(T, kTokTile); a.group = &g1;
        LC_TRY(launch_qgemv(a, m->stream));
        GemvGroup g2 = g1;
        g2.tmaps = w.tm_down; g2.tmaps2 = nullptr; g2.x_by_token = false; g2.planes = m->moe_planes_h;
        // every slot's hidden row (slots of experts that live on other ranks hold stale values nobody reads)
        LC_TRY(launch_gemv_planes(m->d_moe_h, nullptr, 0.f, m->F, T * K, m->moe_planes_h, m->stream));
        GemvArgs d;
        d.w = &w.edown[0]; d.x = m->d_moe_h; d.out = m->d_moe_y; d.m = std::min(T, kTokTile); d.group = &g2;
        LC_TRY(launch_qgemv(d, m->stream));
        LC_TRY(launch_moe_combine(m->d_moe_y, m->d_moe_sel, m->d_moe_w, K, m->H, T, 0, 0, e0, El, residual, out, m->stream));
        m->launches_in_call += 5;
        return LC_OK;
    }
    (void)E;
    for (int e = 0; e < El; e++) {
        GemvArgs g;
        g.w = &w.egate[e]; g.w2 = &w.eup[e]; g.x = x; g.norm_w = norm_w; g.eps = m->cfg.rms_eps; g.out = m->d_ffn; g.epi = EPI_SILU_MUL;
        g.prep_next = true;  // the expert's down projection reads d_ffn next, without a norm
        LC_TRY(gemv_tiled(m, g, T, m->F, m->H));
        GemvArgs d;
        d.w = &w.edown[e]; d.x = m->d_ffn; d.out = m->d_moe_yall + (size_t)e * m->t_cap * m->H;
        LC_TRY(gemv_tiled(m, d, T, m->H, m->F));
    }
    LC_TRY(launch_moe_combine(m->d_moe_yall, m->d_moe_sel, m->d_moe_w, K, m->H, T, 1, (size_t)m->t_cap, e0, El, residual, out, m->stream));
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
    d.out = partial_dst(m, out);
    if (residual && (m->tp == 1 || m->rank == 0)) { d.residual = residual; d.epi = EPI_ADD_RESIDUAL; }
    if (m->tp == 1 && residual && out == m->d_hidden && l + 1 < m->L && m->layers[l + 1].attn_norm) {
        // the next layer's q/k/v product(s) read `out` through that layer's attention norm
        d.prep_next = true; d.next_norm_w = m->layers[l + 1].attn_norm; d.next_eps = m->cfg.rms_eps;
    }
    d.m = T;
    if (m->tp > 1) try_push(m, &d, T);
    return gemv_tiled(m, d, T, m->H, m->F);
}

// The handles that make up the model `m` leads: itself, or every rank of an in-process group.
std::vector<lc_model*> ranks_of(lc_model* m) {
    if (!m->members.empty()) return m->members;
    return std::vector<lc_model*>(1, m);
}

// Sum over the ranks of the partial rows the last column-cut product left, into each rank's pending destination.
int32_t reduce_ranks(lc_model* lead, size_t count) {
    if (lead->tp == 1) return LC_OK;
    std::vector<lc_model*> R = ranks_of(lead);
    if (lead->use_dist) {
        if (lead->pending_pushed) LC_TRY(dist_gather_sum(lead->pending_dst, count, lead->stream));
        else LC_TRY(dist_allreduce_sum(lead->d_part, lead->pending_dst, count, lead->stream));
    } else {
        LC_CHECK((int)R.size() == lead->tp, LC_ERR_STATE, "a model cut into %d ranks needs lc_dist_init or lc_model_group before it can run", lead->tp);
        const float* src[8]; float* dst[8];
        for (int r = 0; r < lead->tp; r++) { src[r] = R[r]->d_part; dst[r] = R[r]->pending_dst; }
        LC_TRY(launch_group_sum(src, dst, lead->tp, count, lead->stream));
    }
    for (lc_model* m : R) m->pending_dst = nullptr;
    lead->launches_in_call += 1;
    return LC_OK;
}

// The transformer layers (engine.rs:95-116) on T tokens described by d_tokens / d_tok_*, for every rank of the model.
int32_t run_layers(lc_model* lead, int T, bool decode_step) {
    std::vector<lc_model*> R = ranks_of(lead);
    for (lc_model* m : R) {
        LC_TRY(launch_embed(m->embed->typ, m->embed->view, m->embed->rows, m->embed->cols, m->d_tokens, T, m->d_hidden, m->stream));
        m->launches_in_call += 1;
    }
    const size_t count = (size_t)T * lead->H;
    for (int l = 0; l < lead->L; l++) {
        for (lc_model* m : R) LC_TRY(attention_block(m, l, m->d_hidden, m->layers[l].attn_norm, T, m->d_hidden, m->d_hidden2, decode_step));
        LC_TRY(reduce_ranks(lead, count));
        for (lc_model* m : R) LC_TRY(ffn_block(m, l, m->d_hidden2, m->layers[l].ffn_norm, T, m->d_hidden2, m->d_hidden, decode_step));
        LC_TRY(reduce_ranks(lead, count));
    }
    return LC_OK;
}

// Engine::forward (engine.rs:78-132): layers, then final norm + head on n_last rows.  identity_last:
// every token is the last of its sequence (a decode step), so no gather is needed; otherwise the rows
// listed in d_last_idx are gathered.  Logits (of this rank's vocabulary rows) land in d_logits rows row0.., greedy picks in d_next.
int32_t forward_tokens(lc_model* lead, int T, int n_last, bool identity_last, int row0) {
    LC_TRY(run_layers(lead, T, identity_last));
    std::vector<lc_model*> R = ranks_of(lead);
    for (lc_model* m : R) {
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
        if (m->tp == 1) LC_TRY(launch_argmax(m->d_logits + (size_t)row0 * m->V, m->V, n_last, m->d_next + row0, m->stream));
        else LC_TRY(launch_argmax_key(m->d_logits + (size_t)row0 * m->V, m->V, n_last, m->v0, m->d_key + row0, m->stream));
        m->launches_in_call += 1;
    }
    if (lead->tp > 1) {  // the pick over the whole vocabulary: the largest (logit, global index) key of the ranks
        if (lead->use_dist) {
            LC_TRY(dist_allreduce_max(lead->d_key, lead->d_key_max, (size_t)(row0 + n_last), lead->stream));
        } else {
            LC_CHECK((int)R.size() == lead->tp, LC_ERR_STATE, "a model cut into %d ranks needs lc_dist_init or lc_model_group before it can run", lead->tp);
            const long long* src[8]; long long* dst[8];
            for (int r = 0; r < lead->tp; r++) { src[r] = R[r]->d_key; dst[r] = R[r]->d_key_max; }
            LC_TRY(launch_group_max(src, dst, lead->tp, (size_t)(row0 + n_last), lead->stream));
        }
        for (lc_model* m : R) LC_TRY(launch_key_to_token(m->d_key_max + row0, n_last, m->d_next + row0, m->stream));
        lead->launches_in_call += 1 + (uint64_t)R.size();
    }
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
    // runs of consecutive positions of one sequence, cut into tiles of 64 tokens, for the tensor-core prefill attention
    std::vector<PrefillTile> tiles;
    for (size_t i = 0; i < T; i++) {
        if (tiles.empty() || tiles.back().n == 64 || seq[i] != seq[i - 1] || pos[i] != pos[i - 1] + 1) tiles.push_back(PrefillTile{(int32_t)i, 0, seq[i], pos[i]});
        tiles.back().n++;
    }
    m->n_tiles = (int)tiles.size();
    if (!tiles.empty()) LC_CUDA(cudaMemcpyAsync(m->d_tiles, tiles.data(), tiles.size() * sizeof(PrefillTile), cudaMemcpyHostToDevice, m->stream));
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
// The device error flag travels with a call's other results (queued before the call's synchronisation) instead of in a
// round trip of its own; flag_result() looks at what arrived.
static int32_t queue_flag_read(lc_model* m) {
    int* f = gemv_error_flag_dev();
    int* dst = reinterpret_cast<int*>(m->pin_next + m->max_seqs);
    *dst = 0;
    if (f) LC_CUDA(cudaMemcpyAsync(dst, f, sizeof(int), cudaMemcpyDeviceToHost, m->stream));
    return LC_OK;
}
static int32_t flag_result(lc_model* m) {
    const int v = *reinterpret_cast<const int*>(m->pin_next + m->max_seqs);
    if (v != 0) {
        cudaMemsetAsync(gemv_error_flag_dev(), 0, sizeof(int), m->stream);
        set_error("a device-side check failed (code %d: %s); the results of this call are not valid", v,
                  v >= 20 ? "an index outside its range" : "a bounded wait ran out");
        return LC_ERR_CUDA;
    }
    return LC_OK;
}

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
    // model parallelism: explicit in the config, or the world of lc_dist_init
    int tp = cfg->tp_size, rk = cfg->tp_rank;
    if (tp <= 0) { tp = dist_active() ? dist_world() : 1; rk = dist_active() ? dist_rank() : 0; }
    if (tp < 1 || tp > 8 || rk < 0 || rk >= tp) { delete m; set_error("tp_size %d / tp_rank %d outside 1..8 / 0..tp_size-1", tp, rk); return LC_ERR_INVALID; }
    const bool experts = cfg->n_experts > 0;
    if (tp > 1 && (cfg->num_heads % tp || cfg->num_kv_heads % tp || cfg->vocab_size % tp || (experts ? cfg->n_experts % tp : cfg->intermediate_size % tp))) {
        delete m;
        set_error("a model of %d heads / %d kv heads / vocabulary %d / %s %d cannot be cut into %d ranks", cfg->num_heads, cfg->num_kv_heads,
                  cfg->vocab_size, experts ? "experts" : "FFN rows", experts ? cfg->n_experts : cfg->intermediate_size, tp);
        return LC_ERR_INVALID;
    }
    m->tp = tp; m->rank = rk;
    m->cfg.tp_size = tp; m->cfg.tp_rank = rk;
    m->use_dist = tp > 1 && dist_active() && dist_world() == tp && dist_rank() == rk;
    m->H = cfg->hidden_size; m->L = cfg->num_layers; m->nh = cfg->num_heads / tp; m->nkv = cfg->num_kv_heads / tp;
    m->hd = m->H / cfg->num_heads; m->F = experts ? cfg->intermediate_size : cfg->intermediate_size / tp; m->V = cfg->vocab_size / tp;
    m->v0 = m->V * rk;
    m->El = experts ? cfg->n_experts / tp : 0; m->e0 = m->El * rk;
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

// Registers a tensor given by its WHOLE dims and allocates this rank's part of it.  *out_t = null when the rank keeps
// nothing of it (an expert of another rank).
static int32_t put_tensor(lc_model* m, const char* name, uint32_t typ, const uint64_t* dims, int32_t ndims, DevTensor** out_t, ShardPlan* out_plan,
                          QuantGeom* out_geom) {
    LC_TRY(check_model(m, false));
    LC_CHECK(!m->finalized, LC_ERR_STATE, "model already finalized");
    LC_CHECK(name && dims && ndims >= 1 && ndims <= 4, LC_ERR_INVALID, "set_tensor: bad argument");
    QuantGeom g;
    LC_CHECK(quant_geom(typ, &g), LC_ERR_UNSUPPORTED, "tensor %s: unsupported ggml type %u", name, typ);
    LC_CHECK(dims[0] % g.block_elems == 0, LC_ERR_INVALID, "tensor %s: row length %llu is not a whole number of blocks", name,
             (unsigned long long)dims[0]);
    std::string key = canonical_name(name);
    ShardPlan pl;
    LC_TRY(shard_plan(m->cfg, m->tp, m->rank, key, dims, ndims, &pl));
    *out_plan = pl;
    *out_geom = g;
    *out_t = nullptr;
    if (pl.kind == SHARD_NONE) return LC_OK;
    if (pl.kind == SHARD_COLS)
        LC_CHECK(pl.count % g.block_elems == 0 && pl.first % g.block_elems == 0, LC_ERR_INVALID,
                 "tensor %s: a column part of %llu elements is not a whole number of %u-element blocks", name, (unsigned long long)pl.count, g.block_elems);
    uint64_t total_rows = 1;
    for (int i = 1; i < ndims; i++) total_rows *= dims[i];
    DevTensor t;
    t.typ = typ;
    t.dims.assign(dims, dims + ndims);
    t.cols = pl.kind == SHARD_COLS ? pl.count : dims[0];  // loader.rs:155: GGUF dims are fastest-first, rows = dims[1]
    t.rows = pl.kind == SHARD_ROWS ? pl.count : total_rows;
    t.nbytes = lc_tensor_bytes(typ, t.rows * t.cols);
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
    ShardPlan pl;
    QuantGeom g;
    LC_TRY(put_tensor(m, name, typ, dims, ndims, &t, &pl, &g));
    size_t count = 1;
    for (int i = 0; i < ndims; i++) count *= dims[i];
    LC_CHECK(lc_tensor_bytes(typ, count) == nbytes, LC_ERR_INVALID, "tensor %s: %zu bytes given, %zu expected", name, nbytes, lc_tensor_bytes(typ, count));
    if (!t) return LC_OK;
    const size_t full_row_bytes = (size_t)dims[0] / g.block_elems * g.block_bytes;
    const uint8_t* src = (const uint8_t*)bytes;
    if (pl.kind == SHARD_COLS) {
        const size_t part = (size_t)pl.count / g.block_elems * g.block_bytes, off = (size_t)pl.first / g.block_elems * g.block_bytes;
        LC_CUDA(cudaMemcpy2DAsync(t->dev, part, src + off, full_row_bytes, part, t->rows, cudaMemcpyHostToDevice, m->stream));
    } else {
        const size_t off = pl.kind == SHARD_ROWS ? (size_t)pl.first * full_row_bytes : 0;
        LC_CUDA(cudaMemcpyAsync(t->dev, src + off, t->nbytes, cudaMemcpyHostToDevice, m->stream));
    }
    LC_CUDA(cudaStreamSynchronize(m->stream));
    return LC_OK;
}

int32_t lc_model_synth_tensor(lc_model* m, const char* name, uint32_t typ, const uint64_t* dims, int32_t ndims, uint64_t seed,
                              float sigma) {
    LC_TRY(check_model(m, false));
    DeviceGuard dg(m->device);
    DevTensor* t = nullptr;
    ShardPlan pl;
    QuantGeom g;
    LC_TRY(put_tensor(m, name, typ, dims, ndims, &t, &pl, &g));
    if (!t) return LC_OK;
    std::string key = canonical_name(name);
    const size_t row_blocks = (size_t)dims[0] / g.block_elems;
    const size_t row0 = pl.kind == SHARD_ROWS ? (size_t)pl.first : 0;
    const size_t blk0 = pl.kind == SHARD_COLS ? (size_t)pl.first / g.block_elems : 0;
    LC_TRY(launch_synth_part(typ, seed, lcs_fnv1a(key.c_str()), sigma, row_blocks, row0, t->rows, blk0, t->cols / g.block_elems, t->dev, m->stream));
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
    DevTensor& t = it->second;  // this rank's experts e0 .. e0 + El - 1 of the stacked tensor
    LC_CHECK((int)t.cols == k && t.rows == (size_t)n * m->El, LC_ERR_INVALID, "tensor %s is [%zu x %zu], expected [%d x %d] per expert",
             stacked.c_str(), t.rows, t.cols, n, k);
    QuantGeom g;
    LC_CHECK(quant_geom(t.typ, &g), LC_ERR_UNSUPPORTED, "tensor %s: unsupported type", stacked.c_str());
    const size_t row_bytes = (size_t)k / g.block_elems * g.block_bytes;
    return qweight_init(w, t.typ, (const uint8_t*)t.view + (size_t)(e - m->e0) * n * row_bytes, n, k);
}

static int32_t finalize_experts(lc_model* m, int l) {
    LayerW& w = m->layers[l];
    const int E = m->cfg.n_experts, H = m->H, F = m->F;
    const std::string p = "blk." + std::to_string(l) + ".";
    LC_TRY(gain_f32(m, p + "ffn_gate_inp.weight", E * H, &w.router));
    const int El = m->El;  // the experts this rank holds: e0 .. e0 + El - 1, stored at 0 .. El - 1
    w.egate.resize(El); w.eup.resize(El); w.edown.resize(El);
    bool q4k = true;
    for (int e = 0; e < El; e++) {
        LC_TRY(expert_weight(m, l, m->e0 + e, "ffn_gate", F, H, &w.egate[e]));
        LC_TRY(expert_weight(m, l, m->e0 + e, "ffn_up", F, H, &w.eup[e]));
        LC_TRY(expert_weight(m, l, m->e0 + e, "ffn_down", H, F, &w.edown[e]));
        LC_CHECK(w.egate[e].typ == w.eup[e].typ, LC_ERR_UNSUPPORTED, "layer %d expert %d: gate/up projections have different quant types", l, m->e0 + e);
        for (const QWeight* q : {&w.egate[e], &w.eup[e], &w.edown[e]}) q4k = q4k && q->typ == LC_TYPE_Q4_K && q->has_tmap;
    }
    w.grouped_ok = q4k && qgemv_mma_supports(H) && qgemv_mma_supports(F);
    if (w.grouped_ok) {
        std::vector<unsigned char> host((size_t)El * 128);
        const std::vector<QWeight>* sets[3] = {&w.egate, &w.eup, &w.edown};
        void** dst[3] = {&w.tm_gate, &w.tm_up, &w.tm_down};
        for (int i = 0; i < 3; i++) {
            for (int e = 0; e < El; e++) memcpy(&host[(size_t)e * 128], (*sets[i])[e].tmap, 128);
            LC_TRY(dalloc((uint8_t**)dst[i], host.size()));
            m->owned.push_back(*dst[i]);
            LC_CUDA(cudaMemcpyAsync(*dst[i], host.data(), host.size(), cudaMemcpyHostToDevice, m->stream));
            LC_CUDA(cudaStreamSynchronize(m->stream));
        }
    }
    uint64_t each = 0;
    for (const QWeight* q : {&w.egate[0], &w.eup[0], &w.edown[0]}) each += (uint64_t)q->n * q->row_bytes;
    m->expert_bytes_each = each;
    m->expert_bytes_all += each * El;
    (void)E;
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
    if (m->tensors.count("output.weight")) {
        LC_TRY(weight_of(m, "output.weight", V, H, &m->head, nullptr));
    } else {  // tied: this rank's vocabulary rows of the (whole) embedding table
        const DevTensor& e = *m->embed;
        LC_CHECK((int)e.rows == m->cfg.vocab_size, LC_ERR_INVALID, "token_embd.weight has %zu rows, vocabulary is %d", e.rows, m->cfg.vocab_size);
        const size_t row_bytes = e.nbytes / e.rows;
        LC_TRY(qweight_init(&m->head, e.typ, (const uint8_t*)e.view + (size_t)m->v0 * row_bytes, V, H));
    }

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
    LC_TRY(dalloc(&m->d_tok_rope, T)); LC_TRY(dalloc(&m->d_last_idx, T)); LC_TRY(dalloc(&m->d_tiles, T));
    LC_TRY(dalloc(&m->d_hidden, (size_t)T * H)); LC_TRY(dalloc(&m->d_hidden2, (size_t)T * H));
    LC_TRY(dalloc(&m->d_qkv, (size_t)T * m->nqkv)); LC_TRY(dalloc(&m->d_attn, (size_t)T * nq));
    LC_TRY(dalloc(&m->d_ffn, (size_t)T * F));
    LC_TRY(qgemm_workspace_alloc(&m->gemm_ws, T, std::max(std::max(H, F), nq)));
    if (m->any_unfused_qkv) LC_TRY(dalloc(&m->d_qkv_parts, (size_t)T * m->nqkv));
    if (m->cfg.n_experts > 0) {
        const int E = m->cfg.n_experts, K = m->cfg.top_k;
        LC_TRY(dalloc(&m->d_moe_sel, (size_t)T * K)); LC_TRY(dalloc(&m->d_moe_w, (size_t)T * K));
        LC_TRY(dalloc(&m->d_moe_cnt, (size_t)E + 1)); LC_TRY(dalloc(&m->d_moe_lists, (size_t)E * kMoeGroupedTokens));
        LC_CUDA(cudaMemsetAsync(m->d_moe_cnt, 0, ((size_t)E + 1) * sizeof(int32_t), m->stream));  // the word behind the counts is the router's ticket
        LC_TRY(dalloc(&m->d_moe_h, (size_t)kMoeGroupedTokens * K * F)); LC_TRY(dalloc(&m->d_moe_y, (size_t)kMoeGroupedTokens * K * H));
        LC_TRY(dalloc(&m->d_moe_yall, (size_t)E * T * H));
        auto planes_alloc = [&](GemvPlanes* pl, size_t rows, int k) -> int32_t {
            const size_t units = rows * (size_t)(k / 256);
            if (units == 0) return LC_OK;
            LC_TRY(dalloc(&pl->planes, units * 768)); LC_TRY(dalloc(&pl->sxf, units * 8)); LC_TRY(dalloc(&pl->inv2s, units));
            return LC_OK;
        };
        LC_TRY(planes_alloc(&m->moe_planes_x, (size_t)kMoeGroupedTokens, H));
        LC_TRY(planes_alloc(&m->moe_planes_h, (size_t)kMoeGroupedTokens * K, F));
        LC_TRY(dalloc(&m->d_moe_touched, 1));
        LC_CUDA(cudaMemsetAsync(m->d_moe_touched, 0, 8, m->stream));
    }
    LC_TRY(dalloc(&m->d_last, (size_t)m->max_seqs * H)); LC_TRY(dalloc(&m->d_logits, (size_t)m->max_seqs * V));
    LC_TRY(dalloc(&m->d_next, m->max_seqs)); LC_TRY(dalloc(&m->d_step_ctr, 1));
    if (m->tp > 1) {
        // partial rows of the column-cut products and the greedy-pick keys: in the buffers the other ranks can read when the
        // ranks are processes (a collective call: every rank finalizes its model at the same point), else plain memory
        LC_TRY(dalloc(&m->d_key_max, (size_t)m->max_seqs));
        LC_TRY(dalloc(&m->d_key, (size_t)m->max_seqs));
        LC_TRY(dalloc(&m->d_part, (size_t)T * H));
        if (m->use_dist) {  // a collective call: every rank finalizes its model at the same point
            LC_TRY(dist_setup());
            LC_TRY(dalloc(&m->d_logits_all, (size_t)m->max_seqs * m->cfg.vocab_size));
        }
    }
    size_t sc = 16;
    for (int t = 1; t <= T; t++) sc = std::max(sc, attention_scratch_bytes(t, m->nh, m->hd, m->cfg.max_seq_len));
    m->attn_scratch_bytes = sc;
    LC_TRY(dalloc((uint8_t**)&m->d_attn_scratch, sc));
    LC_TRY(dalloc(&m->d_attn_counters, (size_t)T * m->nh));
    LC_CUDA(cudaMemsetAsync(m->d_attn_counters, 0, (size_t)T * m->nh * sizeof(int), m->stream));
    LC_CUDA(cudaHostAlloc((void**)&m->pin_tokens, (size_t)m->max_seqs * 8, cudaHostAllocDefault));
    LC_CUDA(cudaHostAlloc((void**)&m->pin_next, ((size_t)m->max_seqs + 1) * 8, cudaHostAllocDefault));  // + one word: the device error flag of a call
    LC_CUDA(cudaHostAlloc((void**)&m->pin_logits, (size_t)m->max_seqs * m->cfg.vocab_size * 4, cudaHostAllocDefault));
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
    if (m->leader) {  // leaving a group: the leader must not drive this handle any more
        auto& mem = m->leader->members;
        for (lc_model* x : mem) if (x != m->leader) x->leader = nullptr;
        mem.clear();
    }
    for (lc_model* x : m->members) if (x != m) x->leader = nullptr;
    void* bufs[] = {m->d_tiles, m->d_part, m->d_key, m->d_key_max, m->d_logits_all, m->d_moe_sel, m->d_moe_w, m->d_moe_cnt, m->d_moe_lists, m->d_moe_h, m->d_moe_y, m->d_moe_yall, m->d_moe_touched,
                    m->moe_planes_x.planes, m->moe_planes_x.sxf, m->moe_planes_x.inv2s, m->moe_planes_h.planes, m->moe_planes_h.sxf, m->moe_planes_h.inv2s,
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

// A handle that another handle drives (rank > 0 of an in-process group) takes no model-level calls of its own.
static int32_t check_drivable(const lc_model* m) {
    LC_CHECK(m->leader == nullptr, LC_ERR_STATE, "this handle is rank %d of a group: make the call on the group's first handle", m->rank);
    return LC_OK;
}

int32_t lc_model_group(lc_model** handles, int32_t n) {
    LC_CHECK(handles && n >= 2 && n <= 8, LC_ERR_INVALID, "lc_model_group: 2..8 handles");
    for (int r = 0; r < n; r++) {
        lc_model* m = handles[r];
        LC_TRY(check_model(m, true));
        LC_CHECK(m->tp == n && m->rank == r && !m->use_dist && m->members.empty() && !m->leader, LC_ERR_INVALID,
                 "lc_model_group: handle %d must be rank %d of %d, not yet grouped and not a rank of lc_dist_init", r, r, n);
        LC_CHECK(m->device == handles[0]->device && m->H == handles[0]->H && m->L == handles[0]->L && m->t_cap == handles[0]->t_cap &&
                     m->max_seqs == handles[0]->max_seqs && m->cfg.max_seq_len == handles[0]->cfg.max_seq_len,
                 LC_ERR_INVALID, "lc_model_group: the handles must be parts of one model on one device");
    }
    handles[0]->members.assign(handles, handles + n);
    for (int r = 1; r < n; r++) handles[r]->leader = handles[0];
    return LC_OK;
}

int32_t lc_shard_plan(const lc_model_config* cfg, const char* name, const uint64_t* dims, int32_t ndims, int32_t* kind, uint64_t* first,
                      uint64_t* count) {
    LC_CHECK(cfg && name && dims && ndims >= 1 && ndims <= 4 && kind && first && count, LC_ERR_INVALID, "lc_shard_plan: bad argument");
    ShardPlan pl;
    LC_TRY(shard_plan(*cfg, cfg->tp_size, cfg->tp_rank, canonical_name(name), dims, ndims, &pl));
    *kind = pl.kind; *first = pl.first; *count = pl.count;
    return LC_OK;
}

int32_t lc_kv_clear(lc_model* lead, int32_t seq_id) {
    LC_TRY(check_model(lead, true));
    LC_TRY(check_drivable(lead));
    LC_CHECK(seq_id >= -1 && seq_id < lead->max_seqs, LC_ERR_INVALID, "sequence id %d outside 0..%d", seq_id, lead->max_seqs - 1);
    for (lc_model* m : ranks_of(lead)) {
        for (int s = 0; s < m->max_seqs; s++) {
            if (seq_id >= 0 && s != seq_id) continue;
            for (int p : m->seq_pages[s]) m->free_pages.push_back(p);
            m->seq_pages[s].clear();
            m->seq_len[s] = 0;
        }
        m->meta_valid = false;
    }
    return LC_OK;
}

int32_t lc_kv_memory_bytes(const lc_model* m, uint64_t* out) {
    LC_TRY(check_model(m, true));
    LC_CHECK(out, LC_ERR_INVALID, "null output");
    uint64_t tokens = 0;
    for (int v : m->seq_len) tokens += v;
    *out = tokens * (uint64_t)m->L * 2 * m->cfg.num_kv_heads * m->hd * m->kv_elt;  // cache/mod.rs:80-84, over all ranks
    return LC_OK;
}

int32_t lc_kv_length(const lc_model* m, int32_t seq_id, int32_t* out) {
    LC_TRY(check_model(m, true));
    LC_CHECK(out && seq_id >= 0 && seq_id < m->max_seqs, LC_ERR_INVALID, "bad sequence id %d", seq_id);
    *out = m->seq_len[seq_id];
    return LC_OK;
}

// The logits rows [0, n_rows) of the whole vocabulary on the host: a whole model copies them; a cut model puts the ranks'
// vocabulary slices side by side (an all-gather when the ranks are processes).
static int32_t fetch_logits(lc_model* lead, int n_rows, float* host_out) {
    const int Vfull = lead->cfg.vocab_size, Vl = lead->V;
    if (lead->tp == 1) {
        LC_CUDA(cudaMemcpyAsync(lead->pin_logits, lead->d_logits, (size_t)n_rows * Vfull * 4, cudaMemcpyDeviceToHost, lead->stream));
        LC_CUDA(cudaStreamSynchronize(lead->stream));
        memcpy(host_out, lead->pin_logits, (size_t)n_rows * Vfull * 4);
        return LC_OK;
    }
    if (lead->use_dist) {
        LC_TRY(dist_allgather(lead->d_logits, lead->d_logits_all, (size_t)n_rows * Vl * 4, lead->stream));
        LC_CUDA(cudaMemcpyAsync(lead->pin_logits, lead->d_logits_all, (size_t)n_rows * Vfull * 4, cudaMemcpyDeviceToHost, lead->stream));
        LC_CUDA(cudaStreamSynchronize(lead->stream));
        for (int r = 0; r < lead->tp; r++)
            for (int row = 0; row < n_rows; row++)
                memcpy(host_out + (size_t)row * Vfull + (size_t)r * Vl, lead->pin_logits + ((size_t)r * n_rows + row) * Vl, (size_t)Vl * 4);
        return LC_OK;
    }
    std::vector<lc_model*> R = ranks_of(lead);
    for (int r = 0; r < lead->tp; r++)
        LC_CUDA(cudaMemcpy2DAsync(lead->pin_logits + (size_t)r * Vl, (size_t)Vfull * 4, R[r]->d_logits, (size_t)Vl * 4, (size_t)Vl * 4, (size_t)n_rows,
                                  cudaMemcpyDeviceToHost, lead->stream));
    LC_CUDA(cudaStreamSynchronize(lead->stream));
    memcpy(host_out, lead->pin_logits, (size_t)n_rows * Vfull * 4);
    return LC_OK;
}

int32_t lc_forward_batch(lc_model* lead, int32_t n_seqs, const int32_t* seq_ids, const int64_t* tokens, const int32_t* n_tokens,
                         float* logits_out, int64_t* next_out) {
    LC_TRY(check_model(lead, true));
    LC_TRY(check_drivable(lead));
    LC_CHECK(n_seqs >= 1 && n_seqs <= lead->max_seqs && seq_ids && tokens && n_tokens, LC_ERR_INVALID, "forward_batch: bad argument");
    DeviceGuard dg(lead->device);
    std::vector<lc_model*> R = ranks_of(lead);
    int total = 0, longest = 0;
    for (int i = 0; i < n_seqs; i++) {
        LC_CHECK(seq_ids[i] >= 0 && seq_ids[i] < lead->max_seqs, LC_ERR_INVALID, "sequence id %d outside 0..%d", seq_ids[i], lead->max_seqs - 1);
        for (int j = 0; j < i; j++) LC_CHECK(seq_ids[j] != seq_ids[i], LC_ERR_INVALID, "sequence id %d listed twice", seq_ids[i]);
        LC_CHECK(n_tokens[i] >= 1, LC_ERR_INVALID, "sequence %d has no tokens in this call", seq_ids[i]);
        for (lc_model* m : R) LC_TRY(ensure_pages(m, seq_ids[i], m->seq_len[seq_ids[i]] + n_tokens[i]));
        total += n_tokens[i];
        longest = std::max(longest, n_tokens[i]);
    }
    for (lc_model* m : R) LC_TRY(sync_page_table(m));
    if (longest == 1) {
        // a decode step: token ids in (pinned staging), graph replay, picks and logits out
        for (lc_model* m : R) {
            LC_TRY(reserve_out_tokens(m, (size_t)n_seqs));
            LC_TRY(stage_decode_meta(m, n_seqs, seq_ids, tokens));
            LC_CUDA(cudaMemsetAsync(m->d_step_ctr, 0, 4, m->stream));
        }
        LC_TRY(run_decode_steps(lead, n_seqs, 1));
        if (next_out) LC_CUDA(cudaMemcpyAsync(lead->pin_next, lead->d_next, (size_t)n_seqs * 8, cudaMemcpyDeviceToHost, lead->stream));
        LC_TRY(queue_flag_read(lead));
        if (logits_out) LC_TRY(fetch_logits(lead, n_seqs, logits_out));
        LC_CUDA(cudaStreamSynchronize(lead->stream));
        if (next_out) memcpy(next_out, lead->pin_next, (size_t)n_seqs * 8);
        for (lc_model* m : R) { after_decode_steps(m, n_seqs, seq_ids, 1); finish_call(m); }
        return flag_result(lead);
    }
    for (lc_model* m : R) m->meta_valid = false;
    // Rotary index = position inside the CALL (reference mode, attention.rs:13-21) or the cache position.
    if (total <= lead->t_cap) {
        std::vector<int64_t> tok; std::vector<int32_t> seq, pos, rope, last;
        int off = 0;
        for (int i = 0; i < n_seqs; i++) {
            for (int t = 0; t < n_tokens[i]; t++) {
                int p = lead->seq_len[seq_ids[i]] + t;
                tok.push_back(tokens[off + t]); seq.push_back(seq_ids[i]); pos.push_back(p);
                rope.push_back(lead->cfg.rope_mode ? p : t);
            }
            off += n_tokens[i];
            last.push_back(off - 1);
        }
        for (lc_model* m : R) LC_TRY(upload_meta(m, tok, seq, pos, rope, last));
        LC_TRY(forward_tokens(lead, total, n_seqs, total == n_seqs, 0));
    } else {
        // long prompts: one sequence after the other, each in chunks of t_cap tokens over its growing cache
        int off = 0;
        for (int i = 0; i < n_seqs; i++) {
            for (int c0 = 0; c0 < n_tokens[i]; c0 += lead->t_cap) {
                int T = std::min(lead->t_cap, n_tokens[i] - c0);
                std::vector<int64_t> tok(T); std::vector<int32_t> seq(T, seq_ids[i]), pos(T), rope(T), last(1, T - 1);
                for (int t = 0; t < T; t++) {
                    tok[t] = tokens[off + c0 + t];
                    pos[t] = lead->seq_len[seq_ids[i]] + c0 + t;
                    rope[t] = lead->cfg.rope_mode ? pos[t] : (c0 + t);
                }
                for (lc_model* m : R) LC_TRY(upload_meta(m, tok, seq, pos, rope, last));
                if (c0 + T == n_tokens[i]) LC_TRY(forward_tokens(lead, T, 1, T == 1, i));
                else LC_TRY(run_layers(lead, T, false));
            }
            off += n_tokens[i];
        }
    }
    for (lc_model* m : R)
        for (int i = 0; i < n_seqs; i++) m->seq_len[seq_ids[i]] += n_tokens[i];
    if (next_out) LC_CUDA(cudaMemcpyAsync(lead->pin_next, lead->d_next, (size_t)n_seqs * 8, cudaMemcpyDeviceToHost, lead->stream));
    if (logits_out) LC_TRY(fetch_logits(lead, n_seqs, logits_out));
    LC_CUDA(cudaStreamSynchronize(lead->stream));
    if (next_out) memcpy(next_out, lead->pin_next, (size_t)n_seqs * 8);
    for (lc_model* m : R) {
        m->ctr.forward_calls += 1;
        m->ctr.tokens_prefilled += total;
        uint64_t used = 0;
        for (auto& pg : m->seq_pages) used += pg.size();
        m->ctr.kv_pages_in_use = used;
        finish_call(m);
    }
    return check_device_flag(lead);
}

int32_t lc_forward(lc_model* m, const int64_t* tokens, int32_t n, float* logits_out) {
    LC_CHECK(tokens && n >= 1 && logits_out, LC_ERR_INVALID, "lc_forward: bad argument");
    int32_t seq = 0;
    return lc_forward_batch(m, 1, &seq, tokens, &n, logits_out, nullptr);
}

// Queues `steps` greedy decode steps for the n_seqs sequences whose metadata is on the device.  The first
// step of a new batch width runs eagerly (it sets kernel attributes), then one step is captured into a
// CUDA graph that later steps replay.  For an in-process group the one graph holds every rank's kernels.
static int32_t run_decode_steps(lc_model* m, int n_seqs, int steps) {
    std::vector<lc_model*> R = ranks_of(m);
    auto one_step = [&]() -> int32_t {
        LC_TRY(forward_tokens(m, n_seqs, n_seqs, true, 0));
        for (lc_model* r : R) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(1);
            cfg.blockDim = dim3(std::max(32, (n_seqs + 31) / 32 * 32));
            cfg.stream = r->stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            LC_CUDA(cudaLaunchKernelEx(&cfg, advance_kernel, (const int64_t*)r->d_next, r->d_tokens, r->d_tok_pos, r->d_tok_rope, (int)n_seqs,
                                       (int)r->cfg.rope_mode, r->d_out_tokens, r->d_step_ctr));
            r->launches_in_call += 1;
        }
        return LC_OK;
    };
    auto launches_now = [&]() { uint64_t t = 0; for (lc_model* r : R) t += r->launches_in_call; return t; };
    static const bool no_graph = getenv("LC_NO_GRAPH") != nullptr;
    cudaGraphExec_t exec = nullptr;
    int done_steps = 0;
    auto it = m->decode_graphs.find(n_seqs);
    if (it != m->decode_graphs.end()) exec = it->second;
    if (!exec && !no_graph) {
        uint64_t before = launches_now();
        LC_TRY(one_step());
        m->graph_nodes = (int)(launches_now() - before);
        done_steps = 1;
        cudaGraph_t graph = nullptr;
        if (cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
            std::vector<uint64_t> keep;
            for (lc_model* r : R) keep.push_back(r->launches_in_call);
            int32_t st = one_step();
            for (size_t i = 0; i < R.size(); i++) R[i]->launches_in_call = keep[i];
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
    lc_model* owner = m->leader ? m->leader : m;  // the graphs bake this pointer in; a group's graphs live on its first handle
    for (auto& g : owner->decode_graphs) cudaGraphExecDestroy(g.second);
    owner->decode_graphs.clear();
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
                                                                                           : (double)m->L * m->El;
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

int32_t lc_decode_loop(lc_model* lead, int32_t n_seqs, const int32_t* seq_ids, const int64_t* first_tokens, int32_t steps,
                       int64_t* out_tokens, float* out_ms) {
    LC_TRY(check_model(lead, true));
    LC_TRY(check_drivable(lead));
    LC_CHECK(n_seqs >= 1 && n_seqs <= lead->max_seqs && seq_ids && first_tokens && steps >= 1, LC_ERR_INVALID, "decode_loop: bad argument");
    DeviceGuard dg(lead->device);
    std::vector<lc_model*> R = ranks_of(lead);
    const size_t need = (size_t)steps * n_seqs;
    for (lc_model* m : R) {
        for (int i = 0; i < n_seqs; i++) {
            LC_CHECK(seq_ids[i] >= 0 && seq_ids[i] < m->max_seqs, LC_ERR_INVALID, "sequence id %d outside 0..%d", seq_ids[i], m->max_seqs - 1);
            for (int j = 0; j < i; j++) LC_CHECK(seq_ids[j] != seq_ids[i], LC_ERR_INVALID, "sequence id %d listed twice", seq_ids[i]);
            LC_TRY(ensure_pages(m, seq_ids[i], m->seq_len[seq_ids[i]] + steps));  // pages for the whole loop up front
        }
        LC_TRY(sync_page_table(m));
        LC_TRY(reserve_out_tokens(m, need));
        LC_TRY(stage_decode_meta(m, n_seqs, seq_ids, first_tokens));
        LC_CUDA(cudaMemsetAsync(m->d_step_ctr, 0, 4, m->stream));
    }
    LC_CUDA(cudaEventRecord(lead->ev0, lead->stream));
    LC_TRY(run_decode_steps(lead, n_seqs, steps));
    LC_CUDA(cudaEventRecord(lead->ev1, lead->stream));
    LC_CUDA(cudaEventSynchronize(lead->ev1));
    float ms = 0.f;
    LC_CUDA(cudaEventElapsedTime(&ms, lead->ev0, lead->ev1));
    if (out_ms) *out_ms = ms;
    if (out_tokens) {
        LC_CUDA(cudaMemcpyAsync(out_tokens, lead->d_out_tokens, need * 8, cudaMemcpyDeviceToHost, lead->stream));
        LC_CUDA(cudaStreamSynchronize(lead->stream));
    }
    for (lc_model* m : R) { after_decode_steps(m, n_seqs, seq_ids, steps); finish_call(m); }
    return check_device_flag(lead);
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

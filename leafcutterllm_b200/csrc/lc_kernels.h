// Internal launch interface: every function queues kernels on `s` and takes
// DEVICE pointers.  The C ABI (host pointers) and the engine both sit on these.
#pragma once
#include "lc_common.cuh"

namespace lc {

// ---- dequant.cu ----
int32_t launch_dequant(uint32_t typ, const void* w, size_t n_elems, float* out, cudaStream_t s);
// sampler::sample_top_p with the caller's uniform draw (sampler.cu); the _sync form reads the token back and takes the
// greedy branch for temperature <= 0.  seeded_uniform: draw `index` of a seeded generation, in [0, 1) on the 2^-24 grid.
int32_t launch_sample_top_p(const float* logits_dev, size_t n, float temperature, float top_p, float u, int64_t* token_dev, cudaStream_t s);
int32_t sample_top_p_sync(const float* logits_dev, size_t n, float temperature, float top_p, float u, int64_t* token_host, cudaStream_t s);
float seeded_uniform(uint64_t seed, uint64_t index);
// Block-scale scan (scan.cu): geometry of every block type the reference's type table knows and how its scales are
// read; the launch adds the number of bad blocks to one 64-bit word on the device.
bool scan_geom(uint32_t typ, uint32_t* block_elems, uint32_t* block_bytes, int* kind);
int32_t launch_scan_scales(uint32_t typ, const void* raw_dev, size_t n_blocks, unsigned long long* counter_dev, cudaStream_t s);
// Adds to *count the number of elements that dequantise to NaN / Inf / |v| > 100
// (the condition of rust/src/model/loader.rs:241-249).
int32_t launch_sanity_scan(uint32_t typ, const void* w, size_t n_elems, unsigned long long* count, cudaStream_t s);
// One f32 row of a quantised [rows, cols] tensor per token id (embedding gather,
// rust/src/inference/engine.rs:134-144; id outside [0, rows) -> zero row).
int32_t launch_embed(uint32_t typ, const void* w, size_t rows, size_t cols, const int64_t* ids, int n, float* out,
                     cudaStream_t s);

// ---- ops.cu ----
int32_t launch_vec_add(const float* a, const float* b, size_t n, float* o, cudaStream_t s);
int32_t launch_vec_mul(const float* a, const float* b, size_t n, float* o, cudaStream_t s);
int32_t launch_vec_scale(const float* a, float sc, size_t n, float* o, cudaStream_t s);
int32_t launch_vec_scale_mul(const float* a, float sc, const float* b, size_t n, float* o, cudaStream_t s);
int32_t launch_silu(const float* x, size_t n, float* o, cudaStream_t s);
int32_t launch_silu_mul(const float* gate, const float* up, size_t n, float* o, cudaStream_t s);
int32_t launch_rms_norm(const float* x, const float* w, float eps, size_t hidden, size_t rows, float* o, cudaStream_t s);
int32_t launch_softmax(const float* x, size_t hidden, size_t rows, float* o, cudaStream_t s);
int32_t launch_sum_sq(const float* x, size_t n, float* out1, cudaStream_t s);
int32_t launch_matmul_f32(const float* a, const float* b, size_t m, size_t k, size_t n, float* c, cudaStream_t s);
int32_t launch_q8_0_shard(const float* a, const float* scales, const int8_t* qs, size_t m, size_t k, size_t n, float* c,
                          cudaStream_t s);
int32_t launch_q4_0_shard(const float* a, const float* scales, const uint8_t* qs, size_t m, size_t k, size_t n, float* c,
                          cudaStream_t s);
int32_t launch_rope(float* x, size_t seq, size_t heads, size_t hd, float theta, const int32_t* pos0_dev, int32_t pos0,
                    cudaStream_t s);
// Greedy pick per row of v[rows, n]: last index among equal maxima under the total order of
// f32 (rust/src/inference/sampler.rs:6-10).
int32_t launch_argmax(const float* v, size_t n, size_t rows, int64_t* out, cudaStream_t s);

// ---- qgemv.cu ----
// A quantised weight matrix resident on the device: `n` output rows of `k`
// inputs, raw GGUF blocks, rows contiguous.
struct QWeight {
    const void* data = nullptr;
    uint32_t typ = 0;
    int n = 0, k = 0;
    size_t row_bytes = 0;
    alignas(64) unsigned char tmap[128];      // CUtensorMap for the TMA-staged kernels: box = one 256-element unit x 32 rows
    alignas(64) unsigned char tmap_wide[128]; // the same tensor with a box of 128 rows (tcgen05 kernel)
    bool has_tmap = false;
};
int32_t qweight_init(QWeight* w, uint32_t typ, const void* data_dev, int n, int k);

enum GemvEpilogue { EPI_STORE = 0, EPI_ADD_RESIDUAL = 1, EPI_SILU_MUL = 2 };
// The experts of one mixture-of-experts layer as ONE product launch (Q4_K experts of equal shape).  The router leaves,
// per expert, how many (token, choice) slots it received and their list (slot = token * top_k + choice, ascending);
// the product of expert e reads the input row of each of its slots (row slot / top_k when x_by_token, else row slot)
// and writes the result to row `slot` of out.  All pointers are device memory.
// Activations of a grouped launch, written once per call by launch_gemv_planes and read by every CTA of the launch: per row
// and 256-element unit the three balanced byte planes of the 24-bit fixed point (768 bytes), the eight sub-block sums and
// the unit's 2^-s.
struct GemvPlanes {
    unsigned char* planes = nullptr;  // [rows][k / 256][8][3][32]
    float* sxf = nullptr;             // [rows][k / 256][8]
    float* inv2s = nullptr;           // [rows][k / 256]
};
inline size_t gemv_planes_bytes(size_t rows, int k) { return rows * (size_t)(k / 256) * 768; }
int32_t launch_gemv_planes(const float* x, const float* norm_w, float eps, int k, int rows, const GemvPlanes& out, cudaStream_t s);
struct GemvGroup {
    const void* tmaps = nullptr;    // [n_experts] tensor maps (128 bytes each) of the first matrix
    const void* tmaps2 = nullptr;   // EPI_SILU_MUL: those of the `up` matrices
    const int32_t* counts = nullptr;
    const int32_t* lists = nullptr; // [n_experts][list_stride]
    int list_stride = 0, n_experts = 0, top_k = 0;
    int max_tokens = 0;             // most slots any expert can receive in this call (= tokens of the call)
    int typical_tokens = 0;         // what an expert receives on average (tokens * top_k / experts, rounded up); 0 = unknown
    bool x_by_token = false;        // the planes are per token (row = slot / top_k) rather than per slot
    GemvPlanes planes;              // the launch's activations (GemvArgs.x / norm_w are not read)
};
// A product whose output rows are one rank's share of a sum over the ranks can write them straight into every rank's
// buffer as tagged words (dist.cu): word tk * n + row of row `rank`, slot (sum number) & 1, sum number = *epoch + 1.
struct GemvPush {
    unsigned long long* peer[8] = {};
    const unsigned* epoch = nullptr;
    int world = 0, rank = 0, row_words = 0;
};
struct GemvArgs {
    const QWeight* w = nullptr;   // first matrix
    const QWeight* w2 = nullptr;  // EPI_SILU_MUL: the `up` matrix (w is `gate`)
    const float* x = nullptr;     // [m, k]
    int m = 1;
    float* out = nullptr;         // [m, n]
    const float* residual = nullptr;  // EPI_ADD_RESIDUAL: out = residual + y
    const float* norm_w = nullptr;    // when set: x is RMS-normalised with this gain before the product
    float eps = 1e-5f;
    GemvEpilogue epi = EPI_STORE;
    const GemvGroup* group = nullptr;  // set: w / w2 only give the experts' common shape and type
    const GemvPush* push = nullptr;    // set (see qgemv_push_supported): the rows go to the ranks' buffers instead of `out`
    // Many-token product only: the caller promises that the next product reads `out` (all m rows) as its input with this
    // gain (null: no norm) -- the kernel that sums the shares of k then also prepares that input, saving a launch.
    bool prep_next = false;
    const float* next_norm_w = nullptr;
    float next_eps = 1e-5f;
};
// y[m,n] = x[m,k] . dequant(W)^T, fp32 activations and accumulation.
int32_t launch_qgemv(const GemvArgs& a, cudaStream_t s);
// true when launch_qgemv would run these arguments on the kernel that implements GemvArgs::push
bool qgemv_push_supported(const GemvArgs& a);
// ---- qgemm_umma.cu ----
// The same product for many tokens (prefill chunks, batched decode) on tcgen05 tensor cores with the weights
// dequantised on the fly.  The workspace holds the activations as f16 high/low halves and the per-token scales.
struct GemmWorkspace {
    void* xh = nullptr;          // [2][t_cap][k] f16: high halves, low halves
    void* sx = nullptr;          // [2][t_cap][k / 16] f16: sums over 32-element sub-blocks, eight + eight zeros per 256-element unit
    float* tok_scale = nullptr;  // [t_cap]
    float* partial = nullptr;    // sums of the shares of k when a product is split over several CTAs per tile
    size_t partial_bytes = 0;
    int t_cap = 0, k_max = 0;
    // what xh / sx / tok_scale hold when the summing kernel of the previous product prepared them (see GemvArgs::prep_next);
    // valid for the very next product only
    mutable const float* prep_x = nullptr;
    mutable const float* prep_norm = nullptr;
    mutable int prep_k = 0, prep_t = 0;
};
int32_t run_tcgen05_probe(double* out16_host, cudaStream_t s);
int32_t qgemm_workspace_alloc(GemmWorkspace* ws, int t_cap, int k_max);
void qgemm_workspace_free(GemmWorkspace* ws);
// true when launch_qgemm implements these arguments for T tokens (Q4_K weights, T at least LC_GEMM_MIN_TOKENS, default 5: up to four tokens the
// matrix-vector kernels are faster, from five on they would run their 8-token form, which this product beats)
bool qgemm_applies(const GemvArgs& a, int T, const GemmWorkspace& ws);
// a.m = number of tokens; queues two kernels (activation preparation, product), three when k is split (reduction)
int32_t launch_qgemm(const GemvArgs& a, const GemmWorkspace& ws, cudaStream_t s, int* launches = nullptr);
// Tensor map over f16 activations [2 halves][rows][k] with a box of 64 elements x box_rows rows x both halves, 128-byte swizzle.
bool make_act_tmap(void* out128, const void* base, uint64_t k, uint64_t rows, uint32_t box_rows);
bool make_act_tmap_chunks(void* out128, const void* base, uint64_t k, uint64_t rows, uint32_t box_rows, uint32_t box_chunks);

// ---- attention.cu ----
struct KvLayout {
    void* k_pool = nullptr;  // [pages][n_kv][page_tokens][hd]  (f16 or f32)
    void* v_pool = nullptr;
    int n_kv = 0, hd = 0, page_tokens = 16;
    int kv_f32 = 0;
    int pool_pages = 0;      // pages in each pool (0 = unknown); kernels that check their page-table entries use it
    const void* k_tmap = nullptr;  // host copies of tensor maps over k_pool and v_pool (make_key_pool_tmap), or null
    const void* v_tmap = nullptr;
};
bool make_key_pool_tmap(void* out128, const void* pool, uint64_t rows);
// For each of the `n_tok` new tokens (token i belongs to sequence row tok_seq[i], at cache
// position tok_pos[i], with rotary position tok_rope[i]): rotate q and k in place
// (rust/src/inference/attention.rs:13-34; q, k, v rows are row_stride floats apart) and store k, v into the paged cache
// (rust/src/cache/mod.rs:33-61: f32 -> f16 round to nearest even).
int32_t launch_rope_kv_append(float* q, float* k, const float* v, int row_stride, int n_tok, int n_heads, const KvLayout& kv,
                              const int32_t* tok_seq, const int32_t* tok_pos, const int32_t* tok_rope,
                              const int32_t* page_table, int pages_per_seq, float theta, cudaStream_t s);
// Causal GQA attention of every new token over its sequence's cache (attention.rs:69-113).
// tok_pos[i] is the cache position of token i (it attends to positions 0..tok_pos[i]).
// scratch: split-KV partials, sized by attention_scratch_bytes().
size_t attention_scratch_bytes(int n_tok, int n_heads, int hd, int max_ctx);
// counters: n_tok*n_heads ints, zero before the first launch (the kernel leaves them zero).
// fuse (decode steps only, every token the single new token of its sequence): q is rotated on load and the new
// key/value are taken from k_new/v_new (rows q_stride floats apart), rotated, and stored into the cache by this kernel,
// so no separate rope/append launch is needed.
// positions_settled: tok_pos was final before the kernel ahead of this one started (true from the second layer of a
// step on; false for the first layer, whose positions the end of the previous step may still be writing), so the
// kernel may read it, and start fetching cached pages, before it waits for the kernel ahead of it.
struct AttnFusion {
    const float* k_new; const float* v_new; const int32_t* tok_rope; float theta; bool positions_settled = false;
    // Cross-CTA merge slots of the single-token streaming kernel (attention_stream_slot_bytes of them, all zero before the
    // first launch; the kernel leaves them zero).  They belong to the caller -- one set per model -- because a captured
    // decode step keeps the pointer.
    unsigned long long* stream_slots = nullptr;
};
int32_t launch_attention(const float* q, int q_stride, float* out, int n_tok, int n_heads, const KvLayout& kv,
                         const int32_t* tok_seq, const int32_t* tok_pos, const int32_t* page_table, int pages_per_seq, int max_ctx,
                         void* scratch, int* counters, const AttnFusion* fuse, cudaStream_t s);
// ---- attention_prefill.cu: many new tokens on the tensor cores (head_dim 128, f16 cache, 16-token pages) ----
// up to 64 consecutive tokens of one sequence: rows tok0 .. tok0 + n - 1 of the call, the first at cache position pos0
struct PrefillTile { int32_t tok0, n, seq, pos0; };
bool attention_prefill_applies(const KvLayout& kv, int n_heads);
// q is already rotated and the new keys / values are already in the cache (launch_rope_kv_append); out is [tokens, n_heads * 128]
int32_t launch_attention_prefill(const float* q, int q_stride, float* out, int n_heads, const KvLayout& kv, const PrefillTile* tiles_dev, int n_tiles,
                                 const int32_t* page_table, int pages_per_seq, cudaStream_t s);
// Bytes of merge slots the single-token streaming kernel needs for this head geometry (0: the kernel does not apply).
size_t attention_stream_slot_bytes(int n_heads, int n_kv);

// ---- moe.cu ----
constexpr int kMaxExperts = 64;
constexpr int kMaxTopK = 8;
struct MoeRouteArgs {
    const float* x = nullptr;         // [T, H] the FFN input before its norm
    const float* norm_w = nullptr;    // FFN norm gain (null: x is used as it is)
    float eps = 1e-5f;
    int H = 0, T = 0;
    const float* w_router = nullptr;  // [n_experts, H] f32
    int n_experts = 0, top_k = 0;
    int32_t* sel = nullptr;           // [T, top_k] chosen experts, ascending
    float* wsel = nullptr;            // [T, top_k] their softmax weights
    // calls of at most 64 tokens may also ask for the experts' slot lists (see GemvGroup); `touched` (optional) is
    // increased by the number of experts that received at least one slot
    int32_t* counts = nullptr;
    int32_t* lists = nullptr;
    int list_stride = 0;
    unsigned long long* touched = nullptr;
    int local_first = 0, local_count = 0;  // experts this rank holds (0 count = all): only those are counted in `touched`
    unsigned* ticket = nullptr;            // with `lists`: a device word, zero between launches (the CTA that finishes last builds the lists)
};
int32_t launch_moe_route(const MoeRouteArgs& a, cudaStream_t s);
// out[t] = residual[t] + sum_j wsel[t][j] * y[row(t, j)] in ascending expert order; mode 0: row = t * top_k + j,
// mode 1: row = (sel[t][j] - local_first) * t_stride + t (every local expert's outputs for every token, a plane of t_stride
// rows per expert); only the experts local_first .. local_first + local_count - 1 are added
int32_t launch_moe_combine(const float* y, const int32_t* sel, const float* wsel, int top_k, int H, int T, int mode, size_t t_stride,
                           int local_first, int local_count, const float* residual, float* out, cudaStream_t s);

// ---- dist.cu: sums over the ranks of a model cut across GPUs ----
bool dist_active();
int dist_rank();
int dist_world();
bool dist_peer_memory();
int32_t dist_setup();                               // collective, once (the first model's finalize): maps the ranks' buffers
int32_t dist_allreduce_sum(const float* src, float* dst, size_t count, cudaStream_t s);
int32_t dist_allreduce_max(const long long* src, long long* dst, size_t count, cudaStream_t s);
bool dist_push_desc(size_t count, GemvPush* out);   // false: sums of `count` values do not take the peer-memory path
int32_t dist_gather_sum(float* dst, size_t count, cudaStream_t s);  // completes a sum whose rows the producer pushed
int32_t dist_allgather(const void* src, void* dst, size_t bytes, cudaStream_t s);
// the same sums for ranks that are handles of one process on one GPU: one kernel over all ranks' rows
int32_t launch_group_sum(const float* const* src, float* const* dst, int n, size_t count, cudaStream_t s);
int32_t launch_group_max(const long long* const* src, long long* const* dst, int n, size_t count, cudaStream_t s);

// ---- synth.cu ----
int32_t launch_synth(uint32_t typ, uint64_t seed, uint64_t name_hash, float sigma, size_t n_elems, void* out_dev,
                     cudaStream_t s);
// Part of a [rows][row_blocks blocks] tensor: rows [row0, row0 + rows) x blocks [blk0, blk0 + blks) of every row, written
// densely; the bytes equal the same region of the whole tensor.
int32_t launch_synth_part(uint32_t typ, uint64_t seed, uint64_t name_hash, float sigma, size_t row_blocks, size_t row0, size_t rows,
                          size_t blk0, size_t blks, void* out_dev, cudaStream_t s);
// Greedy pick per row as a key: (total-order key of the maximum << 32) | (index_base + index), last of equal maxima.
int32_t launch_argmax_key(const float* v, size_t n, size_t rows, int index_base, long long* out_keys, cudaStream_t s);
int32_t launch_key_to_token(const long long* keys, size_t rows, int64_t* out_tokens, cudaStream_t s);

}  // namespace lc

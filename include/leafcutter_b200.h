/* leafcutter_b200 -- C ABI of the B200 (sm_100a) token-generation path.
 *
 * A drop-in for the decode hot path of the LeafcutterLLM Rust crate: the
 * operator level mirrors `trait Backend` and the quantised-matmul free
 * functions, the model level mirrors `Engine` / `ShardEngine` / `KVCache`.
 * Citations are file:line inside the reference project.
 *
 * Conventions
 *   - every entry point returns an int32 status: 0 = ok, negative = lc_status;
 *     no exception or panic crosses this boundary;
 *   - the text of the last error of the calling thread: lc_last_error();
 *   - pointers are HOST pointers unless the name ends in `_dev`;
 *   - outputs are caller-allocated; matrices are row-major f32;
 *   - there is no CPU fallback: without a usable CUDA device every compute
 *     entry point returns LC_ERR_CUDA;
 *   - one lc_model = one engine; calls on one handle must be serialised by the
 *     caller (the reference wraps its Engine in a Mutex, rust/src/api/mod.rs:42,50);
 *     distinct handles may be used from distinct threads.
 */
#ifndef LEAFCUTTER_B200_H
#define LEAFCUTTER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum lc_status {
    LC_OK = 0,
    LC_ERR_INVALID = -1,     /* bad argument / shape mismatch (the reference asserts, rust/src/model/tensor.rs:108-113,139) */
    LC_ERR_UNSUPPORTED = -2, /* quant type or feature not implemented */
    LC_ERR_CUDA = -3,        /* CUDA runtime error or no device; see lc_last_error() */
    LC_ERR_OOM = -4,         /* device allocation failed */
    LC_ERR_KV_FULL = -5,     /* no free KV page / sequence slot */
    LC_ERR_MISSING = -6,     /* a required tensor was never set (the reference panics, rust/src/inference/engine.rs:84,97,101) */
    LC_ERR_STATE = -7        /* call order (e.g. forward before finalize) */
} lc_status;

/* ggml tensor type codes: rust/src/model/quant.rs:45-76 */
enum {
    LC_TYPE_F32 = 0, LC_TYPE_F16 = 1, LC_TYPE_Q4_0 = 2, LC_TYPE_Q8_0 = 8,
    LC_TYPE_Q4_K = 12, LC_TYPE_Q5_K = 13, LC_TYPE_Q6_K = 14, LC_TYPE_IQ4_NL = 20
};

const char* lc_last_error(void);
/* Library version string and the number of CUDA devices visible (0 when none). */
const char* lc_version(void);
int32_t lc_device_count(void);
int32_t lc_set_device(int32_t device);

/* Bytes of a tensor of `count` elements of ggml type `typ`:
 * rust/src/model/quant.rs:254-261 (tensor_size), rust/src/model/gguf.rs:307-313. */
size_t lc_tensor_bytes(uint32_t typ, size_t count);

/* ------------------------------------------------------------------------
 * L1 -- operator level.  One entry per method of `trait Backend`
 * (rust/src/backend/mod.rs:18-46, CPU behaviour rust/src/backend/cpu.rs:13-83).
 * Host slices in, host slice out, as the trait has it.
 * ---------------------------------------------------------------------- */
/* Backend::matmul  (backend/mod.rs:21; cpu.rs:13-23): c[m,n] = a[m,k] . b[k,n] */
int32_t lc_matmul_f32(const float* a, const float* b, size_t m, size_t k, size_t n, float* c);
/* Backend::vec_add (mod.rs:24) */
int32_t lc_vec_add(const float* a, const float* b, size_t n, float* out);
/* Backend::vec_mul (mod.rs:27) */
int32_t lc_vec_mul(const float* a, const float* b, size_t n, float* out);
/* Backend::vec_scale (mod.rs:30) */
int32_t lc_vec_scale(const float* a, float scale, size_t n, float* out);
/* Backend::vec_scale_mul (mod.rs:33): out = (a * scale) * b */
int32_t lc_vec_scale_mul(const float* a, float scale, const float* b, size_t n, float* out);
/* Backend::rms_norm (mod.rs:36; cpu.rs:49-60): x is [rows, hidden] with rows = n / hidden */
int32_t lc_rms_norm(const float* x, const float* weight, float eps, size_t hidden, size_t rows, float* out);
/* Backend::silu (mod.rs:39; cpu.rs:62-64) */
int32_t lc_silu(const float* x, size_t n, float* out);
/* Backend::softmax (mod.rs:42; cpu.rs:66-79) */
int32_t lc_softmax(const float* x, size_t hidden, size_t rows, float* out);
/* Backend::sum_sq (mod.rs:45) */
int32_t lc_sum_sq(const float* x, size_t n, float* out);

/* kernels::dequantize_{q4_0,q8_0,q4_k,q5_k,q6_k,iq4_nl} and the F32/F16 arms of
 * GGUFModel::dequantize (rust/src/kernels/mod.rs:16-216, rust/src/model/loader.rs:205-235).
 * Bit-exact with the reference. */
int32_t lc_dequantize(uint32_t typ, const void* bytes, size_t n_elems, float* out);

/* Tensor::matmul against a quantised weight (rust/src/model/tensor.rs:107-135 after
 * loader.rs:145-168): c[m,n] = a[m,k] . dequant(W)^T, W = raw GGUF blocks, n rows of k/block
 * blocks (quant blocks run along k).  The weight is never expanded to f32 in memory. */
int32_t lc_qmatmul(uint32_t typ, const float* a, const void* w_blocks, size_t m, size_t k, size_t n, float* c);

/* int8_gemm::q8_0_matmul / q4_0_matmul (rust/src/kernels/int8_gemm.rs:172-194, 336-358) over the
 * shard-order matrices of q8_0.rs:56-86 / q4_0.rs:66-94: blocks laid [k rows][n/32], one f32
 * scale per block; Q8_0 qs int8[k*n]; Q4_0 qs uint8[k*n/2] with byte i = elements 2i, 2i+1. */
int32_t lc_q8_0_matmul_shard(const float* a, const float* scales, const int8_t* qs, size_t m, size_t k, size_t n, float* c);
int32_t lc_q4_0_matmul_shard(const float* a, const float* scales, const uint8_t* qs, size_t m, size_t k, size_t n, float* c);

/* attention::apply_rotary_emb (rust/src/inference/attention.rs:13-34), in place on x[seq, heads, head_dim];
 * pos0 = 0 reproduces the reference (position = index inside the call). */
int32_t lc_rope(float* x, size_t seq, size_t heads, size_t head_dim, float theta, size_t pos0);
/* sampler::sample_top_p greedy branch (rust/src/inference/sampler.rs:6-10): LAST index among equal maxima. */
int32_t lc_argmax(const float* v, size_t n, int64_t* out_index);

/* Device-resident variants used to time kernels without host copies.  All pointers are device
 * pointers obtained from lc_dev_alloc; work is queued on the library's stream of the current device. */
int32_t lc_dev_alloc(size_t bytes, void** out_dev);
int32_t lc_dev_free(void* dev);
int32_t lc_dev_upload(void* dst_dev, const void* src_host, size_t bytes);
int32_t lc_dev_download(void* dst_host, const void* src_dev, size_t bytes);
int32_t lc_dev_sync(void);
int32_t lc_qmatmul_dev(uint32_t typ, const float* a_dev, const void* w_dev, size_t m, size_t k, size_t n, float* c_dev);
int32_t lc_dequantize_dev(uint32_t typ, const void* bytes_dev, size_t n_elems, float* out_dev);
/* The attention core of attention_forward (rust/src/inference/attention.rs:69-113: scores / sqrt(head_dim), softmax, weighted
 * sum of V, grouped-query head mapping) for ONE new token over a paged cache that is already on the device.  q_dev is
 * [n_heads * head_dim], already rotated; pools are [page][kv head][page_tokens][head_dim] in f16 (kv_f32 = 0, the storage type
 * of rust/src/cache/mod.rs:33-61) or f32; page_table_dev lists the n_pages pages of the sequence; the token attends to
 * positions 0 .. ctx_len-1; out_dev is [n_heads * head_dim].  Queued on the library's stream (lc_dev_sync to wait).
 * The context is split across CTAs; the split partials live in device scratch that the library allocates and keeps. */
int32_t lc_attention_decode_dev(const float* q_dev, const void* k_pool_dev, const void* v_pool_dev, const int32_t* page_table_dev,
                                int32_t n_pages, int32_t ctx_len, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                                int32_t page_tokens, int32_t kv_f32, float* out_dev);
/* Same operation and same kernels for callers that must not allocate device memory at call time -- code running inside a
 * framework's allocator-owned arena, under a memory budget that is already fully handed out, or in a late phase where
 * cudaMalloc would serialise the device.  It has no counterpart in the reference.  The split partials go to a 1 MiB array
 * built into the library image (every GPU that loads the library holds it until the process exits), and the word the
 * kernels raise when a bounded wait runs out is part of the image too: nothing is allocated or freed, by this call or
 * by anything it uses, also when it is the first call a process makes into the library.
 * Size rule: 256 bytes of bookkeeping + 4 * n_heads rounded up to 256 + the partials must fit 1 MiB, where the partials are
 * n_heads * pieces * (head_dim + 2) * 4 bytes and pieces = ceil(ctx_len / 128) (the context is cut into 128-key pieces, so
 * the need grows with the context; a context under a few hundred keys may be cut finer, into at most 4 * SM count / n_heads
 * pieces of 64 keys).  32 heads of 128 dims are accepted up to ctx_len 7936 and refused from 7937 on;
 * 128 heads of 256 dims fit up to ctx_len 896.  Shapes that do not fit are rejected with LC_ERR_INVALID.
 * The first call on a device looks up the device addresses of the array and of that word; make that first call outside
 * any stream capture.  All calls share the one array, which keeps the previous call's partials: the counters it needs
 * at zero are cleared at the start of every call, and two calls that overlap on the GPU (different streams, different
 * threads) would race -- the library queues them on its single stream, keep it that way. */
int32_t lc_attention_decode_static(const float* q_dev, const void* k_pool_dev, const void* v_pool_dev, const int32_t* page_table_dev,
                                   int32_t n_pages, int32_t ctx_len, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                                   int32_t page_tokens, int32_t kv_f32, float* out_dev);
/* CUDA-event stopwatch on the library's stream: begin, queue work, end -> milliseconds. */
int32_t lc_timer_begin(void);
int32_t lc_timer_end(float* out_ms);
/* Writes `bytes` bytes to a scratch buffer larger than L2 so the next kernel starts from a cold cache. */
int32_t lc_flush_l2(void);

/* Deterministic synthetic tensors (test and benchmark input; no counterpart in the reference).
 * Element i of tensor (seed, name) is N(0, sigma) from a counter-based generator, quantised to
 * `typ` (F32, F16, Q4_0, Q8_0, Q4_K, Q5_K or Q6_K; LC_ERR_UNSUPPORTED otherwise) in GGUF block order.  The host and the
 * device generator produce identical bytes. */
int32_t lc_synth_tensor_host(uint32_t typ, uint64_t seed, const char* name, float sigma, size_t n_elems, void* out_bytes);
int32_t lc_synth_tensor_dev(uint32_t typ, uint64_t seed, const char* name, float sigma, size_t n_elems, void* out_dev);
int32_t lc_synth_tokens(uint64_t seed, size_t n, int64_t vocab, int64_t* out);

/* ------------------------------------------------------------------------
 * L2 -- model level.
 * ---------------------------------------------------------------------- */
typedef struct lc_model lc_model;

/* ModelConfig (rust/src/model/loader.rs:13-22) plus the switches the reference hard-codes. */
typedef struct lc_model_config {
    int32_t hidden_size;
    int32_t num_layers;
    int32_t num_heads;
    int32_t num_kv_heads;
    int32_t intermediate_size;
    int32_t max_seq_len;      /* per-sequence KV capacity in tokens */
    int32_t vocab_size;
    float rope_theta;
    float rms_eps;            /* 0 -> 1e-5, the constant at rust/src/inference/engine.rs:102,111,121 */
    int32_t kv_dtype;         /* 0 = f16 storage as rust/src/cache/mod.rs:33-61; 1 = f32 */
    int32_t rope_mode;        /* 0 = position inside the call, as attention.rs:13-21; 1 = absolute position */
    int32_t n_experts;        /* 0 = dense FFN; > 0: router + n_experts SwiGLU experts per layer, top_k per token (mixture-of-experts
                                 has no counterpart in the reference; the definition is at lc_forward) */
    int32_t top_k;
    int32_t max_seqs;         /* concurrent sequences; 0 -> 1 */
    int32_t kv_page_tokens;   /* tokens per KV page; 0 -> 16 */
    int64_t kv_pool_tokens;   /* KV pool size in tokens over all sequences; 0 -> max_seqs * max_seq_len */
    int32_t device;           /* CUDA device ordinal */
    int32_t tp_size;          /* model-parallel ranks the model is cut into; 0 or 1 = whole model; 0 after lc_dist_init = that world */
    int32_t tp_rank;          /* which of them this handle holds (0 after lc_dist_init = that rank) */
    int32_t reserved[5];
} lc_model_config;

/* ---- Model parallelism (no counterpart in the reference, which runs on one device) ----
 * A model of tp_size ranks is cut the usual tensor-parallel way; every dimension below is the WHOLE model's, and every rank is
 * handed the WHOLE tensor by lc_model_set_tensor / lc_model_synth_tensor and keeps its own part (lc_shard_plan says which):
 *   attn_q / attn_k / attn_v, ffn_gate / ffn_up, output.weight   by output rows (whole heads, whole vocabulary slices);
 *   attn_output, ffn_down                                         by input columns, on quant-block boundaries;
 *   norms, token_embd, the router                                 whole on every rank;
 *   mixture-of-experts layers                                     whole experts, n_experts / tp_size consecutive ones per rank.
 * The KV cache is cut by kv head.  Per layer there are two sums over the ranks -- after attn_output and after ffn_down
 * (or the experts' weighted sum) -- taken in rank order, so every rank holds bit-identical activations; the greedy pick is
 * the maximum over the ranks of (logit, global index), equal logits going to the higher index as on one device.
 * Requirements: num_heads, num_kv_heads, vocab_size, intermediate_size (or n_experts) divisible by tp_size, the column
 * parts whole quant blocks.
 *
 * One process per GPU: rank 0 calls lc_dist_unique_id and hands the 128 bytes to the other ranks by its own means; every
 * rank then calls lc_dist_init(rank, world, id) with its device current, BEFORE lc_model_create, and creates the model with
 * tp_size = tp_rank = 0 (or the same numbers).  All ranks must make the same model-level calls in the same order.  The
 * sums run as NCCL all-reduces (lc_dist_init loads libnccl.so.2 at run time) or, for payloads up to 2 MiB when every peer's
 * buffer could be mapped, as one kernel per sum that reads the peers' partial rows over NVLink in rank order; waits in
 * that kernel are bounded and end in LC_ERR_CUDA.  lc_dist_set_backend(0) forces NCCL, (1) asks for the peer-memory kernel.
 *
 * One process, one GPU, several ranks (testing a cut model where only one GPU is at hand): create tp_size handles with
 * explicit tp_size / tp_rank on the same device, load and finalize each, then lc_model_group(handles, tp_size).  Calls on
 * handles[0] then drive all ranks in lock step on the one stream and the sums run as one kernel over all ranks' rows. */
int32_t lc_dist_unique_id(void* out_id128);
int32_t lc_dist_init(int32_t rank, int32_t world, const void* id128);
int32_t lc_dist_set_backend(int32_t peer_memory);
int32_t lc_dist_finalize(void);
/* What lc_dist_init set up: world 1 / rank 0 without it; *peer_memory = 1 once the ranks' buffers are mapped into each other
 * (known after the first model is finalized or lc_dist_time_allreduce has run), 0 while the sums go through NCCL. */
int32_t lc_dist_info(int32_t* rank, int32_t* world, int32_t* peer_memory);
/* Diagnostics after LC_ERR_CUDA from a cut model: out8[0] != 0 when a wait of a sum ran out, then out8[1..7] = the sum's number,
 * the rank whose value was missing, the value's index, the tag found in its place, whether the kernel also sent, whether it
 * was the greedy-pick maximum, the number of values.  Reading clears the record.  LC_DIST_TIMEOUT_MS (default 10000) bounds
 * those waits. */
int32_t lc_dist_debug(uint32_t* out8);
/* Microseconds per sum of `count` floats over the ranks, averaged over `iters` back-to-back sums on the library's stream
 * (CUDA events; a measurement helper for the all-reduce that sits between a layer's products). */
int32_t lc_dist_time_allreduce(size_t count, int32_t iters, float* out_us);

/* Diagnostic, no counterpart in the reference: SM cycles per operation of the building blocks of the many-token product on
 * this GPU (one CTA, no memory traffic): out16[0..13] = tcgen05.mma M128 K16 issued by one thread at N = 128 and N = 256,
 * by two threads at once, tcgen05.commit, tcgen05.st + wait, the same + fence + barrier arrival of 128 threads,
 * tcgen05.ld + wait, the two tcgen05 fences, a barrier probe + warp vote, arrival -> a waiting thread returns, and the
 * unpacking of one 64-element Q4_K chunk of 32 rows with 4 / 8 / 16 warps at it.  Every wait inside is bounded. */
int32_t lc_tcgen05_probe(double* out16);
int32_t lc_model_group(lc_model** handles, int32_t n);
/* Which part of a tensor a rank keeps: kind 0 = all of it, 1 = rows [first, first + count) (dims[1] index; for stacked expert
 * tensors rows of the flattened [dims[2] * dims[1]] matrix), 2 = columns [first, first + count) of every row (dims[0] index),
 * 3 = nothing (an expert that lives on another rank).  Pure host arithmetic: needs no GPU. */
int32_t lc_shard_plan(const lc_model_config* cfg, const char* name, const uint64_t* dims, int32_t ndims, int32_t* kind,
                      uint64_t* first, uint64_t* count);

/* Engine::load without the file: create, then hand over each tensor, then finalize.
 * rust/src/inference/engine.rs:18-49, rust/src/model/loader.rs:145-203. */
int32_t lc_model_create(const lc_model_config* cfg, lc_model** out);
/* `name` is the GGUF tensor name ("blk.3.attn_q.weight", "token_embd.weight", "output_norm.weight",
 * "output.weight") or the engine name it maps to (rust/src/model/arch.rs:83-96, loader.rs:173-177).
 * `dims` in GGUF order (fastest first).  `bytes` are the raw GGUF blocks on the host. */
int32_t lc_model_set_tensor(lc_model* m, const char* name, uint32_t typ, const uint64_t* dims, int32_t ndims,
                            const void* bytes, size_t nbytes);
/* Same, but the library synthesises the tensor on the device (lc_synth_tensor_dev) -- no host copy. */
int32_t lc_model_synth_tensor(lc_model* m, const char* name, uint32_t typ, const uint64_t* dims, int32_t ndims,
                              uint64_t seed, float sigma);
/* Copies the raw blocks of a tensor back to the host (to hand the same bytes to a checker). */
int32_t lc_model_get_tensor(lc_model* m, const char* name, void* out_bytes, size_t nbytes);
/* Checks completeness (the 9 per-layer tensors + embedding + final norm; tied head when
 * output.weight is absent, loader.rs:192-199), runs the weight sanity scan (loader.rs:241-249:
 * counts elements that dequantise to NaN/Inf/|v|>100), builds the execution plan. */
int32_t lc_model_finalize(lc_model* m);
int32_t lc_model_destroy(lc_model* m);
/* Engine::load(path) (engine.rs:18-49): parse a GGUF v3 file (rust/src/model/gguf.rs:76-119),
 * read the config keys (loader.rs:106-133), upload every tensor, finalize. */
int32_t lc_model_load_gguf(const char* path, const lc_model_config* overrides, lc_model** out);
int32_t lc_model_get_config(const lc_model* m, lc_model_config* out);

/* ---- Pre-flight checks of a GGUF file: capability report + corruption scan ----
 * lc_scan_blocks / lc_scan_blocks_dev: the per-tensor body of scan_for_corruption (rust/src/model/loader.rs:301-422) on the
 * GPU: blocks_total = ceil(n_elems / block size) (:325), blocks_bad = blocks whose scale -- d, and for most types the
 * half-word at byte 2 read as dmin (:366-381) -- is NaN, infinite or above 1e4 in magnitude (:385-392).  Every type code
 * of QuantType::from_u32 (rust/src/model/quant.rs:71-100) is accepted; F32 / F16 / BF16 and unknown codes have no blocks
 * and report 0 / 0 as the reference skips them (:309-322). */
int32_t lc_scan_blocks(uint32_t typ, const void* bytes, size_t n_elems, uint64_t* blocks_total, uint64_t* blocks_bad);
int32_t lc_scan_blocks_dev(uint32_t typ, const void* bytes_dev, size_t n_elems, uint64_t* blocks_total, uint64_t* blocks_bad);

/* One row of CorruptionReport::corrupted_tensors (loader.rs:286-292, 404-413). */
typedef struct lc_corrupt_tensor {
    char name[112];
    uint32_t ggml_type;
    uint32_t reserved;
    uint64_t blocks_total;
    uint64_t blocks_bad;
} lc_corrupt_tensor;

/* GGUFModel::capability_report (loader.rs:54-104) and scan_for_corruption (loader.rs:301-422) of one file. */
typedef struct lc_gguf_report {
    char architecture[16];          /* ModelArchitecture::name (rust/src/model/arch.rs:41-51): "Llama", "Qwen2", "Qwen3.5", ... */
    int32_t arch_supported;         /* arch.rs:71-77 */
    int32_t total_tensors;          /* QuantSummary::total_tensors (rust/src/model/gguf.rs:319) */
    int32_t tensors_by_type[32];    /* index = ggml type code; codes from_u32 does not know are not counted (gguf.rs:321) */
    uint32_t unsupported_types;     /* bit c: a tensor of type code c is present and the type has no dequantiser (quant.rs:243-254) */
    int32_t n_missing;              /* blk.N.<suffix> absent, N < min(layers, 4), the 9 suffixes of arch.rs:83-96 */
    int32_t n_extra;                /* distinct blk.*.weight tensors whose suffix is neither mapped nor a known extra (loader.rs:74-89) */
    int32_t can_run;                /* arch_supported && no unsupported type && nothing missing (loader.rs:91-93) */
    int32_t n_corrupt_tensors;      /* tensors with at least one bad block */
    uint64_t total_blocks_checked;  /* blocks of the tensors that have a bad block (loader.rs:404-406 counts only those) */
    uint64_t total_bad_blocks;
    lc_model_config config;         /* GGUFModel::extract_config (loader.rs:106-141) */
} lc_gguf_report;

/* scan != 0 runs the corruption scan (every block-type tensor of the file is sent through the device once).
 * corrupt[0 .. min(n_corrupt_tensors, corrupt_cap)) is filled in file order.  names (optional) receives one line per
 * finding, "missing <tensor>\n" then "extra <tensor>\n" (sorted), cut at names_cap - 1 characters and 0-terminated. */
int32_t lc_gguf_inspect(const char* path, int32_t scan, lc_gguf_report* report, lc_corrupt_tensor* corrupt, int32_t corrupt_cap,
                        char* names, size_t names_cap);

/* ---- ShardEngine (rust/src/inference/shard_engine.rs:18-167): a model split into per-layer "LEAFSHDR" shards ----
 * lc_shard_engine_load     <-> ShardEngine::load_with_cache(manifest_path, num_layers) (:34-61): reads manifest.json
 *                              (rust/src/shard/loader.rs:13-50) and every shard (format.rs, loader.rs:300-367: F32, Q8_0 or
 *                              Q4_0 blocks along the rows of [k][n] matrices) once; all layers stay in device memory.
 *                              max_seq_len > 0 caps the KV capacity the manifest asks for.
 * lc_shard_engine_forward  <-> ShardEngine::forward(&tokens) (:99-167): logits of the last token (logits_out [vocab], may be
 *                              null) and its greedy pick (next_out, may be null); the cache grows by n.
 * lc_shard_engine_generate <-> ShardEngine::generate (:74-97): clears the cache, first token from the prefill, at most
 *                              max_tokens tokens, stops after token 2; temperature > 0 needs lc_shard_engine_set_seed first
 *                              (draws and arithmetic as in lc_generate), else LC_ERR_UNSUPPORTED.
 * lc_shard_engine_reset_kv_cache / _kv_cache_memory_bytes <-> reset_kv_cache (:64-66) / kv_cache_memory_mb (:69-71). */
typedef struct lc_shard_engine lc_shard_engine;
int32_t lc_shard_engine_load(const char* manifest_path, int32_t max_seq_len, int32_t device, lc_shard_engine** out);
int32_t lc_shard_engine_forward(lc_shard_engine* e, const int64_t* tokens, int32_t n, float* logits_out, int64_t* next_out);
int32_t lc_shard_engine_generate(lc_shard_engine* e, const int64_t* tokens, int32_t n, int32_t max_tokens, float temperature,
                                 float top_p, int64_t* out_tokens, int32_t* n_out);
int32_t lc_shard_engine_set_seed(lc_shard_engine* e, uint64_t seed);
int32_t lc_shard_engine_reset_kv_cache(lc_shard_engine* e);
int32_t lc_shard_engine_kv_cache_memory_bytes(lc_shard_engine* e, uint64_t* out);
int32_t lc_shard_engine_destroy(lc_shard_engine* e);

/* KVCache::clear (rust/src/cache/mod.rs:26-30) for one sequence slot (seq_id < max_seqs); -1 = all. */
int32_t lc_kv_clear(lc_model* m, int32_t seq_id);
/* KVCache::memory_bytes (cache/mod.rs:80-84): bytes of K and V held for the live tokens. */
int32_t lc_kv_memory_bytes(const lc_model* m, uint64_t* out);
/* Tokens currently cached for a sequence. */
int32_t lc_kv_length(const lc_model* m, int32_t seq_id, int32_t* out);

/* Engine::forward (engine.rs:78-132) on sequence slot 0: append n tokens, return the logits of the
 * last one ([vocab]). */
int32_t lc_forward(lc_model* m, const int64_t* tokens, int32_t n, float* logits_out);
/* The same for several sequences in one step (what a server.ModelRunner.RunBatch implementation,
 * pkg/server/scheduler.go:55-60, would call per step).  tokens is ragged: n_tokens[i] ids for
 * seq_ids[i], concatenated.  logits_out is [n_seqs, vocab] (may be NULL); next_out receives the
 * greedy token of each sequence (may be NULL). */
int32_t lc_forward_batch(lc_model* m, int32_t n_seqs, const int32_t* seq_ids, const int64_t* tokens,
                         const int32_t* n_tokens, float* logits_out, int64_t* next_out);

/* sampler::sample_top_p (rust/src/inference/sampler.rs:6-50) on the GPU with the uniform draw u in [0, 1) supplied by the
 * caller (the reference's `rng.gen::<f32>()`, :39): logits / temperature, softmax, stable descending sort, the shortest
 * prefix whose running f32 sum exceeds top_p, pick = first position with u * kept_sum <= running sum.  All f32 sums run in
 * the reference's order; temperature <= 0 is its greedy branch (ties: the last maximum).  n >= 1 (the reference panics on
 * an empty slice). */
int32_t lc_sample_top_p(const float* logits, size_t n, float temperature, float top_p, float u, int64_t* token);
/* Seeded stochastic generation: after this call lc_generate accepts temperature > 0; the draw counter restarts at 0.
 * lc_seeded_uniform(seed, i) is draw i: 24 random bits scaled to [0, 1) (the grid of rand's f32 sampling, not its stream). */
int32_t lc_model_set_seed(lc_model* m, uint64_t seed);
float lc_seeded_uniform(uint64_t seed, uint64_t index);

typedef void (*lc_token_cb)(int64_t token, void* user);
/* Engine::generate (engine.rs:51-76) / Go inference.Model.Generate (pkg/inference/speculative.go:18-20):
 * clears the cache of slot 0, prefills, emits the first token from the prefill logits, then up to
 * max_tokens-1 decode steps.  temperature <= 0 selects greedy (sampler.rs:7-10).  The stochastic
 * branch (sampler.rs:12-50) draws from an unseeded RNG in the reference: here it returns LC_ERR_UNSUPPORTED
 * until lc_model_set_seed has been called, and then uses the draws lc_seeded_uniform(seed, 0), (seed, 1), ...
 * one per emitted token, through the same arithmetic as lc_sample_top_p.
 * stop_on_eos != 0 keeps the reference's stop on token id 2 (engine.rs:60-63,70-72). */
int32_t lc_generate(lc_model* m, const int64_t* tokens, int32_t n, int32_t max_tokens, float temperature,
                    float top_p, int32_t stop_on_eos, int64_t* out_tokens, int32_t* n_out, lc_token_cb cb,
                    void* user);

/* Device-resident decode loop for measurement: `steps` greedy decode steps for every live sequence
 * listed, each step feeding the previous step's token; nothing crosses PCIe inside the loop.
 * out_tokens is [steps, n_seqs] (may be NULL).  *out_ms = CUDA-event time of the loop. */
int32_t lc_decode_loop(lc_model* m, int32_t n_seqs, const int32_t* seq_ids, const int64_t* first_tokens,
                       int32_t steps, int64_t* out_tokens, float* out_ms);

/* Counters since creation or the last reset. */
typedef struct lc_counters {
    uint64_t tokens_prefilled;
    uint64_t tokens_decoded;
    uint64_t forward_calls;
    uint64_t kernel_launches;     /* kernels of this library queued (graph replays count their nodes) */
    uint64_t weight_bytes;        /* quantised weight bytes resident */
    uint64_t kv_pages_in_use;
    uint64_t kv_pages_total;
    uint64_t sanitize_hits;       /* elements the weight sanity scan would zero (loader.rs:241-249) */
    uint64_t algo_bytes_last_step;/* algorithmic HBM bytes of the last decode step */
    uint64_t reserved[7];
} lc_counters;
int32_t lc_get_counters(const lc_model* m, lc_counters* out);
int32_t lc_reset_counters(lc_model* m);

/* Layer-level probes for parity tests: run one sub-block of layer `layer` on host activations
 * through the same kernels lc_forward uses.  attention_forward (attention.rs:37-118) appends to
 * the KV cache of slot 0; ffn_forward (engine.rs:146-164). */
int32_t lc_probe_attention(lc_model* m, int32_t layer, const float* normed, int32_t seq, float* out);
int32_t lc_probe_ffn(lc_model* m, int32_t layer, const float* x, int32_t seq, float* out);

#ifdef __cplusplus
}
#endif
#endif /* LEAFCUTTER_B200_H */

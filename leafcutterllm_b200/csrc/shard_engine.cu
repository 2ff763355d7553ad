// ShardEngine on the device (rust/src/inference/shard_engine.rs:27-167): a model split into per-layer "LEAFSHDR" shard
// files plus a manifest.json (rust/src/shard/format.rs, rust/src/shard/loader.rs:13-50,300-367).  The reference maps one
// layer at a time from disk; here every shard is read once and stays in HBM (its load_with_cache(num_layers) mode).
//
// Weights keep the reference's shard layout -- matrices [k rows][n columns], blocks of 32 along a row -- and the
// products run through the shard-order kernels (ops.cu), whose per-output arithmetic is the reference's: one thread per
// output, k ascending, deq = q * scale rounded once, c = fma(a, deq, c)  (rust/src/kernels/int8_gemm.rs:49-98, 240-280).
// The forward pass is the unfused sequence of shard_engine.rs:99-167: rms_norm(1e-5), q/k/v/o products, rotary embedding
// with the index inside the call, f16 KV cache, residual adds, silu(gate) * up, final norm, head.  One sequence, as there.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <cstring>
#include <map>
#include <string>
#include <vector>
#include <cuda_fp16.h>
#include "lc_kernels.h"

using namespace lc;

namespace {

// ---- a small JSON reader: enough for the manifest (objects, arrays, strings, numbers, true/false/null) ----------------
struct JValue {
    enum Kind { NUL, NUM, STR, BOOL, ARR, OBJ } kind = NUL;
    double num = 0;
    std::string str;
    std::vector<JValue> arr;
    std::map<std::string, JValue> obj;
    const JValue* get(const char* k) const {
        auto it = obj.find(k);
        return it == obj.end() ? nullptr : &it->second;
    }
};
struct JReader {
    const char* p;
    const char* e;
    bool ok = true;
    void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool eat(char c) { ws(); if (p < e && *p == c) { p++; return true; } return false; }
    std::string str() {
        std::string s;
        if (!eat('"')) { ok = false; return s; }
        while (p < e && *p != '"') {
            if (*p == '\\' && p + 1 < e) {
                p++;
                switch (*p) {
                    case 'n': s += '\n'; break;
                    case 't': s += '\t'; break;
                    case 'u': if (p + 4 < e) p += 4; s += '?'; break;  // names and paths in a manifest are ASCII
                    default: s += *p;
                }
                p++;
            } else {
                s += *p++;
            }
        }
        if (p >= e) ok = false; else p++;
        return s;
    }
    JValue value(int depth = 0) {
        JValue v;
        ws();
        if (p >= e || depth > 16) { ok = false; return v; }
        if (*p == '{') {
            p++;
            v.kind = JValue::OBJ;
            if (eat('}')) return v;
            do {
                std::string k = str();
                if (!ok || !eat(':')) { ok = false; return v; }
                v.obj[k] = value(depth + 1);
            } while (ok && eat(','));
            if (!eat('}')) ok = false;
        } else if (*p == '[') {
            p++;
            v.kind = JValue::ARR;
            if (eat(']')) return v;
            do v.arr.push_back(value(depth + 1)); while (ok && eat(','));
            if (!eat(']')) ok = false;
        } else if (*p == '"') {
            v.kind = JValue::STR;
            v.str = str();
        } else if (!strncmp(p, "true", 4) && e - p >= 4) { v.kind = JValue::BOOL; v.num = 1; p += 4; }
        else if (!strncmp(p, "false", 5) && e - p >= 5) { v.kind = JValue::BOOL; p += 5; }
        else if (!strncmp(p, "null", 4) && e - p >= 4) { p += 4; }
        else {
            char* end = nullptr;
            v.kind = JValue::NUM;
            v.num = strtod(p, &end);
            if (end == p || end > e) ok = false; else p = end;
        }
        return v;
    }
};

struct Mapping {
    int fd = -1;
    void* base = MAP_FAILED;
    size_t size = 0;
    int32_t open_file(const std::string& path) {
        fd = open(path.c_str(), O_RDONLY);
        LC_CHECK(fd >= 0, LC_ERR_INVALID, "cannot open %s", path.c_str());
        struct stat st;
        LC_CHECK(fstat(fd, &st) == 0 && st.st_size > 0, LC_ERR_INVALID, "%s: empty or unreadable", path.c_str());
        size = (size_t)st.st_size;
        base = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
        LC_CHECK(base != MAP_FAILED, LC_ERR_INVALID, "cannot map %s", path.c_str());
        return LC_OK;
    }
    ~Mapping() {
        if (base != MAP_FAILED) munmap(base, size);
        if (fd >= 0) close(fd);
    }
};

// One tensor of a shard as the file holds it.
struct RawTensor {
    std::vector<uint64_t> dims;
    const uint8_t* data = nullptr;
    size_t nbytes = 0;
    int fmt = 0;  // QuantFormat of the shard: 0 F32, 1 Q8_0, 2 Q4_0 (format.rs:35-43)
    size_t count() const { size_t c = 1; for (uint64_t d : dims) c *= (size_t)d; return c; }
};

float f16_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

}  // namespace

// A matrix [k][n] on the device in one of the three shard formats.
struct ShardMat {
    int fmt = 0, k = 0, n = 0;
    float* f32 = nullptr;     // fmt 0: [k][n]
    float* scales = nullptr;  // fmt 1, 2: [k][n / 32], widened from f16 (exact)
    void* qs = nullptr;       // fmt 1: int8 [k][n]; fmt 2: packed nibbles [k][n / 2], element 2i low, 2i + 1 high (q4_0.rs:36-46)
};

struct lc_shard_engine {
    int device = 0;
    bool seeded = false;  // lc_shard_engine_set_seed: temperature > 0 allowed, draws seeded_uniform(seed, draws++)
    uint64_t seed = 0, draws = 0;
    cudaStream_t stream = nullptr;
    int L = 0, H = 0, nh = 0, nkv = 0, hd = 0, F = 0, V = 0, nqkv = 0, max_seq = 0;
    float theta = 10000.f;
    struct Layer { ShardMat qkv, o, gate, up, down; float* in_norm = nullptr; float* post_norm = nullptr; };
    std::vector<Layer> layers;
    float* embed = nullptr;  // [V][H] f32 (a quantised table is dequantised: Tensor::from_q8_0 keeps both, tensor.rs:67-76)
    float* final_norm = nullptr;
    ShardMat head;
    // KV cache: one sequence, f16, 16-token pages laid out one after the other (cache/mod.rs:33-77)
    std::vector<void*> k_pools, v_pools;
    int pages = 0, seq_len = 0;
    int32_t* d_page_table = nullptr;
    // step buffers for up to kChunk tokens
    static constexpr int kChunk = 256;
    int64_t* d_tokens = nullptr;
    int32_t *d_seq = nullptr, *d_pos = nullptr, *d_rope = nullptr;
    float *d_hidden = nullptr, *d_hidden2 = nullptr, *d_norm = nullptr, *d_qkv = nullptr, *d_attn = nullptr, *d_o = nullptr;
    float *d_g = nullptr, *d_u = nullptr, *d_act = nullptr, *d_logits = nullptr;
    int64_t* d_next = nullptr;
    void* d_scratch = nullptr;
    int* d_counters = nullptr;
    std::vector<void*> owned;
    uint64_t weight_bytes = 0;
};

namespace {

template <typename T>
int32_t dev_alloc(lc_shard_engine* e, T** p, size_t count) {
    void* q = nullptr;
    cudaError_t err = cudaMalloc(&q, std::max<size_t>(count, 1) * sizeof(T));
    if (err != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("device allocation of %zu bytes failed: %s", count * sizeof(T), cudaGetErrorString(err));
        return LC_ERR_OOM;
    }
    e->owned.push_back(q);
    *p = (T*)q;
    return LC_OK;
}

// parse_shard_from_mmap (shard/loader.rs:300-367): header, tensor table, bounds and size checks
int32_t parse_shard(const std::string& path, const Mapping& mp, std::map<std::string, RawTensor>* out) {
    const uint8_t* b = (const uint8_t*)mp.base;
    LC_CHECK(mp.size >= 32 && !memcmp(b, "LEAFSHDR", 8), LC_ERR_INVALID, "%s: invalid shard file: bad magic", path.c_str());
    uint32_t version, count;
    memcpy(&version, b + 8, 4);
    memcpy(&count, b + 12, 4);
    LC_CHECK(version == 1, LC_ERR_INVALID, "%s: invalid shard file: version %u", path.c_str(), version);
    int fmt = b[24] <= 2 ? b[24] : 0;  // format.rs:113: an unknown code reads as F32
    size_t pos = 32;
    auto need = [&](size_t k) { return k <= mp.size - pos; };
    for (uint32_t i = 0; i < count; i++) {
        uint32_t name_len, rank;
        LC_CHECK(need(4), LC_ERR_INVALID, "%s: truncated tensor table", path.c_str());
        memcpy(&name_len, b + pos, 4); pos += 4;
        LC_CHECK(name_len < 4096 && need(name_len + 4), LC_ERR_INVALID, "%s: truncated tensor table", path.c_str());
        std::string name((const char*)b + pos, name_len); pos += name_len;
        memcpy(&rank, b + pos, 4); pos += 4;
        LC_CHECK(rank <= 8 && need((size_t)rank * 8 + 16), LC_ERR_INVALID, "%s: truncated tensor table", path.c_str());
        RawTensor t;
        t.fmt = fmt;
        for (uint32_t d = 0; d < rank; d++) { uint64_t v; memcpy(&v, b + pos, 8); pos += 8; t.dims.push_back(v); }
        uint64_t off, size;
        memcpy(&off, b + pos, 8); pos += 8;
        memcpy(&size, b + pos, 8); pos += 8;
        LC_CHECK(off <= mp.size && size <= mp.size - off, LC_ERR_INVALID, "%s: shard corrupt: tensor '%s' data out of bounds", path.c_str(), name.c_str());
        const size_t elems = t.count();
        const size_t expect = fmt == 0 ? elems * 4 : fmt == 1 ? elems / 32 * 34 : elems / 32 * 18;
        LC_CHECK(size == expect, LC_ERR_INVALID, "%s: shard corrupt: tensor '%s' size mismatch (%llu bytes vs %zu expected)", path.c_str(),
                 name.c_str(), (unsigned long long)size, expect);
        t.data = b + off;
        t.nbytes = (size_t)size;
        (*out)[name] = t;
    }
    return LC_OK;
}

// The f32 values of a tensor the reference does NOT keep quantised (1-D, or a row length that is not a multiple of 32):
// loader.rs:335-338 / 355-358 run the GGUF-order block decoders of kernels/mod.rs over the bytes.
void dequant_flat(const RawTensor& t, std::vector<float>* out) {
    const size_t n = t.count();
    out->resize(n);
    if (t.fmt == 0) { memcpy(out->data(), t.data, n * 4); return; }
    for (size_t blk = 0; blk < n / 32; blk++) {
        const uint8_t* p = t.data + blk * (t.fmt == 1 ? 34 : 18);
        uint16_t h; memcpy(&h, p, 2);
        const float s = f16_bits_to_f32(h);
        for (int j = 0; j < 32; j++) {
            if (t.fmt == 1) (*out)[blk * 32 + j] = (float)(int8_t)p[2 + j] * s;                         // mod.rs:37-51
            else {                                                                                      // mod.rs:16-34: j low, j + 16 high
                const uint8_t q = p[2 + (j & 15)];
                (*out)[blk * 32 + j] = ((float)(j < 16 ? (q & 0x0F) : (q >> 4)) - 8.0f) * s;
            }
        }
    }
}

// The f32 values of a tensor the reference keeps quantised, as Q8Matrix / Q4Matrix::dequantize give them
// (q8_0.rs:35-40, q4_0.rs:36-46: element 2i in the low nibble of byte i, 2i + 1 in the high one).
void dequant_matrix(const RawTensor& t, std::vector<float>* out) {
    if (t.fmt != 2) { dequant_flat(t, out); return; }
    const size_t n = t.count();
    out->resize(n);
    for (size_t blk = 0; blk < n / 32; blk++) {
        const uint8_t* p = t.data + blk * 18;
        uint16_t h; memcpy(&h, p, 2);
        const float s = f16_bits_to_f32(h);
        for (int j = 0; j < 32; j++) {
            const uint8_t q = p[2 + (j >> 1)];
            (*out)[blk * 32 + j] = ((float)((j & 1) ? (q >> 4) : (q & 0x0F)) - 8.0f) * s;
        }
    }
}

bool kept_quantised(const RawTensor& t) { return t.fmt != 0 && t.dims.size() == 2 && t.dims[1] % 32 == 0; }  // loader.rs:331, 351

int32_t upload_f32(lc_shard_engine* e, const std::vector<float>& v, float** out) {
    LC_TRY(dev_alloc(e, out, v.size()));
    LC_CUDA(cudaMemcpy(*out, v.data(), v.size() * 4, cudaMemcpyHostToDevice));
    e->weight_bytes += v.size() * 4;
    return LC_OK;
}

// Several [k][n_i] tensors of one shard side by side as one [k][sum n_i] device matrix (q, k, v share their input).
int32_t upload_matrix(lc_shard_engine* e, const std::vector<const RawTensor*>& parts, int k, ShardMat* m) {
    int n = 0;
    for (const RawTensor* t : parts) {
        LC_CHECK(t->dims.size() == 2 && (int)t->dims[0] == k, LC_ERR_INVALID, "shard matrix has %llu rows, %d expected",
                 (unsigned long long)(t->dims.empty() ? 0 : t->dims[0]), k);
        LC_CHECK(t->fmt == parts[0]->fmt, LC_ERR_INVALID, "shard matrices of one layer differ in format");
        n += (int)t->dims[1];
    }
    const bool quant = kept_quantised(*parts[0]);
    for (const RawTensor* t : parts) LC_CHECK(kept_quantised(*t) == quant, LC_ERR_UNSUPPORTED, "a projection's width is not a multiple of 32");
    m->k = k; m->n = n; m->fmt = quant ? parts[0]->fmt : 0;
    if (!quant) {
        std::vector<float> all((size_t)k * n), one;
        int c0 = 0;
        for (const RawTensor* t : parts) {
            dequant_flat(*t, &one);
            const int w = (int)t->dims[1];
            for (int r = 0; r < k; r++) memcpy(&all[(size_t)r * n + c0], &one[(size_t)r * w], (size_t)w * 4);
            c0 += w;
        }
        return upload_f32(e, all, &m->f32);
    }
    const int bpr = n / 32;
    std::vector<float> scales((size_t)k * bpr);
    const size_t qbytes = m->fmt == 1 ? (size_t)k * n : (size_t)k * n / 2, per = m->fmt == 1 ? 32 : 16;
    std::vector<uint8_t> qs(qbytes);
    int b0 = 0;
    for (const RawTensor* t : parts) {
        const int wb = (int)t->dims[1] / 32;
        for (int r = 0; r < k; r++)
            for (int bj = 0; bj < wb; bj++) {
                const uint8_t* p = t->data + ((size_t)r * wb + bj) * (2 + per);
                uint16_t h; memcpy(&h, p, 2);
                scales[(size_t)r * bpr + b0 + bj] = f16_bits_to_f32(h);
                memcpy(&qs[((size_t)r * bpr + b0 + bj) * per], p + 2, per);
            }
        b0 += wb;
    }
    LC_TRY(upload_f32(e, scales, &m->scales));
    uint8_t* dq = nullptr;
    LC_TRY(dev_alloc(e, &dq, qbytes));
    LC_CUDA(cudaMemcpy(dq, qs.data(), qbytes, cudaMemcpyHostToDevice));
    m->qs = dq;
    e->weight_bytes += qbytes;
    return LC_OK;
}

int32_t matmul(lc_shard_engine* e, const ShardMat& w, const float* a, int m, float* c) {
    switch (w.fmt) {
        case 0: return launch_matmul_f32(a, w.f32, (size_t)m, (size_t)w.k, (size_t)w.n, c, e->stream);
        case 1: return launch_q8_0_shard(a, w.scales, (const int8_t*)w.qs, (size_t)m, (size_t)w.k, (size_t)w.n, c, e->stream);
        default: return launch_q4_0_shard(a, w.scales, (const uint8_t*)w.qs, (size_t)m, (size_t)w.k, (size_t)w.n, c, e->stream);
    }
}

const RawTensor* find(const std::map<std::string, RawTensor>& ts, const char* name) {
    auto it = ts.find(name);
    return it == ts.end() ? nullptr : &it->second;
}

}  // namespace

// ShardEngine::load_with_cache (shard_engine.rs:27-61); every layer stays resident whatever cache_slots says.
extern "C" int32_t lc_shard_engine_load(const char* manifest_path, int32_t max_seq_len, int32_t device, lc_shard_engine** out) {
    LC_CHECK(manifest_path && out, LC_ERR_INVALID, "lc_shard_engine_load: null argument");
    *out = nullptr;
    if (!have_device()) return LC_ERR_CUDA;
    Mapping mm;
    LC_TRY(mm.open_file(manifest_path));
    JReader jr{(const char*)mm.base, (const char*)mm.base + mm.size};
    JValue man = jr.value();
    LC_CHECK(jr.ok && man.kind == JValue::OBJ, LC_ERR_INVALID, "%s: not a JSON object", manifest_path);
    auto num = [&](const char* k, double* v) { const JValue* j = man.get(k); if (!j || j->kind != JValue::NUM) return false; *v = j->num; return true; };
    double L, H, V, nh, nkv, F, ms, theta;
    LC_CHECK(num("num_layers", &L) && num("hidden_size", &H) && num("vocab_size", &V) && num("num_attention_heads", &nh) &&
                 num("num_key_value_heads", &nkv) && num("intermediate_size", &F) && num("max_seq_len", &ms) && num("rope_theta", &theta),
             LC_ERR_INVALID, "%s: a manifest field is missing (loader.rs:13-27)", manifest_path);
    const JValue* jdir = man.get("shard_dir");
    const JValue* jlayers = man.get("layers");
    const JValue* jspecial = man.get("special");
    LC_CHECK(jdir && jdir->kind == JValue::STR && jlayers && jlayers->kind == JValue::ARR && jspecial && jspecial->kind == JValue::OBJ,
             LC_ERR_INVALID, "%s: shard_dir, layers or special is missing", manifest_path);
    LC_CHECK((int)L >= 1 && (int)jlayers->arr.size() >= (int)L && (int)nh >= 1 && (int)nkv >= 1 && (int)H % (int)nh == 0 && (int)nh % (int)nkv == 0,
             LC_ERR_INVALID, "%s: inconsistent model geometry", manifest_path);

    lc_shard_engine* e = new lc_shard_engine();
    auto fail = [&](int32_t code) { std::string keep = get_error(); lc_shard_engine_destroy(e); set_error("%s", keep.c_str()); return code; };
#define SH_TRY(expr) do { int32_t _s = (expr); if (_s != LC_OK) return fail(_s); } while (0)
    e->device = device;
    if (cudaSetDevice(device) != cudaSuccess) { (void)cudaGetLastError(); set_error("cannot select device %d", device); return fail(LC_ERR_CUDA); }
    e->stream = lc::stream();
    e->L = (int)L; e->H = (int)H; e->V = (int)V; e->nh = (int)nh; e->nkv = (int)nkv; e->F = (int)F; e->theta = (float)theta;
    e->hd = e->H / e->nh;
    e->nqkv = (e->nh + 2 * e->nkv) * e->hd;
    e->max_seq = max_seq_len > 0 ? max_seq_len : (int)ms;
    const std::string dir = jdir->str;
    auto path_of = [&](const std::string& f) { return dir.empty() ? f : dir + "/" + f; };
    const int nq = e->nh * e->hd, nkvd = e->nkv * e->hd;

    // special weights (loader.rs:173-197): embedding table, final norm, head
    {
        const char* keys[3] = {"embed", "norm", "lm_head"};
        std::map<std::string, RawTensor> ts;
        Mapping maps[3];
        for (int i = 0; i < 3; i++) {
            const JValue* f = jspecial->get(keys[i]);
            if (!f || f->kind != JValue::STR) { set_error("%s: special.%s is missing", manifest_path, keys[i]); return fail(LC_ERR_INVALID); }
            SH_TRY(maps[i].open_file(path_of(f->str)));
            SH_TRY(parse_shard(path_of(f->str), maps[i], &ts));
        }
        const RawTensor* te = find(ts, "model.embed_tokens.weight");
        const RawTensor* tn = find(ts, "model.norm.weight");
        const RawTensor* th = find(ts, "lm_head.weight");
        if (!te || !tn || !th) { set_error("%s: missing embed_tokens, final norm or lm_head", manifest_path); return fail(LC_ERR_MISSING); }
        if (te->dims.size() != 2 || (int)te->dims[1] != e->H || (int)tn->count() != e->H) { set_error("special weights do not match hidden_size %d", e->H); return fail(LC_ERR_INVALID); }
        e->V = (int)te->dims[0];
        std::vector<float> v;
        if (kept_quantised(*te)) dequant_matrix(*te, &v); else dequant_flat(*te, &v);
        SH_TRY(upload_f32(e, v, &e->embed));
        dequant_flat(*tn, &v);
        SH_TRY(upload_f32(e, v, &e->final_norm));
        SH_TRY(upload_matrix(e, {th}, e->H, &e->head));
    }
    e->layers.resize(e->L);
    for (int l = 0; l < e->L; l++) {
        const JValue& jl = jlayers->arr[l];
        const JValue* f = jl.get("file");
        if (!f || f->kind != JValue::STR) { set_error("%s: layers[%d].file is missing", manifest_path, l); return fail(LC_ERR_INVALID); }
        Mapping mp;
        std::map<std::string, RawTensor> ts;
        SH_TRY(mp.open_file(path_of(f->str)));
        SH_TRY(parse_shard(path_of(f->str), mp, &ts));
        const char* names[9] = {"self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                                "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight", "input_layernorm.weight",
                                "post_attention_layernorm.weight"};
        const RawTensor* t[9];
        for (int i = 0; i < 9; i++) {
            t[i] = find(ts, names[i]);
            if (!t[i]) { set_error("layer %d: missing %s", l, names[i]); return fail(LC_ERR_MISSING); }
        }
        lc_shard_engine::Layer& w = e->layers[l];
        if ((int)t[0]->dims[1] != nq || (int)t[1]->dims[1] != nkvd || (int)t[2]->dims[1] != nkvd) { set_error("layer %d: projection widths do not match the head counts", l); return fail(LC_ERR_INVALID); }
        SH_TRY(upload_matrix(e, {t[0], t[1], t[2]}, e->H, &w.qkv));
        SH_TRY(upload_matrix(e, {t[3]}, nq, &w.o));
        SH_TRY(upload_matrix(e, {t[4]}, e->H, &w.gate));
        SH_TRY(upload_matrix(e, {t[5]}, e->H, &w.up));
        SH_TRY(upload_matrix(e, {t[6]}, e->F, &w.down));
        if (w.o.n != e->H || w.gate.n != e->F || w.up.n != e->F || w.down.n != e->H) { set_error("layer %d: matrix shapes do not match the manifest", l); return fail(LC_ERR_INVALID); }
        std::vector<float> v;
        dequant_flat(*t[7], &v);
        if ((int)v.size() != e->H) { set_error("layer %d: norm length", l); return fail(LC_ERR_INVALID); }
        SH_TRY(upload_f32(e, v, &w.in_norm));
        dequant_flat(*t[8], &v);
        SH_TRY(upload_f32(e, v, &w.post_norm));
    }
    // KV cache and step buffers
    e->pages = (e->max_seq + 15) / 16;
    const size_t pool = (size_t)e->pages * e->nkv * 16 * e->hd;
    for (int l = 0; l < e->L; l++) {
        __half *k = nullptr, *v = nullptr;
        SH_TRY(dev_alloc(e, &k, pool));
        SH_TRY(dev_alloc(e, &v, pool));
        e->k_pools.push_back(k);
        e->v_pools.push_back(v);
    }
    {
        std::vector<int32_t> pt(e->pages);
        for (int i = 0; i < e->pages; i++) pt[i] = i;
        SH_TRY(dev_alloc(e, &e->d_page_table, pt.size()));
        if (cudaMemcpy(e->d_page_table, pt.data(), pt.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) { set_error("page table upload failed"); return fail(LC_ERR_CUDA); }
    }
    const int C = lc_shard_engine::kChunk;
    SH_TRY(dev_alloc(e, &e->d_tokens, C)); SH_TRY(dev_alloc(e, &e->d_seq, C)); SH_TRY(dev_alloc(e, &e->d_pos, C)); SH_TRY(dev_alloc(e, &e->d_rope, C));
    SH_TRY(dev_alloc(e, &e->d_hidden, (size_t)C * e->H)); SH_TRY(dev_alloc(e, &e->d_hidden2, (size_t)C * e->H));
    SH_TRY(dev_alloc(e, &e->d_norm, (size_t)C * e->H)); SH_TRY(dev_alloc(e, &e->d_qkv, (size_t)C * e->nqkv));
    SH_TRY(dev_alloc(e, &e->d_attn, (size_t)C * nq)); SH_TRY(dev_alloc(e, &e->d_o, (size_t)C * e->H));
    SH_TRY(dev_alloc(e, &e->d_g, (size_t)C * e->F)); SH_TRY(dev_alloc(e, &e->d_u, (size_t)C * e->F)); SH_TRY(dev_alloc(e, &e->d_act, (size_t)C * e->F));
    SH_TRY(dev_alloc(e, &e->d_logits, (size_t)e->V)); SH_TRY(dev_alloc(e, &e->d_next, 1));
    size_t sc = 16;
    for (int t = 1; t <= C; t++) sc = std::max(sc, attention_scratch_bytes(t, e->nh, e->hd, e->max_seq));
    uint8_t* scratch = nullptr;
    SH_TRY(dev_alloc(e, &scratch, sc));
    e->d_scratch = scratch;
    SH_TRY(dev_alloc(e, &e->d_counters, (size_t)C * e->nh));
    if (cudaMemset(e->d_counters, 0, (size_t)C * e->nh * sizeof(int)) != cudaSuccess || cudaMemset(e->d_seq, 0, C * 4) != cudaSuccess) { set_error("clearing step buffers failed"); return fail(LC_ERR_CUDA); }
#undef SH_TRY
    *out = e;
    return LC_OK;
}

extern "C" int32_t lc_shard_engine_destroy(lc_shard_engine* e) {
    if (!e) return LC_OK;
    cudaSetDevice(e->device);
    if (e->stream) cudaStreamSynchronize(e->stream);
    for (void* p : e->owned) cudaFree(p);
    delete e;
    return LC_OK;
}

extern "C" int32_t lc_shard_engine_reset_kv_cache(lc_shard_engine* e) {  // shard_engine.rs:64-66
    LC_CHECK(e, LC_ERR_INVALID, "null engine");
    e->seq_len = 0;
    return LC_OK;
}

extern "C" int32_t lc_shard_engine_kv_cache_memory_bytes(lc_shard_engine* e, uint64_t* out) {  // cache/mod.rs:79-84: f16 keys and values held
    LC_CHECK(e && out, LC_ERR_INVALID, "null argument");
    *out = (uint64_t)e->seq_len * e->L * 2 * e->nkv * e->hd * 2;
    return LC_OK;
}

// ShardEngine::forward (shard_engine.rs:99-167): logits of the last token; the cache grows by n.
extern "C" int32_t lc_shard_engine_forward(lc_shard_engine* e, const int64_t* tokens, int32_t n, float* logits_out, int64_t* next_out) {
    LC_CHECK(e && tokens && n >= 1, LC_ERR_INVALID, "lc_shard_engine_forward: bad argument");
    LC_CHECK(e->seq_len + n <= e->max_seq, LC_ERR_INVALID, "%d cached + %d new tokens exceed max_seq_len %d", e->seq_len, n, e->max_seq);
    LC_CUDA(cudaSetDevice(e->device));
    const int C = lc_shard_engine::kChunk, H = e->H, F = e->F, nq = e->nh * e->hd;
    cudaStream_t s = e->stream;
    for (int c0 = 0; c0 < n; c0 += C) {
        const int T = std::min(C, n - c0);
        std::vector<int32_t> pos(T), rope(T);
        for (int t = 0; t < T; t++) { pos[t] = e->seq_len + t; rope[t] = c0 + t; }  // rotary index = position inside the call (attention.rs:13-21)
        LC_CUDA(cudaMemcpyAsync(e->d_tokens, tokens + c0, (size_t)T * 8, cudaMemcpyHostToDevice, s));
        LC_CUDA(cudaMemcpyAsync(e->d_pos, pos.data(), (size_t)T * 4, cudaMemcpyHostToDevice, s));
        LC_CUDA(cudaMemcpyAsync(e->d_rope, rope.data(), (size_t)T * 4, cudaMemcpyHostToDevice, s));
        LC_CUDA(cudaStreamSynchronize(s));  // the host vectors die with this iteration
        LC_TRY(launch_embed(LC_TYPE_F32, e->embed, (size_t)e->V, (size_t)H, e->d_tokens, T, e->d_hidden, s));
        for (int l = 0; l < e->L; l++) {
            lc_shard_engine::Layer& w = e->layers[l];
            KvLayout kv;
            kv.k_pool = e->k_pools[l]; kv.v_pool = e->v_pools[l]; kv.n_kv = e->nkv; kv.hd = e->hd; kv.page_tokens = 16; kv.kv_f32 = 0;
            kv.pool_pages = e->pages;
            LC_TRY(launch_rms_norm(e->d_hidden, w.in_norm, 1e-5f, (size_t)H, (size_t)T, e->d_norm, s));
            LC_TRY(matmul(e, w.qkv, e->d_norm, T, e->d_qkv));
            float* q = e->d_qkv;
            float* k = q + nq;
            float* v = k + e->nkv * e->hd;
            LC_TRY(launch_rope_kv_append(q, k, v, e->nqkv, T, e->nh, kv, e->d_seq, e->d_pos, e->d_rope, e->d_page_table, e->pages, e->theta, s));
            LC_TRY(launch_attention(q, e->nqkv, e->d_attn, T, e->nh, kv, e->d_seq, e->d_pos, e->d_page_table, e->pages, e->max_seq, e->d_scratch,
                                    e->d_counters, nullptr, s));
            LC_TRY(matmul(e, w.o, e->d_attn, T, e->d_o));
            LC_TRY(launch_vec_add(e->d_hidden, e->d_o, (size_t)T * H, e->d_hidden2, s));
            LC_TRY(launch_rms_norm(e->d_hidden2, w.post_norm, 1e-5f, (size_t)H, (size_t)T, e->d_norm, s));
            LC_TRY(matmul(e, w.gate, e->d_norm, T, e->d_g));
            LC_TRY(matmul(e, w.up, e->d_norm, T, e->d_u));
            LC_TRY(launch_silu_mul(e->d_g, e->d_u, (size_t)T * F, e->d_act, s));
            LC_TRY(matmul(e, w.down, e->d_act, T, e->d_o));
            LC_TRY(launch_vec_add(e->d_hidden2, e->d_o, (size_t)T * H, e->d_hidden, s));
        }
        e->seq_len += T;
        if (c0 + T == n) {
            LC_TRY(launch_rms_norm(e->d_hidden + (size_t)(T - 1) * H, e->final_norm, 1e-5f, (size_t)H, 1, e->d_norm, s));
            LC_TRY(matmul(e, e->head, e->d_norm, 1, e->d_logits));
            LC_TRY(launch_argmax(e->d_logits, (size_t)e->V, 1, e->d_next, s));
        }
    }
    if (logits_out) LC_CUDA(cudaMemcpyAsync(logits_out, e->d_logits, (size_t)e->V * 4, cudaMemcpyDeviceToHost, s));
    if (next_out) LC_CUDA(cudaMemcpyAsync(next_out, e->d_next, 8, cudaMemcpyDeviceToHost, s));
    LC_CUDA(cudaStreamSynchronize(s));
    return LC_OK;
}

// ShardEngine::generate (shard_engine.rs:74-97): clears the cache, first token from the prefill, stops after token 2.
extern "C" int32_t lc_shard_engine_set_seed(lc_shard_engine* e, uint64_t seed) {
    LC_CHECK(e != nullptr, LC_ERR_INVALID, "lc_shard_engine_set_seed: null engine");
    e->seeded = true;
    e->seed = seed;
    e->draws = 0;
    return LC_OK;
}

extern "C" int32_t lc_shard_engine_generate(lc_shard_engine* e, const int64_t* tokens, int32_t n, int32_t max_tokens, float temperature, float top_p,
                                            int64_t* out_tokens, int32_t* n_out) {
    LC_CHECK(e && tokens && n >= 1 && max_tokens >= 1 && out_tokens && n_out, LC_ERR_INVALID, "lc_shard_engine_generate: bad argument");
    const bool stochastic = temperature > 0.f;
    LC_CHECK(!stochastic || e->seeded, LC_ERR_UNSUPPORTED,
             "sampling with temperature > 0 draws from an unseeded generator in the reference (rust/src/inference/sampler.rs:38-39); call "
             "lc_shard_engine_set_seed first, or pass temperature <= 0 for greedy");
    // sample_top_p on the logits the forward left on the device (shard_engine.rs:82, 90)
    auto pick = [&](int64_t* tok) -> int32_t {
        if (!stochastic) return LC_OK;
        LC_CUDA(cudaSetDevice(e->device));
        return sample_top_p_sync(e->d_logits, (size_t)e->V, temperature, top_p, seeded_uniform(e->seed, e->draws++), tok, e->stream);
    };
    e->seq_len = 0;
    int64_t next = 0;
    LC_TRY(lc_shard_engine_forward(e, tokens, n, nullptr, &next));
    LC_TRY(pick(&next));
    int count = 0;
    out_tokens[count++] = next;
    while (next != 2 && count < max_tokens) {
        LC_TRY(lc_shard_engine_forward(e, &next, 1, nullptr, &next));
        LC_TRY(pick(&next));
        out_tokens[count++] = next;
    }
    *n_out = count;
    return LC_OK;
}

// GGUF v3 file loading (Engine::load(path), rust/src/inference/engine.rs:18-49): the container parser
// (rust/src/model/gguf.rs:76-330), the configuration keys (rust/src/model/loader.rs:106-141) and the architecture switch
// (rust/src/model/arch.rs:24-75).  The file is mapped read-only; every tensor the engine uses is handed to
// lc_model_set_tensor as the raw blocks the file holds -- nothing is dequantised or transposed on the way.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>
#include "lc_kernels.h"

using namespace lc;

namespace {

constexpr uint32_t kMagic = 0x46554747;  // "GGUF" little-endian (gguf.rs:12)
constexpr uint32_t kVersion = 3;         // gguf.rs:13

struct Value {
    enum Kind { NONE, INT, FLOAT, BOOL, STRING, ARRAY } kind = NONE;
    int64_t i = 0;        // INT / BOOL; ARRAY: element count
    double f = 0.0;       // FLOAT
    std::string s;        // STRING
    bool one_int = false; // ARRAY of exactly one integer (gguf.rs:145-153 reads it as that integer)
};

struct TensorInfo {
    std::string name;
    std::vector<uint64_t> dims;
    uint32_t typ = 0;
    uint64_t offset = 0;
};

struct Reader {
    const uint8_t* p;
    size_t n, pos = 0;
    bool ok = true;
    bool need(size_t k) {
        if (!ok || k > n - pos) { ok = false; return false; }
        return true;
    }
    template <typename T>
    T get() {
        T v{};
        if (need(sizeof(T))) { memcpy(&v, p + pos, sizeof(T)); pos += sizeof(T); }
        return v;
    }
    std::string str() {
        uint64_t len = get<uint64_t>();
        if (!need(len)) return std::string();
        std::string s((const char*)p + pos, (size_t)len);
        pos += (size_t)len;
        return s;
    }
    // gguf.rs:186-214: value types 0..12
    Value value(uint32_t typ, int depth = 0) {
        Value v;
        switch (typ) {
            case 0: v.kind = Value::INT; v.i = get<uint8_t>(); break;
            case 1: v.kind = Value::INT; v.i = get<int8_t>(); break;
            case 2: v.kind = Value::INT; v.i = get<uint16_t>(); break;
            case 3: v.kind = Value::INT; v.i = get<int16_t>(); break;
            case 4: v.kind = Value::INT; v.i = get<uint32_t>(); break;
            case 5: v.kind = Value::INT; v.i = get<int32_t>(); break;
            case 6: v.kind = Value::FLOAT; v.f = get<float>(); break;
            case 7: v.kind = Value::BOOL; v.i = get<uint8_t>() != 0; break;
            case 8: v.kind = Value::STRING; v.s = str(); break;
            case 9: {
                uint32_t et = get<uint32_t>();
                uint64_t len = get<uint64_t>();
                v.kind = Value::ARRAY;
                v.i = (int64_t)len;
                if (depth > 4) { ok = false; break; }
                for (uint64_t k = 0; k < len && ok; k++) {
                    Value e = value(et, depth + 1);  // walked to find the end; only a lone integer is kept
                    if (len == 1 && e.kind == Value::INT) { v.one_int = true; v.f = (double)e.i; }
                }
                break;
            }
            case 10: v.kind = Value::INT; v.i = (int64_t)get<uint64_t>(); break;
            case 11: v.kind = Value::INT; v.i = get<int64_t>(); break;
            case 12: v.kind = Value::FLOAT; v.f = get<double>(); break;
            default: ok = false;
        }
        return v;
    }
};

// get_metadata_int (gguf.rs:128-156): integers as they are, floats truncated, one-element integer arrays unwrapped
bool meta_int(const std::map<std::string, Value>& md, const std::string& key, int64_t* out) {
    auto it = md.find(key);
    if (it == md.end()) return false;
    const Value& v = it->second;
    if (v.kind == Value::INT) { *out = v.i; return true; }
    if (v.kind == Value::FLOAT) { *out = (int64_t)v.f; return true; }
    if (v.kind == Value::ARRAY && v.one_int) { *out = (int64_t)v.f; return true; }
    return false;
}

struct Mapping {
    int fd = -1;
    void* base = MAP_FAILED;
    size_t size = 0;
    ~Mapping() {
        if (base != MAP_FAILED) munmap(base, size);
        if (fd >= 0) close(fd);
    }
};

struct Parsed {
    Mapping mp;
    std::map<std::string, Value> md;
    std::vector<TensorInfo> infos;
    uint64_t data_offset = 0;
};

// GGUFile::open (gguf.rs:76-119): header, metadata, tensor table, start of the aligned data section.
int32_t parse_gguf(const char* path, Parsed* out) {
    Mapping& mp = out->mp;
    mp.fd = open(path, O_RDONLY);
    LC_CHECK(mp.fd >= 0, LC_ERR_INVALID, "cannot open %s", path);
    struct stat st;
    LC_CHECK(fstat(mp.fd, &st) == 0 && st.st_size >= 24, LC_ERR_INVALID, "%s: not a GGUF file (too short)", path);
    mp.size = (size_t)st.st_size;
    mp.base = mmap(nullptr, mp.size, PROT_READ, MAP_PRIVATE, mp.fd, 0);
    LC_CHECK(mp.base != MAP_FAILED, LC_ERR_INVALID, "cannot map %s", path);

    Reader r{(const uint8_t*)mp.base, mp.size};
    const uint32_t magic = r.get<uint32_t>(), version = r.get<uint32_t>();
    const uint64_t n_tensors = r.get<uint64_t>(), n_meta = r.get<uint64_t>();
    LC_CHECK(magic == kMagic, LC_ERR_INVALID, "%s: invalid GGUF magic %#x", path, magic);                 // gguf.rs:84-86
    LC_CHECK(version == kVersion, LC_ERR_UNSUPPORTED, "%s: unsupported GGUF version %u", path, version);  // gguf.rs:87-89
    LC_CHECK(n_tensors < (1u << 24) && n_meta < (1u << 24), LC_ERR_INVALID, "%s: implausible header counts", path);

    std::map<std::string, Value>& md = out->md;
    for (uint64_t i = 0; i < n_meta && r.ok; i++) {
        std::string key = r.str();
        uint32_t typ = r.get<uint32_t>();
        md[key] = r.value(typ);
    }
    std::vector<TensorInfo>& infos = out->infos;
    infos.resize((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors && r.ok; i++) {
        TensorInfo& t = infos[(size_t)i];
        t.name = r.str();
        uint32_t nd = r.get<uint32_t>();
        if (nd > 4) { r.ok = false; break; }
        for (uint32_t d = 0; d < nd; d++) t.dims.push_back(r.get<uint64_t>());
        t.typ = r.get<uint32_t>();
        t.offset = r.get<uint64_t>();
    }
    LC_CHECK(r.ok, LC_ERR_INVALID, "%s: truncated or malformed GGUF header", path);  // gguf.rs GGUError::TruncatedData

    int64_t alignment = 32;  // gguf.rs:104-113
    (void)meta_int(md, "general.alignment", &alignment);
    LC_CHECK(alignment > 0, LC_ERR_INVALID, "%s: general.alignment is %lld", path, (long long)alignment);
    out->data_offset = (r.pos + (uint64_t)alignment - 1) / (uint64_t)alignment * (uint64_t)alignment;
    return LC_OK;
}

// GGUFModel::extract_config (loader.rs:106-141) over the architecture's key prefix (arch.rs:54-64).
void config_from_metadata(const std::map<std::string, Value>& md, lc_model_config* out) {
    // architecture -> key prefix (arch.rs:24-64): mistral and unknown files use the llama.* keys
    std::string arch = "llama";
    {
        auto it = md.find("general.architecture");
        if (it != md.end() && it->second.kind == Value::STRING) {
            const std::string& a = it->second.s;
            if (a == "qwen2" || a == "qwen35" || a == "phi" || a == "gemma") arch = a;
        }
    }
    auto pick = [&](const char* suffix, int64_t* v) {  // loader.rs:110-131: the architecture's key, then the fallbacks
        const std::string keys[4] = {arch + "." + suffix, std::string("llama.") + suffix, std::string("qwen2.") + suffix,
                                     std::string("qwen35.") + suffix};
        for (const std::string& k : keys)
            if (meta_int(md, k, v)) return true;
        return false;
    };
    lc_model_config cfg;
    memset(&cfg, 0, sizeof(cfg));
    // ModelConfig::default (loader.rs:24-37)
    cfg.hidden_size = 4096; cfg.num_layers = 32; cfg.num_heads = 32; cfg.num_kv_heads = 32; cfg.intermediate_size = 11008;
    cfg.max_seq_len = 4096; cfg.vocab_size = 32000; cfg.rope_theta = 10000.0f;
    int64_t v = 0;
    if (pick("embedding_length", &v)) cfg.hidden_size = (int32_t)v;
    if (pick("block_count", &v)) cfg.num_layers = (int32_t)v;
    if (pick("attention.head_count", &v)) cfg.num_heads = (int32_t)v;
    if (pick("attention.head_count_kv", &v)) cfg.num_kv_heads = (int32_t)v;
    if (pick("feed_forward_length", &v)) cfg.intermediate_size = (int32_t)v;
    if (pick("context_length", &v)) cfg.max_seq_len = (int32_t)v;
    if (meta_int(md, arch + ".vocab_size", &v) || meta_int(md, "tokenizer.ggml.tokens.length", &v) ||
        meta_int(md, "tokenizer.ggml.vocab_size", &v)) {
        cfg.vocab_size = (int32_t)v;
    } else {
        auto it = md.find("tokenizer.ggml.tokens");  // loader.rs:124-128: the length of the token list
        if (it != md.end() && it->second.kind == Value::ARRAY) cfg.vocab_size = (int32_t)it->second.i;
    }
    if (pick("rope.freq_base", &v)) cfg.rope_theta = (float)v;  // loader.rs:130-131 (read through the integer accessor)
    // mixture-of-experts files (no counterpart in the reference's loader): <arch>.expert_count / <arch>.expert_used_count
    if (pick("expert_count", &v) && v > 0) {
        cfg.n_experts = (int32_t)v;
        cfg.top_k = pick("expert_used_count", &v) && v > 0 ? (int32_t)v : 2;
    }
    *out = cfg;
}

}  // namespace

extern "C" int32_t lc_model_load_gguf(const char* path, const lc_model_config* overrides, lc_model** out) {
    LC_CHECK(path && out, LC_ERR_INVALID, "lc_model_load_gguf: null argument");
    *out = nullptr;
    Parsed parsed;
    LC_TRY(parse_gguf(path, &parsed));
    Mapping& mp = parsed.mp;
    std::map<std::string, Value>& md = parsed.md;
    std::vector<TensorInfo>& infos = parsed.infos;
    const uint64_t data_offset = parsed.data_offset;

    lc_model_config cfg;
    config_from_metadata(md, &cfg);
    if (overrides) {
        // switches the file does not carry; a positive max_seq_len caps the KV capacity the model is built with
        if (overrides->max_seq_len > 0) cfg.max_seq_len = overrides->max_seq_len;
        cfg.rms_eps = overrides->rms_eps; cfg.kv_dtype = overrides->kv_dtype; cfg.rope_mode = overrides->rope_mode;
        cfg.max_seqs = overrides->max_seqs; cfg.kv_page_tokens = overrides->kv_page_tokens;
        cfg.kv_pool_tokens = overrides->kv_pool_tokens; cfg.device = overrides->device;
        cfg.tp_size = overrides->tp_size; cfg.tp_rank = overrides->tp_rank;  // a rank of a cut model reads the same file and keeps its part
    }

    lc_model* m = nullptr;
    LC_TRY(lc_model_create(&cfg, &m));
    auto fail = [&](int32_t code) { std::string keep = get_error(); lc_model_destroy(m); set_error("%s", keep.c_str()); return code; };
    for (const TensorInfo& t : infos) {
        const bool wanted = t.name.rfind("blk.", 0) == 0 || t.name == "token_embd.weight" || t.name == "output_norm.weight" ||
                            t.name == "output.weight";
        if (!wanted || t.dims.empty()) continue;
        int layer = -1;
        if (t.name.rfind("blk.", 0) == 0) layer = atoi(t.name.c_str() + 4);
        if (layer >= cfg.num_layers) continue;
        size_t count = 1;
        for (uint64_t d : t.dims) count *= (size_t)d;
        QuantGeom g;
        if (!quant_geom(t.typ, &g)) {
            set_error("%s: tensor %s has ggml type %u, which this library does not implement", path, t.name.c_str(), t.typ);
            return fail(LC_ERR_UNSUPPORTED);
        }
        const size_t nbytes = lc_tensor_bytes(t.typ, count);
        if (data_offset + t.offset > mp.size || nbytes > mp.size - (size_t)(data_offset + t.offset)) {
            set_error("%s: tensor %s reaches past the end of the file", path, t.name.c_str());
            return fail(LC_ERR_INVALID);
        }
        int32_t s = lc_model_set_tensor(m, t.name.c_str(), t.typ, t.dims.data(), (int32_t)t.dims.size(),
                                        (const uint8_t*)mp.base + data_offset + t.offset, nbytes);
        if (s != LC_OK) return fail(s);
    }
    int32_t s = lc_model_finalize(m);
    if (s != LC_OK) return fail(s);
    *out = m;
    return LC_OK;
}

// GGUFModel::capability_report (loader.rs:54-104) + scan_for_corruption (loader.rs:301-422).
extern "C" int32_t lc_gguf_inspect(const char* path, int32_t scan, lc_gguf_report* report, lc_corrupt_tensor* corrupt,
                                   int32_t corrupt_cap, char* names, size_t names_cap) {
    LC_CHECK(path && report, LC_ERR_INVALID, "lc_gguf_inspect: null argument");
    LC_CHECK(corrupt_cap == 0 || corrupt != nullptr, LC_ERR_INVALID, "lc_gguf_inspect: corrupt_cap without a buffer");
    memset(report, 0, sizeof(*report));
    if (names && names_cap) names[0] = 0;
    Parsed parsed;
    LC_TRY(parse_gguf(path, &parsed));
    config_from_metadata(parsed.md, &report->config);

    // ModelArchitecture::detect / name / is_supported (arch.rs:24-77)
    std::string arch_key;
    {
        auto it = parsed.md.find("general.architecture");
        if (it != parsed.md.end() && it->second.kind == Value::STRING) arch_key = it->second.s;
    }
    static const struct { const char* key; const char* name; bool supported; } kArch[] = {
        {"llama", "Llama", true}, {"qwen2", "Qwen2", true}, {"qwen35", "Qwen3.5", false},
        {"mistral", "Mistral", true}, {"phi", "Phi", false}, {"gemma", "Gemma", false}};
    const char* arch_name = "Unknown";
    bool arch_ok = false;
    for (const auto& a : kArch)
        if (arch_key == a.key) { arch_name = a.name; arch_ok = a.supported; }
    snprintf(report->architecture, sizeof(report->architecture), "%s", arch_name);
    report->arch_supported = arch_ok ? 1 : 0;

    // GGUFile::quant_summary (gguf.rs:317-331)
    report->total_tensors = (int32_t)parsed.infos.size();
    for (const TensorInfo& t : parsed.infos) {
        uint32_t e, bb;
        int kind;
        const bool known = t.typ == 0 || t.typ == 1 || t.typ == 30 || scan_geom(t.typ, &e, &bb, &kind);
        if (!known) continue;
        report->tensors_by_type[t.typ]++;
        QuantGeom g;
        if (!quant_geom(t.typ, &g)) report->unsupported_types |= 1u << t.typ;  // quant.rs:243-254: the same eight types
    }

    // missing tensors of the first layers, unrecognised blk.* tensors (loader.rs:59-89)
    static const char* kMapped[9] = {"attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight", "ffn_gate.weight",
                                     "ffn_up.weight", "ffn_down.weight", "attn_norm.weight", "ffn_norm.weight"};
    std::vector<std::string> extra_known;  // arch.rs:99-117
    if (arch_key == "qwen35")
        extra_known = {"attn_gate.weight", "attn_qkv.weight", "post_attention_norm.weight", "attn_q_norm.weight",
                       "attn_k_norm.weight", "attn_q.weight", "attn_v.weight"};
    else if (arch_key == "llama")
        extra_known = {"attn_norm.bias", "ffn_norm.bias"};
    std::map<std::string, const TensorInfo*> by_name;
    for (const TensorInfo& t : parsed.infos) by_name.emplace(t.name, &t);
    std::vector<std::string> missing, extra;
    const int sample_layers = report->config.num_layers < 4 ? report->config.num_layers : 4;
    for (int l = 0; l < sample_layers; l++)
        for (const char* sfx : kMapped) {
            std::string n = "blk." + std::to_string(l) + "." + sfx;
            if (!by_name.count(n)) missing.push_back(n);
        }
    auto ends_with = [](const std::string& s, const char* tail) {
        size_t n = strlen(tail);
        return s.size() >= n && s.compare(s.size() - n, n, tail) == 0;
    };
    for (const TensorInfo& t : parsed.infos) {
        if (t.name.rfind("blk.", 0) != 0 || !ends_with(t.name, ".weight")) continue;
        // splitn(3, '.').nth(2): what follows the second dot, or "" when there is none
        std::string sfx;
        size_t d1 = t.name.find('.');
        size_t d2 = d1 == std::string::npos ? d1 : t.name.find('.', d1 + 1);
        if (d2 != std::string::npos) sfx = t.name.substr(d2 + 1);
        bool known = false;
        for (const char* m : kMapped) known = known || sfx == m;
        for (const std::string& m : extra_known) known = known || sfx == m;
        if (!known) extra.push_back(t.name);
    }
    std::sort(extra.begin(), extra.end());
    extra.erase(std::unique(extra.begin(), extra.end()), extra.end());
    report->n_missing = (int32_t)missing.size();
    report->n_extra = (int32_t)extra.size();
    report->can_run = (arch_ok && report->unsupported_types == 0 && missing.empty()) ? 1 : 0;
    if (names && names_cap) {
        std::string text;
        for (const std::string& n : missing) text += "missing " + n + "\n";
        for (const std::string& n : extra) text += "extra " + n + "\n";
        snprintf(names, names_cap, "%s", text.c_str());
    }
    if (!scan) return LC_OK;

    // scan_for_corruption: every tensor of a block type, in file order
    if (!have_device()) return LC_ERR_CUDA;
    for (const TensorInfo& t : parsed.infos) {
        uint32_t e, bb;
        int kind;
        if (!scan_geom(t.typ, &e, &bb, &kind)) continue;
        size_t count = 1;  // an empty dimension list multiplies out to 1 (loader.rs:324)
        for (uint64_t d : t.dims) count *= (size_t)d;
        const size_t nbytes = (count + e - 1) / e * bb;
        const uint64_t start = parsed.data_offset + t.offset;
        LC_CHECK(start <= parsed.mp.size && nbytes <= parsed.mp.size - (size_t)start, LC_ERR_INVALID,
                 "%s: tensor %s reaches past the end of the file", path, t.name.c_str());
        uint64_t total = 0, bad = 0;
        LC_TRY(lc_scan_blocks(t.typ, (const uint8_t*)parsed.mp.base + start, count, &total, &bad));
        if (bad == 0) continue;
        if (report->n_corrupt_tensors < corrupt_cap) {
            lc_corrupt_tensor& c = corrupt[report->n_corrupt_tensors];
            memset(&c, 0, sizeof(c));
            snprintf(c.name, sizeof(c.name), "%s", t.name.c_str());
            c.ggml_type = t.typ;
            c.blocks_total = total;
            c.blocks_bad = bad;
        }
        report->n_corrupt_tensors++;
        report->total_blocks_checked += total;
        report->total_bad_blocks += bad;
    }
    return LC_OK;
}

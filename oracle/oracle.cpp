// CPU oracle for the LeafcutterLLM token-generation path.
//
// TEST INFRASTRUCTURE ONLY.  This file is a plain C++ restatement of the
// reference Rust crate's CPU arithmetic (file:line citations are paths inside
// the reference project).  It exists so that the CUDA path can be checked
// against it; nothing in the shipped library links, imports or calls it.
//
// Parity pin: the reference cannot be compiled in this build environment (no
// Rust toolchain), so the restatement is pinned against the known-answer
// values held by the reference's own unit tests (tests/golden/reference_kat.json
// lists them with their citations).  Those tests do not cover non-trivial
// Q4_K/Q5_K/Q6_K values, RoPE, attention, RMSNorm values, SiLU/FFN or
// end-to-end logits; for those this restatement itself is the pin
// ("parity unpinned" beyond the known-answer set).
//
// Arithmetic rules that must hold for bit-faithfulness (compile with
// -ffp-contract=off; fused multiply-add appears only where the reference uses
// an FMA intrinsic):
//   * matmul: every output element is one k-ascending chain
//     acc = fma(a[i,k], b[k,j], acc) from 0 (rust/src/kernels/simd.rs:226-249);
//     columns past the last multiple of 8 use unfused mul+add (:238-246).
//   * sum of squares: 4 strided lanes, unfused mul then add, lanes summed
//     0..3, then the scalar tail (simd.rs:373-410).
//   * everything else is scalar f32 in source order with glibc libm.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>
#include <chrono>
#ifdef _OPENMP
#include <omp.h>
#include "../leafcutterllm_b200/csrc/lc_synth.h"
#endif


namespace {

// ---------------------------------------------------------------------------
// f16 <-> f32, IEEE round-to-nearest-even.  Restates the `half` crate 2.7.1
// (rust/Cargo.lock:716-717) conversions used at rust/src/kernels/mod.rs:24,45,
// 72-73 and rust/src/cache/mod.rs:35-36,46-48,71-73.
// ---------------------------------------------------------------------------
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t man = x & 0x007FFFFFu;
    int32_t exp = (int32_t)((x >> 23) & 0xFFu);
    if (exp == 255) {  // inf / nan
        if (man == 0) return (uint16_t)(sign | 0x7C00u);
        return (uint16_t)(sign | 0x7C00u | 0x0200u | (man >> 13));
    }
    int32_t e = exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);  // overflow -> inf
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;  // underflow -> signed zero
        man |= 0x00800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half_man = man >> 13;
    uint32_t rem = man & 0x1FFFu;
    uint16_t out = (uint16_t)(sign | ((uint32_t)e << 10) | half_man);
    if (rem > 0x1000u || (rem == 0x1000u && (half_man & 1u))) out++;  // carries into exponent correctly
    return out;
}

inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// ---------------------------------------------------------------------------
// Block dequantisation: rust/src/kernels/mod.rs
// ---------------------------------------------------------------------------
constexpr int QK_K = 256;

// mod.rs:16-34
void dequantize_q4_0(const uint8_t* data, float* out, size_t n) {
    size_t nb = n / 32;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 18;
        float scale = f16_to_f32(rd16(b));
        for (int j = 0; j < 16; j++) {
            uint8_t qs = b[2 + j];
            float q0 = (float)(qs & 0x0F) - 8.0f;
            float q1 = (float)(qs >> 4) - 8.0f;
            out[i * 32 + j] = q0 * scale;
            out[i * 32 + j + 16] = q1 * scale;
        }
    }
}

// mod.rs:37-51
void dequantize_q8_0(const uint8_t* data, float* out, size_t n) {
    size_t nb = n / 32;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 34;
        float scale = f16_to_f32(rd16(b));
        for (int j = 0; j < 32; j++) out[i * 32 + j] = (float)(int8_t)b[2 + j] * scale;
    }
}

// mod.rs:54-63
inline void get_scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = q[j] & 0x3F;
        *m = q[j + 4] & 0x3F;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

// mod.rs:66-98
void dequantize_q4_k(const uint8_t* data, float* out, size_t n) {
    size_t nb = n / QK_K;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 144;
        float d = f16_to_f32(rd16(b));
        float dmin = f16_to_f32(rd16(b + 2));
        const uint8_t* scales = b + 4;
        const uint8_t* qs = b + 16;
        size_t idx = i * QK_K;
        int is = 0, q_off = 0;
        for (int j = 0; j < QK_K / 64; j++) {
            uint8_t sc1, m1, sc2, m2;
            get_scale_min_k4(is, scales, &sc1, &m1);
            get_scale_min_k4(is + 1, scales, &sc2, &m2);
            float dl1 = d * (float)sc1, dl2 = d * (float)sc2;
            float min1 = dmin * (float)m1, min2 = dmin * (float)m2;
            for (int l = 0; l < 32; l++) {
                out[idx + l] = dl1 * (float)(qs[q_off + l] & 0x0F) - min1;
                out[idx + l + 32] = dl2 * (float)(qs[q_off + l] >> 4) - min2;
            }
            idx += 64; q_off += 32; is += 2;
        }
    }
}

// mod.rs:101-142
void dequantize_q5_k(const uint8_t* data, float* out, size_t n) {
    size_t nb = n / QK_K;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 176;
        float d = f16_to_f32(rd16(b));
        float dmin = f16_to_f32(rd16(b + 2));
        const uint8_t* scales = b + 4;
        const uint8_t* qh = b + 16;
        const uint8_t* ql = b + 48;
        size_t idx = i * QK_K;
        int is = 0, ql_off = 0;
        uint8_t u1 = 1, u2 = 2;
        for (int j = 0; j < QK_K / 64; j++) {
            uint8_t sc1, m1, sc2, m2;
            get_scale_min_k4(is, scales, &sc1, &m1);
            get_scale_min_k4(is + 1, scales, &sc2, &m2);
            float dl1 = d * (float)sc1, dl2 = d * (float)sc2;
            float min1 = dmin * (float)m1, min2 = dmin * (float)m2;
            for (int l = 0; l < 32; l++) {
                uint8_t q = ql[ql_off + l] & 0x0F;
                if (qh[l] & u1) q += 16;
                out[idx + l] = dl1 * (float)q - min1;
                q = ql[ql_off + l] >> 4;
                if (qh[l] & u2) q += 16;
                out[idx + l + 32] = dl2 * (float)q - min2;
            }
            idx += 64; ql_off += 32; is += 2;
            u1 = (uint8_t)(u1 << 2); u2 = (uint8_t)(u2 << 2);
        }
    }
}

// mod.rs:145-180.  `d * scale as f32 * q as f32` associates left to right.
void dequantize_q6_k(const uint8_t* data, float* out, size_t n) {
    size_t nb = n / QK_K;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 210;
        const uint8_t* ql = b;
        const uint8_t* qh = b + 128;
        const int8_t* sc = (const int8_t*)(b + 192);
        float d = f16_to_f32(rd16(b + 208));
        size_t idx = i * QK_K;
        int ql_off = 0, qh_off = 0, sc_off = 0;
        for (int nn = 0; nn < QK_K / 128; nn++) {
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int8_t q1 = (int8_t)((int8_t)((ql[ql_off + l] & 0x0F) | (((qh[qh_off + l] >> 0) & 3) << 4)) - 32);
                int8_t q2 = (int8_t)((int8_t)((ql[ql_off + l + 32] & 0x0F) | (((qh[qh_off + l] >> 2) & 3) << 4)) - 32);
                int8_t q3 = (int8_t)((int8_t)((ql[ql_off + l] >> 4) | (((qh[qh_off + l] >> 4) & 3) << 4)) - 32);
                int8_t q4 = (int8_t)((int8_t)((ql[ql_off + l + 32] >> 4) | (((qh[qh_off + l] >> 6) & 3) << 4)) - 32);
                out[idx + l + 0] = d * (float)sc[sc_off + is + 0] * (float)q1;
                out[idx + l + 32] = d * (float)sc[sc_off + is + 2] * (float)q2;
                out[idx + l + 64] = d * (float)sc[sc_off + is + 4] * (float)q3;
                out[idx + l + 96] = d * (float)sc[sc_off + is + 6] * (float)q4;
            }
            idx += 128; ql_off += 64; qh_off += 32; sc_off += 8;
        }
    }
}

// mod.rs:186-216 (the reference's own float table and its interleaved element order)
const float IQ4NL_TABLE[16] = {-1.0f, -0.6962f, -0.5251f, -0.3952f, -0.2893f, -0.1957f, -0.1107f, -0.0322f,
                               0.0322f, 0.1107f, 0.1957f, 0.2893f, 0.3952f, 0.5251f, 0.6962f, 1.0f};
void dequantize_iq4_nl(const uint8_t* data, float* out, size_t n) {
    size_t nb = n / 32;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 18;
        float scale = f16_to_f32(rd16(b));
        for (int j = 0; j < 16; j++) {
            uint8_t qs = b[2 + j];
            out[i * 32 + j * 2] = scale * IQ4NL_TABLE[qs & 0x0F];
            out[i * 32 + j * 2 + 1] = scale * IQ4NL_TABLE[qs >> 4];
        }
    }
}

// rust/src/model/quant.rs:186-262 (block sizes / bytes of the supported set)
bool quant_geometry(uint32_t typ, size_t* block_elems, size_t* block_bytes) {
    switch (typ) {
        case 0: *block_elems = 1; *block_bytes = 4; return true;     // F32
        case 1: *block_elems = 1; *block_bytes = 2; return true;     // F16
        case 2: *block_elems = 32; *block_bytes = 18; return true;   // Q4_0
        case 8: *block_elems = 32; *block_bytes = 34; return true;   // Q8_0
        case 12: *block_elems = 256; *block_bytes = 144; return true;  // Q4_K
        case 13: *block_elems = 256; *block_bytes = 176; return true;  // Q5_K
        case 14: *block_elems = 256; *block_bytes = 210; return true;  // Q6_K
        case 20: *block_elems = 32; *block_bytes = 18; return true;  // IQ4_NL
        default: return false;
    }
}

// rust/src/model/loader.rs:205-235
int dequantize_any(uint32_t typ, const uint8_t* data, float* out, size_t n) {
    switch (typ) {
        case 0: memcpy(out, data, n * 4); return 0;
        case 1: for (size_t i = 0; i < n; i++) out[i] = f16_to_f32(rd16(data + 2 * i)); return 0;
        case 2: dequantize_q4_0(data, out, n); return 0;
        case 8: dequantize_q8_0(data, out, n); return 0;
        case 12: dequantize_q4_k(data, out, n); return 0;
        case 13: dequantize_q5_k(data, out, n); return 0;
        case 14: dequantize_q6_k(data, out, n); return 0;
        case 20: dequantize_iq4_nl(data, out, n); return 0;
        default: return -1;
    }
}

// loader.rs:241-249
size_t sanitize_weights(float* v, size_t n) {
    size_t hits = 0;
    for (size_t i = 0; i < n; i++) {
        if (std::isnan(v[i]) || std::isinf(v[i]) || std::fabs(v[i]) > 100.0f) { v[i] = 0.0f; hits++; }
    }
    return hits;
}

// ---------------------------------------------------------------------------
// f32 matmul: rust/src/kernels/simd.rs:226-249 (AVX2+FMA path, the one an
// x86-64 host with avx2+fma takes through simd.rs:269-311 and cpu.rs:13-23).
// b is [k,n] row-major as in the reference.
// ---------------------------------------------------------------------------
void matmul_kn(const float* a, const float* b, float* c, size_t m, size_t k, size_t n) {
    size_t n8 = n & ~(size_t)7;
#pragma omp parallel for schedule(static) collapse(2) if (m * n >= 4096)
    for (size_t i = 0; i < m; i++) {
        for (size_t j0 = 0; j0 < n8; j0 += 8) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (size_t l = 0; l < k; l++) {
                float av = a[i * k + l];
                const float* br = b + l * n + j0;
                for (int t = 0; t < 8; t++) acc[t] = __builtin_fmaf(av, br[t], acc[t]);
            }
            for (int t = 0; t < 8; t++) c[i * n + j0 + t] = acc[t];
        }
    }
    for (size_t i = 0; i < m; i++) {
        for (size_t j = n8; j < n; j++) {  // scalar tail: unfused
            float sum = 0.0f;
            for (size_t l = 0; l < k; l++) {
                float p = a[i * k + l] * b[l * n + j];
                sum = sum + p;
            }
            c[i * n + j] = sum;
        }
    }
}

// Same arithmetic, but the weight is held as [n,k] row-major (the GGUF order
// before the reference's transpose, loader.rs:158-160).  Each output is still
// one k-ascending chain, so results are bit-identical to matmul_kn on the
// transposed matrix; only the memory walk differs.
void matmul_nk(const float* a, const float* w, float* c, size_t m, size_t k, size_t n) {
    size_t n8 = n & ~(size_t)7;
#pragma omp parallel for schedule(static)
    for (size_t j0 = 0; j0 < n8; j0 += 8) {
        for (size_t i = 0; i < m; i++) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const float* ar = a + i * k;
            for (size_t l = 0; l < k; l++) {
                float av = ar[l];
                for (int t = 0; t < 8; t++) acc[t] = __builtin_fmaf(av, w[(j0 + t) * k + l], acc[t]);
            }
            for (int t = 0; t < 8; t++) c[i * n + j0 + t] = acc[t];
        }
    }
    for (size_t i = 0; i < m; i++) {
        for (size_t j = n8; j < n; j++) {
            float sum = 0.0f;
            for (size_t l = 0; l < k; l++) {
                float p = a[i * k + l] * w[j * k + l];
                sum = sum + p;
            }
            c[i * n + j] = sum;
        }
    }
}

// simd.rs:373-410
float sum_sq(const float* d, size_t len) {
    float lane[4] = {0, 0, 0, 0};
    size_t i = 0;
    while (i + 4 <= len) {
        for (int t = 0; t < 4; t++) {
            float p = d[i + t] * d[i + t];
            lane[t] = p + lane[t];
        }
        i += 4;
    }
    float s = 0.0f;
    for (int t = 0; t < 4; t++) s = s + lane[t];
    for (; i < len; i++) {
        float p = d[i] * d[i];
        s = s + p;
    }
    return s;
}

// cpu.rs:49-60 with simd.rs:335-370
void rms_norm(const float* x, const float* w, float eps, size_t hidden, size_t rows, float* out) {
    for (size_t r = 0; r < rows; r++) {
        const float* s = x + r * hidden;
        float mean_sq = sum_sq(s, hidden) / (float)hidden;
        float scale = 1.0f / sqrtf(mean_sq + eps);
        for (size_t i = 0; i < hidden; i++) {
            float t = s[i] * scale;
            out[r * hidden + i] = t * w[i];
        }
    }
}

// cpu.rs:62-64
inline float silu1(float v) { return v * (1.0f / (1.0f + expf(-v))); }

// cpu.rs:66-79
void softmax_rows(const float* x, size_t hidden, size_t rows, float* out) {
    for (size_t r = 0; r < rows; r++) {
        const float* s = x + r * hidden;
        float mx = -INFINITY;
        for (size_t i = 0; i < hidden; i++) mx = fmaxf(mx, s[i]);
        float sum = 0.0f;
        for (size_t i = 0; i < hidden; i++) sum = sum + expf(s[i] - mx);
        for (size_t i = 0; i < hidden; i++) out[r * hidden + i] = expf(s[i] - mx) / sum;
    }
}

// rust/src/inference/attention.rs:13-34.  `pos0` is an extension: the
// reference always rotates by the index inside the current call (pos0 = 0).
void apply_rotary_emb(float* x, size_t seq_len, size_t heads, size_t hd, float theta, size_t pos0) {
    for (size_t i = 0; i < seq_len; i++) {
        for (size_t h = 0; h < heads; h++) {
            for (size_t d = 0; d < hd / 2; d++) {
                float freq = 1.0f / powf(theta, 2.0f * (float)d / (float)hd);
                float angle = (float)(i + pos0) * freq;
                float ca = cosf(angle), sa = sinf(angle);
                size_t base = i * heads * hd + h * hd;
                float x1 = x[base + d], x2 = x[base + d + hd / 2];
                float a = x1 * ca, b = x2 * sa;
                x[base + d] = a - b;
                float c2 = x1 * sa, d2 = x2 * ca;
                x[base + d + hd / 2] = c2 + d2;
            }
        }
    }
}

// rust/src/inference/sampler.rs:6-10: max_by(total_cmp) keeps the LAST maximum.
inline int32_t total_key(float f) {
    int32_t b;
    memcpy(&b, &f, 4);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}
size_t argmax_last(const float* v, size_t n) {
    size_t best = 0;
    int32_t bk = total_key(v[0]);
    for (size_t i = 1; i < n; i++) {
        int32_t k = total_key(v[i]);
        if (k >= bk) { bk = k; best = i; }
    }
    return best;
}

// ---------------------------------------------------------------------------
// Model: rust/src/inference/engine.rs + attention.rs + cache/mod.rs +
// model/loader.rs
// ---------------------------------------------------------------------------
struct Config {  // loader.rs:13-22 (+ the switches this build adds)
    int32_t hidden_size, num_layers, num_heads, num_kv_heads, intermediate_size, max_seq_len, vocab_size;
    float rope_theta;
    float rms_eps;       // engine.rs:102,111,121 hard-code 1e-5
    int32_t kv_f32;      // 0: f16 storage as cache/mod.rs; 1: keep f32
    int32_t rope_absolute;  // 0: position inside the call (attention.rs:13-21); 1: absolute position
    int32_t n_experts;   // 0 = dense FFN.  MoE has no counterpart in the reference.
    int32_t top_k;
};

struct RawTensor {
    uint32_t typ;
    std::vector<uint64_t> dims;  // GGUF order (fastest first)
    std::vector<uint8_t> bytes;
    std::vector<float> f32;  // dequantised [rows, cols] = dims reversed (loader.rs:155), sanitised
    size_t rows = 0, cols = 0;
};

struct Model {
    Config cfg;
    std::map<std::string, RawTensor> tensors;
    // cache/mod.rs:9-16: per layer [T, n_kv, hd]; stored as f16 bit patterns (or f32 when kv_f32)
    std::vector<std::vector<uint16_t>> k16, v16;
    std::vector<std::vector<float>> k32, v32;
    bool cache_weights = true;
    int mode = 0;  // 0 cached dequantised weights; 1 reference-faithful per-call dequant + transpose
    size_t sanitized = 0;
    std::string err;
    double t_dequant = 0, t_matmul = 0, t_attn = 0;
};

// arch.rs:83-96 and loader.rs:173-177: GGUF name -> engine name is only a
// relabelling; the oracle keys on the GGUF names.

double now_s() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// loader.rs:145-168: dims reversed -> [rows=out, cols=in] row-major, dequantise, sanitise.
const RawTensor* get_dequant(Model* m, const std::string& name) {
    auto it = m->tensors.find(name);
    if (it == m->tensors.end()) return nullptr;
    RawTensor& t = it->second;
    if (t.f32.empty()) {
        size_t n = 1;
        for (auto d : t.dims) n *= d;
        t.f32.resize(n);
        dequantize_any(t.typ, t.bytes.data(), t.f32.data(), n);
        m->sanitized += sanitize_weights(t.f32.data(), n);
    }
    return &t;
}

// y[m,n] = x[m,k] . W^T with W the dequantised [n,k] tensor.
// mode 1 reproduces what engine.rs:96 + loader.rs:155-161 + tensor.rs:176-188
// do on every call: dequantise the whole tensor, transpose it with the scalar
// double loop, then run the [k,n] matmul.
void linear(Model* m, const std::string& name, const float* x, size_t rows, float* y) {
    if (m->mode == 1) {
        auto it = m->tensors.find(name);
        RawTensor& t = it->second;
        size_t n = t.rows, k = t.cols;
        double t0 = now_s();
        std::vector<float> deq(n * k), tr(n * k);
        dequantize_any(t.typ, t.bytes.data(), deq.data(), n * k);
        for (size_t i = 0; i < n; i++)
            for (size_t j = 0; j < k; j++) tr[j * n + i] = deq[i * k + j];
        sanitize_weights(tr.data(), n * k);
        double t1 = now_s();
        matmul_kn(x, tr.data(), y, rows, k, n);
        double t2 = now_s();
        m->t_dequant += t1 - t0;
        m->t_matmul += t2 - t1;
        return;
    }
    double t0 = now_s();
    const RawTensor* t = get_dequant(m, name);
    double t1 = now_s();
    matmul_nk(x, t->f32.data(), y, rows, t->cols, t->rows);
    double t2 = now_s();
    m->t_dequant += t1 - t0;
    m->t_matmul += t2 - t1;
    if (!m->cache_weights) {
        auto& tt = m->tensors[name];
        std::vector<float>().swap(tt.f32);
    }
}

// cache/mod.rs:33-61: append (f32 -> f16; the reference's decompress/recompress
// of the existing entries is an identity on their bit patterns).
void kv_append(Model* m, size_t layer, const float* k, const float* v, size_t count) {
    if (m->cfg.kv_f32) {
        m->k32[layer].insert(m->k32[layer].end(), k, k + count);
        m->v32[layer].insert(m->v32[layer].end(), v, v + count);
    } else {
        auto& K = m->k16[layer];
        auto& V = m->v16[layer];
        size_t o = K.size();
        K.resize(o + count);
        V.resize(o + count);
        for (size_t i = 0; i < count; i++) { K[o + i] = f32_to_f16(k[i]); V[o + i] = f32_to_f16(v[i]); }
    }
}

// attention.rs:37-118
void attention_forward(Model* m, size_t layer, const float* normed, size_t seq, float* out) {
    const Config& c = m->cfg;
    size_t H = c.hidden_size, nh = c.num_heads, nkv = c.num_kv_heads, hd = H / nh;
    std::string p = "blk." + std::to_string(layer) + ".";
    std::vector<float> q(seq * nh * hd), k(seq * nkv * hd), v(seq * nkv * hd);
    linear(m, p + "attn_q.weight", normed, seq, q.data());
    linear(m, p + "attn_k.weight", normed, seq, k.data());
    linear(m, p + "attn_v.weight", normed, seq, v.data());
    double t0 = now_s();
    size_t cache_len0 = (c.kv_f32 ? m->k32[layer].size() : m->k16[layer].size()) / (nkv * hd);
    size_t pos0 = c.rope_absolute ? cache_len0 : 0;
    apply_rotary_emb(q.data(), seq, nh, hd, c.rope_theta, pos0);
    apply_rotary_emb(k.data(), seq, nkv, hd, c.rope_theta, pos0);
    kv_append(m, layer, k.data(), v.data(), seq * nkv * hd);
    // cache/mod.rs:65-77: whole layer back to f32
    std::vector<float> kc, vc;
    if (c.kv_f32) {
        kc = m->k32[layer]; vc = m->v32[layer];
    } else {
        size_t tot = m->k16[layer].size();
        kc.resize(tot); vc.resize(tot);
        for (size_t i = 0; i < tot; i++) { kc[i] = f16_to_f32(m->k16[layer][i]); vc[i] = f16_to_f32(m->v16[layer][i]); }
    }
    size_t total = kc.size() / (nkv * hd);
    size_t groups = nh / nkv;
    std::vector<float> attn(seq * nh * hd, 0.0f);
    float inv = sqrtf((float)hd);
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (size_t h = 0; h < nh; h++) {
        for (size_t s = 0; s < seq; s++) {
            size_t kvh = h / groups;
            std::vector<float> scores(total);
            size_t cache_len = total - seq;
            for (size_t t = 0; t < total; t++) {
                if (t > cache_len + s) {
                    scores[t] = -INFINITY;
                } else {
                    float dot = 0.0f;
                    const float* qp = &q[s * nh * hd + h * hd];
                    const float* kp = &kc[t * nkv * hd + kvh * hd];
                    for (size_t d = 0; d < hd; d++) {
                        float pr = qp[d] * kp[d];
                        dot = dot + pr;
                    }
                    scores[t] = dot / inv;
                }
            }
            float mx = -INFINITY;
            for (size_t t = 0; t < total; t++) mx = fmaxf(mx, scores[t]);
            float esum = 0.0f;
            for (size_t t = 0; t < total; t++) esum = esum + expf(scores[t] - mx);
            for (size_t t = 0; t < total; t++) scores[t] = expf(scores[t] - mx) / esum;
            for (size_t d = 0; d < hd; d++) {
                float sum = 0.0f;
                for (size_t t = 0; t < total; t++) {
                    float pr = scores[t] * vc[t * nkv * hd + kvh * hd + d];
                    sum = sum + pr;
                }
                attn[s * nh * hd + h * hd + d] = sum;
            }
        }
    }
    m->t_attn += now_s() - t0;
    linear(m, p + "attn_output.weight", attn.data(), seq, out);
}

// engine.rs:146-164
void ffn_forward(Model* m, const std::string& p, const float* x, size_t seq, float* out) {
    size_t F = m->cfg.intermediate_size;
    std::vector<float> gate(seq * F), up(seq * F);
    linear(m, p + "ffn_gate.weight", x, seq, gate.data());
    linear(m, p + "ffn_up.weight", x, seq, up.data());
    for (size_t i = 0; i < seq * F; i++) gate[i] = silu1(gate[i]) * up[i];
    linear(m, p + "ffn_down.weight", gate.data(), seq, out);
}

// Mixture-of-experts FFN.  NO COUNTERPART IN THE REFERENCE (parity unpinned):
// router logits = x . W_r^T (f32 weights, same FMA chain as every matmul);
// top-k by value, ties to the highest index (the convention of sampler.rs:6-10);
// gate weights = softmax over the selected logits; output = sum over the
// selected experts in ascending expert index of weight * expert_ffn(x).
void moe_forward(Model* m, const std::string& p, const float* x, size_t seq, float* out) {
    const Config& c = m->cfg;
    size_t H = c.hidden_size, E = c.n_experts, K = c.top_k;
    std::vector<float> logits(seq * E);
    linear(m, p + "ffn_gate_inp.weight", x, seq, logits.data());
    std::vector<float> y(H);
    for (size_t s = 0; s < seq; s++) {
        std::vector<int> sel;
        std::vector<char> used(E, 0);
        for (size_t kk = 0; kk < K; kk++) {
            int best = -1;
            for (size_t e = 0; e < E; e++) {
                if (used[e]) continue;
                if (best < 0 || total_key(logits[s * E + e]) >= total_key(logits[s * E + best])) best = (int)e;
            }
            used[best] = 1;
            sel.push_back(best);
        }
        float mx = -INFINITY;
        for (int e : sel) mx = fmaxf(mx, logits[s * E + e]);
        std::vector<float> wsel(E, 0.0f);
        float sum = 0.0f;
        for (size_t e = 0; e < E; e++) if (used[e]) sum = sum + expf(logits[s * E + e] - mx);
        for (size_t e = 0; e < E; e++) if (used[e]) wsel[e] = expf(logits[s * E + e] - mx) / sum;
        for (size_t i = 0; i < H; i++) out[s * H + i] = 0.0f;
        for (size_t e = 0; e < E; e++) {
            if (!used[e]) continue;
            ffn_forward(m, p + "expert." + std::to_string(e) + ".", x + s * H, 1, y.data());
            for (size_t i = 0; i < H; i++) {
                float t = wsel[e] * y[i];
                out[s * H + i] = out[s * H + i] + t;
            }
        }
    }
}

// engine.rs:78-132
int forward(Model* m, const int64_t* tokens, size_t seq, float* logits_out, float* hidden_out) {
    const Config& c = m->cfg;
    size_t H = c.hidden_size, V = c.vocab_size;
    const RawTensor* emb = get_dequant(m, "token_embd.weight");
    if (!emb) { m->err = "missing token_embd.weight"; return -1; }
    std::vector<float> hidden(seq * H, 0.0f);
    for (size_t i = 0; i < seq; i++) {  // engine.rs:134-144: out-of-range id -> zero row
        if (tokens[i] >= 0 && (size_t)tokens[i] < emb->rows)
            memcpy(&hidden[i * H], &emb->f32[(size_t)tokens[i] * H], H * 4);
    }
    std::vector<float> normed(seq * H), tmp(seq * H);
    for (int l = 0; l < c.num_layers; l++) {
        std::string p = "blk." + std::to_string(l) + ".";
        const RawTensor* n1 = get_dequant(m, p + "attn_norm.weight");
        const RawTensor* n2 = get_dequant(m, p + "ffn_norm.weight");
        if (!n1 || !n2) { m->err = "missing norm in layer " + std::to_string(l); return -1; }
        rms_norm(hidden.data(), n1->f32.data(), c.rms_eps, H, seq, normed.data());
        attention_forward(m, l, normed.data(), seq, tmp.data());
        for (size_t i = 0; i < seq * H; i++) hidden[i] = hidden[i] + tmp[i];
        rms_norm(hidden.data(), n2->f32.data(), c.rms_eps, H, seq, normed.data());
        if (c.n_experts > 0) moe_forward(m, p, normed.data(), seq, tmp.data());
        else ffn_forward(m, p, normed.data(), seq, tmp.data());
        for (size_t i = 0; i < seq * H; i++) hidden[i] = hidden[i] + tmp[i];
    }
    const RawTensor* fn = get_dequant(m, "output_norm.weight");
    if (!fn) { m->err = "missing output_norm.weight"; return -1; }
    rms_norm(hidden.data(), fn->f32.data(), c.rms_eps, H, seq, normed.data());
    if (hidden_out) memcpy(hidden_out, &normed[(seq - 1) * H], H * 4);
    // engine.rs:123-131 computes every row and returns the last; each row is an
    // independent chain, so only the last row is evaluated here.
    // loader.rs:192-199: tied head when output.weight is absent.
    std::string head = m->tensors.count("output.weight") ? "output.weight" : "token_embd.weight";
    std::vector<float> logits(V);
    linear(m, head, &normed[(seq - 1) * H], 1, logits.data());
    memcpy(logits_out, logits.data(), V * 4);
    return 0;
}

}  // namespace

// ===========================================================================
// C interface for the Python test harness (ctypes)
// ===========================================================================
extern "C" {

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}

float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
void orc_f16_roundtrip(const float* in, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = f16_to_f32(f32_to_f16(in[i]));
}

int orc_dequantize(uint32_t typ, const uint8_t* data, size_t n_elems, float* out) {
    return dequantize_any(typ, data, out, n_elems);
}
size_t orc_sanitize(float* v, size_t n) { return sanitize_weights(v, n); }

// scan_for_corruption, the body run per tensor (rust/src/model/loader.rs:318-402).  Block sizes and bytes for every type
// code of QuantType::from_u32 (rust/src/model/quant.rs:71-100, 160-238).  Returns 0 and leaves the counts at zero for
// types the scan skips (F32, F16, BF16, unknown codes: loader.rs:309-322).
int orc_scan_blocks(uint32_t typ, const uint8_t* raw, size_t n_elems, uint64_t* blocks_total, uint64_t* blocks_bad) {
    *blocks_total = 0;
    *blocks_bad = 0;
    size_t bs = 0, bb = 0;
    switch (typ) {
        case 2: bs = 32; bb = 18; break;    case 3: bs = 32; bb = 20; break;    case 6: bs = 32; bb = 22; break;
        case 7: bs = 32; bb = 24; break;    case 8: bs = 32; bb = 34; break;    case 9: bs = 32; bb = 36; break;
        case 10: bs = 256; bb = 84; break;  case 11: bs = 256; bb = 110; break; case 12: bs = 256; bb = 144; break;
        case 13: bs = 256; bb = 176; break; case 14: bs = 256; bb = 210; break; case 15: bs = 256; bb = 292; break;
        case 16: bs = 256; bb = 66; break;  case 17: bs = 256; bb = 74; break;  case 18: bs = 256; bb = 98; break;
        case 19: bs = 256; bb = 110; break; case 20: bs = 32; bb = 18; break;   case 21: bs = 256; bb = 136; break;
        case 22: bs = 256; bb = 136; break; case 23: bs = 256; bb = 162; break; case 24: bs = 256; bb = 162; break;
        case 25: bs = 256; bb = 176; break;
        default: return 0;
    }
    const size_t num_blocks = (n_elems + bs - 1) / bs;  // loader.rs:325
    auto h = [](const uint8_t* p) { return f16_to_f32((uint16_t)(p[0] | (p[1] << 8))); };
    auto f = [](const uint8_t* p) { float v; memcpy(&v, p, 4); return v; };
    auto is_bad = [](float v) { return std::isnan(v) || std::isinf(v) || std::fabs(v) > 1e4f; };  // loader.rs:385-392
    uint64_t bad = 0;
    for (size_t i = 0; i < num_blocks; i++) {
        const uint8_t* block = raw + i * bb;
        float d, dmin = 0.0f;
        bool has_dmin = false;
        if (typ == 14) {          // Q6_K: the f16 at bytes 208..209 (loader.rs:341-349)
            d = h(block + 208);
        } else if (typ == 15) {   // Q8_K: f32 at 0 (loader.rs:350-357)
            d = f(block);
        } else if (typ == 9) {    // Q8_1: f32 at 0 and f32 at 4 (loader.rs:358-367)
            d = f(block);
            dmin = f(block + 4);
            has_dmin = true;
        } else {                  // every other type: f16 at 0, and f16 at 2 as dmin when the block has 4 bytes (loader.rs:368-381)
            d = h(block);
            if (bb >= 4) { dmin = h(block + 2); has_dmin = true; }
        }
        bool block_bad = is_bad(d);
        if (has_dmin && is_bad(dmin)) block_bad = true;
        if (block_bad) bad++;
    }
    *blocks_total = num_blocks;
    *blocks_bad = bad;
    return 0;
}
size_t orc_tensor_bytes(uint32_t typ, size_t count) {
    size_t be, bb;
    if (!quant_geometry(typ, &be, &bb)) return count;  // gguf.rs:307-313
    return (count + be - 1) / be * bb;
}

// Backend trait, rust/src/backend/mod.rs:18-46 via cpu.rs
void orc_matmul(const float* a, const float* b, size_t m, size_t k, size_t n, float* c) { matmul_kn(a, b, c, m, k, n); }
void orc_matmul_nk(const float* a, const float* w, size_t m, size_t k, size_t n, float* c) { matmul_nk(a, w, c, m, k, n); }
void orc_vec_add(const float* a, const float* b, size_t n, float* o) { for (size_t i = 0; i < n; i++) o[i] = a[i] + b[i]; }
void orc_vec_mul(const float* a, const float* b, size_t n, float* o) { for (size_t i = 0; i < n; i++) o[i] = a[i] * b[i]; }
void orc_vec_scale(const float* a, float s, size_t n, float* o) { for (size_t i = 0; i < n; i++) o[i] = a[i] * s; }
void orc_vec_scale_mul(const float* a, float s, const float* b, size_t n, float* o) {
    for (size_t i = 0; i < n; i++) { float t = a[i] * s; o[i] = t * b[i]; }
}
void orc_rms_norm(const float* x, const float* w, float eps, size_t hidden, size_t rows, float* o) { rms_norm(x, w, eps, hidden, rows, o); }
void orc_silu(const float* x, size_t n, float* o) { for (size_t i = 0; i < n; i++) o[i] = silu1(x[i]); }
void orc_softmax(const float* x, size_t hidden, size_t rows, float* o) { softmax_rows(x, hidden, rows, o); }
float orc_sum_sq(const float* x, size_t n) { return sum_sq(x, n); }
void orc_rope(float* x, size_t seq, size_t heads, size_t hd, float theta, size_t pos0) { apply_rotary_emb(x, seq, heads, hd, theta, pos0); }
size_t orc_argmax(const float* v, size_t n) { return argmax_last(v, n); }

// sampler::sample_top_p (rust/src/inference/sampler.rs:6-50) with the uniform draw passed in (the reference takes it from
// thread_rng, :38-39).  NaN probabilities (which its comparator calls equal to everything) are not expected.
size_t orc_sample_top_p(const float* logits, size_t n, float temperature, float top_p, float u) {
    if (temperature <= 0.0f) return argmax_last(logits, n);                                   // :7-10
    std::vector<std::pair<size_t, float>> probs(n);
    for (size_t i = 0; i < n; i++) probs[i] = {i, logits[i] / temperature};                   // :13
    float max_logit = -INFINITY;
    for (size_t i = 0; i < n; i++) max_logit = fmaxf(max_logit, probs[i].second);             // :16
    float exp_sum = 0.0f;
    for (size_t i = 0; i < n; i++) exp_sum += expf(probs[i].second - max_logit);              // :17
    for (size_t i = 0; i < n; i++) probs[i].second = expf(probs[i].second - max_logit) / exp_sum;  // :18-20
    std::stable_sort(probs.begin(), probs.end(),
                     [](const std::pair<size_t, float>& a, const std::pair<size_t, float>& b) { return a.second > b.second; });  // :23-25
    float cumsum = 0.0f;
    size_t cutoff = n - 1;
    for (size_t i = 0; i < n; i++) {                                                          // :28-32
        cumsum += probs[i].second;
        if (cumsum > top_p) { cutoff = i; break; }
    }
    float sum = 0.0f;
    for (size_t i = 0; i <= cutoff; i++) sum += probs[i].second;                              // :37
    const float rand_val = u * sum;                                                           // :39
    float cum = 0.0f;
    for (size_t i = 0; i <= cutoff; i++) {                                                    // :41-47
        cum += probs[i].second;
        if (rand_val <= cum) return probs[i].first;
    }
    return probs[cutoff].first;                                                               // :49
}

// Quantised matmul, y[m,n] = a[m,k] . deq(W)^T with W raw GGUF blocks [n rows][k/blk]:
// loader.rs:205-235 dequant + tensor.rs:107-135 matmul.
int orc_qmatmul(uint32_t typ, const float* a, const uint8_t* w, size_t m, size_t k, size_t n, float* c) {
    std::vector<float> deq(n * k);
    if (dequantize_any(typ, w, deq.data(), n * k) != 0) return -1;
    matmul_nk(a, deq.data(), c, m, k, n);
    return 0;
}

// Shard-order quantised GEMM: rust/src/kernels/int8_gemm.rs:49-98 (Q8_0) and
// :240-280 (Q4_0), AVX2 path; blocks are [k rows][n/32] with an f32 scale and,
// for Q4_0, byte i -> elements 2i, 2i+1 (q4_0.rs:36-46).  scales[k*n/32],
// qs: Q8_0 int8[k*n], Q4_0 uint8[k*n/2].
int orc_q8_0_matmul_shard(const float* a, const float* scales, const int8_t* qs, size_t m, size_t k, size_t n, float* c) {
    if (n % 32) return -1;
    size_t bpr = n / 32;
    for (size_t i = 0; i < m; i++) {
        for (size_t j = 0; j < n; j++) c[i * n + j] = 0.0f;
        for (size_t l = 0; l < k; l++) {
            float av = a[i * k + l];
            for (size_t b = 0; b < bpr; b++) {
                float s = scales[l * bpr + b];
                for (int jj = 0; jj < 32; jj++) {
                    float deq = (float)qs[(l * bpr + b) * 32 + jj] * s;
                    c[i * n + b * 32 + jj] = __builtin_fmaf(av, deq, c[i * n + b * 32 + jj]);
                }
            }
        }
    }
    return 0;
}
int orc_q4_0_matmul_shard(const float* a, const float* scales, const uint8_t* qs, size_t m, size_t k, size_t n, float* c) {
    if (n % 32) return -1;
    size_t bpr = n / 32;
    for (size_t i = 0; i < m; i++) {
        for (size_t j = 0; j < n; j++) c[i * n + j] = 0.0f;
        for (size_t l = 0; l < k; l++) {
            float av = a[i * k + l];
            for (size_t b = 0; b < bpr; b++) {
                float s = scales[l * bpr + b];
                for (int jj = 0; jj < 16; jj++) {
                    uint8_t byte = qs[(l * bpr + b) * 16 + jj];
                    float d0 = ((float)(byte & 0x0F) - 8.0f) * s;
                    float d1 = ((float)((byte >> 4) & 0x0F) - 8.0f) * s;
                    size_t o = i * n + b * 32 + jj * 2;
                    c[o] = __builtin_fmaf(av, d0, c[o]);
                    c[o + 1] = __builtin_fmaf(av, d1, c[o + 1]);
                }
            }
        }
    }
    return 0;
}
// q8_0.rs:90-122 / q4_0.rs:98-137 quantisers (shard order); out = raw bytes [f16 scale][qs]
void orc_quantize_q8_0_ref(const float* data, size_t n, uint8_t* out) {
    for (size_t b = 0; b < n / 32; b++) {
        const float* s = data + b * 32;
        float max_abs = 0.0f;
        for (int i = 0; i < 32; i++) max_abs = fmaxf(max_abs, fabsf(s[i]));
        float scale = max_abs > 0.0f ? max_abs / 127.0f : 0.0f;
        uint16_t h = f32_to_f16(scale);
        out[b * 34] = (uint8_t)(h & 0xFF); out[b * 34 + 1] = (uint8_t)(h >> 8);
        for (int i = 0; i < 32; i++) {
            int8_t q = 0;
            if (scale > 0.0f) q = (int8_t)fminf(fmaxf(roundf(s[i] / scale), -127.0f), 127.0f);
            out[b * 34 + 2 + i] = (uint8_t)q;
        }
    }
}
void orc_quantize_q4_0_ref(const float* data, size_t n, uint8_t* out) {
    for (size_t b = 0; b < n / 32; b++) {
        const float* s = data + b * 32;
        float max_abs = 0.0f;
        for (int i = 0; i < 32; i++) max_abs = fmaxf(max_abs, fabsf(s[i]));
        float scale = max_abs > 0.0f ? max_abs / 8.0f : 0.0f;
        uint16_t h = f32_to_f16(scale);
        out[b * 18] = (uint8_t)(h & 0xFF); out[b * 18 + 1] = (uint8_t)(h >> 8);
        for (int i = 0; i < 16; i++) {
            uint8_t q0 = 8, q1 = 8;
            if (scale > 0.0f) {
                q0 = (uint8_t)fminf(fmaxf(roundf(s[i * 2] / scale + 8.0f), 0.0f), 15.0f);
                q1 = (uint8_t)fminf(fmaxf(roundf(s[i * 2 + 1] / scale + 8.0f), 0.0f), 15.0f);
            }
            out[b * 18 + 2 + i] = (uint8_t)((q1 << 4) | q0);
        }
    }
}

// ---- model ----
struct orc_config {
    int32_t hidden_size, num_layers, num_heads, num_kv_heads, intermediate_size, max_seq_len, vocab_size;
    float rope_theta, rms_eps;
    int32_t kv_f32, rope_absolute, n_experts, top_k;
};

void* orc_model_create(const orc_config* c) {
    Model* m = new Model();
    m->cfg = Config{c->hidden_size, c->num_layers, c->num_heads, c->num_kv_heads, c->intermediate_size,
                    c->max_seq_len, c->vocab_size, c->rope_theta, c->rms_eps, c->kv_f32, c->rope_absolute,
                    c->n_experts, c->top_k};
    m->k16.resize(c->num_layers); m->v16.resize(c->num_layers);
    m->k32.resize(c->num_layers); m->v32.resize(c->num_layers);
    return m;
}
void orc_model_destroy(void* h) { delete (Model*)h; }
// mode 0: dequantised weights cached; mode 1: per-call dequant + transpose (engine.rs:95-97)
void orc_model_set_mode(void* h, int mode, int cache_weights) {
    Model* m = (Model*)h;
    m->mode = mode;
    m->cache_weights = cache_weights != 0;
}
int orc_model_set_tensor(void* h, const char* gguf_name, uint32_t typ, const uint64_t* dims, int ndims,
                         const void* bytes, size_t nbytes) {
    Model* m = (Model*)h;
    size_t be, bb;
    if (!quant_geometry(typ, &be, &bb)) { m->err = "unsupported type"; return -1; }
    size_t count = 1;
    for (int i = 0; i < ndims; i++) count *= dims[i];
    if ((count + be - 1) / be * bb != nbytes) { m->err = "size mismatch for " + std::string(gguf_name); return -2; }
    RawTensor t;
    t.typ = typ;
    t.dims.assign(dims, dims + ndims);
    t.bytes.assign((const uint8_t*)bytes, (const uint8_t*)bytes + nbytes);
    if (ndims == 2) { t.rows = dims[1]; t.cols = dims[0]; } else { t.rows = 1; t.cols = count; }
    m->tensors[gguf_name] = std::move(t);
    return 0;
}
void orc_kv_clear(void* h) {
    Model* m = (Model*)h;
    for (auto& v : m->k16) v.clear();
    for (auto& v : m->v16) v.clear();
    for (auto& v : m->k32) v.clear();
    for (auto& v : m->v32) v.clear();
}
size_t orc_kv_memory_bytes(void* h) {  // cache/mod.rs:80-84
    Model* m = (Model*)h;
    size_t b = 0;
    for (auto& v : m->k16) b += v.size() * 2;
    for (auto& v : m->v16) b += v.size() * 2;
    for (auto& v : m->k32) b += v.size() * 4;
    for (auto& v : m->v32) b += v.size() * 4;
    return b;
}
int orc_forward(void* h, const int64_t* tokens, size_t n, float* logits) { return forward((Model*)h, tokens, n, logits, nullptr); }
int orc_forward_hidden(void* h, const int64_t* tokens, size_t n, float* logits, float* hidden) {
    return forward((Model*)h, tokens, n, logits, hidden);
}
// engine.rs:51-76.  stop_on_eos=1 reproduces the break on token id 2; the
// metric harness passes 0 so that a fixed number of steps runs.
int orc_generate(void* h, const int64_t* tokens, size_t n, size_t max_tokens, int stop_on_eos, int64_t* out,
                 size_t* n_out, float* margins) {
    Model* m = (Model*)h;
    orc_kv_clear(h);
    std::vector<float> logits(m->cfg.vocab_size);
    if (forward(m, tokens, n, logits.data(), nullptr)) return -1;
    size_t cnt = 0;
    auto record = [&](void) {
        size_t nx = argmax_last(logits.data(), logits.size());
        if (margins) {  // top-1 minus top-2, to read beside any mismatch
            float second = -INFINITY;
            for (size_t i = 0; i < logits.size(); i++) if (i != nx) second = fmaxf(second, logits[i]);
            margins[cnt] = logits[nx] - second;
        }
        out[cnt++] = (int64_t)nx;
        return nx;
    };
    size_t next = record();
    if (!(stop_on_eos && next == 2)) {
        for (size_t s = 0; s + 1 < max_tokens; s++) {
            int64_t t = (int64_t)next;
            if (forward(m, &t, 1, logits.data(), nullptr)) return -1;
            next = record();
            if (stop_on_eos && next == 2) break;
        }
    }
    *n_out = cnt;
    return 0;
}
const char* orc_last_error(void* h) { return ((Model*)h)->err.c_str(); }
size_t orc_sanitized_count(void* h) { return ((Model*)h)->sanitized; }
void orc_timers(void* h, double* out3, int reset) {
    Model* m = (Model*)h;
    out3[0] = m->t_dequant; out3[1] = m->t_matmul; out3[2] = m->t_attn;
    if (reset) m->t_dequant = m->t_matmul = m->t_attn = 0;
}
// Per-op entry points used by the layer-level parity tests.
int orc_attention(void* h, int layer, const float* normed, size_t seq, float* out) {
    attention_forward((Model*)h, (size_t)layer, normed, seq, out);
    return 0;
}
// The benchmark's synthetic inputs (the project's counter-based generator and GGUF-order quantisers, a header shared
// with the CUDA library so that both sides can make identical bytes) for callers that must not load the CUDA library:
// the timed CPU arm of the benchmark.  Inputs only; no arithmetic of the path.
int orc_synth_tensor(uint32_t typ, uint64_t seed, const char* name, float sigma, size_t n_elems, void* out_bytes) {
    uint32_t be = 0, bb = 0;
    switch (typ) {
        case 0: be = 1; bb = 4; break;
        case 1: be = 1; bb = 2; break;
        case 2: be = 32; bb = 18; break;
        case 8: be = 32; bb = 34; break;
        case 12: be = 256; bb = 144; break;
        case 13: be = 256; bb = 176; break;
        case 14: be = 256; bb = 210; break;
        default: return -1;
    }
    if (!name || !out_bytes || n_elems % be) return -1;
    const size_t nb = n_elems / be;
    const uint64_t h = lcs_fnv1a(name);
    uint8_t* out = (uint8_t*)out_bytes;
#pragma omp parallel for schedule(static)
    for (long long b = 0; b < (long long)nb; b++) lcs_synth_block(typ, seed, h, sigma, (uint64_t)b, out + (size_t)b * bb);
    return 0;
}
void orc_synth_tokens(uint64_t seed, size_t n, int64_t vocab, int64_t* out) {
    for (size_t i = 0; i < n; i++) out[i] = (int64_t)lcs_uniform_int(seed, i, (uint64_t)vocab);
}

int orc_ffn(void* h, int layer, const float* x, size_t seq, float* out) {
    Model* m = (Model*)h;
    std::string p = "blk." + std::to_string(layer) + ".";
    if (m->cfg.n_experts > 0) moe_forward(m, p, x, seq, out); else ffn_forward(m, p, x, seq, out);
    return 0;
}

}  // extern "C"

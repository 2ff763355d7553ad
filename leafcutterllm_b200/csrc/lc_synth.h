// Deterministic synthetic weights: a counter-based N(0, sigma) generator and
// GGUF-order Q4_0 / Q8_0 / Q4_K / Q5_K / Q6_K quantisers, written so that the host build and
// the device build of this one file produce IDENTICAL bytes.
//
// How bit-equality across CPU and GPU is kept: only IEEE-exact operations are
// used (+, -, *, /, sqrt, integer ops), through the LCS_* wrappers below, which
// map to the round-to-nearest intrinsics on the device (never contracted into
// FMA) and to plain operators on the host (this file is compiled for the host
// without FMA contraction).  log and sin/cos are evaluated by fixed polynomial
// recipes in double precision instead of libm, for the same reason.
//
// The reference has no GGUF-order quantiser; the Q4_0/Q8_0 rules follow the
// absmax recipes of rust/src/kernels/q4_0.rs:98-137 and q8_0.rs:90-122 with
// the element order of the GGUF dequantisers (rust/src/kernels/mod.rs:16-51).
// The Q4_K rule (per-32 min/max -> 6-bit scale/min against per-256 d, dmin) is
// this project's own and is inverted exactly by rust/src/kernels/mod.rs:54-98;
// Q5_K is the same rule with 32 levels (mod.rs:101-143), Q6_K a per-16 absmax
// against an int8 scale and a per-256 d (mod.rs:145-180).
#pragma once
#include <stdint.h>

#if defined(__CUDA_ARCH__)
#define LCS_HD __host__ __device__ __forceinline__
#define LCS_DMUL(a, b) __dmul_rn((a), (b))
#define LCS_DADD(a, b) __dadd_rn((a), (b))
#define LCS_DSUB(a, b) __dsub_rn((a), (b))
#define LCS_DDIV(a, b) __ddiv_rn((a), (b))
#define LCS_DSQRT(a) __dsqrt_rn((a))
#define LCS_FMUL(a, b) __fmul_rn((a), (b))
#define LCS_FADD(a, b) __fadd_rn((a), (b))
#define LCS_FSUB(a, b) __fsub_rn((a), (b))
#define LCS_FDIV(a, b) __fdiv_rn((a), (b))
#else
#if defined(__CUDACC__)
#define LCS_HD __host__ __device__ inline
#else
#define LCS_HD inline
#endif
#include <math.h>
#define LCS_DMUL(a, b) ((a) * (b))
#define LCS_DADD(a, b) ((a) + (b))
#define LCS_DSUB(a, b) ((a) - (b))
#define LCS_DDIV(a, b) ((a) / (b))
#define LCS_DSQRT(a) sqrt((a))
#define LCS_FMUL(a, b) ((a) * (b))
#define LCS_FADD(a, b) ((a) + (b))
#define LCS_FSUB(a, b) ((a) - (b))
#define LCS_FDIV(a, b) ((a) / (b))
#endif

LCS_HD uint64_t lcs_splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// FNV-1a over the tensor name (host only; the hash travels as a number).
inline uint64_t lcs_fnv1a(const char* s) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (; *s; ++s) { h ^= (uint8_t)*s; h *= 0x100000001B3ull; }
    return h;
}

// ln(u) for u in (0,1): u = m * 2^e with m in [sqrt(1/2), sqrt(2)),
// ln m = 2 atanh(s), s = (m-1)/(m+1), odd series to s^15.
LCS_HD double lcs_log(double u) {
    union { double d; uint64_t b; } v;
    v.d = u;
    int e = (int)((v.b >> 52) & 0x7FF) - 1023;
    v.b = (v.b & 0x000FFFFFFFFFFFFFull) | 0x3FF0000000000000ull;  // m in [1,2)
    double m = v.d;
    if (m > 1.4142135623730951) { m = LCS_DMUL(m, 0.5); e += 1; }
    double s = LCS_DDIV(LCS_DSUB(m, 1.0), LCS_DADD(m, 1.0));
    double s2 = LCS_DMUL(s, s);
    double p = 1.0 / 15.0;
    p = LCS_DADD(LCS_DMUL(p, s2), 1.0 / 13.0);
    p = LCS_DADD(LCS_DMUL(p, s2), 1.0 / 11.0);
    p = LCS_DADD(LCS_DMUL(p, s2), 1.0 / 9.0);
    p = LCS_DADD(LCS_DMUL(p, s2), 1.0 / 7.0);
    p = LCS_DADD(LCS_DMUL(p, s2), 1.0 / 5.0);
    p = LCS_DADD(LCS_DMUL(p, s2), 1.0 / 3.0);
    p = LCS_DADD(LCS_DMUL(p, s2), 1.0);
    double lnm = LCS_DMUL(LCS_DMUL(2.0, s), p);
    return LCS_DADD(lnm, LCS_DMUL((double)e, 0.6931471805599453));
}

// cos and sin of 2*pi*u, u in [0,1): octant split, Taylor series on [0, pi/4).
LCS_HD void lcs_sincos2pi(double u, double* c, double* s) {
    double t = LCS_DMUL(u, 8.0);
    int k = (int)t;
    if (k > 7) k = 7;
    double f = LCS_DSUB(t, (double)k);
    double a = LCS_DMUL(f, 0.7853981633974483);
    double a2 = LCS_DMUL(a, a);
    double sp = -1.0 / 1307674368000.0;                            // a^15
    sp = LCS_DADD(LCS_DMUL(sp, a2), 1.0 / 6227020800.0);            // a^13
    sp = LCS_DADD(LCS_DMUL(sp, a2), -1.0 / 39916800.0);             // a^11
    sp = LCS_DADD(LCS_DMUL(sp, a2), 1.0 / 362880.0);
    sp = LCS_DADD(LCS_DMUL(sp, a2), -1.0 / 5040.0);
    sp = LCS_DADD(LCS_DMUL(sp, a2), 1.0 / 120.0);
    sp = LCS_DADD(LCS_DMUL(sp, a2), -1.0 / 6.0);
    sp = LCS_DADD(LCS_DMUL(sp, a2), 1.0);
    double sa = LCS_DMUL(a, sp);
    double cp = 1.0 / 87178291200.0;                                // a^14
    cp = LCS_DADD(LCS_DMUL(cp, a2), -1.0 / 479001600.0);            // a^12
    cp = LCS_DADD(LCS_DMUL(cp, a2), 1.0 / 3628800.0);
    cp = LCS_DADD(LCS_DMUL(cp, a2), -1.0 / 40320.0);
    cp = LCS_DADD(LCS_DMUL(cp, a2), 1.0 / 720.0);
    cp = LCS_DADD(LCS_DMUL(cp, a2), -1.0 / 24.0);
    cp = LCS_DADD(LCS_DMUL(cp, a2), 0.5);
    double ca = LCS_DSUB(1.0, LCS_DMUL(a2, cp));
    const double R = 0.7071067811865476;
    double ck, sk;
    switch (k) {
        case 0: ck = 1.0; sk = 0.0; break;
        case 1: ck = R; sk = R; break;
        case 2: ck = 0.0; sk = 1.0; break;
        case 3: ck = -R; sk = R; break;
        case 4: ck = -1.0; sk = 0.0; break;
        case 5: ck = -R; sk = -R; break;
        case 6: ck = 0.0; sk = -1.0; break;
        default: ck = R; sk = -R; break;
    }
    *c = LCS_DSUB(LCS_DMUL(ck, ca), LCS_DMUL(sk, sa));
    *s = LCS_DADD(LCS_DMUL(sk, ca), LCS_DMUL(ck, sa));
}

// Element `idx` of the tensor keyed by (seed, name_hash): Box-Muller over two
// 53-bit uniforms drawn from the pair counter idx/2; even idx takes the cosine
// branch, odd idx the sine branch.
LCS_HD float lcs_normal(uint64_t seed, uint64_t name_hash, uint64_t idx, float sigma) {
    uint64_t key = lcs_splitmix64(seed ^ lcs_splitmix64(name_hash));
    uint64_t pair = idx >> 1;
    uint64_t h1 = lcs_splitmix64(key ^ lcs_splitmix64(2 * pair));
    uint64_t h2 = lcs_splitmix64(key ^ lcs_splitmix64(2 * pair + 1));
    double u1 = LCS_DMUL(LCS_DADD((double)(h1 >> 11), 0.5), 1.0 / 9007199254740992.0);
    double u2 = LCS_DMUL((double)(h2 >> 11), 1.0 / 9007199254740992.0);
    double r = LCS_DSQRT(LCS_DMUL(-2.0, lcs_log(u1)));
    double c, s;
    lcs_sincos2pi(u2, &c, &s);
    double z = LCS_DMUL(r, (idx & 1) ? s : c);
    return (float)LCS_DMUL(z, (double)sigma);
}

// Uniform integer in [0, n) for prompts / context lengths.
LCS_HD uint64_t lcs_uniform_int(uint64_t seed, uint64_t idx, uint64_t n) {
    return lcs_splitmix64(lcs_splitmix64(seed) ^ lcs_splitmix64(idx)) % n;
}

// f32 -> f16 bits, round to nearest even (integer-only, same on both sides).
LCS_HD uint16_t lcs_f32_to_f16(float f) {
    union { float f; uint32_t u; } v;
    v.f = f;
    uint32_t x = v.u;
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t man = x & 0x007FFFFFu;
    int32_t exp = (int32_t)((x >> 23) & 0xFFu);
    if (exp == 255) return (uint16_t)(sign | 0x7C00u | (man ? (0x0200u | (man >> 13)) : 0u));
    int32_t e = exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x00800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t hm = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (hm & 1u))) hm++;
        return (uint16_t)(sign | hm);
    }
    uint32_t hm = man >> 13;
    uint32_t rem = man & 0x1FFFu;
    uint32_t out = sign | ((uint32_t)e << 10) | hm;
    if (rem > 0x1000u || (rem == 0x1000u && (hm & 1u))) out++;
    return (uint16_t)out;
}

LCS_HD float lcs_f16_to_f32(uint16_t h) {
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
    union { float f; uint32_t u; } v;
    v.u = bits;
    return v.f;
}

// Round half away from zero on a non-negative or signed small value (exact ops only).
LCS_HD float lcs_round(float v) {
    float a = v < 0.0f ? -v : v;
    float fl = (float)(int32_t)a;  // |v| is far below 2^31 wherever this is used
    float r = (LCS_FSUB(a, fl) >= 0.5f) ? LCS_FADD(fl, 1.0f) : fl;
    return v < 0.0f ? -r : r;
}
LCS_HD float lcs_clamp(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

// Q8_0, 34 bytes per 32 elements: f16 scale, 32 int8.
LCS_HD void lcs_quantize_q8_0_block(const float* x, uint8_t* out) {
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) { float a = x[i] < 0.0f ? -x[i] : x[i]; if (a > amax) amax = a; }
    float scale = amax > 0.0f ? LCS_FDIV(amax, 127.0f) : 0.0f;
    uint16_t h = lcs_f32_to_f16(scale);
    out[0] = (uint8_t)(h & 0xFF); out[1] = (uint8_t)(h >> 8);
    for (int i = 0; i < 32; i++) {
        int q = 0;
        if (scale > 0.0f) q = (int)lcs_clamp(lcs_round(LCS_FDIV(x[i], scale)), -127.0f, 127.0f);
        out[2 + i] = (uint8_t)(int8_t)q;
    }
}

// Q4_0, 18 bytes per 32 elements: f16 scale, byte j = element j (low nibble) | element j+16 (high nibble).
LCS_HD void lcs_quantize_q4_0_block(const float* x, uint8_t* out) {
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) { float a = x[i] < 0.0f ? -x[i] : x[i]; if (a > amax) amax = a; }
    float scale = amax > 0.0f ? LCS_FDIV(amax, 8.0f) : 0.0f;
    uint16_t h = lcs_f32_to_f16(scale);
    out[0] = (uint8_t)(h & 0xFF); out[1] = (uint8_t)(h >> 8);
    for (int j = 0; j < 16; j++) {
        int q0 = 8, q1 = 8;
        if (scale > 0.0f) {
            q0 = (int)lcs_clamp(lcs_round(LCS_FADD(LCS_FDIV(x[j], scale), 8.0f)), 0.0f, 15.0f);
            q1 = (int)lcs_clamp(lcs_round(LCS_FADD(LCS_FDIV(x[j + 16], scale), 8.0f)), 0.0f, 15.0f);
        }
        out[2 + j] = (uint8_t)((q1 << 4) | q0);
    }
}

// Q4_K, 144 bytes per 256 elements: f16 d, f16 dmin, 12 bytes of 6-bit (scale,min) x 8, 128 nibble bytes.
LCS_HD void lcs_quantize_q4_k_block(const float* x, uint8_t* out) {
    float scale[8], mn[8];
    float max_scale = 0.0f, max_min = 0.0f;
    for (int j = 0; j < 8; j++) {
        float lo = 0.0f, hi = 0.0f;  // the offset term can only subtract: clamp the minimum at zero
        for (int i = 0; i < 32; i++) { float v = x[j * 32 + i]; if (v < lo) lo = v; if (v > hi) hi = v; }
        scale[j] = LCS_FDIV(LCS_FSUB(hi, lo), 15.0f);
        mn[j] = -lo;
        if (scale[j] > max_scale) max_scale = scale[j];
        if (mn[j] > max_min) max_min = mn[j];
    }
    uint16_t hd = lcs_f32_to_f16(LCS_FDIV(max_scale, 63.0f));
    uint16_t hm = lcs_f32_to_f16(LCS_FDIV(max_min, 63.0f));
    float d = lcs_f16_to_f32(hd), dmin = lcs_f16_to_f32(hm);
    out[0] = (uint8_t)(hd & 0xFF); out[1] = (uint8_t)(hd >> 8);
    out[2] = (uint8_t)(hm & 0xFF); out[3] = (uint8_t)(hm >> 8);
    uint8_t sc[8], mm[8];
    for (int j = 0; j < 8; j++) {
        sc[j] = d > 0.0f ? (uint8_t)lcs_clamp(lcs_round(LCS_FDIV(scale[j], d)), 0.0f, 63.0f) : 0;
        mm[j] = dmin > 0.0f ? (uint8_t)lcs_clamp(lcs_round(LCS_FDIV(mn[j], dmin)), 0.0f, 63.0f) : 0;
    }
    uint8_t* s = out + 4;
    for (int j = 0; j < 4; j++) {
        s[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
        s[j + 4] = (uint8_t)((mm[j] & 63) | ((mm[j + 4] >> 4) << 6));
        s[j + 8] = (uint8_t)((sc[j + 4] & 0x0F) | ((mm[j + 4] & 0x0F) << 4));
    }
    uint8_t* qs = out + 16;
    for (int g = 0; g < 4; g++) {
        float dl1 = LCS_FMUL(d, (float)sc[2 * g]), ml1 = LCS_FMUL(dmin, (float)mm[2 * g]);
        float dl2 = LCS_FMUL(d, (float)sc[2 * g + 1]), ml2 = LCS_FMUL(dmin, (float)mm[2 * g + 1]);
        for (int l = 0; l < 32; l++) {
            int q1 = 0, q2 = 0;
            if (dl1 > 0.0f) q1 = (int)lcs_clamp(lcs_round(LCS_FDIV(LCS_FADD(x[64 * g + l], ml1), dl1)), 0.0f, 15.0f);
            if (dl2 > 0.0f) q2 = (int)lcs_clamp(lcs_round(LCS_FDIV(LCS_FADD(x[64 * g + 32 + l], ml2), dl2)), 0.0f, 15.0f);
            qs[32 * g + l] = (uint8_t)(q1 | (q2 << 4));
        }
    }
}

// Q5_K, 176 bytes per 256 elements: the Q4_K header, 32 bytes of fifth bits (bit s of byte l = element l of sub-block s),
// 128 nibble bytes.
LCS_HD void lcs_quantize_q5_k_block(const float* x, uint8_t* out) {
    float scale[8], mn[8];
    float max_scale = 0.0f, max_min = 0.0f;
    for (int j = 0; j < 8; j++) {
        float lo = 0.0f, hi = 0.0f;
        for (int i = 0; i < 32; i++) { float v = x[j * 32 + i]; if (v < lo) lo = v; if (v > hi) hi = v; }
        scale[j] = LCS_FDIV(LCS_FSUB(hi, lo), 31.0f);
        mn[j] = -lo;
        if (scale[j] > max_scale) max_scale = scale[j];
        if (mn[j] > max_min) max_min = mn[j];
    }
    uint16_t hd = lcs_f32_to_f16(LCS_FDIV(max_scale, 63.0f));
    uint16_t hm = lcs_f32_to_f16(LCS_FDIV(max_min, 63.0f));
    float d = lcs_f16_to_f32(hd), dmin = lcs_f16_to_f32(hm);
    out[0] = (uint8_t)(hd & 0xFF); out[1] = (uint8_t)(hd >> 8);
    out[2] = (uint8_t)(hm & 0xFF); out[3] = (uint8_t)(hm >> 8);
    uint8_t sc[8], mm[8];
    for (int j = 0; j < 8; j++) {
        sc[j] = d > 0.0f ? (uint8_t)lcs_clamp(lcs_round(LCS_FDIV(scale[j], d)), 0.0f, 63.0f) : 0;
        mm[j] = dmin > 0.0f ? (uint8_t)lcs_clamp(lcs_round(LCS_FDIV(mn[j], dmin)), 0.0f, 63.0f) : 0;
    }
    uint8_t* s = out + 4;
    for (int j = 0; j < 4; j++) {
        s[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
        s[j + 4] = (uint8_t)((mm[j] & 63) | ((mm[j + 4] >> 4) << 6));
        s[j + 8] = (uint8_t)((sc[j + 4] & 0x0F) | ((mm[j + 4] & 0x0F) << 4));
    }
    uint8_t* qh = out + 16;
    uint8_t* qs = out + 48;
    for (int l = 0; l < 32; l++) qh[l] = 0;
    for (int g = 0; g < 4; g++) {
        float dl1 = LCS_FMUL(d, (float)sc[2 * g]), ml1 = LCS_FMUL(dmin, (float)mm[2 * g]);
        float dl2 = LCS_FMUL(d, (float)sc[2 * g + 1]), ml2 = LCS_FMUL(dmin, (float)mm[2 * g + 1]);
        for (int l = 0; l < 32; l++) {
            int q1 = 0, q2 = 0;
            if (dl1 > 0.0f) q1 = (int)lcs_clamp(lcs_round(LCS_FDIV(LCS_FADD(x[64 * g + l], ml1), dl1)), 0.0f, 31.0f);
            if (dl2 > 0.0f) q2 = (int)lcs_clamp(lcs_round(LCS_FDIV(LCS_FADD(x[64 * g + 32 + l], ml2), dl2)), 0.0f, 31.0f);
            qs[32 * g + l] = (uint8_t)((q1 & 15) | ((q2 & 15) << 4));
            qh[l] = (uint8_t)(qh[l] | ((q1 >> 4) << (2 * g)) | ((q2 >> 4) << (2 * g + 1)));
        }
    }
}

// Q6_K, 210 bytes per 256 elements: 128 bytes of low nibbles, 64 bytes of high bit pairs, 16 int8 scales (one per 16
// elements), f16 d.  Element 128 n + 32 j + l: nibble j / 2 of ql[64 n + 32 (j & 1) + l], bits 2 j of qh[32 n + l].
LCS_HD void lcs_quantize_q6_k_block(const float* x, uint8_t* out) {
    float scale[16];
    float max_scale = 0.0f;
    for (int j = 0; j < 16; j++) {
        float amax = 0.0f;
        for (int i = 0; i < 16; i++) { float a = x[j * 16 + i] < 0.0f ? -x[j * 16 + i] : x[j * 16 + i]; if (a > amax) amax = a; }
        scale[j] = LCS_FDIV(amax, 31.0f);
        if (scale[j] > max_scale) max_scale = scale[j];
    }
    uint16_t hd = lcs_f32_to_f16(LCS_FDIV(max_scale, 127.0f));
    float d = lcs_f16_to_f32(hd);
    out[208] = (uint8_t)(hd & 0xFF); out[209] = (uint8_t)(hd >> 8);
    int sc[16];
    for (int j = 0; j < 16; j++) {
        sc[j] = d > 0.0f ? (int)lcs_clamp(lcs_round(LCS_FDIV(scale[j], d)), 0.0f, 127.0f) : 0;
        out[192 + j] = (uint8_t)(int8_t)sc[j];
    }
    for (int i = 0; i < 192; i++) out[i] = 0;
    for (int n = 0; n < 2; n++)
        for (int j = 0; j < 4; j++)
            for (int l = 0; l < 32; l++) {
                int e = 128 * n + 32 * j + l;
                float dl = LCS_FMUL(d, (float)sc[e / 16]);
                int q = 32;
                if (dl > 0.0f) q = (int)lcs_clamp(LCS_FADD(lcs_round(LCS_FDIV(x[e], dl)), 32.0f), 0.0f, 63.0f);
                uint8_t* ql = out + 64 * n + 32 * (j & 1) + l;
                uint8_t* qh = out + 128 + 32 * n + l;
                *ql = (uint8_t)(*ql | ((q & 15) << (4 * (j >> 1))));
                *qh = (uint8_t)(*qh | ((q >> 4) << (2 * j)));
            }
}

// ggml type codes used here (rust/src/model/quant.rs:45-76).
#define LCS_TYPE_F32 0
#define LCS_TYPE_F16 1
#define LCS_TYPE_Q4_0 2
#define LCS_TYPE_Q8_0 8
#define LCS_TYPE_Q4_K 12
#define LCS_TYPE_Q5_K 13
#define LCS_TYPE_Q6_K 14

// Writes the quantised bytes of block `blk` (block index over the flattened
// row-major tensor) of the synthetic tensor into `out`.
LCS_HD void lcs_synth_block(uint32_t typ, uint64_t seed, uint64_t name_hash, float sigma, uint64_t blk, uint8_t* out) {
    if (typ == LCS_TYPE_Q4_K) {
        float x[256];
        for (int i = 0; i < 256; i++) x[i] = lcs_normal(seed, name_hash, blk * 256 + i, sigma);
        lcs_quantize_q4_k_block(x, out);
    } else if (typ == LCS_TYPE_Q5_K || typ == LCS_TYPE_Q6_K) {
        float x[256];
        for (int i = 0; i < 256; i++) x[i] = lcs_normal(seed, name_hash, blk * 256 + i, sigma);
        if (typ == LCS_TYPE_Q5_K) lcs_quantize_q5_k_block(x, out);
        else lcs_quantize_q6_k_block(x, out);
    } else if (typ == LCS_TYPE_Q4_0) {
        float x[32];
        for (int i = 0; i < 32; i++) x[i] = lcs_normal(seed, name_hash, blk * 32 + i, sigma);
        lcs_quantize_q4_0_block(x, out);
    } else if (typ == LCS_TYPE_Q8_0) {
        float x[32];
        for (int i = 0; i < 32; i++) x[i] = lcs_normal(seed, name_hash, blk * 32 + i, sigma);
        lcs_quantize_q8_0_block(x, out);
    } else if (typ == LCS_TYPE_F16) {
        uint16_t h = lcs_f32_to_f16(lcs_normal(seed, name_hash, blk, sigma));
        out[0] = (uint8_t)(h & 0xFF); out[1] = (uint8_t)(h >> 8);
    } else {  // F32
        union { float f; uint32_t u; } v;
        v.f = lcs_normal(seed, name_hash, blk, sigma);
        out[0] = (uint8_t)v.u; out[1] = (uint8_t)(v.u >> 8); out[2] = (uint8_t)(v.u >> 16); out[3] = (uint8_t)(v.u >> 24);
    }
}

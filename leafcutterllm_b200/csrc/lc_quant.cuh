// Device-side block decoders for the ggml quant types of the hot path.
// Every function reproduces the reference's f32 result bit for bit: products
// that the reference rounds once are rounded once here (explicit _rn
// intrinsics, so nothing is contracted into an FMA with different rounding).
// Citations: rust/src/kernels/mod.rs.
#pragma once
#include "lc_common.cuh"

namespace lc {

// mod.rs:54-63 (get_scale_min_k4) on the 12 scale bytes held as three words.
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, uint32_t* sc, uint32_t* m) {
    if (j < 4) {
        *sc = q[j] & 0x3F;
        *m = q[j + 4] & 0x3F;
    } else {
        *sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4);
        *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// All eight (scale, min) pairs of a Q4_K / Q5_K block from the three scale
// words: sc[i], mn[i] as bytes packed four to a word (sc_lo = pairs 0..3,
// sc_hi = pairs 4..7).  Same bit selection as mod.rs:54-63.
__device__ __forceinline__ void unpack_scales_k4(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t* sc_lo, uint32_t* sc_hi,
                                                 uint32_t* mn_lo, uint32_t* mn_hi) {
    *sc_lo = s0 & 0x3F3F3F3Fu;
    *mn_lo = s1 & 0x3F3F3F3Fu;
    *sc_hi = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
    *mn_hi = ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u);
}

// Element `e` (0..block_elems) of a block, exactly as the reference dequantises it.
__device__ __forceinline__ float dequant_elem_q4_0(const uint8_t* b, int e) {  // mod.rs:16-34
    float scale = h2f((uint16_t)(b[0] | (b[1] << 8)));
    uint8_t qs = b[2 + (e & 15)];
    int q = (e < 16) ? (qs & 0x0F) : (qs >> 4);
    return __fmul_rn((float)q - 8.0f, scale);
}
__device__ __forceinline__ float dequant_elem_q8_0(const uint8_t* b, int e) {  // mod.rs:37-51
    float scale = h2f((uint16_t)(b[0] | (b[1] << 8)));
    return __fmul_rn((float)(int8_t)b[2 + e], scale);
}
__device__ __forceinline__ float dequant_elem_q4_k(const uint8_t* b, int e) {  // mod.rs:66-98
    float d = h2f((uint16_t)(b[0] | (b[1] << 8)));
    float dmin = h2f((uint16_t)(b[2] | (b[3] << 8)));
    int g = e >> 6, r = e & 63;
    int is = 2 * g + (r >> 5);
    uint32_t sc, m;
    scale_min_k4(is, b + 4, &sc, &m);
    uint8_t byte = b[16 + 32 * g + (r & 31)];
    int q = (r < 32) ? (byte & 0x0F) : (byte >> 4);
    float dl = __fmul_rn(d, (float)sc), mn = __fmul_rn(dmin, (float)m);
    return __fsub_rn(__fmul_rn(dl, (float)q), mn);
}
__device__ __forceinline__ float dequant_elem_q5_k(const uint8_t* b, int e) {  // mod.rs:101-142
    float d = h2f((uint16_t)(b[0] | (b[1] << 8)));
    float dmin = h2f((uint16_t)(b[2] | (b[3] << 8)));
    int g = e >> 6, r = e & 63, l = r & 31;
    int is = 2 * g + (r >> 5);
    uint32_t sc, m;
    scale_min_k4(is, b + 4, &sc, &m);
    uint8_t ql = b[48 + 32 * g + l];
    uint8_t qh = b[16 + l];
    int q = (r < 32) ? (ql & 0x0F) : (ql >> 4);
    int bit = 2 * g + (r >> 5);
    if (qh & (1 << bit)) q += 16;
    float dl = __fmul_rn(d, (float)sc), mn = __fmul_rn(dmin, (float)m);
    return __fsub_rn(__fmul_rn(dl, (float)q), mn);
}
__device__ __forceinline__ float dequant_elem_q6_k(const uint8_t* b, int e) {  // mod.rs:145-180
    int n = e >> 7, r = e & 127, quad = r >> 5, l = r & 31;
    const uint8_t* ql = b + 64 * n;
    const uint8_t* qh = b + 128 + 32 * n;
    const int8_t* sc = (const int8_t*)(b + 192 + 8 * n);
    float d = h2f((uint16_t)(b[208] | (b[209] << 8)));
    int lo = (quad & 1) ? ql[l + 32] : ql[l];
    lo = (quad & 2) ? (lo >> 4) : (lo & 0x0F);
    int hi = (qh[l] >> (2 * quad)) & 3;
    int q = (int)(int8_t)(lo | (hi << 4)) - 32;
    int is = l / 16;
    float s = (float)sc[is + 2 * quad];
    return __fmul_rn(__fmul_rn(d, s), (float)q);
}
__device__ __forceinline__ float dequant_elem_iq4_nl(const uint8_t* b, int e) {  // mod.rs:186-216
    const float T[16] = {-1.0f, -0.6962f, -0.5251f, -0.3952f, -0.2893f, -0.1957f, -0.1107f, -0.0322f,
                         0.0322f, 0.1107f, 0.1957f, 0.2893f, 0.3952f, 0.5251f, 0.6962f, 1.0f};
    float scale = h2f((uint16_t)(b[0] | (b[1] << 8)));
    uint8_t qs = b[2 + (e >> 1)];
    int nib = (e & 1) ? (qs >> 4) : (qs & 0x0F);
    return __fmul_rn(scale, T[nib]);
}

// One element of a tensor of ggml type `typ` whose raw bytes start at `base`.
__device__ __forceinline__ float dequant_elem(uint32_t typ, const uint8_t* base, size_t idx) {
    switch (typ) {
        case LC_TYPE_F32: return ((const float*)base)[idx];
        case LC_TYPE_F16: return h2f(((const uint16_t*)base)[idx]);
        case LC_TYPE_Q4_0: return dequant_elem_q4_0(base + (idx >> 5) * 18, (int)(idx & 31));
        case LC_TYPE_Q8_0: return dequant_elem_q8_0(base + (idx >> 5) * 34, (int)(idx & 31));
        case LC_TYPE_Q4_K: return dequant_elem_q4_k(base + (idx >> 8) * 144, (int)(idx & 255));
        case LC_TYPE_Q5_K: return dequant_elem_q5_k(base + (idx >> 8) * 176, (int)(idx & 255));
        case LC_TYPE_Q6_K: return dequant_elem_q6_k(base + (idx >> 8) * 210, (int)(idx & 255));
        case LC_TYPE_IQ4_NL: return dequant_elem_iq4_nl(base + (idx >> 5) * 18, (int)(idx & 31));
        default: return 0.0f;
    }
}

}  // namespace lc

// The activations of the integer-tensor-core matrix-vector kernels: a 256-element unit of a token's row as 24-bit fixed
// point against the unit's own power-of-two scale, X = round(x * 2^s), |X| <= 2^22, split into three balanced byte planes
// X = P0 + 256 P1 + 65536 P2 with every digit in [-128, 127].
#pragma once
#include <cstdint>
#include "lc_common.cuh"

namespace lc {

// One warp per unit; lane l holds elements 8 l .. 8 l + 7 in v.  dst = where sub-block 0, plane 0 of this (unit, token)
// goes: plane p of 32-element sub-block sb lies at dst + sb * sb_stride + 32 p.  sx8 (or null) receives the eight
// sub-block sums of the rounded values, *inv2s the factor 2^-s.
__device__ __forceinline__ void unit_planes(const float (&v)[8], int lane, unsigned char* dst, int sb_stride, float* sx8, float* inv2s) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(v[j]));
    amax = warp_max(amax);
    // amax = f * 2^ex with f in [0.5, 1): ex from the exponent field (zero, denormal and non-finite inputs fall into the clamp)
    const int ex = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 126;
    const int s = max(-100, min(100, 22 - ex));  // |x| * 2^s < 2^22
    const float up = __uint_as_float((uint32_t)(127 + s) << 23), dn = __uint_as_float((uint32_t)(127 - s) << 23);
    // The digits are the bytes of X + 0x808080 with their top bits flipped: that sum is b0 + 256 b1 + 65536 b2 with unsigned
    // bytes, so X = (b0 - 128) + 256 (b1 - 128) + 65536 (b2 - 128), and b - 128 as a signed byte is b ^ 0x80.
    uint32_t pw[3][2];
    int xsum = 0;
    uint32_t y[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        float sv = v[j] * up;
        sv = fminf(fmaxf(sv, -4194304.f), 4194304.f);
        const int X = __float2int_rn(sv);
        xsum += X;
        y[j] = (uint32_t)(X + 0x808080) ^ 0x808080u;
    }
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int pl = 0; pl < 3; pl++)  // byte pl of four consecutive elements
            pw[pl][h] = __byte_perm(__byte_perm(y[4 * h], y[4 * h + 1], 0x0040 + 0x11 * pl), __byte_perm(y[4 * h + 2], y[4 * h + 3], 0x0040 + 0x11 * pl), 0x5410);
    const int sb = lane >> 2, inner = (8 * lane) & 31;
#pragma unroll
    for (int pl = 0; pl < 3; pl++) *reinterpret_cast<uint2*>(dst + sb * sb_stride + pl * 32 + inner) = make_uint2(pw[pl][0], pw[pl][1]);
    if (sx8) {
        xsum += __shfl_xor_sync(0xffffffffu, xsum, 1);
        xsum += __shfl_xor_sync(0xffffffffu, xsum, 2);
        if ((lane & 3) == 0) sx8[sb] = (float)xsum * dn;
    }
    if (lane == 0) *inv2s = dn;
}

}  // namespace lc

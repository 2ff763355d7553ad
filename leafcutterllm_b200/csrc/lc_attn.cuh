// Causal grouped-query attention of one (token, head, split) over the paged KV cache, as a device function
// shared by the stand-alone attention kernel and the persistent decode kernel
// (rust/src/inference/attention.rs:69-113, rust/src/cache/mod.rs:33-77).
#pragma once
#include "lc_kernels.h"

namespace lc {

constexpr int kAttnWarps = 4;

struct AttnParams {
    const float* q;        // [n_tok, q_stride]: head h at q + tok*q_stride + h*hd
    int q_stride;
    float* out;            // [n_tok, n_heads*hd]
    int n_heads;
    KvLayout kv;
    const int32_t* tok_seq;
    const int32_t* tok_pos;
    const int32_t* page_table;
    int pages_per_seq;
    int chunk, n_splits;
    float* partial;        // [n_tok*n_heads][n_splits][hd+2]
    int* counters;         // [n_tok*n_heads], zero between launches
    // Decode-step fusion: every token is the only new token of its sequence.  q is rotated on load, the
    // new key/value come from k_new/v_new (rotated, rounded to the cache type exactly as a cache round
    // trip would) and are stored into the cache by the CTA that meets them.
    const float* k_new;    // null = keys and values are already in the cache and q is already rotated
    const float* v_new;
    const int32_t* tok_rope;
    float theta;
    int positions_settled; // decode-step fusion: tok_pos may be read before the grid dependency wait
    int* error_flag;       // set when a bounded wait runs out (may be null)
};

// attention_stream.cu: one new token, head_dim 128, f16 cache of 16-token pages, as a balanced single-wave stream
bool attention_stream_applies(const AttnParams& a, int n_tok);
// slots: attention_stream_slot_bytes(n_heads, n_kv) bytes of zeroed device memory owned by the caller (left zeroed)
int32_t launch_attention_stream(const AttnParams& a, unsigned long long* slots, cudaStream_t s);

template <int DPL, bool F32>
__device__ __forceinline__ void load_slice(const void* pool, size_t elem_off, float (&out)[DPL]) {
    if (F32) {
        const float4* p = reinterpret_cast<const float4*>((const float*)pool + elem_off);
#pragma unroll
        for (int i = 0; i < DPL / 4; i++) { float4 v = p[i]; out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w; }
    } else {
        const uint4* p = reinterpret_cast<const uint4*>((const __half*)pool + elem_off);
#pragma unroll
        for (int i = 0; i < DPL / 8; i++) {
            uint4 v = p[i];
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; j++) { float2 f = __half22float2(h[j]); out[8 * i + 2 * j] = f.x; out[8 * i + 2 * j + 1] = f.y; }
        }
    }
}

// The same slice kept as it lies in the cache (16-byte pieces), so that a pass's loads can be in flight while the pass
// before it is still being computed without doubling the registers that hold them as f32.
template <int DPL, bool F32>
struct RawSlice { uint4 v[F32 ? DPL / 4 : DPL / 8]; };
template <int DPL, bool F32>
__device__ __forceinline__ void load_raw(const void* pool, size_t elem_off, RawSlice<DPL, F32>& r) {
    const uint4* p = F32 ? reinterpret_cast<const uint4*>((const float*)pool + elem_off) : reinterpret_cast<const uint4*>((const __half*)pool + elem_off);
#pragma unroll
    for (int i = 0; i < (F32 ? DPL / 4 : DPL / 8); i++) r.v[i] = p[i];
}
template <int DPL, bool F32>
__device__ __forceinline__ void widen(const RawSlice<DPL, F32>& r, float (&out)[DPL]) {
    if (F32) {
#pragma unroll
        for (int i = 0; i < DPL / 4; i++) {
            out[4 * i] = __uint_as_float(r.v[i].x); out[4 * i + 1] = __uint_as_float(r.v[i].y);
            out[4 * i + 2] = __uint_as_float(r.v[i].z); out[4 * i + 3] = __uint_as_float(r.v[i].w);
        }
    } else {
#pragma unroll
        for (int i = 0; i < DPL / 8; i++) {
            const __half2* h = reinterpret_cast<const __half2*>(&r.v[i]);
#pragma unroll
            for (int j = 0; j < 4; j++) { float2 f = __half22float2(h[j]); out[8 * i + 2 * j] = f.x; out[8 * i + 2 * j + 1] = f.y; }
        }
    }
}

// Dims d0 .. d0+DPL-1 of a head vector at `base`, rotated by position `rp` (attention.rs:13-34: pairs
// (d, d + hd/2), freq = 1 / theta^(2d/hd)).  rp == 0 is the identity and skips the trigonometry.
template <int DPL, int HD>
__device__ __forceinline__ void load_rotated(const float* base, int d0, int rp, float theta, float (&out)[DPL]) {
#pragma unroll
    for (int i = 0; i < DPL; i++) out[i] = __ldcg(base + d0 + i);  // written by another CTA of a persistent kernel: read through L2
    if (rp == 0) return;
    constexpr int HALF = HD / 2;
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = d0 + i, dd = d < HALF ? d : d - HALF;
        const float freq = __fdiv_rn(1.0f, powf(theta, __fdiv_rn(__fmul_rn(2.0f, (float)dd), (float)HD)));
        const float angle = __fmul_rn((float)rp, freq);
        const float ca = cosf(angle), sa = sinf(angle);
        if (d < HALF) out[i] = __fsub_rn(__fmul_rn(__ldcg(base + d), ca), __fmul_rn(__ldcg(base + d + HALF), sa));
        else out[i] = __fadd_rn(__fmul_rn(__ldcg(base + d - HALF), sa), __fmul_rn(__ldcg(base + d), ca));
    }
}

template <int DPL, bool F32>
__device__ __forceinline__ void store_round(void* pool, size_t elem_off, float (&v)[DPL]) {
    if (F32) {
#pragma unroll
        for (int i = 0; i < DPL; i++) ((float*)pool)[elem_off + i] = v[i];
    } else {
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            __half hv = __float2half_rn(v[i]);       // cache/mod.rs:35-36
            ((__half*)pool)[elem_off + i] = hv;
            v[i] = __half2float(hv);                 // attention reads the round-tripped value (cache/mod.rs:65-77)
        }
    }
}

// One group of kAttnWarps warps per (token, head, split).  LPK lanes share a key, each holding DPL = HD / LPK
// dims.  `item` = token*n_heads + head, `tid` = thread index inside the group, BAR = 0: the group is the whole
// CTA (__syncthreads), BAR = 1: named barrier `bar_id` for a 128-thread group inside a larger CTA.  `sh` = 8 + 4*HD
// floats of shared memory private to the group (+1 int).
template <int BAR>
__device__ __forceinline__ void group_sync(int bar_id) {
    if (BAR == 0) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(kAttnWarps * 32) : "memory");
}

template <int HD, bool F32, int BAR>
__device__ __forceinline__ void attention_item(const AttnParams& p, int item, int split, int tid, float* sh, int bar_id = 0) {
    constexpr int DPL = 16 < HD / 2 ? 16 : HD / 2;
    constexpr int LPK = HD / DPL;
    constexpr int KPW = 32 / LPK;               // keys per warp per pass
    constexpr int KPI = KPW * kAttnWarps;       // keys per group per pass
    const int n_heads = p.n_heads;
    const KvLayout& kv = p.kv;
    const int tok = item / n_heads, h = item % n_heads;
    const int pos = p.tok_pos[tok];
    const int ctx = pos + 1;  // causal: positions 0..tok_pos (attention.rs:81-83)
    // pieces of the context that hold at least one key of this token; a CTA of a piece past them has nothing to add and
    // leaves at once (the merge below counts the live pieces only)
    const int live = (p.n_splits == 1) ? 1 : min(p.n_splits, (ctx + p.chunk - 1) / p.chunk);
    if (split >= live) return;
    const int t_begin = split * p.chunk;
    const int t_end = min(ctx, t_begin + p.chunk);
    float* pout = p.partial + ((size_t)item * p.n_splits + split) * (HD + 2);
    const int warp = tid >> 5, lane = tid & 31, grp = lane / LPK, sub = lane % LPK;
    float* sm_m = sh;
    float* sm_l = sh + 4;
    float (*sm_acc)[HD] = reinterpret_cast<float (*)[HD]>(sh + 8);
    int* sm_last = reinterpret_cast<int*>(sh + 8 + kAttnWarps * HD);

    float m = -INFINITY, l = 0.f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; i++) acc[i] = 0.f;

    if (t_begin < t_end) {
        const int gsz = n_heads / kv.n_kv;
        const int kvh = h / gsz;  // attention.rs:75
        const int32_t* pt = p.page_table + (size_t)p.tok_seq[tok] * p.pages_per_seq;
        const float inv_div = sqrtf((float)HD);   // attention.rs:93: dot / sqrt(head_dim)
        const int rp = p.k_new ? p.tok_rope[tok] : 0;
        float qr[DPL];
        load_rotated<DPL, HD>(p.q + (size_t)tok * p.q_stride + h * HD, sub * DPL, rp, p.theta, qr);

        auto key_addr = [&](int t) -> size_t {
            int page = pt[t / kv.page_tokens];
            return (((size_t)page * kv.n_kv + kvh) * kv.page_tokens + t % kv.page_tokens) * HD + sub * DPL;
        };
        // Cached keys are loaded unconditionally (padding lanes re-read the first key of the slice) so that the
        // loads of both keys of a pass are in flight together; the token of this step is handled after the loop.
        typedef RawSlice<DPL, F32> Raw;
        auto fetch = [&](int t, bool valid, Raw& kr, Raw& vr) {
            const size_t a = key_addr(valid ? t : t_begin);
            load_raw<DPL, F32>(kv.k_pool, a, kr);
            load_raw<DPL, F32>(kv.v_pool, a, vr);
        };
        auto update_f = [&](bool valid, const float (&kr)[DPL], const float (&vr)[DPL]) {
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < DPL; i++) dot = fmaf(qr[i], kr[i], dot);
#pragma unroll
            for (int o = 1; o < LPK; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (valid) {
                const float s = dot / inv_div;
                if (s > m) {
                    const float alpha = expf(m - s);  // exp(-inf) = 0 on the first key
                    l *= alpha;
#pragma unroll
                    for (int i = 0; i < DPL; i++) acc[i] *= alpha;
                    m = s;
                }
                const float pexp = expf(s - m);
                l += pexp;
#pragma unroll
                for (int i = 0; i < DPL; i++) acc[i] = fmaf(pexp, vr[i], acc[i]);
            }
        };
        auto update = [&](bool valid, const Raw& kraw, const Raw& vraw) {
            float kr[DPL], vr[DPL];
            widen<DPL, F32>(kraw, kr);
            widen<DPL, F32>(vraw, vr);
            update_f(valid, kr, vr);
        };

        const bool has_new = p.k_new != nullptr && pos >= t_begin && pos < t_end;
        const int t_cached = has_new ? pos : t_end;  // the slot of the new token is not read from the cache
        if (t_begin < t_cached) {
            // software pipeline: the loads of pass i + 1 are issued before pass i is computed
            Raw ka, va, kb, vb;
            {
                const int ta = t_begin + warp * KPW + grp, tb = ta + KPI;
                fetch(ta, ta < t_cached, ka, va);
                fetch(tb, tb < t_cached, kb, vb);
            }
            for (int t0 = t_begin; t0 < t_cached; t0 += 2 * KPI) {
                const int ta = t0 + warp * KPW + grp, tb = ta + KPI;
                const bool va_ok = ta < t_cached, vb_ok = tb < t_cached;
                Raw nka, nva, nkb, nvb;
                const bool more = t0 + 2 * KPI < t_cached;
                if (more) {
                    const int na = ta + 2 * KPI, nb = tb + 2 * KPI;
                    fetch(na, na < t_cached, nka, nva);
                    fetch(nb, nb < t_cached, nkb, nvb);
                }
                update(va_ok, ka, va);
                update(vb_ok, kb, vb);
                if (more) { ka = nka; va = nva; kb = nkb; vb = nvb; }
            }
        }
        if (has_new) {
            // the token of this step: rotate, round through the cache type, and (one head per kv group) store
            float kr[DPL], vr[DPL];
            load_rotated<DPL, HD>(p.k_new + (size_t)tok * p.q_stride + kvh * HD, sub * DPL, rp, p.theta, kr);
            const float* vp = p.v_new + (size_t)tok * p.q_stride + kvh * HD + sub * DPL;
#pragma unroll
            for (int i = 0; i < DPL; i++) vr[i] = __ldcg(vp + i);
            if (h % gsz == 0 && warp == 0 && grp == 0) {
                const size_t a = key_addr(pos);
                store_round<DPL, F32>(kv.k_pool, a, kr);
                store_round<DPL, F32>(kv.v_pool, a, vr);
            } else if (!F32) {
#pragma unroll
                for (int i = 0; i < DPL; i++) { kr[i] = __half2float(__float2half_rn(kr[i])); vr[i] = __half2float(__float2half_rn(vr[i])); }
            }
            update_f(warp == 0 && grp == 0, kr, vr);  // counted once: by the first key group of the first warp
        }
        // merge the key groups of the warp (lanes with equal `sub` hold the same dims), fixed order
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
            const float l2 = __shfl_xor_sync(0xffffffffu, l, o);
            const float mn = fmaxf(m, m2);
            const float a1 = (m == -INFINITY) ? 0.f : expf(m - mn);
            const float a2 = (m2 == -INFINITY) ? 0.f : expf(m2 - mn);
            l = l * a1 + l2 * a2;
#pragma unroll
            for (int i = 0; i < DPL; i++) {
                const float o2 = __shfl_xor_sync(0xffffffffu, acc[i], o);
                acc[i] = acc[i] * a1 + o2 * a2;
            }
            m = mn;
        }
    }
    // merge the warps through shared memory, in warp order
    if (grp == 0) {
        if (sub == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
        for (int i = 0; i < DPL; i++) sm_acc[warp][sub * DPL + i] = acc[i];
    }
    group_sync<BAR>(bar_id);
    for (int d = tid; d < HD; d += kAttnWarps * 32) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; w++) mm = fmaxf(mm, sm_m[w]);
        float ll = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; w++) {
            const float sc = (sm_m[w] == -INFINITY) ? 0.f : expf(sm_m[w] - mm);
            ll += sm_l[w] * sc;
            a += sm_acc[w][d] * sc;
        }
        if (p.n_splits == 1) {
            p.out[(size_t)tok * n_heads * HD + h * HD + d] = a / ll;
        } else {
            if (d == 0) { pout[0] = mm; pout[1] = ll; }
            pout[2 + d] = a;
        }
    }
    if (p.n_splits == 1) return;
    // ---- the last split of this (token, head) to finish merges all of them, in split order ----
    __threadfence();
    group_sync<BAR>(bar_id);
    if (tid == 0) {
        const int done = atomicAdd(&p.counters[item], 1);
        *sm_last = (done == live - 1);
    }
    group_sync<BAR>(bar_id);
    if (!*sm_last) return;
    __threadfence();
    const float* pp = p.partial + (size_t)item * p.n_splits * (HD + 2);
    float mm = -INFINITY;
    for (int s = 0; s < live; s++) mm = fmaxf(mm, __ldcg(pp + (size_t)s * (HD + 2)));
    for (int d = tid; d < HD; d += kAttnWarps * 32) {
        float ll = 0.f, a = 0.f;
        for (int s = 0; s < live; s++) {
            const float* ps = pp + (size_t)s * (HD + 2);
            const float ms = __ldcg(ps);
            if (ms == -INFINITY) continue;  // empty split
            const float sc = expf(ms - mm);
            ll += __ldcg(ps + 1) * sc;
            a += __ldcg(ps + 2 + d) * sc;
        }
        p.out[(size_t)item * HD + d] = a / ll;
    }
    if (tid == 0) p.counters[item] = 0;  // ready for the next launch
}


constexpr int attention_group_smem_floats(int hd) { return 8 + kAttnWarps * hd + 4; }

}  // namespace lc

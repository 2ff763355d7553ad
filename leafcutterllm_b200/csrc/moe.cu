// Mixture-of-experts routing for the FFN position of a decoder layer.  The reference has dense FFNs only
// (rust/src/inference/engine.rs:146-164); the definition implemented here is this project's own and is the one the
// CPU checker restates:
//   router logits = rms_norm(x) . W_r^T with f32 router weights;
//   the top_k experts by logit, equal logits going to the HIGHER expert index (the tie rule of the reference's
//   greedy pick, rust/src/inference/sampler.rs:6-10);
//   gate weights = softmax over the selected logits;
//   output = residual + sum over the selected experts, in ascending expert index, of weight * expert_ffn(rms_norm(x)).
//
// moe_route_kernel   one CTA per token: RMS scale, one warp per (token, expert) dot product, one thread picks and weighs, and
//                    -- for calls of up to 64 tokens -- the CTA that finishes last lists, per expert and in token order, the
//                    (token, choice) slots it received, for the grouped expert product.
// moe_combine_kernel out[t] = residual[t] + sum_j w[t][j] * y[row(t, j)], j in ascending expert order.
#include "lc_kernels.h"

namespace lc {

namespace {

constexpr int kRouteTokens = 64;   // most tokens of a call whose slot lists are built (the grouped expert product's limit)
constexpr int kRouteThreads = 256;

__device__ __forceinline__ int32_t total_key_f(float f) {  // orders f32 bit patterns like Rust's f32::total_cmp
    int32_t b = __float_as_int(f);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}

// One CTA per token: the row comes into shared memory once (float4 reads; the sum of squares on the way), is normalised there,
// the warps share the experts' dot products (float4 pieces per lane in order, then the warp tree), thread 0 picks and weighs.
// The order of every sum is fixed by the block shape alone, so every rank of a cut model and every call computes the same bits.  When the call wants slot lists (`lists`), the CTA that finishes last (a ticket) reads every token's choices back
// and lists, per expert and in token order, the (token, choice) slots it received.
__global__ void __launch_bounds__(kRouteThreads)
moe_route_kernel(const float* __restrict__ x, const float* __restrict__ norm_w, float eps, int H, int T, const float* __restrict__ w_router,
                 int E, int K, int32_t* __restrict__ sel, float* __restrict__ wsel, int32_t* __restrict__ cnt, int32_t* __restrict__ lists,
                 int list_stride, unsigned long long* __restrict__ touched, int local_first, int local_count, unsigned* __restrict__ ticket) {
    extern __shared__ float xs[];  // the token's row, then its normalised form
    __shared__ float part_s[kRouteThreads / 32];
    __shared__ float logit_s[kMaxExperts];
    __shared__ int last_s;
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int t = blockIdx.x;
    const float* xr = x + (size_t)t * H;
    // cpu.rs:49-60: 1 / sqrt(mean(x^2) + eps).  Every thread sums its own float4 pieces in order, the warps' sums are added in warp order.
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i);
        *reinterpret_cast<float4*>(xs + i) = v;
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) part_s[warp] = ss;
    __syncthreads();
    float sc = 1.0f;
    if (norm_w) {
        float tot = 0.f;
        for (int w = 0; w < nwarps; w++) tot += part_s[w];
        sc = 1.0f / sqrtf(tot / (float)H + eps);
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {  // each thread its own pieces: no barrier needed before
            float4 v = *reinterpret_cast<float4*>(xs + i);
            const float4 g = *reinterpret_cast<const float4*>(norm_w + i);
            v.x = (v.x * sc) * g.x; v.y = (v.y * sc) * g.y; v.z = (v.z * sc) * g.z; v.w = (v.w * sc) * g.w;
            *reinterpret_cast<float4*>(xs + i) = v;
        }
    }
    __syncthreads();
    for (int e = warp; e < E; e += nwarps) {  // one warp per expert: lane l takes float4 pieces l, l + 32, ... in order
        const float* wr = w_router + (size_t)e * H;
        float acc = 0.f;
        for (int i = lane * 4; i < H; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(xs + i);
            const float4 w4 = __ldg(reinterpret_cast<const float4*>(wr + i));
            acc = fmaf(v.x, w4.x, acc); acc = fmaf(v.y, w4.y, acc); acc = fmaf(v.z, w4.z, acc); acc = fmaf(v.w, w4.w, acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) logit_s[e] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const float* lg = logit_s;
        unsigned long long used = 0ull;
        for (int kk = 0; kk < K; kk++) {
            int best = -1;
            for (int e = 0; e < E; e++) {
                if ((used >> e) & 1ull) continue;
                if (best < 0 || total_key_f(lg[e]) >= total_key_f(lg[best])) best = e;  // ties: the later index wins
            }
            used |= 1ull << best;
        }
        float mx = -INFINITY;
        for (int e = 0; e < E; e++) if ((used >> e) & 1ull) mx = fmaxf(mx, lg[e]);
        float sum = 0.f;
        for (int e = 0; e < E; e++) if ((used >> e) & 1ull) sum = sum + expf(lg[e] - mx);
        int j = 0;
        for (int e = 0; e < E; e++) {
            if (!((used >> e) & 1ull)) continue;
            sel[(size_t)t * K + j] = e;                       // ascending expert index
            wsel[(size_t)t * K + j] = expf(lg[e] - mx) / sum;
            j++;
        }
    }
    if (lists == nullptr) return;   // many-token calls run every expert on every token and only need sel / wsel
    if (threadIdx.x == 0) {
        __threadfence();  // this token's choices are in global memory before the ticket is
        last_s = atomicAdd(ticket, 1u) == (unsigned)(T - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    if ((int)threadIdx.x < E) {
        const int e = threadIdx.x;
        int n = 0;
        for (int tt = 0; tt < T; tt++)
            for (int j = 0; j < K; j++)
                if (__ldcg(sel + (size_t)tt * K + j) == e) lists[(size_t)e * list_stride + n++] = tt * K + j;
        cnt[e] = n;
        if (touched && n > 0 && e >= local_first && e < local_first + local_count) atomicAdd(touched, 1ull);
    }
    if (threadIdx.x == 0) *ticket = 0;  // every CTA has taken its ticket: ready for the next launch
}

// mode 0: row(t, j) = t * K + j (one row per slot); mode 1: row(t, j) = (sel[t][j] - local_first) * T_stride + t (a plane per
// local expert).  Only experts local_first .. local_first + local_count - 1 are added (a rank of a cut model adds its own).
__global__ void moe_combine_kernel(const float* __restrict__ y, const int32_t* __restrict__ sel, const float* __restrict__ wsel, int K, int H, int T,
                                   int mode, size_t t_stride, int local_first, int local_count, const float* __restrict__ residual,
                                   float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int i4 = threadIdx.x; i4 < H / 4; i4 += blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < K; j++) {
            const int e = sel[(size_t)t * K + j];
            if (e < local_first || e >= local_first + local_count) continue;
            const size_t row = mode == 0 ? (size_t)t * K + j : (size_t)(e - local_first) * t_stride + t;
            const float w = wsel[(size_t)t * K + j];
            const float4 v = *reinterpret_cast<const float4*>(y + row * H + 4 * (size_t)i4);
            acc.x = acc.x + w * v.x; acc.y = acc.y + w * v.y; acc.z = acc.z + w * v.z; acc.w = acc.w + w * v.w;
        }
        if (residual) {
            const float4 r = *reinterpret_cast<const float4*>(residual + (size_t)t * H + 4 * (size_t)i4);
            acc.x = r.x + acc.x; acc.y = r.y + acc.y; acc.z = r.z + acc.z; acc.w = r.w + acc.w;
        }
        *reinterpret_cast<float4*>(out + (size_t)t * H + 4 * (size_t)i4) = acc;
    }
}

template <typename... KArgs, typename... Args>
cudaError_t launch_dep_smem(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    if (smem > 48 * 1024) {
        cudaError_t e = ensure_smem_limit((const void*)kern, smem);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_dep(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

}  // namespace

int32_t launch_moe_route(const MoeRouteArgs& a, cudaStream_t s) {
    LC_CHECK(a.x && a.w_router && a.sel && a.wsel && a.T >= 1 && a.H >= 1, LC_ERR_INVALID, "moe route: null argument");
    LC_CHECK(a.n_experts >= 1 && a.n_experts <= kMaxExperts && a.top_k >= 1 && a.top_k <= kMaxTopK && a.top_k <= a.n_experts, LC_ERR_INVALID,
             "moe route: %d experts / top %d outside 1..%d / 1..%d", a.n_experts, a.top_k, kMaxExperts, kMaxTopK);
    const bool want_lists = a.lists != nullptr;
    if (want_lists) LC_CHECK(a.T <= kRouteTokens && a.counts && a.list_stride >= a.T, LC_ERR_INVALID, "moe route: slot lists need a call of at most %d tokens", kRouteTokens);
    if (want_lists) LC_CHECK(a.ticket != nullptr, LC_ERR_INVALID, "moe route: slot lists need the ticket word");
    LC_CHECK(a.H % 4 == 0 && ((uintptr_t)a.x % 16) == 0 && ((uintptr_t)a.w_router % 16) == 0 && (!a.norm_w || ((uintptr_t)a.norm_w % 16) == 0) &&
                 (size_t)a.H * sizeof(float) <= 160 * 1024,
             LC_ERR_INVALID, "moe route: rows must be 16-byte aligned multiples of four elements");
    LC_CUDA(launch_dep_smem(moe_route_kernel, dim3((unsigned)a.T), dim3(kRouteThreads), (size_t)a.H * sizeof(float), s, a.x, a.norm_w, a.eps, a.H, a.T, a.w_router, a.n_experts, a.top_k, a.sel,
                       a.wsel, a.counts, a.lists, a.list_stride, a.touched, a.local_first, a.local_count > 0 ? a.local_count : a.n_experts, a.ticket));
    return LC_OK;
}

int32_t launch_moe_combine(const float* y, const int32_t* sel, const float* wsel, int top_k, int H, int T, int mode, size_t t_stride,
                           int local_first, int local_count, const float* residual, float* out, cudaStream_t s) {
    LC_CHECK(y && sel && wsel && out && H % 4 == 0 && T >= 1, LC_ERR_INVALID, "moe combine: bad argument");
    LC_CUDA(launch_dep(moe_combine_kernel, dim3((unsigned)T), dim3(256), s, y, sel, wsel, top_k, H, T, mode, t_stride, local_first, local_count, residual, out));
    return LC_OK;
}

}  // namespace lc

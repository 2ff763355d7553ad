// sampler::sample_top_p, stochastic branch (rust/src/inference/sampler.rs:12-50), with the uniform draw supplied by the
// caller: temperature, softmax, stable sort by probability (descending), nucleus cut, renormalised inverse-CDF pick.
// Everything except the draw is deterministic, so with the caller's `rng.gen::<f32>()` handed in the pick equals the
// reference's.  The f32 sums are kept in the reference's order (one thread walks them): the exponent sum over the
// vocabulary in index order (:17), the running sum over the sorted probabilities (:28-32, which is also the sum of the kept
// ones, :37) and the walk to the draw (:41-47).  exp() is evaluated in f64 and rounded to f32, which agrees with a
// correctly rounded expf except within 2^-29 of a rounding boundary.
//
// The sort is a 64-bit radix sort (CUB, part of the CUDA toolkit) of keys [inverted probability bits | index]:
// ascending keys = descending probability, equal probabilities in index order -- what the reference's stable sort_by
// leaves (:23-25; NaN probabilities, which it treats as equal to everything, are not reproduced).
#include <cub/device/device_radix_sort.cuh>
#include <mutex>
#include "lc_kernels.h"

namespace lc {

namespace {

constexpr int kChunk = 8192;
constexpr int kThreads = 1024;

// probs scratch e[n]; keys[n].  One CTA.
__global__ void __launch_bounds__(kThreads)
sample_probs_kernel(const float* __restrict__ logits, int n, float temperature, float* __restrict__ e, unsigned long long* __restrict__ keys) {
    __shared__ float chunk[kChunk];
    __shared__ float sh[32];
    __shared__ float s_sum;
    float mx = -INFINITY;  // fold(NEG_INFINITY, f32::max) (:16): the maximum ignores NaN
    for (int i = threadIdx.x; i < n; i += kThreads) mx = fmaxf(mx, __fdiv_rn(logits[i], temperature));
    mx = block_max(mx, sh);
    for (int i = threadIdx.x; i < n; i += kThreads) {
        const float d = __fsub_rn(__fdiv_rn(logits[i], temperature), mx);
        e[i] = (float)exp((double)d);
    }
    __syncthreads();
    float sum = 0.f;  // iter().sum() (:17): left to right from 0.0
    for (int c0 = 0; c0 < n; c0 += kChunk) {
        const int len = min(kChunk, n - c0);
        for (int i = threadIdx.x; i < len; i += kThreads) chunk[i] = e[c0 + i];
        __syncthreads();
        if (threadIdx.x == 0)
            for (int i = 0; i < len; i++) sum = __fadd_rn(sum, chunk[i]);
        __syncthreads();
    }
    if (threadIdx.x == 0) s_sum = sum;
    __syncthreads();
    sum = s_sum;
    for (int i = threadIdx.x; i < n; i += kThreads) {
        const float p = __fdiv_rn(e[i], sum);  // (:19)
        keys[i] = ((unsigned long long)(~__float_as_uint(p)) << 32) | (unsigned)i;
    }
}

__device__ __forceinline__ float key_prob(unsigned long long k) { return __uint_as_float(~(unsigned)(k >> 32)); }

// keys sorted ascending.  One CTA; thread 0 walks the sums in order, the others stage the chunks.
__global__ void __launch_bounds__(kThreads)
sample_pick_kernel(const unsigned long long* __restrict__ keys, int n, float top_p, float u, long long* __restrict__ token) {
    __shared__ float chunk[kChunk];
    __shared__ int s_stop;
    __shared__ float s_sum;
    __shared__ int s_cut;
    if (threadIdx.x == 0) { s_stop = 0; s_cut = n - 1; }
    __syncthreads();
    // the nucleus: first position whose running sum exceeds top_p, else the last one (:28-32)
    float cum = 0.f;
    for (int c0 = 0; c0 < n; c0 += kChunk) {
        const int len = min(kChunk, n - c0);
        for (int i = threadIdx.x; i < len; i += kThreads) chunk[i] = key_prob(keys[c0 + i]);
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int i = 0; i < len; i++) {
                cum = __fadd_rn(cum, chunk[i]);
                if (cum > top_p) { s_cut = c0 + i; s_stop = 1; break; }
            }
            s_sum = cum;  // the sum of the kept probabilities in the same order (:37)
        }
        __syncthreads();
        if (s_stop) break;
    }
    const int cut = s_cut;
    const float rand_val = __fmul_rn(u, s_sum);  // (:39)
    __syncthreads();
    if (threadIdx.x == 0) s_stop = 0;
    __syncthreads();
    cum = 0.f;
    for (int c0 = 0; c0 <= cut; c0 += kChunk) {
        const int len = min(kChunk, cut + 1 - c0);
        for (int i = threadIdx.x; i < len; i += kThreads) chunk[i] = key_prob(keys[c0 + i]);
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int i = 0; i < len; i++) {
                cum = __fadd_rn(cum, chunk[i]);
                if (rand_val <= cum) { *token = (long long)(unsigned)(keys[c0 + i] & 0xFFFFFFFFull); s_stop = 1; break; }  // (:42-46)
            }
        }
        __syncthreads();
        if (s_stop) return;
    }
    if (threadIdx.x == 0) *token = (long long)(unsigned)(keys[cut] & 0xFFFFFFFFull);  // (:49)
}

struct SampleScratch {
    DevBuf e, keys_a, keys_b, tmp, token;
};
SampleScratch g_scratch[16];
std::mutex g_sample_mutex;

}  // namespace

// logits_dev: n f32 on the device; token_dev: one int64 on the device.  Uses per-device scratch: callers are serialised.
int32_t launch_sample_top_p(const float* logits_dev, size_t n, float temperature, float top_p, float u, int64_t* token_dev, cudaStream_t s) {
    LC_CHECK(logits_dev && token_dev && n >= 1 && n < ((size_t)1 << 31), LC_ERR_INVALID, "sample_top_p: bad argument");
    LC_CHECK(temperature > 0.0f, LC_ERR_INVALID, "sample_top_p: the stochastic branch needs temperature > 0 (greedy is lc_argmax)");
    int d = 0;
    LC_CUDA(cudaGetDevice(&d));
    LC_CHECK(d >= 0 && d < 16, LC_ERR_CUDA, "no current CUDA device");
    SampleScratch& S = g_scratch[d];
    LC_TRY(S.e.reserve(n * 4));
    LC_TRY(S.keys_a.reserve(n * 8));
    LC_TRY(S.keys_b.reserve(n * 8));
    size_t tmp_bytes = 0;
    LC_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, tmp_bytes, (const unsigned long long*)S.keys_a.p, (unsigned long long*)S.keys_b.p, (int)n,
                                           0, 64, s));
    LC_TRY(S.tmp.reserve(tmp_bytes + 16));
    sample_probs_kernel<<<1, kThreads, 0, s>>>(logits_dev, (int)n, temperature, (float*)S.e.p, (unsigned long long*)S.keys_a.p);
    LC_CUDA(cudaGetLastError());
    LC_CUDA(cub::DeviceRadixSort::SortKeys(S.tmp.p, tmp_bytes, (const unsigned long long*)S.keys_a.p, (unsigned long long*)S.keys_b.p, (int)n, 0,
                                           64, s));
    sample_pick_kernel<<<1, kThreads, 0, s>>>((const unsigned long long*)S.keys_b.p, (int)n, top_p, u, (long long*)token_dev);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}

// Launch + read back, serialised over the per-device scratch.  temperature <= 0 is the greedy branch (sampler.rs:7-10).
int32_t sample_top_p_sync(const float* logits_dev, size_t n, float temperature, float top_p, float u, int64_t* token_host, cudaStream_t s) {
    std::lock_guard<std::mutex> lk(g_sample_mutex);
    int d = 0;
    LC_CUDA(cudaGetDevice(&d));
    LC_CHECK(d >= 0 && d < 16, LC_ERR_CUDA, "no current CUDA device");
    LC_TRY(g_scratch[d].token.reserve(8));
    int64_t* tok = (int64_t*)g_scratch[d].token.p;
    if (temperature <= 0.0f) {
        LC_TRY(launch_argmax(logits_dev, n, 1, tok, s));
    } else {
        LC_TRY(launch_sample_top_p(logits_dev, n, temperature, top_p, u, tok, s));
    }
    LC_CUDA(cudaMemcpyAsync(token_host, tok, 8, cudaMemcpyDeviceToHost, s));
    LC_CUDA(cudaStreamSynchronize(s));
    return LC_OK;
}

// The uniform draws of a seeded generation: draw i of seed s is the top 24 bits of splitmix64(s + i) scaled to [0, 1) --
// the grid rand's Standard f32 distribution uses, not its generator (the reference draws from an unseeded thread_rng).
float seeded_uniform(uint64_t seed, uint64_t index) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (index + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

}  // namespace lc

using namespace lc;

extern "C" {

int32_t lc_sample_top_p(const float* logits, size_t n, float temperature, float top_p, float u, int64_t* token) {
    LC_CHECK(logits && token && n >= 1, LC_ERR_INVALID, "lc_sample_top_p: bad argument");
    if (!have_device()) return LC_ERR_CUDA;
    static std::mutex in_mutex;
    std::lock_guard<std::mutex> lk(in_mutex);
    int d = 0;
    LC_CUDA(cudaGetDevice(&d));
    LC_CHECK(d >= 0 && d < 16, LC_ERR_CUDA, "no current CUDA device");
    static DevBuf in[16];
    LC_TRY(in[d].reserve(n * 4));
    LC_CUDA(cudaMemcpyAsync(in[d].p, logits, n * 4, cudaMemcpyHostToDevice, stream()));
    return sample_top_p_sync((const float*)in[d].p, n, temperature, top_p, u, token, stream());
}

float lc_seeded_uniform(uint64_t seed, uint64_t index) { return seeded_uniform(seed, index); }

}  // extern "C"

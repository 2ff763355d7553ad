// Operator-level kernels: one per method of the reference's `trait Backend`
// (rust/src/backend/mod.rs:18-46) plus RoPE, argmax and the shard-order
// quantised GEMMs, and the host-pointer C entry points built on them.
#include <mutex>
#include <algorithm>
#include "lc_kernels.h"
#include "lc_quant.cuh"
#include "lc_tma.cuh"

namespace lc {

static inline int ew_grid(size_t n) {
    size_t g = (n + 255) / 256;
    size_t cap = (size_t)sm_count() * 8;
    return (int)(g < cap ? (g ? g : 1) : cap);
}

#define EW_LOOP(n)                                                      \
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;           \
    size_t stride = (size_t)gridDim.x * blockDim.x;                     \
    for (; i < (n); i += stride)

__global__ void vec_add_kernel(const float* a, const float* b, size_t n, float* o) { EW_LOOP(n) o[i] = __fadd_rn(a[i], b[i]); }
__global__ void vec_mul_kernel(const float* a, const float* b, size_t n, float* o) { EW_LOOP(n) o[i] = __fmul_rn(a[i], b[i]); }
__global__ void vec_scale_kernel(const float* a, float s, size_t n, float* o) { EW_LOOP(n) o[i] = __fmul_rn(a[i], s); }
__global__ void vec_scale_mul_kernel(const float* a, float s, const float* b, size_t n, float* o) {
    EW_LOOP(n) o[i] = __fmul_rn(__fmul_rn(a[i], s), b[i]);
}
// cpu.rs:62-64: v * (1 / (1 + exp(-v)))
__device__ __forceinline__ float silu1(float v) { return __fmul_rn(v, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v)))); }
__global__ void silu_kernel(const float* x, size_t n, float* o) { EW_LOOP(n) o[i] = silu1(x[i]); }
__global__ void silu_mul_kernel(const float* g, const float* u, size_t n, float* o) { EW_LOOP(n) o[i] = __fmul_rn(silu1(g[i]), u[i]); }

// cpu.rs:49-60: scale = 1/sqrt(mean(x^2)+eps); out = (x*scale)*w
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, size_t hidden,
                                float* __restrict__ o) {
    __shared__ float sh[32];
    const float* xr = x + (size_t)blockIdx.x * hidden;
    float* orow = o + (size_t)blockIdx.x * hidden;
    float acc = 0.0f;
    for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) acc = fmaf(xr[i], xr[i], acc);
    float ss = block_sum(acc, sh);
    float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)hidden), eps)));
    for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) orow[i] = __fmul_rn(__fmul_rn(xr[i], scale), w[i]);
}

// cpu.rs:66-79
__global__ void softmax_kernel(const float* __restrict__ x, size_t hidden, float* __restrict__ o) {
    __shared__ float sh[32];
    const float* xr = x + (size_t)blockIdx.x * hidden;
    float* orow = o + (size_t)blockIdx.x * hidden;
    float mx = -INFINITY;
    for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) mx = fmaxf(mx, xr[i]);
    mx = block_max(mx, sh);
    float sum = 0.0f;
    for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) sum += expf(xr[i] - mx);
    sum = block_sum(sum, sh);
    for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) orow[i] = __fdiv_rn(expf(xr[i] - mx), sum);
}

__global__ void sum_sq_kernel(const float* __restrict__ x, size_t n, float* out) {
    __shared__ float sh[32];
    float acc = 0.0f;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) acc = fmaf(x[i], x[i], acc);
    float ss = block_sum(acc, sh);
    if (threadIdx.x == 0) *out = ss;
}

// Backend::matmul.  Each thread owns one output element and walks k in ascending order with one
// fused multiply-add per step, which is exactly the chain of rust/src/kernels/simd.rs:226-249
// (columns past the last multiple of 8 use the unfused tail of :238-246) -- so the result is
// bit-identical to the reference on an AVX2+FMA host.  32x32 tiles of a and b go through shared memory.
__global__ void matmul_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, size_t m, size_t k, size_t n,
                                  float* __restrict__ c) {
    __shared__ float as[32][33];
    __shared__ float bs[32][33];
    size_t row = (size_t)blockIdx.y * 32 + threadIdx.y;
    size_t col = (size_t)blockIdx.x * 32 + threadIdx.x;
    bool fused = col < (n & ~(size_t)7);
    float acc = 0.0f;
    for (size_t k0 = 0; k0 < k; k0 += 32) {
        size_t ka = k0 + threadIdx.x, kb = k0 + threadIdx.y;
        as[threadIdx.y][threadIdx.x] = (row < m && ka < k) ? a[row * k + ka] : 0.0f;
        bs[threadIdx.y][threadIdx.x] = (kb < k && col < n) ? b[kb * n + col] : 0.0f;
        __syncthreads();
        size_t kk = (k - k0 < 32) ? (k - k0) : 32;
        if (fused) {
            for (size_t l = 0; l < kk; l++) acc = fmaf(as[threadIdx.y][l], bs[l][threadIdx.x], acc);
        } else {
            for (size_t l = 0; l < kk; l++) acc = __fadd_rn(acc, __fmul_rn(as[threadIdx.y][l], bs[l][threadIdx.x]));
        }
        __syncthreads();
    }
    if (row < m && col < n) c[row * n + col] = acc;
}

// Shard-order quantised GEMM, rust/src/kernels/int8_gemm.rs:49-98 / :240-280: blocks [k][n/32], f32 scale.
// One thread per output element, l ascending, deq = q*scale (one rounding), c = fma(a, deq, c):
// bit-identical to the reference's AVX2 path.
__global__ void q8_0_shard_kernel(const float* __restrict__ a, const float* __restrict__ scales, const int8_t* __restrict__ qs,
                                  size_t m, size_t k, size_t n, float* __restrict__ c) {
    size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t i = blockIdx.y;
    if (j >= n || i >= m) return;
    size_t bpr = n / 32;
    float acc = 0.0f;
    for (size_t l = 0; l < k; l++) {
        float deq = __fmul_rn((float)qs[l * n + j], scales[l * bpr + (j >> 5)]);
        acc = fmaf(a[i * k + l], deq, acc);
    }
    c[i * n + j] = acc;
}
__global__ void q4_0_shard_kernel(const float* __restrict__ a, const float* __restrict__ scales, const uint8_t* __restrict__ qs,
                                  size_t m, size_t k, size_t n, float* __restrict__ c) {
    size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t i = blockIdx.y;
    if (j >= n || i >= m) return;
    size_t bpr = n / 32;
    float acc = 0.0f;
    for (size_t l = 0; l < k; l++) {
        uint8_t byte = qs[(l * n + j) >> 1];  // q4_0.rs:36-46: byte i holds elements 2i (low) and 2i+1 (high)
        int nib = (j & 1) ? (byte >> 4) : (byte & 0x0F);
        float deq = __fmul_rn(__fsub_rn((float)nib, 8.0f), scales[l * bpr + (j >> 5)]);
        acc = fmaf(a[i * k + l], deq, acc);
    }
    c[i * n + j] = acc;
}

// attention.rs:13-34.  One thread per (position, head, pair).
__global__ void rope_kernel(float* x, size_t seq, size_t heads, size_t hd, float theta, const int32_t* pos0_dev, int32_t pos0) {
    size_t half = hd / 2;
    size_t total = seq * heads * half;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    size_t d = idx % half;
    size_t h = (idx / half) % heads;
    size_t i = idx / (half * heads);
    int32_t p0 = pos0_dev ? *pos0_dev : pos0;
    float freq = __fdiv_rn(1.0f, powf(theta, __fdiv_rn(__fmul_rn(2.0f, (float)d), (float)hd)));
    float angle = __fmul_rn((float)(i + (size_t)p0), freq);
    float ca = cosf(angle), sa = sinf(angle);
    size_t base = i * heads * hd + h * hd;
    float x1 = x[base + d], x2 = x[base + d + half];
    x[base + d] = __fsub_rn(__fmul_rn(x1, ca), __fmul_rn(x2, sa));
    x[base + d + half] = __fadd_rn(__fmul_rn(x1, sa), __fmul_rn(x2, ca));
}

// Key that orders f32 bit patterns like Rust's f32::total_cmp.
__device__ __forceinline__ int32_t total_key(float f) {
    int32_t b = __float_as_int(f);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}
// sampler.rs:6-10: max_by keeps the last of equal maxima -> compare (key, index) pairs.
// The same pick kept as its key, with the index offset by index_base: the maximum of such keys over vocabulary slices is
// the pick over the whole vocabulary, equal maxima still going to the higher index.
__global__ void __launch_bounds__(1024) argmax_key_kernel(const float* __restrict__ v, size_t n, int index_base, long long* out) {
    __shared__ long long shk[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = v + (size_t)blockIdx.x * n;
    long long best = LLONG_MIN;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
        long long key = ((long long)total_key(row[i]) << 32) | (long long)(uint32_t)(index_base + (int)i);
        best = key > best ? key : best;
    }
    for (int o = 16; o > 0; o >>= 1) {
        long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) shk[w] = best;
    __syncthreads();
    if (w == 0) {
        best = lane < nw ? shk[lane] : LLONG_MIN;
        for (int o = 16; o > 0; o >>= 1) {
            long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (lane == 0) out[blockIdx.x] = best;
    }
}
__global__ void key_to_token_kernel(const long long* __restrict__ keys, size_t rows, int64_t* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows) out[i] = (int64_t)(uint32_t)(keys[i] & 0xffffffffll);
}

__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ v, size_t n, int64_t* out) {
    __shared__ long long shk[32];
    pdl_launch_dependents();
    pdl_wait();  // the logits come from the kernel ahead
    const float* row = v + (size_t)blockIdx.x * n;
    long long best = LLONG_MIN;
    auto take = [&](float x, size_t i) {
        const long long key = ((long long)total_key(x) << 32) | (long long)(uint32_t)i;
        best = key > best ? key : best;
    };
    if ((n & 3) == 0 && ((uintptr_t)row & 15) == 0) {
        for (size_t i = (size_t)threadIdx.x * 4; i < n; i += (size_t)blockDim.x * 4) {
            const float4 q = *reinterpret_cast<const float4*>(row + i);
            take(q.x, i); take(q.y, i + 1); take(q.z, i + 2); take(q.w, i + 3);
        }
    } else {
        for (size_t i = threadIdx.x; i < n; i += blockDim.x) take(row[i], i);
    }
    for (int o = 16; o > 0; o >>= 1) {
        long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) shk[w] = best;
    __syncthreads();
    if (w == 0) {
        best = lane < nw ? shk[lane] : LLONG_MIN;
        for (int o = 16; o > 0; o >>= 1) {
            long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (lane == 0) out[blockIdx.x] = (int64_t)(uint32_t)(best & 0xffffffffll);
    }
}

#define LAUNCH_EW(kern, n, ...)                                         \
    do {                                                                \
        if ((n) == 0) return LC_OK;                                     \
        kern<<<ew_grid(n), 256, 0, s>>>(__VA_ARGS__);                   \
        LC_CUDA(cudaGetLastError());                                    \
        return LC_OK;                                                   \
    } while (0)

int32_t launch_vec_add(const float* a, const float* b, size_t n, float* o, cudaStream_t s) { LAUNCH_EW(vec_add_kernel, n, a, b, n, o); }
int32_t launch_vec_mul(const float* a, const float* b, size_t n, float* o, cudaStream_t s) { LAUNCH_EW(vec_mul_kernel, n, a, b, n, o); }
int32_t launch_vec_scale(const float* a, float sc, size_t n, float* o, cudaStream_t s) { LAUNCH_EW(vec_scale_kernel, n, a, sc, n, o); }
int32_t launch_vec_scale_mul(const float* a, float sc, const float* b, size_t n, float* o, cudaStream_t s) {
    LAUNCH_EW(vec_scale_mul_kernel, n, a, sc, b, n, o);
}
int32_t launch_silu(const float* x, size_t n, float* o, cudaStream_t s) { LAUNCH_EW(silu_kernel, n, x, n, o); }
int32_t launch_silu_mul(const float* g, const float* u, size_t n, float* o, cudaStream_t s) { LAUNCH_EW(silu_mul_kernel, n, g, u, n, o); }

int32_t launch_rms_norm(const float* x, const float* w, float eps, size_t hidden, size_t rows, float* o, cudaStream_t s) {
    if (rows == 0 || hidden == 0) return LC_OK;
    rms_norm_kernel<<<(unsigned)rows, 256, 0, s>>>(x, w, eps, hidden, o);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}
int32_t launch_softmax(const float* x, size_t hidden, size_t rows, float* o, cudaStream_t s) {
    if (rows == 0 || hidden == 0) return LC_OK;
    softmax_kernel<<<(unsigned)rows, 256, 0, s>>>(x, hidden, o);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}
int32_t launch_sum_sq(const float* x, size_t n, float* out1, cudaStream_t s) {
    sum_sq_kernel<<<1, 1024, 0, s>>>(x, n, out1);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}
int32_t launch_matmul_f32(const float* a, const float* b, size_t m, size_t k, size_t n, float* c, cudaStream_t s) {
    if (m == 0 || n == 0) return LC_OK;
    dim3 grid((unsigned)((n + 31) / 32), (unsigned)((m + 31) / 32));
    matmul_f32_kernel<<<grid, dim3(32, 32), 0, s>>>(a, b, m, k, n, c);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}
int32_t launch_q8_0_shard(const float* a, const float* scales, const int8_t* qs, size_t m, size_t k, size_t n, float* c, cudaStream_t s) {
    if (m == 0 || n == 0) return LC_OK;
    dim3 grid((unsigned)((n + 127) / 128), (unsigned)m);
    q8_0_shard_kernel<<<grid, 128, 0, s>>>(a, scales, qs, m, k, n, c);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}
int32_t launch_q4_0_shard(const float* a, const float* scales, const uint8_t* qs, size_t m, size_t k, size_t n, float* c, cudaStream_t s) {
    if (m == 0 || n == 0) return LC_OK;
    dim3 grid((unsigned)((n + 127) / 128), (unsigned)m);
    q4_0_shard_kernel<<<grid, 128, 0, s>>>(a, scales, qs, m, k, n, c);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}
int32_t launch_rope(float* x, size_t seq, size_t heads, size_t hd, float theta, const int32_t* pos0_dev, int32_t pos0, cudaStream_t s) {
    size_t total = seq * heads * (hd / 2);
    if (total == 0) return LC_OK;
    rope_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(x, seq, heads, hd, theta, pos0_dev, pos0);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}
int32_t launch_argmax(const float* v, size_t n, size_t rows, int64_t* out, cudaStream_t s) {
    if (rows == 0 || n == 0) return LC_OK;
    LC_CUDA(launch_pdl(argmax_kernel, dim3((unsigned)rows), dim3(1024), 0, s, v, n, out));
    return LC_OK;
}
int32_t launch_argmax_key(const float* v, size_t n, size_t rows, int index_base, long long* out_keys, cudaStream_t s) {
    if (rows == 0 || n == 0) return LC_OK;
    LC_CUDA(launch_pdl(argmax_key_kernel, dim3((unsigned)rows), dim3(1024), 0, s, v, n, index_base, out_keys));
    return LC_OK;
}
int32_t launch_key_to_token(const long long* keys, size_t rows, int64_t* out_tokens, cudaStream_t s) {
    if (rows == 0) return LC_OK;
    LC_CUDA(launch_pdl(key_to_token_kernel, dim3((unsigned)((rows + 127) / 128)), dim3(128), 0, s, keys, rows, out_tokens));
    return LC_OK;
}

}  // namespace lc

// ===========================================================================
// L1 C entry points: host slices in, host slice out (the shape of `trait Backend`).
// Each call stages through device scratch that is kept between calls.
// ===========================================================================
using namespace lc;

namespace {
std::mutex g_l1_mutex;
struct L1Scratch { DevBuf a, b, c, d; };
L1Scratch g_l1[16];

L1Scratch* l1() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
    return &g_l1[dev];
}
int32_t up(DevBuf& buf, const void* host, size_t bytes) {
    LC_TRY(buf.reserve(bytes ? bytes : 1));
    if (bytes) LC_CUDA(cudaMemcpyAsync(buf.p, host, bytes, cudaMemcpyHostToDevice, stream()));
    return LC_OK;
}
int32_t down(void* host, const DevBuf& buf, size_t bytes) {
    if (bytes) LC_CUDA(cudaMemcpyAsync(host, buf.p, bytes, cudaMemcpyDeviceToHost, stream()));
    LC_CUDA(cudaStreamSynchronize(stream()));
    return LC_OK;
}
}  // namespace

#define L1_ENTER()                                       \
    if (!have_device()) return LC_ERR_CUDA;              \
    std::lock_guard<std::mutex> _lk(g_l1_mutex);         \
    L1Scratch* S = l1();                                 \
    LC_CHECK(S != nullptr, LC_ERR_CUDA, "no current CUDA device")

extern "C" {

int32_t lc_matmul_f32(const float* a, const float* b, size_t m, size_t k, size_t n, float* c) {
    LC_CHECK(a && b && c, LC_ERR_INVALID, "lc_matmul_f32: null pointer");
    L1_ENTER();
    LC_TRY(up(S->a, a, m * k * 4));
    LC_TRY(up(S->b, b, k * n * 4));
    LC_TRY(S->c.reserve(m * n * 4 + 4));
    LC_TRY(launch_matmul_f32((float*)S->a.p, (float*)S->b.p, m, k, n, (float*)S->c.p, stream()));
    return down(c, S->c, m * n * 4);
}

#define L1_BINARY(NAME, LAUNCH)                                                    \
    int32_t NAME(const float* a, const float* b, size_t n, float* out) {           \
        LC_CHECK(a && b && out, LC_ERR_INVALID, #NAME ": null pointer");           \
        L1_ENTER();                                                                \
        LC_TRY(up(S->a, a, n * 4));                                                \
        LC_TRY(up(S->b, b, n * 4));                                                \
        LC_TRY(S->c.reserve(n * 4 + 4));                                           \
        LC_TRY(LAUNCH((float*)S->a.p, (float*)S->b.p, n, (float*)S->c.p, stream())); \
        return down(out, S->c, n * 4);                                             \
    }
L1_BINARY(lc_vec_add, launch_vec_add)
L1_BINARY(lc_vec_mul, launch_vec_mul)

int32_t lc_vec_scale(const float* a, float scale, size_t n, float* out) {
    LC_CHECK(a && out, LC_ERR_INVALID, "lc_vec_scale: null pointer");
    L1_ENTER();
    LC_TRY(up(S->a, a, n * 4));
    LC_TRY(S->c.reserve(n * 4 + 4));
    LC_TRY(launch_vec_scale((float*)S->a.p, scale, n, (float*)S->c.p, stream()));
    return down(out, S->c, n * 4);
}
int32_t lc_vec_scale_mul(const float* a, float scale, const float* b, size_t n, float* out) {
    LC_CHECK(a && b && out, LC_ERR_INVALID, "lc_vec_scale_mul: null pointer");
    L1_ENTER();
    LC_TRY(up(S->a, a, n * 4));
    LC_TRY(up(S->b, b, n * 4));
    LC_TRY(S->c.reserve(n * 4 + 4));
    LC_TRY(launch_vec_scale_mul((float*)S->a.p, scale, (float*)S->b.p, n, (float*)S->c.p, stream()));
    return down(out, S->c, n * 4);
}
int32_t lc_rms_norm(const float* x, const float* weight, float eps, size_t hidden, size_t rows, float* out) {
    LC_CHECK(x && weight && out, LC_ERR_INVALID, "lc_rms_norm: null pointer");
    LC_CHECK(hidden > 0, LC_ERR_INVALID, "lc_rms_norm: hidden must be positive");
    L1_ENTER();
    LC_TRY(up(S->a, x, rows * hidden * 4));
    LC_TRY(up(S->b, weight, hidden * 4));
    LC_TRY(S->c.reserve(rows * hidden * 4 + 4));
    LC_TRY(launch_rms_norm((float*)S->a.p, (float*)S->b.p, eps, hidden, rows, (float*)S->c.p, stream()));
    return down(out, S->c, rows * hidden * 4);
}
int32_t lc_silu(const float* x, size_t n, float* out) {
    LC_CHECK(x && out, LC_ERR_INVALID, "lc_silu: null pointer");
    L1_ENTER();
    LC_TRY(up(S->a, x, n * 4));
    LC_TRY(S->c.reserve(n * 4 + 4));
    LC_TRY(launch_silu((float*)S->a.p, n, (float*)S->c.p, stream()));
    return down(out, S->c, n * 4);
}
int32_t lc_softmax(const float* x, size_t hidden, size_t rows, float* out) {
    LC_CHECK(x && out, LC_ERR_INVALID, "lc_softmax: null pointer");
    LC_CHECK(hidden > 0, LC_ERR_INVALID, "lc_softmax: hidden must be positive");
    L1_ENTER();
    LC_TRY(up(S->a, x, rows * hidden * 4));
    LC_TRY(S->c.reserve(rows * hidden * 4 + 4));
    LC_TRY(launch_softmax((float*)S->a.p, hidden, rows, (float*)S->c.p, stream()));
    return down(out, S->c, rows * hidden * 4);
}
int32_t lc_sum_sq(const float* x, size_t n, float* out) {
    LC_CHECK(x && out, LC_ERR_INVALID, "lc_sum_sq: null pointer");
    L1_ENTER();
    LC_TRY(up(S->a, x, n * 4));
    LC_TRY(S->c.reserve(16));
    LC_TRY(launch_sum_sq((float*)S->a.p, n, (float*)S->c.p, stream()));
    return down(out, S->c, 4);
}

int32_t lc_dequantize(uint32_t typ, const void* bytes, size_t n_elems, float* out) {
    LC_CHECK(bytes && out, LC_ERR_INVALID, "lc_dequantize: null pointer");
    QuantGeom g;
    LC_CHECK(quant_geom(typ, &g), LC_ERR_UNSUPPORTED, "lc_dequantize: unsupported ggml type %u", typ);
    LC_CHECK(n_elems % g.block_elems == 0, LC_ERR_INVALID, "lc_dequantize: %zu elements is not a whole number of blocks", n_elems);
    L1_ENTER();
    LC_TRY(up(S->a, bytes, lc_tensor_bytes(typ, n_elems)));
    LC_TRY(S->c.reserve(n_elems * 4 + 4));
    LC_TRY(launch_dequant(typ, S->a.p, n_elems, (float*)S->c.p, stream()));
    return down(out, S->c, n_elems * 4);
}
int32_t lc_dequantize_dev(uint32_t typ, const void* bytes_dev, size_t n_elems, float* out_dev) {
    if (!have_device()) return LC_ERR_CUDA;
    return launch_dequant(typ, bytes_dev, n_elems, out_dev, stream());
}

// Rows of `a` against a quantised matrix: token tiles of at most 8 rows per pass of the matrix-vector kernels, or -- for
// five rows and more of Q4_K or Q5_K -- chunks of up to 512 rows through the tensor-core product (qgemm_umma.cu).
static int32_t qmatmul_rows(const QWeight& w, const float* a_dev, size_t m, float* c_dev) {
    static GemmWorkspace ws;  // callers are serialised (L1 mutex / single library stream)
    GemvArgs probe;
    probe.w = &w;
    probe.x = a_dev;
    probe.out = c_dev;
    const int chunk = 512;
    if ((w.typ == LC_TYPE_Q4_K || w.typ == LC_TYPE_Q5_K) && w.has_tmap && m >= 5) {
        if (!ws.xh || ws.k_max < w.k) {
            qgemm_workspace_free(&ws);
            LC_TRY(qgemm_workspace_alloc(&ws, chunk, w.k));
        }
    }
    for (size_t m0 = 0; m0 < m;) {
        GemvArgs ga;
        ga.w = &w;
        ga.x = a_dev + m0 * w.k;
        ga.out = c_dev + m0 * w.n;
        const int left = (int)std::min<size_t>(m - m0, (size_t)chunk);
        if (ws.xh && qgemm_applies(ga, left, ws)) {
            ga.m = left;
            LC_TRY(launch_qgemm(ga, ws, stream()));
        } else {
            ga.m = std::min(left, 8);
            LC_TRY(launch_qgemv(ga, stream()));
        }
        m0 += ga.m;
    }
    return LC_OK;
}

int32_t lc_qmatmul(uint32_t typ, const float* a, const void* w_blocks, size_t m, size_t k, size_t n, float* c) {
    LC_CHECK(a && w_blocks && c, LC_ERR_INVALID, "lc_qmatmul: null pointer");
    QuantGeom g;
    LC_CHECK(quant_geom(typ, &g), LC_ERR_UNSUPPORTED, "lc_qmatmul: unsupported ggml type %u", typ);
    LC_CHECK(k % g.block_elems == 0, LC_ERR_INVALID, "lc_qmatmul: k=%zu is not a multiple of the block size %u", k, g.block_elems);
    if (m == 0 || n == 0) return LC_OK;
    L1_ENTER();
    LC_TRY(up(S->a, a, m * k * 4));
    LC_TRY(up(S->b, w_blocks, lc_tensor_bytes(typ, n * k)));
    LC_TRY(S->c.reserve(m * n * 4 + 4));
    QWeight w;
    LC_TRY(qweight_init(&w, typ, S->b.p, (int)n, (int)k));
    LC_TRY(qmatmul_rows(w, (float*)S->a.p, m, (float*)S->c.p));
    return down(c, S->c, m * n * 4);
}
int32_t lc_qmatmul_dev(uint32_t typ, const float* a_dev, const void* w_dev, size_t m, size_t k, size_t n, float* c_dev) {
    if (!have_device()) return LC_ERR_CUDA;
    QuantGeom g;
    LC_CHECK(quant_geom(typ, &g), LC_ERR_UNSUPPORTED, "lc_qmatmul_dev: unsupported ggml type %u", typ);
    LC_CHECK(k % g.block_elems == 0, LC_ERR_INVALID, "lc_qmatmul_dev: k=%zu is not a multiple of the block size %u", k, g.block_elems);
    QWeight w;
    LC_TRY(qweight_init(&w, typ, w_dev, (int)n, (int)k));
    return qmatmul_rows(w, a_dev, m, c_dev);
}

int32_t lc_tcgen05_probe(double* out16) {
    if (!have_device()) return LC_ERR_CUDA;
    LC_CHECK(out16 != nullptr, LC_ERR_INVALID, "lc_tcgen05_probe: null pointer");
    return run_tcgen05_probe(out16, stream());
}

int32_t lc_q8_0_matmul_shard(const float* a, const float* scales, const int8_t* qs, size_t m, size_t k, size_t n, float* c) {
    LC_CHECK(a && scales && qs && c, LC_ERR_INVALID, "lc_q8_0_matmul_shard: null pointer");
    LC_CHECK(n % 32 == 0, LC_ERR_INVALID, "lc_q8_0_matmul_shard: n=%zu must be a multiple of 32", n);
    L1_ENTER();
    LC_TRY(up(S->a, a, m * k * 4));
    LC_TRY(up(S->b, scales, k * (n / 32) * 4));
    LC_TRY(up(S->d, qs, k * n));
    LC_TRY(S->c.reserve(m * n * 4 + 4));
    LC_TRY(launch_q8_0_shard((float*)S->a.p, (float*)S->b.p, (int8_t*)S->d.p, m, k, n, (float*)S->c.p, stream()));
    return down(c, S->c, m * n * 4);
}
int32_t lc_q4_0_matmul_shard(const float* a, const float* scales, const uint8_t* qs, size_t m, size_t k, size_t n, float* c) {
    LC_CHECK(a && scales && qs && c, LC_ERR_INVALID, "lc_q4_0_matmul_shard: null pointer");
    LC_CHECK(n % 32 == 0, LC_ERR_INVALID, "lc_q4_0_matmul_shard: n=%zu must be a multiple of 32", n);
    L1_ENTER();
    LC_TRY(up(S->a, a, m * k * 4));
    LC_TRY(up(S->b, scales, k * (n / 32) * 4));
    LC_TRY(up(S->d, qs, k * n / 2));
    LC_TRY(S->c.reserve(m * n * 4 + 4));
    LC_TRY(launch_q4_0_shard((float*)S->a.p, (float*)S->b.p, (uint8_t*)S->d.p, m, k, n, (float*)S->c.p, stream()));
    return down(c, S->c, m * n * 4);
}

int32_t lc_rope(float* x, size_t seq, size_t heads, size_t head_dim, float theta, size_t pos0) {
    LC_CHECK(x, LC_ERR_INVALID, "lc_rope: null pointer");
    LC_CHECK(head_dim % 2 == 0, LC_ERR_INVALID, "lc_rope: head_dim must be even");
    L1_ENTER();
    size_t bytes = seq * heads * head_dim * 4;
    LC_TRY(up(S->a, x, bytes));
    LC_TRY(launch_rope((float*)S->a.p, seq, heads, head_dim, theta, nullptr, (int32_t)pos0, stream()));
    return down(x, S->a, bytes);
}
int32_t lc_argmax(const float* v, size_t n, int64_t* out_index) {
    LC_CHECK(v && out_index && n > 0, LC_ERR_INVALID, "lc_argmax: bad argument");
    L1_ENTER();
    LC_TRY(up(S->a, v, n * 4));
    LC_TRY(S->c.reserve(16));
    LC_TRY(launch_argmax((float*)S->a.p, n, 1, (int64_t*)S->c.p, stream()));
    return down(out_index, S->c, 8);
}

}  // extern "C"

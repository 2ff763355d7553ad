// Runtime plumbing of the library: error text, device/stream management,
// device memory helpers, the event stopwatch and the L2 flush.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>
#include "lc_common.cuh"

namespace lc {

static thread_local char g_err[1024] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
const char* get_error() { return g_err; }

static constexpr int kMaxDev = 16;
static cudaStream_t g_streams[kMaxDev] = {};
static int g_sms[kMaxDev] = {};
static std::mutex g_rt_mutex;

bool have_device() {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        set_error("no usable CUDA device (%s); this library has no CPU fallback",
                  e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
        (void)cudaGetLastError();
        return false;
    }
    return true;
}

cudaStream_t stream() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
    std::lock_guard<std::mutex> lk(g_rt_mutex);
    if (!g_streams[dev]) {
        if (cudaStreamCreateWithFlags(&g_streams[dev], cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    }
    return g_streams[dev];
}

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return 148;
    std::lock_guard<std::mutex> lk(g_rt_mutex);
    if (!g_sms[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        g_sms[dev] = v;
    }
    return g_sms[dev];
}

cudaError_t ensure_smem_limit(const void* kern, size_t bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    static std::map<std::pair<int, const void*>, size_t> done;
    std::lock_guard<std::mutex> lk(g_rt_mutex);
    auto key = std::make_pair(dev, kern);
    auto it = done.find(key);
    if (it != done.end() && it->second >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) done[key] = bytes;
    return e;
}

bool quant_geom(uint32_t typ, QuantGeom* g) {
    switch (typ) {
        case LC_TYPE_F32: *g = {1, 4}; return true;
        case LC_TYPE_F16: *g = {1, 2}; return true;
        case LC_TYPE_Q4_0: *g = {32, 18}; return true;
        case LC_TYPE_Q8_0: *g = {32, 34}; return true;
        case LC_TYPE_Q4_K: *g = {256, 144}; return true;
        case LC_TYPE_Q5_K: *g = {256, 176}; return true;
        case LC_TYPE_Q6_K: *g = {256, 210}; return true;
        case LC_TYPE_IQ4_NL: *g = {32, 18}; return true;
        default: return false;
    }
}

int32_t DevBuf::reserve(size_t bytes) {
    if (bytes <= cap) return LC_OK;
    if (p) { cudaFree(p); p = nullptr; cap = 0; }
    size_t want = (bytes + 255) & ~(size_t)255;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("device allocation of %zu bytes failed: %s", want, cudaGetErrorString(e));
        p = nullptr;
        return LC_ERR_OOM;
    }
    cap = want;
    return LC_OK;
}
void DevBuf::release() {
    if (p) cudaFree(p);
    p = nullptr;
    cap = 0;
}

}  // namespace lc

using namespace lc;

static cudaEvent_t g_ev0[16] = {}, g_ev1[16] = {};
static DevBuf g_flush[16];

__global__ void lc_fill_kernel(uint4* p, size_t n, uint32_t v) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) p[i] = make_uint4(v, v, v, v);
}

extern "C" {

const char* lc_last_error(void) { return get_error(); }
const char* lc_version(void) { return "leafcutter_b200 0.1 (sm_100a)"; }

int32_t lc_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    return n;
}
int32_t lc_set_device(int32_t device) {
    if (!have_device()) return LC_ERR_CUDA;
    LC_CUDA(cudaSetDevice(device));
    return LC_OK;
}

size_t lc_tensor_bytes(uint32_t typ, size_t count) {
    QuantGeom g;
    if (!quant_geom(typ, &g)) return count;
    return (count + g.block_elems - 1) / g.block_elems * g.block_bytes;
}

int32_t lc_dev_alloc(size_t bytes, void** out_dev) {
    LC_CHECK(out_dev != nullptr, LC_ERR_INVALID, "lc_dev_alloc: null output");
    if (!have_device()) return LC_ERR_CUDA;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
        return LC_ERR_OOM;
    }
    *out_dev = p;
    return LC_OK;
}
int32_t lc_dev_free(void* dev) {
    if (dev) LC_CUDA(cudaFree(dev));
    return LC_OK;
}
int32_t lc_dev_upload(void* dst_dev, const void* src_host, size_t bytes) {
    if (!have_device()) return LC_ERR_CUDA;
    LC_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, stream()));
    LC_CUDA(cudaStreamSynchronize(stream()));
    return LC_OK;
}
int32_t lc_dev_download(void* dst_host, const void* src_dev, size_t bytes) {
    if (!have_device()) return LC_ERR_CUDA;
    LC_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, stream()));
    LC_CUDA(cudaStreamSynchronize(stream()));
    return LC_OK;
}
int32_t lc_dev_sync(void) {
    if (!have_device()) return LC_ERR_CUDA;
    LC_CUDA(cudaStreamSynchronize(stream()));
    return LC_OK;
}

int32_t lc_timer_begin(void) {
    if (!have_device()) return LC_ERR_CUDA;
    int dev = 0;
    LC_CUDA(cudaGetDevice(&dev));
    if (!g_ev0[dev]) {
        LC_CUDA(cudaEventCreate(&g_ev0[dev]));
        LC_CUDA(cudaEventCreate(&g_ev1[dev]));
    }
    LC_CUDA(cudaEventRecord(g_ev0[dev], stream()));
    return LC_OK;
}
int32_t lc_timer_end(float* out_ms) {
    LC_CHECK(out_ms != nullptr, LC_ERR_INVALID, "lc_timer_end: null output");
    if (!have_device()) return LC_ERR_CUDA;
    int dev = 0;
    LC_CUDA(cudaGetDevice(&dev));
    LC_CHECK(g_ev0[dev] != nullptr, LC_ERR_STATE, "lc_timer_end without lc_timer_begin");
    LC_CUDA(cudaEventRecord(g_ev1[dev], stream()));
    LC_CUDA(cudaEventSynchronize(g_ev1[dev]));
    LC_CUDA(cudaEventElapsedTime(out_ms, g_ev0[dev], g_ev1[dev]));
    return LC_OK;
}

int32_t lc_flush_l2(void) {
    if (!have_device()) return LC_ERR_CUDA;
    int dev = 0;
    LC_CUDA(cudaGetDevice(&dev));
    const size_t bytes = (size_t)256 << 20;  // twice the 126 MB L2
    LC_TRY(g_flush[dev].reserve(bytes));
    static uint32_t tick = 0;
    lc_fill_kernel<<<sm_count() * 4, 256, 0, stream()>>>((uint4*)g_flush[dev].p, bytes / 16, ++tick);
    LC_CUDA(cudaGetLastError());
    return LC_OK;
}

}  // extern "C"

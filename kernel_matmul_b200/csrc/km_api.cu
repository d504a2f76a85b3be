// Library-wide pieces of the C ABI: error reporting, batch validation, the entry counter and
// the FP32-pipe calibration kernel.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "km_tcgen05.cuh"

namespace km {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t err, const char *what) {
    set_error("%s: CUDA error %d (%s)", what, (int)err, cudaGetErrorString(err));
    return KM_ERR_CUDA;
}

int make_batch(const km_batch *in, Batch *out) {
    KM_REQUIRE(in->ndim >= 0 && in->ndim <= KM_MAX_BATCH_DIMS, KM_ERR_INVALID_ARGUMENT,
               "batch rank %d not in [0, %d]", in->ndim, KM_MAX_BATCH_DIMS);
    out->ndim = in->ndim;
    out->count = 1;
    for (int d = 0; d < KM_MAX_BATCH_DIMS; d++) {
        out->size[d] = d < in->ndim ? in->size[d] : 1;
        KM_REQUIRE(out->size[d] >= 0, KM_ERR_INVALID_ARGUMENT, "negative batch size");
        // the product of the sizes must stay far inside int64: every launcher multiplies it by row
        // blocks and record sizes
        KM_REQUIRE(out->size[d] == 0 || out->count <= (int64_t)KM_MAX_BATCH_COUNT / out->size[d], KM_ERR_UNSUPPORTED,
                   "batch of more than %lld kernels", (long long)KM_MAX_BATCH_COUNT);
        out->count *= out->size[d];
    }
    return KM_OK;
}

static std::atomic<unsigned> g_wait_polls{TC_WAIT_POLLS};

unsigned current_wait_polls() { return g_wait_polls.load(std::memory_order_relaxed); }

// One CTA of one warp waits, with the given poll limit, on an mbarrier that nobody arrives at and
// records whether the wait gave up: the hand-off failure of the tensor-core kernels in isolation.
__global__ void selftest_wait_kernel(unsigned polls, int *status) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const bool ok = mbar_wait_warp(&bar, 0u, polls);
    if (threadIdx.x == 0) *status = ok ? 0 : 1;
}

__global__ void count_entries_kernel(Batch batch, int64_t m, int n, int64_t row_blocks,
                                     View<const int> start, View<const int> end,
                                     unsigned long long *count) {
    const int64_t total = batch.count * row_blocks;
    unsigned long long local = 0;
    for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < total;
         w += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = w / row_blocks, r = w % row_blocks;
        const BatchIndex bi = decompose(batch, b);
        const int lo = clamp_int(batch_ptr(start, bi)[r * start.s0], 0, n);
        const int hi = max(lo, min(batch_ptr(end, bi)[r * end.s0], n));
        const int64_t rows = min((r + 1) * (int64_t)KM_BLOCK_SIZE, m) - r * KM_BLOCK_SIZE;
        local += (unsigned long long)(rows * (hi - lo));
    }
    for (int o = 16; o > 0; o >>= 1) local += __shfl_down_sync(0xffffffffu, local, o);
    if ((threadIdx.x & 31) == 0 && local) atomicAdd(count, local);
}

// 64 independent FMA chains per thread: measures the FP32 FMA issue rate of the SMs.
__global__ void __launch_bounds__(256) fp32_peak_kernel(int64_t iters, float *sink) {
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; i++) acc[i] = (float)(threadIdx.x + i) * 1e-3f;
    const float a = 0.999f + 1e-7f * (float)blockIdx.x, b = 1e-4f;
    for (int64_t it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 64; i++) acc[i] = fmaf(acc[i], a, b);
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 64; i++) s += acc[i];
    if (sink != nullptr && s == 123.456f) *sink = s;
}

// 8 independent chains of SFU exponentials per thread: measures the special-function rate.
__global__ void __launch_bounds__(512) sfu_peak_kernel(int64_t iters, float *sink) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = (float)(threadIdx.x + i) * 1e-3f;
    for (int64_t it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = ex2_approx(v[i]);
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) s += v[i];
    if (sink != nullptr && s == 123.456f) *sink = s;
}

}  // namespace km

extern "C" const char *km_last_error(void) { return km::g_error; }

extern "C" int km_num_params(int kernel_type) {
    return km::valid_kernel_type(kernel_type) ? km::num_params(kernel_type) : -1;
}

extern "C" const char *km_version(void) { return "km_b200 0.1 (sm_100a)"; }

extern "C" int km_count_entries(const km_batch *batch, int64_t m, int64_t n, const km_view *start,
                                const km_view *end, int64_t *count, void *stream) {
    using namespace km;
    KM_REQUIRE(batch && start && end && count, KM_ERR_INVALID_ARGUMENT, "km_count_entries: null argument");
    Batch b;
    int rc = make_batch(batch, &b);
    if (rc != KM_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemsetAsync(count, 0, sizeof(int64_t), s);
    if (err != cudaSuccess) return cuda_fail(err, "km_count_entries memset");
    const int64_t rb = ceil_div(m, KM_BLOCK_SIZE);
    if (b.count * rb == 0) return KM_OK;
    const int blocks = (int)std::min<int64_t>(ceil_div(b.count * rb, 256), 1184);
    count_entries_kernel<<<blocks, 256, 0, s>>>(b, m, (int)n, rb, make_view<const int>(start, b),
                                                make_view<const int>(end, b),
                                                reinterpret_cast<unsigned long long *>(count));
    KM_CHECK_LAUNCH("km_count_entries launch");
    return KM_OK;
}

extern "C" int km_probe_fp32_peak(int64_t iters, float *sink, double *flops_out, void *stream) {
    using namespace km;
    KM_REQUIRE(iters > 0 && iters <= KM_PROBE_MAX_ITERS, KM_ERR_INVALID_ARGUMENT,
               "km_probe_fp32_peak: iters must be in [1, %lld]", (long long)KM_PROBE_MAX_ITERS);
    int dev = 0, sms = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return cuda_fail(err, "cudaGetDevice");
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return cuda_fail(err, "cudaDeviceGetAttribute");
    const int blocks = sms * 4, threads = 256;
    fp32_peak_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(iters, sink);
    KM_CHECK_LAUNCH("km_probe_fp32_peak launch");
    if (flops_out) *flops_out = 2.0 * (double)blocks * threads * (double)iters * 64.0;
    return KM_OK;
}

extern "C" int km_probe_sfu_peak(int64_t iters, float *sink, double *ops_out, void *stream) {
    using namespace km;
    KM_REQUIRE(iters > 0 && iters <= KM_PROBE_MAX_ITERS, KM_ERR_INVALID_ARGUMENT,
               "km_probe_sfu_peak: iters must be in [1, %lld]", (long long)KM_PROBE_MAX_ITERS);
    int dev = 0, sms = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return cuda_fail(err, "cudaGetDevice");
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return cuda_fail(err, "cudaDeviceGetAttribute");
    const int blocks = sms * 2, threads = 512;
    sfu_peak_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(iters, sink);
    KM_CHECK_LAUNCH("km_probe_sfu_peak launch");
    if (ops_out) *ops_out = (double)blocks * threads * (double)iters * 8.0;
    return KM_OK;
}

extern "C" int km_selftest_set_wait_polls(int64_t polls) {
    using namespace km;
    KM_REQUIRE(polls >= -1 && polls <= (int64_t)TC_WAIT_POLLS, KM_ERR_INVALID_ARGUMENT,
               "km_selftest_set_wait_polls: polls must be -1 (default) or in [0, %u]", TC_WAIT_POLLS);
    g_wait_polls.store(polls < 0 ? TC_WAIT_POLLS : (unsigned)polls, std::memory_order_relaxed);
    return KM_OK;
}

extern "C" int km_selftest_bounded_wait(int64_t polls, int32_t *status, void *stream) {
    using namespace km;
    KM_REQUIRE(status != nullptr, KM_ERR_INVALID_ARGUMENT, "km_selftest_bounded_wait: null status pointer");
    KM_REQUIRE(polls >= 0 && polls <= 1 << 16, KM_ERR_INVALID_ARGUMENT,
               "km_selftest_bounded_wait: polls must be in [0, 65536]");
    selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>((unsigned)polls, status);
    KM_CHECK_LAUNCH("km_selftest_bounded_wait launch");
    return KM_OK;
}

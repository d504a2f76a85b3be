// Hyper-parameter gradients of the banded product:
//   grad[b, q] = d/d theta_q  sum_{i, j in band, c} left[b,i,c] * kappa(x1[b,i], x2[b,j]) * right[b,j,c]
// One kernel serves the reference's matmul_bwd (left = out_grad, right = rhs;
// native/matmul_bwd/matmul_bwd.cu:12-221) and bilinear_derivative
// (native/bilinear_derivative/bilinear_derivative.cu:12-183).
//
// Same band walk as the forward product (one CTA per 128-row block and batch, tiles of x2 /
// right staged with cp.async).  Each thread keeps the `left` values of its RPT rows in
// registers for the whole band; per staged column it forms the coefficient
// coeff = <left[i, :], right[j, :]> (KB FMAs per entry), evaluates the factors of d kappa / d p
// once per entry and adds coeff * factor to NSUMS running sums -- k + ~10 FP32 operations per
// entry where the reference's matmul_bwd spends P * k (matmul_bwd.cu:157-166).  Sums are
// reduced warp-shuffle -> shared memory -> one partial per (batch, row block) in the
// workspace; a second small kernel adds the partials of a batch in a fixed order in fp64 and
// applies the chain rule theta <- p, so results are deterministic.
#include <mutex>

#include "km_common.cuh"

namespace km {

struct GradArgs {
    Batch batch;
    int64_t m, n, k;
    int64_t row_blocks;
    View<const float> x1, x2, left, right, params;
    View<const int> start, end;
    View<float> grad;
    float *partials;  // [batch.count][row_blocks][KM_MAX_PARAMS]
    int right_vec_ok;
};

template <int KT, int KB, int RPT, int WN>
__global__ void __launch_bounds__(32 * (128 / (32 * RPT)) * WN)
    grad_band_kernel(const GradArgs a) {
    constexpr int WM = 128 / (32 * RPT);
    constexpr int WARPS = WM * WN;
    constexpr int THREADS = 32 * WARPS;
    constexpr int STAGE_FLOATS = TILE_N * KB + TILE_N;
    constexpr int NS = KernelFn<KT>::NSUMS;

    extern __shared__ __align__(16) float smem[];
    __shared__ float warp_sums[WARPS][KM_MAX_PARAMS];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int wm = warp % WM;
    const int wn = warp / WM;

    int64_t item = blockIdx.x;
    const int64_t b = item % a.batch.count;
    const int64_t r = item / a.batch.count;

    const BatchIndex bi = decompose(a.batch, b);
    const float *x1 = batch_ptr(a.x1, bi);
    const float *x2 = batch_ptr(a.x2, bi);
    const float *left = batch_ptr(a.left, bi);
    const float *right = batch_ptr(a.right, bi);

    KernelFn<KT> fn;
    fn.init(batch_ptr(a.params, bi), a.params.s0);

    const int n = (int)a.n;
    const int band_lo = clamp_int(batch_ptr(a.start, bi)[r * a.start.s0], 0, n);
    const int band_hi = max(band_lo, min(batch_ptr(a.end, bi)[r * a.end.s0], n));
    const int tiles = (band_hi - band_lo + TILE_N - 1) / TILE_N;

    float x1r[RPT];
    const int64_t row_base = r * KM_BLOCK_SIZE + wm * (32 * RPT) + lane;
#pragma unroll
    for (int i = 0; i < RPT; i++) {
        const int64_t row = row_base + 32 * i;
        x1r[i] = row < a.m ? x1[row * a.x1.s0] : 0.0f;
    }

    float sums[NS];
#pragma unroll
    for (int q = 0; q < NS; q++) sums[q] = 0.0f;

    for (int64_t k0 = 0; k0 < a.k; k0 += KB) {
        // left values of this thread's rows for this block of columns (zero for masked rows /
        // columns, which makes their coefficients vanish)
        constexpr bool PACKED = (KB % 2 == 0);
        constexpr int KB2 = PACKED ? KB / 2 : 1;
        float lv[RPT][KB];
        f32x2 lv2[RPT][KB2];
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            const int64_t row = row_base + 32 * i;
#pragma unroll
            for (int c = 0; c < KB; c++)
                lv[i][c] = (row < a.m && k0 + c < a.k) ? left[row * a.left.s0 + (k0 + c) * a.left.s1] : 0.0f;
            if constexpr (PACKED) {
#pragma unroll
                for (int c = 0; c < KB2; c++) lv2[i][c] = pack2(lv[i][2 * c], lv[i][2 * c + 1]);
            }
        }
        const bool vec = (KB % 4 == 0) && a.right_vec_ok && (k0 + KB <= a.k);

        auto stage_tile = [&](int buf, int n0) {
            float *rs = smem + buf * STAGE_FLOATS;
            stage_band_tile<KB, THREADS>(rs, rs + TILE_N * KB, x2, a.x2.s0, right, a.right.s0, a.right.s1, k0,
                                         a.k, n0, min(TILE_N, band_hi - n0), vec, tid);
        };

        if (tiles > 0) {
            stage_tile(0, band_lo);
            cp_async_commit();
        }
        for (int t = 0; t < tiles; t++) {
            const int n0 = band_lo + t * TILE_N;
            if (t + 1 < tiles) {
                stage_tile((t + 1) & 1, n0 + TILE_N);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            const float *rs = smem + (t & 1) * STAGE_FLOATS;
            const float *xs = rs + TILE_N * KB;
            const int cnt = min(TILE_N, band_hi - n0);
#pragma unroll 2
            for (int j = wn; j < cnt; j += WN) {
                const float xj = xs[j];
                if constexpr (PACKED) {
                    // even / odd columns accumulate in the two halves of one packed register
                    f32x2 rv2[KB2];
                    load_staged_row2<KB>(rs, j, rv2);
#pragma unroll
                    for (int i = 0; i < RPT; i++) {
                        f32x2 c2 = 0ull;
#pragma unroll
                        for (int c = 0; c < KB2; c++) c2 = fma2(lv2[i][c], rv2[c], c2);
                        float ce, co;
                        unpack2(c2, ce, co);
                        fn.accumulate(x1r[i] - xj, ce + co, sums);
                    }
                } else {
                    float rv[KB];
                    load_staged_row<KB>(rs, j, rv);
#pragma unroll
                    for (int i = 0; i < RPT; i++) {
                        float coeff = 0.0f;
#pragma unroll
                        for (int c = 0; c < KB; c++) coeff = fmaf(lv[i][c], rv[c], coeff);
                        fn.accumulate(x1r[i] - xj, coeff, sums);
                    }
                }
            }
            __syncthreads();
        }
    }

    // CTA reduction of the NS running sums
#pragma unroll
    for (int q = 0; q < NS; q++) {
        float v = sums[q];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) warp_sums[warp][q] = v;
    }
    __syncthreads();
    if (tid < KM_MAX_PARAMS) {
        float v = 0.0f;
        if (tid < NS) {
#pragma unroll
            for (int w = 0; w < WARPS; w++) v += warp_sums[w][tid];
        }
        a.partials[(b * a.row_blocks + r) * KM_MAX_PARAMS + tid] = v;
    }
}

// grad[b, :] = chain rule applied to the fixed-order fp64 sum of the partials of batch b.
// `units` partial records of KM_MAX_PARAMS values (float or double) per batch.
template <int KT, typename PT>
__global__ void __launch_bounds__(256) grad_finish_kernel(Batch batch, int64_t units, const PT *partials,
                                                          View<const float> params, View<float> grad) {
    constexpr int NS = KernelFn<KT>::NSUMS;
    __shared__ double red[256][KM_MAX_PARAMS];
    const int64_t b = blockIdx.x;
    const PT *p = partials + b * units * KM_MAX_PARAMS;
    double local[KM_MAX_PARAMS] = {0.0, 0.0, 0.0, 0.0};
    for (int64_t u = threadIdx.x; u < units; u += 256) {
#pragma unroll
        for (int q = 0; q < KM_MAX_PARAMS; q++) local[q] += (double)p[u * KM_MAX_PARAMS + q];
    }
#pragma unroll
    for (int q = 0; q < KM_MAX_PARAMS; q++) red[threadIdx.x][q] = local[q];
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) {
#pragma unroll
            for (int q = 0; q < KM_MAX_PARAMS; q++) red[threadIdx.x][q] += red[threadIdx.x + s][q];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const BatchIndex bi = decompose(batch, b);
        KernelFn<KT> fn;
        fn.init(batch_ptr(params, bi), params.s0);
        double sums[KM_MAX_PARAMS];
#pragma unroll
        for (int q = 0; q < KM_MAX_PARAMS; q++) sums[q] = q < NS ? red[0][q] : 0.0;
        float g[KM_MAX_PARAMS];
        fn.finish_grad(sums, g);
        float *out = batch_ptr(grad, bi);
#pragma unroll
        for (int q = 0; q < KernelFn<KT>::P; q++) out[q * grad.s0] = g[q];
    }
}

template <typename PT>
static void launch_finish_typed(int kernel_type, const Batch &batch, int64_t units, const PT *partials,
                                const View<const float> &params, const View<float> &grad, cudaStream_t stream) {
    const unsigned blocks = (unsigned)batch.count;
    switch (kernel_type) {
    case KM_KERNEL_RBF:
        grad_finish_kernel<KM_KERNEL_RBF, PT><<<blocks, 256, 0, stream>>>(batch, units, partials, params, grad);
        break;
    case KM_KERNEL_SPECTRAL:
        grad_finish_kernel<KM_KERNEL_SPECTRAL, PT><<<blocks, 256, 0, stream>>>(batch, units, partials, params, grad);
        break;
    default:
        grad_finish_kernel<KM_KERNEL_LOCALLY_PERIODIC, PT><<<blocks, 256, 0, stream>>>(batch, units, partials, params, grad);
        break;
    }
}

int launch_grad_finish(int kernel_type, const Batch &batch, int64_t units, const void *partials,
                       bool partials_fp64, const View<const float> &params, const View<float> &grad,
                       cudaStream_t stream) {
    if (batch.count == 0) return KM_OK;
    if (batch.count > 0x7fffffffLL) {
        set_error("too many batches (%lld)", (long long)batch.count);
        return KM_ERR_UNSUPPORTED;
    }
    if (partials_fp64)
        launch_finish_typed(kernel_type, batch, units, static_cast<const double *>(partials), params, grad, stream);
    else
        launch_finish_typed(kernel_type, batch, units, static_cast<const float *>(partials), params, grad, stream);
    KM_CHECK_LAUNCH("gradient finish launch");
    return KM_OK;
}

template <int KT, int KB, int RPT, int WN>
static int launch_grad(const GradArgs &a, cudaStream_t stream) {
    constexpr int WM = 128 / (32 * RPT);
    constexpr int THREADS = 32 * WM * WN;
    constexpr size_t smem = 2 * (TILE_N * KB + TILE_N) * sizeof(float);
    const int64_t items = a.batch.count * a.row_blocks;
    if (items > 0x7fffffffLL) {
        set_error("gradient: too many work items (%lld)", (long long)items);
        return KM_ERR_UNSUPPORTED;
    }
    grad_band_kernel<KT, KB, RPT, WN><<<(unsigned)items, THREADS, smem, stream>>>(a);
    KM_CHECK_LAUNCH("gradient band launch");
    return KM_OK;
}

template <int KT>
static int dispatch_grad(const GradArgs &a, cudaStream_t stream) {
    const int64_t k = a.k;
    if (k <= 1) return launch_grad<KT, 1, 4, 4>(a, stream);
    if (k <= 2) return launch_grad<KT, 2, 4, 4>(a, stream);
    if (k <= 4) return launch_grad<KT, 4, 4, 4>(a, stream);
    if (k <= 8) return launch_grad<KT, 8, 4, 4>(a, stream);
    if (k <= 16) return launch_grad<KT, 16, 4, 4>(a, stream);
    return launch_grad<KT, 32, 2, 2>(a, stream);
}

static int grad_entry(const char *name, int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                      const km_view *x1, const km_view *x2, const km_view *left, const km_view *right,
                      const km_view *params, const km_view *start, const km_view *end, const km_view *grad,
                      void *workspace, size_t workspace_bytes, void *stream) {
    KM_REQUIRE(valid_kernel_type(kernel_type), KM_ERR_INVALID_ARGUMENT, "%s: unknown kernel type %d", name, kernel_type);
    KM_REQUIRE(batch && x1 && x2 && left && right && params && start && end && grad, KM_ERR_INVALID_ARGUMENT,
               "%s: null argument", name);
    KM_REQUIRE(m >= 0 && n >= 0 && k >= 0 && n <= 0x7fffffffLL, KM_ERR_INVALID_ARGUMENT, "%s: bad sizes", name);
    GradArgs a;
    int rc = make_batch(batch, &a.batch);
    if (rc != KM_OK) return rc;
    if (a.batch.count == 0) return KM_OK;
    KM_REQUIRE(params->data && grad->data, KM_ERR_INVALID_ARGUMENT, "%s: null data pointer", name);
    const size_t need = km_grad_workspace_bytes(kernel_type, batch, m);
    KM_REQUIRE(workspace_bytes >= need && (need == 0 || workspace != nullptr), KM_ERR_WORKSPACE,
               "%s: workspace of %zu bytes needed, %zu given", name, need, workspace_bytes);
    KM_REQUIRE((uintptr_t)workspace % 16 == 0, KM_ERR_WORKSPACE, "%s: workspace must be 16-byte aligned", name);
    a.m = m;
    a.n = n;
    a.k = k;
    a.row_blocks = ceil_div(m, KM_BLOCK_SIZE);
    a.x1 = make_view<const float>(x1, a.batch);
    a.x2 = make_view<const float>(x2, a.batch);
    a.left = make_view<const float>(left, a.batch);
    a.right = make_view<const float>(right, a.batch);
    a.params = make_view<const float>(params, a.batch);
    a.start = make_view<const int>(start, a.batch);
    a.end = make_view<const int>(end, a.batch);
    a.grad = make_view<float>(grad, a.batch);
    a.partials = static_cast<float *>(workspace);
    a.right_vec_ok = rows_vectorizable(a.right, a.batch) ? 1 : 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (a.row_blocks > 0) {
        KM_REQUIRE(x1->data && left->data && start->data && end->data, KM_ERR_INVALID_ARGUMENT,
                   "%s: null data pointer", name);
        switch (kernel_type) {
        case KM_KERNEL_RBF: rc = dispatch_grad<KM_KERNEL_RBF>(a, s); break;
        case KM_KERNEL_SPECTRAL: rc = dispatch_grad<KM_KERNEL_SPECTRAL>(a, s); break;
        default: rc = dispatch_grad<KM_KERNEL_LOCALLY_PERIODIC>(a, s); break;
        }
        if (rc != KM_OK) return rc;
    }
    return launch_grad_finish(kernel_type, a.batch, a.row_blocks, a.partials, false, a.params, a.grad, s);
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant: the partial sums live in a fixed array inside the library image.
// ---------------------------------------------------------------------------------------

// One record of KM_MAX_PARAMS floats per (batch, row block).  Lives in every CUDA context
// that loads the library, for the lifetime of that context.
static __device__ __align__(256) float g_static_partials[KM_STATIC_GRAD_UNITS * KM_MAX_PARAMS];

static std::mutex g_static_mutex;
static void *g_static_ptr[KM_STATIC_MAX_DEVICES] = {nullptr};

// Device address of g_static_partials on the current device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use, so it is translated with
// cudaGetSymbolAddress once per device (with that device current) and remembered.
static int static_partials_address(void **out) {
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return cuda_fail(err, "km_bilinear_derivative_static_f32: cudaGetDevice");
    KM_REQUIRE(dev >= 0 && dev < KM_STATIC_MAX_DEVICES, KM_ERR_UNSUPPORTED,
               "km_bilinear_derivative_static_f32: device ordinal %d not below %d", dev, KM_STATIC_MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_ptr[dev] == nullptr) {
        void *p = nullptr;
        err = cudaGetSymbolAddress(&p, g_static_partials);
        if (err != cudaSuccess) return cuda_fail(err, "km_bilinear_derivative_static_f32: cudaGetSymbolAddress");
        KM_REQUIRE(p != nullptr, KM_ERR_CUDA, "km_bilinear_derivative_static_f32: null symbol address");
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return KM_OK;
}

}  // namespace km

extern "C" int km_bilinear_derivative_static_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n,
                                                 int64_t k, const km_view *x1, const km_view *x2,
                                                 const km_view *left, const km_view *right,
                                                 const km_view *params, const km_view *start,
                                                 const km_view *end, const km_view *grad, void *stream) {
    using namespace km;
    KM_REQUIRE(batch != nullptr && m >= 0, KM_ERR_INVALID_ARGUMENT, "km_bilinear_derivative_static_f32: bad arguments");
    Batch b;
    int rc = make_batch(batch, &b);
    if (rc != KM_OK) return rc;
    const int64_t units = b.count * ceil_div(m, KM_BLOCK_SIZE);
    KM_REQUIRE(units <= (int64_t)KM_STATIC_GRAD_UNITS, KM_ERR_UNSUPPORTED,
               "km_bilinear_derivative_static_f32: batch count x row blocks = %lld exceeds the built-in scratch of "
               "%d records; use km_bilinear_derivative_f32 with a caller-provided workspace",
               (long long)units, KM_STATIC_GRAD_UNITS);
    void *scratch = nullptr;
    rc = static_partials_address(&scratch);
    if (rc != KM_OK) return rc;
    return grad_entry("km_bilinear_derivative_static_f32", kernel_type, batch, m, n, k, x1, x2, left, right, params,
                      start, end, grad, scratch, sizeof(float) * KM_STATIC_GRAD_UNITS * KM_MAX_PARAMS, stream);
}

extern "C" size_t km_grad_workspace_bytes(int kernel_type, const km_batch *batch, int64_t m) {
    (void)kernel_type;
    km::Batch b;
    if (batch == nullptr || km::make_batch(batch, &b) != KM_OK || m < 0) return 0;
    return (size_t)(b.count * km::ceil_div(m, KM_BLOCK_SIZE)) * KM_MAX_PARAMS * sizeof(float);
}

extern "C" int km_bilinear_derivative_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                                          const km_view *x1, const km_view *x2, const km_view *left,
                                          const km_view *right, const km_view *params, const km_view *start,
                                          const km_view *end, const km_view *grad, void *workspace,
                                          size_t workspace_bytes, void *stream) {
    return km::grad_entry("km_bilinear_derivative_f32", kernel_type, batch, m, n, k, x1, x2, left, right, params,
                          start, end, grad, workspace, workspace_bytes, stream);
}

extern "C" int km_matmul_bwd_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                                 const km_view *x1, const km_view *x2, const km_view *rhs, const km_view *params,
                                 const km_view *start, const km_view *end, const km_view *out_grad,
                                 const km_view *grad, void *workspace, size_t workspace_bytes, void *stream) {
    return km::grad_entry("km_matmul_bwd_f32", kernel_type, batch, m, n, k, x1, x2, out_grad, rhs, params, start,
                          end, grad, workspace, workspace_bytes, stream);
}

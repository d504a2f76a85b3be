// Materialise the masked kernel matrix (dense) and its hyper-parameter gradient (dense_bwd).
//
// dense: HBM-write bound.  One CTA writes a 128-row x 512-column tile of out; threads run
// along the columns so that every row is written as one contiguous 2 KB segment (128-bit
// stores when the rows are 16-byte aligned), and tiles outside the band are written as zeros
// by the same kernel -- no separate zero fill.  The reference stores with threadIdx.x along
// the ROW dimension (stride-n writes) after a full torch::zeros pass
// (native/dense/dense.cu:12-98).
//
// dense_bwd: HBM-read bound on the band part of out_grad.  One CTA per (batch, row block)
// walks the band in 256-column tiles, thread = column, rows streamed; partial sums go through
// the same fixed-order fp64 finish as the other gradient ops (native/dense_bwd/dense_bwd.cu:12-116).
#include "km_common.cuh"

namespace km {

struct DenseArgs {
    Batch batch;
    int64_t m, n;
    int64_t row_blocks, col_tiles;
    View<const float> x1, x2, params;
    View<const int> start, end;
    View<float> out;
};

constexpr int DENSE_TILE_COLS = 512;

template <int KT, bool VEC>
__global__ void __launch_bounds__(256) dense_kernel(const DenseArgs a) {
    __shared__ float x1s[KM_BLOCK_SIZE];

    int64_t item = blockIdx.x;
    const int64_t ct = item % a.col_tiles;
    item /= a.col_tiles;
    const int64_t r = item % a.row_blocks;
    const int64_t b = item / a.row_blocks;

    const BatchIndex bi = decompose(a.batch, b);
    const float *x1 = batch_ptr(a.x1, bi);
    const float *x2 = batch_ptr(a.x2, bi);
    float *out = batch_ptr(a.out, bi);
    KernelFn<KT> fn;
    fn.init(batch_ptr(a.params, bi), a.params.s0);

    const int n = (int)a.n;
    const int band_lo = clamp_int(batch_ptr(a.start, bi)[r * a.start.s0], 0, n);
    const int band_hi = max(band_lo, min(batch_ptr(a.end, bi)[r * a.end.s0], n));

    const int tid = threadIdx.x;
    const int64_t row0 = r * KM_BLOCK_SIZE;
    const int rows = (int)min((int64_t)KM_BLOCK_SIZE, a.m - row0);
    if (tid < KM_BLOCK_SIZE) x1s[tid] = tid < rows ? x1[(row0 + tid) * a.x1.s0] : 0.0f;

    const int col0 = (int)(ct * DENSE_TILE_COLS);
    const int colgroup = tid & 127;  // 128 threads cover the 512 columns of the tile
    const int rowgroup = tid >> 7;   // two row groups take alternate rows

    int cols[4];
    float xj[4];
    bool inband[4];
    bool any = false;
#pragma unroll
    for (int q = 0; q < 4; q++) {
        cols[q] = VEC ? col0 + colgroup * 4 + q : col0 + colgroup + 128 * q;
        inband[q] = cols[q] >= band_lo && cols[q] < band_hi;
        xj[q] = inband[q] ? x2[(int64_t)cols[q] * a.x2.s0] : 0.0f;
        any = any || inband[q];
    }
    __syncthreads();

    const float scale = fn.scale;
    for (int i = rowgroup; i < rows; i += 2) {
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (any) {
            const float xi = x1s[i];
#pragma unroll
            for (int q = 0; q < 4; q++)
                if (inband[q]) v[q] = scale * fn.unscaled(xi - xj[q]);
        }
        float *orow = out + (row0 + i) * a.out.s0;
        if (VEC) {
            if (cols[3] < n) {
                *reinterpret_cast<float4 *>(orow + cols[0]) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
#pragma unroll
                for (int q = 0; q < 4; q++)
                    if (cols[q] < n) orow[cols[q]] = v[q];
            }
        } else {
#pragma unroll
            for (int q = 0; q < 4; q++)
                if (cols[q] < n) orow[(int64_t)cols[q] * a.out.s1] = v[q];
        }
    }
}

struct DenseBwdArgs {
    Batch batch;
    int64_t m, n;
    int64_t row_blocks;
    View<const float> x1, x2, params, out_grad;
    View<const int> start, end;
    float *partials;
};

template <int KT>
__global__ void __launch_bounds__(256) dense_bwd_kernel(const DenseBwdArgs a) {
    constexpr int NS = KernelFn<KT>::NSUMS;
    __shared__ float x1s[KM_BLOCK_SIZE];
    __shared__ float warp_sums[8][KM_MAX_PARAMS];

    const int64_t b = blockIdx.x % a.batch.count;
    const int64_t r = blockIdx.x / a.batch.count;
    const BatchIndex bi = decompose(a.batch, b);
    const float *x1 = batch_ptr(a.x1, bi);
    const float *x2 = batch_ptr(a.x2, bi);
    const float *og = batch_ptr(a.out_grad, bi);
    KernelFn<KT> fn;
    fn.init(batch_ptr(a.params, bi), a.params.s0);

    const int n = (int)a.n;
    const int band_lo = clamp_int(batch_ptr(a.start, bi)[r * a.start.s0], 0, n);
    const int band_hi = max(band_lo, min(batch_ptr(a.end, bi)[r * a.end.s0], n));

    const int tid = threadIdx.x;
    const int64_t row0 = r * KM_BLOCK_SIZE;
    const int rows = (int)min((int64_t)KM_BLOCK_SIZE, a.m - row0);
    if (tid < KM_BLOCK_SIZE) x1s[tid] = tid < rows ? x1[(row0 + tid) * a.x1.s0] : 0.0f;
    __syncthreads();

    float sums[NS];
#pragma unroll
    for (int q = 0; q < NS; q++) sums[q] = 0.0f;

    for (int c = band_lo + tid; c < band_hi; c += 256) {
        const float xj = x2[(int64_t)c * a.x2.s0];
        const float *ocol = og + row0 * a.out_grad.s0 + (int64_t)c * a.out_grad.s1;
        int i = 0;
        for (; i + 8 <= rows; i += 8) {
            float g[8];
#pragma unroll
            for (int u = 0; u < 8; u++) g[u] = ocol[(int64_t)(i + u) * a.out_grad.s0];
#pragma unroll
            for (int u = 0; u < 8; u++) fn.accumulate(x1s[i + u] - xj, g[u], sums);
        }
        for (; i < rows; i++) fn.accumulate(x1s[i] - xj, ocol[(int64_t)i * a.out_grad.s0], sums);
    }

    const int lane = tid & 31, warp = tid >> 5;
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
            for (int w = 0; w < 8; w++) v += warp_sums[w][tid];
        }
        a.partials[(b * a.row_blocks + r) * KM_MAX_PARAMS + tid] = v;
    }
}

template <int KT>
static int launch_dense(const DenseArgs &a, bool vec, cudaStream_t s) {
    const int64_t items = a.batch.count * a.row_blocks * a.col_tiles;
    if (items > 0x7fffffffLL) {
        set_error("km_dense_f32: too many work items (%lld)", (long long)items);
        return KM_ERR_UNSUPPORTED;
    }
    if (vec)
        dense_kernel<KT, true><<<(unsigned)items, 256, 0, s>>>(a);
    else
        dense_kernel<KT, false><<<(unsigned)items, 256, 0, s>>>(a);
    KM_CHECK_LAUNCH("km_dense_f32 launch");
    return KM_OK;
}

}  // namespace km

extern "C" int km_dense_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, const km_view *x1,
                            const km_view *x2, const km_view *params, const km_view *start, const km_view *end,
                            const km_view *out, void *stream) {
    using namespace km;
    KM_REQUIRE(valid_kernel_type(kernel_type), KM_ERR_INVALID_ARGUMENT, "km_dense_f32: unknown kernel type %d", kernel_type);
    KM_REQUIRE(batch && x1 && x2 && params && start && end && out, KM_ERR_INVALID_ARGUMENT, "km_dense_f32: null argument");
    KM_REQUIRE(m >= 0 && n >= 0 && n <= 0x7fffffffLL - 1024, KM_ERR_INVALID_ARGUMENT, "km_dense_f32: bad sizes");
    DenseArgs a;
    int rc = make_batch(batch, &a.batch);
    if (rc != KM_OK) return rc;
    if (a.batch.count == 0 || m == 0 || n == 0) return KM_OK;
    KM_REQUIRE(x1->data && x2->data && params->data && start->data && end->data && out->data,
               KM_ERR_INVALID_ARGUMENT, "km_dense_f32: null data pointer");
    a.m = m;
    a.n = n;
    a.row_blocks = ceil_div(m, KM_BLOCK_SIZE);
    a.col_tiles = ceil_div(n, DENSE_TILE_COLS);
    a.x1 = make_view<const float>(x1, a.batch);
    a.x2 = make_view<const float>(x2, a.batch);
    a.params = make_view<const float>(params, a.batch);
    a.start = make_view<const int>(start, a.batch);
    a.end = make_view<const int>(end, a.batch);
    a.out = make_view<float>(out, a.batch);
    bool vec = a.out.s1 == 1 && a.out.s0 % 4 == 0 && ((uintptr_t)a.out.data % 16 == 0);
    for (int d = 0; d < a.batch.ndim; d++) vec = vec && (a.out.bs[d] % 4 == 0);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (kernel_type) {
    case KM_KERNEL_RBF: return launch_dense<KM_KERNEL_RBF>(a, vec, s);
    case KM_KERNEL_SPECTRAL: return launch_dense<KM_KERNEL_SPECTRAL>(a, vec, s);
    default: return launch_dense<KM_KERNEL_LOCALLY_PERIODIC>(a, vec, s);
    }
}

extern "C" int km_dense_bwd_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, const km_view *x1,
                                const km_view *x2, const km_view *params, const km_view *start,
                                const km_view *end, const km_view *out_grad, const km_view *grad, void *workspace,
                                size_t workspace_bytes, void *stream) {
    using namespace km;
    KM_REQUIRE(valid_kernel_type(kernel_type), KM_ERR_INVALID_ARGUMENT, "km_dense_bwd_f32: unknown kernel type %d", kernel_type);
    KM_REQUIRE(batch && x1 && x2 && params && start && end && out_grad && grad, KM_ERR_INVALID_ARGUMENT,
               "km_dense_bwd_f32: null argument");
    KM_REQUIRE(m >= 0 && n >= 0 && n <= 0x7fffffffLL - 1024, KM_ERR_INVALID_ARGUMENT, "km_dense_bwd_f32: bad sizes");
    DenseBwdArgs a;
    int rc = make_batch(batch, &a.batch);
    if (rc != KM_OK) return rc;
    if (a.batch.count == 0) return KM_OK;
    KM_REQUIRE(params->data && grad->data, KM_ERR_INVALID_ARGUMENT, "km_dense_bwd_f32: null data pointer");
    const size_t need = km_grad_workspace_bytes(kernel_type, batch, m);
    KM_REQUIRE(workspace_bytes >= need && (need == 0 || workspace != nullptr), KM_ERR_WORKSPACE,
               "km_dense_bwd_f32: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    a.m = m;
    a.n = n;
    a.row_blocks = ceil_div(m, KM_BLOCK_SIZE);
    a.x1 = make_view<const float>(x1, a.batch);
    a.x2 = make_view<const float>(x2, a.batch);
    a.params = make_view<const float>(params, a.batch);
    a.out_grad = make_view<const float>(out_grad, a.batch);
    a.start = make_view<const int>(start, a.batch);
    a.end = make_view<const int>(end, a.batch);
    a.partials = static_cast<float *>(workspace);
    const View<float> g = make_view<float>(grad, a.batch);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t items = a.batch.count * a.row_blocks;
    KM_REQUIRE(items <= 0x7fffffffLL, KM_ERR_UNSUPPORTED, "km_dense_bwd_f32: too many work items");
    if (items > 0) {
        KM_REQUIRE(x1->data && start->data && end->data, KM_ERR_INVALID_ARGUMENT, "km_dense_bwd_f32: null data pointer");
        switch (kernel_type) {
        case KM_KERNEL_RBF: dense_bwd_kernel<KM_KERNEL_RBF><<<(unsigned)items, 256, 0, s>>>(a); break;
        case KM_KERNEL_SPECTRAL: dense_bwd_kernel<KM_KERNEL_SPECTRAL><<<(unsigned)items, 256, 0, s>>>(a); break;
        default: dense_bwd_kernel<KM_KERNEL_LOCALLY_PERIODIC><<<(unsigned)items, 256, 0, s>>>(a); break;
        }
        KM_CHECK_LAUNCH("km_dense_bwd_f32 launch");
    }
    return launch_grad_finish(kernel_type, a.batch, a.row_blocks, a.partials, false, a.params, g, s);
}

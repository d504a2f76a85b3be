// Gather single kernel-matrix entries (index) and the gradient of the gather (index_bwd).
//
// index: one lookup per thread, grid-strided; the index streams are read coalesced, x1 / x2 /
// ranges are small and stay in L2.  Out-of-band (and out-of-range) lookups give 0 and every
// output element is written, so no zero fill is needed (reference: zero fill + one 64-thread
// block per 64 lookups, native/index/index.cu:12-101).
//
// index_bwd: every thread accumulates the raw gradient sums of the lookups it visits in
// registers for as long as they belong to one batch, CTAs reduce, and one fp64 atomic per CTA
// and sum lands in a [batch][4] fp64 workspace; the common finish kernel applies the chain
// rule.  The reference writes one slot per lookup and batch into a (B, P, ib, L/64, 64)
// temporary and sums it (native/index_bwd/index_bwd.cu:12-112).
#include "km_common.cuh"

namespace km {

struct IndexArgs {
    Batch batch;
    int64_t m, n, L;
    View<const float> x1, x2, params;
    View<const int> start, end;
    const int32_t *bidx[KM_MAX_BATCH_DIMS];
    const int32_t *row, *col;
    const float *out_grad;
    float *out;
    double *sums;  // index_bwd: [batch.count][KM_MAX_PARAMS]
};

// Resolves lookup l.  Returns false when the lookup is out of range or out of band.
__device__ __forceinline__ bool resolve_lookup(const IndexArgs &a, int64_t l, BatchIndex &bi, int64_t &flat,
                                               float &tau) {
    bool ok = true;
    flat = 0;
#pragma unroll
    for (int d = 0; d < KM_MAX_BATCH_DIMS; d++) {
        if (d < a.batch.ndim) {
            const int64_t v = a.bidx[d][l];
            ok = ok && v >= 0 && v < a.batch.size[d];
            bi.i[d] = v;
            flat = flat * a.batch.size[d] + v;
        } else {
            bi.i[d] = 0;
        }
    }
    const int row = a.row[l], col = a.col[l];
    ok = ok && row >= 0 && row < a.m && col >= 0 && col < a.n;
    if (!ok) return false;
    const int64_t r = row / KM_BLOCK_SIZE;
    const int lo = batch_ptr(a.start, bi)[r * a.start.s0];
    const int hi = batch_ptr(a.end, bi)[r * a.end.s0];
    if (!(lo <= col && col < hi)) return false;
    tau = batch_ptr(a.x1, bi)[(int64_t)row * a.x1.s0] - batch_ptr(a.x2, bi)[(int64_t)col * a.x2.s0];
    return true;
}

template <int KT>
__global__ void __launch_bounds__(256) index_kernel(const IndexArgs a) {
    const bool single = a.batch.count == 1;
    KernelFn<KT> fn;
    if (single) fn.init(a.params.data, a.params.s0);
    for (int64_t l = blockIdx.x * 256LL + threadIdx.x; l < a.L; l += (int64_t)gridDim.x * 256) {
        BatchIndex bi;
        int64_t flat;
        float tau;
        float v = 0.0f;
        if (resolve_lookup(a, l, bi, flat, tau)) {
            if (!single) fn.init(batch_ptr(a.params, bi), a.params.s0);
            v = fn.scale * fn.unscaled(tau);
        }
        a.out[l] = v;
    }
}

template <int KT>
__global__ void __launch_bounds__(256) index_bwd_kernel(const IndexArgs a) {
    constexpr int NS = KernelFn<KT>::NSUMS;
    __shared__ float warp_sums[8][KM_MAX_PARAMS];
    const bool single = a.batch.count == 1;
    KernelFn<KT> fn;
    if (single) fn.init(a.params.data, a.params.s0);

    float sums[NS];
#pragma unroll
    for (int q = 0; q < NS; q++) sums[q] = 0.0f;
    int64_t cur = -1;

    auto flush = [&]() {
        if (cur >= 0) {
#pragma unroll
            for (int q = 0; q < NS; q++) {
                if (sums[q] != 0.0f) atomicAdd(a.sums + cur * KM_MAX_PARAMS + q, (double)sums[q]);
                sums[q] = 0.0f;
            }
        }
    };

    for (int64_t l = blockIdx.x * 256LL + threadIdx.x; l < a.L; l += (int64_t)gridDim.x * 256) {
        BatchIndex bi;
        int64_t flat;
        float tau;
        if (resolve_lookup(a, l, bi, flat, tau)) {
            if (!single) {
                if (flat != cur) {
                    flush();
                    cur = flat;
                    fn.init(batch_ptr(a.params, bi), a.params.s0);
                }
            } else {
                cur = 0;
            }
            fn.accumulate_precise(tau, a.out_grad[l], sums);
        }
    }

    // Several batches: every thread adds what it still holds.  One batch: reduce over the CTA
    // first, then one atomic per sum.
    if (!single) {
        flush();
        return;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int q = 0; q < NS; q++) {
        float v = sums[q];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) warp_sums[warp][q] = v;
    }
    __syncthreads();
    if (threadIdx.x < NS) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; w++) v += warp_sums[w][threadIdx.x];
        if (v != 0.0f) atomicAdd(a.sums + threadIdx.x, (double)v);
    }
}

static int fill_index_args(const char *name, IndexArgs &a, int kernel_type, const km_batch *batch, int64_t m,
                           int64_t n, int64_t L, const km_view *x1, const km_view *x2, const km_view *params,
                           const km_view *start, const km_view *end, const int32_t *const *batch_indices,
                           const int32_t *row, const int32_t *col) {
    KM_REQUIRE(valid_kernel_type(kernel_type), KM_ERR_INVALID_ARGUMENT, "%s: unknown kernel type %d", name, kernel_type);
    KM_REQUIRE(batch && x1 && x2 && params && start && end, KM_ERR_INVALID_ARGUMENT, "%s: null argument", name);
    KM_REQUIRE(m >= 0 && n >= 0 && L >= 0 && n <= 0x7fffffffLL && m <= 0x7fffffffLL, KM_ERR_INVALID_ARGUMENT,
               "%s: bad sizes", name);
    int rc = make_batch(batch, &a.batch);
    if (rc != KM_OK) return rc;
    a.m = m;
    a.n = n;
    a.L = L;
    a.x1 = make_view<const float>(x1, a.batch);
    a.x2 = make_view<const float>(x2, a.batch);
    a.params = make_view<const float>(params, a.batch);
    a.start = make_view<const int>(start, a.batch);
    a.end = make_view<const int>(end, a.batch);
    for (int d = 0; d < KM_MAX_BATCH_DIMS; d++) a.bidx[d] = nullptr;
    if (L > 0) {
        KM_REQUIRE(row && col, KM_ERR_INVALID_ARGUMENT, "%s: null index pointer", name);
        KM_REQUIRE(a.batch.ndim == 0 || batch_indices != nullptr, KM_ERR_INVALID_ARGUMENT, "%s: null batch_indices", name);
        for (int d = 0; d < a.batch.ndim; d++) {
            KM_REQUIRE(batch_indices[d] != nullptr, KM_ERR_INVALID_ARGUMENT, "%s: null batch index array %d", name, d);
            a.bidx[d] = batch_indices[d];
        }
    }
    a.row = row;
    a.col = col;
    a.out_grad = nullptr;
    a.out = nullptr;
    a.sums = nullptr;
    return KM_OK;
}

}  // namespace km

extern "C" int km_index_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t L,
                            const km_view *x1, const km_view *x2, const km_view *params, const km_view *start,
                            const km_view *end, const int32_t *const *batch_indices, const int32_t *row,
                            const int32_t *col, float *out, void *stream) {
    using namespace km;
    IndexArgs a;
    int rc = fill_index_args("km_index_f32", a, kernel_type, batch, m, n, L, x1, x2, params, start, end,
                             batch_indices, row, col);
    if (rc != KM_OK) return rc;
    if (L == 0) return KM_OK;
    KM_REQUIRE(out != nullptr, KM_ERR_INVALID_ARGUMENT, "km_index_f32: null output");
    a.out = out;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(L, 256), 148 * 32);
    switch (kernel_type) {
    case KM_KERNEL_RBF: index_kernel<KM_KERNEL_RBF><<<blocks, 256, 0, s>>>(a); break;
    case KM_KERNEL_SPECTRAL: index_kernel<KM_KERNEL_SPECTRAL><<<blocks, 256, 0, s>>>(a); break;
    default: index_kernel<KM_KERNEL_LOCALLY_PERIODIC><<<blocks, 256, 0, s>>>(a); break;
    }
    KM_CHECK_LAUNCH("km_index_f32 launch");
    return KM_OK;
}

extern "C" size_t km_index_bwd_workspace_bytes(int kernel_type, const km_batch *batch) {
    (void)kernel_type;
    km::Batch b;
    if (batch == nullptr || km::make_batch(batch, &b) != KM_OK) return 0;
    return (size_t)b.count * KM_MAX_PARAMS * sizeof(double);
}

extern "C" int km_index_bwd_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t L,
                                const km_view *x1, const km_view *x2, const km_view *params,
                                const km_view *start, const km_view *end, const int32_t *const *batch_indices,
                                const int32_t *row, const int32_t *col, const float *out_grad,
                                const km_view *grad, void *workspace, size_t workspace_bytes, void *stream) {
    using namespace km;
    IndexArgs a;
    int rc = fill_index_args("km_index_bwd_f32", a, kernel_type, batch, m, n, L, x1, x2, params, start, end,
                             batch_indices, row, col);
    if (rc != KM_OK) return rc;
    KM_REQUIRE(grad != nullptr, KM_ERR_INVALID_ARGUMENT, "km_index_bwd_f32: null argument");
    if (a.batch.count == 0) return KM_OK;
    const size_t need = km_index_bwd_workspace_bytes(kernel_type, batch);
    KM_REQUIRE(workspace_bytes >= need && workspace != nullptr, KM_ERR_WORKSPACE,
               "km_index_bwd_f32: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    KM_REQUIRE(L == 0 || out_grad != nullptr, KM_ERR_INVALID_ARGUMENT, "km_index_bwd_f32: null out_grad");
    a.out_grad = out_grad;
    a.sums = static_cast<double *>(workspace);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemsetAsync(workspace, 0, need, s);
    if (err != cudaSuccess) return cuda_fail(err, "km_index_bwd_f32 memset");
    if (L > 0) {
        const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(L, 256), 148 * 8);
        switch (kernel_type) {
        case KM_KERNEL_RBF: index_bwd_kernel<KM_KERNEL_RBF><<<blocks, 256, 0, s>>>(a); break;
        case KM_KERNEL_SPECTRAL: index_bwd_kernel<KM_KERNEL_SPECTRAL><<<blocks, 256, 0, s>>>(a); break;
        default: index_bwd_kernel<KM_KERNEL_LOCALLY_PERIODIC><<<blocks, 256, 0, s>>>(a); break;
        }
        KM_CHECK_LAUNCH("km_index_bwd_f32 launch");
    }
    return launch_grad_finish(kernel_type, a.batch, 1, a.sums, true, a.params, make_view<float>(grad, a.batch), s);
}

// Band construction on the device: start/end column per 128-row block.
//
// The reference computes these with sequential scans on one CPU thread after copying x to the
// host (native/ranges/ranges.cpp:8-150), which puts a device synchronisation into every kernel
// forward.  Here nothing leaves the device and nothing synchronises.
//
// Parallel formulation.  Every scan of the reference has the form "first grid position
// j >= j0 for which pred_i(j) holds, else n", where the grid is {0, step, 2 step, ..} below n
// and j0 is the result of the previous row block.  When x2 is non-decreasing, pred_i is
// monotone in j (fp32 subtraction and comparison are monotone), so that position is
// max(j0, first_i) with first_i found by binary search over the grid, and the recurrences
// over row blocks turn into prefix maxima:
//   make_ranges:            start[i] = max_{i' <= i} lb_i' ;  end[i] = max(start[i], max_{i' <= i} ub_i')
//   make_ranges_symmetric:  end[i] = max(block, max_{i' <= i} ub_i') ;
//                           start[k] = block * (first i <= k with ceil(end[i] / block) > k), else n
// with every predicate evaluated in fp32 exactly as the reference writes it.  A first kernel
// checks monotonicity per batch row (NaNs count as unsorted); batch rows that fail it are
// processed by a sequential scan kernel that restates the reference loop, so the int32
// results are bit-identical to the reference for every input.
#include "km_common.cuh"

namespace km {

// flags[b] = 1 iff x[b, :] is non-decreasing.  flags must be preset to 1.
// `xs`: elements between batch rows of x (n, or 0 when every batch row shares one x).
__global__ void check_sorted_kernel(int64_t B, int64_t n, const float *x, int64_t xs, int32_t *flags) {
    const int64_t total = B * n;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t j = idx % n, b = idx / n;
        if (j + 1 < n && !(x[b * xs + j] <= x[b * xs + j + 1])) flags[b] = 0;
    }
}

__global__ void fill_flags_kernel(int64_t B, int32_t *flags) {
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < B) flags[i] = 1;
}

// First grid index t in [0, G) with pred(t * step), else G.  pred monotone (false.. true..).
template <typename Pred>
__device__ __forceinline__ int64_t first_true(int64_t G, Pred pred) {
    int64_t lo = 0, hi = G;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (pred(mid)) hi = mid; else lo = mid + 1;
    }
    return lo;
}

// Per (batch, row block): lb (first grid column within cutoff below the block's first row) and
// ub (first grid column beyond cutoff above the block's last row), written to start / end as
// scratch.  mode 0 = make_ranges, mode 1 = symmetric (only ub, predicate with >=).
// `cutoffs` (device, B values) overrides the scalar when not null; x1s / x2s: elements between
// batch rows (0: shared).
__global__ void range_bounds_kernel(int64_t B, int64_t m, int64_t n, int64_t R, const float *x1, int64_t x1s,
                                    const float *x2, int64_t x2s, float cutoff_scalar, const float *cutoffs, int block,
                                    int step, int mode, const int32_t *flags, int32_t *start, int32_t *end) {
    const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (idx >= B * R) return;
    const int64_t b = idx / R, i = idx % R;
    if (!flags[b]) return;
    const float cutoff = cutoffs ? cutoffs[b] : cutoff_scalar;
    const float *a = x1 + b * x1s;
    const float *c = x2 + b * x2s;
    const int64_t G = (n + step - 1) / step;
    const float last = a[min((i + 1) * (int64_t)block, m) - 1];
    if (mode == 0) {
        const float first = a[i * block];
        const int64_t tl = first_true(G, [&](int64_t t) { return first - c[t * step] <= cutoff; });
        const int64_t tu = first_true(G, [&](int64_t t) { return c[t * step] - last > cutoff; });
        start[idx] = (int32_t)min(tl * step, n);
        end[idx] = (int32_t)min(tu * step, n);
    } else {
        const int64_t tu = first_true(G, [&](int64_t t) { return c[t * step] - last >= cutoff; });
        end[idx] = (int32_t)min(tu * step, n);
    }
}

// In-place inclusive prefix maximum over each batch row of `v` (R entries), one CTA per batch;
// optionally a second array `w` becomes max(prefix-max(w), prefix-max(v)) (mode 0: end), or
// v is floored at `floor_value` (mode 1: symmetric end).
__global__ void __launch_bounds__(1024) prefix_max_kernel(int64_t R, const int32_t *flags, int32_t *v, int32_t *w,
                                                           int mode, int floor_value) {
    __shared__ int warp_max_v[32], warp_max_w[32];
    __shared__ int carry_v, carry_w;
    const int64_t b = blockIdx.x;
    if (!flags[b]) return;
    int32_t *pv = v + b * R;
    int32_t *pw = w ? w + b * R : nullptr;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        carry_v = mode == 1 ? floor_value : INT_MIN;
        carry_w = INT_MIN;
    }
    __syncthreads();
    for (int64_t base = 0; base < R; base += 1024) {
        const int64_t i = base + threadIdx.x;
        int xv = i < R ? pv[i] : INT_MIN;
        int xw = (pw && i < R) ? pw[i] : INT_MIN;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int yv = __shfl_up_sync(0xffffffffu, xv, o);
            const int yw = __shfl_up_sync(0xffffffffu, xw, o);
            if (lane >= o) {
                xv = max(xv, yv);
                xw = max(xw, yw);
            }
        }
        if (lane == 31) {
            warp_max_v[warp] = xv;
            warp_max_w[warp] = xw;
        }
        __syncthreads();
        int pre_v = carry_v, pre_w = carry_w;
        for (int q = 0; q < warp; q++) {
            pre_v = max(pre_v, warp_max_v[q]);
            pre_w = max(pre_w, warp_max_w[q]);
        }
        xv = max(xv, pre_v);
        xw = max(xw, pre_w);
        if (i < R) {
            pv[i] = xv;
            if (pw) pw[i] = max(xw, xv);
        }
        __syncthreads();
        if (threadIdx.x == 1023) {
            carry_v = xv;
            carry_w = xw;
        }
        __syncthreads();
    }
}

// Symmetric start from the (non-decreasing) end array.
__global__ void symmetric_start_kernel(int64_t B, int64_t n, int64_t R, int block, const int32_t *flags,
                                       const int32_t *end, int32_t *start) {
    const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (idx >= B * R) return;
    const int64_t b = idx / R, k = idx % R;
    if (!flags[b]) return;
    const int32_t *e = end + b * R;
    // first i in [0, R) with ceil(e[i] / block) > k
    int64_t lo = 0, hi = R;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        const int64_t reach = ((int64_t)e[mid] + block - 1) / block;
        if (reach > k) hi = mid; else lo = mid + 1;
    }
    int32_t s = (lo <= k) ? (int32_t)(lo * block) : (int32_t)n;
    if (k == 0) s = 0;
    start[idx] = s;
}

// Sequential restatement of the reference scans for batch rows whose x2 is not sorted
// (native/ranges/ranges.cpp:24-59 and :76-97).  One thread per batch row.
__global__ void ranges_sequential_kernel(int64_t B, int64_t m, int64_t n, int64_t R, const float *x1, int64_t x1s,
                                         const float *x2, int64_t x2s, float cutoff_scalar, const float *cutoffs,
                                         int block, int step, int mode, const int32_t *flags, int32_t *start,
                                         int32_t *end) {
    const int64_t b = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (b >= B || flags[b]) return;
    const float cutoff = cutoffs ? cutoffs[b] : cutoff_scalar;
    const float *a = x1 + b * x1s;
    const float *c = x2 + b * x2s;
    int32_t *S = start + b * R, *E = end + b * R;
    if (mode == 0) {
        int64_t ps = 0, pe = 0;
        for (int64_t i = 0; i < R; i++) {
            const float first = a[i * block];
            const float last = a[min((i + 1) * (int64_t)block, m) - 1];
            int64_t j = ps;
            while (j < n && !(first - c[j] <= cutoff)) j = min(j + step, n);
            int64_t q = max(pe, j);
            while (q < n && !(c[q] - last > cutoff)) q = min(q + step, n);
            S[i] = (int32_t)j;
            E[i] = (int32_t)q;
            ps = j;
            pe = q;
        }
    } else {
        for (int64_t i = 0; i < R; i++) S[i] = (int32_t)n;
        if (R > 0) S[0] = 0;
        int64_t j = block;
        for (int64_t i = 0; i < R; i++) {
            const float last = a[min((i + 1) * (int64_t)block, n) - 1];
            while (j < n && !(c[j] - last >= cutoff)) j = min(j + block, n);
            E[i] = (int32_t)j;
            const int64_t reach = (j + block - 1) / block;
            for (int64_t t = i; t < reach && t < R; t++) S[t] = min(S[t], (int32_t)(i * block));
        }
    }
}

// transpose: every row block marks the column blocks it touches (integer atomic min / max
// commute, so the result does not depend on the order).
__global__ void transpose_mark_kernel(int64_t B, int64_t R, int64_t C, const int32_t *start, const int32_t *end,
                                      int x1_size, int block, int32_t *start_t, int32_t *end_t) {
    const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (idx >= B * R) return;
    const int64_t b = idx / R, r = idx % R;
    const int s = start[idx], e = end[idx];
    if (s == e) return;
    const int64_t c0 = s / block;
    const int64_t c1 = ((int64_t)e + block - 1) / block;
    const int row0 = (int)(r * block);
    const int row1 = min(row0 + block, x1_size);
    for (int64_t c = max(c0, (int64_t)0); c < c1 && c < C; c++) {
        atomicMin(start_t + b * C + c, row0);
        atomicMax(end_t + b * C + c, row1);
    }
}

__global__ void transpose_init_kernel(int64_t total, int x1_size, int32_t *start_t, int32_t *end_t) {
    const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (idx < total) {
        start_t[idx] = x1_size;
        end_t[idx] = 0;
    }
}

// Untouched column blocks take the start of the nearest touched block to their left (0 if
// none) as an empty range (native/ranges/ranges.cpp:136-146).  One CTA per batch; a chunked
// scan carries the last touched start.
__global__ void __launch_bounds__(1024) transpose_fix_kernel(int64_t C, int x1_size, int32_t *start_t,
                                                              int32_t *end_t) {
    __shared__ int warp_last[32];
    __shared__ int carry;
    int32_t *S = start_t + blockIdx.x * C, *E = end_t + blockIdx.x * C;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry = -1;  // index of the last touched block seen so far
    __syncthreads();
    for (int64_t base = 0; base < C; base += 1024) {
        const int64_t c = base + threadIdx.x;
        const int sv = c < C ? S[c] : x1_size;
        const bool touched = c < C && sv != x1_size;
        int last = touched ? (int)c : -1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, last, o);
            if (lane >= o) last = max(last, y);
        }
        if (lane == 31) warp_last[warp] = last;
        __syncthreads();
        int pre = carry;
        for (int q = 0; q < warp; q++) pre = max(pre, warp_last[q]);
        last = max(last, pre);
        __syncthreads();
        if (threadIdx.x == 1023) carry = last;
        // S[last] for last < c is a touched block and is never rewritten, so reading it here is safe
        if (c < C && !touched) {
            const int v = last >= 0 ? S[last] : 0;
            S[c] = v;
            E[c] = v;
        }
        __syncthreads();
    }
}

// One thread per item on at most 2^20 blocks of 256 threads: callers refuse more items.
constexpr int64_t KM_RANGES_MAX_ITEMS = (1LL << 20) * 256;
static inline unsigned grid_for(int64_t total, int threads) {
    return (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(total, threads), 1 << 20));
}

static int make_ranges_common(const char *name, int64_t B, int64_t m, int64_t n, const float *x1, int64_t x1s,
                              const float *x2, int64_t x2s, float cutoff, const float *cutoffs, int block, int step,
                              int mode, int32_t *start, int32_t *end, int32_t *flags, cudaStream_t s) {
    KM_REQUIRE(B >= 0 && m >= 0 && n >= 0 && n <= 0x7fffffffLL - 2 * (int64_t)block && m <= 0x7fffffffLL,
               KM_ERR_INVALID_ARGUMENT, "%s: bad sizes", name);
    KM_REQUIRE(block >= 1, KM_ERR_INVALID_ARGUMENT, "%s: block_size must be >= 1", name);
    const int64_t R = ceil_div(m, block);
    if (B == 0 || R == 0) return KM_OK;
    KM_REQUIRE(x1 && x2 && start && end && flags, KM_ERR_INVALID_ARGUMENT, "%s: null pointer", name);
    KM_REQUIRE(B <= 0x7fffffffLL, KM_ERR_UNSUPPORTED, "%s: too many batch rows", name);
    // (the per-element kernels run one thread per (batch row, row block) on grids of at most 2^20 blocks)
    KM_REQUIRE(B <= KM_RANGES_MAX_ITEMS / R, KM_ERR_UNSUPPORTED, "%s: more than %lld (batch row, row block) pairs", name,
               (long long)KM_RANGES_MAX_ITEMS);
    fill_flags_kernel<<<grid_for(B, 256), 256, 0, s>>>(B, flags);
    if (n > 1) check_sorted_kernel<<<(unsigned)std::min<int64_t>(ceil_div(B * n, 256), 148 * 16), 256, 0, s>>>(B, n, x2, x2s, flags);
    range_bounds_kernel<<<grid_for(B * R, 256), 256, 0, s>>>(B, m, n, R, x1, x1s, x2, x2s, cutoff, cutoffs, block, step,
                                                             mode, flags, start, end);
    if (mode == 0) {
        prefix_max_kernel<<<(unsigned)B, 1024, 0, s>>>(R, flags, start, end, 0, 0);
    } else {
        prefix_max_kernel<<<(unsigned)B, 1024, 0, s>>>(R, flags, end, nullptr, 1, block);
        symmetric_start_kernel<<<grid_for(B * R, 256), 256, 0, s>>>(B, n, R, block, flags, end, start);
    }
    ranges_sequential_kernel<<<grid_for(B, 32), 32, 0, s>>>(B, m, n, R, x1, x1s, x2, x2s, cutoff, cutoffs, block, step,
                                                            mode, flags, start, end);
    KM_CHECK_LAUNCH(name);
    return KM_OK;
}

}  // namespace km

extern "C" int km_make_ranges_f32(int64_t B, int64_t m, int64_t n, const float *x1, const float *x2, float cutoff,
                                  int32_t block_size, int32_t align, int32_t *start, int32_t *end, int32_t *flags,
                                  void *stream) {
    return km::make_ranges_common("km_make_ranges_f32", B, m, n, x1, m, x2, n, cutoff, nullptr, block_size,
                                  align ? block_size : 1, 0, start, end, flags, static_cast<cudaStream_t>(stream));
}

extern "C" int km_make_ranges_symmetric_f32(int64_t B, int64_t n, const float *x, float cutoff, int32_t block_size,
                                            int32_t *start, int32_t *end, int32_t *flags, void *stream) {
    return km::make_ranges_common("km_make_ranges_symmetric_f32", B, n, n, x, n, x, n, cutoff, nullptr, block_size,
                                  block_size, 1, start, end, flags, static_cast<cudaStream_t>(stream));
}

extern "C" int km_make_ranges_symmetric_cutoffs_f32(int64_t B, int64_t n, const float *x, int64_t x_batch_stride,
                                                    const float *cutoffs, int32_t block_size, int32_t *start,
                                                    int32_t *end, int32_t *flags, void *stream) {
    KM_REQUIRE(cutoffs != nullptr || B == 0, KM_ERR_INVALID_ARGUMENT, "km_make_ranges_symmetric_cutoffs_f32: null cutoffs");
    KM_REQUIRE(x_batch_stride == 0 || x_batch_stride >= n, KM_ERR_INVALID_ARGUMENT,
               "km_make_ranges_symmetric_cutoffs_f32: x_batch_stride must be 0 (shared x) or at least n");
    return km::make_ranges_common("km_make_ranges_symmetric_cutoffs_f32", B, n, n, x, x_batch_stride, x, x_batch_stride,
                                  0.0f, cutoffs, block_size, block_size, 1, start, end, flags,
                                  static_cast<cudaStream_t>(stream));
}

extern "C" int km_transpose_ranges_i32(int64_t B, int64_t R, const int32_t *start, const int32_t *end,
                                       int64_t x1_size, int64_t x2_size, int32_t block_size, int32_t *start_t,
                                       int32_t *end_t, void *stream) {
    using namespace km;
    KM_REQUIRE(B >= 0 && R >= 0 && x1_size >= 0 && x2_size >= 0 && x1_size <= 0x7fffffffLL - block_size &&
                   x2_size <= 0x7fffffffLL - block_size,
               KM_ERR_INVALID_ARGUMENT, "km_transpose_ranges_i32: bad sizes");
    KM_REQUIRE(block_size >= 1, KM_ERR_INVALID_ARGUMENT, "km_transpose_ranges_i32: block_size must be >= 1");
    const int64_t C = ceil_div(x2_size, block_size);
    if (B == 0 || C == 0) return KM_OK;
    KM_REQUIRE(start_t && end_t && (R == 0 || (start && end)), KM_ERR_INVALID_ARGUMENT,
               "km_transpose_ranges_i32: null pointer");
    KM_REQUIRE(B <= 0x7fffffffLL, KM_ERR_UNSUPPORTED, "km_transpose_ranges_i32: too many batch rows");
    KM_REQUIRE(B <= KM_RANGES_MAX_ITEMS / C && (R == 0 || B <= KM_RANGES_MAX_ITEMS / R), KM_ERR_UNSUPPORTED,
               "km_transpose_ranges_i32: more than %lld (batch row, block) pairs", (long long)KM_RANGES_MAX_ITEMS);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    transpose_init_kernel<<<grid_for(B * C, 256), 256, 0, s>>>(B * C, (int)x1_size, start_t, end_t);
    if (R > 0)
        transpose_mark_kernel<<<grid_for(B * R, 256), 256, 0, s>>>(B, R, C, start, end, (int)x1_size, block_size,
                                                                   start_t, end_t);
    transpose_fix_kernel<<<(unsigned)B, 1024, 0, s>>>(C, (int)x1_size, start_t, end_t);
    KM_CHECK_LAUNCH("km_transpose_ranges_i32");
    return KM_OK;
}

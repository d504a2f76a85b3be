// Vector kernels of the row-sharded conjugate-gradient solve (kernel_matmul_b200/cg.py).
//
// The reference has no CG of its own: it inherits LinearOperator.solve from the third-party
// linear_operator package (tests/test_linear_operator.py:9-38).  These kernels are the part of an
// iteration that is not the banded product: q = K p + sigma^2 p, the inner products p.q and
// r.r, and the updates of x, r and p.  All of it is HBM-bound streaming work on (rows, k)
// vectors, so one thread owns one row (k contiguous floats, 16-byte loads when k % 4 == 0), one
// CTA of 128 threads owns one 128-row block at a time, and grids are sized in multiples of the SM
// count.
//
// Inner products are formed so that they do not depend on how rows are dealt out to GPUs:
//   * one partial per 128-row block and column (a fixed shuffle tree inside the CTA),
//   * per SEGMENT of `seg_blocks` consecutive row blocks the partials are added in fp64 in a
//     fixed order (km_cg_segment_sums_f32); segments are aligned at row block 0 and a rank owns
//     whole segments,
//   * the segment sums of all ranks, gathered in rank order (= segment order), are added in that
//     order in fp64 by every CTA that needs alpha or beta.
// The same numbers therefore come out for 1, 2, 4 or 8 ranks.
//
// Rows a rank does not own but needs as right-hand side of its next product (the band's halo)
// are updated redundantly by that rank: it receives the owner's q rows and applies the same
// alpha and beta, so p never has to be exchanged itself.
#include "km_common.cuh"

namespace km {

constexpr int CG_THREADS = 128;  // = rows of a row block

// Adds `v[c]`, c < KC, over the 128 threads of the CTA in a fixed order; the totals arrive in
// thread c (c < KC) of warp 0 as the return value.
template <int KC>
__device__ __forceinline__ float cg_block_reduce(float (&v)[KC], float (*warp_part)[32]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int c = 0; c < KC; c++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v[c] += __shfl_xor_sync(0xffffffffu, v[c], o);
    }
    if (lane == 0) {
#pragma unroll
        for (int c = 0; c < KC; c++) warp_part[warp][c] = v[c];
    }
    __syncthreads();
    float total = 0.0f;
    if (warp == 0 && lane < KC) total = (warp_part[0][lane] + warp_part[1][lane]) + (warp_part[2][lane] + warp_part[3][lane]);
    __syncthreads();
    return total;
}

// k columns of one row, starting at column c0: 16-byte accesses when `vec`.
template <int KC>
__device__ __forceinline__ void cg_load_row(const float *row, int c0, int k, bool vec, float (&v)[KC]) {
    if (KC >= 4 && vec && c0 + KC <= k) {
#pragma unroll
        for (int c = 0; c < KC; c += 4) {
            const float4 t = *reinterpret_cast<const float4 *>(row + c0 + c);
            v[c] = t.x, v[c + 1] = t.y, v[c + 2] = t.z, v[c + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int c = 0; c < KC; c++) v[c] = c0 + c < k ? row[c0 + c] : 0.0f;
    }
}
template <int KC>
__device__ __forceinline__ void cg_store_row(float *row, int c0, int k, bool vec, const float (&v)[KC]) {
    if (KC >= 4 && vec && c0 + KC <= k) {
#pragma unroll
        for (int c = 0; c < KC; c += 4) *reinterpret_cast<float4 *>(row + c0 + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
    } else {
#pragma unroll
        for (int c = 0; c < KC; c++)
            if (c0 + c < k) row[c0 + c] = v[c];
    }
}

// Sum of the gathered segment sums, in slot order: base[rank * rank_stride_bytes + slot * k + c].
__device__ __forceinline__ double cg_total(const unsigned char *base, int64_t rank_stride_bytes, int ranks, int slots,
                                           int64_t k, int c) {
    double t = 0.0;
    for (int rk = 0; rk < ranks; rk++) {
        const double *seg = reinterpret_cast<const double *>(base + rk * rank_stride_bytes);
        for (int s = 0; s < slots; s++) t += seg[s * k + c];
    }
    return t;
}

struct CgDotsArgs {
    int64_t k, row0, row1;       // rows [row0, row1) of this rank (row0 a multiple of 128)
    const float *a, *b;          // plain inner product: a . b
    float *kp;                   // q form: in K p, out q = K p + sigma2 p   (b = p)
    float sigma2;
    float *block_partials;       // [row blocks of the window][k]
    float *send_top, *send_bottom;  // copies of the first / last rows of q for the neighbours
    int64_t top_rows, bottom_rows;
    int vec;
};

// QFORM: q = kp + sigma2 * p written back to kp, partial of p . q, halo copies of q.
// else : partial of a . b.
template <int KC, bool QFORM>
__global__ void __launch_bounds__(CG_THREADS) cg_dots_kernel(const CgDotsArgs g) {
    __shared__ float warp_part[4][32];
    const int64_t blocks = (g.row1 - g.row0 + KM_BLOCK_SIZE - 1) / KM_BLOCK_SIZE;
    const int64_t k = g.k;
    for (int64_t blk = blockIdx.x; blk < blocks; blk += gridDim.x) {
        const int64_t row = g.row0 + blk * KM_BLOCK_SIZE + threadIdx.x;
        const bool live = row < g.row1;
        for (int c0 = 0; c0 < k; c0 += KC) {
            float acc[KC];
#pragma unroll
            for (int c = 0; c < KC; c++) acc[c] = 0.0f;
            if (live) {
                float u[KC], w[KC];
                if (QFORM) {
                    cg_load_row<KC>(g.kp + row * k, c0, (int)k, g.vec, u);
                    cg_load_row<KC>(g.b + row * k, c0, (int)k, g.vec, w);
#pragma unroll
                    for (int c = 0; c < KC; c++) {
                        u[c] = fmaf(g.sigma2, w[c], u[c]);
                        acc[c] = w[c] * u[c];
                    }
                    cg_store_row<KC>(g.kp + row * k, c0, (int)k, g.vec, u);
                    if (row - g.row0 < g.top_rows) cg_store_row<KC>(g.send_top + (row - g.row0) * k, c0, (int)k, g.vec, u);
                    if (g.row1 - row <= g.bottom_rows)
                        cg_store_row<KC>(g.send_bottom + (g.bottom_rows - (g.row1 - row)) * k, c0, (int)k, g.vec, u);
                } else {
                    cg_load_row<KC>(g.a + row * k, c0, (int)k, g.vec, u);
                    cg_load_row<KC>(g.b + row * k, c0, (int)k, g.vec, w);
#pragma unroll
                    for (int c = 0; c < KC; c++) acc[c] = u[c] * w[c];
                }
            }
            const float total = cg_block_reduce<KC>(acc, warp_part);
            if (threadIdx.x < KC && c0 + threadIdx.x < k) g.block_partials[blk * k + c0 + threadIdx.x] = total;
        }
    }
}

// seg_sums[s][c] = sum over the row blocks of segment s of block_partials[blk][c], in fp64: 32
// lanes per column take the blocks lane, lane + 32, ... in order, then a fixed tree over the lanes.
__global__ void __launch_bounds__(512) cg_segment_sums_kernel(int64_t k, const float *block_partials, int64_t blocks,
                                                              int64_t seg_blocks, double *seg_sums) {
    const int64_t s = blockIdx.x;
    const int64_t b0 = s * seg_blocks, b1 = min(b0 + seg_blocks, blocks);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;  // warp = column inside a chunk of 16
    for (int64_t c0 = 0; c0 < k; c0 += 16) {
        const int64_t c = c0 + warp;
        double t = 0.0;
        if (c < k)
            for (int64_t blk = b0 + lane; blk < b1; blk += 32) t += (double)block_partials[blk * k + c];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0 && c < k) seg_sums[s * k + c] = t;
    }
}

struct CgUpdateArgs {
    int64_t k, row0, row1, lo, hi;  // own rows [row0, row1), rows kept up to date [lo, hi)
    float *x, *r, *p;               // (n, k) indexed by global row
    const float *q_own;             // q of own rows, indexed by global row
    const float *q_below, *q_above; // q(row) = q_below[(row - below_origin) * k + c] for row < row0, etc.
    int64_t below_origin, above_origin;
    const unsigned char *seg_base;  // gathered segment sums (p . q for update_xr, r . r for update_p)
    int64_t seg_rank_stride;        // bytes
    int seg_ranks, seg_slots;
    const float *rs_in;             // [k] r . r of the current residual
    float *rs_out;                  // update_p: [k] r . r of the new residual
    float *history;                 // update_p: [k] sqrt(rs_new) / ynorm
    float *coeff_out;               // [k] alpha (update_xr) / beta (update_p) of this iteration, or null
    const float *ynorm;             // [k]
    float *block_partials;          // update_xr: partials of r . r over own row blocks
    float tiny;
    int vec;
};

// x += alpha p (own rows), r -= alpha q (rows [lo, hi)), partials of r . r (own row blocks).
template <int KC>
__global__ void __launch_bounds__(CG_THREADS) cg_update_xr_kernel(const CgUpdateArgs g) {
    __shared__ float warp_part[4][32];
    __shared__ float alpha_s[KC];
    const int64_t k = g.k;
    const int64_t blk_lo = g.lo / KM_BLOCK_SIZE, blk_hi = (g.hi + KM_BLOCK_SIZE - 1) / KM_BLOCK_SIZE;
    const int64_t own_blk0 = g.row0 / KM_BLOCK_SIZE;
    for (int c0 = 0; c0 < k; c0 += KC) {
        __syncthreads();
        if (threadIdx.x < KC && c0 + threadIdx.x < k) {
            const int c = c0 + threadIdx.x;
            const double pq = cg_total(g.seg_base, g.seg_rank_stride, g.seg_ranks, g.seg_slots, k, c);
            alpha_s[threadIdx.x] = g.rs_in[c] / fmaxf((float)pq, g.tiny);
            if (blockIdx.x == 0 && g.coeff_out != nullptr) g.coeff_out[c] = alpha_s[threadIdx.x];
        }
        __syncthreads();
        float alpha[KC];
#pragma unroll
        for (int c = 0; c < KC; c++) alpha[c] = c0 + c < k ? alpha_s[c] : 0.0f;
        for (int64_t blk = blk_lo + blockIdx.x; blk < blk_hi; blk += gridDim.x) {
            const int64_t row = blk * KM_BLOCK_SIZE + threadIdx.x;
            const bool own_block = blk * KM_BLOCK_SIZE >= g.row0 && blk * KM_BLOCK_SIZE < g.row1;
            float acc[KC];
#pragma unroll
            for (int c = 0; c < KC; c++) acc[c] = 0.0f;
            if (row >= g.lo && row < g.hi) {
                const bool own = row >= g.row0 && row < g.row1;
                const float *qsrc = own ? g.q_own + row * k
                                        : (row < g.row0 ? g.q_below + (row - g.below_origin) * k
                                                        : g.q_above + (row - g.above_origin) * k);
                float qv[KC], rv[KC];
                cg_load_row<KC>(qsrc, c0, (int)k, g.vec, qv);
                cg_load_row<KC>(g.r + row * k, c0, (int)k, g.vec, rv);
#pragma unroll
                for (int c = 0; c < KC; c++) rv[c] = fmaf(-alpha[c], qv[c], rv[c]);
                cg_store_row<KC>(g.r + row * k, c0, (int)k, g.vec, rv);
                if (own) {
                    float pv[KC], xv[KC];
                    cg_load_row<KC>(g.p + row * k, c0, (int)k, g.vec, pv);
                    cg_load_row<KC>(g.x + row * k, c0, (int)k, g.vec, xv);
#pragma unroll
                    for (int c = 0; c < KC; c++) {
                        xv[c] = fmaf(alpha[c], pv[c], xv[c]);
                        acc[c] = rv[c] * rv[c];
                    }
                    cg_store_row<KC>(g.x + row * k, c0, (int)k, g.vec, xv);
                }
            }
            if (own_block) {  // CTA-uniform
                const float total = cg_block_reduce<KC>(acc, warp_part);
                if (threadIdx.x < KC && c0 + threadIdx.x < k)
                    g.block_partials[(blk - own_blk0) * k + c0 + threadIdx.x] = total;
            }
        }
    }
}

// p = r + beta p on rows [lo, hi); CTA 0 also stores r . r of the new residual and the relative
// residual norm.
template <int KC>
__global__ void __launch_bounds__(CG_THREADS) cg_update_p_kernel(const CgUpdateArgs g) {
    __shared__ float beta_s[KC];
    const int64_t k = g.k;
    const int64_t blk_lo = g.lo / KM_BLOCK_SIZE, blk_hi = (g.hi + KM_BLOCK_SIZE - 1) / KM_BLOCK_SIZE;
    for (int c0 = 0; c0 < k; c0 += KC) {
        __syncthreads();
        if (threadIdx.x < KC && c0 + threadIdx.x < k) {
            const int c = c0 + threadIdx.x;
            const float rs_new = (float)cg_total(g.seg_base, g.seg_rank_stride, g.seg_ranks, g.seg_slots, k, c);
            beta_s[threadIdx.x] = rs_new / fmaxf(g.rs_in[c], g.tiny);
            if (blockIdx.x == 0) {
                if (g.coeff_out != nullptr) g.coeff_out[c] = beta_s[threadIdx.x];
                g.rs_out[c] = rs_new;
                if (g.history != nullptr) g.history[c] = sqrtf(rs_new) / g.ynorm[c];
            }
        }
        __syncthreads();
        float beta[KC];
#pragma unroll
        for (int c = 0; c < KC; c++) beta[c] = c0 + c < k ? beta_s[c] : 0.0f;
        for (int64_t blk = blk_lo + blockIdx.x; blk < blk_hi; blk += gridDim.x) {
            const int64_t row = blk * KM_BLOCK_SIZE + threadIdx.x;
            if (row >= g.lo && row < g.hi) {
                float pv[KC], rv[KC];
                cg_load_row<KC>(g.p + row * k, c0, (int)k, g.vec, pv);
                cg_load_row<KC>(g.r + row * k, c0, (int)k, g.vec, rv);
#pragma unroll
                for (int c = 0; c < KC; c++) pv[c] = fmaf(beta[c], pv[c], rv[c]);
                cg_store_row<KC>(g.p + row * k, c0, (int)k, g.vec, pv);
            }
        }
    }
}

// rs[c] = total of the gathered segment sums, ynorm[c] = max(sqrt(rs[c]), tiny): the start of a solve.
__global__ void cg_init_scalars_kernel(int64_t k, const unsigned char *seg_base, int64_t seg_rank_stride, int seg_ranks,
                                       int seg_slots, float *rs, float *ynorm, float tiny) {
    for (int64_t c = threadIdx.x; c < k; c += blockDim.x) {
        const float t = (float)cg_total(seg_base, seg_rank_stride, seg_ranks, seg_slots, k, (int)c);
        rs[c] = t;
        ynorm[c] = fmaxf(sqrtf(t), tiny);
    }
}

static int cg_grid(int64_t blocks) {
    // resident CTAs: 148 SMs x 16 CTAs of 128 threads
    return (int)std::max<int64_t>(1, std::min<int64_t>(blocks, 148 * 16));
}

static bool cg_vec_ok(int64_t k, std::initializer_list<const void *> ptrs) {
    bool ok = k % 4 == 0;
    for (const void *p : ptrs) ok = ok && (p == nullptr || (uintptr_t)p % 16 == 0);
    return ok;
}

template <typename F>
static int cg_dispatch_kc(int64_t k, F &&f) {
    if (k <= 1) return f(std::integral_constant<int, 1>{});
    if (k <= 2) return f(std::integral_constant<int, 2>{});
    if (k <= 4) return f(std::integral_constant<int, 4>{});
    if (k <= 8) return f(std::integral_constant<int, 8>{});
    if (k <= 16) return f(std::integral_constant<int, 16>{});
    return f(std::integral_constant<int, 32>{});
}

}  // namespace km

#define KM_CG_ROWS_OK(name)                                                                                      \
    KM_REQUIRE(k >= 1 && row0 >= 0 && row1 >= row0 && row0 % KM_BLOCK_SIZE == 0, KM_ERR_INVALID_ARGUMENT,         \
               "%s: need k >= 1 and a row window [row0, row1) that starts at a row-block boundary", name)

extern "C" int km_cg_block_dots_f32(int64_t k, const float *a, const float *b, int64_t row0, int64_t row1,
                                    float *block_partials, void *stream) {
    using namespace km;
    KM_CG_ROWS_OK("km_cg_block_dots_f32");
    if (row1 == row0) return KM_OK;
    KM_REQUIRE(a && b && block_partials, KM_ERR_INVALID_ARGUMENT, "km_cg_block_dots_f32: null pointer");
    CgDotsArgs g{};
    g.k = k, g.row0 = row0, g.row1 = row1, g.a = a, g.b = b, g.block_partials = block_partials;
    g.vec = cg_vec_ok(k, {a, b}) ? 1 : 0;
    const int64_t blocks = ceil_div(row1 - row0, KM_BLOCK_SIZE);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return cg_dispatch_kc(k, [&](auto kc) {
        cg_dots_kernel<decltype(kc)::value, false><<<cg_grid(blocks), CG_THREADS, 0, s>>>(g);
        KM_CHECK_LAUNCH("km_cg_block_dots_f32 launch");
        return KM_OK;
    });
}

extern "C" int km_cg_q_dots_f32(int64_t k, float *kp, const float *p, float sigma2, int64_t row0, int64_t row1,
                                float *block_partials, float *send_top, int64_t top_rows, float *send_bottom,
                                int64_t bottom_rows, void *stream) {
    using namespace km;
    KM_CG_ROWS_OK("km_cg_q_dots_f32");
    if (row1 == row0) return KM_OK;
    KM_REQUIRE(kp && p && block_partials, KM_ERR_INVALID_ARGUMENT, "km_cg_q_dots_f32: null pointer");
    KM_REQUIRE(top_rows >= 0 && bottom_rows >= 0 && top_rows <= row1 - row0 && bottom_rows <= row1 - row0 &&
                   (top_rows == 0 || send_top) && (bottom_rows == 0 || send_bottom),
               KM_ERR_INVALID_ARGUMENT, "km_cg_q_dots_f32: halo copies must fit the window and have a destination");
    CgDotsArgs g{};
    g.k = k, g.row0 = row0, g.row1 = row1, g.kp = kp, g.b = p, g.sigma2 = sigma2, g.block_partials = block_partials;
    g.send_top = send_top, g.top_rows = top_rows, g.send_bottom = send_bottom, g.bottom_rows = bottom_rows;
    g.vec = cg_vec_ok(k, {kp, p, send_top, send_bottom}) ? 1 : 0;
    const int64_t blocks = ceil_div(row1 - row0, KM_BLOCK_SIZE);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return cg_dispatch_kc(k, [&](auto kc) {
        cg_dots_kernel<decltype(kc)::value, true><<<cg_grid(blocks), CG_THREADS, 0, s>>>(g);
        KM_CHECK_LAUNCH("km_cg_q_dots_f32 launch");
        return KM_OK;
    });
}

extern "C" int km_cg_segment_sums_f32(int64_t k, const float *block_partials, int64_t blocks, int64_t seg_blocks,
                                      double *seg_sums, void *stream) {
    using namespace km;
    KM_REQUIRE(k >= 1 && blocks >= 0 && seg_blocks >= 1, KM_ERR_INVALID_ARGUMENT, "km_cg_segment_sums_f32: bad sizes");
    if (blocks == 0) return KM_OK;
    KM_REQUIRE(block_partials && seg_sums, KM_ERR_INVALID_ARGUMENT, "km_cg_segment_sums_f32: null pointer");
    const int64_t segs = ceil_div(blocks, seg_blocks);
    KM_REQUIRE(segs <= 0x7fffffffLL, KM_ERR_UNSUPPORTED, "km_cg_segment_sums_f32: too many segments");
    cg_segment_sums_kernel<<<(unsigned)segs, 512, 0, static_cast<cudaStream_t>(stream)>>>(k, block_partials, blocks,
                                                                                          seg_blocks, seg_sums);
    KM_CHECK_LAUNCH("km_cg_segment_sums_f32 launch");
    return KM_OK;
}

extern "C" int km_cg_init_scalars_f32(int64_t k, const void *seg_sums, int64_t seg_rank_stride_bytes, int32_t seg_ranks,
                                      int32_t seg_slots, float *rs, float *ynorm, void *stream) {
    using namespace km;
    KM_REQUIRE(k >= 1 && seg_sums && rs && ynorm && seg_ranks >= 1 && seg_slots >= 0 && seg_rank_stride_bytes % 8 == 0,
               KM_ERR_INVALID_ARGUMENT, "km_cg_init_scalars_f32: bad arguments");
    cg_init_scalars_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        k, static_cast<const unsigned char *>(seg_sums), seg_rank_stride_bytes, seg_ranks, seg_slots, rs, ynorm, 1.17549435e-38f);
    KM_CHECK_LAUNCH("km_cg_init_scalars_f32 launch");
    return KM_OK;
}

extern "C" int km_cg_update_xr_f32(int64_t k, float *x, float *r, const float *p, const float *q_own,
                                   const float *q_below, int64_t below_origin, const float *q_above,
                                   int64_t above_origin, int64_t row0, int64_t row1, int64_t lo, int64_t hi,
                                   const void *pq_seg_sums, int64_t seg_rank_stride_bytes, int32_t seg_ranks,
                                   int32_t seg_slots, const float *rs, float *block_partials, float *alpha_row,
                                   void *stream) {
    using namespace km;
    KM_CG_ROWS_OK("km_cg_update_xr_f32");
    KM_REQUIRE(lo >= 0 && lo <= row0 && hi >= row1, KM_ERR_INVALID_ARGUMENT,
               "km_cg_update_xr_f32: [lo, hi) must contain the own rows");
    if (hi == lo) return KM_OK;
    KM_REQUIRE(x && r && p && q_own && pq_seg_sums && rs && block_partials && (lo == row0 || q_below) &&
                   (hi == row1 || q_above) && seg_ranks >= 1 && seg_slots >= 0 && seg_rank_stride_bytes % 8 == 0,
               KM_ERR_INVALID_ARGUMENT, "km_cg_update_xr_f32: bad arguments");
    CgUpdateArgs g{};
    g.k = k, g.row0 = row0, g.row1 = row1, g.lo = lo, g.hi = hi, g.x = x, g.r = r, g.p = const_cast<float *>(p);
    g.q_own = q_own, g.q_below = q_below, g.q_above = q_above, g.below_origin = below_origin, g.above_origin = above_origin;
    g.seg_base = static_cast<const unsigned char *>(pq_seg_sums), g.seg_rank_stride = seg_rank_stride_bytes;
    g.seg_ranks = seg_ranks, g.seg_slots = seg_slots, g.rs_in = rs, g.block_partials = block_partials;
    g.coeff_out = alpha_row;
    g.tiny = 1.17549435e-38f;
    g.vec = cg_vec_ok(k, {x, r, p, q_own, q_below, q_above}) ? 1 : 0;
    const int64_t blocks = ceil_div(hi, KM_BLOCK_SIZE) - lo / KM_BLOCK_SIZE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return cg_dispatch_kc(k, [&](auto kc) {
        cg_update_xr_kernel<decltype(kc)::value><<<cg_grid(blocks), CG_THREADS, 0, s>>>(g);
        KM_CHECK_LAUNCH("km_cg_update_xr_f32 launch");
        return KM_OK;
    });
}

extern "C" int km_cg_update_p_f32(int64_t k, float *p, const float *r, int64_t lo, int64_t hi, const void *rr_seg_sums,
                                  int64_t seg_rank_stride_bytes, int32_t seg_ranks, int32_t seg_slots,
                                  const float *rs_old, float *rs_new, const float *ynorm, float *history_row,
                                  float *beta_row, void *stream) {
    using namespace km;
    KM_REQUIRE(k >= 1 && lo >= 0 && hi >= lo, KM_ERR_INVALID_ARGUMENT, "km_cg_update_p_f32: bad sizes");
    KM_REQUIRE(p && r && rr_seg_sums && rs_old && rs_new && rs_old != rs_new && (history_row == nullptr || ynorm) &&
                   seg_ranks >= 1 && seg_slots >= 0 && seg_rank_stride_bytes % 8 == 0,
               KM_ERR_INVALID_ARGUMENT, "km_cg_update_p_f32: bad arguments (rs_old and rs_new must differ)");
    CgUpdateArgs g{};
    g.k = k, g.lo = lo, g.hi = hi, g.p = p, g.r = const_cast<float *>(r);
    g.seg_base = static_cast<const unsigned char *>(rr_seg_sums), g.seg_rank_stride = seg_rank_stride_bytes;
    g.seg_ranks = seg_ranks, g.seg_slots = seg_slots, g.rs_in = rs_old, g.rs_out = rs_new, g.history = history_row;
    g.ynorm = ynorm, g.tiny = 1.17549435e-38f, g.coeff_out = beta_row;
    g.vec = cg_vec_ok(k, {p, r}) ? 1 : 0;
    const int64_t blocks = std::max<int64_t>(1, ceil_div(hi, KM_BLOCK_SIZE) - lo / KM_BLOCK_SIZE);  // CTA 0 always runs
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return cg_dispatch_kc(k, [&](auto kc) {
        cg_update_p_kernel<decltype(kc)::value><<<cg_grid(blocks), CG_THREADS, 0, s>>>(g);
        KM_CHECK_LAUNCH("km_cg_update_p_f32 launch");
        return KM_OK;
    });
}

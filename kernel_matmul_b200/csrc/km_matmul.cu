// Forward product  out = K(x1, x2; theta) . rhs  over banded row-block ranges (FMA path).
//
// One CTA owns one 128-row block of one batch (and one block of KB rhs columns) and walks the
// block's column band [start, end) in tiles of TILE_N columns.  x2 and rhs tiles are staged in
// shared memory with cp.async, double buffered.  Lanes own rows (RPT rows each, 32 apart, so
// x1 is read coalesced and every shared-memory read in the inner loop is a broadcast); the WN
// warps of a row group take interleaved columns of a tile and their partial sums are combined
// through shared memory once, at the end of the band.  Each kernel entry is generated in
// registers (SFU ex2 / sin / cos + FP32) and immediately contracted against KB rhs values
// held in registers: RPT * KB independent FMAs per staged column and thread.
//
// Replaces kernel_matmul_cuda_kernel + the zero fill, parameter transform and column-slab sum
// around it (reference: native/matmul/matmul.cu:13-203).
#include <cooperative_groups.h>

#include "km_tcgen05.cuh"

namespace km {

namespace cg = cooperative_groups;

template <typename T>
struct MatmulArgs {
    Batch batch;
    int64_t m, n, k;
    int64_t row_blocks;  // row blocks computed by this launch
    int64_t rb_begin;    // first row block of the window; out row 0 is row rb_begin * 128
    int k_blocks;        // ceil(k / KB)
    View<const float> x1, x2, rhs, params;
    View<const int> start, end;
    View<float> out;
    int rhs_vec_ok;  // rhs rows may be copied 16 bytes at a time
    int out_vec_ok;  // out rows may be stored 16 bytes at a time
    int sum_shared_ok;  // batch sum: x1, x2, rhs, start, end are one copy shared by all batches
    int sum_tc_launched;  // batch sum: the tensor-core kernel runs next to this one and takes the shared-lengthscale case
};

// Walks the band [band_lo, band_hi) of one row block and one batch and adds
// kappa(x1r[i], x2[j]) * rhs[j, k0 + c] (times `kscale` if SCALED) to the accumulators.
template <int KT, int KB, int RPT, int WN, bool SCALED>
__device__ __forceinline__ void band_walk(const MatmulArgs<float> &a, const KernelFn<KT> &fn, const float *x2,
                                          const float *rhs, const float (&x1r)[RPT], const int band_lo,
                                          const int band_hi, const int64_t k0, const bool vec, float *smem,
                                          const int tid, const int wn, const float kscale,
                                          float (&acc)[RPT][KB], f32x2 (&acc2)[RPT][(KB % 2 == 0) ? KB / 2 : 1]) {
    constexpr int WM = 128 / (32 * RPT);
    constexpr int THREADS = 32 * WM * WN;
    constexpr int STAGE_FLOATS = TILE_N * KB + TILE_N;  // rhs tile then x2 tile
    constexpr bool PACKED = (KB % 2 == 0);
    constexpr int KB2 = PACKED ? KB / 2 : 1;

    auto stage_tile = [&](int buf, int n0) {
        float *rs = smem + buf * STAGE_FLOATS;
        stage_band_tile<KB, THREADS>(rs, rs + TILE_N * KB, x2, a.x2.s0, rhs, a.rhs.s0, a.rhs.s1, k0, a.k, n0,
                                     min(TILE_N, band_hi - n0), vec, tid);
    };

    const int tiles = (band_hi - band_lo + TILE_N - 1) / TILE_N;
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
                f32x2 rv2[KB2];
                load_staged_row2<KB>(rs, j, rv2);
#pragma unroll
                for (int i = 0; i < RPT; i++) {
                    float kv = fn.unscaled(x1r[i] - xj);
                    if (SCALED) kv *= kscale;
                    const f32x2 kk = pack2(kv, kv);
#pragma unroll
                    for (int c = 0; c < KB2; c++) acc2[i][c] = fma2(kk, rv2[c], acc2[i][c]);
                }
            } else {
                float rv[KB];
                load_staged_row<KB>(rs, j, rv);
#pragma unroll
                for (int i = 0; i < RPT; i++) {
                    float kv = fn.unscaled(x1r[i] - xj);
                    if (SCALED) kv *= kscale;
#pragma unroll
                    for (int c = 0; c < KB; c++) acc[i][c] = fmaf(kv, rv[c], acc[i][c]);
                }
            }
        }
        __syncthreads();
    }
}

// Combines the WN column-interleaved partial sums of a CTA through shared memory, applies
// `scale` and stores the 128 x KB output tile (rows relative to out_row0).
template <int KB, int RPT, int WN>
__device__ __forceinline__ void store_tile(const MatmulArgs<float> &a, float *out, const int64_t r,
                                           const int64_t out_row0, const int64_t k0, const float scale,
                                           float *smem, const int tid, float (&acc)[RPT][KB]) {
    constexpr int WM = 128 / (32 * RPT);
    constexpr int THREADS = 32 * WM * WN;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int wm = warp % WM;
    const int wn = warp / WM;
    if constexpr (WN > 1) {
        float *red = smem;  // red[wn][row_local][KB]
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            const int row_local = wm * (32 * RPT) + lane + 32 * i;
#pragma unroll
            for (int c = 0; c < KB; c++) red[(wn * 128 + row_local) * KB + c] = acc[i][c];
        }
        __syncthreads();
        for (int q = tid; q < 128 * KB; q += THREADS) {
            const int row_local = q / KB, c = q % KB;
            const int64_t row = r * KM_BLOCK_SIZE + row_local;
            if (row < a.m && k0 + c < a.k) {
                float s = 0.0f;
#pragma unroll
                for (int w = 0; w < WN; w++) s += red[(w * 128 + row_local) * KB + c];
                out[(row - out_row0) * a.out.s0 + (k0 + c) * a.out.s1] = s * scale;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            const int64_t row = r * KM_BLOCK_SIZE + wm * (32 * RPT) + lane + 32 * i;
            if (row < a.m) {
#pragma unroll
                for (int c = 0; c < KB; c++)
                    if (k0 + c < a.k) out[(row - out_row0) * a.out.s0 + (k0 + c) * a.out.s1] = acc[i][c] * scale;
            }
        }
    }
}

// One CTA per (batch, row block, block of KB rhs columns).
//
// 3 CTAs of 128 threads per SM: up to 168 registers per thread.  With the register file capped
// for a 4th CTA (128 registers) the compiler can no longer keep the operands of two columns in
// flight and the kernel is 10 % slower despite the extra warps.
template <int KT, int KB, int RPT, int WN>
__global__ void __launch_bounds__(32 * (128 / (32 * RPT)) * WN, 384 / (32 * (128 / (32 * RPT)) * WN))
    matmul_fma_kernel(const MatmulArgs<float> a) {
    constexpr int WM = 128 / (32 * RPT);
    extern __shared__ __align__(16) float smem[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int wm = warp % WM;
    const int wn = warp / WM;

    // work item: batch fastest so that CTAs resident together share rhs / x2 tiles in L2
    int64_t item = blockIdx.x;
    const int64_t b = item % a.batch.count;
    item /= a.batch.count;
    const int64_t r = a.rb_begin + item % a.row_blocks;
    const int kb = (int)(item / a.row_blocks);
    const int64_t k0 = (int64_t)kb * KB;

    const BatchIndex bi = decompose(a.batch, b);
    const float *x1 = batch_ptr(a.x1, bi);
    const float *x2 = batch_ptr(a.x2, bi);
    const float *rhs = batch_ptr(a.rhs, bi);
    float *out = batch_ptr(a.out, bi);

    KernelFn<KT> fn;
    fn.init(batch_ptr(a.params, bi), a.params.s0);

    const int n = (int)a.n;
    const int band_lo = clamp_int(batch_ptr(a.start, bi)[r * a.start.s0], 0, n);
    const int band_hi = max(band_lo, min(batch_ptr(a.end, bi)[r * a.end.s0], n));

    float x1r[RPT];
    const int64_t row_base = r * KM_BLOCK_SIZE + wm * (32 * RPT) + lane;
#pragma unroll
    for (int i = 0; i < RPT; i++) {
        const int64_t row = row_base + 32 * i;
        x1r[i] = row < a.m ? x1[row * a.x1.s0] : 0.0f;
    }

    // accumulators: packed pairs (fma.rn.f32x2) whenever the rhs block has an even width
    constexpr bool PACKED = (KB % 2 == 0);
    constexpr int KB2 = PACKED ? KB / 2 : 1;
    float acc[RPT][KB];
    f32x2 acc2[RPT][KB2];
#pragma unroll
    for (int i = 0; i < RPT; i++) {
#pragma unroll
        for (int c = 0; c < KB; c++) acc[i][c] = 0.0f;
#pragma unroll
        for (int c = 0; c < KB2; c++) acc2[i][c] = 0ull;
    }

    const bool vec = (KB % 4 == 0) && a.rhs_vec_ok && (k0 + KB <= a.k);
    band_walk<KT, KB, RPT, WN, false>(a, fn, x2, rhs, x1r, band_lo, band_hi, k0, vec, smem, tid, wn, 1.0f, acc, acc2);

    if constexpr (PACKED) {
#pragma unroll
        for (int i = 0; i < RPT; i++)
#pragma unroll
            for (int c = 0; c < KB2; c++) unpack2(acc2[i][c], acc[i][2 * c], acc[i][2 * c + 1]);
    }
    store_tile<KB, RPT, WN>(a, out, r, a.rb_begin * KM_BLOCK_SIZE, k0, fn.scale, smem, tid, acc);
}

// The same product for SMALL problems (fewer work items than half the SMs): a thread-block
// cluster of S CTAs shares one work item.  CTA c walks the c-th of S equal segments of the band;
// the 128 x KB partial tiles meet in distributed shared memory, where CTA 0 adds them in rank
// order (deterministic) and stores the result.  Without the split a 32-row-block problem keeps
// 32 of the 148 SMs busy and its run time is the length of one band walk.
template <int KT, int KB, int RPT, int WN>
__global__ void __launch_bounds__(32 * (128 / (32 * RPT)) * WN)
    matmul_fma_cluster_kernel(const MatmulArgs<float> a) {
    constexpr int WM = 128 / (32 * RPT);
    constexpr int THREADS = 32 * WM * WN;
    extern __shared__ __align__(16) float smem[];
    constexpr int WALK_FLOATS = (2 * (TILE_N * KB + TILE_N) > WN * 128 * KB) ? 2 * (TILE_N * KB + TILE_N) : WN * 128 * KB;
    float *tile = smem + WALK_FLOATS;  // this CTA's partial tile (128 x KB), read by CTA 0 of the cluster

    cg::cluster_group cluster = cg::this_cluster();
    const int S = (int)cluster.num_blocks();
    const int c = (int)cluster.block_rank();

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int wm = warp % WM;
    const int wn = warp / WM;

    int64_t item = blockIdx.x / S;
    const int64_t b = item % a.batch.count;
    item /= a.batch.count;
    const int64_t r = a.rb_begin + item % a.row_blocks;
    const int kb = (int)(item / a.row_blocks);
    const int64_t k0 = (int64_t)kb * KB;

    const BatchIndex bi = decompose(a.batch, b);
    const float *x1 = batch_ptr(a.x1, bi);
    const float *x2 = batch_ptr(a.x2, bi);
    const float *rhs = batch_ptr(a.rhs, bi);
    float *out = batch_ptr(a.out, bi);
    KernelFn<KT> fn;
    fn.init(batch_ptr(a.params, bi), a.params.s0);

    const int n = (int)a.n;
    const int band_lo = clamp_int(batch_ptr(a.start, bi)[r * a.start.s0], 0, n);
    const int band_hi = max(band_lo, min(batch_ptr(a.end, bi)[r * a.end.s0], n));
    // this CTA's segment (multiples of 4 columns keep the 16-byte copies of rhs rows aligned)
    const int seg = (((band_hi - band_lo + S - 1) / S) + 3) & ~3;
    const int seg_lo = min(band_hi, band_lo + c * seg);
    const int seg_hi = min(band_hi, seg_lo + seg);

    float x1r[RPT];
    const int64_t row_base = r * KM_BLOCK_SIZE + wm * (32 * RPT) + lane;
#pragma unroll
    for (int i = 0; i < RPT; i++) {
        const int64_t row = row_base + 32 * i;
        x1r[i] = row < a.m ? x1[row * a.x1.s0] : 0.0f;
    }
    constexpr bool PACKED = (KB % 2 == 0);
    constexpr int KB2 = PACKED ? KB / 2 : 1;
    float acc[RPT][KB];
    f32x2 acc2[RPT][KB2];
#pragma unroll
    for (int i = 0; i < RPT; i++) {
#pragma unroll
        for (int q = 0; q < KB; q++) acc[i][q] = 0.0f;
#pragma unroll
        for (int q = 0; q < KB2; q++) acc2[i][q] = 0ull;
    }
    const bool vec = (KB % 4 == 0) && a.rhs_vec_ok && (k0 + KB <= a.k);
    band_walk<KT, KB, RPT, WN, false>(a, fn, x2, rhs, x1r, seg_lo, seg_hi, k0, vec, smem, tid, wn, 1.0f, acc, acc2);
    if constexpr (PACKED) {
#pragma unroll
        for (int i = 0; i < RPT; i++)
#pragma unroll
            for (int q = 0; q < KB2; q++) unpack2(acc2[i][q], acc[i][2 * q], acc[i][2 * q + 1]);
    }

    // CTA partial: combine the WN column-interleaved sums through shared memory
    float *red = smem;  // red[wn][row_local][KB]
#pragma unroll
    for (int i = 0; i < RPT; i++) {
        const int row_local = wm * (32 * RPT) + lane + 32 * i;
#pragma unroll
        for (int q = 0; q < KB; q++) red[(wn * 128 + row_local) * KB + q] = acc[i][q];
    }
    __syncthreads();
    for (int q = tid; q < 128 * KB; q += THREADS) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < WN; w++) v += red[w * 128 * KB + q];
        tile[q] = v;
    }
    cluster.sync();  // every CTA's tile is complete and visible to the cluster
    if (c == 0) {
        const float scale = fn.scale;
        for (int q = tid; q < 128 * KB; q += THREADS) {
            const int row_local = q / KB, col = q % KB;
            const int64_t row = r * KM_BLOCK_SIZE + row_local;
            if (row < a.m && k0 + col < a.k) {
                float v = 0.0f;
                for (int peer = 0; peer < S; peer++) v += cluster.map_shared_rank(tile, peer)[q];
                out[(row - a.rb_begin * KM_BLOCK_SIZE) * a.out.s0 + (k0 + col) * a.out.s1] = v * scale;
            }
        }
    }
    cluster.sync();  // no CTA leaves while its tile may still be read
}

constexpr int SUM_MAX_SHARED = 1024;  // components whose (frequency, scale) fit the shared table

// Band walk for a SUM of spectral components that share inputs, band and lengthscale:
//   sum_b s_b exp(-tau^2 / 2 l^2) cos(2 pi f_b tau) = exp(-tau^2 / 2 l^2) * sum_b s_b cos(w_b tau).
// The envelope is evaluated once per entry, the component loop costs one SFU cosine and two
// FP32 operations per component, and the k contraction FMAs happen once per entry instead of
// once per entry and component.  `comp` holds (w_b, s_b) in shared memory.
template <int KB, int RPT, int WN>
__device__ __forceinline__ void band_walk_shared_envelope(
    const MatmulArgs<float> &a, const float c0, const float2 *comp, const int ncomp, const float *x2,
    const float *rhs, const float (&x1r)[RPT], const int band_lo, const int band_hi, const int64_t k0, const bool vec,
    float *smem, const int tid, const int wn, float (&acc)[RPT][KB], f32x2 (&acc2)[RPT][(KB % 2 == 0) ? KB / 2 : 1]) {
    constexpr int WM = 128 / (32 * RPT);
    constexpr int THREADS = 32 * WM * WN;
    constexpr int STAGE_FLOATS = TILE_N * KB + TILE_N;
    constexpr bool PACKED = (KB % 2 == 0);
    constexpr int KB2 = PACKED ? KB / 2 : 1;

    auto stage_tile = [&](int buf, int n0) {
        float *rs = smem + buf * STAGE_FLOATS;
        stage_band_tile<KB, THREADS>(rs, rs + TILE_N * KB, x2, a.x2.s0, rhs, a.rhs.s0, a.rhs.s1, k0, a.k, n0,
                                     min(TILE_N, band_hi - n0), vec, tid);
    };
    const int tiles = (band_hi - band_lo + TILE_N - 1) / TILE_N;
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
        for (int j = wn; j < cnt; j += WN) {
            const float xj = xs[j];
            float tau[RPT], g[RPT];
#pragma unroll
            for (int i = 0; i < RPT; i++) {
                tau[i] = x1r[i] - xj;
                g[i] = 0.0f;
            }
#pragma unroll 4
            for (int b = 0; b < ncomp; b++) {
                const float2 ws = comp[b];
#pragma unroll
                for (int i = 0; i < RPT; i++) g[i] = fmaf(ws.y, cos_approx(ws.x * tau[i]), g[i]);
            }
            if constexpr (PACKED) {
                f32x2 rv2[KB2];
                load_staged_row2<KB>(rs, j, rv2);
#pragma unroll
                for (int i = 0; i < RPT; i++) {
                    const float kv = g[i] * ex2_approx(c0 * tau[i] * tau[i]);
                    const f32x2 kk = pack2(kv, kv);
#pragma unroll
                    for (int c = 0; c < KB2; c++) acc2[i][c] = fma2(kk, rv2[c], acc2[i][c]);
                }
            } else {
                float rv[KB];
                load_staged_row<KB>(rs, j, rv);
#pragma unroll
                for (int i = 0; i < RPT; i++) {
                    const float kv = g[i] * ex2_approx(c0 * tau[i] * tau[i]);
#pragma unroll
                    for (int c = 0; c < KB; c++) acc[i][c] = fmaf(kv, rv[c], acc[i][c]);
                }
            }
        }
        __syncthreads();
    }
}

// One CTA per (row block, block of KB rhs columns): adds the products of ALL batches
// (components of a sum kernel) in registers; each batch's output scale goes into its kernel
// values.  out has no batch dimension.
template <int KT, int KB, int RPT, int WN>
__global__ void __launch_bounds__(32 * (128 / (32 * RPT)) * WN, 384 / (32 * (128 / (32 * RPT)) * WN))
    matmul_sum_fma_kernel(const MatmulArgs<float> a) {
    constexpr int WM = 128 / (32 * RPT);
    extern __shared__ __align__(16) float smem[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int wm = warp % WM;
    const int wn = warp / WM;

    const int64_t item = blockIdx.x;
    const int64_t r = a.rb_begin + item % a.row_blocks;
    const int64_t k0 = (item / a.row_blocks) * KB;
    const int n = (int)a.n;
    const int64_t row_base = r * KM_BLOCK_SIZE + wm * (32 * RPT) + lane;

    constexpr bool PACKED = (KB % 2 == 0);
    constexpr int KB2 = PACKED ? KB / 2 : 1;
    float acc[RPT][KB];
    f32x2 acc2[RPT][KB2];
#pragma unroll
    for (int i = 0; i < RPT; i++) {
#pragma unroll
        for (int c = 0; c < KB; c++) acc[i][c] = 0.0f;
#pragma unroll
        for (int c = 0; c < KB2; c++) acc2[i][c] = 0ull;
    }
    const bool vec = (KB % 4 == 0) && a.rhs_vec_ok && (k0 + KB <= a.k);

    // Spectral components that share everything but frequency and scale take the
    // shared-envelope walk.  Sharing of the inputs is known on the host; equality of the
    // lengthscales is checked here (one value per component).
    bool shared_envelope = false;
    if constexpr (KT == KM_KERNEL_SPECTRAL) {
        constexpr int STAGE_BYTES_TOTAL = 2 * (TILE_N * KB + TILE_N) * (int)sizeof(float);
        float2 *comp = reinterpret_cast<float2 *>(reinterpret_cast<unsigned char *>(smem) + STAGE_BYTES_TOTAL);
        if (a.sum_shared_ok && a.batch.count <= SUM_MAX_SHARED) {
            const float ell0 = a.params.data[0];
            int same = 1;
            for (int64_t b = tid; b < a.batch.count; b += blockDim.x) {
                const float *th = batch_ptr(a.params, decompose(a.batch, b));
                same &= (th[0] == ell0) ? 1 : 0;
                comp[b] = make_float2(2.0f * KM_PI_F * th[a.params.s0], th[2 * a.params.s0]);
            }
            shared_envelope = __syncthreads_and(same) != 0;
            if (shared_envelope && a.sum_tc_launched) return;  // km_matmul_sum_tc.cu computes this case
            if (shared_envelope) {
                const int band_lo = clamp_int(a.start.data[r * a.start.s0], 0, n);
                const int band_hi = max(band_lo, min(a.end.data[r * a.end.s0], n));
                float x1r[RPT];
#pragma unroll
                for (int i = 0; i < RPT; i++) {
                    const int64_t row = row_base + 32 * i;
                    x1r[i] = row < a.m ? a.x1.data[row * a.x1.s0] : 0.0f;
                }
                const float c0 = -(0.5f / (ell0 * ell0)) * KM_LOG2E_F;
                band_walk_shared_envelope<KB, RPT, WN>(a, c0, comp, (int)a.batch.count, a.x2.data, a.rhs.data, x1r,
                                                       band_lo, band_hi, k0, vec, smem, tid, wn, acc, acc2);
            }
        }
    }

    for (int64_t b = 0; b < (shared_envelope ? 0 : a.batch.count); b++) {
        const BatchIndex bi = decompose(a.batch, b);
        const float *x1 = batch_ptr(a.x1, bi);
        KernelFn<KT> fn;
        fn.init(batch_ptr(a.params, bi), a.params.s0);
        const int band_lo = clamp_int(batch_ptr(a.start, bi)[r * a.start.s0], 0, n);
        const int band_hi = max(band_lo, min(batch_ptr(a.end, bi)[r * a.end.s0], n));
        float x1r[RPT];
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            const int64_t row = row_base + 32 * i;
            x1r[i] = row < a.m ? x1[row * a.x1.s0] : 0.0f;
        }
        band_walk<KT, KB, RPT, WN, true>(a, fn, batch_ptr(a.x2, bi), batch_ptr(a.rhs, bi), x1r, band_lo, band_hi, k0,
                                         vec, smem, tid, wn, fn.scale, acc, acc2);
    }

    if constexpr (PACKED) {
#pragma unroll
        for (int i = 0; i < RPT; i++)
#pragma unroll
            for (int c = 0; c < KB2; c++) unpack2(acc2[i][c], acc[i][2 * c], acc[i][2 * c + 1]);
    }
    store_tile<KB, RPT, WN>(a, a.out.data, r, a.rb_begin * KM_BLOCK_SIZE, k0, 1.0f, smem, tid, acc);
}

template <int KT, int KB, int RPT, int WN, bool SUM>
static int launch_matmul(const MatmulArgs<float> &a, cudaStream_t stream) {
    constexpr int WM = 128 / (32 * RPT);
    constexpr int THREADS = 32 * WM * WN;
    constexpr size_t stage_bytes = 2 * (TILE_N * KB + TILE_N) * sizeof(float);
    constexpr size_t red_bytes = WN > 1 ? (size_t)WN * 128 * KB * sizeof(float) : 0;
    // (the batch-sum kernel keeps a table of SUM_MAX_SHARED (frequency, scale) pairs behind the stages)
    constexpr size_t table_bytes = SUM ? SUM_MAX_SHARED * sizeof(float2) : 0;
    constexpr size_t smem = (stage_bytes + table_bytes > red_bytes) ? stage_bytes + table_bytes : red_bytes;
    auto kernel = SUM ? matmul_sum_fma_kernel<KT, KB, RPT, WN> : matmul_fma_kernel<KT, KB, RPT, WN>;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(matmul)");
    }
    const int64_t items = (SUM ? 1 : a.batch.count) * a.row_blocks * a.k_blocks;
    if (items > 0x7fffffffLL) {
        set_error("km_matmul_f32: too many work items (%lld)", (long long)items);
        return KM_ERR_UNSUPPORTED;
    }
    if constexpr (!SUM && WN > 1) {
        // small problems: split every band over a cluster of S CTAs (S a power of two, <= 8)
        int split = 1;
        while (split < 8 && items * split * 2 <= 148) split *= 2;  // 148 SMs
        if (split > 1) {
            auto ckernel = matmul_fma_cluster_kernel<KT, KB, RPT, WN>;
            // walk stages / reduction buffer, then this CTA's partial tile
            constexpr size_t csmem = (stage_bytes > red_bytes ? stage_bytes : red_bytes) + 128 * KB * sizeof(float);
            if (csmem > 48 * 1024) {
                cudaError_t err = cudaFuncSetAttribute(ckernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csmem);
                if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(matmul cluster)");
            }
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)(items * split));
            cfg.blockDim = dim3(THREADS);
            cfg.dynamicSmemBytes = csmem;
            cfg.stream = stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = (unsigned)split;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            cudaError_t err = cudaLaunchKernelEx(&cfg, ckernel, a);
            if (err != cudaSuccess) return cuda_fail(err, "km_matmul_f32 cluster launch");
            return KM_OK;
        }
    }
    kernel<<<(unsigned)items, THREADS, smem, stream>>>(a);
    KM_CHECK_LAUNCH("km_matmul_f32 launch");
    return KM_OK;
}

template <int KT, bool SUM>
static int dispatch_matmul(MatmulArgs<float> &a, cudaStream_t stream) {
    const int64_t k = a.k;
    auto with_kb = [&](int kb) { a.k_blocks = (int)ceil_div(k, kb); };
    if (k <= 1) { with_kb(1); return launch_matmul<KT, 1, 4, 4, SUM>(a, stream); }
    if (k <= 2) { with_kb(2); return launch_matmul<KT, 2, 4, 4, SUM>(a, stream); }
    if (k <= 4) { with_kb(4); return launch_matmul<KT, 4, 4, 4, SUM>(a, stream); }
    if (k <= 8) { with_kb(8); return launch_matmul<KT, 8, 4, 4, SUM>(a, stream); }
    if (k <= 16) { with_kb(16); return launch_matmul<KT, 16, 4, 4, SUM>(a, stream); }
    with_kb(32);
    return launch_matmul<KT, 32, 2, 2, SUM>(a, stream);
}

static int matmul_entry(const char *name, int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                        const km_view *x1, const km_view *x2, const km_view *rhs, const km_view *params,
                        const km_view *start, const km_view *end, const km_view *out, int64_t rb_begin,
                        int64_t rb_count, bool sum_batches, void *stream, const void *phases = nullptr,
                        size_t phases_bytes = 0) {
    KM_REQUIRE(valid_kernel_type(kernel_type), KM_ERR_INVALID_ARGUMENT, "%s: unknown kernel type %d", name, kernel_type);
    KM_REQUIRE(batch && x1 && x2 && rhs && params && start && end && out, KM_ERR_INVALID_ARGUMENT, "%s: null argument", name);
    KM_REQUIRE(m >= 0 && n >= 0 && k >= 0 && n <= 0x7fffffffLL && m <= 0x7fffffffLL * 64, KM_ERR_INVALID_ARGUMENT,
               "%s: bad sizes m=%lld n=%lld k=%lld", name, (long long)m, (long long)n, (long long)k);
    MatmulArgs<float> a;
    int rc = make_batch(batch, &a.batch);
    if (rc != KM_OK) return rc;
    const int64_t total_blocks = ceil_div(m, KM_BLOCK_SIZE);
    if (rb_count < 0) rb_count = total_blocks - rb_begin;
    KM_REQUIRE(rb_begin >= 0 && rb_count >= 0 && rb_begin + rb_count <= total_blocks, KM_ERR_INVALID_ARGUMENT,
               "%s: row-block window [%lld, %lld) outside [0, %lld)", name, (long long)rb_begin,
               (long long)(rb_begin + rb_count), (long long)total_blocks);
    if (a.batch.count == 0 || rb_count == 0 || k == 0) {
        KM_REQUIRE(!(sum_batches && a.batch.count == 0 && rb_count > 0 && k > 0), KM_ERR_INVALID_ARGUMENT,
                   "%s: summing over an empty batch is not supported", name);
        return KM_OK;
    }
    KM_REQUIRE(x1->data && out->data && params->data && start->data && end->data, KM_ERR_INVALID_ARGUMENT,
               "%s: null data pointer", name);
    KM_REQUIRE(n == 0 || (x2->data && rhs->data), KM_ERR_INVALID_ARGUMENT, "%s: null data pointer", name);
    a.m = m;
    a.n = n;
    a.k = k;
    a.row_blocks = rb_count;
    a.rb_begin = rb_begin;
    a.x1 = make_view<const float>(x1, a.batch);
    a.x2 = make_view<const float>(x2, a.batch);
    a.rhs = make_view<const float>(rhs, a.batch);
    a.params = make_view<const float>(params, a.batch);
    a.start = make_view<const int>(start, a.batch);
    a.end = make_view<const int>(end, a.batch);
    a.out = make_view<float>(out, a.batch);
    a.rhs_vec_ok = rows_vectorizable(a.rhs, a.batch) ? 1 : 0;
    a.out_vec_ok = 0;
    a.sum_shared_ok = 1;
    a.sum_tc_launched = 0;
    for (int d = 0; d < a.batch.ndim; d++)
        if (a.batch.size[d] > 1 && (a.x1.bs[d] || a.x2.bs[d] || a.rhs.bs[d] || a.start.bs[d] || a.end.bs[d])) a.sum_shared_ok = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (sum_batches) {
        // Spectral components sharing everything but frequency and scale: the tensor-core kernel
        // takes the case of one common lengthscale (checked on the device by every CTA of both
        // kernels, so that exactly one of the two does the work).
        if (kernel_type == KM_KERNEL_SPECTRAL && a.sum_shared_ok && a.batch.count >= 2 &&
            a.batch.count <= SUM_TC_MAX_TOTAL && k <= SUM_TC_MAX_K) {
            SumTcArgs t;
            t.batch = a.batch;
            t.m = m;
            t.n = n;
            t.k = k;
            t.row_blocks = rb_count;
            t.rb_begin = rb_begin;
            t.x1 = a.x1;
            t.x2 = a.x2;
            t.rhs = a.rhs;
            t.params = a.params;
            t.start = a.start;
            t.end = a.end;
            t.out = a.out;
            t.comp_begin = 0;
            t.comp_count = 0;
            const int variant = sum_tc_variant();
            const int rc = phases != nullptr
                               ? launch_matmul_sum_ph(t, phases, phases_bytes, s)
                               : (variant == 1 ? launch_matmul_sum_tc(t, s)
                                               : (variant == 2 ? launch_matmul_sum_tc2(t, s) : launch_matmul_sum_tc3(t, s)));
            if (rc != KM_OK) return rc;
            a.sum_tc_launched = 1;
        }
        switch (kernel_type) {
        case KM_KERNEL_RBF: return dispatch_matmul<KM_KERNEL_RBF, true>(a, s);
        case KM_KERNEL_SPECTRAL: return dispatch_matmul<KM_KERNEL_SPECTRAL, true>(a, s);
        default: return dispatch_matmul<KM_KERNEL_LOCALLY_PERIODIC, true>(a, s);
        }
    }
    switch (kernel_type) {
    case KM_KERNEL_RBF: return dispatch_matmul<KM_KERNEL_RBF, false>(a, s);
    case KM_KERNEL_SPECTRAL: return dispatch_matmul<KM_KERNEL_SPECTRAL, false>(a, s);
    default: return dispatch_matmul<KM_KERNEL_LOCALLY_PERIODIC, false>(a, s);
    }
}

}  // namespace km

extern "C" int km_matmul_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                             const km_view *x1, const km_view *x2, const km_view *rhs,
                             const km_view *params, const km_view *start, const km_view *end,
                             const km_view *out, void *stream) {
    return km::matmul_entry("km_matmul_f32", kernel_type, batch, m, n, k, x1, x2, rhs, params, start, end, out, 0, -1,
                            false, stream);
}

extern "C" int km_matmul_rows_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                                  const km_view *x1, const km_view *x2, const km_view *rhs,
                                  const km_view *params, const km_view *start, const km_view *end,
                                  const km_view *out, int64_t row_block_begin, int64_t row_block_count,
                                  int32_t sum_batches, void *stream) {
    return km::matmul_entry("km_matmul_rows_f32", kernel_type, batch, m, n, k, x1, x2, rhs, params, start, end, out,
                            row_block_begin, row_block_count, sum_batches != 0, stream);
}

extern "C" size_t km_sum_phases_workspace_bytes(const km_batch *batch, int64_t m, int64_t n) {
    km::Batch b;
    if (batch == nullptr || m < 0 || n < 0 || km::make_batch(batch, &b) != KM_OK) return 0;
    return km::sum_phases_workspace_bytes(b.count, m, n);
}

extern "C" int km_sum_phases_prepare_f32(const km_batch *batch, int64_t m, int64_t n, const km_view *x1, const km_view *x2,
                                         const km_view *params, int64_t row_begin, int64_t row_end, int64_t col_begin,
                                         int64_t col_end, void *workspace, size_t workspace_bytes, void *stream) {
    if (row_end < 0) row_end = m;
    if (col_end < 0) col_end = n;
    KM_REQUIRE(0 <= row_begin && row_begin <= row_end && row_end <= m && 0 <= col_begin && col_begin <= col_end && col_end <= n,
               KM_ERR_INVALID_ARGUMENT, "km_sum_phases_prepare_f32: rows [%lld, %lld) of %lld, columns [%lld, %lld) of %lld",
               (long long)row_begin, (long long)row_end, (long long)m, (long long)col_begin, (long long)col_end, (long long)n);
    KM_REQUIRE(batch && x1 && x2 && params, KM_ERR_INVALID_ARGUMENT, "km_sum_phases_prepare_f32: null argument");
    KM_REQUIRE(m >= 0 && n >= 0 && n <= 0x7fffffffLL && m <= 0x7fffffffLL * 64, KM_ERR_INVALID_ARGUMENT,
               "km_sum_phases_prepare_f32: bad sizes m=%lld n=%lld", (long long)m, (long long)n);
    km::Batch b;
    const int rc = km::make_batch(batch, &b);
    if (rc != KM_OK) return rc;
    KM_REQUIRE(b.count >= 1 && b.count <= km::SUM_TC_MAX_TOTAL, KM_ERR_UNSUPPORTED,
               "km_sum_phases_prepare_f32: 1 .. %d components, got %lld", km::SUM_TC_MAX_TOTAL, (long long)b.count);
    if (m == 0 && n == 0) return KM_OK;
    KM_REQUIRE(params->data && (m == 0 || x1->data) && (n == 0 || x2->data), KM_ERR_INVALID_ARGUMENT,
               "km_sum_phases_prepare_f32: null data pointer");
    const km::View<const float> v1 = km::make_view<const float>(x1, b), v2 = km::make_view<const float>(x2, b);
    for (int d = 0; d < b.ndim; d++)
        KM_REQUIRE(b.size[d] <= 1 || (v1.bs[d] == 0 && v2.bs[d] == 0), KM_ERR_UNSUPPORTED,
                   "km_sum_phases_prepare_f32: x1 and x2 must be shared by all components (batch stride 0)");
    return km::sum_phases_prepare(b, km::make_view<const float>(params, b), v1, v2, m, n, row_begin, row_end, col_begin, col_end,
                                  workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int km_matmul_rows_phases_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                                         const km_view *x1, const km_view *x2, const km_view *rhs,
                                         const km_view *params, const km_view *start, const km_view *end,
                                         const km_view *out, int64_t row_block_begin, int64_t row_block_count,
                                         const void *phases, size_t phases_bytes, void *stream) {
    KM_REQUIRE(phases != nullptr, KM_ERR_WORKSPACE, "km_matmul_rows_phases_f32: null workspace");
    return km::matmul_entry("km_matmul_rows_phases_f32", kernel_type, batch, m, n, k, x1, x2, rhs, params, start, end, out,
                            row_block_begin, row_block_count, true, stream, phases, phases_bytes);
}

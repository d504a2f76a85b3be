// Forward product on the 5th-generation tensor cores (tcgen05 + TMEM) for wide right-hand sides.
//
//   out[b, i, :] = sum_{j in band} kappa(x1[b,i], x2[b,j]) * rhs[b, j, :]
//
// is a dense contraction once rhs has tens of columns: per 128-row block it is the GEMM
// D[128 x N] = A[128 x band] . B[band x N] whose A operand (the kernel-matrix tile) never
// exists in memory.  One CTA owns a row block; its threads generate A tiles of 128 x 32 entries
// straight into shared memory in the tensor core's K-major core-matrix layout, a single thread
// issues tcgen05.mma instructions that accumulate into tensor memory, and the generation of
// tile t+1 overlaps the MMAs of tile t (two shared-memory stages, mbarrier hand-off through
// tcgen05.commit).  The rhs tiles arrive as one bulk asynchronous copy per tile
// (cp.async.bulk, the non-tensor form of TMA, completing on an mbarrier) from images that a
// small pre-pass kernel lays out once per call.
//
// Precision: the tensor cores multiply TF32 (10-bit mantissa).  To stay within fp32 accuracy
// both operands are split x = hi + lo with hi the TF32-truncated value and lo the exact
// remainder, and three MMAs hi*hi + hi*lo + lo*hi are issued per K step ("3xTF32"); the
// dropped lo*lo term and the truncation of lo are ~2^-21 relative.  The tensor core adds into
// its fp32 accumulator with truncation, a bias that grows with the number of accumulations
// (measured: 1.5e-5 relative after 750 MMAs), so a tensor-memory accumulator only ever holds
// a group of TC_PROMO tiles (16 hi*hi MMAs, bias < 1e-6): within a tile the small cross terms
// are issued first and the hi*hi MMAs last, and a finished group is added to fp32 registers
// (round-to-nearest) while the next groups are generated -- two accumulators alternate.
//
// Every wait on an mbarrier is bounded; a wait that gives up records a code in the status word
// of the workspace and the CTA leaves through the normal exit (tensor memory released).
#include "km_tcgen05.cuh"

namespace km {

constexpr int TC_BK = 32;             // band columns (GEMM K) per stage
constexpr int TC_STAGES = 3;           // A (and rhs-lo) stages
constexpr int TC_B_STAGES = 5;         // raw rhs tiles in flight / in use
constexpr int TC_B_AHEAD = TC_B_STAGES - TC_STAGES;  // prefetch distance in tiles
constexpr int TC_PROMO = 4;           // tiles accumulated in tensor memory before promotion to registers

// ------------------------------------------------------------------------- rhs images pre-pass

// Writes, for every (slot, k block, 32-column tile), the rhs tile transposed into the K-major
// core-matrix layout: image[chunk = jj / 4][c][jj % 4], c the column inside the k block (the
// tensor core reads the TF32 bits of these words as the "hi" operand; the "lo" operand is
// derived from them in shared memory by the product kernel).  Rows past n and columns past k
// are zero.  Also clears the status word.
__global__ void __launch_bounds__(256) tc_rhs_images_kernel(Batch batch, int64_t slots, int64_t n, int64_t k,
                                                            int64_t tiles, int k_blocks, int n_pad,
                                                            View<const float> rhs, float *images, int *status) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *status = 0;
    const int64_t per_tile = (int64_t)TC_BK * n_pad;
    const int64_t total = slots * k_blocks * tiles * (int64_t)TC_BK * n_pad;
    for (int64_t idx = blockIdx.x * 256LL + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * 256) {
        // idx -> (slot, kb, tile, jj, c) with c fastest: coalesced reads of rhs rows
        int64_t rem = idx;
        const int c = (int)(rem % n_pad);
        rem /= n_pad;
        const int jj = (int)(rem % TC_BK);
        rem /= TC_BK;
        const int64_t tile = rem % tiles;
        rem /= tiles;
        const int kb = (int)(rem % k_blocks);
        const int64_t slot = rem / k_blocks;
        const int64_t j = tile * TC_BK + jj;
        const int64_t col = (int64_t)kb * n_pad + c;
        float v = 0.0f;
        if (j < n && col < k) {
            const BatchIndex bi = decompose(batch, slot);
            v = batch_ptr(rhs, bi)[j * rhs.s0 + col * rhs.s1];
        }
        float *img = images + ((slot * k_blocks + kb) * tiles + tile) * per_tile;
        img[(int64_t)(jj >> 2) * (n_pad * 4) + c * 4 + (jj & 3)] = v;
    }
}

// ----------------------------------------------------------------------------------- kernel

// N = GEMM N (rhs columns per CTA, 64 or 128).  128 * G generator threads + one MMA warp.
//
// Generator thread (row = tid % 128, g = tid / 128) produces the columns
// [g * 32 / G, (g + 1) * 32 / G) of its row in every A tile, derives its share of the rhs "lo"
// tile, and owns the output columns [g * N / G, (g + 1) * N / G) of its row in registers.  The
// MMA warp (one lane) fetches rhs tiles ahead of time and issues the MMAs.  The two sides meet
// only through mbarriers -- there is no CTA-wide barrier inside the band loop:
//   bar_full[bs]   raw rhs tile landed (bulk copy transaction count)   MMA warp -> generators
//   bar_ready[s]   A tile and rhs-lo tile of stage s written           generators -> MMA warp
//   bar_empty[s]   MMAs that read stage s are done (tcgen05.commit)     tensor core -> everyone
//   bar_acc[ai]    a group of tiles is complete in accumulator ai      tensor core -> generators
//   bar_free[ai]   accumulator ai has been added to the registers      generators -> MMA warp
template <int KT, int N, int G>
__global__ void __launch_bounds__(128 * G + 32) matmul_tc_kernel(const TcArgs a) {
    constexpr int GEN_THREADS = 128 * G;
    constexpr int GEN_WARPS = 4 * G;
    constexpr int A_PART = 128 * TC_BK;  // floats per hi / lo part of an A stage
    constexpr int B_TILE = TC_BK * N;    // floats per rhs tile image
    constexpr int NPT = N / G;           // accumulator columns per thread
    constexpr int CPT = TC_BK / 4 / G;   // 4-column chunks generated per thread and tile
    static_assert(NPT % 16 == 0, "columns per thread must be a multiple of 16");
    static_assert((B_TILE / 4) % GEN_THREADS == 0, "rhs tile must split evenly over the threads");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[TC_B_STAGES];
    __shared__ __align__(8) uint64_t bar_ready[TC_STAGES];
    __shared__ __align__(8) uint64_t bar_empty[TC_STAGES];
    __shared__ __align__(8) uint64_t bar_acc[2];
    __shared__ __align__(8) uint64_t bar_free[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int fail_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const bool is_mma_warp = warp == GEN_WARPS;
    const int row_local = tid & 127;
    const int g = (tid >> 7) % G;

    // shared memory: [A hi | A lo | rhs lo] x TC_STAGES, then TC_B_STAGES raw rhs tiles
    float *smem_f = reinterpret_cast<float *>(smem_raw);
    constexpr int STAGE_FLOATS = 2 * A_PART + B_TILE;
    auto a_hi = [&](int s) { return smem_f + s * STAGE_FLOATS; };
    auto a_lo = [&](int s) { return smem_f + s * STAGE_FLOATS + A_PART; };
    auto b_lo = [&](int s) { return smem_f + s * STAGE_FLOATS + 2 * A_PART; };
    auto b_raw = [&](int bs) { return smem_f + TC_STAGES * STAGE_FLOATS + bs * B_TILE; };

    // work item
    int64_t item = blockIdx.x;
    const int64_t b = item % a.batch.count;
    item /= a.batch.count;
    const int64_t r = a.rb_begin + item % a.row_blocks;
    const int kb = (int)(item / a.row_blocks);

    const BatchIndex bi = decompose(a.batch, b);
    const float *x1 = batch_ptr(a.x1, bi);
    const float *x2 = batch_ptr(a.x2, bi);
    float *out = batch_ptr(a.out, bi);
    KernelFn<KT> fn;
    fn.init(batch_ptr(a.params, bi), a.params.s0);

    const int n = (int)a.n;
    const int band_lo = clamp_int(batch_ptr(a.start, bi)[r * a.start.s0], 0, n);
    const int band_hi = max(band_lo, min(batch_ptr(a.end, bi)[r * a.end.s0], n));
    const int tile_lo = band_lo / TC_BK;
    const int tile_hi = (band_hi + TC_BK - 1) / TC_BK;  // exclusive
    const int tiles = band_hi > band_lo ? tile_hi - tile_lo : 0;
    const float *images = a.images + (a.image_slot_stride ? b * a.image_slot_stride : 0) +
                          (int64_t)kb * a.tiles * (int64_t)B_TILE;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < TC_B_STAGES; s++) mbar_init(&bar_full[s], 1);
#pragma unroll
        for (int s = 0; s < TC_STAGES; s++) {
            mbar_init(&bar_ready[s], GEN_WARPS);
            mbar_init(&bar_empty[s], 1);
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            mbar_init(&bar_acc[i], 1);
            mbar_init(&bar_free[i], GEN_WARPS);
        }
        fail_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (is_mma_warp) tmem_alloc(&tmem_base_slot, (unsigned)a.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    // instruction descriptor: D fp32, A / B tf32, both K-major, M = 128, N
    constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
    constexpr uint32_t img_bytes = B_TILE * sizeof(float);
    bool failed = false;

    float acc[NPT];
#pragma unroll
    for (int c = 0; c < NPT; c++) acc[c] = 0.0f;

    if (is_mma_warp) {
        // ------------------------------------------------------------ rhs fetch + MMA issue
        if (lane == 0) {
            auto fetch_rhs = [&](int t) {
                const int bs = t % TC_B_STAGES;
                mbar_expect_tx(&bar_full[bs], img_bytes);
                bulk_copy_g2s(b_raw(bs), images + (int64_t)(tile_lo + t) * B_TILE, img_bytes, &bar_full[bs]);
            };
            for (int t = 0; t < min(tiles, TC_B_AHEAD); t++) fetch_rhs(t);
            // Shared-memory descriptors: built once; per tile only the 14-bit start-address field
            // moves (by whole stages), per K step by two core-matrix columns.  This thread is the
            // only one issuing MMAs, so its instruction count per tile is on the critical path.
            constexpr uint32_t lbo_a = 128 * 16, lbo_b = N * 16, sbo = 128;
            constexpr uint64_t stage_step = (uint64_t)(STAGE_FLOATS * 4) >> 4;
            constexpr uint64_t braw_step = (uint64_t)(B_TILE * 4) >> 4;
            constexpr uint64_t ks_a = (uint64_t)(2 * lbo_a) >> 4, ks_b = (uint64_t)(2 * lbo_b) >> 4;
            const uint64_t d_ah0 = smem_desc(smem_u32(a_hi(0)), lbo_a, sbo);
            const uint64_t d_al0 = smem_desc(smem_u32(a_lo(0)), lbo_a, sbo);
            const uint64_t d_bl0 = smem_desc(smem_u32(b_lo(0)), lbo_b, sbo);
            const uint64_t d_br0 = smem_desc(smem_u32(b_raw(0)), lbo_b, sbo);
            int s = 0, use = 0, bs = 0, in_grp = 0, grp = 0;  // ring counters of tile t
            for (int t = 0; t < tiles; t++) {
                const int ai = grp & 1;
                const bool grp_first = in_grp == 0;
                const bool grp_last = in_grp == TC_PROMO - 1 || t == tiles - 1;
                // stage s (and the raw-rhs buffer of tile t - TC_STAGES) is free once its MMAs are done
                if (use > 0 && !mbar_wait(&bar_empty[s], (unsigned)((use - 1) & 1))) failed = true;
                if (!failed && t + TC_B_AHEAD < tiles) fetch_rhs(t + TC_B_AHEAD);
                // the accumulator must have been collected by every generator warp
                if (!failed && grp_first && grp >= 2 && !mbar_wait(&bar_free[ai], (unsigned)(((grp >> 1) - 1) & 1))) failed = true;
                if (!failed && !mbar_wait(&bar_ready[s], (unsigned)(use & 1))) failed = true;
                if (failed) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(ai * N);
                const uint64_t dah = d_ah0 + s * stage_step, dal = d_al0 + s * stage_step;
                const uint64_t dbl = d_bl0 + s * stage_step, dbh = d_br0 + bs * braw_step;
                // cross terms first (tiny accumulator, truncation irrelevant), hi * hi last
#pragma unroll
                for (int ks = 0; ks < TC_BK / 8; ks++) {
                    mma_tf32(d_tmem, dah + ks * ks_a, dbl + ks * ks_b, idesc, (ks > 0 || !grp_first) ? 1u : 0u);
                    mma_tf32(d_tmem, dal + ks * ks_a, dbh + ks * ks_b, idesc, 1u);
                }
#pragma unroll
                for (int ks = 0; ks < TC_BK / 8; ks++) mma_tf32(d_tmem, dah + ks * ks_a, dbh + ks * ks_b, idesc, 1u);
                mma_commit(&bar_empty[s]);
                if (grp_last) mma_commit(&bar_acc[ai]);
                // advance the ring counters
                if (++s == TC_STAGES) {
                    s = 0;
                    use++;
                }
                if (++bs == TC_B_STAGES) bs = 0;
                if (++in_grp == TC_PROMO) {
                    in_grp = 0;
                    grp++;
                }
            }
            if (failed) atomicExch(&fail_flag, 1);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------- generators
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        const float x1v = row < a.m ? x1[row * a.x1.s0] : 0.0f;
        const uint32_t tmem_mine = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(g * NPT);

        auto collect = [&](int ai) {
            tc_fence_after();
            uint32_t v[NPT / 16][16];
#pragma unroll
            for (int q = 0; q < NPT / 16; q++) tmem_ld16_nowait(tmem_mine + (uint32_t)(ai * N + q * 16), v[q]);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < NPT / 16; q++)
#pragma unroll
                for (int u = 0; u < 16; u++) acc[q * 16 + u] += __uint_as_float(v[q][u]);
            tc_fence_before();
        };
        // x2 values of this thread's columns, fetched one tile ahead
        auto load_x2 = [&](int jt, float (&xv)[CPT][4]) {
#pragma unroll
            for (int q = 0; q < CPT; q++)
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int j = jt * TC_BK + (g * CPT + q) * 4 + u;
                    xv[q][u] = j < n ? __ldg(x2 + (int64_t)j * a.x2.s0) : 0.0f;
                }
        };
        float xnext[CPT][4];
        if (tiles > 0) load_x2(tile_lo, xnext);

        for (int t = 0; t < tiles; t++) {
            const int s = t % TC_STAGES, use = t / TC_STAGES, bs = t % TC_B_STAGES;
            const int jt = tile_lo + t;
            const int grp = t / TC_PROMO, ai = grp & 1;
            float xv[CPT][4];
#pragma unroll
            for (int q = 0; q < CPT; q++)
#pragma unroll
                for (int u = 0; u < 4; u++) xv[q][u] = xnext[q][u];
            if (t + 1 < tiles) load_x2(jt + 1, xnext);

            // an accumulator that is about to be reused is first added to the registers
            if ((t % TC_PROMO) == 0 && grp >= 2) {
                if (!mbar_wait(&bar_acc[ai], (unsigned)((grp / 2 - 1) & 1))) {
                    failed = true;
                    break;
                }
                collect(ai);
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_free[ai]);
            }
            // stage s must have been read by the MMAs of tile t - TC_STAGES
            if (use > 0 && !mbar_wait(&bar_empty[s], (unsigned)((use - 1) & 1))) {
                failed = true;
                break;
            }
            // kernel entries: this thread's row, its share of the 32 columns, 4 at a time
            const int j0 = jt * TC_BK;
            const bool partial = (j0 < band_lo) || (j0 + TC_BK > band_hi);
            float *ah = a_hi(s), *al = a_lo(s);
#pragma unroll
            for (int q = 0; q < CPT; q++) {
                const int chunk = g * CPT + q;
                float kv[4], lo[4];
#pragma unroll
                for (int u = 0; u < 4; u++) kv[u] = fn.unscaled(x1v - xv[q][u]);
                if (partial) {
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int j = j0 + chunk * 4 + u;
                        if (j < band_lo || j >= band_hi) kv[u] = 0.0f;
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; u++) lo[u] = kv[u] - tf32_hi(kv[u]);
                // [chunk][row][16 bytes]: the tensor core reads only the TF32 bits of kv as "hi"
                *reinterpret_cast<float4 *>(ah + (chunk * 128 + row_local) * 4) = make_float4(kv[0], kv[1], kv[2], kv[3]);
                *reinterpret_cast<float4 *>(al + (chunk * 128 + row_local) * 4) = make_float4(lo[0], lo[1], lo[2], lo[3]);
            }
            // lo part of the rhs tile (the raw tile itself serves as hi)
            if (!mbar_wait(&bar_full[bs], (unsigned)((t / TC_B_STAGES) & 1))) {
                failed = true;
                break;
            }
            {
                const float4 *raw = reinterpret_cast<const float4 *>(b_raw(bs));
                float4 *lo4 = reinterpret_cast<float4 *>(b_lo(s));
#pragma unroll
                for (int q = 0; q < B_TILE / 4 / GEN_THREADS; q++) {
                    const float4 v = raw[q * GEN_THREADS + tid];
                    lo4[q * GEN_THREADS + tid] =
                        make_float4(v.x - tf32_hi(v.x), v.y - tf32_hi(v.y), v.z - tf32_hi(v.z), v.w - tf32_hi(v.w));
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_ready[s]);
        }

        // drain: the last two groups still sit in tensor memory
        const int groups = (tiles + TC_PROMO - 1) / TC_PROMO;
        for (int grp = max(0, groups - 2); grp < groups && !failed; grp++) {
            if (!mbar_wait(&bar_acc[grp & 1], (unsigned)((grp / 2) & 1))) {
                failed = true;
                break;
            }
            collect(grp & 1);
        }
        if (failed) atomicExch(&fail_flag, 1);
    }

    tc_fence_before();
    __syncthreads();
    if (fail_flag) {
        if (tid == 0) atomicExch(a.status, 1);
    } else if (!is_mma_warp) {
        // Output.  Each thread holds NPT consecutive columns of one row; a warp transposes its
        // 32 x NPT block through shared memory (the stages are idle now) so that every store
        // instruction writes whole 128-byte row segments.
        const float scale = fn.scale;
        const int64_t row0 = r * KM_BLOCK_SIZE + (warp & 3) * 32;  // first row of this warp
        const int64_t out_row0 = row0 - a.rb_begin * KM_BLOCK_SIZE;
        const int64_t col0 = (int64_t)kb * N + g * NPT;
        constexpr int PITCH = NPT + 4;  // floats; keeps float4 alignment, staggers banks
        float *tile = smem_f + warp * (32 * PITCH);
#pragma unroll
        for (int c = 0; c < NPT; c += 4)
            *reinterpret_cast<float4 *>(tile + lane * PITCH + c) =
                make_float4(acc[c] * scale, acc[c + 1] * scale, acc[c + 2] * scale, acc[c + 3] * scale);
        __syncwarp();
        const bool vec_ok = a.out.s1 == 1 && (a.out.s0 % 4 == 0) && (col0 + NPT <= a.k) &&
                            ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
        constexpr int V = NPT / 4;          // float4 per row
        constexpr int ROWS_PER_IT = 32 / V;  // rows written per store instruction
        if (vec_ok) {
#pragma unroll
            for (int it = 0; it < 32 / ROWS_PER_IT; it++) {
                const int rr = it * ROWS_PER_IT + lane / V, cc = (lane % V) * 4;
                if (row0 + rr < a.m)
                    *reinterpret_cast<float4 *>(out + (out_row0 + rr) * a.out.s0 + col0 + cc) =
                        *reinterpret_cast<const float4 *>(tile + rr * PITCH + cc);
            }
        } else {
            for (int rr = 0; rr < 32; rr++) {
                if (row0 + rr >= a.m) break;
                for (int cc = lane; cc < NPT; cc += 32)
                    if (col0 + cc < a.k) out[(out_row0 + rr) * a.out.s0 + (col0 + cc) * a.out.s1] = tile[rr * PITCH + cc];
            }
        }
    }
    if (is_mma_warp) tmem_free(tmem_base, (unsigned)a.tmem_cols);
}

static int tc_n_pad(int64_t k) { return k <= 64 ? 64 : 128; }

template <int KT, int N, int G>
static int launch_tc_n(const TcArgs &a, cudaStream_t s) {
    const int64_t items = a.batch.count * a.row_blocks * a.k_blocks;
    if (items > 0x7fffffffLL) {
        set_error("km_matmul_tc_f32: too many work items (%lld)", (long long)items);
        return KM_ERR_UNSUPPORTED;
    }
    constexpr size_t smem = ((size_t)TC_STAGES * (2 * 128 * TC_BK + TC_BK * N) + (size_t)TC_B_STAGES * TC_BK * N) * sizeof(float);
    auto kernel = matmul_tc_kernel<KT, N, G>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(matmul_tc)");
    kernel<<<(unsigned)items, 128 * G + 32, smem, s>>>(a);
    KM_CHECK_LAUNCH("km_matmul_tc_f32 launch");
    return KM_OK;
}

template <int KT>
static int launch_tc(const TcArgs &a, cudaStream_t s) {
    if (a.n_pad == 64) return launch_tc_n<KT, 64, 2>(a, s);
    return launch_tc_n<KT, 128, 4>(a, s);
}

}  // namespace km

extern "C" size_t km_matmul_tc_workspace_bytes(const km_batch *batch, int64_t n, int64_t k, const km_view *rhs) {
    using namespace km;
    Batch b;
    if (batch == nullptr || rhs == nullptr || make_batch(batch, &b) != KM_OK || n < 0 || k <= 0) return 0;
    const View<const float> rv = make_view<const float>(rhs, b);
    if (k <= TCN_MAX_K) return tcn_workspace_bytes(b, n, rv);
    const int n_pad = tc_n_pad(k);
    const int64_t k_blocks = ceil_div(k, n_pad);
    const int64_t tiles = ceil_div(n, TC_BK);
    return (size_t)TC_STATUS_BYTES + (size_t)(tc_slots(b, rv) * k_blocks * tiles) * (TC_BK * n_pad) * sizeof(float);
}

extern "C" int km_matmul_tc_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                                const km_view *x1, const km_view *x2, const km_view *rhs, const km_view *params,
                                const km_view *start, const km_view *end, const km_view *out, void *workspace,
                                size_t workspace_bytes, void *stream) {
    using namespace km;
    const char *name = "km_matmul_tc_f32";
    KM_REQUIRE(valid_kernel_type(kernel_type), KM_ERR_INVALID_ARGUMENT, "%s: unknown kernel type %d", name, kernel_type);
    KM_REQUIRE(batch && x1 && x2 && rhs && params && start && end && out, KM_ERR_INVALID_ARGUMENT, "%s: null argument", name);
    KM_REQUIRE(m >= 0 && n >= 0 && k >= 0 && n <= 0x7fffffffLL - 64 && m <= 0x7fffffffLL * 64, KM_ERR_INVALID_ARGUMENT,
               "%s: bad sizes", name);
    TcArgs a;
    int rc = make_batch(batch, &a.batch);
    if (rc != KM_OK) return rc;
    if (a.batch.count == 0 || m == 0 || k == 0) return KM_OK;
    KM_REQUIRE(x1->data && out->data && params->data && start->data && end->data, KM_ERR_INVALID_ARGUMENT,
               "%s: null data pointer", name);
    KM_REQUIRE(n == 0 || (x2->data && rhs->data), KM_ERR_INVALID_ARGUMENT, "%s: null data pointer", name);
    const size_t need = km_matmul_tc_workspace_bytes(batch, n, k, rhs);
    KM_REQUIRE(workspace != nullptr && workspace_bytes >= need, KM_ERR_WORKSPACE,
               "%s: workspace of %zu bytes needed, %zu given", name, need, workspace_bytes);
    KM_REQUIRE((uintptr_t)workspace % 256 == 0, KM_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned", name);
    a.m = m;
    a.n = n;
    a.k = k;
    a.row_blocks = ceil_div(m, KM_BLOCK_SIZE);
    a.rb_begin = 0;
    a.col_inv_scale = nullptr;
    a.n_pad = tc_n_pad(k);
    a.k_blocks = (int)ceil_div(k, a.n_pad);
    a.tmem_cols = 32;  // two accumulators of n_pad columns, rounded up to a power of two
    while (a.tmem_cols < TC_STAGES * a.n_pad) a.tmem_cols *= 2;
    a.tiles = ceil_div(n, TC_BK);
    a.x1 = make_view<const float>(x1, a.batch);
    a.x2 = make_view<const float>(x2, a.batch);
    a.params = make_view<const float>(params, a.batch);
    a.start = make_view<const int>(start, a.batch);
    a.end = make_view<const int>(end, a.batch);
    a.out = make_view<float>(out, a.batch);
    const View<const float> rv = make_view<const float>(rhs, a.batch);
    if (k <= TCN_MAX_K) return tcn_matmul(kernel_type, a, rv, workspace, static_cast<cudaStream_t>(stream));
    const int64_t slots = tc_slots(a.batch, rv);
    a.status = static_cast<int *>(workspace);
    float *images = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + TC_STATUS_BYTES);
    a.images = images;
    a.image_slot_stride = slots > 1 ? (int64_t)a.k_blocks * a.tiles * ((int64_t)TC_BK * a.n_pad) : 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    const int64_t total = slots * a.k_blocks * a.tiles * (int64_t)TC_BK * a.n_pad;
    const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(total, 256), 148 * 32));
    tc_rhs_images_kernel<<<blocks, 256, 0, s>>>(a.batch, slots, n, k, a.tiles, a.k_blocks, a.n_pad, rv, images, a.status);
    KM_CHECK_LAUNCH("km_matmul_tc_f32 pre-pass launch");
    switch (kernel_type) {
    case KM_KERNEL_RBF: return launch_tc<KM_KERNEL_RBF>(a, s);
    case KM_KERNEL_SPECTRAL: return launch_tc<KM_KERNEL_SPECTRAL>(a, s);
    default: return launch_tc<KM_KERNEL_LOCALLY_PERIODIC>(a, s);
    }
}

extern "C" int km_workspace_status(const void *workspace, int32_t *status_out, void *stream) {
    using namespace km;
    KM_REQUIRE(workspace && status_out, KM_ERR_INVALID_ARGUMENT, "km_workspace_status: null argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemcpyAsync(status_out, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost, s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    if (err != cudaSuccess) return cuda_fail(err, "km_workspace_status");
    return KM_OK;
}

// Hyper-parameter gradients with the coefficients on the tensor cores.
//
//   grad[b, q] = d/d theta_q  sum_{i, j in band} coeff[i, j] * kappa(x1[b,i], x2[b,j]),
//   coeff[i, j] = <left[b, i, :], right[b, j, :]>
//
// The coefficient tile of a 128-row block against 64 band columns is a small GEMM,
// C[128 x 64] = L[128 x k] . R[64 x k]^T, which the FMA-pipe kernel (km_grad.cu) pays for with k
// FMAs per entry.  Here one lane of a control warp issues it as tcgen05.mma (3xTF32: hi*lo,
// lo*hi, hi*hi; left rows staged once per CTA in shared memory, right tiles arriving as bulk
// copies of images laid out by a pre-pass) into a tensor-memory stage, while the 128 * G consumer
// threads -- one tensor-memory lane = one row each -- read the previous stage with tcgen05.ld,
// evaluate the factors of d kappa / d p per entry and add coeff * factor to their running sums.
// Sines and cosines of the phase difference come from per-row and per-column factors (the
// control warp computes those of a tile's 64 columns), so an entry costs ONE SFU operation.
// (Up to 64 columns per CTA; wider operands are processed in column blocks of 64, whose partial
// sums add up because the coefficient is linear in the columns.)
// Per entry the FP32 pipe runs ~11 operations instead of k + 11, issued as packed f32x2
// instructions for two entries at a time, so the kernel is bound by the SFU operations of kappa
// (3 per spectral entry).
//
// Reduction and chain rule are those of km_grad.cu: one partial record per (batch, row block),
// then the fixed-order fp64 sum of launch_grad_finish.  Every mbarrier wait is bounded; a
// give-up is reported through the status word of the workspace and makes the CTA's partial
// record, and so the gradient of its batch, NaN.
#include <type_traits>

#include "km_tcgen05.cuh"

namespace km {

constexpr int GT_COLS = 64;       // band columns per tile = GEMM N
constexpr int GT_D_STAGES = 2;    // coefficient tiles in tensor memory
constexpr int GT_MAX_SLOTS = 4;   // right / x2 slots in shared memory
constexpr int GT_TMEM_COLS = GT_D_STAGES * GT_COLS;
constexpr int GT_MAX_KP = 64;     // GEMM K per CTA; more columns are processed in blocks of 64

struct GradTcArgs {
    Batch batch;
    int64_t m, n, k;
    int kp;     // GEMM K per column block: min(k, 64) rounded up to a multiple of 8
    int kblocks;  // column blocks (ceil(k / 64))
    int64_t tiles_total;  // 64-column tiles of the whole band range: ceil(n / 64)
    int slots;  // shared-memory slots in use (<= GT_MAX_SLOTS)
    int64_t row_blocks;
    View<const float> x1, x2, left, params;
    View<const int> start, end;
    const float *images;        // [image slot][column block][tile][part: hi, lo][chunk = c / 4][j][c % 4]
    int64_t image_slot_stride;  // floats between batch slots (0: right shared by all batches)
    float *partials;            // [batch.count][row_blocks][kblocks][KM_MAX_PARAMS]
    int *status;
    unsigned wait_polls;        // poll limit of every hand-off wait
};

// Pre-pass: right -> per (image slot, 64-column tile) the K-major core-matrix layout of a B
// operand with N = band column, K = rhs column: image[part][c / 4][j][c % 4].  hi is the raw
// fp32 word (the tensor core reads its TF32 bits), lo = x - trunc_tf32(x); rows past n and
// columns past k are zero.  Also clears the status word.
__global__ void __launch_bounds__(256) grad_tc_images_kernel(Batch batch, int64_t slots, int64_t n, int64_t k, int kp,
                                                             int kblocks, int64_t tiles, View<const float> right,
                                                             float *images, int *status) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *status = 0;
    const int64_t img_floats = 2LL * kp * GT_COLS;
    const int64_t total = slots * kblocks * tiles * (int64_t)GT_COLS * kp;
    for (int64_t idx = blockIdx.x * 256LL + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * 256) {
        int64_t rem = idx;
        const int c = (int)(rem % kp);
        rem /= kp;
        const int jj = (int)(rem % GT_COLS);
        rem /= GT_COLS;
        const int64_t tile = rem % tiles;
        rem /= tiles;
        const int kb = (int)(rem % kblocks);
        const int64_t slot = rem / kblocks;
        const int64_t j = tile * GT_COLS + jj;
        const int64_t col = (int64_t)kb * kp + c;
        float v = 0.0f;
        if (j < n && col < k) {
            const BatchIndex bi = decompose(batch, slot);
            v = batch_ptr(right, bi)[j * right.s0 + col * right.s1];
        }
        float *img = images + ((slot * kblocks + kb) * tiles + tile) * img_floats;
        const int at = (c >> 2) * (GT_COLS * 4) + jj * 4 + (c & 3);
        img[at] = v;
        img[kp * GT_COLS + at] = v - tf32_hi(v);
    }
}

// G consumer groups of 128 threads (group g takes the columns [g * 64 / G, (g + 1) * 64 / G) of
// every tile) + one control warp.
#ifndef GT_MIN_CTAS
#define GT_MIN_CTAS 4
#endif
template <int KT, int G>
__global__ void __launch_bounds__(128 * G + 32, G == 4 ? 2 : GT_MIN_CTAS) grad_tc_kernel(const GradTcArgs a) {
    constexpr int WARPS = 4 * G;
    constexpr int NS = KernelFn<KT>::NSUMS;
    constexpr int CPT = GT_COLS / G;   // columns per thread and tile
    constexpr int PIECES = CPT / 16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[GT_MAX_SLOTS];   // right image + x2 of a slot landed
    __shared__ __align__(8) uint64_t bar_dfull[GT_D_STAGES];   // coefficient tile complete (tcgen05.commit)
    __shared__ __align__(8) uint64_t bar_dfree[GT_D_STAGES];   // coefficient tile consumed
    __shared__ __align__(8) uint64_t bar_drain;                // give-up path: every issued MMA has completed
    __shared__ uint32_t tmem_base_slot;
    __shared__ int fail_flag;
    __shared__ float warp_sums[WARPS][KM_MAX_PARAMS];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const bool is_ctl_warp = warp == WARPS;
    const int kp = a.kp;
    const int ns = a.slots;

    // shared memory: left rows [part][chunk][row][4], then the slots (image, x2)
    float *smem_f = reinterpret_cast<float *>(smem_raw);
    const int left_floats = 2 * kp * 128;
    const int img_floats = 2 * kp * GT_COLS;
    const int slot_floats = img_floats + 3 * GT_COLS;  // image, then per column x2, cos and sin of its phase
    auto slot_img = [&](int sl) { return smem_f + left_floats + sl * slot_floats; };
    auto slot_x2 = [&](int sl) { return smem_f + left_floats + sl * slot_floats + img_floats; };

    int64_t item = blockIdx.x;
    const int64_t b = item % a.batch.count;
    item /= a.batch.count;
    const int64_t r = item % a.row_blocks;
    const int kb = (int)(item / a.row_blocks);  // block of kp columns of left / right

    const BatchIndex bi = decompose(a.batch, b);
    const float *x1 = batch_ptr(a.x1, bi);
    const float *x2 = batch_ptr(a.x2, bi);
    const float *left = batch_ptr(a.left, bi);
    KernelFn<KT> fn;
    fn.init(batch_ptr(a.params, bi), a.params.s0);

    const int n = (int)a.n;
    const int band_lo = clamp_int(batch_ptr(a.start, bi)[r * a.start.s0], 0, n);
    const int band_hi = max(band_lo, min(batch_ptr(a.end, bi)[r * a.end.s0], n));
    const int tile_lo = band_lo / GT_COLS;
    const int tiles = band_hi > band_lo ? (band_hi + GT_COLS - 1) / GT_COLS - tile_lo : 0;
    // origin of the separable phases: the middle row of the block (keeps |x - x0| as small as tau)
    const float x0 = x1[min(r * KM_BLOCK_SIZE + KM_BLOCK_SIZE / 2, a.m - 1) * a.x1.s0];
    const float phase_w = fn.phase_w();
    const float *images = a.images + (a.image_slot_stride ? b * a.image_slot_stride : 0) +
                          (int64_t)kb * a.tiles_total * (2LL * a.kp * GT_COLS);

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < GT_MAX_SLOTS; s++) mbar_init(&bar_full[s], 2);  // expect_tx arrival + lane 0 after the warp's stores
#pragma unroll
        for (int s = 0; s < GT_D_STAGES; s++) {
            mbar_init(&bar_dfull[s], 1);
            mbar_init(&bar_dfree[s], WARPS);
        }
        mbar_init(&bar_drain, 1);
        fail_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (is_ctl_warp) tmem_alloc(&tmem_base_slot, GT_TMEM_COLS);

    // left rows of this row block -> A operand images (hi, lo); rows past m / columns past k are zero
    if (!is_ctl_warp) {
        const int row_local = tid & 127;
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        for (int kc = tid >> 7; kc < kp / 4; kc += G) {
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int64_t c = (int64_t)kb * kp + kc * 4 + u;  // column of left
                v[u] = (row < a.m && c < a.k) ? left[row * a.left.s0 + c * a.left.s1] : 0.0f;
            }
            float *dst = smem_f + (kc * 128 + row_local) * 4;
            *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4 *>(dst + kp * 128) =
                make_float4(v[0] - tf32_hi(v[0]), v[1] - tf32_hi(v[1]), v[2] - tf32_hi(v[2]), v[3] - tf32_hi(v[3]));
        }
        fence_async_smem();
    }
    tc_fence_before();
    // The separable form evaluates sine / cosine at W (x - x0) instead of W tau.  Entries that
    // matter have a small tau, but a row of an unsorted block can be far from x0, and the fp32
    // phase then carries an error no envelope damps: such a block keeps the per-entry evaluation.
    bool use_ph = false;
    {
        const int64_t row = r * KM_BLOCK_SIZE + (tid & 127);
        const bool far = KernelFn<KT>::PHASE && tid < 128 && row < a.m &&
                         fabsf(phase_w * (x1[row * a.x1.s0] - x0)) > KM_PHASE_MAX_ROW_ARG;
        const int any_far = __syncthreads_or(far ? 1 : 0);
        use_ph = KernelFn<KT>::PHASE && !any_far;
    }
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    bool failed = false;
    f32x2 sums2[NS];  // two partial sums per raw sum (packed FP32 arithmetic)
#pragma unroll
    for (int q = 0; q < NS; q++) sums2[q] = 0ull;

    if (is_ctl_warp) {
        // -------------------------------------------- slot fetches (all lanes) + MMA issue (lane 0)
        const uint32_t img_bytes = (uint32_t)img_floats * sizeof(float);
        // Tiles are fetched in increasing order: the x2 values of the next fetch wait in registers
        // (loaded one fetch ahead, so the load latency never stalls the warp that issues the MMAs).
        float x_ahead[GT_COLS / 32];
        auto load_ahead = [&](int t) {
#pragma unroll
            for (int u = 0; u < GT_COLS / 32; u++) {
                const int64_t j = (int64_t)(tile_lo + t) * GT_COLS + lane + 32 * u;
                x_ahead[u] = (t < tiles && j < n) ? __ldg(x2 + j * a.x2.s0) : 0.0f;
            }
        };
        load_ahead(0);
        int fetched = 0, landed = 0;  // tiles whose copies were issued / (set when a wait gives up) were seen complete
        auto fetch = [&](int t) {
            fetched = t + 1;
            const int sl = t % ns;
            const int64_t tile = tile_lo + t;
            if (lane == 0) {
                mbar_expect_tx(&bar_full[sl], img_bytes);
                bulk_copy_g2s(slot_img(sl), images + tile * img_floats, img_bytes, &bar_full[sl]);
            }
            // per column: x2 and the separable phase factors cos / sin(W (x2 - x0)), two columns per lane
            float *xs = slot_x2(sl);
#pragma unroll
            for (int u = 0; u < GT_COLS / 32; u++) {
                const int jj = lane + 32 * u;
                const float xv = x_ahead[u];
                xs[jj] = xv;
                if (use_ph) {
                    const float ph = phase_w * (xv - x0);
                    xs[GT_COLS + jj] = cos_approx(ph);
                    xs[2 * GT_COLS + jj] = sin_approx(ph);
                }
            }
            load_ahead(t + 1);
            __syncwarp();  // the stores of all lanes precede lane 0's (releasing) arrival
            if (lane == 0) mbar_arrive(&bar_full[sl]);
        };
        for (int t = 0; t < min(tiles, ns); t++) fetch(t);

        constexpr uint32_t idesc =
            (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(GT_COLS >> 3) << 17) | ((128u >> 4) << 24);
        constexpr uint32_t lbo_a = 128 * 16, lbo_b = GT_COLS * 16, sbo = 128;
        constexpr uint64_t ks_a = (uint64_t)(2 * lbo_a) >> 4, ks_b = (uint64_t)(2 * lbo_b) >> 4;
        const uint64_t a_part = (uint64_t)(kp * 128 * 4) >> 4, b_part = (uint64_t)(kp * GT_COLS * 4) >> 4;
        const uint64_t slot_step = (uint64_t)(slot_floats * 4) >> 4;
        const uint64_t d_a0 = smem_desc(smem_u32(smem_f), lbo_a, sbo);
        const uint64_t d_b0 = smem_desc(smem_u32(slot_img(0)), lbo_b, sbo);
        const int ksteps = kp / 8;
        static_assert(GT_MAX_KP == 64, "the MMA issue code covers 1 .. 8 k-steps");
        for (int t = 0; t < tiles; t++) {
            const int sl = t % ns;
            const int ds = t & 1;
            bool ok = true;
            // the stage is free once tile t - 2 has been consumed; that also frees its slot
            if (t >= GT_D_STAGES) {
                ok = mbar_wait(&bar_dfree[ds], (unsigned)(((t >> 1) - 1) & 1), a.wait_polls);
                if (__all_sync(0xffffffffu, ok) && t - GT_D_STAGES + ns < tiles) fetch(t - GT_D_STAGES + ns);
            }
            if (ok) ok = mbar_wait(&bar_full[sl], (unsigned)((t / ns) & 1), a.wait_polls);
            if (!__all_sync(0xffffffffu, ok)) {
                failed = true;
                landed = t;
                break;
            }
            tc_fence_after();
            if (lane == 0) {
                const uint32_t d_tmem = tmem_base + (uint32_t)(ds * GT_COLS);
                // The MMAs of a tile are issued from straight-line code chosen by the number of
                // k-steps.  As a loop with a run-time trip count the compiler unrolled them partially
                // (by two or four), and that form produced wrong coefficient tiles as soon as the
                // unrolled body ran; a rolled loop and the fully unrolled form are both correct, the
                // latter ~15 % faster for wide operands (the MMA issue rate bounds those).
                const uint64_t ah = d_a0, al = d_a0 + a_part;
                const uint64_t bh = d_b0 + sl * slot_step, bl = bh + b_part;
                auto issue = [&](auto ks_tag) {
                    constexpr int KS = decltype(ks_tag)::value;
#pragma unroll
                    for (int ks = 0; ks < KS; ks++) {
                        mma_tf32(d_tmem, ah + ks * ks_a, bl + ks * ks_b, idesc, ks > 0 ? 1u : 0u);
                        mma_tf32(d_tmem, al + ks * ks_a, bh + ks * ks_b, idesc, 1u);
                    }
#pragma unroll
                    for (int ks = 0; ks < KS; ks++) mma_tf32(d_tmem, ah + ks * ks_a, bh + ks * ks_b, idesc, 1u);
                };
                switch (ksteps) {  // 1 .. GT_MAX_KP / 8
                    case 1: issue(std::integral_constant<int, 1>{}); break;
                    case 2: issue(std::integral_constant<int, 2>{}); break;
                    case 3: issue(std::integral_constant<int, 3>{}); break;
                    case 4: issue(std::integral_constant<int, 4>{}); break;
                    case 5: issue(std::integral_constant<int, 5>{}); break;
                    case 6: issue(std::integral_constant<int, 6>{}); break;
                    case 7: issue(std::integral_constant<int, 7>{}); break;
                    default: issue(std::integral_constant<int, 8>{}); break;
                }
                mma_commit(&bar_dfull[ds]);
            }
            __syncwarp();
        }
        if (failed) {
            // give-up path: the bulk copies that were issued and not yet seen complete are awaited
            // (with the full poll limit: they do arrive) before the CTA's shared memory is given up
            for (int t = landed; t < fetched; t++) mbar_wait(&bar_full[t % ns], (unsigned)((t / ns) & 1), TC_WAIT_POLLS);
            if (lane == 0) atomicExch(&fail_flag, 1);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------------ consumers
        const int g = tid >> 7;
        const int row_local = tid & 127;
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        const float x1v = row < a.m ? x1[row * a.x1.s0] : x0;
        const f32x2 x1v2 = splat2(x1v);
        // separable phase factors of this row
        const float ph_i = phase_w * (x1v - x0);
        const float c_i = KernelFn<KT>::PHASE ? cos_approx(ph_i) : 1.0f, s_i = KernelFn<KT>::PHASE ? sin_approx(ph_i) : 0.0f;
        const f32x2 ci2 = splat2(c_i), si2 = splat2(s_i), nci2 = splat2(-c_i);
        const uint32_t tmem_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(g * CPT);

        for (int t = 0; t < tiles; t++) {
            const int sl = t % ns;
            const int ds = t & 1;
            if (!mbar_wait_warp(&bar_dfull[ds], (unsigned)((t >> 1) & 1), a.wait_polls) ||
                !mbar_wait_warp(&bar_full[sl], (unsigned)((t / ns) & 1), a.wait_polls)) {
                failed = true;
                break;
            }
            tc_fence_after();
            const int j0 = (tile_lo + t) * GT_COLS + g * CPT;
            const float *xs = slot_x2(sl) + g * CPT;
            // Two copies of the loop body: the band mask costs ~8 instructions per entry when the
            // compiler turns it into selects, and only the first and last tile of a band need it.
            auto consume = [&](auto masked_tag, auto phase_tag) {
                constexpr bool MASKED = decltype(masked_tag)::value;
                constexpr bool SEPARABLE = decltype(phase_tag)::value;
                uint32_t cbuf[2][16];
                tmem_ld16_nowait(tmem_lane + (uint32_t)(ds * GT_COLS), cbuf[0]);
                tmem_ld_wait16(cbuf[0]);
#pragma unroll
                for (int p = 0; p < PIECES; p++) {
                    if (p + 1 < PIECES)
                        tmem_ld16_nowait(tmem_lane + (uint32_t)(ds * GT_COLS + (p + 1) * 16), cbuf[(p + 1) & 1]);
#pragma unroll
                    for (int h = 0; h < 4; h++) {
                        // four entries as two packed pairs
                        const ulonglong2 xv = *reinterpret_cast<const ulonglong2 *>(xs + p * 16 + h * 4);
                        uint32_t cf[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            cf[u] = cbuf[p & 1][h * 4 + u];
                            if (MASKED) {
                                const int j = j0 + p * 16 + h * 4 + u;
                                if (j < band_lo || j >= band_hi) cf[u] = 0u;
                            }
                        }
                        const f32x2 co[2] = {(f32x2)cf[0] | ((f32x2)cf[1] << 32), (f32x2)cf[2] | ((f32x2)cf[3] << 32)};
                        if constexpr (SEPARABLE) {
                            f32x2 cs[2], sn[2];
                            // cos / sin(W tau) = c_i c_j + s_i s_j,  s_i c_j - c_i s_j
                            const ulonglong2 cj = *reinterpret_cast<const ulonglong2 *>(xs + GT_COLS + p * 16 + h * 4);
                            const ulonglong2 sj = *reinterpret_cast<const ulonglong2 *>(xs + 2 * GT_COLS + p * 16 + h * 4);
                            cs[0] = fma2(ci2, cj.x, mul2(si2, sj.x));
                            cs[1] = fma2(ci2, cj.y, mul2(si2, sj.y));
                            sn[0] = fma2(nci2, sj.x, mul2(si2, cj.x));
                            sn[1] = fma2(nci2, sj.y, mul2(si2, cj.y));
                            fn.accumulate2_ph(sub2(x1v2, xv.x), cs[0], sn[0], co[0], sums2);
                            fn.accumulate2_ph(sub2(x1v2, xv.y), cs[1], sn[1], co[1], sums2);
                        } else {
                            fn.accumulate2(sub2(x1v2, xv.x), co[0], sums2);
                            fn.accumulate2(sub2(x1v2, xv.y), co[1], sums2);
                        }
                    }
                    if (p + 1 < PIECES) tmem_ld_wait16(cbuf[(p + 1) & 1]);
                }
            };
            const bool edge = j0 < band_lo || j0 + CPT > band_hi;
            if constexpr (KernelFn<KT>::PHASE) {
                if (use_ph) {
                    if (edge) consume(std::true_type{}, std::true_type{});
                    else consume(std::false_type{}, std::true_type{});
                } else {
                    if (edge) consume(std::true_type{}, std::false_type{});
                    else consume(std::false_type{}, std::false_type{});
                }
            } else {
                if (edge) consume(std::true_type{}, std::false_type{});
                else consume(std::false_type{}, std::false_type{});
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_dfree[ds]);
        }
        if (failed) atomicExch(&fail_flag, 1);
        if (use_ph) fn.rescale_ph(sums2);  // constant factors the factored form left out of the loop

        // warp part of the CTA reduction
#pragma unroll
        for (int q = 0; q < NS; q++) {
            float v, v_hi;
            unpack2(sums2[q], v, v_hi);
            v += v_hi;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) warp_sums[warp][q] = v;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0 && fail_flag) atomicExch(a.status, 1);
    if (tid < KM_MAX_PARAMS) {
        float v = 0.0f;
        if (tid < NS) {
#pragma unroll
            for (int w = 0; w < WARPS; w++) v += warp_sums[w][tid];
            // a wait gave up: the record becomes NaN, and with it the gradient of this batch
            if (fail_flag) v = __int_as_float(0x7fc00000);
        }
        a.partials[((b * a.row_blocks + r) * a.kblocks + kb) * KM_MAX_PARAMS + tid] = v;
    }
    if (is_ctl_warp) {
        if (fail_flag) {
            // after a give-up MMAs may still be running: one commit covers everything this thread
            // has issued; tensor memory is released only when it has completed
            if (lane == 0) {
                mma_commit(&bar_drain);
                mbar_wait(&bar_drain, 0u, TC_WAIT_POLLS);
            }
            __syncwarp();
        }
        tmem_free(tmem_base, GT_TMEM_COLS);
    }
}

static int64_t grad_tc_kblocks(int64_t k) { return std::max<int64_t>(1, ceil_div(k, GT_MAX_KP)); }
static int grad_tc_kp(int64_t k) { return (int)std::max<int64_t>(8, ceil_div(std::min<int64_t>(k, GT_MAX_KP), 8) * 8); }

static size_t grad_tc_partials_bytes(const Batch &b, int64_t m, int64_t k) {
    const size_t raw = (size_t)(b.count * ceil_div(m, KM_BLOCK_SIZE) * grad_tc_kblocks(k)) * KM_MAX_PARAMS * sizeof(float);
    return (raw + 255) / 256 * 256;
}

template <int KT, int G>
static int launch_grad_tc(const GradTcArgs &a, cudaStream_t s) {
    const int64_t items = a.batch.count * a.row_blocks * a.kblocks;
    if (items > 0x7fffffffLL) {
        set_error("gradient (tensor cores): too many work items (%lld)", (long long)items);
        return KM_ERR_UNSUPPORTED;
    }
    size_t smem = ((size_t)2 * a.kp * 128 + (size_t)a.slots * (2 * a.kp * GT_COLS + 3 * GT_COLS)) * sizeof(float);
    // four CTAs of 128 tensor-memory columns fill an SM: keep a fifth from being scheduled
    smem = std::max<size_t>(smem, 46 * 1024);
    auto kernel = grad_tc_kernel<KT, G>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(grad_tc)");
    kernel<<<(unsigned)items, 128 * G + 32, smem, s>>>(a);
    KM_CHECK_LAUNCH("gradient (tensor cores) launch");
    return KM_OK;
}

// consumer groups for up to 16 columns (one group: more registers per thread; measured equal for
// spectral kernels and 10 % faster for RBF than two groups)
#ifndef GT_G_SMALL
#define GT_G_SMALL 1
#endif
template <int KT>
static int dispatch_grad_tc(const GradTcArgs &a, cudaStream_t s) {
    // consumer groups by GEMM K: shared memory (left rows + right tiles) decides the CTAs per SM
    if (a.kp <= 16) return launch_grad_tc<KT, GT_G_SMALL>(a, s);
    if (a.kp <= 32) return launch_grad_tc<KT, 2>(a, s);
    return launch_grad_tc<KT, 4>(a, s);
}

static int grad_tc_entry(const char *name, int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                         const km_view *x1, const km_view *x2, const km_view *left, const km_view *right,
                         const km_view *params, const km_view *start, const km_view *end, const km_view *grad,
                         void *workspace, size_t workspace_bytes, void *stream) {
    KM_REQUIRE(valid_kernel_type(kernel_type), KM_ERR_INVALID_ARGUMENT, "%s: unknown kernel type %d", name, kernel_type);
    KM_REQUIRE(batch && x1 && x2 && left && right && params && start && end && grad, KM_ERR_INVALID_ARGUMENT,
               "%s: null argument", name);
    KM_REQUIRE(m >= 0 && n >= 0 && k >= 0 && n <= 0x7fffffffLL - GT_COLS, KM_ERR_INVALID_ARGUMENT, "%s: bad sizes", name);
    GradTcArgs a;
    int rc = make_batch(batch, &a.batch);
    if (rc != KM_OK) return rc;
    if (a.batch.count == 0) return KM_OK;
    KM_REQUIRE(params->data && grad->data, KM_ERR_INVALID_ARGUMENT, "%s: null data pointer", name);
    const size_t need = km_grad_tc_workspace_bytes(batch, m, n, k, right);
    KM_REQUIRE(workspace != nullptr && workspace_bytes >= need, KM_ERR_WORKSPACE,
               "%s: workspace of %zu bytes needed, %zu given", name, need, workspace_bytes);
    KM_REQUIRE((uintptr_t)workspace % 256 == 0, KM_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned", name);
    a.m = m;
    a.n = n;
    a.k = k;
    a.kp = grad_tc_kp(k);
    a.kblocks = (int)grad_tc_kblocks(k);
    a.slots = a.kp <= 16 ? 4 : 3;
    a.wait_polls = current_wait_polls();
    a.row_blocks = ceil_div(m, KM_BLOCK_SIZE);
    a.x1 = make_view<const float>(x1, a.batch);
    a.x2 = make_view<const float>(x2, a.batch);
    a.left = make_view<const float>(left, a.batch);
    a.params = make_view<const float>(params, a.batch);
    a.start = make_view<const int>(start, a.batch);
    a.end = make_view<const int>(end, a.batch);
    const View<const float> rv = make_view<const float>(right, a.batch);
    const View<float> gv = make_view<float>(grad, a.batch);
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    a.status = reinterpret_cast<int *>(ws);
    a.partials = reinterpret_cast<float *>(ws + TC_STATUS_BYTES);
    float *images = reinterpret_cast<float *>(ws + TC_STATUS_BYTES + grad_tc_partials_bytes(a.batch, m, k));
    a.images = images;
    const int64_t slots = tc_slots(a.batch, rv);
    const int64_t tiles = ceil_div(n, GT_COLS);
    a.tiles_total = tiles;
    a.image_slot_stride = slots > 1 ? a.kblocks * tiles * (2LL * a.kp * GT_COLS) : 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (a.row_blocks > 0) {
        KM_REQUIRE(x1->data && left->data && start->data && end->data, KM_ERR_INVALID_ARGUMENT,
                   "%s: null data pointer", name);
        KM_REQUIRE(n == 0 || (x2->data && right->data), KM_ERR_INVALID_ARGUMENT, "%s: null data pointer", name);
        const int64_t total = slots * a.kblocks * tiles * (int64_t)GT_COLS * a.kp;
        const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(total, 256), 148 * 32));
        grad_tc_images_kernel<<<blocks, 256, 0, s>>>(a.batch, slots, n, k, a.kp, a.kblocks, tiles, rv, images, a.status);
        KM_CHECK_LAUNCH("gradient (tensor cores) pre-pass launch");
        switch (kernel_type) {
        case KM_KERNEL_RBF: rc = dispatch_grad_tc<KM_KERNEL_RBF>(a, s); break;
        case KM_KERNEL_SPECTRAL: rc = dispatch_grad_tc<KM_KERNEL_SPECTRAL>(a, s); break;
        default: rc = dispatch_grad_tc<KM_KERNEL_LOCALLY_PERIODIC>(a, s); break;
        }
        if (rc != KM_OK) return rc;
    }
    return launch_grad_finish(kernel_type, a.batch, a.row_blocks * a.kblocks, a.partials, false, a.params, gv, s);
}

}  // namespace km

extern "C" size_t km_grad_tc_workspace_bytes(const km_batch *batch, int64_t m, int64_t n, int64_t k,
                                             const km_view *right) {
    using namespace km;
    Batch b;
    if (batch == nullptr || right == nullptr || make_batch(batch, &b) != KM_OK || m < 0 || n < 0 || k < 0) return 0;
    const View<const float> rv = make_view<const float>(right, b);
    const int64_t kp = grad_tc_kp(k);
    return (size_t)TC_STATUS_BYTES + grad_tc_partials_bytes(b, m, k) +
           (size_t)(tc_slots(b, rv) * grad_tc_kblocks(k) * ceil_div(n, GT_COLS)) * (2 * kp * GT_COLS) * sizeof(float);
}

extern "C" int km_bilinear_derivative_tc_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                                             const km_view *x1, const km_view *x2, const km_view *left,
                                             const km_view *right, const km_view *params, const km_view *start,
                                             const km_view *end, const km_view *grad, void *workspace,
                                             size_t workspace_bytes, void *stream) {
    return km::grad_tc_entry("km_bilinear_derivative_tc_f32", kernel_type, batch, m, n, k, x1, x2, left, right, params,
                             start, end, grad, workspace, workspace_bytes, stream);
}

extern "C" int km_matmul_bwd_tc_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                                    const km_view *x1, const km_view *x2, const km_view *rhs, const km_view *params,
                                    const km_view *start, const km_view *end, const km_view *out_grad,
                                    const km_view *grad, void *workspace, size_t workspace_bytes, void *stream) {
    return km::grad_tc_entry("km_matmul_bwd_tc_f32", kernel_type, batch, m, n, k, x1, x2, out_grad, rhs, params, start,
                             end, grad, workspace, workspace_bytes, stream);
}

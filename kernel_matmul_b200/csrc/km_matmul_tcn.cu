// Forward product on the tensor cores for NARROW right-hand sides (k <= 16 columns).
//
//   out[b, i, :] = sum_{j in band} kappa(x1[b,i], x2[b,j]) * rhs[b, j, :]
//
// With few rhs columns the contraction is cheap for the tensor core; what bounds the kernel is
// generating the kernel-matrix entries (two SFU operations per spectral entry).  So the CTA is
// built around its 128 generator threads, one per row of the 128-row block:
//
//  * a generator evaluates the 16 entries of its row for a tile of 16 band columns, splits each
//    into hi + lo (3xTF32) and writes both straight into TENSOR MEMORY with tcgen05.st: its row
//    is its tensor-memory lane, the 16 values are 16 consecutive columns.  This is exactly the
//    layout tcgen05.mma takes for an A operand in tensor memory (row i in lane i, one K value per
//    32-bit column), so the kernel matrix never touches shared memory -- per entry the FP32 pipe
//    only runs the ~7 operations of kappa and the split, against 5 + k on the FMA path;
//  * a control warp fetches rhs tiles (images laid out by a pre-pass, one bulk copy per 64
//    columns, hi and lo parts) and x2 values (cp.async) into a ring of shared-memory slots and
//    one of its lanes issues the MMAs D[128 x 16] += A[128 x 8] . B[8 x 16] with A from tensor
//    memory and B from shared memory.  (A CTA gets a tcgen05 instruction issued only every
//    ~45-80 cycles, measured; splitting the MMAs of a tile over several issuing warps
//    (TN_ISSUERS) did not raise that rate and costs issue slots, so there is one.)
//  * accumulators live in tensor memory for at most TN_PROMO tiles (the tensor core adds with
//    truncation; 16 hi*hi MMAs keep that bias below 1e-6) and are then added to fp32 registers
//    of the generator that owns the row, two accumulators alternating.
//
// Four CTAs share an SM (128 tensor-memory columns each).  All hand-offs are mbarriers; every
// wait is bounded and a give-up is reported through the status word of the workspace.
#include "km_tcgen05.cuh"

namespace km {

constexpr int TN_N = 16;                        // GEMM N: rhs columns (padded)
constexpr int TN_BK = 16;                       // band columns per A stage
constexpr int TN_SUPER = 4;                     // A tiles per rhs / x2 slot
constexpr int TN_SCOLS = TN_BK * TN_SUPER;      // band columns per slot (64)
constexpr int TN_A_STAGES = 3;                  // A stages in tensor memory (32 columns each: hi | lo)
constexpr int TN_SLOTS = 4;                     // rhs / x2 slots in shared memory
constexpr int TN_PROMO = 8;                     // tiles per accumulator group
constexpr int TN_IMG_FLOATS = 2 * TN_SCOLS * TN_N;  // hi + lo image of one slot
constexpr int TN_SLOT_FLOATS = TN_IMG_FLOATS + TN_SCOLS;
constexpr int TN_TMEM_COLS = 128;
#ifndef TN_ISSUERS_DEF
#define TN_ISSUERS_DEF 1
#endif
constexpr int TN_ISSUERS = TN_ISSUERS_DEF;        // control warps; warp w issues the 8-column steps w, w + TN_ISSUERS, ..
constexpr int TN_THREADS = 128 + 32 * TN_ISSUERS;
// MMAs of different issuers are not ordered against each other: with several issuers every MMA
// accumulates and the generators zero an accumulator after collecting it; a single issuer
// simply starts each group with a non-accumulating MMA.
constexpr bool TN_ZEROED_ACC = TN_ISSUERS > 1;
constexpr int TN_ACC_COL = TN_A_STAGES * 2 * TN_BK;  // first accumulator column (96)
constexpr size_t TN_SMEM_BYTES = 48 * 1024;     // > slots: caps the SM at four CTAs (4 x 128 tensor-memory columns)
static_assert(TN_ACC_COL + 2 * TN_N <= TN_TMEM_COLS, "tensor-memory budget");
static_assert(TN_SLOTS * TN_SLOT_FLOATS * sizeof(float) <= TN_SMEM_BYTES, "shared-memory budget");

// Pre-pass: rhs -> per (slot, 64-column group) image [part: hi, lo][chunk = jj / 4][c][jj % 4].
// hi is the raw fp32 word (the tensor core reads its TF32 bits), lo = x - trunc_tf32(x).  Rows
// past n and columns past k are zero.  Also clears the status word.
__global__ void __launch_bounds__(256) tcn_rhs_images_kernel(Batch batch, int64_t slots, int64_t n, int64_t k,
                                                             int64_t supers, View<const float> rhs, float *images,
                                                             int *status) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *status = 0;
    const int64_t total = slots * supers * (int64_t)(TN_SCOLS * TN_N);
    for (int64_t idx = blockIdx.x * 256LL + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * 256) {
        int64_t rem = idx;
        const int c = (int)(rem % TN_N);
        rem /= TN_N;
        const int jj = (int)(rem % TN_SCOLS);
        rem /= TN_SCOLS;
        const int64_t sup = rem % supers;
        const int64_t slot = rem / supers;
        const int64_t j = sup * TN_SCOLS + jj;
        float v = 0.0f;
        if (j < n && c < k) {
            const BatchIndex bi = decompose(batch, slot);
            v = batch_ptr(rhs, bi)[j * rhs.s0 + c * rhs.s1];
        }
        float *img = images + (slot * supers + sup) * TN_IMG_FLOATS;
        const int at = (jj >> 2) * (TN_N * 4) + c * 4 + (jj & 3);
        img[at] = v;
        img[TN_SCOLS * TN_N + at] = v - tf32_hi(v);
    }
}

template <int KT>
__global__ void __launch_bounds__(TN_THREADS, 4) matmul_tcn_kernel(const TcArgs a) {
    constexpr int N = TN_N;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[TN_SLOTS];    // rhs image + x2 of a slot landed
    __shared__ __align__(8) uint64_t bar_sfree[TN_SLOTS];   // MMAs reading a slot are done
    __shared__ __align__(8) uint64_t bar_ready[TN_A_STAGES];  // A stage written by the generators
    __shared__ __align__(8) uint64_t bar_empty[TN_A_STAGES];  // MMAs reading an A stage are done
    __shared__ __align__(8) uint64_t bar_acc[2];            // accumulator group complete
    __shared__ __align__(8) uint64_t bar_free[2];           // accumulator added to the registers
    __shared__ uint32_t tmem_base_slot;
    __shared__ int fail_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const bool is_ctl_warp = warp >= 4;
    const int issuer = warp - 4;  // control warps: 0 also fetches

    float *smem_f = reinterpret_cast<float *>(smem_raw);
    auto slot_img = [&](int sl) { return smem_f + sl * TN_SLOT_FLOATS; };
    auto slot_x2 = [&](int sl) { return smem_f + sl * TN_SLOT_FLOATS + TN_IMG_FLOATS; };

    int64_t item = blockIdx.x;
    const int64_t b = item % a.batch.count;
    const int64_t r = a.rb_begin + item / a.batch.count;

    const BatchIndex bi = decompose(a.batch, b);
    const float *x1 = batch_ptr(a.x1, bi);
    const float *x2 = batch_ptr(a.x2, bi);
    float *out = batch_ptr(a.out, bi);
    KernelFn<KT> fn;
    fn.init(batch_ptr(a.params, bi), a.params.s0);

    const int n = (int)a.n;
    const int band_lo = clamp_int(batch_ptr(a.start, bi)[r * a.start.s0], 0, n);
    const int band_hi = max(band_lo, min(batch_ptr(a.end, bi)[r * a.end.s0], n));
    const int tile_lo = band_lo / TN_BK;
    const int tiles = band_hi > band_lo ? (band_hi + TN_BK - 1) / TN_BK - tile_lo : 0;
    const int super_lo = tile_lo / TN_SUPER;
    const int supers = tiles > 0 ? (tile_lo + tiles - 1) / TN_SUPER - super_lo + 1 : 0;
    const float *images = a.images + (a.image_slot_stride ? b * a.image_slot_stride : 0);

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < TN_SLOTS; s++) {
            mbar_init(&bar_full[s], 33);  // 32 lanes' cp.async arrivals + the bulk copy's expect_tx arrival
            mbar_init(&bar_sfree[s], TN_ISSUERS);
        }
#pragma unroll
        for (int s = 0; s < TN_A_STAGES; s++) {
            mbar_init(&bar_ready[s], 4);
            mbar_init(&bar_empty[s], TN_ISSUERS);
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            mbar_init(&bar_acc[i], TN_ISSUERS);
            mbar_init(&bar_free[i], 4);
        }
        fail_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) tmem_alloc(&tmem_base_slot, TN_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    // both accumulators start at zero when every MMA accumulates
    if (TN_ZEROED_ACC && !is_ctl_warp) {
        uint32_t zero[16];
#pragma unroll
        for (int u = 0; u < 16; u++) zero[u] = 0u;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        tmem_st16(lane_addr + (uint32_t)TN_ACC_COL, zero);
        tmem_st16(lane_addr + (uint32_t)(TN_ACC_COL + TN_N), zero);
        tmem_st_wait();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
    bool failed = false;

    float acc[N];
#pragma unroll
    for (int c = 0; c < N; c++) acc[c] = 0.0f;

    if (is_ctl_warp) {
        // ------------------------------------------- slot fetches (all lanes) + MMA issue (lane 0)
        auto fetch = [&](int sr) {
            const int sl = sr % TN_SLOTS;
            const int64_t sup = super_lo + sr;
            float *xs = slot_x2(sl);
#pragma unroll
            for (int u = 0; u < TN_SCOLS / 32; u++) {
                const int jj = lane + 32 * u;
                const int64_t j = sup * TN_SCOLS + jj;
                const bool valid = j < n;
                cp_async4_zfill(xs + jj, x2 + (valid ? j : 0) * a.x2.s0, valid);
            }
            cp_async_mbar_arrive(&bar_full[sl]);
            if (lane == 0) {
                constexpr uint32_t bytes = TN_IMG_FLOATS * sizeof(float);
                mbar_expect_tx(&bar_full[sl], bytes);
                bulk_copy_g2s(slot_img(sl), images + sup * TN_IMG_FLOATS, bytes, &bar_full[sl]);
            }
        };
        if (issuer == 0)
            for (int sr = 0; sr < min(supers, TN_SLOTS); sr++) fetch(sr);

        constexpr uint32_t lbo_b = N * 16, sbo = 128;
        constexpr uint64_t slot_step = (uint64_t)(TN_SLOT_FLOATS * 4) >> 4;
        constexpr uint64_t part_step = (uint64_t)(TN_SCOLS * N * 4) >> 4;  // hi -> lo image
        constexpr uint64_t kstep = (uint64_t)(2 * lbo_b) >> 4;             // 8 band columns = 2 chunks
        const uint64_t d_b0 = smem_desc(smem_u32(slot_img(0)), lbo_b, sbo);
        int s = 0, use = 0, in_grp = 0, grp = 0;
        for (int t = 0; t < tiles; t++) {
            const int ta = tile_lo + t;
            const int q = ta & (TN_SUPER - 1);
            const int sr = ta / TN_SUPER - super_lo;
            const int sl = sr % TN_SLOTS;
            const int ai = grp & 1;
            const bool grp_first = in_grp == 0;
            const bool grp_last = in_grp == TN_PROMO - 1 || t == tiles - 1;
            const bool slot_first = t == 0 || q == 0;
            const bool slot_last = q == TN_SUPER - 1 || t == tiles - 1;
            bool ok = true;
            if (slot_first) ok = mbar_wait(&bar_full[sl], (unsigned)((sr / TN_SLOTS) & 1));
            // the accumulator must have been collected by every generator warp
            if (ok && grp_first && grp >= 2) ok = mbar_wait(&bar_free[ai], (unsigned)(((grp >> 1) - 1) & 1));
            if (ok) ok = mbar_wait(&bar_ready[s], (unsigned)(use & 1));
            if (!__all_sync(0xffffffffu, ok)) {
                failed = true;
                break;
            }
            tc_fence_after();
            if (lane == 0) {
                const uint32_t d_tmem = tmem_base + (uint32_t)(TN_ACC_COL + ai * N);
                const uint32_t a_hi = tmem_base + (uint32_t)(s * 2 * TN_BK), a_lo = a_hi + TN_BK;
                const uint64_t b_hi = d_b0 + sl * slot_step + (uint64_t)(q * (TN_BK / 8)) * kstep, b_lo = b_hi + part_step;
                // this issuer's share of the tile's 8-column steps: the small cross terms first, hi * hi last
#pragma unroll
                for (int ks = issuer; ks < TN_BK / 8; ks += TN_ISSUERS) {
                    mma_tf32_ts(d_tmem, a_hi + ks * 8, b_lo + ks * kstep, idesc,
                                (TN_ZEROED_ACC || ks > 0 || !grp_first) ? 1u : 0u);
                    mma_tf32_ts(d_tmem, a_lo + ks * 8, b_hi + ks * kstep, idesc, 1u);
                }
#pragma unroll
                for (int ks = issuer; ks < TN_BK / 8; ks += TN_ISSUERS)
                    mma_tf32_ts(d_tmem, a_hi + ks * 8, b_hi + ks * kstep, idesc, 1u);
                mma_commit(&bar_empty[s]);
                if (slot_last) mma_commit(&bar_sfree[sl]);
                if (grp_last) mma_commit(&bar_acc[ai]);
            }
            __syncwarp();
            // after the first tile of a slot: the previous slot is re-filled once its MMAs are done
            if (issuer == 0 && slot_first && sr >= 1 && sr - 1 + TN_SLOTS < supers) {
                const int prev = sr - 1;
                ok = mbar_wait(&bar_sfree[prev % TN_SLOTS], (unsigned)((prev / TN_SLOTS) & 1));
                if (!__all_sync(0xffffffffu, ok)) {
                    failed = true;
                    break;
                }
                fetch(prev + TN_SLOTS);
            }
            if (++s == TN_A_STAGES) {
                s = 0;
                use++;
            }
            if (++in_grp == TN_PROMO) {
                in_grp = 0;
                grp++;
            }
        }
        if (failed && lane == 0) atomicExch(&fail_flag, 1);
        // no cp.async may be in flight when the CTA exits
        cp_async_wait<0>();
        __syncwarp();
    } else {
        // ----------------------------------------------------------------------- generators
        const int64_t row = r * KM_BLOCK_SIZE + tid;
        const float x1v = row < a.m ? x1[row * a.x1.s0] : 0.0f;
        const uint32_t tmem_lane = tmem_base + ((uint32_t)(warp * 32) << 16);

        auto collect = [&](int ai, bool rezero) {
            tc_fence_after();
            uint32_t v[16];
            tmem_ld16_nowait(tmem_lane + (uint32_t)(TN_ACC_COL + ai * N), v);
            tmem_ld_wait();
#pragma unroll
            for (int u = 0; u < 16; u++) acc[u] += __uint_as_float(v[u]);
            if (TN_ZEROED_ACC && rezero) {
#pragma unroll
                for (int u = 0; u < 16; u++) v[u] = 0u;
                tmem_st16(tmem_lane + (uint32_t)(TN_ACC_COL + ai * N), v);
                tmem_st_wait();
            }
            tc_fence_before();
        };

        for (int t = 0; t < tiles; t++) {
            const int ta = tile_lo + t;
            const int q = ta & (TN_SUPER - 1);
            const int sr = ta / TN_SUPER - super_lo;
            const int sl = sr % TN_SLOTS;
            const int s = t % TN_A_STAGES, use = t / TN_A_STAGES;
            const int grp = t / TN_PROMO, ai = grp & 1;
            if ((t == 0 || q == 0) && !mbar_wait_warp(&bar_full[sl], (unsigned)((sr / TN_SLOTS) & 1))) {
                failed = true;
                break;
            }
            // an accumulator that is about to be reused is first added to the registers
            if ((t % TN_PROMO) == 0 && grp >= 2) {
                if (!mbar_wait_warp(&bar_acc[ai], (unsigned)((grp / 2 - 1) & 1))) {
                    failed = true;
                    break;
                }
                collect(ai, true);
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_free[ai]);
            }
            // stage s must have been read by the MMAs of tile t - TN_A_STAGES
            if (use > 0) {
                if (!mbar_wait_warp(&bar_empty[s], (unsigned)((use - 1) & 1))) {
                    failed = true;
                    break;
                }
                tc_fence_after();
            }
            const float4 *xs = reinterpret_cast<const float4 *>(slot_x2(sl) + q * TN_BK);
            float kv[TN_BK];
#pragma unroll
            for (int h = 0; h < TN_BK / 4; h++) {
                const float4 xv = xs[h];
                kv[4 * h + 0] = fn.unscaled(x1v - xv.x);
                kv[4 * h + 1] = fn.unscaled(x1v - xv.y);
                kv[4 * h + 2] = fn.unscaled(x1v - xv.z);
                kv[4 * h + 3] = fn.unscaled(x1v - xv.w);
            }
            const int j0 = ta * TN_BK;
            if (j0 < band_lo || j0 + TN_BK > band_hi) {
#pragma unroll
                for (int u = 0; u < TN_BK; u++)
                    if (j0 + u < band_lo || j0 + u >= band_hi) kv[u] = 0.0f;
            }
            // (scalar arithmetic on purpose: packed f32x2 operations made this kernel slower)
            uint32_t hi[TN_BK], lo[TN_BK];
#pragma unroll
            for (int u = 0; u < TN_BK; u++) {
                hi[u] = __float_as_uint(kv[u]);
                lo[u] = __float_as_uint(kv[u] - tf32_hi(kv[u]));
            }
            tmem_st16(tmem_lane + (uint32_t)(s * 2 * TN_BK), hi);
            tmem_st16(tmem_lane + (uint32_t)(s * 2 * TN_BK + TN_BK), lo);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_ready[s]);
        }

        // drain: the last two groups still sit in tensor memory
        const int groups = (tiles + TN_PROMO - 1) / TN_PROMO;
        for (int grp = max(0, groups - 2); grp < groups && !failed; grp++) {
            if (!mbar_wait_warp(&bar_acc[grp & 1], (unsigned)((grp / 2) & 1))) {
                failed = true;
                break;
            }
            collect(grp & 1, false);
        }
        if (failed) atomicExch(&fail_flag, 1);
    }

    tc_fence_before();
    __syncthreads();
    if (fail_flag) {
        if (tid == 0) atomicExch(a.status, 1);
    } else if (!is_ctl_warp) {
        const int64_t row = r * KM_BLOCK_SIZE + tid;
        if (row < a.m) {
            const float scale = fn.scale;
            float *orow = out + (row - a.rb_begin * KM_BLOCK_SIZE) * a.out.s0;
            const bool vec_ok = a.out.s1 == 1 && (a.out.s0 % 4 == 0) && (a.k % 4 == 0) &&
                                ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
            if (vec_ok) {
#pragma unroll
                for (int c = 0; c < N; c += 4)
                    if (c < a.k)
                        *reinterpret_cast<float4 *>(orow + c) =
                            make_float4(acc[c] * scale, acc[c + 1] * scale, acc[c + 2] * scale, acc[c + 3] * scale);
            } else {
#pragma unroll
                for (int c = 0; c < N; c++)
                    if (c < a.k) orow[c * a.out.s1] = acc[c] * scale;
            }
        }
    }
    if (warp == 4) tmem_free(tmem_base, TN_TMEM_COLS);
}

size_t tcn_workspace_bytes(const Batch &b, int64_t n, const View<const float> &rhs) {
    const int64_t supers = ceil_div(n, TN_SCOLS);
    return (size_t)TC_STATUS_BYTES + (size_t)(tc_slots(b, rhs) * supers) * TN_IMG_FLOATS * sizeof(float);
}

template <int KT>
static int launch_tcn(const TcArgs &a, cudaStream_t s) {
    const int64_t items = a.batch.count * a.row_blocks;
    if (items > 0x7fffffffLL) {
        set_error("km_matmul_tc_f32: too many work items (%lld)", (long long)items);
        return KM_ERR_UNSUPPORTED;
    }
    auto kernel = matmul_tcn_kernel<KT>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TN_SMEM_BYTES);
    if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(matmul_tcn)");
    kernel<<<(unsigned)items, TN_THREADS, TN_SMEM_BYTES, s>>>(a);
    KM_CHECK_LAUNCH("km_matmul_tc_f32 (narrow) launch");
    return KM_OK;
}

int tcn_matmul(int kernel_type, TcArgs a, const View<const float> &rhs, void *workspace, cudaStream_t s) {
    const int64_t slots = tc_slots(a.batch, rhs);
    const int64_t supers = ceil_div(a.n, TN_SCOLS);
    a.status = static_cast<int *>(workspace);
    float *images = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + TC_STATUS_BYTES);
    a.images = images;
    a.image_slot_stride = slots > 1 ? supers * (int64_t)TN_IMG_FLOATS : 0;
    const int64_t total = slots * supers * (int64_t)(TN_SCOLS * TN_N);
    const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(total, 256), 148 * 32));
    tcn_rhs_images_kernel<<<blocks, 256, 0, s>>>(a.batch, slots, a.n, a.k, supers, rhs, images, a.status);
    KM_CHECK_LAUNCH("km_matmul_tc_f32 (narrow) pre-pass launch");
    switch (kernel_type) {
    case KM_KERNEL_RBF: return launch_tcn<KM_KERNEL_RBF>(a, s);
    case KM_KERNEL_SPECTRAL: return launch_tcn<KM_KERNEL_SPECTRAL>(a, s);
    default: return launch_tcn<KM_KERNEL_LOCALLY_PERIODIC>(a, s);
    }
}

}  // namespace km

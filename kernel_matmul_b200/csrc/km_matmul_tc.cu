// Forward product on the tensor cores with the kernel-matrix tiles handed over in tensor memory.
//
//   out[b, i, :] = sum_{j in band} kappa(x1[b,i], x2[b,j]) * rhs[b, j, :]
//
// For the widths this path sees (1 ... a few hundred rhs columns) the contraction is cheap for
// the tensor core; what bounds the kernel is generating the kernel-matrix entries (two SFU
// operations per spectral entry) and the rate at which a CTA gets tcgen05 instructions issued
// (one every ~45-100 cycles, measured).  So the
// CTA is built around its 128 generator threads, one per row of the 128-row block, and the
// contraction is arranged to need as few MMA instructions as possible:
//
//  * operands are split into two fp16 parts, x = hi + lo (hi: the 11 leading bits, lo: the next
//    11; the dropped lo * lo term is 2^-22 relative), so one MMA of kind::f16 covers K = 16 band
//    columns and 16 columns take three MMAs, hi*lo + lo*hi + hi*hi (3xTF32 would need six: K = 8
//    per instruction).  Kernel values lie in [-1, 1] and fit fp16 as they are (a lo part below
//    2^-14 is a subnormal with an absolute error of at most 2^-25); the rhs is scaled per column
//    by a power of two so that its largest magnitude lies in [2^13, 2^14) -- a pre-pass finds the
//    column maxima, writes the scaled hi / lo images in the tensor core's K-major layout and
//    the inverse scales, which the epilogue applies;
//  * a generator evaluates the entries of its row for a tile (32 band columns; 64 at N = 128,
//    shared by four generator groups), splits them and writes both
//    parts straight into TENSOR MEMORY with tcgen05.st: its row is its tensor-memory lane, the
//    values are consecutive columns (two fp16 per column) -- exactly the layout tcgen05.mma takes
//    for an A operand in tensor memory, so the kernel matrix never touches shared memory;
//  * a control warp fetches rhs tiles (one bulk copy per 64 band columns) and x2 values
//    (cp.async) into a ring of shared-memory slots and one of its lanes issues the MMAs
//    D[128 x N] += A[128 x 16] . B[16 x N] (N = 16, 32, 64 or 128; wider right-hand sides are
//    processed in blocks of 128 columns), three per 16 band columns;
//  * accumulators live in tensor memory for at most 256 band columns (the tensor core adds with
//    truncation) and are then added to fp32 registers of the generator that owns the row, two
//    accumulators alternating.
//
// Four CTAs share an SM at N = 16 (128 tensor-memory columns each; three at N = 32, two at
// N = 64, one with 512 generator threads at N = 128).  All hand-offs are mbarriers; every
// wait is bounded; a give-up is reported through the status word of the workspace and turns the
// CTA's output rows into NaN.
#include <cuda_fp16.h>

#include "km_tcgen05.cuh"

namespace km {

constexpr int TC_MAX_N = 128;                   // widest GEMM N (rhs columns per CTA) of this kernel
constexpr int TC_SCOLS = 64;                    // band columns per rhs / x2 slot
constexpr int TC_SLOTS = 4;                     // rhs / x2 slots in shared memory
constexpr int TC_GROUP_COLS = 256;              // band columns per accumulator group (48 MMAs)
// per image slot in the workspace: [TC_MAX_N column maxima (bit patterns) | TC_MAX_N inverse scales]
constexpr int TC_SCALE_WORDS = 2 * TC_MAX_N;

// Per GEMM width N (rhs columns padded to 16 / 32 / 64 / 128): tensor-memory and shared-memory budget.
//   N = 16:  3 A stages (96 columns) + 2 accumulators of 16 = 128 columns, 4 CTAs per SM
//   N = 32:  2 A stages (64)         + 2 x 32            = 128 columns, 3 CTAs per SM (registers)
//   N = 64:  3 A stages (96)         + 2 x 64            = 224 -> 256 columns, 2 CTAs per SM with two
//            generator groups: group g generates every second tile (all 32 band columns of it) and
//            owns the accumulator columns [32g, 32g + 32) of its row
//   N = 128: 3 A stages of 64 (192) + 2 x 128           = 448 -> 512 columns, 1 CTA per SM with four
//            generator groups of 128 threads and tiles of 64 band columns: the groups {0, 1} and
//            {2, 3} take alternate tiles, each group 32 band columns of its set's tile; group g owns
//            the accumulator columns [32g, 32g + 32) of its row
// A tile is BK band columns (BK / 16 MMA steps of K = 16); a thread generates 16 columns per step it owns.
template <int N>
struct TcCfg {
    static constexpr int G = N == 128 ? 4 : (N == 64 ? 2 : 1);  // generator groups of 128 threads
    // at N >= 64 a second helper warp does the slot fetches, so that the warp that issues the MMAs
    // never waits for a copy to be issued or for a slot to drain
    static constexpr bool FETCH_WARP = N >= 64;
    // with several generator groups the tiles alternate between two sets of groups: a thread then
    // generates twice as many entries per hand-off (barrier waits, store fence, arrival)
    static constexpr int TILE_SETS = G >= 2 ? 2 : 1;
    static constexpr int SET_GROUPS = G / TILE_SETS;       // groups that share a tile
    static constexpr int THREADS = 128 * G + 32 + (FETCH_WARP ? 32 : 0);
    static constexpr int BK = N == 128 ? 64 : 32;        // band columns per tile
    static constexpr int SUPER = TC_SCOLS / BK;           // tiles per rhs / x2 slot
    static constexpr int A_COLS = BK;                     // tensor-memory columns per A stage: per 16 band columns hi 8 | lo 8
    static constexpr int PROMO = TC_GROUP_COLS / BK;      // tiles per accumulator group
    static constexpr int A_STAGES = N == 32 ? 2 : 3;
    static constexpr int ACC_COL = A_STAGES * A_COLS;
    static constexpr int TMEM_COLS = N <= 32 ? 128 : (N == 64 ? 256 : 512);
    static constexpr int MIN_CTAS = N == 16 ? 4 : (N == 32 ? 3 : (N == 64 ? 2 : 1));
    static constexpr int IMG_HALFS = 2 * TC_SCOLS * N;  // hi + lo image of one slot (fp16 values)
    static constexpr int IMG_BYTES = IMG_HALFS * 2;
    static constexpr int SLOT_BYTES = IMG_BYTES + 3 * TC_SCOLS * 4;  // image + x2 values + separable phase factors (cos, sin)
    // dynamic shared memory: the slots, padded so that no more CTAs fit an SM than its 512
    // tensor-memory columns can serve
    static constexpr size_t SMEM_BYTES = N <= 32 ? 48 * 1024 : (N == 64 ? 80 * 1024 : 136 * 1024);
    static_assert(ACC_COL + 2 * N <= TMEM_COLS, "tensor-memory budget");
    static_assert(TC_SLOTS * SLOT_BYTES <= SMEM_BYTES, "shared-memory budget");
};

// Pre-pass 1: column maxima of |rhs| as float bit patterns (monotone for non-negative floats).
// The maxima words must be zero on entry.  Also clears the status word.
__global__ void __launch_bounds__(256) tc_colmax_kernel(Batch batch, int64_t slots, int64_t n, int64_t k, int npad,
                                                         int kblocks, View<const float> rhs, unsigned *scales,
                                                         int *status) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *status = 0;
    const int64_t rows_per_pass = (int64_t)gridDim.x * 16;
    for (int64_t slot = 0; slot < slots; slot++) {
        const BatchIndex bi = decompose(batch, slot);
        const float *base = batch_ptr(rhs, bi);
        for (int c0 = 0; c0 < k; c0 += 16) {
            const int c = c0 + threadIdx.x % 16;
            unsigned mx = 0u;
            if (c < k)
                for (int64_t j = blockIdx.x * 16 + threadIdx.x / 16; j < n; j += rows_per_pass)
                    mx = max(mx, __float_as_uint(fabsf(base[j * rhs.s0 + c * rhs.s1])));
            // column = lane % 16: lanes l and l + 16 hold the same column
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            if ((threadIdx.x & 31) < 16 && mx != 0u)
                atomicMax(scales + (slot * kblocks + c / npad) * TC_SCALE_WORDS + c % npad, mx);
        }
    }
}

// Power-of-two scale that brings a column maximum into [2^13, 2^14); 1 for empty or non-finite columns.
__device__ __forceinline__ float tc_column_scale(unsigned max_bits) {
    const int e = (int)(max_bits >> 23);  // biased exponent of the maximum: 2^(e - 127) <= max < 2^(e - 126)
    if (e == 0 || e == 255) return 1.0f;
    const int se = min(max(267 - e, 1), 254);  // scale = 2^(14 - (e - 126)), biased exponent 267 - e
    return __uint_as_float((unsigned)se << 23);
}

// Pre-pass 2: rhs -> per (slot, 64-column group) image [part: hi, lo][chunk = jj / 8][c][jj % 8]
// of fp16 values of the scaled column, y s = hi + lo (the K-major core-matrix layout of a
// kind::f16 B operand); rows past n and columns past k are zero.  Also writes the inverse scales.
__global__ void __launch_bounds__(256) tc_rhs_images_kernel(Batch batch, int64_t slots, int64_t n, int64_t k, int npad,
                                                             int kblocks, int64_t supers, View<const float> rhs,
                                                             __half *images, unsigned *scales) {
    const int64_t total = slots * kblocks * supers * (int64_t)(TC_SCOLS * npad);
    for (int64_t idx = blockIdx.x * 256LL + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * 256) {
        int64_t rem = idx;
        const int c = (int)(rem % npad);
        rem /= npad;
        const int jj = (int)(rem % TC_SCOLS);
        rem /= TC_SCOLS;
        const int64_t sup = rem % supers;
        rem /= supers;
        const int kb = (int)(rem % kblocks);
        const int64_t slot = rem / kblocks;
        const int64_t j = sup * TC_SCOLS + jj;
        const int64_t col = (int64_t)kb * npad + c;
        const int64_t rec = (slot * kblocks + kb) * TC_SCALE_WORDS;
        const float sc = tc_column_scale(scales[rec + c]);
        float v = 0.0f;
        if (j < n && col < k) {
            const BatchIndex bi = decompose(batch, slot);
            v = batch_ptr(rhs, bi)[j * rhs.s0 + col * rhs.s1] * sc;
        }
        const __half hi = __float2half_rn(v);
        const __half lo = __float2half_rn(v - __half2float(hi));
        __half *img = images + ((slot * kblocks + kb) * supers + sup) * (2 * TC_SCOLS * npad);
        const int at = (jj >> 3) * (npad * 8) + c * 8 + (jj & 7);
        img[at] = hi;
        img[TC_SCOLS * npad + at] = lo;
        if (sup == 0 && jj == 0) reinterpret_cast<float *>(scales)[rec + TC_MAX_N + c] = 1.0f / sc;
    }
}

template <int KT, int N>
__global__ void __launch_bounds__(TcCfg<N>::THREADS, TcCfg<N>::MIN_CTAS) matmul_tc_kernel(const TcArgs a) {
    using Cfg = TcCfg<N>;
    constexpr int G = Cfg::G;
    constexpr int NPT = N / G;  // accumulator columns per thread
    constexpr int TC_BK = Cfg::BK;
    constexpr int TC_SUPER = Cfg::SUPER;
    constexpr int TC_A_COLS = Cfg::A_COLS;
    constexpr int TC_PROMO = Cfg::PROMO;
    constexpr int TC_A_STAGES = Cfg::A_STAGES;
    constexpr int TC_ACC_COL = Cfg::ACC_COL;
    constexpr int TC_TMEM_COLS = Cfg::TMEM_COLS;
    constexpr int TC_IMG_BYTES = Cfg::IMG_BYTES;
    constexpr int TC_SLOT_BYTES = Cfg::SLOT_BYTES;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[TC_SLOTS];      // rhs image + x2 of a slot landed
    __shared__ __align__(8) uint64_t bar_sfree[TC_SLOTS];     // MMAs reading a slot are done
    __shared__ __align__(8) uint64_t bar_ready[TC_A_STAGES];  // A stage written by the generators
    __shared__ __align__(8) uint64_t bar_empty[TC_A_STAGES];  // MMAs reading an A stage are done
    __shared__ __align__(8) uint64_t bar_acc[2];              // accumulator group complete
    __shared__ __align__(8) uint64_t bar_free[2];             // accumulators added to the registers
    __shared__ __align__(8) uint64_t bar_drain;               // give-up path: every issued MMA has completed
    __shared__ uint32_t tmem_base_slot;
    __shared__ int fail_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    constexpr bool FW = Cfg::FETCH_WARP;
    const bool is_ctl_warp = warp == 4 * G;
    const bool is_fetch_warp = FW && warp == 4 * G + 1;
    const bool is_gen = warp < 4 * G;
    const int g = tid >> 7;            // generator group
    const int row_local = tid & 127;  // row of the block = tensor-memory lane

    auto slot_img = [&](int sl) { return smem_raw + sl * TC_SLOT_BYTES; };
    auto slot_x2 = [&](int sl) { return reinterpret_cast<float *>(smem_raw + sl * TC_SLOT_BYTES + TC_IMG_BYTES); };

    int64_t item = blockIdx.x;
    const int64_t b = item % a.batch.count;
    item /= a.batch.count;
    const int64_t r = a.rb_begin + item % a.row_blocks;
    const int kb = (int)(item / a.row_blocks);  // block of N rhs columns

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
    const int tiles = band_hi > band_lo ? (band_hi + TC_BK - 1) / TC_BK - tile_lo : 0;
    const int super_lo = tile_lo / TC_SUPER;
    const int supers = tiles > 0 ? (tile_lo + tiles - 1) / TC_SUPER - super_lo + 1 : 0;
    // a.images: fp16 images; a.image_slot_stride: bytes between image slots (0: rhs shared by all batches)
    const int64_t img_rec = (a.image_slot_stride ? b : 0) * a.k_blocks + kb;  // (image slot, column block)
    const unsigned char *images = reinterpret_cast<const unsigned char *>(a.images) + img_rec * (a.tiles * (int64_t)TC_IMG_BYTES);
    const float *inv_scale = a.col_inv_scale + img_rec * TC_SCALE_WORDS;
    const int64_t k_here = min((int64_t)N, a.k - (int64_t)kb * N);  // columns of this block

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < TC_SLOTS; s++) {
            // kernels without a phase: 32 lanes' cp.async arrivals + the bulk copy's expect_tx arrival;
            // with one: the expect_tx arrival + lane 0's arrival after the warp's stores
            mbar_init(&bar_full[s], KernelFn<KT>::PHASE ? 2 : 33);
            mbar_init(&bar_sfree[s], 1);
        }
#pragma unroll
        for (int s = 0; s < TC_A_STAGES; s++) {
            mbar_init(&bar_ready[s], 4 * Cfg::SET_GROUPS);
            mbar_init(&bar_empty[s], 1);
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            mbar_init(&bar_acc[i], 1);
            mbar_init(&bar_free[i], 4 * G);
        }
        mbar_init(&bar_drain, 1);
        fail_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (is_ctl_warp) tmem_alloc(&tmem_base_slot, TC_TMEM_COLS);
    tc_fence_before();
    // Separable phases: origin x0 = the block's middle row; a block with a row too far from x0
    // (unsorted inputs) keeps the per-entry sine / cosine.
    const float x0 = KernelFn<KT>::PHASE ? x1[min(r * KM_BLOCK_SIZE + KM_BLOCK_SIZE / 2, a.m - 1) * a.x1.s0] : 0.0f;
    const float phase_w = fn.phase_w();
    bool use_ph = false;
    {
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        const bool far = KernelFn<KT>::PHASE && tid < 128 && row < a.m &&
                         fabsf(phase_w * (x1[row * a.x1.s0] - x0)) > KM_PHASE_MAX_ROW_ARG;
        const int any_far = __syncthreads_or(far ? 1 : 0);
        use_ph = KernelFn<KT>::PHASE && !any_far;
    }
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    // instruction descriptor: D fp32, A / B fp16 (format code 0), both K-major, M = 128, N
    constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
    bool failed = false;

    float acc[NPT];
#pragma unroll
    for (int c = 0; c < NPT; c++) acc[c] = 0.0f;

    if (is_ctl_warp || is_fetch_warp) {
    // ------------------------------------------------------ slot fetches (all lanes of a helper warp)
    // Slots are fetched in increasing order, so a phase kernel keeps the x2 values of the
    // next fetch in registers (loaded one fetch ahead: the load latency never stalls the warp).
    float x_ahead[TC_SCOLS / 32];
    auto load_ahead = [&](int sr) {
#pragma unroll
        for (int u = 0; u < TC_SCOLS / 32; u++) {
            const int64_t j = (int64_t)(super_lo + sr) * TC_SCOLS + lane + 32 * u;
            x_ahead[u] = (sr < supers && j < n) ? __ldg(x2 + j * a.x2.s0) : 0.0f;
        }
    };
    int fetched = 0, landed = 0;  // slots whose copies were issued / (set when a wait gives up) were seen complete
    auto fetch = [&](int sr) {
        fetched = sr + 1;
        const int sl = sr % TC_SLOTS;
        const int64_t sup = super_lo + sr;
        float *xs = slot_x2(sl);
        if (lane == 0) {
            mbar_expect_tx(&bar_full[sl], TC_IMG_BYTES);
            bulk_copy_g2s(slot_img(sl), images + sup * TC_IMG_BYTES, TC_IMG_BYTES, &bar_full[sl]);
        }
        if constexpr (KernelFn<KT>::PHASE) {
#pragma unroll
            for (int u = 0; u < TC_SCOLS / 32; u++) {
                const int jj = lane + 32 * u;
                const float xv = x_ahead[u];
                xs[jj] = xv;
                if (use_ph) {
                    const float ph = phase_w * (xv - x0);
                    xs[TC_SCOLS + jj] = cos_approx(ph);
                    xs[2 * TC_SCOLS + jj] = sin_approx(ph);
                }
            }
            load_ahead(sr + 1);
            __syncwarp();  // every lane's stores precede lane 0's (releasing) arrival
            if (lane == 0) mbar_arrive(&bar_full[sl]);
        } else {
#pragma unroll
            for (int u = 0; u < TC_SCOLS / 32; u++) {
                const int jj = lane + 32 * u;
                const int64_t j = sup * TC_SCOLS + jj;
                const bool valid = j < n;
                cp_async4_zfill(xs + jj, x2 + (valid ? j : 0) * a.x2.s0, valid);
            }
            cp_async_mbar_arrive(&bar_full[sl]);
        }
    };
    if (is_ctl_warp) {
        // ---------------------------------------------------------------- MMA issue (lane 0)
        if constexpr (!FW) {
            if constexpr (KernelFn<KT>::PHASE) load_ahead(0);
            for (int sr = 0; sr < min(supers, TC_SLOTS); sr++) fetch(sr);
        }

        // B: core matrices of 8 columns (N) x 16 bytes (8 fp16 along K); K-adjacent matrices N * 16 bytes apart
        constexpr uint32_t lbo_b = N * 16, sbo = 128;
        constexpr uint64_t slot_step = (uint64_t)TC_SLOT_BYTES >> 4;
        constexpr uint64_t part_step = (uint64_t)(TC_SCOLS * N * 2) >> 4;  // hi -> lo image
        constexpr uint64_t kstep = (uint64_t)(2 * lbo_b) >> 4;             // 16 band columns = 2 chunks
        const uint64_t d_b0 = smem_desc(smem_u32(slot_img(0)), lbo_b, sbo);
        int s = 0, use = 0, in_grp = 0, grp = 0;
        for (int t = 0; t < tiles; t++) {
            const int ta = tile_lo + t;
            const int q = ta & (TC_SUPER - 1);
            const int sr = ta / TC_SUPER - super_lo;
            const int sl = sr % TC_SLOTS;
            const int ai = grp & 1;
            const bool grp_first = in_grp == 0;
            const bool grp_last = in_grp == TC_PROMO - 1 || t == tiles - 1;
            const bool slot_first = t == 0 || q == 0;
            const bool slot_last = q == TC_SUPER - 1 || t == tiles - 1;
            bool ok = true;
            if (slot_first) ok = mbar_wait(&bar_full[sl], (unsigned)((sr / TC_SLOTS) & 1), a.wait_polls);
            // the accumulator must have been collected by every generator warp
            if (ok && grp_first && grp >= 2) ok = mbar_wait(&bar_free[ai], (unsigned)(((grp >> 1) - 1) & 1), a.wait_polls);
            if (ok) ok = mbar_wait(&bar_ready[s], (unsigned)(use & 1), a.wait_polls);
            if (!__all_sync(0xffffffffu, ok)) {
                failed = true;
                landed = sr;
                break;
            }
            tc_fence_after();
            if (lane == 0) {
                const uint32_t d_tmem = tmem_base + (uint32_t)(TC_ACC_COL + ai * N);
                const uint32_t a_hi = tmem_base + (uint32_t)(s * TC_A_COLS), a_lo = a_hi + 8;
                const uint64_t b_hi = d_b0 + sl * slot_step + (uint64_t)(q * (TC_BK / 16)) * kstep, b_lo = b_hi + part_step;
                // the small cross terms first, hi * hi last
#pragma unroll
                for (int ks = 0; ks < TC_BK / 16; ks++) {
                    mma_f16_ts(d_tmem, a_hi + ks * 16, b_lo + ks * kstep, idesc, (ks > 0 || !grp_first) ? 1u : 0u);
                    mma_f16_ts(d_tmem, a_lo + ks * 16, b_hi + ks * kstep, idesc, 1u);
                }
#pragma unroll
                for (int ks = 0; ks < TC_BK / 16; ks++) mma_f16_ts(d_tmem, a_hi + ks * 16, b_hi + ks * kstep, idesc, 1u);
                mma_commit(&bar_empty[s]);
                if (slot_last) mma_commit(&bar_sfree[sl]);
                if (grp_last) mma_commit(&bar_acc[ai]);
            }
            __syncwarp();
            // after the first tile of a slot: the previous slot is re-filled once its MMAs are done
            if (!FW && slot_first && sr >= 1 && sr - 1 + TC_SLOTS < supers) {
                const int prev = sr - 1;
                ok = mbar_wait(&bar_sfree[prev % TC_SLOTS], (unsigned)((prev / TC_SLOTS) & 1), a.wait_polls);
                if (!__all_sync(0xffffffffu, ok)) {
                    failed = true;
                    landed = sr;
                    break;
                }
                fetch(prev + TC_SLOTS);
            }
            if (++s == TC_A_STAGES) {
                s = 0;
                use++;
            }
            if (++in_grp == TC_PROMO) {
                in_grp = 0;
                grp++;
            }
        }
        if (failed) {
            // Give-up path: nothing asynchronous may still be running when the CTA exits and its
            // shared memory goes to the next CTA.  The bulk copies that were issued and not yet
            // seen complete are awaited (with the full poll limit: they do arrive).
            for (int sr = landed; sr < fetched; sr++)
                mbar_wait(&bar_full[sr % TC_SLOTS], (unsigned)((sr / TC_SLOTS) & 1), TC_WAIT_POLLS);
            if (lane == 0) atomicExch(&fail_flag, 1);
        }
        // no cp.async may be in flight when the CTA exits
        cp_async_wait<0>();
        __syncwarp();
    } else if (is_fetch_warp) {
        // ------------------------------------------------------------- slot fetches (N >= 64)
        if constexpr (KernelFn<KT>::PHASE) load_ahead(0);
        for (int sr = 0; sr < supers; sr++) {
            if (sr >= TC_SLOTS) {
                // the slot's previous content has been read by its MMAs (whose A tiles the generators
                // wrote after reading the slot's x2 values)
                const int prev = sr - TC_SLOTS;
                const bool ok = mbar_wait(&bar_sfree[prev % TC_SLOTS], (unsigned)((prev / TC_SLOTS) & 1), a.wait_polls);
                if (!__all_sync(0xffffffffu, ok)) {
                    failed = true;
                    break;
                }
            }
            fetch(sr);
        }
        // No copy may be in flight when the CTA exits: the last copy into every slot has landed
        // (immediately true unless a wait gave up; then with the full poll limit: copies do arrive).
        for (int sr = max(0, fetched - TC_SLOTS); sr < fetched; sr++)
            mbar_wait(&bar_full[sr % TC_SLOTS], (unsigned)((sr / TC_SLOTS) & 1), TC_WAIT_POLLS);
        if (failed && lane == 0) atomicExch(&fail_flag, 1);
        cp_async_wait<0>();
        __syncwarp();
    }
    } else {
        // ----------------------------------------------------------------------- generators
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        const float x1v = row < a.m ? x1[row * a.x1.s0] : x0;
        // separable phase factors of this row
        const float ph_i = phase_w * (x1v - x0);
        const f32x2 ci2 = splat2(use_ph ? cos_approx(ph_i) : 1.0f), si2 = splat2(use_ph ? sin_approx(ph_i) : 0.0f);
        const uint32_t tmem_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);

        auto collect = [&](int ai) {
            tc_fence_after();
#pragma unroll
            for (int q = 0; q < NPT / 16; q++) {
                uint32_t v[16];
                tmem_ld16_nowait(tmem_lane + (uint32_t)(TC_ACC_COL + ai * N + g * NPT + q * 16), v);
                tmem_ld_wait16(v);
#pragma unroll
                for (int u = 0; u < 16; u++) acc[q * 16 + u] += __uint_as_float(v[u]);
            }
            tc_fence_before();
        };

        const int groups = (tiles + TC_PROMO - 1) / TC_PROMO;  // accumulator groups of this row block
        int collected = 0;                                      // groups this thread has added to its registers
        auto collect_group = [&](int cg, bool release) {
            if (!mbar_wait_warp(&bar_acc[cg & 1], (unsigned)((cg / 2) & 1), a.wait_polls)) {
                failed = true;
                return false;
            }
            collect(cg & 1);
            __syncwarp();
            // (the issuing warp waits for these arrivals before group cg + 2 overwrites the accumulator)
            if (release && cg + 2 < groups && lane == 0) mbar_arrive(&bar_free[cg & 1]);
            return true;
        };
        constexpr int TS = Cfg::TILE_SETS, GS = Cfg::SET_GROUPS;
        const int set = g / GS, gi = g % GS;  // this thread's set of groups and its group's place in it
        int seen_sr = -1;                      // last slot this thread has waited for
        for (int t = set; t < tiles; t += TS) {
            const int ta = tile_lo + t;
            const int q = ta & (TC_SUPER - 1);
            const int sr = ta / TC_SUPER - super_lo;
            const int sl = sr % TC_SLOTS;
            const int s = t % TC_A_STAGES, use = t / TC_A_STAGES;
            const int grp = t / TC_PROMO;
            if (sr != seen_sr) {
                if (!mbar_wait_warp(&bar_full[sl], (unsigned)((sr / TC_SLOTS) & 1), a.wait_polls)) {
                    failed = true;
                    break;
                }
                seen_sr = sr;
            }
            // an accumulator that is about to be reused (by accumulator group grp) is first added
            // to the registers: every warp collects every group once, in order
            while (collected + 2 <= grp) {
                if (!collect_group(collected, true)) break;
                collected++;
            }
            if (failed) break;
            // stage s must have been read by the MMAs of tile t - TC_A_STAGES
            if (use > 0) {
                if (!mbar_wait_warp(&bar_empty[s], (unsigned)((use - 1) & 1), a.wait_polls)) {
                    failed = true;
                    break;
                }
                tc_fence_after();
            }
            const float4 *xs = reinterpret_cast<const float4 *>(slot_x2(sl) + q * TC_BK);
            const int j0 = ta * TC_BK;
            const bool partial = j0 < band_lo || j0 + TC_BK > band_hi;
            // 16 entries at a time: hi = kv truncated to fp16 (= the fp32 value with 10 mantissa
            // bits for kv in fp16's normal range; below 2^-14 the two differ by less than 2^-24,
            // far under the tolerance), lo = kv - hi rounded to fp16.  Tensor-memory columns of
            // the 16 band columns: [8 hi pairs | 8 lo pairs].
#pragma unroll
            for (int half = gi; half < TC_BK / 16; half += GS) {  // this group's 16-column steps
                // packed f32x2 arithmetic: two entries per FP32 instruction, kept as pairs up to the
                // fp16 conversions (8 hi words, 8 lo words: the 16 tensor-memory columns of this step)
                const ulonglong2 *xs2 = reinterpret_cast<const ulonglong2 *>(xs);
                const f32x2 x1v2 = splat2(x1v);
                f32x2 kv2[8];
                if (use_ph) {
                    // cos(W tau) = c_i c_j + s_i s_j from the slot's per-column factors
                    const ulonglong2 *cj2 = xs2 + TC_SCOLS / 4, *sj2 = xs2 + 2 * (TC_SCOLS / 4);
#pragma unroll
                    for (int h = 0; h < 4; h++) {
                        const ulonglong2 xv = xs2[half * 4 + h], cj = cj2[half * 4 + h], sj = sj2[half * 4 + h];
                        kv2[2 * h] = fn.unscaled2_ph(sub2(x1v2, xv.x), fma2(ci2, cj.x, mul2(si2, sj.x)), 0ull);
                        kv2[2 * h + 1] = fn.unscaled2_ph(sub2(x1v2, xv.y), fma2(ci2, cj.y, mul2(si2, sj.y)), 0ull);
                    }
                } else {
#pragma unroll
                    for (int h = 0; h < 4; h++) {
                        const ulonglong2 xv = xs2[half * 4 + h];
                        kv2[2 * h] = fn.unscaled2(sub2(x1v2, xv.x));
                        kv2[2 * h + 1] = fn.unscaled2(sub2(x1v2, xv.y));
                    }
                }
                if (partial) {
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int j = j0 + half * 16 + 2 * u;
                        const f32x2 keep = ((j >= band_lo && j < band_hi) ? 0x00000000ffffffffull : 0ull) |
                                           ((j + 1 >= band_lo && j + 1 < band_hi) ? 0xffffffff00000000ull : 0ull);
                        kv2[u] &= keep;
                    }
                }
                // hi = kv truncated to fp16 precision, lo = kv - hi rounded: 8 + 8 words, one store
                split_store16_pairs(tmem_lane + (uint32_t)(s * TC_A_COLS + half * 16), kv2);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_ready[s]);
        }

        // drain: the groups not collected yet (the last two, and any a set of groups had no tile in)
        while (!failed && collected < groups) {
            if (!collect_group(collected, true)) break;
            collected++;
        }
        if (failed) atomicExch(&fail_flag, 1);
    }

    tc_fence_before();
    __syncthreads();
    if (fail_flag) {
        // a wait gave up: the status word says so, and the rows of this CTA become NaN so that the
        // failure also shows in whatever is computed from the result, without a host synchronisation
        if (tid == 0) atomicExch(a.status, 1);
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        if (is_gen && g == 0 && row < a.m) {
            float *orow = out + (row - a.rb_begin * KM_BLOCK_SIZE) * a.out.s0 + (int64_t)kb * N * a.out.s1;
            for (int c = 0; c < (int)k_here; c++) orow[c * a.out.s1] = __int_as_float(0x7fc00000);
        }
    } else if (is_gen) {
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        if (row < a.m) {
            // output scale times the inverse of the rhs column scale
            float *orow = out + (row - a.rb_begin * KM_BLOCK_SIZE) * a.out.s0 + (int64_t)kb * N * a.out.s1;
            const bool vec_ok = a.out.s1 == 1 && (a.out.s0 % 4 == 0) && (k_here % 4 == 0) &&
                                ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
            const float scale = fn.scale;
#pragma unroll
            for (int cl = 0; cl < NPT; cl += 4) {
                const int c = g * NPT + cl;  // column inside this block of N
                if (c < k_here) {
                    const float4 is = *reinterpret_cast<const float4 *>(inv_scale + c);
                    const float4 v = make_float4(acc[cl] * (is.x * scale), acc[cl + 1] * (is.y * scale),
                                                 acc[cl + 2] * (is.z * scale), acc[cl + 3] * (is.w * scale));
                    if (vec_ok) {
                        *reinterpret_cast<float4 *>(orow + c) = v;
                    } else {
                        const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int u = 0; u < 4; u++)
                            if (c + u < k_here) orow[(c + u) * a.out.s1] = e[u];
                    }
                }
            }
        }
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
        tmem_free(tmem_base, TC_TMEM_COLS);
    }
}

// workspace: [status, 256 B][per (image slot, column block): column maxima and inverse scales][images]
static int tc_n_pad(int64_t k) { return k <= 16 ? 16 : (k <= 32 ? 32 : (k <= 64 ? 64 : 128)); }
static int64_t tc_k_blocks(int64_t k) { return std::max<int64_t>(1, ceil_div(k, TC_MAX_N)); }
static size_t tc_scale_bytes(int64_t slots, int64_t kblocks) {
    return (size_t)(slots * kblocks) * TC_SCALE_WORDS * sizeof(float);
}

static size_t tc_workspace_bytes(const Batch &b, int64_t n, int64_t k, const View<const float> &rhs) {
    const int64_t supers = ceil_div(n, TC_SCOLS);
    const int64_t slots = tc_slots(b, rhs), kblocks = tc_k_blocks(k);
    return (size_t)TC_STATUS_BYTES + tc_scale_bytes(slots, kblocks) +
           (size_t)(slots * kblocks * supers) * (2 * TC_SCOLS * tc_n_pad(k)) * 2;
}

template <int KT, int N>
static int launch_tc_n(const TcArgs &a, cudaStream_t s) {
    const int64_t items = a.batch.count * a.row_blocks * a.k_blocks;
    if (items > 0x7fffffffLL) {
        set_error("km_matmul_tc_f32: too many work items (%lld)", (long long)items);
        return KM_ERR_UNSUPPORTED;
    }
    auto kernel = matmul_tc_kernel<KT, N>;
    constexpr size_t smem = TcCfg<N>::SMEM_BYTES;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(matmul_tc)");
    kernel<<<(unsigned)items, TcCfg<N>::THREADS, smem, s>>>(a);
    KM_CHECK_LAUNCH("km_matmul_tc_f32 launch");
    return KM_OK;
}

template <int KT>
static int launch_tc(const TcArgs &a, int n_pad, cudaStream_t s) {
    if (n_pad == 16) return launch_tc_n<KT, 16>(a, s);
    if (n_pad == 32) return launch_tc_n<KT, 32>(a, s);
    if (n_pad == 64) return launch_tc_n<KT, 64>(a, s);
    return launch_tc_n<KT, 128>(a, s);
}

static int tc_matmul(int kernel_type, TcArgs a, const View<const float> &rhs, void *workspace, cudaStream_t s) {
    const int64_t slots = tc_slots(a.batch, rhs);
    const int64_t supers = ceil_div(a.n, TC_SCOLS);
    const int n_pad = tc_n_pad(a.k);
    const int64_t kblocks = tc_k_blocks(a.k);
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    a.status = reinterpret_cast<int *>(ws);
    unsigned *scales = reinterpret_cast<unsigned *>(ws + TC_STATUS_BYTES);
    __half *images = reinterpret_cast<__half *>(ws + TC_STATUS_BYTES + tc_scale_bytes(slots, kblocks));
    a.images = reinterpret_cast<const float *>(images);
    a.image_slot_stride = slots > 1 ? 1 : 0;  // this kernel only asks whether every batch has its own images
    a.k_blocks = (int)kblocks;
    a.tiles = supers;                         // 64-column groups per image
    a.n_pad = n_pad;
    a.col_inv_scale = reinterpret_cast<const float *>(scales) + TC_MAX_N;
    a.wait_polls = current_wait_polls();
    cudaError_t err = cudaMemsetAsync(scales, 0, tc_scale_bytes(slots, kblocks), s);
    if (err != cudaSuccess) return cuda_fail(err, "km_matmul_tc_f32 cudaMemsetAsync");
    const unsigned max_blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(a.n, 16), 148 * 8));
    tc_colmax_kernel<<<max_blocks, 256, 0, s>>>(a.batch, slots, a.n, a.k, n_pad, (int)kblocks, rhs, scales, a.status);
    KM_CHECK_LAUNCH("km_matmul_tc_f32 column-maximum launch");
    const int64_t total = slots * kblocks * supers * (int64_t)(TC_SCOLS * n_pad);
    const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(total, 256), 148 * 32));
    tc_rhs_images_kernel<<<blocks, 256, 0, s>>>(a.batch, slots, a.n, a.k, n_pad, (int)kblocks, supers, rhs, images, scales);
    KM_CHECK_LAUNCH("km_matmul_tc_f32 pre-pass launch");
    switch (kernel_type) {
    case KM_KERNEL_RBF: return launch_tc<KM_KERNEL_RBF>(a, n_pad, s);
    case KM_KERNEL_SPECTRAL: return launch_tc<KM_KERNEL_SPECTRAL>(a, n_pad, s);
    default: return launch_tc<KM_KERNEL_LOCALLY_PERIODIC>(a, n_pad, s);
    }
}

}  // namespace km

extern "C" size_t km_matmul_tc_workspace_bytes(const km_batch *batch, int64_t n, int64_t k, const km_view *rhs) {
    using namespace km;
    Batch b;
    if (batch == nullptr || rhs == nullptr || make_batch(batch, &b) != KM_OK || n < 0 || k <= 0) return 0;
    return tc_workspace_bytes(b, n, k, make_view<const float>(rhs, b));
}

static int km_matmul_tc_entry(const char *name, int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                              const km_view *x1, const km_view *x2, const km_view *rhs, const km_view *params,
                              const km_view *start, const km_view *end, const km_view *out, int64_t rb_begin,
                              int64_t rb_count, void *workspace, size_t workspace_bytes, void *stream) {
    using namespace km;
    KM_REQUIRE(valid_kernel_type(kernel_type), KM_ERR_INVALID_ARGUMENT, "%s: unknown kernel type %d", name, kernel_type);
    KM_REQUIRE(batch && x1 && x2 && rhs && params && start && end && out, KM_ERR_INVALID_ARGUMENT, "%s: null argument", name);
    KM_REQUIRE(m >= 0 && n >= 0 && k >= 0 && n <= 0x7fffffffLL - 64 && m <= 0x7fffffffLL * 64, KM_ERR_INVALID_ARGUMENT,
               "%s: bad sizes", name);
    TcArgs a;
    int rc = make_batch(batch, &a.batch);
    if (rc != KM_OK) return rc;
    const int64_t total_blocks = ceil_div(m, KM_BLOCK_SIZE);
    if (rb_count < 0) rb_count = total_blocks - rb_begin;
    KM_REQUIRE(rb_begin >= 0 && rb_count >= 0 && rb_begin + rb_count <= total_blocks, KM_ERR_INVALID_ARGUMENT,
               "%s: row-block window [%lld, %lld) outside [0, %lld)", name, (long long)rb_begin,
               (long long)(rb_begin + rb_count), (long long)total_blocks);
    if (a.batch.count == 0 || rb_count == 0 || k == 0) return KM_OK;
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
    a.row_blocks = rb_count;
    a.rb_begin = rb_begin;
    a.x1 = make_view<const float>(x1, a.batch);
    a.x2 = make_view<const float>(x2, a.batch);
    a.params = make_view<const float>(params, a.batch);
    a.start = make_view<const int>(start, a.batch);
    a.end = make_view<const int>(end, a.batch);
    a.out = make_view<float>(out, a.batch);
    return tc_matmul(kernel_type, a, make_view<const float>(rhs, a.batch), workspace, static_cast<cudaStream_t>(stream));
}

extern "C" int km_matmul_tc_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                                const km_view *x1, const km_view *x2, const km_view *rhs, const km_view *params,
                                const km_view *start, const km_view *end, const km_view *out, void *workspace,
                                size_t workspace_bytes, void *stream) {
    return km_matmul_tc_entry("km_matmul_tc_f32", kernel_type, batch, m, n, k, x1, x2, rhs, params, start, end, out, 0, -1,
                              workspace, workspace_bytes, stream);
}

extern "C" int km_matmul_tc_rows_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                                     const km_view *x1, const km_view *x2, const km_view *rhs, const km_view *params,
                                     const km_view *start, const km_view *end, const km_view *out,
                                     int64_t row_block_begin, int64_t row_block_count, void *workspace,
                                     size_t workspace_bytes, void *stream) {
    return km_matmul_tc_entry("km_matmul_tc_rows_f32", kernel_type, batch, m, n, k, x1, x2, rhs, params, start, end, out,
                              row_block_begin, row_block_count, workspace, workspace_bytes, stream);
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

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
// ONE 32-column tile: the small cross terms are issued first, the four hi*hi MMAs last, and
// the finished tile is added to fp32 registers (round-to-nearest) while the next tiles are
// generated -- two accumulators in tensor memory alternate.
//
// Every wait on an mbarrier is bounded; a wait that gives up records a code in the status word
// of the workspace and the CTA leaves through the normal exit (tensor memory released).
#include "km_common.cuh"

namespace km {

constexpr int TC_BK = 32;             // band columns (GEMM K) per stage
constexpr int TC_STAGES = 2;
constexpr int TC_STATUS_BYTES = 256;  // status word + padding in front of the images
constexpr unsigned TC_WAIT_POLLS = 400000;

struct TcArgs {
    Batch batch;
    int64_t m, n, k;
    int64_t row_blocks, rb_begin;
    int k_blocks;  // blocks of n_pad rhs columns
    int n_pad;     // GEMM N per block: multiple of 16, <= 256
    int tmem_cols; // power of two >= max(32, n_pad)
    int64_t tiles; // ceil(n / TC_BK)
    View<const float> x1, x2, params;
    View<const int> start, end;
    View<float> out;
    const float *images;         // [slot][k block][tile][hi|lo][chunk][c][4]
    int64_t image_slot_stride;   // floats between batch slots (0: rhs shared by all batches)
    int *status;
};

// ---------------------------------------------------------------------------- PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity.  false = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity) {
    const uint32_t addr = smem_u32(bar);
    for (unsigned poll = 0; poll < TC_WAIT_POLLS; poll++) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(2000u)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void *dst, const void *src, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t *smem_dst, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t taddr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// K-major, no swizzle: core matrices of 8 rows x 16 bytes stored as 128 contiguous bytes;
// `lbo` = bytes between core matrices adjacent in K, `sbo` = bytes between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}
// D (fp32, tensor memory) (+)= A (smem, tf32) . B (smem, tf32); M = 128, N from idesc, K = 8.
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

// ------------------------------------------------------------------------- rhs images pre-pass

// Writes, for every (slot, k block, 32-column tile), the hi and lo parts of the rhs tile in the
// K-major core-matrix layout: part[chunk = jj / 4][c][jj % 4], c the column inside the k block.
// Rows past n and columns past k are zero.  Also clears the status word.
__global__ void __launch_bounds__(256) tc_rhs_images_kernel(Batch batch, int64_t slots, int64_t n, int64_t k,
                                                            int64_t tiles, int k_blocks, int n_pad,
                                                            View<const float> rhs, float *images, int *status) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *status = 0;
    const int64_t per_tile = 2LL * TC_BK * n_pad;
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
        const float hi = tf32_hi(v);
        float *img = images + ((slot * k_blocks + kb) * tiles + tile) * per_tile;
        const int64_t off = (int64_t)(jj >> 2) * (n_pad * 4) + c * 4 + (jj & 3);
        img[off] = hi;
        img[(int64_t)TC_BK * n_pad + off] = v - hi;
    }
}

// ----------------------------------------------------------------------------------- kernel

// N = GEMM N (rhs columns per CTA, 16 .. 128); G threads per row: 128 * G threads, thread
// (row = tid % 128, g = tid / 128) generates the columns [g * 32 / G, (g + 1) * 32 / G) of
// every tile and owns the output columns [g * N / G, (g + 1) * N / G) of its row.
template <int KT, int N, int G>
__global__ void __launch_bounds__(128 * G) matmul_tc_kernel(const TcArgs a) {
    constexpr int A_PART = 128 * TC_BK;  // floats per hi / lo part of an A stage
    constexpr int STAGE_FLOATS = 2 * A_PART + 2 * TC_BK * N;
    constexpr int NPT = N / G;  // accumulator columns per thread
    static_assert(NPT % 8 == 0, "columns per thread must be a multiple of 8");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[TC_STAGES];   // rhs images landed
    __shared__ __align__(8) uint64_t bar_empty[TC_STAGES];  // MMAs of the stage are done
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ __align__(16) float xs[2][TC_BK];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int row_local = tid & 127;
    const int g = tid >> 7;

    float *stage_base = reinterpret_cast<float *>(smem_raw);
    auto a_hi = [&](int s) { return stage_base + s * STAGE_FLOATS; };
    auto a_lo = [&](int s) { return stage_base + s * STAGE_FLOATS + A_PART; };
    auto b_img = [&](int s) { return stage_base + s * STAGE_FLOATS + 2 * A_PART; };

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

    const int64_t row = r * KM_BLOCK_SIZE + row_local;
    const float x1v = row < a.m ? x1[row * a.x1.s0] : 0.0f;
    const float *images = a.images + (a.image_slot_stride ? b * a.image_slot_stride : 0) +
                          (int64_t)kb * a.tiles * (2LL * TC_BK * N);

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < TC_STAGES; s++) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(&tmem_base_slot, (unsigned)a.tmem_cols);
    // x2 values of the first tile
    if (tiles > 0 && tid < TC_BK) {
        const int j = tile_lo * TC_BK + tid;
        xs[0][tid] = j < n ? x2[(int64_t)j * a.x2.s0] : 0.0f;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    // this thread's window of an accumulator: its lane quarter, its column share
    const uint32_t tmem_mine = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(g * NPT);

    // instruction descriptor: D fp32, A / B tf32, both K-major, M = 128, N
    constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
    constexpr uint32_t img_bytes = 2u * TC_BK * N * sizeof(float);
    bool failed = false;

    float acc[NPT];
#pragma unroll
    for (int c = 0; c < NPT; c++) acc[c] = 0.0f;

    // adds the finished tile held by accumulator `s` to the registers
    auto collect = [&](int s) {
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < NPT; c0 += 8) {
            float v[8];
            tmem_ld8(tmem_mine + (uint32_t)(s * N + c0), v);
#pragma unroll
            for (int u = 0; u < 8; u++) acc[c0 + u] += v[u];
        }
        tc_fence_before();
    };

    for (int t = 0; t < tiles; t++) {
        const int s = t % TC_STAGES;
        const int use = t / TC_STAGES;
        const int jt = tile_lo + t;
        // the MMAs of the tile that used this stage (and this accumulator) before must be done
        if (use > 0 && !mbar_wait(&bar_empty[s], (unsigned)((use - 1) & 1))) failed = true;
        if (__syncthreads_or(failed ? 1 : 0)) {
            failed = true;
            break;
        }
        if (use > 0) collect(s);
        if (tid == 0) {
            mbar_expect_tx(&bar_full[s], img_bytes);
            bulk_copy_g2s(b_img(s), images + (int64_t)jt * (2LL * TC_BK * N), img_bytes, &bar_full[s]);
        }
        // prefetch the x2 values of the next tile (visible after this tile's barrier)
        if (t + 1 < tiles && tid < TC_BK) {
            const int j = (jt + 1) * TC_BK + tid;
            xs[(t + 1) & 1][tid] = j < n ? x2[(int64_t)j * a.x2.s0] : 0.0f;
        }

        // generate the A tile: this thread's row, its share of the 32 columns, 4 at a time
        const int j0 = jt * TC_BK;
        const bool partial = (j0 < band_lo) || (j0 + TC_BK > band_hi);
        float *ah = a_hi(s), *al = a_lo(s);
        const float *xt = xs[t & 1];
#pragma unroll
        for (int q = 0; q < TC_BK / 4 / G; q++) {
            const int chunk = g * (TC_BK / 4 / G) + q;
            const float4 xq = *reinterpret_cast<const float4 *>(xt + chunk * 4);
            float kv[4] = {fn.unscaled(x1v - xq.x), fn.unscaled(x1v - xq.y), fn.unscaled(x1v - xq.z),
                           fn.unscaled(x1v - xq.w)};
            if (partial) {
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int j = j0 + chunk * 4 + u;
                    if (j < band_lo || j >= band_hi) kv[u] = 0.0f;
                }
            }
            float lo[4];
#pragma unroll
            for (int u = 0; u < 4; u++) lo[u] = kv[u] - tf32_hi(kv[u]);
            // [chunk][row][16 bytes]: the tensor core reads only the TF32 bits of kv as "hi"
            *reinterpret_cast<float4 *>(ah + (chunk * 128 + row_local) * 4) = make_float4(kv[0], kv[1], kv[2], kv[3]);
            *reinterpret_cast<float4 *>(al + (chunk * 128 + row_local) * 4) = make_float4(lo[0], lo[1], lo[2], lo[3]);
        }
        fence_async_smem();
        __syncthreads();

        if (tid == 0) {
            if (!mbar_wait(&bar_full[s], (unsigned)(use & 1))) {
                abort_flag = 1;
            } else {
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(s * N);
                const uint32_t ah_addr = smem_u32(ah), al_addr = smem_u32(al);
                const uint32_t bh_addr = smem_u32(b_img(s)), bl_addr = bh_addr + TC_BK * N * 4;
                constexpr uint32_t lbo_a = 128 * 16, lbo_b = N * 16, sbo = 128;
                // cross terms first (tiny accumulator, truncation irrelevant), hi * hi last
#pragma unroll
                for (int ks = 0; ks < TC_BK / 8; ks++) {
                    const uint64_t dah = smem_desc(ah_addr + ks * 2 * lbo_a, lbo_a, sbo);
                    const uint64_t dal = smem_desc(al_addr + ks * 2 * lbo_a, lbo_a, sbo);
                    const uint64_t dbh = smem_desc(bh_addr + ks * 2 * lbo_b, lbo_b, sbo);
                    const uint64_t dbl = smem_desc(bl_addr + ks * 2 * lbo_b, lbo_b, sbo);
                    mma_tf32(d_tmem, dah, dbl, idesc, ks > 0 ? 1u : 0u);
                    mma_tf32(d_tmem, dal, dbh, idesc, 1u);
                }
#pragma unroll
                for (int ks = 0; ks < TC_BK / 8; ks++) {
                    const uint64_t dah = smem_desc(ah_addr + ks * 2 * lbo_a, lbo_a, sbo);
                    const uint64_t dbh = smem_desc(bh_addr + ks * 2 * lbo_b, lbo_b, sbo);
                    mma_tf32(d_tmem, dah, dbh, idesc, 1u);
                }
                mma_commit(&bar_empty[s]);
            }
        }
    }

    // drain: the last tiles still sit in tensor memory
    for (int t = max(0, tiles - TC_STAGES); t < tiles && !failed; t++) {
        if (!mbar_wait(&bar_empty[t % TC_STAGES], (unsigned)((t / TC_STAGES) & 1))) failed = true;
        if (__syncthreads_or((failed || abort_flag) ? 1 : 0)) {
            failed = true;
            break;
        }
        collect(t % TC_STAGES);
    }
    if (__syncthreads_or((failed || abort_flag) ? 1 : 0)) failed = true;

    if (failed) {
        if (tid == 0) atomicExch(a.status, 1);
    } else if (row < a.m) {
        const float scale = fn.scale;
        const int64_t out_row = row - a.rb_begin * KM_BLOCK_SIZE;
        const int64_t col0 = (int64_t)kb * N + g * NPT;
#pragma unroll
        for (int c = 0; c < NPT; c++) {
            if (col0 + c < a.k) out[out_row * a.out.s0 + (col0 + c) * a.out.s1] = acc[c] * scale;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_free(tmem_base, (unsigned)a.tmem_cols);
}

static int64_t tc_slots(const Batch &b, const View<const float> &rhs) {
    bool shared = true;
    for (int d = 0; d < b.ndim; d++) shared = shared && (rhs.bs[d] == 0 || b.size[d] == 1);
    return shared ? 1 : b.count;
}

static int tc_n_pad(int64_t k) { return k <= 16 ? 16 : (k <= 32 ? 32 : (k <= 64 ? 64 : 128)); }

template <int KT, int N, int G>
static int launch_tc_n(const TcArgs &a, cudaStream_t s) {
    const int64_t items = a.batch.count * a.row_blocks * a.k_blocks;
    if (items > 0x7fffffffLL) {
        set_error("km_matmul_tc_f32: too many work items (%lld)", (long long)items);
        return KM_ERR_UNSUPPORTED;
    }
    constexpr size_t smem = (size_t)TC_STAGES * (2 * 128 * TC_BK + 2 * TC_BK * N) * sizeof(float);
    auto kernel = matmul_tc_kernel<KT, N, G>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(matmul_tc)");
    kernel<<<(unsigned)items, 128 * G, smem, s>>>(a);
    KM_CHECK_LAUNCH("km_matmul_tc_f32 launch");
    return KM_OK;
}

template <int KT>
static int launch_tc(const TcArgs &a, cudaStream_t s) {
    switch (a.n_pad) {
    case 16: return launch_tc_n<KT, 16, 1>(a, s);
    case 32: return launch_tc_n<KT, 32, 1>(a, s);
    case 64: return launch_tc_n<KT, 64, 2>(a, s);
    default: return launch_tc_n<KT, 128, 2>(a, s);
    }
}

}  // namespace km

extern "C" size_t km_matmul_tc_workspace_bytes(const km_batch *batch, int64_t n, int64_t k, const km_view *rhs) {
    using namespace km;
    Batch b;
    if (batch == nullptr || rhs == nullptr || make_batch(batch, &b) != KM_OK || n < 0 || k <= 0) return 0;
    const View<const float> rv = make_view<const float>(rhs, b);
    const int n_pad = tc_n_pad(k);
    const int64_t k_blocks = ceil_div(k, n_pad);
    const int64_t tiles = ceil_div(n, TC_BK);
    return (size_t)TC_STATUS_BYTES + (size_t)(tc_slots(b, rv) * k_blocks * tiles) * (2 * TC_BK * n_pad) * sizeof(float);
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
    const int64_t slots = tc_slots(a.batch, rv);
    a.status = static_cast<int *>(workspace);
    float *images = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + TC_STATUS_BYTES);
    a.images = images;
    a.image_slot_stride = slots > 1 ? (int64_t)a.k_blocks * a.tiles * (2LL * TC_BK * a.n_pad) : 0;
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

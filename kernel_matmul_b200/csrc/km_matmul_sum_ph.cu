// Batch sum of spectral components on the tensor cores with PRECOMPUTED phase vectors:
//
//   out[i, :] = sum_{j in band} ( sum_b s_b exp(-tau^2 / 2 l^2) cos(w_b tau) ) rhs[j, :],   tau = x_i - x_j
//
// As in km_matmul_sum_tc.cu the sum over the components is the dot product
//   sum_b s_b cos(w_b (x_i - x_j)) = < phi(x_i), psi(x_j) >,
//   phi(x) = (s_b cos(w_b x), s_b sin(w_b x))_b,   psi(x) = (cos(w_b x), sin(w_b x))_b,
// computed by tcgen05.mma from fp16 hi / lo operands.  That kernel evaluates psi of every tile of
// band columns again for every row block (2B SFU operations and ~10 instructions per column and
// component, a quarter of all it issues) -- although psi depends on the operator only, not on the
// vector it is applied to.  An iterative solver applies one operator many times; so here a
// pre-pass (km_sum_phases_prepare_f32) writes psi of all columns and phi of all rows ONCE, as
// images in exactly the layouts the MMAs take them (psi: per 64-column tile the K-major
// shared-memory image [part: hi, lo][chunk = K / 8][j][8 halfs]; phi: per row the tensor-memory
// words [k-step][8 hi pairs | 8 lo pairs]), and the product kernel copies them: one cp.async.bulk
// of 32 KB per tile, 512 bytes of phi per row.  The phases are taken at the points themselves
// (no block origin): sine and cosine are evaluated in fp64 with exact range reduction
// (sincospi(2 f x)), so the images are correctly rounded whatever the size of x.
//
// Workspace: [per chunk of 64 components: psi images of all ceil(n / 64) tiles][per chunk: phi of
// all m rows]; about (m + n) * 8 * B bytes.
#include <cuda_fp16.h>

#include <cstdlib>
#include <type_traits>

#include "km_tcgen05.cuh"

namespace km {

constexpr int PH_COLS = 64;        // band columns per tile = GEMM N
constexpr int PH_IN_STAGES = 4;    // x2 / rhs tiles in shared memory
constexpr int PH_PSI_STAGES = 3;   // psi tiles in shared memory
constexpr int PH_TMEM_COLS = 256;  // phi (2 * 64) + two C stages of 64
constexpr int PH_C_COL = 128;      // first C column

struct PhasesLayout {
    int64_t chunks, tiles, psi_off[SUM_TC_MAX_TOTAL / SUM_TC_MAX_COMPONENTS], phi_off[SUM_TC_MAX_TOTAL / SUM_TC_MAX_COMPONENTS];
    int64_t bytes;
};
static int chunk_comps(int64_t total, int64_t chunk) {
    return (int)std::min<int64_t>(SUM_TC_MAX_COMPONENTS, total - chunk * SUM_TC_MAX_COMPONENTS);
}
static PhasesLayout phases_layout(int64_t components, int64_t m, int64_t n) {
    PhasesLayout L;
    L.chunks = ceil_div(components, (int64_t)SUM_TC_MAX_COMPONENTS);
    L.tiles = ceil_div(n, (int64_t)PH_COLS);
    int64_t at = 0;
    for (int64_t c = 0; c < L.chunks; c++) {
        const int64_t Bp = (chunk_comps(components, c) + 7) & ~7;
        L.psi_off[c] = at;
        at += L.tiles * Bp * 512;  // stage bytes = 2 parts * (2 Bp / 8) chunks * 64 columns * 16 bytes
    }
    for (int64_t c = 0; c < L.chunks; c++) {
        const int64_t Bp = (chunk_comps(components, c) + 7) & ~7;
        L.phi_off[c] = at;
        at += ((m * Bp * 8 + 255) / 256) * 256;  // per row Bp / 8 k-steps of 16 words
    }
    L.bytes = at;
    return L;
}

size_t sum_phases_workspace_bytes(int64_t components, int64_t m, int64_t n) {
    if (components < 1 || components > SUM_TC_MAX_TOTAL) return 0;
    return (size_t)phases_layout(components, m, n).bytes;
}

// fp32 value -> (fp16 hi part = the value truncated to fp16 precision, fp16 lo part = value - its
// leading 10 mantissa bits, rounded), as km_matmul_sum_tc.cu splits them
__device__ __forceinline__ void split_half(float v, unsigned short &hi, unsigned short &lo) {
    hi = __half_as_ushort(__float2half_rz(v));
    lo = __half_as_ushort(__float2half_rn(v - tf32_hi(v)));
}

// One thread per (chunk-of-4-components, column) of the psi images and per (k-step, row) of the phi
// images; only the tiles [tile_begin, tile_end) and the rows [row_begin, row_end) are written.
__global__ void __launch_bounds__(256) sum_phase_images_kernel(Batch batch, View<const float> params, View<const float> x1,
                                                                View<const float> x2, int64_t m, int64_t n, int64_t comp_begin,
                                                                int B, unsigned char *psi_img, uint32_t *phi_img,
                                                                int64_t tile_begin, int64_t tile_end, int64_t row_begin,
                                                                int64_t row_end) {
    const int Bp = (B + 7) & ~7;
    const int64_t psi_items = (tile_end - tile_begin) * PH_COLS * (Bp / 4), phi_items = (row_end - row_begin) * (Bp / 8);
    const int64_t part_bytes = (int64_t)(2 * Bp / 8) * PH_COLS * 16, stage_bytes = 2 * part_bytes;
    for (int64_t it = blockIdx.x * 256LL + threadIdx.x; it < psi_items + phi_items; it += (int64_t)gridDim.x * 256) {
        if (it < psi_items) {
            const int jj = (int)(it % PH_COLS);
            const int64_t rest = it / PH_COLS;
            const int kc = (int)(rest % (Bp / 4));
            const int64_t tile = tile_begin + rest / (Bp / 4);
            const int64_t j = tile * PH_COLS + jj;
            unsigned short h[8], l[8];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int b = kc * 4 + u;
                float c = 0.0f, s = 0.0f;
                if (b < B && j < n) {
                    const float *th = batch_ptr(params, decompose(batch, comp_begin + b));
                    double sd, cd;
                    sincospi(2.0 * (double)th[params.s0] * (double)x2.data[j * x2.s0], &sd, &cd);
                    c = (float)cd;
                    s = (float)sd;
                }
                split_half(c, h[2 * u], l[2 * u]);
                split_half(s, h[2 * u + 1], l[2 * u + 1]);
            }
            unsigned char *dst = psi_img + tile * stage_bytes + (int64_t)kc * (PH_COLS * 16) + jj * 16;
            auto word = [](unsigned short lo16, unsigned short hi16) { return (uint32_t)lo16 | ((uint32_t)hi16 << 16); };
            *reinterpret_cast<uint4 *>(dst) = make_uint4(word(h[0], h[1]), word(h[2], h[3]), word(h[4], h[5]), word(h[6], h[7]));
            *reinterpret_cast<uint4 *>(dst + part_bytes) = make_uint4(word(l[0], l[1]), word(l[2], l[3]), word(l[4], l[5]), word(l[6], l[7]));
        } else {
            const int64_t pit = it - psi_items;
            const int ks = (int)(pit % (Bp / 8));
            const int64_t row = row_begin + pit / (Bp / 8);
            uint32_t w[16];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int b = ks * 8 + u;
                float c = 0.0f, s = 0.0f;
                if (b < B) {
                    const float *th = batch_ptr(params, decompose(batch, comp_begin + b));
                    double sd, cd;
                    sincospi(2.0 * (double)th[params.s0] * (double)x1.data[row * x1.s0], &sd, &cd);
                    const float sc = th[2 * params.s0];
                    c = sc * (float)cd;
                    s = sc * (float)sd;
                }
                unsigned short ch, cl, sh, sl;
                split_half(c, ch, cl);
                split_half(s, sh, sl);
                w[u] = ch | ((uint32_t)sh << 16);
                w[8 + u] = cl | ((uint32_t)sl << 16);
            }
            uint4 *dst = reinterpret_cast<uint4 *>(phi_img + (row * (Bp / 8) + ks) * 16);
#pragma unroll
            for (int q = 0; q < 4; q++) dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
        }
    }
}

int sum_phases_prepare(const Batch &batch, const View<const float> &params, const View<const float> &x1,
                       const View<const float> &x2, int64_t m, int64_t n, int64_t row_begin, int64_t row_end,
                       int64_t col_begin, int64_t col_end, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    const PhasesLayout L = phases_layout(batch.count, m, n);
    const int64_t tile_begin = col_begin / PH_COLS, tile_end = ceil_div(col_end, (int64_t)PH_COLS);
    if (workspace == nullptr || workspace_bytes < (size_t)L.bytes || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0) {
        set_error("km_sum_phases_prepare_f32: workspace of %lld bytes, 256-byte aligned, needed", (long long)L.bytes);
        return KM_ERR_WORKSPACE;
    }
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    for (int64_t c = 0; c < L.chunks; c++) {
        const int B = chunk_comps(batch.count, c), Bp = (B + 7) & ~7;
        const int64_t items = (tile_end - tile_begin) * PH_COLS * (Bp / 4) + (row_end - row_begin) * (Bp / 8);
        if (items <= 0) continue;
        const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(items, (int64_t)256), 148 * 64);
        sum_phase_images_kernel<<<grid, 256, 0, stream>>>(batch, params, x1, x2, m, n, c * SUM_TC_MAX_COMPONENTS, B, ws + L.psi_off[c],
                                                           reinterpret_cast<uint32_t *>(ws + L.phi_off[c]), tile_begin, tile_end,
                                                           row_begin, row_end);
        KM_CHECK_LAUNCH("km_sum_phases_prepare_f32 launch");
    }
    return KM_OK;
}

// KB: rhs columns held per thread (8 or 16).  Two groups of 128 row threads own the same rows
// (tensor-memory lanes) and alternate tiles, each with its own C stage and partial sums (added at
// the end); a control warp fetches the inputs of the tiles (x2 values and rhs rows by cp.async, the
// psi image by one bulk copy) and issues the MMAs.
//
// MS (KB = 8): the contraction with the rhs tile on the warp-level tensor path (mma.sync m16n8k8,
// 3xTF32) instead of the FMA pipe, as in km_matmul_sum_tc.cu: a thread reads C in the register
// layout of an m16n8 accumulator, multiplies by the envelope and uses the products as the A
// fragment; per 128 entries a warp issues three MMAs and reads 8 bytes of rhs per thread, where the
// FMA form issues 16 packed FMAs and reads 128 bytes.
template <int KB, bool MS>
__global__ void __launch_bounds__(288, 2) matmul_sum_ph_kernel(const SumTcArgs a) {
    static_assert(!MS || KB == 8, "the warp-level contraction is written for 8 rhs columns");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_in[PH_IN_STAGES];     // x2 + rhs tile landed
    __shared__ __align__(8) uint64_t bar_psi[PH_PSI_STAGES];   // psi image landed
    __shared__ __align__(8) uint64_t bar_pfree[PH_PSI_STAGES]; // psi image read by its MMAs (tcgen05.commit)
    __shared__ __align__(8) uint64_t bar_cfull[2];             // C tile complete (tcgen05.commit)
    __shared__ __align__(8) uint64_t bar_cfree[2];             // C tile consumed
    __shared__ __align__(8) uint64_t bar_drain;                // give-up path: every issued MMA has completed
    __shared__ uint32_t tmem_base_slot;
    __shared__ int fail_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const bool is_ctl_warp = warp == 8;
    const int g = tid >> 7;            // row group
    const int row_local = tid & 127;  // row of the block = tensor-memory lane
    const int B = (int)a.comp_count;  // components of this launch: [comp_begin, comp_begin + B)
    const int Bp = (B + 7) & ~7;      // components padded to whole MMA steps (K = 2 Bp)
    const int ksteps = Bp / 8;
    static_assert(SUM_TC_MAX_COMPONENTS == 64, "the MMA issue code covers 1 .. 8 k-steps");

    // every CTA checks that the components share one lengthscale; if not, the FMA-pipe kernel
    // launched next to this one does the work and this CTA leaves at once
    const float ell0 = a.params.data[0];
    int same = 1;
    for (int64_t b = tid; b < a.batch.count; b += blockDim.x)
        same &= (batch_ptr(a.params, decompose(a.batch, b))[0] == ell0) ? 1 : 0;
    if (tid == 0) fail_flag = 0;
    if (!__syncthreads_and(same)) return;
    const float c0 = -(0.5f / (ell0 * ell0)) * KM_LOG2E_F;

    // shared memory: three psi stages (the images as they lie in the workspace), then the input stages
    const int b_part_bytes = (2 * Bp / 8) * PH_COLS * 16;
    const int b_stage_bytes = 2 * b_part_bytes;
    unsigned char *in_base = smem_raw + PH_PSI_STAGES * b_stage_bytes;
    // rhs rows lie in shared memory as pairs of band columns: rs[((jj / 2) * RS + c) * 2 + (jj & 1)];
    // RS = 12 spreads the warp-level form's reads over the banks
    constexpr int RS = MS ? 12 : KB;
    constexpr int IN_STAGE_FLOATS = PH_COLS + PH_COLS * RS;  // x2 values, then rhs rows
    auto b_stage = [&](int st) { return smem_raw + st * b_stage_bytes; };
    auto in_x2 = [&](int st) { return reinterpret_cast<float *>(in_base) + st * IN_STAGE_FLOATS; };
    auto in_rhs = [&](int st) { return reinterpret_cast<float *>(in_base) + st * IN_STAGE_FLOATS + PH_COLS; };

    const int64_t r = a.rb_begin + blockIdx.x;
    const int n = (int)a.n;
    const int band_lo = clamp_int(a.start.data[r * a.start.s0], 0, n);
    const int band_hi = max(band_lo, min(a.end.data[r * a.end.s0], n));
    const int tile_lo = band_lo / PH_COLS;
    const int tiles = band_hi > band_lo ? (band_hi + PH_COLS - 1) / PH_COLS - tile_lo : 0;
    const float *x2 = a.x2.data;
    const float *rhs = a.rhs.data;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < PH_IN_STAGES; s++) mbar_init(&bar_in[s], 32);  // one cp.async arrival per lane
#pragma unroll
        for (int s = 0; s < PH_PSI_STAGES; s++) {
            mbar_init(&bar_psi[s], 1);  // the expect_tx arrival
            mbar_init(&bar_pfree[s], 1);
        }
#pragma unroll
        for (int s = 0; s < 2; s++) {
            mbar_init(&bar_cfull[s], 1);
            mbar_init(&bar_cfree[s], 4);
        }
        mbar_init(&bar_drain, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (is_ctl_warp) tmem_alloc(&tmem_base_slot, PH_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    bool failed = false;

    f32x2 acc2[KB];  // per output column: (sum over even band columns, sum over odd band columns)
#pragma unroll
    for (int c = 0; c < KB; c++) acc2[c] = 0ull;
    // warp-level form: accumulator fragments of the warp's two 16-row tiles (thread lane: rows
    // lane / 4 and lane / 4 + 8 of a tile, output columns 2 (lane % 4) and 2 (lane % 4) + 1)
    float dacc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};

    if (is_ctl_warp) {
        // --------------------------------------------- input fetches (all lanes) + MMA issue (lane 0)
        auto fetch_inputs = [&](int t) {
            const int st = t % PH_IN_STAGES;
            const int64_t j0 = (int64_t)(tile_lo + t) * PH_COLS;
            float *xs = in_x2(st);
            float *rs = in_rhs(st);
#pragma unroll
            for (int u = 0; u < PH_COLS / 32; u++) {
                const int jj = lane + 32 * u;
                const bool valid = j0 + jj < n;
                cp_async4_zfill(xs + jj, x2 + (valid ? j0 + jj : 0) * a.x2.s0, valid);
            }
            // rhs rows in pairs: rs[((jj / 2) * RS + c) * 2 + (jj & 1)] = rhs[j0 + jj][c]
            for (int q = lane; q < PH_COLS * KB; q += 32) {
                const int jj = q / KB, c = q % KB;
                const bool valid = j0 + jj < n && c < a.k;
                cp_async4_zfill(rs + (((jj >> 1) * RS + c) << 1) + (jj & 1),
                                rhs + (valid ? (j0 + jj) * a.rhs.s0 + c * a.rhs.s1 : 0), valid);
            }
            cp_async_mbar_arrive(&bar_in[st]);
        };
        int psi_fetched = 0, psi_seen = 0;  // psi copies issued / seen complete
        auto fetch_psi = [&](int t) {
            psi_fetched = t + 1;
            if (lane == 0) {
                const int ps = t % PH_PSI_STAGES;
                mbar_expect_tx(&bar_psi[ps], (unsigned)b_stage_bytes);
                bulk_copy_g2s(b_stage(ps), a.psi_img + (int64_t)(tile_lo + t) * b_stage_bytes, (unsigned)b_stage_bytes, &bar_psi[ps]);
            }
        };
        // psi images are fetched two tiles ahead (three stages): tile t + 2 as soon as the MMAs of tile
        // t - 1, which read the same stage, have completed
        for (int t = 0; t < min(tiles, 2); t++) fetch_psi(t);
        for (int t = 0; t < min(tiles, PH_IN_STAGES); t++) fetch_inputs(t);

        // D fp32, A / B fp16, K-major, M = 128, N = 64
        constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(PH_COLS >> 3) << 17) | ((128u >> 4) << 24);
        constexpr uint32_t lbo_b = PH_COLS * 16, sbo = 128;
        constexpr uint64_t kstep_b = (uint64_t)(2 * lbo_b) >> 4;  // 16 K values = 2 chunks
        const uint64_t part_step = (uint64_t)b_part_bytes >> 4;
        const uint64_t stage_step = (uint64_t)b_stage_bytes >> 4;
        const uint64_t d_b0 = smem_desc(smem_u32(b_stage(0)), lbo_b, sbo);
        // phi of all rows is in tensor memory (the row threads arrive at this barrier after their stores)
        asm volatile("bar.sync 1, 288;" ::: "memory");
        tc_fence_after();
        for (int t = 0; t < tiles; t++) {
            const int st = t & 1, ps = t % PH_PSI_STAGES;
            bool ok = true;
            if (t >= 2) {
                // C stage free = tile t - 2 consumed, which also frees its input stage
                ok = mbar_wait(&bar_cfree[st], (unsigned)(((t >> 1) - 1) & 1), a.wait_polls);
                if (__all_sync(0xffffffffu, ok) && t + 2 < tiles) fetch_inputs(t + 2);
            }
            if (ok) ok = mbar_wait(&bar_psi[ps], (unsigned)((t / PH_PSI_STAGES) & 1), a.wait_polls);
            if (!__all_sync(0xffffffffu, ok)) {
                failed = true;
                break;
            }
            psi_seen = t + 1;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t d_tmem = tmem_base + (uint32_t)(PH_C_COL + st * PH_COLS);
                const uint64_t b_hi = d_b0 + ps * stage_step, b_lo = b_hi + part_step;
                // straight-line code per k-step count (a partially unrolled run-time loop of MMAs gave
                // wrong tiles in the gradient kernel; see there); the small cross terms first
                auto issue = [&](auto ks_tag) {
                    constexpr int KS = decltype(ks_tag)::value;
#pragma unroll
                    for (int ks = 0; ks < KS; ks++) {
                        const uint32_t a_hi = tmem_base + (uint32_t)(16 * ks), a_lo = a_hi + 8;
                        mma_f16_ts(d_tmem, a_hi, b_lo + ks * kstep_b, idesc, ks > 0 ? 1u : 0u);
                        mma_f16_ts(d_tmem, a_lo, b_hi + ks * kstep_b, idesc, 1u);
                    }
#pragma unroll
                    for (int ks = 0; ks < KS; ks++)
                        mma_f16_ts(d_tmem, tmem_base + (uint32_t)(16 * ks), b_hi + ks * kstep_b, idesc, 1u);
                };
                switch (ksteps) {  // 1 .. SUM_TC_MAX_COMPONENTS / 8
                    case 1: issue(std::integral_constant<int, 1>{}); break;
                    case 2: issue(std::integral_constant<int, 2>{}); break;
                    case 3: issue(std::integral_constant<int, 3>{}); break;
                    case 4: issue(std::integral_constant<int, 4>{}); break;
                    case 5: issue(std::integral_constant<int, 5>{}); break;
                    case 6: issue(std::integral_constant<int, 6>{}); break;
                    case 7: issue(std::integral_constant<int, 7>{}); break;
                    default: issue(std::integral_constant<int, 8>{}); break;
                }
                mma_commit(&bar_cfull[st]);
                mma_commit(&bar_pfree[ps]);
            }
            __syncwarp();
            if (t + 2 < tiles) {
                // the stage of tile t + 2 is that of tile t - 1, whose MMAs were issued an iteration ago
                if (t >= 1 && !__all_sync(0xffffffffu, mbar_wait(&bar_pfree[(t - 1) % PH_PSI_STAGES],
                                                                  (unsigned)(((t - 1) / PH_PSI_STAGES) & 1), a.wait_polls))) {
                    failed = true;
                    break;
                }
                fetch_psi(t + 2);
            }
        }
        if (failed) {
            // give-up path: the bulk copies that were issued and not yet seen complete are awaited (with
            // the full poll limit: they do arrive), so that nothing writes this CTA's shared memory later
            for (int t = psi_seen; t < psi_fetched; t++)
                mbar_wait(&bar_psi[t % PH_PSI_STAGES], (unsigned)((t / PH_PSI_STAGES) & 1), TC_WAIT_POLLS);
            if (lane == 0) atomicExch(&fail_flag, 1);
        }
        cp_async_wait<0>();  // no copy may be in flight when the CTA exits
        __syncwarp();
    } else {
        // ------------------------------------------------------------------------ row threads
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        const float x1v = row < a.m ? a.x1.data[row * a.x1.s0] : 0.0f;
        const uint32_t tmem_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);

        // phi of this row: image -> tensor memory, the two groups sharing the k-steps
        for (int ks = g; ks < ksteps; ks += 2) {
            uint32_t w[16];
            if (row < a.m) {
                const uint4 *src = reinterpret_cast<const uint4 *>(a.phi_img + (row * ksteps + ks) * 16);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint4 v = __ldg(src + q);
                    w[4 * q] = v.x, w[4 * q + 1] = v.y, w[4 * q + 2] = v.z, w[4 * q + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int q = 0; q < 16; q++) w[q] = 0u;
            }
            tmem_st16(tmem_lane + (uint32_t)(16 * ks), w);
        }
        tmem_st_wait();
        tc_fence_before();
        // both groups' parts of phi are in place before the first MMA: the control warp waits for
        // this barrier too (288 threads)
        asm volatile("bar.sync 1, 288;" ::: "memory");

        const f32x2 x1v2 = splat2(x1v), c02 = splat2(c0);
        // warp-level form: x1 of this thread's four rows 32 (warp % 4) + 16 mt + lane / 4 + 8 hh, as pairs
        f32x2 xi2[2][2];
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int64_t ri = r * KM_BLOCK_SIZE + (warp & 3) * 32 + 16 * mt + (lane >> 2) + 8 * hh;
                xi2[mt][hh] = splat2((MS && ri < a.m) ? a.x1.data[ri * a.x1.s0] : 0.0f);
            }
        for (int t = g; t < tiles && !failed; t += 2) {
            const int st = t & 1;
            if (!mbar_wait_warp(&bar_in[t % PH_IN_STAGES], (unsigned)((t / PH_IN_STAGES) & 1), a.wait_polls) ||
                !mbar_wait_warp(&bar_cfull[st], (unsigned)((t >> 1) & 1), a.wait_polls)) {
                failed = true;
                break;
            }
            tc_fence_after();
            const int j0 = (tile_lo + t) * PH_COLS;
            const float *xs = in_x2(t % PH_IN_STAGES);
            const float *rs = in_rhs(t % PH_IN_STAGES);
            auto consume = [&](auto masked_tag) {
                constexpr bool MASKED = decltype(masked_tag)::value;
                // the tensor-memory load of the next 16 columns is in flight while these are processed
                uint32_t cbuf[2][16];
                tmem_ld16_nowait(tmem_lane + (uint32_t)(PH_C_COL + st * PH_COLS), cbuf[0]);
                tmem_ld_wait16(cbuf[0]);
#pragma unroll
                for (int p = 0; p < PH_COLS / 16; p++) {
                    if (p + 1 < PH_COLS / 16)
                        tmem_ld16_nowait(tmem_lane + (uint32_t)(PH_C_COL + st * PH_COLS + (p + 1) * 16), cbuf[(p + 1) & 1]);
                    const uint32_t(&cv)[16] = cbuf[p & 1];
#pragma unroll
                    for (int h = 0; h < 4; h++) {
                        // four band columns = two packed pairs
                        const ulonglong2 xq = *reinterpret_cast<const ulonglong2 *>(xs + p * 16 + h * 4);
#pragma unroll
                        for (int q = 0; q < 2; q++) {
                            const int jj = p * 16 + h * 4 + 2 * q;  // even
                            const f32x2 tau2 = sub2(x1v2, q ? xq.y : xq.x);
                            const f32x2 e2 = ex2_approx2(mul2(mul2(tau2, tau2), c02));
                            uint32_t ca = cv[h * 4 + 2 * q], cb = cv[h * 4 + 2 * q + 1];
                            if (MASKED) {
                                if (j0 + jj < band_lo || j0 + jj >= band_hi) ca = 0u;
                                if (j0 + jj + 1 < band_lo || j0 + jj + 1 >= band_hi) cb = 0u;
                            }
                            const f32x2 v2 = mul2((f32x2)ca | ((f32x2)cb << 32), e2);
                            // rhs pairs of the two band columns (a broadcast read): one packed FMA per output column
                            const float *rp = rs + (jj >> 1) * (2 * KB);
#pragma unroll
                            for (int c2 = 0; c2 < KB / 2; c2++) {
                                const ulonglong2 rv = *reinterpret_cast<const ulonglong2 *>(rp + c2 * 4);
                                acc2[c2 * 2 + 0] = fma2(v2, rv.x, acc2[c2 * 2 + 0]);
                                acc2[c2 * 2 + 1] = fma2(v2, rv.y, acc2[c2 * 2 + 1]);
                            }
                        }
                    }
                    if (p + 1 < PH_COLS / 16) tmem_ld_wait16(cbuf[(p + 1) & 1]);
                }
            };
            auto consume_ms = [&](auto masked_tag) {
                constexpr bool MASKED = decltype(masked_tag)::value;
                const int gq = lane >> 2, tq = lane & 3;
                constexpr f32x2 HI2 = 0xffffe000ffffe000ull;  // the tf32 part of both values of a pair
                const uint32_t c_tile = tmem_lane + (uint32_t)(PH_C_COL + st * PH_COLS);
                // the loads of the next 8 columns are in flight while these are processed
                uint32_t cv[2][2][4];  // [buffer][16-row tile][fragment]
                tmem_ld_m16n8_nowait(c_tile, cv[0][0]);
                tmem_ld_m16n8_nowait(c_tile + (16u << 16), cv[0][1]);
                tmem_ld_wait4x2(cv[0][0], cv[0][1]);
#pragma unroll
                for (int cb = 0; cb < PH_COLS / 8; cb++) {
                    if (cb + 1 < PH_COLS / 8) {
                        tmem_ld_m16n8_nowait(c_tile + (uint32_t)((cb + 1) * 8), cv[(cb + 1) & 1][0]);
                        tmem_ld_m16n8_nowait(c_tile + (16u << 16) + (uint32_t)((cb + 1) * 8), cv[(cb + 1) & 1][1]);
                    }
                    const int jj = cb * 8 + 2 * tq;  // this thread's band columns jj, jj + 1 of the tile
                    const f32x2 xj2 = *reinterpret_cast<const f32x2 *>(xs + jj);
                    // B fragment: rhs[jj][gq], rhs[jj + 1][gq], split into tf32 hi and lo
                    const f32x2 b2 = *reinterpret_cast<const f32x2 *>(rs + ((((jj >> 1) * RS) + gq) << 1));
                    const f32x2 bh2 = b2 & HI2, bl2 = sub2(b2, bh2);
                    const uint32_t bh0 = (uint32_t)bh2, bh1 = (uint32_t)(bh2 >> 32), bl0 = (uint32_t)bl2, bl1 = (uint32_t)(bl2 >> 32);
#pragma unroll
                    for (int mt = 0; mt < 2; mt++) {
                        const uint32_t(&c4)[4] = cv[cb & 1][mt];
                        f32x2 wh[2], wl[2];
#pragma unroll
                        for (int hh = 0; hh < 2; hh++) {
                            const f32x2 tau2 = sub2(xi2[mt][hh], xj2);
                            const f32x2 e2 = ex2_approx2(mul2(mul2(tau2, tau2), c02));
                            uint32_t ca = c4[2 * hh], cbv = c4[2 * hh + 1];
                            if (MASKED) {
                                if (j0 + jj < band_lo || j0 + jj >= band_hi) ca = 0u;
                                if (j0 + jj + 1 < band_lo || j0 + jj + 1 >= band_hi) cbv = 0u;
                            }
                            const f32x2 w2 = mul2((f32x2)ca | ((f32x2)cbv << 32), e2);
                            wh[hh] = w2 & HI2;
                            wl[hh] = sub2(w2, wh[hh]);
                        }
                        // A fragment: (row, k) = (hh, band column parity): a0 = (0, 0), a1 = (1, 0), a2 = (0, 1), a3 = (1, 1)
                        mma_sync_tf32(dacc[mt], (uint32_t)wl[0], (uint32_t)wl[1], (uint32_t)(wl[0] >> 32), (uint32_t)(wl[1] >> 32), bh0, bh1);
                        mma_sync_tf32(dacc[mt], (uint32_t)wh[0], (uint32_t)wh[1], (uint32_t)(wh[0] >> 32), (uint32_t)(wh[1] >> 32), bl0, bl1);
                        mma_sync_tf32(dacc[mt], (uint32_t)wh[0], (uint32_t)wh[1], (uint32_t)(wh[0] >> 32), (uint32_t)(wh[1] >> 32), bh0, bh1);
                    }
                    if (cb + 1 < PH_COLS / 8) tmem_ld_wait4x2(cv[(cb + 1) & 1][0], cv[(cb + 1) & 1][1]);
                }
            };
            const bool edge = j0 < band_lo || j0 + PH_COLS > band_hi;
            if constexpr (MS) {
                if (edge)
                    consume_ms(std::true_type{});
                else
                    consume_ms(std::false_type{});
            } else {
                if (edge)
                    consume(std::true_type{});
                else
                    consume(std::false_type{});
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_cfree[st]);
        }
        if (failed) atomicExch(&fail_flag, 1);
    }

    tc_fence_before();
    __syncthreads();
    float acc[KB];
#pragma unroll
    for (int c = 0; c < KB; c++) {
        float even, odd;
        unpack2(acc2[c], even, odd);
        acc[c] = even + odd;
    }
    if constexpr (MS) {
        // both groups' accumulator fragments go through shared memory (the pipelines are done) into
        // row-per-thread order; group 0 adds the two
        float *xch = reinterpret_cast<float *>(smem_raw);
        if (!is_ctl_warp) {
#pragma unroll
            for (int mt = 0; mt < 2; mt++)
#pragma unroll
                for (int hh = 0; hh < 2; hh++)
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int row_in_block = (warp & 3) * 32 + 16 * mt + (lane >> 2) + 8 * hh, c = 2 * (lane & 3) + e;
                        xch[(g * KB + c) * 128 + row_in_block] = dacc[mt][2 * hh + e];
                    }
        }
        __syncthreads();
        if (!is_ctl_warp && g == 0) {
#pragma unroll
            for (int c = 0; c < KB; c++) acc[c] = xch[c * 128 + row_local] + xch[(KB + c) * 128 + row_local];
        }
    } else {
        // the second group hands its partial sums over through shared memory (the pipelines are done)
        float *xch = reinterpret_cast<float *>(smem_raw);
        if (!is_ctl_warp && g == 1) {
#pragma unroll
            for (int c = 0; c < KB; c++) xch[c * 128 + row_local] = acc[c];
        }
        __syncthreads();
        if (!is_ctl_warp && g == 0) {
#pragma unroll
            for (int c = 0; c < KB; c++) acc[c] += xch[c * 128 + row_local];
        }
    }
    if (!is_ctl_warp && g == 0) {
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        if (row < a.m) {
            const bool bad = fail_flag != 0;
            float *orow = a.out.data + (row - a.rb_begin * KM_BLOCK_SIZE) * a.out.s0;
#pragma unroll
            for (int c = 0; c < KB; c++)
                if (c < a.k) {
                    // later chunks of a sum over more than 64 components add to the first chunk's result
                    const float prev = a.comp_begin > 0 ? orow[c * a.out.s1] : 0.0f;
                    orow[c * a.out.s1] = bad ? __int_as_float(0x7fc00000) : acc[c] + prev;
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
        tmem_free(tmem_base, PH_TMEM_COLS);
    }
}

template <int KB, bool MS>
static int launch_sum_ph_kb(const SumTcArgs &a, cudaStream_t stream) {
    const int Bp = ((int)a.comp_count + 7) & ~7;
    const size_t b_stage = (size_t)Bp * 512;
    size_t smem = PH_PSI_STAGES * b_stage + (size_t)PH_IN_STAGES * (PH_COLS + PH_COLS * (MS ? 12 : KB)) * sizeof(float);
    // two CTAs of 256 tensor-memory columns fill an SM: keep a third from being scheduled
    smem = std::max<size_t>(smem, 80 * 1024);
    auto kernel = matmul_sum_ph_kernel<KB, MS>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(matmul_sum_ph)");
    kernel<<<(unsigned)a.row_blocks, 288, smem, stream>>>(a);
    KM_CHECK_LAUNCH("km_matmul_rows_phases_f32 (tensor-core batch sum, precomputed phases) launch");
    return KM_OK;
}

// Contraction with the rhs tile (k <= 8): on the FMA pipe, or on the warp-level tensor path when the
// environment variable KM_SUM_TC_WARP_MMA is 1 (read at every launch).
static bool sum_ph_warp_mma() {
    const char *e = getenv("KM_SUM_TC_WARP_MMA");
    return e != nullptr && e[0] == '1';
}

int launch_matmul_sum_ph(const SumTcArgs &a, const void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (a.row_blocks > 0x7fffffffLL) {
        set_error("km_matmul_rows_phases_f32: too many row blocks (%lld)", (long long)a.row_blocks);
        return KM_ERR_UNSUPPORTED;
    }
    const PhasesLayout L = phases_layout(a.batch.count, a.m, a.n);
    if (workspace == nullptr || workspace_bytes < (size_t)L.bytes || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0) {
        set_error("km_matmul_rows_phases_f32: the workspace written by km_sum_phases_prepare_f32 (%lld bytes) is needed",
                  (long long)L.bytes);
        return KM_ERR_WORKSPACE;
    }
    const unsigned char *ws = static_cast<const unsigned char *>(workspace);
    // more than 64 components: chunks of 64, each launch adding to the result of the previous ones
    // (launches on one stream run in order)
    SumTcArgs chunk = a;
    chunk.wait_polls = current_wait_polls();
    for (int64_t c = 0; c < L.chunks; c++) {
        chunk.comp_begin = c * SUM_TC_MAX_COMPONENTS;
        chunk.comp_count = chunk_comps(a.batch.count, c);
        chunk.psi_img = ws + L.psi_off[c];
        chunk.phi_img = reinterpret_cast<const uint32_t *>(ws + L.phi_off[c]);
        const int rc = a.k <= 8 ? (sum_ph_warp_mma() ? launch_sum_ph_kb<8, true>(chunk, stream) : launch_sum_ph_kb<8, false>(chunk, stream))
                                : launch_sum_ph_kb<16, false>(chunk, stream);
        if (rc != KM_OK) return rc;
    }
    return KM_OK;
}

}  // namespace km

// Batch sum of spectral components with BOTH contractions on the tensor cores:
//
//   out[i, :] = sum_{j in band} ( sum_b s_b exp(-tau^2 / 2 l^2) cos(w_b tau) ) rhs[j, :],   tau = x_i - x_j
//
// for components that share inputs, band, right-hand side and lengthscale (the reference's
// SumKernel over a batch of spectral kernels, kernel_matmul/gpytorch/sum.py:16-24).  As in
// km_matmul_sum_tc.cu the sum over the components is a dot product of per-point phase vectors,
//   C[i, j] = sum_b (s_b / S) cos(w_b (a_i - a_j)) = < phi(a_i), psi(a_j) >,   S = sum_b |s_b|,
// computed by tcgen05.mma (GEMM #1, K = 2B).  That kernel then multiplies C by the envelope and
// contracts with the rhs tile on the FMA pipe, for which every entry needs its rhs row from shared
// memory: two 16-byte broadcast reads per entry kept the shared-memory data pipe 78 % busy and
// bounded the kernel.  Here the row threads write W = C * exp(-tau^2 / 2 l^2) (in [-1, 1]) back
// into the SAME tensor-memory columns as an fp16 hi / lo A operand, and the tensor core does the
// second contraction too (GEMM #2):  D[128 x 16] = W[128 x 48] . rhs_tile[48 x 16], three
// kind::f16 MMAs per 16 band columns (hi*lo + lo*hi + hi*hi).  The rhs tile is converted to
// fp16 hi / lo with one power-of-two scale per column and tile by a converter warp straight from
// global memory; the threads read no rhs value at all.
//
// Tiles are 48 band columns wide so that everything fits 256 tensor-memory columns (two CTAs per
// SM):  phi 128 | C / W stage 0, 1: 2 x 48 | D stage 0, 1: 2 x 16.
//
// Warps of a CTA (320 threads): two row groups of 128 threads (thread = row = tensor-memory lane)
// that alternate tiles -- group g owns psi / C / W / D stage g and the tiles g, g + 2, ... --, a
// control warp (x2 fetches, all MMA issues) and a converter warp (rhs tiles).  Per tile, group:
// psi (written two of its tiles ahead, four psi stages in shared memory, so that GEMM #1 overlaps
// the group's work on the tile before) -> [GEMM #1] -> collect D of the tile before last -> W in
// place -> [GEMM #2].  All hand-offs
// are mbarriers with bounded waits; a CTA whose wait gives up writes NaN into its output rows.
#include <cuda_fp16.h>

#include <cstdlib>
#include <type_traits>

#include "km_tcgen05.cuh"

namespace km {

constexpr int T2_COLS = 48;        // band columns per tile = N of GEMM #1 = K of GEMM #2
constexpr int T2_N2 = 16;          // N of GEMM #2: rhs columns padded to 16
constexpr int T2_X_STAGES = 8;     // x2 tiles in shared memory
constexpr int T2_PSI_STAGES = 4;   // psi tiles in shared memory: a group writes psi two of its tiles ahead
constexpr int T2_TMEM_COLS = 256;
constexpr int T2_CW_COL = 128;     // C / W stage g at 128 + 48 g
constexpr int T2_D_COL = 224;      // D stage g at 224 + 16 g
constexpr int T2_THREADS = 320;
constexpr int T2_B2_PART_BYTES = (T2_COLS / 8) * T2_N2 * 16;  // one part (hi or lo) of an rhs image

__global__ void __launch_bounds__(T2_THREADS, 2) matmul_sum_tc2_kernel(const SumTcArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_in[T2_X_STAGES];  // x2 values of a tile landed
    __shared__ __align__(8) uint64_t bar_bready[T2_PSI_STAGES];  // psi tile written
    __shared__ __align__(8) uint64_t bar_cfull[2];         // C tile complete (GEMM #1 committed)
    __shared__ __align__(8) uint64_t bar_wready[2];        // W written over C
    __shared__ __align__(8) uint64_t bar_b2ready[2];       // rhs image written
    __shared__ __align__(8) uint64_t bar_dfull[2];         // D tile complete (GEMM #2 committed)
    __shared__ __align__(8) uint64_t bar_dfree[2];         // D tile collected
    __shared__ __align__(8) uint64_t bar_drain;            // give-up path: every issued MMA has completed
    __shared__ uint32_t tmem_base_slot;
    __shared__ int fail_flag;
    __shared__ __align__(16) float w_tab[SUM_TC_MAX_COMPONENTS];
    __shared__ __align__(16) float s_tab[SUM_TC_MAX_COMPONENTS];
    __shared__ __align__(16) float inv_scale[4][T2_N2];  // per tile (t & 3) and rhs column: 1 / scale
    __shared__ float s_total;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const bool is_ctl_warp = warp == 8;
    const bool is_cvt_warp = warp == 9;
    const bool is_row = warp < 8;
    const int g = tid >> 7;            // row group (row threads)
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
    for (int b = tid; b < SUM_TC_MAX_COMPONENTS; b += blockDim.x) {
        float w = 0.0f, s = 0.0f;
        if (b < B) {
            const float *th = batch_ptr(a.params, decompose(a.batch, a.comp_begin + b));
            w = 2.0f * KM_PI_F * th[a.params.s0];
            s = th[2 * a.params.s0];
        }
        w_tab[b] = w;
        s_tab[b] = s;
    }
    if (tid == 0) fail_flag = 0;
    if (!__syncthreads_and(same)) return;
    if (tid == 0) {
        float t = 0.0f;
        for (int b = 0; b < SUM_TC_MAX_COMPONENTS; b++) t += fabsf(s_tab[b]);  // fixed order
        s_total = t;
    }
    const float c0 = -(0.5f / (ell0 * ell0)) * KM_LOG2E_F;

    // shared memory: four psi stages [part: hi, lo][chunk = K / 8][j][8 halfs], two rhs images
    // [part][chunk = j / 8][c][8 halfs], then the x2 stages
    const int b_part_bytes = (2 * Bp / 8) * T2_COLS * 16;
    const int b_stage_bytes = 2 * b_part_bytes;
    unsigned char *b2_base = smem_raw + T2_PSI_STAGES * b_stage_bytes;
    float *x_base = reinterpret_cast<float *>(b2_base + 2 * 2 * T2_B2_PART_BYTES);
    auto b_stage = [&](int st) { return smem_raw + st * b_stage_bytes; };
    auto b2_stage = [&](int st) { return b2_base + st * 2 * T2_B2_PART_BYTES; };
    auto in_x2 = [&](int st) { return x_base + st * T2_COLS; };

    const int64_t r = a.rb_begin + blockIdx.x;
    const int n = (int)a.n;
    const int band_lo = clamp_int(a.start.data[r * a.start.s0], 0, n);
    const int band_hi = max(band_lo, min(a.end.data[r * a.end.s0], n));
    const int tile_lo = band_lo / T2_COLS;
    const int tiles = band_hi > band_lo ? (band_hi + T2_COLS - 1) / T2_COLS - tile_lo : 0;
    const float *x2 = a.x2.data;
    // origin of the phases: the middle row of the block
    const float x0 = a.x1.data[min(r * KM_BLOCK_SIZE + KM_BLOCK_SIZE / 2, a.m - 1) * a.x1.s0];

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < T2_X_STAGES; s++) mbar_init(&bar_in[s], 32);  // one cp.async arrival per lane
#pragma unroll
        for (int s = 0; s < T2_PSI_STAGES; s++) mbar_init(&bar_bready[s], 4);
#pragma unroll
        for (int s = 0; s < 2; s++) {
            mbar_init(&bar_cfull[s], 1);
            mbar_init(&bar_wready[s], 4);
            mbar_init(&bar_b2ready[s], 1);
            mbar_init(&bar_dfull[s], 1);
            mbar_init(&bar_dfree[s], 4);
        }
        mbar_init(&bar_drain, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (is_ctl_warp) tmem_alloc(&tmem_base_slot, T2_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const float S = s_total;
    const float inv_S = S > 0.0f ? 1.0f / S : 0.0f;
    bool failed = false;
    const unsigned polls = a.wait_polls;

    float acc[T2_N2];
#pragma unroll
    for (int c = 0; c < T2_N2; c++) acc[c] = 0.0f;

    if (is_ctl_warp) {
        // --------------------------------------------------- x2 fetches (all lanes) + MMA issue (lane 0)
        auto fetch_x = [&](int t) {
            const int st = t % T2_X_STAGES;
            const int64_t j0 = (int64_t)(tile_lo + t) * T2_COLS;
            float *xs = in_x2(st);
            for (int jj = lane; jj < T2_COLS; jj += 32) {
                const bool valid = j0 + jj < n;
                cp_async4_zfill(xs + jj, x2 + (valid ? j0 + jj : 0) * a.x2.s0, valid);
            }
            cp_async_mbar_arrive(&bar_in[st]);
        };
        for (int t = 0; t < min(tiles, T2_X_STAGES); t++) fetch_x(t);

        // D fp32, A / B fp16, K-major, M = 128; N = 48 (GEMM #1) and 16 (GEMM #2)
        constexpr uint32_t idesc1 = (1u << 4) | ((uint32_t)(T2_COLS >> 3) << 17) | ((128u >> 4) << 24);
        constexpr uint32_t idesc2 = (1u << 4) | ((uint32_t)(T2_N2 >> 3) << 17) | ((128u >> 4) << 24);
        constexpr uint32_t lbo1 = T2_COLS * 16, lbo2 = T2_N2 * 16, sbo = 128;
        constexpr uint64_t kstep1 = (uint64_t)(2 * lbo1) >> 4, kstep2 = (uint64_t)(2 * lbo2) >> 4;  // 16 K values = 2 chunks
        const uint64_t part1 = (uint64_t)b_part_bytes >> 4, stage1 = (uint64_t)b_stage_bytes >> 4;
        constexpr uint64_t part2 = (uint64_t)T2_B2_PART_BYTES >> 4, stage2 = (uint64_t)(2 * T2_B2_PART_BYTES) >> 4;
        const uint64_t d_b1 = smem_desc(smem_u32(b_stage(0)), lbo1, sbo);
        const uint64_t d_b2 = smem_desc(smem_u32(b2_stage(0)), lbo2, sbo);
        for (int t = 0; t <= tiles && tiles > 0; t++) {
            bool ok = true;
            if (t < tiles) {
                // GEMM #1 of tile t: C = phi . psi^T into stage t & 1 (the MMAs that read W of tile t - 2
                // from the same columns were issued earlier by this thread and execute first)
                const int st = t & 1, ps = t % T2_PSI_STAGES;
                ok = mbar_wait(&bar_bready[ps], (unsigned)((t / T2_PSI_STAGES) & 1), polls);
                if (!__all_sync(0xffffffffu, ok)) {
                    failed = true;
                    break;
                }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t d_tmem = tmem_base + (uint32_t)(T2_CW_COL + st * T2_COLS);
                    const uint64_t b_hi = d_b1 + ps * stage1, b_lo = b_hi + part1;
                    auto issue = [&](auto ks_tag) {
                        constexpr int KS = decltype(ks_tag)::value;
#pragma unroll
                        for (int ks = 0; ks < KS; ks++) {
                            const uint32_t a_hi = tmem_base + (uint32_t)(16 * ks), a_lo = a_hi + 8;
                            mma_f16_ts(d_tmem, a_hi, b_lo + ks * kstep1, idesc1, ks > 0 ? 1u : 0u);
                            mma_f16_ts(d_tmem, a_lo, b_hi + ks * kstep1, idesc1, 1u);
                        }
#pragma unroll
                        for (int ks = 0; ks < KS; ks++)
                            mma_f16_ts(d_tmem, tmem_base + (uint32_t)(16 * ks), b_hi + ks * kstep1, idesc1, 1u);
                    };
                    switch (ksteps) {  // 1 .. SUM_TC_MAX_COMPONENTS / 8 (straight-line issue code per count)
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
                }
                __syncwarp();
            }
            if (t >= 1) {
                // GEMM #2 of tile u = t - 1: D = W . rhs_tile into D stage u & 1
                const int u = t - 1, st = u & 1;
                ok = mbar_wait(&bar_wready[st], (unsigned)((u >> 1) & 1), polls);
                if (ok) ok = mbar_wait(&bar_b2ready[st], (unsigned)((u >> 1) & 1), polls);
                if (ok && u >= 2) ok = mbar_wait(&bar_dfree[st], (unsigned)(((u >> 1) - 1) & 1), polls);
                if (!__all_sync(0xffffffffu, ok)) {
                    failed = true;
                    break;
                }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t d_tmem = tmem_base + (uint32_t)(T2_D_COL + st * T2_N2);
                    const uint32_t w_tmem = tmem_base + (uint32_t)(T2_CW_COL + st * T2_COLS);
                    const uint64_t b_hi = d_b2 + st * stage2, b_lo = b_hi + part2;
#pragma unroll
                    for (int ks = 0; ks < T2_COLS / 16; ks++) {
                        const uint32_t a_hi = w_tmem + (uint32_t)(16 * ks), a_lo = a_hi + 8;
                        mma_f16_ts(d_tmem, a_hi, b_lo + ks * kstep2, idesc2, ks > 0 ? 1u : 0u);
                        mma_f16_ts(d_tmem, a_lo, b_hi + ks * kstep2, idesc2, 1u);
                    }
#pragma unroll
                    for (int ks = 0; ks < T2_COLS / 16; ks++)
                        mma_f16_ts(d_tmem, w_tmem + (uint32_t)(16 * ks), b_hi + ks * kstep2, idesc2, 1u);
                    mma_commit(&bar_dfull[st]);
                }
                __syncwarp();
                // the x2 stage of tile u has been read (psi and W of tile u are written): refill it
                if (u + T2_X_STAGES < tiles) fetch_x(u + T2_X_STAGES);
            }
        }
        if (failed && lane == 0) atomicExch(&fail_flag, 1);
        cp_async_wait<0>();  // no copy may be in flight when the CTA exits
        __syncwarp();
    } else if (is_cvt_warp) {
        // ------------------------------------------------ rhs tiles -> fp16 hi / lo images (B operand of GEMM #2)
        // lane: column c = lane % KP, rows lane / KP + i * (32 / KP); one power-of-two scale per column
        const int KP = a.k <= 8 ? 8 : 16, RS = 32 / KP;
        const int c = lane % KP, r0 = lane / KP;
        const float *rhs = a.rhs.data;
        for (int t = 0; t < tiles; t++) {
            const int st = t & 1;
            if (t >= 2 && !mbar_wait_warp(&bar_dfull[st], (unsigned)(((t >> 1) - 1) & 1), polls)) {  // image of tile t - 2 read
                failed = true;
                break;
            }
            const int64_t j0 = (int64_t)(tile_lo + t) * T2_COLS;
            float v[T2_COLS / 2];  // KP = 16: 24 rows per lane; KP = 8: 12
            const int cnt = T2_COLS / RS;
            unsigned mx = 0u;
#pragma unroll
            for (int i = 0; i < T2_COLS / 2; i++) {
                v[i] = 0.0f;
                if (i < cnt) {
                    const int64_t j = j0 + r0 + i * RS;
                    if (j < n && c < a.k) v[i] = __ldg(rhs + j * a.rhs.s0 + c * a.rhs.s1);
                    mx = max(mx, __float_as_uint(fabsf(v[i])));
                }
            }
            // lanes with the same column: l, l + KP, ...
            for (int o = KP; o < 32; o <<= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            // scale that brings the column maximum into [2^13, 2^14); 1 for an empty or non-finite column
            const int e = (int)(mx >> 23);
            const float sc = (e == 0 || e == 255) ? 1.0f : __uint_as_float((unsigned)min(max(267 - e, 1), 254) << 23);
            __half *hi = reinterpret_cast<__half *>(b2_stage(st));
            __half *lo = hi + T2_B2_PART_BYTES / 2;
#pragma unroll
            for (int i = 0; i < T2_COLS / 2; i++) {
                if (i < cnt) {
                    const int jj = r0 + i * RS;
                    const float y = v[i] * sc;
                    const __half h = __float2half_rn(y);
                    const int at = (jj >> 3) * (T2_N2 * 8) + c * 8 + (jj & 7);
                    hi[at] = h;
                    lo[at] = __float2half_rn(y - __half2float(h));
                }
            }
            if (KP == 8) {  // columns 8 .. 15 of the padded image are zero
#pragma unroll
                for (int i = 0; i < T2_COLS / 2; i++) {
                    if (i < cnt) {
                        const int jj = r0 + i * RS;
                        const int at = (jj >> 3) * (T2_N2 * 8) + (c + 8) * 8 + (jj & 7);
                        hi[at] = __float2half_rn(0.0f);
                        lo[at] = __float2half_rn(0.0f);
                    }
                }
            }
            if (r0 == 0) {
                inv_scale[t & 3][c] = S / sc;  // undoes the column scale and the normalisation of C
                if (KP == 8) inv_scale[t & 3][c + 8] = 0.0f;
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_b2ready[st]);
        }
        if (failed) atomicExch(&fail_flag, 1);
    } else {
        // ------------------------------------------------------------------------ row threads
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        const float x1v = row < a.m ? a.x1.data[row * a.x1.s0] : x0;
        const uint32_t tmem_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);

        // phi of this row -> tensor memory: per 8 components [8 hi pairs | 8 lo pairs]
        {
            const float ai = x1v - x0;
            for (int ks = g; ks < ksteps; ks += 2) {
                float v[16], lo[16];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const float ph = w_tab[ks * 8 + u] * ai, sc = s_tab[ks * 8 + u] * inv_S;
                    v[2 * u] = sc * cos_approx(ph);
                    v[2 * u + 1] = sc * sin_approx(ph);
                }
#pragma unroll
                for (int u = 0; u < 16; u++) lo[u] = v[u] - tf32_hi(v[u]);
                split_store16(tmem_lane + (uint32_t)(16 * ks), v, lo);
            }
            tmem_st_wait();
            tc_fence_before();
            // both groups' parts of phi are in place before either announces a psi tile
            asm volatile("bar.sync 1, 256;" ::: "memory");
        }

        // psi of a tile's 48 columns -> shared memory: 48 x (Bp / 4) items of 4 components = one 16-byte
        // chunk (8 K values) each in the hi and the lo image
        auto generate = [&](int t) {
            const int st = t % T2_PSI_STAGES;
            const float *xs = in_x2(t % T2_X_STAGES);
            unsigned char *hi = b_stage(st);
            unsigned char *lo = hi + b_part_bytes;
            const int items = T2_COLS * (Bp / 4);
            for (int id = row_local; id < items; id += 128) {
                const int jj = id % T2_COLS, kc = id / T2_COLS;
                const float aj = xs[jj] - x0;
                const float4 wq = *reinterpret_cast<const float4 *>(w_tab + kc * 4);
                const float wv[4] = {wq.x, wq.y, wq.z, wq.w};
                uint32_t h[4], l[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const float ph = wv[u] * aj;
                    const f32x2 v2 = pack2(cos_approx(ph), sin_approx(ph));
                    h[u] = cvt_rz_f16x2_pair(v2);
                    l[u] = cvt_rn_f16x2_pair(sub2(v2, v2 & 0xffffe000ffffe000ull));
                }
                *reinterpret_cast<uint4 *>(hi + kc * (T2_COLS * 16) + jj * 16) = make_uint4(h[0], h[1], h[2], h[3]);
                *reinterpret_cast<uint4 *>(lo + kc * (T2_COLS * 16) + jj * 16) = make_uint4(l[0], l[1], l[2], l[3]);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_bready[st]);
        };

        // D of tile u (this group's stage) -> registers, with the column scales undone
        auto collect = [&](int u) {
            const int st = u & 1;
            uint32_t dv[16];
            tmem_ld16_nowait(tmem_lane + (uint32_t)(T2_D_COL + st * T2_N2), dv);
            tmem_ld_wait16(dv);
            const float *is = inv_scale[u & 3];
#pragma unroll
            for (int c4 = 0; c4 < T2_N2 / 4; c4++) {
                const float4 s4 = *reinterpret_cast<const float4 *>(is + c4 * 4);
                acc[c4 * 4 + 0] = fmaf(__uint_as_float(dv[c4 * 4 + 0]), s4.x, acc[c4 * 4 + 0]);
                acc[c4 * 4 + 1] = fmaf(__uint_as_float(dv[c4 * 4 + 1]), s4.y, acc[c4 * 4 + 1]);
                acc[c4 * 4 + 2] = fmaf(__uint_as_float(dv[c4 * 4 + 2]), s4.z, acc[c4 * 4 + 2]);
                acc[c4 * 4 + 3] = fmaf(__uint_as_float(dv[c4 * 4 + 3]), s4.w, acc[c4 * 4 + 3]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_dfree[st]);
        };

        const f32x2 x1v2 = splat2(x1v), c02 = splat2(c0);
        int last = -1;  // last tile of this group whose GEMM #2 was requested
        // psi is written TWO of this group's tiles ahead (four psi stages), so that GEMM #1 of a tile
        // runs while the group still works on the tile before
        if (g < tiles) {
            if (!mbar_wait_warp(&bar_in[g % T2_X_STAGES], 0u, polls)) failed = true;
            if (!failed) generate(g);
        }
        for (int t = g; t < tiles && !failed; t += 2) {
            const int st = t & 1;  // == g
            if (t + 2 < tiles) {
                // (the psi stage of tile t + 2 was last read by GEMM #1 of tile t - 2, whose completion
                // this thread saw before it wrote W of that tile)
                if (!mbar_wait_warp(&bar_in[(t + 2) % T2_X_STAGES], (unsigned)(((t + 2) / T2_X_STAGES) & 1), polls)) {
                    failed = true;
                    break;
                }
                generate(t + 2);
            }
            if (!mbar_wait_warp(&bar_cfull[st], (unsigned)((t >> 1) & 1), polls)) {
                failed = true;
                break;
            }
            tc_fence_after();
            if (t >= 2) {
                // D of the tile before last of this stage is complete by now in all likelihood
                if (!mbar_wait_warp(&bar_dfull[st], (unsigned)(((t >> 1) - 1) & 1), polls)) {
                    failed = true;
                    break;
                }
                tc_fence_after();
                collect(t - 2);
            }
            // W = C * envelope, in place: 16 columns of C (fp32) -> 8 hi words + 8 lo words (fp16 pairs)
            const int j0 = (tile_lo + t) * T2_COLS;
            const float *xs = in_x2(t % T2_X_STAGES);
            const bool edge = j0 < band_lo || j0 + T2_COLS > band_hi;
            const uint32_t cw = tmem_lane + (uint32_t)(T2_CW_COL + st * T2_COLS);
#pragma unroll
            for (int p = 0; p < T2_COLS / 16; p++) {
                uint32_t cv[16];
                tmem_ld16_nowait(cw + (uint32_t)(p * 16), cv);
                tmem_ld_wait16(cv);
                uint32_t words[16];
#pragma unroll
                for (int h = 0; h < 4; h++) {
                    const ulonglong2 xq = *reinterpret_cast<const ulonglong2 *>(xs + p * 16 + h * 4);
#pragma unroll
                    for (int q = 0; q < 2; q++) {
                        const int jj = p * 16 + h * 4 + 2 * q;
                        const f32x2 tau2 = sub2(x1v2, q ? xq.y : xq.x);
                        const f32x2 e2 = ex2_approx2(mul2(mul2(tau2, tau2), c02));
                        uint32_t ca = cv[h * 4 + 2 * q], cb = cv[h * 4 + 2 * q + 1];
                        if (edge) {
                            if (j0 + jj < band_lo || j0 + jj >= band_hi) ca = 0u;
                            if (j0 + jj + 1 < band_lo || j0 + jj + 1 >= band_hi) cb = 0u;
                        }
                        const f32x2 w2 = mul2((f32x2)ca | ((f32x2)cb << 32), e2);
                        words[h * 2 + q] = cvt_rz_f16x2_pair(w2);
                        words[8 + h * 2 + q] = cvt_rn_f16x2_pair(sub2(w2, w2 & 0xffffe000ffffe000ull));
                    }
                }
                tmem_st16(cw + (uint32_t)(p * 16), words);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_wready[st]);
            last = t;
        }
        // the D tiles still in tensor memory: the last one of this stage (the one before it was
        // collected inside the loop, or there is none)
        if (!failed && last >= 0) {
            if (!mbar_wait_warp(&bar_dfull[g], (unsigned)((last >> 1) & 1), polls)) {
                failed = true;
            } else {
                tc_fence_after();
                collect(last);
            }
        }
        if (failed) atomicExch(&fail_flag, 1);
    }

    tc_fence_before();
    __syncthreads();
    // the second group hands its partial sums over through shared memory (the pipelines are done)
    {
        float *xch = reinterpret_cast<float *>(smem_raw);
        if (is_row && g == 1) {
#pragma unroll
            for (int c = 0; c < T2_N2; c++) xch[c * 128 + row_local] = acc[c];
        }
        __syncthreads();
        if (is_row && g == 0) {
#pragma unroll
            for (int c = 0; c < T2_N2; c++) acc[c] += xch[c * 128 + row_local];
        }
    }
    if (is_row && g == 0) {
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        if (row < a.m) {
            const bool bad = fail_flag != 0;
            float *orow = a.out.data + (row - a.rb_begin * KM_BLOCK_SIZE) * a.out.s0;
#pragma unroll
            for (int c = 0; c < T2_N2; c++)
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
        tmem_free(tmem_base, T2_TMEM_COLS);
    }
}

int launch_matmul_sum_tc2(const SumTcArgs &a, cudaStream_t stream) {
    if (a.row_blocks > 0x7fffffffLL) {
        set_error("km_matmul_rows_f32: too many row blocks (%lld)", (long long)a.row_blocks);
        return KM_ERR_UNSUPPORTED;
    }
    auto kernel = matmul_sum_tc2_kernel;
    SumTcArgs chunk = a;
    chunk.wait_polls = current_wait_polls();
    for (int64_t b0 = 0; b0 < a.batch.count; b0 += SUM_TC_MAX_COMPONENTS) {
        chunk.comp_begin = b0;
        chunk.comp_count = std::min<int64_t>(SUM_TC_MAX_COMPONENTS, a.batch.count - b0);
        const int Bp = ((int)chunk.comp_count + 7) & ~7;
        size_t smem = (size_t)T2_PSI_STAGES * 2 * (2 * Bp / 8) * T2_COLS * 16 + 2 * 2 * T2_B2_PART_BYTES +
                      T2_X_STAGES * T2_COLS * sizeof(float);
        // two CTAs of 256 tensor-memory columns fill an SM: keep a third from being scheduled
        smem = std::max<size_t>(smem, 80 * 1024);
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(matmul_sum_tc2)");
        kernel<<<(unsigned)a.row_blocks, T2_THREADS, smem, stream>>>(chunk);
        KM_CHECK_LAUNCH("km_matmul_rows_f32 (tensor-core batch sum, both contractions) launch");
    }
    return KM_OK;
}

}  // namespace km

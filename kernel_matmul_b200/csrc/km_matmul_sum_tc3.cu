// Batch sum of spectral components on the tensor cores, TWO row blocks per CTA:
//
//   out[i, :] = sum_{j in band} ( sum_b s_b exp(-tau^2 / 2 l^2) cos(w_b tau) ) rhs[j, :],   tau = x_i - x_j
//
// The arithmetic is that of km_matmul_sum_tc.cu (the sum over the components as a dot product of
// per-point phase vectors, C = < phi(a_i), psi(a_j) > on tcgen05.mma, then envelope and rhs
// contraction on the FMA pipe).  That kernel is bounded by the shared-memory data pipe: a thread
// owns one row, and every entry needs its 32 bytes of the rhs tile in registers.  Here a CTA
// takes the row blocks 2q and 2q + 1 of the operator and a thread owns row i of BOTH: the packed
// pair (rhs[j][c], rhs[j + 1][c]) it has loaded serves four entries instead of two, the tile of
// psi vectors (the B operand: 2B SFU operations per column) is generated once for 256 rows, and
// so are the x2 values.  Per entry: 16 bytes from shared memory, 1 + B / 128 SFU operations.
//
// Tensor memory (all 512 columns, one CTA per SM): phi of block A | phi of block B | per row
// group g its C tiles [A: 64 columns | B: 64 columns].  Warps: two groups of 128 row threads that
// alternate tiles (by the parity of the tile's index), one MMA-issuing warp per group, one fetch warp.
// A group writes psi of its NEXT tile (two psi stages per group) while the MMAs of the current
// one run, then reads C, multiplies by the envelope and contracts with the rhs tile for both of
// its rows.  All hand-offs are mbarriers with bounded waits; a CTA whose wait gives up writes NaN
// into its output rows.
#include <cstdlib>
#include <type_traits>

#include "km_tcgen05.cuh"

namespace km {

constexpr int S3_COLS = 64;        // band columns per tile = GEMM N
constexpr int S3_IN_STAGES = 8;    // x2 / rhs tiles in shared memory
constexpr int S3_PSI_STAGES = 4;   // psi tiles in shared memory: two per group
constexpr int S3_TMEM_COLS = 512;
constexpr int S3_PHI_B = 128;      // phi of block B
constexpr int S3_C_COL = 256;      // C of group g, block A at 256 + 128 g, block B 64 columns further
constexpr int S3_THREADS = 352;    // 8 row warps, 2 MMA warps, 1 fetch warp

template <int KB>
__global__ void __launch_bounds__(S3_THREADS, 1) matmul_sum_tc3_kernel(const SumTcArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_in[S3_IN_STAGES];      // x2 + rhs tile landed
    __shared__ __align__(8) uint64_t bar_infree[S3_IN_STAGES];  // x2 + rhs tile consumed
    __shared__ __align__(8) uint64_t bar_bready[S3_PSI_STAGES]; // psi tile written
    __shared__ __align__(8) uint64_t bar_cfull[2];              // C tiles of a group complete (tcgen05.commit)
    __shared__ __align__(8) uint64_t bar_cfree[2];              // C tiles of a group consumed
    __shared__ __align__(8) uint64_t bar_drain[2];              // give-up path: a warp's MMAs have completed
    __shared__ uint32_t tmem_base_slot;
    __shared__ int fail_flag;
    __shared__ __align__(16) float w_tab[SUM_TC_MAX_COMPONENTS];
    __shared__ __align__(16) float s_tab[SUM_TC_MAX_COMPONENTS];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const bool is_row = warp < 8;
    const bool is_mma_warp = warp == 8 || warp == 9;  // warp 8 + g issues the MMAs of group g
    const bool is_fetch_warp = warp == 10;
    const int g = is_row ? (tid >> 7) : (warp - 8);  // row group (row threads, MMA warps)
    const int row_local = tid & 127;                  // row of a block = tensor-memory lane
    const int B = (int)a.comp_count;  // components of this launch: [comp_begin, comp_begin + B)
    const int Bp = (B + 7) & ~7;      // components padded to whole MMA steps (K = 2 Bp)
    const int ksteps = Bp / 8;
    static_assert(SUM_TC_MAX_COMPONENTS == 64, "the MMA issue code covers 1 .. 8 k-steps");

    // every CTA checks that the components share one lengthscale; if not, the FMA-pipe kernel
    // launched next to this one does the work and this CTA leaves at once
    // (the lengthscales of ALL components are compared, so that every launch of a chunked sum and
    // the FMA-pipe kernel come to the same decision)
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
    const float c0 = -(0.5f / (ell0 * ell0)) * KM_LOG2E_F;

    // shared memory: four psi stages [part: hi, lo][chunk = K / 8][j][8 halfs], then the input stages
    const int b_part_bytes = (2 * Bp / 8) * S3_COLS * 16;
    const int b_stage_bytes = 2 * b_part_bytes;
    unsigned char *in_base = smem_raw + S3_PSI_STAGES * b_stage_bytes;
    constexpr int IN_STAGE_FLOATS = S3_COLS + S3_COLS * KB;  // x2 values, then rhs rows
    auto b_stage = [&](int st) { return smem_raw + st * b_stage_bytes; };
    auto in_x2 = [&](int st) { return reinterpret_cast<float *>(in_base) + st * IN_STAGE_FLOATS; };
    auto in_rhs = [&](int st) { return reinterpret_cast<float *>(in_base) + st * IN_STAGE_FLOATS + S3_COLS; };

    // The CTA's row blocks: the pair (2 q, 2 q + 1) of the whole operator, whatever window of row
    // blocks the launch covers -- a row's result (origin of its phases, order of its additions) then
    // does not depend on the window.  A block outside the window is absent: empty band, no MMAs, no
    // output.
    const int64_t rA = 2 * (a.rb_begin / 2 + (int64_t)blockIdx.x);
    const bool has_a = rA >= a.rb_begin, has_b = rA + 1 < a.rb_begin + a.row_blocks;
    const int n = (int)a.n;
    const int lo_a = has_a ? clamp_int(a.start.data[rA * a.start.s0], 0, n) : 0;
    const int hi_a = has_a ? max(lo_a, min(a.end.data[rA * a.end.s0], n)) : 0;
    const int lo_b = has_b ? clamp_int(a.start.data[(rA + 1) * a.start.s0], 0, n) : 0;
    const int hi_b = has_b ? max(lo_b, min(a.end.data[(rA + 1) * a.end.s0], n)) : 0;
    // columns any of the two blocks visits
    const int band_lo = hi_b > lo_b ? (hi_a > lo_a ? min(lo_a, lo_b) : lo_b) : lo_a;
    const int band_hi = hi_b > lo_b ? (hi_a > lo_a ? max(hi_a, hi_b) : hi_b) : hi_a;
    const int tile_lo = band_lo / S3_COLS;
    const int tiles = band_hi > band_lo ? (band_hi + S3_COLS - 1) / S3_COLS - tile_lo : 0;
    const float *x2 = a.x2.data;
    const float *rhs = a.rhs.data;
    // tiles go to the row groups by the parity of their index in the whole operator; group g's
    // first tile of this CTA and the number of its tiles
    const int first_t = (tile_lo + g) & 1;
    // origin of the phases: the first row of block B, the middle of the pair's rows
    const float x0 = a.x1.data[min((rA + 1) * KM_BLOCK_SIZE, a.m - 1) * a.x1.s0];

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < S3_IN_STAGES; s++) {
            mbar_init(&bar_in[s], 32);  // one cp.async arrival per lane
            mbar_init(&bar_infree[s], 4);
        }
#pragma unroll
        for (int s = 0; s < S3_PSI_STAGES; s++) mbar_init(&bar_bready[s], 4);
#pragma unroll
        for (int s = 0; s < 2; s++) {
            mbar_init(&bar_cfull[s], 1);
            mbar_init(&bar_cfree[s], 4);
            mbar_init(&bar_drain[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(&tmem_base_slot, S3_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    bool failed = false;

    // per output column: (sum over even band columns, sum over odd band columns), blocks A and B
    f32x2 acc_a[KB], acc_b[KB];
#pragma unroll
    for (int c = 0; c < KB; c++) acc_a[c] = acc_b[c] = 0ull;

    if (is_fetch_warp) {
        // ------------------------------------------------------------- input fetches (all lanes)
        for (int t = 0; t < tiles; t++) {
            const int st = t % S3_IN_STAGES;
            // the stage's previous tile (t - S3_IN_STAGES) has been consumed
            if (t >= S3_IN_STAGES &&
                !mbar_wait_warp(&bar_infree[st], (unsigned)((t / S3_IN_STAGES - 1) & 1), a.wait_polls)) {
                failed = true;
                break;
            }
            const int64_t j0 = (int64_t)(tile_lo + t) * S3_COLS;
            float *xs = in_x2(st);
            float *rs = in_rhs(st);
#pragma unroll
            for (int u = 0; u < S3_COLS / 32; u++) {
                const int jj = lane + 32 * u;
                const bool valid = j0 + jj < n;
                cp_async4_zfill(xs + jj, x2 + (valid ? j0 + jj : 0) * a.x2.s0, valid);
            }
            // rhs rows in pairs: rs[((jj / 2) * KB + c) * 2 + (jj & 1)] = rhs[j0 + jj][c]
            for (int q = lane; q < S3_COLS * KB; q += 32) {
                const int jj = q / KB, c = q % KB;
                const bool valid = j0 + jj < n && c < a.k;
                cp_async4_zfill(rs + (((jj >> 1) * KB + c) << 1) + (jj & 1),
                                rhs + (valid ? (j0 + jj) * a.rhs.s0 + c * a.rhs.s1 : 0), valid);
            }
            cp_async_mbar_arrive(&bar_in[st]);
        }
        if (failed && lane == 0) atomicExch(&fail_flag, 1);
        cp_async_wait<0>();  // no copy may be in flight when the CTA exits
        __syncwarp();
    } else if (is_mma_warp) {
        // ------------------------------------------------- MMA issue for group g's tiles (lane 0)
        // D fp32, A / B fp16, K-major, M = 128, N = 64
        constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(S3_COLS >> 3) << 17) | ((128u >> 4) << 24);
        constexpr uint32_t lbo_b = S3_COLS * 16, sbo = 128;
        constexpr uint64_t kstep_b = (uint64_t)(2 * lbo_b) >> 4;  // 16 K values = 2 chunks
        const uint64_t part_step = (uint64_t)b_part_bytes >> 4;
        const uint64_t stage_step = (uint64_t)b_stage_bytes >> 4;
        const uint64_t d_b0 = smem_desc(smem_u32(b_stage(0)), lbo_b, sbo);
        for (int t = first_t, u = 0; t < tiles; t += 2, u++) {  // u: count of the group's tiles
            const int ps = g + 2 * (u & 1);
            bool ok = true;
            // the group's C tiles are free = its previous tile has been consumed
            if (u >= 1) ok = mbar_wait(&bar_cfree[g], (unsigned)((u - 1) & 1), a.wait_polls);
            if (ok) ok = mbar_wait(&bar_bready[ps], (unsigned)((u >> 1) & 1), a.wait_polls);
            if (!__all_sync(0xffffffffu, ok)) {
                failed = true;
                break;
            }
            tc_fence_after();
            if (lane == 0) {
                const uint64_t b_hi = d_b0 + ps * stage_step, b_lo = b_hi + part_step;
                // straight-line code per k-step count (a partially unrolled run-time loop of MMAs gave
                // wrong tiles in the gradient kernel; see there); the small cross terms first
                auto issue = [&](auto ks_tag, uint32_t d_tmem, uint32_t phi) {
                    constexpr int KS = decltype(ks_tag)::value;
#pragma unroll
                    for (int ks = 0; ks < KS; ks++) {
                        const uint32_t a_hi = phi + (uint32_t)(16 * ks), a_lo = a_hi + 8;
                        mma_f16_ts(d_tmem, a_hi, b_lo + ks * kstep_b, idesc, ks > 0 ? 1u : 0u);
                        mma_f16_ts(d_tmem, a_lo, b_hi + ks * kstep_b, idesc, 1u);
                    }
#pragma unroll
                    for (int ks = 0; ks < KS; ks++)
                        mma_f16_ts(d_tmem, phi + (uint32_t)(16 * ks), b_hi + ks * kstep_b, idesc, 1u);
                };
                for (int blk = has_a ? 0 : 1; blk < (has_b ? 2 : 1); blk++) {
                    const uint32_t d_tmem = tmem_base + (uint32_t)(S3_C_COL + g * 2 * S3_COLS + blk * S3_COLS);
                    const uint32_t phi = tmem_base + (uint32_t)(blk * S3_PHI_B);
                    switch (ksteps) {  // 1 .. SUM_TC_MAX_COMPONENTS / 8
                        case 1: issue(std::integral_constant<int, 1>{}, d_tmem, phi); break;
                        case 2: issue(std::integral_constant<int, 2>{}, d_tmem, phi); break;
                        case 3: issue(std::integral_constant<int, 3>{}, d_tmem, phi); break;
                        case 4: issue(std::integral_constant<int, 4>{}, d_tmem, phi); break;
                        case 5: issue(std::integral_constant<int, 5>{}, d_tmem, phi); break;
                        case 6: issue(std::integral_constant<int, 6>{}, d_tmem, phi); break;
                        case 7: issue(std::integral_constant<int, 7>{}, d_tmem, phi); break;
                        default: issue(std::integral_constant<int, 8>{}, d_tmem, phi); break;
                    }
                }
                mma_commit(&bar_cfull[g]);
            }
            __syncwarp();
        }
        if (failed && lane == 0) atomicExch(&fail_flag, 1);
        __syncwarp();
    } else {
        // ------------------------------------------------------------------------ row threads
        const int64_t row_a = rA * KM_BLOCK_SIZE + row_local, row_b = row_a + KM_BLOCK_SIZE;
        const float xa = (has_a && row_a < a.m) ? a.x1.data[row_a * a.x1.s0] : x0;
        const float xb = (has_b && row_b < a.m) ? a.x1.data[row_b * a.x1.s0] : x0;
        const uint32_t tmem_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);

        // phi of both rows -> tensor memory: per 8 components [8 hi pairs | 8 lo pairs]; the two
        // groups share the k-steps
        for (int blk = 0; blk < 2; blk++) {
            const float ai = (blk ? xb : xa) - x0;
            for (int ks = g; ks < ksteps; ks += 2) {
                float v[16], lo[16];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const float ph = w_tab[ks * 8 + u] * ai, sc = s_tab[ks * 8 + u];
                    v[2 * u] = sc * cos_approx(ph);
                    v[2 * u + 1] = sc * sin_approx(ph);
                }
#pragma unroll
                for (int u = 0; u < 16; u++) lo[u] = v[u] - tf32_hi(v[u]);
                split_store16(tmem_lane + (uint32_t)(blk * S3_PHI_B + 16 * ks), v, lo);
            }
        }
        tmem_st_wait();
        tc_fence_before();
        // both groups' parts of phi are in place before either announces a psi tile
        asm volatile("bar.sync 1, 256;" ::: "memory");

        // psi of a tile's columns -> shared memory (thread: column row_local % 64, half of the components)
        auto generate = [&](int t, int u) {
            const int ps = g + 2 * (u & 1);
            const int jj = row_local & 63;
            const float aj = in_x2(t % S3_IN_STAGES)[jj] - x0;
            unsigned char *hi = b_stage(ps) + jj * 16;
            unsigned char *lo = hi + b_part_bytes;
            // 4 components = 8 K values = one 16-byte chunk
            for (int kc = (row_local >> 6) * (Bp / 8); kc < ((row_local >> 6) + 1) * (Bp / 8); kc++) {
                // (cos, sin) of one component as a packed pair; hi = the pair truncated to fp16
                // precision (cvt.rz), lo = pair - hi rounded (one packed subtraction)
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
                *reinterpret_cast<uint4 *>(hi + kc * (S3_COLS * 16)) = make_uint4(h[0], h[1], h[2], h[3]);
                *reinterpret_cast<uint4 *>(lo + kc * (S3_COLS * 16)) = make_uint4(l[0], l[1], l[2], l[3]);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_bready[ps]);
        };

        const f32x2 xa2 = splat2(xa), xb2 = splat2(xb), c02 = splat2(c0);
        const int t0 = first_t;
        if (t0 < tiles) {
            if (!mbar_wait_warp(&bar_in[t0 % S3_IN_STAGES], 0u, a.wait_polls)) failed = true;
            if (!failed) generate(t0, 0);
        }
        for (int t = t0, u = 0; t < tiles && !failed; t += 2, u++) {
            // psi of the group's next tile while the MMAs of this one run (its psi stage was read by
            // the MMAs of the group's tile before this one, whose completion this thread saw before
            // it consumed that tile)
            if (t + 2 < tiles) {
                if (!mbar_wait_warp(&bar_in[(t + 2) % S3_IN_STAGES], (unsigned)(((t + 2) / S3_IN_STAGES) & 1), a.wait_polls)) {
                    failed = true;
                    break;
                }
                generate(t + 2, u + 1);
            }
            if (!mbar_wait_warp(&bar_cfull[g], (unsigned)(u & 1), a.wait_polls)) {
                failed = true;
                break;
            }
            tc_fence_after();
            const int j0 = (tile_lo + t) * S3_COLS;
            const float *xs = in_x2(t % S3_IN_STAGES);
            const float *rs = in_rhs(t % S3_IN_STAGES);
            const uint32_t c_a = tmem_lane + (uint32_t)(S3_C_COL + g * 2 * S3_COLS), c_b = c_a + S3_COLS;
            auto consume = [&](auto masked_tag) {
                constexpr bool MASKED = decltype(masked_tag)::value;
                // the tensor-memory loads of the next 16 columns are in flight while these are processed
                uint32_t ca[2][16], cb[2][16];
                tmem_ld16_nowait(c_a, ca[0]);
                tmem_ld16_nowait(c_b, cb[0]);
                tmem_ld_wait16(ca[0]);
                tmem_ld_wait16(cb[0]);
#pragma unroll
                for (int p = 0; p < S3_COLS / 16; p++) {
                    if (p + 1 < S3_COLS / 16) {
                        tmem_ld16_nowait(c_a + (uint32_t)((p + 1) * 16), ca[(p + 1) & 1]);
                        tmem_ld16_nowait(c_b + (uint32_t)((p + 1) * 16), cb[(p + 1) & 1]);
                    }
                    const uint32_t(&va)[16] = ca[p & 1];
                    const uint32_t(&vb)[16] = cb[p & 1];
#pragma unroll
                    for (int h = 0; h < 4; h++) {
                        // four band columns = two packed pairs
                        const ulonglong2 xq = *reinterpret_cast<const ulonglong2 *>(xs + p * 16 + h * 4);
#pragma unroll
                        for (int q = 0; q < 2; q++) {
                            const int jj = p * 16 + h * 4 + 2 * q;  // even
                            const f32x2 xj2 = q ? xq.y : xq.x;
                            const f32x2 ta2 = sub2(xa2, xj2), tb2 = sub2(xb2, xj2);
                            const f32x2 ea2 = ex2_approx2(mul2(mul2(ta2, ta2), c02));
                            const f32x2 eb2 = ex2_approx2(mul2(mul2(tb2, tb2), c02));
                            uint32_t a0 = va[h * 4 + 2 * q], a1 = va[h * 4 + 2 * q + 1];
                            uint32_t b0 = vb[h * 4 + 2 * q], b1 = vb[h * 4 + 2 * q + 1];
                            if (MASKED) {
                                const int j = j0 + jj;
                                if (j < lo_a || j >= hi_a) a0 = 0u;
                                if (j + 1 < lo_a || j + 1 >= hi_a) a1 = 0u;
                                if (j < lo_b || j >= hi_b) b0 = 0u;
                                if (j + 1 < lo_b || j + 1 >= hi_b) b1 = 0u;
                            }
                            const f32x2 wa2 = mul2((f32x2)a0 | ((f32x2)a1 << 32), ea2);
                            const f32x2 wb2 = mul2((f32x2)b0 | ((f32x2)b1 << 32), eb2);
                            // rhs pairs of the two band columns (a broadcast read) serve both rows
                            const float *rp = rs + (jj >> 1) * (2 * KB);
#pragma unroll
                            for (int c2 = 0; c2 < KB / 2; c2++) {
                                const ulonglong2 rv = *reinterpret_cast<const ulonglong2 *>(rp + c2 * 4);
                                acc_a[c2 * 2 + 0] = fma2(wa2, rv.x, acc_a[c2 * 2 + 0]);
                                acc_a[c2 * 2 + 1] = fma2(wa2, rv.y, acc_a[c2 * 2 + 1]);
                                acc_b[c2 * 2 + 0] = fma2(wb2, rv.x, acc_b[c2 * 2 + 0]);
                                acc_b[c2 * 2 + 1] = fma2(wb2, rv.y, acc_b[c2 * 2 + 1]);
                            }
                        }
                    }
                    if (p + 1 < S3_COLS / 16) {
                        tmem_ld_wait16(ca[(p + 1) & 1]);
                        tmem_ld_wait16(cb[(p + 1) & 1]);
                    }
                }
            };
            // (the C tile of an absent block is never written: its mask is empty)
            const bool inside_a = j0 >= lo_a && j0 + S3_COLS <= hi_a, inside_b = j0 >= lo_b && j0 + S3_COLS <= hi_b;
            if (inside_a && inside_b)
                consume(std::false_type{});
            else
                consume(std::true_type{});
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bar_cfree[g]);
                mbar_arrive(&bar_infree[t % S3_IN_STAGES]);
            }
        }
        if (failed) atomicExch(&fail_flag, 1);
    }

    tc_fence_before();
    __syncthreads();
    float out_a[KB], out_b[KB];
#pragma unroll
    for (int c = 0; c < KB; c++) {
        float even, odd;
        unpack2(acc_a[c], even, odd);
        out_a[c] = even + odd;
        unpack2(acc_b[c], even, odd);
        out_b[c] = even + odd;
    }
    {
        // the second group hands its partial sums over through shared memory (the pipelines are done)
        float *xch = reinterpret_cast<float *>(smem_raw);
        if (is_row && g == 1) {
#pragma unroll
            for (int c = 0; c < KB; c++) {
                xch[c * 128 + row_local] = out_a[c];
                xch[(KB + c) * 128 + row_local] = out_b[c];
            }
        }
        __syncthreads();
        if (is_row && g == 0) {
#pragma unroll
            for (int c = 0; c < KB; c++) {
                out_a[c] += xch[c * 128 + row_local];
                out_b[c] += xch[(KB + c) * 128 + row_local];
            }
        }
    }
    if (is_row && g == 0) {
        const bool bad = fail_flag != 0;
        for (int blk = has_a ? 0 : 1; blk < (has_b ? 2 : 1); blk++) {
            const int64_t row = (rA + blk) * KM_BLOCK_SIZE + row_local;
            if (row < a.m) {
                float *orow = a.out.data + (row - a.rb_begin * KM_BLOCK_SIZE) * a.out.s0;
#pragma unroll
                for (int c = 0; c < KB; c++)
                    if (c < a.k) {
                        // later chunks of a sum over more than 64 components add to the first chunk's result
                        const float prev = a.comp_begin > 0 ? orow[c * a.out.s1] : 0.0f;
                        const float v = blk ? out_b[c] : out_a[c];
                        orow[c * a.out.s1] = bad ? __int_as_float(0x7fc00000) : v + prev;
                    }
            }
        }
    }
    if (is_mma_warp && fail_flag) {
        // after a give-up MMAs may still be running: one commit covers everything this thread has
        // issued; tensor memory is released only when both issuing warps have seen theirs complete
        if (lane == 0) {
            mma_commit(&bar_drain[g]);
            mbar_wait(&bar_drain[g], 0u, TC_WAIT_POLLS);
        }
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) tmem_free(tmem_base, S3_TMEM_COLS);
}

template <int KB>
static int launch_sum_tc3_kb(const SumTcArgs &a, cudaStream_t stream) {
    const int Bp = ((int)a.comp_count + 7) & ~7;
    const size_t b_stage = (size_t)2 * (2 * Bp / 8) * S3_COLS * 16;
    size_t smem = S3_PSI_STAGES * b_stage + (size_t)S3_IN_STAGES * (S3_COLS + S3_COLS * KB) * sizeof(float);
    // a CTA takes all 512 tensor-memory columns of an SM: keep a second one from being scheduled there
    smem = std::max<size_t>(smem, 120 * 1024);
    auto kernel = matmul_sum_tc3_kernel<KB>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(matmul_sum_tc3)");
    // the pairs (2 q, 2 q + 1) of row blocks that overlap the window
    const int64_t pairs = (a.rb_begin + a.row_blocks - 1) / 2 - a.rb_begin / 2 + 1;
    kernel<<<(unsigned)pairs, S3_THREADS, smem, stream>>>(a);
    KM_CHECK_LAUNCH("km_matmul_rows_f32 (tensor-core batch sum, two row blocks per CTA) launch");
    return KM_OK;
}

int launch_matmul_sum_tc3(const SumTcArgs &a, cudaStream_t stream) {
    if (a.row_blocks > 0x7fffffffLL) {
        set_error("km_matmul_rows_f32: too many row blocks (%lld)", (long long)a.row_blocks);
        return KM_ERR_UNSUPPORTED;
    }
    if (a.row_blocks <= 0) return KM_OK;
    // more than 64 components: chunks of 64, each launch adding to the result of the previous ones
    // (launches on one stream run in order)
    SumTcArgs chunk = a;
    chunk.wait_polls = current_wait_polls();
    for (int64_t b0 = 0; b0 < a.batch.count; b0 += SUM_TC_MAX_COMPONENTS) {
        chunk.comp_begin = b0;
        chunk.comp_count = std::min<int64_t>(SUM_TC_MAX_COMPONENTS, a.batch.count - b0);
        const int rc = a.k <= 8 ? launch_sum_tc3_kb<8>(chunk, stream) : launch_sum_tc3_kb<16>(chunk, stream);
        if (rc != KM_OK) return rc;
    }
    return KM_OK;
}

}  // namespace km

// Batch sum of spectral components on the tensor cores:
//
//   out[i, :] = sum_{j in band} ( sum_b s_b exp(-tau^2 / 2 l^2) cos(w_b tau) ) rhs[j, :],   tau = x_i - x_j
//
// for components that share inputs, band, right-hand side and lengthscale (64 per launch; the
// reference's SumKernel over a batch of spectral kernels, kernel_matmul/gpytorch/sum.py:16-24).
// The FMA-pipe kernel (km_matmul.cu) evaluates one SFU cosine per entry and component.  Here the
// sum over the components is turned into a dot product the tensor core can do:
//
//   cos(w (a_i - a_j)) = cos(w a_i) cos(w a_j) + sin(w a_i) sin(w a_j),   a = x - x0
//   sum_b s_b cos(w_b tau) = < phi(a_i), psi(a_j) >,
//   phi(a) = (s_b cos(w_b a), s_b sin(w_b a))_b,   psi(a) = (cos(w_b a), sin(w_b a))_b   in R^(2B)
//
// with x0 the centre of the CTA's row block, so that |a| stays as small as |tau| and the phases
// keep their fp32 accuracy.  Per 128-row block and tile of 64 band columns:
//   * phi of the 128 rows is computed once, split into fp16 hi / lo and written to tensor
//     memory (A operand, as in km_matmul_tc.cu);
//   * psi of the 64 columns (2B SFU operations per column) is written to shared memory as the B
//     operand, hi / lo fp16 in the K-major core-matrix layout;
//   * a control warp issues tcgen05.mma kind::f16 (N = 64, K = 16; 3 per 16 values of 2B) into
//     one of two tensor-memory stages: C[128 x 64] = sum_b s_b cos(w_b tau);
//   * the row threads read C with tcgen05.ld, multiply by the envelope exp(-tau^2 / 2 l^2) (one
//     SFU operation per entry) and contract with the rhs tile (k <= 16 columns, FMA pipe).  All of
//     that arithmetic is packed (f32x2): a thread handles the band columns two at a time -- tau,
//     the exponent and the product for (j, j + 1) are one instruction each -- and the rhs tile
//     lies in shared memory as pairs (rhs[j][c], rhs[j + 1][c]), so that one fma.rn.f32x2 adds
//     both columns' contributions to output column c (even and odd band columns keep separate
//     partial sums, added at the end).
// SFU work per entry: 1 + 2B / 128 (psi is shared by the 128 rows) instead of B + 1.
//
// No workspace: a CTA whose bounded wait gives up writes NaN into its output rows.
#include <cstdlib>

#include "km_tcgen05.cuh"

namespace km {

constexpr int ST_COLS = 64;       // band columns per tile = GEMM N
constexpr int ST_IN_STAGES = 4;   // x2 / rhs tiles in shared memory
constexpr int ST_TMEM_COLS = 256; // A (2 * 64) + two C stages of 64
constexpr int ST_C_COL = 128;     // first C column

// KB: rhs columns held per thread (8 or 16).  G: groups of 128 row threads.  With G = 2 the two
// groups own the same rows (tensor-memory lanes) and alternate tiles: group g generates psi for,
// and consumes, the tiles t = g, g + 2, ... through psi / C stage g, each with its own partial
// sums, which are added at the end.  Twice the warps per SM hide the latencies (SFU results,
// tensor-memory loads, MMA completion) that a single group per CTA leaves exposed.
//
// MS (KB = 8, G = 2): the contraction with the rhs tile runs on the warp-level tensor path
// (mma.sync m16n8k8, 3xTF32) instead of the FMA pipe.  A thread then reads C in the register layout
// of an m16n8 accumulator (tcgen05.ld.16x256b: two rows, two adjacent band columns per load),
// multiplies by the envelope and uses the products as the A fragment -- band columns (2t, 2t + 1)
// standing for the fragment's columns (t, t + 4), the rhs pairs in shared memory laid out to
// match -- so that per 128 entries a warp issues three MMAs and reads 8 bytes of rhs per thread,
// where the FMA form issues 16 packed FMAs and reads 128 bytes.
template <int KB, int G, bool MS>
__global__ void __launch_bounds__(128 * G + 32, 2) matmul_sum_tc_kernel(const SumTcArgs a) {
    static_assert(!MS || (KB == 8 && G == 2), "the warp-level contraction is written for 8 rhs columns, two row groups");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_in[ST_IN_STAGES];  // x2 + rhs tile landed
    __shared__ __align__(8) uint64_t bar_bready[3];         // psi tile written
    __shared__ __align__(8) uint64_t bar_pfree[3];          // psi tile read by its MMAs (tcgen05.commit)
    __shared__ __align__(8) uint64_t bar_cfull[2];          // C tile complete (tcgen05.commit)
    __shared__ __align__(8) uint64_t bar_cfree[2];          // C tile consumed
    __shared__ __align__(8) uint64_t bar_drain;             // give-up path: every issued MMA has completed
    __shared__ uint32_t tmem_base_slot;
    __shared__ int fail_flag;
    __shared__ __align__(16) float w_tab[SUM_TC_MAX_COMPONENTS];
    __shared__ __align__(16) float s_tab[SUM_TC_MAX_COMPONENTS];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const bool is_ctl_warp = warp == 4 * G;
    const int g = tid >> 7;            // row group
    const int row_local = tid & 127;  // row of the block = tensor-memory lane
    const int B = (int)a.comp_count;  // components of this launch: [comp_begin, comp_begin + B)
    const int Bp = (B + 7) & ~7;  // components padded to whole MMA steps (K = 2 Bp)
    const int ksteps = Bp / 8;
    static_assert(SUM_TC_MAX_COMPONENTS == 64, "the MMA issue code covers 1 .. 8 k-steps");

    // every CTA checks that the components share one lengthscale; if not, the FMA-pipe kernel
    // launched next to this one does the work and this CTA leaves at once
    const float ell0 = a.params.data[0];
    int same = 1;
    // (the lengthscales of ALL components are compared, so that every launch of a chunked sum and
    // the FMA-pipe kernel come to the same decision)
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

    // shared memory: two psi stages [part: hi, lo][chunk = K / 8][j][8 halfs], then the input stages
    const int b_part_bytes = (2 * Bp / 8) * ST_COLS * 16;
    const int b_stage_bytes = 2 * b_part_bytes;
    // With two row groups and k <= 8 there is room for a third psi stage (two CTAs per SM): a group
    // then writes psi of its NEXT tile while the MMAs of its current one run, instead of idling.
    constexpr bool AHEAD = G == 2 && KB == 8;
    constexpr int P = AHEAD ? 3 : 2;  // psi stages; tile t uses stage t % P
    unsigned char *in_base = smem_raw + P * b_stage_bytes;
    // rhs rows lie in shared memory as pairs of band columns: rs[((jj / 2) * RS + c) * 2 + (jj & 1)];
    // RS = 12 spreads the warp-level form's reads (thread: pair-row 4 cb + lane % 4, column lane / 4)
    // over the banks
    constexpr int RS = MS ? 12 : KB;
    constexpr int IN_STAGE_FLOATS = ST_COLS + ST_COLS * RS;  // x2 values, then rhs rows
    auto b_stage = [&](int st) { return smem_raw + st * b_stage_bytes; };
    auto in_x2 = [&](int st) { return reinterpret_cast<float *>(in_base) + st * IN_STAGE_FLOATS; };
    auto in_rhs = [&](int st) { return reinterpret_cast<float *>(in_base) + st * IN_STAGE_FLOATS + ST_COLS; };

    const int64_t r = a.rb_begin + blockIdx.x;
    const int n = (int)a.n;
    const int band_lo = clamp_int(a.start.data[r * a.start.s0], 0, n);
    const int band_hi = max(band_lo, min(a.end.data[r * a.end.s0], n));
    const int tile_lo = band_lo / ST_COLS;
    const int tiles = band_hi > band_lo ? (band_hi + ST_COLS - 1) / ST_COLS - tile_lo : 0;
    const float *x2 = a.x2.data;
    const float *rhs = a.rhs.data;
    // origin of the phases: the middle row of the block
    const float x0 = a.x1.data[min(r * KM_BLOCK_SIZE + KM_BLOCK_SIZE / 2, a.m - 1) * a.x1.s0];

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < ST_IN_STAGES; s++) mbar_init(&bar_in[s], 32);  // one cp.async arrival per lane
#pragma unroll
        for (int s = 0; s < 2; s++) {
            mbar_init(&bar_cfull[s], 1);
            mbar_init(&bar_cfree[s], 4);
        }
#pragma unroll
        for (int s = 0; s < 3; s++) {
            mbar_init(&bar_bready[s], 4);
            mbar_init(&bar_pfree[s], 1);
        }
        mbar_init(&bar_drain, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (is_ctl_warp) tmem_alloc(&tmem_base_slot, ST_TMEM_COLS);
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
        // ------------------------------------------------ input fetches (all lanes) + MMA issue (lane 0)
        auto fetch = [&](int t) {
            const int st = t % ST_IN_STAGES;
            const int64_t j0 = (int64_t)(tile_lo + t) * ST_COLS;
            float *xs = in_x2(st);
            float *rs = in_rhs(st);
#pragma unroll
            for (int u = 0; u < ST_COLS / 32; u++) {
                const int jj = lane + 32 * u;
                const bool valid = j0 + jj < n;
                cp_async4_zfill(xs + jj, x2 + (valid ? j0 + jj : 0) * a.x2.s0, valid);
            }
            // rhs rows in pairs: rs[((jj / 2) * RS + c) * 2 + (jj & 1)] = rhs[j0 + jj][c]
            for (int q = lane; q < ST_COLS * KB; q += 32) {
                const int jj = q / KB, c = q % KB;
                const bool valid = j0 + jj < n && c < a.k;
                cp_async4_zfill(rs + (((jj >> 1) * RS + c) << 1) + (jj & 1),
                                rhs + (valid ? (j0 + jj) * a.rhs.s0 + c * a.rhs.s1 : 0), valid);
            }
            cp_async_mbar_arrive(&bar_in[st]);
        };
        for (int t = 0; t < min(tiles, ST_IN_STAGES); t++) fetch(t);

        // D fp32, A / B fp16, K-major, M = 128, N = 64
        constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(ST_COLS >> 3) << 17) | ((128u >> 4) << 24);
        constexpr uint32_t lbo_b = ST_COLS * 16, sbo = 128;
        constexpr uint64_t kstep_b = (uint64_t)(2 * lbo_b) >> 4;  // 16 K values = 2 chunks
        const uint64_t part_step = (uint64_t)b_part_bytes >> 4;
        const uint64_t stage_step = (uint64_t)b_stage_bytes >> 4;
        const uint64_t d_b0 = smem_desc(smem_u32(b_stage(0)), lbo_b, sbo);
        for (int t = 0; t < tiles; t++) {
            const int st = t & 1;
            bool ok = true;
            if (t >= 2) {
                // C stage free = tile t - 2 consumed, which also frees its input stage
                ok = mbar_wait(&bar_cfree[st], (unsigned)(((t >> 1) - 1) & 1), a.wait_polls);
                if (__all_sync(0xffffffffu, ok) && t + 2 < tiles) fetch(t + 2);
            }
            if (ok) ok = mbar_wait(&bar_bready[t % P], (unsigned)((t / P) & 1), a.wait_polls);
            if (!__all_sync(0xffffffffu, ok)) {
                failed = true;
                break;
            }
            tc_fence_after();
            if (lane == 0) {
                const uint32_t d_tmem = tmem_base + (uint32_t)(ST_C_COL + st * ST_COLS);
                const uint64_t b_hi = d_b0 + (t % P) * stage_step, b_lo = b_hi + part_step;
                // straight-line code per k-step count (a partially unrolled run-time loop of MMAs gave
                // wrong tiles in the gradient kernel; see there)
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
                if (AHEAD) mma_commit(&bar_pfree[t % P]);
            }
            __syncwarp();
        }
        if (failed && lane == 0) atomicExch(&fail_flag, 1);
        cp_async_wait<0>();  // no copy may be in flight when the CTA exits
        __syncwarp();
    } else {
        // ------------------------------------------------------------------------ row threads
        const int64_t row = r * KM_BLOCK_SIZE + row_local;
        const float x1v = row < a.m ? a.x1.data[row * a.x1.s0] : x0;
        const uint32_t tmem_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        // warp-level form: x1 of this thread's four rows 32 (warp % 4) + 16 mt + lane / 4 + 8 hh, as pairs
        f32x2 xi2[2][2];
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int64_t ri = r * KM_BLOCK_SIZE + (warp & 3) * 32 + 16 * mt + (lane >> 2) + 8 * hh;
                xi2[mt][hh] = splat2((MS && ri < a.m) ? a.x1.data[ri * a.x1.s0] : x0);
            }

        // phi of this row -> tensor memory: per 8 components [8 hi pairs | 8 lo pairs]
        {
            const float ai = x1v - x0;
            for (int ks = g; ks < ksteps; ks += G) {
                float v[16], lo[16];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const float ph = w_tab[ks * 8 + u] * ai, sc = s_tab[ks * 8 + u];
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
            if (G > 1) asm volatile("bar.sync 1, %0;" ::"n"(128 * G) : "memory");
        }

        // psi of the tile's columns -> shared memory (thread: column row_local % 64, half of the components)
        auto generate = [&](int t) {
            const int st = t % P;
            const int jj = row_local & 63;
            const float aj = in_x2(t % ST_IN_STAGES)[jj] - x0;
            unsigned char *hi = b_stage(st) + jj * 16;
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
                    const f32x2 lo2 = sub2(v2, v2 & 0xffffe000ffffe000ull);
                    float vc, vs, lc, ls;
                    unpack2(v2, vc, vs);
                    unpack2(lo2, lc, ls);
                    asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(h[u]) : "f"(vs), "f"(vc));
                    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(l[u]) : "f"(ls), "f"(lc));
                }
                *reinterpret_cast<uint4 *>(hi + kc * (ST_COLS * 16)) = make_uint4(h[0], h[1], h[2], h[3]);
                *reinterpret_cast<uint4 *>(lo + kc * (ST_COLS * 16)) = make_uint4(l[0], l[1], l[2], l[3]);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_bready[st]);
        };

        if (G == 1 && tiles > 0) {
            if (!mbar_wait_warp(&bar_in[0], 0u, a.wait_polls)) failed = true;
            if (!failed) generate(0);
        }
        if (AHEAD && g < tiles) {
            if (!mbar_wait_warp(&bar_in[g], 0u, a.wait_polls)) failed = true;
            if (!failed) generate(g);
        }
        for (int t = (G == 1 ? 0 : g); t < tiles && !failed; t += G) {
            const int st = t & 1;
            if (AHEAD) {
                // psi of this group's next tile while the MMAs of tile t run; its psi stage was last
                // read by the MMAs of tile t - 1
                if (t + 2 < tiles) {
                    bool ok = mbar_wait_warp(&bar_in[(t + 2) % ST_IN_STAGES], (unsigned)(((t + 2) / ST_IN_STAGES) & 1), a.wait_polls);
                    if (ok && t >= 1) ok = mbar_wait_warp(&bar_pfree[(t - 1) % P], (unsigned)(((t - 1) / P) & 1), a.wait_polls);
                    if (!ok) {
                        failed = true;
                        break;
                    }
                    generate(t + 2);
                }
            } else if (G > 1) {
                // this group's tile: psi first, then the product of the tensor core
                if (!mbar_wait_warp(&bar_in[t % ST_IN_STAGES], (unsigned)((t / ST_IN_STAGES) & 1), a.wait_polls)) {
                    failed = true;
                    break;
                }
                generate(t);
            } else if (t + 1 < tiles) {
                // (the psi stage of tile t + 1 was read by the MMAs of tile t - 1, whose completion
                // this thread has seen when it consumed tile t - 1)
                if (!mbar_wait_warp(&bar_in[(t + 1) % ST_IN_STAGES], (unsigned)(((t + 1) / ST_IN_STAGES) & 1), a.wait_polls)) {
                    failed = true;
                    break;
                }
                generate(t + 1);
            }
            if (!mbar_wait_warp(&bar_cfull[st], (unsigned)((t >> 1) & 1), a.wait_polls)) {
                failed = true;
                break;
            }
            tc_fence_after();
            const int j0 = (tile_lo + t) * ST_COLS;
            const float *xs = in_x2(t % ST_IN_STAGES);
            const float *rs = in_rhs(t % ST_IN_STAGES);
            const f32x2 x1v2 = splat2(x1v), c02 = splat2(c0);
            auto consume = [&](auto masked_tag) {
                constexpr bool MASKED = decltype(masked_tag)::value;
                // the tensor-memory load of the next 16 columns is in flight while these are processed
                uint32_t cbuf[2][16];
                tmem_ld16_nowait(tmem_lane + (uint32_t)(ST_C_COL + st * ST_COLS), cbuf[0]);
                tmem_ld_wait16(cbuf[0]);
#pragma unroll
                for (int p = 0; p < ST_COLS / 16; p++) {
                    if (p + 1 < ST_COLS / 16)
                        tmem_ld16_nowait(tmem_lane + (uint32_t)(ST_C_COL + st * ST_COLS + (p + 1) * 16), cbuf[(p + 1) & 1]);
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
                    if (p + 1 < ST_COLS / 16) tmem_ld_wait16(cbuf[(p + 1) & 1]);
                }
            };
            auto consume_ms = [&](auto masked_tag) {
                constexpr bool MASKED = decltype(masked_tag)::value;
                const int gq = lane >> 2, tq = lane & 3;
                constexpr f32x2 HI2 = 0xffffe000ffffe000ull;  // the tf32 part of both values of a pair
                const uint32_t c_tile = tmem_lane + (uint32_t)(ST_C_COL + st * ST_COLS);
                // the loads of the next 8 columns are in flight while these are processed
                uint32_t cv[2][2][4];  // [buffer][16-row tile][fragment]
                tmem_ld_m16n8_nowait(c_tile, cv[0][0]);
                tmem_ld_m16n8_nowait(c_tile + (16u << 16), cv[0][1]);
                tmem_ld_wait4x2(cv[0][0], cv[0][1]);
#pragma unroll
                for (int cb = 0; cb < ST_COLS / 8; cb++) {
                    if (cb + 1 < ST_COLS / 8) {
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
                    if (cb + 1 < ST_COLS / 8) tmem_ld_wait4x2(cv[(cb + 1) & 1][0], cv[(cb + 1) & 1][1]);
                }
            };
            const bool edge = j0 < band_lo || j0 + ST_COLS > band_hi;
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
    } else if (G > 1) {
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
        tmem_free(tmem_base, ST_TMEM_COLS);
    }
}

template <int KB, int G, bool MS = false>
static int launch_sum_tc_kb(const SumTcArgs &a, cudaStream_t stream) {
    const int Bp = ((int)a.comp_count + 7) & ~7;
    const size_t b_stage = (size_t)2 * (2 * Bp / 8) * ST_COLS * 16;
    const int psi_stages = (G == 2 && KB == 8) ? 3 : 2;
    size_t smem = psi_stages * b_stage + (size_t)ST_IN_STAGES * (ST_COLS + ST_COLS * (MS ? 12 : KB)) * sizeof(float);
    // two CTAs of 256 tensor-memory columns fill an SM: keep a third from being scheduled
    smem = std::max<size_t>(smem, 80 * 1024);
    auto kernel = matmul_sum_tc_kernel<KB, G, MS>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(matmul_sum_tc)");
    kernel<<<(unsigned)a.row_blocks, 128 * G + 32, smem, stream>>>(a);
    KM_CHECK_LAUNCH("km_matmul_rows_f32 (tensor-core batch sum) launch");
    return KM_OK;
}

// Row groups per CTA: 2, or what the environment variable KM_SUM_TC_GROUPS says (1 or 2; read at
// every launch; a tuning and comparison hook).
static int sum_tc_groups() {
    const char *e = getenv("KM_SUM_TC_GROUPS");
    return (e != nullptr && e[0] == '1') ? 1 : 2;
}

// Contraction with the rhs tile (two row groups, k <= 8): on the FMA pipe, or on the warp-level
// tensor path when the environment variable KM_SUM_TC_WARP_MMA is 1 (read at every launch; measured
// slower on the 64-component benchmark, 12.6 against 11.6 ms: it reads an eighth of the
// shared-memory bytes, but issues as many instructions, and mma.sync shares the tensor pipe with
// tcgen05.mma: a comparison hook).
static bool sum_tc_warp_mma() {
    const char *e = getenv("KM_SUM_TC_WARP_MMA");
    return e != nullptr && e[0] == '1';
}

int sum_tc_variant() {
    const char *e = getenv("KM_SUM_TC_VARIANT");  // read at every launch: tests switch it at run time
    if (e != nullptr && e[0] == '2') return 2;
    if (e != nullptr && e[0] == '3') return 3;
    return 1;
}

int launch_matmul_sum_tc(const SumTcArgs &a, cudaStream_t stream) {
    if (a.row_blocks > 0x7fffffffLL) {
        set_error("km_matmul_rows_f32: too many row blocks (%lld)", (long long)a.row_blocks);
        return KM_ERR_UNSUPPORTED;
    }
    // more than 64 components: chunks of 64, each launch adding to the result of the previous ones
    // (launches on one stream run in order)
    SumTcArgs chunk = a;
    chunk.wait_polls = current_wait_polls();
    for (int64_t b0 = 0; b0 < a.batch.count; b0 += SUM_TC_MAX_COMPONENTS) {
        chunk.comp_begin = b0;
        chunk.comp_count = std::min<int64_t>(SUM_TC_MAX_COMPONENTS, a.batch.count - b0);
        int rc;
        if (sum_tc_groups() == 1)
            rc = a.k <= 8 ? launch_sum_tc_kb<8, 1>(chunk, stream) : launch_sum_tc_kb<16, 1>(chunk, stream);
        else if (a.k <= 8)
            rc = sum_tc_warp_mma() ? launch_sum_tc_kb<8, 2, true>(chunk, stream) : launch_sum_tc_kb<8, 2>(chunk, stream);
        else
            rc = launch_sum_tc_kb<16, 2>(chunk, stream);
        if (rc != KM_OK) return rc;
    }
    return KM_OK;
}

}  // namespace km

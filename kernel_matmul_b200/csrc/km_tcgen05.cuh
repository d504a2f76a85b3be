// tcgen05 / tensor-memory / mbarrier / bulk-copy PTX wrappers shared by the tensor-core kernels
// (km_matmul_tc.cu, km_grad_tc.cu).  sm_100a only.
#pragma once

#include "km_common.cuh"

namespace km {

constexpr int TC_STATUS_BYTES = 256;  // status word + padding in front of the workspace payload

// Arguments of the tensor-core product (filled by km_matmul_tc_f32).
struct TcArgs {
    Batch batch;
    int64_t m, n, k;
    int64_t row_blocks, rb_begin;
    int k_blocks;   // blocks of n_pad rhs columns
    int n_pad;      // GEMM N per block: 16, 32, 64 or 128
    int64_t tiles;  // 64-column groups per image: ceil(n / 64)
    View<const float> x1, x2, params;
    View<const int> start, end;
    View<float> out;
    const float *images;         // fp16 images [image slot][column block][64-column group][hi, lo][chunk][c][8]
    int64_t image_slot_stride;   // non-zero: every batch has its own images (0: rhs shared by all batches)
    const float *col_inv_scale;  // per (image slot, column block): inverse of the per-column rhs scales
    int *status;
    unsigned wait_polls;         // poll limit of every hand-off wait (TC_WAIT_POLLS unless a self-test lowered it)
};

// Number of distinct rhs images: 1 when every batch shares one rhs (all batch strides 0).
inline int64_t tc_slots(const Batch &b, const View<const float> &rhs) {
    bool shared = true;
    for (int d = 0; d < b.ndim; d++) shared = shared && (rhs.bs[d] == 0 || b.size[d] == 1);
    return shared ? 1 : b.count;
}

constexpr unsigned TC_WAIT_POLLS = 1u << 18;  // each poll may block for a short, system-defined time
// Poll limit the launchers put into the kernel arguments: TC_WAIT_POLLS, or what
// km_selftest_set_wait_polls() set (km_api.cu).
unsigned current_wait_polls();

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity.  false = gave up.  A non-blocking test comes
// first (the phase is usually complete already); then try_wait, which suspends the thread for a
// short, system-defined time per poll (an explicit suspend-time hint only added instructions).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity, unsigned polls) {
    const uint32_t addr = smem_u32(bar);
    {
        // the phase is usually complete already: a non-blocking test first
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    for (unsigned poll = 0; poll < polls; poll++) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// The same wait with a warp-uniform outcome (all 32 lanes must call it): false if any lane gave
// up, so that a warp leaves its loop as a whole and .aligned instructions stay warp-wide.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, unsigned parity, unsigned polls) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, polls));
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
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
                 :
                 : "memory");
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
}

// 16 / 32 consecutive columns of this thread's lane; the wait is issued by the caller
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// A 16-lane x 8-column tile of tensor memory (the lane field of `taddr` names the first of the 16
// lanes: offset 0 or 16 inside the warp's 32) in the register layout of an mma.sync m16n8
// accumulator: thread T holds (lane T / 4, columns 2 (T % 4) and 2 (T % 4) + 1) in r[0], r[1] and
// (lane T / 4 + 8, the same columns) in r[2], r[3].  The wait is issued by the caller.
__device__ __forceinline__ void tmem_ld_m16n8_nowait(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x1.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}
// The wait for two such loads, tied to their registers (see tmem_ld_wait16)
__device__ __forceinline__ void tmem_ld_wait4x2(uint32_t (&p)[4], uint32_t (&q)[4]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(p[0]), "+r"(p[1]), "+r"(p[2]), "+r"(p[3]), "+r"(q[0]), "+r"(q[1]), "+r"(q[2]), "+r"(q[3])
                 :
                 : "memory");
}
// d (16 x 8, fp32) += a (16 x 8, tf32, row-major fragment) . b (8 x 8, tf32, column fragment) on
// the warp-level tensor path; operands are fp32 bit patterns of which the tensor core uses the
// leading 19 bits
__device__ __forceinline__ void mma_sync_tf32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The wait for the loads into `r`, tied to those registers: the registers of a tcgen05.ld are
// valid only after tcgen05.wait::ld, but as operands they look complete to the compiler as soon
// as the load is issued, so arithmetic on them could be scheduled ahead of a wait that does not
// name them (seen as wrong results once the tensor cores were busy enough to delay the load).
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 : "memory");
}

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

// registers -> 16 consecutive tensor-memory columns of this thread's lane
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// A packed pair of fp32 values -> one 32-bit word of two fp16 values (first element in the low
// half), truncating (rz: the fp16 "hi" part of a value) or rounding to nearest (rn).  The pair is
// taken apart inside the asm block, so the compiler sees no separate fp32 values to move around.
__device__ __forceinline__ uint32_t cvt_rz_f16x2_pair(unsigned long long v) {
    uint32_t r;
    asm("{\n\t.reg .f32 a, b;\n\tmov.b64 {a, b}, %1;\n\tcvt.rz.f16x2.f32 %0, b, a;\n\t}" : "=r"(r) : "l"(v));
    return r;
}
__device__ __forceinline__ uint32_t cvt_rn_f16x2_pair(unsigned long long v) {
    uint32_t r;
    asm("{\n\t.reg .f32 a, b;\n\tmov.b64 {a, b}, %1;\n\tcvt.rn.f16x2.f32 %0, b, a;\n\t}" : "=r"(r) : "l"(v));
    return r;
}
// Eight packed pairs of fp32 values (16 kernel entries) -> their fp16 hi parts (truncated) and lo
// parts (value - hi, rounded) -> 16 consecutive tensor-memory columns of this thread's lane:
// [8 hi words | 8 lo words].  One asm block from the pairs to the store, so that the conversions
// write straight into the consecutive registers tcgen05.st takes (with the words as C++ values
// the compiler moved each of them once: two moves per pair of entries).
__device__ __forceinline__ void split_store16_pairs(uint32_t taddr, const unsigned long long (&kv)[8]) {
#define KM_SPLIT_PAIR(U, HI, LO)                                  \
    "mov.b64 {x, y}, %" #U ";\n\t"                                 \
    "cvt.rz.f16x2.f32 " #HI ", y, x;\n\t"                          \
    "and.b64 m, %" #U ", 0xffffe000ffffe000;\n\t"                  \
    "sub.rn.f32x2 d, %" #U ", m;\n\t"                              \
    "mov.b64 {x, y}, d;\n\t"                                       \
    "cvt.rn.f16x2.f32 " #LO ", y, x;\n\t"
    asm volatile(
        "{\n\t"
        ".reg .b32 p<16>;\n\t"
        ".reg .f32 x, y;\n\t"
        ".reg .b64 m, d;\n\t"
        KM_SPLIT_PAIR(1, p0, p8) KM_SPLIT_PAIR(2, p1, p9) KM_SPLIT_PAIR(3, p2, p10) KM_SPLIT_PAIR(4, p3, p11)
        KM_SPLIT_PAIR(5, p4, p12) KM_SPLIT_PAIR(6, p5, p13) KM_SPLIT_PAIR(7, p6, p14) KM_SPLIT_PAIR(8, p7, p15)
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {p0, p1, p2, p3, p4, p5, p6, p7, p8, p9, p10, p11, p12, p13, p14, p15};\n\t"
        "}"
        :
        : "r"(taddr), "l"(kv[0]), "l"(kv[1]), "l"(kv[2]), "l"(kv[3]), "l"(kv[4]), "l"(kv[5]), "l"(kv[6]), "l"(kv[7])
        : "memory");
#undef KM_SPLIT_PAIR
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 4-byte asynchronous copy that writes zero when `valid` is false (the source is not read)
__device__ __forceinline__ void cp_async4_zfill(void *smem, const void *gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const unsigned bytes = valid ? 4u : 0u;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
// arrive on `bar` once all earlier cp.async copies of this thread have landed (the arrival is
// part of the barrier's expected count)
__device__ __forceinline__ void cp_async_mbar_arrive(uint64_t *bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D (fp32, tensor memory) (+)= A (tensor memory, fp16: row i in lane i, two K values per 32-bit
// column) . B (smem, fp16); M = 128, N from idesc, K = 16.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// 16 values and their lo parts -> fp16 pairs [8 hi (truncated) | 8 lo (rounded)] -> 16 consecutive
// tensor-memory columns of this thread's lane.  One asm block, so that the conversions write
// straight into the consecutive registers tcgen05.st needs (no register moves in between).
__device__ __forceinline__ void split_store16(uint32_t taddr, const float (&v)[16], const float (&lo)[16]) {
    asm volatile(
        "{\n\t"
        ".reg .b32 p<16>;\n\t"
        "cvt.rz.f16x2.f32 p0, %2, %1;\n\t"
        "cvt.rz.f16x2.f32 p1, %4, %3;\n\t"
        "cvt.rz.f16x2.f32 p2, %6, %5;\n\t"
        "cvt.rz.f16x2.f32 p3, %8, %7;\n\t"
        "cvt.rz.f16x2.f32 p4, %10, %9;\n\t"
        "cvt.rz.f16x2.f32 p5, %12, %11;\n\t"
        "cvt.rz.f16x2.f32 p6, %14, %13;\n\t"
        "cvt.rz.f16x2.f32 p7, %16, %15;\n\t"
        "cvt.rn.f16x2.f32 p8, %18, %17;\n\t"
        "cvt.rn.f16x2.f32 p9, %20, %19;\n\t"
        "cvt.rn.f16x2.f32 p10, %22, %21;\n\t"
        "cvt.rn.f16x2.f32 p11, %24, %23;\n\t"
        "cvt.rn.f16x2.f32 p12, %26, %25;\n\t"
        "cvt.rn.f16x2.f32 p13, %28, %27;\n\t"
        "cvt.rn.f16x2.f32 p14, %30, %29;\n\t"
        "cvt.rn.f16x2.f32 p15, %32, %31;\n\t"
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {p0, p1, p2, p3, p4, p5, p6, p7, p8, p9, p10, p11, p12, p13, p14, p15};\n\t"
        "}"
        :
        : "r"(taddr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]), "f"(v[8]),
          "f"(v[9]), "f"(v[10]), "f"(v[11]), "f"(v[12]), "f"(v[13]), "f"(v[14]), "f"(v[15]), "f"(lo[0]), "f"(lo[1]),
          "f"(lo[2]), "f"(lo[3]), "f"(lo[4]), "f"(lo[5]), "f"(lo[6]), "f"(lo[7]), "f"(lo[8]), "f"(lo[9]), "f"(lo[10]),
          "f"(lo[11]), "f"(lo[12]), "f"(lo[13]), "f"(lo[14]), "f"(lo[15])
        : "memory");
}


// Batch sum of spectral components on the tensor cores (km_matmul_sum_tc.cu): arguments and launcher.
struct SumTcArgs {
    Batch batch;                // the components
    int64_t m, n, k;
    int64_t row_blocks, rb_begin;
    View<const float> x1, x2, rhs, params;  // x1, x2, rhs: one copy shared by all components
    View<const int> start, end;
    View<float> out;            // (rows_in_window, k)
    int64_t comp_begin, comp_count;  // components of one launch (set by the launcher)
    unsigned wait_polls;        // poll limit of every hand-off wait
    // precomputed phase images of one chunk of components (km_matmul_sum_ph.cu only)
    const unsigned char *psi_img = nullptr;
    const uint32_t *phi_img = nullptr;
};
constexpr int SUM_TC_MAX_COMPONENTS = 64;    // per launch; more are processed in chunks
constexpr int SUM_TC_MAX_TOTAL = 1024;       // (the FMA-pipe kernel's shared-envelope table holds this many)
constexpr int SUM_TC_MAX_K = 16;
int launch_matmul_sum_tc(const SumTcArgs &a, cudaStream_t stream);
// The same sum with the second contraction (kernel tile x rhs tile) on the tensor cores as well
// (km_matmul_sum_tc2.cu): correct, but measured slower than the first form (17.5 against 11.7 ms on
// the 64-component benchmark), so it only runs when asked for.
int launch_matmul_sum_tc2(const SumTcArgs &a, cudaStream_t stream);
// The first form with two row blocks per CTA (km_matmul_sum_tc3.cu): a thread owns a row of each,
// so the rhs values, the psi tile and the x2 values it brings in serve twice the entries.
int launch_matmul_sum_tc3(const SumTcArgs &a, cudaStream_t stream);
// The first form with the phase vectors precomputed once per operator (km_matmul_sum_ph.cu): the
// pre-pass, the size of its workspace and the product that reads it.
size_t sum_phases_workspace_bytes(int64_t components, int64_t m, int64_t n);
int sum_phases_prepare(const Batch &batch, const View<const float> &params, const View<const float> &x1,
                       const View<const float> &x2, int64_t m, int64_t n, int64_t row_begin, int64_t row_end,
                       int64_t col_begin, int64_t col_end, void *workspace, size_t workspace_bytes, cudaStream_t stream);
int launch_matmul_sum_ph(const SumTcArgs &a, const void *workspace, size_t workspace_bytes, cudaStream_t stream);
// Which one runs: 1, 2 or 3, from the environment variable KM_SUM_TC_VARIANT (read at every launch; a
// comparison hook).
int sum_tc_variant();

}  // namespace km

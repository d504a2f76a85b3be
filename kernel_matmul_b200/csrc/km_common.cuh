// Shared device/host helpers of the km_b200 library: argument views, batch addressing, the
// kernel functions and their parameter transforms, error reporting.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <climits>

#include "../../include/km_b200.h"

#define KM_PI_F 3.14159265358979323846f
#define KM_LOG2E_F 1.44269504088896340736f

namespace km {

// ------------------------------------------------------------------------------ host side

void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t err, const char *what);

#define KM_REQUIRE(cond, code, ...)                                                            \
    do {                                                                                       \
        if (!(cond)) {                                                                         \
            km::set_error(__VA_ARGS__);                                                        \
            return (code);                                                                     \
        }                                                                                      \
    } while (0)

#define KM_CHECK_LAUNCH(what)                                                                  \
    do {                                                                                       \
        cudaError_t err__ = cudaGetLastError();                                                \
        if (err__ != cudaSuccess) return km::cuda_fail(err__, what);                           \
    } while (0)

inline bool valid_kernel_type(int kt) { return kt >= 0 && kt <= 2; }
__host__ __device__ constexpr int num_params(int kt) { return kt == 0 ? 2 : (kt == 1 ? 3 : 4); }

// Batch geometry passed to kernels by value.
struct Batch {
    int ndim;
    int64_t size[KM_MAX_BATCH_DIMS];
    int64_t count;  // product of sizes (1 for ndim == 0)
};

// A km_view with typed pointer, passed to kernels by value.
template <typename T>
struct View {
    T *data;
    int64_t bs[KM_MAX_BATCH_DIMS];
    int64_t s0, s1;
};

// Validates a km_batch and fills Batch.  Returns KM_OK or sets the error.
int make_batch(const km_batch *in, Batch *out);

template <typename T>
inline View<T> make_view(const km_view *v, const Batch &b) {
    View<T> r;
    r.data = static_cast<T *>(v->data);
    for (int d = 0; d < KM_MAX_BATCH_DIMS; d++) r.bs[d] = d < b.ndim ? v->batch_stride[d] : 0;
    r.s0 = v->stride[0];
    r.s1 = v->stride[1];
    return r;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Second stage of every gradient op (km_grad.cu): per batch, add `units` partial records of
// KM_MAX_PARAMS values (fp32 or fp64) in a fixed order in fp64, apply the chain rule
// theta <- p and write grad[b, 0..P).
int launch_grad_finish(int kernel_type, const Batch &batch, int64_t units, const void *partials,
                       bool partials_fp64, const View<const float> &params, const View<float> &grad,
                       cudaStream_t stream);

// ---------------------------------------------------------------------------- device side

// Flattened batch index -> per-dimension indices (row-major over the batch dims).
struct BatchIndex {
    int64_t i[KM_MAX_BATCH_DIMS];
};

__device__ __forceinline__ BatchIndex decompose(const Batch &b, int64_t flat) {
    BatchIndex r;
#pragma unroll
    for (int d = KM_MAX_BATCH_DIMS - 1; d >= 0; d--) {
        if (d < b.ndim) {
            r.i[d] = flat % b.size[d];
            flat /= b.size[d];
        } else {
            r.i[d] = 0;
        }
    }
    return r;
}

template <typename T>
__device__ __forceinline__ T *batch_ptr(const View<T> &v, const BatchIndex &bi) {
    int64_t off = 0;
#pragma unroll
    for (int d = 0; d < KM_MAX_BATCH_DIMS; d++) off += bi.i[d] * v.bs[d];
    return v.data + off;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float cos_approx(float x) {
    float y;
    asm("cos.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float sin_approx(float x) {
    float y;
    asm("sin.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed FP32 pairs (Blackwell fma.rn.f32x2): one instruction issues two FMAs, which halves
// the issue slots of the contraction loops and leaves them to the SFU / load instructions.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 splat2(float v) { return pack2(v, v); }
// elementwise SFU functions of a pair
__device__ __forceinline__ f32x2 ex2_approx2(f32x2 x) {
    float a, b;
    unpack2(x, a, b);
    return pack2(ex2_approx(a), ex2_approx(b));
}
__device__ __forceinline__ f32x2 cos_approx2(f32x2 x) {
    float a, b;
    unpack2(x, a, b);
    return pack2(cos_approx(a), cos_approx(b));
}
__device__ __forceinline__ f32x2 sin_approx2(f32x2 x) {
    float a, b;
    unpack2(x, a, b);
    return pack2(sin_approx(a), sin_approx(b));
}

// Kernel functions.
//
// User parameters theta are mapped to device constants once per CTA (the reference launches
// ~6 small ATen kernels per call for this, native/common/kernel_function.cuh:198-219):
//   p0 = 1 / (2 l^2), spectral p1 = 2 f, locally periodic p1 = 2 / l_per, p2 = 1 / period.
// kappa is evaluated WITHOUT the output scale s (applied once per output element / per
// gradient sum) with the exponential on the SFU base-2 unit:
//   rbf               u(tau) = 2^(c0 tau^2),                      c0 = -p0 log2(e)
//   spectral          u(tau) = 2^(c0 tau^2) cos(w tau),           w  = pi p1 = 2 pi f
//   locally periodic  u(tau) = 2^(c0 tau^2 + c1 sin^2(w tau)),    c1 = -p1 log2(e), w = pi p2
// (values: native/common/kernel_function.cuh:25-58).
//
// Separable phases (tensor-core kernels).  cos / sin of a phase difference factor into
// per-point values, cos(W (a_i - a_j)) = c_i c_j + s_i s_j, sin(W (a_i - a_j)) = s_i c_j - c_i s_j
// with c = cos(W a), s = sin(W a): a kernel computes c_i, s_i once per row and c_j, s_j once
// per column of a tile and then needs no SFU sine / cosine per entry.  PHASE says whether the
// kernel type has such a factor, phase_w() is W (spectral: w; locally periodic: 2 w, because
// sin^2(w tau) = (1 - cos(2 w tau)) / 2 and sin(w tau) cos(w tau) = sin(2 w tau) / 2), and the
// *_ph functions take cs = cos(W tau), sn = sin(W tau) from the caller.
// A row block uses the separable form only while |W (x_i - x0)| <= KM_PHASE_MAX_ROW_ARG for all of
// its rows (x0: the block's middle row): the fp32 phase and the SFU's range reduction lose
// about 1e-7 of absolute accuracy per radian of argument.
#define KM_PHASE_MAX_ROW_ARG 16.0f
//
// The gradient code accumulates, per kernel type, NSUMS "raw" sums of coeff * (factor of u);
// finish_grad() turns them into d/d theta including the chain rule of
// native/common/kernel_function.cuh:92-163 and :221-251.
template <int KT>
struct KernelFn;

template <>
struct KernelFn<KM_KERNEL_RBF> {
    static constexpr int P = 2;
    static constexpr int NSUMS = 2;
    float c0, scale, ell;
    __device__ __forceinline__ void init(const float *theta, int64_t stride) {
        ell = theta[0];
        scale = theta[stride];
        c0 = -(0.5f / (ell * ell)) * KM_LOG2E_F;
    }
    __device__ __forceinline__ float unscaled(float tau) const { return ex2_approx(c0 * tau * tau); }
    // sums: [0] = sum coeff * e * tau^2, [1] = sum coeff * e
    __device__ __forceinline__ void accumulate(float tau, float coeff, float *sums) const {
        const float t2 = tau * tau;
        const float v = coeff * ex2_approx(c0 * t2);
        sums[0] = fmaf(v, t2, sums[0]);
        sums[1] += v;
    }
    // the same with full-precision library functions instead of the SFU approximations: for the
    // gather gradient, which adds few terms per batch (no averaging of the approximation errors)
    // and is bound by memory latency, not arithmetic
    __device__ __forceinline__ void accumulate_precise(float tau, float coeff, float *sums) const {
        const float t2 = tau * tau;
        const float v = coeff * exp2f(c0 * t2);
        sums[0] = fmaf(v, t2, sums[0]);
        sums[1] += v;
    }
    // the same for two entries at once with packed FP32 operations (half the issue slots);
    // sums2[q] holds the two partial sums of sums[q]
    __device__ __forceinline__ void accumulate2(f32x2 tau, f32x2 coeff, f32x2 *sums2) const {
        const f32x2 t2 = mul2(tau, tau);
        const f32x2 v = mul2(coeff, ex2_approx2(mul2(splat2(c0), t2)));
        sums2[0] = fma2(v, t2, sums2[0]);
        sums2[1] = add2(v, sums2[1]);
    }
    __device__ __forceinline__ f32x2 unscaled2(f32x2 tau) const {
        return ex2_approx2(mul2(splat2(c0), mul2(tau, tau)));
    }
    static constexpr bool PHASE = false;
    __device__ __forceinline__ float phase_w() const { return 0.0f; }
    __device__ __forceinline__ f32x2 unscaled2_ph(f32x2 tau, f32x2, f32x2) const { return unscaled2(tau); }
    __device__ __forceinline__ void accumulate2_ph(f32x2 tau, f32x2, f32x2, f32x2 coeff, f32x2 *sums2) const {
        accumulate2(tau, coeff, sums2);
    }
    __device__ __forceinline__ void rescale_ph(f32x2 *) const {}
    __device__ __forceinline__ void finish_grad(const double *sums, float *grad) const {
        const double l = ell;
        // d kappa / d p0 = -s e tau^2 ; d p0 / d l = -1 / l^3
        grad[0] = (float)((double)scale * sums[0] / (l * l * l));
        grad[1] = (float)sums[1];
    }
};

template <>
struct KernelFn<KM_KERNEL_SPECTRAL> {
    static constexpr int P = 3;
    static constexpr int NSUMS = 3;
    float c0, w, scale, ell, f2;
    __device__ __forceinline__ void init(const float *theta, int64_t stride) {
        ell = theta[0];
        const float f = theta[stride];
        scale = theta[2 * stride];
        c0 = -(0.5f / (ell * ell)) * KM_LOG2E_F;
        w = 2.0f * KM_PI_F * f;
        f2 = 2.0f * f;  // the phase in units of pi: cos(pi * f2 * tau), as the reference evaluates it
    }
    __device__ __forceinline__ float unscaled(float tau) const {
        return ex2_approx(c0 * tau * tau) * cos_approx(w * tau);
    }
    // sums: [0] = sum coeff e cos tau^2, [1] = sum coeff e sin tau, [2] = sum coeff e cos
    __device__ __forceinline__ void accumulate(float tau, float coeff, float *sums) const {
        const float t2 = tau * tau;
        const float ph = w * tau;
        const float v = coeff * ex2_approx(c0 * t2);
        const float vc = v * cos_approx(ph);
        const float vs = v * sin_approx(ph);
        sums[0] = fmaf(vc, t2, sums[0]);
        sums[1] = fmaf(vs, tau, sums[1]);
        sums[2] += vc;
    }
    __device__ __forceinline__ void accumulate_precise(float tau, float coeff, float *sums) const {
        const float t2 = tau * tau;
        float sn, cs;
        sincospif(f2 * tau, &sn, &cs);  // exact argument reduction
        const float v = coeff * exp2f(c0 * t2);
        const float vc = v * cs;
        sums[0] = fmaf(vc, t2, sums[0]);
        sums[1] = fmaf(v * sn, tau, sums[1]);
        sums[2] += vc;
    }
    __device__ __forceinline__ void accumulate2(f32x2 tau, f32x2 coeff, f32x2 *sums2) const {
        const f32x2 t2 = mul2(tau, tau);
        const f32x2 ph = mul2(splat2(w), tau);
        const f32x2 v = mul2(coeff, ex2_approx2(mul2(splat2(c0), t2)));
        const f32x2 vc = mul2(v, cos_approx2(ph));
        const f32x2 vs = mul2(v, sin_approx2(ph));
        sums2[0] = fma2(vc, t2, sums2[0]);
        sums2[1] = fma2(vs, tau, sums2[1]);
        sums2[2] = add2(vc, sums2[2]);
    }
    __device__ __forceinline__ f32x2 unscaled2(f32x2 tau) const {
        return mul2(ex2_approx2(mul2(splat2(c0), mul2(tau, tau))), cos_approx2(mul2(splat2(w), tau)));
    }
    static constexpr bool PHASE = true;
    __device__ __forceinline__ float phase_w() const { return w; }
    __device__ __forceinline__ f32x2 unscaled2_ph(f32x2 tau, f32x2 cs, f32x2) const {
        return mul2(ex2_approx2(mul2(splat2(c0), mul2(tau, tau))), cs);
    }
    __device__ __forceinline__ void accumulate2_ph(f32x2 tau, f32x2 cs, f32x2 sn, f32x2 coeff, f32x2 *sums2) const {
        const f32x2 t2 = mul2(tau, tau);
        const f32x2 v = mul2(coeff, ex2_approx2(mul2(splat2(c0), t2)));
        const f32x2 vc = mul2(v, cs);
        const f32x2 vs = mul2(v, sn);
        sums2[0] = fma2(vc, t2, sums2[0]);
        sums2[1] = fma2(vs, tau, sums2[1]);
        sums2[2] = add2(vc, sums2[2]);
    }
    __device__ __forceinline__ void rescale_ph(f32x2 *) const {}
    __device__ __forceinline__ void finish_grad(const double *sums, float *grad) const {
        const double l = ell;
        const double pi = 3.14159265358979323846;
        grad[0] = (float)((double)scale * sums[0] / (l * l * l));
        // d kappa / d p1 = -pi s e sin(pi p1 tau) tau ; d p1 / d f = 2
        grad[1] = (float)(-2.0 * pi * (double)scale * sums[1]);
        grad[2] = (float)sums[2];
    }
};

template <>
struct KernelFn<KM_KERNEL_LOCALLY_PERIODIC> {
    static constexpr int P = 4;
    static constexpr int NSUMS = 4;
    float c0, c1, w, scale, ell, ell_per, period;
    __device__ __forceinline__ void init(const float *theta, int64_t stride) {
        ell = theta[0];
        ell_per = theta[stride];
        period = theta[2 * stride];
        scale = theta[3 * stride];
        c0 = -(0.5f / (ell * ell)) * KM_LOG2E_F;
        c1 = -(2.0f / ell_per) * KM_LOG2E_F;
        w = KM_PI_F / period;
    }
    __device__ __forceinline__ void accumulate_precise(float tau, float coeff, float *sums) const {
        float sn, cs;
        sincospif(tau / period, &sn, &cs);  // exact argument reduction
        const float t2 = tau * tau;
        const float sn2 = sn * sn;
        const float v = coeff * exp2f(fmaf(c0, t2, c1 * sn2));
        sums[0] = fmaf(v, t2, sums[0]);
        sums[1] = fmaf(v, sn2, sums[1]);
        sums[2] = fmaf(v * sn, cs * tau, sums[2]);
        sums[3] += v;
    }
    __device__ __forceinline__ float unscaled(float tau) const {
        const float sn = sin_approx(w * tau);
        return ex2_approx(fmaf(c0 * tau, tau, c1 * (sn * sn)));
    }
    // sums: [0] = sum v tau^2, [1] = sum v sin^2, [2] = sum v sin cos tau, [3] = sum v,
    //       v = coeff * e
    __device__ __forceinline__ void accumulate(float tau, float coeff, float *sums) const {
        const float ph = w * tau;
        const float sn = sin_approx(ph);
        const float cs = cos_approx(ph);
        const float t2 = tau * tau;
        const float sn2 = sn * sn;
        const float v = coeff * ex2_approx(fmaf(c0, t2, c1 * sn2));
        sums[0] = fmaf(v, t2, sums[0]);
        sums[1] = fmaf(v, sn2, sums[1]);
        sums[2] = fmaf(v * sn, cs * tau, sums[2]);
        sums[3] += v;
    }
    __device__ __forceinline__ void accumulate2(f32x2 tau, f32x2 coeff, f32x2 *sums2) const {
        const f32x2 ph = mul2(splat2(w), tau);
        const f32x2 sn = sin_approx2(ph);
        const f32x2 cs = cos_approx2(ph);
        const f32x2 t2 = mul2(tau, tau);
        const f32x2 sn2 = mul2(sn, sn);
        const f32x2 v = mul2(coeff, ex2_approx2(fma2(splat2(c0), t2, mul2(splat2(c1), sn2))));
        sums2[0] = fma2(v, t2, sums2[0]);
        sums2[1] = fma2(v, sn2, sums2[1]);
        sums2[2] = fma2(mul2(v, sn), mul2(cs, tau), sums2[2]);
        sums2[3] = add2(v, sums2[3]);
    }
    __device__ __forceinline__ f32x2 unscaled2(f32x2 tau) const {
        const f32x2 sn = sin_approx2(mul2(splat2(w), tau));
        return ex2_approx2(fma2(mul2(splat2(c0), tau), tau, mul2(splat2(c1), mul2(sn, sn))));
    }
    // with cs = cos(2 w tau), sn = sin(2 w tau): sin^2(w tau) = (1 - cs) / 2, sin cos = sn / 2
    static constexpr bool PHASE = true;
    __device__ __forceinline__ float phase_w() const { return 2.0f * w; }
    // (the halves are folded into constants: c1 sin^2 = (c1 / 2) q with q = 1 - cs; the sums [1] and
    // [2] are accumulated as sum v q and sum v sn tau and halved once by rescale_ph)
    __device__ __forceinline__ f32x2 unscaled2_ph(f32x2 tau, f32x2 cs, f32x2) const {
        const f32x2 q = sub2(splat2(1.0f), cs);
        return ex2_approx2(fma2(mul2(splat2(c0), tau), tau, mul2(splat2(0.5f * c1), q)));
    }
    __device__ __forceinline__ void accumulate2_ph(f32x2 tau, f32x2 cs, f32x2 sn, f32x2 coeff, f32x2 *sums2) const {
        const f32x2 t2 = mul2(tau, tau);
        const f32x2 q = sub2(splat2(1.0f), cs);
        const f32x2 v = mul2(coeff, ex2_approx2(fma2(splat2(c0), t2, mul2(splat2(0.5f * c1), q))));
        sums2[0] = fma2(v, t2, sums2[0]);
        sums2[1] = fma2(v, q, sums2[1]);
        sums2[2] = fma2(mul2(v, sn), tau, sums2[2]);
        sums2[3] = add2(v, sums2[3]);
    }
    __device__ __forceinline__ void rescale_ph(f32x2 *sums2) const {
        sums2[1] = mul2(splat2(0.5f), sums2[1]);
        sums2[2] = mul2(splat2(0.5f), sums2[2]);
    }
    __device__ __forceinline__ void finish_grad(const double *sums, float *grad) const {
        const double l = ell, lp = ell_per, pr = period, s = scale;
        const double pi = 3.14159265358979323846;
        grad[0] = (float)(s * sums[0] / (l * l * l));
        // d kappa / d p1 = -s e sin^2 ; d p1 / d l_per = -2 / l_per^2
        grad[1] = (float)(s * sums[1] * 2.0 / (lp * lp));
        // d kappa / d p2 = -2 pi s e p1 sin cos tau ; p1 = 2 / l_per ; d p2 / d period = -1 / period^2
        grad[2] = (float)(2.0 * pi * s * (2.0 / lp) * sums[2] / (pr * pr));
        grad[3] = (float)sums[3];
    }
};

// 4-byte / 16-byte asynchronous global -> shared copies (LDGSTS).
__device__ __forceinline__ void cp_async4(void *smem, const void *gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ int clamp_int(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// Columns of a band tile staged per pipeline stage.
constexpr int TILE_N = 128;

// Issue the asynchronous copies of one band tile: `cnt` values of x2 starting at column n0 into
// xs[0..cnt) and the matching rows of a (n, k) matrix, columns [k0, k0 + KB), into rs[j * KB + c]
// (columns past k are zero filled).  `vec`: rows may be copied 16 bytes at a time.
template <int KB, int THREADS>
__device__ __forceinline__ void stage_band_tile(float *rs, float *xs, const float *x2, int64_t x2_stride,
                                                const float *mat, int64_t mat_s0, int64_t mat_s1,
                                                int64_t k0, int64_t k, int n0, int cnt, bool vec,
                                                int tid) {
    for (int j = tid; j < cnt; j += THREADS) cp_async4(xs + j, x2 + (int64_t)(n0 + j) * x2_stride);
    if (vec) {
        constexpr int V = KB / 4 > 0 ? KB / 4 : 1;
        for (int q = tid; q < cnt * V; q += THREADS) {
            const int j = q / V, c4 = q % V;
            cp_async16(rs + j * KB + c4 * 4, mat + (int64_t)(n0 + j) * mat_s0 + k0 + c4 * 4);
        }
    } else {
        for (int q = tid; q < cnt * KB; q += THREADS) {
            const int j = q / KB, c = q % KB;
            if (k0 + c < k)
                cp_async4(rs + j * KB + c, mat + (int64_t)(n0 + j) * mat_s0 + (k0 + c) * mat_s1);
            else
                rs[j * KB + c] = 0.0f;
        }
    }
}

// Read KB staged values of column j (a broadcast read: every lane uses the same address).
template <int KB>
__device__ __forceinline__ void load_staged_row(const float *rs, int j, float (&rv)[KB]) {
    if constexpr (KB % 4 == 0) {
#pragma unroll
        for (int c4 = 0; c4 < KB / 4; c4++) {
            const float4 v = *reinterpret_cast<const float4 *>(rs + j * KB + c4 * 4);
            rv[c4 * 4 + 0] = v.x;
            rv[c4 * 4 + 1] = v.y;
            rv[c4 * 4 + 2] = v.z;
            rv[c4 * 4 + 3] = v.w;
        }
    } else if constexpr (KB == 2) {
        const float2 v = *reinterpret_cast<const float2 *>(rs + j * 2);
        rv[0] = v.x;
        rv[1] = v.y;
    } else {
#pragma unroll
        for (int c = 0; c < KB; c++) rv[c] = rs[j * KB + c];
    }
}

// Same read as packed pairs: rv2[c] = (row[2c], row[2c + 1]).  KB even.
template <int KB>
__device__ __forceinline__ void load_staged_row2(const float *rs, int j, f32x2 (&rv2)[KB / 2]) {
    if constexpr (KB % 4 == 0) {
#pragma unroll
        for (int c4 = 0; c4 < KB / 4; c4++) {
            const ulonglong2 v = *reinterpret_cast<const ulonglong2 *>(rs + j * KB + c4 * 4);
            rv2[c4 * 2 + 0] = v.x;
            rv2[c4 * 2 + 1] = v.y;
        }
    } else {
        static_assert(KB == 2, "packed rows need KB = 2 or a multiple of 4");
        rv2[0] = *reinterpret_cast<const f32x2 *>(rs + j * 2);
    }
}

// True when rows of a (.., rows, k) fp32 view can be copied 16 bytes at a time for every batch.
inline bool rows_vectorizable(const View<const float> &v, const Batch &b) {
    bool ok = v.s1 == 1 && v.s0 % 4 == 0 && ((uintptr_t)v.data % 16 == 0);
    for (int d = 0; d < b.ndim; d++) ok = ok && (v.bs[d] % 4 == 0);
    return ok;
}

}  // namespace km

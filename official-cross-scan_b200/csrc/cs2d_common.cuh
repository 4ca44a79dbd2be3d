// Shared device helpers for the 2D-CrossScan selective-scan kernels (sm_100a).
//
// Work decomposition used by both kernels
// ---------------------------------------
// There are batch*dim*dstate independent 2-D linear recurrences.  A thread owns
// a strip of STRIP (=8) consecutive columns of ONE row at a time, for a PAIR of
// states (n, n+1) of one channel; the pair is processed with packed fp32x2
// arithmetic (FFMA2/FMUL2/FADD2 of sm_100).  L = 2^k lanes of a warp cover one
// image row (L*8 >= ncols) and rows are walked sequentially, so the previous
// row lives in registers.  The recurrence along a row is a first-order linear
// scan: each lane folds its 8 columns, a log2(L)-step warp-shuffle scan
// combines the lane aggregates, and a second local pass applies the carry.
// Inputs are staged once per CTA (all channels of the tile and all states
// share them) in shared memory, 4 rows at a time.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cs2d.h"

namespace cs2d {

constexpr int STRIP = 8;     // columns per thread
constexpr int RB = 4;        // rows per staged block == checkpoint cadence
constexpr float LOG2E = 1.4426950408889634f;

// Device-side problem description (passed by value to the kernels).
struct Dev {
    int batch, dim, H, W, N, G, ddim;
    int io_dt, out_dt, softplus;
    int dpg;    // channels per B/C group
    int drep;   // channels per delta channel
    int NP;     // state pairs: ceil(N/2)
    int DC;     // channels per CTA
    int ntiles; // channel tiles per group
    int nck;    // checkpoint rows per image: ceil(H/RB)
    const void *u, *delta, *B, *C;
    const float *A, *D, *bias, *decay;
    int64_t u_bs, u_ds, u_hs, dl_bs, dl_ds, dl_hs, A_ds, A_ns;
    int64_t B_bs, B_gs, B_ns, B_hs, C_bs, C_gs, C_ns, C_hs;
    // forward: out; backward: dout
    void *out; int64_t o_bs, o_ds, o_hs;
    float2 *saved;
    // backward only
    void *du, *ddelta;
    float *dA, *dB, *dC, *dD, *dbias, *ddecay;
};

// ---- packed fp32x2 helpers -------------------------------------------------
__device__ __forceinline__ float2 f2(float x, float y) { return make_float2(x, y); }
__device__ __forceinline__ float2 bc(float x) { return make_float2(x, x); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 sub2(float2 a, float2 b) { return __ffma2_rn(b, bc(-1.f), a); }
__device__ __forceinline__ float2 neg2(float2 a) { return make_float2(-a.x, -a.y); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float2 ex2_2(float2 x) { return make_float2(ex2(x.x), ex2(x.y)); }

template <int WIDTH>
__device__ __forceinline__ float2 shfl_up2(float2 v, int off) {
    return make_float2(__shfl_up_sync(0xffffffffu, v.x, off, WIDTH), __shfl_up_sync(0xffffffffu, v.y, off, WIDTH));
}
template <int WIDTH>
__device__ __forceinline__ float2 shfl_down2(float2 v, int off) {
    return make_float2(__shfl_down_sync(0xffffffffu, v.x, off, WIDTH),
                       __shfl_down_sync(0xffffffffu, v.y, off, WIDTH));
}
template <int WIDTH>
__device__ __forceinline__ float2 shfl_xor2(float2 v, int off) {
    return make_float2(__shfl_xor_sync(0xffffffffu, v.x, off, WIDTH), __shfl_xor_sync(0xffffffffu, v.y, off, WIDTH));
}

// ---- dtype-generic element access (staging only; uniform branch) -----------
__device__ __forceinline__ float ld_elem(const void *p, int64_t i, int dt) {
    if (dt == CS2D_F32) return __ldg(reinterpret_cast<const float *>(p) + i);
    if (dt == CS2D_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
    return __half2float(reinterpret_cast<const __half *>(p)[i]);
}
__device__ __forceinline__ void st_elem(void *p, int64_t i, int dt, float v) {
    if (dt == CS2D_F32) reinterpret_cast<float *>(p)[i] = v;
    else if (dt == CS2D_BF16) reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16(v);
    else reinterpret_cast<__half *>(p)[i] = __float2half(v);
}

// softplus with the reference's threshold (fwd kernel :221-224).
__device__ __forceinline__ float softplus20(float x) { return x <= 20.f ? log1pf(__expf(x)) : x; }

// ---- row scans ---------------------------------------------------------------
// Exclusive carry for a forward (left-to-right) scan of h' = a*h + b across the
// L lanes of a row.  In: this lane's aggregate (P = prod a, H = local result with
// zero carry-in), optionally a second sequence S sharing the multipliers.
// Out: the value of the sequence just left of this lane's strip.
template <int L, bool TWO>
__device__ __forceinline__ void carry_fwd(int j, float2 P, float2 H, float2 S, float2 &cH, float2 &cS) {
    if constexpr (L == 1) {
        cH = bc(0.f); cS = bc(0.f);
    } else {
#pragma unroll
        for (int off = 1; off < L; off <<= 1) {
            float2 Pp = shfl_up2<L>(P, off);
            float2 Hp = shfl_up2<L>(H, off);
            float2 Sp = TWO ? shfl_up2<L>(S, off) : bc(0.f);
            if (j >= off) {
                H = fma2(P, Hp, H);
                if (TWO) S = fma2(P, Sp, S);
                P = mul2(P, Pp);
            }
        }
        cH = shfl_up2<L>(H, 1);
        cS = TWO ? shfl_up2<L>(S, 1) : bc(0.f);
        if (j == 0) { cH = bc(0.f); cS = bc(0.f); }
    }
}
// Same for a reverse (right-to-left) scan: carry = value just right of the strip.
template <int L, bool TWO>
__device__ __forceinline__ void carry_rev(int j, float2 P, float2 H, float2 S, float2 &cH, float2 &cS) {
    if constexpr (L == 1) {
        cH = bc(0.f); cS = bc(0.f);
    } else {
#pragma unroll
        for (int off = 1; off < L; off <<= 1) {
            float2 Pp = shfl_down2<L>(P, off);
            float2 Hp = shfl_down2<L>(H, off);
            float2 Sp = TWO ? shfl_down2<L>(S, off) : bc(0.f);
            if (j + off < L) {
                H = fma2(P, Hp, H);
                if (TWO) S = fma2(P, Sp, S);
                P = mul2(P, Pp);
            }
        }
        cH = shfl_down2<L>(H, 1);
        cS = TWO ? shfl_down2<L>(S, 1) : bc(0.f);
        if (j == L - 1) { cH = bc(0.f); cS = bc(0.f); }
    }
}

// One forward row for a strip: given dl (post-softplus delta), dlu = dl*u, B,
// the previous row (h_up, a_up) and the packed A*log2(e) (+ log2 decay), computes
// a, p and h (and the plain row scan s when WITH_S).
//   a = exp2(dl*A2 + lg2decay)                      (reference fwd kernel :245)
//   h = a*(h_left + h_up - 0.5*(a_up + a_left)*h_diag) + p      (:263-271)
//   s = a*s_left + p                                (:306-327)
template <int L, bool WITH_S>
__device__ __forceinline__ void row_forward(int j, const float (&dl)[STRIP], const float (&dlu)[STRIP],
                                            const float2 (&Bv)[STRIP], float2 A2, float2 lgd,
                                            const float2 (&h_up)[STRIP], const float2 (&a_up)[STRIP],
                                            float2 (&a)[STRIP], float2 (&p)[STRIP], float2 (&h)[STRIP],
                                            float2 (&s)[STRIP]) {
#pragma unroll
    for (int i = 0; i < STRIP; ++i) {
        a[i] = ex2_2(fma2(bc(dl[i]), A2, lgd));
        p[i] = mul2(Bv[i], bc(dlu[i]));
    }
    float2 hdiag0 = bc(0.f), aleft0 = bc(0.f);
    if constexpr (L > 1) {
        hdiag0 = shfl_up2<L>(h_up[STRIP - 1], 1);
        aleft0 = shfl_up2<L>(a[STRIP - 1], 1);
        if (j == 0) hdiag0 = bc(0.f);
    }
    float2 beta[STRIP];
    float2 P = bc(1.f), Ht = bc(0.f), St = bc(0.f);
#pragma unroll
    for (int i = 0; i < STRIP; ++i) {
        const float2 al = i ? a[i - 1] : aleft0;
        const float2 hd = i ? h_up[i - 1] : hdiag0;
        const float2 t = mul2(add2(a_up[i], al), hd);
        const float2 kappa = fma2(t, bc(-0.5f), h_up[i]);
        beta[i] = fma2(a[i], kappa, p[i]);
        Ht = fma2(a[i], Ht, beta[i]);
        if (WITH_S) St = fma2(a[i], St, p[i]);
        P = mul2(P, a[i]);
    }
    float2 ch, cs;
    carry_fwd<L, WITH_S>(j, P, Ht, St, ch, cs);
#pragma unroll
    for (int i = 0; i < STRIP; ++i) {
        ch = fma2(a[i], ch, beta[i]);
        h[i] = ch;
        if (WITH_S) { cs = fma2(a[i], cs, p[i]); s[i] = cs; }
    }
}

}  // namespace cs2d

// Streaming forward / backward kernels for dstate == 1 (sm_100a).
//
// With a single state per channel the operator moves 16 bytes per scanned element
// (16-bit I/O) and computes little: it is bandwidth-bound, and the shared-memory tiles
// of the general kernels (built to share u / delta between 8 state pairs) are pure
// overhead.  Here nothing is staged:
//   * a thread owns a strip of 8 consecutive columns of TWO channels of one group,
//     packed into the halves of fp32x2 registers (both channels read the same B / C);
//   * L = 2^k lanes cover a row, a warp holds 32/L channel pairs, a CTA four warps;
//   * a thread walks its channels' image row by row, loading its strip of u, delta
//     (dout), B, C straight from global memory into registers, one row ahead;
//   * the row recurrence is the lane scan of cs2d_common.cuh; the previous row lives in
//     registers for the whole image, so no state goes through memory in the forward
//     except the checkpoint (the h row at the end of every SRB rows) the backward
//     recomputes from;
//   * the backward walks the row blocks bottom-up: h of a block is recomputed from its
//     checkpoint into registers, the reverse sweep keeps the adjoint row in registers
//     from block to block (no scratch memory), dB / dC are summed over the warp's
//     channels with a shuffle reduce-scatter and added to global memory with one
//     vector atomic per thread and row.
// Math: see cs2d_fwd.cu / cs2d_bwd.cu (reference kernels
// include/cusoflex/selective_scan_fwd_kernel_oflex.cuh:214-338 and
// include/cusoflex/selective_scan_bwd_kernel_oflex.cuh:401-819), with N = 1.
#include "cs2d_common.cuh"

namespace cs2d {

constexpr int SNW = 4;               // warps per CTA
constexpr int STHREADS = SNW * 32;
constexpr int SRB = STREAM_RB;       // rows per checkpoint block
constexpr float LN2 = 0.6931471805599453f;

// ---- one strip (8 columns) of one row, as loaded: raw bits, converted when used ----------
template <bool F32>
struct Raw8 { uint32_t w[F32 ? 8 : 4]; };

// `row` = address of the strip's first column; nv = columns of the strip inside the image.
// mode 2: the 8 columns are one aligned 16-byte word (16-bit types) - one load; mode 1: two aligned
// words of 4 columns; mode 0: element by element.  In the vector modes the image width is a multiple
// of the word, so a word is either wholly inside the row or wholly outside: the load is predicated,
// never a divergent branch (an idle lane of a row would otherwise drag its warp through the scalar path).
template <bool F32>
__device__ __forceinline__ void ld_raw8(Raw8<F32> &r, const char *row, int mode, int nv) {
    if constexpr (!F32) {
        if (mode == 2) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (nv >= 8) v = __ldg(reinterpret_cast<const uint4 *>(row));
            r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w;
            return;
        }
    }
    if (mode) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if constexpr (F32) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (nv >= 4 * h + 4) v = __ldg(reinterpret_cast<const uint4 *>(row) + h);
                r.w[4 * h] = v.x; r.w[4 * h + 1] = v.y; r.w[4 * h + 2] = v.z; r.w[4 * h + 3] = v.w;
            } else {
                uint2 v = make_uint2(0u, 0u);
                if (nv >= 4 * h + 4) v = __ldg(reinterpret_cast<const uint2 *>(row) + h);
                r.w[2 * h] = v.x; r.w[2 * h + 1] = v.y;
            }
        }
        return;
    }
    if constexpr (F32) {
        const float *p = reinterpret_cast<const float *>(row);
#pragma unroll
        for (int k = 0; k < 8; ++k) r.w[k] = k < nv ? __float_as_uint(__ldg(p + k)) : 0u;
    } else {
        const uint16_t *p = reinterpret_cast<const uint16_t *>(row);
        uint32_t e[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) e[k] = k < nv ? (uint32_t)__ldg(p + k) : 0u;
#pragma unroll
        for (int k = 0; k < 4; ++k) r.w[k] = e[2 * k] | (e[2 * k + 1] << 16);
    }
}
// 8 results of one strip to a tensor of type dt (fp32 or 16-bit); modes as ld_raw8
__device__ __forceinline__ void st_row8(void *base, int64_t off, int dt, int mode, int nv, const float (&v)[STRIP]) {
    if (nv <= 0) return;
    if (dt != CS2D_F32 && mode == 2) {
        uint4 raw;
        if (dt == CS2D_BF16) {
            *reinterpret_cast<__nv_bfloat162 *>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
            *reinterpret_cast<__nv_bfloat162 *>(&raw.y) = __floats2bfloat162_rn(v[2], v[3]);
            *reinterpret_cast<__nv_bfloat162 *>(&raw.z) = __floats2bfloat162_rn(v[4], v[5]);
            *reinterpret_cast<__nv_bfloat162 *>(&raw.w) = __floats2bfloat162_rn(v[6], v[7]);
        } else {
            *reinterpret_cast<__half2 *>(&raw.x) = __floats2half2_rn(v[0], v[1]);
            *reinterpret_cast<__half2 *>(&raw.y) = __floats2half2_rn(v[2], v[3]);
            *reinterpret_cast<__half2 *>(&raw.z) = __floats2half2_rn(v[4], v[5]);
            *reinterpret_cast<__half2 *>(&raw.w) = __floats2half2_rn(v[6], v[7]);
        }
        *reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(base) + off) = raw;
        return;
    }
    st4(base, off, dt, mode != 0, nv, make_float4(v[0], v[1], v[2], v[3]));
    st4(base, off + 4, dt, mode != 0, nv - 4, make_float4(v[4], v[5], v[6], v[7]));
}
template <bool F32>
__device__ __forceinline__ void cvt8(const Raw8<F32> &r, int dt, float (&v)[STRIP]) {
    if constexpr (F32) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r.w[i]);
    } else if (dt == CS2D_BF16) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(r.w[i] << 16);
            v[2 * i + 1] = __uint_as_float(r.w[i] & 0xffff0000u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&r.w[i]));
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
}

__device__ __forceinline__ float lg2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// dl = softplus(x) with the reference's threshold, sig = d dl / dx.  16-bit I/O (FAST) uses the
// two special-function instructions directly (absolute error ~1e-7, far inside the 16-bit
// tolerance); fp32 I/O keeps log1pf.
template <bool FAST>
__device__ __forceinline__ void softplus_sig(float x, int softplus, float &dl, float &sig) {
    dl = x; sig = 1.f;
    if (softplus && x <= 20.f) {
        if constexpr (FAST) {
            const float t = ex2(x * LOG2E), u = 1.f + t;
            dl = lg2(u) * LN2;
            sig = __fdividef(t, u);
        } else {
            const float t = __expf(x);
            sig = __fdividef(t, 1.f + t);
            dl = log1pf(t);
        }
    }
}

// One forward row of a strip given a and p: h (and the plain row scan s when WITH_S).
//   h = a*(h_left + h_up - 0.5*(a_up + a_left)*h_diag) + p ;  s = a*s_left + p
template <int L, bool WITH_S>
__device__ __forceinline__ void srow_fwd(int j, const float2 (&a)[STRIP], const float2 (&p)[STRIP],
                                         const float2 (&h_up)[STRIP], const float2 (&a_up)[STRIP],
                                         float2 (&h)[STRIP], float2 (&s)[STRIP]) {
    float2 hdiag0 = bc(0.f), aleft0 = bc(0.f);
    if constexpr (L > 1) {
        hdiag0 = shfl_up2<L>(h_up[STRIP - 1], 1);
        aleft0 = shfl_up2<L>(a[STRIP - 1], 1);
        hdiag0.x = j == 0 ? 0.f : hdiag0.x; hdiag0.y = j == 0 ? 0.f : hdiag0.y;
    }
    float2 beta[STRIP];
#pragma unroll
    for (int i = 0; i < STRIP; ++i) {
        const float2 al = i ? a[i - 1] : aleft0;
        const float2 hd = i ? h_up[i - 1] : hdiag0;
        const float2 kappa = fma2(mul2(add2(a_up[i], al), hd), bc(-0.5f), h_up[i]);
        beta[i] = fma2(a[i], kappa, p[i]);
    }
    constexpr int HS = STRIP / 2;
    float2 P0 = a[0], P1 = a[HS], H0 = beta[0], H1 = beta[HS], S0 = p[0], S1 = p[HS];
#pragma unroll
    for (int i = 1; i < HS; ++i) {
        H0 = fma2(a[i], H0, beta[i]);
        H1 = fma2(a[HS + i], H1, beta[HS + i]);
        if (WITH_S) { S0 = fma2(a[i], S0, p[i]); S1 = fma2(a[HS + i], S1, p[HS + i]); }
        P0 = mul2(P0, a[i]);
        P1 = mul2(P1, a[HS + i]);
    }
    float2 ch, cs, Pin;
    carry_fwd<L, WITH_S>(j, mul2(P0, P1), fma2(P1, H0, H1), WITH_S ? fma2(P1, S0, S1) : bc(0.f), ch, cs, Pin);
    float2 ch1 = fma2(P0, ch, H0), cs1 = WITH_S ? fma2(P0, cs, S0) : bc(0.f);
#pragma unroll
    for (int i = 0; i < HS; ++i) {
        ch = fma2(a[i], ch, beta[i]); h[i] = ch;
        ch1 = fma2(a[HS + i], ch1, beta[HS + i]); h[HS + i] = ch1;
        if (WITH_S) {
            cs = fma2(a[i], cs, p[i]); s[i] = cs;
            cs1 = fma2(a[HS + i], cs1, p[HS + i]); s[HS + i] = cs1;
        }
    }
}

// access mode of a tensor (see ld_raw8): bit set in Dev::vec8 -> 2, in Dev::vec -> 1, else 0
__device__ __forceinline__ int vmode(const Dev &P, int bit) { return (P.vec8 & bit) ? 2 : (P.vec & bit) ? 1 : 0; }

// Which channels, rows and columns a thread owns; shared by both kernels.
template <int L>
struct Who {
    static constexpr int CW = 32 / L, PC = SNW * CW, Wp = L * STRIP;
    int j, b, g, q, d0, d1, c0, nv;
    bool on0, on1;
    int64_t ck;   // float2 offset of this thread's strip in checkpoint row 0
    __device__ __forceinline__ Who(const Dev &P) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        j = lane & (L - 1);
        const int cl = lane / L, npairs = (P.dpg + 1) >> 1;
        const int tile = blockIdx.x % P.ntiles, bg = blockIdx.x / P.ntiles;
        g = bg % P.G; b = bg / P.G;
        q = tile * PC + warp * CW + cl;
        on0 = q < npairs; on1 = on0 && 2 * q + 1 < P.dpg;
        const int qc = min(q, npairs - 1);   // idle slots shadow a valid pair (their results are dropped)
        d0 = g * P.dpg + 2 * qc; d1 = min(d0 + 1, (g + 1) * P.dpg - 1);
        c0 = STRIP * j; nv = max(0, min(STRIP, P.W - c0));
        ck = ((((int64_t)b * P.G + g) * npairs + qc) * P.nck) * Wp + c0;
    }
};

template <int L, bool F32>
__global__ void __launch_bounds__(STHREADS, F32 ? 3 : 4) sfwd_kernel(const Dev P) {
    const Who<L> w(P);
    constexpr int Wp = Who<L>::Wp;
    const int j = w.j, H = P.H, nv = w.nv;
    const int es = F32 ? 4 : 2;
    const char *pu0 = reinterpret_cast<const char *>(P.u) + ((int64_t)w.b * P.u_bs + (int64_t)w.d0 * P.u_ds + w.c0) * es;
    const char *pu1 = reinterpret_cast<const char *>(P.u) + ((int64_t)w.b * P.u_bs + (int64_t)w.d1 * P.u_ds + w.c0) * es;
    const char *px0 = reinterpret_cast<const char *>(P.delta) + ((int64_t)w.b * P.dl_bs + (int64_t)(w.d0 / P.drep) * P.dl_ds + w.c0) * es;
    const char *px1 = reinterpret_cast<const char *>(P.delta) + ((int64_t)w.b * P.dl_bs + (int64_t)(w.d1 / P.drep) * P.dl_ds + w.c0) * es;
    const char *pB = reinterpret_cast<const char *>(P.B) + ((int64_t)w.b * P.B_bs + (int64_t)w.g * P.B_gs + w.c0) * es;
    const char *pC = reinterpret_cast<const char *>(P.C) + ((int64_t)w.b * P.C_bs + (int64_t)w.g * P.C_gs + w.c0) * es;
    const int64_t su = P.u_hs * es, sx = P.dl_hs * es, sB = P.B_hs * es, sC = P.C_hs * es;
    const int64_t o0 = (int64_t)w.b * P.o_bs + (int64_t)w.d0 * P.o_ds + w.c0, o1 = (int64_t)w.b * P.o_bs + (int64_t)w.d1 * P.o_ds + w.c0;
    const int vu = vmode(P, VEC_U), vx = vmode(P, VEC_DELTA), vB = vmode(P, VEC_B), vC = vmode(P, VEC_C), vo = vmode(P, VEC_OUT);
    const float2 A2 = mul2(f2(__ldg(P.A + (int64_t)w.d0 * P.A_ds), __ldg(P.A + (int64_t)w.d1 * P.A_ds)), bc(LOG2E));
    const float2 D2 = P.D ? f2(__ldg(P.D + w.d0), __ldg(P.D + w.d1)) : bc(0.f);
    const float2 bias = P.bias ? f2(__ldg(P.bias + w.d0 / P.drep), __ldg(P.bias + w.d1 / P.drep)) : bc(0.f);

    Raw8<F32> ru0, ru1, rx0, rx1, rB, rC;
    auto load = [&](int r) {
        ld_raw8<F32>(ru0, pu0 + r * su, vu, nv); ld_raw8<F32>(ru1, pu1 + r * su, vu, nv);
        ld_raw8<F32>(rx0, px0 + r * sx, vx, nv); ld_raw8<F32>(rx1, px1 + r * sx, vx, nv);
        ld_raw8<F32>(rB, pB + r * sB, vB, nv); ld_raw8<F32>(rC, pC + r * sC, vC, nv);
    };
    load(0);
    float2 h_up[STRIP], a_up[STRIP];
#pragma unroll
    for (int i = 0; i < STRIP; ++i) { h_up[i] = bc(0.f); a_up[i] = bc(0.f); }

    for (int r = 0; r < H; ++r) {
        float u0[STRIP], u1[STRIP], x0[STRIP], x1[STRIP], Bf[STRIP], Cf[STRIP];
        cvt8<F32>(ru0, P.io_dt, u0); cvt8<F32>(ru1, P.io_dt, u1);
        cvt8<F32>(rx0, P.io_dt, x0); cvt8<F32>(rx1, P.io_dt, x1);
        cvt8<F32>(rB, P.io_dt, Bf); cvt8<F32>(rC, P.io_dt, Cf);
        if (r + 1 < H) load(r + 1);   // in flight while this row computes
        float2 a[STRIP], p[STRIP], h[STRIP], s[STRIP];
#pragma unroll
        for (int i = 0; i < STRIP; ++i) {
            float d0v, d1v, unused;
            softplus_sig<!F32>(x0[i] + bias.x, P.softplus, d0v, unused);
            softplus_sig<!F32>(x1[i] + bias.y, P.softplus, d1v, unused);
            if (i >= nv) { d0v = 0.f; d1v = 0.f; }   // columns past the image: a = 1, p = 0
            const float2 dl = f2(d0v, d1v);
            a[i] = ex2_2(mul2(dl, A2));
            p[i] = mul2(bc(Bf[i]), mul2(dl, f2(u0[i], u1[i])));
        }
        srow_fwd<L, true>(j, a, p, h_up, a_up, h, s);
        float y0[STRIP], y1[STRIP];
#pragma unroll
        for (int i = 0; i < STRIP; ++i) {
            const float2 y = fma2(bc(Cf[i]), fma2(p[i], bc(0.25f), sub2(h[i], s[i])), mul2(D2, f2(u0[i], u1[i])));
            y0[i] = y.x; y1[i] = y.y;
            h_up[i] = h[i]; a_up[i] = a[i];
        }
        const int64_t ro = (int64_t)r * P.o_hs;
        if (w.on0) st_row8(P.out, o0 + ro, P.out_dt, vo, nv, y0);
        if (w.on1) st_row8(P.out, o1 + ro, P.out_dt, vo, nv, y1);
        // checkpoint: the last row of every block but the last one
        if (!P.ck_roll && w.on0 && (r + 1) % SRB == 0 && r + 1 < H) {   // every lane: the row is read back whole
            float4 *pk = reinterpret_cast<float4 *>(P.saved + w.ck + (int64_t)(r / SRB) * Wp);
#pragma unroll
            for (int k = 0; k < STRIP / 2; ++k) pk[k] = make_float4(h[2 * k].x, h[2 * k].y, h[2 * k + 1].x, h[2 * k + 1].y);
        }
    }
}

// Sum of 16 per-thread values (dB of the strip's 8 columns, then dC) over the CW = 32/L channel
// pairs of a warp, as a reduce-scatter: every step halves the values a lane keeps and adds the
// partner's copy of them, so a lane ends with 16/CW complete sums, which it adds to global memory.
template <int L>
__device__ __forceinline__ void add_dbc_rows(float (&v)[16], float *rowB, float *rowC, int c0, int W, bool vec,
                                             int lane) {
    constexpr int CW = 32 / L;
    int base = 0;
    if constexpr (CW >= 2) {
        const bool hi = lane & L;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float keep = hi ? v[i + 8] : v[i], send = hi ? v[i] : v[i + 8];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, L);
        }
        base += hi ? 8 : 0;
    }
    if constexpr (CW >= 4) {
        const bool hi = lane & (2 * L);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float keep = hi ? v[i + 4] : v[i], send = hi ? v[i] : v[i + 4];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2 * L);
        }
        base += hi ? 4 : 0;
    }
    if constexpr (CW >= 8) {
        const bool hi = lane & (4 * L);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float keep = hi ? v[i + 2] : v[i], send = hi ? v[i] : v[i + 2];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4 * L);
        }
        base += hi ? 2 : 0;
    }
    if constexpr (CW >= 16) {
        const bool hi = lane & (8 * L);
        const float keep = hi ? v[1] : v[0], send = hi ? v[0] : v[1];
        v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 8 * L);
        base += hi ? 1 : 0;
    }
    bool writer = true;
    if constexpr (CW >= 32) {   // one value left per lane pair: both get the sum, one writes
        v[0] += __shfl_xor_sync(0xffffffffu, v[0], 16);
        writer = !(lane & 16);
    }
    // this lane holds the sums of the original indices base .. base+CNT-1; index i is dB (i < 8) or
    // dC (i >= 8) of column c0 + (i & 7)
    constexpr int CNT = CW >= 16 ? 1 : 16 / CW;
    if constexpr (CNT >= 4) {
#pragma unroll
        for (int k = 0; k < CNT; k += 4) {
            const int idx = base + k, c = c0 + (idx & 7);
            float *dst = idx < 8 ? rowB : rowC;
            if (vec && c + 3 < W) {
                atomicAdd(reinterpret_cast<float4 *>(dst + c), make_float4(v[k], v[k + 1], v[k + 2], v[k + 3]));
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (c + e < W) atomicAdd(dst + c + e, v[k + e]);
            }
        }
    } else {
        const int c = c0 + (base & 7);
        float *dst = base < 8 ? rowB : rowC;
        if constexpr (CNT == 2) {
            if (vec && c + 1 < W) {
                atomicAdd(reinterpret_cast<float2 *>(dst + c), make_float2(v[0], v[1]));
            } else {
                if (c < W) atomicAdd(dst + c, v[0]);
                if (c + 1 < W) atomicAdd(dst + c + 1, v[1]);
            }
        } else {
            if (writer && c < W) atomicAdd(dst + c, v[0]);
        }
    }
}

// Thread-private rows parked in shared memory: row `k` of thread `tid` is four float4 (8 float2) at
// [(k*4 + q) * STHREADS + tid], so that a warp's accesses are consecutive 16-byte words.
constexpr int SB_ROWS = SRB + 3;   // h above the block, h of the block's rows, adjoint row m, its a
constexpr int SB_SMEM = SB_ROWS * 4 * STHREADS * 16;
__device__ __forceinline__ void park(float4 *sm, int k, const float2 (&v)[STRIP]) {
#pragma unroll
    for (int q = 0; q < 4; ++q) sm[(k * 4 + q) * STHREADS] = make_float4(v[2 * q].x, v[2 * q].y, v[2 * q + 1].x, v[2 * q + 1].y);
}
__device__ __forceinline__ void fetch(const float4 *sm, int k, float2 (&v)[STRIP]) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float4 t = sm[(k * 4 + q) * STHREADS];
        v[2 * q] = f2(t.x, t.y); v[2 * q + 1] = f2(t.z, t.w);
    }
}

// G32: dout is fp32 (always with fp32 inputs; with 16-bit inputs when the forward returned fp32).
template <int L, bool F32, bool G32>
__global__ void __launch_bounds__(STHREADS, 2) sbwd_kernel(const Dev P) {
    static_assert(G32 || !F32, "fp32 inputs come with an fp32 dout");
    extern __shared__ __align__(16) float4 sm_all[];
    float4 *sm = sm_all + threadIdx.x;
    constexpr int K_TOP = 0, K_ROW = 1, K_M = SRB + 1, K_A = SRB + 2;
    const Who<L> w(P);
    constexpr int Wp = Who<L>::Wp;
    const int j = w.j, H = P.H, W = P.W, nv = w.nv, lane = threadIdx.x & 31;
    const int es = F32 ? 4 : 2, eso = G32 ? 4 : 2;
    const char *pu0 = reinterpret_cast<const char *>(P.u) + ((int64_t)w.b * P.u_bs + (int64_t)w.d0 * P.u_ds + w.c0) * es;
    const char *pu1 = reinterpret_cast<const char *>(P.u) + ((int64_t)w.b * P.u_bs + (int64_t)w.d1 * P.u_ds + w.c0) * es;
    const char *px0 = reinterpret_cast<const char *>(P.delta) + ((int64_t)w.b * P.dl_bs + (int64_t)(w.d0 / P.drep) * P.dl_ds + w.c0) * es;
    const char *px1 = reinterpret_cast<const char *>(P.delta) + ((int64_t)w.b * P.dl_bs + (int64_t)(w.d1 / P.drep) * P.dl_ds + w.c0) * es;
    const char *pg0 = reinterpret_cast<const char *>(P.out) + ((int64_t)w.b * P.o_bs + (int64_t)w.d0 * P.o_ds + w.c0) * eso;
    const char *pg1 = reinterpret_cast<const char *>(P.out) + ((int64_t)w.b * P.o_bs + (int64_t)w.d1 * P.o_ds + w.c0) * eso;
    const char *pB = reinterpret_cast<const char *>(P.B) + ((int64_t)w.b * P.B_bs + (int64_t)w.g * P.B_gs + w.c0) * es;
    const char *pC = reinterpret_cast<const char *>(P.C) + ((int64_t)w.b * P.C_bs + (int64_t)w.g * P.C_gs + w.c0) * es;
    const int64_t su = P.u_hs * es, sx = P.dl_hs * es, sg = P.o_hs * eso, sB = P.B_hs * es, sC = P.C_hs * es;
    const int vu = vmode(P, VEC_U), vx = vmode(P, VEC_DELTA), vB = vmode(P, VEC_B), vC = vmode(P, VEC_C), vg = vmode(P, VEC_OUT),
              vd = vmode(P, VEC_DU);
    const float2 Araw = f2(__ldg(P.A + (int64_t)w.d0 * P.A_ds), __ldg(P.A + (int64_t)w.d1 * P.A_ds));
    const float2 A2 = mul2(Araw, bc(LOG2E));
    const float2 D2 = P.D ? f2(__ldg(P.D + w.d0), __ldg(P.D + w.d1)) : bc(0.f);
    const float2 bias = P.bias ? f2(__ldg(P.bias + w.d0 / P.drep), __ldg(P.bias + w.d1 / P.drep)) : bc(0.f);
    // du / ddelta rows of the two channels (contiguous (batch, dim, H, W) tensors of the input type)
    const int64_t q0 = ((int64_t)w.b * P.dim + w.d0) * H * W + w.c0, q1 = ((int64_t)w.b * P.dim + w.d1) * H * W + w.c0;
    float *dBp = P.dB + (((int64_t)w.b * P.G + w.g) * H) * W, *dCp = P.dC + (((int64_t)w.b * P.G + w.g) * H) * W;
    const bool vBC = (W % 4) == 0;   // dB / dC are dense fp32: rows start 16-byte aligned when W % 4 == 0
    // idle slots and the missing second channel of an odd group carry no gradient
    const float2 gmask = f2(w.on0 ? 1.f : 0.f, w.on1 ? 1.f : 0.f);

    {
        float2 z[STRIP];
#pragma unroll
        for (int i = 0; i < STRIP; ++i) z[i] = bc(0.f);
        park(sm, K_M, z); park(sm, K_A, z);   // below the image: no adjoint
    }
    float2 dA2 = bc(0.f), dD2 = bc(0.f), db2 = bc(0.f);

    // softplus'd delta of both channels for one raw row pair
    auto soft8 = [&](const Raw8<F32> &r0, const Raw8<F32> &r1, float2 (&dl)[STRIP], float2 (&sig)[STRIP]) {
        float x0[STRIP], x1[STRIP];
        cvt8<F32>(r0, P.io_dt, x0); cvt8<F32>(r1, P.io_dt, x1);
#pragma unroll
        for (int i = 0; i < STRIP; ++i) {
            float d0v, d1v, s0v, s1v;
            softplus_sig<!F32>(x0[i] + bias.x, P.softplus, d0v, s0v);
            softplus_sig<!F32>(x1[i] + bias.y, P.softplus, d1v, s1v);
            if (i >= nv) { d0v = 0.f; d1v = 0.f; s0v = 0.f; s1v = 0.f; }
            dl[i] = f2(d0v, d1v); sig[i] = f2(s0v, s1v);
        }
    };

    for (int blk = P.nck - 1; blk >= 0; --blk) {
        const int r0 = blk * SRB, nr = min(SRB, H - r0);
        {
            // ---- row above the block: h from the checkpoint, a from delta ----
            float2 a_up[STRIP], hprev[STRIP];
            if (r0 > 0) {
                Raw8<F32> rx0, rx1;
                ld_raw8<F32>(rx0, px0 + (r0 - 1) * sx, vx, nv); ld_raw8<F32>(rx1, px1 + (r0 - 1) * sx, vx, nv);
                const float4 *pk = reinterpret_cast<const float4 *>(P.saved + w.ck + (int64_t)(blk - 1) * Wp);
#pragma unroll
                for (int k = 0; k < STRIP / 2; ++k) {
                    const float4 v = __ldg(pk + k);
                    hprev[2 * k] = f2(v.x, v.y); hprev[2 * k + 1] = f2(v.z, v.w);
                }
                float2 dl[STRIP], sig[STRIP];
                soft8(rx0, rx1, dl, sig);
#pragma unroll
                for (int i = 0; i < STRIP; ++i) a_up[i] = ex2_2(mul2(dl[i], A2));
            } else {
#pragma unroll
                for (int i = 0; i < STRIP; ++i) { hprev[i] = bc(0.f); a_up[i] = bc(0.f); }
            }
            park(sm, K_TOP, hprev);
            // ---- recompute h of the block's rows ----
            Raw8<F32> ru0, ru1, rx0, rx1, rB;
            auto load = [&](int r) {
                ld_raw8<F32>(ru0, pu0 + r * su, vu, nv); ld_raw8<F32>(ru1, pu1 + r * su, vu, nv);
                ld_raw8<F32>(rx0, px0 + r * sx, vx, nv); ld_raw8<F32>(rx1, px1 + r * sx, vx, nv);
                ld_raw8<F32>(rB, pB + r * sB, vB, nv);
            };
            load(r0);
            for (int rr = 0; rr < nr; ++rr) {   // not unrolled: the rows live in shared memory, the code stays small
                {
                    float u0[STRIP], u1[STRIP], Bf[STRIP];
                    float2 dl[STRIP], sig[STRIP];
                    cvt8<F32>(ru0, P.io_dt, u0); cvt8<F32>(ru1, P.io_dt, u1); cvt8<F32>(rB, P.io_dt, Bf);
                    soft8(rx0, rx1, dl, sig);
                    if (rr + 1 < nr) load(r0 + rr + 1);
                    float2 a[STRIP], p[STRIP], h[STRIP], sdummy[STRIP];
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) {
                        a[i] = ex2_2(mul2(dl[i], A2));
                        p[i] = mul2(bc(Bf[i]), mul2(dl[i], f2(u0[i], u1[i])));
                    }
                    srow_fwd<L, false>(j, a, p, hprev, a_up, h, sdummy);
                    park(sm, K_ROW + rr, h);
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) { a_up[i] = a[i]; hprev[i] = h[i]; }
                }
            }
        }
        // ---- reverse sweep ----
        Raw8<F32> ru0, ru1, rx0, rx1, rB, rC;
        Raw8<G32> rg0, rg1;
        auto load = [&](int r) {
            ld_raw8<F32>(ru0, pu0 + r * su, vu, nv); ld_raw8<F32>(ru1, pu1 + r * su, vu, nv);
            ld_raw8<F32>(rx0, px0 + r * sx, vx, nv); ld_raw8<F32>(rx1, px1 + r * sx, vx, nv);
            ld_raw8<F32>(rB, pB + r * sB, vB, nv); ld_raw8<F32>(rC, pC + r * sC, vC, nv);
            ld_raw8<G32>(rg0, pg0 + r * sg, vg, nv); ld_raw8<G32>(rg1, pg1 + r * sg, vg, nv);
        };
        load(r0 + nr - 1);
        for (int rr = nr - 1; rr >= 0; --rr) {
            {
                const int r = r0 + rr;
                float Bf[STRIP], Cf[STRIP];
                float2 dl[STRIP], sig[STRIP], g2[STRIP], u2[STRIP];
                {
                    float t0[STRIP], t1[STRIP];
                    cvt8<F32>(ru0, P.io_dt, t0); cvt8<F32>(ru1, P.io_dt, t1);
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) u2[i] = f2(t0[i], t1[i]);
                    cvt8<G32>(rg0, P.out_dt, t0); cvt8<G32>(rg1, P.out_dt, t1);
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) g2[i] = mul2(f2(t0[i], t1[i]), gmask);
                }
                cvt8<F32>(rB, P.io_dt, Bf); cvt8<F32>(rC, P.io_dt, Cf);
                soft8(rx0, rx1, dl, sig);
                if (rr > 0) load(r - 1);
                float2 a[STRIP], p[STRIP], s[STRIP], gC[STRIP], dh[STRIP], ds[STRIP];
#pragma unroll
                for (int i = 0; i < STRIP; ++i) {
                    a[i] = ex2_2(mul2(dl[i], A2));
                    p[i] = mul2(bc(Bf[i]), mul2(dl[i], u2[i]));
                    gC[i] = mul2(bc(Cf[i]), g2[i]);
                }
                float2 a_r7 = bc(0.f);  // next lane's first column
                {
                    float2 m_dn[STRIP], a_dn[STRIP], bt[STRIP], mdr7 = bc(0.f);
                    fetch(sm, K_M, m_dn); fetch(sm, K_A, a_dn);
                    if constexpr (L > 1) {
                        a_r7 = shfl_down2<L>(a[0], 1);
                        mdr7 = shfl_down2<L>(m_dn[0], 1);
                        const bool last = j == L - 1;
                        a_r7.x = last ? 0.f : a_r7.x; a_r7.y = last ? 0.f : a_r7.y;
                        mdr7.x = last ? 0.f : mdr7.x; mdr7.y = last ? 0.f : mdr7.y;
                    }
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) {
                        const float2 ar = i < STRIP - 1 ? a[i + 1] : a_r7;
                        const float2 mdr = i < STRIP - 1 ? m_dn[i + 1] : mdr7;
                        bt[i] = fma2(mul2(add2(ar, a_dn[i]), mdr), bc(-0.5f), add2(gC[i], m_dn[i]));
                    }
                    // s forward, dh and ds reverse (multiplier of column c is a(c+1)), as half chains
                    constexpr int HS = STRIP / 2;
                    float2 Pf0 = a[0], Pf1 = a[HS], S0 = p[0], S1 = p[HS];
                    float2 Pr0 = a_r7, Pr1 = a[HS], H0 = bt[STRIP - 1], H1 = bt[HS - 1];
                    float2 D0 = neg2(gC[STRIP - 1]), D1 = neg2(gC[HS - 1]);
#pragma unroll
                    for (int k = 1; k < HS; ++k) {
                        S0 = fma2(a[k], S0, p[k]); Pf0 = mul2(Pf0, a[k]);
                        S1 = fma2(a[HS + k], S1, p[HS + k]); Pf1 = mul2(Pf1, a[HS + k]);
                        const float2 ar0 = a[STRIP - k], ar1 = a[HS - k];
                        H0 = fma2(ar0, H0, bt[STRIP - 1 - k]); D0 = fma2(ar0, D0, neg2(gC[STRIP - 1 - k]));
                        H1 = fma2(ar1, H1, bt[HS - 1 - k]); D1 = fma2(ar1, D1, neg2(gC[HS - 1 - k]));
                        Pr0 = mul2(Pr0, ar0); Pr1 = mul2(Pr1, ar1);
                    }
                    float2 cs, unused, cdh, cds, Pfin, Prin;
                    carry_fwd<L, false>(j, mul2(Pf0, Pf1), fma2(Pf1, S0, S1), bc(0.f), cs, unused, Pfin);
                    carry_rev<L, true>(j, mul2(Pr0, Pr1), fma2(Pr1, H0, H1), fma2(Pr1, D0, D1), cdh, cds, Prin);
                    float2 cs1 = fma2(Pf0, cs, S0);
                    float2 cdh1 = fma2(Pr0, cdh, H0), cds1 = fma2(Pr0, cds, D0);
#pragma unroll
                    for (int k = 0; k < HS; ++k) {
                        cs = fma2(a[k], cs, p[k]); s[k] = cs;
                        cs1 = fma2(a[HS + k], cs1, p[HS + k]); s[HS + k] = cs1;
                        const float2 ar0 = k ? a[STRIP - k] : a_r7, ar1 = a[HS - k];
                        cdh = fma2(ar0, cdh, bt[STRIP - 1 - k]); dh[STRIP - 1 - k] = cdh;
                        cds = fma2(ar0, cds, neg2(gC[STRIP - 1 - k])); ds[STRIP - 1 - k] = cds;
                        cdh1 = fma2(ar1, cdh1, bt[HS - 1 - k]); dh[HS - 1 - k] = cdh1;
                        cds1 = fma2(ar1, cds1, neg2(gC[HS - 1 - k])); ds[HS - 1 - k] = cds1;
                    }
                }
                float2 m[STRIP], m_dn[STRIP], hrow[STRIP], hup[STRIP];
#pragma unroll
                for (int i = 0; i < STRIP; ++i) m[i] = mul2(a[i], dh[i]);
                fetch(sm, K_M, m_dn); fetch(sm, K_ROW + rr, hrow); fetch(sm, rr > 0 ? K_ROW + rr - 1 : K_TOP, hup);
                float2 m_r7 = bc(0.f), h_l0 = bc(0.f);
                if constexpr (L > 1) {
                    m_r7 = shfl_down2<L>(m[0], 1);
                    h_l0 = shfl_up2<L>(hrow[STRIP - 1], 1);
                    m_r7.x = j == L - 1 ? 0.f : m_r7.x; m_r7.y = j == L - 1 ? 0.f : m_r7.y;
                    h_l0.x = j == 0 ? 0.f : h_l0.x; h_l0.y = j == 0 ? 0.f : h_l0.y;
                }
                park(sm, K_M, m); park(sm, K_A, a);   // the adjoint row for the row above
                float v[16], du0[STRIP], du1[STRIP], dd0[STRIP], dd1[STRIP];
#pragma unroll
                for (int i = 0; i < STRIP; ++i) {
                    const float2 hl = i ? hrow[i - 1] : h_l0;
                    const float2 mr = i < STRIP - 1 ? m[i + 1] : m_r7;
                    const float2 X = fma2(m_dn[i], hl, mul2(mr, hup[i]));
                    const float2 hm = sub2(hrow[i], p[i]);
                    const float2 sm_ = sub2(s[i], p[i]);
                    const float2 Gh = fma2(dh[i], hm, mul2(mul2(a[i], X), bc(-0.5f)));
                    const float2 G = fma2(ds[i], sm_, Gh);
                    const float2 eps = fma2(gC[i], bc(0.25f), add2(dh[i], ds[i]));
                    const float2 t1 = mul2(bc(Bf[i]), eps);
                    const float2 duv = fma2(dl[i], t1, mul2(D2, g2[i]));
                    const float2 ddv = mul2(fma2(u2[i], t1, mul2(Araw, G)), sig[i]);
                    du0[i] = duv.x; du1[i] = duv.y; dd0[i] = ddv.x; dd1[i] = ddv.y;
                    dA2 = fma2(dl[i], G, dA2);
                    dD2 = fma2(g2[i], u2[i], dD2);
                    db2 = add2(db2, ddv);
                    const float2 dBv = mul2(mul2(dl[i], u2[i]), eps);
                    const float2 yt = fma2(p[i], bc(0.25f), sub2(hrow[i], s[i]));
                    const float2 dCv = mul2(g2[i], yt);
                    v[i] = dBv.x + dBv.y;
                    v[8 + i] = dCv.x + dCv.y;
                }
                if (w.on0) {
                    st_row8(P.du, q0 + (int64_t)r * W, P.io_dt, vd, nv, du0);
                    st_row8(P.ddelta, q0 + (int64_t)r * W, P.io_dt, vd, nv, dd0);
                }
                if (w.on1) {
                    st_row8(P.du, q1 + (int64_t)r * W, P.io_dt, vd, nv, du1);
                    st_row8(P.ddelta, q1 + (int64_t)r * W, P.io_dt, vd, nv, dd1);
                }
                add_dbc_rows<L>(v, dBp + (int64_t)r * W, dCp + (int64_t)r * W, w.c0, W, vBC, lane);
            }
        }
    }
    // ---- per-channel parameter gradients: sum over the row's lanes, one atomic per channel ----
    if constexpr (L > 1) {
#pragma unroll
        for (int off = L / 2; off; off >>= 1) {
            dA2 = add2(dA2, shfl_xor2<L>(dA2, off));
            dD2 = add2(dD2, shfl_xor2<L>(dD2, off));
            db2 = add2(db2, shfl_xor2<L>(db2, off));
        }
    }
    if (j == 0) {
        if (w.on0) {
            atomicAdd(P.dA + w.d0, dA2.x);
            if (P.dD) atomicAdd(P.dD + w.d0, dD2.x);
            if (P.dbias) atomicAdd(P.dbias + w.d0, db2.x);
        }
        if (w.on1) {
            atomicAdd(P.dA + w.d1, dA2.y);
            if (P.dD) atomicAdd(P.dD + w.d1, dD2.y);
            if (P.dbias) atomicAdd(P.dbias + w.d1, db2.y);
        }
    }
}

template <int L>
static cudaError_t launch_sf(const Dev &P, int grid, cudaStream_t st) {
    if (P.io_dt == CS2D_F32) sfwd_kernel<L, true><<<grid, STHREADS, 0, st>>>(P);
    else sfwd_kernel<L, false><<<grid, STHREADS, 0, st>>>(P);
    return cudaGetLastError();
}
template <int L, bool F32, bool G32>
static cudaError_t launch_sb3(const Dev &P, int grid, cudaStream_t st) {
    static bool attr_done[64] = {};  // per template instance and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(sbwd_kernel<L, F32, G32>, cudaFuncAttributeMaxDynamicSharedMemorySize, SB_SMEM);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    sbwd_kernel<L, F32, G32><<<grid, STHREADS, SB_SMEM, st>>>(P);
    return cudaGetLastError();
}
template <int L>
static cudaError_t launch_sb(const Dev &P, int grid, cudaStream_t st) {
    if (P.io_dt == CS2D_F32) return launch_sb3<L, true, true>(P, grid, st);
    return P.out_dt == CS2D_F32 ? launch_sb3<L, false, true>(P, grid, st) : launch_sb3<L, false, false>(P, grid, st);
}

// channel pairs per CTA for a row of L lanes
int stream_pairs_per_cta(int L) { return SNW * (32 / L); }

cudaError_t launch_stream_fwd(const Dev &P, int L, int grid, cudaStream_t st) {
    switch (L) {
        case 1: return launch_sf<1>(P, grid, st);
        case 2: return launch_sf<2>(P, grid, st);
        case 4: return launch_sf<4>(P, grid, st);
        case 8: return launch_sf<8>(P, grid, st);
        case 16: return launch_sf<16>(P, grid, st);
        case 32: return launch_sf<32>(P, grid, st);
    }
    return cudaErrorInvalidValue;
}
cudaError_t launch_stream_bwd(const Dev &P, int L, int grid, cudaStream_t st) {
    switch (L) {
        case 1: return launch_sb<1>(P, grid, st);
        case 2: return launch_sb<2>(P, grid, st);
        case 4: return launch_sb<4>(P, grid, st);
        case 8: return launch_sb<8>(P, grid, st);
        case 16: return launch_sb<16>(P, grid, st);
        case 32: return launch_sb<32>(P, grid, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cs2d

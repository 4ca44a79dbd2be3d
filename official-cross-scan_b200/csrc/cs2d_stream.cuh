// Streaming forward / backward kernels for dstate == 1 (sm_100a): shared pieces.
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
//     except the checkpoint (the h row at the end of every STREAM_RB rows) the backward
//     recomputes from;
//   * the backward walks the row blocks bottom-up: h of a block is recomputed from its
//     checkpoint, the adjoint row is carried from block to block on chip (no scratch
//     memory), dB / dC are summed over the warp's channels with a shuffle reduce-scatter
//     and added to global memory with one vector reduction per thread and row.
// Every access that depends on the lane (a strip past the end of the row, an idle channel
// slot) is a predicated instruction, never a branch: a divergent branch drags the whole
// warp through both sides, and taken branches starve the instruction fetch.
// Math: see cs2d_fwd.cu / cs2d_bwd.cu (reference kernels
// include/cusoflex/selective_scan_fwd_kernel_oflex.cuh:214-338 and
// include/cusoflex/selective_scan_bwd_kernel_oflex.cuh:401-819), with N = 1.
#pragma once
#include "cs2d_common.cuh"

namespace cs2d {

constexpr int SNW = 4;               // warps per CTA
constexpr int STHREADS = SNW * 32;
constexpr int SRB = STREAM_RB;       // rows per checkpoint block
constexpr float LN2 = 0.6931471805599453f;
template <int V>
struct Int { static constexpr int value = V; };   // a compile-time integer passed as a function argument

// ---- predicated global access (inline PTX: the guard is a predicate, not a branch) ----------
__device__ __forceinline__ uint4 ldg16_if(const void *p, bool on) {
    uint4 v;
    asm("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;\n\t"
        "@p ld.global.nc.v4.b32 {%0,%1,%2,%3}, [%4];\n\t}"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p), "r"((int)on));
    return v;
}
__device__ __forceinline__ uint2 ldg8_if(const void *p, bool on) {
    uint2 v;
    asm("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %3, 0;\n\tmov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\t"
        "@p ld.global.nc.v2.b32 {%0,%1}, [%2];\n\t}"
        : "=r"(v.x), "=r"(v.y)
        : "l"(p), "r"((int)on));
    return v;
}
__device__ __forceinline__ void stg16_if(void *p, uint4 v, bool on) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t@p st.global.v4.b32 [%0], {%1,%2,%3,%4};\n\t}" ::"l"(p),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"((int)on)
                 : "memory");
}
__device__ __forceinline__ void stg8_if(void *p, uint2 v, bool on) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %3, 0;\n\t@p st.global.v2.b32 [%0], {%1,%2};\n\t}" ::"l"(p), "r"(v.x),
                 "r"(v.y), "r"((int)on)
                 : "memory");
}
__device__ __forceinline__ void stg4_if(void *p, uint32_t v, bool on) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p st.global.b32 [%0], %1;\n\t}" ::"l"(p), "r"(v), "r"((int)on)
                 : "memory");
}
__device__ __forceinline__ void red16_if(float *p, float a, float b, float c, float d, bool on) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t@p red.global.add.v4.f32 [%0], {%1,%2,%3,%4};\n\t}" ::"l"(p),
                 "f"(a), "f"(b), "f"(c), "f"(d), "r"((int)on)
                 : "memory");
}
__device__ __forceinline__ void red8_if(float *p, float a, float b, bool on) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %3, 0;\n\t@p red.global.add.v2.f32 [%0], {%1,%2};\n\t}" ::"l"(p), "f"(a),
                 "f"(b), "r"((int)on)
                 : "memory");
}
__device__ __forceinline__ void red4_if(float *p, float a, bool on) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p red.global.add.f32 [%0], %1;\n\t}" ::"l"(p), "f"(a),
                 "r"((int)on)
                 : "memory");
}

// ---- one strip (8 columns) of one row, as loaded: raw bits, converted when used ----------
// DT is the element type (CS2D_F32 / CS2D_F16 / CS2D_BF16), a template argument: no type branches.
template <int DT>
struct Raw8 { uint32_t w[DT == CS2D_F32 ? 8 : 4]; };

// `row` = address of the strip's first column; nv = columns of the strip inside the image.
// mode 2: the 8 columns are one aligned 16-byte word (16-bit types) - one load; mode 1: two aligned
// words of 4 columns; mode 0: element by element.  In the vector modes the image width is a multiple
// of the word, so a word is either wholly inside the row or wholly outside.  `on` switches the
// whole strip off (reads as zeros).
template <int DT>
__device__ __forceinline__ void ld_raw8(Raw8<DT> &r, const char *row, int mode, int nv, bool on = true) {
    if constexpr (DT != CS2D_F32) {
        if (mode == 2) {
            const uint4 v = ldg16_if(row, on && nv >= 8);
            r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w;
            return;
        }
    }
    if (mode) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if constexpr (DT == CS2D_F32) {
                const uint4 v = ldg16_if(row + 16 * h, on && nv >= 4 * h + 4);
                r.w[4 * h] = v.x; r.w[4 * h + 1] = v.y; r.w[4 * h + 2] = v.z; r.w[4 * h + 3] = v.w;
            } else {
                const uint2 v = ldg8_if(row + 8 * h, on && nv >= 4 * h + 4);
                r.w[2 * h] = v.x; r.w[2 * h + 1] = v.y;
            }
        }
        return;
    }
    if constexpr (DT == CS2D_F32) {
        const float *p = reinterpret_cast<const float *>(row);
#pragma unroll
        for (int k = 0; k < 8; ++k) r.w[k] = (on && k < nv) ? __float_as_uint(__ldg(p + k)) : 0u;
    } else {
        const uint16_t *p = reinterpret_cast<const uint16_t *>(row);
        uint32_t e[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) e[k] = (on && k < nv) ? (uint32_t)__ldg(p + k) : 0u;
#pragma unroll
        for (int k = 0; k < 4; ++k) r.w[k] = e[2 * k] | (e[2 * k + 1] << 16);
    }
}
// ---- asynchronous staging of strips into thread-private shared-memory slots -------------------
// A slot is one 16-byte word per thread (two for fp32: 8 columns are 32 bytes), laid out
// [..][word][thread] so that a warp's accesses are consecutive words.  Each thread copies, waits for
// (cp.async.wait_group) and reads only its own slots, so no barrier is involved.  A strip that is
// switched off, or past the end of the row, is zero-filled (source size 0).
__device__ __forceinline__ void cp16(uint32_t dst, const void *src, bool on) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(on ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp8(uint32_t dst, const void *src, bool on) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(on ? 8 : 0) : "memory");
}
__device__ __forceinline__ void cp4(uint32_t dst, const void *src, bool on) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(on ? 4 : 0) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int DT>
__host__ __device__ constexpr int slot_words() { return DT == CS2D_F32 ? 2 : 1; }
// `slot` points at this thread's first word of the slot; further words follow STHREADS words later
template <int DT, int M>
__device__ __forceinline__ void cp_raw8(uint4 *slot, const char *row, int nv, bool on = true) {
    const uint32_t dst = smem_addr(slot);
    if constexpr (DT == CS2D_F32 && (M == 1 || M == 2)) {   // 16-byte words (mode 3 is handled below)
        cp16(dst, row, on && nv >= 4);
        cp16(dst + STHREADS * 16, row + 16, on && nv >= 8);
    } else if constexpr (DT != CS2D_F32 && M == 2) {
        cp16(dst, row, on && nv >= 8);
    } else if constexpr (DT != CS2D_F32 && M == 1) {
        cp8(dst, row, on && nv >= 4);
        cp8(dst + 8, row + 8, on && nv >= 8);
    } else if constexpr (M == 3) {   // 4-byte words: single fp32 elements, pairs of 16-bit ones (even row width)
        constexpr int EW = DT == CS2D_F32 ? 1 : 2;   // elements per word
#pragma unroll
        for (int k = 0; k < 8 / EW; ++k)
            cp4(dst + (k / 4) * STHREADS * 16 + (k % 4) * 4, row + 4 * k, on && nv >= EW * (k + 1));
    } else {
        Raw8<DT> r;   // element by element: loaded now, parked in the slot
        ld_raw8<DT>(r, row, 0, nv, on);
        slot[0] = make_uint4(r.w[0], r.w[1], r.w[2], r.w[3]);
        if constexpr (DT == CS2D_F32) slot[STHREADS] = make_uint4(r.w[4], r.w[5], r.w[6], r.w[7]);
    }
}
template <int DT>
__device__ __forceinline__ void lds_raw8(Raw8<DT> &r, const uint4 *slot) {
    const uint4 v = slot[0];
    r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w;
    if constexpr (DT == CS2D_F32) {
        const uint4 q = slot[STHREADS];
        r.w[4] = q.x; r.w[5] = q.y; r.w[6] = q.z; r.w[7] = q.w;
    }
}

template <int DT>
__device__ __forceinline__ void cvt8(const Raw8<DT> &r, float (&v)[STRIP]) {
    if constexpr (DT == CS2D_F32) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r.w[i]);
    } else if constexpr (DT == CS2D_BF16) {
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
// 8 results of one strip to a tensor of runtime type dt; modes as ld_raw8
template <int M>
__device__ __forceinline__ void st_row8(void *base, int64_t off, int dt, int nv, bool on, const float (&v)[STRIP]) {
    if constexpr (M == 3) {
        if (dt == CS2D_F32) {
            float *p = reinterpret_cast<float *>(base) + off;
#pragma unroll
            for (int k = 0; k < 8; ++k) stg4_if(p + k, __float_as_uint(v[k]), on && k < nv);
        } else {
            uint16_t *p = reinterpret_cast<uint16_t *>(base) + off;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t raw;
                if (dt == CS2D_BF16) *reinterpret_cast<__nv_bfloat162 *>(&raw) = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
                else *reinterpret_cast<__half2 *>(&raw) = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
                stg4_if(p + 2 * k, raw, on && nv >= 2 * k + 2);
            }
        }
    } else if constexpr (M == 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (on && k < nv) st_elem(base, off + k, dt, v[k]);
    } else if (dt == CS2D_F32) {
        float *p = reinterpret_cast<float *>(base) + off;
        stg16_if(p, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])),
                 on && nv >= 4);
        stg16_if(p + 4, make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7])),
                 on && nv >= 8);
    } else {
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
        uint16_t *p = reinterpret_cast<uint16_t *>(base) + off;
        if constexpr (M == 2) {
            stg16_if(p, raw, on && nv >= 8);
        } else {
            stg8_if(p, make_uint2(raw.x, raw.y), on && nv >= 4);
            stg8_if(p + 4, make_uint2(raw.z, raw.w), on && nv >= 8);
        }
    }
}

__device__ __forceinline__ float lg2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// (dl, sig) = (softplus(x), its derivative) for the two channels of a thread, with the reference's
// threshold: above 20 the result is x itself (fwd kernel :221-224, bwd kernel :785-806).  softplus(x) >
// x always and log(1 + e^20) < 20 + 1e-8, so max(log(1 + e^min(x,20)), x) is that rule without a
// select, and e^20 / (1 + e^20) rounds to 1.  16-bit I/O (FAST) evaluates exp and log with the
// special-function unit directly (absolute error ~1e-7, far inside the 16-bit tolerance); fp32 I/O
// keeps log1pf.
template <bool FAST, bool WITH_SIG>
__device__ __forceinline__ void softplus2(float2 x, float2 &dl, float2 &sig) {
    const float2 xc = f2(fminf(x.x, 20.f), fminf(x.y, 20.f));
    float2 t, l;
    if constexpr (FAST) {
        t = ex2_2(mul2(xc, bc(LOG2E)));
        const float2 u = add2(t, bc(1.f));
        l = mul2(f2(lg2(u.x), lg2(u.y)), bc(LN2));
        if (WITH_SIG) sig = mul2(t, f2(rcp(u.x), rcp(u.y)));
    } else {
        t = f2(__expf(xc.x), __expf(xc.y));
        l = f2(log1pf(t.x), log1pf(t.y));
        if (WITH_SIG) sig = f2(__fdividef(t.x, 1.f + t.x), __fdividef(t.y, 1.f + t.y));
    }
    dl = f2(fmaxf(l.x, x.x), fmaxf(l.y, x.y));
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

// access mode of the launch (see ld_raw8 / cp_raw8): every tensor allows 8-element words -> 2, 4-element words -> 1,
// 4-byte words -> 3, else 0 (element by element)
__device__ __forceinline__ int vmode(const Dev &P, int all) {
    return (P.vec8 & all) == all ? 2 : (P.vec & all) == all ? 1 : (P.vec2 & all) == all ? 3 : 0;
}

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

}  // namespace cs2d

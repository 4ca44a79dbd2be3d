// Streaming backward kernel for dstate == 1 (sm_100a); see cs2d_stream.cuh.
#include "cs2d_stream.cuh"

namespace cs2d {

// Sum of 16 per-thread values (dB of the strip's 8 columns, then dC) over the CW = 32/L channel
// pairs of a warp, as a reduce-scatter: every step halves the values a lane keeps and adds the
// partner's copy of them, so a lane ends with 16/CW complete sums, which it adds to global memory
// with one predicated vector reduction.
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
    // dC (i >= 8) of column c0 + (i & 7).  vec: the rows are 16-byte aligned and W % 4 == 0, so a
    // group of 4 (or 2) columns is wholly inside the row or wholly outside.
    constexpr int CNT = CW >= 16 ? 1 : 16 / CW;
    if constexpr (CNT >= 4) {
#pragma unroll
        for (int k = 0; k < CNT; k += 4) {
            const int idx = base + k, c = c0 + (idx & 7);
            float *dst = (idx < 8 ? rowB : rowC) + c;
            if (vec) {
                red16_if(dst, v[k], v[k + 1], v[k + 2], v[k + 3], c < W);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) red4_if(dst + e, v[k + e], c + e < W);
            }
        }
    } else {
        const int c = c0 + (base & 7);
        float *dst = (base < 8 ? rowB : rowC) + c;
        if constexpr (CNT == 2) {
            if (vec) {
                red8_if(dst, v[0], v[1], c < W);
            } else {
                red4_if(dst, v[0], c < W);
                red4_if(dst + 1, v[1], c + 1 < W);
            }
        } else {
            red4_if(dst, v[0], writer && c < W);
        }
    }
}

// Thread-private rows parked in shared memory: row `k` of thread `tid` is four float4 (8 float2) at
// [(k*4 + q) * STHREADS + tid], so that a warp's accesses are consecutive 16-byte words.
constexpr int SB_ROWS = SRB + 3;   // h above the block, h of the block's rows, adjoint row m, its a
constexpr int SB_PARK = SB_ROWS * 4 * STHREADS * 16;
// Staging ring: every row the thread is going to need - the row above a block (delta and the h
// checkpoint), the block's rows for the recompute (u, delta, B), the same rows bottom-up for the
// reverse sweep (u, delta, dout, B, C) - is copied asynchronously into one of BW_DEPTH slots,
// BW_DEPTH-1 items ahead of its use, in exactly the order of use.  Word offsets inside a slot:
// u0, u1, x0, x1, B, C (SW words each), g0, g1 (GW words each); the checkpoint row (4 words) takes
// the place of B.. in the item of the row above a block.
constexpr int BW_DEPTH = 3;
template <int DT, int GT>
__host__ __device__ constexpr int bw_slot_words() { return 6 * slot_words<DT>() + 2 * slot_words<GT>(); }
template <int DT, int GT>
__host__ __device__ constexpr int bw_smem() { return SB_PARK + BW_DEPTH * bw_slot_words<DT, GT>() * STHREADS * 16; }
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

// DT: type of u, delta, B, C, du, ddelta; G32: dout is fp32 (always with fp32 inputs; with 16-bit
// inputs when the forward returned fp32).
template <int L, int DT, bool G32>
__global__ void __launch_bounds__(STHREADS, DT == CS2D_F32 ? 1 : 2) sbwd_kernel(const Dev P) {
    static_assert(G32 || DT != CS2D_F32, "fp32 inputs come with an fp32 dout");
    extern __shared__ __align__(16) float4 sm_all[];
    float4 *sm = sm_all + threadIdx.x;
    constexpr int K_TOP = 0, K_ROW = 1, K_M = SRB + 1, K_A = SRB + 2;
    constexpr int GT = G32 ? CS2D_F32 : DT;
    constexpr int SW = slot_words<DT>(), GW = slot_words<GT>(), SLOTW = bw_slot_words<DT, GT>();
    constexpr int O_U0 = 0, O_U1 = SW, O_X0 = 2 * SW, O_X1 = 3 * SW, O_B = 4 * SW, O_C = 5 * SW, O_G0 = 6 * SW,
                  O_G1 = 6 * SW + GW, O_CK = 4 * SW;
    static_assert(O_CK + 4 <= SLOTW, "the checkpoint row fits behind the two delta strips");
    uint4 *ring = reinterpret_cast<uint4 *>(sm_all + SB_ROWS * 4 * STHREADS) + threadIdx.x;
    constexpr bool FAST = DT != CS2D_F32;
    const Who<L> w(P);
    constexpr int Wp = Who<L>::Wp;
    const int j = w.j, H = P.H, W = P.W, nv = w.nv, lane = threadIdx.x & 31;
    constexpr int es = DT == CS2D_F32 ? 4 : 2, eso = G32 ? 4 : 2;
    const char *pu0 = reinterpret_cast<const char *>(P.u) + ((int64_t)w.b * P.u_bs + (int64_t)w.d0 * P.u_ds + w.c0) * es;
    const char *pu1 = reinterpret_cast<const char *>(P.u) + ((int64_t)w.b * P.u_bs + (int64_t)w.d1 * P.u_ds + w.c0) * es;
    const char *px0 = reinterpret_cast<const char *>(P.delta) + ((int64_t)w.b * P.dl_bs + (int64_t)(w.d0 / P.drep) * P.dl_ds + w.c0) * es;
    const char *px1 = reinterpret_cast<const char *>(P.delta) + ((int64_t)w.b * P.dl_bs + (int64_t)(w.d1 / P.drep) * P.dl_ds + w.c0) * es;
    const char *pg0 = reinterpret_cast<const char *>(P.out) + ((int64_t)w.b * P.o_bs + (int64_t)w.d0 * P.o_ds + w.c0) * eso;
    const char *pg1 = reinterpret_cast<const char *>(P.out) + ((int64_t)w.b * P.o_bs + (int64_t)w.d1 * P.o_ds + w.c0) * eso;
    const char *pB = reinterpret_cast<const char *>(P.B) + ((int64_t)w.b * P.B_bs + (int64_t)w.g * P.B_gs + w.c0) * es;
    const char *pC = reinterpret_cast<const char *>(P.C) + ((int64_t)w.b * P.C_bs + (int64_t)w.g * P.C_gs + w.c0) * es;
    const int64_t su = P.u_hs * es, sx = P.dl_hs * es, sg = P.o_hs * eso, sB = P.B_hs * es, sC = P.C_hs * es;
    const int vm = vmode(P, VEC_U | VEC_DELTA | VEC_B | VEC_C | VEC_OUT | VEC_DU);   // one access mode for the launch
    const bool softplus = P.softplus != 0;
    const float2 Araw = f2(__ldg(P.A + (int64_t)w.d0 * P.A_ds), __ldg(P.A + (int64_t)w.d1 * P.A_ds));
    const float2 A2 = mul2(Araw, bc(LOG2E));
    const float2 D2 = P.D ? f2(__ldg(P.D + w.d0), __ldg(P.D + w.d1)) : bc(0.f);
    const float2 bias = P.bias ? f2(__ldg(P.bias + w.d0 / P.drep), __ldg(P.bias + w.d1 / P.drep)) : bc(0.f);
    // du / ddelta rows of the two channels (contiguous (batch, dim, H, W) tensors of the input type)
    const int64_t q0 = ((int64_t)w.b * P.dim + w.d0) * H * W + w.c0, q1 = ((int64_t)w.b * P.dim + w.d1) * H * W + w.c0;
    float *dBp = P.dB + (((int64_t)w.b * P.G + w.g) * H) * W, *dCp = P.dC + (((int64_t)w.b * P.G + w.g) * H) * W;
    const bool vBC = (W % 4) == 0;   // dB / dC are dense fp32: rows start 16-byte aligned when W % 4 == 0
    const float2 *ckp = P.saved + w.ck;

    {
        float2 z[STRIP];
#pragma unroll
        for (int i = 0; i < STRIP; ++i) z[i] = bc(0.f);
        park(sm, K_M, z); park(sm, K_A, z);   // below the image: no adjoint
    }
    float2 dA2 = bc(0.f), dD2 = bc(0.f), db2 = bc(0.f);

    // ---- producer side of the staging ring ----
    int pb = P.nck - 1, pp = 0, ps = 0;   // next item: block, position inside it (0 = row above, 1..nr recompute, then reverse), slot
    auto issue_item = [&](auto mode) {
        constexpr int M = decltype(mode)::value;
        const int r0p = pb * SRB, nrp = min(SRB, H - r0p);
        uint4 *s = ring + ps * SLOTW * STHREADS;
        if (pp == 0) {
            const bool top = r0p > 0;
            const int rt = max(r0p - 1, 0);
            cp_raw8<DT, M>(s + O_X0 * STHREADS, px0 + rt * sx, nv, top);
            cp_raw8<DT, M>(s + O_X1 * STHREADS, px1 + rt * sx, nv, top);
            const float2 *ck = ckp + (int64_t)max(pb - 1, 0) * Wp;
#pragma unroll
            for (int k = 0; k < 4; ++k) cp16(smem_addr(s + (O_CK + k) * STHREADS), ck + 2 * k, top);
        } else {
            const bool rev = pp > nrp;
            const int r = rev ? r0p + 2 * nrp - pp : r0p + pp - 1;
            cp_raw8<DT, M>(s + O_U0 * STHREADS, pu0 + r * su, nv); cp_raw8<DT, M>(s + O_U1 * STHREADS, pu1 + r * su, nv);
            cp_raw8<DT, M>(s + O_X0 * STHREADS, px0 + r * sx, nv); cp_raw8<DT, M>(s + O_X1 * STHREADS, px1 + r * sx, nv);
            cp_raw8<DT, M>(s + O_B * STHREADS, pB + r * sB, nv);
            if (rev) {
                cp_raw8<DT, M>(s + O_C * STHREADS, pC + r * sC, nv);
                // idle slots and the missing second channel of an odd group carry no gradient
                cp_raw8<GT, M>(s + O_G0 * STHREADS, pg0 + r * sg, nv, w.on0);
                cp_raw8<GT, M>(s + O_G1 * STHREADS, pg1 + r * sg, nv, w.on1);
            }
        }
        if (++pp > 2 * nrp) { pp = 0; --pb; }
    };
    auto issue_next = [&]() {
        if (pb >= 0) {   // one (uniform) branch on the access mode per item, not one per strip
            if (vm == 2) issue_item(Int<2>()); else if (vm == 1) issue_item(Int<1>()); else if (vm == 3) issue_item(Int<3>()); else issue_item(Int<0>());
        }
        cp_commit();   // an empty group once everything has been asked for: the wait below counts groups
        ps = ps + 1 == BW_DEPTH ? 0 : ps + 1;
    };
    // consumer side: the slot of the item that is due now
    int cs = 0;
    auto next_item = [&]() -> const uint4 * {
        issue_next();
        cp_wait<BW_DEPTH - 1>();
        const uint4 *s = ring + cs * SLOTW * STHREADS;
        cs = cs + 1 == BW_DEPTH ? 0 : cs + 1;
        return s;
    };
#pragma unroll
    for (int k = 0; k < BW_DEPTH - 1; ++k) issue_next();

    // softplus'd delta (and its derivative) of both channels for one raw row pair.  Columns past the
    // image come out as softplus(bias): harmless, because u, dout, B, C read as zeros there (no
    // input, no gradient) and whatever h holds there only flows further right.
    auto soft8 = [&](const Raw8<DT> &r0, const Raw8<DT> &r1, float2 (&dl)[STRIP], float2 (&sig)[STRIP]) {
        float x0[STRIP], x1[STRIP];
        cvt8<DT>(r0, x0); cvt8<DT>(r1, x1);
#pragma unroll
        for (int i = 0; i < STRIP; ++i) { dl[i] = add2(f2(x0[i], x1[i]), bias); sig[i] = bc(1.f); }
        if (softplus) {
#pragma unroll
            for (int i = 0; i < STRIP; ++i) softplus2<FAST, true>(dl[i], dl[i], sig[i]);
        }
    };

    for (int blk = P.nck - 1; blk >= 0; --blk) {
        const int r0 = blk * SRB, nr = min(SRB, H - r0);
        {
            // ---- row above the block: h from the checkpoint, a from delta ----
            float2 a_up[STRIP], hprev[STRIP];
            {
                const uint4 *it = next_item();
                Raw8<DT> rx0, rx1;
                lds_raw8<DT>(rx0, it + O_X0 * STHREADS); lds_raw8<DT>(rx1, it + O_X1 * STHREADS);
#pragma unroll
                for (int k = 0; k < STRIP / 2; ++k) {
                    const uint4 v = it[(O_CK + k) * STHREADS];
                    hprev[2 * k] = f2(__uint_as_float(v.x), __uint_as_float(v.y));
                    hprev[2 * k + 1] = f2(__uint_as_float(v.z), __uint_as_float(v.w));
                }
                float2 dl[STRIP], sig[STRIP];
                soft8(rx0, rx1, dl, sig);
                // above the first row h is zero, so the value of a there never matters
#pragma unroll
                for (int i = 0; i < STRIP; ++i) a_up[i] = ex2_2(mul2(dl[i], A2));
            }
            park(sm, K_TOP, hprev);
            // ---- recompute h of the block's rows ----
            for (int rr = 0; rr < nr; ++rr) {   // not unrolled: the rows live in shared memory, the code stays small
                float u0[STRIP], u1[STRIP], Bf[STRIP];
                float2 dl[STRIP], sig[STRIP];
                {
                    const uint4 *it = next_item();
                    Raw8<DT> q, q2;
                    lds_raw8<DT>(q, it + O_U0 * STHREADS); cvt8<DT>(q, u0);
                    lds_raw8<DT>(q, it + O_U1 * STHREADS); cvt8<DT>(q, u1);
                    lds_raw8<DT>(q, it + O_B * STHREADS); cvt8<DT>(q, Bf);
                    lds_raw8<DT>(q, it + O_X0 * STHREADS); lds_raw8<DT>(q2, it + O_X1 * STHREADS);
                    soft8(q, q2, dl, sig);
                }
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
        // ---- reverse sweep ----
        for (int rr = nr - 1; rr >= 0; --rr) {
            const int r = r0 + rr;
            float Bf[STRIP], Cf[STRIP];
            float2 dl[STRIP], sig[STRIP], g2[STRIP], u2[STRIP];
            {
                const uint4 *it = next_item();
                float t0[STRIP], t1[STRIP];
                Raw8<DT> q, q2;
                Raw8<GT> qg;
                lds_raw8<DT>(q, it + O_U0 * STHREADS); cvt8<DT>(q, t0);
                lds_raw8<DT>(q, it + O_U1 * STHREADS); cvt8<DT>(q, t1);
#pragma unroll
                for (int i = 0; i < STRIP; ++i) u2[i] = f2(t0[i], t1[i]);
                lds_raw8<GT>(qg, it + O_G0 * STHREADS); cvt8<GT>(qg, t0);
                lds_raw8<GT>(qg, it + O_G1 * STHREADS); cvt8<GT>(qg, t1);
#pragma unroll
                for (int i = 0; i < STRIP; ++i) g2[i] = f2(t0[i], t1[i]);
                lds_raw8<DT>(q, it + O_B * STHREADS); cvt8<DT>(q, Bf);
                lds_raw8<DT>(q, it + O_C * STHREADS); cvt8<DT>(q, Cf);
                lds_raw8<DT>(q, it + O_X0 * STHREADS); lds_raw8<DT>(q2, it + O_X1 * STHREADS);
                soft8(q, q2, dl, sig);
            }
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
            fetch(sm, K_M, m_dn); fetch(sm, K_ROW + rr, hrow); fetch(sm, K_ROW + rr - 1, hup);   // K_ROW - 1 == K_TOP
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
            auto store = [&](auto mode) {
                constexpr int M = decltype(mode)::value;
                st_row8<M>(P.du, q0 + (int64_t)r * W, DT, nv, w.on0, du0);
                st_row8<M>(P.ddelta, q0 + (int64_t)r * W, DT, nv, w.on0, dd0);
                st_row8<M>(P.du, q1 + (int64_t)r * W, DT, nv, w.on1, du1);
                st_row8<M>(P.ddelta, q1 + (int64_t)r * W, DT, nv, w.on1, dd1);
            };
            if (vm == 2) store(Int<2>()); else if (vm == 1) store(Int<1>()); else if (vm == 3) store(Int<3>()); else store(Int<0>());
            add_dbc_rows<L>(v, dBp + (int64_t)r * W, dCp + (int64_t)r * W, w.c0, W, vBC, lane);
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

template <int L, int DT, bool G32>
static cudaError_t launch_sb3(const Dev &P, int grid, cudaStream_t st) {
    static bool attr_done[64] = {};  // per template instance and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(sbwd_kernel<L, DT, G32>, cudaFuncAttributeMaxDynamicSharedMemorySize, bw_smem<DT, G32 ? CS2D_F32 : DT>());
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    sbwd_kernel<L, DT, G32><<<grid, STHREADS, bw_smem<DT, G32 ? CS2D_F32 : DT>(), st>>>(P);
    return cudaGetLastError();
}
template <int L>
static cudaError_t launch_sb(const Dev &P, int grid, cudaStream_t st) {
    const bool g32 = P.out_dt == CS2D_F32;
    switch (P.io_dt) {
        case CS2D_F32: return launch_sb3<L, CS2D_F32, true>(P, grid, st);
        case CS2D_F16: return g32 ? launch_sb3<L, CS2D_F16, true>(P, grid, st) : launch_sb3<L, CS2D_F16, false>(P, grid, st);
        default: return g32 ? launch_sb3<L, CS2D_BF16, true>(P, grid, st) : launch_sb3<L, CS2D_BF16, false>(P, grid, st);
    }
}

cudaError_t launch_stream_bwd(const Dev &P, int L, int grid, cudaStream_t st) {
    switch (L) {
#ifndef CS2D_STREAM_L8_ONLY
        case 1: return launch_sb<1>(P, grid, st);
        case 2: return launch_sb<2>(P, grid, st);
        case 4: return launch_sb<4>(P, grid, st);
        case 16: return launch_sb<16>(P, grid, st);
#endif
        case 8: return launch_sb<8>(P, grid, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cs2d

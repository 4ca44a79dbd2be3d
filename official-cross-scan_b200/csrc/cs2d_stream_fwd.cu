// Streaming forward kernel for dstate == 1 (sm_100a); see cs2d_stream.cuh.
#include "cs2d_stream.cuh"

namespace cs2d {

template <int L, int DT>
__global__ void __launch_bounds__(STHREADS, DT == CS2D_F32 ? 3 : 4) sfwd_kernel(const Dev P) {
    const Who<L> w(P);
    constexpr int Wp = Who<L>::Wp;
    constexpr bool FAST = DT != CS2D_F32;
    const int j = w.j, H = P.H, nv = w.nv;
    constexpr int es = DT == CS2D_F32 ? 4 : 2;
    const char *pu0 = reinterpret_cast<const char *>(P.u) + ((int64_t)w.b * P.u_bs + (int64_t)w.d0 * P.u_ds + w.c0) * es;
    const char *pu1 = reinterpret_cast<const char *>(P.u) + ((int64_t)w.b * P.u_bs + (int64_t)w.d1 * P.u_ds + w.c0) * es;
    const char *px0 = reinterpret_cast<const char *>(P.delta) + ((int64_t)w.b * P.dl_bs + (int64_t)(w.d0 / P.drep) * P.dl_ds + w.c0) * es;
    const char *px1 = reinterpret_cast<const char *>(P.delta) + ((int64_t)w.b * P.dl_bs + (int64_t)(w.d1 / P.drep) * P.dl_ds + w.c0) * es;
    const char *pB = reinterpret_cast<const char *>(P.B) + ((int64_t)w.b * P.B_bs + (int64_t)w.g * P.B_gs + w.c0) * es;
    const char *pC = reinterpret_cast<const char *>(P.C) + ((int64_t)w.b * P.C_bs + (int64_t)w.g * P.C_gs + w.c0) * es;
    const int64_t su = P.u_hs * es, sx = P.dl_hs * es, sB = P.B_hs * es, sC = P.C_hs * es;
    const int64_t o0 = (int64_t)w.b * P.o_bs + (int64_t)w.d0 * P.o_ds + w.c0, o1 = (int64_t)w.b * P.o_bs + (int64_t)w.d1 * P.o_ds + w.c0;
    const int64_t so = P.o_hs;
    const int vu = vmode(P, VEC_U), vx = vmode(P, VEC_DELTA), vB = vmode(P, VEC_B), vC = vmode(P, VEC_C), vo = vmode(P, VEC_OUT);
    const int out_dt = P.out_dt;
    const bool softplus = P.softplus != 0, keep = !P.ck_roll && w.on0;
    const float2 A2 = mul2(f2(__ldg(P.A + (int64_t)w.d0 * P.A_ds), __ldg(P.A + (int64_t)w.d1 * P.A_ds)), bc(LOG2E));
    const float2 D2 = P.D ? f2(__ldg(P.D + w.d0), __ldg(P.D + w.d1)) : bc(0.f);
    const float2 bias = P.bias ? f2(__ldg(P.bias + w.d0 / P.drep), __ldg(P.bias + w.d1 / P.drep)) : bc(0.f);
    float2 *ckp = P.saved + w.ck;

    Raw8<DT> ru0, ru1, rx0, rx1, rB, rC;
    auto load = [&](int r) {
        ld_raw8<DT>(ru0, pu0 + r * su, vu, nv); ld_raw8<DT>(ru1, pu1 + r * su, vu, nv);
        ld_raw8<DT>(rx0, px0 + r * sx, vx, nv); ld_raw8<DT>(rx1, px1 + r * sx, vx, nv);
        ld_raw8<DT>(rB, pB + r * sB, vB, nv); ld_raw8<DT>(rC, pC + r * sC, vC, nv);
    };
    load(0);
    float2 h_up[STRIP], a_up[STRIP];
#pragma unroll
    for (int i = 0; i < STRIP; ++i) { h_up[i] = bc(0.f); a_up[i] = bc(0.f); }

    for (int r = 0; r < H; ++r) {
        float u0[STRIP], u1[STRIP], x0[STRIP], x1[STRIP], Bf[STRIP], Cf[STRIP];
        cvt8<DT>(ru0, u0); cvt8<DT>(ru1, u1);
        cvt8<DT>(rx0, x0); cvt8<DT>(rx1, x1);
        cvt8<DT>(rB, Bf); cvt8<DT>(rC, Cf);
        load(min(r + 1, H - 1));   // in flight while this row computes (the last row is fetched twice)
        float2 a[STRIP], p[STRIP], h[STRIP], s[STRIP];
        // columns past the image read u = B = C = 0: p = 0 there, and what h and s hold there only ever
        // flows further right, never into the image
#pragma unroll
        for (int i = 0; i < STRIP; ++i) {
            float2 dl = add2(f2(x0[i], x1[i]), bias), unused;
            if (softplus) softplus2<FAST, false>(dl, dl, unused);
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
        st_row8(P.out, o0 + r * so, out_dt, vo, nv, w.on0, y0);
        st_row8(P.out, o1 + r * so, out_dt, vo, nv, w.on1, y1);
        // checkpoint: the last row of every block but the last one (every lane: the row is read back whole)
        if (keep && (r + 1) % SRB == 0 && r + 1 < H) {
            float4 *pk = reinterpret_cast<float4 *>(ckp + (int64_t)(r / SRB) * Wp);
#pragma unroll
            for (int k = 0; k < STRIP / 2; ++k) pk[k] = make_float4(h[2 * k].x, h[2 * k].y, h[2 * k + 1].x, h[2 * k + 1].y);
        }
    }
}

template <int L>
static cudaError_t launch_sf(const Dev &P, int grid, cudaStream_t st) {
    switch (P.io_dt) {
        case CS2D_F32: sfwd_kernel<L, CS2D_F32><<<grid, STHREADS, 0, st>>>(P); break;
        case CS2D_F16: sfwd_kernel<L, CS2D_F16><<<grid, STHREADS, 0, st>>>(P); break;
        default: sfwd_kernel<L, CS2D_BF16><<<grid, STHREADS, 0, st>>>(P); break;
    }
    return cudaGetLastError();
}

// channel pairs per CTA for a row of L lanes
int stream_pairs_per_cta(int L) { return SNW * (32 / L); }

cudaError_t launch_stream_fwd(const Dev &P, int L, int grid, cudaStream_t st) {
    switch (L) {
#ifndef CS2D_STREAM_L8_ONLY
        case 1: return launch_sf<1>(P, grid, st);
        case 2: return launch_sf<2>(P, grid, st);
        case 4: return launch_sf<4>(P, grid, st);
        case 16: return launch_sf<16>(P, grid, st);
#endif
        case 8: return launch_sf<8>(P, grid, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cs2d

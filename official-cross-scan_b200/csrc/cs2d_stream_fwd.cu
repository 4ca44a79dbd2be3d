// Streaming forward kernel for dstate == 1 (sm_100a); see cs2d_stream.cuh.
#include "cs2d_stream.cuh"

namespace cs2d {

constexpr int FW_DEPTH = 4;   // rows in the staging ring (a power of two)
template <int DT>
constexpr int fw_smem() { return FW_DEPTH * 6 * slot_words<DT>() * STHREADS * 16; }

template <int L, int DT>
__global__ void __launch_bounds__(STHREADS, DT == CS2D_F32 ? 2 : 4) sfwd_kernel(const Dev P) {
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
    const int vm = vmode(P, VEC_U | VEC_DELTA | VEC_B | VEC_C | VEC_OUT);   // one access mode for the launch
    const int out_dt = P.out_dt;
    const bool softplus = P.softplus != 0, keep = !P.ck_roll && w.on0;
    const float2 A2 = mul2(f2(__ldg(P.A + (int64_t)w.d0 * P.A_ds), __ldg(P.A + (int64_t)w.d1 * P.A_ds)), bc(LOG2E));
    const float2 D2 = P.D ? f2(__ldg(P.D + w.d0), __ldg(P.D + w.d1)) : bc(0.f);
    const float2 bias = P.bias ? f2(__ldg(P.bias + w.d0 / P.drep), __ldg(P.bias + w.d1 / P.drep)) : bc(0.f);
    float2 *ckp = P.saved + w.ck;

    // The strips of u, delta (two channels each), B and C of the next FW_DEPTH-1 rows are always in
    // flight into this thread's ring of shared-memory slots: enough bytes on the way to keep HBM busy
    // at 16 resident warps per SM, without holding registers while they travel.
    extern __shared__ __align__(16) uint4 ring_all[];
    constexpr int NT = 6, SW = slot_words<DT>();
    uint4 *ring = ring_all + threadIdx.x;
    auto slot = [&](int stage, int t) { return ring + ((stage * NT + t) * SW) * STHREADS; };
    auto issue_m = [&](int r, auto mode) {
        constexpr int M = decltype(mode)::value;
        const bool on = r < H;
        const int rc = min(r, H - 1), st = r & (FW_DEPTH - 1);
        cp_raw8<DT, M>(slot(st, 0), pu0 + rc * su, nv, on); cp_raw8<DT, M>(slot(st, 1), pu1 + rc * su, nv, on);
        cp_raw8<DT, M>(slot(st, 2), px0 + rc * sx, nv, on); cp_raw8<DT, M>(slot(st, 3), px1 + rc * sx, nv, on);
        cp_raw8<DT, M>(slot(st, 4), pB + rc * sB, nv, on); cp_raw8<DT, M>(slot(st, 5), pC + rc * sC, nv, on);
        cp_commit();
    };
    auto issue = [&](int r) {   // one (uniform) branch per row instead of one per strip
        if (vm == 2) issue_m(r, Int<2>()); else if (vm == 1) issue_m(r, Int<1>()); else if (vm == 3) issue_m(r, Int<3>()); else issue_m(r, Int<0>());
    };
#pragma unroll
    for (int k = 0; k < FW_DEPTH - 1; ++k) issue(k);
    float2 h_up[STRIP], a_up[STRIP];
#pragma unroll
    for (int i = 0; i < STRIP; ++i) { h_up[i] = bc(0.f); a_up[i] = bc(0.f); }

    for (int r = 0; r < H; ++r) {
        issue(r + FW_DEPTH - 1);
        cp_wait<FW_DEPTH - 1>();   // row r has landed
        float u0[STRIP], u1[STRIP], x0[STRIP], x1[STRIP], Bf[STRIP], Cf[STRIP];
        {
            const int st = r & (FW_DEPTH - 1);
            Raw8<DT> q;
            lds_raw8<DT>(q, slot(st, 0)); cvt8<DT>(q, u0);
            lds_raw8<DT>(q, slot(st, 1)); cvt8<DT>(q, u1);
            lds_raw8<DT>(q, slot(st, 2)); cvt8<DT>(q, x0);
            lds_raw8<DT>(q, slot(st, 3)); cvt8<DT>(q, x1);
            lds_raw8<DT>(q, slot(st, 4)); cvt8<DT>(q, Bf);
            lds_raw8<DT>(q, slot(st, 5)); cvt8<DT>(q, Cf);
        }
        float2 a[STRIP], p[STRIP], h[STRIP], s[STRIP];
        // columns past the image read u = B = C = 0: p = 0 there, and what h and s hold there only ever
        // flows further right, never into the image
        float2 dl[STRIP];
#pragma unroll
        for (int i = 0; i < STRIP; ++i) dl[i] = add2(f2(x0[i], x1[i]), bias);
        if (softplus) {
#pragma unroll
            for (int i = 0; i < STRIP; ++i) { float2 unused; softplus2<FAST, false>(dl[i], dl[i], unused); }
        }
#pragma unroll
        for (int i = 0; i < STRIP; ++i) {
            a[i] = ex2_2(mul2(dl[i], A2));
            p[i] = mul2(bc(Bf[i]), mul2(dl[i], f2(u0[i], u1[i])));
        }
        srow_fwd<L, true>(j, a, p, h_up, a_up, h, s);
        float y0[STRIP], y1[STRIP];
#pragma unroll
        for (int i = 0; i < STRIP; ++i) {
            const float2 y = fma2(bc(Cf[i]), fma2(p[i], bc(0.25f), sub2(h[i], s[i])), mul2(D2, f2(u0[i], u1[i])));
            y0[i] = y.x; y1[i] = y.y;
            h_up[i] = h[i]; a_up[i] = a[i];
        }
        if (vm == 2) {
            st_row8<2>(P.out, o0 + r * so, out_dt, nv, w.on0, y0); st_row8<2>(P.out, o1 + r * so, out_dt, nv, w.on1, y1);
        } else if (vm == 1) {
            st_row8<1>(P.out, o0 + r * so, out_dt, nv, w.on0, y0); st_row8<1>(P.out, o1 + r * so, out_dt, nv, w.on1, y1);
        } else if (vm == 3) {
            st_row8<3>(P.out, o0 + r * so, out_dt, nv, w.on0, y0); st_row8<3>(P.out, o1 + r * so, out_dt, nv, w.on1, y1);
        } else {
            st_row8<0>(P.out, o0 + r * so, out_dt, nv, w.on0, y0); st_row8<0>(P.out, o1 + r * so, out_dt, nv, w.on1, y1);
        }
        // checkpoint: the last row of every block but the last one (every lane: the row is read back whole)
        if (keep && (r + 1) % SRB == 0 && r + 1 < H) {
            float4 *pk = reinterpret_cast<float4 *>(ckp + (int64_t)(r / SRB) * Wp);
#pragma unroll
            for (int k = 0; k < STRIP / 2; ++k) pk[k] = make_float4(h[2 * k].x, h[2 * k].y, h[2 * k + 1].x, h[2 * k + 1].y);
        }
    }
}

template <int L, int DT>
static cudaError_t launch_sf2(const Dev &P, int grid, cudaStream_t st) {
    static bool attr_done[64] = {};  // per template instance and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(sfwd_kernel<L, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, fw_smem<DT>());
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    sfwd_kernel<L, DT><<<grid, STHREADS, fw_smem<DT>(), st>>>(P);
    return cudaGetLastError();
}
template <int L>
static cudaError_t launch_sf(const Dev &P, int grid, cudaStream_t st) {
    switch (P.io_dt) {
        case CS2D_F32: return launch_sf2<L, CS2D_F32>(P, grid, st);
        case CS2D_F16: return launch_sf2<L, CS2D_F16>(P, grid, st);
        default: return launch_sf2<L, CS2D_BF16>(P, grid, st);
    }
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

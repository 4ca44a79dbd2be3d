// Backward 2D-CrossScan selective scan (sm_100a).
//
// Replaces selective_scan_bwd_kernel of the reference
// (include/cusoflex/selective_scan_bwd_kernel_oflex.cuh:91-902).  With
// g = dout, m = a*dh, and rows/columns outside the image contributing zero:
//   dh(r,c) = g*C + m(r+1,c) + a(r,c+1)*dh(r,c+1)
//             - 0.5*(a(r,c+1) + a(r+1,c))*m(r+1,c+1)                 (:439-469)
//   ds(r,c) = a(r,c+1)*ds(r,c+1) - g*C                               (:707-724)
//   X       = m(r+1,c)*h(r,c-1) + m(r,c+1)*h(r-1,c)
//   G       = dh*(h-p) + ds*(s-p) - 0.5*a*X      [= a * dLoss/da at (r,c)]
//   eps     = dh + ds + 0.25*g*C
//   du      = D*g + dl*sum_n B*eps          ddl = u*sum_n B*eps + sum_n A*G
//   dA      = sum dl*G      dB = sum_d dl*u*eps      dC = sum_d g*(h - s + 0.25p)
// which is the reference's du/ddelta/dA/dB/dC (:494-595, :730-757) with the
// cross-pixel terms (:544-587) regrouped by the pixel whose delta they touch.
// ddelta = ddl * sigmoid(delta+bias) under softplus (:785-806).
//
// Rows are processed in blocks of RB from the bottom up.  For each block the
// state h is recomputed from the checkpoint row the forward saved, kept in
// registers, and consumed by the reverse sweep; the plain row scan s is
// recomputed per row.  Sums over states (du, ddl) and over channels (dB, dC)
// are formed in shared memory; dB/dC then go to global memory with one atomic
// add per element and CTA.
#include "cs2d_common.cuh"

namespace cs2d {

template <int L>
__global__ void __launch_bounds__(256) bwd_kernel(const Dev P) {
    constexpr int Wp = L * STRIP;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int DC = P.DC, NP = P.NP;
    const int n_in = DC * RB * Wp;
    const int n_bc = NP * RB * Wp;
    float *su = reinterpret_cast<float *>(smem_raw);  // [DC][RB][Wp]
    float *sg = su + n_in;                            // [DC][RB][Wp]  dout
    float *ssig = sg + n_in;                          // [DC][RB][Wp]  d softplus / dx
    float *sdu = ssig + n_in;                         // [DC][RB][Wp]  sum over states
    float *sddl = sdu + n_in;                         // [DC][RB][Wp]
    float *sdl = sddl + n_in;                         // [DC][RB+1][Wp] row 0 = row above block
    float2 *sB = reinterpret_cast<float2 *>(sdl + DC * (RB + 1) * Wp);  // [NP][RB][Wp]
    float2 *sC = sB + n_bc;
    float2 *sdB = sC + n_bc;                          // sums over the CTA's channels
    float2 *sdC = sdB + n_bc;
    float *sred = reinterpret_cast<float *>(sdC + n_bc);  // [DC][2]: dD, ddelta_bias

    const int tid = threadIdx.x;
    const int j = tid & (L - 1);
    const int q = tid / L;
    const int pp = q % NP;
    const int dc = q / NP;
    const int tile = blockIdx.x % P.ntiles;
    const int bg = blockIdx.x / P.ntiles;
    const int g_ = bg % P.G;
    const int b = bg / P.G;
    const int d0 = g_ * P.dpg + tile * DC;
    const int dvalid = min(DC, (g_ + 1) * P.dpg - d0);
    const int d = d0 + min(dc, dvalid - 1);
    const bool ch_ok = dc < dvalid;
    const int H = P.H, W = P.W, N = P.N;
    const int c0 = j * STRIP;
    const int n0 = 2 * pp, n1 = 2 * pp + 1;

    const float decay = P.decay ? __ldg(P.decay) : 1.f;
    const float2 lgd = bc(P.decay ? log2f(decay) : 0.f);
    const float2 Araw = f2(__ldg(P.A + d * P.A_ds + n0 * P.A_ns), n1 < N ? __ldg(P.A + d * P.A_ds + n1 * P.A_ns) : 0.f);
    const float2 A2 = mul2(Araw, bc(LOG2E));
    const bool want_decay = P.ddecay != nullptr;

    if (tid < DC * 2) sred[tid] = 0.f;

    float2 m_dn[STRIP], a_dn[STRIP];
#pragma unroll
    for (int i = 0; i < STRIP; ++i) { m_dn[i] = bc(0.f); a_dn[i] = bc(0.f); }
    float2 dAacc = bc(0.f), ddecay_acc = bc(0.f);

    const int r_last = ((H - 1) / RB) * RB;
    for (int r0 = r_last; r0 >= -RB; r0 -= RB) {
        const int nr = r0 >= 0 ? min(RB, H - r0) : 0;
        // ---- write out the block processed before (r0+RB), stage block r0 ----
        const int rp = r0 + RB;
        const int nrp = rp <= r_last ? min(RB, H - rp) : 0;
        for (int idx = tid; idx < n_in; idx += blockDim.x) {
            const int c = idx % Wp, rr = (idx / Wp) % RB, sdc = idx / (Wp * RB);
            const int sd = d0 + sdc;
            const bool okc = sdc < dvalid && c < W;
            if (nrp > 0) {
                float dDp = 0.f, dbp = 0.f;
                if (okc && rr < nrp) {
                    const float gv = sg[idx];
                    const float dux = (P.D ? __ldg(P.D + sd) * gv : 0.f) + sdu[idx];
                    const float dd = sddl[idx] * ssig[idx];
                    const int64_t o = (((int64_t)b * P.dim + sd) * H + (rp + rr)) * W + c;
                    st_elem(P.du, o, P.io_dt, dux);
                    st_elem(P.ddelta, o, P.io_dt, dd);
                    dDp = gv * su[idx];
                    dbp = dd;
                }
                // RB*Wp is a multiple of 32, so a warp never straddles two channels
#pragma unroll
                for (int off = 16; off; off >>= 1) {
                    dDp += __shfl_xor_sync(0xffffffffu, dDp, off);
                    dbp += __shfl_xor_sync(0xffffffffu, dbp, off);
                }
                if ((tid & 31) == 0) {
                    atomicAdd(sred + 2 * sdc, dDp);
                    atomicAdd(sred + 2 * sdc + 1, dbp);
                }
            }
            float uv = 0.f, dlv = 0.f, gv = 0.f, sig = 0.f;
            if (okc && rr < nr) {
                const int r = r0 + rr;
                uv = ld_elem(P.u, (int64_t)b * P.u_bs + (int64_t)sd * P.u_ds + (int64_t)r * P.u_hs + c, P.io_dt);
                gv = ld_elem(P.out, (int64_t)b * P.o_bs + (int64_t)sd * P.o_ds + (int64_t)r * P.o_hs + c, P.out_dt);
                const int sdd = sd / P.drep;
                float x = ld_elem(P.delta, (int64_t)b * P.dl_bs + (int64_t)sdd * P.dl_ds + (int64_t)r * P.dl_hs + c,
                                  P.io_dt);
                if (P.bias) x += __ldg(P.bias + sdd);
                dlv = x; sig = 1.f;
                if (P.softplus && x <= 20.f) { dlv = log1pf(__expf(x)); sig = 1.f / (1.f + __expf(-x)); }
            }
            su[idx] = uv; sg[idx] = gv; ssig[idx] = sig; sdu[idx] = 0.f; sddl[idx] = 0.f;
            sdl[(sdc * (RB + 1) + rr + 1) * Wp + c] = dlv;
        }
        if (nr > 0) {
            // delta of the row above the block (for a of the checkpoint row)
            for (int idx = tid; idx < DC * Wp; idx += blockDim.x) {
                const int c = idx % Wp, sdc = idx / Wp;
                const int sd = d0 + sdc;
                float dlv = 0.f;
                if (sdc < dvalid && c < W && r0 > 0) {
                    const int sdd = sd / P.drep;
                    float x = ld_elem(P.delta,
                                      (int64_t)b * P.dl_bs + (int64_t)sdd * P.dl_ds + (int64_t)(r0 - 1) * P.dl_hs + c,
                                      P.io_dt);
                    if (P.bias) x += __ldg(P.bias + sdd);
                    dlv = P.softplus ? softplus20(x) : x;
                }
                sdl[(sdc * (RB + 1)) * Wp + c] = dlv;
            }
        }
        for (int idx = tid; idx < n_bc; idx += blockDim.x) {
            const int c = idx % Wp, rr = (idx / Wp) % RB, sp = idx / (Wp * RB);
            if (nrp > 0 && c < W && rr < nrp) {
                const float2 vb = sdB[idx], vc = sdC[idx];
                const int64_t o = ((((int64_t)b * P.G + g_) * N + 2 * sp) * H + (rp + rr)) * W + c;
                atomicAdd(P.dB + o, vb.x);
                atomicAdd(P.dC + o, vc.x);
                if (2 * sp + 1 < N) {
                    atomicAdd(P.dB + o + (int64_t)H * W, vb.y);
                    atomicAdd(P.dC + o + (int64_t)H * W, vc.y);
                }
            }
            float2 bv = bc(0.f), cv = bc(0.f);
            if (c < W && rr < nr) {
                const int r = r0 + rr;
                const int64_t ob = (int64_t)b * P.B_bs + (int64_t)g_ * P.B_gs + (int64_t)r * P.B_hs + c;
                const int64_t oc = (int64_t)b * P.C_bs + (int64_t)g_ * P.C_gs + (int64_t)r * P.C_hs + c;
                bv.x = ld_elem(P.B, ob + (int64_t)(2 * sp) * P.B_ns, P.io_dt);
                cv.x = ld_elem(P.C, oc + (int64_t)(2 * sp) * P.C_ns, P.io_dt);
                if (2 * sp + 1 < N) {
                    bv.y = ld_elem(P.B, ob + (int64_t)(2 * sp + 1) * P.B_ns, P.io_dt);
                    cv.y = ld_elem(P.C, oc + (int64_t)(2 * sp + 1) * P.C_ns, P.io_dt);
                }
            }
            sB[idx] = bv; sC[idx] = cv; sdB[idx] = bc(0.f); sdC[idx] = bc(0.f);
        }
        __syncthreads();
        if (nr == 0) break;

        // ---- recompute h for the block from the checkpoint row ---------------
        float2 hs[RB + 1][STRIP];  // hs[0] = row above the block
        float2 a_up[STRIP];
        {
            const float4 *pd = reinterpret_cast<const float4 *>(sdl + (dc * (RB + 1)) * Wp + c0);
            const float4 e0 = pd[0], e1 = pd[1];
            const float dlt[STRIP] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
            if (r0 > 0 && ch_ok) {
                const float4 *ck = reinterpret_cast<const float4 *>(
                    P.saved + ((((int64_t)b * P.dim + d) * P.nck + (r0 / RB - 1)) * NP + pp) * Wp + c0);
#pragma unroll
                for (int k = 0; k < STRIP / 2; ++k) {
                    const float4 v = __ldg(ck + k);
                    hs[0][2 * k] = f2(v.x, v.y); hs[0][2 * k + 1] = f2(v.z, v.w);
                }
            } else {
#pragma unroll
                for (int i = 0; i < STRIP; ++i) hs[0][i] = bc(0.f);
            }
#pragma unroll
            for (int i = 0; i < STRIP; ++i) a_up[i] = r0 > 0 ? ex2_2(fma2(bc(dlt[i]), A2, lgd)) : bc(0.f);
        }
#pragma unroll
        for (int rr = 0; rr < RB; ++rr) {
            if (rr < nr) {
                float dl[STRIP], dlu[STRIP];
                float2 Bv[STRIP];
                const float4 *pu = reinterpret_cast<const float4 *>(su + (dc * RB + rr) * Wp + c0);
                const float4 *pd = reinterpret_cast<const float4 *>(sdl + (dc * (RB + 1) + rr + 1) * Wp + c0);
                const float4 u0 = pu[0], u1 = pu[1], e0 = pd[0], e1 = pd[1];
                dl[0] = e0.x; dl[1] = e0.y; dl[2] = e0.z; dl[3] = e0.w;
                dl[4] = e1.x; dl[5] = e1.y; dl[6] = e1.z; dl[7] = e1.w;
                dlu[0] = e0.x * u0.x; dlu[1] = e0.y * u0.y; dlu[2] = e0.z * u0.z; dlu[3] = e0.w * u0.w;
                dlu[4] = e1.x * u1.x; dlu[5] = e1.y * u1.y; dlu[6] = e1.z * u1.z; dlu[7] = e1.w * u1.w;
                const float4 *pb = reinterpret_cast<const float4 *>(sB + (pp * RB + rr) * Wp + c0);
#pragma unroll
                for (int k = 0; k < STRIP / 2; ++k) {
                    const float4 bq = pb[k];
                    Bv[2 * k] = f2(bq.x, bq.y); Bv[2 * k + 1] = f2(bq.z, bq.w);
                }
                float2 a[STRIP], p[STRIP], sdummy[STRIP];
                row_forward<L, false>(j, dl, dlu, Bv, A2, lgd, hs[rr], a_up, a, p, hs[rr + 1], sdummy);
#pragma unroll
                for (int i = 0; i < STRIP; ++i) a_up[i] = a[i];
            }
        }

        // ---- reverse sweep over the block --------------------------------------
#pragma unroll
        for (int rr = RB - 1; rr >= 0; --rr) {
            if (rr < nr) {
                float dl[STRIP], uu[STRIP], gg[STRIP];
                float2 Bv[STRIP], Cv[STRIP];
                {
                    const float4 *pu = reinterpret_cast<const float4 *>(su + (dc * RB + rr) * Wp + c0);
                    const float4 *pg = reinterpret_cast<const float4 *>(sg + (dc * RB + rr) * Wp + c0);
                    const float4 *pd = reinterpret_cast<const float4 *>(sdl + (dc * (RB + 1) + rr + 1) * Wp + c0);
                    const float4 u0 = pu[0], u1 = pu[1], e0 = pd[0], e1 = pd[1], g0 = pg[0], g1 = pg[1];
                    dl[0] = e0.x; dl[1] = e0.y; dl[2] = e0.z; dl[3] = e0.w;
                    dl[4] = e1.x; dl[5] = e1.y; dl[6] = e1.z; dl[7] = e1.w;
                    uu[0] = u0.x; uu[1] = u0.y; uu[2] = u0.z; uu[3] = u0.w;
                    uu[4] = u1.x; uu[5] = u1.y; uu[6] = u1.z; uu[7] = u1.w;
                    gg[0] = g0.x; gg[1] = g0.y; gg[2] = g0.z; gg[3] = g0.w;
                    gg[4] = g1.x; gg[5] = g1.y; gg[6] = g1.z; gg[7] = g1.w;
                    const float4 *pb = reinterpret_cast<const float4 *>(sB + (pp * RB + rr) * Wp + c0);
                    const float4 *pc = reinterpret_cast<const float4 *>(sC + (pp * RB + rr) * Wp + c0);
#pragma unroll
                    for (int k = 0; k < STRIP / 2; ++k) {
                        const float4 bq = pb[k], cq = pc[k];
                        Bv[2 * k] = f2(bq.x, bq.y); Bv[2 * k + 1] = f2(bq.z, bq.w);
                        Cv[2 * k] = f2(cq.x, cq.y); Cv[2 * k + 1] = f2(cq.z, cq.w);
                    }
                }
                const float2 (&hrow)[STRIP] = hs[rr + 1];
                const float2 (&hup)[STRIP] = hs[rr];
                float2 a[STRIP], p[STRIP], s[STRIP], gC[STRIP];
                // a, p and the plain row scan s (recomputed)
                {
                    float2 Pm = bc(1.f), St = bc(0.f);
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) {
                        a[i] = ex2_2(fma2(bc(dl[i]), A2, lgd));
                        p[i] = mul2(Bv[i], bc(dl[i] * uu[i]));
                        gC[i] = mul2(Cv[i], bc(gg[i]));
                        St = fma2(a[i], St, p[i]);
                        Pm = mul2(Pm, a[i]);
                    }
                    float2 cs, unused;
                    carry_fwd<L, false>(j, Pm, St, bc(0.f), cs, unused);
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) { cs = fma2(a[i], cs, p[i]); s[i] = cs; }
                }
                // neighbours to the right (next lane's first column)
                float2 a_r7 = bc(0.f), mdr7 = bc(0.f);
                if constexpr (L > 1) {
                    a_r7 = shfl_down2<L>(a[0], 1);
                    mdr7 = shfl_down2<L>(m_dn[0], 1);
                    if (j == L - 1) { a_r7 = bc(0.f); mdr7 = bc(0.f); }
                }
                // reverse scans for dh and ds (shared multipliers a(r,c+1))
                float2 bt[STRIP], dh[STRIP], ds[STRIP];
                {
                    float2 Pm = bc(1.f), Dh = bc(0.f), Ds = bc(0.f);
#pragma unroll
                    for (int i = STRIP - 1; i >= 0; --i) {
                        const float2 ar = i < STRIP - 1 ? a[i + 1] : a_r7;
                        const float2 mdr = i < STRIP - 1 ? m_dn[i + 1] : mdr7;
                        bt[i] = fma2(mul2(add2(ar, a_dn[i]), mdr), bc(-0.5f), add2(gC[i], m_dn[i]));
                        Dh = fma2(ar, Dh, bt[i]);
                        Ds = fma2(ar, Ds, neg2(gC[i]));
                        Pm = mul2(Pm, ar);
                    }
                    float2 cdh, cds;
                    carry_rev<L, true>(j, Pm, Dh, Ds, cdh, cds);
#pragma unroll
                    for (int i = STRIP - 1; i >= 0; --i) {
                        const float2 ar = i < STRIP - 1 ? a[i + 1] : a_r7;
                        cdh = fma2(ar, cdh, bt[i]); dh[i] = cdh;
                        cds = fma2(ar, cds, neg2(gC[i])); ds[i] = cds;
                    }
                }
                float2 m[STRIP];
#pragma unroll
                for (int i = 0; i < STRIP; ++i) m[i] = mul2(a[i], dh[i]);
                float2 m_r7 = bc(0.f), h_l0 = bc(0.f);
                if constexpr (L > 1) {
                    m_r7 = shfl_down2<L>(m[0], 1);
                    h_l0 = shfl_up2<L>(hrow[STRIP - 1], 1);
                    if (j == L - 1) m_r7 = bc(0.f);
                    if (j == 0) h_l0 = bc(0.f);
                }
                float *durow = sdu + (dc * RB + rr) * Wp + c0;
                float *ddrow = sddl + (dc * RB + rr) * Wp + c0;
                float2 *dBrow = sdB + (pp * RB + rr) * Wp + c0;
                float2 *dCrow = sdC + (pp * RB + rr) * Wp + c0;
#pragma unroll
                for (int i = 0; i < STRIP; ++i) {
                    const float2 hl = i ? hrow[i - 1] : h_l0;
                    const float2 mr = i < STRIP - 1 ? m[i + 1] : m_r7;
                    const float2 X = fma2(m_dn[i], hl, mul2(mr, hup[i]));
                    const float2 hm = sub2(hrow[i], p[i]);
                    const float2 sm = sub2(s[i], p[i]);
                    const float2 Gh = fma2(dh[i], hm, mul2(mul2(a[i], X), bc(-0.5f)));
                    const float2 G = fma2(ds[i], sm, Gh);
                    const float2 eps = fma2(gC[i], bc(0.25f), add2(dh[i], ds[i]));
                    const float2 t1 = mul2(Bv[i], eps);
                    const float2 t2 = mul2(Araw, G);
                    const float S1 = t1.x + t1.y;
                    atomicAdd(durow + i, dl[i] * S1);
                    atomicAdd(ddrow + i, fmaf(uu[i], S1, t2.x + t2.y));
                    dAacc = fma2(bc(dl[i]), G, dAacc);
                    if (want_decay) ddecay_acc = add2(ddecay_acc, Gh);
                    const float2 dBv = mul2(bc(dl[i] * uu[i]), eps);
                    const float2 dCv = mul2(bc(gg[i]), fma2(p[i], bc(0.25f), sub2(hrow[i], s[i])));
                    atomicAdd(&dBrow[i].x, dBv.x); atomicAdd(&dBrow[i].y, dBv.y);
                    atomicAdd(&dCrow[i].x, dCv.x); atomicAdd(&dCrow[i].y, dCv.y);
                }
#pragma unroll
                for (int i = 0; i < STRIP; ++i) { m_dn[i] = m[i]; a_dn[i] = a[i]; }
            }
        }
        __syncthreads();
    }

    // ---- per-channel parameter gradients ---------------------------------------
    if constexpr (L > 1) {
#pragma unroll
        for (int off = L / 2; off; off >>= 1) {
            dAacc = add2(dAacc, shfl_xor2<L>(dAacc, off));
            ddecay_acc = add2(ddecay_acc, shfl_xor2<L>(ddecay_acc, off));
        }
    }
    if (j == 0 && ch_ok) {
        atomicAdd(P.dA + (int64_t)d * N + n0, dAacc.x);
        if (n1 < N) atomicAdd(P.dA + (int64_t)d * N + n1, dAacc.y);
        if (want_decay) atomicAdd(P.ddecay, (ddecay_acc.x + (n1 < N ? ddecay_acc.y : 0.f)) / decay);
    }
    __syncthreads();
    if (tid < dvalid * 2) {
        const int sd = d0 + tid / 2;
        if ((tid & 1) == 0) { if (P.dD) atomicAdd(P.dD + sd, sred[tid]); }
        else if (P.dbias) atomicAdd(P.dbias + sd, sred[tid]);
    }
}

size_t bwd_smem_bytes(int L, int DC, int NP) {
    const int Wp = L * STRIP;
    return (size_t)(5 * DC * RB * Wp + DC * (RB + 1) * Wp + 2 * DC) * 4 + (size_t)(4 * NP * RB * Wp) * 8;
}

template <int L>
static cudaError_t launch(const Dev &P, int grid, int threads, size_t smem, cudaStream_t st) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(bwd_kernel<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    bwd_kernel<L><<<grid, threads, smem, st>>>(P);
    return cudaGetLastError();
}

cudaError_t launch_bwd(const Dev &P, int L, int grid, int threads, cudaStream_t st) {
    const size_t smem = bwd_smem_bytes(L, P.DC, P.NP);
    switch (L) {
        case 1: return launch<1>(P, grid, threads, smem, st);
        case 2: return launch<2>(P, grid, threads, smem, st);
        case 4: return launch<4>(P, grid, threads, smem, st);
        case 8: return launch<8>(P, grid, threads, smem, st);
        case 16: return launch<16>(P, grid, threads, smem, st);
        case 32: return launch<32>(P, grid, threads, smem, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cs2d

// Forward 2D-CrossScan selective scan (sm_100a).
//
// Replaces selective_scan_fwd_kernel of the reference
// (include/cusoflex/selective_scan_fwd_kernel_oflex.cuh:80-357):
//   dl = softplus(delta + bias);  a = exp(dl*A)*A_decay;  p = B*dl*u
//   h(r,c) = a*(h(r,c-1) + h(r-1,c) - 0.5*(a(r-1,c)+a(r,c-1))*h(r-1,c-1)) + p
//   s(r,c) = a*s(r,c-1) + p
//   y      = D*u + sum_n C_n*(h_n - s_n + 0.25*p_n)
// One CTA owns DC channels of one (batch, group); B and C are staged once for
// all of them.  Every RB-th row of h is written to the saved-state buffer as a
// checkpoint for the backward pass.
#include "cs2d_common.cuh"

namespace cs2d {

template <int L>
__global__ void __launch_bounds__(256) fwd_kernel(const Dev P) {
    constexpr int Wp = L * STRIP;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int DC = P.DC, NP = P.NP;
    float *su = reinterpret_cast<float *>(smem_raw);          // [DC][RB][Wp]
    float *sdl = su + DC * RB * Wp;                           // [DC][RB][Wp]
    float *sy = sdl + DC * RB * Wp;                           // [DC][RB][Wp]
    float2 *sB = reinterpret_cast<float2 *>(sy + DC * RB * Wp);  // [NP][RB][Wp]
    float2 *sC = sB + NP * RB * Wp;                              // [NP][RB][Wp]

    const int tid = threadIdx.x;
    const int j = tid & (L - 1);
    const int q = tid / L;
    const int pp = q % NP;
    const int dc = q / NP;
    const int tile = blockIdx.x % P.ntiles;
    const int bg = blockIdx.x / P.ntiles;
    const int g = bg % P.G;
    const int b = bg / P.G;
    const int d0 = g * P.dpg + tile * DC;
    const int dvalid = min(DC, (g + 1) * P.dpg - d0);
    const int d = d0 + min(dc, dvalid - 1);
    const bool ch_ok = dc < dvalid;
    const int H = P.H, W = P.W, N = P.N;
    const int c0 = j * STRIP;
    const int n0 = 2 * pp, n1 = 2 * pp + 1;

    const float decay = P.decay ? __ldg(P.decay) : 1.f;
    const float2 lgd = bc(P.decay ? log2f(decay) : 0.f);
    const float2 A2 = f2(__ldg(P.A + d * P.A_ds + n0 * P.A_ns) * LOG2E,
                         n1 < N ? __ldg(P.A + d * P.A_ds + n1 * P.A_ns) * LOG2E : 0.f);

    float2 h_up[STRIP], a_up[STRIP];
#pragma unroll
    for (int i = 0; i < STRIP; ++i) { h_up[i] = bc(0.f); a_up[i] = bc(0.f); }

    const int n_in = DC * RB * Wp;   // elements of the per-channel tiles
    const int n_bc = NP * RB * Wp;   // float2 elements of the B/C tiles

    for (int r0 = 0; r0 < H; r0 += RB) {
        const int nr = min(RB, H - r0);
        // ---- write out the previous block's y, then stage this block --------
        for (int idx = tid; idx < n_in; idx += blockDim.x) {
            const int c = idx % Wp, rr = (idx / Wp) % RB, sdc = idx / (Wp * RB);
            const int sd = d0 + sdc;
            const bool okc = sdc < dvalid && c < W;
            if (r0 > 0 && okc) {  // previous block always has RB rows
                const int64_t o = (int64_t)b * P.o_bs + (int64_t)sd * P.o_ds + (int64_t)(r0 - RB + rr) * P.o_hs + c;
                st_elem(P.out, o, P.out_dt, sy[idx]);
            }
            float uv = 0.f, dlv = 0.f, yv = 0.f;
            if (okc && rr < nr) {
                const int r = r0 + rr;
                uv = ld_elem(P.u, (int64_t)b * P.u_bs + (int64_t)sd * P.u_ds + (int64_t)r * P.u_hs + c, P.io_dt);
                const int sdd = sd / P.drep;
                float x = ld_elem(P.delta, (int64_t)b * P.dl_bs + (int64_t)sdd * P.dl_ds + (int64_t)r * P.dl_hs + c,
                                  P.io_dt);
                if (P.bias) x += __ldg(P.bias + sdd);
                dlv = P.softplus ? softplus20(x) : x;
                yv = P.D ? __ldg(P.D + sd) * uv : 0.f;
            }
            su[idx] = uv; sdl[idx] = dlv; sy[idx] = yv;
        }
        for (int idx = tid; idx < n_bc; idx += blockDim.x) {
            const int c = idx % Wp, rr = (idx / Wp) % RB, sp = idx / (Wp * RB);
            float2 bv = bc(0.f), cv = bc(0.f);
            if (c < W && rr < nr) {
                const int r = r0 + rr;
                const int64_t ob = (int64_t)b * P.B_bs + (int64_t)g * P.B_gs + (int64_t)r * P.B_hs + c;
                const int64_t oc = (int64_t)b * P.C_bs + (int64_t)g * P.C_gs + (int64_t)r * P.C_hs + c;
                bv.x = ld_elem(P.B, ob + (int64_t)(2 * sp) * P.B_ns, P.io_dt);
                cv.x = ld_elem(P.C, oc + (int64_t)(2 * sp) * P.C_ns, P.io_dt);
                if (2 * sp + 1 < N) {
                    bv.y = ld_elem(P.B, ob + (int64_t)(2 * sp + 1) * P.B_ns, P.io_dt);
                    cv.y = ld_elem(P.C, oc + (int64_t)(2 * sp + 1) * P.C_ns, P.io_dt);
                }
            }
            sB[idx] = bv; sC[idx] = cv;
        }
        __syncthreads();

        // ---- scan the rows of this block ------------------------------------
        for (int rr = 0; rr < nr; ++rr) {
            float dl[STRIP], dlu[STRIP];
            float2 Bv[STRIP], Cv[STRIP];
            {
                const float4 *pu = reinterpret_cast<const float4 *>(su + (dc * RB + rr) * Wp + c0);
                const float4 *pd = reinterpret_cast<const float4 *>(sdl + (dc * RB + rr) * Wp + c0);
                const float4 u0 = pu[0], u1 = pu[1], e0 = pd[0], e1 = pd[1];
                dl[0] = e0.x; dl[1] = e0.y; dl[2] = e0.z; dl[3] = e0.w;
                dl[4] = e1.x; dl[5] = e1.y; dl[6] = e1.z; dl[7] = e1.w;
                dlu[0] = e0.x * u0.x; dlu[1] = e0.y * u0.y; dlu[2] = e0.z * u0.z; dlu[3] = e0.w * u0.w;
                dlu[4] = e1.x * u1.x; dlu[5] = e1.y * u1.y; dlu[6] = e1.z * u1.z; dlu[7] = e1.w * u1.w;
                const float4 *pb = reinterpret_cast<const float4 *>(sB + (pp * RB + rr) * Wp + c0);
                const float4 *pc = reinterpret_cast<const float4 *>(sC + (pp * RB + rr) * Wp + c0);
#pragma unroll
                for (int k = 0; k < STRIP / 2; ++k) {
                    const float4 bq = pb[k], cq = pc[k];
                    Bv[2 * k] = f2(bq.x, bq.y); Bv[2 * k + 1] = f2(bq.z, bq.w);
                    Cv[2 * k] = f2(cq.x, cq.y); Cv[2 * k + 1] = f2(cq.z, cq.w);
                }
            }
            float2 a[STRIP], p[STRIP], h[STRIP], s[STRIP];
            row_forward<L, true>(j, dl, dlu, Bv, A2, lgd, h_up, a_up, a, p, h, s);
            float *yrow = sy + (dc * RB + rr) * Wp + c0;
#pragma unroll
            for (int i = 0; i < STRIP; ++i) {
                // C*(h - s + 0.25 p), summed over the two states of the pair
                const float2 t = mul2(Cv[i], fma2(p[i], bc(0.25f), sub2(h[i], s[i])));
                atomicAdd(yrow + i, t.x + t.y);
                h_up[i] = h[i];
                a_up[i] = a[i];
            }
            const int r = r0 + rr;
            if (rr == RB - 1 && r + 1 < H && ch_ok) {
                float4 *ck = reinterpret_cast<float4 *>(
                    P.saved + ((((int64_t)b * P.dim + d) * P.nck + r / RB) * NP + pp) * Wp + c0);
#pragma unroll
                for (int k = 0; k < STRIP / 2; ++k)
                    ck[k] = make_float4(h[2 * k].x, h[2 * k].y, h[2 * k + 1].x, h[2 * k + 1].y);
            }
        }
        __syncthreads();
    }
    // ---- write out the last block -----------------------------------------------
    const int rl = ((H - 1) / RB) * RB, nl = H - rl;
    for (int idx = tid; idx < n_in; idx += blockDim.x) {
        const int c = idx % Wp, rr = (idx / Wp) % RB, sdc = idx / (Wp * RB);
        if (sdc < dvalid && c < W && rr < nl) {
            const int64_t o = (int64_t)b * P.o_bs + (int64_t)(d0 + sdc) * P.o_ds + (int64_t)(rl + rr) * P.o_hs + c;
            st_elem(P.out, o, P.out_dt, sy[idx]);
        }
    }
}

size_t fwd_smem_bytes(int L, int DC, int NP) {
    const int Wp = L * STRIP;
    return (size_t)(3 * DC * RB * Wp) * 4 + (size_t)(2 * NP * RB * Wp) * 8;
}

template <int L>
static cudaError_t launch(const Dev &P, int grid, int threads, size_t smem, cudaStream_t st) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(fwd_kernel<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    fwd_kernel<L><<<grid, threads, smem, st>>>(P);
    return cudaGetLastError();
}

cudaError_t launch_fwd(const Dev &P, int L, int grid, int threads, cudaStream_t st) {
    const size_t smem = fwd_smem_bytes(L, P.DC, P.NP);
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

// Row-walk forward kernel (sm_100a): images of at most 64 columns with more than 8 states per channel.
//
// The tile kernel (cs2d_fwd.cu) solves the recurrence along a row as a scan: every lane folds its strip,
// a shuffle scan combines the lane aggregates, a second pass applies the carries - each row is visited
// twice and every step of the shuffle scan is a latency chain.  Here the lanes of a row are SKEWED in
// time instead: in iteration t the lane that owns strip j works on image row t - j, one row behind
// its left neighbour, so the values that enter its strip from the left (h, s, a of the neighbour's
// last column) were finished one iteration earlier and arrive with one shuffle.  Inside its strip a
// thread simply walks the columns left to right; the row above stays in registers.  No scan, no
// second pass, no barrier inside a row.
//   * thread: a strip of SWD (7 or 8) columns x 2 state pairs (4 states, packed fp32x2 arithmetic);
//   * LR lanes cover a row, QC lanes the state pairs of a channel, a warp holds 32/(LR*QC) channels
//     and walks their whole image (H + LR - 1 iterations), so the pipeline fills and drains once;
//   * softplus(delta + bias) and u of the warp's channels are staged by the warp itself, one
//     iteration ahead, as "diagonal rows" (strip j holds row t - j): entries (dl, dl, dl*u, dl*u),
//     ready for packed use; B and C of the group, which a small kernel has regrouped beforehand into
//     fp32 entries of four states (wbc_kernel), are staged the same way for the whole CTA by the staging
//     warps with asynchronous 16-byte copies into a ring of slots guarded by mbarriers (every wait
//     bounded) - several iterations ahead, no registers held while the data travels;
//   * y: summed over a thread's 4 states, then over the channel's QC lanes with a shuffle
//     reduce-scatter, which leaves every lane two columns to store.
// Strips of 7 columns make 56-, 28-, 14- and 7-column rows fill their lanes exactly, and a strip
// pitch of 7 (9 for 8-column strips) 16-byte entries keeps every 128-bit shared-memory access of a
// quarter warp on distinct banks.
// The checkpoints (h of the last row of every block of RB rows) are written in the tile kernels'
// layout, so either backward kernel can follow.  Math: reference forward kernel
// include/cusoflex/selective_scan_fwd_kernel_oflex.cuh:214-338.
#include "cs2d_common.cuh"

namespace cs2d {

constexpr int WK_NWC = 12;   // compute warps per CTA
constexpr int WK_NWS = 4;    // staging warps (B and C); setmaxnreg acts on whole warpgroups (4 consecutive warps),
                             // so both groups of warps are multiples of 4
constexpr int WK_NS = 8;     // slots of the B / C ring: a slot is refilled when every compute warp is done with it, 7 iterations before its next use
constexpr int WK_THREADS = (WK_NWC + WK_NWS) * 32;
// setmaxnreg: the staging warps hand registers to the compute warps.  The CTA starts with 128 registers per
// thread (512 threads, one CTA per SM) and setmaxnreg.inc blocks until the CTA's own pool has what it asks
// for - for ever, if the two numbers below ask for more than the CTA was given.
constexpr int WK_REGS_LAUNCH = 128, WK_REGS_COMPUTE = 160, WK_REGS_STAGE = 32;
static_assert(WK_NWC % 4 == 0 && WK_NWS % 4 == 0, "setmaxnreg is executed by whole warpgroups");
static_assert(WK_NWC * WK_REGS_COMPUTE + WK_NWS * WK_REGS_STAGE <= (WK_NWC + WK_NWS) * WK_REGS_LAUNCH,
              "setmaxnreg.inc would wait for registers the CTA does not own");
// Waits for a phase of an mbarrier: one test (the usual case: the data is there), then a test every
// `sleep_ns` - a waiting warp must not take issue slots from the working ones.  Gives up after 2^20
// tests (a second at the longer interval) and reports failure, so that the caller can flag it and leave.
__device__ __forceinline__ bool wk_wait(uint64_t *bar, uint32_t parity, unsigned sleep_ns) {
    for (int i = 0; i < (1 << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(sleep_ns);
    }
    return false;
}
// softplus with the reference's threshold (x above 20 passes through; fwd kernel :221-224), on the
// special-function unit: t = e^min(x,20); log(1+t) as lg2(1+t)*ln2, or its series where 1+t would round
// t away (t < 0.03: remainder below t^4/4, relative 7e-6); log(1+e^x) >= x, so the maximum with x applies
// the threshold.
__device__ __forceinline__ float wk_softplus(float x) {
    const float t = ex2(fminf(x, 20.f) * LOG2E);
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(1.f + t));
    const float l = t < 0.03f ? t * fmaf(t, fmaf(t, 0.33333334f, -0.5f), 1.f) : y * 0.6931471805599453f;
    return fmaxf(l, x);
}
// One element, loaded only when `on` (else 0), as raw bits: the guard is a predicate on the load, so that
// nothing depends on the loaded register until the value is used iterations later (a select on the
// result would wait for the memory access on the spot).
template <int DT>
__device__ __forceinline__ uint32_t wk_ld_raw(const void *p, int64_t i, bool on) {
    if constexpr (DT == CS2D_F32) {
        uint32_t v;
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\tmov.b32 %0, 0;\n\t@p ld.global.nc.b32 %0, [%1];\n\t}"
                     : "=r"(v) : "l"(reinterpret_cast<const float *>(p) + i), "r"((int)on));
        return v;
    } else {
        unsigned short v;
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\tmov.b16 %0, 0;\n\t@p ld.global.nc.b16 %0, [%1];\n\t}"
                     : "=h"(v) : "l"(reinterpret_cast<const uint16_t *>(p) + i), "r"((int)on));
        return v;
    }
}
// predicated stores: a guard that differs between the lanes of a warp costs a predicate, not a branch
__device__ __forceinline__ void wk_st8_if(float2 *p, float2 v, bool on) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %3, 0;\n\t@p st.global.v2.f32 [%0], {%1,%2};\n\t}" ::"l"(p), "f"(v.x), "f"(v.y),
                 "r"((int)on)
                 : "memory");
}
__device__ __forceinline__ void wk_st4_if(void *p, uint32_t v, bool on) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p st.global.b32 [%0], %1;\n\t}" ::"l"(p), "r"(v), "r"((int)on) : "memory");
}
__device__ __forceinline__ void wk_st2_if(void *p, unsigned short v, bool on) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p st.global.b16 [%0], %1;\n\t}" ::"l"(p), "h"(v), "r"((int)on) : "memory");
}
__device__ __forceinline__ void wk_sts8_if(float2 *p, float2 v, bool on) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %3, 0;\n\t@p st.shared.v2.f32 [%0], {%1,%2};\n\t}" ::"r"(smem_addr(p)), "f"(v.x),
                 "f"(v.y), "r"((int)on)
                 : "memory");
}
__device__ __forceinline__ void wk_st16_if(float4 *p, float4 v, bool on) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t@p st.global.v4.f32 [%0], {%1,%2,%3,%4};\n\t}" ::"l"(p), "f"(v.x),
                 "f"(v.y), "f"(v.z), "f"(v.w), "r"((int)on)
                 : "memory");
}
// one result element of runtime type dt (the branch on dt is uniform)
__device__ __forceinline__ void wk_st_elem_if(void *base, int64_t i, int dt, float v, bool on) {
    if (dt == CS2D_F32) wk_st4_if(reinterpret_cast<float *>(base) + i, __float_as_uint(v), on);
    else if (dt == CS2D_BF16) wk_st2_if(reinterpret_cast<uint16_t *>(base) + i, __bfloat16_as_ushort(__float2bfloat16(v)), on);
    else wk_st2_if(reinterpret_cast<uint16_t *>(base) + i, __half_as_ushort(__float2half(v)), on);
}
template <int DT>
__device__ __forceinline__ float wk_cvt(uint32_t raw) {
    if constexpr (DT == CS2D_F32) return __uint_as_float(raw);
    else if constexpr (DT == CS2D_BF16) return __uint_as_float(raw << 16);
    else return __half2float(__ushort_as_half((unsigned short)raw));
}
__host__ __device__ constexpr int wk_pitch(int swd) { return swd | 1; }   // strip pitch in 16-byte entries: odd

__device__ __forceinline__ void wk_cp16(void *dst, const void *src, bool on) {   // off: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(on ? 16 : 0) : "memory");
}
// the barrier gets one arrival from this thread when all asynchronous copies it has issued so far have landed
__device__ __forceinline__ void wk_cp_arrive(uint64_t *bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// B and C regrouped for the row-walk kernels: [batch][G][H][QC][W] entries of four consecutive states
// (fp32; states past dstate are zero), so that one 16-byte copy fetches what a thread needs for a column.
template <int QC>
__global__ void wbc_kernel(const Dev P) {
    const int row = blockIdx.x, R = row % P.H, bg = row / P.H, g = bg % P.G, b = bg / P.G;
    const int64_t ob = (int64_t)b * P.B_bs + (int64_t)g * P.B_gs + (int64_t)R * P.B_hs;
    const int64_t oc = (int64_t)b * P.C_bs + (int64_t)g * P.C_gs + (int64_t)R * P.C_hs;
    for (int e = threadIdx.x; e < QC * P.W; e += blockDim.x) {
        const int q = e / P.W, c = e % P.W;
        float vb[4], vc[4];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            const bool on = 4 * q + n < P.N;
            vb[n] = on ? ld_elem(P.B, ob + (int64_t)(4 * q + n) * P.B_ns + c, P.io_dt) : 0.f;
            vc[n] = on ? ld_elem(P.C, oc + (int64_t)(4 * q + n) * P.C_ns + c, P.io_dt) : 0.f;
        }
        P.wbt[(int64_t)row * QC * P.W + e] = make_float4(vb[0], vb[1], vb[2], vb[3]);
        P.wct[(int64_t)row * QC * P.W + e] = make_float4(vc[0], vc[1], vc[2], vc[3]);
    }
}

template <int SWD, int LR, int QC>
struct WalkSmem {
    static constexpr int SP = wk_pitch(SWD), TW = LR * SP, CPW = 32 / (LR * QC), EW = CPW * TW;
    static constexpr size_t bars = 0;                                  // full[WK_NS], free[WK_NS]
    static constexpr size_t B = 128;                                   // float4 [WK_NS][QC][TW]
    static constexpr size_t C = B + (size_t)WK_NS * QC * TW * 16;
    static constexpr size_t DU = C + (size_t)WK_NS * QC * TW * 16;     // float4 [WK_NWC][2][EW]
    static constexpr size_t Du = DU + (size_t)WK_NWC * 2 * EW * 16;    // float  [WK_NWC][2][EW]
    // checkpoint rows on their way out: per compute warp two slots of [CPW channels][2*QC pairs][8*LR columns]
    // float2, rows padded by two entries (the lanes of one store then fall on distinct banks)
    static constexpr int NPR = 2 * QC, WPC = 8 * LR, TP = WPC + 2, CKS = CPW * NPR * TP;
    static constexpr size_t CK = (Du + (size_t)WK_NWC * 2 * EW * 4 + 15) & ~(size_t)15;
    static constexpr size_t total = CK + (size_t)WK_NWC * 2 * CKS * 8;
};

template <int SWD, int LR, int QC, int DT>
__global__ void __launch_bounds__(WK_THREADS, 1) wfwd_kernel(const Dev P) {
    using S = WalkSmem<SWD, LR, QC>;
    static_assert(RB == 4, "checkpoint rows are found with shifts and masks");
    constexpr int SP = S::SP, TW = S::TW, CPW = S::CPW, EW = S::EW;
    constexpr int NE = (EW + 31) / 32;   // dl/u entries a lane stages per iteration
    constexpr int NM = (TW + 31) / 32;   // B/C tile columns a staging lane covers
    extern __shared__ __align__(16) unsigned char wsm[];
    uint64_t *full = reinterpret_cast<uint64_t *>(wsm + S::bars), *freeb = full + WK_NS;
    float4 *sB = reinterpret_cast<float4 *>(wsm + S::B), *sC = reinterpret_cast<float4 *>(wsm + S::C);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x % P.ntiles, bg = blockIdx.x / P.ntiles, g = bg % P.G, b = bg / P.G;
    constexpr int CT = WK_NWC * CPW;
    const int dbase = g * P.dpg + tile * CT, nch = min(CT, (g + 1) * P.dpg - dbase);
    const int H = P.H, W = P.W, N = P.N;
    const int niter = H + LR - 1;
    const int nactive = min(WK_NWC, (nch + CPW - 1) / CPW);   // compute warps that hold a channel
    if (tid == 0) {
        for (int s = 0; s < WK_NS; ++s) { mbar_init(full + s, 32); mbar_init(freeb + s, nactive); }
        mbar_init_fence();
    }
    __syncthreads();

    if (warp >= WK_NWC) {
        // ---- staging warps: B and C of iteration t, strip jj holding image row t - jj ----
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(WK_REGS_STAGE));
        const int ws = warp - WK_NWC;
        int s_jj[NM], s_off[NM];   // strip and source offset (column) of the tile columns this lane copies
        bool s_on[NM];
#pragma unroll
        for (int m = 0; m < NM; ++m) {
            const int cc = lane + 32 * m, i = cc % SP;
            s_jj[m] = cc / SP;
            s_off[m] = s_jj[m] * SWD + i;
            s_on[m] = cc < TW && i < SWD && s_off[m] < W;
        }
        const float4 *bt = P.wbt + (int64_t)bg * H * QC * W, *ct = P.wct + (int64_t)bg * H * QC * W;
        for (int t = ws; t < niter; t += WK_NWS) {
            const int slot = t % WK_NS, use = t / WK_NS;
            if (use > 0 && !__all_sync(0xffffffffu, wk_wait(freeb + slot, (use - 1) & 1, 1000))) {
                atomicOr(P.status, ERR_STAGE_TIMEOUT);
                return;
            }
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                const int cc = lane + 32 * m, R = t - s_jj[m];
                const bool on = s_on[m] && R >= 0 && R < H;
                const int src = on ? R * QC * W + s_off[m] : 0;
                if (cc < TW) {
#pragma unroll
                    for (int q = 0; q < QC; ++q) {
                        wk_cp16(sB + (slot * QC + q) * TW + cc, bt + src + q * W, on);
                        wk_cp16(sC + (slot * QC + q) * TW + cc, ct + src + q * W, on);
                    }
                }
            }
            wk_cp_arrive(full + slot);   // arrives when this lane's copies have landed
        }
        return;
    }
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(WK_REGS_COMPUTE));
    if (warp >= nactive) return;   // no channel left for this warp (the barriers do not count it)

    // ---- compute warps ----
    const int j = lane % LR, q = (lane / LR) % QC, chw = lane / (LR * QC);
    const int chl = warp * CPW + chw;
    const bool ch_ok = chl < nch;
    const int d = dbase + min(chl, nch - 1);   // idle channel slots shadow a valid channel, their results are dropped
    float4 *sDU = reinterpret_cast<float4 *>(wsm + S::DU) + warp * 2 * EW;
    float *sDu = reinterpret_cast<float *>(wsm + S::Du) + warp * 2 * EW;
    const float2 lgd = bc(P.decay ? log2f(__ldg(P.decay)) : 0.f);
    float2 A2[2];
    bool pair_on[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int n0 = 2 * (2 * q + k), n1 = n0 + 1;
        pair_on[k] = n0 < N;
        A2[k] = f2(n0 < N ? __ldg(P.A + (int64_t)d * P.A_ds + n0 * P.A_ns) * LOG2E : 0.f,
                   n1 < N ? __ldg(P.A + (int64_t)d * P.A_ds + n1 * P.A_ns) * LOG2E : 0.f);
    }

    // the dl / u entries this lane stages: entry e -> channel, strip, column inside the strip.  ox / ou
    // are the element offsets of the entry in the image row the NEXT call of stage_load wants.
    int e_jj[NE];
    int64_t ox[NE], ou[NE];
    float e_bias[NE], e_D[NE];
    bool e_on[NE];
    const int64_t dl_hs = P.dl_hs, u_hs = P.u_hs;
#pragma unroll
    for (int m = 0; m < NE; ++m) {
        const int e = lane + 32 * m, cw = e / TW, cc = e % TW, i = cc % SP;
        e_jj[m] = cc / SP;
        const int c = e_jj[m] * SWD + i, che = warp * CPW + cw;
        e_on[m] = e < EW && i < SWD && c < W && che < nch;
        const int de = dbase + min(che, nch - 1);
        ox[m] = (int64_t)b * P.dl_bs + (int64_t)(de / P.drep) * P.dl_ds + c - (int64_t)e_jj[m] * dl_hs;
        ou[m] = (int64_t)b * P.u_bs + (int64_t)de * P.u_ds + c - (int64_t)e_jj[m] * u_hs;
        e_bias[m] = P.bias ? __ldg(P.bias + de / P.drep) : 0.f;
        e_D[m] = P.D ? __ldg(P.D + de) : 0.f;
    }
    const bool softplus = P.softplus != 0;
    // raw values travel for two iterations: two register sets, used in turn
    uint32_t rx[2][NE], ru[2][NE];
    auto stage_load = [&](int t2, uint32_t (&vx)[NE], uint32_t (&vu)[NE]) {   // raw delta and u of iteration t2 (calls come in order of t2)
#pragma unroll
        for (int m = 0; m < NE; ++m) {
            const int R = t2 - e_jj[m];
            const bool on = e_on[m] && R >= 0 && R < H;
            vx[m] = wk_ld_raw<DT>(P.delta, ox[m], on);
            vu[m] = wk_ld_raw<DT>(P.u, ou[m], on);
            ox[m] += dl_hs; ou[m] += u_hs;
        }
    };
    auto stage_store = [&](int t2, const uint32_t (&vx)[NE], const uint32_t (&vu)[NE]) {  // ... transformed, into the warp's slot of iteration t2
#pragma unroll
        for (int m = 0; m < NE; ++m) {
            const int e = lane + 32 * m, R = t2 - e_jj[m];
            const bool on = e_on[m] && R >= 0 && R < H;
            const float uv = wk_cvt<DT>(vu[m]);
            float dl = wk_cvt<DT>(vx[m]) + e_bias[m];
            // fp32 I/O: the same evaluation as the backward's recompute (h - s cancels, the two must agree to the last bit)
            if (softplus) dl = DT == CS2D_F32 ? softplus20(dl) : wk_softplus(dl);
            dl = on ? dl : 0.f;   // columns and rows outside the image: a = 1, p = 0
            if (e < EW) {
                sDU[(t2 & 1) * EW + e] = make_float4(dl, dl, dl * uv, dl * uv);
                sDu[(t2 & 1) * EW + e] = e_D[m] * uv;
            }
        }
    };
    stage_load(0, rx[0], ru[0]);
    stage_store(0, rx[0], ru[0]);
    stage_load(1, rx[1], ru[1]);
    stage_load(2, rx[0], ru[0]);
    __syncwarp();

    // row above (h, a), per state pair; values handed to the right neighbour; the diagonal carry
    float2 h_up[2][SWD], a_up[2][SWD], h_last[2], s_last[2], a_last[2], hd_prev[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
#pragma unroll
        for (int i = 0; i < SWD; ++i) { h_up[k][i] = bc(0.f); a_up[k][i] = bc(0.f); }
        h_last[k] = s_last[k] = a_last[k] = hd_prev[k] = bc(0.f);
    }
    // what this lane stores of a row: the columns the reduce-scatter below leaves it with
    constexpr int CNT = 8 / QC;
    const int ybase = (QC >= 2 && (q & 1) ? 4 : 0) + (QC >= 4 && (q & 2) ? 2 : 0);
    bool y_on[CNT];
#pragma unroll
    for (int x = 0; x < CNT; ++x) y_on[x] = ch_ok && ybase + x < SWD && j * SWD + ybase + x < W;
    const int64_t o_hs = P.o_hs;
    int64_t yo = (int64_t)b * P.o_bs + (int64_t)d * P.o_ds + j * SWD + ybase - (int64_t)j * o_hs;   // row t - j of iteration t = 0
    int du_idx[CNT];   // D*u of those columns; a column the lane does not store reads (and drops) the strip's last entry
#pragma unroll
    for (int x = 0; x < CNT; ++x) du_idx[x] = chw * TW + j * SP + min(ybase + x, SWD - 1);
    // Checkpoint rows: this lane's strips go to the warp's shared tile (two slots: the next checkpoint row
    // begins before the last lane has finished this one), the warp writes the finished row.  The tile is
    // zero-filled once: columns no strip covers and idle pairs stay finite for the backward's padded strips.
    constexpr int NPR = S::NPR, WPC = S::WPC, TP = S::TP, CKS = S::CKS;
    float2 *sCK = reinterpret_cast<float2 *>(wsm + S::CK) + warp * 2 * CKS;
    for (int i = lane; i < 2 * CKS; i += 32) sCK[i] = bc(0.f);
    float2 *ck_mine = sCK + (chw * NPR + 2 * q) * TP + j * SWD;   // pair k: + k*TP; slot: + CKS
    const bool keep_ck = !P.ck_roll;
    // flush: float4 number lane + 32*m of a slot (m < 8) belongs to channel m / LR of the warp, pair row
    // lane / (4*LR) + (8/LR) * (m % LR), column pair lane % (4*LR)
    const float4 *ck_src0 = reinterpret_cast<const float4 *>(sCK + (lane / (4 * LR)) * TP + 2 * (lane % (4 * LR)));
    const int ck_lane4 = (lane / (4 * LR)) * (WPC / 2) + lane % (4 * LR);
    float4 *saved4 = reinterpret_cast<float4 *>(P.saved);
    const int ck_step4 = NPR * WPC / 2;   // float4 per checkpoint block of a channel
    const int out_dt = P.out_dt;

    const float4 *sB0 = sB + q * TW + j * SP, *sC0 = sC + q * TW + j * SP, *sDU0 = sDU + chw * TW + j * SP;

    for (int t = 0; t < niter; ++t) {
        const int slot = t % WK_NS;
        if (!__all_sync(0xffffffffu, wk_wait(full + slot, (t / WK_NS) & 1, 100))) {   // the warp leaves as a whole
            atomicOr(P.status, ERR_STAGE_TIMEOUT);
            return;
        }
        const float4 *tB = sB0 + slot * QC * TW, *tC = sC0 + slot * QC * TW;
        const float4 *tDU = sDU0 + (t & 1) * EW;
        // h, s, a of the column left of the strip: the left neighbour finished them one iteration ago
        float2 hl[2], sl[2], al[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            if constexpr (LR > 1) {
                hl[k] = shfl_up2<LR>(h_last[k], 1); sl[k] = shfl_up2<LR>(s_last[k], 1); al[k] = shfl_up2<LR>(a_last[k], 1);
                if (j == 0) { hl[k] = bc(0.f); sl[k] = bc(0.f); al[k] = bc(0.f); }
            } else {
                hl[k] = sl[k] = al[k] = bc(0.f);
            }
        }
        const int R = t - j;
        const bool act = R >= 0 && R < H;
        float yv[8];
        yv[7] = 0.f;
        {   // lanes whose row is outside the image work on zero-filled entries: whatever they produce is
            // never stored, and no lane inside the image ever receives it (see the skew)
            float2 hleft[2], sleft[2], aleft[2], hdg[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) { hleft[k] = hl[k]; sleft[k] = sl[k]; aleft[k] = al[k]; hdg[k] = hd_prev[k]; }
#pragma unroll
            for (int i = 0; i < SWD; ++i) {
                const float4 du = tDU[i], Bv = tB[i], Cv = tC[i];
                const float2 dl2 = f2(du.x, du.y), dlu2 = f2(du.z, du.w);
                float2 ys = bc(0.f);
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const float2 Bk = k ? f2(Bv.z, Bv.w) : f2(Bv.x, Bv.y), Ck = k ? f2(Cv.z, Cv.w) : f2(Cv.x, Cv.y);
                    const float2 a = ex2_2(fma2(dl2, A2[k], lgd));
                    const float2 p = mul2(Bk, dlu2);
                    // h = a*(h_left + h_up - 0.5*(a_up + a_left)*h_diag) + p ;  s = a*s_left + p
                    const float2 kap = fma2(mul2(add2(a_up[k][i], aleft[k]), hdg[k]), bc(-0.5f), h_up[k][i]);
                    const float2 beta = fma2(a, kap, p);
                    const float2 h = fma2(a, hleft[k], beta);
                    const float2 s = fma2(a, sleft[k], p);
                    hdg[k] = h_up[k][i];
                    h_up[k][i] = h; a_up[k][i] = a;
                    aleft[k] = a; hleft[k] = h; sleft[k] = s;
                    ys = fma2(Ck, fma2(p, bc(0.25f), sub2(h, s)), ys);
                }
                yv[i] = ys.x + ys.y;
            }
#pragma unroll
            for (int k = 0; k < 2; ++k) { h_last[k] = hleft[k]; s_last[k] = sleft[k]; a_last[k] = aleft[k]; hd_prev[k] = hl[k]; }
        }
        // sum over the channel's QC lanes: each step halves what a lane keeps
        if constexpr (QC >= 2) {
            const bool hi = q & 1;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float keep = hi ? yv[i + 4] : yv[i], send = hi ? yv[i] : yv[i + 4];
                yv[i] = keep + __shfl_xor_sync(0xffffffffu, send, LR);
            }
        }
        if constexpr (QC >= 4) {
            const bool hi = q & 2;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float keep = hi ? yv[i + 2] : yv[i], send = hi ? yv[i] : yv[i + 2];
                yv[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2 * LR);
            }
        }
#pragma unroll
        for (int x = 0; x < CNT; ++x)
            wk_st_elem_if(P.out, yo + x, out_dt, yv[x] + sDu[(t & 1) * EW + du_idx[x]], act && y_on[x]);
        // the last row of a block of RB rows is the checkpoint of that block (none after the last block).  The
        // lanes of a row are at different image rows, so in every iteration some of them are at such a row.
        {
            const bool ck_on = act && keep_ck && (R & (RB - 1)) == RB - 1 && R + 1 < H;
            float2 *mine = ck_mine + ((R >> 2) & 1) * CKS;
#pragma unroll
            for (int k = 0; k < 2; ++k)
#pragma unroll
                for (int i = 0; i < SWD; ++i) wk_sts8_if(mine + k * TP + i, h_up[k][i], ck_on);
        }
        {   // the row the last lane has just finished: complete, written by the whole warp
            const int Rf = t - (LR - 1);
            if (keep_ck && Rf >= 0 && (Rf & (RB - 1)) == RB - 1 && Rf + 1 < H) {   // uniform
                __syncwarp();
                const int so = ((Rf >> 2) & 1) * (CKS / 2);   // float4 units: CKS is even
                const int64_t go = (int64_t)(Rf >> 2) * ck_step4;
#pragma unroll
                for (int m = 0; m < 8; ++m) {
                    const int cw = m / LR, rowm = cw * NPR + (8 / LR) * (m % LR);   // compile-time
                    const int che = warp * CPW + cw;
                    const int64_t dm = (int64_t)b * P.dim + dbase + min(che, nch - 1);
                    wk_st16_if(saved4 + dm * P.nck * ck_step4 + go + (8 / LR) * (m % LR) * (WPC / 2) + ck_lane4,
                               ck_src0[so + rowm * (TP / 2)], che < nch);
                }
            }
        }
        yo += o_hs;
        __syncwarp();                                    // every lane is done with slot t
        if (lane == 0) mbar_arrive(freeb + slot);
        if (t + 1 < niter) {   // the set of iteration t+1 was loaded two iterations ago and is free for t+3 afterwards
            if ((t + 1) & 1) { stage_store(t + 1, rx[1], ru[1]); stage_load(t + 3, rx[1], ru[1]); }
            else { stage_store(t + 1, rx[0], ru[0]); stage_load(t + 3, rx[0], ru[0]); }
            __syncwarp();
        }
    }
}

template <int SWD, int LR, int QC, int DT>
static cudaError_t launch_wf4(const Dev &P, int grid, cudaStream_t st) {
    using S = WalkSmem<SWD, LR, QC>;
    static bool attr_done[64] = {};  // per template instance and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(wfwd_kernel<SWD, LR, QC, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::total);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    wbc_kernel<QC><<<P.batch * P.G * P.H, 128, 0, st>>>(P);
    wfwd_kernel<SWD, LR, QC, DT><<<grid, WK_THREADS, S::total, st>>>(P);
    return cudaGetLastError();
}
template <int SWD, int LR, int QC>
static cudaError_t launch_wf3(const Dev &P, int grid, cudaStream_t st) {
    switch (P.io_dt) {
        case CS2D_F32: return launch_wf4<SWD, LR, QC, CS2D_F32>(P, grid, st);
        case CS2D_F16: return launch_wf4<SWD, LR, QC, CS2D_F16>(P, grid, st);
        default: return launch_wf4<SWD, LR, QC, CS2D_BF16>(P, grid, st);
    }
}
template <int SWD>
static cudaError_t launch_wf2(const Dev &P, int LR, int grid, cudaStream_t st) {
    switch (LR) {
        case 1: return launch_wf3<SWD, 1, 4>(P, grid, st);
        case 2: return launch_wf3<SWD, 2, 4>(P, grid, st);
        case 4: return launch_wf3<SWD, 4, 4>(P, grid, st);
        case 8: return launch_wf3<SWD, 8, 4>(P, grid, st);
    }
    return cudaErrorInvalidValue;
}

// Strip width and lanes per row for rows of `ncols` columns (ncols <= 64): strips of 7 when they need
// no more lanes than strips of 8 (every multiple of 7 up to 56 then fills its lanes exactly).
void walk_geometry(int ncols, int *swd, int *lr) {
    int l7 = 1, l8 = 1;
    while (l7 * 7 < ncols) l7 <<= 1;
    while (l8 * 8 < ncols) l8 <<= 1;
    if (l7 <= l8 && l7 <= 8) { *swd = 7; *lr = l7; } else { *swd = 8; *lr = l8; }
}
// channels per CTA
int walk_channels_per_cta(int lr) { return WK_NWC * (32 / (lr * 4)); }
// bytes of the regrouped B and C that follow the checkpoints in the saved-state buffer
size_t walk_bc_bytes(int batch, int groups, int nrows, int ncols) { return (size_t)2 * batch * groups * nrows * 4 * ncols * sizeof(float4); }

cudaError_t launch_walk_fwd(const Dev &P, int grid, cudaStream_t st) {
    int swd, lr;
    walk_geometry(P.W, &swd, &lr);
    // the checkpoint layout the kernel writes: 8 pair slots (more than 8 states), 8*lr columns per row
    if (P.NPp != 8 || P.ck_wp != 8 * lr) return cudaErrorInvalidValue;
    return swd == 7 ? launch_wf2<7>(P, lr, grid, st) : launch_wf2<8>(P, lr, grid, st);
}

}  // namespace cs2d

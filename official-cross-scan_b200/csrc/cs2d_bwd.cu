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
// Row blocks are processed from the bottom up; inside a block the CTA walks its
// channels in passes.  For each (pass, block) h is recomputed from the
// checkpoint row the forward saved, kept in registers, and consumed by the
// reverse sweep; the plain row scan s is recomputed per row.  The adjoint row m
// that crosses the block boundary is parked in a global scratch buffer.
// dB/dC are summed over the warp's channels through a per-warp transposition
// buffer and accumulated over passes in shared memory, then added to global
// memory once per block and CTA.
#include "cs2d_common.cuh"

// This file is compiled twice: as it is (every group of a launch is served by CTAs of its own), and
// from cs2d_bwd_serial.cu with CS2D_SERIAL_DIRS = 1 (the reproducible direction merge: one CTA walks all
// groups of its channel tile).  The choice is a compile-time constant so that the common form carries
// no trace of the loop over directions.
#ifndef CS2D_SERIAL_DIRS
#define CS2D_SERIAL_DIRS 0
#endif

namespace cs2d {
constexpr bool SERIAL = CS2D_SERIAL_DIRS != 0;

static_assert(RB == STREAM_RB, "the tile backward reads the streaming forward's checkpoints at its own row-block cadence");

template <int L>
struct BwdSmem {
    static constexpr int Wp = L * STRIP, CW = 32 / L;
    static constexpr int CS4 = chan_stride<L>(RB), CS6 = chan_stride<L>(RB + 2);
    // float offsets
    static __host__ __device__ constexpr int u(int) { return 0; }
    static __host__ __device__ constexpr int g(int CP) { return CP * CS4; }
    static __host__ __device__ constexpr int sig(int CP) { return 2 * CP * CS4; }
    static __host__ __device__ constexpr int dl(int CP) { return 3 * CP * CS4; }                 // RB+2 rows
    static __host__ __device__ constexpr int pdu(int CP) { return dl(CP) + CP * CS6; }           // [warps][CW][CS4]
    static __host__ __device__ constexpr int pdd(int CP, int nw) { return pdu(CP) + nw * CW * CS4; }
    static __host__ __device__ constexpr int tr(int CP, int nw) { return pdd(CP, nw) + nw * CW * CS4; }   // [warps][2][256] float2
    static __host__ __device__ constexpr int B(int CP, int nw) { return tr(CP, nw) + (CW > 1 ? nw * 1024 : 0); }  // [NPp][RB][Wp] float2
    static __host__ __device__ constexpr int C(int CP, int NPp, int nw) { return B(CP, nw) + NPp * RB * Wp * 2; }
    static __host__ __device__ constexpr int aB(int CP, int NPp, int nw) { return C(CP, NPp, nw) + NPp * RB * Wp * 2; }  // [warps][RB][Wp] float2
    static __host__ __device__ constexpr int aC(int CP, int NPp, int nw, bool acc) { return aB(CP, NPp, nw) + (acc ? nw * RB * Wp * 2 : 0); }
    static __host__ __device__ constexpr int dA(int CP, int NPp, int nw, bool acc) { return aC(CP, NPp, nw, acc) + (acc ? nw * RB * Wp * 2 : 0); }
    // one set of staged per-channel tiles (u, dout, sigmoid, delta), rounded to 16 bytes
    static __host__ __device__ constexpr int set_floats(int CP) { return (dl(CP) + CP * CS6 + 3) & ~3; }
    // dD / ddelta_bias partial sums: one slot per (channel, segment of the channel's RB*T4 write-out
    // items that one warp reduces), so that every slot has a single owner and needs no atomics
    static constexpr int SEG = RB * (Wp / 4) < 32 ? RB * (Wp / 4) : 32, NSEG = RB * (Wp / 4) / SEG;
    // dA: [CT][2*NPp], red: [CT][NSEG][2], decay: [warps], par: [CT][2] (D, delta_bias of the CTA's
    // channels), merge weights [CT], dw: [CT][NPp]
    static __host__ __device__ constexpr int total(int CP, int NPp, int CT, int nw, bool acc) {
        return dA(CP, NPp, nw, acc) + CT * 2 * NPp + CT * NSEG * 2 + nw + CT * 3 + CT * NPp;
    }
};

// Row-by-row addition of one state pair's dB/dC values to global memory (shapes whose dB/dC
// tiles do not fit in shared memory).  Deterministic mode adds onto the CTA's own zero-filled
// plane (det_ts elements per channel tile; 0 otherwise): with one channel group per CTA the lane
// that owns (pair, column) is the only one that ever touches that element, pass after pass, so
// the atomic adds arrive in program order.
__device__ __forceinline__ void add_dbc(const Dev &P, int tile, int64_t og, bool two, float2 vb, float2 vc) {
    const int64_t ns = (int64_t)P.H * P.Wout;
    float *qb = P.dB + (int64_t)tile * P.det_ts + og, *qc = P.dC + (int64_t)tile * P.det_ts + og;
    atomicAdd(qb, vb.x);
    atomicAdd(qc, vc.x);
    if (two) { atomicAdd(qb + ns, vb.y); atomicAdd(qc + ns, vc.y); }
}

// NPC = 8 specialises the common geometry (8 state-pair slots, one channel group, 8 warps) so
// that every shared-memory offset is a compile-time constant; NPC = 0 reads it from P.
// TILED compiles the column-tile edge handling in; the common single-tile launch leaves it out.
// WS (with NPC = 8) is the warp-specialised form: warps 0-7 compute as before and
// write out the previous step, warps 8-11 load and transform (softplus, sigmoid) the tiles of
// the NEXT step into a second tile set meanwhile, so that the staging - global-memory latency
// and the transcendental chains - no longer sits between two compute phases.  The two groups
// meet on mbarriers (tile set full / tile set free), every wait bounded.  The staging warps
// give most of their registers to the compute warps (setmaxnreg).
constexpr int WS_COMPUTE = 256, WS_STAGE = 128, WS_REGS_COMPUTE = 232, WS_REGS_STAGE = 40;
// SER = SERIAL: part of the kernel's name, so that the two compilations of this file define distinct kernels
template <int L, int NPC, bool TILED, bool WS, bool SER>
__global__ void __launch_bounds__(WS ? WS_COMPUTE + WS_STAGE : MAX_THREADS, 1) bwd_kernel(const Dev P) {
    static_assert(!WS || NPC == 8, "the warp-specialised form covers the common geometry only");
    using S = BwdSmem<L>;
    constexpr int Wp = S::Wp, CW = S::CW, T4 = Wp / 4, CS4 = S::CS4, CS6 = S::CS6, L4 = 4 * L, L2 = 2 * L;
    constexpr int NU = CW >= 8 ? 1 : 8 / CW;  // columns of a strip owned by a lane after the channel sum
    extern __shared__ __align__(16) float smem[];
    const int NPp = NPC ? NPC : P.NPp, CG = NPC ? MAX_WARPS / NPC : P.CG, CP = CG * CW, CT = P.CT;
    const int nw = NPp * CG, nthr = nw * 32;
    // staged tiles of the step being computed; WS alternates between two sets
    float *su = smem + S::u(CP), *sg = smem + S::g(CP), *ssig = smem + S::sig(CP), *sdl = smem + S::dl(CP);
    float *spdu = smem + S::pdu(CP), *spdd = smem + S::pdd(CP, nw);
    float2 *str = reinterpret_cast<float2 *>(smem + S::tr(CP, nw));
    const bool acc_on = P.acc_dbc != 0;  // dB/dC accumulated over passes in shared memory
    float2 *sB = reinterpret_cast<float2 *>(smem + S::B(CP, nw));
    float2 *sC = reinterpret_cast<float2 *>(smem + S::C(CP, NPp, nw));
    float2 *saB = reinterpret_cast<float2 *>(smem + S::aB(CP, NPp, nw));
    float2 *saC = reinterpret_cast<float2 *>(smem + S::aC(CP, NPp, nw, acc_on));
    float *sdA = smem + S::dA(CP, NPp, nw, acc_on);
    float *sred = sdA + CT * 2 * NPp;
    float *sdecay = sred + CT * S::NSEG * 2;
    float *spar = sdecay + nw;
    float *smw = spar + 2 * CT, *sdw = smw + CT;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int j = lane & (L - 1), cl = lane / L;
    const int pp = warp % NPp, cg = warp / NPp;
    const int cp = cg * CW + cl;
    const int tile = blockIdx.x % P.ntiles, bg = blockIdx.x / P.ntiles;
    // Normally a CTA serves one group (scan direction).  With Dev::dir_serial (the reproducible direction
    // merge) it owns its channel tile for ALL groups and walks them one after the other, so that the merged du
    // image is written by this CTA alone: stored by the first direction, read-modify-written by the
    // others in a fixed order, no atomics; the barriers between the directions order those accesses.
    const int ng = SERIAL ? P.G : 1;
    const int b = SERIAL ? bg : bg / P.G;
    int g_ = 0, dbase = 0, nch = 0, ush = 0, gsh = 0, gi = 0;
    bool fh = false, fw = false;
    int64_t cs = 0;
    auto set_dir = [&](int i) {
        gi = i;
        g_ = SERIAL ? i : bg % P.G;
        dbase = g_ * P.dpg + tile * CT;
        nch = min(CT, (g_ + 1) * P.dpg - dbase);
        fh = (P.flip_h >> g_) & 1u; fw = (P.flip_w >> g_) & 1u;   // scan direction of this group
        ush = (P.u_shared & 1) ? g_ * P.dpg : 0;                    // u indexed by channel - ush
        gsh = (P.u_shared & 2) ? g_ * P.dpg : 0;                    // dout indexed by channel - gsh
        cs = fw ? P.cshift : 0;                                     // see Dev::cshift
    };
    set_dir(0);
    const int H = P.H, W = P.W, N = P.N;
    const int n0 = 2 * pp, n1 = n0 + 1;
    const bool pair_on = n0 < N;
    const float decay = P.decay ? __ldg(P.decay) : 1.f;
    const float2 lgd = bc(P.decay ? log2f(decay) : 0.f);
    const bool want_decay = P.ddecay != nullptr;

    float2 ddecay_acc = bc(0.f);
    auto init_dir = [&]() {   // accumulators and parameter copies of the current direction
        for (int i = tid; i < nw * CW * CS4; i += nthr) { spdu[i] = 0.f; spdd[i] = 0.f; }
        if (acc_on)
            for (int i = tid; i < nw * RB * Wp; i += nthr) { saB[i] = bc(0.f); saC[i] = bc(0.f); }
        for (int i = tid; i < CT * 2 * NPp + CT * S::NSEG * 2 + nw; i += nthr) sdA[i] = 0.f;
        // D, delta_bias and merge weight of this CTA's channels; slots past the last valid channel
        // are read too (their staged values are zero, so the weight has to be finite)
        for (int i = tid; i < CT; i += nthr) {
            const bool on = i < nch;
            spar[2 * i] = on && P.D ? __ldg(P.D + dbase + i) : 0.f;
            spar[2 * i + 1] = on && P.bias ? __ldg(P.bias + (dbase + i) / P.drep) : 0.f;
            smw[i] = on && P.mw ? __ldg(P.mw + dbase + i) : 1.f;
        }
        for (int i = tid; i < CT * NPp; i += nthr) sdw[i] = 0.f;
        ddecay_acc = bc(0.f);
    };
    init_dir();

    const int nblk = P.nck, npass = P.npass;
    const int steps = nblk * npass;

    // Bulk asynchronous staging: the raw row blocks of u, dout and delta of step k+1
    // are copied global -> shared by the copy engine while step k computes; an
    // mbarrier per stage counts the bytes.  One thread issues, everybody waits (bounded).
    const bool bulk = P.bulk != 0;
    const int es = P.io_dt == CS2D_F32 ? 4 : 2, eso = P.out_dt == CS2D_F32 ? 4 : 2;
    // tile-edge values staged per step (see Dev::edge_in / adj_in): h,s of the column left of
    // the tile for rows r0-1..r0+RB-1, dh,ds of the column right of it for rows r0..r0+RB, and
    // the softplus'd delta of those two columns
    const int tot4 = (S::total(CP, NPp, CT, nw, acc_on) + 3) & ~3;
    float4 *sedge = reinterpret_cast<float4 *>(smem + tot4);
    // (the four edge areas only exist in the kernels that handle column tiles)
    float4 *sadj = sedge + (TILED ? CP * NPp * (RB + 1) : 0);
    float *sedl_l = reinterpret_cast<float *>(sadj + (TILED ? CP * NPp * (RB + 1) : 0));   // [CP][RB]
    float *sedl_r = sedl_l + (TILED ? CP * 4 : 0);                                          // [CP][RB+1] (pitch 8)
    const bool has_left = TILED && P.tile_left != 0, has_right = TILED && P.tile_right != 0;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sedl_r + (TILED ? CP * 8 : 0));
    unsigned char *raw = reinterpret_cast<unsigned char *>(bars + 2);
    const int stage_bytes = CP * W * (RB * es + RB * eso + (RB + 2) * es);
    auto issue = [&](int k) {  // called by every lane of warp 0: one copy per lane and round
        const int kblk = nblk - 1 - k / npass, kpass = k % npass;
        const int kr0 = kblk * RB, knr = min(RB, H - kr0), kch0 = kpass * CP;
        const int lo = max(kr0 - 1, 0), hi = min(kr0 + knr + 1, H);
        const int nv = max(0, min(CP, nch - kch0));
        uint64_t *bar = bars + (k & 1);
        unsigned char *ru = raw + (size_t)(k & 1) * stage_bytes, *rg = ru + (size_t)CP * RB * W * es;
        unsigned char *rd = rg + (size_t)CP * RB * W * eso;
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)(nv * W * (knr * es + knr * eso + (hi - lo) * es)));
        __syncwarp();
        for (int i = lane; i < 3 * nv; i += 32) {
            const int sc = i / 3, kind = i - 3 * sc;
            const int sd = dbase + kch0 + sc;
            if (kind == 0) {
                bulk_g2s(ru + (size_t)sc * RB * W * es,
                         reinterpret_cast<const char *>(P.u) + ((int64_t)b * P.u_bs + (int64_t)sd * P.u_ds + (int64_t)kr0 * W) * es,
                         (uint32_t)(knr * W * es), bar);
            } else if (kind == 1) {
                bulk_g2s(rg + (size_t)sc * RB * W * eso,
                         reinterpret_cast<const char *>(P.out) + ((int64_t)b * P.o_bs + (int64_t)sd * P.o_ds + (int64_t)kr0 * W) * eso,
                         (uint32_t)(knr * W * eso), bar);
            } else {
                bulk_g2s(rd + (size_t)sc * (RB + 2) * W * es,
                         reinterpret_cast<const char *>(P.delta) +
                             ((int64_t)b * P.dl_bs + (int64_t)(sd / P.drep) * P.dl_ds + (int64_t)lo * W) * es,
                         (uint32_t)((hi - lo) * W * es), bar);
            }
        }
    };
    // WS: second tile set and the full / free mbarriers of the two sets
    float *set1 = reinterpret_cast<float *>(bars + 4);
    uint64_t *full = bars, *freeb = bars + 2;
    if (WS) {
        if (tid == 0) {
            mbar_init(full, WS_STAGE); mbar_init(full + 1, WS_STAGE);
            mbar_init(freeb, WS_COMPUTE); mbar_init(freeb + 1, WS_COMPUTE);
            mbar_init_fence();
        }
    } else if (bulk && tid == 0) {
        mbar_init(bars, 1); mbar_init(bars + 1, 1); mbar_init_fence();
    }
    __syncthreads();  // barriers initialised, parameter copies and zeroed tiles visible
    if (!WS && bulk && warp == 0 && steps > 0) issue(0);

    // loads and transforms the tiles of step k (row block kblk, channels kch0..) into the set at `base`
    auto stage_step = [&](int k, float *base, const unsigned char *raw_k, int t0, int nt) {
        float *tu = base + S::u(CP), *tg = base + S::g(CP), *tsig = base + S::sig(CP), *tdl = base + S::dl(CP);
        const int kblk = nblk - 1 - k / npass, kch0 = (k % npass) * CP;
        const int kr0 = kblk * RB, knr = k < steps ? min(RB, H - kr0) : 0;
        const int lo = max(kr0 - 1, 0);
        const unsigned char *raw_u = raw_k, *raw_g = raw_u + (size_t)CP * RB * W * es;
        const unsigned char *raw_dl = raw_g + (size_t)CP * RB * W * eso;
        for (int it = t0; it < CP * RB * T4; it += nt) {
            const int t = it % T4, rr = (it / T4) % RB, sc = it / (T4 * RB);
            const int c = 4 * t, o4 = sc * CS4 + rr * Wp + pos4<L>(t);
            float4 uv = make_float4(0.f, 0.f, 0.f, 0.f), gv = uv, xv = uv, sv = uv;
            if (rr < knr && kch0 + sc < nch && c < W) {
                const int sd = dbase + kch0 + sc, r = kr0 + rr, sdd = sd / P.drep;
                if (!WS && bulk) {
                    uv = lds4(raw_u, (sc * RB + rr) * W + c, P.io_dt);
                    gv = lds4(raw_g, (sc * RB + rr) * W + c, P.out_dt);
                    xv = lds4(raw_dl, (sc * (RB + 2) + (r - lo)) * W + c, P.io_dt);
                } else {
                    uv = ld4d(P.u, (int64_t)b * P.u_bs + (int64_t)(sd - ush) * P.u_ds + cs, P.u_hs, r, c, H, W, fh, fw,
                              P.io_dt, P.vec & VEC_U);
                    gv = ld4d(P.out, (int64_t)b * P.o_bs + (int64_t)(sd - gsh) * P.o_ds + cs, P.o_hs, r, c, H, W, fh, fw,
                              P.out_dt, P.vec & VEC_OUT);
                    xv = ld4d(P.delta, (int64_t)b * P.dl_bs + (int64_t)sdd * P.dl_ds + cs, P.dl_hs, r, c, H, W, fh, fw,
                              P.io_dt, P.vec & VEC_DELTA);
                }
                soft4(xv, sv, spar[2 * (kch0 + sc) + 1], P.softplus, W - c);
            }
            *reinterpret_cast<float4 *>(tu + o4) = uv;
            *reinterpret_cast<float4 *>(tg + o4) = gv;
            *reinterpret_cast<float4 *>(tsig + o4) = sv;
            *reinterpret_cast<float4 *>(tdl + sc * CS6 + (rr + 1) * Wp + pos4<L>(t)) = xv;
        }
        if (knr > 0) {  // delta of the rows just above and just below the block, one column per item
            for (int it = t0; it < CP * 2 * Wp; it += nt) {
                const int c = it % Wp, which = (it / Wp) & 1, sc = it / (Wp * 2);
                const int rr = which ? RB + 1 : 0, r = kr0 + rr - 1;
                float x = 0.f;
                if (r >= 0 && r < H && rr - 1 <= knr && kch0 + sc < nch && c < W) {
                    const int sdd = (dbase + kch0 + sc) / P.drep;
                    if (!WS && bulk)
                        x = lds1(raw_dl, (sc * (RB + 2) + (r - lo)) * W + c, P.io_dt);
                    else
                        x = ld_elem(P.delta, (int64_t)b * P.dl_bs + (int64_t)sdd * P.dl_ds + cs +
                                                 (int64_t)(fh ? H - 1 - r : r) * P.dl_hs + (fw ? W - 1 - c : c), P.io_dt);
                    x += spar[2 * (kch0 + sc) + 1];
                    if (P.softplus) x = softplus20(x);
                }
                tdl[sc * CS6 + rr * Wp + pos1<L>(c)] = x;
            }
        }
    };

    if constexpr (WS) {
        if (warp >= WS_COMPUTE / 32) {  // ---- staging warps ----
            asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(WS_REGS_STAGE));
            for (int d = 0; d < ng; ++d) {
                if (d > 0) { set_dir(d); __syncthreads(); }   // the compute warps have refilled the parameter copies
                for (int k = 0; k < steps; ++k) {
                    const int gk = d * steps + k, set = gk & 1;   // tile sets and barrier phases run on across directions
                    if (gk >= 2 && !mbar_wait_bounded_lazy(freeb + set, ((gk >> 1) - 1) & 1)) {
                        atomicOr(P.status, ERR_STAGE_TIMEOUT);  // the compute warps give up on `full` in turn
                        return;
                    }
                    stage_step(k, set ? set1 : smem, nullptr, tid - WS_COMPUTE, WS_STAGE);
                    mbar_arrive(full + set);  // release: the tile writes above are visible to the waiters
                }
                if (d + 1 < ng) __syncthreads();   // end of a direction
            }
            return;
        }
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(WS_REGS_COMPUTE));
    }
    auto cta_sync = [&]() {
        if constexpr (WS) group_sync(1, WS_COMPUTE); else __syncthreads();
    };
    for (int dir = 0; dir < ng; ++dir) {
    if (dir > 0) {   // next direction of a merged launch: fresh accumulators and parameter copies
        set_dir(dir);
        init_dir();
        __syncthreads();
    }
    const int sbase = dir * steps;   // tile sets and barrier phases run on across directions
    for (int step = 0; step <= steps; ++step) {
        const int gs = sbase + step;
        const int blk = nblk - 1 - step / npass, pass = step % npass;  // bottom-up
        const int r0 = blk * RB, nr = step < steps ? min(RB, H - r0) : 0;
        const int ch0 = pass * CP;
        const int pstep = step - 1;
        const int pblk = nblk - 1 - pstep / npass, ppass = pstep % npass;
        const int pr0 = pblk * RB, pnr = step > 0 ? min(RB, H - pr0) : 0, pch0 = ppass * CP;
        // The checkpoint row above this block and the adjoint row below it are private
        // to this thread; fetch them now so that they arrive while phase A runs.
        float4 ck_pre[STRIP / 2], adj_pre[STRIP / 2];
        float2 Araw = bc(0.f);  // this thread's two A values, fetched with them
        {
            const bool ok = nr > 0 && pair_on && ch0 + cp < nch;
            const int dq = dbase + min(ch0 + cp, nch - 1);
            if (nr > 0 && pair_on)
                Araw = f2(__ldg(P.A + dq * P.A_ds + n0 * P.A_ns), n1 < N ? __ldg(P.A + dq * P.A_ds + n1 * P.A_ns) : 0.f);
            const float4 *pk = reinterpret_cast<const float4 *>(
                P.saved + ((((int64_t)b * P.dim + dq) * P.nck + (blk - 1)) * NPp + pp) * Wp + j * STRIP);
            const float4 *pa = reinterpret_cast<const float4 *>(
                P.adj + (((int64_t)b * P.dim + dq) * NPp + pp) * Wp + j * STRIP);
            if (P.ck_pairs) {
                // checkpoints of the streaming forward (single state): one value holds channels 2q, 2q+1
                // of the group
                const int dl_ = dq - g_ * P.dpg;
                const float4 *pq = reinterpret_cast<const float4 *>(
                    P.saved + ((((int64_t)b * P.G + g_) * ((P.dpg + 1) >> 1) + (dl_ >> 1)) * P.nck + (blk - 1)) * Wp + j * STRIP);
#pragma unroll
                for (int k = 0; k < STRIP / 2; ++k) {
                    const float4 v = (ok && r0 > 0) ? __ldg(pq + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                    ck_pre[k] = (dl_ & 1) ? make_float4(v.y, 0.f, v.w, 0.f) : make_float4(v.x, 0.f, v.z, 0.f);
                    adj_pre[k] = (ok && r0 + RB < H) ? pa[k] : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            } else {
#pragma unroll
            for (int k = 0; k < STRIP / 2; ++k) {
                ck_pre[k] = (ok && r0 > 0) ? __ldg(pk + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                adj_pre[k] = (ok && r0 + RB < H) ? pa[k] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            }
        }
        // ---- phase A: write out the previous step, stage this one -------------------
        if (!WS && bulk) {
            if (warp == 0 && step + 1 < steps) issue(step + 1);   // lands while this step computes
            bool ok = nr == 0 || mbar_wait_bounded(bars + (step & 1), (step >> 1) & 1);
            if (__syncthreads_or(!ok)) {  // give up: flag it, drain the other stage, leave
                if (tid == 0) atomicOr(P.status, ERR_BULK_COPY_TIMEOUT);
                if (step + 1 < steps) mbar_wait_bounded(bars + ((step + 1) & 1), ((step + 1) >> 1) & 1);
                return;
            }
        }
        {
            // tiles of the previous step (being written out) and of this one
            float *prev = WS && ((gs - 1) & 1) ? set1 : smem, *cur = WS && (gs & 1) ? set1 : smem;
            const float *psu = prev + S::u(CP), *psg = prev + S::g(CP), *pssig = prev + S::sig(CP);
            su = cur + S::u(CP); sg = cur + S::g(CP); ssig = cur + S::sig(CP); sdl = cur + S::dl(CP);
            const int items = pnr > 0 ? CP * RB * T4 : 0;
            for (int it = tid; it < items; it += nthr) {
                const int t = it % T4, rr = (it / T4) % RB, sc = it / (T4 * RB);
                const int c = 4 * t, o4 = sc * CS4 + rr * Wp + pos4<L>(t);
                float dDp = 0.f, dbp = 0.f;
                if (rr < pnr && pch0 + sc < nch) {
                    const int sd = dbase + pch0 + sc;
                    const int scg = sc / CW, scl = sc % CW;
                    float4 a1 = make_float4(0.f, 0.f, 0.f, 0.f), a2 = a1;
                    for (int q = 0; q < NPp; ++q) {
                        const int o = ((scg * NPp + q) * CW + scl) * CS4 + rr * Wp + pos4<L>(t);
                        const float4 v1 = *reinterpret_cast<const float4 *>(spdu + o);
                        const float4 v2 = *reinterpret_cast<const float4 *>(spdd + o);
                        a1.x += v1.x; a1.y += v1.y; a1.z += v1.z; a1.w += v1.w;
                        a2.x += v2.x; a2.y += v2.y; a2.z += v2.z; a2.w += v2.w;
                    }
                    const float4 gv = *reinterpret_cast<const float4 *>(psg + o4);
                    const float4 uv = *reinterpret_cast<const float4 *>(psu + o4);
                    const float4 sv = *reinterpret_cast<const float4 *>(pssig + o4);
                    const float Dv = spar[2 * (pch0 + sc)];
                    a1.x = fmaf(Dv, gv.x, a1.x); a1.y = fmaf(Dv, gv.y, a1.y);
                    a1.z = fmaf(Dv, gv.z, a1.z); a1.w = fmaf(Dv, gv.w, a1.w);
                    a2.x *= sv.x; a2.y *= sv.y; a2.z *= sv.z; a2.w *= sv.w;
                    const int64_t o = ((int64_t)b * P.dim + sd) * H * P.Wout + cs;
                    if (P.mw) {  // direction merge: the sweep ran on the raw dy; w enters here
                        const float wv = smw[pch0 + sc];
                        a1.x *= wv; a1.y *= wv; a1.z *= wv; a1.w *= wv;
                        a2.x *= wv; a2.y *= wv; a2.z *= wv; a2.w *= wv;
                        const int64_t plane = ((int64_t)b * P.dpg + sd - g_ * P.dpg) * H * P.Wout + cs;
                        if (SERIAL)
                            acc4d(reinterpret_cast<float *>(P.du), plane, P.Wout, pr0 + rr, c, H, W, fh, fw, P.vec & VEC_MDU,
                                  P.merge_store && gi == 0, a1);
                        else
                            red4d(reinterpret_cast<float *>(P.du), plane, P.Wout, pr0 + rr, c, H, W, fh, fw, a1);
                    } else {
                        st4d(P.du, o, P.Wout, pr0 + rr, c, H, W, fh, fw, P.io_dt, P.vec & VEC_DU, a1);
                    }
                    st4d(P.ddelta, o, P.Wout, pr0 + rr, c, H, W, fh, fw, P.io_dt, P.vec & VEC_DU, a2);
                    // columns past the image carry g = 0 and ddl = 0
                    dDp = gv.x * uv.x + gv.y * uv.y + gv.z * uv.z + gv.w * uv.w;
                    dbp = a2.x + a2.y + a2.z + a2.w;
                }
                // the RB*T4 items of a channel are consecutive: segmented warp sum
                constexpr int SEG = S::SEG;
#pragma unroll
                for (int off = SEG / 2; off; off >>= 1) {
                    dDp += __shfl_xor_sync(0xffffffffu, dDp, off);
                    dbp += __shfl_xor_sync(0xffffffffu, dbp, off);
                }
                if ((lane & (SEG - 1)) == 0 && pch0 + sc < nch) {  // the slot's only writer
                    float *q = sred + ((pch0 + sc) * S::NSEG + (it % (RB * T4)) / SEG) * 2;
                    q[0] += dDp;
                    q[1] += dbp;
                }
            }
            if constexpr (WS) {
                // the previous step's tile set may be refilled by the staging warps from here on
                if (step > 0) mbar_arrive(freeb + ((gs - 1) & 1));
            } else {
                // every thread replaces the tile entries it has just read (same item mapping)
                stage_step(step, smem, raw + (size_t)(step & 1) * stage_bytes, tid, nthr);
            }
            // a row block is complete when its last pass has been written out
            if (acc_on && pnr > 0 && ppass == npass - 1) {
                const int itemsB = NPp * RB * Wp;  // one float2 (two states) per item
                for (int it = tid; it < itemsB; it += nthr) {
                    const int c = it % Wp, rr = (it / Wp) % RB, spp = it / (Wp * RB);
                    float2 vb = bc(0.f), vc = bc(0.f);
                    for (int scg = 0; scg < CG; ++scg) {  // the CTA's channel groups, in order
                        const int o = ((scg * NPp + spp) * RB + rr) * Wp + pos2<L>(c);
                        vb = add2(vb, saB[o]); vc = add2(vc, saC[o]);
                        saB[o] = bc(0.f); saC[o] = bc(0.f);
                    }
                    if (c < W && rr < pnr && 2 * spp < N) {
                        const int64_t og = ((((int64_t)b * P.G + g_) * N + 2 * spp) * H + (fh ? H - 1 - (pr0 + rr) : pr0 + rr)) * P.Wout +
                                           (fw ? W - 1 - c : c) + cs;
                        if (P.det) {  // this channel tile's own plane: each element has one writer
                            float *qb = P.dB + (int64_t)tile * P.det_ts + og, *qc = P.dC + (int64_t)tile * P.det_ts + og;
                            qb[0] = vb.x; qc[0] = vc.x;
                            if (2 * spp + 1 < N) { qb[(int64_t)H * P.Wout] = vb.y; qc[(int64_t)H * P.Wout] = vc.y; }
                        } else {
                            atomicAdd(P.dB + og, vb.x);
                            atomicAdd(P.dC + og, vc.x);
                            if (2 * spp + 1 < N) {
                                atomicAdd(P.dB + og + (int64_t)H * P.Wout, vb.y);
                                atomicAdd(P.dC + og + (int64_t)H * P.Wout, vc.y);
                            }
                        }
                    }
                }
            }
            if (nr > 0 && pass == 0) stage_BC<L>(P, b, g_, r0, nr, sB, sC, fh, fw, tid, nthr);
            if (nr > 0 && (has_left || has_right)) {
                for (int it = tid; it < CP * NPp * (RB + 1); it += nthr) {
                    const int k = it % (RB + 1), q = (it / (RB + 1)) % NPp, sc = it / ((RB + 1) * NPp);
                    const int64_t base = (((int64_t)b * P.dim + dbase + ch0 + sc) * NPp + q) * H;
                    float4 e = make_float4(0.f, 0.f, 0.f, 0.f), f = e;
                    if (ch0 + sc < nch) {
                        const int rl = r0 - 1 + k, rr2 = r0 + k;
                        if (has_left && rl >= 0 && rl < H) e = __ldg(P.edge_in + base + rl);
                        if (has_right && rr2 < H) f = P.adj_in[base + rr2];
                    }
                    sedge[it] = e; sadj[it] = f;
                }
                for (int it = tid; it < CP * 8; it += nthr) {
                    const int k = it % 8, sc = it / 8;
                    float xl = 0.f, xr = 0.f;
                    if (ch0 + sc < nch) {
                        const int sdd = (dbase + ch0 + sc) / P.drep;
                        const float bv = P.bias ? __ldg(P.bias + sdd) : 0.f;
                        const int64_t row0 = (int64_t)b * P.dl_bs + (int64_t)sdd * P.dl_ds + cs +
                                             (int64_t)(fh ? H - 1 - (r0 + k) : r0 + k) * P.dl_hs;
                        if (has_left && k < nr) {   // scan column -1
                            xl = ld_elem(P.delta, row0 + (fw ? W : -1), P.io_dt) + bv;
                            if (P.softplus) xl = softplus20(xl);
                        }
                        if (has_right && k <= RB && r0 + k < H) {
                            xr = ld_elem(P.delta, row0 + (fw ? -1 : W), P.io_dt) + bv;   // scan column W
                            if (P.softplus) xr = softplus20(xr);
                        }
                    }
                    if (k < RB) sedl_l[sc * 4 + k] = xl;
                    sedl_r[sc * 8 + k] = xr;
                }
            }
        }
        if constexpr (WS) {  // this step's tiles have to be complete
            const bool ok = nr == 0 || mbar_wait_bounded(full + (gs & 1), (gs >> 1) & 1);
            if (group_or(2, WS_COMPUTE, !ok)) {  // the staging warps stopped (they flagged why): leave together
                if (tid == 0) atomicOr(P.status, ERR_STAGE_TIMEOUT);
                return;
            }
        }
        cta_sync();
        if (nr == 0) break;

        // ---- compute ---------------------------------------------------------------------
        if (pair_on) {
            const bool ch_ok = ch0 + cp < nch;
            const int d = dbase + min(ch0 + cp, nch - 1);
            const float2 A2 = mul2(Araw, bc(LOG2E));
            const float *dlc = sdl + cp * CS6;
            // The recomputed h rows are parked in this thread's own slots of the partial
            // tiles: a row of h (8 x float2) is exactly the size of the du and ddl
            // partial sums (8 + 8 floats) that replace it once the reverse sweep has
            // consumed the row.  Only the row above the block stays in registers.
            float *slot_u = spdu + (warp * CW + cl) * CS4, *slot_d = spdd + (warp * CW + cl) * CS4;
            float2 htop[STRIP];
            // -- recompute h for the block from the checkpoint row --
            {
                float2 a_up[STRIP], hprev[STRIP];
                if (r0 > 0) {
                    float dlt[STRIP];
                    unpack8(dlc, L4, j, dlt);
#pragma unroll
                    for (int k = 0; k < STRIP / 2; ++k) {
                        htop[2 * k] = f2(ck_pre[k].x, ck_pre[k].y); htop[2 * k + 1] = f2(ck_pre[k].z, ck_pre[k].w);
                    }
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) a_up[i] = ex2_2(fma2(bc(dlt[i]), A2, lgd));
                } else {
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) { htop[i] = bc(0.f); a_up[i] = bc(0.f); }
                }
#pragma unroll
                for (int i = 0; i < STRIP; ++i) hprev[i] = htop[i];
#pragma unroll
                for (int rr = 0; rr < RB; ++rr) {
                    {   // rows past the image are staged as zeros and carry zero adjoints
                        float dl[STRIP], uu[STRIP], dlu[STRIP];
                        float2 Bv[STRIP];
                        unpack8(su + cp * CS4 + rr * Wp, L4, j, uu);
                        unpack8(dlc + (rr + 1) * Wp, L4, j, dl);
#pragma unroll
                        for (int i = 0; i < STRIP; ++i) dlu[i] = dl[i] * uu[i];
                        unpack8x2(sB + (pp * RB + rr) * Wp, L2, j, Bv);
                        float2 a[STRIP], p[STRIP], hcur[STRIP], sdummy[STRIP];
                        LeftEdge le = {bc(0.f), bc(0.f), bc(0.f), bc(0.f)};
                        if (has_left && j == 0) {
                            const float4 e0 = sedge[(cp * NPp + pp) * (RB + 1) + rr];
                            const float4 e1 = sedge[(cp * NPp + pp) * (RB + 1) + rr + 1];
                            le.h_prev = f2(e0.x, e0.y); le.h = f2(e1.x, e1.y);
                            le.a = ex2_2(fma2(bc(sedl_l[cp * 4 + rr]), A2, lgd));
                        }
                        row_forward<L, false>(j, dl, dlu, Bv, A2, lgd, hprev, a_up, a, p, hcur, sdummy, has_left, le);
                        park8x2(slot_u + rr * Wp, slot_d + rr * Wp, L4, j, hcur);
#pragma unroll
                        for (int i = 0; i < STRIP; ++i) { a_up[i] = a[i]; hprev[i] = hcur[i]; }
                    }
                }
            }
            // -- adjoint row below the block --
            float2 m_dn[STRIP], a_dn[STRIP];
            float2 *adj = P.adj + (((int64_t)b * P.dim + d) * NPp + pp) * Wp + j * STRIP;
            if (r0 + RB < H) {
                float dlt[STRIP];
                unpack8(dlc + (RB + 1) * Wp, L4, j, dlt);
#pragma unroll
                for (int k = 0; k < STRIP / 2; ++k) {
                    m_dn[2 * k] = f2(adj_pre[k].x, adj_pre[k].y); m_dn[2 * k + 1] = f2(adj_pre[k].z, adj_pre[k].w);
                }
#pragma unroll
                for (int i = 0; i < STRIP; ++i) a_dn[i] = ex2_2(fma2(bc(dlt[i]), A2, lgd));
            } else {
#pragma unroll
                for (int i = 0; i < STRIP; ++i) { m_dn[i] = bc(0.f); a_dn[i] = bc(0.f); }
            }
            float2 dAacc = bc(0.f), dwacc = bc(0.f);
            const float wv = smw[min(ch0 + cp, CT - 1)];   // 1 unless directions are merged
            // -- reverse sweep over the block --
            float2 hrow[STRIP], hup[STRIP];
            fetch8x2(slot_u + (RB - 1) * Wp, slot_d + (RB - 1) * Wp, L4, j, hrow);
#pragma unroll
            for (int rr = RB - 1; rr >= 0; --rr) {
                {
                    float dl[STRIP], uu[STRIP], gg[STRIP];
                    float2 Bv[STRIP], Cv[STRIP];
                    unpack8(su + cp * CS4 + rr * Wp, L4, j, uu);
                    unpack8(sg + cp * CS4 + rr * Wp, L4, j, gg);
                    unpack8(dlc + (rr + 1) * Wp, L4, j, dl);
                    unpack8x2(sB + (pp * RB + rr) * Wp, L2, j, Bv);
                    unpack8x2(sC + (pp * RB + rr) * Wp, L2, j, Cv);
                    if (rr > 0) {
                        fetch8x2(slot_u + (rr - 1) * Wp, slot_d + (rr - 1) * Wp, L4, j, hup);
                    } else {
#pragma unroll
                        for (int i = 0; i < STRIP; ++i) hup[i] = htop[i];
                    }
                    float2 a[STRIP], p[STRIP], s[STRIP], gC[STRIP];
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) {
                        a[i] = ex2_2(fma2(bc(dl[i]), A2, lgd));
                        p[i] = mul2(Bv[i], bc(dl[i] * uu[i]));
                        gC[i] = mul2(Cv[i], bc(gg[i]));
                    }
                    float2 a_r7 = bc(0.f), mdr7 = bc(0.f);  // next lane's first column
                    if constexpr (L > 1) {
                        a_r7 = shfl_down2<L>(a[0], 1);
                        mdr7 = shfl_down2<L>(m_dn[0], 1);
                        const bool last = j == L - 1;
                        a_r7.x = last ? 0.f : a_r7.x; a_r7.y = last ? 0.f : a_r7.y;
                        mdr7.x = last ? 0.f : mdr7.x; mdr7.y = last ? 0.f : mdr7.y;
                    }
                    // first column of the tile to the right (full tiles end at lane L-1's last column)
                    float2 e_dh = bc(0.f), e_ds = bc(0.f);
                    if (has_right && j == L - 1) {
                        const float4 e0 = sadj[(cp * NPp + pp) * (RB + 1) + rr], e1 = sadj[(cp * NPp + pp) * (RB + 1) + rr + 1];
                        e_dh = f2(e0.x, e0.y); e_ds = f2(e0.z, e0.w);
                        a_r7 = ex2_2(fma2(bc(sedl_r[cp * 8 + rr]), A2, lgd));
                        // m(r+1, c_end) = a(r+1, c_end) * dh(r+1, c_end); zero below the image
                        mdr7 = r0 + rr + 1 < H ? mul2(ex2_2(fma2(bc(sedl_r[cp * 8 + rr + 1]), A2, lgd)), f2(e1.x, e1.y))
                                               : bc(0.f);
                    }
                    // Three scans share this row: s forward (recomputed plain row scan), dh and ds
                    // reverse with multipliers a(r,c+1).  They are independent, so they are folded
                    // together, each as two 4-column half chains.
                    float2 bt[STRIP], dh[STRIP], ds[STRIP];
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) {
                        const float2 ar = i < STRIP - 1 ? a[i + 1] : a_r7;
                        const float2 mdr = i < STRIP - 1 ? m_dn[i + 1] : mdr7;
                        bt[i] = fma2(mul2(add2(ar, a_dn[i]), mdr), bc(-0.5f), add2(gC[i], m_dn[i]));
                    }
                    {
                        constexpr int HS = STRIP / 2;
                        // forward halves: columns 0..3 and 4..7; reverse halves: 7..4 and 3..0
                        float2 Pf0 = a[0], Pf1 = a[HS], S0 = p[0], S1 = p[HS];
                        float2 Pr0 = a_r7, Pr1 = a[HS], H0 = bt[STRIP - 1], H1 = bt[HS - 1];
                        float2 D0 = neg2(gC[STRIP - 1]), D1 = neg2(gC[HS - 1]);
#pragma unroll
                        for (int k = 1; k < HS; ++k) {
                            S0 = fma2(a[k], S0, p[k]); Pf0 = mul2(Pf0, a[k]);
                            S1 = fma2(a[HS + k], S1, p[HS + k]); Pf1 = mul2(Pf1, a[HS + k]);
                            const float2 ar0 = a[STRIP - k];  // multiplier of column 7-k is a of column 8-k
                            const float2 ar1 = a[HS - k];
                            H0 = fma2(ar0, H0, bt[STRIP - 1 - k]); D0 = fma2(ar0, D0, neg2(gC[STRIP - 1 - k]));
                            H1 = fma2(ar1, H1, bt[HS - 1 - k]); D1 = fma2(ar1, D1, neg2(gC[HS - 1 - k]));
                            Pr0 = mul2(Pr0, ar0); Pr1 = mul2(Pr1, ar1);
                        }
                        float2 cs, unused, cdh, cds, Pfin, Prin;
                        carry_fwd<L, false>(j, mul2(Pf0, Pf1), fma2(Pf1, S0, S1), bc(0.f), cs, unused, Pfin);
                        carry_rev<L, true>(j, mul2(Pr0, Pr1), fma2(Pr1, H0, H1), fma2(Pr1, D0, D1), cdh, cds, Prin);
                        if (has_right) {  // dh, ds of the column right of the tile reach every lane
                            cdh = add2(cdh, edge_term_rev<L>(j, Prin, e_dh));
                            cds = add2(cds, edge_term_rev<L>(j, Prin, e_ds));
                        }
                        if (has_left) {   // s of the column left of the tile
                            float2 e_s = bc(0.f);
                            if (j == 0) {
                                const float4 e1 = sedge[(cp * NPp + pp) * (RB + 1) + rr + 1];
                                e_s = f2(e1.z, e1.w);
                            }
                            cs = add2(cs, edge_term_fwd<L>(j, Pfin, e_s));
                        }
                        float2 cs1 = fma2(Pf0, cs, S0);                           // into columns 4..7
                        float2 cdh1 = fma2(Pr0, cdh, H0), cds1 = fma2(Pr0, cds, D0);  // into columns 3..0
#pragma unroll
                        for (int k = 0; k < HS; ++k) {
                            cs = fma2(a[k], cs, p[k]); s[k] = cs;
                            cs1 = fma2(a[HS + k], cs1, p[HS + k]); s[HS + k] = cs1;
                            const float2 ar0 = k ? a[STRIP - k] : a_r7;
                            const float2 ar1 = a[HS - k];
                            cdh = fma2(ar0, cdh, bt[STRIP - 1 - k]); dh[STRIP - 1 - k] = cdh;
                            cds = fma2(ar0, cds, neg2(gC[STRIP - 1 - k])); ds[STRIP - 1 - k] = cds;
                            cdh1 = fma2(ar1, cdh1, bt[HS - 1 - k]); dh[HS - 1 - k] = cdh1;
                            cds1 = fma2(ar1, cds1, neg2(gC[HS - 1 - k])); ds[HS - 1 - k] = cds1;
                        }
                    }
                    float2 m[STRIP];
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) m[i] = mul2(a[i], dh[i]);
                    float2 m_r7 = bc(0.f), h_l0 = bc(0.f);
                    if constexpr (L > 1) {
                        m_r7 = shfl_down2<L>(m[0], 1);
                        h_l0 = shfl_up2<L>(hrow[STRIP - 1], 1);
                        m_r7.x = j == L - 1 ? 0.f : m_r7.x; m_r7.y = j == L - 1 ? 0.f : m_r7.y;
                        h_l0.x = j == 0 ? 0.f : h_l0.x; h_l0.y = j == 0 ? 0.f : h_l0.y;
                    }
                    if (has_right && j == L - 1) m_r7 = mul2(a_r7, e_dh);
                    if (has_left && j == 0) {
                        const float4 e1 = sedge[(cp * NPp + pp) * (RB + 1) + rr + 1];
                        h_l0 = f2(e1.x, e1.y);
                        if (ch_ok && r0 + rr < H)  // dh, ds of this tile's first column for the tile to the left
                            P.adj_out[(((int64_t)b * P.dim + d) * NPp + pp) * H + r0 + rr] =
                                make_float4(dh[0].x, dh[0].y, ds[0].x, ds[0].y);
                    }
                    float duv[STRIP], ddv[STRIP];
                    // dB/dC are summed over the warp's CW channels by transposing through
                    // shared memory (each lane then adds up NU columns) and accumulated over
                    // passes in the warp's private tile.  Column i is rotated by its owner
                    // so that the owners' reads hit distinct banks.
                    float2 *trB = str + warp * 512, *trC = trB + 256;
                    float2 *accB = saB + (warp * RB + rr) * Wp, *accC = saC + (warp * RB + rr) * Wp;
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
                        duv[i] = dl[i] * S1;
                        ddv[i] = fmaf(uu[i], S1, t2.x + t2.y);
                        dAacc = fma2(bc(dl[i]), G, dAacc);
                        ddecay_acc = fma2(bc(wv), Gh, ddecay_acc);   // only read when dA_decay is wanted (wv: merge weight or 1)
                        const float2 dBv = mul2(bc(dl[i] * uu[i] * wv), eps);
                        const float2 yt = fma2(p[i], bc(0.25f), sub2(hrow[i], s[i]));
                        const float2 dCv = mul2(bc(gg[i] * wv), yt);
                        dwacc = fma2(gC[i], yt, dwacc);   // dy * (C*(h - s + p/4)): this pair's share of dy*y (read when merging)
                        if constexpr (CW == 1) {
                            if (acc_on) {
                                float2 *qb = accB + pos2<L>(j * STRIP + i), *qc = accC + pos2<L>(j * STRIP + i);
                                *qb = add2(*qb, dBv);
                                *qc = add2(*qc, dCv);
                            } else if (ch_ok && j * STRIP + i < W) {
                                const int64_t og = ((((int64_t)b * P.G + g_) * N + n0) * H + (fh ? H - 1 - (r0 + rr) : r0 + rr)) * P.Wout +
                                                   (fw ? W - 1 - (j * STRIP + i) : j * STRIP + i) + cs;
                                add_dbc(P, tile, og, n1 < N, dBv, dCv);
                            }
                        } else {
                            const int o = i * 32 + ((lane + L * (i / NU)) & 31);
                            trB[o] = dBv;
                            trC[o] = dCv;
                        }
                    }
                    // sums over the state pairs: per-warp partial tiles, added up at write-out
                    pack8(spdu + (warp * CW + cl) * CS4 + rr * Wp, L4, j, duv);
                    pack8(spdd + (warp * CW + cl) * CS4 + rr * Wp, L4, j, ddv);
                    if constexpr (CW > 1) {
                        __syncwarp();
                        if (cl < 8) {
                            const int my = CW >= 8 ? cl : cl * NU;  // first owned column
#pragma unroll
                            for (int t = 0; t < NU; ++t) {
                                const int col = my + t;
                                float2 sb = bc(0.f), sc2 = bc(0.f);
#pragma unroll
                                for (int c2 = 0; c2 < CW; ++c2) {
                                    const int o = col * 32 + ((c2 * L + j + L * (col / NU)) & 31);
                                    sb = add2(sb, trB[o]);
                                    sc2 = add2(sc2, trC[o]);
                                }
                                if (acc_on) {
                                    float2 *qb = accB + pos2<L>(j * STRIP + col), *qc = accC + pos2<L>(j * STRIP + col);
                                    *qb = add2(*qb, sb);
                                    *qc = add2(*qc, sc2);
                                } else if (j * STRIP + col < W) {
                                    const int64_t og =
                                        ((((int64_t)b * P.G + g_) * N + n0) * H + (fh ? H - 1 - (r0 + rr) : r0 + rr)) * P.Wout +
                                        (fw ? W - 1 - (j * STRIP + col) : j * STRIP + col) + cs;
                                    add_dbc(P, tile, og, n1 < N, sb, sc2);
                                }
                            }
                        }
                        __syncwarp();
                    }
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) { m_dn[i] = m[i]; a_dn[i] = a[i]; hrow[i] = hup[i]; }
                }
            }
            if (r0 > 0 && ch_ok) {  // park the adjoint row for the block above
                float4 *pk = reinterpret_cast<float4 *>(adj);
#pragma unroll
                for (int k = 0; k < STRIP / 2; ++k)
                    pk[k] = make_float4(m_dn[2 * k].x, m_dn[2 * k].y, m_dn[2 * k + 1].x, m_dn[2 * k + 1].y);
            }
            if constexpr (L > 1) {
#pragma unroll
                for (int off = L / 2; off; off >>= 1) {
                    dAacc = add2(dAacc, shfl_xor2<L>(dAacc, off));
                    dwacc = add2(dwacc, shfl_xor2<L>(dwacc, off));
                }
            }
            if (j == 0 && ch_ok) {  // one owner per (channel, pair): no atomics needed
                float *q = sdA + (ch0 + cp) * 2 * NPp + 2 * pp;
                q[0] += dAacc.x; q[1] += dAacc.y;
                sdw[(ch0 + cp) * NPp + pp] += dwacc.x + dwacc.y;
            }
        }
        cta_sync();
    }

    // ---- per-channel parameter gradients ---------------------------------------
    if (want_decay) {
        float v = ddecay_acc.x + (n1 < N ? ddecay_acc.y : 0.f);
        if (!pair_on) v = 0.f;
#pragma unroll
        for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) sdecay[warp] = v;
    }
    cta_sync();
    // deterministic mode: this batch entry's own slots instead of atomics onto the results
    const int64_t slot = P.det ? (int64_t)b * P.dim : 0;
    for (int i = tid; i < nch * 2 * NPp; i += nthr) {
        const int sc = i / (2 * NPp), n = i % (2 * NPp);
        if (n < N) {
            float *q = P.dA + (slot + dbase + sc) * N + n;
            const float v = sdA[i] * smw[sc];
            if (P.det) *q = v; else atomicAdd(q, v);
        }
    }
    for (int i = tid; i < nch * 2; i += nthr) {
        const int sd = dbase + i / 2;
        float v = 0.f;
        for (int q = 0; q < S::NSEG; ++q) v += sred[((i / 2) * S::NSEG + q) * 2 + (i & 1)];
        // dD slots hold sum dy*u of the raw gradient: dD = w*that, and D*that is dw's D*u share
        if ((i & 1) == 0) {
            if (P.mw && P.dw) {
                float dwv = spar[i] * v;
                for (int q = 0; q < NPp; ++q) dwv += sdw[(i / 2) * NPp + q];
                atomicAdd(P.dw + sd, dwv);
            }
            v *= smw[i / 2];
        }
        float *q = (i & 1) == 0 ? P.dD : P.dbias;
        if (q) { if (P.det) q[slot + sd] = v; else atomicAdd(q + sd, v); }
    }
    if (want_decay && tid == 0) {
        float v = 0.f;
        for (int w = 0; w < nw; ++w) v += sdecay[w];
        if (P.det) P.ddecay[blockIdx.x] = v / decay; else atomicAdd(P.ddecay, v / decay);
    }
    if (dir + 1 < ng) __syncthreads();   // end of a direction: its share of the merged du image is written
    }
}

#if !CS2D_SERIAL_DIRS
template <int L>
static size_t smem_floats(int CP, int NPp, int CT, int nw, bool acc, bool ws) {
    return (size_t)((BwdSmem<L>::total(CP, NPp, CT, nw, acc) + 3) & ~3) + (ws ? BwdSmem<L>::set_floats(CP) : 0);
}

size_t bwd_smem_bytes(int L, int CG, int NPp, int CT, bool acc, int W, int es, int eso, bool bulk, bool tiled, bool ws) {
    const int nw = CG * NPp;
    const int CP = CG * (32 / L);
    // after the tiles: tile-edge areas (tiled kernels), the mbarriers, then either the raw row
    // blocks of the bulk copies (two stages) or, warp-specialised, the second tile set
    const size_t extra = (size_t)(tiled ? 2 * CP * NPp * (RB + 1) * 4 + CP * 12 : 0) * 4 + (ws ? 32 : 16) +
                         (bulk && !ws ? 2 * (size_t)CP * W * (RB * es + RB * eso + (RB + 2) * es) : 0);
    switch (L) {
        case 1: return smem_floats<1>(CP, NPp, CT, nw, acc, ws) * 4 + extra;
        case 2: return smem_floats<2>(CP, NPp, CT, nw, acc, ws) * 4 + extra;
        case 4: return smem_floats<4>(CP, NPp, CT, nw, acc, ws) * 4 + extra;
        case 8: return smem_floats<8>(CP, NPp, CT, nw, acc, ws) * 4 + extra;
        case 16: return smem_floats<16>(CP, NPp, CT, nw, acc, ws) * 4 + extra;
        default: return smem_floats<32>(CP, NPp, CT, nw, acc, ws) * 4 + extra;
    }
}

#else
size_t bwd_smem_bytes(int L, int CG, int NPp, int CT, bool acc, int W, int es, int eso, bool bulk, bool tiled, bool ws);
#endif

template <int L, int NPC, bool TILED, bool WS>
static cudaError_t launch(const Dev &P, int grid, size_t smem, cudaStream_t st) {
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(bwd_kernel<L, NPC, TILED, WS, SERIAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    bwd_kernel<L, NPC, TILED, WS, SERIAL><<<grid, WS ? WS_COMPUTE + WS_STAGE : 32 * P.CG * P.NPp, smem, st>>>(P);
    return cudaGetLastError();
}

template <int L>
static cudaError_t launch_L(const Dev &P, int grid, size_t smem, cudaStream_t st) {
    const bool spec = P.NPp == 8 && P.CG == 1, tiled = P.tile_left || P.tile_right;
    if (P.ws) return tiled ? launch<L, 8, true, true>(P, grid, smem, st) : launch<L, 8, false, true>(P, grid, smem, st);
    return tiled ? (spec ? launch<L, 8, true, false>(P, grid, smem, st) : launch<L, 0, true, false>(P, grid, smem, st))
                 : (spec ? launch<L, 8, false, false>(P, grid, smem, st) : launch<L, 0, false, false>(P, grid, smem, st));
}

#if CS2D_SERIAL_DIRS
cudaError_t launch_bwd_serial(const Dev &P, int L, int grid, cudaStream_t st) {
#else
cudaError_t launch_bwd(const Dev &P, int L, int grid, cudaStream_t st) {
#endif
    const bool tiled = P.tile_left || P.tile_right;
    if (P.ws && (P.NPp != 8 || P.CG != 1)) return cudaErrorInvalidValue;
    const size_t smem = bwd_smem_bytes(L, P.CG, P.NPp, P.CT, P.acc_dbc != 0, P.W, P.io_dt == CS2D_F32 ? 4 : 2,
                                       P.out_dt == CS2D_F32 ? 4 : 2, P.bulk != 0, tiled, P.ws != 0);
    switch (L) {
        case 1: return launch_L<1>(P, grid, smem, st);
        case 2: return launch_L<2>(P, grid, smem, st);
        case 4: return launch_L<4>(P, grid, smem, st);
        case 8: return launch_L<8>(P, grid, smem, st);
        case 16: return launch_L<16>(P, grid, smem, st);
        case 32: return launch_L<32>(P, grid, smem, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cs2d

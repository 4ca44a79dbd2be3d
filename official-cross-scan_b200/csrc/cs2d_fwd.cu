// Forward 2D-CrossScan selective scan (sm_100a).
//
// Replaces selective_scan_fwd_kernel of the reference
// (include/cusoflex/selective_scan_fwd_kernel_oflex.cuh:80-357):
//   dl = softplus(delta + bias);  a = exp(dl*A)*A_decay;  p = B*dl*u
//   h(r,c) = a*(h(r,c-1) + h(r-1,c) - 0.5*(a(r-1,c)+a(r,c-1))*h(r-1,c-1)) + p
//   s(r,c) = a*s(r,c-1) + p
//   y      = D*u + sum_n C_n*(h_n - s_n + 0.25*p_n)
// One CTA owns CT channels of one (batch, group) and walks them in passes of CP
// channels per block of RB rows; B and C are staged once per row block for all
// of them.  The last h row of every block is written to the saved-state buffer:
// it is the checkpoint the backward starts from and the state this kernel
// itself reloads when it comes back to the channel for the next row block.
#include "cs2d_common.cuh"

// This file is compiled twice: as it is (every group of a launch is served by CTAs of its own), and
// from cs2d_fwd_serial.cu with CS2D_SERIAL_DIRS = 1 (the reproducible direction merge: one CTA walks all
// groups of its channel tile).  The choice is a compile-time constant so that the common form carries
// no trace of the loop over directions.
#ifndef CS2D_SERIAL_DIRS
#define CS2D_SERIAL_DIRS 0
#endif

namespace cs2d {
constexpr bool SERIAL = CS2D_SERIAL_DIRS != 0;

template <int L>
struct FwdSmem {
    static constexpr int Wp = L * STRIP, CW = 32 / L;
    static constexpr int CS4 = chan_stride<L>(RB), CS5 = chan_stride<L>(RB + 1);
    // float offsets
    static __host__ __device__ constexpr int u(int) { return 0; }
    static __host__ __device__ constexpr int dl(int CP) { return CP * CS4; }
    static __host__ __device__ constexpr int y(int CP) { return dl(CP) + CP * CS5; }            // [warps][CW][CS4]
    static __host__ __device__ constexpr int B(int CP, int nw) { return y(CP) + nw * CW * CS4; }  // float2 tiles
    static __host__ __device__ constexpr int total(int CP, int NPp, int nw) {
        return B(CP, nw) + 2 * 2 * NPp * RB * Wp;
    }
    // after the tiles: two mbarriers (4 floats), then two stages of raw row blocks
    // (u: RB rows, delta: RB+1 rows per channel, in the input dtype)
    // left-edge values of a column tile: [CP][NPp][RB+1] float4 (h, s of rows r0-1..r0+RB-1)
    // and the softplus'd delta of the column left of the tile [CP][RB] (padded to 4 floats)
    // (both only exist in the kernels that handle column tiles)
    static __host__ __device__ constexpr int edge(int CP, int NPp, int nw) { return total(CP, NPp, nw); }
    static __host__ __device__ constexpr int edl(int CP, int NPp, int nw, bool tiled) {
        return edge(CP, NPp, nw) + (tiled ? CP * NPp * (RB + 1) * 4 : 0);
    }
    // D and delta_bias of the CTA's CT channels: [CT][2], padded to 16 bytes
    static __host__ __device__ constexpr int par(int CP, int NPp, int nw, bool tiled) {
        return edl(CP, NPp, nw, tiled) + (tiled ? CP * 4 : 0);
    }
    static __host__ __device__ constexpr int bars(int CP, int NPp, int nw, bool tiled, int CT) {
        return par(CP, NPp, nw, tiled) + ((3 * CT + 3) & ~3);   // D, delta_bias, merge weight
    }
    static __host__ __device__ constexpr int raw(int CP, int NPp, int nw, bool tiled, int CT) {
        return bars(CP, NPp, nw, tiled, CT) + 4;
    }
    static __host__ __device__ constexpr int stage_bytes(int CP, int W, int es) { return CP * (2 * RB + 1) * W * es; }
    // one set of staged per-channel tiles (u, delta), rounded to 16 bytes
    static __host__ __device__ constexpr int set_floats(int CP) { return (y(CP) + 3) & ~3; }
};

// NPC = 8 specialises the common geometry (8 state-pair slots, one channel group, 8 warps) so
// that every shared-memory offset is a compile-time constant; NPC = 0 reads it from P.
// TILED compiles the column-tile edge handling in; the common single-tile launch leaves it out.
// WS (with NPC = 8) is the warp-specialised form: warps 0-7 compute and write out the
// previous step, warps 8-11 load and transform (softplus) the tiles of the NEXT step into a
// second tile set meanwhile; the groups meet on mbarriers (tile set full / free), every wait
// bounded, and the staging warps give registers to the compute warps (setmaxnreg).  Two such
// CTAs share an SM: 2 * (256 * 104 + 128 * 32) registers.
constexpr int FWS_COMPUTE = 256, FWS_STAGE = 128, FWS_REGS_COMPUTE = 104, FWS_REGS_STAGE = 32;
// SER = SERIAL: part of the kernel's name, so that the two compilations of this file define distinct kernels
template <int L, int NPC, bool TILED, bool WS, bool SER>
__global__ void __launch_bounds__(WS ? FWS_COMPUTE + FWS_STAGE : MAX_THREADS, 2) fwd_kernel(const Dev P) {
    static_assert(!WS || NPC == 8, "the warp-specialised form covers the common geometry only");
    using S = FwdSmem<L>;
    constexpr int Wp = S::Wp, CW = S::CW, T4 = Wp / 4, CS4 = S::CS4, CS5 = S::CS5, L4 = 4 * L, L2 = 2 * L;
    extern __shared__ __align__(16) float smem[];
    const int NPp = NPC ? NPC : P.NPp, CG = NPC ? MAX_WARPS / NPC : P.CG, CP = CG * CW;
    const int nw = NPp * CG, nthr = nw * 32;
    float *su = smem + S::u(CP);
    float *sdl = smem + S::dl(CP);   // row 0 = row above the block
    float *sy = smem + S::y(CP);     // per-warp partial sums over the warp's state pair
    float2 *sB = reinterpret_cast<float2 *>(smem + S::B(CP, nw));
    float2 *sC = sB + NPp * RB * Wp;
    float4 *sedge = reinterpret_cast<float4 *>(smem + S::edge(CP, NPp, nw));
    float *sedl = smem + S::edl(CP, NPp, nw, TILED);
    float *spar = smem + S::par(CP, NPp, nw, TILED);
    const bool has_left = TILED && P.tile_left != 0;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int j = lane & (L - 1), cl = lane / L;
    const int pp = warp % NPp, cg = warp / NPp;
    const int cp = cg * CW + cl;  // channel slot inside a pass
    const int tile = blockIdx.x % P.ntiles, bg = blockIdx.x / P.ntiles;
    // Normally a CTA serves one group (scan direction).  With Dev::dir_serial (the reproducible direction
    // merge) it owns its channel tile for ALL groups and walks them one after the other: the merged image
    // is then written by this CTA alone - stored by the first direction, read-modify-written by the others
    // in a fixed order, no atomics - and the barriers between the directions order those accesses.
    const int ng = SERIAL ? P.G : 1;
    const int b = SERIAL ? bg : bg / P.G;
    int g = 0, ush = 0, dbase = 0, nch = 0, gi = 0;
    bool fh = false, fw = false;
    int64_t cs = 0;
    auto set_dir = [&](int i) {
        gi = i;
        g = SERIAL ? i : bg % P.G;
        fh = (P.flip_h >> g) & 1u; fw = (P.flip_w >> g) & 1u;   // scan direction of this group
        ush = (P.u_shared & 1) ? g * P.dpg : 0;                    // u is indexed by channel - ush
        cs = fw ? P.cshift : 0;                                    // see Dev::cshift
        dbase = g * P.dpg + tile * P.CT;
        nch = min(P.CT, (g + 1) * P.dpg - dbase);                  // valid channels of this CTA
    };
    set_dir(0);
    const int H = P.H, W = P.W, N = P.N;
    const int n0 = 2 * pp, n1 = n0 + 1;
    const bool pair_on = n0 < N;  // warp-uniform
    const float lgdv = P.decay ? log2f(__ldg(P.decay)) : 0.f;
    const float2 lgd = bc(lgdv);

    // the partial tiles of idle pair slots are summed too: keep them zero
    for (int i = tid; i < nw * CW * CS4; i += nthr) sy[i] = 0.f;
    auto fill_par = [&]() {  // D, delta_bias and merge weight of this CTA's channels in the current direction
        for (int i = tid; i < nch; i += nthr) {
            spar[2 * i] = P.D ? __ldg(P.D + dbase + i) : 0.f;
            spar[2 * i + 1] = P.bias ? __ldg(P.bias + (dbase + i) / P.drep) : 0.f;
            spar[2 * P.CT + i] = P.mw ? __ldg(P.mw + dbase + i) : 1.f;
        }
    };
    fill_par();

    const int nblk = P.nck;
    const int steps = nblk * P.npass;
    // rows of the state buffer per (batch, channel): every block's last h row when a backward
    // will follow, one rolling row otherwise
    const int ckn = P.ck_roll ? 1 : nblk;

    // Bulk asynchronous staging: the raw row blocks of u and delta of step k+1 are
    // copied global -> shared by the copy engine while step k computes; an mbarrier
    // per stage counts the bytes.  One thread issues, everybody waits (bounded).
    const bool bulk = P.bulk != 0;
    const int es = P.io_dt == CS2D_F32 ? 4 : 2;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S::bars(CP, NPp, nw, TILED, P.CT));
    unsigned char *raw = reinterpret_cast<unsigned char *>(smem + S::raw(CP, NPp, nw, TILED, P.CT));
    const int stage_bytes = S::stage_bytes(CP, W, es);
    auto issue = [&](int k) {  // called by every lane of warp 0: one copy per lane and round
        const int kblk = k / P.npass, kpass = k % P.npass;
        const int kr0 = kblk * RB, knr = min(RB, H - kr0), kch0 = kpass * CP;
        const int lo = max(kr0 - 1, 0), nrows_dl = kr0 + knr - lo;
        const int nv = max(0, min(CP, nch - kch0));
        uint64_t *bar = bars + (k & 1);
        unsigned char *ru = raw + (size_t)(k & 1) * stage_bytes, *rd = ru + (size_t)CP * RB * W * es;
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)(nv * (knr + nrows_dl) * W * es));
        __syncwarp();
        for (int i = lane; i < 2 * nv; i += 32) {
            const int sc = i >> 1, sd = dbase + kch0 + sc;
            if ((i & 1) == 0) {
                bulk_g2s(ru + (size_t)sc * RB * W * es,
                         reinterpret_cast<const char *>(P.u) + ((int64_t)b * P.u_bs + (int64_t)sd * P.u_ds + (int64_t)kr0 * W) * es,
                         (uint32_t)(knr * W * es), bar);
            } else {
                bulk_g2s(rd + (size_t)sc * (RB + 1) * W * es,
                         reinterpret_cast<const char *>(P.delta) +
                             ((int64_t)b * P.dl_bs + (int64_t)(sd / P.drep) * P.dl_ds + (int64_t)lo * W) * es,
                         (uint32_t)(nrows_dl * W * es), bar);
            }
        }
    };
    // WS: second tile set and the full / free mbarriers of the two sets
    float *set1 = reinterpret_cast<float *>(bars + 4);
    uint64_t *full = bars, *freeb = bars + 2;
    if (WS) {
        if (tid == 0) {
            mbar_init(full, FWS_STAGE); mbar_init(full + 1, FWS_STAGE);
            mbar_init(freeb, FWS_COMPUTE); mbar_init(freeb + 1, FWS_COMPUTE);
            mbar_init_fence();
        }
    } else if (bulk && tid == 0) {
        mbar_init(bars, 1); mbar_init(bars + 1, 1); mbar_init_fence();
    }
    __syncthreads();  // barriers initialised, parameter copies and zeroed tiles visible
    if (!WS && bulk && warp == 0 && steps > 0) issue(0);

    // loads and transforms u and delta of step k into the tile set at `base`
    auto stage_step = [&](int k, float *base, const unsigned char *raw_k, int t0, int nt) {
        float *tu = base + S::u(CP), *tdl = base + S::dl(CP);
        const int kblk = k / P.npass, kch0 = (k % P.npass) * CP;
        const int kr0 = kblk * RB, knr = k < steps ? min(RB, H - kr0) : 0;
        const int lo = max(kr0 - 1, 0);
        const unsigned char *raw_u = raw_k, *raw_dl = raw_u + (size_t)CP * RB * W * es;
        for (int it = t0; it < CP * RB * T4; it += nt) {
            const int t = it % T4, rr = (it / T4) % RB, sc = it / (T4 * RB);
            const int c = 4 * t, o4 = sc * CS4 + rr * Wp + pos4<L>(t);
            float4 uv = make_float4(0.f, 0.f, 0.f, 0.f), x = uv;
            if (rr < knr && kch0 + sc < nch && c < W) {
                const int sdd = (dbase + kch0 + sc) / P.drep;
                if (!WS && bulk) {
                    uv = lds4(raw_u, (sc * RB + rr) * W + c, P.io_dt);
                    x = lds4(raw_dl, (sc * (RB + 1) + (kr0 + rr - lo)) * W + c, P.io_dt);
                } else {
                    uv = ld4d(P.u, (int64_t)b * P.u_bs + (int64_t)(dbase + kch0 + sc - ush) * P.u_ds + cs, P.u_hs, kr0 + rr, c,
                              H, W, fh, fw, P.io_dt, P.vec & VEC_U);
                    x = ld4d(P.delta, (int64_t)b * P.dl_bs + (int64_t)sdd * P.dl_ds + cs, P.dl_hs, kr0 + rr, c, H, W, fh, fw,
                             P.io_dt, P.vec & VEC_DELTA);
                }
                const float bv = spar[2 * (kch0 + sc) + 1];
                x.x += bv; x.y += bv; x.z += bv; x.w += bv;
                if (P.softplus) {
                    x.x = softplus20(x.x); x.y = softplus20(x.y); x.z = softplus20(x.z); x.w = softplus20(x.w);
                }
                const int nv = W - c;  // columns past the image keep dl = 0
                if (nv < 4) { x.w = 0.f; if (nv < 3) x.z = 0.f; if (nv < 2) x.y = 0.f; }
            }
            *reinterpret_cast<float4 *>(tu + o4) = uv;
            *reinterpret_cast<float4 *>(tdl + sc * CS5 + (rr + 1) * Wp + pos4<L>(t)) = x;
        }
        if (knr > 0) {
            // delta of the row above the block, one column per item so that all warps share it
            for (int it = t0; it < CP * Wp; it += nt) {
                const int c = it % Wp, sc = it / Wp, r = kr0 - 1;
                float x = 0.f;
                if (r >= 0 && kch0 + sc < nch && c < W) {
                    const int sdd = (dbase + kch0 + sc) / P.drep;
                    if (!WS && bulk)
                        x = lds1(raw_dl, sc * (RB + 1) * W + c, P.io_dt);
                    else
                        x = ld_elem(P.delta, (int64_t)b * P.dl_bs + (int64_t)sdd * P.dl_ds + cs +
                                                 (int64_t)(fh ? H - 1 - r : r) * P.dl_hs + (fw ? W - 1 - c : c), P.io_dt);
                    x += spar[2 * (kch0 + sc) + 1];
                    if (P.softplus) x = softplus20(x);
                }
                tdl[sc * CS5 + pos1<L>(c)] = x;
            }
        }
    };

    if constexpr (WS) {
        if (warp >= FWS_COMPUTE / 32) {  // ---- staging warps ----
            asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FWS_REGS_STAGE));
            for (int d = 0; d < ng; ++d) {
                if (d > 0) { set_dir(d); __syncthreads(); }   // the compute warps have refilled the parameter copies
                for (int k = 0; k < steps; ++k) {
                    const int gk = d * steps + k, set = gk & 1;   // tile sets and barrier phases run on across directions
                    if (gk >= 2 && !mbar_wait_bounded_lazy(freeb + set, ((gk >> 1) - 1) & 1)) {
                        atomicOr(P.status, ERR_STAGE_TIMEOUT);  // the compute warps give up on `full` in turn
                        return;
                    }
                    stage_step(k, set ? set1 : smem, nullptr, tid - FWS_COMPUTE, FWS_STAGE);
                    mbar_arrive(full + set);  // release: the tile writes above are visible to the waiters
                }
                if (d + 1 < ng) __syncthreads();   // end of a direction
            }
            return;
        }
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FWS_REGS_COMPUTE));
    }
    auto cta_sync = [&]() {
        if constexpr (WS) group_sync(1, FWS_COMPUTE); else __syncthreads();
    };
    for (int dir = 0; dir < ng; ++dir) {
    if (dir > 0) {   // next direction of a merged launch: new parameter copies, then everybody goes on
        set_dir(dir);
        fill_par();
        __syncthreads();
    }
    const int sbase = dir * steps;   // tile sets and barrier phases run on across directions
    for (int step = 0; step <= steps; ++step) {
        const int gs = sbase + step;
        const int blk = step / P.npass, pass = step % P.npass;
        const int r0 = blk * RB, nr = step < steps ? min(RB, H - r0) : 0;
        const int ch0 = pass * CP;
        // The checkpoint row above this block is private to this thread (it wrote it
        // when it last had the channel); fetch it now so it arrives during phase A.
        float4 ck_pre[STRIP / 2];
        float2 A2 = bc(0.f);  // this thread's two A values (times log2 e), fetched with it
        {
            const bool ok = nr > 0 && r0 > 0 && pair_on && ch0 + cp < nch;
            const int dq = dbase + min(ch0 + cp, nch - 1);
            if (nr > 0 && pair_on)   // raw values here; the scaling waits until they are used
                A2 = f2(__ldg(P.A + dq * P.A_ds + n0 * P.A_ns), n1 < N ? __ldg(P.A + dq * P.A_ds + n1 * P.A_ns) : 0.f);
            const float4 *pk = reinterpret_cast<const float4 *>(
                P.saved + ((((int64_t)b * P.dim + dq) * ckn + (P.ck_roll ? 0 : blk - 1)) * NPp + pp) * Wp + j * STRIP);
#pragma unroll
            for (int k = 0; k < STRIP / 2; ++k) ck_pre[k] = ok ? pk[k] : make_float4(0.f, 0.f, 0.f, 0.f);
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
            const int pstep = step - 1;
            const int pblk = pstep / P.npass, ppass = pstep % P.npass;
            const int pr0 = pblk * RB, pnr = step > 0 ? min(RB, H - pr0) : 0, pch0 = ppass * CP;
            // tiles of the previous step (its u is needed for D*u) and of this one
            float *prev = WS && ((gs - 1) & 1) ? set1 : smem, *cur = WS && (gs & 1) ? set1 : smem;
            const float *psu = prev + S::u(CP);
            su = cur + S::u(CP); sdl = cur + S::dl(CP);
            const int items = pnr > 0 ? CP * RB * T4 : 0;
            for (int it = tid; it < items; it += nthr) {
                const int t = it % T4, rr = (it / T4) % RB, sc = it / (T4 * RB);
                const int c = 4 * t, o4 = sc * CS4 + rr * Wp + pos4<L>(t);
                if (rr < pnr && pch0 + sc < nch) {
                    const int sd = dbase + pch0 + sc;
                    const int scg = sc / CW, scl = sc % CW;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int q = 0; q < NPp; ++q) {
                        const float4 v = *reinterpret_cast<const float4 *>(
                            sy + ((scg * NPp + q) * CW + scl) * CS4 + rr * Wp + pos4<L>(t));
                        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                    }
                    if (P.D) {
                        const float Dv = spar[2 * (pch0 + sc)];
                        const float4 uv = *reinterpret_cast<const float4 *>(psu + o4);
                        acc.x = fmaf(Dv, uv.x, acc.x); acc.y = fmaf(Dv, uv.y, acc.y);
                        acc.z = fmaf(Dv, uv.z, acc.z); acc.w = fmaf(Dv, uv.w, acc.w);
                    }
                    if (P.mw) {  // direction merge: w*y goes onto the image shared by the directions
                        const float wv = spar[2 * P.CT + pch0 + sc];
                        acc.x *= wv; acc.y *= wv; acc.z *= wv; acc.w *= wv;
                        const int64_t plane = (int64_t)b * P.o_bs + (int64_t)(sd - g * P.dpg) * P.o_ds + cs;
                        if (SERIAL)
                            acc4d(reinterpret_cast<float *>(P.out), plane, P.o_hs, pr0 + rr, c, H, W, fh, fw, P.vec & VEC_OUT,
                                  P.merge_store && gi == 0, acc);
                        else
                            red4d(reinterpret_cast<float *>(P.out), plane, P.o_hs, pr0 + rr, c, H, W, fh, fw, acc);
                    } else {
                        st4d(P.out, (int64_t)b * P.o_bs + (int64_t)sd * P.o_ds + cs, P.o_hs, pr0 + rr, c, H, W, fh, fw, P.out_dt,
                             P.vec & VEC_OUT, acc);
                    }
                }
            }
            if constexpr (WS) {
                // the previous step's tile set may be refilled by the staging warps from here on
                if (step > 0) mbar_arrive(freeb + ((gs - 1) & 1));
            } else {
                // every thread replaces the tile entries it has just read (same item mapping)
                stage_step(step, smem, raw + (size_t)(step & 1) * stage_bytes, tid, nthr);
            }
            if (nr > 0) {
                if (pass == 0) stage_BC<L>(P, b, g, r0, nr, sB, sC, fh, fw, tid, nthr);
                if (has_left) {  // column left of this tile: h, s written by the tile to the left; delta
                    for (int it = tid; it < CP * NPp * (RB + 1); it += nthr) {
                        const int k = it % (RB + 1), q = (it / (RB + 1)) % NPp, sc = it / ((RB + 1) * NPp);
                        const int r = r0 - 1 + k;
                        float4 e = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (r >= 0 && r < H && ch0 + sc < nch)
                            e = __ldg(P.edge_in + (((int64_t)b * P.dim + dbase + ch0 + sc) * NPp + q) * H + r);
                        sedge[it] = e;
                    }
                    for (int it = tid; it < CP * RB; it += nthr) {
                        const int rr = it % RB, sc = it / RB;
                        float x = 0.f;
                        if (rr < nr && ch0 + sc < nch) {
                            const int sdd = (dbase + ch0 + sc) / P.drep;
                            x = ld_elem(P.delta, (int64_t)b * P.dl_bs + (int64_t)sdd * P.dl_ds + cs +
                                                     (int64_t)(fh ? H - 1 - (r0 + rr) : r0 + rr) * P.dl_hs + (fw ? W : -1), P.io_dt);
                            if (P.bias) x += __ldg(P.bias + sdd);
                            if (P.softplus) x = softplus20(x);
                        }
                        sedl[it] = x;
                    }
                }
            }
        }
        if constexpr (WS) {  // this step's tiles have to be complete
            const bool ok = nr == 0 || mbar_wait_bounded(full + (gs & 1), (gs >> 1) & 1);
            if (group_or(2, FWS_COMPUTE, !ok)) {  // the staging warps stopped (they flagged why): leave together
                if (tid == 0) atomicOr(P.status, ERR_STAGE_TIMEOUT);
                return;
            }
        }
        cta_sync();
        if (nr == 0) break;

        // ---- compute: RB rows of CP channels ----------------------------------------
        if (pair_on) {
            const bool ch_ok = ch0 + cp < nch;
            const int d = dbase + min(ch0 + cp, nch - 1);
            A2 = mul2(A2, bc(LOG2E));
            float2 h_up[STRIP], a_up[STRIP];
            float2 *ck = P.saved + ((((int64_t)b * P.dim + d) * ckn + (P.ck_roll ? 0 : blk)) * NPp + pp) * Wp + j * STRIP;
            if (r0 > 0) {
                float dlt[STRIP];
                unpack8(sdl + cp * CS5, L4, j, dlt);
#pragma unroll
                for (int k = 0; k < STRIP / 2; ++k) {
                    h_up[2 * k] = f2(ck_pre[k].x, ck_pre[k].y); h_up[2 * k + 1] = f2(ck_pre[k].z, ck_pre[k].w);
                }
#pragma unroll
                for (int i = 0; i < STRIP; ++i) a_up[i] = ex2_2(fma2(bc(dlt[i]), A2, lgd));
            } else {
#pragma unroll
                for (int i = 0; i < STRIP; ++i) { h_up[i] = bc(0.f); a_up[i] = bc(0.f); }
            }
#pragma unroll
            for (int rr = 0; rr < RB; ++rr) {
                {   // rows past the image are staged as zeros: their results are never written out
                    float dl[STRIP], uu[STRIP], dlu[STRIP];
                    float2 Bv[STRIP], Cv[STRIP];
                    unpack8(su + cp * CS4 + rr * Wp, L4, j, uu);
                    unpack8(sdl + cp * CS5 + (rr + 1) * Wp, L4, j, dl);
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) dlu[i] = dl[i] * uu[i];
                    unpack8x2(sB + (pp * RB + rr) * Wp, L2, j, Bv);
                    unpack8x2(sC + (pp * RB + rr) * Wp, L2, j, Cv);
                    float2 a[STRIP], p[STRIP], h[STRIP], s[STRIP];
                    LeftEdge le = {bc(0.f), bc(0.f), bc(0.f), bc(0.f)};
                    if (has_left && j == 0) {
                        const float4 e0 = sedge[(cp * NPp + pp) * (RB + 1) + rr], e1 = sedge[(cp * NPp + pp) * (RB + 1) + rr + 1];
                        le.h_prev = f2(e0.x, e0.y); le.h = f2(e1.x, e1.y); le.s = f2(e1.z, e1.w);
                        le.a = ex2_2(fma2(bc(sedl[cp * RB + rr]), A2, lgd));
                    }
                    row_forward<L, true>(j, dl, dlu, Bv, A2, lgd, h_up, a_up, a, p, h, s, has_left, le);
                    if (TILED && P.tile_right && j == L - 1 && ch_ok && r0 + rr < H)  // last column of a full tile
                        P.edge_out[(((int64_t)b * P.dim + d) * NPp + pp) * H + r0 + rr] =
                            make_float4(h[STRIP - 1].x, h[STRIP - 1].y, s[STRIP - 1].x, s[STRIP - 1].y);
                    float yv[STRIP];
#pragma unroll
                    for (int i = 0; i < STRIP; ++i) {
                        // C*(h - s + 0.25 p), summed over the two states of the pair
                        const float2 t = mul2(Cv[i], fma2(p[i], bc(0.25f), sub2(h[i], s[i])));
                        yv[i] = t.x + t.y;
                        h_up[i] = h[i];
                        a_up[i] = a[i];
                    }
                    pack8(sy + (warp * CW + cl) * CS4 + rr * Wp, L4, j, yv);
                }
            }
            if (r0 + RB < H && ch_ok) {
                float4 *pk = reinterpret_cast<float4 *>(ck);
#pragma unroll
                for (int k = 0; k < STRIP / 2; ++k)
                    pk[k] = make_float4(h_up[2 * k].x, h_up[2 * k].y, h_up[2 * k + 1].x, h_up[2 * k + 1].y);
            }
        }
        cta_sync();
    }
    if (dir + 1 < ng) __syncthreads();   // end of a direction: its part of the merged image is written
    }
}

#if !CS2D_SERIAL_DIRS
template <int L>
static size_t smem_floats(int CP, int NPp, int nw, bool ws) {
    return (size_t)FwdSmem<L>::total(CP, NPp, nw) + (ws ? FwdSmem<L>::set_floats(CP) : 0);
}

size_t fwd_smem_bytes(int L, int CG, int NPp, int W, int es, bool bulk, int CT, bool tiled, bool ws) {
    const int nw = CG * NPp;
    const int CP = CG * (32 / L);
    // after the tiles: tile-edge areas (tiled kernels), the parameter copies, the mbarriers, then
    // either the raw row blocks of the bulk copies (two stages) or, warp-specialised, the second tile set
    const size_t extra = (size_t)((tiled ? CP * NPp * (RB + 1) * 4 + CP * 4 : 0) + ((3 * CT + 3) & ~3)) * 4 + (ws ? 32 : 16) +
                         (bulk && !ws ? 2 * (size_t)CP * (2 * RB + 1) * W * es : 0);
    switch (L) {
        case 1: return smem_floats<1>(CP, NPp, nw, ws) * 4 + extra;
        case 2: return smem_floats<2>(CP, NPp, nw, ws) * 4 + extra;
        case 4: return smem_floats<4>(CP, NPp, nw, ws) * 4 + extra;
        case 8: return smem_floats<8>(CP, NPp, nw, ws) * 4 + extra;
        case 16: return smem_floats<16>(CP, NPp, nw, ws) * 4 + extra;
        default: return smem_floats<32>(CP, NPp, nw, ws) * 4 + extra;
    }
}

#else
size_t fwd_smem_bytes(int L, int CG, int NPp, int W, int es, bool bulk, int CT, bool tiled, bool ws);
#endif

template <int L, int NPC, bool TILED, bool WS>
static cudaError_t launch(const Dev &P, int grid, size_t smem, cudaStream_t st) {
    static bool attr_done[64] = {};  // per template instance and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(fwd_kernel<L, NPC, TILED, WS, SERIAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    fwd_kernel<L, NPC, TILED, WS, SERIAL><<<grid, WS ? FWS_COMPUTE + FWS_STAGE : 32 * P.CG * P.NPp, smem, st>>>(P);
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
cudaError_t launch_fwd_serial(const Dev &P, int L, int grid, cudaStream_t st) {
#else
cudaError_t launch_fwd(const Dev &P, int L, int grid, cudaStream_t st) {
#endif
    const bool tiled = P.tile_left || P.tile_right;
    if (P.ws && (P.NPp != 8 || P.CG != 1)) return cudaErrorInvalidValue;
    const size_t smem = fwd_smem_bytes(L, P.CG, P.NPp, P.W, P.io_dt == CS2D_F32 ? 4 : 2, P.bulk != 0, P.CT, tiled, P.ws != 0);
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

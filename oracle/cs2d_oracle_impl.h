/*
 * TEST INFRASTRUCTURE - NOT PRODUCT CODE.
 *
 * CPU restatement of the reference's 2D-CrossScan selective scan
 * (longlong-yu/official-cross-scan, kernels/selective_nd_scan).  It is the
 * parity checker for the CUDA kernels and the timed CPU baseline; the product
 * path never links or calls it.
 *
 * The reference ships no CPU implementation and no tests/golden vectors for
 * this path; its only implementation is the CUDA extension.  This restatement
 * follows the device code line by line in *math*, not in structure:
 *   forward   include/cusoflex/selective_scan_fwd_kernel_oflex.cuh:159-337
 *   adjoint   include/cusoflex/selective_scan_bwd_kernel_oflex.cuh:383-476 (dh),
 *             :689-724 (ds)
 *   gradients include/cusoflex/selective_scan_bwd_kernel_oflex.cuh:494-595,
 *             :730-757, softplus chain :785-806, bias sum :808-819
 * It is pinned against outputs of the reference extension itself (built from
 * the reference sources by oracle/Makefile, run on a B200, stored under
 * tests/golden/ by oracle/gen_golden.py).
 *
 * This header is included twice by cs2d_oracle.c with REAL = double / float
 * and SUF = _f64 / _f32.
 */

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUF)

/* softplus with the reference's threshold (fwd kernel :221-224). */
static inline REAL FN(softplus_)(REAL x, int on) {
    if (on && x <= (REAL)20) return (REAL)log1p(exp((double)x));
    return x;
}

/*
 * Forward for one (batch b, channel d): fills a,p,h,s for every state
 * ([N][H][W] each) and accumulates y ([H][W]).
 *   a = exp(dl*A) * A_decay                       (fwd kernel :245)
 *   p = B * dl * u                                (:225,:265)
 *   h = a*(h_left + h_up - 0.5*(a_up+a_left)*h_diag) + p   (:263-271 + scan monoid
 *        selective_scan_common.h:104-106)
 *   s = a*s_left + p                              (:306-327)
 *   y = D*u + sum_n C*(h - s + 0.25*p)            (:227,:301,:334)
 */
static void FN(fwd_plane_)(const cs2d_oracle_shape *sh, int b, int d,
                           const REAL *u, const REAL *delta, const REAL *A,
                           const REAL *Bm, const REAL *Cm, const REAL *Dv,
                           const REAL *bias, REAL A_decay,
                           REAL *dl /*[H][W]*/, REAL *a, REAL *p, REAL *h, REAL *s,
                           REAL *y /*[H][W]*/) {
    const int H = sh->nrows, W = sh->ncols, N = sh->dstate;
    const int g = d / (sh->dim / sh->n_groups);
    const int dg = d / (sh->dim / sh->delta_dim);
    const size_t HW = (size_t)H * W;
    const REAL *up = u + ((size_t)b * sh->dim + d) * HW;
    const REAL *dp = delta + ((size_t)b * sh->delta_dim + dg) * HW;
    const REAL bv = bias ? bias[dg] : (REAL)0;
    const REAL Dval = Dv ? Dv[d] : (REAL)0;
    for (size_t i = 0; i < HW; ++i) {
        dl[i] = FN(softplus_)(dp[i] + bv, sh->delta_softplus);
        y[i] = Dval * up[i];
    }
    for (int n = 0; n < N; ++n) {
        const REAL An = A[(size_t)d * N + n];
        const REAL *Bp = Bm + (((size_t)b * sh->n_groups + g) * N + n) * HW;
        const REAL *Cp = Cm + (((size_t)b * sh->n_groups + g) * N + n) * HW;
        REAL *an = a + n * HW, *pn = p + n * HW, *hn = h + n * HW, *sn = s + n * HW;
        for (int r = 0; r < H; ++r) {
            for (int c = 0; c < W; ++c) {
                const size_t i = (size_t)r * W + c;
                const REAL av = (REAL)exp((double)(dl[i] * An)) * A_decay;
                const REAL pv = Bp[i] * (dl[i] * up[i]);
                const REAL hl = c > 0 ? hn[i - 1] : (REAL)0;
                const REAL hu = r > 0 ? hn[i - W] : (REAL)0;
                const REAL hd = (r > 0 && c > 0) ? hn[i - W - 1] : (REAL)0;
                const REAL au = r > 0 ? an[i - W] : A_decay;
                const REAL al = c > 0 ? an[i - 1] : A_decay;
                const REAL hv = av * (hl + hu - (REAL)0.5 * (au + al) * hd) + pv;
                const REAL sv = av * (c > 0 ? sn[i - 1] : (REAL)0) + pv;
                an[i] = av; pn[i] = pv; hn[i] = hv; sn[i] = sv;
                y[i] += Cp[i] * (hv - sv + (REAL)0.25 * pv);
            }
        }
    }
}

int FN(cs2d_oracle_fwd)(const cs2d_oracle_shape *sh,
                        const REAL *u, const REAL *delta, const REAL *A,
                        const REAL *Bm, const REAL *Cm, const REAL *Dv,
                        const REAL *bias, const REAL *A_decay_p, REAL *out) {
    if (sh->dstate > 16 || sh->dim % sh->n_groups || sh->dim % sh->delta_dim) return -1;
    const int H = sh->nrows, W = sh->ncols, N = sh->dstate;
    const size_t HW = (size_t)H * W;
    const REAL A_decay = A_decay_p ? A_decay_p[0] : (REAL)1;
    const long planes = (long)sh->batch * sh->dim;
    int fail = 0;
#pragma omp parallel
    {
        REAL *buf = (REAL *)malloc(sizeof(REAL) * HW * (1 + 4 * (size_t)N));
        if (!buf) {
#pragma omp atomic write
            fail = 1;
        }
#pragma omp for schedule(dynamic, 4)
        for (long pl = 0; pl < planes; ++pl) {
            if (!buf) continue;
            const int b = (int)(pl / sh->dim), d = (int)(pl % sh->dim);
            REAL *dl = buf, *a = dl + HW, *p = a + N * HW, *h = p + N * HW, *s = h + N * HW;
            FN(fwd_plane_)(sh, b, d, u, delta, A, Bm, Cm, Dv, bias, A_decay,
                           dl, a, p, h, s, out + (size_t)pl * HW);
        }
        free(buf);
    }
    return fail ? -2 : 0;
}

/*
 * Backward.  ddelta is written at full channel resolution (batch, dim, H, W)
 * and ddelta_bias as (dim) exactly as the reference kernel does; the host
 * reduction to delta_dim (selective_scan_oflex.cpp:433-438) is left to the
 * caller.  dB/dC are sums over the channels of a group.
 * dA_decay_ref reproduces the reference (h-path terms only, bwd kernel
 * :519,:548,:556,:572,:585); dA_decay_true adds the row-scan term it omits.
 * Any of dD, ddelta_bias, dA_decay_* may be NULL.
 */
int FN(cs2d_oracle_bwd)(const cs2d_oracle_shape *sh,
                        const REAL *u, const REAL *delta, const REAL *A,
                        const REAL *Bm, const REAL *Cm, const REAL *Dv,
                        const REAL *bias, const REAL *A_decay_p, const REAL *dout,
                        REAL *du, REAL *ddelta, REAL *dA, REAL *dB, REAL *dC,
                        REAL *dD, REAL *ddelta_bias,
                        REAL *dA_decay_ref, REAL *dA_decay_true) {
    if (sh->dstate > 16 || sh->dim % sh->n_groups || sh->dim % sh->delta_dim) return -1;
    const int H = sh->nrows, W = sh->ncols, N = sh->dstate, G = sh->n_groups;
    const int dpg = sh->dim / G;
    const size_t HW = (size_t)H * W;
    const REAL A_decay = A_decay_p ? A_decay_p[0] : (REAL)1;
    memset(dA, 0, sizeof(REAL) * (size_t)sh->dim * N);
    memset(dB, 0, sizeof(REAL) * (size_t)sh->batch * G * N * HW);
    memset(dC, 0, sizeof(REAL) * (size_t)sh->batch * G * N * HW);
    if (dD) memset(dD, 0, sizeof(REAL) * sh->dim);
    if (ddelta_bias) memset(ddelta_bias, 0, sizeof(REAL) * sh->dim);
    double decay_ref = 0, decay_true = 0;
    int fail = 0;
    const long units = (long)sh->batch * G; /* (b, group): owns its dB/dC slab */
#pragma omp parallel
    {
        REAL *buf = (REAL *)malloc(sizeof(REAL) * HW * (3 + 6 * (size_t)N));
        double *dA_loc = (double *)calloc((size_t)sh->dim * N + 2 * (size_t)sh->dim, sizeof(double));
        double dr_loc = 0, dt_loc = 0;
        if (!buf || !dA_loc) {
#pragma omp atomic write
            fail = 1;
        }
        double *dD_loc = dA_loc ? dA_loc + (size_t)sh->dim * N : 0;
        double *db_loc = dD_loc ? dD_loc + sh->dim : 0;
#pragma omp for schedule(dynamic, 1)
        for (long un = 0; un < units; ++un) {
            if (!buf || !dA_loc) continue;
            const int b = (int)(un / G), g = (int)(un % G);
            REAL *dl = buf, *y = dl + HW, *dd = y + HW; /* dd: d(loss)/d(dl) */
            REAL *a = dd + HW, *p = a + N * HW, *h = p + N * HW, *s = h + N * HW;
            REAL *dh = s + N * HW, *ds = dh + N * HW;
            for (int d = g * dpg; d < (g + 1) * dpg; ++d) {
                const int dg = d / (sh->dim / sh->delta_dim);
                FN(fwd_plane_)(sh, b, d, u, delta, A, Bm, Cm, Dv, bias, A_decay, dl, a, p, h, s, y);
                const REAL *up = u + ((size_t)b * sh->dim + d) * HW;
                const REAL *gp = dout + ((size_t)b * sh->dim + d) * HW;
                const REAL *xp = delta + ((size_t)b * sh->delta_dim + dg) * HW;
                const REAL bv = bias ? bias[dg] : (REAL)0;
                const REAL Dval = Dv ? Dv[d] : (REAL)0;
                REAL *dup = du + ((size_t)b * sh->dim + d) * HW;
                REAL *ddp = ddelta + ((size_t)b * sh->dim + d) * HW;
                for (size_t i = 0; i < HW; ++i) {
                    dd[i] = 0;
                    dup[i] = Dval * gp[i];                      /* bwd kernel :211 */
                    dD_loc[d] += (double)(gp[i] * up[i]);       /* :212 */
                }
                for (int n = 0; n < N; ++n) {
                    const REAL An = A[(size_t)d * N + n];
                    const REAL *Bp = Bm + (((size_t)b * G + g) * N + n) * HW;
                    const REAL *Cp = Cm + (((size_t)b * G + g) * N + n) * HW;
                    REAL *dBp = dB + (((size_t)b * G + g) * N + n) * HW;
                    REAL *dCp = dC + (((size_t)b * G + g) * N + n) * HW;
                    REAL *an = a + n * HW, *pn = p + n * HW, *hn = h + n * HW, *sn = s + n * HW;
                    REAL *dhn = dh + n * HW, *dsn = ds + n * HW;
                    double dAacc = 0;
                    for (int r = H - 1; r >= 0; --r) {
                        for (int c = W - 1; c >= 0; --c) {
                            const size_t i = (size_t)r * W + c;
                            const int hr = r + 1 < H, hc = c + 1 < W;
                            const REAL gC = gp[i] * Cp[i];
                            /* bwd kernel :439-469 */
                            REAL v = gC;
                            if (hr) v += an[i + W] * dhn[i + W];
                            if (hc) v += an[i + 1] * dhn[i + 1];
                            if (hr && hc)
                                v -= (REAL)0.5 * an[i + W + 1] * (an[i + 1] + an[i + W]) * dhn[i + W + 1];
                            dhn[i] = v;
                            /* bwd kernel :707-724 */
                            dsn[i] = (hc ? an[i + 1] * dsn[i + 1] : (REAL)0) - gC;
                        }
                    }
                    for (int r = 0; r < H; ++r) {
                        for (int c = 0; c < W; ++c) {
                            const size_t i = (size_t)r * W + c;
                            const REAL dhv = dhn[i], dsv = dsn[i], gv = gp[i];
                            const REAL e = dhv + dsv;
                            const REAL hm = hn[i] - pn[i], sm = sn[i] - pn[i];
                            const REAL q = (REAL)0.25 * gv * Bp[i] * Cp[i];
                            /* :514 and :750 */
                            dup[i] += e * Bp[i] * dl[i] + q * dl[i];
                            /* :516 and :752 */
                            dd[i] += e * Bp[i] * up[i] + An * (dhv * hm + dsv * sm) + q * up[i];
                            /* :518 and :753 */
                            dAacc += (double)(dl[i] * (dhv * hm + dsv * sm));
                            dr_loc += (double)(dhv * hm / A_decay);
                            dt_loc += (double)((dhv * hm + dsv * sm) / A_decay);
                            /* cross terms, credited as the kernel does (:544-587) */
                            if (r > 0 && c > 0) {
                                const REAL X = -(REAL)0.5 * dhv * hn[i - W - 1] * an[i];
                                const REAL Tup = X * an[i - W], Tle = X * an[i - 1];
                                dd[i - W] += An * Tup;
                                dd[i - 1] += An * Tle;
                                dAacc += (double)(dl[i - W] * Tup + dl[i - 1] * Tle);
                                dr_loc += (double)((Tup + Tle) / A_decay);
                                dt_loc += (double)((Tup + Tle) / A_decay);
                            }
                            /* :589-590 and :754-755 */
                            dBp[i] += e * dl[i] * up[i] + (REAL)0.25 * gv * up[i] * dl[i] * Cp[i];
                            dCp[i] += gv * (hn[i] - sn[i] + (REAL)0.25 * pn[i]);
                        }
                    }
                    dA_loc[(size_t)d * N + n] += dAacc;
                }
                /* softplus chain rule :785-806, bias sum :808-819 */
                for (size_t i = 0; i < HW; ++i) {
                    const REAL x = xp[i] + bv;
                    REAL v = dd[i];
                    if (sh->delta_softplus && x <= (REAL)20) v = v / ((REAL)1 + (REAL)exp(-(double)x));
                    ddp[i] = v;
                    db_loc[d] += (double)v;
                }
            }
        }
#pragma omp critical
        {
            if (dA_loc) {
                for (size_t i = 0; i < (size_t)sh->dim * N; ++i) dA[i] += (REAL)dA_loc[i];
                for (int d = 0; d < sh->dim; ++d) {
                    if (dD) dD[d] += (REAL)dD_loc[d];
                    if (ddelta_bias) ddelta_bias[d] += (REAL)db_loc[d];
                }
            }
            decay_ref += dr_loc;
            decay_true += dt_loc;
        }
        free(buf);
        free(dA_loc);
    }
    if (dA_decay_ref) dA_decay_ref[0] = (REAL)decay_ref;
    if (dA_decay_true) dA_decay_true[0] = (REAL)decay_true;
    return fail ? -2 : 0;
}

#undef FN
#undef CAT
#undef CAT_

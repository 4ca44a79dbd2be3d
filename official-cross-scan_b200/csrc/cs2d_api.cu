// extern "C" boundary of the cs2d library: validation, launch geometry, errors.
// Mirrors the checks of the reference host binding
// (src/cusoflex/selective_scan_oflex.cpp:188-245 and :298-391) on raw pointers.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <initializer_list>

#include "cs2d_common.cuh"

namespace cs2d {
cudaError_t launch_fwd(const Dev &P, int L, int grid, cudaStream_t st);
cudaError_t launch_bwd(const Dev &P, int L, int grid, cudaStream_t st);
cudaError_t launch_fwd_serial(const Dev &P, int L, int grid, cudaStream_t st);   // one CTA walks all groups of its tile
cudaError_t launch_bwd_serial(const Dev &P, int L, int grid, cudaStream_t st);
cudaError_t launch_stream_fwd(const Dev &P, int L, int grid, cudaStream_t st);
cudaError_t launch_stream_bwd(const Dev &P, int L, int grid, cudaStream_t st);
int stream_pairs_per_cta(int L);
cudaError_t launch_walk_fwd(const Dev &P, int grid, cudaStream_t st);
void walk_geometry(int ncols, int *swd, int *lr);
int walk_channels_per_cta(int lr);
size_t walk_bc_bytes(int batch, int groups, int nrows, int ncols);
size_t fwd_smem_bytes(int L, int CG, int NPp, int W, int es, bool bulk, int CT, bool tiled, bool ws);
size_t bwd_smem_bytes(int L, int CG, int NPp, int CT, bool acc, int W, int es, int eso, bool bulk, bool tiled, bool ws);
static __device__ int g_cs2d_status = 0;  // see ERR_* in cs2d_common.cuh

// Device address of the status word on the current device (looked up once per device).
static int *status_ptr() {
    static int *ptr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptr[dev] && cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr[dev]), g_cs2d_status) != cudaSuccess)
        ptr[dev] = nullptr;
    return ptr[dev];
}

static thread_local char g_err[512] = "";
static std::atomic<int64_t> g_launches{0};

static int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

struct Geometry { int L, NPp, CG, CP, CT, npass, ntiles, grid, nck, acc, bulk, ws; };

static const size_t kMaxSmem = 227 * 1024;   // largest dynamic shared memory of one CTA
static const size_t kSmSmem = 228 * 1024;    // shared memory of one SM; every resident CTA also reserves 1 KB
static const size_t kCtaReserve = 1024;
static const int kSMs = 148;

// Lanes per row, state-pair slots, channels per pass and per CTA, and the grid.
// serial: the CTAs walk all groups of their channel tile one after the other (direction merge), so the
// grid has no group dimension.
static int plan(const cs2d_problem *p, bool backward, bool bulk_ok, bool tiled, Geometry *g, bool serial = false) {
    const int W = p->ncols, es = p->io_dtype == CS2D_F32 ? 4 : 2, eso = p->out_dtype == CS2D_F32 ? 4 : 2;
    const int strips = (p->ncols + STRIP - 1) / STRIP;
    int L = 1;
    while (L < strips) L <<= 1;
    if (L > 32) return fail(CS2D_ERR_INVALID, "internal: a column tile of %d columns", p->ncols);
    const int NP = (p->dstate + 1) / 2;
    int NPp = 1;
    while (NPp < NP) NPp <<= 1;
    const int dpg = p->dim / p->n_groups;
    // Channel groups per pass: fill the CTA up to 8 warps, but keep the staged
    // per-channel tiles small enough that the shared memory fits.
    int CG = MAX_WARPS / NPp;
    while (CG > 1 && (backward ? bwd_smem_bytes(L, CG, NPp, CG * (32 / L), false, W, es, eso, false, tiled, false) > kMaxSmem
                               : 2 * (fwd_smem_bytes(L, CG, NPp, W, es, false, CG * (32 / L), tiled, false) + kCtaReserve) > kSmSmem))
        CG >>= 1;
    const int CP = CG * (32 / L);
    const int pmax = (dpg + CP - 1) / CP;  // passes that cover a whole group
    // Channels per CTA (1..8 passes): B/C staging and the dB/dC atomics are paid once per CTA,
    // but the grid has to fill whole waves (5.2 waves waste 14% of the machine in the last one).
    const int slots = kSMs * (backward ? 1 : 2);
    // Cost model: a CTA pays the B/C staging of a row block once (about one pass worth of
    // work when a warp holds a single channel, 1/CW of it otherwise) plus np passes, and the
    // launch takes waves(np) rounds of CTAs.
    int npass = 1;
    double best = 1e300;
    const double stage = 1.0 / (32 / L);
    for (int np = 1; np <= (pmax < 8 ? pmax : 8); ++np) {
        const int64_t chunks = (dpg + np * CP - 1) / (np * CP);
        const int64_t grid = (int64_t)p->batch * (serial ? 1 : p->n_groups) * chunks;
        const int64_t waves = (grid + slots - 1) / slots;
        const double cost = (double)waves * (stage + np);
        if (cost < best - 1e-9) { best = cost; npass = np; }
    }
    g->acc = 1;
    g->ws = 0;
    g->bulk = bulk_ok ? 1 : 0;
    if (backward) {
        // drop, in this order, the bulk staging buffers, then the dB/dC accumulators, then passes
        if (bwd_smem_bytes(L, CG, NPp, npass * CP, true, W, es, eso, g->bulk, tiled, false) > kMaxSmem) g->bulk = 0;
        if (bwd_smem_bytes(L, CG, NPp, npass * CP, true, W, es, eso, false, tiled, false) > kMaxSmem) g->acc = 0;
        while (npass > 1 && bwd_smem_bytes(L, CG, NPp, npass * CP, g->acc, W, es, eso, false, tiled, false) > kMaxSmem) --npass;
        if (bwd_smem_bytes(L, CG, NPp, npass * CP, g->acc, W, es, eso, false, tiled, false) > kMaxSmem)
            return fail(CS2D_ERR_UNSUPPORTED, "ncols=%d with dstate=%d needs more shared memory than one SM has",
                        p->ncols, p->dstate);
        // The common geometry (8 state-pair slots, one channel group, one column tile) runs
        // warp-specialised when the second tile set fits: staging warps replace the bulk copies.
        if (NPp == 8 && CG == 1 &&
            bwd_smem_bytes(L, CG, NPp, npass * CP, g->acc, W, es, eso, false, tiled, true) <= kMaxSmem) {
            g->ws = 1;
            g->bulk = 0;
        }
    } else {
        // keep two CTAs per SM
        if (2 * (fwd_smem_bytes(L, CG, NPp, W, es, g->bulk, npass * CP, tiled, false) + kCtaReserve) > kSmSmem) g->bulk = 0;
        if (fwd_smem_bytes(L, CG, NPp, W, es, false, npass * CP, tiled, false) > kMaxSmem)
            return fail(CS2D_ERR_UNSUPPORTED, "ncols=%d with dstate=%d needs more shared memory than one SM has",
                        p->ncols, p->dstate);
        // warp-specialised like the backward, as long as two CTAs still share an SM
        if (NPp == 8 && CG == 1 &&
            2 * (fwd_smem_bytes(L, CG, NPp, W, es, false, npass * CP, tiled, true) + kCtaReserve) <= kSmSmem) {
            g->ws = 1;
            g->bulk = 0;
        }
    }
    g->L = L; g->NPp = NPp; g->CG = CG; g->CP = CP; g->npass = npass; g->CT = npass * CP;
    g->ntiles = (dpg + g->CT - 1) / g->CT;
    g->grid = p->batch * (serial ? 1 : p->n_groups) * g->ntiles;
    g->nck = (p->nrows + RB - 1) / RB;
    return CS2D_OK;
}

static int validate(const cs2d_problem *p) {
    if (!p) return fail(CS2D_ERR_INVALID, "problem is NULL");
    if (p->batch <= 0 || p->dim <= 0 || p->nrows <= 0 || p->ncols <= 0 || p->dstate <= 0 || p->n_groups <= 0 ||
        p->delta_dim <= 0)
        return fail(CS2D_ERR_INVALID, "all sizes must be positive");
    if (p->io_dtype < CS2D_F32 || p->io_dtype > CS2D_BF16)
        return fail(CS2D_ERR_INVALID, "input type must be float32, float16 or bfloat16");
    if (p->out_dtype != p->io_dtype && p->out_dtype != CS2D_F32)
        return fail(CS2D_ERR_INVALID, "out/dout type must equal the input type or be float32");
    if (p->dim % p->n_groups) return fail(CS2D_ERR_INVALID, "dims should be dividable by n_groups");
    if (p->dim % p->delta_dim) return fail(CS2D_ERR_INVALID, "dims should be dividable by delta_dim");
    if (p->dstate > CS2D_MAX_DSTATE)
        return fail(CS2D_ERR_INVALID, "selective_scan only supports state dimension <= %d", CS2D_MAX_DSTATE);
    if (!p->u || !p->delta || !p->A || !p->B || !p->C) return fail(CS2D_ERR_INVALID, "u, delta, A, B, C must be given");
    return CS2D_OK;
}

// A tensor may be accessed four elements at a time when its base address is
// aligned to four elements and every stride that separates rows is a multiple
// of four (rows then start aligned whenever ncols is a multiple of four).
static bool vec_ok(const void *ptr, int esize, int ncols, std::initializer_list<int64_t> strides) {
    if (ncols % 4) return false;
    if (reinterpret_cast<uintptr_t>(ptr) % (4 * esize)) return false;
    for (int64_t s : strides)
        if (s % 4) return false;
    return true;
}
static int esize(int dt) { return dt == CS2D_F32 ? 4 : 2; }
// the same for aligned 4-byte words: every fp32 element, or pairs of 16-bit elements of even-width rows
static bool word_ok(const void *ptr, int esize, int ncols, std::initializer_list<int64_t> strides) {
    const int ew = 4 / esize;   // elements per word
    if (ncols % ew) return false;
    if (reinterpret_cast<uintptr_t>(ptr) % 4) return false;
    for (int64_t s : strides)
        if (s % ew) return false;
    return true;
}
// the same for 8 elements at a time (the streaming kernels' one-word strips of 16-bit types)
static bool vec8_ok(const void *ptr, int esize, int ncols, std::initializer_list<int64_t> strides) {
    if (ncols % 8) return false;
    if (reinterpret_cast<uintptr_t>(ptr) % (8 * esize)) return false;
    for (int64_t s : strides)
        if (s % 8) return false;
    return true;
}

// A (batch, channel, nrows, ncols) tensor can be fetched with bulk copies of whole
// row blocks when its rows are 16-byte multiples, rows of a plane are contiguous,
// and the base address and the plane/batch strides are 16-byte multiples.
static bool bulk_ok1(const void *ptr, int es, int ncols, int64_t bs, int64_t ds, int64_t hs) {
    return ptr && (ncols * es) % 16 == 0 && hs == ncols && reinterpret_cast<uintptr_t>(ptr) % 16 == 0 &&
           (bs * es) % 16 == 0 && (ds * es) % 16 == 0;
}

static void fill(Dev &d, const cs2d_problem *p, const Geometry &g) {
    d.batch = p->batch; d.dim = p->dim; d.H = p->nrows; d.W = p->ncols; d.N = p->dstate; d.G = p->n_groups;
    d.ddim = p->delta_dim; d.io_dt = p->io_dtype; d.out_dt = p->out_dtype; d.softplus = p->delta_softplus;
    d.dpg = p->dim / p->n_groups; d.drep = p->dim / p->delta_dim;
    d.acc_dbc = g.acc; d.bulk = g.bulk; d.ws = g.ws; d.NPp = g.NPp; d.CG = g.CG; d.CT = g.CT; d.npass = g.npass; d.ntiles = g.ntiles; d.nck = g.nck;
    d.u = p->u; d.delta = p->delta; d.B = p->B; d.C = p->C; d.A = p->A; d.D = p->D; d.bias = p->delta_bias;
    d.decay = p->A_decay;
    d.u_bs = p->u_bs; d.u_ds = p->u_ds; d.u_hs = p->u_hs;
    d.dl_bs = p->delta_bs; d.dl_ds = p->delta_ds; d.dl_hs = p->delta_hs;
    d.A_ds = p->A_ds; d.A_ns = p->A_ns;
    d.B_bs = p->B_bs; d.B_gs = p->B_gs; d.B_ns = p->B_ns; d.B_hs = p->B_hs;
    d.C_bs = p->C_bs; d.C_gs = p->C_gs; d.C_ns = p->C_ns; d.C_hs = p->C_hs;
    const int es = esize(p->io_dtype);
    d.vec = 0; d.vec8 = 0; d.vec2 = 0;
    if (vec_ok(p->u, es, p->ncols, {p->u_bs, p->u_ds, p->u_hs})) d.vec |= VEC_U;
    if (vec_ok(p->delta, es, p->ncols, {p->delta_bs, p->delta_ds, p->delta_hs})) d.vec |= VEC_DELTA;
    if (vec_ok(p->B, es, p->ncols, {p->B_bs, p->B_gs, p->B_ns, p->B_hs})) d.vec |= VEC_B;
    if (vec_ok(p->C, es, p->ncols, {p->C_bs, p->C_gs, p->C_ns, p->C_hs})) d.vec |= VEC_C;
    d.adj = nullptr;
    d.det = 0; d.det_ts = 0;
    d.mw = nullptr; d.dw = nullptr;
    d.cshift = 0;
    d.ck_roll = 0;
    d.ck_pairs = 0;
    d.ck_wp = g.L * STRIP;
    d.wbt = nullptr; d.wct = nullptr;
    d.dir_serial = 0; d.merge_store = 0;
    d.status = nullptr;
    d.tile_left = d.tile_right = 0; d.Wout = p->ncols;
    d.flip_h = d.flip_w = 0; d.u_shared = 0;
    d.edge_in = nullptr; d.edge_out = nullptr; d.adj_in = nullptr; d.adj_out = nullptr;
    d.du = d.ddelta = nullptr; d.dA = d.dB = d.dC = d.dD = d.dbias = d.ddecay = nullptr;
}
}  // namespace cs2d

using namespace cs2d;

extern "C" {

// ---- column tiles ------------------------------------------------------------------------
// A launch covers at most 256 columns (32 lanes x 8).  Wider rows are cut into tiles of 256
// columns that are processed by successive launches on the same stream: left to right in
// the forward (each tile leaves h and s of its last column for its right neighbour), right
// to left in the backward (each tile leaves dh and ds of its first column for its left
// neighbour).  Stream order is the only synchronisation between tiles.
static const int kTileCols = 32 * STRIP;
// Rows that need several tiles anyway are cut into 64-column tiles: those run the 8-lane kernels
// (four channels per warp, dB/dC tiles in shared memory, warp-specialised), which cost far less per
// element than the 32-lane ones a 256-column tile would use.
static const int kNarrowTileCols = 8 * STRIP;
static int tile_cols(int ncols) { return ncols > kTileCols ? kNarrowTileCols : kTileCols; }
static int n_tiles(int ncols) { return (ncols + tile_cols(ncols) - 1) / tile_cols(ncols); }

struct TileView {
    cs2d_problem q;   // the problem restricted to the tile (pointers moved, ncols = tile width)
    int c0;           // first column
    Geometry g;
    size_t saved_off, saved_bytes, adj_off, adj_bytes;   // byte offsets inside saved / scratch
};

static const char *at(const void *p, int64_t elems, int es) {
    return p ? reinterpret_cast<const char *>(p) + elems * es : nullptr;
}

// Fills `tv` for tile t and returns the bytes of the per-tile buffers; edge buffers follow them.
static int tile_view(const cs2d_problem *p, int t, bool backward, bool bulk_ok, TileView *tv, bool serial = false) {
    const int es = esize(p->io_dtype);
    const int tc = tile_cols(p->ncols);
    tv->c0 = t * tc;
    tv->q = *p;
    tv->q.ncols = p->ncols - tv->c0 < tc ? p->ncols - tv->c0 : tc;
    tv->q.u = at(p->u, tv->c0, es);
    tv->q.delta = at(p->delta, tv->c0, es);
    tv->q.B = at(p->B, tv->c0, es);
    tv->q.C = at(p->C, tv->c0, es);
    int rc = plan(&tv->q, backward, bulk_ok, n_tiles(p->ncols) > 1, &tv->g, serial);
    if (rc) return rc;
    const size_t per = (size_t)p->batch * p->dim * tv->g.NPp * (tv->g.L * STRIP) * sizeof(float2);
    tv->saved_bytes = per * tv->g.nck;
    tv->adj_bytes = per;
    return CS2D_OK;
}

static bool walk_shape(const cs2d_problem *p) { return p->dstate > 8 && p->ncols <= 8 * STRIP; }

static size_t edge_bytes(const cs2d_problem *p, int NPp) {
    return (size_t)p->batch * p->dim * NPp * p->nrows * sizeof(float4);
}

// backward: adjoint rows; otherwise the forward's state rows - all checkpoints, or (rolling) one
// row per channel and state pair for a forward that no backward follows
static size_t layout_bytes(const cs2d_problem *p, bool backward, bool rolling = false) {
    if (validate(p) != CS2D_OK) return 0;
    const int nt = n_tiles(p->ncols);
    size_t total = 0;
    int NPp = 1;
    for (int t = 0; t < nt; ++t) {
        TileView tv;
        if (tile_view(p, t, backward, false, &tv) != CS2D_OK) return 0;
        total += backward || rolling ? tv.adj_bytes : tv.saved_bytes;
        NPp = tv.g.NPp;
    }
    total += (size_t)(nt - 1) * edge_bytes(p, NPp);
    // the row-walk forward keeps B and C, regrouped, behind the checkpoints (whatever the scan directions
    // turn out to be: the size depends on the problem alone)
    if (!backward && walk_shape(p)) total += walk_bc_bytes(p->batch, p->n_groups, p->nrows, p->ncols);
    return total;
}

size_t cs2d_saved_bytes(const cs2d_problem *p) { return layout_bytes(p, false); }

size_t cs2d_bwd_scratch_bytes(const cs2d_problem *p) { return layout_bytes(p, true); }

size_t cs2d_fwd_only_scratch_bytes(const cs2d_problem *p) { return layout_bytes(p, false, true); }

// A group that walks the columns right-to-left sees the tile's scan columns at mirrored image
// columns (Dev::cshift); 4-element accesses are only kept when that shift preserves 16-byte alignment.
static void tile_flip(Dev &d, int ncols, int c0, int tw, int nt) {
    if (nt <= 1 || !d.flip_w) return;
    d.cshift = (int64_t)ncols - 2 * (int64_t)c0 - tw;
    if (d.cshift % 8) d.vec = 0;
}

static int check_dirs(const cs2d_problem *p, const cs2d_dirs *o) {
    if (!o || (!o->flip_rows_mask && !o->flip_cols_mask && !o->shared_input && !o->merge_w)) return CS2D_OK;
    if (p->n_groups > 32) return fail(CS2D_ERR_INVALID, "direction masks cover at most 32 groups");
    return CS2D_OK;
}

// ---- streaming kernels (cs2d_stream.cu) -------------------------------------------------------
// A problem with a single state per channel, one scan orientation, no A_decay and rows of at most
// 128 columns (16 lanes of 8) runs on the streaming kernels: no shared-memory tiles, no backward scratch, and
// checkpoints that pack two channels per value (half the bytes of the tile kernels' layout, which
// is what cs2d_saved_bytes reports and therefore always large enough).  The choice depends on
// nothing but these properties, so the forward and the backward of a problem always agree.
static bool has_dirs(const cs2d_dirs *o) {
    return o && (o->flip_rows_mask || o->flip_cols_mask || o->shared_input || o->merge_w);
}
static bool stream_ok(const cs2d_problem *p, const cs2d_dirs *o) {
    return p->dstate == 1 && !has_dirs(o) && !p->A_decay && p->ncols <= 16 * STRIP;
}
static int stream_lanes(const cs2d_problem *p) {
    const int strips = (p->ncols + STRIP - 1) / STRIP;
    int L = 1;
    while (L < strips) L <<= 1;
    return L;
}
// Geometry shared by both streaming launches: lanes per row, CTAs per (batch, group), grid.
static void stream_fill(Dev &d, const cs2d_problem *p, int *L, int *grid) {
    Geometry g = {};
    g.L = stream_lanes(p);
    g.NPp = 1; g.CG = 1; g.CP = 1; g.CT = 1; g.npass = 1;
    const int npairs = (p->dim / p->n_groups + 1) / 2, pc = stream_pairs_per_cta(g.L);
    g.ntiles = (npairs + pc - 1) / pc;
    g.nck = (p->nrows + STREAM_RB - 1) / STREAM_RB;
    g.grid = p->batch * p->n_groups * g.ntiles;
    fill(d, p, g);
    const int es = esize(p->io_dtype);
    if (vec8_ok(p->u, es, p->ncols, {p->u_bs, p->u_ds, p->u_hs})) d.vec8 |= VEC_U;
    if (word_ok(p->u, es, p->ncols, {p->u_bs, p->u_ds, p->u_hs})) d.vec2 |= VEC_U;
    if (vec8_ok(p->delta, es, p->ncols, {p->delta_bs, p->delta_ds, p->delta_hs})) d.vec8 |= VEC_DELTA;
    if (word_ok(p->delta, es, p->ncols, {p->delta_bs, p->delta_ds, p->delta_hs})) d.vec2 |= VEC_DELTA;
    if (vec8_ok(p->B, es, p->ncols, {p->B_bs, p->B_gs, p->B_ns, p->B_hs})) d.vec8 |= VEC_B;
    if (word_ok(p->B, es, p->ncols, {p->B_bs, p->B_gs, p->B_ns, p->B_hs})) d.vec2 |= VEC_B;
    if (vec8_ok(p->C, es, p->ncols, {p->C_bs, p->C_gs, p->C_ns, p->C_hs})) d.vec8 |= VEC_C;
    if (word_ok(p->C, es, p->ncols, {p->C_bs, p->C_gs, p->C_ns, p->C_hs})) d.vec2 |= VEC_C;
    *L = g.L; *grid = g.grid;
}

// ---- row-walk forward (cs2d_walk_fwd.cu) ---------------------------------------------------------
// Rows of at most 64 columns with more than 8 states per channel and one scan orientation: the lanes
// of a row work one image row apart, so the recurrence needs no scan.  It writes y and the checkpoints
// exactly where the tile forward would, so the choice is invisible to the backward.
static bool walk_fwd_ok(const cs2d_problem *p, const cs2d_dirs *o) { return walk_shape(p) && !has_dirs(o); }

static int fwd_impl(const cs2d_problem *p, const cs2d_dirs *o, void *out, int64_t out_bs, int64_t out_ds,
                    int64_t out_hs, void *saved, void *stream, bool rolling = false) {
    int rc = validate(p);
    if (rc) return rc;
    if ((rc = check_dirs(p, o))) return rc;
    const bool dirs = has_dirs(o);
    if (!out || !saved) return fail(CS2D_ERR_INVALID, "out and saved must be given");
    if (o && o->merge_w && p->out_dtype != CS2D_F32)
        return fail(CS2D_ERR_INVALID, "the direction merge adds onto an fp32 image: out_dtype must be CS2D_F32");
    if (reinterpret_cast<uintptr_t>(saved) & 15) return fail(CS2D_ERR_INVALID, "saved must be 16-byte aligned");
    int *status = status_ptr();
    if (!status) return fail(CS2D_ERR_CUDA, "cannot locate the device status word");
    if (stream_ok(p, o)) {
        Dev d;
        int L, grid;
        stream_fill(d, p, &L, &grid);
        d.out = out; d.o_bs = out_bs; d.o_ds = out_ds; d.o_hs = out_hs;
        if (vec_ok(out, esize(p->out_dtype), p->ncols, {out_bs, out_ds, out_hs})) d.vec |= VEC_OUT;
        if (vec8_ok(out, esize(p->out_dtype), p->ncols, {out_bs, out_ds, out_hs})) d.vec8 |= VEC_OUT;
        if (word_ok(out, esize(p->out_dtype), p->ncols, {out_bs, out_ds, out_hs})) d.vec2 |= VEC_OUT;
        d.saved = reinterpret_cast<float2 *>(saved);
        d.ck_roll = rolling;
        d.status = status;
        cudaError_t e = launch_stream_fwd(d, L, grid, reinterpret_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return fail(CS2D_ERR_CUDA, "forward launch failed: %s", cudaGetErrorString(e));
        g_launches.fetch_add(1);
        return CS2D_OK;
    }
    if (walk_fwd_ok(p, o)) {
        TileView tv;
        if ((rc = tile_view(p, 0, false, false, &tv))) return rc;   // the checkpoint layout is the tile kernels'
        Dev d;
        fill(d, &tv.q, tv.g);
        int swd, lr;
        walk_geometry(p->ncols, &swd, &lr);
        const int ct = walk_channels_per_cta(lr), dpg = p->dim / p->n_groups;
        d.ntiles = (dpg + ct - 1) / ct;
        d.out = out; d.o_bs = out_bs; d.o_ds = out_ds; d.o_hs = out_hs;
        d.saved = reinterpret_cast<float2 *>(saved);
        d.ck_roll = rolling;
        d.status = status;
        char *bc = reinterpret_cast<char *>(saved) + (rolling ? tv.adj_bytes : tv.saved_bytes);
        d.wbt = reinterpret_cast<float4 *>(bc);
        d.wct = reinterpret_cast<float4 *>(bc + walk_bc_bytes(p->batch, p->n_groups, p->nrows, p->ncols) / 2);
        cudaError_t e = launch_walk_fwd(d, p->batch * p->n_groups * d.ntiles, reinterpret_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return fail(CS2D_ERR_CUDA, "forward launch failed: %s", cudaGetErrorString(e));
        g_launches.fetch_add(2);   // the regrouping of B and C, then the scan
        return CS2D_OK;
    }
    const int es = esize(p->io_dtype), eso = esize(p->out_dtype), nt = n_tiles(p->ncols);
    // saved = [checkpoints tile 0 | ... | checkpoints tile nt-1 | edge 0|1 | ... | edge nt-2|nt-1]
    size_t ck_total = 0;
    for (int t = 0; t < nt; ++t) {
        TileView tv;
        if ((rc = tile_view(p, t, false, false, &tv))) return rc;
        ck_total += rolling ? tv.adj_bytes : tv.saved_bytes;
    }
    size_t ck_off = 0;
    for (int t = 0; t < nt; ++t) {
        TileView tv;
        const bool bulk = nt == 1 && !dirs && bulk_ok1(p->u, es, p->ncols, p->u_bs, p->u_ds, p->u_hs) &&
                          bulk_ok1(p->delta, es, p->ncols, p->delta_bs, p->delta_ds, p->delta_hs);
        const bool serial = o && o->merge_w && (o->flags & CS2D_DIRS_SERIAL);   // a CTA walks all directions of its channel tile
        if ((rc = tile_view(p, t, false, bulk, &tv, serial))) return rc;
        Dev d;
        fill(d, &tv.q, tv.g);
        d.dir_serial = serial; d.merge_store = serial && nt == 1;
        d.out = const_cast<char *>(at(out, tv.c0, eso)); d.o_bs = out_bs; d.o_ds = out_ds; d.o_hs = out_hs;
        if (vec_ok(d.out, eso, tv.q.ncols, {out_bs, out_ds, out_hs})) d.vec |= VEC_OUT;
        d.saved = reinterpret_cast<float2 *>(reinterpret_cast<char *>(saved) + ck_off);
        ck_off += rolling ? tv.adj_bytes : tv.saved_bytes;
        d.ck_roll = rolling;
        d.status = status;
        d.tile_left = t > 0; d.tile_right = t + 1 < nt; d.Wout = p->ncols;
        const size_t eb = edge_bytes(p, tv.g.NPp);
        char *edges = reinterpret_cast<char *>(saved) + ck_total;
        d.edge_in = t > 0 ? reinterpret_cast<const float4 *>(edges + (size_t)(t - 1) * eb) : nullptr;
        d.edge_out = t + 1 < nt ? reinterpret_cast<float4 *>(edges + (size_t)t * eb) : nullptr;
        if (dirs) {
            d.flip_h = o->flip_rows_mask; d.flip_w = o->flip_cols_mask; d.u_shared = o->shared_input; d.mw = o->merge_w;
            tile_flip(d, p->ncols, tv.c0, tv.q.ncols, nt);
        }
        cudaError_t e = (serial ? launch_fwd_serial : launch_fwd)(d, tv.g.L, tv.g.grid, reinterpret_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return fail(CS2D_ERR_CUDA, "forward launch failed: %s", cudaGetErrorString(e));
        g_launches.fetch_add(1);
    }
    return CS2D_OK;
}

int cs2d_fwd(const cs2d_problem *p, void *out, int64_t out_bs, int64_t out_ds, int64_t out_hs, void *saved,
             void *stream) {
    return fwd_impl(p, nullptr, out, out_bs, out_ds, out_hs, saved, stream);
}

int cs2d_fwd_only(const cs2d_problem *p, const cs2d_dirs *dirs, void *out, int64_t out_bs, int64_t out_ds,
                  int64_t out_hs, void *scratch, void *stream) {
    return fwd_impl(p, dirs, out, out_bs, out_ds, out_hs, scratch, stream, true);
}

int cs2d_fwd_dir(const cs2d_problem *p, const cs2d_dirs *dirs, void *out, int64_t out_bs, int64_t out_ds,
                 int64_t out_hs, void *saved, void *stream) {
    return fwd_impl(p, dirs, out, out_bs, out_ds, out_hs, saved, stream);
}

// out[i] += part[i] + part[stride + i] + ... (count terms, in this order): the second step of the
// deterministic backward
__global__ void sum_slots(float *out, const float *part, int64_t n, int count, int64_t stride) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int t = 0; t < count; ++t) v += part[t * stride + i];
        out[i] += v;
    }
}

static cudaError_t launch_sum(float *out, const float *part, int64_t n, int count, int64_t stride, void *stream) {
    if (!out || n <= 0) return cudaSuccess;
    const int block = 256;
    const int64_t want = (n + block - 1) / block;
    sum_slots<<<(unsigned)(want < 8 * kSMs ? want : 8 * kSMs), block, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        out, part, n, count, stride);
    g_launches.fetch_add(1);
    return cudaGetLastError();
}

// layout of the deterministic backward's scratch, in floats
struct DetLayout { int64_t nB, dB, dC, dA, dD, dbias, ddecay, total; int ntiles, grid, zero; };
static int det_layout(const cs2d_problem *p, DetLayout *l) {
    if (n_tiles(p->ncols) > 1)
        return fail(CS2D_ERR_UNSUPPORTED, "the deterministic backward covers ncols <= %d", kTileCols);
    TileView tv;
    int rc = tile_view(p, 0, true, false, &tv);
    if (rc) return rc;
    // Without the dB/dC tiles in shared memory the CTA adds to its plane row by row, which has a
    // single writer per element only when the CTA holds one channel group (see add_dbc).
    if (!tv.g.acc && tv.g.CG != 1)
        return fail(CS2D_ERR_UNSUPPORTED, "no deterministic backward for ncols=%d with dstate=%d "
                                          "(dB/dC tiles do not fit in shared memory and several channel groups share a CTA)",
                    p->ncols, p->dstate);
    l->zero = !tv.g.acc;
    l->ntiles = tv.g.ntiles; l->grid = tv.g.grid;
    l->nB = (int64_t)p->batch * p->n_groups * p->dstate * p->nrows * p->ncols;
    l->dB = 0; l->dC = l->dB + l->ntiles * l->nB; l->dA = l->dC + l->ntiles * l->nB;
    l->dD = l->dA + (int64_t)p->batch * p->dim * p->dstate; l->dbias = l->dD + (int64_t)p->batch * p->dim;
    l->ddecay = l->dbias + (int64_t)p->batch * p->dim; l->total = l->ddecay + l->grid;
    return CS2D_OK;
}

static int bwd_impl(const cs2d_problem *p, const cs2d_dirs *o, const void *dout, int64_t dout_bs, int64_t dout_ds,
                    int64_t dout_hs, const void *saved, void *scratch, void *du, void *ddelta, float *dA, float *dB,
                    float *dC, float *dD, float *ddelta_bias, float *dA_decay, void *stream, float *det = nullptr) {
    int rc = validate(p);
    if (rc) return rc;
    if ((rc = check_dirs(p, o))) return rc;
    DetLayout dl = {};
    if (det && (rc = det_layout(p, &dl))) return rc;
    const bool dirs = o && (o->flip_rows_mask || o->flip_cols_mask || o->shared_input || o->merge_w);
    if (o && o->merge_w && (det || !(o->shared_input & 2)))
        return fail(CS2D_ERR_INVALID, "the direction merge needs the shared gradient image (shared_input bit 1) "
                                      "and is not combined with the deterministic backward");
    if (!dout || !saved || !scratch || !du || !ddelta || !dA || !dB || !dC)
        return fail(CS2D_ERR_INVALID, "dout, saved, scratch, du, ddelta, dA, dB, dC must be given");
    if ((reinterpret_cast<uintptr_t>(saved) | reinterpret_cast<uintptr_t>(scratch)) & 15)
        return fail(CS2D_ERR_INVALID, "saved and scratch must be 16-byte aligned");
    if (dA_decay && !p->A_decay) return fail(CS2D_ERR_INVALID, "dA_decay requested without A_decay");
    int *status = status_ptr();
    if (!status) return fail(CS2D_ERR_CUDA, "cannot locate the device status word");
    const bool streamed = stream_ok(p, o);   // the forward of this problem ran on the streaming kernel
    if (streamed && !det) {
        Dev d;
        int L, grid;
        stream_fill(d, p, &L, &grid);
        d.out = const_cast<void *>(dout); d.o_bs = dout_bs; d.o_ds = dout_ds; d.o_hs = dout_hs;
        if (vec_ok(dout, esize(p->out_dtype), p->ncols, {dout_bs, dout_ds, dout_hs})) d.vec |= VEC_OUT;
        if (vec8_ok(dout, esize(p->out_dtype), p->ncols, {dout_bs, dout_ds, dout_hs})) d.vec8 |= VEC_OUT;
        if (word_ok(dout, esize(p->out_dtype), p->ncols, {dout_bs, dout_ds, dout_hs})) d.vec2 |= VEC_OUT;
        d.du = du; d.ddelta = ddelta;
        if (vec_ok(du, esize(p->io_dtype), p->ncols, {(int64_t)p->ncols}) &&
            vec_ok(ddelta, esize(p->io_dtype), p->ncols, {(int64_t)p->ncols}))
            d.vec |= VEC_DU;
        if (vec8_ok(du, esize(p->io_dtype), p->ncols, {(int64_t)p->ncols}) &&
            vec8_ok(ddelta, esize(p->io_dtype), p->ncols, {(int64_t)p->ncols}))
            d.vec8 |= VEC_DU;
        if (word_ok(du, esize(p->io_dtype), p->ncols, {(int64_t)p->ncols}) &&
            word_ok(ddelta, esize(p->io_dtype), p->ncols, {(int64_t)p->ncols}))
            d.vec2 |= VEC_DU;
        d.saved = reinterpret_cast<float2 *>(const_cast<void *>(saved));
        d.dA = dA; d.dB = dB; d.dC = dC; d.dD = dD; d.dbias = ddelta_bias;
        d.status = status;
        cudaError_t e = launch_stream_bwd(d, L, grid, reinterpret_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return fail(CS2D_ERR_CUDA, "backward launch failed: %s", cudaGetErrorString(e));
        g_launches.fetch_add(1);
        return CS2D_OK;
    }
    const int es = esize(p->io_dtype), eso = esize(p->out_dtype), nt = n_tiles(p->ncols);
    // saved as laid out by the forward; scratch = [adjoint rows tile 0 | ... | dh/ds edges]
    size_t ck_total = 0, adj_total = 0;
    size_t ck_offs[64], adj_offs[64];
    if (nt > 64) return fail(CS2D_ERR_UNSUPPORTED, "more than 64 column tiles");
    for (int t = 0; t < nt; ++t) {
        TileView tv;
        if ((rc = tile_view(p, t, true, false, &tv))) return rc;
        ck_offs[t] = ck_total; adj_offs[t] = adj_total;
        ck_total += tv.saved_bytes; adj_total += tv.adj_bytes;
    }
    for (int t = nt - 1; t >= 0; --t) {
        TileView tv;
        const bool bulk = nt == 1 && !dirs && bulk_ok1(p->u, es, p->ncols, p->u_bs, p->u_ds, p->u_hs) &&
                          bulk_ok1(p->delta, es, p->ncols, p->delta_bs, p->delta_ds, p->delta_hs) &&
                          bulk_ok1(dout, eso, p->ncols, dout_bs, dout_ds, dout_hs);
        const bool serial = o && o->merge_w && (o->flags & CS2D_DIRS_SERIAL);   // a CTA walks all directions of its channel tile
        if ((rc = tile_view(p, t, true, bulk, &tv, serial))) return rc;
        Dev d;
        fill(d, &tv.q, tv.g);
        d.dir_serial = serial; d.merge_store = serial && nt == 1;
        d.out = const_cast<char *>(at(dout, tv.c0, eso)); d.o_bs = dout_bs; d.o_ds = dout_ds; d.o_hs = dout_hs;
        if (vec_ok(d.out, eso, tv.q.ncols, {dout_bs, dout_ds, dout_hs})) d.vec |= VEC_OUT;
        d.du = const_cast<char *>(at(du, tv.c0, o && o->merge_w ? 4 : es));   // the merged du image is fp32
        d.ddelta = const_cast<char *>(at(ddelta, tv.c0, es));
        if (vec_ok(d.du, es, tv.q.ncols, {(int64_t)p->ncols}) && vec_ok(d.ddelta, es, tv.q.ncols, {(int64_t)p->ncols}))
            d.vec |= VEC_DU;
        if (serial && vec_ok(d.du, 4, tv.q.ncols, {(int64_t)p->ncols})) d.vec |= VEC_MDU;   // the merged du image is fp32
        d.saved = reinterpret_cast<float2 *>(const_cast<char *>(reinterpret_cast<const char *>(saved)) + ck_offs[t]);
        d.adj = reinterpret_cast<float2 *>(reinterpret_cast<char *>(scratch) + adj_offs[t]);
        d.dA = dA; d.dB = dB + tv.c0; d.dC = dC + tv.c0; d.dD = dD; d.dbias = ddelta_bias; d.ddecay = dA_decay;
        d.status = status;
        d.ck_pairs = streamed;   // deterministic backward of a streamed forward: read its checkpoint layout
        d.tile_left = t > 0; d.tile_right = t + 1 < nt; d.Wout = p->ncols;
        const size_t eb = edge_bytes(p, tv.g.NPp);
        const char *edges = reinterpret_cast<const char *>(saved) + ck_total;
        char *aedges = reinterpret_cast<char *>(scratch) + adj_total;
        d.edge_in = t > 0 ? reinterpret_cast<const float4 *>(edges + (size_t)(t - 1) * eb) : nullptr;
        d.adj_in = t + 1 < nt ? reinterpret_cast<const float4 *>(aedges + (size_t)t * eb) : nullptr;
        d.adj_out = t > 0 ? reinterpret_cast<float4 *>(aedges + (size_t)(t - 1) * eb) : nullptr;
        if (dirs) {
            d.flip_h = o->flip_rows_mask; d.flip_w = o->flip_cols_mask; d.u_shared = o->shared_input;
            d.mw = o->merge_w; d.dw = o->merge_dw;
            tile_flip(d, p->ncols, tv.c0, tv.q.ncols, nt);
        }
        if (det) {  // per-tile planes and per-batch slots instead of the results themselves
            if (dl.zero && cudaMemsetAsync(det + dl.dB, 0, (size_t)(2 * dl.ntiles * dl.nB) * sizeof(float),
                                           reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess)
                return fail(CS2D_ERR_CUDA, "cannot clear the deterministic scratch");
            d.det = 1; d.det_ts = dl.nB;
            d.dB = det + dl.dB; d.dC = det + dl.dC; d.dA = det + dl.dA;
            d.dD = dD ? det + dl.dD : nullptr; d.dbias = ddelta_bias ? det + dl.dbias : nullptr;
            d.ddecay = dA_decay ? det + dl.ddecay : nullptr;
        }
        cudaError_t e = (serial ? launch_bwd_serial : launch_bwd)(d, tv.g.L, tv.g.grid, reinterpret_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return fail(CS2D_ERR_CUDA, "backward launch failed: %s", cudaGetErrorString(e));
        g_launches.fetch_add(1);
    }
    if (det) {
        const int64_t nA = (int64_t)p->dim * p->dstate;
        cudaError_t e = launch_sum(dB, det + dl.dB, dl.nB, dl.ntiles, dl.nB, stream);
        if (e == cudaSuccess) e = launch_sum(dC, det + dl.dC, dl.nB, dl.ntiles, dl.nB, stream);
        if (e == cudaSuccess) e = launch_sum(dA, det + dl.dA, nA, p->batch, nA, stream);
        if (e == cudaSuccess) e = launch_sum(dD, det + dl.dD, p->dim, p->batch, p->dim, stream);
        if (e == cudaSuccess) e = launch_sum(ddelta_bias, det + dl.dbias, p->dim, p->batch, p->dim, stream);
        if (e == cudaSuccess) e = launch_sum(dA_decay, det + dl.ddecay, 1, dl.grid, 1, stream);
        if (e != cudaSuccess) return fail(CS2D_ERR_CUDA, "deterministic reduction failed: %s", cudaGetErrorString(e));
    }
    return CS2D_OK;
}

size_t cs2d_bwd_det_scratch_bytes(const cs2d_problem *p) {
    DetLayout dl = {};
    if (validate(p) != CS2D_OK || det_layout(p, &dl) != CS2D_OK) return 0;
    return (size_t)dl.total * sizeof(float);
}

int cs2d_bwd_det(const cs2d_problem *p, const cs2d_dirs *dirs, const void *dout, int64_t dout_bs, int64_t dout_ds,
                 int64_t dout_hs, const void *saved, void *scratch, void *det_scratch, void *du, void *ddelta,
                 float *dA, float *dB, float *dC, float *dD, float *ddelta_bias, float *dA_decay, void *stream) {
    if (!det_scratch || (reinterpret_cast<uintptr_t>(det_scratch) & 15))
        return fail(CS2D_ERR_INVALID, "det_scratch must be given and 16-byte aligned");
    return bwd_impl(p, dirs, dout, dout_bs, dout_ds, dout_hs, saved, scratch, du, ddelta, dA, dB, dC, dD, ddelta_bias,
                    dA_decay, stream, static_cast<float *>(det_scratch));
}

int cs2d_bwd(const cs2d_problem *p, const void *dout, int64_t dout_bs, int64_t dout_ds, int64_t dout_hs,
             const void *saved, void *scratch, void *du, void *ddelta, float *dA, float *dB, float *dC,
             float *dD, float *ddelta_bias, float *dA_decay, void *stream) {
    return bwd_impl(p, nullptr, dout, dout_bs, dout_ds, dout_hs, saved, scratch, du, ddelta, dA, dB, dC, dD,
                    ddelta_bias, dA_decay, stream);
}

int cs2d_bwd_dir(const cs2d_problem *p, const cs2d_dirs *dirs, const void *dout, int64_t dout_bs, int64_t dout_ds,
                 int64_t dout_hs, const void *saved, void *scratch, void *du, void *ddelta, float *dA, float *dB,
                 float *dC, float *dD, float *ddelta_bias, float *dA_decay, void *stream) {
    return bwd_impl(p, dirs, dout, dout_bs, dout_ds, dout_hs, saved, scratch, du, ddelta, dA, dB, dC, dD,
                    ddelta_bias, dA_decay, stream);
}

/*
 * Backward for callers that must not allocate.
 *
 * Some hosts of this library cannot call cudaMalloc at the point where they run
 * the backward: a serving or training runtime that hands every byte of device
 * memory to its own pool at start-up, a plugin called from inside somebody
 * else's allocator callback, or a binding (a JNI / cgo stub, say) that is only
 * given the tensors it was called with.  For them the adjoint-row scratch that
 * cs2d_bwd takes as an argument lives inside the library instead: a fixed
 * device array that every GPU loading the library carries until the process
 * exits.  In host code the array's name is only a handle, not a device address,
 * so the address is looked up with cudaGetSymbolAddress - once per device, with
 * that device current, on the first call there.  That first call should
 * therefore happen before any stream capture is started.
 *
 * Everything else is cs2d_bwd: same inputs, same caller-provided outputs, same
 * kernel.  Nothing in the array has to be cleared between calls (each row is
 * written before it is read), but all calls share it: two calls that can run
 * at the same time on one GPU would overwrite each other's rows.
 */
static __device__ __align__(256) unsigned char g_noalloc_scratch[CS2D_NOALLOC_SCRATCH_BYTES];

static void *noalloc_scratch_ptr() {
    static void *ptr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptr[dev]) {
        void *q = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&q, g_noalloc_scratch);
        if (e != cudaSuccess || !q) {
            fail(CS2D_ERR_CUDA, "cudaGetSymbolAddress(built-in scratch) failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        ptr[dev] = q;
    }
    return ptr[dev];
}

int cs2d_bwd_noalloc(const cs2d_problem *p, const void *dout, int64_t dout_bs, int64_t dout_ds, int64_t dout_hs,
                     const void *saved, void *du, void *ddelta, float *dA, float *dB, float *dC, float *dD,
                     float *ddelta_bias, float *dA_decay, void *stream) {
    int rc = validate(p);
    if (rc) return rc;
    const size_t need = cs2d_bwd_scratch_bytes(p);
    if (need == 0) return CS2D_ERR_UNSUPPORTED;  // message already set by the planner
    if (need > (size_t)CS2D_NOALLOC_SCRATCH_BYTES)
        return fail(CS2D_ERR_UNSUPPORTED,
                    "this problem needs %zu bytes of backward scratch but the built-in buffer holds %zu; "
                    "split the batch or call cs2d_bwd with your own scratch",
                    need, (size_t)CS2D_NOALLOC_SCRATCH_BYTES);
    void *scratch = noalloc_scratch_ptr();
    if (!scratch) return CS2D_ERR_CUDA;
    return cs2d_bwd(p, dout, dout_bs, dout_ds, dout_hs, saved, scratch, du, ddelta, dA, dB, dC, dD, ddelta_bias,
                    dA_decay, stream);
}

int cs2d_device_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_cs2d_status, sizeof(int)) != cudaSuccess) return CS2D_ERR_CUDA;
    if (v != 0) {
        cudaMemcpyToSymbol(g_cs2d_status, &zero, sizeof(int));
        fail(CS2D_ERR_CUDA, "a kernel gave up on a bounded wait (status %d: %s%s); its outputs are invalid", v,
             (v & ERR_BULK_COPY_TIMEOUT) ? "bulk copy " : "", (v & ERR_STAGE_TIMEOUT) ? "staging warps" : "");
    }
    return v;
}

const char *cs2d_last_error(void) { return g_err; }
int cs2d_abi_version(void) { return CS2D_ABI_VERSION; }
int64_t cs2d_launch_count(void) { return g_launches.load(); }

}  // extern "C"

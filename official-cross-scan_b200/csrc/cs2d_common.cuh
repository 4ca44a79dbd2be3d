// Shared device helpers for the 2D-CrossScan selective-scan kernels (sm_100a).
//
// Work decomposition used by both kernels
// ---------------------------------------
// There are batch*dim*dstate independent 2-D linear recurrences.  A thread owns
// a strip of STRIP (=8) consecutive columns of ONE row at a time, for a PAIR of
// states (n, n+1) of one channel; the pair is processed with packed fp32x2
// arithmetic (FFMA2/FMUL2/FADD2 of sm_100).  L = 2^k lanes cover one image row
// (L*8 >= ncols) and rows are walked sequentially, so the previous row lives in
// registers.  The recurrence along a row is a first-order linear scan: each
// lane folds its 8 columns, a log2(L)-step warp-shuffle scan combines the lane
// aggregates, and a second local pass applies the carry.
//
// A warp holds CW = 32/L channels of the SAME state pair, so B and C are read
// from shared memory as broadcasts and the sums over channels (dB, dC) are
// formed inside the warp.  A CTA has NPp state pairs x CG channel groups
// (at most 8 warps) and walks its CT channels in passes of CP = CG*CW channels; sums over
// state pairs (y, du, ddelta) go through per-warp partial tiles.  No shared
// memory atomics are used anywhere (fp32 shared atomics are CAS loops).
//
// Rows are processed in blocks of RB = 4.  The state that crosses a block
// boundary lives in global memory: the last h row of each block is the
// checkpoint the backward needs anyway, and the backward keeps its adjoint row
// in a scratch buffer.  Both are read back by the thread that wrote them.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cs2d.h"

namespace cs2d {

constexpr int STRIP = 8;     // columns per thread
constexpr int RB = 4;        // rows per block == checkpoint cadence
constexpr int STREAM_RB = 4; // the same for the streaming (dstate 1) kernels; the tile backward can read their checkpoints
constexpr int MAX_WARPS = 8;  // warps per CTA: state-pair slots x channel groups, at most 8
constexpr int MAX_THREADS = MAX_WARPS * 32;
constexpr float LOG2E = 1.4426950408889634f;

// Device-side problem description (passed by value to the kernels).
struct Dev {
    int batch, dim, H, W, N, G, ddim;
    int io_dt, out_dt, softplus;
    int dpg;    // channels per B/C group
    int drep;   // channels per delta channel
    int NPp;    // state-pair slots per channel: power of two >= ceil(N/2)
    int CG;     // channel groups per pass; the CTA has NPp * CG warps
    int CT;     // channels per CTA
    int npass;  // passes per row block = CT / (CG * 32/L)
    int ntiles; // channel tiles per group
    int nck;    // row blocks per image: ceil(H/RB)
    int acc_dbc; // backward: 1 = dB/dC accumulated over the CTA's passes in shared memory,
                 //           0 = added to global memory row by row (wide rows: tiles do not fit)
    // Scan directions: bit g of flip_h / flip_w set = group g walks the image rows bottom-up /
    // the columns right-to-left.  Tensors stay in image coordinates; the flips are index maps
    // applied when tiles are staged and results written.  u_shared: u and dout have dim/G
    // channels shared by all groups (the four corner directions read the same image).
    unsigned flip_h, flip_w;
    int u_shared;
    int vec;    // bit i set: tensor i may be accessed 4 elements at a time
    int vec8;   // bit i set: ... 8 elements at a time (streaming kernels, 16-bit types: one 16-byte word per strip)
    int vec2;   // bit i set: ... in aligned 4-byte words (streaming kernels: fp32 elements, pairs of 16-bit ones)
    int ws;     // backward: 1 = warp-specialised kernel (8 compute warps + 4 staging warps)
    int bulk;   // 1: row blocks of u, delta (and dout) are fetched with bulk asynchronous copies
                //    (rows are 16-byte multiples, planes contiguous and aligned); 0: plain loads
    int *status; // device status word (see ERR_*)
    const void *u, *delta, *B, *C;
    const float *A, *D, *bias, *decay;
    int64_t u_bs, u_ds, u_hs, dl_bs, dl_ds, dl_hs, A_ds, A_ns;
    int64_t B_bs, B_gs, B_ns, B_hs, C_bs, C_gs, C_ns, C_hs;
    void *out; int64_t o_bs, o_ds, o_hs;  // forward: out; backward: dout
    float2 *saved;                         // [batch][dim][nck][NPp][L*8] checkpoints of h
    int ck_roll;                           // forward without backward: one rolling row [batch][dim][1][NPp][L*8]
    int ck_pairs;                          // checkpoints were written by the streaming forward (dstate 1):
                                           // [batch][G][ceil(dpg/2)][nck][L*8] float2 = two CHANNELS per value
    int ck_wp;                             // L*8: columns of a checkpoint row (the row-walk forward writes the same layout)
    float4 *wbt, *wct;                     // row-walk kernels: B and C regrouped as [batch][G][H][4][W] entries of four states
    // Column tiling of rows wider than 256 columns: this launch covers one tile (all
    // tensor pointers are already moved to the tile's first column).  The values that
    // cross a tile boundary travel through global edge buffers [batch][dim][NPp][H] float4
    // written by the neighbouring tile's launch: (h.x, h.y, s.x, s.y) of the column left of
    // the tile, (dh.x, dh.y, ds.x, ds.y) of the column right of it.
    int tile_left, tile_right;             // the tile has a neighbour on that side
    int Wout;                              // row pitch (full image width) of du, ddelta, dB, dC
    const float4 *edge_in; float4 *edge_out;          // h/s edge: read (left side), written (right side)
    const float4 *adj_in; float4 *adj_out;            // dh/ds edge: read (right side), written (left side)
    // backward only
    float2 *adj;                           // [batch][dim][NPp][L*8] adjoint row between blocks
    void *du, *ddelta;
    float *dA, *dB, *dC, *dD, *dbias, *ddecay;
    // Deterministic mode: no global atomics.  Every CTA stores (does not add) its dB/dC sums
    // into the plane of its channel tile (dB/dC then point at tile 0's plane, det_ts elements
    // apart) and its per-channel sums into per-batch slots: dA [batch][dim][N], dD and dbias
    // [batch][dim], ddecay [grid]; a second kernel adds the planes and slots up in a fixed order.
    int det;
    int64_t det_ts;
    // Direction merge (four-corner CrossScan with fusion weights w[dim], one per (direction,
    // channel)): the forward ADDS w[d]*y_d onto an fp32 image out[batch][dim/G][H][W] shared by the
    // G directions; the backward reads the shared raw gradient dy of that image (u_shared bit 1),
    // ADDS w[d]*du_d onto an fp32 du[batch][dim/G][H][W], scales every other gradient of channel d
    // by w[d] and accumulates dw[d] = sum dy*y_d.
    const float *mw;
    float *dw;
    // dir_serial (the reproducible form of the direction merge): a CTA walks all G groups of its channel
    // tile one after the other (the grid has no group dimension) and owns the merged images; merge_store:
    // the first direction stores them (the launch covers the whole row width), otherwise every direction
    // adds onto zero-filled images.  Without dir_serial the directions are separate CTAs that add onto the
    // zero-filled images with atomics (faster: four times the CTAs, no read-modify-write latency).
    int dir_serial, merge_store;
    // Column tiles of a group that walks the columns right-to-left: the launch's scan columns
    // c0..c0+W-1 are image columns Wfull-c0-W..Wfull-c0-1, so every tensor access of such a group
    // adds cshift = Wfull - 2*c0 - W elements to the (c0-shifted) pointers.  0 without tiles.
    int64_t cshift;
};
enum { VEC_U = 1, VEC_DELTA = 2, VEC_B = 4, VEC_C = 8, VEC_OUT = 16, VEC_DU = 32,
       VEC_MDU = 64 };   // VEC_MDU: the merged fp32 du image of a direction merge

// Device-side status word of the library (0 = fine).  A kernel that gives up on a
// bounded wait records why here instead of spinning; the host reads and clears it
// through cs2d_device_status().
enum { ERR_BULK_COPY_TIMEOUT = 1, ERR_STAGE_TIMEOUT = 2 };

// ---- packed fp32x2 helpers -------------------------------------------------
__device__ __forceinline__ float2 f2(float x, float y) { return make_float2(x, y); }
__device__ __forceinline__ float2 bc(float x) { return make_float2(x, x); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 sub2(float2 a, float2 b) { return __ffma2_rn(b, bc(-1.f), a); }
__device__ __forceinline__ float2 neg2(float2 a) { return make_float2(-a.x, -a.y); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float2 ex2_2(float2 x) { return make_float2(ex2(x.x), ex2(x.y)); }

template <int WIDTH>
__device__ __forceinline__ float2 shfl_up2(float2 v, int off) {
    return make_float2(__shfl_up_sync(0xffffffffu, v.x, off, WIDTH), __shfl_up_sync(0xffffffffu, v.y, off, WIDTH));
}
template <int WIDTH>
__device__ __forceinline__ float2 shfl_down2(float2 v, int off) {
    return make_float2(__shfl_down_sync(0xffffffffu, v.x, off, WIDTH),
                       __shfl_down_sync(0xffffffffu, v.y, off, WIDTH));
}
template <int WIDTH>
__device__ __forceinline__ float2 shfl_xor2(float2 v, int off) {
    return make_float2(__shfl_xor_sync(0xffffffffu, v.x, off, WIDTH), __shfl_xor_sync(0xffffffffu, v.y, off, WIDTH));
}

// ---- dtype-generic global access (staging / write-out only) -------------------
__device__ __forceinline__ float ld_elem(const void *p, int64_t i, int dt) {
    if (dt == CS2D_F32) return __ldg(reinterpret_cast<const float *>(p) + i);
    if (dt == CS2D_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
    return __half2float(reinterpret_cast<const __half *>(p)[i]);
}
__device__ __forceinline__ void st_elem(void *p, int64_t i, int dt, float v) {
    if (dt == CS2D_F32) reinterpret_cast<float *>(p)[i] = v;
    else if (dt == CS2D_BF16) reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16(v);
    else reinterpret_cast<__half *>(p)[i] = __float2half(v);
}
// 4 consecutive elements starting at i; `nvalid` (<=4) of them exist, the rest read as 0.
__device__ __forceinline__ float4 ld4(const void *p, int64_t i, int dt, bool vec, int nvalid) {
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    if (nvalid <= 0) return r;
    if (vec && nvalid >= 4) {
        if (dt == CS2D_F32) return __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p) + i));
        const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(p) + i));
        if (dt == CS2D_BF16) {
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
            return make_float4(a.x, a.y, b.x, b.y);
        }
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    r.x = ld_elem(p, i, dt);
    if (nvalid > 1) r.y = ld_elem(p, i + 1, dt);
    if (nvalid > 2) r.z = ld_elem(p, i + 2, dt);
    if (nvalid > 3) r.w = ld_elem(p, i + 3, dt);
    return r;
}
__device__ __forceinline__ void st4(void *p, int64_t i, int dt, bool vec, int nvalid, float4 v) {
    if (nvalid <= 0) return;
    if (vec && nvalid >= 4) {
        if (dt == CS2D_F32) {
            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p) + i) = v;
        } else {
            uint2 raw;
            if (dt == CS2D_BF16) {
                *reinterpret_cast<__nv_bfloat162 *>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
                *reinterpret_cast<__nv_bfloat162 *>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
            } else {
                *reinterpret_cast<__half2 *>(&raw.x) = __floats2half2_rn(v.x, v.y);
                *reinterpret_cast<__half2 *>(&raw.y) = __floats2half2_rn(v.z, v.w);
            }
            *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(p) + i) = raw;
        }
        return;
    }
    st_elem(p, i, dt, v.x);
    if (nvalid > 1) st_elem(p, i + 1, dt, v.y);
    if (nvalid > 2) st_elem(p, i + 2, dt, v.z);
    if (nvalid > 3) st_elem(p, i + 3, dt, v.w);
}

// ---- bulk asynchronous copies (TMA engine, untiled form) + mbarrier ----------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// global -> this CTA's shared memory; both addresses and the size are multiples of 16 bytes
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// Barrier / OR-reduction among `n` threads of the CTA (a multiple of 32) on hardware barrier `id`
// (1..15; 0 is __syncthreads).  Used where only some of the CTA's warps take part.
__device__ __forceinline__ void group_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ bool group_or(int id, int n, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, %2, %3, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)pred), "r"(id), "r"(n)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for a phase of the barrier, but never forever: after ~2^22 polls (seconds)
// it reports failure so that the caller can flag the error and leave.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
    for (int i = 0; i < (1 << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}
// The same for a warp that runs well ahead of the one it waits for (the staging warps): it backs
// off at once and for longer, so that its polling does not take issue slots from the warps that
// share its scheduler.  Still bounded: 2^21 polls of >= 256 ns.
__device__ __forceinline__ bool mbar_wait_bounded_lazy(uint64_t *bar, uint32_t parity) {
    for (int i = 0; i < (1 << 21); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(256);
    }
    return false;
}
// 4 consecutive elements of a raw (input dtype) shared-memory row as floats
__device__ __forceinline__ float4 lds4(const unsigned char *raw, int idx, int dt) {
    if (dt == CS2D_F32) return *reinterpret_cast<const float4 *>(raw + (size_t)idx * 4);
    const uint2 v = *reinterpret_cast<const uint2 *>(raw + (size_t)idx * 2);
    if (dt == CS2D_BF16) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

// one element of a raw (input dtype) shared-memory row as a float
__device__ __forceinline__ float lds1(const unsigned char *raw, int idx, int dt) {
    if (dt == CS2D_F32) return reinterpret_cast<const float *>(raw)[idx];
    if (dt == CS2D_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(raw)[idx]);
    return __half2float(reinterpret_cast<const __half *>(raw)[idx]);
}

// w*y (or w*du) of 4 consecutive SCAN columns c..c+3 of scan row r goes onto an fp32 image plane shared by
// the scan directions.  red4d: the directions run as separate CTAs and add with atomics (the image starts
// zero-filled).
__device__ __forceinline__ void red4d(float *p, int64_t plane, int64_t hs, int r, int c, int H, int W, bool fh, bool fw,
                                      float4 v) {
    float *row = p + plane + (int64_t)(fh ? H - 1 - r : r) * hs;
    const int nv = W - c;
    const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k)
        if (k < nv) atomicAdd(row + (fw ? W - 1 - (c + k) : c + k), e[k]);
}
// acc4d: one CTA owns the image and walks the directions itself (Dev::dir_serial): plain stores by the
// first direction (`store`), read-modify-write by the following ones.  The reads bypass L1: the earlier
// direction's stores were made by other threads of this CTA, behind a CTA barrier.
__device__ __forceinline__ void acc4d(float *p, int64_t plane, int64_t hs, int r, int c, int H, int W, bool fh, bool fw,
                                      bool vec, bool store, float4 v) {
    float *row = p + plane + (int64_t)(fh ? H - 1 - r : r) * hs;
    const int nv = W - c;
    if (nv <= 0) return;
    if (vec && nv >= 4) {
        float4 *q = reinterpret_cast<float4 *>(row + (fw ? W - 4 - c : c));
        float4 t = fw ? make_float4(v.w, v.z, v.y, v.x) : v;
        if (!store) {
            const float4 o = __ldcg(q);
            t.x += o.x; t.y += o.y; t.z += o.z; t.w += o.w;
        }
        *q = t;
        return;
    }
    const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k)
        if (k < nv) {
            float *q = row + (fw ? W - 1 - (c + k) : c + k);
            *q = store ? e[k] : __ldcg(q) + e[k];
        }
}

// Direction-aware access to 4 consecutive SCAN columns c..c+3 of scan row r of an image plane
// (element offset `plane`, row pitch `hs`): rows are mirrored when fh, columns when fw.
__device__ __forceinline__ float4 ld4d(const void *p, int64_t plane, int64_t hs, int r, int c, int H, int W, bool fh,
                                       bool fw, int dt, bool vec) {
    const int64_t row = plane + (int64_t)(fh ? H - 1 - r : r) * hs;
    if (!fw) return ld4(p, row + c, dt, vec, W - c);
    const int nv = W - c;
    if (nv >= 4) {
        const float4 v = ld4(p, row + (W - 4 - c), dt, vec, 4);
        return make_float4(v.w, v.z, v.y, v.x);
    }
    float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
    if (nv > 0) q.x = ld_elem(p, row + W - 1 - c, dt);
    if (nv > 1) q.y = ld_elem(p, row + W - 2 - c, dt);
    if (nv > 2) q.z = ld_elem(p, row + W - 3 - c, dt);
    return q;
}
__device__ __forceinline__ void st4d(void *p, int64_t plane, int64_t hs, int r, int c, int H, int W, bool fh, bool fw,
                                     int dt, bool vec, float4 v) {
    const int64_t row = plane + (int64_t)(fh ? H - 1 - r : r) * hs;
    if (!fw) { st4(p, row + c, dt, vec, W - c, v); return; }
    const int nv = W - c;
    if (nv >= 4) { st4(p, row + (W - 4 - c), dt, vec, 4, make_float4(v.w, v.z, v.y, v.x)); return; }
    if (nv > 0) st_elem(p, row + W - 1 - c, dt, v.x);
    if (nv > 1) st_elem(p, row + W - 2 - c, dt, v.y);
    if (nv > 2) st_elem(p, row + W - 3 - c, dt, v.z);
}

// softplus with the reference's threshold (fwd kernel :221-224).
__device__ __forceinline__ float softplus20(float x) { return x <= 20.f ? log1pf(__expf(x)) : x; }

// delta -> softplus(delta + bias) in place, d softplus/dx into `sig`; the reference's
// threshold and chain rule (bwd kernel :785-806).  Columns past the image read as 0.
__device__ __forceinline__ void soft4(float4 &x, float4 &sig, float bias, int softplus, int nvalid) {
    float xs[4] = {x.x + bias, x.y + bias, x.z + bias, x.w + bias}, sg[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        sg[e] = 1.f;
        if (softplus && xs[e] <= 20.f) {
            const float t = __expf(xs[e]);       // <= e^20: 1 + t stays finite and exact enough
            sg[e] = __fdividef(t, 1.f + t);      // sigmoid(x) = e^x / (1 + e^x)
            xs[e] = log1pf(t);
        }
        if (e >= nvalid) { xs[e] = 0.f; sg[e] = 0.f; }
    }
    x = make_float4(xs[0], xs[1], xs[2], xs[3]);
    sig = make_float4(sg[0], sg[1], sg[2], sg[3]);
}

// ---- shared-memory tile layouts ---------------------------------------------------
// Per-channel float tiles are [channel][row][Wp]; inside a row the 8 columns of
// strip j are stored as two float4 at 4j and 4L+4j, so the two LDS.128 of the
// L lanes of a row hit consecutive 16-byte words.  The channel stride is padded
// so that the CW channel groups of a warp fall on different banks.
template <int L>
__host__ __device__ constexpr int chan_stride(int rows) {
    const int base = rows * L * STRIP;
    const int want = (4 * L) % 32;
    return base + ((want - base % 32) + 32) % 32;
}
// float offset of the float4 holding columns 4t..4t+3 of a row
template <int L>
__device__ __forceinline__ int pos4(int t) { return (t & 1) * (4 * L) + 4 * (t >> 1); }
// float offset of column c of a row
template <int L>
__device__ __forceinline__ int pos1(int c) { return pos4<L>(c >> 2) + (c & 3); }
// Pair tiles are [slot][row][Wp] float2; the 8 columns of strip j are four
// float4 (two columns x two states) at float2 offsets k*2L + 2j, k = 0..3.
template <int L>
__device__ __forceinline__ int pos2(int c) { return ((c & 7) >> 1) * (2 * L) + 2 * (c >> 3) + (c & 1); }

__device__ __forceinline__ void unpack8(const float *row, int L4, int j, float (&v)[STRIP]) {
    const float4 a = *reinterpret_cast<const float4 *>(row + 4 * j);
    const float4 b = *reinterpret_cast<const float4 *>(row + L4 + 4 * j);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void pack8(float *row, int L4, int j, const float (&v)[STRIP]) {
    *reinterpret_cast<float4 *>(row + 4 * j) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4 *>(row + L4 + 4 * j) = make_float4(v[4], v[5], v[6], v[7]);
}
// A row of 8 float2 parked in two float rows (columns 0-3 in `ra`, 4-7 in `rb`).
__device__ __forceinline__ void park8x2(float *ra, float *rb, int L4, int j, const float2 (&v)[STRIP]) {
    *reinterpret_cast<float4 *>(ra + 4 * j) = make_float4(v[0].x, v[0].y, v[1].x, v[1].y);
    *reinterpret_cast<float4 *>(ra + L4 + 4 * j) = make_float4(v[2].x, v[2].y, v[3].x, v[3].y);
    *reinterpret_cast<float4 *>(rb + 4 * j) = make_float4(v[4].x, v[4].y, v[5].x, v[5].y);
    *reinterpret_cast<float4 *>(rb + L4 + 4 * j) = make_float4(v[6].x, v[6].y, v[7].x, v[7].y);
}
__device__ __forceinline__ void fetch8x2(const float *ra, const float *rb, int L4, int j, float2 (&v)[STRIP]) {
    const float4 a = *reinterpret_cast<const float4 *>(ra + 4 * j);
    const float4 b = *reinterpret_cast<const float4 *>(ra + L4 + 4 * j);
    const float4 c = *reinterpret_cast<const float4 *>(rb + 4 * j);
    const float4 d = *reinterpret_cast<const float4 *>(rb + L4 + 4 * j);
    v[0] = f2(a.x, a.y); v[1] = f2(a.z, a.w); v[2] = f2(b.x, b.y); v[3] = f2(b.z, b.w);
    v[4] = f2(c.x, c.y); v[5] = f2(c.z, c.w); v[6] = f2(d.x, d.y); v[7] = f2(d.z, d.w);
}
__device__ __forceinline__ void unpack8x2(const float2 *row, int L2, int j, float2 (&v)[STRIP]) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float4 q = *reinterpret_cast<const float4 *>(row + k * L2 + 2 * j);
        v[2 * k] = f2(q.x, q.y); v[2 * k + 1] = f2(q.z, q.w);
    }
}

// ---- row scans ---------------------------------------------------------------
// Exclusive carry for a forward (left-to-right) scan of h' = a*h + b across the
// L lanes of a row.  In: this lane's aggregate (P = prod a, H = local result with
// zero carry-in), optionally a second sequence S sharing the multipliers.
// Out: the value of the sequence just left of this lane's strip.
template <int L, bool TWO>
__device__ __forceinline__ void carry_fwd(int j, float2 P, float2 H, float2 S, float2 &cH, float2 &cS,
                                          float2 &Pincl) {
    if constexpr (L == 1) {
        cH = bc(0.f); cS = bc(0.f); Pincl = P;
    } else {
#pragma unroll
        for (int off = 1; off < L; off <<= 1) {
            // lanes without a partner 'off' to the left combine with the identity (1, 0): no branch
            const bool on = j >= off;
            float2 Pp = shfl_up2<L>(P, off);
            float2 Hp = shfl_up2<L>(H, off);
            Pp.x = on ? Pp.x : 1.f; Pp.y = on ? Pp.y : 1.f;
            Hp.x = on ? Hp.x : 0.f; Hp.y = on ? Hp.y : 0.f;
            H = fma2(P, Hp, H);
            if (TWO) {
                float2 Sp = shfl_up2<L>(S, off);
                Sp.x = on ? Sp.x : 0.f; Sp.y = on ? Sp.y : 0.f;
                S = fma2(P, Sp, S);
            }
            P = mul2(P, Pp);
        }
        Pincl = P;
        cH = shfl_up2<L>(H, 1);
        cS = TWO ? shfl_up2<L>(S, 1) : bc(0.f);
        const bool first = j == 0;
        cH.x = first ? 0.f : cH.x; cH.y = first ? 0.f : cH.y;
        cS.x = first ? 0.f : cS.x; cS.y = first ? 0.f : cS.y;
    }
}
// A value c_in entering a row of lanes from outside (a column-tile boundary) reaches
// lane j as P_excl(j) * c_in, P_excl = product of the multipliers of the lanes before it.
// `Pincl` is the inclusive product a scan returned, `e` the value held by the boundary lane.
template <int L>
__device__ __forceinline__ float2 edge_term_fwd(int j, float2 Pincl, float2 e) {
    float2 cP = bc(1.f);
    if constexpr (L > 1) {
        cP = shfl_up2<L>(Pincl, 1);
        cP.x = j == 0 ? 1.f : cP.x; cP.y = j == 0 ? 1.f : cP.y;
        e = make_float2(__shfl_sync(0xffffffffu, e.x, 0, L), __shfl_sync(0xffffffffu, e.y, 0, L));
    }
    return mul2(cP, e);
}
template <int L>
__device__ __forceinline__ float2 edge_term_rev(int j, float2 Pincl, float2 e) {
    float2 cP = bc(1.f);
    if constexpr (L > 1) {
        cP = shfl_down2<L>(Pincl, 1);
        cP.x = j == L - 1 ? 1.f : cP.x; cP.y = j == L - 1 ? 1.f : cP.y;
        e = make_float2(__shfl_sync(0xffffffffu, e.x, L - 1, L), __shfl_sync(0xffffffffu, e.y, L - 1, L));
    }
    return mul2(cP, e);
}

// Same for a reverse (right-to-left) scan: carry = value just right of the strip.
template <int L, bool TWO>
__device__ __forceinline__ void carry_rev(int j, float2 P, float2 H, float2 S, float2 &cH, float2 &cS,
                                          float2 &Pincl) {
    if constexpr (L == 1) {
        cH = bc(0.f); cS = bc(0.f); Pincl = P;
    } else {
#pragma unroll
        for (int off = 1; off < L; off <<= 1) {
            const bool on = j + off < L;
            float2 Pp = shfl_down2<L>(P, off);
            float2 Hp = shfl_down2<L>(H, off);
            Pp.x = on ? Pp.x : 1.f; Pp.y = on ? Pp.y : 1.f;
            Hp.x = on ? Hp.x : 0.f; Hp.y = on ? Hp.y : 0.f;
            H = fma2(P, Hp, H);
            if (TWO) {
                float2 Sp = shfl_down2<L>(S, off);
                Sp.x = on ? Sp.x : 0.f; Sp.y = on ? Sp.y : 0.f;
                S = fma2(P, Sp, S);
            }
            P = mul2(P, Pp);
        }
        Pincl = P;
        cH = shfl_down2<L>(H, 1);
        cS = TWO ? shfl_down2<L>(S, 1) : bc(0.f);
        const bool last = j == L - 1;
        cH.x = last ? 0.f : cH.x; cH.y = last ? 0.f : cH.y;
        cS.x = last ? 0.f : cS.x; cS.y = last ? 0.f : cS.y;
    }
}

// Values of the column just left of a column tile, for the lane that owns the tile's first
// column: h of the previous row, a of this row, h and s of this row.
struct LeftEdge { float2 h_prev, a, h, s; };

// One forward row for a strip: given dl (post-softplus delta), dlu = dl*u, B,
// the previous row (h_up, a_up) and the packed A*log2(e) (+ log2 decay), computes
// a, p and h (and the plain row scan s when WITH_S).
//   a = exp2(dl*A2 + lg2decay)                      (reference fwd kernel :245)
//   h = a*(h_left + h_up - 0.5*(a_up + a_left)*h_diag) + p      (:263-271)
//   s = a*s_left + p                                (:306-327)
template <int L, bool WITH_S>
__device__ __forceinline__ void row_forward(int j, const float (&dl)[STRIP], const float (&dlu)[STRIP],
                                            const float2 (&Bv)[STRIP], float2 A2, float2 lgd,
                                            const float2 (&h_up)[STRIP], const float2 (&a_up)[STRIP],
                                            float2 (&a)[STRIP], float2 (&p)[STRIP], float2 (&h)[STRIP],
                                            float2 (&s)[STRIP], bool has_left, const LeftEdge &le) {
#pragma unroll
    for (int i = 0; i < STRIP; ++i) {
        a[i] = ex2_2(fma2(bc(dl[i]), A2, lgd));
        p[i] = mul2(Bv[i], bc(dlu[i]));
    }
    float2 hdiag0 = bc(0.f), aleft0 = bc(0.f);
    if constexpr (L > 1) {
        hdiag0 = shfl_up2<L>(h_up[STRIP - 1], 1);
        aleft0 = shfl_up2<L>(a[STRIP - 1], 1);
        hdiag0.x = j == 0 ? 0.f : hdiag0.x; hdiag0.y = j == 0 ? 0.f : hdiag0.y;
    }
    if (has_left && j == 0) { hdiag0 = le.h_prev; aleft0 = le.a; }
    // Each strip is folded as two independent 4-column halves so that the serial
    // chains are half as long and twice as many (h and s, low and high half).
    float2 beta[STRIP];
#pragma unroll
    for (int i = 0; i < STRIP; ++i) {
        const float2 al = i ? a[i - 1] : aleft0;
        const float2 hd = i ? h_up[i - 1] : hdiag0;
        const float2 t = mul2(add2(a_up[i], al), hd);
        const float2 kappa = fma2(t, bc(-0.5f), h_up[i]);
        beta[i] = fma2(a[i], kappa, p[i]);
    }
    constexpr int HS = STRIP / 2;
    float2 P0 = a[0], P1 = a[HS], H0 = beta[0], H1 = beta[HS], S0 = p[0], S1 = p[HS];
#pragma unroll
    for (int i = 1; i < HS; ++i) {
        H0 = fma2(a[i], H0, beta[i]);
        H1 = fma2(a[HS + i], H1, beta[HS + i]);
        if (WITH_S) { S0 = fma2(a[i], S0, p[i]); S1 = fma2(a[HS + i], S1, p[HS + i]); }
        P0 = mul2(P0, a[i]);
        P1 = mul2(P1, a[HS + i]);
    }
    float2 ch, cs, Pin;
    carry_fwd<L, WITH_S>(j, mul2(P0, P1), fma2(P1, H0, H1), WITH_S ? fma2(P1, S0, S1) : bc(0.f), ch, cs, Pin);
    if (has_left) {  // h, s of the column left of the tile enter at lane 0 and reach every lane
        ch = add2(ch, edge_term_fwd<L>(j, Pin, le.h));
        if (WITH_S) cs = add2(cs, edge_term_fwd<L>(j, Pin, le.s));
    }
    float2 ch1 = fma2(P0, ch, H0), cs1 = WITH_S ? fma2(P0, cs, S0) : bc(0.f);  // carries into the high half
#pragma unroll
    for (int i = 0; i < HS; ++i) {
        ch = fma2(a[i], ch, beta[i]); h[i] = ch;
        ch1 = fma2(a[HS + i], ch1, beta[HS + i]); h[HS + i] = ch1;
        if (WITH_S) {
            cs = fma2(a[i], cs, p[i]); s[i] = cs;
            cs1 = fma2(a[HS + i], cs1, p[HS + i]); s[HS + i] = cs1;
        }
    }
}

// ---- staging shared by both kernels ---------------------------------------------
// B and C of one row block for every state pair: sB/sC[NPp][RB][Wp] float2.
template <int L>
__device__ __forceinline__ void stage_BC(const Dev &P, int b, int g, int r0, int nr, float2 *sB, float2 *sC,
                                         bool fh, bool fw, int tid, int nthr) {
    const int64_t cs = fw ? P.cshift : 0;
    constexpr int Wp = L * STRIP, T4 = Wp / 4;
    const int items = P.NPp * RB * T4;
    for (int it = tid; it < items; it += nthr) {
        const int t = it % T4, rr = (it / T4) % RB, sp = it / (T4 * RB);
        const int c = 4 * t, n0 = 2 * sp;
        float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0, c0 = b0, c1 = b0;
        if (rr < nr && n0 < P.N) {
            const int r = r0 + rr;
            const int64_t ob = (int64_t)b * P.B_bs + (int64_t)g * P.B_gs + cs, oc = (int64_t)b * P.C_bs + (int64_t)g * P.C_gs + cs;
            b0 = ld4d(P.B, ob + (int64_t)n0 * P.B_ns, P.B_hs, r, c, P.H, P.W, fh, fw, P.io_dt, P.vec & VEC_B);
            c0 = ld4d(P.C, oc + (int64_t)n0 * P.C_ns, P.C_hs, r, c, P.H, P.W, fh, fw, P.io_dt, P.vec & VEC_C);
            if (n0 + 1 < P.N) {
                b1 = ld4d(P.B, ob + (int64_t)(n0 + 1) * P.B_ns, P.B_hs, r, c, P.H, P.W, fh, fw, P.io_dt, P.vec & VEC_B);
                c1 = ld4d(P.C, oc + (int64_t)(n0 + 1) * P.C_ns, P.C_hs, r, c, P.H, P.W, fh, fw, P.io_dt, P.vec & VEC_C);
            }
        }
        const int base = (sp * RB + rr) * Wp + pos2<L>(c);  // columns c, c+1; c+2, c+3 follow 2L float2 later
        *reinterpret_cast<float4 *>(sB + base) = make_float4(b0.x, b1.x, b0.y, b1.y);
        *reinterpret_cast<float4 *>(sB + base + 2 * L) = make_float4(b0.z, b1.z, b0.w, b1.w);
        *reinterpret_cast<float4 *>(sC + base) = make_float4(c0.x, c1.x, c0.y, c1.y);
        *reinterpret_cast<float4 *>(sC + base + 2 * L) = make_float4(c0.z, c1.z, c0.w, c1.w);
    }
}

}  // namespace cs2d

/*
 * cs2d - 2D-CrossScan selective scan for NVIDIA B200 (sm_100a).
 *
 * C ABI of the drop-in replacement for the two operators that
 * longlong-yu/official-cross-scan exposes from its CUDA extension
 * `selective_nd_scan_cuda_oflex` (kernels/selective_nd_scan).  A host binding
 * (the Python module of the same name shipped in this repository, or any FFI)
 * validates tensors, allocates outputs and calls these entry points with raw
 * device pointers.  Nothing here takes or returns a framework type, allocates
 * device memory, or synchronises the stream.
 *
 * All functions return 0 on success and a negative cs2d_status otherwise;
 * cs2d_last_error() gives the message for the calling thread.
 */
#ifndef CS2D_H_
#define CS2D_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CS2D_ABI_VERSION 2
#define CS2D_MAX_DSTATE 16 /* reference: MAX_DSTATE, include/selective_scan_common.h:13 */

typedef enum {
    CS2D_OK = 0,
    CS2D_ERR_INVALID = -1,     /* bad shape / dtype / pointer / stride           */
    CS2D_ERR_UNSUPPORTED = -2, /* valid for the reference, not implemented here  */
    CS2D_ERR_CUDA = -3         /* a CUDA runtime call or the launch failed       */
} cs2d_status;

typedef enum { CS2D_F32 = 0, CS2D_F16 = 1, CS2D_BF16 = 2 } cs2d_dtype;

/*
 * Problem description shared by forward and backward.  It replaces the
 * reference's launch-parameter struct SSMParamsBase
 * (include/cusoflex/selective_scan_oflex.h:4-51), filled there by
 * set_ssm_params_fwd (src/cusoflex/selective_scan_oflex.cpp:37-112).
 *
 * Tensor meaning and layout are the reference's: u (batch, dim, nrows, ncols),
 * delta (batch, delta_dim, nrows, ncols), A (dim, dstate) fp32,
 * B and C (batch, n_groups, dstate, nrows, ncols), D (dim) fp32 or NULL,
 * delta_bias (delta_dim) fp32 or NULL, A_decay (1) fp32 or NULL.
 * Strides are in ELEMENTS (64-bit, the reference uses 32-bit); the innermost
 * (ncols) stride of u, delta, B, C, out/dout must be 1 as the reference
 * requires (selective_scan_oflex.cpp:203-204,227,229,318).
 */
typedef struct {
    int32_t batch, dim, nrows, ncols, dstate, n_groups, delta_dim;
    int32_t io_dtype;       /* cs2d_dtype of u, delta, B, C (and du, ddelta)          */
    int32_t out_dtype;      /* cs2d_dtype of out (fwd) / dout (bwd): io_dtype or F32  */
    int32_t delta_softplus; /* nonzero: delta = softplus(delta + bias), threshold 20  */
    const void *u;      int64_t u_bs, u_ds, u_hs;
    const void *delta;  int64_t delta_bs, delta_ds, delta_hs;
    const float *A;     int64_t A_ds, A_ns;
    const void *B;      int64_t B_bs, B_gs, B_ns, B_hs;
    const void *C;      int64_t C_bs, C_gs, C_ns, C_hs;
    const float *D;          /* may be NULL */
    const float *delta_bias; /* may be NULL */
    const float *A_decay;    /* may be NULL (then 1.0); must be > 0 when given */
} cs2d_problem;

/*
 * Bytes of the saved-state buffer the forward writes and the backward reads
 * (row checkpoints of the state h; for rows of at most 64 columns with more
 * than 8 states also the forward's regrouped fp32 copy of B and C, behind the
 * checkpoints).  It takes the place of the reference's
 * three side tensors x, x_v, x_sd (selective_scan_oflex.cpp:251-258); unlike
 * them it is NOT modified by the backward, so backward may run twice on it.
 * Returns 0 for an invalid problem.
 */
size_t cs2d_saved_bytes(const cs2d_problem *p);

/*
 * Bytes of the scratch buffer the backward needs (one adjoint row per channel
 * and state pair, carried between row blocks).  Contents are undefined before
 * and after a call.  The reference keeps the equivalent state in the x / x_sd
 * tensors it overwrites (selective_scan_bwd_kernel_oflex.cuh:490,726).
 * Returns 0 for an invalid or unsupported problem.
 */
size_t cs2d_bwd_scratch_bytes(const cs2d_problem *p);

/*
 * Forward.  Replaces selective_scan_fwd_cuda<input_t, float, output_t>
 * (include/cusoflex/selective_scan_fwd_kernel_oflex.cuh:376-392) as called by
 * selective_scan_fwd (src/cusoflex/selective_scan_oflex.cpp:275-281).
 *   out   (batch, dim, nrows, ncols) of out_dtype, strides out_bs/ds/hs, inner 1
 *   saved device buffer of cs2d_saved_bytes(p) bytes, 16-byte aligned
 * Launches on `stream` (a cudaStream_t) of the current device; asynchronous.
 */
int cs2d_fwd(const cs2d_problem *p, void *out, int64_t out_bs, int64_t out_ds, int64_t out_hs,
             void *saved, void *stream);

/*
 * Backward.  Replaces selective_scan_bwd_cuda<input_t, float, output_t>
 * (include/cusoflex/selective_scan_bwd_kernel_oflex.cuh:922-938) as called by
 * selective_scan_bwd (src/cusoflex/selective_scan_oflex.cpp:424-430).
 *   dout   (batch, dim, nrows, ncols) of p->out_dtype
 *   scratch device buffer of cs2d_bwd_scratch_bytes(p) bytes, 16-byte aligned;
 *          concurrent calls must not share it
 *   du     (batch, dim, nrows, ncols) of io_dtype
 *   ddelta (batch, dim, nrows, ncols) of io_dtype - at full channel resolution
 *          like the reference kernel; the host reduces it to delta_dim
 *          (selective_scan_oflex.cpp:433-438)
 *   dA (dim, dstate), dB, dC (batch, n_groups, dstate, nrows, ncols): fp32,
 *          contiguous, ACCUMULATED into - the caller zero-fills them, exactly as
 *          the reference host does (selective_scan_oflex.cpp:395,398-399)
 *   dD (dim), ddelta_bias (dim), dA_decay (1): fp32, accumulated into, or NULL
 *   du, ddelta: contiguous.
 * dA_decay reproduces the reference's value (it omits the row-scan term).
 */
int cs2d_bwd(const cs2d_problem *p, const void *dout, int64_t dout_bs, int64_t dout_ds, int64_t dout_hs,
             const void *saved, void *scratch, void *du, void *ddelta, float *dA, float *dB, float *dC,
             float *dD, float *ddelta_bias, float *dA_decay, void *stream);

/*
 * Scan directions for the four-corner CrossScan.  The reference kernel scans one
 * orientation only and leaves "change the scan order per group" as a TODO
 * (include/cusoflex/selective_scan_fwd_kernel_oflex.cuh:140); its caller has to
 * materialise flipped copies.  Here group g (0 <= g < n_groups <= 32) walks the
 * image rows bottom-up when bit g of flip_rows_mask is set and the columns
 * right-to-left when bit g of flip_cols_mask is set, while every tensor stays in
 * IMAGE coordinates (the flips are index maps inside the kernels).  shared_input
 * bit 0: u has dim/n_groups channels that all groups read - channel d of group g
 * reads u channel d - g*dim/n_groups, u_ds being the stride of those channels;
 * bit 1: the same for dout in the backward.  out, du, ddelta keep `dim` channels
 * (one result per direction).
 *
 * Direction merge (merge_w != NULL): the weighted sum over the directions happens
 * inside the kernels.  merge_w holds one fp32 weight per channel (dim values:
 * direction-major, w[g][d]).
 *   forward:  `out` is an fp32 image (batch, dim/n_groups, nrows, ncols)
 *             (p->out_dtype = CS2D_F32) that receives sum_g w[g][d] * y_g[d] - no
 *             per-direction outputs exist.
 *   backward: `dout` is the gradient of that image (dim/n_groups channels, set
 *             shared_input bit 1); `du` is an fp32 image (batch, dim/n_groups, nrows,
 *             ncols) that receives sum_g w*du_g; ddelta, dA, dB, dC, dD, ddelta_bias,
 *             dA_decay come out scaled by w as the chain rule asks; merge_dw (dim fp32
 *             values, zero-filled, may be NULL) receives dw[g][d] = sum dy*y_g[d].
 * Two forms, chosen by `flags`:
 *   0                 the directions run as separate CTAs and ADD onto the merged images with
 *                     fp32 atomics: zero-fill `out` / `du` first; the last bit of the sums
 *                     depends on the order in which the CTAs arrive.
 *   CS2D_DIRS_SERIAL  one CTA owns a channel tile for ALL directions and walks them one
 *                     after the other, so every element of the merged images has a single
 *                     writer: no atomics, the same bits on every run.  For ncols <= 256 the
 *                     images are WRITTEN (they need not be initialised); wider rows run as
 *                     column tiles in several launches, which add onto them: zero-fill them
 *                     first.  Slower (measured +17 % to +24 % on the stage-1 and
 *                     segmentation-scale maps, far more when batch x channel tiles leave
 *                     most SMs idle): a quarter of the CTAs, and the read-modify-write of
 *                     the merged image sits in the write-out path.
 * The deterministic backward (cs2d_bwd_det) is not combined with the merge (dB, dC and the
 * parameter gradients still sum over channel tiles with atomics).
 */
#define CS2D_DIRS_SERIAL 1
typedef struct {
    uint32_t flip_rows_mask, flip_cols_mask;
    int32_t shared_input;
    int32_t flags;           /* 0 or CS2D_DIRS_SERIAL (merge only) */
    const float *merge_w;    /* NULL: no merge */
    float *merge_dw;
} cs2d_dirs;

/* cs2d_fwd / cs2d_bwd with scan directions (dirs may be NULL = cs2d_fwd / cs2d_bwd). */
int cs2d_fwd_dir(const cs2d_problem *p, const cs2d_dirs *dirs, void *out, int64_t out_bs, int64_t out_ds,
                 int64_t out_hs, void *saved, void *stream);
int cs2d_bwd_dir(const cs2d_problem *p, const cs2d_dirs *dirs, const void *dout, int64_t dout_bs,
                 int64_t dout_ds, int64_t dout_hs, const void *saved, void *scratch, void *du, void *ddelta,
                 float *dA, float *dB, float *dC, float *dD, float *ddelta_bias, float *dA_decay,
                 void *stream);

/*
 * Deterministic backward: bit-identical results from run to run.  cs2d_bwd (like
 * the reference, selective_scan_bwd_kernel_oflex.cuh:608-609,770-771,886-901)
 * adds the sums that cross CTAs - dB and dC over the channels of a group, dA, dD,
 * ddelta_bias, dA_decay over the batch - with floating-point atomics, whose order
 * varies.  Here every CTA stores its sums into slots of its own inside
 * det_scratch (cs2d_bwd_det_scratch_bytes(p) bytes, 16-byte aligned, contents
 * undefined before and after) and a second kernel adds them in a fixed order.
 * Results are ADDED to dA, dB, dC, dD, ddelta_bias, dA_decay exactly as in
 * cs2d_bwd (zero-fill them first).  dirs may be NULL.  Limits: ncols <= 256, and
 * for ncols > 64 dstate > 8; otherwise CS2D_ERR_UNSUPPORTED
 * (cs2d_bwd_det_scratch_bytes returns 0).
 */
size_t cs2d_bwd_det_scratch_bytes(const cs2d_problem *p);
int cs2d_bwd_det(const cs2d_problem *p, const cs2d_dirs *dirs, const void *dout, int64_t dout_bs, int64_t dout_ds,
                 int64_t dout_hs, const void *saved, void *scratch, void *det_scratch, void *du, void *ddelta,
                 float *dA, float *dB, float *dC, float *dD, float *ddelta_bias, float *dA_decay, void *stream);

/*
 * Forward that no backward will follow (inference, evaluation).  Same results as
 * cs2d_fwd / cs2d_fwd_dir (dirs may be NULL), but instead of the saved-state
 * buffer it takes a scratch buffer of cs2d_fwd_only_scratch_bytes(p) bytes
 * (16-byte aligned, contents undefined before and after): one rolling row of h
 * per channel and state pair instead of one per four image rows.  The reference
 * always writes its three side tensors (selective_scan_oflex.cpp:251-258,
 * selective_scan_fwd_kernel_oflex.cuh:289-295); it has no such mode.
 */
size_t cs2d_fwd_only_scratch_bytes(const cs2d_problem *p);
int cs2d_fwd_only(const cs2d_problem *p, const cs2d_dirs *dirs, void *out, int64_t out_bs, int64_t out_ds,
                  int64_t out_hs, void *scratch, void *stream);

/*
 * Backward without any allocation on the caller's side: identical to cs2d_bwd
 * except that the scratch buffer is a fixed device array inside the library
 * (CS2D_NOALLOC_SCRATCH_BYTES per GPU, held from library load to process exit).
 * It is meant for hosts that cannot call cudaMalloc where they run the backward
 * - a runtime that owns all device memory through its own pool, a plugin invoked
 * from an allocator callback, a thin FFI stub that only sees its arguments.
 * This entry point has no counterpart in the reference (whose host binding
 * allocates with torch).
 *   - inputs, saved state and ALL outputs are still passed by the caller;
 *   - problems whose cs2d_bwd_scratch_bytes() exceeds CS2D_NOALLOC_SCRATCH_BYTES
 *     are rejected with CS2D_ERR_UNSUPPORTED and a message (split the batch);
 *   - the first call on a device looks up the array's device address (a host
 *     call, no allocation); make that first call before starting a stream capture;
 *   - nothing needs clearing between calls, but the array is shared: calls that
 *     may overlap on the same GPU (different streams or threads) race on it.
 */
#define CS2D_NOALLOC_SCRATCH_BYTES (32u << 20)
int cs2d_bwd_noalloc(const cs2d_problem *p, const void *dout, int64_t dout_bs, int64_t dout_ds,
                     int64_t dout_hs, const void *saved, void *du, void *ddelta, float *dA, float *dB,
                     float *dC, float *dD, float *ddelta_bias, float *dA_decay, void *stream);

/*
 * Reads and clears the device-side status word of the current device
 * (synchronises with the device).  0 = no kernel reported a problem; nonzero =
 * a kernel gave up on a bounded wait (bit 0: for one of its asynchronous copies,
 * bit 1: for the tiles its staging warps hand to its compute warps) and
 * returned early, so the outputs of the calls since the last check are invalid
 * (cs2d_last_error() then describes it).  Negative: the query itself failed.
 * The reference has no counterpart; its kernels contain no waits.
 */
int cs2d_device_status(void);

/* Message of the last failure on the calling thread ("" if none). */
const char *cs2d_last_error(void);

/* CS2D_ABI_VERSION the library was built with. */
int cs2d_abi_version(void);

/* Number of kernels this library has launched in this process (for benchmarks). */
int64_t cs2d_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* CS2D_H_ */

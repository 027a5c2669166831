/* Allocation-free entry point of the rumus_b200 CUDA library.
 *
 * This entry point has no counterpart in the reference framework.
 *
 * Who it is for: code that may not allocate device memory at the moment it needs a LayerNorm /
 * RMSNorm backward — a real-time or safety-rated host loop with a fixed memory budget, a plugin
 * running inside another engine's memory pool, a caller that holds a lock under which
 * cudaMalloc (which can synchronise the whole device) is forbidden.  The regular entry point
 * rb_norm_bwd expects the caller to hand in a scratch buffer for the per-block partial sums of
 * d_gamma / d_beta; such callers have nowhere to get one.  This variant brings its own.
 *
 * What it does: same computation and same arguments as rb_norm_bwd, minus the scratch pointer.
 * The partial sums go to a fixed array compiled into the library
 * (RB_NORM_BWD_NOALLOC_MAX_PARTIALS x 2 x RB_NORM_BWD_NOALLOC_MAX_DIM floats = 2 MiB).  The
 * array is part of the library image: every GPU that loads the library keeps those 2 MiB until
 * the process exits.  The call performs no cudaMalloc / cudaFree and uses no allocating library
 * routine; inputs and outputs are still the caller's buffers.
 *
 * Limits and rules:
 *  - row length D must be in 1..RB_NORM_BWD_NOALLOC_MAX_DIM; anything larger is refused with
 *    RB_NOALLOC_ERR_TOO_LARGE and a message on stderr (nothing is launched);
 *  - the first call on each device looks up the device address of the built-in array (with that
 *    device current) and caches it; make that first call before starting any stream capture;
 *  - the grid is limited to RB_NORM_BWD_NOALLOC_MAX_PARTIALS (64) blocks, one partial row each, so
 *    on a 148-SM GPU this variant runs slower than rb_norm_bwd (which uses two blocks per SM): it
 *    trades speed for a fixed footprint;
 *  - all calls on a device share the one array and it keeps the previous call's contents.
 *    Nothing in it has to start at zero — every partial row that is read was written earlier in
 *    the same call — but two calls that overlap on the GPU (different streams, no ordering
 *    between them) race on it.  Order them on one stream or with events.
 *
 * Arguments (all pointers are device pointers; dtype: 0 = fp32, 1 = fp16, 2 = bf16):
 *   rms     0 = LayerNorm, 1 = RMSNorm
 *   x       [rows, D]  the tensor that was normalised in forward
 *   dy      [rows, D]  gradient of the output
 *   gamma   [D]        scale
 *   stats   [rows, 2]  fp32 (mean, 1/std) saved by rb_norm_fwd
 *   dres    [rows, D]  optional gradient to add to dx (may be null)
 *   dx      [rows, D]  out
 *   dgamma  [D]        out
 *   dbeta   [D]        out (ignored for RMSNorm, may be null)
 *   stream  cudaStream_t
 * Returns 0 on success, one of the RB_NOALLOC_ERR_* codes, or 3000 + a cudaError_t.
 */
#ifndef RUMUS_B200_NOALLOC_H_
#define RUMUS_B200_NOALLOC_H_

#define RB_NORM_BWD_NOALLOC_MAX_PARTIALS 64
#define RB_NORM_BWD_NOALLOC_MAX_DIM 4096

#define RB_NOALLOC_ERR_TOO_LARGE 40
#define RB_NOALLOC_ERR_SYMBOL 41
#define RB_NOALLOC_ERR_DEVICE 42

#ifdef __cplusplus
extern "C" {
#endif

int rb_norm_bwd_noalloc(int dtype, int rms, const void* x, const void* dy, const void* gamma,
                        const float* stats, const void* dres, void* dx, void* dgamma, void* dbeta,
                        long long rows, int D, void* stream);

/* Largest row length the built-in scratch supports. */
int rb_norm_bwd_noalloc_max_dim(void);

#ifdef __cplusplus
}
#endif
#endif /* RUMUS_B200_NOALLOC_H_ */

/*
 * fm_scan_b200 -- C ABI of the B200 (sm_100a) first-order linear-recurrence scan.
 *
 * This is the drop-in boundary for the scan path of lexionbear/fm.  The reference binds
 * two C++ functions into Python (fm/scan/fm_scan.py:8-16,34-35):
 *
 *   at::Tensor fm_scan_forward (gates, tokens, initial_state, out)          fm/scan/fm_scan.cuh:344-358
 *   void       fm_scan_backward(gates, outGrad, firstPropGrad, tokenGradOut,
 *                               cached_output, input_tokens, gateGradOut)   fm/scan/fm_scan.cuh:361-381
 *
 * The functions below are what those two would call instead of the reference's
 * fmscan_launch<> (fm/scan/fm_scan.cuh:248-331): raw device pointers, sizes, a dtype tag
 * and a stream.  No torch types appear here.
 *
 * Conventions (all entry points unless stated otherwise)
 *  - return value: 0 (FMS_OK) or an fms_status code; nothing throws;
 *  - nothing allocates or frees device memory, nothing synchronises the device or the
 *    stream; kernels are enqueued on `stream` of the CURRENT device (the caller selects
 *    the device; the reference never did, fm/scan/fm_scan.cuh:271-272);
 *  - tensors are contiguous, row-major, last axis = time; any T >= 0 and any number of
 *    rows (the reference accepted 13 powers of two only, fm/scan/fm_scan.cuh:275-329);
 *    offsets are 64-bit (the reference's were 32-bit, fm/scan/fm_scan.cuh:76-82);
 *  - `dtype` is the STORAGE type of the big tensors; arithmetic is fp32 throughout
 *    (fm/scan/fm_scan.cuh:14-40); per-row carries (h0, h_last, carry_in, grad_h0, P, S)
 *    are always fp32;
 *  - pointers must be aligned to their element size.  Rows that are 16-byte aligned in
 *    every tensor (T*sizeof(element) % 16 == 0 and 16-byte aligned bases) take the fully
 *    vectorised path; everything else takes the masked path with identical results.
 *
 * PLAIN mode:   h[r,t] = a[r,t] * h[r,t-1] + x[r,t]                    rows r < R
 * FM mode   :   h[b,m,d,t] = g[b,m,t] * h[b,m,d,t-1] + (1 - g[b,m,t]) * x[b,d,t]
 *               (the reference's operator, fm/scan/fm_pytorch.py:19-42)
 */
#ifndef FM_SCAN_B200_H_
#define FM_SCAN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque stream handle: pass a cudaStream_t (NULL = the legacy default stream). */
typedef void *fms_stream_t;

typedef enum fms_dtype {
    FMS_F32 = 0,  /* float          (reference: <float, float>,               fm_scan.cuh:338-339) */
    FMS_F16 = 1,  /* __half         (reference: <__half, at::Half>,           fm_scan.cuh:336-337) */
    FMS_BF16 = 2  /* __nv_bfloat16  (reference: <__nv_bfloat16, at::BFloat16>, fm_scan.cuh:334-335) */
} fms_dtype;

typedef enum fms_status {
    FMS_OK = 0,
    FMS_ERR_BAD_SHAPE = 1,      /* negative size, or a size product that overflows int64          */
    FMS_ERR_BAD_DTYPE = 2,      /* dtype tag not in fms_dtype (reference: fm_scan.cuh:340-341)    */
    FMS_ERR_NULL_POINTER = 3,   /* a required pointer is NULL while the problem is non-empty      */
    FMS_ERR_MISALIGNED = 4,     /* a pointer is not aligned to its element size                   */
    FMS_ERR_LAUNCH = 5,         /* the CUDA runtime refused a launch or a copy (see fms_last_cuda_error) */
    FMS_ERR_WORKSPACE = 6,      /* workspace pointer NULL/misaligned or smaller than the query said */
    FMS_ERR_TOO_LARGE = 7,      /* problem exceeds a stated fixed capacity                        */
    FMS_ERR_NO_DEVICE = 8       /* no CUDA device / wrong architecture (needs sm_100)              */
} fms_status;

/* Library version (major*10000 + minor*100 + patch) and a static description of a status. */
int fms_version(void);
const char *fms_status_string(int status);
/* The cudaError_t (as int) recorded by the last failing runtime call of this thread, 0 if none. */
int fms_last_cuda_error(void);
/*
 * Launch-shape knobs (warps per row, tiles per step, the persistent walk, ...) can be forced with
 * FMS_TUNE_* environment variables.  The library reads them once, at its first launch in the
 * process; this call reads them again (tests and tuning sweeps use it; it is not synchronised
 * with launches running on other threads).  No reference counterpart: the reference's launch
 * geometry is compile-time (fm/scan/fm_scan.cuh:221-244).
 */
void fms_tune_reload(void);

/* ------------------------------------------------------------------ PLAIN mode, one GPU ---- */

/*
 * Forward scan.  Replaces the launch inside fm_scan_forward (fm/scan/fm_scan.cuh:344-358) for
 * the layout gates, tokens, states : (rows, T).
 *   h0      nullable; per-row initial state h[r,-1] (reference: initial_state,
 *           fm/scan/fm_scan.py:47-51; NULL = zeros as fm_scan.py:48)
 *   h_last  nullable; receives h[r,T-1] in fp32 before rounding to storage (equals h0 when T == 0)
 */
int fms_plain_forward(const void *gates, const void *tokens, const float *h0, void *states,
                      float *h_last, int64_t rows, int64_t T, int dtype, fms_stream_t stream);

/*
 * Backward scan.  Replaces the launch inside fm_scan_backward (fm/scan/fm_scan.cuh:361-381) plus
 * the reductions of fm/scan/fm_scan.py:75-78, which are the identity in this layout.
 *   delta_t = grad_states_t + a_{t+1} delta_{t+1};  grad_tokens_t = delta_t;
 *   grad_gates_t = delta_t * h_{t-1}   (h_{-1} = h0)
 *   states      the forward output (reference: cached_output)
 *   h0          nullable; the forward initial state (the reference passed zeros here,
 *               fm/scan/fm_scan.py:65, which is only right when the forward h0 was zero)
 *   carry_in    nullable; a_T * delta_T flowing in from positions beyond this block (split along T)
 *   grad_h0     nullable; receives a_0 * delta_0 = dL/dh0 (the reference returns None,
 *               fm/scan/fm_scan.py:80-81)
 */
int fms_plain_backward(const void *gates, const void *states, const void *grad_states,
                       const float *h0, const float *carry_in, void *grad_gates,
                       void *grad_tokens, float *grad_h0, int64_t rows, int64_t T, int dtype,
                       fms_stream_t stream);

/*
 * Carries of a block of T positions, without writing states (first pass of the split-along-T
 * scheme; the reference has no counterpart, its longest sequence is one CTA's serial chunk
 * loop, fm/scan/fm_scan.cuh:84,211-216).
 *   P[r] = prod_t a[r,t]         S[r] = h[r,T-1] given h[r,-1] = 0
 * so that for any carry-in  h[r,T-1] = P[r]*h_in + S[r].
 */
int fms_plain_reduce(const void *gates, const void *tokens, float *P, float *S, int64_t rows,
                     int64_t T, int dtype, fms_stream_t stream);

/*
 * Reverse carries of a block: S_rev[r] = a_0 * delta_0 given carry_in = 0 (P is the same product
 * as in fms_plain_reduce and may be NULL), so that grad_h0 = P*carry_in + S_rev.
 */
int fms_plain_reduce_reverse(const void *gates, const void *grad_states, float *P, float *S_rev,
                             int64_t rows, int64_t T, int dtype, fms_stream_t stream);

/*
 * Fold the carries of `nchunks` consecutive blocks of every row into the carry-in of each block.
 *   P, S      : (nchunks, rows) fp32, chunk-major (the layout an all-gather over ranks produces)
 *   carry0    : nullable (rows) carry entering the first block in scan order
 *   carry_out : (nchunks, rows); carry_out[k] is the carry entering block k
 *   total     : nullable (rows); the carry leaving the last block in scan order
 *   reverse   : 0 = forward order (block k receives blocks < k), 1 = reverse (receives blocks > k)
 */
int fms_combine_carries(const float *P, const float *S, const float *carry0, float *carry_out,
                        float *total, int64_t nchunks, int64_t rows, int reverse,
                        fms_stream_t stream);

/* ------------------------------------------------------------------ FM mode, one GPU ------- */

/*
 * The reference's literal operator (fm/scan/fm_pytorch.py:19-42, fm/scan/fm_scan.cuh:42-218):
 *   gates g (B,M,L), tokens x (B,D,L), h0 (B,M,D) fp32 or NULL, states h (B,M,D,L)
 *   h[b,m,d,t] = g[b,m,t] * h[b,m,d,t-1] + (1 - g[b,m,t]) * x[b,d,t]
 * Replaces the launch inside fm_scan_forward (fm/scan/fm_scan.cuh:344-358) for that layout; the
 * token weight is applied in fp32 as the token is unpacked (fm/scan/fm_scan.cuh:116).
 */
int fms_fm_forward(const void *gates, const void *tokens, const float *h0, void *states, int64_t B,
                   int64_t M, int64_t D, int64_t L, int dtype, fms_stream_t stream);

/*
 * FM backward with the gradient reductions fused: replaces fm_scan_backward
 * (fm/scan/fm_scan.cuh:361-381) AND the two full-size temporaries plus sums of
 * fm/scan/fm_scan.py:70-78.
 *   grad_gates  (B,M,L) = sum_d (h[b,m,d,t-1] - x[b,d,t]) * delta[b,m,d,t]
 *   grad_tokens (B,D,L) = sum_m (1 - g[b,m,t]) * delta[b,m,d,t]
 *   grad_h0     (B,M,D) fp32, nullable = g_0 * delta_0
 * h0 is the forward initial state (h[.,-1]); the reference used zeros there
 * (fm/scan/fm_scan.cuh:195-196 with fm/scan/fm_scan.py:65).
 * The sums are accumulated in fp32 with atomic vector reductions (their order, hence the last
 * bits, can differ from run to run).  fp32 outputs are accumulated in place; fp16/bf16 outputs
 * need fms_fm_backward_workspace_bytes() of caller scratch (fp32 accumulators, cast at the end).
 */
size_t fms_fm_backward_workspace_bytes(int64_t B, int64_t M, int64_t D, int64_t L, int dtype);
int fms_fm_backward(const void *gates, const void *tokens, const void *states, const void *grad_states,
                    const float *h0, void *grad_gates, void *grad_tokens, float *grad_h0, int64_t B,
                    int64_t M, int64_t D, int64_t L, int dtype, void *workspace, size_t workspace_bytes,
                    fms_stream_t stream);

/*
 * FM backward WITHOUT the reductions, for the unmodified reference caller: fm_scan_backward's own
 * output contract (fm/scan/fm_scan.cuh:184-207) is two (B,M,D,L) tensors
 *   grad_tokens_full[b,m,d,t] = (1 - g[b,m,t]) * delta[b,m,d,t]
 *   grad_gates_full [b,m,d,t] = (h[b,m,d,t-1] - x[b,d,t]) * delta[b,m,d,t]
 * which FM_Scan.backward then sums over m and d itself (fm/scan/fm_scan.py:70-78).  Same inputs as
 * fms_fm_backward; no workspace.  It moves the two full-size outputs that fms_fm_backward exists to
 * avoid, so prefer that one wherever the caller can take reduced gradients.
 */
int fms_fm_backward_unreduced(const void *gates, const void *tokens, const void *states, const void *grad_states,
                              const float *h0, void *grad_gates_full, void *grad_tokens_full, float *grad_h0,
                              int64_t B, int64_t M, int64_t D, int64_t L, int dtype, fms_stream_t stream);

/*
 * Read-out of the layer around the scan WITHOUT materialising the states: what
 * fm/scan/fm_scan.py:122-131 computes as states (B,M,D,L) -> RMS norm over D -> contraction with
 * the output weight over M, for callers that need only the layer output (inference).
 *   out[b,d,t] = sum_m w[b,m,t] * rsqrt(mean_d h[b,m,d,t]^2 + eps) * h[b,m,d,t]     (mem_norm != 0)
 *   out[b,d,t] = sum_m w[b,m,t] * h[b,m,d,t]                                        (mem_norm == 0)
 * with h the FM-mode states of (gates, tokens, h0).  gates and out_weight are (B,M,L), tokens and
 * out are (B,D,L), all of the storage dtype.  The scan is recomputed in two passes (sum of
 * squares, then read-out); HBM traffic is the four small tensors plus fp32 scratch of
 * fms_fm_readout_workspace_bytes().  Arithmetic is fp32 throughout, including the norm, which the
 * reference evaluates in the storage dtype.  Requires 16-byte aligned rows (L * element size
 * % 16 == 0, aligned bases); otherwise FMS_ERR_MISALIGNED is returned and nothing is launched.
 */
size_t fms_fm_readout_workspace_bytes(int64_t B, int64_t M, int64_t D, int64_t L, int dtype);
int fms_fm_readout(const void *gates, const void *tokens, const void *out_weight, const float *h0, void *out,
                   int64_t B, int64_t M, int64_t D, int64_t L, int dtype, int mem_norm, float eps,
                   void *workspace, size_t workspace_bytes, fms_stream_t stream);

/*
 * The same layer for training (fm/scan/fm_scan.py:122-131 followed by autograd).
 * fms_fm_layer_forward: one recomputing pass for the norm, then one pass that writes the
 * NORMALISED states (the tensor the reference's layer returns) and the output together.
 *   states_norm (B,M,D,L) out;  rnorm (B,M,L) fp32 out, the norm factor (NULL allowed iff
 *   mem_norm == 0);  workspace: fms_fm_readout_workspace_bytes().
 * fms_fm_layer_backward: gradients of gates (B,M,L), tokens (B,D,L), out_weight (B,M,L) and h0
 * from grad_out (B,D,L) and, optionally, grad_states_norm (B,M,D,L; NULL when the caller did not
 * use the returned states).  The gradient of the raw states is generated inside the reverse scan,
 *   G = r*(Ghn - hn*c),  Ghn = grad_states_norm + w*grad_out,  c = mean_d(Ghn*hn),
 * so the only (B,M,D,L) tensors read are states_norm (twice) and grad_states_norm if given;
 * the reference's autograd reads and writes ~10 such tensors.  Pass rnorm == NULL iff the forward
 * ran with mem_norm == 0.  Same alignment rule as fms_fm_readout.
 */
int fms_fm_layer_forward(const void *gates, const void *tokens, const void *out_weight, const float *h0, void *out,
                         void *states_norm, float *rnorm, int64_t B, int64_t M, int64_t D, int64_t L, int dtype,
                         int mem_norm, float eps, void *workspace, size_t workspace_bytes, fms_stream_t stream);
size_t fms_fm_layer_backward_workspace_bytes(int64_t B, int64_t M, int64_t D, int64_t L, int dtype);
int fms_fm_layer_backward(const void *gates, const void *tokens, const void *out_weight, const void *states_norm,
                          const float *rnorm, const void *grad_out, const void *grad_states_norm, const float *h0,
                          void *grad_gates, void *grad_tokens, void *grad_out_weight, float *grad_h0, int64_t B,
                          int64_t M, int64_t D, int64_t L, int dtype, void *workspace, size_t workspace_bytes,
                          fms_stream_t stream);

/* ------------------------------------------------------------ channel-last layout (B, T, D) ---- */

/*
 * The plain scan on tensors laid out (B, T, D): one recurrence per (b, d) along T, channels
 * contiguous.  This is the layout the reference's layer receives before it transposes to
 * (B, ., L) for every call (fm/scan/fm_scan.py:118-119); scanning it directly removes those
 * transposes.  h0, h_last, grad_h0: (B, D) fp32, nullable.  Time is cut into chunks (carries of
 * every chunk, fold, scan from the true carry-in), which needs fms_btd_workspace_bytes() of
 * caller scratch.  D * element size must be a multiple of 16 bytes and the bases 16-byte
 * aligned (FMS_ERR_MISALIGNED otherwise).
 */
size_t fms_btd_workspace_bytes(int64_t B, int64_t T, int64_t D, int dtype);
int fms_btd_forward(const void *gates, const void *tokens, const float *h0, void *states, float *h_last,
                    int64_t B, int64_t T, int64_t D, int dtype, void *workspace, size_t workspace_bytes,
                    fms_stream_t stream);
int fms_btd_backward(const void *gates, const void *states, const void *grad_states, const float *h0,
                     void *grad_gates, void *grad_tokens, float *grad_h0, int64_t B, int64_t T, int64_t D,
                     int dtype, void *workspace, size_t workspace_bytes, fms_stream_t stream);

/* ------------------------------------------------- few, long rows: split inside one GPU ---- */

/*
 * With fewer rows than the GPU has warps to fill (a handful of very long sequences), one warp
 * per row leaves most of the machine idle.  The split entry points cut every row into `nseg`
 * segments and run three launches: carries of every segment, a fold per row, then the ordinary
 * scan of every segment from its true carry-in.  Results equal the unsplit entry points' up to
 * fp32 re-association of the carries.  The reference has no counterpart (one CTA walks a whole
 * row serially, fm/scan/fm_scan.cuh:84).
 *
 * fms_plain_split_segments: segments per row the library would use for this shape (1 = the
 * split does not pay; call the ordinary entry points).
 * fms_plain_split_workspace_bytes: device scratch the split entry points need for this shape
 * (3 fp32 per segment, rounded up; 0 when segments == 1).  The caller owns the scratch; it may
 * be reused by the next call on the same stream.
 * Arguments of the two entry points are those of fms_plain_forward / fms_plain_backward plus
 * the scratch.  With segments == 1 they forward to the ordinary entry points.
 * fms_plain_split_recommended: 1 when the split is expected to beat the ordinary entry points on
 * this GPU (measured rule: fewer than one row per four SMs, and long enough to split), else 0;
 * the torch shim routes by it.  The split entry points themselves honour
 * fms_plain_split_segments whenever they are called.
 */
int64_t fms_plain_split_segments(int64_t rows, int64_t T, int dtype);
int fms_plain_split_recommended(int64_t rows, int64_t T, int dtype);
size_t fms_plain_split_workspace_bytes(int64_t rows, int64_t T, int dtype);
int fms_plain_forward_split(const void *gates, const void *tokens, const float *h0, void *states,
                            float *h_last, int64_t rows, int64_t T, int dtype, void *workspace,
                            size_t workspace_bytes, fms_stream_t stream);
int fms_plain_backward_split(const void *gates, const void *states, const void *grad_states,
                             const float *h0, const float *carry_in, void *grad_gates,
                             void *grad_tokens, float *grad_h0, int64_t rows, int64_t T, int dtype,
                             void *workspace, size_t workspace_bytes, fms_stream_t stream);

/*
 * Forward scan of few, long rows for callers that must not allocate device memory.
 * (No counterpart in the reference.)
 *
 * Some hosts of this library cannot hand it scratch: a plugin inside a serving framework that
 * owns every byte of device memory and forbids its plugins the CUDA allocator; a control loop
 * that cannot afford the device-wide synchronisation cudaMalloc implies; a process whose memory
 * pool has already taken the whole GPU, so that an allocation would simply fail.  For them this
 * entry point does what fms_plain_forward_split does, with the per-segment carries kept in a
 * fixed array inside the library's device image instead of a caller workspace.  It calls no
 * cudaMalloc / cudaFree and no allocating library routine; inputs and outputs are still the
 * caller's.
 *
 * Limit: at most FMS_STATIC_SCRATCH_MAX_UNITS = 4096 scan units (rows x segments per row); the
 * array is 3 x 4096 fp32 = 48 KiB and every GPU that loads the library holds it until the
 * process exits.  When the library's usual plan (fms_plain_split_segments) would need more units
 * than that, this entry point re-plans with fewer, longer segments -- at most 4096 / rows per
 * row -- so every shape with rows <= 2048 is accepted; with more rows than that (and a shape that
 * would be split at all) the call is refused with FMS_ERR_TOO_LARGE and nothing is launched.
 * Shapes that need no split (segments == 1) use no scratch and are always accepted.
 *
 * Set-up: the first call on each device looks up the array's device address (once per device,
 * with that device current) and caches it.  Make that first call during initialisation, before
 * any stream capture is begun on the device.  The cached address belongs to the device's current
 * primary context: a host that resets the device (cudaDeviceReset) must not call this entry
 * point again in the same process.
 *
 * Sharing: all calls on a device use the same array and it keeps the last call's contents.
 * Nothing in it has to start at zero -- every call overwrites each slot it later reads -- but
 * two calls whose kernels overlap on the GPU (different streams, no ordering between them)
 * race on it.  Order such calls on one stream or with events.
 */
#define FMS_STATIC_SCRATCH_MAX_UNITS 4096
int fms_plain_forward_split_static(const void *gates, const void *tokens, const float *h0,
                                   void *states, float *h_last, int64_t rows, int64_t T, int dtype,
                                   fms_stream_t stream);

/* --------------------------------------- carry exchange over peer-mapped memory (one box) ---- */

/*
 * The exchange step of the split-along-T scan without a collective library: every rank owns a
 * buffer of fms_peer_exchange_bytes() that all ranks have mapped (CUDA IPC / symmetric memory,
 * zero-initialised once).  No reference counterpart (the reference is single-GPU).
 *
 * fms_peer_publish: store this block's carries (P, S) -- forward (reverse = 0) or reverse
 * (reverse = 1; S is then the reverse carry) -- into slot `rank` of every peer's buffer and raise
 * a flag there.  `peer_buffers` is a HOST array of `world` device pointers: rank p's buffer as
 * mapped in this process (entry `rank` is the local buffer).  Plain peer stores only.
 *
 * fms_peer_wait_fold: wait until the blocks this rank depends on (those before it for forward,
 * after it for reverse) have published exchange number `exchange`, polling flags in LOCAL memory,
 * then fold their carries with `carry0` (nullable; the carry entering the first block in scan
 * order) into carry_out (rows), and acknowledge the exchange to every rank (peer stores).
 *
 * Numbering and back-pressure: `exchange` numbers start at 1 and grow by one per exchange and
 * direction on ALL ranks alike.  There are two generations of slots (by parity of the number), so
 * exchange e+2 reuses the slots of e.  fms_peer_publish(e) therefore first waits until every rank
 * that reads this rank's slot has acknowledged e-2: a rank runs at most one exchange ahead of the
 * slowest rank that reads from it, whatever the mix of directions (forward-only loops included).
 *
 * Every wait is bounded by `max_wait_seconds` (<= 30; 2 if out of range) and polls local memory
 * only.  When something goes wrong the kernel still ends normally and the FIRST fault is written
 * to the local buffer's status word (fms_peer_exchange_status_offset() bytes into the buffer;
 * the host reads it):
 *   FMS_PEER_ERR_WAIT_TIMEOUT(_REVERSE)  a block this rank depends on was not published in time;
 *                                        carry0 is passed through to carry_out
 *   FMS_PEER_ERR_OVERRUN                 a slot already held a later exchange than the one asked
 *                                        for (the numbering was broken); carry0 is passed through
 *   FMS_PEER_ERR_ACK_TIMEOUT             a reader did not acknowledge e-2 in time; nothing is
 *                                        published (the slot may still be in use)
 * A fold that saw a fault, or a non-zero status word, sends no acknowledgement.  After a fault the
 * exchange numbers of the ranks no longer agree: build new buffers.
 */
#define FMS_MAX_PEERS 8
#define FMS_PEER_ERR_WAIT_TIMEOUT 1
#define FMS_PEER_ERR_WAIT_TIMEOUT_REVERSE 2
#define FMS_PEER_ERR_OVERRUN 3
#define FMS_PEER_ERR_ACK_TIMEOUT 4
size_t fms_peer_exchange_bytes(int64_t rows, int world);
size_t fms_peer_exchange_status_offset(int64_t rows, int world);
int fms_peer_publish(const float *P, const float *S, int64_t rows, void *const *peer_buffers, int world, int rank,
                     int reverse, uint32_t exchange, double max_wait_seconds, fms_stream_t stream);
int fms_peer_wait_fold(void *const *peer_buffers, const float *carry0, float *carry_out, int64_t rows, int world,
                       int rank, int reverse, uint32_t exchange, double max_wait_seconds, fms_stream_t stream);

/* ------------------------- split along T as one kernel per direction (one box, peer memory) ---- */

/*
 * The whole split-along-T step of one rank in ONE launch per direction: carry pass, exchange of
 * the carries over peer-mapped memory and scan pass, fused row by row, so that the second pass
 * finds the row's operands still in L2 and the block costs the HBM traffic of an unsplit scan
 * (3 element passes forward, 5 backward, instead of 5 and 7 with fms_plain_reduce + exchange +
 * fms_plain_forward).  No reference counterpart (the reference is single-GPU and stops at 131072
 * steps, fm/scan/fm_scan.cuh:323-329).
 *
 * Every rank owns a buffer of fms_tsplit_exchange_bytes(rows, world) that all ranks have mapped
 * (symmetric memory / CUDA IPC), zeroed once before first use; `peer_buffers` is a HOST array of
 * the `world` device pointers as mapped in this process.  Rank k holds time block k of every row:
 * gates, tokens, states ... are this rank's (rows, T) blocks.  All ranks call with the same
 * `exchange` number, counted from 1 per direction, and must be running concurrently on DIFFERENT
 * GPUs (the kernels wait on one another; never run two ranks as separate launches on one GPU
 * unless an earlier rank's kernel has finished before a later one starts).
 *
 * fms_tsplit_forward:  h0 (rank 0 only, nullable) is the state before the first block;
 *                      h_in_out (rows, fp32) receives the carry that entered this block.
 * fms_tsplit_backward: h_in is that carry; grad_h0 (nullable, meaningful on rank 0) receives the
 *                      carry leaving this block towards earlier time, a_0 * delta_0.
 *
 * Requirements: T * element size a multiple of 16 bytes and 16-byte aligned tensors
 * (FMS_ERR_MISALIGNED otherwise: use the three-step path), T >= 1.  Peer traffic is plain stores
 * into peer buffers and local loads.  Waits are bounded by max_wait_seconds (<= 30; 2 if out of
 * range); faults are reported in the local buffer's status word
 * (fms_tsplit_exchange_status_offset) with the FMS_PEER_ERR_* codes, the kernel always ends, and
 * the outputs of rows whose carries did not arrive are computed from a zero carry.  Slot
 * generations and acknowledgements work as for fms_peer_publish: a rank runs at most one exchange
 * ahead of the slowest rank that reads from it.
 */
size_t fms_tsplit_exchange_bytes(int64_t rows, int world);
size_t fms_tsplit_exchange_status_offset(int64_t rows, int world);
int fms_tsplit_forward(const void *gates, const void *tokens, const float *h0, void *states, float *h_in_out,
                       int64_t rows, int64_t T, int dtype, void *const *peer_buffers, int world, int rank,
                       uint32_t exchange, double max_wait_seconds, fms_stream_t stream);
int fms_tsplit_backward(const void *gates, const void *states, const void *grad_states, const float *h_in,
                        void *grad_gates, void *grad_tokens, float *grad_h0, int64_t rows, int64_t T, int dtype,
                        void *const *peer_buffers, int world, int rank, uint32_t exchange, double max_wait_seconds,
                        fms_stream_t stream);

/* ------------------------------------------------------- host-buffer pipeline (one GPU) ---- */

/*
 * Forward + backward with inputs and outputs in HOST memory, for callers whose tensors live
 * on the host (the reference's CPU path fm/scan/fm_pytorch.py:3-42 is such a caller's
 * alternative).  Rows are cut into blocks (up to 32); host->device copies, the two kernels and
 * device->host copies of consecutive blocks overlap on three internal streams (both PCIe
 * directions busy at once).  The reference has no counterpart: its extension only accepts
 * CUDA tensors (fm/scan/fm_scan.cuh:346-348).
 *
 * fms_pipeline_create makes the streams and events on the CURRENT device.  It allocates no
 * device memory: the staging area is the caller's `workspace` (device memory, 256-byte
 * aligned).  The block size follows from its size: a block of r rows needs
 * 12 * round_up(r*T*sizeof(element), 256) bytes (two input slots a,x,G and two output slots
 * h,grad_a,grad_x); fms_pipeline_workspace_bytes returns that figure.
 */
typedef struct fms_pipeline fms_pipeline;

size_t fms_pipeline_workspace_bytes(int64_t rows_per_block, int64_t T, int dtype);
int fms_pipeline_create(fms_pipeline **out, void *workspace, size_t workspace_bytes);
int fms_pipeline_destroy(fms_pipeline *pipe);

/*
 * Enqueue fwd+bwd of (rows, T) from host buffers to host buffers.  Asynchronous: work that was
 * enqueued on `stream` before the call is waited for, and on return `stream` waits for the
 * whole pipeline, so synchronising `stream` (or anything ordered after it) completes the call.
 * Host buffers should be page-locked; pageable memory works but the copies then serialise.
 * Calls on one pipeline must not overlap in time (they share the staging area).
 * Returns FMS_ERR_WORKSPACE if the workspace cannot hold a block of even one row.
 */
int fms_plain_forward_backward_host(fms_pipeline *pipe, const void *gates_h, const void *tokens_h,
                                    const void *grad_states_h, void *states_h, void *grad_gates_h,
                                    void *grad_tokens_h, int64_t rows, int64_t T, int dtype,
                                    fms_stream_t stream);

/*
 * The same pipeline with the kernels left out: the three inputs go host -> device into the
 * staging slots and the three output slots come back device -> host, block by block, with the
 * same streams, events and ordering.  The output buffers receive whatever the staging slots held;
 * the call exists to MEASURE the ceiling the copies alone put on the end-to-end rate of this box
 * (a benchmark reports it beside the full call).  Same arguments and rules as
 * fms_plain_forward_backward_host.  No reference counterpart.
 */
int fms_pipeline_copy_probe(fms_pipeline *pipe, const void *gates_h, const void *tokens_h,
                            const void *grad_states_h, void *states_h, void *grad_gates_h,
                            void *grad_tokens_h, int64_t rows, int64_t T, int dtype, fms_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FM_SCAN_B200_H_ */

/* C ABI of the B200 (sm_100a) LUCID forward-substitution library.
 *
 * These entry points are what a binding of the reference's operator layer
 * (lucid_kernels/cute/forward_sub_interface.py) calls instead of JIT-compiling and launching its
 * CuTe-DSL kernels.  Plain pointers and sizes only; every device pointer must belong to the current
 * CUDA device; all work is enqueued on `cuda_stream` (a cudaStream_t) and nothing synchronises
 * unless stated.
 *
 * Tensors are (B, N, H, 128) fp16 or bf16 with a contiguous last dimension ("BSHD"); `*_strides`
 * give the element strides of the first three dimensions {batch, sequence, head}.  Base addresses
 * must be 16-byte aligned and the strides multiples of 8 elements; a dimension of extent 1 may carry any
 * such stride, a longer one must not have stride 0 (expanded tensors are refused with LUCID_E_BAD_STRIDE:
 * the reference makes such inputs contiguous first, forward_sub_interface.py:26-27,81).  N must be a
 * multiple of 128.
 *
 * Return value: 0 on success, a negative LUCID_E_* code for a rejected argument, or a positive
 * cudaError_t from the runtime.  Device-side waits are bounded; a wait that runs out does not hang
 * the GPU but is recorded in the workspace and reported by lucid_read_status().
 */
#ifndef LUCID_B200_H_
#define LUCID_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LUCID_DTYPE_FP16 0
#define LUCID_DTYPE_BF16 1

/* flags */
#define LUCID_FLAG_DIAG_SOLVE 1   /* apply inv(tril(exp(K_i K_i^T))) on the diagonal blocks           */
#define LUCID_FLAG_NO_SYNC 2      /* skip inter-block flag waits (profiling only, results undefined)  */
#define LUCID_FLAG_INSTRUMENT 4   /* record per-row-block timestamps in the workspace                  */
#define LUCID_FLAG_REUSE_DIAG 8   /* the workspace still holds the diagonal-block inverses of THIS k from
                                     the previous call (same values, same shape): skip recomputing them.
                                     The reference recomputes them in every call
                                     (forward_sub_interface.py:116,230,311).                            */

/* backward modes */
#define LUCID_BWD_DV_ONLY 0       /* dV only                                                          */
#define LUCID_BWD_COMBINED 1      /* dV and the full dK (off-diagonal and diagonal terms)             */

#define LUCID_E_BAD_SHAPE (-1)
#define LUCID_E_BAD_DTYPE (-2)
#define LUCID_E_BAD_ALIGNMENT (-3)
#define LUCID_E_WORKSPACE_TOO_SMALL (-4)
#define LUCID_E_NULL_POINTER (-5)
#define LUCID_E_TENSOR_MAP (-6)
#define LUCID_E_NO_DEVICE (-7)
#define LUCID_E_STATIC_SCRATCH_TOO_SMALL (-8)
#define LUCID_E_BAD_STRIDE (-9)   /* zero stride in a dimension of extent > 1 (an expanded tensor) */

/* Size of the scratch array that lucid_fwd_sub_static() keeps inside the library (per GPU). */
#define LUCID_STATIC_SCRATCH_BYTES (9u << 20)

/* Bytes of scratch the calls below need for a (B, N, H, 128) problem.  The workspace holds the
 * inter-block flags, the scheduler's control words, the per-block unit-triangular inverses
 * (B*H*N*128 16-bit values) and their row scales, and 64 KiB of fp32 dK partial sums per 128 rows (the sums
 * the one-launch backward exchanges between work items, or the upper-triangle sums the reverse solve hands to
 * the dK kernel; a call given less than this, but at least lucid_fwd_workspace_bytes(), runs the variants that
 * do not need them).  Replaces the per-call torch.zeros / torch.empty
 * allocations of forward_sub_interface.py:97-103,217-219,297-300 and the diag_inv tensor of :109-117. */
size_t lucid_workspace_bytes(int B, int N, int H);

/* The part of that workspace a forward call (or a dV-only backward call) needs: everything except the dK
 * partial sums.  lucid_fwd_sub accepts a workspace of this size. */
size_t lucid_fwd_workspace_bytes(int B, int N, int H);

/* V' = L^-1 V.  Replaces _forward_sub_fwd (forward_sub_interface.py:56-165): _compute_diag_inv (:30-53)
 * and the ForwardSubSm90 launch (:153-158).  `window_blocks` < 0 means full causality (the reference's
 * window_size=None); otherwise only the last `window_blocks` blocks are subtracted, 0 meaning none at all,
 * i.e. only the diagonal-block solve (n_block_count = min(m_block, window_size), forward_sub_fwd.py:518-519).
 * `chain_group` = how many (batch, head) systems the scheduler advances together (0 = choose from the
 * problem size: as many as keep the K and V' they stream again and again at about the size of the L2 cache,
 * in groups of equal size). */
int lucid_fwd_sub(const void* k, const void* v, void* v_prime, const int64_t k_strides[3],
                  const int64_t v_strides[3], const int64_t vp_strides[3], int B, int N, int H, int D, int dtype,
                  int flags, int window_blocks, int chain_group, void* workspace, size_t workspace_bytes,
                  void* cuda_stream);

/* The forward solve for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference (whose interface allocates its flags, timestamps
 * and diagonal inverses with torch on every call).  It exists for hosts that drive the solve from a
 * context where cudaMalloc is off limits: a real-time or latency-critical serving loop that has frozen
 * its memory plan, a plugin called while another component owns the allocator, code running under a
 * memory-pool policy that forbids growth, or a process that has already handed all device memory to a
 * framework.  Such a caller still passes k, v and v_prime, but no workspace: the flags, control words,
 * per-block unit-triangular inverses and row scales go into an array that is part of the library's own
 * device image (LUCID_STATIC_SCRATCH_BYTES = 9 MiB, held by every GPU that loads the library until the
 * process exits).  The call path performs no cudaMalloc, cudaFree or allocating library call.
 *
 * Limits and rules:
 *  - the problem must fit the array: lucid_fwd_workspace_bytes(B, N, H) <= LUCID_STATIC_SCRATCH_BYTES - 1023
 *    (the array is re-aligned to 1 KiB), about 33 KiB per 128 rows, i.e. up to B*H*N = 36096 rows (for
 *    example B=1, H=2, N=16384, or B=2, H=4, N=4096); larger problems are refused with
 *    LUCID_E_STATIC_SCRATCH_TOO_SMALL and nothing is launched;
 *  - make the FIRST call on each device at start-up, as a warm-up, outside any stream capture: it looks up
 *    the array's device address (cudaGetSymbolAddress), and with CUDA's lazy module loading that is also
 *    the moment the driver loads this library's device code and reserves the 9 MiB array on that GPU - the
 *    one step on this path that takes device memory, and one that can fail on a GPU that is already full.
 *    Later calls take nothing;
 *  - all calls on a device share the one array, so two calls that can overlap on the GPU (different
 *    streams, or host threads) race with each other: serialise them;
 *  - the array keeps the previous call's contents; the call clears what must start at zero (flags and
 *    control words) itself and always recomputes the diagonal inverses; LUCID_FLAG_REUSE_DIAG and
 *    LUCID_FLAG_INSTRUMENT are ignored (the caller has no pointer to read timestamps back through);
 *  - status_out may be NULL (nothing synchronises); if it is not, the call synchronises cuda_stream and
 *    fills it exactly like lucid_read_status().
 * All other arguments are those of lucid_fwd_sub. */
int lucid_fwd_sub_static(const void* k, const void* v, void* v_prime, const int64_t k_strides[3],
                         const int64_t v_strides[3], const int64_t vp_strides[3], int B, int N, int H, int D,
                         int dtype, int flags, int window_blocks, int chain_group, void* cuda_stream,
                         int32_t status_out[8]);

/* dV = L^-T dV' and, in LUCID_BWD_COMBINED mode, dK.  Replaces _forward_sub_bwd
 * (forward_sub_interface.py:357-378): _compute_diag_inv_transpose (:177-193), the BackwardSubSm90
 * launches of _forward_sub_bwd_dv (:196-268) / _forward_sub_bwd_combined (:271-354) and the host-side
 * _add_diagonal_dk_correction (:381-405).  `dk` may be NULL in LUCID_BWD_DV_ONLY mode. */
int lucid_bwd_sub(const void* k, const void* v_prime, const void* dv_prime, void* dv, void* dk,
                  const int64_t k_strides[3], const int64_t vp_strides[3], const int64_t dvp_strides[3],
                  const int64_t dv_strides[3], const int64_t dk_strides[3], int B, int N, int H, int D, int dtype,
                  int flags, int mode, int chain_group, void* workspace, size_t workspace_bytes, void* cuda_stream);

/* Synchronises `cuda_stream` and copies the eight status words of the last call that used
 * `workspace`: out[0] = 0 ok / 1 in-CTA barrier wait timed out / 2 a predecessor row-block was never
 * published / 3 left early after another CTA's error; out[1] = kernel (0 prep, 1 solve, 2 dK);
 * out[2] = (batch*H + head); out[3] = row-block; out[4] = detail (awaited row-block); out[5] = barrier
 * id.  Returns 0 or a cudaError_t.  The reference has no counterpart: its waits spin forever
 * (forward_sub_fwd.py:536-544). */
int lucid_read_status(const void* workspace, void* cuda_stream, int32_t out[8]);

/* Diagnostic, no counterpart in the reference: measures how fast TMA delivers operand tiles from L2 into the
 * shared memory of every SM at once - the ceiling of the solve and dK kernels' operand streams (64 KiB per
 * tile of work each), whatever they compute.  One CTA per SM (at most clocks_len of them) streams
 * boxes_per_sm 16 KiB boxes (64 columns x 128 rows) of the (B, N, H, 128) 16-bit tensor - the loads the kernels
 * issue - through a ring of `slots` stages (1..12) and writes to clocks[cta] (device memory) the SM clocks that
 * took, or -1 if a wait ran out.  Bytes per clock per SM = boxes_per_sm * 16384 / clocks[cta].  Asynchronous
 * on cuda_stream; returns 0, a negative LUCID_E_* code or a cudaError_t. */
int lucid_probe_tma_delivery(const void* tensor, const int64_t strides[3], int B, int N, int H, int dtype, int slots,
                             int boxes_per_sm, long long* clocks, int clocks_len, void* cuda_stream);

/* Human-readable name of a status word out[0] or of a negative return code. */
const char* lucid_status_string(int code);

/* Sets the time limit (nanoseconds) of every device-side wait; default 2e9.  The kernels look at the clock
 * only every few hundred polls, so limits below some tens of microseconds take effect late; 0 means "do not
 * wait": any wait not satisfied at its first poll is reported as timed out (for testing the error path). */
void lucid_set_wait_limit_ns(uint64_t ns);

/* The same two operators for keys that the caller would otherwise scale first: the operator acts on
 * k_scale * K (LUCID's call site uses k * d^-1/4, bench_lucid_model.py:164-170), the kernels read K as it is
 * and fold k_scale^2 into the multiplier of every exponential; dK is the gradient with respect to the
 * unscaled K (k_scale^2 times the accumulated product).  Saves the elementwise pass over K and the rounding
 * of k_scale * K to 16 bits.  k_scale must be positive and finite; 1 gives lucid_fwd_sub / lucid_bwd_sub. */
int lucid_fwd_sub_scaled(const void* k, const void* v, void* v_prime, const int64_t k_strides[3],
                         const int64_t v_strides[3], const int64_t vp_strides[3], int B, int N, int H, int D,
                         int dtype, int flags, int window_blocks, int chain_group, float k_scale, void* workspace,
                         size_t workspace_bytes, void* cuda_stream);
int lucid_bwd_sub_scaled(const void* k, const void* v_prime, const void* dv_prime, void* dv, void* dk,
                         const int64_t k_strides[3], const int64_t vp_strides[3], const int64_t dvp_strides[3],
                         const int64_t dv_strides[3], const int64_t dk_strides[3], int B, int N, int H, int D,
                         int dtype, int flags, int mode, int chain_group, float k_scale, void* workspace,
                         size_t workspace_bytes, void* cuda_stream);

/* Scheduler knob: the first `steps` row-blocks of every (batch, head) system are scheduled for all systems
 * together (they are short and bound by the hand-over latency between consecutive row-blocks), the rest in
 * groups of `chain_group` systems; negative restores the default (0, i.e. groups from the start: the
 * head phase did not pay off in measurements and is kept as an experiment knob).  No counterpart in the reference,
 * whose grid is one CTA per row-block in launch order (tile_scheduler.py:105-117). */
void lucid_set_head_steps(int steps);

/* Scheduler knob: the first `steps` row-blocks of every group of systems but the first are dealt out
 * alternately with the last `steps` row-blocks of the group before, so that the short, latency-bound start of a
 * group runs beside long row-blocks that keep the other SMs busy (< 0 = default).  No counterpart in the
 * reference, whose grid is one CTA per row-block. */
void lucid_set_group_overlap(int steps);

/* One-launch backward (see lucid_set_fused_backward) with one or two systems: a row-block's dK tiles are dealt
 * out as two work items whose fp32 sums meet through the workspace, so that the launch ends in units of half a
 * row-block (on = 1, default) instead of a whole one (on = 0).  No counterpart in the reference. */
void lucid_set_dk_split(int on);

/* Combined backward (mode LUCID_BWD_COMBINED): with at most `max_chains` (batch, head) systems the reverse
 * solve, then bound by its chain latency, and the dK program run in ONE launch - `solve_ctas` CTAs solve,
 * the others compute dK row-blocks as the solve publishes them and are joined by the solving CTAs at the
 * end (0 = automatic share, 47 %).  Default max_chains = 2; 0 disables the fusion.  The reference's BackwardSubSm90 likewise runs its two phases in one
 * launch (forward_sub_bwd.py:1053-1269). */
void lucid_set_fused_backward(int max_chains, int solve_ctas);

/* Solves with at most `max_chains` (batch, head) systems (and an even number of 128-row blocks, the diagonal
 * solve, no window) run as clusters of two CTAs that solve pairs of consecutive row-blocks and hand the first
 * result to the second through shared memory; 0 disables it.  Default 8.  No counterpart in the reference,
 * which publishes every row-block through global memory (forward_sub_fwd.py:536-544). */
void lucid_set_pair_solve(int max_chains);

/* The same switch with its second limit: pairs are used with at most `max_chains` systems and at most
 * `max_row_blocks` 128-row blocks over all systems (B*H*N/128; default 768; <= 0 restores the default). */
void lucid_set_pair_limits(int max_chains, int max_row_blocks);

/* Combined backward with more systems than the one-launch limit: the reverse solve also accumulates the
 * upper-triangle dK terms of the tiles it streams, as Phase 1 of the reference's BackwardSubSm90 does
 * (forward_sub_bwd.py:1113-1195), and the dK kernel runs the rest (on = 1, default); 0 = the reverse solve and
 * a dK kernel over all tiles.  Needs the full workspace of lucid_workspace_bytes(). */
void lucid_set_upper_in_solve(int on);

/* 1 if a combined backward (diagonal solve, full workspace) of this problem would run that way under the current
 * settings on the current device, else 0 (benchmarks use it to label what they measured). */
int lucid_query_upper_in_solve(int B, int N, int H);

/* How many (batch, head) systems the scheduler advances together when `chain_group` is 0: for the forward
 * solve (and the dV-only backward), or with combined_backward != 0 for the combined backward.  Plain host
 * arithmetic (no device needed); 0 for an invalid shape. */
int lucid_query_chain_group(int B, int N, int H, int combined_backward);

/* Kernel variant of the stand-alone solves: bit 0 = the S products read K_i from tensor memory instead of
 * shared memory (two S buffers instead of three).  No counterpart in the reference. */
void lucid_set_solve_variant(int bits);

/* 1 if lucid_fwd_sub with the diagonal solve and full causality would run this problem in that pair mode
 * under the current limits, else 0 (benchmarks use it to label what they measured). */
int lucid_query_pair_solve(int B, int N, int H);

/* The id of the capture `cuda_stream` is recording into (cudaStreamGetCaptureInfo), 0 when it is not
 * capturing.  Host layers that remember what a workspace holds between calls use it to keep work recorded
 * into a CUDA graph (which runs later, at replay) apart from work that ran at once.  No counterpart in the
 * reference. */
unsigned long long lucid_stream_capture_id(void* cuda_stream);

/* Per-kernel timing for benchmarks: the NEXT lucid_fwd_sub / lucid_bwd_sub call made BY THE CALLING THREAD records these
 * cudaEvent_t handles on its stream (before the diagonal-prep kernel, after it, after the solve kernel,
 * after the dK kernel); any of them may be NULL.  The handles are forgotten after that call.  Stands in
 * for the reference's `instrument=True` compile flag (forward_sub_interface.py:62) at kernel granularity. */
void lucid_profile_next_call(void* ev_begin, void* ev_after_prep, void* ev_after_solve, void* ev_after_dk);

/* Offsets inside the workspace, for tools that read the instrumentation:
 * timestamps are int64[(B*H)][T][8] = {start, loop end, published, ns spent in flag waits, CTA, tiles, SM cycles start..published}
 * (cf. the (T, 8) buffer of forward_sub_interface.py:103). */
size_t lucid_workspace_timestamps_offset(int B, int N, int H);

#ifdef __cplusplus
}
#endif
#endif /* LUCID_B200_H_ */

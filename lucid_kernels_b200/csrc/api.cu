// C ABI: argument checking, workspace carving, tensor maps and kernel launches.
#include <stdio.h>
#include <string.h>

#include "../../include/lucid_b200.h"
#include "kernels.h"
#include "tmap.h"

namespace lucid {

static unsigned long long g_wait_ns = 2000000000ull;
// optional per-kernel timing: events recorded around the kernels of the NEXT call made by the same host
// thread, then forgotten (thread-local, so one thread's request is never consumed by another thread's call)
static thread_local cudaEvent_t g_events[4] = {nullptr, nullptr, nullptr, nullptr};
static long long* g_trace = nullptr;
static int g_fuse_max_chains = 2;   // combined backward: fuse solve and dK into one launch up to this many chains
static int g_fuse_solve_ctas = 0;   // 0 = automatic share
static int g_pair_max_chains = 8;   // solve pairs of row-blocks with clusters of two CTAs up to this many chains
static int g_pair_max_blocks = 768; // ... and up to this many row-blocks in all (chains * T)
static int g_solve_variant = 0;     // bit 0: the stand-alone solves read K_i from tensor memory
static int g_upper_in_solve = 1;    // combined backward: the reverse solve also accumulates the upper-triangle dK
static int g_head = -1;   // scheduler knob; < 0 = default
static int g_overlap = -1;   // scheduler knob; < 0 = default
static int g_dk_split = 1;   // one-launch backward: dK row-blocks as two work items
static inline void record_event(int i, cudaStream_t stream) {
  if (g_events[i]) cudaEventRecord(g_events[i], stream);
}

// ---- workspace layout ----------------------------------------------------------------------
//   [0, 256)            three Control blocks: 0 = diag prep, 1 = solve, 2 = dK; word 24 = arrival counter of the
//                       one-launch backward (which CTAs take the solve role)
//   [256, 256 + 4*C*T)  flags
//   X                   C*T tiles of 32 KiB (1 KiB aligned)
//   lam_inv             C*T*128 fp32
//   timestamps          C*T*8 int64
//   partial             C*T*128*128 fp32 (combined backward only; a call given a workspace without it runs the
//                       variants that do not need it)
struct Layout {
  size_t flags, dksync, x, lam, ts, partial, need, total;   // need: without the dK partial sums
};
// dK work items split in two are used with at most this many chains (the fp32 sums of the half that finishes
// first go through the workspace: 64 KiB per row-block)
constexpr int kSplitMaxChains = 2;
static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static Layout make_layout(int B, int N, int H) {
  const size_t CT = (size_t)B * H * (N / kBlock);
  Layout l;
  l.flags = 256;
  l.dksync = l.flags + CT * 4;                         // claim counters and completion flags, zeroed with the flags
  l.x = align_up(l.dksync + CT * 8, 1024);
  l.lam = l.x + CT * kTileBytes;
  l.ts = align_up(l.lam + CT * kBlock * 4, 256);
  l.need = l.ts + CT * 8 * 8;
  // One fp32 128 x 128 tile per row-block: with one or two chains the partial sums of dK work items split in two
  // (one-launch backward), with more chains the upper-triangle dK sums that the reverse solve accumulates for
  // the dK kernel.  Never both.
  l.partial = align_up(l.need, 1024);
  l.total = l.partial + CT * (size_t)kBlock * kBlock * 4;
  return l;
}

static int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

// st = element strides {batch, sequence, head}; ext = the extents of those dimensions.  A zero stride in a
// dimension of extent > 1 is an expanded (broadcast) tensor: the tensor maps cannot express it, and writing
// through one would alias.
static int check_tensor(const void* p, const int64_t st[3], int B, int N, int H) {
  if (!p || !st) return LUCID_E_NULL_POINTER;
  if (reinterpret_cast<uintptr_t>(p) % 16) return LUCID_E_BAD_ALIGNMENT;
  const int ext[3] = {B, N, H};
  for (int i = 0; i < 3; ++i) {
    if (st[i] % 8 || st[i] < 0) return LUCID_E_BAD_ALIGNMENT;
    if (st[i] == 0 && ext[i] > 1) return LUCID_E_BAD_STRIDE;
  }
  return 0;
}

static int check_shape(int B, int N, int H, int D, int dtype) {
  if (B <= 0 || N <= 0 || H <= 0 || D != kBlock || N % kBlock) return LUCID_E_BAD_SHAPE;
  if ((long long)B * H * (N / kBlock) > (1ll << 30) / kBlock) return LUCID_E_BAD_SHAPE;
  if (dtype != LUCID_DTYPE_FP16 && dtype != LUCID_DTYPE_BF16) return LUCID_E_BAD_DTYPE;
  return 0;
}

// (B, N, H, 128) tensor -> 4-D map {d, n, h, b}
static int bshd_map(CUtensorMap* m, bool bf16, const void* p, const int64_t st[3], int B, int N, int H,
                    uint32_t box_rows) {
  uint64_t dims[4] = {(uint64_t)kBlock, (uint64_t)N, (uint64_t)H, (uint64_t)B};
  // size-1 dimensions may carry any stride; give them a harmless valid one.  (Zero strides of longer
  // dimensions never get here: check_tensor refuses them.)
  uint64_t sn = (uint64_t)st[1] * 2, sh = (uint64_t)st[2] * 2, sb = (uint64_t)st[0] * 2;
  if (H == 1) sh = 256;
  if (B == 1) sb = 256;
  if (sn == 0 || sh == 0 || sb == 0) return LUCID_E_BAD_STRIDE;
  uint64_t strides[3] = {sn, sh, sb};
  return make_tmap_16bit(m, bf16, p, 4, dims, strides, box_rows) ? LUCID_E_TENSOR_MAP : 0;
}

static int auto_group(int C, int N, int requested, bool backward) {
  if (requested > 0) return requested < C ? requested : C;
  // K and Y of one chain take N * 512 bytes, and every row-block of a group streams them again and again: TMA
  // delivers such tiles at 65 bytes per clock per SM while the streamed set is below about 64 MB, at 47-53 beyond
  // that; but a group must also hold enough chains to keep all SMs busy, and every group pays the chain latency of
  // its first row-blocks.  Measured on B200, forward + backward of the present kernels in ms, by group size:
  //   B*H=16, N=32768:   4: 4.4 + 13.2   6: 4.8 + 12.6   8: 4.7 + 13.3   16: 5.1 + 14.2   (benchmark step, one graph:
  //                      17.5 / 16.9 / 17.0 ms with 4 / 6 / 8 for both)
  //   B*H=8,  N=65536:   2: 9.8 + 25.8   3: 10.4 + 25.9   4: 9.0 + 24.8   8: 10.1 + 26.0
  //   B*H=8,  N=131072:  1: 39.4 + 107.4   2: 39.2 + 98.2   3: 41.9 + 97.3   4: 43.5 + 96.5
  //   B*H=4,  N=65536:   1: 7.0 + 16.2   2: 5.4 + 13.0   4: 4.4 + 12.5
  //   B*H=16, N=16384:   4: 1.8 + 4.2   8: 1.3 + 3.3   16: 1.3 + 3.4
  // The forward does best with K and Y of a group at about the size of the L2 (128 MiB); the backward, which streams
  // three tensors per tile in its dK part, with 104 MiB but never fewer than four chains.  The groups are made
  // equal in size.
  const long long per_chain = (long long)N * 512;
  const long long budget = backward ? (104ll << 20) : (128ll << 20);
  long long gmax = budget / per_chain;
  const long long floor_chains = backward ? 4 : 1;
  if (gmax < floor_chains) gmax = floor_chains;
  if (gmax >= C) return C;
  const long long ng = (C + gmax - 1) / gmax;
  return (int)((C + ng - 1) / ng);
}

static Problem make_problem(int B, int N, int H, int flags, int window, int group, float k_scale,
                            bool backward = false) {
  Problem p;
  p.exp_scale = kLog2e * k_scale * k_scale;
  p.out_scale = k_scale * k_scale;
  p.B = B;
  p.N = N;
  p.H = H;
  p.T = N / kBlock;
  p.C = B * H;
  p.group = auto_group(p.C, N, group, backward);
  // Optionally the short, latency-bound first row-blocks of every chain are scheduled for all chains
  // together before the groups start.  Off by default: on B=2, N=32768, H=8 a sweep over 0 / 48 / 96 / 144 /
  // 192 / 256 steps gave 4.7-5.9 / 5.0-5.2 / 5.1-5.2 / 5.2-5.4 / 5.5 / 6.1 ms for the forward, i.e. no gain
  // beyond run-to-run noise and a loss once the head is long.
  p.head = g_head >= 0 ? g_head : 0;
  if (p.head > p.T) p.head = p.T;
  // Likewise off by default: dealing the first steps of a group out alternately with the last steps of the
  // group before halves the time the CTAs spend waiting for flags (B=2, N=32768, H=8, 96 steps: 0.51 -> 0.26 ms
  // per CTA; B=1, N=131072, H=8, 512 steps: 3.9 -> 1.9 ms), but on the power-capped part the time per tile rises
  // by as much and the step time stays where it was (20.8 against 20.6 ms in an alternating comparison).
  p.overlap = g_overlap >= 0 ? g_overlap : 0;
  if (p.overlap > (p.T - p.head) / 2) p.overlap = (p.T - p.head) / 2;
  p.use_diag = (flags & LUCID_FLAG_DIAG_SOLVE) ? 1 : 0;
  p.window = window;
  p.no_sync = (flags & LUCID_FLAG_NO_SYNC) ? 1 : 0;
  p.instrument = (flags & LUCID_FLAG_INSTRUMENT) ? 1 : 0;
  p.reuse_diag = (flags & LUCID_FLAG_REUSE_DIAG) ? 1 : 0;
  p.wait_ns = g_wait_ns;
  return p;
}

// Whether a stand-alone solve of this problem runs as clusters of two CTAs over pairs of row-blocks.
static bool pair_eligible(const Problem& p) {
  return p.C <= g_pair_max_chains && p.C * p.T <= g_pair_max_blocks && p.use_diag && p.window < 0 && !p.no_sync &&
         (p.T % 2) == 0 && p.head == 0 && p.overlap == 0;
}

// What the combined backward hands to run_solve when the dK program is to run in the solve's launch.
struct FusedDk {
  CUtensorMap tm_vp, tm_dv;
  DkArgs args;
  int n_solve;
};

// What the combined backward hands to run_solve when the reverse solve is to accumulate the upper-triangle dK.
struct UpperPlan {
  CUtensorMap tm_vp;
  float* upper;
};

// shared by forward and backward: prep (if diag) + one solve (+ the dK program in the same launch)
static int run_solve(bool reverse, const void* k, const void* in, void* out, const int64_t ks[3],
                     const int64_t ins[3], const int64_t outs[3], const Problem& p, bool bf16, uint8_t* ws,
                     const Layout& lay, cudaStream_t stream, FusedDk* fused = nullptr, UpperPlan* upper = nullptr) {
  const int CT = p.C * p.T;
  Control* ctl = reinterpret_cast<Control*>(ws);
  CUtensorMap tm_k, tm_in, tm_out, tm_x, tm_st;
  int rc;
  if ((rc = bshd_map(&tm_k, bf16, k, ks, p.B, p.N, p.H, 128))) return rc;
  if ((rc = bshd_map(&tm_in, bf16, in, ins, p.B, p.N, p.H, 128))) return rc;
  if ((rc = bshd_map(&tm_out, bf16, out, outs, p.B, p.N, p.H, 64))) return rc;
  if ((rc = bshd_map(&tm_st, bf16, out, outs, p.B, p.N, p.H, 128))) return rc;
  {
    uint64_t dims[2] = {(uint64_t)kBlock, (uint64_t)CT * kBlock};
    uint64_t str[1] = {256};
    if (make_tmap_16bit(&tm_x, bf16, ws + lay.x, 2, dims, str, 128)) return LUCID_E_TENSOR_MAP;
  }
  cudaError_t e;
  record_event(0, stream);
  if (p.use_diag && !p.reuse_diag) {
    PrepArgs pa;
    pa.x = ws + lay.x;
    pa.lam_inv = reinterpret_cast<float*>(ws + lay.lam);
    pa.ctl = ctl + 0;
    pa.T = p.T;
    pa.H = p.H;
    pa.exp_scale = p.exp_scale;
    pa.wait_ns = p.wait_ns;
    if ((e = launch_diag_prep(bf16, tm_k, pa, CT, stream)) != cudaSuccess) return (int)e;
  }
  record_event(1, stream);
  SolveArgs sa;
  sa.out = out;
  sa.out_strides = Strides{outs[0], outs[1], outs[2]};
  sa.lam_inv = reinterpret_cast<const float*>(ws + lay.lam);
  sa.flags = reinterpret_cast<int*>(ws + lay.flags);
  sa.ctl = ctl + 1;
  sa.timestamps = p.instrument ? reinterpret_cast<long long*>(ws + lay.ts) : nullptr;
  sa.trace = g_trace;
  sa.p = p;
  const int sms = sm_count();
  if (sms <= 0) return LUCID_E_NO_DEVICE;
  const int grid = CT < sms ? CT : sms;
  if (upper) {
    RevDkArgs ra;
    ra.out = out;
    ra.lam_inv = sa.lam_inv;
    ra.flags = sa.flags;
    ra.ctl = sa.ctl;
    ra.upper = upper->upper;
    ra.trace = g_trace;
    ra.p = p;
    e = launch_revdk(bf16, tm_k, tm_in, tm_st, upper->tm_vp, tm_x, ra, grid, stream);
  } else if (fused) {
    fused->args.follow_flags = sa.flags;
    fused->args.follow_ctl = sa.ctl;
    e = launch_bwd_fused(bf16, tm_k, tm_in, tm_out, tm_x, tm_st, fused->tm_vp, fused->tm_dv, sa, fused->args,
                         fused->n_solve, reinterpret_cast<int*>(ws) + 24, sms, stream);
  } else {
    // Few chains: the hand-over latency between consecutive row-blocks limits the solve; pairs of row-blocks
    // are then solved by clusters of two CTAs, the first handing its result to the second through shared memory.
    // Worth it only while the chain latency, not the tile throughput, bounds the solve: about C * T <= 768
    // on B200 (forward, ms, pairs against single row-blocks: 8 chains of N=8192 0.255 / 0.270, 1 and 2 chains of
    // N=32768 0.82 / 0.93 and 0.95 / 1.00, but 4 chains of N=65536 5.5 / 4.9 - the pairs are taken in a fixed
    // rotation, which balances the tile work less well than the ticket counter).
    const bool pair = pair_eligible(p);
    int pgrid = grid;
    if (pair) {
      const int items = CT / 2;
      pgrid = 2 * (items < sms / 2 ? items : sms / 2);
    }
    const bool kt = (g_solve_variant & 1) != 0;
    e = launch_solve(bf16, reverse, pair, kt, tm_k, tm_in, tm_out, tm_x, tm_st, sa, pair ? pgrid : grid, stream);
    if (pair && e != cudaSuccess) {
      // no room for clusters on this device (a partitioned GPU, for instance): single row-blocks always launch
      (void)cudaGetLastError();
      e = launch_solve(bf16, reverse, false, kt, tm_k, tm_in, tm_out, tm_x, tm_st, sa, grid, stream);
    }
  }
  if (e != cudaSuccess) return (int)e;
  record_event(2, stream);
  return 0;
}

}  // namespace lucid

using namespace lucid;

extern "C" {

size_t lucid_workspace_bytes(int B, int N, int H) {
  if (B <= 0 || N <= 0 || H <= 0 || N % kBlock) return 0;
  return make_layout(B, N, H).total;
}

size_t lucid_fwd_workspace_bytes(int B, int N, int H) {
  if (B <= 0 || N <= 0 || H <= 0 || N % kBlock) return 0;
  return make_layout(B, N, H).need;
}

unsigned long long lucid_stream_capture_id(void* cuda_stream) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  unsigned long long id = 0;
  if (cudaStreamGetCaptureInfo(static_cast<cudaStream_t>(cuda_stream), &st, &id) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return st == cudaStreamCaptureStatusActive ? id : 0;
}

size_t lucid_workspace_timestamps_offset(int B, int N, int H) {
  if (B <= 0 || N <= 0 || H <= 0 || N % kBlock) return 0;
  return make_layout(B, N, H).ts;
}

void lucid_set_wait_limit_ns(uint64_t ns) { g_wait_ns = ns; }

void lucid_set_head_steps(int steps) { g_head = steps; }

void lucid_set_group_overlap(int steps) { g_overlap = steps; }

void lucid_set_dk_split(int on) { g_dk_split = on; }

int lucid_query_pair_solve(int B, int N, int H) {
  if (B <= 0 || N <= 0 || H <= 0 || N % kBlock) return 0;
  return pair_eligible(make_problem(B, N, H, LUCID_FLAG_DIAG_SOLVE, -1, 0, 1.0f)) ? 1 : 0;
}

void lucid_set_solve_variant(int bits) { g_solve_variant = bits; }

void lucid_set_upper_in_solve(int on) { g_upper_in_solve = on; }

int lucid_query_upper_in_solve(int B, int N, int H) {
  if (B <= 0 || N <= 0 || H <= 0 || N % kBlock) return 0;
  const int C = B * H, CT = C * (N / kBlock), sms = sm_count();
  const bool fuse = C <= g_fuse_max_chains && sms > 0 && CT >= 2 * sms;
  return (!fuse && g_upper_in_solve) ? 1 : 0;
}

int lucid_query_chain_group(int B, int N, int H, int combined_backward) {
  if (B <= 0 || N <= 0 || H <= 0 || N % kBlock) return 0;
  return auto_group(B * H, N, 0, combined_backward != 0);
}

void lucid_set_pair_solve(int max_chains) { g_pair_max_chains = max_chains; }

void lucid_set_pair_limits(int max_chains, int max_row_blocks) {
  g_pair_max_chains = max_chains;
  g_pair_max_blocks = max_row_blocks > 0 ? max_row_blocks : 768;
}

void lucid_set_fused_backward(int max_chains, int solve_ctas) {
  g_fuse_max_chains = max_chains;
  g_fuse_solve_ctas = solve_ctas;
}

#ifdef LUCID_TRACE
void lucid_debug_set_trace(void* buf) { g_trace = static_cast<long long*>(buf); }
#endif

void lucid_profile_next_call(void* ev_begin, void* ev_after_prep, void* ev_after_solve, void* ev_after_dk) {
  g_events[0] = static_cast<cudaEvent_t>(ev_begin);
  g_events[1] = static_cast<cudaEvent_t>(ev_after_prep);
  g_events[2] = static_cast<cudaEvent_t>(ev_after_solve);
  g_events[3] = static_cast<cudaEvent_t>(ev_after_dk);
}

int lucid_fwd_sub(const void* k, const void* v, void* v_prime, const int64_t k_strides[3],
                  const int64_t v_strides[3], const int64_t vp_strides[3], int B, int N, int H, int D, int dtype,
                  int flags, int window_blocks, int chain_group, void* workspace, size_t workspace_bytes,
                  void* cuda_stream) {
  return lucid_fwd_sub_scaled(k, v, v_prime, k_strides, v_strides, vp_strides, B, N, H, D, dtype, flags,
                              window_blocks, chain_group, 1.0f, workspace, workspace_bytes, cuda_stream);
}

int lucid_fwd_sub_scaled(const void* k, const void* v, void* v_prime, const int64_t k_strides[3],
                         const int64_t v_strides[3], const int64_t vp_strides[3], int B, int N, int H, int D,
                         int dtype, int flags, int window_blocks, int chain_group, float k_scale, void* workspace,
                         size_t workspace_bytes, void* cuda_stream) {
  int rc;
  if (!(k_scale > 0.0f) || !(k_scale < 1e18f)) return LUCID_E_BAD_SHAPE;
  if ((rc = check_shape(B, N, H, D, dtype))) return rc;
  if ((rc = check_tensor(k, k_strides, B, N, H)) || (rc = check_tensor(v, v_strides, B, N, H)) ||
      (rc = check_tensor(v_prime, vp_strides, B, N, H)))
    return rc;
  if (!workspace) return LUCID_E_NULL_POINTER;
  if (reinterpret_cast<uintptr_t>(workspace) % 1024) return LUCID_E_BAD_ALIGNMENT;
  const Layout lay = make_layout(B, N, H);
  if (workspace_bytes < lay.need) return LUCID_E_WORKSPACE_TOO_SMALL;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  cudaError_t e = cudaMemsetAsync(ws, 0, lay.x, stream);   // control words + flags
  if (e != cudaSuccess) return (int)e;
  const Problem p = make_problem(B, N, H, flags, window_blocks, chain_group, k_scale);
  rc = run_solve(false, k, v, v_prime, k_strides, v_strides, vp_strides, p, dtype == LUCID_DTYPE_BF16, ws, lay,
                 stream);
  memset(g_events, 0, sizeof(g_events));
  return rc;
}

// ---- forward solve on library-owned scratch (no allocation anywhere on the call path) ----------------
// The scratch lives in the library's device image: every GPU that loads the library carries these 9 MiB
// until the process exits.  Host code may not use the array's name as a pointer; its device address is
// fetched once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[LUCID_STATIC_SCRATCH_BYTES];
static unsigned char* g_static_scratch_ptr[64] = {nullptr};

int lucid_fwd_sub_static(const void* k, const void* v, void* v_prime, const int64_t k_strides[3],
                         const int64_t v_strides[3], const int64_t vp_strides[3], int B, int N, int H, int D,
                         int dtype, int flags, int window_blocks, int chain_group, void* cuda_stream,
                         int32_t status_out[8]) {
  int rc;
  if ((rc = check_shape(B, N, H, D, dtype))) return rc;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return LUCID_E_NO_DEVICE;
  if (!g_static_scratch_ptr[dev]) {
    // first call on this device: resolve the device address of the array (do this before any capture)
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    g_static_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  // the kernels want a 1 KiB aligned base; the array is only guaranteed 256-byte alignment
  uintptr_t base = reinterpret_cast<uintptr_t>(g_static_scratch_ptr[dev]);
  const uintptr_t aligned = (base + 1023) & ~uintptr_t(1023);
  const size_t usable = LUCID_STATIC_SCRATCH_BYTES - (aligned - base);
  const size_t need = make_layout(B, N, H).need;
  if (need > usable) return LUCID_E_STATIC_SCRATCH_TOO_SMALL;
  // the array still holds whatever the previous call left: never trust a cached inverse in it; and the caller
  // has no pointer through which it could read instrumentation back
  flags &= ~(LUCID_FLAG_REUSE_DIAG | LUCID_FLAG_INSTRUMENT);
  rc = lucid_fwd_sub(k, v, v_prime, k_strides, v_strides, vp_strides, B, N, H, D, dtype, flags, window_blocks,
                     chain_group, reinterpret_cast<void*>(aligned), usable, cuda_stream);
  if (rc) return rc;
  if (status_out) return lucid_read_status(reinterpret_cast<void*>(aligned), cuda_stream, status_out);
  return 0;
}

int lucid_bwd_sub(const void* k, const void* v_prime, const void* dv_prime, void* dv, void* dk,
                  const int64_t k_strides[3], const int64_t vp_strides[3], const int64_t dvp_strides[3],
                  const int64_t dv_strides[3], const int64_t dk_strides[3], int B, int N, int H, int D, int dtype,
                  int flags, int mode, int chain_group, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  return lucid_bwd_sub_scaled(k, v_prime, dv_prime, dv, dk, k_strides, vp_strides, dvp_strides, dv_strides,
                              dk_strides, B, N, H, D, dtype, flags, mode, chain_group, 1.0f, workspace,
                              workspace_bytes, cuda_stream);
}

int lucid_bwd_sub_scaled(const void* k, const void* v_prime, const void* dv_prime, void* dv, void* dk,
                         const int64_t k_strides[3], const int64_t vp_strides[3], const int64_t dvp_strides[3],
                         const int64_t dv_strides[3], const int64_t dk_strides[3], int B, int N, int H, int D,
                         int dtype, int flags, int mode, int chain_group, float k_scale, void* workspace,
                         size_t workspace_bytes, void* cuda_stream) {
  int rc;
  if (!(k_scale > 0.0f) || !(k_scale < 1e18f)) return LUCID_E_BAD_SHAPE;
  if ((rc = check_shape(B, N, H, D, dtype))) return rc;
  if (mode != LUCID_BWD_DV_ONLY && mode != LUCID_BWD_COMBINED) return LUCID_E_BAD_SHAPE;
  if ((rc = check_tensor(k, k_strides, B, N, H)) || (rc = check_tensor(dv_prime, dvp_strides, B, N, H)) ||
      (rc = check_tensor(dv, dv_strides, B, N, H)))
    return rc;
  if (mode == LUCID_BWD_COMBINED) {
    if ((rc = check_tensor(v_prime, vp_strides, B, N, H)) || (rc = check_tensor(dk, dk_strides, B, N, H))) return rc;
  }
  if (!workspace) return LUCID_E_NULL_POINTER;
  if (reinterpret_cast<uintptr_t>(workspace) % 1024) return LUCID_E_BAD_ALIGNMENT;
  const Layout lay = make_layout(B, N, H);
  if (workspace_bytes < lay.need) return LUCID_E_WORKSPACE_TOO_SMALL;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  cudaError_t e = cudaMemsetAsync(ws, 0, lay.x, stream);
  if (e != cudaSuccess) return (int)e;
  const bool bf16 = dtype == LUCID_DTYPE_BF16;
  const Problem p = make_problem(B, N, H, flags, -1, chain_group, k_scale, mode == LUCID_BWD_COMBINED);
  const int sms = sm_count();
  if (sms <= 0) return LUCID_E_NO_DEVICE;
  const int CT = p.C * p.T;
  FusedDk fd;
  CUtensorMap tm_k;
  if (mode == LUCID_BWD_COMBINED) {
    if ((rc = bshd_map(&tm_k, bf16, k, k_strides, B, N, H, 128))) return rc;
    if ((rc = bshd_map(&fd.tm_vp, bf16, v_prime, vp_strides, B, N, H, 128))) return rc;
    if ((rc = bshd_map(&fd.tm_dv, bf16, dv, dv_strides, B, N, H, 128))) return rc;
    fd.args.dk = dk;
    fd.args.dk_strides = Strides{dk_strides[0], dk_strides[1], dk_strides[2]};
    fd.args.ctl = reinterpret_cast<Control*>(ws) + 2;
    fd.args.follow_flags = nullptr;
    fd.args.follow_ctl = nullptr;
    fd.args.trace = g_trace;
    fd.args.split = 0;
    fd.args.partial = reinterpret_cast<float*>(ws + lay.partial);
    fd.args.sync = reinterpret_cast<int*>(ws + lay.dksync);
    fd.args.lower_only = 0;
    fd.args.upper = nullptr;
    fd.args.p = p;
  }
  // With one or two chains the reverse solve is bound by its chain latency and leaves SMs idle: the dK
  // program then runs in the same launch on the other CTAs, and the solve's CTAs join it when the solve's
  // row-blocks have all been taken.  Measured on B200 (backward, ms, separate launches against one launch
  // with 45 / 56 / 64 / 72 / 90 solve CTAs): 2 chains of N=32768: 2.14 against 2.24 / 1.98 / 1.88 / 1.87 /
  // 1.95; 1 chain: 1.75 against 1.60 / 1.50 / 1.50 / 1.49 / 1.49; 4 chains: 3.62 against 4.27 / 3.80 / 3.73 /
  // 3.78 / 3.78 (no gain, hence the limit of 2).  Needs at least two row-blocks per SM.
  int n_solve = g_fuse_solve_ctas > 0 ? g_fuse_solve_ctas : (sms * 47 + 50) / 100;
  if (n_solve >= sms) n_solve = sms - 1;
  const bool fuse = mode == LUCID_BWD_COMBINED && p.C <= g_fuse_max_chains && !p.instrument && !p.no_sync &&
                    CT >= 2 * sms && n_solve >= 1;
  fd.n_solve = n_solve;
  // In that launch a row-block of dK (0.31 ms at N=32768) is the unit in which the launch ends; two half items
  // per row-block halve it.
  if (fuse && g_dk_split && p.C <= kSplitMaxChains && workspace_bytes >= lay.total) fd.args.split = 1;
  // More chains than that: the reverse solve streams K_j and dV_j and forms exp(S) for every later block anyway,
  // so it also accumulates the upper-triangle dK terms of those tiles (two more products per tile) and the dK
  // kernel that follows runs only the lower part, the diagonal tiles and the first upper tile of every row-block.
  UpperPlan up;
  const bool upper_in_solve = mode == LUCID_BWD_COMBINED && !fuse && g_upper_in_solve && p.use_diag && !p.instrument &&
                              !p.no_sync && workspace_bytes >= lay.total;
  if (upper_in_solve) {
    up.tm_vp = fd.tm_vp;
    up.upper = reinterpret_cast<float*>(ws + lay.partial);
    fd.args.lower_only = 1;
    fd.args.upper = up.upper;
  }
  rc = run_solve(true, k, dv_prime, dv, k_strides, dvp_strides, dv_strides, p, bf16, ws, lay, stream,
                 fuse ? &fd : nullptr, upper_in_solve ? &up : nullptr);
  cudaEvent_t ev_dk = g_events[3];
  memset(g_events, 0, sizeof(g_events));
  if (rc) return rc;
  if (mode == LUCID_BWD_COMBINED) {
    if (!fuse) {
      const int grid = CT < sms ? CT : sms;
      if ((e = launch_dk(bf16, tm_k, fd.tm_vp, fd.tm_dv, fd.args, grid, stream)) != cudaSuccess) return (int)e;
    }
    if (ev_dk) cudaEventRecord(ev_dk, stream);
  }
  return 0;
}

int lucid_probe_tma_delivery(const void* tensor, const int64_t strides[3], int B, int N, int H, int dtype, int slots,
                             int boxes_per_sm, long long* clocks, int clocks_len, void* cuda_stream) {
  int rc = check_shape(B, N, H, kBlock, dtype);
  if (rc) return rc;
  if ((rc = check_tensor(tensor, strides, B, N, H))) return rc;
  if (!clocks) return LUCID_E_NULL_POINTER;
  if (slots < 1 || slots > 12 || boxes_per_sm < 1 || clocks_len < 1) return LUCID_E_BAD_SHAPE;
  const int sms = sm_count();
  if (sms <= 0) return LUCID_E_NO_DEVICE;
  CUtensorMap tm;
  if ((rc = bshd_map(&tm, dtype == LUCID_DTYPE_BF16, tensor, strides, B, N, H, 128))) return rc;
  const int grid = sms < clocks_len ? sms : clocks_len;
  cudaError_t e = launch_delivery_probe(tm, slots, boxes_per_sm, B * H, N / kBlock, H, clocks, grid,
                                        static_cast<cudaStream_t>(cuda_stream));
  return e == cudaSuccess ? 0 : (int)e;
}

int lucid_read_status(const void* workspace, void* cuda_stream, int32_t out[8]) {
  if (!workspace || !out) return LUCID_E_NULL_POINTER;
  int32_t host[24];
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e = cudaMemcpyAsync(host, workspace, sizeof(host), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return (int)e;
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return (int)e;
  memset(out, 0, 8 * sizeof(int32_t));
  for (int kern = 0; kern < 3; ++kern) {
    const int32_t* c = host + kern * 8;   // {ticket, status[7]}
    if (c[1] != 0) {
      out[0] = c[1];
      out[1] = kern;
      out[2] = c[2];
      out[3] = c[3];
      out[4] = c[4];
      out[5] = c[5];
      out[6] = c[0];
      return 0;
    }
  }
  return 0;
}

const char* lucid_status_string(int code) {
  switch (code) {
    case 0: return "ok";
    case 1: return "device-side barrier wait timed out";
    case 2: return "a predecessor row-block was never published (flag wait timed out)";
    case 3: return "kernel left early after another CTA reported an error";
    case LUCID_E_BAD_SHAPE: return "bad shape: need B,N,H > 0, head_dim == 128, N % 128 == 0";
    case LUCID_E_BAD_DTYPE: return "bad dtype: need fp16 (0) or bf16 (1)";
    case LUCID_E_BAD_ALIGNMENT: return "bad alignment: 16-byte aligned bases, strides multiples of 8 elements";
    case LUCID_E_WORKSPACE_TOO_SMALL: return "workspace too small (see lucid_workspace_bytes)";
    case LUCID_E_NULL_POINTER: return "null pointer";
    case LUCID_E_TENSOR_MAP: return "cuTensorMapEncodeTiled rejected a tensor";
    case LUCID_E_NO_DEVICE: return "no CUDA device";
    case LUCID_E_BAD_STRIDE:
      return "zero stride in a dimension of extent > 1 (expanded tensor): make the tensor contiguous first";
    case LUCID_E_STATIC_SCRATCH_TOO_SMALL:
      return "problem too large for the library-owned scratch of lucid_fwd_sub_static "
             "(lucid_workspace_bytes(B, N, H) must not exceed LUCID_STATIC_SCRATCH_BYTES - 1023)";
    default: return code > 0 ? "CUDA runtime error" : "unknown";
  }
}

}  // extern "C"

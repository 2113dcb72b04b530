// Block-triangular substitution on sm_100a: the forward solve V' = L^-1 V and, with kReverse, the
// transposed solve dV = L^-T dV' of the backward pass.  Replaces the reference's ForwardSubSm90
// (lucid_kernels/cute/forward_sub_fwd.py:47-841) and the dV part of BackwardSubSm90
// (lucid_kernels/cute/forward_sub_bwd.py:1053-1107).
//
// One persistent CTA per SM takes row-blocks (chain, i) from a global ticket counter in dependency
// order.  For every earlier block j of the chain it computes S = K_i K_j^T (tcgen05, both operands
// from shared memory), P = exp(S) on the TMEM -> register path, and ACC += P * Y_j with P fed back
// from TMEM (Y = V' forward, dV reverse).  The row-block then forms rhs = Y_in_i - ACC, applies the
// unit-triangular inverse X_i (precomputed by diag_prep.cu) as one more MMA together with the row
// scaling exp(-|k_r|^2), stores Y_i and publishes it by raising flag[chain][i] with release semantics (one
// increment per storing warp).  Consumers acquire the complete flag before their TMA load of Y_i.
//
// Critical path.  A chain advances one row-block per "publish -> flag -> load -> finish -> publish"
// hand-over, so everything that does not need the newest predecessor Y_l (l = i-1 forward, i+1 reverse) is
// taken off that hand-over.  With P_l = exp(K_i K_l^T) and A = X_i (forward, rows of the right-hand side
// scaled by lam) or X_i^T (reverse, result rows scaled by lam),
//     Y_i = A (Y_in_i - sum_{j != l} P_j Y_j) - (A P_l) Y_l  =  z - Q Y_l,
// and both z and Q = A P_l are formed while Y_l is still being computed by another CTA: P_l goes to
// shared memory (into the K_i buffer, which the S products no longer need) as the right-hand side of one
// more diagonal product, Q comes back through the idle S buffer, is negated, rounded to 16 bits and parked
// in the idle P buffer.  Once Y_l has arrived a single product OUT += (-Q) Y_l finishes the row-block.
//
// Pair mode (few chains, where the hand-over latency between consecutive row-blocks is what limits a
// chain): the grid is launched as clusters of two CTAs, work items are pairs of consecutive row-blocks of
// a chain.  CTA 0 of a cluster draws the pair's ticket from the global counter and passes it to CTA 1
// through a small mailbox in CTA 1's shared memory, so pairs are claimed in dependency order by clusters
// that are running, exactly like single row-blocks; CTA 0 solves the first row-block and CTA 1 the second.  CTA 0 hands its result to CTA 1 directly: CTA 1 claims the two ring stages of its
// last tile, arms their barriers with the byte count and bumps a counter in CTA 0's shared memory; CTA 0
// stages the tile as always and one thread copies it into those stages with four bulk shared-to-shared
// copies (each with one destination), whose arrival completes CTA 1's stage barriers like a TMA load.  That replaces
// "TMA store, release the flag, acquire it, TMA load" for every second hand-over of the chain.  CTA 0
// still stores and publishes the tile for all later row-blocks; CTA 1 acknowledges receipt on the barrier
// that guards CTA 0's staging buffer.
//
// Warp roles (128 + 128 * kG threads): warp 0 K-producer (tickets, K_i, K_j half-tiles, X_i), warp 1 issues the
// S products and owns TMEM, warp 2 Y-producer (rhs tile, flag waits, Y_j half-tiles), warp 3 issues the
// P*Y and diagonal products, then kG exp groups of four warps (kG = 4 in the stand-alone kernels, 2 when the
// program shares a launch with the dK program) that split every tile's columns (128 / kG each) and share
// the epilogue the same way.  Two issuing warps because tcgen05.mma issue is nearly synchronous
// with execution (the queue holds only a few instructions): the waits of one overlap the MMAs of the other.
//
// Variant kKT ("K_i in tensor memory"): the exp groups copy K_i from shared memory into 64 TMEM columns once
// per row-block and every S product reads its A operand from there, so a tile's S product reads 32 KiB less
// from shared memory, whose port (128 bytes per clock: 64 KiB of tile loads landing, 96 KiB of operand
// reads per tile) is otherwise the busiest unit of the SM.  It pays for the columns with one S buffer (two
// instead of three).
//
// TMEM: three S buffers (tile g uses buffer g % 3) and the accumulator.  An exp thread streams its
// columns of S through registers in 16-column chunks (the next chunk's load in flight) and writes the
// packed P chunk over S columns it has already consumed, so P needs no buffer of its own and the S
// products run up to three tiles ahead of the P*Y products; a buffer returns to the S issuer when the
// P*Y product that read it has completed.
#include <type_traits>
#include "kernels.h"

namespace lucid {

struct SolveSmem {
  alignas(1024) uint8_t ki[kTileBytes];        // K_i: two 64-column panels, 128B-swizzled
  alignas(1024) uint8_t x[kTileBytes];         // X_i, same layout
  alignas(1024) uint8_t rhs[kTileBytes];       // V_i (then rhs) as [row][64-col panel] panels
  alignas(1024) uint8_t kring[4][kHalfBytes];  // K_j panels (64 columns of d x 128 rows)
  alignas(1024) uint8_t vring[4][kHalfBytes];  // Y_j row halves (2 panels x 64 rows x 64 columns)
  alignas(8) uint64_t k_full[4];
  uint64_t k_empty[4], v_full[4], v_empty[4];
  uint64_t ki_full, ki_free, x_full, vi_full, xr_free, r_free, stage_full, kit_full;
  uint64_t s_full[3], sbuf_free[3], p_full[3];
  uint64_t acc_full, acc_free, rhs_full, out_full, pq_full, q_full;

  uint64_t tk_full[2], tk_empty[2];
  int tk_slot[2];
  uint32_t tmem_base;
  int abort_flag;
  int peer_items;        // pair mode, CTA 0: items for whose handed-over tile CTA 1 has claimed its ring stages
  int mail[4];           // pair mode, CTA 1: tickets drawn by CTA 0 (item `it` in slot it & 3; -1 = nothing yet)
};

enum SolveBar : int {
  BAR_K_FULL = 1, BAR_K_EMPTY, BAR_V_FULL, BAR_V_EMPTY, BAR_KI_FULL, BAR_KI_FREE, BAR_X_FULL, BAR_VI_FULL,
  BAR_XR_FREE, BAR_S_FULL, BAR_P_FULL, BAR_ACC_FULL, BAR_ACC_FREE, BAR_RHS_FULL, BAR_OUT_FULL, BAR_TK_FULL,
  BAR_TK_EMPTY, BAR_S_FREE, BAR_P_FREE, BAR_R_FREE, BAR_STAGE_FULL, BAR_PQ_FULL, BAR_Q_FULL, BAR_PEER_READY,
  BAR_PEER_TICKET, BAR_KIT_FULL
};

// Block size: four service warps plus kG exp groups of four warps (128 threads, one per row).
constexpr int solve_threads(int groups) { return 128 + 128 * groups; }
constexpr int kSolveThreads = solve_threads(2);          // the variant that shares a launch with the dK program
constexpr int kSolveGroups = 4;                          // the stand-alone kernels
// TMEM columns: three S buffers (fp32, 128 columns each; P is packed over columns 0-31 and 64-95 of the
// same buffer) and the accumulator; the diagonal product reuses the accumulator's columns once the
// epilogue has read them.  Tile g uses S[g % 3].
constexpr int kTmemS = 0, kTmemAcc = 384, kTmemOut = 384;
constexpr int kTmemKi = 256;      // variant kKT: K_i as a TMEM operand (64 columns), in place of the third S buffer
// Register budget per thread after the role split: the exp / epilogue groups hold a whole S row (128
// fp32) in registers, the four service warps need few.  128 * 56 + 256 * 224 = 64512 <= 65536.
// Register budgets after the role split (setmaxnreg), for kG = 2: 128 * 72 + 256 * 216 = 64512; for kG = 4
// (640 threads, 96 registers each at launch): 128 * 64 + 512 * 104 = 61440.
template <int kG> struct SolveRegs;
template <> struct SolveRegs<2> { static constexpr int service = 72, exp = 216, launch = 168; };
template <> struct SolveRegs<4> { static constexpr int service = 64, exp = 104, launch = 96; };

// The whole CTA program, callable from more than one kernel (the tensor maps must be __grid_constant__
// parameters of the calling kernel).
template <bool kBf16, bool kReverse, int kG, bool kPair = false, bool kKT = false>
__device__ __forceinline__ void solve_body(const CUtensorMap& tm_k,     // K, box 64 x 128
                                           const CUtensorMap& tm_in,    // V (or dV'), box 64 x 128
                                           const CUtensorMap& tm_out,   // Y, box 64 x 64
                                           const CUtensorMap& tm_x,     // X workspace (2D), box 64 x 128
                                           const CUtensorMap& tm_st,    // Y, box 64 x 128, for the TMA store
                                           const SolveArgs& args,
                                           const bool last_program = true) {   // no TMEM allocation follows
  extern __shared__ uint8_t smem_raw[];
  SolveSmem& s = *reinterpret_cast<SolveSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const Problem& P = args.p;
  Control* ctl = args.ctl;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = P.T, H = P.H;
  const unsigned long long limit = P.wait_ns;
  volatile int* cta_abort = &s.abort_flag;
  constexpr int kExpThreads = 128 * kG;      // exp / epilogue threads
  constexpr int kNS = kKT ? 2 : 3;           // S buffers in TMEM
  constexpr int kCols = 128 / kG;            // columns of a tile (and of the output) per exp group
  constexpr int kRegsService = SolveRegs<kG>::service, kRegsExp = SolveRegs<kG>::exp,
                kRegsLaunch = SolveRegs<kG>::launch;

  if (tid == 0) {
    for (int i = 0; i < 4; ++i) {
      mbar_init(&s.k_full[i], 1);
      mbar_init(&s.k_empty[i], 1);
      mbar_init(&s.v_full[i], 1);
      mbar_init(&s.v_empty[i], 1);
    }
    mbar_init(&s.ki_full, 1);
    mbar_init(&s.ki_free, 1);
    mbar_init(&s.x_full, 1);
    mbar_init(&s.vi_full, 1);
    mbar_init(&s.xr_free, 1);
    // pair mode, first CTA: the staged tile is also copied to the peer, which acknowledges receipt
    mbar_init(&s.r_free, (kPair && cluster_ctarank() == 0) ? 2 : 1);
    mbar_init(&s.stage_full, kExpThreads);
    mbar_init(&s.kit_full, kExpThreads);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&s.s_full[i], 1);
      mbar_init(&s.sbuf_free[i], 1);
      mbar_init(&s.p_full[i], kExpThreads);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.tk_full[i], 1);
      mbar_init(&s.tk_empty[i], 3 + 4 * kG);
    }
    mbar_init(&s.acc_full, 1);
    mbar_init(&s.acc_free, kExpThreads);
    mbar_init(&s.rhs_full, kExpThreads);
    mbar_init(&s.out_full, 1);
    mbar_init(&s.pq_full, kExpThreads);
    mbar_init(&s.q_full, 1);
    s.abort_flag = 0;
    s.peer_items = 0;
    for (int i = 0; i < 4; ++i) s.mail[i] = -1;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, 512);
    // giving up the allocation permit is final for the CTA: only when no other program follows in this kernel
    if (last_program) tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  // pair mode: the peer's barriers exist before anybody arrives on them
  const uint32_t crank = kPair ? cluster_ctarank() : 0u;
  if (kPair) cluster_sync_all();
  // tracing builds: wall time and SM cycles at the start and end of this CTA (role 6) give the SM clock
  {
    int slot6 = (kReverse ? 2 : 0);
    (void)slot6;
    if (tid == 0) LUCID_TR(args.trace, 6, slot6, 90, (long long)globaltimer_ns());
  }
  tc_fence_after_sync();
  const uint32_t tmem = s.tmem_base;

  // Every role walks the same sequence of items; `it` counts items, `g` counts (i, j) tiles and `u`
  // half-tiles, all per CTA, so that ring stages and barrier phases agree between roles.  Tile g uses
  // S buffer g % 3 in phase (g / 3) & 1.
  auto item_geometry = [&](int ticket, int& chain, int& i, int& n, int& jfirst) -> bool {
    int step;
    if (kPair) {
      // a work item is a pair of consecutive row-blocks (T is even): this CTA solves the first or second
      int ps;
      if (!decode_ticket(ticket, P.C, T >> 1, P.group, 0, 0, chain, ps)) return false;
      step = 2 * ps + (int)crank;
    } else if (!decode_ticket(ticket, P.C, T, P.group, P.head, P.overlap, chain, step)) {
      return false;
    }
    if (kReverse) {
      i = T - 1 - step;
      n = step;           // blocks i+1 .. T-1, visited from T-1 down to i+1
      jfirst = T - 1;
    } else {
      i = step;
      n = (P.window >= 0) ? min(step, P.window) : step;
      jfirst = i - n;     // visited upward to i-1
    }
    return true;
  };
  auto tile_j = [&](int jfirst, int q) -> int { return kReverse ? jfirst - q : jfirst + q; };
  // Items with a diagonal inverse and at least one predecessor finish through Q (see the file header):
  // their last tile is not accumulated but folded into OUT after the diagonal product.
  auto q_route = [&](int n) -> bool { return P.use_diag && n > 0; };

  // Each role sets its register budget inside its own branch, so that the compiler ties the budget to
  // the code that runs under it (warps 0-3 form one warpgroup and all execute the same decrease).
  if (warp == 0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsService));
    // =========================== K producer (one lane) ===========================
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_x);
      const uint64_t pol_once = l2_policy_evict_first();     // X_i: read once per row-block
      uint32_t u = 0;
      bool alive = true;
      int trc = 0;
      (void)trc;
      int last_ticket = -1;      // pair mode, CTA 1: the newest ticket taken from the mailbox
      (void)last_ticket;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_empty[slot], ((it >> 1) & 1) ^ 1, cta_abort, ctl, limit, -1, -1, BAR_TK_EMPTY)) break;
        // Pair mode: both CTAs of a cluster work on the same pair.  CTA 0 draws the ticket and posts it in
        // CTA 1's mailbox; CTA 1 takes it from there.  Tickets of a cluster increase, so a slot holds news
        // once its value exceeds the last ticket seen.  Four slots suffice: CTA 0 draws the ticket of item m
        // only after all its roles have started item m - 2, i.e. after it handed over the tile of item
        // m - 3, for which CTA 1 had to have taken ticket m - 3 - so at most three tickets are in flight.
        int ticket;
        if (!kPair || crank == 0) {
          ticket = atomicAdd(&ctl->ticket, 1);
          if (kPair) st_release_cluster(mapa_u32(smem_u32(&s.mail[it & 3]), 1), ticket);
        } else {
          const int* slot_word = &s.mail[it & 3];
          ticket = ld_acquire_cluster_local(slot_word);
          if (ticket <= last_ticket) {
            const uint64_t t0 = globaltimer_ns();
            uint32_t spins = 0;
            while ((ticket = ld_acquire_cluster_local(slot_word)) <= last_ticket) {
              if ((++spins & 63u) == 0) {
                if (*cta_abort) break;
                if (globaltimer_ns() - t0 > limit) {
                  *cta_abort = 1;
                  report_error(ctl, kErrBarrierTimeout, -1, -1, it, BAR_PEER_TICKET);
                  break;
                }
              }
            }
            if (ticket <= last_ticket) break;
          }
          last_ticket = ticket;
        }
        s.tk_slot[slot] = ticket;
        mbar_arrive(&s.tk_full[slot]);
        int chain, i, n, jfirst;
        if (!item_geometry(ticket, chain, i, n, jfirst)) break;
        const int b = chain / H, h = chain % H;
        // K_i once the previous item's S products have drained
        if (!wait_barrier(&s.ki_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, BAR_KI_FREE)) break;
        mbar_expect_tx(&s.ki_full, kTileBytes);
        tma_load_4d(s.ki, &tm_k, &s.ki_full, 0, i * kBlock, h, b);
        tma_load_4d(s.ki + kHalfBytes, &tm_k, &s.ki_full, 64, i * kBlock, h, b);
        bool x_loaded = !P.use_diag;
        for (int q = 0; q < n && alive; ++q) {
          const int j = tile_j(jfirst, q);
          for (int half = 0; half < 2; ++half, ++u) {
            const int st = u & 3;
            if (!wait_barrier(&s.k_empty[st], ((u >> 2) & 1) ^ 1, cta_abort, ctl, limit, chain, i, BAR_K_EMPTY)) {
              alive = false;
              break;
            }
            mbar_expect_tx(&s.k_full[st], kHalfBytes);
            tma_load_4d(s.kring[st], &tm_k, &s.k_full[st], 64 * half, j * kBlock, h, b);
            LUCID_TR(args.trace, 0, trc, 10, u);
          }
          if (alive && !x_loaded && mbar_try_wait(&s.xr_free, (it & 1) ^ 1)) {
            mbar_expect_tx(&s.x_full, kTileBytes);
            tma_load_2d_hint(s.x, &tm_x, &s.x_full, 0, (chain * T + i) * kBlock, pol_once);
            tma_load_2d_hint(s.x + kHalfBytes, &tm_x, &s.x_full, 64, (chain * T + i) * kBlock, pol_once);
            x_loaded = true;
          }
        }
        if (alive && !x_loaded) {
          if (!wait_barrier(&s.xr_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, BAR_XR_FREE)) break;
          mbar_expect_tx(&s.x_full, kTileBytes);
          tma_load_2d_hint(s.x, &tm_x, &s.x_full, 0, (chain * T + i) * kBlock, pol_once);
          tma_load_2d_hint(s.x + kHalfBytes, &tm_x, &s.x_full, 64, (chain * T + i) * kBlock, pol_once);
        }
      }
    }
  } else if (warp == 2) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsService));
    // =========================== Y producer (one lane) ===========================
    if (lane == 0) {
      tma_prefetch_desc(&tm_in);
      tma_prefetch_desc(&tm_out);
      const uint64_t pol_once = l2_policy_evict_first();     // the row-block's own right-hand side: read once
      uint32_t u = 0;
      bool alive = true;
      int trc = 0;
      (void)trc;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, BAR_TK_FULL)) break;
        const int ticket = s.tk_slot[slot];
        mbar_arrive(&s.tk_empty[slot]);
        int chain, i, n, jfirst;
        if (!item_geometry(ticket, chain, i, n, jfirst)) break;
        const int b = chain / H, h = chain % H;
        // This row-block's own right-hand side goes into the rhs buffer as soon as the previous
        // item's diagonal product has released it; the ring loads below do not wait for that.
        bool vi_loaded = false;
        auto load_vi = [&]() {
          mbar_expect_tx(&s.vi_full, kTileBytes);
          tma_load_4d_hint(s.rhs, &tm_in, &s.vi_full, 0, i * kBlock, h, b, pol_once);
          tma_load_4d_hint(s.rhs + kHalfBytes, &tm_in, &s.vi_full, 64, i * kBlock, h, b, pol_once);
          vi_loaded = true;
        };
        unsigned long long waited = 0;
        // one look at the block kFlagProbe steps behind the newest predecessor usually spares the older tiles
        // their own flag round trip (see flags_known_up)
        const int skip_until = P.no_sync ? 0 : flags_known_up(args.flags + chain * T, n, tile_j(jfirst, n - kFlagProbe));
        for (int q = 0; q < n && alive; ++q) {
          const int j = tile_j(jfirst, q);
          if (!vi_loaded && mbar_try_wait(&s.r_free, (it & 1) ^ 1)) load_vi();
          // Both ring stages of this tile are claimed before the flag is awaited, so that only the proxy
          // fence stands between observing the flag and issuing the four loads.
          const int st0 = u & 3, st1 = (u + 1) & 3;
          if (!wait_barrier(&s.v_empty[st0], ((u >> 2) & 1) ^ 1, cta_abort, ctl, limit, chain, i, BAR_V_EMPTY) ||
              !wait_barrier(&s.v_empty[st1], (((u + 1) >> 2) & 1) ^ 1, cta_abort, ctl, limit, chain, i, BAR_V_EMPTY)) {
            alive = false;
            break;
          }
          if (kPair && crank == 1 && q == n - 1) {
            // The newest predecessor is the row-block the peer CTA is solving: it writes the tile into the
            // two stages just claimed and arrives on their barriers itself.
            mbar_expect_tx(&s.v_full[st0], kHalfBytes);
            mbar_expect_tx(&s.v_full[st1], kHalfBytes);
            st_release_cluster(mapa_u32(smem_u32(&s.peer_items), 0), it + 1);
            u += 2;
            continue;
          }
          if (!P.no_sync && q >= skip_until) {
            if (!wait_flag(args.flags + chain * T + j, cta_abort, ctl, limit, chain, i, j,
                           P.instrument ? &waited : nullptr)) {
              alive = false;
              break;
            }
            fence_proxy_async_all();   // flag acquired in the generic proxy; the tile is read by TMA
          }
          LUCID_TR(args.trace, 1, trc, 20, q);
          mbar_expect_tx(&s.v_full[st0], kHalfBytes);
          tma_load_4d(s.vring[st0], &tm_out, &s.v_full[st0], 0, j * kBlock, h, b);
          tma_load_4d(s.vring[st0] + 8192, &tm_out, &s.v_full[st0], 64, j * kBlock, h, b);
          mbar_expect_tx(&s.v_full[st1], kHalfBytes);
          tma_load_4d(s.vring[st1], &tm_out, &s.v_full[st1], 0, j * kBlock + 64, h, b);
          tma_load_4d(s.vring[st1] + 8192, &tm_out, &s.v_full[st1], 64, j * kBlock + 64, h, b);
          LUCID_TR(args.trace, 1, trc, 21, u);
          u += 2;
        }
        if (alive && !vi_loaded) {
          if (!wait_barrier(&s.r_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, BAR_R_FREE)) break;
          load_vi();
        }
        if (P.instrument && args.timestamps) args.timestamps[(chain * T + i) * 8 + 3] = (long long)waited;
      }
    }
  } else if (warp == 1) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsService));
    // =========================== S issuer ===========================
    // The whole warp walks the loop (uniform control flow, waits included); one elected lane issues.
    {
      const bool leader = (lane == 0);
      (void)leader;
      constexpr int fmt = kBf16 ? 1 : 0;
      constexpr uint32_t idesc_s = umma_idesc(fmt, 0, 0, 128, 128);    // S = K_i K_j^T
      const uint64_t d_ki = umma_smem_desc(smem_u32(s.ki), 16, 1024);
      const uint64_t d_kr0 = umma_smem_desc(smem_u32(s.kring[0]), 16, 1024);     // stage st: + st * 16 KiB
      uint32_t g = 0;            // tiles issued so far
      bool alive = true;
      int trc = 0;
      (void)trc;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, BAR_TK_FULL)) break;
        const int ticket = s.tk_slot[slot];
        __syncwarp();
        mbar_arrive_w(&s.tk_empty[slot]);
        int chain, i, n, jfirst;
        if (!item_geometry(ticket, chain, i, n, jfirst)) break;
        // K_i is in place: in shared memory, or (kKT) copied into tensor memory by the exp groups
        if (kKT ? !wait_barrier(&s.kit_full, it & 1, cta_abort, ctl, limit, chain, i, BAR_KIT_FULL)
                : !wait_barrier(&s.ki_full, it & 1, cta_abort, ctl, limit, chain, i, BAR_KI_FULL))
          break;
        tc_fence_after_sync();
        if (leader) LUCID_TR(args.trace, 2, trc, 35, n);
        for (int q = 0; q < n; ++q) {
          const uint32_t gq = g + q;
          const uint32_t buf = gq % kNS;
          // the P*Y product of kNS tiles ago, which read P from this buffer, has completed
          if (!wait_barrier(&s.sbuf_free[buf], ((gq / kNS) & 1) ^ 1, cta_abort, ctl, limit, chain, i, BAR_S_FREE)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t dst = tmem + kTmemS + buf * 128;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const uint32_t u = gq * 2 + half;
            const uint32_t st = u & 3;
            if (!wait_barrier(&s.k_full[st], (u >> 2) & 1, cta_abort, ctl, limit, chain, i, BAR_K_FULL)) {
              alive = false;
              break;
            }
            tc_fence_after_sync();
            if (leader) LUCID_TR(args.trace, 2, trc, 30, u);
            const uint64_t da = desc_advance(d_ki, half * kHalfBytes);
            const uint64_t db = d_kr0 + st * (kHalfBytes >> 4);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              if (kKT) umma_ts_w(dst, tmem + kTmemKi + (half * 4 + kk) * 8, db + kk * 2, idesc_s, (half | kk) ? 1u : 0u);
              else umma_ss_w(dst, da + kk * 2, db + kk * 2, idesc_s, (half | kk) ? 1u : 0u);
            }
            umma_commit_w(&s.k_empty[st]);
          }
          if (!alive) break;
          umma_commit_w(&s.s_full[buf]);
          if (leader) LUCID_TR(args.trace, 2, trc, 31, gq);
        }
        if (!alive) break;
        g += n;
        // every S product of this item has been issued: K_i may be replaced once they complete, unless
        // the buffer goes on to hold P_l for the Q product (then the P*Y issuer releases it)
        if (!q_route(n)) {
          if (n > 0) umma_commit_w(&s.ki_free);
          else mbar_arrive_w(&s.ki_free);
        }
      }
    }
  } else if (warp == 3) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsService));
    // =========================== P*Y and diagonal-product issuer ===========================
    {
      const bool leader = (lane == 0);
      (void)leader;
      constexpr int fmt = kBf16 ? 1 : 0;
      constexpr uint32_t idesc_pv = umma_idesc(fmt, 0, 1, 128, 128);   // ACC += P Y_j   (B: rows = k)
      constexpr uint32_t idesc_out = umma_idesc(fmt, kReverse ? 1 : 0, 1, 128, 128);  // OUT = X(^T) rhs
      const uint64_t d_x = kReverse ? umma_smem_desc(smem_u32(s.x), kHalfBytes, 1024)
                                    : umma_smem_desc(smem_u32(s.x), 16, 1024);
      const uint64_t d_rhs = umma_smem_desc(smem_u32(s.rhs), kHalfBytes, 1024);
      const uint64_t d_pl = umma_smem_desc(smem_u32(s.ki), kHalfBytes, 1024);      // P_l, laid out like rhs
      const uint64_t d_vr0 = umma_smem_desc(smem_u32(s.vring[0]), 8192, 1024);
      uint32_t g = 0;
      uint32_t nq = 0;           // items finished through Q so far (phase of pq_full / q_full)
      bool alive = true;
      int trc = 0;
      (void)trc;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, BAR_TK_FULL)) break;
        const int ticket = s.tk_slot[slot];
        __syncwarp();
        mbar_arrive_w(&s.tk_empty[slot]);
        int chain, i, n, jfirst;
        if (!item_geometry(ticket, chain, i, n, jfirst)) break;
        const bool via_q = q_route(n);
        const int n_acc = via_q ? n - 1 : n;      // tiles accumulated before the diagonal product
        // ACC (or OUT, with fold) += P[buf] * Y ring tile of tile gq
        auto issue_py = [&](uint32_t gq, bool first, bool fold) -> bool {
          const uint32_t buf = gq % kNS;
          if (!wait_barrier(&s.p_full[buf], (gq / kNS) & 1, cta_abort, ctl, limit, chain, i, BAR_P_FULL)) return false;
          if (leader) LUCID_TR(args.trace, 5, trc, 32, gq);
          if (first && !wait_barrier(&s.acc_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, BAR_ACC_FREE))
            return false;
          const uint32_t p_tmem = tmem + kTmemS + buf * 128;   // group g's P: columns g*kCols .. + kCols/2
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const uint32_t u = gq * 2 + half;
            const uint32_t st = u & 3;
            if (!wait_barrier(&s.v_full[st], (u >> 2) & 1, cta_abort, ctl, limit, chain, i, BAR_V_FULL)) return false;
            // pair mode: the handed-over tile has arrived (second half), the peer may reuse its staging buffer
            if (kPair && fold && crank == 1 && half == 1 && elect_one())
              mbar_arrive_cluster(mapa_u32(smem_u32(&s.r_free), 0));
            tc_fence_after_sync();
            if (leader) LUCID_TR(args.trace, 5, trc, 33, u);
            const uint64_t db = d_vr0 + st * (kHalfBytes >> 4);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              // k-step ks = 4*half + kk covers K columns 16*ks ..: group ks / (kCols/16), its chunk ks % (kCols/16)
              umma_ts_w(tmem + kTmemAcc,
                        p_tmem + ((half * 4 + kk) / (kCols / 16)) * kCols + ((half * 4 + kk) % (kCols / 16)) * 8,
                        db + kk * (2048 >> 4), idesc_pv,
                        (!first || fold || half || kk) ? 1u : 0u);
            }
            umma_commit_w(&s.v_empty[st]);
          }
          umma_commit_w(&s.sbuf_free[buf]);
          if (leader) LUCID_TR(args.trace, 5, trc, 34, gq);
          return true;
        };
        // Pair mode: a chain's row-blocks are published in quick pairs, so the last TWO predecessors of a
        // row-block arrive late and close together; Q, which needs no Y at all, is therefore formed before
        // the last accumulated tile instead of after it.
        const int n_early = (kPair && via_q && n_acc >= 1) ? n_acc - 1 : n_acc;
        for (int q = 0; q < n_early; ++q) {
          if (!issue_py(g + q, q == 0, false)) {
            alive = false;
            break;
          }
        }
        if (!alive) break;
        if (n_early == n_acc) umma_commit_w(&s.acc_full);
        if (via_q) {
          // Q = X(^T) P_l into the S buffer the last tile came from (its group has drained it)
          if (!wait_barrier(&s.pq_full, nq & 1, cta_abort, ctl, limit, chain, i, BAR_PQ_FULL)) break;
          if (!wait_barrier(&s.x_full, it & 1, cta_abort, ctl, limit, chain, i, BAR_X_FULL)) break;
          tc_fence_after_sync();
          const uint32_t q_tmem = tmem + kTmemS + ((g + n - 1) % kNS) * 128;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t da = kReverse ? desc_advance(d_x, k * 2048)
                                         : desc_advance(d_x, (k >> 2) * kHalfBytes + (k & 3) * 32);
            umma_ss_w(q_tmem, da, desc_advance(d_pl, k * 2048), idesc_out, k ? 1u : 0u);
          }
          umma_commit_w(&s.q_full);
          umma_commit_w(&s.ki_free);
        }
        if (n_early < n_acc) {
          if (!issue_py(g + n_acc - 1, n_acc == 1, false)) break;
          umma_commit_w(&s.acc_full);
        }
        // diagonal step
        if (!wait_barrier(&s.rhs_full, it & 1, cta_abort, ctl, limit, chain, i, BAR_RHS_FULL)) break;
        tc_fence_after_sync();
        if (leader) LUCID_TR(args.trace, 5, trc, 36, 0);
        if (P.use_diag) {
          if (!wait_barrier(&s.x_full, it & 1, cta_abort, ctl, limit, chain, i, BAR_X_FULL)) break;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t da = kReverse ? desc_advance(d_x, k * 2048)
                                         : desc_advance(d_x, (k >> 2) * kHalfBytes + (k & 3) * 32);
            umma_ss_w(tmem + kTmemOut, da, desc_advance(d_rhs, k * 2048), idesc_out, k ? 1u : 0u);
          }
          umma_commit_w(&s.xr_free);
          if (leader) LUCID_TR(args.trace, 5, trc, 37, 0);
          if (via_q) {
            // OUT += (-Q) Y_l: the only product that waits for the newest predecessor
            if (!issue_py(g + n - 1, false, true)) break;
            ++nq;
          }
          umma_commit_w(&s.out_full);
        } else {
          mbar_arrive_w(&s.xr_free);
          mbar_arrive_w(&s.r_free);
        }
        g += n;
      }
    }
  } else if (warp >= 4) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsExp));
    // =========================== exp groups + epilogue ===========================
    const int wg = (warp - 4) >> 2;                  // exp group: columns kCols*wg .. of every tile and of the output
    const float xs = P.exp_scale;                    // exp(k_scale^2 * S) = exp2(S * xs)
    constexpr int kCh = kCols / 16;                  // 16-column chunks per thread and tile
    constexpr int kVec = kCols / 8;                  // 16-byte vectors of 16-bit values per thread and row
    uint8_t* const my_ki = s.ki + (wg * kCols / 64) * kHalfBytes;     // this group's 64-column panel ...
    uint8_t* const my_rhs = s.rhs + (wg * kCols / 64) * kHalfBytes;
    const uint32_t vec0 = (wg * kCols % 64) / 8;                       // ... and its first vector in a panel row
    const int row = ((warp & 3) << 5) + lane;        // TMEM lane == row of the block
    const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    uint32_t g = 0;
    uint32_t nq = 0;             // items finished through Q so far (phase of pq_full / q_full)
    uint32_t u_peer = 0;         // pair mode, CTA 0: half-tiles the peer CTA's rings have seen so far
    bool alive = true;
    int trc = 0;
    (void)trc;
    const bool tr_lead = (tid == 128 || tid == 256) && wg < 2;
    (void)tr_lead;
    for (int it = 0; alive; ++it) {
      const int slot = it & 1;
      if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, BAR_TK_FULL)) break;
      const int ticket = s.tk_slot[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.tk_empty[slot]);
      int chain, i, n, jfirst;
      if (!item_geometry(ticket, chain, i, n, jfirst)) break;
      const int b = chain / H, h = chain % H;
      const bool via_q = q_route(n);
      long long t_start = 0, c_start = 0;
      if (P.instrument && tid == 128) {
        t_start = (long long)globaltimer_ns();
        c_start = clock64();
      }
      const float lam = P.use_diag ? args.lam_inv[(chain * T + i) * kBlock + row] : 1.0f;

      if (kKT) {
        // K_i, shared memory -> tensor memory: this thread's row, this group's kCols columns (kCols / 2 words of
        // 16-bit pairs).  The region's previous reader, the last S product of the item before, completed before
        // the load of this K_i was even issued.
        if (!wait_barrier(&s.ki_full, it & 1, cta_abort, ctl, limit, chain, i, BAR_KI_FULL)) break;
#pragma unroll
        for (int c = 0; c < kCols / 32; ++c) {
          uint32_t w[16];
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            const uint4 t4 = *reinterpret_cast<const uint4*>(my_ki + sw128_off(row, vec0 + c * 4 + v4));
            w[4 * v4] = t4.x; w[4 * v4 + 1] = t4.y; w[4 * v4 + 2] = t4.z; w[4 * v4 + 3] = t4.w;
          }
          tmem_st16(lane_base + kTmemKi + wg * (kCols / 2) + c * 16, w);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&s.kit_full);
      }

      // ---- P = exp(S): this group's kCols columns of every tile ----
      for (int q = 0; q < n; ++q) {
        const uint32_t gq = g + q;
        const uint32_t buf = gq % kNS;
        const uint32_t ph = (gq / kNS) & 1;
        if (!wait_barrier(&s.s_full[buf], ph, cta_abort, ctl, limit, chain, i, BAR_S_FULL)) {
          alive = false;
          break;
        }
        tc_fence_after_sync();
        if (tr_lead) LUCID_TR(args.trace, 3 + wg, trc, 40, gq);
        const uint32_t s_tmem = lane_base + kTmemS + buf * 128 + wg * kCols;
        if (via_q && q == n - 1) {
          // ---- last tile of a Q-route item: P_l to shared memory, Q back through this S buffer ----
          // P_l (forward: rows scaled by lam, folded into the exponent) in the layout of the rhs buffer,
          // written over K_i: s_full of the last tile implies that every S product has completed.  This
          // group's columns sit inside one 64-column panel.
          uint32_t v[kCols];
#pragma unroll
          for (int c = 0; c < kCols / 32; ++c) tmem_ld32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
          tmem_wait_ld();
          const float shift = (P.use_diag && !kReverse) ? __log2f(lam) : 0.0f;
#pragma unroll
          for (int c = 0; c < kVec; ++c) {
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float e0 = ex2_approx(fmaf(__uint_as_float(v[c * 8 + 2 * e]), xs, shift));
              const float e1 = ex2_approx(fmaf(__uint_as_float(v[c * 8 + 2 * e + 1]), xs, shift));
              o[e] = pack2_fast<kBf16>(e0, e1);
            }
            *reinterpret_cast<uint4*>(my_ki + sw128_off(row, vec0 + c)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
          fence_proxy_async_smem();
          tc_fence_before_sync();
          mbar_arrive(&s.pq_full);          // all groups: S has been read, P_l is in shared memory
          if (!wait_barrier(&s.q_full, nq & 1, cta_abort, ctl, limit, chain, i, BAR_Q_FULL)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < kCols / 32; ++c) tmem_ld32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
          tmem_wait_ld();
          // -Q, rounded to 16 bits, over the first half of the columns just read
#pragma unroll
          for (int c = 0; c < kCols / 32; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e)
              pk[e] = pack2<kBf16>(-__uint_as_float(v[c * 32 + 2 * e]), -__uint_as_float(v[c * 32 + 2 * e + 1]));
            tmem_st16(s_tmem + c * 16, pk);
          }
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(&s.p_full[buf]);      // -Q is in place for the closing product
          if (tr_lead) LUCID_TR(args.trace, 3 + wg, trc, 41, gq);
          continue;
        }
        // Chunk c: columns 16c .. 16c+15 of this thread's range; its packed P lands on columns 8c .. 8c+7,
        // inside chunks <= c, which are already in registers.
        uint32_t sv[2][16];
        tmem_ld16(s_tmem, sv[0]);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < kCh; ++c) {
          if (c + 1 < kCh) tmem_ld16(s_tmem + (c + 1) * 16, sv[(c + 1) & 1]);
          uint32_t pk[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float e0 = ex2_mixed(__uint_as_float(sv[c & 1][2 * e]) * xs, 2 * e);
            const float e1 = ex2_mixed(__uint_as_float(sv[c & 1][2 * e + 1]) * xs, 2 * e + 1);
            pk[e] = pack2_fast<kBf16>(e0, e1);
          }
          if (c + 1 < kCh) tmem_wait_ld();
          tmem_st8(s_tmem + c * 8, pk);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&s.p_full[buf]);
        if (tr_lead) LUCID_TR(args.trace, 3 + wg, trc, 41, gq);
      }
      if (!alive) break;
      g += n;
      if (via_q) ++nq;

      // ---- epilogue: this group owns output columns kCols*wg .. + kCols-1 ----
      // Everything that does not depend on the accumulator is done before waiting for it: this
      // row-block's own right-hand side is read from shared memory now.
      if (!wait_barrier(&s.vi_full, it & 1, cta_abort, ctl, limit, chain, i, BAR_VI_FULL)) break;
      uint8_t* panel = my_rhs;
      uint4 vin[kVec];
#pragma unroll
      for (int c = 0; c < kVec; ++c) vin[c] = *reinterpret_cast<const uint4*>(panel + sw128_off(row, vec0 + c));
      const float pre = (P.use_diag && !kReverse) ? lam : 1.0f;   // forward: rows scaled before X
      const float post = (P.use_diag && kReverse) ? lam : 1.0f;   // reverse: rows scaled after X^T
      typedef typename std::conditional<kBf16, __nv_bfloat16, __half>::type elem_t;
      elem_t* out_row = reinterpret_cast<elem_t*>(args.out) + (long long)b * args.out_strides.b +
                        (long long)(i * kBlock + row) * args.out_strides.n + (long long)h * args.out_strides.h +
                        wg * kCols;
      uint32_t acc[kCols];
      if (!wait_barrier(&s.acc_full, it & 1, cta_abort, ctl, limit, chain, i, BAR_ACC_FULL)) break;
      if ((via_q ? n - 1 : n) > 0) {      // tiles accumulated before the diagonal product
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < kCols / 32; ++c)
          tmem_ld32(lane_base + kTmemAcc + wg * kCols + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[c * 32]));
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int e = 0; e < kCols; ++e) acc[e] = 0u;
      }
      // The diagonal product is written over the accumulator, so with use_diag the accumulator is
      // released only after that product has been read back (below).
      if (!P.use_diag) {
        tc_fence_before_sync();
        mbar_arrive(&s.acc_free);
      }
      if (tr_lead) LUCID_TR(args.trace, 3 + wg, trc, 42, n);
      long long t_loop = 0;
      if (P.instrument && tid == 128) t_loop = (long long)globaltimer_ns();
#pragma unroll
      for (int c = 0; c < kVec; ++c) {
        const uint32_t in[4] = {vin[c].x, vin[c].y, vin[c].z, vin[c].w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack2<kBf16>(in[e]);
          const float r0 = (f.x - __uint_as_float(acc[c * 8 + 2 * e])) * pre;
          const float r1 = (f.y - __uint_as_float(acc[c * 8 + 2 * e + 1])) * pre;
          o[e] = pack2<kBf16>(r0, r1);
        }
        const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
        if (P.use_diag) *reinterpret_cast<uint4*>(panel + sw128_off(row, vec0 + c)) = ov;
        else *reinterpret_cast<uint4*>(out_row + c * 8) = ov;
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&s.rhs_full);
      if (tr_lead) LUCID_TR(args.trace, 3 + wg, trc, 43, 0);

      if (P.use_diag) {
        if (!wait_barrier(&s.out_full, it & 1, cta_abort, ctl, limit, chain, i, BAR_OUT_FULL)) break;
        tc_fence_after_sync();
        if (tr_lead) LUCID_TR(args.trace, 3 + wg, trc, 44, 0);
#pragma unroll
        for (int c = 0; c < kCols / 32; ++c)
          tmem_ld32(lane_base + kTmemOut + wg * kCols + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[c * 32]));
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(&s.acc_free);
        // Y_i goes back into the rhs buffer (the diagonal product has finished reading it), in the layout
        // the TMA store expects, and one thread stores the tile, waits for the store to complete and
        // releases the flag: a single bulk store and a release by a thread with nothing else in flight
        // publish faster than 256 threads' plain stores followed by GPU-scope fences.
        // Pair mode, CTA 0: the same values also go straight into the peer CTA's ring, into the two stages
        // it has claimed for its last tile (rows 0-63 and 64-127 of the tile, two 64-column panels each).
        uint32_t st0 = 0, st1 = 0;
        const bool hand_over = kPair && crank == 0;
        if (hand_over) {
          const uint32_t u_last = u_peer + 2 * (uint32_t)n;          // the peer's item has n + 1 tiles
          st0 = u_last & 3;
          st1 = (u_last + 1) & 3;
          u_peer = u_last + 2;
        }
#pragma unroll
        for (int c = 0; c < kVec; ++c) {
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            o[e] = pack2<kBf16>(__uint_as_float(acc[c * 8 + 2 * e]) * post, __uint_as_float(acc[c * 8 + 2 * e + 1]) * post);
          }
          *reinterpret_cast<uint4*>(panel + sw128_off(row, vec0 + c)) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        // local staging: read by the TMA store (async proxy).  The peer's copy is fenced on the peer's side,
        // after it has acquired the barrier: a cluster-wide proxy fence here cost 4000 cycles per row-block.
        fence_proxy_async_smem();
        mbar_arrive(&s.stage_full);
        if (tid == 128) {
          if (hand_over) {
            if (!wait_barrier(&s.stage_full, it & 1, cta_abort, ctl, limit, chain, i, BAR_STAGE_FULL)) break;
            // Has the peer claimed its stages for this item?  A counter, not a barrier phase: the peer's
            // producer may run an item ahead.  Only this thread needs to know (cluster-scope acquire loads
            // are expensive), and normally the answer has been yes for a while.
            if (ld_acquire_cluster_local(&s.peer_items) <= it) {
              const uint64_t t0 = globaltimer_ns();
              uint32_t spins = 0;
              bool ok = true;
              while (ld_acquire_cluster_local(&s.peer_items) <= it) {
                if ((++spins & 63u) == 0) {
                  if (*cta_abort) { ok = false; break; }
                  if (globaltimer_ns() - t0 > limit) {
                    *cta_abort = 1;
                    report_error(ctl, kErrBarrierTimeout, chain, i, 0, BAR_PEER_READY);
                    ok = false;
                    break;
                  }
                }
              }
              if (!ok) break;
            }
            // The staged tile (two 64-column panels of 128 rows) goes to the peer as four 8 KiB bulk copies:
            // rows 0-63 of both panels into stage st0, rows 64-127 into st1 - the layout of a ring stage, and
            // the swizzle pattern repeats every 8 rows, so the bytes are copied as they are.  Their arrival
            // completes the peer's stage barriers like a TMA load; the peer acknowledges on r_free.
#pragma unroll
            for (int hp = 0; hp < 4; ++hp) {
              const uint32_t half_rows = hp >> 1, pnl = hp & 1;
              const uint32_t st = half_rows ? st1 : st0;
              bulk_copy_to_peer(mapa_u32(smem_u32(s.vring[st]) + pnl * 8192u, 1),
                                smem_u32(s.rhs) + pnl * kHalfBytes + half_rows * 8192u, 8192u,
                                mapa_u32(smem_u32(&s.v_full[st]), 1));
            }
          } else if (!wait_barrier(&s.stage_full, it & 1, cta_abort, ctl, limit, chain, i, BAR_STAGE_FULL)) {
            break;
          }
          LUCID_TR(args.trace, 3, trc, 47, i);
          tma_store_4d(&tm_st, s.rhs, 0, i * kBlock, h, b);
          tma_store_4d(&tm_st, s.rhs + kHalfBytes, 64, i * kBlock, h, b);
          tma_store_commit();
          tma_store_wait_read();
          LUCID_TR(args.trace, 3, trc, 48, i);
          mbar_arrive(&s.r_free);          // the next row-block's right-hand side may be loaded
          tma_store_wait_all();
          LUCID_TR(args.trace, 3, trc, 49, i);
          fence_proxy_async_all();
          st_release_gpu(args.flags + chain * T + i, kFlagComplete);
        }
      } else {
        // ---- publish (identity diagonal: the result was stored with plain stores above) ----
        // Each warp orders its lanes' stores with a warp barrier and then adds its share to the flag with
        // release semantics at GPU scope; a consumer that acquires the full value observes all warps' stores.
        __syncwarp();
        if (lane == 0) red_release_gpu_add(args.flags + chain * T + i, kFlagComplete / (4 * kG));
      }
      if (tid == 128) {
        LUCID_TR(args.trace, 3, trc, 45, i);
        if (P.instrument && args.timestamps) {
          long long* ts = args.timestamps + (long long)(chain * T + i) * 8;
          ts[0] = t_start;
          ts[1] = t_loop;
          ts[2] = (long long)globaltimer_ns();
          ts[4] = blockIdx.x;
          ts[5] = n;
          ts[6] = clock64() - c_start;   // SM cycles from start to publication (ts[2] - ts[0] in ns)
        }
      }
    }
  }

  // teardown: everybody meets here, also after an abort
  if (kPair && s.abort_flag && crank == 0 && tid == 0) {
    // the peer's producer must not wait for tickets that will never be drawn: post one beyond the last item
    for (int i = 0; i < 4; ++i) st_release_cluster(mapa_u32(smem_u32(&s.mail[i]), 1), 0x7fffffff);
  }
  if (s.abort_flag) {
    // give copies and MMAs still in flight time to land before shared memory and TMEM are released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    if (tid == 0) report_error(ctl, kErrAborted, -1, -1, blockIdx.x, 0);
  }
  tc_fence_before_sync();
  {
    int slot6 = (kReverse ? 2 : 0) + 1;
    (void)slot6;
    if (tid == 0) LUCID_TR(args.trace, 6, slot6, 91, (long long)globaltimer_ns());
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
  // pair mode: the peer no longer writes into this CTA's shared memory or arrives on its barriers
  if (kPair) cluster_sync_all();
  if (!last_program) {
    // Another CTA program follows in the same kernel: it lays its own barriers over this memory, and its
    // warps run with the kernel's launch-time register count again (the exp warpgroups give back what the
    // service warpgroup then takes).
    if (tid == 0) {
      for (uint64_t* b = &s.k_full[0]; b < reinterpret_cast<uint64_t*>(&s.tk_slot[0]); ++b) mbar_inval(b);
    }
    if (warp >= 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLaunch));
    else asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsLaunch));
    __syncthreads();
  }
}

#ifndef LUCID_BODY_ONLY
template <bool kBf16, bool kReverse, bool kPair, bool kKT>
__global__ void __launch_bounds__(solve_threads(kSolveGroups), 1)
solve_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_in,
             const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_x,
             const __grid_constant__ CUtensorMap tm_st, const SolveArgs args) {
  solve_body<kBf16, kReverse, kSolveGroups, kPair, kKT>(tm_k, tm_in, tm_out, tm_x, tm_st, args);
}

// ---------------------------------------------------------------------------------------------
// host launcher
// ---------------------------------------------------------------------------------------------
size_t solve_smem_bytes() { return sizeof(SolveSmem) + 1024; }

template <bool kBf16, bool kReverse, bool kPair, bool kKT>
static cudaError_t launch_solve_t(const CUtensorMap& tm_k, const CUtensorMap& tm_in, const CUtensorMap& tm_out,
                                  const CUtensorMap& tm_x, const CUtensorMap& tm_st, const SolveArgs& args, int grid,
                                  cudaStream_t stream) {
  auto kern = solve_kernel<kBf16, kReverse, kPair, kKT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)solve_smem_bytes());
  if (e != cudaSuccess) return e;
  if (!kPair) {
    kern<<<grid, solve_threads(kSolveGroups), solve_smem_bytes(), stream>>>(tm_k, tm_in, tm_out, tm_x, tm_st, args);
    return cudaGetLastError();
  }
  // clusters of two CTAs (the two CTAs of a cluster wait for one another; clusters take pairs by ticket, so no
  // cluster waits for one that is not running); more clusters than fit the device at once would only idle
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(solve_threads(kSolveGroups));
  cfg.dynamicSmemBytes = solve_smem_bytes();
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int max_clusters = 0;
  e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
  if (e != cudaSuccess) return e;
  if (max_clusters < 1) return cudaErrorLaunchOutOfResources;
  if (grid > 2 * max_clusters) cfg.gridDim = dim3(2 * max_clusters);
  return cudaLaunchKernelEx(&cfg, kern, tm_k, tm_in, tm_out, tm_x, tm_st, args);
}

template <bool kBf16, bool kReverse>
static cudaError_t launch_solve_v(bool pair, bool kt, const CUtensorMap& tm_k, const CUtensorMap& tm_in,
                                  const CUtensorMap& tm_out, const CUtensorMap& tm_x, const CUtensorMap& tm_st,
                                  const SolveArgs& args, int grid, cudaStream_t stream) {
  if (pair)
    return kt ? launch_solve_t<kBf16, kReverse, true, true>(tm_k, tm_in, tm_out, tm_x, tm_st, args, grid, stream)
              : launch_solve_t<kBf16, kReverse, true, false>(tm_k, tm_in, tm_out, tm_x, tm_st, args, grid, stream);
  return kt ? launch_solve_t<kBf16, kReverse, false, true>(tm_k, tm_in, tm_out, tm_x, tm_st, args, grid, stream)
            : launch_solve_t<kBf16, kReverse, false, false>(tm_k, tm_in, tm_out, tm_x, tm_st, args, grid, stream);
}

cudaError_t launch_solve(bool bf16, bool reverse, bool pair, bool ki_in_tmem, const CUtensorMap& tm_k,
                         const CUtensorMap& tm_in, const CUtensorMap& tm_out, const CUtensorMap& tm_x,
                         const CUtensorMap& tm_st, const SolveArgs& args, int grid, cudaStream_t stream) {
#define LUCID_LAUNCH(BF, REV) \
  launch_solve_v<BF, REV>(pair, ki_in_tmem, tm_k, tm_in, tm_out, tm_x, tm_st, args, grid, stream)
  if (bf16) return reverse ? LUCID_LAUNCH(true, true) : LUCID_LAUNCH(true, false);
  return reverse ? LUCID_LAUNCH(false, true) : LUCID_LAUNCH(false, false);
#undef LUCID_LAUNCH
}
#endif  // LUCID_BODY_ONLY

}  // namespace lucid

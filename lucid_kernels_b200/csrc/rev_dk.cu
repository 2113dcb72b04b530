// Reverse solve dV = L^-T dV' that also accumulates the upper-triangle dK terms of the tiles it streams.
// Counterpart of Phase 1 of the reference's BackwardSubSm90 (lucid_kernels/cute/forward_sub_bwd.py:1113-1195,
// sub_one_n_block_dk: S, G, exp(S) once, acc_dV += P dV_j and acc_dK += dS K_j from the same tile).
//
// For row-block i of a chain and every later block j (visited from T-1 down to i+1):
//     S = K_i K_j^T,  P = exp(S)                     ACC_dV += P dV_j            (the solve, as in solve.cu)
//     G = V'_i dV_j^T,  W = -P o G                   ACC_dK += W K_j             (upper-triangle dK of row-block i)
// K_j and dV_j are streamed anyway and S and exp(S) are formed anyway, so the dK terms cost two more products
// per tile instead of the three (and a second exponential, and a second pass over K_j and dV_j) they cost in
// the stand-alone dK kernel.  The newest predecessor l = i+1 is the exception: dV_l arrives last, on the chain's
// critical path, and is folded in through Q = X_i^T P_l exactly as in solve.cu; its dK tile is left to the dK
// kernel, which then runs the lower part, the two diagonal tiles and that one upper tile per row-block
// (DkArgs::lower_only) and adds the fp32 sums this kernel leaves in the workspace.
//
// TMEM (512 columns): region B holds S (and, for the newest predecessor, Q), region A holds G and then the
// packed W and P of the same tile, then ACC_dV (reused for the diagonal product and the closing product) and
// ACC_dK.  There is no room for a second S or G buffer, so the registers of the exp groups are the second buffer:
// an exp thread pulls its 32 columns of S into registers as soon as S is complete and says so, which frees
// region B for the next tile's S while this tile's exponentials are still being formed; it pulls G likewise,
// and when all threads hold their G values (one named barrier) W and P are packed over region A.  One warp
// issues the products on region A in the order  G(q), W(q) K_j, P(q) dV_j, G(q+1), ...  - the tensor pipe executes
// one thread's products in order, so G(q+1) may be queued right behind the products that still read W(q) and
// P(q) - and an item's first S; another warp issues S(q+1) as soon as region B is free, which covers the time the
// exp groups need between G(q) and W(q).
//
// Shared memory: K_i (then P_l for the Q product), V'_i (then X_i, once the last G product is done), the
// right-hand side / staging tile, and two rings of two whole tiles (K_j; dV_j), each tile as two 64-column
// panels so that it serves as a K-major operand (S, G) and as an MN-major operand (P dV_j, W K_j).
//
// Warp roles (640 threads): warp 0 K producer (tickets, K_i, V'_i, K_j, X_i), warp 2 dV producer (right-hand
// side, flag waits, dV_j), warp 1 issues G, an item's first S and everything that reads P, W, Q or X, warp 3 issues
// the other S products, warps 4-19
// are four exp groups of 128 threads (one row each; group g forms k-steps g and 4+g of every tile and owns output
// columns 32g..32g+31).  K_j's last reader (W K_j) is issued before dV_j's (P dV_j), because K_j is the operand the
// next but one tile wants first (for its S).  Row-blocks are taken by ticket in dependency order; every wait is bounded.
#include <type_traits>
#include "kernels.h"

namespace lucid {

struct RevDkSmem {
  alignas(1024) uint8_t ki[kTileBytes];        // K_i: two 64-column panels; later P_l (rows = k of the Q product)
  alignas(1024) uint8_t vx[kTileBytes];        // V'_i, then X_i
  alignas(1024) uint8_t rhs[kTileBytes];       // dV'_i, then the right-hand side, then dV_i staged for the store
  alignas(1024) uint8_t kring[2][kTileBytes];  // K_j, tile g in stage g & 1
  alignas(1024) uint8_t vring[2][kTileBytes];  // dV_j
  alignas(8) uint64_t kt_full[2];
  uint64_t kt_empty[2], vt_full[2], vt_empty[2];
  uint64_t ki_full, ki_free, vpi_full, x_full, vx_free, g_done, vi_full, r_free, stage_full;
  uint64_t s_full, s_loaded, g_full, pw_full[2];
  uint64_t acc_full, acc_free, acck_full, acck_free, rhs_full, out_full, pq_full, q_full, p_full;
  uint64_t tk_full[2], tk_empty[2];
  int tk_slot[2];
  uint32_t tmem_base;
  int abort_flag;
};

enum RevDkBar : int {
  RD_KT_FULL = 301, RD_KT_EMPTY, RD_VT_FULL, RD_VT_EMPTY, RD_KI_FULL, RD_KI_FREE, RD_VPI_FULL, RD_X_FULL, RD_VX_FREE,
  RD_G_DONE, RD_VI_FULL, RD_R_FREE, RD_STAGE_FULL, RD_S_FULL, RD_S_LOADED, RD_G_FULL, RD_PW_FULL, RD_ACC_FULL, RD_ACC_FREE,
  RD_ACCK_FULL, RD_ACCK_FREE, RD_RHS_FULL, RD_OUT_FULL, RD_PQ_FULL, RD_Q_FULL, RD_P_FULL, RD_TK_FULL, RD_TK_EMPTY
};

constexpr int kRdThreads = 640;
constexpr int kRdExp = 512;
constexpr int kRdS = 0, kRdG = 128, kRdAcc = 256, kRdAccK = 384;   // region B (S, Q), region A (G, then W and P)
constexpr int kRdP = kRdG, kRdW = kRdG + 64;        // packed operands of a tile: k-step ks at +8 ks
constexpr int kRdRegsService = 64, kRdRegsExp = 104;

template <bool kBf16>
__global__ void __launch_bounds__(kRdThreads, 1)
revdk_kernel(const __grid_constant__ CUtensorMap tm_k,     // K,   box 64 x 128
             const __grid_constant__ CUtensorMap tm_dvp,   // dV', box 64 x 128
             const __grid_constant__ CUtensorMap tm_dv,    // dV,  box 64 x 128 (loads and the store)
             const __grid_constant__ CUtensorMap tm_vp,    // V',  box 64 x 128
             const __grid_constant__ CUtensorMap tm_x,     // X workspace (2D), box 64 x 128
             const RevDkArgs args) {
  extern __shared__ uint8_t smem_raw[];
  RevDkSmem& s = *reinterpret_cast<RevDkSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const Problem& P = args.p;
  Control* ctl = args.ctl;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = P.T, H = P.H;
  const unsigned long long limit = P.wait_ns;
  volatile int* cta_abort = &s.abort_flag;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.kt_full[i], 1);
      mbar_init(&s.kt_empty[i], 1);
      mbar_init(&s.vt_full[i], 1);
      mbar_init(&s.vt_empty[i], 1);
      mbar_init(&s.pw_full[i], kRdExp);
      mbar_init(&s.tk_full[i], 1);
      mbar_init(&s.tk_empty[i], 3 + 16);
    }
    mbar_init(&s.ki_full, 1);
    mbar_init(&s.ki_free, 1);
    mbar_init(&s.vpi_full, 1);
    mbar_init(&s.x_full, 1);
    mbar_init(&s.vx_free, 1);
    mbar_init(&s.g_done, 1);
    mbar_init(&s.vi_full, 1);
    mbar_init(&s.r_free, 1);
    mbar_init(&s.stage_full, kRdExp);
    mbar_init(&s.s_full, 1);
    mbar_init(&s.s_loaded, kRdExp);
    mbar_init(&s.g_full, 1);
    mbar_init(&s.acc_full, 1);
    mbar_init(&s.acc_free, kRdExp);
    mbar_init(&s.acck_full, 1);
    mbar_init(&s.acck_free, kRdExp);
    mbar_init(&s.rhs_full, kRdExp);
    mbar_init(&s.out_full, 1);
    mbar_init(&s.pq_full, kRdExp);
    mbar_init(&s.q_full, 1);
    mbar_init(&s.p_full, kRdExp);
    s.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s.tmem_base;

  // Item = row-block i = T-1-step of a chain; tiles q = 0 .. n-1 are the blocks j = T-1-q (n = step).  Tiles
  // q < n-1 are "full" tiles (solve and dK terms); tile n-1 is the newest predecessor (solve only, through Q).
  // Counters per CTA: `it` items, `g` tiles (ring stage g & 1, S/G phase g & 1), `gf` full tiles (pw_full phase).
  auto item_geometry = [&](int ticket, int& chain, int& i, int& n) -> bool {
    int step;
    if (!decode_ticket(ticket, P.C, T, P.group, P.head, P.overlap, chain, step)) return false;
    i = T - 1 - step;
    n = step;
    return true;
  };

  if (warp == 0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRdRegsService));
    // =========================== K producer (one lane) ===========================
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_vp);
      tma_prefetch_desc(&tm_x);
      uint32_t g = 0, ng = 0;      // tiles loaded; items that had G products (phase of g_done)
      bool alive = true;
      int trc = 0;
      (void)trc;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_empty[slot], ((it >> 1) & 1) ^ 1, cta_abort, ctl, limit, -1, -1, RD_TK_EMPTY)) break;
        const int ticket = atomicAdd(&ctl->ticket, 1);
        s.tk_slot[slot] = ticket;
        mbar_arrive(&s.tk_full[slot]);
        int chain, i, n;
        if (!item_geometry(ticket, chain, i, n)) break;
        const int b = chain / H, h = chain % H;
        if (!wait_barrier(&s.ki_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, RD_KI_FREE)) break;
        mbar_expect_tx(&s.ki_full, kTileBytes);
        tma_load_4d(s.ki, &tm_k, &s.ki_full, 0, i * kBlock, h, b);
        tma_load_4d(s.ki + kHalfBytes, &tm_k, &s.ki_full, 64, i * kBlock, h, b);
        // the V'_i / X_i buffer: free once the previous item's diagonal products have read X
        if (!wait_barrier(&s.vx_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, RD_VX_FREE)) break;
        const bool has_g = n >= 2;
        if (has_g) {
          mbar_expect_tx(&s.vpi_full, kTileBytes);
          tma_load_4d(s.vx, &tm_vp, &s.vpi_full, 0, i * kBlock, h, b);
          tma_load_4d(s.vx + kHalfBytes, &tm_vp, &s.vpi_full, 64, i * kBlock, h, b);
        }
        for (int q = 0; q < n; ++q, ++g) {
          const int j = T - 1 - q;
          const int st = g & 1;
          if (!wait_barrier(&s.kt_empty[st], ((g >> 1) & 1) ^ 1, cta_abort, ctl, limit, chain, i, RD_KT_EMPTY)) {
            alive = false;
            break;
          }
          LUCID_TR(args.trace, 0, trc, 41, g);
          mbar_expect_tx(&s.kt_full[st], kTileBytes);
          tma_load_4d(s.kring[st], &tm_k, &s.kt_full[st], 0, j * kBlock, h, b);
          tma_load_4d(s.kring[st] + kHalfBytes, &tm_k, &s.kt_full[st], 64, j * kBlock, h, b);
        }
        if (!alive) break;
        // X_i replaces V'_i once the item's last G product has completed
        if (has_g) {
          if (!wait_barrier(&s.g_done, ng & 1, cta_abort, ctl, limit, chain, i, RD_G_DONE)) break;
          ++ng;
        }
        mbar_expect_tx(&s.x_full, kTileBytes);
        tma_load_2d(s.vx, &tm_x, &s.x_full, 0, (chain * T + i) * kBlock);
        tma_load_2d(s.vx + kHalfBytes, &tm_x, &s.x_full, 64, (chain * T + i) * kBlock);
      }
    }
  } else if (warp == 2) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRdRegsService));
    // =========================== dV producer (one lane) ===========================
    if (lane == 0) {
      tma_prefetch_desc(&tm_dvp);
      tma_prefetch_desc(&tm_dv);
      uint32_t g = 0;
      bool alive = true;
      int trc = 0;
      (void)trc;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, RD_TK_FULL)) break;
        const int ticket = s.tk_slot[slot];
        mbar_arrive(&s.tk_empty[slot]);
        int chain, i, n;
        if (!item_geometry(ticket, chain, i, n)) break;
        const int b = chain / H, h = chain % H;
        bool vi_loaded = false;
        auto load_vi = [&]() {
          mbar_expect_tx(&s.vi_full, kTileBytes);
          tma_load_4d(s.rhs, &tm_dvp, &s.vi_full, 0, i * kBlock, h, b);
          tma_load_4d(s.rhs + kHalfBytes, &tm_dvp, &s.vi_full, 64, i * kBlock, h, b);
          vi_loaded = true;
        };
        // A row-block publishes itself only after it has acquired the flags of all its predecessors, so one
        // flag that is up vouches for every block published before it: one look at the block kFlagProbe steps
        // behind the newest predecessor usually spares the older tiles their flag round trip (an L2 round trip
        // in series with every tile load otherwise).
        const int skip_until = flags_known_up(args.flags + chain * T, n, T - 1 - (n - kFlagProbe));
        for (int q = 0; q < n; ++q, ++g) {
          const int j = T - 1 - q;
          if (!vi_loaded && mbar_try_wait(&s.r_free, (it & 1) ^ 1)) load_vi();
          const int st = g & 1;
          if (!wait_barrier(&s.vt_empty[st], ((g >> 1) & 1) ^ 1, cta_abort, ctl, limit, chain, i, RD_VT_EMPTY)) {
            alive = false;
            break;
          }
          LUCID_TR(args.trace, 1, trc, 30, g);
          if (q >= skip_until) {
            if (!wait_flag(args.flags + chain * T + j, cta_abort, ctl, limit, chain, i, j, nullptr)) {
              alive = false;
              break;
            }
            fence_proxy_async_all();   // flag acquired in the generic proxy; the tile is read by TMA
          }
          LUCID_TR(args.trace, 1, trc, 32, g);
          mbar_expect_tx(&s.vt_full[st], kTileBytes);
          tma_load_4d(s.vring[st], &tm_dv, &s.vt_full[st], 0, j * kBlock, h, b);
          tma_load_4d(s.vring[st] + kHalfBytes, &tm_dv, &s.vt_full[st], 64, j * kBlock, h, b);
        }
        if (!alive) break;
        if (!vi_loaded) {
          if (!wait_barrier(&s.r_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, RD_R_FREE)) break;
          load_vi();
        }
      }
    }
  } else if (warp == 1) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRdRegsService));
    // =========================== the issuer of all products but S(1), S(2), ... ===========================
    // Program order per tile: G, then (as the exp groups deliver them) the products that read W and P; the next
    // tile's G follows at once.  The tensor pipe runs one thread's products in order, so the G columns are never
    // overwritten before the products that read W and P there have done so.
    {
      constexpr int fmt = kBf16 ? 1 : 0;
      constexpr uint32_t idesc_kk = umma_idesc(fmt, 0, 0, 128, 128);    // both operands K-major
      constexpr uint32_t idesc_tb = umma_idesc(fmt, 0, 1, 128, 128);    // A from TMEM, B with rows = k
      constexpr uint32_t idesc_xt = umma_idesc(fmt, 1, 1, 128, 128);    // A = X^T (X read with rows = k), B rows = k
      const uint64_t d_ki = umma_smem_desc(smem_u32(s.ki), 16, 1024);
      const uint64_t d_vpi = umma_smem_desc(smem_u32(s.vx), 16, 1024);
      const uint64_t d_kr0 = umma_smem_desc(smem_u32(s.kring[0]), 16, 1024);     // stage: + 32 KiB
      const uint64_t d_vr0 = umma_smem_desc(smem_u32(s.vring[0]), 16, 1024);
      const uint64_t d_x = umma_smem_desc(smem_u32(s.vx), kHalfBytes, 1024);
      const uint64_t d_rhs = umma_smem_desc(smem_u32(s.rhs), kHalfBytes, 1024);
      const uint64_t d_pl = umma_smem_desc(smem_u32(s.ki), kHalfBytes, 1024);
      const uint64_t d_kr0_mn = umma_smem_desc(smem_u32(s.kring[0]), kHalfBytes, 1024);   // rows = k
      const uint64_t d_vr0_mn = umma_smem_desc(smem_u32(s.vring[0]), kHalfBytes, 1024);
      uint32_t g = 0, gf = 0, ng = 0, nq = 0;
      bool alive = true;
      int trc = 0;
      (void)trc;
      const bool leader = lane == 0;
      (void)leader;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, RD_TK_FULL)) break;
        const int ticket = s.tk_slot[slot];
        __syncwarp();
        mbar_arrive_w(&s.tk_empty[slot]);
        int chain, i, n;
        if (!item_geometry(ticket, chain, i, n)) break;
        if (!wait_barrier(&s.ki_full, it & 1, cta_abort, ctl, limit, chain, i, RD_KI_FULL)) break;
        const bool has_g = n >= 2;
        if (has_g) {
          if (!wait_barrier(&s.vpi_full, ng & 1, cta_abort, ctl, limit, chain, i, RD_VPI_FULL)) break;
          ++ng;
        }
        tc_fence_after_sync();
        // S of a tile into region B (the exp groups hold the S of the tile before in registers)
        auto issue_s = [&](uint32_t gt) -> bool {
          const uint32_t st = gt & 1;
          if (!wait_barrier(&s.kt_full[st], (gt >> 1) & 1, cta_abort, ctl, limit, chain, i, RD_KT_FULL)) return false;
          tc_fence_after_sync();
          if (leader) LUCID_TR(args.trace, 2, trc, 18, gt);
          const uint64_t dbk = d_kr0 + st * (kTileBytes >> 4);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
            umma_ss_w(tmem + kRdS, d_ki + off, dbk + off, idesc_kk, k ? 1u : 0u);
#ifdef LUCID_TRACE_MMA
            if (leader) LUCID_TR(args.trace, 2, trc, 50 + k, gt);
#endif
          }
          umma_commit_w(&s.s_full);
          if (leader) LUCID_TR(args.trace, 2, trc, 12, gt);
          return true;
        };
        if (n >= 1) {
          if (!issue_s(g)) break;
          if (n == 1) umma_commit_w(&s.kt_empty[g & 1]);     // the newest predecessor's K_j has no other reader
        }
        for (int q = 0; q + 1 < n; ++q, ++g) {
          const uint32_t st = g & 1;
          // ---- G(q) into region A (its previous readers, the products of the tile before, were issued above) ----
          if (leader) LUCID_TR(args.trace, 2, trc, 9, g);
          if (!wait_barrier(&s.vt_full[st], (g >> 1) & 1, cta_abort, ctl, limit, chain, i, RD_VT_FULL)) { alive = false; break; }
          tc_fence_after_sync();
          if (leader) LUCID_TR(args.trace, 2, trc, 17, g);
          const uint64_t dbv = d_vr0 + st * (kTileBytes >> 4);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
            umma_ss_w(tmem + kRdG, d_vpi + off, dbv + off, idesc_kk, k ? 1u : 0u);
#ifdef LUCID_TRACE_MMA
            if (leader) LUCID_TR(args.trace, 2, trc, 60 + k, g);
#endif
          }
          umma_commit_w(&s.g_full);
          if (leader) LUCID_TR(args.trace, 2, trc, 10, g);
          if (q == n - 2) umma_commit_w(&s.g_done);      // V'_i is no longer needed: X_i may take its buffer
          // (S(q+1) is issued by the other issuing warp as soon as every exp thread has S(q) in registers)
          // ---- ACC_dK += W K_j, then ACC_dV += P dV_j ----
          const uint64_t dbv_mn = d_vr0_mn + st * (kTileBytes >> 4);
          const uint64_t dbk_mn = d_kr0_mn + st * (kTileBytes >> 4);
          if (q == 0) {
            // the accumulators of the item before have been read out
            if (!wait_barrier(&s.acc_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, RD_ACC_FREE) ||
                !wait_barrier(&s.acck_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, RD_ACCK_FREE)) {
              alive = false;
              break;
            }
          }
          if (!wait_barrier(&s.pw_full[0], gf & 1, cta_abort, ctl, limit, chain, i, RD_PW_FULL)) { alive = false; break; }
          // K_j: its S product (from the other warp for q > 0) is long complete, so this wait is over at once; it
          // is made because this warp's products read the tile too
          if (!wait_barrier(&s.kt_full[st], (g >> 1) & 1, cta_abort, ctl, limit, chain, i, RD_KT_FULL)) { alive = false; break; }
          tc_fence_after_sync();
          if (leader) LUCID_TR(args.trace, 2, trc, 13, g);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ts_w(tmem + kRdAccK, tmem + kRdW + 8 * ks, dbk_mn + ks * (2048 >> 4), idesc_tb, (q | ks) ? 1u : 0u);
          umma_commit_w(&s.kt_empty[st]);
          if (leader) LUCID_TR(args.trace, 2, trc, 14, g);
          if (!wait_barrier(&s.pw_full[1], gf & 1, cta_abort, ctl, limit, chain, i, RD_PW_FULL)) { alive = false; break; }
          tc_fence_after_sync();
          if (leader) LUCID_TR(args.trace, 2, trc, 15, g);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ts_w(tmem + kRdAcc, tmem + kRdP + 8 * ks, dbv_mn + ks * (2048 >> 4), idesc_tb, (q | ks) ? 1u : 0u);
          umma_commit_w(&s.vt_empty[st]);
          if (leader) LUCID_TR(args.trace, 2, trc, 16, g);
          ++gf;
        }
        if (!alive) break;
        if (n < 2) {
          // no full tile: nothing was accumulated, but the previous item's readers must be done before the
          // diagonal product below writes over ACC_dV
          if (!wait_barrier(&s.acc_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, RD_ACC_FREE) ||
              !wait_barrier(&s.acck_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, RD_ACCK_FREE))
            break;
        }
        umma_commit_w(&s.acc_full);
        umma_commit_w(&s.acck_full);
        const uint32_t st_l = g & 1;               // ring stage of the newest predecessor (n >= 1)
        if (n >= 1) {
          // Q = X^T P_l into the S columns (every exp thread has read S_l and put P_l into shared memory)
          if (!wait_barrier(&s.pq_full, nq & 1, cta_abort, ctl, limit, chain, i, RD_PQ_FULL)) break;
          if (!wait_barrier(&s.x_full, it & 1, cta_abort, ctl, limit, chain, i, RD_X_FULL)) break;
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_ss_w(tmem + kRdS, desc_advance(d_x, k * 2048), desc_advance(d_pl, k * 2048), idesc_xt, k ? 1u : 0u);
          umma_commit_w(&s.q_full);
          umma_commit_w(&s.ki_free);
        } else {
          mbar_arrive_w(&s.ki_free);
        }
        // diagonal step: OUT = X^T rhs over ACC_dV
        if (!wait_barrier(&s.rhs_full, it & 1, cta_abort, ctl, limit, chain, i, RD_RHS_FULL)) break;
        if (!wait_barrier(&s.x_full, it & 1, cta_abort, ctl, limit, chain, i, RD_X_FULL)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss_w(tmem + kRdAcc, desc_advance(d_x, k * 2048), desc_advance(d_rhs, k * 2048), idesc_xt, k ? 1u : 0u);
        umma_commit_w(&s.vx_free);
        if (n >= 1) {
          // OUT += (-Q) dV_l: the only product that waits for the newest predecessor
          if (!wait_barrier(&s.p_full, nq & 1, cta_abort, ctl, limit, chain, i, RD_P_FULL)) break;
          if (!wait_barrier(&s.vt_full[st_l], (g >> 1) & 1, cta_abort, ctl, limit, chain, i, RD_VT_FULL)) break;
          tc_fence_after_sync();
          const uint64_t dbv_mn = d_vr0_mn + st_l * (kTileBytes >> 4);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ts_w(tmem + kRdAcc, tmem + kRdS + 16 * ks, dbv_mn + ks * (2048 >> 4), idesc_tb, 1u);
          umma_commit_w(&s.vt_empty[st_l]);
          ++nq;
          ++g;
        }
        umma_commit_w(&s.out_full);
      }
    }
  } else if (warp == 3) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRdRegsService));
    // =========================== the issuer of S(1), S(2), ... of every item ===========================
    // S(q+1) needs K_j in shared memory and region B, which is free as soon as every exp thread holds S(q) in
    // registers; nothing else.  Issued from the other warp it stood, with its waits, in the middle of the chain
    // G(q) -> W(q), P(q) -> their products -> G(q+1) that bounds a tile, and the tensor pipe runs two warps'
    // products closer together than one warp's.  The FIRST S of an item stays with the other warp, behind the
    // closing product of the item before in that warp's program order: that product reads -Q from region B, and
    // this way no barrier has to say across warps that it is done.  This warp touches region B only between
    // s_loaded of a tile and s_full of the next, when the other warp has no product on it; it waits for every
    // s_loaded phase and for the ticket of every item, so no barrier it reads can run two phases ahead of it.
    {
      constexpr int fmt = kBf16 ? 1 : 0;
      constexpr uint32_t idesc_kk = umma_idesc(fmt, 0, 0, 128, 128);
      const uint64_t d_ki = umma_smem_desc(smem_u32(s.ki), 16, 1024);
      const uint64_t d_kr0 = umma_smem_desc(smem_u32(s.kring[0]), 16, 1024);     // stage: + 32 KiB
      uint32_t g0 = 0, gf = 0;       // tiles and full tiles of the items before (as counted by the other roles)
      bool alive = true;
      int trc = 0;
      (void)trc;
      const bool leader = lane == 0;
      (void)leader;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, RD_TK_FULL)) break;
        const int ticket = s.tk_slot[slot];
        __syncwarp();
        mbar_arrive_w(&s.tk_empty[slot]);
        int chain, i, n;
        if (!item_geometry(ticket, chain, i, n)) break;
        for (int q = 1; q < n; ++q, ++gf) {
          // every exp thread holds S(q-1), a full tile (q - 1 <= n - 2); K_i is in place (S(0) has used it)
          if (!wait_barrier(&s.s_loaded, gf & 1, cta_abort, ctl, limit, chain, i, RD_S_LOADED)) { alive = false; break; }
          const uint32_t gt = g0 + q;
          const uint32_t st = gt & 1;
          if (!wait_barrier(&s.kt_full[st], (gt >> 1) & 1, cta_abort, ctl, limit, chain, i, RD_KT_FULL)) { alive = false; break; }
          tc_fence_after_sync();
          if (leader) LUCID_TR(args.trace, 5, trc, 18, gt);
          const uint64_t dbk = d_kr0 + st * (kTileBytes >> 4);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
            umma_ss_w(tmem + kRdS, d_ki + off, dbk + off, idesc_kk, k ? 1u : 0u);
          }
          umma_commit_w(&s.s_full);
          if (q == n - 1) umma_commit_w(&s.kt_empty[st]);     // the newest predecessor: S_l is K_l's only reader
          if (leader) LUCID_TR(args.trace, 5, trc, 12, gt);
        }
        g0 += n;
      }
    }
  } else if (warp >= 4) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRdRegsExp));
    // =========================== exp groups + epilogue ===========================
    const int wg = (warp - 4) >> 2;                  // group: k-steps wg and 4 + wg; output columns 32 wg ..
    const float xs = P.exp_scale;
    const int row = ((warp & 3) << 5) + lane;        // TMEM lane == row of the block
    const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    uint8_t* const my_rhs = s.rhs + (wg >> 1) * kHalfBytes;            // output columns 32 wg ..: panel and first vector
    const uint32_t vec0 = (wg & 1) * 4;
    uint32_t g = 0, gf = 0, nq = 0;
    bool alive = true;
    int trc = 0;
    (void)trc;
    const bool tr_lead = tid == 128;
    (void)tr_lead;
    typedef typename std::conditional<kBf16, __nv_bfloat16, __half>::type elem_t;
    for (int it = 0; alive; ++it) {
      const int slot = it & 1;
      if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, RD_TK_FULL)) break;
      const int ticket = s.tk_slot[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.tk_empty[slot]);
      int chain, i, n;
      if (!item_geometry(ticket, chain, i, n)) break;
      const int b = chain / H, h = chain % H;
      const float lam = args.lam_inv[(chain * T + i) * kBlock + row];

      // ---- full tiles: P = exp(S), W = -P o G for k-steps wg and 4 + wg (columns 16 wg .. and 64 + 16 wg ..) ----
      for (int q = 0; q + 1 < n; ++q, ++g, ++gf) {
        if (tr_lead) LUCID_TR(args.trace, 3, trc, 19, g);
        if (!wait_barrier(&s.s_full, g & 1, cta_abort, ctl, limit, chain, i, RD_S_FULL)) { alive = false; break; }
        tc_fence_after_sync();
        if (tr_lead) LUCID_TR(args.trace, 3, trc, 20, g);
        uint32_t sv[32], gv[32];
        tmem_ld16(lane_base + kRdS + 16 * wg, *reinterpret_cast<uint32_t(*)[16]>(&sv[0]));
        tmem_ld16(lane_base + kRdS + 64 + 16 * wg, *reinterpret_cast<uint32_t(*)[16]>(&sv[16]));
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(&s.s_loaded);            // region B may take the next tile's S
        if (tr_lead) LUCID_TR(args.trace, 3, trc, 21, g);
        float ev[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) ev[e] = ex2_approx(__uint_as_float(sv[e]) * xs);
        if (tr_lead) LUCID_TR(args.trace, 3, trc, 22, g);
        if (!wait_barrier(&s.g_full, gf & 1, cta_abort, ctl, limit, chain, i, RD_G_FULL)) { alive = false; break; }
        tc_fence_after_sync();
        if (tr_lead) LUCID_TR(args.trace, 3, trc, 23, g);
        tmem_ld16(lane_base + kRdG + 16 * wg, *reinterpret_cast<uint32_t(*)[16]>(&gv[0]));
        tmem_ld16(lane_base + kRdG + 64 + 16 * wg, *reinterpret_cast<uint32_t(*)[16]>(&gv[16]));
        tmem_wait_ld();
        // W and P are packed over G's columns, other threads' included: everybody holds its G values first
        if (tr_lead) LUCID_TR(args.trace, 3, trc, 24, g);
        named_bar_sync(2, kRdExp);
        if (tr_lead) LUCID_TR(args.trace, 3, trc, 25, g);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t wk[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            wk[e] = pack2_fast<kBf16>(-ev[16 * c + 2 * e] * __uint_as_float(gv[16 * c + 2 * e]),
                                      -ev[16 * c + 2 * e + 1] * __uint_as_float(gv[16 * c + 2 * e + 1]));
          tmem_st8(lane_base + kRdW + 8 * (4 * c + wg), wk);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&s.pw_full[0]);
        if (tr_lead) LUCID_TR(args.trace, 3, trc, 26, g);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) pk[e] = pack2_fast<kBf16>(ev[16 * c + 2 * e], ev[16 * c + 2 * e + 1]);
          tmem_st8(lane_base + kRdP + 8 * (4 * c + wg), pk);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&s.pw_full[1]);
        if (tr_lead) LUCID_TR(args.trace, 3, trc, 27, g);
      }
      if (!alive) break;

      // ---- the newest predecessor: P_l to shared memory, Q back through the S columns ----
      if (n >= 1) {
        if (!wait_barrier(&s.s_full, g & 1, cta_abort, ctl, limit, chain, i, RD_S_FULL)) break;
        tc_fence_after_sync();
        uint32_t v[32];
        tmem_ld16(lane_base + kRdS + 16 * wg, *reinterpret_cast<uint32_t(*)[16]>(&v[0]));
        tmem_ld16(lane_base + kRdS + 64 + 16 * wg, *reinterpret_cast<uint32_t(*)[16]>(&v[16]));
        tmem_wait_ld();
        // P_l in the layout of the right-hand-side tile (rows = this block's rows), written over K_i: s_full of
        // the last tile implies that every S product of the item has completed
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint8_t* panel = s.ki + c * kHalfBytes;           // columns 16 wg .. of panel c
#pragma unroll
          for (int vv = 0; vv < 2; ++vv) {
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float e0 = ex2_approx(__uint_as_float(v[16 * c + 8 * vv + 2 * e]) * xs);
              const float e1 = ex2_approx(__uint_as_float(v[16 * c + 8 * vv + 2 * e + 1]) * xs);
              o[e] = pack2_fast<kBf16>(e0, e1);
            }
            *reinterpret_cast<uint4*>(panel + sw128_off(row, 2 * wg + vv)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(&s.pq_full);
        if (!wait_barrier(&s.q_full, nq & 1, cta_abort, ctl, limit, chain, i, RD_Q_FULL)) break;
        tc_fence_after_sync();
        tmem_ld16(lane_base + kRdS + 16 * wg, *reinterpret_cast<uint32_t(*)[16]>(&v[0]));
        tmem_ld16(lane_base + kRdS + 64 + 16 * wg, *reinterpret_cast<uint32_t(*)[16]>(&v[16]));
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            pk[e] = pack2<kBf16>(-__uint_as_float(v[16 * c + 2 * e]), -__uint_as_float(v[16 * c + 2 * e + 1]));
          tmem_st8(lane_base + kRdS + 16 * (4 * c + wg), pk);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&s.p_full);
        ++nq;
        ++g;
      }

      // ---- epilogue, part 1: rhs = dV'_i - ACC_dV, this group's 32 output columns ----
      if (!wait_barrier(&s.vi_full, it & 1, cta_abort, ctl, limit, chain, i, RD_VI_FULL)) break;
      uint4 vin[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) vin[c] = *reinterpret_cast<const uint4*>(my_rhs + sw128_off(row, vec0 + c));
      uint32_t acc[32];
      if (!wait_barrier(&s.acc_full, it & 1, cta_abort, ctl, limit, chain, i, RD_ACC_FULL)) break;
      if (n >= 2) {
        tc_fence_after_sync();
        tmem_ld32(lane_base + kRdAcc + wg * 32, acc);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[e] = 0u;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t in[4] = {vin[c].x, vin[c].y, vin[c].z, vin[c].w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack2<kBf16>(in[e]);
          o[e] = pack2<kBf16>(f.x - __uint_as_float(acc[c * 8 + 2 * e]), f.y - __uint_as_float(acc[c * 8 + 2 * e + 1]));
        }
        *reinterpret_cast<uint4*>(my_rhs + sw128_off(row, vec0 + c)) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&s.rhs_full);

      // ---- epilogue, part 2: dV_i = lam * (X^T rhs - Q dV_l), staged, stored, published ----
      if (!wait_barrier(&s.out_full, it & 1, cta_abort, ctl, limit, chain, i, RD_OUT_FULL)) break;
      tc_fence_after_sync();
      tmem_ld32(lane_base + kRdAcc + wg * 32, acc);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(&s.acc_free);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          o[e] = pack2<kBf16>(__uint_as_float(acc[c * 8 + 2 * e]) * lam, __uint_as_float(acc[c * 8 + 2 * e + 1]) * lam);
        *reinterpret_cast<uint4*>(my_rhs + sw128_off(row, vec0 + c)) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      fence_proxy_async_smem();
      mbar_arrive(&s.stage_full);
      if (tid == 128) {
        if (!wait_barrier(&s.stage_full, it & 1, cta_abort, ctl, limit, chain, i, RD_STAGE_FULL)) break;
        tma_store_4d(&tm_dv, s.rhs, 0, i * kBlock, h, b);
        tma_store_4d(&tm_dv, s.rhs + kHalfBytes, 64, i * kBlock, h, b);
        tma_store_commit();
        tma_store_wait_read();
        mbar_arrive(&s.r_free);          // the next row-block's right-hand side may be loaded
        tma_store_wait_all();
        fence_proxy_async_all();
        st_release_gpu(args.flags + chain * T + i, kFlagComplete);
      }

      // ---- the upper-triangle dK sums of this row-block (tiles j >= i + 2), fp32, to the workspace ----
      if (!wait_barrier(&s.acck_full, it & 1, cta_abort, ctl, limit, chain, i, RD_ACCK_FULL)) break;
      float* up = args.upper + ((long long)(chain * T + i) * kBlock + row) * kBlock + wg * 32;
      if (n >= 2) {
        tc_fence_after_sync();
        tmem_ld32(lane_base + kRdAccK + wg * 32, acc);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[e] = 0u;
      }
      tc_fence_before_sync();
      mbar_arrive(&s.acck_free);
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(up + c * 4) = make_uint4(acc[c * 4], acc[c * 4 + 1], acc[c * 4 + 2], acc[c * 4 + 3]);
    }
  }

  // teardown: everybody meets here, also after an abort
  if (s.abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    if (tid == 0) report_error(ctl, kErrAborted, -1, -1, blockIdx.x, 0);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

size_t revdk_smem_bytes() { return sizeof(RevDkSmem) + 1024; }

cudaError_t launch_revdk(bool bf16, const CUtensorMap& tm_k, const CUtensorMap& tm_dvp, const CUtensorMap& tm_dv,
                         const CUtensorMap& tm_vp, const CUtensorMap& tm_x, const RevDkArgs& args, int grid,
                         cudaStream_t stream) {
  cudaError_t e;
  if (bf16) {
    e = cudaFuncSetAttribute(revdk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)revdk_smem_bytes());
    if (e != cudaSuccess) return e;
    revdk_kernel<true><<<grid, kRdThreads, revdk_smem_bytes(), stream>>>(tm_k, tm_dvp, tm_dv, tm_vp, tm_x, args);
  } else {
    e = cudaFuncSetAttribute(revdk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)revdk_smem_bytes());
    if (e != cudaSuccess) return e;
    revdk_kernel<false><<<grid, kRdThreads, revdk_smem_bytes(), stream>>>(tm_k, tm_dvp, tm_dv, tm_vp, tm_x, args);
  }
  return cudaGetLastError();
}

}  // namespace lucid

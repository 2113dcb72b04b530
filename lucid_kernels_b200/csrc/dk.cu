// dK of the LUCID block-triangular solve on sm_100a.  Replaces the dK half of the reference's
// BackwardSubSm90 (lucid_kernels/cute/forward_sub_bwd.py:1113-1269, Phase 1 upper-triangle and Phase 2
// lower-triangle accumulation) and the host-side diagonal term _add_diagonal_dk_correction
// (lucid_kernels/cute/forward_sub_interface.py:381-405), which here runs on the device in the same loop.
//
// With E_ij = exp(K_i K_j^T) and dV already solved,
//     dK_i = sum_{j<i} W_ij K_j + sum_{j>i} W_ij K_j + (D1 + D2) K_i
//     W_ij = -(dV_i V'_j^T) o E_ij   (j < i)          W_ij = -(V'_i dV_j^T) o E_ij   (j > i)
//     D1   = tril(-(dV_i V'_i^T) o E_ii)               D2   = triu(-(V'_i dV_i^T) o E_ii) = D1^T
// so every term is "S = K_i K_j^T, G = A_i Z_j^T, W = -exp(S) o G (masked on the diagonal), ACC += W K_j"
// with (A, Z) = (dV, V') for the lower part and (V', dV) for the upper part.  Row-blocks are independent:
// no flags, no ordering; a CTA owns row-block i and streams all T blocks j past it (T + 1 tiles).
//
// Warp roles (384 threads): warp 0 producer (tickets, K_i, A_i, K_j ring of 3, Z_j ring of 2), warps 1, 2
// and 3 issue the G, S and W*K_j products (one warp per product stream: an issuing thread runs only a
// few MMAs ahead of the tensor pipe, so a warp that issued two streams would delay the second behind
// the first), warp 1 owns TMEM, warps 4-11 form W: both groups work on the same tile, 64 columns each.
//
// A W-forming thread first pulls its 64 columns of G(q) into registers and releases the single G buffer
// at once, so that the product G(q+1) runs while W(q) is being formed; it then streams S(q) through in
// 16-column chunks (the next chunk's TMEM load in flight under the current chunk's arithmetic), forming
// w = -exp(s) * g in one pass, and writes the packed chunk over S columns it has already consumed.
// S(q+1) reuses the buffer W(q-1) sat in and is issued as soon as that product has completed.
//
// With args.lower_only an item ends after the first upper tile (j = i + 1): the remaining upper tiles were
// accumulated, unscaled and in fp32, by the reverse solve that also streams their operands (rev_dk.cu), and the
// epilogue adds those sums.
//
// Work items: a whole row-block, or (args.split, used by the one-launch backward with one or two chains,
// where the launch would otherwise end in units of a whole row-block) half of its tiles; the two halves
// meet in the epilogue through fp32 sums in the workspace.
#include <type_traits>
#include "kernels.h"

namespace lucid {

struct DkSmem {
  alignas(1024) uint8_t ki[kTileBytes];        // K_i
  alignas(1024) uint8_t ai[kTileBytes];        // dV_i for the lower part, then V'_i for the upper part
  alignas(1024) uint8_t kring[3][kTileBytes];  // K_j
  alignas(1024) uint8_t zring[2][kTileBytes];  // V'_j (lower) or dV_j (upper)
  alignas(8) uint64_t k_full[3];
  uint64_t k_empty[3], z_full[2], z_empty[2];
  uint64_t ki_full, ki_free, ai_full, ai_free;
  uint64_t s_full[2], g_full, g_free, w_ready[2], sbuf_free[2];
  uint64_t acc_full, acc_free;
  uint64_t tk_full[2], tk_empty[2];
  int tk_slot[2];
  uint32_t tmem_base;
  int abort_flag;
  int claim;       // split items: 0 = this CTA finished its half of the row-block first, 1 = second
};

enum DkBar : int {
  DK_K_FULL = 201, DK_K_EMPTY, DK_Z_FULL, DK_Z_EMPTY, DK_KI_FULL, DK_KI_FREE, DK_AI_FULL, DK_AI_FREE, DK_S_FULL,
  DK_G_FULL, DK_G_FREE, DK_ACC_FULL, DK_ACC_FREE, DK_TK_FULL, DK_TK_EMPTY, DK_SBUF_FREE, DK_W_READY
};

constexpr int kDkThreads = 384;
constexpr int kDkS0 = 0, kDkS1 = 128, kDkG = 256, kDkAcc = 384;

// The whole CTA program, callable from more than one kernel (the tensor maps must be __grid_constant__
// parameters of the calling kernel).  With args.follow_flags set, the CTA runs beside the reverse solve in
// the same launch: row-blocks are taken from the last one downwards, step-major over the chains, and each
// waits (bounded) for the flag with which the solve publishes dV_i - dV_j of every later block has then
// been published as well, and dK_i needs nothing else of the solve.
template <bool kBf16>
__device__ __forceinline__ void dk_body(const CUtensorMap& tm_k,    // K,   box 64 x 128
                                        const CUtensorMap& tm_vp,   // V',  box 64 x 128
                                        const CUtensorMap& tm_dv,   // dV,  box 64 x 128
                                        const DkArgs& args) {
  extern __shared__ uint8_t smem_raw[];
  DkSmem& s = *reinterpret_cast<DkSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const Problem& P = args.p;
  Control* ctl = args.ctl;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = P.T, H = P.H;
  const unsigned long long limit = P.wait_ns;
  volatile int* cta_abort = &s.abort_flag;
  // With identity diagonal blocks (use_diag == 0) the operator has no diagonal-block dependence on K.
  const bool diag_tiles = P.use_diag != 0;

  if (tid == 0) {
    for (int i = 0; i < 3; ++i) {
      mbar_init(&s.k_full[i], 1);
      mbar_init(&s.k_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.z_full[i], 1);
      mbar_init(&s.z_empty[i], 1);
      mbar_init(&s.s_full[i], 1);
      mbar_init(&s.sbuf_free[i], 1);
      mbar_init(&s.w_ready[i], 256);
      mbar_init(&s.tk_full[i], 1);
      mbar_init(&s.tk_empty[i], 11);
    }
    mbar_init(&s.ki_full, 1);
    mbar_init(&s.ki_free, 1);
    mbar_init(&s.ai_full, 1);
    mbar_init(&s.ai_free, 1);
    mbar_init(&s.g_full, 1);
    mbar_init(&s.g_free, 256);
    mbar_init(&s.acc_full, 1);
    mbar_init(&s.acc_free, 256);
    s.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  // tracing builds: wall time and SM cycles at the start and end of this CTA (role 6) give the SM clock
  {
    int slot6 = 4;
    (void)slot6;
    if (tid == 0) LUCID_TR(args.trace, 6, slot6, 90, (long long)globaltimer_ns());
  }
  tc_fence_after_sync();
  const uint32_t tmem = s.tmem_base;

  // Tile q of row-block i (n tiles): the lower part j = 0..i-1, [D1, D2 at j = i], the upper part.
  //   n_low = i (+1 with D1); tiles q < n_low are "lower" (A = dV_i, Z = V'_j).
  // With args.split a row-block's tiles are dealt out as two work items, tiles [q0, q1) each; the item that
  // finishes second adds the other's partial sums (see the epilogue).
  auto item_geometry = [&](int ticket, int& chain, int& i, int& n_low, int& q0, int& q1) -> bool {
    return dk_item(ticket, P.C, T, args.follow_flags != nullptr, args.split != 0, diag_tiles, chain, i, n_low, q0, q1,
                   args.lower_only != 0);
  };

  if (warp == 0) {
    // =========================== producer (one lane) ===========================
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_vp);
      tma_prefetch_desc(&tm_dv);
      uint32_t g = 0;      // tiles loaded so far
      uint32_t swaps = 0;  // loads of the A buffer so far
      bool alive = true;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_empty[slot], ((it >> 1) & 1) ^ 1, cta_abort, ctl, limit, -1, -1, DK_TK_EMPTY)) break;
        const int ticket = atomicAdd(&ctl->ticket, 1);
        s.tk_slot[slot] = ticket;
        mbar_arrive(&s.tk_full[slot]);
        int chain, i, n_low, q0, q1;
        if (!item_geometry(ticket, chain, i, n_low, q0, q1)) break;
        const int b = chain / H, h = chain % H;
        if (!wait_barrier(&s.ki_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, DK_KI_FREE)) break;
        mbar_expect_tx(&s.ki_full, kTileBytes);
        tma_load_4d(s.ki, &tm_k, &s.ki_full, 0, i * kBlock, h, b);
        tma_load_4d(s.ki + kHalfBytes, &tm_k, &s.ki_full, 64, i * kBlock, h, b);
        if (args.follow_flags) {
          // dV_i (and with it every dV_j, j > i) has been published by the reverse solve of this launch
          if (!wait_flag(args.follow_flags + chain * T + i, cta_abort, args.follow_ctl, limit, chain, i, i, nullptr))
            break;
          fence_proxy_async_all();   // flag acquired in the generic proxy; dV is read by TMA
        }
        // A buffer: dV_i for the lower tiles (skipped when there are none), V'_i for the upper tiles
        auto load_a = [&](const CUtensorMap* tm) -> bool {
          if (!wait_barrier(&s.ai_free, (swaps & 1) ^ 1, cta_abort, ctl, limit, chain, i, DK_AI_FREE)) return false;
          mbar_expect_tx(&s.ai_full, kTileBytes);
          tma_load_4d(s.ai, tm, &s.ai_full, 0, i * kBlock, h, b);
          tma_load_4d(s.ai + kHalfBytes, tm, &s.ai_full, 64, i * kBlock, h, b);
          ++swaps;
          return true;
        };
        if (q0 < q1 && !load_a(dk_first_a_is_dv(q0, n_low) ? &tm_dv : &tm_vp)) break;
        for (int q = q0; q < q1 && alive; ++q) {
          if (dk_reloads_a_at(q, q0, n_low)) {
            if (!load_a(&tm_vp)) { alive = false; break; }
          }
          const int j = dk_tile_j(n_low, q, diag_tiles);
          const uint32_t gq = g + (q - q0);
          const int ks = gq % 3, zs = gq & 1;
          if (!wait_barrier(&s.k_empty[ks], ((gq / 3) & 1) ^ 1, cta_abort, ctl, limit, chain, i, DK_K_EMPTY)) {
            alive = false;
            break;
          }
          mbar_expect_tx(&s.k_full[ks], kTileBytes);
          tma_load_4d(s.kring[ks], &tm_k, &s.k_full[ks], 0, j * kBlock, h, b);
          tma_load_4d(s.kring[ks] + kHalfBytes, &tm_k, &s.k_full[ks], 64, j * kBlock, h, b);
          if (!wait_barrier(&s.z_empty[zs], ((gq >> 1) & 1) ^ 1, cta_abort, ctl, limit, chain, i, DK_Z_EMPTY)) {
            alive = false;
            break;
          }
          const CUtensorMap* tz = (q < n_low) ? &tm_vp : &tm_dv;
          mbar_expect_tx(&s.z_full[zs], kTileBytes);
          tma_load_4d(s.zring[zs], tz, &s.z_full[zs], 0, j * kBlock, h, b);
          tma_load_4d(s.zring[zs] + kHalfBytes, tz, &s.z_full[zs], 64, j * kBlock, h, b);
        }
        g += q1 - q0;
      }
    }
  } else if (warp == 1) {
    // =========================== G issuer (owns TMEM) ===========================
    // Warp-uniform control flow; one elected lane issues tcgen05 instructions and arrivals.
    {
      constexpr int fmt = kBf16 ? 1 : 0;
      constexpr uint32_t idesc_kk = umma_idesc(fmt, 0, 0, 128, 128);   // both operands K-major
      const uint64_t d_ai = umma_smem_desc(smem_u32(s.ai), 16, 1024);
      const uint64_t d_zr0 = umma_smem_desc(smem_u32(s.zring[0]), 16, 1024);             // stage: + 32 KiB
      uint32_t g = 0, swaps = 0;
      bool alive = true;
      int trc = 0;
      (void)trc;
      const bool leader = (lane == 0);
      (void)leader;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, DK_TK_FULL)) break;
        const int ticket = s.tk_slot[slot];
        __syncwarp();
        mbar_arrive_w(&s.tk_empty[slot]);
        int chain, i, n_low, q0, q1;
        if (!item_geometry(ticket, chain, i, n_low, q0, q1)) break;
        for (int q = q0; q < q1; ++q) {
          const uint32_t gq = g + (q - q0);
          // G(gq-1) is in the registers of all 256 threads: the single G buffer is free again
          if (gq > 0 &&
              !wait_barrier(&s.g_free, (gq - 1) & 1, cta_abort, ctl, limit, chain, i, DK_G_FREE)) { alive = false; break; }
          if (leader) LUCID_TR(args.trace, 2, trc, 34, gq);
          // the A buffer changes from dV_i to V'_i at q == n_low; wait for the load that serves tile q
          if (dk_waits_a_at(q, q0, n_low)) {
            if (!wait_barrier(&s.ai_full, swaps & 1, cta_abort, ctl, limit, chain, i, DK_AI_FULL)) { alive = false; break; }
            ++swaps;
          }
          const uint32_t zs = gq & 1;
          if (!wait_barrier(&s.z_full[zs], (gq >> 1) & 1, cta_abort, ctl, limit, chain, i, DK_Z_FULL)) { alive = false; break; }
          tc_fence_after_sync();
          if (leader) LUCID_TR(args.trace, 2, trc, 32, gq);
          const uint64_t db = d_zr0 + zs * (kTileBytes >> 4);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
            umma_ss_w(tmem + kDkG, d_ai + off, db + off, idesc_kk, k ? 1u : 0u);
          }
          umma_commit_w(&s.z_empty[zs]);
          umma_commit_w(&s.g_full);
          if (leader) LUCID_TR(args.trace, 2, trc, 33, gq);
          // last lower tile (or last tile): the A buffer may be overwritten once this product is done
          if (dk_frees_a_after(q, q0, q1, n_low)) umma_commit_w(&s.ai_free);
        }
        if (!alive) break;
        g += q1 - q0;
      }
    }
  } else if (warp == 2) {
    // =========================== S issuer ===========================
    // Runs ahead of the G issuer as far as the two S buffers allow.
    {
      constexpr int fmt = kBf16 ? 1 : 0;
      constexpr uint32_t idesc_kk = umma_idesc(fmt, 0, 0, 128, 128);
      const uint64_t d_ki = umma_smem_desc(smem_u32(s.ki), 16, 1024);
      const uint64_t d_kr0 = umma_smem_desc(smem_u32(s.kring[0]), 16, 1024);             // stage: + 32 KiB
      uint32_t g = 0;
      bool alive = true;
      int trc = 0;
      (void)trc;
      const bool leader = (lane == 0);
      (void)leader;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, DK_TK_FULL)) break;
        const int ticket = s.tk_slot[slot];
        __syncwarp();
        mbar_arrive_w(&s.tk_empty[slot]);
        int chain, i, n_low, q0, q1;
        if (!item_geometry(ticket, chain, i, n_low, q0, q1)) break;
        if (!wait_barrier(&s.ki_full, it & 1, cta_abort, ctl, limit, chain, i, DK_KI_FULL)) break;
        tc_fence_after_sync();
        if (leader) LUCID_TR(args.trace, 1, trc, 35, q1 - q0);
        for (int q = q0; q < q1; ++q) {
          const uint32_t gq = g + (q - q0);
          const uint32_t ks = gq % 3;
          const uint32_t buf = gq & 1;
          // W of two tiles ago lived in this buffer: its W*K_j product must have completed
          if (!wait_barrier(&s.sbuf_free[buf], ((gq >> 1) & 1) ^ 1, cta_abort, ctl, limit, chain, i, DK_SBUF_FREE)) {
            alive = false;
            break;
          }
          if (leader) LUCID_TR(args.trace, 1, trc, 29, gq);
          if (!wait_barrier(&s.k_full[ks], (gq / 3) & 1, cta_abort, ctl, limit, chain, i, DK_K_FULL)) { alive = false; break; }
          tc_fence_after_sync();
          if (leader) LUCID_TR(args.trace, 1, trc, 30, gq);
          const uint32_t dst = tmem + (buf ? kDkS1 : kDkS0);
          const uint64_t db = d_kr0 + ks * (kTileBytes >> 4);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
            umma_ss_w(dst, d_ki + off, db + off, idesc_kk, k ? 1u : 0u);
          }
          umma_commit_w(&s.s_full[buf]);
          if (leader) LUCID_TR(args.trace, 1, trc, 31, gq);
        }
        if (!alive) break;
        g += q1 - q0;
        // K_i may be replaced once the S products of this item are complete
        if (q1 > q0) umma_commit_w(&s.ki_free);
        else mbar_arrive_w(&s.ki_free);
      }
    }
  } else if (warp == 3) {
    // =========================== W*K_j issuer ===========================
    {
      constexpr int fmt = kBf16 ? 1 : 0;
      constexpr uint32_t idesc_wk = umma_idesc(fmt, 0, 1, 128, 128);   // ACC += W K_j: B rows = k
      const uint64_t d_kr0_mn = umma_smem_desc(smem_u32(s.kring[0]), kHalfBytes, 1024);
      uint32_t g = 0;
      bool alive = true;
      int trc = 0;
      (void)trc;
      const bool leader = (lane == 0);
      (void)leader;
      for (int it = 0; alive; ++it) {
        const int slot = it & 1;
        if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, DK_TK_FULL)) break;
        const int ticket = s.tk_slot[slot];
        __syncwarp();
        mbar_arrive_w(&s.tk_empty[slot]);
        int chain, i, n_low, q0, q1;
        if (!item_geometry(ticket, chain, i, n_low, q0, q1)) break;
        for (int q = q0; q < q1; ++q) {
          const uint32_t gq = g + (q - q0);
          // per-buffer barrier: the exp groups may be one tile ahead of this warp, never two on one buffer
          if (!wait_barrier(&s.w_ready[gq & 1], (gq >> 1) & 1, cta_abort, ctl, limit, chain, i, DK_W_READY)) {
            alive = false;
            break;
          }
          if (q == q0 &&
              !wait_barrier(&s.acc_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, DK_ACC_FREE)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
          if (leader) LUCID_TR(args.trace, 5, trc, 50, gq);
          const uint32_t ks = gq % 3;
          const uint32_t buf = gq & 1;
          const uint32_t w_tmem = tmem + (buf ? kDkS1 : kDkS0);
          const uint64_t db = d_kr0_mn + ks * (kTileBytes >> 4);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            // W columns: k-steps 0-3 packed at columns 0-31, k-steps 4-7 at columns 64-95 of the S buffer
            const uint32_t a_col = (k < 4) ? k * 8 : 64 + (k - 4) * 8;
            umma_ts_w(tmem + kDkAcc, w_tmem + a_col, db + k * (2048 >> 4), idesc_wk, ((q - q0) | k) ? 1u : 0u);
          }
          umma_commit_w(&s.k_empty[ks]);
          umma_commit_w(&s.sbuf_free[buf]);
          if (leader) LUCID_TR(args.trace, 5, trc, 51, gq);
        }
        if (!alive) break;
        g += q1 - q0;
        // an item without tiles must not run ahead of the epilogue that still owns the previous phase
        if (q1 == q0 && !wait_barrier(&s.acc_free, (it & 1) ^ 1, cta_abort, ctl, limit, chain, i, DK_ACC_FREE)) break;
        umma_commit_w(&s.acc_full);
      }
    }
  } else if (warp >= 4) {
    // =========================== W = -exp(S) o G, then the dK epilogue ===========================
    const int wg = (warp - 4) >> 2;                  // column half: 64*wg .. 64*wg+63
    const float xs = P.exp_scale;                    // exp(k_scale^2 * S) = exp2(S * xs)
    const int row = ((warp & 3) << 5) + lane;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    uint32_t g = 0;
    bool alive = true;
    int trc = 0;
    (void)trc;
    const bool tr_lead = (tid == 128 || tid == 256);
    (void)tr_lead;
    for (int it = 0; alive; ++it) {
      const int slot = it & 1;
      if (!wait_barrier(&s.tk_full[slot], (it >> 1) & 1, cta_abort, ctl, limit, -1, -1, DK_TK_FULL)) break;
      const int ticket = s.tk_slot[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.tk_empty[slot]);
      int chain, i, n_low, q0, q1;
      if (!item_geometry(ticket, chain, i, n_low, q0, q1)) break;
      const int b = chain / H, h = chain % H;
      for (int q = q0; q < q1; ++q) {
        const uint32_t gq = g + (q - q0);
        const uint32_t s_tmem = lane_base + ((gq & 1) ? kDkS1 : kDkS0) + wg * 64;
        const uint32_t g_tmem = lane_base + kDkG + wg * 64;
        if (!wait_barrier(&s.g_full, gq & 1, cta_abort, ctl, limit, chain, i, DK_G_FULL)) {
          alive = false;
          break;
        }
        tc_fence_after_sync();
        uint32_t gv0[32], gv1[32];
        tmem_ld32(g_tmem, gv0);
        tmem_ld32(g_tmem + 32, gv1);
        if (!wait_barrier(&s.s_full[gq & 1], (gq >> 1) & 1, cta_abort, ctl, limit, chain, i, DK_S_FULL)) {
          alive = false;
          break;
        }
        tc_fence_after_sync();
        if (tr_lead) LUCID_TR(args.trace, 3 + wg, trc, 40, gq);
        uint32_t sva[16], svb[16];
        tmem_ld16(s_tmem, sva);
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(&s.g_free);             // to the S/G issuer: G(q) is in registers
        if (tr_lead) LUCID_TR(args.trace, 3 + wg, trc, 41, gq);
        // Diagonal tiles keep c <= r (D1, the last lower tile) or c >= r (D2, the first upper tile): the
        // mask is applied to G here, once per tile, so that the chunk loop stays branch-free.
        const int mask_mode = !diag_tiles ? 0 : (q == n_low - 1 ? 1 : (q == n_low ? 2 : 0));
        if (mask_mode) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int c0 = wg * 64 + e, c1 = c0 + 32;
            const bool keep0 = (mask_mode == 1) ? (c0 <= row) : (c0 >= row);
            const bool keep1 = (mask_mode == 1) ? (c1 <= row) : (c1 >= row);
            gv0[e] = keep0 ? gv0[e] : 0u;
            gv1[e] = keep1 ? gv1[e] : 0u;
          }
        }
        // Chunk c: columns 16c .. 16c+15 of this thread's range; its packed W lands on columns
        // 8c .. 8c+7, inside chunks <= c, which are already in registers.
#define LUCID_DK_CHUNK(C, CUR, NXT, GV, GOFF)                                                          \
        {                                                                                              \
          if ((C) < 3) tmem_ld16(s_tmem + ((C) + 1) * 16, NXT);                                        \
          uint32_t pk[8];                                                                              \
          _Pragma("unroll") for (int e = 0; e < 8; ++e) {                                              \
            const float e0 = ex2_approx(__uint_as_float(CUR[2 * e]) * xs);                             \
            const float e1 = ex2_approx(__uint_as_float(CUR[2 * e + 1]) * xs);                         \
            pk[e] = pack2_fast<kBf16>(-e0 * __uint_as_float(GV[(GOFF) + 2 * e]),                       \
                                      -e1 * __uint_as_float(GV[(GOFF) + 2 * e + 1]));                  \
          }                                                                                            \
          if ((C) < 3) tmem_wait_ld();                                                                 \
          tmem_st8(s_tmem + (C) * 8, pk);                                                              \
        }
        LUCID_DK_CHUNK(0, sva, svb, gv0, 0)
        LUCID_DK_CHUNK(1, svb, sva, gv0, 16)
        LUCID_DK_CHUNK(2, sva, svb, gv1, 0)
        LUCID_DK_CHUNK(3, svb, sva, gv1, 16)
#undef LUCID_DK_CHUNK
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&s.w_ready[gq & 1]);    // to the W*K_j issuer: W(q) is in place
        if (tr_lead) LUCID_TR(args.trace, 3 + wg, trc, 43, gq);
      }
      if (!alive) break;
      g += q1 - q0;

      // ---- epilogue: dK_i columns 64*wg .. +63 ----
      if (!wait_barrier(&s.acc_full, it & 1, cta_abort, ctl, limit, chain, i, DK_ACC_FULL)) break;
      tc_fence_after_sync();
      typedef typename std::conditional<kBf16, __nv_bfloat16, __half>::type elem_t;
      elem_t* out_row = reinterpret_cast<elem_t*>(args.dk) + (long long)b * args.dk_strides.b +
                        (long long)(i * kBlock + row) * args.dk_strides.n + (long long)h * args.dk_strides.h + wg * 64;
      // Split items: whichever half of the row-block finishes first leaves its fp32 sums in the workspace and
      // sets a flag; the other half waits for that flag (bounded; the first half is already in its epilogue
      // when the second learns that it is second), adds the sums and writes dK_i.
      int order = -1;
      float* part_row = nullptr;
      const int rb = chain * T + i;
      if (args.split) {
        part_row = args.partial + ((long long)rb * kBlock + row) * kBlock + wg * 64;
        if (tid == 128) s.claim = atomicAdd(args.sync + rb, 1);
        named_bar_sync(1, 256);
        order = s.claim;
        if (order == 1) {
          if (tid == 128 && !wait_flag(args.sync + P.C * T + rb, cta_abort, ctl, limit, chain, i, i, nullptr))
            *cta_abort = 1;
          named_bar_sync(1, 256);
          if (*cta_abort) break;
        }
      }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t v[32];
        if (q1 > q0) {
          tmem_ld32(lane_base + kDkAcc + wg * 64 + cc * 32, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
        }
        if (order == 0) {
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(part_row + cc * 32 + c * 4) = make_uint4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
          continue;
        }
        if (args.lower_only) {
          // the upper tiles j >= i + 2 were accumulated by the reverse solve that ran before this launch
          const float* up = args.upper + ((long long)rb * kBlock + row) * kBlock + wg * 64 + cc * 32;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 o = __ldcg(reinterpret_cast<const float4*>(up + c * 4));
            v[c * 4] = __float_as_uint(__uint_as_float(v[c * 4]) + o.x);
            v[c * 4 + 1] = __float_as_uint(__uint_as_float(v[c * 4 + 1]) + o.y);
            v[c * 4 + 2] = __float_as_uint(__uint_as_float(v[c * 4 + 2]) + o.z);
            v[c * 4 + 3] = __float_as_uint(__uint_as_float(v[c * 4 + 3]) + o.w);
          }
        }
        if (order == 1) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 o = __ldcg(reinterpret_cast<const float4*>(part_row + cc * 32 + c * 4));
            v[c * 4] = __float_as_uint(__uint_as_float(v[c * 4]) + o.x);
            v[c * 4 + 1] = __float_as_uint(__uint_as_float(v[c * 4 + 1]) + o.y);
            v[c * 4 + 2] = __float_as_uint(__uint_as_float(v[c * 4 + 2]) + o.z);
            v[c * 4 + 3] = __float_as_uint(__uint_as_float(v[c * 4 + 3]) + o.w);
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            o[e] = pack2<kBf16>(__uint_as_float(v[c * 8 + 2 * e]) * P.out_scale,
                                __uint_as_float(v[c * 8 + 2 * e + 1]) * P.out_scale);
          *reinterpret_cast<uint4*>(out_row + cc * 32 + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      if (order == 0) {
        // every thread's sums are ordered before the flag: fence, meet, then one release store
        __threadfence();
        named_bar_sync(1, 256);
        if (tid == 128) st_release_gpu(args.sync + P.C * T + rb, kFlagComplete);
      }
      tc_fence_before_sync();
      mbar_arrive(&s.acc_free);
    }
  }

  if (s.abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    if (tid == 0) report_error(ctl, kErrAborted, -1, -1, blockIdx.x, 0);
  }
  tc_fence_before_sync();
  {
    int slot6 = 4 + 1;
    (void)slot6;
    if (tid == 0) LUCID_TR(args.trace, 6, slot6, 91, (long long)globaltimer_ns());
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

#ifndef LUCID_BODY_ONLY
template <bool kBf16>
__global__ void __launch_bounds__(kDkThreads, 1)
dk_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_vp,
          const __grid_constant__ CUtensorMap tm_dv, const DkArgs args) {
  dk_body<kBf16>(tm_k, tm_vp, tm_dv, args);
}

size_t dk_smem_bytes() { return sizeof(DkSmem) + 1024; }

cudaError_t launch_dk(bool bf16, const CUtensorMap& tm_k, const CUtensorMap& tm_vp, const CUtensorMap& tm_dv,
                      const DkArgs& args, int grid, cudaStream_t stream) {
  cudaError_t e;
  if (bf16) {
    e = cudaFuncSetAttribute(dk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dk_smem_bytes());
    if (e != cudaSuccess) return e;
    dk_kernel<true><<<grid, kDkThreads, dk_smem_bytes(), stream>>>(tm_k, tm_vp, tm_dv, args);
  } else {
    e = cudaFuncSetAttribute(dk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dk_smem_bytes());
    if (e != cudaSuccess) return e;
    dk_kernel<false><<<grid, kDkThreads, dk_smem_bytes(), stream>>>(tm_k, tm_vp, tm_dv, args);
  }
  return cudaGetLastError();
}
#endif  // LUCID_BODY_ONLY

}  // namespace lucid

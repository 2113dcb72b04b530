// Argument blocks and host launchers of the three kernels (definitions in solve.cu, diag_prep.cu, dk.cu).
#pragma once
#include "common.cuh"

namespace lucid {

struct SolveArgs {
  void* out;              // Y (V' or dV), written with plain stores, streamed back through a tensor map
  Strides out_strides;
  const float* lam_inv;   // (C, T, 128) exp(-|k_r|^2)
  int* flags;             // (C, T)
  Control* ctl;
  long long* timestamps;  // (C, T, 8) or null
  long long* trace;       // debugging builds only (LUCID_TRACE); null otherwise
  Problem p;
};

struct PrepArgs {
  void* x;          // (C*T, 128, 128) 16-bit
  float* lam_inv;   // (C*T, 128)
  Control* ctl;
  int T, H;
  float exp_scale;        // log2(e) * k_scale^2
  unsigned long long wait_ns;
};

struct DkArgs {
  void* dk;
  Strides dk_strides;
  Control* ctl;
  const int* follow_flags;  // (C, T) flags of the reverse solve running in the same launch, or null
  Control* follow_ctl;      // that solve's control block (its failure releases the flag waits)
  long long* trace;         // debugging builds only (LUCID_TRACE); null otherwise
  int split;                // 1: a row-block's tiles are two work items whose sums meet through `partial`
  float* partial;           // (C*T, 128, 128) fp32 sums of the half that finished first (split only)
  int* sync;                // (2, C*T) zeroed: claim counters, then completion flags (split only)
  int lower_only;           // 1: items end after the first upper tile; `upper` holds the rest of the upper part
  const float* upper;       // (C*T, 128, 128) fp32 sums over the upper tiles j >= i + 2, written by revdk_kernel
  Problem p;
};

// Reverse solve that also accumulates the upper-triangle dK terms of the tiles it streams (see rev_dk.cu).
struct RevDkArgs {
  void* out;                // dV, streamed back through tm_dv
  const float* lam_inv;     // (C, T, 128)
  int* flags;               // (C, T)
  Control* ctl;
  float* upper;             // (C*T, 128, 128) fp32: sum over j >= i + 2 of W_ij K_j, unscaled
  long long* trace;         // debugging builds only (LUCID_TRACE); null otherwise
  Problem p;
};

// pair = clusters of two CTAs solving pairs of consecutive row-blocks (needs an even number of row-blocks per
// chain, the diagonal solve and full causality); grid is then rounded to whole resident clusters.
// ki_in_tmem = the variant whose S products read K_i from tensor memory (two S buffers instead of three).
cudaError_t launch_solve(bool bf16, bool reverse, bool pair, bool ki_in_tmem, const CUtensorMap& tm_k,
                         const CUtensorMap& tm_in, const CUtensorMap& tm_out, const CUtensorMap& tm_x,
                         const CUtensorMap& tm_st, const SolveArgs& args, int grid, cudaStream_t stream);
cudaError_t launch_diag_prep(bool bf16, const CUtensorMap& tm_k, const PrepArgs& args, int nblocks,
                             cudaStream_t stream);
// tm_dvp: dV' (box 64 x 128); tm_dv: dV (box 64 x 128, loads of published row-blocks and the store);
// tm_vp: V' (box 64 x 128); tm_x: the X workspace (2D).
cudaError_t launch_revdk(bool bf16, const CUtensorMap& tm_k, const CUtensorMap& tm_dvp, const CUtensorMap& tm_dv,
                         const CUtensorMap& tm_vp, const CUtensorMap& tm_x, const RevDkArgs& args, int grid,
                         cudaStream_t stream);
cudaError_t launch_dk(bool bf16, const CUtensorMap& tm_k, const CUtensorMap& tm_vp, const CUtensorMap& tm_dv,
                      const DkArgs& args, int grid, cudaStream_t stream);
// Reverse solve (the first n_solve CTAs to start, counted in *arrivals, which must be zero at launch) and dK
// (the remaining CTAs) in one launch; dargs.follow_flags must point at the solve's flags.
cudaError_t launch_bwd_fused(bool bf16, const CUtensorMap& tm_k, const CUtensorMap& tm_in, const CUtensorMap& tm_out,
                             const CUtensorMap& tm_x, const CUtensorMap& tm_st, const CUtensorMap& tm_vp,
                             const CUtensorMap& tm_dv, const SolveArgs& sargs, const DkArgs& dargs, int n_solve,
                             int* arrivals, int grid, cudaStream_t stream);

// Diagnostic (probe.cu): `grid` CTAs each stream `boxes` 16 KiB boxes of the tensor behind tm (box 64 x 128)
// through a ring of `slots` stages and write the SM clocks that took to clocks[cta] (-1: a wait ran out).
cudaError_t launch_delivery_probe(const CUtensorMap& tm, int slots, int boxes, int chains, int T, int H,
                                  long long* clocks, int grid, cudaStream_t stream);

}  // namespace lucid

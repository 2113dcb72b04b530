// Per-block preparation of the diagonal solve.  Replaces the reference's host-side
// _compute_diag_inv / _compute_diag_inv_transpose (lucid_kernels/cute/forward_sub_interface.py:30-53,
// 177-193), which form inv(tril(exp(K_i K_i^T))) with batched ATen kernels.
//
// The diagonal block factors as M_i = Lambda (I + N) with Lambda = diag(exp(|k_r|^2)) and N strictly
// lower, N_rc = exp(k_r.k_c - |k_r|^2), so M_i^-1 = (I + N)^-1 Lambda^-1.  This kernel writes, per block,
//   X_i   = (I + N)^-1            as a 128 x 128 16-bit tile (row-major, contiguous), and
//   lam_r = exp(-|k_r|^2)         as 128 fp32 values.
// The solve kernels apply X_i (or its transpose) with one tensor-core product and the row scaling in
// fp32, which keeps every 16-bit operand O(1) instead of spanning exp(-|k|^2) ~ 1e-3 .. 1e-7.
//
// One CTA (128 threads) per block: TMA brings K_i into shared memory, tcgen05 forms S = K_i K_i^T in
// TMEM, thread r turns row r into N (fp32, stored transposed in shared memory), then thread c
// back-substitutes column c of X with its 128 running values in registers.
#include <type_traits>
#include "kernels.h"

namespace lucid {

struct PrepSmem {
  alignas(1024) uint8_t k[kTileBytes];   // K_i (two swizzled panels); reused to stage X on the way out
  alignas(16) float nt[kBlock][kBlock];  // nt[c][r] = N[r][c]  (zero on and above the diagonal)
  alignas(8) uint64_t bar_load;
  uint64_t bar_mma;
  uint32_t tmem_base;
  int abort_flag;
};

template <bool kBf16>
__global__ void __launch_bounds__(128) diag_prep_kernel(const __grid_constant__ CUtensorMap tm_k, const PrepArgs args) {
  extern __shared__ uint8_t smem_raw[];
  PrepSmem& s = *reinterpret_cast<PrepSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5;
  const int blk = blockIdx.x;           // chain * T + i
  const int chain = blk / args.T, i = blk % args.T;
  const int b = chain / args.H, h = chain % args.H;
  volatile int* cta_abort = &s.abort_flag;

  if (tid == 0) {
    mbar_init(&s.bar_load, 1);
    mbar_init(&s.bar_mma, 1);
    s.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&s.tmem_base, 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s.tmem_base;

  if (tid == 0) {
    mbar_expect_tx(&s.bar_load, kTileBytes);
    tma_load_4d(s.k, &tm_k, &s.bar_load, 0, i * kBlock, h, b);
    tma_load_4d(s.k + kHalfBytes, &tm_k, &s.bar_load, 64, i * kBlock, h, b);
    if (wait_barrier(&s.bar_load, 0, cta_abort, args.ctl, args.wait_ns, chain, i, 101)) {
      constexpr uint32_t idesc = umma_idesc(kBf16 ? 1 : 0, 0, 0, 128, 128);
      const uint64_t d = umma_smem_desc(smem_u32(s.k), 16, 1024);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint64_t dk = desc_advance(d, (k >> 2) * kHalfBytes + (k & 3) * 32);
        umma_ss(tmem, dk, dk, idesc, k ? 1u : 0u);
      }
      umma_commit(&s.bar_mma);
    }
  }
  bool ok = wait_barrier(&s.bar_mma, 0, cta_abort, args.ctl, args.wait_ns, chain, i, 102);
  tc_fence_after_sync();

  // ---- S row r -> shared memory (transposed) ----
  const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  if (ok) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t v[32];
      tmem_ld32(lane_base + c * 32, v);
      tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 32; ++e) s.nt[c * 32 + e][tid] = __uint_as_float(v[e]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();   // also: the MMA has finished reading s.k
  if (ok) {
    const float srr = s.nt[tid][tid];
    args.lam_inv[(long long)blk * kBlock + tid] = ex2_approx(-srr * args.exp_scale);
    for (int c = 0; c < kBlock; ++c) {
      const float v = s.nt[c][tid];
      s.nt[c][tid] = (c < tid) ? ex2_approx((v - srr) * args.exp_scale) : 0.f;
    }
  }
  __syncthreads();

  // ---- column sweep: thread c owns column c of X = (I + N)^-1 ----
  // Rows are taken in panels of 16.  Panel p first subtracts the contribution of the rows already
  // solved (a rolled loop over k with the 16 running values in registers), then solves its own 16 x 16
  // unit-triangular block.  Solved values X[k][c] (k >= c) are parked in nt[k][c], the half of `nt`
  // that N does not use, where thread c reads them back conflict-free.
  if (ok) {
    typedef typename std::conditional<kBf16, __nv_bfloat16, __half>::type elem_t;
    elem_t* stage = reinterpret_cast<elem_t*>(s.k);   // X as 16-bit row-major, in the (now idle) K buffer
    const int c = tid;
    const int kstart = warp * 32;                     // rows above 32*warp are zero for the whole warp
#pragma unroll 1
    for (int p = 0; p < kBlock / 16; ++p) {
      const int r0 = p * 16;
      float y[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) y[j] = (r0 + j == c) ? 1.f : 0.f;
      if (r0 + 15 >= kstart) {
#pragma unroll 4
        for (int k = kstart; k < r0; ++k) {
          const float xk = (k >= c) ? s.nt[k][c] : 0.f;
          const float4* nrow = reinterpret_cast<const float4*>(&s.nt[k][r0]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 n4 = nrow[q];
            y[4 * q + 0] = fmaf(-n4.x, xk, y[4 * q + 0]);
            y[4 * q + 1] = fmaf(-n4.y, xk, y[4 * q + 1]);
            y[4 * q + 2] = fmaf(-n4.z, xk, y[4 * q + 2]);
            y[4 * q + 3] = fmaf(-n4.w, xk, y[4 * q + 3]);
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float xj = y[j];
#pragma unroll
          for (int jj = j + 1; jj < 16; ++jj) y[jj] = fmaf(-s.nt[r0 + j][r0 + jj], xj, y[jj]);
        }
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int r = r0 + j;
        if (r >= c) s.nt[r][c] = y[j];
        if constexpr (kBf16) stage[r * kBlock + c] = __float2bfloat16_rn(r >= c ? y[j] : 0.f);
        else stage[r * kBlock + c] = __float2half_rn(r >= c ? y[j] : 0.f);
      }
    }
  }
  __syncthreads();
  if (s.abort_flag) {
    // a wait ran out: give the tile load that may still be in flight time to land before this CTA's shared
    // memory is handed to another CTA
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000ull) __nanosleep(1000);
  }
  if (ok) {
    const uint4* src = reinterpret_cast<const uint4*>(s.k);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(args.x) + (long long)blk * kTileBytes);
#pragma unroll
    for (int q = 0; q < 16; ++q) dst[q * 128 + tid] = src[q * 128 + tid];
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

size_t prep_smem_bytes() { return sizeof(PrepSmem) + 1024; }

cudaError_t launch_diag_prep(bool bf16, const CUtensorMap& tm_k, const PrepArgs& args, int nblocks,
                             cudaStream_t stream) {
  cudaError_t e;
  if (bf16) {
    e = cudaFuncSetAttribute(diag_prep_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)prep_smem_bytes());
    if (e != cudaSuccess) return e;
    diag_prep_kernel<true><<<nblocks, 128, prep_smem_bytes(), stream>>>(tm_k, args);
  } else {
    e = cudaFuncSetAttribute(diag_prep_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)prep_smem_bytes());
    if (e != cudaSuccess) return e;
    diag_prep_kernel<false><<<nblocks, 128, prep_smem_bytes(), stream>>>(tm_k, args);
  }
  return cudaGetLastError();
}

}  // namespace lucid

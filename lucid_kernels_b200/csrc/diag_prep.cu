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
// One CTA (128 threads) per block, all products on the tensor cores:
//   1. TMA brings K_i into shared memory, tcgen05 forms S = K_i K_i^T in TMEM, thread r turns row r into
//      row r of N (fp16 in shared memory as an MMA operand; its kBase x kBase diagonal sub-block also in fp32).
//   2. The kBase x kBase diagonal sub-blocks of I + N are inverted in fp32 by substitution, one column per
//      thread: X_d = blockdiag of those inverses.
//   3. Doubling: with D the block-diagonal inverse for sub-blocks of size s, the one for size 2s is
//      D - D N_off D, where N_off is the part of N between the two halves of each 2s block.  Because D is
//      block diagonal, block (p, q) of D N D is D_pp N_pq D_qq, so the full products T = N D and U = D T
//      (two 128^3 MMAs, fp16 operands, fp32 accumulation) carry exactly the wanted sub-blocks at the wanted
//      places; -U is copied into those places of X_d and everything else of U is ignored.  Three levels
//      (16 -> 32 -> 64 -> 128) finish X.
// The 16-bit operands of steps 2-3 are fp16 whatever the input type: N lies in [0, 1) and the entries of X
// are O(1), so fp16's 11 significant bits (against bf16's 8) keep the doubling error below the rounding of
// the final X to the input type.
#include <type_traits>
#include "kernels.h"

namespace lucid {

constexpr int kBase = 16;    // size of the sub-blocks inverted by substitution (16 or 32)

struct PrepSmem {
  alignas(1024) uint8_t k[kTileBytes];   // K_i (two swizzled panels); then the fp32 sub-blocks; then T (fp16)
  alignas(1024) uint8_t n[kTileBytes];   // N  (fp16), row r = row of the block, two swizzled 64-column panels
  alignas(1024) uint8_t x[kTileBytes];   // X_d (fp16), same layout; operand A (rows = m) and operand B (rows = k)
  alignas(8) uint64_t bar_load;
  uint64_t bar_mma;
  uint32_t tmem_base;
  int abort_flag;
};

// 32 consecutive columns (chunk c32 of 4) of row `row` of a tile held as two swizzled 64-column panels
__device__ __forceinline__ void store_chunk16(uint8_t* tile, int row, int c32, const uint32_t (&pk)[16]) {
  uint8_t* panel = tile + (c32 >> 1) * kHalfBytes;
  const uint32_t v0 = (c32 & 1) * 4;
#pragma unroll
  for (int v = 0; v < 4; ++v)
    *reinterpret_cast<uint4*>(panel + sw128_off(row, v0 + v)) =
        make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
}

template <bool kBf16>
__global__ void __launch_bounds__(128) diag_prep_kernel(const __grid_constant__ CUtensorMap tm_k, const PrepArgs args) {
  extern __shared__ uint8_t smem_raw[];
  PrepSmem& s = *reinterpret_cast<PrepSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int blk = blockIdx.x;           // chain * T + i
  const int chain = blk / args.T, i = blk % args.T;
  const int b = chain / args.H, h = chain % args.H;
  volatile int* cta_abort = &s.abort_flag;
  const float xs = args.exp_scale;

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
  const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  uint32_t phase = 0;        // completed waits on bar_mma
  // every thread waits for the product just committed; false after a timeout (anybody's)
  auto product_done = [&](int id) -> bool {
    const bool ok = wait_barrier(&s.bar_mma, phase & 1, cta_abort, args.ctl, args.wait_ns, chain, i, id);
    ++phase;
    tc_fence_after_sync();
    return ok;
  };
  // D[tmem] = A B with A = tile `a` (rows = m, K-major) and B = tile `bt` (rows = k, MN-major), fp16 operands
  auto issue_product = [&](const uint8_t* a, const uint8_t* bt) {
    constexpr uint32_t idesc = umma_idesc(0, 0, 1, 128, 128);
    const uint64_t da = umma_smem_desc(smem_u32(a), 16, 1024);
    const uint64_t db = umma_smem_desc(smem_u32(bt), kHalfBytes, 1024);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      umma_ss(tmem, desc_advance(da, (k >> 2) * kHalfBytes + (k & 3) * 32), desc_advance(db, k * 2048), idesc,
              k ? 1u : 0u);
    umma_commit(&s.bar_mma);
  };

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
  bool ok = product_done(102);

  // ---- step 1: row r of N (fp16 operand), its diagonal sub-block in fp32 ----
  const int r = tid;
  float* nd = reinterpret_cast<float*>(s.k);                   // [128 / kBase][kBase][kBase]: N sub-blocks
  float* xd = nd + (kBlock / kBase) * kBase * kBase;           // same shape: their inverses
  const int sb = r / kBase, sr = r % kBase;                    // sub-block of row r, row inside it
  if (ok) {
    uint32_t v[32];
    tmem_ld32(lane_base + warp * 32, v);                       // the chunk that holds S_rr (column r = 32 warp + lane)
    tmem_wait_ld();
    float srr = 0.f;
#pragma unroll
    for (int e = 0; e < 32; ++e) srr = (e == lane) ? __uint_as_float(v[e]) : srr;
    args.lam_inv[(long long)blk * kBlock + r] = ex2_approx(-srr * xs);
    const float shift = -srr * xs;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      tmem_ld32(lane_base + c * 32, v);
      tmem_wait_ld();
      float nv[32];
#pragma unroll
      for (int e = 0; e < 32; ++e)
        nv[e] = (c * 32 + e < r) ? ex2_approx(fmaf(__uint_as_float(v[e]), xs, shift)) : 0.f;
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) pk[e] = pack2<false>(nv[2 * e], nv[2 * e + 1]);
      store_chunk16(s.n, r, c, pk);
      if (c == warp) {                                         // the chunk that holds this row's sub-block
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if ((c * 32 + e) / kBase == sb) nd[(sb * kBase + sr) * kBase + (c * 32 + e) % kBase] = nv[e];
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();             // every thread has read S (also: the MMA has finished reading K_i)
  ok = !s.abort_flag;

  // ---- step 2: invert the unit lower-triangular sub-blocks, one column per thread ----
  if (ok) {
    const int j = sr;                                          // column j of sub-block sb
    const float* nb = nd + sb * kBase * kBase;
    float y[kBase];
#pragma unroll
    for (int q = 0; q < kBase; ++q) {
      float acc = (q == j) ? 1.f : 0.f;
#pragma unroll
      for (int m = 0; m < q; ++m) acc = fmaf(-nb[q * kBase + m], y[m], acc);
      y[q] = acc;                                              // zero above the diagonal by construction
    }
#pragma unroll
    for (int q = 0; q < kBase; ++q) xd[(sb * kBase + q) * kBase + j] = y[q];
  }
  __syncthreads();
  if (ok) {
    // row r of X_d: its sub-block's row, zero elsewhere
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const int c0 = c * 32 + 2 * e;
        const float lo = (c0 / kBase == sb) ? xd[(sb * kBase + sr) * kBase + c0 % kBase] : 0.f;
        const float hi = ((c0 + 1) / kBase == sb) ? xd[(sb * kBase + sr) * kBase + (c0 + 1) % kBase] : 0.f;
        pk[e] = pack2<false>(lo, hi);
      }
      store_chunk16(s.x, r, c, pk);
    }
  }

  // ---- step 3: doubling ----
#pragma unroll 1
  for (int sz = kBase; sz < kBlock; sz <<= 1) {
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    ok = !s.abort_flag;
    if (ok && tid == 0) {
      tc_fence_after_sync();
      issue_product(s.n, s.x);                                 // T = N X_d
    }
    if (ok) ok = product_done(103);
    if (ok) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(lane_base + c * 32, v);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) pk[e] = pack2<false>(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
        store_chunk16(s.k, r, c, pk);                          // T as an operand with rows = k
      }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    ok = !s.abort_flag;
    if (ok && tid == 0) {
      tc_fence_after_sync();
      issue_product(s.x, s.k);                                 // U = X_d T
    }
    if (ok) ok = product_done(104);
    if (ok) {
      // Rows in the second half of their 2*sz block get -U in the columns of the first half.  Which 32-column
      // chunks those are is the same for all rows of a warp; with sz = 16 only the upper half-warp has any.
      const int w0 = warp * 32;
      const bool warp_has = (sz >= 32) ? ((w0 % (2 * sz)) >= sz) : true;
      if (warp_has) {
        const int col0 = (sz >= 32) ? (w0 - (w0 % (2 * sz))) : w0;        // first column of the first half
        const int nch = (sz >= 32) ? (sz / 32) : 1;
        const bool mine = (r % (2 * sz)) >= sz;
        for (int cc = 0; cc < nch; ++cc) {
          const int c = col0 / 32 + cc;
          uint32_t v[32];
          tmem_ld32(lane_base + c * 32, v);
          tmem_wait_ld();
          if (mine) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e)
              pk[e] = pack2<false>(-__uint_as_float(v[2 * e]), -__uint_as_float(v[2 * e + 1]));
            uint8_t* panel = s.x + (c >> 1) * kHalfBytes;
            const uint32_t v0 = (c & 1) * 4;
            const int nvec = (sz >= 32) ? 4 : 2;                          // sz = 16: columns col0 .. col0 + 15 only
            for (int q = 0; q < nvec; ++q)
              *reinterpret_cast<uint4*>(panel + sw128_off(r, v0 + q)) =
                  make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  ok = !s.abort_flag;
  if (!ok) {
    // a wait ran out: give a tile load or product that may still be in flight time to land before this
    // CTA's shared memory and tensor memory are handed to another CTA
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000ull) __nanosleep(1000);
  }
  if (ok) {
    // X (fp16, swizzled panels) -> global, row-major, in the input's 16-bit type; consecutive threads write
    // consecutive 16-byte pieces
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(args.x) + (long long)blk * kTileBytes);
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      const int idx = q * 128 + tid;          // piece idx: row idx / 16, 16-byte vector idx % 16 of the row
      const int row = idx >> 4, vec = idx & 15;
      uint4 w = *reinterpret_cast<const uint4*>(s.x + (vec >> 3) * kHalfBytes + sw128_off(row, vec & 7));
      if constexpr (kBf16) {
        uint32_t in[4] = {w.x, w.y, w.z, w.w}, o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack2<false>(in[e]);
          o[e] = pack2<true>(f.x, f.y);
        }
        w = make_uint4(o[0], o[1], o[2], o[3]);
      }
      dst[idx] = w;
    }
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

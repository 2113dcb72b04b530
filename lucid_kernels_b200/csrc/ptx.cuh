// Thin inline-PTX wrappers for the Blackwell (sm_100a) primitives the LUCID kernels use:
// mbarrier, TMA tiled loads (every load has a single destination CTA), tcgen05 MMA / TMEM, proxy fences,
// and release/acquire flag accesses.  Everything here is device-only and header-only.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace lucid {

// ---------------------------------------------------------------------------------------------
// misc
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .pred P1;\n"
      "elect.sync _|P1, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, P1;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------------
// mbarrier (CTA-local shared memory)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  // make barrier initialisation visible to the async proxy (TMA / tcgen05.commit)
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// ---------------------------------------------------------------------------------------------
// thread-block clusters: the peer CTA's shared memory and barriers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// address of the peer CTA's copy of a shared-memory location of this CTA
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta_rank));
  return r;
}
// arrive on a barrier of the peer CTA; releases this thread's earlier writes at cluster scope
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// bulk copy from this CTA's shared memory into the peer's (one destination); completion is counted in bytes on
// a barrier of the peer, like a TMA load there.  All addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster_addr, uint32_t src_local_addr, uint32_t bytes,
                                                  uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   dst_cluster_addr),
               "r"(src_local_addr), "r"(bytes), "r"(bar_cluster_addr)
               : "memory");
}
// a word in the peer CTA's shared memory, written with release / read with acquire at cluster scope
__device__ __forceinline__ void st_release_cluster(uint32_t cluster_addr, int v) {
  asm volatile("st.release.cluster.shared::cluster.b32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_cluster_local(const int* p) {
  int v;
  asm volatile("ld.acquire.cluster.shared::cta.b32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
// all threads of both CTAs: nobody passes before everybody has arrived (start: the peer's barriers are
// initialised; end: the peer no longer touches this CTA's shared memory)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// fences
// ---------------------------------------------------------------------------------------------
// generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05.mma operands)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// generic <-> async proxy ordering for global memory (flag acquire, then TMA load of the tile)
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// release / acquire flags in global memory
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_relaxed_gpu(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ---------------------------------------------------------------------------------------------
// TMA tiled loads (tensor map in kernel parameter space), completion on an mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// The same loads with an L2 eviction policy.  Tiles that are read once per row-block (its own right-hand side, its
// inverse block) are loaded evict-first, so that they do not push out the K_j and Y_j tiles every row-block of the
// scheduler group streams again and again: the rate at which TMA delivers those drops from 65 to 47 bytes per clock
// per SM once the re-read set grows past about 64 MB (measured, csrc/probe.cu).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], "
      "[%2], %5;" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_hint(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                                 int c2, int c3, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, "
      "%5, %6}], [%2], %7;" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
      : "memory");
}

// TMA tiled store shared -> global (bulk async-group completion)
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all committed stores have finished READING shared memory (the buffer may be reused)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all committed stores are complete (their writes have been performed)
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// TMEM allocation (one full warp executes these)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------------------------------------
// UMMA descriptors
// ---------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a 16-bit operand tile held in the 128-byte-swizzled layout that a
// TMA box of 64 elements x R rows produces: row r of the box sits at r*128 bytes, its eight 16-byte
// chunks XOR-permuted by (r & 7); eight rows form one 1024-byte swizzle atom.
//   * "K-major" use  (rows = M or N index, the 64 contiguous elements = K): SBO = 1024 (next 8 rows),
//     LBO unused by the hardware for swizzled K-major tiles.
//   * "MN-major" use (rows = K index, the 64 contiguous elements = M or N): SBO = 1024 (next 8 K rows),
//     LBO = byte distance between consecutive 64-element column panels of the tile.
// Bits: [0,14) start>>4, [16,30) LBO>>4, [32,46) SBO>>4, [46,48) version=1, [61,64) layout (2 = SW128).
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 (fp16/bf16 operands, fp32 accumulate), dense, no negate.
//   ab_fmt: 0 = fp16, 1 = bf16.  a_mn / b_mn: 1 when that operand is MN-major in shared memory.
__host__ __device__ constexpr uint32_t umma_idesc(int ab_fmt, int a_mn, int b_mn, int M, int N) {
  return (1u << 4)                                  // accumulator format: fp32
         | (static_cast<uint32_t>(ab_fmt) << 7)     // A format
         | (static_cast<uint32_t>(ab_fmt) << 10)    // B format
         | (static_cast<uint32_t>(a_mn) << 15)      // A major
         | (static_cast<uint32_t>(b_mn) << 16)      // B major
         | (static_cast<uint32_t>(N >> 3) << 17)    // N / 8
         | (static_cast<uint32_t>(M >> 4) << 24);   // M / 16
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A is M x K, 16-bit pairs packed along K in 32-bit TMEM columns.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Whole-warp variants: every lane of a converged warp calls them with warp-uniform arguments and one
// elected lane issues the instruction.  Keeping the call sites convergent lets the compiler hold
// descriptors and addresses in uniform registers.  elect.sync with a full mask names the same lane on
// every call, so a commit tracks the MMAs issued through these wrappers.
__device__ __forceinline__ void umma_ss_w(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  if (elect_one()) umma_ss(d_tmem, adesc, bdesc, idesc, accumulate);
}
__device__ __forceinline__ void umma_ts_w(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  if (elect_one()) umma_ts(d_tmem, a_tmem, bdesc, idesc, accumulate);
}
__device__ __forceinline__ void umma_commit_w(uint64_t* bar) {
  if (elect_one()) umma_commit(bar);
}
__device__ __forceinline__ void mbar_arrive_w(uint64_t* bar) {
  if (elect_one()) mbar_arrive(bar);
}

// ---------------------------------------------------------------------------------------------
// TMEM <-> registers.  Warp w of a 4-warp group owns lanes 32*(w%4) .. +31; each thread gets one row.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// numeric helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two exponentials per MUFU instruction: 2^x for a pair of values through ex2.approx.f16x2.  The
// MUFU pipe issues 16 results per clock per SM for fp32 and as many *instructions* for f16x2, so this
// halves the MUFU time of a 128 x 128 tile (16384 exponentials) from 1024 to 512 cycles.  Accuracy: x is
// rounded to fp16 (11 significant bits) first, a relative error of the result of at most 2^-11 * ln2 * |x|
// rounded up to a power of two: 3.4e-4 for |x| < 2, 1.4e-3 for |x| < 8, below or at the size of the bf16
// rounding the result undergoes anyway.  Range: results above 65504 (x >= 16) overflow and results below
// 6e-8 vanish, so callers route any group of values whose maximum is not below 15.9 through
// the fp32 instruction instead.  Measured on B200 (B=2, N=32768, H=8): 11 % slower than the fp32
// instruction in both kernels (the guard and the extra conversions cost more than the MUFU time saved),
// so it is off by default.
__device__ __forceinline__ uint32_t ex2_f16x2(float x_lo, float x_hi) {
  uint32_t xh, r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(xh) : "f"(x_hi), "f"(x_lo));
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(r) : "r"(xh));
  return r;
}
#ifndef LUCID_EXP_F16X2
#define LUCID_EXP_F16X2 0
#endif
constexpr bool kExpF16x2 = LUCID_EXP_F16X2 != 0;
constexpr float kExpF16x2Max = 15.9f;

// 2^x on the FMA and ALU pipes, for use beside ex2.approx when the MUFU pipe (16 results per clock per
// SM) is the bottleneck.  Cody-Waite split: adding 1.5 * 2^23 rounds x to the nearest integer n in the
// low mantissa bits; 2^f for f = x - n in [-0.5, 0.5] is a degree-3 minimax polynomial (max relative
// error 7.5e-5, twenty times below a bf16 half-ulp); n is added into the exponent field.  Inputs are
// clamped to [-125, 125] so the exponent arithmetic cannot wrap.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fminf(fmaxf(x, -125.f), 125.f);
  const float t = x + 12582912.f;
  const float f = x - (t - 12582912.f);
  float p = fmaf(f, 0.0551716610789299f, 0.2426111251115799f);
  p = fmaf(p, f, 0.6932609677314758f);
  p = fmaf(p, f, 0.9999280571937561f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
// Element e of a row uses the polynomial when e % kExpPolyPeriod == kExpPolyPeriod - 1 (0 disables it).
// Measured on B200 (B=2, N=32768, H=8): periods 2, 3 and 4 were all slower than 0, because a polynomial
// costs about as many FMA + ALU issue cycles per warp as the 8 cycles of one MUFU instruction, so it
// is off by default.
#ifndef LUCID_EXP_POLY_PERIOD
#define LUCID_EXP_POLY_PERIOD 0
#endif
constexpr int kExpPolyPeriod = LUCID_EXP_POLY_PERIOD;
__device__ __forceinline__ float ex2_mixed(float x, int e) {
  if (kExpPolyPeriod > 0 && (e % (kExpPolyPeriod > 0 ? kExpPolyPeriod : 1)) == kExpPolyPeriod - 1) return ex2_poly(x);
  return ex2_approx(x);
}

// pack two fp32 into one 32-bit word of bf16 (is_bf16) or fp16, round-to-nearest-even; `lo` lands in
// the low half (the lower K / column index).
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  if constexpr (kBf16) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}
// The same packing for bf16 done with integer instructions: add half an ulp of the 16-bit result to the
// fp32 bit pattern (round to nearest, ties away from zero; infinities stay infinities) and splice the two
// upper halves with one byte permute.  Used in the exp loops, where the conversion instruction would
// compete with ex2 for the MUFU pipe.  Measured on B200: no gain (dK kernel 3 % slower), so off by default.
#ifndef LUCID_PACK_ALU
#define LUCID_PACK_ALU 0
#endif
__device__ __forceinline__ uint32_t pack2_bf16_alu(float lo, float hi) {
  const uint32_t a = __float_as_uint(lo) + 0x8000u;
  const uint32_t b = __float_as_uint(hi) + 0x8000u;
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2_fast(float lo, float hi) {
  if constexpr (kBf16 && (LUCID_PACK_ALU != 0)) return pack2_bf16_alu(lo, hi);
  else return pack2<kBf16>(lo, hi);
}

template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  float2 f;
  if constexpr (kBf16) {
    f.x = __uint_as_float(w << 16);
    f.y = __uint_as_float(w & 0xFFFF0000u);
  } else {
    __half2 h = *reinterpret_cast<__half2*>(&w);
    f = __half22float2(h);
  }
  return f;
}

// exp2 of 32 consecutive values (given as fp32 bit patterns, to be multiplied by `scale` first) packed
// into 16 words of bf16 or fp16 pairs, optionally negated.  Uses the paired fp16 instruction unless the
// largest argument is too big for an fp16 result.
template <bool kBf16, bool kNegate>
__device__ __forceinline__ void exp2_pack32(const uint32_t* v, float scale, uint32_t (&pk)[16]) {
  if constexpr (kExpF16x2) {
    float m = __uint_as_float(v[0]);
#pragma unroll
    for (int e = 1; e < 32; ++e) m = fmaxf(m, __uint_as_float(v[e]));
    if (m * scale < kExpF16x2Max) {
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        uint32_t h = ex2_f16x2(__uint_as_float(v[2 * e]) * scale, __uint_as_float(v[2 * e + 1]) * scale);
        if constexpr (kNegate) h ^= 0x80008000u;
        if constexpr (kBf16) {
          const float2 f = unpack2<false>(h);
          pk[e] = pack2<true>(f.x, f.y);
        } else {
          pk[e] = h;
        }
      }
      return;
    }
  }
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    float e0 = ex2_mixed(__uint_as_float(v[2 * e]) * scale, 2 * e);
    float e1 = ex2_mixed(__uint_as_float(v[2 * e + 1]) * scale, 2 * e + 1);
    if constexpr (kNegate) {
      e0 = -e0;
      e1 = -e1;
    }
    pk[e] = pack2_fast<kBf16>(e0, e1);
  }
}

// -2^(v * scale) for 32 consecutive values, kept in fp32 (same fp16-pair shortcut and guard as above).
__device__ __forceinline__ void neg_exp2_f32x32(const uint32_t* v, float scale, float* out) {
  if constexpr (kExpF16x2) {
    float m = __uint_as_float(v[0]);
#pragma unroll
    for (int e = 1; e < 32; ++e) m = fmaxf(m, __uint_as_float(v[e]));
    if (m * scale < kExpF16x2Max) {
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const uint32_t h = ex2_f16x2(__uint_as_float(v[2 * e]) * scale, __uint_as_float(v[2 * e + 1]) * scale) ^ 0x80008000u;
        const float2 f = unpack2<false>(h);
        out[2 * e] = f.x;
        out[2 * e + 1] = f.y;
      }
      return;
    }
  }
#pragma unroll
  for (int e = 0; e < 32; ++e) out[e] = -ex2_approx(__uint_as_float(v[e]) * scale);
}

// Byte offset of 16-byte chunk `chunk` (0..7 within a 64-element panel) of row `row` inside a
// 128-byte-swizzled panel (rows of 128 bytes, 1024-byte-aligned base).
__device__ __forceinline__ uint32_t sw128_off(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

}  // namespace lucid

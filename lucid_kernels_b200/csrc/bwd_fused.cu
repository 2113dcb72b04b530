// Backward pass in one launch for problems with few chains per GPU: the reverse solve is then bound by
// its chain latency (T publish -> acquire hand-overs) and leaves most SMs idle, while the dK kernel that
// follows is bound by throughput.  Here the first n_solve CTAs to START (an arrival counter in the workspace,
// not the block index: a CTA that draws a number is running) take the reverse solve and join the dK program
// when the solve's row-blocks have all been taken; the other CTAs run the dK program from the start, each dK
// row-block waiting (bounded) for the solve's flag of that row-block.  The solve never waits for dK, and its
// own row-blocks are claimed by ticket in dependency order, so the waits make progress however few CTAs of
// the launch are resident at a time.  Replaces the two phases of the reference's
// BackwardSubSm90 (lucid_kernels/cute/forward_sub_bwd.py:1053-1269), which also run in one launch.
#define LUCID_BODY_ONLY
#include "solve.cu"
#include "dk.cu"

namespace lucid {

template <bool kBf16>
__global__ void __launch_bounds__(kSolveThreads, 1)
bwd_fused_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_in,
                 const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_x,
                 const __grid_constant__ CUtensorMap tm_st, const __grid_constant__ CUtensorMap tm_vp,
                 const __grid_constant__ CUtensorMap tm_dv, const SolveArgs sargs, const DkArgs dargs,
                 const int n_solve, int* const arrivals) {
  __shared__ int arrival;
  if (threadIdx.x == 0) arrival = atomicAdd(arrivals, 1);
  __syncthreads();
  // A solve CTA joins the dK program once the solve's row-blocks have all been taken.
  if (arrival < n_solve) solve_body<kBf16, true, 2>(tm_k, tm_in, tm_out, tm_x, tm_st, sargs, false);
  dk_body<kBf16>(tm_k, tm_vp, tm_dv, dargs);
}

cudaError_t launch_bwd_fused(bool bf16, const CUtensorMap& tm_k, const CUtensorMap& tm_in, const CUtensorMap& tm_out,
                             const CUtensorMap& tm_x, const CUtensorMap& tm_st, const CUtensorMap& tm_vp,
                             const CUtensorMap& tm_dv, const SolveArgs& sargs, const DkArgs& dargs, int n_solve,
                             int* arrivals, int grid, cudaStream_t stream) {
  static_assert(kSolveThreads == kDkThreads, "both programs run with the same block size");
  const size_t smem = sizeof(SolveSmem) > sizeof(DkSmem) ? sizeof(SolveSmem) + 1024 : sizeof(DkSmem) + 1024;
  cudaError_t e;
  if (bf16) {
    e = cudaFuncSetAttribute(bwd_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    bwd_fused_kernel<true><<<grid, kSolveThreads, smem, stream>>>(tm_k, tm_in, tm_out, tm_x, tm_st, tm_vp, tm_dv,
                                                                  sargs, dargs, n_solve, arrivals);
  } else {
    e = cudaFuncSetAttribute(bwd_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    bwd_fused_kernel<false><<<grid, kSolveThreads, smem, stream>>>(tm_k, tm_in, tm_out, tm_x, tm_st, tm_vp, tm_dv,
                                                                   sargs, dargs, n_solve, arrivals);
  }
  return cudaGetLastError();
}

}  // namespace lucid

// Delivery-rate probe: how fast TMA brings operand tiles from L2 into the shared memory of every SM at once.
// A diagnostic with no counterpart in the reference.  The solve and dK kernels stream two 32 KiB operand tiles
// per tile of work into each SM; this kernel does the same loads (16 KiB boxes of a (B, N, H, 128) tensor, 64
// columns x 128 rows, 128-byte swizzle, the ring of `slots` stages the kernels use) and nothing else, so its
// bytes per clock per SM are the ceiling those kernels' operand streams can reach, whatever they compute.
//
// One persistent CTA per SM, two threads at work: thread 0 issues the loads as stages come free, thread 32 waits
// for each stage to fill and frees it at once.  Every wait is bounded; a CTA that gives up writes -1.
#include "kernels.h"

namespace lucid {

constexpr int kProbeMaxSlots = 12;
constexpr uint32_t kProbeSpinLimit = 1u << 27;

__global__ void __launch_bounds__(64, 1)
delivery_probe_kernel(const __grid_constant__ CUtensorMap tm,   // box 64 x 128
                      int slots, int boxes, int chains, int T, int H, long long* clocks) {
  extern __shared__ uint8_t probe_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(probe_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(base + slots * kHalfBytes);
  uint64_t* empty = full + slots;
  if (threadIdx.x == 0) {
    for (int i = 0; i < slots; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  // CTAs are dealt over the chains like the solve's row-blocks, so several SMs stream the same tiles
  const int chain = blockIdx.x % chains, b = chain / H, h = chain % H;
  const long long t0 = clock64();
  // stage and phase are carried along (no division in the loops: one thread has to issue a box every ~350 clocks)
  if (threadIdx.x == 0) {
    int st = 0, tile = (blockIdx.x * 3) % T;      // the two 64-column halves of a tile, then the next tile
    uint32_t ph = 0;
    for (int u = 0; u < boxes; ++u) {
      uint32_t spins = 0;
      while (!mbar_try_wait(&empty[st], ph ^ 1))
        if (++spins > kProbeSpinLimit) return;
      mbar_expect_tx(&full[st], kHalfBytes);
      tma_load_4d(base + st * kHalfBytes, &tm, &full[st], 64 * (u & 1), tile * kBlock, h, b);
      if ((u & 1) && ++tile == T) tile = 0;
      if (++st == slots) {
        st = 0;
        ph ^= 1;
      }
    }
  } else if (threadIdx.x == 32) {
    long long result = -1;
    int st = 0, u = 0;
    uint32_t ph = 0;
    for (; u < boxes; ++u) {
      uint32_t spins = 0;
      bool ok = true;
      while (!mbar_try_wait(&full[st], ph))
        if (++spins > kProbeSpinLimit) { ok = false; break; }
      if (!ok) break;
      mbar_arrive(&empty[st]);
      if (++st == slots) {
        st = 0;
        ph ^= 1;
      }
    }
    if (u == boxes) result = clock64() - t0;
    clocks[blockIdx.x] = result;
  }
}

cudaError_t launch_delivery_probe(const CUtensorMap& tm, int slots, int boxes, int chains, int T, int H,
                                  long long* clocks, int grid, cudaStream_t stream) {
  if (slots < 1 || slots > kProbeMaxSlots) return cudaErrorInvalidValue;
  const size_t smem = (size_t)slots * kHalfBytes + 2 * slots * sizeof(uint64_t) + 1024 + 64;
  cudaError_t e = cudaFuncSetAttribute(delivery_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  delivery_probe_kernel<<<grid, 64, smem, stream>>>(tm, slots, boxes, chains, T, H, clocks);
  return cudaGetLastError();
}

}  // namespace lucid

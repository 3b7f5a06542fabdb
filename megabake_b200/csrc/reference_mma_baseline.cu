// Measurement baseline, not part of the decoder path: the algorithm of the reference's only
// sm_100 kernel (src/megabake/bodies/blackwell.py:91-159, provider "blackwell_mma"), restated in
// CUDA C so that the projection engine can be timed against it on the same GPU.  The reference
// emits it as CuTe-DSL Python for its own JIT; what is restated here is its algorithm as that
// source states it: one CTA of four warps per 16 x 32 output tile, each warp one
// mma.sync.m16n8k16 (bf16 in, fp32 accumulate) per 16-element K step, operand fragments gathered
// element by element from global memory under M/N/K predicates, no shared memory, no TMA, no
// pipeline, no bias.  y[M, N] = x[M, K] . w[N, K]^T.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/megabake_b200.h"

namespace {

__device__ __forceinline__ uint32_t pack_pair(const __nv_bfloat16* base, long long row, int ld, int k, bool row_ok, int kmax) {
  // two consecutive K elements of one row, each under its own predicate (the reference predicates every element)
  const unsigned short lo = (row_ok && k < kmax) ? __bfloat16_as_ushort(base[row * ld + k]) : 0;
  const unsigned short hi = (row_ok && k + 1 < kmax) ? __bfloat16_as_ushort(base[row * ld + k + 1]) : 0;
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

__global__ void __launch_bounds__(128) reference_mma_16x32(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ y, int m, int n, int k) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = (n + 31) / 32;
  const int tiles = ((m + 15) / 16) * ntiles;
  const int r = lane >> 2, c2 = (lane & 3) * 2;
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int row_base = (tile / ntiles) * 16;
    const int col_base = (tile % ntiles) * 32 + warp * 8;  // this warp's eight output columns
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int kbase = 0; kbase < k; kbase += 16) {
      uint32_t a[4], b[2];
      const int m0 = row_base + r, m1 = m0 + 8;
      a[0] = pack_pair(x, m0, k, kbase + c2, m0 < m, k);
      a[1] = pack_pair(x, m1, k, kbase + c2, m1 < m, k);
      a[2] = pack_pair(x, m0, k, kbase + c2 + 8, m0 < m, k);
      a[3] = pack_pair(x, m1, k, kbase + c2 + 8, m1 < m, k);
      const int nn = col_base + r;
      b[0] = pack_pair(w, nn, k, kbase + c2, nn < n, k);
      b[1] = pack_pair(w, nn, k, kbase + c2 + 8, nn < n, k);
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
          : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
          : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
    const int m0 = row_base + r, m1 = m0 + 8, n0 = col_base + c2;
    if (m0 < m && n0 < n) y[static_cast<long long>(m0) * n + n0] = __float2bfloat16_rn(acc[0]);
    if (m0 < m && n0 + 1 < n) y[static_cast<long long>(m0) * n + n0 + 1] = __float2bfloat16_rn(acc[1]);
    if (m1 < m && n0 < n) y[static_cast<long long>(m1) * n + n0] = __float2bfloat16_rn(acc[2]);
    if (m1 < m && n0 + 1 < n) y[static_cast<long long>(m1) * n + n0 + 1] = __float2bfloat16_rn(acc[3]);
  }
}

}  // namespace

extern "C" int mk_baseline_mma_gemm(const void* x, const void* weight, void* y, int m, int n, int k, void* stream) {
  if (!x || !weight || !y || m < 1 || n < 1 || k < 1) return MK_ERR_INVALID;
  const long long tiles = static_cast<long long>((m + 15) / 16) * ((n + 31) / 32);
  const int grid = static_cast<int>(tiles < (1 << 20) ? tiles : (1 << 20));  // one CTA per tile, as the reference launches it
  reference_mma_16x32<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(y), m, n, k);
  return cudaGetLastError() == cudaSuccess ? MK_OK : MK_ERR_CUDA;
}

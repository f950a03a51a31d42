// CUDA-core twin of the masked GEMM: same operands and semantics as the tensor-core kernel, fp32
// arithmetic on the SIMT pipes.  It mirrors the role of the reference's CUDA_MODE build
// (StreamMaskedGEMM/perf/basic_nn.cu:55-71,239-246; masked SIMT iterators in
// StreamMaskedGEMM/cutlass/gemm/gemm_global_tile.h:358-390, :667-763): an independent code path
// through the same gather/scatter definition, used to cross-check the tcgen05 kernel on sizes the
// CPU oracle cannot reach.  It is not tuned.
#include "ts_common.cuh"
#include "ts_kernels.h"

namespace ts {

namespace {

constexpr int kJB = 8;  // output columns per thread

template <int DT>
__global__ void __launch_bounds__(256)
masked_gemm_simt_kernel(const TileDesc* __restrict__ tiles, const uint16_t* __restrict__ Wp,
                        long long ldw, const uint16_t* __restrict__ At, long long lda,
                        uint16_t* __restrict__ Ct, long long ldc, int M, float alpha, float beta) {
  const TileDesc td = tiles[blockIdx.y];
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  const int j0 = blockIdx.z * kJB;
  if (j0 >= td.n_count) return;
  __shared__ uint16_t w_s[kJB][64];
  float acc[kJB];
#pragma unroll
  for (int j = 0; j < kJB; ++j) acc[j] = 0.0f;

  for (int i0 = 0; i0 < td.k_count; i0 += 64) {
    __syncthreads();
    for (int e = threadIdx.x; e < kJB * 64; e += blockDim.x) {
      const int j = e >> 6, i = i0 + (e & 63);
      uint16_t w = 0;
      if (i < td.k_count && j0 + j < td.n_count) {
        w = Wp[static_cast<long long>(td.w_row0 + j0 + j) * ldw + i];
      }
      w_s[j][e & 63] = w;
    }
    __syncthreads();
    if (m < M) {
      const int iend = min(64, td.k_count - i0);
      for (int ii = 0; ii < iend; ++ii) {
        const int i = i0 + ii;
        const int kk = td.k_list[i] + (td.relative ? i : 0);
        const float a = unpack1<DT>(At[static_cast<long long>(kk) * lda + m]);
#pragma unroll
        for (int j = 0; j < kJB; ++j) acc[j] = fmaf(unpack1<DT>(w_s[j][ii]), a, acc[j]);
      }
    }
  }
  if (m >= M) return;
#pragma unroll
  for (int j = 0; j < kJB; ++j) {
    const int jj = j0 + j;
    if (jj >= td.n_count) break;
    const long long c_row = td.c_row0 + (td.n_list ? td.n_list[jj] + (td.relative ? jj : 0) : jj);
    uint16_t* dst = Ct + c_row * ldc + m;
    float v = alpha * acc[j];
    if (beta != 0.0f) v += beta * unpack1<DT>(*dst);
    const uint32_t p = pack2<DT>(v, 0.0f);
    *dst = static_cast<uint16_t>(p & 0xffffu);
  }
}

}  // namespace

cudaError_t masked_gemm_simt_launch(int dtype, const TileDesc* tiles, int n_tiles, const void* Wp,
                                    long long ldw, const void* At, long long lda, void* Ct,
                                    long long ldc, int M, float alpha, float beta,
                                    cudaStream_t stream) {
  if (n_tiles <= 0 || M <= 0) return cudaSuccess;
  dim3 grid((M + 255) / 256, n_tiles, 128 / kJB);
  auto kern = dtype == kBF16 ? masked_gemm_simt_kernel<kBF16> : masked_gemm_simt_kernel<kF16>;
  kern<<<grid, 256, 0, stream>>>(tiles, static_cast<const uint16_t*>(Wp), ldw,
                                 static_cast<const uint16_t*>(At), lda, static_cast<uint16_t*>(Ct),
                                 ldc, M, alpha, beta);
  return cudaGetLastError();
}

}  // namespace ts

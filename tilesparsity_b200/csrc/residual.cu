// Element-wise residual of TEW masks as a separate sparse term.
//
// The reference's TEW patterns (tw1m / tw2m, Pruning/VGG/prune_algo.py:151-191) add a small share of
// individual weights on top of the tile-wise mask; in the reference they only exist as extra ones in
// the dense 0/1 mask (its GPU driver has no kernel for them).  Here the tile-wise part runs on the
// tensor cores and the residual elements are applied afterwards as a sparse term:
//
//     Ct[n][m] (+)= alpha * sum over residual elements (k, n) of  W[k][n] * At[k][m]
//
// stored column-wise (CSC of W = CSR of W^T): col_ptr[N+1], row_idx[nnz] (k), val[nnz] (16-bit).
// With the batch contiguous in both At and Ct, one warp owns one output row segment Ct[n][m0..m0+256)
// and every non-zero adds a scaled, fully coalesced 512-byte piece of an At row to it: 2*M bytes of
// L2 -> SM traffic per non-zero, with no reuse a register file could exploit (the rows of different
// non-zeros are unrelated).  Measured on B200 (NMT LSTM shape, 125 829 non-zeros, M = 6400): SM
// instruction issue 71 %, L1 60 %, L2 53 % of peak -- issue-bound first, L2-bound right behind.
#include "ts_common.cuh"
#include "ts_kernels.h"

namespace ts {

namespace {

template <int DT>
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = unpack1<DT>(static_cast<uint16_t>(w[i] & 0xffffu));
    f[2 * i + 1] = unpack1<DT>(static_cast<uint16_t>(w[i] >> 16));
  }
}

// grid: (ceil(M / 256), ceil(N / 4)); block 128 = 4 warps, warp w handles column blockIdx.y*4 + w.
template <int DT>
__global__ void __launch_bounds__(128)
residual_spmm_kernel(const int* __restrict__ col_ptr, const int* __restrict__ row_idx,
                     const uint16_t* __restrict__ val, const uint8_t* __restrict__ col_written,
                     const uint16_t* __restrict__ At, long long lda, uint16_t* __restrict__ Ct,
                     long long ldc, int M, int N, float alpha) {
  const int n = blockIdx.y * 4 + (threadIdx.x >> 5);
  if (n >= N) return;
  const int p0 = col_ptr[n], p1 = col_ptr[n + 1];
  const bool written = col_written ? col_written[n] != 0 : true;
  if (p0 == p1 && written) return;       // nothing to add, the dense kernel's result stands
  const int m = blockIdx.x * 256 + (threadIdx.x & 31) * 8;
  if (m >= M) return;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  int p = p0;
  for (; p + 4 <= p1; p += 4) {
    uint4 a[4];
    uint16_t wraw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = __ldg(row_idx + p + u);
      wraw[u] = __ldg(val + p + u);
      a[u] = __ldg(reinterpret_cast<const uint4*>(At + static_cast<long long>(k) * lda + m));
    }
    if constexpr (DT == kF16) {
      // The kernel is bound by instruction issue (conversions and FMAs), not by L2: four products
      // at a time are summed with packed half-precision FMAs and join the fp32 accumulators as one
      // value, which halves the instruction count.  The four-term partial sum carries a relative
      // error of about 2^-10 of a term that is itself a small share of the output.
      __half2 part[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) part[i] = __float2half2_rn(0.0f);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const __half wh = *reinterpret_cast<const __half*>(&wraw[u]);
        const __half2 w2 = __half2half2(wh);
        const __half2* av = reinterpret_cast<const __half2*>(&a[u]);
#pragma unroll
        for (int i = 0; i < 4; ++i) part[i] = __hfma2(w2, av[i], part[i]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(part[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    } else {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float w = unpack1<DT>(wraw[u]);
        float f[8];
        unpack8<DT>(a[u], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(w, f[i], acc[i]);
      }
    }
  }
  for (; p < p1; ++p) {
    const int k = __ldg(row_idx + p);
    const float w = unpack1<DT>(__ldg(val + p));
    float f[8];
    unpack8<DT>(__ldg(reinterpret_cast<const uint4*>(At + static_cast<long long>(k) * lda + m)), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(w, f[i], acc[i]);
  }
  uint4* dst = reinterpret_cast<uint4*>(Ct + static_cast<long long>(n) * ldc + m);
  float base[8];
  if (written) {
    unpack8<DT>(*dst, base);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) base[i] = 0.0f;
  }
  uint4 o;
  o.x = pack2<DT>(base[0] + alpha * acc[0], base[1] + alpha * acc[1]);
  o.y = pack2<DT>(base[2] + alpha * acc[2], base[3] + alpha * acc[3]);
  o.z = pack2<DT>(base[4] + alpha * acc[4], base[5] + alpha * acc[5]);
  o.w = pack2<DT>(base[6] + alpha * acc[6], base[7] + alpha * acc[7]);
  *dst = o;
}

}  // namespace

cudaError_t residual_spmm_launch(int dtype, const int* col_ptr, const int* row_idx, const void* val,
                                 const uint8_t* col_written, const void* At, long long lda, void* Ct,
                                 long long ldc, int M, int N, float alpha, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return cudaSuccess;
  dim3 grid((M + 255) / 256, (N + 3) / 4);
  auto kern = dtype == kBF16 ? residual_spmm_kernel<kBF16> : residual_spmm_kernel<kF16>;
  kern<<<grid, 128, 0, stream>>>(col_ptr, row_idx, static_cast<const uint16_t*>(val), col_written,
                                 static_cast<const uint16_t*>(At), lda, static_cast<uint16_t*>(Ct), ldc, M, N,
                                 alpha);
  return cudaGetLastError();
}

}  // namespace ts

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
//
// Every non-zero needs one row piece of At per batch column: nnz * M * 2 bytes of operand reads, with
// no reuse a register file could exploit (the rows of different non-zeros are unrelated).  Two kernels:
//
//  * residual_slab_kernel (K * 64 bytes fit in shared memory): a persistent CTA copies the slab
//    At[0..K)[m0..m0+32) into shared memory once and serves every non-zero of its columns from there,
//    so the operand reads run at shared-memory instead of L2 bandwidth.  Work is split over the CTAs by
//    position in the (batch block, non-zero) sequence, i.e. balanced by non-zeros, at column granularity.
//  * residual_spmm_kernel (any K): one warp owns one output row segment Ct[n][m0..m0+256) and every
//    non-zero adds a scaled, fully coalesced 512-byte piece of an At row from L2 (2*M bytes per non-zero).
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
    float w[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = __ldg(row_idx + p + u);
      w[u] = unpack1<DT>(__ldg(val + p + u));
      a[u] = __ldg(reinterpret_cast<const uint4*>(At + static_cast<long long>(k) * lda + m));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float f[8];
      unpack8<DT>(a[u], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[u], f[i], acc[i]);
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

// Slab variant.  Block: 512 threads = 16 warps.  A warp works on 8 columns at a time: lane group
// g = lane / 4 takes column n, its 4 lanes cover the slab's 32 batch columns (8 each, 16 bytes).
constexpr int kSlabCols = 32;
constexpr int kSlabThreads = 512;

template <int DT>
__global__ void __launch_bounds__(kSlabThreads, 1)
residual_slab_kernel(const int* __restrict__ col_ptr, const int* __restrict__ row_idx,
                     const uint16_t* __restrict__ val, const uint8_t* __restrict__ col_written,
                     const uint16_t* __restrict__ At, long long lda, uint16_t* __restrict__ Ct,
                     long long ldc, int M, int N, int K, float alpha) {
  extern __shared__ __align__(16) uint8_t slab[];   // [K][64 bytes]
  const int m_blocks = (M + kSlabCols - 1) / kSlabCols;
  const long long nnz = col_ptr[N];
  // Position of column n of batch block b in the work sequence: b * (nnz + N) + col_ptr[n] + n
  // (one extra per column, so that empty columns, which may still need zero-filling, count too).
  const long long per_block = nnz + N;
  const long long total = per_block * m_blocks;
  const long long begin = total * blockIdx.x / gridDim.x;
  const long long end = total * (blockIdx.x + 1) / gridDim.x;
  if (begin >= end) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  for (int b = static_cast<int>(begin / per_block); b < m_blocks && b * per_block < end; ++b) {
    // columns of this batch block whose position lies in [begin, end)
    const long long lo = begin - b * per_block, hi = end - b * per_block;
    auto first_at_or_after = [&](long long pos) {   // smallest n with col_ptr[n] + n >= pos
      int a = 0, z = N;
      while (a < z) {
        const int mid = (a + z) >> 1;
        if (static_cast<long long>(__ldg(col_ptr + mid)) + mid >= pos) z = mid;
        else a = mid + 1;
      }
      return a;
    };
    const int n_lo = lo <= 0 ? 0 : first_at_or_after(lo);
    const int n_hi = hi >= per_block ? N : first_at_or_after(hi);
    if (n_lo >= n_hi) continue;
    const int m0 = b * kSlabCols;
    __syncthreads();   // everyone is done with the previous slab
    for (int i = threadIdx.x; i < K * 4; i += kSlabThreads) {
      const int k = i >> 2, c = i & 3;
      const int m = m0 + c * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < M) v = __ldg(reinterpret_cast<const uint4*>(At + static_cast<long long>(k) * lda + m));
      *reinterpret_cast<uint4*>(slab + k * 64 + c * 16) = v;
    }
    __syncthreads();
    const int m = m0 + q * 8;
    for (int n = n_lo + warp * 8 + g; n < n_hi; n += (kSlabThreads / 32) * 8) {
      const int p0 = __ldg(col_ptr + n), p1 = __ldg(col_ptr + n + 1);
      const bool written = col_written ? col_written[n] != 0 : true;
      if ((p0 == p1 && written) || m >= M) continue;
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
      int p = p0;
      for (; p + 4 <= p1; p += 4) {
        uint4 a[4];
        float w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int k = __ldg(row_idx + p + u);
          w[u] = unpack1<DT>(__ldg(val + p + u));
          a[u] = *reinterpret_cast<const uint4*>(slab + k * 64 + q * 16);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float f[8];
          unpack8<DT>(a[u], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[u], f[i], acc[i]);
        }
      }
      for (; p < p1; ++p) {
        const int k = __ldg(row_idx + p);
        const float w = unpack1<DT>(__ldg(val + p));
        float f[8];
        unpack8<DT>(*reinterpret_cast<const uint4*>(slab + k * 64 + q * 16), f);
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
  }
}

}  // namespace

cudaError_t residual_spmm_launch(int dtype, const int* col_ptr, const int* row_idx, const void* val,
                                 const uint8_t* col_written, const void* At, long long lda, void* Ct,
                                 long long ldc, int M, int N, int K, float alpha, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return cudaSuccess;
  const size_t slab_bytes = static_cast<size_t>(K) * 64;
  if (K > 0 && slab_bytes <= 200 * 1024) {
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    auto slab = dtype == kBF16 ? residual_slab_kernel<kBF16> : residual_slab_kernel<kF16>;
    e = cudaFuncSetAttribute(slab, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(slab_bytes));
    if (e != cudaSuccess) return e;
    slab<<<sms, kSlabThreads, slab_bytes, stream>>>(col_ptr, row_idx, static_cast<const uint16_t*>(val), col_written,
                                                   static_cast<const uint16_t*>(At), lda, static_cast<uint16_t*>(Ct),
                                                   ldc, M, N, K, alpha);
    return cudaGetLastError();
  }
  dim3 grid((M + 255) / 256, (N + 3) / 4);
  auto kern = dtype == kBF16 ? residual_spmm_kernel<kBF16> : residual_spmm_kernel<kF16>;
  kern<<<grid, 128, 0, stream>>>(col_ptr, row_idx, static_cast<const uint16_t*>(val), col_written,
                                 static_cast<const uint16_t*>(At), lda, static_cast<uint16_t*>(Ct), ldc, M, N,
                                 alpha);
  return cudaGetLastError();
}

}  // namespace ts

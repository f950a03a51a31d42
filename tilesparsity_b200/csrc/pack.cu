// Weight packing and 16-bit transpose.
//
// pack: builds the per-tile compacted weight matrix the masked GEMM consumes, the device-side
// counterpart of the reference's host loop gen_masked_stream_weight
// (StreamMaskedGEMM/perf/basic_nn.cu:757-769) and of the kernel compaction in exportPrunedModel
// (Pruning/BERT/utils/MyHook.py:76-85):  Wp[w_row0 + j][i] = W[kept_k[i]][kept_col(j)], K contiguous.
// Rows and K positions beyond the kept counts stay zero (the caller clears Wp before the launch).
// HBM-bound: reads the kept entries of W once, writes 2 bytes per kept entry.
//
// transpose16: out[c][r] = in[r][c] for 16-bit elements; turns a row-major activation matrix
// [M][K] into the K-major [K][M] layout the GEMM gathers from (the reference keeps its activations
// in that layout throughout, basic_nn.cu:823,1014).
#include "ts_common.cuh"
#include "ts_kernels.h"

namespace ts {

namespace {

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}

// grid: (ceil(max_k / 64), n_tiles); block 256.  Each block moves a 64 (kept rows) x 128 (kept
// columns) patch through shared memory so that both the read (along columns) and the write (along
// K) are coalesced.
template <typename TIn, int DT>
__global__ void __launch_bounds__(256)
pack_weights_kernel(const TIn* __restrict__ W, long long ld_w, const TileDesc* __restrict__ tiles,
                    uint16_t* __restrict__ Wp, long long ldw) {
  const TileDesc td = tiles[blockIdx.y];
  const int i0 = blockIdx.x * 64;
  if (i0 >= td.k_count) return;
  __shared__ uint16_t patch[64][130];
  const int tx = threadIdx.x & 127;   // column inside the tile
  const int ty = threadIdx.x >> 7;    // 0..1
  long long col = -1;
  if (tx < td.n_count) {
    col = td.c_row0 + (td.n_list ? td.n_list[tx] + (td.relative ? tx : 0) : tx);
  }
  for (int ii = ty; ii < 64; ii += 2) {
    const int i = i0 + ii;
    uint16_t v = 0;
    if (i < td.k_count && col >= 0) {
      const int kk = td.k_list[i] + (td.relative ? i : 0);
      const float f = load_as_float<TIn>(W + static_cast<long long>(kk) * ld_w + col);
      v = static_cast<uint16_t>(pack2<DT>(f, 0.0f) & 0xffffu);
    }
    patch[ii][tx] = v;
  }
  __syncthreads();
  const int wi = threadIdx.x & 63;    // K position inside the patch
  const int wj = threadIdx.x >> 6;    // 0..3
  if (i0 + wi < td.k_count) {
    for (int j = wj; j < td.n_count; j += 4) {
      Wp[static_cast<long long>(td.w_row0 + j) * ldw + i0 + wi] = patch[wi][j];
    }
  }
}

__global__ void __launch_bounds__(256)
transpose16_kernel(const uint16_t* __restrict__ in, long long ld_in, uint16_t* __restrict__ out,
                   long long ld_out, int rows, int cols) {
  __shared__ uint16_t t[64][66];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int rr = ty; rr < 64; rr += 4) {
    const int r = r0 + rr, c = c0 + tx;
    t[rr][tx] = (r < rows && c < cols) ? in[static_cast<long long>(r) * ld_in + c] : 0;
  }
  __syncthreads();
  for (int cc = ty; cc < 64; cc += 4) {
    const int c = c0 + cc, r = r0 + tx;
    if (c < cols && r < rows) out[static_cast<long long>(c) * ld_out + r] = t[tx][cc];
  }
}

}  // namespace

cudaError_t pack_weights_launch(int w_dtype, int out_dtype, const void* W, long long ld_w,
                                const TileDesc* tiles, int n_tiles, int max_k, void* Wp,
                                long long ldw, cudaStream_t stream) {
  if (n_tiles <= 0 || max_k <= 0) return cudaSuccess;
  dim3 grid((max_k + 63) / 64, n_tiles);
  uint16_t* out = static_cast<uint16_t*>(Wp);
#define TS_PACK(TIN, DT) \
  pack_weights_kernel<TIN, DT><<<grid, 256, 0, stream>>>(static_cast<const TIN*>(W), ld_w, tiles, out, ldw)
  if (out_dtype == kBF16) {
    if (w_dtype == kF32) TS_PACK(float, kBF16);
    else if (w_dtype == kF16) TS_PACK(__half, kBF16);
    else TS_PACK(__nv_bfloat16, kBF16);
  } else {
    if (w_dtype == kF32) TS_PACK(float, kF16);
    else if (w_dtype == kF16) TS_PACK(__half, kF16);
    else TS_PACK(__nv_bfloat16, kF16);
  }
#undef TS_PACK
  return cudaGetLastError();
}

cudaError_t transpose16_launch(const void* in, long long ld_in, void* out, long long ld_out,
                               int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  transpose16_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(in), ld_in,
                                               static_cast<uint16_t*>(out), ld_out, rows, cols);
  return cudaGetLastError();
}

}  // namespace ts

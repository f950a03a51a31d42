// Front end and back end of the implicit-GEMM convolution.
//
// The reference prunes conv kernels as 2-D matrices [(kh*kw*cin), cout] with row index
// k = (r*kw + j)*cin + c (img2col_forward, Pruning/VGG/prune_algo.py:16-24), which makes a stride-1
// same-padded convolution the masked GEMM  C = im2col(X) . (W .* mask).  The im2col matrix is kh*kw
// times the input and is never built here.  Instead the input is stored once per horizontal tap:
//
//   planes[j][c][b*Hp*Wp + y*Wp + x] = Xpad[b][y][x + j][c]        j in [0, kw), c in [0, cin)
//
// (Xpad: the image with (kh-1)/2 rows and (kw-1)/2 columns of zeros in front; Hp = H + kh - 1 rows;
// Wp = W + kw - 1 rounded up to a multiple of 8 columns; zeros where the index leaves the image).
// Row k of the im2col matrix, for the output pixel at m = b*Hp*Wp + y*Wp + x, is then
// planes[j][c][m + r*Wp]: a contiguous run that starts on a 16-byte boundary for every (r, j, c).
// The masked GEMM gathers those runs exactly as it gathers the rows of an activation matrix; its
// output Ct[cout][m] lives in the same padded pixel space (positions with y >= H or x >= W are scratch).
#include "ts_common.cuh"
#include "ts_kernels.h"

namespace ts {

namespace {

constexpr int kPackCh = 64;    // channels per block
constexpr int kPackPx = 64;    // padded pixels of one image row per pass

// grid (Hp, B, ceil(C / 64)), block 256.  One block: one padded image row of one image, 64 channels.
__global__ void __launch_bounds__(256)
conv_pack_input_kernel(const uint16_t* __restrict__ x, int B, int H, int W, int C, int kh, int kw, int Hp, int Wp,
                       uint16_t* __restrict__ planes, long long plane_ld) {
  __shared__ uint16_t tile[kPackPx + 8][kPackCh + 2];   // [padded column][channel]
  const int yp = blockIdx.x, b = blockIdx.y, c0 = blockIdx.z * kPackCh;
  const int y = yp - (kh - 1) / 2, pw = (kw - 1) / 2;
  const bool row_in = y >= 0 && y < H;
  const long long out_row = (static_cast<long long>(b) * Hp + yp) * Wp;
  for (int x0 = 0; x0 < Wp; x0 += kPackPx) {
    // padded columns x0 .. x0 + 64 + kw - 1 of this row, all 64 channels (channels fastest in x)
    const int span = kPackPx + kw - 1;
    __syncthreads();
    for (int i = threadIdx.x; i < span * kPackCh; i += blockDim.x) {
      const int cc = i % kPackCh, xx = i / kPackCh;
      const int xs = x0 + xx - pw;                     // source column in the image
      uint16_t v = 0;
      if (row_in && xs >= 0 && xs < W && c0 + cc < C) {
        v = __ldg(x + ((static_cast<long long>(b) * H + y) * W + xs) * C + c0 + cc);
      }
      tile[xx][cc] = v;
    }
    __syncthreads();
    const int n_px = min(kPackPx, Wp - x0);
    for (int i = threadIdx.x; i < kw * kPackCh * kPackPx; i += blockDim.x) {
      const int px = i % kPackPx, cc = (i / kPackPx) % kPackCh, j = i / (kPackPx * kPackCh);
      if (px < n_px && c0 + cc < C) {
        planes[(static_cast<long long>(j) * C + c0 + cc) * plane_ld + out_row + x0 + px] = tile[px + j][cc];
      }
    }
  }
}

// y[b][yy][xx][n] = Ct[n][b*Hp*Wp + yy*Wp + xx] for yy < H, xx < W.  grid (H, B, ceil(N / 64)), block 256.
__global__ void __launch_bounds__(256)
conv_unpack_output_kernel(const uint16_t* __restrict__ ct, long long ldc, int B, int H, int W, int Hp, int Wp, int N,
                          uint16_t* __restrict__ y) {
  __shared__ uint16_t tile[kPackCh][kPackPx + 2];       // [output channel][column]
  const int yy = blockIdx.x, b = blockIdx.y, n0 = blockIdx.z * kPackCh;
  const long long in_row = (static_cast<long long>(b) * Hp + yy) * Wp;
  for (int x0 = 0; x0 < W; x0 += kPackPx) {
    const int n_px = min(kPackPx, W - x0);
    __syncthreads();
    for (int i = threadIdx.x; i < kPackCh * kPackPx; i += blockDim.x) {
      const int px = i % kPackPx, nn = i / kPackPx;
      if (px < n_px && n0 + nn < N) tile[nn][px] = __ldg(ct + static_cast<long long>(n0 + nn) * ldc + in_row + x0 + px);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kPackCh * kPackPx; i += blockDim.x) {
      const int nn = i % kPackCh, px = i / kPackCh;
      if (px < n_px && n0 + nn < N) {
        y[((static_cast<long long>(b) * H + yy) * W + x0 + px) * N + n0 + nn] = tile[nn][px];
      }
    }
  }
}

}  // namespace

cudaError_t conv_pack_input_launch(const void* x_nhwc, int B, int H, int W, int C, int kh, int kw, int Hp, int Wp,
                                   void* planes, long long plane_ld, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0) return cudaSuccess;
  // the tail of every plane past the last image (read by the lowest kernel rows of the last pixels)
  const long long m_pad = static_cast<long long>(B) * Hp * Wp;
  if (plane_ld > m_pad) {
    cudaError_t e = cudaMemset2DAsync(static_cast<uint16_t*>(planes) + m_pad, plane_ld * 2, 0, (plane_ld - m_pad) * 2,
                                      static_cast<size_t>(kw) * C, stream);
    if (e != cudaSuccess) return e;
  }
  dim3 grid(Hp, B, (C + kPackCh - 1) / kPackCh);
  conv_pack_input_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x_nhwc), B, H, W, C, kh, kw, Hp, Wp,
                                                   static_cast<uint16_t*>(planes), plane_ld);
  return cudaGetLastError();
}

cudaError_t conv_unpack_output_launch(const void* ct, long long ldc, int B, int H, int W, int Hp, int Wp, int N,
                                      void* y_nhwc, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || W <= 0 || N <= 0) return cudaSuccess;
  dim3 grid(H, B, (N + kPackCh - 1) / kPackCh);
  conv_unpack_output_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(ct), ldc, B, H, W, Hp, Wp, N,
                                                      static_cast<uint16_t*>(y_nhwc));
  return cudaGetLastError();
}

}  // namespace ts

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
constexpr int kPackRows = 4;   // padded image rows per pass
constexpr int kTilePitch = kPackPx + 10;   // halves per tile row: 37 words, odd, so a column is conflict-free

// grid (ceil(Hp / 4), B, ceil(C / 64)), block 256.  One pass: 4 padded image rows x 64 columns of one
// image, 64 channels.  The input is read with 16-byte loads along the channels, transposed through
// shared memory, and every plane row leaves with 16-byte stores along the pixels (Wp, the row
// starts and plane_ld are multiples of 8 elements).  Needs C % 8 == 0 and 16-byte aligned pointers.
__global__ void __launch_bounds__(256)
conv_pack_input_kernel(const uint16_t* __restrict__ x, int B, int H, int W, int C, int kh, int kw, int Hp, int Wp,
                       uint16_t* __restrict__ planes, long long plane_ld) {
  __shared__ __align__(16) uint16_t tile[kPackRows][kPackCh][kTilePitch];   // [row][channel][padded column]
  const int yp0 = blockIdx.x * kPackRows, b = blockIdx.y, c0 = blockIdx.z * kPackCh;
  const int ph = (kh - 1) / 2, pw = (kw - 1) / 2;
  const int span = kPackPx + kw - 1;
  for (int x0 = 0; x0 < Wp; x0 += kPackPx) {
    __syncthreads();
    // loads: (row, padded column, 8 channels) per thread and step
    for (int i = threadIdx.x; i < kPackRows * span * (kPackCh / 8); i += blockDim.x) {
      const int c8 = i % (kPackCh / 8), xx = (i / (kPackCh / 8)) % span, rr = i / ((kPackCh / 8) * span);
      const int y = yp0 + rr - ph, xs = x0 + xx - pw;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (y >= 0 && y < H && xs >= 0 && xs < W && c0 + c8 * 8 < C) {
        v = __ldg(reinterpret_cast<const uint4*>(x + ((static_cast<long long>(b) * H + y) * W + xs) * C + c0 + c8 * 8));
      }
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        tile[rr][c8 * 8 + 2 * e][xx] = static_cast<uint16_t>(w[e] & 0xffffu);
        tile[rr][c8 * 8 + 2 * e + 1][xx] = static_cast<uint16_t>(w[e] >> 16);
      }
    }
    __syncthreads();
    const int n_px8 = (min(kPackPx, Wp - x0) + 7) / 8;
    for (int i = threadIdx.x; i < kPackRows * kw * kPackCh * n_px8; i += blockDim.x) {
      const int p8 = i % n_px8, cc = (i / n_px8) % kPackCh, j = (i / (n_px8 * kPackCh)) % kw;
      const int rr = i / (n_px8 * kPackCh * kw);
      const int yp = yp0 + rr;
      if (yp >= Hp || c0 + cc >= C) continue;
      const uint16_t* src = &tile[rr][cc][p8 * 8 + j];
      uint4 o;
      o.x = src[0] | (static_cast<uint32_t>(src[1]) << 16);
      o.y = src[2] | (static_cast<uint32_t>(src[3]) << 16);
      o.z = src[4] | (static_cast<uint32_t>(src[5]) << 16);
      o.w = src[6] | (static_cast<uint32_t>(src[7]) << 16);
      const long long off = (static_cast<long long>(j) * C + c0 + cc) * plane_ld +
                            (static_cast<long long>(b) * Hp + yp) * Wp + x0 + p8 * 8;
      *reinterpret_cast<uint4*>(planes + off) = o;
    }
  }
}

// y[b][yy][xx][n] = Ct[n][b*Hp*Wp + yy*Wp + xx] for yy < H, xx < W.  grid (ceil(H / 4), B, ceil(N / 64)),
// block 256: 16-byte loads along the pixels, 16-byte stores along the channels.  Needs N % 8 == 0,
// ldc % 8 == 0 and 16-byte aligned pointers.
__global__ void __launch_bounds__(256)
conv_unpack_output_kernel(const uint16_t* __restrict__ ct, long long ldc, int B, int H, int W, int Hp, int Wp, int N,
                          uint16_t* __restrict__ y) {
  __shared__ __align__(16) uint16_t tile[kPackRows][kPackCh][kTilePitch];   // [row][output channel][column]
  const int y0 = blockIdx.x * kPackRows, b = blockIdx.y, n0 = blockIdx.z * kPackCh;
  for (int x0 = 0; x0 < W; x0 += kPackPx) {
    const int n_px = min(kPackPx, W - x0);
    const int n_px8 = (n_px + 7) / 8;      // Wp is a multiple of 8, so whole groups stay inside the padded row
    __syncthreads();
    for (int i = threadIdx.x; i < kPackRows * kPackCh * n_px8; i += blockDim.x) {
      const int p8 = i % n_px8, nn = (i / n_px8) % kPackCh, rr = i / (n_px8 * kPackCh);
      if (y0 + rr >= H || n0 + nn >= N) continue;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(
          ct + static_cast<long long>(n0 + nn) * ldc + (static_cast<long long>(b) * Hp + y0 + rr) * Wp + x0 + p8 * 8));
      uint32_t* dst = reinterpret_cast<uint32_t*>(&tile[rr][nn][p8 * 8]);   // 4-byte aligned (odd word pitch)
      dst[0] = v.x;
      dst[1] = v.y;
      dst[2] = v.z;
      dst[3] = v.w;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kPackRows * n_px * (kPackCh / 8); i += blockDim.x) {
      const int n8 = i % (kPackCh / 8), px = (i / (kPackCh / 8)) % n_px, rr = i / ((kPackCh / 8) * n_px);
      if (y0 + rr >= H || n0 + n8 * 8 >= N) continue;
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        w[e] = tile[rr][n8 * 8 + 2 * e][px] | (static_cast<uint32_t>(tile[rr][n8 * 8 + 2 * e + 1][px]) << 16);
      }
      *reinterpret_cast<uint4*>(y + ((static_cast<long long>(b) * H + y0 + rr) * W + x0 + px) * N + n0 + n8 * 8) =
          make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// Padded-space output of one convolution -> input planes of the next (same image size and padding
// geometry): planes[j][c][m] = Ct[c][m - ph*Wp + j - pw] where that position is a real pixel, else 0.
// Both sides are channel-major, so this is a shifted, masked copy: 16-byte stores, the one-pixel
// shifts of the taps assembled from two aligned 16-byte loads.  grid (ceil(m_pad / 8 / 256), C, kw).
__global__ void __launch_bounds__(256)
conv_repack_kernel(const uint16_t* __restrict__ ct, long long ldc, int H, int W, int Hp, int Wp, int kh, int kw,
                   long long m_pad, uint16_t* __restrict__ planes, long long plane_ld, int C) {
  const long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;   // group of 8 padded pixels
  const long long m0 = g * 8;
  if (m0 >= m_pad) return;
  const int c = blockIdx.y, j = blockIdx.z;
  const int ph = (kh - 1) / 2, pw = (kw - 1) / 2;
  const int x0 = static_cast<int>(m0 % Wp);
  const int yp = static_cast<int>((m0 / Wp) % Hp);
  const int y = yp - ph;
  uint16_t out[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) out[e] = 0;
  if (y >= 0 && y < H) {
    const long long s0 = m0 - static_cast<long long>(ph) * Wp + (j - pw);   // source index of element 0
    const uint16_t* row = ct + static_cast<long long>(c) * ldc;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int xs = x0 + e + j - pw;
      if (xs >= 0 && xs < W) out[e] = __ldg(row + s0 + e);
    }
  }
  uint4 o;
  o.x = out[0] | (static_cast<uint32_t>(out[1]) << 16);
  o.y = out[2] | (static_cast<uint32_t>(out[3]) << 16);
  o.z = out[4] | (static_cast<uint32_t>(out[5]) << 16);
  o.w = out[6] | (static_cast<uint32_t>(out[7]) << 16);
  *reinterpret_cast<uint4*>(planes + (static_cast<long long>(j) * C + c) * plane_ld + m0) = o;
}

}  // namespace

cudaError_t conv_repack_launch(const void* ct, long long ldc, int B, int H, int W, int Hp, int Wp, int kh, int kw,
                               int C, void* planes, long long plane_ld, cudaStream_t stream) {
  if (B <= 0 || C <= 0) return cudaSuccess;
  const long long m_pad = static_cast<long long>(B) * Hp * Wp;
  if (plane_ld > m_pad) {
    cudaError_t e = cudaMemset2DAsync(static_cast<uint16_t*>(planes) + m_pad, plane_ld * 2, 0, (plane_ld - m_pad) * 2,
                                      static_cast<size_t>(kw) * C, stream);
    if (e != cudaSuccess) return e;
  }
  dim3 grid(static_cast<unsigned>((m_pad / 8 + 255) / 256), C, kw);
  conv_repack_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(ct), ldc, H, W, Hp, Wp, kh, kw, m_pad,
                                               static_cast<uint16_t*>(planes), plane_ld, C);
  return cudaGetLastError();
}

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
  dim3 grid((Hp + kPackRows - 1) / kPackRows, B, (C + kPackCh - 1) / kPackCh);
  conv_pack_input_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x_nhwc), B, H, W, C, kh, kw, Hp, Wp,
                                                   static_cast<uint16_t*>(planes), plane_ld);
  return cudaGetLastError();
}

cudaError_t conv_unpack_output_launch(const void* ct, long long ldc, int B, int H, int W, int Hp, int Wp, int N,
                                      void* y_nhwc, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || W <= 0 || N <= 0) return cudaSuccess;
  dim3 grid((H + kPackRows - 1) / kPackRows, B, (N + kPackCh - 1) / kPackCh);
  conv_unpack_output_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(ct), ldc, B, H, W, Hp, Wp, N,
                                                      static_cast<uint16_t*>(y_nhwc));
  return cudaGetLastError();
}

}  // namespace ts

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
#include <algorithm>

#include "ts_common.cuh"
#include "ts_kernels.h"

namespace ts {

namespace {

constexpr int kPackCh = 64;    // channels per block
constexpr int kPackPx = 64;    // padded pixels of one image row per pass
constexpr int kPackRows = 4;   // padded image rows per pass
constexpr int kTilePitch = kPackPx + 10;   // halves per tile row: 37 words, odd, so a column is conflict-free
// halves between the image rows of a tile: 8 words past a multiple of 32, so that lanes which differ in
// the image row (0..3), the channel (4 neighbours) and the 8-pixel group (0..1) hit 32 different banks
constexpr int kTileRow = kPackCh * kTilePitch + 16;

// Division of a small index by a small run-time divisor without the integer-division sequence (the
// pack kernel was bound by its index arithmetic): floor(i / d) = umulhi(i, ceil(2^32 / d)) for
// d <= 2^16 and i < 2^16.
struct SmallDiv {
  uint32_t mul, d;
  __device__ __forceinline__ explicit SmallDiv(int div) : mul(div > 1 ? 0xffffffffu / static_cast<uint32_t>(div) + 1u : 0u),
                                                          d(static_cast<uint32_t>(div)) {}
  __device__ __forceinline__ int quot(int i) const { return d > 1 ? static_cast<int>(__umulhi(static_cast<uint32_t>(i), mul)) : i; }
};

// grid (ceil(Hp / 4), B, ceil(C / 64)), block 256.  One pass: 4 padded image rows x 64 columns of one
// image, 64 channels.  The input is read with 16-byte loads along the channels, transposed through
// shared memory, and every plane row leaves with 16-byte stores along the pixels (Wp, the row
// starts and plane_ld are multiples of 8 elements).  Needs C % 8 == 0 and 16-byte aligned pointers.
__global__ void __launch_bounds__(256)
conv_pack_input_kernel(const uint16_t* __restrict__ x, int B, int H, int W, int C, int kh, int kw, int Hp, int Wp,
                       uint16_t* __restrict__ planes, long long plane_ld) {
  __shared__ __align__(16) uint16_t tile[kPackRows * kTileRow];   // [row][channel][padded column]
  const int yp0 = blockIdx.x * kPackRows, b = blockIdx.y, c0 = blockIdx.z * kPackCh;
  const int ph = (kh - 1) / 2, pw = (kw - 1) / 2;
  const int span = kPackPx + kw - 1;
  for (int x0 = 0; x0 < Wp; x0 += kPackPx) {
    __syncthreads();
    // The copy-out below reads columns [0, n_px8 * 8 + kw - 1) of every tile row.  Zero them (halo, the
    // rows above and below the image, the padding of Wp), then load only the pixels that exist: for a
    // 14-pixel image row that is a fifth of the pass's 64 + kw - 1 columns.
    const int n_cols = min(span, ((min(kPackPx, Wp - x0) + 7) / 8) * 8 + kw - 1);
    const int n_w32 = (n_cols + 1) / 2;
    const SmallDiv by_w32(n_w32);
    for (int i = threadIdx.x; i < kPackRows * kPackCh * n_w32; i += blockDim.x) {
      const int rc = by_w32.quot(i), w32 = i - rc * n_w32;
      reinterpret_cast<uint32_t*>(tile + (rc / kPackCh) * kTileRow + (rc % kPackCh) * kTilePitch)[w32] = 0u;
    }
    __syncthreads();
    const int xx_lo = max(0, pw - x0), xx_hi = min(n_cols, W + pw - x0);   // padded columns that hold pixels
    const int rr_lo = max(0, ph - yp0), rr_hi = min(kPackRows, H + ph - yp0);
    const int n_xx = xx_hi - xx_lo, n_rr = rr_hi - rr_lo;
    if (n_xx > 0 && n_rr > 0) {
      // loads: (row, padded column, 8 channels) per thread and step
      const SmallDiv by_xx(n_xx);
      for (int i = threadIdx.x; i < n_rr * n_xx * (kPackCh / 8); i += blockDim.x) {
        const int c8 = i % (kPackCh / 8), px = i / (kPackCh / 8), r_ = by_xx.quot(px);
        const int xx = xx_lo + px - r_ * n_xx, rr = rr_lo + r_;
        if (c0 + c8 * 8 >= C) continue;
        const int y = yp0 + rr - ph, xs = x0 + xx - pw;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + ((static_cast<long long>(b) * H + y) * W + xs) * C + c0 + c8 * 8));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          tile[rr * kTileRow + (c8 * 8 + 2 * e) * kTilePitch + xx] = static_cast<uint16_t>(w[e] & 0xffffu);
          tile[rr * kTileRow + (c8 * 8 + 2 * e + 1) * kTilePitch + xx] = static_cast<uint16_t>(w[e] >> 16);
        }
      }
    }
    __syncthreads();
    const int n_px8 = (min(kPackPx, Wp - x0) + 7) / 8;
    // lanes run over the 8-pixel groups of a row first, then over the image rows: where a padded row is
    // narrower than the pass (small images) consecutive rows are consecutive in the plane, and a warp's
    // stores fall into a few long runs instead of one 16-byte piece per channel
    const SmallDiv by_px8(n_px8);
    for (int i = threadIdx.x; i < kPackRows * kw * kPackCh * n_px8; i += blockDim.x) {
      const int q_ = by_px8.quot(i), p8 = i - q_ * n_px8;
      const int rr = q_ % kPackRows, cc = (q_ / kPackRows) % kPackCh, j = q_ / (kPackRows * kPackCh);
      const int yp = yp0 + rr;
      if (yp >= Hp || c0 + cc >= C) continue;
      const uint16_t* src = &tile[rr * kTileRow + cc * kTilePitch + p8 * 8 + j];
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

// The same packing without shared memory, for images whose padded pixel count stays below the range of
// the reciprocal divisions: a thread takes one group of 8 padded pixels and 8 channels, reads the
// 8 + KW - 1 input pixels the group's taps touch (16 bytes = 8 channels each; zeros outside the image),
// transposes them in registers (two byte permutes per output word) and writes, for every tap and every
// one of its channels, the 8 pixels as one 16-byte store.  Lanes run along the pixel groups, so a warp's
// store instruction covers 512 contiguous bytes of one plane row; the loads of a warp touch 32 pixels,
// whose other channels neighbouring blocks (blockIdx.y) pick up from L2.  Threads past the last image
// zero the planes' tails.  grid (ceil(plane_ld / 8 / 128), C / 8), block 128.
template <int KW>
__global__ void __launch_bounds__(128)
conv_pack_input_reg_kernel(const uint16_t* __restrict__ x, int H, int W, int C, int kh, int Hp, int Wp,
                           int n_groups, int n_groups_ld, uint32_t mul_wp8, uint32_t mul_hp,
                           uint16_t* __restrict__ planes, long long plane_ld) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;   // group of 8 padded pixels
  if (g >= n_groups_ld) return;
  const int c0 = blockIdx.y * 8;
  const long long m0 = static_cast<long long>(g) << 3;
  if (g >= n_groups) {
#pragma unroll
    for (int j = 0; j < KW; ++j) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        *reinterpret_cast<uint4*>(planes + (static_cast<long long>(j) * C + c0 + c) * plane_ld + m0) = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }
  constexpr int PW = (KW - 1) / 2;
  const int ph = (kh - 1) / 2;
  const int wp8 = Wp >> 3;
  const int row = mul_wp8 ? static_cast<int>(__umulhi(static_cast<uint32_t>(g), mul_wp8)) : g;   // padded image row, all images
  const int x0 = (g - row * wp8) << 3;
  const int img = mul_hp ? static_cast<int>(__umulhi(static_cast<uint32_t>(row), mul_hp)) : row;
  const int y = row - img * Hp - ph;
  uint4 px[8 + KW - 1];
  const bool row_ok = y >= 0 && y < H;
  const uint16_t* src = x + ((static_cast<long long>(img) * H + (row_ok ? y : 0)) * W) * C + c0;
#pragma unroll
  for (int k = 0; k < 8 + KW - 1; ++k) {
    const int xs = x0 + k - PW;
    px[k] = (row_ok && xs >= 0 && xs < W) ? __ldg(reinterpret_cast<const uint4*>(src + static_cast<long long>(xs) * C))
                                          : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int j = 0; j < KW; ++j) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {           // channel pair (2q, 2q + 1): word q of every pixel
      uint32_t lo[4], hi[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {         // pixels 2t, 2t + 1 of the tap's window
        const uint4 a = px[j + 2 * t], b = px[j + 2 * t + 1];
        const uint32_t wa = q == 0 ? a.x : (q == 1 ? a.y : (q == 2 ? a.z : a.w));
        const uint32_t wb = q == 0 ? b.x : (q == 1 ? b.y : (q == 2 ? b.z : b.w));
        lo[t] = __byte_perm(wa, wb, 0x5410);
        hi[t] = __byte_perm(wa, wb, 0x7632);
      }
      uint16_t* dst = planes + (static_cast<long long>(j) * C + c0 + 2 * q) * plane_ld + m0;
      *reinterpret_cast<uint4*>(dst) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      *reinterpret_cast<uint4*>(dst + plane_ld) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    }
  }
}

// y[b][yy][xx][n] = Ct[n][b*Hp*Wp + yy*Wp + xx] for yy < H, xx < W.  grid (ceil(H / 4), B, ceil(N / 64)),
// block 256: 16-byte loads along the pixels, 16-byte stores along the channels.  Needs N % 8 == 0,
// ldc % 8 == 0 and 16-byte aligned pointers.
__global__ void __launch_bounds__(256)
conv_unpack_output_kernel(const uint16_t* __restrict__ ct, long long ldc, int B, int H, int W, int Hp, int Wp, int N,
                          uint16_t* __restrict__ y) {
  __shared__ __align__(16) uint16_t tile[kPackRows * kTileRow];   // [row][output channel][column]
  const int y0 = blockIdx.x * kPackRows, b = blockIdx.y, n0 = blockIdx.z * kPackCh;
  for (int x0 = 0; x0 < W; x0 += kPackPx) {
    const int n_px = min(kPackPx, W - x0);
    const int n_px8 = (n_px + 7) / 8;      // Wp is a multiple of 8, so whole groups stay inside the padded row
    __syncthreads();
    const SmallDiv by_px8(n_px8), by_px(n_px);
    for (int i = threadIdx.x; i < kPackRows * kPackCh * n_px8; i += blockDim.x) {
      const int q_ = by_px8.quot(i), p8 = i - q_ * n_px8;
      const int rr = q_ % kPackRows, nn = q_ / kPackRows;   // rows before channels, as in the pack
      if (y0 + rr >= H || n0 + nn >= N) continue;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(
          ct + static_cast<long long>(n0 + nn) * ldc + (static_cast<long long>(b) * Hp + y0 + rr) * Wp + x0 + p8 * 8));
      uint32_t* dst = reinterpret_cast<uint32_t*>(&tile[rr * kTileRow + nn * kTilePitch + p8 * 8]);   // 4-byte aligned (odd word pitch)
      dst[0] = v.x;
      dst[1] = v.y;
      dst[2] = v.z;
      dst[3] = v.w;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kPackRows * n_px * (kPackCh / 8); i += blockDim.x) {
      const int n8 = i % (kPackCh / 8), pq = i / (kPackCh / 8), rr = by_px.quot(pq), px = pq - rr * n_px;
      if (y0 + rr >= H || n0 + n8 * 8 >= N) continue;
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        w[e] = tile[rr * kTileRow + (n8 * 8 + 2 * e) * kTilePitch + px] |
               (static_cast<uint32_t>(tile[rr * kTileRow + (n8 * 8 + 2 * e + 1) * kTilePitch + px]) << 16);
      }
      *reinterpret_cast<uint4*>(y + ((static_cast<long long>(b) * H + y0 + rr) * W + x0 + px) * N + n0 + n8 * 8) =
          make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// The unpacking without shared memory: a thread takes one group of 8 padded pixels and 8 output channels,
// reads the 8 channel rows (16 bytes each, a warp 512 contiguous bytes per row), transposes in registers
// and writes the pixels that exist as 16-byte pieces of their NHWC rows (the neighbouring channel blocks
// complete the sectors in L2).  grid (ceil(m_pad / 8 / 128), N / 8), block 128.
__global__ void __launch_bounds__(128)
conv_unpack_output_reg_kernel(const uint16_t* __restrict__ ct, long long ldc, int H, int W, int Hp, int Wp, int N,
                              int n_groups, uint32_t mul_wp8, uint32_t mul_hp, uint16_t* __restrict__ y) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;   // group of 8 padded pixels
  if (g >= n_groups) return;
  const int n0 = blockIdx.y * 8;
  const int wp8 = Wp >> 3;
  const int row = mul_wp8 ? static_cast<int>(__umulhi(static_cast<uint32_t>(g), mul_wp8)) : g;
  const int x0 = (g - row * wp8) << 3;
  const int img = mul_hp ? static_cast<int>(__umulhi(static_cast<uint32_t>(row), mul_hp)) : row;
  const int yy = row - img * Hp;
  if (yy >= H || x0 >= W) return;                         // scratch rows and columns of the padded space
  const uint4* src = reinterpret_cast<const uint4*>(ct + static_cast<long long>(n0) * ldc) + g;
  const long long ld8 = ldc >> 3;
  uint4 ch[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) ch[c] = __ldg(src + c * ld8);
  uint16_t* dst = y + ((static_cast<long long>(img) * H + yy) * W + x0) * N + n0;
#pragma unroll
  for (int t = 0; t < 4; ++t) {           // pixels 2t, 2t + 1: word t of every channel row
    uint32_t lo[4], hi[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {         // channels 2q, 2q + 1
      const uint4 a = ch[2 * q], b = ch[2 * q + 1];
      const uint32_t wa = t == 0 ? a.x : (t == 1 ? a.y : (t == 2 ? a.z : a.w));
      const uint32_t wb = t == 0 ? b.x : (t == 1 ? b.y : (t == 2 ? b.z : b.w));
      lo[q] = __byte_perm(wa, wb, 0x5410);
      hi[q] = __byte_perm(wa, wb, 0x7632);
    }
    if (x0 + 2 * t < W) *reinterpret_cast<uint4*>(dst + static_cast<long long>(2 * t) * N) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    if (x0 + 2 * t + 1 < W) *reinterpret_cast<uint4*>(dst + static_cast<long long>(2 * t + 1) * N) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
  }
}

// Padded-space output of one convolution -> input planes of the next (same image size and padding
// geometry): planes[j][c][m] = Ct[c][m - ph*Wp + j - pw] where that position is a real pixel, else 0.
// Both sides are channel-major, so this is a shifted, masked copy with 16-byte stores.  The source of
// a group of 8 pixels starts d = j - pw elements off a 16-byte boundary: one 16-byte load for d = 0,
// otherwise five aligned 32-bit words, realigned by a funnel shift when d is odd.  The position of a
// group inside its image row and image comes from two reciprocal multiplications (the 64-bit
// divisions this kernel started with cost more than its memory traffic).
// grid (ceil(plane_ld / 8 / 256), ceil(C / 8), kw), eight channels per thread; (m_pad / 8) * max(Wp / 8, Hp) < 2^32.
constexpr int kRepackCh = 8;
__global__ void __launch_bounds__(256)
conv_repack_kernel(const uint16_t* __restrict__ ct, long long ldc, int H, int W, int Hp, int Wp, int kh, int kw,
                   int n_groups, int n_groups_ld, uint32_t mul_wp8, uint32_t mul_hp,
                   uint16_t* __restrict__ planes, long long plane_ld, int C) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;   // group of 8 padded pixels
  if (g >= n_groups_ld) return;
  const int c_begin = blockIdx.y * kRepackCh, c_end = min(C, c_begin + kRepackCh), j = blockIdx.z;
  if (g >= n_groups) {
    // the tail of every plane past the last image (read by the lowest kernel rows of the last pixels)
    for (int c = c_begin; c < c_end; ++c) {
      *reinterpret_cast<uint4*>(planes + (static_cast<long long>(j) * C + c) * plane_ld + (static_cast<long long>(g) << 3)) =
          make_uint4(0, 0, 0, 0);
    }
    return;
  }
  const int ph = (kh - 1) / 2, pw = (kw - 1) / 2;
  const int wp8 = Wp >> 3;
  // (a multiplier of 0 stands for a divisor of 1)
  const int row = mul_wp8 ? static_cast<int>(__umulhi(static_cast<uint32_t>(g), mul_wp8)) : g;   // padded image row, all images
  const int x0 = (g - row * wp8) << 3;
  const int img = mul_hp ? static_cast<int>(__umulhi(static_cast<uint32_t>(row), mul_hp)) : row;
  const int y = row - img * Hp - ph;
  const long long m0 = static_cast<long long>(g) << 3;
  const int d = j - pw;
  const bool inside = y >= 0 && y < H && x0 + d < W && x0 + 7 + d >= 0;
#pragma unroll 4
  for (int c = c_begin; c < c_end; ++c) {
  uint4 o = make_uint4(0, 0, 0, 0);
  if (inside) {
    const uint16_t* src_row = ct + static_cast<long long>(c) * ldc;
    const long long s0 = m0 - static_cast<long long>(ph) * Wp + d;      // source index of element 0
    uint32_t r[4];
    if (d == 0) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(src_row + s0));
      r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
    } else {
      const bool odd = (d & 1) != 0;
      const long long w0 = (s0 - (odd ? 1 : 0)) >> 1;                    // first 32-bit word (an even element)
      const uint32_t* rw = reinterpret_cast<const uint32_t*>(src_row);
      uint32_t w[5];
#pragma unroll
      for (int k = 0; k < 5; ++k) {
        // words outside the row are never selected below; their address is not touched
        const long long wi = w0 + k;
        w[k] = (wi >= 0 && wi * 2 + 1 < ldc) ? __ldg(rw + wi) : 0u;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) r[k] = odd ? __funnelshift_r(w[k], w[k + 1], 16) : w[k];
    }
    // zero the elements whose tap leaves the image row
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int xa = x0 + 2 * k + d, xb = xa + 1;
      if (xa < 0 || xa >= W) r[k] &= 0xffff0000u;
      if (xb < 0 || xb >= W) r[k] &= 0x0000ffffu;
    }
    o = make_uint4(r[0], r[1], r[2], r[3]);
  }
  *reinterpret_cast<uint4*>(planes + (static_cast<long long>(j) * C + c) * plane_ld + m0) = o;
  }
}

// The repack with all taps of a pixel group produced from one read: a thread loads, per channel, the
// three aligned 16-byte groups around the source position (24 elements; the neighbours' groups come out
// of L1) and cuts every tap's 8 elements out of them with funnel shifts; 16-byte stores, lanes along the
// pixel groups.  grid (ceil(plane_ld / 8 / 128), ceil(C / 8)), block 128, kRepackCh channels per thread.
template <int KW>
__global__ void __launch_bounds__(128)
conv_repack_reg_kernel(const uint16_t* __restrict__ ct, long long ldc, int H, int W, int Hp, int Wp, int kh,
                       int n_groups, int n_groups_ld, uint32_t mul_wp8, uint32_t mul_hp,
                       uint16_t* __restrict__ planes, long long plane_ld, int C) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;   // group of 8 padded pixels
  if (g >= n_groups_ld) return;
  const int c_begin = blockIdx.y * kRepackCh, c_end = min(C, c_begin + kRepackCh);
  const long long m0 = static_cast<long long>(g) << 3;
  constexpr int PW = (KW - 1) / 2;
  const int ph = (kh - 1) / 2;
  const int wp8 = Wp >> 3;
  int x0 = 0, y = -1;
  if (g < n_groups) {
    const int row = mul_wp8 ? static_cast<int>(__umulhi(static_cast<uint32_t>(g), mul_wp8)) : g;
    x0 = (g - row * wp8) << 3;
    const int img = mul_hp ? static_cast<int>(__umulhi(static_cast<uint32_t>(row), mul_hp)) : row;
    y = row - img * Hp - ph;
  }
  const bool inside = g < n_groups && y >= 0 && y < H && x0 - PW < W;   // else zeros (halo rows, scratch, tails)
  const long long gs = static_cast<long long>(g) - static_cast<long long>(ph) * wp8;   // source group of tap offset 0
  const long long ld8 = ldc >> 3;
  for (int c = c_begin; c < c_end; ++c) {
    uint32_t w[12];
#pragma unroll
    for (int k = 0; k < 12; ++k) w[k] = 0u;
    if (inside) {
      const uint4* src_row = reinterpret_cast<const uint4*>(ct + static_cast<long long>(c) * ldc);
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        const long long gi = gs + k - 1;
        if (gi >= 0 && gi < ld8) {
          const uint4 v = __ldg(src_row + gi);
          w[4 * k] = v.x; w[4 * k + 1] = v.y; w[4 * k + 2] = v.z; w[4 * k + 3] = v.w;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < KW; ++j) {
      constexpr int kBase = 8 - PW;                 // window element of output element 0 for tap 0
      const int first = kBase + j;                  // ... for tap j (compile-time after unrolling)
      uint32_t r[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int e0 = first + 2 * t;               // window element of output element 2t
        r[t] = (e0 & 1) ? __funnelshift_r(w[e0 >> 1], w[(e0 >> 1) + 1], 16) : w[e0 >> 1];
        const int xa = x0 + 2 * t + j - PW, xb = xa + 1;
        if (xa < 0 || xa >= W) r[t] &= 0xffff0000u;
        if (xb < 0 || xb >= W) r[t] &= 0x0000ffffu;
      }
      *reinterpret_cast<uint4*>(planes + (static_cast<long long>(j) * C + c) * plane_ld + m0) =
          make_uint4(r[0], r[1], r[2], r[3]);
    }
  }
}

}  // namespace

cudaError_t conv_repack_launch(const void* ct, long long ldc, int B, int H, int W, int Hp, int Wp, int kh, int kw,
                               int C, void* planes, long long plane_ld, cudaStream_t stream) {
  if (B <= 0 || C <= 0) return cudaSuccess;
  const long long m_pad = static_cast<long long>(B) * Hp * Wp;
  const long long n_groups = m_pad / 8, n_groups_ld = plane_ld / 8;   // the kernel zeroes the planes' tails too
  // floor(i / d) = umulhi(i, ceil(2^32 / d)) holds for i * d < 2^32
  if (n_groups * std::max<long long>(Wp / 8, Hp) >= (1LL << 32) || n_groups_ld >= (1LL << 31)) return cudaErrorInvalidValue;
  const uint32_t mul_wp8 = Wp / 8 > 1 ? 0xffffffffu / static_cast<uint32_t>(Wp / 8) + 1u : 0u;
  const uint32_t mul_hp = Hp > 1 ? 0xffffffffu / static_cast<uint32_t>(Hp) + 1u : 0u;
  if (kw == 1 || kw == 3 || kw == 5 || kw == 7 || kw == 9) {
    dim3 rgrid(static_cast<unsigned>((n_groups_ld + 127) / 128), (C + kRepackCh - 1) / kRepackCh);
#define TS_REPACK(KW)                                                                                           \
  conv_repack_reg_kernel<KW><<<rgrid, 128, 0, stream>>>(static_cast<const uint16_t*>(ct), ldc, H, W, Hp, Wp, kh, \
                                                        static_cast<int>(n_groups), static_cast<int>(n_groups_ld),  \
                                                        mul_wp8, mul_hp, static_cast<uint16_t*>(planes), plane_ld, C)
    switch (kw) {
      case 1: TS_REPACK(1); break;
      case 3: TS_REPACK(3); break;
      case 5: TS_REPACK(5); break;
      case 7: TS_REPACK(7); break;
      default: TS_REPACK(9); break;
    }
#undef TS_REPACK
    return cudaGetLastError();
  }
  dim3 grid(static_cast<unsigned>((n_groups_ld + 255) / 256), (C + kRepackCh - 1) / kRepackCh, kw);
  conv_repack_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(ct), ldc, H, W, Hp, Wp, kh, kw,
                                               static_cast<int>(n_groups), static_cast<int>(n_groups_ld), mul_wp8,
                                               mul_hp, static_cast<uint16_t*>(planes), plane_ld, C);
  return cudaGetLastError();
}

cudaError_t conv_pack_input_launch(const void* x_nhwc, int B, int H, int W, int C, int kh, int kw, int Hp, int Wp,
                                   void* planes, long long plane_ld, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0) return cudaSuccess;
  const long long m_pad = static_cast<long long>(B) * Hp * Wp;
  const long long n_groups = m_pad / 8, n_groups_ld = plane_ld / 8;
  // register-transpose kernel: floor(i / d) = umulhi(i, ceil(2^32 / d)) holds for i * d < 2^32
  const bool reg_ok = (C % 8) == 0 && C / 8 <= 65535 && n_groups_ld < (1LL << 31) &&
                      n_groups * std::max<long long>(Wp / 8, Hp) < (1LL << 32) &&
                      (kw == 1 || kw == 3 || kw == 5 || kw == 7 || kw == 9);
  if (reg_ok) {
    const uint32_t mul_wp8 = Wp / 8 > 1 ? 0xffffffffu / static_cast<uint32_t>(Wp / 8) + 1u : 0u;
    const uint32_t mul_hp = Hp > 1 ? 0xffffffffu / static_cast<uint32_t>(Hp) + 1u : 0u;
    dim3 grid(static_cast<unsigned>((n_groups_ld + 127) / 128), C / 8);
    const uint16_t* xin = static_cast<const uint16_t*>(x_nhwc);
    uint16_t* pl = static_cast<uint16_t*>(planes);
#define TS_PACK(KW)                                                                                             \
  conv_pack_input_reg_kernel<KW><<<grid, 128, 0, stream>>>(xin, H, W, C, kh, Hp, Wp, static_cast<int>(n_groups), \
                                                           static_cast<int>(n_groups_ld), mul_wp8, mul_hp, pl, plane_ld)
    switch (kw) {
      case 1: TS_PACK(1); break;
      case 3: TS_PACK(3); break;
      case 5: TS_PACK(5); break;
      case 7: TS_PACK(7); break;
      default: TS_PACK(9); break;
    }
#undef TS_PACK
    return cudaGetLastError();
  }
  // the tail of every plane past the last image (read by the lowest kernel rows of the last pixels)
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
  const long long n_groups = static_cast<long long>(B) * Hp * Wp / 8;
  // register-transpose kernel: floor(i / d) = umulhi(i, ceil(2^32 / d)) holds for i * d < 2^32
  if ((N % 8) == 0 && N / 8 <= 65535 && n_groups < (1LL << 31) && n_groups * std::max<long long>(Wp / 8, Hp) < (1LL << 32)) {
    const uint32_t mul_wp8 = Wp / 8 > 1 ? 0xffffffffu / static_cast<uint32_t>(Wp / 8) + 1u : 0u;
    const uint32_t mul_hp = Hp > 1 ? 0xffffffffu / static_cast<uint32_t>(Hp) + 1u : 0u;
    dim3 rgrid(static_cast<unsigned>((n_groups + 127) / 128), N / 8);
    conv_unpack_output_reg_kernel<<<rgrid, 128, 0, stream>>>(static_cast<const uint16_t*>(ct), ldc, H, W, Hp, Wp, N,
                                                             static_cast<int>(n_groups), mul_wp8, mul_hp,
                                                             static_cast<uint16_t*>(y_nhwc));
    return cudaGetLastError();
  }
  dim3 grid((H + kPackRows - 1) / kPackRows, B, (N + kPackCh - 1) / kPackCh);
  conv_unpack_output_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(ct), ldc, B, H, W, Hp, Wp, N,
                                                      static_cast<uint16_t*>(y_nhwc));
  return cudaGetLastError();
}

}  // namespace ts

// Host-callable launchers of the tile-sparse kernels.  Internal to the library; the public surface
// is the C ABI in include/tilesparse.h.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

#include "ts_common.cuh"

namespace ts {

// Tensor-core masked GEMM (masked_gemm_sm100.cu).  `sched` holds rounds*grid work items; entry
// r*grid + b is the r-th unit of CTA b (tile < 0: none, and none after it).  unit_rows is the
// number of batch rows per work unit the schedule was built for: 128 or 256.  `block_meta` is the
// same schedule at K-block granularity: CTA b's 64-row blocks in processing order, one record of
// kBlockMetaInts ints each, at block_meta[b*blk_stride*kBlockMetaInts ...], terminated (and padded
// to blk_stride records) by end markers; expand_block_meta_launch writes it from the descriptors.
// tmap_c != nullptr enables TMA stores (tensor map over Ct [N][ldc], box 64 x 128, 128-byte swizzle)
// for the work items whose flags say their kept columns are consecutive rows of Ct.  early_start
// allows programmatic dependent launch: the kernel reads sched, block_meta and the packed weights before
// it waits for the kernel before it in the stream, so it must be false when that kernel wrote them.
// lean: every unit of the schedule has kItemDenseRows set (the kernel then takes its store-only variant
// when the epilogue is alpha * acc).
cudaError_t masked_gemm_launch(int dtype, int unit_rows, const CUtensorMap& tmap_w, const CUtensorMap* tmap_c,
                               const WorkItem* sched, int rounds, int grid, const int* block_meta,
                               int blk_stride, const void* At, long long lda, void* Ct, long long ldc, int M,
                               const EpilogueArgs& ep, int* status, bool early_start, bool lean,
                               cudaStream_t stream);

// Adds up the fp32 partial sums the split-K units of a schedule left in `scratch` and finishes the
// epilogue (beta * Ct, bias, activation, conversion) for the kept columns of the split tiles.
cudaError_t split_reduce_launch(int dtype, const SplitTile* tiles, int n_split, const float* scratch, long long sld,
                                void* Ct, long long ldc, int M, float beta, const float* bias, int act,
                                cudaStream_t stream);

// meta[b*kBlockMetaInts ...] = record of block b, for all n_blocks (= grid*blk_stride) descriptors:
// resolves the kept-row lists, relative or absolute, into the 16-byte segment at which each kept row
// of the activations starts (`map`: a matrix with its row pitch, or a convolution's input planes).
cudaError_t expand_block_meta_launch(const BlockDesc* blocks, long long n_blocks, int* meta, const RowMap& map,
                                     cudaStream_t stream);

// CUDA-core twin of the masked GEMM with the same operands (masked_gemm_simt.cu).
cudaError_t masked_gemm_simt_launch(int dtype, const TileDesc* tiles, int n_tiles, const void* Wp,
                                    long long ldw, const void* At, long long lda, void* Ct,
                                    long long ldc, int M, float alpha, float beta,
                                    cudaStream_t stream);

// Weight packing (pack.cu): Wp[w_row0 + j][i] = W[kept_k[i]][c_row(j)]; the caller zero-fills Wp first.
cudaError_t pack_weights_launch(int w_dtype, int out_dtype, const void* W, long long ld_w,
                                const TileDesc* tiles, int n_tiles, int max_k, void* Wp,
                                long long ldw, cudaStream_t stream);

// Sparse residual term (residual.cu): Ct[n][m] = (col_written[n] ? Ct[n][m] : 0) + alpha * sum over the
// non-zeros p of column n of val[p] * At[row_idx[p]][m].  col_written may be nullptr (all written).
cudaError_t residual_spmm_launch(int dtype, const int* col_ptr, const int* row_idx, const void* val,
                                 const uint8_t* col_written, const void* At, long long lda, void* Ct,
                                 long long ldc, int M, int N, float alpha, cudaStream_t stream);

// Implicit-GEMM convolution (conv.cu): NHWC input -> kw shifted, zero-padded, channel-major planes
// [kw][C][plane_ld] (16-bit), and the GEMM's padded-pixel output Ct[N][ldc] -> NHWC [B][H][W][N].
// Hp = H + kh - 1, Wp = (W + kw - 1) rounded up to 8.
cudaError_t conv_pack_input_launch(const void* x_nhwc, int B, int H, int W, int C, int kh, int kw, int Hp, int Wp,
                                   void* planes, long long plane_ld, cudaStream_t stream);
// The padded-space output Ct[C][ldc] of one convolution as the input planes of the next one (same
// image size, same kernel size): a shifted, masked copy, no NHWC round trip.
cudaError_t conv_repack_launch(const void* ct, long long ldc, int B, int H, int W, int Hp, int Wp, int kh, int kw,
                               int C, void* planes, long long plane_ld, cudaStream_t stream);
cudaError_t conv_unpack_output_launch(const void* ct, long long ldc, int B, int H, int W, int Hp, int Wp, int N,
                                      void* y_nhwc, cudaStream_t stream);

// out[c][r] = in[r][c] for 16-bit elements (pack.cu).
cudaError_t transpose16_launch(const void* in, long long ld_in, void* out, long long ld_out,
                               int rows, int cols, cudaStream_t stream);

}  // namespace ts

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
// number of batch rows per work unit the schedule was built for: 128 or 256.  `blocks` is the same
// schedule at K-block granularity: CTA b's 64-row blocks in processing order at
// blocks[b*blk_stride ...], terminated (and padded to blk_stride) by end markers.
cudaError_t masked_gemm_launch(int dtype, int unit_rows, const CUtensorMap& tmap_w,
                               const WorkItem* sched, int rounds, int grid,
                               const BlockDesc* blocks, int blk_stride, const void* At,
                               long long lda, void* Ct, long long ldc, int M, float alpha,
                               float beta, int* status, cudaStream_t stream);

#ifdef TS_KERNEL_TRACE
cudaError_t masked_gemm_read_trace(long long* out64, bool clear);
#endif

// CUDA-core twin of the masked GEMM with the same operands (masked_gemm_simt.cu).
cudaError_t masked_gemm_simt_launch(int dtype, const TileDesc* tiles, int n_tiles, const void* Wp,
                                    long long ldw, const void* At, long long lda, void* Ct,
                                    long long ldc, int M, float alpha, float beta,
                                    cudaStream_t stream);

// Weight packing (pack.cu): Wp[w_row0 + j][i] = W[kept_k[i]][c_row(j)]; the caller zero-fills Wp first.
cudaError_t pack_weights_launch(int w_dtype, int out_dtype, const void* W, long long ld_w,
                                const TileDesc* tiles, int n_tiles, int max_k, void* Wp,
                                long long ldw, cudaStream_t stream);

// out[c][r] = in[r][c] for 16-bit elements (pack.cu).
cudaError_t transpose16_launch(const void* in, long long ld_in, void* out, long long ld_out,
                               int rows, int cols, cudaStream_t stream);

}  // namespace ts

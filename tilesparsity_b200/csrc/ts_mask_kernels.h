// Host-callable launchers of the mask-construction kernels (mask_build.cu).  Internal.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace ts {

// norms[t*K + k] = ||score[k, bounds[t]:bounds[t+1]] (.* colmask)||_2, divided by the tile width
// when `divide` is set.  bounds_dev holds n_tiles+1 column indices on the device.  n_uniform128 > 0
// promises that the first n_uniform128 tiles are the fixed tiles [128 t, 128 (t+1)).
cudaError_t tile_row_norms_launch(const float* score, long long ld, int K, const int* bounds_dev,
                                  int n_tiles, const uint8_t* colmask, float* norms, int divide,
                                  int n_uniform128, cudaStream_t s);
// out[t*K + k] = sum of |score[k, c]| over the tile's columns, left to right.
cudaError_t tile_row_l1_launch(const float* score, long long ld, int K, const int* bounds_dev,
                               int n_tiles, float* out, cudaStream_t s);
// out[n] = ||score[:, n]||_2 / K, rows accumulated in order.
cudaError_t col_norms_launch(const float* score, long long ld, int K, int N, float* out,
                             cudaStream_t s);
// One digit pass of the radix select: hist[256] must be zero on entry.
cudaError_t select_hist_launch(const float* vals, long long n, uint32_t prefix, int shift,
                               unsigned int* hist, cudaStream_t s);
// *count_le += #{key <= key}; *min_gt = min(*min_gt, smallest key above `key`).
cudaError_t select_neighbor_launch(const float* vals, long long n, uint32_t key,
                                   unsigned long long* count_le, unsigned int* min_gt,
                                   cudaStream_t s);
// State of one radix select kept on the device between its passes.
struct SelectState {
  uint32_t prefix;              // key bits fixed so far
  uint32_t error;               // 1: the rank was not among the keys (non-finite input)
  unsigned long long rank;      // rank still to be located inside the current prefix
  unsigned long long count_le;  // #{key <= selected key}
  uint32_t min_gt;              // smallest key above the selected one
  uint32_t pad_;
};

// np.percentile(vals, q) enqueued without any read-back: ranks pi <= ni <= pi+1 and the interpolation
// weight come from the host (they depend on n and q only); the threshold lands in *thr_out (device),
// the two order statistics in ab_out[0..1] (device, optional).  arith: 0 float32 everywhere, 1 double
// with a float32 difference, 2 double everywhere.  hist: 256 counters.
cudaError_t percentile_dev_launch(const float* vals, long long n, long long pi, long long ni, float gamma_f,
                                  double gamma_d, int arith, SelectState* st, unsigned int* hist,
                                  double* thr_out, float* ab_out, cudaStream_t s);

// Double-precision twins for float64 scores (mask_build_f64.cu): tile-row norms by the general kernel,
// the percentile with everything in double (eight digit passes over 64-bit keys), the threshold.
struct SelectState64 {
  unsigned long long prefix;
  unsigned long long rank;
  unsigned long long count_le;
  unsigned long long min_gt;
  uint32_t error;
  uint32_t pad_;
};
cudaError_t tile_row_norms64_launch(const double* score, long long ld, int K, const int* bounds_dev, int n_tiles,
                                    double* norms, int divide, cudaStream_t s);
cudaError_t percentile64_dev_launch(const double* vals, long long n, long long pi, long long ni, double gamma,
                                    SelectState64* st, unsigned int* hist, double* thr_out, cudaStream_t s);
cudaError_t threshold64_dev_launch(const double* vals, long long n, const double* thr, uint8_t* keep,
                                   cudaStream_t s);
// acc[i] += square(grad[i] * weight[i]), the product and the square in float32, the sum in double.
cudaError_t taylor_accumulate_launch(const float* grad, const float* weight, double* acc, long long n,
                                     cudaStream_t s);

// keep[i] = vals[i] > *thr, the threshold read from device memory.
cudaError_t threshold_dev_launch(const float* vals, long long n, const double* thr, uint8_t* keep,
                                 cudaStream_t s);

cudaError_t threshold_launch(const float* vals, long long n, double thr, uint8_t* keep,
                             cudaStream_t s);
cudaError_t segment_count_launch(const uint8_t* keep, const long long* seg_ptr, int n_seg, int* counts,
                                 cudaStream_t s);
// out_ptr[0..n_seg] = exclusive prefix sums of counts (device to device).
cudaError_t segment_offsets_launch(const int* counts, int n_seg, int* out_ptr, cudaStream_t s);
cudaError_t segment_compact_launch(const uint8_t* keep, const long long* seg_ptr, int n_seg,
                                   const int* out_ptr, int* list, cudaStream_t s);
cudaError_t dense_mask_launch(const uint8_t* rowkeep, const uint8_t* colkeep, const int* tile_of_col,
                              int K, int N, uint8_t* mask, long long ld_mask, cudaStream_t s);
// |score| of one layer into a dense [K][N] float array (element-wise baseline).
cudaError_t abs_values_launch(const float* score, long long ld, int K, int N, float* vals, cudaStream_t s);

// Vector-wise baseline mask: blocks of 16 rows of one column, keep above the (topk+1)-th largest.
cudaError_t vw_mask_launch(const float* score, long long ld, int K, int N, int topk, uint8_t* mask,
                           long long ld_mask, cudaStream_t s);

// Block-wise baseline: out[bi * nbj + bj] = Frobenius norm of the 32 x 32 block (bi, bj) of score;
// mask[k][n] = keep[block of (k, n)].
cudaError_t block_norms_launch(const float* score, long long ld, int K, int N, float* out, cudaStream_t s);
cudaError_t block_mask_launch(const uint8_t* keep, int K, int N, uint8_t* mask, long long ld_mask, cudaStream_t s);

cudaError_t tew_values_launch(const float* score, long long ld, const uint8_t* mask, long long ld_mask,
                              int K, int N, float* vals, cudaStream_t s);
cudaError_t tew_apply_launch(const float* vals, const double* thr, int K, int N, uint8_t* mask,
                             long long ld_mask, uint8_t* residual, cudaStream_t s);
cudaError_t tile_rank_launch(const float* vals, int K, int n_tiles, int mode, int k_keep, int pi,
                             int ni, uint8_t* keep, float* stats, cudaStream_t s);
cudaError_t threshold_per_tile_launch(const float* vals, int K, int n_tiles, const double* thr,
                                      uint8_t* keep, cudaStream_t s);

}  // namespace ts

// Importance scores accumulated on the device, and the float64 row stage of the tile-wise masks.
//
// The reference's pruning hooks score a weight by the first-order Taylor term: per training step
// square(dL/dmask * w) in float32 (compute_taylor_score, Pruning/VGG/myhook.py:44-48;
// Pruning/BERT/utils/MyHook.py:178-182), added step after step into float64 host arrays
// (after_run, myhook.py:248-257: np.zeros(shape) += float32 scores).  The masks are then built from
// those float64 arrays, so NumPy does every step in double: squares, the pairwise add.reduce of
// np.linalg.norm(axis=1), sqrt, the division by the width, the percentile and the comparison.  The
// kernels here are the double-precision twins of the float32 ones in mask_build.cu, with the same
// operation order and single IEEE-754 steps (no fused multiply-add).
#include "ts_common.cuh"
#include "ts_mask_kernels.h"

namespace ts {

namespace {

// acc[i] += (double) fl32(fl32(g[i] * w[i])^2)
__global__ void __launch_bounds__(256)
taylor_accumulate_kernel(const float* __restrict__ grad, const float* __restrict__ weight,
                         double* __restrict__ acc, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float t = __fmul_rn(__ldg(grad + i), __ldg(weight + i));
    acc[i] = __dadd_rn(acc[i], static_cast<double>(__fmul_rn(t, t)));
  }
}

// ---------------------------------------------------------------------------------------------
// Row norms in double: NumPy's pairwise sum of the squares of a run, by 8 cooperating lanes
// (see mask_build.cu for the float32 twin and the summation order)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ double sq_at64(const double* row, int i) {
  const double x = __ldg(row + i);
  return __dmul_rn(x, x);
}

__device__ __forceinline__ double shfl_xor64(double v, int mask) {
  return __shfl_xor_sync(0xffffffffu, v, mask);
}

__device__ __forceinline__ double leaf_sum8_64(const double* row, int o, int n, int j) {
  double r = sq_at64(row, o + j);
  const int body = n - (n % 8);
  for (int i = 8; i < body; i += 8) r = __dadd_rn(r, sq_at64(row, o + i + j));
  r = __dadd_rn(r, shfl_xor64(r, 1));
  r = __dadd_rn(r, shfl_xor64(r, 2));
  r = __dadd_rn(r, shfl_xor64(r, 4));
  for (int i = body; i < n; ++i) r = __dadd_rn(r, sq_at64(row, o + i));
  return r;
}

__device__ double pairwise_sq_sum64(const double* row, int o, int n, int j) {
  if (n < 8) {
    double r = 0.0;
    for (int i = 0; i < n; ++i) r = __dadd_rn(r, sq_at64(row, o + i));
    return r;
  }
  if (n <= 128) return leaf_sum8_64(row, o, n, j);
  int n2 = n / 2;
  n2 -= n2 % 8;
  const double a = pairwise_sq_sum64(row, o, n2, j);
  const double b = pairwise_sq_sum64(row, o + n2, n - n2, j);
  return __dadd_rn(a, b);
}

// norms[t*K + k] = ||score[k, bounds[t]:bounds[t+1]]||_2 (/ width);  grid (ceil(K/32), n_tiles), block 256
__global__ void __launch_bounds__(256)
tile_row_norms64_kernel(const double* __restrict__ score, long long ld, int K, const int* __restrict__ bounds,
                        double* __restrict__ norms, int divide) {
  const int t = blockIdx.y;
  const int c0 = bounds[t], width = bounds[t + 1] - c0;
  const int group = threadIdx.x >> 3, j = threadIdx.x & 7;
  const int k = blockIdx.x * 32 + group;
  const int kk = k < K ? k : K - 1;   // clamped rows keep the warp converged; their result is dropped
  const double sum = pairwise_sq_sum64(score + static_cast<long long>(kk) * ld + c0, 0, width, j);
  double v = __dsqrt_rn(sum);
  if (divide) v = __ddiv_rn(v, static_cast<double>(width));
  if (k < K && j == 0) norms[static_cast<long long>(t) * K + k] = v;
}

// ---------------------------------------------------------------------------------------------
// Radix select over float64 values (order-preserving 64-bit keys, eight 8-bit digits), state on the
// device
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long double_key(double f) {
  const unsigned long long b = static_cast<unsigned long long>(__double_as_longlong(f));
  return (b >> 63) ? ~b : (b | 0x8000000000000000ull);
}

__device__ __forceinline__ double key_to_double(unsigned long long k) {
  return __longlong_as_double(static_cast<long long>((k >> 63) ? (k & 0x7fffffffffffffffull) : ~k));
}

__global__ void __launch_bounds__(256)
select64_begin_kernel(SelectState64* __restrict__ st, unsigned int* __restrict__ hist, unsigned long long rank) {
  hist[threadIdx.x] = 0;
  if (threadIdx.x == 0) {
    st->prefix = 0;
    st->error = 0;
    st->rank = rank;
    st->count_le = 0;
    st->min_gt = 0xffffffffffffffffull;
  }
}

__global__ void __launch_bounds__(256)
select64_hist_kernel(const double* __restrict__ vals, long long n, const SelectState64* __restrict__ st,
                     int shift, unsigned int* __restrict__ hist) {
  __shared__ unsigned int h[256];
  h[threadIdx.x] = 0;
  __syncthreads();
  const unsigned long long prefix = st->prefix;
  const unsigned long long hi_mask = shift >= 56 ? 0ull : (0xffffffffffffffffull << (shift + 8));
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const unsigned long long key = double_key(__ldg(vals + i));
    if ((key & hi_mask) == (prefix & hi_mask)) atomicAdd(&h[(key >> shift) & 0xffu], 1u);
  }
  __syncthreads();
  if (h[threadIdx.x]) atomicAdd(&hist[threadIdx.x], h[threadIdx.x]);
}

__global__ void __launch_bounds__(256)
select64_pick_kernel(SelectState64* __restrict__ st, unsigned int* __restrict__ hist, int shift) {
  __shared__ unsigned long long cum[256];
  const int t = threadIdx.x;
  const unsigned long long mine = hist[t];
  const unsigned long long rank = st->rank;
  cum[t] = mine;
  __syncthreads();
  for (int o = 1; o < 256; o <<= 1) {
    const unsigned long long add = t >= o ? cum[t - o] : 0;
    __syncthreads();
    cum[t] += add;
    __syncthreads();
  }
  const unsigned long long incl = cum[t], excl = incl - mine;
  if (excl <= rank && rank < incl) {
    st->prefix |= static_cast<unsigned long long>(t) << shift;
    st->rank = rank - excl;
  }
  if (t == 255 && rank >= incl) st->error = 1;
  hist[t] = 0;
}

__global__ void __launch_bounds__(256)
select64_neighbor_kernel(const double* __restrict__ vals, long long n, SelectState64* __restrict__ st) {
  const unsigned long long key = st->prefix;
  unsigned long long c = 0, m = 0xffffffffffffffffull;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const unsigned long long k = double_key(__ldg(vals + i));
    if (k <= key) ++c;
    else m = m < k ? m : k;
  }
  for (int o = 16; o > 0; o >>= 1) {
    c += __shfl_xor_sync(0xffffffffu, c, o);
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, m, o);
    m = m < other ? m : other;
  }
  if ((threadIdx.x & 31) == 0) {
    if (c) atomicAdd(&st->count_le, c);
    if (m != 0xffffffffffffffffull) atomicMin(&st->min_gt, m);
  }
}

// The two order statistics and NumPy's _lerp between them, everything in double.
__global__ void select64_finish_kernel(SelectState64* __restrict__ st, long long pi, long long ni, double gamma,
                                       double* __restrict__ thr_out) {
  const double a = key_to_double(st->prefix);
  double b = a;
  if (ni != pi && static_cast<long long>(st->count_le) < ni + 1) b = key_to_double(st->min_gt);
  const double diff = __dsub_rn(b, a);
  double res = __dadd_rn(a, __dmul_rn(diff, gamma));
  if (gamma >= 0.5) res = __dsub_rn(b, __dmul_rn(diff, __dsub_rn(1.0, gamma)));
  *thr_out = res;
}

__global__ void __launch_bounds__(256)
threshold64_dev_kernel(const double* __restrict__ vals, long long n, const double* __restrict__ thr,
                       uint8_t* __restrict__ keep) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i < n) keep[i] = vals[i] > *thr ? 1 : 0;
}

int stream_grid64(long long n) {
  long long b = (n + 255) / 256;
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace

cudaError_t taylor_accumulate_launch(const float* grad, const float* weight, double* acc, long long n,
                                     cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  taylor_accumulate_kernel<<<stream_grid64(n), 256, 0, s>>>(grad, weight, acc, n);
  return cudaGetLastError();
}

cudaError_t tile_row_norms64_launch(const double* score, long long ld, int K, const int* bounds_dev, int n_tiles,
                                    double* norms, int divide, cudaStream_t s) {
  if (K <= 0 || n_tiles <= 0) return cudaSuccess;
  dim3 grid((K + 31) / 32, n_tiles);
  tile_row_norms64_kernel<<<grid, 256, 0, s>>>(score, ld, K, bounds_dev, norms, divide);
  return cudaGetLastError();
}

cudaError_t percentile64_dev_launch(const double* vals, long long n, long long pi, long long ni, double gamma,
                                    SelectState64* st, unsigned int* hist, double* thr_out, cudaStream_t s) {
  select64_begin_kernel<<<1, 256, 0, s>>>(st, hist, static_cast<unsigned long long>(pi));
  for (int shift = 56; shift >= 0; shift -= 8) {
    select64_hist_kernel<<<stream_grid64(n), 256, 0, s>>>(vals, n, st, shift, hist);
    select64_pick_kernel<<<1, 256, 0, s>>>(st, hist, shift);
  }
  if (ni != pi) select64_neighbor_kernel<<<stream_grid64(n), 256, 0, s>>>(vals, n, st);
  select64_finish_kernel<<<1, 1, 0, s>>>(st, pi, ni, gamma, thr_out);
  return cudaGetLastError();
}

cudaError_t threshold64_dev_launch(const double* vals, long long n, const double* thr, uint8_t* keep,
                                   cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  threshold64_dev_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(vals, n, thr, keep);
  return cudaGetLastError();
}

}  // namespace ts

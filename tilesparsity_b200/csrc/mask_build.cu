// Tile-wise (TW / TEW) mask construction kernels.
//
// Device-side counterpart of the reference's NumPy mask builder (Pruning/VGG/prune_algo.py:55-193;
// BERT variants Pruning/BERT/utils/MyHook.py:202-313).  The masks must equal the reference's bit
// for bit, so every float32 step reproduces what NumPy computes there, in the same order and with
// the same roundings (no fused multiply-add anywhere):
//
//   row norms   np.linalg.norm(tile, axis=1) / width   (prune_algo.py:90,128): squares rounded to
//               float32, NumPy's pairwise add.reduce (eight running sums over elements j, j+8, ...
//               combined as ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7)), leftovers in order; runs longer than
//               128 split at n/2 rounded down to a multiple of 8), sqrt, division by the width;
//   col norms   np.linalg.norm(score, axis=0) / K      (prune_algo.py:64): squares summed down the
//               rows in order;
//   percentile  np.percentile(all norms, q)            (prune_algo.py:66,95,134,166): two exact
//               order statistics by radix select; the interpolation between them runs on the host
//               (capi.cu) in the arithmetic type NumPy would use;
//   keep        norm > threshold, strict               (prune_algo.py:67,99,140,171).
//
// All kernels are HBM-bound streaming passes: the score matrix is read once per norm pass (4 bytes
// per element), the radix select reads its 4-byte keys once per 8-bit digit.
#include "ts_common.cuh"
#include "ts_mask_kernels.h"

namespace ts {

namespace {

// ---------------------------------------------------------------------------------------------
// NumPy's pairwise float32 sum of the squares of a strided run, computed by 8 cooperating lanes.
// ---------------------------------------------------------------------------------------------
struct RowSrc {
  const float* row;        // first element of the run
  const uint8_t* colmask;  // nullptr, or one byte per element of the run (0: element counts as +0)
};

__device__ __forceinline__ float sq_at(const RowSrc& s, int i) {
  if (s.colmask && !s.colmask[i]) return 0.0f;
  const float x = __ldg(s.row + i);
  return __fmul_rn(x, x);
}

// Sum of run [o, o+n), 8 <= n <= 128, by the 8 lanes of a group; every lane returns the sum.
__device__ __forceinline__ float leaf_sum8(const RowSrc& s, int o, int n, int j) {
  float r = sq_at(s, o + j);
  const int body = n - (n % 8);
  for (int i = 8; i < body; i += 8) r = __fadd_rn(r, sq_at(s, o + i + j));
  r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 1));   // r0+r1, r2+r3, r4+r5, r6+r7
  r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 2));   // (r0+r1)+(r2+r3), (r4+r5)+(r6+r7)
  r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 4));
  for (int i = body; i < n; ++i) r = __fadd_rn(r, sq_at(s, o + i));
  return r;
}

// Whole run of any length.  The control flow depends only on n, which is uniform across a warp.
__device__ float pairwise_sq_sum(const RowSrc& s, int o, int n, int j) {
  if (n < 8) {
    float r = 0.0f;
    for (int i = 0; i < n; ++i) r = __fadd_rn(r, sq_at(s, o + i));
    return r;
  }
  if (n <= 128) return leaf_sum8(s, o, n, j);
  int n2 = n / 2;
  n2 -= n2 % 8;
  const float a = pairwise_sq_sum(s, o, n2, j);
  const float b = pairwise_sq_sum(s, o + n2, n - n2, j);
  return __fadd_rn(a, b);
}

// norms[t*K + k] = ||score[k, bounds[t]:bounds[t+1]] (.* colmask)||_2 (/ width)
// grid: (ceil(K / 32), n_tiles), block 256 = 32 groups of 8 lanes, one (row, tile) per group.
__global__ void __launch_bounds__(256)
tile_row_norms_kernel(const float* __restrict__ score, long long ld, int K,
                      const int* __restrict__ bounds, const uint8_t* __restrict__ colmask,
                      float* __restrict__ norms, int divide) {
  const int t = blockIdx.y;
  const int c0 = bounds[t], width = bounds[t + 1] - c0;
  const int group = threadIdx.x >> 3, j = threadIdx.x & 7;
  const int k = blockIdx.x * 32 + group;
  const int kk = k < K ? k : K - 1;   // clamped rows keep the warp converged; their result is dropped
  RowSrc s;
  s.row = score + static_cast<long long>(kk) * ld + c0;
  s.colmask = colmask ? colmask + c0 : nullptr;
  const float sum = pairwise_sq_sum(s, 0, width, j);
  float v = __fsqrt_rn(sum);
  if (divide) v = __fdiv_rn(v, static_cast<float>(width));
  if (k < K && j == 0) norms[static_cast<long long>(t) * K + k] = v;
}

// Fast path of the row norms for tiles that are exactly 128 columns wide and carry no column mask
// (every tile of tw1 when N is a multiple of 128): a block stages 32 rows x 128 columns through
// shared memory with fully coalesced 16-byte loads, then the same 8-lane groups reduce them in
// NumPy's order (leaf of 128 elements: eight running sums, tree, no leftovers).
// grid: (ceil(K / 32), n_tiles_128), block 256.
__global__ void __launch_bounds__(256)
tile_row_norms128_kernel(const float* __restrict__ score, long long ld, int K,
                         float* __restrict__ norms, int divide) {
  constexpr int kPitch = 136;   // floats per staged row: rows 8 banks apart, 16-byte aligned
  __shared__ __align__(16) float tile[32 * kPitch];
  const int t = blockIdx.y;
  const int k0 = blockIdx.x * 32;
  const float* base = score + static_cast<long long>(t) * 128;
  const bool vec_ok = (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(score) & 15u) == 0);
  for (int v = threadIdx.x; v < 32 * 32; v += 256) {   // 32 rows x 32 float4
    const int r = v >> 5, c4 = v & 31;
    const int k = k0 + r;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (k < K) {
      const float* p = base + static_cast<long long>(k) * ld + c4 * 4;
      if (vec_ok) {
        x = __ldg(reinterpret_cast<const float4*>(p));
      } else {
        x = make_float4(__ldg(p), __ldg(p + 1), __ldg(p + 2), __ldg(p + 3));
      }
    }
    *reinterpret_cast<float4*>(&tile[r * kPitch + c4 * 4]) = x;
  }
  __syncthreads();
  const int group = threadIdx.x >> 3, j = threadIdx.x & 7;
  const float* row = &tile[group * kPitch];
  float x = row[j];
  float r = __fmul_rn(x, x);
#pragma unroll
  for (int i = 8; i < 128; i += 8) {
    x = row[i + j];
    r = __fadd_rn(r, __fmul_rn(x, x));
  }
  r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 1));
  r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 2));
  r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 4));
  float v = __fsqrt_rn(r);
  if (divide) v = __fdiv_rn(v, 128.0f);
  const int k = k0 + group;
  if (k < K && j == 0) norms[static_cast<long long>(t) * K + k] = v;
}

// l1[t*K + k] = sum_c |score[k, c]| over the tile's columns, left to right.
__global__ void __launch_bounds__(256)
tile_row_l1_kernel(const float* __restrict__ score, long long ld, int K,
                   const int* __restrict__ bounds, float* __restrict__ out) {
  const int t = blockIdx.y;
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= K) return;
  const int c0 = bounds[t], c1 = bounds[t + 1];
  const float* row = score + static_cast<long long>(k) * ld;
  float r = 0.0f;
  for (int c = c0; c < c1; ++c) r = __fadd_rn(r, fabsf(__ldg(row + c)));
  out[static_cast<long long>(t) * K + k] = r;
}

// out[n] = sqrt(sum_k score[k][n]^2 in row order) / K
//
// The sum of one column is a chain of K dependent additions (NumPy reduces axis 0 row by row), so
// the only parallelism is across columns.  A block owns kColsPerBlock columns: all 256 threads fetch
// the next kColRows x kColsPerBlock slab (global loads in flight) while the first kColsPerBlock
// threads walk the previous slab in shared memory, so the chain waits on shared memory, never on DRAM.
constexpr int kColsPerBlock = 16;
constexpr int kColRows = 128;
constexpr int kColPerThread = kColsPerBlock * kColRows / 256;  // 8

__global__ void __launch_bounds__(256)
col_norms_kernel(const float* __restrict__ score, long long ld, int K, int N,
                 float* __restrict__ out) {
  __shared__ float slab[2][kColRows][kColsPerBlock];
  const int n0 = blockIdx.x * kColsPerBlock;
  const int tid = threadIdx.x;
  const int lc = tid % kColsPerBlock;       // column inside the slab
  const int lr = tid / kColsPerBlock;       // first row this thread fetches (stride 16 rows)
  const bool col_ok = n0 + lc < N;
  float reg[kColPerThread];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < kColPerThread; ++i) {
      const int k = k0 + lr + i * (256 / kColsPerBlock);
      reg[i] = (col_ok && k < K) ? __ldg(score + static_cast<long long>(k) * ld + n0 + lc) : 0.0f;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < kColPerThread; ++i) slab[buf][lr + i * (256 / kColsPerBlock)][lc] = reg[i];
  };
  fetch(0);
  stash(0);
  __syncthreads();
  float acc = 0.0f;
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += kColRows) {
    const bool more = k0 + kColRows < K;
    if (more) fetch(k0 + kColRows);
    if (tid < kColsPerBlock) {
      const int rows = min(kColRows, K - k0);
      int r = 0;
      if (k0 == 0) {
        const float x = slab[buf][0][tid];
        acc = __fmul_rn(x, x);
        r = 1;
      }
#pragma unroll 8
      for (; r < rows; ++r) {
        const float x = slab[buf][r][tid];
        acc = __fadd_rn(acc, __fmul_rn(x, x));
      }
    }
    if (more) stash(buf ^ 1);
    __syncthreads();
    buf ^= 1;
  }
  if (tid < kColsPerBlock && n0 + tid < N)
    out[n0 + tid] = __fdiv_rn(__fsqrt_rn(acc), static_cast<float>(K));
}

// ---------------------------------------------------------------------------------------------
// Radix select over float32 values (order-preserving 32-bit keys)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// hist[d] += #{i : key_i agrees with `prefix` on the bits above shift+8 and has digit d at shift}
__global__ void __launch_bounds__(256)
select_hist_kernel(const float* __restrict__ vals, long long n, uint32_t prefix, int shift,
                   unsigned int* __restrict__ hist) {
  __shared__ unsigned int h[256];
  h[threadIdx.x] = 0;
  __syncthreads();
  const uint32_t hi_mask = shift >= 24 ? 0u : (0xffffffffu << (shift + 8));
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint32_t key = float_key(__ldg(vals + i));
    if ((key & hi_mask) == (prefix & hi_mask)) atomicAdd(&h[(key >> shift) & 0xffu], 1u);
  }
  __syncthreads();
  if (h[threadIdx.x]) atomicAdd(&hist[threadIdx.x], h[threadIdx.x]);
}

// Block-wide sum of c and minimum of m (256 threads), then one atomic of each per block.
__device__ __forceinline__ void block_count_min(unsigned long long c, unsigned int m,
                                                unsigned long long* count_le, unsigned int* min_gt) {
  __shared__ unsigned long long sc[8];
  __shared__ unsigned int sm[8];
  for (int o = 16; o > 0; o >>= 1) {
    c += __shfl_xor_sync(0xffffffffu, c, o);
    m = min(m, __shfl_xor_sync(0xffffffffu, m, o));
  }
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) {
    sc[w] = c;
    sm[w] = m;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) {
      c += sc[i];
      m = min(m, sm[i]);
    }
    if (c) atomicAdd(count_le, c);
    if (m != 0xffffffffu) atomicMin(min_gt, m);
  }
}

// res[0..1] (64-bit) += #{key_i <= key};  res[2] = min(res[2], min{key_i : key_i > key})
__global__ void __launch_bounds__(256)
select_neighbor_kernel(const float* __restrict__ vals, long long n, uint32_t key,
                       unsigned long long* __restrict__ count_le, unsigned int* __restrict__ min_gt) {
  unsigned long long c = 0;
  unsigned int m = 0xffffffffu;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint32_t k = float_key(__ldg(vals + i));
    if (k <= key) ++c;
    else m = min(m, k);
  }
  block_count_min(c, m, count_le, min_gt);
}

// ---------------------------------------------------------------------------------------------
// The same select with its digit choice on the device: nothing is read back between the passes
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
select_begin_kernel(SelectState* __restrict__ st, unsigned int* __restrict__ hist, unsigned long long rank) {
  hist[threadIdx.x] = 0;
  if (threadIdx.x == 0) {
    st->prefix = 0;
    st->error = 0;
    st->rank = rank;
    st->count_le = 0;
    st->min_gt = 0xffffffffu;
  }
}

__global__ void __launch_bounds__(256)
select_hist_dev_kernel(const float* __restrict__ vals, long long n, const SelectState* __restrict__ st,
                       int shift, unsigned int* __restrict__ hist) {
  __shared__ unsigned int h[256];
  h[threadIdx.x] = 0;
  __syncthreads();
  const uint32_t prefix = st->prefix;
  const uint32_t hi_mask = shift >= 24 ? 0u : (0xffffffffu << (shift + 8));
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint32_t key = float_key(__ldg(vals + i));
    if ((key & hi_mask) == (prefix & hi_mask)) atomicAdd(&h[(key >> shift) & 0xffu], 1u);
  }
  __syncthreads();
  if (h[threadIdx.x]) atomicAdd(&hist[threadIdx.x], h[threadIdx.x]);
}

// One block: the digit whose bin holds the wanted rank joins the prefix; the histogram is cleared
// for the next pass.
__global__ void __launch_bounds__(256)
select_pick_kernel(SelectState* __restrict__ st, unsigned int* __restrict__ hist, int shift) {
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
    st->prefix |= static_cast<uint32_t>(t) << shift;
    st->rank = rank - excl;
  }
  if (t == 255 && rank >= incl) st->error = 1;   // the rank lies beyond the keys that matched (non-finite input)
  hist[t] = 0;
}

__global__ void __launch_bounds__(256)
select_neighbor_dev_kernel(const float* __restrict__ vals, long long n, SelectState* __restrict__ st) {
  const uint32_t key = st->prefix;
  unsigned long long c = 0;
  unsigned int m = 0xffffffffu;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint32_t k = float_key(__ldg(vals + i));
    if (k <= key) ++c;
    else m = min(m, k);
  }
  block_count_min(c, m, &st->count_le, &st->min_gt);
}

__device__ __forceinline__ float key_to_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// The two order statistics and NumPy's _lerp between them (a + (b-a)*t, or b - (b-a)*(1-t) when
// t >= 0.5), with the operand types NumPy uses: arith 0 = all float32; 1 = t in double but b-a in
// float32 (float32 array, float64 q); 2 = all double (float64 array).
__global__ void select_finish_kernel(SelectState* __restrict__ st, long long pi, long long ni, float gamma_f,
                                     double gamma_d, int arith, double* __restrict__ thr_out,
                                     float* __restrict__ ab_out) {
  const float a = key_to_float(st->prefix);
  float b = a;
  if (ni != pi && static_cast<long long>(st->count_le) < ni + 1) b = key_to_float(st->min_gt);
  double res;
  if (arith == 0) {
    const float diff = __fsub_rn(b, a);
    float r = __fadd_rn(a, __fmul_rn(diff, gamma_f));
    if (gamma_f >= 0.5f) r = __fsub_rn(b, __fmul_rn(diff, __fsub_rn(1.0f, gamma_f)));
    res = static_cast<double>(r);
  } else {
    const double diff = arith == 1 ? static_cast<double>(__fsub_rn(b, a))
                                   : __dsub_rn(static_cast<double>(b), static_cast<double>(a));
    res = __dadd_rn(static_cast<double>(a), __dmul_rn(diff, gamma_d));
    if (gamma_d >= 0.5) res = __dsub_rn(static_cast<double>(b), __dmul_rn(diff, __dsub_rn(1.0, gamma_d)));
  }
  *thr_out = res;
  if (ab_out) {
    ab_out[0] = a;
    ab_out[1] = b;
  }
}

// The whole percentile in one block of 1024 threads, for inputs small enough that a launch costs more
// than a pass over them: the same four digit passes, neighbour pass and interpolation as the kernels
// above, with the histogram in shared memory and block barriers where those have kernel boundaries.
// The select state is written as the multi-kernel path leaves it.
constexpr long long kSmallSelect = 1 << 15;   // measured: 18 Ki values win a quarter of the call, 64 Ki lose half
__global__ void __launch_bounds__(1024)
percentile_small_kernel(const float* __restrict__ vals, int n, long long pi, long long ni, float gamma_f,
                        double gamma_d, int arith, SelectState* __restrict__ st, double* __restrict__ thr_out,
                        float* __restrict__ ab_out) {
  __shared__ unsigned int h[256];
  __shared__ unsigned long long cum[256];
  __shared__ uint32_t s_prefix, s_error, s_min;
  __shared__ unsigned long long s_rank, s_count;
  const int t = threadIdx.x;
  if (t == 0) {
    s_prefix = 0;
    s_error = 0;
    s_rank = static_cast<unsigned long long>(pi);
    s_count = 0;
    s_min = 0xffffffffu;
  }
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (t < 256) h[t] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t hi_mask = shift >= 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = t; i < n; i += 1024) {
      const uint32_t key = float_key(__ldg(vals + i));
      if ((key & hi_mask) == (prefix & hi_mask)) atomicAdd(&h[(key >> shift) & 0xffu], 1u);
    }
    __syncthreads();
    // inclusive scan of the 256 bins by the first 256 threads
    const unsigned long long mine = t < 256 ? h[t] : 0;
    if (t < 256) cum[t] = mine;
    __syncthreads();
    for (int o = 1; o < 256; o <<= 1) {
      const unsigned long long add = (t < 256 && t >= o) ? cum[t - o] : 0;
      __syncthreads();
      if (t < 256) cum[t] += add;
      __syncthreads();
    }
    const unsigned long long rank = s_rank;
    __syncthreads();
    if (t < 256) {
      const unsigned long long incl = cum[t], excl = incl - mine;
      if (excl <= rank && rank < incl) {
        s_prefix = prefix | (static_cast<uint32_t>(t) << shift);
        s_rank = rank - excl;
      }
      if (t == 255 && rank >= incl) s_error = 1;
    }
    __syncthreads();
  }
  const uint32_t key = s_prefix;
  if (ni != pi) {
    unsigned long long c = 0;
    unsigned int m = 0xffffffffu;
    for (int i = t; i < n; i += 1024) {
      const uint32_t k = float_key(__ldg(vals + i));
      if (k <= key) ++c;
      else m = min(m, k);
    }
    for (int o = 16; o > 0; o >>= 1) {
      c += __shfl_xor_sync(0xffffffffu, c, o);
      m = min(m, __shfl_xor_sync(0xffffffffu, m, o));
    }
    if ((t & 31) == 0) {
      if (c) atomicAdd(&s_count, c);
      if (m != 0xffffffffu) atomicMin(&s_min, m);
    }
    __syncthreads();
  }
  if (t == 0) {
    st->prefix = key;
    st->error = s_error;
    st->rank = s_rank;
    st->count_le = s_count;
    st->min_gt = s_min;
    const float a = key_to_float(key);
    float b = a;
    if (ni != pi && static_cast<long long>(s_count) < ni + 1) b = key_to_float(s_min);
    double res;
    if (arith == 0) {
      const float diff = __fsub_rn(b, a);
      float r = __fadd_rn(a, __fmul_rn(diff, gamma_f));
      if (gamma_f >= 0.5f) r = __fsub_rn(b, __fmul_rn(diff, __fsub_rn(1.0f, gamma_f)));
      res = static_cast<double>(r);
    } else {
      const double diff = arith == 1 ? static_cast<double>(__fsub_rn(b, a))
                                     : __dsub_rn(static_cast<double>(b), static_cast<double>(a));
      res = __dadd_rn(static_cast<double>(a), __dmul_rn(diff, gamma_d));
      if (gamma_d >= 0.5) res = __dsub_rn(static_cast<double>(b), __dmul_rn(diff, __dsub_rn(1.0, gamma_d)));
    }
    *thr_out = res;
    if (ab_out) {
      ab_out[0] = a;
      ab_out[1] = b;
    }
  }
}

__global__ void __launch_bounds__(256)
threshold_dev_kernel(const float* __restrict__ vals, long long n, const double* __restrict__ thr,
                     uint8_t* __restrict__ keep) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i < n) keep[i] = static_cast<double>(vals[i]) > *thr ? 1 : 0;
}

// ---------------------------------------------------------------------------------------------
// Thresholding and list building
// ---------------------------------------------------------------------------------------------
// keep[i] = vals[i] > thr  (compared in double: exact for both float32 and float64 thresholds)
__global__ void __launch_bounds__(256)
threshold_kernel(const float* __restrict__ vals, long long n, double thr, uint8_t* __restrict__ keep) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i < n) keep[i] = static_cast<double>(vals[i]) > thr ? 1 : 0;
}

// One block per segment: counts[s] = number of set flags in keep[seg_ptr[s] .. seg_ptr[s+1]).
__global__ void __launch_bounds__(256)
segment_count_kernel(const uint8_t* __restrict__ keep, const long long* __restrict__ seg_ptr,
                     int* __restrict__ counts) {
  const long long a = seg_ptr[blockIdx.x], b = seg_ptr[blockIdx.x + 1];
  int c = 0;
  for (long long i = a + threadIdx.x; i < b; i += blockDim.x) c += keep[i];
  __shared__ int red[256];
  red[threadIdx.x] = c;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[blockIdx.x] = red[0];
}

// out_ptr[0..n] = exclusive prefix sums of counts[0..n): one block, so that the lists can be compacted
// without the counts going to the host and back.
__global__ void __launch_bounds__(256)
segment_offsets_kernel(const int* __restrict__ counts, int n, int* __restrict__ out_ptr) {
  __shared__ int part[256];
  __shared__ int carry;
  if (threadIdx.x == 0) {
    carry = 0;
    out_ptr[0] = 0;
  }
  __syncthreads();
  for (int base = 0; base < n; base += 256) {
    const int i = base + threadIdx.x;
    const int c = i < n ? counts[i] : 0;
    part[threadIdx.x] = c;
    __syncthreads();
    for (int o = 1; o < 256; o <<= 1) {
      const int add = threadIdx.x >= o ? part[threadIdx.x - o] : 0;
      __syncthreads();
      part[threadIdx.x] += add;
      __syncthreads();
    }
    if (i < n) out_ptr[i + 1] = carry + part[threadIdx.x];
    __syncthreads();
    if (threadIdx.x == 255) carry += part[255];
    __syncthreads();
  }
}

// One block per segment: list[out_ptr[s] + r] = position (inside the segment) of its r-th set flag.
__global__ void __launch_bounds__(256)
segment_compact_kernel(const uint8_t* __restrict__ keep, const long long* __restrict__ seg_ptr,
                       const int* __restrict__ out_ptr, int* __restrict__ list) {
  const long long a = seg_ptr[blockIdx.x], b = seg_ptr[blockIdx.x + 1];
  int* out = list + out_ptr[blockIdx.x];
  // 256 flags per step: ranks inside a warp by ballot, across the eight warps by a small table
  __shared__ int warp_cnt[8];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int base = 0;   // kept flags before this step (the same value in every thread)
  for (long long i0 = a; i0 < b; i0 += blockDim.x) {
    const long long i = i0 + threadIdx.x;
    const int f = (i < b) ? keep[i] : 0;
    const unsigned int bal = __ballot_sync(0xffffffffu, f != 0);
    if (lane == 0) warp_cnt[w] = __popc(bal);
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = warp_cnt[j];
      if (j < w) before += c;
      total += c;
    }
    if (f) out[base + before + __popc(bal & ((1u << lane) - 1u))] = static_cast<int>(i - a);
    base += total;
    __syncthreads();
  }
}

// mask[k][n] = rowkeep[tile(n)*K + k] & colkeep[n] (| residual[k][n])
__global__ void __launch_bounds__(256)
dense_mask_kernel(const uint8_t* __restrict__ rowkeep, const uint8_t* __restrict__ colkeep,
                  const int* __restrict__ tile_of_col, int K, int N, uint8_t* __restrict__ mask,
                  long long ld_mask) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const int t = tile_of_col[n];
  for (int k = blockIdx.y; k < K; k += gridDim.y) {   // gridDim.y is capped at 65535 rows
    uint8_t m = rowkeep[static_cast<long long>(t) * K + k];
    if (colkeep) m &= colkeep[n];
    mask[static_cast<long long>(k) * ld_mask + n] = m;
  }
}

// Same result, 16 mask bytes per thread and kDenseRows rows per block: needs N, ld_mask and the
// mask pointer to be multiples of 16.  The column flags and tile ids of a thread's 16 columns are
// read once and reused for every row; one row-keep byte serves the whole run when the 16 columns
// share a tile.
constexpr int kDenseRows = 16;

__global__ void __launch_bounds__(256)
dense_mask16_kernel(const uint8_t* __restrict__ rowkeep, const uint8_t* __restrict__ colkeep,
                    const int* __restrict__ tile_of_col, int K, int N, uint8_t* __restrict__ mask,
                    long long ld_mask) {
  const int n0 = (blockIdx.x * blockDim.x + threadIdx.x) * 16;
  if (n0 >= N) return;
  int tile[16];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int4 v = *reinterpret_cast<const int4*>(tile_of_col + n0 + q * 4);
    tile[q * 4 + 0] = v.x; tile[q * 4 + 1] = v.y; tile[q * 4 + 2] = v.z; tile[q * 4 + 3] = v.w;
  }
  bool same = true;
#pragma unroll
  for (int j = 1; j < 16; ++j) same &= tile[j] == tile[0];
  uint32_t cmask[4] = {0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u};
  if (colkeep) {
    const uint4 c = *reinterpret_cast<const uint4*>(colkeep + n0);
    cmask[0] = c.x; cmask[1] = c.y; cmask[2] = c.z; cmask[3] = c.w;
  }
  const int k_begin = blockIdx.y * kDenseRows;
  const int k_end = min(K, k_begin + kDenseRows);
  for (int k = k_begin; k < k_end; ++k) {
    uint32_t w[4];
    if (same) {
      const uint32_t b = rowkeep[static_cast<long long>(tile[0]) * K + k] * 0x01010101u;
      w[0] = w[1] = w[2] = w[3] = b;
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t x = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          x |= static_cast<uint32_t>(rowkeep[static_cast<long long>(tile[q * 4 + j]) * K + k]) << (8 * j);
        w[q] = x;
      }
    }
    uint4 o;
    o.x = w[0] & cmask[0]; o.y = w[1] & cmask[1]; o.z = w[2] & cmask[2]; o.w = w[3] & cmask[3];
    *reinterpret_cast<uint4*>(mask + static_cast<long long>(k) * ld_mask + n0) = o;
  }
}

// vals[k*N + n] = |score[k][n]|   (element-wise baseline, prune_algo.py:38-46)
__global__ void __launch_bounds__(256)
abs_values_kernel(const float* __restrict__ score, long long ld, int K, int N, float* __restrict__ vals) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  for (int k = blockIdx.y; k < K; k += gridDim.y) {
    vals[static_cast<long long>(k) * N + n] = fabsf(__ldg(score + static_cast<long long>(k) * ld + n));
  }
}

// Vector-wise baseline (prune_algo.py:196-227): one thread per (block of 16 rows, column) keeps the
// elements above the block's (topk+1)-th largest value (duplicates counted), or above 0 when the
// block has at most topk+1 rows.
constexpr int kVwBlock = 16;

__global__ void __launch_bounds__(256)
vw_mask_kernel(const float* __restrict__ score, long long ld, int K, int N, int topk,
               uint8_t* __restrict__ mask, long long ld_mask) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int k0 = blockIdx.y * kVwBlock;
  if (n >= N) return;
  const int len = min(kVwBlock, K - k0);
  float v[kVwBlock];
#pragma unroll
  for (int i = 0; i < kVwBlock; ++i) {
    v[i] = i < len ? __ldg(score + static_cast<long long>(k0 + i) * ld + n) : 0.0f;
  }
  float thr = 0.0f;
  if (topk + 1 < len) {
#pragma unroll
    for (int i = 0; i < kVwBlock; ++i) {
      if (i < len) {
        int gt = 0, ge = 0;
#pragma unroll
        for (int j = 0; j < kVwBlock; ++j) {
          if (j < len) {
            gt += v[j] > v[i];
            ge += v[j] >= v[i];
          }
        }
        if (gt <= topk && topk < ge) thr = v[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kVwBlock; ++i) {
    if (i < len) mask[static_cast<long long>(k0 + i) * ld_mask + n] = v[i] > thr ? 1 : 0;
  }
}

// Block-wise baseline (prune_algo.py:229-264): Frobenius norm of every 32 x 32 block (ragged at the
// edges), blocks numbered row-major.  The reference's norm of a 2-D slice goes through BLAS sdot, whose
// summation order depends on the host CPU, so there is no order to reproduce: one warp per block, lane =
// column, rows in order, then a shuffle tree.  grid (ceil(nbj / 8), nbi), block 256 = 8 warps.
constexpr int kBwBlock = 32;

__global__ void __launch_bounds__(256)
block_norms_kernel(const float* __restrict__ score, long long ld, int K, int N, int nbj, float* __restrict__ out) {
  const int bj = blockIdx.x * 8 + (threadIdx.x >> 5), bi = blockIdx.y;
  if (bj >= nbj) return;
  const int lane = threadIdx.x & 31;
  const int n = bj * kBwBlock + lane;
  const int k0 = bi * kBwBlock, k1 = min(K, k0 + kBwBlock);
  float acc = 0.0f;
  if (n < N) {
    for (int k = k0; k < k1; ++k) {
      const float x = __ldg(score + static_cast<long long>(k) * ld + n);
      acc = fmaf(x, x, acc);
    }
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[static_cast<long long>(bi) * nbj + bj] = sqrtf(acc);
}

// mask[k][n] = keep[(k / 32) * nbj + n / 32]
__global__ void __launch_bounds__(256)
block_mask_kernel(const uint8_t* __restrict__ keep, int K, int N, int nbj, uint8_t* __restrict__ mask,
                  long long ld_mask) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  for (int k = blockIdx.y; k < K; k += gridDim.y) {
    mask[static_cast<long long>(k) * ld_mask + n] = keep[static_cast<long long>(k / kBwBlock) * nbj + n / kBwBlock];
  }
}

// TEW ranking values: v[k*N + n] = sqrt(w*w) - mask[k][n]   (prune_algo.py:156-159)
__global__ void __launch_bounds__(256)
tew_values_kernel(const float* __restrict__ score, long long ld, const uint8_t* __restrict__ mask,
                  long long ld_mask, int K, int N, float* __restrict__ vals) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  for (int k = blockIdx.y; k < K; k += gridDim.y) {
    const float x = __ldg(score + static_cast<long long>(k) * ld + n);
    const float a = __fsqrt_rn(__fmul_rn(x, x));
    const float m = mask[static_cast<long long>(k) * ld_mask + n] ? 1.0f : 0.0f;
    vals[static_cast<long long>(k) * N + n] = __fsub_rn(a, m);
  }
}

// mask[k][n] |= v > thr; residual[k][n] = (v > thr) & !mask_before   (prune_algo.py:171-175)
__global__ void __launch_bounds__(256)
tew_apply_kernel(const float* __restrict__ vals, const double* __restrict__ thr_dev, int K, int N,
                 uint8_t* __restrict__ mask, long long ld_mask, uint8_t* __restrict__ residual) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const double thr = *thr_dev;
  for (int k = blockIdx.y; k < K; k += gridDim.y) {
    const long long mi = static_cast<long long>(k) * ld_mask + n;
    const bool extra = static_cast<double>(vals[static_cast<long long>(k) * N + n]) > thr;
    const uint8_t before = mask[mi];
    if (residual) residual[static_cast<long long>(k) * N + n] = (extra && !before) ? 1 : 0;
    if (extra) mask[mi] = 1;
  }
}

// ---------------------------------------------------------------------------------------------
// Per-tile selection by rank counting (one block per tile, the tile's K values in shared memory)
// ---------------------------------------------------------------------------------------------
// mode 0: keep the k_keep largest values, ties to the lower row index.
// mode 1: per-tile percentile (MyHook.py:202-214): the two order statistics at ranks pi / ni are
//         written to stats[2t], stats[2t+1]; the host interpolates and thresholds afterwards.
__global__ void __launch_bounds__(256)
tile_rank_kernel(const float* __restrict__ vals, int K, int mode, int k_keep, int pi, int ni,
                 uint8_t* __restrict__ keep, float* __restrict__ stats) {
  extern __shared__ float sv[];
  const float* v = vals + static_cast<long long>(blockIdx.x) * K;
  for (int i = threadIdx.x; i < K; i += blockDim.x) sv[i] = v[i];
  __syncthreads();
  for (int i = threadIdx.x; i < K; i += blockDim.x) {
    const float x = sv[i];
    int rank = 0;
    if (mode == 0) {
      for (int jj = 0; jj < K; ++jj) {
        const float y = sv[jj];
        rank += (y > x) || (y == x && jj < i);
      }
      keep[static_cast<long long>(blockIdx.x) * K + i] = rank < k_keep ? 1 : 0;
    } else {
      for (int jj = 0; jj < K; ++jj) {
        const float y = sv[jj];
        rank += (y < x) || (y == x && jj < i);
      }
      if (rank == pi) stats[2 * blockIdx.x] = x;
      if (rank == ni) stats[2 * blockIdx.x + 1] = x;
    }
  }
}

// keep[t*K + k] = vals[t*K + k] > thr[t]
__global__ void __launch_bounds__(256)
threshold_per_tile_kernel(const float* __restrict__ vals, int K, const double* __restrict__ thr,
                          uint8_t* __restrict__ keep) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  const int t = blockIdx.y;
  if (k >= K) return;
  const long long i = static_cast<long long>(t) * K + k;
  keep[i] = static_cast<double>(vals[i]) > thr[t] ? 1 : 0;
}

int stream_grid(long long n) {
  long long b = (n + 255) / 256;
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace

cudaError_t tile_row_norms_launch(const float* score, long long ld, int K, const int* bounds_dev,
                                  int n_tiles, const uint8_t* colmask, float* norms, int divide,
                                  int n_uniform128, cudaStream_t s) {
  if (K <= 0 || n_tiles <= 0) return cudaSuccess;
  // the first n_uniform128 tiles are known to be the fixed tiles [128 t, 128 (t+1)) without a
  // column mask: they take the staged fast path, the others the general kernel
  int first = 0;
  if (!colmask && n_uniform128 > 0) {
    first = n_uniform128 < n_tiles ? n_uniform128 : n_tiles;
    dim3 grid((K + 31) / 32, first);
    tile_row_norms128_kernel<<<grid, 256, 0, s>>>(score, ld, K, norms, divide);
  }
  if (first < n_tiles) {
    dim3 grid((K + 31) / 32, n_tiles - first);
    tile_row_norms_kernel<<<grid, 256, 0, s>>>(score, ld, K, bounds_dev + first, colmask,
                                               norms + static_cast<long long>(first) * K, divide);
  }
  return cudaGetLastError();
}

cudaError_t tile_row_l1_launch(const float* score, long long ld, int K, const int* bounds_dev,
                               int n_tiles, float* out, cudaStream_t s) {
  if (K <= 0 || n_tiles <= 0) return cudaSuccess;
  dim3 grid((K + 255) / 256, n_tiles);
  tile_row_l1_kernel<<<grid, 256, 0, s>>>(score, ld, K, bounds_dev, out);
  return cudaGetLastError();
}

cudaError_t col_norms_launch(const float* score, long long ld, int K, int N, float* out,
                             cudaStream_t s) {
  if (K <= 0 || N <= 0) return cudaSuccess;
  col_norms_kernel<<<(N + kColsPerBlock - 1) / kColsPerBlock, 256, 0, s>>>(score, ld, K, N, out);
  return cudaGetLastError();
}

cudaError_t select_hist_launch(const float* vals, long long n, uint32_t prefix, int shift,
                               unsigned int* hist, cudaStream_t s) {
  select_hist_kernel<<<stream_grid(n), 256, 0, s>>>(vals, n, prefix, shift, hist);
  return cudaGetLastError();
}

cudaError_t select_neighbor_launch(const float* vals, long long n, uint32_t key,
                                   unsigned long long* count_le, unsigned int* min_gt,
                                   cudaStream_t s) {
  select_neighbor_kernel<<<stream_grid(n), 256, 0, s>>>(vals, n, key, count_le, min_gt);
  return cudaGetLastError();
}

cudaError_t percentile_dev_launch(const float* vals, long long n, long long pi, long long ni, float gamma_f,
                                  double gamma_d, int arith, SelectState* st, unsigned int* hist,
                                  double* thr_out, float* ab_out, cudaStream_t s) {
  if (n <= kSmallSelect) {
    // `hist` stays all-zero, as every multi-kernel select leaves it
    percentile_small_kernel<<<1, 1024, 0, s>>>(vals, static_cast<int>(n), pi, ni, gamma_f, gamma_d, arith, st,
                                               thr_out, ab_out);
    return cudaGetLastError();
  }
  select_begin_kernel<<<1, 256, 0, s>>>(st, hist, static_cast<unsigned long long>(pi));
  for (int shift = 24; shift >= 0; shift -= 8) {
    select_hist_dev_kernel<<<stream_grid(n), 256, 0, s>>>(vals, n, st, shift, hist);
    select_pick_kernel<<<1, 256, 0, s>>>(st, hist, shift);
  }
  if (ni != pi) select_neighbor_dev_kernel<<<stream_grid(n), 256, 0, s>>>(vals, n, st);
  select_finish_kernel<<<1, 1, 0, s>>>(st, pi, ni, gamma_f, gamma_d, arith, thr_out, ab_out);
  return cudaGetLastError();
}

cudaError_t threshold_dev_launch(const float* vals, long long n, const double* thr, uint8_t* keep,
                                 cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  threshold_dev_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(vals, n, thr, keep);
  return cudaGetLastError();
}

cudaError_t threshold_launch(const float* vals, long long n, double thr, uint8_t* keep,
                             cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  threshold_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(vals, n, thr, keep);
  return cudaGetLastError();
}

cudaError_t segment_count_launch(const uint8_t* keep, const long long* seg_ptr, int n_seg, int* counts,
                                 cudaStream_t s) {
  if (n_seg <= 0) return cudaSuccess;
  segment_count_kernel<<<n_seg, 256, 0, s>>>(keep, seg_ptr, counts);
  return cudaGetLastError();
}

cudaError_t segment_offsets_launch(const int* counts, int n_seg, int* out_ptr, cudaStream_t s) {
  segment_offsets_kernel<<<1, 256, 0, s>>>(counts, n_seg < 0 ? 0 : n_seg, out_ptr);
  return cudaGetLastError();
}

cudaError_t segment_compact_launch(const uint8_t* keep, const long long* seg_ptr, int n_seg,
                                   const int* out_ptr, int* list, cudaStream_t s) {
  if (n_seg <= 0) return cudaSuccess;
  segment_compact_kernel<<<n_seg, 256, 0, s>>>(keep, seg_ptr, out_ptr, list);
  return cudaGetLastError();
}

cudaError_t dense_mask_launch(const uint8_t* rowkeep, const uint8_t* colkeep, const int* tile_of_col,
                              int K, int N, uint8_t* mask, long long ld_mask, cudaStream_t s) {
  if (K <= 0 || N <= 0) return cudaSuccess;
  const bool aligned = N % 16 == 0 && ld_mask % 16 == 0 && reinterpret_cast<uintptr_t>(mask) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(tile_of_col) % 16 == 0 &&
                       (!colkeep || reinterpret_cast<uintptr_t>(colkeep) % 16 == 0);
  if (aligned) {
    const int threads = N / 16 >= 128 ? 128 : 64;
    dim3 grid16((N / 16 + threads - 1) / threads, (K + kDenseRows - 1) / kDenseRows);
    dense_mask16_kernel<<<grid16, threads, 0, s>>>(rowkeep, colkeep, tile_of_col, K, N, mask, ld_mask);
    return cudaGetLastError();
  }
  dim3 grid((N + 255) / 256, K < 65535 ? K : 65535);
  dense_mask_kernel<<<grid, 256, 0, s>>>(rowkeep, colkeep, tile_of_col, K, N, mask, ld_mask);
  return cudaGetLastError();
}

cudaError_t abs_values_launch(const float* score, long long ld, int K, int N, float* vals, cudaStream_t s) {
  if (K <= 0 || N <= 0) return cudaSuccess;
  dim3 grid((N + 255) / 256, K < 65535 ? K : 65535);
  abs_values_kernel<<<grid, 256, 0, s>>>(score, ld, K, N, vals);
  return cudaGetLastError();
}

cudaError_t vw_mask_launch(const float* score, long long ld, int K, int N, int topk, uint8_t* mask,
                           long long ld_mask, cudaStream_t s) {
  if (K <= 0 || N <= 0) return cudaSuccess;
  dim3 grid((N + 127) / 128, (K + kVwBlock - 1) / kVwBlock);
  vw_mask_kernel<<<grid, 128, 0, s>>>(score, ld, K, N, topk, mask, ld_mask);
  return cudaGetLastError();
}

cudaError_t block_norms_launch(const float* score, long long ld, int K, int N, float* out, cudaStream_t s) {
  const int nbi = (K + kBwBlock - 1) / kBwBlock, nbj = (N + kBwBlock - 1) / kBwBlock;
  dim3 grid((nbj + 7) / 8, nbi);
  block_norms_kernel<<<grid, 256, 0, s>>>(score, ld, K, N, nbj, out);
  return cudaGetLastError();
}

cudaError_t block_mask_launch(const uint8_t* keep, int K, int N, uint8_t* mask, long long ld_mask, cudaStream_t s) {
  const int nbj = (N + kBwBlock - 1) / kBwBlock;
  dim3 grid((N + 255) / 256, K < 65535 ? K : 65535);
  block_mask_kernel<<<grid, 256, 0, s>>>(keep, K, N, nbj, mask, ld_mask);
  return cudaGetLastError();
}

cudaError_t tew_values_launch(const float* score, long long ld, const uint8_t* mask, long long ld_mask,
                              int K, int N, float* vals, cudaStream_t s) {
  if (K <= 0 || N <= 0) return cudaSuccess;
  dim3 grid((N + 255) / 256, K < 65535 ? K : 65535);
  tew_values_kernel<<<grid, 256, 0, s>>>(score, ld, mask, ld_mask, K, N, vals);
  return cudaGetLastError();
}

cudaError_t tew_apply_launch(const float* vals, const double* thr, int K, int N, uint8_t* mask,
                             long long ld_mask, uint8_t* residual, cudaStream_t s) {
  if (K <= 0 || N <= 0) return cudaSuccess;
  dim3 grid((N + 255) / 256, K < 65535 ? K : 65535);
  tew_apply_kernel<<<grid, 256, 0, s>>>(vals, thr, K, N, mask, ld_mask, residual);
  return cudaGetLastError();
}

cudaError_t tile_rank_launch(const float* vals, int K, int n_tiles, int mode, int k_keep, int pi,
                             int ni, uint8_t* keep, float* stats, cudaStream_t s) {
  if (K <= 0 || n_tiles <= 0) return cudaSuccess;
  const size_t smem = static_cast<size_t>(K) * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(tile_rank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  tile_rank_kernel<<<n_tiles, 256, smem, s>>>(vals, K, mode, k_keep, pi, ni, keep, stats);
  return cudaGetLastError();
}

cudaError_t threshold_per_tile_launch(const float* vals, int K, int n_tiles, const double* thr,
                                      uint8_t* keep, cudaStream_t s) {
  if (K <= 0 || n_tiles <= 0) return cudaSuccess;
  dim3 grid((K + 255) / 256, n_tiles);
  threshold_per_tile_kernel<<<grid, 256, 0, s>>>(vals, K, thr, keep);
  return cudaGetLastError();
}

}  // namespace ts

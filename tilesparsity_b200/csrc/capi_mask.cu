// C ABI of the mask builder: host orchestration of the kernels in mask_build.cu.
//
// The host side owns the parts of the reference algorithm that are scalar: the percentile's index
// arithmetic and interpolation (np.percentile, method "linear"), the sparsity remap of the 2-D
// variant (Pruning/VGG/prune_algo.py:61) and the regrouping of surviving columns into tiles
// (prune_algo.py:72-89).  They are written as single IEEE-754 operations in the arithmetic type
// NumPy would use, so that thresholds, and with them the masks, come out bit-identical.
#include "../../include/tilesparse.h"

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <limits>
#include <mutex>
#include <string>
#include <vector>

#include "ts_mask_kernels.h"

// error reporting shared with capi.cu
int ts_internal_fail(int code, const char* fmt, ...);

namespace {

#define TSM_CUDA(expr)                                                                         \
  do {                                                                                         \
    cudaError_t e_ = (expr);                                                                   \
    if (e_ != cudaSuccess) {                                                                   \
      return ts_internal_fail(e_ == cudaErrorMemoryAllocation ? TS_ERR_NOMEM : TS_ERR_CUDA,    \
                              "%s failed: %s", #expr, cudaGetErrorString(e_));                 \
    }                                                                                          \
  } while (0)

#define TSM_OK(expr)          \
  do {                        \
    int rc_ = (expr);         \
    if (rc_ != TS_OK) return rc_; \
  } while (0)

// Device scratch of one call: carved out of a block that is kept between calls (one per device, grown
// on demand), so a mask build in steady state makes no cudaMalloc / cudaFree calls (each of which
// would synchronise the device).  Calls on one device take turns: the lock is held for the whole
// call.  If a call needs more than the block holds, the extra allocations are individual and freed
// at the end of the call, and the block is replaced by a larger one for the next call.
struct ScratchBlock {
  void* base = nullptr;
  size_t cap = 0;
  void* pinned = nullptr;      // page-locked host block for the read-backs (asynchronous copies)
  size_t pinned_cap = 0;
  std::mutex mu;
};
ScratchBlock g_scratch[64];

struct Arena {
  ScratchBlock* blk = nullptr;
  size_t used = 0, wanted = 0;
  std::vector<void*> extra;
  std::unique_lock<std::mutex> lock;

  Arena() {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
      blk = &g_scratch[dev];
      lock = std::unique_lock<std::mutex>(blk->mu);
    }
  }
  ~Arena() {
    for (void* p : extra) cudaFree(p);
    if (blk && wanted > blk->cap) {   // grow the kept block for the next call
      cudaFree(blk->base);
      blk->base = nullptr;
      blk->cap = 0;
      const size_t want = wanted + wanted / 4 + (1 << 20);
      if (cudaMalloc(&blk->base, want) == cudaSuccess) blk->cap = want;
      else cudaGetLastError();
    }
  }
  // Page-locked host memory of at least `bytes` (kept between calls, grown on demand), or nullptr when
  // it cannot be had or the request is unreasonably large: the caller then copies to pageable memory.
  void* pinned(size_t bytes) {
    if (!blk || bytes > (static_cast<size_t>(8) << 20)) return nullptr;
    if (bytes > blk->pinned_cap) {
      if (blk->pinned) cudaFreeHost(blk->pinned);
      blk->pinned = nullptr;
      blk->pinned_cap = 0;
      const size_t want = std::max<size_t>(bytes + bytes / 2, static_cast<size_t>(1) << 18);
      if (cudaHostAlloc(&blk->pinned, want, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError();
        blk->pinned = nullptr;
        return nullptr;
      }
      blk->pinned_cap = want;
    }
    return blk->pinned;
  }
  template <typename T>
  int alloc(T** out, size_t count) {
    const size_t bytes = (std::max<size_t>(count, 1) * sizeof(T) + 255) & ~static_cast<size_t>(255);
    wanted += bytes;
    if (blk && blk->base && used + bytes <= blk->cap) {
      *out = reinterpret_cast<T*>(static_cast<char*>(blk->base) + used);
      used += bytes;
      return TS_OK;
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
      return ts_internal_fail(TS_ERR_NOMEM, "device allocation of %zu bytes failed: %s", bytes,
                              cudaGetErrorString(e));
    }
    extra.push_back(p);
    *out = static_cast<T*>(p);
    return TS_OK;
  }
};

uint32_t float_key(float f) {
  uint32_t b;
  memcpy(&b, &f, 4);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

float key_float(uint32_t k) {
  const uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  float f;
  memcpy(&f, &b, 4);
  return f;
}

// The pi-th and ni-th smallest of vals[0..n) (0-based, pi <= ni <= pi+1), by an 8-bit radix select
// driven from the host (four histogram passes, then one pass for the upper neighbour).
// scratch: 256 uint32 + one uint64 + one uint32, all on the device.
int order_statistics(const float* vals, long long n, long long pi, long long ni, float* a, float* b,
                     unsigned int* d_hist, unsigned long long* d_count, unsigned int* d_min,
                     cudaStream_t s) {
  if (n <= 0 || pi < 0 || ni >= n || ni < pi || ni > pi + 1) {
    return ts_internal_fail(TS_ERR_INVALID, "order_statistics: bad ranks %lld/%lld of %lld", pi, ni, n);
  }
  uint32_t prefix = 0;
  long long rank = pi;
  unsigned int hist[256];
  for (int shift = 24; shift >= 0; shift -= 8) {
    TSM_CUDA(cudaMemsetAsync(d_hist, 0, 256 * sizeof(unsigned int), s));
    TSM_CUDA(ts::select_hist_launch(vals, n, prefix, shift, d_hist, s));
    TSM_CUDA(cudaMemcpyAsync(hist, d_hist, sizeof(hist), cudaMemcpyDeviceToHost, s));
    TSM_CUDA(cudaStreamSynchronize(s));
    long long cum = 0;
    int d = 0;
    for (; d < 256; ++d) {
      if (cum + hist[d] > rank) break;
      cum += hist[d];
    }
    if (d == 256) return ts_internal_fail(TS_ERR_CUDA, "radix select lost its rank (non-finite input?)");
    rank -= cum;
    prefix |= static_cast<uint32_t>(d) << shift;
  }
  *a = key_float(prefix);
  *b = *a;
  if (ni != pi) {
    const unsigned int init_min = 0xffffffffu;
    TSM_CUDA(cudaMemsetAsync(d_count, 0, sizeof(unsigned long long), s));
    TSM_CUDA(cudaMemcpyAsync(d_min, &init_min, sizeof(init_min), cudaMemcpyHostToDevice, s));
    TSM_CUDA(ts::select_neighbor_launch(vals, n, prefix, d_count, d_min, s));
    unsigned long long count_le = 0;
    unsigned int min_gt = 0;
    TSM_CUDA(cudaMemcpyAsync(&count_le, d_count, sizeof(count_le), cudaMemcpyDeviceToHost, s));
    TSM_CUDA(cudaMemcpyAsync(&min_gt, d_min, sizeof(min_gt), cudaMemcpyDeviceToHost, s));
    TSM_CUDA(cudaStreamSynchronize(s));
    if (static_cast<long long>(count_le) < ni + 1) *b = key_float(min_gt);  // next rank is a larger value
  }
  return TS_OK;
}

// np.percentile's rank arithmetic ("linear": virtual index (n-1)*q, neighbours floor and floor+1).
// With a weak (Python) q everything is float32; with a float64 q it is double.
struct Ranks {
  long long pi, ni;
  float gamma_f;
  double gamma_d;
};

Ranks percentile_ranks(long long n, double q, bool wide) {
  Ranks r;
  if (wide) {
    volatile double qd = q / 100.0;
    volatile double virt = static_cast<double>(n - 1) * qd;
    const double prev = std::floor(virt);
    r.pi = static_cast<long long>(prev);
    r.ni = r.pi + 1;
    if (virt >= static_cast<double>(n - 1)) r.pi = r.ni = n - 1;
    r.gamma_d = virt - prev;
    r.gamma_f = 0.0f;
  } else {
    volatile float qf = static_cast<float>(q) / 100.0f;
    volatile float virt = static_cast<float>(n - 1) * qf;
    const float prev = std::floor(virt);
    r.pi = static_cast<long long>(prev);
    r.ni = r.pi + 1;
    if (virt >= static_cast<float>(n - 1)) r.pi = r.ni = n - 1;
    r.gamma_f = virt - prev;
    r.gamma_d = 0.0;
  }
  if (r.pi < 0) r.pi = r.ni = 0;
  if (r.ni > n - 1) r.ni = n - 1;
  return r;
}

// NumPy's _lerp: a + (b-a)*t, replaced by b - (b-a)*(1-t) when t >= 0.5.  The difference b-a is a
// float32 operation in both paths (a and b are float32 array elements); the rest follows t's type.
double percentile_lerp(float a, float b, const Ranks& r, bool wide) {
  volatile float diff = b - a;
  if (wide) {
    const double t = r.gamma_d;
    volatile double prod = static_cast<double>(diff) * t;
    volatile double res = static_cast<double>(a) + prod;
    if (t >= 0.5) {
      volatile double omt = 1.0 - t;
      volatile double prod2 = static_cast<double>(diff) * omt;
      res = static_cast<double>(b) - prod2;
    }
    return res;
  }
  const float t = r.gamma_f;
  volatile float prod = diff * t;
  volatile float res = a + prod;
  if (t >= 0.5f) {
    volatile float omt = 1.0f - t;
    volatile float prod2 = diff * omt;
    res = b - prod2;
  }
  return static_cast<double>(res);
}

// A tile ends right after its G-th kept column; no cut at the matrix edge (prune_algo.py:72-89).
std::vector<int> regroup_bounds(const uint8_t* colkeep, int N, int G) {
  std::vector<int> b{0};
  int count = 0;
  for (int c = 0; c < N; ++c) {
    if (colkeep[c]) ++count;
    if (count == G) {
      if (c + 1 < N) {
        b.push_back(c + 1);
        count = 0;
      }
    }
  }
  b.push_back(N);
  return b;
}

std::vector<int> fixed_bounds(int N, int G) {
  std::vector<int> b;
  for (int c = 0; c < N; c += G) b.push_back(c);
  b.push_back(N);
  return b;
}

struct LayerIn {
  const float* score;     // float32 scores, or (f64 row stage) the same pointer holding doubles
  int K, N;
  long long ld;
  uint8_t* mask;
  long long ld_mask;
  uint8_t* residual;
};

}  // namespace

struct ts_mask_result {
  struct Layer {
    int K = 0, N = 0;
    std::vector<int> bounds, tile_k_ptr, kept_k, tile_n_ptr, kept_n;
  };
  std::vector<Layer> layers;
  double thr[3] = {std::numeric_limits<double>::quiet_NaN(), std::numeric_limits<double>::quiet_NaN(),
                   std::numeric_limits<double>::quiet_NaN()};
};

namespace {

struct Scratch {
  ts::SelectState64* st64 = nullptr;   // state of the double-precision select
  unsigned int* hist = nullptr;
  unsigned long long* count = nullptr;
  unsigned int* min_gt = nullptr;
  ts::SelectState* st = nullptr;   // state of the device-driven select
  double* thr = nullptr;           // 4 thresholds on the device: column stage, row stage, residual, spare
};

int alloc_scratch(Arena& arena, Scratch* sc) {
  TSM_OK(arena.alloc(&sc->hist, 256));
  TSM_OK(arena.alloc(&sc->count, 1));
  TSM_OK(arena.alloc(&sc->min_gt, 1));
  TSM_OK(arena.alloc(&sc->st, 1));
  TSM_OK(arena.alloc(&sc->st64, 1));
  TSM_OK(arena.alloc(&sc->thr, 4));
  return TS_OK;
}

// np.percentile(vals, q) into sc.thr[slot], enqueued on s without reading anything back.
int percentile_to_device(const float* vals, long long n, double q, bool wide, bool f64_values, const Scratch& sc,
                         int slot, cudaStream_t s) {
  if (n <= 0) return ts_internal_fail(TS_ERR_INVALID, "percentile of an empty set");
  const Ranks r = percentile_ranks(n, q, wide);
  const int arith = f64_values ? 2 : (wide ? 1 : 0);
  TSM_CUDA(ts::percentile_dev_launch(vals, n, r.pi, r.ni, r.gamma_f, r.gamma_d, arith, sc.st, sc.hist,
                                     sc.thr + slot, nullptr, s));
  return TS_OK;
}

// Reads thresholds and the select's error flag back (one blocking copy each).
int read_thresholds(const Scratch& sc, int slot, double* out, cudaStream_t s) {
  ts::SelectState st;
  TSM_CUDA(cudaMemcpyAsync(out, sc.thr + slot, sizeof(double), cudaMemcpyDeviceToHost, s));
  TSM_CUDA(cudaMemcpyAsync(&st, sc.st, sizeof(st), cudaMemcpyDeviceToHost, s));
  TSM_CUDA(cudaStreamSynchronize(s));
  if (st.error) return ts_internal_fail(TS_ERR_CUDA, "radix select lost its rank (non-finite input?)");
  return TS_OK;
}

// Row stage shared by every mode: norms of all tile-rows of all layers, a keep flag for each, the
// per-tile kept-row lists, and (optionally) the dense masks.
//   sel: 0 = one global percentile over all layers (tw1 / tw2 stage 2), 1 = per-tile percentile
//        (BERT type 2), 2 = per-tile top-k by L1 (k = round(K * (1 - q/100))).
int row_stage(const std::vector<LayerIn>& L, const std::vector<std::vector<int>>& bounds,
              const std::vector<uint8_t*>& colkeep_dev, const std::vector<std::vector<uint8_t>>& colkeep_host,
              int sel, double q, bool wide, ts_mask_result* res, double* thr_out, Arena& arena,
              const Scratch& sc, cudaStream_t s, bool f64 = false) {
  const int nl = static_cast<int>(L.size());
  std::vector<long long> off(nl + 1, 0);
  std::vector<int> tile_off(nl + 1, 0);
  for (int l = 0; l < nl; ++l) {
    const int nt = static_cast<int>(bounds[l].size()) - 1;
    off[l + 1] = off[l] + static_cast<long long>(nt) * L[l].K;
    tile_off[l + 1] = tile_off[l] + nt;
  }
  const long long total = off[nl];
  const int total_tiles = tile_off[nl];
  float* norms = nullptr;
  double* norms64 = nullptr;   // float64 scores: norms, percentile and comparison all in double
  uint8_t* keep = nullptr;
  if (f64) {
    if (sel != 0 || !colkeep_dev.empty()) {
      return ts_internal_fail(TS_ERR_UNSUPPORTED, "float64 scores are supported by the tw1 row stage only");
    }
    TSM_OK(arena.alloc(&norms64, total));
  } else {
    TSM_OK(arena.alloc(&norms, total));
  }
  TSM_OK(arena.alloc(&keep, total));
  std::vector<int*> bounds_dev(nl, nullptr);
  for (int l = 0; l < nl; ++l) {
    TSM_OK(arena.alloc(&bounds_dev[l], bounds[l].size()));
    TSM_CUDA(cudaMemcpyAsync(bounds_dev[l], bounds[l].data(), bounds[l].size() * sizeof(int),
                             cudaMemcpyHostToDevice, s));
    const int nt = static_cast<int>(bounds[l].size()) - 1;
    if (f64) {
      TSM_CUDA(ts::tile_row_norms64_launch(reinterpret_cast<const double*>(L[l].score), L[l].ld, L[l].K,
                                           bounds_dev[l], nt, norms64 + off[l], 1, s));
    } else if (sel == 2) {
      TSM_CUDA(ts::tile_row_l1_launch(L[l].score, L[l].ld, L[l].K, bounds_dev[l], nt, norms + off[l], s));
    } else {
      int uniform = 0;   // leading tiles that are exactly [128 t, 128 (t+1))
      if (colkeep_dev.empty()) {
        while (uniform < nt && bounds[l][uniform] == 128 * uniform && bounds[l][uniform + 1] == 128 * (uniform + 1)) ++uniform;
      }
      TSM_CUDA(ts::tile_row_norms_launch(L[l].score, L[l].ld, L[l].K, bounds_dev[l], nt,
                                         colkeep_dev.empty() ? nullptr : colkeep_dev[l], norms + off[l],
                                         sel == 0 ? 1 : 0, uniform, s));
    }
  }
  if (f64) {
    const Ranks r = percentile_ranks(total, q, true);
    TSM_CUDA(ts::percentile64_dev_launch(norms64, total, r.pi, r.ni, r.gamma_d, sc.st64, sc.hist, sc.thr + 1, s));
    TSM_CUDA(ts::threshold64_dev_launch(norms64, total, sc.thr + 1, keep, s));
    ts::SelectState64 st64;
    TSM_CUDA(cudaMemcpyAsync(&st64, sc.st64, sizeof(st64), cudaMemcpyDeviceToHost, s));
    if (thr_out) TSM_CUDA(cudaMemcpyAsync(thr_out, sc.thr + 1, sizeof(double), cudaMemcpyDeviceToHost, s));
    TSM_CUDA(cudaStreamSynchronize(s));
    if (st64.error) return ts_internal_fail(TS_ERR_CUDA, "radix select lost its rank (non-finite input?)");
  } else if (sel == 0) {
    TSM_OK(percentile_to_device(norms, total, q, wide, false, sc, 1, s));
    TSM_CUDA(ts::threshold_dev_launch(norms, total, sc.thr + 1, keep, s));
    // the threshold and the select's error flag are read back with the lists, further down
  } else {
    for (int l = 0; l < nl; ++l) {
      const int nt = static_cast<int>(bounds[l].size()) - 1;
      const int K = L[l].K;
      if (sel == 2) {
        const int k_keep = static_cast<int>(std::nearbyint(K * (1.0 - q / 100.0)));
        TSM_CUDA(ts::tile_rank_launch(norms + off[l], K, nt, 0, k_keep, 0, 0, keep + off[l], nullptr, s));
      } else {
        const Ranks r = percentile_ranks(K, q, wide);
        float* stats = nullptr;
        double* thr_dev = nullptr;
        TSM_OK(arena.alloc(&stats, 2 * static_cast<size_t>(nt)));
        TSM_OK(arena.alloc(&thr_dev, nt));
        TSM_CUDA(ts::tile_rank_launch(norms + off[l], K, nt, 1, 0, static_cast<int>(r.pi),
                                      static_cast<int>(r.ni), nullptr, stats, s));
        std::vector<float> st(2 * static_cast<size_t>(nt));
        TSM_CUDA(cudaMemcpyAsync(st.data(), stats, st.size() * sizeof(float), cudaMemcpyDeviceToHost, s));
        TSM_CUDA(cudaStreamSynchronize(s));
        std::vector<double> thr(nt);
        for (int t = 0; t < nt; ++t) thr[t] = percentile_lerp(st[2 * t], st[2 * t + 1], r, wide);
        TSM_CUDA(cudaMemcpyAsync(thr_dev, thr.data(), nt * sizeof(double), cudaMemcpyHostToDevice, s));
        TSM_CUDA(ts::threshold_per_tile_launch(norms + off[l], K, nt, thr_dev, keep + off[l], s));
        TSM_CUDA(cudaStreamSynchronize(s));  // thr (host) must outlive the copy
      }
    }
  }

  // kept-row lists: one segment per (layer, tile).  Counts, their prefix sums and the compaction all
  // stay on the device; the dense masks are enqueued behind them; one blocking read-back at the end
  // brings the thresholds, the select's error flag, the offsets and the lists.
  std::vector<long long> seg(total_tiles + 1, 0);
  for (int l = 0; l < nl; ++l) {
    const int nt = tile_off[l + 1] - tile_off[l];
    for (int t = 0; t <= nt; ++t) seg[tile_off[l] + t] = off[l] + static_cast<long long>(t) * L[l].K;
  }
  long long* seg_dev = nullptr;
  int* counts_dev = nullptr;
  int* optr_dev = nullptr;
  int* list_dev = nullptr;
  TSM_OK(arena.alloc(&seg_dev, seg.size()));
  TSM_OK(arena.alloc(&counts_dev, total_tiles));
  TSM_OK(arena.alloc(&optr_dev, total_tiles + 1));
  TSM_OK(arena.alloc(&list_dev, total));      // room for every tile-row: the kept ones are a subset
  TSM_CUDA(cudaMemcpyAsync(seg_dev, seg.data(), seg.size() * sizeof(long long), cudaMemcpyHostToDevice, s));
  TSM_CUDA(ts::segment_count_launch(keep, seg_dev, total_tiles, counts_dev, s));
  TSM_CUDA(ts::segment_offsets_launch(counts_dev, total_tiles, optr_dev, s));
  TSM_CUDA(ts::segment_compact_launch(keep, seg_dev, total_tiles, optr_dev, list_dev, s));
  std::vector<std::vector<int>> tile_of_col(nl);
  for (int l = 0; l < nl; ++l) {
    if (!L[l].mask) continue;
    const int nt = tile_off[l + 1] - tile_off[l];
    tile_of_col[l].resize(L[l].N);
    for (int t = 0; t < nt; ++t) {
      for (int c = bounds[l][t]; c < bounds[l][t + 1]; ++c) tile_of_col[l][c] = t;
    }
    int* toc_dev = nullptr;
    TSM_OK(arena.alloc(&toc_dev, tile_of_col[l].size()));
    TSM_CUDA(cudaMemcpyAsync(toc_dev, tile_of_col[l].data(), tile_of_col[l].size() * sizeof(int),
                             cudaMemcpyHostToDevice, s));
    TSM_CUDA(ts::dense_mask_launch(keep + off[l], colkeep_dev.empty() ? nullptr : colkeep_dev[l], toc_dev,
                                   L[l].K, L[l].N, L[l].mask, L[l].ld_mask, s));
  }
  // Read-back: threshold, the select's error flag, the offsets and (up to 64 Ki tile-rows) the whole
  // upper-bound list array in one round trip; beyond that the exact size is awaited first (a second
  // round trip is cheaper than the extra bytes).  The copies land in page-locked memory when it can be
  // had, so they are asynchronous and the host blocks once.
  ts::SelectState st_host;
  memset(&st_host, 0, sizeof(st_host));
  const bool want_sel = sel == 0 && !f64;
  const bool one_trip = total <= (1 << 16);
  std::vector<int> optr(total_tiles + 1, 0);
  std::vector<int> list;
  const size_t head_bytes = 256;   // [0, 8): threshold, [64, 64 + sizeof(SelectState)): select state
  static_assert(sizeof(ts::SelectState) <= head_bytes - 64, "select state does not fit the read-back header");
  const size_t optr_bytes = (optr.size() * sizeof(int) + 255) & ~static_cast<size_t>(255);
  const size_t list_bytes = one_trip ? static_cast<size_t>(total) * sizeof(int) : 0;
  char* pin = static_cast<char*>(arena.pinned(head_bytes + optr_bytes + list_bytes));
  if (pin) {
    if (want_sel) {
      TSM_CUDA(cudaMemcpyAsync(pin, sc.thr + 1, sizeof(double), cudaMemcpyDeviceToHost, s));
      TSM_CUDA(cudaMemcpyAsync(pin + 64, sc.st, sizeof(st_host), cudaMemcpyDeviceToHost, s));
    }
    TSM_CUDA(cudaMemcpyAsync(pin + head_bytes, optr_dev, optr.size() * sizeof(int), cudaMemcpyDeviceToHost, s));
    if (one_trip && total > 0) {
      TSM_CUDA(cudaMemcpyAsync(pin + head_bytes + optr_bytes, list_dev, list_bytes, cudaMemcpyDeviceToHost, s));
    }
    TSM_CUDA(cudaStreamSynchronize(s));   // seg, tile_of_col (host) must outlive their copies; everything is done
    if (want_sel) {
      if (thr_out) memcpy(thr_out, pin, sizeof(double));
      memcpy(&st_host, pin + 64, sizeof(st_host));
    }
    memcpy(optr.data(), pin + head_bytes, optr.size() * sizeof(int));
    if (one_trip) {
      const int* lp = reinterpret_cast<const int*>(pin + head_bytes + optr_bytes);
      list.assign(lp, lp + optr[total_tiles]);     // the kept ones: a prefix of the upper-bound array
    }
  } else {
    if (want_sel) {
      if (thr_out) TSM_CUDA(cudaMemcpyAsync(thr_out, sc.thr + 1, sizeof(double), cudaMemcpyDeviceToHost, s));
      TSM_CUDA(cudaMemcpyAsync(&st_host, sc.st, sizeof(st_host), cudaMemcpyDeviceToHost, s));
    }
    TSM_CUDA(cudaMemcpyAsync(optr.data(), optr_dev, optr.size() * sizeof(int), cudaMemcpyDeviceToHost, s));
    if (one_trip) {
      list.resize(total);
      if (total > 0) TSM_CUDA(cudaMemcpyAsync(list.data(), list_dev, total * sizeof(int), cudaMemcpyDeviceToHost, s));
    }
    TSM_CUDA(cudaStreamSynchronize(s));
  }
  if (st_host.error) return ts_internal_fail(TS_ERR_CUDA, "radix select lost its rank (non-finite input?)");
  if (!one_trip) {
    list.resize(optr[total_tiles]);
    if (!list.empty()) {
      TSM_CUDA(cudaMemcpyAsync(list.data(), list_dev, list.size() * sizeof(int), cudaMemcpyDeviceToHost, s));
      TSM_CUDA(cudaStreamSynchronize(s));
    }
  }

  res->layers.resize(nl);
  for (int l = 0; l < nl; ++l) {
    ts_mask_result::Layer& R = res->layers[l];
    const int nt = tile_off[l + 1] - tile_off[l];
    R.K = L[l].K;
    R.N = L[l].N;
    R.bounds = bounds[l];
    R.tile_k_ptr.assign(nt + 1, 0);
    R.tile_n_ptr.assign(nt + 1, 0);
    R.kept_k.clear();
    R.kept_n.clear();
    for (int t = 0; t < nt; ++t) {
      const int gt = tile_off[l] + t;
      R.kept_k.insert(R.kept_k.end(), list.begin() + optr[gt], list.begin() + optr[gt + 1]);
      R.tile_k_ptr[t + 1] = static_cast<int>(R.kept_k.size());
      for (int c = bounds[l][t]; c < bounds[l][t + 1]; ++c) {
        if (colkeep_host.empty() || colkeep_host[l][c]) R.kept_n.push_back(c);
      }
      R.tile_n_ptr[t + 1] = static_cast<int>(R.kept_n.size());
    }
  }
  return TS_OK;
}

}  // namespace

extern "C" {

}  // extern "C"

namespace {
int build_tw_mask_impl(int mode, int n_layers, const void* const* scores_dev, const int* Ks, const int* Ns,
                       const int64_t* lds, int G, double sparsity, int sparsity_is_f64, double g1percent,
                       uint8_t* const* masks_dev, const int64_t* ld_masks, uint8_t* const* residual_dev,
                       ts_mask_result_t** out, void* stream, bool f64) {
  if (!out) return ts_internal_fail(TS_ERR_INVALID, "out is NULL");
  *out = nullptr;
  if (mode < TS_MASK_TW1 || mode > TS_MASK_TW_COLS_ROWS) return ts_internal_fail(TS_ERR_INVALID, "unknown mode %d", mode);
  if (n_layers <= 0 || !scores_dev || !Ks || !Ns) return ts_internal_fail(TS_ERR_INVALID, "no layers");
  if (G <= 0) return ts_internal_fail(TS_ERR_INVALID, "G=%d must be positive", G);
  if (!(sparsity >= 0.0 && sparsity <= 100.0)) {
    return ts_internal_fail(TS_ERR_INVALID, "sparsity=%g must be in [0, 100]", sparsity);
  }
  const bool tew = mode == TS_MASK_TW1M || mode == TS_MASK_TW2M;
  if (tew && !(g1percent >= 0.0 && sparsity + g1percent <= 100.0)) {
    return ts_internal_fail(TS_ERR_INVALID, "g1percent=%g out of range", g1percent);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Arena arena;
  std::vector<LayerIn> L(n_layers);
  for (int l = 0; l < n_layers; ++l) {
    if (!scores_dev[l] || Ks[l] <= 0 || Ns[l] <= 0) return ts_internal_fail(TS_ERR_INVALID, "layer %d is empty", l);
    L[l].score = static_cast<const float*>(scores_dev[l]);
    L[l].K = Ks[l];
    L[l].N = Ns[l];
    L[l].ld = lds ? lds[l] : Ns[l];
    if (L[l].ld < L[l].N) return ts_internal_fail(TS_ERR_INVALID, "layer %d: ld smaller than N", l);
    // launch geometry: column tiles, and 16-row blocks of K, are grid y dimensions (at most 65535)
    if ((L[l].N + G - 1) / G > 65535 || L[l].K > 65535 * 16) {
      return ts_internal_fail(TS_ERR_UNSUPPORTED, "layer %d: %d x %d at G=%d exceeds 65535 column tiles or 1048560 rows",
                              l, L[l].K, L[l].N, G);
    }
    L[l].mask = masks_dev ? masks_dev[l] : nullptr;
    L[l].ld_mask = (ld_masks && L[l].mask) ? ld_masks[l] : Ns[l];
    L[l].residual = residual_dev ? residual_dev[l] : nullptr;
    if (tew && !L[l].mask) {  // the residual ranking needs the dense TW mask
      TSM_OK(arena.alloc(&L[l].mask, static_cast<size_t>(L[l].K) * L[l].N));
      L[l].ld_mask = L[l].N;
    }
    const bool divisible = mode == TS_MASK_BERT_PER_TILE || mode == TS_MASK_BERT_TW_K;
    if (divisible && (L[l].N % G) != 0) {
      return ts_internal_fail(TS_ERR_INVALID, "layer %d: N=%d is not divisible by the granularity %d", l, L[l].N, G);
    }
  }
  Scratch sc;
  TSM_OK(alloc_scratch(arena, &sc));
  ts_mask_result* res = new ts_mask_result();

  if (mode == TS_MASK_TW_COLS_ROWS && !(g1percent >= 0.0 && g1percent <= 100.0)) {
    return ts_internal_fail(TS_ERR_INVALID, "column sparsity %g must be in [0, 100]", g1percent);
  }
  const bool two_d = mode == TS_MASK_TW2 || mode == TS_MASK_TW2M || mode == TS_MASK_BERT_TW_KN ||
                     mode == TS_MASK_TW_COLS_ROWS;
  double q = tew ? sparsity + g1percent : sparsity;
  bool wide = sparsity_is_f64 != 0;
  if (mode == TS_MASK_TW2 || mode == TS_MASK_TW2M) {
    volatile double x = q * 100.0;
    volatile double y = 10000.0 - x;
    volatile double z = std::sqrt(y);
    q = 100.0 - z;                       // prune_algo.py:61, a NumPy float64 from here on
    wide = true;
  }
  std::vector<std::vector<int>> bounds(n_layers);
  std::vector<uint8_t*> colkeep_dev;
  std::vector<std::vector<uint8_t>> colkeep_host;
  int rc = TS_OK;
  do {
    if (two_d) {
      // stage 1: global percentile over the column norms of all layers (prune_algo.py:64-67)
      long long totalN = 0;
      for (int l = 0; l < n_layers; ++l) totalN += L[l].N;
      float* cn = nullptr;
      uint8_t* ck = nullptr;
      if ((rc = arena.alloc(&cn, totalN)) != TS_OK) break;
      if ((rc = arena.alloc(&ck, totalN)) != TS_OK) break;
      long long o = 0;
      cudaError_t e = cudaSuccess;
      for (int l = 0; l < n_layers && e == cudaSuccess; ++l) {
        e = ts::col_norms_launch(L[l].score, L[l].ld, L[l].K, L[l].N, cn + o, s);
        o += L[l].N;
      }
      if (e != cudaSuccess) {
        rc = ts_internal_fail(TS_ERR_CUDA, "column norm kernel failed: %s", cudaGetErrorString(e));
        break;
      }
      const double q_col = mode == TS_MASK_TW_COLS_ROWS ? g1percent : q;
      if ((rc = percentile_to_device(cn, totalN, q_col, wide, false, sc, 0, s)) != TS_OK) break;
      e = ts::threshold_dev_launch(cn, totalN, sc.thr + 0, ck, s);
      std::vector<uint8_t> all(totalN);
      if (e == cudaSuccess) e = cudaMemcpyAsync(all.data(), ck, totalN, cudaMemcpyDeviceToHost, s);
      if (e == cudaSuccess && (rc = read_thresholds(sc, 0, &res->thr[0], s)) != TS_OK) break;
      if (e != cudaSuccess) {
        rc = ts_internal_fail(TS_ERR_CUDA, "column threshold failed: %s", cudaGetErrorString(e));
        break;
      }
      o = 0;
      colkeep_dev.resize(n_layers);
      colkeep_host.resize(n_layers);
      for (int l = 0; l < n_layers; ++l) {
        colkeep_dev[l] = ck + o;
        colkeep_host[l].assign(all.begin() + o, all.begin() + o + L[l].N);
        bounds[l] = regroup_bounds(colkeep_host[l].data(), L[l].N, G);
        o += L[l].N;
      }
    } else {
      for (int l = 0; l < n_layers; ++l) bounds[l] = fixed_bounds(L[l].N, G);
    }
    const int sel = mode == TS_MASK_BERT_PER_TILE ? 1 : (mode == TS_MASK_TOPK_L1 ? 2 : 0);
    if ((rc = row_stage(L, bounds, colkeep_dev, colkeep_host, sel, q, wide, res, &res->thr[1], arena, sc, s, f64)) != TS_OK) break;

    if (tew) {
      // element-wise residual (tw_mix_fn, prune_algo.py:151-177): rank |w| - mask over every
      // element of every layer, keep the top g1percent percent on top of the TW mask
      long long total = 0;
      for (int l = 0; l < n_layers; ++l) total += static_cast<long long>(L[l].K) * L[l].N;
      float* vals = nullptr;
      if ((rc = arena.alloc(&vals, total)) != TS_OK) break;
      long long o = 0;
      cudaError_t e = cudaSuccess;
      for (int l = 0; l < n_layers && e == cudaSuccess; ++l) {
        e = ts::tew_values_launch(L[l].score, L[l].ld, L[l].mask, L[l].ld_mask, L[l].K, L[l].N, vals + o, s);
        o += static_cast<long long>(L[l].K) * L[l].N;
      }
      if (e != cudaSuccess) {
        rc = ts_internal_fail(TS_ERR_CUDA, "residual value kernel failed: %s", cudaGetErrorString(e));
        break;
      }
      const double q2 = 100.0 - g1percent;
      const bool wide2 = sparsity_is_f64 != 0;
      if ((rc = percentile_to_device(vals, total, q2, wide2, false, sc, 2, s)) != TS_OK) break;
      o = 0;
      for (int l = 0; l < n_layers && e == cudaSuccess; ++l) {
        e = ts::tew_apply_launch(vals + o, sc.thr + 2, L[l].K, L[l].N, L[l].mask, L[l].ld_mask, L[l].residual, s);
        o += static_cast<long long>(L[l].K) * L[l].N;
      }
      if (e == cudaSuccess && (rc = read_thresholds(sc, 2, &res->thr[2], s)) != TS_OK) break;
      if (e != cudaSuccess) {
        rc = ts_internal_fail(TS_ERR_CUDA, "residual apply kernel failed: %s", cudaGetErrorString(e));
        break;
      }
    }
  } while (false);
  cudaStreamSynchronize(s);  // the arena is freed on return
  if (rc != TS_OK) {
    delete res;
    return rc;
  }
  *out = res;
  return TS_OK;
}
}  // namespace

extern "C" {

int ts_build_tw_mask(int mode, int n_layers, const void* const* scores_dev, const int* Ks, const int* Ns,
                     const int64_t* lds, int G, double sparsity, int sparsity_is_f64, double g1percent,
                     uint8_t* const* masks_dev, const int64_t* ld_masks, uint8_t* const* residual_dev,
                     ts_mask_result_t** out, void* stream) {
  return build_tw_mask_impl(mode, n_layers, scores_dev, Ks, Ns, lds, G, sparsity, sparsity_is_f64, g1percent,
                            masks_dev, ld_masks, residual_dev, out, stream, false);
}

int ts_build_tw_mask_f64(int mode, int n_layers, const void* const* scores_dev, const int* Ks, const int* Ns,
                         const int64_t* lds, int G, double sparsity, uint8_t* const* masks_dev,
                         const int64_t* ld_masks, ts_mask_result_t** out, void* stream) {
  if (mode != TS_MASK_TW1 && mode != TS_MASK_BERT_TW_K) {
    if (out) *out = nullptr;
    return ts_internal_fail(TS_ERR_UNSUPPORTED, "float64 scores: only TS_MASK_TW1 and TS_MASK_BERT_TW_K are offered");
  }
  return build_tw_mask_impl(mode, n_layers, scores_dev, Ks, Ns, lds, G, sparsity, 1, 0.0, masks_dev, ld_masks,
                            nullptr, out, stream, true);
}

int ts_taylor_accumulate(const float* grad_dev, const float* weight_dev, double* acc_dev, int64_t n, void* stream) {
  if (n < 0) return ts_internal_fail(TS_ERR_INVALID, "n=%lld is negative", static_cast<long long>(n));
  if (n == 0) return TS_OK;
  if (!grad_dev || !weight_dev || !acc_dev) return ts_internal_fail(TS_ERR_INVALID, "NULL argument");
  TSM_CUDA(ts::taylor_accumulate_launch(grad_dev, weight_dev, acc_dev, n, static_cast<cudaStream_t>(stream)));
  return TS_OK;
}

int ts_mask_result_layer(const ts_mask_result_t* r, int layer, int* n_tiles, int* total_kept_k,
                         int* total_kept_n) {
  if (!r || layer < 0 || layer >= static_cast<int>(r->layers.size())) {
    return ts_internal_fail(TS_ERR_INVALID, "bad mask result / layer index");
  }
  const ts_mask_result::Layer& R = r->layers[layer];
  if (n_tiles) *n_tiles = static_cast<int>(R.bounds.size()) - 1;
  if (total_kept_k) *total_kept_k = static_cast<int>(R.kept_k.size());
  if (total_kept_n) *total_kept_n = static_cast<int>(R.kept_n.size());
  return TS_OK;
}

int ts_mask_result_copy(const ts_mask_result_t* r, int layer, int32_t* tile_bounds, int32_t* tile_k_ptr,
                        int32_t* kept_k, int32_t* tile_n_ptr, int32_t* kept_n) {
  if (!r || layer < 0 || layer >= static_cast<int>(r->layers.size())) {
    return ts_internal_fail(TS_ERR_INVALID, "bad mask result / layer index");
  }
  const ts_mask_result::Layer& R = r->layers[layer];
  auto cp = [](int32_t* dst, const std::vector<int>& v) {
    if (dst && !v.empty()) memcpy(dst, v.data(), v.size() * sizeof(int));
  };
  cp(tile_bounds, R.bounds);
  cp(tile_k_ptr, R.tile_k_ptr);
  cp(kept_k, R.kept_k);
  cp(tile_n_ptr, R.tile_n_ptr);
  cp(kept_n, R.kept_n);
  return TS_OK;
}

int ts_mask_result_thresholds(const ts_mask_result_t* r, double* out3) {
  if (!r || !out3) return ts_internal_fail(TS_ERR_INVALID, "NULL argument");
  for (int i = 0; i < 3; ++i) out3[i] = r->thr[i];
  return TS_OK;
}

int ts_mask_result_destroy(ts_mask_result_t* r) {
  delete r;
  return TS_OK;
}

int ts_order_statistics(const float* vals_dev, int64_t n, int64_t rank_lo, int64_t rank_hi, float* out2,
                        void* stream) {
  if (!vals_dev || !out2) return ts_internal_fail(TS_ERR_INVALID, "NULL argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Arena arena;
  Scratch sc;
  TSM_OK(arena.alloc(&sc.hist, 256));
  TSM_OK(arena.alloc(&sc.count, 1));
  TSM_OK(arena.alloc(&sc.min_gt, 1));
  return order_statistics(vals_dev, n, rank_lo, rank_hi, &out2[0], &out2[1], sc.hist, sc.count, sc.min_gt, s);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the tw1 row stage
// ---------------------------------------------------------------------------------------------
}  // extern "C"

namespace {

// Everything ts_tw1_row_keep_noalloc needs beyond its inputs and outputs.  One copy per GPU that
// loads the library, held until the process exits.
struct NoAllocScratch {
  unsigned int hist[256];              // radix-select digit histogram (cleared before every pass)
  unsigned long long count_le;         // cleared before use
  unsigned int min_gt;                 // reset before use
  unsigned int pad_;
  int bounds[TS_NOALLOC_MAX_TILES + 1];
  float norms[TS_NOALLOC_MAX_NORMS];   // fully overwritten by every call before it is read
};

static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a kernel could
// use; the device address is looked up once per device, with that device current.
NoAllocScratch* g_noalloc_dev_ptr[64] = {};

int noalloc_scratch(NoAllocScratch** out) {
  int dev = 0;
  TSM_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ts_internal_fail(TS_ERR_UNSUPPORTED, "device index %d out of range", dev);
  if (!g_noalloc_dev_ptr[dev]) {
    void* p = nullptr;
    TSM_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    g_noalloc_dev_ptr[dev] = static_cast<NoAllocScratch*>(p);
  }
  *out = g_noalloc_dev_ptr[dev];
  return TS_OK;
}

}  // namespace

extern "C" {

int ts_tw1_row_keep_noalloc(const float* score_dev, int64_t ld, int K, int N, int G, double sparsity,
                            int sparsity_is_f64, uint8_t* keep_dev, double* threshold_out, void* stream) {
  if (!score_dev || !keep_dev) return ts_internal_fail(TS_ERR_INVALID, "NULL argument");
  if (K <= 0 || N <= 0 || G <= 0 || ld < N) return ts_internal_fail(TS_ERR_INVALID, "bad shape K=%d N=%d G=%d", K, N, G);
  if (!(sparsity >= 0.0 && sparsity <= 100.0)) {
    return ts_internal_fail(TS_ERR_INVALID, "sparsity=%g must be in [0, 100]", sparsity);
  }
  const long long n_tiles = (static_cast<long long>(N) + G - 1) / G;
  const long long total = n_tiles * K;
  if (n_tiles > TS_NOALLOC_MAX_TILES || total > TS_NOALLOC_MAX_NORMS) {
    return ts_internal_fail(TS_ERR_UNSUPPORTED,
                            "%lld tiles x %d rows = %lld tile-rows exceed the built-in scratch (%d tiles, %d "
                            "tile-rows); use ts_build_tw_mask, which allocates what it needs",
                            n_tiles, K, total, TS_NOALLOC_MAX_TILES, TS_NOALLOC_MAX_NORMS);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  NoAllocScratch* sc = nullptr;
  TSM_OK(noalloc_scratch(&sc));
  int bounds[TS_NOALLOC_MAX_TILES + 1];
  for (long long t = 0; t < n_tiles; ++t) bounds[t] = static_cast<int>(t * G);
  bounds[n_tiles] = N;
  TSM_CUDA(cudaMemcpyAsync(sc->bounds, bounds, (n_tiles + 1) * sizeof(int), cudaMemcpyHostToDevice, s));
  TSM_CUDA(cudaStreamSynchronize(s));  // `bounds` lives on this stack frame
  TSM_CUDA(ts::tile_row_norms_launch(score_dev, ld, K, sc->bounds, static_cast<int>(n_tiles), nullptr, sc->norms, 1,
                                     G == 128 ? N / 128 : 0, s));
  const Ranks r = percentile_ranks(total, sparsity, sparsity_is_f64 != 0);
  float a = 0, b = 0;
  // order_statistics clears the histogram before every digit pass and the two counters before use
  TSM_OK(order_statistics(sc->norms, total, r.pi, r.ni, &a, &b, sc->hist, &sc->count_le, &sc->min_gt, s));
  const double thr = percentile_lerp(a, b, r, sparsity_is_f64 != 0);
  TSM_CUDA(ts::threshold_launch(sc->norms, total, thr, keep_dev, s));
  TSM_CUDA(cudaStreamSynchronize(s));
  if (threshold_out) *threshold_out = thr;
  return TS_OK;
}

int ts_build_pattern_mask(int pattern, int n_layers, const void* const* scores_dev, const int* Ks, const int* Ns,
                          const int64_t* lds, double sparsity, uint8_t* const* masks_dev, const int64_t* ld_masks,
                          double* threshold_out, void* stream) {
  if (pattern != TS_PATTERN_EW && pattern != TS_PATTERN_VW && pattern != TS_PATTERN_BW) {
    return ts_internal_fail(TS_ERR_INVALID, "unknown pattern %d", pattern);
  }
  if (n_layers <= 0 || !scores_dev || !Ks || !Ns || !masks_dev) return ts_internal_fail(TS_ERR_INVALID, "NULL or empty argument");
  if (!(sparsity >= 0.0 && sparsity <= 100.0)) return ts_internal_fail(TS_ERR_INVALID, "sparsity=%g must be in [0, 100]", sparsity);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  long long total = 0;
  for (int l = 0; l < n_layers; ++l) {
    if (!scores_dev[l] || !masks_dev[l] || Ks[l] <= 0 || Ns[l] <= 0) return ts_internal_fail(TS_ERR_INVALID, "layer %d: bad argument", l);
    if (Ks[l] > 65535 * 16) {   // vector-wise: 16-row blocks of K are a grid y dimension
      return ts_internal_fail(TS_ERR_UNSUPPORTED, "layer %d: K=%d exceeds 1048560 rows", l, Ks[l]);
    }
    if ((lds && lds[l] < Ns[l]) || (ld_masks && ld_masks[l] < Ns[l])) return ts_internal_fail(TS_ERR_INVALID, "layer %d: leading dimension too small", l);
    total += static_cast<long long>(Ks[l]) * Ns[l];
  }
  if (threshold_out) *threshold_out = std::nan("");
  if (pattern == TS_PATTERN_VW) {
    // topk = int((1 - sparsity/100) * 16), in the double arithmetic of the Python expression
    volatile double frac = 1.0 - sparsity / 100.0;
    volatile double scaled = frac * 16.0;
    const int topk = static_cast<int>(scaled);
    for (int l = 0; l < n_layers; ++l) {
      TSM_CUDA(ts::vw_mask_launch(static_cast<const float*>(scores_dev[l]), lds ? lds[l] : Ns[l], Ks[l], Ns[l], topk,
                                  masks_dev[l], ld_masks ? ld_masks[l] : Ns[l], s));
    }
    TSM_CUDA(cudaStreamSynchronize(s));
    return TS_OK;
  }
  if (pattern == TS_PATTERN_BW) {
    // block-wise: one percentile over the Frobenius norms of the 32 x 32 blocks of all layers (a list
    // of float32 values and a Python-number q: float32 percentile arithmetic), blocks above it are kept
    Arena arena;
    Scratch sc;
    TSM_OK(alloc_scratch(arena, &sc));
    long long n_blocks = 0;
    std::vector<long long> boff(n_layers + 1, 0);
    for (int l = 0; l < n_layers; ++l) {
      n_blocks += static_cast<long long>((Ks[l] + 31) / 32) * ((Ns[l] + 31) / 32);
      boff[l + 1] = n_blocks;
    }
    float* norms = nullptr;
    uint8_t* keep = nullptr;
    TSM_OK(arena.alloc(&norms, static_cast<size_t>(n_blocks)));
    TSM_OK(arena.alloc(&keep, static_cast<size_t>(n_blocks)));
    for (int l = 0; l < n_layers; ++l) {
      TSM_CUDA(ts::block_norms_launch(static_cast<const float*>(scores_dev[l]), lds ? lds[l] : Ns[l], Ks[l], Ns[l],
                                      norms + boff[l], s));
    }
    TSM_OK(percentile_to_device(norms, n_blocks, sparsity, /*wide=*/false, /*f64_values=*/false, sc, 3, s));
    TSM_CUDA(ts::threshold_dev_launch(norms, n_blocks, sc.thr + 3, keep, s));
    for (int l = 0; l < n_layers; ++l) {
      TSM_CUDA(ts::block_mask_launch(keep + boff[l], Ks[l], Ns[l], masks_dev[l], ld_masks ? ld_masks[l] : Ns[l], s));
    }
    double thr = 0.0;
    TSM_OK(read_thresholds(sc, 3, &thr, s));
    if (threshold_out) *threshold_out = thr;
    return TS_OK;
  }
  // element-wise: one percentile over |score| of all layers.  The reference flattens through Python
  // lists, so the values are float64 copies of the float32 elements and every step of the
  // percentile, the difference of the two order statistics included, is a double operation.
  Arena arena;
  Scratch sc;
  TSM_OK(alloc_scratch(arena, &sc));
  float* vals = nullptr;
  TSM_OK(arena.alloc(&vals, static_cast<size_t>(total)));
  long long off = 0;
  for (int l = 0; l < n_layers; ++l) {
    TSM_CUDA(ts::abs_values_launch(static_cast<const float*>(scores_dev[l]), lds ? lds[l] : Ns[l], Ks[l], Ns[l],
                                   vals + off, s));
    off += static_cast<long long>(Ks[l]) * Ns[l];
  }
  TSM_OK(percentile_to_device(vals, total, sparsity, /*wide=*/true, /*f64_values=*/true, sc, 3, s));
  off = 0;
  for (int l = 0; l < n_layers; ++l) {
    const long long n_el = static_cast<long long>(Ks[l]) * Ns[l];
    const long long ldm = ld_masks ? ld_masks[l] : Ns[l];
    if (ldm == Ns[l]) {
      TSM_CUDA(ts::threshold_dev_launch(vals + off, n_el, sc.thr + 3, masks_dev[l], s));
    } else {
      for (int k = 0; k < Ks[l]; ++k) {
        TSM_CUDA(ts::threshold_dev_launch(vals + off + static_cast<long long>(k) * Ns[l], Ns[l], sc.thr + 3,
                                          masks_dev[l] + static_cast<long long>(k) * ldm, s));
      }
    }
    off += n_el;
  }
  double thr = 0.0;
  TSM_OK(read_thresholds(sc, 3, &thr, s));
  if (threshold_out) *threshold_out = thr;
  return TS_OK;
}

int ts_percentile_f32(const float* vals_dev, int64_t n, double q, int q_is_f64, double* out, void* stream) {
  if (!vals_dev || !out || n <= 0) return ts_internal_fail(TS_ERR_INVALID, "bad argument");
  if (!(q >= 0.0 && q <= 100.0)) return ts_internal_fail(TS_ERR_INVALID, "q=%g must be in [0, 100]", q);
  const Ranks r = percentile_ranks(n, q, q_is_f64 != 0);
  float ab[2];
  TSM_OK(ts_order_statistics(vals_dev, n, r.pi, r.ni, ab, stream));
  *out = percentile_lerp(ab[0], ab[1], r, q_is_f64 != 0);
  return TS_OK;
}

}  // extern "C"

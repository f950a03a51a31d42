// C ABI of libtilesparse: argument checking, device bookkeeping, scheduling and kernel launches.
// See include/tilesparse.h for the contract of every entry point.
#include "../../include/tilesparse.h"

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cmath>
#include <cstring>
#include <map>
#include <mutex>
#include <queue>
#include <string>
#include <tuple>
#include <vector>

#include "ts_kernels.h"

namespace {
thread_local std::string g_last_error;
}  // namespace

// Records the calling thread's error text and returns `code`; shared by every C-ABI source file.
int ts_internal_fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}
#define fail ts_internal_fail

namespace {

#define TS_CUDA(expr)                                                                    \
  do {                                                                                   \
    cudaError_t e_ = (expr);                                                             \
    if (e_ != cudaSuccess) {                                                             \
      return fail(e_ == cudaErrorMemoryAllocation ? TS_ERR_NOMEM : TS_ERR_CUDA,          \
                  "%s failed: %s", #expr, cudaGetErrorString(e_));                       \
    }                                                                                    \
  } while (0)

// cuTensorMapEncodeTiled is fetched through the runtime so the library links against cudart only.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

// Tensor map over a packed weight matrix [rows][ldw] of 16-bit elements, box 64 (K) x 128 (rows),
// 128-byte swizzle, zero fill outside the matrix.
int make_weight_tmap(CUtensorMap* map, int dtype, const void* base, long long rows, long long ldw) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (ldw * 2) % 16 != 0) {
    return fail(TS_ERR_INVALID, "packed weights need a 16-byte aligned base and row pitch");
  }
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(ldw), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldw) * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype == TS_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return TS_OK;
}

// Tensor map over the output Ct [n_rows][ldc] for the epilogue's TMA stores: box 64 batch columns x 128
// rows, 128-byte swizzle.
int make_out_tmap(CUtensorMap* map, int dtype, const void* Ct, long long n_rows, long long M, long long ldc) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(n_rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldc) * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype == TS_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  2, const_cast<void*>(Ct), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed (%d)", (int)r);
  return TS_OK;
}

// Tensor map over the fp32 scratch [rows][M] of a split-K schedule: box 32 floats x 128 rows, 128-byte
// swizzle (one staging group of the epilogue).
int make_scratch_tmap(CUtensorMap* map, const float* scratch, long long rows, long long M) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(M) * 4};
  cuuint32_t box[2] = {32, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(scratch), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TS_ERR_CUDA, "cuTensorMapEncodeTiled (scratch) failed (%d)", (int)r);
  return TS_OK;
}

struct Schedule {
  ts::WorkItem* d_units = nullptr;
  ts::BlockDesc* d_blocks = nullptr;
  int* d_meta = nullptr;       // one resolved record (ts::kBlockMetaInts ints) per descriptor of d_blocks
  int blk_stride = 0;
  int rounds = 0;
  int grid = 0;
  int n_units = 0;
  int unit_rows = 0;
  std::vector<float> cta_cost;
  // split-K: tiles whose kept rows are spread over several units per batch block, the fp32 scratch
  // their partial sums go to ([scratch_rows][scratch_ld]) and the descriptors for the second pass
  int n_split = 0;
  ts::SplitTile* d_split = nullptr;
  float* d_scratch = nullptr;
  long long scratch_ld = 0;
  CUtensorMap* d_scratch_map = nullptr;   // tensor map over d_scratch, in device memory
  bool all_dense = false;                 // every unit's tile keeps 128 consecutive columns (TMA tile stores only)
};

void free_schedule(Schedule& s) {
  cudaFree(s.d_units);
  cudaFree(s.d_blocks);
  cudaFree(s.d_meta);
  cudaFree(s.d_split);
  cudaFree(s.d_scratch);
  cudaFree(s.d_scratch_map);
  s.d_scratch_map = nullptr;
  s.d_units = nullptr;
  s.d_blocks = nullptr;
  s.d_meta = nullptr;
  s.d_split = nullptr;
  s.d_scratch = nullptr;
}

inline bool small_activations(long long at_rows, int M);   // defined with the scheduler below

// Split-K plan: parts[t] >= 1 units per batch block for tile t.  A unit's K blocks run one after the
// other on one SM, so a launch cannot be shorter than its longest tile's K_t / 64 blocks.  A tile whose
// share of the SMs (by its share of the K blocks) is at least twice its number of 256-row units has
// SMs to spare or gets cut into needlessly narrow units; its kept rows are then cut into up to four
// ranges of whole K blocks (at least 12 each), as many as keep one full-width unit per SM.  Each range
// runs as a unit of its own whose fp32 partial sums a second kernel adds up.  Short chains (< 32
// blocks) stay whole: the second pass costs a launch and a round trip of the partial sums.
// Measured on B200 (VGG16 conv5, batch 64): "10 % columns + 75 % rows" as the implicit convolution
// 66.8 -> 50.7 us with its 70-block tile cut in two; tw2 as a GEMM over the im2col matrix 41.6 -> 34.4 us
// (list schedule: 50 SMs were idle); tw2 as the implicit convolution (share 1.9 units per SM-share, the
// contiguous partition already fills the machine) 33.0 -> 37.2 us when cut, hence the exact "twice" there
// and a tolerance of a tenth where the list schedule works with whole 256-row units.
void plan_split(const std::vector<int>& k_counts, const std::vector<int>& n_counts, long long at_rows, int M,
                int n_ctas, std::vector<int>* parts) {
  const size_t nt = k_counts.size();
  parts->assign(nt, 1);
  if (M <= 0 || n_ctas <= 0) return;
  const double units = (M + 255) / 256;
  double blocks = 0.0;
  long long live = 0;
  for (size_t t = 0; t < nt; ++t) {
    if (n_counts[t] > 0) {
      blocks += (k_counts[t] + 63) / 64;
      ++live;
    }
  }
  if (blocks <= 0.0) return;
  // the regime build_schedule will choose: batch rows cut freely (contiguous partition) or whole units
  const bool contiguous = small_activations(at_rows, M) && live * static_cast<long long>(units) <= 3LL * n_ctas;
  const double slack = contiguous ? 1e-9 : 0.1;
  for (size_t t = 0; t < nt; ++t) {
    const int kb = (k_counts[t] + 63) / 64;
    if (n_counts[t] <= 0 || kb < 32) continue;
    const double sms = n_ctas * (kb / blocks);                // the tile's share of the machine
    const int fit = static_cast<int>(std::floor(sms / units + slack));
    (*parts)[t] = std::max(1, std::min({4, fit, kb / 12}));
  }
}

// Cost of one work unit of `granules` 64-row batch granules over a tile with k_count kept rows, in
// units of 8 KiB moved between L2 and the SM: per 64-row K block 16 KiB of packed weights and 8 KiB of
// gathered activations per granule; per granule 16 KiB of output; and a constant for the hand-over
// between consecutive units of a CTA (accumulator swap, pipeline refill).
inline float unit_cost(int k_count, int granules) {
  const int kb = (k_count + 63) / 64;
  return static_cast<float>(kb * (2 + granules) + 2 * granules + 3);
}

struct Unit {
  int tile, m_begin, m_len;
  float cost;
};

// The balanced contiguous partition is used when there are few work units per SM (at most three
// 256-row units each) and the activations fit comfortably in L2 (K*M*2 bytes <= 64 MiB); otherwise the
// list schedule further down.  Measured on B200: the contiguous partition wins where the list
// schedule leaves SMs idle or a partial last wave (768-column BERT layers: 6.2 vs 6.7 us and 11.4 vs
// 11.8 us), and loses where there is plenty of work (a 4096-square layer with skewed tiles: 54 vs
// 40 us), because it has every tile in flight at once at a different batch position, while the
// tile-major list order keeps the CTAs on a few tiles whose kept rows and weights stay hot in L2.
inline bool small_activations(long long at_rows, int M) { return 2LL * at_rows * M <= (64LL << 20); }

// Balanced contiguous partition.  The 64-row batch granules of all tiles, tile after tile in `order`,
// form one line; every CTA receives one contiguous piece of it, cut into units of at most `cap`
// granules that do not cross a tile boundary.  Three candidates: (a) the pieces whose largest cost is
// minimal (binary search on the bound, greedy filling for a given bound); (b) pieces of equal weight
// (kept K blocks + output per granule), which always spreads the line over all n_ctas SMs; (c) when
// there are no more tiles than SMs, every tile split evenly among a number of CTAs of its own, the
// CTAs handed out one by one to the tile with the costliest piece, so that no CTA changes tile and
// re-fetches packed weights.  (c) is taken when its largest piece is no costlier than the others'
// (within 3 %), else (b) under the same rule, else (a).  All of them fill the machine when there are
// fewer 256-row units than SMs (a 768-column layer has 6 tiles x 16 such units for 148 SMs) and leave
// no partial last wave.  A CTA's units are consecutive runs of one tile.
void partition_contiguous(const std::vector<ts::TileDesc>& tiles, const std::vector<int>& order, int M, int cap,
                          int n_ctas, std::vector<std::vector<Unit>>* lists) {
  const int granules = (M + 63) / 64;
  const long long line = static_cast<long long>(order.size()) * granules;
  // pieces given by their exclusive end positions on the line -> unit lists and the largest cost
  auto cut = [&](const std::vector<long long>& ends, std::vector<std::vector<Unit>>* out) -> double {
    double worst = 0.0;
    if (out) out->clear();
    long long pos = 0;
    for (long long end : ends) {
      if (end <= pos) continue;
      if (out) out->push_back({});
      double load = 0.0;
      while (pos < end) {
        const int t = order[pos / granules];
        const int g0 = static_cast<int>(pos % granules);
        const int len = static_cast<int>(std::min<long long>({cap, granules - g0, end - pos}));
        const Unit u{t, g0 * 64, len * 64, unit_cost(tiles[t].k_count, len)};
        if (out) out->back().push_back(u);
        load += u.cost;
        pos += len;
      }
      worst = std::max(worst, load);
    }
    return worst;
  };
  // (a) greedy filling under a bound; returns false when it needs more than n_ctas pieces
  auto fill = [&](double bound, std::vector<long long>* ends) -> bool {
    if (ends) ends->clear();
    int used = 1;
    double load = 0.0;
    int open_tile = -1, open_len = 0;
    long long pos = 0;
    for (int t : order) {
      const int kc = tiles[t].k_count;
      const double first = unit_cost(kc, 1), more = unit_cost(kc, 2) - unit_cost(kc, 1);
      for (int g = 0; g < granules; ++g, ++pos) {
        const bool extend = open_tile == t && open_len < cap;
        double delta = extend ? more : first;
        if (load > 0.0 && load + delta > bound) {
          if (++used > n_ctas) return false;
          if (ends) ends->push_back(pos);
          load = 0.0;
          delta = first;
          open_len = 0;
        } else if (!extend) {
          open_len = 0;
        }
        open_tile = t;
        ++open_len;
        load += delta;
      }
    }
    if (ends) ends->push_back(line);
    return true;
  };
  double lo = 0.0, hi = 0.0, weight = 0.0;
  for (int t : order) {
    lo = std::max<double>(lo, unit_cost(tiles[t].k_count, 1));
    hi += static_cast<double>(unit_cost(tiles[t].k_count, 1)) * granules;
    weight += static_cast<double>((tiles[t].k_count + 63) / 64 + 2) * granules;
  }
  lo = std::max(lo, hi / std::max(1, n_ctas) * 0.25);
  for (int it = 0; it < 40 && hi - lo > 0.25; ++it) {
    const double mid = 0.5 * (lo + hi);
    if (fill(mid, nullptr)) hi = mid;
    else lo = mid;
  }
  std::vector<long long> ends_a, ends_b;
  fill(hi, &ends_a);
  // (b) equal weight: granule i belongs to the piece its weight midpoint falls into
  {
    const double share = weight / n_ctas;
    double cum = 0.0;
    int piece = 0;
    long long pos = 0;
    for (int t : order) {
      const double wt = static_cast<double>((tiles[t].k_count + 63) / 64 + 2);
      for (int g = 0; g < granules; ++g, ++pos) {
        const int want = std::min<int>(n_ctas - 1, static_cast<int>((cum + 0.5 * wt) / share));
        while (piece < want) {
          ends_b.push_back(pos);
          ++piece;
        }
        cum += wt;
      }
    }
    ends_b.push_back(line);
  }
  // (c) per-tile split
  std::vector<long long> ends_c;
  const int nt = static_cast<int>(order.size());
  if (nt <= n_ctas) {
    auto piece_cost = [&](int t, int pieces) {   // cost of the largest of `pieces` even parts of tile t
      const int len = (granules + pieces - 1) / pieces;
      double c = 0.0;
      for (int g = 0; g < len; g += cap) c += unit_cost(tiles[t].k_count, std::min(cap, len - g));
      return c;
    };
    std::vector<int> parts(nt, 1);
    typedef std::pair<double, int> Top;   // (cost of the tile's largest piece, position in order)
    std::priority_queue<Top> heap;
    for (int i = 0; i < nt; ++i) heap.push({piece_cost(order[i], 1), i});
    int spare = n_ctas - nt;
    while (spare > 0 && !heap.empty()) {
      const int i = heap.top().second;
      heap.pop();
      if (parts[i] >= granules) continue;   // one granule per CTA already; the tile leaves the heap
      ++parts[i];
      --spare;
      heap.push({piece_cost(order[i], parts[i]), i});
    }
    for (int i = 0; i < nt; ++i) {
      for (int p = 1; p <= parts[i]; ++p) {
        ends_c.push_back(static_cast<long long>(i) * granules + static_cast<long long>(granules) * p / parts[i]);
      }
    }
  }
  const double worst_a = cut(ends_a, nullptr), worst_b = cut(ends_b, nullptr);
  const double worst_c = ends_c.empty() ? 1e300 : cut(ends_c, nullptr);
  const std::vector<long long>* pick = &ends_a;
  if (worst_c <= std::min(worst_a, worst_b) * 1.03) pick = &ends_c;
  else if (worst_b <= worst_a * 1.03) pick = &ends_b;
  cut(*pick, lists);
  if (lists->empty()) lists->assign(1, {});
}

// Blocked list schedule for activations far larger than L2.  Tiles are taken in descending kept-K
// order and cut into units of `cap` granules (the last unit of a tile may be narrower).  Every
// tile's pass over At would come from HBM, so the tiles are taken in groups whose packed weights fit
// comfortably in L2 (32 MiB) and, inside a group, the batch blocks become the outer loop: concurrent
// CTAs then share one slab of At, whose rows are fetched from HBM once per group instead of once per
// tile.  Units go to the CTAs by longest-processing-time list scheduling in that order.
void partition_blocked(const std::vector<ts::TileDesc>& tiles, const std::vector<int>& order, long long at_rows,
                       int M, int cap, int n_ctas, std::vector<std::vector<Unit>>* lists) {
  const int granules = (M + 63) / 64;
  const int full_per_tile = granules / cap;
  const int tail_gran = granules - full_per_tile * cap;
  const bool blocked = 2LL * at_rows * M > (192LL << 20);
  long long wbytes = 0;
  for (int t : order) wbytes += 2LL * tiles[t].k_count * 128;
  const long long avg_tile = std::max<long long>(1, wbytes / std::max<size_t>(1, order.size()));
  const int group = blocked ? static_cast<int>(std::max<long long>(8, std::min<long long>(order.size(), (32LL << 20) / avg_tile)))
                            : 1;
  std::vector<Unit> units;
  const int blocks_per_tile = full_per_tile + (tail_gran > 0 ? 1 : 0);
  for (size_t g0 = 0; g0 < order.size(); g0 += group) {
    const size_t g1 = std::min(order.size(), g0 + group);
    for (int u = 0; u < blocks_per_tile; ++u) {
      for (size_t i = g0; i < g1; ++i) {
        const int t = order[i];
        const int len = u < full_per_tile ? cap : tail_gran;
        units.push_back(Unit{t, u * cap * 64, len * 64, unit_cost(tiles[t].k_count, len)});
      }
    }
  }
  const int g = std::max<int>(1, std::min<int>(n_ctas, static_cast<int>(units.size())));
  lists->assign(g, {});
  typedef std::pair<float, int> Load;  // (load, cta), smallest load first, then lowest cta
  std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
  for (int b = 0; b < g; ++b) heap.push({0.0f, b});
  for (const Unit& u : units) {
    Load l = heap.top();
    heap.pop();
    (*lists)[l.second].push_back(u);
    l.first += u.cost;
    heap.push(l);
  }
}

// Work distribution for the persistent kernel.  Units are (tile, run of batch rows); a run is a
// multiple of 64 rows, at most *unit_rows (128 or 256: the kernel variant).  forced_unit_rows (0, 128,
// 256) pins the variant; otherwise 256-row units are used unless no CTA would receive more than 128
// batch rows of work.
// Output: flat [rounds][grid] table; a CTA's units fill its column from round 0 without gaps,
// tile = -1 marks the end.
// part_kb0 (optional, one entry per tile): >= 0 marks a split-K part that starts at that K block of its
// tile (the TileDesc then describes the part: its slice of the kept-row list, its scratch rows as
// c_row0, no column list).
void build_schedule(const std::vector<ts::TileDesc>& tiles, long long at_rows, int M, int forced_unit_rows,
                    int n_ctas, std::vector<ts::WorkItem>* flat, int* rounds, int* grid, int* n_units,
                    int* unit_rows, std::vector<float>* cta_cost, std::vector<ts::BlockDesc>* blocks,
                    int* blk_stride, const std::vector<int>* part_kb0 = nullptr) {
  std::vector<int> order;
  for (int t = 0; t < static_cast<int>(tiles.size()); ++t) {
    if (tiles[t].n_count > 0) order.push_back(t);
  }
  std::stable_sort(order.begin(), order.end(),
                   [&](int a, int b) { return tiles[a].k_count > tiles[b].k_count; });
  const long long granules = (M + 63) / 64;
  const long long total = granules * static_cast<long long>(order.size());
  const long long units256_all = static_cast<long long>(order.size()) * ((M + 255) / 256);
  const bool contiguous = small_activations(at_rows, M) && units256_all <= 3LL * n_ctas;
  int cap;
  if (forced_unit_rows == 128 || forced_unit_rows == 256) {
    cap = forced_unit_rows / 64;
  } else if (contiguous) {
    cap = (total + n_ctas - 1) / std::max(1, n_ctas) <= 2 ? 2 : 4;
  } else {
    cap = 2 * units256_all >= n_ctas ? 4 : 2;
  }
  *unit_rows = cap * 64;
  std::vector<std::vector<Unit>> ulists;
  if (order.empty() || M <= 0) {
    ulists.assign(1, {});
  } else if (contiguous) {
    partition_contiguous(tiles, order, M, cap, n_ctas, &ulists);
  } else {
    partition_blocked(tiles, order, at_rows, M, cap, n_ctas, &ulists);
  }
  const int g = std::max<int>(1, static_cast<int>(ulists.size()));
  std::vector<std::vector<ts::WorkItem>> lists(g);
  cta_cost->assign(g, 0.0f);
  *n_units = 0;
  for (int b = 0; b < static_cast<int>(ulists.size()); ++b) {
    for (const Unit& u : ulists[b]) {
      const ts::TileDesc& td = tiles[u.tile];
      ts::WorkItem w;
      w.k_list = td.k_list;
      w.n_list = td.n_list;
      w.k_count = td.k_count;
      w.n_count = td.n_count;
      w.w_row0 = td.w_row0;
      w.c_row0 = td.c_row0;
      w.flags = (td.relative ? ts::kItemRelative : 0) | (td.pad_ ? ts::kItemDenseRows : 0);
      const int kb0 = part_kb0 ? (*part_kb0)[u.tile] : -1;
      if (kb0 >= 0) w.flags |= ts::kItemScratch | (kb0 << ts::kItemKb0Shift);
      w.m_begin = u.m_begin;
      w.m_len = u.m_len;
      w.tile = u.tile;
      lists[b].push_back(w);
      (*cta_cost)[b] += u.cost;
      ++*n_units;
    }
  }
  int r = 0;
  for (const auto& l : lists) r = std::max<int>(r, static_cast<int>(l.size()));
  ts::WorkItem none;
  memset(&none, 0, sizeof(none));
  none.tile = -1;
  flat->assign(static_cast<size_t>(r) * g, none);
  for (int b = 0; b < g; ++b) {
    for (size_t i = 0; i < lists[b].size(); ++i) (*flat)[i * g + b] = lists[b][i];
  }
  *rounds = r;
  *grid = g;

  // The same lists at K-block granularity for the gather warps.  The stream of every CTA ends with
  // end markers; 24 of them cover the deepest look-ahead (a gather warp requests the record of the
  // block up to 16 positions past the one it is copying) with room to spare.
  size_t max_blocks = 0;
  for (const auto& l : lists) {
    size_t nb = 0;
    for (const ts::WorkItem& w : l) nb += (w.k_count + 63) / 64;
    max_blocks = std::max(max_blocks, nb);
  }
  *blk_stride = static_cast<int>(max_blocks) + 24;
  ts::BlockDesc end;
  end.idx = nullptr;
  end.m0 = 0;
  end.meta = ts::kBlockEnd;
  blocks->assign(static_cast<size_t>(g) * *blk_stride, end);
  for (int b = 0; b < g; ++b) {
    size_t o = static_cast<size_t>(b) * *blk_stride;
    for (const ts::WorkItem& w : lists[b]) {
      for (int pos = 0; pos < w.k_count; pos += 64) {
        ts::BlockDesc d;
        d.idx = w.k_list + pos;
        d.m0 = w.m_begin;
        // position of the block's first row inside the tile's list (a split-K part starts further in)
        const int first = pos + ((w.flags & ts::kItemScratch) ? (w.flags >> ts::kItemKb0Shift) * 64 : 0);
        d.meta = static_cast<uint32_t>(std::min(64, w.k_count - pos)) | ((w.flags & ts::kItemRelative) ? 0x80u : 0u) |
                 (static_cast<uint32_t>(w.m_len / 64 - 1) << 8) | (static_cast<uint32_t>(first) << 10);
        (*blocks)[o++] = d;
      }
    }
  }
}

int current_sm_count(int* out) {
  int dev = 0;
  TS_CUDA(cudaGetDevice(&dev));
  TS_CUDA(cudaDeviceGetAttribute(out, cudaDevAttrMultiProcessorCount, dev));
  return TS_OK;
}

}  // namespace

struct ts_layer {
  int K = 0, N = 0, G = 0, dtype = 0;
  int device = 0;
  int sm_count = 0;
  int n_tiles = 0;
  std::vector<int> tile_k_ptr, kept_k, tile_n_ptr, kept_n;  // absolute indices
  std::vector<int> k_counts, n_counts;
  int max_k = 0;
  int* d_kept_k = nullptr;
  int* d_kept_n = nullptr;
  ts::TileDesc* d_tiles = nullptr;
  std::vector<ts::TileDesc> h_tiles;
  uint16_t* d_wp = nullptr;
  long long wp_rows = 0, ldw = 0;
  bool packed = false;
  CUtensorMap tmap;
  int* d_status = nullptr;
  // keyed by (batch size, activation row pitch, 1 for the convolution row map)
  // ... and 1 when split-K units are allowed (never for calls that also write peers)
  std::map<std::tuple<int, long long, int, int>, Schedule> schedules;
  bool split_k = true;         // ts_layer_set_split_k
  int conv_cin = 0, conv_kh = 0, conv_kw = 0;   // set by ts_layer_set_conv: K = kh * kw * cin
  void* d_at = nullptr;
  size_t at_bytes = 0;
  void* d_ct = nullptr;
  size_t ct_bytes = 0;
  // Host-buffer path: copy-in, compute and copy-out streams and the events that chain them.
  cudaStream_t s_in = nullptr, s_mm = nullptr, s_out = nullptr;
  std::vector<cudaEvent_t> events;
  // The host-buffer path zeroes its staging output once and then relies on the kernel overwriting the
  // same places every call; that holds only while the batch size (the row pitch) and the tile set stay
  // the same and no beta pass has brought the caller's values in.
  bool ct_dirty = true;
  int ct_zeroed_m = -1;
  int forced_unit_rows = 0;    // 0: the scheduler chooses between 128- and 256-row units
  bool wp_fresh = false;       // packed weights were (re)written on a stream since the last GEMM launch
  bool host_pending = false;   // events[1] marks the end of the latest host-buffer call
  // Tensor maps over the peers' output buffers of a tile-sharded layer (device copy, and the host
  // copy it was uploaded from with the arguments it was encoded for).
  CUtensorMap* d_peer_maps = nullptr;
  CUtensorMap h_peer_maps[7];
  void* peer_map_ptrs[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  long long peer_map_m = -1, peer_map_ldc = -1;
  int peer_map_count = 0;
};

namespace {

void free_tiles(ts_layer* l) {
  cudaFree(l->d_kept_k);
  cudaFree(l->d_kept_n);
  cudaFree(l->d_tiles);
  cudaFree(l->d_wp);
  l->d_kept_k = l->d_kept_n = nullptr;
  l->d_tiles = nullptr;
  l->d_wp = nullptr;
  for (auto& kv : l->schedules) free_schedule(kv.second);
  l->schedules.clear();
  l->packed = false;
  l->ct_dirty = true;   // another tile set leaves other places of the staging output unwritten
}

// Schedule for batch size M over activations whose kept rows are `ld` elements apart (a matrix), or
// over a convolution's input planes of pitch `ld` with padded image width conv_wp (conv_wp > 0).
int get_schedule(ts_layer* l, int M, long long ld, int conv_wp, bool allow_split, Schedule** out) {
  const auto key = std::make_tuple(M, ld, conv_wp, allow_split ? 1 : 0);
  auto it = l->schedules.find(key);
  if (it != l->schedules.end()) {
    *out = &it->second;
    return TS_OK;
  }
  if (l->schedules.size() >= 16) {  // bounded cache: drop everything, rebuild on demand
    TS_CUDA(cudaDeviceSynchronize());
    for (auto& kv : l->schedules) free_schedule(kv.second);
    l->schedules.clear();
  }
  Schedule s;
  // frees what has been allocated so far if a step below fails
  struct Guard {
    Schedule* s;
    bool armed;
    ~Guard() {
      if (armed) free_schedule(*s);
    }
  } guard{&s, true};
  std::vector<ts::WorkItem> flat;
  std::vector<ts::BlockDesc> blocks;
  ts::RowMap map;
  memset(&map, 0, sizeof(map));
  map.ld8 = ld / 8;
  long long at_rows = l->K;
  if (conv_wp > 0) {
    map.conv_cin = l->conv_cin;
    map.conv_kw = l->conv_kw;
    map.conv_wp8 = conv_wp / 8;
    at_rows = static_cast<long long>(l->conv_kw) * l->conv_cin;   // the planes that exist in memory
  }
  if (at_rows * (ld / 8) + static_cast<long long>(l->conv_kh) * (conv_wp / 8) >= (1LL << 31)) {
    return fail(TS_ERR_UNSUPPORTED, "activations of %lld rows x %lld elements exceed the 32 GiB the block records address",
                at_rows, ld);
  }
  // Split-K: tiles with a long chain of K blocks become several "tiles" of the schedule, one per range
  // of K blocks, each writing to scratch rows of its own.
  std::vector<int> parts;
  if (allow_split) plan_split(l->k_counts, l->n_counts, at_rows, M, l->sm_count, &parts);
  bool any_split = false;
  for (int p : parts) any_split = any_split || p > 1;
  if (any_split) {
    std::vector<ts::TileDesc> vt;
    std::vector<int> kb0;
    std::vector<ts::SplitTile> st;
    int scratch_rows = 0;
    for (size_t t = 0; t < l->h_tiles.size(); ++t) {
      const ts::TileDesc& td = l->h_tiles[t];
      if (parts[t] <= 1) {
        vt.push_back(td);
        kb0.push_back(-1);
        continue;
      }
      ts::SplitTile sp;
      sp.n_list = td.n_list;
      sp.n_count = td.n_count;
      sp.c_row0 = td.c_row0;
      sp.relative = td.relative;
      sp.parts = parts[t];
      sp.scratch_row0 = scratch_rows;
      sp.pad_ = 0;
      st.push_back(sp);
      const int kb = (td.k_count + 63) / 64;
      for (int p = 0; p < parts[t]; ++p) {
        const int b0 = static_cast<int>(static_cast<long long>(kb) * p / parts[t]);
        const int b1 = static_cast<int>(static_cast<long long>(kb) * (p + 1) / parts[t]);
        ts::TileDesc part = td;
        part.k_list = td.k_list + static_cast<size_t>(b0) * 64;
        part.k_count = std::min(td.k_count, b1 * 64) - b0 * 64;
        part.n_list = nullptr;
        part.c_row0 = scratch_rows;
        part.pad_ = 0;          // scratch rows are written from the registers, never by a TMA store
        vt.push_back(part);
        kb0.push_back(b0);
        scratch_rows += 128;
      }
    }
    build_schedule(vt, at_rows, M, l->forced_unit_rows, l->sm_count, &flat, &s.rounds, &s.grid, &s.n_units,
                   &s.unit_rows, &s.cta_cost, &blocks, &s.blk_stride, &kb0);
    s.n_split = static_cast<int>(st.size());
    s.scratch_ld = M;
    TS_CUDA(cudaMalloc(&s.d_split, st.size() * sizeof(ts::SplitTile)));
    TS_CUDA(cudaMemcpy(s.d_split, st.data(), st.size() * sizeof(ts::SplitTile), cudaMemcpyHostToDevice));
    TS_CUDA(cudaMalloc(&s.d_scratch, static_cast<size_t>(scratch_rows) * M * sizeof(float)));
    CUtensorMap smap;
    int mrc = make_scratch_tmap(&smap, s.d_scratch, scratch_rows, M);
    if (mrc != TS_OK) return mrc;
    TS_CUDA(cudaMalloc(&s.d_scratch_map, sizeof(CUtensorMap)));
    TS_CUDA(cudaMemcpy(s.d_scratch_map, &smap, sizeof(CUtensorMap), cudaMemcpyHostToDevice));
  } else {
    build_schedule(l->h_tiles, at_rows, M, l->forced_unit_rows, l->sm_count, &flat, &s.rounds, &s.grid, &s.n_units,
                   &s.unit_rows, &s.cta_cost, &blocks, &s.blk_stride);
  }
  s.all_dense = s.n_split == 0;
  for (const ts::WorkItem& w : flat) {
    if (w.tile >= 0 && !(w.flags & ts::kItemDenseRows)) s.all_dense = false;
  }
  if (!flat.empty()) {
    TS_CUDA(cudaMalloc(&s.d_units, flat.size() * sizeof(ts::WorkItem)));
    TS_CUDA(cudaMemcpy(s.d_units, flat.data(), flat.size() * sizeof(ts::WorkItem),
                       cudaMemcpyHostToDevice));
    TS_CUDA(cudaMalloc(&s.d_blocks, blocks.size() * sizeof(ts::BlockDesc)));
    TS_CUDA(cudaMemcpy(s.d_blocks, blocks.data(), blocks.size() * sizeof(ts::BlockDesc),
                       cudaMemcpyHostToDevice));
    TS_CUDA(cudaMalloc(&s.d_meta, blocks.size() * ts::kBlockMetaInts * sizeof(int)));
    TS_CUDA(ts::expand_block_meta_launch(s.d_blocks, static_cast<long long>(blocks.size()), s.d_meta, map, nullptr));
    TS_CUDA(cudaStreamSynchronize(nullptr));
  }
  guard.armed = false;
  auto ins = l->schedules.emplace(key, s);
  *out = &ins.first->second;
  return TS_OK;
}

int check_gemm_args(const ts_layer* l, int M, const void* At, int64_t lda, const void* Ct,
                    int64_t ldc) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  if (!l->packed) return fail(TS_ERR_INVALID, "layer has no packed weights (call ts_layer_pack_weights)");
  if (M < 0 || (M % 8) != 0) return fail(TS_ERR_INVALID, "M=%d must be a non-negative multiple of 8", M);
  if (M == 0) return TS_OK;
  if (!At || !Ct) return fail(TS_ERR_INVALID, "At/Ct is NULL");
  if (lda < M || ldc < M || (lda % 8) != 0 || (ldc % 8) != 0) {
    return fail(TS_ERR_INVALID, "lda=%lld / ldc=%lld must be multiples of 8 and >= M=%d",
                (long long)lda, (long long)ldc, M);
  }
  if ((reinterpret_cast<uintptr_t>(At) & 15u) || (reinterpret_cast<uintptr_t>(Ct) & 15u)) {
    return fail(TS_ERR_INVALID, "At and Ct must be 16-byte aligned");
  }
  return TS_OK;
}

}  // namespace

extern "C" {

int ts_version(void) { return 100; }

int ts_last_error(char* buf, int n) {
  if (!buf || n <= 0) return 0;
  const int len = std::min<int>(n - 1, static_cast<int>(g_last_error.size()));
  memcpy(buf, g_last_error.data(), len);
  buf[len] = 0;
  return len;
}

int ts_layer_create(ts_layer_t** out, int K, int N, int G, int dtype) {
  if (!out) return fail(TS_ERR_INVALID, "out is NULL");
  *out = nullptr;
  if (K <= 0 || N <= 0) return fail(TS_ERR_INVALID, "K=%d and N=%d must be positive", K, N);
  if (G <= 0 || G > 128) return fail(TS_ERR_INVALID, "G=%d must be in [1, 128]", G);
  if (dtype != TS_DTYPE_F16 && dtype != TS_DTYPE_BF16) {
    return fail(TS_ERR_INVALID, "dtype must be TS_DTYPE_F16 or TS_DTYPE_BF16");
  }
  int dev = 0, sms = 0, major = 0;
  TS_CUDA(cudaGetDevice(&dev));
  TS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  TS_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) {
    return fail(TS_ERR_UNSUPPORTED, "device %d has compute capability %d.x; this library is sm_100a only",
                dev, major);
  }
  ts_layer* l = new ts_layer();
  l->K = K;
  l->N = N;
  l->G = G;
  l->dtype = dtype;
  l->device = dev;
  l->sm_count = sms;
  cudaError_t e = cudaMalloc(&l->d_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(l->d_status, 0, sizeof(int));
  if (e != cudaSuccess) {
    delete l;
    return fail(TS_ERR_CUDA, "status word allocation failed: %s", cudaGetErrorString(e));
  }
  *out = l;
  return TS_OK;
}

int ts_layer_destroy(ts_layer_t* l) {
  if (!l) return TS_OK;
  cudaDeviceSynchronize();
  free_tiles(l);
  cudaFree(l->d_status);
  cudaFree(l->d_peer_maps);
  cudaFree(l->d_at);
  cudaFree(l->d_ct);
  for (cudaEvent_t e : l->events) cudaEventDestroy(e);
  if (l->s_in) cudaStreamDestroy(l->s_in);
  if (l->s_mm) cudaStreamDestroy(l->s_mm);
  if (l->s_out) cudaStreamDestroy(l->s_out);
  delete l;
  return TS_OK;
}

int ts_layer_set_tiles(ts_layer_t* l, int n_tiles, const int32_t* tile_k_ptr,
                       const int32_t* kept_k_idx, const int32_t* tile_n_ptr,
                       const int32_t* kept_n_idx, int index_format) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  if (n_tiles < 0) return fail(TS_ERR_INVALID, "n_tiles=%d is negative", n_tiles);
  if (n_tiles > 0 && (!tile_k_ptr || !tile_n_ptr)) return fail(TS_ERR_INVALID, "tile pointers are NULL");
  if (index_format != TS_INDEX_ABSOLUTE && index_format != TS_INDEX_RELATIVE) {
    return fail(TS_ERR_INVALID, "unknown index_format %d", index_format);
  }
  std::vector<int> kp(n_tiles + 1, 0), np(n_tiles + 1, 0), kk, nn, kc(n_tiles), nc(n_tiles);
  if (n_tiles > 0) {
    if (tile_k_ptr[0] != 0 || tile_n_ptr[0] != 0) return fail(TS_ERR_INVALID, "tile pointers must start at 0");
    for (int t = 0; t < n_tiles; ++t) {
      if (tile_k_ptr[t + 1] < tile_k_ptr[t] || tile_n_ptr[t + 1] < tile_n_ptr[t]) {
        return fail(TS_ERR_INVALID, "tile pointers must be non-decreasing (tile %d)", t);
      }
    }
    const int tk = tile_k_ptr[n_tiles], tn = tile_n_ptr[n_tiles];
    if ((tk > 0 && !kept_k_idx) || (tn > 0 && !kept_n_idx)) return fail(TS_ERR_INVALID, "index lists are NULL");
    kk.resize(tk);
    nn.resize(tn);
    for (int t = 0; t < n_tiles; ++t) {
      kp[t + 1] = tile_k_ptr[t + 1];
      np[t + 1] = tile_n_ptr[t + 1];
      kc[t] = kp[t + 1] - tile_k_ptr[t];
      nc[t] = np[t + 1] - tile_n_ptr[t];
      if (nc[t] > l->G) return fail(TS_ERR_INVALID, "tile %d keeps %d columns, more than G=%d", t, nc[t], l->G);
      int prev = -1;
      for (int i = 0; i < kc[t]; ++i) {
        const int p = tile_k_ptr[t] + i;
        const int v = kept_k_idx[p] + (index_format == TS_INDEX_RELATIVE ? i : 0);
        if (v < 0 || v >= l->K) return fail(TS_ERR_INVALID, "tile %d: kept row %d out of [0,%d)", t, v, l->K);
        if (v <= prev) return fail(TS_ERR_INVALID, "tile %d: kept rows must be strictly ascending", t);
        prev = v;
        kk[p] = v;
      }
      for (int j = 0; j < nc[t]; ++j) {
        const int p = tile_n_ptr[t] + j;
        const int v = kept_n_idx[p] + (index_format == TS_INDEX_RELATIVE ? j : 0);
        if (v < 0 || v >= l->N) return fail(TS_ERR_INVALID, "tile %d: kept column %d out of [0,%d)", t, v, l->N);
        nn[p] = v;
      }
    }
  }
  TS_CUDA(cudaSetDevice(l->device));
  TS_CUDA(cudaDeviceSynchronize());
  free_tiles(l);
  l->n_tiles = n_tiles;
  l->tile_k_ptr = kp;
  l->tile_n_ptr = np;
  l->kept_k = kk;
  l->kept_n = nn;
  l->k_counts = kc;
  l->n_counts = nc;
  l->max_k = 0;
  for (int v : kc) l->max_k = std::max(l->max_k, v);
  l->ldw = std::max<long long>(64, (l->max_k + 63) / 64 * 64);
  l->wp_rows = static_cast<long long>(std::max(1, n_tiles)) * 128;
  TS_CUDA(cudaMalloc(&l->d_kept_k, std::max<size_t>(1, kk.size()) * sizeof(int)));
  TS_CUDA(cudaMalloc(&l->d_kept_n, std::max<size_t>(1, nn.size()) * sizeof(int)));
  TS_CUDA(cudaMalloc(&l->d_tiles, std::max(1, n_tiles) * sizeof(ts::TileDesc)));
  TS_CUDA(cudaMalloc(&l->d_wp, static_cast<size_t>(l->wp_rows) * l->ldw * 2));
  if (!kk.empty()) TS_CUDA(cudaMemcpy(l->d_kept_k, kk.data(), kk.size() * sizeof(int), cudaMemcpyHostToDevice));
  if (!nn.empty()) TS_CUDA(cudaMemcpy(l->d_kept_n, nn.data(), nn.size() * sizeof(int), cudaMemcpyHostToDevice));
  std::vector<ts::TileDesc> td(n_tiles);
  for (int t = 0; t < n_tiles; ++t) {
    td[t].k_list = l->d_kept_k + kp[t];
    td[t].n_list = l->d_kept_n + np[t];
    td[t].k_count = kc[t];
    td[t].n_count = nc[t];
    td[t].w_row0 = t * 128;
    td[t].c_row0 = 0;
    td[t].relative = 0;
    // kept columns consecutive in Ct and filling the 128-row store box (or ending at the last row)
    bool dense = nc[t] > 0;
    for (int j = 1; j < nc[t] && dense; ++j) dense = nn[np[t] + j] == nn[np[t]] + j;
    if (dense && nc[t] < 128) dense = nn[np[t]] + nc[t] == l->N;
    td[t].pad_ = dense ? 1 : 0;
  }
  if (n_tiles > 0) {
    TS_CUDA(cudaMemcpy(l->d_tiles, td.data(), td.size() * sizeof(ts::TileDesc), cudaMemcpyHostToDevice));
  }
  l->h_tiles = td;
  return make_weight_tmap(&l->tmap, l->dtype, l->d_wp, l->wp_rows, l->ldw);
}

int ts_layer_pack_weights(ts_layer_t* l, const void* W_dev, int64_t ldw_in, int w_dtype, void* stream) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  if (!l->d_wp) return fail(TS_ERR_INVALID, "layer has no tiles (call ts_layer_set_tiles)");
  if (!W_dev) return fail(TS_ERR_INVALID, "W is NULL");
  if (ldw_in < l->N) return fail(TS_ERR_INVALID, "ldw_in=%lld is smaller than N=%d", (long long)ldw_in, l->N);
  if (w_dtype != TS_DTYPE_F16 && w_dtype != TS_DTYPE_BF16 && w_dtype != TS_DTYPE_F32) {
    return fail(TS_ERR_INVALID, "unknown weight dtype %d", w_dtype);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TS_CUDA(cudaMemsetAsync(l->d_wp, 0, static_cast<size_t>(l->wp_rows) * l->ldw * 2, s));
  TS_CUDA(ts::pack_weights_launch(w_dtype, l->dtype, W_dev, ldw_in, l->d_tiles, l->n_tiles, l->max_k,
                                  l->d_wp, l->ldw, s));
  l->packed = true;
  l->wp_fresh = true;
  return TS_OK;
}

int ts_layer_set_unit_rows(ts_layer_t* l, int unit_rows) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  if (unit_rows != 0 && unit_rows != 128 && unit_rows != 256) {
    return fail(TS_ERR_INVALID, "unit_rows=%d must be 0 (automatic), 128 or 256", unit_rows);
  }
  if (unit_rows == l->forced_unit_rows) return TS_OK;
  TS_CUDA(cudaSetDevice(l->device));
  TS_CUDA(cudaDeviceSynchronize());   // cached schedules may be in use by queued launches
  for (auto& kv : l->schedules) free_schedule(kv.second);
  l->schedules.clear();
  l->forced_unit_rows = unit_rows;
  return TS_OK;
}

int ts_layer_set_split_k(ts_layer_t* l, int enabled) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  l->split_k = enabled != 0;
  return TS_OK;
}

int ts_plan_split(int n_tiles, const int32_t* k_counts, const int32_t* n_counts, int64_t K, int M, int n_ctas,
                  int32_t* parts_out) {
  if (n_tiles < 0 || (n_tiles > 0 && (!k_counts || !n_counts || !parts_out))) return fail(TS_ERR_INVALID, "NULL argument");
  if (M <= 0 || n_ctas <= 0) return fail(TS_ERR_INVALID, "M=%d and n_ctas=%d must be positive", M, n_ctas);
  std::vector<int> kc(k_counts, k_counts + n_tiles), nc(n_counts, n_counts + n_tiles), parts;
  plan_split(kc, nc, K, M, n_ctas, &parts);
  for (int t = 0; t < n_tiles; ++t) parts_out[t] = parts[t];
  return TS_OK;
}

int ts_layer_get_packed(const ts_layer_t* l, void* out_host, int64_t* rows, int64_t* ldw) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  if (rows) *rows = l->wp_rows;
  if (ldw) *ldw = l->ldw;
  if (!out_host) return TS_OK;
  if (!l->packed) return fail(TS_ERR_INVALID, "layer has no packed weights");
  TS_CUDA(cudaDeviceSynchronize());
  TS_CUDA(cudaMemcpy(out_host, l->d_wp, static_cast<size_t>(l->wp_rows) * l->ldw * 2, cudaMemcpyDeviceToHost));
  return TS_OK;
}

int ts_layer_stats(const ts_layer_t* l, int64_t* kept_flops_per_row, int64_t* packed_bytes,
                   int64_t* index_bytes, int* n_tiles, int* max_kept_k) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  int64_t kn = 0, idx = 0;
  for (int t = 0; t < l->n_tiles; ++t) {
    kn += static_cast<int64_t>(l->k_counts[t]) * l->n_counts[t];
    idx += l->k_counts[t] + l->n_counts[t];
  }
  if (kept_flops_per_row) *kept_flops_per_row = 2 * kn;
  if (packed_bytes) *packed_bytes = 2 * kn;
  if (index_bytes) *index_bytes = 4 * idx;
  if (n_tiles) *n_tiles = l->n_tiles;
  if (max_kept_k) *max_kept_k = l->max_k;
  return TS_OK;
}

}  // extern "C"

namespace {
// The masked GEMM over a matrix At[K][lda] (conv_wp == 0) or over a convolution's input planes.
int run_masked_gemm(ts_layer_t* l, int M, const void* At, int64_t lda, void* Ct, int64_t ldc,
                    const ts_epilogue_t* epi, void* stream, int conv_wp) {
  int rc = check_gemm_args(l, M, At, lda, Ct, ldc);
  if (rc != TS_OK) return rc;
  if (!epi) return fail(TS_ERR_INVALID, "epilogue is NULL");
  if (epi->activation < TS_ACT_NONE || epi->activation > TS_ACT_GELU) {
    return fail(TS_ERR_INVALID, "unknown activation %d", epi->activation);
  }
  if (epi->n_peers < 0 || epi->n_peers > 7) return fail(TS_ERR_INVALID, "n_peers=%d out of [0, 7]", epi->n_peers);
  ts::EpilogueArgs ep;
  ep.alpha = epi->alpha;
  ep.beta = epi->beta;
  ep.bias = epi->bias_dev;
  ep.act = epi->activation;
  ep.n_peers = epi->n_peers;
  for (int p = 0; p < 7; ++p) {
    ep.peers[p] = p < epi->n_peers ? static_cast<uint16_t*>(epi->peer_ct[p]) : nullptr;
    if (p < epi->n_peers && (!ep.peers[p] || (reinterpret_cast<uintptr_t>(ep.peers[p]) & 15u))) {
      return fail(TS_ERR_INVALID, "peer buffer %d is NULL or not 16-byte aligned", p);
    }
  }
  ep.multicast = static_cast<uint16_t*>(epi->multicast_ct);
  if (ep.multicast && ((reinterpret_cast<uintptr_t>(ep.multicast) & 15u) || epi->beta != 0.0f)) {
    return fail(TS_ERR_INVALID, "the multicast address must be 16-byte aligned and needs beta == 0");
  }
  if (M == 0 || l->n_tiles == 0) return TS_OK;
  Schedule* s = nullptr;
  // split-K units write fp32 partial sums to scratch memory of the schedule and a second kernel
  // finishes them; calls that also write peers (tile-sharded layers) keep whole units
  const bool allow_split = l->split_k && ep.n_peers == 0 && ep.multicast == nullptr;
  rc = get_schedule(l, M, lda, conv_wp, allow_split, &s);
  if (rc != TS_OK) return rc;
  if (s->n_units == 0) return TS_OK;
  ep.scratch = s->d_scratch;
  ep.scratch_ld = s->scratch_ld;
  ep.scratch_map = s->d_scratch_map;
  CUtensorMap tmap_c;
  rc = make_out_tmap(&tmap_c, l->dtype, Ct, l->N, M, ldc);
  if (rc != TS_OK) return rc;
  // Tile-sharded layers: the peers' copies of a full tile leave by TMA stores as well.  The maps are
  // encoded once per set of peer buffers and kept on the device.
  ep.peer_maps = nullptr;
  if (ep.n_peers > 0 && ep.multicast == nullptr && ep.beta == 0.0f) {
    bool same = l->d_peer_maps && l->peer_map_count == ep.n_peers && l->peer_map_m == M && l->peer_map_ldc == ldc;
    for (int p = 0; same && p < ep.n_peers; ++p) same = l->peer_map_ptrs[p] == ep.peers[p];
    if (!same) {
      if (!l->d_peer_maps) TS_CUDA(cudaMalloc(&l->d_peer_maps, sizeof(l->h_peer_maps)));
      l->peer_map_count = 0;
      for (int p = 0; p < ep.n_peers; ++p) {
        rc = make_out_tmap(&l->h_peer_maps[p], l->dtype, ep.peers[p], l->N, M, ldc);
        if (rc != TS_OK) return rc;
        l->peer_map_ptrs[p] = ep.peers[p];
      }
      // in stream order ahead of the launch below (the host copy lives in the layer)
      TS_CUDA(cudaMemcpyAsync(l->d_peer_maps, l->h_peer_maps, sizeof(CUtensorMap) * ep.n_peers,
                              cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
      l->peer_map_count = ep.n_peers;
      l->peer_map_m = M;
      l->peer_map_ldc = ldc;
    }
    ep.peer_maps = l->d_peer_maps;
  }
  // The kernel fetches packed weights before it waits for the kernel ahead of it in the stream.
  // The first launch after ts_layer_pack_weights may directly follow the packing kernel, so it runs
  // as an ordinary (fully ordered) launch; from then on the weights are old data.
  const bool early = !l->wp_fresh;
  TS_CUDA(ts::masked_gemm_launch(l->dtype, s->unit_rows, l->tmap, &tmap_c, s->d_units, s->rounds,
                                 s->grid, s->d_meta, s->blk_stride, At, lda, Ct, ldc, M, ep, l->d_status,
                                 early, s->all_dense, static_cast<cudaStream_t>(stream)));
  l->wp_fresh = false;
  if (s->n_split > 0) {
    TS_CUDA(ts::split_reduce_launch(l->dtype, s->d_split, s->n_split, s->d_scratch, s->scratch_ld, Ct, ldc, M,
                                    ep.beta, ep.bias, ep.act, static_cast<cudaStream_t>(stream)));
  }
  return TS_OK;
}
}  // namespace

extern "C" {

int ts_masked_gemm_ex(ts_layer_t* l, int M, const void* At, int64_t lda, void* Ct, int64_t ldc,
                      const ts_epilogue_t* epi, void* stream) {
  return run_masked_gemm(l, M, At, lda, Ct, ldc, epi, stream, 0);
}

int ts_layer_set_conv(ts_layer_t* l, int cin, int kh, int kw) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  if (cin <= 0 || kh <= 0 || kw <= 0 || (kh % 2) == 0 || (kw % 2) == 0 || kw > 9 || kh > 9) {
    return fail(TS_ERR_INVALID, "cin=%d, kh=%d, kw=%d: the kernel must be odd-sized, at most 9 x 9", cin, kh, kw);
  }
  if (static_cast<long long>(cin) * kh * kw != l->K) {
    return fail(TS_ERR_INVALID, "kh*kw*cin = %lld differs from the layer's K = %d", static_cast<long long>(cin) * kh * kw, l->K);
  }
  l->conv_cin = cin;
  l->conv_kh = kh;
  l->conv_kw = kw;
  return TS_OK;
}

int ts_conv_geometry(int B, int H, int W, int kh, int kw, int* Hp, int* Wp, int64_t* m_padded, int64_t* plane_ld) {
  if (B <= 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0) return fail(TS_ERR_INVALID, "non-positive size");
  const int hp = H + kh - 1, wp = (W + kw - 1 + 7) / 8 * 8;
  const int64_t m = static_cast<int64_t>(B) * hp * wp;
  if (m > 0x7fffffff - 4096) return fail(TS_ERR_UNSUPPORTED, "%lld padded pixels exceed the batch dimension's range", (long long)m);
  if (Hp) *Hp = hp;
  if (Wp) *Wp = wp;
  if (m_padded) *m_padded = m;
  if (plane_ld) *plane_ld = m + static_cast<int64_t>(kh - 1) * wp;
  return TS_OK;
}

int ts_conv_pack_input(const void* x_nhwc_dev, int B, int H, int W, int C, int kh, int kw, void* planes_dev,
                       int64_t plane_ld, void* stream) {
  int hp = 0, wp = 0;
  int64_t m = 0, need = 0;
  int rc = ts_conv_geometry(B, H, W, kh, kw, &hp, &wp, &m, &need);
  if (rc != TS_OK) return rc;
  if (C <= 0 || (C % 8) != 0 || (kh % 2) == 0 || (kw % 2) == 0 || kw > 9 || kh > 9) {
    return fail(TS_ERR_INVALID, "C=%d must be a multiple of 8; kh=%d, kw=%d must be odd and at most 9", C, kh, kw);
  }
  if (!x_nhwc_dev || !planes_dev || ((reinterpret_cast<uintptr_t>(x_nhwc_dev) | reinterpret_cast<uintptr_t>(planes_dev)) & 15u)) {
    return fail(TS_ERR_INVALID, "the input and the planes must be non-NULL and 16-byte aligned");
  }
  if (plane_ld < need || (plane_ld % 8) != 0) {
    return fail(TS_ERR_INVALID, "plane_ld=%lld must be a multiple of 8 and >= %lld", (long long)plane_ld, (long long)need);
  }
  if (B > 65535 || hp > 65535) return fail(TS_ERR_UNSUPPORTED, "more than 65535 images or padded rows");
  TS_CUDA(ts::conv_pack_input_launch(x_nhwc_dev, B, H, W, C, kh, kw, hp, wp, planes_dev, plane_ld,
                                     static_cast<cudaStream_t>(stream)));
  return TS_OK;
}

int ts_conv_repack(const void* Ct_dev, int64_t ldc, int B, int H, int W, int C, int kh, int kw, void* planes_dev,
                   int64_t plane_ld, void* stream) {
  int hp = 0, wp = 0;
  int64_t m = 0, need = 0;
  int rc = ts_conv_geometry(B, H, W, kh, kw, &hp, &wp, &m, &need);
  if (rc != TS_OK) return rc;
  if (C <= 0 || C > 65535 || (kh % 2) == 0 || (kw % 2) == 0 || kw > 9 || kh > 9) {
    return fail(TS_ERR_INVALID, "C=%d must be in [1, 65535]; kh=%d, kw=%d must be odd and at most 9", C, kh, kw);
  }
  if (!Ct_dev || !planes_dev || ((reinterpret_cast<uintptr_t>(planes_dev) | reinterpret_cast<uintptr_t>(Ct_dev)) & 15u) ||
      ldc < m || (ldc % 8) != 0) {
    return fail(TS_ERR_INVALID, "NULL or unaligned pointer, or ldc not a multiple of 8 >= the padded pixel count");
  }
  if (plane_ld < need || (plane_ld % 8) != 0) {
    return fail(TS_ERR_INVALID, "plane_ld=%lld must be a multiple of 8 and >= %lld", (long long)plane_ld, (long long)need);
  }
  TS_CUDA(ts::conv_repack_launch(Ct_dev, ldc, B, H, W, hp, wp, kh, kw, C, planes_dev, plane_ld,
                                 static_cast<cudaStream_t>(stream)));
  return TS_OK;
}

int ts_masked_conv(ts_layer_t* l, int B, int H, int W, const void* planes_dev, int64_t plane_ld, void* Ct_dev,
                   int64_t ldc, const ts_epilogue_t* epi, void* stream) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  if (l->conv_cin <= 0) return fail(TS_ERR_INVALID, "the layer has no convolution geometry (call ts_layer_set_conv)");
  int hp = 0, wp = 0;
  int64_t m = 0, need = 0;
  int rc = ts_conv_geometry(B, H, W, l->conv_kh, l->conv_kw, &hp, &wp, &m, &need);
  if (rc != TS_OK) return rc;
  if (plane_ld < need) return fail(TS_ERR_INVALID, "plane_ld=%lld is smaller than %lld", (long long)plane_ld, (long long)need);
  return run_masked_gemm(l, static_cast<int>(m), planes_dev, plane_ld, Ct_dev, ldc, epi, stream, wp);
}

int ts_conv_unpack_output(const void* Ct_dev, int64_t ldc, int B, int H, int W, int kh, int kw, int N, void* y_nhwc_dev,
                          void* stream) {
  int hp = 0, wp = 0;
  int64_t m = 0;
  int rc = ts_conv_geometry(B, H, W, kh, kw, &hp, &wp, &m, nullptr);
  if (rc != TS_OK) return rc;
  if (N <= 0 || (N % 8) != 0 || !Ct_dev || !y_nhwc_dev || ldc < m || (ldc % 8) != 0 ||
      ((reinterpret_cast<uintptr_t>(Ct_dev) | reinterpret_cast<uintptr_t>(y_nhwc_dev)) & 15u)) {
    return fail(TS_ERR_INVALID, "N and ldc must be multiples of 8 (ldc >= the padded pixel count), pointers 16-byte aligned");
  }
  if (B > 65535 || H > 65535) return fail(TS_ERR_UNSUPPORTED, "more than 65535 images or rows");
  TS_CUDA(ts::conv_unpack_output_launch(Ct_dev, ldc, B, H, W, hp, wp, N, y_nhwc_dev, static_cast<cudaStream_t>(stream)));
  return TS_OK;
}

int ts_masked_gemm(ts_layer_t* l, int M, const void* At, int64_t lda, void* Ct, int64_t ldc,
                   float alpha, float beta, void* stream) {
  ts_epilogue_t epi;
  memset(&epi, 0, sizeof(epi));
  epi.alpha = alpha;
  epi.beta = beta;
  return ts_masked_gemm_ex(l, M, At, lda, Ct, ldc, &epi, stream);
}

int ts_masked_gemm_simt(ts_layer_t* l, int M, const void* At, int64_t lda, void* Ct, int64_t ldc,
                        float alpha, float beta, void* stream) {
  int rc = check_gemm_args(l, M, At, lda, Ct, ldc);
  if (rc != TS_OK) return rc;
  if (M == 0 || l->n_tiles == 0) return TS_OK;
  TS_CUDA(ts::masked_gemm_simt_launch(l->dtype, l->d_tiles, l->n_tiles, l->d_wp, l->ldw, At, lda, Ct, ldc,
                                      M, alpha, beta, static_cast<cudaStream_t>(stream)));
  return TS_OK;
}

int ts_masked_gemm_host_async(ts_layer_t* l, int M, const void* At_host, void* Ct_host, float alpha,
                              float beta, void* stream) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  if (M <= 0 || (M % 8) != 0) return fail(TS_ERR_INVALID, "M=%d must be a positive multiple of 8", M);
  if (!At_host || !Ct_host) return fail(TS_ERR_INVALID, "host buffers are NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t a_bytes = static_cast<size_t>(l->K) * M * 2, c_bytes = static_cast<size_t>(l->N) * M * 2;
  if (a_bytes > l->at_bytes) {
    TS_CUDA(cudaDeviceSynchronize());
    cudaFree(l->d_at);
    l->d_at = nullptr;
    l->at_bytes = 0;
    TS_CUDA(cudaMalloc(&l->d_at, a_bytes));
    l->at_bytes = a_bytes;
  }
  if (c_bytes > l->ct_bytes) {
    TS_CUDA(cudaDeviceSynchronize());
    cudaFree(l->d_ct);
    l->d_ct = nullptr;
    l->ct_bytes = 0;
    TS_CUDA(cudaMalloc(&l->d_ct, c_bytes));
    l->ct_bytes = c_bytes;
    l->ct_dirty = true;
  }
  if (!l->s_in) {
    TS_CUDA(cudaStreamCreateWithFlags(&l->s_in, cudaStreamNonBlocking));
    TS_CUDA(cudaStreamCreateWithFlags(&l->s_mm, cudaStreamNonBlocking));
    TS_CUDA(cudaStreamCreateWithFlags(&l->s_out, cudaStreamNonBlocking));
  }
  // One contiguous copy in, one launch, one contiguous copy out, on three streams of the layer's own.
  // Cutting the batch into column blocks so that copy-in, GEMM and copy-out of one call overlap was
  // measured and dropped: a column block of a [K][M] buffer is a strided 2-D copy, which crosses the
  // PCIe link at 7-13 GB/s against 50-56 GB/s for a contiguous one.  The overlap that pays is between
  // calls on different layers (one call's copy-out under the next call's copy-in), which the
  // asynchronous form gives.
  const size_t need_events = 4;
  while (l->events.size() < need_events) {
    cudaEvent_t e;
    TS_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    l->events.push_back(e);
  }
  cudaEvent_t e_begin = l->events[0], e_end = l->events[1], e_in = l->events[2], e_mm = l->events[3];
  // A call on this layer that is still in flight uses the same staging buffers: the activations
  // may be overwritten once its GEMM has run, the output once its copy-out has.
  const bool rezero = beta == 0.0f && (l->ct_dirty || l->ct_zeroed_m != M);
  if (l->host_pending) {
    TS_CUDA(cudaStreamWaitEvent(l->s_in, (rezero || beta != 0.0f) ? e_end : e_mm, 0));
    TS_CUDA(cudaStreamWaitEvent(l->s_mm, e_end, 0));
  }
  // everything this call does comes after what the caller has queued on its stream ...
  TS_CUDA(cudaEventRecord(e_begin, s));
  TS_CUDA(cudaStreamWaitEvent(l->s_in, e_begin, 0));
  // Columns no tile keeps are never written by the kernel: with beta == 0 they must come back as zeros.
  if (rezero) {
    TS_CUDA(cudaMemsetAsync(l->d_ct, 0, c_bytes, l->s_in));
    l->ct_zeroed_m = M;
  }
  TS_CUDA(cudaMemcpyAsync(l->d_at, At_host, a_bytes, cudaMemcpyHostToDevice, l->s_in));
  if (beta != 0.0f) TS_CUDA(cudaMemcpyAsync(l->d_ct, Ct_host, c_bytes, cudaMemcpyHostToDevice, l->s_in));
  TS_CUDA(cudaEventRecord(e_in, l->s_in));
  TS_CUDA(cudaStreamWaitEvent(l->s_mm, e_in, 0));
  {
    int rc = ts_masked_gemm(l, M, l->d_at, M, l->d_ct, M, alpha, beta, l->s_mm);
    if (rc != TS_OK) return rc;
  }
  TS_CUDA(cudaEventRecord(e_mm, l->s_mm));
  TS_CUDA(cudaStreamWaitEvent(l->s_out, e_mm, 0));
  TS_CUDA(cudaMemcpyAsync(Ct_host, l->d_ct, c_bytes, cudaMemcpyDeviceToHost, l->s_out));
  // ... and ts_masked_gemm_host_wait orders a stream after the arrival of the last block
  TS_CUDA(cudaEventRecord(e_end, l->s_out));
  l->host_pending = true;
  l->ct_dirty = beta != 0.0f;   // a beta pass leaves the caller's values in the columns no tile keeps
  return TS_OK;
}

int ts_masked_gemm_host_wait(ts_layer_t* l, void* stream) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  if (!l->host_pending) return TS_OK;
  TS_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), l->events[1], 0));
  return TS_OK;
}

int ts_masked_gemm_host(ts_layer_t* l, int M, const void* At_host, void* Ct_host, float alpha,
                        float beta, void* stream) {
  int rc = ts_masked_gemm_host_async(l, M, At_host, Ct_host, alpha, beta, stream);
  if (rc != TS_OK) return rc;
  rc = ts_masked_gemm_host_wait(l, stream);
  if (rc != TS_OK) return rc;
  TS_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return TS_OK;
}

int ts_layer_check(ts_layer_t* l, void* stream) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int st = 0;
  TS_CUDA(cudaMemcpyAsync(&st, l->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
  TS_CUDA(cudaStreamSynchronize(s));
  if (st != 0) {
    TS_CUDA(cudaMemsetAsync(l->d_status, 0, sizeof(int), s));
    TS_CUDA(cudaStreamSynchronize(s));
    return fail(st, "a masked GEMM kernel reported status %d (%s)", st,
                st == TS_ERR_TIMEOUT ? "a bounded device-side wait ran out" : "unknown");
  }
  return TS_OK;
}

int ts_layer_schedule_stats(ts_layer_t* l, int M, int* n_ctas, float* cta_cost, int* n_units) {
  if (!l) return fail(TS_ERR_INVALID, "layer is NULL");
  if (M <= 0) return fail(TS_ERR_INVALID, "M=%d must be positive", M);
  if (!l->d_tiles) return fail(TS_ERR_INVALID, "layer has no tiles");
  Schedule* s = nullptr;
  int rc = get_schedule(l, M, M, 0, l->split_k, &s);
  if (rc != TS_OK) return rc;
  if (n_ctas) *n_ctas = s->grid;
  if (n_units) *n_units = s->n_units;
  if (cta_cost) memcpy(cta_cost, s->cta_cost.data(), s->cta_cost.size() * sizeof(float));
  return TS_OK;
}

// Workspace of the reference-signature entry point: one per device, grown on demand, reused by
// every call (calls on one device must be issued on one stream or externally ordered).
namespace {
struct ShimWorkspace {
  ts::WorkItem* d_units = nullptr;
  size_t unit_cap = 0;
  ts::BlockDesc* d_blocks = nullptr;
  int* d_meta = nullptr;
  long long n_blocks = 0;
  size_t block_cap = 0;
  // The schedule of the previous call, reused when the next call describes the same tiles (a perf
  // loop calls with identical arguments every iteration).
  std::vector<long long> key;
  int rounds = 0, grid = 0, blk_stride = 0, unit_rows = 0;
  int* d_status = nullptr;
};
std::mutex g_shim_mu;
std::map<int, ShimWorkspace> g_shim_ws;
}  // namespace

int ts_stream_gemm_nn(int M, int N, int K, float alpha, const void* A, const void* B, float beta,
                      void* C, int block_num, const int* N_cal, const int* K_cal,
                      int* const* mask_n, int* const* mask_k, const int* off_B, const int* off_C,
                      int dtype, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return fail(TS_ERR_INVALID, "M, N, K must be positive");
  if ((M % 8) != 0 || (K % 8) != 0) return fail(TS_ERR_INVALID, "M and K must be multiples of 8");
  if (block_num < 0 || block_num > 32) {
    return fail(TS_ERR_INVALID, "block_num=%d out of [0, 32] (MAX_BLOCK_NUM of the reference)", block_num);
  }
  if (dtype != TS_DTYPE_F16 && dtype != TS_DTYPE_BF16) return fail(TS_ERR_INVALID, "dtype must be f16 or bf16");
  if (static_cast<long long>(K) * (M / 8) >= (1LL << 31)) {
    return fail(TS_ERR_UNSUPPORTED, "A of %d x %d elements exceeds the 32 GiB the block records address", K, M);
  }
  if (block_num == 0) return TS_OK;
  if (!A || !B || !C || !N_cal || !K_cal || !mask_n || !mask_k || !off_B || !off_C) {
    return fail(TS_ERR_INVALID, "NULL argument");
  }
  if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(C) & 15u)) {
    return fail(TS_ERR_INVALID, "A and C must be 16-byte aligned");
  }
  std::vector<ts::TileDesc> td(block_num);
  std::vector<int> kc(block_num), nc(block_num);
  for (int t = 0; t < block_num; ++t) {
    if (N_cal[t] < 0 || N_cal[t] > 128) return fail(TS_ERR_INVALID, "N_cal[%d]=%d out of [0,128]", t, N_cal[t]);
    if (K_cal[t] < 0 || K_cal[t] > K) return fail(TS_ERR_INVALID, "K_cal[%d]=%d out of [0,K]", t, K_cal[t]);
    if (off_B[t] % K != 0 || off_C[t] % M != 0) {
      return fail(TS_ERR_INVALID, "off_B[%d] must be a multiple of K and off_C[%d] of M", t, t);
    }
    if ((K_cal[t] > 0 && !mask_k[t]) || (N_cal[t] > 0 && !mask_n[t])) {
      return fail(TS_ERR_INVALID, "mask pointer of tile %d is NULL", t);
    }
    td[t].k_list = mask_k[t];
    td[t].n_list = mask_n[t];
    td[t].k_count = kc[t] = K_cal[t];
    td[t].n_count = nc[t] = N_cal[t];
    td[t].w_row0 = off_B[t] / K;
    td[t].c_row0 = off_C[t] / M;
    td[t].relative = 1;
    td[t].pad_ = 0;
  }
  int dev = 0, sms = 0;
  TS_CUDA(cudaGetDevice(&dev));
  int rc = current_sm_count(&sms);
  if (rc != TS_OK) return rc;
  CUtensorMap tmap;
  rc = make_weight_tmap(&tmap, dtype, B, N, K);
  if (rc != TS_OK) return rc;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  std::lock_guard<std::mutex> lock(g_shim_mu);
  ShimWorkspace& ws = g_shim_ws[dev];
  if (!ws.d_status) {
    TS_CUDA(cudaMalloc(&ws.d_status, sizeof(int)));
    TS_CUDA(cudaMemset(ws.d_status, 0, sizeof(int)));
  }
  std::vector<long long> key = {M, N, K, block_num, dtype};
  for (int t = 0; t < block_num; ++t) {
    key.push_back(N_cal[t]);
    key.push_back(K_cal[t]);
    key.push_back(off_B[t]);
    key.push_back(off_C[t]);
    key.push_back(reinterpret_cast<long long>(mask_k[t]));
    key.push_back(reinterpret_cast<long long>(mask_n[t]));
  }
  if (key != ws.key) {
    std::vector<ts::WorkItem> flat;
    std::vector<float> cost;
    std::vector<ts::BlockDesc> blocks;
    int n_units = 0;
    build_schedule(td, K, M, 0, sms, &flat, &ws.rounds, &ws.grid, &n_units, &ws.unit_rows, &cost, &blocks,
                   &ws.blk_stride);
    ws.key.clear();
    if (n_units == 0) return TS_OK;
    if (flat.size() > ws.unit_cap) {
      TS_CUDA(cudaStreamSynchronize(s));
      cudaFree(ws.d_units);
      ws.d_units = nullptr;
      ws.unit_cap = 0;
      TS_CUDA(cudaMalloc(&ws.d_units, flat.size() * sizeof(ts::WorkItem)));
      ws.unit_cap = flat.size();
    }
    if (blocks.size() > ws.block_cap) {
      TS_CUDA(cudaStreamSynchronize(s));
      cudaFree(ws.d_blocks);
      cudaFree(ws.d_meta);
      ws.d_blocks = nullptr;
      ws.d_meta = nullptr;
      ws.block_cap = 0;
      TS_CUDA(cudaMalloc(&ws.d_blocks, blocks.size() * sizeof(ts::BlockDesc)));
      TS_CUDA(cudaMalloc(&ws.d_meta, blocks.size() * ts::kBlockMetaInts * sizeof(int)));
      ws.block_cap = blocks.size();
    }
    // Pageable sources: the runtime stages them before returning, so the vectors may die after this.
    TS_CUDA(cudaMemcpyAsync(ws.d_units, flat.data(), flat.size() * sizeof(ts::WorkItem), cudaMemcpyHostToDevice, s));
    TS_CUDA(cudaMemcpyAsync(ws.d_blocks, blocks.data(), blocks.size() * sizeof(ts::BlockDesc),
                            cudaMemcpyHostToDevice, s));
    ws.key = key;
    ws.n_blocks = static_cast<long long>(blocks.size());
  }
  // The caller owns the offset lists and may have rewritten them since the schedule was cached:
  // they are resolved again on every call.
  ts::RowMap map;
  memset(&map, 0, sizeof(map));
  map.ld8 = M / 8;
  TS_CUDA(ts::expand_block_meta_launch(ws.d_blocks, ws.n_blocks, ws.d_meta, map, s));
  const int rounds = ws.rounds, grid = ws.grid, blk_stride = ws.blk_stride, unit_rows = ws.unit_rows;
  ts::EpilogueArgs ep;
  memset(&ep, 0, sizeof(ep));
  ep.alpha = alpha;
  ep.beta = beta;
  TS_CUDA(ts::masked_gemm_launch(dtype, unit_rows, tmap, nullptr, ws.d_units, rounds, grid,
                                 ws.d_meta, blk_stride, A, M, C, M, M, ep, ws.d_status, /*early_start=*/false,
                                 /*lean=*/false, s));
  return TS_OK;
}

int ts_residual_gemm(int dtype, int M, int N, const int32_t* col_ptr_dev, const int32_t* row_idx_dev,
                     const void* val_dev, const uint8_t* col_written_dev, const void* At_dev, int64_t lda,
                     void* Ct_dev, int64_t ldc, float alpha, void* stream) {
  if (dtype != TS_DTYPE_F16 && dtype != TS_DTYPE_BF16) return fail(TS_ERR_INVALID, "dtype must be f16 or bf16");
  if (M < 0 || N < 0 || (M % 8) != 0) return fail(TS_ERR_INVALID, "M=%d must be a non-negative multiple of 8", M);
  if (M == 0 || N == 0) return TS_OK;
  if (!col_ptr_dev || !At_dev || !Ct_dev) return fail(TS_ERR_INVALID, "NULL argument");
  if (lda < M || ldc < M || (lda % 8) != 0 || (ldc % 8) != 0) {
    return fail(TS_ERR_INVALID, "lda / ldc must be multiples of 8 and >= M");
  }
  if ((reinterpret_cast<uintptr_t>(At_dev) & 15u) || (reinterpret_cast<uintptr_t>(Ct_dev) & 15u)) {
    return fail(TS_ERR_INVALID, "At and Ct must be 16-byte aligned");
  }
  TS_CUDA(ts::residual_spmm_launch(dtype, col_ptr_dev, row_idx_dev, val_dev, col_written_dev, At_dev, lda, Ct_dev,
                                   ldc, M, N, alpha, static_cast<cudaStream_t>(stream)));
  return TS_OK;
}

int ts_transpose16(const void* in_dev, int64_t ld_in, void* out_dev, int64_t ld_out, int rows,
                   int cols, void* stream) {
  if (rows < 0 || cols < 0) return fail(TS_ERR_INVALID, "negative shape");
  if (rows == 0 || cols == 0) return TS_OK;
  if (!in_dev || !out_dev) return fail(TS_ERR_INVALID, "NULL pointer");
  if (ld_in < cols || ld_out < rows) return fail(TS_ERR_INVALID, "leading dimensions too small");
  TS_CUDA(ts::transpose16_launch(in_dev, ld_in, out_dev, ld_out, rows, cols, static_cast<cudaStream_t>(stream)));
  return TS_OK;
}

int ts_plan_schedule(int n_tiles, const int32_t* k_counts, const int32_t* n_counts, int64_t K, int M, int n_ctas,
                     int unit_rows, int* unit_rows_out, int* n_ctas_out, int* n_units_out, int32_t* units_out,
                     int max_units, float* cta_cost_out) {
  if (n_tiles < 0 || M <= 0 || K <= 0 || n_ctas <= 0) {
    return fail(TS_ERR_INVALID, "n_tiles=%d, K=%lld, M=%d, n_ctas=%d", n_tiles, (long long)K, M, n_ctas);
  }
  if (n_tiles > 0 && (!k_counts || !n_counts)) return fail(TS_ERR_INVALID, "NULL argument");
  if (unit_rows != 0 && unit_rows != 128 && unit_rows != 256) {
    return fail(TS_ERR_INVALID, "unit_rows=%d must be 0 (automatic), 128 or 256", unit_rows);
  }
  std::vector<ts::TileDesc> td(n_tiles);
  for (int t = 0; t < n_tiles; ++t) {
    if (k_counts[t] < 0 || n_counts[t] < 0 || n_counts[t] > 128) {
      return fail(TS_ERR_INVALID, "tile %d: k_count=%d, n_count=%d", t, k_counts[t], n_counts[t]);
    }
    memset(&td[t], 0, sizeof(td[t]));
    td[t].k_count = k_counts[t];
    td[t].n_count = n_counts[t];
    td[t].w_row0 = t * 128;
  }
  std::vector<ts::WorkItem> flat;
  std::vector<ts::BlockDesc> blocks;
  std::vector<float> cost;
  int rounds = 0, grid = 0, n_units = 0, urows = 0, blk_stride = 0;
  build_schedule(td, K, M, unit_rows, n_ctas, &flat, &rounds, &grid, &n_units, &urows, &cost, &blocks, &blk_stride);
  if (unit_rows_out) *unit_rows_out = urows;
  if (n_ctas_out) *n_ctas_out = grid;
  if (n_units_out) *n_units_out = n_units;
  if (cta_cost_out) memcpy(cta_cost_out, cost.data(), cost.size() * sizeof(float));
  if (units_out) {
    if (n_units > max_units) return fail(TS_ERR_INVALID, "units_out holds %d units, the schedule has %d", max_units, n_units);
    int o = 0;
    for (int b = 0; b < grid; ++b) {
      for (int r = 0; r < rounds; ++r) {
        const ts::WorkItem& w = flat[static_cast<size_t>(r) * grid + b];
        if (w.tile < 0) break;
        units_out[4 * o] = b;
        units_out[4 * o + 1] = w.tile;
        units_out[4 * o + 2] = w.m_begin;
        units_out[4 * o + 3] = w.m_len;
        ++o;
      }
    }
  }
  return TS_OK;
}

int ts_shard_plan(int n_tiles, const int64_t* cost, int n_parts, int32_t* owner_out) {
  if (n_tiles < 0 || n_parts <= 0) return fail(TS_ERR_INVALID, "n_tiles=%d, n_parts=%d", n_tiles, n_parts);
  if (n_tiles == 0) return TS_OK;
  if (!cost || !owner_out) return fail(TS_ERR_INVALID, "NULL argument");
  std::vector<int> order(n_tiles);
  for (int t = 0; t < n_tiles; ++t) order[t] = t;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost[a] > cost[b]; });
  typedef std::pair<int64_t, int> Load;
  std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
  for (int p = 0; p < n_parts; ++p) heap.push({0, p});
  for (int t : order) {
    Load l = heap.top();
    heap.pop();
    owner_out[t] = l.second;
    l.first += std::max<int64_t>(cost[t], 0);
    heap.push(l);
  }
  return TS_OK;
}

}  // extern "C"

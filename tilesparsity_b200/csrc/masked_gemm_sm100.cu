// Persistent grouped masked GEMM for tile-wise sparse weights (sm_100a: tcgen05 + TMEM + TMA).
//
// Replaces the reference's per-tile CUTLASS launches (one stream per column tile,
// StreamMaskedGEMM/perf/basic_nn.cu:378-445; kernel StreamMaskedGEMM/cutlass/gemm/gemm.h:45-61 with
// the masked A loads of cutlass/tile_iterator.h:786-816 and the masked stores of :1262-1292) by ONE
// launch over a work list.  Data layout is the reference's (column-major everywhere,
// basic_nn.cu:412-426):
//
//   At : activations, stored [K][lda] with the batch dimension M contiguous (column-major M x K)
//   Wp : packed weights, stored [rows][ldw] with K contiguous; tile t owns rows w_row0 .. +n_count,
//        entry (j, i) = W[kept_k[i], kept_n[j]]   (gen_masked_stream_weight, basic_nn.cu:757-769)
//   Ct : output, stored [N][ldc] with M contiguous; kept column j of a tile lands in row c_row(j)
//
// and the product computed per tile is  Ct[c_row(j), m] = alpha * sum_i Wp[j, i] * At[kept_k[i], m]
// (+ beta * Ct), accumulated in fp32.
//
// Mapping onto the tensor core: the tile's kept columns are the MMA's M dimension (128 TMEM lanes),
// the batch is its N dimension (MT = 128 or 256 columns per instruction), the kept rows are K.  The
// packed weights are the K-major A operand, fetched by TMA with 128-byte swizzle; the gathered
// activation rows are the MN-major B operand, fetched with 16-byte cp.async into the same swizzle
// pattern (one kept row is one contiguous 2*MT-byte global segment).  The four gather warps fill
// each 64-row K block together; block descriptors and kept-row indices are prefetched into small
// shared-memory rings; each lane
// hands its copies to the stage's mbarrier with cp.async.mbarrier.arrive, so a stage is released to
// the MMA warp the moment its bytes have landed.  Accumulators live in TMEM, double buffered: the
// epilogue of one work unit overlaps the main loop of the next.  Eight epilogue warps (two per TMEM
// lane quarter, each taking half of the unit's batch columns) convert their rows to 16 bit into a
// 128-byte-swizzled staging tile in shared memory.  When the tile's kept columns are consecutive
// rows of Ct (no column pruning) the tile leaves with one TMA store per 64 batch columns; otherwise
// the epilogue warps write the rows with 16-byte coalesced stores through the kept-column list.
//
// Warp roles (448 threads): warp 0 = weight TMA, warp 1 = TMEM allocation + MMA issue,
// warps 2-5 = activation gather, warps 6-13 = epilogue.
#include <cstdlib>

#include "ts_common.cuh"
#include "ts_kernels.h"

namespace ts {

namespace {

constexpr int kNT = 128;                 // columns per tile (MMA M, TMEM lanes)
constexpr int kKB = 64;                  // kept rows per pipeline stage
constexpr int kWBytes = kNT * kKB * 2;   // 16 KiB of packed weights per stage
constexpr int kThreads = 448;
constexpr int kEpiThreads = 256;
constexpr uint32_t kASbo = 1024;         // bytes between 8-row K groups of the gathered operand
constexpr uint32_t kALbo = kKB * 128;    // bytes between its 64-column batch groups
constexpr uint32_t kWSbo = 1024;         // bytes between 8-row groups of the weight operand
constexpr int kMaxStages = 5;

// Compile-time shape of one kernel variant: MT batch rows per work unit.
template <int MT>
struct Cfg {
  static constexpr int kStages = MT == 256 ? 3 : 5;
  static constexpr int kABytes = kKB * MT * 2;
  static constexpr int kStageBytes = kWBytes + kABytes;
  static constexpr int kEpiGroupBytes = kNT * 128;   // staging: one 128-row x 64-column swizzled group
  static constexpr int kEpiBytes = (MT / 64) * kEpiGroupBytes;
  static constexpr int kTmemCols = 2 * MT;          // two accumulators of MT fp32 columns
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 6144 + 1024;
  static constexpr int kLanesPerRow = MT / 8;       // 16-byte chunks in one gathered row
  static constexpr int kRowsPerInstr = 32 / kLanesPerRow;
};

// Optional cycle-stamp trace of CTA 0 (debug builds only: -DTS_KERNEL_TRACE).  Slot i receives
// clock64() the first time the kernel passes trace point i.
#ifdef TS_KERNEL_TRACE
__device__ long long g_trace[256];
#define TS_TRACE(id, leader)                                                       \
  do {                                                                             \
    if (blockIdx.x == 0 && (leader) && g_trace[id] == 0) g_trace[id] = clock64();  \
  } while (0)
// Per-unit stamps: slot 64 + kind*8 + unit for the CTA's first eight units.
#define TS_TRACE_U(kind, unit, leader)                                              \
  do {                                                                             \
    if ((unit) < 8) TS_TRACE(64 + (kind)*8 + (unit), leader);                       \
  } while (0)
#else
#define TS_TRACE(id, leader) \
  do {                       \
  } while (0)
#define TS_TRACE_U(kind, unit, leader) \
  do {                                 \
  } while (0)
#endif

struct Barriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int c_row[kNT];  // Ct row of each tile column of the unit in the epilogue (-1: not kept)
  // Per gather warp: ring of block descriptors (8 slots) and of kept-row indices (4 slots x 64).
  BlockDesc desc_ring[4][8];
  int idx_ring[4][4][kKB];
};

__device__ __forceinline__ WorkItem load_item(const WorkItem* p) {
  const int4* q = reinterpret_cast<const int4*>(p);
  union {
    int4 v[3];
    WorkItem w;
  } u;
  u.v[0] = __ldg(q);
  u.v[1] = __ldg(q + 1);
  u.v[2] = __ldg(q + 2);
  return u.w;
}

// Work item of CTA `cta` in round r, or an empty item past the end of the schedule.
__device__ __forceinline__ WorkItem fetch_item(const WorkItem* sched, int rounds, int grid, int cta,
                                               int r) {
  if (r < rounds) return load_item(sched + static_cast<size_t>(r) * grid + cta);
  WorkItem w;
  w.k_list = nullptr;
  w.n_list = nullptr;
  w.k_count = w.n_count = w.w_row0 = w.c_row0 = w.flags = w.m_begin = w.m_len = 0;
  w.tile = -1;
  return w;
}

__device__ __forceinline__ int k_blocks(const WorkItem& w) { return (w.k_count + kKB - 1) / kKB; }

// Ct row (global column of W) of tile column j of a work item.
__device__ __forceinline__ long long c_row_of(const WorkItem& w, int j) {
  return w.c_row0 + (w.n_list ? __ldg(w.n_list + j) + ((w.flags & kItemRelative) ? j : 0) : j);
}

__device__ __forceinline__ float apply_act(float x, int act) {
  if (act == kActRelu) return fmaxf(x, 0.0f);
  if (act == kActGelu) {
    // x * 0.5 * (1 + tanh(sqrt(2/pi) * (x + 0.044715 x^3)))   (Pruning/BERT/utils/modeling.py:264-277)
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(u));
  }
  return x;
}

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int DT, int MT, int TMA_ROWS>
__global__ void __launch_bounds__(kThreads, 1)
masked_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                   const __grid_constant__ CUtensorMap tmap_c, int use_tma_store,
                   const WorkItem* __restrict__ sched,
                   int rounds, const BlockDesc* __restrict__ blocks, int blk_stride, int K_oob,
                   const uint16_t* __restrict__ At, long long lda,
                   uint16_t* __restrict__ Ct, long long ldc, int M, const EpilogueArgs ep,
                   int* __restrict__ status) {
  const float alpha = ep.alpha, beta = ep.beta;
  using C = Cfg<MT>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the swizzle pattern is a function of the shared-memory address bits.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi = smem + kStages * C::kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(epi + C::kEpiBytes);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int grid = gridDim.x;
  const int cta = blockIdx.x;
  TS_TRACE(0, threadIdx.x == 0);

  // First work item (and, for the gather warps, its first kept-row indices): requested before the
  // set-up below so their latency overlaps it.
  WorkItem w = fetch_item(sched, rounds, grid, cta, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      // weight TMA thread + the gather leader's expect-tx arrival (rows fetched by TMA) + the 128
      // cp.async lanes (rows fetched through the load/store unit)
      mbar_init(smem_u32(&bars->full[s]), 1 + (TMA_ROWS > 0 ? 1 : 0) + (TMA_ROWS < kKB ? 128 : 0));
      mbar_init(smem_u32(&bars->empty[s]), 1);       // one tcgen05.commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bars->acc_full[a]), 1);
      mbar_init(smem_u32(&bars->acc_empty[a]), kEpiThreads);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  TS_TRACE(1, threadIdx.x == 0);
  // The next kernel in the stream may begin its own set-up now (it cannot touch this kernel's
  // outputs before its grid_dependency_wait, which returns only when this grid has completed).
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------------ weight TMA producer
    if (lane == 0) tma_prefetch_desc(&tmap_w);
    uint32_t it = 0;
    bool ok = true;
    for (int r = 0; ok && w.tile >= 0; ++r) {
      const WorkItem wn = fetch_item(sched, rounds, grid, cta, r + 1);
      const int nkb = (w.k_count + kKB - 1) / kKB;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const uint32_t s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        ok = mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t bar = smem_u32(&bars->full[s]);
          mbar_arrive_expect_tx(bar, kWBytes);
          tma_load_2d(smem_u32(smem + s * C::kStageBytes), &tmap_w, kb * kKB, w.w_row0, bar);
        }
        __syncwarp();
      }
      w = wn;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // the MMA's N dimension is the unit's batch-row count (a multiple of 64, at most MT)
    constexpr uint32_t idesc0 = umma_idesc_f16(DT == kBF16 ? 1 : 0, /*a_mn=*/0, /*b_mn=*/1, kNT, 0);
    uint32_t it = 0, acc_it = 0;
    bool ok = true;
    for (int r = 0; ok && w.tile >= 0; ++r) {
      const WorkItem wn = fetch_item(sched, rounds, grid, cta, r + 1);
      const int nkb = (w.k_count + kKB - 1) / kKB;
      const uint32_t a = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      ok = mbar_wait(smem_u32(&bars->acc_empty[a]), aph ^ 1u, abort_flag);
      if (!ok) break;
      TS_TRACE_U(0, acc_it, lane == 0);
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + a * MT;
      const uint32_t idesc = idesc0 | (static_cast<uint32_t>(w.m_len >> 3) << 17);
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const uint32_t s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        ok = mbar_wait(smem_u32(&bars->full[s]), ph, abort_flag);
        if (!ok) break;
        TS_TRACE(8 + (it < 4 ? it : 4), lane == 0);
        if (kb == 0) TS_TRACE_U(1, acc_it, lane == 0);
        if (kb == nkb - 1) TS_TRACE_U(2, acc_it, lane == 0);
        // The gathered rows were written through the generic proxy; the MMA reads them through
        // the async proxy.
        fence_proxy_async_smem();
        tc_fence_after_sync();
        if (lane == 0) {
          const int krem = w.k_count - kb * kKB;
          const int nk16 = krem >= kKB ? kKB / 16 : (krem + 15) / 16;
          const uint32_t w_addr = smem_u32(smem + s * C::kStageBytes);
          const uint32_t a_addr = w_addr + kWBytes;
          for (int k = 0; k < nk16; ++k) {
            // weights: K-major, 16 K elements = 32 bytes inside the 128-byte swizzled row
            const uint64_t dw = umma_smem_desc_sw128(w_addr + k * 32, 16, kWSbo);
            // activations: MN-major, 16 K rows = two 8-row groups
            const uint64_t da = umma_smem_desc_sw128(a_addr + k * 2 * kASbo, kALbo, kASbo);
            umma_f16(tmem_d, dw, da, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&bars->empty[s]));
        }
        __syncwarp();
      }
      if (!ok) break;
      if (lane == 0) {
        if (nkb > 0) {
          umma_commit(smem_u32(&bars->acc_full[a]));
        } else {
          mbar_arrive(smem_u32(&bars->acc_full[a]));  // tile with no kept rows: nothing to wait for
        }
      }
      __syncwarp();
      TS_TRACE(16, lane == 0);
      ++acc_it;
      w = wn;
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ activation gather
    // The four gather warps fill every 64-row K block together, a quarter of its copies each, so a
    // stage is occupied only briefly before the MMA warp can consume it.  Everything a warp needs
    // arrives by cp.async, requested ahead of use: the descriptor of block j+4 and the kept-row
    // indices of block j+2 are requested while block j is copied, so no step of the loop waits on
    // a dependent global read.
    constexpr int kGW = 4;
    const int gw = warp - 2;
    const BlockDesc* bd = blocks + static_cast<size_t>(cta) * blk_stride;
    BlockDesc* dring = bars->desc_ring[gw];
    int(*iring)[kKB] = bars->idx_ring[gw];

    auto request_indices = [&](int jj) {
      const BlockDesc d = dring[jj & 7];
      if (d.meta != kBlockEnd) {
        const int nv = static_cast<int>(d.meta & 0x7fu);
        if (lane < nv) cp_async_4(smem_u32(&iring[jj & 3][lane]), d.idx + lane);
        if (lane + 32 < nv) cp_async_4(smem_u32(&iring[jj & 3][lane + 32]), d.idx + lane + 32);
      }
    };
    // prologue: descriptors of blocks 0..3 by plain loads, indices of blocks 0 and 1 requested
    if (lane < 4) dring[lane] = bd[lane];
    __syncwarp();
    request_indices(0);
    cp_async_commit();
    request_indices(1);
    cp_async_commit();
    // The schedule and the index lists are static; the activations may be the previous kernel's
    // output: wait for it before the first row is copied.
    grid_dependency_wait();

    bool ok = true;
    for (int j = 0; ok; ++j) {
      cp_async_wait_group<1>();   // indices of block j and descriptor of block j+2 have landed
      __syncwarp();
      const BlockDesc d = dring[j & 7];
      if (d.meta == kBlockEnd) break;
      request_indices(j + 2);
      if (lane == 0) cp_async_16_ca(smem_u32(&dring[(j + 4) & 7]), bd + j + 4);
      cp_async_commit();

      const uint32_t it = static_cast<uint32_t>(j);
      const uint32_t s = it % kStages;
      const uint32_t ph = (it / kStages) & 1u;
      if (j < 8) TS_TRACE(208 + j, lane == 0 && gw == 0);
      ok = mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag);
      if (!ok) break;
      if (j < 8) TS_TRACE(192 + j * 2, lane == 0 && gw == 0);
      const int nv = static_cast<int>(d.meta & 0x7fu);
      const int rel = (d.meta & 0x80u) ? static_cast<int>(d.meta >> 10) : -1;  // list position, if relative
      const int m_len = (static_cast<int>((d.meta >> 8) & 3u) + 1) * 64;        // batch rows of the unit
      const int* idx = iring[j & 3];
      const uint32_t a_base = smem_u32(smem + s * C::kStageBytes + kWBytes);
      const uint32_t bar = smem_u32(&bars->full[s]);
      // The block's first TMA_ROWS rows come through the copy engine (tile::gather4), the rest
      // through the load/store unit (cp.async): the two paths run side by side.
      if constexpr (TMA_ROWS > 0) {
        // One gather4 per four kept rows and 64 batch columns (512 bytes).  Rows past the end of the
        // list use a row index outside the tensor, which reads as zeros.
        if (gw == 0 && lane == 0) mbar_arrive_expect_tx(bar, TMA_ROWS * m_len * 2);
        constexpr int kKg = TMA_ROWS / 4;                 // groups of four rows
        constexpr int kOps = kKg * (MT / 64);
        constexpr int kOpsPerWarp = (kOps + kGW - 1) / kGW;
        static_assert(kOpsPerWarp <= 32, "one gather4 per lane");
        const int qq = gw * kOpsPerWarp + lane;
        if (lane < kOpsPerWarp && qq < kOps && (qq / kKg) * 64 < m_len) {
          const int kg = qq % kKg, mg = qq / kKg;
          const int4 r4 = *reinterpret_cast<const int4*>(idx + kg * 4);
          const int base = kg * 4;
          const int add = rel >= 0 ? rel + base : 0;
          const int step = rel >= 0 ? 1 : 0;
          const int r0 = base + 0 < nv ? r4.x + add : K_oob;
          const int r1 = base + 1 < nv ? r4.y + add + step : K_oob;
          const int r2 = base + 2 < nv ? r4.z + add + 2 * step : K_oob;
          const int r3 = base + 3 < nv ? r4.w + add + 3 * step : K_oob;
          tma_gather4(a_base + mg * kALbo + (kg >> 1) * kASbo + (kg & 1) * 512, &tmap_a, d.m0 + mg * 64, r0,
                      r1, r2, r3, bar);
        }
      }
      if constexpr (TMA_ROWS < kKB) {
        // 16-byte cp.async copies: this warp takes a quarter of the remaining rows.  Their indices
        // are read into registers before the first copy goes out (a shared-memory read between two
        // copies would serialise them).
        constexpr int kLpr = C::kLanesPerRow, kRpi = C::kRowsPerInstr;
        constexpr int kLsuRows = kKB - TMA_ROWS;
        constexpr int kRowsPerWarp = kLsuRows / kGW;
        static_assert(kLsuRows % (kGW * kRpi) == 0, "rows must split evenly over the gather warps");
        constexpr int kCopies = kRowsPerWarp / kRpi;
        const int chunk = lane % kLpr, sub = lane / kLpr;
        const int g = chunk >> 3, c = chunk & 7;
        const int m = d.m0 + chunk * 8;
        const bool m_ok = m < M;
        const uint16_t* src_col = At + (m_ok ? m : 0);
        const int row0 = TMA_ROWS + gw * kRowsPerWarp;
        int krow[kCopies];
#pragma unroll
        for (int e = 0; e < kCopies; ++e) {
          const int row = row0 + e * kRpi + sub;
          krow[e] = (row < nv) ? idx[row] + (rel >= 0 ? rel + row : 0) : 0;
        }
        const uint32_t dst0 = a_base + g * kALbo;
        const bool lane_live = chunk * 8 < m_len;           // columns past the unit are never read
        if (nv == kKB && d.m0 + m_len <= M) {
          if (lane_live) {
#pragma unroll
            for (int e = 0; e < kCopies; ++e) {
              const int row = row0 + e * kRpi + sub;
              cp_async_16_full(dst0 + (row >> 3) * kASbo + (row & 7) * 128 + ((c ^ (row & 7)) << 4),
                               src_col + static_cast<long long>(krow[e]) * lda);
            }
          }
        } else if (lane_live) {
#pragma unroll
          for (int e = 0; e < kCopies; ++e) {
            const int row = row0 + e * kRpi + sub;
            const bool valid = (row < nv) && m_ok;
            cp_async_16(dst0 + (row >> 3) * kASbo + (row & 7) * 128 + ((c ^ (row & 7)) << 4),
                        valid ? src_col + static_cast<long long>(krow[e]) * lda : At, valid ? 16u : 0u);
          }
        }
        cp_async_arrive_noinc(bar);
      }
      TS_TRACE(24 + (it < 4 ? it : 4), lane == 0 && gw == 0);
      if (j < 8) TS_TRACE(193 + j * 2, lane == 0 && gw == 0);
    }
    cp_async_wait_all();  // nothing of this thread is in flight when the CTA retires
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ epilogue
    constexpr int kGroups = MT / 128;            // 64-column groups per epilogue thread
    const int ew = warp - 6;                     // 0..7
    const int half = ew >> 2;                    // takes the 64-column groups half, half+2, ...
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int j = q * 32 + lane;                 // tile column owned by this thread
    const bool leader = (warp == 6 && lane == 0);
    uint32_t acc_it = 0;
    bool ok = true;
    grid_dependency_wait();   // Ct may still be read or written by the previous kernel
    for (int r = 0; ok && w.tile >= 0; ++r) {
      const WorkItem wn = fetch_item(sched, rounds, grid, cta, r + 1);
      const uint32_t a = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      const int m0 = w.m_begin;
      const int m_cnt = min(w.m_len, M - m0);
      const bool active = j < w.n_count;
      // TMA store: consecutive Ct rows, nothing to read back, no peer copies
      const bool tma_store = use_tma_store && (w.flags & kItemDenseRows) && beta == 0.0f && ep.n_peers == 0;
      const bool plain = beta == 0.0f && ep.bias == nullptr && ep.act == kActNone;
      const long long c_row = active ? c_row_of(w, j) : 0;
      const float bias_j = (ep.bias != nullptr && active) ? __ldg(ep.bias + c_row) : 0.0f;
      uint16_t* gdst = Ct + c_row * ldc + m0;
      ok = mbar_wait(smem_u32(&bars->acc_full[a]), aph, abort_flag);
      if (!ok) break;
      TS_TRACE(32, threadIdx.x == 192);
      TS_TRACE_U(3, acc_it, threadIdx.x == 192);
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + a * MT + (static_cast<uint32_t>(q * 32) << 16);
      const bool has_acc = w.k_count > 0;
      // TMEM is read one 64-column group (two 32-column reads, one wait) at a time: a read's latency
      // is far longer than the conversion of one chunk, so the two must overlap each other.
      constexpr int kBatch = 2;
#pragma unroll
      for (int gi = 0; gi < kGroups; ++gi) {
        const int grp_col = (gi * 2 + half) * 64;        // first batch column of this thread's group
        const bool grp_live = grp_col < m_cnt;           // uniform over the warp
        uint32_t v[kBatch][32];
        if (grp_live) {
          if (has_acc) {
#pragma unroll
            for (int b = 0; b < kBatch; ++b) tmem_ld_32x32(taddr + grp_col + b * 32, v[b]);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int b = 0; b < kBatch; ++b)
#pragma unroll
              for (int e = 0; e < 32; ++e) v[b][e] = 0u;
          }
        }
        if (gi == kGroups - 1) {
          // every TMEM read of this accumulator has completed: hand it back to the MMA warp
          tc_fence_before_sync();
          mbar_arrive(smem_u32(&bars->acc_empty[a]));
        }
        if (gi == 0) {
          // the staging tile is free once the previous unit's TMA store has read it (the leader
          // waits for that) and every thread has finished the previous copy-out
          if (leader) bulk_wait_read_all();
          named_barrier_sync(1, kEpiThreads);
        }
        if (!grp_live) continue;
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          const int col0 = grp_col + b * 32;             // first batch column of the chunk
          uint32_t(&cur)[32] = v[b];
          uint32_t o[16];
          if (plain && alpha == 1.0f) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              o[e] = pack2<DT>(__uint_as_float(cur[2 * e]), __uint_as_float(cur[2 * e + 1]));
            }
          } else if (plain) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              o[e] = pack2<DT>(alpha * __uint_as_float(cur[2 * e]),
                               alpha * __uint_as_float(cur[2 * e + 1]));
            }
          } else {
            // general form: alpha * x + beta * Ct_old + bias, then the activation
            const bool read_old = beta != 0.0f && active && (col0 < m_cnt);
            const uint4* cs = reinterpret_cast<const uint4*>(gdst + col0);
#pragma unroll
            for (int e4 = 0; e4 < 4; ++e4) {
              uint4 old = make_uint4(0, 0, 0, 0);
              if (read_old && col0 + e4 * 8 < m_cnt) old = cs[e4];
              const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float c0f = unpack1<DT>(static_cast<uint16_t>(ow[e] & 0xffffu));
                const float c1f = unpack1<DT>(static_cast<uint16_t>(ow[e] >> 16));
                const int idx = e4 * 8 + e * 2;
                const float y0 = alpha * __uint_as_float(cur[idx]) + beta * c0f + bias_j;
                const float y1 = alpha * __uint_as_float(cur[idx + 1]) + beta * c1f + bias_j;
                o[e4 * 4 + e] = pack2<DT>(apply_act(y0, ep.act), apply_act(y1, ep.act));
              }
            }
          }
          // staging: [64-column group][tile column j][128 bytes], 16-byte chunks swizzled by j & 7
          const int g16 = col0 >> 3;                     // first 16-byte chunk of these 32 columns
          uint8_t* grp = epi + (g16 >> 3) * C::kEpiGroupBytes + j * 128;
#pragma unroll
          for (int e4 = 0; e4 < 4; ++e4) {
            const int c = (g16 & 7) + e4;
            *reinterpret_cast<uint4*>(grp + ((c ^ (j & 7)) << 4)) =
                make_uint4(o[e4 * 4], o[e4 * 4 + 1], o[e4 * 4 + 2], o[e4 * 4 + 3]);
          }
        }
      }
      if (half == 0) bars->c_row[j] = active ? static_cast<int>(c_row) : -1;
      TS_TRACE(33, threadIdx.x == 192);
      TS_TRACE_U(4, acc_it, threadIdx.x == 192);
      if (tma_store) fence_proxy_async_smem();
      named_barrier_sync(1, kEpiThreads);       // all rows are staged
      TS_TRACE_U(5, acc_it, threadIdx.x == 192);
      if (tma_store) {
        if (leader) {
          const int row0 = w.c_row0 + (w.n_list ? __ldg(w.n_list) + 0 : 0);
#pragma unroll
          for (int mg = 0; mg < MT / 64; ++mg) {
            if (mg * 64 < m_cnt) {
              tma_store_2d(&tmap_c, smem_u32(epi + mg * C::kEpiGroupBytes), m0 + mg * 64, row0);
            }
          }
          bulk_commit();
        }
      } else {
        // copy-out through the kept-column list: 16 rows per warp, 16 bytes per lane
        constexpr int kLpr = C::kLanesPerRow, kRpi = C::kRowsPerInstr;
        const int chunk = lane % kLpr, sub = lane / kLpr;
        const bool m_ok = chunk * 8 < m_cnt;
#pragma unroll
        for (int r4 = 0; r4 < 16 / kRpi; r4 += 4) {
          // four rows per batch: shared-memory reads first, then the global stores
          int cr[4];
          uint4 val[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int row = ew * 16 + (r4 + e) * kRpi + sub;
            cr[e] = bars->c_row[row];
            val[e] = *reinterpret_cast<const uint4*>(epi + (chunk >> 3) * C::kEpiGroupBytes + row * 128 +
                                                     (((chunk & 7) ^ (row & 7)) << 4));
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (cr[e] >= 0 && m_ok) {
              const long long off = static_cast<long long>(cr[e]) * ldc + m0 + chunk * 8;
              *reinterpret_cast<uint4*>(Ct + off) = val[e];
              // tile-sharded layers: the same rows go to the other GPUs' copies of Ct over NVLink
              for (int p = 0; p < ep.n_peers; ++p) *reinterpret_cast<uint4*>(ep.peers[p] + off) = val[e];
            }
          }
        }
      }
      TS_TRACE_U(6, acc_it, threadIdx.x == 192);
      ++acc_it;
      w = wn;
    }
    if (leader) bulk_wait_all();                // the last TMA store has been written
    TS_TRACE(34, threadIdx.x == 192);
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
  if (threadIdx.x == 0 && bars->abort_flag) atomicExch(status, kErrTimeout);
  TS_TRACE(2, threadIdx.x == 0);
}

template <int DT, int MT, int TMA_ROWS>
cudaError_t launch_variant(const CUtensorMap& tmap_w, const CUtensorMap& tmap_a, const CUtensorMap& tmap_c,
                           int use_tma_store, int K_oob,
                           const WorkItem* sched, int rounds, int grid,
                           const BlockDesc* blocks, int blk_stride, const void* At, long long lda, void* Ct, long long ldc, int M,
                           const EpilogueArgs& ep, int* status, cudaStream_t stream) {
  // Programmatic dependent launch lets this kernel's set-up overlap the tail of the kernel before
  // it in the stream.  TS_PDL=0 turns it off.
  static const bool pdl = [] {
    const char* e = getenv("TS_PDL");
    return !(e && e[0] == '0');
  }();
  auto kern = masked_gemm_kernel<DT, MT, TMA_ROWS>;
  // The dynamic shared-memory limit is a per-device, per-kernel attribute: set it once for each.
  static bool attr_set[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 64 || !attr_set[dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<MT>::kSmemBytes);
    if (e != cudaSuccess) return e;
    if (dev < 64) attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = Cfg<MT>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, tmap_w, tmap_a, tmap_c, use_tma_store, sched, rounds, blocks, blk_stride,
                            K_oob, static_cast<const uint16_t*>(At), lda, static_cast<uint16_t*>(Ct), ldc, M,
                            ep, status);
}

}  // namespace

cudaError_t masked_gemm_launch(int dtype, int unit_rows, int tma_rows, const CUtensorMap& tmap_w,
                               const CUtensorMap* tmap_a, const CUtensorMap* tmap_c, int K_oob,
                               const WorkItem* sched, int rounds,
                               int grid, const BlockDesc* blocks, int blk_stride, const void* At,
                               long long lda, void* Ct, long long ldc, int M, const EpilogueArgs& ep,
                               int* status, cudaStream_t stream) {
  if (tma_rows > 0 && !tmap_a) return cudaErrorInvalidValue;
#define TS_LAUNCH(DT, MT, TR)                                                                        \
  launch_variant<DT, MT, TR>(tmap_w, TR > 0 ? *tmap_a : tmap_w, tmap_c ? *tmap_c : tmap_w,            \
                             tmap_c ? 1 : 0, K_oob, sched, rounds, grid, blocks,                      \
                             blk_stride, At, lda, Ct, ldc, M, ep, status, stream)
#define TS_BY_ROWS(DT, MT)                      \
  switch (tma_rows) {                           \
    case 0: return TS_LAUNCH(DT, MT, 0);        \
    case 64: return TS_LAUNCH(DT, MT, 64);      \
    default: return cudaErrorInvalidValue;      \
  }
  const bool bf = dtype == kBF16;
  if (unit_rows == 256) {
    if (bf) { TS_BY_ROWS(kBF16, 256) } else { TS_BY_ROWS(kF16, 256) }
  }
  if (unit_rows == 128) {
    if (bf) { TS_BY_ROWS(kBF16, 128) } else { TS_BY_ROWS(kF16, 128) }
  }
#undef TS_BY_ROWS
#undef TS_LAUNCH
  return cudaErrorInvalidValue;
}

#ifdef TS_KERNEL_TRACE
cudaError_t masked_gemm_read_trace(long long* out64, bool clear) {
  cudaError_t e = cudaMemcpyFromSymbol(out64, g_trace, sizeof(long long) * 256);
  if (e == cudaSuccess && clear) {
    long long z[256] = {};
    e = cudaMemcpyToSymbol(g_trace, z, sizeof(z));
  }
  return e;
}
#endif

}  // namespace ts

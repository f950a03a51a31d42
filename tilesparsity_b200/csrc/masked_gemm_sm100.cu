// Persistent grouped masked GEMM for tile-wise sparse weights (sm_100a: tcgen05 + TMEM + TMA).
//
// Replaces the reference's per-tile CUTLASS launches (one stream per column tile,
// StreamMaskedGEMM/perf/basic_nn.cu:378-445; kernel StreamMaskedGEMM/cutlass/gemm/gemm.h:45-61 with
// the masked A loads of cutlass/tile_iterator.h:786-816 and the masked stores of :1262-1292) by ONE
// launch over a work list.  Data layout is the reference's (column-major everywhere,
// basic_nn.cu:412-426):
//
//   At : activations, stored [K][lda] with the batch dimension M contiguous (column-major M x K);
//        the kernel only sees where each kept row starts (16-byte segment numbers in the block records),
//        which is how a convolution's shifted input planes stand in for an im2col matrix
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
// pattern (one kept row is one contiguous 2*MT-byte global segment).
//
// Pipeline: four stages of 64 kept rows (six for 128-row units).  The four gather warps fill every
// block together, a quarter of its rows each; all a warp needs to know about a block is one
// shared-memory record (descriptor + 64 resolved row numbers) that it prefetched by cp.async during
// the block before.  Each lane hands its copies to the stage's mbarrier with
// cp.async.mbarrier.arrive, so a stage is released to the MMA warp the moment its bytes have landed.  Accumulators live in TMEM, double buffered: the
// epilogue of one work unit overlaps the main loop of the next.  Eight epilogue warps (two per TMEM
// lane quarter; each half of them takes every other 64-column group of the unit) convert their rows
// to 16 bit into a 128-byte-swizzled 16 KiB staging group per half.  When the tile's kept columns
// are consecutive rows of Ct (no column pruning) a group leaves with one TMA store; otherwise each
// warp writes its 32 rows with 16-byte coalesced stores through the kept-column list.
//
// Warp roles (448 threads): warp 0 = weight TMA, warp 1 = TMEM allocation + MMA issue,
// warps 2-5 = activation gather, warps 6-13 = epilogue.  (Eight gather warps were measured: 18 warps
// leave 96 registers per thread, the kernel spills, and every workload got slower.)
#include "ts_common.cuh"
#include "ts_kernels.h"

namespace ts {

namespace {

constexpr int kNT = 128;                 // columns per tile (MMA M, TMEM lanes)
constexpr int kKB = 64;                  // kept rows per pipeline stage
constexpr int kWBytes = kNT * kKB * 2;   // 16 KiB of packed weights per stage
constexpr int kEpiThreads = 256;
constexpr uint32_t kASbo = 1024;         // bytes between 8-row K groups of the gathered operand
constexpr uint32_t kALbo = kKB * 128;    // bytes between its 64-column batch groups
constexpr uint32_t kWSbo = 1024;         // bytes between 8-row groups of the weight operand
constexpr int kMaxStages = 6;
#ifndef TS_GATHER_WARPS
#define TS_GATHER_WARPS 4
#endif
constexpr int kGW = TS_GATHER_WARPS;     // gather warps
constexpr int kEpiWarp0 = 2 + kGW;       // first epilogue warp
constexpr int kThreads = 32 * kEpiWarp0 + kEpiThreads;
// Gather warps that share one K block.  Measured on B200 with 1, 2 and 4: 4 is best or within 3 % of
// the best on every workload tried (1 loses up to 30 % where the activations stream from DRAM,
// because the blocks of different warps then land out of order and the MMA warp consumes them in
// order).  With fewer than 4 the per-warp record slices grow and the ring below must shrink to fit.
#ifndef TS_WARPS_PER_BLOCK
#define TS_WARPS_PER_BLOCK 4
#endif
constexpr int kWarpsPerBlock = TS_WARPS_PER_BLOCK;
constexpr int kWarpGroups = kGW / kWarpsPerBlock;    // group p of warps takes blocks p, p+kWarpGroups, ...
constexpr int kRowsPerWarp = kKB / kWarpsPerBlock;
constexpr int kMetaInts = kBlockMetaInts;  // one block record: {m0, meta, 0, 0} + 64 row numbers
constexpr int kAhead = 4;                // a warp requests its part of a record this many of its blocks ahead
constexpr int kMetaSlots = 6;            // ring slots per warp (> kAhead)

struct Barriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  // Per gather warp: ring of the parts of the coming blocks' records that the warp needs: the
  // descriptor words and the row numbers of its slice.
  alignas(16) int meta_ring[kGW][kMetaSlots][4 + kRowsPerWarp];
};

// Compile-time shape of one kernel variant: MT batch rows per work unit.
template <int MT>
struct Cfg {
  // As many stages as fit beside the staging groups in 227 KiB.  A warp group must never run two
  // phases of one stage ahead of the MMA warp (the parity wait could not tell them apart), which
  // holds as long as there are at least as many stages as warp groups.
  static constexpr int kStages = MT == 256 ? 4 : 6;
  static_assert(kStages <= kMaxStages && kStages >= kWarpGroups, "stage count");
  static constexpr int kABytes = kKB * MT * 2;
  static constexpr int kStageBytes = kWBytes + kABytes;
  static constexpr int kEpiGroupBytes = kNT * 128;   // staging: one 128-row x 64-column swizzled group
  static constexpr int kEpiBytes = 2 * kEpiGroupBytes;  // one group per half of the epilogue warps
  static constexpr int kTmemCols = 2 * MT;          // two accumulators of MT fp32 columns
  // stages + staging + barriers/records + what the 1024-byte alignment of the first stage may skip
  static constexpr int kUsedBytes = kStages * kStageBytes + kEpiBytes + static_cast<int>(sizeof(Barriers));
  static constexpr int kSmemBytes = (kUsedBytes + 1023 + 1023) / 1024 * 1024 > 232448 ? 232448
                                                                                      : (kUsedBytes + 1023 + 1023) / 1024 * 1024;
  static_assert(kUsedBytes <= kSmemBytes, "stages, staging and barriers exceed the shared memory of one CTA");
  static constexpr int kLanesPerRow = MT / 8;       // 16-byte chunks in one gathered row
  static constexpr int kRowsPerInstr = 32 / kLanesPerRow;
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

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
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

// MODE selects what the epilogue can do: kModeLean only alpha * acc through TMA tile stores (the host
// picks it when beta == 0, there is no bias or activation and every scheduled tile keeps 128 consecutive
// columns), kModePlain every epilogue form and the list-driven stores, kModeSplit in addition the fp32
// partial sums of split-K parts, kModePeers the copies for the other GPUs of a tile-sharded layer.
// Code a call cannot reach stays out of the variant it runs; measured on the BERT layer step (39.6 us):
// the split-K code inside the common kernel +1.3 %, the peers' TMA stores +3.3 %, and the lean variant
// against the plain one -3 %.
constexpr int kModePlain = 0, kModeSplit = 1, kModePeers = 2, kModeLean = 3;
template <int DT, int MT, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
masked_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w,
                   const __grid_constant__ CUtensorMap tmap_c, int use_tma_store,
                   const WorkItem* __restrict__ sched, int rounds,
                   const int* __restrict__ block_meta, int blk_stride,
                   const uint16_t* __restrict__ At, long long lda,
                   uint16_t* __restrict__ Ct, long long ldc, int M, const __grid_constant__ EpilogueArgs ep,
                   int* __restrict__ status) {
  const float alpha = ep.alpha, beta = ep.beta;
  constexpr bool SPLIT = MODE == kModeSplit, PEERS = MODE == kModePeers, LEAN = MODE == kModeLean;
  using C = Cfg<MT>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the swizzle pattern is a function of the shared-memory address bits.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  if (static_cast<int>(smem - smem_raw) + C::kUsedBytes > C::kSmemBytes) {
    // the dynamic shared-memory window starts at an address this layout was not sized for
    if (threadIdx.x == 0) atomicExch(status, kErrUnsupported);
    return;
  }
  uint8_t* epi = smem + kStages * C::kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(epi + C::kEpiBytes);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int grid = gridDim.x;
  const int cta = blockIdx.x;

  // First work item, and for the gather warps the record of their first block: requested before
  // the set-up below so their latency overlaps it.  The schedule is static data.
  WorkItem w = fetch_item(sched, rounds, grid, cta, 0);
  const int gw = warp - 2;                                  // gather warp number (warps 2..5)
  const int* recs = block_meta + static_cast<size_t>(cta) * blk_stride * kMetaInts;
  // lanes 0..: one 16-byte piece each: the descriptor, then the warp's slice of the row numbers
  const int meta_piece = lane == 0 ? 0 : 4 + (gw % kWarpsPerBlock) * kRowsPerWarp + (lane - 1) * 4;
  constexpr int kMetaLanes = 1 + kRowsPerWarp / 4;
  if (warp >= 2 && warp < kEpiWarp0) {
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      if (lane < kMetaLanes) {
        cp_async_16_ca(smem_u32(&bars->meta_ring[gw][i][lane * 4]),
                       recs + static_cast<size_t>(gw / kWarpsPerBlock + i * kWarpGroups) * kMetaInts + meta_piece);
      }
      cp_async_commit();
    }
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      // weight TMA thread + the cp.async lanes of the warps that fill the stage
      mbar_init(smem_u32(&bars->full[s]), 1 + 32 * kWarpsPerBlock);
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
          // (a split-K part starts at K block flags >> 8 of its tile's packed weights)
          const int kb_first = SPLIT ? static_cast<int>(static_cast<uint32_t>(w.flags) >> kItemKb0Shift) : 0;
          tma_load_2d(smem_u32(smem + s * C::kStageBytes), &tmap_w, (kb + kb_first) * kKB, w.w_row0, bar);
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
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + a * MT;
      const uint32_t idesc = idesc0 | (static_cast<uint32_t>(w.m_len >> 3) << 17);
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const uint32_t s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        ok = mbar_wait(smem_u32(&bars->full[s]), ph, abort_flag);
        if (!ok) break;
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
      ++acc_it;
      w = wn;
    }
  } else if (warp < kEpiWarp0) {
    // ------------------------------------------------------------------ activation gather
    // kWarpsPerBlock warps share one block (a slice of its rows each); group p of warps takes the
    // blocks p, p+kWarpGroups, ... of the CTA's stream, block j lives in stage j % kStages.  Per block: wait
    // for its record (requested kAhead blocks earlier), wait for the stage, issue the
    // warp's rows in one burst (row numbers read from the record into registers first: a
    // shared-memory read between two copies stalls the warp until the load/store unit has taken the
    // copies before it), hand the copies to the stage's barrier.  One cp.async group is committed
    // per block, made of the block's row copies and the request for the record kAhead blocks on;
    // "all but the latest kAhead - 1 groups have completed" therefore says that this block's
    // record has landed while the rows of the kAhead - 1 blocks before it may still be in flight.
    constexpr int kLpr = C::kLanesPerRow, kRpi = C::kRowsPerInstr;
    const int chunk = lane % kLpr, sub = lane / kLpr;
    const int g = chunk >> 3, c = chunk & 7;
    const int grp = gw / kWarpsPerBlock;                    // group of warps this warp belongs to
    const int row_base = (gw % kWarpsPerBlock) * kRowsPerWarp;   // first row of the warp's slice
    // The schedule is static; the activations may be the previous kernel's output: wait for it
    // before the first row is copied.
    grid_dependency_wait();

    for (uint32_t it = 0;; ++it) {
      const int j = grp + static_cast<int>(it) * kWarpGroups;
      cp_async_wait_group<kAhead - 1>();
      __syncwarp();
      const int* rec = bars->meta_ring[gw][it % kMetaSlots];
      const int m0 = rec[0];
      const uint32_t meta = static_cast<uint32_t>(rec[1]);
      if (meta == kBlockEnd) break;
      const int nv = static_cast<int>(meta & 0x7fu);
      const int m_len = (static_cast<int>((meta >> 8) & 3u) + 1) * 64;          // batch rows of the unit
      const int m = m0 + chunk * 8;
      const bool m_ok = m < M;
      const uint16_t* src_col = At + (m_ok ? m : 0);
      const bool lane_live = chunk * 8 < m_len;             // columns past the unit are never read
      const bool full_block = nv == kKB && m0 + m_len <= M;
      const uint32_t s = static_cast<uint32_t>(j) % kStages;
      const uint32_t ph = (static_cast<uint32_t>(j) / kStages) & 1u;
      const uint32_t dst0 = smem_u32(smem + s * C::kStageBytes + kWBytes) + g * kALbo;
      const uint32_t bar = smem_u32(&bars->full[s]);
      if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag)) break;
      int rr[kRowsPerWarp];
#pragma unroll
      for (int q4 = 0; q4 < kRowsPerWarp / 4; ++q4) {
        const int4 v = reinterpret_cast<const int4*>(rec + 4)[q4];
        rr[q4 * 4] = v.x;
        rr[q4 * 4 + 1] = v.y;
        rr[q4 * 4 + 2] = v.z;
        rr[q4 * 4 + 3] = v.w;
      }
      // Two separate bursts: mixing the zero-fill form into the loop of plain copies makes every
      // copy as slow as the zero-fill form.
      if (full_block) {
        if (lane_live) {
#pragma unroll
          for (int e = 0; e < kRowsPerWarp / kRpi; ++e) {
            const int row = row_base + e * kRpi + sub;
            int kr;
            if constexpr (kRpi == 1) {
              kr = rr[e];
            } else {
              kr = sub ? rr[e * 2 + 1] : rr[e * 2];
            }
            cp_async_16_full(dst0 + (row >> 3) * kASbo + (row & 7) * 128 + ((c ^ (row & 7)) << 4),
                             src_col + (static_cast<long long>(kr) << 3));
          }
        }
      } else if (lane_live) {
#pragma unroll
        for (int e = 0; e < kRowsPerWarp / kRpi; ++e) {
          const int row = row_base + e * kRpi + sub;
          int kr;
          if constexpr (kRpi == 1) {
            kr = rr[e];
          } else {
            kr = sub ? rr[e * 2 + 1] : rr[e * 2];
          }
          const bool valid = (row < nv) && m_ok;
          cp_async_16(dst0 + (row >> 3) * kASbo + (row & 7) * 128 + ((c ^ (row & 7)) << 4),
                      valid ? src_col + (static_cast<long long>(kr) << 3) : At, valid ? 16u : 0u);
        }
      }
      cp_async_arrive_noinc(bar);
      // request the warp's part of the record kAhead of its blocks ahead; one group per block
      if (lane < kMetaLanes) {
        cp_async_16_ca(smem_u32(&bars->meta_ring[gw][(it + kAhead) % kMetaSlots][lane * 4]),
                       recs + static_cast<size_t>(j + kAhead * kWarpGroups) * kMetaInts + meta_piece);
      }
      cp_async_commit();
    }
    cp_async_wait_all();  // nothing of this thread is in flight when the CTA retires
  } else if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------------ epilogue
    constexpr int kGroups = MT / 128;            // 64-column groups per epilogue thread
    const int ew = warp - kEpiWarp0;             // 0..7
    const int half = ew >> 2;                    // takes the 64-column groups half, half+2, ...
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int j = q * 32 + lane;                 // tile column owned by this thread
    const bool leader = ((ew & 3) == 0 && lane == 0);   // one per half
    const int half_bar = 1 + half;               // named barrier of this half (128 threads)
    const int peer_rot = (PEERS && ep.n_peers > 0) ? cta % ep.n_peers : 0;   // the peer this CTA writes first
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
      // TMA store of the local copy: consecutive Ct rows, nothing to read back
      const bool tma_store = LEAN || (use_tma_store && (w.flags & kItemDenseRows) && beta == 0.0f &&
                                      (!PEERS || ep.multicast == nullptr));
      const bool tma_peers = PEERS && tma_store && ep.peer_maps != nullptr;   // the peers' copies leave by TMA too
      // The CTA's last unit: every K block has been consumed, so the pipeline stages are free and
      // each 64-column group gets a staging group of its own there; no group waits for the store
      // of the one before it.
      const bool last_unit = wn.tile < 0;
      const bool plain = LEAN || (beta == 0.0f && ep.bias == nullptr && ep.act == kActNone);
      const long long c_row = active ? c_row_of(w, j) : 0;
      const int c_row_or_none = active ? static_cast<int>(c_row) : -1;
      const float bias_j = (ep.bias != nullptr && active) ? __ldg(ep.bias + c_row) : 0.0f;
      uint16_t* gdst = Ct + c_row * ldc + m0;
      const int tile_row0 = w.c_row0 + ((tma_store && w.n_list) ? __ldg(w.n_list) : 0);
      ok = mbar_wait(smem_u32(&bars->acc_full[a]), aph, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + a * MT + (static_cast<uint32_t>(q * 32) << 16);
      const bool has_acc = w.k_count > 0;
      // TMEM is read one 64-column group (two 32-column reads, one wait) at a time: a read's latency
      // is far longer than the conversion of one chunk, so the two must overlap each other.
      constexpr int kBatch = 2;
      // Not unrolled: the epilogue's hot code stays small enough for the instruction cache it
      // shares with the other roles (-3 % on the BERT layer).
#pragma unroll 1
      for (int gi = 0; gi < kGroups; ++gi) {
        const int grp_col = (gi * 2 + half) * 64;        // first batch column of this thread's group
        const bool grp_live = grp_col < m_cnt;           // uniform over the half
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
        if (!grp_live) continue;
        if constexpr (SPLIT) if (w.flags & kItemScratch) {
          // split-K part: alpha * acc leaves as fp32 for the part's 128 scratch rows.  32 fp32 columns
          // fill one 128-row x 128-byte staging group, which goes out as one TMA tile store; bias, beta
          // and the activation are applied by the kernel that adds the parts up.  (Tile columns past
          // n_count carry zero weights, so their rows receive zeros.)
          uint8_t* stage = epi + half * C::kEpiGroupBytes;
#pragma unroll
          for (int b = 0; b < kBatch; ++b) {
            if (grp_col + b * 32 >= m_cnt) break;              // uniform over the half
            if (leader) bulk_wait_read_all();
            named_barrier_sync(half_bar, 128);
            uint8_t* row_ptr = stage + j * 128;
#pragma unroll
            for (int cc = 0; cc < 8; ++cc) {
              *reinterpret_cast<float4*>(row_ptr + ((cc ^ (j & 7)) << 4)) =
                  make_float4(alpha * __uint_as_float(v[b][cc * 4]), alpha * __uint_as_float(v[b][cc * 4 + 1]),
                              alpha * __uint_as_float(v[b][cc * 4 + 2]), alpha * __uint_as_float(v[b][cc * 4 + 3]));
            }
            fence_proxy_async_smem();
            named_barrier_sync(half_bar, 128);
            if (leader) {
              tma_store_2d(ep.scratch_map, smem_u32(stage), m0 + grp_col + b * 32, w.c_row0);
              bulk_commit();
            }
          }
          continue;
        }
        uint8_t* stage_grp = last_unit ? smem + (half * kGroups + gi) * C::kEpiGroupBytes
                                       : epi + half * C::kEpiGroupBytes;
        if (!last_unit) {
          // The half's staging group is free once its previous TMA store has read it (the leader
          // waits for that) and every warp of the half has finished its previous copy-out.
          if (leader) bulk_wait_read_all();
          named_barrier_sync(half_bar, 128);
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          const int col0 = grp_col + b * 32;             // first batch column of the chunk
          uint32_t(&cur)[32] = v[b];
          uint32_t o[16];
          if (plain) {
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
          // staging: [tile column j][128 bytes], 16-byte chunks swizzled by j & 7
          uint8_t* row_ptr = stage_grp + j * 128;
#pragma unroll
          for (int e4 = 0; e4 < 4; ++e4) {
            const int cc = b * 4 + e4;
            *reinterpret_cast<uint4*>(row_ptr + ((cc ^ (j & 7)) << 4)) =
                make_uint4(o[e4 * 4], o[e4 * 4 + 1], o[e4 * 4 + 2], o[e4 * 4 + 3]);
          }
        }
        if (tma_store) {
          fence_proxy_async_smem();
          named_barrier_sync(half_bar, 128);     // the whole group is staged
          if (leader) {
            tma_store_2d(&tmap_c, smem_u32(stage_grp), m0 + grp_col, tile_row0);
            if constexpr (PEERS) if (tma_peers) {
              for (int p = 0; p < ep.n_peers; ++p) {
                int pp = p + peer_rot;
                if (pp >= ep.n_peers) pp -= ep.n_peers;
                tma_store_2d(ep.peer_maps + pp, smem_u32(stage_grp), m0 + grp_col, tile_row0);
              }
            }
            bulk_commit();
          }
        }
        if (!tma_store || (PEERS && ep.n_peers > 0 && !tma_peers)) {
          // copy-out through the kept-column list: this warp's own 32 rows, four rows per
          // instruction, 16 bytes per lane; to Ct unless the TMA store took it, and to every peer.
          // Tile-sharded layers: the peers are the other GPUs' copies of Ct, written over NVLink;
          // CTAs start at different peers so that the GPUs' stores do not converge on one
          // destination at a time.
          __syncwarp();
          const int cchunk = lane & 7, rsub = lane >> 3;
          const bool m_ok = grp_col + cchunk * 8 < m_cnt;
#pragma unroll
          for (int r4 = 0; r4 < 32; r4 += 16) {
            int cr[4];
            uint4 val[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int lrow = r4 + e * 4 + rsub;           // row inside the warp's quarter
              const int row = q * 32 + lrow;
              cr[e] = __shfl_sync(0xffffffffu, c_row_or_none, lrow);
              val[e] = *reinterpret_cast<const uint4*>(stage_grp + row * 128 + ((cchunk ^ (row & 7)) << 4));
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (cr[e] >= 0 && m_ok) {
                const long long off = static_cast<long long>(cr[e]) * ldc + m0 + grp_col + cchunk * 8;
                if constexpr (PEERS) {
                  if (ep.multicast != nullptr) {
                    multimem_st_16(ep.multicast + off, val[e]);     // every GPU's copy, this one included
                    continue;
                  }
                }
                if (!tma_store) *reinterpret_cast<uint4*>(Ct + off) = val[e];
                if constexpr (PEERS) {
                  for (int p = 0; p < ep.n_peers; ++p) {
                    int pp = p + peer_rot;
                    if (pp >= ep.n_peers) pp -= ep.n_peers;
                    *reinterpret_cast<uint4*>(ep.peers[pp] + off) = val[e];
                  }
                }
              }
            }
          }
          __syncwarp();
        }
      }
      ++acc_it;
      w = wn;
    }
    // The CTA may retire once its last TMA stores have read the staging groups; the stores
    // themselves complete before the grid does.
    if (leader) bulk_wait_read_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
  if (threadIdx.x == 0 && bars->abort_flag) atomicExch(status, kErrTimeout);
}

// One record per K block of a schedule: {first batch row of the unit, meta word, 0, 0} followed by
// the start of the 64 rows the block gathers (0 past the block's last row), each as a count of
// 16-byte segments from the activation base pointer.  For a matrix At[K][lda] kept row k starts at
// segment k * lda / 8.  For a convolution the "matrix" is never materialised: kept row
// k = (r * kw + j) * cin + c of the im2col matrix (Pruning/VGG/prune_algo.py:16-24 fixes that order)
// is channel c of the copy of the padded input shifted by j pixels, read r image rows further down:
// segment ((j * cin + c) * plane_ld + r * Wp) / 8.  The kept row number itself comes from the tile's
// list, or list position + offset for lists in the reference's relative form.
__global__ void __launch_bounds__(256)
expand_block_meta_kernel(const BlockDesc* __restrict__ blocks, long long n_blocks, int* __restrict__ meta,
                         const RowMap map) {
  const long long b = blockIdx.x * 4LL + (threadIdx.x >> 6);
  const int r = threadIdx.x & 63;
  if (b >= n_blocks) return;
  const BlockDesc d = blocks[b];
  int v = 0;
  if (d.meta != kBlockEnd && r < static_cast<int>(d.meta & 0x7fu)) {
    v = __ldg(d.idx + r);
    if (d.meta & 0x80u) v += static_cast<int>(d.meta >> 10) + r;
    if (map.conv_cin > 0) {
      const int c = v % map.conv_cin, rj = v / map.conv_cin;
      const int j = rj % map.conv_kw, rr = rj / map.conv_kw;
      v = static_cast<int>((static_cast<long long>(j) * map.conv_cin + c) * map.ld8 + static_cast<long long>(rr) * map.conv_wp8);
    } else {
      v = static_cast<int>(static_cast<long long>(v) * map.ld8);
    }
  }
  int* rec = meta + b * kMetaInts;
  rec[4 + r] = v;
  if (r < 4) rec[r] = r == 0 ? d.m0 : (r == 1 ? static_cast<int>(d.meta) : 0);
}

// Second pass of a split-K schedule: Ct[row][m] = act(sum of the parts' fp32 partial sums + beta * Ct[row][m]
// + bias[row]) for every kept column of every split tile.  grid (ceil(M / 8 / 256), 128, split tiles).
template <int DT>
__global__ void __launch_bounds__(256)
split_reduce_kernel(const SplitTile* __restrict__ tiles, const float* __restrict__ scratch, long long sld,
                    uint16_t* __restrict__ Ct, long long ldc, int M, float beta, const float* __restrict__ bias,
                    int act) {
  const SplitTile t = tiles[blockIdx.z];
  const int j = blockIdx.y;
  const int m = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (j >= t.n_count || m >= M) return;
  const long long row = t.c_row0 + (t.n_list ? __ldg(t.n_list + j) + (t.relative ? j : 0) : j);
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
  for (int p = 0; p < t.parts; ++p) {
    const float4* src = reinterpret_cast<const float4*>(scratch + (static_cast<long long>(t.scratch_row0) + p * 128 + j) * sld + m);
    const float4 a = src[0], b = src[1];
    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
    acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
  }
  uint4* dst = reinterpret_cast<uint4*>(Ct + row * ldc + m);
  uint32_t oldw[4] = {0, 0, 0, 0};
  if (beta != 0.0f) {
    const uint4 o = *dst;
    oldw[0] = o.x; oldw[1] = o.y; oldw[2] = o.z; oldw[3] = o.w;
  }
  const float bj = bias ? __ldg(bias + row) : 0.0f;
  uint32_t out[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float c0 = unpack1<DT>(static_cast<uint16_t>(oldw[e] & 0xffffu));
    const float c1 = unpack1<DT>(static_cast<uint16_t>(oldw[e] >> 16));
    const float y0 = acc[2 * e] + beta * c0 + bj;
    const float y1 = acc[2 * e + 1] + beta * c1 + bj;
    out[e] = pack2<DT>(apply_act(y0, act), apply_act(y1, act));
  }
  *dst = make_uint4(out[0], out[1], out[2], out[3]);
}

template <int DT, int MT, int MODE>
cudaError_t launch_variant(const CUtensorMap& tmap_w, const CUtensorMap& tmap_c, int use_tma_store,
                           const WorkItem* sched, int rounds, int grid, const int* block_meta, int blk_stride,
                           const void* At, long long lda, void* Ct, long long ldc, int M,
                           const EpilogueArgs& ep, int* status, bool early_start, cudaStream_t stream) {
  // Programmatic dependent launch lets this kernel's set-up overlap the tail of the kernel before
  // it in the stream.  The kernel reads its schedule and its packed weights before it waits for that
  // kernel, so the caller allows this only when neither was written by it.
  const bool pdl = early_start;
  auto kern = masked_gemm_kernel<DT, MT, MODE>;
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
  return cudaLaunchKernelEx(&cfg, kern, tmap_w, tmap_c, use_tma_store, sched, rounds, block_meta, blk_stride,
                            static_cast<const uint16_t*>(At), lda, static_cast<uint16_t*>(Ct), ldc, M,
                            ep, status);
}

}  // namespace

cudaError_t masked_gemm_launch(int dtype, int unit_rows, const CUtensorMap& tmap_w, const CUtensorMap* tmap_c,
                               const WorkItem* sched, int rounds, int grid, const int* block_meta,
                               int blk_stride, const void* At, long long lda, void* Ct, long long ldc, int M,
                               const EpilogueArgs& ep, int* status, bool early_start, bool lean,
                               cudaStream_t stream) {
#define TS_LAUNCH(DT, MT, MD)                                                                                  \
  launch_variant<DT, MT, MD>(tmap_w, tmap_c ? *tmap_c : tmap_w, tmap_c ? 1 : 0, sched, rounds, grid, block_meta, \
                             blk_stride, At, lda, Ct, ldc, M, ep, status, early_start, stream)
#define TS_LAUNCH_DT(MT, MD) (dtype == kBF16 ? TS_LAUNCH(kBF16, MT, MD) : TS_LAUNCH(kF16, MT, MD))
  if (unit_rows != 256 && unit_rows != 128) return cudaErrorInvalidValue;
  // a schedule with split-K parts never writes peers (the host keeps the two apart)
  if (ep.scratch_map != nullptr) return unit_rows == 256 ? TS_LAUNCH_DT(256, kModeSplit) : TS_LAUNCH_DT(128, kModeSplit);
  if (ep.n_peers > 0 || ep.multicast != nullptr) {
    return unit_rows == 256 ? TS_LAUNCH_DT(256, kModePeers) : TS_LAUNCH_DT(128, kModePeers);
  }
  // lean: the caller has checked that every unit takes the TMA store and that the epilogue is alpha * acc
  if (lean && tmap_c != nullptr && ep.beta == 0.0f && ep.bias == nullptr && ep.act == kActNone) {
    return unit_rows == 256 ? TS_LAUNCH_DT(256, kModeLean) : TS_LAUNCH_DT(128, kModeLean);
  }
  return unit_rows == 256 ? TS_LAUNCH_DT(256, kModePlain) : TS_LAUNCH_DT(128, kModePlain);
#undef TS_LAUNCH_DT
#undef TS_LAUNCH
  return cudaErrorInvalidValue;
}

cudaError_t split_reduce_launch(int dtype, const SplitTile* tiles, int n_split, const float* scratch, long long sld,
                                void* Ct, long long ldc, int M, float beta, const float* bias, int act,
                                cudaStream_t stream) {
  if (n_split <= 0 || M <= 0) return cudaSuccess;
  dim3 grid(static_cast<unsigned>((M / 8 + 255) / 256), 128, n_split);
  if (dtype == kBF16) {
    split_reduce_kernel<kBF16><<<grid, 256, 0, stream>>>(tiles, scratch, sld, static_cast<uint16_t*>(Ct), ldc, M, beta, bias, act);
  } else {
    split_reduce_kernel<kF16><<<grid, 256, 0, stream>>>(tiles, scratch, sld, static_cast<uint16_t*>(Ct), ldc, M, beta, bias, act);
  }
  return cudaGetLastError();
}

cudaError_t expand_block_meta_launch(const BlockDesc* blocks, long long n_blocks, int* meta, const RowMap& map,
                                     cudaStream_t stream) {
  if (n_blocks <= 0) return cudaSuccess;
  expand_block_meta_kernel<<<static_cast<unsigned>((n_blocks + 3) / 4), 256, 0, stream>>>(blocks, n_blocks, meta, map);
  return cudaGetLastError();
}

}  // namespace ts

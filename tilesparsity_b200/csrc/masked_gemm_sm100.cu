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
// pattern (one kept row is one contiguous 2*MT-byte global segment).  The gather warps (four, or
// three when only three stages fit) take the 64-row K blocks round-robin, one whole pipeline stage
// each, so several stages fill concurrently and a warp's kept-row indices are fetched a full turn
// ahead; each lane
// hands its copies to the stage's mbarrier with cp.async.mbarrier.arrive, so a stage is released to
// the MMA warp the moment its bytes have landed.  Accumulators live in TMEM, double buffered: the
// epilogue of one work unit overlaps the main loop of the next.  The epilogue thread that owns TMEM
// lane j converts its row to 16 bit in shared memory; the four epilogue warps then write the rows
// to Ct with 16-byte coalesced stores (an output row of a unit is one contiguous global segment).
//
// Warp roles (320 threads): warp 0 = weight TMA, warp 1 = TMEM allocation + MMA issue,
// warps 2-5 = activation gather (warp 5 idles in the three-stage variant), warps 6-9 = epilogue.
#include "ts_common.cuh"
#include "ts_kernels.h"

namespace ts {

namespace {

constexpr int kNT = 128;                 // columns per tile (MMA M, TMEM lanes)
constexpr int kKB = 64;                  // kept rows per pipeline stage
constexpr int kWBytes = kNT * kKB * 2;   // 16 KiB of packed weights per stage
constexpr int kThreads = 320;
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
  static constexpr int kEpiRowBytes = MT * 2 + 16;  // +16: rows start in distinct bank groups
  static constexpr int kEpiBytes = kNT * kEpiRowBytes;
  static constexpr int kTmemCols = 2 * MT;          // two accumulators of MT fp32 columns
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 6144 + 1024;
  // Gather warps take K blocks round-robin; a warp must never be more than one barrier phase
  // ahead of the MMA warp (a parity wait cannot tell phase n from phase n+2), so its stride may
  // not exceed the number of stages.
  static constexpr int kGatherWarps = kStages < 4 ? kStages : 4;
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
  w.k_count = w.n_count = w.w_row0 = w.c_row0 = w.relative = w.mblock = 0;
  w.tile = -1;
  w.pad_ = 0;
  return w;
}

__device__ __forceinline__ int k_blocks(const WorkItem& w) { return (w.k_count + kKB - 1) / kKB; }

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int DT, int MT>
__global__ void __launch_bounds__(kThreads, 1)
masked_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const WorkItem* __restrict__ sched,
                   int rounds, const BlockDesc* __restrict__ blocks, int blk_stride,
                   const uint16_t* __restrict__ At, long long lda,
                   uint16_t* __restrict__ Ct, long long ldc, int M, float alpha, float beta,
                   int* __restrict__ status) {
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
      mbar_init(smem_u32(&bars->full[s]), 32 + 1);   // one gather warp + the TMA thread
      mbar_init(smem_u32(&bars->empty[s]), 1);       // one tcgen05.commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bars->acc_full[a]), 1);
      mbar_init(smem_u32(&bars->acc_empty[a]), 128);
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
    constexpr uint32_t idesc = umma_idesc_f16(DT == kBF16 ? 1 : 0, /*a_mn=*/0, /*b_mn=*/1, kNT, MT);
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
  } else if (warp < 2 + C::kGatherWarps) {
    // ------------------------------------------------------------------ activation gather
    // This warp takes blocks gw, gw+kGW, gw+2*kGW, ... of the CTA's block stream; "j" counts its
    // own blocks.  Everything it needs arrives by cp.async, requested ahead of use: the descriptor
    // of block j+4 and the kept-row indices of block j+2 are requested while block j is copied, so
    // no step of the loop waits on a dependent global read.
    constexpr int kGW = C::kGatherWarps;
    const int gw = warp - 2;
    const int chunk = lane % C::kLanesPerRow;      // 16-byte chunk of the row this lane copies
    const int sub = lane / C::kLanesPerRow;        // row of the instruction this lane copies
    const int g = chunk >> 3;                      // 64-column batch group of the chunk
    const int c = chunk & 7;                       // chunk inside the 128-byte swizzled row
    const BlockDesc* bd = blocks + static_cast<size_t>(cta) * blk_stride + gw;  // stride kGW
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
    if (lane < 4) dring[lane] = bd[static_cast<size_t>(lane) * kGW];
    __syncwarp();
    request_indices(0);
    cp_async_commit();
    request_indices(1);
    cp_async_commit();

    bool ok = true;
    for (int j = 0; ok; ++j) {
      cp_async_wait_group<1>();   // indices of block j and descriptor of block j+2 have landed
      __syncwarp();
      const BlockDesc d = dring[j & 7];
      if (d.meta == kBlockEnd) break;
      request_indices(j + 2);
      if (lane == 0) cp_async_16_ca(smem_u32(&dring[(j + 4) & 7]), bd + static_cast<size_t>(j + 4) * kGW);
      cp_async_commit();

      const uint32_t it = static_cast<uint32_t>(gw + j * kGW);
      const uint32_t s = it % kStages;
      const uint32_t ph = (it / kStages) & 1u;
      if (j < 8) TS_TRACE(208 + j, lane == 0 && gw == 0);
      ok = mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag);
      if (!ok) break;
      if (j < 8) TS_TRACE(192 + j * 2, lane == 0 && gw == 0);
      const int nv = static_cast<int>(d.meta & 0x7fu);
      const int rel = (d.meta & 0x80u) ? static_cast<int>(d.meta >> 8) : -1;  // list position, if relative
      const int m = d.m0 + chunk * 8;
      const bool m_ok = m < M;
      const uint16_t* src_col = At + (m_ok ? m : 0);
      const int* idx = iring[j & 3];
      const uint32_t a_stage = smem_u32(smem + s * C::kStageBytes + kWBytes);
      constexpr int kRpi = C::kRowsPerInstr;
      constexpr int kCopies = kKB / kRpi;                     // copies per lane and block
      // Every kept-row index this lane needs is read into registers before the first copy goes
      // out: a shared-memory read between two copies would serialise the whole block.
      long long krow[kCopies];
#pragma unroll
      for (int e = 0; e < kCopies; ++e) {
        const int row = e * kRpi + sub;
        krow[e] = (row < nv) ? idx[row] + (rel >= 0 ? rel + row : 0) : 0;
      }
      const uint32_t dst0 = a_stage + g * kALbo;
      if (nv == kKB && d.m0 + MT <= M) {
        // interior block: every row and every batch column is valid
#pragma unroll
        for (int e = 0; e < kCopies; ++e) {
          const int row = e * kRpi + sub;
          cp_async_16_full(dst0 + (row >> 3) * kASbo + (row & 7) * 128 + ((c ^ (row & 7)) << 4),
                           src_col + krow[e] * lda);
        }
      } else {
        // ragged block: rows past the list and columns past M are zero-filled
#pragma unroll
        for (int e = 0; e < kCopies; ++e) {
          const int row = e * kRpi + sub;
          const bool valid = (row < nv) && m_ok;
          cp_async_16(dst0 + (row >> 3) * kASbo + (row & 7) * 128 + ((c ^ (row & 7)) << 4),
                      valid ? src_col + krow[e] * lda : At, valid ? 16u : 0u);
        }
      }
      cp_async_arrive_noinc(smem_u32(&bars->full[s]));
      TS_TRACE(24 + (it < 4 ? it : 4), lane == 0);
      if (j < 8) TS_TRACE(193 + j * 2, lane == 0 && gw == 0);
    }
    cp_async_wait_all();  // nothing of this thread is in flight when the CTA retires
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ epilogue
    constexpr int kChunks = MT / 32;
    const int q = warp & 3;             // TMEM lane quarter this warp may read
    const int j = q * 32 + lane;        // tile column owned by this thread
    uint8_t* my_row = epi + j * C::kEpiRowBytes;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int r = 0; ok && w.tile >= 0; ++r) {
      const WorkItem wn = fetch_item(sched, rounds, grid, cta, r + 1);
      const uint32_t a = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      const int m0 = w.mblock * MT;
      const int m_cnt = min(MT, M - m0);
      const bool active = j < w.n_count;
      long long c_row = 0;
      if (active) {
        c_row = w.c_row0 + (w.n_list ? __ldg(w.n_list + j) + (w.relative ? j : 0) : j);
      }
      uint16_t* gdst = Ct + c_row * ldc + m0;
      ok = mbar_wait(smem_u32(&bars->acc_full[a]), aph, abort_flag);
      if (!ok) break;
      TS_TRACE(32, threadIdx.x == 192);
      TS_TRACE_U(3, acc_it, threadIdx.x == 192);
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + a * MT + (static_cast<uint32_t>(q * 32) << 16);
      const bool has_acc = w.k_count > 0;
      // TMEM reads are issued four chunks (128 columns) at a time and awaited once: a read's
      // latency is far longer than the conversion of one chunk, so they must overlap each other.
      constexpr int kBatch = 4;
#pragma unroll
      for (int c0 = 0; c0 < kChunks; c0 += kBatch) {
        uint32_t v[kBatch][32];
        if (has_acc) {
#pragma unroll
          for (int b = 0; b < kBatch; ++b) tmem_ld_32x32(taddr + (c0 + b) * 32, v[b]);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int b = 0; b < kBatch; ++b)
#pragma unroll
            for (int e = 0; e < 32; ++e) v[b][e] = 0u;
        }
        if (c0 + kBatch == kChunks) {
          // every TMEM read of this accumulator has completed: hand it back to the MMA warp
          tc_fence_before_sync();
          mbar_arrive(smem_u32(&bars->acc_empty[a]));
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          const int cc = c0 + b;
          uint32_t(&cur)[32] = v[b];
          uint32_t o[16];
          if (beta != 0.0f && active && (cc * 32 < m_cnt)) {
            const uint4* cs = reinterpret_cast<const uint4*>(gdst + cc * 32);
#pragma unroll
            for (int e4 = 0; e4 < 4; ++e4) {
              uint4 old = make_uint4(0, 0, 0, 0);
              if (cc * 32 + e4 * 8 < m_cnt) old = cs[e4];
              const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float c0f = unpack1<DT>(static_cast<uint16_t>(ow[e] & 0xffffu));
                const float c1f = unpack1<DT>(static_cast<uint16_t>(ow[e] >> 16));
                const int idx = e4 * 8 + e * 2;
                o[e4 * 4 + e] = pack2<DT>(alpha * __uint_as_float(cur[idx]) + beta * c0f,
                                          alpha * __uint_as_float(cur[idx + 1]) + beta * c1f);
              }
            }
          } else if (alpha == 1.0f) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              o[e] = pack2<DT>(__uint_as_float(cur[2 * e]), __uint_as_float(cur[2 * e + 1]));
            }
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              o[e] = pack2<DT>(alpha * __uint_as_float(cur[2 * e]),
                               alpha * __uint_as_float(cur[2 * e + 1]));
            }
          }
          uint4* dst = reinterpret_cast<uint4*>(my_row + cc * 64);
#pragma unroll
          for (int e4 = 0; e4 < 4; ++e4) {
            dst[e4] = make_uint4(o[e4 * 4], o[e4 * 4 + 1], o[e4 * 4 + 2], o[e4 * 4 + 3]);
          }
        }
      }
      bars->c_row[j] = active ? static_cast<int>(c_row) : -1;
      TS_TRACE(33, threadIdx.x == 192);
      TS_TRACE_U(4, acc_it, threadIdx.x == 192);
      named_barrier_sync(1, 128);       // all 128 rows are staged
      TS_TRACE_U(5, acc_it, threadIdx.x == 192);
      {
        constexpr int kLpr = C::kLanesPerRow, kRpi = C::kRowsPerInstr;
        const int chunk = lane % kLpr, sub = lane / kLpr;
        const bool m_ok = chunk * 8 < m_cnt;
#pragma unroll
        for (int r4 = 0; r4 < 32 / kRpi; r4 += 4) {
          // four rows per batch: shared-memory reads first, then the global stores
          int cr[4];
          uint4 val[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int row = q * 32 + (r4 + e) * kRpi + sub;
            cr[e] = bars->c_row[row];
            val[e] = *reinterpret_cast<const uint4*>(epi + row * C::kEpiRowBytes + chunk * 16);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (cr[e] >= 0 && m_ok) {
              *reinterpret_cast<uint4*>(Ct + static_cast<long long>(cr[e]) * ldc + m0 + chunk * 8) = val[e];
            }
          }
        }
      }
      TS_TRACE_U(6, acc_it, threadIdx.x == 192);
      named_barrier_sync(1, 128);       // the staging rows may be overwritten
      TS_TRACE_U(7, acc_it, threadIdx.x == 192);
      ++acc_it;
      w = wn;
    }
    TS_TRACE(34, threadIdx.x == 192);
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
  if (threadIdx.x == 0 && bars->abort_flag) atomicExch(status, kErrTimeout);
  TS_TRACE(2, threadIdx.x == 0);
}

template <int DT, int MT>
cudaError_t launch_variant(const CUtensorMap& tmap_w, const WorkItem* sched, int rounds, int grid,
                           const BlockDesc* blocks, int blk_stride, const void* At, long long lda, void* Ct, long long ldc, int M,
                           float alpha, float beta, int* status, cudaStream_t stream) {
  auto kern = masked_gemm_kernel<DT, MT>;
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
  kern<<<grid, kThreads, Cfg<MT>::kSmemBytes, stream>>>(tmap_w, sched, rounds, blocks, blk_stride,
                                                        static_cast<const uint16_t*>(At), lda,
                                                        static_cast<uint16_t*>(Ct), ldc, M, alpha,
                                                        beta, status);
  return cudaGetLastError();
}

}  // namespace

cudaError_t masked_gemm_launch(int dtype, int unit_rows, const CUtensorMap& tmap_w,
                               const WorkItem* sched, int rounds, int grid,
                               const BlockDesc* blocks, int blk_stride, const void* At,
                               long long lda, void* Ct, long long ldc, int M, float alpha,
                               float beta, int* status, cudaStream_t stream) {
  if (unit_rows == 256) {
    return dtype == kBF16 ? launch_variant<kBF16, 256>(tmap_w, sched, rounds, grid, blocks, blk_stride, At, lda, Ct, ldc,
                                                       M, alpha, beta, status, stream)
                          : launch_variant<kF16, 256>(tmap_w, sched, rounds, grid, blocks, blk_stride, At, lda, Ct, ldc,
                                                      M, alpha, beta, status, stream);
  }
  if (unit_rows == 128) {
    return dtype == kBF16 ? launch_variant<kBF16, 128>(tmap_w, sched, rounds, grid, blocks, blk_stride, At, lda, Ct, ldc,
                                                       M, alpha, beta, status, stream)
                          : launch_variant<kF16, 128>(tmap_w, sched, rounds, grid, blocks, blk_stride, At, lda, Ct, ldc,
                                                      M, alpha, beta, status, stream);
  }
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

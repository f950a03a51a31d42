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
// the batch is its N dimension (MT = 256 columns per instruction), the kept rows are K.  The packed
// weights are the K-major A operand, fetched by TMA with 128-byte swizzle; the gathered activation
// rows are the MN-major B operand, fetched with 16-byte cp.async into the same swizzle pattern (one
// kept row is one contiguous 2*MT-byte global segment, one warp instruction each).  Accumulators
// live in TMEM, double buffered, so the epilogue of one work unit overlaps the main loop of the
// next.  The epilogue thread that owns TMEM lane j converts its row to 16 bit in shared memory and
// writes it to Ct with one bulk copy: an output row of a unit is one contiguous global segment.
//
// Warp roles (320 threads): warp 0 = weight TMA, warp 1 = TMEM allocation + MMA issue,
// warps 2-5 = activation gather, warps 6-9 = epilogue.
#include "ts_common.cuh"
#include "ts_kernels.h"

namespace ts {

namespace {

constexpr int kMT = 256;                 // batch rows per work unit (MMA N)
constexpr int kNT = 128;                 // columns per tile (MMA M, TMEM lanes)
constexpr int kKB = 64;                  // kept rows per pipeline stage
constexpr int kStages = 3;
constexpr int kLag = kStages - 1;        // gather stages in flight per producer thread
constexpr int kWBytes = kNT * kKB * 2;   // 16 KiB
constexpr int kABytes = kKB * kMT * 2;   // 32 KiB
constexpr int kStageBytes = kWBytes + kABytes;
constexpr int kEpiRowBytes = kMT * 2 + 16;  // +16: rows land in distinct bank groups
constexpr int kEpiBytes = kNT * kEpiRowBytes;
constexpr int kBarBytes = 256;
constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarBytes + 1024;
constexpr int kThreads = 320;
constexpr int kTmemCols = 512;           // two accumulators of kMT fp32 columns
constexpr uint32_t kALbo = kKB * 128;    // bytes between 64-row batch groups of the gathered operand
constexpr uint32_t kASbo = 1024;         // bytes between 8-row K groups
constexpr uint32_t kWSbo = 1024;         // bytes between 8-row groups of the weight operand

struct Barriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int DT>
__global__ void __launch_bounds__(kThreads, 1)
masked_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const TileDesc* __restrict__ tiles,
                   const WorkUnit* __restrict__ sched, int rounds, const uint16_t* __restrict__ At,
                   long long lda, uint16_t* __restrict__ Ct, long long ldc, int M, float alpha,
                   float beta, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the swizzle pattern is a function of the shared-memory address bits.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi = smem + kStages * kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(epi + kEpiBytes);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int grid = gridDim.x;
  const int cta = blockIdx.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 128 + 1);  // 128 gather threads + the TMA thread
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
    tmem_alloc(smem_u32(&bars->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ weight TMA producer
    if (lane == 0) tma_prefetch_desc(&tmap_w);
    uint32_t it = 0;
    bool ok = true;
    for (int r = 0; r < rounds && ok; ++r) {
      const WorkUnit u = sched[static_cast<size_t>(r) * grid + cta];
      if (u.tile < 0) continue;
      const TileDesc td = tiles[u.tile];
      const int nkb = (td.k_count + kKB - 1) / kKB;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const uint32_t s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        ok = mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t bar = smem_u32(&bars->full[s]);
          mbar_arrive_expect_tx(bar, kWBytes);
          tma_load_2d(smem_u32(smem + s * kStageBytes), &tmap_w, kb * kKB, td.w_row0, bar);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = umma_idesc_f16(DT == kBF16 ? 1 : 0, /*a_mn=*/0, /*b_mn=*/1, kNT, kMT);
    uint32_t it = 0, acc_it = 0;
    bool ok = true;
    for (int r = 0; r < rounds && ok; ++r) {
      const WorkUnit u = sched[static_cast<size_t>(r) * grid + cta];
      if (u.tile < 0) continue;
      const TileDesc td = tiles[u.tile];
      const int nkb = (td.k_count + kKB - 1) / kKB;
      const uint32_t a = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      ok = mbar_wait(smem_u32(&bars->acc_empty[a]), aph ^ 1u, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + a * kMT;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const uint32_t s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        ok = mbar_wait(smem_u32(&bars->full[s]), ph, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        if (lane == 0) {
          const int krem = td.k_count - kb * kKB;
          const int nk16 = krem >= kKB ? kKB / 16 : (krem + 15) / 16;
          const uint32_t w_addr = smem_u32(smem + s * kStageBytes);
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
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ activation gather
    const int gw = warp - 2;            // 0..3: owns rows gw*16 .. +16 of every 64-row stage
    const int g = lane >> 3;            // 64-row batch group of this lane's 16-byte chunk
    const int c = lane & 7;             // chunk inside the 128-byte row
    uint32_t it = 0, done = 0;          // stages issued / stages signalled
    bool ok = true;
    for (int r = 0; r < rounds && ok; ++r) {
      const WorkUnit u = sched[static_cast<size_t>(r) * grid + cta];
      if (u.tile < 0) continue;
      const TileDesc td = tiles[u.tile];
      const int nkb = (td.k_count + kKB - 1) / kKB;
      const int m = u.mblock * kMT + lane * 8;
      const bool m_ok = m < M;
      const uint16_t* src_col = At + (m_ok ? m : 0);
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const uint32_t s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        // kept-row indices of this warp's 16 rows: one coalesced read, then shuffles
        const int i_mine = kb * kKB + gw * 16 + (lane & 15);
        int k_mine = -1;
        if (i_mine < td.k_count) k_mine = td.k_list[i_mine] + (td.relative ? i_mine : 0);
        ok = mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t a_stage = smem_u32(smem + s * kStageBytes + kWBytes);
#pragma unroll
        for (int rr = 0; rr < 16; ++rr) {
          const int kk = __shfl_sync(0xffffffffu, k_mine, rr);
          const int row = gw * 16 + rr;
          const uint32_t dst = a_stage + g * kALbo + (row >> 3) * kASbo + (row & 7) * 128 +
                               ((c ^ (row & 7)) << 4);
          const bool valid = (kk >= 0) && m_ok;
          const uint16_t* src = valid ? src_col + static_cast<long long>(kk) * lda : At;
          cp_async_16(dst, src, valid ? 16u : 0u);
        }
        cp_async_commit();
        if (it - done >= static_cast<uint32_t>(kLag)) {
          cp_async_wait_group<kLag>();
          fence_proxy_async_smem();
          mbar_arrive(smem_u32(&bars->full[done % kStages]));
          ++done;
        }
      }
    }
    // drain: everything this thread issued has to land before the last stages are signalled
    cp_async_wait_group<0>();
    fence_proxy_async_smem();
    if (ok) {
      for (; done < it; ++done) mbar_arrive(smem_u32(&bars->full[done % kStages]));
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;             // TMEM lane quarter this warp may read
    const int j = q * 32 + lane;        // tile column owned by this thread
    uint8_t* my_row = epi + j * kEpiRowBytes;
    const uint32_t my_row_s = smem_u32(my_row);
    uint32_t acc_it = 0;
    bool ok = true;
    for (int r = 0; r < rounds && ok; ++r) {
      const WorkUnit u = sched[static_cast<size_t>(r) * grid + cta];
      if (u.tile < 0) continue;
      const TileDesc td = tiles[u.tile];
      const uint32_t a = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      const int m0 = u.mblock * kMT;
      const int m_cnt = min(kMT, M - m0);
      const bool active = j < td.n_count;
      long long c_row = 0;
      if (active) {
        c_row = td.c_row0 + (td.n_list ? td.n_list[j] + (td.relative ? j : 0) : j);
      }
      uint16_t* gdst = Ct + c_row * ldc + m0;
      ok = mbar_wait(smem_u32(&bars->acc_full[a]), aph, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      bulk_wait_read_all();             // my previous row has left shared memory
      const uint32_t taddr = tmem_base + a * kMT + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int cc = 0; cc < kMT / 32; ++cc) {
        uint32_t v[32];
        if (td.k_count > 0) {
          tmem_ld_32x32(taddr + cc * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
        }
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
              const float c0 = unpack1<DT>(static_cast<uint16_t>(ow[e] & 0xffffu));
              const float c1 = unpack1<DT>(static_cast<uint16_t>(ow[e] >> 16));
              const int idx = e4 * 8 + e * 2;
              o[e4 * 4 + e] = pack2<DT>(alpha * __uint_as_float(v[idx]) + beta * c0,
                                        alpha * __uint_as_float(v[idx + 1]) + beta * c1);
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            o[e] = pack2<DT>(alpha * __uint_as_float(v[2 * e]), alpha * __uint_as_float(v[2 * e + 1]));
          }
        }
        uint4* dst = reinterpret_cast<uint4*>(my_row + cc * 64);
#pragma unroll
        for (int e4 = 0; e4 < 4; ++e4) {
          dst[e4] = make_uint4(o[e4 * 4], o[e4 * 4 + 1], o[e4 * 4 + 2], o[e4 * 4 + 3]);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&bars->acc_empty[a]));
      if (active && m_cnt > 0) {
        fence_proxy_async_smem();
        bulk_store(gdst, my_row_s, static_cast<uint32_t>(m_cnt) * 2u);
        bulk_commit();
      }
      ++acc_it;
    }
    bulk_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && bars->abort_flag) atomicExch(status, kErrTimeout);
}

}  // namespace

int masked_gemm_unit_rows() { return kMT; }

cudaError_t masked_gemm_launch(int dtype, const CUtensorMap& tmap_w, const TileDesc* tiles,
                               const WorkUnit* sched, int rounds, int grid, const void* At,
                               long long lda, void* Ct, long long ldc, int M, float alpha,
                               float beta, int* status, cudaStream_t stream) {
  auto kern = dtype == kBF16 ? masked_gemm_kernel<kBF16> : masked_gemm_kernel<kF16>;
  // The dynamic shared-memory limit is a per-device, per-kernel attribute: set it once for each.
  static bool attr_set[2][64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const int di = dtype == kBF16 ? 1 : 0;
  if (dev >= 64 || !attr_set[di][dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    if (dev < 64) attr_set[di][dev] = true;
  }
  kern<<<grid, kThreads, kSmemBytes, stream>>>(tmap_w, tiles, sched, rounds,
                                               static_cast<const uint16_t*>(At), lda,
                                               static_cast<uint16_t*>(Ct), ldc, M, alpha, beta,
                                               status);
  return cudaGetLastError();
}

}  // namespace ts

// Shared device-side helpers for the tile-sparse kernels (sm_100a only).
//
// Thin wrappers over the PTX this library needs: mbarrier, cp.async, bulk/TMA copies, tcgen05
// (tensor-memory allocation, MMA issue, commit, loads) and proxy fences.  Every blocking wait is
// bounded: a wait that runs out sets a CTA-wide abort flag and returns false, so a broken pipeline
// ends the kernel with an error status instead of hanging the GPU.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace ts {

// ---------------------------------------------------------------------------------------------
// Status codes shared by host and device (mirrored in include/tilesparse.h).
// ---------------------------------------------------------------------------------------------
enum : int {
  kOk = 0,
  kErrInvalid = 1,
  kErrCuda = 2,
  kErrTimeout = 3,
  kErrUnsupported = 4,
  kErrNoMem = 5,
};

enum : int { kF16 = 0, kBF16 = 1, kF32 = 2 };

// One column tile of a tile-wise sparse layer, as the GEMM kernels see it.
//   kept K row i of the tile  -> row  k_list[i] + (relative ? i : 0)              of A^T
//   kept column j of the tile -> row  c_row0 + (n_list ? n_list[j] + (relative ? j : 0) : j) of C^T
//   packed weights of the tile start at row w_row0 of the packed-W matrix ([rows][K-contiguous]).
struct TileDesc {
  const int* k_list;
  const int* n_list;
  int k_count;
  int n_count;
  int w_row0;
  int c_row0;
  int relative;
  int pad_;
};

// One unit of work of the persistent GEMM: one column tile x a run of batch rows.  Entries are
// self-contained (they carry the tile's lists and counts) so a CTA reaches its first data request
// with two dependent global reads: work item -> kept-row indices -> activation rows.
//   flags bit 0: the index lists hold relative offsets (index - position)
//   flags bit 1: the tile's kept columns are consecutive rows of Ct and fill a 128-row store box
//   m_begin / m_len: the unit's batch rows; m_len is a multiple of 64, at most the kernel's MT
struct alignas(16) WorkItem {
  const int* k_list;
  const int* n_list;
  int k_count;
  int n_count;
  int w_row0;
  int c_row0;
  int flags;
  int m_begin;
  int m_len;
  int tile;  // < 0: no unit
};
constexpr int kItemRelative = 1;
constexpr int kItemDenseRows = 2;
// Split-K part: the unit covers only a range of the tile's kept rows (K blocks flags >> 8 onwards,
// k_list / k_count already describe the part) and writes alpha * acc as fp32 into the schedule's
// scratch rows c_row0 + j instead of Ct; a second kernel adds the parts up and finishes the epilogue.
constexpr int kItemScratch = 4;
constexpr int kItemKb0Shift = 8;
static_assert(sizeof(WorkItem) == 48, "WorkItem is read as three 16-byte words");

// What the GEMM epilogue does with an accumulator value x of tile column n before it is stored:
//     y = act(alpha * x + beta * Ct_old + bias[n])
// and where the result goes besides Ct: up to 7 peer buffers with the same layout (other GPUs'
// copies of Ct, written with plain stores over NVLink: the all-gather of a tile-sharded layer).
enum : int { kActNone = 0, kActRelu = 1, kActGelu = 2 };
struct EpilogueArgs {
  float alpha;
  float beta;
  const float* bias;   // indexed by Ct row (global column of W), or nullptr
  int act;
  int n_peers;
  uint16_t* peers[7];
  // Multicast address of Ct (an NVSwitch multicast mapping of the same buffer on every GPU of the
  // group, this one included), or nullptr: every kept row is then stored once with multimem.st and
  // the switch delivers it to all copies; Ct itself and peers[] are not written by plain stores.
  uint16_t* multicast;
  // One tensor map per peer (in global memory, same box and swizzle as the map over Ct), or nullptr:
  // a tile whose kept columns are consecutive rows of Ct then leaves for every peer as TMA tile
  // stores issued by one thread, like the local copy, instead of 16-byte stores from every lane.
  const CUtensorMap* peer_maps;
  // fp32 partial sums of split-K units: scratch[row][m], row pitch scratch_ld elements, and a tensor
  // map over it in global memory (box 32 floats x 128 rows, 128-byte swizzle) for the units' TMA stores
  float* scratch;
  long long scratch_ld;
  const CUtensorMap* scratch_map;
};

// One tile whose kept rows were split over `parts` units per batch block: part p wrote its fp32 partial
// sums to scratch rows scratch_row0 + p * 128 + j (j = position of the kept column in the tile).
struct SplitTile {
  const int* n_list;
  int n_count;
  int c_row0;
  int relative;
  int parts;
  int scratch_row0;
  int pad_;
};

// One 64-row K block of a work unit.  A CTA's blocks are stored in processing order; the host
// builds these descriptors and a small kernel resolves them into the records the gather warps read.
//   meta: bits 0-6 number of valid rows (1..64), bit 7 relative-offset lists, bits 8-9 the unit's
//   batch rows in 64-row groups minus one, bits 10-31 position of the block's first row inside the
//   tile's list; 0xFFFFFFFF marks the end of the CTA's stream.
struct alignas(16) BlockDesc {
  const int* idx;  // the block's first kept-row index (tile list + position)
  int m0;          // first batch row of the unit
  uint32_t meta;
};
static_assert(sizeof(BlockDesc) == 16, "BlockDesc is copied as one 16-byte word");
constexpr uint32_t kBlockEnd = 0xFFFFFFFFu;
// The gather warps read a block as one resolved record of kBlockMetaInts ints: {m0, meta, 0, 0}
// followed by where each of the block's 64 kept rows starts, in 16-byte segments from the base pointer.
constexpr int kBlockMetaInts = 4 + 64;

// How a kept row number becomes a segment number.  Matrix: row * ld8 (ld8 = row pitch / 8 elements).
// Convolution (conv_cin > 0): row = (r * conv_kw + j) * conv_cin + c  ->  (j * conv_cin + c) * ld8 + r * conv_wp8,
// with ld8 the pitch of one input plane and conv_wp8 the padded image width, both in 8-element units.
struct RowMap {
  long long ld8;
  int conv_cin;
  int conv_kw;
  int conv_wp8;
  int pad_;
};

// ---------------------------------------------------------------------------------------------
// Generic helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// try_wait that lets the hardware park the thread for up to `hint_ns` while the phase is pending.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Cycle budget of one wait (about two seconds at 2 GHz).  A healthy pipeline waits microseconds.
constexpr long long kWaitCycleLimit = 4000000000LL;

// Bounded wait.  Returns false when the CTA is aborting (another wait ran out) or this one did.
// A waiting warp shares its scheduler with warps that have work to issue, so between polls it
// sleeps instead of spinning.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_hint(bar, parity, 4000u)) return true;
    __nanosleep(32);
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycleLimit) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start while the kernel before it in the stream is still running.  grid_dependency_wait() blocks
// until that kernel has completed and its writes are visible; grid_launch_dependents() lets the
// kernel after this one start early in turn.  Both are no-ops in an ordinary launch.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// Proxy / tcgen05 fences
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// cp.async (16-byte, L2-only) with zero fill when src_bytes == 0
// ---------------------------------------------------------------------------------------------
// No "memory" clobber on purpose: the destination is only ever read by the tensor core through a
// descriptor and the source is read-only input, so the compiler may move ordinary loads (the
// kept-row index reads that feed the next copy's address) across it.  Ordering against the stage's
// mbarrier comes from cp.async.mbarrier.arrive, which is volatile and follows in program order.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}

__device__ __forceinline__ void cp_async_16_ca(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// Plain 16-byte copy (no zero-fill operand): the form the load/store unit issues fastest.
__device__ __forceinline__ void cp_async_16_full(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}

__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// The mbarrier receives one (pre-counted) arrival once every cp.async this thread issued so far
// has written its bytes.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_all;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------------
// TMA tile load (2-D, no multicast) and row-wise bulk store
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, "
      "%3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// TMA tile store: the box of `map` leaves shared memory for the tensor at column x, row y.  Parts of
// the box outside the tensor are not written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void bulk_store(void* gdst, uint32_t ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(ssrc), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

__device__ __forceinline__ void bulk_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// One 16-byte store to a multicast address: NVSwitch writes it into every GPU's copy of the buffer.
// (A store only: nothing here ever loads through a multicast mapping.)
__device__ __forceinline__ void multimem_st_16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// Tensor memory and tcgen05.mma (one CTA per MMA, cta_group::1)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate == 0 overwrites D.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive on an mbarrier once every MMA this thread issued so far has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// 32 lanes x 32 columns of fp32: thread l of the warp receives row (lane base + l), 32 columns.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle, Blackwell version field set.
//   lbo / sbo: leading / stride byte offsets (multiples of 16).
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t saddr, uint32_t lbo,
                                                         uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;  // layout type: SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 with fp32 accumulation.
//   fmt: 0 = f16, 1 = bf16 (both operands); a_mn / b_mn: 1 when that operand is MN-major in smem.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int fmt, int a_mn, int b_mn, int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
         (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// 16-bit packing
// ---------------------------------------------------------------------------------------------
template <int DT>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (DT == kF16) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

template <int DT>
__device__ __forceinline__ float unpack1(uint16_t v) {
  if constexpr (DT == kF16) {
    return __half2float(*reinterpret_cast<const __half*>(&v));
  } else {
    return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&v));
  }
}

}  // namespace ts

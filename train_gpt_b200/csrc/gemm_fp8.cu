// Block-scaled e4m3 GEMM for sm_100a:  D[m,n] = sum_kb SA(m,kb) SB(n,kb) sum_{k in kb} A[m,k] B[n,k]
//
// Replaces jax.nn.scaled_matmul as train-gpt calls it (fp8.py:70-76) plus the bf16 cast of
// fp8.py:78, and -- with other operand orientations -- the backward GEMMs of fp8.py:96-97.
//
// The scales are float32 (amax/448), not powers of two, so the tensor core's own
// block-scale path (UE8M0 factors) cannot apply them bit-faithfully.  Instead every
// 128-deep contraction block is issued as its own tcgen05.mma chain into a fresh TMEM
// accumulator buffer, and sixteen "promotion" warps pull each finished buffer out of TMEM
// (tcgen05.ld), hand it back to the tensor core, multiply by SA*SB and add into float32
// register accumulators with packed f32x2 FMAs while the tensor core fills the next buffer.
//
// Tile: 128 rows x BN columns, BN = 256 (two 256-column TMEM buffers) or 128 (four).  The
// wide tile halves the shared-memory and L2 traffic per FLOP and doubles the tensor-core
// time per issued instruction, which is what keeps the single-thread issue loop and the
// barrier round trips off the critical path.
//
// Warp roles in the CTA (persistent, one CTA per SM, tiles round-robin):
//   warps 0..P-1 promotion + epilogue (P = 16, or 12 for 192-column tiles); warp w may touch TMEM
//                lanes 32*(w%4).. (a hardware rule) and owns accumulator columns (BN/4)*(w/4)..;
//                four warps per scheduler hide each other's TMEM-load latency.  bf16 tiles leave
//                through one bulk tensor store per warp (registers -> the warp's swizzled staging
//                rows -> cp.async.bulk.tensor), waited for only when the rows are reused a tile
//                later; float32 tiles use the warp's own 16-byte coalesced stores.
//   warp P       TMA producer: A (one 128 x 128-byte box) and B (BN/128 boxes), 128B swizzle
//   warp P+1     MMA issuer (owns the TMEM allocation): one lane-split barrier wait per block
//   warps P+2,3  (256-column tiles only) idle padding of the producer's warpgroup, so that it can
//                release registers to the promotion warpgroups with setmaxnreg: 96 -> 40 / 104.
//                The 8 extra registers take the tile-boundary spills from 14 stores / 8 loads to
//                3 / 7; their reloads miss the 28 KB of L1 left beside 214 KB of shared memory.
//
// Operand orientation is data, not code: the TMA box is 128 bytes x 128 rows for both
// K-major and MN-major storage (only the coordinates swap), and the shared-memory operand
// descriptors / instruction descriptor carry the major-ness, so dgrad and wgrad read the
// same buffers the forward wrote, untransposed.
//
// Every wait on an mbarrier is bounded: when the limit runs out the waiting role raises a
// CTA-wide abort flag, stores a code in *status, and all roles fall through to the common
// teardown (TMEM is always freed).
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"

namespace tg {

constexpr int BM = 128;          // tile rows (TMEM lanes)
constexpr int BK = 128;          // contraction block = scale granularity (fp8.py:27)
constexpr int UMMA_K = 32;       // K of one tcgen05.mma.kind::f8f6f4
constexpr int kTmemCols = 512;
constexpr int kTileBytes = 128 * 128;            // one operand TMA box: 128 rows x 128 bytes
constexpr int kIssuers = 1;                      // MMA-issuing warps
constexpr int kSmemLimit = 227 * 1024;
constexpr long long kWaitLimitCycles = 4000000000LL;  // ~2 s at 2 GHz

// Compile-time plan of one kernel variant.
template <int BN_, int SB_GRAN, bool OUT_F32, bool CTA2>
struct Cfg {
  static constexpr int BN = BN_;
  // 192-column tiles run 12 promotion warps (14 warps in all: 128 registers per thread instead
  // of the 96 an 18-warp CTA gets), the others 16
  static constexpr int promo_warps = BN == 192 ? 12 : 16;
  // Warp layout: promotion warps 0..P-1 (whole warpgroups), then the TMA producer, then the MMA
  // issuer.  The 256-column tile pads that last warpgroup with two idle warps so that it can hand
  // registers over with setmaxnreg: 20 warps start at 96 registers per thread; the producer's
  // warpgroup drops to `service_regs` and each promotion warpgroup grows to `promo_regs`
  // (service_regs + 4 * promo_regs <= 5 * 96 per scheduler, so the growth never waits for
  // registers that nobody releases).
  static constexpr bool regsteal = BN == 256;
  static constexpr int producer_warp = promo_warps;
  static constexpr int issuer_warp = promo_warps + 1;
  static constexpr int warps = promo_warps + (regsteal ? 4 : 2);
  static constexpr int threads = 32 * warps;
  static constexpr int promo_regs = 104, service_regs = 40;
  static_assert(service_regs + 4 * promo_regs <= 5 * 96, "register hand-over asks for more than is released");
  static constexpr int tmem_bufs = BN > 128 ? 2 : 4;
  static constexpr int tmem_stride = kTmemCols / tmem_bufs;   // columns between accumulator buffers
  static constexpr int cols_per_warp = BN / (promo_warps / 4);  // 64 or 32
  static constexpr int b_boxes = CTA2 ? 1 : (BN + 127) / 128; // a CTA of a pair loads half of B
  static constexpr int stage_bytes = kTileBytes * (1 + b_boxes);
  static constexpr int esize = OUT_F32 ? 4 : 2;
  // epilogue: a warp stages its 32 rows x `phase_cols` columns at a time (rows of <= 128
  // bytes; a fourth pipeline stage bought with narrower staging rows measured no faster)
  static constexpr int row_bytes = cols_per_warp * esize;     // 64, 128 or 256
  static constexpr int phase_cap = 128;
  static constexpr int phase_row_bytes = row_bytes < phase_cap ? row_bytes : phase_cap;
  static constexpr int phases = row_bytes / phase_row_bytes;
  static constexpr int phase_cols = phase_row_bytes / esize;
  // bf16 tiles leave through bulk tensor stores (one 32-row box per promotion warp, never waited
  // for inside the tile loop); float32 tiles (two staging phases per warp, and the split-contraction
  // slices whose row bound is not the tensor's) keep the warp's own coalesced stores
  static constexpr bool bulk_store = !OUT_F32 && !CTA2;
  static constexpr int warp_out_bytes = 32 * phase_row_bytes;
  static constexpr int out_bytes = promo_warps * warp_out_bytes;
  // per-column scales: float[warps][2][cols_per_warp column scales + 32 row scales], double-buffered
  static constexpr int sc_slot = cols_per_warp + 32;
  static constexpr int sb_bytes = SB_GRAN == 1 ? promo_warps * 2 * sc_slot * 4 : 0;
  // 64-column warps with per-column scales read TMEM in the MMA fragment layout (a thread holds 4 rows
  // x 16 columns instead of 1 x 64): a column scale is then shared by 8 lanes instead of all 32, and
  // the block's 64 of them cost 8 conflict-free 8-byte reads per thread instead of 16 broadcasts of 16
  // bytes, which a warp is served a quarter at a time (64 -> 16 shared-memory wavefronts per warp)
  static constexpr bool frag = SB_GRAN == 1 && cols_per_warp == 64 && !CTA2;
  static constexpr int misc_bytes = 512;                      // barriers, TMEM pointer, abort flag
  static constexpr int stages_fit = (kSmemLimit - 1024 - out_bytes - sb_bytes - misc_bytes) / stage_bytes;
  static constexpr int stages = stages_fit > 6 ? 6 : stages_fit;
  // offsets from the 1024-aligned base of dynamic shared memory
  static constexpr int off_out = stages * stage_bytes;
  static constexpr int off_sb = off_out + out_bytes;
  static constexpr int off_bars = off_sb + sb_bytes;
  // (handing the wide accumulator over in two 128-column halves, each with its own barriers
  // and N=128 MMAs, was tried: 7 % slower -- A is read twice and twice as many MMAs issue)
  static constexpr int halves = 1;
  static constexpr int n_tbars = tmem_bufs * halves;
  static constexpr int n_bars = 2 * stages + 2 * n_tbars + kIssuers;
  static_assert(!CTA2 || BN == 256, "the 2-CTA variant is built for 256-column tiles");
  static constexpr int off_tmem_ptr = off_bars + n_bars * 8;
  static constexpr int off_abort = off_tmem_ptr + 4;
  static constexpr int smem_bytes = off_bars + misc_bytes + 1024;  // + slack for manual alignment
  static_assert(n_bars * 8 + 8 <= misc_bytes, "misc area too small");
  static_assert(stages >= 3, "pipeline too shallow");
  static_assert(smem_bytes <= kSmemLimit, "shared-memory plan exceeds the 227 KB a CTA may use");
};

struct GemmParams {
  const float* sa;
  long long sa_sm, sa_sk;
  const float* sb;
  long long sb_sn, sb_sk;
  void* d;              // output, row pitch ldd elements
  long long ldd;
  int M, N, nkb;        // nkb = contraction blocks per work item (all of them unless the contraction is split)
  int a_mn, b_mn;       // 1 = MN-major storage
  int tiles_m, tiles_n;
  int ksplit;           // the contraction is cut into this many equal ranges; range s of a tile is its own
                        // work item and writes its float32 partial sums to d + s * slice_elems
  long long slice_elems;
  unsigned* status;
};

// ---- PTX wrappers ----------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// One lane of a converged warp (warp-uniform callers keep operands in uniform registers).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
      "elect.sync rx|px, 0xffffffff;\n\t"
      "@px mov.s32 %0, 1;\n\t}"
      : "+r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking probe of a barrier phase.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false if the CTA is aborting (this call may be the one that
// raises the abort, tagging *status with `who`).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned* status, unsigned who) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 63u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *abort_flag = 1;
        if (status != nullptr) atomicCAS(status, 0u, who);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Bulk tensor store of one box from shared memory; completion is tracked by the issuing thread's
// bulk async-group, so the same lane must commit and later wait.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// returns once every bulk store this thread committed has finished READING shared memory
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 consecutive columns of 32-bit: thread i <- lane (base_lane + i), v[j] <- column j
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// Wait for this thread's outstanding tcgen05.ld.  The registers are listed as in/out
// operands so that no use of them can be scheduled above the wait.
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
        "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
        "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
        "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
      :
      : "memory");
}

// 16-column variants (fewer live registers: used by the 64-columns-per-warp tile)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld16(uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
        "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
      :
      : "memory");
}

// 16 lanes x 16 consecutive columns of 32-bit, in the fragment layout of an MMA accumulator: thread
// t (g = t / 4, j = t % 4) gets, for k = 0, 1:  v[4k], v[4k+1] <- lane base + g,     columns 8k + 2j, 8k + 2j + 1
//                                               v[4k+2], v[4k+3] <- lane base + g + 8, same columns
__device__ __forceinline__ void tmem_ld_frag16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void st_shared_b32(uint32_t addr, uint32_t x) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(x) : "memory");
}
__device__ __forceinline__ void st_shared_v2(uint32_t addr, uint32_t x, uint32_t y) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(x), "r"(y) : "memory");
}

// ---- CTA-pair (cta_group::2) variants ---------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes) : "memory");
}
// TMA load into THIS CTA's shared memory whose completion is counted on a barrier that may
// live in the pair's other CTA (no multicast: each CTA fetches its own boxes)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// arrive (when the issuing thread's MMAs retire) on the barrier at this offset in BOTH CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(uint16_t(3)) : "memory");
}
__device__ __forceinline__ void umma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory operand descriptor, 128-byte swizzle, 8-row groups 1024 bytes apart.
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 descriptor version (1 on sm_100)
//   bits 61-63 layout (2 = 128B swizzle)
// K-major: rows of 128 contraction bytes; 8 rows per swizzle atom; LBO unused.
// MN-major: rows of 128 m/n bytes, one row per k; SBO = stride between 8-k groups; LBO =
// stride between 128-wide m/n chunks (one chunk here).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= uint64_t((saddr >> 4) & 0x3FFFu);
  d |= uint64_t(kTileBytes >> 4) << 16;
  d |= uint64_t(1024 >> 4) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

__device__ __forceinline__ float ldg_f32(const float* ptr) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(ptr));   // L1-allocating: an activation scale's line serves 16-32 blocks
  return v;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// ---- kernel ----------------------------------------------------------------------------

// acc[j] += scale * v[2j..2j+1] for NC TMEM columns; SB_GRAN == 1 multiplies by the per-column
// scales staged in shared memory first.
template <int SB_GRAN, int NC>
__device__ __forceinline__ void promote(float2* acc, const uint32_t (&v)[NC], const float* stage, float sa_v, float s_scalar) {
  if (SB_GRAN == 1) {
    const float2 sa2 = make_float2(sa_v, sa_v);
#pragma unroll
    for (int j = 0; j < NC / 4; ++j) {
      const float4 sb4 = *reinterpret_cast<const float4*>(stage + 4 * j);
      const float2 p0 = make_float2(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]));
      const float2 p1 = make_float2(__uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
      acc[2 * j] = __ffma2_rn(__fmul2_rn(p0, make_float2(sb4.x, sb4.y)), sa2, acc[2 * j]);
      acc[2 * j + 1] = __ffma2_rn(__fmul2_rn(p1, make_float2(sb4.z, sb4.w)), sa2, acc[2 * j + 1]);
    }
  } else {
    const float2 s2 = make_float2(s_scalar, s_scalar);
#pragma unroll
    for (int j = 0; j < NC / 2; ++j) {
      const float2 pv = make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
      acc[j] = __ffma2_rn(pv, s2, acc[j]);
    }
  }
}

template <int BN_, int SB_GRAN, bool OUT_F32, bool CTA2>
__global__ void __launch_bounds__((Cfg<BN_, SB_GRAN, OUT_F32, CTA2>::threads), 1)
gemm_fp8_blockscaled_kernel(const __grid_constant__ CUtensorMap tmap_a,
                            const __grid_constant__ CUtensorMap tmap_b,
                            const __grid_constant__ CUtensorMap tmap_d, const GemmParams p) {
  using C = Cfg<BN_, SB_GRAN, OUT_F32, CTA2>;
  constexpr int BN = C::BN, kStages = C::stages, kTmemBufs = C::tmem_bufs, kCols = C::cols_per_warp;
  constexpr int kPromoWarps = C::promo_warps;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::off_bars;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
  constexpr int kHalves = C::halves, kTBars = C::n_tbars;
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * kStages + kTBars + b); };
  auto drain_bar = [&](int i) { return bar0 + 8u * (2 * kStages + 2 * kTBars + i); };
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + C::off_tmem_ptr);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::off_abort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = p.tiles_m * p.tiles_n;
  const int n_items = n_tiles * p.ksplit;     // work item i = (tile i % n_tiles, contraction range i / n_tiles)
  // A pair (cluster of two CTAs) shares one 256 x 256 tile: CTA r of the pair owns rows
  // r*128.. of it (its A tile, its TMEM, its output rows) and fetches B rows r*128.. for both.
  const uint32_t crank = CTA2 ? cluster_ctarank() : 0u;
  const bool leader = crank == 0;
  const int first_tile = CTA2 ? int(blockIdx.x >> 1) : int(blockIdx.x);
  const int tile_step = CTA2 ? int(gridDim.x >> 1) : int(gridDim.x);
  const int row_off = int(crank) * BM;         // this CTA's rows inside the (pair) tile
  constexpr int TM = CTA2 ? 2 * BM : BM;       // rows of a tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), CTA2 ? 2 : 1);   // one expect_tx arrival per CTA of the pair
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < kTBars; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), CTA2 ? 2 * kPromoWarps : kPromoWarps / kHalves);
    }
    for (int i = 0; i < kIssuers; ++i) mbar_init(drain_bar(i), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_b)) : "memory");
  }
  if (warp == C::issuer_warp) {
    if (CTA2) {
      tmem_alloc_pair(sbase + C::off_tmem_ptr, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(sbase + C::off_tmem_ptr, kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (CTA2) cluster_sync_all();   // both CTAs' barriers exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp >= C::promo_warps) {
    if (C::regsteal) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::service_regs));
    if (warp == C::producer_warp) {
      // ------------------------------ TMA producer -------------------------------------
      // The whole warp walks the loop (uniform control flow); one elected lane issues.
      uint32_t it = 0;
      bool ok = true;
      for (int item = first_tile; ok && item < n_items; item += tile_step) {
        const int tile = item % n_tiles, kb_off = (item / n_tiles) * p.nkb;
        const int m0 = (tile / p.tiles_n) * TM + row_off, n0 = (tile % p.tiles_n) * BN;
        for (int kb = 0; kb < p.nkb; ++kb, ++it) {
          const int s = it % kStages;
          ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), ((it / kStages) & 1u) ^ 1u, abort_flag, p.status, 1u));
          if (!ok) break;
          if (elect_one()) {
            const int k0 = (kb_off + kb) * BK;
            const uint32_t dst = sbase + s * C::stage_bytes;
            if (CTA2) {
              // both CTAs count their bytes on the LEADER's barrier: its MMA thread consumes both halves
              const uint32_t bar = mapa(full_bar(s), 0u);
              mbar_expect_tx_cluster(bar, C::stage_bytes);
              const int nb = n0 + int(crank) * 128;
              tma_load_2d_pair(dst, &tmap_a, bar, p.a_mn ? m0 : k0, p.a_mn ? k0 : m0);
              tma_load_2d_pair(dst + kTileBytes, &tmap_b, bar, p.b_mn ? nb : k0, p.b_mn ? k0 : nb);
            } else {
              mbar_expect_tx(full_bar(s), C::stage_bytes);
              tma_load_2d(dst, &tmap_a, full_bar(s), p.a_mn ? m0 : k0, p.a_mn ? k0 : m0);
#pragma unroll
              for (int b = 0; b < C::b_boxes; ++b) {
                const int nb = n0 + b * 128;  // a box wholly past N is still loaded: it arrives as zeros
                tma_load_2d(dst + (1 + b) * kTileBytes, &tmap_b, full_bar(s), p.b_mn ? nb : k0, p.b_mn ? k0 : nb);
              }
            }
          }
          __syncwarp();
        }
      }
    } else if (warp == C::issuer_warp && leader) {
      // ------------------------------ MMA issuers --------------------------------------
      // Issuer i takes the contraction blocks with (global block counter) % kIssuers == i.
      // Blocks are independent: each has its own TMEM buffer and shared-memory stage.
      const int issuer = 0;
      // instruction descriptor: D f32 (bit 4), A/B e4m3 (0), major bits 15/16, N>>3 at 17, M>>4 at 24
      const uint32_t idesc = (1u << 4) | (uint32_t(p.a_mn) << 15) | (uint32_t(p.b_mn) << 16) |
                             (uint32_t((BN / C::halves) >> 3) << 17) | (uint32_t(TM >> 4) << 24);
      // descriptor start-address step per UMMA_K: 32 bytes along a K-major row, 32 rows of 128 B otherwise
      const uint32_t a_step = p.a_mn ? (UMMA_K * 128) >> 4 : UMMA_K >> 4;
      const uint32_t b_step = p.b_mn ? (UMMA_K * 128) >> 4 : UMMA_K >> 4;
      const uint64_t a_desc0 = make_smem_desc(sbase);
      const uint64_t b_desc0 = make_smem_desc(sbase + kTileBytes);
      int my_tiles = 0;
      for (int item = first_tile; item < n_items; item += tile_step) ++my_tiles;
      const uint32_t total = uint32_t(my_tiles) * uint32_t(p.nkb);
      bool ok = true;
      // One barrier operation costs ~150 cycles even when the barrier is already complete (measured
      // with clock64 stamps: two waits plus two look-ahead probes per block made this loop ~1040
      // cycles long against 512 of tensor work per block).  So the loop does ONE wait instruction per
      // block: lanes 0-15 poll the accumulator buffer's barrier, lanes 16-31 the stage's.
      const bool stage_lane = lane >= 16;
      for (uint32_t it = issuer; ok && it < total; it += kIssuers) {
        const int s = it % kStages, buf = it % kTmemBufs;
        const uint32_t bar = stage_lane ? full_bar(s) : tempty_bar(buf * kHalves);
        const uint32_t par = stage_lane ? ((it / kStages) & 1u) : (((it / kTmemBufs) & 1u) ^ 1u);
        ok = __all_sync(0xffffffffu, mbar_wait(bar, par, abort_flag, p.status, stage_lane ? 3u : 2u));
        if (!ok) break;
        tc_fence_after();
        const uint64_t a_desc = a_desc0 + uint64_t((s * C::stage_bytes) >> 4);
        const uint64_t b_desc = b_desc0 + uint64_t((s * C::stage_bytes) >> 4);
        const uint32_t d_tmem = tmem_base + uint32_t(buf * C::tmem_stride);
        if (CTA2) {
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_f8_pair(d_tmem, a_desc + uint64_t(k * a_step), b_desc + uint64_t(k * b_step), idesc, k > 0 ? 1u : 0u);
            umma_commit_pair(empty_bar(s));    // frees the stage in both CTAs
            umma_commit_pair(tfull_bar(buf));  // both CTAs' promotion warps may read their half
          }
        } else {
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_f8(d_tmem, a_desc + uint64_t(k * a_step), b_desc + uint64_t(k * b_step), idesc, k > 0 ? 1u : 0u);
            umma_commit(empty_bar(s));    // shared-memory stage free once these MMAs retire
            umma_commit(tfull_bar(buf));  // accumulator buffer ready for promotion
          }
        }
        __syncwarp();
      }
      // make sure nothing issued here is still running when TMEM is freed
      if (elect_one()) {
        if (CTA2) asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(drain_bar(issuer)) : "memory");
        else umma_commit(drain_bar(issuer));
        mbar_wait(drain_bar(issuer), 0u, abort_flag, p.status, 4u);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------ promotion + epilogue --------------------------------
    if (C::regsteal) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::promo_regs));
    const int pw = warp;                       // 0..kPromoWarps-1
    const int quarter = warp & 3;              // TMEM lanes this warp may touch
    const int cg = pw >> 2;                    // column group
    const int r = quarter * 32 + lane;         // row inside the tile
    const int c0 = cg * kCols;                 // first column inside the tile
    float* sb_stage = reinterpret_cast<float*>(smem + C::off_sb) + pw * (2 * C::sc_slot);  // warp-private, double-buffered
    constexpr bool kFrag = C::frag;
    const int fg = lane >> 2, fj = lane & 3;     // fragment coordinates: rows fg + 8 i, column pairs 8 k + 2 fj
    const uint32_t out_base = sbase + C::off_out + uint32_t(pw) * C::warp_out_bytes + uint32_t(lane) * C::phase_row_bytes;
    // TMA swizzle of this row: 16-byte chunk index XOR address bits 7.. (128B: 3 bits, 64B: 2, 32B: 1)
    const int swz = C::phase_row_bytes == 128 ? (lane & 7) : C::phase_row_bytes == 64 ? ((lane >> 1) & 3) : ((lane >> 2) & 1);
    uint32_t it = 0;
    bool ok = true;

    // per-tile state, computed one tile ahead so that the first scale loads are in flight
    // during the previous tile's epilogue
    int m0 = 0, n0 = 0;
    bool m_ok = false, sb_ok = false;
    const float* sa_ptr = p.sa;
    const float* sb_ptr = p.sb;
    // The scales of block k+1 are loaded at the top of block k's iteration, by volatile asm so
    // that the compiler cannot sink the loads to their use: with ordinary loads it did, and clock64
    // stamps showed ~450 cycles of exposed L2 latency per block in these warps.  (Two blocks ahead
    // costs three more registers, which the 96-register variants do not have: measured slower.)
    float sa_q0 = 0.f;
    float2 sb_q0 = make_float2(0.f, 0.f);
    // per-column scales: lane j stages column c0 + j (32-column warps) or the pair c0 + 2j, c0 + 2j + 1
    constexpr int kPerLane = kCols / 32;
    auto load_sa = [&](int kb) {
      float v = 0.f;
      if (m_ok && kb < p.nkb) v = ldg_f32(sa_ptr + (long long)kb * p.sa_sk);
      return v;
    };
    // One scale per 128 columns: its address changes line with every block, so a load per block
    // misses L1 every time and the loop would run at one L2 round trip per block.  Instead lane l
    // fetches the scale of block 32 g + l once per 32 blocks and a shuffle hands each block its value.
    float sb_grp = 0.f, sb_nxt = 0.f;
    auto load_sb_lane = [&](int g) {
      float v = 0.f;
      const int kb = 32 * g + lane;
      if (sb_ok && kb < p.nkb) v = ldg_f32(sb_ptr + (long long)kb * p.sb_sk);
      return v;
    };
    auto load_sb = [&](int kb) {
      float2 v = make_float2(0.f, 0.f);
      if (sb_ok && kb < p.nkb) {
        const float* q = sb_ptr + (long long)kb * p.sb_sk;
        v.x = ldg_f32(q);
        if (SB_GRAN == 1 && kPerLane == 2) v.y = ldg_f32(q + p.sb_sn);
      }
      return v;
    };
    uint8_t* d_base = static_cast<uint8_t*>(p.d);
    auto open_tile = [&](int item) {
      const int tile = item % n_tiles;
      const long long ks = item / n_tiles, kb_off = ks * p.nkb;
      d_base = static_cast<uint8_t*>(p.d) + ks * p.slice_elems * C::esize;
      m0 = (tile / p.tiles_n) * TM + row_off;
      n0 = (tile % p.tiles_n) * BN;
      const int m = m0 + r;
      m_ok = m < p.M;
      sa_ptr = p.sa + (long long)(m_ok ? m : 0) * p.sa_sm + kb_off * p.sa_sk;
      if (SB_GRAN == 1) {
        const int col = n0 + c0 + kPerLane * lane;   // N % 8 == 0, so a pair is in or out together
        sb_ok = col < p.N;
        sb_ptr = p.sb + (long long)(sb_ok ? col : 0) * p.sb_sn + kb_off * p.sb_sk;
      } else {                                       // one scale per 128 columns
        const int nblk = (n0 + c0) / 128;
        sb_ok = true;
        sb_ptr = p.sb + (long long)((nblk * 128 < p.N) ? nblk : 0) * p.sb_sn + kb_off * p.sb_sk;
      }
      sa_q0 = load_sa(0);
      if (SB_GRAN == 1) sb_q0 = load_sb(0);
      else sb_grp = load_sb_lane(0);
    };

    if (first_tile < n_items) open_tile(first_tile);
    const uint32_t tempty_remote0 = CTA2 ? mapa(tempty_bar(0), 0u) : 0u;  // the leader's barrier, as seen from here
    for (int tile = first_tile; tile < n_items; tile += tile_step) {
      const int tile_m0 = m0, tile_n0 = n0;
      uint8_t* const tile_d = d_base;
      float2 acc[kCols / 2];
#pragma unroll
      for (int j = 0; j < kCols / 2; ++j) acc[j] = make_float2(0.f, 0.f);

      for (int kb = 0; kb < p.nkb; ++kb, ++it) {
        const int buf = it % kTmemBufs;
        const float sa_v = sa_q0;
        float2 sb_v = sb_q0;
        sa_q0 = load_sa(kb + 1);
        if (SB_GRAN == 1) {
          sb_q0 = load_sb(kb + 1);
        } else {
          const int kl = kb & 31;
          if (kl == 0) {
            if (kb != 0) sb_grp = sb_nxt;
            sb_nxt = load_sb_lane((kb >> 5) + 1);
          }
          sb_v.x = __shfl_sync(0xffffffffu, sb_grp, kl);
        }
        float* stage = sb_stage + (it & 1u) * C::sc_slot;
        if (SB_GRAN == 1) {
          if (kPerLane == 2) *reinterpret_cast<float2*>(stage + 2 * lane) = sb_v;
          else stage[lane] = sb_v.x;
          if (kFrag) stage[kCols + lane] = sa_v;   // row 32 * quarter + lane
          __syncwarp();
        }
        // After an abort the remaining iterations only keep the loop counters in step.
        const int tb = buf * kHalves + (kHalves == 2 ? (cg >> 1) : 0);   // this warp's half of the buffer
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(tb), (it / kTmemBufs) & 1u, abort_flag, p.status, 5u));
        if (!ok) continue;
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(buf * C::tmem_stride + c0);
        const float s_scalar = sa_v * sb_v.x;
        if (kCols > 32 && kPromoWarps == 12 && SB_GRAN != 1) {
          // 64 columns in two 32-column loads (128 registers per thread make room): one TMEM round
          // trip and 16 packed FMAs stand between the barrier and the buffer's release, not three
          uint32_t v[32];
          tmem_ld32(taddr, v);
          tmem_wait_ld(v);
          promote<SB_GRAN, 32>(acc, v, stage, sa_v, s_scalar);
          tmem_ld32(taddr + 32, v);
          tmem_wait_ld(v);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(tb));
          promote<SB_GRAN, 32>(acc + 16, v, stage + 32, sa_v, s_scalar);
        } else if (kFrag) {
          // acc[(4 q + i) * 2 + k] holds rows fg + 8 i, columns 16 q + 8 k + 2 fj (+1)
          float sa_r[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) sa_r[i] = stage[kCols + fg + 8 * i];
          // two staging sets: the loads of piece q + 1 are in flight while piece q is promoted
          uint32_t va[16], vb[16];
          tmem_ld_frag16(taddr, va);
          tmem_ld_frag16(taddr + (16u << 16), va + 8);
          tmem_wait_ld16(va);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t (&cur)[16] = (q & 1) ? vb : va;
            uint32_t (&nxt)[16] = (q & 1) ? va : vb;
            if (q < 3) {
              tmem_ld_frag16(taddr + 16 * (q + 1), nxt);
              tmem_ld_frag16(taddr + (16u << 16) + 16 * (q + 1), nxt + 8);
            }
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              const float2 sb2 = *reinterpret_cast<const float2*>(stage + 16 * q + 8 * k + 2 * fj);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int o = 8 * (i >> 1) + 4 * k + 2 * (i & 1);
                const float2 pv = make_float2(__uint_as_float(cur[o]), __uint_as_float(cur[o + 1]));
                float2& a = acc[(4 * q + i) * 2 + k];
                a = __ffma2_rn(__fmul2_rn(pv, sb2), make_float2(sa_r[i], sa_r[i]), a);
              }
            }
            if (q < 3) tmem_wait_ld16(nxt);
            if (q == 2) {        // every load of the buffer has landed
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(tempty_bar(tb));
            }
          }
        } else if (kCols > 32) {
          // 64 columns in four 16-column pieces; the buffer goes back after the last load lands
          uint32_t v[16];
#pragma unroll
          for (int q = 0; q < 3; ++q) {
            tmem_ld16(taddr + 16 * q, v);
            tmem_wait_ld16(v);
            promote<SB_GRAN, 16>(acc + 8 * q, v, stage + 16 * q, sa_v, s_scalar);
          }
          tmem_ld16(taddr + 48, v);
          tmem_wait_ld16(v);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) { if (CTA2) mbar_arrive_cluster(tempty_remote0 + 8u * buf); else mbar_arrive(tempty_bar(tb)); }
          promote<SB_GRAN, 16>(acc + 24, v, stage + 48, sa_v, s_scalar);
        } else {
          uint32_t v[32];
          tmem_ld32(taddr, v);
          tmem_wait_ld(v);
          // every partial sum of the buffer is in registers: hand it back to the tensor core
          tc_fence_before();
          __syncwarp();
          if (lane == 0) { if (CTA2) mbar_arrive_cluster(tempty_remote0 + 8u * buf); else mbar_arrive(tempty_bar(tb)); }
          promote<SB_GRAN, 32>(acc, v, stage, sa_v, s_scalar);
        }
      }

      // start the next tile's first scale loads before the stores of this one
      if (tile + tile_step < n_items) open_tile(tile + tile_step);

      // ---- epilogue: registers -> this warp's swizzled staging rows -> coalesced stores ------
      // Each thread holds one row; a warp-private transpose through shared memory lets every
      // store instruction write whole 128-byte lines (4 or 8 rows x one staging row each).  No
      // asynchronous proxy is involved, so there is nothing to fence or wait for: the warp's
      // own program order (plus __syncwarp) protects the staging rows.
      if (!ok) continue;
      const int row_base = tile_m0 + quarter * 32;
      constexpr int PRB = C::phase_row_bytes, LPR = PRB / 16, RPI = 32 / LPR;
      uint8_t* warp_out = smem + C::off_out + pw * C::warp_out_bytes;
      const int my_chunk = lane % LPR;
      if (C::bulk_store) {
        // bf16 output: the warp's 32 x kCols piece is one box.  Lane 0 hands it to the copy engine
        // and the warp goes straight on to the next tile; the wait for the engine to have read the
        // staging rows comes only before they are overwritten, one whole tile later.
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
        if (kFrag) {
          const uint32_t wb = sbase + C::off_out + uint32_t(pw) * C::warp_out_bytes;
#pragma unroll
          for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int k = 0; k < 2; ++k) {   // row fg + 8 i (row & 7 == fg & 7), 16-byte chunk 2 q + k, 4 fj bytes in
                const float2 a = acc[(4 * q + i) * 2 + k];
                st_shared_b32(wb + uint32_t(fg + 8 * i) * PRB + (uint32_t((2 * q + k) ^ (fg & 7)) << 4) + 4u * fj,
                              pack_bf16x2(a.x, a.y));
              }
        } else
#pragma unroll
        for (int c = 0; c < PRB / 16; ++c) {   // 8 bf16 per 16-byte chunk
          const int j = 4 * c;
          st_shared_v4(out_base + (uint32_t(c ^ swz) << 4), pack_bf16x2(acc[j].x, acc[j].y),
                       pack_bf16x2(acc[j + 1].x, acc[j + 1].y), pack_bf16x2(acc[j + 2].x, acc[j + 2].y),
                       pack_bf16x2(acc[j + 3].x, acc[j + 3].y));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the copy engine
        __syncwarp();
        if (lane == 0)   // rows past M and columns past N are clipped by the tensor map
          tma_store_2d(&tmap_d, sbase + C::off_out + uint32_t(pw) * C::warp_out_bytes, tile_n0 + c0, row_base);
        continue;
      }
#pragma unroll
      for (int ph = 0; ph < C::phases; ++ph) {
        __syncwarp();  // the previous read-back of these staging rows is complete
        if (kFrag && OUT_F32) {
          const uint32_t wb = sbase + C::off_out + uint32_t(pw) * C::warp_out_bytes;
#pragma unroll
          for (int qq = 0; qq < 2; ++qq)     // this phase's 32 columns are pieces 2 ph, 2 ph + 1
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int k = 0; k < 2; ++k) {   // column 16 qq + 8 k + 2 fj of the phase: chunk of 4 floats, 8-byte half
                const float2 a = acc[(4 * (2 * ph + qq) + i) * 2 + k];
                st_shared_v2(wb + uint32_t(fg + 8 * i) * PRB + (uint32_t((4 * qq + 2 * k + (fj >> 1)) ^ (fg & 7)) << 4) + 8u * (fj & 1),
                             __float_as_uint(a.x), __float_as_uint(a.y));
              }
        } else if (OUT_F32) {
#pragma unroll
          for (int c = 0; c < PRB / 16; ++c) {   // 4 floats per 16-byte chunk
            const int j = ph * (C::phase_cols / 2) + 2 * c;
            st_shared_v4(out_base + (uint32_t(c ^ swz) << 4), __float_as_uint(acc[j].x), __float_as_uint(acc[j].y),
                         __float_as_uint(acc[j + 1].x), __float_as_uint(acc[j + 1].y));
          }
        } else {
#pragma unroll
          for (int c = 0; c < PRB / 16; ++c) {   // 8 bf16 per 16-byte chunk
            const int j = ph * (C::phase_cols / 2) + 4 * c;
            st_shared_v4(out_base + (uint32_t(c ^ swz) << 4), pack_bf16x2(acc[j].x, acc[j].y),
                         pack_bf16x2(acc[j + 1].x, acc[j + 1].y), pack_bf16x2(acc[j + 2].x, acc[j + 2].y),
                         pack_bf16x2(acc[j + 3].x, acc[j + 3].y));
          }
        }
        __syncwarp();
        const int col = tile_n0 + c0 + ph * C::phase_cols + my_chunk * (16 / C::esize);
        uint8_t* dcol = tile_d + (long long)col * C::esize;
#pragma unroll
        for (int i = 0; i < 32 / RPI; ++i) {
          const int rr = i * RPI + lane / LPR;
          const int sw = PRB == 128 ? (rr & 7) : ((rr >> 1) & 3);
          const uint4 val = *reinterpret_cast<const uint4*>(warp_out + rr * PRB + ((my_chunk ^ sw) << 4));
          if (row_base + rr < p.M && col < p.N)
            *reinterpret_cast<uint4*>(dcol + (long long)(row_base + rr) * p.ldd * C::esize) = val;
        }
      }
    }
  }

  // ------------------------------ teardown ----------------------------------------------
  // the last bulk stores must have read their staging rows before the CTA's shared memory goes away
  if (C::bulk_store && warp < C::promo_warps && lane == 0) tma_store_wait_read();
  tc_fence_before();
  __syncthreads();
  if (CTA2) cluster_sync_all();   // the peer no longer reads this CTA's shared memory or signals its barriers
  if (warp == C::issuer_warp) {
    __syncwarp();
    tc_fence_after();
    if (CTA2) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host ------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int get_encode_fn(EncodeTiledFn* out) {
  static EncodeTiledFn cached = nullptr;
  if (cached == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    TG_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr)
      return record_cuda_error(cudaErrorSymbolNotFound, "cuTensorMapEncodeTiled entry point");
    cached = reinterpret_cast<EncodeTiledFn>(fn);
  }
  *out = cached;
  return TG_OK;
}

// 2-D tensor [outer][inner] of `esize`-byte elements, row pitch `pitch_bytes`; box of
// `box_inner_bytes` (32, 64 or 128, = the swizzle span) x `box_rows`.
static int make_tmap(CUtensorMap* map, CUtensorMapDataType dt, int esize, const void* base, int64_t inner,
                     int64_t outer, int64_t pitch_bytes, int box_inner_bytes, int box_rows) {
  EncodeTiledFn enc;
  if (int rc = get_encode_fn(&enc)) return rc;
  cuuint64_t dims[2] = {cuuint64_t(inner), cuuint64_t(outer)};
  cuuint64_t strides[1] = {cuuint64_t(pitch_bytes)};
  cuuint32_t box[2] = {cuuint32_t(box_inner_bytes / esize), cuuint32_t(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   box_inner_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                   : box_inner_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  return TG_OK;
}

template <int BN_, int SB_GRAN, bool OUT_F32, bool CTA2 = false>
static int launch_gemm(const tg_gemm_args* a, GemmParams p, cudaStream_t st) {
  using C = Cfg<BN_, SB_GRAN, OUT_F32, CTA2>;
  auto kern = gemm_fp8_blockscaled_kernel<BN_, SB_GRAN, OUT_F32, CTA2>;
  CUtensorMap ta, tb;
  const int64_t a_inner = p.a_mn ? a->M : a->K, a_outer = p.a_mn ? a->K : a->M;
  const int64_t b_inner = p.b_mn ? a->N : a->K, b_outer = p.b_mn ? a->K : a->N;
  if (int rc = make_tmap(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->a, a_inner, a_outer, a->lda, 128, 128)) return rc;
  if (int rc = make_tmap(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->b, b_inner, b_outer, a->ldb, 128, 128)) return rc;
  CUtensorMap td = ta;   // placeholder where the kernel variant does not use it
  if (C::bulk_store) {
    static_assert(!C::bulk_store || C::phases == 1, "one box per warp");
    if (int rc = make_tmap(&td, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.d, a->N, a->M, p.ldd * 2, C::phase_row_bytes, 32)) return rc;
  }
  constexpr int TM = CTA2 ? 2 * BM : BM;
  p.tiles_m = int((a->M + TM - 1) / TM);
  p.tiles_n = int((a->N + BN_ - 1) / BN_);
  const int64_t n_tiles = int64_t(p.tiles_m) * p.tiles_n * p.ksplit;   // work items
  if (n_tiles > INT32_MAX || n_tiles * p.nkb > INT32_MAX) return TG_ERR_TOO_LARGE;
  const int sms = sm_count();
  int grid = int(n_tiles < sms ? n_tiles : sms);
  // the attribute is per device: set it once for each device this instantiation runs on
  static bool attr_set[64] = {};
  int dev = 0;
  TG_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TG_ERR_SHAPE;
  if (!attr_set[dev]) {
    TG_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::smem_bytes));
    attr_set[dev] = true;
  }
  if (CTA2) {
    // A persistent grid must be co-resident.  Pairs need two free SMs in one GPC, and GPCs
    // with an odd SM count strand one, so ask the runtime how many pairs fit (cached per device).
    static int max_pairs[64] = {};
    if (max_pairs[dev] == 0) {
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(2 * (sms / 2));
      q.blockDim = dim3(C::threads);
      q.dynamicSmemBytes = C::smem_bytes;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2;
      qa[0].val.clusterDim.y = 1;
      qa[0].val.clusterDim.z = 1;
      q.attrs = qa;
      q.numAttrs = 1;
      int n = 0;
      TG_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, kern, &q));
      if (n < 1) return record_cuda_error(cudaErrorLaunchOutOfResources, "no CTA pair fits on this device");
      max_pairs[dev] = n;
    }
    const int pairs = max_pairs[dev];
    grid = 2 * int(n_tiles < pairs ? n_tiles : pairs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(C::threads);
    cfg.dynamicSmemBytes = C::smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TG_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, ta, tb, td, p));
  } else {
    kern<<<grid, C::threads, C::smem_bytes, st>>>(ta, tb, td, p);
  }
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}

// ---- split contraction -------------------------------------------------------------------
// A GEMM with few output tiles and a long contraction (the weight gradient: d_model x d_model
// outputs, tens of thousands of tokens contracted) leaves most SMs idle.  With caller-provided
// workspace the contraction is cut into S equal ranges, every (tile, range) pair becomes a work
// item writing float32 partial sums to its own slice of the workspace, and a second kernel adds
// the slices in range order (deterministic) and converts to the output type.

template <bool OUT_F32>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ d, int M, int N, long long ldd, int S,
                     long long slice_elems) {
  const long long quads = (long long)M * (N / 4);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < quads; i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / (N / 4);
    const int n = int(i % (N / 4)) * 4;
    float4 acc = *reinterpret_cast<const float4*>(ws + m * N + n);
    for (int sl = 1; sl < S; ++sl) {
      const float4 v = *reinterpret_cast<const float4*>(ws + sl * slice_elems + m * N + n);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (OUT_F32) {
      *reinterpret_cast<float4*>(static_cast<float*>(d) + m * ldd + n) = acc;
    } else {
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(d) + m * ldd + n) =
          make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
    }
  }
}

struct SplitPlan {
  int S;             // 1 = no split
  int64_t bytes;     // workspace the split needs
};

// S in {1, 2, 4, 8} (dividing the block count, every range at least 8 blocks) with the lowest
// modelled time, in units of one contraction block on one SM: waves x (blocks per item + ~3 for an
// item's ramp and stores), plus for S > 1 the reduce pass over S float32 slices at ~4 MB per unit.
// A 2048 x 6144 weight gradient is 512 tiles = 3.5 waves of 256 blocks; cut in two it is 6.9 waves
// of 128 (measured 6 % faster with the reduce); 2048 x 8192 (4.6 waves) is left whole.
static SplitPlan plan_split(const tg_gemm_args* a, int bn) {
  SplitPlan pl = {1, 0};
  if (a->K % BK != 0) return pl;
  const int64_t nkb = a->K / BK;
  const int64_t tiles = ((a->M + BM - 1) / BM) * ((a->N + bn - 1) / bn);
  const int sms = sm_count();
  if (sms <= 0) return pl;
  double best = 0.0;
  for (int S = 1; S <= 8; S *= 2) {
    if (nkb % S != 0 || (S > 1 && nkb / S < 8)) break;
    const int64_t waves = (tiles * S + sms - 1) / sms;
    double cost = double(waves) * (double(nkb / S) + 3.0);
    if (S > 1) cost += double(4 * S + 2) * double(a->M) * double(a->N) / 4.0e6;
    if (S == 1 || cost < best * 0.98) { best = cost; pl.S = S; }
  }
  if (pl.S > 1) pl.bytes = int64_t(pl.S) * a->M * a->N * int64_t(sizeof(float));
  return pl;
}

}  // namespace tg

using namespace tg;

// Tile width of a problem.  One scale per 128 columns: 128 x 256 tiles, 16 promotion warps
// (measured 1.70 / 1.92 PFLOP/s forward / dgrad against 1.53 / 1.59 for 128 x 192).  A scale per
// column (the weight gradient): 128 x 192 tiles with 12 promotion warps, whose 128 registers per
// thread hold the 64 accumulator columns plus the scale staging that 96 do not (1.04 PFLOP/s
// against 0.85 for 128 x 128).  TG_GEMM_BN=128|192|256 overrides, for measurements.
static int tile_width(const tg_gemm_args* a) {
  if (a->N <= 128) return 128;
  const char* e = getenv("TG_GEMM_BN");
  const int want = e != nullptr ? atoi(e) : 0;
  if (a->sb_gran_n == 1) return want == 128 ? 128 : 192;
  return want == 192 ? 192 : (want == 128 ? 128 : 256);
}

static int validate_gemm(const tg_gemm_args* a) {
  if (a == nullptr) return TG_ERR_SHAPE;
  if (a->M < 0 || a->N < 0 || a->K < 0) return TG_ERR_SHAPE;
  if (a->M > INT32_MAX || a->N > INT32_MAX || a->K > INT32_MAX) return TG_ERR_TOO_LARGE;
  if ((a->a_major != TG_MAJOR_K && a->a_major != TG_MAJOR_MN) || (a->b_major != TG_MAJOR_K && a->b_major != TG_MAJOR_MN))
    return TG_ERR_SHAPE;
  if (a->sb_gran_n != 1 && a->sb_gran_n != 128) return TG_ERR_SHAPE;
  if (a->out_dtype != TG_OUT_BF16 && a->out_dtype != TG_OUT_F32) return TG_ERR_SHAPE;
  if (a->N % 8 != 0 || a->ldd % 8 != 0 || a->ldd < a->N) return TG_ERR_SHAPE;
  if (a->lda % 16 != 0 || a->ldb % 16 != 0) return TG_ERR_SHAPE;
  const int64_t a_inner = a->a_major == TG_MAJOR_K ? a->K : a->M;
  const int64_t b_inner = a->b_major == TG_MAJOR_K ? a->K : a->N;
  if (a->lda < a_inner || a->ldb < b_inner) return TG_ERR_SHAPE;
  return TG_OK;
}

extern "C" int64_t tg_gemm_workspace_bytes(const tg_gemm_args* a) {
  if (validate_gemm(a) != TG_OK || a->M == 0 || a->N == 0 || a->K == 0) return 0;
  return plan_split(a, tile_width(a)).bytes;
}

extern "C" int tg_gemm_fp8_blockscaled(const tg_gemm_args* a, void* stream) {
  if (int rc = validate_gemm(a)) return rc;
  if (a->M == 0 || a->N == 0) return TG_OK;
  if (!aligned16(a->a) || !aligned16(a->b) || !aligned16(a->d)) return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool f32 = a->out_dtype == TG_OUT_F32;
  if (a->K == 0) {
    const size_t esz = f32 ? 4 : 2;
    TG_CUDA_CHECK(cudaMemset2DAsync(a->d, size_t(a->ldd) * esz, 0, size_t(a->N) * esz, size_t(a->M), st));
    return TG_OK;
  }
  GemmParams p;
  p.sa = a->sa; p.sa_sm = a->sa_stride_m; p.sa_sk = a->sa_stride_kb;
  p.sb = a->sb; p.sb_sn = a->sb_stride_n; p.sb_sk = a->sb_stride_kb;
  p.d = a->d; p.ldd = a->ldd;
  p.M = int(a->M); p.N = int(a->N); p.nkb = int((a->K + BK - 1) / BK);
  p.a_mn = a->a_major == TG_MAJOR_MN; p.b_mn = a->b_major == TG_MAJOR_MN;
  p.tiles_m = p.tiles_n = 0;
  p.ksplit = 1;
  p.slice_elems = 0;
  p.status = a->status;
  const bool g1 = a->sb_gran_n == 1;
  const int bn = tile_width(a);
  const bool wide = bn == 256;
  // CTA pairs (cta_group::2, 256 x 256 tiles, half the B bytes per CTA) are built and pass the
  // parity tests, but measure SLOWER than one CTA per tile (1.03 vs 1.70 PFLOP/s forward): with
  // only two 256-column TMEM buffers the barrier round trip through both CTAs' promotion warps
  // is longer than one block of tensor work.  Kept behind TG_GEMM_PAIR=1 for the next attempt.
  if (!g1 && a->N > 128 && a->M > 128 && getenv("TG_GEMM_PAIR") != nullptr)
    return f32 ? launch_gemm<256, 128, true, true>(a, p, st) : launch_gemm<256, 128, false, true>(a, p, st);
  const SplitPlan pl = plan_split(a, bn);
  if (pl.S > 1 && a->workspace != nullptr && a->workspace_bytes >= pl.bytes && aligned16(a->workspace)) {
    p.ksplit = pl.S;
    p.nkb /= pl.S;
    p.slice_elems = a->M * a->N;
    p.d = a->workspace;
    p.ldd = a->N;
    int rc;
    if (bn == 256) rc = launch_gemm<256, 128, true>(a, p, st);
    else if (bn == 192) rc = g1 ? launch_gemm<192, 1, true>(a, p, st) : launch_gemm<192, 128, true>(a, p, st);
    else rc = g1 ? launch_gemm<128, 1, true>(a, p, st) : launch_gemm<128, 128, true>(a, p, st);
    if (rc != TG_OK) return rc;
    const long long quads = a->M * (a->N / 4);
    const int blocks = int(quads / 256 + 1 < 4096 ? quads / 256 + 1 : 4096);
    if (f32)
      splitk_reduce_kernel<true><<<blocks, 256, 0, st>>>(static_cast<const float*>(a->workspace), a->d, int(a->M),
                                                         int(a->N), a->ldd, pl.S, p.slice_elems);
    else
      splitk_reduce_kernel<false><<<blocks, 256, 0, st>>>(static_cast<const float*>(a->workspace), a->d, int(a->M),
                                                          int(a->N), a->ldd, pl.S, p.slice_elems);
    TG_CUDA_CHECK(cudaGetLastError());
    return TG_OK;
  }
  if (wide) return f32 ? launch_gemm<256, 128, true>(a, p, st) : launch_gemm<256, 128, false>(a, p, st);
  if (bn == 192 && g1) return f32 ? launch_gemm<192, 1, true>(a, p, st) : launch_gemm<192, 1, false>(a, p, st);
  if (bn == 192) return f32 ? launch_gemm<192, 128, true>(a, p, st) : launch_gemm<192, 128, false>(a, p, st);
  if (g1) return f32 ? launch_gemm<128, 1, true>(a, p, st) : launch_gemm<128, 1, false>(a, p, st);
  return f32 ? launch_gemm<128, 128, true>(a, p, st) : launch_gemm<128, 128, false>(a, p, st);
}

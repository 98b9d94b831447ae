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
// Warp roles in the CTA (persistent, one CTA per SM; work items numbered in bands, see tile_coords):
//   warps 0..P-1 promotion + epilogue (P = 16, or 12 for 192-column tiles); warp w may touch TMEM
//                lanes 32*(w%4).. (a hardware rule) and owns accumulator columns (BN/4)*(w/4)..;
//                four warps per scheduler hide each other's TMEM-load latency.  Tiles leave through
//                bulk tensor stores (registers -> the warp's swizzled staging rows ->
//                cp.async.bulk.tensor, one box per 128 bytes of row), waited for only when the rows
//                are reused a tile later.
//   warp P       TMA producer: A (one 128 x 128-byte box) and B (BN/128 boxes), 128B swizzle
//   warp P+1     MMA issuer (owns the TMEM allocation): one lane-split barrier wait per block
//   warps P+2,3  (256-column tiles only) idle padding of the producer's warpgroup, so that it can
//                release registers to the promotion warpgroups with setmaxnreg: 96 -> 40 / 104.
//
// The loops of all three roles carry their state (stage, buffer, phase, scale offsets) instead of
// deriving it from a block counter, and the barriers live in static shared memory, so that a block
// costs the promotion warps little more than its 32 packed FMAs and 4 TMEM loads: the first builds
// spent four fifths of their instructions on address arithmetic and were bound by issue.
//
// Operand orientation is data, not code: the TMA box is 128 bytes x 128 rows for both
// K-major and MN-major storage (only the coordinates swap), and the shared-memory operand
// descriptors / instruction descriptor carry the major-ness, so dgrad and wgrad read the
// same buffers the forward wrote, untransposed.  Few output tiles with a long contraction are
// cut along the contraction (plan_split); few rows against a wide weight run with the operands
// swapped (plan_skinny).
//
// Every wait on an mbarrier is bounded: when the limit runs out the waiting role raises a
// CTA-wide abort flag, stores a code in *status, and all roles fall through to the common
// teardown (TMEM is always freed).
#include <cuda.h>

#include "common.cuh"
#include "mbarrier.cuh"

#ifndef TG_X_BAND
#define TG_X_BAND 16
#endif
#ifndef TG_X_PROMO_REGS
#define TG_X_PROMO_REGS 104
#endif
#ifndef TG_X_SERVICE_REGS
#define TG_X_SERVICE_REGS 40
#endif

namespace tg {

constexpr int BM = 128;          // tile rows (TMEM lanes)
constexpr int BK = 128;          // contraction block = scale granularity (fp8.py:27)
constexpr int UMMA_K = 32;       // K of one tcgen05.mma.kind::f8f6f4
constexpr int kTmemCols = 512;
constexpr int kTileBytes = 128 * 128;            // one operand TMA box: 128 rows x 128 bytes
constexpr int kSmemLimit = 227 * 1024;
constexpr int kBandRows = TG_X_BAND;             // tile rows per band of the tile numbering (see tile_coords)

// Compile-time plan of one kernel variant.
template <int BN_, int SB_GRAN, bool OUT_F32>
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
  static constexpr int promo_regs = TG_X_PROMO_REGS, service_regs = TG_X_SERVICE_REGS;
  static_assert(service_regs + 4 * promo_regs <= 5 * 96, "register hand-over asks for more than is released");
  static constexpr int tmem_bufs = BN > 128 ? 2 : 4;
  static constexpr int tmem_stride = kTmemCols / tmem_bufs;   // columns between accumulator buffers
  static constexpr int cols_per_warp = BN / (promo_warps / 4);  // 64 or 32
  static constexpr int b_boxes = (BN + 127) / 128;
  static constexpr int stage_bytes = kTileBytes * (1 + b_boxes);
  static constexpr int esize = OUT_F32 ? 4 : 2;
  // epilogue: a warp stages its 32 rows x `phase_cols` columns at a time (rows of <= 128
  // bytes; a fourth pipeline stage bought with narrower staging rows measured no faster)
  static constexpr int row_bytes = cols_per_warp * esize;     // 64, 128 or 256
  static constexpr int phase_cap = 128;
  static constexpr int phase_row_bytes = row_bytes < phase_cap ? row_bytes : phase_cap;
  static constexpr int phases = row_bytes / phase_row_bytes;
  static constexpr int phase_cols = phase_row_bytes / esize;
  // tiles leave through bulk tensor stores: per promotion warp one 32-row box for bf16 (never waited
  // for inside the tile loop), two for float32 through the same staging rows
  static constexpr int warp_out_bytes = 32 * phase_row_bytes;
  static constexpr int out_bytes = promo_warps * warp_out_bytes;
  // per-column scales: float[warps][2][cols_per_warp column scales + 32 row scales], double-buffered
  static constexpr int sc_slot = cols_per_warp + 32;
  static constexpr int sb_bytes = SB_GRAN == 1 ? promo_warps * 2 * sc_slot * 4 : 0;
  // 64-column warps with per-column scales read TMEM in the MMA fragment layout (a thread holds 4 rows
  // x 16 columns instead of 1 x 64): a column scale is then shared by 8 lanes instead of all 32, and
  // the block's 64 of them cost 8 conflict-free 8-byte reads per thread instead of 16 broadcasts of 16
  // bytes, which a warp is served a quarter at a time (64 -> 16 shared-memory wavefronts per warp)
  static constexpr bool frag = SB_GRAN == 1 && cols_per_warp == 64;
  // the barriers, the TMEM pointer and the abort flag are static shared memory (fixed addresses: the
  // loops address them with immediates); the dynamic part starts at the next 1024-byte boundary
  static constexpr int static_reserve = 1024;
  static constexpr int stages_fit = (kSmemLimit - static_reserve - out_bytes - sb_bytes) / stage_bytes;
  static constexpr int stages = stages_fit > 6 ? 6 : stages_fit;
  // offsets from the 1024-aligned base of dynamic shared memory
  static constexpr int off_out = stages * stage_bytes;
  static constexpr int off_sb = off_out + out_bytes;
  // (handing the wide accumulator over in two 128-column halves, each with its own barriers
  // and N=128 MMAs, was tried: 7 % slower -- A is read twice and twice as many MMAs issue)
  // With one staging phase per tile and idle warps to spare, one of them issues the tile's bulk
  // stores: the copy engine accepts a promotion warp's 4 KB box only after the boxes before it (a
  // 64 KB tile takes it ~1000 cycles at the SM's write bandwidth), and the sixteen warps used to sit
  // in that queue instead of draining the next tile's accumulators.
  static constexpr bool store_warp_on = regsteal && phases == 1;
  static constexpr int store_warp = promo_warps + 2;
  static constexpr int n_bars = 2 * stages + 2 * tmem_bufs + 1 + 2;
  static constexpr int smem_bytes = off_sb + sb_bytes;       // dynamic shared memory
  static_assert(n_bars <= 24, "control block too small");
  static_assert(stages >= 3, "pipeline too shallow");
  static_assert(smem_bytes + static_reserve <= kSmemLimit, "shared-memory plan exceeds the 227 KB a CTA may use");
};

struct GemmParams {
  const float* sa;
  long long sa_sm, sa_sk;
  int sa_shift;         // SA is indexed by (row >> sa_shift): 0 = a scale per row, 7 = one per 128 rows
  const float* sb;
  long long sb_sn, sb_sk;
  void* d;              // output, row pitch ldd elements
  long long ldd;
  int M, N, nkb;        // nkb = contraction blocks per work item (all of them unless the contraction is split)
  int nkb_rem;          // ... plus one for the first nkb_rem ranges of a split contraction (ranges need not be equal)
  int a_mn, b_mn;       // 1 = MN-major storage
  int tiles_m, tiles_n;
  int band;             // tile rows per band of the tile numbering
  // ceil(2^40 / d) for the three divisors of the item -> tile arithmetic (tiles per contraction range,
  // tiles per band, rows of the last band), 0 = divide the slow way (the exactness bound x * d < 2^40
  // does not hold); rows of a full band = `band`, its reciprocal in mg_band
  unsigned long long mg_tiles, mg_per_band, mg_band, mg_last;
  int ksplit;           // the contraction is cut into this many ranges; range s of a tile is its own
                        // work item and writes its float32 partial sums to d + s * slice_elems
  long long slice_elems;
  unsigned* status;
};

// ---- PTX wrappers ----------------------------------------------------------------------

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Bulk tensor store of one box from shared memory; completion is tracked by the issuing thread's
// bulk async-group, so the same lane must commit and later wait.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_3d_nocommit(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
// returns once every bulk store this thread committed has finished READING shared memory
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
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

// Staging stores of the epilogue, address = (base + OFF) ^ flip with OFF a compile-time constant.
// The address is formed inside the asm block so that the compiler cannot hoist one register per
// store out of the unrolled loops: the accumulators leave no room for that (it spilled loop
// invariants of the mainloop instead).  `base` has bits 4-6 clear or small enough that adding OFF
// never carries past bit 6, so the xor is the 128-byte swizzle of the 16-byte chunk index.
template <int OFF>
__device__ __forceinline__ void sts_swz_b32(uint32_t base, uint32_t flip, uint32_t x) {
  asm volatile("{\n\t.reg .b32 t;\n\tadd.u32 t, %0, %1;\n\txor.b32 t, t, %2;\n\tst.shared.b32 [t], %3;\n\t}"
               ::"r"(base), "n"(OFF), "r"(flip), "r"(x) : "memory");
}
// (float operands are passed as floats: routing accumulator halves through integer registers kept
// ptxas from leaving them in their packed pairs and cost ~25 spilled registers)
template <int OFF>
__device__ __forceinline__ void sts_swz_f32x2(uint32_t base, uint32_t flip, float2 v) {
  asm volatile("{\n\t.reg .b32 t;\n\tadd.u32 t, %0, %1;\n\txor.b32 t, t, %2;\n\tst.shared.v2.f32 [t], {%3, %4};\n\t}"
               ::"r"(base), "n"(OFF), "r"(flip), "f"(v.x), "f"(v.y) : "memory");
}
template <int OFF>
__device__ __forceinline__ void sts_swz_f32x4(uint32_t base, uint32_t flip, float2 v, float2 w) {
  asm volatile("{\n\t.reg .b32 t;\n\tadd.u32 t, %0, %1;\n\txor.b32 t, t, %2;\n\tst.shared.v4.f32 [t], {%3, %4, %5, %6};\n\t}"
               ::"r"(base), "n"(OFF), "r"(flip), "f"(v.x), "f"(v.y), "f"(w.x), "f"(w.y) : "memory");
}
template <int OFF>
__device__ __forceinline__ void sts_swz_v4(uint32_t base, uint32_t flip, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("{\n\t.reg .b32 t;\n\tadd.u32 t, %0, %1;\n\txor.b32 t, t, %2;\n\tst.shared.v4.b32 [t], {%3, %4, %5, %6};\n\t}"
               ::"r"(base), "n"(OFF), "r"(flip), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// ---- kernel ----------------------------------------------------------------------------

// which accumulator buffer a block uses: a constant, or the value of the carried counter
template <int B> struct StaticBuf { __device__ static constexpr uint32_t get(uint32_t) { return uint32_t(B); } };
struct DynBuf { __device__ static uint32_t get(uint32_t b) { return b; } };

// f(integral_constant<int, 0>) ... f(integral_constant<int, N-1>): a loop whose index is a constant
// expression inside the body (template arguments, "n" asm operands)
template <int I> struct IntC { static constexpr int value = I; };
template <int N, int I = 0, typename F>
__device__ __forceinline__ void static_loop(F&& f) {
  if constexpr (I < N) {
    f(IntC<I>{});
    static_loop<N, I + 1>(f);
  }
}

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

// Work item -> tile coordinates.  Tiles are numbered in bands of `band` tile rows; inside a band
// the numbering runs down the rows first, then across the columns, so that the CTAs of a wave
// (consecutive numbers) cover a near-square patch of the output: the A and B panels they fetch
// together are as few as possible, which is what keeps the operands' L2 lines alive between the
// CTAs that share them.  (Row-major numbering made a 148-CTA wave touch every B panel of a
// 24-tile-wide problem plus 7 A panels; in bands of 16 it touches 16 + 10.)
// x / d through a multiplication by mg = ceil(2^40 / d): exact while x * d < 2^40 (the host checks
// and passes 0 otherwise).  A 32-bit division by a run-time value costs ~20 dependent instructions,
// and every role does three of them at each tile boundary.
__device__ __forceinline__ int fast_div(int x, int d, unsigned long long mg) {
  return mg != 0 ? int((static_cast<unsigned long long>(static_cast<unsigned>(x)) * mg) >> 40) : x / d;
}
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& tm, int& tn) {
  const int per_band = p.band * p.tiles_n;
  const int b = fast_div(tile, per_band, p.mg_per_band), w = tile - b * per_band;
  const int left = p.tiles_m - b * p.band;
  const bool full = left >= p.band;
  const int rows = full ? p.band : left;
  tn = fast_div(w, rows, full ? p.mg_band : p.mg_last);
  tm = b * p.band + (w - tn * rows);
}
// work item -> (contraction range, tile)
__device__ __forceinline__ void item_split(const GemmParams& p, int item, int n_tiles, int& ks, int& tile) {
  ks = fast_div(item, n_tiles, p.mg_tiles);
  tile = item - ks * n_tiles;
}
// contraction range -> its first block and its number of blocks
__device__ __forceinline__ int range_blocks(const GemmParams& p, int ks) { return p.nkb + (ks < p.nkb_rem ? 1 : 0); }
__device__ __forceinline__ int range_first(const GemmParams& p, int ks) { return ks * p.nkb + min(ks, p.nkb_rem); }

template <int BN_, int SB_GRAN, bool OUT_F32>
__global__ void __launch_bounds__((Cfg<BN_, SB_GRAN, OUT_F32>::threads), 1)
gemm_fp8_blockscaled_kernel(const __grid_constant__ CUtensorMap tmap_a,
                            const __grid_constant__ CUtensorMap tmap_b,
                            const __grid_constant__ CUtensorMap tmap_d, const GemmParams p) {
  using C = Cfg<BN_, SB_GRAN, OUT_F32>;
  constexpr int BN = C::BN, kStages = C::stages, kTmemBufs = C::tmem_bufs, kCols = C::cols_per_warp;
  constexpr int kPromoWarps = C::promo_warps;
  // operand stages (1024-byte aligned for the 128-byte swizzle), output staging, scale staging
  extern __shared__ __align__(1024) uint8_t smem[];
  // barriers, 8 bytes each: full[kStages], empty[kStages], tfull[kTmemBufs], tempty[kTmemBufs], drain, staged, unstaged
  __shared__ __align__(16) uint64_t ctl_bars[24];
  __shared__ uint32_t ctl_tmem_ptr;
  __shared__ int ctl_abort;
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = smem_u32(ctl_bars);
  const uint32_t full0 = bar0, empty0 = bar0 + 8u * kStages;
  const uint32_t tfull0 = bar0 + 16u * kStages, tempty0 = tfull0 + 8u * kTmemBufs;
  const uint32_t drain_bar = tempty0 + 8u * kTmemBufs;
  const uint32_t staged_bar = drain_bar + 8u, unstaged_bar = drain_bar + 16u;   // the store warp's pair (see Cfg::store_warp_on)
  volatile uint32_t* tmem_ptr_smem = &ctl_tmem_ptr;
  volatile int* abort_flag = &ctl_abort;
  if ((sbase & 1023u) != 0) {   // the swizzled operand layout needs this alignment; never seen, but not assumed
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0u, 6u);
    return;
  }

  // the warp index through a shuffle: the compiler then knows it is the same in every lane and keeps
  // what derives from it (role, TMEM address, barrier addresses) in uniform registers
  const int warp = __shfl_sync(0xffffffffu, int(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int n_tiles = p.tiles_m * p.tiles_n;
  const int n_items = n_tiles * p.ksplit;     // work item i = (tile i % n_tiles, contraction range i / n_tiles)
  const int first_item = int(blockIdx.x), item_step = int(gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8u * s, 1);
      mbar_init(empty0 + 8u * s, 1);
    }
    for (int b = 0; b < kTmemBufs; ++b) {
      mbar_init(tfull0 + 8u * b, 1);
      mbar_init(tempty0 + 8u * b, kPromoWarps);
    }
    mbar_init(drain_bar, 1);
    mbar_init(staged_bar, kPromoWarps);
    mbar_init(unstaged_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_b)) : "memory");
  }
  if (warp == C::issuer_warp) {
    tmem_alloc(smem_u32(&ctl_tmem_ptr), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp >= C::promo_warps) {
    if (C::regsteal) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::service_regs));
    if (warp == C::producer_warp) {
      // ------------------------------ TMA producer -------------------------------------
      // The whole warp walks the loop (uniform control flow); one elected lane issues.  Stage index
      // and phase are carried, not derived from a block counter (no modulo in the loop).
      uint32_t s = 0, ph = 1;                 // the first pass over the stages finds them all free
      bool ok = true;
      for (int item = first_item; ok && item < n_items; item += item_step) {
        int ks, tile, tm, tn;
        item_split(p, item, n_tiles, ks, tile);
        tile_coords(p, tile, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        int k0 = range_first(p, ks) * BK;
        const int nkb = range_blocks(p, ks);
        for (int kb = 0; kb < nkb; ++kb, k0 += BK) {
          ok = __all_sync(0xffffffffu, mbar_wait(empty0 + 8u * s, ph, abort_flag, p.status, 1u));
          if (!ok) break;
          if (elect_one()) {
            const uint32_t dst = sbase + s * C::stage_bytes, fb = full0 + 8u * s;
            mbar_expect_tx(fb, C::stage_bytes);
            tma_load_2d(dst, &tmap_a, fb, p.a_mn ? m0 : k0, p.a_mn ? k0 : m0);
#pragma unroll
            for (int b = 0; b < C::b_boxes; ++b) {
              const int nb = n0 + b * 128;  // a box wholly past N is still loaded: it arrives as zeros
              tma_load_2d(dst + (1 + b) * kTileBytes, &tmap_b, fb, p.b_mn ? nb : k0, p.b_mn ? k0 : nb);
            }
          }
          __syncwarp();
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
      }
    } else if (warp == C::issuer_warp) {
      // ------------------------------ MMA issuer ---------------------------------------
      // Blocks are independent: each has its own TMEM buffer and shared-memory stage.
      // instruction descriptor: D f32 (bit 4), A/B e4m3 (0), major bits 15/16, N>>3 at 17, M>>4 at 24
      const uint32_t idesc = (1u << 4) | (uint32_t(p.a_mn) << 15) | (uint32_t(p.b_mn) << 16) |
                             (uint32_t(BN >> 3) << 17) | (uint32_t(BM >> 4) << 24);
      // descriptor start-address step per UMMA_K: 32 bytes along a K-major row, 32 rows of 128 B otherwise
      const uint32_t a_step = p.a_mn ? (UMMA_K * 128) >> 4 : UMMA_K >> 4;
      const uint32_t b_step = p.b_mn ? (UMMA_K * 128) >> 4 : UMMA_K >> 4;
      // a descriptor's low word holds (address >> 4) in 14 bits: shared memory ends below 2^18, so
      // adding block offsets to the low word never carries out of the field
      const uint64_t desc_a0 = make_smem_desc(sbase), desc_b0 = make_smem_desc(sbase + kTileBytes);
      const uint32_t desc_hi = uint32_t(desc_a0 >> 32);
      const uint32_t a_lo0 = uint32_t(desc_a0), b_lo0 = uint32_t(desc_b0);
      uint32_t total = 0;                     // contraction blocks of all this block's work items
      for (int item = first_item; item < n_items; item += item_step) {
        int ks, tile;
        item_split(p, item, n_tiles, ks, tile);
        total += uint32_t(range_blocks(p, ks));
      }
      bool ok = true;
      // A barrier operation has tens of cycles of latency even when the barrier is already complete,
      // and this loop is a chain of them: it does ONE wait instruction per block, lanes 0-15 polling
      // the accumulator buffer's barrier and lanes 16-31 the stage's.
      const bool stage_lane = lane >= 16;
      uint32_t s = 0, sph = 0, buf = 0, bph = 1, soff = 0;
      for (uint32_t it = 0; ok && it < total; ++it) {
        const uint32_t bar = stage_lane ? full0 + 8u * s : tempty0 + 8u * buf;
        const uint32_t par = stage_lane ? sph : bph;
        ok = __all_sync(0xffffffffu, mbar_wait(bar, par, abort_flag, p.status, stage_lane ? 3u : 2u));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          const uint32_t d_tmem = tmem_base + buf * uint32_t(C::tmem_stride);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f8(d_tmem, (uint64_t(desc_hi) << 32) | (a_lo0 + soff + k * a_step),
                    (uint64_t(desc_hi) << 32) | (b_lo0 + soff + k * b_step), idesc, k > 0 ? 1u : 0u);
          umma_commit(empty0 + 8u * s);      // shared-memory stage free once these MMAs retire
          umma_commit(tfull0 + 8u * buf);    // accumulator buffer ready for promotion
        }
        __syncwarp();
        soff += uint32_t(C::stage_bytes >> 4);
        if (++s == kStages) { s = 0; sph ^= 1u; soff = 0; }
        if (++buf == kTmemBufs) { buf = 0; bph ^= 1u; }
      }
      // make sure nothing issued here is still running when TMEM is freed
      if (elect_one()) {
        umma_commit(drain_bar);
        mbar_wait(drain_bar, 0u, abort_flag, p.status, 4u);
      }
      __syncwarp();
    } else if (C::store_warp_on && warp == C::store_warp) {
      // ------------------------------ tile store issuer -----------------------------------
      // Per tile: wait until all promotion warps have staged their rows, hand the sixteen boxes to the
      // copy engine, wait until it has read them, give the staging rows back.
      uint32_t sph = 0;
      for (int item = first_item; item < n_items; item += item_step) {
        int ks, tile, tm, tn;
        item_split(p, item, n_tiles, ks, tile);
        tile_coords(p, tile, tm, tn);
        if (!__all_sync(0xffffffffu, mbar_wait(staged_bar, sph, abort_flag, p.status, 7u))) break;
        sph ^= 1u;
        if (elect_one()) {
#pragma unroll 1
          for (int w = 0; w < kPromoWarps; ++w)
            tma_store_3d_nocommit(&tmap_d, sbase + C::off_out + uint32_t(w) * C::warp_out_bytes, tn * BN + (w >> 2) * kCols,
                                  tm * BM + (w & 3) * 32, ks);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          tma_store_wait_read();
          mbar_arrive(unstaged_bar);
        }
        __syncwarp();
      }
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
    bool ok = true;

    // The promotion loop is bound by instruction issue (four such warps share a scheduler, and per
    // block each has 32 packed FMAs and four TMEM loads of payload), so everything else in it is
    // carried incrementally: the accumulator buffer's barrier addresses, TMEM address and phase
    // are toggled, the scale pointers are bumped, and rows / columns outside the problem read a
    // clamped (valid) address instead of being predicated off.
    uint32_t buf = 0, bph = 0, uph = 0;
    const uint32_t tcol0 = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(c0);

    // Per-tile state is ONE register pair of scale offsets, set one tile ahead so that the first scale
    // loads are in flight during the previous tile's epilogue; the epilogue derives the tile's
    // coordinates from the item number again rather than keeping them live through the loop.
    uint32_t sa_off = 0, sb_off = 0;           // element offsets into p.sa / p.sb (the host checks they fit 32 bits)
    // The scales of block k+1 are loaded at the top of block k's iteration, by volatile asm so
    // that the compiler cannot sink the loads to their use: with ordinary loads it did, and clock64
    // stamps showed ~450 cycles of exposed L2 latency per block in these warps.
    float sa_q0 = 0.f;
    float2 sb_q0 = make_float2(0.f, 0.f);
    // per-column scales: lane j stages column c0 + j (32-column warps) or the pair c0 + 2j, c0 + 2j + 1
    constexpr int kPerLane = kCols / 32;
    // One scale per 128 columns: its address changes line with every block, so a load per block
    // misses L1 every time and the loop would run at one L2 round trip per block.  Instead lane l
    // fetches the scale of block 32 g + l once per 32 blocks and a shuffle hands each block its value.
    float sb_grp = 0.f, sb_nxt = 0.f;
    int open_nkb = p.nkb;          // contraction blocks of the work item opened last (ranges of a split need not be equal)
    auto load_sb_lane = [&](int g) {
      float v = 0.f;
      const int kb = 32 * g + lane;
      if (kb < open_nkb) v = ldg_f32(p.sb + sb_off + uint32_t(kb) * uint32_t(p.sb_sk));
      return v;
    };
    auto load_sb_cols = [&]() {     // per-column scales of the block sb_off points at
      float2 v;
      v.x = ldg_f32(p.sb + sb_off);
      v.y = kPerLane == 2 ? ldg_f32(p.sb + sb_off + uint32_t(p.sb_sn)) : 0.f;
      return v;
    };
    auto open_tile = [&](int item) {
      int ks, tile, tm, tn;
      item_split(p, item, n_tiles, ks, tile);
      const uint32_t kb_off = uint32_t(range_first(p, ks));
      open_nkb = range_blocks(p, ks);
      tile_coords(p, tile, tm, tn);
      const int n0 = tn * BN;
      const int m = min(tm * BM + r, p.M - 1);       // rows past M: a valid scale, results never stored
      sa_off = uint32_t(m >> p.sa_shift) * uint32_t(p.sa_sm) + kb_off * uint32_t(p.sa_sk);
      if (SB_GRAN == 1) {
        const int col = min(n0 + c0 + kPerLane * lane, p.N - kPerLane);   // N % 8 == 0: a pair is in or out together
        sb_off = uint32_t(col) * uint32_t(p.sb_sn) + kb_off * uint32_t(p.sb_sk);
        sb_q0 = load_sb_cols();
        sb_off += uint32_t(p.sb_sk);
      } else {                                       // one scale per 128 columns
        const int nblk = min((n0 + c0) / 128, (p.N - 1) / 128);
        sb_off = uint32_t(nblk) * uint32_t(p.sb_sn) + kb_off * uint32_t(p.sb_sk);
        sb_grp = load_sb_lane(0);
      }
      sa_q0 = ldg_f32(p.sa + sa_off);
      sa_off += uint32_t(p.sa_sk);
    };
    const uint32_t is_lane0 = lane == 0;
    auto release = [&](uint32_t b) {   // every partial sum of the buffer is in registers: hand it back to the tensor core
      tc_fence_before();
      __syncwarp();
      mbar_arrive_if(tempty0 + 8u * b, is_lane0);     // predicated, no branch
    };

    if (first_item < n_items) open_tile(first_item);
    for (int item = first_item; item < n_items; item += item_step) {
      float2 acc[kCols / 2];
#pragma unroll
      for (int j = 0; j < kCols / 2; ++j) acc[j] = make_float2(0.f, 0.f);

      const int nkb = open_nkb;    // set when this item was opened (before the previous tile's epilogue)
      // One contraction block.  `bsel` says which accumulator buffer it drains: a compile-time constant
      // in the two-buffer variants (the block loop below is unrolled by two, so barrier addresses, TMEM
      // address and staging slot are immediates), the carried counter otherwise.
      auto do_block = [&](auto bsel, int kb) -> bool {
        const uint32_t b = bsel.get(buf);
        const float sa_v = sa_q0;
        float2 sb_v = sb_q0;
        const bool more = kb + 1 < nkb;
        if (more) sa_q0 = ldg_f32(p.sa + sa_off);
        sa_off += uint32_t(p.sa_sk);
        if (SB_GRAN == 1) {
          if (more) sb_q0 = load_sb_cols();
          sb_off += uint32_t(p.sb_sk);
        } else {
          const int kl = kb & 31;
          if (kl == 0) {
            if (kb != 0) sb_grp = sb_nxt;
            sb_nxt = load_sb_lane((kb >> 5) + 1);
          }
          sb_v.x = __shfl_sync(0xffffffffu, sb_grp, kl);
        }
        float* stage = sb_stage + (b & 1u) * C::sc_slot;      // two slots: consecutive blocks alternate
        if (SB_GRAN == 1) {
          if (kPerLane == 2) *reinterpret_cast<float2*>(stage + 2 * lane) = sb_v;
          else stage[lane] = sb_v.x;
          if (kFrag) stage[kCols + lane] = sa_v;   // row 32 * quarter + lane
          __syncwarp();
        }
        if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8u * b, bph, abort_flag, p.status, 5u))) return false;
        tc_fence_after();
        const uint32_t taddr = tcol0 + b * uint32_t(C::tmem_stride);
        const float s_scalar = sa_v * sb_v.x;
        if (kFrag) {
          // acc[(4 q + i) * 2 + k] holds rows fg + 8 i, columns 16 q + 8 k + 2 fj (+1)
          float sa_r[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) sa_r[i] = stage[kCols + fg + 8 * i];
          auto promote_piece = [&](const uint32_t (&cur)[16], int q) {
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
          };
          {
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
              promote_piece(cur, q);
              if (q < 3) tmem_wait_ld16(nxt);
              if (q == 2) release(b);        // every load of the buffer has landed
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
          release(b);
          promote<SB_GRAN, 16>(acc + 24, v, stage + 48, sa_v, s_scalar);
        } else {
          uint32_t v[32];
          tmem_ld32(taddr, v);
          tmem_wait_ld(v);
          release(b);
          promote<SB_GRAN, 32>(acc, v, stage, sa_v, s_scalar);
        }
        // keep this block's FMAs above the next block's first instructions (no instruction is emitted)
        if constexpr (kTmemBufs == 2 && !kFrag) {
#pragma unroll
          for (int j = 0; j < kCols / 2; ++j) asm volatile("" : "+f"(acc[j].x), "+f"(acc[j].y));
        }
        return true;
      };
      // (unrolling the per-column-scale variant measured 7-10 % slower: its blocks overlap better as a rolled loop)
      if constexpr (kTmemBufs == 2 && !kFrag) {
        int kb = 0;
        if (buf != 0) {                      // a previous tile ended on an odd block: drain buffer 1 first
          ok = do_block(StaticBuf<1>{}, kb++);
          buf = 0;
          bph ^= 1u;
        }
        for (; ok && kb + 1 < nkb; kb += 2) {
          ok = do_block(StaticBuf<0>{}, kb) && do_block(StaticBuf<1>{}, kb + 1);
          bph ^= 1u;
        }
        if (ok && kb < nkb) {
          ok = do_block(StaticBuf<0>{}, kb);
          buf = 1;
        }
      } else {
        for (int kb = 0; ok && kb < nkb; ++kb) {
          ok = do_block(DynBuf{}, kb);
          if (++buf == kTmemBufs) { buf = 0; bph ^= 1u; }
        }
      }
      if (!ok) break;   // aborting: every other role sees the flag in its own wait

      // start the next tile's first scale loads before the stores of this one
      if (item + item_step < n_items) open_tile(item + item_step);
      int tile_m0 = 0, tile_n0 = 0, tile_ks = 0;
      if constexpr (!C::store_warp_on) {
        int tile, tm, tn;
        item_split(p, item, n_tiles, tile_ks, tile);
        tile_coords(p, tile, tm, tn);
        tile_m0 = tm * BM;
        tile_n0 = tn * BN;
      }

      // ---- epilogue: registers -> this warp's swizzled staging rows -> bulk tensor stores ----------
      // The warp's 32 rows x kCols columns leave as one box per 128 bytes of row (one box for bf16,
      // two for float32).  Lane 0 hands a box to the copy engine and the warp goes straight on; the
      // wait for the engine to have read the staging rows comes only before they are overwritten
      // (for the first box of a tile that is one whole tile later).  Rows past M and columns past N
      // are clipped by the tensor map, whose third coordinate is the contraction slice.
      constexpr int PRB = C::phase_row_bytes;
      const uint32_t wb = sbase + C::off_out + uint32_t(pw) * C::warp_out_bytes;
      if constexpr (C::store_warp_on) {
        // the staging rows are free once the store warp's boxes of the tile before have been read
        // (a whole tile ago: this does not wait in practice); first tile: nothing to wait for
        if (item != first_item) {
          ok = __all_sync(0xffffffffu, mbar_wait(unstaged_bar, uph, abort_flag, p.status, 8u));
          if (!ok) break;
          uph ^= 1u;
        }
      }
#pragma unroll
      for (int ph = 0; ph < C::phases; ++ph) {
        if constexpr (!C::store_warp_on) {
          if (lane == 0) tma_store_wait_read();
        }
        __syncwarp();
        if (kFrag && OUT_F32) {
          // thread (fg, fj) holds rows fg + 8 i, columns 16 qq + 8 k + 2 fj (+1) of the phase: 16-byte chunk
          // 4 qq + 2 k + (fj >> 1), 8-byte half fj & 1
          const uint32_t fbase = wb + uint32_t(fg) * PRB + (uint32_t(fj >> 1) << 4) + 8u * uint32_t(fj & 1);
          const uint32_t flip = uint32_t(fg & 7) << 4;
          static_loop<2>([&](auto qq) {
            static_loop<4>([&](auto i) {
              static_loop<2>([&](auto k) {
                const float2 a = acc[(4 * (2 * ph + qq.value) + i.value) * 2 + k.value];
                sts_swz_f32x2<i.value * 8 * PRB + (4 * qq.value + 2 * k.value) * 16>(fbase, flip, a);
              });
            });
          });
        } else if (kFrag) {
          // rows fg + 8 i, 16-byte chunk 2 q + k, 4 fj bytes in
          const uint32_t fbase = wb + uint32_t(fg) * PRB + 4u * uint32_t(fj);
          const uint32_t flip = uint32_t(fg & 7) << 4;
          static_loop<4>([&](auto q) {
            static_loop<4>([&](auto i) {
              static_loop<2>([&](auto k) {
                const float2 a = acc[(4 * q.value + i.value) * 2 + k.value];
                sts_swz_b32<i.value * 8 * PRB + (2 * q.value + k.value) * 16>(fbase, flip, pack_bf16x2(a.x, a.y));
              });
            });
          });
        } else if (OUT_F32) {
          static_loop<PRB / 16>([&](auto c) {     // 4 floats per 16-byte chunk
            const int j = ph * (C::phase_cols / 2) + 2 * c.value;
            sts_swz_f32x4<c.value * 16>(out_base, uint32_t(swz) << 4, acc[j], acc[j + 1]);
          });
        } else {
          static_loop<PRB / 16>([&](auto c) {     // 8 bf16 per 16-byte chunk
            const int j = ph * (C::phase_cols / 2) + 4 * c.value;
            sts_swz_v4<c.value * 16>(out_base, uint32_t(swz) << 4, pack_bf16x2(acc[j].x, acc[j].y),
                                     pack_bf16x2(acc[j + 1].x, acc[j + 1].y), pack_bf16x2(acc[j + 2].x, acc[j + 2].y),
                                     pack_bf16x2(acc[j + 3].x, acc[j + 3].y));
          });
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the copy engine
        __syncwarp();
        if constexpr (C::store_warp_on) {
          mbar_arrive_if(staged_bar, is_lane0);
        } else {
          if (lane == 0) tma_store_3d(&tmap_d, wb, tile_n0 + c0 + ph * C::phase_cols, tile_m0 + quarter * 32, tile_ks);
        }
      }
    }
  }

  // ------------------------------ teardown ----------------------------------------------
  // the last bulk stores must have read their staging rows before the CTA's shared memory goes away
  if (!C::store_warp_on && warp < C::promo_warps && lane == 0) tma_store_wait_read();
  tc_fence_before();
  __syncthreads();
  if (warp == C::issuer_warp) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
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

template <int BN_, int SB_GRAN, bool OUT_F32>
static int launch_gemm(const tg_gemm_args* a, GemmParams p, cudaStream_t st) {
  using C = Cfg<BN_, SB_GRAN, OUT_F32>;
  auto kern = gemm_fp8_blockscaled_kernel<BN_, SB_GRAN, OUT_F32>;
  CUtensorMap ta, tb;
  const int64_t a_inner = p.a_mn ? a->M : a->K, a_outer = p.a_mn ? a->K : a->M;
  const int64_t b_inner = p.b_mn ? a->N : a->K, b_outer = p.b_mn ? a->K : a->N;
  if (int rc = make_tmap(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->a, a_inner, a_outer, a->lda, 128, 128)) return rc;
  if (int rc = make_tmap(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->b, b_inner, b_outer, a->ldb, 128, 128)) return rc;
  // output map: [contraction slice][row][column]; a launch that is not cut has one slice
  CUtensorMap td;
  {
    EncodeTiledFn enc;
    if (int rc = get_encode_fn(&enc)) return rc;
    const int esz = C::esize;
    cuuint64_t dims[3] = {cuuint64_t(a->N), cuuint64_t(a->M), cuuint64_t(p.ksplit)};
    cuuint64_t strides[2] = {cuuint64_t(p.ldd) * esz, cuuint64_t(p.ksplit > 1 ? p.slice_elems : a->M * p.ldd) * esz};
    cuuint32_t box[3] = {cuuint32_t(C::phase_cols), 32u, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    constexpr int span = C::phase_row_bytes;
    CUresult r = enc(&td, OUT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, p.d, dims, strides,
                     box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     span == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : span == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled (output)");
  }
  p.tiles_m = int((a->M + BM - 1) / BM);
  p.tiles_n = int((a->N + BN_ - 1) / BN_);
  p.band = p.tiles_m < kBandRows ? p.tiles_m : kBandRows;
  const int64_t n_items = int64_t(p.tiles_m) * p.tiles_n * p.ksplit;
  {
    // reciprocals for the kernel's item -> tile arithmetic: q = (x * ceil(2^40 / d)) >> 40 is x / d
    // for every x <= x_max when x_max * d < 2^40
    auto magic = [](int64_t x_max, int64_t d) -> unsigned long long {
      if (d <= 0 || x_max >= (int64_t(1) << 31) || x_max * d >= (int64_t(1) << 40)) return 0ull;
      return ((1ull << 40) + uint64_t(d) - 1) / uint64_t(d);
    };
    const int64_t n_tiles = int64_t(p.tiles_m) * p.tiles_n, per_band = int64_t(p.band) * p.tiles_n;
    const int64_t last_rows = p.tiles_m % p.band;
    p.mg_tiles = magic(n_items, n_tiles);
    p.mg_per_band = magic(n_tiles, per_band);
    p.mg_band = magic(per_band, p.band);
    p.mg_last = last_rows > 0 ? magic(per_band, last_rows) : 0ull;
  }
  if (n_items > INT32_MAX || n_items * (p.nkb + 1) > INT32_MAX) return TG_ERR_TOO_LARGE;
  const int sms = gemm_sms();
  const int grid = int(n_items < sms ? n_items : sms);
  // the attribute is per device: set it once for each device this instantiation runs on
  static bool attr_set[64] = {};
  int dev = 0;
  TG_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TG_ERR_SHAPE;
  if (!attr_set[dev]) {
    TG_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::smem_bytes));
    attr_set[dev] = true;
  }
  kern<<<grid, C::threads, C::smem_bytes, st>>>(ta, tb, td, p);
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

// The same reduction for a problem that ran with its operands swapped (see plan_skinny): the slices
// hold D^T, [S][N][pitch] float32 with the M tokens along the fast axis; the output is D [M][ldd].
// One block transposes a 32 x 32 patch through shared memory so that reads and writes both coalesce.
template <bool OUT_F32>
__global__ void __launch_bounds__(256)
splitk_reduce_transpose_kernel(const float* __restrict__ ws, void* __restrict__ d, int M, int N, long long ldd, int S,
                               long long slice_elems, int pitch) {
  __shared__ float tile[32][33];
  const int n0 = blockIdx.x * 32, m0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 32 x 8
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int n = n0 + ty + 8 * i, m = m0 + tx;
    float acc = 0.f;
    if (n < N && m < M) {
      const float* q = ws + (long long)n * pitch + m;
      acc = q[0];
      for (int sl = 1; sl < S; ++sl) acc += q[sl * slice_elems];
    }
    tile[ty + 8 * i][tx] = acc;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty + 8 * i, n = n0 + tx;
    if (n < N && m < M) {
      const float v = tile[tx][ty + 8 * i];
      if (OUT_F32) static_cast<float*>(d)[(long long)m * ldd + n] = v;
      else static_cast<__nv_bfloat16*>(d)[(long long)m * ldd + n] = __float2bfloat16_rn(v);
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
  const int sms = gemm_sms();
  if (sms <= 0) return pl;
  // S ranges of nkb / S blocks, the first nkb % S of them one longer; the longest sets the pace of a wave
  double best = 0.0;
  for (int S = 1; S <= 8; ++S) {
    if (S > 1 && nkb / S < 8) break;
    const int64_t waves = (tiles * S + sms - 1) / sms;
    double cost = double(waves) * (double((nkb + S - 1) / S) + 3.0);
    if (S > 1) cost += double(4 * S + 2) * double(a->M) * double(a->N) / 4.0e6;
    if (S == 1 || cost < best * 0.98) { best = cost; pl.S = S; }
  }
  if (pl.S > 1) pl.bytes = int64_t(pl.S) * a->M * a->N * int64_t(sizeof(float));
  return pl;
}

// ---- few tokens, wide weight ---------------------------------------------------------------
// With M <= 128 rows a 128-row MMA tile is mostly dead rows and there are only N / 256 output tiles
// for 148 SMs, while the whole job is one pass over the weight (K x N bytes): it is bound by HBM, not by
// the tensor core.  Such a problem runs TRANSPOSED: the weight's N becomes the MMA's 128-row dimension
// (no dead rows, N / 128 tiles), the M tokens its 128 columns, the contraction is cut so that every SM
// streams its own piece of the weight, and the float32 partial sums of D^T are added and transposed
// back by splitk_reduce_transpose_kernel.  The per-token scales become per-column scales, the weight's
// scales per-row (one per 128 rows for 128 x 128 weight tiles).  Measured at K = N = 8192 (CUDA-graph
// replays): M = 16 20.6 us against 29.6 us the ordinary way (3.3 against 2.3 TB/s of weight stream),
// M = 64 22.8 / 30.3, M = 128 27.2; from M = 192 on the ordinary tiling is faster (37 against ~33 us).
struct SkinnyPlan {
  bool on;
  int bn;            // tile width over the tokens
  int S;             // contraction ranges
  int pitch;         // row pitch of a D^T slice, in floats
  int64_t bytes;     // workspace
};

static SkinnyPlan plan_skinny(const tg_gemm_args* a) {
  SkinnyPlan pl = {false, 0, 1, 0, 0};
  if (a->M > 128 || a->M % 8 != 0 || a->N < 1024 || a->K % BK != 0 || a->K < 1024) return pl;
  if (a->a_major != TG_MAJOR_K) return pl;          // the activation must be [M][K]: it becomes the K-major B operand
  const int sms = gemm_sms();
  if (sms <= 0) return pl;
  pl.on = true;
  pl.bn = 128;
  const int64_t tiles = ((a->N + BM - 1) / BM) * ((a->M + pl.bn - 1) / pl.bn);
  const int64_t nkb = a->K / BK;
  while (pl.S < 8 && tiles * pl.S < sms && nkb % (2 * pl.S) == 0 && nkb / (2 * pl.S) >= 4) pl.S *= 2;
  pl.pitch = int((a->M + 3) / 4 * 4);
  pl.bytes = int64_t(pl.S) * a->N * pl.pitch * int64_t(sizeof(float));
  return pl;
}

}  // namespace tg

using namespace tg;

// Tile width of a problem.  One scale per 128 columns: 128 x 256 tiles, 16 promotion warps
// (measured 1.70 / 1.92 PFLOP/s forward / dgrad against 1.53 / 1.59 for 128 x 192).  A scale per
// column (the weight gradient): 128 x 192 tiles with 12 promotion warps, whose 128 registers per
// thread hold the 64 accumulator columns plus the scale staging that 96 do not (1.04 PFLOP/s
// against 0.85 for 128 x 128).
static int tile_width(const tg_gemm_args* a) {
  if (a->N <= 128) return 128;
  return a->sb_gran_n == 1 ? 192 : 256;
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
  const SkinnyPlan sk = plan_skinny(a);
  if (sk.on) return sk.bytes;
  return plan_split(a, tile_width(a)).bytes;
}

// The transposed run of a few-token problem (plan_skinny): D^T = B A^T into the workspace, then reduce + transpose.
static int run_skinny(const tg_gemm_args* a, const SkinnyPlan& sk, cudaStream_t st) {
  tg_gemm_args t = *a;
  t.a = a->b; t.lda = a->ldb; t.a_major = a->b_major;
  t.b = a->a; t.ldb = a->lda; t.b_major = a->a_major;
  t.M = a->N; t.N = a->M;
  GemmParams p;
  p.sa = a->sb; p.sa_sm = a->sb_stride_n; p.sa_sk = a->sb_stride_kb; p.sa_shift = a->sb_gran_n == 128 ? 7 : 0;
  p.sb = a->sa; p.sb_sn = a->sa_stride_m; p.sb_sk = a->sa_stride_kb;
  p.d = a->workspace; p.ldd = sk.pitch;
  p.M = int(t.M); p.N = int(t.N); p.nkb = int(a->K / BK) / sk.S;
  p.nkb_rem = 0;
  p.a_mn = t.a_major == TG_MAJOR_MN; p.b_mn = false;
  p.tiles_m = p.tiles_n = 0;
  p.band = 1;
  p.ksplit = sk.S;
  p.slice_elems = t.M * sk.pitch;
  p.status = a->status;
  const int rc = launch_gemm<128, 1, true>(&t, p, st);
  if (rc != TG_OK) return rc;
  const dim3 grid(unsigned((a->N + 31) / 32), unsigned((a->M + 31) / 32));
  if (a->out_dtype == TG_OUT_F32)
    splitk_reduce_transpose_kernel<true><<<grid, 256, 0, st>>>(static_cast<const float*>(a->workspace), a->d, int(a->M), int(a->N),
                                                                  a->ldd, sk.S, p.slice_elems, sk.pitch);
  else
    splitk_reduce_transpose_kernel<false><<<grid, 256, 0, st>>>(static_cast<const float*>(a->workspace), a->d, int(a->M), int(a->N),
                                                                   a->ldd, sk.S, p.slice_elems, sk.pitch);
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
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
  {
    // the kernel walks the scale arrays with 32-bit element offsets
    const int64_t nkb_all = (a->K + BK - 1) / BK;
    const int64_t n_sb = a->sb_gran_n == 1 ? a->N : (a->N + 127) / 128;
    if (a->sa_stride_m < 0 || a->sa_stride_kb < 0 || a->sb_stride_n < 0 || a->sb_stride_kb < 0) return TG_ERR_SHAPE;
    if (a->M * a->sa_stride_m + nkb_all * a->sa_stride_kb > INT32_MAX ||
        n_sb * a->sb_stride_n + nkb_all * a->sb_stride_kb > INT32_MAX)
      return TG_ERR_TOO_LARGE;
  }
  {
    const SkinnyPlan sk = plan_skinny(a);
    if (sk.on && a->workspace != nullptr && a->workspace_bytes >= sk.bytes && aligned16(a->workspace))
      return run_skinny(a, sk, st);
  }
  GemmParams p;
  p.sa = a->sa; p.sa_sm = a->sa_stride_m; p.sa_sk = a->sa_stride_kb; p.sa_shift = 0;
  p.sb = a->sb; p.sb_sn = a->sb_stride_n; p.sb_sk = a->sb_stride_kb;
  p.d = a->d; p.ldd = a->ldd;
  p.M = int(a->M); p.N = int(a->N); p.nkb = int((a->K + BK - 1) / BK);
  p.nkb_rem = 0;
  p.a_mn = a->a_major == TG_MAJOR_MN; p.b_mn = a->b_major == TG_MAJOR_MN;
  p.tiles_m = p.tiles_n = 0;
  p.band = 1;
  p.ksplit = 1;
  p.slice_elems = 0;
  p.status = a->status;
  const bool g1 = a->sb_gran_n == 1;
  const int bn = tile_width(a);
  const SplitPlan pl = plan_split(a, bn);
  if (pl.S > 1 && a->workspace != nullptr && a->workspace_bytes >= pl.bytes && aligned16(a->workspace)) {
    p.ksplit = pl.S;
    p.nkb_rem = p.nkb % pl.S;
    p.nkb /= pl.S;
    p.slice_elems = a->M * a->N;
    p.d = a->workspace;
    p.ldd = a->N;
    int rc;
    if (bn == 256) rc = launch_gemm<256, 128, true>(a, p, st);
    else if (bn == 192) rc = launch_gemm<192, 1, true>(a, p, st);
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
  if (bn == 256) return f32 ? launch_gemm<256, 128, true>(a, p, st) : launch_gemm<256, 128, false>(a, p, st);
  if (bn == 192) return f32 ? launch_gemm<192, 1, true>(a, p, st) : launch_gemm<192, 1, false>(a, p, st);
  if (g1) return f32 ? launch_gemm<128, 1, true>(a, p, st) : launch_gemm<128, 1, false>(a, p, st);
  return f32 ? launch_gemm<128, 128, true>(a, p, st) : launch_gemm<128, 128, false>(a, p, st);
}

// FP8 (e4m3) flash-attention forward for sm_100a.
//
// Replaces the reference's Ada kernel flash_attention_v2_cutlass_kernel
// (csrc/flash_attention.cu:330-584) together with its tile traits
// (csrc/kernel_traits.h:33-130), FP8 mma.sync atoms (csrc/mma_sm89.hpp,
// csrc/mma_traits_sm89.hpp) and the C->A register shuffle (csrc/reg2reg.h).
//
// The grid is persistent (one CTA per SM); a CTA takes one work item after the other,
// each being two 128-row query tiles of one (batch, head) slice (one tile at head_dim
// 256), and walks the key/value sequence; K and V^T arrive as 128-position tiles, the
// arithmetic runs on 64-position sub-blocks so that each query tile has two (head_dim
// 64: three) score buffers in tensor memory and its next S = Q K^T is computed while
// the softmax of the current sub-block is still running:
//
//   warp 18     TMA producer: Q tiles (double-buffered across work items), then K_j /
//               V_j tiles into a ring of shared-memory slots, each guarded by a
//               full/empty mbarrier pair.
//   warps 16,17 MMA issuers, one per query tile (one elected lane each):
//               S_i[sb % kSBuf] = Q_i K_sb^T (M128 N64) and O_i += P_i(sb) V_sb
//               (M128 N=head_dim) as tcgen05.mma kind::f8f6f4 with fp32 accumulators
//               in tensor memory; completion is signalled with tcgen05.commit on
//               mbarriers.
//   warps 0-7   online softmax for query tile 0, warps 8-15 for tile 1.  A TMEM lane
//               is a query row (tcgen05.ld 32x32b: one row per thread, no shuffles).
//               Warps w and w+4 of a tile own the same 32 rows and take the sub-blocks
//               in turn, so four softmax warps per scheduler keep the special-function
//               and FMA pipes fed.  exp2 with the scale folded in, row sum from the fp32
//               probabilities, P re-quantised to e4m3 and written back to TMEM over
//               its own S buffer as the A operand of the second GEMM; fp32 rescale of
//               O in TMEM when the row maximum has to be raised.  At the end of a work
//               item each warp scales its share of O, stages it as fp16 in shared
//               memory and hands it to the copy engine as a tiled bulk store.
//
// TMEM columns: tile i owns [256*i, 256*i + 256) (all 512 at head_dim 256): its S buffers
// at +64*b (64 fp32 columns each; P, 64 e4m3 = 16 columns, overlays the buffer it was
// computed from), O_i after them (Cfg<D>).
//
// Numerics follow the reference: P = exp(scale*(S - m)) unnormalised, converted to
// e4m3 round-to-nearest-even/saturating (csrc/flash_attention.cu:163-179,524), the
// row sum taken from fp32 P (:239-240,:264-271), final O/l with the zero/NaN guard
// (:542-554).  Differences: the output is fp16 (the reference rounds it to e4m3,
// :556-557); m is the exact row maximum after the first sub-block and is then
// raised only when a sub-block's sum of P would exceed 448, the largest e4m3 value (the
// reference raises it on every block, :233-273), which leaves O/l unchanged up to the
// rounding of P.
//
// Every mbarrier wait is bounded: when a wait runs out, the waiting thread
// records a code in the status word and in the library's host-visible flag, raises a
// CTA-wide abort flag and
// every role leaves its loop, drains its own copies / MMAs (bounded again),
// frees tensor memory and returns.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "fa8_kernel.h"
#include "ptx_sm100.cuh"

namespace fa8 {

namespace {

constexpr int kTileM = 128;        // query rows per tile = TMEM lanes
constexpr int kBlockN = 128;       // key/value positions per TMA tile
constexpr int kSubN = 64;          // key/value positions per MMA / softmax sub-block
constexpr int kMmaWarp0 = 16;      // warps 16 and 17: MMA issuers of query tile 0 and 1
constexpr int kLoadWarp = 18;
// Sixteen softmax warps, then the two MMA issuers and the producer: 608 threads.  With 640 (a
// fourth, idle warp completes the last warpgroup) registers can be re-allocated between the
// warpgroups at kernel start (setmaxnreg); measured, the larger CTA is 5 % slower with or
// without the re-allocation, so 608 is the default.
#ifndef FA8_THREADS
#define FA8_THREADS 608
#endif
constexpr int kThreads = FA8_THREADS;
static_assert(kThreads == 608 || kThreads == 640, "19 or 20 warps");
// Registers per thread after the re-allocation at kernel start.  The pool the warpgroups trade
// in is what the CTA was given at launch, 640 threads x 96 registers (the most a launch of 640
// threads can have), not the SM's whole register file: a request beyond it would block for ever.
constexpr uint32_t kRegsLaunch = 96;
#ifndef FA8_REGS_SOFTMAX
#define FA8_REGS_SOFTMAX (FA8_THREADS == 640 ? 104 : 96)
#endif
constexpr uint32_t kRegsSoftmax = FA8_REGS_SOFTMAX;
#ifndef FA8_REGS_AUX
#define FA8_REGS_AUX (FA8_THREADS == 640 ? 56 : 96)
#endif
constexpr uint32_t kRegsAux = FA8_REGS_AUX;
static_assert(512 * kRegsSoftmax + (kThreads - 512) * kRegsAux <= kThreads * kRegsLaunch,
              "register re-allocation exceeds the CTA's pool");
static_assert(kThreads == 640 || (kRegsSoftmax == kRegsLaunch && kRegsAux == kRegsLaunch),
              "setmaxnreg needs whole warpgroups: 640 threads");
static_assert(kRegsSoftmax % 8 == 0 && kRegsAux % 8 == 0 && kRegsAux >= 24, "setmaxnreg wants multiples of 8, at least 24");
constexpr uint32_t kTmemCols = 512;

template <int D>
struct Cfg {
  static_assert(D == 64 || D == 128 || D == 256, "head_dim must be 64, 128 or 256");
  // Rows longer than 128 bytes are stored as column blocks of 128 bytes, one after the other
  // (each block a 128-row swizzled tile of its own).
  static constexpr int kBlkD = (D < 128) ? D : 128;    // bytes per row of a column block
  static constexpr int kNBlk = D / kBlkD;
  static constexpr int kBlkBytes = 128 * kBlkD;
  static constexpr int kTileBytes = 128 * D;           // Q, K and V^T tiles alike
  // Query tiles per CTA: two, or one where O alone takes half of tensor memory (head_dim 256).
  static constexpr int kTiles = (D <= 128) ? 2 : 1;
  // Softmax warps per 32-row group of a tile: they take the sub-blocks in turn, warp j the
  // sub-blocks j, j + kW, ...  Two per group; at head_dim 256 that leaves eight of the sixteen
  // softmax warps without work (four per group on the one tile measured 25 % slower: the
  // hand-over of P is ordered, so more warps per group only lengthen that chain).
#ifndef FA8_D256_KW
#define FA8_D256_KW 2
#endif
  static constexpr int kW = (D == 256) ? FA8_D256_KW : 2;
  // Score buffers per tile, 64 fp32 columns each, used round robin (sub-block sb in buffer
  // sb % kSBuf).  A tile owns 512 / kTiles columns of tensor memory:
  //   head_dim  64: 3 x 64 + 64  = 256;  with three buffers the score of a warp's next sub-block
  //                 is computed while the warp still works on the current one
  //   head_dim 128: 2 x 64 + 128 = 256
  //   head_dim 256: 2 x 64 + 256 = 384 of 512 (four buffers fit; measured no faster)
#ifndef FA8_D256_NB
#define FA8_D256_NB 2
#endif
  static constexpr int kSBuf = (D == 64) ? 3 : (D == 128 ? 2 : FA8_D256_NB);
  static constexpr uint32_t kTileCols = kTmemCols / kTiles;     // tile i starts at column i * kTileCols
  static constexpr uint32_t kOCol = kSubN * kSBuf;              // O follows the tile's score buffers
  static_assert(kOCol + D <= kTileCols, "tensor-memory budget");
  static_assert(4 * kW * kTiles <= 16, "sixteen softmax warps");
  static constexpr int kSlots = (D == 128) ? 8 : (D == 64 ? 16 : 4);   // ring slots, one K or V tile each
  static constexpr int kQBytes = 2 * kTiles * kTileBytes;  // tiles x two stages (work items)
  static constexpr int kRingBytes = kSlots * kTileBytes;
  // Write-out of O: every softmax warp stages 32 rows x kEpiCols fp16 columns in shared memory
  // and hands them to the copy engine as one tiled store (a thread storing its own row straight
  // from registers touches 32 different 128-byte lines per instruction; measured, that made the
  // write-out of a work item cost 2600 cycles).  The width is what the shared memory left beside
  // the ring allows: 2 KB per warp, 1 KB at head_dim 128.
#ifndef FA8_EPI_COLS_128
#define FA8_EPI_COLS_128 16
#endif
#ifndef FA8_EPI_BUFS_128
#define FA8_EPI_BUFS_128 1
#endif
  static constexpr int kEpiCols = (D == 128) ? FA8_EPI_COLS_128 : epi_cols(D);
  static_assert(kEpiCols == epi_cols(D), "the host builds O's tensor map from epi_cols()");
  // Staging buffers per warp: with two, the copy engine reads one while the warp fills the other.
  static constexpr int kEpiBufs = (D == 128) ? FA8_EPI_BUFS_128 : 1;
  static constexpr int kEpiBytes = kEpiBufs * 32 * kEpiCols * 2;       // per warp
  static constexpr int kEpiWarps = 4 * kW * kTiles;                    // softmax warps that have rows
  static constexpr int kEpiOffset = kQBytes + kRingBytes;
  static constexpr int kBarOffset = kEpiOffset + kEpiWarps * kEpiBytes;
  // row-group scratch shared by the warps of a 32-row group, see RowGroupShared
  static constexpr int kGroups = 16 / kW;          // one per 32-row group of a tile slot (slot 1 idles at head_dim 256)
  static constexpr int kGroupBytes = kGroups * (160 + 512 * kW);
  static constexpr int kNumBars = 4 /*q_full*/ + 4 /*q_empty*/ + 2 * kSlots + 8 /*s_full*/ + 8 /*p_full*/ +
                                  2 /*o_done*/ + 2 /*o_final*/ + 2 /*o_free*/ + 2 /*drain*/;
  static constexpr int kSmemBytes = kBarOffset + kNumBars * 8 + 16 /*tmem ptr, abort*/ + kGroupBytes + 1024 /*align*/;
  // Q and K rows are D bytes long: one 128-byte swizzle row for D=128, a 64-byte one for D=64.
  static constexpr uint32_t kQKLayout = (D >= 128) ? 2u : 4u;   // UMMA SWIZZLE_128B / SWIZZLE_64B
  static constexpr uint32_t kQKSbo = 8 * kBlkD;                  // bytes between 8-row groups
};

// Shared-memory matrix descriptor for a K-major swizzled operand tile (rows of at most 128
// bytes, eight rows per swizzle atom): start address >> 4 in bits 0-13, leading-dimension
// offset 1 at bit 16, stride between 8-row groups >> 4 at bit 32, version 1 at bit 46, swizzle
// mode in bits 61-63.  Kept as two 32-bit words: only the low word (start address) changes
// from one operand slice to the next.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr) {
  return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
}
__device__ __forceinline__ uint32_t umma_desc_hi(uint32_t sbo_bytes, uint32_t layout_type) {
  return (sbo_bytes >> 4) | (1u << 14) | (layout_type << 29);
}
__device__ __forceinline__ uint64_t make_desc(uint32_t lo, uint32_t hi) {
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
// kind::f8f6f4 instruction descriptor: fp8 x fp8 -> f32, both operands K-major; `fmt` is the
// element format of A and B alike (0 = e4m3, 1 = e5m2; bits 7-9 and 10-12).
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, uint32_t fmt = 0) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

struct WaitCtx {
  volatile int* abort_flag;
  int* status;
  volatile int* host_status;     // mapped host word the library itself watches (may be null)
  unsigned long long limit_ns;
};

// Waits for the phase with the given parity; gives up after limit_ns or when
// another thread of the CTA already gave up.
__device__ __forceinline__ bool wait_bounded(const WaitCtx& w, uint32_t bar, uint32_t parity,
                                             int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 31u) == 0) {
      if (*w.abort_flag) return false;
      if (global_timer_ns() - t0 > w.limit_ns) {
        *w.abort_flag = 1;
        if (w.status) atomicCAS(w.status, 0, code);
        if (w.host_status) {
          *w.host_status = code;
          __threadfence_system();
        }
        return false;
      }
    }
  }
}

// ------------------------------------------------------------ softmax passes
// Which of the 32 element pairs of a 64-key sub-block take their exponential on the FMA
// pipe instead of the special-function unit (bit p = columns 2p and 2p+1).  The
// special-function unit delivers 16 exponentials per clock and SM, which is what bounds an
// FP8 forward; every pair moved over costs issue slots and FMA-pipe cycles instead.
#ifndef FA8_POLY_MASK
#define FA8_POLY_MASK 0x00000000u
#endif
// Degree of the polynomial for 2^f on [-1/2, 1/2]: 3 (relative error 7.5e-5) or 2 (1.7e-3;
// P is rounded to three mantissa bits afterwards, a relative step of 6e-2).
#ifndef FA8_POLY_DEG
#define FA8_POLY_DEG 3
#endif
// A sub-block's sum of P (hence every P in it) may grow to kLazyLimit before the row maximum
// is raised: 448, the largest e4m3 value (e5m2 reaches further).  fp8 keeps its relative
// precision over that range, so nothing is lost by letting P grow.  Measured on the bench
// workload with outliers: 2 % faster than a limit of 128, 20 % faster than 32.
// Scores fetched from tensor memory per load: two loads of 32 per sub-block, or all 64 at once
// (measured 2 % slower: the one long load is exposed, the second short one is not).
#ifndef FA8_CHUNK
#define FA8_CHUNK 32
#endif
#ifndef FA8_LAZY_LIMIT
#define FA8_LAZY_LIMIT 448.f
#endif
constexpr float kLazyLimit = FA8_LAZY_LIMIT;
// The FMA-pipe exponential clamps its argument to [kPolyLo, kPolyHi]: 2^kPolyLo is the smallest
// normal number (it rounds to zero in fp8 and adds nothing visible to a row sum that is at least
// 1), 2^kPolyHi lies above the lazy limit, so a clamped value still raises the row maximum.
constexpr float kPolyLo = -126.f, kPolyHi = 9.f, kPolyRange = kPolyHi - kPolyLo;
static_assert(kLazyLimit <= 448.f, "lazy limit");

// Four fp32 -> four fp8 (e4m3, or e5m2 when the inputs are e5m2, as the reference does with
// its Element type, csrc/flash_attention.cu:163-179) in one word, ascending index = ascending
// byte; round-to-nearest-even, saturating.
template <bool kE5M2>
__device__ __forceinline__ uint32_t pack4_fp8(float a, float b, float c, float d) {
  uint32_t r;
  if (kE5M2) {
    asm("{\n\t.reg .b16 lo, hi;\n\t"
        "cvt.rn.satfinite.e5m2x2.f32 lo, %2, %1;\n\t"
        "cvt.rn.satfinite.e5m2x2.f32 hi, %4, %3;\n\t"
        "mov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
  } else {
    asm("{\n\t.reg .b16 lo, hi;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
        "mov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
  }
  return r;
}

// Constants of the exponential P = 2^(c*s + neg_mc).  The part that depends on the row maximum
// is refreshed only when the maximum changes; everything stays in registers across sub-blocks.
// The FMA-pipe form evaluates, for x = c*s + neg_mc,
//   y  = sat(s*c/R + (neg_mc - lo)/R)          x clamped to [lo, hi] = lo + R*y
//   t  = R*y + (M + lo),  M = 1.5*2^23         t = M + n, n = round(x)
//   f  = R*y - (t - (M + lo)) = x - n          |f| <= 1/2
//   2^x = poly(f) * 2^n                        the exponent is added in the integer domain
struct ExpConsts {
  f32x2_t c2, nm2;          // x = c*s + neg_mc, two lanes
  float cr, nmr;            // the same map scaled into [0,1] for the saturating FMA
  __device__ __forceinline__ void set_scale(float c) {
    c2 = pack2(c, c);
    cr = c * (1.f / kPolyRange);
  }
  __device__ __forceinline__ void set_max(float neg_mc) {
    nm2 = pack2(neg_mc, neg_mc);
    nmr = (neg_mc - kPolyLo) * (1.f / kPolyRange);
  }
};

// P of one 64-key sub-block of this thread's row (TMEM columns t_sb..+63): P = 2^(c*s + neg_mc),
// packed to fp8 into pk[16] (four per word, ascending key index); returns the fp32 row sum.
// Columns >= lim are masked.  kAllowFma: the pairs selected by FA8_POLY_MASK take the FMA-pipe
// exponential.
template <bool kAllowFma, bool kE5M2>
__device__ __forceinline__ float softmax_pass(uint32_t t_sb, int lim, const ExpConsts& k,
                                              uint32_t (&pk)[16]) {
  const f32x2_t kr2 = pack2(kPolyRange, kPolyRange);
  const f32x2_t magic2 = pack2(12582912.f + kPolyLo, 12582912.f + kPolyLo);
  const f32x2_t neg1 = pack2(-1.f, -1.f);
#if FA8_POLY_DEG == 3
  const f32x2_t pc3 = pack2(0.055171654f, 0.055171654f), pc2 = pack2(0.24261114f, 0.24261114f);
  const f32x2_t pc1 = pack2(0.69326097f, 0.69326097f), pc0 = pack2(0.99992806f, 0.99992806f);
#else
  const f32x2_t pc2 = pack2(0.23842894f, 0.23842894f), pc1 = pack2(0.703448f, 0.703448f);
  const f32x2_t pc0 = pack2(1.0004431f, 1.0004431f);
#endif
  f32x2_t ls[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
  for (int c0 = 0; c0 < 64; c0 += FA8_CHUNK) {
    uint32_t s[FA8_CHUNK];
#if FA8_CHUNK == 64
    tmem_ld_32x32b_x64(t_sb, s);
#else
    tmem_ld_32x32b_x32(t_sb + c0, s);
#endif
    tmem_wait_ld();
    if (lim < c0 + FA8_CHUNK) {
#pragma unroll
      for (int e = 0; e < FA8_CHUNK; ++e)
        if (c0 + e >= lim) s[e] = 0xff800000u;   // -inf
    }
#pragma unroll
    for (int e = 0; e < FA8_CHUNK; e += 4) {
      float p[4];
#pragma unroll
      for (int u = 0; u < 4; u += 2) {
        const float s0 = __uint_as_float(s[e + u]), s1 = __uint_as_float(s[e + u + 1]);
        const bool on_fma = kAllowFma && (((FA8_POLY_MASK) >> ((c0 + e + u) / 2)) & 1u);
        if (on_fma) {
          const f32x2_t y2 = pack2(fma_sat(s0, k.cr, k.nmr), fma_sat(s1, k.cr, k.nmr));
          const f32x2_t t2 = fma2(y2, kr2, magic2);
          const f32x2_t nneg2 = fma2(t2, neg1, magic2);           // -(n - lo)
          const f32x2_t f2 = fma2(y2, kr2, nneg2);
#if FA8_POLY_DEG == 3
          f32x2_t r2 = fma2(f2, pc3, pc2);
          r2 = fma2(r2, f2, pc1);
#else
          f32x2_t r2 = fma2(f2, pc2, pc1);
#endif
          r2 = fma2(r2, f2, pc0);
          float r0, r1, t0, t1;
          unpack2(r2, r0, r1);
          unpack2(t2, t0, t1);
          // t = M + n has the mantissa field 2^22 + n: shifted left by 23 its low bits land in
          // the exponent field, which adds n (two's complement, modulo 2^9) to poly's exponent.
          p[u] = __int_as_float(__float_as_int(r0) + (__float_as_int(t0) << 23));
          p[u + 1] = __int_as_float(__float_as_int(r1) + (__float_as_int(t1) << 23));
        } else {
          float x0, x1;
          unpack2(fma2(pack2(s0, s1), k.c2, k.nm2), x0, x1);
          p[u] = ex2_approx(x0);
          p[u + 1] = ex2_approx(x1);
        }
        ls[u >> 1] = add2(ls[u >> 1], pack2(p[u], p[u + 1]));
      }
      pk[(c0 + e) / 4] = pack4_fp8<kE5M2>(p[0], p[1], p[2], p[3]);
    }
  }
  float a0, a1, a2, a3;
  unpack2(ls[0], a0, a1);
  unpack2(ls[1], a2, a3);
  return (a0 + a1) + (a2 + a3);
}

// Maximum of the (masked) 64 scores of this thread's row in one S buffer.  Out of line:
// it runs once per tile plus whenever a row maximum has to be raised.
__device__ __noinline__ float row_max(uint32_t t_s, int lim) {
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  for (int q = 0; q < 2; ++q) {
    uint32_t s[32];
    tmem_ld_32x32b_x32(t_s + 32 * q, s);
    tmem_wait_ld();
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const float v = (q * 32 + e < lim) ? __uint_as_float(s[e]) : -INFINITY;
      mx[e & 3] = fmaxf(mx[e & 3], v);
    }
  }
  return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

// Multiplies `chunks` x 32 fp32 columns of this thread's TMEM lane by alpha (the rare
// rescale of O when a row maximum is raised).  Out of line so that its registers do not
// weigh on the softmax loop.
__device__ __noinline__ void rescale_o_columns(uint32_t t_o, int chunks, float alpha) {
  for (int q = 0; q < chunks; ++q) {
    uint32_t orow[32];
    tmem_ld_32x32b_x32(t_o + 32 * q, orow);
    tmem_wait_ld();
#pragma unroll
    for (int e = 0; e < 32; ++e) orow[e] = __float_as_uint(__uint_as_float(orow[e]) * alpha);
    tmem_st_32x32b_x32(t_o + 32 * q, orow);
  }
  tmem_wait_st();
}

// What the kW warps of a 32-row group share: the row maxima the exponentials are taken
// against, a version counter bumped whenever they are raised, and each warp's final (row
// sum, maximum it refers to) for the epilogue.
template <int kW>
struct RowGroupShared {
  volatile float m[32];
  volatile uint32_t version;
  uint32_t pad[7];
  volatile float l_part[2][kW][32];   // [work item parity][warp of the group][row]
  volatile float m_part[2][kW][32];
};
static_assert(sizeof(RowGroupShared<2>) == 160 + 512 * 2 && sizeof(RowGroupShared<4>) == 160 + 512 * 4,
              "RowGroupShared layout");

// One work item: two 128-row query tiles of one (batch, head) slice (one tile at head_dim 256).
struct Item {
  int bh;          // slice
  int row0;        // first query row of tile 0
  int nsb_t[2];    // 64-key sub-blocks each tile visits (0 = the tile lies past the end)
  int nsb;         // max of the two
  int nb;          // 128-key K/V tiles to load
};

// Work decomposition of the persistent grid.  CTA c takes units c, c + gridDim.x, ...
// A work item is rows_per_item query rows of one slice: both tiles of the CTA, or (small
// problems, see plan_work) one tile, the second staying idle.  Non-causal: a unit is one
// item, slice-major (the CTAs running side by side work on the same few slices, whose K and
// V stay in L2).  Causal: the cost of an item grows with its position, so a unit folds item
// f with item n-1-f of the same slice (heavy one first) and every unit costs the same;
// without folding (a grid with an SM for every item) a unit is one item, heaviest first.
template <bool kCausal, int kTiles>
__device__ __forceinline__ bool get_item(const KernelArgs& a, int unit, int k, Item& it) {
  const int n_pairs = a.n_pairs;
  int pair;
  if (!kCausal || !a.fold) {
    if (k > 0) return false;
    it.bh = unit / n_pairs;
    pair = unit - it.bh * n_pairs;
    if (kCausal) pair = n_pairs - 1 - pair;
  } else {
    const int n_fold = (n_pairs + 1) >> 1;
    it.bh = unit / n_fold;
    const int f = unit - it.bh * n_fold;
    const int hi = n_pairs - 1 - f;
    if (k == 0) {
      pair = hi;
    } else {
      if (hi == f) return false;
      pair = f;
    }
  }
  it.row0 = pair * a.rows_per_item;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r0 = it.row0 + i * kTileM;
    int n = 0;
    if (i < kTiles && i * kTileM < a.rows_per_item && r0 < a.seqlen) {
      // one past the last visible key; the causal mask is aligned top-left (key <= query row),
      // like the reference's (csrc/flash_attention.cu:24-71, test.py:25-33)
      const int col_end = kCausal ? min(r0 + kTileM, a.seqlen_k) : a.seqlen_k;
      n = (col_end + kSubN - 1) / kSubN;
    }
    it.nsb_t[i] = n;
  }
  it.nsb = max(it.nsb_t[0], it.nsb_t[1]);
  it.nb = (it.nsb + 1) >> 1;
  return true;
}

}  // namespace

template <int D, bool kCausal, bool kVNatural, bool kE5M2>
__global__ void __launch_bounds__(kThreads, 1)
fa8_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
               const KernelArgs args) {
  using C = Cfg<D>;
  constexpr int kItemsPerUnit = kCausal ? 2 : 1;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  // Q tiles are double-buffered across work items: s_q + (2*stage + tile) * kTileBytes.
  const uint32_t s_q = smem_base;
  const uint32_t s_ring = smem_base + C::kQBytes;
  const uint32_t s_bar = smem_base + C::kBarOffset;
  int bar_idx = 0;
  auto take = [&](int n) { const uint32_t a = s_bar + 8u * bar_idx; bar_idx += n; return a; };
  const uint32_t b_q_full = take(4), b_q_empty = take(4);            // [tile][stage]
  const uint32_t b_kv_full = take(C::kSlots), b_kv_empty = take(C::kSlots);
  const uint32_t b_s_full = take(8), b_p_full = take(8);             // [tile][S buffer]
  const uint32_t b_o_done = take(2), b_o_final = take(2), b_o_free = take(2);
  const uint32_t bar_drain = take(2);
  auto bar_q_full = [&](int i, int st) { return b_q_full + 8u * (2 * i + st); };
  auto bar_q_empty = [&](int i, int st) { return b_q_empty + 8u * (2 * i + st); };
  auto bar_kv_full = [&](int s) { return b_kv_full + 8u * s; };
  auto bar_kv_empty = [&](int s) { return b_kv_empty + 8u * s; };
  auto bar_s_full = [&](int i, int b) { return b_s_full + 8u * (C::kSBuf * i + b); };
  // One P barrier per S buffer: the four warps (one per 32-row group) that took the sub-block arrive.
  auto bar_p_full = [&](int i, int b) { return b_p_full + 8u * (C::kSBuf * i + b); };
  // o_done[i]: one phase per PV of tile i.  o_final[i]: one phase per work item, after the
  // tile's last PV (the epilogue cannot use o_done: warps get there at different distances
  // from the end, which a parity wait cannot tell apart).  o_free[i]: one phase per work
  // item, when all eight warps of the tile have read O out of tensor memory.
  auto bar_o_done = [&](int i) { return b_o_done + 8u * i; };
  auto bar_o_final = [&](int i) { return b_o_final + 8u * i; };
  auto bar_o_free = [&](int i) { return b_o_free + 8u * i; };
  volatile uint32_t* tmem_ptr_slot =
      reinterpret_cast<volatile uint32_t*>(smem_gen + C::kBarOffset + C::kNumBars * 8);
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(smem_gen + C::kBarOffset + C::kNumBars * 8 + 4);
  volatile int* skip_flag =
      reinterpret_cast<volatile int*>(smem_gen + C::kBarOffset + C::kNumBars * 8 + 8);
  RowGroupShared<C::kW>* groups =
      reinterpret_cast<RowGroupShared<C::kW>*>(smem_gen + C::kBarOffset + C::kNumBars * 8 + 16);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int seqlen = args.seqlen;
  const WaitCtx wctx{abort_flag, args.status, args.host_status, args.timeout_ns};

  // Set-up, spread over three warps so that the three latencies overlap: thread 0 initialises
  // the barriers, the first issuer warp allocates tensor memory, and lane 0 of warp 1 reads
  // the status word from global memory.
  if (threadIdx.x == 0) {
    for (int x = 0; x < 4; ++x) {
      mbar_init(b_q_full + 8u * x, 1);
      mbar_init(b_q_empty + 8u * x, 1);
    }
    for (int x = 0; x < 8; ++x) {
      mbar_init(b_s_full + 8u * x, 1);
      mbar_init(b_p_full + 8u * x, 4);     // one arrive per 32-row group
    }
    for (int s = 0; s < C::kSlots; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 2);       // both MMA issuers hand a slot back
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_o_done(i), 1);
      mbar_init(bar_o_final(i), 1);
      mbar_init(bar_o_free(i), 4 * C::kW);   // one arrive per softmax warp of the tile
    }
    mbar_init(bar_drain, 1);
    mbar_init(bar_drain + 8u, 1);
    for (int g = 0; g < C::kGroups; ++g) groups[g].version = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  } else if (threadIdx.x == 32) {
    // A status word that is already non-zero (an earlier CTA of this launch gave up, or the
    // caller did not clear it) makes the CTA return at once: a failed launch then costs one
    // wait limit, not one per CTA.  skip_flag is written here only; abort_flag is what a
    // wait that gives up raises later.
    const bool stale = args.status != nullptr && *reinterpret_cast<volatile int*>(args.status) != 0;
    *abort_flag = stale ? 2 : 0;
    *skip_flag = stale ? 1 : 0;
    // The skipped launch leaves O unwritten: the host must hear of it even if the word's first
    // report has already been collected.
    if (stale && args.host_status != nullptr && *args.host_status == 0) *args.host_status = 0x5717;
  } else if (warp == kLoadWarp && lane == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  if (warp == kMmaWarp0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;
  const bool skip_cta = (*skip_flag != 0);

  // Warps 16-19 form a warpgroup of their own (producer, two MMA issuers, one spare): it
  // hands most of its registers to the four softmax warpgroups.
  if (warp >= kMmaWarp0) {
    if constexpr (kRegsAux != kRegsLaunch) setmaxnreg_dec<kRegsAux>();
    if (skip_cta) {
      // fall through to the teardown
    } else if (warp == kLoadWarp) {
      // ------------------------------------------------------------ TMA producer
      if (elect_one()) {
        bool ok = true;
        int it = 0;                 // K/V loads issued so far; slot = it % kSlots
        int qn[2] = {0, 0};         // Q loads issued so far per tile; stage = qn & 1
        // One tile of 128 rows of head_dim bytes (Q, K, natural V): a copy per 128-byte column block.
        auto load_rows = [&](uint32_t dst, const CUtensorMap* tm, uint32_t bar, int row, int bh) {
  #pragma unroll
          for (int b = 0; b < C::kNBlk; ++b) tma_load_3d(dst + b * C::kBlkBytes, tm, bar, b * C::kBlkD, row, bh);
        };
        auto load_kv = [&](const CUtensorMap* tm, bool rows, int c0, int c1, int bh) {
          const int slot = it % C::kSlots;
          const uint32_t round = static_cast<uint32_t>(it / C::kSlots);
          if (ok) ok = wait_bounded(wctx, bar_kv_empty(slot), (round & 1u) ^ 1u, 0x100 + slot);
          if (ok) {
            mbar_arrive_expect_tx(bar_kv_full(slot), C::kTileBytes);
            if (rows) load_rows(s_ring + slot * C::kTileBytes, tm, bar_kv_full(slot), c1, bh);
            else tma_load_3d(s_ring + slot * C::kTileBytes, tm, bar_kv_full(slot), c0, c1, bh);
            ++it;
          }
        };
        for (int unit = blockIdx.x; unit < args.n_units && ok; unit += gridDim.x) {
          for (int k = 0; k < kItemsPerUnit && ok; ++k) {
            Item w;
            if (!get_item<kCausal, C::kTiles>(args, unit, k, w)) continue;
  #pragma unroll
            for (int i = 0; i < 2; ++i) {
              if (w.nsb_t[i] > 0 && ok) {
                const int st = qn[i] & 1;
                const uint32_t round = static_cast<uint32_t>(qn[i] >> 1);
                ok = wait_bounded(wctx, bar_q_empty(i, st), (round & 1u) ^ 1u, 0x180 + i);
                if (ok) {
                  mbar_arrive_expect_tx(bar_q_full(i, st), C::kTileBytes);
                  load_rows(s_q + (C::kTiles * st + i) * C::kTileBytes, &tm_q, bar_q_full(i, st),
                            w.row0 + i * kTileM, w.bh);
                  ++qn[i];
                }
              }
            }
            // Grouped-query attention: query head h of a batch entry reads K/V head h / group.
            const int b_idx = w.bh / args.heads;
            const int kv_bh = b_idx * args.heads_kv + (w.bh - b_idx * args.heads) / (args.heads / args.heads_kv);
            for (int j = 0; j < w.nb && ok; ++j) {
              load_kv(&tm_k, true, 0, j * kBlockN, kv_bh);
              if (kVNatural) load_kv(&tm_v, true, 0, j * kBlockN, kv_bh);    // [keys, head_dim] rows
              else load_kv(&tm_v, false, j * kBlockN, 0, kv_bh);             // [head_dim, keys] rows
            }
          }
        }
        if (!ok) {
          // Abort: let this CTA's copies that are still in flight land before the shared
          // memory is given back.  K/V loads [it - kSlots, it) and the last two Q loads of
          // each tile may be pending.
          for (int p = max(0, it - C::kSlots); p < it; ++p) {
            const int slot = p % C::kSlots;
            const uint32_t round = static_cast<uint32_t>(p / C::kSlots);
            const uint64_t t0 = global_timer_ns();
            while (!mbar_try_wait(bar_kv_full(slot), round & 1u)) {
              if (global_timer_ns() - t0 > 20000000ull) break;
            }
          }
  #pragma unroll
          for (int i = 0; i < 2; ++i) {
            for (int p = max(0, qn[i] - 2); p < qn[i]; ++p) {
              const uint64_t t0 = global_timer_ns();
              while (!mbar_try_wait(bar_q_full(i, p & 1), static_cast<uint32_t>(p >> 1) & 1u)) {
                if (global_timer_ns() - t0 > 20000000ull) break;
              }
            }
          }
        }
      }
      __syncwarp();
    } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
      // ------------------------------------------------- MMA issuers, one per query tile
      // Each issues, for its tile i, S_i[sb % kSBuf] = Q_i K_sb^T and O_i += P_i(sb) V_sb.  The two
      // never wait for one another; a K/V ring slot goes back to the producer when both have
      // committed it (kv_empty counts two arrivals).
      if (elect_one()) {
        const int i = warp - kMmaWarp0;
        constexpr uint32_t kFmt = kE5M2 ? 1u : 0u;
        constexpr uint32_t kIdescQK = umma_idesc(kTileM, kSubN, kFmt);
        // V in its natural [keys, head_dim] layout is an MN-major B operand (bit 16).
        constexpr uint32_t kIdescPV = umma_idesc(kTileM, C::kBlkD, kFmt) | (kVNatural ? (1u << 16) : 0u);
        constexpr uint32_t kBlk16 = C::kBlkBytes / 16;       // one column block in descriptor address units
        constexpr uint32_t kSlotMask = C::kSlots - 1;
        static_assert((C::kSlots & (C::kSlots - 1)) == 0, "ring size must be a power of two");
        constexpr int kSlotShift = (C::kSlots == 4) ? 2 : (C::kSlots == 8 ? 3 : 4);
        static_assert((1 << kSlotShift) == C::kSlots, "ring size");
        constexpr uint32_t kTile16 = C::kTileBytes / 16;     // one tile in descriptor address units
        // This one thread paces the whole tile, so its instruction count per step is kept low:
        // descriptors are 32-bit low words (start address in units of 16 bytes; the high word
        // never changes), barrier addresses and parities are carried, not recomputed.
        const uint32_t qk_hi = umma_desc_hi(C::kQKSbo, C::kQKLayout);
        const uint32_t v_hi = kVNatural ? qk_hi : umma_desc_hi(1024u, 2u);
        const uint32_t q_lo0 = umma_desc_lo(s_q + i * C::kTileBytes);
        const uint32_t ring_lo = umma_desc_lo(s_ring);
        const uint32_t t_tile = tmem_base + i * C::kTileCols;        // score buffer b at t_tile + 64 b
        const uint32_t t_s0 = t_tile, t_s1 = t_tile + kSubN;
        const uint32_t t_o = t_tile + C::kOCol;
        const uint32_t b_sf0 = bar_s_full(i, 0), b_sf1 = bar_s_full(i, 1);
        const uint32_t b_pf0 = bar_p_full(i, 0), b_pf1 = bar_p_full(i, 1);
        const uint32_t b_od = bar_o_done(i), b_ofin = bar_o_final(i), b_ofree = bar_o_free(i);
        // The V^T tile is D rows of 128 key positions (K-major, 128-byte swizzle), of which
        // sub-block h covers bytes 64h..64h+63 of every row = K-steps 2h and 2h+1.  In the
        // natural layout the tile is 128 key rows of D bytes (swizzled like K): a K-step of 32
        // keys is 32 rows further down.
        constexpr uint32_t kVStep = kVNatural ? (32u * C::kBlkD / 16u) : 2u;   // descriptor units per 32 keys
        constexpr uint32_t kKHalf = kSubN * C::kBlkD / 16;                     // rows 64..127 of a K tile
        // S_i[h] = Q_i K_sb^T: D/32 steps of K = 32 bytes along the swizzled rows.
        auto issue_qk = [&](uint32_t ts, uint32_t q_lo, uint32_t k_lo) {
  #pragma unroll
          for (int k = 0; k < D / 32; ++k) {
            // K-step k lies in column block k / 4 (four steps of 32 bytes per 128-byte row)
            const uint32_t off = (C::kNBlk > 1 ? (k >> 2) * kBlk16 : 0u) + 2u * (C::kNBlk > 1 ? (k & 3) : k);
            mma_f8_ss(ts, make_desc(q_lo + off, qk_hi), make_desc(k_lo + off, qk_hi), kIdescQK, k > 0);
          }
        };
        // O_i (+)= P_i(sb) V_sb: P is 128 rows x 64 fp8 = 16 TMEM columns over S_i[h].
        auto issue_pv = [&](uint32_t ts, uint32_t v_lo, bool acc) {
  #pragma unroll
          for (int nb = 0; nb < C::kNBlk; ++nb)         // 128 output columns per MMA: one column block of V
  #pragma unroll
            for (int k = 0; k < kSubN / 32; ++k)
              mma_f8_ts(t_o + nb * C::kBlkD, ts + 8u * k, make_desc(v_lo + nb * kBlk16 + kVStep * k, v_hi), kIdescPV,
                        (acc || k > 0) ? 1u : 0u);
        };
        auto kv_wait = [&](uint32_t load) {
          const uint32_t slot = load & kSlotMask;
          return wait_bounded(wctx, b_kv_full + 8u * slot, (load >> kSlotShift) & 1u, 0x200 + slot);
        };
        auto kv_release = [&](uint32_t load) { tc_commit(b_kv_empty + 8u * (load & kSlotMask)); };
        auto kv_lo = [&](uint32_t load) { return ring_lo + (load & kSlotMask) * kTile16; };

        bool ok = true;
        uint32_t ld = 0;                 // index of the current item's first K/V load (K_0)
        uint32_t qn = 0;                 // work items of this tile so far
        uint32_t pp0 = 0, pp1 = 0;       // parity of the next P phase per S buffer (two-buffer path)
        uint32_t pp = 0;                 // the same, one bit per buffer (general path)

        for (int unit = blockIdx.x; unit < args.n_units && ok; unit += gridDim.x) {
          for (int kk = 0; kk < kItemsPerUnit && ok; ++kk) {
            Item w;
            if (!get_item<kCausal, C::kTiles>(args, unit, kk, w)) continue;
            const int nsb = (i == 0) ? w.nsb_t[0] : w.nsb_t[1];
            // The item's loads are K_0, V_0, K_1, V_1, ... = ld + 0, 1, 2, ...  Each is handed
            // back to the producer exactly once by this thread, whether or not its tile reads
            // it; `rel` is the next one to hand back.
            const uint32_t ld_end = ld + 2u * static_cast<uint32_t>(w.nb);
            uint32_t rel = ld;
            if (nsb > 0) {
              const uint32_t st = qn & 1u;
              const uint32_t q_lo = q_lo0 + st * (C::kTiles * kTile16);
              const uint32_t b_qe = bar_q_empty(i, st);
              if constexpr (C::kSBuf == 2) {
              // Prologue: the first two S need no P.
              ok = kv_wait(ld);
              if (ok) ok = wait_bounded(wctx, bar_q_full(i, st), (qn >> 1) & 1u, 0x300 + i);
              if (!ok) break;
              tc_fence_after();
              issue_qk(t_s0, q_lo, kv_lo(ld));
              tc_commit(b_sf0);
              if (nsb > 1) {
                issue_qk(t_s1, q_lo, kv_lo(ld) + kKHalf);
                tc_commit(b_sf1);
              }
              if (nsb <= 2) tc_commit(b_qe);
              kv_release(ld);                                         // K_0
              rel = ld + 1;
              // Steps 2j and 2j+1: PV(sb), then QK(sb+2) into the S buffer PV just freed.
              // Both read V_j; the QKs read the two halves of K_{j+1}.
              const int n_pairs_kv = (nsb + 1) >> 1;
              for (int j = 0; j < n_pairs_kv; ++j) {
                const uint32_t lv = ld + 2u * j + 1u, lk = lv + 1u;   // loads V_j, K_{j+1}
                const int sb = 2 * j;
                const bool qk0 = sb + 2 < nsb, pv1 = sb + 1 < nsb, qk1 = sb + 3 < nsb;
                const uint32_t v_lo = kv_lo(lv), k_lo = kv_lo(lk);
                ok = kv_wait(lv);
                if (qk0 && ok) ok = kv_wait(lk);
                if (ok) ok = wait_bounded(wctx, b_pf0, pp0, 0x400 + i);
                if (j == 0 && qn > 0 && ok)                            // O_i of the previous item read out?
                  ok = wait_bounded(wctx, b_ofree, (qn - 1) & 1u, 0x480 + i);
                if (!ok) break;
                pp0 ^= 1u;
                tc_fence_after();
                issue_pv(t_s0, v_lo, j > 0);
                tc_commit(b_od);
                if (!pv1) tc_commit(b_ofin);
                if (qk0) {
                  issue_qk(t_s0, q_lo, k_lo);
                  tc_commit(b_sf0);                                    // S_i[0] now holds sub-block sb+2
                  if (sb + 2 == nsb - 1) tc_commit(b_qe);
                }
                if (pv1) {
                  ok = wait_bounded(wctx, b_pf1, pp1, 0x400 + i);
                  if (!ok) break;
                  pp1 ^= 1u;
                  tc_fence_after();
                  issue_pv(t_s1, v_lo + 2u * kVStep, true);
                  tc_commit(b_od);
                  if (sb + 1 == nsb - 1) tc_commit(b_ofin);
                  if (qk1) {
                    issue_qk(t_s1, q_lo, k_lo + kKHalf);
                    tc_commit(b_sf1);                                  // S_i[1] now holds sub-block sb+3
                    if (sb + 3 == nsb - 1) tc_commit(b_qe);
                  }
                }
                // V_j was last read by PV(2j+1), K_{j+1} by QK(2j+3).
                kv_release(lv);
                rel = lk;
                if (qk0) {
                  kv_release(lk);
                  rel = lk + 1u;
                }
              }
              } else {
                // Any number of score buffers: sub-block sb lives in buffer sb % kSBuf.  The first
                // kSBuf scores need no P; after that QK(sb + kSBuf) follows PV(sb) into the buffer
                // that PV has just read.  K_t (load ld + 2t) serves the QKs of sub-blocks 2t and
                // 2t + 1, V_t (load ld + 2t + 1) their PVs; each goes back after its last reader.
                constexpr int kNB = C::kSBuf;
                auto qk_step = [&](int s, int b) -> bool {          // false when a wait ran out
                  const uint32_t lk = ld + 2u * static_cast<uint32_t>(s >> 1);
                  if ((s & 1) == 0 && !kv_wait(lk)) return false;
                  issue_qk(t_tile + b * kSubN, q_lo, kv_lo(lk) + ((s & 1) ? kKHalf : 0u));
                  tc_commit(bar_s_full(i, b));
                  if (s == nsb - 1) tc_commit(b_qe);
                  if ((s & 1) || s == nsb - 1) kv_release(lk);
                  return true;
                };
                ok = wait_bounded(wctx, bar_q_full(i, st), (qn >> 1) & 1u, 0x300 + i);
                if (!ok) break;
                tc_fence_after();
                for (int sq = 0; sq < kNB && sq < nsb && ok; ++sq) ok = qk_step(sq, sq);
                int b = 0;
                for (int sb = 0; sb < nsb && ok; ++sb) {
                  const uint32_t lv = ld + 2u * static_cast<uint32_t>(sb >> 1) + 1u;
                  if ((sb & 1) == 0) ok = kv_wait(lv);
                  if (ok) ok = wait_bounded(wctx, bar_p_full(i, b), (pp >> b) & 1u, 0x400 + i);
                  if (sb == 0 && qn > 0 && ok)                           // O_i of the previous item read out?
                    ok = wait_bounded(wctx, b_ofree, (qn - 1) & 1u, 0x480 + i);
                  if (!ok) break;
                  pp ^= 1u << b;
                  tc_fence_after();
                  issue_pv(t_tile + b * kSubN, kv_lo(lv) + ((sb & 1) ? 2u * kVStep : 0u), sb > 0);
                  tc_commit(b_od);
                  if (sb == nsb - 1) tc_commit(b_ofin);
                  if (sb + kNB < nsb) ok = qk_step(sb + kNB, b);
                  if ((sb & 1) || sb == nsb - 1) kv_release(lv);
                  b = (b + 1 == kNB) ? 0 : b + 1;
                }
                if (!ok) break;
                rel = ld + 2u * static_cast<uint32_t>((nsb + 1) >> 1);
              }
              ++qn;
            }
            // Loads this tile did not read.  Waiting for each before handing it back keeps this
            // thread from arriving twice in one phase of a slot's barrier: the load can only
            // have been issued after both tiles handed back the slot's previous occupant.
            for (; rel < ld_end && ok; ++rel) {
              ok = kv_wait(rel);
              if (ok) kv_release(rel);
            }
            ld = ld_end;
          }
        }
        if (!ok) {
          // Abort: wait (bounded) for the MMAs already issued before TMEM is freed.
          const uint32_t bd = bar_drain + 8u * i;
          tc_commit(bd);
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(bd, 0)) {
            if (global_timer_ns() - t0 > 20000000ull) break;
          }
        }
      }
      __syncwarp();
    }
  } else {
    if constexpr (kRegsSoftmax != kRegsLaunch) setmaxnreg_inc<kRegsSoftmax>();
    if (!skip_cta) {
      // ------------------------------------------------- softmax + epilogue warps
      constexpr int kW = C::kW, kNB = C::kSBuf;
      const int i = warp / (4 * kW);                     // query tile of this warp
      const int h = (warp >> 2) % kW;                    // which of the row group's warps: sub-blocks h, h + kW, ...
      const int quarter = warp & 3;                      // TMEM lane quarter = 32-row group
      const int row = quarter * 32 + lane;               // row in the tile = TMEM lane
      const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
      const uint32_t t_tile = tmem_base + lane_sel + i * C::kTileCols;       // score buffer b at t_tile + 64 b
      const uint32_t t_o = t_tile + C::kOCol;
      // Per-tensor descales that live on the device (written by the quantisation pre-pass)
      // fold into the softmax scale (Q, K) and the output scale (V).
      // With descale_per_head they are arrays, one entry per (batch, head) for Q and per
      // (batch, key/value head) for K and V, re-read for every work item.
      float qk_descale = 1.f, o_scale = args.o_scale;
      if (!args.descale_per_head) {
        if (args.descale_q != nullptr) qk_descale *= __ldg(args.descale_q);
        if (args.descale_k != nullptr) qk_descale *= __ldg(args.descale_k);
        if (args.descale_v != nullptr) o_scale *= __ldg(args.descale_v);
      }
      float c = args.scale_log2 * qk_descale;
      float sm_scale = args.softmax_scale * qk_descale;
      RowGroupShared<kW>& grp = groups[i * 4 + quarter];
      // This warp's staging buffer for the write-out of O (warps without rows have none).
      const uint32_t s_stage = smem_base + C::kEpiOffset + static_cast<uint32_t>(warp % C::kEpiWarps) * C::kEpiBytes;
      if (lane == 0) prefetch_tensormap(&tm_o);
      // Running phases of the barriers this warp waits on.  Sub-block sb of an item uses phase
      // number (uses of its buffer in earlier items) + sb / kNB of s_full and p_full alike; bit b
      // of ph_bits is the parity of the first of these for buffer b.
      uint32_t ph_bits = 0;
      uint32_t pv_cnt = 0;         // PVs of this tile before the current item: o_done[i] base
      uint32_t items = 0;          // work items of this tile so far: o_final[i] phase, l_part buffer
      uint32_t version = 0;        // last value of grp.version this warp has seen
      bool ok = true;
      ExpConsts ek;
      ek.set_scale(c);
      ek.set_max(0.f);

      for (int unit = blockIdx.x; unit < args.n_units && ok; unit += gridDim.x) {
        for (int kk = 0; kk < kItemsPerUnit && ok; ++kk) {
          Item w;
          if (!get_item<kCausal, C::kTiles>(args, unit, kk, w)) continue;
          const int tile_nsb = w.nsb_t[i];
          if (tile_nsb == 0) continue;
          const int q_row = w.row0 + i * kTileM + row;       // global query row, may be >= seqlen
          const int col_lim = kCausal ? min(args.seqlen_k, q_row + 1) : args.seqlen_k;   // keys this row may see
          const uint32_t ib = items & 1u;
          if (args.descale_per_head) {
            const int b_idx = w.bh / args.heads;
            const int kv_bh = b_idx * args.heads_kv + (w.bh - b_idx * args.heads) / (args.heads / args.heads_kv);
            qk_descale = 1.f;
            o_scale = args.o_scale;
            if (args.descale_q != nullptr) qk_descale *= __ldg(args.descale_q + w.bh);
            if (args.descale_k != nullptr) qk_descale *= __ldg(args.descale_k + kv_bh);
            if (args.descale_v != nullptr) o_scale *= __ldg(args.descale_v + kv_bh);
            c = args.scale_log2 * qk_descale;
            sm_scale = args.softmax_scale * qk_descale;
            ek.set_scale(c);
          }
          // m is the row maximum the exponentials are taken against, shared by the warps
          // of the row group through grp.m / grp.version: exact after sub-block 0, then raised
          // only by the exact path below.  l is this warp's share of the row sum, kept relative
          // to m.  O and both shares are sums against the same m, so O/l does not depend on
          // when m is raised.
          float m = -INFINITY, l = 0.f;
          bool have_m = false;

          for (int sb = h; sb < tile_nsb; sb += kW) {
            const int b = sb % kNB;                          // the score buffer of this sub-block
            const uint32_t t_sb = t_tile + b * kSubN;
            bool ok_s = wait_bounded(wctx, bar_s_full(i, b), ((ph_bits >> b) ^ static_cast<uint32_t>(sb / kNB)) & 1u,
                                     0x500 + i);
            tc_fence_after();
            const int lim = col_lim - sb * kSubN;            // sub-block-local first masked column

            uint32_t pk[16];
            float bsum = 0.f;
            // Fast path: one pass, exponentials against the maximum known so far.
            if (have_m) {
              if (kCausal && __all_sync(0xffffffffu, lim <= 0)) {
                // Every row of this warp lies above the diagonal of this sub-block: P = 0.
  #pragma unroll
                for (int e = 0; e < 16; ++e) pk[e] = 0u;
              } else {
                bsum = softmax_pass<true, kE5M2>(t_sb, lim, ek, pk);
              }
            }
            // P(sb) may be handed over only after P(sb-1) has been (by the warp before this one in
            // the rotation): from then on nobody else can raise the maximum before PV(sb) is issued.
            if (sb > 0) {
              const int bp = (sb - 1) % kNB;
              ok_s = wait_bounded(wctx, bar_p_full(i, bp),
                                  ((ph_bits >> bp) ^ static_cast<uint32_t>((sb - 1) / kNB)) & 1u, 0x800 + i) && ok_s;
            }
            // One vote settles the common case: waits fine, maximum unchanged, no overflow.
            // Some P above kLazyLimit implies a sum above it (all P >= 0); a false alarm only
            // costs the exact path.  Decided for the warp's 32 rows as a whole.
            const uint32_t v = grp.version;
            const bool calm = ok_s && have_m && (v == version) && (bsum <= kLazyLimit);
            if (!__all_sync(0xffffffffu, calm)) {
              ok = __all_sync(0xffffffffu, ok_s);
              if (!ok) break;
              bool exact = (sb == 0);
              if (!exact) {
                if (v != version || !have_m) {
                  // Another warp raised the maximum (or this is my first sub-block of the item).
                  __threadfence_block();
                  const float m_new = grp.m[lane];
                  if (have_m) l *= ex2_approx((m - m_new) * c);
                  m = m_new;
                  version = v;
                  have_m = true;
                  ek.set_max(-m * c);
                  bsum = softmax_pass<false, kE5M2>(t_sb, lim, ek, pk);
                }
                exact = __any_sync(0xffffffffu, !(bsum <= kLazyLimit));
              }
              if (exact) {
                // Exact path (first sub-block, or the maximum is too low for some row of this
                // warp): true row maximum, rescale l and O, publish, redo the exponentials.
                const float m_new = fmaxf(m, row_max(t_sb, lim));
                if (sb > 0) {
                  // O_i must be quiescent: PV_i(sb-1) complete; PV_i(sb) waits for this warp.
                  ok = wait_bounded(wctx, bar_o_done(i), (pv_cnt + static_cast<uint32_t>(sb - 1)) & 1u, 0x700 + i);
                  ok = __all_sync(0xffffffffu, ok);
                  if (!ok) break;
                  tc_fence_after();
                  float alpha = ex2_approx((m - m_new) * c);
                  if (m == -INFINITY) alpha = 1.f;
                  l *= alpha;
                  rescale_o_columns(t_o, D / 32, alpha);
                }
                m = m_new;
                have_m = true;
                grp.m[lane] = m_new;
                __threadfence_block();
                __syncwarp();
                version = grp.version + 1;
                __syncwarp();
                if (lane == 0) grp.version = version;
                ek.set_max((m == -INFINITY) ? 0.f : -m * c);
                bsum = softmax_pass<false, kE5M2>(t_sb, lim, ek, pk);
              }
            }
            l += bsum;
            if (sb + kW >= tile_nsb) {                       // my last sub-block: leave my share for the epilogue
              grp.l_part[ib][h][lane] = l;
              grp.m_part[ib][h][lane] = m;
              __threadfence_block();
            }
            tmem_st_32x32b_x16(t_sb, pk);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_full(i, b));
          }
          if (!ok) break;
  #pragma unroll
          for (int b = 0; b < kNB; ++b)                      // buffer b served (tile_nsb - b) / kNB, rounded up, sub-blocks
            if (((tile_nsb + kNB - 1 - b) / kNB) & 1) ph_bits ^= 1u << b;
          pv_cnt += static_cast<uint32_t>(tile_nsb);

          // Epilogue: O_i / l -> fp16 -> global; each warp of the group writes its share of the head dim.
          ok = wait_bounded(wctx, bar_o_final(i), items & 1u, 0x600 + i);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          __threadfence_block();
          // Row sum = the warps' shares, each brought to the final maximum.
          float l_tot = 0.f, m_fin = -INFINITY;
  #pragma unroll
          for (int w2 = 0; w2 < kW; ++w2)
            if (w2 < tile_nsb) m_fin = fmaxf(m_fin, grp.m_part[ib][w2][lane]);
  #pragma unroll
          for (int w2 = 0; w2 < kW; ++w2) {
            if (w2 < tile_nsb) {
              const float mp = grp.m_part[ib][w2][lane], lp = grp.l_part[ib][w2][lane];
              l_tot += (mp == -INFINITY) ? 0.f : lp * ex2_approx((mp - m_fin) * c);
            }
          }
          const float inv = ((l_tot == 0.f || l_tot != l_tot) ? 1.f : 1.f / l_tot) * o_scale;
          if (args.lse != nullptr && h == 0 && q_row < seqlen)    // log(sum exp(scale*s)) = scale*m + log(l)
            args.lse[static_cast<size_t>(w.bh) * seqlen + q_row] = m_fin * sm_scale + __logf(l_tot);
          // Rows of O are args.head_dim long; the kernel's columns beyond that are padding, and
          // the tile may reach past the last query row: the copy engine drops both.
          const int d_out = args.head_dim;
          constexpr int kMyCols = D / kW;                     // this warp's share of the head dimension
          constexpr int kEC = C::kEpiCols;
          const int row0_warp = w.row0 + i * kTileM + quarter * 32;
  #pragma unroll
          for (int q = 0; q < kMyCols / kEC; ++q) {
            uint32_t orow[kEC];
            if constexpr (kEC == 8) tmem_ld_32x32b_x8(t_o + h * kMyCols + kEC * q, orow);
            else if constexpr (kEC == 16) tmem_ld_32x32b_x16(t_o + h * kMyCols + kEC * q, orow);
            else tmem_ld_32x32b_x32(t_o + h * kMyCols + kEC * q, orow);
            // a staging buffer is free once the copy engine has read the store that last used it
            const uint32_t s_buf = s_stage + static_cast<uint32_t>((q % C::kEpiBufs) * 32 * kEC * 2);
            if (lane == 0) {
              if constexpr (C::kEpiBufs == 2) bulk_wait_group_read1();
              else bulk_wait_group_read0();
            }
            tmem_wait_ld();
            if (q == kMyCols / kEC - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(bar_o_free(i));      // the next item's PV may overwrite O_i
            } else {
              __syncwarp();
            }
            // Chunks past head_dim (a padded head dim) or past the last query row are not staged
            // at all: a skipped store commits no group, and the count of groups in flight is what
            // tells when a staging buffer may be written again.
            const int col0 = h * kMyCols + kEC * q;
            if (col0 < d_out && row0_warp < seqlen) {
  #pragma unroll
              for (int e = 0; e < kEC; e += 8) {
                st_shared_v4(s_buf + static_cast<uint32_t>(lane * kEC * 2 + e * 2),
                             pack_half2(__uint_as_float(orow[e + 0]) * inv, __uint_as_float(orow[e + 1]) * inv),
                             pack_half2(__uint_as_float(orow[e + 2]) * inv, __uint_as_float(orow[e + 3]) * inv),
                             pack_half2(__uint_as_float(orow[e + 4]) * inv, __uint_as_float(orow[e + 5]) * inv),
                             pack_half2(__uint_as_float(orow[e + 6]) * inv, __uint_as_float(orow[e + 7]) * inv));
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&tm_o, s_buf, col0, row0_warp, w.bh);
                bulk_commit_group();
              }
            }
          }
          ++items;
        }
      }
      // This warp's stores of O have been read out of shared memory (the CTA may give it back);
      // their writes to global memory are complete when the kernel is.
      if (lane == 0) bulk_wait_group_read0();
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Self-test of the bounded wait: one CTA waits on an mbarrier that nobody ever arrives on.
// The wait gives up after `limit_ns`, records 0x7e57 in the status word and the kernel
// returns normally, leaving the context usable.
__global__ void fa8_expired_wait_kernel(int* status, int* host_status, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  __syncthreads();
  const WaitCtx w{&abort_flag, status, host_status, limit_ns};
  wait_bounded(w, smem_u32(&bar), 0, 0x7e57);
}

cudaError_t launch_expired_wait(int* status, int* host_status, unsigned long long limit_ns, cudaStream_t stream) {
  fa8_expired_wait_kernel<<<1, 32, 0, stream>>>(status, host_status, limit_ns);
  return cudaGetLastError();
}

// ------------------------------------------------------------------- launcher
// Chooses the work items of one launch (rows_per_item, n_pairs, fold, n_units of KernelArgs).
// Large problems: items of both query tiles, causal ones folded into equal-cost units - the
// steady state of the kernel.  When that leaves more than half of the SMs without work, the
// finer plans that still fit one wave of the grid are weighed by an estimate of the longest
// unit in 64-key steps: an item costs its sub-blocks plus kBoundarySteps (pipeline ramp at each
// item), and a step of a one-tile item costs kSingleStep of a two-tile one (eight softmax
// warps instead of sixteen share the special-function unit).  Both constants are fits to
// launches of 16-64 slices of 1024-4096 rows: a step 0.6 us, a boundary 3 us, one-tile steps
// 0.41 us.  Plans of several waves of one-tile items were measured too and lose (the boundary
// is paid per tile).  A tile's result does not depend on the plan: each tile is computed by
// its own warps from its own tensor-memory columns in either.
#ifndef FA8_PLAN
#define FA8_PLAN 0          // 0 choose; 1-4 force candidate 0-3 (measurement builds)
#endif
template <int kTiles, bool kCausal>
static void plan_work(KernelArgs& a, int sms) {
  constexpr double kBoundarySteps = 5.0, kSingleStep = 0.68;
  const int64_t slices = a.n_slices;
  const int n_tiles = (a.seqlen + kTileM - 1) / kTileM;
  struct Plan { int rows, fold; };
  const Plan cand[4] = {{kTiles * kTileM, kCausal ? 1 : 0}, {kTileM, kCausal ? 1 : 0},
                        {kTiles * kTileM, 0}, {kTileM, 0}};
  auto items_of = [&](const Plan& p) { return (a.seqlen + p.rows - 1) / p.rows; };
  auto units_of = [&](const Plan& p) {
    const int n = items_of(p);
    return slices * (p.fold ? (n + 1) / 2 : n);
  };
  auto steps_of = [&](const Plan& p) -> double {        // the longest unit, in two-tile steps
    const int n = items_of(p);
    auto item = [&](int idx) {
      const int last_tile = min(idx * (p.rows / kTileM) + p.rows / kTileM - 1, n_tiles - 1);
      const int col_end = kCausal ? min((last_tile + 1) * kTileM, a.seqlen_k) : a.seqlen_k;
      return (col_end + kSubN - 1) / kSubN + kBoundarySteps;
    };
    const double unit = (p.fold && n > 1) ? item(n - 1) + item(0) : item(n - 1);
    return unit * ((p.rows == kTileM && kTiles == 2) ? kSingleStep : 1.0);
  };
  int best = 0;
  if (FA8_PLAN > 0) {
    best = FA8_PLAN - 1;
  } else if (2 * units_of(cand[0]) <= sms) {
    double best_steps = steps_of(cand[0]);
    for (int c = 1; c < 4; ++c) {
      if (kTiles == 1 && cand[c].rows != cand[0].rows) continue;
      if (!kCausal && c >= 2) continue;
      if (units_of(cand[c]) > sms) continue;      // one wave (unfolded causal items differ in cost)
      const double st = steps_of(cand[c]);
      if (st < 0.95 * best_steps) { best = c; best_steps = st; }
    }
  }
  a.rows_per_item = cand[best].rows;
  a.fold = cand[best].fold;
  a.n_pairs = items_of(cand[best]);
  a.n_units = static_cast<int>(units_of(cand[best]));
}

template <int D>
static constexpr int smem_bytes_for() { return Cfg<D>::kSmemBytes; }

template <int D, bool kCausal, bool kVNatural, bool kE5M2>
static cudaError_t launch_one(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                              const CUtensorMap& to, const KernelArgs& args, cudaStream_t stream) {
  auto kernel = &fa8_fwd_kernel<D, kCausal, kVNatural, kE5M2>;
  constexpr int smem = Cfg<D>::kSmemBytes;
  // Per device and kernel variant: the shared-memory opt-in is made once, and the SM count is
  // remembered (0 = not yet).  Two host threads making their first call together both set the
  // attribute and store the same count, which is harmless; the atomic makes the hand-over of
  // the count well defined.
  static std::atomic<int> sm_count[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool cached = dev >= 0 && dev < 64;
  int sms = cached ? sm_count[dev].load(std::memory_order_acquire) : 0;
  if (sms == 0) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    if (sms <= 0) return cudaErrorInvalidDevice;
    if (cached) sm_count[dev].store(sms, std::memory_order_release);
  }
  // Persistent grid: one CTA per SM (shared and tensor memory allow no more), each walking
  // its share of the work units.
  KernelArgs a = args;
  plan_work<Cfg<D>::kTiles, kCausal>(a, sms);
  dim3 grid(a.n_units < sms ? a.n_units : sms, 1, 1);
  kernel<<<grid, kThreads, smem, stream>>>(tq, tk, tv, to, a);
  return cudaGetLastError();
}

template <int D, bool kCausal>
static cudaError_t launch_layout(bool v_natural, bool e5m2, const CUtensorMap& tq, const CUtensorMap& tk,
                                 const CUtensorMap& tv, const CUtensorMap& to, const KernelArgs& args,
                                 cudaStream_t stream) {
  if (v_natural) {
    return e5m2 ? launch_one<D, kCausal, true, true>(tq, tk, tv, to, args, stream)
                : launch_one<D, kCausal, true, false>(tq, tk, tv, to, args, stream);
  }
  return e5m2 ? launch_one<D, kCausal, false, true>(tq, tk, tv, to, args, stream)
              : launch_one<D, kCausal, false, false>(tq, tk, tv, to, args, stream);
}

bool plan_fwd(int head_dim, bool causal, KernelArgs& a, int sms) {
  if (sms <= 0) return false;
  if (head_dim == 256) {
    causal ? plan_work<Cfg<256>::kTiles, true>(a, sms) : plan_work<Cfg<256>::kTiles, false>(a, sms);
  } else if (head_dim == 64 || head_dim == 128) {
    causal ? plan_work<2, true>(a, sms) : plan_work<2, false>(a, sms);
  } else {
    return false;
  }
  return true;
}
static_assert(Cfg<64>::kTiles == 2 && Cfg<128>::kTiles == 2, "plan_fwd assumes two query tiles per CTA at head dims 64 and 128");

cudaError_t launch_fwd(int head_dim, bool causal, bool v_natural, bool e5m2, const CUtensorMap& tq,
                       const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to, const KernelArgs& args,
                       cudaStream_t stream) {
  if (head_dim == 128) {
    return causal ? launch_layout<128, true>(v_natural, e5m2, tq, tk, tv, to, args, stream)
                  : launch_layout<128, false>(v_natural, e5m2, tq, tk, tv, to, args, stream);
  }
  if (head_dim == 64) {
    return causal ? launch_layout<64, true>(v_natural, e5m2, tq, tk, tv, to, args, stream)
                  : launch_layout<64, false>(v_natural, e5m2, tq, tk, tv, to, args, stream);
  }
  if (head_dim == 256) {
    return causal ? launch_layout<256, true>(v_natural, e5m2, tq, tk, tv, to, args, stream)
                  : launch_layout<256, false>(v_natural, e5m2, tq, tk, tv, to, args, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace fa8

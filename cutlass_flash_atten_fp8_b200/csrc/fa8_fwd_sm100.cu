// FP8 (e4m3) flash-attention forward for sm_100a.
//
// Replaces the reference's Ada kernel flash_attention_v2_cutlass_kernel
// (csrc/flash_attention.cu:330-584) together with its tile traits
// (csrc/kernel_traits.h:33-130), FP8 mma.sync atoms (csrc/mma_sm89.hpp,
// csrc/mma_traits_sm89.hpp) and the C->A register shuffle (csrc/reg2reg.h).
//
// One CTA owns two 128-row query tiles of one (batch, head) slice and walks the
// key/value sequence; K and V^T arrive as 128-position tiles, the arithmetic runs
// on 64-position sub-blocks so that each query tile has TWO score buffers in
// tensor memory and its next S = Q K^T is computed while the softmax of the
// current sub-block is still running:
//
//   warp 17     TMA producer: Q tiles once, then K_j / V_j tiles into a ring of
//               shared-memory slots, each guarded by a full/empty mbarrier pair.
//   warp 16     MMA issuer (one elected lane): S_i[sb&1] = Q_i K_sb^T (M128 N64)
//               and O_i += P_i(sb) V_sb (M128 N=head_dim) as tcgen05.mma
//               kind::f8f6f4 with fp32 accumulators in tensor memory; completion
//               is signalled with tcgen05.commit on mbarriers.
//   warps 0-7   online softmax for query tile 0, warps 8-15 for tile 1.  A TMEM lane
//               is a query row (tcgen05.ld 32x32b: one row per thread, no shuffles).
//               Warps w and w+4 of a tile own the same 32 rows: the first takes the
//               even sub-blocks (S buffer 0), the second the odd ones (S buffer 1),
//               so four softmax warps per scheduler keep the special-function and
//               FMA pipes fed.  exp2 with the scale folded in, row sum from the fp32
//               probabilities, P re-quantised to e4m3 and written back to TMEM over
//               its own S buffer as the A operand of the second GEMM; fp32 rescale of
//               O in TMEM when the row maximum has to be raised.
//
// TMEM columns: tile i has S buffers at 128*i and 128*i+64 (64 fp32 columns each;
// P, 64 e4m3 = 16 columns, overlays the buffer it was computed from) and O_i at
// 256 + head_dim*i.
//
// Numerics follow the reference: P = exp(scale*(S - m)) unnormalised, converted to
// e4m3 round-to-nearest-even/saturating (csrc/flash_attention.cu:163-179,524), the
// row sum taken from fp32 P (:239-240,:264-271), final O/l with the zero/NaN guard
// (:542-554).  Differences: the output is fp16 (the reference rounds it to e4m3,
// :556-557); m is the exact row maximum after the first sub-block and is then
// raised only when a sub-block would push P beyond 2^8 (the reference raises it on
// every block, :233-273), which leaves O/l unchanged up to the rounding of P.
//
// Every mbarrier wait is bounded: when a wait runs out, the waiting thread
// records a code in the caller's status word, raises a CTA-wide abort flag and
// every role leaves its loop, drains its own copies / MMAs (bounded again),
// frees tensor memory and returns.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "fa8_kernel.h"
#include "ptx_sm100.cuh"

namespace fa8 {

namespace {

constexpr int kTileM = 128;        // query rows per tile = TMEM lanes
constexpr int kBlockN = 128;       // key/value positions per TMA tile
constexpr int kSubN = 64;          // key/value positions per MMA / softmax sub-block
constexpr int kMmaWarp = 16;
constexpr int kLoadWarp = 17;
constexpr int kThreads = 576;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemO = 256;   // first O column; S_0 at 0, S_1 at 128

template <int D>
struct Cfg {
  static_assert(D == 64 || D == 128, "head_dim must be 64 or 128");
  static constexpr int kTileBytes = 128 * D;           // Q, K and V^T tiles alike
  static constexpr int kSlots = (D == 128) ? 8 : 16;   // ring slots, one K or V tile each
  static constexpr int kQBytes = 2 * kTileBytes;
  static constexpr int kRingBytes = kSlots * kTileBytes;
  static constexpr int kBarOffset = kQBytes + kRingBytes;
  // row-group scratch shared by the two warps of a 32-row group, see RowGroupShared
  static constexpr int kGroupBytes = 8 * 672;
  static constexpr int kNumBars = 2 /*q_full*/ + 2 * kSlots + 4 /*s_full*/ + 4 /*p_full*/ + 2 /*o_done*/ + 2 /*o_final*/ + 1 /*drain*/;
  static constexpr int kSmemBytes = kBarOffset + kNumBars * 8 + 16 /*tmem ptr, abort*/ + kGroupBytes + 1024 /*align*/;
  // Q and K rows are D bytes long: one 128-byte swizzle row for D=128, a 64-byte one for D=64.
  static constexpr uint32_t kQKLayout = (D == 128) ? 2u : 4u;   // UMMA SWIZZLE_128B / SWIZZLE_64B
  static constexpr uint32_t kQKSbo = 8 * D;                      // bytes between 8-row groups
};

// Shared-memory matrix descriptor for a K-major swizzled operand tile
// (rows of `row_bytes` <= 128, eight rows per swizzle atom).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) |
         (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) |
         (static_cast<uint64_t>(layout_type) << 61);
}
// kind::f8f6f4 instruction descriptor: e4m3 x e4m3 -> f32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

struct WaitCtx {
  volatile int* abort_flag;
  int* status;
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
        return false;
      }
    }
  }
}

// ------------------------------------------------------------ softmax passes
// Which of the 16 element pairs of a 32-column chunk take their exponential on the FMA
// pipe instead of the special-function unit (bit p = pair p).
#ifndef FA8_POLY_PAIR_MASK
#define FA8_POLY_PAIR_MASK 0x1111
#endif
// P may grow to kLazyLimit (<= 448, the e4m3 maximum, with room for the polynomial
// path's clamp at 2^8) before the row maximum is raised.
constexpr float kLazyLimit = 128.f;

// Four fp32 -> four e4m3 in one word (ascending index = ascending byte).
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}

// One pass over 32 of the scores of this thread's row (TMEM columns t_cols..+31):
// P = 2^(c*s + neg_mc), packed to e4m3 into pk[8] (four per word, ascending key
// index); adds the fp32 P into the two packed accumulators ls[].  Columns >= lim
// (relative to the first of the 32) are masked.
//
// kAllowFma: the pairs selected by FA8_POLY_PAIR_MASK evaluate 2^x on the FMA pipe:
//   y  = sat(s*c/128 + (neg_mc + 120)/128)     x = 128y - 120 clamped to [-120, 8]
//   t  = 128y + (M - 120),  M = 1.5*2^23       t = M + n, n = round(x)
//   f  = 128y - (t - (M - 120)) = x - n        |f| <= 1/2
//   2^x = poly3(f) * 2^n                       cubic minimax, rel. error 7.5e-5; the
//                                              exponent is added in the integer domain
// A value clamped from above reads 2^8 > kLazyLimit, so the caller's overflow test
// still fires.
template <bool kAllowFma>
__device__ __forceinline__ void softmax_chunk(uint32_t t_cols, int lim, float c, float neg_mc,
                                              uint32_t* pk, f32x2_t (&ls)[2]) {
  const f32x2_t c2 = pack2(c, c), nm2 = pack2(neg_mc, neg_mc);
  const float c128 = c * (1.f / 128.f), nm128 = (neg_mc + 120.f) * (1.f / 128.f);
  const f32x2_t k128 = pack2(128.f, 128.f);
  const f32x2_t magicp2 = pack2(12582912.f - 120.f, 12582912.f - 120.f);
  const f32x2_t neg1 = pack2(-1.f, -1.f);
  const f32x2_t pc3 = pack2(0.055171654f, 0.055171654f), pc2 = pack2(0.24261114f, 0.24261114f);
  const f32x2_t pc1 = pack2(0.69326097f, 0.69326097f), pc0 = pack2(0.99992806f, 0.99992806f);
  uint32_t s[32];
  tmem_ld_32x32b_x32(t_cols, s);
  tmem_wait_ld();
  if (lim < 32) {
#pragma unroll
    for (int e = 0; e < 32; ++e)
      if (e >= lim) s[e] = 0xff800000u;   // -inf
  }
#pragma unroll
  for (int e = 0; e < 32; e += 4) {
    float p[4];
#pragma unroll
    for (int u = 0; u < 4; u += 2) {
      const float s0 = __uint_as_float(s[e + u]), s1 = __uint_as_float(s[e + u + 1]);
      const bool on_fma = kAllowFma && (((FA8_POLY_PAIR_MASK) >> ((e + u) / 2)) & 1);
      if (on_fma) {
        const f32x2_t y2 = pack2(fma_sat(s0, c128, nm128), fma_sat(s1, c128, nm128));
        const f32x2_t t2 = fma2(y2, k128, magicp2);
        const f32x2_t nneg2 = fma2(t2, neg1, magicp2);          // -(n + 120)
        const f32x2_t f2 = fma2(y2, k128, nneg2);
        f32x2_t r2 = fma2(f2, pc3, pc2);
        r2 = fma2(r2, f2, pc1);
        r2 = fma2(r2, f2, pc0);
        float r0, r1, t0, t1;
        unpack2(r2, r0, r1);
        unpack2(t2, t0, t1);
        p[u] = __int_as_float(__float_as_int(r0) + (__float_as_int(t0) << 23));
        p[u + 1] = __int_as_float(__float_as_int(r1) + (__float_as_int(t1) << 23));
      } else {
        float x0, x1;
        unpack2(fma2(pack2(s0, s1), c2, nm2), x0, x1);
        p[u] = ex2_approx(x0);
        p[u + 1] = ex2_approx(x1);
      }
      ls[u >> 1] = add2(ls[u >> 1], pack2(p[u], p[u + 1]));
    }
    pk[e / 4] = pack4_e4m3(p[0], p[1], p[2], p[3]);
  }
}

// P of one 64-key sub-block of this thread's row -> pk[16]; returns the fp32 row sum.
template <bool kAllowFma>
__device__ __forceinline__ float softmax_pass(uint32_t t_sb, int lim, float c, float neg_mc,
                                              uint32_t (&pk)[16]) {
  f32x2_t ls[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
  softmax_chunk<kAllowFma>(t_sb, lim, c, neg_mc, pk, ls);
  softmax_chunk<kAllowFma>(t_sb + 32, lim - 32, c, neg_mc, pk + 8, ls);
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

// What the two warps of a 32-row group share (672 bytes per group): the row maxima the
// exponentials are taken against, a version counter bumped whenever they are raised,
// and each warp's final (row sum, maximum it refers to) for the epilogue.
struct RowGroupShared {
  volatile float m[32];
  volatile uint32_t version;
  uint32_t pad[7];
  volatile float l_part[2][32];
  volatile float m_part[2][32];
};
static_assert(sizeof(RowGroupShared) == 672, "RowGroupShared layout");

}  // namespace

template <int D, bool kCausal>
__global__ void __launch_bounds__(kThreads, 1)
fa8_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const KernelArgs args) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t s_q = smem_base;
  const uint32_t s_ring = smem_base + C::kQBytes;
  const uint32_t s_bar = smem_base + C::kBarOffset;
  auto bar_q_full = [&](int i) { return s_bar + 8u * i; };
  auto bar_kv_full = [&](int s) { return s_bar + 8u * (2 + s); };
  auto bar_kv_empty = [&](int s) { return s_bar + 8u * (2 + C::kSlots + s); };
  auto bar_s_full = [&](int i, int h) { return s_bar + 8u * (2 + 2 * C::kSlots + 2 * i + h); };
  // One P barrier per S buffer: a softmax warp may run one sub-block ahead of its
  // siblings (the next S is already there), never two.
  auto bar_p_full = [&](int i, int h) { return s_bar + 8u * (6 + 2 * C::kSlots + 2 * i + h); };
  auto bar_o_done = [&](int i) { return s_bar + 8u * (10 + 2 * C::kSlots + i); };
  // Completes once, after the last PV of tile i.  (The epilogue cannot use o_done: a warp
  // that ran ahead of its siblings may get there two phases early, which a parity wait
  // cannot tell from "done".)
  auto bar_o_final = [&](int i) { return s_bar + 8u * (12 + 2 * C::kSlots + i); };
  const uint32_t bar_drain = s_bar + 8u * (14 + 2 * C::kSlots);
  volatile uint32_t* tmem_ptr_slot =
      reinterpret_cast<volatile uint32_t*>(smem_gen + C::kBarOffset + C::kNumBars * 8);
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(smem_gen + C::kBarOffset + C::kNumBars * 8 + 4);
  RowGroupShared* groups =
      reinterpret_cast<RowGroupShared*>(smem_gen + C::kBarOffset + C::kNumBars * 8 + 16);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int seqlen = args.seqlen;
  // Causal work grows with the query position: schedule the long tiles first.
  const int pair = kCausal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int bh = blockIdx.y;
  const int row0 = pair * 2 * kTileM;                 // first query row of tile 0
  // Number of 64-position sub-blocks each tile visits (0 = the tile lies past the end).
  int nsb_t[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r0 = row0 + i * kTileM;
    int n = 0;
    if (r0 < seqlen) {
      const int col_end = kCausal ? min(r0 + kTileM, seqlen) : seqlen;   // one past the last visible key
      n = (col_end + kSubN - 1) / kSubN;
    }
    nsb_t[i] = n;
  }
  const int nsb = max(nsb_t[0], nsb_t[1]);
  const int nb = (nsb + 1) / 2;                       // K/V tiles to load

  const WaitCtx wctx{abort_flag, args.status, args.timeout_ns};

  if (threadIdx.x == 0) {
    // A status word that is already non-zero (an earlier CTA of this launch gave up, or the
    // caller did not clear it) makes the CTA return at once: a failed launch then costs one
    // wait limit, not one per wave of CTAs.
    *abort_flag = (args.status != nullptr && *reinterpret_cast<volatile int*>(args.status) != 0) ? 2 : 0;
    for (int i = 0; i < 2; ++i) mbar_init(bar_q_full(i), 1);
    for (int s = 0; s < C::kSlots; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s_full(i, 0), 1);
      mbar_init(bar_s_full(i, 1), 1);
      mbar_init(bar_p_full(i, 0), 4);   // one arrive per softmax warp
      mbar_init(bar_p_full(i, 1), 4);
      mbar_init(bar_o_done(i), 1);
      mbar_init(bar_o_final(i), 1);
    }
    mbar_init(bar_drain, 1);
    for (int g = 0; g < 8; ++g) groups[g].version = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;
  const bool skip_cta = (*abort_flag == 2);
  __syncthreads();            // nobody raises the flag before everyone has read it

  if (skip_cta) {
    // fall through to the teardown
  } else if (warp == kLoadWarp) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      bool ok = true;
      int it = 0;   // K_j is load 2j, V_j is load 2j+1
      auto load_kv = [&](const CUtensorMap* tm, int c0, int c1) {
        const int slot = it % C::kSlots;
        const uint32_t round = static_cast<uint32_t>(it / C::kSlots);
        if (ok) ok = wait_bounded(wctx, bar_kv_empty(slot), (round & 1u) ^ 1u, 0x100 + slot);
        if (ok) {
          mbar_arrive_expect_tx(bar_kv_full(slot), C::kTileBytes);
          tma_load_3d(s_ring + slot * C::kTileBytes, tm, bar_kv_full(slot), c0, c1, bh);
          ++it;
        }
      };
      load_kv(&tm_k, 0, 0);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (nsb_t[i] > 0) {
          mbar_arrive_expect_tx(bar_q_full(i), C::kTileBytes);
          tma_load_3d(s_q + i * C::kTileBytes, &tm_q, bar_q_full(i), 0, row0 + i * kTileM, bh);
        }
      }
      load_kv(&tm_v, 0, 0);
      for (int j = 1; j < nb && ok; ++j) {
        load_kv(&tm_k, 0, j * kBlockN);
        load_kv(&tm_v, j * kBlockN, 0);
      }
      if (!ok) {
        // Abort: let this CTA's copies that are still in flight land before the
        // shared memory is given back.  Loads [it - kSlots, it) may be pending.
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
          if (nsb_t[i] > 0) {
            const uint64_t t0 = global_timer_ns();
            while (!mbar_try_wait(bar_q_full(i), 0)) {
              if (global_timer_ns() - t0 > 20000000ull) break;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t kIdescQK = umma_idesc(kTileM, kSubN);
      constexpr uint32_t kIdescPV = umma_idesc(kTileM, D);
      bool ok = true;
      auto slot_of = [&](int load) { return load % C::kSlots; };
      auto parity_of = [&](int load) { return static_cast<uint32_t>(load / C::kSlots) & 1u; };
      auto wait_load = [&](int load) {
        if (ok) ok = wait_bounded(wctx, bar_kv_full(slot_of(load)), parity_of(load), 0x200 + slot_of(load));
      };
      // S_i[h] = Q_i K_sb^T for sub-block sb = 2j+h: rows 64h..64h+63 of tile K_j;
      // D/32 steps of K=32 bytes along the swizzled rows.
      auto issue_qk = [&](int i, int h, int load) {
        const uint64_t dq = umma_desc(s_q + i * C::kTileBytes, C::kQKSbo, C::kQKLayout);
        const uint64_t dk = umma_desc(s_ring + slot_of(load) * C::kTileBytes + h * kSubN * D,
                                      C::kQKSbo, C::kQKLayout);
#pragma unroll
        for (int k = 0; k < D / 32; ++k)
          mma_f8_ss(tmem_base + i * kBlockN + h * kSubN, dq + 2u * k, dk + 2u * k, kIdescQK, k > 0);
      };
      // O_i (+)= P_i(sb) V_sb: P is 128 rows x 64 e4m3 = 16 TMEM columns over S_i[h];
      // the V^T tile is D rows of 128 key positions (K-major, 128-byte swizzle), of which
      // sub-block h covers bytes 64h..64h+63 of every row = K-steps 2h and 2h+1.
      auto issue_pv = [&](int i, int h, int load, bool acc) {
        const uint64_t dv = umma_desc(s_ring + slot_of(load) * C::kTileBytes, 1024u, 2u);
#pragma unroll
        for (int k = 0; k < kSubN / 32; ++k)
          mma_f8_ts(tmem_base + kTmemO + i * D, tmem_base + i * kBlockN + h * kSubN + 8u * k,
                    dv + 2u * (2 * h + k), kIdescPV, (acc || k > 0) ? 1u : 0u);
      };

      wait_load(0);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (nsb_t[i] > 0) {
          if (ok) ok = wait_bounded(wctx, bar_q_full(i), 0, 0x300 + i);
          if (ok) {
            tc_fence_after();
            issue_qk(i, 0, 0);
            tc_commit(bar_s_full(i, 0));
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (nsb_t[i] > 1 && ok) {
          issue_qk(i, 1, 0);
          tc_commit(bar_s_full(i, 1));
        }
      }
      if (ok) tc_commit(bar_kv_empty(slot_of(0)));

      for (int sb = 0; sb < nsb && ok; ++sb) {
        const int j = sb >> 1, h = sb & 1;
        const int ld_v = 2 * j + 1, ld_kn = 2 * j + 2;      // V_j and K_{j+1}
        const bool kn_loaded = (2 * j + 2 < nsb);
        if (h == 0) {
          wait_load(ld_v);
          if (kn_loaded) wait_load(ld_kn);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (sb < nsb_t[i]) {
            if (ok) ok = wait_bounded(wctx, bar_p_full(i, h), static_cast<uint32_t>(sb >> 1) & 1u, 0x400 + i);
            if (ok) {
              tc_fence_after();
              issue_pv(i, h, ld_v, sb > 0);
              tc_commit(bar_o_done(i));                    // phase sb: PV_i(0..sb) complete
              if (sb == nsb_t[i] - 1) tc_commit(bar_o_final(i));
              if (sb + 2 < nsb_t[i]) {
                issue_qk(i, h, ld_kn);
                tc_commit(bar_s_full(i, h));               // S_i[h] now holds sub-block sb+2
              }
            }
          }
        }
        if (ok && (h == 1 || sb == nsb - 1)) {
          tc_commit(bar_kv_empty(slot_of(ld_v)));
          if (h == 1 && kn_loaded) tc_commit(bar_kv_empty(slot_of(ld_kn)));
        }
      }
      if (!ok) {
        // Abort: wait (bounded) for the MMAs already issued before TMEM is freed.
        tc_commit(bar_drain);
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(bar_drain, 0)) {
          if (global_timer_ns() - t0 > 20000000ull) break;
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------- softmax + epilogue warps
    const int i = warp >> 3;                           // query tile of this warp
    const int h = (warp >> 2) & 1;                     // S buffer = parity of my sub-blocks
    const int quarter = warp & 3;                      // TMEM lane quarter = 32-row group
    const int row = quarter * 32 + lane;               // row in the tile = TMEM lane
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_sb = tmem_base + lane_sel + i * kBlockN + h * kSubN;   // my S buffer
    const uint32_t t_o = tmem_base + lane_sel + kTmemO + i * D;
    const int q_row = row0 + i * kTileM + row;         // global query row, may be >= seqlen
    const int tile_nsb = nsb_t[i];
    const int col_lim = kCausal ? min(seqlen, q_row + 1) : seqlen;   // keys this row may see
    const float c = args.scale_log2;
    RowGroupShared& grp = groups[i * 4 + quarter];
    // m is the row maximum the exponentials are taken against, shared by the two warps of
    // the row group through grp.m / grp.version: exact after sub-block 0, then raised only
    // by the exact path below.  l is this warp's share of the row sum, kept relative to m.
    // O and both shares are sums against the same m, so O/l does not depend on when m is
    // raised.
    float m = -INFINITY, l = 0.f;
    uint32_t version = 0;
    bool ok = true;

    // Brings m (and l with it) up to date with the partner's latest raise.
    auto adopt = [&]() -> bool {
      const uint32_t v = grp.version;
      if (v == version) return false;
      __threadfence_block();
      const float m_new = grp.m[lane];
      if (m != -INFINITY) l *= ex2_approx((m - m_new) * c);
      m = m_new;
      version = v;
      return true;
    };

    for (int sb = h; sb < tile_nsb; sb += 2) {
      const uint32_t ph = static_cast<uint32_t>(sb >> 1) & 1u;
      ok = wait_bounded(wctx, bar_s_full(i, h), ph, 0x500 + i);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int lim = col_lim - sb * kSubN;            // sub-block-local first masked column

      uint32_t pk[16];
      float bsum = 0.f;
      const bool have_m = (version != 0);              // warp-uniform
      if (have_m) {
        // Fast path: one pass, exponentials against the maximum known so far.
        bsum = softmax_pass<true>(t_sb, lim, c, -m * c, pk);
      }
      // P(sb) may be handed over only after the partner has handed over P(sb-1): from then
      // on nobody else can raise the maximum before PV(sb) is issued.
      if (sb > 0) {
        ok = wait_bounded(wctx, bar_p_full(i, h ^ 1), static_cast<uint32_t>((sb - 1) >> 1) & 1u, 0x800 + i);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      bool redo = adopt() || !have_m;                  // warp-uniform: version is per group
      redo = __any_sync(0xffffffffu, redo);
      // Some P above kLazyLimit implies a sum above it (all P >= 0); a false alarm only
      // costs the exact path.  Decided for the warp's 32 rows as a whole.
      bool exact = (sb == 0);
      if (!exact && !redo) exact = __any_sync(0xffffffffu, !(bsum <= kLazyLimit));
      if (!exact && redo) {
        bsum = softmax_pass<false>(t_sb, lim, c, -m * c, pk);
        exact = __any_sync(0xffffffffu, !(bsum <= kLazyLimit));
      }
      if (exact) {
        // Exact path (first sub-block, or the maximum is too low for some row of this
        // warp): true row maximum, rescale l and O, publish, redo the exponentials.
        const float m_new = fmaxf(m, row_max(t_sb, lim));
        if (sb > 0) {
          // O_i must be quiescent: PV_i(sb-1) complete; PV_i(sb) waits for this warp.
          ok = wait_bounded(wctx, bar_o_done(i), static_cast<uint32_t>(sb - 1) & 1u, 0x700 + i);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          float alpha = ex2_approx((m - m_new) * c);
          if (m == -INFINITY) alpha = 1.f;
          l *= alpha;
          rescale_o_columns(t_o, D / 32, alpha);
        }
        m = m_new;
        grp.m[lane] = m_new;
        __threadfence_block();
        __syncwarp();
        ++version;
        if (lane == 0) grp.version = version;
        bsum = softmax_pass<false>(t_sb, lim, c, (m == -INFINITY) ? 0.f : -m * c, pk);
      }
      l += bsum;
      if (sb + 2 >= tile_nsb) {                        // my last sub-block: leave my share for the epilogue
        grp.l_part[h][lane] = l;
        grp.m_part[h][lane] = m;
        __threadfence_block();
      }
      tmem_st_32x32b_x16(t_sb, pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full(i, h));
    }

    if (ok && tile_nsb > 0) {
      ok = wait_bounded(wctx, bar_o_final(i), 0, 0x600 + i);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        __threadfence_block();
        // Row sum = both warps' shares, each brought to the final maximum.
        float l_tot = 0.f, m_fin = -INFINITY;
#pragma unroll
        for (int w2 = 0; w2 < 2; ++w2)
          if (w2 < tile_nsb) m_fin = fmaxf(m_fin, grp.m_part[w2][lane]);
#pragma unroll
        for (int w2 = 0; w2 < 2; ++w2) {
          if (w2 < tile_nsb) {
            const float mp = grp.m_part[w2][lane], lp = grp.l_part[w2][lane];
            l_tot += (mp == -INFINITY) ? 0.f : lp * ex2_approx((mp - m_fin) * c);
          }
        }
        const float inv = ((l_tot == 0.f || l_tot != l_tot) ? 1.f : 1.f / l_tot) * args.o_scale;
        // Each warp of the pair writes half of the head dimension.
        __half* o_row = args.o + (static_cast<size_t>(bh) * seqlen + q_row) * D + h * (D / 2);
#pragma unroll
        for (int q = 0; q < D / 64; ++q) {
          uint32_t orow[32];
          tmem_ld_32x32b_x32(t_o + h * (D / 2) + 32 * q, orow);
          tmem_wait_ld();
          if (q_row < seqlen) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              st_global_v4(o_row + 32 * q + e,
                           pack_half2(__uint_as_float(orow[e + 0]) * inv, __uint_as_float(orow[e + 1]) * inv),
                           pack_half2(__uint_as_float(orow[e + 2]) * inv, __uint_as_float(orow[e + 3]) * inv),
                           pack_half2(__uint_as_float(orow[e + 4]) * inv, __uint_as_float(orow[e + 5]) * inv),
                           pack_half2(__uint_as_float(orow[e + 6]) * inv, __uint_as_float(orow[e + 7]) * inv));
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------- launcher
template <int D>
static constexpr int smem_bytes_for() { return Cfg<D>::kSmemBytes; }

template <int D, bool kCausal>
static cudaError_t launch_one(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                              const KernelArgs& args, int n_pairs, int bh, cudaStream_t stream) {
  auto kernel = &fa8_fwd_kernel<D, kCausal>;
  constexpr int smem = Cfg<D>::kSmemBytes;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  dim3 grid(n_pairs, bh, 1);
  kernel<<<grid, kThreads, smem, stream>>>(tq, tk, tv, args);
  return cudaGetLastError();
}

cudaError_t launch_fwd(int head_dim, bool causal, const CUtensorMap& tq, const CUtensorMap& tk,
                       const CUtensorMap& tv, const KernelArgs& args, int n_pairs, int bh,
                       cudaStream_t stream) {
  if (head_dim == 128) {
    return causal ? launch_one<128, true>(tq, tk, tv, args, n_pairs, bh, stream)
                  : launch_one<128, false>(tq, tk, tv, args, n_pairs, bh, stream);
  }
  if (head_dim == 64) {
    return causal ? launch_one<64, true>(tq, tk, tv, args, n_pairs, bh, stream)
                  : launch_one<64, false>(tq, tk, tv, args, n_pairs, bh, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace fa8

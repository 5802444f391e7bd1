// Internal interface between the C-ABI layer (fa8_capi.cu) and the sm_100a
// kernel (fa8_fwd_sm100.cu).  Not installed; callers use include/fa8_b200.h.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace fa8 {

// By-value kernel arguments.  Plays the role of the reference's
// Flash_fwd_params (csrc/flash.h:6-61) minus its dead fields; tensor addresses
// and strides travel in the three TMA descriptors instead.
struct KernelArgs {
  __half* o;                      // [batch*heads, seqlen, head_dim] fp16
  int seqlen;                     // query rows per slice
  int seqlen_k;                   // key/value rows per slice
  int head_dim;                   // row length of Q, K, V and O (<= the kernel's head dim)
  int heads;                      // query heads per batch entry
  int heads_kv;                   // K/V heads per batch entry (divides heads)
  int n_slices;                   // batch * heads
  // Work plan, filled in by launch_fwd (see plan_work): the caller sets n_slices only.
  int rows_per_item;              // query rows of a work item: 256 (two 128-row tiles) or 128 (one tile)
  int n_pairs;                    // work items per slice: ceil(seqlen / rows_per_item)
  int fold;                       // causal: a unit is item f followed by item n-1-f of a slice (equal cost)
  int n_units;                    // work units of the persistent grid (see get_item)
  float scale_log2;               // softmax_scale * log2(e)
  float o_scale;                  // multiplies O/l (1 = reference behaviour)
  const float* descale_q;         // optional device scalars: softmax scale *= dq*dk, O *= dv
  const float* descale_k;
  const float* descale_v;
  int descale_per_head;           // the three are arrays: [batch*heads] for Q, [batch*heads_kv] for K, V
  float* lse;                     // optional [batch*heads, seqlen] fp32: log-sum-exp of the scaled scores
  float softmax_scale;            // as given by the caller (natural-log units, for lse)
  int* status;                    // device word; non-zero after a bounded wait expired (later CTAs then return at once)
  int* host_status;               // optional word in mapped host memory: receives the same code, so that
                                  // the host learns of it without a copy or a synchronisation
  unsigned long long timeout_ns;  // bound of every mbarrier wait
};

// Launches the persistent forward kernel for head_dim in {64,128,256}.
// v_natural: V is [slices, seqlen, head_dim] (tv describes it like K) instead of the
// reference's transposed [slices, head_dim, seqlen].
// e5m2: Q, K, V (and P) are e5m2 instead of e4m3.
// to: O as a 3-D fp16 tensor {head_dim, seqlen, slices} with a {epi_cols(head_dim), 32, 1} box
// (see epi_cols below), through which the softmax warps store their rows.
cudaError_t launch_fwd(int head_dim, bool causal, bool v_natural, bool e5m2, const CUtensorMap& tq,
                       const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to, const KernelArgs& args,
                       cudaStream_t stream);

// The work plan launch_fwd would choose on a GPU of `sms` SMs: fills rows_per_item, n_pairs,
// fold and n_units of `a` from its seqlen, seqlen_k and n_slices.  Host arithmetic only.
// head_dim is the kernel's (64, 128 or 256); false for any other or for sms <= 0.
bool plan_fwd(int head_dim, bool causal, KernelArgs& a, int sms);

// fp16 columns per store box of the kernel built for head dim 64, 128 or 256.
#ifndef FA8_EPI_COLS_128
#define FA8_EPI_COLS_128 16
#endif
constexpr int epi_cols(int kernel_head_dim) { return kernel_head_dim == 128 ? FA8_EPI_COLS_128 : 32; }

// One warp waits (bounded by limit_ns) on a barrier that never completes; see fa8_selftest_expired_wait.
cudaError_t launch_expired_wait(int* status, int* host_status, unsigned long long limit_ns, cudaStream_t stream);

// Amax quantisation fp16/bf16 -> e4m3 (fa8_quant.cu) of n_seg contiguous segments of n
// elements each: amax[s] = max|src_s|, dst_s = e4m3(src_s * 448 / amax[s]),
// descale[s] = amax[s] / 448 (descale may be null).
cudaError_t launch_quantize(const void* src, bool bf16, void* dst, int64_t n, int n_seg, float* amax,
                            float* descale, cudaStream_t stream);

}  // namespace fa8

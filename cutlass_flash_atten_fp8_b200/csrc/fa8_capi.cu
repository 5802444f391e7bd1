// C-ABI layer of libfa8_b200.so: argument validation, TMA descriptor
// construction and kernel launch.  Declared in include/fa8_b200.h.
//
// Stands where the reference has flash_attention_v2_cutlass
// (csrc/flash_attention.cu:639-668), set_params_fprop (:277-318) and the
// dispatch chain run_flash_attn_cutlass / run_flash_fwd_ / run_flash_fwd
// (:586-637).  No torch types, no exceptions, no exit().
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "fa8_b200.h"
#include "fa8_kernel.h"

namespace {

thread_local char g_detail[320] = "";

void set_detail(const char* what, const char* msg) {
  std::snprintf(g_detail, sizeof(g_detail), "%s: %s", what, msg ? msg : "?");
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is fetched through the runtime so that the library
// carries no link-time dependency on libcuda.
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 3-D byte tensor {inner, mid, outer} with a {box_inner, box_mid, 1} tile.
bool make_map_3d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t mid, uint64_t outer,
                 uint32_t box_inner, uint32_t box_mid, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    set_detail("cudaGetDriverEntryPoint", "cuTensorMapEncodeTiled not available");
    return false;
  }
  cuuint64_t dims[3] = {inner, mid, outer};
  cuuint64_t strides[2] = {inner, inner * mid};   // bytes, for dims 1 and 2
  cuuint32_t box[3] = {box_inner, box_mid, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[64];
    std::snprintf(buf, sizeof(buf), "CUresult %d", static_cast<int>(r));
    set_detail("cuTensorMapEncodeTiled", buf);
    return false;
  }
  return true;
}

// O: 3-D fp16 tensor {head_dim, seqlen, slices}, stored through {box_cols, 32, 1} boxes, no swizzle.
bool make_map_o(CUtensorMap* out, void* base, uint64_t head_dim, uint64_t seqlen, uint64_t slices, uint32_t box_cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    set_detail("cudaGetDriverEntryPoint", "cuTensorMapEncodeTiled not available");
    return false;
  }
  cuuint64_t dims[3] = {head_dim, seqlen, slices};
  cuuint64_t strides[2] = {head_dim * 2, head_dim * seqlen * 2};   // bytes, for dims 1 and 2
  cuuint32_t box[3] = {box_cols, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[64];
    std::snprintf(buf, sizeof(buf), "CUresult %d", static_cast<int>(r));
    set_detail("cuTensorMapEncodeTiled (O)", buf);
    return false;
  }
  return true;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The library's own status word, one per device that loads the module: used when the caller
// passes none, so that an expired wait is never lost.
__device__ int g_status_word;

// Per-device state, set up by the first call on that device:
//   dev_word   address of g_status_word on the device;
//   host_flag  one int of mapped, pinned host memory that a kernel stores its code into when
//              a bounded wait runs out (whatever status word the launch was given).  The host
//              reads it at the start of every later call: a failed launch is then reported by
//              the next call at the latest, with no copy and no synchronisation in between.
struct DeviceState {
  std::once_flag once;
  bool ok = false;
  int* dev_word = nullptr;
  volatile int* host_flag = nullptr;
  int* host_flag_dev = nullptr;
};
constexpr int kMaxDevices = 64;
DeviceState g_dev[kMaxDevices];

DeviceState* device_state() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  DeviceState& st = g_dev[dev];
  std::call_once(st.once, [&st] {
    void* word = nullptr;
    void* host = nullptr;
    void* host_dev = nullptr;
    if (cudaGetSymbolAddress(&word, g_status_word) != cudaSuccess) return;    // zero at module load
    if (cudaHostAlloc(&host, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return;
    *static_cast<volatile int*>(host) = 0;
    if (cudaHostGetDevicePointer(&host_dev, host, 0) != cudaSuccess) {
      cudaFreeHost(host);
      return;
    }
    st.dev_word = static_cast<int*>(word);
    st.host_flag = static_cast<volatile int*>(host);
    st.host_flag_dev = static_cast<int*>(host_dev);
    st.ok = true;
  });
  if (!st.ok) {
    cudaGetLastError();     // the failure is reported by the caller as "no state", not left pending
    return nullptr;
  }
  return &st;
}

// Scratch of fa8_quantize_e4m3_segments_noalloc: the per-segment |x| maxima that the first pass
// accumulates and the second pass reads.  A file-scope device array instead of memory from the
// allocator: 16 KB on every GPU that loads the library, held until the process exits, shared by
// every call (so it keeps the last call's contents and is cleared at the start of each).
static __device__ __align__(256) float g_quant_amax_scratch[FA8_NOALLOC_MAX_SEGMENTS];

// In host code the array's name is only a handle for the runtime, not an address a kernel can
// use: the device address is asked for once per device, with that device current, and kept.
std::atomic<float*> g_quant_scratch_addr[kMaxDevices];

float* quant_scratch(cudaError_t* err) {
  *err = cudaSuccess;
  int dev = -1;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  const bool cached = dev >= 0 && dev < kMaxDevices;
  if (cached) {
    float* known = g_quant_scratch_addr[dev].load(std::memory_order_acquire);
    if (known) return known;
  }
  void* addr = nullptr;
  *err = cudaGetSymbolAddress(&addr, g_quant_amax_scratch);
  if (*err != cudaSuccess) return nullptr;
  if (cached) g_quant_scratch_addr[dev].store(static_cast<float*>(addr), std::memory_order_release);
  return static_cast<float*>(addr);
}

// Collects a failure an earlier launch on this device left in the host flag: clears the flag
// and, stream-ordered, the device words, and returns the code (0 = none).
int collect_earlier_failure(DeviceState* st, int32_t* caller_word, cudaStream_t stream) {
  if (!st) return 0;
  const int code = *st->host_flag;
  if (code == 0) return 0;
  *st->host_flag = 0;
  cudaMemsetAsync(st->dev_word, 0, sizeof(int), stream);
  if (caller_word) cudaMemsetAsync(caller_word, 0, sizeof(int), stream);
  return code;
}

}  // namespace

extern "C" {

int fa8_version(void) { return 109; }

const char* fa8_error_string(int code) {
  switch (code) {
    case FA8_OK: return "ok";
    case FA8_ERR_BAD_ARG: return "bad argument (null or misaligned pointer, non-positive size or scale)";
    case FA8_ERR_UNSUPPORTED:
      return "unsupported shape or layout (head_dim must be a multiple of 32 up to 256; with V transposed the "
             "key/value length must be a multiple of 16)";
    case FA8_ERR_CUDA: return "CUDA call failed";
    case FA8_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel expired";
    default: return "unknown fa8 status";
  }
}

const char* fa8_last_error_detail(void) { return g_detail; }

int fa8_supported(int32_t seqlen_k, int32_t head_dim, int32_t v_layout) {
  if (head_dim < 32 || head_dim > 256 || (head_dim % 32) != 0) return FA8_ERR_UNSUPPORTED;
  if (v_layout != FA8_V_TRANSPOSED && v_layout != FA8_V_NATURAL) return FA8_ERR_UNSUPPORTED;
  if (seqlen_k <= 0) return FA8_ERR_UNSUPPORTED;
  // Only V^T has the sequence as its contiguous axis: a row of it is seqlen_k bytes long, and
  // the copy engine wants row strides in multiples of 16 bytes.  Rows of Q, K and natural V are
  // head_dim bytes, so their sequence lengths are free.
  if (v_layout == FA8_V_TRANSPOSED && (seqlen_k % 16) != 0) return FA8_ERR_UNSUPPORTED;
  return FA8_OK;
}

// head dim of the kernel that serves `head_dim` (the next of 64, 128, 256)
static int kernel_head_dim(int32_t head_dim) { return head_dim <= 64 ? 64 : (head_dim <= 128 ? 128 : 256); }

int fa8_work_plan(int32_t slices, int32_t seqlen, int32_t seqlen_k, int32_t head_dim, int32_t is_causal,
                  int32_t sm_count, int32_t plan[4]) {
  if (!plan || slices <= 0 || seqlen <= 0 || seqlen_k < 0 || sm_count <= 0) return FA8_ERR_BAD_ARG;
  if (head_dim < 32 || head_dim > 256 || (head_dim % 32) != 0) return FA8_ERR_UNSUPPORTED;
  if (static_cast<int64_t>(slices) * ((static_cast<int64_t>(seqlen) + 127) / 128) > 0x7fffffff) return FA8_ERR_UNSUPPORTED;
  fa8::KernelArgs a{};
  a.n_slices = slices;
  a.seqlen = seqlen;
  a.seqlen_k = seqlen_k > 0 ? seqlen_k : seqlen;
  if (!fa8::plan_fwd(kernel_head_dim(head_dim), is_causal != 0, a, sm_count)) return FA8_ERR_UNSUPPORTED;
  plan[0] = a.rows_per_item;
  plan[1] = a.fold;
  plan[2] = a.n_pairs;
  plan[3] = a.n_units;
  return FA8_OK;
}

int fa8_fwd(const fa8_fwd_params* p, void* cuda_stream) {
  g_detail[0] = '\0';
  if (!p || !p->q || !p->k || !p->v || !p->o) return FA8_ERR_BAD_ARG;
  if (p->batch <= 0 || p->heads <= 0 || p->seqlen <= 0 || p->head_dim <= 0) return FA8_ERR_BAD_ARG;
  if (!(p->softmax_scale > 0.f) || !std::isfinite(p->softmax_scale)) return FA8_ERR_BAD_ARG;
  if (!std::isfinite(p->o_scale)) return FA8_ERR_BAD_ARG;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->o)) return FA8_ERR_BAD_ARG;
  if (p->status_word && (reinterpret_cast<uintptr_t>(p->status_word) & 3u)) return FA8_ERR_BAD_ARG;
  if (p->softmax_lse && (reinterpret_cast<uintptr_t>(p->softmax_lse) & 3u)) return FA8_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(p->descale_q) | reinterpret_cast<uintptr_t>(p->descale_k) |
       reinterpret_cast<uintptr_t>(p->descale_v)) & 3u) return FA8_ERR_BAD_ARG;
  if (p->v_layout != FA8_V_TRANSPOSED && p->v_layout != FA8_V_NATURAL) return FA8_ERR_BAD_ARG;
  if (p->fp8_format != FA8_FP8_E4M3 && p->fp8_format != FA8_FP8_E5M2) return FA8_ERR_BAD_ARG;
  if (p->seqlen_k < 0) return FA8_ERR_BAD_ARG;
  const int32_t seqlen_k = p->seqlen_k > 0 ? p->seqlen_k : p->seqlen;
  int sup = fa8_supported(seqlen_k, p->head_dim, p->v_layout);
  if (sup != FA8_OK) return sup;
  const int64_t bh = static_cast<int64_t>(p->batch) * p->heads;
  const int32_t heads_kv = p->heads_kv > 0 ? p->heads_kv : p->heads;
  if (heads_kv > p->heads || p->heads % heads_kv != 0) return FA8_ERR_BAD_ARG;
  const int64_t bh_kv = static_cast<int64_t>(p->batch) * heads_kv;

  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // A launch that went wrong earlier on this device is reported now, before anything new is
  // enqueued (the reference's only error path is exit(), include/attention_api.cuh:20-29).
  DeviceState* dstate = device_state();
  if (const int code = collect_earlier_failure(dstate, p->status_word, stream)) {
    char buf[96];
    std::snprintf(buf, sizeof(buf), "device code 0x%x; this call was not enqueued", code);
    set_detail("an earlier launch on this device reported an expired wait", buf);
    return FA8_ERR_DEVICE_TIMEOUT;
  }
  const uint64_t S = static_cast<uint64_t>(p->seqlen), D = static_cast<uint64_t>(p->head_dim);
  const uint64_t Sk = static_cast<uint64_t>(seqlen_k);
  // The kernel is built for head dims 64, 128 and 256 (the reference's switch has eight
  // buckets, csrc/static_switch.h:50-77).  The others run on the next one up: the tensor maps
  // keep the true extent and the copy engine fills the box's missing columns (rows, for V^T)
  // with zeros, which add nothing to either product.  Rows longer than 128 bytes are copied as
  // column blocks of 128 bytes.
  const uint32_t d_box = static_cast<uint32_t>(kernel_head_dim(p->head_dim));
  const uint32_t d_blk = d_box < 128u ? d_box : 128u;
  const CUtensorMapSwizzle sw_qk = (d_box >= 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  // The four tensor maps depend on the addresses, the extents and the layout only.  A caller
  // that comes back with the same buffers (a decode loop, a benchmark, a layer called once per
  // step on a static memory plan) gets the maps of its previous call on this thread instead of
  // four more driver calls.
  struct MapKey {
    const void *q, *k, *v, *o;
    uint64_t S, Sk, D;
    int64_t bh, bh_kv;
    int32_t v_layout;
    bool operator==(const MapKey& r) const {
      return q == r.q && k == r.k && v == r.v && o == r.o && S == r.S && Sk == r.Sk && D == r.D && bh == r.bh &&
             bh_kv == r.bh_kv && v_layout == r.v_layout;
    }
  };
  struct MapSet {
    MapKey key;
    bool valid;
    CUtensorMap tq, tk, tv, to;
  };
  thread_local MapSet last{};
  const MapKey key{p->q, p->k, p->v, p->o, S, Sk, D, bh, bh_kv, p->v_layout};
  if (!(last.valid && last.key == key)) {
    last.valid = false;
    if (!make_map_o(&last.to, p->o, D, S, static_cast<uint64_t>(bh),
                    static_cast<uint32_t>(fa8::epi_cols(static_cast<int>(d_box)))))
      return FA8_ERR_CUDA;
    if (!make_map_3d(&last.tq, p->q, D, S, bh, d_blk, 128, sw_qk)) return FA8_ERR_CUDA;
    if (!make_map_3d(&last.tk, p->k, D, Sk, bh_kv, d_blk, 128, sw_qk)) return FA8_ERR_CUDA;
    if (p->v_layout == FA8_V_NATURAL) {
      // V: [bh, S, D] like K; a tile is 128 key rows of D bytes.
      if (!make_map_3d(&last.tv, p->v, D, Sk, bh_kv, d_blk, 128, sw_qk)) return FA8_ERR_CUDA;
    } else {
      // V^T: [bh, D, S]; a tile is D rows of 128 consecutive key positions.
      if (!make_map_3d(&last.tv, p->v, Sk, D, bh_kv, 128, d_box, CU_TENSOR_MAP_SWIZZLE_128B)) return FA8_ERR_CUDA;
    }
    last.key = key;
    last.valid = true;
  }
  const CUtensorMap &tq = last.tq, &tk = last.tk, &tv = last.tv, &to = last.to;

  fa8::KernelArgs args;
  args.o = static_cast<__half*>(p->o);
  args.seqlen = p->seqlen;
  args.seqlen_k = seqlen_k;
  args.head_dim = p->head_dim;
  args.scale_log2 = p->softmax_scale * 1.4426950408889634f;
  args.o_scale = p->o_scale;
  args.status = p->status_word ? p->status_word : (dstate ? dstate->dev_word : nullptr);
  args.host_status = dstate ? dstate->host_flag_dev : nullptr;
  args.lse = p->softmax_lse;
  args.descale_q = p->descale_q;
  args.descale_k = p->descale_k;
  args.descale_v = p->descale_v;
  args.descale_per_head = p->descale_per_head != 0;
  args.heads = p->heads;
  args.heads_kv = heads_kv;
  args.softmax_scale = p->softmax_scale;
  args.timeout_ns = 2000000000ull;
  // one work item per 128 query rows is the finest plan the launcher can choose
  if (bh * ((static_cast<int64_t>(p->seqlen) + 127) / 128) > 0x7fffffff) return FA8_ERR_UNSUPPORTED;
  args.n_slices = static_cast<int>(bh);
  cudaError_t e = fa8::launch_fwd(static_cast<int>(d_box), p->is_causal != 0, p->v_layout == FA8_V_NATURAL,
                                  p->fp8_format == FA8_FP8_E5M2, tq, tk, tv, to, args, stream);
  if (e != cudaSuccess) {
    set_detail("kernel launch", cudaGetErrorString(e));
    return FA8_ERR_CUDA;
  }
  return FA8_OK;
}

int fa8_quantize_e4m3(const void* src, int32_t src_dtype, void* dst, int64_t n, float* amax,
                      float* descale, void* cuda_stream) {
  g_detail[0] = '\0';
  if (!src || !dst || !amax || n <= 0) return FA8_ERR_BAD_ARG;
  if (src_dtype != FA8_DTYPE_FP16 && src_dtype != FA8_DTYPE_BF16) return FA8_ERR_BAD_ARG;
  if (!aligned16(src) || !aligned16(dst)) return FA8_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(amax) & 3u) || (reinterpret_cast<uintptr_t>(descale) & 3u)) return FA8_ERR_BAD_ARG;
  cudaError_t e = fa8::launch_quantize(src, src_dtype == FA8_DTYPE_BF16, dst, n, 1, amax, descale,
                                       static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) {
    set_detail("quantize launch", cudaGetErrorString(e));
    return FA8_ERR_CUDA;
  }
  return FA8_OK;
}

int fa8_quantize_e4m3_segments(const void* src, int32_t src_dtype, void* dst, int64_t seg_len, int32_t n_seg,
                               float* amax, float* descale, void* cuda_stream) {
  g_detail[0] = '\0';
  if (!src || !dst || !amax || seg_len <= 0 || n_seg <= 0 || n_seg > 65535) return FA8_ERR_BAD_ARG;
  if (src_dtype != FA8_DTYPE_FP16 && src_dtype != FA8_DTYPE_BF16) return FA8_ERR_BAD_ARG;
  if (!aligned16(src) || !aligned16(dst) || (seg_len % 8) != 0) return FA8_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(amax) & 3u) || (reinterpret_cast<uintptr_t>(descale) & 3u)) return FA8_ERR_BAD_ARG;
  cudaError_t e = fa8::launch_quantize(src, src_dtype == FA8_DTYPE_BF16, dst, seg_len, n_seg, amax, descale,
                                       static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) {
    set_detail("quantize launch", cudaGetErrorString(e));
    return FA8_ERR_CUDA;
  }
  return FA8_OK;
}

int fa8_quantize_e4m3_segments_noalloc(const void* src, int32_t src_dtype, void* dst, int64_t seg_len,
                                       int32_t n_seg, float* descale, void* cuda_stream) {
  g_detail[0] = '\0';
  if (!src || !dst || !descale || seg_len <= 0 || n_seg <= 0) return FA8_ERR_BAD_ARG;
  if (src_dtype != FA8_DTYPE_FP16 && src_dtype != FA8_DTYPE_BF16) return FA8_ERR_BAD_ARG;
  if (!aligned16(src) || !aligned16(dst) || (n_seg > 1 && (seg_len % 8) != 0)) return FA8_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(descale) & 3u) return FA8_ERR_BAD_ARG;
  if (n_seg > FA8_NOALLOC_MAX_SEGMENTS) {
    char buf[128];
    std::snprintf(buf, sizeof(buf), "%d segments asked for, the built-in scratch holds %d; use "
                  "fa8_quantize_e4m3_segments with a buffer of your own", n_seg, FA8_NOALLOC_MAX_SEGMENTS);
    set_detail("fa8_quantize_e4m3_segments_noalloc", buf);
    return FA8_ERR_UNSUPPORTED;
  }
  cudaError_t e = cudaSuccess;
  float* amax = quant_scratch(&e);
  if (!amax) {
    set_detail("cudaGetSymbolAddress (quantiser scratch)", cudaGetErrorString(e));
    return FA8_ERR_CUDA;
  }
  // launch_quantize clears the n_seg maxima it is about to accumulate (stream-ordered), runs the
  // two passes and allocates nothing.
  e = fa8::launch_quantize(src, src_dtype == FA8_DTYPE_BF16, dst, seg_len, n_seg, amax, descale,
                           static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) {
    set_detail("quantize launch", cudaGetErrorString(e));
    return FA8_ERR_CUDA;
  }
  return FA8_OK;
}

int fa8_selftest_expired_wait(int32_t* status_word, uint32_t limit_us, void* cuda_stream) {
  g_detail[0] = '\0';
  if (reinterpret_cast<uintptr_t>(status_word) & 3u) return FA8_ERR_BAD_ARG;
  if (limit_us == 0 || limit_us > 1000000u) return FA8_ERR_BAD_ARG;     // at most one second
  DeviceState* dstate = device_state();
  if (!status_word && !dstate) return FA8_ERR_BAD_ARG;
  cudaError_t e = fa8::launch_expired_wait(status_word ? status_word : dstate->dev_word,
                                           dstate ? dstate->host_flag_dev : nullptr, 1000ull * limit_us,
                                           static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) {
    set_detail("kernel launch", cudaGetErrorString(e));
    return FA8_ERR_CUDA;
  }
  return FA8_OK;
}

int fa8_check_status(const int32_t* status_word, void* cuda_stream, int32_t* code_out) {
  g_detail[0] = '\0';
  DeviceState* dstate = device_state();
  const int32_t* word = status_word ? status_word : (dstate ? dstate->dev_word : nullptr);
  if (!word) return FA8_ERR_BAD_ARG;
  int32_t host = 0;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e = cudaMemcpyAsync(&host, word, sizeof(host), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    set_detail("status read-back", cudaGetErrorString(e));
    return FA8_ERR_CUDA;
  }
  if (host != 0 && dstate) {
    // Reported here: the next fa8_fwd need not report it again.  The library's own word is
    // cleared as well; a caller's word is the caller's to clear.
    *dstate->host_flag = 0;
    if (!status_word) {
      e = cudaMemsetAsync(dstate->dev_word, 0, sizeof(int), st);
      if (e == cudaSuccess) e = cudaStreamSynchronize(st);
      if (e != cudaSuccess) {
        set_detail("status reset", cudaGetErrorString(e));
        return FA8_ERR_CUDA;
      }
    }
  }
  if (code_out) *code_out = host;
  return host == 0 ? FA8_OK : FA8_ERR_DEVICE_TIMEOUT;
}

}  // extern "C"

// Per-tensor amax quantisation fp16/bf16 -> e4m3: the step before the attention path in
// the reference's own pipeline (test.py:12-23 casts with torch, test.py:68-70), here as two
// HBM-bound kernels so that a caller can go from half-precision Q/K/V to the FP8 operator
// without leaving the stream.
//
//   pass 1  amax = max |x|             reads 2N bytes, one atomicMax per CTA into *amax
//   pass 2  y = e4m3(x * 448 / amax)   reads 2N bytes, writes N bytes; round-to-nearest-even,
//           descale = amax / 448       saturating (cvt.rn.satfinite.e4m3x2.f32)
//
// Both use 16-byte loads, a grid of a few CTAs per SM and grid-stride loops.  amax and descale
// are caller-provided device floats (outputs); nothing else is written.  With n_seg > 1 the
// tensor is n_seg equal, contiguous segments (one per head, say), each with its own amax and
// descale: blockIdx.y picks the segment.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "fa8_kernel.h"
#include "ptx_sm100.cuh"

namespace fa8 {

namespace {

constexpr int kQuantThreads = 256;

template <bool kBf16>
__device__ __forceinline__ float2 unpack_pair(uint32_t w) {
  if (kBf16) {
    // bf16 -> fp32 is a 16-bit shift
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  }
  const __half2 h = *reinterpret_cast<const __half2*>(&w);
  return __half22float2(h);
}

template <bool kBf16>
__global__ void __launch_bounds__(kQuantThreads) amax_kernel(const uint4* __restrict__ x, int64_t n_vec,
                                                            const uint16_t* __restrict__ tail, int n_tail,
                                                            float* __restrict__ amax) {
  x += blockIdx.y * n_vec;
  amax += blockIdx.y;
  float m = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 v = x[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_pair<kBf16>(w[k]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < n_tail) {
    const uint32_t w = tail[threadIdx.x];
    m = fmaxf(m, fabsf(unpack_pair<kBf16>(w).x));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float part[kQuantThreads / 32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = threadIdx.x < kQuantThreads / 32 ? part[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // Non-negative floats order like their bit patterns.  fmaxf drops NaN inputs, so a NaN does
    // not reach amax (it still casts to the fp8 NaN in pass 2); an infinite input makes amax
    // infinite, the scale 448/inf = 0 and every finite output 0 (inf * 0 = NaN for the infinite
    // ones): inputs are expected to be finite.
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(m));
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(kQuantThreads) cast_kernel(const uint4* __restrict__ x, uint2* __restrict__ y,
                                                            int64_t n_vec, const uint16_t* __restrict__ tail_in,
                                                            uint8_t* __restrict__ tail_out, int n_tail,
                                                            const float* __restrict__ amax,
                                                            float* __restrict__ descale) {
  x += blockIdx.y * n_vec;
  y += blockIdx.y * n_vec;
  amax += blockIdx.y;
  if (descale != nullptr) descale += blockIdx.y;
  const float a = *amax;
  const float scale = a > 0.f ? 448.f / a : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0 && descale != nullptr) *descale = a > 0.f ? a / 448.f : 1.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 v = x[i];
    const float2 f0 = unpack_pair<kBf16>(v.x), f1 = unpack_pair<kBf16>(v.y);
    const float2 f2 = unpack_pair<kBf16>(v.z), f3 = unpack_pair<kBf16>(v.w);
    uint2 o;
    o.x = cvt_e4m3x2(f0.x * scale, f0.y * scale) | (cvt_e4m3x2(f1.x * scale, f1.y * scale) << 16);
    o.y = cvt_e4m3x2(f2.x * scale, f2.y * scale) | (cvt_e4m3x2(f3.x * scale, f3.y * scale) << 16);
    y[i] = o;
  }
  if (blockIdx.x == 0 && threadIdx.x < n_tail) {
    const float f = unpack_pair<kBf16>(tail_in[threadIdx.x]).x * scale;
    tail_out[threadIdx.x] = static_cast<uint8_t>(cvt_e4m3x2(f, 0.f) & 0xffu);
  }
}

}  // namespace

cudaError_t launch_quantize(const void* src, bool bf16, void* dst, int64_t n, int n_seg, float* amax,
                            float* descale, cudaStream_t stream) {
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  // n = elements per segment; segments other than a lone one are whole 16-byte vectors
  const int64_t n_vec = n / 8;
  const int n_tail = static_cast<int>(n - n_vec * 8);
  if (n_seg < 1 || n_seg > 65535 || (n_seg > 1 && n_tail != 0)) return cudaErrorInvalidValue;
  const int64_t want = (n_vec + kQuantThreads - 1) / kQuantThreads;
  const int64_t cap = (8ll * sms + n_seg - 1) / n_seg;      // about eight CTAs per SM in all
  const dim3 grid(static_cast<unsigned>(want < 1 ? 1 : (want > cap ? cap : want)), static_cast<unsigned>(n_seg), 1);
  const uint4* x = static_cast<const uint4*>(src);
  const uint16_t* tail_in = static_cast<const uint16_t*>(src) + n_vec * 8;
  uint8_t* tail_out = static_cast<uint8_t*>(dst) + n_vec * 8;
  e = cudaMemsetAsync(amax, 0, sizeof(float) * n_seg, stream);
  if (e != cudaSuccess) return e;
  if (bf16) {
    amax_kernel<true><<<grid, kQuantThreads, 0, stream>>>(x, n_vec, tail_in, n_tail, amax);
    cast_kernel<true><<<grid, kQuantThreads, 0, stream>>>(x, static_cast<uint2*>(dst), n_vec, tail_in, tail_out,
                                                          n_tail, amax, descale);
  } else {
    amax_kernel<false><<<grid, kQuantThreads, 0, stream>>>(x, n_vec, tail_in, n_tail, amax);
    cast_kernel<false><<<grid, kQuantThreads, 0, stream>>>(x, static_cast<uint2*>(dst), n_vec, tail_in, tail_out,
                                                           n_tail, amax, descale);
  }
  return cudaGetLastError();
}

}  // namespace fa8

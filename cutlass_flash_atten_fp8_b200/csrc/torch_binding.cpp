// Compiled torch binding over the C ABI of libfa8_b200.so.
//
// Provides what the reference extension provides: a pybind11 module named
// attention_cutlass_fp8 (setup.py:45, csrc/attention_api.cpp:6-10) whose one function
//   flash_attention_v2_cutlass(q, k, v, is_causal = false, softmax_scale = 1) -> [O]
// takes torch tensors (include/attention_api.h:10-11).  The body stands where the reference
// has csrc/flash_attention.cu:639-668: input checks, output allocation with torch's allocator,
// parameter packing, dispatch - here one call of fa8_fwd on torch's current stream.  Nothing
// in this file touches the GPU except through that call.
//
// Differences from the reference, as everywhere in this library: O is fp16, the call does not
// synchronise the device, and every failure is a C++ exception (RuntimeError in Python) instead
// of exit().  Two keyword arguments are added after the reference's five: v_layout
// ("transposed", the reference's [batch, heads, head_dim, seqlen], or "natural") and o_scale.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <string>
#include <vector>

#include "fa8_b200.h"

namespace {

// CHECK_INPUT of include/attention_api.cuh:12-18
void check_input(const torch::Tensor& x, const char* name) {
  TORCH_CHECK(x.device().is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(x.is_contiguous(), name, " must be contiguous");
}

std::vector<torch::Tensor> flash_attention_v2_cutlass(torch::Tensor q, torch::Tensor k, torch::Tensor v,
                                                      bool is_causal, float softmax_scale,
                                                      const std::string& v_layout, float o_scale) {
  check_input(q, "q");
  check_input(k, "k");
  check_input(v, "v");
  const auto dtype = q.scalar_type();
  TORCH_CHECK(dtype == at::kFloat8_e4m3fn || dtype == at::kFloat8_e5m2,
              "q must be float8_e4m3fn (or float8_e5m2), got ", q.dtype());
  TORCH_CHECK(k.scalar_type() == dtype && v.scalar_type() == dtype, "k and v must have q's dtype");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4,
              "q, k and v must have 4 dimensions [batch, heads, seqlen, head_dim]");
  TORCH_CHECK(k.device() == q.device() && v.device() == q.device(), "q, k and v must be on the same device");
  const int64_t B = q.size(0), H = q.size(1), S = q.size(2), D = q.size(3);
  const int64_t Hk = k.size(1), Sk = k.size(2);
  TORCH_CHECK(k.size(0) == B && k.size(3) == D && Hk >= 1 && H % Hk == 0,
              "k must be [batch, heads_kv, seqlen_k, head_dim] with heads_kv dividing q's heads");
  int32_t layout;
  if (v_layout == "transposed") {
    layout = FA8_V_TRANSPOSED;
    TORCH_CHECK(v.size(0) == B && v.size(1) == Hk && v.size(2) == D && v.size(3) == Sk,
                "v must be [batch, heads_kv, head_dim, seqlen_k] for v_layout='transposed'");
  } else if (v_layout == "natural") {
    layout = FA8_V_NATURAL;
    TORCH_CHECK(v.size(0) == B && v.size(1) == Hk && v.size(2) == Sk && v.size(3) == D,
                "v must be [batch, heads_kv, seqlen_k, head_dim] for v_layout='natural'");
  } else {
    TORCH_CHECK(false, "v_layout must be 'transposed' or 'natural'");
  }
  TORCH_CHECK(B <= INT32_MAX && H <= INT32_MAX && S <= INT32_MAX && Sk <= INT32_MAX && D <= INT32_MAX,
              "tensor extents must fit 32 bits");

  const c10::cuda::CUDAGuard guard(q.device());
  // The reference allocates with torch's allocator as well (csrc/flash_attention.cu:656), in e4m3.
  torch::Tensor out = torch::empty({B, H, S, D}, q.options().dtype(torch::kFloat16));

  fa8_fwd_params p{};
  p.q = q.data_ptr();
  p.k = k.data_ptr();
  p.v = v.data_ptr();
  p.o = out.data_ptr();
  p.batch = static_cast<int32_t>(B);
  p.heads = static_cast<int32_t>(H);
  p.seqlen = static_cast<int32_t>(S);
  p.head_dim = static_cast<int32_t>(D);
  p.softmax_scale = softmax_scale;
  p.is_causal = is_causal ? 1 : 0;
  p.v_layout = layout;
  p.o_scale = o_scale;
  p.status_word = nullptr;   // the library's own word; a failed launch surfaces at the next call
  p.heads_kv = static_cast<int32_t>(Hk);
  p.fp8_format = (dtype == at::kFloat8_e5m2) ? FA8_FP8_E5M2 : FA8_FP8_E4M3;
  p.seqlen_k = static_cast<int32_t>(Sk);
  const int rc = fa8_fwd(&p, c10::cuda::getCurrentCUDAStream(q.device().index()).stream());
  TORCH_CHECK(rc == FA8_OK, "fa8 error ", rc, ": ", fa8_error_string(rc), " [", fa8_last_error_detail(), "]");
  return {out};
}

// Synchronises torch's current stream on `device_index` (-1 = current device) and raises if a
// launch of this library reported an expired wait; stands where the reference has
// cudaDeviceSynchronize + CUDA_ERROR_CHECK (csrc/flash_attention.cu:663-665).
void check_status(int64_t device_index) {
  const c10::DeviceIndex idx =
      device_index < 0 ? c10::cuda::current_device() : static_cast<c10::DeviceIndex>(device_index);
  const c10::cuda::CUDAGuard guard(idx);
  int32_t code = 0;
  const int rc = fa8_check_status(nullptr, c10::cuda::getCurrentCUDAStream(idx).stream(), &code);
  TORCH_CHECK(rc == FA8_OK, "fa8 error ", rc, ": ", fa8_error_string(rc), " (device code ", code, ") [",
              fa8_last_error_detail(), "]");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("flash_attention_v2_cutlass", &flash_attention_v2_cutlass,
        "FP8 flash-attention forward on sm_100a: e4m3 (or e5m2) q, k [batch, heads, seqlen, head_dim] and "
        "v -> [fp16 O]",
        py::arg("q"), py::arg("k"), py::arg("v"), py::arg("is_causal") = false, py::arg("softmax_scale") = 1.0f,
        py::kw_only(), py::arg("v_layout") = "transposed", py::arg("o_scale") = 1.0f);
  m.def("check_status", &check_status, "synchronise the current stream and raise if a launch reported a failure",
        py::arg("device_index") = -1);
  m.def("abi_version", [] { return fa8_version(); }, "version of the C ABI the module was linked against");
}

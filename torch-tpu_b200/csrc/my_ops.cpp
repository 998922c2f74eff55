// torch.ops.my_ops.* - the reference's custom-op surface for the fused-MoE path, same op names and the
// same C++ signatures (hence the same inferred schemas) as torch_tpu/csrc/ops/my_ops/ops.hpp:279-306,
// 610-676, 716-722, registered the way torch_tpu/csrc/ops/my_ops/myOps.cpp:29-80 does.  Each wrapper
// validates its arguments (always, not only in debug builds as CHECK_TENSOR_IN_DEVICE does,
// torch_tpu/csrc/core/TPUTorchUtils.h:70-92), takes the current CUDA stream where the reference takes the
// current TPU stream (my_ops/fusedMoE.cpp:185) and calls the C ABI of libb200moe, checking its status the
// way the reference checks tpudnnStatus_t (my_ops/fusedMoE.cpp:231).  There is no CPU fallback.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <ATen/ATen.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <algorithm>
#include <initializer_list>
#include <map>
#include <sstream>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "../../include/b200moe.h"

namespace at {
namespace {

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == B200MOE_OK, what, " failed: ", b200moe_error_string(rc), " (", rc, ")");
}

void check_cuda_contig(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

// ---- profiling toggles ------------------------------------------------------------------------------
// torch.ops.my_ops.enable_profile(max_record_num, mode) / disable_profile(), as the reference registers them
// (torch_tpu/csrc/ops/my_ops/myOps.cpp:67-68, profile.cpp:12-53: they switch the runtime's per-op profile on the
// current stream).  Here: while enabled, every op of this library opens an NVTX range under its own name and, with
// mode bit 0 (the default), brackets its launches with two CUDA events on the current stream; disable_profile()
// synchronises those events, prints calls / total / average device time per op and keeps the table for
// my_ops.b200_profile_summary().  At most max_record_num calls are timed (later ones only get their NVTX range).
struct OpProfile {
  struct Rec {
    const char* name;
    cudaEvent_t a, b;
  };
  std::mutex mu;
  bool on = false;
  int64_t max_records = 40960, mode = 1;
  std::vector<Rec> recs;
  std::string summary;
};
OpProfile& op_profile() {
  static OpProfile p;
  return p;
}

struct OpScope {
  cudaEvent_t b = nullptr;
  cudaStream_t st = nullptr;
  bool ranged = false;
  explicit OpScope(const char* name) {
    OpProfile& p = op_profile();
    std::lock_guard<std::mutex> lock(p.mu);
    if (!p.on) return;
    nvtxRangePushA(name);
    ranged = true;
    if (!(p.mode & 1) || (int64_t)p.recs.size() >= p.max_records) return;
    cudaEvent_t a = nullptr;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) {
      if (a) cudaEventDestroy(a);
      b = nullptr;
      return;
    }
    st = at::cuda::getCurrentCUDAStream();
    cudaEventRecord(a, st);
    p.recs.push_back({name, a, b});
  }
  ~OpScope() {
    if (b) cudaEventRecord(b, st);
    if (ranged) nvtxRangePop();
  }
};

void enable_profile(c10::optional<int64_t> max_record_num, c10::optional<int64_t> mode) {
  OpProfile& p = op_profile();
  std::lock_guard<std::mutex> lock(p.mu);
  for (auto& r : p.recs) {
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
  }
  p.recs.clear();
  p.max_records = max_record_num.has_value() ? std::max<int64_t>(0, *max_record_num) : 40960;
  p.mode = mode.has_value() ? *mode : 1;
  p.on = true;
}

void disable_profile() {
  OpProfile& p = op_profile();
  std::lock_guard<std::mutex> lock(p.mu);
  p.on = false;
  std::map<std::string, std::pair<int64_t, double>> agg;  // op -> (calls, ms)
  for (auto& r : p.recs) {
    float ms = 0.f;
    if (cudaEventSynchronize(r.b) == cudaSuccess && cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
      auto& e = agg[r.name];
      e.first += 1;
      e.second += ms;
    }
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
  }
  p.recs.clear();
  std::ostringstream os;
  os << "my_ops profile: op, calls, total ms, average us\n";
  for (auto& kv : agg)
    os << "  " << kv.first << ", " << kv.second.first << ", " << kv.second.second << ", "
       << 1000.0 * kv.second.second / (double)kv.second.first << "\n";
  p.summary = os.str();
  std::fputs(p.summary.c_str(), stdout);
}

std::string b200_profile_summary() {
  OpProfile& p = op_profile();
  std::lock_guard<std::mutex> lock(p.mu);
  return p.summary;
}

int scale_dtype_of(const Tensor& s) {
  if (s.scalar_type() == kFloat) return B200MOE_F32;
  if (s.scalar_type() == kBFloat16) return B200MOE_BF16;
  TORCH_CHECK(false, "block scales must be float32 or bfloat16");
}

int score_dtype_of(const Tensor& s) {
  if (s.scalar_type() == kFloat) return B200MOE_F32;
  if (s.scalar_type() == kBFloat16) return B200MOE_BF16;
  if (s.scalar_type() == kHalf) return B200MOE_F16;
  TORCH_CHECK(false, "scores must be float32, bfloat16 or float16");
}

// MOE_ACT_MODE = w8a8 (default: e4m3 activations, FP8 tensor cores) | w8a16 (the reference's arithmetic)
int act_mode_from_env() {
  const char* v = std::getenv("MOE_ACT_MODE");
  if (v && std::strcmp(v, "w8a16") == 0) return B200MOE_ACT_W8A16;
  return B200MOE_ACT_W8A8;
}

// Grow-only workspace per (device, stream).  The reference's callers pass scratch tensors in; ours may pass
// None, so the op layer keeps one buffer from torch's caching allocator.  The C ABI itself never allocates.
Tensor workspace_for(const Device& dev, cudaStream_t st, size_t bytes) {
  static std::mutex mu;
  static std::unordered_map<uint64_t, Tensor> cache;
  std::lock_guard<std::mutex> lock(mu);
  const uint64_t key = (uint64_t)reinterpret_cast<uintptr_t>(st) * 131 + (uint64_t)dev.index();
  auto it = cache.find(key);
  if (it == cache.end() || (size_t)it->second.numel() < bytes) {
    Tensor t = at::empty({(int64_t)(bytes + bytes / 8 + 256)}, TensorOptions().dtype(kByte).device(dev));
    cache[key] = t;
    return t;
  }
  return it->second;
}

// One int32 status word per device (see the status bits in b200moe.h), handed to every experts call.  Expert ids
// outside [0,E) never index anything (the permutation drops them) and raise bit 0 here.  The op stays asynchronous
// by default; with MOE_CHECK_STATUS=1 it synchronises after every call and raises, which is what a debugging session
// wants.  my_ops.b200_moe_status() returns the word's tensor.
Tensor status_word(const Device& dev) {
  static std::mutex mu;
  static std::unordered_map<int, Tensor> words;
  std::lock_guard<std::mutex> lock(mu);
  auto it = words.find(dev.index());
  if (it == words.end()) it = words.emplace(dev.index(), at::zeros({1}, TensorOptions().dtype(kInt).device(dev))).first;
  return it->second;
}

bool check_status_from_env() {
  const char* v = std::getenv("MOE_CHECK_STATUS");
  return v && v[0] == '1';
}

// fp32 copies of bf16 block scales, made once per scale tensor (keyed by storage address, size and version counter)
// instead of on every call: the tensor-core kernels read fp32 scales only.
Tensor scales_as_f32(const Tensor& s) {
  if (s.scalar_type() == kFloat) return s;
  struct Entry {
    int64_t numel;
    uint32_t version;
    Tensor f32;
  };
  static std::mutex mu;
  static std::unordered_map<const void*, Entry> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(s.data_ptr());
  if (it == cache.end() || it->second.numel != s.numel() || it->second.version != s._version()) {
    if (cache.size() > 64) cache.clear();
    it = cache.insert_or_assign(s.data_ptr(), Entry{s.numel(), (uint32_t)s._version(), s.to(kFloat)}).first;
  }
  return it->second.f32;
}

// bf16-weight experts (scales = None in the reference call, python/test/fused_moe_bf16.py:113-122): same pipeline,
// the bf16 tensor-core kernels read the weights as they are
Tensor run_experts_bf16(Tensor& output, const Tensor& input, const Tensor& gate_w, const Tensor& up_w,
                        const Tensor& down_w, const Tensor& select_experts, const Tensor& routing_weights,
                        int64_t num_experts, int64_t top_k) {
  for (const Tensor* t : std::initializer_list<const Tensor*>{&output, &input, &gate_w, &up_w, &down_w, &select_experts,
                                                              &routing_weights})
    check_cuda_contig(*t, "fused_moe_fused_experts argument");
  TORCH_CHECK(select_experts.scalar_type() == kInt, "select_experts must be int32 dtype");
  TORCH_CHECK(input.dim() == 2 && input.scalar_type() == kBFloat16, "input must be bf16 [T,H]");
  TORCH_CHECK(output.scalar_type() == kBFloat16, "output must be bf16");
  TORCH_CHECK(gate_w.scalar_type() == kBFloat16 && up_w.scalar_type() == kBFloat16 && down_w.scalar_type() == kBFloat16,
              "without block scales the expert weights must be bfloat16");
  const int64_t T = input.size(0), H = input.size(1);
  TORCH_CHECK(gate_w.dim() == 3 && gate_w.size(0) == num_experts && gate_w.size(2) == H, "gate_weights must be [E,I,H]");
  TORCH_CHECK(up_w.sizes() == gate_w.sizes() && down_w.sizes() == gate_w.sizes(),
              "up/down weights must be [E,I,H] (down = W_down^T, contiguous)");
  TORCH_CHECK(select_experts.dim() == 2 && select_experts.size(0) == T && select_experts.size(1) == top_k,
              "select_experts must be [T,k]");
  TORCH_CHECK(routing_weights.numel() == T * top_k, "routing_weights must be [T,k]");
  b200moe_experts_desc d{};
  d.T = T, d.H = H, d.I = gate_w.size(1), d.E = num_experts, d.k = top_k;
  if (output.dim() == 3) {
    TORCH_CHECK(output.size(0) == T && output.size(1) == top_k && output.size(2) == H, "output must be [T,k,H]");
    d.out_mode = B200MOE_OUT_PER_SLOT;
  } else {
    TORCH_CHECK(output.dim() == 2 && output.size(0) == T && output.size(1) == H, "output must be [T,k,H] or [T,H]");
    d.out_mode = B200MOE_OUT_COMBINED;
  }
  d.act_mode = B200MOE_ACT_W8A16;
  d.weights_bf16 = 1;
  d.scale_dtype = B200MOE_F32;
  if (routing_weights.scalar_type() == kFloat) d.w_dtype = B200MOE_F32;
  else if (routing_weights.scalar_type() == kBFloat16) d.w_dtype = B200MOE_BF16;
  else TORCH_CHECK(false, "routing_weights must be float32 or bfloat16");
  c10::cuda::CUDAGuard guard(input.device());
  cudaStream_t st = at::cuda::getCurrentCUDAStream();
  const size_t need = b200moe_experts_workspace_bytes(&d);
  TORCH_CHECK(need > 0 || T == 0, "fused_moe_fused_experts: unsupported sizes (H and I must be multiples of 128)");
  Tensor ws = workspace_for(input.device(), st, need);
  void* wsp = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(ws.data_ptr()) + 255) & ~uintptr_t(255));
  const size_t ws_bytes = (size_t)ws.numel() - (reinterpret_cast<char*>(wsp) - reinterpret_cast<char*>(ws.data_ptr()));
  Tensor status = status_word(input.device());
  check_rc(b200moe_experts(output.data_ptr(), input.data_ptr(), gate_w.data_ptr(), up_w.data_ptr(), down_w.data_ptr(),
                           nullptr, nullptr, nullptr, select_experts.data_ptr<int32_t>(), routing_weights.data_ptr(),
                           nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, &d, wsp, ws_bytes,
                           status.data_ptr<int32_t>(), st),
           "b200moe_experts");
  return output;
}

Tensor run_experts(Tensor& output, const Tensor& input, const Tensor& gate_w, const Tensor& up_w,
                   const Tensor& down_w, const Tensor& gate_s, const Tensor& up_s, const Tensor& down_s,
                   const Tensor& select_experts, const Tensor& routing_weights, int64_t blocksize,
                   int64_t num_experts, int64_t top_k, int act_mode) {
  check_cuda_contig(output, "output");
  check_cuda_contig(input, "input");
  check_cuda_contig(gate_w, "gate_weights");
  check_cuda_contig(up_w, "up_weights");
  check_cuda_contig(down_w, "down_weights");
  check_cuda_contig(gate_s, "gate_scales");
  check_cuda_contig(up_s, "up_scales");
  check_cuda_contig(down_s, "down_scales");
  check_cuda_contig(select_experts, "select_experts");
  check_cuda_contig(routing_weights, "routing_weights");
  TORCH_CHECK(select_experts.scalar_type() == kInt, "select_experts must be int32 dtype");
  TORCH_CHECK(blocksize == 128, "blocksize must be 128");
  TORCH_CHECK(input.dim() == 2 && input.scalar_type() == kBFloat16, "input must be bf16 [T,H]");
  TORCH_CHECK(output.scalar_type() == kBFloat16, "output must be bf16");
  TORCH_CHECK(gate_w.scalar_type() == kFloat8_e4m3fn && up_w.scalar_type() == kFloat8_e4m3fn &&
                  down_w.scalar_type() == kFloat8_e4m3fn,
              "expert weights must be float8_e4m3fn");
  const int64_t T = input.size(0), H = input.size(1);
  TORCH_CHECK(gate_w.dim() == 3 && gate_w.size(0) == num_experts && gate_w.size(2) == H,
              "gate_weights must be [E,I,H]");
  const int64_t I = gate_w.size(1);
  TORCH_CHECK(up_w.sizes() == gate_w.sizes() && down_w.sizes() == gate_w.sizes(),
              "up/down weights must be [E,I,H] (down = W_down^T, contiguous)");
  const int64_t nI = (I + 127) / 128, nH = (H + 127) / 128;
  for (const Tensor* s : {&gate_s, &up_s, &down_s})
    TORCH_CHECK(s->dim() == 3 && s->size(0) == num_experts && s->size(1) == nI && s->size(2) == nH,
                "block scales must be [E, I/128, H/128]");
  TORCH_CHECK(gate_s.scalar_type() == up_s.scalar_type() && gate_s.scalar_type() == down_s.scalar_type(),
              "the three scale tensors must share a dtype");
  TORCH_CHECK(select_experts.dim() == 2 && select_experts.size(0) == T && select_experts.size(1) == top_k,
              "select_experts must be [T,k]");
  TORCH_CHECK(routing_weights.numel() == T * top_k, "routing_weights must be [T,k]");

  // the FP8 tensor-core path reads fp32 scales: convert bf16 ones once per tensor, not per call
  const bool to_f32 = act_mode == B200MOE_ACT_W8A8 && gate_s.scalar_type() == kBFloat16;
  const Tensor gs = to_f32 ? scales_as_f32(gate_s) : gate_s, us = to_f32 ? scales_as_f32(up_s) : up_s,
               ds = to_f32 ? scales_as_f32(down_s) : down_s;
  b200moe_experts_desc d{};
  d.T = T;
  d.H = H;
  d.I = I;
  d.E = num_experts;
  d.k = top_k;
  d.I_shared = 0;
  if (output.dim() == 3) {
    TORCH_CHECK(output.size(0) == T && output.size(1) == top_k && output.size(2) == H, "output must be [T,k,H]");
    d.out_mode = B200MOE_OUT_PER_SLOT;
  } else {
    TORCH_CHECK(output.dim() == 2 && output.size(0) == T && output.size(1) == H, "output must be [T,k,H] or [T,H]");
    d.out_mode = B200MOE_OUT_COMBINED;
  }
  d.act_mode = act_mode;
  d.impl = B200MOE_IMPL_AUTO;
  d.scale_dtype = scale_dtype_of(gs);
  if (routing_weights.scalar_type() == kFloat) d.w_dtype = B200MOE_F32;
  else if (routing_weights.scalar_type() == kBFloat16) d.w_dtype = B200MOE_BF16;
  else TORCH_CHECK(false, "routing_weights must be float32 or bfloat16");

  c10::cuda::CUDAGuard guard(input.device());
  cudaStream_t st = at::cuda::getCurrentCUDAStream();
  const size_t need = b200moe_experts_workspace_bytes(&d);
  TORCH_CHECK(need > 0 || T == 0, "fused_moe_fused_experts: unsupported sizes (H and I must be multiples of 128)");
  Tensor ws = workspace_for(input.device(), st, need);
  void* wsp = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(ws.data_ptr()) + 255) & ~uintptr_t(255));
  const size_t ws_bytes = (size_t)ws.numel() - (reinterpret_cast<char*>(wsp) - reinterpret_cast<char*>(ws.data_ptr()));
  Tensor status = status_word(input.device());
  int rc = b200moe_experts(output.data_ptr(), input.data_ptr(), gate_w.data_ptr(), up_w.data_ptr(),
                           down_w.data_ptr(), gs.data_ptr(), us.data_ptr(), ds.data_ptr(),
                           select_experts.data_ptr<int32_t>(), routing_weights.data_ptr(), nullptr, nullptr,
                           nullptr, nullptr, nullptr, nullptr, &d, wsp, ws_bytes, status.data_ptr<int32_t>(), st);
  check_rc(rc, "b200moe_experts");
  if (check_status_from_env()) {
    const int sw = status.item<int>();
    status.zero_();
    TORCH_CHECK((sw & 1) == 0, "fused_moe_fused_experts: select_experts holds ids outside [0, num_experts); "
                               "those (token,slot) pairs were skipped");
    TORCH_CHECK(sw == 0, "fused_moe_fused_experts: device status word ", sw, " (a bounded wait inside a kernel gave up)");
  }
  return output;
}

void reject_unused(const c10::optional<Tensor>& output_sample, const c10::optional<Tensor>& input_sample,
                   const c10::optional<Tensor>& num_select_experts, const c10::optional<Tensor>& silu,
                   const c10::optional<Tensor>& sigmoid, const c10::optional<Tensor>& m0, bool save_mid_res) {
  // None/False in every reference call (python/regression/test_llm/test_moe.py:105-107,129,140)
  TORCH_CHECK(!output_sample.has_value() && !input_sample.has_value(),
              "output_sample / input_sample are not supported (pass None)");
  if (num_select_experts.has_value())
    TORCH_CHECK(num_select_experts.value().scalar_type() == kLong, "num_select_experts must be int64 dtype");
  TORCH_CHECK(!silu.has_value() && !sigmoid.has_value() && !m0.has_value() && !save_mid_res,
              "saving intermediate results (silu/sigmoid/m0/save_mid_res) is not supported");
}

}  // namespace

Tensor fused_moe_fused_experts(
    Tensor& output, Tensor& input, const c10::optional<Tensor>& output_sample,
    const c10::optional<Tensor>& input_sample, Tensor& gate_weights, Tensor& up_weights, Tensor& down_weights,
    const c10::optional<Tensor>& gate_scales, const c10::optional<Tensor>& up_scales,
    const c10::optional<Tensor>& down_scales, Tensor& select_experts, Tensor& routing_weights,
    const c10::optional<Tensor>& num_select_experts, const c10::optional<Tensor>& select_experts_middle,
    const c10::optional<Tensor>& routing_weights_middle, int64_t blocksize, int64_t num_experts,
    int64_t num_experts_per_tok, bool use_grouped_topk, int64_t num_expert_group, int64_t topk_group,
    const c10::optional<Tensor>& silu, const c10::optional<Tensor>& sigmoid, const c10::optional<Tensor>& m0,
    bool save_mid_res) {
  OpScope op_scope("fused_moe_fused_experts");
  reject_unused(output_sample, input_sample, num_select_experts, silu, sigmoid, m0, save_mid_res);
  (void)select_experts_middle;  // caller scratch of the reference kernels; not needed here
  (void)routing_weights_middle;
  (void)use_grouped_topk;       // routing is already done: select_experts is an input
  (void)num_expert_group;
  (void)topk_group;
  if (!gate_scales.has_value() && !up_scales.has_value() && !down_scales.has_value())
    return run_experts_bf16(output, input, gate_weights, up_weights, down_weights, select_experts, routing_weights,
                            num_experts, num_experts_per_tok);
  TORCH_CHECK(gate_scales.has_value() && up_scales.has_value() && down_scales.has_value(),
              "fused_moe_fused_experts: FP8 weights need all three block-scale tensors");
  return run_experts(output, input, gate_weights, up_weights, down_weights, gate_scales.value(), up_scales.value(),
                     down_scales.value(), select_experts, routing_weights, blocksize, num_experts,
                     num_experts_per_tok, act_mode_from_env());
}

Tensor fused_moe_fused_experts_v2(
    Tensor& output, Tensor& input, const c10::optional<Tensor>& output_sample,
    const c10::optional<Tensor>& input_sample, Tensor& gate_weights, Tensor& up_weights, Tensor& down_weights,
    const c10::optional<Tensor>& gate_scales, const c10::optional<Tensor>& up_scales,
    const c10::optional<Tensor>& down_scales, Tensor& select_experts, Tensor& routing_weights,
    const c10::optional<Tensor>& num_select_experts, const c10::optional<Tensor>& select_experts_middle,
    const c10::optional<Tensor>& routing_weights_middle, const c10::optional<Tensor>& gather_buffer,
    const c10::optional<Tensor>& scatter_buffer, int64_t blocksize, int64_t num_experts,
    int64_t num_experts_per_tok, bool use_grouped_topk, int64_t num_expert_group, int64_t topk_group,
    const c10::optional<Tensor>& silu, const c10::optional<Tensor>& sigmoid, const c10::optional<Tensor>& m0,
    bool save_mid_res) {
  OpScope op_scope("fused_moe_fused_experts_v2");
  (void)gather_buffer;
  (void)scatter_buffer;
  return fused_moe_fused_experts(output, input, output_sample, input_sample, gate_weights, up_weights,
                                 down_weights, gate_scales, up_scales, down_scales, select_experts,
                                 routing_weights, num_select_experts, select_experts_middle,
                                 routing_weights_middle, blocksize, num_experts, num_experts_per_tok,
                                 use_grouped_topk, num_expert_group, topk_group, silu, sigmoid, m0, save_mid_res);
}

// Router matmul + softmax + top-k with caller-provided scratch (my_ops/fusedMoE.cpp:82-115).  The reference
// has no test and no CPU twin of this op and its device code is closed, so the mapping of the ten tensors is
// inferred from their names: left [T,H] and right [E,H] fp32 with bf16 copies, matmul_res / softmax_res [T,E]
// fp32, max [T] fp32, topk_weights_res [T,k] fp32 (+ bf16 copy), topk_experts_res [T,k] int32.  Here:
// logits = left_bf16 . right_bf16^T, softmax, top-k, weights renormalised to sum 1.
Tensor fused_moe_grouped_topk(Tensor& topk_experts_res, Tensor& topk_weights_res_bf16, Tensor& left_bf16,
                              Tensor& right_bf16, Tensor& topk_weights_res, Tensor& left, Tensor& right,
                              Tensor& max, Tensor& matmul_res, Tensor& softmax_res) {
  OpScope op_scope("fused_moe_grouped_topk");
  check_cuda_contig(topk_experts_res, "topk_experts_res");
  check_cuda_contig(topk_weights_res_bf16, "topk_weights_res_bf16");
  check_cuda_contig(left_bf16, "left_bf16");
  check_cuda_contig(right_bf16, "right_bf16");
  check_cuda_contig(topk_weights_res, "topk_weights_res");
  check_cuda_contig(matmul_res, "matmul_res");
  TORCH_CHECK(topk_experts_res.scalar_type() == kInt, "topk_experts_res must be int32");
  TORCH_CHECK(left_bf16.scalar_type() == kBFloat16 && right_bf16.scalar_type() == kBFloat16 &&
                  topk_weights_res_bf16.scalar_type() == kBFloat16,
              "*_bf16 tensors must be bfloat16");
  TORCH_CHECK(topk_weights_res.scalar_type() == kFloat && matmul_res.scalar_type() == kFloat,
              "topk_weights_res and matmul_res must be float32");
  TORCH_CHECK(left_bf16.dim() == 2 && right_bf16.dim() == 2 && left_bf16.size(1) == right_bf16.size(1),
              "left_bf16 [T,H], right_bf16 [E,H]");
  const int64_t T = left_bf16.size(0), H = left_bf16.size(1), E = right_bf16.size(0);
  TORCH_CHECK(topk_experts_res.dim() == 2 && topk_experts_res.size(0) == T, "topk_experts_res must be [T,k]");
  const int64_t k = topk_experts_res.size(1);
  TORCH_CHECK(matmul_res.numel() == T * E && topk_weights_res.numel() == T * k &&
                  topk_weights_res_bf16.numel() == T * k,
              "scratch/result shapes do not match [T,E] / [T,k]");
  (void)left;
  (void)right;
  (void)max;
  (void)softmax_res;
  c10::cuda::CUDAGuard guard(left_bf16.device());
  cudaStream_t st = at::cuda::getCurrentCUDAStream();
  check_rc(b200moe_router_logits(matmul_res.data_ptr<float>(), left_bf16.data_ptr(), right_bf16.data_ptr(), T, H, E, st),
           "b200moe_router_logits");
  check_rc(b200moe_route(topk_experts_res.data_ptr<int32_t>(), topk_weights_res.data_ptr<float>(),
                         topk_weights_res_bf16.data_ptr(), matmul_res.data_ptr<float>(), nullptr, nullptr, T, E, k,
                         B200MOE_SCORE_SOFTMAX, 1, 1, 1, 1.0f, st),
           "b200moe_route");
  return topk_experts_res;
}

// my_ops/NoauxTcTopk.cpp:9-67 - same checks, same order of arguments
Tensor noaux_tc_topk(Tensor& values, Tensor& indices, const Tensor& scores, int64_t n_groups,
                     int64_t topk_groups, int64_t top_k) {
  OpScope op_scope("noaux_tc_topk");
  check_cuda_contig(values, "values");
  check_cuda_contig(indices, "indices");
  check_cuda_contig(scores, "scores");
  TORCH_CHECK(values.dtype() == scores.dtype(), "values and scores must have the same dtype");
  TORCH_CHECK(indices.dtype() == kInt, "indices must be int32");
  TORCH_CHECK(scores.dim() == 2, "scores must be 2D tensor");
  const int64_t batch_size = scores.size(0), total_size = scores.size(1);
  TORCH_CHECK(values.dim() == 2 && values.size(0) == batch_size && values.size(1) == top_k,
              "values shape must be [batch_size, top_k]");
  TORCH_CHECK(indices.dim() == 2 && indices.size(0) == batch_size && indices.size(1) == top_k,
              "indices shape must be [batch_size, top_k]");
  TORCH_CHECK(n_groups > 0 && total_size % n_groups == 0, "total_size must be divisible by n_groups");
  TORCH_CHECK(topk_groups <= n_groups, "topk_groups must be <= n_groups");
  TORCH_CHECK(top_k > 0, "top_k must be positive");
  c10::cuda::CUDAGuard guard(scores.device());
  cudaStream_t st = at::cuda::getCurrentCUDAStream();
  check_rc(b200moe_noaux_tc_topk(values.data_ptr(), indices.data_ptr<int32_t>(), scores.data_ptr(),
                                 score_dtype_of(scores), batch_size, total_size, n_groups, topk_groups, top_k, st),
           "b200moe_noaux_tc_topk");
  return values;
}

namespace {
// Dense FP8 gated MLP = one expert applied to every row (the shared-expert op).  Weights [I,H] x3 with the
// down projection passed transposed (python/regression/test_llm/test_mlp_w8a16_dq.py:102-105).
Tensor dense_mlp(Tensor& input, Tensor& gate_weight, Tensor& up_weight, Tensor& down_weight, Tensor& gate_scale,
                 Tensor& up_scale, Tensor& down_scale, Tensor& output, int64_t blocksize, int act_mode) {
  TORCH_CHECK(input.dim() == 2 && gate_weight.dim() == 2, "input [T,H], weights [I,H]");
  TORCH_CHECK(output.dim() == 2 && output.sizes() == input.sizes(), "output must be [T,H]");
  const int64_t T = input.size(0);
  // expert id 0 and weight 1 for every row: grow-only constants per device, so that the op allocates nothing per call
  static std::mutex mu;
  static std::unordered_map<int, std::pair<Tensor, Tensor>> consts;
  Tensor ids, w;
  {
    std::lock_guard<std::mutex> lock(mu);
    auto& c = consts[input.device().index()];
    if (!c.first.defined() || c.first.size(0) < T) {
      const int64_t cap = std::max<int64_t>(T, 1024);
      c.first = at::zeros({cap, 1}, input.options().dtype(kInt));
      c.second = at::ones({cap, 1}, input.options().dtype(kFloat));
    }
    ids = c.first.narrow(0, 0, T);
    w = c.second.narrow(0, 0, T);
  }
  Tensor out3 = output.view({T, 1, input.size(1)});
  Tensor gw = gate_weight.unsqueeze(0), uw = up_weight.unsqueeze(0), dw = down_weight.unsqueeze(0);
  Tensor gs = gate_scale.unsqueeze(0), us = up_scale.unsqueeze(0), ds = down_scale.unsqueeze(0);
  run_experts(out3, input, gw, uw, dw, gs, us, ds, ids, w, blocksize, 1, 1, act_mode);
  return output;
}
}  // namespace

// my_ops/MlpW8A16Dq.cpp:189-243 (reference arithmetic: bf16 activations)
Tensor mlp_w8a16_dq_forward(Tensor& input, Tensor& gate_weight, Tensor& up_weight, Tensor& down_weight,
                            Tensor& gate_scale, Tensor& up_scale, Tensor& down_scale, Tensor& output,
                            int64_t blocksize) {
  OpScope op_scope("mlp_w8a16_dq_forward");
  return dense_mlp(input, gate_weight, up_weight, down_weight, gate_scale, up_scale, down_scale, output, blocksize,
                   B200MOE_ACT_W8A16);
}

// my_ops/MlpW8A8Quant.cpp:12-50 (activations quantised: FP8 tensor cores)
Tensor mlp_w8a8_quant_forward(Tensor& input, Tensor& gate_weight, Tensor& up_weight, Tensor& down_weight,
                              Tensor& gate_scale, Tensor& up_scale, Tensor& down_scale, Tensor& output,
                              int64_t blocksize) {
  OpScope op_scope("mlp_w8a8_quant_forward");
  return dense_mlp(input, gate_weight, up_weight, down_weight, gate_scale, up_scale, down_scale, output, blocksize,
                   B200MOE_ACT_W8A8);
}

// my_ops/MmW8A16Dq.cpp:185-229: output[M,N] = input[M,K] . dequant(weight [N,K], scale)^T.  Runs on the FP8 tensor
// cores (activations quantised per row per 128 columns), like the expert GEMMs.
Tensor mm_w8a16_dq_forward(Tensor& input, Tensor& weight, Tensor& scale, Tensor& output, int64_t blocksize) {
  OpScope op_scope("mm_w8a16_dq_forward");
  check_cuda_contig(input, "input");
  check_cuda_contig(weight, "weight");
  check_cuda_contig(scale, "scale");
  check_cuda_contig(output, "output");
  TORCH_CHECK(blocksize == 128, "blocksize must be 128");
  TORCH_CHECK(input.dim() == 2 && input.scalar_type() == kBFloat16, "input must be bf16 [M,K]");
  TORCH_CHECK(weight.dim() == 2 && weight.scalar_type() == kFloat8_e4m3fn && weight.size(1) == input.size(1),
              "weight must be float8_e4m3fn [N,K]");
  const int64_t M = input.size(0), K = input.size(1), N = weight.size(0);
  TORCH_CHECK(output.scalar_type() == kBFloat16 && output.dim() == 2 && output.size(0) == M && output.size(1) == N,
              "output must be bf16 [M,N]");
  TORCH_CHECK(scale.dim() == 2 && scale.size(0) == (N + 127) / 128 && scale.size(1) == (K + 127) / 128,
              "scale must be [ceil(N/128), ceil(K/128)]");
  c10::cuda::CUDAGuard guard(input.device());
  cudaStream_t st = at::cuda::getCurrentCUDAStream();
  const int sdt = scale_dtype_of(scale);
  const size_t need = b200moe_linear_workspace_bytes(M, K, N, sdt);
  TORCH_CHECK(need > 0 || M == 0, "mm_w8a16_dq_forward: unsupported sizes (K % 128 == 0 and N % 64 == 0 required)");
  Tensor ws = workspace_for(input.device(), st, need);
  void* wsp = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(ws.data_ptr()) + 255) & ~uintptr_t(255));
  const size_t ws_bytes = (size_t)ws.numel() - (reinterpret_cast<char*>(wsp) - reinterpret_cast<char*>(ws.data_ptr()));
  check_rc(b200moe_linear_w8(output.data_ptr(), input.data_ptr(), weight.data_ptr(), scale.data_ptr(), sdt, M, K, N,
                             wsp, ws_bytes, nullptr, st),
           "b200moe_linear_w8");
  return output;
}

// aten::_scaled_mm as the reference implements it on its device (native_ops/Scaled_mm.cpp:55-88 -> tpudnnMatmulFp8Async):
// self [M,K] and mat2 [N,K] float8_e4m3fn (the reference's caller passes the transposed, contiguous second operand,
// python/test/_scaled_mm.py:8), one fp32 scale per operand, result [M,N] in out_dtype (bf16 or fp32; default bf16).
// Registered under my_ops because on CUDA aten::_scaled_mm already belongs to PyTorch; argument order as in the
// reference's wrapper.  bias and scale_result are not supported (None in the reference's test).
Tensor scaled_mm_fp8(const Tensor& self, const Tensor& mat2, const Tensor& scale_a, const Tensor& scale_b,
                     const c10::optional<Tensor>& bias, const c10::optional<Tensor>& scale_result,
                     c10::optional<ScalarType> out_dtype, bool use_fast_accum) {
  OpScope op_scope("_scaled_mm");
  (void)use_fast_accum;
  check_cuda_contig(self, "self");
  check_cuda_contig(mat2, "mat2");
  TORCH_CHECK(self.dim() == 2, "self must be a matrix");
  TORCH_CHECK(mat2.dim() == 2, "mat2 must be a matrix");
  TORCH_CHECK(self.scalar_type() == kFloat8_e4m3fn && mat2.scalar_type() == kFloat8_e4m3fn,
              "self and mat2 must be float8_e4m3fn");
  TORCH_CHECK(self.size(1) == mat2.size(1), "self [M,K] and mat2 [N,K] must share K");
  TORCH_CHECK(!bias.has_value() && !scale_result.has_value(), "bias / scale_result are not supported (pass None)");
  TORCH_CHECK(scale_a.numel() == 1 && scale_b.numel() == 1, "scale_a and scale_b must hold one value each");
  const ScalarType odt = out_dtype.value_or(kBFloat16);
  TORCH_CHECK(odt == kBFloat16 || odt == kFloat, "out_dtype must be bfloat16 or float32");
  const int64_t M = self.size(0), K = self.size(1), N = mat2.size(0);
  c10::cuda::CUDAGuard guard(self.device());
  cudaStream_t st = at::cuda::getCurrentCUDAStream();
  Tensor sa = scale_a.to(self.device(), kFloat).contiguous(), sb = scale_b.to(self.device(), kFloat).contiguous();
  Tensor out = at::empty({M, N}, self.options().dtype(odt));   // the reference allocates its result too (:118)
  const size_t need = b200moe_scaled_mm_workspace_bytes(M, K, N);
  TORCH_CHECK(need > 0 || M == 0, "_scaled_mm: unsupported sizes (K % 128 == 0 and N % 64 == 0 required)");
  Tensor ws = workspace_for(self.device(), st, need);
  void* wsp = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(ws.data_ptr()) + 255) & ~uintptr_t(255));
  const size_t ws_bytes = (size_t)ws.numel() - (reinterpret_cast<char*>(wsp) - reinterpret_cast<char*>(ws.data_ptr()));
  check_rc(b200moe_scaled_mm(out.data_ptr(), odt == kFloat ? B200MOE_F32 : B200MOE_BF16, self.data_ptr(),
                             mat2.data_ptr(), sa.data_ptr<float>(), sb.data_ptr<float>(), M, K, N, wsp, ws_bytes,
                             nullptr, st),
           "b200moe_scaled_mm");
  return out;
}

// The device status word of the current device (int32 [1]; bits in include/b200moe.h).  Not part of the reference's
// surface: the reference reports device errors through its runtime, this library through that word.
Tensor b200_moe_status() {
  return status_word(Device(kCUDA, (c10::DeviceIndex)at::cuda::current_device()));
}

TORCH_LIBRARY(my_ops, m) {
  m.def("b200_moe_status", b200_moe_status);
  m.def("enable_profile", enable_profile);
  m.def("disable_profile", disable_profile);
  m.def("b200_profile_summary", b200_profile_summary);
  m.def("_scaled_mm", scaled_mm_fp8);
  m.def("fused_moe_grouped_topk", fused_moe_grouped_topk);
  m.def("fused_moe_fused_experts", fused_moe_fused_experts);
  m.def("fused_moe_fused_experts_v2", fused_moe_fused_experts_v2);
  m.def("noaux_tc_topk", noaux_tc_topk);
  m.def("mlp_w8a16_dq_forward", mlp_w8a16_dq_forward);
  m.def("mlp_w8a8_quant_forward", mlp_w8a8_quant_forward);
  m.def("mm_w8a16_dq_forward", mm_w8a16_dq_forward);
}

}  // namespace at

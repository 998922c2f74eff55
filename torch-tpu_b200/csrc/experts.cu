// The expert pipeline behind b200moe_experts: permute -> (quantise) -> grouped gate/up GEMM with SiLU*up
// -> grouped down GEMM -> scatter or weighted combine, all enqueued on one stream into a caller-owned
// workspace.  Stands in for tpudnnFusedMoEFusedExpertsMultiCoreAsync
// (third_party/tpuDNN/include/tpuDNNTensor.h:1585-1611) and the PPL kernel my_ops/fusedMoE.pl:795-810.
#include "internal.h"

namespace {

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

constexpr int64_t kSplitMaxPairs = 512;  // the down GEMM splits K over CTAs only for batches this small

// K splits of the down GEMM.  With few (token,slot) pairs there are fewer output tiles than SMs and every tile has a
// long K loop (K = I), so the weight stream would be pulled by a handful of SMs, or by one and a half waves of work
// items.  The critical path of a persistent launch is (waves of work items) x (K blocks per item), plus what the
// partial sums cost: every split adds one fp32 reduction per output value, and reductions that meet at one address
// are slow (measured: at 1024 pairs a 3-way split lost more than it won, so larger batches are never split - which
// also keeps every prefill-size result bit-reproducible).  Pick the split that makes the sum shortest.  The number
// of m-tiles is a device-side value; the host estimates it from the sizes.
int choose_ksplit(int64_t P, int64_t E, int64_t H, int64_t I) {
  if (P > kSplitMaxPairs) return 1;
  const int64_t experts = P < E ? P : E;                    // activated experts, at most
  const int64_t mtiles_even = (3 * P / 2 + kTileM - 1) / kTileM;  // uneven loads: some experts spill into a second tile
  const int64_t tiles = (experts > mtiles_even ? experts : mtiles_even) * ((H + 255) / 256);
  const int64_t kb = I / kBlock, sms = moe_device_sm_count();
  int best = 1;
  int64_t best_cost = ((tiles + sms - 1) / sms) * kb;
  for (int ks = 2; ks <= 16 && ks * 2 <= kb; ++ks) {
    const int64_t cost = ((tiles * ks + sms - 1) / sms) * ((kb + ks - 1) / ks) + P * (H / 4) * ks / 30000;
    if (cost * 100 < best_cost * 97) best = ks, best_cost = cost;  // a split must buy at least 3 %
  }
  return best;
}

struct WsLayout {
  size_t offsets, sorted, scratch, mtiles, nmt, xq, xs, hq, hs, y, sc32, s_sc32, y32, s_y32, acc32;
  size_t s_offsets, s_mtiles, s_nmt, s_xq, s_xs, s_hq, s_hs, s_y;
  size_t total;
  int64_t P, ld, lds;
  int max_mtiles, s_max_mtiles;
};

WsLayout make_layout(const b200moe_experts_desc& d) {
  WsLayout L{};
  size_t o = 0;
  auto take = [&](size_t bytes) {
    size_t at = o;
    o = align_up(o + bytes, 256);
    return at;
  };
  const int64_t P = d.T * d.k;
  L.P = P;
  L.ld = (int64_t)align_up((size_t)P, kTileM);
  L.lds = (int64_t)align_up((size_t)d.T, kTileM);
  L.max_mtiles = (int)(P / kTileM + d.E);
  L.s_max_mtiles = (int)((d.T + kTileM - 1) / kTileM);
  const bool w8a8 = d.act_mode == B200MOE_ACT_W8A8;
  const size_t nH = d.H / kBlock, nI = d.I / kBlock;
  L.offsets = take((d.E + 1) * sizeof(int32_t));
  L.sorted = take((size_t)P * sizeof(int32_t));
  L.scratch = take(b200moe_permute_scratch_ints(P, d.E) * sizeof(int32_t));
  L.mtiles = take((size_t)L.max_mtiles * 2 * sizeof(int32_t));
  L.nmt = take(sizeof(int32_t));
  L.xq = take(w8a8 ? (size_t)P * d.H : (size_t)P * d.H * 2);  // W8A16: the bf16 rows of x gathered into sorted order
  L.xs = take(w8a8 ? nH * (size_t)L.ld * sizeof(float) : 0);
  L.hq = take(w8a8 ? (size_t)P * d.I : (size_t)P * d.I * 2);
  L.hs = take(w8a8 ? nI * (size_t)L.ld * sizeof(float) : 0);
  // combined output: per-slot rows for the separate combine kernel; the fused combine adds into an fp32 [T,H] buffer
  // instead (both are laid out, so that one workspace serves either mode of the same sizes)
  L.y = take(d.out_mode != B200MOE_OUT_PER_SLOT ? (size_t)P * d.H * 2 : 0);
  // (also used by B200MOE_OUT_COMBINED at decode sizes: the K-split partial sums of the down GEMM are reductions
  // anyway, so they go straight into the combined rows instead of through per-slot rows and the combine kernel)
  // (in that case for min(T, limit) tokens whatever T is, so that the workspace size never shrinks when T grows)
  const int64_t acc_tokens = d.out_mode == B200MOE_OUT_COMBINED_FUSED ? d.T
                             : d.out_mode == B200MOE_OUT_COMBINED     ? (d.T < kSplitMaxPairs ? d.T : kSplitMaxPairs)
                                                                      : 0;
  L.acc32 = take(w8a8 ? (size_t)acc_tokens * d.H * sizeof(float) : 0);
  // fp32 partial sums of the K-split down GEMM (decode-size batches only)
  // (sized for min(P, limit) rows whatever P is, so that the workspace size never shrinks when T grows)
  L.y32 = take(w8a8 ? (size_t)(P < kSplitMaxPairs ? P : kSplitMaxPairs) * d.H * sizeof(float) : 0);
  // fp32 copies of bf16 block scales (the tensor-core kernels read fp32 scales only)
  L.sc32 = take(d.scale_dtype == B200MOE_BF16 && w8a8 ? 3 * (size_t)d.E * nI * nH * sizeof(float) : 0);
  if (d.I_shared > 0) {
    const size_t nIs = d.I_shared / kBlock;
    L.s_offsets = take(2 * sizeof(int32_t));
    L.s_mtiles = take((size_t)L.s_max_mtiles * 2 * sizeof(int32_t));
    L.s_nmt = take(sizeof(int32_t));
    L.s_xq = take(w8a8 ? (size_t)d.T * d.H : 0);
    L.s_xs = take(w8a8 ? nH * (size_t)L.lds * sizeof(float) : 0);
    L.s_hq = take(w8a8 ? (size_t)d.T * d.I_shared : (size_t)d.T * d.I_shared * 2);
    L.s_hs = take(w8a8 ? nIs * (size_t)L.lds * sizeof(float) : 0);
    L.s_y = take((size_t)d.T * d.H * 2);
    L.s_y32 = take(w8a8 ? (size_t)(d.T < kSplitMaxPairs ? d.T : kSplitMaxPairs) * d.H * sizeof(float) : 0);
    L.s_sc32 = take(d.scale_dtype == B200MOE_BF16 && w8a8 ? 3 * nIs * nH * sizeof(float) : 0);
  }
  L.total = o;
  return L;
}

__global__ void scales_to_f32_kernel(float* __restrict__ dst, const __nv_bfloat16* __restrict__ a,
                                     const __nv_bfloat16* __restrict__ b, const __nv_bfloat16* __restrict__ c, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    dst[i] = __bfloat162float(a[i]);
    dst[n + i] = __bfloat162float(b[i]);
    dst[2 * n + i] = __bfloat162float(c[i]);
  }
}

// Side stream on which the shared expert of a decode-size batch runs next to the routed experts (neither pass fills
// the GPU on its own there).  Created once per device on first use; the fork/join is by events, so it can be captured
// into a CUDA graph together with the caller's stream.
struct SideStream {
  cudaStream_t s = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};
SideStream* side_stream() {
  constexpr int kMaxDevices = 64;
  static SideStream tab[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  SideStream& t = tab[dev];
  if (!t.s) {
    if (cudaStreamCreateWithFlags(&t.s, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&t.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&t.join, cudaEventDisableTiming) != cudaSuccess)
      return nullptr;
  }
  return &t;
}
constexpr int64_t kSharedOverlapMaxTokens = 64;

int check_desc(const b200moe_experts_desc* d) {
  MOE_CHECK_ARG(d);
  MOE_CHECK_ARG(d->T >= 0 && d->H > 0 && d->I > 0 && d->E > 0 && d->k > 0 && d->I_shared >= 0);
  MOE_CHECK_ARG(d->out_mode == B200MOE_OUT_PER_SLOT || d->out_mode == B200MOE_OUT_COMBINED ||
                d->out_mode == B200MOE_OUT_COMBINED_FUSED);
  MOE_CHECK_ARG(d->impl_gate_up >= B200MOE_IMPL_AUTO && d->impl_gate_up <= B200MOE_IMPL_TCGEN05);
  MOE_CHECK_ARG(d->impl_down >= B200MOE_IMPL_AUTO && d->impl_down <= B200MOE_IMPL_TCGEN05);
  MOE_CHECK_ARG((d->stages & ~B200MOE_STAGE_ALL) == 0);
  MOE_CHECK_ARG(d->max_ctas >= 0);
  MOE_CHECK_ARG(d->weights_bf16 == 0 || d->weights_bf16 == 1);
  if (d->weights_bf16)
    MOE_CHECK_ARG(d->act_mode == B200MOE_ACT_W8A16 && d->impl != B200MOE_IMPL_SIMPLE &&
                  d->impl_gate_up != B200MOE_IMPL_SIMPLE && d->impl_down != B200MOE_IMPL_SIMPLE);
  MOE_CHECK_ARG(d->act_mode == B200MOE_ACT_W8A8 || d->act_mode == B200MOE_ACT_W8A16);
  MOE_CHECK_ARG(d->impl >= B200MOE_IMPL_AUTO && d->impl <= B200MOE_IMPL_TCGEN05);
  MOE_CHECK_ARG(d->scale_dtype == B200MOE_F32 || d->scale_dtype == B200MOE_BF16);
  MOE_CHECK_ARG(d->w_dtype == B200MOE_F32 || d->w_dtype == B200MOE_BF16);
  MOE_CHECK_SHAPE(d->H % kBlock == 0 && d->I % kBlock == 0 && d->I_shared % kBlock == 0);
  MOE_CHECK_SHAPE(d->E <= 1024 && d->T * d->k < (1 << 24));
  MOE_CHECK_SHAPE(d->H < (1 << 24) && d->I < (1 << 24) && d->E * d->I < (int64_t(1) << 31));
  if (d->I_shared > 0) MOE_CHECK_ARG(d->out_mode != B200MOE_OUT_PER_SLOT);
  return B200MOE_OK;
}

}  // namespace

extern "C" size_t b200moe_experts_workspace_bytes(const b200moe_experts_desc* d) {
  if (check_desc(d) != B200MOE_OK) return 0;
  return make_layout(*d).total;
}

extern "C" int b200moe_experts(void* out, const void* x, const void* w_gate, const void* w_up,
                               const void* w_down, const void* s_gate, const void* s_up, const void* s_down,
                               const int32_t* ids, const void* topk_w, const void* shared_w_gate,
                               const void* shared_w_up, const void* shared_w_down,
                               const void* shared_s_gate, const void* shared_s_up,
                               const void* shared_s_down, const b200moe_experts_desc* d, void* workspace,
                               size_t workspace_bytes, int32_t* status, void* stream) {
  int rc = check_desc(d);
  if (rc != B200MOE_OK) return rc;
  if (d->T == 0) return B200MOE_OK;  // nothing to do; empty tensors may carry null pointers
  MOE_CHECK_ARG(out && x && w_gate && w_up && w_down && ids);
  if (!d->weights_bf16) MOE_CHECK_ARG(s_gate && s_up && s_down);
  if (d->out_mode != B200MOE_OUT_PER_SLOT) MOE_CHECK_ARG(topk_w);
  if (d->I_shared > 0)
    MOE_CHECK_ARG(shared_w_gate && shared_w_up && shared_w_down &&
                  (d->weights_bf16 || (shared_s_gate && shared_s_up && shared_s_down)));
  if (!moe_aligned16(out) || !moe_aligned16(x) || !moe_aligned16(w_gate) || !moe_aligned16(w_up) ||
      !moe_aligned16(w_down))
    return B200MOE_EALIGN;
  const WsLayout L = make_layout(*d);
  if (!workspace || workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return B200MOE_EWORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = reinterpret_cast<char*>(workspace);
  auto I32 = [&](size_t off) { return reinterpret_cast<int32_t*>(ws + off); };
  const bool w8a8 = d->act_mode == B200MOE_ACT_W8A8;
  const bool use_tc = w8a8 && d->impl != B200MOE_IMPL_SIMPLE && moe_tc_available();
  // W8A16 (the reference's arithmetic) has its own tensor-core kernels: bf16 x bf16 with the weights dequantised in
  // shared memory
  const bool use_tc16 = !w8a8 && d->impl != B200MOE_IMPL_SIMPLE && moe_tc_available();
  if (d->impl == B200MOE_IMPL_TCGEN05 && !use_tc && !use_tc16) return B200MOE_EDRIVER;
  if (d->weights_bf16 && !use_tc16) return B200MOE_EDRIVER;  // bf16 weights exist on the tensor-core path only
  const bool combined = d->out_mode != B200MOE_OUT_PER_SLOT;
  // per-GEMM kernel family (A/B tests), else the call's
  const bool tc1 = w8a8 && moe_tc_available() && (d->impl_gate_up ? d->impl_gate_up == B200MOE_IMPL_TCGEN05 : use_tc);
  const bool tc2 = w8a8 && moe_tc_available() && (d->impl_down ? d->impl_down == B200MOE_IMPL_TCGEN05 : use_tc);
  const bool tc1_16 = !w8a8 && moe_tc_available() && (d->impl_gate_up ? d->impl_gate_up == B200MOE_IMPL_TCGEN05 : use_tc16);
  const bool tc2_16 = !w8a8 && moe_tc_available() && (d->impl_down ? d->impl_down == B200MOE_IMPL_TCGEN05 : use_tc16);
  // the fused combine lives in the tensor-core down GEMM's epilogue; other paths combine with the separate kernel
  const int ksplit = tc2 ? choose_ksplit(L.P, d->E, d->H, d->I) : 1;
  const bool fused = tc2 && (d->out_mode == B200MOE_OUT_COMBINED_FUSED || (d->out_mode == B200MOE_OUT_COMBINED && ksplit > 1));
  // a stage may be re-run alone on a workspace that a whole call of the same sizes has filled
  const int stages = d->stages ? d->stages : B200MOE_STAGE_ALL;
  const bool do_prep = stages & B200MOE_STAGE_PREP, do_g1 = stages & B200MOE_STAGE_GATE_UP,
             do_g2 = stages & B200MOE_STAGE_DOWN, do_comb = stages & B200MOE_STAGE_COMBINE;

  // Decode-size batches with a shared expert: the shared expert runs on a side stream beside the routed experts.
  // The fork is recorded before any routed work is queued, so both passes start together; they share no workspace
  // region.  One call per device at a time may use the side stream (calls on one device are expected to be queued
  // from one host thread).
  // fused combine: the sums of the routed AND the shared expert meet in this buffer, so it is cleared before the
  // side stream forks off
  float* acc32 = reinterpret_cast<float*>(ws + L.acc32);
  if (fused && do_g2) cudaMemsetAsync(acc32, 0, (size_t)d->T * d->H * sizeof(float), st);
  SideStream* side = (d->I_shared > 0 && use_tc && d->T <= kSharedOverlapMaxTokens && stages == B200MOE_STAGE_ALL)
                         ? side_stream() : nullptr;
  if (side) {
    if (cudaEventRecord(side->fork, st) != cudaSuccess || cudaStreamWaitEvent(side->s, side->fork, 0) != cudaSuccess)
      return (int)cudaGetLastError();
  }

  if (do_prep) {
    bool tiles_done = false;
    rc = moe_permute_impl(I32(L.sorted), I32(L.offsets), ids, d->T, d->k, d->E, I32(L.scratch), status, I32(L.mtiles),
                          I32(L.nmt), L.max_mtiles, &tiles_done, stream);
    if (rc) return rc;
    if (!tiles_done) {
      rc = moe_build_mtiles(I32(L.mtiles), I32(L.nmt), I32(L.offsets), (int)d->E, L.P, L.max_mtiles, st);
      if (rc) return rc;
    }
  }
  if (w8a8 && do_prep) {
    rc = b200moe_quant_rows(reinterpret_cast<uint8_t*>(ws + L.xq), reinterpret_cast<float*>(ws + L.xs), L.ld,
                            x, I32(L.sorted), d->k, L.P, d->H, stream);
    if (rc) return rc;
  }

  const bool cvt = d->scale_dtype == B200MOE_BF16 && (tc1 || tc2);
  const int64_t nsc = d->E * (d->I / kBlock) * (d->H / kBlock);
  if (cvt && do_prep) {
    scales_to_f32_kernel<<<(unsigned)((nsc + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<float*>(ws + L.sc32), reinterpret_cast<const __nv_bfloat16*>(s_gate),
        reinterpret_cast<const __nv_bfloat16*>(s_up), reinterpret_cast<const __nv_bfloat16*>(s_down), nsc);
    rc = moe_launch_status();
    if (rc) return rc;
  }
  const float* sc32 = reinterpret_cast<const float*>(ws + L.sc32);

  MoeGemmArgs g{};
  g.aq = reinterpret_cast<const uint8_t*>(ws + L.xq);
  g.as_t = reinterpret_cast<const float*>(ws + L.xs);
  g.ld = L.ld;
  g.a16 = reinterpret_cast<const __nv_bfloat16*>(x);
  g.row_map = I32(L.sorted);
  g.div = (int)d->k;
  g.w0 = reinterpret_cast<const uint8_t*>(w_gate);
  g.w1 = reinterpret_cast<const uint8_t*>(w_up);
  g.s0 = s_gate;
  g.s1 = s_up;
  g.scale_dtype = d->scale_dtype;
  g.w_bf16 = d->weights_bf16;
  g.mtiles = I32(L.mtiles);
  g.num_mtiles = I32(L.nmt);
  g.offsets = I32(L.offsets);
  g.max_mtiles = L.max_mtiles;
  g.max_ctas = d->max_ctas;
  g.P = L.P;
  g.H = (int)d->H;
  g.I = (int)d->I;
  g.E = (int)d->E;
  g.hq = reinterpret_cast<uint8_t*>(ws + L.hq);
  g.hs_t = reinterpret_cast<float*>(ws + L.hs);
  g.h16 = reinterpret_cast<__nv_bfloat16*>(ws + L.hq);
  g.status = status;
  __nv_bfloat16* xg = reinterpret_cast<__nv_bfloat16*>(ws + L.xq);  // W8A16 tensor-core path: x rows in sorted order
  if (tc1_16 && do_prep) {
    rc = moe_gather_rows_bf16(xg, reinterpret_cast<const __nv_bfloat16*>(x), I32(L.sorted), (int)d->k, L.P, (int)d->H, st);
    if (rc) return rc;
  }
  if (do_g1) {
    if (tc1) {
      MoeGemmArgs t = g;
      if (cvt) t.s0 = sc32, t.s1 = sc32 + nsc, t.scale_dtype = B200MOE_F32;
      rc = moe_gemm1_tc(t, st);
    } else if (tc1_16) {
      MoeGemmArgs t = g;
      t.a16 = xg;
      rc = moe_gemm1_w8a16_tc(t, st);
    } else {
      rc = moe_gemm1_simple(g, d->act_mode, st);
    }
  }
  if (rc) return rc;

  MoeGemmArgs g2 = g;
  g2.aq = g.hq;
  g2.as_t = g.hs_t;
  g2.a16 = g.h16;
  g2.w0 = reinterpret_cast<const uint8_t*>(w_down);
  g2.w1 = nullptr;
  g2.s0 = s_down;
  g2.s1 = nullptr;
  g2.out = reinterpret_cast<__nv_bfloat16*>(combined ? (void*)(ws + L.y) : out);
  if (do_g2) {
    if (tc2) {
      MoeGemmArgs t = g2;
      if (cvt) t.s0 = sc32 + 2 * nsc, t.scale_dtype = B200MOE_F32;
      t.ksplit = ksplit;
      if (fused) {
        t.comb32 = acc32;
        t.comb_w = topk_w;
        t.comb_wdt = d->w_dtype;
      } else if (t.ksplit > 1) {
        t.out32 = reinterpret_cast<float*>(ws + L.y32);
        cudaMemsetAsync(t.out32, 0, (size_t)L.P * d->H * sizeof(float), st);
      }
      rc = moe_gemm2_tc(t, st);
      if (!rc && !fused && t.ksplit > 1) rc = moe_f32_rows_to_bf16(g2.out, t.out32, L.P * d->H, st);
    } else if (tc2_16) {
      rc = moe_gemm2_w8a16_tc(g2, st);
    } else {
      rc = moe_gemm2_simple(g2, d->act_mode, st);
    }
  }
  if (rc) return rc;

  const void* add = nullptr;
  if (d->I_shared > 0) {
    cudaStream_t ss = side ? side->s : st;
    if (do_prep) {
      rc = moe_fill_identity_offsets(I32(L.s_offsets), d->T, ss);
      if (rc) return rc;
      rc = moe_build_mtiles(I32(L.s_mtiles), I32(L.s_nmt), I32(L.s_offsets), 1, d->T, L.s_max_mtiles, ss);
      if (rc) return rc;
    }
    if (w8a8 && do_prep) {
      rc = b200moe_quant_rows(reinterpret_cast<uint8_t*>(ws + L.s_xq), reinterpret_cast<float*>(ws + L.s_xs),
                              L.lds, x, nullptr, 1, d->T, d->H, (void*)ss);
      if (rc) return rc;
    }
    const int64_t nscs = (d->I_shared / kBlock) * (d->H / kBlock);
    if (cvt && do_prep) {
      scales_to_f32_kernel<<<(unsigned)((nscs + 255) / 256), 256, 0, ss>>>(
          reinterpret_cast<float*>(ws + L.s_sc32), reinterpret_cast<const __nv_bfloat16*>(shared_s_gate),
          reinterpret_cast<const __nv_bfloat16*>(shared_s_up), reinterpret_cast<const __nv_bfloat16*>(shared_s_down),
          nscs);
      rc = moe_launch_status();
      if (rc) return rc;
    }
    const float* ssc32 = reinterpret_cast<const float*>(ws + L.s_sc32);
    MoeGemmArgs s = g;
    s.aq = reinterpret_cast<const uint8_t*>(ws + L.s_xq);
    s.as_t = reinterpret_cast<const float*>(ws + L.s_xs);
    s.ld = L.lds;
    s.row_map = nullptr;
    s.div = 1;
    s.w0 = reinterpret_cast<const uint8_t*>(shared_w_gate);
    s.w1 = reinterpret_cast<const uint8_t*>(shared_w_up);
    s.s0 = shared_s_gate;
    s.s1 = shared_s_up;
    s.mtiles = I32(L.s_mtiles);
    s.num_mtiles = I32(L.s_nmt);
    s.offsets = I32(L.s_offsets);
    s.max_mtiles = L.s_max_mtiles;
    s.max_ctas = d->max_ctas;
    s.P = d->T;
    s.I = (int)d->I_shared;
    s.E = 1;
    s.hq = reinterpret_cast<uint8_t*>(ws + L.s_hq);
    s.hs_t = reinterpret_cast<float*>(ws + L.s_hs);
    s.h16 = reinterpret_cast<__nv_bfloat16*>(ws + L.s_hq);
    if (do_g1) {
      if (tc1) {
        MoeGemmArgs t = s;
        if (cvt) t.s0 = ssc32, t.s1 = ssc32 + nscs, t.scale_dtype = B200MOE_F32;
        rc = moe_gemm1_tc(t, ss);
      } else if (tc1_16) {
        rc = moe_gemm1_w8a16_tc(s, ss);   // identity rows: x itself is the A operand
      } else {
        rc = moe_gemm1_simple(s, d->act_mode, ss);
      }
    }
    if (rc) return rc;
    MoeGemmArgs s2 = s;
    s2.aq = s.hq;
    s2.as_t = s.hs_t;
    s2.a16 = s.h16;
    s2.w0 = reinterpret_cast<const uint8_t*>(shared_w_down);
    s2.w1 = nullptr;
    s2.s0 = shared_s_down;
    s2.s1 = nullptr;
    s2.out = reinterpret_cast<__nv_bfloat16*>(ws + L.s_y);
    if (do_g2) {
      if (tc2) {
        MoeGemmArgs t = s2;
        if (cvt) t.s0 = ssc32 + 2 * nscs, t.scale_dtype = B200MOE_F32;
        t.ksplit = choose_ksplit(d->T, 1, d->H, d->I_shared);
        if (fused) {  // weight 1, identity rows; joins the routed experts' sums in the same fp32 buffer
          t.comb32 = acc32;
          t.comb_w = nullptr;
          t.div = 1;
        } else if (t.ksplit > 1) {
          t.out32 = reinterpret_cast<float*>(ws + L.s_y32);
          cudaMemsetAsync(t.out32, 0, (size_t)d->T * d->H * sizeof(float), ss);
        }
        rc = moe_gemm2_tc(t, ss);
        if (!rc && !fused && t.ksplit > 1) rc = moe_f32_rows_to_bf16(s2.out, t.out32, d->T * d->H, ss);
      } else if (tc2_16) {
        rc = moe_gemm2_w8a16_tc(s2, ss);
      } else {
        rc = moe_gemm2_simple(s2, d->act_mode, ss);
      }
    }
    if (rc) return rc;
    if (side) {
      if (cudaEventRecord(side->join, ss) != cudaSuccess || cudaStreamWaitEvent(st, side->join, 0) != cudaSuccess)
        return (int)cudaGetLastError();
    }
    add = ws + L.s_y;
  }
  if (fused && do_comb) {
    rc = moe_f32_rows_to_bf16(reinterpret_cast<__nv_bfloat16*>(out), acc32, d->T * d->H, st);
    if (rc) return rc;
  } else if (combined && do_comb) {
    rc = b200moe_combine_masked(out, ws + L.y, nullptr, topk_w, d->w_dtype, add, ids, d->E, d->T, d->k, d->H, stream);
    if (rc) return rc;
  }
  return B200MOE_OK;
}

// ---- grouped MLP on rows that are already quantised and sorted by expert ------------------------------------------
namespace {
struct GmLayout {
  size_t mtiles, nmt, hq, hs, sc32, total;
  int max_mtiles;
};
GmLayout gm_layout(int64_t R, int64_t H, int64_t I, int64_t E, int64_t ld, int scale_dtype) {
  GmLayout L{};
  size_t o = 0;
  auto take = [&](size_t bytes) {
    size_t at = o;
    o = align_up(o + bytes, 256);
    return at;
  };
  L.max_mtiles = (int)(R / kTileM + E);
  L.mtiles = take((size_t)L.max_mtiles * 2 * sizeof(int32_t));
  L.nmt = take(sizeof(int32_t));
  L.hq = take((size_t)R * I);
  L.hs = take((size_t)(I / kBlock) * ld * sizeof(float));
  L.sc32 = take(scale_dtype == B200MOE_BF16 ? 3 * (size_t)E * (I / kBlock) * (H / kBlock) * sizeof(float) : 0);
  L.total = o;
  return L;
}
}  // namespace

extern "C" size_t b200moe_grouped_mlp_workspace_bytes(int64_t R, int64_t H, int64_t I, int64_t E, int64_t ld,
                                                      int scale_dtype) {
  if (R < 0 || H <= 0 || I <= 0 || E <= 0 || H % kBlock || I % kBlock || ld < R) return 0;
  return gm_layout(R, H, I, E, ld, scale_dtype).total;
}

namespace {
// shared body of b200moe_grouped_mlp (y/row_map) and b200moe_grouped_mlp_remote (row_src/out_tbl)
int grouped_mlp_impl(void* y, const uint8_t* xq, const float* xs_t, int64_t ld, const int32_t* expert_offsets,
                     const int32_t* row_map, const int32_t* row_src, const uint64_t* out_tbl, const void* w_gate,
                     const void* w_up, const void* w_down, const void* s_gate, const void* s_up, const void* s_down,
                     int scale_dtype, int64_t R, int64_t H, int64_t I, int64_t E, int impl, void* workspace,
                     size_t workspace_bytes, int32_t* status, void* stream) {
  MOE_CHECK_ARG(R >= 0 && H > 0 && I > 0 && E > 0 && ld >= R);
  MOE_CHECK_ARG(scale_dtype == B200MOE_F32 || scale_dtype == B200MOE_BF16);
  MOE_CHECK_ARG(impl >= B200MOE_IMPL_AUTO && impl <= B200MOE_IMPL_TCGEN05);
  MOE_CHECK_SHAPE(H % kBlock == 0 && I % kBlock == 0 && E <= 1024 && R < (1 << 24) && E * I < (int64_t(1) << 31));
  if (R == 0) return B200MOE_OK;
  MOE_CHECK_ARG((y || row_src) && xq && xs_t && expert_offsets && w_gate && w_up && w_down && s_gate && s_up && s_down);
  if ((y && !moe_aligned16(y)) || !moe_aligned16(xq) || !moe_aligned16(w_gate) || !moe_aligned16(w_up) ||
      !moe_aligned16(w_down))
    return B200MOE_EALIGN;
  const GmLayout L = gm_layout(R, H, I, E, ld, scale_dtype);
  if (!workspace || workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return B200MOE_EWORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = reinterpret_cast<char*>(workspace);
  const bool use_tc = impl != B200MOE_IMPL_SIMPLE && moe_tc_available();
  if (impl == B200MOE_IMPL_TCGEN05 && !use_tc) return B200MOE_EDRIVER;
  if (row_src && !use_tc) return B200MOE_EDRIVER;  // peer output exists on the tensor-core path only
  int32_t* mtiles = reinterpret_cast<int32_t*>(ws + L.mtiles);
  int32_t* nmt = reinterpret_cast<int32_t*>(ws + L.nmt);
  int rc = moe_build_mtiles(mtiles, nmt, expert_offsets, (int)E, R, L.max_mtiles, st);
  if (rc) return rc;
  const void *sg = s_gate, *su = s_up, *sd = s_down;
  int sdt = scale_dtype;
  if (use_tc && scale_dtype == B200MOE_BF16) {
    const int64_t nsc = E * (I / kBlock) * (H / kBlock);
    float* sc32 = reinterpret_cast<float*>(ws + L.sc32);
    scales_to_f32_kernel<<<(unsigned)((nsc + 255) / 256), 256, 0, st>>>(
        sc32, reinterpret_cast<const __nv_bfloat16*>(s_gate), reinterpret_cast<const __nv_bfloat16*>(s_up),
        reinterpret_cast<const __nv_bfloat16*>(s_down), nsc);
    rc = moe_launch_status();
    if (rc) return rc;
    sg = sc32, su = sc32 + nsc, sd = sc32 + 2 * nsc, sdt = B200MOE_F32;
  }
  MoeGemmArgs g{};
  g.aq = xq;
  g.as_t = xs_t;
  g.ld = ld;
  g.row_map = nullptr;
  g.div = 1;
  g.w0 = reinterpret_cast<const uint8_t*>(w_gate);
  g.w1 = reinterpret_cast<const uint8_t*>(w_up);
  g.s0 = sg;
  g.s1 = su;
  g.scale_dtype = sdt;
  g.mtiles = mtiles;
  g.num_mtiles = nmt;
  g.offsets = expert_offsets;
  g.max_mtiles = L.max_mtiles;
  g.P = R;
  g.H = (int)H;
  g.I = (int)I;
  g.E = (int)E;
  g.hq = reinterpret_cast<uint8_t*>(ws + L.hq);
  g.hs_t = reinterpret_cast<float*>(ws + L.hs);
  g.status = status;
  rc = use_tc ? moe_gemm1_tc(g, st) : moe_gemm1_simple(g, B200MOE_ACT_W8A8, st);
  if (rc) return rc;
  MoeGemmArgs g2 = g;
  g2.aq = g.hq;
  g2.as_t = g.hs_t;
  g2.row_map = row_map;
  g2.row_src = row_src;
  g2.out_tbl = out_tbl;
  g2.w0 = reinterpret_cast<const uint8_t*>(w_down);
  g2.w1 = nullptr;
  g2.s0 = sd;
  g2.s1 = nullptr;
  g2.out = reinterpret_cast<__nv_bfloat16*>(y);
  return use_tc ? moe_gemm2_tc(g2, st) : moe_gemm2_simple(g2, B200MOE_ACT_W8A8, st);
}
}  // namespace

extern "C" int b200moe_grouped_mlp(void* y, const uint8_t* xq, const float* xs_t, int64_t ld,
                                   const int32_t* expert_offsets, const int32_t* row_map, const void* w_gate,
                                   const void* w_up, const void* w_down, const void* s_gate, const void* s_up,
                                   const void* s_down, int scale_dtype, int64_t R, int64_t H, int64_t I, int64_t E,
                                   int impl, void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  MOE_CHECK_ARG(y);
  return grouped_mlp_impl(y, xq, xs_t, ld, expert_offsets, row_map, nullptr, nullptr, w_gate, w_up, w_down, s_gate,
                          s_up, s_down, scale_dtype, R, H, I, E, impl, workspace, workspace_bytes, status, stream);
}

extern "C" int b200moe_grouped_mlp_remote(const uint64_t* out_tbl, const int32_t* row_src, const uint8_t* xq,
                                          const float* xs_t, int64_t ld, const int32_t* expert_offsets,
                                          const void* w_gate, const void* w_up, const void* w_down,
                                          const void* s_gate, const void* s_up, const void* s_down, int scale_dtype,
                                          int64_t R_capacity, int64_t H, int64_t I, int64_t E, void* workspace,
                                          size_t workspace_bytes, int32_t* status, void* stream) {
  MOE_CHECK_ARG(out_tbl && row_src);
  return grouped_mlp_impl(nullptr, xq, xs_t, ld, expert_offsets, nullptr, row_src, out_tbl, w_gate, w_up, w_down,
                          s_gate, s_up, s_down, scale_dtype, R_capacity, H, I, E, B200MOE_IMPL_TCGEN05, workspace,
                          workspace_bytes, status, stream);
}

// ---- plain FP8 block-scaled linear layer -----------------------------------------------------------------
namespace {
struct LinLayout {
  size_t offsets, mtiles, nmt, xq, xs, sc32, total;
  int64_t ld;
  int max_mtiles;
};
LinLayout lin_layout(int64_t M, int64_t K, int64_t N, int scale_dtype) {
  LinLayout L{};
  size_t o = 0;
  auto take = [&](size_t bytes) {
    size_t at = o;
    o = (o + bytes + 255) & ~(size_t)255;
    return at;
  };
  L.ld = (M + kTileM - 1) / kTileM * kTileM;
  if (L.ld == 0) L.ld = kTileM;
  L.max_mtiles = (int)(L.ld / kTileM);
  L.offsets = take(2 * sizeof(int32_t));
  L.mtiles = take((size_t)L.max_mtiles * 2 * sizeof(int32_t));
  L.nmt = take(sizeof(int32_t));
  L.xq = take((size_t)L.ld * K);
  L.xs = take((size_t)(K / kBlock) * L.ld * sizeof(float));
  L.sc32 = take(scale_dtype == B200MOE_BF16 ? (size_t)((N + kBlock - 1) / kBlock) * (K / kBlock) * sizeof(float) : 0);
  L.total = o;
  return L;
}
__global__ void scales1_to_f32_kernel(float* __restrict__ dst, const __nv_bfloat16* __restrict__ s, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __bfloat162float(s[i]);
}
}  // namespace

extern "C" size_t b200moe_linear_workspace_bytes(int64_t M, int64_t K, int64_t N, int scale_dtype) {
  if (M < 0 || K <= 0 || N <= 0 || K % kBlock || N % 64) return 0;
  return lin_layout(M, K, N, scale_dtype).total;
}

extern "C" int b200moe_linear_w8(void* out, const void* x, const void* w, const void* scale, int scale_dtype,
                                 int64_t M, int64_t K, int64_t N, void* workspace, size_t workspace_bytes,
                                 int32_t* status, void* stream) {
  MOE_CHECK_ARG(M >= 0 && K > 0 && N > 0);
  MOE_CHECK_ARG(scale_dtype == B200MOE_F32 || scale_dtype == B200MOE_BF16);
  MOE_CHECK_SHAPE(K % kBlock == 0 && N % 64 == 0 && M < (1 << 24) && N < (int64_t(1) << 31));
  if (M == 0) return B200MOE_OK;
  MOE_CHECK_ARG(out && x && w && scale);
  if (!moe_aligned16(out) || !moe_aligned16(x) || !moe_aligned16(w)) return B200MOE_EALIGN;
  if (!moe_tc_available()) return B200MOE_EDRIVER;
  const LinLayout L = lin_layout(M, K, N, scale_dtype);
  if (!workspace || workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return B200MOE_EWORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = reinterpret_cast<char*>(workspace);
  int32_t* offsets = reinterpret_cast<int32_t*>(ws + L.offsets);
  int32_t* mtiles = reinterpret_cast<int32_t*>(ws + L.mtiles);
  int32_t* nmt = reinterpret_cast<int32_t*>(ws + L.nmt);
  int rc = moe_fill_identity_offsets(offsets, M, st);
  if (rc) return rc;
  rc = moe_build_mtiles(mtiles, nmt, offsets, 1, M, L.max_mtiles, st);
  if (rc) return rc;
  rc = b200moe_quant_rows(reinterpret_cast<uint8_t*>(ws + L.xq), reinterpret_cast<float*>(ws + L.xs), L.ld, x, nullptr,
                          1, M, K, stream);
  if (rc) return rc;
  const void* sc = scale;
  if (scale_dtype == B200MOE_BF16) {
    const int64_t n = ((N + kBlock - 1) / kBlock) * (K / kBlock);
    scales1_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<float*>(ws + L.sc32), reinterpret_cast<const __nv_bfloat16*>(scale), n);
    rc = moe_launch_status();
    if (rc) return rc;
    sc = ws + L.sc32;
  }
  MoeGemmArgs g{};
  g.aq = reinterpret_cast<const uint8_t*>(ws + L.xq);
  g.as_t = reinterpret_cast<const float*>(ws + L.xs);
  g.ld = L.ld;
  g.div = 1;
  g.w0 = reinterpret_cast<const uint8_t*>(w);
  g.s0 = sc;
  g.scale_dtype = B200MOE_F32;
  g.mtiles = mtiles;
  g.num_mtiles = nmt;
  g.offsets = offsets;
  g.max_mtiles = L.max_mtiles;
  g.P = M;
  g.H = (int)K;
  g.I = (int)N;
  g.E = 1;
  g.out = reinterpret_cast<__nv_bfloat16*>(out);
  g.status = status;
  return moe_linear_tc(g, st);
}

// ---- FP8 x FP8 matrix product with one scale per operand ------------------------------------------------------------
namespace {
__global__ void fill_scalar_scale_kernel(float* __restrict__ dst, const float* __restrict__ scale, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = scale ? *scale : 1.0f;
}
struct SmmLayout {
  size_t offsets, mtiles, nmt, xs, ws, total;
  int64_t ld;
  int max_mtiles;
};
SmmLayout smm_layout(int64_t M, int64_t K, int64_t N) {
  SmmLayout L{};
  size_t o = 0;
  auto take = [&](size_t bytes) {
    size_t at = o;
    o = (o + bytes + 255) & ~(size_t)255;
    return at;
  };
  L.ld = (M + kTileM - 1) / kTileM * kTileM;
  if (L.ld == 0) L.ld = kTileM;
  L.max_mtiles = (int)(L.ld / kTileM);
  L.offsets = take(2 * sizeof(int32_t));
  L.mtiles = take((size_t)L.max_mtiles * 2 * sizeof(int32_t));
  L.nmt = take(sizeof(int32_t));
  L.xs = take((size_t)(K / kBlock) * L.ld * sizeof(float));
  L.ws = take((size_t)((N + kBlock - 1) / kBlock) * (K / kBlock) * sizeof(float));
  L.total = o;
  return L;
}
}  // namespace

extern "C" size_t b200moe_scaled_mm_workspace_bytes(int64_t M, int64_t K, int64_t N) {
  if (M < 0 || K <= 0 || N <= 0 || K % kBlock || N % 64) return 0;
  return smm_layout(M, K, N).total;
}

extern "C" int b200moe_scaled_mm(void* out, int out_dtype, const void* a, const void* b, const float* scale_a,
                                 const float* scale_b, int64_t M, int64_t K, int64_t N, void* workspace,
                                 size_t workspace_bytes, int32_t* status, void* stream) {
  MOE_CHECK_ARG(M >= 0 && K > 0 && N > 0);
  MOE_CHECK_ARG(out_dtype == B200MOE_BF16 || out_dtype == B200MOE_F32);
  MOE_CHECK_SHAPE(K % kBlock == 0 && N % 64 == 0 && M < (1 << 24) && N < (int64_t(1) << 31));
  if (M == 0) return B200MOE_OK;
  MOE_CHECK_ARG(out && a && b);
  if (!moe_aligned16(out) || !moe_aligned16(a) || !moe_aligned16(b)) return B200MOE_EALIGN;
  if (!moe_tc_available()) return B200MOE_EDRIVER;
  const SmmLayout L = smm_layout(M, K, N);
  if (!workspace || workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return B200MOE_EWORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = reinterpret_cast<char*>(workspace);
  int32_t* offsets = reinterpret_cast<int32_t*>(ws + L.offsets);
  int32_t* mtiles = reinterpret_cast<int32_t*>(ws + L.mtiles);
  int32_t* nmt = reinterpret_cast<int32_t*>(ws + L.nmt);
  int rc = moe_fill_identity_offsets(offsets, M, st);
  if (rc) return rc;
  rc = moe_build_mtiles(mtiles, nmt, offsets, 1, M, L.max_mtiles, st);
  if (rc) return rc;
  // the kernel applies act_scale[row,kb] * weight_scale[nb,kb] to every 128-deep partial sum: constant grids here
  const int64_t nxs = (K / kBlock) * L.ld, nws = ((N + kBlock - 1) / kBlock) * (K / kBlock);
  fill_scalar_scale_kernel<<<(unsigned)((nxs + 255) / 256), 256, 0, st>>>(reinterpret_cast<float*>(ws + L.xs), scale_a, nxs);
  fill_scalar_scale_kernel<<<(unsigned)((nws + 255) / 256), 256, 0, st>>>(reinterpret_cast<float*>(ws + L.ws), scale_b, nws);
  rc = moe_launch_status();
  if (rc) return rc;
  MoeGemmArgs g{};
  g.aq = reinterpret_cast<const uint8_t*>(a);
  g.as_t = reinterpret_cast<const float*>(ws + L.xs);
  g.ld = L.ld;
  g.div = 1;
  g.w0 = reinterpret_cast<const uint8_t*>(b);
  g.s0 = ws + L.ws;
  g.scale_dtype = B200MOE_F32;
  g.mtiles = mtiles;
  g.num_mtiles = nmt;
  g.offsets = offsets;
  g.max_mtiles = L.max_mtiles;
  g.P = M;
  g.H = (int)K;
  g.I = (int)N;
  g.E = 1;
  if (out_dtype == B200MOE_F32) g.out32 = reinterpret_cast<float*>(out);
  else g.out = reinterpret_cast<__nv_bfloat16*>(out);
  g.status = status;
  return moe_linear_tc(g, st);
}

extern "C" int b200moe_abi_version(void) { return B200MOE_ABI_VERSION; }

extern "C" const char* b200moe_error_string(int code) {
  switch (code) {
    case B200MOE_OK: return "ok";
    case B200MOE_EINVAL: return "invalid argument (null pointer, non-positive size or unknown enum)";
    case B200MOE_ESHAPE: return "unsupported size";
    case B200MOE_EWORKSPACE: return "workspace too small or not 256-byte aligned";
    case B200MOE_EALIGN: return "pointer not 16-byte aligned";
    case B200MOE_EDRIVER: return "tensor-core path unavailable (no sm_100 device or no tensor-map driver entry point)";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
  }
}

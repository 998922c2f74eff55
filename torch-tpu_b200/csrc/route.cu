// Routing kernels: plain / grouped top-k on given scores, the fused score->select->normalise chain,
// and the router GEMM.  One warp owns one row; element e of the row lives in lane e%32, register e/32,
// so loads are coalesced and every selection step is a register scan plus five shuffles.
//
// Tie rule everywhere: among equal values the LOWEST index wins (the reference leaves tie order open:
// aten::topk on its CPU path and an index-perturbation on its device path, native_ops/Topk.pl:82-100).
#include <float.h>
#include <limits.h>
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kWarpsPerBlock = 4;

__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, v, o);
    int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) {
      v = ov;
      idx = oi;
    }
  }
}

// Top-k of a row held as v[j] <-> element lane + 32*j (elements >= n are not candidates).
// Lane j (< k) returns the j-th result in (rv, ri).
template <int VPT>
__device__ __forceinline__ void warp_topk(const float (&v)[VPT], int n, int k, int lane, float& rv,
                                          int& ri) {
  uint32_t taken = 0;
  rv = -INFINITY;
  ri = 0;
  for (int it = 0; it < k; ++it) {
    float bv = -INFINITY;
    int bi = INT_MAX;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int e = lane + 32 * j;
      bool cand = e < n && !((taken >> j) & 1u);
      if (cand && (bi == INT_MAX || v[j] > bv)) {  // ascending e inside a lane: first max wins
        bv = v[j];
        bi = e;
      }
    }
    warp_argmax(bv, bi);
    if (bi != INT_MAX && (bi & 31) == lane) taken |= 1u << (bi >> 5);
    if (lane == it) {
      rv = bv;
      ri = bi == INT_MAX ? 0 : bi;
    }
  }
}

// Group-limited masking (python/regression/test_llm/test_noaux_tc_topk.py:10-35): group score = sum of
// the two largest members (formed in `dtype`), keep `topk_groups` groups, mask the rest to -inf.
template <int VPT>
__device__ __forceinline__ void group_mask(float (&v)[VPT], int n, int n_groups, int topk_groups,
                                           int dtype, int lane) {
  const int gsz = n / n_groups;
  float my_gs = -INFINITY;  // lane g holds the score of group g
  for (int g = 0; g < n_groups; ++g) {
    float a1 = -INFINITY, a2 = -INFINITY;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int e = lane + 32 * j;
      if (e < n && e / gsz == g) {
        float x = v[j];
        if (x > a1) {
          a2 = a1;
          a1 = x;
        } else if (x > a2) {
          a2 = x;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float b1 = __shfl_xor_sync(0xffffffffu, a1, o);
      float b2 = __shfl_xor_sync(0xffffffffu, a2, o);
      float hi = fmaxf(a1, b1);
      float lo = fmaxf(fminf(a1, b1), fmaxf(a2, b2));
      a1 = hi;
      a2 = lo;
    }
    float gs = gsz > 1 ? moe_add_in_dtype(a1, a2, dtype) : a1;
    if (lane == g) my_gs = gs;
  }
  uint32_t keep = 0;
  bool used = false;
  for (int it = 0; it < topk_groups; ++it) {
    float bv = (lane < n_groups && !used) ? my_gs : -INFINITY;
    int bi = (lane < n_groups && !used) ? lane : INT_MAX;
    warp_argmax(bv, bi);
    if (bi != INT_MAX) {
      keep |= 1u << bi;
      if (bi == lane) used = true;
    }
  }
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    int e = lane + 32 * j;
    if (e < n && !((keep >> (e / gsz)) & 1u)) v[j] = -INFINITY;
  }
}

template <int VPT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
topk_kernel(void* __restrict__ values, int32_t* __restrict__ indices, const void* __restrict__ scores,
            int dtype, int64_t batch, int n, int n_groups, int topk_groups, int k) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= batch) return;
  float v[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    int e = lane + 32 * j;
    v[j] = e < n ? moe_load_as_f32(scores, row * n + e, dtype) : -INFINITY;
  }
  if (n_groups > 1) group_mask<VPT>(v, n, n_groups, topk_groups, dtype, lane);
  float rv;
  int ri;
  warp_topk<VPT>(v, n, k, lane, rv, ri);
  if (lane < k) {
    moe_store_from_f32(values, row * k + lane, dtype, rv);
    indices[row * k + lane] = ri;
  }
}

template <int VPT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
route_kernel(int32_t* __restrict__ ids, float* __restrict__ w, __nv_bfloat16* __restrict__ w_bf16,
             const float* __restrict__ logits, const float* __restrict__ logit_bias,
             const float* __restrict__ bias, int64_t T, int n, int k, int score_func, int n_groups, int topk_groups, int renorm, float scale) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= T) return;
  float s[VPT];    // un-biased scores
  float sel[VPT];  // selection scores
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    int e = lane + 32 * j;
    s[j] = e < n ? (logit_bias ? logits[row * n + e] + logit_bias[e] : logits[row * n + e]) : -INFINITY;
  }
  if (score_func == B200MOE_SCORE_SOFTMAX) {
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < VPT; ++j) m = fmaxf(m, s[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int e = lane + 32 * j;
      s[j] = e < n ? expf(s[j] - m) : 0.f;
      sum += s[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
    for (int j = 0; j < VPT; ++j) s[j] = s[j] / sum;
  } else {
#pragma unroll
    for (int j = 0; j < VPT; ++j) s[j] = 1.0f / (1.0f + expf(-s[j]));
  }
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    int e = lane + 32 * j;
    sel[j] = e < n ? (bias ? s[j] + bias[e] : s[j]) : -INFINITY;
  }
  if (n_groups > 1) group_mask<VPT>(sel, n, n_groups, topk_groups, B200MOE_F32, lane);
  float rv;
  int ri;
  warp_topk<VPT>(sel, n, k, lane, rv, ri);
  // gather the un-biased score of the chosen expert: it lives in lane ri%32, register ri/32
  float wv = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    // every lane publishes register j; lane `it` picks the one it needs
    float cand = __shfl_sync(0xffffffffu, s[j], ri & 31);
    if ((ri >> 5) == j) wv = cand;
  }
  if (lane >= k) wv = 0.f;
  if (renorm) {
    float sum = wv;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    wv = wv / sum;
  }
  wv = wv * scale;
  if (lane < k) {
    ids[row * k + lane] = ri;
    w[row * k + lane] = wv;
    if (w_bf16) w_bf16[row * k + lane] = __float2bfloat16_rn(wv);
  }
}

// ---- router GEMM ---------------------------------------------------------------------------------
// logits[t,e] = sum_h x[t,h] * wr[e,h]; bf16 operands, fp32 accumulation on the warp-level tensor path
// (mma.sync m16n8k16).  It is ~0.5 % of the layer's FLOPs, so it stays a small, plain kernel: CTA tile
// 32 tokens x 64 experts, K chunks of 64 staged in shared memory, 4 warps each owning 16 token rows x 32 experts.
constexpr int RG_BM = 32, RG_BN = 64, RG_BK = 64, RG_LD = RG_BK + 8, RG_STAGES = 3;  // +8 bf16: conflict-free fragment reads

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// 16-byte asynchronous copy global -> shared; bytes = 0 writes zeros (rows / columns past the end)
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
               "l"(gsrc), "r"(bytes)
               : "memory");
}

__global__ void __launch_bounds__(128)
router_gemm_kernel(float* __restrict__ logits, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ wr, int64_t T, int64_t H, int64_t E) {
  // Three stages: the copies of K chunks kt+1 and kt+2 are in flight while the MMAs of chunk kt run.  The MMAs of a
  // chunk are a few hundred cycles and a copy is an L2 round trip, so the kernel lives on copies in flight: tiles
  // of 32 rows (twice the blocks of a 64-row tile, two or three per SM) and three stages keep about four chunks
  // per SM on their way.  A sum over K is formed in the same order whatever the tiling: logits do not change.
  __shared__ __align__(16) __nv_bfloat16 sA[RG_STAGES][RG_BM * RG_LD];
  __shared__ __align__(16) __nv_bfloat16 sB[RG_STAGES][RG_BN * RG_LD];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp & 1, wn = warp >> 1;  // the warp's 16 rows and 32 columns of the 32 x 64 tile
  const int64_t t0 = (int64_t)blockIdx.x * RG_BM, e0 = (int64_t)blockIdx.y * RG_BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int g = lane >> 2, tq = lane & 3;
  auto load_stage = [&](int st, int64_t k0) {
    // A: 32 rows x 64 bf16 = 256 chunks of 16 B (128 threads x 2); B: 64 rows = 512 chunks (x 4)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = tid + i * 128;
      const int r = c >> 3, cc = (c & 7) * 8;
      const bool ok = k0 + cc < H && t0 + r < T;
      cp_async16(sA[st] + r * RG_LD + cc, ok ? x + (t0 + r) * H + k0 + cc : x, ok ? 16 : 0);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = tid + i * 128;
      const int r = c >> 3, cc = (c & 7) * 8;
      const bool ok = k0 + cc < H && e0 + r < E;
      cp_async16(sB[st] + r * RG_LD + cc, ok ? wr + (e0 + r) * H + k0 + cc : wr, ok ? 16 : 0);
    }
  };
  const int nk = (int)((H + RG_BK - 1) / RG_BK);
  // one commit group per chunk, empty where there is no chunk left, so that "all but the two newest groups are
  // complete" always means "chunk kt has landed"
  load_stage(0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  if (nk > 1) load_stage(1, RG_BK);
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int kt = 0; kt < nk; ++kt) {
    const int st = kt % RG_STAGES;
    if (kt + 2 < nk) load_stage((kt + 2) % RG_STAGES, (int64_t)(kt + 2) * RG_BK);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 2;" ::: "memory");
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < RG_BK; kk += 16) {
      uint32_t a[4];
      const __nv_bfloat16* pa = sA[st] + (wm * 16 + g) * RG_LD + kk + tq * 2;
      a[0] = *reinterpret_cast<const uint32_t*>(pa);
      a[1] = *reinterpret_cast<const uint32_t*>(pa + 8 * RG_LD);
      a[2] = *reinterpret_cast<const uint32_t*>(pa + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(pa + 8 * RG_LD + 8);
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        uint32_t b[2];
        const __nv_bfloat16* pb = sB[st] + (wn * 32 + nb * 8 + g) * RG_LD + kk + tq * 2;
        b[0] = *reinterpret_cast<const uint32_t*>(pb);
        b[1] = *reinterpret_cast<const uint32_t*>(pb + 8);
        mma_bf16_16816(acc[nb], a, b);
      }
    }
    __syncthreads();  // the stage is overwritten by the copies issued at the top of the next iteration
  }
#pragma unroll
  for (int nb = 0; nb < 4; ++nb) {
    int64_t r0 = t0 + wm * 16 + g, c0 = e0 + wn * 32 + nb * 8 + tq * 2;
    if (r0 < T) {
      if (c0 < E) logits[r0 * E + c0] = acc[nb][0];
      if (c0 + 1 < E) logits[r0 * E + c0 + 1] = acc[nb][1];
    }
    if (r0 + 8 < T) {
      if (c0 < E) logits[(r0 + 8) * E + c0] = acc[nb][2];
      if (c0 + 1 < E) logits[(r0 + 8) * E + c0 + 1] = acc[nb][3];
    }
  }
}

// Small-T variant (decode): one block per expert row; its 4 warps split H (16-byte loads) and dot the slice with up
// to RV_MAXT token rows; the warps' partial sums are added in warp order (deterministic).  The grid covers all
// experts, so the read of the router weights is spread over many SMs and only H/1024 loads deep.
constexpr int RV_MAXT = 8;
__global__ void __launch_bounds__(128)
router_gemv_kernel(float* __restrict__ logits, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ wr, int64_t T, int64_t H, int64_t E) {
  __shared__ float part[4][RV_MAXT];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t e = blockIdx.x;
  const int64_t t0 = (int64_t)blockIdx.y * RV_MAXT;
  float acc[RV_MAXT];
#pragma unroll
  for (int t = 0; t < RV_MAXT; ++t) acc[t] = 0.f;
  for (int64_t h = (int64_t)threadIdx.x * 8; h < H; h += 1024) {
    uint4 wv = *reinterpret_cast<const uint4*>(wr + e * H + h);
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
    for (int t = 0; t < RV_MAXT; ++t) {
      if (t0 + t < T) {
        uint4 xv = *reinterpret_cast<const uint4*>(x + (t0 + t) * H + h);
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 a = __bfloat1622float2(w2[i]), b = __bfloat1622float2(x2[i]);
          acc[t] = fmaf(a.x, b.x, acc[t]);
          acc[t] = fmaf(a.y, b.y, acc[t]);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < RV_MAXT; ++t) {
    float v = acc[t];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) part[warp][t] = v;
  }
  __syncthreads();
  if (threadIdx.x < RV_MAXT && t0 + threadIdx.x < T)
    logits[(t0 + threadIdx.x) * E + e] = part[0][threadIdx.x] + part[1][threadIdx.x] + part[2][threadIdx.x] + part[3][threadIdx.x];
}

constexpr int RS_TOK = 4, RS_WARPS = 8;
// Few-experts variant (E <= 16, e.g. 8 for Mixtral): the 64x64 tensor-core tile would be mostly padding, and the
// op is a read of x.  A block owns RS_TOK tokens and its 8 warps split H between them (interleaved 256-column
// slices, 16-byte loads of x and of the L2-resident router weights), so that decode-size batches still fill more
// than a handful of SMs; the per-warp partial sums meet in shared memory and are added in warp order, so the
// result does not depend on timing.
template <int EP>
__global__ void __launch_bounds__(RS_WARPS * 32)
router_small_e_kernel(float* __restrict__ logits, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ wr, int64_t T, int64_t H, int E) {
  __shared__ float part[RS_WARPS][RS_TOK][EP];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t0 = (int64_t)blockIdx.x * RS_TOK;
  float acc[RS_TOK][EP];
#pragma unroll
  for (int i = 0; i < RS_TOK; ++i)
#pragma unroll
    for (int e = 0; e < EP; ++e) acc[i][e] = 0.f;
  for (int64_t col = (int64_t)(warp * 32 + lane) * 8; col < H; col += RS_WARPS * 256) {
    float xv[RS_TOK][8];
#pragma unroll
    for (int i = 0; i < RS_TOK; ++i) {
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (t0 + i < T) raw = *reinterpret_cast<const uint4*>(x + (t0 + i) * H + col);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(b2[j]);
        xv[i][2 * j] = f.x;
        xv[i][2 * j + 1] = f.y;
      }
    }
#pragma unroll
    for (int e = 0; e < EP; ++e) {
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (e < E) raw = *reinterpret_cast<const uint4*>(wr + (int64_t)e * H + col);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(b2[j]);
#pragma unroll
        for (int i = 0; i < RS_TOK; ++i) {
          acc[i][e] = fmaf(xv[i][2 * j], f.x, acc[i][e]);
          acc[i][e] = fmaf(xv[i][2 * j + 1], f.y, acc[i][e]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < RS_TOK; ++i)
#pragma unroll
    for (int e = 0; e < EP; ++e) {
      float v = acc[i][e];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) part[warp][i][e] = v;
    }
  __syncthreads();
  if (threadIdx.x < RS_TOK * EP) {
    const int i = threadIdx.x / EP, e = threadIdx.x % EP;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < RS_WARPS; ++w) v += part[w][i][e];
    if (t0 + i < T && e < E) logits[(t0 + i) * E + e] = v;
  }
}

template <typename F>
int dispatch_vpt(int64_t n, F&& f) {
  if (n <= 32) return f(std::integral_constant<int, 1>{});
  if (n <= 64) return f(std::integral_constant<int, 2>{});
  if (n <= 128) return f(std::integral_constant<int, 4>{});
  if (n <= 256) return f(std::integral_constant<int, 8>{});
  if (n <= 512) return f(std::integral_constant<int, 16>{});
  return f(std::integral_constant<int, 32>{});
}

int launch_topk(void* values, int32_t* indices, const void* scores, int dtype, int64_t batch, int64_t n,
                int64_t n_groups, int64_t topk_groups, int64_t k, void* stream) {
  MOE_CHECK_ARG(values && indices && scores);
  MOE_CHECK_ARG(dtype == B200MOE_F32 || dtype == B200MOE_BF16 || dtype == B200MOE_F16);
  MOE_CHECK_ARG(batch >= 0 && n > 0 && k > 0);
  MOE_CHECK_SHAPE(n <= 1024 && k <= 32 && k <= n);
  if (n_groups > 1) {
    MOE_CHECK_SHAPE(n_groups <= 32 && n % n_groups == 0 && topk_groups >= 1 && topk_groups <= n_groups);
    MOE_CHECK_SHAPE(k <= topk_groups * (n / n_groups));
  }
  if (batch == 0) return B200MOE_OK;
  dim3 grid((unsigned)((batch + kWarpsPerBlock - 1) / kWarpsPerBlock));
  return dispatch_vpt(n, [&](auto vpt) {
    topk_kernel<decltype(vpt)::value><<<grid, kWarpsPerBlock * 32, 0, (cudaStream_t)stream>>>(
        values, indices, scores, dtype, batch, (int)n, (int)n_groups, (int)topk_groups, (int)k);
    return moe_launch_status();
  });
}

}  // namespace

extern "C" int b200moe_noaux_tc_topk(void* values, int32_t* indices, const void* scores, int dtype,
                                     int64_t batch, int64_t n_experts, int64_t n_groups,
                                     int64_t topk_groups, int64_t top_k, void* stream) {
  MOE_CHECK_ARG(n_groups >= 1);
  return launch_topk(values, indices, scores, dtype, batch, n_experts, n_groups, topk_groups, top_k, stream);
}

extern "C" int b200moe_topk(void* values, int32_t* indices, const void* x, int dtype, int64_t batch,
                            int64_t n, int64_t k, void* stream) {
  return launch_topk(values, indices, x, dtype, batch, n, 1, 1, k, stream);
}

extern "C" int b200moe_route(int32_t* ids, float* w, void* w_bf16, const float* logits,
                             const float* logit_bias, const float* bias, int64_t T, int64_t E, int64_t k, int score_func, int64_t n_groups,
                             int64_t topk_groups, int renorm, float scale, void* stream) {
  MOE_CHECK_ARG(ids && w && logits && T >= 0 && E > 0 && k > 0);
  MOE_CHECK_ARG(score_func == B200MOE_SCORE_SOFTMAX || score_func == B200MOE_SCORE_SIGMOID);
  MOE_CHECK_SHAPE(E <= 1024 && k <= 32 && k <= E);
  if (n_groups > 1) {
    MOE_CHECK_SHAPE(n_groups <= 32 && E % n_groups == 0 && topk_groups >= 1 && topk_groups <= n_groups);
    MOE_CHECK_SHAPE(k <= topk_groups * (E / n_groups));
  }
  if (T == 0) return B200MOE_OK;
  dim3 grid((unsigned)((T + kWarpsPerBlock - 1) / kWarpsPerBlock));
  return dispatch_vpt(E, [&](auto vpt) {
    route_kernel<decltype(vpt)::value><<<grid, kWarpsPerBlock * 32, 0, (cudaStream_t)stream>>>(
        ids, w, reinterpret_cast<__nv_bfloat16*>(w_bf16), logits, logit_bias, bias, T, (int)E, (int)k, score_func,
        (int)(n_groups > 1 ? n_groups : 1), (int)topk_groups, renorm, scale);
    return moe_launch_status();
  });
}

extern "C" int b200moe_router_logits(float* logits, const void* x, const void* wr, int64_t T, int64_t H,
                                     int64_t E, void* stream) {
  MOE_CHECK_ARG(logits && x && wr && T >= 0 && H > 0 && E > 0);
  MOE_CHECK_SHAPE(H % 8 == 0);
  if (!moe_aligned16(x) || !moe_aligned16(wr)) return B200MOE_EALIGN;
  if (T == 0) return B200MOE_OK;
  auto xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto wb = reinterpret_cast<const __nv_bfloat16*>(wr);
  if (T <= 2 * RV_MAXT) {
    dim3 grid((unsigned)E, (unsigned)((T + RV_MAXT - 1) / RV_MAXT));
    router_gemv_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(logits, xb, wb, T, H, E);
  } else if (E <= 16) {
    const unsigned grid = (unsigned)((T + RS_TOK - 1) / RS_TOK);
    if (E <= 8) router_small_e_kernel<8><<<grid, RS_WARPS * 32, 0, (cudaStream_t)stream>>>(logits, xb, wb, T, H, (int)E);
    else router_small_e_kernel<16><<<grid, RS_WARPS * 32, 0, (cudaStream_t)stream>>>(logits, xb, wb, T, H, (int)E);
  } else {
    dim3 grid((unsigned)((T + RG_BM - 1) / RG_BM), (unsigned)((E + RG_BN - 1) / RG_BN));
    router_gemm_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(logits, xb, wb, T, H, E);
  }
  return moe_launch_status();
}

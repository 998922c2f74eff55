// Plain CUDA-core grouped GEMMs: the small, obviously-correct implementation of the two expert GEMMs.
// It exists so that the tensor-core kernels can be A/B-checked on the device (same inputs, same
// workspace layout) and it carries the W8A16 arithmetic of the reference (weights dequantised to bf16,
// every intermediate rounded to bf16: my_ops/fusedMoE.pl:217-269, python/regression/test_llm/test_moe.py:63-84).
// Tile: 16 rows x 128 columns per CTA of 256 threads (thread = row tid/16, columns tid%16 + 16*i).
#include "internal.h"

namespace {

constexpr int SR = 16;   // rows per CTA
constexpr int SKC = 32;  // K chunk staged in shared memory

__device__ __forceinline__ float scale_at(const void* s, int64_t i, int dtype) { return moe_load_as_f32(s, i, dtype); }

template <int ACT>
__global__ void __launch_bounds__(256) gemm1_simple_kernel(MoeGemmArgs a) {
  __shared__ float sA[SR][SKC + 1];
  __shared__ float sG[128][SKC + 1];
  __shared__ float sU[128][SKC + 1];
  const int nt = blockIdx.x;
  const int mt = blockIdx.y >> 3, sub = blockIdx.y & 7;
  if (mt >= *a.num_mtiles) return;
  const int e = a.mtiles[2 * mt];
  const int row0 = a.mtiles[2 * mt + 1] + sub * SR;
  const int row_end = min(a.offsets[e + 1], (int)a.P);
  if (row0 >= row_end) return;
  const int tid = threadIdx.x, r = tid >> 4, cg = tid & 15;
  const int H = a.H, I = a.I, nH = H / kBlock, nI = I / kBlock;
  const int n0 = nt * 128;
  const int row = row0 + r;
  const bool rv = row < row_end;
  float accg[8], accu[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) accg[i] = accu[i] = 0.f;

  for (int kb = 0; kb < nH; ++kb) {
    float pg[8], pu[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) pg[i] = pu[i] = 0.f;
    float wsg = 1.f, wsu = 1.f;
    if (ACT == B200MOE_ACT_W8A16) {
      wsg = scale_at(a.s0, ((int64_t)e * nI + nt) * nH + kb, a.scale_dtype);
      wsu = scale_at(a.s1, ((int64_t)e * nI + nt) * nH + kb, a.scale_dtype);
    }
    for (int kc = 0; kc < kBlock / SKC; ++kc) {
      const int k0 = kb * kBlock + kc * SKC;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        int idx = tid + i * 256, rr = idx >> 5, kk = idx & 31, grow = row0 + rr;
        float v = 0.f;
        if (grow < row_end) {
          if (ACT == B200MOE_ACT_W8A8) {
            v = moe_e4m3_to_f32(a.aq[(int64_t)grow * H + k0 + kk]);
          } else {
            int64_t src = a.row_map ? a.row_map[grow] / a.div : grow;
            v = __bfloat162float(a.a16[src * H + k0 + kk]);
          }
        }
        sA[rr][kk] = v;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        int idx = tid + i * 256, n = idx >> 5, kk = idx & 31;
        int64_t off = ((int64_t)e * I + n0 + n) * H + k0 + kk;
        float g = moe_e4m3_to_f32(a.w0[off]), u = moe_e4m3_to_f32(a.w1[off]);
        if (ACT == B200MOE_ACT_W8A16) {
          g = moe_bf16_round(g * wsg);
          u = moe_bf16_round(u * wsu);
        }
        sG[n][kk] = g;
        sU[n][kk] = u;
      }
      __syncthreads();
#pragma unroll 8
      for (int kk = 0; kk < SKC; ++kk) {
        float av = sA[r][kk];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          pg[i] = fmaf(av, sG[cg + 16 * i][kk], pg[i]);
          pu[i] = fmaf(av, sU[cg + 16 * i][kk], pu[i]);
        }
      }
      __syncthreads();
    }
    if (ACT == B200MOE_ACT_W8A8) {
      float sa = rv ? a.as_t[(int64_t)kb * a.ld + row] : 0.f;
      float fg = sa * scale_at(a.s0, ((int64_t)e * nI + nt) * nH + kb, a.scale_dtype);
      float fu = sa * scale_at(a.s1, ((int64_t)e * nI + nt) * nH + kb, a.scale_dtype);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        accg[i] = fmaf(pg[i], fg, accg[i]);
        accu[i] = fmaf(pu[i], fu, accu[i]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        accg[i] += pg[i];
        accu[i] += pu[i];
      }
    }
  }

  if (ACT == B200MOE_ACT_W8A8) {
    float h[8], amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      h[i] = moe_silu(accg[i]) * accu[i];
      amax = fmaxf(amax, fabsf(h[i]));
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    amax = fmaxf(amax, kAmaxFloor);
    const float inv = kFp8Max / amax;
    if (rv) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        a.hq[(int64_t)row * I + n0 + cg + 16 * i] =
            (uint8_t)__nv_cvt_float_to_fp8(h[i] * inv, __NV_SATFINITE, __NV_E4M3);
      if (cg == 0) a.hs_t[(int64_t)nt * a.ld + row] = amax / kFp8Max;
    }
  } else if (rv) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float g = moe_bf16_round(accg[i]);
      float act = moe_bf16_round(moe_silu(g));
      float u = moe_bf16_round(accu[i]);
      a.h16[(int64_t)row * I + n0 + cg + 16 * i] = __float2bfloat16_rn(act * u);
    }
  }
}

template <int ACT>
__global__ void __launch_bounds__(256) gemm2_simple_kernel(MoeGemmArgs a) {
  __shared__ float sA[SR][SKC + 1];
  __shared__ float sB[SKC][128];
  const int nt = blockIdx.x;
  const int mt = blockIdx.y >> 3, sub = blockIdx.y & 7;
  if (mt >= *a.num_mtiles) return;
  const int e = a.mtiles[2 * mt];
  const int row0 = a.mtiles[2 * mt + 1] + sub * SR;
  const int row_end = min(a.offsets[e + 1], (int)a.P);
  if (row0 >= row_end) return;
  const int tid = threadIdx.x, r = tid >> 4, cg = tid & 15;
  const int H = a.H, I = a.I, nH = H / kBlock, nI = I / kBlock;
  const int n0 = nt * 128;
  const int row = row0 + r;
  const bool rv = row < row_end;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  for (int kb = 0; kb < nI; ++kb) {
    float p[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = 0.f;
    const float ws = scale_at(a.s0, ((int64_t)e * nI + kb) * nH + nt, a.scale_dtype);
    for (int kc = 0; kc < kBlock / SKC; ++kc) {
      const int k0 = kb * kBlock + kc * SKC;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        int idx = tid + i * 256, rr = idx >> 5, kk = idx & 31, grow = row0 + rr;
        float v = 0.f;
        if (grow < row_end) {
          if (ACT == B200MOE_ACT_W8A8) v = moe_e4m3_to_f32(a.aq[(int64_t)grow * I + k0 + kk]);
          else v = __bfloat162float(a.a16[(int64_t)grow * I + k0 + kk]);
        }
        sA[rr][kk] = v;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        int idx = tid + i * 256, kk = idx >> 7, n = idx & 127;
        float w = moe_e4m3_to_f32(a.w0[((int64_t)e * I + k0 + kk) * H + n0 + n]);
        if (ACT == B200MOE_ACT_W8A16) w = moe_bf16_round(w * ws);
        sB[kk][n] = w;
      }
      __syncthreads();
#pragma unroll 8
      for (int kk = 0; kk < SKC; ++kk) {
        float av = sA[r][kk];
#pragma unroll
        for (int i = 0; i < 8; ++i) p[i] = fmaf(av, sB[kk][cg + 16 * i], p[i]);
      }
      __syncthreads();
    }
    if (ACT == B200MOE_ACT_W8A8) {
      float f = (rv ? a.as_t[(int64_t)kb * a.ld + row] : 0.f) * ws;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(p[i], f, acc[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += p[i];
    }
  }
  if (rv) {
    const int64_t dst = a.row_map ? a.row_map[row] : row;
#pragma unroll
    for (int i = 0; i < 8; ++i) a.out[dst * H + n0 + cg + 16 * i] = __float2bfloat16_rn(acc[i]);
  }
}

__global__ void __launch_bounds__(1024)
build_mtiles_kernel(int32_t* __restrict__ mtiles, int32_t* __restrict__ num_mtiles,
                    const int32_t* __restrict__ offsets, int E, int max_rows, int max_mtiles) {
  __shared__ int tmp[1024];
  const int t = threadIdx.x;
  int b = 0, n = 0;
  if (t < E) {
    // rows at or past max_rows do not exist in the operand buffers (offsets that a caller computed for more rows
    // than the buffers hold are clipped here, and every kernel clips its row ranges the same way)
    b = min(offsets[t], max_rows);
    n = (min(offsets[t + 1], max_rows) - b + kTileM - 1) / kTileM;
  }
  tmp[t] = n;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {
    int v = t >= d ? tmp[t - d] : 0;
    __syncthreads();
    tmp[t] += v;
    __syncthreads();
  }
  const int base = tmp[t] - n;
  for (int i = 0; i < n && base + i < max_mtiles; ++i) {
    mtiles[2 * (base + i)] = t;
    mtiles[2 * (base + i) + 1] = b + i * kTileM;
  }
  if (t == 1023) *num_mtiles = min(tmp[1023], max_mtiles);
}

__global__ void identity_offsets_kernel(int32_t* offsets, int T) {
  offsets[0] = 0;
  offsets[1] = T;
}

// out[t,:] = bf16( sum_j w[t,j]*y[t,j,:] (+ add[t,:]) ); one thread per 8 columns (16-byte accesses)
__global__ void __launch_bounds__(256)
combine_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ y, const void* __restrict__ w,
               int w_dtype, const __nv_bfloat16* __restrict__ add, const int32_t* __restrict__ pos,
               const int32_t* __restrict__ ids, int E, int64_t T, int k, int H) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int hv = H / 8;
  if (idx >= T * hv) return;
  const int64_t t = idx / hv;
  const int c = (int)(idx % hv) * 8;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int j = 0; j < k; ++j) {
    const float wj = moe_load_as_f32(w, t * k + j, w_dtype);
    const int64_t yr = pos ? (int64_t)pos[t * k + j] : t * k + j;
    // a slot whose expert id was out of range has no result row (nothing ever wrote it): it contributes nothing
    if (yr < 0 || (ids && (ids[t * k + j] < 0 || ids[t * k + j] >= E))) continue;
    uint4 raw = *reinterpret_cast<const uint4*>(y + yr * H + c);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(b2[i]);
      acc[2 * i] = fmaf(wj, f.x, acc[2 * i]);
      acc[2 * i + 1] = fmaf(wj, f.y, acc[2 * i + 1]);
    }
  }
  if (add) {
    uint4 raw = *reinterpret_cast<const uint4*>(add + t * H + c);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(b2[i]);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
  uint4 o;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  *reinterpret_cast<uint4*>(out + t * H + c) = o;
}

}  // namespace

int moe_build_mtiles(int32_t* mtiles, int32_t* num_mtiles, const int32_t* offsets, int E, int64_t max_rows,
                     int max_mtiles, cudaStream_t st) {
  build_mtiles_kernel<<<1, 1024, 0, st>>>(mtiles, num_mtiles, offsets, E, (int)max_rows, max_mtiles);
  return moe_launch_status();
}

int moe_fill_identity_offsets(int32_t* offsets, int64_t T, cudaStream_t st) {
  identity_offsets_kernel<<<1, 1, 0, st>>>(offsets, (int)T);
  return moe_launch_status();
}

int moe_gemm1_simple(const MoeGemmArgs& a, int act_mode, cudaStream_t st) {
  dim3 grid((unsigned)(a.I / 128), (unsigned)(a.max_mtiles * 8));
  if (act_mode == B200MOE_ACT_W8A8) gemm1_simple_kernel<B200MOE_ACT_W8A8><<<grid, 256, 0, st>>>(a);
  else gemm1_simple_kernel<B200MOE_ACT_W8A16><<<grid, 256, 0, st>>>(a);
  return moe_launch_status();
}

int moe_gemm2_simple(const MoeGemmArgs& a, int act_mode, cudaStream_t st) {
  dim3 grid((unsigned)(a.H / 128), (unsigned)(a.max_mtiles * 8));
  if (act_mode == B200MOE_ACT_W8A8) gemm2_simple_kernel<B200MOE_ACT_W8A8><<<grid, 256, 0, st>>>(a);
  else gemm2_simple_kernel<B200MOE_ACT_W8A16><<<grid, 256, 0, st>>>(a);
  return moe_launch_status();
}

extern "C" int b200moe_combine_masked(void* out, const void* y, const int32_t* pos, const void* w, int w_dtype,
                                      const void* add, const int32_t* ids, int64_t E, int64_t T, int64_t k, int64_t H,
                                      void* stream) {
  MOE_CHECK_ARG(out && y && w && T >= 0 && k > 0 && H > 0 && (!ids || E > 0));
  MOE_CHECK_ARG(w_dtype == B200MOE_F32 || w_dtype == B200MOE_BF16 || w_dtype == B200MOE_F16);
  MOE_CHECK_SHAPE(H % 8 == 0);
  if (!moe_aligned16(out) || !moe_aligned16(y) || (add && !moe_aligned16(add))) return B200MOE_EALIGN;
  if (T == 0) return B200MOE_OK;
  const int64_t n = T * (H / 8);
  combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<__nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(y), w, w_dtype,
      reinterpret_cast<const __nv_bfloat16*>(add), pos, ids, (int)E, T, (int)k, (int)H);
  return moe_launch_status();
}

extern "C" int b200moe_combine_indexed(void* out, const void* y, const int32_t* pos, const void* w, int w_dtype,
                                       const void* add, int64_t T, int64_t k, int64_t H, void* stream) {
  return b200moe_combine_masked(out, y, pos, w, w_dtype, add, nullptr, 0, T, k, H, stream);
}

extern "C" int b200moe_combine(void* out, const void* y, const void* w, int w_dtype, const void* add, int64_t T,
                               int64_t k, int64_t H, void* stream) {
  return b200moe_combine_indexed(out, y, nullptr, w, w_dtype, add, T, k, H, stream);
}

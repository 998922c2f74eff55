// Shared device/host helpers of the fused-MoE kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200moe.h"

#define B200MOE_STATUS_BAD_EXPERT 1
#define B200MOE_STATUS_WAIT_TIMEOUT 2
#define B200MOE_STATUS_PEER_TIMEOUT 4
#define B200MOE_STATUS_PEER_OVERFLOW 8

constexpr int kBlock = 128;          // quantisation block (columns per activation scale, weight tile edge)
constexpr float kFp8Max = 448.0f;    // largest finite e4m3 value
constexpr float kAmaxFloor = 1e-12f; // floor of a group's max|x| before the scale is formed

#define MOE_CHECK_ARG(cond)            \
  do {                                 \
    if (!(cond)) return B200MOE_EINVAL; \
  } while (0)
#define MOE_CHECK_SHAPE(cond)          \
  do {                                 \
    if (!(cond)) return B200MOE_ESHAPE; \
  } while (0)

static inline int moe_launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? B200MOE_OK : (int)e;
}

static inline bool moe_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- scalar loads of score / scale tensors in their storage dtype -----------------------------
__device__ __forceinline__ float moe_load_as_f32(const void* p, int64_t i, int dtype) {
  if (dtype == B200MOE_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == B200MOE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void moe_store_from_f32(void* p, int64_t i, int dtype, float v) {
  if (dtype == B200MOE_F32) reinterpret_cast<float*>(p)[i] = v;
  else if (dtype == B200MOE_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}
// a + b rounded into `dtype` (what an add of two tensors of that dtype yields)
__device__ __forceinline__ float moe_add_in_dtype(float a, float b, int dtype) {
  float s = a + b;
  if (dtype == B200MOE_BF16) return __bfloat162float(__float2bfloat16_rn(s));
  if (dtype == B200MOE_F16) return __half2float(__float2half_rn(s));
  return s;
}

// ---- e4m3 conversion ---------------------------------------------------------------------------
__device__ __forceinline__ float moe_e4m3_to_f32(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(__half(h));
}
// two floats -> two e4m3 bytes (RNE, saturating to +-448); low byte = a
__device__ __forceinline__ uint16_t moe_f32x2_to_e4m3x2(float a, float b) {
  return __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ uint32_t moe_f32x4_to_e4m3x4(float a, float b, float c, float d) {
  return (uint32_t)moe_f32x2_to_e4m3x2(a, b) | ((uint32_t)moe_f32x2_to_e4m3x2(c, d) << 16);
}

__device__ __forceinline__ float moe_bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// SiLU in fp32: x * 1/(1+exp(-x))
__device__ __forceinline__ float moe_silu(float x) { return x / (1.0f + expf(-x)); }

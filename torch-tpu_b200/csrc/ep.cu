// Expert-parallel plumbing kernels: pack quantised rows for the dispatch all-to-all, unpack what was received into
// the layout the grouped GEMMs read, and the small index helpers around them.  The reference has no expert
// parallelism (its only MoE-adjacent collective is an equal-split all-to-all,
// torch_tpu/csrc/distributed/c10d/ProcessGroupSCCL.cpp:714-743); this is the path benchmark configurations with
// 2/4/8 GPUs ask for: experts sharded contiguously over ranks, tokens stay data-parallel.
//
// Packed row (what travels): [H bytes e4m3][H/128 fp32 scales][int32 expert id local to the destination][pad to 16 B].
#include "common.cuh"

namespace {

__host__ __device__ inline int64_t packed_row_bytes(int64_t H) {
  return (H + 4 * (H / kBlock) + 4 + 15) / 16 * 16;
}

// one warp per sorted row: gather the token row, quantise 1x128, write the packed row
__global__ void __launch_bounds__(256)
ep_pack_rows_kernel(uint8_t* __restrict__ rows, const __nv_bfloat16* __restrict__ x,
                    const int32_t* __restrict__ sorted_pair, const int32_t* __restrict__ ids, int k,
                    int experts_per_rank, int64_t P, int H, int64_t RB) {
  const int lane = threadIdx.x & 31;
  const int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (p >= P) return;
  const int pair = sorted_pair[p];
  if (pair < 0) return;  // position of a dropped pair (id out of range): nothing to pack
  const __nv_bfloat16* xr = x + (int64_t)(pair / k) * H;
  uint8_t* out = rows + p * RB;
  float* sc = reinterpret_cast<float*>(out + H);
  for (int c0 = 0; c0 < H; c0 += 256) {
    const int c = c0 + lane * 8;
    float v[8];
    float amax = 0.f;
    if (c < H) {
      uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(b2[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (c < H) {
      amax = fmaxf(amax, kAmaxFloor);
      const float inv = kFp8Max / amax;
      uint2 o2;
      o2.x = moe_f32x4_to_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
      o2.y = moe_f32x4_to_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
      *reinterpret_cast<uint2*>(out + c) = o2;
      if ((lane & 15) == 0) sc[c >> 7] = amax / kFp8Max;
    }
  }
  if (lane == 0) *reinterpret_cast<int32_t*>(out + H + 4 * (H / kBlock)) = ids[pair] % experts_per_rank;
}

__global__ void ep_unpack_ids_kernel(int32_t* __restrict__ eid, const uint8_t* __restrict__ rows, int64_t R, int H,
                                     int64_t RB) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r < R) eid[r] = *reinterpret_cast<const int32_t*>(rows + r * RB + H + 4 * (H / kBlock));
}

// one warp per destination row p: source row order[p]; bytes -> xq[p,:], scales -> xs_t[g, p]
__global__ void __launch_bounds__(256)
ep_unpack_rows_kernel(uint8_t* __restrict__ xq, float* __restrict__ xs_t, int64_t ld,
                      const uint8_t* __restrict__ rows, const int32_t* __restrict__ order, int64_t R, int H,
                      int64_t RB) {
  const int lane = threadIdx.x & 31;
  const int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (p >= R || order[p] < 0) return;  // -1: position of a row whose expert id was out of range
  const uint8_t* src = rows + (int64_t)order[p] * RB;
  for (int c = lane * 16; c < H; c += 512)
    *reinterpret_cast<uint4*>(xq + p * H + c) = *reinterpret_cast<const uint4*>(src + c);
  const float* sc = reinterpret_cast<const float*>(src + H);
  for (int g = lane; g < H / kBlock; g += 32) xs_t[(int64_t)g * ld + p] = sc[g];
}

__global__ void invert_permutation_kernel(int32_t* __restrict__ inv, const int32_t* __restrict__ perm, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && perm[i] >= 0 && perm[i] < n) inv[perm[i]] = (int32_t)i;
}

}  // namespace

extern "C" int64_t b200moe_ep_packed_row_bytes(int64_t H) { return H > 0 && H % kBlock == 0 ? packed_row_bytes(H) : 0; }

extern "C" int b200moe_ep_pack_rows(uint8_t* rows, const void* x, const int32_t* sorted_pair, const int32_t* ids,
                                    int64_t T, int64_t k, int64_t experts_per_rank, int64_t H, void* stream) {
  MOE_CHECK_ARG(rows && x && sorted_pair && ids && T >= 0 && k > 0 && experts_per_rank > 0 && H > 0);
  MOE_CHECK_SHAPE(H % kBlock == 0);
  if (!moe_aligned16(rows) || !moe_aligned16(x)) return B200MOE_EALIGN;
  const int64_t P = T * k;
  if (P == 0) return B200MOE_OK;
  ep_pack_rows_kernel<<<(unsigned)((P + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      rows, reinterpret_cast<const __nv_bfloat16*>(x), sorted_pair, ids, (int)k, (int)experts_per_rank, P, (int)H,
      packed_row_bytes(H));
  return moe_launch_status();
}

extern "C" int b200moe_ep_unpack_ids(int32_t* eid, const uint8_t* rows, int64_t R, int64_t H, void* stream) {
  MOE_CHECK_ARG(eid && rows && R >= 0 && H > 0);
  MOE_CHECK_SHAPE(H % kBlock == 0);
  if (R == 0) return B200MOE_OK;
  ep_unpack_ids_kernel<<<(unsigned)((R + 255) / 256), 256, 0, (cudaStream_t)stream>>>(eid, rows, R, (int)H,
                                                                                     packed_row_bytes(H));
  return moe_launch_status();
}

extern "C" int b200moe_ep_unpack_rows(uint8_t* xq, float* xs_t, int64_t ld, const uint8_t* rows, const int32_t* order,
                                      int64_t R, int64_t H, void* stream) {
  MOE_CHECK_ARG(xq && xs_t && rows && order && R >= 0 && H > 0 && ld >= R);
  MOE_CHECK_SHAPE(H % kBlock == 0);
  if (!moe_aligned16(xq) || !moe_aligned16(rows)) return B200MOE_EALIGN;
  if (R == 0) return B200MOE_OK;
  ep_unpack_rows_kernel<<<(unsigned)((R + 7) / 8), 256, 0, (cudaStream_t)stream>>>(xq, xs_t, ld, rows, order, R, (int)H,
                                                                                  packed_row_bytes(H));
  return moe_launch_status();
}

extern "C" int b200moe_invert_permutation(int32_t* inv, const int32_t* perm, int64_t n, void* stream) {
  MOE_CHECK_ARG(inv && perm && n >= 0);
  if (n == 0) return B200MOE_OK;
  // entries that no perm[i] names (perm carries -1 for dropped pairs) stay -1
  cudaMemsetAsync(inv, 0xFF, (size_t)n * sizeof(int32_t), (cudaStream_t)stream);
  invert_permutation_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(inv, perm, n);
  return moe_launch_status();
}

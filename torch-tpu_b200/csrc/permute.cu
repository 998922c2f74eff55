// Token permutation: a STABLE counting sort of the T*k (token,slot) pairs by expert id, the tile list
// that the grouped GEMMs walk, and the row gather + 1x128 e4m3 activation quantisation.
//
// The sort reproduces the reference device kernel's per-expert `nonzero` (my_ops/fusedMoE.pl:737-755):
// inside one expert the flat pair ids t*k+j ascend.  It is deterministic (no atomics decide order):
//   hist    : chunk c (1024 pairs) counts its pairs per expert            -> chunk_cnt[c][e]
//   scan    : per expert a running sum over chunks, then a scan over experts -> chunk_base, offsets
//   scatter : position = offsets[e] + chunk_base[c][e] + (pairs of e in earlier warps of the chunk)
//             + (pairs of e in lower lanes of the warp)
// For P <= 1024 all three steps run in one single-CTA kernel.
#include "common.cuh"

namespace {

constexpr int kChunk = 1024;  // pairs per CTA (32 warps)
constexpr int kMaxE = 1024;
constexpr int kRowsPerTile = 128;  // rows of one m-tile of the grouped GEMMs
constexpr int kMaxDevices = 64;  // per-device caches below are indexed by the CUDA device ordinal

// Per-warp histogram of this chunk in shared memory: wh[w*E + e].  Returns the pair's expert (or -1)
// and its rank among equal experts in lower lanes of its warp.
__device__ __forceinline__ int chunk_hist(const int32_t* __restrict__ ids, int64_t P, int E, int64_t p,
                                          int* wh, int& rank_in_warp, int32_t* status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) wh[i] = 0;
  __syncthreads();
  int e = -1;
  if (p < P) {
    e = ids[p];
    if (e < 0 || e >= E) {
      e = -1;
      if (status) atomicOr(status, B200MOE_STATUS_BAD_EXPERT);
    }
  }
  unsigned peers = __match_any_sync(0xffffffffu, e);
  rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank_in_warp == 0) wh[warp * E + e] = __popc(peers);
  __syncthreads();
  return e;
}

__global__ void __launch_bounds__(kChunk)
permute_hist_kernel(const int32_t* __restrict__ ids, int64_t P, int E, int32_t* __restrict__ chunk_cnt,
                    int32_t* status) {
  extern __shared__ int wh[];
  int rank;
  chunk_hist(ids, P, E, (int64_t)blockIdx.x * kChunk + threadIdx.x, wh, rank, status);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int s = 0;
#pragma unroll 8
    for (int w = 0; w < 32; ++w) s += wh[w * E + e];
    chunk_cnt[(int64_t)blockIdx.x * E + e] = s;
  }
}

// exclusive scan of cnt[0..E) by one CTA of 1024 threads (E <= 1024); result in offs[0..E], smem tmp[1024]
__device__ __forceinline__ void block_exclusive_scan(int my, int E, int32_t* __restrict__ offs, int* tmp) {
  const int t = threadIdx.x;
  tmp[t] = t < E ? my : 0;
  __syncthreads();
  for (int d = 1; d < kChunk; d <<= 1) {
    int v = t >= d ? tmp[t - d] : 0;
    __syncthreads();
    tmp[t] += v;
    __syncthreads();
  }
  if (t < E) offs[t + 1] = tmp[t];
  if (t == 0) offs[0] = 0;
}

__global__ void __launch_bounds__(kChunk)
permute_scan_kernel(int32_t* __restrict__ chunk_cnt, int nchunks, int E, int32_t* __restrict__ offsets) {
  __shared__ int tmp[kChunk];
  int total = 0;
  if ((int)threadIdx.x < E) {
    // eight counts are requested before the first is used: walked one by one, every chunk costs an L2 round trip
    // (64 chunks of a 65536-pair batch: 20 us for this one block)
    for (int c0 = 0; c0 < nchunks; c0 += 8) {
      int v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = c0 + i < nchunks ? chunk_cnt[(int64_t)(c0 + i) * E + threadIdx.x] : 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (c0 + i < nchunks) chunk_cnt[(int64_t)(c0 + i) * E + threadIdx.x] = total;  // becomes chunk_base
        total += v[i];
      }
    }
  }
  block_exclusive_scan(total, E, offsets, tmp);
}

__global__ void __launch_bounds__(kChunk)
permute_scatter_kernel(const int32_t* __restrict__ ids, int64_t P, int E,
                       const int32_t* __restrict__ chunk_base, const int32_t* __restrict__ offsets,
                       int32_t* __restrict__ sorted_pair) {
  extern __shared__ int wh[];
  int rank;
  const int64_t p = (int64_t)blockIdx.x * kChunk + threadIdx.x;
  int e = chunk_hist(ids, P, E, p, wh, rank, nullptr);
  for (int x = threadIdx.x; x < E; x += blockDim.x) {  // warp histogram -> exclusive prefix over warps
    int s = 0;
#pragma unroll 8
    for (int w = 0; w < 32; ++w) {
      int v = wh[w * E + x];
      wh[w * E + x] = s;
      s += v;
    }
  }
  __syncthreads();
  if (e >= 0) {
    int pos = offsets[e] + chunk_base[(int64_t)blockIdx.x * E + e] + wh[(threadIdx.x >> 5) * E + e] + rank;
    sorted_pair[pos] = (int32_t)p;
  }
  // Pairs whose id was out of range have no position: the tail [offsets[E], P) is filled with -1 so that no consumer
  // ever indexes with an unwritten entry (valid positions all lie below offsets[E], so this does not race with them).
  if (p < P && p >= offsets[E]) sorted_pair[p] = -1;
}

// P <= 1024: histogram, scan and scatter in one CTA
__global__ void __launch_bounds__(kChunk)
permute_small_kernel(const int32_t* __restrict__ ids, int64_t P, int E, int32_t* __restrict__ offsets,
                     int32_t* __restrict__ sorted_pair, int32_t* status, int32_t* __restrict__ mtiles,
                     int32_t* __restrict__ num_mtiles, int max_mtiles) {
  extern __shared__ int wh[];
  __shared__ int tmp[kChunk];
  __shared__ int soffs[kMaxE + 1];
  int rank;
  int e = chunk_hist(ids, P, E, threadIdx.x, wh, rank, status);
  int total = 0;
  if ((int)threadIdx.x < E) {
#pragma unroll 8
    for (int w = 0; w < 32; ++w) {
      int v = wh[w * E + threadIdx.x];
      wh[w * E + threadIdx.x] = total;
      total += v;
    }
  }
  block_exclusive_scan(total, E, soffs, tmp);
  __syncthreads();
  for (int i = threadIdx.x; i <= E; i += blockDim.x) offsets[i] = soffs[i];
  if (e >= 0) sorted_pair[soffs[e] + wh[(threadIdx.x >> 5) * E + e] + rank] = (int32_t)threadIdx.x;
  if ((int64_t)threadIdx.x < P && (int)threadIdx.x >= soffs[E]) sorted_pair[threadIdx.x] = -1;  // dropped pairs: see above
  if (mtiles) {
    // the m-tile list of the grouped GEMMs ({expert, first row} per 128 rows of an expert) from the same offsets:
    // one launch less on the decode path
    __syncthreads();
    const int t = threadIdx.x;
    const int b = t < E ? soffs[t] : 0;
    const int n = t < E ? (soffs[t + 1] - b + kRowsPerTile - 1) / kRowsPerTile : 0;
    __shared__ int toffs[kMaxE + 1];
    block_exclusive_scan(n, E, toffs, tmp);
    __syncthreads();
    for (int i = 0; i < n && toffs[t] + i < max_mtiles; ++i) {
      mtiles[2 * (toffs[t] + i)] = t;
      mtiles[2 * (toffs[t] + i) + 1] = b + i * kRowsPerTile;
    }
    if (t == 0) *num_mtiles = min(toffs[E], max_mtiles);
  }
}

__global__ void gather_scatter_index_kernel(int32_t* __restrict__ gather_index,
                                            int32_t* __restrict__ scatter_index,
                                            int32_t* __restrict__ num_per_expert,
                                            const int32_t* __restrict__ sorted_pair,
                                            const int32_t* __restrict__ offsets, int64_t T, int k) {
  const int e = blockIdx.x;
  const int b = offsets[e], n = offsets[e + 1] - b;
  if (threadIdx.x == 0) num_per_expert[e] = n;
  for (int i = threadIdx.x; i < n && i < T; i += blockDim.x) {
    int pr = sorted_pair[b + i];
    scatter_index[(int64_t)e * T + i] = pr;
    gather_index[(int64_t)e * T + i] = pr / k;
  }
}

// ---- row gather + 1x128 e4m3 quantisation -------------------------------------------------------
// A warp owns `cpw` consecutive 256-column chunks of one output row: a lane owns 8 consecutive bf16 (one 16-byte
// load), 16 lanes own one 128-column group.  The groups of a row are independent, so with few rows (decode sizes)
// they are spread over warps (cpw = 1: the kernel is one load-and-store deep instead of H/256); with many rows one
// warp walks a whole row (fewer blocks, the row's gather index read once).
__global__ void __launch_bounds__(256)
quant_rows_kernel(uint8_t* __restrict__ q, float* __restrict__ s_t, int64_t ld,
                  const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ row_map, int div,
                  int64_t rows, int H, int cpw, int warps_per_row) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t r = w / warps_per_row;
  if (r >= rows) return;
  const int c_begin = (int)(w - r * warps_per_row) * cpw * 256;
  if (row_map && row_map[r] < 0) return;  // position of a dropped pair (id out of range): no row
  const int64_t src = row_map ? (int64_t)(row_map[r] / div) : r;
  const __nv_bfloat16* xr = x + src * H;
  const int c_end = min(c_begin + cpw * 256, H);
  // Four 256-column chunks at a time, their loads issued before the first is used: taken one by one, every chunk of a
  // row costs the warp a whole round trip to L2 (Qwen3 shape, 65536 rows of 2048: 73 us for 400 MB).
  for (int c0 = c_begin; c0 < c_end; c0 += 4 * 256) {
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * 256 + lane * 8;
      raw[u] = c < c_end ? *reinterpret_cast<const uint4*>(xr + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * 256 + lane * 8;
      if (c0 + u * 256 >= c_end) break;  // uniform over the warp
      float v[8];
      float amax = 0.f;
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(b2[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (c < c_end) {
        amax = fmaxf(amax, kAmaxFloor);
        const float inv = kFp8Max / amax;
        uint2 out;
        out.x = moe_f32x4_to_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
        out.y = moe_f32x4_to_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
        *reinterpret_cast<uint2*>(q + r * H + c) = out;
        if ((lane & 15) == 0) s_t[(int64_t)(c >> 7) * ld + r] = amax / kFp8Max;
      }
    }
  }
}

}  // namespace

extern "C" size_t b200moe_permute_scratch_ints(int64_t P, int64_t E) {
  if (P <= kChunk) return 1;
  return (size_t)((P + kChunk - 1) / kChunk) * (size_t)E;
}

// b200moe_permute; with `mtiles` != NULL and at most 1024 pairs the one-CTA kernel writes the GEMMs' m-tile list too and
// *tiles_done is set (else the caller builds the list from expert_offsets)
int moe_permute_impl(int32_t* sorted_pair, int32_t* expert_offsets, const int32_t* ids, int64_t T, int64_t k, int64_t E,
                     int32_t* scratch, int32_t* status, int32_t* mtiles, int32_t* num_mtiles, int max_mtiles,
                     bool* tiles_done, void* stream) {
  if (tiles_done) *tiles_done = false;
  MOE_CHECK_ARG(sorted_pair && expert_offsets && ids && T >= 0 && k > 0 && E > 0);
  const int64_t P = T * k;
  MOE_CHECK_SHAPE(E <= kMaxE && P < (1 << 24));
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)32 * E * sizeof(int);
  // The dynamic shared-memory cap of a kernel is a per-DEVICE attribute: set it once on every device that comes here.
  static bool attr_done[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200MOE_EDRIVER;
  if (!attr_done[dev]) {
    cudaFuncSetAttribute(permute_hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * kMaxE * 4);
    cudaFuncSetAttribute(permute_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * kMaxE * 4);
    cudaFuncSetAttribute(permute_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * kMaxE * 4);
    attr_done[dev] = true;
  }
  if (P <= kChunk) {
    permute_small_kernel<<<1, kChunk, smem, st>>>(ids, P, (int)E, expert_offsets, sorted_pair, status, mtiles,
                                                  num_mtiles, max_mtiles);
    if (tiles_done) *tiles_done = mtiles != nullptr;
    return moe_launch_status();
  }
  MOE_CHECK_ARG(scratch);
  const int nchunks = (int)((P + kChunk - 1) / kChunk);
  permute_hist_kernel<<<nchunks, kChunk, smem, st>>>(ids, P, (int)E, scratch, status);
  permute_scan_kernel<<<1, kChunk, 0, st>>>(scratch, nchunks, (int)E, expert_offsets);
  permute_scatter_kernel<<<nchunks, kChunk, smem, st>>>(ids, P, (int)E, scratch, expert_offsets, sorted_pair);
  return moe_launch_status();
}

extern "C" int b200moe_permute(int32_t* sorted_pair, int32_t* expert_offsets, const int32_t* ids, int64_t T,
                               int64_t k, int64_t E, int32_t* scratch, int32_t* status, void* stream) {
  return moe_permute_impl(sorted_pair, expert_offsets, ids, T, k, E, scratch, status, nullptr, nullptr, 0, nullptr,
                          stream);
}

extern "C" int b200moe_gather_scatter_index(int32_t* gather_index, int32_t* scatter_index,
                                            int32_t* num_per_expert, const int32_t* sorted_pair,
                                            const int32_t* expert_offsets, int64_t T, int64_t k, int64_t E,
                                            void* stream) {
  MOE_CHECK_ARG(gather_index && scatter_index && num_per_expert && sorted_pair && expert_offsets);
  MOE_CHECK_ARG(T >= 0 && k > 0 && E > 0);
  if (T == 0) return B200MOE_OK;
  gather_scatter_index_kernel<<<(unsigned)E, 256, 0, (cudaStream_t)stream>>>(
      gather_index, scatter_index, num_per_expert, sorted_pair, expert_offsets, T, (int)k);
  return moe_launch_status();
}

extern "C" int b200moe_quant_rows(uint8_t* q, float* s_t, int64_t ld, const void* x, const int32_t* row_map,
                                  int64_t div, int64_t rows, int64_t H, void* stream) {
  MOE_CHECK_ARG(q && s_t && x && rows >= 0 && H > 0 && div > 0 && ld >= rows);
  MOE_CHECK_SHAPE(H % kBlock == 0);
  if (!moe_aligned16(x) || !moe_aligned16(q)) return B200MOE_EALIGN;
  if (rows == 0) return B200MOE_OK;
  const int chunks = (int)((H + 255) / 256);
  const int cpw = rows >= 2048 ? chunks : 1;
  const int warps_per_row = (chunks + cpw - 1) / cpw;
  quant_rows_kernel<<<(unsigned)((rows * warps_per_row + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      q, s_t, ld, reinterpret_cast<const __nv_bfloat16*>(x), row_map, (int)div, rows, (int)H, cpw, warps_per_row);
  return moe_launch_status();
}

// ---- permutation without caller-provided scratch ---------------------------------------------------
// For hosts that must not (or cannot) allocate device memory around the call - a serving process whose
// memory pool is fixed at start-up, a plugin that is only handed input and output buffers.  The chunk-count table that b200moe_permute takes from the caller lives here in
// a fixed array inside the library image instead; every GPU that loads the library holds these 256 KB until
// the process exits.
constexpr size_t kStaticScratchInts = 64 * 1024;  // 256 KB: e.g. 65536 pairs x 1024 experts, 262144 pairs x 256
static __device__ __align__(256) int32_t g_permute_scratch[kStaticScratchInts];

namespace {
// In host code `g_permute_scratch` is only a handle for the runtime, not a device address, so the address the
// kernels need is looked up once per device, with that device current.
int static_scratch_ptr(int32_t** out) {
  static int32_t* ptrs[kMaxDevices] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return B200MOE_ESHAPE;
  if (!ptrs[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_permute_scratch);
    if (e != cudaSuccess) return (int)e;
    ptrs[dev] = reinterpret_cast<int32_t*>(p);
  }
  *out = ptrs[dev];
  return B200MOE_OK;
}
}  // namespace

extern "C" size_t b200moe_permute_static_max_scratch_ints(void) { return kStaticScratchInts; }

extern "C" int b200moe_permute_static(int32_t* sorted_pair, int32_t* expert_offsets, const int32_t* ids,
                                      int64_t T, int64_t k, int64_t E, int32_t* status, void* stream) {
  MOE_CHECK_ARG(T >= 0 && k > 0 && E > 0);
  if (b200moe_permute_scratch_ints(T * k, E) > kStaticScratchInts) return B200MOE_ESHAPE;
  int32_t* scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);
  if (rc != B200MOE_OK) return rc;
  // The table is written in full by the histogram step before it is read, so nothing has to be cleared.
  return b200moe_permute(sorted_pair, expert_offsets, ids, T, k, E, scratch, status, stream);
}

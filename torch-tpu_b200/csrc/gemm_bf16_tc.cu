// The reference's own arithmetic (W8A16) on the sm_100a tensor cores: bf16 activations x FP8 weights that are
// dequantised block-wise to bf16 IN SHARED MEMORY, tcgen05.mma kind::f16 with fp32 accumulation in tensor memory over
// the whole K range, every intermediate rounded to bf16 where the reference rounds it.
//
//   gemm1  g = bf16(x Wg'^T), u = bf16(x Wu'^T), h = bf16(bf16(SiLU(g)) * u)   with W' = bf16(f32(Wq) * scale)
//          (my_ops/fusedMoE.pl:11-34 weight_dequant_bc + :217-259; CPU statement order of
//          python/regression/test_llm/test_moe.py:63-84)
//   gemm2  y = bf16(h Wd')                                                      (my_ops/fusedMoE.pl:264-269)
//
// Because the block scale is applied to the B operand BEFORE the product, a tile accumulates over all of K in tensor
// memory and is read back once (no per-K-block promotion as in the FP8 x FP8 kernels).  One persistent CTA per SM,
// 16 warps:
//   warp 0      TMA producer: per 64-deep K step the A tile (128 rows x 64 bf16, 128-byte swizzle) and the raw FP8
//               weight tile (gemm1: 128 gate + 128 up rows x 64 B; gemm2: 64 K rows x 256 B), 4-stage ring
//   warp 1      MMA issuer (one thread) and tensor-memory owner: 4 x (M128 N256 K16) per K step
//   warps 4-11  dequantisation: raw FP8 tile -> fp32 * scale -> bf16, written in the swizzled operand layout the MMA
//               reads (K-major for gemm1, MN-major for gemm2: weights keep the reference layout [E,I,H]), 2 slots
//   warps 12-15 epilogue: one 256-column accumulator per tile, read once (two tensor-memory buffers: the epilogue of a
//               tile overlaps the main loop of the next)
// With bf16 weights (the reference op called with scales = None, python/test/fused_moe_bf16.py:113-122) there is
// nothing to dequantise: the producer loads the operand tile itself (4 stages of A + B) and warps 4-11 stay idle.
// No multicast loads.  Every wait is bounded; on a time-out status bit 1 is raised and all roles leave together.
#include "tc_ptx.cuh"

namespace {

constexpr int BT_THREADS = 512;
constexpr int BT_STAGES = 4;                  // ring of A + raw weight tiles
constexpr int BT_BK = 64;                     // K elements per step (128 bytes of bf16)
constexpr int BT_A_BYTES = 128 * BT_BK * 2;   // 16 KB
constexpr int BT_RAW_BYTES = 256 * BT_BK;     // 16 KB of e4m3
constexpr int BT_STAGE_BYTES = BT_A_BYTES + BT_RAW_BYTES;
constexpr int BT_B_BYTES = 256 * BT_BK * 2;   // 32 KB: the dequantised operand tile
constexpr int BT_BSLOTS = 2;
constexpr int BT_DEQ_WARPS = 8, BT_EPI_WARPS = 4;
constexpr int BT_WSTAGE_BYTES = BT_A_BYTES + BT_B_BYTES;  // bf16 weights: a stage is A + the operand tile (48 KB)
static_assert(BT_STAGES * BT_WSTAGE_BYTES <= BT_STAGES * (BT_A_BYTES + BT_RAW_BYTES) + BT_BSLOTS * BT_B_BYTES,
              "the bf16-weight ring must fit the space of the two rings it replaces");

struct BtShared {
  uint64_t full[BT_STAGES];    // TMA bytes of the stage have landed
  uint64_t empty[BT_STAGES];   // the MMAs that read the stage (and its operand slot) are complete
  uint64_t bfull[BT_BSLOTS];   // the dequantised operand tile of the slot is written
  uint64_t tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  alignas(16) uint8_t ostage[4][32 * 128];  // per epilogue warp: 32 rows x 128 B of results on their way to row stores
};
constexpr size_t BT_SMEM_BYTES =
    1024 + (size_t)BT_STAGES * BT_STAGE_BYTES + (size_t)BT_BSLOTS * BT_B_BYTES + sizeof(BtShared);
static_assert(BT_SMEM_BYTES <= 232448, "more than the 227 KB of shared memory a CTA can have");

struct BtArgs {
  const void* s0;            // weight scales: gemm1 gate [E,nI,nH]; gemm2 down [E,nI,nH]
  const void* s1;            // gemm1 up
  int scale_dtype;
  const int32_t* mtiles;
  const int32_t* num_mtiles;
  const int32_t* offsets;
  const int32_t* row_map;    // gemm2: destination row of sorted row r (NULL = r)
  int H, I, NT, m_major;
  int P;                     // rows the operand buffers hold: row ranges are clipped to it
  int bf16w;                 // weights are bf16 [E,I,H] (no scales): B tiles come straight from global memory
  __nv_bfloat16* out;        // gemm1: h [P,I]; gemm2: y rows of H
  int32_t* status;
};

// kind::f16, bf16 x bf16 -> fp32, M = 128, N = 256
__host__ __device__ constexpr uint32_t bt_idesc(int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 16 e4m3 bytes -> 16 bf16 of bf16(f32(w) * scale): the reference's weight_dequant, one rounding
__device__ __forceinline__ void dequant16(const uint4& raw, float scale, uint4& lo, uint4& hi) {
  const uint16_t* p = reinterpret_cast<const uint16_t*>(&raw);
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(p[i], __NV_E4M3);
    const float2 f = __half22float2(__half2(h2));
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x * scale, f.y * scale);
    o[i] = *reinterpret_cast<const uint32_t*>(&b);
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

template <bool GEMM2>
__global__ void __launch_bounds__(BT_THREADS, 1)
moe_gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                        const __grid_constant__ CUtensorMap tmB1, const BtArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bslots = smem + (size_t)BT_STAGES * BT_STAGE_BYTES;
  BtShared* sh = reinterpret_cast<BtShared*>(bslots + (size_t)BT_BSLOTS * BT_B_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem), bslot_base = smem_u32(bslots);
  volatile int* abort_flag = &sh->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < BT_STAGES; ++s) {
      mbar_init(smem_u32(&sh->full[s]), 1);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->bfull[b]), BT_DEQ_WARPS);
      mbar_init(smem_u32(&sh->tmem_full[b]), 1);
      mbar_init(smem_u32(&sh->tmem_empty[b]), BT_EPI_WARPS);
    }
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  const int num_mtiles = *a.num_mtiles;
  const int total_tiles = num_mtiles * a.NT;
  const int K = GEMM2 ? a.I : a.H;
  const int KS = K / BT_BK;  // K steps of a tile
  const int nH = a.H / kBlock, nI = a.I / kBlock;
  auto tile_of = [&](int t, int& nt, int& mt) {
    nt = a.m_major ? t % a.NT : t / num_mtiles;
    mt = a.m_major ? t / a.NT : t - nt * num_mtiles;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (one thread)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int nt, mt;
        tile_of(t, nt, mt);
        const int e = a.mtiles[2 * mt], row0 = a.mtiles[2 * mt + 1];
        for (int ks = 0; ks < KS; ++ks, ++it) {
          const int s = it % BT_STAGES;
          if (!mbar_wait(smem_u32(&sh->empty[s]), ((it / BT_STAGES) & 1) ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&sh->full[s]);
          if (a.bf16w) {  // A + the bf16 operand tile itself: [A 16 KB | B 32 KB] per stage
            const uint32_t sa = smem_base + s * BT_WSTAGE_BYTES, sb = sa + BT_A_BYTES;
            mbar_arrive_expect_tx(full, BT_WSTAGE_BYTES);
            tma_load_2d(sa, &tmA, ks * BT_BK, row0, full);
            if (!GEMM2) {
              tma_load_2d(sb, &tmB0, ks * BT_BK, e * a.I + nt * 128, full);                // gate rows, K-major
              tma_load_2d(sb + 128 * 128, &tmB1, ks * BT_BK, e * a.I + nt * 128, full);    // up rows
            } else {
#pragma unroll
              for (int cn = 0; cn < 4; ++cn)  // four 64-column chunks of (64 K rows x 128 B), MN-major
                tma_load_2d(sb + cn * (64 * 128), &tmB0, nt * 256 + cn * 64, e * a.I + ks * BT_BK, full);
            }
            continue;
          }
          const uint32_t sa = smem_base + s * BT_STAGE_BYTES, sr = sa + BT_A_BYTES;
          mbar_arrive_expect_tx(full, BT_STAGE_BYTES);
          tma_load_2d(sa, &tmA, ks * BT_BK, row0, full);  // bf16 elements
          if (!GEMM2) {
            tma_load_2d(sr, &tmB0, ks * BT_BK, e * a.I + nt * 128, full);             // gate rows
            tma_load_2d(sr + 128 * BT_BK, &tmB1, ks * BT_BK, e * a.I + nt * 128, full);  // up rows
          } else {
            tma_load_2d(sr, &tmB0, nt * 256, e * a.I + ks * BT_BK, full);  // 64 K rows x 256 columns of H
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t idesc = bt_idesc(GEMM2 ? 1 : 0);
      const uint64_t adesc0 = make_smem_desc(smem_base, 16, 1024);
      // gemm1: K-major, 256 rows of 128 B; gemm2: MN-major, four 64-column chunks of (64 K rows x 128 B) = 8 KB each
      const uint64_t bdesc0 = GEMM2 ? make_smem_desc(bslot_base, 64 * 128, 1024) : make_smem_desc(bslot_base, 16, 1024);
      const uint64_t bdescw0 = GEMM2 ? make_smem_desc(smem_base + BT_A_BYTES, 64 * 128, 1024)
                                     : make_smem_desc(smem_base + BT_A_BYTES, 16, 1024);
      uint32_t it = 0, n = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++n) {
        const uint32_t buf = n & 1;
        if (!mbar_wait(smem_u32(&sh->tmem_empty[buf]), ((n >> 1) & 1) ^ 1, abort_flag)) break;
        const uint32_t d = tmem_base + buf * 256;
        for (int ks = 0; ks < KS; ++ks, ++it) {
          const uint32_t s = it % BT_STAGES, j = it % BT_BSLOTS;
          if (!mbar_wait(smem_u32(&sh->full[s]), (it / BT_STAGES) & 1, abort_flag) ||
              (!a.bf16w && !mbar_wait(smem_u32(&sh->bfull[j]), (it / BT_BSLOTS) & 1, abort_flag))) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = adesc0 + (uint64_t)(s * ((a.bf16w ? BT_WSTAGE_BYTES : BT_STAGE_BYTES) >> 4));
          const uint64_t bdesc = a.bf16w ? bdescw0 + (uint64_t)(s * (BT_WSTAGE_BYTES >> 4))
                                         : bdesc0 + (uint64_t)(j * (BT_B_BYTES >> 4));
#pragma unroll
          for (int k16 = 0; k16 < BT_BK / 16; ++k16) {
            // K advances 16 elements: +32 B inside the swizzle atom (K-major) or +16 rows of 128 B (MN-major)
            const uint64_t ad = adesc + (uint64_t)(k16 * 2);
            const uint64_t bd = bdesc + (uint64_t)(GEMM2 ? k16 * 128 : k16 * 2);
            tc_mma_bf16(d, ad, bd, idesc, (ks > 0 || k16 > 0) ? 1u : 0u);
          }
          tc_commit(smem_u32(&sh->empty[s]));  // stage and operand slot may be refilled
        }
        if (ok) tc_commit(smem_u32(&sh->tmem_full[buf]));  // the tile's accumulator is complete
      }
    }
  } else if (warp >= 4 && warp < 4 + BT_DEQ_WARPS) {
    // ------------------------------------------------------------------ dequantisation (8 warps)
    const int dt = threadIdx.x - 128;  // 0..255
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok && !a.bf16w; t += gridDim.x) {
      int nt, mt;
      tile_of(t, nt, mt);
      const int e = a.mtiles[2 * mt];
      for (int ks = 0; ks < KS; ++ks, ++it) {
        const int s = it % BT_STAGES, j = it % BT_BSLOTS;
        const int kb = (ks * BT_BK) / kBlock;  // 128-deep scale block of this step
        // block scales of this step: gemm1 one per operand half (gate, up); gemm2 one per 128 columns of H
        float sc0, sc1;
        if (!GEMM2) {
          const int64_t i0 = ((int64_t)e * nI + nt) * nH + kb;
          sc0 = moe_load_as_f32(a.s0, i0, a.scale_dtype);
          sc1 = moe_load_as_f32(a.s1, i0, a.scale_dtype);
        } else {
          const int64_t i0 = ((int64_t)e * nI + kb) * nH + 2 * nt;
          sc0 = moe_load_as_f32(a.s0, i0, a.scale_dtype);
          sc1 = (2 * nt + 1 < nH) ? moe_load_as_f32(a.s0, i0 + 1, a.scale_dtype) : 0.f;
        }
        if (!mbar_wait(smem_u32(&sh->full[s]), (it / BT_STAGES) & 1, abort_flag)) {
          ok = false;
          break;
        }
        // the slot is free once the MMAs of step it - 2 are complete: that is the commit that frees ring stage (it-2)%4
        if (it >= BT_BSLOTS &&
            !mbar_wait(smem_u32(&sh->empty[(it - BT_BSLOTS) % BT_STAGES]), ((it - BT_BSLOTS) / BT_STAGES) & 1, abort_flag)) {
          ok = false;
          break;
        }
        const uint8_t* raw = smem + (size_t)s * BT_STAGE_BYTES + BT_A_BYTES;
        uint8_t* dst = bslots + (size_t)j * BT_B_BYTES;
        if (!GEMM2) {
          // raw: 256 rows (n) x 64 B (k), row-major.  16-byte chunk q: row n = q / 4, bytes k = (q % 4) * 16 .. +16.
          // dest: K-major, 128-byte swizzle: row n at n * 128, 16-byte chunk c of the row stored at chunk c ^ (n % 8).
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int q = r * 256 + dt;
            const int n = q >> 2, c4 = q & 3;
            const uint4 v = *reinterpret_cast<const uint4*>(raw + q * 16);
            uint4 lo, hi;
            dequant16(v, n < 128 ? sc0 : sc1, lo, hi);
            uint8_t* row = dst + n * 128;
            *reinterpret_cast<uint4*>(row + (((2 * c4) ^ (n & 7)) << 4)) = lo;
            *reinterpret_cast<uint4*>(row + (((2 * c4 + 1) ^ (n & 7)) << 4)) = hi;
          }
        } else {
          // raw: 64 rows (k) x 256 B (n), row-major.  chunk q: k = q / 16, n = (q % 16) * 16 .. +16.
          // dest: MN-major: column chunk cn = n / 64 (8 KB each); inside it row k at k * 128, 16-byte chunk of 8 n.
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int q = r * 256 + dt;
            const int k = q >> 4, n16 = q & 15;
            const uint4 v = *reinterpret_cast<const uint4*>(raw + q * 16);
            uint4 lo, hi;
            dequant16(v, n16 < 8 ? sc0 : sc1, lo, hi);
            uint8_t* row = dst + (n16 >> 2) * (64 * 128) + k * 128;
            const int c = (n16 & 3) * 2;  // 16-byte chunk (8 bf16) inside the 64-column row
            *reinterpret_cast<uint4*>(row + ((c ^ (k & 7)) << 4)) = lo;
            *reinterpret_cast<uint4*>(row + (((c + 1) ^ (k & 7)) << 4)) = hi;
          }
        }
        // make the generic-proxy writes visible to the tensor core (async proxy), then hand the slot over
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh->bfull[j]));
      }
    }
  } else if (warp >= 4 + BT_DEQ_WARPS) {
    // ------------------------------------------------------------------ epilogue (4 warps, one lane quarter each)
    const int q = warp & 3;
    const int rit = q * 32 + lane;
    uint32_t n = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++n) {
      int nt, mt;
      tile_of(t, nt, mt);
      const int e = a.mtiles[2 * mt], row0 = a.mtiles[2 * mt + 1];
      const int row_end = min(a.offsets[e + 1], a.P);
      const int grow = row0 + rit;
      const bool valid = grow < row_end;
      const uint32_t buf = n & 1;
      if (!mbar_wait(smem_u32(&sh->tmem_full[buf]), (n >> 1) & 1, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t tb = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256;
      const bool warp_has_rows = row0 + q * 32 < row_end;
      if (warp_has_rows) {
        // Results leave through a warp-private patch of shared memory (16-byte chunks, XOR-swizzled by row): a thread
        // owns one row, so stores from registers would put 16 bytes into 32 different rows per instruction; from
        // the patch a warp stores four rows' whole 128-byte lines per instruction.
        uint4* wst = reinterpret_cast<uint4*>(sh->ostage[q]);
        const int OUTW = GEMM2 ? a.H : a.I;
        const int64_t dstrow = valid ? (GEMM2 && a.row_map ? a.row_map[grow] : grow) : 0;
        const unsigned long long my_dst =
            valid ? reinterpret_cast<unsigned long long>(a.out) + (unsigned long long)dstrow * OUTW * 2 : 0ull;
        auto store_patch = [&](int col0) {  // 64 columns from column col0 of the output rows
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + (lane >> 3), c8 = lane & 7;
            const unsigned long long dst = __shfl_sync(0xffffffffu, my_dst, r);
            const uint4 v = wst[r * 8 + (c8 ^ (r & 7))];
            if (dst) *reinterpret_cast<uint4*>(dst + (unsigned long long)(col0 + c8 * 8) * 2) = v;
          }
          __syncwarp();
        };
        if (!GEMM2) {
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t g[16], u[16];
            tc_ld_issue(tb + c * 16, g);
            tc_ld_issue(tb + 128 + c * 16, u);
            tc_ld_wait(g, u);
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float h2[2];
#pragma unroll
              for (int w = 0; w < 2; ++w) {
                const float gv = moe_bf16_round(__uint_as_float(g[2 * i + w]));   // out00 = bf16(x W0^T)
                const float av = moe_bf16_round(moe_silu(gv));                    // out0 = bf16(silu)
                const float uv = moe_bf16_round(__uint_as_float(u[2 * i + w]));   // out1 = bf16(x W1^T)
                h2[w] = av * uv;                                                  // out2, rounded below
              }
              const __nv_bfloat162 b = __floats2bfloat162_rn(h2[0], h2[1]);
              o[i] = *reinterpret_cast<const uint32_t*>(&b);
            }
            const int ch = (c & 3) * 2;  // 16-byte chunk of the 128-byte patch row
            wst[lane * 8 + (ch ^ (lane & 7))] = make_uint4(o[0], o[1], o[2], o[3]);
            wst[lane * 8 + ((ch + 1) ^ (lane & 7))] = make_uint4(o[4], o[5], o[6], o[7]);
            if ((c & 3) == 3) store_patch(nt * 128 + (c >> 2) * 64);
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < 16; c += 2) {
            uint32_t v0[16], v1[16];
            tc_ld_issue(tb + c * 16, v0);
            tc_ld_issue(tb + (c + 1) * 16, v1);
            tc_ld_wait(v0, v1);
            const int col0 = nt * 256 + (c >> 2) * 64;  // the 64-column round this pair of chunks belongs to
            if (col0 >= a.H) break;                     // uniform (the last n-tile may be narrower; H % 128 == 0)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const uint32_t(&v)[16] = half ? v1 : v0;
              uint32_t o[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                o[i] = *reinterpret_cast<const uint32_t*>(&b);
              }
              const int ch = ((c & 2) + half) * 2;
              wst[lane * 8 + (ch ^ (lane & 7))] = make_uint4(o[0], o[1], o[2], o[3]);
              wst[lane * 8 + ((ch + 1) ^ (lane & 7))] = make_uint4(o[4], o[5], o[6], o[7]);
            }
            if (c & 2) store_patch(col0);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->tmem_empty[buf]));
    }
  }

  // ---- teardown: every role arrives here, also after a time-out ---------------------------------------
  tc_fence_before();
  __syncthreads();
  if (sh->abort_flag) {
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, B200MOE_STATUS_WAIT_TIMEOUT);
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // copies and MMAs still in flight land before memory is released
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// row-major matrix of `es`-byte elements [rows, cols], box `bc` x `br` elements
bool bt_make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, int es, uint32_t bc, uint32_t br,
                 bool swizzle128) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (uint64_t)es};
  cuuint32_t box[2] = {bc, br};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, es == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base),
             dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool GEMM2>
int launch_bt(const MoeGemmArgs& g, cudaStream_t st) {
  const int K = GEMM2 ? g.I : g.H;
  if (K % BT_BK) return B200MOE_ESHAPE;
  CUtensorMap tmA, tmB0, tmB1;
  // A: bf16 rows, already in sorted order (gemm1: gathered x [P,H]; gemm2: h [P,I])
  if (!bt_make_map(&tmA, g.a16, (uint64_t)g.P, (uint64_t)K, 2, BT_BK, 128, true)) return B200MOE_EDRIVER;
  if (g.w_bf16) {  // bf16 weights: operand tiles straight from global memory, 128-byte swizzle
    const uint32_t br = GEMM2 ? BT_BK : 128;  // gemm1: 128 rows x 64 K elements; gemm2: 64 K rows x 64 columns
    if (!bt_make_map(&tmB0, g.w0, (uint64_t)g.E * g.I, (uint64_t)g.H, 2, 64, br, true)) return B200MOE_EDRIVER;
    if (!bt_make_map(&tmB1, GEMM2 ? g.w0 : g.w1, (uint64_t)g.E * g.I, (uint64_t)g.H, 2, 64, br, true)) return B200MOE_EDRIVER;
  } else if (!GEMM2) {
    if (!bt_make_map(&tmB0, g.w0, (uint64_t)g.E * g.I, (uint64_t)g.H, 1, BT_BK, 128, false)) return B200MOE_EDRIVER;
    if (!bt_make_map(&tmB1, g.w1, (uint64_t)g.E * g.I, (uint64_t)g.H, 1, BT_BK, 128, false)) return B200MOE_EDRIVER;
  } else {
    if (!bt_make_map(&tmB0, g.w0, (uint64_t)g.E * g.I, (uint64_t)g.H, 1, 256, BT_BK, false)) return B200MOE_EDRIVER;
    tmB1 = tmB0;
  }
  BtArgs a{};
  a.s0 = g.s0;
  a.s1 = g.s1;
  a.scale_dtype = g.scale_dtype;
  a.mtiles = g.mtiles;
  a.num_mtiles = g.num_mtiles;
  a.offsets = g.offsets;
  a.row_map = GEMM2 ? g.row_map : nullptr;
  a.H = g.H;
  a.I = g.I;
  a.P = (int)g.P;
  a.bf16w = g.w_bf16;
  a.NT = GEMM2 ? (g.H + 255) / 256 : g.I / 128;
  {
    const double a_bytes = (double)g.P * K * 2;
    const double w_expert = (double)(GEMM2 ? g.H : 2 * g.I) * K;
    a.m_major = (a_bytes > 48e6 && w_expert <= 64e6) ? 1 : 0;
  }
  a.out = GEMM2 ? g.out : g.h16;
  a.status = g.status;
  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200MOE_EDRIVER;
  if (!attr_set[dev]) {  // per-device attribute
    cudaFuncSetAttribute(moe_gemm_bf16_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BT_SMEM_BYTES);
    cudaFuncSetAttribute(moe_gemm_bf16_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BT_SMEM_BYTES);
    attr_set[dev] = true;
  }
  const long long max_tiles = (long long)g.max_mtiles * a.NT;
  const int sms = g.max_ctas > 0 && g.max_ctas < moe_device_sm_count() ? g.max_ctas : moe_device_sm_count();
  const int grid = (int)(max_tiles < sms ? max_tiles : sms);
  moe_gemm_bf16_tc_kernel<GEMM2><<<grid, BT_THREADS, BT_SMEM_BYTES, st>>>(tmA, tmB0, tmB1, a);
  return moe_launch_status();
}

// gather of bf16 rows into sorted order: dst[r,:] = x[row_map[r] / div, :] (16-byte accesses; one warp per row)
__global__ void __launch_bounds__(256)
gather_rows_bf16_kernel(__nv_bfloat16* __restrict__ dst, const __nv_bfloat16* __restrict__ x,
                        const int32_t* __restrict__ row_map, int div, int64_t rows, int H) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int pr = row_map ? row_map[r] : (int)r;
  if (pr < 0) return;  // position of a dropped pair
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)(pr / div) * H);
  uint4* d = reinterpret_cast<uint4*>(dst + r * H);
  for (int c = lane; c < H / 8; c += 32) d[c] = src[c];
}

}  // namespace

int moe_gather_rows_bf16(__nv_bfloat16* dst, const __nv_bfloat16* x, const int32_t* row_map, int div, int64_t rows,
                         int H, cudaStream_t st) {
  if (rows == 0) return B200MOE_OK;
  gather_rows_bf16_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(dst, x, row_map, div, rows, H);
  return moe_launch_status();
}
int moe_gemm1_w8a16_tc(const MoeGemmArgs& a, cudaStream_t st) { return launch_bt<false>(a, st); }
int moe_gemm2_w8a16_tc(const MoeGemmArgs& a, cudaStream_t st) { return launch_bt<true>(a, st); }

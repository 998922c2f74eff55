// Grouped FP8 (e4m3 x e4m3 -> fp32) expert GEMMs on the sm_100a tensor cores: tcgen05.mma with the
// accumulator in tensor memory, operands staged in shared memory by TMA, block scales applied by the
// epilogue warps ("promotion": every 128-deep K block is accumulated on its own in TMEM, read back,
// multiplied by act_scale[row,kb] * weight_scale[nb,kb] and added to fp32 registers).
//
//   gemm1  h = SiLU(x Wg^T) * (x Wu^T)  per expert, then per-row 1x128 e4m3 requantisation
//          (stands in for the gate/up part of my_ops/fusedMoE.pl:217-259)
//   gemm2  y = h Wd                      per expert, rows scattered to their (token,slot) position
//          (my_ops/fusedMoE.pl:264-269 + scatter_store :55-96); with a peer table the rows go straight to
//          the rank that owns the token (expert parallelism over peer memory: plain peer stores)
//   linear out = x W^T with W [N,K]      one "expert", no activation, bf16 rows out (my_ops/MmW8A16Dq.cpp:185-229)
//
// One persistent CTA per SM, 12 warps: warp 0 = TMA producer, warp 1 = MMA issuer (one thread) and TMEM
// owner, warp 2 = scout (walks the next work item's expert, row range and first scales and leaves them in shared
// memory), warp 3 idle, warps 4..11 = epilogue (TMEM lane quarter = warp%4, column half = (warp-4)/4).  setmaxnreg
// moves registers from the first warpgroup to the epilogue.  Results leave through shared memory: every epilogue warp
// turns its 32 rows x 64 columns through a private patch and stores whole 64- or 128-byte row segments.
// A tile is 128 rows x 256 MMA columns: gemm1 -> 128 gate + 128 up columns of one 128-wide slice of I
// (so SiLU*up and the 1x128 requantisation stay inside the CTA); gemm2 -> 256 columns of H.
// Weights keep the reference layout [E,I,H]: for gemm1 the B operand is K-major, for gemm2 (K = I is the
// slow axis) it is MN-major; both use the 128-byte swizzle that TMA writes.
//
// No multicast loads anywhere.  Every wait is bounded: on a time-out the CTA raises status bit 1, all roles
// leave their loops, tensor memory is released and the kernel returns.
#include "tc_ptx.cuh"

namespace {

#ifndef MOE_TC_CG
#define MOE_TC_CG 2
#endif
constexpr int TC_CG = MOE_TC_CG;             // epilogue column groups (each 4 warps = the four TMEM lane quarters)
constexpr int TC_CW = 128 / TC_CG;           // columns of each 128-column half that one epilogue thread owns
constexpr int TC_CH = 16;                    // columns per tcgen05.ld (= registers of one staging set)
constexpr int TC_CPH = TC_CW / TC_CH;        // TMEM chunks per half
constexpr int TC_NC = 2 * TC_CPH;            // chunks per thread and K block
constexpr int TC_EPI_THREADS = 128 * TC_CG;
constexpr int TC_THREADS = 128 + TC_EPI_THREADS;  // warpgroup 0 = {producer, MMA, scout, idle}, then the epilogue warps
// setmaxnreg targets: warpgroup 0 gives registers to the epilogue.  The increase blocks until the CTA's pool (the
// launch-time count x threads) holds enough, so 128 * LO + TC_EPI_THREADS * HI must not exceed that pool:
// 384 threads x 168 = 128 x 72 + 256 x 216; 640 threads x 96 = 128 x 32 + 512 x 112.
#ifndef MOE_TC_REG_HI
#define MOE_TC_REG_HI (MOE_TC_CG == 2 ? 216 : 112)
#endif
constexpr int TC_REG_HI = MOE_TC_REG_HI;
constexpr int TC_REG_LO = TC_CG == 2 ? (64512 - 256 * TC_REG_HI) / 128 : 32;
constexpr int TC_REG_LAUNCH = (65536 / TC_THREADS) / 8 * 8;  // what __launch_bounds__(TC_THREADS, 1) lets ptxas use
static_assert(128 * TC_REG_LO + TC_EPI_THREADS * TC_REG_HI <= TC_THREADS * TC_REG_LAUNCH,
              "setmaxnreg.inc would wait for registers that the CTA's pool never holds");
constexpr int TC_STAGES = 4;
constexpr int TC_A_BYTES = 128 * 128;       // 128 rows x 128 B
constexpr int TC_B_BYTES = 2 * 128 * 128;   // two 128 x 128 B boxes
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr int TC_TMEM_COLS = 512;           // two accumulator buffers of 256 fp32 columns

struct TcShared {
  uint64_t full[TC_STAGES];
  uint64_t empty[TC_STAGES];  // MMAs of the stage's K block are complete: the stage may be refilled AND the block's
                              // accumulator buffer may be read (one tcgen05.commit per K block serves both)
  uint64_t tmem_empty[2];
  uint64_t head_full, head_empty;  // one-slot hand-over of a work item's starting values (scout warp -> epilogue warps)
  uint64_t dst_full, dst_empty;    // same for the destinations of the item's result rows (taken at the item's END)
  uint32_t tmem_base;
  int abort_flag;
  int head_item[8];        // expert, first row, end of the expert's rows, n-tile, first K block, K blocks
  float head_w[4];         // weight scales of the item's first two K blocks: (gate|half 0, up|half 1) x 2
  float head_sa[2][128];   // activation scales of the first two K blocks, per row of the tile
  int head_dst[128];       // bf16 result rows: destination row (or origin tag) of every row of the tile, -1 = no row
  // results on their way to row-segment stores, one private patch per epilogue warp (down GEMM: 32 rows x 128 B at
  // warp * 4096; gate/up GEMM: 32 rows x 64 B at 4096 + warp * 2048, behind the row maxima that the epilogue's column
  // groups exchange, float [2][TC_CG][128])
  alignas(16) uint8_t ostage[128 * 256];
};
constexpr size_t TC_SMEM_BYTES = 1024 /*alignment slack*/ + (size_t)TC_STAGES * TC_STAGE_BYTES + sizeof(TcShared);
static_assert(TC_SMEM_BYTES <= 232448, "more than the 227 KB of shared memory a CTA can have");

struct TcArgs {
  const float* as_t;
  int64_t ld;
  const void* s0;
  const void* s1;
  const int32_t* mtiles;
  const int32_t* num_mtiles;
  const int32_t* offsets;
  const int32_t* row_map;
  const int32_t* row_src;   // down GEMM over peer memory: origin tag (rank << 24 | row) of every row ...
  const uint64_t* out_tbl;  // ... and the per-rank output buffers (device array of pointers)
  int H, I, NT;
  int P;         // rows the operand buffers hold: row ranges are clipped to it
  int KS;        // K splits (down GEMM of decode-size batches); 1 = none
  int m_major;   // work-item order: 0 = n-tile slow, m-tile fast; 1 = m-tile slow, n-tile fast (see launch_tc)
  float* out32;  // fp32 accumulation target when KS > 1; with KS == 1 (linear layer only): fp32 rows stored instead of bf16
  // down GEMM with the weighted combine fused in: row r adds comb_w[pair] * y[r,:] into comb32[pair / div, :] (fp32,
  // red.global.add; pair = row_map[r] or r, comb_w NULL = weight 1); overrides out / out32
  float* comb32;
  const void* comb_w;
  int comb_wdt, div;
  uint8_t* hq;
  float* hs_t;
  __nv_bfloat16* out;
  int32_t* status;
};

// A pair of fp32 accumulators (two scalar FMAs per pair: on this part the packed fma.rn.f32x2 form was no faster in
// the tensor-memory read-back loop, and the scalar form leaves the register allocator free to place the pairs)
struct acc2_t {
  float x, y;
};
__device__ __forceinline__ acc2_t acc2_zero() { return acc2_t{0.f, 0.f}; }
__device__ __forceinline__ acc2_t pack2(float lo, float hi) { return acc2_t{lo, hi}; }
__device__ __forceinline__ acc2_t pack2u(uint32_t lo, uint32_t hi) { return acc2_t{__uint_as_float(lo), __uint_as_float(hi)}; }
__device__ __forceinline__ float2 unpack2(acc2_t v) { return make_float2(v.x, v.y); }
__device__ __forceinline__ acc2_t ffma2(acc2_t a, acc2_t b, acc2_t c) { return acc2_t{fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y)}; }

// SiLU through one special-function operation per value: x * sigmoid(x) with sigmoid(x) = 0.5 * tanh(0.5 x) + 0.5
// (tanh.approx.f32, absolute error of the sigmoid below 2^-11: far inside the e4m3 requantisation that follows; the
// exp + reciprocal form costs two such operations, and the tile end of the gate/up GEMM is bound by that unit)
__device__ __forceinline__ float moe_silu_fast(float x) {
  const float hx = 0.5f * x;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(hx));
  return fmaf(hx, t, hx);
}

// Instruction descriptor, kind::f8f6f4: D fp32, A/B e4m3, M = 128, N = 256
__host__ __device__ constexpr uint32_t make_idesc(int b_mn_major) {
  return (1u << 4) | ((uint32_t)b_mn_major << 16) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
}

// MODE 0 = gate/up GEMM (+ SiLU*up + requantise), 1 = down GEMM, 2 = plain linear layer: out[r, :N] = A[r, :K] W^T with
// W [N, K] K-major (the gate/up operand path with the down GEMM's bf16 store; a.I = N, a.H = K, 256 outputs per tile)
template <int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
moe_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                   const __grid_constant__ CUtensorMap tmB1, const TcArgs a) {
  constexpr bool GEMM2 = MODE == 1, DENSE = MODE == 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  TcShared* sh = reinterpret_cast<TcShared*>(smem + (size_t)TC_STAGES * TC_STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  volatile int* abort_flag = &sh->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(smem_u32(&sh->full[s]), 1);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->tmem_empty[b]), 4 * TC_CG);
    }
    mbar_init(smem_u32(&sh->head_full), 1);
    mbar_init(smem_u32(&sh->head_empty), 4 * TC_CG);
    mbar_init(smem_u32(&sh->dst_full), 1);
    mbar_init(smem_u32(&sh->dst_empty), 4 * TC_CG);
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)),
                 "r"(TC_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  const int num_mtiles = *a.num_mtiles;
  const int total_tiles = num_mtiles * a.NT * a.KS;  // work items: (n-tile, m-tile, K split)
  const int KB_all = (GEMM2 ? a.I : a.H) / kBlock;
  const int nH = a.H / kBlock, nI = a.I / kBlock;

  // weight-scale addressing: gemm1 s[e, nt, kb] (gate, up); gemm2 s[e, kb, 2*nt + j]; scales are fp32 here.
  // Indices are rebuilt from a few 32-bit values every K block instead of keeping pointers alive: the epilogue
  // loop runs at the edge of the register file and a spilled value costs an L2 round trip here.
  const float* const S0 = reinterpret_cast<const float*>(a.s0);
  const float* const S1 = (GEMM2 || DENSE) ? S0 : reinterpret_cast<const float*>(a.s1);  // one scale tensor
  const int sstep = GEMM2 ? nH : 1;
  const int nIs = (a.I + kBlock - 1) / kBlock;  // scale rows of one expert (= nI unless a linear layer's N % 128 != 0)
  struct Item {
    int nt, mt, kb0, KB;
  };
  auto item_of = [&](int t) {
    Item w;
    const int ks = t % a.KS, tt = t / a.KS;
    w.nt = a.m_major ? tt % a.NT : tt / num_mtiles;
    w.mt = a.m_major ? tt / a.NT : tt - w.nt * num_mtiles;
    w.kb0 = (int)((int64_t)KB_all * ks / a.KS);
    w.KB = (int)((int64_t)KB_all * (ks + 1) / a.KS) - w.kb0;  // K blocks of this work item
    return w;
  };
  // (32-bit: the launcher refuses scale tensors of 2^31 elements or more)
  auto scale_index = [&](const Item& w, int e, int& w0i, int& w1i) {
    w0i = (GEMM2 ? e * nI * nH + 2 * w.nt : DENSE ? (e * nIs + 2 * w.nt) * nH : (e * nI + w.nt) * nH) + w.kb0 * sstep;
    w1i = w0i + (GEMM2 ? ((2 * w.nt + 1 < nH) ? 1 : 0) : DENSE ? ((2 * w.nt + 1 < nIs) ? nH : 0) : 0);
  };
  // results are bf16 rows stored to row_map / row_src destinations (uniform over the launch)
  const bool rows_out = MODE != 0 && (a.row_src || (a.KS == 1 && !a.comb32 && !(DENSE && a.out32)));
  if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TC_REG_LO));
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (one thread)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      // the m-tile list entry of the NEXT work item is requested while this one's loads are issued: when the weights
      // stream from HBM the ring is empty at every tile start, and a dependent L2 round trip there is pure idle time
      auto mtile_of = [&](int t) {
        const int tt = t / a.KS;
        return a.m_major ? tt / a.NT : tt % num_mtiles;
      };
      int nx_e = 0, nx_row0 = 0;
      if ((int)blockIdx.x < total_tiles) nx_e = a.mtiles[2 * mtile_of(blockIdx.x)], nx_row0 = a.mtiles[2 * mtile_of(blockIdx.x) + 1];
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int ks = t % a.KS, tt = t / a.KS;
        const int nt = a.m_major ? tt % a.NT : tt / num_mtiles;
        const int e = nx_e, row0 = nx_row0;
        if (t + (int)gridDim.x < total_tiles) {
          const int mn = mtile_of(t + gridDim.x);
          nx_e = a.mtiles[2 * mn], nx_row0 = a.mtiles[2 * mn + 1];
        }
        const int kb0 = (int)((int64_t)KB_all * ks / a.KS), kb1 = (int)((int64_t)KB_all * (ks + 1) / a.KS);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % TC_STAGES;
          const uint32_t ph = (it / TC_STAGES) & 1;
          if (!mbar_wait(smem_u32(&sh->empty[s]), ph ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&sh->full[s]);
          const uint32_t sa = smem_base + s * TC_STAGE_BYTES, sb = sa + TC_A_BYTES;
          mbar_arrive_expect_tx(full, TC_STAGE_BYTES);
          tma_load_2d(sa, &tmA, kb * kBlock, row0, full);
          if (DENSE) {
            tma_load_2d(sb, &tmB0, kb * kBlock, e * a.I + nt * 256, full);
            tma_load_2d(sb + 128 * 128, &tmB0, kb * kBlock, e * a.I + nt * 256 + 128, full);
          } else if (!GEMM2) {
            tma_load_2d(sb, &tmB0, kb * kBlock, e * a.I + nt * 128, full);
            tma_load_2d(sb + 128 * 128, &tmB1, kb * kBlock, e * a.I + nt * 128, full);
          } else {
            tma_load_2d(sb, &tmB0, nt * 256, e * a.I + kb * kBlock, full);
            tma_load_2d(sb + 128 * 128, &tmB0, nt * 256 + 128, e * a.I + kb * kBlock, full);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (one thread)
    // The loop is flat (the K blocks of all work items of this CTA in one count) and the descriptors are built once:
    // every instruction of this single thread between two K blocks is latency on the accumulator hand-off.
    if (lane == 0) {
      const uint32_t idesc = make_idesc(GEMM2 ? 1 : 0);
      const uint64_t adesc0 = make_smem_desc(smem_base, 16, 1024);
      const uint64_t bdesc0 = GEMM2 ? make_smem_desc(smem_base + TC_A_BYTES, 128 * 128, 1024)
                                    : make_smem_desc(smem_base + TC_A_BYTES, 16, 1024);
      uint32_t n_it = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        const int ks = t % a.KS;
        n_it += (uint32_t)((int)((int64_t)KB_all * (ks + 1) / a.KS) - (int)((int64_t)KB_all * ks / a.KS));
      }
      for (uint32_t it = 0; it < n_it; ++it) {
        const uint32_t s = it % TC_STAGES, buf = it & 1;
        if (!mbar_wait(smem_u32(&sh->full[s]), (it / TC_STAGES) & 1, abort_flag)) break;
        if (!mbar_wait(smem_u32(&sh->tmem_empty[buf]), ((it >> 1) & 1) ^ 1, abort_flag)) break;
        tc_fence_after();
        // the stage's byte offset, in the descriptors' 16-byte units, stays inside the 14-bit address field
        const uint64_t adesc = adesc0 + (uint64_t)(s * (TC_STAGE_BYTES >> 4));
        const uint64_t bdesc = bdesc0 + (uint64_t)(s * (TC_STAGE_BYTES >> 4));
        const uint32_t d = tmem_base + buf * 256;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          // K advances 32 elements: +32 B inside the swizzle atom (K-major) or +32 rows of 128 B (MN-major)
          const uint64_t ad = adesc + (uint64_t)(ks * 2);
          const uint64_t bd = bdesc + (uint64_t)(GEMM2 ? ks * 256 : ks * 2);
          tc_mma_f8(d, ad, bd, idesc, ks > 0 ? 1u : 0u);
        }
        tc_commit(smem_u32(&sh->empty[s]));  // wakes the producer (refill) and the epilogue (accumulator ready)
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ scout: the next work item's starting values
    // What an item starts from sits behind three dependent L2 round trips (m-tile list -> the expert's row range ->
    // the scales of the first two K blocks): 2000 to 3000 cycles when an epilogue warp walks them at the start of the
    // item, a tenth of a short item, and the epilogue's K loop has no registers to carry them ahead.  This warp walks
    // them one item ahead and leaves them in shared memory.
    bool ok = true;
    uint32_t n = 0;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++n) {
      const Item w = item_of(t);
      const int e = a.mtiles[2 * w.mt], row0 = a.mtiles[2 * w.mt + 1];
      const int row_end = min(a.offsets[e + 1], a.P);
      int w0i, w1i;
      scale_index(w, e, w0i, w1i);
      float sa[2][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = row0 + i * 32 + lane;
        sa[0][i] = row < row_end ? a.as_t[(int64_t)w.kb0 * a.ld + row] : 0.f;
        sa[1][i] = row < row_end && w.KB > 1 ? a.as_t[(int64_t)(w.kb0 + 1) * a.ld + row] : 0.f;
      }
      int dst[4] = {-1, -1, -1, -1};  // where the item's result rows go (down GEMM / linear layer with bf16 rows out)
      if (rows_out) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = row0 + i * 32 + lane;
          if (row < row_end) dst[i] = a.row_src ? a.row_src[row] : a.row_map ? a.row_map[row] : row;
        }
      }
      float wv = 0.f;  // lanes 0..3: S0[w0i], S1[w1i], S0[w0i + sstep], S1[w1i + sstep]
      if (lane < 2 || (lane < 4 && w.KB > 1)) wv = ((lane & 1) ? S1 : S0)[((lane & 1) ? w1i : w0i) + ((lane >> 1) ? sstep : 0)];
      // the slot is free once every epilogue warp has taken item n - 1 out of it
      if (n > 0 && !mbar_wait(smem_u32(&sh->head_empty), (n - 1) & 1, abort_flag)) {
        ok = false;
        break;
      }
      if (lane == 0) {
        sh->head_item[0] = e, sh->head_item[1] = row0, sh->head_item[2] = row_end;
        sh->head_item[3] = w.nt, sh->head_item[4] = w.kb0, sh->head_item[5] = w.KB;
      }
      if (lane < 4) sh->head_w[lane] = wv;
#pragma unroll
      for (int i = 0; i < 4; ++i) sh->head_sa[0][i * 32 + lane] = sa[0][i], sh->head_sa[1][i * 32 + lane] = sa[1][i];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->head_full));
      if (rows_out) {
        // (free once every epilogue warp has stored item n - 1: this wait ends at the END of that item, after the
        // head of item n went out above, so neither hand-over holds the other up)
        if (n > 0 && !mbar_wait(smem_u32(&sh->dst_empty), (n - 1) & 1, abort_flag)) {
          ok = false;
          break;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) sh->head_dst[i * 32 + lane] = dst[i];
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh->dst_full));
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue (4 * TC_CG warps)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(TC_REG_HI));
    const int q = warp & 3, cg = (warp - 4) >> 2;
    const int rit = q * 32 + lane;  // row inside the tile == TMEM lane
    uint32_t it = 0;
    bool ok = true;
    int ntile = 0;  // work items this CTA has finished
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++ntile) {
      // the item (its integer divisions included), its expert and rows and the scales of its first two K blocks: left
      // in shared memory by the scout warp
      Item w{0, 0, 0, 0};
      int e = 0, row0 = 0, row_end = 0;
      float f0 = 0.f, f1 = 0.f, sa1 = 0.f, wa1 = 0.f, wb1 = 0.f;
      if (!mbar_wait(smem_u32(&sh->head_full), ntile & 1, abort_flag)) ok = false;
      if (ok) {
        e = sh->head_item[0], row0 = sh->head_item[1], row_end = sh->head_item[2];
        w.nt = sh->head_item[3], w.kb0 = sh->head_item[4], w.KB = sh->head_item[5];
        // Scale factors f0 = sa[row,kb] * sw_gate[kb], f1 = sa[row,kb] * sw_up[kb]: the products of block kb + 1 are
        // formed and the values of block kb + 2 are requested while block kb's TMEM loads are in flight.
        const float sa0 = sh->head_sa[0][rit];
        f0 = sa0 * sh->head_w[0], f1 = sa0 * sh->head_w[1];
        sa1 = sh->head_sa[1][rit], wa1 = sh->head_w[2], wb1 = sh->head_w[3];
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh->head_empty));
      }
      const int nt = w.nt, kb0 = w.kb0, KB = w.KB;
      const int grow = row0 + rit;
      const bool valid = grow < row_end;
      const bool warp_has_rows = row0 + q * 32 < row_end;  // uniform over the warp
      int w0i, w1i;
      scale_index(w, e, w0i, w1i);
      // accumulators as packed fp32 pairs: acc[j][p] = columns (2p, 2p+1) of this thread's TC_CW-column span of half j
      // (cleared below, under the first tensor-memory loads of the item)
      acc2_t acc[2][TC_CW / 2];
      auto clear_acc = [&]() {
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int i = 0; i < TC_CW / 2; ++i) acc[j][i] = acc2_zero();
      };
      auto load_sa = [&](int kb) { return valid ? a.as_t[(int64_t)(kb0 + kb) * a.ld + grow] : 0.f; };
      if (!warp_has_rows) {
        // decode-size batches: most row quarters hold no rows; such a warp only hands every buffer straight back
        clear_acc();
        for (int kb = 0; kb < KB && ok; ++kb, ++it) {
          if (!mbar_wait(smem_u32(&sh->empty[it % TC_STAGES]), (it / TC_STAGES) & 1, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sh->tmem_empty[it & 1]));
        }
      } else if (ok) {
        // The thread's 2 x TC_CW columns leave TMEM in 16-column chunks through two 16-register staging sets: while
        // one set feeds 8 packed FMAs the other set's load is in flight.  The chain runs ACROSS K blocks: the wait for
        // block kb + 1's accumulator, the scale products and the hand-back of block kb's buffer all sit under loads in
        // flight, and block kb + 1's first two loads are issued between block kb's last FMAs.  (A warp that walks
        // wait -> loads -> FMAs -> hand-back strictly block by block spends most of a K block waiting on one of them.)
        uint32_t s0[TC_CH], s1[TC_CH];
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16) + cg * TC_CW;
        auto chunk_addr = [&](uint32_t tb, int c) { return tb + (c / TC_CPH) * 128 + (c % TC_CPH) * TC_CH; };
        acc2_t f0p = acc2_zero(), f1p = acc2_zero();
        auto fma_chunk = [&](int c, const uint32_t (&sv)[TC_CH]) {
          const acc2_t fp = (c / TC_CPH) ? f1p : f0p;
#pragma unroll
          for (int i = 0; i < TC_CH / 2; ++i)
            acc[c / TC_CPH][(c % TC_CPH) * (TC_CH / 2) + i] =
                ffma2(pack2u(sv[2 * i], sv[2 * i + 1]), fp, acc[c / TC_CPH][(c % TC_CPH) * (TC_CH / 2) + i]);
        };
        if (!mbar_wait(smem_u32(&sh->empty[it % TC_STAGES]), (it / TC_STAGES) & 1, abort_flag)) ok = false;
        if (ok) {
          tc_fence_after();
          const uint32_t tb = lane_base + (it & 1) * 256;
          tc_ld_issue(chunk_addr(tb, 0), s0);
          tc_ld_issue(chunk_addr(tb, 1), s1);
        }
        clear_acc();
        for (int kb = 0; kb < KB && ok; ++kb, ++it) {
          const bool more = kb + 1 < KB;
          const uint32_t tb = lane_base + (it & 1) * 256;
          f0p = pack2(f0, f0), f1p = pack2(f1, f1);
          const float nf0 = sa1 * wa1, nf1 = sa1 * wb1;  // block kb + 1
          if (kb + 2 < KB) {
            sa1 = load_sa(kb + 2);
            wa1 = S0[w0i + (kb + 2) * sstep];
            wb1 = S1[w1i + (kb + 2) * sstep];
          }
          tc_ld_wait(s0, s1);
#pragma unroll
          for (int c = 0; c < TC_NC - 2; c += 2) {
            fma_chunk(c, s0);
            tc_ld_issue(chunk_addr(tb, c + 2), s0);
            fma_chunk(c + 1, s1);
            tc_ld_issue(chunk_addr(tb, c + 3), s1);
            if (c + 4 < TC_NC) tc_ld_wait(s0, s1);
          }
          const uint32_t nbar = smem_u32(&sh->empty[(it + 1) % TC_STAGES]), npar = ((it + 1) / TC_STAGES) & 1;
          // The last two chunks of this block are in flight.  Is the next block's accumulator there already (it is
          // whenever this warp is what the MMAs wait for)?  Only a test: the buffer goes back before any real wait,
          // or the MMA issuer, which needs this buffer for block kb + 2, would idle until block kb + 1 is done.
          const bool next_ready = more && mbar_test(nbar, npar);
          tc_ld_wait(s0, s1);
          tc_fence_before();  // all of this block is in registers: hand the buffer back
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sh->tmem_empty[it & 1]));
          const uint32_t tn = lane_base + ((it + 1) & 1) * 256;
          if (next_ready) {
            tc_fence_after();
            fma_chunk(TC_NC - 2, s0);
            tc_ld_issue(chunk_addr(tn, 0), s0);
            fma_chunk(TC_NC - 1, s1);
            tc_ld_issue(chunk_addr(tn, 1), s1);
          } else {
            fma_chunk(TC_NC - 2, s0);
            fma_chunk(TC_NC - 1, s1);
            if (more) {
              if (!mbar_wait(nbar, npar, abort_flag)) {
                ok = false;
                break;
              }
              tc_fence_after();
              tc_ld_issue(chunk_addr(tn, 0), s0);
              tc_ld_issue(chunk_addr(tn, 1), s1);
            }
          }
          f0 = nf0, f1 = nf1;
        }
      } else {
        clear_acc();  // (a wait ran out: nothing below stores anything, but nothing reads an unset register either)
      }
      float amax = 0.f;
      if (MODE == 0) {
        // SiLU(gate) * up; the row's 128 values are split over TC_CG warps, which exchange their maxima through
        // shared memory (two copies, alternating by tile, so that one barrier per tile is enough)
#pragma unroll
        for (int i = 0; i < TC_CW / 2; ++i) {  // h overwrites the gate accumulators: no second array of 64 registers
          const float2 g = unpack2(acc[0][i]), u = unpack2(acc[1][i]);
          const float hx = moe_silu_fast(g.x) * u.x, hy = moe_silu_fast(g.y) * u.y;
          acc[0][i] = pack2(hx, hy);
          amax = fmaxf(amax, fmaxf(fabsf(hx), fabsf(hy)));
        }
        reinterpret_cast<float*>(sh->ostage)[((ntile & 1) * TC_CG + cg) * 128 + rit] = amax;
      }
      // One decision for all epilogue warps before anything that couples them (the named barriers of the tile end): a
      // warp whose wait ran out comes here like the others, and if any did, all of them leave together.
      {
        uint32_t any_bad;
        asm volatile(
            "{\n\t.reg .pred p, r;\n\t"
            "setp.ne.b32 p, %1, 0;\n\t"
            "bar.red.or.pred r, 1, %2, p;\n\t"
            "selp.u32 %0, 1, 0, r;\n\t}"
            : "=r"(any_bad)
            : "r"((uint32_t)(ok ? 0 : 1)), "n"(TC_EPI_THREADS)
            : "memory");
        if (any_bad) {
          ok = false;
          break;
        }
      }
      // Results leave through shared memory.  A thread owns one row, so stores from registers would put 16 bytes per
      // lane into 32 different rows per instruction: half-used sectors (and, to a peer, 32 small packets), which cost
      // several thousand cycles per tile.  Each warp turns its own 32 rows x TC_CW columns through a private patch of
      // shared memory instead (16-byte chunks, XOR-swizzled so that neither side has bank conflicts; only warp-level
      // synchronisation) and then stores whole 64- or 128-byte row segments per group of lanes.
      static_assert(TC_CW == 64, "the row-segment stores below are laid out for 64 columns per warp");
      const int wepi = warp - 4;
      if (MODE == 0) {
#pragma unroll
        for (int o = 0; o < TC_CG; ++o) amax = fmaxf(amax, reinterpret_cast<const float*>(sh->ostage)[((ntile & 1) * TC_CG + o) * 128 + rit]);
        amax = fmaxf(amax, kAmaxFloor);
        const float inv = kFp8Max / amax;
        uint4* wst = reinterpret_cast<uint4*>(sh->ostage + 4096 + wepi * 2048);  // 32 rows x 64 B, past the row maxima
#pragma unroll
        for (int v4 = 0; v4 < TC_CW / 16; ++v4) {
          uint4 o;
          uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
          for (int w4 = 0; w4 < 4; ++w4) {
            const float2 p0 = unpack2(acc[0][v4 * 8 + w4 * 2]), p1 = unpack2(acc[0][v4 * 8 + w4 * 2 + 1]);
            ow[w4] = moe_f32x4_to_e4m3x4(p0.x * inv, p0.y * inv, p1.x * inv, p1.y * inv);
          }
          wst[lane * 4 + (v4 ^ ((lane >> 1) & 3))] = o;
        }
        if (valid && cg == 0) a.hs_t[(int64_t)nt * a.ld + grow] = amax / kFp8Max;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // 8 rows x 64 B per instruction
          const int r = i * 8 + (lane >> 2), c = lane & 3;
          const int orow = row0 + q * 32 + r;
          if (orow < row_end)
            *reinterpret_cast<uint4*>(a.hq + (int64_t)orow * a.I + nt * 128 + cg * TC_CW + c * 16) = wst[r * 4 + (c ^ ((r >> 1) & 3))];
        }
        __syncwarp();
      } else if (a.row_src || (a.KS == 1 && !a.comb32 && !(DENSE && a.out32))) {
        // bf16 result rows, to this GPU's output (row r of the tile -> out[row_map[r]]) or, under expert parallelism,
        // to the rank that owns the token (plain peer stores)
        const int OUTW = DENSE ? a.I : a.H;  // columns of an output row
        // destination of this lane's row: fetched by the scout warp (origin tag rank << 24 | row under expert
        // parallelism, else the output row; -1 = the lane has no row)
        unsigned long long my_dst = 0;  // byte address of this lane's output row; 0 = the lane has no row
        if (mbar_wait(smem_u32(&sh->dst_full), ntile & 1, abort_flag)) {
          const int tag = sh->head_dst[rit];
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sh->dst_empty));
          if (tag >= 0)
            my_dst = a.row_src ? a.out_tbl[tag >> 24] + (unsigned long long)(tag & 0xFFFFFF) * OUTW * 2
                               : reinterpret_cast<unsigned long long>(a.out) + (unsigned long long)tag * OUTW * 2;
        } else {
          ok = false;  // (the flag is up: every warp leaves at the next item's barrier; nothing is stored here)
        }
        uint4* wst = reinterpret_cast<uint4*>(sh->ostage + wepi * 4096);  // 32 rows x 128 B
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int col0 = nt * 256 + j * 128 + cg * TC_CW;
          if (col0 < OUTW) {  // uniform over the warp (a linear layer's last tile may be narrower)
#pragma unroll
            for (int v4 = 0; v4 < TC_CW / 8; ++v4) {
              uint4 o;
              __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int w4 = 0; w4 < 4; ++w4) {
                const float2 v = unpack2(acc[j][v4 * 4 + w4]);
                o2[w4] = __floats2bfloat162_rn(v.x, v.y);
              }
              wst[lane * 8 + (v4 ^ (lane & 7))] = o;
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {  // 4 rows x 128 B per instruction
              const int r = i * 4 + (lane >> 3), c = lane & 7;
              const unsigned long long dst = __shfl_sync(0xffffffffu, my_dst, r);
              const uint4 v = wst[r * 8 + (c ^ (r & 7))];
              if (dst) *reinterpret_cast<uint4*>(dst + (unsigned long long)(col0 + c * 8) * 2) = v;
            }
            __syncwarp();
          }
        }
      } else if (valid && a.comb32) {
        // Fused weighted combine: the k rows of one token come from different experts, i.e. from different CTAs, so they
        // meet in an fp32 buffer through 16-byte reductions (their order, and with it the last bit of the sum, is not
        // fixed).  K-split partial sums take the same way: the combine is linear.
        const int pair = a.row_map ? a.row_map[grow] : grow;
        const float w = a.comb_w ? moe_load_as_f32(a.comb_w, pair, a.comb_wdt) : 1.f;
        float* drow = a.comb32 + (int64_t)(pair / a.div) * a.H;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int col = nt * 256 + j * 128 + cg * TC_CW;
          if (col >= a.H) continue;
#pragma unroll
          for (int v4 = 0; v4 < TC_CW / 4; ++v4) {
            const float2 p0 = unpack2(acc[j][v4 * 2]), p1 = unpack2(acc[j][v4 * 2 + 1]);
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(drow + col + v4 * 4), "f"(p0.x * w),
                         "f"(p0.y * w), "f"(p1.x * w), "f"(p1.y * w)
                         : "memory");
          }
        }
      } else if (valid) {
        // fp32 targets: K-split partial sums, or a linear layer's fp32 output
        const int64_t dstrow = a.row_map ? a.row_map[grow] : grow;
        const int OUTW = DENSE ? a.I : a.H;  // columns of an output row
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int col = nt * 256 + j * 128 + cg * TC_CW;
          if (col < OUTW && a.KS > 1) {  // K split: partial sums meet in the fp32 buffer
            float* dst32 = a.out32 + dstrow * OUTW + col;
#pragma unroll
            for (int v4 = 0; v4 < TC_CW / 4; ++v4) {
              const float2 p0 = unpack2(acc[j][v4 * 2]), p1 = unpack2(acc[j][v4 * 2 + 1]);
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst32 + v4 * 4), "f"(p0.x), "f"(p0.y),
                           "f"(p1.x), "f"(p1.y)
                           : "memory");
            }
          } else if (col < OUTW && DENSE && a.out32) {  // fp32 output rows (plain stores)
            float4* dst = reinterpret_cast<float4*>(a.out32 + dstrow * OUTW + col);
#pragma unroll
            for (int v4 = 0; v4 < TC_CW / 4; ++v4) {
              const float2 p0 = unpack2(acc[j][v4 * 2]), p1 = unpack2(acc[j][v4 * 2 + 1]);
              dst[v4] = make_float4(p0.x, p0.y, p1.x, p1.y);
            }
          }
        }
      }
    }
  }

  // ---- teardown: every role arrives here, also after a time-out ---------------------------------------
  tc_fence_before();
  __syncthreads();
  if (sh->abort_flag) {
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, B200MOE_STATUS_WAIT_TIMEOUT);
    // give copies and MMAs that are still in flight time to land before shared/tensor memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------------------------
// row-major u8 matrix [rows, cols], box 128 x 128 bytes, 128-byte swizzle, zero fill outside
bool make_map_u8(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols};
  cuuint32_t box[2] = {128, 128};
  cuuint32_t es[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Per-device facts and one-time set-up, indexed by the CUDA device ordinal: a process that drives several GPUs comes
// here with each of them current in turn (the dynamic shared-memory cap of a kernel is a per-device attribute).
constexpr int kMaxDevices = 64;
struct DeviceInfo {
  int sm_count = 0;  // 0 = not looked up yet
  bool tc_ok = false, attr_set = false;
};
DeviceInfo* device_info() {
  static DeviceInfo tab[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  DeviceInfo& d = tab[dev];
  if (d.sm_count == 0) {
    int v = 0, major = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    d.tc_ok = major == 10 && get_encode_fn() != nullptr;
    d.sm_count = v > 0 ? v : 1;
  }
  return &d;
}

int device_sm_count() {
  DeviceInfo* d = device_info();
  return d ? d->sm_count : 1;
}

template <int MODE>
int launch_tc(const MoeGemmArgs& g, cudaStream_t st) {
  constexpr bool GEMM2 = MODE == 1, DENSE = MODE == 2;
  if (g.scale_dtype != B200MOE_F32) return B200MOE_EINVAL;  // the caller converts bf16 scales first
  if ((int64_t)g.E * ((g.I + kBlock - 1) / kBlock) * (g.H / kBlock) >= (int64_t(1) << 31)) return B200MOE_EINVAL;  // 32-bit scale indices
  const int K = GEMM2 ? g.I : g.H;
  CUtensorMap tmA, tmB0, tmB1;
  if (!make_map_u8(&tmA, g.aq, (uint64_t)g.P, (uint64_t)K)) return B200MOE_EDRIVER;
  if (!make_map_u8(&tmB0, g.w0, (uint64_t)g.E * g.I, (uint64_t)g.H)) return B200MOE_EDRIVER;
  if (!make_map_u8(&tmB1, (GEMM2 || DENSE) ? g.w0 : g.w1, (uint64_t)g.E * g.I, (uint64_t)g.H)) return B200MOE_EDRIVER;
  TcArgs a{};
  a.as_t = g.as_t;
  a.ld = g.ld;
  a.s0 = g.s0;
  a.s1 = g.s1;
  a.mtiles = g.mtiles;
  a.num_mtiles = g.num_mtiles;
  a.offsets = g.offsets;
  a.row_map = g.row_map;
  a.row_src = GEMM2 ? g.row_src : nullptr;
  a.out_tbl = g.out_tbl;
  a.H = g.H;
  a.I = g.I;
  a.P = (int)g.P;
  a.NT = GEMM2 ? (g.H + 255) / 256 : DENSE ? (g.I + 255) / 256 : g.I / 128;
  a.comb32 = (GEMM2 && !g.row_src) ? g.comb32 : nullptr;
  a.comb_w = g.comb_w;
  a.comb_wdt = g.comb_wdt;
  a.div = g.div > 0 ? g.div : 1;
  a.KS = (GEMM2 && g.ksplit > 1 && (g.out32 || a.comb32) && !g.row_src) ? g.ksplit : 1;
  // Work-item order.  The CTAs that run together hold about one SM count of consecutive work items.  With the
  // n-tile as the slow index they share a few weight tiles and sweep ALL rows of A once per group of n-tiles: right
  // while A stays in L2.  When A is larger than that (prefill-size down GEMM: P x I bytes; many-token gate/up GEMM
  // with small experts), the m-tile becomes the slow index: an m-tile's rows are read once, by the CTAs of all its
  // n-tiles at the same time, and an expert's weights are shared by its consecutive m-tiles through L2 as long as
  // one expert's weights for this GEMM fit there.  Measured on the Mixtral down GEMM at 4096 tokens: DRAM reads
  // 1.43 GB with the n-tile slow (hq re-read 7x), against 0.59 GB algorithmic.
  {
    const double a_bytes = (double)g.P * K;
    const double w_expert = (double)(GEMM2 ? g.H : DENSE ? g.I : 2 * g.I) * K;
    a.m_major = (a_bytes > 48e6 && w_expert <= 64e6) ? 1 : 0;
  }
  a.out32 = g.out32;
  a.hq = g.hq;
  a.hs_t = g.hs_t;
  a.out = g.out;
  a.status = g.status;
  DeviceInfo* di = device_info();
  if (!di) return B200MOE_EDRIVER;
  if (!di->attr_set) {
    cudaFuncSetAttribute(moe_gemm_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES);
    cudaFuncSetAttribute(moe_gemm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES);
    cudaFuncSetAttribute(moe_gemm_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES);
    di->attr_set = true;
  }
  const long long max_tiles = (long long)g.max_mtiles * a.NT * a.KS;
  const int sms = g.max_ctas > 0 && g.max_ctas < device_sm_count() ? g.max_ctas : device_sm_count();
  const int grid = (int)(max_tiles < sms ? max_tiles : sms);
  moe_gemm_tc_kernel<MODE><<<grid, TC_THREADS, TC_SMEM_BYTES, st>>>(tmA, tmB0, tmB1, a);
  return moe_launch_status();
}

}  // namespace

bool moe_tc_available() {
  DeviceInfo* d = device_info();
  return d && d->tc_ok;
}

namespace {
__global__ void f32_rows_to_bf16_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ in, int64_t n) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    const float4 v = *reinterpret_cast<const float4*>(in + i);
    *reinterpret_cast<__nv_bfloat162*>(out + i) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(out + i + 2) = __floats2bfloat162_rn(v.z, v.w);
  }
}
}  // namespace

int moe_f32_rows_to_bf16(__nv_bfloat16* out, const float* in, int64_t n, cudaStream_t st) {
  f32_rows_to_bf16_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, st>>>(out, in, n);
  return moe_launch_status();
}

int moe_device_sm_count() { return device_sm_count(); }

int moe_gemm1_tc(const MoeGemmArgs& a, cudaStream_t st) { return launch_tc<0>(a, st); }
int moe_gemm2_tc(const MoeGemmArgs& a, cudaStream_t st) { return launch_tc<1>(a, st); }
int moe_linear_tc(const MoeGemmArgs& a, cudaStream_t st) { return launch_tc<2>(a, st); }

// Launchers shared between the translation units of libb200moe (not part of the C ABI).
#pragma once
#include "common.cuh"

constexpr int kTileM = 128;  // rows of one m-tile of the grouped GEMMs

// One grouped-GEMM problem: rows [0,P) sorted by expert, m-tiles built from expert_offsets.
struct MoeGemmArgs {
  // activations
  const uint8_t* aq;        // W8A8: e4m3 [P,K]
  const float* as_t;        // W8A8: scales [K/128, ld]
  int64_t ld;               // leading dimension of transposed scale arrays
  const __nv_bfloat16* a16; // W8A16: bf16 rows; gemm1: x [T,H] gathered through row_map/div; gemm2: h [P,I]
  const int32_t* row_map;   // sorted_pair (flat t*k+j) or nullptr for identity
  int div;                  // k (pair -> token)
  // weights of this problem ([E,I,H] e4m3, scales [E,I/128,H/128])
  const uint8_t* w0;        // gemm1: gate; gemm2: down
  const uint8_t* w1;        // gemm1: up
  const void* s0;
  const void* s1;
  int scale_dtype;
  int w_bf16;               // weights are bf16 (no scales): W8A16 tensor-core kernels only
  // tiling
  const int32_t* mtiles;    // int2 {expert, row0} per m-tile
  const int32_t* num_mtiles;
  const int32_t* offsets;   // expert_offsets[E+1]
  int max_mtiles;
  int max_ctas;             // 0 = all SMs; else the cap on the tensor-core kernels' persistent grid
  int64_t P;
  int H, I, E;
  // outputs
  uint8_t* hq;              // gemm1 W8A8: e4m3 [P,I]
  float* hs_t;              // gemm1 W8A8: [I/128, ld]
  __nv_bfloat16* h16;       // gemm1 W8A16: bf16 [P,I]
  __nv_bfloat16* out;       // gemm2: bf16 rows of H, row index = row_map ? row_map[r] : r
  int ksplit;               // gemm2 (tensor-core path): > 1 splits K over CTAs, partial sums added into out32
  float* out32;             // fp32 [rows,H], zero on entry, same row indexing as out (needed when ksplit > 1)
  // gemm2 with the weighted combine fused in (tensor-core path only): row r adds comb_w[pair] * y[r,:] into
  // comb32[pair / div, :], pair = row_map ? row_map[r] : r; comb32 fp32 [T,H], zero on entry; comb_w NULL = weight 1
  float* comb32;
  const void* comb_w;
  int comb_wdt;
  // gemm2 over peer memory (tensor-core path only): row r goes to rank (row_src[r] >> 24), row (row_src[r] & 0xFFFFFF)
  // of that rank's buffer out_tbl[rank] (bf16 rows of H); overrides out/row_map
  const int32_t* row_src;
  const uint64_t* out_tbl;
  int32_t* status;
};

// b200moe_permute that also writes the m-tile list when one CTA does the whole sort (at most 1024 pairs)
int moe_permute_impl(int32_t* sorted_pair, int32_t* expert_offsets, const int32_t* ids, int64_t T, int64_t k, int64_t E,
                     int32_t* scratch, int32_t* status, int32_t* mtiles, int32_t* num_mtiles, int max_mtiles,
                     bool* tiles_done, void* stream);
// tiles of rows [offsets[e], offsets[e+1]) clipped to max_rows; at most max_mtiles entries are written
int moe_build_mtiles(int32_t* mtiles, int32_t* num_mtiles, const int32_t* offsets, int E, int64_t max_rows,
                     int max_mtiles, cudaStream_t st);
// identity problem (one expert, rows 0..T): offsets = {0,T}
int moe_fill_identity_offsets(int32_t* offsets, int64_t T, cudaStream_t st);

int moe_gemm1_simple(const MoeGemmArgs& a, int act_mode, cudaStream_t st);
int moe_gemm2_simple(const MoeGemmArgs& a, int act_mode, cudaStream_t st);
int moe_gemm1_tc(const MoeGemmArgs& a, cudaStream_t st);
int moe_gemm2_tc(const MoeGemmArgs& a, cudaStream_t st);
// plain linear layer: out[r, :I] = A[r, :H] * w0^T, w0 [E*I, H] K-major with scales s0 [E, ceil(I/128), H/128]; bf16 rows of I
int moe_linear_tc(const MoeGemmArgs& a, cudaStream_t st);
// the reference arithmetic (bf16 activations, weights dequantised to bf16) on the tensor cores; a16 = rows in sorted order
int moe_gemm1_w8a16_tc(const MoeGemmArgs& a, cudaStream_t st);
int moe_gemm2_w8a16_tc(const MoeGemmArgs& a, cudaStream_t st);
int moe_gather_rows_bf16(__nv_bfloat16* dst, const __nv_bfloat16* x, const int32_t* row_map, int div, int64_t rows,
                         int H, cudaStream_t st);
int moe_f32_rows_to_bf16(__nv_bfloat16* out, const float* in, int64_t n, cudaStream_t st);
int moe_device_sm_count();
bool moe_tc_available();

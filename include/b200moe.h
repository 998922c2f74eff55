/* b200moe.h - C ABI of the B200 (sm_100a) fused-MoE kernels.
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer unless stated otherwise, every
 * call enqueues work on `stream` (a cudaStream_t passed as void*) of the CURRENT device and returns
 * without synchronising.  Nothing here allocates device memory: the caller owns inputs, outputs and
 * the workspace (size from b200moe_experts_workspace_bytes).
 *
 * Return value: 0 = enqueued; negative = argument rejected on the host before any launch
 * (B200MOE_E*); positive = the cudaError_t of a failed launch.
 *
 * These entry points are what the reference's vendor C ABI (third_party/tpuDNN/include/tpuDNN.h:6-48,
 * tpuDNNTensor.h) is to its op wrappers in torch_tpu/csrc/ops/my_ops/: each one names the reference
 * interface it stands in for.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_ABI_VERSION 3

enum {
  B200MOE_OK = 0,
  B200MOE_EINVAL = -1,     /* null pointer, non-positive size, unknown enum */
  B200MOE_ESHAPE = -2,     /* a size the kernels do not support (see each call) */
  B200MOE_EWORKSPACE = -3, /* workspace too small or misaligned */
  B200MOE_EALIGN = -4,     /* a pointer that must be 16-byte aligned is not */
  B200MOE_EDRIVER = -5     /* the CUDA driver entry point for tensor maps is unavailable */
};

/* element types of score / scale / weight tensors */
enum { B200MOE_F32 = 0, B200MOE_BF16 = 1, B200MOE_F16 = 2 };

/* score functions of b200moe_route */
enum { B200MOE_SCORE_SOFTMAX = 0, B200MOE_SCORE_SIGMOID = 1 };

/* output modes of b200moe_experts */
enum {
  B200MOE_OUT_PER_SLOT = 0, /* out [T,k,H] bf16, un-weighted (what the reference op returns) */
  B200MOE_OUT_COMBINED = 1, /* out [T,H] bf16 = sum_j w[t,j] * y[t,j,:] (+ shared expert): per-slot rows go to
                               the workspace and a second kernel sums them in slot order (bit-reproducible) */
  B200MOE_OUT_COMBINED_FUSED = 2 /* the same sum formed inside the down GEMM's epilogue: every result row is
                               multiplied by its routing weight and added (fp32 reductions) into a [T,H]
                               buffer, then rounded to bf16 once.  No per-slot rows in memory; the order of
                               the k additions is not fixed, so the last bit may differ from run to run.
                               Tensor-core path only (elsewhere it behaves like B200MOE_OUT_COMBINED). */
};

/* stages of b200moe_experts (b200moe_experts_desc.stages) */
enum {
  B200MOE_STAGE_PREP = 1,    /* permutation, tile list, activation quantisation, scale conversion */
  B200MOE_STAGE_GATE_UP = 2, /* gate/up GEMM + SiLU*up (+ requantisation) */
  B200MOE_STAGE_DOWN = 4,    /* down GEMM + scatter (or fused combine) */
  B200MOE_STAGE_COMBINE = 8, /* weighted combine / final rounding */
  B200MOE_STAGE_ALL = 15
};

/* arithmetic of the expert GEMMs */
enum {
  B200MOE_ACT_W8A8 = 0,  /* activations quantised per token per 128 columns to e4m3; FP8 tensor cores */
  B200MOE_ACT_W8A16 = 1  /* reference arithmetic: weights dequantised to bf16, bf16 roundings kept   */
};

/* kernel family selector (tests use it to A/B the two implementations) */
enum { B200MOE_IMPL_AUTO = 0, B200MOE_IMPL_SIMPLE = 1, B200MOE_IMPL_TCGEN05 = 2 };

int b200moe_abi_version(void);
const char* b200moe_error_string(int code);

/* Device-side status word of the last kernels that ran with `status` != NULL: 0 = ok, bit 0 = an
 * expert id outside [0,E) was skipped, bit 1 = a bounded wait inside a kernel gave up, bit 2 = a wait for a
 * peer rank's flag gave up (peer-memory expert parallelism), bit 3 = a dispatched row did not fit the
 * destination's capacity and was dropped. */

/* ---- routing -------------------------------------------------------------------------------- */

/* Grouped top-k on given scores.  Stands in for tpudnnNoauxTcTopkAsync
 * (third_party/tpuDNN/include/tpuDNNTensor.h:728-737; wrapper my_ops/NoauxTcTopk.cpp:9-67).
 * scores [batch, n_experts] of `dtype`; values [batch, top_k] of the same dtype; indices int32.
 * Group score = sum of the group's two largest scores, formed in `dtype`; ties -> lowest index.
 * Limits: n_experts <= 1024, n_groups <= 32, top_k <= 32. */
int b200moe_noaux_tc_topk(void* values, int32_t* indices, const void* scores, int dtype,
                          int64_t batch, int64_t n_experts, int64_t n_groups, int64_t topk_groups,
                          int64_t top_k, void* stream);

/* Plain descending top-k along the last dim, int32 indices.  Stands in for tpudnnTopkAsync as used by
 * aten::topk on the device (native_ops/Topk.cpp:90-150).  n <= 1024, k <= 32. */
int b200moe_topk(void* values, int32_t* indices, const void* x, int dtype, int64_t batch, int64_t n,
                 int64_t k, void* stream);

/* Router GEMM: logits[T,E] (fp32) = x[T,H] (bf16) . wr[E,H]^T (bf16).  First op of the caller-side
 * routing chain (python/regression/test_llm/test_torch_ops.py:439-455).  H % 8 == 0. */
int b200moe_router_logits(float* logits, const void* x, const void* wr, int64_t T, int64_t H,
                          int64_t E, void* stream);

/* The rest of that chain in one kernel: (+logit_bias) -> score (softmax | sigmoid) -> (+bias, selection only) ->
 * group-limited top-k -> gather un-biased scores -> optional renormalisation -> * scale.
 * logits fp32 [T,E]; logit_bias, bias fp32 [E] or NULL; ids int32 [T,k]; w fp32 [T,k]; w_bf16 (optional) bf16
 * [T,k].  n_groups <= 1 disables grouping.  Also the arithmetic behind
 * tpudnnFusedMoEGroupedTopkMultiCoreAsync (tpuDNNTensor.h:1572-1583). */
int b200moe_route(int32_t* ids, float* w, void* w_bf16, const float* logits, const float* logit_bias,
                  const float* bias, int64_t T, int64_t E, int64_t k, int score_func, int64_t n_groups,
                  int64_t topk_groups, int renorm, float scale, void* stream);

/* ---- permutation ------------------------------------------------------------------------------ */

/* Stable sort of the T*k (token,slot) pairs by expert id: sorted_pair[P] (flat t*k+j, ascending
 * inside an expert), expert_offsets[E+1].  The device twin of phases 1-2 of the reference kernel
 * (my_ops/fusedMoE.pl:624-756).  scratch: int32[b200moe_permute_scratch_ints(P,E)].
 * Ids outside [0,E) are dropped (status bit 0): expert_offsets[E] is then smaller than T*k and the tail
 * sorted_pair[expert_offsets[E] .. T*k) holds -1; every kernel of this library that walks sorted_pair skips
 * negative entries, and in the per-slot output the rows of dropped pairs are left untouched. */
size_t b200moe_permute_scratch_ints(int64_t P, int64_t E);
int b200moe_permute(int32_t* sorted_pair, int32_t* expert_offsets, const int32_t* ids, int64_t T,
                    int64_t k, int64_t E, int32_t* scratch, int32_t* status, void* stream);

/* b200moe_permute for callers that cannot hand over scratch memory.  No counterpart in the reference (its
 * callers always pass scratch tensors in): it exists for hosts that must not allocate on the device around the
 * call - a server with a memory pool fixed at start-up, a plugin that only receives input and output buffers.
 * The chunk-count table lives in a fixed 256 KB array inside the library (held by every GPU that loads it, until
 * the process exits); no cudaMalloc/cudaFree or other allocating routine is called.
 * Limit: b200moe_permute_scratch_ints(T*k, E) <= b200moe_permute_static_max_scratch_ints() (65536; e.g. 262144
 * pairs x 256 experts), otherwise B200MOE_ESHAPE.  The first call on each device looks up the array's device
 * address; make that first call outside any stream capture.  All calls on a device share the one array: two calls
 * whose kernels may overlap on the GPU (different streams) race - serialise them.  Nothing needs clearing
 * between calls (the table is rewritten in full before it is read). */
size_t b200moe_permute_static_max_scratch_ints(void);
int b200moe_permute_static(int32_t* sorted_pair, int32_t* expert_offsets, const int32_t* ids, int64_t T,
                           int64_t k, int64_t E, int32_t* status, void* stream);

/* The reference's own scratch layout (fusedMoE.cpp:303-306, fusedMoE.pl:737-755): gather_index[E,T]
 * (token ids), scatter_index[E,T] (flat pair ids), num_per_expert[E]; unused tail entries are left
 * untouched.  Computed from sorted_pair / expert_offsets. */
int b200moe_gather_scatter_index(int32_t* gather_index, int32_t* scatter_index,
                                 int32_t* num_per_expert, const int32_t* sorted_pair,
                                 const int32_t* expert_offsets, int64_t T, int64_t k, int64_t E,
                                 void* stream);

/* Row gather + per-row 1x128 e4m3 quantisation: for r in [0,rows): src = row_map ? row_map[r]/div : r;
 * q[r,:] = e4m3(x[src,:] * 448/amax), s_t[g, r] = amax/448 (scales stored group-major, [H/128, ld]).
 * x bf16 [*,H]; H % 128 == 0. */
int b200moe_quant_rows(uint8_t* q, float* s_t, int64_t ld, const void* x, const int32_t* row_map,
                       int64_t div, int64_t rows, int64_t H, void* stream);

/* ---- experts ------------------------------------------------------------------------------------ */

/* Everything after routing: permute -> quantise -> grouped gate/up GEMM + SiLU*up (+ requantise) ->
 * grouped down GEMM -> scatter (per-slot) or weighted combine.  Stands in for
 * tpudnnFusedMoEFusedExpertsMultiCoreAsync (tpuDNNTensor.h:1585-1611; wrapper my_ops/fusedMoE.cpp:117-236)
 * and for the PPL kernel behind fused_moe_fused_experts_v2 (my_ops/fusedMoE.pl:795-810).
 *
 *   x        bf16 [T,H]
 *   w_gate, w_up, w_down   e4m3 [E,I,H]  (down = W_down^T, contiguous: test_moe.py:285)
 *   s_gate, s_up, s_down   [E, I/128, H/128] of scale_dtype (fp32 or bf16); ignored (may be NULL) with
 *                          weights_bf16 = 1, where the three weight tensors are bf16
 *   ids      int32 [T,k];  topk_w  [T,k] of w_dtype (needed for B200MOE_OUT_COMBINED, else may be NULL)
 *   shared_* optional dense expert applied to every token with weight 1 (combined mode only), same
 *            layouts with E = 1 and intermediate size I_shared; pass NULL / 0 to disable
 *   out      bf16 [T,k,H] or [T,H] by out_mode
 *   workspace  >= b200moe_experts_workspace_bytes(...) bytes, 256-byte aligned
 *   status   optional int32 device word (see above)
 * H % 128 == 0, I % 128 == 0, T*k < 2^24.  */
typedef struct {
  int64_t T, H, I, E, k;
  int64_t I_shared;   /* 0 = no shared expert */
  int out_mode;       /* B200MOE_OUT_* */
  int act_mode;       /* B200MOE_ACT_* */
  int impl;           /* B200MOE_IMPL_* */
  int scale_dtype;    /* B200MOE_F32 | B200MOE_BF16 */
  int w_dtype;        /* dtype of topk_w: B200MOE_F32 | B200MOE_BF16 */
  int impl_gate_up;   /* B200MOE_IMPL_AUTO = follow `impl`; else the kernel family of the gate/up GEMM alone */
  int impl_down;      /* the same for the down GEMM (tests A/B one GEMM at a time with these two) */
  int weights_bf16;   /* 0 = e4m3 weights with block scales.  1 = bf16 weights [E,I,H] without scales (the reference op
                         called with scales = None, python/test/fused_moe_bf16.py:113-122): scale pointers are
                         ignored, act_mode must be B200MOE_ACT_W8A16, tensor-core path only */
  int stages;         /* 0 = the whole call.  Else a mask of B200MOE_STAGE_*: only those stages are enqueued, on
                         a workspace that a whole call with the same sizes and inputs has filled before (how a
                         benchmark times one GEMM alone).  Any other bit is rejected. */
  int max_ctas;       /* 0 = the tensor-core GEMMs use every SM.  n > 0: their persistent grids are capped at n
                         CTAs (one per SM), which leaves the other SMs to kernels of another stream - how the
                         expert-parallel step runs the shared expert beside its dispatch phase. */
} b200moe_experts_desc;

size_t b200moe_experts_workspace_bytes(const b200moe_experts_desc* d);

int b200moe_experts(void* out, const void* x, const void* w_gate, const void* w_up,
                    const void* w_down, const void* s_gate, const void* s_up, const void* s_down,
                    const int32_t* ids, const void* topk_w, const void* shared_w_gate,
                    const void* shared_w_up, const void* shared_w_down, const void* shared_s_gate,
                    const void* shared_s_up, const void* shared_s_down,
                    const b200moe_experts_desc* d, void* workspace, size_t workspace_bytes,
                    int32_t* status, void* stream);

/* Weighted combine on its own (the caller-side bmm of python/regression/test_llm/test_bmm.py:118-134):
 * out[t,:] = bf16( sum_j w[t,j] * y[t,j,:] (+ add[t,:]) ), fp32 accumulation. */
int b200moe_combine(void* out, const void* y, const void* w, int w_dtype, const void* add, int64_t T,
                    int64_t k, int64_t H, void* stream);

/* Same with the rows of y taken through an index: row of pair (t,j) = pos[t*k+j] (pos NULL = t*k+j); a negative
 * pos entry contributes nothing. */
int b200moe_combine_indexed(void* out, const void* y, const int32_t* pos, const void* w, int w_dtype,
                            const void* add, int64_t T, int64_t k, int64_t H, void* stream);
/* Same, and slots whose expert id ids[t*k+j] lies outside [0,E) contribute nothing either (their rows of y were
 * never written: the permutation drops such pairs).  ids NULL = no such check. */
int b200moe_combine_masked(void* out, const void* y, const int32_t* pos, const void* w, int w_dtype, const void* add,
                           const int32_t* ids, int64_t E, int64_t T, int64_t k, int64_t H, void* stream);

/* ---- expert parallelism ------------------------------------------------------------------------------------
 * The reference has no expert-parallel path (its only MoE-adjacent collective is an equal-split all-to-all,
 * torch_tpu/csrc/distributed/c10d/ProcessGroupSCCL.cpp:714-743); these calls are the device side of one:
 * experts sharded contiguously over ranks, tokens data-parallel, rows exchanged by the caller's all-to-all. */

/* The middle of b200moe_experts for callers that dispatch rows themselves: rows xq [R,H] e4m3 ALREADY sorted by
 * (local) expert with group-major scales xs_t [H/128, ld] and expert_offsets[E+1]; gate/up GEMM + SiLU*up +
 * requantise + down GEMM; y row r is written at row_map[r] (row_map NULL = r).  bf16 [*,H]. */
size_t b200moe_grouped_mlp_workspace_bytes(int64_t R, int64_t H, int64_t I, int64_t E, int64_t ld, int scale_dtype);
int b200moe_grouped_mlp(void* y, const uint8_t* xq, const float* xs_t, int64_t ld, const int32_t* expert_offsets,
                        const int32_t* row_map, const void* w_gate, const void* w_up, const void* w_down,
                        const void* s_gate, const void* s_up, const void* s_down, int scale_dtype, int64_t R,
                        int64_t H, int64_t I, int64_t E, int impl, void* workspace, size_t workspace_bytes,
                        int32_t* status, void* stream);

/* Dispatch rows.  A packed row is [H bytes e4m3][H/128 fp32 scales][int32 expert id local to the destination rank]
 * padded to 16 bytes (b200moe_ep_packed_row_bytes).  pack: row p = quantised x[sorted_pair[p]/k] (sorted_pair from
 * b200moe_permute over GLOBAL expert ids, so rows are grouped by destination rank).  unpack_ids: the local expert
 * id of every received row; unpack_rows: received row order[p] -> xq[p,:], xs_t[:, p] (order from b200moe_permute
 * over the received ids with k = 1). */
int64_t b200moe_ep_packed_row_bytes(int64_t H);
int b200moe_ep_pack_rows(uint8_t* rows, const void* x, const int32_t* sorted_pair, const int32_t* ids, int64_t T,
                         int64_t k, int64_t experts_per_rank, int64_t H, void* stream);
int b200moe_ep_unpack_ids(int32_t* eid, const uint8_t* rows, int64_t R, int64_t H, void* stream);
int b200moe_ep_unpack_rows(uint8_t* xq, float* xs_t, int64_t ld, const uint8_t* rows, const int32_t* order,
                           int64_t R, int64_t H, void* stream);
/* inv[perm[i]] = i; entries of perm outside [0,n) are skipped and entries of inv that nothing names are -1 */
int b200moe_invert_permutation(int32_t* inv, const int32_t* perm, int64_t n, void* stream);

/* ---- FP8 block-scaled linear layer ----------------------------------------------------------------------
 * out[M,N] (bf16) = x[M,K] (bf16, quantised per row per 128 columns to e4m3 on the fly) . dequant(w)^T with
 * w [N,K] e4m3 and scale [ceil(N/128), K/128] (fp32 or bf16): the expert GEMM with one expert, no activation
 * and the tensor-core path only.  Stands in for tpudnnMmW8A16DqAsync behind my_ops.mm_w8a16_dq_forward
 * (my_ops/MmW8A16Dq.cpp:185-229), with activations in FP8 instead of bf16.  K % 128 == 0, N % 64 == 0. */
size_t b200moe_linear_workspace_bytes(int64_t M, int64_t K, int64_t N, int scale_dtype);
int b200moe_linear_w8(void* out, const void* x, const void* w, const void* scale, int scale_dtype, int64_t M,
                      int64_t K, int64_t N, void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* FP8 x FP8 product with one scale per operand: out[M,N] = (a[M,K] . b[N,K]^T) * scale_a * scale_b, a and b e4m3,
 * scale_a / scale_b device pointers to ONE fp32 value each (NULL = 1), out bf16 or fp32 (out_dtype).  Stands in for
 * tpudnnMatmulFp8Async behind aten::_scaled_mm on the reference device (native_ops/Scaled_mm.cpp:55-88; mat2 arrives
 * as [N,K] there too, python/test/_scaled_mm.py:8).  Scales multiply, as in torch's own _scaled_mm; the reference's
 * test only ever passes 1 (python/test/_scaled_mm.py:43-44).  K % 128 == 0, N % 64 == 0; tensor-core path only. */
size_t b200moe_scaled_mm_workspace_bytes(int64_t M, int64_t K, int64_t N);
int b200moe_scaled_mm(void* out, int out_dtype, const void* a, const void* b, const float* scale_a,
                      const float* scale_b, int64_t M, int64_t K, int64_t N, void* workspace, size_t workspace_bytes,
                      int32_t* status, void* stream);

/* ---- expert parallelism over peer memory (NVLink) --------------------------------------------------
 * No reference counterpart (the reference has no expert parallelism).  One process per GPU of one node; every
 * rank allocates the same set of buffers, exports them (CUDA IPC) and imports its peers' handles, then builds
 * device arrays of N pointers ("tables", entry r = rank r's buffer, the own entry being the own allocation).
 * A layer call is: exchange_counts -> plan -> dispatch -> barrier -> transpose_scales -> grouped_mlp_remote ->
 * barrier -> combine;
 * all data movement between GPUs is plain peer stores issued by those kernels, and the only waits are flag
 * barriers with a time limit (status bit 2).  `epoch` must grow by one with every barrier (exchange_counts
 * contains one) and take the same values on every rank.  Alternatively pass `epoch_counter`, a device word (zero
 * at start, one per rank): the barrier then uses counter + 1 and advances the counter itself, so the launches carry
 * no per-call value and a whole layer call can be captured into a CUDA graph and replayed.
 *
 * Buffers of one rank, for capacity C rows (C >= the most rows the rank can receive, e.g. N*T*k; with a smaller C the
 * rows that do not fit are dropped by dispatch - status bit 3 - and every later kernel clips its row ranges to C):
 *   flags   uint32 [8]            zero at start            cnt    int32 [N][E]
 *   xq      u8 [C][H]             xs_rows f32 [C][H/128]              src   int32 [C]   (written by the peers)
 *   xs_t    f32 [H/128][ld], ld >= C      (local: the scales in the layout the GEMMs read)
 *   y       bf16 [T*k][H]         per-slot results of the rank's OWN tokens, written by the expert owners */
int b200moe_p2p_alloc(void** ptr, size_t bytes);                 /* device allocation, zero-filled */
int b200moe_p2p_free(void* ptr);
int b200moe_p2p_export(unsigned char* handle64, void* ptr);      /* 64-byte handle another process can import */
int b200moe_p2p_import(void** ptr, const unsigned char* handle64);
int b200moe_p2p_release(void* ptr);                              /* unmap an imported buffer */
int b200moe_p2p_barrier(const uint64_t* flag_tbl, int64_t N, int64_t rank, uint32_t epoch,
                        uint32_t* epoch_counter, int32_t* status, void* stream);
/* expert_offsets [E+1] of the rank's own permutation over GLOBAL expert ids -> row `rank` of every peer's cnt;
 * returns after a barrier, so every rank's cnt is complete for the kernels that follow on the stream */
int b200moe_ep_exchange_counts(const uint64_t* cnt_tbl, const uint64_t* flag_tbl, const int32_t* expert_offsets,
                               int64_t E, int64_t N, int64_t rank, uint32_t epoch, uint32_t* epoch_counter,
                               int32_t* status, void* stream);
/* dst_row0 [E]: first row, in the destination's buffers, of this rank's rows of global expert e;
 * recv_offsets [E/N + 1]: expert_offsets of the rows this rank receives (local experts) */
int b200moe_ep_plan(int32_t* dst_row0, int32_t* recv_offsets, const int32_t* cnt, int64_t E, int64_t N,
                    int64_t rank, void* stream);
/* gather + 1x128 e4m3 quantisation of every (token,slot) row, stored into the owner rank's xq/xs_rows/src
 * (xs_tbl holds the xs_rows buffers; src = rank << 24 | flat pair index t*k+j); H <= 8192 */
int b200moe_ep_dispatch(const uint64_t* xq_tbl, const uint64_t* xs_tbl, const uint64_t* src_tbl, const void* x,
                        const int32_t* sorted_pair, const int32_t* ids, const int32_t* expert_offsets,
                        const int32_t* dst_row0, int64_t T, int64_t k, int64_t H, int64_t E, int64_t N, int64_t rank,
                        int64_t capacity, int32_t* status, void* stream);
/* after the barrier that follows dispatch: xs_t[g][r] = xs_rows[r][g] for r < *n_rows (device value, e.g. the
 * last entry of recv_offsets) */
int b200moe_ep_transpose_scales(float* xs_t, int64_t ld, const float* xs_rows, const int32_t* n_rows, int64_t H,
                                int64_t capacity, void* stream);
/* b200moe_grouped_mlp on the received rows, each result row stored to out_tbl[src >> 24][(src & 0xFFFFFF), :].
 * R_capacity bounds the rows (the true count is read from expert_offsets on the device); tensor-core path only;
 * workspace as b200moe_grouped_mlp_workspace_bytes(R_capacity, ...). */
int b200moe_grouped_mlp_remote(const uint64_t* out_tbl, const int32_t* row_src, const uint8_t* xq, const float* xs_t,
                               int64_t ld, const int32_t* expert_offsets, const void* w_gate, const void* w_up,
                               const void* w_down, const void* s_gate, const void* s_up, const void* s_down,
                               int scale_dtype, int64_t R_capacity, int64_t H, int64_t I, int64_t E, void* workspace,
                               size_t workspace_bytes, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */

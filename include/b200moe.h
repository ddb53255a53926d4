/*
 * b200moe -- C ABI of the sm_100a routed-MoE expert path.
 *
 * Every entry point takes raw device pointers, explicit sizes / pitches and a
 * cudaStream_t (passed as void*), enqueues its kernels on that stream and returns at
 * once: 0 on success or one of the negative B200MOE_ERR_* codes below.  Nothing here
 * allocates, synchronises or throws.  Kernels that can wait on something (the GEMMs) or
 * validate device-side data also take `status`, a device int32[4] block that the
 * caller zeroes once and reads after a synchronisation of its own:
 *   status[0] 0 = fine, 1 = a bounded wait ran out, 2 = malformed offsets / ids
 *   status[1] block index, status[2] where, status[3] detail.
 *
 * "Reference" citations name the function of als244/mlops that the entry point
 * replaces, by path inside that project.
 *
 * Pitches named ld* are in ELEMENTS of the tensor they belong to unless the comment
 * says bytes.  All E4M3 tensors hold torch.float8_e4m3fn bytes.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_OK 0
#define B200MOE_ERR_ARG (-1)       /* null pointer, negative size, unsupported combination */
#define B200MOE_ERR_ALIGN (-2)     /* pointer / pitch alignment requirement not met */
#define B200MOE_ERR_TENSORMAP (-3) /* the driver refused a TMA tensor map for an operand */
#define B200MOE_ERR_LAUNCH (-4)    /* a kernel launch failed */
#define B200MOE_ERR_DRIVER (-5)    /* cuTensorMapEncodeTiled not available */
#define B200MOE_ERR_LIMIT (-6)     /* a size exceeds a documented maximum */

/* Routing modes of b200moe_route_topk. */
#define B200MOE_ROUTE_TOPK_THEN_SOFTMAX 0
#define B200MOE_ROUTE_SOFTMAX_THEN_TOPK 1
#define B200MOE_ROUTE_SIGMOID_NOAUX_TC 2

/* Activation scale granularity of b200moe_quantize_rows. */
#define B200MOE_SCALE_BLOCK128 0 /* one fp32 scale per row and 128-column block */
#define B200MOE_SCALE_ROW 1      /* one fp32 scale per row */

/*
 * Top-k routing from fp32 logits [tokens, experts] (row pitch ld).  Writes
 * weights fp32 [tokens, top_k] and ids int32 [tokens, top_k], picks in descending
 * selection value, ties to the lowest expert id.  `bias` (fp32 [experts], may be NULL),
 * n_group, topk_group and routed_scaling are read in mode SIGMOID_NOAUX_TC only.
 * NaN selection values rank above every number (the order of a stable descending sort), so
 * ids are always K distinct experts in range; the NaN shows in the weights.
 * Limits: experts <= 1024, top_k <= 32, n_group <= 32 when group selection is active.
 * Reference: src/mlops/kernels/moe_router.py:235-344 (`route`).
 */
int b200moe_route_topk(const float* logits, long long ld, int tokens, int experts, int top_k, int mode,
                       const float* bias, int n_group, int topk_group, float routed_scaling,
                       float* weights, int32_t* ids, void* stream);

/*
 * Column sums of the per-token routing probabilities of fp32 logits [tokens, experts] (row pitch
 * ld): softmax of the logits (modes TOPK_THEN_SOFTMAX, SOFTMAX_THEN_TOPK) or sigmoid scores
 * normalised per token (SIGMOID_NOAUX_TC) -> probability_sum fp32 [experts].  Formed in a fixed
 * order (bitwise repeatable).  `workspace` holds
 * b200moe_routing_probability_sum_workspace_bytes(...) bytes.  experts <= 1024.
 * Reference: src/mlops/providers/moe_common.py:32-71 (`routing_statistics`: `probability_sum`;
 * the auxiliary loss is [experts]-sized arithmetic on it and on the sort's counts).
 */
long long b200moe_routing_probability_sum_workspace_bytes(long long tokens, int experts);
int b200moe_routing_probability_sum(const float* logits, long long ld, long long tokens, int experts, int mode,
                                    void* workspace, float* probability_sum, void* stream);

/*
 * Gradient of the logits (fp32 [tokens, experts], pitch ldg) from the cotangents of
 *   the route weights   grad_route_weights fp32 [tokens, top_k] (with ids and, except in mode
 *                       SOFTMAX_THEN_TOPK, the route weights themselves),
 *   the auxiliary loss  grad_aux (device scalar, NULL for none) with frequency fp32 [experts] and
 *                       aux_scale: experts / tokens_total for the softmax modes, 1 / tokens of the
 *                       sequence for the sigmoid mode (call once per sequence, with that sequence's
 *                       rows and frequency),
 *   the probability sum grad_probability_sum fp32 [experts] (NULL for none).
 * Reference: src/mlops/providers/moe_common.py:74-124 (`routing_gradient`),
 * src/mlops/kernels/moe_router.py:403-502 (`route_backward`, `add_aux_gradient_`,
 * `add_sequence_aux_gradient_`).
 */
int b200moe_routing_gradient(const float* logits, long long ld, long long tokens, int experts, int top_k,
                             int mode, const int32_t* ids, const float* route_weights,
                             const float* grad_route_weights, const float* grad_aux, const float* frequency,
                             float aux_scale, const float* grad_probability_sum, float* grad_logits,
                             long long ldg, void* stream);

/*
 * Stable sort of the flat ids [assignments] by expert:
 *   order [assignments] int32, offsets [experts + 1] int32, slots [assignments] int32,
 *   counts64 [experts] int64 (may be NULL).
 * `workspace` must hold b200moe_sort_assignments_workspace_bytes(...) bytes.
 * Limits: experts <= 1024, assignments < 2^31.
 * Reference: src/mlops/kernels/moe_dispatch.py:106-119 (`sort_assignments`).
 */
long long b200moe_sort_assignments_workspace_bytes(long long assignments, int experts);
int b200moe_sort_assignments(const int32_t* ids, long long assignments, int experts, int32_t* order,
                             int32_t* offsets, int32_t* slots, long long* counts64, void* workspace,
                             int32_t* status, void* stream);

/*
 * b200moe_sort_assignments without a workspace argument, for callers that cannot allocate
 * one (a process whose own arena owns all device memory; a call site where cudaMalloc, which
 * may synchronise the device, must not run).  The scratch is a 1 MiB array inside the library
 * image, resident on every GPU that loads the library until exit.  Same outputs as
 * b200moe_sort_assignments.  Limit: ceil(assignments / 4096) * experts <= 262144, else
 * B200MOE_ERR_LIMIT.  No allocation of any kind happens here.  The first call on a device
 * resolves the array's address and should be made outside stream capture.  All calls share
 * the array (its old contents are overwritten before they are read, nothing needs clearing);
 * calls that overlap on the GPU race, so keep them ordered on one stream.
 * This entry point has no counterpart in the reference.
 */
int b200moe_sort_assignments_static(const int32_t* ids, long long assignments, int experts,
                                    int32_t* order, int32_t* offsets, int32_t* slots,
                                    long long* counts64, int32_t* status, void* stream);

/*
 * E4M3 quantisation of bf16 rows, optionally gathered: output row r reads input row
 * gather[r] / gather_div (gather may be NULL: row r) of x [src_rows, width]; an index outside
 * [0, src_rows) is reported in `status` (code 2) and row 0 is read instead.
 * q is [rows, width] bytes with
 * byte pitch ldq; scale of (row r, block b) is written to
 * scales[r * scale_row_stride + b * scale_block_stride] (block b = columns 128b..128b+127;
 * mode B200MOE_SCALE_ROW writes only b = 0).  width % 8 == 0.  `copy` (optional, 1x128 mode)
 * also receives the gathered rows unquantised (bf16 [rows, width], pitch ldc): the operand of
 * a weight gradient, from the same pass over the source.
 * Reference: src/mlops/kernels/quack_moe/quantize_rows.py:140-207 (`quantize_rows_fp8`,
 * per-row); the 1x128 mode applies the same equations per block.
 */
int b200moe_quantize_rows(const void* x, long long ldx, long long src_rows, const int32_t* gather,
                          int gather_div, long long rows, int width, void* q, long long ldq, float* scales,
                          long long scale_row_stride, long long scale_block_stride, int mode, void* copy,
                          long long ldc, int32_t* status, void* stream);

/*
 * The gathered quantisation from the token's side: row t of x [tokens, width] is quantised once
 * (1x128 scales) and written to each of the `fanout` output rows slots[t * fanout + k]
 * (k < fanout <= 32; a slot outside [0, rows_out) is reported in `status` and skipped).  With
 * slots = the sort's inverse permutation this gives exactly the bytes and scales of
 * b200moe_quantize_rows with gather = order, gather_div = fanout, for 1/fanout of the
 * arithmetic and source reads.  `copy` (optional) receives the bf16 rows the same way.
 * Reference: src/mlops/kernels/quack_moe/quantize_rows.py:140-207 (`quantize_rows_fp8` with
 * `gather`), whose result it reproduces.
 */
int b200moe_quantize_rows_scatter(const void* x, long long ldx, long long tokens, const int32_t* slots,
                                  int fanout, long long rows_out, int width, void* q, long long ldq,
                                  float* scales, long long scale_row_stride, long long scale_block_stride,
                                  void* copy, long long ldc, int32_t* status, void* stream);

/*
 * SwiGLU of h13 = [gate | up] (bf16 [rows, 2*width]) computed in fp32 and rounded once
 * to E4M3 with 1x128 scales (act_q, scales) and/or bf16 (act_bf16); either output may be
 * NULL.  `limited` != 0 caps the gate at `limit` and clips up to [-limit, limit].
 * Reference: src/mlops/kernels/quack_moe/swiglu_rows.py:246-256 (`swiglu_quantize_rows_fp8`),
 * clamp semantics src/mlops/kernels/moe_reference.py:12-17.
 */
int b200moe_swiglu_quantize(const void* h13, long long ldh, long long rows, int width, void* act_q,
                            long long ldq, float* scales, long long scale_row_stride,
                            long long scale_block_stride, void* act_bf16, long long lda, float limit,
                            int limited, void* stream);

/*
 * Routed SwiGLU backward.  r = dy_row @ W2 before the route weight (bf16 [rows, width]),
 * score(row) = route_weights[order[row]] (route_weights has n_weights entries; an order entry
 * outside is reported in `status` and entry 0 is used).  Outputs (each may be NULL):
 *   dscore fp32 [rows] = <r, act>; grad_h13 = dSwiGLU(score * r) as E4M3 + 1x128 scales
 *   ([rows, 2*width], needs width % 128 == 0) and/or bf16; act_scaled = score * act (bf16).
 * Reference: src/mlops/kernels/quack_moe/swiglu_rows.py:292-316
 * (`routed_swiglu_rows_backward`).
 */
int b200moe_dswiglu_routed(const void* h13, long long ldh, const void* r, long long ldr,
                           const float* route_weights, long long n_weights, const int32_t* order,
                           long long rows, int width, float* dscore, void* grad_h13_q, long long ldq,
                           float* grad_h13_scales, long long scale_row_stride, long long scale_block_stride,
                           void* grad_h13_bf16, long long ldg, void* act_scaled, long long lda,
                           float limit, int limited, int32_t* status, void* stream);

/*
 * Weight quantisation: w [experts, out, in] (bf16, or fp32 when src_is_fp32) ->
 * q E4M3 same shape, scale fp32 [experts, ceil(out/128), ceil(in/128)].
 * Reference: src/mlops/kernels/block_fp8.py:63-93 (`quantize_blocks`).
 */
int b200moe_quantize_blocks(const void* w, int src_is_fp32, int experts, int out, int in, void* q,
                            float* scale, void* stream);

/*
 * Grouped block-FP8 GEMM, bf16 output.  Rows offsets[g]..offsets[g+1] of A belong to
 * group g:  d[row, :] = (A_q . a_scale)[row, :] @ (B_q . b_scale)[g]^T.
 *   a        E4M3 [rows_total, K], byte pitch lda (multiple of 16)
 *   a_scale  fp32, scale of (row, K block kb) at a_scale[row*as_row_stride + kb*as_kb_stride]
 *            (as_kb_stride = 0 gives one scale per row)
 *   b        E4M3, contiguous; b_mn_major == 0: [groups, N, K] with scales
 *            [groups, ceil(N/128), ceil(K/128)] (the forward products);
 *            b_mn_major != 0: [groups, K, N] with scales [groups, ceil(K/128), ceil(N/128)]
 *            (the stored weight read along its rows: input gradients, no transposed copy)
 *   d        bf16 [rows_total, N], pitch ldd
 *   addend   optional bf16 [rows_total, N] (pitch ldc) added to the fp32 sums before the one
 *            rounding (the LoRA term of a projection); NULL for none
 *   block_n  128 or 256: tile width
 * Every 128-wide K block is accumulated on the tensor cores from zero and promoted in
 * fp32 by a_scale * b_scale.  N % 8 == 0, K % 16 == 0 (N % 16 for b_mn_major),
 * groups <= 1024.  `weights` is the number of weight matrices in b: group g multiplies
 * matrix g % weights (groups must be a multiple of it), so rows that arrive as
 * [source rank][local expert] segments need no regrouping; weights == groups is the plain case.
 * Tile scheduling: launches on an ordinary stream draw their tiles from a device-side counter
 * owned by that stream (up to 64 streams per device get one; launches on one stream never
 * overlap, so a counter is never shared by two running kernels).  Launches into a stream under
 * capture, into the per-thread default stream, or into a 65th stream assign tiles by CTA index
 * instead: same results, no shared state, safe under any graph replay.
 * Reference: src/mlops/kernels/block_fp8.py:249-341 (`grouped_block_gemm`) and
 * src/mlops/kernels/quack_moe/block_fp8_gemm.py:1424-1484 (`block_fp8_gemm`,
 * `block_fp8_transposed_gemm`).
 */
int b200moe_grouped_gemm_fp8(const void* a, long long lda, const float* a_scale, long long as_row_stride,
                             long long as_kb_stride, const void* b, const float* b_scale, void* d,
                             long long ldd, const void* addend, long long ldc, const int32_t* offsets,
                             int groups, int weights,
                             long long rows_total, int N, int K, int b_mn_major, int block_n,
                             int32_t* status, void* stream);

/*
 * b200moe_grouped_gemm_fp8 with a scattered store: d[row_map[r], 0:N] = product[r, 0:N]
 * (row_map: int32 [rows_total], a permutation of the rows that belong to a group; an entry
 * outside [0, rows_total) is reported in `status` and that row is not stored).  The
 * expert-parallel layer multiplies received rows in expert order and gives them back in the
 * [source rank][expert] order the return exchange wants, without a pass of its own.
 * No counterpart in the reference (its transport returns rows through MoonEP's own buffers,
 * src/mlops/expert_parallel/quack/layer.py).
 */
int b200moe_grouped_gemm_fp8_scatter(const void* a, long long lda, const float* a_scale,
                                     long long as_row_stride, long long as_kb_stride, const void* b,
                                     const float* b_scale, void* d, long long ldd, const int32_t* row_map,
                                     const void* addend, long long ldc, const int32_t* offsets, int groups,
                                     int weights, long long rows_total, int N, int K, int b_mn_major,
                                     int block_n, int32_t* status, void* stream);

/*
 * The up projection with its SwiGLU fused into the GEMM epilogue: one kernel writes
 *   h13   bf16 [rows_total, 2F] (pitch ldh): gate columns then up columns, the residual the
 *         backward pass reads, and
 *   act_q E4M3 [rows_total, F] (byte pitch ldq) = silu(gate) * up (from the bf16 values of h13,
 *         fp32 math, GLM clamp when `limited`), with one fp32 scale per row and 128 columns at
 *         act_scale[row*acts_row_stride + block*acts_block_stride].
 * b is w13 [weights, 2F, K] (gate rows then up rows) with its 128x128 scales; the other
 * arguments are those of b200moe_grouped_gemm_fp8.  F % 128 == 0.
 * Reference: src/mlops/kernels/quack_moe/block_fp8_gemm.py:1484 (`block_fp8_gemm_swiglu`),
 * epilogue :1195-1206; dispatch src/mlops/providers/sonicmoe/block_fp8.py:114-125.
 */
int b200moe_grouped_gemm_fp8_swiglu(const void* a, long long lda, const float* a_scale,
                                    long long as_row_stride, long long as_kb_stride, const void* b,
                                    const float* b_scale, void* h13, long long ldh, void* act_q, long long ldq,
                                    float* act_scale, long long acts_row_stride, long long acts_block_stride,
                                    const int32_t* offsets, int groups, int weights, long long rows_total,
                                    int F, int K, float limit, int limited, int32_t* status, void* stream);

/*
 * The down projection with the un-permute / combine fused into its store: instead of bf16
 * expert-order rows the kernel adds, with 16-byte fp32 atomics,
 *   out_f32[row_token[r], 0:N] += row_weight[r] * bf16(product[r, 0:N])
 * (the product rounded to bf16 first, as the stored expert output would be).  out_f32
 * [tokens, N] (pitch ldo floats, a multiple of 4) must hold each token's starting value (zero);
 * row_token / row_weight give, per expert-order row, its token and route weight (a token outside
 * [0, tokens) is reported in `status` and its row is not added).  The other
 * arguments are those of b200moe_grouped_gemm_fp8 (tile width 256).  The K contributions of a
 * token arrive in no fixed order: results are not bitwise repeatable, which is why the
 * two-kernel form (b200moe_grouped_gemm_fp8 + b200moe_combine) is the default.
 * b200moe_finish_combine then writes out[t] = bf16(sums[t] + residual[t]) (residual may be NULL).
 * Reference: src/mlops/kernels/moe_dispatch.py:168-196 (`combine`) after
 * src/mlops/kernels/block_fp8.py:249-341; the fused form is the one
 * src/mlops/providers/sonicmoe names `down projection + scatter`.
 */
int b200moe_grouped_gemm_fp8_combine(const void* a, long long lda, const float* a_scale,
                                     long long as_row_stride, long long as_kb_stride, const void* b,
                                     const float* b_scale, float* out_f32, long long ldo, long long tokens,
                                     const int32_t* row_token, const float* row_weight, const void* addend,
                                     long long ldc, const int32_t* offsets, int groups, int weights,
                                     long long rows_total, int N, int K, int b_mn_major, int32_t* status,
                                     void* stream);
int b200moe_finish_combine(const float* sums, long long lds, const void* residual, long long ldr, void* out,
                           long long ldo, long long tokens, int width, void* stream);

/*
 * Process-wide cap on the CTAs the persistent tensor-core kernels launch (they launch one CTA
 * per SM and leave no room for another kernel on an SM they occupy).  A caller that overlaps
 * them with communication kernels keeps a few SMs free: ctas = SM count - reserved; 0 restores
 * "every SM".  The reference's expert-parallel runtime reserves SMs for its transport the same
 * way (src/mlops/expert_parallel/quack/config.py, `num_sms`).
 */
int b200moe_set_cta_limit(int ctas);

/*
 * Which form of the wide-tile FP8 GEMM serves b200moe_grouped_gemm_fp8[_scatter]:
 *   mode -1 (default), 0  the single-CTA form (tiles drawn from a counter: CTAs that start late,
 *                         because a collective holds their SM, take fewer tiles)
 *   mode  1               the CTA-pair form (clusters of two CTAs on a 256 x 256 tile,
 *                         tcgen05.mma.cta_group::2, tiles assigned by pair index) whenever it can
 *                         serve the call (block_n 256, no CTA limit)
 * Both forms give bit-identical results; the single-CTA form measured faster at every shape tried,
 * so the pair form is opt-in.  Process-wide, like b200moe_set_cta_limit.  The reference picks its
 * tile shapes per token bucket in the same spirit (src/mlops/kernels/quack_moe/policy.py:52-150).
 */
int b200moe_set_gemm_pair(int mode);

/*
 * Rank-r side products of expert LoRA on expert-sorted rows (rank <= 64, bf16, fp32 sums).
 * project: t[row, 0:rank] = x[row, 0:K] . W_e, with W [experts, rank, K] (rank_major != 0) or
 *          [experts, K, rank].  expand: c[row, 0:N] = scale * t[row, 0:rank] . W_e, with
 *          W [experts, N, rank] (wide_major != 0) or [experts, rank, N].  W_e is the factor of
 *          the expert that owns the row (offsets as in the GEMMs, experts <= 1024).
 * Reference: src/mlops/lora/grouped.py:19-110 (`grouped_linear` on the factors),
 * src/mlops/lora/experts.py:140-167.
 */
int b200moe_lora_project(const void* x, long long ldx, const void* w, int rank_major,
                         const int32_t* offsets, int experts, long long rows, int K, int rank, void* t,
                         long long ldt, void* stream);
int b200moe_lora_expand(const void* t, long long ldt, const void* w, int wide_major, const int32_t* offsets,
                        int experts, long long rows, int N, int rank, float scale, void* c, long long ldc,
                        void* stream);

/*
 * Grouped weight gradient: out[g] (M x N) = G[rows of g, 0:M]^T @ X[rows of g, 0:N],
 * bf16 operands (pitches ldg, ldx), fp32 sums, out [groups, M, N] contiguous in bf16 or
 * fp32 (out_is_fp32).  Groups without rows get zeros.  M % 8 == 0, N % 8 == 0.
 * `offsets` holds segments*groups + 1 entries: group g sums over the row ranges
 * offsets[s*groups+g] .. offsets[s*groups+g+1] for s < segments (segments == 1 is the plain
 * expert-sorted layout; with rows laid out [source rank][local expert] it is the rank count).
 * Reference: src/mlops/kernels/moe_grouped_gemm.py:300-342 (`grouped_mm_wgrad`).
 */
int b200moe_grouped_wgrad_bf16(const void* g, long long ldg, const void* x, long long ldx,
                               const int32_t* offsets, int groups, int segments, long long rows_total,
                               int M, int N, void* out, int out_is_fp32, int32_t* status, void* stream);

/*
 * The same product written into a gradient buffer the caller keeps across calls:
 *   out[g] = out[g] + scale * G[rows of g]^T @ X[rows of g]      (fp32, one rounding)
 * so the gradients of several micro-batches accumulate in place, with an explicit gradient
 * scale folded into the GEMM's store, and no separate add pass runs.  Groups without rows
 * leave their block untouched.
 * Reference: src/mlops/providers/sonicmoe/lora_destinations.py:28-432 (destinations for
 * parameter-gradient products: accumulate in the GEMM epilogue, explicit gradient scale).
 */
int b200moe_grouped_wgrad_bf16_accumulate(const void* g, long long ldg, const void* x, long long ldx,
                                          const int32_t* offsets, int groups, int segments,
                                          long long rows_total, int M, int N, void* out, int out_is_fp32,
                                          float scale, int32_t* status, void* stream);

/*
 * bf16 grouped GEMM of the bf16 compute path (fp32 sums in TMEM over the whole K loop):
 *   d[rows of g, 0:N] = alpha * a[rows of g, 0:K] @ op(b[g % weights])  (+ addend), rounded once to bf16
 * b_mn_major = 0: b is [weights, N, K] (y = x W^T on the stored nn.Linear weight);
 * b_mn_major = 1: b is [weights, K, N] read along its rows (dx = dy W on the SAME stored weight
 * [out = K, in = N]; no transposed copy).  N, K and the pitches are multiples of 8; either may be as
 * small as 8 (the rank-r products of expert LoRA run on this kernel: the unused part of a tile is
 * zero-filled by the TMA unit and costs no memory traffic).
 * Reference: src/mlops/kernels/moe_grouped_gemm.py:201-299 (`grouped_mm_forward`,
 * `grouped_mm_dgrad`; CPU form `_native_torch` :185-198).
 */
int b200moe_grouped_gemm_bf16(const void* a, long long lda, const void* b, void* d, long long ldd,
                              const void* addend, long long ldc, const int32_t* offsets, int groups, int weights,
                              long long rows_total, int N, int K, int b_mn_major, float alpha, int32_t* status,
                              void* stream);

/*
 * Expert-parallel dispatch as one kernel: gather + transfer over NVLink peer memory.  Send row i
 * is the bf16 row src[gather[i]]; send rows [send_start[r], send_start[r+1]) belong to rank r and
 * are written, in order, from row dest_row0[r] of dest[r] on: dest[r] is rank r's receive arena as
 * mapped into THIS process (symmetric / peer memory; r == own rank: a local pointer).  Plain
 * 16-byte stores; the kernel waits for nobody.  The caller orders the ranks afterwards (any
 * collective on the same stream) before an arena is read, and before one is written again.
 * world <= 16.  (No reference counterpart: the reference's transport is MoonEP, a third-party
 * library, src/mlops/expert_parallel/quack/communication.py; its plan -- send once per
 * destination rank, receive grouped by source -- is the same.)
 */
int b200moe_peer_dispatch_rows(const void* src, long long lds, long long src_rows, const int32_t* gather,
                               long long rows, int width, void* const* dest, long long ldd, long long dest_rows,
                               const int32_t* send_start, const long long* dest_row0, int world, int32_t* status,
                               void* stream);

/*
 * The sender's plan of a de-duplicated expert-parallel dispatch, in one launch: one copy of a token
 * per rank holding at least one of its experts (rank = keys[t, k] / local), ordered by rank, then
 * token.  copy_start (HOST array, world + 1 entries): where each rank's copies begin.  Outputs:
 * token_of [copies], meta [copies, 2 * top_k] = [local expert id or -1 | route weight bits or 0],
 * token_copies [tokens, world] = position of the token's copy for each rank or -1.
 * Reference: src/mlops/expert_parallel/quack/runtime.py:93-108 (the dispatch plan, "dedup").
 */
int b200moe_build_copies(const int32_t* keys, const float* weights, int tokens, int top_k, int world, int local,
                         const int32_t* copy_start, int32_t* token_of, int32_t* meta, int32_t* token_copies,
                         int32_t* status, void* stream);

/*
 * E4M3 rows of x [rows, width] (bf16, token-major) with ONE SCALE PER (GROUP, COLUMN):
 *   scales[g, c] = max(max over the rows of group g of |x[r, c]| * fp32(1/448), 1e-12)
 *   q[r, c]      = e4m3_rn(clamp(x[r, c] / scales[g(r), c], -448, 448))     (RN division)
 * `offsets` holds segments * groups + 1 ascending row boundaries; range i belongs to group
 * i % groups (segments = 1: the sort's offsets).  The output stays token-major: the FP8 weight
 * gradient reads it MN-major, no transpose is stored.  A group without rows gets scale 1e-12.
 * Reference: src/mlops/kernels/quack_moe/quantize_transpose.py:126-133 (per-feature scales of an
 * expert's token block, the row quantiser's equations applied to a column); the reference's
 * implementation is a Triton kernel that also stores the transpose.
 */
int b200moe_quantize_columns(const void* x, long long ldx, long long rows, int width, const int32_t* offsets,
                             int groups, int segments, void* q, long long ldq, float* scales, void* stream);

/*
 * Weight gradient from E4M3 operands:
 *   out[g] (M x N) (+)= scale * (g_scale[g, :, None] * x_scale[g, None, :]) * (Gq[rows of g]^T @ Xq[rows of g])
 * Gq [rows_total, M] and Xq [rows_total, N] are column-scaled E4M3 (b200moe_quantize_columns),
 * multiplied on the tensor cores at the FP8 rate with fp32 sums over ALL rows of the group (the
 * scales do not vary along the contraction, so nothing is promoted in between); accumulate != 0
 * adds to what `out` holds.  M, N and both pitches are multiples of 16.
 * Reference: src/mlops/kernels/quack_moe/wgrad.py:30-69 (`expert_weight_gradient`).
 */
int b200moe_grouped_wgrad_fp8(const void* g, long long ldg, const float* g_scale, const void* x, long long ldx,
                              const float* x_scale, const int32_t* offsets, int groups, int segments,
                              long long rows_total, int M, int N, void* out, int out_is_fp32, float scale,
                              int accumulate, int32_t* status, void* stream);

/*
 * out[t] = residual[t] + sum_k weights[t,k] * src[slots[t,k]] (fp32 sums, k ascending, one
 * rounding).  weights NULL = 1, residual NULL = 0.  All row tensors bf16.  A negative slot adds
 * nothing (the expert-parallel layer's "this assignment lives on another rank").
 * Reference: src/mlops/kernels/moe_dispatch.py:136-196 (`combine`, `dispatch_backward`).
 */
int b200moe_combine(const void* src, long long lds, long long src_rows, const int32_t* slots,
                    const float* weights, const void* residual, long long ldr, void* out, long long ldo,
                    long long tokens, int width, int top_k, void* stream);

/*
 * dst[r] = src[gather[r] / gather_div], bf16 rows of src [src_rows, width].  An index outside
 * [0, src_rows) is reported in `status` (code 2) and row 0 is copied instead.
 * Reference: src/mlops/kernels/moe_dispatch.py:122-124 (`dispatch`).
 */
int b200moe_gather_rows(const void* src, long long lds, long long src_rows, const int32_t* gather,
                        int gather_div, long long rows, int width, void* dst, long long ldd,
                        int32_t* status, void* stream);

/*
 * out[i] = values[slots[i]] for i < n (fp32): a per-sorted-row scalar in assignment order.
 * values has n_values entries; a slot outside is reported in `status` and entry 0 is read.
 * Reference: src/mlops/providers/moe_common.py:325-329 (route-weight gradient gather).
 */
int b200moe_gather_scalar(const float* values, long long n_values, const int32_t* slots, long long n,
                          float* out, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */

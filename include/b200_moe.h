/*
 * C ABI of libb200moe.so: the routed MXFP4 x MXFP4 MoE block (hidden 6144, intermediate 768, up to 128 experts, top-4)
 * as hand-written sm_100a kernels. Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (passed as void*, a cudaStream_t), launches on that stream without synchronising, allocates nothing unless stated, and
 * returns an int status: 0 = launched, negative = rejected argument (B200MOE_E_*), positive = CUDA runtime error code.
 * Device-side conditions (a bounded wait that ran out) are reported through the caller-provided `status` word, which a
 * kernel sets to a non-zero B200MOE_DEV_* code and never clears; callers zero it before a call and read it after a sync.
 *
 * Each function names the reference interface it replaces, as path:line inside the amd-kernels project with
 * MOE/ = amd_kernels/moe/mxfp4_h6144_i768_e128_top4/.
 *
 * Data formats
 *   E2M1 codes: two per byte along K, even element in the low nibble; code = index into {0,.5,1,1.5,2,3,4,6} | sign<<3.
 *   E8M0 scales: one byte per 32 elements along K, value 2^(byte-127).
 *   "scale atom": 512 bytes holding 4 consecutive scale bytes of up to 128 rows, byte (r%32)*16 + (r/32)*4 + j for row r
 *   and scale j -- the image tcgen05.cp.32x128b.warpx4 moves to tensor memory in one instruction.
 *   "tile record": one weight tile of 128 rows x 256 K-elements as 17408 consecutive bytes: 16384 bytes of codes in the
 *   128-byte-swizzled shared-memory image (row r, 16-byte chunk c at r*128 + ((c ^ (r&7))*16)) followed by the tile's two
 *   scale atoms. Preshuffled W13 = [E][12 tiles][24 K-tiles] records, tile t row r holding gate (r/32 even) or up (r/32
 *   odd) row 64*t + 32*(r/64) + r%32 of the checkpoint (gate rows 0..767, up rows 768..1535); preshuffled W2 =
 *   [E][48 tiles][3 K-tiles] records in checkpoint row order. Activation scales: [row block][K/128 atoms].
 *   Sorted rows: (token, slot) pairs grouped by expert ascending, pair order 4*token+slot inside an expert, every expert
 *   padded to a multiple of bm rows; sorted_ids = token | slot<<24, padding rows carry token = T and weight 0.
 */
#ifndef B200_MOE_H
#define B200_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_H 6144
#ifndef B200MOE_I /* intermediate size of the build: 768 (libb200moe.so) or 1536 (libb200moe_i1536.so, the TP2 sibling shape) */
#define B200MOE_I 768
#endif
#define B200MOE_E 128
#define B200MOE_TOPK 4
#define B200MOE_MAX_TOKENS 87381 /* MOE/chain.py:13-18, variant_for rejects more */

#define B200MOE_E_ARG (-1)     /* null pointer, size out of range, unsupported bm */
#define B200MOE_E_ALIGN (-2)   /* a pointer that must be 16-byte (workspace: 256-byte) aligned is not */
#define B200MOE_E_DRIVER (-3)  /* the CUDA driver entry point for tensor maps is unavailable */
#define B200MOE_E_TOO_LARGE (-4) /* more tokens than the allocation-free entry point's built-in scratch holds */
#define B200MOE_STATIC_SORT_MAX_TOKENS 8192
#define B200MOE_DEV_TIMEOUT 1  /* a bounded mbarrier wait ran out inside a kernel */
#define B200MOE_DEV_BAD_INDEX 2 /* a block count or expert id read from the routing table was out of range */

#define B200MOE_ROUTE_SIGMOID_BIAS 0 /* the reference's rule */
#define B200MOE_ROUTE_SOFTMAX 1      /* softmax, top-4, renormalised over the picks */

/* Library version and the SM architecture it was built for ("sm_100a"). */
int b200moe_version(void);
const char* b200moe_arch(void);

/* Upper bound of padded sorted rows for T tokens and block height bm (MOE/common/sort.py:19-23, max_sorted_rows). */
int64_t b200moe_max_sorted_rows(int64_t tokens, int bm, int num_experts);

/* Block height the library picks for T tokens: 16 / 32 / 64 / 128 (role of MOE/chain.py:13-18 DISPATCH, by size only). */
int b200moe_block_rows(int64_t tokens);

/* Weight preshuffle, once at load time (MOE/chain.py:41-50 MoeWeights.from_row_major; MOE/layout.py:24-38 w13_layout,
 * w2_layout; MOE/prefill_h6144_i768.py:34-45 Mxfp4PrefillScales.from_row_major). Checkpoint tensors in, tile records
 * out (see "Data formats"): w13t [E][12][24][17408], w2t [E][48][3][17408]; all device pointers, 16-byte aligned. */
int b200moe_preshuffle_w13(const uint8_t* w13, const uint8_t* w13_scale, int num_experts, uint8_t* w13t, void* stream);
int b200moe_preshuffle_w2(const uint8_t* w2, const uint8_t* w2_scale, int num_experts, uint8_t* w2t, void* stream);

/* Router GEMM (MOE/router_gemm.py:390-467 router_gemm_partials; oracle MOE/reference.py:101-111): x bf16 [T][6144] times the
 * fp32 gate [num_experts][6144] as split-K partials fp32 [splits][T][num_experts] (partial s covers K elements
 * [s*6144/splits, (s+1)*6144/splits)); each partial is within 2^-18 * sum|x||w| of the exact product, results are the
 * same on every run. b200moe_router_splits(T) is the split count the library uses (16 up to 2048 tokens, 4 above). Feed
 * the partials to b200moe_route_topk with stride_t = num_experts, stride_s = T*num_experts. */
int b200moe_router_splits(int64_t tokens);
int b200moe_router_gemm(const void* x_bf16, const float* gate, int64_t tokens, int num_experts, int splits,
                        float* partials, void* stream);

/* The same partials on the tensor cores, for 128 tokens and more (MOE/router_gemm.py:32-44 _split3, :48-290 the bf16x3
 * MMA kernel): b200moe_router_split_gate turns the fp32 gate into its three bf16 terms RN(w), RN(w - w0), RN(w - w0 - w1)
 * once at load time (split_bf16: bf16 [3][128][6144], rows from num_experts on zero); b200moe_router_gemm_tc multiplies
 * with tcgen05.mma kind::f16 into fp32 accumulators. Same layout and the same error bound as b200moe_router_gemm (the
 * bits differ: the sum runs in another order); splits must divide 96. `status` as in the grouped GEMMs. */
int b200moe_router_split_gate(const float* gate, int num_experts, void* split_bf16, void* stream);
int b200moe_router_gemm_tc(const void* x_bf16, const void* gate_split_bf16, int64_t tokens, int num_experts, int splits,
                           float* partials, int32_t* status, void* stream);

/* The router GEMM fused with the input quantisers: one pass over x writes the split-K partials as above and, row-major,
 * the routed experts' MXFP4 operands (codes4 [T][3072], scales4 [T][192], the bits of b200moe_quant_mxfp4) and, when
 * codes8 / scales8 are given, the shared expert's MXFP8 operands ([T][6144], [T][192], the bits of
 * b200moe_shared_quant_rows) (MOE/router_mxfp4_quant_line_layout.py:48-400,
 * MOE/router_mxfp4_mxfp8_quant_row_scales.py router_mxfp4_mxfp8_quant_row_scales). */
int b200moe_router_gemm_quant(const void* x_bf16, const float* gate, int64_t tokens, int num_experts, int splits,
                              float* partials, uint8_t* codes4, uint8_t* scales4, uint8_t* codes8, uint8_t* scales8,
                              void* stream);

/* Router top-4 (MOE/router_topk.py:239-272 splitk_biased_topk). logits[t][e] = sum over s<S of
 * partials[t*stride_t + s*stride_s + e], added from 0.0 in split order; plain logits are S=1. mode SIGMOID_BIAS:
 * s = sigmoid(logit), choice = s + bias[e], weight = s*scale / sum of the 4 chosen s. mode SOFTMAX: choice = logit,
 * weight = scale * exp(l - max) / sum over the 4 picks. Picks are in descending choice order, exactly equal choices go
 * to the lower expert id. bias may be null (zero). out_w fp32 [T][4], out_ids int32 [T][4]. */
int b200moe_route_topk(const float* partials, int64_t stride_t, int64_t stride_s, int splits, const float* bias,
                       int64_t tokens, int num_experts, int mode, float scale, float* out_w, int32_t* out_ids,
                       void* stream);

/* Activation quantisation bf16 [T][K] -> codes [T][K/2], scales [T][K/32], row-major, bit-exact "Quark even" rule
 * (MOE/quant.py:32-106 mxfp4_quant; oracle MOE/reference.py:32-46). K is a multiple of 256. */
int b200moe_quant_mxfp4(const void* x_bf16, int64_t tokens, int k, uint8_t* codes, uint8_t* scales, void* stream);

/* Routing sort (MOE/common/sort.py:19-65 SortBuffers; MOE/sort_a16w4.py:217-242 moe_sort_a16w4;
 * MOE/common/sort_count_all.py:188 moe_sort_count_all). ids/w [T][4] -> sorted_ids int32 [max_rows], sorted_w fp32
 * [max_rows], block_expert int32 [max_rows/bm], num_valid int32 [2] = {padded rows, first row of the last non-empty
 * expert}. `scratch` is int32 [ceil(4T/1024)][num_experts], needed only when 4T > 1024 (b200moe_permute_scratch_bytes).
 * bm is 16, 32, 64 or 128; bm = 1 (no padding, block_expert = one entry per row) groups pairs by an arbitrary small key. */
size_t b200moe_permute_scratch_bytes(int64_t tokens, int num_experts);
int b200moe_permute(const int32_t* ids, const float* w, int64_t tokens, int num_experts, int bm, int32_t* sorted_ids,
                    float* sorted_w, int32_t* block_expert, int32_t* num_valid, int32_t* scratch, void* stream);

/* b200moe_permute over the first *live_pairs pairs only (a device int32; null = all 4*tokens): pairs from there on are
 * ignored whatever their expert id. For buffers that are sorted at their full capacity while the number of filled rows is
 * known on the device only (the expert-parallel receive buffers). No counterpart in the reference. */
int b200moe_permute_live(const int32_t* ids, const float* w, int64_t tokens, int num_experts, int bm,
                         const int32_t* live_pairs, int32_t* sorted_ids, float* sorted_w, int32_t* block_expert,
                         int32_t* num_valid, int32_t* scratch, void* stream);

/* The routing sort for callers that cannot allocate device memory (no counterpart in the reference, whose hosts allocate
 * every scratch buffer with torch.empty). Same inputs, outputs and results as b200moe_permute, but the chunk-count scratch
 * is a 16 KB array inside the library image instead of a caller buffer; the call performs no cudaMalloc / cudaFree and
 * calls no allocating routine. Limit: tokens <= B200MOE_STATIC_SORT_MAX_TOKENS (8192), otherwise B200MOE_E_TOO_LARGE.
 * Every GPU that loads the library holds the array until the process exits. The first call on a device looks up the
 * array's device address (that device must be current, and `stream` must belong to it): make that first call before any
 * stream capture begins. All calls on one device share the array and it keeps the previous call's contents (nothing in
 * it needs clearing: the count pass overwrites every entry the placement pass reads), so two calls that overlap on the
 * GPU -- different streams, no ordering between them -- race; order them or use b200moe_permute with separate scratch. */
int b200moe_permute_static(const int32_t* ids, const float* w, int64_t tokens, int num_experts, int bm,
                           int32_t* sorted_ids, float* sorted_w, int32_t* block_expert, int32_t* num_valid, void* stream);

/* How long a wait inside a kernel (on an mbarrier, or on the completion count of b200moe_gemm12) may last before the
 * kernel gives up, sets status = B200MOE_DEV_TIMEOUT, lets its copies land, frees its tensor memory and returns
 * (the bounded form of the reference's wait_ready, MOE/a16w4_utils.py:44-61, which spins without a limit). Default
 * 2,000,000,000 ns. Applies to the CURRENT device and to kernels launched after the call; synchronous. */
int b200moe_set_wait_limit_ns(uint64_t ns);

/* b200moe_route_sort on split-K partials (layout as in b200moe_route_topk), added in split order. */
int b200moe_route_sort_partials(const float* partials, int64_t stride_t, int64_t stride_s, int splits, const float* bias,
                                int64_t tokens, int num_experts, int mode, float scale, int bm, float* out_w,
                                int32_t* out_ids, int32_t* sorted_ids, float* sorted_w, int32_t* block_expert,
                                int32_t* num_valid, int32_t* scratch, void* stream);

/* Router top-4 on plain fp32 logits [T][num_experts] followed by the routing sort; one single-CTA kernel up to 32
 * tokens, b200moe_route_topk + b200moe_permute above (the fused top-k + sort of the reference's small tier,
 * MOE/router_topk_sorted.py:43). Outputs of both. */
int b200moe_route_sort(const float* logits, const float* bias, int64_t tokens, int num_experts, int mode, float scale,
                       int bm, float* out_w, int32_t* out_ids, int32_t* sorted_ids, float* sorted_w,
                       int32_t* block_expert, int32_t* num_valid, int32_t* scratch, void* stream);

/* Gather of quantised token rows into sorted order with the scales laid out as atoms (the activation-scale gather of
 * MOE/common/scale_sort_tile_map.py:253 scale_sort_tile_map, plus the row gather the reference does inside GEMM1,
 * MOE/gemm1_prefill_h6144_i768.py:209-228). xq_sorted [max_rows][3072], sfx [max_rows/bm][48][512]; padding rows are
 * written as zero codes with scale byte 1 (the byte of an all-zero block). by_pair != 0: codes/scales hold one row per (token, slot) pair, row
 * 4*token+slot (rows that arrived from other ranks), instead of one row per token. */
int b200moe_dispatch_rows(const uint8_t* codes, const uint8_t* scales, const int32_t* sorted_ids,
                          const int32_t* num_valid, int64_t tokens, int bm, int by_pair, int64_t max_rows,
                          uint8_t* xq_sorted, uint8_t* sfx, void* stream);

/* Quantisation fused with the gather: bf16 x [T][6144] -> xq_sorted / sfx as above, same bits as b200moe_quant_mxfp4
 * followed by b200moe_dispatch_rows
 * (the fused router + quant launches of the reference, MOE/router_topk_mxfp4_mxfp8_quant.py:35). `done` (may be null):
 * int32 [max_rows/bm], zeroed by this kernel for a following b200moe_gemm12. */
int b200moe_quant_dispatch(const void* x_bf16, const int32_t* sorted_ids, const int32_t* num_valid, int64_t tokens,
                           int bm, int64_t max_rows, uint8_t* xq_sorted, uint8_t* sfx, int32_t* done, void* stream);

/* Expert-parallel send plan on the device (no counterpart in the reference, which has no expert parallelism).
 * b200moe_ep_dest: ids int32 [T][4] -> dest int32 [4T] (the rank that owns each pair's expert: id / experts_per_rank, or
 * id % world when interleaved) and counts int64 [world] (pairs per destination). After the ranks exchanged their counts,
 * b200moe_ep_offsets turns matrix int64 [world][world] (matrix[s][d] = pairs from s to d) into this rank's seg_start int32
 * [world], dst_base int64 [world] (the arguments of b200moe_quant_push) and recv_pairs int32 [1] (the pairs it receives). */
int b200moe_ep_dest(const int32_t* ids, int64_t tokens, int world, int experts_per_rank, int interleaved, int32_t* dest,
                    int64_t* counts, void* stream);
int b200moe_ep_offsets(const int64_t* matrix, int world, int rank, int32_t* seg_start, int64_t* dst_base,
                       int32_t* recv_pairs, void* stream);

/* Expert parallel: one ordering point between the ranks of a node, over peer mappings instead of a collective call.
 * peer_flags[r]: rank r's flag array (int32 [world], zero at start, writable by every rank); the launch stores this rank's
 * next epoch into slot `rank` of every peer's array and waits (bounded: status B200MOE_DEV_TIMEOUT) until every slot of its
 * own array has reached it. `epoch_counter`: a device int32 local to the rank, zero at start, advanced by the launch (so the
 * call can be captured in a CUDA graph); the ranks must make the same sequence of calls. With `my_counts` (int64 [world],
 * rows this rank sends to every rank) and peer_matrices[r] (rank r's int64 [world][world]): also stores the counts as row
 * `rank` of every peer's matrix before the flag, which replaces the all-gather of the send plan. (The reference's own
 * collectives order their ranks with flags in IPC pools the same way: amd_kernels/collectives/pull_collectives_ranks4/
 * kernel.py:3-20.) */
int b200moe_ep_sync(void* const* peer_flags, void* const* peer_matrices, const int64_t* my_counts, int world, int rank,
                    int32_t* epoch_counter, int32_t* status, void* stream);

/* Expert-parallel dispatch fused with the activation quantisation (no counterpart in the reference; its multi-GPU input
 * hand-off is the all-gather of prepared inputs, MOE/prepared_input.py:116-209). send_ids / send_w / send_rank describe
 * this rank's 4T pairs grouped by destination rank (b200moe_permute on the destination ranks with bm = 1: sorted_ids,
 * sorted_w, block_expert). Send row i goes to row dst_base[d] + (i - seg_start[d]) of destination d's receive buffers
 * (dst_base int64 [world] and seg_start int32 [world] are DEVICE arrays, so the row counts never have to reach the host):
 * peer_codes[d] u8 [capacity][3072], peer_scales[d] u8 [capacity][192] (row-major, bit-identical to b200moe_quant_mxfp4
 * of the token's row), peer_meta[d] int32 [4][capacity] = column arrays of {expert id local to d, routing-weight
 * bits, source pair 4*token+slot, source rank}. Pointers are device pointers valid on this GPU (peer mappings over NVLink; this rank's own
 * buffers at index `rank`); world <= 8. Rows outside [0, capacity) are not stored and set status = B200MOE_DEV_BAD_INDEX. */
int b200moe_quant_push(const void* x_bf16, const int32_t* ids, const int32_t* send_ids, const float* send_w,
                       const int32_t* send_rank, int64_t tokens, int world, int rank, int experts_per_rank,
                       int interleaved, void* const* peer_codes, void* const* peer_scales, void* const* peer_meta,
                       const int64_t* dst_base, const int32_t* seg_start, int64_t capacity, int32_t* status, void* stream);

/* Grouped GEMM1 + SwiGLU-OAI + MXFP4 requantisation on tcgen05 block-scaled FP4 MMA
 * (MOE/gemm1_prefill_h6144_i768.py:71-898, MOE/gemm1_a4w4_small.py:75-164; oracle MOE/reference.py:66-72).
 * hq [max_rows][384] codes of h in sorted-row order, sfh [max_rows/bm][6][512] scale atoms. All pointers 16-byte
 * aligned. `status` (device int32) receives B200MOE_DEV_* codes. `prefetch_w2t` (may be null): the W2 tile records;
 * each CTA, once its own weight stream has ended, then asks L2 for the tiles a following GEMM2 reads first. */
int b200moe_gemm1_swiglu_quant(const uint8_t* w13t, int num_experts, const uint8_t* xq_sorted, const uint8_t* sfx,
                               const int32_t* block_expert, const int32_t* num_valid, int64_t max_rows, int bm,
                               uint8_t* hq, uint8_t* sfh, const uint8_t* prefetch_w2t, int32_t* status, void* stream);

/* The same GEMM1 at block height 128 on CTA pairs: a cluster of two CTAs issues tcgen05.mma.cta_group::2 of 256 token rows
 * (two row blocks of one expert) x 256 weight rows (two W13 tiles), each CTA staging its own half of both operands, so
 * shared memory moves half the bytes per flop (the role of the reference's persistent prefill kernel at its widest tile,
 * MOE/gemm1_prefill_h6144_i768.py:560-598 K-loop, :689-768 epilogue). Same inputs, outputs and bits as
 * b200moe_gemm1_swiglu_quant with bm = 128. b200moe_gemm1_pair_supported(): 1 when the current device can launch it.
 * b200moe_gemm1_swiglu_quant_wide: the same 256-column unit on one CTA (128 token rows x 256 weight rows per MMA, every
 * row block a unit), same bits again. */
int b200moe_gemm1_swiglu_quant_wide(const uint8_t* w13t, int num_experts, const uint8_t* xq_sorted, const uint8_t* sfx,
                                    const int32_t* block_expert, const int32_t* num_valid, int64_t max_rows, uint8_t* hq,
                                    uint8_t* sfh, int32_t* status, void* stream);
/* The 256-column GEMM1 reading UNSORTED tokens: `codes` [tokens][H/2] and `scales` [tokens][H/32] are the row-major output
 * of b200moe_quant_mxfp4, `sorted_ids` the sorted (token | slot << 24) list of b200moe_moe_sort at block height 128. Each
 * CTA gathers its 128 token rows itself (16-byte asynchronous copies, a padding row reads as zeros), so no sorted copy of
 * the activations is written or read (the reference's prefill GEMM1 gathers through sorted_token_ids the same way,
 * MOE/gemm1_prefill_h6144_i768.py:560-598). `by_pair` != 0: codes / scales hold one row per (token, slot) pair, row
 * 4 * token + slot (rows that arrived from other ranks). Same hq / sfh bits as the kernels above. */
int b200moe_gemm1_swiglu_quant_gather(const uint8_t* w13t, int num_experts, const uint8_t* codes, const uint8_t* scales,
                                      int64_t tokens, int by_pair, const int32_t* sorted_ids, const int32_t* block_expert,
                                      const int32_t* num_valid, int64_t max_rows, uint8_t* hq, uint8_t* sfh,
                                      int32_t* status, void* stream);
/* The same launch restricted to the row blocks [block_range[0], block_range[1]) (device int32 pair, may be null: all) and
 * to at most `max_ctas` CTAs (0: one per SM). A caller splits the row blocks into chunks (b200moe_block_chunks) so that the
 * kernel that consumes hq can start on one chunk while this one works on the next, beside it on the remaining SMs. */
int b200moe_gemm1_swiglu_quant_gather_range(const uint8_t* w13t, int num_experts, const uint8_t* codes, const uint8_t* scales,
                                            int64_t tokens, int by_pair, const int32_t* sorted_ids,
                                            const int32_t* block_expert, const int32_t* num_valid, int64_t max_rows,
                                            uint8_t* hq, uint8_t* sfh, const int32_t* block_range, int max_ctas,
                                            int32_t* status, void* stream);
/* ranges int32 [chunks][2]: the sorted row blocks (num_valid / bm of them, a device count) in `chunks` runs of nearly equal
 * length; chunks <= 32. */
int b200moe_block_chunks(const int32_t* num_valid, int bm, int chunks, int32_t* ranges, void* stream);
int b200moe_gemm1_pair_supported(void);
int b200moe_gemm1_swiglu_quant_pair(const uint8_t* w13t, int num_experts, const uint8_t* xq_sorted, const uint8_t* sfx,
                                    const int32_t* block_expert, const int32_t* num_valid, int64_t max_rows, uint8_t* hq,
                                    uint8_t* sfh, int32_t* status, void* stream);

/* Grouped GEMM2, times the routing weight, rounded to bf16, one writer per (token, slot, column)
 * (MOE/gemm2_a4w4_small.py:19-79, MOE/gemm2_a4w4_bm128.py:52; oracle MOE/reference.py:73-74).
 * slots bf16 [T][4][6144]; padding rows are dropped. */
int b200moe_gemm2_weighted(const uint8_t* w2t, int num_experts, const uint8_t* hq, const uint8_t* sfh,
                           const int32_t* block_expert, const int32_t* num_valid, const int32_t* sorted_ids,
                           const float* sorted_w, int64_t max_rows, int bm, int64_t tokens, void* slots_bf16,
                           int32_t* status, void* stream);

/* Both grouped GEMMs in ONE persistent launch, for bm = 16 / 32 / 64 (MOE/gemm12_a4w4.py:24 gemm12_a4w4: GEMM1 and GEMM2
 * work in one launch ordered by ready counters). Same inputs, outputs and bits as b200moe_gemm1_swiglu_quant followed by
 * b200moe_gemm2_weighted. `done` int32 [max_rows/bm] must be zero on entry (b200moe_quant_dispatch zeroes it); it counts
 * the finished GEMM1 tiles of every row block, and a GEMM2 unit starts when its block shows 12. Unlike the reference's
 * wait, the wait here is bounded (about two seconds, then status = B200MOE_DEV_TIMEOUT and the kernel winds down), and
 * GEMM1 work never waits, so completion does not depend on the order in which CTAs are scheduled. */
int b200moe_gemm12(const uint8_t* w13t, const uint8_t* w2t, int num_experts, const uint8_t* xq_sorted, const uint8_t* sfx,
                   const int32_t* block_expert, const int32_t* num_valid, const int32_t* sorted_ids, const float* sorted_w,
                   int64_t max_rows, int bm, int64_t tokens, uint8_t* hq, uint8_t* sfh, int32_t* done, void* slots_bf16,
                   int32_t* status, void* stream);

/* GEMM2 fused with the expert-parallel combine (no counterpart in the reference, which has no expert parallelism; its
 * multi-GPU tail is MOE/prepared_input.py:189-209 + amd_kernels/collectives/pull_collectives_ranks4). Same computation as
 * b200moe_gemm2_weighted, but result row of pair r (r = 4*token+slot of THIS rank's received rows) is stored straight
 * into rank row_rank[r]'s slot buffer at pair row_pair[r]: peer_slots[k] is a device pointer to rank k's bf16 [pairs][6144]
 * buffer of peer_rows rows (this rank's own buffer at index `rank`, the others peer mappings over NVLink); world <= 8.
 * A rank or pair index outside those bounds is not stored and sets status = B200MOE_DEV_BAD_INDEX.
 * Plain peer stores from the epilogue, no multicast, no waits. The caller orders the ranks afterwards (any collective on
 * the same streams) before a rank reads its buffer. */
int b200moe_gemm2_weighted_peer(const uint8_t* w2t, int num_experts, const uint8_t* hq, const uint8_t* sfh,
                                const int32_t* block_expert, const int32_t* num_valid, const int32_t* sorted_ids,
                                const float* sorted_w, int64_t max_rows, int bm, int64_t tokens, const int32_t* row_rank,
                                const int32_t* row_pair, void* const* peer_slots, int world, int64_t peer_rows, int32_t* status,
                                void* stream);
/* b200moe_gemm2_weighted_peer on the row blocks [block_range[0], block_range[1]) only (may be null: all), on at most
 * `max_ctas` CTAs (0: one per SM). */
int b200moe_gemm2_weighted_peer_range(const uint8_t* w2t, int num_experts, const uint8_t* hq, const uint8_t* sfh,
                                      const int32_t* block_expert, const int32_t* num_valid, const int32_t* sorted_ids,
                                      const float* sorted_w, int64_t max_rows, int bm, int64_t tokens,
                                      const int32_t* row_rank, const int32_t* row_pair, void* const* peer_slots, int world,
                                      int64_t peer_rows, const int32_t* block_range, int max_ctas, int32_t* status,
                                      void* stream);

/* Plain CUDA-core versions of the two grouped GEMMs on checkpoint-layout weights and row-major activations, same
 * outputs and output layouts as the tcgen05 kernels. They exist so the tensor-core kernels and the preshuffle can be
 * checked on the GPU at sizes the CPU oracle cannot reach; the product path never selects them. `rows`/`n_rows`: the
 * sorted rows to compute (null = all rows below num_valid[0]). */
int b200moe_gemm1_simt(const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* codes, const uint8_t* scales,
                       const int32_t* sorted_ids, const int32_t* block_expert, const int32_t* num_valid,
                       const int32_t* rows, int64_t n_rows, int64_t max_rows, int bm, int64_t tokens, uint8_t* hq,
                       uint8_t* sfh, void* stream);
int b200moe_gemm2_simt(const uint8_t* w2, const uint8_t* w2_scale, const uint8_t* hq, const uint8_t* sfh,
                       const int32_t* sorted_ids, const float* sorted_w, const int32_t* block_expert,
                       const int32_t* num_valid, const int32_t* rows, int64_t n_rows, int64_t max_rows, int bm,
                       int64_t tokens, void* slots_bf16, void* stream);

/* Slot reduce (MOE/common/reduce_slots_shared.py:16-41 reduce_slots_shared; oracle MOE/reference.py:151-159):
 * out = bf16( (((+0 + s0) + s1) + s2) + s3 (+ shared) ) in fp32, bit-exact. shared may be null. */
int b200moe_reduce_slots(const void* slots_bf16, const void* shared_bf16, int64_t tokens, void* out_bf16, void* stream);

/* The layer's fused tail (amd_kernels/collectives/pull_collectives_ranks4/README.md:25-27
 * slots4_reduce_scatter_add_rmsnorm_mxfp8 at one rank; sum: .../pull_collectives_ranks4/reference.py:74-91
 * slots4_reduce_scatter_reference; add + norm + quant: amd_kernels/norm/gemma_add_rmsnorm_h6144/reference.py steps 2-4):
 *   x = bf16((((s0 + s1) + s2) + s3) (+ shared)) in fp32;  s = fp32(x) + fp32(residual);  residual_out = bf16(s);
 *   y = (s * rstd) * (weight + 1), rstd = 1/sqrt(sum(s^2)/6144 + eps);  out = bf16(y) (out may be null);
 *   per 32 columns of y: scale byte = clamp(ceil(log2(max(max|y|, 2^-126) / 448)) + 127, 0, 254) and E4M3 codes of
 *   y * 2^(127 - byte) (codes8 [T][6144] and scales8 [T][192] row-major; both may be null).
 * The sum and the residual are bit-exact; y is fp32 arithmetic with a fixed-order sum of squares (the same bits on every
 * run), within the reference's tolerances of its fp64 statement. slots bf16 [T][4][6144], shared (may be null) /
 * residual / residual_out / out bf16 [T][6144], weight bf16 [6144]; all 16-byte aligned. */
int b200moe_reduce_slots_add_rmsnorm_quant(const void* slots_bf16, const void* shared_bf16, const void* residual_bf16,
                                           const void* weight_bf16, float eps, int64_t tokens, void* residual_out_bf16,
                                           void* out_bf16, uint8_t* codes8, uint8_t* scales8, void* stream);

/* ---- the MXFP8 shared expert (MOE/shared_expert.py: SharedWeights, shared_expert; oracle MOE/reference.py:162-189
 * shared_mxfp8_quant_ref / shared_mxfp8_ref): a dense SwiGLU-OAI MLP on every token, E4M3 codes with one E8M0 scale
 * per 32 elements for weights, the input and the SwiGLU output; fp32 accumulation; bf16 result rows.
 *
 * b200moe_preshuffle_shared: row-major w13 E4M3 [1536][6144] + scales [1536][192], w2 E4M3 [6144][768] + scales
 * [6144][24] (the layout MOE/__init__.py:19-31 unsupported_reason checks) -> tile records: w13t 12*48 and w2t 48*6
 * records of 17408 bytes (16384 swizzled code bytes, one 512-byte scale atom, padding). W13 tiles interleave gate and
 * up rows like the routed ones. */
int b200moe_preshuffle_shared(const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* w2, const uint8_t* w2_scale,
                              uint8_t* w13t, uint8_t* w2t, void* stream);
#define B200MOE_SHARED_W13T_BYTES ((2 * B200MOE_I / 128) * 48 * 17408)
#define B200MOE_SHARED_W2T_BYTES (48 * (B200MOE_I / 128) * 17408)

/* The dense block height the shared expert uses at T tokens: 16 / 32 / 64 up to that many tokens, else 128. */
int b200moe_shared_block_rows(int64_t tokens);

/* Input quantiser of the shared expert (MOE/reference.py:162-171 shared_mxfp8_quant_ref: scale = ceil_pow2(amax/448),
 * exponent byte >= 1, round to nearest even), bit-exact. x bf16 [T][6144] -> codes8 [ceil(T/bm)*bm][6144] (padding
 * rows zero) and scale atoms [ceil(T/bm)][48][512]: row r of a block keeps scale j of K-tile a at byte
 * a*512 + (r%32)*16 + (r/32)*4 + j. bm in {16,32,64,128}. */
int b200moe_shared_quant(const void* x_bf16, int64_t tokens, int bm, uint8_t* codes8, uint8_t* atoms, void* stream);

/* The shared expert on one stream (MOE/shared_expert.py shared_expert): quantise -> GEMM1 + SwiGLU-OAI + MXFP8
 * requantise -> GEMM2 -> out bf16 [T][6144]. workspace: b200moe_shared_workspace_bytes(T) bytes, 256-byte aligned.
 * status as in the routed kernels. */
size_t b200moe_shared_workspace_bytes(int64_t tokens);
int b200moe_shared_expert(const uint8_t* w13t, const uint8_t* w2t, const void* x_bf16, int64_t tokens, void* workspace,
                          size_t workspace_bytes, void* out_bf16, int32_t* status, void* stream);

/* The shared expert's input quantiser with row-major scales [T][192] (the prepared-input payload,
 * MOE/prepared_input.py:16-36 MoeInput.shared_codes / shared_scales), and the shared expert on such pre-quantised rows
 * (MOE/shared_expert.py:70 shared_expert(..., x_quant=)): codes8 [T][6144] need no padding rows. */
int b200moe_shared_quant_rows(const void* x_bf16, int64_t tokens, uint8_t* codes8, uint8_t* scales, void* stream);
int b200moe_shared_expert_quantized(const uint8_t* w13t, const uint8_t* w2t, const uint8_t* codes8, const uint8_t* scales,
                                    int64_t tokens, void* workspace, size_t workspace_bytes, void* out_bf16,
                                    int32_t* status, void* stream);
/* Row-major scale bytes [T][cols] -> scale atoms [ceil(T/bm)][cols/4][512] of bm-row blocks (rows beyond T: byte 1). */
int b200moe_scales_to_atoms(const uint8_t* rows, int64_t tokens, int cols, int bm, uint8_t* atoms, void* stream);

/* ---- the compact prepared input (MOE/prepared_input.py:79-114 MoeInputCompact; MOE/sidecar_pack.py, sidecar_unpack.py;
 * oracle MOE/reference.py:198-235 mxfp4_sidecar_pack_ref / _unpack_ref). A token's FP4 codes q4 [T][3072] are rebuilt
 * bit for bit (signed zeros included) from its FP8 codes q8 [T][6144], both scale rows s4 / s8 [T][192] and a
 * correction mask [T][768] (bit i%8 of byte i/8 is value i). pack writes the mask, unpack writes q4. */
int b200moe_sidecar_pack(const uint8_t* q4, const uint8_t* s4, const uint8_t* q8, const uint8_t* s8, int64_t tokens,
                         uint8_t* mask, void* stream);
int b200moe_sidecar_unpack(const uint8_t* mask, const uint8_t* s4, const uint8_t* q8, const uint8_t* s8, int64_t tokens,
                           uint8_t* q4, void* stream);

/* The same reduce over slot rows that sit in another order: index int32 [T][4] gives, for pair 4*token+slot, its row in
 * rows_bf16 [N][6144] (the expert-parallel combine: rows come back from the other ranks in send order). Same arithmetic
 * and the same bits as b200moe_reduce_slots on the reordered rows. No counterpart in the reference (it has no expert
 * parallelism); the fixed slot order is that of MOE/reference.py:151-159. */
int b200moe_reduce_rows(const void* rows_bf16, const int32_t* index, const void* shared_bf16, int64_t tokens,
                        void* out_bf16, void* stream);

/* The whole routed layer on one stream (MOE/chain.py:127-197 mxfp4_moe without the shared expert): route -> quantise
 * -> sort -> gather -> GEMM1 -> GEMM2 -> (reduce). `workspace` of b200moe_workspace_bytes(T, num_experts) bytes,
 * 256-byte aligned; out bf16 [T][6144] may be null when only slots [T][4][6144] are wanted (partials mode). */
typedef struct b200moe_weights {
  const uint8_t* w13t; /* tile records, b200moe_preshuffle_w13 */
  const uint8_t* w2t;  /* tile records, b200moe_preshuffle_w2 */
  const float* bias;   /* may be null */
  int num_experts;
  int route_mode;
  float route_scale;
  const float* gate;   /* router weight fp32 [num_experts][6144]; needed by b200moe_forward_x only, else may be null */
  const void* gate_split; /* b200moe_router_split_gate of `gate` (bf16 [3][128][6144]) or null: the tensor-core router */
} b200moe_weights;
size_t b200moe_workspace_bytes(int64_t tokens, int num_experts);
int b200moe_forward(const b200moe_weights* w, const void* x_bf16, const float* logits, int64_t tokens, void* workspace,
                    size_t workspace_bytes, void* slots_bf16, void* out_bf16, int32_t* status, void* stream);

/* The same layer with the router inside the call -- the call vLLM makes, MOE/chain.py:127-197 mxfp4_moe(x, w) with its
 * fused router + input quantiser (MOE/chain.py:75-103; MOE/router_mxfp4_quant_line_layout.py:48-400): one pass over x
 * gives the split-K logit partials (w->gate) and the row-major MXFP4 operands, then top-4 on the partials added in split
 * order -> sort -> gather of the quantised rows -> GEMM1 -> GEMM2 -> (reduce). Workspace of
 * b200moe_workspace_bytes_x(T, num_experts) bytes, 256-byte aligned. Same slots / out as b200moe_forward fed with the
 * logits b200moe_router_gemm produces. */
size_t b200moe_workspace_bytes_x(int64_t tokens, int num_experts);
int b200moe_forward_x(const b200moe_weights* w, const void* x_bf16, int64_t tokens, void* workspace,
                      size_t workspace_bytes, void* slots_bf16, void* out_bf16, int32_t* status, void* stream);

/* Host-buffer form of the same call, the one the end-to-end benchmark times: copies x and logits from (pinned) host
 * memory to `dev_x`/`dev_logits`, runs b200moe_forward, copies out to `host_out`, all on `stream`, no synchronise. */
int b200moe_forward_host(const b200moe_weights* w, const void* host_x_bf16, const float* host_logits, int64_t tokens,
                         void* dev_x, float* dev_logits, void* workspace, size_t workspace_bytes, void* slots_bf16,
                         void* dev_out, void* host_out_bf16, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_MOE_H */

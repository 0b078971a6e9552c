/*
 * paired_nvfp4_b200 -- C ABI of the B200 (sm_100a) paired-4:8 sparse NVFP4 grouped MoE GEMM path.
 *
 * Every entry point takes raw device pointers, extents, scalar options and a CUDA stream, only
 * enqueues work on that stream, never synchronises and never reads device memory on the host, so
 * every forward call may be captured into a CUDA graph.  Unless a comment says otherwise a call
 * allocates nothing: the caller owns every buffer, sized with the query functions below.
 *
 * Return value: 0 on success, a PNV_ERR_* code otherwise; pnv_last_error() then returns a
 * NUL-terminated description (thread-local, valid until the next failing call on that thread).
 *
 * Each declaration names the interface of the reference project (IST-DASLab/grouped-sparse-GEMM,
 * paths relative to its root) that it stands in for.
 */
#ifndef PAIRED_NVFP4_B200_H_
#define PAIRED_NVFP4_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PNV_ABI_VERSION 2

#define PNV_OK 0
#define PNV_ERR_INVALID_ARGUMENT 1 /* a shape / option the reference rejects with TORCH_CHECK */
#define PNV_ERR_CUDA 2             /* a CUDA runtime or driver call failed at enqueue time */
#define PNV_ERR_UNSUPPORTED 3      /* valid for the reference, not implemented by this build */

/* Same handle as cudaStream_t / CUstream. */
typedef struct CUstream_st* pnv_stream_t;

/* Gated activation kinds of silu_mul_quant_act (csrc/layout.cuh:197-202, GatedAct::Kind). */
#define PNV_ACT_SILU 0
#define PNV_ACT_SITU 1

int pnv_abi_version(void);
const char* pnv_last_error(void);

/* Buffers for the direct expert-parallel exchange, where the *_parts entry points below store rows straight into
 * another rank's memory (one node, GPUs with peer access; no counterpart in the reference).  Set-up time only.
 *   pnv_peer_buffer_alloc  cudaMalloc on the current device + the 64-byte interprocess handle of the allocation
 *   pnv_peer_buffer_open   in ANOTHER process: maps the allocation into the current device's address space
 *                          (cudaIpcOpenMemHandle with lazy peer access), so that kernels launched on the current
 *                          device can store into it
 *   pnv_peer_buffer_close  unmaps an opened buffer;  pnv_peer_buffer_free  frees an allocated one (after every
 *                          process that opened it has closed it) */
#define PNV_PEER_HANDLE_BYTES 64
int pnv_peer_buffer_alloc(int64_t bytes, void** ptr_out, void* handle_out);
int pnv_peer_buffer_open(const void* handle, void** ptr_out);
int pnv_peer_buffer_close(void* ptr);
int pnv_peer_buffer_free(void* ptr);

/* Device status word of the group_mm launches on the current device since the last read: 0 when every
 * bounded wait inside the kernels completed, otherwise the code of a wait that gave up (its launch's
 * results are then undefined).  Every wait inside the kernels is bounded so that a lost copy or a logic
 * error ends the launch instead of hanging the GPU; the enqueueing call has long returned PNV_OK by
 * then, so a caller that wants to know reads this word at one of its own synchronisation points.
 * Reading synchronises the device and clears the word.
 * (No counterpart in the reference, whose kernel waits without bound.) */
int pnv_group_mm_device_status(int* status_out);

/* Testing aid (allocates 4 bytes, synchronises; no counterpart in the reference): runs a one-thread kernel
 * that waits, with a short budget, on a barrier nothing arrives on, i.e. the give-up path of the bounded
 * waits without anything in flight.  *gave_up_out becomes 1 when the wait ran out as it should, and the
 * device status word then reads 99 until pnv_group_mm_device_status clears it. */
int pnv_selftest_bounded_wait(int* gave_up_out);

/* ---- size queries ------------------------------------------------------------------------- */

/* physical_dims(features, k, groups) (csrc/layout.cuh:83-91): a_comp is
 * [E, *m_aligned_ac, *k_aligned_ac / 2] bytes, e_meta is [E, *m_aligned_e, *k_aligned_e] bytes. */
int pnv_physical_dims(int features, int k, int* m_aligned_ac, int* k_aligned_ac, int* m_aligned_e,
                      int* k_aligned_e);

/* sfa_numel / sfb_numel (csrc/layout.cuh:95-102): bytes of a swizzled scale buffer holding
 * `rows` rows (features for SFA, max_n or cap for SFB) of ceil(k / 32) scales for `groups` experts. */
int64_t pnv_sf_numel(int rows, int k, int groups);

/* ---- load time ---------------------------------------------------------------------------- */

/* paired_nvfp4_compress (csrc/ops.cu:156-223).  w_packed u8[E, M, K/2] (two e2m1 per byte, low
 * nibble = lower K, paired-4:8 zeros in place), w_blockscale u8[E, M, ceil(K/32)] raw UE4M3 in
 * natural order.  Writes every byte of a_comp, e_meta and sfa (padding is zero). */
int pnv_compress(const uint8_t* w_packed, const uint8_t* w_blockscale, int experts, int features,
                 int k, uint8_t* a_comp, uint8_t* e_meta, uint8_t* sfa, pnv_stream_t stream);

/* ---- activation quantizers ---------------------------------------------------------------- */

/* paired_nvfp4_quant_act (csrc/ops.cu:230-262 -> quant_act_kernel, csrc/quant.cuh:238-268).
 * x bf16[E, max_n, K]; gscale f32[E] (gscale_per_expert != 0) or f32[1]; counts i32[E].
 * b_act u8[E, max_n, K/2]: rows t >= counts[e] are not written.  sfb u8[pnv_sf_numel(max_n, K, E)]:
 * every byte is written (quantized scales, 0x38 elsewhere). */
int pnv_quant_act(const void* x, const float* gscale, int gscale_per_expert, const int32_t* counts,
                  int experts, int max_n, int k, uint8_t* b_act, uint8_t* sfb, int sm_count,
                  pnv_stream_t stream);

/* paired_nvfp4_silu_mul_quant_act (csrc/ops.cu:269-306 -> silu_mul_quant_kernel,
 * csrc/quant.cuh:290-331; activation: make_gated_act csrc/ops.cu:128-141, gated_act
 * csrc/layout.cuh:204-216).  x2 bf16[E, max_n, 2n]: [gate | up] halves, or, when interleaved != 0,
 * 64-column blocks of 32 gate then the 32 matching up columns.  beta / linear_beta are read only
 * for PNV_ACT_SITU.  Outputs as pnv_quant_act with k = n. */
int pnv_silu_mul_quant_act(const void* x2, const float* gscale, int gscale_per_expert,
                           const int32_t* counts, int experts, int max_n, int n, int interleaved,
                           int act_kind, float beta, float linear_beta, uint8_t* b_act,
                           uint8_t* sfb, int sm_count, pnv_stream_t stream);

/* paired_nvfp4_scatter_quant_act (csrc/ops.cu:314-367 -> scatter_quant_kernel,
 * csrc/quant.cuh:360-404).  a1 bf16[T, K]; flat_tok / dest_global i64[n_routes]; topk_weights
 * f32[n_routes] or NULL; routing i with dest_global[i] == experts * cap is dropped.
 * b_act u8[E * cap, K/2]; sfb u8[pnv_sf_numel(cap, K, E)], fully written. */
int pnv_scatter_quant_act(const void* a1, const int64_t* flat_tok, const int64_t* dest_global,
                          const float* topk_weights, const float* gscale, int gscale_per_expert,
                          int64_t n_routes, int k, int experts, int cap, uint8_t* b_act,
                          uint8_t* sfb, int sm_count, pnv_stream_t stream);

/* ---- routing plan, planned scatter, FP4-on-the-wire helpers, combine ------------------------------ */

/* paired_nvfp4_dispatch_plan (csrc/ops.cu:374-411 -> dispatch_plan, csrc/moe_routing.cuh:93-193).
 * topk_ids i32 or i64 [tokens, topk] global expert ids; this rank owns experts
 * [first_expert, first_expert + num_local_experts).  Writes counts i32[E] (clamped to cap),
 * route_dest i32[tokens * topk] (row e*cap + r, or -1), and src_tok / src_route i32[E * cap] for the
 * assigned rows (other slots are not written).  Plans of more than 1024 routings need `scratch`:
 * pnv_dispatch_plan_scratch_ints(tokens * topk, E) ints (the reference allocates the same buffer inside
 * the op, csrc/ops.cu:397-398); smaller plans accept NULL. */
int64_t pnv_dispatch_plan_scratch_ints(int64_t n_routes, int num_local_experts);
int pnv_dispatch_plan(const void* topk_ids, int ids_are_int64, int64_t tokens, int topk, int first_expert,
                      int num_local_experts, int cap, int32_t* counts, int32_t* route_dest,
                      int32_t* src_tok, int32_t* src_route, int32_t* scratch, pnv_stream_t stream);

/* The same plan for expert ids that do not sit back to back: id i is read at topk_ids[i * id_stride] (stride in
 * elements of the id type).  This is how a receiving rank plans straight from the wire rows of an
 * expert-parallel dispatch (pnv_pack_wire_rows), whose expert ids sit one per row.  No counterpart in the
 * reference, which leaves the exchange to its caller. */
int pnv_dispatch_plan_strided(const void* topk_ids, int ids_are_int64, int64_t id_stride, int64_t tokens, int topk,
                              int first_expert, int num_local_experts, int cap, int32_t* counts,
                              int32_t* route_dest, int32_t* src_tok, int32_t* src_route, int32_t* scratch,
                              pnv_stream_t stream);

/* pnv_dispatch_plan without any allocation, by anyone.  It has no counterpart in the reference.
 * The plan's scratch (per-chunk expert totals) lives in an array built into the library instead of a
 * caller buffer, for callers that cannot obtain device memory at call time: a serving process that
 * handed the whole GPU to its own arena at start-up, or a latency-critical loop that must not take
 * cudaMalloc's device-wide stall.  Inputs and outputs are still the caller's.
 *   - Limit: ceil(tokens * topk / 1024) * num_local_experts <= pnv_dispatch_plan_noalloc_max_scratch_ints()
 *     (65536 ints = 256 KiB, resident on every GPU that loads the library); larger plans are rejected
 *     with PNV_ERR_INVALID_ARGUMENT and a message naming the limit.
 *   - The first call on each device looks up the array's device address (no allocation); make that call
 *     before starting any stream capture on the device.
 *   - All calls on a device share the one array, and it keeps the previous call's contents.  Nothing
 *     in it needs clearing (every value a plan reads was written by that plan first), but two calls
 *     whose kernels overlap on the GPU - different streams, no ordering between them - race on it. */
int64_t pnv_dispatch_plan_noalloc_max_scratch_ints(void);
int pnv_dispatch_plan_noalloc(const void* topk_ids, int ids_are_int64, int64_t tokens, int topk,
                              int first_expert, int num_local_experts, int cap, int32_t* counts,
                              int32_t* route_dest, int32_t* src_tok, int32_t* src_route,
                              pnv_stream_t stream);

/* paired_nvfp4_scatter_quant_act_planned (csrc/ops.cu:418-468 -> scatter_quant_planned_kernel,
 * csrc/quant.cuh:431-471).  a1 bf16[T, K]; src_tok / src_route from pnv_dispatch_plan; topk_weights
 * f32[T * topk] or NULL.  Outputs as pnv_quant_act with max_n = cap. */
int pnv_scatter_quant_act_planned(const void* a1, const int32_t* src_tok, const int32_t* src_route,
                                  const float* topk_weights, const float* gscale, int gscale_per_expert,
                                  const int32_t* counts, int k, int experts, int cap, uint8_t* b_act,
                                  uint8_t* sfb, int sm_count, pnv_stream_t stream);

/* paired_nvfp4_quant_rows (csrc/ops.cu:476-500 -> quant_rows_kernel, csrc/quant.cuh:492-508).
 * x bf16[tokens, K] -> q u8[tokens, K/2], q_sf u8[tokens, K/32] (natural order), scale gscale[0]. */
int pnv_quant_rows(const void* x, const float* gscale, int64_t tokens, int k, uint8_t* q, uint8_t* q_sf,
                   int sm_count, pnv_stream_t stream);

/* paired_nvfp4_scatter_fp4_planned (csrc/ops.cu:502-541 -> scatter_fp4_planned_kernel,
 * csrc/quant.cuh:525-552): places pnv_quant_rows output into the batched operands. */
int pnv_scatter_fp4_planned(const uint8_t* q, const uint8_t* q_sf, const int32_t* src_tok,
                            const int32_t* counts, int k, int experts, int cap, uint8_t* b_act,
                            uint8_t* sfb, int sm_count, pnv_stream_t stream);

/* Expert-parallel dispatch in fixed-capacity slabs (no counterpart in the reference, which offers quant_rows /
 * scatter_fp4_planned, csrc/quant.cuh:485-562, and leaves the exchange between them to the caller).
 * A wire row is one routed token row as it crosses the link:
 *   [k/2 bytes e2m1 codes][k/32 UE4M3 scales][padding to 16 bytes][int32 expert id local to the receiver][12 bytes]
 * = pnv_wire_row_bytes(k) bytes.  The sender plans its routings by destination rank with
 * pnv_dispatch_plan(topk_ids / experts_per_rank ..., num_local_experts = ranks, cap = slab): slot s of slab w
 * is live when s < slab_counts[w] and then carries token slot_tok[w * slab + s] of routing
 * slot_route[w * slab + s]; pnv_pack_wire_rows builds wire u8[ranks * slab, row bytes] from pnv_quant_rows
 * output, writing expert id -1 into dead slots (their other bytes stay undefined).  After an equal-split
 * all-to-all the receiver plans with pnv_dispatch_plan_strided on the ids inside the rows (dead slots fall
 * out as "not local") and pnv_scatter_fp4_wire places codes and scales like pnv_scatter_fp4_planned. */
int64_t pnv_wire_row_bytes(int k);
int pnv_pack_wire_rows(const uint8_t* q, const uint8_t* q_sf, const void* topk_ids, int ids_are_int64,
                       const int32_t* slot_tok, const int32_t* slot_route, const int32_t* slab_counts, int ranks,
                       int slab, int experts_per_rank, int k, uint8_t* wire, pnv_stream_t stream);
/* pnv_pack_wire_rows with slab w written to wire_parts[w] (a HOST array of `ranks` device pointers, at most 16,
 * each to slab * row bytes): with peer memory of the receiving ranks mapped into this process the pack is the
 * dispatch, the rows cross NVLink as the kernel stores them. */
int pnv_pack_wire_rows_parts(const uint8_t* q, const uint8_t* q_sf, const void* topk_ids, int ids_are_int64,
                             const int32_t* slot_tok, const int32_t* slot_route, const int32_t* slab_counts,
                             int ranks, int slab, int experts_per_rank, int k, void* const* wire_parts,
                             pnv_stream_t stream);
int pnv_scatter_fp4_wire(const uint8_t* wire, const int32_t* src_tok, const int32_t* counts, int k, int experts,
                         int cap, uint8_t* b_act, uint8_t* sfb, int sm_count, pnv_stream_t stream);

/* paired_nvfp4_moe_finalize (csrc/ops.cu:548-575 -> finalize_kernel, csrc/moe_routing.cuh:203-244).
 * out bf16[tokens, K] = sum over kept routings in top-k order of fused bf16[E * cap, K] rows
 * (route_dest i32[tokens, topk], -1 = dropped), weighted by topk_weights f32[tokens, topk] when given. */
int pnv_moe_finalize(void* out, const void* fused, const int32_t* route_dest, const float* topk_weights,
                     int64_t tokens, int topk, int k, pnv_stream_t stream);

/* Row gather for the expert-parallel exchange (no counterpart in the reference, which leaves the permutation
 * either side of the exchange to the caller's framework; the plan tensors are those of dispatch_plan,
 * csrc/ops.cu:374-411): dst[i, :] = idx[i] >= 0 ? src[idx[i], :] : 0 for rows of row_bytes bytes
 * (a multiple of 16; both buffers 16-byte aligned). */
int pnv_gather_rows(const void* src, const int32_t* idx, int64_t n_idx, int64_t row_bytes, void* dst,
                    pnv_stream_t stream);

/* Rows whose flag is negative become zero, the others are left alone (dst [rows, row_bytes], row_bytes a
 * multiple of 16).  With pnv_group_mm_rows this stands in for pnv_gather_rows on the way back from the experts:
 * the GEMM writes every kept row straight into return order, this zeroes the slots no row lands on. */
int pnv_zero_rows(void* dst, const int32_t* flags, int64_t rows, int64_t row_bytes, pnv_stream_t stream);

/* pnv_zero_rows over the same kind of parts table as pnv_group_mm_rows_parts: flags has n_parts * rows_per_part
 * entries, row q is row q % rows_per_part of parts[q / rows_per_part]. */
int pnv_zero_rows_parts(void* const* parts, int n_parts, int64_t rows_per_part, const int32_t* flags,
                        int64_t row_bytes, pnv_stream_t stream);

/* The unfused gated activation the quantizer above folds in (gated_act, csrc/layout.cuh:204-216;
 * device replica ref_silu_mul_kernel, csrc/testing/selftest.cu:750-760): y bf16[rows, n] from
 * x2 bf16[rows, 2n].  pnv_silu_mul_quant_act == pnv_gated_act followed by pnv_quant_act, byte for
 * byte. */
int pnv_gated_act(const void* x2, int64_t rows, int n, int interleaved, int act_kind, float beta,
                  float linear_beta, void* y, pnv_stream_t stream);

/* Testing aid (no reference counterpart): SiLU is evaluated through a 65536-entry table of bf16(g / (1 + expf(-g)))
 * built into the library and filled on the device with that same expression; 0 switches the table off so that a
 * test can compare both paths bit for bit.  Process-wide; default on. */
int pnv_set_silu_table(int enabled);

/* ---- grouped GEMM ------------------------------------------------------------------------- */

/* paired_nvfp4_group_mm_configs (csrc/ops.cu:665-670; table kGroupMmKinds,
 * csrc/sm100/tactics.cu:35-44): tile-variant names indexed by config_id. */
int pnv_group_mm_num_configs(void);
const char* pnv_group_mm_config_name(int config_id);

/* paired_nvfp4_group_mm (csrc/ops.cu:672-735 -> run_group_mm_variant, csrc/group_mm.cuh:92-179;
 * cluster rules check_cluster, csrc/sm100/tactics.cu:62-69).
 * out bf16[E, max_n, features]: out[e, t, m] = bf16(alphas[e] * sum_k dq(w)[e,m,k] dq(b)[e,t,k])
 * for t < counts[e]; every other row keeps the caller's bytes.  a_comp / e_meta / sfa are
 * pnv_compress outputs for (features, k); b_act / sfb a quantizer's outputs for (max_n, k).
 * pdl != 0 launches with programmatic dependent launch (the kernel waits on its stream
 * predecessor before its first dependent read; csrc/pdl.cuh:42-80).
 * workspace (the reference allocates its own inside the op, csrc/group_mm.cuh:163-165): NULL, or
 * pnv_group_mm_workspace_bytes(experts, features, max_n, sm_count) bytes, 256-byte aligned, for splitting K
 * across CTAs.  Only decode-sized problems (max_n <= 32) with fewer than 1.5 tiles per SM (decided on the device
 * from the counts) use it: the K stages of all tiles are dealt evenly
 * to the SMs, a tile shared by several CTAs is summed from fp32 partials in K order by whichever arrives
 * last (so the result does not depend on timing).  The first 4 * experts * ceil(features / 128) bytes are
 * arrival counters: they must be zero before the first launch that uses the buffer, every launch leaves
 * them zero, and two launches that may overlap on the GPU must not share a workspace. */
int64_t pnv_group_mm_workspace_bytes(int experts, int features, int max_n, int sm_count);
int pnv_group_mm(void* out, const uint8_t* a_comp, const uint8_t* e_meta, const uint8_t* sfa,
                 const uint8_t* b_act, const uint8_t* sfb, const float* alphas,
                 const int32_t* counts, int experts, int features, int k, int max_n, int config_id,
                 int cluster_m, int cluster_n, int sm_count, int pdl, void* workspace,
                 int64_t workspace_bytes, pnv_stream_t stream);

/* pnv_group_mm with the output rows permuted on the way out (no counterpart in the reference, whose caller
 * permutes the expert outputs after the GEMM): token row (e, t), t < counts[e], is written to row
 * row_map[e * max_n + t] of out bf16[rows, features] and not at all where the map is negative; map entries of rows
 * at or past counts[e] are not read.  The caller guarantees 0 <= row_map[...] < rows for the rows it keeps.  With
 * the src_tok of the dispatch_plan that placed the rows (topk = 1) the outputs land in the plan's input order. */
int pnv_group_mm_rows(void* out, const int32_t* row_map, const uint8_t* a_comp, const uint8_t* e_meta,
                      const uint8_t* sfa, const uint8_t* b_act, const uint8_t* sfb, const float* alphas,
                      const int32_t* counts, int experts, int features, int k, int max_n, int config_id,
                      int cluster_m, int cluster_n, int sm_count, int pdl, void* workspace,
                      int64_t workspace_bytes, pnv_stream_t stream);

/* pnv_group_mm_rows whose output rows are spread over n_parts buffers (1..16): row q of the logical
 * [n_parts * rows_per_part, features] output is row q % rows_per_part of out_parts[q / rows_per_part].  out_parts is a
 * HOST array of device pointers (16-byte aligned); they may be peer memory of other GPUs mapped into this process, so
 * that an expert-parallel rank stores every expert output row straight into the buffer of the rank that sent the
 * token (plain stores over NVLink; the caller orders them against the reader with its own barrier). */
int pnv_group_mm_rows_parts(void* const* out_parts, int n_parts, int64_t rows_per_part, const int32_t* row_map,
                            const uint8_t* a_comp, const uint8_t* e_meta, const uint8_t* sfa, const uint8_t* b_act,
                            const uint8_t* sfb, const float* alphas, const int32_t* counts, int experts,
                            int features, int k, int max_n, int config_id, int cluster_m, int cluster_n,
                            int sm_count, int pdl, void* workspace, int64_t workspace_bytes, pnv_stream_t stream);

/* paired_nvfp4_group_mm_swiglu_configs / paired_nvfp4_group_mm_swiglu_quant (csrc/ops.cu:585-658 ->
 * SwigluFp4Epilogue, csrc/sm100/swiglu_epilogue.cuh:52-236; variant table kSwigluMmKinds,
 * csrc/sm100/tactics.cu:52-57).  GEMM1 on a W13 whose rows are interleaved in 64-row blocks (32 gate
 * rows, then the 32 matching up rows; features = 2N, a multiple of 128), with the gated activation
 * and GEMM2's input quantization fused into the epilogue: writes b_out u8[E, max_n, N/2] (rows
 * t >= counts[e] untouched) and sfb_out u8[pnv_sf_numel(max_n, N, E)] (every byte), byte-identical
 * to pnv_group_mm followed by pnv_silu_mul_quant_act(interleaved = 1) with the same gscale (and the same
 * workspace choice: splitting K changes the order of the fp32 sum).  workspace as for pnv_group_mm. */
int pnv_group_mm_swiglu_num_configs(void);
const char* pnv_group_mm_swiglu_config_name(int config_id);
int pnv_group_mm_swiglu_quant(uint8_t* b_out, uint8_t* sfb_out, const uint8_t* a_comp,
                              const uint8_t* e_meta, const uint8_t* sfa, const uint8_t* b_act,
                              const uint8_t* sfb, const float* alphas, const int32_t* counts,
                              const float* gscale, int gscale_per_expert, int experts, int features,
                              int k, int max_n, int config_id, int cluster_m, int cluster_n,
                              int act_kind, float beta, float linear_beta, int sm_count, int pdl,
                              void* workspace, int64_t workspace_bytes, pnv_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PAIRED_NVFP4_B200_H_ */

/*
 * nanoserve_b200 — C ABI of the sm_100a kernels behind nanoserve's continuous-batching forward path.
 *
 * Every entry point takes raw device pointers, explicit sizes / strides (in ELEMENTS unless a name says
 * bytes), a dtype enum and the CUDA stream to launch on, and returns an ns_status (0 = ok). Nothing here
 * allocates, frees, synchronises or reads device memory on the host, so every call can be captured in a
 * CUDA graph. The caller owns all buffers, including the attention workspace. After a non-zero return,
 * ns_last_error() gives a human-readable reason (thread-local).
 *
 * The reference has no FFI: its kernels are Python functions that the model imports by name. Each
 * declaration below names the reference function it stands in for (path inside the reference project).
 */
#ifndef NANOSERVE_B200_H
#define NANOSERVE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    NS_OK = 0,
    NS_ERR_INVALID_ARG = 1,   /* null pointer, negative size, misaligned buffer */
    NS_ERR_UNSUPPORTED = 2,   /* head layout / dtype / block size this build has no kernel for */
    NS_ERR_WORKSPACE = 3,     /* workspace too small for the given batch */
    NS_ERR_CUDA = 4           /* a CUDA runtime call (launch, attribute) failed */
} ns_status;

typedef enum { NS_BF16 = 0, NS_F32 = 1 } ns_dtype;

/* Library version (major*10000 + minor*100 + patch) and last error text of the calling thread. */
int ns_version(void);
const char* ns_last_error(void);
/* Number of SMs of the current device (grid sizing of the persistent kernels); <= 0 on error. */
int ns_sm_count(void);

/* Process-wide tuning knobs of the attention planner and dispatcher, read on the host when a call is issued (so a
 * captured CUDA graph keeps the values it was captured with, except those the plan kernel receives as arguments).
 * They exist for A/B measurements and for tests that force a path; serving code leaves them at their defaults.
 * No counterpart in the reference (its Triton kernels have a fixed grid, nanoserve/kernels/paged_attention.py:84-105). */
typedef enum {
    NS_TUNE_PREFILL_IMPL = 0,        /* 0 (default): tcgen05 prefill kernel where supported; 1: always the mma.sync kernel */
    NS_TUNE_PREFILL_OVERLAP = 1,     /* 1 (default): a mixed call's prefill kernel runs beside its decode kernel; 0: after it */
    NS_TUNE_DECODE_SPLIT_BLOCKS = 2, /* decode KV blocks above which a step runs two virtual CTAs per CTA; < 0 (default): built-in */
    NS_TUNE_DECODE_MIN_BLOCKS = 3,   /* lower bound of a decode CTA's range in KV blocks; <= 0 (default): built-in */
    NS_TUNE_DECODE_SNAP_BLOCKS = 4,  /* how far a cut may move to reach a row boundary; <= 0 (default): built-in */
    NS_TUNE_DECODE_BALANCE = 5,      /* 2 (default): row-aligned balanced cuts for large steps; 0: equal cuts snapped to rows */
    NS_TUNE_DECODE_CLUSTER = 6,      /* 1 (default): small decode steps give every row a thread-block cluster of CTAs; 0: off */
    NS_TUNE_DECODE_CLUSTER_BLOCKS = 7, /* decode KV blocks up to which a step may run in cluster mode; <= 0 (default): built-in */
    NS_TUNE_PREFILL_CLUSTER = 8,     /* CTAs that share a prefill work item's key tiles: 1, 2 or 4; 0 (default): built-in (4 / 2) */
    NS_TUNE_COUNT = 9
} ns_tuning_knob;
int ns_set_tuning(int knob, int value);
int ns_get_tuning(int knob);

/* One status word per engine step, written on the device: *status = number of bounded waits that have run out so far
 * in this library's kernels on the current device (bulk-copy / mbarrier waits of the decode GEMMs, tcgen05 waits of the
 * prefill attention kernel counted in attn_workspace's plan header; attn_workspace may be NULL) plus the violations
 * ns_check_step_metadata has counted. The counts are
 * cumulative; a caller compares with the value it saw last. Results of a launch that raised the count are undefined.
 * Graph-capturable once it has run once on the device outside capture (it resolves device symbol addresses then).
 * No counterpart in the reference (device code there never reports errors, nanoserve/kernels/fused.py). */
int ns_collect_status(const void* attn_workspace, int64_t* status, void* stream);

/* Bounds check of one step's device metadata (the stand-in for a memory checker on this path; one small kernel): block
 * ids of every sequence's context < num_blocks; cu_seqlens starts at 0, is non-decreasing and stays within n_tokens; every
 * seq_len >= its query length; when slot_mapping and positions are given (both or neither), every new token's position
 * is context + its index and its slot is table[pos / block_size] * block_size + pos % block_size, inside the pool; when
 * tokens is given, ids lie in [0, vocab). Violations are counted into the status word of ns_collect_status; nothing
 * traps and no access is skipped. cu_seqlens / table_rows may be NULL as in ns_ragged_paged_attn.
 * No counterpart in the reference (its device code checks nothing; it would run under compute-sanitizer instead). */
int ns_check_step_metadata(const int32_t* block_tables, const int32_t* table_rows, int64_t table_stride,
                           const int32_t* seq_lens, const int32_t* cu_seqlens, const int64_t* slot_mapping,
                           const int64_t* positions, const int64_t* tokens, int32_t n_seqs, int64_t n_tokens,
                           int32_t num_blocks, int32_t block_size, int32_t vocab, void* stream);

/* Tensor parallelism: all-reduce (sum) of every rank's partial [rows, hidden] bf16, fused with what follows it at both
 * sites of a layer: x_out = residual + sum (rounded), h_out = weight * rmsnorm(x_out). peer_partials[w] / peer_flags[w]
 * are HOST arrays of `world` device pointers as mapped in the calling process: rank w's partial for THIS call (written
 * by the kernel before this one on rank w's stream) and rank w's flag array (world x uint32, zero at start, peer
 * mapped). state: 2 x uint32 of this rank, zero at start. Every rank makes the same sequence of calls; callers alternate
 * two partial buffers from call to call. The kernel announces its partial to the peers, waits (bounded, on local
 * memory) for theirs, and reads them with ordinary loads over NVLink in rank order, so the result is bitwise equal on
 * every rank. world 2, 4 or 8; hidden % 8 == 0, <= 4096; bf16. A wait that runs out is counted in ns_collect_status.
 * Replaces: torch.distributed.all_reduce + the add + RMSNorm after it at the all-reduce sites nanoserve/model.py:256-257
 * (the reference lists tensor parallelism and this fusion as not implemented, README.md:252-254). */
int ns_tp_allreduce_add_rmsnorm(const void* const* peer_partials, void* const* peer_flags, void* state,
                                const void* residual, const void* weight, void* out_h, void* out_x, int64_t rows,
                                int32_t hidden, float eps, int32_t rank, int32_t world, void* stream);

/* Set-up of the peer-visible buffers of ns_tp_allreduce_add_rmsnorm. The ONLY entry points of this library that
 * allocate, map or free device memory; they belong to start-up and shutdown, never to a step or a stream capture.
 * ns_peer_alloc: cudaMalloc + zero fill on the current device. ns_peer_export: a 64-byte handle of such an allocation
 * for other processes on this machine. ns_peer_open (in another process, its own GPU current): maps the allocation and
 * enables peer access to the exporting GPU; the pointer is valid in kernels of the opening process. ns_peer_close /
 * ns_peer_free undo them. No counterpart in the reference (single GPU). */
int ns_peer_alloc(int64_t bytes, void** ptr);
int ns_peer_free(void* ptr);
int ns_peer_export(void* ptr, void* handle64);
int ns_peer_open(const void* handle64, void** ptr);
int ns_peer_close(void* ptr);

/* ------------------------------------------------------------------------------------------------
 * Fused token-wise ops.
 * ---------------------------------------------------------------------------------------------- */

/* out = weight * rmsnorm(r), r = residual + x rounded to dtype (or r = x when residual == NULL); when
 * residual != NULL, r is also stored to residual_out. fp32 mean of squares, the normalised value is rounded
 * to dtype BEFORE the weight multiply. rows x hidden, contiguous; hidden % 8 == 0 (bf16) / % 4 == 0 (f32).
 * Replaces: nanoserve/kernels/fused.py:45 rms_norm (+ _rms_norm_kernel :26-42); torch twin
 * nanoserve/model.py:140-146. */
int ns_add_rmsnorm(const void* x, const void* residual, const void* weight, void* out, void* residual_out,
                   int64_t rows, int32_t hidden, float eps, int dtype, void* stream);

/* out[r, c] = round(silu(gate_up[r, c])) * gate_up[r, inter + c], rounded; gate_up is [rows, 2*inter].
 * Replaces: nanoserve/kernels/fused.py:75 silu_mul (+ _silu_mul_kernel :63-72). */
int ns_silu_mul(const void* gate_up, void* out, int64_t rows, int32_t inter, int dtype, void* stream);

/* cos/sin tables [n_tokens, head_dim] in dtype from int64 positions and fp32 inv_freq[head_dim/2]:
 * angle = float(position) * inv_freq[d % (head_dim/2)], cos/sin in fp32, then rounded to dtype.
 * Replaces: nanoserve/model.py:212-217 Qwen2Model.rope. */
int ns_rope_cos_sin(const int64_t* positions, const float* inv_freq, void* cos_out, void* sin_out,
                    int64_t n_tokens, int32_t head_dim, int dtype, void* stream);

/* Per token: rotate the n_heads query heads and n_kv_heads key heads of one merged QKV row (non-interleaved
 * halves; every product and every sum rounded to dtype), copy the value heads, store q / k / v densely
 * (any of q_out, k_out, v_out may be NULL to skip that store) and, when k_cache != NULL, store k and v into
 * one layer's paged pool [num_blocks, block_size, n_kv_heads, head_dim] (contiguous) at flat row slots[t].
 * Replaces: nanoserve/kernels/fused.py:156 rope_qkv (+ _rope_qkv_kernel :107-153) and the unfused
 * nanoserve/kv_cache.py:274-279 PagedKVCache.write. */
int ns_rope_qkv_kvwrite(const void* qkv, const void* cos, const void* sin, void* q_out, void* k_out, void* v_out,
                        void* k_cache, void* v_cache, const int64_t* slots, int64_t n_tokens, int32_t n_heads,
                        int32_t n_kv_heads, int32_t head_dim, int dtype, void* stream);

/* Plain KV write: pool_row[slots[t]] = k_new[t] / v_new[t] for t < n_tokens (rows of n_kv_heads*head_dim).
 * Replaces: nanoserve/kv_cache.py:274-279 PagedKVCache.write. */
int ns_kv_write(const void* k_new, const void* v_new, void* k_cache, void* v_cache, const int64_t* slots,
                int64_t n_tokens, int32_t row_elems, int dtype, void* stream);

/* Weight-streaming GEMM for decode-sized batches, with the neighbouring token-wise ops fused in (bf16 only):
 *   out = epilogue( prologue(x) . w^T ),  x: [M <= 64, K], w: [N, K] row-major, fp32 accumulation.
 * prologue (ln_w != NULL): r = residual + x rounded to bf16 (r = x when residual == NULL), stored to residual_out
 *   when given; the GEMM input is ln_w * bf16(r * rsqrt(mean(r^2) + eps)).
 * epilogue 0: out[M, N] = bf16(acc + bias) (bias may be NULL);
 * epilogue 1: w = [gate; up] (N = 2*inter rows), out[M, inter] = bf16(bf16(silu(bf16(gate))) * bf16(up));
 * epilogue 2: w = merged QKV of 64-wide heads with bias; rotates q and k heads with cos/sin [M, 64] (every product
 *   and sum rounded to bf16), writes q to out [M, n_heads*64] and k / v into one layer's paged pool at slots[m].
 * split_k (1, 2, 4, 8) spreads K over a thread-block cluster whose partial tiles are summed through distributed
 * shared memory in a fixed order. K must be a multiple of 16*split_k.
 * Replaces, fused: nanoserve/model.py:231 (rms_norm + merged QKV F.linear + rope_qkv), :256 (o_proj), :256-257
 * (add + rms_norm + gate/up F.linear + silu_mul) and :257 (down_proj) for steps of at most 64 token rows. */
int ns_skinny_gemm(const void* x, const void* residual, const void* ln_w, void* residual_out, const void* w,
                   const void* bias, void* out, int32_t M, int32_t N, int32_t K, int32_t split_k, float eps,
                   int32_t epilogue, int32_t inter, const void* cos, const void* sin, void* k_cache, void* v_cache,
                   const int64_t* slots, int32_t n_heads, int32_t n_kv_heads, void* stream);

/* Narrow GEMM for decode-sized batches without a split over K across CTAs (bf16 only):
 *   out = epilogue( x . w^T ),  x: [M <= 64, K], w: [N, K] row-major, fp32 accumulation, K % 128 == 0, N % 8 == 0,
 *   (8 or 16 + M rounded up to 16, 32 or 64) rows of K must fit 220 KB of shared memory.
 * One CTA per eight weight rows over all of K (sixteen where N / 8 > 148 and N % 16 == 0, so that the grid stays one
 * wave of a 148-SM part): a GEMM with N around 1000 is one CTA per SM; the weight rows are
 * requested (16-byte cp.async, each warp its own quarter of K) before the kernel waits for its predecessor in the
 * stream, every CTA then fetches all of x by bulk copies on one mbarrier (bounded wait, counted in
 * ns_thin_gemm_errors when it runs out), and the four warps' partial tiles are summed through shared memory in a
 * fixed order. No thread-block cluster.
 * epilogue 0: out[M, N] = bf16(acc + bias) (bias may be NULL);
 * epilogue 2: as ns_skinny_gemm's epilogue 2 (merged QKV: bias, RoPE, q to out, k / v into one layer's paged pool
 *   at slots[m]) for heads of 64 or 128 (head_dim = N / (n_heads + 2 * n_kv_heads); cos / sin are [M, head_dim]).
 * Replaces, fused: nanoserve/model.py:231 (merged QKV F.linear + rope_qkv with the KV write) and :256 (o_proj) for
 * steps of at most 64 token rows. */
int ns_thin_gemm(const void* x, const void* w, const void* bias, void* out, int32_t M, int32_t N, int32_t K,
                 int32_t epilogue, const void* cos, const void* sin, void* k_cache, void* v_cache, const int64_t* slots,
                 int32_t n_heads, int32_t n_kv_heads, void* stream);

/* gate/up projection + SiLU*mul for at most 32 token rows (bf16 only), same construction as ns_thin_gemm:
 *   w = [gate; up] (2*inter rows of K), out[M, inter] = bf16(bf16(silu(bf16(x.gate^T))) * bf16(x.up^T)).
 * A CTA keeps nine tiles of four gate rows + the matching four up rows and all of x in shared memory (K % 128 == 0,
 * (72 + M rounded up to 16 or 32) rows of K within 227 KB: K <= 1024); inter % 4 == 0; ceil(inter / 36) CTAs.
 * x arrives by bulk copies whose bounded wait is counted in ns_thin_gemm_errors when it runs out (0 unless a fault).
 * Replaces, fused: nanoserve/model.py:256-257 (gate/up F.linear + silu_mul) for steps of at most 32 token rows. */
int ns_thin_swiglu_gemm(const void* x, const void* w, void* out, int32_t M, int32_t inter, int32_t K, void* stream);
/* The o_proj -> residual add -> RMSNorm -> gate/up boundary of a decode layer in two kernels instead of three:
 * ns_thin_gemm_residual: out = bf16(residual + bf16(x . w^T)) (the new residual stream, [M, N]) and ss_out[M][N / 8] =
 * the sum of squares of each 8-column piece of out's rows. Shapes and limits as ns_thin_gemm.
 * ns_thin_swiglu_gemm_norm: as ns_thin_swiglu_gemm, on h = ln_w * bf16(x * rsqrt(sum(x^2) / K + eps)) computed in shared
 * memory from the ss_parts pieces per row that ns_thin_gemm_residual left (ss_in [M][ss_parts], ss_parts = K / 8).
 * Rounding points as the unfused ops; the row's sum of squares is added in another order than ns_add_rmsnorm's.
 * Replace: nanoserve/model.py:256 (o_proj, x + ...), :251 rms_norm, :257 gate/up + silu_mul of steps <= 32 rows. */
int ns_thin_gemm_residual(const void* x, const void* w, const void* residual, void* out, float* ss_out, int32_t M,
                          int32_t N, int32_t K, void* stream);
int ns_thin_swiglu_gemm_norm(const void* x, const float* ss_in, int32_t ss_parts, const void* ln_w, float eps,
                             const void* w, void* out, int32_t M, int32_t inter, int32_t K, void* stream);
int ns_thin_gemm_errors(int32_t* count);

/* Persistent weight-streaming GEMM for decode-sized batches (bf16 only):
 *   out = epilogue( prologue(x) . w^T ),  x: [M <= 64, K], w: [N, K] row-major, fp32 accumulation, N % 16 == 0,
 *   K one of 896, 1024, 1536 (64 token rows only up to K = 1024).
 * One CTA per SM walks 16-row units of w through a shared-memory ring fed by bulk copies; the activations stay in
 * registers; K is split over 8 warps whose partial sums are added in a fixed order.
 * prologue (ln_w != NULL), the GEMM input is ln_w * bf16(r * rsqrt(mean(r^2) + eps)) with
 *   ss_in == NULL: r = residual + x rounded to bf16 (r = x when residual == NULL), stored to residual_out when given;
 *   ss_in != NULL: r = x, and mean(r^2) comes from ss_in[M, ss_parts], the per-row partial sums of r^2 that the GEMM
 *                  which produced x left behind (epilogue 2 below), added in order.
 * epilogue 0: out[M, N] = bf16(acc + bias) (bias may be NULL);
 * epilogue 1: w = [gate; up] (N = 2*inter rows), out[M, inter] = bf16(bf16(silu(bf16(gate))) * bf16(up));
 * epilogue 2: out[M, N] = bf16(add_in + bf16(acc + bias)), the new residual stream, and ss_out[M, N/16] = the sum of
 *             out^2 over each 16-column unit (ss_out may be NULL).
 * Replaces, fused: nanoserve/model.py:256-257 (o_proj + residual add; rms_norm + gate/up F.linear + silu_mul) for
 * steps of at most 64 token rows. */
int ns_stream_gemm(const void* x, const void* residual, const void* ln_w, void* residual_out, const float* ss_in,
                   int32_t ss_parts, const void* w, const void* bias, void* out, const void* add_in, float* ss_out,
                   int32_t M, int32_t N, int32_t K, float eps, int32_t epilogue, void* stream);

/* Decode-sized gate/up projection with SiLU(gate)*up on tcgen05 tensor cores, weights streamed by tiled TMA loads (bf16):
 *   out[M <= 64, inter] = bf16( bf16(silu(bf16(x . Wg^T))) * bf16(x . Wu^T) ),  w_gate_up = [Wg; Wu]: [2*inter, K] row-major.
 * K must be a multiple of 64; x: [M, K] contiguous. One CTA per SM owns a contiguous share of the gate rows and the
 * matching up rows as (part of) the 128-row M operand of the UMMA tile (the token rows are the N operand) and
 * accumulates in tensor memory.
 * Replaces, fused: nanoserve/model.py:257 (gate/up F.linear + silu_mul) for steps of at most 64 token rows. */
int ns_swiglu_gemm(const void* x, const void* w_gate_up, void* out, int32_t M, int32_t inter, int32_t K, void* stream);

/* Number of bounded waits that ran out inside ns_swiglu_gemm kernels since the library was loaded (0 in a healthy run).
 * Synchronises the device. No reference counterpart. */
int ns_umma_gemm_errors(uint32_t* count);

/* Number of bounded waits that ran out inside ns_stream_gemm kernels since the library was loaded (0 in a healthy
 * run; results of a launch that raised it are undefined). Synchronises the device. No reference counterpart. */
int ns_stream_gemm_errors(uint32_t* count);

/* ------------------------------------------------------------------------------------------------
 * Ragged paged attention.
 *
 * A batch is S sequences over N flattened query tokens: sequence s owns query rows
 * cu_seqlens[s] .. cu_seqlens[s+1]-1 and seq_lens[s] keys (cached context + this step's tokens, whose K/V
 * are already in the pool); query j of a sequence with T new tokens sees keys 0 .. seq_len - T + j.
 * Sequences with T == 1 are "decode" rows (HBM-bound, split over the KV length); T > 1 are prefill chunks
 * (tensor-core tiles). Keys live in one layer's pool [num_blocks, block_size, n_kv_heads, head_dim]
 * addressed through block_tables[row(s), j] (int32, row stride table_stride), row(s) = table_rows[s], or s
 * when table_rows == NULL. cu_seqlens == NULL means every sequence has exactly one query token.
 *
 * The tensor-core path (bf16, block_size 16, head_dim 64 / 128, GQA group <= 8) needs a caller-owned
 * workspace: ns_attn_workspace_bytes(ws_max_seqs, ws_max_tokens, ...) bytes, 256-byte aligned, zeroed once
 * before first use; the same (ws_max_seqs, ws_max_tokens) must be passed to every call using it. Other
 * layouts and fp32 run the scalar kernel and ignore the workspace.
 * ---------------------------------------------------------------------------------------------- */

int64_t ns_attn_workspace_bytes(int32_t max_seqs, int32_t max_tokens, int32_t n_heads, int32_t head_dim);

/* Build the per-step plan in the workspace (shared by every layer of the step): the decode rows' KV blocks
 * are cut into equal ranges, one per persistent decode CTA, and prefill chunks into query tiles. The
 * attention calls that follow must be given the same seq_lens / cu_seqlens / table_rows.
 * No reference counterpart (the reference plans on the host, nanoserve/kv_manager.py:158-179). */
int ns_attn_plan(const int32_t* seq_lens, const int32_t* cu_seqlens, const int32_t* table_rows, int32_t n_seqs,
                 int32_t block_size, int32_t n_heads, int32_t head_dim, void* workspace, int64_t workspace_bytes,
                 int32_t ws_max_seqs, int32_t ws_max_tokens, void* stream);

/* One layer of attention over the batch described by the last ns_attn_plan call on this workspace.
 * q, out: [N, n_heads, head_dim], row strides q_stride / out_stride (head stride = head_dim).
 * Pool strides: pool_block_stride (per block), pool_pos_stride (per token in a block), pool_head_stride.
 * Replaces: nanoserve/model.py:262-323 Qwen2Model._attend (per-sequence SDPA loop, gather, masks) together
 * with nanoserve/kernels/paged_attention.py:85-105 paged_attention_decode (_paged_decode_kernel :34-82). */
int ns_ragged_paged_attn(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_tables,
                         const int32_t* table_rows, const int32_t* seq_lens, const int32_t* cu_seqlens, void* out,
                         int32_t n_seqs, int64_t n_tokens, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                         int32_t block_size, int64_t table_stride, int64_t q_stride, int64_t out_stride,
                         int64_t pool_block_stride, int64_t pool_pos_stride, int64_t pool_head_stride, float scale,
                         int dtype, void* workspace, int64_t workspace_bytes, int32_t ws_max_seqs,
                         int32_t ws_max_tokens, void* stream);

/* Decode-only convenience: plan + attention for `batch` rows of one query token each (context_lens include
 * the new token, whose K/V are already written).
 * Replaces: nanoserve/kernels/paged_attention.py:85-105 paged_attention_decode. */
int ns_paged_attn_decode(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_tables,
                         const int32_t* context_lens, void* out, int32_t batch, int32_t n_heads,
                         int32_t n_kv_heads, int32_t head_dim, int32_t block_size, int64_t table_stride,
                         int64_t q_stride, int64_t out_stride, int64_t pool_block_stride, int64_t pool_pos_stride,
                         int64_t pool_head_stride, float scale, int dtype, void* workspace,
                         int64_t workspace_bytes, int32_t ws_max_seqs, int32_t ws_max_tokens, void* stream);

/* ns_paged_attn_decode for callers that must not allocate device memory (code running inside someone else's
 * stream capture, plugins whose host forbids allocation after start-up, processes whose memory pool belongs to
 * another runtime): the plan and the split-KV partials live in a fixed array inside the library image instead of a
 * caller-owned workspace. It has no counterpart in the reference. The array costs
 * ns_paged_attn_decode_static_bytes() (11 MiB) on every GPU that loads the library. Limits: batch <= 64,
 * n_heads <= 32, head_dim <= 128, tensor-core layouts only (bf16, block size 16, head_dim 64 / 128, GQA group <= 8);
 * anything larger returns NS_ERR_WORKSPACE and launches nothing. Calls on one GPU share the array, so calls that
 * overlap on the device race: keep them on one stream or order them. The first call on each device resolves the
 * array's address with that device current; make it before any stream capture. */
int64_t ns_paged_attn_decode_static_bytes(void);
int ns_paged_attn_decode_static(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_tables,
                                const int32_t* context_lens, void* out, int32_t batch, int32_t n_heads,
                                int32_t n_kv_heads, int32_t head_dim, int32_t block_size, int64_t table_stride,
                                int64_t q_stride, int64_t out_stride, int64_t pool_block_stride,
                                int64_t pool_pos_stride, int64_t pool_head_stride, float scale, int dtype,
                                void* stream);

/* Scalar implementation of the same ragged attention (fp32 accumulation, one warp per (query token, head));
 * any head layout, bf16 or fp32. Serves fp32 models and on-device cross-checks.
 * Replaces: nanoserve/kernels/paged_attention.py:108-121 paged_attention_reference (gather + SDPA). */
int ns_ragged_paged_attn_simple(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_tables,
                                const int32_t* table_rows, const int32_t* seq_lens, const int32_t* cu_seqlens,
                                void* out, int32_t n_seqs, int64_t n_tokens, int32_t n_heads, int32_t n_kv_heads,
                                int32_t head_dim, int32_t block_size, int64_t table_stride, int64_t q_stride,
                                int64_t out_stride, int64_t pool_block_stride, int64_t pool_pos_stride,
                                int64_t pool_head_stride, float scale, int dtype, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Step metadata and greedy sampling on the device.
 *
 * The host sends one packed int32 buffer per step: a header, one record per scheduled sequence
 * {seat, ctx, n_new, tok_off}, the block-table entries appended since the previous step
 * {seat, index, block}, and the token ids of prefill chunks. One kernel expands it into the static buffers
 * a CUDA graph reads, padded to the graph bucket with rows that only touch the garbage block.
 * Replaces the host-side list building of nanoserve/kv_manager.py:153-190 (begin_step / seq_input /
 * decode_meta / forward_kwargs / graph_inputs) and the per-step torch.tensor(...) uploads of
 * nanoserve/cuda_graphs.py:112-117 and :250-252.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t n_seqs;          /* real sequences this step */
    int32_t n_tokens;        /* real flattened tokens this step */
    int32_t pad_seqs;        /* sequences after padding to the graph bucket (>= n_seqs); padding = 1 token each */
    int32_t pad_tokens;      /* token rows to fill (>= n_tokens + pad_seqs - n_seqs) */
    int32_t n_appends;       /* block-table appends carried by this buffer */
    int32_t garbage_block;   /* block every padding row reads and writes */
    int32_t block_size;
    int32_t table_width;     /* row stride of the device block-table mirror */
} ns_step_header;

/* packed (device, int32): [ns_step_header][n_seqs x {seat, ctx, n_new, tok_off}][n_appends x {seat, index,
 * block}][token ids ...]. tok_off >= 0: the sequence's n_new token ids start at token ids[tok_off];
 * tok_off == -1: a single decode token read from last_tokens[seat] (left there by ns_argmax_rows).
 * Outputs: tokens / positions / slot_mapping int64 [pad_tokens]; cu_seqlens int32 [pad_seqs + 1]; seq_lens
 * int32 [pad_seqs]; seat_of int32 [pad_seqs] (row of table_mirror per sequence; padding -> pad_seat, whose
 * row must start with garbage_block); last_rows int64 [pad_seqs] (flattened row of each sequence's last token). */
int ns_build_step_metadata(const int32_t* packed, int32_t packed_ints, int32_t* table_mirror,
                           const int64_t* last_tokens, int32_t pad_seat, int64_t* tokens, int64_t* positions,
                           int64_t* slot_mapping, int32_t* cu_seqlens, int32_t* seq_lens, int32_t* seat_of,
                           int64_t* last_rows, int32_t max_seqs, int32_t max_tokens, void* stream);

/* out[r] = argmax(logits[r, :vocab]) (lowest index on ties); when seat_of != NULL also
 * last_tokens[seat_of[r]] = out[r], so the next step's decode token never leaves the device.
 * Replaces: nanoserve/engine.py:239 logits.argmax(-1) (the .tolist() copy stays with the caller). */
int ns_argmax_rows(const void* logits, int64_t row_stride, int32_t rows, int32_t vocab, int64_t* out,
                   const int32_t* seat_of, int64_t* last_tokens, int dtype, void* stream);

/* Sampling with temperature / top-k / top-p for the rows that ask for it, after ns_argmax_rows has filled `out`:
 * params is rows x 8 32-bit words {float temperature, float top_p, int32 top_k, int32 enabled, uint32 seed_lo,
 * uint32 seed_hi, 0, 0}. A row with enabled == 0 keeps its greedy token. Otherwise x = float(logit) / temperature;
 * top_k > 0 keeps x >= the k-th largest x; top_p < 1 keeps, in descending order of x, the tokens whose softmax mass
 * ranked above them is < top_p (equal values together; the best token always survives); the token is
 * argmax_j(x_j + g_j) over the survivors with Gumbel noise g_j = -log(-log(u_j)), u_j in [1e-20, 1 - 1e-7] drawn from a
 * counter-based generator keyed by (seed, j) - so a row's token depends only on its logits, its parameters and its
 * seed, never on its neighbours or its row index. The caller passes seed = mix_seed(request seed, tokens generated so
 * far). out / seat_of / last_tokens as in ns_argmax_rows. threshold_out (float [rows]) and kept_out (int32 [rows]) may
 * be NULL; when given they receive the smallest surviving x and the number of survivors of every enabled row.
 * Replaces: nanoserve/sampling.py:54-90 sample (called at nanoserve/engine.py:233-237). Individual draws differ from
 * the reference's (another random stream); kept set and distribution are the same. */
int ns_sample_rows(const void* logits, int64_t row_stride, int32_t rows, int32_t vocab, const void* params,
                   int64_t* out, const int32_t* seat_of, int64_t* last_tokens, float* threshold_out,
                   int32_t* kept_out, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NANOSERVE_B200_H */

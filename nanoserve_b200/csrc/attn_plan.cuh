// Workspace layout and per-step plan shared by the ragged paged-attention kernels.
//
// The plan is built once per engine step (ns_attn_plan) and reused by every layer:
//   * decode rows (one query token) are listed in batch order; their KV blocks form one flattened list of
//     `dec_total` block-units that is cut into contiguous ranges of (nearly) equal size, one per persistent
//     decode CTA (stream-K style): every CTA reads about the same number of bytes whatever the mix of context
//     lengths. A cut that falls close to a row boundary is moved onto it, and ranges are never smaller than
//     kMinBlocksPerCta, so short rows stay whole (no partials, no cross-CTA reduce);
//   * prefill rows are cut into query tiles, heaviest (latest) tile first.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace ns {

constexpr int kMaxDecodeCtas = 1024;      // upper bound on the persistent decode grid
constexpr int kMaxKvHeads = 8;            // counters per decode row
constexpr int kPrefillTileTokens = 16;    // query tokens per prefill work item
constexpr int kMinBlocksPerCta = 32;      // a decode CTA's range is never cut below this many 16-token blocks: splitting
                                          // a row costs a partial write, a fence, an atomic and a cross-CTA reduce. Timed
                                          // alone, 32 rows x ~500 tokens run faster with 8 (10.7 vs 13.1 us), but inside a
                                          // layer, where the kernel's start overlaps the QKV GEMM, 32 wins (7.3 vs 9.5 us)
constexpr int kSplitBlocks = 15360;       // steps with more decode KV blocks than this run two virtual CTAs per CTA.
                                          // Measured (hd 64, 14q/2kv, balanced ranges): up to ~14K blocks one 16-warp CTA per
                                          // SM is as fast or faster (32 rows x 500 tokens: 6.8 vs 12.1 us; 128 rows x 1400:
                                          // 17.3 vs 20.5; 48 rows x U[128,8192], 14.1K blocks: 24.2 vs 24.4); from ~16K blocks
                                          // two 8-warp halves win (256 rows x 1000: 23.6 vs 25.7; 27.5K blocks: 42.6 vs 44.4)
constexpr int kClusterBlocks = 6144;      // steps with at most this many decode KV blocks (and few enough rows) run in cluster
                                          // mode: every row gets a whole cluster of CTAs instead of one CTA
constexpr int kClusterSlackBlocks = 48;   // cluster mode is kept while (longest row / cluster) <= balanced range + this many blocks
constexpr int kSnapBlocks = 32;           // ranges up to twice this long per 8 warps may move a cut by half a range to
                                          // reach a row boundary (a whole row needs no partials); longer ranges by an eighth

struct PlanHeader {
    int32_t n_dec;          // decode rows
    int32_t dec_total;      // sum of their KV blocks
    int32_t dec_per_cta;    // block-units per decode CTA (>= 1)
    int32_t dec_ctas;       // decode CTAs that own a non-empty range
    int32_t n_prefill_items;
    int32_t n_seqs;
    int32_t block_size;
    int32_t mode;           // 1: one range per decode CTA; 2: every decode CTA runs two virtual CTAs of half its warps
    int32_t errors;         // bounded waits of the attention kernels that ran out (cumulative; only the host clears it:
                            // the plan kernel leaves this word alone, the workspace starts zero-filled)
    int32_t cluster;        // > 1: small step in cluster mode - decode row c is streamed by the `cluster` CTAs c*cluster ..
                            // c*cluster + cluster - 1 (one thread-block cluster when the kernel is launched with that cluster
                            // size), which combine through the first CTA's shared memory; 0: ranges as cut by the planner
    int32_t pad[6];
};

// Byte offsets inside the workspace; everything 256-byte aligned.
struct WsLayout {
    int64_t header;         // PlanHeader
    int64_t dec_info;       // int4[max_seqs]     decode row i: {batch index, seq_len, table row, query row}
    int64_t dec_indptr;     // int32[max_seqs+1]  first block-unit of decode row i
    int64_t cta_start;      // int32[kMaxDecodeCtas+1] first block-unit of each decode CTA (cut points)
    int64_t cta_first;      // int32[kMaxDecodeCtas+1] decode row holding the first block-unit of each CTA
    int64_t dec_span;       // int2[max_seqs] decode row i: {first CTA touching it, number of CTAs touching it}
    int64_t cta_rec;        // int4[2*max_ctas] per decode CTA: {u0, u1, first row, its first unit} {its end unit, len, table row, q row}
    int64_t counters;       // int32[max_seqs*kMaxKvHeads] arrivals per (decode row, kv head); zero between launches
    int64_t prefill_items;  // int2[max_prefill_items] (batch index, first query token of the tile)
    int64_t partials;       // float[kMaxDecodeCtas*2][n_heads][head_dim+4]
    int64_t total;
};

// Cluster size proposed for a step of n_seqs sequences on a grid of `ctas` persistent decode CTAs: the largest of 4, 2
// that divides the grid and leaves a cluster per sequence; 1 = none. The plan and the launch both derive it from the
// same two numbers, which a CUDA graph fixes at capture.
__host__ __device__ inline int plan_cluster(int n_seqs, int ctas) {
    if (n_seqs <= 0) return 1;
    if (ctas % 4 == 0 && n_seqs <= ctas / 4) return 4;
    if (ctas % 2 == 0 && n_seqs <= ctas / 2) return 2;
    return 1;
}

__host__ __device__ inline int64_t align256(int64_t v) { return (v + 255) & ~int64_t(255); }

__host__ __device__ inline WsLayout ws_layout(int max_seqs, int max_tokens, int n_heads, int head_dim,
                                              int max_ctas = kMaxDecodeCtas) {
    WsLayout L;
    int64_t o = 0;
    L.header = o;         o = align256(o + (int64_t)sizeof(PlanHeader));
    L.dec_info = o;       o = align256(o + 16 * (int64_t)max_seqs);
    L.dec_indptr = o;     o = align256(o + 4 * (int64_t)(max_seqs + 1));
    L.cta_start = o;      o = align256(o + 4 * (int64_t)(max_ctas + 1));
    L.cta_first = o;      o = align256(o + 4 * (int64_t)(max_ctas + 1));
    L.dec_span = o;       o = align256(o + 8 * (int64_t)max_seqs);
    L.cta_rec = o;        o = align256(o + 32 * (int64_t)max_ctas);
    L.counters = o;       o = align256(o + 4 * (int64_t)max_seqs * kMaxKvHeads);
    const int64_t max_items = (int64_t)max_tokens / kPrefillTileTokens + max_seqs + 1;
    L.prefill_items = o;  o = align256(o + 8 * max_items);
    L.partials = o;       o = align256(o + 4 * (int64_t)max_ctas * 2 * n_heads * (head_dim + 4));
    L.total = o;
    return L;
}

// Arguments shared by the tensor-core attention kernels (bf16).
struct AttnParams {
    const __nv_bfloat16* q;
    const __nv_bfloat16* k_pool;
    const __nv_bfloat16* v_pool;
    const int32_t* block_tables;
    const int32_t* table_rows;     // may be null: sequence s uses row s of block_tables
    const int32_t* seq_lens;
    const int32_t* cu_seqlens;     // may be null: sequence s owns exactly query row s
    __nv_bfloat16* out;
    uint8_t* ws;
    WsLayout L;
    int64_t table_stride, q_stride, out_stride, blk_stride, pos_stride, head_stride;
    int n_heads, n_kv_heads, group;
    float scale_log2;              // softmax scale * log2(e)
    long long* timeline;           // profiling hook, normally null: 4 globaltimer stamps per decode CTA
    // Mixed steps: the prefill kernel that follows the decode kernel in the stream does not depend on it (they read the
    // same Q / pools and write different rows of out). With this flag the decode kernel lets its successor be scheduled
    // only AFTER its own dependency wait (so Q and the new K/V rows exist when the prefill kernel starts), the prefill
    // kernel runs beside it and waits for the decode kernel's completion before it exits, which keeps the stream's
    // order for whatever comes next.
    int overlap_prefill = 0;
    // 1: the plan in `ws` was written by the launch directly before this one in the stream (a call that plans and
    // attends in one go). A kernel launched with programmatic stream serialization sees its predecessor's writes only
    // after griddepcontrol.wait, so the decode kernel then waits BEFORE its first read of the workspace instead of
    // prefetching plan records, block ids and K/V tiles ahead of the wait. 0: the plan is older (an engine step plans
    // once, several kernels before the first layer's attention) and the early reads are safe.
    int plan_fresh = 0;
    int n_seqs = 0;                // sequences of the call (sizes the thread-block cluster of small steps)
    int sm_count = 0;              // SMs of the device (the prefill kernel pairs heavy and light items on an SM)
};

}  // namespace ns

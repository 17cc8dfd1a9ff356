// C ABI glue: error reporting and the attention entry points (dispatch between the tensor-core kernels and
// the scalar kernel).
#include <cstdarg>
#include <cstdio>

#include "attn_plan.cuh"
#include "common.cuh"

namespace ns {

static thread_local char g_err[512] = "";

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
    return NS_OK;
}

// attn_plan.cu / attn_decode.cu / attn_prefill_mma.cu
int launch_attn_plan(const int32_t* seq_lens, const int32_t* cu_seqlens, const int32_t* table_rows, int n_seqs,
                     int block_size, int base_ctas, int max_mode,
                     void* ws, const WsLayout& L, int max_items, cudaStream_t st);
bool decode_fast_supported(int n_heads, int n_kv_heads, int head_dim, int block_size);
int launch_paged_decode(const AttnParams& p, int head_dim, int sms, cudaStream_t st);
int decode_grid(int head_dim, int sms);
int decode_max_mode(int head_dim);
bool prefill_mma_supported(int n_heads, int n_kv_heads, int head_dim, int block_size);
int launch_prefill_mma(const AttnParams& p, int head_dim, int max_items, cudaStream_t st);
bool prefill_tc_supported(int n_heads, int n_kv_heads, int head_dim, int block_size);
int launch_prefill_tc(const AttnParams& p, int max_items, cudaStream_t st);
static int g_prefill_impl = 0;          // 0 = tcgen05 where supported, 1 = always the mma.sync kernel
static int g_overlap_prefill = 1;       // 1 = the prefill kernel of a mixed step runs beside the decode kernel

static long long* g_timeline = nullptr;
static int g_sm_count = 0;
static int sm_count() {
    if (g_sm_count <= 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        g_sm_count = n;
    }
    return g_sm_count;
}

}  // namespace ns

using namespace ns;

namespace ns { void debug_set_min_blocks(int n); void debug_set_split_blocks(int n); void debug_set_snap_blocks(int n); }
extern "C" void ns_debug_snap_blocks(int n) { ns::debug_set_snap_blocks(n); }
namespace ns { void debug_set_balance(int on); }
// Debug hook (not part of the public header): 0 = equal cuts snapped to row boundaries also for large steps.
extern "C" void ns_debug_balance(int on) { ns::debug_set_balance(on); }
// Debug hook (not part of the public header): decode KV blocks above which a step runs two virtual CTAs per CTA (< 0 = default).
extern "C" void ns_debug_split_blocks(int n) { ns::debug_set_split_blocks(n); }
// Debug hook (not part of the public header): lower bound of a decode CTA's range in KV blocks (0 = default).
extern "C" void ns_debug_min_blocks(int n) { ns::debug_set_min_blocks(n); }

extern "C" int ns_version(void) { return 100; }
extern "C" const char* ns_last_error(void) { return g_err; }
extern "C" int ns_sm_count(void) { return sm_count(); }
extern "C" void ns_debug_decode_timeline(long long* device_buffer) { g_timeline = device_buffer; }
extern "C" void ns_debug_prefill_impl(int impl) { g_prefill_impl = impl; }
// Debug hook (not part of the public header): 0 = prefill kernel strictly after the decode kernel of the same call.
extern "C" void ns_debug_overlap_prefill(int on) { g_overlap_prefill = on; }

extern "C" int64_t ns_attn_workspace_bytes(int32_t max_seqs, int32_t max_tokens, int32_t n_heads, int32_t head_dim) {
    if (max_seqs <= 0 || max_tokens < 0 || n_heads <= 0 || head_dim <= 0) return -1;
    return ws_layout(max_seqs, max_tokens, n_heads, head_dim).total;
}

static int plan_impl(const int32_t* seq_lens, const int32_t* cu_seqlens, const int32_t* table_rows, int n_seqs, int block_size, void* ws,
                     int64_t ws_bytes, int ws_max_seqs, int ws_max_tokens, int n_heads, int head_dim, cudaStream_t st) {
    NS_REQUIRE(seq_lens && ws, NS_ERR_INVALID_ARG, "attn_plan: null pointer");
    NS_REQUIRE(n_seqs >= 0 && n_seqs <= ws_max_seqs, NS_ERR_WORKSPACE, "attn_plan: %d sequences > workspace capacity %d",
               n_seqs, ws_max_seqs);
    NS_REQUIRE(block_size > 0, NS_ERR_INVALID_ARG, "attn_plan: block_size %d", block_size);
    const WsLayout L = ws_layout(ws_max_seqs, ws_max_tokens, n_heads, head_dim);
    NS_REQUIRE(ws_bytes >= L.total, NS_ERR_WORKSPACE, "attn_plan: workspace of %lld bytes < %lld needed", (long long)ws_bytes,
               (long long)L.total);
    NS_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 255) == 0, NS_ERR_INVALID_ARG, "attn_plan: workspace not 256-byte aligned");
    const int sms = sm_count();
    NS_REQUIRE(sms > 0, NS_ERR_CUDA, "attn_plan: cannot query the SM count");
    const int ctas = decode_grid(head_dim, sms), max_mode = decode_max_mode(head_dim);
    NS_REQUIRE(ctas * max_mode <= kMaxDecodeCtas, NS_ERR_UNSUPPORTED, "attn_plan: %d decode CTAs exceed the workspace layout",
               ctas * max_mode);
    const int max_items = ws_max_tokens / kPrefillTileTokens + ws_max_seqs + 1;
    return launch_attn_plan(seq_lens, cu_seqlens, table_rows, n_seqs, block_size, ctas, max_mode, ws, L, max_items, st);
}

extern "C" int ns_attn_plan(const int32_t* seq_lens, const int32_t* cu_seqlens, const int32_t* table_rows,
                            int32_t n_seqs, int32_t block_size,
                            int32_t n_heads, int32_t head_dim, void* workspace, int64_t workspace_bytes,
                            int32_t ws_max_seqs, int32_t ws_max_tokens, void* stream) {
    return plan_impl(seq_lens, cu_seqlens, table_rows, n_seqs, block_size, workspace, workspace_bytes, ws_max_seqs,
                     ws_max_tokens, n_heads, head_dim, (cudaStream_t)stream);
}

extern "C" int ns_ragged_paged_attn(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_tables,
                                    const int32_t* table_rows, const int32_t* seq_lens, const int32_t* cu_seqlens,
                                    void* out, int32_t n_seqs, int64_t n_tokens, int32_t n_heads, int32_t n_kv_heads,
                                    int32_t head_dim, int32_t block_size, int64_t table_stride, int64_t q_stride,
                                    int64_t out_stride, int64_t pool_block_stride, int64_t pool_pos_stride,
                                    int64_t pool_head_stride, float scale, int dtype, void* workspace,
                                    int64_t workspace_bytes, int32_t ws_max_seqs, int32_t ws_max_tokens, void* stream) {
    NS_REQUIRE(q && k_pool && v_pool && block_tables && seq_lens && out, NS_ERR_INVALID_ARG, "ragged_paged_attn: null pointer");
    NS_REQUIRE(n_seqs >= 0 && n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && block_size > 0,
               NS_ERR_INVALID_ARG, "ragged_paged_attn: bad shape");
    NS_REQUIRE(n_heads % n_kv_heads == 0, NS_ERR_INVALID_ARG, "ragged_paged_attn: %d heads not divisible by %d kv heads",
               n_heads, n_kv_heads);
    NS_REQUIRE(cu_seqlens != nullptr || n_tokens == n_seqs, NS_ERR_INVALID_ARG,
               "ragged_paged_attn: without cu_seqlens every sequence has one token");
    if (n_seqs == 0 || n_tokens == 0) return NS_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const bool fast = dtype == NS_BF16 && decode_fast_supported(n_heads, n_kv_heads, head_dim, block_size) &&
                      prefill_mma_supported(n_heads, n_kv_heads, head_dim, block_size) && n_kv_heads <= kMaxKvHeads;
    if (!fast)
        return ns_ragged_paged_attn_simple(q, k_pool, v_pool, block_tables, table_rows, seq_lens, cu_seqlens, out, n_seqs,
                                           n_tokens, n_heads, n_kv_heads, head_dim, block_size, table_stride, q_stride,
                                           out_stride, pool_block_stride, pool_pos_stride, pool_head_stride, scale, dtype,
                                           stream);
    NS_REQUIRE(workspace, NS_ERR_INVALID_ARG, "ragged_paged_attn: workspace is null");
    NS_REQUIRE(n_seqs <= ws_max_seqs && n_tokens <= ws_max_tokens, NS_ERR_WORKSPACE,
               "ragged_paged_attn: batch (%d seqs, %lld tokens) exceeds workspace capacity (%d, %d)", n_seqs,
               (long long)n_tokens, ws_max_seqs, ws_max_tokens);
    const WsLayout L = ws_layout(ws_max_seqs, ws_max_tokens, n_heads, head_dim);
    NS_REQUIRE(workspace_bytes >= L.total, NS_ERR_WORKSPACE, "ragged_paged_attn: workspace of %lld bytes < %lld needed",
               (long long)workspace_bytes, (long long)L.total);
    NS_REQUIRE(q_stride % 8 == 0 && out_stride % 2 == 0 && pool_pos_stride % 8 == 0 && pool_head_stride % 8 == 0 &&
                   pool_block_stride % 8 == 0, NS_ERR_INVALID_ARG, "ragged_paged_attn: strides must keep 16-byte alignment");
    NS_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool)) & 15) == 0,
               NS_ERR_INVALID_ARG, "ragged_paged_attn: q / pools must be 16-byte aligned");
    NS_REQUIRE((reinterpret_cast<uintptr_t>(out) & 7) == 0 && out_stride % 4 == 0, NS_ERR_INVALID_ARG,
               "ragged_paged_attn: out must be 8-byte aligned with a row stride that is a multiple of 4 elements");
    const float kLog2e = 1.4426950408889634f;
    const int sms = sm_count();
    NS_REQUIRE(sms > 0 && decode_grid(head_dim, sms) * decode_max_mode(head_dim) <= kMaxDecodeCtas, NS_ERR_CUDA,
               "ragged_paged_attn: bad SM count");

    AttnParams a;
    a.q = (const __nv_bfloat16*)q; a.k_pool = (const __nv_bfloat16*)k_pool; a.v_pool = (const __nv_bfloat16*)v_pool;
    a.block_tables = block_tables; a.table_rows = table_rows; a.seq_lens = seq_lens; a.cu_seqlens = cu_seqlens;
    a.out = (__nv_bfloat16*)out; a.ws = (uint8_t*)workspace; a.L = L;
    a.table_stride = table_stride; a.q_stride = q_stride; a.out_stride = out_stride; a.blk_stride = pool_block_stride;
    a.pos_stride = pool_pos_stride; a.head_stride = pool_head_stride;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.group = n_heads / n_kv_heads; a.scale_log2 = scale * kLog2e;
    a.timeline = g_timeline;
    const bool has_prefill = cu_seqlens != nullptr && n_tokens > n_seqs;
    a.overlap_prefill = (has_prefill && g_overlap_prefill) ? 1 : 0;
    int rc = launch_paged_decode(a, head_dim, sms, st);
    if (rc != NS_OK) return rc;
    if (cu_seqlens != nullptr && n_tokens > n_seqs) {
        // Upper bound on prefill tiles from sizes the host knows (graph-safe).
        int64_t max_items = n_tokens / kPrefillTileTokens + n_seqs;
        const int64_t cap = (int64_t)ws_max_tokens / kPrefillTileTokens + ws_max_seqs + 1;
        if (max_items > cap) max_items = cap;
        if (g_prefill_impl == 0 && prefill_tc_supported(n_heads, n_kv_heads, head_dim, block_size))
            rc = launch_prefill_tc(a, (int)max_items, st);
        else
            rc = launch_prefill_mma(a, head_dim, (int)max_items, st);
    }
    return rc;
}

extern "C" int ns_paged_attn_decode(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_tables,
                                    const int32_t* context_lens, void* out, int32_t batch, int32_t n_heads,
                                    int32_t n_kv_heads, int32_t head_dim, int32_t block_size, int64_t table_stride,
                                    int64_t q_stride, int64_t out_stride, int64_t pool_block_stride,
                                    int64_t pool_pos_stride, int64_t pool_head_stride, float scale, int dtype,
                                    void* workspace, int64_t workspace_bytes, int32_t ws_max_seqs,
                                    int32_t ws_max_tokens, void* stream) {
    if (batch == 0) return NS_OK;
    NS_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, NS_ERR_INVALID_ARG, "paged_attn_decode: bad heads");
    const bool fast = dtype == NS_BF16 && decode_fast_supported(n_heads, n_kv_heads, head_dim, block_size) &&
                      prefill_mma_supported(n_heads, n_kv_heads, head_dim, block_size) && n_kv_heads <= kMaxKvHeads;
    if (fast) {
        const int rc = plan_impl(context_lens, nullptr, nullptr, batch, block_size, workspace, workspace_bytes, ws_max_seqs,
                                 ws_max_tokens, n_heads, head_dim, (cudaStream_t)stream);
        if (rc != NS_OK) return rc;
    }
    return ns_ragged_paged_attn(q, k_pool, v_pool, block_tables, nullptr, context_lens, nullptr, out, batch, batch, n_heads,
                                n_kv_heads, head_dim, block_size, table_stride, q_stride, out_stride, pool_block_stride,
                                pool_pos_stride, pool_head_stride, scale, dtype, workspace, workspace_bytes, ws_max_seqs,
                                ws_max_tokens, stream);
}

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
int launch_prefill_tc(const AttnParams& p, int head_dim, int max_items, cudaStream_t st);
// Process-wide tuning knobs (ns_set_tuning); read on the host when a call is issued.
static int g_tuning[NS_TUNE_COUNT] = {0, 1, -1, 0, 0, 2, 1, 0, 0};
// The workspace / stream of the newest ns_attn_plan issued by this thread that no attention call has used yet: the
// first attention launch after a plan on the same stream is its direct successor and must not read the plan ahead of
// its dependency wait (AttnParams::plan_fresh).
static thread_local const void* g_fresh_plan_ws = nullptr;
static thread_local cudaStream_t g_fresh_plan_stream = nullptr;

// Per-device SM count (a process may drive several GPUs).
static int g_sm_count[kMaxDevices] = {};
static int sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < kMaxDevices && g_sm_count[dev] > 0) return g_sm_count[dev];
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < kMaxDevices) g_sm_count[dev] = n;
    return n;
}

int device_sm_count() { return sm_count(); }

int prefill_cluster_size() {
    const int v = g_tuning[NS_TUNE_PREFILL_CLUSTER];
    return (v == 1 || v == 2 || v == 4) ? v : 0;
}

bool decode_cluster_enabled() { return g_tuning[NS_TUNE_DECODE_CLUSTER] != 0; }

void plan_knobs(int* min_blocks, int* split_blocks, int* snap_blocks, int* balance, int* cluster_on, int* cluster_blocks) {
    *cluster_on = g_tuning[NS_TUNE_DECODE_CLUSTER];
    *cluster_blocks = g_tuning[NS_TUNE_DECODE_CLUSTER_BLOCKS] > 0 ? g_tuning[NS_TUNE_DECODE_CLUSTER_BLOCKS] : kClusterBlocks;
    *min_blocks = g_tuning[NS_TUNE_DECODE_MIN_BLOCKS] > 0 ? g_tuning[NS_TUNE_DECODE_MIN_BLOCKS] : kMinBlocksPerCta;
    *split_blocks = g_tuning[NS_TUNE_DECODE_SPLIT_BLOCKS] >= 0 ? g_tuning[NS_TUNE_DECODE_SPLIT_BLOCKS] : kSplitBlocks;
    *snap_blocks = g_tuning[NS_TUNE_DECODE_SNAP_BLOCKS] > 0 ? g_tuning[NS_TUNE_DECODE_SNAP_BLOCKS] : kSnapBlocks;
    *balance = g_tuning[NS_TUNE_DECODE_BALANCE];
}

}  // namespace ns

using namespace ns;

extern "C" int ns_set_tuning(int knob, int value) {
    NS_REQUIRE(knob >= 0 && knob < NS_TUNE_COUNT, NS_ERR_INVALID_ARG, "set_tuning: unknown knob %d", knob);
    g_tuning[knob] = value;
    return NS_OK;
}
extern "C" int ns_get_tuning(int knob) { return (knob >= 0 && knob < NS_TUNE_COUNT) ? g_tuning[knob] : 0; }

extern "C" int ns_version(void) { return 101; }
extern "C" const char* ns_last_error(void) { return g_err; }
extern "C" int ns_sm_count(void) { return sm_count(); }

#ifdef NS_DEBUG_HOOKS
static long long* g_timeline = nullptr;
// Profiling build only: 4 globaltimer stamps per decode CTA are written to this device buffer.
extern "C" void ns_debug_decode_timeline(long long* device_buffer) { g_timeline = device_buffer; }
#else
static long long* const g_timeline = nullptr;
#endif

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
    const int rc = launch_attn_plan(seq_lens, cu_seqlens, table_rows, n_seqs, block_size, ctas, max_mode, ws, L, max_items, st);
    if (rc == NS_OK) {
        g_fresh_plan_ws = ws;
        g_fresh_plan_stream = st;
    }
    return rc;
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
    a.overlap_prefill = (has_prefill && g_tuning[NS_TUNE_PREFILL_OVERLAP]) ? 1 : 0;
    a.n_seqs = n_seqs;
    a.sm_count = sms;
    a.plan_fresh = (g_fresh_plan_ws == workspace && g_fresh_plan_stream == st) ? 1 : 0;
    g_fresh_plan_ws = nullptr;
    int rc = launch_paged_decode(a, head_dim, sms, st);
    if (rc != NS_OK) return rc;
    if (cu_seqlens != nullptr && n_tokens > n_seqs) {
        // Upper bound on prefill tiles from sizes the host knows (graph-safe).
        int64_t max_items = n_tokens / kPrefillTileTokens + n_seqs;
        const int64_t cap = (int64_t)ws_max_tokens / kPrefillTileTokens + ws_max_seqs + 1;
        if (max_items > cap) max_items = cap;
        rc = NS_ERR_UNSUPPORTED;
        if (g_tuning[NS_TUNE_PREFILL_IMPL] == 0 && prefill_tc_supported(n_heads, n_kv_heads, head_dim, block_size))
            rc = launch_prefill_tc(a, head_dim, (int)max_items, st);      // NS_ERR_UNSUPPORTED: no tensor map over these pools
        if (rc == NS_ERR_UNSUPPORTED) rc = launch_prefill_mma(a, head_dim, (int)max_items, st);
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

// ---- one status word per engine step -----------------------------------------------------------------------------
namespace ns {
int stream_gemm_error_counter(const unsigned int** out);
int thin_gemm_error_counter(const unsigned int** out);
int umma_gemm_error_counter(const unsigned int** out);
int skinny_gemm_error_counter(const unsigned int** out);
int check_error_counter(const unsigned int** out);
int tp_error_counter(const unsigned int** out);

__global__ void collect_status_kernel(const unsigned int* a, const unsigned int* b, const unsigned int* c, const unsigned int* d,
                                      const unsigned int* e, const unsigned int* f, const int32_t* ws_errors,
                                      int64_t* out) {
    if (threadIdx.x == 0)
        *out = (int64_t)*a + (int64_t)*b + (int64_t)*c + (int64_t)*d + (int64_t)*e + (int64_t)*f + (ws_errors != nullptr ? (int64_t)*ws_errors : 0);
}
}  // namespace ns

extern "C" int ns_collect_status(const void* attn_workspace, int64_t* status, void* stream) {
    NS_REQUIRE(status != nullptr, NS_ERR_INVALID_ARG, "collect_status: null pointer");
    const unsigned int *a = nullptr, *b = nullptr, *c = nullptr, *d = nullptr, *e = nullptr, *f = nullptr;
    int rc = thin_gemm_error_counter(&a);
    if (rc == NS_OK) rc = stream_gemm_error_counter(&b);
    if (rc == NS_OK) rc = umma_gemm_error_counter(&c);
    if (rc == NS_OK) rc = skinny_gemm_error_counter(&d);
    if (rc == NS_OK) rc = check_error_counter(&e);
    if (rc == NS_OK) rc = tp_error_counter(&f);
    if (rc != NS_OK) return rc;
    const int32_t* ws_errors = nullptr;
    if (attn_workspace != nullptr) {
        // the header is the first region of every layout, whatever the sizes it was built for
        const WsLayout L = ws_layout(1, 1, 1, 1);
        ws_errors = &reinterpret_cast<const PlanHeader*>(static_cast<const uint8_t*>(attn_workspace) + L.header)->errors;
    }
    collect_status_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(a, b, c, d, e, f, ws_errors, status);
    return check_launch("collect_status");
}

// Decode paged attention for callers that cannot allocate device memory.
//
// Who needs this: code that runs where cudaMalloc is off limits — inside a region that is being captured into a
// CUDA graph by somebody else, in a plugin whose host forbids allocations after start-up, or in a process whose
// memory pool is owned by another runtime that hands out no scratch. ns_paged_attn_decode wants a caller-owned
// workspace (plan + split-KV partials); here the same kernels run with that workspace placed in a fixed-size
// array that is part of the library image, so the caller passes inputs and outputs only.
//
// Costs and rules that follow from that:
//   * the array below occupies kStaticWsBytes on EVERY GPU that loads this library, until the process exits;
//   * sizes are capped (kStaticMaxBatch rows, kStaticMaxHeads query heads, head_dim <= kStaticMaxHeadDim); larger
//     requests are refused with NS_ERR_WORKSPACE, nothing is launched;
//   * all calls on one GPU share the one array and it keeps the previous call's contents: the arrival counters
//     are cleared at the start of every call, everything else is rewritten by the plan kernel before it is read;
//     two calls whose kernels overlap on the GPU (different streams, no dependency) race on it — serialise them;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
//     current). Make that first call outside any stream capture.
#include "attn_plan.cuh"
#include "common.cuh"

namespace ns {

int launch_attn_plan(const int32_t* seq_lens, const int32_t* cu_seqlens, const int32_t* table_rows, int n_seqs,
                     int block_size, int base_ctas, int max_mode, void* ws, const WsLayout& L, int max_items,
                     cudaStream_t st);
bool decode_fast_supported(int n_heads, int n_kv_heads, int head_dim, int block_size);
int launch_paged_decode(const AttnParams& p, int head_dim, int sms, cudaStream_t st);
int decode_grid(int head_dim, int sms);
int decode_max_mode(int head_dim);

constexpr int kStaticMaxBatch = 64;
constexpr int kStaticMaxHeads = 32;
constexpr int kStaticMaxHeadDim = 128;
constexpr int kStaticMaxCtas = 320;       // persistent decode CTAs the layout has room for (2 per SM up to 160 SMs)

// Upper bound of ws_layout(kStaticMaxBatch, kStaticMaxBatch, kStaticMaxHeads, kStaticMaxHeadDim, kStaticMaxCtas):
// partials 320*2*32*132*4 = 10.8 MB plus a few KB of plan arrays.
constexpr size_t kStaticWsBytes = 11 * 1024 * 1024;

// In host code this name is only a handle for cudaGetSymbolAddress — it is NOT a device pointer.
static __device__ __align__(256) unsigned char g_static_ws[kStaticWsBytes];

static unsigned char* g_ws_addr[kMaxDevices] = {};     // device address of g_static_ws, per device ordinal

// Device address of the array on the current device; resolved once per device.
static int static_ws_address(unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "paged_attn_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(NS_ERR_UNSUPPORTED, "paged_attn_decode_static: device ordinal %d", dev);
    if (g_ws_addr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_ws);
        if (e != cudaSuccess || ptr == nullptr)
            return fail(NS_ERR_CUDA, "paged_attn_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_ws_addr[dev] = static_cast<unsigned char*>(ptr);
    }
    *out = g_ws_addr[dev];
    return NS_OK;
}

}  // namespace ns

using namespace ns;

extern "C" int64_t ns_paged_attn_decode_static_bytes(void) { return (int64_t)kStaticWsBytes; }

extern "C" int ns_paged_attn_decode_static(const void* q, const void* k_pool, const void* v_pool,
                                           const int32_t* block_tables, const int32_t* context_lens, void* out,
                                           int32_t batch, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                                           int32_t block_size, int64_t table_stride, int64_t q_stride,
                                           int64_t out_stride, int64_t pool_block_stride, int64_t pool_pos_stride,
                                           int64_t pool_head_stride, float scale, int dtype, void* stream) {
    NS_REQUIRE(batch >= 0, NS_ERR_INVALID_ARG, "paged_attn_decode_static: negative batch");
    if (batch == 0) return NS_OK;
    NS_REQUIRE(q && k_pool && v_pool && block_tables && context_lens && out, NS_ERR_INVALID_ARG,
               "paged_attn_decode_static: null pointer");
    NS_REQUIRE(dtype == NS_BF16 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 &&
                   decode_fast_supported(n_heads, n_kv_heads, head_dim, block_size) && n_kv_heads <= kMaxKvHeads,
               NS_ERR_UNSUPPORTED,
               "paged_attn_decode_static: only the tensor-core layouts are offered here (bf16, block size 16, "
               "head_dim 64/128, GQA group <= 8)");
    NS_REQUIRE(batch <= kStaticMaxBatch && n_heads <= kStaticMaxHeads && head_dim <= kStaticMaxHeadDim, NS_ERR_WORKSPACE,
               "paged_attn_decode_static: batch %d / heads %d / head_dim %d exceed the built-in scratch (max %d / %d / %d); "
               "use ns_paged_attn_decode with a workspace of your own", batch, n_heads, head_dim, kStaticMaxBatch,
               kStaticMaxHeads, kStaticMaxHeadDim);
    NS_REQUIRE(q_stride % 8 == 0 && out_stride % 4 == 0 && pool_pos_stride % 8 == 0 && pool_head_stride % 8 == 0 &&
                   pool_block_stride % 8 == 0, NS_ERR_INVALID_ARG, "paged_attn_decode_static: strides must keep 16-byte alignment");
    NS_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 7) == 0, NS_ERR_INVALID_ARG, "paged_attn_decode_static: misaligned buffer");
    int dev = 0, sms = 0;
    NS_REQUIRE(cudaGetDevice(&dev) == cudaSuccess &&
                   cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0,
               NS_ERR_CUDA, "paged_attn_decode_static: cannot query the device");
    const int max_mode = decode_max_mode(head_dim);
    const int ctas = decode_grid(head_dim, sms) * max_mode;          // virtual CTAs the scratch must hold
    NS_REQUIRE(ctas <= kStaticMaxCtas, NS_ERR_WORKSPACE, "paged_attn_decode_static: %d decode CTAs exceed the built-in scratch (%d)",
               ctas, kStaticMaxCtas);
    const WsLayout L = ws_layout(kStaticMaxBatch, kStaticMaxBatch, n_heads, head_dim, kStaticMaxCtas);
    NS_REQUIRE((size_t)L.total <= kStaticWsBytes, NS_ERR_WORKSPACE, "paged_attn_decode_static: layout does not fit the built-in scratch");

    unsigned char* ws = nullptr;
    int rc = static_ws_address(&ws);
    if (rc != NS_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // the arrival counters must start at zero; an earlier call that was cut short may have left some behind
    cudaError_t e = cudaMemsetAsync(ws + L.counters, 0, 4 * (size_t)kStaticMaxBatch * kMaxKvHeads, st);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "paged_attn_decode_static: cudaMemsetAsync: %s", cudaGetErrorString(e));
    const int max_items = kStaticMaxBatch / kPrefillTileTokens + kStaticMaxBatch + 1;
    rc = launch_attn_plan(context_lens, nullptr, nullptr, batch, block_size, ctas / max_mode, max_mode, ws, L, max_items, st);
    if (rc != NS_OK) return rc;
    AttnParams a;
    a.q = (const __nv_bfloat16*)q; a.k_pool = (const __nv_bfloat16*)k_pool; a.v_pool = (const __nv_bfloat16*)v_pool;
    a.block_tables = block_tables; a.table_rows = nullptr; a.seq_lens = context_lens; a.cu_seqlens = nullptr;
    a.out = (__nv_bfloat16*)out; a.ws = ws; a.L = L;
    a.table_stride = table_stride; a.q_stride = q_stride; a.out_stride = out_stride; a.blk_stride = pool_block_stride;
    a.pos_stride = pool_pos_stride; a.head_stride = pool_head_stride;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.group = n_heads / n_kv_heads;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.timeline = nullptr;
    a.n_seqs = batch;
    a.plan_fresh = 1;                 // the plan kernel above is this launch's direct predecessor
    return launch_paged_decode(a, head_dim, sms, st);
}

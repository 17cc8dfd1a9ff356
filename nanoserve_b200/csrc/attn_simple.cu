// Scalar ragged paged attention: one warp per (query token, query head), fp32 everywhere.
//
// This is the accuracy-first implementation: it serves fp32 models (the strict parity gate), head layouts
// the tensor-core kernels do not cover, and on-device cross-checks of the fast kernels. Keys are taken 32
// at a time: each lane scores one key (a full dot product against the query, which sits in shared memory),
// the warp agrees on the running max, then the 32 probabilities are broadcast one by one while each lane
// accumulates its own slice of the head dimension of P.V.
#include "common.cuh"

namespace ns {

constexpr int kSimpleWarps = 4;
constexpr int kSimpleMaxHd = 256;

template <typename T>
__global__ void __launch_bounds__(kSimpleWarps * 32) ragged_attn_simple_kernel(
    const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
    const int32_t* __restrict__ block_tables, const int32_t* __restrict__ table_rows,
    const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ cu_seqlens, T* __restrict__ out, int n_seqs, int64_t n_tokens, int NH, int NKV, int HD,
    int block_size, int64_t table_stride, int64_t q_stride, int64_t out_stride, int64_t blk_stride,
    int64_t pos_stride, int64_t head_stride, float scale) {
    __shared__ float q_sm[kSimpleWarps][kSimpleMaxHd];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * kSimpleWarps + warp;
    if (unit >= n_tokens * NH) return;
    const int64_t t = unit / NH;
    const int h = (int)(unit - t * NH);
    const int g = h / (NH / NKV);

    // sequence owning flattened token t
    int s, j, T_new;
    if (cu_seqlens == nullptr) {
        s = (int)t; j = 0; T_new = 1;
    } else {
        int lo = 0, hi = n_seqs;              // cu[lo] <= t < cu[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (cu_seqlens[mid] <= t) lo = mid; else hi = mid;
        }
        s = lo;
        j = (int)(t - cu_seqlens[s]);
        T_new = cu_seqlens[s + 1] - cu_seqlens[s];
    }
    const int n_keys = seq_lens[s] - T_new + j + 1;   // causal: query j sees keys 0 .. ctx + j
    const T* qrow = q + t * q_stride + (int64_t)h * HD;
    for (int d = lane; d < HD; d += 32) q_sm[warp][d] = to_f32(qrow[d]);
    __syncwarp();
    const int32_t* table = block_tables + (int64_t)(table_rows ? table_rows[s] : s) * table_stride;

    float m = -INFINITY, l = 0.f;
    float acc[kSimpleMaxHd / 32];
#pragma unroll
    for (int i = 0; i < kSimpleMaxHd / 32; ++i) acc[i] = 0.f;

    for (int base = 0; base < n_keys; base += 32) {
        const int key = base + lane;
        float sc = -INFINITY;
        int64_t row_off = 0;
        if (key < n_keys) {
            const int blk = table[key / block_size];
            row_off = (int64_t)blk * blk_stride + (int64_t)(key % block_size) * pos_stride + (int64_t)g * head_stride;
            const T* kr = k_pool + row_off;
            float dot = 0.f;
            for (int d = 0; d < HD; ++d) dot = fmaf(q_sm[warp][d], to_f32(kr[d]), dot);
            sc = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(sc));
        const float alpha = expf(m - m_new);
        const float pr = key < n_keys ? expf(sc - m_new) : 0.f;
        l = l * alpha + warp_sum(pr);
        m = m_new;
#pragma unroll
        for (int i = 0; i < kSimpleMaxHd / 32; ++i) acc[i] *= alpha;
        const int cnt = min(32, n_keys - base);
        for (int kk = 0; kk < cnt; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, pr, kk);
            const int64_t ro = __shfl_sync(0xffffffffu, row_off, kk);
            const T* vr = v_pool + ro;
#pragma unroll
            for (int i = 0; i < kSimpleMaxHd / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < HD) acc[i] = fmaf(pk, to_f32(vr[d]), acc[i]);
            }
        }
    }
    T* orow = out + t * out_stride + (int64_t)h * HD;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < kSimpleMaxHd / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < HD) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

}  // namespace ns

using namespace ns;

extern "C" int ns_ragged_paged_attn_simple(const void* q, const void* k_pool, const void* v_pool,
                                           const int32_t* block_tables, const int32_t* table_rows,
                                           const int32_t* seq_lens, const int32_t* cu_seqlens, void* out, int32_t n_seqs, int64_t n_tokens,
                                           int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, int32_t block_size,
                                           int64_t table_stride, int64_t q_stride, int64_t out_stride,
                                           int64_t pool_block_stride, int64_t pool_pos_stride,
                                           int64_t pool_head_stride, float scale, int dtype, void* stream) {
    NS_REQUIRE(q && k_pool && v_pool && block_tables && seq_lens && out, NS_ERR_INVALID_ARG, "attn_simple: null pointer");
    NS_REQUIRE(n_seqs >= 0 && n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && block_size > 0, NS_ERR_INVALID_ARG,
               "attn_simple: bad shape");
    NS_REQUIRE(n_heads % n_kv_heads == 0, NS_ERR_INVALID_ARG, "attn_simple: %d heads not divisible by %d kv heads",
               n_heads, n_kv_heads);
    NS_REQUIRE(head_dim > 0 && head_dim <= kSimpleMaxHd, NS_ERR_UNSUPPORTED, "attn_simple: head_dim %d > %d", head_dim,
               kSimpleMaxHd);
    NS_REQUIRE(cu_seqlens != nullptr || n_tokens == n_seqs, NS_ERR_INVALID_ARG,
               "attn_simple: without cu_seqlens every sequence has one token");
    if (n_tokens == 0 || n_seqs == 0) return NS_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t units = n_tokens * n_heads;
    const unsigned grid = (unsigned)((units + kSimpleWarps - 1) / kSimpleWarps);
    if (dtype == NS_BF16)
        ragged_attn_simple_kernel<__nv_bfloat16><<<grid, kSimpleWarps * 32, 0, st>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, block_tables, table_rows,
            seq_lens, cu_seqlens, (__nv_bfloat16*)out, n_seqs, n_tokens, n_heads, n_kv_heads, head_dim, block_size, table_stride,
            q_stride, out_stride, pool_block_stride, pool_pos_stride, pool_head_stride, scale);
    else if (dtype == NS_F32)
        ragged_attn_simple_kernel<float><<<grid, kSimpleWarps * 32, 0, st>>>(
            (const float*)q, (const float*)k_pool, (const float*)v_pool, block_tables, table_rows, seq_lens, cu_seqlens,
            (float*)out, n_seqs, n_tokens, n_heads, n_kv_heads, head_dim, block_size, table_stride, q_stride,
            out_stride, pool_block_stride, pool_pos_stride, pool_head_stride, scale);
    else
        return fail(NS_ERR_UNSUPPORTED, "attn_simple: dtype %d", dtype);
    return check_launch("ragged_attn_simple");
}

// Decode paged attention for sm_100a: HBM-bound GQA over 16-token KV blocks.
//
// Grid  : one persistent CTA per SM. The flattened list of (decode row, KV block) units is cut into equal
//         contiguous ranges (attn_plan.cuh), so every CTA streams the same number of bytes.
// Warp  : owns one KV head and every (warps-per-head)-th block of the CTA's range. It runs its own
//         cp.async ring (STAGES tiles of 16 tokens, K and V, 128-bit copies, XOR-swizzled rows) with no
//         CTA-wide barrier in the steady state, so up to (STAGES-1) tiles per warp are always in flight.
// Math  : the GROUP (<= 8) query heads sharing the KV head are rows 0..GROUP-1 of an m16n8k16 bf16 MMA tile
//         (rows 8..15 are zero); scores and the running max / sum are fp32, probabilities are rounded to
//         bf16 before P.V, the row max is reduced with warp shuffles (online softmax).
// Split : a row whose blocks span several warps / CTAs is combined in two levels: the warps of one head
//         through shared memory, CTAs through fp32 partials in the workspace, where the LAST CTA to arrive
//         (atomic counter, no waiting) does the final reduction. Counters are left at zero.
#include "attn_plan.cuh"
#include "common.cuh"

namespace ns {

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Byte offset of 16-byte chunk `chunk` of row `row` inside a [rows x HD] bf16 tile with XOR-swizzled chunks
// (ldmatrix reads 8 rows x 16 bytes at a time: the swizzle spreads them over all banks).
template <int HD> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    constexpr int CPR = HD / 8;   // chunks per row
    return (uint32_t)(row * (HD * 2) + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4));
    (void)CPR;
}

template <int HD, int NWARPS, int STAGES>
__global__ void __launch_bounds__(NWARPS * 32, 1) paged_decode_kernel(const AttnParams p) {
    constexpr int CPR = HD / 8;                       // 16-byte chunks per K/V row
    constexpr int KV_TILE = 16 * HD * 2;              // bytes of one K (or V) tile
    constexpr int Q_TILE = 8 * HD * 2;                // 8 query rows
    constexpr int STAGE_BYTES = 2 * KV_TILE + Q_TILE;
    constexpr int RED_ROW = HD + 2;                   // floats: O[HD], m, l
    extern __shared__ __align__(128) uint8_t smem[];

    const PlanHeader* hdr = reinterpret_cast<const PlanHeader*>(p.ws + p.L.header);
    const int per = hdr->dec_per_cta;
    const int total = hdr->dec_total;
    const int cta = blockIdx.x;
    const long long start = (long long)cta * per;
    if (start >= total) return;
    const int u0 = (int)start;
    const int u1 = min(u0 + per, total);

    const int32_t* __restrict__ dec_seq = reinterpret_cast<const int32_t*>(p.ws + p.L.dec_seq);
    const int32_t* __restrict__ indptr = reinterpret_cast<const int32_t*>(p.ws + p.L.dec_indptr);
    const int32_t* __restrict__ cta_first = reinterpret_cast<const int32_t*>(p.ws + p.L.cta_first);
    int32_t* counters = reinterpret_cast<int32_t*>(p.ws + p.L.counters);
    float* partials = reinterpret_cast<float*>(p.ws + p.L.partials);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NKV = p.n_kv_heads;
    const int g = warp % NKV;                 // KV head of this warp
    const int stripe = warp / NKV;            // which share of the blocks
    const int wph = NWARPS / NKV;             // warps per head
    const int GROUP = p.group;
    const int gt = stripe * 32 + lane;        // thread index inside the head group
    const int gthreads = wph * 32;

    uint8_t* my_stages = smem + (size_t)warp * STAGES * STAGE_BYTES;
    float* red = reinterpret_cast<float*>(smem + (size_t)NWARPS * STAGES * STAGE_BYTES);   // [NWARPS][8][RED_ROW]
    __shared__ int last_flag[kMaxKvHeads];

    const int i_first = cta_first[cta];

    // ---- prefetch cursor (runs STAGES-1 tiles ahead of the compute cursor) ------------------------------------
    int pf_i = i_first, pf_hi = indptr[i_first + 1], pf_lo = indptr[i_first];
    int pf_seq = dec_seq[pf_i], pf_len = p.seq_lens[pf_seq];
    const int32_t* pf_table = p.block_tables + (int64_t)(p.table_rows ? p.table_rows[pf_seq] : pf_seq) * p.table_stride;
    int pf_q_staged = -1;                     // decode row whose Q was last staged by this warp

    auto issue = [&](int t) {
        const int u = u0 + stripe + wph * t;
        if (u < u1) {
            while (u >= pf_hi) {
                ++pf_i;
                pf_lo = pf_hi;
                pf_hi = indptr[pf_i + 1];
                pf_seq = dec_seq[pf_i];
                pf_len = p.seq_lens[pf_seq];
                pf_table = p.block_tables + (int64_t)(p.table_rows ? p.table_rows[pf_seq] : pf_seq) * p.table_stride;
            }
            uint8_t* st = my_stages + (size_t)(t % STAGES) * STAGE_BYTES;
            const int j = u - pf_lo;
            const int blk = pf_table[j];
            const int valid = min(16, pf_len - 16 * j);
            const __nv_bfloat16* kb = p.k_pool + (int64_t)blk * p.blk_stride + (int64_t)g * p.head_stride;
            const __nv_bfloat16* vb = p.v_pool + (int64_t)blk * p.blk_stride + (int64_t)g * p.head_stride;
            const uint32_t ks = smem_u32(st), vs = ks + KV_TILE;
#pragma unroll
            for (int it = 0; it < (16 * CPR) / 32; ++it) {
                const int qd = it * 32 + lane;
                const int row = qd / CPR, ch = qd % CPR;
                const int nbytes = row < valid ? 16 : 0;
                const int64_t goff = (int64_t)row * p.pos_stride + ch * 8;
                cp_async16(ks + tile_off<HD>(row, ch), kb + goff, nbytes);
                cp_async16(vs + tile_off<HD>(row, ch), vb + goff, nbytes);
            }
            if (pf_q_staged != pf_i) {
                pf_q_staged = pf_i;
                const int64_t qrow = p.cu_seqlens ? p.cu_seqlens[pf_seq] : pf_seq;
                const __nv_bfloat16* qb = p.q + qrow * p.q_stride + (int64_t)g * GROUP * HD;
                const uint32_t qs = vs + KV_TILE;
#pragma unroll
                for (int it = 0; it < (8 * CPR + 31) / 32; ++it) {
                    const int qd = it * 32 + lane;
                    if (qd < 8 * CPR) {
                        const int row = qd / CPR, ch = qd % CPR;
                        cp_async16(qs + tile_off<HD>(row, ch), qb + row * HD + ch * 8, row < GROUP ? 16 : 0);
                    }
                }
            }
        }
        cp_async_commit();
    };

    // ---- running state of this warp for the current decode row ---------------------------------------------------
    float m_run = -INFINITY, l_run = 0.f;     // row = lane/4; l is this lane's share of the row sum
    float o[HD / 8][2];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = 0.f;
    uint32_t qa[HD / 16][2];                  // A fragments (rows 0..7): [k-step][k-low, k-high]
    int cc_i = i_first, cc_lo = indptr[i_first], cc_hi = indptr[i_first + 1];
    int cc_len = p.seq_lens[dec_seq[i_first]];
    int qa_row = -1;

    const int row8 = lane >> 2;               // MMA accumulator row of this lane
    const int colp = (lane & 3) * 2;          // first of its two columns inside an 8-wide n-tile

    // Combine the warps of this head for decode row i, then write the final output or a partial.
    auto flush = [&](int i) {
        float* mine = red + (size_t)warp * 8 * RED_ROW;
        float lsum = l_run;
        lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
        lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
#pragma unroll
        for (int d = 0; d < HD / 8; ++d)
            *reinterpret_cast<float2*>(mine + row8 * RED_ROW + d * 8 + colp) = make_float2(o[d][0], o[d][1]);
        if ((lane & 3) == 0) {
            mine[row8 * RED_ROW + HD] = m_run;
            mine[row8 * RED_ROW + HD + 1] = lsum;
        }
        named_barrier(1 + g, gthreads);

        const int lo = indptr[i], hi = indptr[i + 1];
        const bool complete = lo >= u0 && hi <= u1;
        const int s = dec_seq[i];
        const int64_t qrow = p.cu_seqlens ? p.cu_seqlens[s] : s;
        const int slot = (i == i_first) ? 0 : 1;
        float* part = partials + ((size_t)(cta * 2 + slot) * p.n_heads + (size_t)g * GROUP) * RED_ROW;
        for (int e = gt; e < GROUP * HD; e += gthreads) {
            const int r = e / HD, c = e - r * HD;
            float M = -INFINITY;
            for (int w = 0; w < wph; ++w) M = fmaxf(M, red[((size_t)(g + NKV * w) * 8 + r) * RED_ROW + HD]);
            float acc = 0.f, Ls = 0.f;
            for (int w = 0; w < wph; ++w) {
                const float* rw = red + ((size_t)(g + NKV * w) * 8 + r) * RED_ROW;
                const float sc = fast_exp2(rw[HD] - M);
                acc = fmaf(sc, rw[c], acc);
                Ls = fmaf(sc, rw[HD + 1], Ls);
            }
            if (complete) {
                p.out[qrow * p.out_stride + (int64_t)(g * GROUP + r) * HD + c] = __float2bfloat16_rn(Ls > 0.f ? acc / Ls : 0.f);
            } else {
                part[r * RED_ROW + c] = acc;
                if (c == 0) {
                    part[r * RED_ROW + HD] = M;
                    part[r * RED_ROW + HD + 1] = Ls;
                }
            }
        }
        if (!complete) {
            // Last-arriver reduction: publish the partial, count arrivals for (row, head); whoever completes the
            // count owns the final combine. Nobody waits.
            const int c_first = lo / per, c_last = (hi - 1) / per;
            __threadfence();
            named_barrier(1 + g, gthreads);
            if (gt == 0) {
                const int old = atomicAdd(&counters[i * kMaxKvHeads + g], 1);
                last_flag[g] = (old == c_last - c_first);
            }
            named_barrier(1 + g, gthreads);
            if (last_flag[g]) {
                __threadfence();
                for (int e = gt; e < GROUP * HD; e += gthreads) {
                    const int r = e / HD, c = e - r * HD;
                    float M = -INFINITY;
                    for (int cc = c_first; cc <= c_last; ++cc) {
                        const int sl = (__ldcg(&cta_first[cc]) == i) ? 0 : 1;
                        const float* pr = partials + ((size_t)(cc * 2 + sl) * p.n_heads + (size_t)g * GROUP + r) * RED_ROW;
                        M = fmaxf(M, __ldcg(pr + HD));
                    }
                    float acc = 0.f, Ls = 0.f;
                    for (int cc = c_first; cc <= c_last; ++cc) {
                        const int sl = (__ldcg(&cta_first[cc]) == i) ? 0 : 1;
                        const float* pr = partials + ((size_t)(cc * 2 + sl) * p.n_heads + (size_t)g * GROUP + r) * RED_ROW;
                        const float sc = fast_exp2(__ldcg(pr + HD) - M);
                        acc = fmaf(sc, __ldcg(pr + c), acc);
                        Ls = fmaf(sc, __ldcg(pr + HD + 1), Ls);
                    }
                    p.out[qrow * p.out_stride + (int64_t)(g * GROUP + r) * HD + c] = __float2bfloat16_rn(Ls > 0.f ? acc / Ls : 0.f);
                }
                if (gt == 0) counters[i * kMaxKvHeads + g] = 0;
            }
        }
        named_barrier(1 + g, gthreads);       // `red` may be overwritten after this point
        m_run = -INFINITY;
        l_run = 0.f;
#pragma unroll
        for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = 0.f;
    };

    // ---- pipeline ---------------------------------------------------------------------------------------------------
    const int my_tiles = (u1 - u0 - stripe + wph - 1) / wph;      // may be <= 0
#pragma unroll
    for (int t = 0; t < STAGES - 1; ++t) issue(t);

    for (int t = 0; t < my_tiles; ++t) {
        cp_async_wait<STAGES - 2>();          // tile t has landed (one commit group per tile, empty or not)
        __syncwarp();
        issue(t + STAGES - 1);                // refills the stage computed in iteration t-1

        const int u = u0 + stripe + wph * t;
        while (u >= cc_hi) {
            flush(cc_i);
            ++cc_i;
            cc_lo = cc_hi;
            cc_hi = indptr[cc_i + 1];
            cc_len = p.seq_lens[dec_seq[cc_i]];
        }
        const uint8_t* st = my_stages + (size_t)(t % STAGES) * STAGE_BYTES;
        const uint32_t ks = smem_u32(st), vs = ks + KV_TILE, qs = vs + KV_TILE;
        if (qa_row != cc_i) {                 // first tile of this row for this warp: its Q came with this stage
            qa_row = cc_i;
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk += 2) {
                // matrices: (rows 0-7, chunk 2kk), (2kk+1), (2kk+2), (2kk+3)
                const int ch = 2 * kk + (lane >> 3);
                ldmatrix_x4(qs + tile_off<HD>(lane & 7, ch), qa[kk][0], qa[kk][1], qa[kk + 1][0], qa[kk + 1][1]);
            }
        }
        const int valid = min(16, cc_len - 16 * (u - cc_lo));

        // S = Q K^T : two n-tiles of 8 tokens
        float sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            uint32_t b00, b01, b10, b11;
            const int row = (lane & 7) + ((lane >> 4) << 3);
            const int ch = 2 * kk + ((lane >> 3) & 1);
            ldmatrix_x4(ks + tile_off<HD>(row, ch), b00, b01, b10, b11);
            const uint32_t a[4] = {qa[kk][0], 0u, qa[kk][1], 0u};
            mma_bf16_16816(sc[0], a, b00, b01);
            mma_bf16_16816(sc[1], a, b10, b11);
        }
        // online softmax on row `row8` (4 lanes share a row; each holds 4 of its 16 scores)
        float x[4];
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tk = 8 * j + colp + e;
                const float v = tk < valid ? sc[j][e] * p.scale_log2 : -INFINITY;
                x[2 * j + e] = v;
                mx = fmaxf(mx, v);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float alpha = fast_exp2(m_run - m_new);
        float psum = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            x[e] = fast_exp2(x[e] - m_new);
            psum += x[e];
        }
        l_run = fmaf(l_run, alpha, psum);
        m_run = m_new;
        const uint32_t pa[4] = {pack_bf16x2(x[0], x[1]), 0u, pack_bf16x2(x[2], x[3]), 0u};
        // O = alpha * O + P V
#pragma unroll
        for (int dd = 0; dd < HD / 16; ++dd) {
            uint32_t v00, v01, v10, v11;
            const int row = (lane & 7) + (((lane >> 3) & 1) << 3);
            const int ch = 2 * dd + (lane >> 4);
            ldmatrix_x4_trans(vs + tile_off<HD>(row, ch), v00, v01, v10, v11);
            float acc0[4] = {o[2 * dd][0] * alpha, o[2 * dd][1] * alpha, 0.f, 0.f};
            float acc1[4] = {o[2 * dd + 1][0] * alpha, o[2 * dd + 1][1] * alpha, 0.f, 0.f};
            mma_bf16_16816(acc0, pa, v00, v01);
            mma_bf16_16816(acc1, pa, v10, v11);
            o[2 * dd][0] = acc0[0];
            o[2 * dd][1] = acc0[1];
            o[2 * dd + 1][0] = acc1[0];
            o[2 * dd + 1][1] = acc1[1];
        }
    }
    cp_async_wait<0>();
    // Every warp of a head walks every decode row of the CTA's range, with or without tiles of its own, so the
    // group barriers inside flush() always match.
    while (cc_hi < u1) {
        flush(cc_i);
        ++cc_i;
        cc_lo = cc_hi;
        cc_hi = indptr[cc_i + 1];
    }
    flush(cc_i);
}

template <int HD, int NWARPS, int STAGES> static int launch_decode_cfg(const AttnParams& p, int grid, cudaStream_t st) {
    constexpr int smem = NWARPS * STAGES * (2 * 16 * HD * 2 + 8 * HD * 2) + NWARPS * 8 * (HD + 2) * 4;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(paged_decode_kernel<HD, NWARPS, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "decode attention: cannot reserve %d bytes of shared memory: %s",
                                          smem, cudaGetErrorString(e));
        configured = true;
    }
    paged_decode_kernel<HD, NWARPS, STAGES><<<grid, NWARPS * 32, smem, st>>>(p);
    return check_launch("paged_decode");
}

// Returns NS_ERR_UNSUPPORTED (without setting an error) when this layout has no fast kernel.
bool decode_fast_supported(int n_heads, int n_kv_heads, int head_dim, int block_size) {
    if (block_size != 16 || n_heads % n_kv_heads != 0) return false;
    const int group = n_heads / n_kv_heads;
    if (group > 8) return false;
    if (head_dim == 64) return n_kv_heads == 1 || n_kv_heads == 2 || n_kv_heads == 4 || n_kv_heads == 8;
    if (head_dim == 128) return n_kv_heads == 1 || n_kv_heads == 2 || n_kv_heads == 3 || n_kv_heads == 6 ||
                                n_kv_heads == 4 || n_kv_heads == 8;
    return false;
}

int launch_paged_decode(const AttnParams& p, int head_dim, int grid, cudaStream_t st) {
    if (head_dim == 64) return launch_decode_cfg<64, 8, 4>(p, grid, st);
    if (p.n_kv_heads == 4 || p.n_kv_heads == 8) return launch_decode_cfg<128, 8, 2>(p, grid, st);
    return launch_decode_cfg<128, 6, 3>(p, grid, st);
}

}  // namespace ns

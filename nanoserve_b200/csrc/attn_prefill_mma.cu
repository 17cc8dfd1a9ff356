// Prefill-chunk paged attention with warp-level bf16 MMA (m16n8k16), FlashAttention-2 style.
//
// Work item = (sequence, 16 query tokens, KV head). The CTA has one warp per query head of the GQA group, so
// the K/V tiles (64 keys = 4 pool blocks, staged with 128-bit cp.async into XOR-swizzled shared memory,
// 3-stage ring) are fetched once and shared by all heads of the group. Query j of a chunk sitting on `ctx`
// cached tokens sees keys 0 .. ctx + j. Scores, running max and sum are fp32; P is rounded to bf16 for P.V.
#include "attn_plan.cuh"
#include "common.cuh"

namespace ns {

__device__ __forceinline__ float pf_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int HD> __device__ __forceinline__ uint32_t pf_tile_off(int row, int chunk) {
    return (uint32_t)(row * (HD * 2) + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4));
}

template <int HD, int STAGES>
__global__ void __launch_bounds__(256) prefill_mma_kernel(const AttnParams p) {
    constexpr int BN = 64;                     // keys per tile
    constexpr int CPR = HD / 8;
    constexpr int TILE = BN * HD * 2;          // bytes of one K (or V) tile
    extern __shared__ __align__(128) uint8_t smem[];

    const PlanHeader* hdr = reinterpret_cast<const PlanHeader*>(p.ws + p.L.header);
    if ((int)blockIdx.x >= hdr->n_prefill_items) {
        if (p.overlap_prefill) pdl_wait();        // the grid must not complete before the decode kernel it overlaps
        return;
    }
    const int2 item = reinterpret_cast<const int2*>(p.ws + p.L.prefill_items)[blockIdx.x];
    const int s = item.x, q_start = item.y;
    const int g = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = g * p.group + warp;
    const int q0 = p.cu_seqlens[s];
    const int T = p.cu_seqlens[s + 1] - q0;
    const int len = p.seq_lens[s];
    const int ctx = len - T;
    const int32_t* table = p.block_tables + (int64_t)(p.table_rows ? p.table_rows[s] : s) * p.table_stride;
    const int kv_end = min(len, ctx + q_start + kPrefillTileTokens);    // keys any row of this tile can see
    const int n_tiles = (kv_end + BN - 1) / BN;

    const int r0 = lane >> 2, colp = (lane & 3) * 2;
    // Q fragments straight from global memory (once per CTA).
    uint32_t qa[HD / 16][4];
    {
        const int tok0 = q_start + r0, tok1 = tok0 + 8;
        const __nv_bfloat16* qr0 = p.q + (int64_t)(q0 + tok0) * p.q_stride + (int64_t)h * HD;
        const __nv_bfloat16* qr1 = p.q + (int64_t)(q0 + tok1) * p.q_stride + (int64_t)h * HD;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            const int c = 16 * kk + colp;
            qa[kk][0] = tok0 < T ? *reinterpret_cast<const uint32_t*>(qr0 + c) : 0u;
            qa[kk][1] = tok1 < T ? *reinterpret_cast<const uint32_t*>(qr1 + c) : 0u;
            qa[kk][2] = tok0 < T ? *reinterpret_cast<const uint32_t*>(qr0 + c + 8) : 0u;
            qa[kk][3] = tok1 < T ? *reinterpret_cast<const uint32_t*>(qr1 + c + 8) : 0u;
        }
    }

    auto load_tile = [&](int kt) {
        if (kt < n_tiles) {
            const uint32_t ks = smem_u32(smem + (size_t)(kt % STAGES) * 2 * TILE), vs = ks + TILE;
            for (int qd = threadIdx.x; qd < BN * CPR; qd += blockDim.x) {
                const int row = qd / CPR, ch = qd - row * CPR;
                const int key = kt * BN + row;
                const bool ok = key < len;
                const int blk = ok ? table[key >> 4] : 0;
                const int64_t goff = (int64_t)blk * p.blk_stride + (int64_t)(key & 15) * p.pos_stride +
                                     (int64_t)g * p.head_stride + ch * 8;
                cp_async16(ks + pf_tile_off<HD>(row, ch), p.k_pool + goff, ok ? 16 : 0);
                cp_async16(vs + pf_tile_off<HD>(row, ch), p.v_pool + goff, ok ? 16 : 0);
            }
        }
        cp_async_commit();
    };

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) load_tile(st);

    const int lim0 = ctx + q_start + r0;       // last visible key of row r0; row r0+8 sees 8 more
    for (int kt = 0; kt < n_tiles; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        load_tile(kt + STAGES - 1);
        const uint32_t ks = smem_u32(smem + (size_t)(kt % STAGES) * 2 * TILE), vs = ks + TILE;

        float sc[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
            for (int pr = 0; pr < BN / 16; ++pr) {
                uint32_t b00, b01, b10, b11;
                const int row = 16 * pr + (lane & 7) + ((lane >> 4) << 3);
                const int ch = 2 * kk + ((lane >> 3) & 1);
                ldmatrix_x4(ks + pf_tile_off<HD>(row, ch), b00, b01, b10, b11);
                mma_bf16_16816(sc[2 * pr], qa[kk], b00, b01);
                mma_bf16_16816(sc[2 * pr + 1], qa[kk], b10, b11);
            }
        }
        // mask + online softmax (rows r0 and r0+8)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < BN / 8; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = kt * BN + 8 * n + colp + e;
                sc[n][e] = key <= lim0 ? sc[n][e] * p.scale_log2 : -INFINITY;
                sc[n][2 + e] = key <= lim0 + 8 ? sc[n][2 + e] * p.scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, sc[n][e]);
                mx1 = fmaxf(mx1, sc[n][2 + e]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        // Key 0 is visible to every row, so mn0/mn1 are finite from the first tile on.
        const float a0 = pf_exp2(m_run[0] - mn0), a1 = pf_exp2(m_run[1] - mn1);
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int n = 0; n < BN / 8; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                sc[n][e] = pf_exp2(sc[n][e] - mn0);
                sc[n][2 + e] = pf_exp2(sc[n][2 + e] - mn1);
                ps0 += sc[n][e];
                ps1 += sc[n][2 + e];
            }
        l_run[0] = fmaf(l_run[0], a0, ps0);
        l_run[1] = fmaf(l_run[1], a1, ps1);
        m_run[0] = mn0;
        m_run[1] = mn1;
#pragma unroll
        for (int d = 0; d < HD / 8; ++d) {
            o[d][0] *= a0; o[d][1] *= a0; o[d][2] *= a1; o[d][3] *= a1;
        }
#pragma unroll
        for (int k16 = 0; k16 < BN / 16; ++k16) {
            const uint32_t pa[4] = {pack_bf16x2(sc[2 * k16][0], sc[2 * k16][1]), pack_bf16x2(sc[2 * k16][2], sc[2 * k16][3]),
                                    pack_bf16x2(sc[2 * k16 + 1][0], sc[2 * k16 + 1][1]),
                                    pack_bf16x2(sc[2 * k16 + 1][2], sc[2 * k16 + 1][3])};
#pragma unroll
            for (int dd = 0; dd < HD / 16; ++dd) {
                uint32_t v00, v01, v10, v11;
                const int row = 16 * k16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                const int ch = 2 * dd + (lane >> 4);
                ldmatrix_x4_trans(vs + pf_tile_off<HD>(row, ch), v00, v01, v10, v11);
                mma_bf16_16816(o[2 * dd], pa, v00, v01);
                mma_bf16_16816(o[2 * dd + 1], pa, v10, v11);
            }
        }
    }
    cp_async_wait<0>();

    float ls0 = l_run[0], ls1 = l_run[1];
    ls0 += __shfl_xor_sync(0xffffffffu, ls0, 1);
    ls0 += __shfl_xor_sync(0xffffffffu, ls0, 2);
    ls1 += __shfl_xor_sync(0xffffffffu, ls1, 1);
    ls1 += __shfl_xor_sync(0xffffffffu, ls1, 2);
    const float i0 = ls0 > 0.f ? 1.f / ls0 : 0.f, i1 = ls1 > 0.f ? 1.f / ls1 : 0.f;
    const int tok0 = q_start + r0, tok1 = tok0 + 8;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
        const int c = 8 * d + colp;
        if (tok0 < T)
            *reinterpret_cast<uint32_t*>(p.out + (int64_t)(q0 + tok0) * p.out_stride + (int64_t)h * HD + c) =
                pack_bf16x2(o[d][0] * i0, o[d][1] * i0);
        if (tok1 < T)
            *reinterpret_cast<uint32_t*>(p.out + (int64_t)(q0 + tok1) * p.out_stride + (int64_t)h * HD + c) =
                pack_bf16x2(o[d][2] * i1, o[d][3] * i1);
    }
    if (p.overlap_prefill) pdl_wait();            // complete only after the decode kernel this one ran beside
}

template <int HD, int STAGES> static int launch_prefill_cfg(const AttnParams& p, int max_items, cudaStream_t st) {
    constexpr int smem = STAGES * 2 * 64 * HD * 2;
    static SmemOptIn optin;
    if (optin.needs((size_t)smem)) {
        cudaError_t e = cudaFuncSetAttribute(prefill_mma_kernel<HD, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "prefill attention: cannot reserve %d bytes of shared memory: %s",
                                          smem, cudaGetErrorString(e));
        optin.done((size_t)smem);
    }
    dim3 grid((unsigned)max_items, (unsigned)p.n_kv_heads);
    if (p.overlap_prefill) {
        cudaError_t e = launch_pdl(prefill_mma_kernel<HD, STAGES>, grid, dim3((unsigned)(p.group * 32)), (size_t)smem, st, p);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "prefill attention: launch failed: %s", cudaGetErrorString(e));
        return NS_OK;
    }
    prefill_mma_kernel<HD, STAGES><<<grid, p.group * 32, smem, st>>>(p);
    return check_launch("prefill_mma");
}

bool prefill_mma_supported(int n_heads, int n_kv_heads, int head_dim, int block_size) {
    if (block_size != 16 || n_heads % n_kv_heads != 0) return false;
    const int group = n_heads / n_kv_heads;
    return group >= 1 && group <= 8 && (head_dim == 64 || head_dim == 128);
}

int launch_prefill_mma(const AttnParams& p, int head_dim, int max_items, cudaStream_t st) {
    if (max_items <= 0) return NS_OK;
    if (head_dim == 64) return launch_prefill_cfg<64, 3>(p, max_items, st);
    return launch_prefill_cfg<128, 3>(p, max_items, st);
}

}  // namespace ns

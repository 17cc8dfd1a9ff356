// Decode paged attention for sm_100a: HBM-bound GQA over 16-token KV blocks.
//
// Grid  : one persistent CTA per SM (16 warps for head_dim 64, 8 for 128). The flattened list of (decode row, KV block)
//         units is cut into contiguous ranges by the plan kernel (attn_plan.cuh): balanced whole rows / equal pieces of
//         long rows for large steps (optionally two virtual 8-warp CTAs per CTA), and for small steps one thread-block
//         cluster of CTAs per row (cluster mode, see below).
// Warp  : owns one KV head and every (warps-per-head)-th block of the CTA's range. It runs its own
//         cp.async ring (STAGES tiles of 16 tokens, K and V, 128-bit copies, XOR-swizzled rows) with no
//         CTA-wide barrier in the steady state, so up to (STAGES-1) tiles per warp are always in flight.
//         Block ids are fetched 32 at a time, and the next row's Q fragments are loaded into registers as soon
//         as the prefetch cursor reaches that row, so no tile waits on a dependent load.
// Math  : the GROUP (<= 8) query heads sharing the KV head are rows 0..GROUP-1 of an m16n8k16 bf16 MMA tile
//         (rows 8..15 are zero); scores and the running max / sum are fp32, probabilities are rounded to
//         bf16 before P.V, the row max is reduced with warp shuffles (online softmax).
// Split : a row whose blocks span several warps / CTAs is combined in two levels: the warps of one head
//         through shared memory, CTAs through fp32 partials in the workspace, where the LAST CTA to arrive
//         (atomic counter, no waiting) does the final reduction. Counters are left at zero. In cluster mode the CTAs of a
//         row's cluster write their pieces into the first CTA's shared memory (DSMEM) instead, and one cluster barrier
//         later that CTA sums them: no global partials, no atomics.
#include "attn_plan.cuh"
#include "common.cuh"

namespace ns {

bool decode_cluster_enabled();      // c_api.cu: NS_TUNE_DECODE_CLUSTER

__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

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


// Cluster mode, first CTA of the cluster, after the cluster barrier: pieces[rank][kv head][8 rows][HD + 4] hold every
// rank's partial of the cluster's decode row (O[HD], m, l; row 0 also carries the query row and a "delivered" flag). Sum
// them and write the row. A row that one CTA held completely was written by that CTA and delivered nothing.
template <int HD>
__device__ __forceinline__ void cluster_combine(const AttnParams& p, const float* pieces, int cm, int tid, int nthreads) {
    constexpr int RED_ROW = HD + 4, V4 = HD / 4;
    const int NKV = p.n_kv_heads, GROUP = p.group;
    for (int e = tid; e < NKV * GROUP * V4; e += nthreads) {
        const int g = e / (GROUP * V4), rem = e - g * (GROUP * V4);
        const int r = rem / V4, c4 = rem - r * V4;
        float M = -INFINITY;
        int qrow = -1;
        for (int k = 0; k < cm; ++k) {
            const float* head = pieces + (size_t)(k * NKV + g) * 8 * RED_ROW;
            if (head[HD + 3] != 0.f) {
                qrow = __float_as_int(head[HD + 2]);
                M = fmaxf(M, head[r * RED_ROW + HD]);
            }
        }
        if (qrow < 0) continue;
        float Ls = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < cm; ++k) {
            const float* head = pieces + (size_t)(k * NKV + g) * 8 * RED_ROW;
            if (head[HD + 3] == 0.f) continue;
            const float* row = head + r * RED_ROW;
            const float w = row[HD] > -INFINITY ? fast_exp2(row[HD] - M) : 0.f;
            const float4 v = *reinterpret_cast<const float4*>(row + 4 * c4);
            acc.x = fmaf(w, v.x, acc.x);
            acc.y = fmaf(w, v.y, acc.y);
            acc.z = fmaf(w, v.z, acc.z);
            acc.w = fmaf(w, v.w, acc.w);
            Ls = fmaf(w, row[HD + 1], Ls);
        }
        const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
        uint2 packed;
        packed.x = pack_bf16x2(acc.x * inv, acc.y * inv);
        packed.y = pack_bf16x2(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(p.out + (int64_t)qrow * p.out_stride + (int64_t)(g * GROUP + r) * HD + 4 * c4) = packed;
    }
}

// MAX_MODE = 2: the plan may ask every CTA to act as TWO virtual CTAs of NWARPS/2 warps, each with its own range
// (header field `mode`). Small steps (one CTA per row or less) want all 16 warps on one row; large ones want twice as
// many, shorter ranges. Which one is decided on the device, per step, by the plan kernel: the launch never changes.
template <int HD, int NWARPS, int STAGES, int CTAS_PER_SM, int MAX_MODE>
__global__ void __launch_bounds__(NWARPS * 32, CTAS_PER_SM) paged_decode_kernel(const AttnParams p) {
    constexpr int CPR = HD / 8;                       // 16-byte chunks per K/V row
    constexpr int KV_TILE = 16 * HD * 2;              // bytes of one K (or V) tile
    constexpr int STAGE_BYTES = 2 * KV_TILE;
    constexpr int RED_ROW = HD + 4;                   // floats: O[HD], m, l, pad (rows stay 16-byte aligned)
    constexpr int STAGE_PARTS = 16;                   // partials whose (m, l) are staged at once
    extern __shared__ __align__(128) uint8_t smem[];

    // This kernel may be scheduled while the kernel that produces Q and this step's K/V rows (the QKV projection with
    // its RoPE + KV-write epilogue) is still running. Until pdl_wait() below it touches only what earlier steps and
    // the step's plan left behind: the plan records, the block tables and the K/V rows of OLDER tokens.
    if (!p.overlap_prefill) pdl_launch_dependents();          // o_proj may start fetching its weights while attention runs
    if (p.plan_fresh) pdl_wait();                             // the plan is the predecessor's output: nothing is read before
    if (p.timeline && threadIdx.x == 0) p.timeline[blockIdx.x * 4] = global_ns();
    const PlanHeader* hdr = reinterpret_cast<const PlanHeader*>(p.ws + p.L.header);
    const int32_t* __restrict__ cta_start = reinterpret_cast<const int32_t*>(p.ws + p.L.cta_start);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int HALF_WARPS = NWARPS / 2;
    // one 32-byte record holds a (virtual) CTA's range and its first row's description. The record index depends on the
    // plan's mode, so both candidates are fetched together with the mode: still a single round trip.
    const int4* __restrict__ rec_base = reinterpret_cast<const int4*>(p.ws + p.L.cta_rec);
    const int4* rec1 = rec_base + 2 * (int)blockIdx.x;
    const int4* rec2 = rec_base + 2 * (2 * (int)blockIdx.x + (MAX_MODE == 2 ? warp / HALF_WARPS : 0));
    int4 rec_a = rec1[0], rec_b = rec1[1];
    bool split = false;
    if (MAX_MODE == 2) {
        const int4 a2 = rec2[0], b2 = rec2[1];
        split = hdr->mode == 2;
        if (split) {
            rec_a = a2;
            rec_b = b2;
        }
    }
    // Cluster mode (small steps, chosen by the plan): this CTA's range is one piece of ONE decode row, the other pieces
    // belong to the other CTAs of its thread-block cluster, and the pieces meet in the first CTA's shared memory
    // (no global partials, no atomics, no second pass over them). It needs the launch's cluster size to be the plan's.
    uint32_t crank, csize;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
    asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(csize));
    const int cm = (csize > 1 && hdr->cluster == (int)csize) ? (int)csize : 0;
    const int half = split ? warp / HALF_WARPS : 0;           // which virtual CTA of this physical one
    const int vwarps = split ? HALF_WARPS : NWARPS;           // warps of a virtual CTA
    const int lw = warp - half * vwarps;                      // warp index inside it
    const int cta = split ? 2 * (int)blockIdx.x + half : (int)blockIdx.x;
    const int u0 = rec_a.x, u1 = rec_a.y, i_first = rec_a.z;

    __shared__ int4 pend[2 * kMaxKvHeads][2];     // rows a virtual CTA holds only in part: {row, first unit, query row, -}
    __shared__ int2 pend_span[2 * kMaxKvHeads][2];
    __shared__ int pend_n[2 * kMaxKvHeads];
    __shared__ int pend_last[2 * kMaxKvHeads][2];
    if (threadIdx.x < 2 * kMaxKvHeads) pend_n[threadIdx.x] = 0;
    // cluster mode: slot [rank][head][row 0][HD + 3] of the first CTA's staging area says whether that rank delivered a
    // piece; the first CTA clears the flags before anybody can write them (the cluster barrier below orders it)
    float* const xstage = reinterpret_cast<float*>(smem + (size_t)NWARPS * STAGES * STAGE_BYTES);
    if (cm && crank == 0)
        for (int e = threadIdx.x; e < cm * p.n_kv_heads; e += blockDim.x) xstage[(size_t)e * 8 * RED_ROW + HD + 3] = 0.f;
    __syncthreads();                              // the only CTA-wide barrier; everything below is per head group
    if (cm) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    if (u0 >= u1) {
        if (p.overlap_prefill || cm) pdl_wait();  // an exit counts as the trigger: it must not come before Q exists
        if (cm) {                                 // nothing to deliver: keep the cluster's two barriers matched
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            if (crank == 0) cluster_combine<HD>(p, xstage, cm, threadIdx.x, blockDim.x);
        }
        return;
    }

    const int4* __restrict__ dec_info = reinterpret_cast<const int4*>(p.ws + p.L.dec_info);   // {seq, len, table row, q row}
    const int2* __restrict__ dec_span = reinterpret_cast<const int2*>(p.ws + p.L.dec_span);   // {first CTA, CTAs} per row
    const int32_t* __restrict__ indptr = reinterpret_cast<const int32_t*>(p.ws + p.L.dec_indptr);
    int32_t* counters = reinterpret_cast<int32_t*>(p.ws + p.L.counters);
    float* partials = reinterpret_cast<float*>(p.ws + p.L.partials);

    const int NKV = p.n_kv_heads;
    const int g = lw % NKV;                   // KV head of this warp
    const int stripe = lw / NKV;              // which share of the blocks
    const int wph = vwarps / NKV;             // warps per head
    const int hg = half * NKV + g;            // head group inside the physical CTA: named barrier id, staging slot
    const int wbase = half * vwarps;          // first physical warp of this virtual CTA
    const int GROUP = p.group;
    const int gt = stripe * 32 + lane;        // thread index inside the head group
    const int gthreads = wph * 32;
    const int row8 = lane >> 2;               // MMA accumulator row of this lane
    const int colp = (lane & 3) * 2;          // first of its two columns inside an 8-wide n-tile

    uint8_t* my_stages = smem + (size_t)warp * STAGES * STAGE_BYTES;
    constexpr int ML_STRIDE = STAGE_PARTS * 16 + 16;  // floats per head group: (m, l) x 8 rows x parts, rowM[8], rowL[8]
    float* ml_stage = reinterpret_cast<float*>(smem + (size_t)NWARPS * STAGES * STAGE_BYTES);
    __shared__ int red_stage[NWARPS];         // which idle stage of each warp holds its (m, l, O) during a combine
    int my_red = STAGES - 1;
    auto red_of = [&](int w, int stage) -> float* {
        return reinterpret_cast<float*>(smem + ((size_t)w * STAGES + stage) * STAGE_BYTES);   // [8][RED_ROW]
    };

    // ---- prefetch cursor (runs STAGES-1 tiles ahead of the compute cursor) ------------------------------------
    int pf_i = i_first, pf_lo = rec_a.w, pf_hi = rec_b.x;
    int4 pf_info = make_int4(0, rec_b.y, rec_b.z, rec_b.w);
    const int32_t* pf_table = p.block_tables + (int64_t)pf_info.z * p.table_stride;
    int pf_bids = 0, pf_bt = -1000000;        // lane L holds the block id of this warp's tile pf_bt + L
    uint32_t qn[HD / 16][2];                  // Q fragments of the row the prefetch cursor is in
    int qn_row = -1;

    // Q fragments (rows 0..7 = heads of the group; a0 = cols colp..+1, a2 = cols colp+8..+9 of each k-step)
    auto load_q = [&](uint32_t (&dst)[HD / 16][2], int qrow) {
        const __nv_bfloat16* qb = p.q + (int64_t)qrow * p.q_stride + (int64_t)(g * GROUP + row8) * HD + colp;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            dst[kk][0] = row8 < GROUP ? *reinterpret_cast<const uint32_t*>(qb + 16 * kk) : 0u;
            dst[kk][1] = row8 < GROUP ? *reinterpret_cast<const uint32_t*>(qb + 16 * kk + 8) : 0u;
        }
    };

    // per-lane constants of the tile copy: chunk q = it*32 + lane -> row = q / CPR, ch = q % CPR
    const int cp_row0 = lane / CPR, cp_ch = lane % CPR;
    constexpr int ROWS_PER_IT = 32 / CPR;

    // Tiles issued before pdl_wait(): the row of the step's new token (always the last of its block) is left out and
    // fetched afterwards; which tile, which row and where from is remembered here.
    int early_valid[STAGES];
    int64_t early_base[STAGES];
#pragma unroll
    for (int t = 0; t < STAGES; ++t) early_valid[t] = 0;
    int early_q_i = -1, early_q_row = 0;

    auto issue = [&](int t, bool early) {
        const int u = u0 + stripe + wph * t;
        if (u < u1) {
            bool moved = false;
            while (u >= pf_hi) {
                ++pf_i;
                pf_lo = pf_hi;
                pf_hi = indptr[pf_i + 1];
                moved = true;
            }
            if (moved) {
                pf_info = dec_info[pf_i];
                pf_table = p.block_tables + (int64_t)pf_info.z * p.table_stride;
            }
            if (moved || t - pf_bt >= 32) {   // one coalesced load fetches the next 32 block ids of this row
                pf_bt = t;
                const int jj = (u - pf_lo) + wph * lane;
                pf_bids = (pf_lo + jj < pf_hi) ? pf_table[jj] : 0;
            }
            if (qn_row != pf_i) {             // first tile of a row: start loading its Q now
                if (early) {
                    early_q_i = pf_i;         // Q is not there yet: loaded right after pdl_wait()
                    early_q_row = pf_info.w;
                } else {
                    qn_row = pf_i;
                    load_q(qn, pf_info.w);
                }
            }
            const int j = u - pf_lo;
            const int blk = __shfl_sync(0xffffffffu, pf_bids, t - pf_bt);
            int valid = min(16, pf_info.y - 16 * j);
            const int64_t base = (int64_t)blk * p.blk_stride + (int64_t)g * p.head_stride + cp_ch * 8;
            int skip_row = -1;
            if (early && pf_info.y - 16 * j <= 16) {      // the row's last block: its last token is this step's
                skip_row = valid - 1;
#pragma unroll
                for (int e = 0; e < STAGES; ++e)
                    if (e == t) {
                        early_valid[e] = valid;
                        early_base[e] = (int64_t)blk * p.blk_stride + (int64_t)g * p.head_stride;
                    }
            }
            const uint32_t ks = smem_u32(my_stages + (size_t)(t % STAGES) * STAGE_BYTES), vs = ks + KV_TILE;
#pragma unroll
            for (int it = 0; it < 16 / ROWS_PER_IT; ++it) {
                const int row = it * ROWS_PER_IT + cp_row0;
                const int nbytes = row < valid ? 16 : 0;
                const int64_t goff = base + (int64_t)row * p.pos_stride;
                const uint32_t so = tile_off<HD>(row, cp_ch);
                if (row != skip_row) {
                    cp_async16(ks + so, p.k_pool + goff, nbytes);
                    cp_async16(vs + so, p.v_pool + goff, nbytes);
                }
            }
        }
        cp_async_commit();
    };

    float* xremote = xstage;                  // cluster mode: the first CTA's staging area, through distributed shared memory
    if (cm) {
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(smem_u32(xstage)));
        uint64_t generic;
        asm volatile("cvta.shared::cluster.u64 %0, %1;" : "=l"(generic) : "l"((uint64_t)remote));
        xremote = reinterpret_cast<float*>(generic);
    }

    // ---- running state of this warp for the current decode row ---------------------------------------------------
    float m_run = -INFINITY, l_run = 0.f;     // row = lane/4; l is this lane's share of the row sum
    float o[HD / 8][2];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = 0.f;
    uint32_t qa[HD / 16][2];                  // A fragments of the row being computed
    int qa_row = -1;
    int cc_i = i_first, cc_lo = pf_lo, cc_hi = pf_hi;
    int cc_len = pf_info.y, cc_qrow = pf_info.w;
    int2 cc_span = dec_span[i_first];         // only needed at the first flush: off the critical path

    // Combine the warps of this head for the current decode row [cc_lo, cc_hi), then write the final output or a
    // partial. Every value it needs is already in registers: no dependent global load on this path.
    auto flush = [&]() {
        float* mine = red_of(warp, my_red);
        if (lane == 0) red_stage[warp] = my_red;
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
        named_barrier(hg, gthreads);

        const int i = cc_i, lo = cc_lo, hi = cc_hi;
        const bool complete = lo >= u0 && hi <= u1;
        const int64_t qrow = cc_qrow;
        const int slot = (i == i_first) ? 0 : 1;
        float* part = partials + ((size_t)(cta * 2 + slot) * p.n_heads + (size_t)g * GROUP) * RED_ROW;
        // four output columns per thread: 16-byte reads of the warps' scratch, 16-byte (partial) or 8-byte (final) stores
        for (int e = gt; e < GROUP * (HD / 4); e += gthreads) {
            const int r = e / (HD / 4), c = (e - r * (HD / 4)) * 4;
            float M = -INFINITY;
            for (int w = 0; w < wph; ++w) M = fmaxf(M, red_of(wbase + g + NKV * w, red_stage[wbase + g + NKV * w])[r * RED_ROW + HD]);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float Ls = 0.f;
            for (int w = 0; w < wph; ++w) {
                const float* rw = red_of(wbase + g + NKV * w, red_stage[wbase + g + NKV * w]) + r * RED_ROW;
                const float sc = fast_exp2(rw[HD] - M);
                const float4 v = *reinterpret_cast<const float4*>(rw + c);
                acc.x = fmaf(sc, v.x, acc.x);
                acc.y = fmaf(sc, v.y, acc.y);
                acc.z = fmaf(sc, v.z, acc.z);
                acc.w = fmaf(sc, v.w, acc.w);
                Ls = fmaf(sc, rw[HD + 1], Ls);
            }
            if (complete) {
                const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
                uint2 packed;
                packed.x = pack_bf16x2(acc.x * inv, acc.y * inv);
                packed.y = pack_bf16x2(acc.z * inv, acc.w * inv);
                *reinterpret_cast<uint2*>(p.out + qrow * p.out_stride + (int64_t)(g * GROUP + r) * HD + c) = packed;
            } else if (cm) {
                // this CTA's piece of the row goes straight into the first CTA's shared memory
                float* dst = xremote + ((size_t)(crank * NKV + g) * 8 + r) * RED_ROW;
                *reinterpret_cast<float4*>(dst + c) = acc;
                if (c == 0) {
                    *reinterpret_cast<float2*>(dst + HD) = make_float2(M, Ls);
                    if (r == 0) *reinterpret_cast<float2*>(dst + HD + 2) = make_float2(__int_as_float((int)qrow), 1.f);
                }
            } else {
                *reinterpret_cast<float4*>(part + r * RED_ROW + c) = acc;
                if (c == 0) *reinterpret_cast<float2*>(part + r * RED_ROW + HD) = make_float2(M, Ls);
            }
        }
        if (!complete && !cm && gt == 0) {    // cross-CTA work for this row is deferred to the end of the CTA
            const int k = pend_n[hg]++;
            pend[hg][k] = make_int4(i, lo, (int)qrow, 0);
            pend_span[hg][k] = cc_span;
        }
        named_barrier(hg, gthreads);       // every warp's scratch has been consumed
        m_run = -INFINITY;
        l_run = 0.f;
#pragma unroll
        for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = 0.f;
    };

    auto next_row = [&]() {
        ++cc_i;
        cc_lo = cc_hi;
        cc_hi = indptr[cc_i + 1];
        const int4 info = dec_info[cc_i];
        cc_len = info.y;
        cc_qrow = info.w;
        cc_span = dec_span[cc_i];
    };

    // ---- pipeline ---------------------------------------------------------------------------------------------------
    const int my_tiles = (u1 - u0 - stripe + wph - 1) / wph;      // may be <= 0
#pragma unroll
    for (int t = 0; t < STAGES - 1; ++t) issue(t, true);
    // Nothing is computed before the wait, so the ring's last stage can carry a tile as well: a warp then has STAGES
    // tiles in flight while the QKV kernel runs (rows up to 16 x STAGES x warps-per-head tokens arrive completely before
    // Q exists). Only when this warp's first tile lies in the CTA's first row: otherwise iteration 0 starts with a
    // flush(), whose scratch is that stage.
    const bool full_ring = u0 + stripe < rec_b.x;
    if (full_ring) issue(STAGES - 1, true);
    pdl_wait();                               // Q and the new token's K/V row exist from here on
    if (p.overlap_prefill) pdl_launch_dependents();           // the prefill kernel may run beside this one from here on
    if (cm) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // the first CTA runs and has cleared its flags
    if (early_q_i >= 0) {
        qn_row = early_q_i;
        load_q(qn, early_q_row);
    }
    {
        bool patched = false;
#pragma unroll
        for (int t = 0; t < STAGES; ++t) {
            if (early_valid[t] > 0) {
                patched = true;
                const int row = early_valid[t] - 1;
                if (lane < 2 * CPR) {
                    const int ch = lane % CPR;
                    const bool is_v = lane >= CPR;
                    const uint32_t dst = smem_u32(my_stages + (size_t)(t % STAGES) * STAGE_BYTES) + (is_v ? KV_TILE : 0) +
                                         tile_off<HD>(row, ch);
                    const int64_t goff = early_base[t] + ch * 8 + (int64_t)row * p.pos_stride;
                    cp_async16(dst, (is_v ? p.v_pool : p.k_pool) + goff, 16);
                }
            }
        }
        if (patched) {                        // rare past a row's first step range: one extra group, drained here
            cp_async_commit();
            cp_async_wait<0>();
            __syncwarp();
        }
    }

    for (int t = 0; t < my_tiles; ++t) {
        cp_async_wait<STAGES - 2>();          // tile t has landed (one commit group per tile, empty or not)
        __syncwarp();
        if (p.timeline && threadIdx.x == 0 && t == 0) p.timeline[blockIdx.x * 4 + 1] = global_ns();
        const int u = u0 + stripe + wph * t;
        if (u >= cc_hi) {
            // the stage consumed in iteration t-1 is idle: it is this warp's scratch for the combine
            my_red = (t + STAGES - 1) % STAGES;
            do {
                flush();
                next_row();
            } while (u >= cc_hi);
        }
        if (qa_row != cc_i) {                 // first tile of this row for this warp
            qa_row = cc_i;
            if (qn_row == cc_i) {
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) { qa[kk][0] = qn[kk][0]; qa[kk][1] = qn[kk][1]; }
            } else {
                load_q(qa, cc_qrow);          // the prefetch cursor is already rows ahead (very short rows)
            }
        }
        if (t == 0 && full_ring)
            cp_async_commit();                // that tile is already on its way: keep one commit group per iteration
        else
            issue(t + STAGES - 1, false);     // refills the stage computed in iteration t-1
        const uint32_t ks = smem_u32(my_stages + (size_t)(t % STAGES) * STAGE_BYTES), vs = ks + KV_TILE;
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
    __syncwarp();
    if (p.timeline && threadIdx.x == 0) p.timeline[blockIdx.x * 4 + 2] = global_ns();
    // Every warp of a head walks every decode row of the CTA's range, with or without tiles of its own, so the
    // group barriers inside flush() always match. All stages are idle now: stage 0 is the scratch.
    my_red = 0;
    while (cc_hi < u1) {
        flush();
        next_row();
    }
    flush();

    if (cm) {
        // every CTA of the cluster has delivered (or has nothing): the first one sums the pieces and writes the row
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (crank == 0) cluster_combine<HD>(p, xstage, cm, threadIdx.x, blockDim.x);
        if (p.timeline && threadIdx.x == 0) p.timeline[blockIdx.x * 4 + 3] = global_ns();
        return;
    }

    // ---- cross-CTA combine of the rows this CTA saw only a part of (at most its first and its last row) ------------
    // The partials were stored by every thread of the group before the barrier that ends flush(); the leader's fence
    // publishes them (fences are cumulative over what the barrier ordered before it). Whoever completes a row's
    // arrival count combines it. Nobody waits.
    const int n_pend = pend_n[hg];
    if (n_pend > 0) {
        if (gt == 0) {
            // one acquire-release atomic per row instead of fence, atomic, fence: it releases the partials the barrier in
            // flush() ordered before it and acquires those of the CTAs that arrived earlier
            for (int k = 0; k < n_pend; ++k) {
                int prev;
                asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;"
                             : "=r"(prev)
                             : "l"(&counters[pend[hg][k].x * kMaxKvHeads + g])
                             : "memory");
                pend_last[hg][k] = prev == pend_span[hg][k].y - 1;
            }
        }
        named_barrier(hg, gthreads);
        for (int k = 0; k < n_pend; ++k) {
            if (!pend_last[hg][k]) continue;
            const int i = pend[hg][k].x, lo = pend[hg][k].y;
            const int64_t qrow = pend[hg][k].z;
            const int c_first = pend_span[hg][k].x, n_parts = pend_span[hg][k].y, c_last = c_first + n_parts - 1;
            float* st = ml_stage + (size_t)hg * ML_STRIDE;       // [STAGE_PARTS][8][2] = (m -> weight, l)
            float* rowM = st + STAGE_PARTS * 16;                // [8]
            float* rowL = rowM + 8;                             // [8]
            const int first_cut = __ldcg(&cta_start[c_first]);
            // CTA cc holds this row in slot 0 unless the row begins inside cc's range (only possible for c_first)
            auto part_row = [&](int cc, int r) -> const float* {
                const int sl = (cc == c_first && lo != first_cut) ? 1 : 0;
                return partials + ((size_t)(cc * 2 + sl) * p.n_heads + (size_t)g * GROUP + r) * RED_ROW;
            };
            auto stage_ml = [&](int base, int cnt) {
                for (int idx = gt; idx < cnt * 8; idx += gthreads) {
                    const int pt = idx >> 3, r = idx & 7;
                    float mv = -INFINITY, lv = 0.f;
                    if (r < GROUP) {
                        const float* pr = part_row(base + pt, r);
                        mv = __ldcg(pr + HD);
                        lv = __ldcg(pr + HD + 1);
                    }
                    st[idx * 2] = mv;
                    st[idx * 2 + 1] = lv;
                }
                named_barrier(hg, gthreads);
            };
            if (n_parts <= STAGE_PARTS) {
                // Few parts (the usual case): every thread fetches, for ITS row and four output columns, (m, l) of all
                // parts and the first eight partial vectors at once - one round trip, no staging, no barrier.
                constexpr int V4 = HD / 4;
                for (int e = gt; e < GROUP * V4; e += gthreads) {
                    const int r = e / V4, c4 = e - r * V4;
                    float2 ml[STAGE_PARTS];
                    float4 v[8];
#pragma unroll
                    for (int pt = 0; pt < STAGE_PARTS; ++pt)
                        ml[pt] = pt < n_parts ? __ldcg(reinterpret_cast<const float2*>(part_row(c_first + pt, r) + HD))
                                              : make_float2(-INFINITY, 0.f);
#pragma unroll
                    for (int pt = 0; pt < 8; ++pt)
                        v[pt] = pt < n_parts ? __ldcg(reinterpret_cast<const float4*>(part_row(c_first + pt, r)) + c4)
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
                    float M = -INFINITY;
#pragma unroll
                    for (int pt = 0; pt < STAGE_PARTS; ++pt) M = fmaxf(M, ml[pt].x);
                    float Ls = 0.f;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int pt = 0; pt < STAGE_PARTS; ++pt) {
                        const float wgt = ml[pt].x > -INFINITY ? fast_exp2(ml[pt].x - M) : 0.f;
                        ml[pt].x = wgt;
                        Ls = fmaf(wgt, ml[pt].y, Ls);
                    }
#pragma unroll
                    for (int pt = 0; pt < 8; ++pt) {
                        acc.x = fmaf(ml[pt].x, v[pt].x, acc.x);
                        acc.y = fmaf(ml[pt].x, v[pt].y, acc.y);
                        acc.z = fmaf(ml[pt].x, v[pt].z, acc.z);
                        acc.w = fmaf(ml[pt].x, v[pt].w, acc.w);
                    }
                    for (int pt = 8; pt < n_parts; ++pt) {             // parts nine and up: a second round trip
                        const float4 w4 = __ldcg(reinterpret_cast<const float4*>(part_row(c_first + pt, r)) + c4);
                        acc.x = fmaf(ml[pt].x, w4.x, acc.x);
                        acc.y = fmaf(ml[pt].x, w4.y, acc.y);
                        acc.z = fmaf(ml[pt].x, w4.z, acc.z);
                        acc.w = fmaf(ml[pt].x, w4.w, acc.w);
                    }
                    const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
                    uint2 packed;
                    packed.x = pack_bf16x2(acc.x * inv, acc.y * inv);
                    packed.y = pack_bf16x2(acc.z * inv, acc.w * inv);
                    *reinterpret_cast<uint2*>(p.out + qrow * p.out_stride + (int64_t)(g * GROUP + r) * HD + 4 * c4) = packed;
                }
                if (gt == 0) counters[i * kMaxKvHeads + g] = 0;
                continue;
            }
            const bool single = false;                         // more parts than one staging holds: staged in batches
            float myM = -INFINITY;                             // threads 0..7 of the group: row maxima
            for (int base = c_first; base <= c_last; base += STAGE_PARTS) {
                const int cnt = min(STAGE_PARTS, c_last - base + 1);
                stage_ml(base, cnt);
                if (gt < 8)
                    for (int pt = 0; pt < cnt; ++pt) myM = fmaxf(myM, st[(pt * 8 + gt) * 2]);
                if (!single) named_barrier(hg, gthreads);
            }
            if (gt < 8) rowM[gt] = myM;
            named_barrier(hg, gthreads);
            float myL = 0.f;
            auto to_weights = [&](int cnt, bool add_l) {       // m -> exp2(m - rowM) in place
                for (int idx = gt; idx < cnt * 8; idx += gthreads) {
                    const int r = idx & 7;
                    const float mv = st[idx * 2];
                    st[idx * 2] = (r < GROUP && mv > -INFINITY) ? fast_exp2(mv - rowM[r]) : 0.f;
                }
                named_barrier(hg, gthreads);
                if (add_l && gt < 8)
                    for (int pt = 0; pt < cnt; ++pt) myL = fmaf(st[(pt * 8 + gt) * 2], st[(pt * 8 + gt) * 2 + 1], myL);
            };
            if (single) to_weights(n_parts, true);
            // each thread owns float4 columns of the [GROUP x HD] output; the loads over the partials are independent
            constexpr int V4_PER_ROW = HD / 4;
            for (int kg = 0; kg * gthreads < GROUP * V4_PER_ROW; ++kg) {
                const int e = gt + gthreads * kg;
                const bool mine = e < GROUP * V4_PER_ROW;
                const int r = mine ? e / V4_PER_ROW : 0, c4 = mine ? e - r * V4_PER_ROW : 0;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int base = c_first; base <= c_last; base += STAGE_PARTS) {
                    const int cnt = min(STAGE_PARTS, c_last - base + 1);
                    if (!single) {
                        stage_ml(base, cnt);
                        to_weights(cnt, kg == 0);
                    }
                    if (mine) {
#pragma unroll 8
                        for (int pt = 0; pt < cnt; ++pt) {
                            const float wgt = st[(pt * 8 + r) * 2];
                            const float4 v = __ldcg(reinterpret_cast<const float4*>(part_row(base + pt, r)) + c4);
                            acc.x = fmaf(wgt, v.x, acc.x);
                            acc.y = fmaf(wgt, v.y, acc.y);
                            acc.z = fmaf(wgt, v.z, acc.z);
                            acc.w = fmaf(wgt, v.w, acc.w);
                        }
                    }
                    if (!single) named_barrier(hg, gthreads);
                }
                if (kg == 0) {
                    if (gt < 8) rowL[gt] = myL;
                    named_barrier(hg, gthreads);
                }
                if (mine) {
                    const float Ls = rowL[r];
                    const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
                    uint2 packed;
                    packed.x = pack_bf16x2(acc.x * inv, acc.y * inv);
                    packed.y = pack_bf16x2(acc.z * inv, acc.w * inv);
                    *reinterpret_cast<uint2*>(p.out + qrow * p.out_stride + (int64_t)(g * GROUP + r) * HD + 4 * c4) = packed;
                }
            }
            if (gt == 0) counters[i * kMaxKvHeads + g] = 0;
            named_barrier(hg, gthreads);               // the staging area is reused by the next pending row
        }
    }
    if (p.timeline && threadIdx.x == 0) p.timeline[blockIdx.x * 4 + 3] = global_ns();
}

template <int HD, int NWARPS, int STAGES, int CTAS_PER_SM, int MAX_MODE>
static int launch_decode_cfg(const AttnParams& p, int sms, cudaStream_t st) {
    constexpr int smem = NWARPS * STAGES * (2 * 16 * HD * 2) + 2 * kMaxKvHeads * (16 * 16 + 16) * 4;
    static_assert(8 * (HD + 4) * 4 <= 2 * 16 * HD * 2, "the combine scratch must fit in one stage");
    static SmemOptIn optin;
    if (optin.needs((size_t)smem)) {
        cudaError_t e = cudaFuncSetAttribute(paged_decode_kernel<HD, NWARPS, STAGES, CTAS_PER_SM, MAX_MODE>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "decode attention: cannot reserve %d bytes of shared memory: %s",
                                          smem, cudaGetErrorString(e));
        optin.done((size_t)smem);
    }
    // cluster size for small steps: what the plan proposed for this many sequences, as long as the pieces of a row
    // (cluster x kv heads x 8 rows x (HD + 4) floats) fit the staging area they meet in
    const int grid = sms * CTAS_PER_SM;
    int cl = decode_cluster_enabled() ? plan_cluster(p.n_seqs, grid) : 1;
    constexpr int stage_bytes = 2 * kMaxKvHeads * (16 * 16 + 16) * 4;
    while (cl > 1 && cl * p.n_kv_heads * 8 * (HD + 4) * 4 > stage_bytes) cl >>= 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(NWARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)cl;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, paged_decode_kernel<HD, NWARPS, STAGES, CTAS_PER_SM, MAX_MODE>, p);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "decode attention: launch failed: %s", cudaGetErrorString(e));
    return NS_OK;
}

bool decode_fast_supported(int n_heads, int n_kv_heads, int head_dim, int block_size) {
    if (block_size != 16 || n_heads % n_kv_heads != 0) return false;
    const int group = n_heads / n_kv_heads;
    if (group > 8) return false;
    if (head_dim != 64 && head_dim != 128) return false;
    return n_kv_heads == 1 || n_kv_heads == 2 || n_kv_heads == 4 || n_kv_heads == 8;
}

// Number of persistent decode CTAs for this head_dim on a device with `sms` SMs (the plan must be built for it).
// Physical persistent decode CTAs for this head_dim on a device with `sms` SMs, and how many virtual CTAs each may
// be split into (the plan must be built with the same two numbers).
int decode_grid(int head_dim, int sms) { (void)head_dim; return sms; }
int decode_max_mode(int head_dim) { return head_dim == 64 ? 2 : 1; }

int launch_paged_decode(const AttnParams& p, int head_dim, int sms, cudaStream_t st) {
    if (head_dim == 64) return launch_decode_cfg<64, 16, 3, 1, 2>(p, sms, st);
    return launch_decode_cfg<128, 8, 3, 1, 1>(p, sms, st);
}

}  // namespace ns

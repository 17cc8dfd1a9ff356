// Prefill-chunk paged attention on the 5th-generation tensor cores (tcgen05) with accumulators in tensor memory.
//
// Work item = (sequence, 16 query tokens, KV head): the 16 tokens x (up to 8) query heads of the GQA group form the
// 128 rows of one UMMA tile (row r = token r/8, head r%8), so Q.K^T and P.V are dense 128-row contractions even
// though each sequence contributes few tokens per head.
//   S[128 x 64]  = Q[128 x 64] . K_tile[64 keys x 64]^T     tcgen05.mma kind::f16, A and B K-major, SWIZZLE_128B
//   PV[128 x 64] = P[128 x 64 keys] . V_tile[64 keys x 64]  A K-major (P written to shared memory as bf16),
//                                                            B MN-major (V rows are the pool's rows, untransposed)
// Both accumulators live in TMEM (128 columns per CTA). After each MMA batch a tcgen05.commit arrives on an mbarrier;
// every thread then reads ITS OWN row with tcgen05.ld (lane = row), so the online softmax needs no shuffles. The
// running output is kept in registers and rescaled there, PV is accumulated fresh per tile.
// K/V tiles (4 pool blocks of 16 tokens) are staged with 128-bit cp.async into the XOR-swizzled layout the
// SWIZZLE_128B descriptors expect (16-byte chunk index ^ row%8, 1024-byte aligned tiles), double buffered.
// Every mbarrier wait is bounded: on expiry the CTA records an error, skips its stores, frees its TMEM and returns.
#include "attn_plan.cuh"
#include "common.cuh"

namespace ns {

namespace tc {

constexpr int kRows = 128;          // UMMA M
constexpr int kKeys = 64;           // keys per tile (UMMA N of S, K extent of P.V)
constexpr int kHD = 64;             // head_dim handled here
constexpr int kTmemCols = 128;      // S: columns 0..63, PV: columns 64..127
constexpr int kStages = 4;          // K/V tiles in shared memory: copies run kStages-1 tiles ahead of the tile in use
constexpr uint32_t kWaitLimit = 1u << 22;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 64-bit shared-memory matrix descriptor, SWIZZLE_128B, version 1 (sm_100): start address, leading-dimension byte
// offset and stride byte offset are stored without their 4 low bits.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16: fp32 accumulate, bf16 A and B, M = 128, N = 64.
__host__ __device__ constexpr uint32_t instr_desc(bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(kKeys >> 3) << 17) |
           ((uint32_t)(kRows >> 4) << 24);
}

__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_commit(uint32_t mbar_saddr) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar_saddr) : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint32_t mbar_saddr, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(done)
            : "r"(mbar_saddr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

}  // namespace tc

__global__ void __launch_bounds__(tc::kRows, 2) prefill_tc_kernel(const AttnParams p) {
    using namespace tc;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t mbar;
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;

    const PlanHeader* hdr = reinterpret_cast<const PlanHeader*>(p.ws + p.L.header);
    if ((int)blockIdx.x >= hdr->n_prefill_items) {
        if (p.overlap_prefill) pdl_wait();        // the grid must not complete before the decode kernel it overlaps
        return;
    }
    const int2 item = reinterpret_cast<const int2*>(p.ws + p.L.prefill_items)[blockIdx.x];
    const int s = item.x, q_start = item.y, g = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int q0 = p.cu_seqlens[s];
    const int T = p.cu_seqlens[s + 1] - q0;
    const int len = p.seq_lens[s];
    const int ctx = len - T;
    const int32_t* table = p.block_tables + (int64_t)(p.table_rows ? p.table_rows[s] : s) * p.table_stride;
    const int kv_end = min(len, ctx + q_start + kPrefillTileTokens);
    const int n_tiles = (kv_end + kKeys - 1) / kKeys;

    // shared memory: 1024-byte aligned tiles (the swizzle pattern repeats every 8 rows x 128 bytes)
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = base, sK = sQ + kRows * 128, sV = sK + kStages * kKeys * 128, sP = sV + kStages * kKeys * 128;
    const uint32_t mbar_s = smem_u32(&mbar);

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar_s) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        failed = 0;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    const uint32_t t_lane = tmem + ((uint32_t)(32 * warp) << 16);     // this warp's 32 lanes; lane = row

    // row of this thread
    const int tok = q_start + (tid >> 3), hh = tid & 7;
    const bool row_ok = tok < T && hh < p.group;
    const int h = g * p.group + hh;

    // Q tile: one 128-byte row per thread
    {
        const __nv_bfloat16* src = p.q + (int64_t)(q0 + (row_ok ? tok : 0)) * p.q_stride + (int64_t)(row_ok ? h : 0) * kHD;
#pragma unroll
        for (int c = 0; c < 8; ++c)
            cp_async16(sQ + tid * 128 + ((c ^ (tid & 7)) << 4), src + c * 8, row_ok ? 16 : 0);
    }
    // Block ids of a tile: its 64 keys are 4 pool blocks, the same 4 for every thread (row = it*16 + tid/8). They are
    // fetched ONE TILE AHEAD of the copies that need them, so no copy waits on a dependent table load (measured: ~500 of
    // a tile's ~3600 cycles before this).
    int blk_next[kKeys / 16];
    auto fetch_ids = [&](int kt) {
#pragma unroll
        for (int it = 0; it < kKeys / 16; ++it) {
            const int key0 = kt * kKeys + it * 16;
            blk_next[it] = (kt < n_tiles && key0 < len) ? table[key0 >> 4] : 0;
        }
    };
    auto load_kv = [&](int kt) {                    // uses blk_next (the ids of tile kt), then fetches those of tile kt + 1
        if (kt < n_tiles) {
            const uint32_t ks = sK + (kt % kStages) * kKeys * 128, vs = sV + (kt % kStages) * kKeys * 128;
#pragma unroll
            for (int it = 0; it < (kKeys * 8) / kRows; ++it) {
                const int qd = it * kRows + tid;
                const int row = qd >> 3, c = qd & 7;               // row >> 4 == it
                const int key = kt * kKeys + row;
                const bool ok = key < len;
                const int64_t goff = (int64_t)blk_next[it] * p.blk_stride + (int64_t)(key & 15) * p.pos_stride +
                                     (int64_t)g * p.head_stride + c * 8;
                const uint32_t off = row * 128 + ((c ^ (row & 7)) << 4);
                cp_async16(ks + off, p.k_pool + goff, ok ? 16 : 0);
                cp_async16(vs + off, p.v_pool + goff, ok ? 16 : 0);
            }
        }
        cp_async_commit();
        fetch_ids(kt + 1);
    };
    static_assert((kKeys * 8) / kRows == kKeys / 16, "one pool block per copy iteration");
    fetch_ids(0);
    load_kv(0);                       // group 0 = Q + tile 0
#pragma unroll
    for (int t = 1; t < kStages - 1; ++t) load_kv(t);

    constexpr uint32_t idesc_s = instr_desc(false), idesc_pv = instr_desc(true);
    float o[kHD];
#pragma unroll
    for (int d = 0; d < kHD; ++d) o[d] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    uint32_t phase = 0;
    const int limit = ctx + tok;      // last key this row may see
    bool ok = true;

    for (int kt = 0; kt < n_tiles && ok; ++kt) {
        load_kv(kt + kStages - 1);                                     // into the buffer tile kt-1 has left
        cp_async_wait<kStages - 1>();                                  // tile kt (and Q) landed for this thread
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        const uint32_t ks = sK + (kt % kStages) * kKeys * 128, vs = sV + (kt % kStages) * kKeys * 128;
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kk = 0; kk < kHD / 16; ++kk)                      // K extent 16 per instruction = 32 bytes
                mma_f16(tmem, smem_desc(sQ + kk * 32, 16, 1024), smem_desc(ks + kk * 32, 16, 1024), idesc_s, kk > 0);
            mma_commit(mbar_s);
        }
        if (!mbar_wait(mbar_s, phase)) { ok = false; }
        phase ^= 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        ok = __syncthreads_and(ok);
        if (!ok) break;

        // ---- online softmax on this thread's row ---------------------------------------------------------------
        float sc[kKeys];
        {
            float lo[32], hi[32];
            tmem_ld32(t_lane, lo);
            tmem_ld32(t_lane + 32, hi);
#pragma unroll
            for (int i = 0; i < 32; ++i) { sc[i] = lo[i]; sc[32 + i] = hi[i]; }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < kKeys; ++c) {
            const int key = kt * kKeys + c;
            sc[c] = key <= limit ? sc[c] * p.scale_log2 : -INFINITY;
            mx = fmaxf(mx, sc[c]);
        }
        const float m_new = fmaxf(m_run, mx);                          // key 0 is visible to every row: finite
        const float alpha = ex2(m_run - m_new);
        float psum = 0.f;
#pragma unroll
        for (int c = 0; c < kKeys; ++c) {
            sc[c] = ex2(sc[c] - m_new);
            psum += sc[c];
        }
        l_run = fmaf(l_run, alpha, psum);
        m_run = m_new;
#pragma unroll
        for (int d = 0; d < kHD; ++d) o[d] *= alpha;
        // P row as bf16 into shared memory (K-major, swizzled like the other operands)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            uint4 v;
            v.x = pack_bf16x2(sc[8 * c + 0], sc[8 * c + 1]);
            v.y = pack_bf16x2(sc[8 * c + 2], sc[8 * c + 3]);
            v.z = pack_bf16x2(sc[8 * c + 4], sc[8 * c + 5]);
            v.w = pack_bf16x2(sc[8 * c + 6], sc[8 * c + 7]);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sP + tid * 128 + ((c ^ (tid & 7)) << 4)), "r"(v.x),
                         "r"(v.y), "r"(v.z), "r"(v.w)
                         : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kk = 0; kk < kKeys / 16; ++kk)                    // 16 keys per instruction: 32 bytes of P, 16 rows of V
                mma_f16(tmem + 64, smem_desc(sP + kk * 32, 16, 1024), smem_desc(vs + kk * 2048, 1024, 1024), idesc_pv, kk > 0);
            mma_commit(mbar_s);
        }
        if (!mbar_wait(mbar_s, phase)) { ok = false; }
        phase ^= 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        ok = __syncthreads_and(ok);
        if (!ok) break;
        {
            float lo[32], hi[32];
            tmem_ld32(t_lane + 64, lo);
            tmem_ld32(t_lane + 96, hi);
#pragma unroll
            for (int i = 0; i < 32; ++i) { o[i] += lo[i]; o[32 + i] += hi[i]; }
        }
    }
    cp_async_wait<0>();

    if (ok && row_ok) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* dst = p.out + (int64_t)(q0 + tok) * p.out_stride + (int64_t)h * kHD;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            uint4 v;
            v.x = pack_bf16x2(o[8 * c + 0] * inv, o[8 * c + 1] * inv);
            v.y = pack_bf16x2(o[8 * c + 2] * inv, o[8 * c + 3] * inv);
            v.z = pack_bf16x2(o[8 * c + 4] * inv, o[8 * c + 5] * inv);
            v.w = pack_bf16x2(o[8 * c + 6] * inv, o[8 * c + 7] * inv);
            *reinterpret_cast<uint4*>(dst + c * 8) = v;
        }
    }
    if (!ok && tid == 0)        // a wait expired: count it where the host can read it (ns_collect_status)
        atomicAdd(&reinterpret_cast<PlanHeader*>(p.ws + p.L.header)->errors, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    if (p.overlap_prefill) pdl_wait();            // complete only after the decode kernel this one ran beside
}

bool prefill_tc_supported(int n_heads, int n_kv_heads, int head_dim, int block_size) {
    if (block_size != 16 || n_heads % n_kv_heads != 0) return false;
    const int group = n_heads / n_kv_heads;
    return group >= 1 && group <= 8 && head_dim == tc::kHD;
}

int launch_prefill_tc(const AttnParams& p, int max_items, cudaStream_t st) {
    if (max_items <= 0) return NS_OK;
    constexpr int smem = (tc::kRows + 2 * tc::kStages * tc::kKeys + tc::kRows) * 128 + 1024;
    static SmemOptIn optin;
    if (optin.needs((size_t)smem)) {
        cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "prefill attention (tcgen05): cannot reserve %d bytes of shared memory: %s",
                                          smem, cudaGetErrorString(e));
        optin.done((size_t)smem);
    }
    dim3 grid((unsigned)max_items, (unsigned)p.n_kv_heads);
    if (p.overlap_prefill) {
        cudaError_t e = launch_pdl(prefill_tc_kernel, grid, dim3(tc::kRows), (size_t)smem, st, p);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "prefill attention (tcgen05): launch failed: %s", cudaGetErrorString(e));
        return NS_OK;
    }
    prefill_tc_kernel<<<grid, tc::kRows, smem, st>>>(p);
    return check_launch("prefill_tc");
}

}  // namespace ns

// Prefill-chunk paged attention on the 5th-generation tensor cores (tcgen05) with accumulators in tensor memory.
//
// Work item = (sequence, 16 query tokens, KV head): the 16 tokens x (up to 8) query heads of the GQA group form the
// 128 rows of one UMMA tile (row r = token r/8, head r%8), so Q.K^T and P.V are dense 128-row contractions even
// though each sequence contributes few tokens per head. head_dim HD = 64 or 128.
//   S[128 x 64]  = Q[128 x HD] . K_tile[64 keys x HD]^T     tcgen05.mma kind::f16, A and B K-major, SWIZZLE_128B
//   O[128 x HD] += P[128 x 64 keys] . V_tile[64 keys x HD]  A K-major (P written to shared memory as bf16),
//                                                            B MN-major (V rows are the pool's rows, untransposed)
// Three roles (192 threads):
//   warps 0-3  one softmax thread per row (lane = row of tensor memory): S(j) -> P(j)
//   warp 4     lane 0 issues every tcgen05.mma with PRECOMPUTED descriptors (a tcgen05.mma of this size occupies the
//              tensor pipe for ~50 cycles; building two 64-bit descriptors per instruction in a lone thread cost three
//              times that)
//   warp 5     lane 0 fetches the K/V tiles: one tiled TMA load (cp.async.bulk.tensor, no multicast) per pool block of 16
//              tokens and 128-byte atom from a 4-D tensor map over THIS GPU's pool [head_dim, kv head, position, block],
//              128-byte swizzle, K three tiles deep and V four (head_dim 128: one and two); a stage is refilled when the
//              MMA that read it has committed (tcgen05.commit -> mbarrier). The softmax threads never touch K or V.
// Two CTAs per SM at both head sizes (Depth<HD> below). Pipeline over the key tiles (S and P double buffered, the output O
// single): S runs two tiles ahead,
//   softmax thread, tile j:  wait S(j) | 64 scores into registers | max | (rescale O) | exp, sum, P(j) to shared memory
//                            | arrive on "P(j) ready" - and on to tile j+1 without waiting for the other rows
//   issuing lane, tile j:    wait until all 128 rows delivered P(j) | issue PV(j) (O += P.V in tensor memory), S(j+2)
// so the tensor cores compute PV(j-1) and S(j+1) while the threads are in softmax(j). O stays in tensor memory: it is
// rescaled only when a row's maximum outgrew the exponent's reference by more than 2^8 (see the kernel), and read once
// at the end. No CTA-wide barrier inside the loop. Tiles wholly below every row's causal limit skip the mask. Rows of a sequence's last V tile at or past its length are zeroed in shared memory (a block's
// unused slots may hold anything, and 0 x NaN would poison the row). Every mbarrier wait is bounded: on expiry the CTA
// counts an error in the plan header (ns_collect_status), skips its stores, waits for its copies in flight, frees its
// tensor memory and returns.
#include <cuda.h>

#include "attn_plan.cuh"
#include "common.cuh"

namespace ns {

int prefill_cluster_size();      // c_api.cu: NS_TUNE_PREFILL_CLUSTER (0 = built-in choice)

namespace tc {

constexpr int kRows = 128;          // UMMA M = softmax threads (one per row)
constexpr int kThreads = kRows + 64; // + one warp whose first lane issues every tcgen05.mma + one whose first lane copies
constexpr int kKeys = 64;           // keys per tile (UMMA N of S, K extent of P.V)
// Pipeline depth per head size. head_dim 64: K three tiles deep (S runs two tiles ahead of the tile in softmax), V four, P
// double buffered - 104 KB, two CTAs per SM. head_dim 128 (tiles twice as large): ONE K stage (K(j+2) is fetched as soon as
// S(j+1) has committed, a whole tile before S(j+2) is issued), two V, P double buffered - 112 KB, so that two CTAs fit an
// SM there too. (Two K stages with a single P buffer, where every softmax thread waits for PV(j-1) before it overwrites P,
// measured 4 % slower.)
template <int HD> struct Depth {
    static constexpr int K = HD == 64 ? 3 : 1, V = HD == 64 ? 4 : 2, P = 2;
    // mbarriers: S0 S1 PV0 PV1 | K full | V full | K free | V free | P0 P1 ready (one arrival per softmax thread)
    static constexpr int BarS = 0, BarPV = 2, BarKFull = 4, BarVFull = BarKFull + K, BarKFree = BarVFull + V, BarVFree = BarKFree + K,
                         BarPReady = BarVFree + V, Bars = BarPReady + 2;
};
constexpr int kTailBytes = 256;     // mbarriers, the tensor-memory address and the abort flag, behind the tiles
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr int kDefaultCluster = 1;  // CTAs sharing one work item's key tiles (see launch_prefill_tc_hd)

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two fp32 values in one 64-bit register pair and the packed FMA-pipe instructions on them.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
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

// Instruction descriptor for kind::f16: fp32 accumulate, bf16 A and B, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(bool b_mn_major, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
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

// The copying thread's wait: also gives up when the softmax threads raised the CTA's abort flag.
__device__ __forceinline__ bool mbar_wait_or_abort(uint32_t mbar_saddr, uint32_t parity, const volatile uint32_t* abort_flag) {
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
        if (*abort_flag) return false;
    }
    return false;
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar_saddr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar_saddr), "r"(bytes) : "memory");
}

// One box [64 elements, 1 head, 16 positions, 1 block] of a pool into shared memory (2 KB, 128-byte swizzle).
__device__ __forceinline__ void tma_load_block(uint32_t dst, const CUtensorMap* map, int elem, int head, int block, uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
        "l"(map), "r"(elem), "r"(head), "r"(0), "r"(block), "r"(mbar)
        : "memory");
}

// Named barrier 1: the 128 softmax threads and the issuing warp meet once, when Q is in place.
__device__ __forceinline__ void q_ready_barrier() { asm volatile("bar.sync 1, %0;" ::"r"(kRows + 32) : "memory"); }

__device__ __forceinline__ void mbar_arrive(uint32_t mbar_saddr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar_saddr) : "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane, requested only: tmem_ld_wait() before the values are used.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
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
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

constexpr float kRescaleStep = 8.f;   // the exponent's reference may lag the row maximum by up to 2^8 (see the kernel)

}  // namespace tc

template <int HD>
__global__ void __launch_bounds__(tc::kThreads, 2)
prefill_tc_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map, const AttnParams p) {
    using namespace tc;
    using D = Depth<HD>;
    constexpr int kStagesK = D::K, kStagesV = D::V, kBufsP = D::P;
    constexpr int kBarS = D::BarS, kBarPV = D::BarPV, kBarKFull = D::BarKFull, kBarVFull = D::BarVFull, kBarKFree = D::BarKFree,
                  kBarVFree = D::BarVFree, kBarPReady = D::BarPReady, kBars = D::Bars;
    static_assert(kBars * 8 + 8 <= kTailBytes, "the tail holds the barriers and two words");
    constexpr int ATOMS = HD / 64;                  // 128-byte-wide swizzle atoms per head row
    constexpr int Q_BYTES = kRows * 128 * ATOMS;    // [atom][128 rows][128 B]
    constexpr int KV_BYTES = kKeys * 128 * ATOMS;   // [atom][64 keys][128 B]
    constexpr int P_BYTES = kRows * 128;            // [128 rows][64 keys] bf16
    constexpr uint32_t COL_S = 0, COL_O = 2 * kKeys;             // tensor memory: S0, S1, O
    constexpr uint32_t TMEM_COLS = 256;                            // 128 + HD rounded up to a power of two
    // No static shared memory: the dynamic array then starts at the CTA's first usable byte, which is 1024-byte aligned
    // on this architecture (the launcher adds 1 KB of slack where there is room, and the kernel checks - see below).
    extern __shared__ __align__(1024) uint8_t smem_raw[];

    const PlanHeader* hdr = reinterpret_cast<const PlanHeader*>(p.ws + p.L.header);
    // The CTAs of a thread-block cluster share one work item: rank r takes the r-th share of its key tiles and the shares
    // meet in the first CTA's shared memory (an item's cost grows with its context: without the split the longest item
    // alone set the kernel's duration).
    uint32_t crank, csize;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
    asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(csize));
    // Which (item, KV head) this CTA takes. The plan lists the items heaviest first. Without cluster sharing the CTAs take
    // them in the order the hardware hands CTAs out (linear block id): longest first. Where the units are more than one CTA
    // per SM but at most two (one wave), ids past the first SM-count take the LIGHTEST units first, so that an SM's second
    // CTA is light where its first is heavy: the kernel lasts as long as its slowest SM, and two heavy items on one SM
    // (40 + 36 key tiles of 64 in benchmark configuration 1) were that.
    int item_idx, g;
    {
        const int n_items = hdr->n_prefill_items, n_kv = (int)gridDim.y;
        if (csize > 1) {
            item_idx = (int)(blockIdx.x / csize);
            g = blockIdx.y;
        } else {
            const int units = n_items * n_kv, S = p.sm_count;
            const int lin = (int)(blockIdx.x + gridDim.x * blockIdx.y);
            int r = lin;
            if (S > 0 && units > S && units <= 2 * S && lin >= S) r = units - 1 - (lin - S);
            item_idx = lin < units ? r / n_kv : n_items;
            g = r % n_kv;
        }
        if (item_idx >= n_items) {                // the whole cluster leaves together
            if (p.overlap_prefill) pdl_wait();    // the grid must not complete before the decode kernel it overlaps
            return;
        }
    }
    const int2 item = reinterpret_cast<const int2*>(p.ws + p.L.prefill_items)[item_idx];
    const int s = item.x, q_start = item.y;
    const int tid = threadIdx.x, warp = tid >> 5;
    const bool worker = tid < kRows;              // one softmax thread per row
    const bool issuer = tid == kRows;             // first lane of warp 4: every tcgen05.mma
    const bool copier = tid == kRows + 32;        // first lane of warp 5: every K/V copy
    const int q0 = p.cu_seqlens[s];
    const int T = p.cu_seqlens[s + 1] - q0;
    const int len = p.seq_lens[s];
    const int ctx = len - T;
    const int32_t* table = p.block_tables + (int64_t)(p.table_rows ? p.table_rows[s] : s) * p.table_stride;
    const int kv_end = min(len, ctx + q_start + kPrefillTileTokens);
    const int all_tiles = (kv_end + kKeys - 1) / kKeys;
    const int tile0 = (int)(((long long)all_tiles * crank) / csize);              // this CTA's tiles: [tile0, tile0 + n_tiles)
    const int n_tiles = (int)(((long long)all_tiles * (crank + 1)) / csize) - tile0;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t sQ = base, sK = sQ + Q_BYTES, sV = sK + kStagesK * KV_BYTES, sP = sV + kStagesV * KV_BYTES;
    const uint32_t bar0 = sP + kBufsP * P_BYTES;    // the tail: barriers, then two words
    auto bar = [&](int i) -> uint32_t { return bar0 + 8u * (uint32_t)i; };
    volatile uint32_t* tail_words = reinterpret_cast<volatile uint32_t*>(smem_raw + (bar0 - raw) + kBars * 8);
    volatile uint32_t& tmem_slot = tail_words[0];
    volatile uint32_t& abort_flag = tail_words[1];  // raised when a bounded wait ran out: the copying thread stops too
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if (bar0 - raw + kTailBytes > dyn_bytes) {      // the array did not start where the launcher's size assumes: never expected
        if (tid == 0) atomicAdd(&reinterpret_cast<PlanHeader*>(p.ws + p.L.header)->errors, 1);
        if (p.overlap_prefill) pdl_wait();
        return;
    }

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kBars; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar(i)), "r"(i >= kBarPReady ? kRows : 1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        abort_flag = 0;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(bar0 + kBars * 8), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // row of this thread
    const int tok = q_start + ((tid & (kRows - 1)) >> 3), hh = tid & 7;
    const bool row_ok = worker && tok < T && hh < p.group;
    const int h = g * p.group + hh;
    // Q tile: one head row per thread, 128 bytes per atom
    if (worker) {
        const __nv_bfloat16* src = p.q + (int64_t)(q0 + (row_ok ? tok : 0)) * p.q_stride + (int64_t)(row_ok ? h : 0) * HD;
#pragma unroll
        for (int c = 0; c < 8 * ATOMS; ++c)
            cp_async16(sQ + (c >> 3) * (kRows * 128) + tid * 128 + (((c & 7) ^ (tid & 7)) << 4), src + c * 8, row_ok ? 16 : 0);
    }
    cp_async_commit();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();                  // barriers initialised, tensor memory allocated; Q is still on its way, so that the
                                      // copying lane's first K/V requests travel beside it
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    const uint32_t t_lane = tmem + ((uint32_t)(32 * (warp & 3)) << 16);     // this warp's 32 lanes; lane = row

    // keys of tile kt that exist in the pool and may be seen by this item: whole blocks up to kv_end
    auto tile_blocks = [&](int kt) -> int { return min(kKeys / 16, (kv_end - (tile0 + kt) * kKeys + 15) >> 4); };
    bool ok = true;
    float m_run = -INFINITY, l_run = 0.f;   // this row's exponent reference and sum (softmax threads)
    int k_issued = 0, v_issued = 0;   // copying thread: tiles whose copies were issued

    if (copier) {
        // ---- K/V tiles: block ids one tile ahead of the copies that need them
        int ids[kKeys / 16], ids_next[kKeys / 16];
        auto fetch_ids = [&](int kt, int (&dst)[kKeys / 16]) {
#pragma unroll
            for (int it = 0; it < kKeys / 16; ++it)
                dst[it] = (kt < n_tiles && it < tile_blocks(kt)) ? table[(((tile0 + kt) * kKeys) >> 4) + it] : 0;
        };
        fetch_ids(0, ids_next);
        for (int kt = 0; kt < n_tiles; ++kt) {
#pragma unroll
            for (int it = 0; it < kKeys / 16; ++it) ids[it] = ids_next[it];
            fetch_ids(kt + 1, ids_next);
            const int nb = tile_blocks(kt), sk = kt % kStagesK, sv = kt % kStagesV;
            const uint32_t bytes = (uint32_t)nb * 16u * 128u * ATOMS;
            // K(kt) goes where K(kt - 3) was: free once S(kt - 3) has committed
            if (kt >= kStagesK && !mbar_wait_or_abort(bar(kBarKFree + sk), (uint32_t)((kt / kStagesK - 1) & 1), tail_words + 1)) { ok = false; break; }
            mbar_expect_tx(bar(kBarKFull + sk), bytes);
#pragma unroll
            for (int it = 0; it < kKeys / 16; ++it)
                if (it < nb) {
#pragma unroll
                    for (int a = 0; a < ATOMS; ++a)
                        tma_load_block(sK + sk * KV_BYTES + a * (kKeys * 128) + it * 2048, &k_map, a * 64, g, ids[it], bar(kBarKFull + sk));
                }
            k_issued = kt + 1;
            if (kt >= kStagesV && !mbar_wait_or_abort(bar(kBarVFree + sv), (uint32_t)((kt / kStagesV - 1) & 1), tail_words + 1)) { ok = false; break; }
            mbar_expect_tx(bar(kBarVFull + sv), bytes);
#pragma unroll
            for (int it = 0; it < kKeys / 16; ++it)
                if (it < nb) {
#pragma unroll
                    for (int a = 0; a < ATOMS; ++a)
                        tma_load_block(sV + sv * KV_BYTES + a * (kKeys * 128) + it * 2048, &v_map, a * 64, g, ids[it], bar(kBarVFull + sv));
                }
            v_issued = kt + 1;
        }
        if (!ok) abort_flag = 1;
    } else if (warp == 4) {
        q_ready_barrier();            // the softmax threads' Q rows are in shared memory and visible to the tensor cores
        if (issuer) {
        // ---- descriptors, built once: an instruction's operand is the base plus a byte offset (>> 4) in the address field
        constexpr uint32_t idesc_s = instr_desc(false, kKeys), idesc_pv = instr_desc(true, HD);
        const uint64_t dQ = smem_desc(sQ, 16, 1024), dK = smem_desc(sK, 16, 1024);
        const uint64_t dP = smem_desc(sP, 16, 1024);
        const uint64_t dV = smem_desc(sV, kKeys * 128, 1024);          // MN-major B: next 64-column atom kKeys * 128 bytes on
        auto issue_s = [&](int kt) {                                    // S(kt) = Q . K(kt)^T into S buffer kt & 1
            const int sk = kt % kStagesK;
            if (!mbar_wait(bar(kBarKFull + sk), (uint32_t)((kt / kStagesK) & 1))) { ok = false; return; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t k0 = dK + (uint64_t)((sk * KV_BYTES) >> 4);
            const uint32_t d = tmem + COL_S + (uint32_t)((kt & 1) * kKeys);
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {                      // K extent 16 per instruction = 32 bytes inside an atom
                const uint32_t a_off = (uint32_t)(((kk >> 2) * (kRows * 128) + (kk & 3) * 32) >> 4);
                const uint32_t b_off = (uint32_t)(((kk >> 2) * (kKeys * 128) + (kk & 3) * 32) >> 4);
                mma_f16(d, dQ + a_off, k0 + b_off, idesc_s, kk > 0);
            }
            mma_commit(bar(kBarS + (kt & 1)));                          // the softmax threads' signal
            mma_commit(bar(kBarKFree + sk));                            // and the copying thread's: K's buffer is free
        };
        auto issue_pv = [&](int kt) {                                   // O += P(kt) . V(kt)
            const int sv = kt % kStagesV;
            if (!mbar_wait(bar(kBarVFull + sv), (uint32_t)((kt / kStagesV) & 1))) { ok = false; return; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t p0 = dP + (uint64_t)(((kt % kBufsP) * P_BYTES) >> 4);
            const uint64_t v0 = dV + (uint64_t)((sv * KV_BYTES) >> 4);
            const uint32_t d = tmem + COL_O;
#pragma unroll
            for (int kk = 0; kk < kKeys / 16; ++kk)                     // 16 keys per instruction: 32 bytes of P, 16 rows of V
                mma_f16(d, p0 + (uint32_t)((kk * 32) >> 4), v0 + (uint32_t)((kk * 2048) >> 4), idesc_pv, (kt > 0 || kk > 0) ? 1u : 0u);
            mma_commit(bar(kBarPV + (kt & 1)));
            mma_commit(bar(kBarVFree + sv));
        };

        // S(0) and S(1) first; then, per tile, PV(kt) and S(kt + 2) as soon as every softmax thread has delivered P(kt) -
        // which also says that each of them has read S(kt) for the last time and left the output alone
        if (n_tiles > 0) issue_s(0);
        if (n_tiles > 1) issue_s(1);
        for (int kt = 0; kt < n_tiles && ok; ++kt) {
            if (!mbar_wait_or_abort(bar(kBarPReady + (kt & 1)), (uint32_t)((kt >> 1) & 1), tail_words + 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_pv(kt);
            if (kt + 2 < n_tiles) issue_s(kt + 2);
        }
        if (!ok) abort_flag = 1;
        }
    } else if (worker) {
        cp_async_wait<0>();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy writes of Q -> visible to the MMA
        q_ready_barrier();
        const int limit = ctx + tok;      // last key this row may see
        const uint32_t t_o = t_lane + COL_O;
        const volatile uint32_t* abort_now = tail_words + 1;

#ifdef NS_DEBUG_HOOKS
        // profiling build: clock64 stamps of the first work item's thread 0, 8 per key tile, first 16 tiles
        long long* stamps = (p.timeline != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0) ? p.timeline : nullptr;
#define NS_STAMP(i) do { if (stamps != nullptr && kt < 16) stamps[kt * 8 + (i)] = clock64(); } while (0)
#else
#define NS_STAMP(i) do { } while (0)
#endif
        for (int kt = 0; kt < n_tiles; ++kt) {
            NS_STAMP(0);
            if (*abort_now) ok = false;                                    // another thread's wait ran out
            if (!ok) break;
            {
                if (!mbar_wait(bar(kBarS + (kt & 1)), (uint32_t)((kt >> 1) & 1))) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                NS_STAMP(1);

                // ---- softmax on this thread's row, the tile's 64 scores in registers (the running output stays in tensor
                // memory). Four independent chains for the maximum and for the sum; the softmax scale is folded into the
                // exponent's multiply-add.
                const uint32_t s_src = t_lane + COL_S + (uint32_t)((kt & 1) * kKeys);
                const bool masked = (tile0 + kt) * kKeys + kKeys - 1 > ctx + q_start;    // else every row sees every key of the tile
                const int key_base = (tile0 + kt) * kKeys;
                uint32_t sr[2][32];
                tmem_ld32_issue(s_src, sr[0]);
                tmem_ld32_issue(s_src + 32, sr[1]);
                tmem_ld_wait();
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                if (masked) {                                              // scores past the row's causal limit leave the tile
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (key_base + 32 * hf + i > limit) sr[hf][i] = 0xff800000u;      // -inf: 2^(-inf) = 0 below
                }
#pragma unroll
                for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sr[hf][i]));
                NS_STAMP(2);
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
                // The exponent's reference m_run follows the row maximum lazily: it moves only when the maximum has grown by
                // more than kRescaleStep (or was -inf), so p = 2^(s - m_run) <= 2^kRescaleStep and most tiles leave the
                // output in tensor memory untouched. (o, l) stay consistent with whatever reference they were summed
                // under: when it moves both are multiplied by 2^(old - new). The decision is per warp (the tensor-memory
                // accesses are warp-wide); rows that need no move then refresh their reference too.
                const bool move = __any_sync(0xffffffffu, mx > m_run + kRescaleStep);
                NS_STAMP(6);
#ifdef NS_DEBUG_HOOKS
                if (stamps != nullptr && kt < 16) stamps[kt * 8 + 7] = move ? 1 : 0;
#endif
                // With two P buffers P(kt) overwrites what PV(kt-2) read: PV(kt-2) was issued before S(kt) by the same thread, so
                // S(kt)'s commit, waited for above, covers it. With one buffer, and for a move (which rewrites the output), PV(kt-1)
                // - issued when the last row of tile kt-1 arrived - has to be over.
                if ((kBufsP == 1 || move) && kt > 0) {
                    if (!mbar_wait(bar(kBarPV + ((kt - 1) & 1)), (uint32_t)(((kt - 1) >> 1) & 1))) ok = false;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                if (move) {
                    const float m_new = fmaxf(m_run, mx);
                    const float alpha = m_new == -INFINITY ? 1.f : ex2(m_run - m_new);      // 0 while the row has seen nothing
                    m_run = m_new;
                    l_run *= alpha;
                    if (kt > 0) {
#pragma unroll
                        for (int c = 0; c < HD / 32; ++c) {
                            uint32_t r[32];
                            tmem_ld32_issue(t_o + 32 * c, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                            tmem_st32(t_o + 32 * c, r);
                        }
                        tmem_st_wait();
                    }
                }
                // a CTA that holds only late tiles of its item can meet rows that see none of its keys yet
                const float m_ref = m_run == -INFINITY ? 0.f : m_run;
                // exponent arguments and row sums two at a time (fma / add .f32x2: half the FMA-pipe instructions)
                const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2), neg_m2 = pack_f32x2(-m_ref, -m_ref);
                uint64_t ps2[2] = {0ull, 0ull};                           // (0.f, 0.f) twice: four chains
                const uint32_t p_dst = sP + (kt % kBufsP) * P_BYTES + tid * 128;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float x0, x1;
                        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sr[hf][i]), __uint_as_float(sr[hf][i + 1])), scale2, neg_m2), x0, x1);
                        v[i] = ex2(x0);
                        v[i + 1] = ex2(x1);
                        ps2[(i >> 1) & 1] = add_f32x2(ps2[(i >> 1) & 1], pack_f32x2(v[i], v[i + 1]));
                    }
                    // P row as bf16 into shared memory (K-major, swizzled like the other operands)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint4 pk;
                        pk.x = pack_bf16x2(v[8 * c + 0], v[8 * c + 1]);
                        pk.y = pack_bf16x2(v[8 * c + 2], v[8 * c + 3]);
                        pk.z = pack_bf16x2(v[8 * c + 4], v[8 * c + 5]);
                        pk.w = pack_bf16x2(v[8 * c + 6], v[8 * c + 7]);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_dst + (((4 * hf + c) ^ (tid & 7)) << 4)),
                                     "r"(pk.x), "r"(pk.y), "r"(pk.z), "r"(pk.w)
                                     : "memory");
                    }
                }
                {
                    float a0, a1, b0, b1;
                    unpack_f32x2(ps2[0], a0, a1);
                    unpack_f32x2(ps2[1], b0, b1);
                    l_run += (a0 + a1) + (b0 + b1);
                }
                NS_STAMP(3);
                // V rows the copies did not bring (blocks past kv_end) or that lie at or past the sequence's length hold
                // whatever shared memory or the pool's unused slots held: zero them (their P columns are zero, but 0 x NaN is
                // NaN). Only a sequence's last tile has such rows.
                const int v_rows = min(len, key_base + 16 * tile_blocks(kt)) - key_base;
                if (v_rows < kKeys) {
                    const int sv = kt % kStagesV;
                    if (!mbar_wait(bar(kBarVFull + sv), (uint32_t)((kt / kStagesV) & 1))) ok = false;
                    for (int c = v_rows * 8 * ATOMS + tid; c < kKeys * 8 * ATOMS; c += kRows) {
                        const int row = c / (8 * ATOMS), cc = c % (8 * ATOMS);   // cc: atom * 8 + 16-byte chunk (the swizzle only permutes chunks inside a row)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(sV + sv * KV_BYTES + (cc >> 3) * (kKeys * 128) + row * 128 + ((cc & 7) << 4)),
                                     "r"(0)
                                     : "memory");
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes of P (and V's tail) -> the MMA
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (!ok) break;                                                // (no arrival: the issuing thread gives up on the flag)
            mbar_arrive(bar(kBarPReady + (kt & 1)));                       // no softmax thread waits for another one
            NS_STAMP(4);
        }
        if (!ok) abort_flag = 1;                                           // (every thread that saw a failure writes the same value)
    }
    __syncthreads();                  // all three roles are through their tiles (or gave up)
    if (abort_flag) {
        ok = false;
        if (copier) {
            // the copies already issued must land before this CTA's shared memory goes away (bounded like every wait)
            for (int t = max(0, k_issued - kStagesK); t < k_issued; ++t) mbar_wait(bar(kBarKFull + t % kStagesK), (uint32_t)((t / kStagesK) & 1));
            for (int t = max(0, v_issued - kStagesV); t < v_issued; ++t) mbar_wait(bar(kBarVFull + t % kStagesV), (uint32_t)((t / kStagesV) & 1));
        }
        __syncthreads();
    }

    // The row's output leaves tensor memory once, after the last PV, 32 columns at a time (registers: the loop above and
    // this epilogue share one budget that lets two CTAs fit an SM).
    const bool have_o = ok && worker && n_tiles > 0;      // warp-uniform
    if (have_o) {
        if (!mbar_wait(bar(kBarPV + ((n_tiles - 1) & 1)), (uint32_t)(((n_tiles - 1) >> 1) & 1))) ok = false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    auto load_o = [&](int c, float (&v)[32]) {            // columns [32 c, 32 c + 32) of this row; zeros without tiles
        if (have_o) {
            uint32_t r[32];
            tmem_ld32_issue(t_lane + COL_O + 32 * c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
    };
    __nv_bfloat16* out_row = p.out + (int64_t)(q0 + (row_ok ? tok : 0)) * p.out_stride + (int64_t)(row_ok ? h : 0) * HD;
    auto store_o = [&](int c, const float (&v)[32], float inv) {
        if (!(ok && row_ok)) return;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            uint4 w;
            w.x = pack_bf16x2(v[8 * e + 0] * inv, v[8 * e + 1] * inv);
            w.y = pack_bf16x2(v[8 * e + 2] * inv, v[8 * e + 3] * inv);
            w.z = pack_bf16x2(v[8 * e + 4] * inv, v[8 * e + 5] * inv);
            w.w = pack_bf16x2(v[8 * e + 6] * inv, v[8 * e + 7] * inv);
            *reinterpret_cast<uint4*>(out_row + 32 * c + 8 * e) = w;
        }
    };

    if (csize > 1) {
        // every CTA of the cluster is through its tiles: the first CTA's shared memory is free to receive the others'
        // (o, m, l) rows, one row per thread, HD + 4 floats apart
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        constexpr int PART_ROW = HD + 4;
        if (crank != 0 && worker) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(base));
            uint64_t generic;
            asm volatile("cvta.shared::cluster.u64 %0, %1;" : "=l"(generic) : "l"((uint64_t)remote));
            float* dst = reinterpret_cast<float*>(generic) + ((size_t)(crank - 1) * kRows + tid) * PART_ROW;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                float v[32];
                load_o(c, v);
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    *reinterpret_cast<float4*>(dst + 32 * c + 4 * e) = make_float4(v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
            }
            *reinterpret_cast<float2*>(dst + HD) = make_float2(m_run, l_run);
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (crank == 0 && worker) {
            const float* mine = reinterpret_cast<const float*>(smem_raw + (base - raw));
            // weights of the shares under the common maximum, then the output 32 columns at a time
            float m_fin = m_run;
            for (uint32_t r = 1; r < csize; ++r) m_fin = fmaxf(m_fin, mine[((size_t)(r - 1) * kRows + tid) * PART_ROW + HD]);
            float wgt[4] = {0.f, 0.f, 0.f, 0.f};            // [0]: this CTA's share; clusters have at most 4 CTAs
            float l_fin = 0.f;
            if (m_fin != -INFINITY) {
                wgt[0] = ex2(m_run - m_fin);
                l_fin = l_run * wgt[0];
                for (uint32_t r = 1; r < csize && r < 4; ++r) {
                    const float2 ml = *reinterpret_cast<const float2*>(mine + ((size_t)(r - 1) * kRows + tid) * PART_ROW + HD);
                    wgt[r] = ex2(ml.x - m_fin);
                    l_fin = fmaf(ml.y, wgt[r], l_fin);
                }
            }
            const float inv = l_fin > 0.f ? 1.f / l_fin : 0.f;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                float v[32];
                load_o(c, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] *= wgt[0];
                for (uint32_t r = 1; r < csize && r < 4; ++r) {
                    const float* src = mine + ((size_t)(r - 1) * kRows + tid) * PART_ROW + 32 * c;
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float4 t = *reinterpret_cast<const float4*>(src + 4 * e);
                        v[4 * e] = fmaf(t.x, wgt[r], v[4 * e]);
                        v[4 * e + 1] = fmaf(t.y, wgt[r], v[4 * e + 1]);
                        v[4 * e + 2] = fmaf(t.z, wgt[r], v[4 * e + 2]);
                        v[4 * e + 3] = fmaf(t.w, wgt[r], v[4 * e + 3]);
                    }
                }
                store_o(c, v, inv);
            }
        }
    } else if (worker) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
            float v[32];
            load_o(c, v);
            store_o(c, v, inv);
        }
    }
    if (!ok && tid == 0)        // a wait expired: count it where the host can read it (ns_collect_status)
        atomicAdd(&reinterpret_cast<PlanHeader*>(p.ws + p.L.header)->errors, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    if (p.overlap_prefill) pdl_wait();            // complete only after the decode kernel this one ran beside
}

bool prefill_tc_supported(int n_heads, int n_kv_heads, int head_dim, int block_size) {
    if (block_size != 16 || n_heads % n_kv_heads != 0) return false;
    const int group = n_heads / n_kv_heads;
    return group >= 1 && group <= 8 && (head_dim == 64 || head_dim == 128);
}

namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// 4-D tensor map over one layer's K or V pool, innermost first: [head_dim, kv heads, 16 positions of a block, blocks],
// bf16, strides as the caller gave them; a box is one head's 64 elements (one 128-byte atom) x 16 positions of one block,
// written to shared memory with the 128-byte swizzle the UMMA descriptors expect. The pool's block count is not part of
// the attention call: the block extent is the largest the map takes, and block ids come from the block tables.
static bool make_pool_map(CUtensorMap* map, const void* pool, int head_dim, int n_kv_heads, int64_t blk_stride, int64_t pos_stride,
                          int64_t head_stride) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t gdim[4] = {(cuuint64_t)head_dim, (cuuint64_t)n_kv_heads, 16, (cuuint64_t)1 << 31};
    const cuuint64_t gstride[3] = {(cuuint64_t)head_stride * 2, (cuuint64_t)pos_stride * 2, (cuuint64_t)blk_stride * 2};
    const cuuint32_t box[4] = {64, 1, 16, 1};
    const cuuint32_t estride[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(pool), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc

// NS_ERR_UNSUPPORTED: the driver refused a tensor map over these pools (strides it cannot express); the caller then uses
// the mma.sync kernel.
template <int HD>
static int launch_prefill_tc_hd(const AttnParams& p, int max_items, cudaStream_t st) {
    constexpr int atoms = HD / 64;
    using D = tc::Depth<HD>;
    // tiles + tail; 1 KB of slack for the 1024-byte alignment where two CTAs still fit an SM with it (head_dim 64)
    constexpr int smem = tc::kRows * 128 * atoms + (D::K + D::V) * tc::kKeys * 128 * atoms + D::P * tc::kRows * 128 + tc::kTailBytes +
                         (HD == 64 ? 1024 : 0);
    CUtensorMap k_map, v_map;
    if (!tc::make_pool_map(&k_map, p.k_pool, HD, p.n_kv_heads, p.blk_stride, p.pos_stride, p.head_stride) ||
        !tc::make_pool_map(&v_map, p.v_pool, HD, p.n_kv_heads, p.blk_stride, p.pos_stride, p.head_stride))
        return NS_ERR_UNSUPPORTED;
    static SmemOptIn optin;
    if (optin.needs((size_t)smem)) {
        cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "prefill attention (tcgen05): cannot reserve %d bytes of shared memory: %s",
                                          smem, cudaGetErrorString(e));
        optin.done((size_t)smem);
    }
    // a work item's key tiles can be shared by a cluster of CTAs (NS_TUNE_PREFILL_CLUSTER); clamped to what fits: the
    // other CTAs' rows of HD + 4 floats land in the first CTA's shared memory
    int cl = prefill_cluster_size() > 0 ? prefill_cluster_size() : tc::kDefaultCluster;
    while (cl > 1 && ((cl - 1) * tc::kRows * (HD + 4) * 4 > smem - 1024 - tc::kTailBytes || cl > 4)) cl >>= 1;     // the other CTAs' rows must fit the first one's
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(max_items * cl), (unsigned)p.n_kv_heads);
    cfg.blockDim = dim3(tc::kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cl;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.overlap_prefill ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, prefill_tc_kernel<HD>, k_map, v_map, p);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "prefill attention (tcgen05): launch failed: %s", cudaGetErrorString(e));
    return NS_OK;
}

int launch_prefill_tc(const AttnParams& p, int head_dim, int max_items, cudaStream_t st) {
    if (max_items <= 0) return NS_OK;
    return head_dim == 64 ? launch_prefill_tc_hd<64>(p, max_items, st) : launch_prefill_tc_hd<128>(p, max_items, st);
}

}  // namespace ns

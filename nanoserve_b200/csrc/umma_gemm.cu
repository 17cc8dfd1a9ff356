// Decode-sized gate/up projection with SiLU(gate)*up on the 5th-generation tensor cores (tcgen05), weights by TMA.
//
//   out[M <= 64, inter] = bf16( bf16(silu(bf16(x . Wg^T))) * bf16(x . Wu^T) ),   W = [Wg; Wu] (2*inter rows of K), bf16
//
// At M <= 64 the product is a read of 2*inter*K*2 weight bytes. The kernels of this library that stream such weights
// through mma.sync spend ~700 cycles of tensor-core time per 16 weight rows (the legacy path); here the WEIGHT rows are
// the M operand of one UMMA tile (swap A/B), so a CTA's 128 weight rows x K cost 4 tcgen05.mma per 64 columns:
//   * one CTA per SM (a tiled TMA load of 128-byte rows was measured at ~44 GB/s per SM: every SM has to pull); CTA i owns a
//     contiguous share of inter/#SM gate rows (some CTAs one more) and the matching up rows: gate rows sit at tile row
//     0, up rows at tile row `region`, the remaining rows of the 128-row tile are never read back. Per 64-column chunk
//     and region one TMA box of `base` rows plus, where the share has one more, a one-row box
//     (cp.async.bulk.tensor.2d, SWIZZLE_128B: exactly the layout the K-major UMMA descriptor reads), into a ring of
//     stages with a full / empty mbarrier pair each (at the model's sizes all of K is in flight at once); the weights
//     are requested BEFORE griddepcontrol.wait, i.e. while the kernel that produces x still runs;
//   * B = the activations [NT token rows x K], fetched once by TMA (rows beyond M are out of bounds: zero filled);
//   * D[128 weight rows x NT tokens] accumulates in tensor memory (NT columns); one thread issues the MMAs, one the TMA
//     loads (four lanes side by side), all 128 read their own accumulator row (lane = tile row) with tcgen05.ld and park
//     it in shared memory, from where consecutive threads finish consecutive output columns of a token.
// Rounding points are those of the unfused ops. Every mbarrier wait is bounded; a wait that runs out raises an error
// count (ns_umma_gemm_errors), skips the stores and still frees the CTA's tensor memory.
#include <cuda.h>

#include "common.cuh"

namespace ns {

namespace ug {

constexpr int kRows = 128;               // UMMA M: 64 gate rows + 64 up rows
constexpr int kChunk = 64;               // K columns per stage: 128 bytes, one swizzle atom wide
constexpr int kAStage = kRows * 128;     // bytes of one A stage
constexpr int kMaxStages = 28;
constexpr uint32_t kWaitLimit = 1u << 22;

__device__ unsigned int g_errors = 0;
static long long* g_timeline = nullptr;

__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(done)
            : "r"(mbar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// 2-D tiled TMA load (no multicast): box at element coordinates {x (innermost, a multiple of 8), y} -> shared memory.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(mbar)
                 : "memory");
}
// 64-bit shared-memory matrix descriptor, K-major, SWIZZLE_128B (8-row x 128-byte atoms 1024 bytes apart), sm_100 version.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((16u >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((1024u >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: fp32 accumulate, bf16 A and B (both K-major), M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
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
__device__ __forceinline__ void mma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
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

struct Params {
    __nv_bfloat16* out;      // [M, inter]
    int M, inter, K;
    int n_chunks;            // K / 64
    int stages;              // A ring depth (<= n_chunks)
    int base, rem;           // CTA i owns base + (i < rem) gate rows starting at i*base + min(i, rem), and the same up rows
    int region;              // tile rows reserved per region (gate rows at tile row 0, up rows at tile row `region`)
    long long* timeline;     // debug: clock64 stamps of CTA 0 (null in normal use): [0..15] producer, [16..47] MMA, [48..63] epilogue
};

}  // namespace ug

// NT = token rows of the B operand (UMMA N): 32 or 64.
template <int NT>
__global__ void __launch_bounds__(ug::kRows, 1)
swiglu_umma_kernel(const __grid_constant__ CUtensorMap w_main, const __grid_constant__ CUtensorMap w_one,
                   const __grid_constant__ CUtensorMap x_map, const ug::Params p) {
    using namespace ug;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], b_full, acc_full;
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    const int n_rows = p.base + (cta < p.rem ? 1 : 0);           // gate rows (= up rows) of this CTA
    const int row0 = cta * p.base + min(cta, p.rem);             // its first gate row
    const int S = p.stages, NC = p.n_chunks, R = p.region;
    const uint32_t stage_bytes = (uint32_t)(2 * R) * 128;        // the MMA reads 128 tile rows: the rest is whatever follows
    constexpr int kBChunk = NT * 128;                            // bytes of one B chunk (NT token rows x 64 columns)
    // 1024-byte aligned tiles: [A ring][B chunks][exchange NT x 128 fp32]
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA = base, sB = sA + (uint32_t)S * stage_bytes;
    float* exch = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)) + (size_t)S * stage_bytes + (size_t)NC * kBChunk);

    long long* tl = (p.timeline != nullptr && blockIdx.x == 0) ? p.timeline : nullptr;
    const long long t_start = clock64();
    pdl_launch_dependents();
    if (tid == 0) {
        for (int i = 0; i < S; ++i) {
            mbar_init(smem_u32(&full_bar[i]), 1);
            mbar_init(smem_u32(&empty_bar[i]), 1);
        }
        mbar_init(smem_u32(&b_full), 1);
        mbar_init(smem_u32(&acc_full), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        failed = 0;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(NT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;

    if (warp == 1) {
        // ---- TMA producer warp: weights first (they do not depend on the preceding kernel), then the activations. Lanes
        //      0..3 issue the (up to) four boxes of a chunk side by side: gate main, gate extra row, up main, up extra row.
        const bool extra = n_rows > p.base;
        const uint32_t a_bytes = (uint32_t)(2 * n_rows) * 128;
        auto load_a = [&](int c) {
            const uint32_t mb = smem_u32(&full_bar[c % S]);
            const uint32_t dst = sA + (uint32_t)(c % S) * stage_bytes;
            if (lane == 0) mbar_expect_tx(mb, a_bytes);
            __syncwarp();
            if (lane == 0) tma_load_2d(dst, &w_main, c * kChunk, row0, mb);
            if (lane == 1 && extra) tma_load_2d(dst + (uint32_t)p.base * 128, &w_one, c * kChunk, row0 + p.base, mb);
            if (lane == 2) tma_load_2d(dst + (uint32_t)R * 128, &w_main, c * kChunk, p.inter + row0, mb);
            if (lane == 3 && extra) tma_load_2d(dst + (uint32_t)(R + p.base) * 128, &w_one, c * kChunk, p.inter + row0 + p.base, mb);
        };
        const int first = NC < S ? NC : S;
        if (tl && lane == 0) tl[0] = clock64() - t_start;
        for (int c = 0; c < first; ++c) load_a(c);
        if (tl && lane == 0) tl[1] = clock64() - t_start;
        pdl_wait();
        if (lane == 0) mbar_expect_tx(smem_u32(&b_full), (uint32_t)NC * kBChunk);
        __syncwarp();
        for (int c = lane; c < NC; c += 32) tma_load_2d(sB + (uint32_t)c * kBChunk, &x_map, c * kChunk, 0, smem_u32(&b_full));
        if (tl && lane == 0) tl[3] = clock64() - t_start;
        for (int c = S; c < NC; ++c) {
            bool freed = true;
            if (lane == 0) freed = mbar_wait(smem_u32(&empty_bar[c % S]), (uint32_t)((c / S - 1) & 1));
            freed = __shfl_sync(0xffffffffu, freed, 0);
            if (!freed) {
                if (lane == 0) atomicExch(&failed, 1);
                break;
            }
            load_a(c);
        }
    } else if (warp == 0 && lane == 0) {
        // ---- MMA issuer ---------------------------------------------------------------------------------------------
        constexpr uint32_t idesc = instr_desc(NT);
        const uint64_t dA = smem_desc(sA), dB = smem_desc(sB);
        bool ok = mbar_wait(smem_u32(&b_full), 0);
        if (tl) tl[16] = clock64() - t_start;
        for (int c = 0; c < NC && ok; ++c) {
            ok = mbar_wait(smem_u32(&full_bar[c % S]), (uint32_t)((c / S) & 1));
            if (!ok) break;
            if (tl && c < 30) tl[17 + c] = clock64() - t_start;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // descriptors = the bases built once + a byte offset (>> 4) in the address field: a lone thread that builds two
            // 64-bit descriptors per instruction needs ~190 cycles per tcgen05.mma, one that adds an offset ~40
            const uint64_t a = dA + (uint64_t)(((uint32_t)(c % S) * stage_bytes) >> 4), b = dB + (uint64_t)(((uint32_t)c * kBChunk) >> 4);
#pragma unroll
            for (int kk = 0; kk < kChunk / 16; ++kk)       // 16 columns per instruction = 32 bytes along K
                mma_f16(tmem, a + (uint64_t)((kk * 32) >> 4), b + (uint64_t)((kk * 32) >> 4), idesc, (c > 0 || kk > 0) ? 1u : 0u);
            mma_commit(smem_u32(&empty_bar[c % S]));       // arrives when the MMAs above have read the stage
        }
        if (!ok) atomicExch(&failed, 1);
        mma_commit(smem_u32(&acc_full));                   // arrives when every MMA issued so far is complete
    }

    // ---- epilogue: thread `tid` reads accumulator row `tid` (lane = tile row: gate rows from 0, up rows from R) -------------
    __syncwarp();
    bool ok = mbar_wait(smem_u32(&acc_full), 0);
    if (tl && tid == 127) tl[48] = clock64() - t_start;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    ok = __syncthreads_and(ok && failed == 0);
    if (ok) {
        const uint32_t t_lane = tmem + ((uint32_t)(32 * warp) << 16);
#pragma unroll
        for (int c0 = 0; c0 < NT; c0 += 32) {
            float v[32];
            tmem_ld32(t_lane + c0, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) exch[(c0 + i) * kRows + tid] = round_to<__nv_bfloat16>(v[i]);   // bf16(gemm), as the unfused op
        }
    }
    __syncthreads();
    if (tl && tid == 127) tl[49] = clock64() - t_start;
    if (ok) {
        // outputs of this CTA: M tokens x n_rows columns, consecutive threads on consecutive columns
        const int total = p.M * n_rows;
        for (int idx = tid; idx < total; idx += kRows) {
            const int t = idx / n_rows, j = idx - t * n_rows;
            const float g = exch[t * kRows + j], u = exch[t * kRows + R + j];
            const float sg_ = round_to<__nv_bfloat16>(g / (1.0f + expf(-g)));
            p.out[(int64_t)t * p.inter + row0 + j] = __float2bfloat16_rn(sg_ * u);
        }
    }
    if (tl && tid == 127) tl[50] = clock64() - t_start;
    if (!ok && tid == 0) atomicAdd(&g_errors, 1u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NT) : "memory");
}

namespace ug {

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

// Row-major bf16 matrix [rows, cols] -> 2-D tensor map with boxes of 64 columns x box_rows rows, 128-byte swizzle,
// zero fill outside the matrix.
static int make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return fail(NS_ERR_CUDA, "swiglu_gemm: the driver does not export cuTensorMapEncodeTiled");
    const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kChunk, (cuuint32_t)box_rows};
    const cuuint32_t estride[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estride,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NS_ERR_CUDA, "swiglu_gemm: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return NS_OK;
}

static int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return sms;
}

// Grid and row split for `inter` gate rows: one CTA per SM when every CTA's share fits half a 128-row tile.
static bool plan_rows(int inter, int* grid, int* base, int* rem, int* region) {
    int g = sm_count();
    if (g <= 0) return false;
    if (g > inter) g = inter;
    while ((inter + g - 1) / g > 64) ++g;                 // more CTAs than SMs only if a share would exceed 64 rows
    *grid = g;
    *base = inter / g;
    *rem = inter % g;
    *region = ((*base + (*rem ? 1 : 0)) + 7) & ~7;
    return *base >= 1;
}

template <int NT>
static int launch(const void* x, const void* w, Params p, cudaStream_t st) {
    int grid = 0;
    if (!plan_rows(p.inter, &grid, &p.base, &p.rem, &p.region))
        return fail(NS_ERR_CUDA, "swiglu_gemm: cannot query the SM count");
    const size_t stage = (size_t)2 * p.region * 128, b_bytes = (size_t)p.n_chunks * NT * 128, exch = (size_t)NT * kRows * 4;
    // the MMA reads 128 tile rows (16 KB) from every stage start: the last stage must have that much allocated after it
    const size_t tail = 16384 > stage + b_bytes + exch ? 16384 - (stage + b_bytes + exch) : 0;
    const size_t budget = 224 * 1024 - 1024;
    if (b_bytes + exch + tail + 2 * stage > budget)
        return fail(NS_ERR_UNSUPPORTED, "swiglu_gemm: K=%d with %d token rows does not fit shared memory", p.K, NT);
    int stages = (int)((budget - b_bytes - exch - tail) / stage);
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > p.n_chunks) stages = p.n_chunks;
    p.stages = stages;
    const size_t smem = (size_t)stages * stage + b_bytes + exch + tail + 1024;
    CUtensorMap w_main, w_one, x_map;
    int rc = make_map(&w_main, w, 2 * (int64_t)p.inter, p.K, p.base);
    if (rc != NS_OK) return rc;
    rc = make_map(&w_one, w, 2 * (int64_t)p.inter, p.K, 1);
    if (rc != NS_OK) return rc;
    rc = make_map(&x_map, x, p.M, p.K, NT);
    if (rc != NS_OK) return rc;
    static SmemOptIn optin;
    if (optin.needs(smem)) {
        cudaError_t e = cudaFuncSetAttribute(swiglu_umma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "swiglu_gemm: cannot reserve %zu bytes of shared memory: %s", smem,
                                          cudaGetErrorString(e));
        optin.done(smem);
    }
    cudaError_t e = launch_pdl(swiglu_umma_kernel<NT>, dim3((unsigned)grid), dim3(kRows), smem, st, w_main, w_one, x_map, p);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "swiglu_gemm: launch failed: %s", cudaGetErrorString(e));
    return NS_OK;
}

}  // namespace ug

}  // namespace ns

using namespace ns;

extern "C" int ns_swiglu_gemm(const void* x, const void* w_gate_up, void* out, int32_t M, int32_t inter, int32_t K,
                              void* stream) {
    NS_REQUIRE(M >= 0 && inter > 0 && K > 0, NS_ERR_INVALID_ARG, "swiglu_gemm: bad shape");
    if (M == 0) return NS_OK;
    NS_REQUIRE(x && w_gate_up && out, NS_ERR_INVALID_ARG, "swiglu_gemm: null pointer");
    NS_REQUIRE(M <= 64, NS_ERR_UNSUPPORTED, "swiglu_gemm: %d token rows > 64 (use the library GEMM for large batches)", M);
    NS_REQUIRE(K % 64 == 0, NS_ERR_UNSUPPORTED, "swiglu_gemm: K=%d must be a multiple of 64", K);
    NS_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_gate_up)) & 15) == 0, NS_ERR_INVALID_ARG,
               "swiglu_gemm: x / w must be 16-byte aligned");
    ug::Params p;
    p.out = (__nv_bfloat16*)out; p.M = M; p.inter = inter; p.K = K; p.n_chunks = K / 64; p.stages = 0;
    p.base = p.rem = p.region = 0; p.timeline = ug::g_timeline;
    cudaStream_t st = (cudaStream_t)stream;
    return M <= 32 ? ug::launch<32>(x, w_gate_up, p, st) : ug::launch<64>(x, w_gate_up, p, st);
}

// Debug hook (not part of the public header): clock64 stamps of CTA 0 go to `buf` (device memory, 64 slots).
#ifdef NS_DEBUG_HOOKS
extern "C" void ns_debug_umma_timeline(long long* buf) { ns::ug::g_timeline = buf; }
#endif

namespace ns {
// Device address of this file's error counter on the current device (resolved once per device; the first call on a
// device must come before any stream capture). Used by ns_collect_status.
int umma_gemm_error_counter(const unsigned int** out) {
    static const unsigned int* addr[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(NS_ERR_CUDA, "umma_gemm_error_counter: no current device");
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, ug::g_errors);
        if (e != cudaSuccess || p == nullptr) return fail(NS_ERR_CUDA, "umma_gemm_error_counter: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        addr[dev] = static_cast<const unsigned int*>(p);
    }
    *out = addr[dev];
    return NS_OK;
}
}  // namespace ns

extern "C" int ns_umma_gemm_errors(uint32_t* count) {
    NS_REQUIRE(count != nullptr, NS_ERR_INVALID_ARG, "umma_gemm_errors: null pointer");
    cudaError_t e = cudaMemcpyFromSymbol(count, ug::g_errors, sizeof(uint32_t));
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "umma_gemm_errors: %s", cudaGetErrorString(e));
    return NS_OK;
}

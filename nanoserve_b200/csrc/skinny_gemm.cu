// Weight-streaming GEMM for decode-sized batches (M <= 64 token rows) with the layer's token-wise ops fused in.
//
// At M <= 64 a transformer GEMM is a weight read: Y[M,N] = X[M,K] . W[N,K]^T moves N*K*2 bytes of weights and
// next to nothing else, so the kernel is built like the other HBM-bound kernels here, not like a tensor-core GEMM:
//   * a CTA owns 64 weight rows and a K-slice; rows arrive by TMA bulk copies (cp.async.bulk, one per row: the
//     k-slice of a row is one contiguous run) completing on mbarriers - one per warp for its own 16 weight rows, one
//     for the activations - so a CTA issues ~100 copy instructions instead of ~10,000 16-byte ones; rows are padded
//     by 16 bytes in shared memory so ldmatrix is conflict-free without a swizzle. The plain GEMM (no prologue, bias
//     epilogue: down_proj) fetches its WEIGHTS by tiled TMA loads instead - boxes of 64 rows x 32 columns from a tensor
//     map over W, 64-byte swizzle, 19 instructions for a 608-column slice where the per-row copies were 64: issuing the
//     copies was 1.4 us of the kernel's 5.7;
//   * 4 warps x (16 weight rows x all token rows) of mma.sync m16n8k16 bf16 -> fp32;
//   * narrow-N GEMMs (o_proj, down_proj, QKV) are split over K across a thread-block cluster; the partial tiles are
//     pushed into the shared memory of the rank that finishes the row and summed there in rank order (deterministic,
//     no atomics, no second kernel, one cluster barrier between the last mma and the epilogue);
//   * prologue (optional): r = residual + a rounded to bf16, X = ln_w * bf16(r * rsqrt(mean(r^2) + eps)) computed on
//     the fly (replaces a separate add+RMSNorm kernel; r is stored once for the residual stream);
//   * epilogue: bias; or SiLU(gate)*up (the CTA's 64 weight rows are 32 gate rows + the matching 32 up rows); or
//     RoPE + paged KV write (one CTA tile = one 64-wide head of the merged QKV projection).
// Rounding points are those of the unfused ops: GEMM result (+bias) rounded to bf16 first, then every elementwise op
// rounded to bf16 as the framework would.
#include <cooperative_groups.h>
#include <cuda.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace ns {

__device__ unsigned int g_skinny_errors = 0;   // bulk copies that did not land within the bounded wait (never expected)


enum GemmEpilogue { kEpiBias = 0, kEpiSiluMul = 1, kEpiRopeKv = 2 };

struct GemmParams {
    const __nv_bfloat16* x;          // [M, K] activations (without prologue) or the pre-norm input `a`
    const __nv_bfloat16* residual;   // prologue: added to x before the norm (may be null: plain norm of x)
    const __nv_bfloat16* ln_w;       // prologue: RMSNorm weight [K]; null = no prologue
    __nv_bfloat16* residual_out;     // prologue: r = residual + x, [M, K] (may be null)
    const __nv_bfloat16* w;          // [N, K] row-major weights
    const __nv_bfloat16* bias;       // [N] or null
    __nv_bfloat16* out;              // kEpiBias: [M, N]; kEpiSiluMul: [M, inter]; kEpiRopeKv: q [M, n_heads*64]
    const __nv_bfloat16* cos;        // kEpiRopeKv: [M, 64]
    const __nv_bfloat16* sin;
    __nv_bfloat16* k_cache;          // kEpiRopeKv: one layer's pool, rows of n_kv_heads*64
    __nv_bfloat16* v_cache;
    const int64_t* slots;            // kEpiRopeKv: [M]
    int M, N, K, k_slice;            // k_slice = K / cluster size
    int inter;                       // kEpiSiluMul: columns of gate (= rows of W / 2)
    int n_heads, n_kv_heads;         // kEpiRopeKv
    float eps;
};

// ---- TMA bulk copy (1-D, no tensor map) completing on an mbarrier; every wait is bounded -----------------------
__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(mbar)
                 : "memory");
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
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

// Split cluster barrier: arrive early, wait where the guarantee is needed.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// One box [64 rows x 32 columns] of a row-major bf16 matrix into shared memory (4 KB, 64-byte swizzle); no multicast.
__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap* map, int col, int row, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(col), "r"(row), "r"(mbar)
                 : "memory");
}
constexpr int kBoxCols = 32;         // columns per weight box: 64 bytes, the span of the 64-byte swizzle

constexpr int kBN = 64;              // weight rows per CTA
constexpr int kGemmThreads = 128;

// WTMA: the weights arrive by tiled TMA loads into [k-slice / 32 boxes][64 rows][64 bytes], 64-byte swizzle (16-byte
// chunk c of row r sits at chunk c ^ ((r >> 1) & 3)), instead of one bulk copy per row into padded rows.
template <int MT, int EPI, bool WTMA>
__global__ void __launch_bounds__(kGemmThreads) skinny_gemm_kernel(const __grid_constant__ CUtensorMap w_map, const GemmParams p) {
    constexpr int MP = 16 * MT;                         // padded token rows
    extern __shared__ __align__(128) uint8_t smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();         // K-slice of this CTA
    const int csize = (int)cluster.num_blocks();
    const int tile = blockIdx.x;                        // which 64 weight rows
    const int k0 = rank * p.k_slice, ks = p.k_slice;
    const int a_stride = ks * 2 + 16;                   // bytes per activation row in shared memory (+16: no bank conflicts)
    uint8_t* a_sm = smem;
    uint8_t* w_sm = smem + (size_t)MP * a_stride;       // 4 warps x [16 weight rows][k-slice], rows padded like a_sm
    constexpr uint32_t W_ALIGN = WTMA ? 1024 : 128;
    w_sm += (W_ALIGN - (smem_u32(w_sm) & (W_ALIGN - 1))) & (W_ALIGN - 1);
    float* c_sm = reinterpret_cast<float*>(w_sm + (WTMA ? (size_t)kBN * ks * 2 : (size_t)kBN * a_stride));   // [csize][rows per rank][64] fp32

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // QKV only: the attention kernel that follows fetches its plan, block ids and older K/V rows while this GEMM runs.
    // (Not for the other epilogues: a successor that starts streaming ITS weights now would compete with this kernel's;
    // for down_proj, whose successor is the norm kernel, an early trigger measured the same at engine level.)
    if (EPI == kEpiRopeKv) pdl_launch_dependents();

    // weight row of the CTA's local row t
    auto w_row = [&](int t) -> int {
        if (EPI == kEpiSiluMul) return t < 32 ? tile * 32 + t : p.inter + tile * 32 + (t - 32);
        return tile * kBN + t;
    };
    // Loads: one TMA bulk copy per row (the k-slice of a row is one contiguous run), completing on mbarriers: one
    // barrier for the activations, one per warp for its own 16 weight rows. ~100 copy instructions per CTA.
    __shared__ __align__(8) uint64_t mbars[5];
    const uint32_t mb_a = smem_u32(&mbars[4]), mb_w = smem_u32(&mbars[WTMA ? 0 : warp]);
    const uint32_t row_bytes = (uint32_t)ks * 2;
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 5; ++i) mbar_init(smem_u32(&mbars[i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the byte counts are known now; every copy that completes on these barriers is issued after the barrier below
        if (WTMA) {
            mbar_expect_tx(smem_u32(&mbars[0]), (uint32_t)kBN * row_bytes);     // a box counts in full, rows past N arrive as zeros
        } else {
            for (int i = 0; i < 4; ++i) {
                int valid = 0;
                for (int r = 0; r < 16; ++r) valid += w_row(16 * i + r) < p.N;
                mbar_expect_tx(smem_u32(&mbars[i]), valid * row_bytes);
            }
        }
        if (p.ln_w == nullptr) mbar_expect_tx(mb_a, (uint32_t)p.M * row_bytes);
    }
    __syncthreads();
    cluster_arrive();                                   // "this CTA runs": peers wait for it before they store into c_sm
    const uint32_t my_w = smem_u32(w_sm) + (uint32_t)(16 * warp) * a_stride;
    if (WTMA) {
        if (tid == 0) {
            const uint32_t wb = smem_u32(w_sm);
            for (int j = 0; j < ks / kBoxCols; ++j) tma_load_box(wb + j * (kBN * kBoxCols * 2), &w_map, k0 + j * kBoxCols, tile * kBN, mb_w);
        }
    } else {
        // this warp's weight rows
        if (lane < 16) {
            const int wr = w_row(16 * warp + lane);
            if (wr < p.N) {
                bulk_g2s(my_w + lane * a_stride, p.w + (int64_t)wr * p.K + k0, row_bytes, mb_w);
            } else {
                for (uint32_t c = 0; c < row_bytes; c += 16)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(my_w + lane * a_stride + c), "r"(0) : "memory");
            }
        }
    }
    pdl_wait();        // everything above touched only weights; the activations come from the preceding kernel
    if (p.ln_w == nullptr && lane < 8) {
        // plain activations: bulk copies of the valid rows, spread over the four warps (a bulk copy costs its issuing
        // lane ~100 cycles, one lane after the other: 32 copies from one warp were 1 us on the critical path). Padding
        // rows stay unwritten: they only feed rows of the result that are never stored.
        const uint32_t ab = smem_u32(a_sm);
        for (int m = warp + 4 * lane; m < p.M; m += 32) bulk_g2s(ab + m * a_stride, p.x + (int64_t)m * p.K + k0, row_bytes, mb_a);
    }

    // ---- activations of this K-slice into shared memory --------------------------------------------------------
    if (p.ln_w != nullptr) {
        // r = residual + x (bf16), inv = rsqrt(mean(r^2) + eps) over the FULL row, X = ln_w * bf16(r * inv)
        for (int m = warp; m < MP; m += kGemmThreads / 32) {
            if (m < p.M) {
                const __nv_bfloat16* xr = p.x + (int64_t)m * p.K;
                const __nv_bfloat16* rr = p.residual ? p.residual + (int64_t)m * p.K : nullptr;
                float ss = 0.f;
                for (int c = lane; c < p.K / 8; c += 32) {
                    Vec16<__nv_bfloat16> v = load16(xr + c * 8);
                    if (rr) {
                        Vec16<__nv_bfloat16> r = load16(rr + c * 8);
#pragma unroll
                        for (int j = 0; j < 8; ++j) v.set(j, r.get(j) + v.get(j));
                        if (p.residual_out && tile == 0 && c * 8 >= k0 && c * 8 < k0 + ks)
                            store16(p.residual_out + (int64_t)m * p.K + c * 8, v);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) ss = fmaf(v.get(j), v.get(j), ss);
                }
                ss = warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss / (float)p.K + p.eps);
                for (int c = lane; c < ks / 8; c += 32) {
                    const int k = k0 + c * 8;
                    Vec16<__nv_bfloat16> v = load16(xr + k);
                    if (rr) {
                        Vec16<__nv_bfloat16> r = load16(rr + k);
#pragma unroll
                        for (int j = 0; j < 8; ++j) v.set(j, r.get(j) + v.get(j));
                    }
                    Vec16<__nv_bfloat16> wv = load16(p.ln_w + k);
                    Vec16<__nv_bfloat16> o;
#pragma unroll
                    for (int j = 0; j < 8; ++j) o.set(j, wv.get(j) * round_to<__nv_bfloat16>(v.get(j) * inv));
                    *reinterpret_cast<uint4*>(a_sm + (size_t)m * a_stride + c * 16) = o.raw;
                }
            } else {
                for (int c = lane; c < ks / 8; c += 32)
                    *reinterpret_cast<uint4*>(a_sm + (size_t)m * a_stride + c * 16) = make_uint4(0, 0, 0, 0);
            }
        }
    }

    // ---- main loop: warp w owns weight rows [16w, 16w+16) x all token rows ---------------------------------------
    float acc[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < 2; ++j) acc[mt][j][0] = acc[mt][j][1] = acc[mt][j][2] = acc[mt][j][3] = 0.f;
    const uint32_t a_base = smem_u32(a_sm);
    __syncthreads();                                     // prologue stores / zero rows visible to every warp
    bool landed = mbar_wait_bounded(mb_w, 0);
    if (p.ln_w == nullptr) landed = mbar_wait_bounded(mb_a, 0) && landed;
    if (!landed && lane == 0) atomicAdd(&g_skinny_errors, 1u);       // reported through ns_collect_status
    if (landed) {
        // fragments one k-step ahead of the mma that use them (ldmatrix -> mma back to back was ~100 cycles per k-step)
        struct Frag { uint32_t b[4]; uint32_t a[MT][4]; };
        const uint32_t b_addr = my_w + ((lane & 7) + ((lane >> 4) << 3)) * a_stride + (((lane >> 3) & 1) << 3) * 2;
        // WTMA: this lane's row of the CTA tile, its swizzle term and which 16-byte half of a k-step it fetches
        const uint32_t b_row = (uint32_t)(16 * warp + (lane & 7) + ((lane >> 4) << 3)), b_half = (lane >> 3) & 1;
        const uint32_t b_tma = smem_u32(w_sm) + b_row * (kBoxCols * 2), b_sw = (b_row >> 1) & 3;
        const uint32_t a_addr = a_base + ((lane & 7) + (((lane >> 3) & 1) << 3)) * a_stride + ((lane >> 4) << 3) * 2;
        auto load_frag = [&](Frag& f, int kk) {
            if (WTMA)
                ldmatrix_x4(b_tma + (uint32_t)(kk >> 1) * (kBN * kBoxCols * 2) + ((((uint32_t)(kk & 1) << 1 | b_half) ^ b_sw) << 4), f.b[0],
                            f.b[1], f.b[2], f.b[3]);
            else
                ldmatrix_x4(b_addr + kk * 32, f.b[0], f.b[1], f.b[2], f.b[3]);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(a_addr + 16 * mt * a_stride + kk * 32, f.a[mt][0], f.a[mt][1], f.a[mt][2], f.a[mt][3]);
        };
        auto compute = [&](const Frag& f) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_bf16_16816(acc[mt][0], f.a[mt], f.b[0], f.b[1]);
                mma_bf16_16816(acc[mt][1], f.a[mt], f.b[2], f.b[3]);
            }
        };
        const int ksteps = ks / 16;
        Frag f0, f1;
        load_frag(f0, 0);
        for (int kk = 0; kk < ksteps; kk += 2) {
            if (kk + 1 < ksteps) load_frag(f1, kk + 1);
            compute(f0);
            if (kk + 2 < ksteps) load_frag(f0, kk + 2);
            if (kk + 1 < ksteps) compute(f1);
        }
    }

    // ---- cluster reduction: every CTA pushes its partial rows into the shared memory of the rank that finishes them ----
    // Rank q finishes token rows q, q + csize, ...; its receive buffer is [csize senders][rows per rank][64] fp32. Stores
    // into a peer's shared memory are one-way, so the only cluster barrier on the critical path is the one between the
    // stores and the sums; the first barrier (every CTA of the cluster is running) was arrived at before the loads.
    const int rpr = (MP + csize - 1) / csize;           // receive rows per rank
    const bool pow2 = (csize & (csize - 1)) == 0;       // 1, 2, 4, 8: shifts instead of divisions
    const int cshift = __ffs(csize) - 1;
    cluster_wait();
    {
        const int r0 = lane >> 2, cp = (lane & 3) * 2;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int m = 16 * mt + r0 + 8 * half;
                if (m >= p.M) continue;
                const int owner = pow2 ? (m & (csize - 1)) : m % csize, slot = pow2 ? (m >> cshift) : m / csize;
                float* dst = cluster.map_shared_rank(c_sm, owner) + ((size_t)rank * rpr + slot) * kBN + 16 * warp + cp;
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    *reinterpret_cast<float2*>(dst + 8 * j) = make_float2(acc[mt][j][2 * half], acc[mt][j][2 * half + 1]);
            }
    }
    cluster_arrive();
    cluster_wait();
    // sum the partial rows in rank order (deterministic), then the epilogue
    for (int slot = warp; rank + slot * csize < p.M; slot += kGemmThreads / 32) {          // each warp one row at a time
        const int m = rank + slot * csize;
        float lo = 0.f, hi = 0.f;                       // columns lane and lane + 32 of the tile
#pragma unroll 8
        for (int r = 0; r < csize; ++r) {
            const float* part = c_sm + ((size_t)r * rpr + slot) * kBN;
            lo += part[lane];
            hi += part[lane + 32];
        }
        if (EPI == kEpiBias) {
            const int n_lo = tile * kBN + lane, n_hi = n_lo + 32;
            if (n_lo < p.N) p.out[(int64_t)m * p.N + n_lo] = __float2bfloat16_rn(lo + (p.bias ? __bfloat162float(p.bias[n_lo]) : 0.f));
            if (n_hi < p.N) p.out[(int64_t)m * p.N + n_hi] = __float2bfloat16_rn(hi + (p.bias ? __bfloat162float(p.bias[n_hi]) : 0.f));
        } else if (EPI == kEpiSiluMul) {
            const int n = tile * 32 + lane;
            if (n < p.inter) {
                const float g = round_to<__nv_bfloat16>(lo), u = round_to<__nv_bfloat16>(hi);
                const float sg = round_to<__nv_bfloat16>(g / (1.0f + expf(-g)));
                p.out[(int64_t)m * p.inter + n] = __float2bfloat16_rn(sg * u);
            }
        } else {
            // tile = one head of the merged QKV row: lane holds x_lo = col lane, x_hi = col lane + 32
            const int h = tile;
            float xl = lo, xh = hi;
            if (p.bias) {
                xl += __bfloat162float(p.bias[h * 64 + lane]);
                xh += __bfloat162float(p.bias[h * 64 + lane + 32]);
            }
            xl = round_to<__nv_bfloat16>(xl);
            xh = round_to<__nv_bfloat16>(xh);
            if (h < p.n_heads + p.n_kv_heads) {
                const float cl = __bfloat162float(p.cos[m * 64 + lane]), ch = __bfloat162float(p.cos[m * 64 + 32 + lane]);
                const float sl = __bfloat162float(p.sin[m * 64 + lane]), sh = __bfloat162float(p.sin[m * 64 + 32 + lane]);
                const float a = round_to<__nv_bfloat16>(__fmul_rn(xl, cl)), b = round_to<__nv_bfloat16>(__fmul_rn(xh, sl));
                const float d = round_to<__nv_bfloat16>(__fmul_rn(xh, ch)), e = round_to<__nv_bfloat16>(__fmul_rn(xl, sh));
                xl = round_to<__nv_bfloat16>(__fadd_rn(a, -b));
                xh = round_to<__nv_bfloat16>(__fadd_rn(d, e));
            }
            __nv_bfloat16* dst;
            if (h < p.n_heads) {
                dst = p.out + ((int64_t)m * p.n_heads + h) * 64;
            } else if (h < p.n_heads + p.n_kv_heads) {
                dst = p.k_cache + (p.slots[m] * p.n_kv_heads + (h - p.n_heads)) * 64;
            } else {
                dst = p.v_cache + (p.slots[m] * p.n_kv_heads + (h - p.n_heads - p.n_kv_heads)) * 64;
            }
            dst[lane] = __float2bfloat16_rn(xl);
            dst[lane + 32] = __float2bfloat16_rn(xh);
        }
    }
}

}  // namespace ns

namespace ns {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map over row-major bf16 weights [N, K] for boxes of 64 rows x 32 columns, 64-byte swizzle, zero fill past the
// matrix. Weights do not move: the last few maps are kept per thread, keyed by (pointer, N, K).
static const CUtensorMap* weight_map(const void* w, int N, int K) {
    struct Entry { const void* w; int N, K; CUtensorMap map; };
    static thread_local Entry cache[64];
    static thread_local int next = 0;
    for (Entry& e : cache)
        if (e.w == w && e.N == N && e.K == K) return &e.map;
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    Entry& e = cache[next];
    const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)N};
    const cuuint64_t gstride[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBoxCols, (cuuint32_t)kBN};
    const cuuint32_t estride[2] = {1, 1};
    if (fn(&e.map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
        e.w = nullptr;
        return nullptr;
    }
    e.w = w; e.N = N; e.K = K;
    next = (next + 1) % 64;
    return &e.map;
}

template <int MT, int EPI, bool WTMA>
static int launch_skinny_impl(const GemmParams& p, const CUtensorMap& w_map, int tiles, int split_k, cudaStream_t st) {
    const size_t smem = (size_t)(16 * MT + kBN) * (p.k_slice * 2 + 16) + (WTMA ? 1024 : 128) + (size_t)(16 * MT + 8) * kBN * 4;
    static SmemOptIn optin;
    if (optin.needs(smem)) {
        cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<MT, EPI, WTMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "skinny_gemm: cannot reserve %zu bytes of shared memory: %s", smem,
                                          cudaGetErrorString(e));
        optin.done(smem);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)tiles, (unsigned)split_k, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)split_k;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, skinny_gemm_kernel<MT, EPI, WTMA>, w_map, p);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "skinny_gemm: launch failed: %s", cudaGetErrorString(e));
    return NS_OK;
}

template <int MT, int EPI>
static int launch_skinny(const GemmParams& p, int tiles, int split_k, cudaStream_t st) {
    // the plain GEMM fetches its weights by tiled TMA loads where the K slice is whole boxes and the driver gives a map
    if (EPI == kEpiBias && p.ln_w == nullptr && p.k_slice % kBoxCols == 0 && (p.K * 2) % 16 == 0) {
        const CUtensorMap* map = weight_map(p.w, p.N, p.K);
        if (map != nullptr) return launch_skinny_impl<MT, EPI, EPI == kEpiBias>(p, *map, tiles, split_k, st);
    }
    static const CUtensorMap none = {};
    return launch_skinny_impl<MT, EPI, false>(p, none, tiles, split_k, st);
}

template <int EPI> static int dispatch_mt(const GemmParams& p, int tiles, int split_k, cudaStream_t st) {
    if (p.M <= 16) return launch_skinny<1, EPI>(p, tiles, split_k, st);
    if (p.M <= 32) return launch_skinny<2, EPI>(p, tiles, split_k, st);
    return launch_skinny<4, EPI>(p, tiles, split_k, st);
}

// Device address of this file's error counter on the current device (resolved once per device; the first call on a
// device must come before any stream capture). Used by ns_collect_status.
int skinny_gemm_error_counter(const unsigned int** out) {
    static const unsigned int* addr[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(NS_ERR_CUDA, "skinny_gemm_error_counter: no current device");
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_skinny_errors);
        if (e != cudaSuccess || p == nullptr) return fail(NS_ERR_CUDA, "skinny_gemm_error_counter: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        addr[dev] = static_cast<const unsigned int*>(p);
    }
    *out = addr[dev];
    return NS_OK;
}

}  // namespace ns

using namespace ns;

extern "C" int ns_skinny_gemm(const void* x, const void* residual, const void* ln_w, void* residual_out, const void* w,
                              const void* bias, void* out, int32_t M, int32_t N, int32_t K, int32_t split_k, float eps,
                              int32_t epilogue, int32_t inter, const void* cos, const void* sin, void* k_cache,
                              void* v_cache, const int64_t* slots, int32_t n_heads, int32_t n_kv_heads, void* stream) {
    NS_REQUIRE(M >= 0 && N > 0 && K > 0, NS_ERR_INVALID_ARG, "skinny_gemm: bad shape");
    if (M == 0) return NS_OK;
    NS_REQUIRE(x && w && out, NS_ERR_INVALID_ARG, "skinny_gemm: null pointer");
    NS_REQUIRE(M <= 64, NS_ERR_UNSUPPORTED, "skinny_gemm: %d token rows > 64 (use the library GEMM for large batches)", M);
    NS_REQUIRE(split_k >= 1 && split_k <= 8, NS_ERR_INVALID_ARG, "skinny_gemm: split_k must be between 1 and 8");
    NS_REQUIRE(K % (16 * split_k) == 0, NS_ERR_UNSUPPORTED, "skinny_gemm: K=%d is not a multiple of 16*split_k", K);
    NS_REQUIRE(residual == nullptr || ln_w != nullptr, NS_ERR_INVALID_ARG, "skinny_gemm: residual needs the norm prologue");
    NS_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0, NS_ERR_INVALID_ARG,
               "skinny_gemm: x / w must be 16-byte aligned");
    GemmParams p;
    p.x = (const __nv_bfloat16*)x; p.residual = (const __nv_bfloat16*)residual; p.ln_w = (const __nv_bfloat16*)ln_w;
    p.residual_out = (__nv_bfloat16*)residual_out; p.w = (const __nv_bfloat16*)w; p.bias = (const __nv_bfloat16*)bias;
    p.out = (__nv_bfloat16*)out; p.cos = (const __nv_bfloat16*)cos; p.sin = (const __nv_bfloat16*)sin;
    p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache; p.slots = slots;
    p.M = M; p.N = N; p.K = K; p.k_slice = K / split_k; p.inter = inter; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads;
    p.eps = eps;
    const int mp = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    const size_t a_bytes = (size_t)(mp + kBN) * (p.k_slice * 2 + 16);
    // (what launch_skinny_impl reserves: both tiles in padded rows, the alignment slack of the TMA form, the receive buffer;
    // 227 KB is a CTA's limit and the kernel's static shared memory is a few barriers)
    NS_REQUIRE(a_bytes + (size_t)(mp + 8) * kBN * 4 + 1024 <= 226 * 1024, NS_ERR_UNSUPPORTED,
               "skinny_gemm: K slice of %d does not fit shared memory (raise split_k)", p.k_slice);
    cudaStream_t st = (cudaStream_t)stream;
    if (epilogue == kEpiBias) return dispatch_mt<kEpiBias>(p, (N + kBN - 1) / kBN, split_k, st);
    if (epilogue == kEpiSiluMul) {
        NS_REQUIRE(inter > 0 && N == 2 * inter && inter % 32 == 0 && bias == nullptr, NS_ERR_INVALID_ARG,
                   "skinny_gemm: SiLU*mul wants W = [gate; up] with 2*inter rows, inter a multiple of 32, no bias");
        return dispatch_mt<kEpiSiluMul>(p, inter / 32, split_k, st);
    }
    if (epilogue == kEpiRopeKv) {
        NS_REQUIRE(n_heads > 0 && n_kv_heads > 0 && N == (n_heads + 2 * n_kv_heads) * 64, NS_ERR_UNSUPPORTED,
                   "skinny_gemm: the RoPE + KV-write epilogue handles head_dim 64 only");
        NS_REQUIRE(cos && sin && k_cache && v_cache && slots, NS_ERR_INVALID_ARG, "skinny_gemm: RoPE epilogue needs cos, sin, caches, slots");
        return dispatch_mt<kEpiRopeKv>(p, n_heads + 2 * n_kv_heads, split_k, st);
    }
    return fail(NS_ERR_INVALID_ARG, "skinny_gemm: unknown epilogue %d", epilogue);
}

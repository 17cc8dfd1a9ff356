// Narrow decode-sized GEMMs (QKV, o_proj: K = hidden size) without any split over K across CTAs.
//
// Y[M <= 64, N] = X[M, K] . W[N, K]^T. A CTA owns EIGHT weight rows over the whole of K (one mma n-tile), so a GEMM
// with N = 896..1152 is 112..144 CTAs: about one per SM. The four warps split K between them and each warp fetches
// only ITS quarter of the weight rows (before the dependency wait, so they stream while the preceding kernel runs)
// and of the activation rows (after the wait; every CTA reads all of X: 57 KB at 32 rows, from L2) with 16-byte
// cp.async copies into padded rows, waits for its own copies only, keeps its partial 16x8 tiles in registers (two
// independent accumulator sets per m-tile) and meets the other warps once in shared memory: no mbarrier, no
// thread-block cluster, no distributed shared memory, no barrier but one __syncthreads.
//
// Why: cycle stamps of the 64-row-tile, 8-way split-K kernel in skinny_gemm.cu inside a decode layer showed where its
// 4.8 us after the wait go: ~1.0 us issuing 32 activation bulk copies from one warp (a bulk copy costs its issuing
// lane 60-140 cycles, one after the other), 0.6 us in 7 dependent k-steps, 0.55 us pushing partial tiles to peer CTAs,
// 0.7 us in the cluster barrier, 1.5 us in the RoPE epilogue behind its loads. This kernel needs ~1.2 us after the wait.
//
// Epilogues: bias (optional); or RoPE + paged KV write for a merged QKV projection with 64-wide heads: the CTA's
// eight rows are then four rows of a head's first half and the matching four of its second half, so every rotation
// pair (i, i + 32) is finished by one thread. Rounding points are those of the unfused ops.
#include "common.cuh"

namespace ns {
namespace {

enum ThinEpilogue { kThinBias = 0, kThinRopeKv = 2 };

struct ThinParams {
    const __nv_bfloat16* x;          // [M, K]
    const __nv_bfloat16* w;          // [N, K]
    const __nv_bfloat16* bias;       // [N] or null
    __nv_bfloat16* out;              // kThinBias: [M, N]; kThinRopeKv: q [M, n_heads * 64]
    const __nv_bfloat16* cos;        // kThinRopeKv: [M, 64]
    const __nv_bfloat16* sin;
    __nv_bfloat16* k_cache;          // kThinRopeKv: one layer's pool, rows of n_kv_heads * 64
    __nv_bfloat16* v_cache;
    const int64_t* slots;            // kThinRopeKv: [M]
    int M, N, K;
    int n_heads, n_kv_heads;
};

constexpr int kThinThreads = 128;
constexpr int kThinRows = 8;          // weight rows per CTA

template <int MT, int EPI>
__global__ void __launch_bounds__(kThinThreads) thin_gemm_kernel(const ThinParams p) {
    constexpr int MP = 16 * MT;                          // padded token rows
    constexpr int PASSES = MT >= 2 ? MT / 2 : 1;         // epilogue: MP * 4 (row, column pair) items over 128 threads
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x;
    const uint32_t pitch = (uint32_t)p.K * 2 + 16;       // bytes per row in shared memory (+16: ldmatrix without conflicts)
    const uint32_t w_sm = smem_u32(smem);                // [8][pitch]
    const uint32_t x_sm = w_sm + kThinRows * pitch;      // [MP][pitch] (rows >= M stay unwritten: they only feed rows
                                                         // of the result that are never stored)
    float* c_sm = reinterpret_cast<float*>(smem + (size_t)(kThinRows + MP) * pitch);      // [4 warps][MP][8] fp32

    pdl_launch_dependents();
    // weight row of the CTA's local row t
    int head = 0, sub = 0;
    if (EPI == kThinRopeKv) { head = tile >> 3; sub = tile & 7; }
    auto w_row = [&](int t) -> int {
        if (EPI == kThinRopeKv) return head * 64 + (t < 4 ? 0 : 32) + sub * 4 + (t & 3);
        return tile * kThinRows + t;
    };
    const int qchunks = p.K / 32;                         // 16-byte chunks in a warp's quarter of a row
    const uint32_t kbase = (uint32_t)warp * (uint32_t)(p.K / 4) * 2;      // byte offset of this warp's K range in a row
    // this warp's quarter of the eight weight rows: lane = chunk column, one copy per row
    for (int cc = lane; cc < qchunks; cc += 32) {
#pragma unroll
        for (int t = 0; t < kThinRows; ++t)
            cp_async16(w_sm + t * pitch + kbase + cc * 16, reinterpret_cast<const uint8_t*>(p.w + (int64_t)w_row(t) * p.K) + kbase + cc * 16, 16);
    }
    cp_async_commit();
    pdl_wait();        // everything above touched only weights; the activations come from the preceding kernel
    for (int cc = lane; cc < qchunks; cc += 32) {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.x) + kbase + cc * 16;
        const uint32_t dst = x_sm + kbase + cc * 16;
#pragma unroll 8
        for (int m = 0; m < p.M; ++m) cp_async16(dst + m * pitch, src + (size_t)m * p.K * 2, 16);
    }
    cp_async_commit();

    // ---- epilogue inputs into registers while the activations are on their way -------------------------------------
    // (raw bf16 values: converting here would make the warp wait for the loads before it reaches the k-loop)
    __nv_bfloat16 e_bias[PASSES][2], e_cos[PASSES][2], e_sin[PASSES][2];
    int64_t e_slot[PASSES];
#pragma unroll
    for (int ps = 0; ps < PASSES; ++ps) {
        const int idx = tid + ps * kThinThreads, row = idx >> 2, j = idx & 3;
        e_bias[ps][0] = e_bias[ps][1] = __float2bfloat16_rn(0.f);
        e_cos[ps][0] = e_cos[ps][1] = __float2bfloat16_rn(1.f);
        e_sin[ps][0] = e_sin[ps][1] = __float2bfloat16_rn(0.f);
        e_slot[ps] = 0;
        if (row >= p.M || idx >= MP * 4) continue;
        if (EPI == kThinBias) {
            if (p.bias) {
                e_bias[ps][0] = p.bias[tile * kThinRows + 2 * j];
                e_bias[ps][1] = p.bias[tile * kThinRows + 2 * j + 1];
            }
        } else {
            const int d = sub * 4 + j;                    // rotation pair (d, d + 32) of the head
            if (p.bias) {
                e_bias[ps][0] = p.bias[head * 64 + d];
                e_bias[ps][1] = p.bias[head * 64 + 32 + d];
            }
            if (head < p.n_heads + p.n_kv_heads) {
                e_cos[ps][0] = p.cos[row * 64 + d];
                e_cos[ps][1] = p.cos[row * 64 + 32 + d];
                e_sin[ps][0] = p.sin[row * 64 + d];
                e_sin[ps][1] = p.sin[row * 64 + 32 + d];
            }
            if (head >= p.n_heads) e_slot[ps] = p.slots[row];
        }
    }

    // ---- main loop: warp w owns K / 4 of every row; two k-steps (32 columns) per iteration, fragments one iteration
    // ahead; the two k-steps of an iteration accumulate into separate sets so four mma chains run side by side
    float acc[2][MT][4];
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) acc[s][mt][0] = acc[s][mt][1] = acc[s][mt][2] = acc[s][mt][3] = 0.f;
    const int iters = p.K / 128;                          // per warp
    // B: one ldmatrix.x4 = rows 0..7 x columns [0,8) [8,16) [16,24) [24,32) of the iteration
    const uint32_t b_addr = w_sm + (lane & 7) * pitch + kbase + (lane >> 3) * 16;
    // A: per m-tile and k-step one ldmatrix.x4 (rows 0..7 / 8..15 x columns [0,8) / [8,16))
    const uint32_t a_addr = x_sm + ((lane & 7) + (((lane >> 3) & 1) << 3)) * pitch + kbase + (lane >> 4) * 16;
    struct Frag { uint32_t b[4]; uint32_t a[2][MT][4]; };
    auto load_frag = [&](Frag& f, int it) {
        ldmatrix_x4(b_addr + it * 64, f.b[0], f.b[1], f.b[2], f.b[3]);
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                ldmatrix_x4(a_addr + 16 * mt * pitch + it * 64 + s * 32, f.a[s][mt][0], f.a[s][mt][1], f.a[s][mt][2], f.a[s][mt][3]);
    };
    auto compute = [&](const Frag& f) {
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) mma_bf16_16816(acc[s][mt], f.a[s][mt], f.b[2 * s], f.b[2 * s + 1]);
    };
    cp_async_wait<0>();                                   // this warp's own copies: nobody else reads them
    __syncwarp();
    {
        Frag f0, f1;
        load_frag(f0, 0);
        for (int it = 0; it < iters; it += 2) {
            if (it + 1 < iters) load_frag(f1, it + 1);
            compute(f0);
            if (it + 2 < iters) load_frag(f0, it + 2);
            if (it + 1 < iters) compute(f1);
        }
    }

    // ---- the four warps' partial tiles meet in shared memory -----------------------------------------------------
    {
        const int r0 = lane >> 2, cp = (lane & 3) * 2;
        float* mine = c_sm + (size_t)warp * MP * 8;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            *reinterpret_cast<float2*>(mine + (16 * mt + r0) * 8 + cp) =
                make_float2(acc[0][mt][0] + acc[1][mt][0], acc[0][mt][1] + acc[1][mt][1]);
            *reinterpret_cast<float2*>(mine + (16 * mt + r0 + 8) * 8 + cp) =
                make_float2(acc[0][mt][2] + acc[1][mt][2], acc[0][mt][3] + acc[1][mt][3]);
        }
    }
    __syncthreads();
#pragma unroll
    for (int ps = 0; ps < PASSES; ++ps) {
        const int idx = tid + ps * kThinThreads, row = idx >> 2, j = idx & 3;
        if (row >= p.M || idx >= MP * 4) continue;
        if (EPI == kThinBias) {
            float lo = 0.f, hi = 0.f;                     // columns 2j, 2j + 1 of the tile, summed in warp order
#pragma unroll
            for (int wv = 0; wv < 4; ++wv) {
                const float2 v = *reinterpret_cast<const float2*>(c_sm + ((size_t)wv * MP + row) * 8 + 2 * j);
                lo += v.x;
                hi += v.y;
            }
            const uint32_t packed = pack_bf16x2(lo + __bfloat162float(e_bias[ps][0]), hi + __bfloat162float(e_bias[ps][1]));
            *reinterpret_cast<uint32_t*>(p.out + (int64_t)row * p.N + tile * kThinRows + 2 * j) = packed;
        } else {
            float xl = 0.f, xh = 0.f;                     // columns j (first half) and j + 4 (second half) of the tile
#pragma unroll
            for (int wv = 0; wv < 4; ++wv) {
                xl += c_sm[((size_t)wv * MP + row) * 8 + j];
                xh += c_sm[((size_t)wv * MP + row) * 8 + 4 + j];
            }
            xl = round_to<__nv_bfloat16>(xl + __bfloat162float(e_bias[ps][0]));
            xh = round_to<__nv_bfloat16>(xh + __bfloat162float(e_bias[ps][1]));
            if (head < p.n_heads + p.n_kv_heads) {
                const float cl = __bfloat162float(e_cos[ps][0]), ch = __bfloat162float(e_cos[ps][1]);
                const float sl = __bfloat162float(e_sin[ps][0]), sh = __bfloat162float(e_sin[ps][1]);
                const float a = round_to<__nv_bfloat16>(__fmul_rn(xl, cl)), b = round_to<__nv_bfloat16>(__fmul_rn(xh, sl));
                const float d = round_to<__nv_bfloat16>(__fmul_rn(xh, ch)), e = round_to<__nv_bfloat16>(__fmul_rn(xl, sh));
                xl = round_to<__nv_bfloat16>(__fadd_rn(a, -b));
                xh = round_to<__nv_bfloat16>(__fadd_rn(d, e));
            }
            __nv_bfloat16* dst;
            if (head < p.n_heads) {
                dst = p.out + ((int64_t)row * p.n_heads + head) * 64;
            } else if (head < p.n_heads + p.n_kv_heads) {
                dst = p.k_cache + (e_slot[ps] * p.n_kv_heads + (head - p.n_heads)) * 64;
            } else {
                dst = p.v_cache + (e_slot[ps] * p.n_kv_heads + (head - p.n_heads - p.n_kv_heads)) * 64;
            }
            const int d = sub * 4 + j;
            dst[d] = __float2bfloat16_rn(xl);
            dst[d + 32] = __float2bfloat16_rn(xh);
        }
    }
}

template <int MT, int EPI>
int launch_thin(const ThinParams& p, int tiles, cudaStream_t st) {
    const size_t smem = (size_t)(kThinRows + 16 * MT) * ((size_t)p.K * 2 + 16) + (size_t)4 * 16 * MT * 8 * 4;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(thin_gemm_kernel<MT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "thin_gemm: cannot reserve %zu bytes of shared memory: %s", smem,
                                          cudaGetErrorString(e));
        configured = smem;
    }
    cudaError_t e = launch_pdl(thin_gemm_kernel<MT, EPI>, dim3((unsigned)tiles), dim3(kThinThreads), smem, st, p);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "thin_gemm: launch failed: %s", cudaGetErrorString(e));
    return NS_OK;
}

template <int EPI> int dispatch_thin(const ThinParams& p, int tiles, cudaStream_t st) {
    if (p.M <= 16) return launch_thin<1, EPI>(p, tiles, st);
    if (p.M <= 32) return launch_thin<2, EPI>(p, tiles, st);
    return launch_thin<4, EPI>(p, tiles, st);
}

}  // namespace
}  // namespace ns

using namespace ns;

extern "C" int ns_thin_gemm(const void* x, const void* w, const void* bias, void* out, int32_t M, int32_t N, int32_t K,
                            int32_t epilogue, const void* cos, const void* sin, void* k_cache, void* v_cache,
                            const int64_t* slots, int32_t n_heads, int32_t n_kv_heads, void* stream) {
    NS_REQUIRE(M >= 0 && N > 0 && K > 0, NS_ERR_INVALID_ARG, "thin_gemm: bad shape");
    if (M == 0) return NS_OK;
    NS_REQUIRE(x && w && out, NS_ERR_INVALID_ARG, "thin_gemm: null pointer");
    NS_REQUIRE(M <= 64, NS_ERR_UNSUPPORTED, "thin_gemm: %d token rows > 64 (use the library GEMM for large batches)", M);
    NS_REQUIRE(K % 128 == 0 && N % 8 == 0, NS_ERR_UNSUPPORTED, "thin_gemm: K=%d must be a multiple of 128 and N=%d of 8", K, N);
    NS_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 3) == 0,
               NS_ERR_INVALID_ARG, "thin_gemm: x / w must be 16-byte aligned, out 4-byte aligned");
    const int mp = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    NS_REQUIRE((size_t)(kThinRows + mp) * ((size_t)K * 2 + 16) + (size_t)4 * mp * 8 * 4 <= 220 * 1024, NS_ERR_UNSUPPORTED,
               "thin_gemm: %d rows of K=%d do not fit shared memory", mp, K);
    ThinParams p;
    p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.bias = (const __nv_bfloat16*)bias;
    p.out = (__nv_bfloat16*)out; p.cos = (const __nv_bfloat16*)cos; p.sin = (const __nv_bfloat16*)sin;
    p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache; p.slots = slots;
    p.M = M; p.N = N; p.K = K; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads;
    cudaStream_t st = (cudaStream_t)stream;
    if (epilogue == kThinBias) return dispatch_thin<kThinBias>(p, N / kThinRows, st);
    if (epilogue == kThinRopeKv) {
        NS_REQUIRE(n_heads > 0 && n_kv_heads > 0 && N == (n_heads + 2 * n_kv_heads) * 64, NS_ERR_UNSUPPORTED,
                   "thin_gemm: the RoPE + KV-write epilogue handles head_dim 64 only");
        NS_REQUIRE(cos && sin && k_cache && v_cache && slots, NS_ERR_INVALID_ARG, "thin_gemm: RoPE epilogue needs cos, sin, caches, slots");
        return dispatch_thin<kThinRopeKv>(p, N / kThinRows, st);
    }
    return fail(NS_ERR_INVALID_ARG, "thin_gemm: unknown epilogue %d (0 = bias, 2 = RoPE + KV write)", epilogue);
}

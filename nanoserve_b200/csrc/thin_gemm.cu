// Narrow decode-sized GEMMs (QKV, o_proj: K = hidden size) without any split over K across CTAs.
//
// Y[M <= 64, N] = X[M, K] . W[N, K]^T. A CTA owns EIGHT weight rows over the whole of K (one mma n-tile; sixteen where
// eight would be more than one wave of CTAs), so a GEMM with N = 896..1152 is 112..144 CTAs: about one per SM. The four
// warps split K between them. Each warp fetches its quarter of the weight rows with 16-byte cp.async copies before the
// dependency wait (they stream while the preceding kernel runs) and waits for its own copies only; after the wait all
// M activation rows arrive by bulk copies on one mbarrier (every CTA reads all of X: 57 KB at 32 rows, from L2). Every
// warp keeps its partial 16x8 tiles in registers (two independent accumulator sets per m-tile) and meets the others
// once in shared memory: no thread-block cluster, no distributed shared memory, one __syncthreads after the k-loop.
//
// Why: cycle stamps of the 64-row-tile, 8-way split-K kernel in skinny_gemm.cu inside a decode layer showed where its
// 4.8 us after the wait go: ~1.0 us issuing 32 activation bulk copies from one warp, 0.6 us in 7 dependent k-steps,
// 0.55 us pushing partial tiles to peer CTAs, 0.7 us in the cluster barrier, 1.5 us in the RoPE epilogue behind its
// loads. This kernel needs 2.3 us after the wait for QKV and 1.5 us for o_proj.
//
// Epilogues: bias (optional); or RoPE + paged KV write for a merged QKV projection with 64- or 128-wide heads: an
// n-tile is then four rows of a head's first half and the matching four of its second half, so every rotation pair
// (i, i + head_dim / 2) is finished by one thread. Rounding points are those of the unfused ops.
#include "common.cuh"

namespace ns {
namespace {

enum ThinEpilogue { kThinBias = 0, kThinRopeKv = 2, kThinResidual = 3 };

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
    const __nv_bfloat16* residual;   // kThinResidual: [M, N], added to the product; out = the new residual stream
    float* ss_out;                   // kThinResidual: [M, N / 8] sums of squares of out's 8-column pieces
    int M, N, K;
    int n_heads, n_kv_heads, head_dim;
};

__device__ unsigned int g_thin_errors = 0;   // bulk copies that did not land within the bounded wait (never expected)

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

constexpr int kThinThreads = 128;
constexpr int kThinRows = 8;          // weight rows per CTA

template <int MT, int NT, int EPI>
__global__ void __launch_bounds__(kThinThreads) thin_gemm_kernel(const ThinParams p) {
    constexpr int MP = 16 * MT;                          // padded token rows
    constexpr int R = kThinRows * NT;                    // weight rows per CTA: NT mma n-tiles
    constexpr int ITEMS = MP * 4 * NT;                   // epilogue items (n-tile, token row, column pair)
    constexpr int PASSES = (ITEMS + kThinThreads - 1) / kThinThreads;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x;
    const uint32_t pitch = (uint32_t)p.K * 2 + 16;       // bytes per row in shared memory (+16: ldmatrix without conflicts)
    const uint32_t w_sm = smem_u32(smem);                // [R][pitch]
    const uint32_t x_sm = w_sm + R * pitch;              // [MP][pitch] (rows >= M stay unwritten: they only feed rows
                                                         // of the result that are never stored)
    float* c_sm = reinterpret_cast<float*>(smem + (size_t)(R + MP) * pitch);      // [4 warps][NT][MP][8] fp32

    pdl_launch_dependents();
    // X arrives by bulk copies (one per token row, issued after the dependency wait, eight per warp at 32 rows) on this
    // barrier. 16-byte cp.async copies of X (every warp its own K quarter, no barrier at all) were measured slower: the
    // load/store pipe moves ~36 bytes per clock per SM for cp.async, so 57 KB of X took 0.8 us longer than the bulk copies.
    __shared__ __align__(8) uint64_t x_bar;
    const uint32_t mb_x = smem_u32(&x_bar);
    if (tid == 0) {
        mbar_init(mb_x, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(mb_x, (uint32_t)p.M * (uint32_t)p.K * 2);
    }
    __syncthreads();
    // RoPE epilogue: n-tile g = tile * NT + nt is rows [4 sub, 4 sub + 4) of a head's first half + the matching four of
    // its second half; a head has head_dim / 8 such tiles
    const int half = p.head_dim >> 1, per_head = p.head_dim >> 3;
    auto w_row = [&](int t) -> int {                     // weight row of the CTA's local row t
        if (EPI == kThinRopeKv) {
            const int g = tile * NT + (t >> 3), head = g / per_head, sub = g - head * per_head;
            return head * p.head_dim + ((t & 4) ? half : 0) + sub * 4 + (t & 3);
        }
        return tile * R + t;
    };
    const int qchunks = p.K / 32;                         // 16-byte chunks in a warp's quarter of a row
    const uint32_t kbase = (uint32_t)warp * (uint32_t)(p.K / 4) * 2;      // byte offset of this warp's K range in a row
    // this warp's quarter of the weight rows: lane = chunk column, one copy per row
    for (int cc = lane; cc < qchunks; cc += 32) {
#pragma unroll
        for (int t = 0; t < R; ++t)
            cp_async16(w_sm + t * pitch + kbase + cc * 16, reinterpret_cast<const uint8_t*>(p.w + (int64_t)w_row(t) * p.K) + kbase + cc * 16, 16);
    }
    cp_async_commit();
    pdl_wait();        // everything above touched only weights; the activations come from the preceding kernel
    if (lane < 8) {
        for (int m = warp + 4 * lane; m < p.M; m += 32) bulk_g2s(x_sm + m * pitch, p.x + (int64_t)m * p.K, (uint32_t)p.K * 2, mb_x);
    }

    // ---- epilogue inputs into registers while the activations are on their way -------------------------------------
    // (raw bf16 values: converting here would make the warp wait for the loads before it reaches the k-loop)
    __nv_bfloat16 e_bias[PASSES][2], e_cos[PASSES][2], e_sin[PASSES][2];
    int64_t e_slot[PASSES];
#pragma unroll
    for (int ps = 0; ps < PASSES; ++ps) {
        const int idx = tid + ps * kThinThreads, j = idx & 3, row = (idx >> 2) & (MP - 1), nt = idx / (4 * MP);
        e_bias[ps][0] = e_bias[ps][1] = __float2bfloat16_rn(0.f);
        e_cos[ps][0] = e_cos[ps][1] = __float2bfloat16_rn(1.f);
        e_sin[ps][0] = e_sin[ps][1] = __float2bfloat16_rn(0.f);
        e_slot[ps] = 0;
        if (row >= p.M || idx >= ITEMS) continue;
        if (EPI == kThinBias) {
            if (p.bias) {
                e_bias[ps][0] = p.bias[tile * R + nt * 8 + 2 * j];
                e_bias[ps][1] = p.bias[tile * R + nt * 8 + 2 * j + 1];
            }
        } else if (EPI == kThinResidual) {
            e_bias[ps][0] = p.residual[(int64_t)row * p.N + tile * R + nt * 8 + 2 * j];
            e_bias[ps][1] = p.residual[(int64_t)row * p.N + tile * R + nt * 8 + 2 * j + 1];
        } else {
            const int g = tile * NT + nt, head = g / per_head, d = (g - head * per_head) * 4 + j;   // rotation pair (d, d + half)
            if (p.bias) {
                e_bias[ps][0] = p.bias[head * p.head_dim + d];
                e_bias[ps][1] = p.bias[head * p.head_dim + half + d];
            }
            if (head < p.n_heads + p.n_kv_heads) {
                e_cos[ps][0] = p.cos[row * p.head_dim + d];
                e_cos[ps][1] = p.cos[row * p.head_dim + half + d];
                e_sin[ps][0] = p.sin[row * p.head_dim + d];
                e_sin[ps][1] = p.sin[row * p.head_dim + half + d];
            }
            if (head >= p.n_heads) e_slot[ps] = p.slots[row];
        }
    }

    // ---- main loop: warp w owns K / 4 of every row; two k-steps (32 columns) per iteration, fragments one iteration
    // ahead; the two k-steps of an iteration accumulate into separate sets so the mma chains run side by side
    float acc[2][MT][NT][4];
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) acc[s][mt][nt][0] = acc[s][mt][nt][1] = acc[s][mt][nt][2] = acc[s][mt][nt][3] = 0.f;
    const int iters = p.K / 128;                          // per warp
    // B: per n-tile one ldmatrix.x4 = rows 0..7 x columns [0,8) [8,16) [16,24) [24,32) of the iteration
    const uint32_t b_addr = w_sm + (lane & 7) * pitch + kbase + (lane >> 3) * 16;
    // A: per m-tile and k-step one ldmatrix.x4 (rows 0..7 / 8..15 x columns [0,8) / [8,16))
    const uint32_t a_addr = x_sm + ((lane & 7) + (((lane >> 3) & 1) << 3)) * pitch + kbase + (lane >> 4) * 16;
    struct Frag { uint32_t b[NT][4]; uint32_t a[2][MT][4]; };
    auto load_frag = [&](Frag& f, int it) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) ldmatrix_x4(b_addr + nt * 8 * pitch + it * 64, f.b[nt][0], f.b[nt][1], f.b[nt][2], f.b[nt][3]);
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
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(acc[s][mt][nt], f.a[s][mt], f.b[nt][2 * s], f.b[nt][2 * s + 1]);
    };
    cp_async_wait<0>();                                   // this warp's own weight copies: nobody else reads them
    __syncwarp();
    if (!mbar_wait_bounded(mb_x, 0) && lane == 0) atomicAdd(&g_thin_errors, 1u);
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
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float* mine = c_sm + (size_t)(warp * NT + nt) * MP * 8;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                *reinterpret_cast<float2*>(mine + (16 * mt + r0) * 8 + cp) =
                    make_float2(acc[0][mt][nt][0] + acc[1][mt][nt][0], acc[0][mt][nt][1] + acc[1][mt][nt][1]);
                *reinterpret_cast<float2*>(mine + (16 * mt + r0 + 8) * 8 + cp) =
                    make_float2(acc[0][mt][nt][2] + acc[1][mt][nt][2], acc[0][mt][nt][3] + acc[1][mt][nt][3]);
            }
        }
    }
    __syncthreads();
    if (EPI == kThinResidual) {
        // new residual = bf16(residual + bf16(x . w^T)), stored where the next layer piece reads it, plus the sum of its
        // squares over this n-tile's eight columns: the consumer's RMSNorm adds the N / 8 pieces of a row instead of
        // re-reading the row (the four lanes of a (row, n-tile) item meet by shuffles, so no lane leaves early)
#pragma unroll
        for (int ps = 0; ps < PASSES; ++ps) {
            const int idx = tid + ps * kThinThreads, j = idx & 3, row = (idx >> 2) & (MP - 1), nt = idx / (4 * MP);
            const bool valid = row < p.M && idx < ITEMS;
            float lo = 0.f, hi = 0.f;
            if (idx < ITEMS) {
#pragma unroll
                for (int wv = 0; wv < 4; ++wv) {
                    const float2 v = *reinterpret_cast<const float2*>(c_sm + ((size_t)(wv * NT + nt) * MP + row) * 8 + 2 * j);
                    lo += v.x;
                    hi += v.y;
                }
            }
            const float r0 = round_to<__nv_bfloat16>(__bfloat162float(e_bias[ps][0]) + round_to<__nv_bfloat16>(lo));
            const float r1 = round_to<__nv_bfloat16>(__bfloat162float(e_bias[ps][1]) + round_to<__nv_bfloat16>(hi));
            float ss = valid ? fmaf(r0, r0, r1 * r1) : 0.f;
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            if (valid) {
                *reinterpret_cast<uint32_t*>(p.out + (int64_t)row * p.N + tile * R + nt * 8 + 2 * j) = pack_bf16x2(r0, r1);
                if (j == 0) p.ss_out[(int64_t)row * (p.N / 8) + tile * NT + nt] = ss;
            }
        }
        return;
    }
#pragma unroll
    for (int ps = 0; ps < PASSES; ++ps) {
        const int idx = tid + ps * kThinThreads, j = idx & 3, row = (idx >> 2) & (MP - 1), nt = idx / (4 * MP);
        if (row >= p.M || idx >= ITEMS) continue;
        if (EPI == kThinBias) {
            float lo = 0.f, hi = 0.f;                     // columns 2j, 2j + 1 of the n-tile, summed in warp order
#pragma unroll
            for (int wv = 0; wv < 4; ++wv) {
                const float2 v = *reinterpret_cast<const float2*>(c_sm + ((size_t)(wv * NT + nt) * MP + row) * 8 + 2 * j);
                lo += v.x;
                hi += v.y;
            }
            const uint32_t packed = pack_bf16x2(lo + __bfloat162float(e_bias[ps][0]), hi + __bfloat162float(e_bias[ps][1]));
            *reinterpret_cast<uint32_t*>(p.out + (int64_t)row * p.N + tile * R + nt * 8 + 2 * j) = packed;
        } else {
            float xl = 0.f, xh = 0.f;                     // columns j (first half) and j + 4 (second half) of the n-tile
#pragma unroll
            for (int wv = 0; wv < 4; ++wv) {
                xl += c_sm[((size_t)(wv * NT + nt) * MP + row) * 8 + j];
                xh += c_sm[((size_t)(wv * NT + nt) * MP + row) * 8 + 4 + j];
            }
            const int g = tile * NT + nt, head = g / per_head, d = (g - head * per_head) * 4 + j;
            xl = round_to<__nv_bfloat16>(xl + __bfloat162float(e_bias[ps][0]));
            xh = round_to<__nv_bfloat16>(xh + __bfloat162float(e_bias[ps][1]));
            if (head < p.n_heads + p.n_kv_heads) {
                const float cl = __bfloat162float(e_cos[ps][0]), ch = __bfloat162float(e_cos[ps][1]);
                const float sl = __bfloat162float(e_sin[ps][0]), sh = __bfloat162float(e_sin[ps][1]);
                const float a = round_to<__nv_bfloat16>(__fmul_rn(xl, cl)), b = round_to<__nv_bfloat16>(__fmul_rn(xh, sl));
                const float dd = round_to<__nv_bfloat16>(__fmul_rn(xh, ch)), e = round_to<__nv_bfloat16>(__fmul_rn(xl, sh));
                xl = round_to<__nv_bfloat16>(__fadd_rn(a, -b));
                xh = round_to<__nv_bfloat16>(__fadd_rn(dd, e));
            }
            __nv_bfloat16* dst;
            if (head < p.n_heads) {
                dst = p.out + ((int64_t)row * p.n_heads + head) * p.head_dim;
            } else if (head < p.n_heads + p.n_kv_heads) {
                dst = p.k_cache + (e_slot[ps] * p.n_kv_heads + (head - p.n_heads)) * p.head_dim;
            } else {
                dst = p.v_cache + (e_slot[ps] * p.n_kv_heads + (head - p.n_heads - p.n_kv_heads)) * p.head_dim;
            }
            dst[d] = __float2bfloat16_rn(xl);
            dst[d + half] = __float2bfloat16_rn(xh);
        }
    }
}

// ---- gate/up + SiLU*mul: nine 8-row tiles per CTA, twelve warps ----------------------------------------------------
// W = [gate; up] with 2 * inter rows. A tile is FOUR gate rows and the matching four up rows (one mma n-tile), a CTA owns
// nine consecutive tiles (inter = 4864 -> 1216 tiles -> 136 CTAs: one wave) and keeps their weight rows (130 KB) and all
// of X in shared memory. Warp w works on K quarter w % 4 - so the four SM sub-partitions carry the same number of mma -
// for the three tiles 3 * (w / 4) + {0, 1, 2} at once: one set of activation fragments feeds three weight tiles, which
// keeps shared-memory reads (the bound after the tensor pipe at this shape) at 3.5 KB per 12 mma. The four K quarters of
// a tile meet in shared memory (the activation rows' space, free by then) and one thread finishes (tile, token row):
// bf16(gate), bf16(up), SiLU in fp32 rounded to bf16, product rounded to bf16, one 8-byte store.
constexpr int kSwTiles = 9;
constexpr int kSwThreads = 384;

// NORM: x is the un-normalised residual stream and the RMSNorm is applied here, in shared memory, before the k-loop:
// h = ln_w * bf16(x * rsqrt(sum(x^2) / K + eps)) with sum(x^2) handed over as ss_parts pieces per row by the kernel
// that produced x (ns_thin_gemm_residual). Every CTA normalises its own copy of the rows (M x K elements on twelve warps:
// about half a microsecond) - less than the separate norm kernel and its boundary cost inside a decode layer.
template <int MT, bool NORM>
__global__ void __launch_bounds__(kSwThreads) thin_swiglu_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                                 __nv_bfloat16* __restrict__ out, int M, int K, int inter,
                                                                 const float* __restrict__ ss_in, int ss_parts,
                                                                 const __nv_bfloat16* __restrict__ ln_w, float eps) {
    constexpr int MP = 16 * MT;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q = warp & 3, grp = warp >> 2;             // K quarter; which three of the CTA's nine tiles
    const uint32_t pitch = (uint32_t)K * 2 + 16;
    const uint32_t x_sm = smem_u32(smem);                // [MP][pitch]; later the partial tiles [9][4][MP][8] fp32
    const uint32_t w_sm = x_sm + MP * pitch;             // [9 * 8][pitch]
    float* c_sm = reinterpret_cast<float*>(smem);
    const uint32_t ln_sm = w_sm + kSwTiles * 8 * pitch;  // NORM: [K] bf16 norm weights
    const int n_tiles = inter / 4;
    const int tile0 = blockIdx.x * kSwTiles + grp * 3;   // this warp's first tile
    pdl_launch_dependents();                              // the next kernel's launch latency passes while this one runs
    // X arrives by bulk copies (one per token row, issued after the dependency wait) on this barrier: they do not queue
    // behind the weights' cp.async traffic in the load/store pipe the way ordinary loads of X would
    __shared__ __align__(8) uint64_t x_bar;
    const uint32_t mb_x = smem_u32(&x_bar);
    if (tid == 0) {
        mbar_init(mb_x, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(mb_x, (uint32_t)M * (uint32_t)K * 2);
    }
    __syncthreads();
    const uint32_t kbase = (uint32_t)q * (uint32_t)(K / 4) * 2;      // byte offset of this warp's K quarter in a row
    if (NORM) {                                           // the norm weights are weights too: fetched before the wait, as
        for (int c = tid; c < K / 8; c += kSwThreads) cp_async16(ln_sm + c * 16, ln_w + c * 8, 16);   // the OLDEST group
        cp_async_commit();
    }
    // This warp's quarter of its three tiles' weight rows, before the dependency wait (they stream while the norm runs),
    // in the order the k-loop uses them: one commit group per iteration (32 columns = 64 bytes of each of the 24 rows;
    // lane = (row, 16-byte chunk)), so the loop can start on the first group while the rest is still on its way.
    const int iters = K / 128;
    {
        const int r = lane >> 2, c = lane & 3;
        const uint8_t* src[3];
        uint32_t dst[3];
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const int gt = min(tile0 + i, n_tiles - 1);   // a tile past the end re-reads the last one; it is never stored
            const int row = (r < 4 ? 0 : inter) + 4 * gt + (r & 3);
            src[i] = reinterpret_cast<const uint8_t*>(w + (int64_t)row * K) + kbase + c * 16;
            dst[i] = w_sm + ((grp * 3 + i) * 8 + r) * pitch + kbase + c * 16;
        }
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int i = 0; i < 3; ++i) cp_async16(dst[i] + it * 64, src[i] + it * 64, 16);
            cp_async_commit();
        }
    }
    pdl_wait();
    if (lane < 3) {                                       // token rows over the twelve warps, up to three copies each
        const int m = warp + 12 * lane;
        if (m < M) bulk_g2s(x_sm + m * pitch, x + (int64_t)m * K, (uint32_t)K * 2, mb_x);
    }
    float rstd[3] = {0.f, 0.f, 0.f};                      // NORM: of rows warp, warp + 12, warp + 24
    if (NORM) {
        // all of a warp's pieces are requested before any is used: one L2 round trip, under the X copies' own
        float part[3] = {0.f, 0.f, 0.f};
        if ((ss_parts & 3) == 0) {
            float4 v[3];
#pragma unroll
            for (int i = 0; i < 3; ++i) v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c = lane; c < ss_parts / 4; c += 32) {
#pragma unroll
                for (int i = 0; i < 3; ++i)
                    if (warp + 12 * i < M) {
                        const float4 t = *reinterpret_cast<const float4*>(ss_in + (int64_t)(warp + 12 * i) * ss_parts + 4 * c);
                        v[i].x += t.x; v[i].y += t.y; v[i].z += t.z; v[i].w += t.w;
                    }
            }
#pragma unroll
            for (int i = 0; i < 3; ++i) part[i] = (v[i].x + v[i].y) + (v[i].z + v[i].w);
        } else {
            for (int c = lane; c < ss_parts; c += 32)
#pragma unroll
                for (int i = 0; i < 3; ++i)
                    if (warp + 12 * i < M) part[i] += ss_in[(int64_t)(warp + 12 * i) * ss_parts + c];
        }
#pragma unroll
        for (int i = 0; i < 3; ++i) rstd[i] = rsqrtf(warp_sum(part[i]) / (float)K + eps);
    }

    float acc[3][MT][4];
#pragma unroll
    for (int i = 0; i < 3; ++i)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) acc[i][mt][0] = acc[i][mt][1] = acc[i][mt][2] = acc[i][mt][3] = 0.f;
    const uint32_t b_addr = w_sm + (grp * 24 + (lane & 7)) * pitch + kbase + (lane >> 3) * 16;
    const uint32_t a_addr = x_sm + ((lane & 7) + (((lane >> 3) & 1) << 3)) * pitch + kbase + (lane >> 4) * 16;
    struct Frag { uint32_t b[3][4]; uint32_t a[2][MT][4]; };
    auto load_frag = [&](Frag& f, int it) {
#pragma unroll
        for (int i = 0; i < 3; ++i) ldmatrix_x4(b_addr + i * 8 * pitch + it * 64, f.b[i][0], f.b[i][1], f.b[i][2], f.b[i][3]);
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
            for (int i = 0; i < 3; ++i)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) mma_bf16_16816(acc[i][mt], f.a[s][mt], f.b[i][2 * s], f.b[i][2 * s + 1]);
    };
    // group `it` holds iteration it's weights: at most iters - 1 - it younger groups may still be pending
    auto wait_for = [&](int it) {
        switch (iters - 1 - it) {
            case 0: cp_async_wait<0>(); break;
            case 1: cp_async_wait<1>(); break;
            case 2: cp_async_wait<2>(); break;
            case 3: cp_async_wait<3>(); break;
            case 4: cp_async_wait<4>(); break;
            case 5: cp_async_wait<5>(); break;
            case 6: cp_async_wait<6>(); break;
            case 7: cp_async_wait<7>(); break;
            default: break;                               // more than 7 younger groups: this one is waited for later
        }
        __syncwarp();
    };
    {
        Frag f0, f1;
        if (iters > 8) cp_async_wait<7>();                // groups 0 .. iters - 9: the switch above covers the last eight
        if (!mbar_wait_bounded(mb_x, 0) && lane == 0) atomicAdd(&g_thin_errors, 1u);
        if (NORM) {
            // every thread waits for its own copies of the norm weights: the oldest group, so the seven youngest (the
            // weights of the last iterations) may stay in flight
            cp_async_wait<7>();
            __syncthreads();
            // 16 bytes (eight elements) per lane and step; the three rows of a warp side by side for the loads' latency
            for (int c = lane; c < K / 8; c += 32) {
                uint4 wv;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(wv.x), "=r"(wv.y), "=r"(wv.z), "=r"(wv.w) : "r"(ln_sm + c * 16));
                uint4 xv[3];
#pragma unroll
                for (int i = 0; i < 3; ++i)
                    if (warp + 12 * i < M)
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(xv[i].x), "=r"(xv[i].y), "=r"(xv[i].z), "=r"(xv[i].w)
                                     : "r"(x_sm + (warp + 12 * i) * pitch + c * 16));
#pragma unroll
                for (int i = 0; i < 3; ++i) {
                    if (warp + 12 * i >= M) continue;
                    uint32_t* xe = reinterpret_cast<uint32_t*>(&xv[i]);
                    const uint32_t* we = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&xe[e]);
                        const __nv_bfloat162 n = __floats2bfloat162_rn(__bfloat162float(v.x) * rstd[i], __bfloat162float(v.y) * rstd[i]);
                        const __nv_bfloat162 h = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&we[e]), n);
                        xe[e] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(x_sm + (warp + 12 * i) * pitch + c * 16), "r"(xv[i].x),
                                 "r"(xv[i].y), "r"(xv[i].z), "r"(xv[i].w)
                                 : "memory");
                }
            }
            __syncthreads();
        }
        wait_for(0);
        load_frag(f0, 0);
        for (int it = 0; it < iters; it += 2) {
            if (it + 1 < iters) { wait_for(it + 1); load_frag(f1, it + 1); }
            compute(f0);
            if (it + 2 < iters) { wait_for(it + 2); load_frag(f0, it + 2); }
            if (it + 1 < iters) compute(f1);
        }
    }
    __syncthreads();                                      // every warp is done reading X: its space takes the partial tiles
    {
        const int r0 = lane >> 2, cp = (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            float* mine = c_sm + ((size_t)((grp * 3 + i) * 4 + q) * MP) * 8;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                *reinterpret_cast<float2*>(mine + (16 * mt + r0) * 8 + cp) = make_float2(acc[i][mt][0], acc[i][mt][1]);
                *reinterpret_cast<float2*>(mine + (16 * mt + r0 + 8) * 8 + cp) = make_float2(acc[i][mt][2], acc[i][mt][3]);
            }
        }
    }
    __syncthreads();
    if (tid < kSwTiles * MP) {
        const int lt = tid / MP, row = tid % MP;
        const int gt = blockIdx.x * kSwTiles + lt;
        if (row < M && gt < n_tiles) {
            float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int qq = 0; qq < 4; ++qq) {              // K quarters in order
                const float4 a = *reinterpret_cast<const float4*>(c_sm + ((size_t)(lt * 4 + qq) * MP + row) * 8);
                const float4 b = *reinterpret_cast<const float4*>(c_sm + ((size_t)(lt * 4 + qq) * MP + row) * 8 + 4);
                g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w;
                u[0] += b.x; u[1] += b.y; u[2] += b.z; u[3] += b.w;
            }
            float r[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float gg = round_to<__nv_bfloat16>(g[j]), uu = round_to<__nv_bfloat16>(u[j]);
                const float sg = round_to<__nv_bfloat16>(gg / (1.0f + expf(-gg)));
                r[j] = sg * uu;
            }
            uint2 packed;
            packed.x = pack_bf16x2(r[0], r[1]);
            packed.y = pack_bf16x2(r[2], r[3]);
            *reinterpret_cast<uint2*>(out + (int64_t)row * inter + 4 * gt) = packed;
        }
    }
}

template <int MT, bool NORM>
int launch_thin_swiglu(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* out, int M, int K, int inter, const float* ss_in,
                       int ss_parts, const __nv_bfloat16* ln_w, float eps, cudaStream_t st) {
    const size_t smem = (size_t)(16 * MT + kSwTiles * 8) * ((size_t)K * 2 + 16) + (NORM ? (size_t)K * 2 : 0);
    static SmemOptIn optin;
    if (optin.needs(smem)) {
        cudaError_t e = cudaFuncSetAttribute(thin_swiglu_kernel<MT, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "thin_swiglu_gemm: cannot reserve %zu bytes of shared memory: %s", smem,
                                          cudaGetErrorString(e));
        optin.done(smem);
    }
    const int grid = (inter / 4 + kSwTiles - 1) / kSwTiles;
    cudaError_t e = launch_pdl(thin_swiglu_kernel<MT, NORM>, dim3((unsigned)grid), dim3(kSwThreads), smem, st, x, w, out, M, K, inter,
                               ss_in, ss_parts, ln_w, eps);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "thin_swiglu_gemm: launch failed: %s", cudaGetErrorString(e));
    return NS_OK;
}

// n-tiles per CTA: one while N / 8 CTAs are a single wave of the device's SMs, else two if that makes them one
inline int thin_ntiles(int N) {
    int sms = device_sm_count();
    if (sms <= 0) sms = 148;              // no device to ask (argument validation on a machine without one): B200
    return (N / kThinRows <= sms || N % (2 * kThinRows) != 0) ? 1 : 2;
}
inline size_t thin_smem(int mp, int nt, int K) {
    return (size_t)(kThinRows * nt + mp) * ((size_t)K * 2 + 16) + (size_t)4 * nt * mp * 8 * 4;
}

template <int MT, int NT, int EPI>
int launch_thin(const ThinParams& p, cudaStream_t st) {
    const size_t smem = thin_smem(16 * MT, NT, p.K);
    static SmemOptIn optin;
    if (optin.needs(smem)) {
        cudaError_t e = cudaFuncSetAttribute(thin_gemm_kernel<MT, NT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "thin_gemm: cannot reserve %zu bytes of shared memory: %s", smem,
                                          cudaGetErrorString(e));
        optin.done(smem);
    }
    const int tiles = p.N / (kThinRows * NT);
    cudaError_t e = launch_pdl(thin_gemm_kernel<MT, NT, EPI>, dim3((unsigned)tiles), dim3(kThinThreads), smem, st, p);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "thin_gemm: launch failed: %s", cudaGetErrorString(e));
    return NS_OK;
}

template <int EPI> int dispatch_thin(const ThinParams& p, cudaStream_t st) {
    if (thin_ntiles(p.N) == 1) {
        if (p.M <= 16) return launch_thin<1, 1, EPI>(p, st);
        if (p.M <= 32) return launch_thin<2, 1, EPI>(p, st);
        return launch_thin<4, 1, EPI>(p, st);
    }
    if (p.M <= 16) return launch_thin<1, 2, EPI>(p, st);
    if (p.M <= 32) return launch_thin<2, 2, EPI>(p, st);
    return launch_thin<4, 2, EPI>(p, st);
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
    NS_REQUIRE(thin_smem(mp, thin_ntiles(N), K) <= 220 * 1024, NS_ERR_UNSUPPORTED,
               "thin_gemm: %d token rows + %d weight rows of K=%d do not fit shared memory", mp, kThinRows * thin_ntiles(N), K);
    ThinParams p;
    p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.bias = (const __nv_bfloat16*)bias;
    p.out = (__nv_bfloat16*)out; p.cos = (const __nv_bfloat16*)cos; p.sin = (const __nv_bfloat16*)sin;
    p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache; p.slots = slots;
    p.M = M; p.N = N; p.K = K; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (epilogue == kThinBias) return dispatch_thin<kThinBias>(p, st);
    if (epilogue == kThinRopeKv) {
        NS_REQUIRE(n_heads > 0 && n_kv_heads > 0 && N % (n_heads + 2 * n_kv_heads) == 0, NS_ERR_INVALID_ARG,
                   "thin_gemm: N is not (n_heads + 2 * n_kv_heads) * head_dim");
        p.head_dim = N / (n_heads + 2 * n_kv_heads);
        NS_REQUIRE(p.head_dim == 64 || p.head_dim == 128, NS_ERR_UNSUPPORTED,
                   "thin_gemm: the RoPE + KV-write epilogue handles head_dim 64 and 128, not %d", p.head_dim);
        NS_REQUIRE(cos && sin && k_cache && v_cache && slots, NS_ERR_INVALID_ARG, "thin_gemm: RoPE epilogue needs cos, sin, caches, slots");
        return dispatch_thin<kThinRopeKv>(p, st);
    }
    return fail(NS_ERR_INVALID_ARG, "thin_gemm: unknown epilogue %d (0 = bias, 2 = RoPE + KV write)", epilogue);
}

extern "C" int ns_thin_swiglu_gemm(const void* x, const void* w, void* out, int32_t M, int32_t inter, int32_t K, void* stream) {
    NS_REQUIRE(M >= 0 && inter > 0 && K > 0, NS_ERR_INVALID_ARG, "thin_swiglu_gemm: bad shape");
    if (M == 0) return NS_OK;
    NS_REQUIRE(x && w && out, NS_ERR_INVALID_ARG, "thin_swiglu_gemm: null pointer");
    NS_REQUIRE(M <= 32, NS_ERR_UNSUPPORTED, "thin_swiglu_gemm: %d token rows > 32", M);
    NS_REQUIRE(K % 128 == 0 && inter % 4 == 0, NS_ERR_UNSUPPORTED, "thin_swiglu_gemm: K=%d must be a multiple of 128 and inter=%d of 4", K, inter);
    NS_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 7) == 0,
               NS_ERR_INVALID_ARG, "thin_swiglu_gemm: x / w must be 16-byte aligned, out 8-byte aligned");
    const int mp = M <= 16 ? 16 : 32;
    const size_t smem = (size_t)(mp + kSwTiles * 8) * ((size_t)K * 2 + 16);
    NS_REQUIRE(smem <= 227 * 1024 && (size_t)kSwTiles * 4 * mp * 8 * 4 <= (size_t)mp * ((size_t)K * 2 + 16), NS_ERR_UNSUPPORTED,
               "thin_swiglu_gemm: K=%d does not fit shared memory (72 weight rows + %d token rows)", K, mp);
    cudaStream_t st = (cudaStream_t)stream;
    if (M <= 16) return launch_thin_swiglu<1, false>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, K, inter, nullptr, 0, nullptr, 0.f, st);
    return launch_thin_swiglu<2, false>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, K, inter, nullptr, 0, nullptr, 0.f, st);
}

extern "C" int ns_thin_gemm_residual(const void* x, const void* w, const void* residual, void* out, float* ss_out, int32_t M,
                                     int32_t N, int32_t K, void* stream) {
    NS_REQUIRE(M >= 0 && N > 0 && K > 0, NS_ERR_INVALID_ARG, "thin_gemm_residual: bad shape");
    if (M == 0) return NS_OK;
    NS_REQUIRE(x && w && residual && out && ss_out, NS_ERR_INVALID_ARG, "thin_gemm_residual: null pointer");
    NS_REQUIRE(M <= 64, NS_ERR_UNSUPPORTED, "thin_gemm_residual: %d token rows > 64", M);
    NS_REQUIRE(K % 128 == 0 && N % 8 == 0, NS_ERR_UNSUPPORTED, "thin_gemm_residual: K=%d must be a multiple of 128 and N=%d of 8", K, N);
    NS_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0 &&
                   ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(residual)) & 3) == 0,
               NS_ERR_INVALID_ARG, "thin_gemm_residual: x / w must be 16-byte aligned, out / residual 4-byte aligned");
    const int mp = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    NS_REQUIRE(thin_smem(mp, thin_ntiles(N), K) <= 220 * 1024, NS_ERR_UNSUPPORTED,
               "thin_gemm_residual: %d token rows + %d weight rows of K=%d do not fit shared memory", mp, kThinRows * thin_ntiles(N), K);
    ThinParams p = {};
    p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.out = (__nv_bfloat16*)out;
    p.residual = (const __nv_bfloat16*)residual; p.ss_out = ss_out;
    p.M = M; p.N = N; p.K = K;
    return dispatch_thin<kThinResidual>(p, (cudaStream_t)stream);
}

extern "C" int ns_thin_swiglu_gemm_norm(const void* x, const float* ss_in, int32_t ss_parts, const void* ln_w, float eps,
                                        const void* w, void* out, int32_t M, int32_t inter, int32_t K, void* stream) {
    NS_REQUIRE(M >= 0 && inter > 0 && K > 0 && ss_parts > 0, NS_ERR_INVALID_ARG, "thin_swiglu_gemm_norm: bad shape");
    if (M == 0) return NS_OK;
    NS_REQUIRE(x && w && out && ss_in && ln_w, NS_ERR_INVALID_ARG, "thin_swiglu_gemm_norm: null pointer");
    NS_REQUIRE(M <= 32, NS_ERR_UNSUPPORTED, "thin_swiglu_gemm_norm: %d token rows > 32", M);
    NS_REQUIRE(K % 128 == 0 && inter % 4 == 0, NS_ERR_UNSUPPORTED, "thin_swiglu_gemm_norm: K=%d must be a multiple of 128 and inter=%d of 4", K, inter);
    NS_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(ln_w)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 7) == 0,
               NS_ERR_INVALID_ARG, "thin_swiglu_gemm_norm: x / w / ln_w must be 16-byte aligned, out 8-byte aligned");
    const int mp = M <= 16 ? 16 : 32;
    const size_t smem = (size_t)(mp + kSwTiles * 8) * ((size_t)K * 2 + 16) + (size_t)K * 2;
    NS_REQUIRE(smem <= 227 * 1024 && (size_t)kSwTiles * 4 * mp * 8 * 4 <= (size_t)mp * ((size_t)K * 2 + 16), NS_ERR_UNSUPPORTED,
               "thin_swiglu_gemm_norm: K=%d does not fit shared memory (72 weight rows + %d token rows)", K, mp);
    cudaStream_t st = (cudaStream_t)stream;
    if (M <= 16)
        return launch_thin_swiglu<1, true>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, K, inter, ss_in,
                                           ss_parts, (const __nv_bfloat16*)ln_w, eps, st);
    return launch_thin_swiglu<2, true>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, K, inter, ss_in, ss_parts,
                                       (const __nv_bfloat16*)ln_w, eps, st);
}

namespace ns {
// Device address of this file's error counter on the current device (resolved once per device; the first call on a
// device must come before any stream capture). Used by ns_collect_status.
int thin_gemm_error_counter(const unsigned int** out) {
    static const unsigned int* addr[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(NS_ERR_CUDA, "thin_gemm_error_counter: no current device");
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_thin_errors);
        if (e != cudaSuccess || p == nullptr) return fail(NS_ERR_CUDA, "thin_gemm_error_counter: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        addr[dev] = static_cast<const unsigned int*>(p);
    }
    *out = addr[dev];
    return NS_OK;
}
}  // namespace ns

extern "C" int ns_thin_gemm_errors(int32_t* count) {
    NS_REQUIRE(count != nullptr, NS_ERR_INVALID_ARG, "thin_gemm_errors: null pointer");
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_thin_errors, sizeof(v));
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "thin_gemm_errors: %s", cudaGetErrorString(e));
    *count = (int32_t)v;
    return NS_OK;
}

// Persistent weight-streaming GEMM for decode-sized batches (M <= 64 token rows) and WIDE outputs: the MLP's merged
// gate/up projection with the preceding residual-add + RMSNorm and the following SiLU(gate)*up fused in, and plain
// Y = X W^T (+bias).
//
// At M <= 64 the GEMM is a read of N*K*2 weight bytes; everything here serves keeping that read going:
//   * one CTA per SM, each walking units of 16 weight rows (unit u, u + grid, ...); a unit's rows arrive by TMA bulk
//     copies (cp.async.bulk, one per row, completing on the stage's mbarrier) into a ring of shared-memory stages that
//     a dedicated producer warp keeps full; at the model's sizes a CTA's whole share is in flight from its first
//     microsecond, and it is issued BEFORE griddepcontrol.wait, i.e. while the preceding kernel still runs;
//   * activations are STATIONARY IN REGISTERS: the 8 consumer warps split K, each keeps the mma A-fragments of its
//     K/8 columns for all token rows (7 k-steps at K = 896), so the inner loop reads shared memory for weights only
//     (one ldmatrix.x4 per 2*MT mma.sync m16n8k16);
//   * per unit the 8 K-partials [tokens x 16] are summed through shared memory in warp order (deterministic), and the
//     epilogue runs on the sums: bias, or SiLU(gate)*up where a unit is 8 gate rows + the matching 8 up rows;
//   * prologue (optional): r = residual + a rounded to bf16 (stored once as the new residual stream), then
//     X = ln_w * bf16(r * rsqrt(mean(r^2) + eps)): the separate add+RMSNorm kernel disappears.
// Rounding points are those of the unfused ops (GEMM result rounded to bf16, then each elementwise op rounded).
// Every mbarrier wait is bounded; a wait that runs out raises a device-side error count (ns_stream_gemm_errors).
#include "common.cuh"

namespace ns {

enum StreamEpilogue { kSgBias = 0, kSgSiluMul = 1, kSgResidual = 2 };

struct StreamGemmParams {
    const __nv_bfloat16* x;          // [M, K] activations, or the pre-norm addend `a` when ln_w is set
    const __nv_bfloat16* residual;   // prologue: added to x before the norm (may be null: plain norm of x)
    const __nv_bfloat16* ln_w;       // prologue: RMSNorm weight [K]; null = no prologue
    __nv_bfloat16* residual_out;     // prologue: r = residual + x, [M, K] (may be null)
    const __nv_bfloat16* w;          // [N, K] row-major weights
    const __nv_bfloat16* bias;       // [N] or null (kSgBias only)
    __nv_bfloat16* out;              // kSgBias, kSgResidual: [M, N]; kSgSiluMul: [M, inter]
    const float* ss_in;              // prologue: [M, ss_parts] partial sums of x^2 left by the GEMM that produced x
    int ss_parts;                    //           (then x is already the residual stream: no add, no second pass)
    const __nv_bfloat16* add_in;     // kSgResidual: [M, N] residual stream the result is added to
    float* ss_out;                   // kSgResidual: [M, N/16] sum over each unit's 16 columns of out^2
    int M, N, K;
    int inter;                       // kSgSiluMul: rows of gate (= N / 2)
    int units;                       // N / 16
    int stages;                      // ring depth
    float eps;
    long long* timeline;             // debug: clock64 stamps of CTA 0 (null in normal use)
};

__device__ unsigned int g_stream_gemm_errors = 0;
static long long* g_sg_timeline = nullptr;

namespace sg {

__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t mbar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar) : "memory");
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

// ---- two bf16 values in one register: the token-wise ops with the unfused ops' rounding points ------------------
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
// bf16(a + b) per half: fp32 add, one rounding (what the framework's bf16 add does)
__device__ __forceinline__ uint32_t add_pair(uint32_t a, uint32_t b) {
    return pack_bf16x2(__fadd_rn(bf_lo(a), bf_lo(b)), __fadd_rn(bf_hi(a), bf_hi(b)));
}
__device__ __forceinline__ float sq_pair(uint32_t v, float acc) {
    const float lo = bf_lo(v), hi = bf_hi(v);
    return fmaf(hi, hi, fmaf(lo, lo, acc));
}
// w * bf16(v * inv) per half, the product rounded to bf16 (a product of two bf16 values is exact in fp32)
__device__ __forceinline__ uint32_t norm_pair(uint32_t v, float inv, uint32_t w) {
    const uint32_t n = pack_bf16x2(__fmul_rn(bf_lo(v), inv), __fmul_rn(bf_hi(v), inv));
    return pack_bf16x2(__fmul_rn(bf_lo(w), bf_lo(n)), __fmul_rn(bf_hi(w), bf_hi(n)));
}

}  // namespace sg

constexpr int kSgConsumerWarps = 8;                  // mma warps: each owns K/8 columns
constexpr int kSgConsumers = kSgConsumerWarps * 32;
constexpr int kSgEpiWarps = 4;                       // epilogue warps: sum the K-partials, apply the epilogue, store
constexpr int kSgEpiThreads = kSgEpiWarps * 32;
constexpr int kSgProducerWarp = kSgConsumerWarps + kSgEpiWarps;
constexpr int kSgThreads = (kSgProducerWarp + 1) * 32;
constexpr int kSgRedBufs = 3;                        // K-partial buffers in flight between mma and epilogue warps
constexpr int kSgMaxStages = 8;
constexpr int kSgUnitRows = 16;

// MT: 16-row token tiles; KS: k-steps (of 16) per consumer warp, K = 128 * KS.
template <int MT, int KS, int EPI>
__global__ void __launch_bounds__(kSgThreads, 1) stream_gemm_kernel(const StreamGemmParams p) {
    constexpr int MP = 16 * MT;
    constexpr int K = 128 * KS;
    constexpr int ROW = K * 2 + 16;                    // bytes per shared-memory row (+16: conflict-free ldmatrix)
    constexpr uint32_t ROW_BYTES = K * 2;
    constexpr int STAGE = kSgUnitRows * ROW;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[kSgMaxStages], empty_bar[kSgMaxStages];
    __shared__ __align__(8) uint64_t part_full[kSgRedBufs], part_empty[kSgRedBufs];
    // [ring: stages x 16 weight rows][A staging MP rows, reused afterwards for the K-partials (kSgRedBufs x 8 x MP x 16 fp32)]
    uint8_t* ring = smem;
    uint8_t* a_sm = smem + (size_t)p.stages * STAGE;
    float* red = reinterpret_cast<float*>(a_sm);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.stages;
    const int n_my = (p.units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // units of this CTA

    int tl = 0;
    auto stamp = [&]() {
        if (p.timeline != nullptr && blockIdx.x == 0 && tid == 0) p.timeline[tl] = clock64();
        ++tl;
    };
    stamp();
    pdl_launch_dependents();
    if (tid == 0) {
        for (int i = 0; i < S; ++i) {
            sg::mbar_init(smem_u32(&full_bar[i]), 1);
            sg::mbar_init(smem_u32(&empty_bar[i]), kSgConsumerWarps);
        }
        for (int i = 0; i < kSgRedBufs; ++i) {
            sg::mbar_init(smem_u32(&part_full[i]), kSgConsumerWarps);
            sg::mbar_init(smem_u32(&part_empty[i]), kSgEpiWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    auto unit_row = [&](int unit, int r) -> int {      // weight row behind local row r of a unit
        if (EPI == kSgSiluMul) return r < 8 ? unit * 8 + r : p.inter + unit * 8 + (r - 8);
        return unit * kSgUnitRows + r;
    };

    if (warp == kSgProducerWarp) {
        // ---- producer: weights only, so it never waits for the preceding kernel ------------------------------
        auto fill = [&](int i) {
            const int slot = i % S;
            const uint32_t mb = smem_u32(&full_bar[slot]);
            if (lane == 0) sg::mbar_expect_tx(mb, kSgUnitRows * ROW_BYTES);
            __syncwarp();
            if (lane < kSgUnitRows) {
                const int unit = (int)blockIdx.x + i * (int)gridDim.x;
                sg::bulk_g2s(smem_u32(ring) + slot * STAGE + lane * ROW, p.w + (int64_t)unit_row(unit, lane) * K, ROW_BYTES, mb);
            }
        };
        const int first = n_my < S ? n_my : S;
        for (int i = 0; i < first; ++i) fill(i);
        for (int i = S; i < n_my; ++i) {
            bool freed = true;
            if (lane == 0) freed = sg::mbar_wait_bounded(smem_u32(&empty_bar[i % S]), (uint32_t)((i / S - 1) & 1));
            freed = __shfl_sync(0xffffffffu, freed, 0);
            if (!freed) {
                if (lane == 0) atomicAdd(&g_stream_gemm_errors, 1u);
                break;
            }
            fill(i);
        }
        return;
    }

    if (warp >= kSgConsumerWarps) {
        // ---- epilogue warps: unit j's eight K-partials sit in buffer j % kSgRedBufs once all mma warps have arrived ----
        constexpr int MPc = 16 * MT;
        const int et = tid - kSgConsumers;
        for (int j = 0; j < n_my; ++j) {
            const int b = j % kSgRedBufs;
            if (!sg::mbar_wait_bounded(smem_u32(&part_full[b]), (uint32_t)((j / kSgRedBufs) & 1))) {
                if (lane == 0) atomicAdd(&g_stream_gemm_errors, 1u);
                return;
            }
            const int unit = (int)blockIdx.x + j * (int)gridDim.x;
            const float* part = red + (size_t)b * kSgConsumerWarps * (MPc * 16);
            if (EPI == kSgSiluMul) {
                for (int e = et; e < p.M * 8; e += kSgEpiThreads) {
                    const int m = e >> 3, c = e & 7;
                    float g = 0.f, u = 0.f;
#pragma unroll
                    for (int w8 = 0; w8 < kSgConsumerWarps; ++w8) {
                        g += part[w8 * (MPc * 16) + m * 16 + c];
                        u += part[w8 * (MPc * 16) + m * 16 + 8 + c];
                    }
                    g = round_to<__nv_bfloat16>(g);
                    u = round_to<__nv_bfloat16>(u);
                    const float sg_ = round_to<__nv_bfloat16>(g / (1.0f + expf(-g)));
                    p.out[(int64_t)m * p.inter + unit * 8 + c] = __float2bfloat16_rn(sg_ * u);
                }
            } else {
                for (int e = et; e < MPc * 16; e += kSgEpiThreads) {     // whole half-warps share a row (shuffles below)
                    const int m = e >> 4, c = e & 15;
                    float v = 0.f;
#pragma unroll
                    for (int w8 = 0; w8 < kSgConsumerWarps; ++w8) v += part[w8 * (MPc * 16) + m * 16 + c];
                    const int n = unit * 16 + c;
                    if (p.bias) v += __bfloat162float(p.bias[n]);
                    if (EPI == kSgResidual) {
                        // r = bf16(residual + bf16(gemm)); the unit's share of sum(r^2) for the consumer's RMSNorm
                        float r = 0.f;
                        if (m < p.M) {
                            r = round_to<__nv_bfloat16>(__fadd_rn(__bfloat162float(p.add_in[(int64_t)m * p.N + n]), round_to<__nv_bfloat16>(v)));
                            p.out[(int64_t)m * p.N + n] = __float2bfloat16_rn(r);
                        }
                        float sq = r * r;
#pragma unroll
                        for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                        if (c == 0 && m < p.M && p.ss_out != nullptr) p.ss_out[(int64_t)m * p.units + unit] = sq;
                    } else if (m < p.M) {
                        p.out[(int64_t)m * p.N + n] = __float2bfloat16_rn(v);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) sg::mbar_arrive(smem_u32(&part_empty[b]));      // this warp has read the buffer
        }
        return;
    }

    // ---- consumers ---------------------------------------------------------------------------------------------
    // Warp w prepares token rows w, w + 8, ...; lane l owns the 16-byte chunks l, l + 32, ... of a row. Every x row
    // of the warp is fetched by 16-byte cp.async at once (one round trip); what the norm needs besides (residual
    // rows, or the per-row sum-of-squares partials left by the producing GEMM) is loaded to registers meanwhile.
    constexpr int RPW = MP / kSgConsumerWarps;          // rows per warp
    constexpr int CH = (K / 8 + 31) / 32;               // chunks per lane
    constexpr int RB = CH > 4 ? (RPW < 2 ? RPW : 2) : (RPW < 4 ? RPW : 4);   // rows per batch (register budget)
    stamp();
    pdl_wait();                                         // activations come from the preceding kernel
    stamp();
    uint32_t afrag[KS][MT][4];       // this warp's A fragments: columns [warp*KS*16, (warp+1)*KS*16) of every token row
    if (p.ln_w == nullptr) {
        // Plain activations: straight from global memory into the mma fragment registers (a0 = row r, cols c..c+1;
        // a1 = row r+8; a2 = cols c+8..c+9; a3 = both), every load independent: one round trip, no staging, no barrier.
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int kcol = (warp * KS + ks) * 16 + c0;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int ra = 16 * mt + r0, rb = ra + 8;
                const __nv_bfloat16* pa = p.x + (int64_t)ra * K + kcol;
                const __nv_bfloat16* pb = p.x + (int64_t)rb * K + kcol;
                afrag[ks][mt][0] = ra < p.M ? *reinterpret_cast<const uint32_t*>(pa) : 0u;
                afrag[ks][mt][1] = rb < p.M ? *reinterpret_cast<const uint32_t*>(pb) : 0u;
                afrag[ks][mt][2] = ra < p.M ? *reinterpret_cast<const uint32_t*>(pa + 8) : 0u;
                afrag[ks][mt][3] = rb < p.M ? *reinterpret_cast<const uint32_t*>(pb + 8) : 0u;
            }
        }
    } else {
#pragma unroll
    for (int j = 0; j < RPW; ++j) {
        const int m = warp + kSgConsumerWarps * j;
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const int c = lane + 32 * i;
            if (c < K / 8) {
                const uint32_t dst = smem_u32(a_sm) + m * ROW + c * 16;
                if (m < p.M) cp_async16(dst, p.x + (int64_t)m * K + c * 8, 16);
                else asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
            }
        }
    }
    cp_async_commit();
    stamp();
    {
        uint4 lnw[CH];
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const int c = lane + 32 * i;
            lnw[i] = c < K / 8 ? *reinterpret_cast<const uint4*>(p.ln_w + c * 8) : make_uint4(0, 0, 0, 0);
        }
        if (p.ss_in != nullptr) {
            // the producing GEMM left sum(r^2) over each of its column units: add them in unit order
            float inv[RPW];
#pragma unroll
            for (int j = 0; j < RPW; ++j) {
                const int m = warp + kSgConsumerWarps * j;
                float ss = 0.f;
                if (m < p.M)
                    for (int u = lane; u < p.ss_parts; u += 32) ss += p.ss_in[(int64_t)m * p.ss_parts + u];
                ss = warp_sum(ss);
                inv[j] = 1.0f / sqrtf(ss / (float)K + p.eps);
            }
            stamp();
            cp_async_wait<0>();
            __syncwarp();
            stamp();
#pragma unroll
            for (int j = 0; j < RPW; ++j) {
                const int m = warp + kSgConsumerWarps * j;
                if (m >= p.M) continue;
                uint8_t* dst = a_sm + (size_t)m * ROW;
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    const int c = lane + 32 * i;
                    if (c < K / 8) {
                        uint4 v = *reinterpret_cast<const uint4*>(dst + c * 16);
                        v.x = sg::norm_pair(v.x, inv[j], lnw[i].x);
                        v.y = sg::norm_pair(v.y, inv[j], lnw[i].y);
                        v.z = sg::norm_pair(v.z, inv[j], lnw[i].z);
                        v.w = sg::norm_pair(v.w, inv[j], lnw[i].w);
                        *reinterpret_cast<uint4*>(dst + c * 16) = v;
                    }
                }
            }
        } else {
#pragma unroll
            for (int b0 = 0; b0 < RPW; b0 += RB) {
                uint4 res[RB][CH];
#pragma unroll
                for (int j = 0; j < RB; ++j) {
                    const int m = warp + kSgConsumerWarps * (b0 + j);
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        const int c = lane + 32 * i;
                        res[j][i] = (p.residual != nullptr && m < p.M && c < K / 8)
                                        ? *reinterpret_cast<const uint4*>(p.residual + (int64_t)m * K + c * 8)
                                        : make_uint4(0, 0, 0, 0);
                    }
                }
                if (b0 == 0) {
                    cp_async_wait<0>();
                    __syncwarp();
                }
#pragma unroll
                for (int j = 0; j < RB; ++j) {
                    const int m = warp + kSgConsumerWarps * (b0 + j);
                    if (m >= p.M) continue;
                    uint8_t* dst = a_sm + (size_t)m * ROW;
                    const bool store_r = p.residual_out != nullptr && p.residual != nullptr && (m % (int)gridDim.x) == (int)blockIdx.x;
                    uint4 v[CH];
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        const int c = lane + 32 * i;
                        if (c < K / 8) {
                            v[i] = *reinterpret_cast<const uint4*>(dst + c * 16);
                            if (p.residual != nullptr) {
                                v[i].x = sg::add_pair(res[j][i].x, v[i].x);
                                v[i].y = sg::add_pair(res[j][i].y, v[i].y);
                                v[i].z = sg::add_pair(res[j][i].z, v[i].z);
                                v[i].w = sg::add_pair(res[j][i].w, v[i].w);
                                if (store_r) *reinterpret_cast<uint4*>(p.residual_out + (int64_t)m * K + c * 8) = v[i];
                            }
                            ss = sg::sq_pair(v[i].x, ss);
                            ss = sg::sq_pair(v[i].y, ss);
                            ss = sg::sq_pair(v[i].z, ss);
                            ss = sg::sq_pair(v[i].w, ss);
                        }
                    }
                    ss = warp_sum(ss);
                    const float inv = 1.0f / sqrtf(ss / (float)K + p.eps);
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        const int c = lane + 32 * i;
                        if (c < K / 8) {
                            v[i].x = sg::norm_pair(v[i].x, inv, lnw[i].x);
                            v[i].y = sg::norm_pair(v[i].y, inv, lnw[i].y);
                            v[i].z = sg::norm_pair(v[i].z, inv, lnw[i].z);
                            v[i].w = sg::norm_pair(v[i].w, inv, lnw[i].w);
                            *reinterpret_cast<uint4*>(dst + c * 16) = v[i];
                        }
                    }
                }
            }
        }
    }
    stamp();
    named_barrier(1, kSgConsumers);
    stamp();
    {
        const uint32_t a_base = smem_u32(a_sm);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int kcol = (warp * KS + ks) * 16;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int row = 16 * mt + (lane & 7) + (((lane >> 3) & 1) << 3);
                const int kbyte = (kcol + ((lane >> 4) << 3)) * 2;
                ldmatrix_x4(a_base + row * ROW + kbyte, afrag[ks][mt][0], afrag[ks][mt][1], afrag[ks][mt][2], afrag[ks][mt][3]);
            }
        }
    }
    named_barrier(1, kSgConsumers);                    // the staging area becomes the partial-sum buffers
    }
    stamp();

    // Main loop of the mma warps: unit j of this CTA sits in ring slot j % S; its K-partials go to buffer j % kSgRedBufs,
    // handed to the epilogue warps through part_full / part_empty, so the mma warps never wait for an epilogue.
    bool ok = true;
    for (int j = 0; j < n_my; ++j) {
        const int slot = j % S, b = j % kSgRedBufs;
        float acc[MT][2][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int q = 0; q < 2; ++q) acc[mt][q][0] = acc[mt][q][1] = acc[mt][q][2] = acc[mt][q][3] = 0.f;
        if (ok) ok = sg::mbar_wait_bounded(smem_u32(&full_bar[slot]), (uint32_t)((j / S) & 1));
        stamp();
        if (ok) {
            const uint32_t wb = smem_u32(ring) + slot * STAGE + ((lane & 7) + ((lane >> 4) << 3)) * ROW +
                                (warp * KS * 16 + (((lane >> 3) & 1) << 3)) * 2;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t b00, b01, b10, b11;
                ldmatrix_x4(wb + ks * 32, b00, b01, b10, b11);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_bf16_16816(acc[mt][0], afrag[ks][mt], b00, b01);
                    mma_bf16_16816(acc[mt][1], afrag[ks][mt], b10, b11);
                }
            }
        } else if (lane == 0) {
            atomicAdd(&g_stream_gemm_errors, 1u);
        }
        __syncwarp();
        if (lane == 0) sg::mbar_arrive(smem_u32(&empty_bar[slot]));        // this warp is done with the stage
        if (ok && j >= kSgRedBufs) ok = sg::mbar_wait_bounded(smem_u32(&part_empty[b]), (uint32_t)((j / kSgRedBufs - 1) & 1));
        float* mine = red + ((size_t)b * kSgConsumerWarps + warp) * (MP * 16);
        {
            const int r0 = lane >> 2, cp = (lane & 3) * 2;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    *reinterpret_cast<float2*>(mine + (16 * mt + r0) * 16 + 8 * q + cp) = make_float2(acc[mt][q][0], acc[mt][q][1]);
                    *reinterpret_cast<float2*>(mine + (16 * mt + r0 + 8) * 16 + 8 * q + cp) = make_float2(acc[mt][q][2], acc[mt][q][3]);
                }
        }
        __syncwarp();
        if (lane == 0) sg::mbar_arrive(smem_u32(&part_full[b]));           // release: the stores above are visible to waiters
        stamp();
    }
}

template <int MT, int KS, int EPI>
static int launch_stream(const StreamGemmParams& p0, cudaStream_t st) {
    StreamGemmParams p = p0;
    constexpr int MP = 16 * MT, K = 128 * KS, ROW = K * 2 + 16, STAGE = kSgUnitRows * ROW;
    const size_t staging = (size_t)MP * ROW, red = (size_t)kSgRedBufs * kSgConsumerWarps * MP * 16 * 4;
    const size_t fixed = staging > red ? staging : red;
    const size_t budget = 224 * 1024;
    int stages = (int)((budget - fixed) / STAGE);
    if (stages > kSgMaxStages) stages = kSgMaxStages;
    if (stages < 2) return fail(NS_ERR_UNSUPPORTED, "stream_gemm: M=%d, K=%d leaves no room for two weight stages", p.M, K);
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const int grid = p.units < sms ? p.units : sms;
    const int per_cta = (p.units + grid - 1) / grid;
    if (stages > per_cta) stages = per_cta < 2 ? 2 : per_cta;
    p.stages = stages;
    const size_t smem = (size_t)stages * STAGE + fixed;
    static SmemOptIn optin;
    if (optin.needs(smem)) {
        cudaError_t e = cudaFuncSetAttribute(stream_gemm_kernel<MT, KS, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(NS_ERR_CUDA, "stream_gemm: cannot reserve %zu bytes of shared memory: %s", smem,
                                          cudaGetErrorString(e));
        optin.done(smem);
    }
    cudaError_t e = launch_pdl(stream_gemm_kernel<MT, KS, EPI>, dim3((unsigned)grid), dim3(kSgThreads), smem, st, p);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "stream_gemm: launch failed: %s", cudaGetErrorString(e));
    return NS_OK;
}

template <int KS, int EPI> static int stream_dispatch_mt(const StreamGemmParams& p, cudaStream_t st) {
    if (p.M <= 16) return launch_stream<1, KS, EPI>(p, st);
    if (p.M <= 32) return launch_stream<2, KS, EPI>(p, st);
    if constexpr (KS * 4 * 4 <= 128) return launch_stream<4, KS, EPI>(p, st);
    return fail(NS_ERR_UNSUPPORTED, "stream_gemm: %d token rows at K=%d exceed the register budget (use the library GEMM)",
                p.M, 128 * KS);
}

template <int EPI> static int stream_dispatch_k(const StreamGemmParams& p, cudaStream_t st) {
    switch (p.K) {
        case 896: return stream_dispatch_mt<7, EPI>(p, st);
        case 1024: return stream_dispatch_mt<8, EPI>(p, st);
        case 1536: return stream_dispatch_mt<12, EPI>(p, st);
        default: return fail(NS_ERR_UNSUPPORTED, "stream_gemm: K=%d is not built (896, 1024, 1536)", p.K);
    }
}

}  // namespace ns

using namespace ns;

extern "C" int ns_stream_gemm(const void* x, const void* residual, const void* ln_w, void* residual_out, const float* ss_in,
                              int32_t ss_parts, const void* w, const void* bias, void* out, const void* add_in, float* ss_out,
                              int32_t M, int32_t N, int32_t K, float eps, int32_t epilogue, void* stream) {
    NS_REQUIRE(M >= 0 && N > 0 && K > 0, NS_ERR_INVALID_ARG, "stream_gemm: bad shape");
    if (M == 0) return NS_OK;
    NS_REQUIRE(x && w && out, NS_ERR_INVALID_ARG, "stream_gemm: null pointer");
    NS_REQUIRE(M <= 64, NS_ERR_UNSUPPORTED, "stream_gemm: %d token rows > 64 (use the library GEMM for large batches)", M);
    NS_REQUIRE(residual == nullptr || ln_w != nullptr, NS_ERR_INVALID_ARG, "stream_gemm: residual needs the norm prologue");
    NS_REQUIRE(ss_in == nullptr || (ln_w != nullptr && residual == nullptr && ss_parts > 0), NS_ERR_INVALID_ARG,
               "stream_gemm: ss_in needs ln_w, ss_parts > 0 and no residual (x is the residual stream already)");
    NS_REQUIRE(N % 16 == 0, NS_ERR_UNSUPPORTED, "stream_gemm: N=%d is not a multiple of 16", N);
    NS_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(residual) |
                 reinterpret_cast<uintptr_t>(ln_w) | reinterpret_cast<uintptr_t>(residual_out)) & 15) == 0,
               NS_ERR_INVALID_ARG, "stream_gemm: x / w / residual / ln_w must be 16-byte aligned");
    StreamGemmParams p;
    p.x = (const __nv_bfloat16*)x; p.residual = (const __nv_bfloat16*)residual; p.ln_w = (const __nv_bfloat16*)ln_w;
    p.residual_out = (__nv_bfloat16*)residual_out; p.w = (const __nv_bfloat16*)w; p.bias = (const __nv_bfloat16*)bias;
    p.out = (__nv_bfloat16*)out; p.M = M; p.N = N; p.K = K; p.inter = N / 2; p.units = N / 16; p.stages = 0; p.eps = eps;
    p.timeline = g_sg_timeline; p.ss_in = ss_in; p.ss_parts = ss_parts; p.add_in = (const __nv_bfloat16*)add_in; p.ss_out = ss_out;
    cudaStream_t st = (cudaStream_t)stream;
    if (epilogue == kSgBias) return stream_dispatch_k<kSgBias>(p, st);
    if (epilogue == kSgSiluMul) {
        NS_REQUIRE(bias == nullptr, NS_ERR_INVALID_ARG, "stream_gemm: the SiLU*mul epilogue takes no bias");
        return stream_dispatch_k<kSgSiluMul>(p, st);
    }
    if (epilogue == kSgResidual) {
        NS_REQUIRE(add_in != nullptr, NS_ERR_INVALID_ARG, "stream_gemm: the residual epilogue needs add_in");
        return stream_dispatch_k<kSgResidual>(p, st);
    }
    return fail(NS_ERR_INVALID_ARG, "stream_gemm: unknown epilogue %d", epilogue);
}

// Debug hook (not part of the public header): clock64 stamps of CTA 0 thread 0 go to `buf` (device memory, 64 slots).
#ifdef NS_DEBUG_HOOKS
extern "C" void ns_debug_stream_gemm_timeline(long long* buf) { g_sg_timeline = buf; }
#endif

namespace ns {
// Device address of this file's error counter on the current device (resolved once per device; the first call on a
// device must come before any stream capture). Used by ns_collect_status.
int stream_gemm_error_counter(const unsigned int** out) {
    static const unsigned int* addr[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(NS_ERR_CUDA, "stream_gemm_error_counter: no current device");
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_stream_gemm_errors);
        if (e != cudaSuccess || p == nullptr) return fail(NS_ERR_CUDA, "stream_gemm_error_counter: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        addr[dev] = static_cast<const unsigned int*>(p);
    }
    *out = addr[dev];
    return NS_OK;
}
}  // namespace ns

extern "C" int ns_stream_gemm_errors(uint32_t* count) {
    NS_REQUIRE(count != nullptr, NS_ERR_INVALID_ARG, "stream_gemm_errors: null pointer");
    cudaError_t e = cudaMemcpyFromSymbol(count, g_stream_gemm_errors, sizeof(uint32_t));
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "stream_gemm_errors: %s", cudaGetErrorString(e));
    return NS_OK;
}

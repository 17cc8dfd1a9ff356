// Per-request sampling on the device: temperature, top-k, top-p (nucleus) and a Gumbel-max draw over one logits row
// per CTA. Stands in for nanoserve/sampling.py:54-90 (`sample`), which builds a torch.Generator per request and step on
// the host and runs topk / sort / softmax / cumsum over [rows, vocab] tensors.
//
// What is kept from the reference, exactly:
//   x = float(logits) / temperature (IEEE division);
//   top-k keeps x >= (k-th largest x), ties at the threshold included;
//   top-p keeps, in descending order of x, every token whose probability mass ranked ABOVE it is < p (softmax over the
//   top-k survivors), so the best token always survives; tokens of equal x are kept or dropped together;
//   token = argmax_j (x_j + g_j), g_j = -log(-log(u_j)), u_j clamped to [1e-20, 1 - 1e-7];
//   the draw of request r's n-th token depends only on mix_seed(seed_r, n) (passed in by the host), the row's logits and
//   its parameters - not on the batch it shares, its row index, or the launch shape.
// What differs: u_j comes from a counter-based generator (one splitmix64 output per (draw seed, token index)) instead of
// the host generator's stream, so individual samples are not bit-equal to the reference's; the distribution is the same.
//
// No sort: the two thresholds are found by radix selection over an order-preserving 32-bit key of x, 8 bits per pass -
// by element COUNT for top-k and by probability MASS for top-p. Masses are integers (exp(x - max) in units of 2^-40), so the
// histogram sums do not depend on the order of the atomic adds and a row's kept set is reproducible bit for bit.
#include "common.cuh"

namespace ns {

struct SampleRow {            // one per logits row; 32 bytes (ns_sample_rows documents the layout)
    float temperature;
    float top_p;
    int32_t top_k;
    int32_t enabled;          // 0: the row keeps the token its greedy argmax produced
    uint32_t seed_lo, seed_hi;
    int32_t pad[2];
};

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// One warp-aggregated histogram update: lanes with equal digits elect a leader that adds the group's total.
__device__ __forceinline__ void hist_count(uint32_t* hist, bool active, uint32_t digit, int lane) {
    const unsigned mask = __ballot_sync(0xffffffffu, active);
    if (active) {
        const unsigned peers = __match_any_sync(mask, digit);
        if (lane == __ffs(peers) - 1) atomicAdd(&hist[digit], (uint32_t)__popc(peers));
    }
}
__device__ __forceinline__ void hist_mass(unsigned long long* hist, bool active, uint32_t digit, uint64_t fx, int lane) {
    const unsigned mask = __ballot_sync(0xffffffffu, active);
    if (active) {
        const unsigned peers = __match_any_sync(mask, digit);
        // fx <= 2^40: two 20-bit limbs whose 32-lane sums fit 32 bits
        const uint32_t lo = __reduce_add_sync(peers, (uint32_t)(fx & 0xFFFFFu));
        const uint32_t hi = __reduce_add_sync(peers, (uint32_t)(fx >> 20));
        if (lane == __ffs(peers) - 1) atomicAdd(&hist[digit], (unsigned long long)lo + ((unsigned long long)hi << 20));
    }
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads) sample_rows_kernel(const T* __restrict__ logits, int64_t row_stride, int vocab,
                                                                     const SampleRow* __restrict__ params, int64_t* __restrict__ out,
                                                                     const int32_t* __restrict__ seat_of,
                                                                     int64_t* __restrict__ last_tokens,
                                                                     float* __restrict__ threshold_out,
                                                                     int32_t* __restrict__ kept_out) {
    const int row_id = blockIdx.x;
    const SampleRow sp = params[row_id];
    if (!sp.enabled) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* row = logits + (int64_t)row_id * row_stride;
    const float temp = sp.temperature;
    auto x_at = [&](int i) { return __fdiv_rn(to_f32(row[i]), temp); };

    __shared__ uint32_t cnt[256];
    __shared__ unsigned long long mass[256];
    __shared__ float redf[32];
    __shared__ int redi[32];
    __shared__ unsigned long long redu[32];
    __shared__ uint32_t s_prefix;
    __shared__ uint32_t s_k;
    __shared__ unsigned long long s_above;
    __shared__ float s_max;
    __shared__ unsigned long long s_total;

    // ---- row maximum of x (the softmax shift) ------------------------------------------------------------------------
    float m = -INFINITY;
    for (int i = tid; i < vocab; i += kSampleThreads) m = fmaxf(m, x_at(i));
    m = warp_max(m);
    if (lane == 0) redf[warp] = m;
    __syncthreads();
    if (warp == 0) {
        m = warp_max(redf[lane]);
        if (lane == 0) s_max = m;
    }
    __syncthreads();
    m = s_max;

    // ---- top-k: key of the k-th largest x, by radix selection on counts -------------------------------------------------
    uint32_t key_k = 0;                                     // every key is >= 0: nothing dropped
    if (sp.top_k > 0 && sp.top_k < vocab) {
        if (tid == 0) { s_prefix = 0; s_k = (uint32_t)sp.top_k; }
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) cnt[tid] = 0;
            __syncthreads();
            const uint32_t prefix = s_prefix;
            for (int base = 0; base < vocab; base += kSampleThreads) {
                const int i = base + tid;
                uint32_t key = 0;
                bool active = i < vocab;
                if (active) {
                    key = order_key(x_at(i));
                    active = shift == 24 || (key >> (shift + 8)) == prefix;
                }
                hist_count(cnt, active, (key >> shift) & 255u, lane);
            }
            __syncthreads();
            if (tid == 0) {
                uint32_t need = s_k, seen = 0;
                int d = 255;
                for (; d > 0; --d) {
                    if (seen + cnt[d] >= need) break;
                    seen += cnt[d];
                }
                s_k = need - seen;
                s_prefix = (prefix << 8) | (uint32_t)d;
            }
            __syncthreads();
        }
        key_k = s_prefix;
    }

    // ---- top-p: key of the lowest token whose mass ranked above it is < p, by radix selection on mass -------------------
    uint32_t key_p = 0;
    if (sp.top_p < 1.0f) {
        auto fixed_mass = [&](float x) { return (uint64_t)__float2ull_rn(expf(x - m) * 1099511627776.0f); };   // 2^40
        unsigned long long z = 0;
        for (int i = tid; i < vocab; i += kSampleThreads) {
            const float x = x_at(i);
            if (order_key(x) >= key_k) z += fixed_mass(x);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
        if (lane == 0) redu[warp] = z;
        __syncthreads();
        if (tid == 0) {
            unsigned long long t = 0;
            for (int w = 0; w < kSampleThreads / 32; ++w) t += redu[w];
            s_total = t;
            s_prefix = 0;
            s_above = 0;
        }
        __syncthreads();
        const double limit = (double)sp.top_p * (double)s_total;      // "mass above >= p" drops a token
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) mass[tid] = 0;
            __syncthreads();
            const uint32_t prefix = s_prefix;
            for (int base = 0; base < vocab; base += kSampleThreads) {
                const int i = base + tid;
                uint32_t key = 0;
                uint64_t fx = 0;
                bool active = i < vocab;
                if (active) {
                    const float x = x_at(i);
                    key = order_key(x);
                    active = key >= key_k && (shift == 24 || (key >> (shift + 8)) == prefix);
                    if (active) {
                        fx = fixed_mass(x);
                        active = fx != 0;
                    }
                }
                hist_mass(mass, active, (key >> shift) & 255u, fx, lane);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long above = s_above, chosen_above = s_above;
                int chosen = -1;
                for (int d = 255; d >= 0; --d) {
                    if ((double)above >= limit) break;
                    if (mass[d] != 0) { chosen = d; chosen_above = above; }
                    above += mass[d];
                }
                if (chosen < 0) chosen = 255;              // cannot happen: the best token's bin has mass and above == 0 < limit
                s_above = chosen_above;
                s_prefix = (prefix << 8) | (uint32_t)chosen;
            }
            __syncthreads();
        }
        key_p = s_prefix;
    }
    const uint32_t key_min = key_k > key_p ? key_k : key_p;

    // ---- Gumbel-max over the survivors -------------------------------------------------------------------------------
    const uint64_t seed = ((uint64_t)sp.seed_hi << 32) | sp.seed_lo;
    float best = -INFINITY;
    int best_i = 0x7fffffff, kept = 0;
    for (int i = tid; i < vocab; i += kSampleThreads) {
        const float x = x_at(i);
        if (order_key(x) < key_min) continue;
        ++kept;
        const uint64_t bits = splitmix64(seed + (uint64_t)(i + 1) * 0x9E3779B97F4A7C15ull);
        float u = (float)(bits >> 40) * 5.9604644775390625e-08f + 2.98023223876953125e-08f;      // (n + 0.5) / 2^24
        u = fminf(fmaxf(u, 1e-20f), 0.99999988f);
        const float score = x - logf(-logf(u));
        if (score > best || (score == best && i < best_i)) { best = score; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        kept += __shfl_xor_sync(0xffffffffu, kept, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    __syncthreads();                                       // redf was read above by warp 0
    if (lane == 0) { redf[warp] = best; redi[warp] = best_i; redu[warp] = (unsigned long long)kept; }
    __syncthreads();
    if (tid == 0) {
        int total = 0;
        for (int w = 0; w < kSampleThreads / 32; ++w) {
            total += (int)redu[w];
            if (redf[w] > best || (redf[w] == best && redi[w] < best_i)) { best = redf[w]; best_i = redi[w]; }
        }
        const int64_t tok = best_i == 0x7fffffff ? 0 : best_i;
        out[row_id] = tok;
        if (seat_of != nullptr) last_tokens[seat_of[row_id]] = tok;
        if (threshold_out != nullptr) threshold_out[row_id] = key_value(key_min == 0 ? order_key(-INFINITY) : key_min);
        if (kept_out != nullptr) kept_out[row_id] = total;
    }
}

}  // namespace ns

using namespace ns;

extern "C" int ns_sample_rows(const void* logits, int64_t row_stride, int32_t rows, int32_t vocab, const void* params,
                              int64_t* out, const int32_t* seat_of, int64_t* last_tokens, float* threshold_out,
                              int32_t* kept_out, int dtype, void* stream) {
    NS_REQUIRE(logits && params && out, NS_ERR_INVALID_ARG, "sample_rows: null pointer");
    NS_REQUIRE(rows >= 0 && vocab > 0, NS_ERR_INVALID_ARG, "sample_rows: bad shape");
    NS_REQUIRE(seat_of == nullptr || last_tokens != nullptr, NS_ERR_INVALID_ARG, "sample_rows: seat_of without last_tokens");
    NS_REQUIRE((reinterpret_cast<uintptr_t>(params) & 15) == 0, NS_ERR_INVALID_ARG, "sample_rows: params must be 16-byte aligned");
    static_assert(sizeof(SampleRow) == 32, "ns_sample_rows documents 8 x 32-bit words per row");
    if (rows == 0) return NS_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const SampleRow* sp = static_cast<const SampleRow*>(params);
    if (dtype == NS_BF16)
        sample_rows_kernel<__nv_bfloat16><<<rows, kSampleThreads, 0, st>>>((const __nv_bfloat16*)logits, row_stride, vocab, sp, out,
                                                                            seat_of, last_tokens, threshold_out, kept_out);
    else if (dtype == NS_F32)
        sample_rows_kernel<float><<<rows, kSampleThreads, 0, st>>>((const float*)logits, row_stride, vocab, sp, out, seat_of,
                                                                   last_tokens, threshold_out, kept_out);
    else
        return fail(NS_ERR_UNSUPPORTED, "sample_rows: dtype %d", dtype);
    return check_launch("sample_rows");
}

// Token-wise fused ops: residual-add + RMSNorm, SiLU*mul, RoPE cos/sin tables, RoPE + paged KV write.
//
// All four are HBM-bound streaming kernels: 16-byte vector loads/stores, one pass over the data, and the
// rounding points of the unfused framework ops kept (round to the storage dtype after every elementwise op
// the reference performs in that dtype), so bf16 results agree with the unfused path bit for bit except
// where an fp32 sum is accumulated in another order.
#include "common.cuh"

namespace ns {

// ------------------------------------------------------------------------------------------------ RMSNorm
// One CTA per row. Each thread keeps its (up to MAXC) 16-byte chunks of the row in registers between the
// sum-of-squares pass and the scaling pass, so the row is read exactly once.
template <typename T, bool HAS_RES, int MAXC>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ res,
                                                           const T* __restrict__ w, T* __restrict__ out,
                                                           T* __restrict__ res_out, int hidden, float eps) {
    constexpr int V = Vec16<T>::N;
    const int64_t row = blockIdx.x;
    const int chunks = hidden / V;
    pdl_launch_dependents();
    pdl_wait();
    const T* xr = x + row * hidden;
    Vec16<T> vals[MAXC];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            Vec16<T> v = load16(xr + c * V);
            if (HAS_RES) {
                Vec16<T> r = load16(res + row * hidden + c * V);
#pragma unroll
                for (int j = 0; j < V; ++j) v.set(j, r.get(j) + v.get(j));   // rounded to T: the framework's `res + x`
                store16(res_out + row * hidden + c * V, v);
            }
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const float f = v.get(j);
                ss = fmaf(f, f, ss);
            }
            vals[i] = v;
        }
    }
    __shared__ float warp_part[32];
    __shared__ float total;
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = (threadIdx.x < (blockDim.x + 31) / 32) ? warp_part[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) total = t;
    }
    __syncthreads();
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            Vec16<T> wv = load16(w + c * V);
            Vec16<T> o;
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const float y = round_to<T>(vals[i].get(j) * inv);   // cast back BEFORE the weight multiply
                o.set(j, wv.get(j) * y);
            }
            store16(out + row * hidden + c * V, o);
        }
    }
}

template <typename T>
static int launch_add_rmsnorm(const void* x, const void* res, const void* w, void* out, void* res_out, int64_t rows,
                              int hidden, float eps, cudaStream_t st) {
    constexpr int V = Vec16<T>::N;
    constexpr int MAXC = 4;
    NS_REQUIRE(hidden % V == 0, NS_ERR_UNSUPPORTED, "add_rmsnorm: hidden=%d is not a multiple of %d", hidden, V);
    const int chunks = hidden / V;
    int threads = ((chunks + 31) / 32) * 32;
    if (threads > 1024) threads = 1024;
    NS_REQUIRE(chunks <= threads * MAXC, NS_ERR_UNSUPPORTED, "add_rmsnorm: hidden=%d too wide", hidden);
    if (rows == 0) return NS_OK;
    dim3 grid((unsigned)rows);
    if (res != nullptr)
        launch_pdl(add_rmsnorm_kernel<T, true, MAXC>, grid, dim3(threads), 0, st, (const T*)x, (const T*)res, (const T*)w,
                   (T*)out, (T*)res_out, hidden, eps);
    else
        launch_pdl(add_rmsnorm_kernel<T, false, MAXC>, grid, dim3(threads), 0, st, (const T*)x, (const T*)nullptr,
                   (const T*)w, (T*)out, (T*)nullptr, hidden, eps);
    return check_launch("add_rmsnorm");
}

// ------------------------------------------------------------------------------------------------ SiLU * mul
template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t rows,
                                                       int inter) {
    constexpr int V = Vec16<T>::N;
    const int cpr = inter / V;                       // chunks per row
    const int64_t total = rows * cpr;
    pdl_launch_dependents();          // down_proj may start streaming its weights while this kernel runs
    pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cpr;
        const int c = (int)(i - r * cpr);
        const T* base = gu + r * 2 * (int64_t)inter + c * V;
        Vec16<T> g = load16(base);
        Vec16<T> u = load16(base + inter);
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float gf = g.get(j);
            const float s = round_to<T>(gf / (1.0f + expf(-gf)));   // silu in fp32, rounded like F.silu's output
            o.set(j, s * u.get(j));
        }
        store16(out + r * (int64_t)inter + c * V, o);
    }
}

// ------------------------------------------------------------------------------------------------ RoPE tables
template <typename T>
__global__ void rope_cos_sin_kernel(const int64_t* __restrict__ pos, const float* __restrict__ inv_freq,
                                    T* __restrict__ cos_out, T* __restrict__ sin_out, int64_t n, int hd) {
    const int half = hd / 2;
    const int64_t total = n * half;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / half;
        const int d = (int)(i - t * half);
        const float ang = __fmul_rn((float)pos[t], inv_freq[d]);
        float s, c;
        sincosf(ang, &s, &c);
        const T cv = from_f32<T>(c), sv = from_f32<T>(s);
        cos_out[t * hd + d] = cv;
        cos_out[t * hd + half + d] = cv;
        sin_out[t * hd + d] = sv;
        sin_out[t * hd + half + d] = sv;
    }
}

// ------------------------------------------------------------------------------------------------ RoPE + KV write
// Work unit = (token, head, 16-byte chunk of the low half). Heads 0..NH-1 are queries, NH..NH+NKV-1 keys,
// the last NKV values. rotate_half(x) = [-x_hi, x_lo]:
//   out_lo = rnd(rnd(x_lo*cos_lo) - rnd(x_hi*sin_lo)),  out_hi = rnd(rnd(x_hi*cos_hi) + rnd(x_lo*sin_hi)).
// __fmul_rn / __fadd_rn keep the compiler from contracting a product into the following add.
template <typename T>
__global__ void __launch_bounds__(256) rope_qkv_kernel(const T* __restrict__ qkv, const T* __restrict__ cosT,
                                                       const T* __restrict__ sinT, T* __restrict__ q_out,
                                                       T* __restrict__ k_out, T* __restrict__ v_out,
                                                       T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                       const int64_t* __restrict__ slots, int64_t n_tokens, int NH,
                                                       int NKV, int HD) {
    constexpr int V = Vec16<T>::N;
    const int half = HD / 2;
    const int cph = half / V;                         // chunks per head (low half)
    const int heads = NH + 2 * NKV;
    const int64_t total = n_tokens * heads * cph;
    const int W = heads * HD;
    pdl_launch_dependents();          // the attention kernel that follows may get scheduled while this one runs
    pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % cph);
        const int64_t th = i / cph;
        const int h = (int)(th % heads);
        const int64_t t = th / heads;
        const T* src = qkv + t * W + h * HD + c * V;
        Vec16<T> lo = load16(src), hi = load16(src + half);
        if (h < NH + NKV) {
            const T* cp = cosT + t * HD + c * V;
            const T* sp = sinT + t * HD + c * V;
            Vec16<T> cl = load16(cp), ch = load16(cp + half), sl = load16(sp), sh = load16(sp + half);
            Vec16<T> olo, ohi;
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const float xl = lo.get(j), xh = hi.get(j);
                const float a = round_to<T>(__fmul_rn(xl, cl.get(j)));
                const float b = round_to<T>(__fmul_rn(xh, sl.get(j)));
                const float d = round_to<T>(__fmul_rn(xh, ch.get(j)));
                const float e = round_to<T>(__fmul_rn(xl, sh.get(j)));
                olo.set(j, __fadd_rn(a, -b));
                ohi.set(j, __fadd_rn(d, e));
            }
            lo = olo;
            hi = ohi;
        }
        if (h < NH) {
            if (q_out != nullptr) {
                T* dst = q_out + (t * NH + h) * HD + c * V;
                store16(dst, lo);
                store16(dst + half, hi);
            }
        } else {
            const bool is_k = h < NH + NKV;
            const int g = is_k ? h - NH : h - NH - NKV;
            T* dense = is_k ? k_out : v_out;
            if (dense != nullptr) {
                T* dst = dense + (t * NKV + g) * HD + c * V;
                store16(dst, lo);
                store16(dst + half, hi);
            }
            T* cache = is_k ? k_cache : v_cache;
            if (cache != nullptr) {
                T* dst = cache + (slots[t] * NKV + g) * HD + c * V;
                store16(dst, lo);
                store16(dst + half, hi);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ plain KV write
template <typename T>
__global__ void __launch_bounds__(256) kv_write_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new,
                                                       T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                       const int64_t* __restrict__ slots, int64_t n_tokens,
                                                       int row_elems) {
    constexpr int V = Vec16<T>::N;
    const int cpr = row_elems / V;
    const int64_t total = n_tokens * cpr;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / cpr;
        const int c = (int)(i - t * cpr);
        const int64_t dst = slots[t] * row_elems + c * V;
        store16(k_cache + dst, load16(k_new + t * row_elems + c * V));
        store16(v_cache + dst, load16(v_new + t * row_elems + c * V));
    }
}

// Grid of a grid-stride kernel: enough CTAs for the work, at most 8 resident CTAs per SM of the current device.
static inline unsigned grid_for(int64_t work_items, int threads) {
    int sms = device_sm_count();
    if (sms <= 0) sms = 148;
    const int max_ctas = sms * 8;
    int64_t g = (work_items + threads - 1) / threads;
    if (g < 1) g = 1;
    if (g > max_ctas) g = max_ctas;
    return (unsigned)g;
}

template <typename T>
static int launch_silu_mul(const void* gu, void* out, int64_t rows, int inter, cudaStream_t st) {
    constexpr int V = Vec16<T>::N;
    NS_REQUIRE(inter % V == 0, NS_ERR_UNSUPPORTED, "silu_mul: width %d is not a multiple of %d", inter, V);
    if (rows == 0) return NS_OK;
    launch_pdl(silu_mul_kernel<T>, dim3(grid_for(rows * (inter / V), 256)), dim3(256), 0, st, (const T*)gu, (T*)out, rows, inter);
    return check_launch("silu_mul");
}

template <typename T>
static int launch_rope(const void* qkv, const void* c, const void* s, void* q, void* k, void* v, void* kc, void* vc,
                       const int64_t* slots, int64_t n, int NH, int NKV, int HD, cudaStream_t st) {
    constexpr int V = Vec16<T>::N;
    NS_REQUIRE(HD % (2 * V) == 0, NS_ERR_UNSUPPORTED, "rope_qkv: head_dim=%d is not a multiple of %d", HD, 2 * V);
    if (n == 0) return NS_OK;
    const int64_t work = n * (NH + 2 * NKV) * (HD / 2 / V);
    launch_pdl(rope_qkv_kernel<T>, dim3(grid_for(work, 256)), dim3(256), 0, st, (const T*)qkv, (const T*)c, (const T*)s,
               (T*)q, (T*)k, (T*)v, (T*)kc, (T*)vc, slots, n, NH, NKV, HD);
    return check_launch("rope_qkv_kvwrite");
}

}  // namespace ns

using namespace ns;

extern "C" int ns_add_rmsnorm(const void* x, const void* residual, const void* weight, void* out, void* residual_out,
                              int64_t rows, int32_t hidden, float eps, int dtype, void* stream) {
    NS_REQUIRE(rows >= 0 && hidden > 0, NS_ERR_INVALID_ARG, "add_rmsnorm: bad shape %lld x %d", (long long)rows, hidden);
    if (rows == 0) return NS_OK;
    NS_REQUIRE(x && weight && out, NS_ERR_INVALID_ARG, "add_rmsnorm: null pointer");
    NS_REQUIRE(residual == nullptr || residual_out != nullptr, NS_ERR_INVALID_ARG,
               "add_rmsnorm: residual given without residual_out");
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == NS_BF16) return launch_add_rmsnorm<__nv_bfloat16>(x, residual, weight, out, residual_out, rows, hidden, eps, st);
    if (dtype == NS_F32) return launch_add_rmsnorm<float>(x, residual, weight, out, residual_out, rows, hidden, eps, st);
    return fail(NS_ERR_UNSUPPORTED, "add_rmsnorm: dtype %d", dtype);
}

extern "C" int ns_silu_mul(const void* gate_up, void* out, int64_t rows, int32_t inter, int dtype, void* stream) {
    NS_REQUIRE(rows >= 0 && inter > 0, NS_ERR_INVALID_ARG, "silu_mul: bad shape");
    if (rows == 0) return NS_OK;
    NS_REQUIRE(gate_up && out, NS_ERR_INVALID_ARG, "silu_mul: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == NS_BF16) return launch_silu_mul<__nv_bfloat16>(gate_up, out, rows, inter, st);
    if (dtype == NS_F32) return launch_silu_mul<float>(gate_up, out, rows, inter, st);
    return fail(NS_ERR_UNSUPPORTED, "silu_mul: dtype %d", dtype);
}

extern "C" int ns_rope_cos_sin(const int64_t* positions, const float* inv_freq, void* cos_out, void* sin_out,
                               int64_t n_tokens, int32_t head_dim, int dtype, void* stream) {
    NS_REQUIRE(n_tokens >= 0 && head_dim > 0 && head_dim % 2 == 0, NS_ERR_INVALID_ARG, "rope_cos_sin: bad shape");
    if (n_tokens == 0) return NS_OK;
    NS_REQUIRE(positions && inv_freq && cos_out && sin_out, NS_ERR_INVALID_ARG, "rope_cos_sin: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = grid_for(n_tokens * (head_dim / 2), 256);
    if (dtype == NS_BF16)
        rope_cos_sin_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(positions, inv_freq, (__nv_bfloat16*)cos_out,
                                                                 (__nv_bfloat16*)sin_out, n_tokens, head_dim);
    else if (dtype == NS_F32)
        rope_cos_sin_kernel<float><<<grid, 256, 0, st>>>(positions, inv_freq, (float*)cos_out, (float*)sin_out,
                                                         n_tokens, head_dim);
    else
        return fail(NS_ERR_UNSUPPORTED, "rope_cos_sin: dtype %d", dtype);
    return check_launch("rope_cos_sin");
}

extern "C" int ns_rope_qkv_kvwrite(const void* qkv, const void* cos, const void* sin, void* q_out, void* k_out,
                                   void* v_out, void* k_cache, void* v_cache, const int64_t* slots, int64_t n_tokens,
                                   int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, int dtype, void* stream) {
    NS_REQUIRE(n_tokens >= 0, NS_ERR_INVALID_ARG, "rope_qkv: bad shape");
    if (n_tokens == 0) return NS_OK;
    NS_REQUIRE(qkv && cos && sin, NS_ERR_INVALID_ARG, "rope_qkv: null pointer");
    NS_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), NS_ERR_INVALID_ARG, "rope_qkv: need both caches or none");
    NS_REQUIRE(k_cache == nullptr || slots != nullptr, NS_ERR_INVALID_ARG, "rope_qkv: cache given without slots");
    NS_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0, NS_ERR_INVALID_ARG, "rope_qkv: bad shape");
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == NS_BF16)
        return launch_rope<__nv_bfloat16>(qkv, cos, sin, q_out, k_out, v_out, k_cache, v_cache, slots, n_tokens, n_heads, n_kv_heads, head_dim, st);
    if (dtype == NS_F32)
        return launch_rope<float>(qkv, cos, sin, q_out, k_out, v_out, k_cache, v_cache, slots, n_tokens, n_heads, n_kv_heads, head_dim, st);
    return fail(NS_ERR_UNSUPPORTED, "rope_qkv: dtype %d", dtype);
}

extern "C" int ns_kv_write(const void* k_new, const void* v_new, void* k_cache, void* v_cache, const int64_t* slots,
                           int64_t n_tokens, int32_t row_elems, int dtype, void* stream) {
    NS_REQUIRE(n_tokens >= 0 && row_elems > 0, NS_ERR_INVALID_ARG, "kv_write: bad shape");
    if (n_tokens == 0) return NS_OK;
    NS_REQUIRE(k_new && v_new && k_cache && v_cache && slots, NS_ERR_INVALID_ARG, "kv_write: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == NS_BF16) {
        NS_REQUIRE(row_elems % 8 == 0, NS_ERR_UNSUPPORTED, "kv_write: row of %d bf16 is not a multiple of 16 bytes", row_elems);
        kv_write_kernel<__nv_bfloat16><<<grid_for(n_tokens * (row_elems / 8), 256), 256, 0, st>>>(
            (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
            slots, n_tokens, row_elems);
    } else if (dtype == NS_F32) {
        NS_REQUIRE(row_elems % 4 == 0, NS_ERR_UNSUPPORTED, "kv_write: row of %d f32 is not a multiple of 16 bytes", row_elems);
        kv_write_kernel<float><<<grid_for(n_tokens * (row_elems / 4), 256), 256, 0, st>>>(
            (const float*)k_new, (const float*)v_new, (float*)k_cache, (float*)v_cache, slots, n_tokens, row_elems);
    } else {
        return fail(NS_ERR_UNSUPPORTED, "kv_write: dtype %d", dtype);
    }
    return check_launch("kv_write");
}

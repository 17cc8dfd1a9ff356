// Tensor parallelism: one-shot all-reduce over peer memory fused with the residual add and the RMSNorm that follow it.
//
// The two all-reduce sites of a layer (after o_proj and after down_proj, nanoserve/model.py:256-257) are each followed
// by "x = x + a; h = rmsnorm(x)". With NCCL that is a collective (about 15 us for the 0.46 MB of a 64-row decode step)
// and then a separate kernel. Here every rank's GEMM writes its partial [rows, hidden] into a buffer the other GPUs can
// read over NVLink (peer-mapped), and ONE kernel per rank
//   1. tells every peer "my partial of call c is complete" (a release store of c into slot `rank` of each peer's flags),
//   2. waits until its own flags say the same of every peer (bounded spin on LOCAL memory),
//   3. reads the W partials row by row with ordinary 16-byte loads (its own from HBM, the peers' over NVLink), sums them
//      in fp32 in rank order - the same order on every rank, so the result is bitwise identical everywhere, which the
//      lock-step schedulers rely on -, rounds the sum to bf16 (what an all-reduce of bf16 tensors returns), adds the
//      residual, and applies the RMSNorm with the reference's rounding points (fused.py:33-42).
// No TMA, no multicast, no bulk copy touches a peer's memory: plain ld.global only. Partials are double buffered by the
// caller (two buffers used in turn): rank r can only get to call c+2, which overwrites call c's buffer, after every
// peer has signalled call c+1, i.e. finished reading call c. The call number lives on the device (a CUDA graph replays
// the same launch with the same arguments); the last CTA to finish advances it.
// A wait that runs out (a peer that never arrives) is counted (ns_collect_status), the kernel goes on and returns: its
// results are then undefined, the context stays usable.
#include <cstring>

#include "common.cuh"

namespace ns {

constexpr int kTpMaxWorld = 8;
constexpr uint32_t kTpSpinLimit = 1u << 22;       // x ~50 ns: about a fifth of a second

__device__ unsigned int g_tp_errors = 0;

struct TpPeers {
    const __nv_bfloat16* partial[kTpMaxWorld];    // rank r's partial for this call, as mapped in THIS process
    uint32_t* flags[kTpMaxWorld];                 // rank r's flag array [world], as mapped in this process
};

__device__ __forceinline__ uint4 ld_peer16(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// state[0] = number of completed calls, state[1] = CTAs of the current call that have finished
template <int WORLD>
__global__ void __launch_bounds__(512) tp_allreduce_add_rmsnorm_kernel(TpPeers peers, uint32_t* __restrict__ state,
                                                                       const __nv_bfloat16* __restrict__ residual,
                                                                       const __nv_bfloat16* __restrict__ weight,
                                                                       __nv_bfloat16* __restrict__ out_h,
                                                                       __nv_bfloat16* __restrict__ out_x, int hidden, float eps,
                                                                       int rank) {
    const int row = blockIdx.x, tid = threadIdx.x;
    const uint32_t call = *reinterpret_cast<volatile uint32_t*>(state) + 1;
    __shared__ int gave_up;
    if (tid == 0) gave_up = 0;
    __syncthreads();
    // 1. announce (one CTA does it: the partial was written by the kernel before this one in the stream)
    if (row == 0 && tid < WORLD) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[tid] + rank), "r"(call) : "memory");
    }
    // 2. wait for every peer's announcement of this call (flags only grow)
    if (tid < WORLD) {
        const uint32_t* f = peers.flags[rank] + tid;
        uint32_t seen = 0, spins = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
            if ((int32_t)(seen - call) >= 0) break;
            if (++spins > kTpSpinLimit) {
                gave_up = 1;
                break;
            }
            __nanosleep(40);
        }
    }
    __syncthreads();
    if (gave_up && tid == 0) atomicAdd(&g_tp_errors, 1u);

    // 3. sum, residual, norm: one 16-byte chunk per thread (hidden / 8 threads)
    const int chunks = hidden / 8;
    float r[8];
    float ss = 0.f;
    const bool mine = tid < chunks;
    if (mine) {
        const int64_t off = (int64_t)row * hidden + 8 * tid;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
        for (int w = 0; w < WORLD; ++w) {
            const uint4 raw = ld_peer16(peers.partial[w] + off);
            const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += __bfloat162float(v[i]);
        }
        const uint4 rraw = *reinterpret_cast<const uint4*>(residual + off);
        const __nv_bfloat16* rv = reinterpret_cast<const __nv_bfloat16*>(&rraw);
        uint4 xraw;
        __nv_bfloat16* xv = reinterpret_cast<__nv_bfloat16*>(&xraw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float a = round_to<__nv_bfloat16>(acc[i]);                   // the all-reduced bf16 value
            xv[i] = __float2bfloat16_rn(__bfloat162float(rv[i]) + a);           // r = residual + a, rounded
            r[i] = __bfloat162float(xv[i]);
            ss = fmaf(r[i], r[i], ss);
        }
        *reinterpret_cast<uint4*>(out_x + off) = xraw;
    }
    __shared__ float red[16];
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid < 32) {
        float t = tid < (int)(blockDim.x >> 5) ? red[tid] : 0.f;
        t = warp_sum(t);
        if (tid == 0) red[0] = t;
    }
    __syncthreads();
    if (mine) {
        const float rstd = rsqrtf(red[0] / (float)hidden + eps);
        const uint4 wraw = *reinterpret_cast<const uint4*>(weight + 8 * tid);
        const __nv_bfloat16* wv = reinterpret_cast<const __nv_bfloat16*>(&wraw);
        uint4 hraw;
        __nv_bfloat16* hv = reinterpret_cast<__nv_bfloat16*>(&hraw);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            hv[i] = __float2bfloat16_rn(__bfloat162float(wv[i]) * round_to<__nv_bfloat16>(r[i] * rstd));
        *reinterpret_cast<uint4*>(out_h + (int64_t)row * hidden + 8 * tid) = hraw;
    }
    // 4. the last CTA to finish closes the call
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned done = atomicAdd(state + 1, 1u) + 1;
        if (done == gridDim.x) {
            state[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(state) = call;
        }
    }
}

int tp_error_counter(const unsigned int** out) {
    static const unsigned int* addr[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(NS_ERR_CUDA, "tp_error_counter: no current device");
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_tp_errors);
        if (e != cudaSuccess || p == nullptr) return fail(NS_ERR_CUDA, "tp_error_counter: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        addr[dev] = static_cast<const unsigned int*>(p);
    }
    *out = addr[dev];
    return NS_OK;
}

}  // namespace ns

using namespace ns;

extern "C" int ns_tp_allreduce_add_rmsnorm(const void* const* peer_partials, void* const* peer_flags, void* state,
                                           const void* residual, const void* weight, void* out_h, void* out_x, int64_t rows,
                                           int32_t hidden, float eps, int32_t rank, int32_t world, void* stream) {
    NS_REQUIRE(peer_partials && peer_flags && state && residual && weight && out_h && out_x, NS_ERR_INVALID_ARG,
               "tp_allreduce_add_rmsnorm: null pointer");
    NS_REQUIRE(world == 2 || world == 4 || world == 8, NS_ERR_UNSUPPORTED, "tp_allreduce_add_rmsnorm: world size %d (2, 4 or 8)", world);
    NS_REQUIRE(rank >= 0 && rank < world, NS_ERR_INVALID_ARG, "tp_allreduce_add_rmsnorm: rank %d of %d", rank, world);
    NS_REQUIRE(hidden > 0 && hidden % 8 == 0 && hidden / 8 <= 512, NS_ERR_UNSUPPORTED,
               "tp_allreduce_add_rmsnorm: hidden %d (a multiple of 8, at most 4096)", hidden);
    NS_REQUIRE(rows >= 0 && rows <= 65535, NS_ERR_INVALID_ARG, "tp_allreduce_add_rmsnorm: %lld rows", (long long)rows);
    if (rows == 0) return NS_OK;
    TpPeers peers;
    for (int w = 0; w < world; ++w) {
        NS_REQUIRE(peer_partials[w] != nullptr && peer_flags[w] != nullptr, NS_ERR_INVALID_ARG,
                   "tp_allreduce_add_rmsnorm: peer %d has no buffer", w);
        NS_REQUIRE((reinterpret_cast<uintptr_t>(peer_partials[w]) & 15) == 0, NS_ERR_INVALID_ARG,
                   "tp_allreduce_add_rmsnorm: partials must be 16-byte aligned");
        peers.partial[w] = static_cast<const __nv_bfloat16*>(peer_partials[w]);
        peers.flags[w] = static_cast<uint32_t*>(peer_flags[w]);
    }
    const int threads = ((hidden / 8 + 31) / 32) * 32;
    cudaStream_t st = (cudaStream_t)stream;
    auto args = [&](auto kernel) {
        kernel<<<(unsigned)rows, threads, 0, st>>>(peers, static_cast<uint32_t*>(state), (const __nv_bfloat16*)residual,
                                                   (const __nv_bfloat16*)weight, (__nv_bfloat16*)out_h, (__nv_bfloat16*)out_x,
                                                   hidden, eps, rank);
    };
    if (world == 2) args(tp_allreduce_add_rmsnorm_kernel<2>);
    else if (world == 4) args(tp_allreduce_add_rmsnorm_kernel<4>);
    else args(tp_allreduce_add_rmsnorm_kernel<8>);
    return check_launch("tp_allreduce_add_rmsnorm");
}

// ---- set-up of peer-visible buffers (NOT on the serving path: these four calls allocate, map and free) -------------
// One process per GPU: a rank allocates its partial buffers and flags with ns_peer_alloc (zero-filled), exports a handle,
// the handles travel through the host (any channel: the caller's process group), and every other rank maps them with
// ns_peer_open, which also enables peer access from the calling process's current device to the exporting GPU.
extern "C" int ns_peer_alloc(int64_t bytes, void** ptr) {
    NS_REQUIRE(ptr != nullptr && bytes > 0, NS_ERR_INVALID_ARG, "peer_alloc: bad arguments");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "peer_alloc: cudaMalloc(%lld): %s", (long long)bytes, cudaGetErrorString(e));
    e = cudaMemset(p, 0, (size_t)bytes);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(NS_ERR_CUDA, "peer_alloc: cudaMemset: %s", cudaGetErrorString(e));
    }
    *ptr = p;
    return NS_OK;
}

extern "C" int ns_peer_free(void* ptr) {
    if (ptr == nullptr) return NS_OK;
    const cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "peer_free: %s", cudaGetErrorString(e));
    return NS_OK;
}

extern "C" int ns_peer_export(void* ptr, void* handle64) {
    NS_REQUIRE(ptr != nullptr && handle64 != nullptr, NS_ERR_INVALID_ARG, "peer_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    const cudaError_t e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), ptr);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "peer_export: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    return NS_OK;
}

extern "C" int ns_peer_open(const void* handle64, void** ptr) {
    NS_REQUIRE(handle64 != nullptr && ptr != nullptr, NS_ERR_INVALID_ARG, "peer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "peer_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    *ptr = p;
    return NS_OK;
}

extern "C" int ns_peer_close(void* ptr) {
    if (ptr == nullptr) return NS_OK;
    const cudaError_t e = cudaIpcCloseMemHandle(ptr);
    if (e != cudaSuccess) return fail(NS_ERR_CUDA, "peer_close: cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
    return NS_OK;
}

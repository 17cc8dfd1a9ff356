// Shared device helpers for the nanoserve_b200 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nanoserve_b200.h"

namespace ns {

// ---- host-side error plumbing (c_api.cu owns the storage) -------------------------------------------------
int fail(int status, const char* fmt, ...);
int check_launch(const char* what);
int device_sm_count();      // SMs of the current device; <= 0 when none can be queried

#define NS_REQUIRE(cond, status, ...)                 \
    do {                                              \
        if (!(cond)) return ns::fail(status, __VA_ARGS__); \
    } while (0)

// The dynamic shared-memory opt-in (cudaFuncAttributeMaxDynamicSharedMemorySize) is a per-DEVICE attribute of a kernel:
// a process that drives several GPUs has to repeat it on each one. One static instance per launcher remembers, per
// device ordinal, the largest size already opted in.
constexpr int kMaxDevices = 64;
struct SmemOptIn {
    size_t have[kMaxDevices] = {};
    int dev = -1;
    bool needs(size_t smem) {
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { dev = -1; return true; }
        return smem > have[dev];
    }
    void done(size_t smem) { if (dev >= 0) have[dev] = smem; }
};

// ---- scalar conversions -------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Round an fp32 value to the storage dtype and back: the "rounding point" of an unfused framework op.
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

// ---- vector access: 16 bytes per thread ------------------------------------------------------------------
template <typename T> struct Vec16;
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    uint4 raw;
    __device__ __forceinline__ float get(int i) const {
        const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(&raw);
        return __bfloat162float(p[i]);
    }
    __device__ __forceinline__ void set(int i, float v) {
        __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(&raw);
        p[i] = __float2bfloat16_rn(v);
    }
};
template <> struct Vec16<float> {
    static constexpr int N = 4;
    uint4 raw;
    __device__ __forceinline__ float get(int i) const { return reinterpret_cast<const float*>(&raw)[i]; }
    __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<float*>(&raw)[i] = v; }
};

template <typename T> __device__ __forceinline__ Vec16<T> load16(const T* p) {
    Vec16<T> v;
    v.raw = *reinterpret_cast<const uint4*>(p);
    return v;
}
template <typename T> __device__ __forceinline__ void store16(T* p, const Vec16<T>& v) {
    *reinterpret_cast<uint4*>(p) = v.raw;
}

// ---- warp reductions ------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- async copies, ldmatrix, mma (bf16 m16n8k16, fp32 accumulate) --------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// 16-byte global->shared copy that bypasses L1; src_bytes == 0 zero-fills the destination.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Programmatic dependent launch: a kernel launched with launch_pdl() may be scheduled while its predecessor in the
// stream is still draining; pdl_wait() (griddepcontrol.wait) blocks until the predecessor's memory is visible and
// must precede the first read of anything the predecessor wrote. It is a no-op in a normally launched kernel.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel in the stream (if it was launched with launch_pdl) start being scheduled now; it still blocks in
// its own pdl_wait() until this grid has completed and its writes are visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Sub-CTA named barrier over `threads` threads (a multiple of 32); id 0 is __syncthreads' barrier.
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace ns

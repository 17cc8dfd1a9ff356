// Step metadata built on the device, and greedy sampling that leaves the sampled token on the device.
//
// The host ships one packed int32 buffer per step (a few hundred bytes for a decode step): a header, one
// record per scheduled sequence, the block-table entries appended since the last step, and the token ids of
// prefill chunks. One CTA expands it into the static buffers a CUDA graph reads: token ids, positions,
// slot mapping, cu_seqlens, seq_lens, table rows and the row of each sequence's last token, padded to the
// graph bucket with rows that only touch the reserved garbage block.
#include <cooperative_groups.h>

#include "common.cuh"

namespace ns {

constexpr int kMetaThreads = 1024;

__global__ void __launch_bounds__(kMetaThreads) build_step_metadata_kernel(
    const int32_t* __restrict__ packed, int32_t* __restrict__ mirror, const int64_t* __restrict__ last_tokens,
    int pad_seat, int64_t* __restrict__ tokens, int64_t* __restrict__ positions, int64_t* __restrict__ slot_mapping,
    int32_t* __restrict__ cu_seqlens, int32_t* __restrict__ seq_lens, int32_t* __restrict__ seat_of,
    int64_t* __restrict__ last_rows, int max_seqs, int max_tokens) {
    extern __shared__ int32_t cu_sm[];        // [max_seqs + 1]
    __shared__ int warp_sums[33];
    const ns_step_header hd = *reinterpret_cast<const ns_step_header*>(packed);
    const int S = min(hd.n_seqs, max_seqs);
    const int PS = min(hd.pad_seqs, max_seqs);
    const int PT = min(hd.pad_tokens, max_tokens);
    const int32_t* rec = packed + sizeof(ns_step_header) / 4;
    const int32_t* app = rec + 4 * hd.n_seqs;
    const int32_t* tok = app + 3 * hd.n_appends;
    const int W = hd.table_width, bs = hd.block_size;

    // 1. block-table appends into the mirror
    for (int a = threadIdx.x; a < hd.n_appends; a += kMetaThreads)
        mirror[(int64_t)app[3 * a] * W + app[3 * a + 1]] = app[3 * a + 2];

    // 2. cu_seqlens = exclusive scan of n_new over real sequences, then one token per padding sequence
    int carry = 0;
    for (int base = 0; base < PS; base += kMetaThreads) {
        const int s = base + threadIdx.x;
        const int n = s < S ? rec[4 * s + 2] : (s < PS ? 1 : 0);
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        int inc = n;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += v;
        }
        if (lane == 31) warp_sums[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            const int w = warp_sums[lane];
            int winc = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, winc, o);
                if (lane >= o) winc += v;
            }
            warp_sums[lane] = winc - w;
            if (lane == 31) warp_sums[32] = winc;
        }
        __syncthreads();
        if (s < PS) cu_sm[s] = carry + warp_sums[warp] + inc - n;
        carry += warp_sums[32];
        __syncthreads();
    }
    if (threadIdx.x == 0) cu_sm[PS] = carry;
    __syncthreads();

    // 3. per-sequence outputs
    for (int s = threadIdx.x; s <= PS; s += kMetaThreads) {
        cu_seqlens[s] = cu_sm[s];
        if (s < PS) {
            const bool real = s < S;
            seq_lens[s] = real ? rec[4 * s + 1] + rec[4 * s + 2] : 1;
            seat_of[s] = real ? rec[4 * s] : pad_seat;
            last_rows[s] = cu_sm[s + 1] - 1;
        }
    }
    // 4. per-token outputs (binary search of the owning sequence in shared memory)
    const int covered = min(cu_sm[PS], PT);
    const int64_t gslot = (int64_t)hd.garbage_block * bs;
    for (int t = threadIdx.x; t < PT; t += kMetaThreads) {
        int64_t token = 0, pos = 0, slot = gslot;
        if (t < covered) {
            int lo = 0, hi = PS;
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (cu_sm[mid] <= t) lo = mid; else hi = mid;
            }
            if (lo < S) {
                const int seat = rec[4 * lo], ctx = rec[4 * lo + 1], toff = rec[4 * lo + 3];
                const int j = t - cu_sm[lo];
                const int ps = ctx + j;
                pos = ps;
                slot = (int64_t)mirror[(int64_t)seat * W + ps / bs] * bs + ps % bs;
                token = toff >= 0 ? (int64_t)tok[toff + j] : last_tokens[seat];
            }
        }
        tokens[t] = token;
        positions[t] = pos;
        slot_mapping[t] = slot;
    }
}

// Bounds check of one step's device metadata, the stand-in for a memory checker on this path: every block id a
// sequence's context touches is < num_blocks, every slot is < num_blocks * block_size and is the slot its table gives for
// its position, cu_seqlens starts at 0, is non-decreasing and stays within n_tokens, every sequence's length is at least its query length,
// token ids are inside the vocabulary. A violation is COUNTED (g_check_errors, reported through ns_collect_status) -
// nothing traps and nothing is skipped: the caller decides what a non-zero count means.
__device__ unsigned int g_check_errors = 0;

__global__ void __launch_bounds__(256) check_step_metadata_kernel(
    const int32_t* __restrict__ block_tables, const int32_t* __restrict__ table_rows, int64_t table_stride,
    const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ cu_seqlens, const int64_t* __restrict__ slot_mapping,
    const int64_t* __restrict__ positions, const int64_t* __restrict__ tokens, int n_seqs, int64_t n_tokens,
    int num_blocks, int block_size, int vocab) {
    unsigned bad = 0;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
    for (int s = tid; s < n_seqs; s += nthreads) {
        const int q0 = cu_seqlens ? cu_seqlens[s] : s, q1 = cu_seqlens ? cu_seqlens[s + 1] : s + 1;
        const int len = seq_lens[s];
        if (q1 < q0 || len < q1 - q0 || len < 0) { ++bad; continue; }
        if (q1 > n_tokens) ++bad;                  // (a padded step may leave rows past the last sequence unused)
        if (s == 0 && q0 != 0) ++bad;
        const int32_t* row = block_tables + (int64_t)(table_rows ? table_rows[s] : s) * table_stride;
        const int nb = (len + block_size - 1) / block_size;
        if (nb > table_stride) { ++bad; continue; }
        for (int j = 0; j < nb; ++j)
            if (row[j] < 0 || row[j] >= num_blocks) ++bad;
        // this step's new tokens: position = ctx + j, slot = table[pos / bs] * bs + pos % bs
        if (slot_mapping != nullptr && positions != nullptr)
            for (int t = q0; t < q1; ++t) {
                const int64_t pos = positions[t], slot = slot_mapping[t];
                if (pos != (int64_t)(len - (q1 - q0)) + (t - q0)) { ++bad; continue; }
                if (slot < 0 || slot >= (int64_t)num_blocks * block_size) { ++bad; continue; }
                const int32_t b = row[pos / block_size];
                if (b >= 0 && b < num_blocks && slot != (int64_t)b * block_size + pos % block_size) ++bad;
            }
    }
    if (tokens != nullptr && vocab > 0)
        for (int64_t t = tid; t < n_tokens; t += nthreads)
            if (tokens[t] < 0 || tokens[t] >= vocab) ++bad;
    if (bad) atomicAdd(&g_check_errors, bad);
}

// Device address of the check counter on the current device (resolved once per device, outside stream capture).
int check_error_counter(const unsigned int** out) {
    static const unsigned int* addr[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(NS_ERR_CUDA, "check_error_counter: no current device");
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_check_errors);
        if (e != cudaSuccess || p == nullptr) return fail(NS_ERR_CUDA, "check_error_counter: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        addr[dev] = static_cast<const unsigned int*>(p);
    }
    *out = addr[dev];
    return NS_OK;
}

// Greedy sampling: a cluster of CTAs per logits row (each scans a share of the vocabulary; the candidates meet in the
// first CTA's shared memory through DSMEM, no global scratch); ties resolve to the lowest index. The token is stored
// to out[row] and, when seat_of != NULL, to last_tokens[seat_of[row]] so the next step can read it without a host
// round trip. One CTA alone scanned a 152K-entry row in ~8 us; the row is 304 KB, so four CTAs share it.
template <typename T>
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const T* __restrict__ logits, int64_t row_stride, int vocab,
                                                           int64_t* __restrict__ out, const int32_t* __restrict__ seat_of,
                                                           int64_t* __restrict__ last_tokens) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank(), csize = (int)cluster.num_blocks();
    const int row_id = blockIdx.x / csize;
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // "this CTA runs", waited for before the DSMEM stores
    constexpr int V = Vec16<T>::N;
    const T* row = logits + (int64_t)row_id * row_stride;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    const int chunks = vocab / V;
    const int c_lo = (int)((long long)chunks * rank / csize), c_hi = (int)((long long)chunks * (rank + 1) / csize);
    for (int c = c_lo + threadIdx.x; c < c_hi; c += blockDim.x) {
        Vec16<T> v = load16(row + c * V);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float f = v.get(j);
            if (f > best) { best = f; best_i = c * V + j; }
        }
    }
    for (int i = chunks * V + threadIdx.x; i < vocab && rank == csize - 1; i += blockDim.x) {
        const float f = to_f32(row[i]);
        if (f > best || (f == best && i < best_i)) { best = f; best_i = i; }
    }
    __shared__ float sv[32];
    __shared__ int si[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = (blockDim.x + 31) / 32;
        best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
        best_i = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
    }
    // every CTA's candidate goes to slot `rank` of the first CTA's shared memory; the first CTA picks among them
    __shared__ float cv[8];
    __shared__ int ci[8];
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");     // the first CTA is running: its shared memory exists
    if (threadIdx.x == 0) {
        *cluster.map_shared_rank(&cv[rank], 0) = best;
        *cluster.map_shared_rank(&ci[rank], 0) = best_i;
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x == 0) {
        for (int r = 0; r < csize; ++r)
            if (cv[r] > best || (cv[r] == best && ci[r] < best_i)) { best = cv[r]; best_i = ci[r]; }
        const int64_t tokv = best_i == 0x7fffffff ? 0 : best_i;
        out[row_id] = tokv;
        if (seat_of != nullptr) last_tokens[seat_of[row_id]] = tokv;
    }
}

template <typename T>
static cudaError_t launch_argmax(const T* logits, int64_t row_stride, int rows, int vocab, int64_t* out, const int32_t* seat_of,
                                 int64_t* last_tokens, cudaStream_t st) {
    const int csize = vocab >= 32768 ? 4 : 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(rows * csize));
    cfg.blockDim = dim3(1024);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, argmax_rows_kernel<T>, logits, row_stride, vocab, out, seat_of, last_tokens);
}

}  // namespace ns

using namespace ns;

extern "C" int ns_build_step_metadata(const int32_t* packed, int32_t packed_ints, int32_t* table_mirror,
                                      const int64_t* last_tokens, int32_t pad_seat, int64_t* tokens,
                                      int64_t* positions, int64_t* slot_mapping, int32_t* cu_seqlens,
                                      int32_t* seq_lens, int32_t* seat_of, int64_t* last_rows, int32_t max_seqs,
                                      int32_t max_tokens, void* stream) {
    NS_REQUIRE(packed && table_mirror && last_tokens && tokens && positions && slot_mapping && cu_seqlens && seq_lens &&
                   seat_of && last_rows, NS_ERR_INVALID_ARG, "build_step_metadata: null pointer");
    NS_REQUIRE(packed_ints >= (int)(sizeof(ns_step_header) / 4), NS_ERR_INVALID_ARG, "build_step_metadata: packed buffer too small");
    NS_REQUIRE(max_seqs > 0 && max_tokens > 0, NS_ERR_INVALID_ARG, "build_step_metadata: bad capacity");
    const size_t smem = 4 * (size_t)(max_seqs + 1);
    NS_REQUIRE(smem <= 40 * 1024, NS_ERR_UNSUPPORTED, "build_step_metadata: max_seqs %d too large", max_seqs);
    build_step_metadata_kernel<<<1, kMetaThreads, smem, (cudaStream_t)stream>>>(
        packed, table_mirror, last_tokens, pad_seat, tokens, positions, slot_mapping, cu_seqlens, seq_lens, seat_of,
        last_rows, max_seqs, max_tokens);
    return check_launch("build_step_metadata");
}

extern "C" int ns_argmax_rows(const void* logits, int64_t row_stride, int32_t rows, int32_t vocab, int64_t* out,
                              const int32_t* seat_of, int64_t* last_tokens, int dtype, void* stream) {
    NS_REQUIRE(logits && out, NS_ERR_INVALID_ARG, "argmax_rows: null pointer");
    NS_REQUIRE(rows >= 0 && vocab > 0, NS_ERR_INVALID_ARG, "argmax_rows: bad shape");
    NS_REQUIRE(seat_of == nullptr || last_tokens != nullptr, NS_ERR_INVALID_ARG, "argmax_rows: seat_of without last_tokens");
    if (rows == 0) return NS_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == NS_BF16) {
        NS_REQUIRE(row_stride % 8 == 0, NS_ERR_UNSUPPORTED, "argmax_rows: row stride must be a multiple of 16 bytes");
        launch_argmax((const __nv_bfloat16*)logits, row_stride, rows, vocab, out, seat_of, last_tokens, st);
    } else if (dtype == NS_F32) {
        NS_REQUIRE(row_stride % 4 == 0, NS_ERR_UNSUPPORTED, "argmax_rows: row stride must be a multiple of 16 bytes");
        launch_argmax((const float*)logits, row_stride, rows, vocab, out, seat_of, last_tokens, st);
    } else {
        return fail(NS_ERR_UNSUPPORTED, "argmax_rows: dtype %d", dtype);
    }
    return check_launch("argmax_rows");
}

extern "C" int ns_check_step_metadata(const int32_t* block_tables, const int32_t* table_rows, int64_t table_stride,
                                      const int32_t* seq_lens, const int32_t* cu_seqlens, const int64_t* slot_mapping,
                                      const int64_t* positions, const int64_t* tokens, int32_t n_seqs, int64_t n_tokens,
                                      int32_t num_blocks, int32_t block_size, int32_t vocab, void* stream) {
    NS_REQUIRE(block_tables && seq_lens, NS_ERR_INVALID_ARG, "check_step_metadata: null pointer");
    NS_REQUIRE(n_seqs >= 0 && n_tokens >= 0 && num_blocks > 0 && block_size > 0 && table_stride > 0, NS_ERR_INVALID_ARG,
               "check_step_metadata: bad shape");
    NS_REQUIRE((slot_mapping == nullptr) == (positions == nullptr), NS_ERR_INVALID_ARG,
               "check_step_metadata: slot_mapping and positions go together");
    if (n_seqs == 0) return NS_OK;
    const int grid = (int)((n_tokens > n_seqs ? n_tokens : n_seqs) + 255) / 256;
    check_step_metadata_kernel<<<grid < 1 ? 1 : (grid > 64 ? 64 : grid), 256, 0, (cudaStream_t)stream>>>(
        block_tables, table_rows, table_stride, seq_lens, cu_seqlens, slot_mapping, positions, tokens, n_seqs, n_tokens,
        num_blocks, block_size, vocab);
    return check_launch("check_step_metadata");
}

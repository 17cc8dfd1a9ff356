// Per-step attention plan: one small kernel whose output every layer of the step reuses.
#include "attn_plan.cuh"
#include "common.cuh"

namespace ns {

constexpr int kPlanThreads = 1024;

// Block-wide exclusive scan of one int per thread (kPlanThreads threads). Returns the exclusive prefix and the
// block total through `total`.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = warp_sums[lane];
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        warp_sums[lane] = winc - w;          // exclusive prefix of the warp sums
        if (lane == 31) warp_sums[32] = winc;
    }
    __syncthreads();
    const int excl = warp_sums[warp] + inc - v;
    total = warp_sums[32];
    __syncthreads();
    return excl;
}

__global__ void __launch_bounds__(kPlanThreads) attn_plan_kernel(const int32_t* __restrict__ seq_lens,
                                                                 const int32_t* __restrict__ cu_seqlens,
                                                                 const int32_t* __restrict__ table_rows, int n_seqs,
                                                                 int block_size, int base_ctas, int max_mode,
                                                                 int split_blocks, uint8_t* ws, WsLayout L, int max_items,
                                                                 int min_blocks, int snap_blocks, int balance, int cluster,
                                                                 int cluster_blocks) {
    constexpr int kSmemRows = 2048;            // decode rows whose prefix is mirrored in shared memory
    __shared__ int warp_sums[33];
    __shared__ int indptr_sm[kSmemRows + 1];
    PlanHeader* hdr = reinterpret_cast<PlanHeader*>(ws + L.header);
    int4* dec_info = reinterpret_cast<int4*>(ws + L.dec_info);
    int32_t* dec_indptr = reinterpret_cast<int32_t*>(ws + L.dec_indptr);
    int32_t* cta_first = reinterpret_cast<int32_t*>(ws + L.cta_first);
    int2* items = reinterpret_cast<int2*>(ws + L.prefill_items);

    int n_dec = 0, dec_blocks = 0, n_items = 0, my_max_nb = 0;
    for (int base = 0; base < n_seqs; base += kPlanThreads) {
        const int s = base + threadIdx.x;
        int is_dec = 0, nb = 0, tiles = 0, T = 0, len = 0, qrow = s;
        if (s < n_seqs) {
            if (cu_seqlens) {
                qrow = cu_seqlens[s];
                T = cu_seqlens[s + 1] - qrow;
            } else {
                T = 1;
            }
            len = seq_lens[s];
            if (T == 1) {
                is_dec = 1;
                nb = (len + block_size - 1) / block_size;
            } else if (T > 1) {
                tiles = (T + kPrefillTileTokens - 1) / kPrefillTileTokens;
            }
        }
        int tot;
        const int pos = block_exclusive_scan(is_dec, warp_sums, tot);
        const int d_tot = tot;
        const int boff = block_exclusive_scan(nb, warp_sums, tot);
        const int b_tot = tot;
        const int ioff = block_exclusive_scan(tiles, warp_sums, tot);
        const int i_tot = tot;
        if (is_dec) {
            my_max_nb = max(my_max_nb, nb);
            dec_info[n_dec + pos] = make_int4(s, len, table_rows ? table_rows[s] : s, qrow);
            dec_indptr[n_dec + pos] = dec_blocks + boff;
            if (n_dec + pos <= kSmemRows) indptr_sm[n_dec + pos] = dec_blocks + boff;
        }
        // Latest query tile first: under the causal mask it attends to the most keys, so the heaviest items
        // start earliest.
        for (int k = 0; k < tiles; ++k) {
            const int idx = n_items + ioff + k;
            if (idx < max_items) items[idx] = make_int2(s, (tiles - 1 - k) * kPrefillTileTokens);
        }
        n_dec += d_tot;
        dec_blocks += b_tot;
        n_items += i_tot;
    }
    __shared__ int max_nb_sm;
    if (threadIdx.x == 0) {
        dec_indptr[n_dec] = dec_blocks;
        if (n_dec <= kSmemRows) indptr_sm[n_dec] = dec_blocks;
        max_nb_sm = 0;
    }
    __syncthreads();
    // Prefill items heaviest first over the whole step (weight = key tiles of 64 the item walks), ties in the order they
    // were written: the prefill kernels hand them to CTAs in this order (longest first; where the items are one wave of
    // two CTAs per SM, the heaviest next to the lightest). One item per thread; steps with more items keep the order above.
    {
        __shared__ int item_key[kPlanThreads];
        const int n = n_items < max_items ? n_items : max_items;
        if (n > 1 && n <= kPlanThreads) {
            const int i = threadIdx.x;
            int2 mine = make_int2(0, 0);
            if (i < n) {
                mine = items[i];
                const int q0 = cu_seqlens[mine.x], T = cu_seqlens[mine.x + 1] - q0, len = seq_lens[mine.x];
                const int kv_end = min(len, len - T + mine.y + kPrefillTileTokens);
                item_key[i] = (kv_end + 63) >> 6;
            }
            __syncthreads();
            int rank = 0;
            if (i < n) {
                const int k = item_key[i];
                for (int j = 0; j < n; ++j) {
                    const int kj = item_key[j];
                    rank += (kj > k || (kj == k && j < i)) ? 1 : 0;
                }
            }
            __syncthreads();
            if (i < n) items[rank] = mine;
        }
    }
    if (my_max_nb > 0) atomicMax(&max_nb_sm, my_max_nb);
    __syncthreads();
    const int max_nb = max_nb_sm;                  // blocks of the longest decode row
    const int* ip = n_dec <= kSmemRows ? indptr_sm : dec_indptr;

    // Large steps run every decode CTA as two virtual CTAs of half the warps (twice as many, shorter ranges); small
    // ones keep all warps of a CTA on one range. The decode kernel reads the choice from the header.
    const int mode = (max_mode >= 2 && dec_blocks > split_blocks) ? 2 : 1;
    const int decode_ctas = base_ctas * mode;
    int per = (dec_blocks + decode_ctas - 1) / decode_ctas;
    if (per < min_blocks) per = min_blocks;
    const int used = (dec_blocks + per - 1) / per;
    const int slack = per <= 2 * snap_blocks * (mode == 1 && max_mode >= 2 ? 2 : 1) ? per / 2 : per / 8;   // how far a cut may move to reach a row boundary
    int32_t* cta_start = reinterpret_cast<int32_t*>(ws + L.cta_start);
    int2* dec_span = reinterpret_cast<int2*>(ws + L.dec_span);
    __shared__ int cuts_sm[kMaxDecodeCtas + 1];
    // row containing block-unit u (u < dec_blocks): the last row whose first unit is <= u
    auto row_of = [&](int u) {
        int lo = 0, hi = n_dec;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (ip[mid] <= u) lo = mid; else hi = mid;
        }
        return lo;
    };
    // Steps with the row prefix in shared memory, large ones (mode 2) always: ROW-ALIGNED BALANCED cuts. Rows are packed whole into a
    // CTA up to T blocks; a row longer than T starts a CTA of its own and is cut into ceil(L / T) equal pieces. T is the
    // smallest of 64 candidates in [per, 3 per) for which that needs no more CTAs than there are: every range is at most
    // T blocks and no CTA holds part of two rows. (Equal cuts snapped to row boundaries, below, leave ranges between 0.5
    // and 2 times the average: measured on 48 rows x U[128,8192] tokens the slowest CTA streamed 20.8 us, the median 14.9.)
    // ... and for small steps whose rows are, on average, at least three quarters of a range long (many short rows per
    // range pack better with the equal cuts below: 256 rows x U[64,1024] tokens 19.4 vs 20.9 us)
    // Small steps: fewer rows than clusters and not much to stream. One CTA per row would leave most SMs idle and push a
    // whole row through one SM's load path; instead row c gets cluster c: its blocks are cut into `cluster` equal
    // contiguous pieces, CTA c * cluster + r takes piece r (the kernel combines the pieces through shared memory).
    // ... and only while the longest row's piece is not much more than a balanced range would be: a step with a few
    // very long rows is better cut into equal ranges over ALL CTAs, whose cross-CTA combine costs about as much as
    // streaming kClusterSlackBlocks blocks.
    const bool cluster_mode = cluster > 1 && mode == 1 && n_dec > 0 && n_dec * cluster <= base_ctas && n_dec <= kSmemRows &&
                              dec_blocks <= cluster_blocks &&
                              (max_nb + cluster - 1) / cluster <= dec_blocks / base_ctas + kClusterSlackBlocks;
    const bool balanced = !cluster_mode && balance != 0 && n_dec <= kSmemRows &&
                          (mode == 2 || (balance >= 2 && 4LL * dec_blocks >= 3LL * n_dec * per));
    // small steps: a row of up to 2 * min_blocks blocks is never split (a cross-CTA combine costs more than it saves)
    const int no_split = mode == 2 ? 0 : 2 * min_blocks;
    __shared__ int cand_ok[64];
    if (cluster_mode) {
        for (int c = threadIdx.x; c <= decode_ctas; c += kPlanThreads) {
            const int row = c / cluster, r = c - row * cluster;
            int cut = dec_blocks;
            if (row < n_dec) {
                // pieces differ by at most one block and the empty ones (rows shorter than the cluster) come last, on
                // the row's end: a CTA between two equal cuts never sits inside a row (the span logic below and the
                // kernel's fallback to global partials rely on it)
                const int start = ip[row], len = ip[row + 1] - start;
                const int piece = len / cluster, extra = len - piece * cluster;
                cut = start + r * piece + min(r, extra);
            }
            cuts_sm[c] = cut;
            cta_start[c] = cut;
        }
    } else if (balanced) {
        if (threadIdx.x < 64) {
            const int T = per + (per * (int)threadIdx.x) / 32;
            int ctas = 0, cur = 0;
            for (int i = 0; i < n_dec; ++i) {
                const int len = ip[i + 1] - ip[i];
                if (len > T) {
                    ctas += (cur > 0) + (len > no_split ? (len + T - 1) / T : 1);
                    cur = 0;
                } else if (cur + len > T) {
                    ++ctas;
                    cur = len;
                } else {
                    cur += len;
                }
            }
            cand_ok[threadIdx.x] = ctas + (cur > 0) <= decode_ctas;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int best = 63;
            for (int l = 62; l >= 0; --l)
                if (cand_ok[l]) best = l;
            const int T = cand_ok[best] ? per + (per * best) / 32 : dec_blocks;       // nothing fits: one open-ended pass
            int c = 0, cur = 0;
            cuts_sm[0] = 0;
            for (int i = 0; i < n_dec && c < decode_ctas; ++i) {
                const int start = ip[i], len = ip[i + 1] - start;
                if (len > T) {
                    if (cur > 0) cuts_sm[++c] = start;
                    cur = 0;
                    const int k = len > no_split ? (len + T - 1) / T : 1;
                    for (int j = 1; j <= k && c < decode_ctas; ++j) cuts_sm[++c] = start + (int)(((long long)j * len) / k);
                } else if (cur + len > T) {
                    cuts_sm[++c] = start;
                    cur = len;
                } else {
                    cur += len;
                }
            }
            if (cur > 0 && c < decode_ctas) ++c;
            for (; c <= decode_ctas; ++c) cuts_sm[c] = dec_blocks;      // closes the last range; the rest are empty
        }
        __syncthreads();
        for (int c = threadIdx.x; c <= decode_ctas; c += kPlanThreads) cta_start[c] = cuts_sm[c];
    } else {
    for (int c = threadIdx.x; c <= decode_ctas; c += kPlanThreads) {
        long long u = (long long)c * per;
        int cut = u >= dec_blocks ? dec_blocks : (int)u;
        if (cut > 0 && cut < dec_blocks) {
            const int r = row_of(cut);
            const int below = ip[r], above = ip[r + 1];
            if (cut - below <= above - cut) {
                if (cut - below <= slack) cut = below;
            } else if (above - cut <= slack) {
                cut = above;
            }
        }
        cuts_sm[c] = cut;
        cta_start[c] = cut;
    }
    }
    __syncthreads();
    int4* cta_rec = reinterpret_cast<int4*>(ws + L.cta_rec);
    for (int c = threadIdx.x; c <= decode_ctas; c += kPlanThreads) {
        const int first = cuts_sm[c] >= dec_blocks ? n_dec : row_of(cuts_sm[c]);
        cta_first[c] = first;
        if (c < decode_ctas) {
            // everything a decode CTA needs before its first K/V load, in one 32-byte record
            int4 a = make_int4(cuts_sm[c], cuts_sm[c + 1], first, 0), b = make_int4(0, 0, 0, 0);
            if (first < n_dec) {
                const int4 info = dec_info[first];
                a.w = ip[first];
                b = make_int4(ip[first + 1], info.y, info.z, info.w);
            }
            cta_rec[2 * c] = a;
            cta_rec[2 * c + 1] = b;
        }
    }
    // CTAs touching each row: the last CTA starting at or before the row's first unit .. the last CTA starting
    // before its end (CTAs between two equal cuts are empty and sit on a row boundary, never inside a row)
    for (int i = threadIdx.x; i < n_dec; i += kPlanThreads) {
        const int lo_u = ip[i], hi_u = ip[i + 1];
        int first = 0, last = 0;
        if (hi_u > lo_u) {
            int a = 0, b2 = decode_ctas;             // last c with cuts[c] <= lo_u
            while (b2 - a > 1) {
                const int mid = (a + b2) >> 1;
                if (cuts_sm[mid] <= lo_u) a = mid; else b2 = mid;
            }
            first = a;
            a = 0; b2 = decode_ctas;                 // last c with cuts[c] < hi_u
            while (b2 - a > 1) {
                const int mid = (a + b2) >> 1;
                if (cuts_sm[mid] < hi_u) a = mid; else b2 = mid;
            }
            last = a;
        }
        dec_span[i] = make_int2(first, last - first + 1);
    }
    if (threadIdx.x == 0) {
        hdr->n_dec = n_dec;
        hdr->dec_total = dec_blocks;
        hdr->dec_per_cta = per;
        hdr->dec_ctas = used;
        hdr->n_prefill_items = n_items < max_items ? n_items : max_items;
        hdr->n_seqs = n_seqs;
        hdr->block_size = block_size;
        hdr->mode = mode;
        hdr->cluster = cluster_mode ? cluster : 0;
    }
}

void plan_knobs(int* min_blocks, int* split_blocks, int* snap_blocks, int* balance, int* cluster_on,
                int* cluster_blocks);      // c_api.cu: ns_set_tuning

int launch_attn_plan(const int32_t* seq_lens, const int32_t* cu_seqlens, const int32_t* table_rows, int n_seqs,
                     int block_size, int base_ctas, int max_mode,
                     void* ws, const WsLayout& L, int max_items, cudaStream_t st) {
    int min_blocks, split_blocks, snap_blocks, balance, cluster_on, cluster_blocks;
    plan_knobs(&min_blocks, &split_blocks, &snap_blocks, &balance, &cluster_on, &cluster_blocks);
    const int cluster = cluster_on ? plan_cluster(n_seqs, base_ctas) : 1;
    attn_plan_kernel<<<1, kPlanThreads, 0, st>>>(seq_lens, cu_seqlens, table_rows, n_seqs, block_size, base_ctas, max_mode,
                                                 split_blocks, (uint8_t*)ws, L, max_items, min_blocks, snap_blocks, balance,
                                                 cluster, cluster_blocks);
    return check_launch("attn_plan");
}

}  // namespace ns

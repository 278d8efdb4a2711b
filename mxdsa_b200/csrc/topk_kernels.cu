// Index selection: one row of scores per query pair (or per request) -> the row of key indices that
// the attention entry points consume (int32, ascending, -1 padded, plus the row's valid length).
//
// The attention operators take their keys from `indices[pair][topk]` with the conventions of the
// reference's callers (reference tests/benchmark.py:119-147: one row per pair of query tokens, entries
// -1 never attended, decode pools addressed by request * pool_len + slot; csrc/bindings/binding.cpp:12-15 and
// csrc/bindings/dual_mxfp8_sparse_decode.h:13-20 for the shapes; `topk_length` bounds the attended prefix).  The reference
// has no producer for that tensor; this is the selection step of a sparse-attention indexer in the
// form those conventions need.
//
// Definition (the CPU oracle restates it with a stable sort):
//   * candidates of row r: keys j < lengths[r] (all s_kv keys without lengths) whose score is neither
//     NaN nor -inf; with group == 2 the score of key j is the larger of the two tokens' scores
//     (a NaN on one side is ignored);
//   * selected: the min(topk, #candidates) candidates of highest score, ties going to the smaller j
//     (-0 and +0 tie);
//   * written in ascending j (+ row_offset[r]), then -1 up to topk; topk_length[r] = number selected.
//
// Method: exact radix selection on the order-preserving 32-bit image of the float, three histogram
// passes (11 + 11 + 10 bits) with shared-memory atomics, keys of a row held in registers (one HBM read
// per score for rows of up to 16 384 keys; longer rows are swept again from L2).  No pass branches per
// key: the first counts every key, the later ones send keys outside the current prefix to a per-lane
// spare bin.  Packed per-chunk counts and two block scans then give every selected key its output
// position; the row is staged in shared memory and written in whole lines.  No sort, no global atomics,
// deterministic.
//
// Bound: HBM on paper (group * s_kv * 4 bytes read + topk * 4 written per row); in practice the integer
// pipe (about 25 instructions per key), so every step is written to save instructions, not bytes.
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../../include/mxdsa.h"

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kChunks = 8;                         // float4 loads per thread and sweep
constexpr int kKpt = kChunks * 4;                  // keys per thread and sweep
constexpr int kSweep = kThreads * kKpt;            // 16 384 keys
constexpr int kBins = 2048;
constexpr int kStage = 4096;                       // rows of up to this many indices are staged in shared memory

struct TopkShared {
    uint32_t hist[kBins + 32];                     // + one never-read bin per lane for keys outside the current prefix
    uint32_t warp_tot[kWarps];                     // find_bin: per-warp histogram mass
    uint32_t chunk_tot[kChunks * kWarps];          // output scan: packed (greater | equal << 16) per (chunk, warp)
    uint32_t sel_bin, sel_above, sel_count;        // result of find_bin
    uint32_t sweep_tot;                            // packed totals of one sweep
    int32_t stage[kStage];                         // a row's output, staged for coalesced stores
};

// float -> unsigned key with the same order.  Usable scores map to [0x00800000 (-FLT_MAX), 0xff800000
// (+inf)].  A NaN is first turned into -inf (fmaxf returns its other argument); -inf lands just below the
// usable interval: it falls into histogram bins 0-3, which pass 0 ignores, and lies below every threshold,
// so it needs no further special case.  Keys outside the row's length become 0.
__device__ __forceinline__ uint32_t score_key(float s) {
    const uint32_t u = __float_as_uint(fmaxf(s, -CUDART_INF_F) + 0.0f);           // NaN -> -inf, -0 -> +0
    return u ^ ((uint32_t)((int32_t)u >> 31) | 0x80000000u);
}

// One sweep of a row into registers.  All loads of a batch are issued before the first conversion, so a
// sweep exposes one memory latency (two with GROUP == 2, whose two score rows are taken in two batches
// of four chunks to stay inside the register budget), not one per load.
template <int GROUP>
__device__ __forceinline__ void load_keys(const float* __restrict__ row0, const float* __restrict__ row1, int sweep,
                                          int s_kv, int len, uint32_t (&key)[kKpt]) {
    constexpr int kBatch = GROUP == 2 ? kChunks / 2 : kChunks;
#pragma unroll
    for (int c0 = 0; c0 < kChunks; c0 += kBatch) {
        float4 a[kBatch], b[GROUP == 2 ? kBatch : 1];
#pragma unroll
        for (int c = 0; c < kBatch; ++c) {
            const int j = sweep * kSweep + ((c0 + c) * kThreads + (int)threadIdx.x) * 4;
            a[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (GROUP == 2) b[c] = a[c];
            if (j < s_kv) {
                a[c] = __ldg(reinterpret_cast<const float4*>(row0 + j));
                if (GROUP == 2) b[c] = __ldg(reinterpret_cast<const float4*>(row1 + j));
            }
        }
#pragma unroll
        for (int c = 0; c < kBatch; ++c) {
            const int j = sweep * kSweep + ((c0 + c) * kThreads + (int)threadIdx.x) * 4;
            float4 v = a[c];
            if (GROUP == 2) v = make_float4(fmaxf(v.x, b[c].x), fmaxf(v.y, b[c].y), fmaxf(v.z, b[c].z), fmaxf(v.w, b[c].w));
            const int nin = len - j;                  // keys of this chunk inside the row's length
            key[4 * (c0 + c) + 0] = score_key(v.x);
            key[4 * (c0 + c) + 1] = score_key(v.y);
            key[4 * (c0 + c) + 2] = score_key(v.z);
            key[4 * (c0 + c) + 3] = score_key(v.w);
            if (nin < 4) {                            // the chunk straddles (or lies beyond) the row's length
#pragma unroll
                for (int e = 0; e < 4; ++e) key[4 * (c0 + c) + e] = e < nin ? key[4 * (c0 + c) + e] : 0u;
            }
        }
    }
}

__device__ __forceinline__ uint32_t warp_inclusive_scan(uint32_t v, int lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t n = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += n;
    }
    return v;
}

// After a histogram is complete: the bin that holds the k-th largest entry (k counted from the top,
// 1 <= k <= total), the mass above that bin and the bin's own count.  Returns the histogram total.
// Ends with a barrier; the result is in sm.sel_*.
__device__ __forceinline__ uint32_t find_bin(TopkShared& sm, uint32_t k_or_cap, bool cap_to_total, uint32_t& k_out, int nbins) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint4 h = *reinterpret_cast<const uint4*>(&sm.hist[4 * tid]);
    if (cap_to_total && tid == 0) h = make_uint4(0u, 0u, 0u, 0u);   // pass 0: bins 0-3 collect the non-candidates
    if (4 * tid >= nbins) h = make_uint4(0u, 0u, 0u, 0u);           // beyond the digits: spare bins
    const uint32_t local = h.x + h.y + h.z + h.w;
    const uint32_t inc = warp_inclusive_scan(local, lane);
    if (lane == 31) sm.warp_tot[warp] = inc;
    __syncthreads();
    // lane l holds warp l's mass; two warp reductions give the total and the mass of the warps below
    const uint32_t wt = lane < kWarps ? sm.warp_tot[lane] : 0u;
    const uint32_t total = __reduce_add_sync(0xffffffffu, wt);
    const uint32_t below_warps = __reduce_add_sync(0xffffffffu, lane < warp ? wt : 0u);
    const uint32_t k = cap_to_total ? min(k_or_cap, total) : k_or_cap;
    k_out = k;
    uint32_t run = total - (below_warps + inc);    // mass in bins above this thread's four
    if (run < k && run + local >= k) {             // the k-th entry is in one of this thread's bins
        const uint32_t hh[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
        for (int b = 3; b >= 0; --b) {
            if (run < k && run + hh[b] >= k) {
                sm.sel_bin = 4 * tid + b;
                sm.sel_above = run;
                sm.sel_count = hh[b];
            }
            run += hh[b];
        }
    }
    __syncthreads();
    return total;
}

// Writes the selected keys of one sweep at their output positions and advances the running counts.
// Per thread and chunk the counts (0..4) are packed four chunks to a word, 8 bits each, so two warp scans
// cover the eight chunks (a warp's inclusive total per chunk is at most 128).
template <bool TIES, bool STAGED>
__device__ __forceinline__ void emit_sweep(TopkShared& sm, const uint32_t (&key)[kKpt], uint32_t thr, uint32_t need_eq,
                                           int32_t* __restrict__ out, int32_t off, int sw, uint32_t& base_gt,
                                           uint32_t& base_eq) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t own_a[2] = {0u, 0u}, own_e[2] = {0u, 0u};   // a: key > thr (TIES) or key >= thr; e: key == thr
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        uint32_t na = 0, ne = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t kk = key[4 * c + e];
            na += (TIES ? kk > thr : kk >= thr) ? 1u : 0u;
            if (TIES) ne += kk == thr ? 1u : 0u;
        }
        own_a[c >> 2] |= na << (8 * (c & 3));
        if (TIES) own_e[c >> 2] |= ne << (8 * (c & 3));
    }
    uint32_t inc_a[2], inc_e[2] = {0u, 0u};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        inc_a[h] = warp_inclusive_scan(own_a[h], lane);
        if (TIES) inc_e[h] = warp_inclusive_scan(own_e[h], lane);
    }
    if (lane == 31) {
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
            sm.chunk_tot[c * kWarps + warp] = ((inc_a[c >> 2] >> (8 * (c & 3))) & 0xffu) | (((inc_e[c >> 2] >> (8 * (c & 3))) & 0xffu) << 16);
    }
    __syncthreads();
    if (warp == 0) {                     // exclusive scan of the 128 (chunk, warp) totals, packed a | e << 16
        const uint4 t = *reinterpret_cast<const uint4*>(&sm.chunk_tot[4 * lane]);
        const uint32_t s = t.x + t.y + t.z + t.w;
        const uint32_t incl = warp_inclusive_scan(s, lane);
        const uint32_t ex = incl - s;
        *reinterpret_cast<uint4*>(&sm.chunk_tot[4 * lane]) = make_uint4(ex, ex + t.x, ex + t.x + t.y, ex + t.x + t.y + t.z);
        if (lane == 31) sm.sweep_tot = incl;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const uint32_t before = sm.chunk_tot[c * kWarps + warp];
        const int sh = 8 * (c & 3);
        uint32_t a = base_gt + (before & 0xffffu) + ((inc_a[c >> 2] >> sh) & 0xffu) - ((own_a[c >> 2] >> sh) & 0xffu);
        const int j0 = sw * kSweep + (c * kThreads + tid) * 4 + off;
        if (!TIES) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (key[4 * c + e] >= thr) {
                    if (STAGED) sm.stage[a++] = j0 + e;
                    else out[a++] = j0 + e;
                }
            }
        } else {
            uint32_t q = base_eq + (before >> 16) + ((inc_e[c >> 2] >> sh) & 0xffu) - ((own_e[c >> 2] >> sh) & 0xffu);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t kk = key[4 * c + e];
                const bool is_gt = kk > thr, is_eq = kk == thr;
                if (is_gt || (is_eq && q < need_eq)) {
                    if (STAGED) sm.stage[a + min(q, need_eq)] = j0 + e;
                    else out[a + min(q, need_eq)] = j0 + e;
                }
                a += is_gt ? 1u : 0u;
                q += is_eq ? 1u : 0u;
            }
        }
    }
    const uint32_t st = sm.sweep_tot;
    base_gt += st & 0xffffu;
    base_eq += st >> 16;
    __syncthreads();                     // chunk_tot / sweep_tot are rewritten by the next sweep or row
}

template <int GROUP, bool STAGED>
__global__ void __launch_bounds__(kThreads, 2)
mxdsa_topk_rows_kernel(const float* __restrict__ scores, long long score_stride, const int32_t* __restrict__ lengths,
                       const int32_t* __restrict__ row_offset, int32_t* __restrict__ indices, long long index_stride,
                       int32_t* __restrict__ topk_length, int rows, int s_kv, int topk) {
    __shared__ __align__(16) TopkShared sm;
    const int tid = threadIdx.x, lane = tid & 31;
    const int nsweeps = (s_kv + kSweep - 1) / kSweep;
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* row0 = scores + (long long)r * GROUP * score_stride;
        const float* row1 = row0 + score_stride;
        int len = s_kv;
        if (lengths != nullptr) len = min(max(__ldg(lengths + r), 0), s_kv);
        uint32_t key[kKpt];
        // the row this CTA takes next: ask L2 for it now, so that its loads do not wait for HBM
        if (r + (int)gridDim.x < rows && tid * 32 < s_kv && nsweeps == 1) {
            const float* nx = scores + (long long)(r + (int)gridDim.x) * GROUP * score_stride + tid * 32;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(nx));
            if (GROUP == 2) asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + score_stride));
        }

        // ---- three radix passes: prefix = the bits of the threshold key found so far
        uint32_t prefix = 0, k = (uint32_t)topk, n_sel = 0;
#pragma unroll 1
        for (int pass = 0; pass < 3; ++pass) {
            const int lo = pass == 0 ? 21 : (pass == 1 ? 10 : 0);       // lowest bit of this pass's digit
            const int hi = pass == 0 ? 32 : (pass == 1 ? 21 : 10);      // bits above the digit are the prefix
            *reinterpret_cast<uint4*>(&sm.hist[4 * tid]) = make_uint4(0u, 0u, 0u, 0u);
            __syncthreads();
            if (pass == 0) {
                // every key takes part (non-candidates fall into bins 0-3, which find_bin ignores)
#pragma unroll 1
                for (int sw = 0; sw < nsweeps; ++sw) {
                    load_keys<GROUP>(row0, row1, sw, s_kv, len, key);
#pragma unroll
                    for (int i = 0; i < kKpt; ++i) atomicAdd(&sm.hist[key[i] >> 21], 1u);
                }
            } else {
                // keys outside the prefix add to a per-lane spare bin: no branch, no bank conflict
#pragma unroll 1
                for (int sw = 0; sw < nsweeps; ++sw) {
                    if (nsweeps > 1) load_keys<GROUP>(row0, row1, sw, s_kv, len, key);
                    // distance from the first key of the prefix: inside the prefix it is below 2^hi and its top
                    // bits are the digit; everything else (wrapped or large) is clamped onto the spare bins
                    const uint32_t first = prefix << hi, spare = (uint32_t)((kBins >> (pass - 1)) + lane);   // 2048 / 1024 digits
#pragma unroll
                    for (int i = 0; i < kKpt; ++i) atomicAdd(&sm.hist[min((key[i] - first) >> lo, spare)], 1u);
                }
            }
            __syncthreads();
            uint32_t k_now;
            const uint32_t total = find_bin(sm, k, pass == 0, k_now, pass == 2 ? kBins / 2 : kBins);
            if (pass == 0) n_sel = k_now;            // min(topk, candidates)
            if (total == 0u || k_now == 0u) { n_sel = 0; break; }
            prefix = pass == 0 ? sm.sel_bin : ((prefix << (hi - lo)) | sm.sel_bin);
            k = k_now - sm.sel_above;                // rank inside the chosen bin, 1-based
        }
        // all threads agree on n_sel (computed from shared totals); prefix is now the full threshold key
        const uint32_t thr = prefix, need_eq = k;    // take `need_eq` keys equal to thr, smallest index first

        // ---- output positions: ascending index, order (sweep, chunk, thread, element).
        // Without surplus ties (every key equal to the threshold is taken -- the rule unless scores repeat)
        // "selected" is key >= thr and one count per key suffices; otherwise the equal keys are ranked too.
        int32_t* out = indices + (long long)r * index_stride;
        const int32_t off = row_offset != nullptr ? __ldg(row_offset + r) : 0;
        if (n_sel > 0u) {
            const bool ties = need_eq != sm.sel_count;
            uint32_t base_gt = 0, base_eq = 0;
#pragma unroll 1
            for (int sw = 0; sw < nsweeps; ++sw) {
                if (nsweeps > 1) load_keys<GROUP>(row0, row1, sw, s_kv, len, key);
                if (!ties) emit_sweep<false, STAGED>(sm, key, thr, need_eq, out, off, sw, base_gt, base_eq);
                else emit_sweep<true, STAGED>(sm, key, thr, need_eq, out, off, sw, base_gt, base_eq);
            }
        }
        if (STAGED) {                                // topk <= kStage: positions were staged in shared memory
            for (uint32_t pos = tid; pos < (uint32_t)topk; pos += kThreads) out[pos] = pos < n_sel ? sm.stage[pos] : -1;
        } else {
            for (uint32_t pos = n_sel + tid; pos < (uint32_t)topk; pos += kThreads) out[pos] = -1;
        }
        if (topk_length != nullptr && tid == 0) topk_length[r] = (int32_t)n_sel;
        __syncthreads();                             // sm.sel_* and the histogram belong to the next row from here
    }
}

thread_local int tl_topk_cuda_error = 0;

}  // namespace

extern "C" int mxdsa_topk_select(const mxdsa_topk_params* p) {
    if (p == nullptr || p->scores == nullptr || p->indices == nullptr) return MXDSA_ERR_NULL;
    if (p->rows < 0 || p->s_kv <= 0 || p->topk <= 0 || (p->group != 1 && p->group != 2) || (p->s_kv & 3)) return MXDSA_ERR_SHAPE;
    if (p->rows == 0) return MXDSA_OK;
    const long long ss = p->score_stride ? p->score_stride : p->s_kv;
    const long long is = p->index_stride ? p->index_stride : p->topk;
    if (((uintptr_t)p->scores & 15) || (ss & 3) || ss < p->s_kv || is < p->topk || ((uintptr_t)p->indices & 3)) return MXDSA_ERR_ALIGN;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return MXDSA_ERR_CUDA;
    const int grid = p->rows < sms * 2 ? p->rows : sms * 2;      // two resident CTAs of 512 threads per SM
    const cudaStream_t s = static_cast<cudaStream_t>(p->stream);
    auto kern = p->topk <= kStage ? (p->group == 2 ? mxdsa_topk_rows_kernel<2, true> : mxdsa_topk_rows_kernel<1, true>)
                                  : (p->group == 2 ? mxdsa_topk_rows_kernel<2, false> : mxdsa_topk_rows_kernel<1, false>);
    kern<<<grid, kThreads, 0, s>>>(p->scores, ss, p->lengths, p->row_offset, p->indices, is, p->topk_length, p->rows, p->s_kv,
                                   p->topk);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        tl_topk_cuda_error = (int)e;
        return MXDSA_ERR_CUDA;
    }
    return MXDSA_OK;
}

extern "C" int mxdsa_topk_last_cuda_error(void) { return tl_topk_cuda_error; }

// MXFP8 sparse attention for sm_100a: one kernel body for prefill and split-KV decode.
//
// Work decomposition
//   A CTA pair (cluster of 2) owns one query PAIR: query tokens 2p and 2p+1 share one row of
//   key indices, so their 2 x 64 heads form the 128 rows of every tensor-core tile.  CTA c of
//   the pair holds the 64 rows of token 2p+c.  All MMAs are tcgen05 cta_group::2, M = 128:
//     QK : P[128 x 128 keys]  += Q[128 x 32] . K[128 keys x 32]^T      16 steps over the 512 dims
//     PV : O[128 x 256 dims]  += S[128 x 32 keys] . V[32 keys x 256]   4 key steps x 2 dim chunks
//   K rows are split between the CTAs by key (CTA c stages keys 64c..64c+63 of the tile, all 512
//   bytes), V rows by dimension (CTA c stages all 128 keys, bytes 256c..256c+255).  The
//   accumulators live in tensor memory: per CTA 128 lanes x (256 O + 2 x 64 P) columns; lane L
//   holds row L%64, and column half L/64 (P: keys 64*(L/64).., O: dims 256*(L/64)..).
//
// Roles (warp-specialised, 8 warps per CTA)
//   warp 0  gather producer : reads key indices, issues TMA gather4 row copies into the K/V ring
//   warp 1  QK issuer (CTA 0, one thread); in CTA 1 idle
//   warp 2  PV issuer (CTA 0, one thread); in CTA 1 idle
//   warp 3  operand stager  : Q tile TMA + Q scale rows (per pair); K scale rows, key token
//           scales and validity bits (per tile)
//   warps 4-7 softmax       : P -> registers, running max with lazy rescale, exp2, token-scale,
//           per-32-key UE8M0 requantisation to E4M3 S, O rescale, and the epilogue.
//
// Numerical contract (identical to the reference kernels, reference file:line in brackets)
//   * keys are consumed in numerical tiles of NT = 128 (prefill, topk >= 512) or 64 keys
//     [csrc/attention/launch.h:14-22]; a tensor-core tile always spans 128 keys, so with NT = 64
//     its two halves are two consecutive numerical tiles.
//   * x = acc * (sm_scale*log2e); running max m starts at -1e30 and is raised to max(m, tile max)
//     only if some row among the 32 rows of the warp has tile max - m > 6
//     [prefill_kernel.cuh:780-800, 872-890]; p = ex2.approx(x - m); l accumulates p in fp32.
//   * s = p * 2^(key scale byte 0 - 127); per 32 keys e = max(cvt.rp.ue8m0(amax/448), 61),
//     S = cvt.rn.satfinite.e4m3(s * 2^(127-e))  [prefill_kernel.cuh:803-830, 905-935].
//   * out = O / (l + 2^(sink*log2e - m)), 0 if l == 0; lse = m*ln2 + ln l (+inf if no key);
//     max_logits = true max * ln2 [prefill_kernel.cuh:988-1019]; decode splits write O/l and
//     log2(l)+m for the combine step [decode_kernel.cuh:199-218].
//
// Every wait is bounded (see sm100_ptx.cuh); on expiry the pair raises `fault` and leaves through
// the normal tear-down.
#pragma once

#include <cuda_bf16.h>
#include <math_constants.h>

#include "sm100_ptx.cuh"

namespace mxdsa {

using namespace sm100;

static constexpr int kHeads = 64;
static constexpr int kDim = 512;
static constexpr int kRowBytes = 528;
static constexpr int kTileKeys = 128;    // keys per tensor-core tile
static constexpr int kStages = 2;        // K/V ring depth (64 KB per stage and CTA)
static constexpr int kScStages = 4;      // scale/validity ring depth
static constexpr int kThreads = 256;

// tensor-memory columns
static constexpr uint32_t kColO = 0;      // 256 columns
static constexpr uint32_t kColP = 256;    // 2 buffers x 64
static constexpr uint32_t kColQs = 384;   // 4: Q scale bytes 0-3 (rows 0-31, 32-63), bytes 4-7
static constexpr uint32_t kColKs = 388;   // 4: K scale bytes 0-3 (keys 0-31, 32-63 of the half), 4-7
static constexpr uint32_t kColSs = 392;   // 2 buffers x 4 (2 used)
static constexpr uint32_t kColVs = 400;   // 8: w words 0-7
static constexpr uint32_t kTmemCols = 512;

struct DeviceFault {
    int flag;       // 1 when any wait was abandoned
    int where;      // code of the first abandoned wait
};

struct AttnParams {
    // common
    const uint8_t* q;         // packed Q rows
    long long stride_q_tok, stride_q_b;  // bytes
    int s_q;                  // prefill: query tokens; decode: tokens per request
    int topk;                 // main index row length
    float scale_log2;         // sm_scale * log2(e), fp32 product as the reference forms it
    const float* attn_sink;   // [64] or null
    const int* indices;       // main index rows
    long long idx_stride_row; // elements between rows (prefill: pairs; decode: tokens)
    long long idx_stride_b;   // decode: elements between requests
    const int* topk_length;   // prefill [pairs], decode [b]; or null
    __nv_bfloat16* out;       // prefill [s_q][64][512]; decode [b][s_q][64][512]
    float* lse;               // prefill [s_q][64]; decode [b][s_q][64]
    float* max_logits;        // prefill only
    uint32_t w1[8], w2[8];
    DeviceFault* fault;
    // prefill
    int s_kv;
    int num_pairs;
    const uint8_t* kv_scales; // prefill: start of the 16-byte slot plane
    // decode
    int b;
    int page_size, rows_per_block;            // rows_per_block = stride_block / 512
    int extra_topk, extra_page_size, extra_rows_per_block;
    const uint8_t* kv;        // decode: pool base (scale slots live inside the pages)
    const uint8_t* extra_kv;
    long long stride_block, extra_stride_block; // bytes
    const int* extra_indices;
    long long eidx_stride_row, eidx_stride_b;
    const int* extra_topk_length;
    const int* sched_meta;    // [parts][8]
    const int* num_splits;    // [b+1]
    float* o_accum;           // [splits][s_q][64][512]
    float* lse_accum;         // [splits][s_q][64]
};

struct TensorMaps {
    CUtensorMap q;        // 5-D {128 B, 64 heads, 4 chunks, tokens, requests}
    CUtensorMap kv;       // 2-D {512 B, rows}
    CUtensorMap extra_kv; // decode only
};

// One unit of work for a CTA pair: a query pair and a range of 64-key blocks of its key list.
struct WorkItem {
    int req;            // decode: request; prefill: 0
    int pair;           // pair index inside the request (prefill: global pair)
    const int* row;     // main index row
    const int* erow;    // extra index row (decode) or null
    int len, elen;      // attended lengths
    int n_main_blocks;  // 64-key blocks of the main part
    int blk_begin, blk_end;
    int split;          // decode: 1 -> write fp32 partials for the combine step
    int split_idx;
};

struct __align__(1024) SmemPlan {
    uint8_t q[4 * 64 * 128];                       // [chunk][head][128 B], 128-byte swizzle
    uint8_t k[kStages][4 * 64 * 128];              // [chunk][key of this CTA][128 B]
    uint8_t v[kStages][2 * 128 * 128];             // [chunk of this CTA][key][128 B]
    uint8_t s[2][64 * 128];                        // [row][128 keys], 128-byte swizzle
    __align__(128) uint32_t q_sf[64 * 4];          // scale rows for tcgen05.cp (64 rows x 16 B)
    __align__(128) uint32_t k_sf[kScStages][64 * 4];
    __align__(128) uint32_t s_sf[2][64 * 4];
    __align__(128) uint32_t v_sf[2][64 * 4];
    __align__(16) float tok_scale[kScStages][kTileKeys];
    __align__(16) uint32_t valid[kScStages][4];
    float xmax[2][128];                            // row-max exchange between the two key halves
    float xl[128];                                 // l exchange at the end of a pair
    uint64_t bar_q_landed;                         // local: Q bytes landed
    uint64_t bar_q_full;                           // CTA0: Q data + scale rows of both CTAs ready
    uint64_t bar_q_empty;                          // both: last QK of the pair finished
    uint64_t bar_k_full[kStages], bar_v_full[kStages];      // CTA0
    uint64_t bar_k_empty[kStages], bar_v_empty[kStages];    // both
    uint64_t bar_sc_full[kScStages];               // CTA0: K scale rows of both CTAs written
    uint64_t bar_tok_full[kScStages];              // local: token scales + validity written
    uint64_t bar_sc_empty[kScStages];              // local: cp finished and softmax read the stage
    uint64_t bar_p_full[2];                        // both
    uint64_t bar_p_empty[2];                       // CTA0
    uint64_t bar_s_full[2][2];                     // CTA0: [buffer][key half]
    uint64_t bar_pv_half[2];                       // both: first key half of the tile accumulated
    uint64_t bar_pv_done[2];                       // both: whole tile accumulated
    uint64_t bar_o_empty;                          // CTA0: epilogue has drained O
    uint32_t tmem_base;
    int abort_word;
};

// ----------------------------------------------------------------------------------------------
template <bool DECODE> struct WorkIter {
    const AttnParams& p;
    int next_pair, pair_step;      // prefill
    int req, end_req;              // decode
    int meta[8];
    bool started;

    __device__ WorkIter(const AttnParams& params) : p(params), started(false) {
        if constexpr (!DECODE) {
            next_pair = blockIdx.x / 2;
            pair_step = gridDim.x / 2;
        } else {
            const int4* m = reinterpret_cast<const int4*>(p.sched_meta + 8 * blockIdx.y);
            int4 a = __ldg(m), b2 = __ldg(m + 1);
            meta[0] = a.x; meta[1] = a.y; meta[2] = a.z; meta[3] = a.w;
            meta[4] = b2.x; meta[5] = b2.y; meta[6] = b2.z; meta[7] = b2.w;
            req = meta[0];
            end_req = meta[0] >= p.b ? -1 : meta[1];
        }
    }
    template <int NT> __device__ bool next(WorkItem& w) {
        if constexpr (!DECODE) {
            if (next_pair >= p.num_pairs) return false;
            w.req = 0;
            w.pair = next_pair;
            next_pair += pair_step;
            w.row = p.indices + (long long)w.pair * p.idx_stride_row;
            w.erow = nullptr;
            w.len = p.topk_length ? __ldg(p.topk_length + w.pair) : p.topk;
            w.elen = 0;
            const int ntiles = max((w.len + NT - 1) / NT, 1);
            w.n_main_blocks = ntiles * (NT / 64);
            w.blk_begin = 0;
            w.blk_end = w.n_main_blocks;
            w.split = 0;
            w.split_idx = 0;
            return true;
        } else {
            if (req > end_req) return false;
            const int r = req++;
            w.req = r;
            w.pair = blockIdx.x / 2;
            w.row = p.indices + (long long)r * p.idx_stride_b + (long long)w.pair * p.idx_stride_row;
            w.erow = p.extra_topk > 0
                         ? p.extra_indices + (long long)r * p.eidx_stride_b + (long long)w.pair * p.eidx_stride_row
                         : nullptr;
            w.len = p.topk_length ? __ldg(p.topk_length + r) : p.topk;
            w.elen = p.extra_topk > 0 ? (p.extra_topk_length ? __ldg(p.extra_topk_length + r) : p.extra_topk) : 0;
            w.n_main_blocks = max((w.len + 63) / 64, 1);
            const int total = w.n_main_blocks + (w.elen + 63) / 64;
            w.blk_begin = r == meta[0] ? meta[2] : 0;
            w.blk_end = r == meta[1] ? meta[3] : total;
            w.split = r == meta[0] ? meta[5] : (r == meta[1] ? meta[6] : 0);
            w.split_idx = __ldg(p.num_splits + r) + (r == meta[0] ? meta[4] : 0);
            return true;
        }
    }
};

// Index and validity of the key at position `j` (0..63) of 64-key block `blk` of a work item.
// Returns the TMA row coordinate (-1 = no row, reads as zeros) and writes the byte address of
// the key's 16-byte scale slot.
template <bool DECODE>
__device__ __forceinline__ int key_lookup(const AttnParams& p, const WorkItem& w, int blk, int j, bool& valid,
                                          const uint8_t*& slot) {
    valid = false;
    slot = nullptr;
    if (blk >= w.blk_end) return -1;
    if constexpr (!DECODE) {
        const int pos = blk * 64 + j;
        if (pos >= p.topk) return -1;
        const int idx = __ldg(w.row + pos);
        valid = idx >= 0 && idx < p.s_kv && pos < w.len;
        if (idx >= 0 && idx < p.s_kv) slot = p.kv_scales + (long long)idx * 16;
        return idx;  // out-of-range rows read as zeros; masked by `valid`
    } else {
        const bool extra = blk >= w.n_main_blocks;
        const int pos = (extra ? blk - w.n_main_blocks : blk) * 64 + j;
        const int row_len = extra ? p.extra_topk : p.topk;
        const int idx = pos < row_len ? __ldg((extra ? w.erow : w.row) + pos) : -1;
        valid = idx != -1 && pos < (extra ? w.elen : w.len);
        if (!valid) return -1;
        const unsigned psz = extra ? p.extra_page_size : p.page_size;
        const unsigned page = (unsigned)idx / psz, in_page = (unsigned)idx % psz;
        slot = (extra ? p.extra_kv : p.kv) + (long long)page * (extra ? p.extra_stride_block : p.stride_block) +
               (long long)psz * kDim + (long long)in_page * 16;
        return (int)(page * (unsigned)(extra ? p.extra_rows_per_block : p.rows_per_block) + in_page);
    }
}

// multiply this thread's 256 O columns (its tensor-memory lane) by f
__device__ __forceinline__ void rescale_o(uint32_t lane_addr, float f) {
#pragma unroll 1
    for (int c = 0; c < 256; c += 32) {
        uint32_t v[32];
        tmem_ld32(lane_addr + kColO + c, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
        tmem_st32(lane_addr + kColO + c, v);
    }
    tmem_wait_st();
}

#define MXDSA_WAIT(bar, parity, code)                                   \
    do {                                                                \
        if (!mbar_wait(smem_u32(&(bar)), (parity), &sm.abort_word)) {   \
            raise_fault(p, sm, (code));                                 \
            goto done;                                                  \
        }                                                               \
    } while (0)

__device__ __noinline__ void raise_fault(const AttnParams& p, SmemPlan& sm, int code) {
    sm.abort_word = 1;
    // tell the peer CTA so that its roles stop waiting as well
    const uint32_t peer = map_to_cta(smem_u32(&sm.abort_word), cluster_cta_rank() ^ 1u);
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer), "r"(1) : "memory");
    if (atomicCAS(&p.fault->flag, 0, 1) == 0) p.fault->where = code;
}

template <bool DECODE, int NT>
__global__ void __launch_bounds__(kThreads, 1)
mxdsa_attn_kernel(const __grid_constant__ AttnParams p, const __grid_constant__ TensorMaps maps) {
    extern __shared__ uint8_t smem_raw[];
    SmemPlan& sm = *reinterpret_cast<SmemPlan*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const uint32_t cta = cluster_cta_rank();
    const uint32_t peer = cta ^ 1u;

    // ------------------------------------------------------------------ set-up
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&sm.bar_q_landed), 1);
        mbar_init(smem_u32(&sm.bar_q_full), 2);
        mbar_init(smem_u32(&sm.bar_q_empty), 1);
        for (int i = 0; i < kStages; ++i) {
            mbar_init(smem_u32(&sm.bar_k_full[i]), 2);
            mbar_init(smem_u32(&sm.bar_v_full[i]), 2);
            mbar_init(smem_u32(&sm.bar_k_empty[i]), 1);
            mbar_init(smem_u32(&sm.bar_v_empty[i]), 1);
        }
        for (int i = 0; i < kScStages; ++i) {
            mbar_init(smem_u32(&sm.bar_sc_full[i]), 2);
            mbar_init(smem_u32(&sm.bar_tok_full[i]), 1);
            mbar_init(smem_u32(&sm.bar_sc_empty[i]), 1 + 4);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&sm.bar_p_full[i]), 1);
            mbar_init(smem_u32(&sm.bar_p_empty[i]), 8);
            mbar_init(smem_u32(&sm.bar_s_full[i][0]), 8);
            mbar_init(smem_u32(&sm.bar_s_full[i][1]), 8);
            mbar_init(smem_u32(&sm.bar_pv_half[i]), 1);
            mbar_init(smem_u32(&sm.bar_pv_done[i]), 1);
        }
        mbar_init(smem_u32(&sm.bar_o_empty), 8);
        sm.abort_word = 0;
        fence_mbar_init();
    }
    if (warp == 3) {
        // V dimension scales: rows 0-31 feed lane quadrants 0,1 (dims of CTA 0 = w1), rows 32-63
        // quadrants 2,3 (dims of CTA 1 = w2); every row of a group is the same four words.
        for (int i = lane; i < 64; i += 32) {
            const uint32_t* w = i < 32 ? p.w1 : p.w2;
            for (int c = 0; c < 4; ++c) {
                sm.v_sf[0][i * 4 + c] = w[c];
                sm.v_sf[1][i * 4 + c] = w[4 + c];
            }
        }
        fence_proxy_async_smem();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&maps.q);
        prefetch_tensormap(&maps.kv);
        if (DECODE) prefetch_tensormap(&maps.extra_kv);
    }
    __syncthreads();
    cluster_sync();
    if (warp == 2) {
        tmem_alloc<2>(smem_u32(&sm.tmem_base), kTmemCols);
        tmem_relinquish<2>();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    const uint64_t desc_k128 = smem_desc_base(16, 1024, 2);   // K-major, 128-byte swizzle
    const uint64_t desc_v = smem_desc_base(16384, 1024, 2);   // MN-major, 128-byte swizzle
    const uint64_t desc_sf = smem_desc_base(0, 128, 0);       // scale rows, 16 bytes each

    // ------------------------------------------------------------------ roles
    if (warp == 0) {
        // ===================== gather producer =====================
        WorkIter<DECODE> it(p);
        WorkItem w;
        uint32_t gt = 0;  // tiles issued so far (ring position)
        const uint32_t k_full0 = map_to_cta(smem_u32(&sm.bar_k_full[0]), 0);
        const uint32_t v_full0 = map_to_cta(smem_u32(&sm.bar_v_full[0]), 0);
        while (it.template next<NT>(w)) {
            const int ntiles = (w.blk_end - w.blk_begin + 1) / 2;
            if (ntiles <= 0) continue;  // never produced by the scheduler; keeps the roles in step
            for (int t = 0; t < ntiles; ++t, ++gt) {
                const uint32_t s = gt % kStages, ph = (gt / kStages) & 1;
                // lane L owns keys 4L..4L+3 of the tile (block = L/16)
                int coord[4];
                const int blk = w.blk_begin + 2 * t + lane / 16;
                bool extra_pool = false;
                if constexpr (DECODE) extra_pool = blk >= w.n_main_blocks;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    bool valid;
                    const uint8_t* slot;
                    coord[i] = key_lookup<DECODE>(p, w, blk, (lane % 16) * 4 + i, valid, slot);
                }
                // K: keys of this CTA's half (block `cta`), 16 groups x 4 chunks = 2 copies per lane
                const int src_lane = cta * 16 + lane % 16;
                int kc[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) kc[i] = __shfl_sync(0xffffffffu, coord[i], src_lane);
                const bool k_extra = __shfl_sync(0xffffffffu, (int)extra_pool, src_lane) != 0;
                MXDSA_WAIT(sm.bar_k_empty[s], ph ^ 1, 10);
                if (lane == 0) {
                    const uint32_t bar = k_full0 + s * 8;
                    asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar),
                                 "r"(4 * 64 * 128)
                                 : "memory");
                }
                {
                    const void* map = (DECODE && k_extra) ? &maps.extra_kv : &maps.kv;
                    const int g = lane % 16;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int chunk = 2 * (lane / 16) + j;
                        tma_gather4_pair(smem_u32(&sm.k[s][chunk * 8192 + g * 512]), map, chunk * 128, kc[0], kc[1],
                                         kc[2], kc[3], k_full0 + s * 8, kEvictLast);
                    }
                }
                // V: all 128 keys, this CTA's two 128-byte chunks
                MXDSA_WAIT(sm.bar_v_empty[s], ph ^ 1, 11);
                if (lane == 0) {
                    const uint32_t bar = v_full0 + s * 8;
                    asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar),
                                 "r"(2 * 128 * 128)
                                 : "memory");
                }
                {
                    const void* map = (DECODE && extra_pool) ? &maps.extra_kv : &maps.kv;
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        tma_gather4_pair(smem_u32(&sm.v[s][j * 16384 + lane * 512]), map, (2 * cta + j) * 128,
                                         coord[0], coord[1], coord[2], coord[3], v_full0 + s * 8, kEvictLast);
                }
            }
        }
    } else if (warp == 1) {
        // ===================== QK issuer (CTA 0) =====================
        if (cta == 0 && lane == 0) {
            WorkIter<DECODE> it(p);
            WorkItem w;
            uint32_t gt = 0, gw = 0;
            const uint32_t p_full_peer = map_to_cta(smem_u32(&sm.bar_p_full[0]), 1);
            const uint32_t k_empty_peer = map_to_cta(smem_u32(&sm.bar_k_empty[0]), 1);
            const uint32_t sc_empty_peer = map_to_cta(smem_u32(&sm.bar_sc_empty[0]), 1);
            const uint32_t q_empty_peer = map_to_cta(smem_u32(&sm.bar_q_empty), 1);
            const uint64_t a_base = smem_desc(desc_k128, smem_u32(sm.q));
            while (it.template next<NT>(w)) {
                const int ntiles = (w.blk_end - w.blk_begin + 1) / 2;
            if (ntiles <= 0) continue;  // never produced by the scheduler; keeps the roles in step
                MXDSA_WAIT(sm.bar_q_full, gw & 1, 20);
                tc_fence_after();
                tmem_cp_sf_pair(tmem + kColQs, smem_desc(desc_sf, smem_u32(sm.q_sf)));
                for (int t = 0; t < ntiles; ++t, ++gt) {
                    const uint32_t s = gt % kStages, ph = (gt / kStages) & 1;
                    const uint32_t sc = gt % kScStages, sph = (gt / kScStages) & 1;
                    const uint32_t b = gt & 1, bph = (gt >> 1) & 1;
                    MXDSA_WAIT(sm.bar_sc_full[sc], sph, 21);
                    MXDSA_WAIT(sm.bar_p_empty[b], bph ^ 1, 22);
                    MXDSA_WAIT(sm.bar_k_full[s], ph, 23);
                    tc_fence_after();
                    tmem_cp_sf_pair(tmem + kColKs, smem_desc(desc_sf, smem_u32(sm.k_sf[sc])));
                    const uint64_t b_base = smem_desc(desc_k128, smem_u32(sm.k[s]));
#pragma unroll
                    for (int kk = 0; kk < 16; ++kk) {
                        // Q bytes (kk%8)*64 + (kk/8)*32 of the row meet K bytes 32*kk
                        const uint32_t a_off = ((kk % 8) / 2) * 8192 + ((kk % 8) % 2) * 64 + (kk / 8) * 32;
                        const uint32_t b_off = (kk / 4) * 8192 + (kk % 4) * 32;
                        mma_mxf8<2>(tmem + kColP + b * 64, a_base + (a_off >> 4), b_base + (b_off >> 4),
                                    mx_idesc(128, 128, false, kk & 3, (kk / 2) & 3), tmem + kColQs + 2 * ((kk / 4) & 1),
                                    tmem + kColKs + 2 * (kk / 8), kk != 0);
                    }
                    mma_commit<2>(smem_u32(&sm.bar_p_full[b]));
                    mma_commit<2>(p_full_peer + b * 8);
                    mma_commit<2>(smem_u32(&sm.bar_k_empty[s]));
                    mma_commit<2>(k_empty_peer + s * 8);
                    mma_commit<2>(smem_u32(&sm.bar_sc_empty[sc]));
                    mma_commit<2>(sc_empty_peer + sc * 8);
                }
                mma_commit<2>(smem_u32(&sm.bar_q_empty));
                mma_commit<2>(q_empty_peer);
                ++gw;
            }
        }
    } else if (warp == 2) {
        // ===================== PV issuer (CTA 0) =====================
        if (cta == 0 && lane == 0) {
            WorkIter<DECODE> it(p);
            WorkItem w;
            uint32_t gt = 0, gw = 0;
            const uint32_t pv_half_peer = map_to_cta(smem_u32(&sm.bar_pv_half[0]), 1);
            const uint32_t pv_done_peer = map_to_cta(smem_u32(&sm.bar_pv_done[0]), 1);
            const uint32_t v_empty_peer = map_to_cta(smem_u32(&sm.bar_v_empty[0]), 1);
            tmem_cp_sf_pair(tmem + kColVs, smem_desc(desc_sf, smem_u32(sm.v_sf[0])));
            tmem_cp_sf_pair(tmem + kColVs + 4, smem_desc(desc_sf, smem_u32(sm.v_sf[1])));
            while (it.template next<NT>(w)) {
                const int ntiles = (w.blk_end - w.blk_begin + 1) / 2;
            if (ntiles <= 0) continue;  // never produced by the scheduler; keeps the roles in step
                MXDSA_WAIT(sm.bar_o_empty, (gw & 1) ^ 1, 30);
                tc_fence_after();
                for (int t = 0; t < ntiles; ++t, ++gt) {
                    const uint32_t s = gt % kStages, ph = (gt / kStages) & 1;
                    const uint32_t b = gt & 1, bph = (gt >> 1) & 1;
                    MXDSA_WAIT(sm.bar_v_full[s], ph, 31);
                    const uint64_t a_base = smem_desc(desc_k128, smem_u32(sm.s[b]));
                    const uint64_t b_base = smem_desc(desc_v, smem_u32(sm.v[s]));
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        MXDSA_WAIT(sm.bar_s_full[b][h], bph, 32 + h);
                        tc_fence_after();
                        tmem_cp_sf_pair(tmem + kColSs + 4 * b, smem_desc(desc_sf, smem_u32(sm.s_sf[b])));
#pragma unroll
                        for (int ks = 2 * h; ks < 2 * h + 2; ++ks) {
#pragma unroll
                            for (int n = 0; n < 2; ++n) {
                                mma_mxf8<2>(tmem + kColO + n * 128, a_base + ((ks * 32) >> 4),
                                            b_base + ((n * 16384 + ks * 4096) >> 4),
                                            mx_idesc(128, 256, true, ks, NT == 64 ? (ks & 1) : ks), tmem + kColSs + 4 * b,
                                            tmem + kColVs + 4 * n, !(t == 0 && ks == 0));
                            }
                        }
                        if (h == 0) {
                            mma_commit<2>(smem_u32(&sm.bar_pv_half[b]));
                            mma_commit<2>(pv_half_peer + b * 8);
                        }
                    }
                    mma_commit<2>(smem_u32(&sm.bar_pv_done[b]));
                    mma_commit<2>(pv_done_peer + b * 8);
                    mma_commit<2>(smem_u32(&sm.bar_v_empty[s]));
                    mma_commit<2>(v_empty_peer + s * 8);
                }
                ++gw;
            }
        }
    } else if (warp == 3) {
        // ===================== operand stager =====================
        WorkIter<DECODE> it(p);
        WorkItem w;
        uint32_t gt = 0, gw = 0;
        const uint32_t q_full0 = map_to_cta(smem_u32(&sm.bar_q_full), 0);
        const uint32_t sc_full0 = map_to_cta(smem_u32(&sm.bar_sc_full[0]), 0);
        while (it.template next<NT>(w)) {
            const int ntiles = (w.blk_end - w.blk_begin + 1) / 2;
            if (ntiles <= 0) continue;  // never produced by the scheduler; keeps the roles in step
            // ---- Q tile and Q scale rows of this CTA's token
            const int tok = min(2 * w.pair + (int)cta, p.s_q - 1);
            MXDSA_WAIT(sm.bar_q_empty, (gw & 1) ^ 1, 40);
            if (lane == 0) {
                mbar_expect_tx(smem_u32(&sm.bar_q_landed), 4 * 64 * 128);
                asm volatile(
                    "cp.async.bulk.tensor.5d.shared::cta.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
                    " [%0], [%1, {%2, %3, %4, %5, %6}], [%7], %8;"
                    :
                    : "r"(smem_u32(sm.q)), "l"(&maps.q), "r"(0), "r"(0), "r"(0), "r"(tok), "r"(w.req),
                      "r"(smem_u32(&sm.bar_q_landed)), "l"(kEvictFirst)
                    : "memory");
            }
            {
                // lane L stages heads L and L+32: words {bytes0-3[L], bytes0-3[L+32], bytes4-7[L], bytes4-7[L+32]}
                const uint8_t* base = p.q + (long long)w.req * p.stride_q_b + (long long)tok * p.stride_q_tok + kDim;
                const uint2 lo = __ldg(reinterpret_cast<const uint2*>(base + (long long)lane * kRowBytes));
                const uint2 hi = __ldg(reinterpret_cast<const uint2*>(base + (long long)(lane + 32) * kRowBytes));
                const uint4 row = make_uint4(lo.x, hi.x, lo.y, hi.y);
                *reinterpret_cast<uint4*>(&sm.q_sf[lane * 4]) = row;
                *reinterpret_cast<uint4*>(&sm.q_sf[(lane + 32) * 4]) = row;
                fence_proxy_async_smem();
                __syncwarp();
            }
            MXDSA_WAIT(sm.bar_q_landed, gw & 1, 41);
            if (lane == 0) mbar_arrive_cluster(q_full0);
            // ---- per tile: K scale rows, key token scales, validity
            for (int t = 0; t < ntiles; ++t, ++gt) {
                const uint32_t sc = gt % kScStages, sph = (gt / kScStages) & 1;
                uint2 sv[4];
                uint32_t vbits[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // lane L looks after keys L, L+32 (block 0) and L+64, L+96 (block 1)
                    bool valid;
                    const uint8_t* slot;
                    key_lookup<DECODE>(p, w, w.blk_begin + 2 * t + j / 2, (j % 2) * 32 + lane, valid, slot);
                    sv[j] = slot != nullptr ? __ldg(reinterpret_cast<const uint2*>(slot)) : make_uint2(0u, 0u);
                    vbits[j] = __ballot_sync(0xffffffffu, valid);
                }
                MXDSA_WAIT(sm.bar_sc_empty[sc], sph ^ 1, 42);
                // rows for tcgen05.cp: row r = (half of the tile)*32 + L holds keys (half*64 + L) and (+32):
                // {bytes0-3[k0], bytes0-3[k1], bytes4-7[k0], bytes4-7[k1]}
                *reinterpret_cast<uint4*>(&sm.k_sf[sc][lane * 4]) = make_uint4(sv[0].x, sv[1].x, sv[0].y, sv[1].y);
                *reinterpret_cast<uint4*>(&sm.k_sf[sc][(32 + lane) * 4]) = make_uint4(sv[2].x, sv[3].x, sv[2].y, sv[3].y);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    sm.tok_scale[sc][j * 32 + lane] = __uint_as_float((sv[j].x & 0xffu) << 23);
                if (lane < 4) sm.valid[sc][lane] = vbits[lane];
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(&sm.bar_tok_full[sc]));
                    mbar_arrive_cluster(sc_full0 + sc * 8);
                }
            }
            ++gw;
        }
    } else {
        // ===================== softmax + epilogue (warps 4-7) =====================
        const int q4 = warp - 4;                 // lane quadrant of tensor memory
        const int L = q4 * 32 + lane;            // tensor-memory lane
        const int row = L % 64;                  // head
        const int half = L / 64;                 // key half of a tile / dim half of O
        const uint32_t lane_addr = tmem + (uint32_t(q4 * 32) << 16);
        const uint32_t p_empty0 = map_to_cta(smem_u32(&sm.bar_p_empty[0]), 0);
        const uint32_t s_full0 = map_to_cta(smem_u32(&sm.bar_s_full[0][0]), 0);
        const uint32_t o_empty0 = map_to_cta(smem_u32(&sm.bar_o_empty), 0);
        WorkIter<DECODE> it(p);
        WorkItem w;
        uint32_t gt = 0;
        while (it.template next<NT>(w)) {
            const int ntiles = (w.blk_end - w.blk_begin + 1) / 2;
            if (ntiles <= 0) continue;  // never produced by the scheduler; keeps the roles in step
            float m = -1e30f, l = 0.f, real_m = -CUDART_INF_F;
            for (int t = 0; t < ntiles; ++t, ++gt) {
                const uint32_t sc = gt % kScStages, sph = (gt / kScStages) & 1;
                const uint32_t b = gt & 1, bph = (gt >> 1) & 1;
                MXDSA_WAIT(sm.bar_tok_full[sc], sph, 50);
                const uint32_t v0 = sm.valid[sc][2 * half], v1 = sm.valid[sc][2 * half + 1];
                MXDSA_WAIT(sm.bar_p_full[b], bph, 51);
                tc_fence_after();
                float x[64];
                tmem_ld32(lane_addr + kColP + b * 64, reinterpret_cast<uint32_t*>(x));
                tmem_ld32(lane_addr + kColP + b * 64 + 32, reinterpret_cast<uint32_t*>(x + 32));
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(p_empty0 + b * 8);
                float own_max = -CUDART_INF_F;
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const bool ok = ((i < 32 ? v0 : v1) >> (i & 31)) & 1u;
                    x[i] = ok ? x[i] : -CUDART_INF_F;
                    own_max = fmaxf(own_max, x[i]);
                }
                own_max *= p.scale_log2;
                sm.xmax[gt & 1][L] = own_max;
                named_bar_sync(1, 128);
                const float peer_max = sm.xmax[gt & 1][L ^ 64];
                // numerical tiles: NT = 128 -> one per tensor-core tile; NT = 64 -> key half 0 then 1
                float m_used, scale0 = 1.f, scale1 = 1.f;
                bool grow0, grow1 = false;
                if constexpr (NT == 128) {
                    const float tmax = fmaxf(own_max, peer_max);
                    real_m = fmaxf(real_m, tmax);
                    grow0 = __any_sync(0xffffffffu, tmax - m > 6.0f);
                    const float nm = grow0 ? fmaxf(m, tmax) : m;
                    scale0 = grow0 ? ex2_approx(m - nm) : 1.f;
                    m = nm;
                    m_used = m;
                } else {
                    const float t0 = half == 0 ? own_max : peer_max;
                    const float t1 = half == 0 ? peer_max : own_max;
                    real_m = fmaxf(real_m, fmaxf(t0, t1));
                    grow0 = __any_sync(0xffffffffu, t0 - m > 6.0f);
                    const float m1 = grow0 ? fmaxf(m, t0) : m;
                    scale0 = grow0 ? ex2_approx(m - m1) : 1.f;
                    grow1 = __any_sync(0xffffffffu, t1 - m1 > 6.0f);
                    const float m2 = grow1 ? fmaxf(m1, t1) : m1;
                    scale1 = grow1 ? ex2_approx(m1 - m2) : 1.f;
                    m_used = half == 0 ? m1 : m2;
                    m = m2;
                }
                // probabilities, key-scaled, re-quantised per 32 keys
                const float* tok = &sm.tok_scale[sc][half * 64];
                float sum = 0.f;
                uint32_t s8[16];
                uint32_t e_bytes = 0;
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    float amax = 0.f;
                    float partial[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int c = g * 32 + i;
                        const float pv = ex2_approx(fmaf(x[c], p.scale_log2, -m_used));
                        partial[i & 3] += pv;
                        const float sv = pv * tok[c];
                        amax = fmaxf(amax, sv);
                        x[c] = sv;
                    }
                    sum += (partial[0] + partial[1]) + (partial[2] + partial[3]);
                    uint32_t e = cvt_ue8m0_roundup(amax > 0.f ? __fdividef(amax, 448.0f) : 1.0f);
                    e = max(e, 61u);
                    e_bytes |= e << (8 * g);
                    const float mul = __uint_as_float((254u - e) << 23);
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const int c = g * 32 + i;
                        const uint32_t lo = cvt_e4m3x2(x[c] * mul, x[c + 1] * mul);
                        const uint32_t hi = cvt_e4m3x2(x[c + 2] * mul, x[c + 3] * mul);
                        s8[c / 4] = lo | (hi << 16);
                    }
                }
                // l bookkeeping: every m update rescales both halves' partial sums
                if constexpr (NT == 128) {
                    l = fmaf(l, scale0, sum);
                } else {
                    if (half == 0) l = fmaf(l, scale0, sum) * scale1;
                    else l = fmaf(l * scale0, scale1, sum);
                }
                // S buffer b is free once the PV of tile gt-2 has finished
                if (gt >= 2) MXDSA_WAIT(sm.bar_pv_done[b], bph ^ 1, 52);
                {
                    uint8_t* srow = sm.s[b];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        *reinterpret_cast<uint4*>(srow + swz128(row, half * 64 + i * 16)) =
                            make_uint4(s8[4 * i], s8[4 * i + 1], s8[4 * i + 2], s8[4 * i + 3]);
                    // scale rows: row (row%32) and its copy at +32; word row/32; bytes 2*half, 2*half+1
                    uint16_t* w0 = reinterpret_cast<uint16_t*>(&sm.s_sf[b][(row % 32) * 4 + row / 32]) + half;
                    uint16_t* w1 = reinterpret_cast<uint16_t*>(&sm.s_sf[b][(32 + row % 32) * 4 + row / 32]) + half;
                    *w0 = (uint16_t)e_bytes;
                    *w1 = (uint16_t)e_bytes;
                }
                // O rescale before the first key half is accumulated
                if (grow0 && t > 0) {
                    MXDSA_WAIT(sm.bar_pv_done[b ^ 1], ((gt - 1) >> 1) & 1, 53);
                    tc_fence_after();
                    rescale_o(lane_addr, scale0);
                    tc_fence_before();
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(s_full0 + (b * 2 + 0) * 8);
                if constexpr (NT == 64) {
                    if (grow1) {
                        MXDSA_WAIT(sm.bar_pv_half[b], bph, 54);
                        tc_fence_after();
                        rescale_o(lane_addr, scale1);
                        tc_fence_before();
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_cluster(s_full0 + (b * 2 + 1) * 8);
                    mbar_arrive(smem_u32(&sm.bar_sc_empty[sc]));
                }
            }
            // ---------------- end of the pair: combine the halves' l, drain O
            if (real_m == -CUDART_INF_F) {
                l = 0.f;
                m = -CUDART_INF_F;
            }
            sm.xl[L] = l;
            named_bar_sync(1, 128);
            const float l_tot = l + sm.xl[L ^ 64];
            const uint32_t last = gt - 1;
            MXDSA_WAIT(sm.bar_pv_done[last & 1], (last >> 1) & 1, 55);
            tc_fence_after();
            const int tok_idx = 2 * w.pair + (int)cta;
            const bool store = tok_idx < p.s_q;
            const float sink = p.attn_sink ? __ldg(p.attn_sink + row) : -CUDART_INF_F;
            float oscale;
            if (!DECODE || !w.split) oscale = __fdividef(1.0f, l_tot + ex2_approx(fmaf(sink, CUDART_L2E_F, -m)));
            else oscale = __fdividef(1.0f, l_tot);
            if (l_tot == 0.f) oscale = 0.f;
            if (half == 0 && store) {
                if (!DECODE || !w.split) {
                    float lse = fmaf(m, CUDART_LN2_F, CUDART_LN2_F * lg2_approx(l_tot));
                    if (l_tot == 0.f || lse == -CUDART_INF_F) lse = CUDART_INF_F;
                    const long long o = ((long long)w.req * p.s_q + tok_idx) * kHeads + row;
                    p.lse[o] = lse;
                    if (!DECODE) p.max_logits[o] = real_m * CUDART_LN2_F;
                } else {
                    p.lse_accum[((long long)w.split_idx * p.s_q + tok_idx) * kHeads + row] = lg2_approx(l_tot) + m;
                }
            }
            if (!DECODE || !w.split) {
                __nv_bfloat16* dst = p.out + (((long long)w.req * p.s_q + tok_idx) * kHeads + row) * kDim + half * 256;
#pragma unroll 1
                for (int c = 0; c < 256; c += 32) {
                    float o[32];
                    tmem_ld32(lane_addr + kColO + c, reinterpret_cast<uint32_t*>(o));
                    tmem_wait_ld();
                    if (store) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            __nv_bfloat162 v[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                v[j] = __floats2bfloat162_rn(o[i + 2 * j] * oscale, o[i + 2 * j + 1] * oscale);
                            *reinterpret_cast<uint4*>(dst + c + i) = *reinterpret_cast<uint4*>(v);
                        }
                    }
                }
            } else {
                float* dst = p.o_accum + (((long long)w.split_idx * p.s_q + tok_idx) * kHeads + row) * kDim + half * 256;
#pragma unroll 1
                for (int c = 0; c < 256; c += 32) {
                    float o[32];
                    tmem_ld32(lane_addr + kColO + c, reinterpret_cast<uint32_t*>(o));
                    tmem_wait_ld();
                    if (store) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4*>(dst + c + i) =
                                make_float4(o[i] * oscale, o[i + 1] * oscale, o[i + 2] * oscale, o[i + 3] * oscale);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(o_empty0);
        }
    }

done:
    // ------------------------------------------------------------------ tear-down
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 2) tmem_dealloc<2>(tmem, kTmemCols);
}

}  // namespace mxdsa

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
// Roles (warp-specialised, 28 warps per CTA; the launch gives every thread 72 registers, re-balanced with
// setmaxnreg to 48 / 32 / 64 / 104 / 48 for the five kinds of warp below)
//   warps 0-3   K producers: read key indices one tile ahead and copy the selected rows of this CTA's 64 keys
//               into the K ring with 16-byte cp.async; one warp instruction moves one 512-byte row straight
//               into the 128-byte-swizzled operand layout.  The same warps gather the 8 scale bytes of all 128
//               keys of the tile into the row layout that tcgen05.cp wants, and vote the validity bits.
//   warps 4-7   V producers: TMA gather4 (four rows x 128 bytes per request) of the 256-byte halves of all 128
//               keys into the V ring; every lane works out one key's row coordinate, eight lanes per warp
//               collect four each and issue.  The bytes of both CTAs complete on one barrier of CTA 0.
//               (cp.async carrying V as well makes the K rows -- which the next QK waits for -- land late; the
//               copy engine alone is the slower of the two paths, which is why K is not on it.)
//   warp 8      CTA 0: QK issuer for even tiles      (issuers run as converged warps, one elected lane
//   warp 9      CTA 0: QK issuer for odd tiles        issues fully unrolled MMAs; each has its own P buffer
//   warp 10     CTA 0: PV issuer                      and scale columns)
//   warp 11     operand stager: Q tile by TMA + Q scale rows per pair (the next pair's tile is requested into
//               L2 a pair ahead); per tile it waits for "K landed", fences and publishes "scale rows ready"
//               to CTA 0 -- no global load sits between a landed K tile and its QK -- then derives the key
//               token scales and validity words that the softmax reads.
//   warps 12-23 softmax: three groups of four warps take tiles in turn (each thread one row and one 64-key
//               half of its tile): P -> registers, running max with lazy rescale handed from group to group,
//               exp2, token scale, per-32-key UE8M0 requantisation to E4M3 S (ring of three), O rescale.
//               At the end of a pair the groups add up their row sums and hand 1/l to the epilogue warps.
//   warps 24-27 epilogue: drain O (tensor memory -> bf16 `out` through small staging tiles and tiled TMA
//               stores, or fp32 split partials) while the other warps are already working on the next pair;
//               only that pair's first PV waits, and only until the last columns have been read.
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
// Every wait is bounded (the loops are written out at the wait sites below); on expiry the pair raises `fault` and leaves through
// the normal tear-down.
#pragma once

#include <cuda_bf16.h>
#include <math_constants.h>

#include "sm100_ptx.cuh"


#ifndef MXDSA_V_HINT
#define MXDSA_V_HINT kEvictLast
#endif
// How many tiles ahead of the copies the index rows are asked into L2 (0: never)
#ifndef MXDSA_INDEX_AHEAD
#define MXDSA_INDEX_AHEAD 4
#endif
// 1: the epilogue warps write bf16 output through shared memory and tiled TMA stores; 0: 32-byte stores per lane
#ifndef MXDSA_TMA_EPILOGUE
#define MXDSA_TMA_EPILOGUE 1
#endif
#ifndef MXDSA_OUT_TILES
#define MXDSA_OUT_TILES 2
#endif
#ifndef MXDSA_K_STAGES
#define MXDSA_K_STAGES 2
#define MXDSA_V_STAGES 2
#endif
#ifndef MXDSA_S_BUFS
#define MXDSA_S_BUFS 3
#endif

namespace mxdsa {

using namespace sm100;

static constexpr int kHeads = 64;
static constexpr int kDim = 512;
static constexpr int kRowBytes = 528;
static constexpr int kTileKeys = 128;    // keys per tensor-core tile
static constexpr int kKStages = MXDSA_K_STAGES;       // K ring depth (32 KB per stage and CTA); freed as soon as QK is done
static constexpr int kVStages = MXDSA_V_STAGES;       // V ring depth (32 KB per stage and CTA); held until PV is done
static constexpr int kOutTiles = MXDSA_OUT_TILES;   // staging tiles per epilogue warp: stores in flight while the next tile is filled
static constexpr int kSBufs = MXDSA_S_BUFS;      // S (quantised probabilities) ring: how far the softmax may run ahead of PV
#ifndef MXDSA_SC_STAGES
#define MXDSA_SC_STAGES 4
#endif
static constexpr int kScStages = MXDSA_SC_STAGES;      // scale/validity ring depth; also the depth of the
                                         // per-tile "QK done" / "PV done" barrier rings
// registers per thread that a launch of 512 + 128 G threads gets (65536 / threads, rounded down to a multiple of 8)
__host__ __device__ constexpr int launch_regs(int g) { return g == 2 ? 80 : 72; }
static constexpr int kBaseThreads = 512;   // warps 0-11: K producers, V producers, control; then G x 4 softmax warps; then 4 epilogue warps
static constexpr int kMaxGroups = 3;     // softmax groups of four warps (template parameter G = 2 or 3); tile g is handled by group g % G

// tensor-memory columns
static constexpr uint32_t kColO = 0;      // 256 columns
static constexpr uint32_t kColP = 256;    // 2 buffers x 64
static constexpr uint32_t kColQs = 384;   // 2 x 4 (one set per QK issuer): Q scale bytes 0-3 / 4-7 of rows 0-31, 32-63
static constexpr uint32_t kColKs = 392;   // 2 x 4: K scale bytes 0-3 / 4-7 of keys 0-31, 32-63 of the half
static constexpr uint32_t kColSs = 400;   // kSBufs x 4 (2 used)
static constexpr uint32_t kColVs = 416;   // 8: w words 0-7
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
    const uint8_t* kv_scales; // prefill: start of the 16-byte slot plane (kv = data rows)
    // decode
    int b;
    int page_size, rows_per_block;            // rows_per_block = stride_block / 512
    int extra_topk, extra_page_size, extra_rows_per_block;
    const uint8_t* kv;        // prefill: data rows; decode: pool base (slots live inside the pages)
    const uint8_t* extra_kv;
    long long stride_block, extra_stride_block; // bytes
    const int* extra_indices;
    long long eidx_stride_row, eidx_stride_b;
    const int* extra_topk_length;
    const int* sched_meta;    // [parts][8]
    const int* num_splits;    // [b+1]
    float* o_accum;           // [splits][s_q][64][512]
    float* lse_accum;         // [splits][s_q][64]
    int page_shift, extra_page_shift;         // log2(page size) when it is a power of two, else -1
    unsigned pool_rows32, extra_pool_rows32;  // decode: keys in each pool (num_blocks * page_size, at most 2^31); indices beyond are skipped
    unsigned row_gap, extra_row_gap;          // rows_per_block - page_size: rows of the 512-byte view that a page's scale slots take
};

struct TensorMaps {
    CUtensorMap q;        // 5-D {128 B, 64 heads, 4 chunks, tokens, requests}
    CUtensorMap kv;       // 2-D {512 B, rows}: data rows of the (main) KV store, row pitch 512 B; gather4 source for V
    CUtensorMap ekv;      // decode: the same over the extra pool
    CUtensorMap out;      // 2-D {512 bf16, tokens x 64 heads} over the output; one store box = 32 columns of 32 rows
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
    uint8_t k[kKStages][4 * 64 * 128];             // [chunk][key of this CTA][128 B]
    uint8_t v[kVStages][2 * 128 * 128];            // [chunk of this CTA][key][128 B]
    uint8_t s[kSBufs][64 * 128];                        // [row][128 keys], 128-byte swizzle
#if MXDSA_TMA_EPILOGUE
    uint8_t o_stage[4][kOutTiles][32 * 64];        // per epilogue warp: tiles of 32 rows x 32 bf16 on their way out, 64-byte swizzle
#endif
    __align__(16) uint16_t kvalid[kKStages][8];     // validity bits of the tile's keys, 16 per entry (K ring)
    __align__(128) uint32_t q_sf[64 * 4];          // scale rows for tcgen05.cp (64 rows x 16 B)
    __align__(128) uint32_t k_sf[kKStages][64 * 4];   // per K stage: K scale rows for tcgen05.cp, gathered by the producers with the rows
    __align__(128) uint32_t s_sf[kSBufs][64 * 4];
    __align__(16) float tok_scale[kScStages][kTileKeys];
    __align__(16) uint32_t valid[kScStages][4];
    float xmax[kMaxGroups][2][128];                   // [group][parity of the group's tile count][lane]: row max of the lane's 64 keys
    float m_pub[kMaxGroups][64];                      // [group][row]: running max after the group's latest tile
    float xl[kMaxGroups * 128], xr[kMaxGroups * 128];    // [group*128 + lane]: partial l and true max at the end of a pair
    uint64_t bar_q_landed;                         // local: Q bytes landed
    uint64_t bar_q_full;                           // CTA0: Q data + scale rows of both CTAs ready
    uint64_t bar_q_empty;                          // both: every QK of the pair finished (2 arrivals)
    uint64_t bar_k_landed[kKStages];               // local: this CTA's K rows landed (128 arrivals)
    uint64_t bar_v_full[kVStages];                 // CTA0: V rows of both CTAs landed (8 arrivals + 64 KB of gather4 bytes)
    uint64_t bar_qk_done[kScStages];               // both: QK of tile g finished (ring by g % 4)
    uint64_t bar_pv_done[kScStages];               // both: PV of tile g finished
    uint64_t bar_pv_half[kSBufs];                       // both: first key half accumulated (64-key tiles)
    uint64_t bar_sc_full[kScStages];               // CTA0: K scale rows of both CTAs written
    uint64_t bar_tok_full[kScStages];              // local: token scales + validity written
    uint64_t bar_tok_empty[kScStages];             // local: softmax has read the stage
    uint64_t bar_p_empty[2];                       // CTA0: P buffer copied to registers
    uint64_t bar_s_full[kSBufs][2];                     // CTA0: [buffer][key half]
    float oscale[2][64];                           // [pair parity][row]: 1 / (l + sink term), what the epilogue multiplies O by
    uint64_t bar_os_full[2];                       // local: oscale of the pair written (2 arrivals)
    uint64_t bar_os_empty[2];                      // local: the epilogue warps have read it (4 arrivals)
    uint64_t bar_o_empty;                          // CTA0: epilogue has drained O (4 warps of each CTA)
    uint64_t bar_m_ready[kMaxGroups];                 // local: group g published the running max of its tile
    uint32_t tmem_base;
    int abort_word;
    DeviceFault* fault;                            // copy of the kernel parameter, for the out-of-line wait path
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
            if (w.split && p.o_accum == nullptr) {
                // a divided request in a launch without partials (decode without a combine pass needs a schedule of
                // whole requests): flag it and write what this part has straight to `out` rather than through a
                // null pointer
                if (atomicCAS(&p.fault->flag, 0, 1) == 0) p.fault->where = 71;
                w.split = 0;
            }
            return true;
        }
    }
};


// Position in the sequence of 128-key tiles that a CTA pair walks: work item after work item.
template <bool DECODE, int NT> struct TileCursor {
    WorkIter<DECODE> it;
    WorkItem w;
    int t, ntiles;
    bool live;
    __device__ TileCursor(const AttnParams& params) : it(params), t(0), ntiles(0) { live = fetch(); }
    __device__ bool fetch() {
        while (it.template next<NT>(w)) {
            ntiles = (w.blk_end - w.blk_begin + 1) / 2;
            if (ntiles > 0) {   // empty items are never produced by the scheduler; skipping keeps the roles in step
                t = 0;
                return true;
            }
        }
        return false;
    }
    __device__ void advance() {
        if (++t >= ntiles) live = fetch();
    }
};

// Key at position `j` (0..63) of 64-key block `blk` of a work item, in two steps so that callers can
// keep the index load and the loads that depend on it in flight for different tiles.
// Step 1: the raw index (-1 when the position does not exist).
template <bool DECODE>
__device__ __forceinline__ int key_index(const AttnParams& p, const WorkItem& w, int blk, int j) {
    if (blk >= w.blk_end) return -1;
    if constexpr (!DECODE) {
        const int pos = blk * 64 + j;
        return pos < p.topk ? __ldg(w.row + pos) : -1;
    } else {
        const bool extra = blk >= w.n_main_blocks;
        const int pos = (extra ? blk - w.n_main_blocks : blk) * 64 + j;
        return pos < (extra ? p.extra_topk : p.topk) ? __ldg((extra ? w.erow : w.row) + pos) : -1;
    }
}
// Ask for the index lines of the two 64-key blocks blk, blk + 1 into L2: lane 0..3 takes 128-byte line lane % 2 of
// block blk + lane / 2 (nothing where the block or the position does not exist).
template <bool DECODE>
__device__ __forceinline__ void prefetch_index_lines(const AttnParams& p, const WorkItem& w, int blk, int lane) {
    const int b = blk + (lane >> 1);
    if (b >= w.blk_end) return;
    if constexpr (!DECODE) {
        const int pos = b * 64 + (lane & 1) * 32;
        if (pos < p.topk) prefetch_l2(w.row + pos);
    } else {
        const bool extra = b >= w.n_main_blocks;
        const int pos = (extra ? b - w.n_main_blocks : b) * 64 + (lane & 1) * 32;
        if (pos < (extra ? p.extra_topk : p.topk)) prefetch_l2((extra ? w.erow : w.row) + pos);
    }
}
// Step 2: is the key attended, where are its 512 data bytes (nullptr = no row, the operand rows are
// zero-filled) and its 16-byte scale slot.
template <bool DECODE>
__device__ __forceinline__ const uint8_t* key_resolve(const AttnParams& p, const WorkItem& w, int blk, int j, int idx,
                                                      bool& valid, const uint8_t*& slot) {
    valid = false;
    slot = nullptr;
    if (blk >= w.blk_end) return nullptr;
    if constexpr (!DECODE) {
        const int pos = blk * 64 + j;
        if (idx < 0 || idx >= p.s_kv) return nullptr;
        valid = pos < w.len;
        slot = p.kv_scales + (long long)idx * 16;
        return p.kv + (long long)idx * kDim;
    } else {
        const bool extra = blk >= w.n_main_blocks;
        const int pos = (extra ? blk - w.n_main_blocks : blk) * 64 + j;
        // an index outside the pool (stale or corrupt) is treated like -1: not attended, nothing dereferenced
        // (one unsigned compare: a negative index is a huge unsigned one)
        valid = (unsigned)idx < (extra ? p.extra_pool_rows32 : p.pool_rows32) && pos < (extra ? w.elen : w.len);
        if (!valid) return nullptr;
        const unsigned psz = extra ? p.extra_page_size : p.page_size;
        const int sh = extra ? p.extra_page_shift : p.page_shift;   // pages are powers of two as a rule: no division then
        unsigned page, in_page;
        if (__builtin_expect(sh >= 0, 1)) {
            page = (unsigned)idx >> sh;
            in_page = (unsigned)idx & (psz - 1);
        } else {
            page = (unsigned)idx / psz;
            in_page = (unsigned)idx - page * psz;
        }
        const uint8_t* pg = (extra ? p.extra_kv : p.kv) + (long long)page * (extra ? p.extra_stride_block : p.stride_block);
        slot = pg + psz * kDim + in_page * 16;
        return pg + in_page * kDim;
    }
}
template <bool DECODE>
__device__ __forceinline__ const uint8_t* key_lookup(const AttnParams& p, const WorkItem& w, int blk, int j,
                                                     bool& valid, const uint8_t*& slot) {
    return key_resolve<DECODE>(p, w, blk, j, key_index<DECODE>(p, w, blk, j), valid, slot);
}


// Row coordinate of one key in the 2-D view {512 B, rows} of its KV store (-1 = no row: the copy engine fills
// zeros), from the key's raw index.
template <bool DECODE>
__device__ __forceinline__ int key_row(const AttnParams& p, const WorkItem& w, int blk, int j, int idx) {
    if (blk >= w.blk_end) return -1;
    if constexpr (!DECODE) {
        return (idx >= 0 && idx < p.s_kv) ? idx : -1;
    } else {
        const bool extra = blk >= w.n_main_blocks;
        const int pos = (extra ? blk - w.n_main_blocks : blk) * 64 + j;
        if ((unsigned)idx >= (extra ? p.extra_pool_rows32 : p.pool_rows32) || pos >= (extra ? w.elen : w.len)) return -1;
        // row = page * rows_per_block + slot in page = idx + page * (rows_per_block - page_size)
        const int sh = extra ? p.extra_page_shift : p.page_shift;
        const unsigned gap = extra ? p.extra_row_gap : p.row_gap;
        const unsigned page = __builtin_expect(sh >= 0, 1) ? (unsigned)idx >> sh
                                                           : (unsigned)idx / (unsigned)(extra ? p.extra_page_size : p.page_size);
        return (int)((unsigned)idx + page * gap);
    }
}
// The tensor map that the rows of 64-key block `blk` are gathered through.
template <bool DECODE>
__device__ __forceinline__ const void* key_map(const AttnParams& p, const TensorMaps& maps, const WorkItem& w, int blk) {
    if constexpr (!DECODE) return &maps.kv;
    // without an extra pool there is no second map: positions past the main list have no row anyway
    else return (blk >= w.n_main_blocks && p.extra_topk > 0) ? &maps.ekv : &maps.kv;
}

// packed fp32 pairs (one instruction for two lanes of data)
__device__ __forceinline__ float2 f2_fma(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)),
          "l"(reinterpret_cast<unsigned long long&>(c)));
    return d;
}
__device__ __forceinline__ float2 f2_mul(float2 a, float2 b) {
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return d;
}
__device__ __forceinline__ float2 f2_add(float2 a, float2 b) {
    float2 d;
    asm("add.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return d;
}

// 16-byte asynchronous copy global -> shared; `bytes` = 16 copies, 0 writes zeros.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
// 8-byte flavour (through L1; the 16-byte one is the only size that may bypass it)
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
// one arrival on `bar` once all cp.async issued so far by this thread have landed
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
template <int N> __device__ __forceinline__ void setmaxnreg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void setmaxnreg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// multiply the 256 O columns of this thread's tensor-memory lane by f (out of line: one copy)
__device__ __noinline__ void rescale_o(uint32_t lane_addr, float f) {
    // 64 columns per round: half as many exposed load latencies
#pragma unroll 1
    for (int c = 0; c < 256; c += 64) {
        uint32_t v[64];
        tmem_ld32(lane_addr + kColO + c, v);
        tmem_ld32(lane_addr + kColO + c + 32, v + 32);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 64; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
        tmem_st32(lane_addr + kColO + c, v);
        tmem_st32(lane_addr + kColO + c + 32, v + 32);
    }
    tmem_wait_st();
}
// one 32-byte store (a whole sector); the address must be 32-byte aligned
__device__ __forceinline__ void st_global_32B(void* dst, const unsigned long long (&u)[4]) {
    asm volatile("st.global.v4.b64 [%0], {%1, %2, %3, %4};" ::"l"(dst), "l"(u[0]), "l"(u[1]), "l"(u[2]), "l"(u[3]) : "memory");
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}


// Bounded waits, always called by whole, converged warps.  Every lane watches the barrier itself and takes
// the decision itself: all lanes of a warp execute the same barrier test in the same instruction and get the
// same answer, so the warp stays together.  (Two alternatives were measured: one elected lane that polls and
// broadcasts the outcome costs 35-50% end to end; a warp vote on every decision costs 5-9% at topk 4096.)
//   MXDSA_WAIT       suspending wait (producers, stager, epilogue)
//   MXDSA_WAIT_POLL  polling with a short back-off (softmax)
//   MXDSA_WAIT_TIGHT polling without back-off (MMA issuers, stager on "K landed")
#ifndef MXDSA_POLL_BACKOFF_NS
#define MXDSA_POLL_BACKOFF_NS 40
#endif
// The loops are written out at every site, as lean as they get (a counter, not a clock), and the
// only call -- raise_fault -- sits on the path that never comes back, so no register has to survive
// it: a call on the waiting path costs about 1 KB of save/restore code per site, and the kernel's
// instruction footprint is what limits it (the SM's instruction cache holds about 32 KB).
// Bounds: polling 2^24 tries (>= 0.2 s), suspending kWaitSlices slices of kWaitSliceNs.
#define MXDSA_WAIT_LIMITED_(mode, addr, parity, code, poll_log2, slices)                                              \
    do {                                                                                            \
        if (__builtin_expect(!mbar_try_wait((addr), (parity)), 0)) {                                \
            uint32_t spins__ = 0;                                                                   \
            while (true) {                                                                          \
                if ((mode) < 0) {                                                                   \
                    if (mbar_try_wait_suspend((addr), (parity), kWaitSliceNs, false)) break;        \
                    if (++spins__ > (uint32_t)(slices) || *(volatile int*)&sm.abort_word != 0) {    \
                        raise_fault(sm, (code));                                                    \
                        goto done;                                                                  \
                    }                                                                               \
                } else {                                                                            \
                    if ((mode) > 0) __nanosleep((mode) > 0 ? (mode) : 1);                           \
                    if (mbar_try_wait((addr), (parity))) break;                                     \
                    if ((++spins__ & 1023u) == 0 &&                                                 \
                        (spins__ >= (1u << (poll_log2)) || *(volatile int*)&sm.abort_word != 0)) {  \
                        raise_fault(sm, (code));                                                    \
                        goto done;                                                                  \
                    }                                                                               \
                }                                                                                   \
            }                                                                                       \
        }                                                                                           \
    } while (0)
#define MXDSA_WAIT_ADDR_(mode, addr, parity, code) MXDSA_WAIT_LIMITED_(mode, addr, parity, code, 24, kWaitSlices)
#define MXDSA_WAIT_POLL(bar, parity, code) MXDSA_WAIT_ADDR_(MXDSA_POLL_BACKOFF_NS, smem_u32(&(bar)), parity, code)
#define MXDSA_WAIT_TIGHT(bar, parity, code) MXDSA_WAIT_ADDR_(0, smem_u32(&(bar)), parity, code)
#define MXDSA_WAIT(bar, parity, code) MXDSA_WAIT_ADDR_(-1, smem_u32(&(bar)), parity, code)

// A wait was abandoned: mark both CTAs of the pair and the device fault record.
template <typename Plan> __device__ __noinline__ void raise_fault(Plan& sm, int code) {
    sm.abort_word = 1;
    // tell the peer CTA so that its roles stop waiting as well
    const uint32_t peer = map_to_cta(smem_u32(&sm.abort_word), cluster_cta_rank() ^ 1u);
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer), "r"(1) : "memory");
    if (atomicCAS(&sm.fault->flag, 0, 1) == 0) sm.fault->where = code;
}

template <bool DECODE, int NT, int G>
__global__ void __launch_bounds__(kBaseThreads + 128 * G, 1)
mxdsa_attn_kernel(const __grid_constant__ AttnParams p, const __grid_constant__ TensorMaps maps) {
    extern __shared__ uint8_t smem_raw[];
    // The plan starts at the first 1024-byte boundary.  The pointer is formed by adding an offset to
    // the shared array (not by rounding an integer), so the compiler still knows that every access
    // through it is a shared-memory access and emits 32-bit shared loads and stores.
    SmemPlan& sm = *reinterpret_cast<SmemPlan*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const uint32_t cta = cluster_cta_rank();

    // ------------------------------------------------------------------ set-up
    // decode: the combine grid that follows may be set up from now on (it waits for this grid's completion
    // before it reads the partials)
    if constexpr (DECODE) asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&sm.bar_q_landed), 1);
        mbar_init(smem_u32(&sm.bar_q_full), 2);
        mbar_init(smem_u32(&sm.bar_q_empty), 2);
        for (int i = 0; i < kKStages; ++i) {
            mbar_init(smem_u32(&sm.bar_k_landed[i]), 128 + 4);   // 128 copy completions + one plain arrival per producer warp
        }
        for (int i = 0; i < kVStages; ++i) {
            mbar_init(smem_u32(&sm.bar_v_full[i]), 8);
        }
        for (int i = 0; i < kScStages; ++i) {
            mbar_init(smem_u32(&sm.bar_qk_done[i]), 1);
            mbar_init(smem_u32(&sm.bar_pv_done[i]), 1);
            mbar_init(smem_u32(&sm.bar_sc_full[i]), 2);
            mbar_init(smem_u32(&sm.bar_tok_full[i]), 1);
            mbar_init(smem_u32(&sm.bar_tok_empty[i]), 4);
        }
        for (int i = 0; i < 2; ++i) mbar_init(smem_u32(&sm.bar_p_empty[i]), 8);
        for (int i = 0; i < kSBufs; ++i) {
            mbar_init(smem_u32(&sm.bar_s_full[i][0]), 8);
            mbar_init(smem_u32(&sm.bar_s_full[i][1]), 8);
            mbar_init(smem_u32(&sm.bar_pv_half[i]), 1);
        }
        mbar_init(smem_u32(&sm.bar_o_empty), 8);
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&sm.bar_os_full[i]), 2);
            mbar_init(smem_u32(&sm.bar_os_empty[i]), 4);
        }
        for (int i = 0; i < kMaxGroups; ++i) mbar_init(smem_u32(&sm.bar_m_ready[i]), 4);
        sm.abort_word = 0;
        sm.fault = p.fault;
        fence_mbar_init();
    }
    if (warp == 11 && lane == 0) prefetch_tensormap(&maps.q);
    __syncthreads();
    cluster_sync();
    if (warp == 10) {
        tmem_alloc<2>(smem_u32(&sm.tmem_base), kTmemCols);
        tmem_relinquish<2>();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    if (warp >= 12 && warp < 16) {
        // V dimension scales (B-operand scale columns of every PV): lanes 0-63 hold the dims of CTA 0's half
        // (w1), lanes 64-127 those of CTA 1's half (w2); column c = word c.  Written once, straight from
        // registers; the barriers below order it before the first MMA of either CTA.
        const uint32_t* wv = (warp & 3) < 2 ? p.w1 : p.w2;
        uint32_t v[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) v[c] = wv[c];
        tmem_st8(tmem + (uint32_t((warp & 3) * 32) << 16) + kColVs, v);
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    tc_fence_after();

    const uint64_t desc_k128 = smem_desc_base(16, 1024, 2);   // K-major, 128-byte swizzle
    const uint64_t desc_v = smem_desc_base(16384, 1024, 2);   // MN-major, 128-byte swizzle
    const uint64_t desc_sf = smem_desc_base(0, 128, 0);       // scale rows, 16 bytes each

    // ------------------------------------------------------------------ roles
    // Register budget.  The launch gives every thread kLaunchRegs (the most that 640 or 768 threads can have),
    // and that allocation -- not the SM's whole file -- is the pool setmaxnreg draws from: an increase beyond
    // what the other warps have released would block for ever, hence the static_assert, and the host refuses
    // to launch unless the compiled kernel really has kLaunchRegs registers.  The copy and control warps hand
    // most of theirs back so that the softmax warps (64 logits per thread in registers) work without spilling.
    // Each setmaxnreg is executed by the four warps of one aligned warp group with the same value.
    constexpr int kGroups = G;
    constexpr int kThreads = kBaseThreads + 128 * G;
    constexpr int kLaunchRegs = launch_regs(G);
    constexpr bool kRebalanceRegs = true;
    constexpr int kRegsCopy = G == 2 ? 64 : 48, kRegsGather = G == 2 ? 40 : 32, kRegsCtl = 64, kRegsEpi = G == 2 ? 56 : 48;
    constexpr int kRegsSoftmax = G == 2 ? 128 : 104;
    static_assert(4 * 32 * (kRegsCopy + kRegsGather + kRegsCtl + kRegsEpi) + 4 * G * 32 * kRegsSoftmax <= kThreads * kLaunchRegs,
                  "register budget must fit in the launch allocation");
    if (warp < 8) {
        if (warp < 4) {
            if constexpr (kRebalanceRegs) setmaxnreg_dec<kRegsCopy>();
            // ===================== K producers (warps 0-3): 16-byte cp.async =====================
            // Warp pw copies rows 64*cta + 16*pw + i (i < 16) of every tile, whole 512-byte rows, one row per
            // instruction: lane L writes byte chunk L of the row -> chunk tile L/8, 16-byte column (L%8) ^ (row%8).
            // It also gathers the 8 scale bytes of 32 keys of the tile (its own 16 and the matching 16 of the
            // peer CTA's half) into sm.k_sf: every CTA needs the scales of all 128 keys.
            // Raw indices are loaded one tile ahead and turned into addresses only when the tile is copied: a warp
            // issues in order, so an address computed at load time would hold the warp until the load is back.
            const int pw = warp;
            const int key = lane < 16 ? 64 * (int)cta + 16 * pw + lane : 64 * (1 - (int)cta) + 16 * pw + (lane - 16);
            TileCursor<DECODE, NT> ck(p);
            uint32_t kt = 0;
            int idx = ck.live ? key_index<DECODE>(p, ck.w, ck.w.blk_begin + 2 * ck.t + key / 64, key % 64) : -1;
            const uint32_t k_stage0 = smem_u32(sm.k[0]) + (lane / 8) * 8192;
            // Where the key's row and scale slot are is worked out as soon as the tile's index is back, before the
            // wait for a free stage: the wait then covers what is left of the index load's latency.
            const uint8_t* cur = nullptr;
            const uint8_t* slot = nullptr;
            uint32_t vbits = 0;
            auto resolve_tile = [&]() {
                bool valid;
                cur = key_resolve<DECODE>(p, ck.w, ck.w.blk_begin + 2 * ck.t + key / 64, key % 64, idx, valid, slot);
                vbits = __ballot_sync(0xffffffffu, valid);
            };
            if (ck.live) resolve_tile();
#pragma unroll 1
            while (ck.live) {
                const uint32_t s = kt % kKStages;
                if (kt >= (uint32_t)kKStages) {   // stage s was last used by tile kt-2: its QK must be done
                    const uint32_t g = kt - kKStages;
                    MXDSA_WAIT(sm.bar_qk_done[g % kScStages], (g / kScStages) & 1, 10);
                }
                // The index rows are read once, front to back, and never fit in L2 as a whole: four lanes of one
                // warp ask for the 512 bytes that a tile further on will need, so that the index loads of all three
                // roles that read them (these warps, the V producers, the stager) come back from L2, not from HBM.
                if constexpr (MXDSA_INDEX_AHEAD > 0) {
                    if (pw == 0 && cta == 0 && lane < 4 && ck.t + MXDSA_INDEX_AHEAD < ck.ntiles)
                        prefetch_index_lines<DECODE>(p, ck.w, ck.w.blk_begin + 2 * (ck.t + MXDSA_INDEX_AHEAD), lane);
                }
                // the next tile's indices: the loads run while this tile's rows are issued
                ck.advance();
                idx = ck.live ? key_index<DECODE>(p, ck.w, ck.w.blk_begin + 2 * ck.t + key / 64, key % 64) : -1;
                const uint32_t base = k_stage0 + s * 32768;
#pragma unroll 4
                for (int i = 0; i < 16; ++i) {
                    const uint8_t* src = reinterpret_cast<const uint8_t*>(
                        __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(cur), i));
                    const int r = 16 * pw + i;
                    cp_async16(base + r * 128 + (((lane & 7) ^ (r & 7)) << 4), src ? src + lane * 16 : p.kv, src ? 16u : 0u);
                }
                // the key's 8 scale bytes go straight into the row layout that tcgen05.cp wants: row (key/64)*32 +
                // key%32 holds {bytes0-3[k], bytes0-3[k+32], bytes4-7[k], bytes4-7[k+32]} of keys k and k+32
                {
                    const uint32_t dst = smem_u32(&sm.k_sf[s][((key >> 6) * 32 + (key & 31)) * 4 + ((key >> 5) & 1)]);
                    cp_async4(dst, slot ? slot : p.kv, slot ? 4u : 0u);
                    cp_async4(dst + 8, slot ? slot + 4 : p.kv, slot ? 4u : 0u);
                }
                cp_async_arrive(smem_u32(&sm.bar_k_landed[s]));
                if (lane == 0) {   // validity of the warp's 32 keys: a plain store, released by a plain arrival
                    sm.kvalid[s][4 * cta + pw] = (uint16_t)vbits;
                    sm.kvalid[s][4 * (1 - cta) + pw] = (uint16_t)(vbits >> 16);
                    mbar_arrive(smem_u32(&sm.bar_k_landed[s]));
                }
                ++kt;
                if (ck.live) resolve_tile();
            }
        } else {
            if constexpr (kRebalanceRegs) setmaxnreg_dec<kRegsGather>();
            // ===================== V producers (warps 4-7): TMA gather4 =====================
            // CTA c stages bytes 256c .. 256c+255 of all 128 keys of a tile as [chunk of 128 B][key][128 B].
            // Warp pw takes keys 32*pw .. 32*pw+31; its lanes 0-7 own four keys each and issue two gather4
            // copies (one per chunk) of four rows (measured: the copy engine takes requests fastest from a few
            // lanes of several warps -- 4 warps x 8 lanes reach 21 B/clk, one warp of 32 lanes 8 B/clk).  Rows
            // that do not exist (index -1, position beyond the list, row outside the store) get a coordinate
            // outside the tensor map, which the copy engine fills with zeros.  The bytes of both CTAs complete
            // on ONE barrier of CTA 0, where the PV issuer waits; nothing else needs to know that V has landed.
            const int pw = warp - 4;
            const int jl = 32 * pw + lane;               // the key whose row this lane works out
            const int j0 = 32 * pw + 4 * (lane & 7);     // first of the four keys this lane requests (lanes 0-7)
            TileCursor<DECODE, NT> cv(p);
            uint32_t vt = 0;
            const uint32_t v_full0 = map_to_cta(smem_u32(&sm.bar_v_full[0]), 0);
            const uint32_t v_dst0 = smem_u32(sm.v[0]) + j0 * 128;
            // Every lane turns ONE index into a row coordinate and the requesting lanes collect four of them: the
            // warp's instructions are issued between those of six other warps of its scheduler, and a chain of
            // address arithmetic four keys long per lane cost about 1000 cycles per tile.  The coordinates of a
            // tile are worked out right after the requests of the tile before it, ahead of the wait for a free
            // stage, and the index load they need is issued before those requests, which hold the warp long
            // enough for it to come back.
            int row = -1;
            const void* map = &maps.kv;
            auto locate = [&](int idx) {
                const int blk = cv.w.blk_begin + 2 * cv.t + jl / 64;   // the same block for the warp's 32 keys
                row = key_row<DECODE>(p, cv.w, blk, jl % 64, idx);
                map = key_map<DECODE>(p, maps, cv.w, blk);
            };
            bool live = cv.live;
            if (live) locate(key_index<DECODE>(p, cv.w, cv.w.blk_begin + 2 * cv.t + jl / 64, jl % 64));
#pragma unroll 1
            while (live) {
                const uint32_t s = vt % kVStages;
                if (vt >= (uint32_t)kVStages) {   // stage s was last used by tile vt-3: its PV must be done
                    const uint32_t g = vt - kVStages;
                    MXDSA_WAIT(sm.bar_pv_done[g % kScStages], (g / kScStages) & 1, 11);
                }
                const void* map_cur = map;
                int r[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) r[i] = __shfl_sync(0xffffffffu, row, 4 * (lane & 7) + i);
                cv.advance();
                live = cv.live;
                int idx = -1;
                if (live) idx = key_index<DECODE>(p, cv.w, cv.w.blk_begin + 2 * cv.t + jl / 64, jl % 64);
                if (lane == 0) mbar_expect_tx_cluster(v_full0 + s * 8, 2 * 32 * 128);
                __syncwarp();
                if (lane < 8) {
                    const uint32_t dst = v_dst0 + s * 32768;
                    tma_gather4_pair(dst, map_cur, 256 * (int)cta, r[0], r[1], r[2], r[3], v_full0 + s * 8, MXDSA_V_HINT);
                    tma_gather4_pair(dst + 16384, map_cur, 256 * (int)cta + 128, r[0], r[1], r[2], r[3], v_full0 + s * 8, MXDSA_V_HINT);
                }
                __syncwarp();
                ++vt;
                if (live) locate(idx);
            }
        }
    } else if (warp < 12) {
    if constexpr (kRebalanceRegs) setmaxnreg_dec<kRegsCtl>();
    if (warp == 8 || warp == 9) {
        if (cta == 0) {
            // ===================== QK issuers (CTA 0): warp 8 even tiles, warp 9 odd tiles ==========
            // The whole warp walks the schedule and waits; one elected lane issues.  Keeping the warp
            // converged lets the descriptor arithmetic run on the uniform datapath, and the 16 steps
            // are unrolled so that every operand is "base + constant": issued this way the tensor
            // core, not the issuing thread, sets the pace (measured: 1040 cycles for a tile's 24
            // instructions against 2670 from a single thread in a rolled loop).
            const uint32_t e = __shfl_sync(0xffffffffu, warp - 8, 0);   // tile parity = P buffer = scale column set
            WorkIter<DECODE> it(p);
            WorkItem w;
            uint32_t gt = 0, gw = 0;
            const uint32_t qk_done_peer = map_to_cta(smem_u32(&sm.bar_qk_done[0]), 1);
            const uint32_t q_empty_peer = map_to_cta(smem_u32(&sm.bar_q_empty), 1);
            const uint64_t a_base = smem_desc(desc_k128, smem_u32(sm.q));
            const uint32_t d_p = tmem + kColP + e * 64, sfa0 = tmem + kColQs + 4 * e, sfb0 = tmem + kColKs + 4 * e;
#pragma unroll 1
            while (it.template next<NT>(w)) {
                const int ntiles = (w.blk_end - w.blk_begin + 1) / 2;
                if (ntiles <= 0) continue;  // never produced by the scheduler; keeps the roles in step
                // Both issuers observe every phase of q_full, also for a pair in which they own no
                // tile: a parity wait that skipped a phase would be satisfied by the stale one.
                MXDSA_WAIT_TIGHT(sm.bar_q_full, gw & 1, 20);
                bool mine = false;
#pragma unroll 1
                for (int t = 0; t < ntiles; ++t, ++gt) {
                    if ((gt & 1) != e) continue;
                    const uint32_t s = gt % kKStages;
                    const uint32_t sc = gt % kScStages, sph = (gt / kScStages) & 1;
                    const uint32_t bph = (gt >> 1) & 1;
                    MXDSA_WAIT_TIGHT(sm.bar_sc_full[sc], sph, 21);
                    MXDSA_WAIT_TIGHT(sm.bar_p_empty[e], bph ^ 1, 22);
                    // "scale rows ready" comes from the stagers of both CTAs, each of which has seen its CTA's K rows
                    // land and has fenced them towards the tensor core: nothing else to wait for
                    fence_proxy_async_smem();
                    tc_fence_after();
                    __syncwarp();
                    if (elect_one()) {
                        if (!mine)   // first own tile of this pair: the pair's Q scale rows
                            tmem_cp_sf_pair(sfa0, smem_desc(desc_sf, smem_u32(sm.q_sf)));
                        tmem_cp_sf_pair(sfb0, smem_desc(desc_sf, smem_u32(sm.k_sf[s])));
                        const uint64_t b_base = smem_desc(desc_k128, smem_u32(sm.k[s]));
#pragma unroll
                        for (int kk = 0; kk < 16; ++kk) {
                            // Q bytes (kk%8)*64 + (kk/8)*32 of the row meet K bytes 32*kk
                            const uint32_t a_off = ((kk & 7) >> 1) * 8192 + (kk & 1) * 64 + (kk >> 3) * 32;
                            const uint32_t b_off = (kk >> 2) * 8192 + (kk & 3) * 32;
                            mma_mxf8<2>(d_p, a_base + (a_off >> 4), b_base + (b_off >> 4),
                                        mx_idesc(128, 128, false, kk & 3, (kk >> 1) & 3), sfa0 + 2 * ((kk >> 2) & 1),
                                        sfb0 + 2 * (kk >> 3), kk != 0);
                        }
                        mma_commit<2>(smem_u32(&sm.bar_qk_done[sc]));
                        mma_commit<2>(qk_done_peer + sc * 8);
                    }
                    __syncwarp();
                    mine = true;
                }
                // Q may be overwritten once both issuers' QKs of this pair have finished
                if (elect_one()) {
                    if (mine) {
                        mma_commit<2>(smem_u32(&sm.bar_q_empty));
                        mma_commit<2>(q_empty_peer);
                    } else {
                        mbar_arrive(smem_u32(&sm.bar_q_empty));
                        mbar_arrive_cluster(q_empty_peer);
                    }
                }
                __syncwarp();
                ++gw;
            }
        }
    } else if (warp == 10) {
        if (cta == 0) {
            // ===================== PV issuer (CTA 0): converged warp, one elected lane issues ==========
            WorkIter<DECODE> it(p);
            WorkItem w;
            uint32_t gt = 0, gw = 0;
            const uint32_t pv_half_peer = map_to_cta(smem_u32(&sm.bar_pv_half[0]), 1);
            const uint32_t pv_done_peer = map_to_cta(smem_u32(&sm.bar_pv_done[0]), 1);
#pragma unroll 1
            while (it.template next<NT>(w)) {
                const int ntiles = (w.blk_end - w.blk_begin + 1) / 2;
                if (ntiles <= 0) continue;  // never produced by the scheduler; keeps the roles in step
                MXDSA_WAIT_TIGHT(sm.bar_o_empty, (gw & 1) ^ 1, 30);
                tc_fence_after();
#pragma unroll 1
                for (int t = 0; t < ntiles; ++t, ++gt) {
                    const uint32_t s = gt % kVStages, ph = (gt / kVStages) & 1;
                    const uint32_t b = gt % kSBufs, bph = (gt / kSBufs) & 1;   // S buffer and the phase of its barriers
                    const uint32_t sc = gt % kScStages;
                    MXDSA_WAIT_TIGHT(sm.bar_v_full[s], ph, 34);
                    const uint64_t a_base = smem_desc(desc_k128, smem_u32(sm.s[b]));
                    const uint64_t b_base = smem_desc(desc_v, smem_u32(sm.v[s]));
                    const uint32_t sfa = tmem + kColSs + 4 * b;
                    const bool fresh = t == 0;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (NT == 128 && h == 0) continue;   // 128-key tiles: one wait, after both halves are in
                        MXDSA_WAIT_TIGHT(sm.bar_s_full[b][h], bph, 32 + h);
                        tc_fence_after();
                        __syncwarp();
                        if (elect_one()) {
                            tmem_cp_sf_pair(sfa, smem_desc(desc_sf, smem_u32(sm.s_sf[b])));
#pragma unroll
                            for (int i = (NT == 64 ? 4 * h : 0); i < 4 * h + 4; ++i) {
                                const int ks = i >> 1, n = i & 1;   // key step (32 keys), dim chunk (128 dims of each CTA)
                                mma_mxf8<2>(tmem + kColO + n * 128, a_base + ((ks * 32) >> 4),
                                            b_base + ((n * 16384 + ks * 4096) >> 4),
                                            mx_idesc(128, 256, true, ks, NT == 64 ? (ks & 1) : ks), sfa,
                                            tmem + kColVs + 4 * n, !(fresh && ks == 0));
                            }
                            if (NT == 64 && h == 0) {
                                mma_commit<2>(smem_u32(&sm.bar_pv_half[b]));
                                mma_commit<2>(pv_half_peer + b * 8);
                            } else {
                                mma_commit<2>(smem_u32(&sm.bar_pv_done[sc]));
                                mma_commit<2>(pv_done_peer + sc * 8);
                            }
                        }
                        __syncwarp();
                    }
                }
                ++gw;
            }
        }
    } else if (warp == 11) {
        // ===================== operand stager =====================
        WorkIter<DECODE> it(p);
        WorkItem w;
        uint32_t gt = 0, gw = 0;
        const uint32_t q_full0 = map_to_cta(smem_u32(&sm.bar_q_full), 0);
        const uint32_t sc_full0 = map_to_cta(smem_u32(&sm.bar_sc_full[0]), 0);
#pragma unroll 1
        while (it.template next<NT>(w)) {
            const int ntiles = (w.blk_end - w.blk_begin + 1) / 2;
            if (ntiles <= 0) continue;  // never produced by the scheduler; keeps the roles in step
            // ---- Q tile and Q scale rows of this CTA's token
            const int tok = min(2 * w.pair + (int)cta, p.s_q - 1);
            if (lane == 0) {   // ask for the NEXT work item's Q tile to be brought into L2 while this one is worked on
                WorkIter<DECODE> peek = it;
                WorkItem wn;
                if (peek.template next<NT>(wn)) {
                    const int tokn = min(2 * wn.pair + (int)cta, p.s_q - 1);
                    asm volatile("cp.async.bulk.prefetch.tensor.5d.L2.global.tile [%0, {%1, %2, %3, %4, %5}];" ::"l"(&maps.q),
                                 "r"(0), "r"(0), "r"(0), "r"(tokn), "r"(wn.req)
                                 : "memory");
                }
            }
            __syncwarp();
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
            // ---- per tile: K scale rows, key token scales, validity.  Everything arrives in shared memory with the
            // K rows (the producers gather the scale slots and vote the validity bits), so no global load sits
            // between "K landed" and "QK may start".  lane L looks after keys L, L+32 (block 0) and L+64, L+96.
#pragma unroll 1
            for (int t = 0; t < ntiles; ++t) {
                const uint32_t sc = gt % kScStages, sph = (gt / kScStages) & 1;
                const uint32_t ks = gt % kKStages;
                MXDSA_WAIT_TIGHT(sm.bar_k_landed[ks], (gt / kKStages) & 1, 44);
                // The K rows, the scale rows and the validity bits of this CTA have landed.  Publish at once (the
                // fence makes what cp.async wrote visible to the tensor core), then derive what the softmax reads.
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(sc_full0 + sc * 8);
                // token scale = 2^(scale byte 0 - 127); keys L, L+32 sit in words 0, 1 of row L, keys L+64, L+96 in row 32+L
                const uint2 lo = *reinterpret_cast<const uint2*>(&sm.k_sf[ks][lane * 4]);
                const uint2 hi = *reinterpret_cast<const uint2*>(&sm.k_sf[ks][(32 + lane) * 4]);
                const uint32_t vword = reinterpret_cast<const uint32_t*>(sm.kvalid[ks])[lane & 3];
                // ring of 4: a stage is free once the softmax of tile gt-4 is through
                if (gt >= kScStages) MXDSA_WAIT(sm.bar_tok_empty[sc], sph ^ 1, 43);
                sm.tok_scale[sc][lane] = __uint_as_float((lo.x & 0xffu) << 23);
                sm.tok_scale[sc][32 + lane] = __uint_as_float((lo.y & 0xffu) << 23);
                sm.tok_scale[sc][64 + lane] = __uint_as_float((hi.x & 0xffu) << 23);
                sm.tok_scale[sc][96 + lane] = __uint_as_float((hi.y & 0xffu) << 23);
                if (lane < 4) sm.valid[sc][lane] = vword;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sm.bar_tok_full[sc]));
                if (t == 0) {   // the pair's Q tile: its latency hides behind the first tile's staging
                    MXDSA_WAIT(sm.bar_q_landed, gw & 1, 41);
                    if (lane == 0) mbar_arrive_cluster(q_full0);
                }
                ++gt;
            }
            ++gw;
        }
    }
    } else if (warp < 12 + 4 * G) {
        if constexpr (kRebalanceRegs) setmaxnreg_inc<kRegsSoftmax>();
        // ===================== softmax + epilogue (warps 12 ..) =====================
        // Two groups of four warps take alternate tiles (group = tile parity = P buffer), so one
        // group's exp / quantise / store phase overlaps the other group's load / max phase.  Inside a
        // group a thread owns one row and one 64-key half of the tile (two UE8M0 scale groups of S).
        // The only serial link between consecutive tiles is the running maximum: after deciding m_t a
        // group publishes it (sm.m_pub) and the other group picks it up before deciding m_{t+1}.
        const int grp = (warp - 12) >> 2;
        const int prev_grp = (grp + kGroups - 1) % kGroups;
        const int q4 = warp & 3;                 // lane quadrant of tensor memory
        const int L = q4 * 32 + lane;            // tensor-memory lane
        const int row = L % 64;                  // head
        const int half = L / 64;                 // key half of a tile / dim half of O
        const uint32_t lane_addr = tmem + (uint32_t(q4 * 32) << 16);
        const uint32_t p_empty0 = map_to_cta(smem_u32(&sm.bar_p_empty[0]), 0);
        const uint32_t s_full0 = map_to_cta(smem_u32(&sm.bar_s_full[0][0]), 0);
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
        WorkIter<DECODE> it(p);
        WorkItem w;
        uint32_t gt = 0, gw = 0;
#pragma unroll 1
        while (it.template next<NT>(w)) {
            const int ntiles = (w.blk_end - w.blk_begin + 1) / 2;
            if (ntiles <= 0) continue;  // never produced by the scheduler; keeps the roles in step
            float m_own = -1e30f;   // running max after this group's latest tile of the pair
            float l = 0.f, real_m = -CUDART_INF_F;
#pragma unroll 1
            for (int t = 0; t < ntiles; ++t, ++gt) {
                if ((int)(gt % kGroups) != grp) continue;
                const uint32_t sc = gt % kScStages, sph = (gt / kScStages) & 1;
                const uint32_t pb = gt & 1;                              // P buffer
                const uint32_t b = gt % kSBufs, bph = (gt / kSBufs) & 1;   // S buffer and the phase of its barriers
                MXDSA_WAIT_POLL(sm.bar_tok_full[sc], sph, 50);
                const uint32_t v0 = sm.valid[sc][2 * half], v1 = sm.valid[sc][2 * half + 1];
                MXDSA_WAIT_POLL(sm.bar_qk_done[sc], sph, 51);
                tc_fence_after();
                float x[64];
                tmem_ld32(lane_addr + kColP + pb * 64, reinterpret_cast<uint32_t*>(x));
                tmem_ld32(lane_addr + kColP + pb * 64 + 32, reinterpret_cast<uint32_t*>(x + 32));
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(p_empty0 + pb * 8);
                if ((v0 & v1) != 0xffffffffu) {
#pragma unroll
                    for (int i = 0; i < 64; ++i) x[i] = (((i < 32 ? v0 : v1) >> (i & 31)) & 1u) ? x[i] : -CUDART_INF_F;
                }
                float mx8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = x[i];
#pragma unroll
                for (int i = 8; i < 64; i += 16) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) mx8[j] = fmax3(mx8[j], x[i + j], x[i + 8 + j < 64 ? i + 8 + j : i + j]);
                }
                const float own_max = fmaxf(fmax3(mx8[0], mx8[1], mx8[2]), fmaxf(fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]))) * p.scale_log2;
                float* xm = sm.xmax[grp][(gt / kGroups) & 1];
                xm[L] = own_max;
                named_bar_sync(1 + grp, 128);
                const float peer_max = xm[L ^ 64];
                // the running maximum handed over by the other group (value ignored on a pair's first
                // tile, but every phase of that barrier is observed)
                if (gt > 0) MXDSA_WAIT_POLL(sm.bar_m_ready[prev_grp], ((gt - 1) / kGroups) & 1, 58);
                const float m_prev = t == 0 ? -1e30f : sm.m_pub[prev_grp][row];
                const float sprev = (m_own == m_prev) ? 1.f : ex2_approx(m_own - m_prev);
                // numerical tiles: NT = 128 -> one per tensor-core tile; NT = 64 -> key half 0 then 1
                float m_used, scale0 = 1.f, scale1 = 1.f;
                bool grow0, grow1 = false;
                if constexpr (NT == 128) {
                    const float tmax = fmaxf(own_max, peer_max);
                    real_m = fmaxf(real_m, tmax);
                    grow0 = __any_sync(0xffffffffu, tmax - m_prev > 6.0f);
                    const float nm = grow0 ? fmaxf(m_prev, tmax) : m_prev;
                    scale0 = grow0 ? ex2_approx(m_prev - nm) : 1.f;
                    m_own = nm;
                    m_used = nm;
                } else {
                    const float t0 = half == 0 ? own_max : peer_max;
                    const float t1 = half == 0 ? peer_max : own_max;
                    real_m = fmaxf(real_m, fmaxf(t0, t1));
                    grow0 = __any_sync(0xffffffffu, t0 - m_prev > 6.0f);
                    const float m1 = grow0 ? fmaxf(m_prev, t0) : m_prev;
                    scale0 = grow0 ? ex2_approx(m_prev - m1) : 1.f;
                    grow1 = __any_sync(0xffffffffu, t1 - m1 > 6.0f);
                    const float m2 = grow1 ? fmaxf(m1, t1) : m1;
                    scale1 = grow1 ? ex2_approx(m1 - m2) : 1.f;
                    m_used = half == 0 ? m1 : m2;
                    m_own = m2;
                }
                sm.m_pub[grp][row] = m_own;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sm.bar_m_ready[grp]));
                // S buffer b is free once the PV of tile gt - kSBufs has finished (long ago, as a rule)
                if (gt >= (uint32_t)kSBufs) {
                    const uint32_t g = gt - kSBufs;
                    MXDSA_WAIT_POLL(sm.bar_pv_done[g % kScStages], (g / kScStages) & 1, 52);
                }
                // probabilities, key-scaled, re-quantised per 32 keys and stored
                const float2 negm2 = make_float2(-m_used, -m_used);
                const float4* tok4 = reinterpret_cast<const float4*>(&sm.tok_scale[sc][half * 64]);
                uint8_t* srow = sm.s[b];
                float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
                uint32_t e_bytes = 0;
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    uint32_t s8[8];
                    uint32_t e;
                    float am0 = 0.f, am1 = 0.f;
                    float* xg = x + 32 * g;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float4 tk = tok4[g * 8 + i / 4];
                        float2 a = f2_fma(make_float2(xg[i], xg[i + 1]), scale2, negm2);
                        float2 c = f2_fma(make_float2(xg[i + 2], xg[i + 3]), scale2, negm2);
                        a = make_float2(ex2_approx(a.x), ex2_approx(a.y));
                        c = make_float2(ex2_approx(c.x), ex2_approx(c.y));
                        sum2[0] = f2_add(sum2[0], a);
                        sum2[1] = f2_add(sum2[1], c);
                        a = f2_mul(a, make_float2(tk.x, tk.y));
                        c = f2_mul(c, make_float2(tk.z, tk.w));
                        am0 = fmax3(am0, a.x, a.y);
                        am1 = fmax3(am1, c.x, c.y);
                        xg[i] = a.x; xg[i + 1] = a.y; xg[i + 2] = c.x; xg[i + 3] = c.y;
                    }
                    const float am = fmaxf(am0, am1);
                    e = cvt_ue8m0_roundup(am > 0.f ? __fdividef(am, 448.0f) : 1.0f);
                    e = max(e, 61u);
                    const float mulf = __uint_as_float((254u - e) << 23);
                    const float2 mul2 = make_float2(mulf, mulf);
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float2 a = f2_mul(make_float2(xg[i], xg[i + 1]), mul2);
                        const float2 c = f2_mul(make_float2(xg[i + 2], xg[i + 3]), mul2);
                        s8[i / 4] = (uint32_t)cvt_e4m3x2(a.x, a.y) | ((uint32_t)cvt_e4m3x2(c.x, c.y) << 16);
                    }
                    e_bytes |= e << (8 * g);
                    *reinterpret_cast<uint4*>(srow + swz128(row, half * 64 + g * 32)) = make_uint4(s8[0], s8[1], s8[2], s8[3]);
                    *reinterpret_cast<uint4*>(srow + swz128(row, half * 64 + g * 32 + 16)) = make_uint4(s8[4], s8[5], s8[6], s8[7]);
                }
                // scale rows: row (row%32) and its copy at +32; word row/32; bytes 2*half, 2*half+1
                reinterpret_cast<uint16_t*>(&sm.s_sf[b][(row % 32) * 4 + row / 32])[half] = (uint16_t)e_bytes;
                reinterpret_cast<uint16_t*>(&sm.s_sf[b][(32 + row % 32) * 4 + row / 32])[half] = (uint16_t)e_bytes;
                const float2 s2 = f2_add(sum2[0], sum2[1]);
                const float sum = s2.x + s2.y;
                // l bookkeeping: every update of m rescales all partial sums of the row
                if constexpr (NT == 128) {
                    l = fmaf(l * sprev, scale0, sum);
                } else {
                    if (half == 0) l = fmaf(l * sprev, scale0, sum) * scale1;
                    else l = fmaf(l * sprev * scale0, scale1, sum);
                }
                // O rescale before the first key half is accumulated (this thread: its whole lane)
                if (grow0 && t > 0)
                {
                    MXDSA_WAIT_POLL(sm.bar_pv_done[(gt - 1) % kScStages], ((gt - 1) / kScStages) & 1, 53);
                    tc_fence_after();
                    rescale_o(lane_addr, scale0);
                    tc_fence_before();
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(s_full0 + (b * 2 + 0) * 8);
                if constexpr (NT == 64) {
                    if (grow1) {
                        MXDSA_WAIT_POLL(sm.bar_pv_half[b], bph, 54);
                        tc_fence_after();
                        rescale_o(lane_addr, scale1);
                        tc_fence_before();
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_cluster(s_full0 + (b * 2 + 1) * 8);
                    mbar_arrive(smem_u32(&sm.bar_tok_empty[sc]));
                }
            }
            // ---------------- end of the pair: final m, the four partial l of each row, drain O
            const uint32_t last = gt - 1;
            float m_fin = m_own;
            const int last_grp = (int)(last % kGroups);
            if (last_grp != grp) {
                MXDSA_WAIT_POLL(sm.bar_m_ready[last_grp], (last / kGroups) & 1, 59);
                m_fin = sm.m_pub[last_grp][row];
                l *= (m_own == m_fin) ? 1.f : ex2_approx(m_own - m_fin);
            }
            sm.xl[grp * 128 + L] = l;
            sm.xr[grp * 128 + L] = real_m;
            named_bar_sync(1 + kGroups, kGroups * 128);
            const float* xl = sm.xl;
            const float* xr = sm.xr;
            float l_tot = (xl[row] + xl[64 + row]) + (xl[128 + row] + xl[192 + row]);
            float real_all = fmaxf(fmaxf(xr[row], xr[64 + row]), fmaxf(xr[128 + row], xr[192 + row]));
            if constexpr (kGroups == 3) {
                l_tot += xl[256 + row] + xl[320 + row];
                real_all = fmaxf(real_all, fmaxf(xr[256 + row], xr[320 + row]));
            }
            named_bar_sync(1 + kGroups, kGroups * 128);   // everybody has read the exchange area before the next pair writes it
            // The first two warps of group 0 (one thread per row) turn the row sums into what the epilogue warps
            // need, write lse / max_logits, and every softmax warp goes straight on to the next pair: O is drained
            // by warps of its own while the next pair's tiles are worked on.
            if (grp == 0 && half == 0) {
                float m = m_fin;
                if (real_all == -CUDART_INF_F) {
                    l_tot = 0.f;
                    m = -CUDART_INF_F;
                }
                const int tok_idx = 2 * w.pair + (int)cta;
                const float sink = p.attn_sink ? __ldg(p.attn_sink + row) : -CUDART_INF_F;
                float oscale;
                if (!DECODE || !w.split) oscale = __fdividef(1.0f, l_tot + ex2_approx(fmaf(sink, CUDART_L2E_F, -m)));
                else oscale = __fdividef(1.0f, l_tot);
                if (l_tot == 0.f) oscale = 0.f;
                if (tok_idx < p.s_q) {
                    if (!DECODE || !w.split) {
                        float lse = fmaf(m, CUDART_LN2_F, CUDART_LN2_F * lg2_approx(l_tot));
                        if (l_tot == 0.f || lse == -CUDART_INF_F) lse = CUDART_INF_F;
                        const long long o = ((long long)w.req * p.s_q + tok_idx) * kHeads + row;
                        p.lse[o] = lse;
                        if (!DECODE) p.max_logits[o] = real_all * CUDART_LN2_F;
                    } else {
                        p.lse_accum[((long long)w.split_idx * p.s_q + tok_idx) * kHeads + row] = lg2_approx(l_tot) + m;
                    }
                }
                // oscale is handed over through a two-deep buffer: slot gw & 1 was last used by pair gw - 2
                if (gw >= 2) MXDSA_WAIT_POLL(sm.bar_os_empty[gw & 1], ((gw >> 1) & 1) ^ 1, 56);
                sm.oscale[gw & 1][row] = oscale;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sm.bar_os_full[gw & 1]));
            }
            ++gw;
        }
    } else {
        if constexpr (kRebalanceRegs) setmaxnreg_dec<kRegsEpi>();
        // ===================== epilogue (last four warps): O -> out =====================
        // A thread drains its tensor-memory lane: row L%64, the 256 dims of half L/64, 32 columns at a time,
        // multiplied by the row's oscale.  Unsplit work goes to `out` as bf16, split decode work to the fp32
        // partials.  The next pair's first PV waits for "O drained"; everything else of the next pair (gathers,
        // QK, softmax) runs meanwhile.
        const int q4 = warp & 3;
        const int L = q4 * 32 + lane;
        const int row = L % 64;
        const int half = L / 64;
        const uint32_t lane_addr = tmem + (uint32_t(q4 * 32) << 16);
        const uint32_t o_empty0 = map_to_cta(smem_u32(&sm.bar_o_empty), 0);
        // O is free for the next pair's first PV as soon as this warp has READ its last columns; the stores of
        // those columns (which may have to wait for a staging tile) follow after the release.
        auto release_o = [&]() {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(o_empty0);
        };
        WorkIter<DECODE> it(p);
        WorkItem w;
        uint32_t gt = 0, gw = 0;
        uint32_t round = 0;   // output rounds of this warp so far (staging tile = round % kOutTiles)
#pragma unroll 1
        while (it.template next<NT>(w)) {
            const int ntiles = (w.blk_end - w.blk_begin + 1) / 2;
            if (ntiles <= 0) continue;  // never produced by the scheduler; keeps the roles in step
            gt += ntiles;
            const uint32_t last = gt - 1;
            MXDSA_WAIT(sm.bar_os_full[gw & 1], (gw >> 1) & 1, 60);
            const float oscale = sm.oscale[gw & 1][row];
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.bar_os_empty[gw & 1]));
            MXDSA_WAIT(sm.bar_pv_done[last % kScStages], (last / kScStages) & 1, 55);
            tc_fence_after();
            const int tok_idx = 2 * w.pair + (int)cta;
            const bool store = tok_idx < p.s_q;
            if (!DECODE || !w.split) {
#if MXDSA_TMA_EPILOGUE
                // 32 columns at a time: one load becomes 32 rows x 64 bytes of the warp's staging area (16-byte
                // chunk c of row r sits at chunk c ^ ((r / 2) % 4), the 64-byte swizzle that the tensor map undoes
                // and that keeps the eight lanes of a store phase on different banks), then one tiled store.  The
                // area holds kOutTiles such tiles, so that the copy engine reads some while the warp fills another: an
                // SM writes about 32 bytes per clock to global memory at best, and only with stores kept in flight
                // (measured alone: 64 KB in 2470 cycles this way, 3330 with one tile, 3890 with 32-byte stores
                // from the lanes).
                const uint32_t stage0 = smem_u32(sm.o_stage[q4]);
                const int out_row0 = (w.req * p.s_q + tok_idx) * kHeads + (q4 & 1) * 32;
#pragma unroll 1
                for (int c = 0; c < 256; c += 32) {
                    float o[32];
                    tmem_ld32(lane_addr + kColO + c, reinterpret_cast<uint32_t*>(o));
                    tmem_wait_ld();
                    if (c == 256 - 32) release_o();   // the last columns are in registers: the next pair's PV may go
                    const uint32_t tile = stage0 + (round % kOutTiles) * 2048;   // tiles rotate across pairs too
                    ++round;
                    if (lane == 0) tma_store_wait_read<kOutTiles - 1>();   // the tile written kOutTiles rounds ago has been read
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint32_t u[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const __nv_bfloat162 v = __floats2bfloat162_rn(o[i + 2 * j] * oscale, o[i + 2 * j + 1] * oscale);
                            u[j] = *reinterpret_cast<const uint32_t*>(&v);
                        }
                        st_shared_16B(tile + lane * 64 + (((i >> 3) ^ ((lane >> 1) & 3)) << 4), u[0], u[1], u[2], u[3]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {   // a group per round, empty when nothing is stored, keeps "kOutTiles - 1 pending" exact
                        if (store) tma_store_2d(&maps.out, tile, half * 256 + c, out_row0);
                        tma_store_commit();
                    }
                }
#else
                __nv_bfloat16* dst = p.out + (((long long)w.req * p.s_q + tok_idx) * kHeads + row) * kDim + half * 256;
#pragma unroll 1
                for (int c = 0; c < 256; c += 32) {
                    float o[32];
                    tmem_ld32(lane_addr + kColO + c, reinterpret_cast<uint32_t*>(o));
                    tmem_wait_ld();
                    if (c == 256 - 32) release_o();   // the last columns are in registers: the next pair's PV may go
                    if (store) {
                        // 32 columns -> 64 bytes of bf16: two 32-byte stores per lane (whole sectors; sixteen-byte
                        // stores from 32 lanes to 32 rows touch every sector twice and took twice as long)
#pragma unroll
                        for (int i = 0; i < 32; i += 16) {
                            unsigned long long u[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const __nv_bfloat162 lo = __floats2bfloat162_rn(o[i + 4 * j] * oscale, o[i + 4 * j + 1] * oscale);
                                const __nv_bfloat162 hi = __floats2bfloat162_rn(o[i + 4 * j + 2] * oscale, o[i + 4 * j + 3] * oscale);
                                u[j] = (unsigned long long)(*reinterpret_cast<const uint32_t*>(&lo)) |
                                       ((unsigned long long)(*reinterpret_cast<const uint32_t*>(&hi)) << 32);
                            }
                            st_global_32B(dst + c + i, u);
                        }
                    }
                }
#endif
            } else {
                float* dst = p.o_accum + (((long long)w.split_idx * p.s_q + tok_idx) * kHeads + row) * kDim + half * 256;
#pragma unroll 1
                for (int c = 0; c < 256; c += 32) {
                    float o[32];
                    tmem_ld32(lane_addr + kColO + c, reinterpret_cast<uint32_t*>(o));
                    tmem_wait_ld();
                    if (c == 256 - 32) release_o();   // the last columns are in registers: the next pair's PV may go
                    if (store) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            unsigned long long u[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                u[j] = (unsigned long long)__float_as_uint(o[i + 2 * j] * oscale) |
                                       ((unsigned long long)__float_as_uint(o[i + 2 * j + 1] * oscale) << 32);
                            st_global_32B(dst + c + i, u);
                        }
                    }
                }
            }
            ++gw;
        }
    }

done:
    // ------------------------------------------------------------------ tear-down
#if MXDSA_TMA_EPILOGUE
    // stores still reading this CTA's shared memory must have done so before the CTA may end
    if (warp >= 12 + 4 * G && lane == 0) tma_store_wait_read<0>();
#endif
    // After a fault, softmax threads leave at different points; one extra arrival per leaving thread
    // completes the exchange barrier for those still parked on it (they fail their next wait and
    // follow).  In a normal exit the arrivals are harmless: nobody waits on that barrier any more.
    if (warp >= 12 && warp < 12 + 4 * G) {
        named_bar_arrive(1 + ((warp - 12) >> 2), 128);
        named_bar_arrive(1 + kGroups, kGroups * 128);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 10) tmem_dealloc<2>(tmem, kTmemCols);
}

// ----------------------------------------------------------------------------------------------
// Self-test of the bounded waits.  A CTA pair of two warps waits on a barrier that nobody ever arrives on --
// warp 0 with the polling loop, warp 1 with the suspending loop, the very loops of the attention kernel with
// their limits turned down to about a millisecond -- gives up, raises the device fault record and leaves
// through a normal tear-down.  Nothing faults and nothing hangs: it exists so that the give-up path, which in
// the attention kernel only runs when something is already wrong, is executed by a test.
// ----------------------------------------------------------------------------------------------
struct WaitSelftestPlan {
    uint64_t bar_never;
    int abort_word;
    DeviceFault* fault;
};
__global__ void __launch_bounds__(64, 1) mxdsa_wait_selftest_kernel(DeviceFault* fault, int* reached_teardown) {
    __shared__ WaitSelftestPlan sm;
    const int warp = threadIdx.x / 32;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&sm.bar_never), 1);
        sm.abort_word = 0;
        sm.fault = fault;
        fence_mbar_init();
    }
    __syncthreads();
    cluster_sync();
    if (warp == 0) {
        MXDSA_WAIT_LIMITED_(40, smem_u32(&sm.bar_never), 0, 90, 14, 8);   // 2^14 polls with back-off
    } else {
        MXDSA_WAIT_LIMITED_(-1, smem_u32(&sm.bar_never), 0, 91, 14, 8);   // 8 slices of kWaitSliceNs
    }
done:
    __syncthreads();
    cluster_sync();
    if (threadIdx.x == 0) atomicAdd(reached_teardown, 1);
}

// ----------------------------------------------------------------------------------------------
// Issue-only tensor-core rate probe: what the block-scaled E4M3 MMA of this library's shapes can do when
// nothing else is in the way.  A CTA pair keeps issuing cta_group::2 kind::mxf8f6f4 MMAs (M = 128, K = 32,
// N = `n` of 128 or 256) on operand bytes that sit in shared memory (copied once from `data`, so that the
// multipliers see real bit patterns, not zeros), accumulating into tensor memory; a commit and a bounded wait
// every 64 instructions keep the queue shallow.  Flops = pairs x iters x 64 x 2 x 128 x n x 32.
// The roofline fractions of the attention kernel are quoted against this number beside 2 x the bf16 GEMM rate.
// ----------------------------------------------------------------------------------------------
struct MmaRatePlan {
    uint64_t bar_done;
    uint32_t tmem_base;
    int abort_word;
    DeviceFault* fault;
};
__global__ void __launch_bounds__(128, 1) mxdsa_mma_rate_kernel(const uint4* data, int n, int iters, DeviceFault* fault) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 64 KB of operands, then the plan
    MmaRatePlan& sm = *reinterpret_cast<MmaRatePlan*>(tiles + 65536);
    const int warp = threadIdx.x / 32;
    const uint32_t cta = cluster_cta_rank();
    for (int i = threadIdx.x; i < 65536 / 16; i += blockDim.x) reinterpret_cast<uint4*>(tiles)[i] = __ldg(data + i);
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&sm.bar_done), 1);
        sm.abort_word = 0;
        sm.fault = fault;
        fence_mbar_init();
    }
    fence_proxy_async_smem();
    __syncthreads();
    cluster_sync();
    if (warp == 0) {
        tmem_alloc<2>(smem_u32(&sm.tmem_base), 512);
        tmem_relinquish<2>();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    if (warp == 1 && cta == 0) {
        const uint64_t desc_k = smem_desc_base(16, 1024, 2), desc_v = smem_desc_base(16384, 1024, 2);
        const uint64_t a_base = smem_desc(desc_k, smem_u32(tiles));               // [4 chunks][64 rows][128 B]
        const uint64_t b_k = smem_desc(desc_k, smem_u32(tiles + 32768));          // K-like operand (N = 128)
        const uint64_t b_v = smem_desc(desc_v, smem_u32(tiles + 32768));          // V-like operand (N = 256)
        const uint32_t peer_done = map_to_cta(smem_u32(&sm.bar_done), 1);
        constexpr int kBatch = 16;
#pragma unroll 1
        for (int it = 0; it < iters; ++it) {
            __syncwarp();
            if (elect_one()) {
#pragma unroll 1
              for (int rep = 0; rep < 4; ++rep) {      // four batches of 16 per commit: the wait is amortised over 64 instructions
                if (n == 128) {
#pragma unroll
                    for (int kk = 0; kk < kBatch; ++kk) {
                        const uint32_t a_off = ((kk & 7) >> 1) * 8192 + (kk & 1) * 64 + (kk >> 3) * 32;
                        const uint32_t b_off = (kk >> 2) * 8192 + (kk & 3) * 32;
                        mma_mxf8<2>(tmem + 256 + (kk & 1) * 64, a_base + (a_off >> 4), b_k + (b_off >> 4),
                                    mx_idesc(128, 128, false, kk & 3, (kk >> 1) & 3), tmem + 448, tmem + 456, true);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < kBatch; ++i) {
                        const int ks = (i >> 1) & 3, c = i & 1;
                        mma_mxf8<2>(tmem + c * 128, a_base + ((ks * 32) >> 4), b_v + ((c * 16384 + ks * 4096) >> 4),
                                    mx_idesc(128, 256, true, ks, ks), tmem + 448, tmem + 456, true);
                    }
                }
              }
                mma_commit<2>(smem_u32(&sm.bar_done));
                (void)peer_done;
            }
            __syncwarp();
            MXDSA_WAIT_LIMITED_(0, smem_u32(&sm.bar_done), it & 1, 92, 24, 8);
        }
    }
done:
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 0) tmem_dealloc<2>(tmem, 512);
}

}  // namespace mxdsa

/*
 * libmxdsa.so -- C ABI of the B200-native MXFP8 DeepSeek-Sparse-Attention library.
 *
 * Plain C: device pointers, sizes, strides, a CUDA stream handle.  No torch types.  Every entry
 * point returns an mxdsa_status (0 = success) instead of throwing, exiting or trapping, and never
 * synchronises the stream.  All pointers are DEVICE pointers unless stated otherwise.
 *
 * The reference project (dingirsu/MXDSA) has no extern "C" interface: its standalone library
 * exports C++ launchers that take parameter structs by reference.  Each entry point below names
 * the reference interface it stands in for (paths relative to the reference project).
 *
 * Packed operand format (reference tests/mxfp8_test_utils.py:30-104, csrc/attention/config.h:64-76)
 *   Q row     : 528 bytes per (token, head): 512 E4M3 bytes, then 8 UE8M0 scale bytes (one per
 *               pair of 32-wide chunks), then the same 8 bytes again.
 *   prefill KV: one flat buffer, s_kv*512 data bytes followed by s_kv 16-byte scale slots
 *               (8 UE8M0 bytes, one per 64 dims, stored twice).
 *   decode KV : pages; each page is page_size*512 data bytes followed by page_size scale slots;
 *               the page stride must be a multiple of 512 bytes.
 *   V         : the same E4M3 bytes as K, scaled by the token's first scale byte and by the
 *               per-dimension scale words w1 (dims 0-255) / w2 (dims 256-511): word j covers 32
 *               dims and holds one UE8M0 byte four times.
 */
#ifndef MXDSA_H_
#define MXDSA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MXDSA_HEADS 64        /* query heads per token                     */
#define MXDSA_DIM 512         /* latent K/V width                          */
#define MXDSA_ROW_BYTES 528   /* 512 data bytes + 16-byte scale slot       */
#define MXDSA_SCHED_META_INTS 8

typedef enum mxdsa_status {
    MXDSA_OK = 0,
    MXDSA_ERR_NULL = 1,          /* a required pointer is NULL                                  */
    MXDSA_ERR_SHAPE = 2,         /* a size rule is violated (see the entry point)               */
    MXDSA_ERR_ALIGN = 3,         /* a pointer or stride breaks an alignment rule                */
    MXDSA_ERR_DEVICE = 4,        /* not a compute-capability 10.x device                        */
    MXDSA_ERR_CUDA = 5,          /* a CUDA runtime/driver call failed; see mxdsa_last_cuda_error */
    MXDSA_ERR_WORKSPACE = 6,     /* workspace missing or too small                              */
    MXDSA_ERR_DEVICE_TIMEOUT = 7 /* a kernel gave up on a wait (reported by mxdsa_device_fault)  */
} mxdsa_status;

const char* mxdsa_status_string(int status);
/* cudaError_t of the most recent failing CUDA call made by this thread through the library. */
int mxdsa_last_cuda_error(void);
/* Synchronises `stream` and returns MXDSA_ERR_DEVICE_TIMEOUT if any kernel of this library on the
 * current device abandoned a bounded wait since the last call, else MXDSA_OK.  For tests and
 * debugging; the hot path never calls it. */
int mxdsa_device_fault(void* stream);

/* ------------------------------------------------------------------------------------------
 * Prefill.  Stands in for mxdsa::attention::run_dual_mxfp8_phase1_kernel<Prefill,512>
 * (reference csrc/attention/launch.h:10-19, prefill_kernel.cuh:1039-1110) driven by
 * MxFp8SparseAttnFwdParams (csrc/common/params.h:358-389), i.e. the device work behind
 * dual_mxfp8_head64_sparse_prefill_fwd (csrc/bindings/binding.cpp:12-113).
 *
 * Query tokens 2p and 2p+1 share index row p.  Key j of row p is attended when
 * 0 <= indices[p][j] < s_kv and j < topk_length[p] (topk when topk_length is NULL).
 * Rules: s_q > 0; topk > 0; q, kv 16-byte aligned; out 32-byte aligned; stride_q_token a multiple
 * of 16 bytes.  The reference operator additionally demands an even s_q and topk % 64 == 0
 * (binding.cpp:36-45); those two rules live in the operator layer above this call, so that the
 * same entry point also serves an odd s_q (ceil(s_q/2) index rows, the last one used by one
 * token) and any topk (positions >= topk are not attended; tiles of 128 keys from topk 512 on).
 * ------------------------------------------------------------------------------------------ */
typedef struct mxdsa_prefill_params {
    int32_t s_q, s_kv, topk;
    float sm_scale;
    const void* q;               /* u8 [s_q][64][528]                                   */
    int64_t stride_q_token;      /* bytes between query tokens (>= 64*528)              */
    const void* kv;              /* u8 flat: s_kv*512 data bytes, then s_kv*16 slots    */
    const int32_t* indices;      /* [ceil(s_q/2)][topk]                                 */
    int64_t stride_indices_pair; /* elements between index rows                         */
    const float* attn_sink;      /* [64] or NULL                                        */
    const int32_t* topk_length;  /* [ceil(s_q/2)] or NULL                               */
    uint32_t w1[8], w2[8];
    void* out;                   /* bf16 [s_q][64][512]                                 */
    float* max_logits;           /* [s_q][64]  max of sm_scale*logit, -inf if no key    */
    float* lse;                  /* [s_q][64]  natural-log sum-exp, +inf if no key      */
    void* stream;                /* cudaStream_t                                        */
} mxdsa_prefill_params;

int mxdsa_prefill_fwd(const mxdsa_prefill_params* p);

/* ------------------------------------------------------------------------------------------
 * Decode.  num_sm_parts = max(SM count / s_q, 1), as the reference binding computes it
 * (csrc/bindings/dual_mxfp8_sparse_decode.h:116).
 * ------------------------------------------------------------------------------------------ */
int mxdsa_num_sm_parts(int device, int s_q);

/* Split-KV schedule.  Stands in for mxdsa::split_kv::run_get_decoding_sched_meta_kernel
 * (reference csrc/split_kv/scheduler.cu:11-126, GetDecodeSchedMetaParams params.h:262-278).
 * Produces, bit for bit, the reference's DecodingSchedMeta records (params.h:12-18):
 *   sched_meta[i] = {begin_req, end_req (inclusive), begin_block, end_block (exclusive),
 *                    begin_split, first_req_is_split, last_req_is_split, 0}
 * for 64-key blocks over [main keys padded to 64 | extra keys], and num_splits[b+1] prefix sums. */
typedef struct mxdsa_sched_params {
    int32_t b, s_q, topk, extra_topk;   /* extra_topk = 0 when there is no extra cache */
    const int32_t* topk_length;         /* [b] or NULL */
    const int32_t* extra_topk_length;   /* [b] or NULL */
    int32_t num_sm_parts;
    int32_t* sched_meta;                /* out [num_sm_parts][8] */
    int32_t* num_splits;                /* out [b+1]             */
    void* stream;
} mxdsa_sched_params;

int mxdsa_decode_sched(const mxdsa_sched_params* p);

/* Bytes of scratch that mxdsa_decode_fwd needs: fp32 partial outputs and base-2 LSEs for
 * (b + num_sm_parts) splits, the shapes the reference allocates on every call
 * (dual_mxfp8_sparse_decode.h:203-206). */
size_t mxdsa_decode_workspace_bytes(int b, int s_q, int num_sm_parts);

/* Decode attention + split combine.  Stands in for
 * run_dual_mxfp8_phase1_kernel<DecodeWithSplitKV,512> (reference decode_kernel.cuh:989-1083,
 * SparseAttnDualMxfp8DecodeParams params.h:198-238) followed by run_flash_mla_combine_kernel<bf16>
 * (csrc/split_kv/combine.cu:415-448, CombineParams params.h:240-260).
 *
 * indices hold global slot ids (page * page_size + slot).  Queries 2p and 2p+1 of a request both
 * follow index row p of that request, as in the reference (decode_kernel.cuh:108, 554-558).
 * Key j is attended when indices[..][j] != -1 and j < topk_length[request].
 * Rules: topk > 0 and a multiple of 64; page strides multiples of 512 bytes; extra_* all present
 * or all absent (extra_topk_length optional); pointers 16-byte aligned, out and workspace 32-byte
 * aligned. */
typedef struct mxdsa_decode_params {
    int32_t b, s_q, topk, extra_topk;
    float sm_scale;
    const void* q;                    /* u8 [b][s_q][64][528] */
    int64_t stride_q_b, stride_q_s;   /* bytes                */
    const void* kv;                   /* page pool            */
    int32_t num_blocks, page_block_size;
    int64_t stride_kv_block;          /* bytes, multiple of 512 */
    const int32_t* indices;           /* [b][s_q][topk] */
    int64_t stride_indices_b, stride_indices_s; /* elements */
    const int32_t* topk_length;       /* [b] or NULL */
    const float* attn_sink;           /* [64] or NULL */
    const void* extra_kv;             /* or NULL */
    int32_t extra_num_blocks, extra_page_block_size;
    int64_t stride_extra_kv_block;
    const int32_t* extra_indices;     /* [b][s_q][extra_topk] or NULL */
    int64_t stride_extra_indices_b, stride_extra_indices_s;
    const int32_t* extra_topk_length; /* [b] or NULL */
    uint32_t w1[8], w2[8];
    void* out;                        /* bf16 [b][s_q][64][512] */
    float* lse;                       /* [b][s_q][64], natural log, without the sink term */
    const int32_t* sched_meta;        /* [num_sm_parts][8] from mxdsa_decode_sched */
    const int32_t* num_splits;        /* [b+1] */
    int32_t num_sm_parts;
    void* workspace;                  /* mxdsa_decode_workspace_bytes(...) bytes, 32-byte aligned */
    size_t workspace_bytes;
    void* stream;
} mxdsa_decode_params;

int mxdsa_decode_fwd(const mxdsa_decode_params* p);

/* The combine step alone.  Stands in for run_flash_mla_combine_kernel<bf16> (reference
 * csrc/split_kv/combine.cu:415-448, CombineParams params.h:240-260) for callers that sequence the
 * attention and the combine themselves; mxdsa_decode_fwd already runs it.  `workspace` is the buffer
 * an earlier mxdsa_decode_fwd with the same b, s_q, num_sm_parts, sched_meta and num_splits filled.
 * Only requests that the schedule splits over several parts are written (out and lse). */
typedef struct mxdsa_combine_params {
    int32_t b, s_q, num_sm_parts;
    const int32_t* sched_meta;        /* [num_sm_parts][8] */
    const int32_t* num_splits;        /* [b+1] */
    const void* workspace;            /* mxdsa_decode_workspace_bytes(...) bytes, 32-byte aligned */
    size_t workspace_bytes;
    const float* attn_sink;           /* [64] or NULL */
    void* out;                        /* bf16 [b][s_q][64][512], 32-byte aligned */
    float* lse;                       /* [b][s_q][64] */
    void* stream;
} mxdsa_combine_params;
int mxdsa_decode_combine(const mxdsa_combine_params* p);

/* ------------------------------------------------------------------------------------------
 * Decode without a combine pass (no counterpart in the reference, whose scheduler always divides
 * requests between parts: csrc/split_kv/scheduler.cu:61-112).
 *
 * mxdsa_decode_sched_whole writes records of the same layout as mxdsa_decode_sched in which every
 * request belongs to exactly one part (consecutive requests per part, balanced by their number of
 * 64-key blocks; num_splits[i] = i).  With such a schedule the attention kernel writes every
 * output itself: mxdsa_decode_fwd_nocombine launches it alone -- `workspace` is ignored, nothing
 * is merged afterwards.  The price is balance: a part's load is a whole number of requests.
 * Should the schedule handed to mxdsa_decode_fwd_nocombine divide a request after all, that
 * request's output is incomplete and the device fault record is raised (mxdsa_device_fault).
 * The records are also valid input for mxdsa_decode_fwd (its combine then finds nothing to do).
 * ------------------------------------------------------------------------------------------ */
int mxdsa_decode_sched_whole(const mxdsa_sched_params* p);
int mxdsa_decode_fwd_nocombine(const mxdsa_decode_params* p);

/* Self-test of the kernels' bounded waits.  (No counterpart in the reference, whose kernels trap or spin.)
 * Launches a two-CTA kernel that waits -- with the attention kernel's own wait loops, limits turned down to
 * about a millisecond -- on a barrier nobody arrives on, gives up, raises the device fault record and leaves
 * through its normal tear-down.  Nothing faults or hangs.  Afterwards mxdsa_device_fault(stream) returns
 * MXDSA_ERR_DEVICE_TIMEOUT once and clears the record.  mxdsa_selftest_teardowns() synchronises the stream
 * and returns how many self-test CTAs have reached their tear-down since the library was loaded. */
int mxdsa_selftest_bounded_wait(void* stream);
int mxdsa_selftest_teardowns(void* stream);

/* Issue-only tensor-core rate probe.  (No counterpart in the reference.)  Every CTA pair of the device issues
 * `iters` batches of 64 block-scaled E4M3 MMAs (tcgen05 kind::mxf8f6f4, cta_group::2) of shape M128 x N`n` x K32
 * (n = 128: the QK shape, n = 256: the PV shape) on 64 KB of operand bytes copied from `data`.  The caller times
 * the launch: flops = (SMs / 2) * iters * 64 * 2 * 128 * n * 32.  Used as the measured MXFP8 roof. */
int mxdsa_selftest_mma_rate(const void* data, int n, int iters, void* stream);

/* Decode without caller-provided scratch.  (No counterpart in the reference, whose binding
 * allocates its scratch with torch on every call.)
 *
 * For hosts that cannot give this library device memory at call time -- a process that forbids
 * cudaMalloc once it is serving, a plugin slot with no allocator handle, a caller already inside
 * code where the CUDA allocator must not be entered.  Same contract as mxdsa_decode_fwd, except
 * that p->workspace / p->workspace_bytes are ignored: the split partials live in an array that is
 * part of the library image, MXDSA_STATIC_SCRATCH_BYTES per GPU that loads the library, held
 * until the process exits.  The entry point calls no cudaMalloc, cudaFree or allocating routine.
 *
 *  - Returns MXDSA_ERR_WORKSPACE when mxdsa_decode_workspace_bytes(b, s_q, num_sm_parts) exceeds
 *    MXDSA_STATIC_SCRATCH_BYTES (the limit is (b + num_sm_parts) * s_q <= 255 partial slots).
 *  - The first call on a device looks the array's device address up; make that call before any
 *    CUDA stream capture begins on that device.
 *  - All calls on a device share the one array and it keeps the previous call's contents.  Nothing
 *    in it has to start at zero (every slot that is read is written earlier in the same call), but
 *    two calls that overlap on the GPU -- different streams, or a capture replayed while another
 *    call is in flight -- would overwrite each other's partials: serialise them. */
#define MXDSA_STATIC_SCRATCH_BYTES (32u << 20)
int mxdsa_decode_fwd_static(const mxdsa_decode_params* p);

/* ------------------------------------------------------------------------------------------
 * Quantise-and-pack: the step in front of the attention entry points.  Stands in for the reference's
 * Python packers (reference tests/mxfp8_test_utils.py: _quantize_groups :11-27, pack_dual_q64 :30-63,
 * pack_dual_prefill_kv64 :66-78, pack_dual_decode_kv_pages :81-104), which the reference runs as a
 * chain of torch kernels outside its timed path.  Byte-identical output for the same input values:
 * scale = 2^ceil(log2(max(amax/448, 2^-126))), code = E4M3(clamp(x/scale, +-448)), each scale byte
 * stored twice in the row's 16-byte slot.
 * ------------------------------------------------------------------------------------------ */
#define MXDSA_DTYPE_BF16 0
#define MXDSA_DTYPE_F32 1

/* Q rows.  One row = one (token, head): 512 values in, 528 bytes out.  Scale g is shared by dims
 * [32g,32g+32) and [256+32g,256+32g+32).  paired_storage = 0 keeps the reference packer's natural
 * byte order; 1 stores the bytes in the order [g][half][32] in which the attention kernel contracts
 * them with K's natural order.  Strides of 0 mean densely packed (512 elements / 528 bytes).
 * Rules: src, dst 16-byte aligned; row strides multiples of 16 bytes. */
typedef struct mxdsa_pack_q_params {
    int64_t rows;              /* tokens * 64 */
    const void* src;           /* [rows][512] bf16 or f32 */
    int32_t src_dtype;         /* MXDSA_DTYPE_* */
    int64_t src_stride_row;    /* elements */
    void* dst;                 /* u8 [rows][528] */
    int64_t dst_stride_row;    /* bytes */
    int32_t paired_storage;
    void* stream;
} mxdsa_pack_q_params;
int mxdsa_pack_q(const mxdsa_pack_q_params* p);

/* KV rows.  Scale g covers dims [64g,64g+64).  The output is a sequence of pages; a page holds
 * rows_per_page*512 data bytes followed by rows_per_page 16-byte slots.  The prefill buffer is the
 * one-page case (rows_per_page = rows = s_kv); decode pools use rows_per_page = page size and
 * dst_stride_page = bytes between pages (0 = rows_per_page*528).  rows must be a multiple of
 * rows_per_page. */
typedef struct mxdsa_pack_kv_params {
    int64_t rows;
    const void* src;           /* [rows][512] bf16 or f32 */
    int32_t src_dtype;
    int64_t src_stride_row;    /* elements */
    void* dst;
    int32_t rows_per_page;
    int64_t dst_stride_page;   /* bytes */
    void* stream;
} mxdsa_pack_kv_params;
int mxdsa_pack_kv(const mxdsa_pack_kv_params* p);
/* cudaError_t of the most recent failing launch of a pack kernel on this thread. */
int mxdsa_pack_last_cuda_error(void);

/* ------------------------------------------------------------------------------------------
 * Index selection: scores -> the int32 index rows (and valid lengths) that mxdsa_prefill_fwd and
 * mxdsa_decode_fwd consume.  The reference has no producer for `indices`; its callers define the
 * conventions this follows (reference tests/benchmark.py:119-147: one row per pair of query tokens,
 * -1 entries never attended, decode pools addressed by request * pool_len + slot; csrc/bindings/binding.cpp
 * :12-15 and csrc/bindings/dual_mxfp8_sparse_decode.h:13-20 for shapes and topk_length).
 *
 * Row r takes the min(topk, candidates) highest-scoring keys among j < lengths[r] (all s_kv when
 * lengths is NULL); a score that is NaN or -inf is no candidate; ties go to the smaller j.  With
 * group = 2 the score of key j is the larger of score rows 2r and 2r+1 (the two tokens of a pair).
 * The selected j (+ row_offset[r] when given) are written in ascending order, then -1 up to topk;
 * topk_length[r] = the number selected.  Exact and deterministic.
 * Rules: s_kv a multiple of 4; scores 16-byte aligned, score_stride a multiple of 4 elements;
 * strides of 0 mean densely packed.
 * ------------------------------------------------------------------------------------------ */
typedef struct mxdsa_topk_params {
    const float* scores;        /* f32 [rows*group][s_kv]                         */
    int64_t score_stride;       /* elements between score rows                    */
    const int32_t* lengths;     /* [rows] or NULL                                 */
    const int32_t* row_offset;  /* [rows] or NULL: added to every selected index  */
    int32_t* indices;           /* out [rows][topk]                               */
    int64_t index_stride;       /* elements between index rows                    */
    int32_t* topk_length;       /* out [rows] or NULL                             */
    int32_t rows, group, s_kv, topk;
    void* stream;
} mxdsa_topk_params;
int mxdsa_topk_select(const mxdsa_topk_params* p);
/* cudaError_t of the most recent failing launch of the selection kernel on this thread. */
int mxdsa_topk_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
#endif /* MXDSA_H_ */

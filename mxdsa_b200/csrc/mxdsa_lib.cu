// libmxdsa.so: C ABI (include/mxdsa.h) over the sm_100a kernels.
//
// Host side of the path: argument validation (the launcher-level rules of the reference,
// csrc/attention/prefill_kernel.cuh:1044-1058 and decode_kernel.cuh:993-1010), tensor-map
// construction, cluster launches on the caller's stream, the split-KV scheduler kernel and the
// split-combine kernel.  No allocation, no synchronisation, no exceptions.
#include <cstdio>
#include <cstring>
#include <mutex>

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include "../../include/mxdsa.h"
#include "attn_sm100.cuh"

namespace {

thread_local int tl_last_cuda_error = 0;

#define MX_CUDA(call)                                  \
    do {                                               \
        cudaError_t e__ = (call);                      \
        if (e__ != cudaSuccess) {                      \
            tl_last_cuda_error = (int)e__;             \
            return MXDSA_ERR_CUDA;                     \
        }                                              \
    } while (0)

__device__ mxdsa::DeviceFault g_fault = {0, 0};   // zero at load: the first call needs no memset (and so no implicit synchronisation)

__device__ int g_selftest_teardowns = 0;

struct DeviceInfo {
    bool ready = false;
    int major = 0, sm_count = 0;
    mxdsa::DeviceFault* fault = nullptr;
};
DeviceInfo g_dev[64];
std::mutex g_dev_mutex;
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

int device_info(DeviceInfo** out) {
    int dev = 0;
    MX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return MXDSA_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo& d = g_dev[dev];
    if (!d.ready) {
        MX_CUDA(cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev));
        MX_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        if (d.major == 10) {
            void* sym = nullptr;
            MX_CUDA(cudaGetSymbolAddress(&sym, g_fault));
            d.fault = static_cast<mxdsa::DeviceFault*>(sym);
        }
        if (g_encode == nullptr) {
            cudaDriverEntryPointQueryResult q;
            void* fn = nullptr;
            MX_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
            if (q != cudaDriverEntryPointSuccess || fn == nullptr) return MXDSA_ERR_CUDA;
            g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
        }
        d.ready = true;
    }
    *out = &d;
    return d.major == 10 ? MXDSA_OK : MXDSA_ERR_DEVICE;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }   // outputs: 32-byte stores

// 5-D map over packed Q: {128 bytes, 64 heads, 4 chunks, tokens, requests}; one box = the 512 data
// bytes of all 64 heads of one token, landing as [chunk][head][128 B].
int make_q_map(CUtensorMap* map, const void* base, uint64_t tokens, uint64_t reqs, uint64_t stride_tok,
               uint64_t stride_req) {
    cuuint64_t dims[5] = {128, 64, 4, tokens, reqs};
    cuuint64_t strides[4] = {528, 128, stride_tok, stride_req};
    cuuint32_t box[5] = {128, 64, 4, 1, 1};
    cuuint32_t es[5] = {1, 1, 1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, const_cast<void*>(base), dims, strides, box, es,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        tl_last_cuda_error = (int)r;
        return MXDSA_ERR_CUDA;
    }
    return MXDSA_OK;
}

// 2-D map over the data rows of a KV store viewed as rows of 512 bytes (prefill: the token rows; decode:
// the whole pool, whose pages start on multiples of 512 bytes, so that row = page * (stride / 512) + slot).
// One gather4 box = 4 rows x 128 bytes, landing as four 128-byte-swizzled rows.
int make_kv_map(CUtensorMap* map, const void* base, uint64_t rows) {
    cuuint64_t dims[2] = {512, rows};
    cuuint64_t strides[1] = {512};
    cuuint32_t box[2] = {128, 1};
    cuuint32_t es[2] = {1, 1};
#ifndef MXDSA_KV_PROMO
#define MXDSA_KV_PROMO CU_TENSOR_MAP_L2_PROMOTION_L2_256B
#endif
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, es,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          MXDSA_KV_PROMO, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        tl_last_cuda_error = (int)r;
        return MXDSA_ERR_CUDA;
    }
    return MXDSA_OK;
}

// 2-D map over the bf16 output viewed as {512 columns, tokens x 64 heads}: the epilogue stores boxes of
// 32 columns x 32 rows out of 64-byte-swizzled staging tiles.
int make_out_map(CUtensorMap* map, void* base, uint64_t tokens) {
    cuuint64_t dims[2] = {MXDSA_DIM, tokens * MXDSA_HEADS};
    cuuint64_t strides[1] = {MXDSA_DIM * 2};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t es[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, es,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        tl_last_cuda_error = (int)r;
        return MXDSA_ERR_CUDA;
    }
    return MXDSA_OK;
}

constexpr size_t kSmemBytes = sizeof(mxdsa::SmemPlan) + 1024;

#ifndef MXDSA_COMBINE_PDL
#define MXDSA_COMBINE_PDL 1
#endif
#ifndef MXDSA_GROUPS_PREFILL
#define MXDSA_GROUPS_PREFILL 3
#endif
#ifndef MXDSA_GROUPS_DECODE
#define MXDSA_GROUPS_DECODE 3
#endif

// `groups` = softmax groups of the instantiation (the template's G): it fixes the block size and the register
// allocation that the kernel's setmaxnreg budget assumes.
template <typename K>
int launch_pairs(K kernel, int groups, dim3 grid, cudaStream_t stream, const mxdsa::AttnParams& ap,
                 const mxdsa::TensorMaps& maps) {
    static_assert(kSmemBytes <= 227 * 1024, "shared-memory plan exceeds the 227 KB per-CTA limit");
    // The kernel re-balances registers between its roles against a pool of launch_regs(groups) per thread.
    // If this build of the kernel was given a different number (another toolkit or flag set), an increase
    // beyond the pool would block in hardware for ever: refuse to launch instead.
    cudaFuncAttributes fa;
    MX_CUDA(cudaFuncGetAttributes(&fa, kernel));
    if (fa.numRegs != mxdsa::launch_regs(groups)) return MXDSA_ERR_DEVICE;
    MX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(mxdsa::kBaseThreads + 128 * groups);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim = {2, 1, 1};
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    MX_CUDA(cudaLaunchKernelEx(&cfg, kernel, ap, maps));
    return MXDSA_OK;
}

// ------------------------------------------------------------------------------------------
// Split-KV scheduler: greedy partition of the requests' 64-key blocks over num_sm_parts parts.
// cost(request) = blocks + 5; a part's budget is ceil(total cost / parts) + 5; a part takes whole
// requests while they fit, then as many blocks of the next one as budget - 5 allows.
// Same records as the reference's scheduler kernel (csrc/split_kv/scheduler.cu:11-118), including
// what it writes for parts that receive no work (it reads one element past its per-request
// arrays there: begin_block = last block of request 0, end fields of request b-1).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32) mxdsa_sched_kernel(int b, int topk, int extra_topk, const int* topk_length,
                                                        const int* extra_topk_length, int parts, int* meta,
                                                        int* num_splits) {
    extern __shared__ int nblk[];  // [b] blocks per request, then [b+1] split prefix sums
    int* splits = nblk + b;
    int cost = 0;
    for (int i = threadIdx.x; i < b; i += 32) {
        int len = topk_length ? topk_length[i] : topk;
        len = len == 0 ? 1 : len;
        if (extra_topk) len = (len + 63) / 64 * 64 + (extra_topk_length ? extra_topk_length[i] : extra_topk);
        const int n = (max(len - 1, 0)) / 64 + 1;
        nblk[i] = n;
        cost += n + 5;
    }
    for (int o = 16; o; o >>= 1) cost += __shfl_xor_sync(0xffffffffu, cost, o);
    __syncwarp();
    if (threadIdx.x == 0) {
        const int budget = (cost + parts - 1) / parts + 5;
        int req = 0, blk = 0, nsplit = 0, cum = 0;
        splits[0] = 0;
        for (int i = 0; i < parts; ++i) {
            int rec[8];
            rec[0] = req;
            rec[2] = req < b ? blk : blk + nblk[0] - 1;
            rec[4] = nsplit;
            int first = blk != 0;
            int left = budget;
            while (req < b) {
                const int rest = nblk[req] - blk;
                if (left >= rest + 5) {
                    cum += nsplit + 1;
                    splits[req + 1] = cum;
                    left -= rest + 5;
                    ++req;
                    blk = 0;
                    nsplit = 0;
                } else {
                    if (left - 5 > 0) {
                        blk += left - 5;
                        ++nsplit;
                        left = 0;
                    }
                    break;
                }
            }
            rec[1] = blk > 0 ? req : req - 1;
            rec[3] = blk > 0 ? blk : nblk[req - 1];
            int last = rec[3] != nblk[rec[1]];
            if (rec[0] == rec[1]) first = last = (first || last);
            rec[5] = first;
            rec[6] = last;
            rec[7] = 0;
            for (int k = 0; k < 8; ++k) meta[8 * i + k] = rec[k];
        }
    }
    __syncwarp();
    for (int i = threadIdx.x; i <= b; i += 32) num_splits[i] = splits[i];
}

// ------------------------------------------------------------------------------------------
// Whole-request scheduler: the same records, but no request is divided between parts, so that the attention
// kernel writes every output itself and no combine pass is needed.  Part i takes the consecutive requests whose
// midpoint (in 64-key blocks, prefix-summed) falls into the i-th of `parts` equal shares of the total; a part
// without requests gets begin_req > end_req.  num_splits[i] = i.  The reference has no such schedule
// (its scheduler, csrc/split_kv/scheduler.cu:61-112, always fills parts to an equal budget and splits).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32) mxdsa_sched_whole_kernel(int b, int topk, int extra_topk, const int* topk_length,
                                                              const int* extra_topk_length, int parts, int* meta,
                                                              int* num_splits) {
    extern __shared__ int nblk[];  // [b] blocks per request
    int total = 0;
    for (int i = threadIdx.x; i < b; i += 32) {
        int len = topk_length ? topk_length[i] : topk;
        len = len == 0 ? 1 : len;
        if (extra_topk) len = (len + 63) / 64 * 64 + (extra_topk_length ? extra_topk_length[i] : extra_topk);
        const int n = (max(len - 1, 0)) / 64 + 1;
        nblk[i] = n;
        total += n;
    }
    for (int o = 16; o; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    __syncwarp();
    if (threadIdx.x == 0) {
        int req = 0;
        long long before = 0;   // blocks of the requests already given away
        for (int i = 0; i < parts; ++i) {
            const long long limit = (long long)total * (i + 1);   // midpoint * parts < limit  <=>  it lies in share i
            const int first = req;
            while (req < b && (i == parts - 1 || (2 * before + nblk[req]) * parts < 2 * limit)) before += nblk[req++];
            int* rec = meta + 8 * i;
            rec[0] = first;
            rec[1] = req - 1;
            rec[2] = 0;
            rec[3] = req > first ? nblk[req - 1] : 0;
            rec[4] = 0;
            rec[5] = 0;
            rec[6] = 0;
            rec[7] = 0;
        }
    }
    for (int i = threadIdx.x; i <= b; i += 32) num_splits[i] = i;
}

// ------------------------------------------------------------------------------------------
// Split combine.  A request whose key blocks were divided between sm-parts has one fp32 partial
// (O/l, log2 l + m) per split.  Every split request ends some part while continuing into the
// next one; the part in which it STARTS (split 0) owns its merge.  One CTA per (part, token,
// group of 8 heads), one warp per head:
//   g = log2 sum_i 2^lse_i ; lse = g / log2e ; with a sink g += log2(1 + 2^(sink*log2e - g));
//   out = sum_i 2^(lse_i - g) * o_i                       (reference csrc/split_kv/combine.cu:66-160)
// ------------------------------------------------------------------------------------------
constexpr int kMaxSplits = 192;

__global__ void __launch_bounds__(256) mxdsa_combine_kernel(int b, int s_q, int parts, const int* meta,
                                                           const int* num_splits, const float* o_accum,
                                                           const float* lse_accum, const float* sink,
                                                           __nv_bfloat16* out, float* lse) {
    __shared__ float weight[8][kMaxSplits];
    const int part = blockIdx.x / s_q, tok = blockIdx.x % s_q;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int head = blockIdx.y * 8 + warp;
    const int* rec = meta + 8 * part;
    const int begin_req = rec[0], r = rec[1];
    if (begin_req >= b || r < 0 || r >= b) return;
    if (!(begin_req < r || rec[2] == 0)) return;           // the request started in an earlier part
    const int s0 = num_splits[r], n = num_splits[r + 1] - s0;
    if (n <= 1) return;
    // Launched as a programmatic dependent of the attention kernel (mxdsa_decode_fwd), this grid may start while
    // that one is still running: everything above reads the schedule only, everything below reads the partials,
    // which are complete and visible once the wait returns.  After a plain launch the wait returns at once.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float* lse_in = lse_accum + ((long long)s0 * s_q + tok) * 64 + head;
    const long long lse_stride = (long long)s_q * 64;
    float mx = -CUDART_INF_F;
    for (int i = lane; i < n; i += 32) mx = fmaxf(mx, lse_in[i * lse_stride]);
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (mx == -CUDART_INF_F) mx = 0.f;
    float sum = 0.f;
    for (int i = lane; i < n; i += 32) sum += sm100::ex2_approx(lse_in[i * lse_stride] - mx);
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    float g = sum == 0.f ? CUDART_INF_F : sm100::lg2_approx(sum) + mx;
    if (lane == 0) lse[((long long)r * s_q + tok) * 64 + head] = g / 1.4426950408889634f;
    if (sink != nullptr) {
        const float sk = sink[head];
        if (g != CUDART_INF_F) g += sm100::lg2_approx(1.f + sm100::ex2_approx(sk * CUDART_L2E_F - g));
        else g = sk == -CUDART_INF_F ? CUDART_INF_F : sk * CUDART_L2E_F;
    }
    for (int i = lane; i < n; i += 32) weight[warp][i] = sm100::ex2_approx(lse_in[i * lse_stride] - g);
    __syncwarp();
    const float* o_in = o_accum + (((long long)s0 * s_q + tok) * 64 + head) * 512;
    const long long o_stride = (long long)s_q * 64 * 512;
    float4 acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = 0; i < n; ++i) {
        const float wgt = weight[warp][i];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 v = *reinterpret_cast<const float4*>(o_in + i * o_stride + j * 128 + lane * 4);
            acc[j].x += wgt * v.x;
            acc[j].y += wgt * v.y;
            acc[j].z += wgt * v.z;
            acc[j].w += wgt * v.w;
        }
    }
    __nv_bfloat16* dst = out + (((long long)r * s_q + tok) * 64 + head) * 512;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc[j].x, acc[j].y), hi = __floats2bfloat162_rn(acc[j].z, acc[j].w);
        uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        *reinterpret_cast<uint2*>(dst + j * 128 + lane * 4) = pk;
    }
}

}  // namespace

// ==============================================================================================
extern "C" {

const char* mxdsa_status_string(int status) {
    switch (status) {
        case MXDSA_OK: return "ok";
        case MXDSA_ERR_NULL: return "a required pointer is NULL";
        case MXDSA_ERR_SHAPE: return "a size rule is violated";
        case MXDSA_ERR_ALIGN: return "a pointer or stride is misaligned";
        case MXDSA_ERR_DEVICE: return "the current device is not compute capability 10.x";
        case MXDSA_ERR_CUDA: return "a CUDA call failed (see mxdsa_last_cuda_error)";
        case MXDSA_ERR_WORKSPACE: return "workspace missing or too small";
        case MXDSA_ERR_DEVICE_TIMEOUT: return "a kernel abandoned a bounded wait";
        default: return "unknown status";
    }
}

int mxdsa_last_cuda_error(void) { return tl_last_cuda_error; }

int mxdsa_device_fault(void* stream) {
    DeviceInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MXDSA_OK) return st;
    MX_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    mxdsa::DeviceFault f;
    MX_CUDA(cudaMemcpy(&f, d->fault, sizeof(f), cudaMemcpyDeviceToHost));
    if (f.flag != 0) {
        fprintf(stderr, "mxdsa: a kernel abandoned wait #%d\n", f.where);
        MX_CUDA(cudaMemset(d->fault, 0, sizeof(f)));
        return MXDSA_ERR_DEVICE_TIMEOUT;
    }
    return MXDSA_OK;
}


// Runs the bounded-wait self-test kernel (attn_sm100.cuh) on `stream`.  Afterwards mxdsa_device_fault(stream)
// reports MXDSA_ERR_DEVICE_TIMEOUT once and clears the record; the context stays usable.
int mxdsa_selftest_bounded_wait(void* stream) {
    DeviceInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MXDSA_OK) return st;
    void* counter = nullptr;
    MX_CUDA(cudaGetSymbolAddress(&counter, g_selftest_teardowns));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2);
    cfg.blockDim = dim3(64);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim = {2, 1, 1};
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    MX_CUDA(cudaLaunchKernelEx(&cfg, mxdsa::mxdsa_wait_selftest_kernel, d->fault, static_cast<int*>(counter)));
    return MXDSA_OK;
}

// Launches the issue-only tensor-core rate probe (attn_sm100.cuh) on every CTA pair of the device: `iters` batches
// of 64 block-scaled E4M3 MMAs of shape M128 x N`n` x K32 per pair.  `data` = at least 64 KB of operand bytes.
// The caller times the launch; flops = (SMs / 2) * iters * 64 * 2 * 128 * n * 32.
int mxdsa_selftest_mma_rate(const void* data, int n, int iters, void* stream) {
    if (data == nullptr) return MXDSA_ERR_NULL;
    if ((n != 128 && n != 256) || iters <= 0) return MXDSA_ERR_SHAPE;
    if (!aligned16(data)) return MXDSA_ERR_ALIGN;
    DeviceInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MXDSA_OK) return st;
    const int smem = 65536 + 1024 + 256;
    MX_CUDA(cudaFuncSetAttribute(mxdsa::mxdsa_mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (d->sm_count / 2));
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim = {2, 1, 1};
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    MX_CUDA(cudaLaunchKernelEx(&cfg, mxdsa::mxdsa_mma_rate_kernel, static_cast<const uint4*>(data), n, iters, d->fault));
    return MXDSA_OK;
}

// Number of CTAs of the self-test that have left through their tear-down since the library was loaded.
int mxdsa_selftest_teardowns(void* stream) {
    MX_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    int n = 0;
    MX_CUDA(cudaMemcpyFromSymbol(&n, g_selftest_teardowns, sizeof(int)));
    return n;
}

int mxdsa_prefill_fwd(const mxdsa_prefill_params* p) {
    if (p == nullptr || p->q == nullptr || p->kv == nullptr || p->indices == nullptr || p->out == nullptr ||
        p->max_logits == nullptr || p->lse == nullptr)
        return MXDSA_ERR_NULL;
    if (p->s_q <= 0 || p->s_kv <= 0 || p->topk <= 0) return MXDSA_ERR_SHAPE;
    if (p->stride_q_token < (int64_t)MXDSA_HEADS * MXDSA_ROW_BYTES || p->stride_indices_pair < p->topk)
        return MXDSA_ERR_SHAPE;
    if (!aligned16(p->q) || !aligned16(p->kv) || (p->stride_q_token & 15) || !aligned32(p->out))
        return MXDSA_ERR_ALIGN;
    DeviceInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MXDSA_OK) return st;

    mxdsa::AttnParams ap;
    memset(&ap, 0, sizeof(ap));
    ap.q = static_cast<const uint8_t*>(p->q);
    ap.stride_q_tok = p->stride_q_token;
    ap.stride_q_b = p->stride_q_token * p->s_q;
    ap.s_q = p->s_q;
    ap.topk = p->topk;
    ap.scale_log2 = p->sm_scale * 1.44269504f;
    ap.attn_sink = p->attn_sink;
    ap.indices = p->indices;
    ap.idx_stride_row = p->stride_indices_pair;
    ap.topk_length = p->topk_length;
    ap.out = static_cast<__nv_bfloat16*>(p->out);
    ap.lse = p->lse;
    ap.max_logits = p->max_logits;
    memcpy(ap.w1, p->w1, sizeof(ap.w1));
    memcpy(ap.w2, p->w2, sizeof(ap.w2));
    ap.fault = d->fault;
    ap.s_kv = p->s_kv;
    ap.num_pairs = (p->s_q + 1) / 2;   // the last pair of an odd batch has one token: its second half is computed on a repeated row and not stored
    ap.kv = static_cast<const uint8_t*>(p->kv);
    ap.kv_scales = static_cast<const uint8_t*>(p->kv) + (size_t)p->s_kv * MXDSA_DIM;
    ap.b = 1;

    mxdsa::TensorMaps maps;
    memset(&maps, 0, sizeof(maps));
    st = make_q_map(&maps.q, p->q, (uint64_t)p->s_q, 1, (uint64_t)p->stride_q_token, (uint64_t)ap.stride_q_b);
    if (st != MXDSA_OK) return st;
    st = make_kv_map(&maps.kv, p->kv, (uint64_t)p->s_kv);
    if (st != MXDSA_OK) return st;
    st = make_out_map(&maps.out, p->out, (uint64_t)p->s_q);
    if (st != MXDSA_OK) return st;

    const int clusters = ap.num_pairs < d->sm_count / 2 ? ap.num_pairs : d->sm_count / 2;
    const dim3 grid(2 * clusters, 1, 1);
    cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
    constexpr int G = MXDSA_GROUPS_PREFILL;
    if (p->topk >= 512) return launch_pairs(mxdsa::mxdsa_attn_kernel<false, 128, G>, G, grid, stream, ap, maps);
    return launch_pairs(mxdsa::mxdsa_attn_kernel<false, 64, G>, G, grid, stream, ap, maps);
}

int mxdsa_num_sm_parts(int device, int s_q) {
    int sms = 0;
    if (s_q <= 0 || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
    int parts = sms / s_q;
    return parts > 1 ? parts : 1;
}

int mxdsa_decode_sched(const mxdsa_sched_params* p) {
    if (p == nullptr || p->sched_meta == nullptr || p->num_splits == nullptr) return MXDSA_ERR_NULL;
    if (p->b <= 0 || p->s_q <= 0 || p->topk <= 0 || p->extra_topk < 0 || p->num_sm_parts <= 0) return MXDSA_ERR_SHAPE;
    const size_t smem = sizeof(int) * (2 * (size_t)p->b + 1);
    if (smem > 200 * 1024) return MXDSA_ERR_SHAPE;
    MX_CUDA(cudaFuncSetAttribute(mxdsa_sched_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mxdsa_sched_kernel<<<1, 32, smem, static_cast<cudaStream_t>(p->stream)>>>(
        p->b, p->topk, p->extra_topk, p->topk_length, p->extra_topk_length, p->num_sm_parts, p->sched_meta,
        p->num_splits);
    MX_CUDA(cudaGetLastError());
    return MXDSA_OK;
}

// The whole-request schedule (see mxdsa_sched_whole_kernel): for mxdsa_decode_fwd_nocombine.
int mxdsa_decode_sched_whole(const mxdsa_sched_params* p) {
    if (p == nullptr || p->sched_meta == nullptr || p->num_splits == nullptr) return MXDSA_ERR_NULL;
    if (p->b <= 0 || p->s_q <= 0 || p->topk <= 0 || p->extra_topk < 0 || p->num_sm_parts <= 0) return MXDSA_ERR_SHAPE;
    const size_t smem = sizeof(int) * (2 * (size_t)p->b + 1);
    if (smem > 200 * 1024) return MXDSA_ERR_SHAPE;
    MX_CUDA(cudaFuncSetAttribute(mxdsa_sched_whole_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mxdsa_sched_whole_kernel<<<1, 32, smem, static_cast<cudaStream_t>(p->stream)>>>(
        p->b, p->topk, p->extra_topk, p->topk_length, p->extra_topk_length, p->num_sm_parts, p->sched_meta,
        p->num_splits);
    MX_CUDA(cudaGetLastError());
    return MXDSA_OK;
}

size_t mxdsa_decode_workspace_bytes(int b, int s_q, int num_sm_parts) {
    if (b <= 0 || s_q <= 0 || num_sm_parts <= 0) return 0;
    const size_t splits = (size_t)b + (size_t)num_sm_parts;
    return splits * s_q * MXDSA_HEADS * (MXDSA_DIM + 1) * sizeof(float);
}

static int decode_impl(const mxdsa_decode_params* p, bool combine) {
    if (p == nullptr || p->q == nullptr || p->kv == nullptr || p->indices == nullptr || p->out == nullptr ||
        p->lse == nullptr || p->sched_meta == nullptr || p->num_splits == nullptr)
        return MXDSA_ERR_NULL;
    if (p->b <= 0 || p->s_q <= 0 || p->topk <= 0 || (p->topk % 64) != 0 || p->extra_topk < 0 ||
        p->num_sm_parts <= 0 || p->num_sm_parts > kMaxSplits || p->page_block_size <= 0 || p->num_blocks <= 0)
        return MXDSA_ERR_SHAPE;
    const bool has_extra = p->extra_kv != nullptr;
    if (has_extra != (p->extra_indices != nullptr)) return MXDSA_ERR_SHAPE;
    if (!has_extra && (p->extra_topk != 0 || p->extra_topk_length != nullptr)) return MXDSA_ERR_SHAPE;
    if (has_extra && (p->extra_page_block_size <= 0 || p->extra_num_blocks <= 0)) return MXDSA_ERR_SHAPE;
    if ((p->stride_kv_block % 512) != 0 || p->stride_kv_block < (int64_t)p->page_block_size * MXDSA_ROW_BYTES)
        return MXDSA_ERR_ALIGN;
    if (has_extra && ((p->stride_extra_kv_block % 512) != 0 ||
                      p->stride_extra_kv_block < (int64_t)p->extra_page_block_size * MXDSA_ROW_BYTES))
        return MXDSA_ERR_ALIGN;
    if (!aligned16(p->q) || !aligned16(p->kv) || (has_extra && !aligned16(p->extra_kv)) || (p->stride_q_s & 15) ||
        (p->stride_q_b & 15) || !aligned32(p->out))
        return MXDSA_ERR_ALIGN;
    if (p->stride_q_s < (int64_t)MXDSA_HEADS * MXDSA_ROW_BYTES) return MXDSA_ERR_SHAPE;
    const size_t need = mxdsa_decode_workspace_bytes(p->b, p->s_q, p->num_sm_parts);
    if (combine && (p->workspace == nullptr || p->workspace_bytes < need || !aligned32(p->workspace)))
        return MXDSA_ERR_WORKSPACE;
    DeviceInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MXDSA_OK) return st;

    // without a combine step there are no partials: the schedule must give every request to one part
    const size_t splits = (size_t)p->b + (size_t)p->num_sm_parts;
    float* o_accum = combine ? static_cast<float*>(p->workspace) : nullptr;
    float* lse_accum = combine ? o_accum + splits * p->s_q * MXDSA_HEADS * MXDSA_DIM : nullptr;

    mxdsa::AttnParams ap;
    memset(&ap, 0, sizeof(ap));
    ap.q = static_cast<const uint8_t*>(p->q);
    ap.stride_q_tok = p->stride_q_s;
    ap.stride_q_b = p->stride_q_b;
    ap.s_q = p->s_q;
    ap.topk = p->topk;
    ap.scale_log2 = p->sm_scale * 1.44269504f;
    ap.attn_sink = p->attn_sink;
    ap.indices = p->indices;
    ap.idx_stride_row = p->stride_indices_s;
    ap.idx_stride_b = p->stride_indices_b;
    ap.topk_length = p->topk_length;
    ap.out = static_cast<__nv_bfloat16*>(p->out);
    ap.lse = p->lse;
    memcpy(ap.w1, p->w1, sizeof(ap.w1));
    memcpy(ap.w2, p->w2, sizeof(ap.w2));
    ap.fault = d->fault;
    ap.b = p->b;
    ap.page_size = p->page_block_size;
    ap.rows_per_block = (int)(p->stride_kv_block / 512);
    ap.kv = static_cast<const uint8_t*>(p->kv);
    ap.stride_block = p->stride_kv_block;
    ap.extra_topk = has_extra ? p->extra_topk : 0;
    if (has_extra) {
        ap.extra_page_size = p->extra_page_block_size;
        ap.extra_rows_per_block = (int)(p->stride_extra_kv_block / 512);
        ap.extra_kv = static_cast<const uint8_t*>(p->extra_kv);
        ap.extra_stride_block = p->stride_extra_kv_block;
        ap.extra_indices = p->extra_indices;
        ap.eidx_stride_row = p->stride_extra_indices_s;
        ap.eidx_stride_b = p->stride_extra_indices_b;
        ap.extra_topk_length = p->extra_topk_length;
    }
    auto log2_exact = [](int v) { int s = 0; while ((1 << s) < v) ++s; return (1 << s) == v ? s : -1; };
    ap.page_shift = log2_exact(p->page_block_size);
    ap.extra_page_shift = has_extra ? log2_exact(p->extra_page_block_size) : -1;
    auto rows32 = [](long long blocks, long long page) {
        const long long r = blocks * page;
        return (unsigned)(r > 0x80000000ll ? 0x80000000ll : r);   // indices are int32: nothing beyond 2^31 can be named
    };
    ap.pool_rows32 = rows32(p->num_blocks, p->page_block_size);
    ap.extra_pool_rows32 = has_extra ? rows32(p->extra_num_blocks, p->extra_page_block_size) : 0u;
    ap.row_gap = (unsigned)(ap.rows_per_block - p->page_block_size);
    ap.extra_row_gap = has_extra ? (unsigned)(ap.extra_rows_per_block - p->extra_page_block_size) : 0u;
    ap.sched_meta = p->sched_meta;
    ap.num_splits = p->num_splits;
    ap.o_accum = o_accum;
    ap.lse_accum = lse_accum;

    mxdsa::TensorMaps maps;
    memset(&maps, 0, sizeof(maps));
    st = make_q_map(&maps.q, p->q, (uint64_t)p->s_q, (uint64_t)p->b, (uint64_t)p->stride_q_s,
                    p->b > 1 ? (uint64_t)p->stride_q_b : (uint64_t)p->stride_q_s * p->s_q);
    if (st != MXDSA_OK) return st;
    // the last page of a pool may be shorter than the page stride: only its data rows are in the view
    st = make_kv_map(&maps.kv, p->kv,
                     (uint64_t)(p->num_blocks - 1) * (uint64_t)ap.rows_per_block + (uint64_t)p->page_block_size);
    if (st != MXDSA_OK) return st;
    if (has_extra) {
        st = make_kv_map(&maps.ekv, p->extra_kv, (uint64_t)(p->extra_num_blocks - 1) * (uint64_t)ap.extra_rows_per_block +
                                                     (uint64_t)p->extra_page_block_size);
        if (st != MXDSA_OK) return st;
    }

    st = make_out_map(&maps.out, p->out, (uint64_t)p->b * (uint64_t)p->s_q);
    if (st != MXDSA_OK) return st;

    cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
    const dim3 grid(2 * ((p->s_q + 1) / 2), p->num_sm_parts, 1);
    st = launch_pairs(mxdsa::mxdsa_attn_kernel<true, 64, MXDSA_GROUPS_DECODE>, MXDSA_GROUPS_DECODE, grid, stream, ap, maps);
    if (st != MXDSA_OK) return st;
    if (!combine) return MXDSA_OK;
    const dim3 cgrid(p->num_sm_parts * p->s_q, MXDSA_HEADS / 8, 1);
    // programmatic dependent launch: the combine grid is set up while the attention grid drains (the attention
    // kernel releases its dependents as soon as it has started; the combine kernel waits before it reads)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = cgrid;
    cfg.blockDim = dim3(256, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = MXDSA_COMBINE_PDL;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MX_CUDA(cudaLaunchKernelEx(&cfg, mxdsa_combine_kernel, (int)p->b, (int)p->s_q, (int)p->num_sm_parts,
                               (const int*)p->sched_meta, (const int*)p->num_splits, (const float*)o_accum,
                               (const float*)lse_accum, (const float*)p->attn_sink,
                               static_cast<__nv_bfloat16*>(p->out), (float*)p->lse));
    return MXDSA_OK;
}

extern "C" int mxdsa_decode_fwd(const mxdsa_decode_params* p) { return decode_impl(p, true); }

// Decode without a combine pass: attention only, no workspace.  The schedule must not divide any request between
// parts (mxdsa_decode_sched_whole writes such a schedule); if it does, the kernel leaves the divided request's
// output incomplete and raises the device fault record (code 71, reported by mxdsa_device_fault) instead of
// writing partials that nobody would merge.
extern "C" int mxdsa_decode_fwd_nocombine(const mxdsa_decode_params* p) { return decode_impl(p, false); }

// ------------------------------------------------------------------------------------------
// The combine step on its own: merges the split partials that an earlier mxdsa_decode_fwd (or any
// producer of the same workspace layout) left in `workspace`.  mxdsa_decode_fwd runs it itself; this
// entry point exists for callers that sequence attention and combine separately, as the reference's
// binding does (run_flash_mla_combine_kernel, reference csrc/split_kv/combine.cu:415-448).
// ------------------------------------------------------------------------------------------
extern "C" int mxdsa_decode_combine(const mxdsa_combine_params* p) {
    if (p == nullptr || p->sched_meta == nullptr || p->num_splits == nullptr || p->out == nullptr || p->lse == nullptr)
        return MXDSA_ERR_NULL;
    if (p->b <= 0 || p->s_q <= 0 || p->num_sm_parts <= 0 || p->num_sm_parts > kMaxSplits) return MXDSA_ERR_SHAPE;
    const size_t need = mxdsa_decode_workspace_bytes(p->b, p->s_q, p->num_sm_parts);
    if (p->workspace == nullptr || p->workspace_bytes < need || !aligned32(p->workspace)) return MXDSA_ERR_WORKSPACE;
    if (!aligned32(p->out)) return MXDSA_ERR_ALIGN;
    const size_t slots = (size_t)(p->b + p->num_sm_parts) * p->s_q * MXDSA_HEADS;
    const float* o_accum = static_cast<const float*>(p->workspace);
    const float* lse_accum = o_accum + slots * MXDSA_DIM;
    const dim3 cgrid(p->num_sm_parts * p->s_q, MXDSA_HEADS / 8, 1);
    mxdsa_combine_kernel<<<cgrid, 256, 0, static_cast<cudaStream_t>(p->stream)>>>(
        p->b, p->s_q, p->num_sm_parts, p->sched_meta, p->num_splits, o_accum, lse_accum, p->attn_sink,
        static_cast<__nv_bfloat16*>(p->out), p->lse);
    MX_CUDA(cudaGetLastError());
    return MXDSA_OK;
}

// ------------------------------------------------------------------------------------------
// Decode for callers that cannot allocate device memory.
//
// Some hosts of this library hand out no allocator at all: a serving process that gives every
// plugin a fixed memory budget and forbids cudaMalloc after start-up, or a caller that is already
// inside a region where the CUDA allocator must not be entered.  mxdsa_decode_fwd needs scratch
// for the split partials, and normally the caller provides it.  This variant keeps that scratch in
// the library image instead: a file-scope device array of MXDSA_STATIC_SCRATCH_BYTES, which every
// GPU that loads the library holds until the process exits.
//
// The array's name is only a host-side handle here; the device address is looked up once per
// device with cudaGetSymbolAddress (with that device current) and then passed to the kernels like
// any other workspace pointer.
// ------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[MXDSA_STATIC_SCRATCH_BYTES];

namespace {
void* g_static_scratch_addr[64] = {};
std::mutex g_static_scratch_mutex;
}  // namespace

int mxdsa_decode_fwd_static(const mxdsa_decode_params* p) {
    if (p == nullptr) return MXDSA_ERR_NULL;
    const size_t need = mxdsa_decode_workspace_bytes(p->b, p->s_q, p->num_sm_parts);
    if (need == 0) return MXDSA_ERR_SHAPE;
    if (need > (size_t)MXDSA_STATIC_SCRATCH_BYTES) return MXDSA_ERR_WORKSPACE;
    int dev = 0;
    MX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return MXDSA_ERR_DEVICE;
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (g_static_scratch_addr[dev] == nullptr) {
            void* addr = nullptr;
            MX_CUDA(cudaGetSymbolAddress(&addr, g_static_scratch));   // first call on this device
            g_static_scratch_addr[dev] = addr;
        }
        scratch = g_static_scratch_addr[dev];
    }
    mxdsa_decode_params q = *p;
    q.workspace = scratch;
    q.workspace_bytes = MXDSA_STATIC_SCRATCH_BYTES;
    return mxdsa_decode_fwd(&q);
}

}  // extern "C"

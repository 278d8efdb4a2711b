// Quantise-and-pack kernels: activations / KV rows (bf16 or fp32) -> the uint8 wire format that the
// attention entry points consume.  One pass over HBM: a warp reads one 512-wide row, forms the eight
// group maxima with two shuffles, derives the UE8M0 scales, converts to E4M3 and writes the 512 data
// bytes (one 16-byte store per lane) and the 16-byte scale slot.
//
// Same arithmetic as the reference's Python packers (reference tests/mxfp8_test_utils.py:11-27):
//   scale = 2^ceil(log2(max(amax/448, 2^-126)));  code = e4m3(clamp(x / scale, -448, 448))
// with the ceil(log2()) taken exactly from the bits of the float (exponent, +1 when the mantissa is
// not zero).  Compiled WITHOUT fast-math: amax/448 must be the correctly rounded quotient.
//
// Bound: HBM.  Algorithmic bytes per row: 512 * sizeof(input element) read + 528 written.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mxdsa.h"

namespace {

constexpr int kDim = 512;
constexpr int kWarpsPerBlock = 8;

// UE8M0 byte of 2^ceil(log2(max(amax/448, 2^-126))) and the factor 2^-e to multiply by
__device__ __forceinline__ uint32_t scale_byte(float amax, float& inv_scale) {
    float s = __fdiv_rn(amax, 448.0f);
    s = fmaxf(s, 1.17549435e-38f);                       // 2^-126
    const uint32_t bits = __float_as_uint(s);
    const uint32_t byte = (bits >> 23) + ((bits & 0x7FFFFFu) != 0u ? 1u : 0u);   // e + 127, 1..254
    inv_scale = __uint_as_float((254u - byte) << 23);    // 2^(127 - byte) = 2^-e
    return byte;
}

__device__ __forceinline__ uint16_t e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

template <typename T> __device__ __forceinline__ void load16(const T* src, float (&x)[16]);
template <> __device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* src, float (&x)[16]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(src));
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(src) + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        x[2 * i] = __uint_as_float(w[i] << 16);
        x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
template <> __device__ __forceinline__ void load16<float>(const float* src, float (&x)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(src) + i);
        x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
    }
}

// QGROUPS: true  -> Q rows: scale g covers dims [32g,32g+32) and [256+32g,256+32g+32)
//          false -> KV rows: scale g covers dims [64g,64g+64)
// Lane L owns dims [16L, 16L+16).
template <typename T, bool QGROUPS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
mxdsa_pack_rows_kernel(const T* __restrict__ src, long long src_stride, long long rows, uint8_t* __restrict__ data,
                       long long data_stride, uint8_t* __restrict__ slots, long long slot_stride, int rows_per_page,
                       long long page_stride, int paired_storage) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * kWarpsPerBlock;
    for (long long r = warp0; r < rows; r += nwarps) {
        float x[16];
        load16<T>(src + r * src_stride + 16 * lane, x);
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
        // the group's four lanes: Q {2g, 2g+1, 2g+16, 2g+17}; KV {4g .. 4g+3}
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, QGROUPS ? 16 : 2));
        float inv;
        const uint32_t byte = scale_byte(amax, inv);
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = fminf(fmaxf(x[4 * i + j] * inv, -448.0f), 448.0f);
            w[i] = (uint32_t)e4m3x2(v[0], v[1]) | ((uint32_t)e4m3x2(v[2], v[3]) << 16);
        }
        // page addressing: rows_per_page rows of data, then their slots (prefill plane: one page of all rows)
        const long long page = r / rows_per_page, in_page = r % rows_per_page;
        uint8_t* drow = data + page * page_stride + in_page * data_stride;
        uint8_t* srow = slots + page * page_stride + in_page * slot_stride;
        int off = 16 * lane;
        if (QGROUPS && paired_storage) {   // [g][half][32]: natural chunk c = lane/2 -> chunk 2*(c%8) + c/8
            const int c = lane >> 1;
            off = (2 * (c & 7) + (c >> 3)) * 32 + (lane & 1) * 16;
        }
        *reinterpret_cast<uint4*>(drow + off) = make_uint4(w[0], w[1], w[2], w[3]);
        const bool leader = QGROUPS ? (lane < 16 && (lane & 1) == 0) : ((lane & 3) == 0);
        if (leader) {
            const int g = QGROUPS ? (lane >> 1) : (lane >> 2);
            srow[g] = (uint8_t)byte;
            srow[8 + g] = (uint8_t)byte;
        }
    }
}

thread_local int tl_pack_cuda_error = 0;

template <typename T, bool Q>
int launch(const T* src, long long src_stride, long long rows, uint8_t* data, long long data_stride, uint8_t* slots,
           long long slot_stride, int rows_per_page, long long page_stride, int paired, cudaStream_t stream) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return MXDSA_ERR_CUDA;
    const long long want = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const int grid = (int)(want < (long long)sms * 8 ? want : (long long)sms * 8);   // 8 resident CTAs of 256 threads per SM
    mxdsa_pack_rows_kernel<T, Q><<<grid, kWarpsPerBlock * 32, 0, stream>>>(src, src_stride, rows, data, data_stride, slots,
                                                                           slot_stride, rows_per_page, page_stride, paired);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        tl_pack_cuda_error = (int)e;
        return MXDSA_ERR_CUDA;
    }
    return MXDSA_OK;
}

}  // namespace

extern "C" int mxdsa_pack_q(const mxdsa_pack_q_params* p) {
    if (p == nullptr || p->src == nullptr || p->dst == nullptr) return MXDSA_ERR_NULL;
    if (p->rows < 0 || (p->src_dtype != MXDSA_DTYPE_BF16 && p->src_dtype != MXDSA_DTYPE_F32)) return MXDSA_ERR_SHAPE;
    if (p->rows == 0) return MXDSA_OK;
    const long long st = p->src_stride_row ? p->src_stride_row : kDim;
    const long long dt = p->dst_stride_row ? p->dst_stride_row : MXDSA_ROW_BYTES;
    if (((uintptr_t)p->src & 15) || ((uintptr_t)p->dst & 15) || (dt & 15) || dt < MXDSA_ROW_BYTES ||
        (st * (p->src_dtype == MXDSA_DTYPE_BF16 ? 2 : 4)) % 16 != 0 || st < kDim)
        return MXDSA_ERR_ALIGN;
    uint8_t* dst = static_cast<uint8_t*>(p->dst);
    const cudaStream_t s = static_cast<cudaStream_t>(p->stream);
    // Q rows: data and slot of a row are adjacent; one "page" holds every row
    const int big = 0x7fffffff;
    if (p->src_dtype == MXDSA_DTYPE_BF16)
        return launch<__nv_bfloat16, true>(static_cast<const __nv_bfloat16*>(p->src), st, p->rows, dst, dt, dst + kDim, dt, big,
                                           0, p->paired_storage, s);
    return launch<float, true>(static_cast<const float*>(p->src), st, p->rows, dst, dt, dst + kDim, dt, big, 0,
                               p->paired_storage, s);
}

extern "C" int mxdsa_pack_kv(const mxdsa_pack_kv_params* p) {
    if (p == nullptr || p->src == nullptr || p->dst == nullptr) return MXDSA_ERR_NULL;
    if (p->rows < 0 || p->rows_per_page <= 0 || (p->src_dtype != MXDSA_DTYPE_BF16 && p->src_dtype != MXDSA_DTYPE_F32))
        return MXDSA_ERR_SHAPE;
    if (p->rows == 0) return MXDSA_OK;
    if (p->rows % p->rows_per_page != 0) return MXDSA_ERR_SHAPE;
    const long long st = p->src_stride_row ? p->src_stride_row : kDim;
    const long long pg = p->dst_stride_page ? p->dst_stride_page : (long long)p->rows_per_page * MXDSA_ROW_BYTES;
    if (((uintptr_t)p->src & 15) || ((uintptr_t)p->dst & 15) || (pg & 15) ||
        pg < (long long)p->rows_per_page * MXDSA_ROW_BYTES ||
        (st * (p->src_dtype == MXDSA_DTYPE_BF16 ? 2 : 4)) % 16 != 0 || st < kDim)
        return MXDSA_ERR_ALIGN;
    uint8_t* dst = static_cast<uint8_t*>(p->dst);
    uint8_t* slots = dst + (long long)p->rows_per_page * kDim;
    const cudaStream_t s = static_cast<cudaStream_t>(p->stream);
    if (p->src_dtype == MXDSA_DTYPE_BF16)
        return launch<__nv_bfloat16, false>(static_cast<const __nv_bfloat16*>(p->src), st, p->rows, dst, kDim, slots, 16,
                                            p->rows_per_page, pg, 0, s);
    return launch<float, false>(static_cast<const float*>(p->src), st, p->rows, dst, kDim, slots, 16, p->rows_per_page, pg, 0, s);
}

extern "C" int mxdsa_pack_last_cuda_error(void) { return tl_pack_cuda_error; }

// PyTorch extension module `mxdsa_ext`: the operator-level interface of the library.
//
// Exposes the two entry points of the reference extension with the same positional arguments,
// validation rules and return values (reference csrc/bindings/binding.cpp:12-118 and
// csrc/bindings/dual_mxfp8_sparse_decode.h:13-243), implemented over the C ABI of libmxdsa.so.
// torch supplies tensors, the caching allocator and the current stream; all device work happens
// inside the library.  Nothing here synchronises.
#include <optional>
#include <string>
#include <tuple>
#include <vector>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "mxdsa.h"

namespace {

using OptTensor = std::optional<at::Tensor>;

constexpr int64_t kDim = MXDSA_DIM;
constexpr int64_t kRow = MXDSA_ROW_BYTES;
constexpr int64_t kHeads = MXDSA_HEADS;

void require_status(int status, const char* what) {
    TORCH_CHECK(status == MXDSA_OK, what, ": ", mxdsa_status_string(status), " (status ", status, ", cuda error ",
                mxdsa_last_cuda_error(), ")");
}

// shape / dtype / placement rule for an optional tensor argument
void check_optional(const OptTensor& t, const char* name, at::ScalarType dtype, at::IntArrayRef shape) {
    if (!t.has_value()) return;
    TORCH_CHECK(t->is_cuda(), name, " must be on CUDA");
    TORCH_CHECK(t->scalar_type() == dtype, name, " must have dtype ", dtype);
    TORCH_CHECK(t->sizes() == shape, name, " must have shape ", shape);
    TORCH_CHECK(t->dim() == 0 || t->size(-1) == 1 || t->stride(-1) == 1, name, " must have contiguous last dimension");
}

template <typename T> T* opt_ptr(const OptTensor& t) {
    return t.has_value() && t->has_storage() ? static_cast<T*>(t->data_ptr()) : nullptr;
}

void copy_words(const std::vector<uint32_t>& w1, const std::vector<uint32_t>& w2, uint32_t* d1, uint32_t* d2) {
    TORCH_CHECK(w1.size() == 8 && w2.size() == 8, "w1 and w2 must each contain 8 pre-expanded TMEM scale words");
    for (int i = 0; i < 8; ++i) {
        d1[i] = w1[i];
        d2[i] = w2[i];
    }
}

bool is_e4m3_storage(const at::Tensor& t) {
    return t.scalar_type() == at::kByte || t.scalar_type() == at::kFloat8_e4m3fn;
}

// `extended` = false: the reference operator's rules to the letter (csrc/bindings/binding.cpp:36-71).
// `extended` = true: the same operator without three of its restrictions -- an odd number of query tokens (the last
// pair has one token; indices [ceil(s_q/2), 1, topk]), any positive topk (positions beyond it count as not attended,
// tiles of 128 keys from topk 512 on as in the reference), and torch.float8_e4m3fn as well as uint8 for q / kv (the
// bytes are the same; the decode operator of the reference already accepts both).
std::vector<at::Tensor> prefill_impl(const at::Tensor& q, const at::Tensor& kv, const at::Tensor& indices,
                                     double sm_scale, const std::vector<uint32_t>& w1,
                                     const std::vector<uint32_t>& w2, const OptTensor& attn_sink,
                                     const OptTensor& topk_length, bool extended) {
    TORCH_CHECK(q.dim() == 3, "q must have 3 dimensions");
    TORCH_CHECK(kv.dim() == 3, "kv must have 3 dimensions");
    TORCH_CHECK(indices.dim() == 3, "indices must have 3 dimensions");
    const int64_t s_q = q.size(0), h_q = q.size(1), s_kv = kv.size(0), h_kv = kv.size(1), topk = indices.size(2);
    TORCH_CHECK(s_q > 0 && (extended || s_q % 2 == 0), "q must contain an even, positive number of query tokens");
    const int64_t pairs = (s_q + 1) / 2;
    TORCH_CHECK(h_q == kHeads, "q must have shape [s_q, 64, 528]");
    TORCH_CHECK(h_kv == 1, "kv must have shape [s_kv, 1, 528]");
    TORCH_CHECK(q.size(2) == kRow,
                "q must store 512 E4M3 bytes followed by a replicated 16-byte UE8M0 scale slot per head");
    TORCH_CHECK(kv.size(2) == kRow, "kv must provide a 528-byte envelope per token for replicated page-tail scales");
    TORCH_CHECK(topk > 0 && (extended || topk % 64 == 0), "topk must be a positive multiple of 64");
    mxdsa_prefill_params p{};
    copy_words(w1, w2, p.w1, p.w2);
    TORCH_CHECK(q.is_cuda(), "q must be on CUDA");
    TORCH_CHECK(kv.is_cuda(), "kv must be on CUDA");
    TORCH_CHECK(indices.is_cuda(), "indices must be on CUDA");
    const bool fp8_ok = extended;
    TORCH_CHECK(q.scalar_type() == at::kByte || (fp8_ok && q.scalar_type() == at::kFloat8_e4m3fn),
                "q must have dtype torch.uint8");
    TORCH_CHECK(kv.scalar_type() == at::kByte || (fp8_ok && kv.scalar_type() == at::kFloat8_e4m3fn),
                "kv must have dtype torch.uint8");
    TORCH_CHECK(indices.scalar_type() == at::kInt, "indices must have dtype torch.int32");
    TORCH_CHECK(q.stride(-1) == 1, "q must have contiguous last dimension");
    TORCH_CHECK(kv.is_contiguous(), "kv must be contiguous");
    TORCH_CHECK(indices.stride(-1) == 1, "indices must have contiguous last dimension");
    TORCH_CHECK(indices.sizes() == at::IntArrayRef({pairs, 1, topk}),
                "indices must have shape (num_q_pairs, h_kv, topk)");
    check_optional(attn_sink, "attn_sink", at::kFloat, {kHeads});
    check_optional(topk_length, "topk_length", at::kInt, {pairs});
    TORCH_CHECK(q.stride(1) == kRow, "Q head stride must be 512 e4m3 bytes + an aligned 16-byte scale slot");
    for (int64_t st : q.strides()) TORCH_CHECK(st <= INT32_MAX, "Stride exceeds int32 limit: ", st);
    for (int64_t st : indices.strides()) TORCH_CHECK(st <= INT32_MAX, "Stride exceeds int32 limit: ", st);

    c10::cuda::CUDAGuard guard(q.device());
    TORCH_CHECK(at::cuda::getCurrentDeviceProperties()->major == 10,
                "Dual MXFP8 head64 sparse prefill requires SM100f.");
    const auto opts = q.options();
    at::Tensor out = at::empty({s_q, h_q, kDim}, opts.dtype(at::kBFloat16));
    at::Tensor max_logits = at::empty({s_q, h_q}, opts.dtype(at::kFloat));
    at::Tensor lse = at::empty({s_q, h_q}, opts.dtype(at::kFloat));
    p.s_q = (int32_t)s_q;
    p.s_kv = (int32_t)s_kv;
    p.topk = (int32_t)topk;
    p.sm_scale = (float)sm_scale;
    p.q = q.data_ptr();
    p.stride_q_token = q.stride(0);
    p.kv = kv.data_ptr();
    p.indices = indices.data_ptr<int32_t>();
    p.stride_indices_pair = indices.stride(0);
    p.attn_sink = opt_ptr<float>(attn_sink);
    p.topk_length = opt_ptr<int32_t>(topk_length);
    p.out = out.data_ptr();
    p.max_logits = max_logits.data_ptr<float>();
    p.lse = lse.data_ptr<float>();
    p.stream = at::cuda::getCurrentCUDAStream().stream();
    require_status(mxdsa_prefill_fwd(&p), "mxdsa_prefill_fwd");
    return {out, max_logits, lse};
}

std::vector<at::Tensor> prefill_fwd(const at::Tensor& q, const at::Tensor& kv, const at::Tensor& indices, double sm_scale,
                                    const std::vector<uint32_t>& w1, const std::vector<uint32_t>& w2,
                                    const OptTensor& attn_sink, const OptTensor& topk_length) {
    return prefill_impl(q, kv, indices, sm_scale, w1, w2, attn_sink, topk_length, false);
}
std::vector<at::Tensor> prefill_fwd_ex(const at::Tensor& q, const at::Tensor& kv, const at::Tensor& indices,
                                       double sm_scale, const std::vector<uint32_t>& w1, const std::vector<uint32_t>& w2,
                                       const OptTensor& attn_sink, const OptTensor& topk_length) {
    return prefill_impl(q, kv, indices, sm_scale, w1, w2, attn_sink, topk_length, true);
}

// `whole` = false: the reference operator.  `whole` = true: the same operator with a schedule of whole requests
// (mxdsa_decode_sched_whole), attention only -- no scratch, no combine pass; scheduling tensors passed in must come
// from an earlier call of the same entry point.
std::tuple<at::Tensor, at::Tensor, OptTensor, OptTensor> decode_impl(
    const at::Tensor& q, const at::Tensor& kv, const at::Tensor& indices, const OptTensor& topk_length,
    const OptTensor& attn_sink, OptTensor tile_scheduler_metadata, OptTensor num_splits, const OptTensor& extra_kv,
    const OptTensor& extra_indices, const OptTensor& extra_topk_length, int64_t d_qk, int64_t d_v, double sm_scale,
    const std::vector<uint32_t>& w1, const std::vector<uint32_t>& w2, bool whole) {
    TORCH_CHECK(q.dim() == 4, "q must have 4 dimensions");
    TORCH_CHECK(kv.dim() == 4, "kv must have 4 dimensions");
    TORCH_CHECK(indices.dim() == 3, "indices must have 3 dimensions");
    const int64_t b = q.size(0), s_q = q.size(1), h_q = q.size(2);
    const int64_t num_blocks = kv.size(0), page = kv.size(1), h_kv = kv.size(2), topk = indices.size(2);
    const bool have_extra = extra_kv.has_value();
    const int64_t extra_topk = extra_indices.has_value() ? extra_indices->size(2) : 0;
    TORCH_CHECK(b > 0 && s_q > 0, "b and s_q must be positive");
    TORCH_CHECK(h_q == kHeads, "Dual MXFP8 decode supports head64 only; got h_q=", h_q);
    TORCH_CHECK(h_kv == 1, "Dual MXFP8 decode requires h_kv=1");
    TORCH_CHECK(d_qk == kDim && d_v == kDim, "Dual MXFP8 decode requires d_qk=d_v=512");
    TORCH_CHECK(topk > 0 && topk % 64 == 0, "topk must be a positive multiple of 64");
    mxdsa_decode_params p{};
    copy_words(w1, w2, p.w1, p.w2);
    TORCH_CHECK(q.size(3) == kRow, "q must use the 528-byte head64 envelope");
    TORCH_CHECK(kv.size(3) == kRow, "kv must use the 528-byte head64 envelope");
    TORCH_CHECK(!have_extra || extra_indices.has_value(), "extra_indices must be provided with extra_kv");
    TORCH_CHECK(have_extra || (!extra_indices.has_value() && !extra_topk_length.has_value()),
                "extra indices require extra_kv");
    TORCH_CHECK(q.is_cuda() && kv.is_cuda() && indices.is_cuda(), "q, kv and indices must be on CUDA");
    TORCH_CHECK(is_e4m3_storage(q), "q must have E4M3 storage (uint8 or float8_e4m3fn)");
    TORCH_CHECK(is_e4m3_storage(kv), "kv must have E4M3 storage (uint8 or float8_e4m3fn)");
    TORCH_CHECK(indices.scalar_type() == at::kInt, "indices must have dtype torch.int32");
    TORCH_CHECK(q.stride(-1) == 1, "q must have contiguous last dimension");
    TORCH_CHECK(kv.is_contiguous(), "kv must be contiguous");
    TORCH_CHECK(indices.stride(-1) == 1, "indices must have contiguous last dimension");
    TORCH_CHECK(indices.sizes() == at::IntArrayRef({b, s_q, topk}), "indices must have shape (b, s_q, topk)");
    check_optional(topk_length, "topk_length", at::kInt, {b});
    check_optional(attn_sink, "attn_sink", at::kFloat, {kHeads});
    check_optional(extra_topk_length, "extra_topk_length", at::kInt, {b});
    if (have_extra) {
        TORCH_CHECK(extra_kv->is_cuda() && extra_indices->is_cuda(), "extra_kv and extra_indices must be on CUDA");
        TORCH_CHECK(is_e4m3_storage(*extra_kv), "extra_kv must have E4M3 storage");
        TORCH_CHECK(extra_kv->dim() == 4 && extra_kv->size(2) == 1 && extra_kv->size(3) == kRow,
                    "extra_kv must have shape [blocks, page, 1, 528]");
        TORCH_CHECK(extra_kv->stride(-1) == 1, "extra_kv must have contiguous last dimension");
        TORCH_CHECK(extra_indices->scalar_type() == at::kInt &&
                        extra_indices->sizes() == at::IntArrayRef({b, s_q, extra_topk}),
                    "extra_indices must have shape (b, s_q, extra_topk)");
        TORCH_CHECK(extra_topk == 0 || extra_indices->stride(-1) == 1,
                    "extra_indices must have contiguous last dimension");
        TORCH_CHECK(extra_kv->stride(1) == kRow, "dual extra KV row stride must be 528 bytes");
        TORCH_CHECK(extra_kv->stride(0) % 512 == 0, "dual extra KV page stride must be divisible by 512 bytes");
    }
    TORCH_CHECK(kv.stride(1) == kRow, "dual KV row stride must be 528 bytes, got ", kv.stride(1));
    TORCH_CHECK(kv.stride(0) % 512 == 0, "dual KV page stride must be divisible by 512 bytes, got ", kv.stride(0));
    TORCH_CHECK(q.stride(2) == kRow, "Q head stride must be 512 e4m3 bytes + an aligned 16-byte scale slot");

    c10::cuda::CUDAGuard guard(q.device());
    TORCH_CHECK(at::cuda::getCurrentDeviceProperties()->major == 10, "Dual MXFP8 head64 decode requires SM100f.");
    const auto opts = q.options();
    const auto stream = at::cuda::getCurrentCUDAStream();
    at::Tensor out = at::empty({b, s_q, h_q, kDim}, opts.dtype(at::kBFloat16));
    at::Tensor lse = at::empty({b, s_q, h_q}, opts.dtype(at::kFloat));
    const int parts = mxdsa_num_sm_parts(q.get_device(), (int)s_q);
    TORCH_CHECK(parts > 0, "could not query the device");
    if (!tile_scheduler_metadata.has_value()) {
        tile_scheduler_metadata = at::empty({parts, MXDSA_SCHED_META_INTS}, opts.dtype(at::kInt));
        num_splits = at::empty({b + 1}, opts.dtype(at::kInt));
        mxdsa_sched_params sp{};
        sp.b = (int32_t)b;
        sp.s_q = (int32_t)s_q;
        sp.topk = (int32_t)topk;
        sp.extra_topk = (int32_t)extra_topk;
        sp.topk_length = opt_ptr<int32_t>(topk_length);
        sp.extra_topk_length = opt_ptr<int32_t>(extra_topk_length);
        sp.num_sm_parts = parts;
        sp.sched_meta = tile_scheduler_metadata->data_ptr<int32_t>();
        sp.num_splits = num_splits->data_ptr<int32_t>();
        sp.stream = stream.stream();
        require_status(whole ? mxdsa_decode_sched_whole(&sp) : mxdsa_decode_sched(&sp), "mxdsa_decode_sched");
    }
    check_optional(tile_scheduler_metadata, "tile_scheduler_metadata", at::kInt, {parts, MXDSA_SCHED_META_INTS});
    TORCH_CHECK(num_splits.has_value(), "num_splits must be provided with tile_scheduler_metadata");
    check_optional(num_splits, "num_splits", at::kInt, {b + 1});
    TORCH_CHECK(tile_scheduler_metadata->is_contiguous() && num_splits->is_contiguous(),
                "scheduling tensors must be contiguous");

    // whole-request schedules need no partials, hence no scratch
    const size_t ws_bytes = whole ? 0 : mxdsa_decode_workspace_bytes((int)b, (int)s_q, parts);
    at::Tensor workspace = at::empty({(int64_t)ws_bytes}, opts.dtype(at::kByte));
    p.b = (int32_t)b;
    p.s_q = (int32_t)s_q;
    p.topk = (int32_t)topk;
    p.extra_topk = (int32_t)extra_topk;
    p.sm_scale = (float)sm_scale;
    p.q = q.data_ptr();
    p.stride_q_b = q.stride(0);
    p.stride_q_s = q.stride(1);
    p.kv = kv.data_ptr();
    p.num_blocks = (int32_t)num_blocks;
    p.page_block_size = (int32_t)page;
    p.stride_kv_block = kv.stride(0);
    p.indices = indices.data_ptr<int32_t>();
    p.stride_indices_b = indices.stride(0);
    p.stride_indices_s = indices.stride(1);
    p.topk_length = opt_ptr<int32_t>(topk_length);
    p.attn_sink = opt_ptr<float>(attn_sink);
    if (have_extra) {
        p.extra_kv = extra_kv->data_ptr();
        p.extra_num_blocks = (int32_t)extra_kv->size(0);
        p.extra_page_block_size = (int32_t)extra_kv->size(1);
        p.stride_extra_kv_block = extra_kv->stride(0);
        p.extra_indices = extra_indices->data_ptr<int32_t>();
        p.stride_extra_indices_b = extra_indices->stride(0);
        p.stride_extra_indices_s = extra_indices->stride(1);
        p.extra_topk_length = opt_ptr<int32_t>(extra_topk_length);
    }
    p.out = out.data_ptr();
    p.lse = lse.data_ptr<float>();
    p.sched_meta = tile_scheduler_metadata->data_ptr<int32_t>();
    p.num_splits = num_splits->data_ptr<int32_t>();
    p.num_sm_parts = parts;
    p.workspace = whole ? nullptr : workspace.data_ptr();
    p.workspace_bytes = ws_bytes;
    p.stream = stream.stream();
    if (whole) {
        require_status(mxdsa_decode_fwd_nocombine(&p), "mxdsa_decode_fwd_nocombine");
    } else {
        require_status(mxdsa_decode_fwd(&p), "mxdsa_decode_fwd");
        // the scratch is read by kernels queued on this stream after this function has returned
        c10::cuda::CUDACachingAllocator::recordStream(workspace.storage().data_ptr(), stream);
    }
    return {out, lse.transpose(1, 2), tile_scheduler_metadata, num_splits};
}

std::tuple<at::Tensor, at::Tensor, OptTensor, OptTensor> decode_fwd(
    const at::Tensor& q, const at::Tensor& kv, const at::Tensor& indices, const OptTensor& topk_length,
    const OptTensor& attn_sink, OptTensor tile_scheduler_metadata, OptTensor num_splits, const OptTensor& extra_kv,
    const OptTensor& extra_indices, const OptTensor& extra_topk_length, int64_t d_qk, int64_t d_v, double sm_scale,
    const std::vector<uint32_t>& w1, const std::vector<uint32_t>& w2) {
    return decode_impl(q, kv, indices, topk_length, attn_sink, std::move(tile_scheduler_metadata), std::move(num_splits),
                       extra_kv, extra_indices, extra_topk_length, d_qk, d_v, sm_scale, w1, w2, false);
}
std::tuple<at::Tensor, at::Tensor, OptTensor, OptTensor> decode_fwd_whole(
    const at::Tensor& q, const at::Tensor& kv, const at::Tensor& indices, const OptTensor& topk_length,
    const OptTensor& attn_sink, OptTensor tile_scheduler_metadata, OptTensor num_splits, const OptTensor& extra_kv,
    const OptTensor& extra_indices, const OptTensor& extra_topk_length, int64_t d_qk, int64_t d_v, double sm_scale,
    const std::vector<uint32_t>& w1, const std::vector<uint32_t>& w2) {
    return decode_impl(q, kv, indices, topk_length, attn_sink, std::move(tile_scheduler_metadata), std::move(num_splits),
                       extra_kv, extra_indices, extra_topk_length, d_qk, d_v, sm_scale, w1, w2, true);
}

void device_fault() {
    require_status(mxdsa_device_fault(at::cuda::getCurrentCUDAStream().stream()), "device check");
}

}  // namespace

static void define_module(pybind11::module_& m) {
    m.def("dual_mxfp8_head64_sparse_prefill_fwd", &prefill_fwd);
    m.def("dual_mxfp8_head64_sparse_prefill_fwd_ex", &prefill_fwd_ex);
    m.def("dual_mxfp8_sparse_decode_fwd", &decode_fwd);
    m.def("dual_mxfp8_sparse_decode_fwd_whole", &decode_fwd_whole);
    m.def("device_fault", &device_fault);
}

// Two import names for the same shared object: `mxdsa_ext` is the reference's module name (drop-in
// for callers that load the file by path under that name); `mxdsa_b200_ext` is what the Python
// package uses, so that it can live in one process with the reference's own extension.
PYBIND11_MODULE(mxdsa_ext, m) { define_module(m); }
PYBIND11_MODULE(mxdsa_b200_ext, m) { define_module(m); }

// PyTorch operator library `torch.ops.gpuk.*` over the C ABI of include/gpuk_b200.h.
//
// The schema strings are those of the reference's src/register.cpp:5-40, so code written
// against the reference's operator API runs unchanged.  This layer only unwraps tensors:
// checks (contiguity as in src/ops/all_reduce_fusion.cpp:341,366-367), device guard, current
// stream (src/ops/ops.h:15), dtype code -- and turns a non-zero status into an exception.
// The four fused_*rope* operators of register.cpp:42-63 are a different op family and are
// not provided.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>
#include <torch/library.h>

#include <cstring>
#include <stdexcept>
#include <vector>

#include "gpuk_b200.h"

using at::Tensor;
using fptr_t = int64_t;   // src/ops/ops.h:20-21: the workspace travels through Python as an int64

namespace {

gpuk_ws *ws_of(fptr_t fptr) {
    TORCH_CHECK(fptr != 0, "gpuk: null workspace handle");
    return reinterpret_cast<gpuk_ws *>(fptr);
}

void check(int status, const char *what) {
    TORCH_CHECK(status == GPUK_OK, "gpuk::", what, ": ", gpuk_status_string(status), ": ", gpuk_last_error());
}

int dtype_code(const Tensor &t) {
    switch (t.scalar_type()) {
    case at::kBFloat16: return GPUK_DTYPE_BF16;
    case at::kHalf: return GPUK_DTYPE_F16;
    case at::kFloat: return GPUK_DTYPE_F32;
    default: TORCH_CHECK(false, "gpuk: unsupported dtype ", t.scalar_type(), " (bfloat16, float16 and float32 are built)");
    }
    return -1;
}

Tensor handle_tensor(const uint8_t *bytes) {
    auto t = at::empty({GPUK_IPC_HANDLE_BYTES}, at::TensorOptions().dtype(at::kByte).device(at::kCPU));
    std::memcpy(t.data_ptr(), bytes, GPUK_IPC_HANDLE_BYTES);
    return t;
}

std::vector<uint8_t> pack_handles(const std::vector<Tensor> &handles) {
    std::vector<uint8_t> flat(handles.size() * GPUK_IPC_HANDLE_BYTES);
    for (size_t i = 0; i < handles.size(); ++i) {
        const Tensor h = handles[i].contiguous().cpu();
        TORCH_CHECK(h.numel() * h.element_size() == GPUK_IPC_HANDLE_BYTES, "gpuk: IPC handle ", i, " is not 64 bytes");
        std::memcpy(flat.data() + i * GPUK_IPC_HANDLE_BYTES, h.data_ptr(), GPUK_IPC_HANDLE_BYTES);
    }
    return flat;
}

fptr_t init_ar_fusion(int64_t device_id, int64_t rank, int64_t world_size, int64_t max_size_in_bytes,
                      int64_t comm_ptrs_buf_len) {
    gpuk_ws *ws = nullptr;
    int rc = gpuk_ws_create(static_cast<int>(device_id), static_cast<int>(rank), static_cast<int>(world_size),
                            max_size_in_bytes, comm_ptrs_buf_len, &ws);
    if (rc == GPUK_ERR_INVALID_ARGUMENT) throw std::invalid_argument(gpuk_last_error());   // all_reduce_fusion.cpp:263,266
    check(rc, "init_ar_fusion");
    return reinterpret_cast<fptr_t>(ws);
}

void destroy_ar_fusion(fptr_t fptr) { gpuk_ws_destroy(reinterpret_cast<gpuk_ws *>(fptr)); }

Tensor get_ar_fusion_barrier_handle(fptr_t fptr) {
    uint8_t h[GPUK_IPC_HANDLE_BYTES];
    check(gpuk_ws_get_barrier_handle(ws_of(fptr), h), "get_ar_fusion_barrier_handle");
    return handle_tensor(h);
}

Tensor get_ar_fusion_data_handle(fptr_t fptr) {
    uint8_t h[GPUK_IPC_HANDLE_BYTES];
    check(gpuk_ws_get_data_handle(ws_of(fptr), h), "get_ar_fusion_data_handle");
    return handle_tensor(h);
}

void open_ar_fusion_barrier_handles(fptr_t fptr, std::vector<Tensor> handles) {
    auto flat = pack_handles(handles);
    check(gpuk_ws_open_barrier_handles(ws_of(fptr), flat.data(), static_cast<int>(handles.size())),
          "open_ar_fusion_barrier_handles");
}

void open_ar_fusion_data_handles(fptr_t fptr, std::vector<Tensor> handles) {
    auto flat = pack_handles(handles);
    check(gpuk_ws_open_data_handles(ws_of(fptr), flat.data(), static_cast<int>(handles.size())),
          "open_ar_fusion_data_handles");
}

void ar_fusion_capture_clear(fptr_t fptr) { check(gpuk_ws_capture_clear(ws_of(fptr)), "ar_fusion_capture_clear"); }

Tensor get_ar_fusion_tensor_handle(fptr_t fptr, Tensor &input) {
    (void)ws_of(fptr);
    uint8_t h[GPUK_IPC_HANDLE_BYTES];
    c10::cuda::CUDAGuard guard(input.device());
    check(gpuk_tensor_ipc_handle(input.data_ptr(), h), "get_ar_fusion_tensor_handle");
    return handle_tensor(h);
}

int64_t get_ar_fusion_tensor_offset(fptr_t fptr, Tensor &input) {
    (void)ws_of(fptr);
    int64_t off = 0;
    c10::cuda::CUDAGuard guard(input.device());
    check(gpuk_tensor_ipc_offset(input.data_ptr(), &off), "get_ar_fusion_tensor_offset");
    return off;
}

std::vector<Tensor> get_ar_fusion_captured_handles(fptr_t fptr) {
    int n = 0;
    check(gpuk_ws_captured_count(ws_of(fptr), &n), "get_ar_fusion_captured_handles");
    return {};   // captured calls need no registration: peers never read an input tensor
}

Tensor get_ar_fusion_captured_offsets(fptr_t fptr) {
    int n = 0;
    check(gpuk_ws_captured_count(ws_of(fptr), &n), "get_ar_fusion_captured_offsets");
    return at::empty({0}, at::TensorOptions().dtype(at::kLong).device(at::kCPU));
}

void open_ar_fusion_captured_handles(fptr_t fptr, std::vector<Tensor> handles, std::vector<int64_t> offsets,
                                     int64_t ptr_idx) {
    auto flat = pack_handles(handles);
    check(gpuk_ws_open_captured_handles(ws_of(fptr), flat.data(), offsets.data(), static_cast<int>(handles.size()), ptr_idx),
          "open_ar_fusion_captured_handles");
}

void allreduce_inplace(fptr_t fptr, Tensor &input) {
    TORCH_CHECK(input.is_contiguous());
    c10::cuda::CUDAGuard guard(input.device());
    auto stream = at::cuda::getCurrentCUDAStream();
    check(gpuk_allreduce_inplace(ws_of(fptr), input.data_ptr(), input.numel(), dtype_code(input), stream.stream()),
          "allreduce_inplace");
}

void allreduce_rms(fptr_t fptr, Tensor &allreduce_in, Tensor &residual_in, Tensor &rms_gamma, Tensor &residual_out,
                   Tensor &norm_out, Tensor &scale_out, double eps, int64_t quant_type) {
    TORCH_CHECK(allreduce_in.is_contiguous() && residual_in.is_contiguous() && rms_gamma.is_contiguous());
    TORCH_CHECK(residual_out.is_contiguous() && norm_out.is_contiguous() && scale_out.is_contiguous());
    TORCH_CHECK(allreduce_in.dim() >= 1, "gpuk: allreduce_in needs a hidden dimension");
    TORCH_CHECK(residual_in.scalar_type() == allreduce_in.scalar_type() && rms_gamma.scalar_type() == allreduce_in.scalar_type() &&
                    residual_out.scalar_type() == allreduce_in.scalar_type(),
                "gpuk: residual, gamma and residual_out must have the dtype of allreduce_in");
    TORCH_CHECK(scale_out.scalar_type() == at::kFloat, "gpuk: scale_out must be float32");
    const int64_t numel = allreduce_in.numel();
    const int64_t hidden = allreduce_in.size(-1);
    TORCH_CHECK(residual_in.numel() == numel && residual_out.numel() == numel && norm_out.numel() == numel &&
                    rms_gamma.numel() == hidden,
                "gpuk: tensor sizes do not match allreduce_in");
    if (quant_type == GPUK_QUANT_NONE) {
        TORCH_CHECK(norm_out.scalar_type() == allreduce_in.scalar_type(), "gpuk: norm_out must have the input dtype without quantisation");
    } else {
        TORCH_CHECK(norm_out.element_size() == 1, "gpuk: norm_out must be an 8-bit tensor with quantisation");
        const int64_t need = quant_type == GPUK_QUANT_FP8_E4M3FN_448_STATIC ? 1 : (hidden ? numel / hidden : 0);
        TORCH_CHECK(scale_out.numel() >= need, "gpuk: scale_out has ", scale_out.numel(), " elements, needs ", need);
    }
    c10::cuda::CUDAGuard guard(allreduce_in.device());
    auto stream = at::cuda::getCurrentCUDAStream();
    int rc;
    if (fptr == 0) {
        // a group of one has no workspace: the no-communication kernel
        rc = gpuk_residual_rms_quant(allreduce_in.data_ptr(), residual_in.data_ptr(), rms_gamma.data_ptr(),
                                     residual_out.data_ptr(), norm_out.data_ptr(), scale_out.data_ptr<float>(), numel,
                                     static_cast<int>(hidden), dtype_code(allreduce_in), static_cast<float>(eps),
                                     static_cast<int>(quant_type), stream.stream());
    } else {
        rc = gpuk_allreduce_rms(ws_of(fptr), allreduce_in.data_ptr(), residual_in.data_ptr(), rms_gamma.data_ptr(),
                                residual_out.data_ptr(), norm_out.data_ptr(), scale_out.data_ptr<float>(), numel,
                                static_cast<int>(hidden), dtype_code(allreduce_in), static_cast<float>(eps),
                                static_cast<int>(quant_type), stream.stream());
    }
    check(rc, "allreduce_rms");
}

}  // namespace

TORCH_LIBRARY(gpuk, m) {
    m.def("init_ar_fusion(SymInt device_id, SymInt rank, SymInt world_size, SymInt max_size_in_bytes, SymInt comm_ptrs_buf_len) -> int");
    m.impl("init_ar_fusion", &init_ar_fusion);
    m.def("destroy_ar_fusion(SymInt fptr) -> ()");
    m.impl("destroy_ar_fusion", &destroy_ar_fusion);

    m.def("get_ar_fusion_barrier_handle(SymInt fptr) -> Tensor");
    m.impl("get_ar_fusion_barrier_handle", &get_ar_fusion_barrier_handle);
    m.def("get_ar_fusion_data_handle(SymInt fptr) -> Tensor");
    m.impl("get_ar_fusion_data_handle", &get_ar_fusion_data_handle);

    m.def("open_ar_fusion_barrier_handles(SymInt fptr, Tensor[] handles) -> ()");
    m.impl("open_ar_fusion_barrier_handles", &open_ar_fusion_barrier_handles);
    m.def("open_ar_fusion_data_handles(SymInt fptr, Tensor[] handles) -> ()");
    m.impl("open_ar_fusion_data_handles", &open_ar_fusion_data_handles);

    m.def("ar_fusion_capture_clear(SymInt fptr) -> ()");
    m.impl("ar_fusion_capture_clear", &ar_fusion_capture_clear);

    m.def("get_ar_fusion_tensor_handle(SymInt fptr, Tensor input) -> Tensor");
    m.impl("get_ar_fusion_tensor_handle", &get_ar_fusion_tensor_handle);
    m.def("get_ar_fusion_tensor_offset(SymInt fptr, Tensor input) -> int");
    m.impl("get_ar_fusion_tensor_offset", &get_ar_fusion_tensor_offset);

    m.def("get_ar_fusion_captured_handles(SymInt fptr) -> Tensor[]");
    m.impl("get_ar_fusion_captured_handles", &get_ar_fusion_captured_handles);
    m.def("get_ar_fusion_captured_offsets(SymInt fptr) -> Tensor");
    m.impl("get_ar_fusion_captured_offsets", &get_ar_fusion_captured_offsets);
    m.def("open_ar_fusion_captured_handles(SymInt fptr, Tensor[] handles, int[] offsets, SymInt ptr_idx) -> ()");
    m.impl("open_ar_fusion_captured_handles", &open_ar_fusion_captured_handles);

    m.def("allreduce_inplace(SymInt fptr, Tensor input) -> ()");
    m.impl("allreduce_inplace", c10::kCUDA, &allreduce_inplace);
    m.def("allreduce_rms(SymInt fptr, Tensor allreduce_in, "
          "Tensor residual_in, Tensor rms_gamma, Tensor residual_out, Tensor "
          "norm_out, Tensor scale_out, float eps, SymInt quant_type) -> ()");
    m.impl("allreduce_rms", c10::kCUDA, &allreduce_rms);
}

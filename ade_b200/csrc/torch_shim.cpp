// Thin torch binding of the two hot entry points of the C ABI (include/ade_b200.h): tensors in, tensor out, the
// output allocated from torch's caching allocator, the launch on torch's current stream.  It plays the role of the
// pybind launchers the reference builds with load_inline (run_ab / ade_recon_int4, src/kernels.py:383-397, 935-966),
// but contains no kernel: everything it does is fill an ade_delta_t and call libade_b200.so.
//
//   torch.ops.ade_b200.factored(x, weight?, y_dense?, uq, vq, vt, us, uz, vs, vz, M, N, r, blocks, scratch) -> out
//   torch.ops.ade_b200.recon(base, uq, vq, vt, us, uz, vs, vz, M, N, r, dbg_acc?, status?, u8?, v8?) -> merged
//   torch.ops.ade_b200.expand(uq, vq, vt, us, uz, vs, vz, M, N, r) -> (u8, v8)
//
// Built with the host compiler only (no nvcc): `python -m ade_b200.build`.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include "../../include/ade_b200.h"

namespace {

const char* err_name(int rc) {
    switch (rc) {
        case ADE_ERR_NULL: return "ADE_ERR_NULL: a required pointer is NULL";
        case ADE_ERR_SHAPE: return "ADE_ERR_SHAPE: a dimension is outside the supported set";
        case ADE_ERR_ALIGN: return "ADE_ERR_ALIGN: a pointer is not 16-byte aligned";
        case ADE_ERR_SCRATCH: return "ADE_ERR_SCRATCH: scratch buffer too small";
        case ADE_ERR_CUDA: return "ADE_ERR_CUDA: a CUDA runtime call failed";
        case ADE_ERR_DEVICE: return "ADE_ERR_DEVICE: the current device is not compute capability 10.x";
        default: return "unknown status";
    }
}

void check_stored(const at::Tensor& t, const char* name, const at::Tensor& like) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.device() == like.device(), "stored form tensor ", name,
                " must be a contiguous CUDA tensor on the device of the activations");
}

ade_delta_t make_delta(const at::Tensor& uq, const at::Tensor& vq, const at::Tensor& vt, const at::Tensor& us, const at::Tensor& uz,
                       const at::Tensor& vs, const at::Tensor& vz, int64_t M, int64_t N, int64_t r, at::IntArrayRef blocks,
                       const at::Tensor& like) {
    check_stored(uq, "uq", like);
    check_stored(vq, "vq", like);
    check_stored(vt, "vt", like);
    check_stored(us, "us", like);
    check_stored(uz, "uz", like);
    check_stored(vs, "vs", like);
    check_stored(vz, "vz", like);
    ade_delta_t d = {};
    d.uq = static_cast<const uint8_t*>(uq.data_ptr());
    d.vq = static_cast<const uint8_t*>(vq.data_ptr());
    d.vt = static_cast<const uint8_t*>(vt.data_ptr());
    d.us = static_cast<const uint16_t*>(us.data_ptr());
    d.uz = static_cast<const uint8_t*>(uz.data_ptr());
    d.vs = static_cast<const uint16_t*>(vs.data_ptr());
    d.vz = static_cast<const uint8_t*>(vz.data_ptr());
    d.M = static_cast<int>(M);
    d.N = static_cast<int>(N);
    d.r = static_cast<int>(r);
    // blocks: (row_begin, group_begin) pairs of a block-diagonal U^, closed by (M, ng); empty = dense
    TORCH_CHECK(blocks.size() % 2 == 0 && blocks.size() <= 2 * (ADE_B200_MAX_BLOCKS + 1), "blocks: at most ", ADE_B200_MAX_BLOCKS,
                " (row, group) pairs plus the closing one");
    if (!blocks.empty()) {
        d.n_blocks = static_cast<int>(blocks.size() / 2) - 1;
        for (size_t i = 0; i < blocks.size() / 2; ++i) {
            d.block_rows[i] = static_cast<int>(blocks[2 * i]);
            d.block_groups[i] = static_cast<int>(blocks[2 * i + 1]);
        }
    }
    return d;
}

at::Tensor factored(const at::Tensor& x, const c10::optional<at::Tensor>& weight, const c10::optional<at::Tensor>& y_dense,
                    const at::Tensor& uq, const at::Tensor& vq, const at::Tensor& vt, const at::Tensor& us, const at::Tensor& uz,
                    const at::Tensor& vs, const at::Tensor& vz, int64_t M, int64_t N, int64_t r, at::IntArrayRef blocks,
                    const at::Tensor& scratch) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous() && x.size(1) == N,
                "x must be a contiguous CUDA bfloat16 tensor of shape (T, ", N, ")");
    TORCH_CHECK(weight.has_value() != y_dense.has_value(), "give exactly one of weight (fused base GEMM) or y_dense");
    const int64_t T = x.size(0);
    if (weight.has_value())
        TORCH_CHECK(weight->scalar_type() == at::kBFloat16 && weight->is_contiguous() && weight->dim() == 2 && weight->size(0) == M &&
                        weight->size(1) == N && weight->device() == x.device(),
                    "weight must be a contiguous bfloat16 (d_o, d_i) tensor on x's device");
    if (y_dense.has_value())
        TORCH_CHECK(y_dense->scalar_type() == at::kBFloat16 && y_dense->is_contiguous() && y_dense->dim() == 2 && y_dense->size(0) == T &&
                        y_dense->size(1) == M && y_dense->device() == x.device(),
                    "y_dense must be a contiguous bfloat16 (T, d_o) tensor on x's device");
    TORCH_CHECK(scratch.is_cuda() && scratch.device() == x.device() && scratch.is_contiguous(), "scratch must be a CUDA buffer on x's device");
    const c10::cuda::CUDAGuard guard(x.device());
    const ade_delta_t d = make_delta(uq, vq, vt, us, uz, vs, vz, M, N, r, blocks, x);
    at::Tensor out = at::empty({T, M}, x.options());
    const int rc = ade_b200_factored(&d, x.data_ptr(), y_dense.has_value() ? y_dense->data_ptr() : nullptr,
                                     weight.has_value() ? weight->data_ptr() : nullptr, out.data_ptr(), scratch.data_ptr(),
                                     static_cast<size_t>(scratch.nbytes()), static_cast<int>(T),
                                     c10::cuda::getCurrentCUDAStream(x.get_device()).stream());
    TORCH_CHECK(rc == ADE_OK, "ade_b200_factored: ", err_name(rc), rc == ADE_ERR_CUDA ? " (cudaError " : "",
                rc == ADE_ERR_CUDA ? std::to_string(ade_b200_last_cuda_error()) + ")" : std::string());
    return out;
}

at::Tensor recon(const at::Tensor& base, const at::Tensor& uq, const at::Tensor& vq, const at::Tensor& vt, const at::Tensor& us,
                 const at::Tensor& uz, const at::Tensor& vs, const at::Tensor& vz, int64_t M, int64_t N, int64_t r,
                 const c10::optional<at::Tensor>& dbg_acc, const c10::optional<at::Tensor>& status,
                 const c10::optional<at::Tensor>& u8, const c10::optional<at::Tensor>& v8) {
    TORCH_CHECK(u8.has_value() == v8.has_value(), "u8 and v8 come together");
    if (u8.has_value())
        TORCH_CHECK(u8->scalar_type() == at::kChar && v8->scalar_type() == at::kChar && u8->is_contiguous() && v8->is_contiguous() &&
                        u8->dim() == 2 && v8->dim() == 2 && u8->size(0) == M && u8->size(1) == r && v8->size(0) == N && v8->size(1) == r &&
                        u8->device() == base.device() && v8->device() == base.device(),
                    "expanded operands must be contiguous int8 (d_o, r) and (d_i, r) tensors on the device of base");
    TORCH_CHECK(base.is_cuda() && base.scalar_type() == at::kBFloat16 && base.dim() == 2 && base.size(0) == M && base.size(1) == N,
                "base must be a CUDA bfloat16 (", M, ", ", N, ") tensor");
    const at::Tensor b = base.contiguous();
    if (dbg_acc.has_value())
        TORCH_CHECK(dbg_acc->scalar_type() == at::kInt && dbg_acc->is_contiguous() && dbg_acc->dim() == 3 && dbg_acc->size(0) == r / 128 &&
                        dbg_acc->size(1) == M && dbg_acc->size(2) == N && dbg_acc->device() == base.device(),
                    "dbg_acc must be a contiguous int32 (ng, d_o, d_i) tensor");
    if (status.has_value())
        TORCH_CHECK(status->scalar_type() == at::kInt && status->numel() >= 1 && status->device() == base.device(),
                    "status must be an int32 tensor on the device of base");
    const c10::cuda::CUDAGuard guard(base.device());
    const ade_delta_t d = make_delta(uq, vq, vt, us, uz, vs, vz, M, N, r, {}, base);
    at::Tensor out = at::empty_like(b);
    int32_t* dbg = dbg_acc.has_value() ? static_cast<int32_t*>(dbg_acc->data_ptr()) : nullptr;
    int* st = status.has_value() ? static_cast<int*>(status->data_ptr()) : nullptr;
    void* stream = c10::cuda::getCurrentCUDAStream(base.get_device()).stream();
    const int rc = u8.has_value() ? ade_b200_recon_expanded(&d, u8->data_ptr(), v8->data_ptr(), b.data_ptr(), out.data_ptr(), dbg, st, stream)
                                  : ade_b200_recon(&d, b.data_ptr(), out.data_ptr(), dbg, st, stream);
    TORCH_CHECK(rc == ADE_OK, "ade_b200_recon: ", err_name(rc), rc == ADE_ERR_CUDA ? " (cudaError " : "",
                rc == ADE_ERR_CUDA ? std::to_string(ade_b200_last_cuda_error()) + ")" : std::string());
    return out;
}

// int8 operands (code minus zero-point) of a stored form, for recon(..., u8, v8)
std::tuple<at::Tensor, at::Tensor> expand(const at::Tensor& uq, const at::Tensor& vq, const at::Tensor& vt, const at::Tensor& us,
                                          const at::Tensor& uz, const at::Tensor& vs, const at::Tensor& vz, int64_t M, int64_t N, int64_t r) {
    TORCH_CHECK(uq.is_cuda(), "stored form must be on a CUDA device");
    const c10::cuda::CUDAGuard guard(uq.device());
    const ade_delta_t d = make_delta(uq, vq, vt, us, uz, vs, vz, M, N, r, {}, uq);
    at::Tensor u8 = at::empty({M, r}, uq.options().dtype(at::kChar));
    at::Tensor v8 = at::empty({N, r}, uq.options().dtype(at::kChar));
    const int rc = ade_b200_expand_codes(&d, u8.data_ptr(), v8.data_ptr(), c10::cuda::getCurrentCUDAStream(uq.get_device()).stream());
    TORCH_CHECK(rc == ADE_OK, "ade_b200_expand_codes: ", err_name(rc), rc == ADE_ERR_CUDA ? " (cudaError " : "",
                rc == ADE_ERR_CUDA ? std::to_string(ade_b200_last_cuda_error()) + ")" : std::string());
    return {u8, v8};
}

}  // namespace

TORCH_LIBRARY(ade_b200, m) {
    m.def("factored(Tensor x, Tensor? weight, Tensor? y_dense, Tensor uq, Tensor vq, Tensor vt, Tensor us, Tensor uz, Tensor vs, Tensor vz, "
          "int M, int N, int r, int[] blocks, Tensor scratch) -> Tensor");
    m.def("recon(Tensor base, Tensor uq, Tensor vq, Tensor vt, Tensor us, Tensor uz, Tensor vs, Tensor vz, int M, int N, int r, "
          "Tensor? dbg_acc, Tensor? status, Tensor? u8, Tensor? v8) -> Tensor");
    m.def("expand(Tensor uq, Tensor vq, Tensor vt, Tensor us, Tensor uz, Tensor vs, Tensor vz, int M, int N, int r) -> (Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(ade_b200, CUDA, m) {
    m.impl("factored", &factored);
    m.impl("recon", &recon);
    m.impl("expand", &expand);
}

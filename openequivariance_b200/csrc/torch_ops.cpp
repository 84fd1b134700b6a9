// The six libtorch_tp_jit::jit_* operators registered from C++ on top of the C ABI of liboeq_b200.so.
//
// Counterpart of the reference's op layer (extension/torch_core.hpp:274-644: op bodies, check_tensor, output
// allocation, TORCH_LIBRARY schemas at :626-644; extension/libtorch_tp_jit.cpp:17-108: stream and registration glue).
// Same schemas, same argument checks with the same messages, outputs allocated with the inputs' options, launches on
// the current CUDA stream of the tensors' device.  Being registered in C++, the operators exist in any process that
// loads this library (an AOTInductor package run from C++ included) and a call costs a few microseconds of host time;
// the Python module openequivariance_b200/_torch/ops.py adds the fake, autograd and autocast registrations on top and
// carries an equivalent Python implementation for installations where this file was not built.
//
// Built by openequivariance_b200/build_native.py (g++ against the installed torch; links liboeq_b200.so).

#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <memory>
#include <mutex>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "../../include/oeq_b200.h"

namespace {

[[noreturn]] void refuse(const std::string& message) { TORCH_CHECK(false, message); }

struct Problem {
    std::string desc;
    oeqb_kernel_prop prop;
};

std::mutex g_mutex;
std::unordered_map<int64_t, std::shared_ptr<Problem>> g_problems;

// key -> descriptor text and properties; the tensor -> bytes copy happens once per key
std::shared_ptr<Problem> problem(const at::Tensor& json_bytes, int64_t key) {
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        auto it = g_problems.find(key);
        if (it != g_problems.end()) return it->second;
    }
    at::Tensor host = json_bytes.detach().to(at::kCPU).contiguous();
    if (host.scalar_type() != at::kByte) refuse("json_bytes must be a uint8 tensor");
    auto p = std::make_shared<Problem>();
    p->desc.assign(reinterpret_cast<const char*>(host.data_ptr<uint8_t>()), (size_t)host.numel());
    const int rc = oeqb_query(p->desc.data(), p->desc.size(), key, &p->prop);
    if (rc != 0) refuse("oeqb_query failed (code " + std::to_string(rc) + "): " + oeqb_last_error());
    std::lock_guard<std::mutex> lock(g_mutex);
    g_problems[key] = p;
    return p;
}

at::ScalarType torch_dtype(int e) {
    switch (e) {
        case 1: return at::kFloat;
        case 2: return at::kDouble;
        case 3: return at::kInt;
        case 4: return at::kLong;
        default: return at::kByte;
    }
}

// Messages are put together with std::string and std::to_string only: no iostream formatting in this library.
// (A shape message formatted through std::ostringstream crashed inside the stream's integer insertion on GPU machines,
// in processes where the CUDA driver's libraries were loaded, and only there; the cause was not found.)
std::string shape_str(const std::vector<int64_t>& s) {
    std::string o = "[";
    for (size_t i = 0; i < s.size(); ++i) o += (i ? ", " : "") + std::to_string(s[i]);
    return o + "]";
}



// Messages as in check_tensor (torch_core.hpp:109-134); -1 in `shape` accepts any extent.
void check(const at::Tensor& t, const std::vector<int64_t>& shape, at::ScalarType dt, const char* name) {
    const std::vector<int64_t> got = t.sizes().vec();
    bool ok = got.size() == shape.size();
    for (size_t i = 0; ok && i < shape.size(); ++i)
        if (shape[i] >= 0 && got[i] != shape[i]) ok = false;
    if (!ok) refuse(std::string("Shape mismatch for tensor '") + name + "'. Expected: " + shape_str(shape) + ". Got: " + shape_str(got));
#ifndef OEQB_TEST_ANY_DEVICE   // (a test build runs the argument checks on CPU tensors)
    if (!t.is_cuda()) refuse(std::string("Tensor '") + name + "' is not on the GPU.");
#endif
    if (t.scalar_type() != dt)
        refuse(std::string("Dtype mismatch for tensor '") + name + "'. Expected: " + c10::toString(dt) + ". Got: " +
               c10::toString(t.scalar_type()));
}

int64_t first_dim(const at::Tensor& t, const char* name) {
    if (t.dim() < 1)
        refuse(std::string("Shape mismatch for tensor '") + name + "'. Expected a leading batch dimension. Got: " +
               shape_str(t.sizes().vec()));
    return t.size(0);
}

const void* ptr(const at::Tensor& t) { return t.numel() > 0 ? t.data_ptr() : nullptr; }
void* mptr(at::Tensor& t) { return t.numel() > 0 ? t.data_ptr() : nullptr; }

void* current_stream(const at::Tensor& t) { return (void*)c10::cuda::getCurrentCUDAStream(t.device().index()).stream(); }

void done(int rc, const char* what) {
    if (rc != 0) refuse(std::string(what) + " failed (code " + std::to_string(rc) + "): " + oeqb_last_error());
}

int64_t tp_checks(const Problem& p, const at::Tensor& x, const at::Tensor& y, const at::Tensor& W) {
    const at::ScalarType dt = torch_dtype(p.prop.irrep_dtype);
    const int64_t B = first_dim(x, "L1_in");
    check(x, {B, p.prop.L1_dim}, dt, "L1_in");
    check(y, {B, p.prop.L2_dim}, dt, "L2_in");
    if (p.prop.shared_weights) check(W, {p.prop.weight_numel}, torch_dtype(p.prop.weight_dtype), "W");
    else check(W, {B, p.prop.weight_numel}, torch_dtype(p.prop.weight_dtype), "W");
    return B;
}

at::Tensor jit_tp_forward(const at::Tensor& json_bytes, int64_t hash, const at::Tensor& L1_in, const at::Tensor& L2_in,
                          const at::Tensor& W, int64_t L3_dim) {
    (void)L3_dim;
    auto p = problem(json_bytes, hash);
    const int64_t B = tp_checks(*p, L1_in, L2_in, W);
    at::Tensor x = L1_in.contiguous(), y = L2_in.contiguous(), w = W.contiguous();
    at::Tensor out = at::empty({B, p->prop.L3_dim}, x.options());
    c10::cuda::CUDAGuard guard(x.device());
    done(oeqb_tp_forward(p->desc.data(), p->desc.size(), hash, B, ptr(x), ptr(y), ptr(w), mptr(out), current_stream(x)),
         "jit_tp_forward");
    return out;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> jit_tp_backward(const at::Tensor& json_bytes, int64_t hash,
                                                               const at::Tensor& L1_in, const at::Tensor& L2_in,
                                                               const at::Tensor& W, const at::Tensor& L3_grad) {
    auto p = problem(json_bytes, hash);
    const int64_t B = tp_checks(*p, L1_in, L2_in, W);
    check(L3_grad, {B, p->prop.L3_dim}, torch_dtype(p->prop.irrep_dtype), "L3_grad");
    at::Tensor x = L1_in.contiguous(), y = L2_in.contiguous(), w = W.contiguous(), g = L3_grad.contiguous();
    at::Tensor dx = at::empty_like(x), dy = at::empty_like(y), dw = at::empty_like(w);
    c10::cuda::CUDAGuard guard(x.device());
    done(oeqb_tp_backward(p->desc.data(), p->desc.size(), hash, B, ptr(x), ptr(y), ptr(w), ptr(g), mptr(dx), mptr(dy), mptr(dw),
                          current_stream(x)),
         "jit_tp_backward");
    return {dx, dy, dw};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> jit_tp_double_backward(
    const at::Tensor& json_bytes, int64_t hash, const at::Tensor& L1_in, const at::Tensor& L2_in, const at::Tensor& W,
    const at::Tensor& L3_grad, const at::Tensor& L1_dgrad, const at::Tensor& L2_dgrad, const at::Tensor& W_dgrad) {
    auto p = problem(json_bytes, hash);
    const int64_t B = tp_checks(*p, L1_in, L2_in, W);
    const at::ScalarType dt = torch_dtype(p->prop.irrep_dtype);
    check(L3_grad, {B, p->prop.L3_dim}, dt, "L3_grad");
    check(L1_dgrad, {B, p->prop.L1_dim}, dt, "L1_dgrad");
    check(L2_dgrad, {B, p->prop.L2_dim}, dt, "L2_dgrad");
    check(W_dgrad, W.sizes().vec(), W.scalar_type(), "W_dgrad");
    at::Tensor x = L1_in.contiguous(), y = L2_in.contiguous(), w = W.contiguous(), g = L3_grad.contiguous();
    at::Tensor x2 = L1_dgrad.contiguous(), y2 = L2_dgrad.contiguous(), w2 = W_dgrad.contiguous();
    at::Tensor dx = at::empty_like(x), dy = at::empty_like(y), dw = at::empty_like(w), dg = at::empty_like(g);
    c10::cuda::CUDAGuard guard(x.device());
    done(oeqb_tp_double_backward(p->desc.data(), p->desc.size(), hash, B, ptr(x), ptr(y), ptr(w), ptr(g), ptr(x2), ptr(y2),
                                 ptr(w2), mptr(dx), mptr(dy), mptr(dw), mptr(dg), current_stream(x)),
         "jit_tp_double_backward");
    return {dx, dy, dw, dg};
}

struct ConvSizes { int64_t N, E; };

ConvSizes conv_checks(const Problem& p, const at::Tensor& x, const at::Tensor& y, const at::Tensor& W, const at::Tensor& rows,
                      const at::Tensor& cols, const at::Tensor& workspace, const at::Tensor& perm) {
    const at::ScalarType dt = torch_dtype(p.prop.irrep_dtype), it = torch_dtype(p.prop.idx_dtype);
    const int64_t N = first_dim(x, "L1_in"), E = first_dim(rows, "rows");
    check(x, {N, p.prop.L1_dim}, dt, "L1_in");
    check(y, {E, p.prop.L2_dim}, dt, "L2_in");
    if (p.prop.shared_weights) check(W, {p.prop.weight_numel}, torch_dtype(p.prop.weight_dtype), "W");
    else check(W, {E, p.prop.weight_numel}, torch_dtype(p.prop.weight_dtype), "W");
    check(rows, {E}, it, "rows");
    check(cols, {E}, it, "cols");
    if (p.prop.deterministic) check(perm, {E}, it, "transpose_perm");
    check(workspace, {-1}, at::kByte, "workspace");
    return {N, E};
}

// the caller's workspace when it is large enough, else a fresh one from torch's caching allocator
at::Tensor scratch(const Problem& p, int64_t key, int direction, ConvSizes s, const at::Tensor& workspace) {
    const int64_t need = oeqb_conv_workspace_bytes(p.desc.data(), p.desc.size(), key, direction, s.N, s.E);
    if (need < 0) refuse("oeqb_conv_workspace_bytes failed (code " + std::to_string(-need) + "): " + oeqb_last_error());
    if (workspace.numel() >= need) return workspace;
    return at::empty({need}, workspace.options());
}

at::Tensor jit_conv_forward(const at::Tensor& json_bytes, int64_t hash, const at::Tensor& L1_in, const at::Tensor& L2_in,
                            const at::Tensor& W, int64_t L3_dim, const at::Tensor& rows, const at::Tensor& cols,
                            const at::Tensor& workspace, const at::Tensor& transpose_perm) {
    (void)L3_dim;
    auto p = problem(json_bytes, hash);
    const ConvSizes s = conv_checks(*p, L1_in, L2_in, W, rows, cols, workspace, transpose_perm);
    at::Tensor x = L1_in.contiguous(), y = L2_in.contiguous(), w = W.contiguous();
    at::Tensor r = rows.contiguous(), c = cols.contiguous(), pm = transpose_perm.contiguous();
    at::Tensor out = at::empty({s.N, p->prop.L3_dim}, x.options());
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor ws = scratch(*p, hash, 0, s, workspace);
    done(oeqb_conv_forward(p->desc.data(), p->desc.size(), hash, s.N, s.E, ptr(x), ptr(y), ptr(w), mptr(out), ptr(r), ptr(c),
                           p->prop.deterministic ? ptr(pm) : nullptr, mptr(ws), ws.numel(), current_stream(x)),
         "jit_conv_forward");
    return out;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> jit_conv_backward(const at::Tensor& json_bytes, int64_t hash,
                                                                 const at::Tensor& L1_in, const at::Tensor& L2_in,
                                                                 const at::Tensor& W, const at::Tensor& L3_grad,
                                                                 const at::Tensor& rows, const at::Tensor& cols,
                                                                 const at::Tensor& workspace, const at::Tensor& transpose_perm) {
    auto p = problem(json_bytes, hash);
    const ConvSizes s = conv_checks(*p, L1_in, L2_in, W, rows, cols, workspace, transpose_perm);
    check(L3_grad, {s.N, p->prop.L3_dim}, torch_dtype(p->prop.irrep_dtype), "L3_grad");
    at::Tensor x = L1_in.contiguous(), y = L2_in.contiguous(), w = W.contiguous(), g = L3_grad.contiguous();
    at::Tensor r = rows.contiguous(), c = cols.contiguous(), pm = transpose_perm.contiguous();
    at::Tensor dx = at::empty_like(x), dy = at::empty_like(y), dw = at::empty_like(w);
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor ws = scratch(*p, hash, 1, s, workspace);
    done(oeqb_conv_backward(p->desc.data(), p->desc.size(), hash, s.N, s.E, ptr(x), ptr(y), ptr(w), ptr(g), mptr(dx), mptr(dy),
                            mptr(dw), ptr(r), ptr(c), p->prop.deterministic ? ptr(pm) : nullptr, mptr(ws), ws.numel(),
                            current_stream(x)),
         "jit_conv_backward");
    return {dx, dy, dw};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> jit_conv_double_backward(
    const at::Tensor& json_bytes, int64_t hash, const at::Tensor& L1_in, const at::Tensor& L2_in, const at::Tensor& W,
    const at::Tensor& L3_grad, const at::Tensor& L1_dgrad, const at::Tensor& L2_dgrad, const at::Tensor& W_dgrad,
    const at::Tensor& rows, const at::Tensor& cols, const at::Tensor& workspace, const at::Tensor& transpose_perm) {
    auto p = problem(json_bytes, hash);
    const ConvSizes s = conv_checks(*p, L1_in, L2_in, W, rows, cols, workspace, transpose_perm);
    const at::ScalarType dt = torch_dtype(p->prop.irrep_dtype);
    check(L3_grad, {s.N, p->prop.L3_dim}, dt, "L3_grad");
    check(L1_dgrad, {s.N, p->prop.L1_dim}, dt, "L1_dgrad");
    check(L2_dgrad, {s.E, p->prop.L2_dim}, dt, "L2_dgrad");
    check(W_dgrad, W.sizes().vec(), W.scalar_type(), "W_dgrad");
    at::Tensor x = L1_in.contiguous(), y = L2_in.contiguous(), w = W.contiguous(), g = L3_grad.contiguous();
    at::Tensor x2 = L1_dgrad.contiguous(), y2 = L2_dgrad.contiguous(), w2 = W_dgrad.contiguous();
    at::Tensor r = rows.contiguous(), c = cols.contiguous(), pm = transpose_perm.contiguous();
    at::Tensor dx = at::empty_like(x), dy = at::empty_like(y), dw = at::empty_like(w), dg = at::empty_like(g);
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor ws = scratch(*p, hash, 2, s, workspace);
    done(oeqb_conv_double_backward(p->desc.data(), p->desc.size(), hash, s.N, s.E, ptr(x), ptr(y), ptr(w), ptr(g), ptr(x2),
                                   ptr(y2), ptr(w2), mptr(dx), mptr(dy), mptr(dw), mptr(dg), ptr(r), ptr(c),
                                   p->prop.deterministic ? ptr(pm) : nullptr, mptr(ws), ws.numel(), current_stream(x)),
         "jit_conv_double_backward");
    return {dx, dy, dw, dg};
}

}  // namespace

TORCH_LIBRARY(libtorch_tp_jit, m) {
    m.def("jit_tp_forward(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, int L3_dim) -> Tensor");
    m.def("jit_tp_backward(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, Tensor L3_grad) -> (Tensor, Tensor, Tensor)");
    m.def("jit_tp_double_backward(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, Tensor L3_grad, Tensor L1_dgrad, Tensor L2_dgrad, Tensor W_dgrad) -> (Tensor, Tensor, Tensor, Tensor)");
    m.def("jit_conv_forward(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, int L3_dim, Tensor rows, Tensor cols, Tensor workspace, Tensor transpose_perm) -> Tensor");
    m.def("jit_conv_backward(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, Tensor L3_grad, Tensor rows, Tensor cols, Tensor workspace, Tensor transpose_perm) -> (Tensor, Tensor, Tensor)");
    m.def("jit_conv_double_backward(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, Tensor L3_grad, Tensor L1_dgrad, Tensor L2_dgrad, Tensor W_dgrad, Tensor rows, Tensor cols, Tensor workspace, Tensor transpose_perm) -> (Tensor, Tensor, Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(libtorch_tp_jit, CUDA, m) {
    m.impl("jit_tp_forward", &jit_tp_forward);
    m.impl("jit_tp_backward", &jit_tp_backward);
    m.impl("jit_tp_double_backward", &jit_tp_double_backward);
    m.impl("jit_conv_forward", &jit_conv_forward);
    m.impl("jit_conv_backward", &jit_conv_backward);
    m.impl("jit_conv_double_backward", &jit_conv_double_backward);
}

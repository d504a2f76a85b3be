// kernel_matmul_b200._C -- the thin PyTorch C++ extension over the C ABI of libkm_b200.so.
//
// One ahead-of-time module with the ten functions the reference reaches through its per-op
// pybind11 modules (native/<op>/<op>.cpp `call`, native/ranges/ranges.cpp:152-156), the kernel
// type passed as a runtime integer (KM_KERNEL_*) instead of a -DKM_KERNEL_* define.  Each
// function checks its arguments with the reference's messages (native/common/entrypoint.h:3-14),
// allocates outputs and workspaces through ATen on x1's device, and launches on the current
// PyTorch stream under a device guard with the GIL released.  No arithmetic happens here.
#include <torch/extension.h>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <vector>

#include "../../include/km_b200.h"

namespace {

void check_cuda(const torch::Tensor &x) { TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor"); }
void check_f32(const torch::Tensor &x) {
    check_cuda(x);
    TORCH_CHECK(x.scalar_type() == torch::kFloat32, "x must be float32");
}
void check_i32(const torch::Tensor &x) {
    check_cuda(x);
    TORCH_CHECK(x.scalar_type() == torch::kInt32, "x must be int32");
}

int num_params(int64_t kernel_type) {
    const int p = km_num_params((int)kernel_type);
    TORCH_CHECK(p > 0, "Unknown kernel type: ", kernel_type);
    return p;
}

// Broadcast the leading dims of all arguments to one batch shape and describe it for the C ABI.
struct Call {
    std::vector<int64_t> batch;
    km_batch kb{};
    std::vector<torch::Tensor> keep;  // expanded views (kept alive until the launch is queued)

    void add_batch(const torch::Tensor &t, int nonbatch) {
        TORCH_CHECK(t.dim() >= nonbatch, "tensor of rank ", t.dim(), " needs at least ", nonbatch, " trailing dims");
        std::vector<int64_t> lead(t.sizes().begin(), t.sizes().end() - nonbatch);
        batch = at::infer_size(batch, lead);
    }
    void finish() {
        TORCH_CHECK((int)batch.size() <= KM_MAX_BATCH_DIMS, "at most ", KM_MAX_BATCH_DIMS, " batch dims");
        kb.ndim = (int32_t)batch.size();
        for (size_t d = 0; d < batch.size(); d++) kb.size[d] = batch[d];
    }
    km_view view(const torch::Tensor &t, int nonbatch) {
        std::vector<int64_t> shape(batch);
        shape.insert(shape.end(), t.sizes().end() - nonbatch, t.sizes().end());
        torch::Tensor e = t.expand(shape);
        keep.push_back(e);
        km_view v{};
        v.data = e.data_ptr();
        const int nb = (int)batch.size();
        for (int d = 0; d < nb; d++) v.batch_stride[d] = e.stride(d);
        for (int d = 0; d < nonbatch; d++) v.stride[d] = e.stride(nb + d);
        return v;
    }
    std::vector<int64_t> out_shape(std::initializer_list<int64_t> tail) const {
        std::vector<int64_t> s(batch);
        s.insert(s.end(), tail.begin(), tail.end());
        return s;
    }
};

void *stream_of(const torch::Tensor &t) { return c10::cuda::getCurrentCUDAStream(t.device().index()).stream(); }

void raise_on(int rc) { TORCH_CHECK(rc == KM_OK, "[km status ", rc, "] ", km_last_error()); }

Call prep(int64_t kernel_type, const torch::Tensor &x1, const torch::Tensor &x2, const torch::Tensor &params,
          const torch::Tensor &start, const torch::Tensor &end, std::initializer_list<std::pair<torch::Tensor, int>> extra) {
    check_f32(x1), check_f32(x2), check_f32(params), check_i32(start), check_i32(end);
    const int P = num_params(kernel_type);
    TORCH_CHECK(params.size(-1) == P, "params must have ", P, " entries in the last dim");
    const int64_t R = (x1.size(-1) + KM_BLOCK_SIZE - 1) / KM_BLOCK_SIZE;
    TORCH_CHECK(start.size(-1) == R && end.size(-1) == R, "start/end must have ceil(m/128) = ", R, " entries");
    Call c;
    for (const torch::Tensor *t : {&x1, &x2, &params, &start, &end}) {
        TORCH_CHECK(t->device() == x1.device(), "all tensors must be on the same CUDA device");
        c.add_batch(*t, 1);
    }
    for (const auto &e : extra) {
        check_f32(e.first);
        TORCH_CHECK(e.first.device() == x1.device(), "all tensors must be on the same CUDA device");
        c.add_batch(e.first, e.second);
    }
    c.finish();
    return c;
}

torch::Tensor workspace(const torch::Tensor &like, size_t bytes) {
    return torch::empty({(int64_t)std::max<size_t>(bytes, 256)}, like.options().dtype(torch::kUInt8));
}

// matmul.call(x1, x2, rhs, params, start, end)  (native/matmul/matmul.cpp:6-17); tensor cores from 9
// columns on problems with at least 256 (batch, row block) items, as kernel_matmul_b200.ops.matmul.
torch::Tensor matmul(int64_t kernel_type, torch::Tensor x1, torch::Tensor x2, torch::Tensor rhs, torch::Tensor params,
                     torch::Tensor start, torch::Tensor end, bool tensor_cores_auto) {
    Call c = prep(kernel_type, x1, x2, params, start, end, {{rhs, 2}});
    const int64_t m = x1.size(-1), n = x2.size(-1), k = rhs.size(-1);
    TORCH_CHECK(rhs.size(-2) == n, "rhs must have n = ", n, " rows");
    const c10::cuda::CUDAGuard guard(x1.device());
    torch::Tensor out = torch::empty(c.out_shape({m, k}), x1.options());
    const km_view vx1 = c.view(x1, 1), vx2 = c.view(x2, 1), vr = c.view(rhs, 2), vp = c.view(params, 1),
                  vs = c.view(start, 1), ve = c.view(end, 1), vo = c.view(out, 2);
    int64_t items = (m + KM_BLOCK_SIZE - 1) / KM_BLOCK_SIZE;
    for (int64_t b : c.batch) items *= b;
    void *stream = stream_of(x1);
    if (tensor_cores_auto && k >= 9 && items >= 256) {
        const size_t bytes = km_matmul_tc_workspace_bytes(&c.kb, n, k, &vr);
        torch::Tensor ws = workspace(x1, bytes);
        void *wsp = ws.data_ptr();
        int rc;
        {
            pybind11::gil_scoped_release nogil;
            rc = km_matmul_tc_f32((int)kernel_type, &c.kb, m, n, k, &vx1, &vx2, &vr, &vp, &vs, &ve, &vo, wsp, bytes, stream);
        }
        raise_on(rc);
        return out;
    }
    int rc;
    {
        pybind11::gil_scoped_release nogil;
        rc = km_matmul_f32((int)kernel_type, &c.kb, m, n, k, &vx1, &vx2, &vr, &vp, &vs, &ve, &vo, stream);
    }
    raise_on(rc);
    return out;
}

// bilinear_derivative.call(x1, x2, left, right, params, start, end)
// (native/bilinear_derivative/bilinear_derivative.cpp:6-21)
torch::Tensor bilinear_derivative(int64_t kernel_type, torch::Tensor x1, torch::Tensor x2, torch::Tensor left,
                                  torch::Tensor right, torch::Tensor params, torch::Tensor start, torch::Tensor end) {
    Call c = prep(kernel_type, x1, x2, params, start, end, {{left, 2}, {right, 2}});
    const int64_t m = x1.size(-1), n = x2.size(-1), k = left.size(-1);
    TORCH_CHECK(left.size(-2) == m && right.size(-2) == n && right.size(-1) == k,
                "left must be (.., m, k) and right (.., n, k)");
    const c10::cuda::CUDAGuard guard(x1.device());
    torch::Tensor grad = torch::empty(c.out_shape({(int64_t)num_params(kernel_type)}), x1.options());
    const km_view vx1 = c.view(x1, 1), vx2 = c.view(x2, 1), vl = c.view(left, 2), vr = c.view(right, 2),
                  vp = c.view(params, 1), vs = c.view(start, 1), ve = c.view(end, 1), vg = c.view(grad, 1);
    const size_t bytes = km_grad_workspace_bytes((int)kernel_type, &c.kb, m);
    torch::Tensor ws = workspace(x1, bytes);
    void *wsp = ws.data_ptr(), *stream = stream_of(x1);
    int rc;
    {
        pybind11::gil_scoped_release nogil;
        rc = km_bilinear_derivative_f32((int)kernel_type, &c.kb, m, n, k, &vx1, &vx2, &vl, &vr, &vp, &vs, &ve, &vg, wsp,
                                        ws.numel(), stream);
    }
    raise_on(rc);
    return grad;
}

// matmul_bwd.call(x1, x2, rhs, params, start, end, out_grad)  (native/matmul_bwd/matmul_bwd.cpp:6-19)
torch::Tensor matmul_bwd(int64_t kernel_type, torch::Tensor x1, torch::Tensor x2, torch::Tensor rhs, torch::Tensor params,
                         torch::Tensor start, torch::Tensor end, torch::Tensor out_grad) {
    return bilinear_derivative(kernel_type, x1, x2, out_grad, rhs, params, start, end);
}

// dense.call(x1, x2, params, start, end)  (native/dense/dense.cpp:6-17)
torch::Tensor dense(int64_t kernel_type, torch::Tensor x1, torch::Tensor x2, torch::Tensor params, torch::Tensor start,
                    torch::Tensor end) {
    Call c = prep(kernel_type, x1, x2, params, start, end, {});
    const int64_t m = x1.size(-1), n = x2.size(-1);
    const c10::cuda::CUDAGuard guard(x1.device());
    torch::Tensor out = torch::empty(c.out_shape({m, n}), x1.options());
    const km_view vx1 = c.view(x1, 1), vx2 = c.view(x2, 1), vp = c.view(params, 1), vs = c.view(start, 1),
                  ve = c.view(end, 1), vo = c.view(out, 2);
    void *stream = stream_of(x1);
    int rc;
    {
        pybind11::gil_scoped_release nogil;
        rc = km_dense_f32((int)kernel_type, &c.kb, m, n, &vx1, &vx2, &vp, &vs, &ve, &vo, stream);
    }
    raise_on(rc);
    return out;
}

// dense_bwd.call(x1, x2, params, start, end, out_grad)  (native/dense_bwd/dense_bwd.cpp:6-17)
torch::Tensor dense_bwd(int64_t kernel_type, torch::Tensor x1, torch::Tensor x2, torch::Tensor params, torch::Tensor start,
                        torch::Tensor end, torch::Tensor out_grad) {
    Call c = prep(kernel_type, x1, x2, params, start, end, {{out_grad, 2}});
    const int64_t m = x1.size(-1), n = x2.size(-1);
    TORCH_CHECK(out_grad.size(-2) == m && out_grad.size(-1) == n, "out_grad must be (.., m, n)");
    const c10::cuda::CUDAGuard guard(x1.device());
    torch::Tensor grad = torch::empty(c.out_shape({(int64_t)num_params(kernel_type)}), x1.options());
    const km_view vx1 = c.view(x1, 1), vx2 = c.view(x2, 1), vp = c.view(params, 1), vs = c.view(start, 1),
                  ve = c.view(end, 1), vog = c.view(out_grad, 2), vg = c.view(grad, 1);
    const size_t bytes = km_grad_workspace_bytes((int)kernel_type, &c.kb, m);
    torch::Tensor ws = workspace(x1, bytes);
    void *wsp = ws.data_ptr(), *stream = stream_of(x1);
    int rc;
    {
        pybind11::gil_scoped_release nogil;
        rc = km_dense_bwd_f32((int)kernel_type, &c.kb, m, n, &vx1, &vx2, &vp, &vs, &ve, &vog, &vg, wsp, ws.numel(), stream);
    }
    raise_on(rc);
    return grad;
}

struct Lookups {
    std::vector<int64_t> shape;
    std::vector<torch::Tensor> flat;  // batch indices..., row, col: contiguous int32 of L entries
    const int32_t *bptr[KM_MAX_BATCH_DIMS] = {nullptr, nullptr, nullptr, nullptr};
    int64_t L = 0;
};

Lookups lookups(const Call &c, const std::vector<torch::Tensor> &batch_indices, const torch::Tensor &row,
                const torch::Tensor &col) {
    TORCH_CHECK(batch_indices.size() == c.batch.size(), "expected ", c.batch.size(), " batch index tensors, got ",
                batch_indices.size());
    Lookups l;
    l.shape = at::infer_size(row.sizes().vec(), col.sizes().vec());
    for (const auto &b : batch_indices) l.shape = at::infer_size(l.shape, b.sizes().vec());
    auto flat = [&](const torch::Tensor &t) {
        check_i32(t);
        return t.expand(l.shape).contiguous().reshape({-1});
    };
    for (const auto &b : batch_indices) l.flat.push_back(flat(b));
    l.flat.push_back(flat(row));
    l.flat.push_back(flat(col));
    for (size_t d = 0; d < batch_indices.size(); d++) l.bptr[d] = l.flat[d].data_ptr<int32_t>();
    l.L = l.flat.back().numel();
    return l;
}

// index.call(x1, x2, params, start, end, batch_indices, row_index, col_index)  (native/index/index.cpp:6-24)
torch::Tensor op_index(int64_t kernel_type, torch::Tensor x1, torch::Tensor x2, torch::Tensor params, torch::Tensor start,
                    torch::Tensor end, std::vector<torch::Tensor> batch_indices, torch::Tensor row_index,
                    torch::Tensor col_index) {
    Call c = prep(kernel_type, x1, x2, params, start, end, {});
    Lookups l = lookups(c, batch_indices, row_index, col_index);
    const c10::cuda::CUDAGuard guard(x1.device());
    torch::Tensor out = torch::empty({l.L}, x1.options());
    const km_view vx1 = c.view(x1, 1), vx2 = c.view(x2, 1), vp = c.view(params, 1), vs = c.view(start, 1), ve = c.view(end, 1);
    const int32_t *row = l.flat[l.flat.size() - 2].data_ptr<int32_t>(), *col = l.flat.back().data_ptr<int32_t>();
    float *outp = out.data_ptr<float>();
    void *stream = stream_of(x1);
    int rc;
    {
        pybind11::gil_scoped_release nogil;
        rc = km_index_f32((int)kernel_type, &c.kb, x1.size(-1), x2.size(-1), l.L, &vx1, &vx2, &vp, &vs, &ve, l.bptr, row, col,
                          outp, stream);
    }
    raise_on(rc);
    return out.reshape(l.shape);
}

// index_bwd.call(..., out_grad)  (native/index_bwd/index_bwd.cpp:6-27)
torch::Tensor op_index_bwd(int64_t kernel_type, torch::Tensor x1, torch::Tensor x2, torch::Tensor params, torch::Tensor start,
                        torch::Tensor end, std::vector<torch::Tensor> batch_indices, torch::Tensor row_index,
                        torch::Tensor col_index, torch::Tensor out_grad) {
    Call c = prep(kernel_type, x1, x2, params, start, end, {});
    Lookups l = lookups(c, batch_indices, row_index, col_index);
    check_f32(out_grad);
    const c10::cuda::CUDAGuard guard(x1.device());
    torch::Tensor og = out_grad.expand(l.shape).contiguous().reshape({-1});
    torch::Tensor grad = torch::empty(c.out_shape({(int64_t)num_params(kernel_type)}), x1.options());
    const km_view vx1 = c.view(x1, 1), vx2 = c.view(x2, 1), vp = c.view(params, 1), vs = c.view(start, 1),
                  ve = c.view(end, 1), vg = c.view(grad, 1);
    const size_t bytes = km_index_bwd_workspace_bytes((int)kernel_type, &c.kb);
    torch::Tensor ws = workspace(x1, bytes);
    const int32_t *row = l.flat[l.flat.size() - 2].data_ptr<int32_t>(), *col = l.flat.back().data_ptr<int32_t>();
    const float *ogp = og.data_ptr<float>();
    void *wsp = ws.data_ptr(), *stream = stream_of(x1);
    int rc;
    {
        pybind11::gil_scoped_release nogil;
        rc = km_index_bwd_f32((int)kernel_type, &c.kb, x1.size(-1), x2.size(-1), l.L, &vx1, &vx2, &vp, &vs, &ve, l.bptr, row,
                              col, ogp, &vg, wsp, ws.numel(), stream);
    }
    raise_on(rc);
    return grad;
}

// ranges.make_ranges(x1, x2, cutoff, block_size, align)  (native/ranges/ranges.cpp:8-62), on the device
std::tuple<torch::Tensor, torch::Tensor> make_ranges(torch::Tensor x1, torch::Tensor x2, double cutoff, int64_t block_size,
                                                     bool align) {
    check_f32(x1), check_f32(x2);
    TORCH_CHECK(x1.dim() == 2 && x2.dim() == 2 && x1.size(0) == x2.size(0), "x1 and x2 must be (B, m) and (B, n)");
    const c10::cuda::CUDAGuard guard(x1.device());
    torch::Tensor a = x1.contiguous(), b = x2.contiguous();
    const int64_t B = a.size(0), m = a.size(1), n = b.size(1), R = (m + block_size - 1) / block_size;
    auto iopt = x1.options().dtype(torch::kInt32);
    torch::Tensor start = torch::empty({B, R}, iopt), end = torch::empty({B, R}, iopt), flags = torch::empty({std::max<int64_t>(B, 1)}, iopt);
    raise_on(km_make_ranges_f32(B, m, n, a.data_ptr<float>(), b.data_ptr<float>(), (float)cutoff, (int32_t)block_size,
                                align ? 1 : 0, start.data_ptr<int32_t>(), end.data_ptr<int32_t>(), flags.data_ptr<int32_t>(),
                                stream_of(x1)));
    return {start, end};
}

// ranges.make_ranges_symmetric(x, cutoff, block_size)  (native/ranges/ranges.cpp:64-101)
std::tuple<torch::Tensor, torch::Tensor> make_ranges_symmetric(torch::Tensor x, double cutoff, int64_t block_size) {
    check_f32(x);
    TORCH_CHECK(x.dim() == 2, "x must be (B, n)");
    const c10::cuda::CUDAGuard guard(x.device());
    torch::Tensor a = x.contiguous();
    const int64_t B = a.size(0), n = a.size(1), R = (n + block_size - 1) / block_size;
    auto iopt = x.options().dtype(torch::kInt32);
    torch::Tensor start = torch::empty({B, R}, iopt), end = torch::empty({B, R}, iopt), flags = torch::empty({std::max<int64_t>(B, 1)}, iopt);
    raise_on(km_make_ranges_symmetric_f32(B, n, a.data_ptr<float>(), (float)cutoff, (int32_t)block_size,
                                          start.data_ptr<int32_t>(), end.data_ptr<int32_t>(), flags.data_ptr<int32_t>(),
                                          stream_of(x)));
    return {start, end};
}

// ranges.transpose_ranges(start, end, x1_size, x2_size, block_size)  (native/ranges/ranges.cpp:103-150)
std::tuple<torch::Tensor, torch::Tensor> transpose_ranges(torch::Tensor start, torch::Tensor end, int64_t x1_size,
                                                          int64_t x2_size, int64_t block_size) {
    check_i32(start), check_i32(end);
    TORCH_CHECK(start.dim() == 2 && end.sizes() == start.sizes(), "start and end must be (B, R)");
    const c10::cuda::CUDAGuard guard(start.device());
    torch::Tensor s = start.contiguous(), e = end.contiguous();
    const int64_t B = s.size(0), R = s.size(1), C = (x2_size + block_size - 1) / block_size;
    torch::Tensor st = torch::empty({B, C}, s.options()), et = torch::empty({B, C}, s.options());
    raise_on(km_transpose_ranges_i32(B, R, s.data_ptr<int32_t>(), e.data_ptr<int32_t>(), x1_size, x2_size, (int32_t)block_size,
                                     st.data_ptr<int32_t>(), et.data_ptr<int32_t>(), stream_of(start)));
    return {st, et};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "B200 kernel-matmul ops: PyTorch binding of libkm_b200.so";
    m.attr("KERNEL_RBF") = (int)KM_KERNEL_RBF;
    m.attr("KERNEL_SPECTRAL") = (int)KM_KERNEL_SPECTRAL;
    m.attr("KERNEL_LOCALLY_PERIODIC") = (int)KM_KERNEL_LOCALLY_PERIODIC;
    m.def("matmul", &matmul, pybind11::arg("kernel_type"), pybind11::arg("x1"), pybind11::arg("x2"), pybind11::arg("rhs"),
          pybind11::arg("params"), pybind11::arg("start"), pybind11::arg("end"), pybind11::arg("tensor_cores_auto") = true);
    m.def("matmul_bwd", &matmul_bwd);
    m.def("bilinear_derivative", &bilinear_derivative);
    m.def("dense", &dense);
    m.def("dense_bwd", &dense_bwd);
    m.def("index", &op_index);
    m.def("index_bwd", &op_index_bwd);
    m.def("make_ranges", &make_ranges);
    m.def("make_ranges_symmetric", &make_ranges_symmetric);
    m.def("transpose_ranges", &transpose_ranges);
}

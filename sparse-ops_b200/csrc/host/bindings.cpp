// bindings.cpp -- pybind11 module `sparseops_backend`, drop-in for the reference's module of the
// same name (src/bindings.cpp:50-217): class Ellpack (read-only m, n, r, Wd, idx, Xt),
// convert_to_ellpack, decode_from_ellpack, ellpack_matvec, ellpack_matmul (same error strings),
// class SparseOnnxModel(path).run(X).  All multiplies run on the GPU through libspx_b200.so.
//
// Additions (a strict superset): Ellpack.nnz / nnz_total / shard_rows, bias=None, shape checks
// in ellpack_matvec, SparseOnnxModel.resize_buffers / run_device / shard_rows, constructors from
// CSR or raw ELLPACK arrays, and *_device calls that take raw device pointers (ints) so that
// device-resident tensors (e.g. torch CUDA tensors via .data_ptr()) avoid the PCIe round trip.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include "ellpack.hpp"
#include "rbm.hpp"
#include "sparse_onnx.hpp"

namespace py = pybind11;
using spx::Ellpack;
using spx::SparseOnnxModel;
using farray = py::array_t<float, py::array::c_style | py::array::forcecast>;
using u32array = py::array_t<uint32_t, py::array::c_style | py::array::forcecast>;
using u64array = py::array_t<uint64_t, py::array::c_style | py::array::forcecast>;

static Ellpack convert_to_ellpack_py(farray W)
{
    auto buf = W.request();
    if (buf.ndim != 2) throw std::runtime_error("W must be 2D (m \xC3\x97 n)");
    const float* data = static_cast<const float*>(buf.ptr);
    const uint32_t m = uint32_t(buf.shape[0]), n = uint32_t(buf.shape[1]);
    py::gil_scoped_release nogil;
    return spx::convert_to_ellpack(data, m, n);
}

static py::array_t<float> decode_from_ellpack_py(const Ellpack& E)
{
    py::array_t<float> W({ py::ssize_t(E.m), py::ssize_t(E.n) });
    auto buf = W.request();
    if (size_t(buf.size) != size_t(E.m) * E.n) throw std::runtime_error("Output buffer size mismatch");
    spx::decode_from_ellpack(E, static_cast<float*>(buf.ptr));
    return W;
}

template <class T>
static py::array_t<T> copy2d(const T* src, uint32_t m, uint32_t r)
{
    py::array_t<T> a({ py::ssize_t(m), py::ssize_t(r) });
    if (m && r) std::memcpy(a.mutable_data(), src, size_t(m) * r * sizeof(T));
    return a;
}

static const float* optional_bias(const py::object& bias, farray& keep, uint32_t m, const char* msg)
{
    if (bias.is_none()) return nullptr;
    keep = farray::ensure(bias);
    if (!keep) throw std::runtime_error("bias must be convertible to a float32 array");
    if (uint32_t(keep.size()) != m) throw std::runtime_error(msg);
    return keep.data();
}

PYBIND11_MODULE(sparseops_backend, m)
{
    m.doc() = "Sparse GPU kernels (ELLPACK) for NVIDIA B200, API-compatible with sparse-ops' sparseops_backend";

    py::class_<Ellpack>(m, "Ellpack", py::module_local())
        .def_readonly("m", &Ellpack::m)
        .def_readonly("n", &Ellpack::n)
        .def_readonly("r", &Ellpack::r)
        .def_property_readonly("Wd", [](const Ellpack& E) { return copy2d<float>(E.Wd.ptr, E.m, E.r); })
        .def_property_readonly("on_device", [](const Ellpack& E) { return E.dev != nullptr; })
        .def_property_readonly("idx", [](const Ellpack& E) { return copy2d<uint32_t>(E.idx.data(), E.m, E.r); })
        .def_property_readonly("Xt", [](const Ellpack& E) {
            auto xt = E.gathered_x();
            return copy2d<float>(xt.data(), E.m, E.r);
        })
        .def_property_readonly("nnz", [](const Ellpack& E) {
            py::array_t<uint32_t> a(py::ssize_t(E.m));
            if (E.m) std::memcpy(a.mutable_data(), E.nnz.data(), size_t(E.m) * 4);
            return a;
        })
        .def_property_readonly("nnz_total", &Ellpack::nnz_total)
        .def("shard_rows", [](const Ellpack& E, uint32_t g, uint32_t G, bool upload) { return E.shard_rows(g, G, upload); },
             py::arg("index"), py::arg("count"), py::arg("upload") = true,
             "Rows [index*ceil(m/count), ...) as an independent Ellpack (uploaded unless upload=False)")
        .def("shard_range", [](const Ellpack& E, uint32_t lo, uint32_t hi, bool upload) { return E.shard_range(lo, hi, upload); },
             py::arg("lo"), py::arg("hi"), py::arg("upload") = true, "Rows [lo, hi) as an independent Ellpack")
        .def("balanced_row_split", [](const Ellpack& E, uint32_t G, uint32_t row_cost) { return E.balanced_row_split(G, row_cost); },
             py::arg("count"), py::arg("row_cost") = 8,
             "count+1 row bounds cutting the rows into contiguous ranges of near-equal nnz + row_cost per row");

    m.def("convert_to_ellpack", &convert_to_ellpack_py, "Convert dense NumPy matrix -> ELLPACK handle (device-resident)");
    m.def("decode_from_ellpack", &decode_from_ellpack_py, "Convert ELLPACK handle -> dense NumPy matrix");

    m.def("ellpack_from_csr", [](uint32_t mm, uint32_t nn, u64array rowptr, u32array col, farray val) {
        if (size_t(rowptr.size()) != size_t(mm) + 1) throw std::runtime_error("rowptr must have m+1 entries");
        if (col.size() != val.size() || uint64_t(col.size()) != rowptr.data()[mm])
            throw std::runtime_error("col / val length must equal rowptr[m]");
        return spx::ellpack_from_csr(mm, nn, rowptr.data(), col.data(), val.data());
    }, py::arg("m"), py::arg("n"), py::arg("rowptr"), py::arg("col"), py::arg("val"));

    m.def("ellpack_from_arrays", [](uint32_t nn, farray Wd, u32array idx, u32array nnz) {
        if (Wd.ndim() != 2 || idx.ndim() != 2 || Wd.shape(0) != idx.shape(0) || Wd.shape(1) != idx.shape(1))
            throw std::runtime_error("Wd and idx must be 2D arrays of the same shape (m, r)");
        if (nnz.size() != Wd.shape(0)) throw std::runtime_error("nnz must have m entries");
        Ellpack E(uint32_t(Wd.shape(0)), nn, uint32_t(Wd.shape(1)));
        const size_t tot = size_t(E.m) * E.r;
        if (tot) {
            std::memcpy(E.Wd.ptr, Wd.data(), tot * 4);
            std::memcpy(E.idx.data(), idx.data(), tot * 4);
        }
        if (E.m) std::memcpy(E.nnz.data(), nnz.data(), size_t(E.m) * 4);
        E.upload();
        return E;
    }, py::arg("n"), py::arg("Wd"), py::arg("idx"), py::arg("nnz"));

    m.def("ellpack_matvec", [](const Ellpack& E, farray x_arr, py::object bias) {
        if (uint32_t(x_arr.size()) != E.n) throw std::runtime_error("Input length must equal E.n");
        farray keep;
        const float* b = optional_bias(bias, keep, E.m, "Bias length must equal E.m");
        py::array_t<float> y(py::ssize_t(E.m));
        float* yp = y.mutable_data();
        const float* xp = x_arr.data();
        {
            py::gil_scoped_release nogil;
            spx::ellpack_matvec(E, xp, b, yp);
        }
        return y;
    }, py::arg("E"), py::arg("x"), py::arg("bias") = py::none(), "y = E x + bias (ELLPACK SpMV on the GPU)");

    m.def("ellpack_matmul", [](const Ellpack& E, farray X_arr, py::object bias) {
        auto buf_X = X_arr.request();
        if (buf_X.ndim != 2) throw std::runtime_error("X must be 2D (n \xC3\x97 C)");
        if (uint32_t(buf_X.shape[0]) != E.n) throw std::runtime_error("Input row count must equal E.n");
        farray keep;
        const float* b = optional_bias(bias, keep, E.m, "Bias length must equal E.m");
        const uint32_t C = uint32_t(buf_X.shape[1]);
        py::array_t<float> Y({ py::ssize_t(E.m), py::ssize_t(C) });
        float* yp = Y.mutable_data();
        const float* xp = static_cast<const float*>(buf_X.ptr);
        {
            py::gil_scoped_release nogil;
            spx::ellpack_matmul(E, xp, C, b, yp);
        }
        return Y;
    }, py::arg("E"), py::arg("X"), py::arg("bias") = py::none(),
       "Y = E X + bias: E ELLPACK (m x n), X (n x C) float32, bias (m,) -> Y (m x C)");

    m.def("ellpack_matmul_device", [](const Ellpack& E, uintptr_t X, uint32_t C, uint64_t ldx, uintptr_t bias, int act,
                                      uintptr_t Y, uint64_t ldy, uintptr_t stream) {
        spx::ellpack_matmul_device(E, reinterpret_cast<const float*>(X), C, ldx, reinterpret_cast<const float*>(bias), act,
                                   reinterpret_cast<float*>(Y), ldy, reinterpret_cast<void*>(stream));
    }, py::arg("E"), py::arg("X"), py::arg("C"), py::arg("ldx"), py::arg("bias"), py::arg("act"), py::arg("Y"),
       py::arg("ldy"), py::arg("stream") = 0, "SpMM on raw device pointers (asynchronous on `stream`)");

    m.def("ellpack_matvec_device", [](const Ellpack& E, uintptr_t x, uintptr_t bias, uintptr_t y, uintptr_t stream) {
        spx::ellpack_matvec_device(E, reinterpret_cast<const float*>(x), reinterpret_cast<const float*>(bias),
                                   reinterpret_cast<float*>(y), reinterpret_cast<void*>(stream));
    }, py::arg("E"), py::arg("x"), py::arg("bias"), py::arg("y"), py::arg("stream") = 0);

    m.def("build_rbm_from_ellpack", [](const Ellpack& E, py::object bias, uint32_t ct_max) {
        farray keep;
        const float* b = optional_bias(bias, keep, E.m, "Bias length must equal E.m");
        spx::RBMPlan P = spx::build_rbm_from_ellpack(E, b, ct_max);
        py::list blocks;
        for (const auto& B : P.blocks) {
            py::dict d;
            d["M0"] = B.M0;
            d["Ct"] = B.Ct;
            d["krel"] = py::array_t<uint32_t>(py::ssize_t(B.krel.size()), B.krel.data());
            d["colptr"] = py::array_t<uint32_t>(py::ssize_t(B.colptr.size()), B.colptr.data());
            py::array_t<uint16_t> rows(py::ssize_t(B.pairs.size()));
            py::array_t<float> w(py::ssize_t(B.pairs.size()));
            for (size_t t = 0; t < B.pairs.size(); ++t) { rows.mutable_data()[t] = B.pairs[t].row; w.mutable_data()[t] = B.pairs[t].w; }
            d["rows"] = rows;
            d["w"] = w;
            d["bias"] = py::array_t<float>(py::ssize_t(B.bias.size()), B.bias.data());
            blocks.append(d);
        }
        return blocks;
    }, py::arg("E"), py::arg("bias") = py::none(), py::arg("ct_max") = 8);

    m.def("encode_host", [](farray W) {
        if (W.ndim() != 2) throw std::runtime_error("W must be 2D (m \xC3\x97 n)");
        return spx::encode_host(W.data(), uint32_t(W.shape(0)), uint32_t(W.shape(1)));
    }, "ELLPACK-encode on the host only (no device copy; for inspection, cannot multiply)");
    m.def("launch_count", []() { return spx_launch_count(); }, "Kernels launched by the library so far");
    m.def("set_device", [](int d) { spx::check(spx_set_device(d), "set_device"); });
    m.def("device_count", []() { int n = 0; spx::check(spx_device_count(&n), "device_count"); return n; });
    m.def("comm_unique_id", []() {
        char id[SPX_UNIQUE_ID_BYTES];
        spx::check(spx_comm_unique_id(id), "comm_unique_id");
        return py::bytes(id, SPX_UNIQUE_ID_BYTES);
    });

    py::class_<SparseOnnxModel>(m, "SparseOnnxModel", py::module_local())
        .def(py::init<const std::string&, bool>(), py::arg("path"), py::arg("upload_weights") = true,
             "Load an ONNX model and pre-encode weights to device-resident ELLPACK "
             "(upload_weights=False: parse and plan only, no GPU needed, cannot run)")
        .def("run", [](const SparseOnnxModel& model, farray X) {
            auto buf = X.request();
            if (buf.ndim < 1) throw std::runtime_error("X must have a batch dimension");
            const uint32_t B = uint32_t(buf.shape[0]);
            if (size_t(buf.size) != size_t(B) * model.in_features())
                throw std::runtime_error("X must hold batch x in_features values");
            std::vector<size_t> dims = model.output_shape();
            if (!dims.empty()) dims[0] = B;
            py::array_t<float> Y(dims);
            float* yp = Y.mutable_data();
            const float* xp = static_cast<const float*>(buf.ptr);
            {
                py::gil_scoped_release nogil;
                model.run(xp, B, yp);
            }
            return Y;
        }, "Run inference; memory in and out is feature-major ([features x B], B fastest), as in the reference")
        .def("resize_buffers", &SparseOnnxModel::resize_buffers, py::arg("batch"))
        .def("run_device", [](const SparseOnnxModel& model, uintptr_t x, uint32_t B, uintptr_t y, uintptr_t stream) {
            model.run_device(reinterpret_cast<const float*>(x), B, reinterpret_cast<float*>(y), reinterpret_cast<void*>(stream));
        }, py::arg("x"), py::arg("batch"), py::arg("y"), py::arg("stream") = 0)
        .def("device_input_ptr", [](const SparseOnnxModel& m_) { return reinterpret_cast<uintptr_t>(m_.device_input()); })
        .def("device_output_ptr", [](const SparseOnnxModel& m_) { return reinterpret_cast<uintptr_t>(m_.device_output()); })
        .def_property_readonly("activation_buffers", &SparseOnnxModel::activation_buffers,
                               "distinct device buffers holding activations in the current plan (reused by liveness)")
        .def("run_resident", [](const SparseOnnxModel& m_, uintptr_t stream) { m_.run_resident(reinterpret_cast<void*>(stream)); },
             py::arg("stream") = 0, "Replay the captured layer loop on the model's own device buffers (asynchronous)")
        .def("shard_rows", [](SparseOnnxModel& model, int rank, int world, py::bytes id) {
            std::string s = id;
            if (world > 1 && s.size() != SPX_UNIQUE_ID_BYTES) throw std::runtime_error("unique id must be 128 bytes");
            model.shard_rows(rank, world, world > 1 ? s.data() : nullptr);
        }, py::arg("rank"), py::arg("world"), py::arg("unique_id") = py::bytes())
        .def("output_shape", &SparseOnnxModel::output_shape)
        .def_property_readonly("batch", &SparseOnnxModel::batch)
        .def_property_readonly("in_features", &SparseOnnxModel::in_features)
        .def_property_readonly("out_features", &SparseOnnxModel::out_features)
        .def("flops_per_run", &SparseOnnxModel::flops_per_run, py::arg("batch"))
        .def("layer_summary", [](const SparseOnnxModel& model) {
            py::list out;
            static const char* names[] = { "MatMul", "Relu", "Sigmoid", "Tanh", "Add", "Conv", "MaxPool", "GlobalAveragePool" };
            for (size_t i = 0; i < model.num_layers(); ++i) {
                const spx::Layer& L = model.layer(i);
                py::dict d;
                d["op"] = names[int(L.op)];
                d["act"] = L.act;
                d["bias"] = !L.bias.empty();
                d["inputs"] = L.inputs;
                d["outputs"] = L.outputs;
                if (L.E) { d["m"] = L.E->m; d["n"] = L.E->n; d["r"] = L.E->r; d["nnz"] = L.E->nnz_total(); }
                out.append(d);
            }
            return out;
        });
}

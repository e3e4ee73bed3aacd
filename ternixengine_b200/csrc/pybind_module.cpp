// Python module `ternix_engine`: the reference's binding surface (bindings/python/pybind11_wrapper.cpp:75-98)
// as a thin caller of the C ABI.  Same function names, defaults, shapes, dtypes and exception types.
// Every `impl` name of the reference is accepted and runs the B200 path; there is no CPU kernel here.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <climits>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "ternix_b200.h"

namespace py = pybind11;

namespace {

// numpy arguments arrive as C-ordered arrays of the element type the C ABI takes; other dtypes and layouts are
// converted on the way in, as the reference binding does (bindings/python/pybind11_wrapper.cpp:17-18).
using HostI8 = py::array_t<int8_t, py::array::c_style | py::array::forcecast>;
using HostU8 = py::array_t<uint8_t, py::array::c_style | py::array::forcecast>;

[[noreturn]] void bad_value(const std::string& what) { throw std::invalid_argument(what); }

// Rows and columns of a matrix argument; anything that is not a matrix is a ValueError.
struct Extent {
    py::ssize_t rows, cols;
};
Extent matrix_extent(const py::array& arr, const char* name, const char* layout) {
    if (arr.ndim() != 2) bad_value(std::string(name) + ": a 2-D " + layout + " array is required, got " +
                                   std::to_string(arr.ndim()) + " dimension(s)");
    return {arr.shape(0), arr.shape(1)};
}

// Turns a C-ABI status into the exception type the reference binding raises for that kind of failure
// (ValueError for bad arguments, RuntimeError "CUDA error: ..." for the device; pybind11_wrapper.cpp:62-69).
void raise_for_status(int rc, int cuda_err) {
    switch (rc) {
        case TERNIX_B200_OK: return;
        case TERNIX_B200_ERR_CUDA:
            throw std::runtime_error(std::string("CUDA error: ") + ternix_b200_cuda_error_string(cuda_err));
        case TERNIX_B200_ERR_INVALID_SHAPE:
        case TERNIX_B200_ERR_INVALID_ARG:
        case TERNIX_B200_ERR_UNSUPPORTED:
            bad_value(ternix_b200_status_string(rc));
        default: throw std::runtime_error(ternix_b200_status_string(rc));
    }
}

// pack_ternary(w): (K, N) int8 with entries in {-1, 0, +1} -> (K, N/4) uint8.  ValueError for a non-matrix, a column
// count that is not a multiple of 4, or an entry outside the ternary domain (the entry's position is reported).
HostU8 pack_ternary(HostI8 w) {
    const Extent e = matrix_extent(w, "pack_ternary(w)", "(K, N)");
    if (e.cols % 4) bad_value("pack_ternary(w): " + std::to_string(e.cols) + " columns; four weights share a byte, so N % 4 must be 0");
    const size_t count = static_cast<size_t>(e.rows) * static_cast<size_t>(e.cols);
    const long long bad = ternix_b200_find_non_ternary(w.data(), count);
    if (bad >= 0)
        bad_value("pack_ternary(w): entry " + std::to_string(bad) + " (row-major) is outside {-1, 0, +1}");
    HostU8 packed({e.rows, e.cols / 4});
    ternix_b200_pack_ternary(packed.mutable_data(), w.data(), count);
    return packed;
}

// unpack_ternary(packed): (K, N/4) uint8 -> (K, N) int8; the undefined code 10 comes back as 0.
HostI8 unpack_ternary(HostU8 packed) {
    const Extent e = matrix_extent(packed, "unpack_ternary(packed)", "(K, N/4)");
    HostI8 w({e.rows, e.cols * 4});
    ternix_b200_unpack_ternary(w.mutable_data(), packed.data(), static_cast<size_t>(e.rows) * static_cast<size_t>(e.cols) * 4);
    return w;
}

// Maps an `impl` string to a kernel selector.  The reference's six names are all accepted (its binding dispatches
// on them, pybind11_wrapper.cpp:49-69) and all run the GPU path chosen by shape; the two AVX2 names keep their
// N % 8 contract.  The b200_* names pick one of this library's kernels, for tests and tuning.
int kernel_of(const std::string& impl, size_t N) {
    static const struct { const char* name; int kernel; bool needs_n8; } table[] = {
        {"avx2_blocked", TERNIX_B200_KERNEL_AUTO, true},   {"avx2", TERNIX_B200_KERNEL_AUTO, true},
        {"scalar", TERNIX_B200_KERNEL_AUTO, false},        {"naive", TERNIX_B200_KERNEL_AUTO, false},
        {"cuda_naive", TERNIX_B200_KERNEL_AUTO, false},    {"cuda_tiled", TERNIX_B200_KERNEL_AUTO, false},
        {"b200", TERNIX_B200_KERNEL_AUTO, false},          {"auto", TERNIX_B200_KERNEL_AUTO, false},
        {"b200_generic", TERNIX_B200_KERNEL_GENERIC, false},
        {"b200_gemv", TERNIX_B200_KERNEL_GEMV, false},
        {"b200_gemm_tc", TERNIX_B200_KERNEL_GEMM_TC, false},
        {"b200_decode_mma", TERNIX_B200_KERNEL_DECODE_MMA, false},
        {"b200_skinny_tc", TERNIX_B200_KERNEL_SKINNY_TC, false},
    };
    for (const auto& row : table) {
        if (impl != row.name) continue;
        if (row.needs_n8 && N % 8) bad_value("impl '" + impl + "' keeps the AVX2 kernels' contract: N % 8 must be 0");
        return row.kernel;
    }
    bad_value("ternary_matmul: no implementation is called '" + impl + "'");
}

// ternary_matmul on host arrays: upload, product, download through the host-pointer entry point.  The GIL is
// dropped while the device works.
py::array_t<int32_t> ternary_matmul(HostI8 a, HostU8 b_packed, const std::string& impl) {
    const Extent ea = matrix_extent(a, "ternary_matmul(a)", "(M, K)");
    const Extent eb = matrix_extent(b_packed, "ternary_matmul(b_packed)", "(K, N/4)");
    if (ea.cols != eb.rows)
        bad_value("ternary_matmul: a has K = " + std::to_string(ea.cols) + " but b_packed has " + std::to_string(eb.rows) + " rows");
    const long long m = ea.rows, k = ea.cols, n = static_cast<long long>(eb.cols) * 4;
    if (m > INT32_MAX || k > INT32_MAX || n > INT32_MAX) bad_value("ternary_matmul: a dimension does not fit in int32");
    const int kernel = kernel_of(impl, static_cast<size_t>(n));
    py::array_t<int32_t> c({ea.rows, static_cast<py::ssize_t>(n)});
    const int8_t* a_ptr = a.data();
    const uint8_t* w_ptr = b_packed.data();
    int32_t* c_ptr = c.mutable_data();
    int rc = TERNIX_B200_OK, cuda_err = 0;
    {
        py::gil_scoped_release unlocked;
        rc = ternix_b200_matmul_host(a_ptr, w_ptr, c_ptr, static_cast<int>(m), static_cast<int>(k), static_cast<int>(n), kernel);
        if (rc == TERNIX_B200_ERR_CUDA) cuda_err = ternix_b200_last_cuda_error();
    }
    raise_for_status(rc, cuda_err);
    return c;
}

// Device-resident path: objects that expose __cuda_array_interface__ (torch / cupy / numba arrays) are used in
// place, without a host round trip (the reference's binding copies through host memory on every call,
// src/cuda_kernels.cu:142-156).  Asynchronous on `stream`; `out` is required and returned.
struct DeviceArray {
    uintptr_t ptr = 0;
    std::vector<py::ssize_t> shape, strides;     // strides in bytes (empty = C-contiguous)
    std::string typestr;
};

bool has_cai(const py::object& o) { return py::hasattr(o, "__cuda_array_interface__"); }

DeviceArray parse_cai(const py::object& o, const char* what) {
    py::dict d = o.attr("__cuda_array_interface__").cast<py::dict>();
    DeviceArray a;
    a.ptr = d["data"].cast<py::tuple>()[0].cast<uintptr_t>();
    a.shape = d["shape"].cast<std::vector<py::ssize_t>>();
    a.typestr = d["typestr"].cast<std::string>();
    if (d.contains("strides") && !d["strides"].is_none()) a.strides = d["strides"].cast<std::vector<py::ssize_t>>();
    if (a.shape.size() != 2) throw std::invalid_argument(std::string(what) + " must be 2-D");
    return a;
}

py::object ternary_matmul_device(const py::object& a, const py::object& b_packed, const std::string& impl,
                                 const py::object& out, uintptr_t stream) {
    if (out.is_none() || !has_cai(out) || !has_cai(b_packed))
        throw std::invalid_argument("device arrays need device b_packed and an `out` device array");
    const DeviceArray A = parse_cai(a, "a"), B = parse_cai(b_packed, "b_packed"), C = parse_cai(out, "out");
    if (A.typestr != "|i1" || B.typestr != "|u1" || (C.typestr != "<i4" && C.typestr != "=i4"))
        throw std::invalid_argument("dtypes must be int8 (a), uint8 (b_packed), int32 (out)");
    const py::ssize_t M = A.shape[0], K = A.shape[1], N = B.shape[1] * 4;
    if (B.shape[0] != K) throw std::invalid_argument("inner dimensions do not match");
    if (C.shape[0] != M || C.shape[1] != N) throw std::invalid_argument("out must be (M, N)");
    if ((!A.strides.empty() && (A.strides[1] != 1 || A.strides[0] != K)) ||
        (!B.strides.empty() && (B.strides[1] != 1 || B.strides[0] != N / 4)))
        throw std::invalid_argument("a and b_packed must be C-contiguous");
    py::ssize_t ldc = N;
    if (!C.strides.empty()) {
        if (C.strides[1] != 4 || C.strides[0] % 4) throw std::invalid_argument("out needs unit column stride");
        ldc = C.strides[0] / 4;
    }
    const int kernel = kernel_of(impl, static_cast<size_t>(N));
    const int rc = ternix_b200_matmul_ex(reinterpret_cast<const int8_t*>(A.ptr), reinterpret_cast<const uint8_t*>(B.ptr),
                                         reinterpret_cast<int32_t*>(C.ptr), static_cast<int>(M), static_cast<int>(K),
                                         static_cast<int>(N), ldc, kernel, nullptr, reinterpret_cast<void*>(stream));
    raise_for_status(rc, rc == TERNIX_B200_ERR_CUDA ? ternix_b200_last_cuda_error() : 0);
    return out;
}

py::object ternary_matmul_any(const py::object& a, const py::object& b_packed, const std::string& impl,
                              const py::object& out, uintptr_t stream) {
    if (has_cai(a)) return ternary_matmul_device(a, b_packed, impl, out, stream);
    return ternary_matmul(a.cast<HostI8>(), b_packed.cast<HostU8>(), impl);
}

// reference: include/ternix/model.hpp, src/model.cpp:5-13 -- a placeholder there too (it reads no file
// and runs no inference); kept only so that code which constructs it keeps importing.
struct Model {
    explicit Model(std::string p) : path(std::move(p)) {}
    void load() {}
    std::string path;
    int vocab_size = 32000, hidden_size = 4096, num_layers = 32;
};

}  // namespace

PYBIND11_MODULE(ternix_engine, m) {
    m.doc() = "TernixEngine ternary GEMM on B200 (sm_100a): packing utilities and the matmul entry point";
    m.def("pack_ternary", &pack_ternary, py::arg("w"),
          "(K, N) int8 weights with entries -1, 0 or +1 -> (K, N/4) uint8, four 2-bit codes per byte (00 zero, 01 plus one, "
          "11 minus one, lowest bits first along N)");
    m.def("unpack_ternary", &unpack_ternary, py::arg("packed"), "(K, N/4) uint8 packed weights -> (K, N) int8; undoes pack_ternary");
    m.def("ternary_matmul", &ternary_matmul_any, py::arg("a"), py::arg("b_packed"), py::arg("impl") = "avx2_blocked",
          py::arg("out") = py::none(), py::arg("stream") = 0,
          "C = A (M,K int8) @ W (K,N ternary packed) -> (M,N int32). impl: naive | scalar | avx2 | avx2_blocked | "
          "cuda_naive | cuda_tiled (all run the B200 path) | b200_generic | b200_gemv | b200_gemm_tc | b200_decode_mma | b200_skinny_tc.  Host arrays are "
          "uploaded and the result downloaded; arrays with __cuda_array_interface__ are used in place (pass `out`, "
          "optionally a CUDA stream handle) and the call is asynchronous.");
    m.attr("has_cuda") = true;
    py::class_<Model>(m, "Model")
        .def(py::init<const std::string&>())
        .def("load", &Model::load)
        .def_readwrite("vocab_size", &Model::vocab_size)
        .def_readwrite("hidden_size", &Model::hidden_size)
        .def_readwrite("num_layers", &Model::num_layers);
}

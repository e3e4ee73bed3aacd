// Python module `ternix_engine`: the reference's binding surface (bindings/python/pybind11_wrapper.cpp:75-98)
// as a thin caller of the C ABI.  Same function names, defaults, shapes, dtypes and exception types.
// Every `impl` name of the reference is accepted and runs the B200 path; there is no CPU kernel here.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "ternix_b200.h"

namespace py = pybind11;

namespace {

using i8_array = py::array_t<int8_t, py::array::c_style | py::array::forcecast>;
using u8_array = py::array_t<uint8_t, py::array::c_style | py::array::forcecast>;

// reference: pybind11_wrapper.cpp:21-31
u8_array pack_ternary(i8_array w) {
    if (w.ndim() != 2) throw std::invalid_argument("pack_ternary expects a 2-D (K, N) array");
    const py::ssize_t K = w.shape(0), N = w.shape(1);
    if (N % 4 != 0) throw std::invalid_argument("N must be a multiple of 4");
    if (ternix_b200_find_non_ternary(w.data(), static_cast<size_t>(K * N)) >= 0)
        throw std::invalid_argument("weights must be in {-1, 0, +1}");
    u8_array out({K, N / 4});
    ternix_b200_pack_ternary(out.mutable_data(), w.data(), static_cast<size_t>(K * N));
    return out;
}

// reference: pybind11_wrapper.cpp:33-39
i8_array unpack_ternary(u8_array packed) {
    if (packed.ndim() != 2) throw std::invalid_argument("unpack_ternary expects a 2-D (K, N/4) array");
    const py::ssize_t K = packed.shape(0), N4 = packed.shape(1);
    i8_array out({K, N4 * 4});
    ternix_b200_unpack_ternary(out.mutable_data(), packed.data(), static_cast<size_t>(K * N4 * 4));
    return out;
}

int kernel_of(const std::string& impl, size_t N) {
    // reference names (pybind11_wrapper.cpp:49-69): all of them run the GPU path, kernel chosen by shape
    if (impl == "naive" || impl == "scalar" || impl == "cuda_naive" || impl == "cuda_tiled") return TERNIX_B200_KERNEL_AUTO;
    if (impl == "avx2" || impl == "avx2_blocked") {
        if (N % 8 != 0) throw std::invalid_argument("AVX2 kernels need N to be a multiple of 8");
        return TERNIX_B200_KERNEL_AUTO;
    }
    // names of this library's own kernels, for tests and tuning
    if (impl == "b200" || impl == "auto") return TERNIX_B200_KERNEL_AUTO;
    if (impl == "b200_generic") return TERNIX_B200_KERNEL_GENERIC;
    if (impl == "b200_gemv") return TERNIX_B200_KERNEL_GEMV;
    if (impl == "b200_gemm_tc") return TERNIX_B200_KERNEL_GEMM_TC;
    if (impl == "b200_decode_mma") return TERNIX_B200_KERNEL_DECODE_MMA;
    throw std::invalid_argument("unknown impl '" + impl + "'");
}

// reference: pybind11_wrapper.cpp:41-71
py::array_t<int32_t> ternary_matmul(i8_array a, u8_array b_packed, const std::string& impl) {
    if (a.ndim() != 2 || b_packed.ndim() != 2) throw std::invalid_argument("A must be (M, K) and B_packed (K, N/4)");
    const size_t M = a.shape(0), K = a.shape(1), N = static_cast<size_t>(b_packed.shape(1)) * 4;
    if (static_cast<size_t>(b_packed.shape(0)) != K) throw std::invalid_argument("inner dimensions do not match");
    const int kernel = kernel_of(impl, N);
    if (M > 0x7fffffff || K > 0x7fffffff || N > 0x7fffffff) throw std::invalid_argument("dimension exceeds int32");
    py::array_t<int32_t> c({static_cast<py::ssize_t>(M), static_cast<py::ssize_t>(N)});
    const int8_t* pa = a.data();
    const uint8_t* pb = b_packed.data();
    int32_t* pc = c.mutable_data();
    int rc, cuda_err = 0;
    {
        py::gil_scoped_release release;
        rc = ternix_b200_matmul_host(pa, pb, pc, static_cast<int>(M), static_cast<int>(K), static_cast<int>(N), kernel);
        cuda_err = ternix_b200_last_cuda_error();
    }
    if (rc == TERNIX_B200_ERR_CUDA)
        throw std::runtime_error(std::string("CUDA error: ") + ternix_b200_cuda_error_string(cuda_err));
    if (rc == TERNIX_B200_ERR_UNSUPPORTED || rc == TERNIX_B200_ERR_INVALID_SHAPE || rc == TERNIX_B200_ERR_INVALID_ARG)
        throw std::invalid_argument(ternix_b200_status_string(rc));
    if (rc != TERNIX_B200_OK) throw std::runtime_error(ternix_b200_status_string(rc));
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
    if (rc == TERNIX_B200_ERR_CUDA)
        throw std::runtime_error(std::string("CUDA error: ") + ternix_b200_cuda_error_string(ternix_b200_last_cuda_error()));
    if (rc != TERNIX_B200_OK) throw std::invalid_argument(ternix_b200_status_string(rc));
    return out;
}

py::object ternary_matmul_any(const py::object& a, const py::object& b_packed, const std::string& impl,
                              const py::object& out, uintptr_t stream) {
    if (has_cai(a)) return ternary_matmul_device(a, b_packed, impl, out, stream);
    return ternary_matmul(a.cast<i8_array>(), b_packed.cast<u8_array>(), impl);
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
    m.def("pack_ternary", &pack_ternary, py::arg("w"), "Pack a (K, N) int8 array in {-1,0,1} into a (K, N/4) uint8 array");
    m.def("unpack_ternary", &unpack_ternary, py::arg("packed"), "Inverse of pack_ternary");
    m.def("ternary_matmul", &ternary_matmul_any, py::arg("a"), py::arg("b_packed"), py::arg("impl") = "avx2_blocked",
          py::arg("out") = py::none(), py::arg("stream") = 0,
          "C = A (M,K int8) @ W (K,N ternary packed) -> (M,N int32). impl: naive | scalar | avx2 | avx2_blocked | "
          "cuda_naive | cuda_tiled (all run the B200 path) | b200_generic | b200_gemv | b200_gemm_tc.  Host arrays are "
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

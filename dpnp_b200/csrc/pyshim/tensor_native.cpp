// pybind11 face of libdpnp_b200: the thin shim between the Python array layer and the C ABI.
//
// In the reference the same place is taken by the pybind11 modules
// _tensor_impl / _tensor_elementwise_impl / _tensor_reductions_impl
// (dpnp/tensor/libtensor/source/tensor_elementwise.cpp:42-45,
// source/elementwise_functions/add.cpp:176-241, tensor_reductions.cpp:40-43), whose functions
// receive `usm_ndarray` objects through the caster of dpnp/include/dpnp4pybind11.hpp:341-621
// (pointer, shape, strides, typenum, flags read once per argument).  Here an array's view is a
// `ArrayCore` object built once per Python array and kept on it; every call hands the C ABI the
// `dpb_array` inside.  No kernel and no validation lives here: the library does both
// (dpb_unary_ufunc, dpb_binary_ufunc, dpb_reduction_over_axis, ...), this file only converts
// arguments and turns status codes into the exceptions the reference raises
// (py::value_error -> ValueError, std::runtime_error -> RuntimeError).
#include <pybind11/pybind11.h>

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>

#include "../../../include/dpnp_b200.h"

namespace py = pybind11;

namespace {

[[noreturn]] void raise_status(int status)
{
    const char *msg = dpb_last_error();
    switch (status) {
    case DPB_ERR_VALUE: throw py::value_error(msg);
    case DPB_ERR_TYPE: throw py::type_error(msg);
    case DPB_ERR_MEMORY: PyErr_SetString(PyExc_MemoryError, msg); throw py::error_already_set();
    default: throw std::runtime_error(msg);
    }
}

inline void check(int status)
{
    if (status != DPB_OK) raise_status(status);
}

// The view of one array as the library wants it; shape and strides live inside the object.
struct ArrayCore {
    dpb_array d;
    int64_t dims[2 * DPB_MAX_ND];

    ArrayCore(uintptr_t ptr, int typenum, int flags, int device, const py::tuple &shape, const py::tuple &strides)
    {
        const Py_ssize_t nd = PyTuple_GET_SIZE(shape.ptr());
        if (nd > DPB_MAX_ND || PyTuple_GET_SIZE(strides.ptr()) != nd)
            throw py::value_error("shape and strides must have the same length, at most 32");
        for (Py_ssize_t i = 0; i < nd; ++i) {
            dims[i] = PyLong_AsLongLong(PyTuple_GET_ITEM(shape.ptr(), i));
            dims[DPB_MAX_ND + i] = PyLong_AsLongLong(PyTuple_GET_ITEM(strides.ptr(), i));
        }
        if (PyErr_Occurred()) throw py::error_already_set();
        d.data = reinterpret_cast<void *>(ptr);
        d.nd = static_cast<int32_t>(nd);
        d.typenum = typenum;
        d.flags = flags;
        d.device = device;
        d.shape = dims;
        d.strides = dims + DPB_MAX_ND;
    }
    ArrayCore(const ArrayCore &) = delete;
    ArrayCore &operator=(const ArrayCore &) = delete;
};

inline void *as_stream(uintptr_t s) { return reinterpret_cast<void *>(s); }

inline void use_device(int device) { check(dpb_set_device(device)); }

// One block of the stream-ordered pool; returned to the pool, ordered after the work already
// queued on its stream, when the last Python reference goes away.
struct Block {
    void *ptr = nullptr;
    size_t nbytes = 0;
    int device = 0;
    void *stream = nullptr;

    Block(size_t n, int dev, uintptr_t s) : nbytes(n), device(dev), stream(as_stream(s))
    {
        use_device(dev);
        check(dpb_malloc(n, stream, &ptr));
    }
    Block(const Block &) = delete;
    Block &operator=(const Block &) = delete;
    void release()
    {
        void *p = ptr;
        ptr = nullptr;
        if (p) {
            dpb_set_device(device);
            dpb_free(p, stream);
        }
    }
    ~Block() { release(); }
};

}  // namespace

PYBIND11_MODULE(_tensor_native, m, py::mod_gil_not_used())
{
    m.doc() = "pybind11 shim over the C ABI of libdpnp_b200";

    py::class_<ArrayCore>(m, "ArrayCore")
        .def(py::init<uintptr_t, int, int, int, const py::tuple &, const py::tuple &>(), py::arg("ptr"),
             py::arg("typenum"), py::arg("flags"), py::arg("device"), py::arg("shape"), py::arg("strides"))
        .def_property_readonly("ptr", [](const ArrayCore &a) { return reinterpret_cast<uintptr_t>(a.d.data); })
        .def_property_readonly("typenum", [](const ArrayCore &a) { return a.d.typenum; })
        .def_property_readonly("flags", [](const ArrayCore &a) { return a.d.flags; })
        .def_property_readonly("device", [](const ArrayCore &a) { return a.d.device; })
        .def_property_readonly("address", [](const ArrayCore &a) { return reinterpret_cast<uintptr_t>(&a.d); },
                               "address of the dpb_array inside (for callers that go through ctypes)");

    py::class_<Block>(m, "Block")
        .def(py::init<size_t, int, uintptr_t>(), py::arg("nbytes"), py::arg("device"), py::arg("stream"))
        .def_property_readonly("ptr", [](const Block &b) { return reinterpret_cast<uintptr_t>(b.ptr); })
        .def_property_readonly("nbytes", [](const Block &b) { return b.nbytes; })
        .def("release", &Block::release);

    // _<op>(src, dst, sycl_queue, depends) of _tensor_elementwise_impl
    m.def("unary", [](int op, const ArrayCore &src, const ArrayCore &dst, uintptr_t stream) {
        use_device(dst.d.device);
        check(dpb_unary_ufunc(op, &src.d, &dst.d, as_stream(stream)));
    });
    // _<op>(src1, src2, dst, sycl_queue, depends)
    m.def("binary", [](int op, const ArrayCore &a, const ArrayCore &b, const ArrayCore &dst, uintptr_t stream) {
        use_device(dst.d.device);
        check(dpb_binary_ufunc(op, &a.d, &b.d, &dst.d, as_stream(stream)));
    });
    // _<op>_inplace(lhs, rhs, sycl_queue, depends)
    m.def("binary_inplace", [](int op, const ArrayCore &lhs, const ArrayCore &rhs, uintptr_t stream) {
        use_device(lhs.d.device);
        check(dpb_binary_inplace_ufunc(op, &lhs.d, &rhs.d, as_stream(stream)));
    });
    // _where(condition, x1, x2, dst, sycl_queue, depends) of _tensor_impl
    m.def("where", [](const ArrayCore &c, const ArrayCore &a, const ArrayCore &b, const ArrayCore &dst,
                      uintptr_t stream) {
        use_device(dst.d.device);
        check(dpb_where(&c.d, &a.d, &b.d, &dst.d, as_stream(stream)));
    });
    // _copy_usm_ndarray_into_usm_ndarray(src, dst, sycl_queue, depends)
    m.def("copy", [](const ArrayCore &src, const ArrayCore &dst, uintptr_t stream) {
        use_device(dst.d.device);
        check(dpb_copy_array_into_array(&src.d, &dst.d, as_stream(stream)));
    });
    m.def("divide_by_scalar", [](const ArrayCore &src, double scalar, const ArrayCore &dst, uintptr_t stream) {
        use_device(dst.d.device);
        check(dpb_divide_by_scalar(&src.d, scalar, &dst.d, as_stream(stream)));
    });
    // _full_usm_ndarray(fill_value, dst, sycl_queue, depends): the value arrives as the bytes of one element
    m.def("full", [](const ArrayCore &dst, const py::bytes &bits, uintptr_t stream) {
        char buf[16] = {0};
        const std::string s = bits;
        std::memcpy(buf, s.data(), s.size() < sizeof(buf) ? s.size() : sizeof(buf));
        use_device(dst.d.device);
        check(dpb_full_array(&dst.d, buf, as_stream(stream)));
    });
    // _<op>_over_axis(src, trailing_dims_to_reduce, dst, sycl_queue, depends) of _tensor_reductions_impl
    m.def("reduce", [](int op, const ArrayCore &src, int trailing, const ArrayCore &dst, uintptr_t stream) {
        use_device(dst.d.device);
        check(dpb_reduction_over_axis(op, &src.d, trailing, &dst.d, as_stream(stream)));
    });
    m.def("search", [](int op, const ArrayCore &src, int trailing, const ArrayCore &dst, uintptr_t stream) {
        use_device(dst.d.device);
        check(dpb_search_over_axis(op, &src.d, trailing, &dst.d, as_stream(stream)));
    });
    m.def("accumulate", [](int op, const ArrayCore &src, const ArrayCore &dst, int include_initial,
                           uintptr_t stream) {
        use_device(dst.d.device);
        check(dpb_accumulate_over_axis(op, &src.d, &dst.d, include_initial, as_stream(stream)));
    });
    m.def("unary_result_type", &dpb_unary_result_type);
    m.def("binary_result_type", &dpb_binary_result_type);
    m.def("reduce_dtype_supported", &dpb_reduce_dtype_supported);
    m.def("array_overlap", [](const ArrayCore &a, const ArrayCore &b) {
        int r = 0;
        check(dpb_array_overlap(&a.d, &b.d, &r));
        return r != 0;
    });
    m.def("same_logical_tensors", [](const ArrayCore &a, const ArrayCore &b) {
        int r = 0;
        check(dpb_same_logical_tensors(&a.d, &b.d, &r));
        return r != 0;
    });
    m.def("stream_synchronize", [](int device, uintptr_t stream) {
        use_device(device);
        int st;
        {
            py::gil_scoped_release nogil;   // other Python threads run while this one waits
            st = dpb_stream_synchronize(as_stream(stream));
        }
        check(st);
    });
    m.def("version", []() { return std::string(dpb_version()); });
}

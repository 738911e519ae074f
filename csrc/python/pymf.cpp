// Python bindings. The module layout follows the reference's _pymf_hybrid (module functions + `bm` and `shm` submodules,
// src/smem/csrc/python_wrapper/memfabric_hybrid/pymf_hybrid.cpp:303-640) and _pymf_transfer (TransferEngine,
// src/smem/csrc/python_wrapper/mk_transfer_adapter/csrc/pytransfer.cpp:362-433). Addresses are Python ints, tensors are
// passed as data_ptr(); every call that can block releases the GIL. A `native` submodule exposes the control-plane
// classes and raw kernel launchers for tests and benchmarks.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <mutex>

#include "pymf_parts.h"

namespace py = pybind11;

static std::mutex g_loggerMu;
static py::function *g_pyLogger = nullptr;

static void LoggerTrampoline(int level, const char *msg)
{
    std::lock_guard<std::mutex> g(g_loggerMu);
    if (g_pyLogger == nullptr) {
        return;
    }
    py::gil_scoped_acquire gil;
    try {
        (*g_pyLogger)(level, std::string(msg));
    } catch (py::error_already_set &e) {
        e.discard_as_unraisable("memfabric logger callback");
    }
}

PYBIND11_MODULE(_pymf, m)
{
    m.doc() = "memfabric-b200 native bindings";
    m.def("initialize", [](uint32_t flags) { return mf_init(flags); }, py::arg("flags") = 0, py::call_guard<py::gil_scoped_release>());
    m.def("uninitialize", []() { mf_uninit(); }, py::call_guard<py::gil_scoped_release>());
    m.def("set_log_level", &mf_set_log_level, py::arg("level"));
    m.def("set_extern_logger", [](py::object fn) {
        {
            std::lock_guard<std::mutex> g(g_loggerMu);
            delete g_pyLogger;
            g_pyLogger = fn.is_none() ? nullptr : new py::function(fn.cast<py::function>());
        }
        return mf_set_extern_logger(fn.is_none() ? nullptr : LoggerTrampoline);
    });
    m.def("get_last_err_msg", []() { return std::string(mf_get_last_err_msg()); });
    m.def("get_and_clear_last_err_msg", []() { return std::string(mf_get_and_clear_last_err_msg()); });
    m.def("set_conf_store_tls", [](bool enable, const std::string &info) { return mf_set_conf_store_tls(enable, info.c_str(), (uint32_t)info.size()); },
          py::arg("enable"), py::arg("tls_info") = "");
    m.def("set_conf_store_tls_key", [](const std::string &, const std::string &, py::object) { return mf_set_config_store_tls_key(nullptr, 0, nullptr, 0, nullptr); });
    m.def("create_config_store", [](const std::string &url) { return mf_create_config_store(url.c_str()); }, py::arg("store_url"),
          py::call_guard<py::gil_scoped_release>());
    m.def("destroy_config_store", [](const std::string &url) { mf_destroy_config_store(url.c_str()); }, py::arg("store_url"),
          py::call_guard<py::gil_scoped_release>());
    m.def("version", []() { return std::string(mf_version()); });
    m.def("trace_enable", [](const std::string &dir) { return mf_trace_enable(dir.empty() ? nullptr : dir.c_str()); }, py::arg("dump_dir") = "");
    m.def("trace_disable", &mf_trace_disable);
    m.def("trace_dump", [](bool reset) {
        size_t n = mf_trace_dump(nullptr, 0, false);
        std::string s(n + 1, '\0');
        mf_trace_dump(&s[0], s.size(), reset);
        s.resize(n);
        return s;
    }, py::arg("reset") = false);

    BindBm(m);
    BindShm(m);
    BindTrans(m);
    BindNative(m);
    BindOps(m);
}

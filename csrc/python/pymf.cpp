// Python bindings. The module layout follows the reference's _pymf_hybrid (module functions + `bm` and `shm` submodules,
// src/smem/csrc/python_wrapper/memfabric_hybrid/pymf_hybrid.cpp:303-640) and _pymf_transfer (TransferEngine,
// src/smem/csrc/python_wrapper/mk_transfer_adapter/csrc/pytransfer.cpp:362-433). Addresses are Python ints, tensors are
// passed as data_ptr(); every call that can block releases the GIL. A `native` submodule exposes the control-plane
// classes and raw kernel launchers for tests and benchmarks.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>

#include <cstring>
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

py::function *g_pyDecrypt = nullptr;

int DecryptTrampoline(const char *cipher, size_t cipherLen, char *plain, size_t *plainLen)
{
    if (cipher == nullptr || plain == nullptr || plainLen == nullptr || cipherLen > (10u << 20)) {
        return -1;
    }
    py::gil_scoped_acquire gil;
    std::lock_guard<std::mutex> g(g_loggerMu);
    if (g_pyDecrypt == nullptr) {
        return -1;
    }
    try {
        py::object r = (*g_pyDecrypt)(py::bytes(cipher, cipherLen));
        std::string out = py::isinstance<py::bytes>(r) ? std::string(r.cast<py::bytes>()) : r.cast<std::string>();
        int rc = -1;
        if (out.size() <= *plainLen) {
            std::memcpy(plain, out.data(), out.size());
            *plainLen = out.size();
            rc = 0;
        }
        volatile char *w = out.empty() ? nullptr : &out[0];
        for (size_t i = 0; i < out.size(); i++) {
            w[i] = 0;
        }
        return rc;
    } catch (const std::exception &) {
        return -1;
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
    // decrypt_fn(cipher: bytes) -> str | bytes turns a stored (encrypted) pass phrase into the real one; None = the pass phrase is
    // given in clear. Mirrors the reference's binding (pymf_hybrid.cpp:256-294): 10 MiB cipher cap, temporaries are wiped.
    m.def("set_conf_store_tls_key", [](const std::string &pk, const std::string &pw, py::object decrypt) {
        {
            std::lock_guard<std::mutex> g(g_loggerMu);
            delete g_pyDecrypt;
            g_pyDecrypt = decrypt.is_none() ? nullptr : new py::function(decrypt.cast<py::function>());
        }
        return mf_set_config_store_tls_key(pk.data(), (uint32_t)pk.size(), pw.data(), (uint32_t)pw.size(), decrypt.is_none() ? nullptr : DecryptTrampoline);
    }, py::arg("tls_pk"), py::arg("tls_pk_pw") = "", py::arg("decrypt_fn") = py::none());
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
    BindTransport(m);
}

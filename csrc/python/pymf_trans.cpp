// TransferEngine binding (reference: _pymf_transfer, src/smem/csrc/python_wrapper/mk_transfer_adapter/csrc/pytransfer.cpp:40-81
// initialize, :362-433 module; class layout include/pytransfer.h:31-95). Same method names; `initialize` returns as soon as
// the engine is registered with the store (the reference sleeps 10 s there).
#include <pybind11/stl.h>

#include <string>
#include <vector>

#include "mf/mf_trans.h"
#include "pymf_parts.h"

namespace py = pybind11;

namespace {

enum class TransferOpcode : int { READ = 0, WRITE = 1 };

class TransferEngine {
public:
    ~TransferEngine() { Destroy(); }

    int Initialize(const std::string &storeUrl, const std::string &uniqueId, const std::string &role, int deviceId, mf_bm_data_op_type opType)
    {
        mf_trans_config_t cfg;
        mf_trans_config_init(&cfg);
        if (role == "Prefill") {
            cfg.role = MF_TRANS_SENDER;
        } else if (role == "Decode") {
            cfg.role = MF_TRANS_RECEIVER;
        } else if (role == "Both" || role.empty()) {
            cfg.role = MF_TRANS_BOTH;
        } else {
            return MF_INVALID_PARAM;
        }
        cfg.deviceId = deviceId < 0 ? 0 : (uint32_t)deviceId;
        cfg.dataOpType = opType;
        int rc = mf_trans_init(&cfg);
        if (rc != MF_OK) {
            return rc;
        }
        h_ = mf_trans_create(storeUrl.c_str(), uniqueId.c_str(), &cfg);
        if (h_ == nullptr) {
            return MF_ERROR;
        }
        size_t colon = uniqueId.rfind(':');
        port_ = colon == std::string::npos ? 0 : std::atoi(uniqueId.c_str() + colon + 1);
        return MF_OK;
    }
    int RpcPort() const { return port_; }
    void Destroy()
    {
        if (h_ != nullptr) {
            mf_trans_destroy(h_, 0);
            h_ = nullptr;
        }
    }
    mf_trans_t h_{nullptr};
    int port_{0};
};

int Batch(TransferEngine &e, bool write, const std::string &dest, std::vector<uint64_t> &locals, std::vector<uint64_t> &peers, std::vector<uint64_t> &lens,
          bool async, uint64_t stream)
{
    if (locals.size() != peers.size() || locals.size() != lens.size() || locals.empty()) {
        return MF_INVALID_PARAM;
    }
    std::vector<size_t> sizes(lens.begin(), lens.end());
    uint32_t n = (uint32_t)locals.size();
    if (write) {
        return async ? mf_trans_batch_write_submit(e.h_, (const void **)locals.data(), dest.c_str(), (void **)peers.data(), sizes.data(), n, (void *)stream, 0)
                     : mf_trans_batch_write(e.h_, (const void **)locals.data(), dest.c_str(), (void **)peers.data(), sizes.data(), n, 0);
    }
    return async ? mf_trans_batch_read_submit(e.h_, (void **)locals.data(), dest.c_str(), (const void **)peers.data(), sizes.data(), n, (void *)stream, 0)
                 : mf_trans_batch_read(e.h_, (void **)locals.data(), dest.c_str(), (const void **)peers.data(), sizes.data(), n, 0);
}

}  // namespace

void BindTrans(py::module_ &m)
{
    py::enum_<TransferOpcode>(m, "TransferOpcode").value("READ", TransferOpcode::READ).value("WRITE", TransferOpcode::WRITE).export_values();
    m.attr("TransDataOpType") = m.attr("bm").attr("BmDataOpType");  // same values, one C++ enum

    py::class_<TransferEngine>(m, "TransferEngine")
        .def(py::init<>())
        .def("initialize", [](TransferEngine &e, const std::string &url, const std::string &id, const std::string &role, int dev, py::object op) {
            mf_bm_data_op_type t = op.is_none() ? MF_BM_DATA_OP_SDMA : (mf_bm_data_op_type)op.cast<int>();
            py::gil_scoped_release nogil;
            return e.Initialize(url, id, role, dev, t);
        }, py::arg("store_url"), py::arg("unique_id"), py::arg("role"), py::arg("device_id"), py::arg("op_type") = py::none())
        .def("get_rpc_port", &TransferEngine::RpcPort)
        .def("get_rank", [](TransferEngine &e) { return mf_trans_get_rank(e.h_); })
        .def("malloc", [](TransferEngine &e, uint64_t size) { return (uint64_t)mf_trans_malloc(e.h_, size); }, py::call_guard<py::gil_scoped_release>())
        .def("free", [](TransferEngine &e, uint64_t addr) { return mf_trans_free(e.h_, (void *)addr); }, py::call_guard<py::gil_scoped_release>())
        .def("register_memory", [](TransferEngine &e, uint64_t addr, uint64_t size) { return mf_trans_register_mem(e.h_, (void *)addr, size, 0); },
             py::arg("buffer_addr"), py::arg("capacity"), py::call_guard<py::gil_scoped_release>())
        .def("unregister_memory", [](TransferEngine &e, uint64_t addr) { return mf_trans_deregister_mem(e.h_, (void *)addr); }, py::arg("buffer_addr"),
             py::call_guard<py::gil_scoped_release>())
        .def("batch_register_memory", [](TransferEngine &e, std::vector<uint64_t> addrs, std::vector<uint64_t> sizes) {
            if (addrs.size() != sizes.size() || addrs.empty()) {
                return (int)MF_INVALID_PARAM;
            }
            std::vector<size_t> caps(sizes.begin(), sizes.end());
            return mf_trans_batch_register_mem(e.h_, (void **)addrs.data(), caps.data(), (uint32_t)addrs.size(), 0);
        }, py::arg("buffer_addrs"), py::arg("capacities"), py::call_guard<py::gil_scoped_release>())
        .def("transfer_sync_write", [](TransferEngine &e, const std::string &dest, uint64_t buf, uint64_t peer, uint64_t len) {
            return mf_trans_write(e.h_, (const void *)buf, dest.c_str(), (void *)peer, len, 0);
        }, py::arg("destflag"), py::arg("buffer"), py::arg("peer_buffer_address"), py::arg("length"), py::call_guard<py::gil_scoped_release>())
        .def("transfer_sync_read", [](TransferEngine &e, const std::string &dest, uint64_t buf, uint64_t peer, uint64_t len) {
            return mf_trans_read(e.h_, (void *)buf, dest.c_str(), (const void *)peer, len, 0);
        }, py::arg("destflag"), py::arg("buffer"), py::arg("peer_buffer_address"), py::arg("length"), py::call_guard<py::gil_scoped_release>())
        .def("batch_transfer_sync_write", [](TransferEngine &e, const std::string &dest, std::vector<uint64_t> b, std::vector<uint64_t> p, std::vector<uint64_t> l) {
            return Batch(e, true, dest, b, p, l, false, 0);
        }, py::arg("destflag"), py::arg("buffers"), py::arg("peer_buffer_addresses"), py::arg("lengths"), py::call_guard<py::gil_scoped_release>())
        .def("batch_transfer_sync_read", [](TransferEngine &e, const std::string &dest, std::vector<uint64_t> b, std::vector<uint64_t> p, std::vector<uint64_t> l) {
            return Batch(e, false, dest, b, p, l, false, 0);
        }, py::arg("destflag"), py::arg("buffers"), py::arg("peer_buffer_addresses"), py::arg("lengths"), py::call_guard<py::gil_scoped_release>())
        .def("transfer_async_write_submit", [](TransferEngine &e, const std::string &dest, uint64_t buf, uint64_t peer, uint64_t len, uint64_t stream) {
            return mf_trans_write_submit(e.h_, (const void *)buf, dest.c_str(), (void *)peer, len, (void *)stream, 0);
        }, py::arg("destflag"), py::arg("buffer"), py::arg("peer_buffer_address"), py::arg("length"), py::arg("stream"), py::call_guard<py::gil_scoped_release>())
        .def("transfer_async_read_submit", [](TransferEngine &e, const std::string &dest, uint64_t buf, uint64_t peer, uint64_t len, uint64_t stream) {
            return mf_trans_read_submit(e.h_, (void *)buf, dest.c_str(), (const void *)peer, len, (void *)stream, 0);
        }, py::arg("destflag"), py::arg("buffer"), py::arg("peer_buffer_address"), py::arg("length"), py::arg("stream"), py::call_guard<py::gil_scoped_release>())
        .def("batch_transfer_async_write_submit", [](TransferEngine &e, const std::string &dest, std::vector<uint64_t> b, std::vector<uint64_t> p,
                                                     std::vector<uint64_t> l, uint64_t stream) { return Batch(e, true, dest, b, p, l, true, stream); },
             py::arg("destflag"), py::arg("buffers"), py::arg("peer_buffer_addresses"), py::arg("lengths"), py::arg("stream"), py::call_guard<py::gil_scoped_release>())
        .def("batch_transfer_async_read_submit", [](TransferEngine &e, const std::string &dest, std::vector<uint64_t> b, std::vector<uint64_t> p,
                                                    std::vector<uint64_t> l, uint64_t stream) { return Batch(e, false, dest, b, p, l, true, stream); },
             py::arg("destflag"), py::arg("buffers"), py::arg("peer_buffer_addresses"), py::arg("lengths"), py::arg("stream"), py::call_guard<py::gil_scoped_release>())
        .def("destroy", [](TransferEngine &e) { e.Destroy(); }, py::call_guard<py::gil_scoped_release>())
        .def("unInitialize", [](TransferEngine &e) {
            e.Destroy();
            mf_trans_uninit(0);
        }, py::call_guard<py::gil_scoped_release>());
}

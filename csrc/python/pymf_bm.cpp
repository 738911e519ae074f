// `bm` submodule: BmConfig, enums, initialize/uninitialize/bm_rank_id/create and the BigMemory class
// (reference: pymf_hybrid.cpp:112-233 BigMemory holder, :420-560 bm submodule).
#include <pybind11/stl.h>

#include <cstring>
#include <stdexcept>

#include "pymf_parts.h"

namespace py = pybind11;

namespace {

struct BigMemory {
    mf_bm_t h{nullptr};
    ~BigMemory() { Destroy(); }
    void Destroy()
    {
        if (h != nullptr) {
            mf_bm_destroy(h);
            h = nullptr;
        }
    }
};

uint32_t g_worldSize = 0;

}  // namespace

void BindBm(py::module_ &m)
{
    py::module_ bm = m.def_submodule("bm", "Big Memory: pooled HBM + DRAM over a global virtual address space");

    py::enum_<mf_bm_copy_type>(bm, "BmCopyType")
        .value("L2G", MF_BM_COPY_L2G)
        .value("G2L", MF_BM_COPY_G2L)
        .value("G2H", MF_BM_COPY_G2H)
        .value("H2G", MF_BM_COPY_H2G)
        .value("L2GH", MF_BM_COPY_L2GH)
        .value("GH2L", MF_BM_COPY_GH2L)
        .value("GH2H", MF_BM_COPY_GH2H)
        .value("H2GH", MF_BM_COPY_H2GH)
        .value("G2G", MF_BM_COPY_G2G)
        .value("AUTO", MF_BM_COPY_AUTO)
        .export_values();
    py::enum_<mf_bm_mem_type>(bm, "BmMemType")
        .value("LOCAL_DEVICE", MF_MEM_TYPE_LOCAL_DEVICE)
        .value("LOCAL_HOST", MF_MEM_TYPE_LOCAL_HOST)
        .value("DEVICE", MF_MEM_TYPE_DEVICE)
        .value("HOST", MF_MEM_TYPE_HOST)
        .export_values();
    py::enum_<mf_bm_data_op_type>(bm, "BmDataOpType", py::arithmetic())
        .value("SDMA", MF_BM_DATA_OP_SDMA)
        .value("HOST_RDMA", MF_BM_DATA_OP_HOST_RDMA)
        .value("HOST_TCP", MF_BM_DATA_OP_HOST_TCP)
        .value("DEVICE_RDMA", MF_BM_DATA_OP_DEVICE_RDMA)
        .value("HOST_URMA", MF_BM_DATA_OP_HOST_URMA)
        .export_values();

    py::class_<mf_bm_config_t>(bm, "BmConfig")
        .def(py::init([]() {
            mf_bm_config_t c;
            mf_bm_config_init(&c);
            return c;
        }))
        .def_readwrite("init_timeout", &mf_bm_config_t::initTimeout)
        .def_readwrite("create_timeout", &mf_bm_config_t::createTimeout)
        .def_readwrite("operation_timeout", &mf_bm_config_t::controlOperationTimeout)
        .def_readwrite("start_store", &mf_bm_config_t::startConfigStoreServer)
        .def_readwrite("start_store_only", &mf_bm_config_t::startConfigStoreOnly)
        .def_readwrite("dynamic_world_size", &mf_bm_config_t::dynamicWorldSize)
        .def_readwrite("unified_address_space", &mf_bm_config_t::unifiedAddressSpace)
        .def_readwrite("auto_ranking", &mf_bm_config_t::autoRanking)
        .def_readwrite("rank_id", &mf_bm_config_t::rankId)
        .def_readwrite("flags", &mf_bm_config_t::flags)
        .def("set_nic", [](mf_bm_config_t &c, const std::string &nic) {
            std::strncpy(c.hcomUrl, nic.c_str(), sizeof(c.hcomUrl) - 1);
        });

    bm.def("initialize", [](const std::string &url, uint32_t worldSize, int deviceId, const mf_bm_config_t &cfg) {
        g_worldSize = worldSize;
        py::gil_scoped_release nogil;
        return mf_bm_init(url.c_str(), worldSize, deviceId < 0 ? (uint16_t)0xFFFF : (uint16_t)deviceId, &cfg);
    }, py::arg("store_url"), py::arg("world_size"), py::arg("device_id"), py::arg("config"));
    bm.def("uninitialize", [](uint32_t flags) { mf_bm_uninit(flags); }, py::arg("flags") = 0, py::call_guard<py::gil_scoped_release>());
    bm.def("bm_rank_id", &mf_bm_get_rank_id);

    auto create = [](uint32_t id, uint64_t localDram, uint64_t localHbm, mf_bm_data_op_type op, uint32_t flags, uint64_t maxDram, uint64_t maxHbm,
                     const std::string &tag, const std::string &tagOpInfo, int shmFd) {
        mf_bm_create_option_t o;
        std::memset(&o, 0, sizeof(o));
        o.localDRAMSize = localDram;
        o.localHBMSize = localHbm;
        o.maxDramSize = maxDram ? maxDram : localDram;
        o.maxHbmSize = maxHbm ? maxHbm : localHbm;
        o.dataOpType = op;
        o.flags = flags;
        o.dramShmFd = shmFd;
        std::strncpy(o.tag, tag.c_str(), sizeof(o.tag) - 1);
        std::strncpy(o.tagOpInfo, tagOpInfo.c_str(), sizeof(o.tagOpInfo) - 1);
        mf_bm_t h;
        {
            py::gil_scoped_release nogil;
            h = mf_bm_create2(id, &o);
        }
        if (h == nullptr) {
            throw std::runtime_error(std::string("bm.create failed: ") + mf_get_last_err_msg());
        }
        auto *b = new BigMemory();
        b->h = h;
        return b;
    };
    bm.def("create", create, py::arg("id"), py::arg("local_dram_size"), py::arg("local_hbm_size"), py::arg("data_op_type") = MF_BM_DATA_OP_SDMA,
           py::arg("flags") = 0, py::arg("max_dram_size") = 0, py::arg("max_hbm_size") = 0, py::arg("tag") = "", py::arg("tag_op_info") = "",
           py::arg("dram_shm_fd") = -1, py::return_value_policy::take_ownership);

    py::class_<BigMemory>(bm, "BigMemory")
        .def("join", [](BigMemory &b, uint32_t flags) { return mf_bm_join(b.h, flags); }, py::arg("flags") = 0, py::call_guard<py::gil_scoped_release>())
        .def("leave", [](BigMemory &b, uint32_t flags) { return mf_bm_leave(b.h, flags); }, py::arg("flags") = 0, py::call_guard<py::gil_scoped_release>())
        .def("local_mem_size", [](BigMemory &b, mf_bm_mem_type t) { return mf_bm_get_local_mem_size_by_mem_type(b.h, t); }, py::arg("mem_type") = MF_MEM_TYPE_DEVICE)
        .def("peer_rank_ptr", [](BigMemory &b, mf_bm_mem_type t, uint32_t rank) { return (uint64_t)mf_bm_ptr_by_mem_type(b.h, t, (uint16_t)rank); },
             py::arg("mem_type"), py::arg("rank"))
        .def("destroy", [](BigMemory &b) { b.Destroy(); }, py::call_guard<py::gil_scoped_release>())
        .def("get_rank_id_by_gva", [](BigMemory &b, uint64_t gva) { return mf_bm_get_rank_id_by_gva(b.h, (void *)gva); })
        .def("joined_size", [](BigMemory &b) { return mf_bm_get_joined_size(b.h); })
        .def("register", [](BigMemory &b, uint64_t addr, uint64_t size) { return mf_bm_register_user_mem(b.h, addr, size); }, py::call_guard<py::gil_scoped_release>())
        .def("unregister", [](BigMemory &b, uint64_t addr) { return mf_bm_unregister_user_mem(b.h, addr); }, py::call_guard<py::gil_scoped_release>())
        .def("copy_data", [](BigMemory &b, uint64_t src, uint64_t dst, uint64_t size, mf_bm_copy_type t, uint32_t flags) {
            mf_copy_params p{(const void *)src, (void *)dst, (size_t)size};
            return mf_bm_copy(b.h, &p, t, flags);
        }, py::arg("src"), py::arg("dest"), py::arg("size"), py::arg("type") = MF_BM_COPY_AUTO, py::arg("flags") = 0, py::call_guard<py::gil_scoped_release>())
        .def("copy_data_on_stream", [](BigMemory &b, uint64_t src, uint64_t dst, uint64_t size, mf_bm_copy_type t, uint64_t stream, uint32_t flags) {
            mf_copy_params p{(const void *)src, (void *)dst, (size_t)size};
            return mf_bm_copy_on_stream(b.h, &p, t, (void *)stream, flags);
        }, py::arg("src"), py::arg("dest"), py::arg("size"), py::arg("type"), py::arg("stream"), py::arg("flags") = 0, py::call_guard<py::gil_scoped_release>())
        .def("copy_data_batch", [](BigMemory &b, std::vector<uint64_t> srcs, std::vector<uint64_t> dsts, std::vector<uint64_t> sizes, uint32_t count,
                                   mf_bm_copy_type t, uint32_t flags) {
            if (srcs.size() < count || dsts.size() < count || sizes.size() < count) {
                return (int32_t)MF_INVALID_PARAM;
            }
            mf_batch_copy_params p{(void **)srcs.data(), (void **)dsts.data(), sizes.data(), count};
            return mf_bm_copy_batch(b.h, &p, t, flags);
        }, py::arg("src_addrs"), py::arg("dest_addrs"), py::arg("sizes"), py::arg("count"), py::arg("type") = MF_BM_COPY_AUTO, py::arg("flags") = 0,
             py::call_guard<py::gil_scoped_release>())
        .def("copy_data_batch_on_stream", [](BigMemory &b, std::vector<uint64_t> srcs, std::vector<uint64_t> dsts, std::vector<uint64_t> sizes,
                                             mf_bm_copy_type t, uint64_t stream, uint32_t flags) {
            uint32_t count = (uint32_t)sizes.size();
            if (srcs.size() != count || dsts.size() != count) {
                return (int32_t)MF_INVALID_PARAM;
            }
            mf_batch_copy_params p{(void **)srcs.data(), (void **)dsts.data(), sizes.data(), count};
            return mf_bm_copy_batch_on_stream(b.h, &p, t, (void *)stream, flags);
        }, py::arg("src_addrs"), py::arg("dest_addrs"), py::arg("sizes"), py::arg("type"), py::arg("stream"), py::arg("flags") = 0,
             py::call_guard<py::gil_scoped_release>())
        .def("wait", [](BigMemory &b) { return mf_bm_wait(b.h); }, py::call_guard<py::gil_scoped_release>());
}

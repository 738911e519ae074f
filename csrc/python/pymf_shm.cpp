// `shm` submodule: ShmConfig, ShmDataOpType, initialize/uninitialize/create and the ShareMemory class
// (reference: pymf_hybrid.cpp:31-110 ShareMemory holder, :560-640 shm submodule).
#include <pybind11/functional.h>
#include <pybind11/stl.h>

#include <stdexcept>

#include "mf/mf_shm.h"
#include "pymf_parts.h"

namespace py = pybind11;

namespace {

struct ShareMemory {
    mf_shm_t h{nullptr};
    uint64_t gva{0};
    uint64_t symmetricSize{0};
    ~ShareMemory() { Destroy(); }
    void Destroy()
    {
        if (h != nullptr) {
            mf_shm_destroy(h, 0);
            h = nullptr;
        }
    }
};

py::function *g_exitFn = nullptr;
void ExitTrampoline(int status)
{
    if (g_exitFn == nullptr) {
        return;
    }
    py::gil_scoped_acquire gil;
    try {
        (*g_exitFn)(status);
    } catch (py::error_already_set &e) {
        e.discard_as_unraisable("memfabric exit callback");
    }
}

}  // namespace

void BindShm(py::module_ &m)
{
    py::module_ shm = m.def_submodule("shm", "Share Memory: a symmetric heap reachable from CUDA kernels of every rank");

    py::enum_<mf_shm_data_op_type>(shm, "ShmDataOpType", py::arithmetic())
        .value("MTE", MF_SHM_DATA_OP_MTE)
        .value("SDMA", MF_SHM_DATA_OP_SDMA)
        .value("RDMA", MF_SHM_DATA_OP_RDMA)
        .export_values();

    py::class_<mf_shm_config_t>(shm, "ShmConfig")
        .def(py::init([]() {
            mf_shm_config_t c;
            mf_shm_config_init(&c);
            return c;
        }))
        .def_readwrite("init_timeout", &mf_shm_config_t::shmInitTimeout)
        .def_readwrite("create_timeout", &mf_shm_config_t::shmCreateTimeout)
        .def_readwrite("operation_timeout", &mf_shm_config_t::controlOperationTimeout)
        .def_readwrite("start_store", &mf_shm_config_t::startConfigStoreServer)
        .def_readwrite("flags", &mf_shm_config_t::flags);

    shm.def("initialize", [](const std::string &url, uint32_t world, uint32_t rank, int device, mf_shm_config_t cfg) {
        py::gil_scoped_release nogil;
        return mf_shm_init(url.c_str(), world, rank, device < 0 ? (uint16_t)0xFFFF : (uint16_t)device, &cfg);
    }, py::arg("store_url"), py::arg("world_size"), py::arg("rank_id"), py::arg("device_id"), py::arg("config"));
    shm.def("uninitialize", [](uint32_t flags) { mf_shm_uninit(flags); }, py::arg("flags") = 0, py::call_guard<py::gil_scoped_release>());
    shm.def("query_support_data_operation", &mf_shm_query_support_data_operation);
    shm.def("create", [](uint32_t id, uint32_t rankSize, uint32_t rankId, uint64_t symSize, uint32_t opType, uint32_t flags) {
        void *gva = nullptr;
        mf_shm_t h;
        {
            py::gil_scoped_release nogil;
            h = mf_shm_create(id, rankSize, rankId, symSize, (mf_shm_data_op_type)opType, flags, &gva);
        }
        if (h == nullptr) {
            throw std::runtime_error(std::string("shm.create failed: ") + mf_get_last_err_msg());
        }
        auto *s = new ShareMemory();
        s->h = h;
        s->gva = (uint64_t)gva;
        s->symmetricSize = symSize;
        return s;
    }, py::arg("id"), py::arg("rank_size"), py::arg("rank_id"), py::arg("local_mem_size"), py::arg("data_op_type") = (uint32_t)MF_SHM_DATA_OP_MTE,
            py::arg("flags") = 0, py::return_value_policy::take_ownership);

    py::class_<ShareMemory>(shm, "ShareMemory")
        .def("set_context", [](ShareMemory &s, py::bytes ctx) {
            std::string c(ctx);
            return mf_shm_set_extra_context(s.h, c.data(), (uint32_t)c.size());
        })
        .def_property_readonly("local_rank", [](ShareMemory &s) { return mf_shm_get_global_rank(s.h); })
        .def_property_readonly("rank_size", [](ShareMemory &s) { return mf_shm_get_global_rank_size(s.h); })
        .def_property_readonly("gva", [](ShareMemory &s) { return s.gva; })
        .def_property_readonly("symmetric_size", [](ShareMemory &s) { return s.symmetricSize; })
        .def_property_readonly("device_meta", [](ShareMemory &s) { return (uint64_t)mf_shm_get_device_meta(s.h); })
        .def_property_readonly("signal_base", [](ShareMemory &s) { return (uint64_t)mf_shm_get_signal_base(s.h); })
        .def_property_readonly("multicast_ptr", [](ShareMemory &s) { return (uint64_t)mf_shm_get_multicast_ptr(s.h); })
        .def("local_ptr", [](ShareMemory &s) { return s.gva + (uint64_t)mf_shm_get_global_rank(s.h) * s.symmetricSize; })
        .def("peer_ptr", [](ShareMemory &s, uint32_t rank) { return s.gva + (uint64_t)rank * s.symmetricSize; })
        .def("set_debug_flags", [](ShareMemory &s, uint64_t flags) { return mf_shm_set_debug_flags(s.h, flags); }, py::arg("flags"))
        .def("next_epoch", [](ShareMemory &s, uint32_t channel) { return mf_shm_next_epoch(s.h, channel); }, py::arg("channel") = 0)
        .def("destroy", [](ShareMemory &s) { s.Destroy(); }, py::call_guard<py::gil_scoped_release>())
        .def("query_support_data_operation", [](ShareMemory &) { return mf_shm_query_support_data_operation(); })
        .def("barrier", [](ShareMemory &s) { return mf_shm_control_barrier(s.h); }, py::call_guard<py::gil_scoped_release>())
        .def("all_gather", [](ShareMemory &s, py::bytes send) {
            std::string in(send);
            std::string out(in.size() * mf_shm_get_global_rank_size(s.h), '\0');
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = mf_shm_control_allgather(s.h, in.data(), (uint32_t)in.size(), &out[0], (uint32_t)out.size());
            }
            if (rc != 0) {
                throw std::runtime_error(std::string("all_gather failed: ") + mf_get_last_err_msg());
            }
            return py::bytes(out);
        })
        .def("subgroup_barrier", [](ShareMemory &s, const std::string &key, uint32_t size, uint32_t rank) {
            return mf_shm_subgroup_barrier(s.h, key.c_str(), size, rank);
        }, py::call_guard<py::gil_scoped_release>())
        .def("subgroup_all_gather", [](ShareMemory &s, const std::string &key, uint32_t size, uint32_t rank, py::bytes send) {
            std::string in(send);
            std::string out(in.size() * size, '\0');
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = mf_shm_subgroup_allgather(s.h, key.c_str(), size, rank, in.data(), (uint32_t)in.size(), &out[0], (uint32_t)out.size());
            }
            if (rc != 0) {
                throw std::runtime_error(std::string("subgroup_all_gather failed: ") + mf_get_last_err_msg());
            }
            return py::bytes(out);
        })
        .def("topology_can_reach", [](ShareMemory &s, uint32_t rank) {
            uint32_t info = 0;
            int rc = mf_shm_topology_can_reach(s.h, rank, &info);
            return py::make_tuple(rc, info);
        })
        .def("atomic_alloc_value", [](ShareMemory &s, uint32_t limit) {
            uint32_t v = 0;
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = mf_shm_atomic_alloc_value(s.h, limit, &v);
            }
            return py::make_tuple(rc, v);
        })
        .def("atomic_release_value", [](ShareMemory &s, uint32_t v) { return mf_shm_atomic_release_value(s.h, v); }, py::call_guard<py::gil_scoped_release>())
        .def("register_exit", [](ShareMemory &s, py::function fn) {
            delete g_exitFn;
            g_exitFn = new py::function(std::move(fn));
            return mf_shm_register_exit(s.h, ExitTrampoline);
        })
        .def("global_exit", [](ShareMemory &s, int status) { return mf_shm_global_exit(s.h, status); }, py::call_guard<py::gil_scoped_release>());
}

// Bindings of the transport layer (native.Transport): enough to drive a transport directly from tests and tools.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../transport/mf_compose_transport.h"
#include "../transport/mf_host_tcp_transport.h"
#include "../transport/mf_peer_link_manager.h"
#include "../transport/mf_transport.h"
#include "../util/mf_net_util.h"

namespace py = pybind11;
using namespace mf;
using namespace mf::transport;

namespace {

PrepareOptions ToPrepare(const py::dict &d)
{
    // {rank: {"nic": "ip:port", "role": 0, "keys": [(token, addr, size, access, flags), ...]}}
    PrepareOptions out;
    for (auto item : d) {
        RankInfo info;
        py::dict rec = item.second.cast<py::dict>();
        if (rec.contains("nic")) {
            info.nic = rec["nic"].cast<std::string>();
        }
        if (rec.contains("role")) {
            info.role = (hybm::Role)rec["role"].cast<uint32_t>();
        }
        if (rec.contains("keys")) {
            for (auto k : rec["keys"].cast<py::list>()) {
                py::tuple t = k.cast<py::tuple>();
                MemoryKey key;
                key.token = t[0].cast<uint64_t>();
                key.addr = t[1].cast<uint64_t>();
                key.size = t[2].cast<uint64_t>();
                key.access = t[3].cast<uint32_t>();
                key.flags = t[4].cast<uint32_t>();
                info.keys.push_back(key);
            }
        }
        out.ranks[item.first.cast<uint32_t>()] = std::move(info);
    }
    return out;
}

}  // namespace

void BindTransport(py::module_ &m)
{
    py::module_ n = m.attr("native").cast<py::module_>();
    n.attr("TT_DEVICE_PEER") = (uint32_t)TT_DEVICE_PEER;
    n.attr("TT_HOST_TCP") = (uint32_t)TT_HOST_TCP;
    n.attr("TT_COMPOSE") = (uint32_t)TT_COMPOSE;
    n.attr("MR_FLAG_DRAM") = MR_FLAG_DRAM;
    n.attr("MR_FLAG_HBM") = MR_FLAG_HBM;
    n.attr("MR_ACCESS_REMOTE_WRITE") = MR_ACCESS_REMOTE_WRITE;
    n.attr("MR_ACCESS_REMOTE_READ") = MR_ACCESS_REMOTE_READ;
    n.attr("MR_ACCESS_ALL") = MR_ACCESS_ALL;

    py::class_<TransportManager, std::shared_ptr<TransportManager>>(n, "Transport")
        .def(py::init([](uint32_t type) { return TransportManager::Create((TransportType)type); }), py::arg("type"))
        .def("open", [](TransportManager &t, uint32_t rank, uint32_t count, uint32_t role, const std::string &nic, uint32_t workers,
                        uint64_t sliceBytes, int64_t opTimeoutMs, const std::string &tlsInfo, const std::string &tlsPk) {
            Options o;
            o.rankId = rank;
            o.rankCount = count;
            o.role = (hybm::Role)role;
            o.nic = nic;
            o.workers = workers;
            o.sliceBytes = sliceBytes;
            o.opTimeoutMs = opTimeoutMs;
            if (!tlsInfo.empty()) {
                std::string err;
                if (!net::ParseTlsInfo(tlsInfo, &o.tls, &err)) {
                    throw std::invalid_argument(err);
                }
                o.tls.enable = true;
                o.tls.pk = tlsPk;
            }
            py::gil_scoped_release nogil;
            return t.OpenDevice(o);
        }, py::arg("rank"), py::arg("rank_count"), py::arg("role") = 0, py::arg("nic") = "127.0.0.1:0", py::arg("workers") = 4,
           py::arg("slice_bytes") = 4u << 20, py::arg("op_timeout_ms") = 30000, py::arg("tls_info") = "", py::arg("tls_pk") = "")
        .def("close", &TransportManager::CloseDevice, py::call_guard<py::gil_scoped_release>())
        .def("nic", &TransportManager::GetNic)
        .def("register_region", [](TransportManager &t, uint64_t addr, uint64_t size, uint32_t access, uint32_t flags) {
            MemoryRegion mr;
            mr.addr = addr;
            mr.size = size;
            mr.access = access;
            mr.flags = flags;
            return t.RegisterMemoryRegion(mr);
        }, py::arg("addr"), py::arg("size"), py::arg("access") = MR_ACCESS_ALL, py::arg("flags") = MR_FLAG_DRAM)
        .def("unregister_region", &TransportManager::UnregisterMemoryRegion, py::call_guard<py::gil_scoped_release>())
        .def("has_registered", &TransportManager::QueryHasRegistered)
        .def("memory_key", [](TransportManager &t, uint64_t addr) -> py::object {
            MemoryKey k;
            if (t.QueryMemoryKey(addr, &k) != 0) {
                return py::none();
            }
            return py::make_tuple(k.token, k.addr, k.size, k.access, k.flags);
        })
        .def("prepare", [](TransportManager &t, const py::dict &d) { return t.Prepare(ToPrepare(d)); })
        .def("update_ranks", [](TransportManager &t, const py::dict &d) {
            PrepareOptions o = ToPrepare(d);
            py::gil_scoped_release nogil;
            return t.UpdateRankOptions(o);
        })
        .def("remove_ranks", &TransportManager::RemoveRanks, py::call_guard<py::gil_scoped_release>())
        .def("connect", &TransportManager::Connect, py::call_guard<py::gil_scoped_release>())
        .def("async_connect", &TransportManager::AsyncConnect, py::call_guard<py::gil_scoped_release>())
        .def("wait_connected", &TransportManager::WaitForConnected, py::arg("timeout_ns") = -1, py::call_guard<py::gil_scoped_release>())
        .def("write", &TransportManager::WriteRemote, py::arg("rank"), py::arg("local"), py::arg("remote"), py::arg("size"),
             py::call_guard<py::gil_scoped_release>())
        .def("read", &TransportManager::ReadRemote, py::arg("rank"), py::arg("local"), py::arg("remote"), py::arg("size"),
             py::call_guard<py::gil_scoped_release>())
        .def("write_async", &TransportManager::WriteRemoteAsync, py::call_guard<py::gil_scoped_release>())
        .def("read_async", &TransportManager::ReadRemoteAsync, py::call_guard<py::gil_scoped_release>())
        .def("write_batch_async", [](TransportManager &t, uint32_t rank, std::vector<uint64_t> local, std::vector<uint64_t> remote,
                                     std::vector<uint64_t> sizes) {
            CopyBatch b{std::move(local), std::move(remote), std::move(sizes)};
            py::gil_scoped_release nogil;
            return t.WriteRemoteBatchAsync(rank, b);
        })
        .def("read_batch_async", [](TransportManager &t, uint32_t rank, std::vector<uint64_t> local, std::vector<uint64_t> remote,
                                    std::vector<uint64_t> sizes) {
            CopyBatch b{std::move(local), std::move(remote), std::move(sizes)};
            py::gil_scoped_release nogil;
            return t.ReadRemoteBatchAsync(rank, b);
        })
        .def("synchronize", &TransportManager::Synchronize, py::call_guard<py::gil_scoped_release>())
        .def("stats", [](TransportManager &t) -> py::dict {
            py::dict d;
            HostTcpTransport *h = dynamic_cast<HostTcpTransport *>(&t);
            if (auto *c = dynamic_cast<ComposeTransport *>(&t)) {
                h = c->Host().get();
            }
            if (h != nullptr) {
                const HostTcpStats &s = h->Stats();
                d["bytes_written"] = s.bytesWritten.load();
                d["bytes_read"] = s.bytesRead.load();
                d["bytes_served"] = s.bytesServed.load();
                d["slices"] = s.slices.load();
                d["reconnects"] = s.reconnects.load();
                d["refused"] = s.refused.load();
            }
            return d;
        })
        .def("linked", [](TransportManager &t, uint32_t rank) {
            HostTcpTransport *h = dynamic_cast<HostTcpTransport *>(&t);
            if (auto *c = dynamic_cast<ComposeTransport *>(&t)) {
                h = c->Host().get();
            }
            return h != nullptr && h->Linked(rank);
        })
        .def("route_of", [](TransportManager &t, uint32_t rank, uint64_t addr, uint64_t size) -> int {
            auto *c = dynamic_cast<ComposeTransport *>(&t);
            return c == nullptr ? -1 : (int)c->RouteOf(rank, addr, size);
        })
        // Device transport and compose: copies between addresses this process can dereference are done by this callable
        // (dst, src, size, is_async) -> int; tests pass a ctypes.memmove wrapper, the entity passes its copy kernel.
        .def("set_device_hooks", [](TransportManager &t, py::object mapPeer, py::object unmapPeer, py::object copy) {
            DevicePeerTransport *d = dynamic_cast<DevicePeerTransport *>(&t);
            if (auto *c = dynamic_cast<ComposeTransport *>(&t)) {
                d = c->Device().get();
            }
            if (d == nullptr) {
                return -1;
            }
            DeviceHooks h;
            auto wrap1 = [](py::object fn) -> std::function<int(uint32_t)> {
                if (fn.is_none()) {
                    return nullptr;
                }
                auto holder = std::make_shared<py::object>(fn);
                return [holder](uint32_t r) {
                    py::gil_scoped_acquire gil;
                    return (*holder)(r).cast<int>();
                };
            };
            h.mapPeer = wrap1(mapPeer);
            h.unmapPeer = wrap1(unmapPeer);
            if (!copy.is_none()) {
                auto holder = std::make_shared<py::object>(copy);
                h.copy = [holder](uint64_t dst, uint64_t src, uint64_t size, bool async) {
                    py::gil_scoped_acquire gil;
                    return (*holder)(dst, src, size, async).cast<int>();
                };
            }
            d->SetHooks(std::move(h));
            return 0;
        }, py::arg("map_peer") = py::none(), py::arg("unmap_peer") = py::none(), py::arg("copy") = py::none())
        .def("links", [](TransportManager &t) -> py::list {
            py::list out;
            DevicePeerTransport *d = dynamic_cast<DevicePeerTransport *>(&t);
            if (auto *c = dynamic_cast<ComposeTransport *>(&t)) {
                d = c->Device().get();
            }
            if (d != nullptr) {
                for (const PeerLink &l : d->Links().Snapshot()) {
                    py::dict e;
                    e["rank"] = l.rank;
                    e["role"] = (uint32_t)l.role;
                    e["state"] = std::string(LinkStateName(l.state));
                    e["same_host"] = l.sameHost;
                    e["slices"] = l.slices;
                    e["bytes"] = l.bytes;
                    e["changes"] = l.changes;
                    out.append(e);
                }
            }
            return out;
        });

    n.def("role_permits_link", [](uint32_t mine, uint32_t theirs) { return RolePermitsLink((hybm::Role)mine, (hybm::Role)theirs); });
    n.def("is_valid_ipv4", &util::IsValidIpv4, py::arg("text"), py::arg("allow_any") = false);
    n.def("ipv4_in_cidr", &util::Ipv4InCidr);
}

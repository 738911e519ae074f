// `native` submodule: direct access to control-plane classes (store server/client, prefix store, group engine, VA
// manager, tag rules) and to raw kernel launchers. Used by the test-suite and the benchmarks; applications use bm/shm/
// TransferEngine.
#include <pybind11/functional.h>
#include <pybind11/stl.h>

#include <cstring>
#include <map>

#include "../group/mf_group.h"
#include "../net/mf_tls.h"
#include "../hybm/mf_cuda.h"
#include "../hybm/mf_data_op.h"
#include "../hybm/mf_range_pool.h"
#include "../hybm/mf_tag_info.h"
#include "../util/mf_log.h"
#include "../util/mf_retry.h"
#include "../util/mf_tracer.h"
#include "../hybm/mf_va_manager.h"
#include "../kernels/mf_kernels.h"
#include "../kernels/mf_xcopy_noalloc.h"
#include "../net/mf_rpc.h"
#include "../store/mf_store_client.h"
#include "pymf_parts.h"

namespace py = pybind11;
using namespace mf;

namespace {

net::Endpoint Ep(const std::string &host, int port)
{
    net::Endpoint ep;
    ep.host = host;
    ep.port = (uint16_t)port;
    ep.v6 = host.find(':') != std::string::npos;
    return ep;
}

struct PyServer {
    store::StoreServer s;
};

// The last reference to a Python callable may be dropped on a native thread: take the GIL for the decref.
std::shared_ptr<py::function> HoldPy(py::function fn)
{
    return std::shared_ptr<py::function>(new py::function(std::move(fn)), [](py::function *p) {
        py::gil_scoped_acquire gil;
        delete p;
    });
}

// Python callbacks are invoked from native threads: take the GIL, never let an exception escape.
template <typename... A>
std::function<void(A...)> WrapCb(py::function fn)
{
    auto holder = HoldPy(std::move(fn));
    return [holder](A... a) {
        py::gil_scoped_acquire gil;
        try {
            (*holder)(a...);
        } catch (py::error_already_set &e) {
            e.discard_as_unraisable("memfabric callback");
        }
    };
}

}  // namespace

void BindNative(py::module_ &m)
{
    py::module_ n = m.def_submodule("native", "control-plane classes and raw kernel launchers");

    n.def("parse_url", [](const std::string &url) -> py::object {
        net::Endpoint ep;
        if (!net::ParseUrl(url, &ep)) {
            return py::none();
        }
        return py::make_tuple(ep.host, (int)ep.port, ep.v6);
    });
    n.def("set_heartbeat_ms", [](uint32_t ms, uint32_t missLimit) {
        store::GlobalTiming().heartbeatIntervalMs = ms;
        store::GlobalTiming().heartbeatMissLimit = missLimit;
    }, py::arg("interval_ms"), py::arg("miss_limit") = 3);
    n.def("pack_message", [](int64_t userDef, std::vector<std::string> keys, std::vector<py::bytes> values) {
        store::StoreMessage msg;
        msg.userDef = userDef;
        msg.keys = std::move(keys);
        for (auto &v : values) {
            msg.values.push_back(std::string(v));
        }
        return py::bytes(store::PackMessage(msg));
    });
    n.def("unpack_message", [](py::bytes buf) -> py::object {
        store::StoreMessage msg;
        if (!store::UnpackMessage(std::string(buf), &msg)) {
            return py::none();
        }
        std::vector<py::bytes> vals;
        for (auto &v : msg.values) {
            vals.emplace_back(v);
        }
        return py::make_tuple(msg.userDef, msg.keys, vals);
    });

    py::class_<PyServer>(n, "StoreServer")
        .def(py::init<>())
        .def("start", [](PyServer &s, const std::string &host, int port, uint32_t world) { return s.s.Start(Ep(host, port), world); }, py::arg("host"),
             py::arg("port"), py::arg("world_size") = 0, py::call_guard<py::gil_scoped_release>())
        .def("stop", [](PyServer &s) { s.s.Stop(); }, py::call_guard<py::gil_scoped_release>())
        .def("port", [](PyServer &s) { return (int)s.s.Port(); })
        .def("alive_links", [](PyServer &s) { return s.s.AliveLinks(); })
        .def("size", [](PyServer &s) { return s.s.Backend()->Size(); })
        .def("set_mute", [](PyServer &s, bool mute) { s.s.SetMute(mute); });

    py::class_<store::ConfigStore, store::StorePtr>(n, "ConfigStore")
        .def("set", [](store::ConfigStore &s, const std::string &k, const std::string &v) { return s.Set(k, v); }, py::call_guard<py::gil_scoped_release>())
        .def("get", [](store::ConfigStore &s, const std::string &k, int64_t timeoutMs) {
            std::string v;
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = s.Get(k, &v, timeoutMs);
            }
            return py::make_tuple(rc, py::bytes(v));
        }, py::arg("key"), py::arg("timeout_ms") = -1)
        .def("add", [](store::ConfigStore &s, const std::string &k, int64_t d) {
            int64_t nv = 0;
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = s.Add(k, d, &nv);
            }
            return py::make_tuple(rc, nv);
        })
        .def("remove", [](store::ConfigStore &s, const std::string &k) { return s.Remove(k, true); }, py::call_guard<py::gil_scoped_release>())
        .def("append", [](store::ConfigStore &s, const std::string &k, py::bytes v) {
            uint64_t sz = 0;
            std::string val(v);
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = s.Append(k, val, &sz);
            }
            return py::make_tuple(rc, sz);
        })
        .def("arrive", [](store::ConfigStore &s, const std::string &counter, const std::string &wake, uint32_t expected, int64_t timeoutMs,
                          const std::vector<std::string> &gc) {
            int64_t arrived = 0;
            py::gil_scoped_release nogil;
            return s.Arrive(counter, wake, expected, timeoutMs, gc, &arrived);
        }, py::arg("counter_key"), py::arg("wake_key"), py::arg("expected"), py::arg("timeout_ms"), py::arg("gc_keys") = std::vector<std::string>())
        .def("gather", [](store::ConfigStore &s, const std::string &data, const std::string &wake, py::bytes record, uint64_t fullSize,
                          int64_t timeoutMs, const std::vector<std::string> &gc) {
            std::string rec(record), all;
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = s.Gather(data, wake, rec, fullSize, timeoutMs, gc, &all);
            }
            return py::make_tuple(rc, py::bytes(all));
        }, py::arg("data_key"), py::arg("wake_key"), py::arg("record"), py::arg("full_size"), py::arg("timeout_ms"),
           py::arg("gc_keys") = std::vector<std::string>())
        .def("cas", [](store::ConfigStore &s, const std::string &k, py::bytes expect, py::bytes exchange) {
            std::string prev, e(expect), x(exchange);
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = s.Cas(k, e, x, &prev);
            }
            return py::make_tuple(rc, py::bytes(prev));
        })
        .def("write", [](store::ConfigStore &s, const std::string &k, const std::string &v, uint32_t off) { return s.Write(k, v, off); },
             py::call_guard<py::gil_scoped_release>())
        .def("watch", [](store::ConfigStore &s, const std::string &k, py::function cb) {
            auto f = WrapCb<int, std::string, py::bytes>(std::move(cb));
            uint32_t wid = 0;
            int rc = s.Watch(k, [f](int r, const std::string &key, const std::string &v) {
                py::gil_scoped_acquire gil;
                f(r, key, py::bytes(v));
            }, &wid);
            return py::make_tuple(rc, wid);
        })
        .def("watch_rank_down", [](store::ConfigStore &s, py::function cb) {
            auto f = WrapCb<uint32_t>(std::move(cb));
            uint32_t wid = 0;
            int rc = s.WatchRankDown(f, &wid);
            return py::make_tuple(rc, wid);
        })
        .def("unwatch", [](store::ConfigStore &s, uint32_t wid) { return s.Unwatch(wid); })
        .def("connected", [](store::ConfigStore &s) { return s.Connected(); })
        .def("common_prefix", [](store::ConfigStore &s) { return s.CommonPrefix(); })
        .def("reconnect", [](store::ConfigStore &s, int retries) { return s.ReconnectAfterBroken(retries); }, py::arg("retries") = 3,
             py::call_guard<py::gil_scoped_release>())
        .def("set_broken_handler", [](store::ConfigStore &s, py::function cb) { s.SetBrokenHandler(WrapCb<>(std::move(cb))); })
        .def("set_reconnect_handler", [](store::ConfigStore &s, py::function cb) { s.SetReconnectHandler(WrapCb<>(std::move(cb))); });

    py::class_<store::TcpStore, store::ConfigStore, std::shared_ptr<store::TcpStore>>(n, "TcpStore")
        .def(py::init([](const std::string &host, int port, bool isServer, uint32_t world, int rank) {
                 return std::make_shared<store::TcpStore>(Ep(host, port), isServer, world, rank);
             }),
             py::arg("host"), py::arg("port"), py::arg("is_server") = false, py::arg("world_size") = 0, py::arg("rank") = -1)
        .def("startup", [](store::TcpStore &s, int retries, int delayMs) { return s.Startup(retries, delayMs); }, py::arg("retries") = 60,
             py::arg("retry_delay_ms") = 1000, py::call_guard<py::gil_scoped_release>())
        .def("shutdown", [](store::TcpStore &s) { s.Shutdown(); }, py::call_guard<py::gil_scoped_release>())
        .def("server_port", [](store::TcpStore &s) { return s.Server() ? (int)s.Server()->Port() : 0; })
        .def("server_set_mute", [](store::TcpStore &s, bool mute) {
            if (s.Server()) {
                s.Server()->SetMute(mute);
            }
        })
        .def("set_drop_heartbeat", [](store::TcpStore &s, bool d) { s.SetDropHeartbeat(d); });

    // TLS helpers for tests and operations: does the option text (+ registered key) build a working context, and what does the
    // certificate validity check say (0 fine, 1 expires within ahead_days, -1 expired / unusable)?
    n.def("tls_check_certificates", [](const std::string &info, const std::string &pk, const std::string &pw, int aheadDays) -> py::object {
        net::TlsOptions opt;
        std::string err;
        if (!net::ParseTlsInfo(info, &opt, &err)) {
            return py::make_tuple(-2, err);
        }
        opt.pk = pk;
        opt.pkPwd = pw;
        auto ctx = net::TlsContext::Create(opt, false, &err);
        if (!ctx) {
            return py::make_tuple(-1, err);
        }
        std::string detail;
        int rc = ctx->CheckCertificates(aheadDays, &detail);
        return py::make_tuple(rc, detail);
    }, py::arg("tls_info"), py::arg("tls_pk"), py::arg("tls_pk_pw") = "", py::arg("ahead_days") = 30);
    n.def("tls_cert_check_params", []() {
        int p = 0, d = 0;
        net::CertCheckParams(&p, &d);
        return py::make_tuple(p, d);
    });
    n.def("set_retry_policy", [](uint32_t attempts, uint32_t firstDelayMs, uint32_t factor) {
        RetryPolicy &p = GlobalRetryPolicy();
        p.attempts = attempts == 0 ? 1 : attempts;
        p.firstDelayMs = firstDelayMs;
        p.factor = factor == 0 ? 1 : factor;
    }, py::arg("attempts") = 3, py::arg("first_delay_ms") = 1000, py::arg("factor") = 2);
    n.def("retry_stats", []() { return py::make_tuple(GlobalRetryStats().retries.load(), GlobalRetryStats().gaveUp.load()); });
    n.def("set_server_linger_ms", [](uint32_t ms) { store::GlobalTiming().serverLingerMs = ms; });
    n.def("prefix_store", [](store::StorePtr base, const std::string &prefix) { return store::StoreFactory::PrefixOf(base, prefix); });
    n.def("ha_store", [](store::StorePtr base) { return std::static_pointer_cast<store::ConfigStore>(std::make_shared<store::HaStore>(base)); });

    py::class_<group::GroupEngine, std::shared_ptr<group::GroupEngine>>(n, "GroupEngine")
        .def(py::init([](store::StorePtr st, uint32_t rankSize, uint32_t rank, uint32_t timeoutMs, bool dynamic, py::object joinCb, py::object leaveCb) {
                 group::GroupOption o;
                 o.rankSize = rankSize;
                 o.rank = rank;
                 o.timeoutMs = timeoutMs;
                 o.dynamic = dynamic;
                 auto wrap = [](py::object cb) -> group::RankCallback {
                     if (cb.is_none()) {
                         return nullptr;
                     }
                     auto holder = HoldPy(cb.cast<py::function>());
                     return [holder](uint32_t r) {
                         py::gil_scoped_acquire gil;
                         try {
                             py::object ret = (*holder)(r);
                             return ret.is_none() ? 0 : ret.cast<int>();
                         } catch (py::error_already_set &e) {
                             e.discard_as_unraisable("memfabric group callback");
                             return -1;
                         }
                     };
                 };
                 o.joinCb = wrap(joinCb);
                 o.leaveCb = wrap(leaveCb);
                 auto g = group::GroupEngine::Create(st, o);
                 if (!g) {
                     throw std::runtime_error("invalid group option");
                 }
                 return g;
             }),
             py::arg("store"), py::arg("rank_size"), py::arg("rank"), py::arg("timeout_ms") = 120000, py::arg("dynamic") = false,
             py::arg("join_cb") = py::none(), py::arg("leave_cb") = py::none())
        .def("repairs", &group::GroupEngine::Repairs)
        .def("barrier", &group::GroupEngine::GroupBarrier, py::call_guard<py::gil_scoped_release>())
        .def("allgather", [](group::GroupEngine &g, py::bytes send) {
            std::string s(send);
            std::string recv(s.size() * std::max<uint32_t>(g.RankSize(), 1), '\0');
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = g.GroupAllGather(s.data(), (uint32_t)s.size(), &recv[0], (uint32_t)recv.size());
            }
            return py::make_tuple(rc, py::bytes(recv));
        })
        .def("subgroup_barrier", &group::GroupEngine::SubGroupBarrier, py::call_guard<py::gil_scoped_release>())
        .def("subgroup_allgather", [](group::GroupEngine &g, const std::string &key, uint32_t size, uint32_t rank, py::bytes send) {
            std::string s(send);
            std::string recv(s.size() * size, '\0');
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = g.SubGroupAllGather(key, size, rank, s.data(), (uint32_t)s.size(), &recv[0], (uint32_t)recv.size());
            }
            return py::make_tuple(rc, py::bytes(recv));
        })
        .def("join", &group::GroupEngine::GroupJoin, py::call_guard<py::gil_scoped_release>())
        .def("leave", &group::GroupEngine::GroupLeave, py::call_guard<py::gil_scoped_release>())
        .def("start_listen", &group::GroupEngine::StartListenEvent)
        .def("stop", &group::GroupEngine::Stop, py::call_guard<py::gil_scoped_release>())
        .def("alloc_number", [](group::GroupEngine &g, uint32_t limit) {
            uint32_t v = 0;
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = g.AllocNumber(limit, &v);
            }
            return py::make_tuple(rc, v);
        })
        .def("release_number", &group::GroupEngine::ReleaseNumber, py::call_guard<py::gil_scoped_release>())
        .def("register_exit", [](group::GroupEngine &g, py::function cb) { return g.RegisterExit(WrapCb<int>(std::move(cb))); })
        .def("broadcast_exit", &group::GroupEngine::GroupBroadcastExit, py::call_guard<py::gil_scoped_release>())
        .def("rank_size", &group::GroupEngine::RankSize)
        .def("version", &group::GroupEngine::Version)
        .def("joined", &group::GroupEngine::Joined)
        .def("members", &group::GroupEngine::Members);

    // ---- pure-logic helpers
    n.def("va_find_free_window", [](uint64_t size, uint64_t hint) { return hybm::VaManager::Instance().FindFreeWindow(size, hint); }, py::arg("size"),
          py::arg("hint") = 0);
    n.def("va_add_reserved", [](uint64_t base, uint64_t size, uint32_t entity, uint32_t memType) {
        return hybm::VaManager::Instance().AddReserved(hybm::ReservedRange{base, size, entity, memType});
    });
    n.def("va_remove_reserved", [](uint64_t base) { return hybm::VaManager::Instance().RemoveReserved(base); });
    n.def("va_add_allocated", [](uint64_t gva, uint64_t size, uint32_t memType, uint32_t rank, uint32_t entity, bool imported) {
        hybm::AllocatedRange a;
        a.gva = gva;
        a.size = size;
        a.memType = memType;
        a.ownerRank = rank;
        a.entityId = entity;
        a.imported = imported;
        return hybm::VaManager::Instance().AddAllocated(a);
    });
    n.def("va_remove_allocated", [](uint64_t gva) { return hybm::VaManager::Instance().RemoveAllocated(gva); });
    n.def("va_find_allocated", [](uint64_t addr, uint64_t len) -> py::object {
        hybm::AllocatedRange a;
        if (!hybm::VaManager::Instance().FindAllocated(addr, len, &a)) {
            return py::none();
        }
        return py::make_tuple(a.gva, a.size, a.memType, a.ownerRank, a.entityId, a.imported);
    });
    n.def("va_classify", [](uint64_t addr) { return (int)hybm::VaManager::Instance().Classify(addr); });
    n.def("va_direction", [](int s, int d) { return (int)hybm::DirectionOf((hybm::PtrClass)s, (hybm::PtrClass)d); });
    n.def("va_direction_name", [](int d) { return std::string(hybm::DirectionName((hybm::CopyDirection)d)); });
    n.def("va_dump", []() { return hybm::VaManager::Instance().Dump(); });
    n.def("va_info", [](uint64_t addr) { return hybm::VaManager::Instance().VaToInfo(addr); });
    n.def("va_clear", []() { hybm::VaManager::Instance().Clear(); });
    n.def("slice_handle", [](uint16_t index, uint32_t memType) {
        hybm::MemSlice s;
        s.index = index;
        s.memType = memType;
        return s.ToHandle();
    });
    n.def("slice_decode", [](uint64_t h) -> py::object {
        uint16_t idx;
        uint32_t mt;
        if (!hybm::MemSlice::Decode(h, &idx, &mt)) {
            return py::none();
        }
        return py::make_tuple(idx, mt);
    });

    py::class_<hybm::RangePool>(n, "RangePool")
        .def(py::init<uint64_t, uint64_t, uint64_t>(), py::arg("base"), py::arg("size"), py::arg("align") = 256)
        .def("allocate", &hybm::RangePool::Allocate)
        .def("release", &hybm::RangePool::Release)
        .def("in_use", &hybm::RangePool::InUse)
        .def("capacity", &hybm::RangePool::Capacity)
        .def("largest_free", &hybm::RangePool::LargestFree)
        .def("free_blocks", &hybm::RangePool::FreeBlocks);
    n.def("trace_point", [](int tp, const std::string &name, int ret, uint64_t busyNs) {
        // Records one begin/end pair on tracepoint `tp` (test hook for the aggregate tracer).
        static std::map<int, std::string> names;
        auto it = names.emplace(tp, name).first;
        Tracer::Instance().Begin(tp, it->second.c_str());
        Tracer::Instance().End(tp, NowNs() - busyNs, ret);
    });
    n.def("trace_query", [](int tp) -> py::object {
        uint64_t v[4];
        if (!Tracer::Instance().Query(tp, v)) {
            return py::none();
        }
        return py::make_tuple(v[0], v[1], v[2], v[3]);
    });

    py::class_<hybm::TagInfo, std::shared_ptr<hybm::TagInfo>>(n, "TagInfo")
        .def(py::init<>())
        .def("init", &hybm::TagInfo::Init)
        .def("add_rank_tag", &hybm::TagInfo::AddRankTag)
        .def("remove_rank_tag", &hybm::TagInfo::RemoveRankTag)
        .def("tag_of", &hybm::TagInfo::TagOf)
        .def("allowed_ops", &hybm::TagInfo::AllowedOps)
        .def_static("valid_tag", &hybm::TagInfo::ValidTag)
        .def_static("op_type_from_name", &hybm::TagInfo::OpTypeFromName);

    // Names of the engines the composite data operator would try, in order (exposed to test the selection policy).
    n.def("compose_candidates", [](int device, uint32_t allowed, int dir, uint64_t bytes, bool batch, bool srcVisible, bool dstVisible, uint32_t flags) {
        hybm::ComposeDataOp op(device, allowed, nullptr);
        op.Initialize();
        hybm::ExtOptions o;
        o.srcDeviceVisible = srcVisible;
        o.dstDeviceVisible = dstVisible;
        o.flags = flags;
        std::vector<std::string> names;
        for (auto &e : op.Candidates((hybm::CopyDirection)dir, o, bytes, batch)) {
            names.emplace_back(e->Name());
        }
        return names;
    });

    // ---- CUDA
    n.def("cuda_available", []() { return cu::Available(); });
    n.def("device_count", []() { return cu::DeviceCount(); });
    n.def("device_caps", [](int dev) -> py::object {
        cu::DeviceCaps c;
        if (cu::ProbeDevice(dev, &c) != 0) {
            return py::none();
        }
        py::dict d;
        d["vmm"] = c.vmm;
        d["posix_fd"] = c.posixFdHandle;
        d["fabric"] = c.fabricHandle;
        d["multicast"] = c.multicast;
        d["host_numa_vmm"] = c.hostNumaVmm;
        d["host_ptr_for_registered"] = c.hostPtrForRegistered;
        d["numa_node"] = c.numaNode;
        d["sm_count"] = c.smCount;
        d["driver"] = c.driverVersion;
        d["runtime"] = c.runtimeVersion;
        return d;
    });
    n.def("data_op_stats", []() {
        hybm::DataOpStats st = hybm::GetDataOpStats();
        py::dict d;
        d["kernel_calls"] = st.kernelCalls;
        d["kernel_elems"] = st.kernelElems;
        d["copy_engine_calls"] = st.copyEngineCalls;
        d["copy_engine_elems"] = st.copyEngineElems;
        d["cpu_calls"] = st.cpuCalls;
        d["cpu_elems"] = st.cpuElems;
        d["batch_groups_last"] = st.batchGroupsLast;
        d["remote_calls"] = st.remoteCalls;
        d["remote_elems"] = st.remoteElems;
        return d;
    });
    n.def("xcopy", [](uint64_t dst, uint64_t src, uint64_t nbytes, int ctas, uint64_t stream) {
        return mf_k_xcopy((void *)dst, (const void *)src, nbytes, ctas, (mf_stream_t)stream);
    }, py::arg("dst"), py::arg("src"), py::arg("nbytes"), py::arg("ctas") = 0, py::arg("stream") = 0);
    n.def("xcopy_shaped", [](uint64_t dst, uint64_t src, uint64_t nbytes, uint32_t tile, uint32_t stages, uint32_t inflight, uint32_t blocked,
                             int ctas, uint64_t stream) {
        return mf_k_xcopy_shaped((void *)dst, (const void *)src, nbytes, tile, stages, inflight, blocked, ctas, (mf_stream_t)stream);
    }, py::arg("dst"), py::arg("src"), py::arg("nbytes"), py::arg("tile"), py::arg("stages"), py::arg("inflight"), py::arg("blocked") = 0,
       py::arg("ctas") = 0, py::arg("stream") = 0);
    n.def("copy_engine", [](uint64_t dst, uint64_t src, uint64_t nbytes, uint64_t stream) {
        return mf_k_memcpy_async((void *)dst, (const void *)src, nbytes, (mf_stream_t)stream);
    }, py::arg("dst"), py::arg("src"), py::arg("nbytes"), py::arg("stream") = 0);
    n.def("batch_xcopy_inline", [](std::vector<uint64_t> srcs, std::vector<uint64_t> dsts, std::vector<uint64_t> sizes, int ctas, uint64_t stream) {
        std::vector<mf_copy_desc_t> d;
        uint32_t chunks = 0;
        for (size_t i = 0; i < sizes.size(); i++) {
            d.push_back(mf_copy_desc_t{srcs[i], dsts[i], (uint32_t)sizes[i], chunks});
            chunks += (uint32_t)((sizes[i] + MF_BATCH_CHUNK_BYTES - 1) / MF_BATCH_CHUNK_BYTES);
        }
        if (d.size() > MF_BATCH_INLINE_MAX) {
            return (int)MF_K_TOO_LARGE;
        }
        return mf_k_batch_xcopy(d.data(), nullptr, (uint32_t)d.size(), chunks, nullptr, nullptr, 0, ctas, (mf_stream_t)stream);
    }, py::arg("srcs"), py::arg("dsts"), py::arg("sizes"), py::arg("ctas") = 0, py::arg("stream") = 0);
    // Any number of copies up to the limits of the allocation-free entry point; tables longer than the inline limit run
    // through the table kernel.
    n.def("batch_xcopy_noalloc", [](std::vector<uint64_t> srcs, std::vector<uint64_t> dsts, std::vector<uint64_t> sizes, uint64_t stream) {
        if (srcs.size() != dsts.size() || srcs.size() != sizes.size()) {
            return (int)MF_K_INVALID;
        }
        return mf_batch_xcopy_noalloc(srcs.data(), dsts.data(), sizes.data(), (uint32_t)srcs.size(), (void *)stream);
    }, py::arg("srcs"), py::arg("dsts"), py::arg("sizes"), py::arg("stream") = 0);
    n.def("fill_pattern", [](uint64_t dst, uint64_t nbytes, uint64_t seed, uint64_t stream) {
        return mf_k_fill_pattern((void *)dst, nbytes, seed, (mf_stream_t)stream);
    }, py::arg("dst"), py::arg("nbytes"), py::arg("seed"), py::arg("stream") = 0);
    n.def("check_pattern", [](uint64_t buf, uint64_t nbytes, uint64_t seed, uint64_t mismatchPtr, uint64_t stream) {
        return mf_k_check_pattern((const void *)buf, nbytes, seed, (unsigned long long *)mismatchPtr, (mf_stream_t)stream);
    }, py::arg("buf"), py::arg("nbytes"), py::arg("seed"), py::arg("mismatch_ptr"), py::arg("stream") = 0);
    n.def("checksum", [](uint64_t buf, uint64_t nbytes, uint64_t outPtr, uint64_t stream) {
        return mf_k_checksum((const void *)buf, nbytes, (unsigned long long *)outPtr, (mf_stream_t)stream);
    }, py::arg("buf"), py::arg("nbytes"), py::arg("out_ptr"), py::arg("stream") = 0);
    n.def("pattern_bytes", [](uint64_t seed, uint64_t start, uint64_t count) {
        std::string s(count, '\0');
        for (uint64_t i = 0; i < count; i++) {
            s[i] = (char)mf_k_pattern_byte_host(seed, start + i);
        }
        return py::bytes(s);
    });
    n.def("checksum_host", [](py::bytes b) {
        std::string s(b);
        return mf_k_checksum_host(s.data(), s.size());
    });
    // Raw host memory helpers for tests that run without torch tensors (addresses are ints).
    n.def("host_write", [](uint64_t addr, py::bytes b) {
        std::string s(b);
        std::memcpy((void *)addr, s.data(), s.size());
    });
    n.def("host_read", [](uint64_t addr, uint64_t nbytes) { return py::bytes((const char *)addr, nbytes); });
}

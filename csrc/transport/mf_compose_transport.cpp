#include "mf_compose_transport.h"

#include "../util/mf_log.h"

namespace mf {
namespace transport {

using hybm::BM_INVALID_PARAM;
using hybm::BM_OK;

ComposeTransport::ComposeTransport() : device_(std::make_shared<DevicePeerTransport>()), host_(std::make_shared<HostTcpTransport>()) {}

ComposeTransport::ComposeTransport(std::shared_ptr<DevicePeerTransport> device, std::shared_ptr<HostTcpTransport> host)
    : device_(std::move(device)), host_(std::move(host))
{
}

int ComposeTransport::OpenDevice(const Options &opt)
{
    self_ = opt.rankId;
    int rc = device_->OpenDevice(opt);
    if (rc != BM_OK) {
        return rc;
    }
    rc = host_->OpenDevice(opt);
    if (rc != BM_OK) {
        device_->CloseDevice();
    }
    return rc;
}

int ComposeTransport::CloseDevice()
{
    int a = device_->CloseDevice();
    int b = host_->CloseDevice();
    return a != BM_OK ? a : b;
}

int ComposeTransport::RegisterMemoryRegion(const MemoryRegion &mr)
{
    if ((mr.flags & (MR_FLAG_HBM | MR_FLAG_DRAM)) == 0) {
        MF_ERROR("compose transport: a region must say whether it is device or host memory");
        return BM_INVALID_PARAM;
    }
    if ((mr.flags & MR_FLAG_HBM) == 0) {
        return host_->RegisterMemoryRegion(mr);
    }
    int rc = device_->RegisterMemoryRegion(mr);
    if (rc == BM_OK && serveDeviceMemory_) {
        // Ranks on other hosts reach this device memory through the host transport's staging copier.
        rc = host_->RegisterMemoryRegion(mr);
        if (rc != BM_OK) {
            device_->UnregisterMemoryRegion(mr.addr);
        }
    }
    return rc;
}

int ComposeTransport::UnregisterMemoryRegion(uint64_t addr)
{
    if (device_->QueryHasRegistered(addr, 1)) {
        if (host_->QueryHasRegistered(addr, 1)) {
            host_->UnregisterMemoryRegion(addr);
        }
        return device_->UnregisterMemoryRegion(addr);
    }
    return host_->UnregisterMemoryRegion(addr);
}

bool ComposeTransport::QueryHasRegistered(uint64_t addr, uint64_t size)
{
    return device_->QueryHasRegistered(addr, size) || host_->QueryHasRegistered(addr, size);
}

int ComposeTransport::QueryMemoryKey(uint64_t addr, MemoryKey *key)
{
    // The host transport's key carries the token a request over the wire must present; device-only regions have none.
    return host_->QueryMemoryKey(addr, key) == BM_OK ? BM_OK : device_->QueryMemoryKey(addr, key);
}

void ComposeTransport::Split(const PrepareOptions &in, PrepareOptions *device, PrepareOptions *host)
{
    for (const auto &kv : in.ranks) {
        RankInfo d, h;
        d.nic = h.nic = kv.second.nic;
        d.role = h.role = kv.second.role;
        d.sameHost = h.sameHost = kv.second.sameHost;
        for (const auto &k : kv.second.keys) {
            // Device memory of a rank on this host is reached through the mapping; everything else over the wire (the
            // owner's host transport stages its device memory).
            (((k.flags & MR_FLAG_HBM) && kv.second.sameHost) ? d : h).keys.push_back(k);
        }
        device->ranks[kv.first] = std::move(d);
        if (!kv.second.nic.empty()) {
            host->ranks[kv.first] = std::move(h);  // a rank without an address serves no host memory over the wire
        }
    }
}

int ComposeTransport::Prepare(const PrepareOptions &opt)
{
    PrepareOptions d, h;
    Split(opt, &d, &h);
    {
        util::WriteGuard g(mu_);
        ranks_ = opt.ranks;
    }
    int rc = device_->Prepare(d);
    return rc != BM_OK ? rc : host_->Prepare(h);
}

int ComposeTransport::UpdateRankOptions(const PrepareOptions &opt)
{
    PrepareOptions d, h;
    Split(opt, &d, &h);
    {
        util::WriteGuard g(mu_);
        for (const auto &kv : opt.ranks) {
            ranks_[kv.first] = kv.second;
        }
    }
    int rc = device_->UpdateRankOptions(d);
    return rc != BM_OK ? rc : host_->UpdateRankOptions(h);
}

int ComposeTransport::RemoveRanks(const std::vector<uint32_t> &ranks)
{
    {
        util::WriteGuard g(mu_);
        for (uint32_t r : ranks) {
            ranks_.erase(r);
        }
    }
    device_->RemoveRanks(ranks);
    return host_->RemoveRanks(ranks);
}

int ComposeTransport::Connect()
{
    int rc = device_->Connect();
    int rh = host_->Connect();
    return rc != BM_OK ? rc : rh;
}

int ComposeTransport::AsyncConnect()
{
    int rc = device_->AsyncConnect();
    return rc != BM_OK ? rc : host_->AsyncConnect();
}

int ComposeTransport::WaitForConnected(int64_t timeoutNs)
{
    int rc = device_->WaitForConnected(timeoutNs);
    int rh = host_->WaitForConnected(timeoutNs);
    return rc != BM_OK ? rc : rh;
}

TransportManager *ComposeTransport::Pick(uint32_t rankId, uint64_t remoteAddr, uint64_t size)
{
    if (rankId == self_) {
        if (device_->QueryHasRegistered(remoteAddr, size)) {
            return device_.get();
        }
        return host_->QueryHasRegistered(remoteAddr, size) ? host_.get() : nullptr;
    }
    util::ReadGuard g(mu_);
    auto it = ranks_.find(rankId);
    if (it == ranks_.end()) {
        return nullptr;
    }
    for (const auto &k : it->second.keys) {
        if (k.Covers(remoteAddr, size)) {
            return ((k.flags & MR_FLAG_HBM) && it->second.sameHost) ? (TransportManager *)device_.get() : (TransportManager *)host_.get();
        }
    }
    return nullptr;
}

TransportType ComposeTransport::RouteOf(uint32_t rankId, uint64_t remoteAddr, uint64_t size)
{
    TransportManager *t = Pick(rankId, remoteAddr, size);
    if (t == nullptr) {
        return TT_COMPOSE;
    }
    return t == device_.get() ? TT_DEVICE_PEER : TT_HOST_TCP;
}

#define MF_COMPOSE_ROUTE(call)                                                                                                      \
    TransportManager *t = Pick(rankId, remoteAddr, size);                                                                           \
    if (t == nullptr) {                                                                                                             \
        MF_ERROR("compose transport: rank " << rankId << " registered nothing that covers 0x" << std::hex << remoteAddr << "+0x" << size \
                                            << std::dec);                                                                           \
        return BM_INVALID_PARAM;                                                                                                    \
    }                                                                                                                               \
    return t->call(rankId, localAddr, remoteAddr, size)

int ComposeTransport::ReadRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) { MF_COMPOSE_ROUTE(ReadRemote); }
int ComposeTransport::WriteRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) { MF_COMPOSE_ROUTE(WriteRemote); }
int ComposeTransport::ReadRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) { MF_COMPOSE_ROUTE(ReadRemoteAsync); }
int ComposeTransport::WriteRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) { MF_COMPOSE_ROUTE(WriteRemoteAsync); }
#undef MF_COMPOSE_ROUTE

int ComposeTransport::Synchronize(uint32_t rankId)
{
    int a = device_->Synchronize(rankId);
    int b = rankId == self_ ? BM_OK : host_->Synchronize(rankId);
    if (b == BM_INVALID_PARAM) {
        b = BM_OK;  // the rank serves no host memory over the wire: nothing was queued there
    }
    return a != BM_OK ? a : b;
}

}  // namespace transport
}  // namespace mf

// Router over one device-memory transport and one host-memory transport.
//
// A region goes to the transport of its memory kind (MR_FLAG_HBM / MR_FLAG_DRAM); the rank records handed to Prepare are split
// the same way, so each child only sees the keys it can serve; a one-sided operation goes to whichever child holds a key of
// that rank covering the remote address. Synchronize waits on both. Role of the reference's compose manager
// (src/hybm/csrc/transport/compose/compose_transport_manager.cpp: region routing by flag, key halves per child, operation
// routing by address lookup).
#pragma once
#include "mf_host_tcp_transport.h"
#include "mf_peer_link_manager.h"
#include "mf_transport.h"

namespace mf {
namespace transport {

class ComposeTransport : public TransportManager {
public:
    ComposeTransport();
    ComposeTransport(std::shared_ptr<DevicePeerTransport> device, std::shared_ptr<HostTcpTransport> host);
    std::shared_ptr<DevicePeerTransport> Device() const { return device_; }
    std::shared_ptr<HostTcpTransport> Host() const { return host_; }

    int OpenDevice(const Options &opt) override;
    int CloseDevice() override;
    int RegisterMemoryRegion(const MemoryRegion &mr) override;
    int UnregisterMemoryRegion(uint64_t addr) override;
    bool QueryHasRegistered(uint64_t addr, uint64_t size) override;
    int QueryMemoryKey(uint64_t addr, MemoryKey *key) override;
    int Prepare(const PrepareOptions &opt) override;
    int Connect() override;
    int AsyncConnect() override;
    int WaitForConnected(int64_t timeoutNs) override;
    int UpdateRankOptions(const PrepareOptions &opt) override;
    int RemoveRanks(const std::vector<uint32_t> &ranks) override;
    std::string GetNic() const override { return host_->GetNic(); }
    int ReadRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int WriteRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int ReadRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int WriteRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int Synchronize(uint32_t rankId) override;

    // Device regions are also registered with the host transport, whose copier stages them for ranks on other hosts.
    // Needs HostTcpTransport::SetDeviceCopier on Host(). Call before registering regions.
    void ServeDeviceMemoryOverTheWire(bool on) { serveDeviceMemory_ = on; }
    // For an owner that opened the two children itself: tells the router which rank is the local one.
    void SetSelf(uint32_t rankId) { self_ = rankId; }

    // Which child would carry an operation on this remote range: TT_DEVICE_PEER, TT_HOST_TCP, or TT_COMPOSE for "nobody".
    TransportType RouteOf(uint32_t rankId, uint64_t remoteAddr, uint64_t size);

private:
    static void Split(const PrepareOptions &in, PrepareOptions *device, PrepareOptions *host);
    TransportManager *Pick(uint32_t rankId, uint64_t remoteAddr, uint64_t size);
    std::shared_ptr<DevicePeerTransport> device_;
    std::shared_ptr<HostTcpTransport> host_;
    util::RwLock mu_;
    std::unordered_map<uint32_t, RankInfo> ranks_;
    uint32_t self_{0};
    bool serveDeviceMemory_{false};
};

}  // namespace transport
}  // namespace mf

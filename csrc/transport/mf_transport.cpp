#include "mf_transport.h"

#include "mf_compose_transport.h"
#include "mf_host_tcp_transport.h"
#include "mf_peer_link_manager.h"

namespace mf {
namespace transport {

std::shared_ptr<TransportManager> TransportManager::Create(TransportType type)
{
    switch (type) {
        case TT_DEVICE_PEER:
            return std::make_shared<DevicePeerTransport>();
        case TT_HOST_TCP:
            return std::make_shared<HostTcpTransport>();
        case TT_COMPOSE:
            return std::make_shared<ComposeTransport>();
    }
    return nullptr;
}

static int RunBatch(TransportManager *t, uint32_t rankId, const CopyBatch &b, bool write)
{
    if (b.local.size() != b.remote.size() || b.local.size() != b.sizes.size()) {
        return hybm::BM_INVALID_PARAM;
    }
    for (size_t i = 0; i < b.local.size(); i++) {
        int rc = write ? t->WriteRemoteAsync(rankId, b.local[i], b.remote[i], b.sizes[i]) : t->ReadRemoteAsync(rankId, b.local[i], b.remote[i], b.sizes[i]);
        if (rc != hybm::BM_OK) {
            return rc;  // what was queued before still completes; Synchronize reports it
        }
    }
    return hybm::BM_OK;
}

int TransportManager::ReadRemoteBatchAsync(uint32_t rankId, const CopyBatch &batch) { return RunBatch(this, rankId, batch, false); }
int TransportManager::WriteRemoteBatchAsync(uint32_t rankId, const CopyBatch &batch) { return RunBatch(this, rankId, batch, true); }

}  // namespace transport
}  // namespace mf

// Helpers shared by the public API translation units.
#pragma once
#include <algorithm>
#include <cerrno>
#include <string>

#include "../group/mf_group.h"
#include "../hybm/mf_entity.h"
#include "../store/mf_store.h"
#include "../store/mf_store_server.h"

namespace mf {
namespace api {

int MapHybmCode(int rc);
int MapGroupCode(int rc);
// Opens (or returns the cached) store for `url`. tryServe: attempt to host the server first; an address already served
// by somebody else then degrades to a client unless mustServe.
store::StorePtr OpenStore(const std::string &url, bool tryServe, bool mustServe, uint32_t worldSize, int32_t rankId, uint32_t timeoutSec,
                          int *rcOut);
// True if the url's host is an address of this machine.
bool UrlIsLocal(const std::string &url);
// Installs the transfer engine's server-side bookkeeping (which link owns which rank/slot records) on a store server.
void AttachTransFaultHandler(store::StoreServer *server);

// Agrees on one window address among the ranks of a static group: everybody proposes its first free window, the
// maximum wins, everybody tries it; on any failure the search restarts above the failed address.
// reserve(hintHbm, hintDram) must reserve-or-fail without side effects on failure; bases() returns what was reserved.
struct WindowProposal {
    uint64_t hbm;
    uint64_t dram;
    uint32_t ok;
    uint32_t pad;
};

}  // namespace api
}  // namespace mf

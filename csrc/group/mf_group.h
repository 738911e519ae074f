// Group engine: control-plane collectives and membership built only from config-store primitives.
//
// Algorithms follow the reference's SmemNetGroupEngine (src/smem/csrc/net/smem_net_group_engine.cpp):
//   barrier    ADD "<ver>_<sn>_BA"; the last arriver SETs "<ver>_<sn>_BW"; everyone blocking-GETs it (:122-188)
//   allgather  APPEND (rank,payload) to "<ver>_<sn>_GA"; last arriver SETs "_GW"; GET the whole value, sort by rank (:350-436)
//   subgroup   the same under a caller-supplied key with explicit (rankSize, rankId) (:190-269,438-534)
//   join/leave serialised by CAS on "EVENT" ("" → "J<rank>" / "L<rank>"), group (version,size) packed in one
//              counter "DSIZE" = version << 30 | size, a listener thread per member runs the join/leave callbacks
//              so that the collectives inside them line up (:47-87,596-732,907-1014)
//   rank down  store notification → drop the rank locally, leave callback, one member repairs DSIZE (:734-823)
//   numbers    CAS on a 1024-bit bitmap (:536-594); exit broadcast through a watched "EXIT" key (:290-348)
// Keys of round sn-2 are garbage-collected by the first arriver of round sn (:1085-1109).
#pragma once
#include <atomic>
#include <bitset>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../store/mf_store.h"

namespace mf {
namespace group {

constexpr uint32_t GROUP_RANK_MAX = 1024;
constexpr uint32_t GROUP_NUMBER_MAX = 1024;
constexpr uint32_t GROUP_ALLGATHER_MAX_PAYLOAD = 65536;

enum GroupCode : int {
    GR_OK = 0,
    GR_ERROR = -1,
    GR_INVALID_PARAM = -2000,
    GR_TIMEOUT = -2004,
    GR_NOT_STARTED = -2003,
};

using RankCallback = std::function<int(uint32_t rank)>;

struct GroupOption {
    uint32_t rankSize{0};  // static: fixed world; dynamic: upper bound of ranks
    uint32_t rank{0};
    uint32_t timeoutMs{120000};
    bool dynamic{false};
    RankCallback joinCb;   // run on every member (and on the joiner) when `rank` joins
    RankCallback leaveCb;  // run on every remaining member when `rank` leaves or dies
};

class GroupEngine {
public:
    static std::shared_ptr<GroupEngine> Create(store::StorePtr st, const GroupOption &opt);
    ~GroupEngine();

    int GroupBarrier();
    // recv holds one sendSize slot per member, ordered by rank id (i-th smallest joined rank for dynamic groups).
    int GroupAllGather(const void *send, uint32_t sendSize, void *recv, uint32_t recvSize);
    int SubGroupBarrier(const std::string &key, uint32_t rankSize, uint32_t rankId);
    int SubGroupAllGather(const std::string &key, uint32_t rankSize, uint32_t rankId, const void *send, uint32_t sendSize,
                          void *recv, uint32_t recvSize);
    int GroupJoin();
    int GroupLeave();
    int AllocNumber(uint32_t limit, uint32_t *out);
    int ReleaseNumber(uint32_t value);
    int RegisterExit(std::function<void(int)> fn);
    int GroupBroadcastExit(int status);
    int StartListenEvent();
    void Stop();

    uint32_t LocalRank() const { return opt_.rank; }
    uint32_t RankSize() const { return size_.load(); }
    uint32_t Version() const { return version_.load(); }
    bool Joined() const { return joined_.load(); }
    std::vector<uint32_t> Members();

    static uint64_t PackVerSize(uint32_t ver, uint32_t size) { return ((uint64_t)ver << 30) | size; }
    static void UnpackVerSize(uint64_t v, uint32_t *ver, uint32_t *size)
    {
        *ver = (uint32_t)(v >> 30);
        *size = (uint32_t)(v & ((1u << 30) - 1));
    }

private:
    GroupEngine(store::StorePtr st, const GroupOption &opt);
    int BarrierOn(const std::string &prefix, uint32_t size, const std::vector<std::string> &gcKeys);
    int AllGatherOn(const std::string &prefix, uint32_t size, uint32_t myRank, const void *send, uint32_t sendSize,
                    void *recv, uint32_t recvSize, std::vector<uint32_t> *ranksOut, const std::vector<std::string> &gcKeys);
    std::string RoundPrefix(uint32_t *snOut);
    static std::vector<std::string> GcKeys(uint32_t ver, uint32_t sn);
    void ListenLoop();
    void HandleEvent(const std::string &value);
    void HandleRankDown(uint32_t rank);
    void ApplyMembership(uint32_t rank, bool join);
    void ArmWatches();
    // After the link to the store came back (the server may have restarted empty): re-arm the rank-down and exit watches and
    // put this group's shared state — the packed (version, size) counter and the member list — back where it is missing.
    // Deferred: the reconnect notification only raises a flag, the next collective (or the listener thread) does the work.
    void RepairAfterReconnect();

    store::StorePtr store_;
    GroupOption opt_;
    std::atomic<uint32_t> size_{0};
    std::atomic<uint32_t> version_{0};
    std::atomic<uint32_t> sn_{0};
    std::atomic<bool> joined_{false};
    std::atomic<bool> stop_{false};
    std::mutex memberMu_;
    std::bitset<GROUP_RANK_MAX> members_;
    std::mutex opMu_;  // one collective at a time per engine
    std::thread listener_;
    std::string lastEvent_;
    uint32_t rankDownWid_{0};
    uint32_t exitWid_{0};
    std::function<void(int)> exitFn_;
    std::mutex subMu_;
    std::unordered_map<std::string, uint32_t> subSn_;
    std::mutex downMu_;
    std::vector<uint32_t> pendingDown_;
    std::atomic<bool> needRepair_{false};
    std::mutex repairMu_;
    uint32_t reconnectListener_{0};
    std::atomic<uint32_t> repairs_{0};

public:
    uint32_t Repairs() const { return repairs_.load(); }
};

}  // namespace group
}  // namespace mf

#include "mf_group.h"

#include <algorithm>
#include <cstring>
#include <unistd.h>

#include "../util/mf_log.h"
#include "../util/mf_tracer.h"

namespace mf {
namespace group {

using store::ST_NOT_EXIST;
using store::ST_OK;
using store::ST_TIMEOUT;

static const char *kEventKey = "EVENT";
static const char *kSizeKey = "DSIZE";
static const char *kExitKey = "EXIT";
static const char *kNumbersKey = "NUMBERS";
static constexpr uint64_t kVerOne = 1ull << 30;

static const char *kMembersKey = "MEMBERS";

static std::string EncodeMembers(const std::bitset<GROUP_RANK_MAX> &m)
{
    std::string out;
    for (uint32_t i = 0; i < GROUP_RANK_MAX; i++) {
        if (m.test(i)) {
            out += std::to_string(i) + ",";
        }
    }
    return out;
}

static void DecodeMembers(const std::string &s, std::bitset<GROUP_RANK_MAX> *m)
{
    size_t pos = 0;
    while (pos < s.size()) {
        size_t comma = s.find(',', pos);
        if (comma == std::string::npos) {
            break;
        }
        uint32_t r = (uint32_t)std::strtoul(s.substr(pos, comma - pos).c_str(), nullptr, 10);
        if (r < GROUP_RANK_MAX) {
            m->set(r);
        }
        pos = comma + 1;
    }
}

static int MapStoreCode(int rc)
{
    if (rc == ST_OK) {
        return GR_OK;
    }
    return rc == ST_TIMEOUT ? GR_TIMEOUT : GR_ERROR;
}

GroupEngine::GroupEngine(store::StorePtr st, const GroupOption &opt) : store_(std::move(st)), opt_(opt) {}

std::shared_ptr<GroupEngine> GroupEngine::Create(store::StorePtr st, const GroupOption &opt)
{
    if (!st || opt.rankSize == 0 || opt.rankSize > GROUP_RANK_MAX || opt.rank >= opt.rankSize || opt.timeoutMs == 0) {
        MF_ERROR("group: invalid option rankSize=" << opt.rankSize << " rank=" << opt.rank);
        return nullptr;
    }
    std::shared_ptr<GroupEngine> g(new GroupEngine(std::move(st), opt));
    GroupEngine *raw = g.get();
    g->reconnectListener_ = g->store_->AddReconnectListener([raw]() { raw->needRepair_.store(true); });
    if (!opt.dynamic) {
        g->size_.store(opt.rankSize);
        g->joined_.store(true);
        for (uint32_t i = 0; i < opt.rankSize; i++) {
            g->members_.set(i);
        }
    }
    return g;
}

GroupEngine::~GroupEngine() { Stop(); }

void GroupEngine::Stop()
{
    if (stop_.exchange(true)) {
        return;
    }
    if (reconnectListener_ != 0) {
        store_->RemoveReconnectListener(reconnectListener_);
        reconnectListener_ = 0;
    }
    if (listener_.joinable()) {
        listener_.join();
    }
    if (rankDownWid_ != 0) {
        store_->Unwatch(rankDownWid_);
    }
    if (exitWid_ != 0) {
        store_->Unwatch(exitWid_);
    }
}

void GroupEngine::RepairAfterReconnect()
{
    if (!needRepair_.load()) {
        return;
    }
    std::lock_guard<std::mutex> g(repairMu_);
    if (!needRepair_.exchange(false)) {
        return;
    }
    // Watches were tied to the old link.
    if (opt_.dynamic && listener_.joinable()) {
        rankDownWid_ = 0;
        ArmWatches();
    }
    if (exitFn_) {
        auto fn = exitFn_;
        store_->Watch(kExitKey, [fn](int rc, const std::string &, const std::string &v) {
            if (rc == ST_OK) {
                fn((int)std::strtol(v.c_str(), nullptr, 10));
            }
        }, &exitWid_);
    }
    if (opt_.dynamic && joined_.load()) {
        // A restarted server knows nothing: the first member that gets here restores the counter and the list, the others find
        // them in place. A server that merely lost the link still has both and nothing is written.
        const uint64_t want = PackVerSize(version_.load(), size_.load());
        int64_t cur = 0;
        if (store_->Add(kSizeKey, 0, &cur) == ST_OK && (uint64_t)cur < want) {
            std::string prev;
            store_->Cas(kSizeKey, std::to_string(cur), std::to_string(want), &prev);
        }
        std::string stored;
        if (store_->Get(kMembersKey, &stored, 0) != ST_OK) {
            std::lock_guard<std::mutex> gm(memberMu_);
            std::string prev;
            store_->Cas(kMembersKey, "", EncodeMembers(members_), &prev);
        }
    }
    repairs_.fetch_add(1);
    MF_INFO("group: state repaired after the store link came back (rank " << opt_.rank << ", version " << version_.load() << ", size " << size_.load()
                                                                          << ")");
}

std::vector<uint32_t> GroupEngine::Members()
{
    std::lock_guard<std::mutex> g(memberMu_);
    std::vector<uint32_t> out;
    for (uint32_t i = 0; i < GROUP_RANK_MAX; i++) {
        if (members_.test(i)) {
            out.push_back(i);
        }
    }
    return out;
}

std::string GroupEngine::RoundPrefix(uint32_t *snOut)
{
    uint32_t sn = sn_.fetch_add(1);
    if (snOut != nullptr) {
        *snOut = sn;
    }
    return std::to_string(version_.load()) + "_" + std::to_string(sn);
}

// Keys of round sn-2, which every member has left once round sn completes: the request that completes round sn drops them
// on the server, so garbage collection costs no round trip of its own.
std::vector<std::string> GroupEngine::GcKeys(uint32_t ver, uint32_t sn)
{
    std::vector<std::string> keys;
    if (sn >= 2) {
        std::string old = std::to_string(ver) + "_" + std::to_string(sn - 2);
        for (const char *suffix : {"_BA", "_BW", "_GA", "_GW"}) {
            keys.push_back(old + suffix);
        }
    }
    return keys;
}

int GroupEngine::BarrierOn(const std::string &prefix, uint32_t size, const std::vector<std::string> &gcKeys)
{
    int64_t val = 0;
    int rc = store_->Arrive(prefix + "_BA", prefix + "_BW", size, opt_.timeoutMs, gcKeys, &val);
    if (rc != ST_OK) {
        MF_ERROR("group barrier: failed rc=" << rc << " key=" << prefix << " arrived=" << val << "/" << size);
    }
    return MapStoreCode(rc);
}

int GroupEngine::GroupBarrier()
{
    if (!joined_.load()) {
        return GR_NOT_STARTED;
    }
    int ret = 0;
    MF_TRACE_SCOPE(MF_TP(TM_GROUP, 0), "GROUP_BARRIER", &ret);
    std::lock_guard<std::mutex> g(opMu_);
    RepairAfterReconnect();
    uint32_t sn = 0;
    uint32_t ver = version_.load();
    std::string prefix = RoundPrefix(&sn);
    ret = BarrierOn(prefix, size_.load(), GcKeys(ver, sn));
    return ret;
}

int GroupEngine::AllGatherOn(const std::string &prefix, uint32_t size, uint32_t myRank, const void *send, uint32_t sendSize,
                             void *recv, uint32_t recvSize, std::vector<uint32_t> *ranksOut,
                             const std::vector<std::string> &gcKeys)
{
    if (send == nullptr || recv == nullptr || sendSize == 0 || sendSize > GROUP_ALLGATHER_MAX_PAYLOAD ||
        (uint64_t)recvSize < (uint64_t)sendSize * size) {
        MF_ERROR("group allgather: invalid sizes send=" << sendSize << " recv=" << recvSize << " members=" << size);
        return GR_INVALID_PARAM;
    }
    std::string rec((const char *)&myRank, 4);
    rec.append((const char *)send, sendSize);
    const uint64_t full = (uint64_t)size * (4 + sendSize);
    std::string all;
    int rc = store_->Gather(prefix + "_GA", prefix + "_GW", rec, full, opt_.timeoutMs, gcKeys, &all);
    if (rc != ST_OK) {
        MF_ERROR("group allgather: failed rc=" << rc << " key=" << prefix << " expected bytes=" << full);
        return MapStoreCode(rc);
    }
    if (all.size() != full) {
        MF_ERROR("group allgather: bad gathered size " << all.size() << " expected " << full);
        return GR_ERROR;
    }
    std::vector<std::pair<uint32_t, const char *>> recs;
    for (uint32_t i = 0; i < size; i++) {
        const char *p = all.data() + (size_t)i * (4 + sendSize);
        uint32_t r;
        std::memcpy(&r, p, 4);
        recs.emplace_back(r, p + 4);
    }
    std::sort(recs.begin(), recs.end(), [](const auto &a, const auto &b) { return a.first < b.first; });
    for (uint32_t i = 0; i < size; i++) {
        std::memcpy((char *)recv + (size_t)i * sendSize, recs[i].second, sendSize);
        if (ranksOut != nullptr) {
            ranksOut->push_back(recs[i].first);
        }
    }
    return GR_OK;
}

int GroupEngine::GroupAllGather(const void *send, uint32_t sendSize, void *recv, uint32_t recvSize)
{
    if (!joined_.load()) {
        return GR_NOT_STARTED;
    }
    int ret = 0;
    MF_TRACE_SCOPE(MF_TP(TM_GROUP, 1), "GROUP_ALLGATHER", &ret);
    std::lock_guard<std::mutex> g(opMu_);
    RepairAfterReconnect();
    uint32_t sn = 0;
    uint32_t ver = version_.load();
    std::string prefix = RoundPrefix(&sn);
    std::vector<uint32_t> ranks;
    ret = AllGatherOn(prefix, size_.load(), opt_.rank, send, sendSize, recv, recvSize, &ranks, GcKeys(ver, sn));
    if (ret == GR_OK && opt_.dynamic) {
        // A fresh joiner learns the membership from the first allgather it takes part in.
        std::lock_guard<std::mutex> mg(memberMu_);
        members_.reset();
        for (uint32_t r : ranks) {
            if (r < GROUP_RANK_MAX) {
                members_.set(r);
            }
        }
    }
    return ret;
}

int GroupEngine::SubGroupBarrier(const std::string &key, uint32_t rankSize, uint32_t rankId)
{
    if (key.empty() || rankSize == 0 || rankId >= rankSize) {
        return GR_INVALID_PARAM;
    }
    uint32_t sn;
    {
        std::lock_guard<std::mutex> g(subMu_);
        sn = subSn_["B" + key]++;
    }
    std::string prefix = "SUB_" + key + "_" + std::to_string(sn);
    std::vector<std::string> gc;
    if (sn >= 2) {
        std::string old = "SUB_" + key + "_" + std::to_string(sn - 2);
        gc = {old + "_BA", old + "_BW"};
    }
    return BarrierOn(prefix, rankSize, gc);
}

int GroupEngine::SubGroupAllGather(const std::string &key, uint32_t rankSize, uint32_t rankId, const void *send,
                                   uint32_t sendSize, void *recv, uint32_t recvSize)
{
    if (key.empty() || rankSize == 0 || rankId >= rankSize) {
        return GR_INVALID_PARAM;
    }
    uint32_t sn;
    {
        std::lock_guard<std::mutex> g(subMu_);
        sn = subSn_["G" + key]++;
    }
    std::string prefix = "SUBG_" + key + "_" + std::to_string(sn);
    std::vector<std::string> gc;
    if (sn >= 2) {
        std::string old = "SUBG_" + key + "_" + std::to_string(sn - 2);
        gc = {old + "_GA", old + "_GW"};
    }
    return AllGatherOn(prefix, rankSize, rankId, send, sendSize, recv, recvSize, nullptr, gc);
}

// ---------------------------------------------------------------------------------------------- dynamic membership

void GroupEngine::ApplyMembership(uint32_t rank, bool join)
{
    std::lock_guard<std::mutex> g(memberMu_);
    if (join) {
        if (!members_.test(rank)) {
            members_.set(rank);
            size_.fetch_add(1);
        }
    } else {
        if (members_.test(rank)) {
            members_.reset(rank);
            size_.fetch_sub(1);
        }
    }
    version_.fetch_add(1);
    sn_.store(0);
}

int GroupEngine::StartListenEvent()
{
    if (!opt_.dynamic || listener_.joinable()) {
        return GR_OK;
    }
    ArmWatches();
    listener_ = std::thread([this]() { ListenLoop(); });
    return GR_OK;
}

void GroupEngine::ArmWatches()
{
    if (opt_.dynamic) {
        // The callback runs on the store's reader thread, which must not issue store calls: hand over to the listener.
        store_->WatchRankDown(
            [this](uint32_t rank) {
                std::lock_guard<std::mutex> g(downMu_);
                pendingDown_.push_back(rank);
            },
            &rankDownWid_);
    }
}

void GroupEngine::ListenLoop()
{
    while (!stop_.load()) {
        std::vector<uint32_t> down;
        {
            std::lock_guard<std::mutex> g(downMu_);
            down.swap(pendingDown_);
        }
        for (uint32_t r : down) {
            HandleRankDown(r);
        }
        if (store_->Connected()) {
            RepairAfterReconnect();
        }
        if (!store_->Connected()) {
            usleep(100 * 1000);
            continue;
        }
        std::string value;
        int rc = store_->Get(kEventKey, &value, 100);
        if (rc != ST_OK) {
            lastEvent_.clear();
            if (rc != ST_TIMEOUT && rc != ST_NOT_EXIST) {
                usleep(50 * 1000);
            }
            continue;
        }
        if (value != lastEvent_) {
            lastEvent_ = value;
            HandleEvent(value);
        }
        // Wait until the initiator retires this event (or replaces it) before blocking on the key again.
        while (!stop_.load()) {
            std::string cur;
            rc = store_->Get(kEventKey, &cur, 0);
            if (rc != ST_OK || cur != lastEvent_) {
                break;
            }
            {
                std::lock_guard<std::mutex> g(downMu_);
                if (!pendingDown_.empty()) {
                    break;
                }
            }
            usleep(2000);
        }
    }
}

static bool ParseEvent(const std::string &v, char *kind, uint32_t *rank, std::string *nonce)
{
    if (v.size() < 2) {
        return false;
    }
    *kind = v[0];
    size_t colon = v.find(':');
    std::string num = v.substr(1, colon == std::string::npos ? std::string::npos : colon - 1);
    if (num.empty() || num.find_first_not_of("0123456789") != std::string::npos) {
        return false;
    }
    *rank = (uint32_t)std::strtoul(num.c_str(), nullptr, 10);
    *nonce = colon == std::string::npos ? "" : v.substr(colon + 1);
    return true;
}

void GroupEngine::HandleEvent(const std::string &value)
{
    char kind = 0;
    uint32_t rank = 0;
    std::string nonce;
    if (!ParseEvent(value, &kind, &rank, &nonce) || !joined_.load() || rank == opt_.rank) {
        return;
    }
    if (kind == 'J') {
        MF_INFO("group: rank " << rank << " joins (seen by rank " << opt_.rank << ")");
        ApplyMembership(rank, true);
        if (opt_.joinCb) {
            int rc = opt_.joinCb(rank);
            if (rc != 0) {
                MF_ERROR("group: join callback for rank " << rank << " failed rc=" << rc);
            }
        }
        int64_t acks = 0;
        store_->Add("EVACK_" + nonce, 1, &acks);  // the joiner keeps the event up until every member has seen it
    } else if (kind == 'L') {
        bool member;
        {
            std::lock_guard<std::mutex> g(memberMu_);
            member = members_.test(rank);
        }
        if (member) {
            MF_INFO("group: rank " << rank << " leaves (seen by rank " << opt_.rank << ")");
            if (opt_.leaveCb) {
                opt_.leaveCb(rank);
            }
            ApplyMembership(rank, false);
        }
        int64_t acks = 0;
        store_->Add("EVACK_" + nonce, 1, &acks);
    }
}

void GroupEngine::HandleRankDown(uint32_t rank)
{
    if (!joined_.load() || rank == opt_.rank) {
        return;
    }
    {
        std::lock_guard<std::mutex> g(memberMu_);
        if (!members_.test(rank)) {
            return;
        }
    }
    MF_WARN("group: rank " << rank << " is down, removing it (seen by rank " << opt_.rank << ")");
    // If the dead rank was in the middle of a join/leave, one member retires its event.
    std::string ev;
    bool midJoin = false;
    if (store_->Get(kEventKey, &ev, 0) == ST_OK) {
        char kind = 0;
        uint32_t r = 0;
        std::string nonce;
        if (ParseEvent(ev, &kind, &r, &nonce) && r == rank && (kind == 'J' || kind == 'L')) {
            std::string prev;
            midJoin = kind == 'J';
            if (store_->Cas(kEventKey, ev, "U" + std::to_string(rank), &prev) == ST_OK && prev == ev) {
                if (midJoin) {
                    // Members already counted the joiner locally and now drop it again: two version bumps, size unchanged.
                    int64_t nv = 0;
                    store_->Add(kSizeKey, (int64_t)(2 * kVerOne), &nv);
                }
                store_->Remove(kEventKey, true);
            }
        }
    }
    if (opt_.leaveCb) {
        opt_.leaveCb(rank);
    }
    ApplyMembership(rank, false);
    if (!midJoin) {
        // Exactly one survivor repairs the shared (version,size) counter.
        std::string prev;
        std::string key = "DOWN_" + std::to_string(version_.load()) + "_" + std::to_string(rank);
        if (store_->Cas(key, "", "1", &prev) == ST_OK && prev.empty()) {
            int64_t nv = 0;
            store_->Add(kSizeKey, (int64_t)kVerOne - 1, &nv);
            std::lock_guard<std::mutex> g(memberMu_);
            store_->Set(kMembersKey, EncodeMembers(members_));
        }
    }
}

int GroupEngine::GroupJoin()
{
    if (!opt_.dynamic) {
        return GR_INVALID_PARAM;
    }
    if (joined_.load()) {
        return GR_OK;
    }
    StartListenEvent();
    const std::string joinNonce = std::to_string(NowNs());
    const std::string mine = "J" + std::to_string(opt_.rank) + ":" + joinNonce;
    uint64_t deadline = NowMs() + opt_.timeoutMs;
    while (true) {
        std::string prev;
        int rc = store_->Cas(kEventKey, "", mine, &prev);
        if (rc != ST_OK) {
            return MapStoreCode(rc);
        }
        if (prev.empty()) {
            break;
        }
        if (NowMs() > deadline) {
            MF_ERROR("group join: another membership change (" << prev << ") did not finish in time");
            return GR_TIMEOUT;
        }
        usleep(5000);
    }
    int64_t packed = 0;
    int rc = store_->Add(kSizeKey, 0, &packed);
    if (rc != ST_OK) {
        store_->Remove(kEventKey, true);
        return MapStoreCode(rc);
    }
    uint32_t ver = 0, size = 0;
    UnpackVerSize((uint64_t)packed, &ver, &size);
    {
        std::string stored;
        std::lock_guard<std::mutex> g(memberMu_);
        members_.reset();
        if (store_->Get(kMembersKey, &stored, 0) == ST_OK) {
            DecodeMembers(stored, &members_);  // who is in already (the event key serialises writers of this list)
        }
        members_.set(opt_.rank);
        size_.store(size + 1);
        version_.store(ver + 1);
        sn_.store(0);
    }
    joined_.store(true);
    int cbRc = opt_.joinCb ? opt_.joinCb(opt_.rank) : 0;
    int64_t nv = 0;
    if (cbRc == 0) {
        // Every existing member must have seen the event before it is retired, or a quick join could go unnoticed.
        uint64_t until = NowMs() + opt_.timeoutMs;
        while (size > 0 && NowMs() < until) {
            std::string acks;
            if (store_->Get("EVACK_" + joinNonce, &acks, 0) == ST_OK && std::strtoul(acks.c_str(), nullptr, 10) >= size) {
                break;
            }
            usleep(1000);
        }
        {
            std::lock_guard<std::mutex> g(memberMu_);
            store_->Set(kMembersKey, EncodeMembers(members_));
        }
        store_->Add(kSizeKey, (int64_t)(kVerOne | 1), &nv);
        store_->Remove("EVACK_" + joinNonce, true);
        store_->Remove(kEventKey, true);
        return GR_OK;
    }
    MF_ERROR("group join: join callback failed rc=" << cbRc << ", withdrawing");
    // Withdraw: turn the event into a leave so that members which already counted us drop us again.
    joined_.store(false);
    const std::string nonce = std::to_string(NowNs());
    store_->Set(kEventKey, "L" + std::to_string(opt_.rank) + ":" + nonce);
    uint64_t until = NowMs() + 2000;
    while (NowMs() < until) {
        std::string acks;
        if (store_->Get("EVACK_" + nonce, &acks, 0) == ST_OK && std::strtoul(acks.c_str(), nullptr, 10) >= size) {
            break;
        }
        usleep(5000);
    }
    store_->Add(kSizeKey, (int64_t)(2 * kVerOne), &nv);
    store_->Remove("EVACK_" + nonce, true);
    store_->Remove(kEventKey, true);
    return GR_ERROR;
}

int GroupEngine::GroupLeave()
{
    if (!opt_.dynamic) {
        return GR_INVALID_PARAM;
    }
    if (!joined_.load()) {
        return GR_OK;
    }
    const std::string nonce = std::to_string(NowNs());
    const std::string mine = "L" + std::to_string(opt_.rank) + ":" + nonce;
    uint64_t deadline = NowMs() + opt_.timeoutMs;
    while (true) {
        std::string prev;
        int rc = store_->Cas(kEventKey, "", mine, &prev);
        if (rc != ST_OK) {
            return MapStoreCode(rc);
        }
        if (prev.empty()) {
            break;
        }
        if (NowMs() > deadline) {
            return GR_TIMEOUT;
        }
        usleep(5000);
    }
    uint32_t others = size_.load() > 0 ? size_.load() - 1 : 0;
    joined_.store(false);
    uint64_t until = NowMs() + std::min<uint32_t>(opt_.timeoutMs, 10000);
    while (others > 0 && NowMs() < until) {
        std::string acks;
        if (store_->Get("EVACK_" + nonce, &acks, 0) == ST_OK && std::strtoul(acks.c_str(), nullptr, 10) >= others) {
            break;
        }
        usleep(2000);
    }
    int64_t nv = 0;
    {
        std::lock_guard<std::mutex> g(memberMu_);
        members_.reset(opt_.rank);
        store_->Set(kMembersKey, EncodeMembers(members_));
        members_.reset();
        size_.store(0);
    }
    store_->Add(kSizeKey, (int64_t)kVerOne - 1, &nv);
    store_->Remove("EVACK_" + nonce, true);
    store_->Remove(kEventKey, true);
    return GR_OK;
}

// ---------------------------------------------------------------------------------------------- numbers / exit

int GroupEngine::AllocNumber(uint32_t limit, uint32_t *out)
{
    if (out == nullptr || limit == 0 || limit > GROUP_NUMBER_MAX) {
        return GR_INVALID_PARAM;
    }
    for (int attempt = 0; attempt < 10000; attempt++) {
        std::string cur;
        int rc = store_->Get(kNumbersKey, &cur, 0);
        if (rc != ST_OK && rc != ST_NOT_EXIST) {
            return MapStoreCode(rc);
        }
        std::string next = cur;
        next.resize(GROUP_NUMBER_MAX / 8, '\0');
        uint32_t pick = limit;
        for (uint32_t i = 0; i < limit; i++) {
            if (!((unsigned char)next[i / 8] & (1u << (i % 8)))) {
                pick = i;
                break;
            }
        }
        if (pick == limit) {
            MF_ERROR("group: no free number below " << limit);
            return GR_ERROR;
        }
        next[pick / 8] = (char)((unsigned char)next[pick / 8] | (1u << (pick % 8)));
        std::string prev;
        rc = store_->Cas(kNumbersKey, cur, next, &prev);
        if (rc != ST_OK) {
            return MapStoreCode(rc);
        }
        if (prev == cur) {
            *out = pick;
            return GR_OK;
        }
    }
    return GR_TIMEOUT;
}

int GroupEngine::ReleaseNumber(uint32_t value)
{
    if (value >= GROUP_NUMBER_MAX) {
        return GR_INVALID_PARAM;
    }
    for (int attempt = 0; attempt < 10000; attempt++) {
        std::string cur;
        int rc = store_->Get(kNumbersKey, &cur, 0);
        if (rc == ST_NOT_EXIST) {
            return GR_OK;
        }
        if (rc != ST_OK) {
            return MapStoreCode(rc);
        }
        std::string next = cur;
        next.resize(GROUP_NUMBER_MAX / 8, '\0');
        next[value / 8] = (char)((unsigned char)next[value / 8] & ~(1u << (value % 8)));
        std::string prev;
        rc = store_->Cas(kNumbersKey, cur, next, &prev);
        if (rc != ST_OK) {
            return MapStoreCode(rc);
        }
        if (prev == cur) {
            return GR_OK;
        }
    }
    return GR_TIMEOUT;
}

int GroupEngine::RegisterExit(std::function<void(int)> fn)
{
    if (!fn) {
        return GR_INVALID_PARAM;
    }
    exitFn_ = std::move(fn);
    int rc = store_->Watch(
        kExitKey,
        [this](int result, const std::string &, const std::string &value) {
            if (result == ST_OK && exitFn_) {
                exitFn_((int)std::strtol(value.c_str(), nullptr, 10));
            }
        },
        &exitWid_);
    return MapStoreCode(rc);
}

int GroupEngine::GroupBroadcastExit(int status) { return MapStoreCode(store_->Set(kExitKey, std::to_string(status))); }

}  // namespace group
}  // namespace mf

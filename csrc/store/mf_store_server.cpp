#include "mf_store_server.h"

#include "../net/mf_tls.h"

#include <cerrno>
#include <cstdlib>
#include <cstring>

#include "../util/mf_log.h"

namespace mf {
namespace store {

// ---------------------------------------------------------------------------------------------- message codec
// Layout (little-endian): i64 userDef | u32 nKeys | u32 nValues | {u32 len, bytes} × nKeys | {u32 len, bytes} × nValues.

static void PutU32(std::string &s, uint32_t v) { s.append((const char *)&v, 4); }

std::string PackMessage(const StoreMessage &m)
{
    std::string out;
    size_t total = 16;
    for (auto &k : m.keys) {
        total += 4 + k.size();
    }
    for (auto &v : m.values) {
        total += 4 + v.size();
    }
    out.reserve(total);
    out.append((const char *)&m.userDef, 8);
    PutU32(out, (uint32_t)m.keys.size());
    PutU32(out, (uint32_t)m.values.size());
    for (auto &k : m.keys) {
        PutU32(out, (uint32_t)k.size());
        out.append(k);
    }
    for (auto &v : m.values) {
        PutU32(out, (uint32_t)v.size());
        out.append(v);
    }
    return out;
}

bool UnpackMessage(const std::string &buf, StoreMessage *out)
{
    if (buf.size() < 16) {
        return false;
    }
    size_t pos = 0;
    uint32_t nk, nv;
    std::memcpy(&out->userDef, buf.data(), 8);
    std::memcpy(&nk, buf.data() + 8, 4);
    std::memcpy(&nv, buf.data() + 12, 4);
    pos = 16;
    if (nk > MAX_KEYS_PER_MSG || nv > MAX_VALUES_PER_MSG) {
        return false;
    }
    out->keys.clear();
    out->values.clear();
    auto readList = [&](uint32_t n, size_t maxLen, std::vector<std::string> &dst) {
        for (uint32_t i = 0; i < n; i++) {
            if (buf.size() - pos < 4) {
                return false;
            }
            uint32_t len;
            std::memcpy(&len, buf.data() + pos, 4);
            pos += 4;
            if (len > maxLen || buf.size() - pos < len) {
                return false;
            }
            dst.emplace_back(buf.data() + pos, len);
            pos += len;
        }
        return true;
    };
    if (!readList(nk, MAX_KEY_LEN_SERVER, out->keys) || !readList(nv, MAX_VALUE_LEN, out->values)) {
        return false;
    }
    return pos == buf.size();
}

// ---------------------------------------------------------------------------------------------- local memory backend

bool LocalMemoryBackend::Expired(const Entry &e) const { return e.expireAtMs != 0 && NowMs() >= e.expireAtMs; }

bool LocalMemoryBackend::Get(const std::string &key, std::string *value)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = kv_.find(key);
    if (it == kv_.end()) {
        return false;
    }
    if (Expired(it->second)) {
        kv_.erase(it);
        return false;
    }
    if (value != nullptr) {
        *value = it->second.value;
    }
    return true;
}

void LocalMemoryBackend::Put(const std::string &key, const std::string &value, uint64_t ttlMs)
{
    std::lock_guard<std::mutex> g(mu_);
    Entry &e = kv_[key];
    e.value = value;
    e.expireAtMs = ttlMs ? NowMs() + ttlMs : 0;
}

bool LocalMemoryBackend::Delete(const std::string &key)
{
    std::lock_guard<std::mutex> g(mu_);
    return kv_.erase(key) > 0;
}

bool LocalMemoryBackend::Exist(const std::string &key) { return Get(key, nullptr); }

void LocalMemoryBackend::Clear()
{
    std::lock_guard<std::mutex> g(mu_);
    kv_.clear();
    locks_.clear();
}

size_t LocalMemoryBackend::Size()
{
    std::lock_guard<std::mutex> g(mu_);
    return kv_.size();
}

std::string *LocalMemoryBackend::Mutable(const std::string &key)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = kv_.find(key);
    if (it == kv_.end() || Expired(it->second)) {
        return nullptr;
    }
    return &it->second.value;
}

bool LocalMemoryBackend::TryLock(const std::string &name, const std::string &owner, uint64_t leaseMs)
{
    std::lock_guard<std::mutex> g(mu_);
    uint64_t now = NowMs();
    auto it = locks_.find(name);
    if (it != locks_.end() && it->second.owner != owner && (it->second.expireAtMs == 0 || now < it->second.expireAtMs)) {
        return false;
    }
    locks_[name] = LockRec{owner, leaseMs ? now + leaseMs : 0};
    return true;
}

bool LocalMemoryBackend::Unlock(const std::string &name, const std::string &owner)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = locks_.find(name);
    if (it == locks_.end() || it->second.owner != owner) {
        return false;
    }
    locks_.erase(it);
    return true;
}

// ---------------------------------------------------------------------------------------------- server

ServerTiming &GlobalTiming()
{
    static ServerTiming t = []() {
        ServerTiming x;
        const char *env = std::getenv("MF_STORE_HEARTBEAT_MS");
        if (env != nullptr) {
            long v = std::strtol(env, nullptr, 10);
            if (v >= 10 && v <= 600000) {
                x.heartbeatIntervalMs = (uint32_t)v;
            }
        }
        return x;
    }();
    return t;
}

StoreServer::StoreServer() : backend_(new LocalMemoryBackend()) {}
StoreServer::~StoreServer() { Stop(); }

int StoreServer::Start(const net::Endpoint &ep, uint32_t worldSize)
{
    worldSize_ = worldSize;
    rpc_.SetHandlers([this](net::LinkId l, const net::Frame &f) { OnMessage(l, f); },
                     [this](net::LinkId l, uint64_t id) { return OnLinkUp(l, id); }, [this](net::LinkId l) { OnLinkDown(l); });
    net::TlsOptions tls = net::GetStoreTlsOptions();
    if (tls.enable) {
        std::string err;
        auto ctx = net::TlsContext::Create(tls, true, &err);
        if (!ctx) {
            MF_ERROR("store server: TLS is enabled but cannot be set up: " << err);
            return -EPROTO;
        }
        rpc_.SetTls(ctx);
    } else {
        rpc_.SetTls(nullptr);
    }
    int rc = rpc_.Start(ep);
    if (rc != 0) {
        return rc;
    }
    stop_.store(false);
    house_ = std::thread([this]() { HouseKeeping(); });
    MF_INFO("store server listening on " << ep.host << ":" << rpc_.Port());
    return 0;
}

void StoreServer::Stop()
{
    if (stop_.exchange(true) && !house_.joinable()) {
        return;
    }
    cv_.notify_all();
    if (house_.joinable()) {
        house_.join();
    }
    rpc_.Stop();
    std::lock_guard<std::mutex> g(mu_);
    keyWaiters_.clear();
    timed_.clear();
    rankWatchers_.clear();
    lastSeenMs_.clear();
    helloId_.clear();
    linkRanks_.clear();
    usedRanks_.clear();
    linkWorldRank_.clear();
}

size_t StoreServer::AliveLinks()
{
    std::lock_guard<std::mutex> g(mu_);
    return lastSeenMs_.size();
}

bool StoreServer::OnLinkUp(net::LinkId link, uint64_t peerId)
{
    std::lock_guard<std::mutex> g(mu_);
    lastSeenMs_[link] = NowMs();
    helloId_[link] = peerId;
    uint32_t rank = (uint32_t)(peerId & 0xffffffffu);
    if (rank != 0xffffffffu) {
        linkWorldRank_[link] = rank;
    }
    return true;
}

void StoreServer::OnLinkDown(net::LinkId link) { LinkGone(link, false); }

void StoreServer::LinkGone(net::LinkId link, bool fromHeartbeat)
{
    std::vector<std::pair<net::LinkId, uint32_t>> watchers;
    std::vector<uint32_t> deadRanks;
    bool clearAll = false;
    {
        std::lock_guard<std::mutex> g(mu_);
        if (lastSeenMs_.erase(link) == 0) {
            return;  // already processed (heartbeat expiry followed by the socket closing)
        }
        helloId_.erase(link);
        auto lr = linkRanks_.find(link);
        if (lr != linkRanks_.end()) {
            for (auto &kv : lr->second) {
                usedRanks_[kv.first].erase(kv.second);
                deadRanks.push_back(kv.second);
            }
            linkRanks_.erase(lr);
        }
        auto wr = linkWorldRank_.find(link);
        if (wr != linkWorldRank_.end()) {
            if (deadRanks.empty()) {
                deadRanks.push_back(wr->second);
            }
            linkWorldRank_.erase(wr);
        }
        // Eagerly drop whatever the dead link parked.
        for (auto it = keyWaiters_.begin(); it != keyWaiters_.end();) {
            auto &vec = it->second;
            for (size_t i = 0; i < vec.size();) {
                if (vec[i].link == link) {
                    vec.erase(vec.begin() + (long)i);
                } else {
                    i++;
                }
            }
            it = vec.empty() ? keyWaiters_.erase(it) : std::next(it);
        }
        for (size_t i = 0; i < rankWatchers_.size();) {
            if (rankWatchers_[i].first == link) {
                rankWatchers_.erase(rankWatchers_.begin() + (long)i);
            } else {
                i++;
            }
        }
        watchers = rankWatchers_;
        clearAll = lastSeenMs_.empty() && !brokenHook_;
        if (clearAll) {
            keyWaiters_.clear();
            timed_.clear();
            usedRanks_.clear();
        }
    }
    if (brokenHook_) {
        brokenHook_(link, backend_.get());
    } else if (clearAll) {
        backend_->Clear();  // the same server can now host the next job
        MF_INFO("store server: last client left, store cleared");
    }
    if (fromHeartbeat) {
        rpc_.CloseLink(link);
    }
    for (uint32_t rank : deadRanks) {
        MF_INFO("store server: rank " << rank << " is down (link " << link << ")");
        std::string payload((const char *)&rank, sizeof(rank));
        for (auto &w : watchers) {
            ReplyText(w.first, w.second, OP_WATCH_RANK_STATE, ST_OK, payload);
        }
    }
}

void StoreServer::ReplyText(net::LinkId link, uint32_t seq, uint16_t type, int result, const std::string &value)
{
    if (mute_.load()) {
        return;
    }
    net::Frame r;
    r.type = type;
    r.seq = seq;
    r.result = (int16_t)result;
    r.body = value;
    rpc_.Send(link, r);
}

void StoreServer::Reply(net::LinkId link, const net::Frame &req, int result, const std::string &value)
{
    ReplyText(link, req.seq, req.type, result, value);
}

void StoreServer::WakeWaiters(const std::string &key, const std::string &value)
{
    std::vector<Waiter> woken;
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = keyWaiters_.find(key);
        if (it == keyWaiters_.end()) {
            return;
        }
        woken.swap(it->second);
        keyWaiters_.erase(it);
    }
    for (auto &w : woken) {
        ReplyText(w.link, w.seq, OP_GET, ST_OK, value);
    }
}

int StoreServer::AssignRank(net::LinkId link, const std::string &key, std::string *out)
{
    std::lock_guard<std::mutex> g(mu_);
    auto &mine = linkRanks_[link];
    auto it = mine.find(key);
    if (it != mine.end()) {
        *out = std::to_string(it->second);
        return ST_OK;
    }
    auto &used = usedRanks_[key];
    uint32_t r = 0;
    while (used.count(r)) {
        r++;
    }
    if (worldSize_ != 0 && r >= worldSize_) {
        return ST_ERROR;
    }
    used.insert(r);
    mine[key] = r;
    *out = std::to_string(r);
    return ST_OK;
}

void StoreServer::HandleGet(net::LinkId link, const net::Frame &f, const StoreMessage &m)
{
    const std::string &key = m.keys[0];
    std::string value;
    if (key.find(AUTO_RANKING_PREFIX) != std::string::npos) {
        int rc = AssignRank(link, key, &value);
        Reply(link, f, rc, value);
        return;
    }
    // Check-and-park must be atomic with respect to SET's put-and-wake, so both run under mu_.
    {
        std::unique_lock<std::mutex> lk(mu_);
        if (backend_->Get(key, &value)) {
            lk.unlock();
            Reply(link, f, ST_OK, value);
            return;
        }
        if (opHook_) {
            lk.unlock();
            std::string reply;
            int rc = opHook_(OP_GET, link, key, "", &reply);
            if (rc == ST_RESTORE || rc == ST_OK) {
                Reply(link, f, rc, reply);
                return;
            }
            lk.lock();
            if (backend_->Get(key, &value)) {
                lk.unlock();
                Reply(link, f, ST_OK, value);
                return;
            }
        }
        if (m.userDef == 0) {
            lk.unlock();
            Reply(link, f, ST_NOT_EXIST, "");
            return;
        }
        Waiter w{link, f.seq, m.userDef > 0 ? NowMs() + (uint64_t)m.userDef : 0, nextWaiterId_++};
        keyWaiters_[key].push_back(w);
        if (w.deadlineMs != 0) {
            timed_.emplace(w.deadlineMs, std::make_pair(key, w.id));
        }
    }
    cv_.notify_all();
}

// OP_ARRIVE (keys: counter, wake, then keys to drop on completion; values: expected count) and OP_GATHER (keys: data, wake,
// then keys to drop; values: record, full size). The request that completes the rendezvous stores the wake key, which answers every parked
// request of the round through the ordinary waiter list; all others are parked on the wake key exactly like a blocking GET.
// What a waiter receives is the wake key's value: "ok" for a barrier, the gathered bytes for an all-gather (the wake key of
// a gather holds the data so that late or repeated GETs of it see the same thing).
void StoreServer::HandleRendezvous(net::LinkId link, const net::Frame &f, const StoreMessage &m)
{
    const bool gather = f.type == OP_GATHER;
    if (m.keys.size() < 2 || m.values.size() != (gather ? 2u : 1u)) {
        Reply(link, f, ST_INVALID_MESSAGE, "bad rendezvous message");
        return;
    }
    for (const auto &k : m.keys) {
        if (k.empty() || k.size() > MAX_KEY_LEN_SERVER) {
            Reply(link, f, ST_INVALID_KEY, "invalid key");
            return;
        }
    }
    char *end = nullptr;
    errno = 0;
    const std::string &targetText = m.values[gather ? 1 : 0];
    unsigned long long target = std::strtoull(targetText.c_str(), &end, 10);
    if (targetText.empty() || *end != '\0' || errno != 0 || target == 0 || (gather && target > MAX_VALUE_LEN)) {
        Reply(link, f, ST_INVALID_MESSAGE, "bad rendezvous target");
        return;
    }
    const std::string &key = m.keys[0];
    const std::string &wake = m.keys[1];
    std::string wakeValue;
    bool complete = false;
    {
        std::unique_lock<std::mutex> lk(mu_);
        std::string cur;
        bool had = backend_->Get(key, &cur);
        if (gather) {
            if (cur.size() + m.values[0].size() > target) {
                lk.unlock();
                Reply(link, f, ST_INVALID_MESSAGE, "gather overflows its full size");
                return;
            }
            cur.append(m.values[0]);
            backend_->Put(key, cur);
            complete = cur.size() == target;
            if (complete) {
                wakeValue = cur;
            }
        } else {
            unsigned long long v = (had ? std::strtoull(cur.c_str(), nullptr, 10) : 0) + 1;
            backend_->Put(key, std::to_string(v));
            complete = v == target;
            if (complete) {
                wakeValue = "ok";
            }
        }
        if (complete) {
            for (size_t i = 2; i < m.keys.size(); i++) {
                backend_->Delete(m.keys[i]);
            }
            backend_->Put(wake, wakeValue);
        } else if (backend_->Get(wake, &wakeValue)) {
            complete = true;  // a member that arrives after the round completed (re-sent request): answer at once
        } else {
            Waiter w{link, f.seq, m.userDef > 0 ? NowMs() + (uint64_t)m.userDef : 0, nextWaiterId_++};
            keyWaiters_[wake].push_back(w);
            if (w.deadlineMs != 0) {
                timed_.emplace(w.deadlineMs, std::make_pair(wake, w.id));
            }
        }
    }
    if (complete) {
        WakeWaiters(wake, wakeValue);
        Reply(link, f, ST_OK, wakeValue);
    } else {
        cv_.notify_all();
    }
}

void StoreServer::OnMessage(net::LinkId link, const net::Frame &f)
{
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = lastSeenMs_.find(link);
        if (it != lastSeenMs_.end()) {
            it->second = NowMs();
        }
    }
    if (f.type == OP_HEARTBEAT) {
        Reply(link, f, ST_OK, "");
        return;
    }
    StoreMessage m;
    if (!UnpackMessage(f.body, &m)) {
        Reply(link, f, ST_INVALID_MESSAGE, "invalid message");
        return;
    }
    if (f.type == OP_WATCH_RANK_STATE) {
        std::lock_guard<std::mutex> g(mu_);
        rankWatchers_.emplace_back(link, f.seq);
        return;  // no immediate reply: notifications are pushed on this seq
    }
    if (f.type == OP_ARRIVE || f.type == OP_GATHER) {
        HandleRendezvous(link, f, m);
        return;
    }
    if (m.keys.size() != 1 || m.keys[0].empty() || m.keys[0].size() > MAX_KEY_LEN_SERVER) {
        Reply(link, f, ST_INVALID_KEY, "invalid key");
        return;
    }
    const std::string &key = m.keys[0];
    switch (f.type) {
        case OP_SET: {
            if (m.values.size() != 1) {
                Reply(link, f, ST_INVALID_MESSAGE, "set needs one value");
                return;
            }
            {
                std::lock_guard<std::mutex> g(mu_);
                backend_->Put(key, m.values[0]);
            }
            WakeWaiters(key, m.values[0]);
            if (opHook_) {
                opHook_(OP_SET, link, key, m.values[0], nullptr);
            }
            Reply(link, f, ST_OK, "success");
            return;
        }
        case OP_GET:
            HandleGet(link, f, m);
            return;
        case OP_ADD: {
            if (m.values.size() != 1) {
                Reply(link, f, ST_INVALID_MESSAGE, "add needs one value");
                return;
            }
            char *end = nullptr;
            errno = 0;
            long long delta = std::strtoll(m.values[0].c_str(), &end, 10);
            if (m.values[0].empty() || *end != '\0' || errno != 0) {
                Reply(link, f, ST_INVALID_MESSAGE, "add needs a decimal integer");
                return;
            }
            std::string text;
            bool created = false;
            {
                std::lock_guard<std::mutex> g(mu_);
                std::string cur;
                long long v = delta;
                if (backend_->Get(key, &cur)) {
                    v = std::strtoll(cur.c_str(), nullptr, 10) + delta;
                } else {
                    created = true;
                }
                text = std::to_string(v);
                backend_->Put(key, text);
            }
            if (created) {
                WakeWaiters(key, text);
            }
            if (opHook_ && delta > 0) {
                opHook_(OP_ADD, link, key, text, nullptr);
            }
            Reply(link, f, ST_OK, text);
            return;
        }
        case OP_REMOVE: {
            bool had;
            {
                std::lock_guard<std::mutex> g(mu_);
                had = backend_->Delete(key);
            }
            Reply(link, f, had ? ST_OK : ST_NOT_EXIST, had ? "success" : "not exist");
            return;
        }
        case OP_APPEND: {
            if (m.values.size() != 1) {
                Reply(link, f, ST_INVALID_MESSAGE, "append needs one value");
                return;
            }
            std::string whole;
            bool created = false;
            {
                std::lock_guard<std::mutex> g(mu_);
                std::string *cur = backend_->Mutable(key);
                if (cur == nullptr) {
                    backend_->Put(key, m.values[0]);
                    whole = m.values[0];
                    created = true;
                } else if (cur->size() + m.values[0].size() > MAX_VALUE_LEN) {
                    whole.clear();
                    created = false;
                    cur = nullptr;
                    // fallthrough to error below
                    Reply(link, f, ST_INVALID_MESSAGE, "value too large");
                    return;
                } else {
                    cur->append(m.values[0]);
                    whole = *cur;
                }
            }
            if (created) {
                WakeWaiters(key, whole);
            }
            if (opHook_) {
                opHook_(OP_APPEND, link, key, m.values[0], nullptr);
            }
            Reply(link, f, ST_OK, std::to_string(whole.size()));
            return;
        }
        case OP_WRITE: {
            if (m.values.size() != 1 || m.values[0].size() < 4) {
                Reply(link, f, ST_INVALID_MESSAGE, "write needs offset+data");
                return;
            }
            uint32_t off;
            std::memcpy(&off, m.values[0].data(), 4);
            size_t len = m.values[0].size() - 4;
            if ((uint64_t)off + len > MAX_VALUE_LEN) {
                Reply(link, f, ST_INVALID_MESSAGE, "write beyond the value limit");
                return;
            }
            std::string whole;
            bool created = false;
            {
                std::lock_guard<std::mutex> g(mu_);
                std::string *cur = backend_->Mutable(key);
                if (cur == nullptr) {
                    backend_->Put(key, std::string());
                    cur = backend_->Mutable(key);
                    created = true;
                }
                if (cur->size() < off + len) {
                    cur->resize(off + len, '\0');
                }
                std::memcpy(&(*cur)[off], m.values[0].data() + 4, len);
                whole = *cur;
            }
            if (created) {
                WakeWaiters(key, whole);
            }
            if (opHook_) {
                opHook_(OP_WRITE, link, key, m.values[0], nullptr);
            }
            Reply(link, f, ST_OK, "success");
            return;
        }
        case OP_CAS: {
            if (m.values.size() != 2) {
                Reply(link, f, ST_INVALID_MESSAGE, "cas needs expected+exchange");
                return;
            }
            std::string prev;
            bool created = false;
            {
                std::lock_guard<std::mutex> g(mu_);
                bool have = backend_->Get(key, &prev);
                if (!have && m.values[0].empty()) {
                    backend_->Put(key, m.values[1]);
                    created = true;
                } else if (have && prev == m.values[0]) {
                    backend_->Put(key, m.values[1]);
                }
            }
            if (created) {
                WakeWaiters(key, m.values[1]);
            }
            Reply(link, f, ST_OK, prev);
            return;
        }
        default:
            Reply(link, f, ST_INVALID_MESSAGE, "unknown op");
            return;
    }
}

void StoreServer::HouseKeeping()
{
    std::unique_lock<std::mutex> lk(mu_);
    uint64_t nextBeatCheck = NowMs() + GlobalTiming().heartbeatIntervalMs;
    uint64_t lastBeatCheck = NowMs();
    while (!stop_.load()) {
        uint64_t now = NowMs();
        uint64_t wake = nextBeatCheck;
        if (!timed_.empty()) {
            wake = std::min(wake, timed_.begin()->first);
        }
        if (wake > now) {
            cv_.wait_for(lk, std::chrono::milliseconds(std::min<uint64_t>(wake - now, 500)));
            if (stop_.load()) {
                break;
            }
            now = NowMs();
        }
        // 1. expire timed GETs
        std::vector<Waiter> expired;
        while (!timed_.empty() && timed_.begin()->first <= now) {
            auto ent = timed_.begin()->second;
            timed_.erase(timed_.begin());
            auto it = keyWaiters_.find(ent.first);
            if (it == keyWaiters_.end()) {
                continue;
            }
            auto &vec = it->second;
            for (size_t i = 0; i < vec.size(); i++) {
                if (vec[i].id == ent.second) {
                    expired.push_back(vec[i]);
                    vec.erase(vec.begin() + (long)i);
                    break;
                }
            }
            if (vec.empty()) {
                keyWaiters_.erase(it);
            }
        }
        // 2. heartbeat supervision
        std::vector<net::LinkId> dead;
        if (now >= nextBeatCheck) {
            const ServerTiming &t = GlobalTiming();
            nextBeatCheck = now + t.heartbeatIntervalMs;
            // A link is judged by what the event loop has read from it. If this thread overslept (the whole process was held:
            // eight ranks pinning 8 GiB of host memory each stopped one for ten seconds) or the event loop has not come round
            // lately, the silence is this server's, not the peers': their heartbeats sit unread in the sockets. Then every link
            // is taken as seen one interval ago and judged again on later passes.
            const uint64_t gap = now - lastBeatCheck;
            const uint64_t loopBeat = rpc_.LoopBeatMs();
            // (thresholds well above the jitter of a loaded machine: this thread wakes at least every interval, the event loop
            // at least every 200 ms)
            const uint64_t slack = std::max<uint64_t>(2ull * t.heartbeatIntervalMs, 1000);
            const bool ownStall = gap > t.heartbeatIntervalMs + slack || (loopBeat != 0 && now > loopBeat && now - loopBeat > slack);
            lastBeatCheck = now;
            if (ownStall) {
                MF_WARN("store server: was held for " << gap << " ms; heartbeat supervision starts over");
                for (auto &kv : lastSeenMs_) {
                    kv.second = std::max(kv.second, now - std::min<uint64_t>(now, t.heartbeatIntervalMs));
                }
            } else {
                for (auto &kv : lastSeenMs_) {
                    if ((now - kv.second) / t.heartbeatIntervalMs > t.heartbeatMissLimit) {
                        dead.push_back(kv.first);
                    }
                }
            }
        }
        lk.unlock();
        for (auto &w : expired) {
            ReplyText(w.link, w.seq, OP_GET, ST_TIMEOUT, "timeout");
        }
        for (auto l : dead) {
            MF_WARN("store server: link " << l << " missed its heartbeats, declaring it dead");
            LinkGone(l, true);
        }
        lk.lock();
    }
}

}  // namespace store
}  // namespace mf

#include "mf_rpc.h"

#include <algorithm>

#include "../util/mf_net_util.h"
#include "mf_tls.h"

#include <arpa/inet.h>
#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <ifaddrs.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <unistd.h>
#include <vector>

#include "../util/mf_log.h"

namespace mf {
namespace net {

// ---------------------------------------------------------------------------------------------- URL / address helpers

bool ParseUrl(const std::string &urlIn, Endpoint *out)
{
    std::string url = urlIn;
    bool v6 = false;
    if (url.rfind("tcp6://", 0) == 0) {
        url = url.substr(7);
        v6 = true;
    } else if (url.rfind("tcp://", 0) == 0) {
        url = url.substr(6);
    }
    if (url.empty()) {
        return false;
    }
    std::string host, port;
    if (url[0] == '[') {
        size_t rb = url.find(']');
        if (rb == std::string::npos || rb + 1 >= url.size() || url[rb + 1] != ':') {
            return false;
        }
        host = url.substr(1, rb - 1);
        port = url.substr(rb + 2);
        v6 = true;
    } else {
        size_t c = url.rfind(':');
        if (c == std::string::npos || c == 0) {
            return false;
        }
        host = url.substr(0, c);
        port = url.substr(c + 1);
        if (host.find(':') != std::string::npos) {
            v6 = true;  // bare IPv6 literal followed by :port
        }
    }
    if (host.empty() || port.empty() || port.size() > 5) {
        return false;
    }
    for (char ch : port) {
        if (ch < '0' || ch > '9') {
            return false;
        }
    }
    long p = std::strtol(port.c_str(), nullptr, 10);
    if (p <= 0 || p > 65535) {
        return false;
    }
    // Validate literals early so a typo fails at parse time rather than at connect time.
    unsigned char buf[16];
    if (v6) {
        if (inet_pton(AF_INET6, host.c_str(), buf) != 1) {
            return false;
        }
    } else if (std::isdigit((unsigned char)host[0])) {
        // Dotted quad: four 0-255 fields without leading zeros (0.0.0.0 is a legal listen address).
        if (!util::IsValidIpv4(host, true) || inet_pton(AF_INET, host.c_str(), buf) != 1) {
            return false;
        }
    }
    out->host = host;
    out->port = (uint16_t)p;
    out->v6 = v6;
    return true;
}

static int Resolve(const Endpoint &ep, sockaddr_storage *ss, socklen_t *len, bool passive)
{
    addrinfo hints{};
    hints.ai_family = ep.v6 ? AF_INET6 : AF_UNSPEC;
    hints.ai_socktype = SOCK_STREAM;
    hints.ai_flags = AI_NUMERICSERV | (passive ? AI_PASSIVE : 0);
    addrinfo *res = nullptr;
    std::string port = std::to_string(ep.port);
    int rc = getaddrinfo(ep.host.c_str(), port.c_str(), &hints, &res);
    if (rc != 0 || res == nullptr) {
        return -1;
    }
    std::memcpy(ss, res->ai_addr, res->ai_addrlen);
    *len = res->ai_addrlen;
    freeaddrinfo(res);
    return 0;
}

std::string LocalIpToward(const Endpoint &target)
{
    sockaddr_storage ss{};
    socklen_t len = 0;
    if (Resolve(target, &ss, &len, false) != 0) {
        return "";
    }
    int fd = ::socket(ss.ss_family, SOCK_DGRAM | SOCK_CLOEXEC, 0);
    if (fd < 0) {
        return "";
    }
    std::string out;
    if (::connect(fd, (sockaddr *)&ss, len) == 0) {
        sockaddr_storage me{};
        socklen_t ml = sizeof(me);
        if (getsockname(fd, (sockaddr *)&me, &ml) == 0) {
            char buf[INET6_ADDRSTRLEN] = {0};
            if (me.ss_family == AF_INET) {
                inet_ntop(AF_INET, &((sockaddr_in *)&me)->sin_addr, buf, sizeof(buf));
            } else {
                inet_ntop(AF_INET6, &((sockaddr_in6 *)&me)->sin6_addr, buf, sizeof(buf));
            }
            out = buf;
        }
    }
    ::close(fd);
    return out;
}

std::vector<std::string> LocalIpv4List()
{
    std::vector<std::string> out;
    ifaddrs *ifs = nullptr;
    if (getifaddrs(&ifs) != 0) {
        return out;
    }
    for (ifaddrs *p = ifs; p != nullptr; p = p->ifa_next) {
        if (p->ifa_addr == nullptr || p->ifa_addr->sa_family != AF_INET) {
            continue;
        }
        char buf[INET_ADDRSTRLEN] = {0};
        inet_ntop(AF_INET, &((sockaddr_in *)p->ifa_addr)->sin_addr, buf, sizeof(buf));
        if (std::strncmp(buf, "127.", 4) != 0) {
            out.emplace_back(buf);
        }
    }
    freeifaddrs(ifs);
    return out;
}

static void SetNonBlock(int fd)
{
    int fl = fcntl(fd, F_GETFL, 0);
    fcntl(fd, F_SETFL, fl | O_NONBLOCK);
}

static void SetNoDelay(int fd)
{
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}

static std::string Encode(const Frame &f)
{
    WireHeader h{kWireMagic, f.type, f.result, (uint32_t)f.body.size(), f.seq};
    std::string out;
    out.resize(sizeof(h) + f.body.size());
    std::memcpy(&out[0], &h, sizeof(h));
    if (!f.body.empty()) {
        std::memcpy(&out[sizeof(h)], f.body.data(), f.body.size());
    }
    return out;
}

// ---------------------------------------------------------------------------------------------- server

struct RpcServer::Conn {
    std::unique_ptr<TlsSession> tls;  // guarded by RpcServer::mu_
    int fd{-1};
    LinkId id{0};
    bool hello{false};
    bool dead{false};
    Frame frame;  // the frame being delivered (I/O thread only)
    std::string in;
    std::deque<std::string> out;  // guarded by RpcServer::mu_
    size_t outOff{0};
    bool wantWrite{false};
};

RpcServer::RpcServer() = default;
RpcServer::~RpcServer() { Stop(); }

void RpcServer::SetTls(std::shared_ptr<TlsContext> ctx) { tls_ = std::move(ctx); }

void RpcServer::SetHandlers(MsgHandler onMsg, LinkUpHandler onUp, LinkDownHandler onDown)
{
    onMsg_ = std::move(onMsg);
    onUp_ = std::move(onUp);
    onDown_ = std::move(onDown);
}

int RpcServer::Start(const Endpoint &ep)
{
    if (running_.load()) {
        return 0;
    }
    sockaddr_storage ss{};
    socklen_t len = 0;
    if (Resolve(ep, &ss, &len, true) != 0) {
        MF_ERROR("rpc server: cannot resolve " << ep.host);
        return -EINVAL;
    }
    listenFd_ = ::socket(ss.ss_family, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (listenFd_ < 0) {
        return -errno;
    }
    int one = 1;
    setsockopt(listenFd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    if (::bind(listenFd_, (sockaddr *)&ss, len) != 0) {
        int e = errno;
        ::close(listenFd_);
        listenFd_ = -1;
        return -e;
    }
    if (::listen(listenFd_, 512) != 0) {
        int e = errno;
        ::close(listenFd_);
        listenFd_ = -1;
        return -e;
    }
    sockaddr_storage me{};
    socklen_t ml = sizeof(me);
    getsockname(listenFd_, (sockaddr *)&me, &ml);
    port_ = ntohs(me.ss_family == AF_INET ? ((sockaddr_in *)&me)->sin_port : ((sockaddr_in6 *)&me)->sin6_port);
    SetNonBlock(listenFd_);
    epfd_ = epoll_create1(EPOLL_CLOEXEC);
    wakeFd_ = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
    epoll_event ev{};
    ev.events = EPOLLIN;
    ev.data.fd = listenFd_;
    epoll_ctl(epfd_, EPOLL_CTL_ADD, listenFd_, &ev);
    ev.data.fd = wakeFd_;
    epoll_ctl(epfd_, EPOLL_CTL_ADD, wakeFd_, &ev);
    running_.store(true);
    io_ = std::thread([this]() { Loop(); });
    return 0;
}

void RpcServer::Stop()
{
    if (!running_.load()) {
        return;
    }
    {
        // Orderly end: every peer hears it before its socket closes.
        std::vector<LinkId> ids;
        {
            std::lock_guard<std::mutex> g(mu_);
            for (auto &kv : conns_) {
                if (kv.second->hello) {
                    ids.push_back(kv.first);
                }
            }
        }
        Frame bye;
        bye.type = MSG_GOODBYE;
        for (LinkId id : ids) {
            Send(id, bye);
        }
    }
    if (!running_.exchange(false)) {
        return;
    }
    Wake();
    if (io_.joinable()) {
        io_.join();
    }
    std::vector<std::shared_ptr<Conn>> all;
    {
        std::lock_guard<std::mutex> g(mu_);
        for (auto &kv : conns_) {
            all.push_back(kv.second);
        }
        conns_.clear();
        byFd_.clear();
    }
    for (auto &c : all) {
        ::close(c->fd);
    }
    ::close(listenFd_);
    ::close(epfd_);
    ::close(wakeFd_);
    listenFd_ = epfd_ = wakeFd_ = -1;
}

void RpcServer::Wake()
{
    uint64_t one = 1;
    if (wakeFd_ >= 0) {
        ssize_t r = ::write(wakeFd_, &one, sizeof(one));
        (void)r;
    }
}

size_t RpcServer::LinkCount()
{
    std::lock_guard<std::mutex> g(mu_);
    return conns_.size();
}

int RpcServer::Send(LinkId link, const Frame &f)
{
    std::string bytes = Encode(f);
    std::lock_guard<std::mutex> g(mu_);
    auto it = conns_.find(link);
    if (it == conns_.end() || it->second->dead) {
        return -1;
    }
    Conn &c = *it->second;
    if (c.tls) {
        std::string wire;
        if (c.tls->Encrypt(bytes.data(), bytes.size(), &wire) != 0) {
            MF_WARN("rpc server: tls write failed on link " << c.id << ": " << c.tls->LastError());
            return -1;
        }
        bytes.swap(wire);
    }
    return SendBytesLocked(c, std::move(bytes));
}

int RpcServer::SendWithPayload(LinkId link, const Frame &f, const void *payload, size_t payloadLen)
{
    if (payloadLen > kMaxBodyLen) {
        return -1;
    }
    WireHeader h{kWireMagic, f.type, f.result, (uint32_t)payloadLen, f.seq};
    std::lock_guard<std::mutex> g(mu_);
    auto it = conns_.find(link);
    if (it == conns_.end() || it->second->dead) {
        return -1;
    }
    Conn &c = *it->second;
    if (c.tls || !c.out.empty()) {
        // Encrypted links need one plaintext; a link with a backlog must keep its order: both take the copying path.
        std::string bytes;
        bytes.reserve(sizeof(h) + payloadLen);
        bytes.append((const char *)&h, sizeof(h));
        bytes.append((const char *)payload, payloadLen);
        if (c.tls) {
            std::string wire;
            if (c.tls->Encrypt(bytes.data(), bytes.size(), &wire) != 0) {
                return -1;
            }
            bytes.swap(wire);
        }
        return SendBytesLocked(c, std::move(bytes));
    }
    iovec iov[2] = {{&h, sizeof(h)}, {const_cast<void *>(payload), payloadLen}};
    size_t idx = 0;
    while (idx < 2) {
        msghdr mh{};
        mh.msg_iov = iov + idx;
        mh.msg_iovlen = 2 - idx;
        ssize_t n = ::sendmsg(c.fd, &mh, MSG_NOSIGNAL | MSG_DONTWAIT);
        if (n < 0 && errno == EINTR) {
            continue;
        }
        if (n <= 0) {
            break;  // EAGAIN or error: the rest is queued and the I/O thread finishes or drops it
        }
        size_t adv = (size_t)n;
        while (adv > 0 && idx < 2) {
            const size_t take = adv < iov[idx].iov_len ? adv : iov[idx].iov_len;
            iov[idx].iov_base = (char *)iov[idx].iov_base + take;
            iov[idx].iov_len -= take;
            adv -= take;
            if (iov[idx].iov_len == 0) {
                idx++;
            }
        }
    }
    if (idx == 2) {
        return 0;
    }
    std::string rest;
    for (size_t i = idx; i < 2; i++) {
        rest.append((const char *)iov[i].iov_base, iov[i].iov_len);
    }
    return SendBytesLocked(c, std::move(rest));
}

int RpcServer::SendBytesLocked(Conn &c, std::string bytes)
{
    size_t off = 0;
    if (c.out.empty()) {
        // Fast path: nothing queued, try to push the bytes out right now.
        while (off < bytes.size()) {
            ssize_t n = ::send(c.fd, bytes.data() + off, bytes.size() - off, MSG_NOSIGNAL | MSG_DONTWAIT);
            if (n > 0) {
                off += (size_t)n;
            } else if (n < 0 && errno == EINTR) {
                continue;
            } else {
                break;  // EAGAIN or error: the I/O thread finishes or drops it
            }
        }
        if (off == bytes.size()) {
            return 0;
        }
    }
    c.out.emplace_back(bytes.substr(off));
    if (!c.wantWrite) {
        c.wantWrite = true;
        epoll_event ev{};
        ev.events = EPOLLIN | EPOLLOUT;
        ev.data.fd = c.fd;
        epoll_ctl(epfd_, EPOLL_CTL_MOD, c.fd, &ev);
    }
    return 0;
}

void RpcServer::CloseLink(LinkId link)
{
    {
        std::lock_guard<std::mutex> g(mu_);
        pendingClose_.push_back(link);
    }
    Wake();
}

void RpcServer::Accept()
{
    while (true) {
        int fd = ::accept4(listenFd_, nullptr, nullptr, SOCK_CLOEXEC | SOCK_NONBLOCK);
        if (fd < 0) {
            return;
        }
        SetNoDelay(fd);
        auto c = std::make_shared<Conn>();
        c->fd = fd;
        if (tls_) {
            c->tls = tls_->NewSession();
            if (!c->tls) {
                ::close(fd);
                continue;
            }
        }
        {
            std::lock_guard<std::mutex> g(mu_);
            c->id = nextLink_++;
            conns_[c->id] = c;
            byFd_[fd] = c->id;
        }
        epoll_event ev{};
        ev.events = EPOLLIN;
        ev.data.fd = fd;
        epoll_ctl(epfd_, EPOLL_CTL_ADD, fd, &ev);
    }
}

void RpcServer::Drop(const std::shared_ptr<Conn> &c)
{
    bool wasUp;
    {
        std::lock_guard<std::mutex> g(mu_);
        if (c->dead) {
            return;
        }
        c->dead = true;
        wasUp = c->hello;
        conns_.erase(c->id);
        byFd_.erase(c->fd);
    }
    epoll_ctl(epfd_, EPOLL_CTL_DEL, c->fd, nullptr);
    ::close(c->fd);
    if (wasUp && onDown_) {
        onDown_(c->id);
    }
}

void RpcServer::Flush(const std::shared_ptr<Conn> &c)
{
    std::lock_guard<std::mutex> g(mu_);
    while (!c->out.empty()) {
        std::string &front = c->out.front();
        ssize_t n = ::send(c->fd, front.data() + c->outOff, front.size() - c->outOff, MSG_NOSIGNAL | MSG_DONTWAIT);
        if (n > 0) {
            c->outOff += (size_t)n;
            if (c->outOff == front.size()) {
                c->out.pop_front();
                c->outOff = 0;
            }
        } else if (n < 0 && errno == EINTR) {
            continue;
        } else {
            break;
        }
    }
    if (c->out.empty() && c->wantWrite) {
        c->wantWrite = false;
        epoll_event ev{};
        ev.events = EPOLLIN;
        ev.data.fd = c->fd;
        epoll_ctl(epfd_, EPOLL_CTL_MOD, c->fd, &ev);
    }
}

void RpcServer::OnReadable(const std::shared_ptr<Conn> &c)
{
    char buf[65536];
    std::string raw;
    std::string &sink = c->tls ? raw : c->in;
    bool eof = false;
    while (true) {
        ssize_t n = ::recv(c->fd, buf, sizeof(buf), 0);
        if (n > 0) {
            sink.append(buf, (size_t)n);
            if (sink.size() >= (8u << 20)) {
                break;  // hand what has arrived to the parser before reading on (the socket is level-triggered)
            }
            // A short read does not mean the socket is empty (a bulk sender delivers segment by segment): read until EAGAIN.
        } else if (n == 0) {
            eof = true;
            break;
        } else if (errno == EINTR) {
            continue;
        } else if (errno == EAGAIN || errno == EWOULDBLOCK) {
            break;
        } else {
            eof = true;
            break;
        }
    }
    if (c->tls && !raw.empty()) {
        // Ciphertext in, plaintext out; records the session itself wants to send (handshake, alerts) go to the queue.
        std::string wire;
        bool ok;
        {
            std::lock_guard<std::mutex> g(mu_);
            ok = c->tls->Feed(raw.data(), raw.size()) && c->tls->Pump(&c->in, &wire) == 0;
            if (!wire.empty() && !c->dead) {
                SendBytesLocked(*c, std::move(wire));
            }
        }
        if (!ok) {
            MF_WARN("rpc server: tls failure on link " << c->id << " (" << c->tls->LastError() << "), dropping the link");
            Flush(c);
            Drop(c);
            return;
        }
    }
    if (eof && c->in.size() < sizeof(WireHeader)) {
        Drop(c);
        return;
    }
    size_t pos = 0;
    while (c->in.size() - pos >= sizeof(WireHeader)) {
        WireHeader h;
        std::memcpy(&h, c->in.data() + pos, sizeof(h));
        if (h.magic != kWireMagic || h.bodyLen > kMaxBodyLen) {
            MF_WARN("rpc server: bad frame on link " << c->id << ", dropping the link");
            Drop(c);
            return;
        }
        if (c->in.size() - pos < sizeof(h) + h.bodyLen) {
            break;
        }
        Frame &f = c->frame;  // one per link, so that a stream of large frames reuses one buffer instead of allocating afresh
        f.type = h.type;
        f.result = h.result;
        f.seq = h.seq;
        f.body.assign(c->in.data() + pos + sizeof(h), h.bodyLen);
        pos += sizeof(h) + h.bodyLen;
        if (!c->hello) {
            HelloBody hb{};
            bool ok = f.type == MSG_HELLO && f.body.size() == sizeof(hb);
            if (ok) {
                std::memcpy(&hb, f.body.data(), sizeof(hb));
                ok = hb.version == kWireVersion;
            }
            if (ok && onUp_) {
                ok = onUp_(c->id, hb.peerId);
            }
            Frame ack;
            ack.type = MSG_HELLO_ACK;
            ack.seq = f.seq;
            ack.result = (int16_t)(ok ? 0 : -1);
            c->hello = ok;
            Send(c->id, ack);
            if (!ok) {
                Flush(c);
                Drop(c);
                return;
            }
            continue;
        }
        if (onMsg_) {
            onMsg_(c->id, f);
        }
        if (c->dead) {
            return;
        }
    }
    if (pos > 0) {
        c->in.erase(0, pos);
    }
    if (eof) {
        Drop(c);
    }
}

void RpcServer::Loop()
{
    std::vector<epoll_event> evs(128);
    while (running_.load()) {
        loopBeatMs_.store(NowMs(), std::memory_order_relaxed);
        int n = epoll_wait(epfd_, evs.data(), (int)evs.size(), 200);
        if (n < 0 && errno != EINTR) {
            break;
        }
        for (int i = 0; i < n; i++) {
            int fd = evs[i].data.fd;
            if (fd == listenFd_) {
                Accept();
                continue;
            }
            if (fd == wakeFd_) {
                uint64_t v;
                ssize_t r = ::read(wakeFd_, &v, sizeof(v));
                (void)r;
                continue;
            }
            std::shared_ptr<Conn> c;
            {
                std::lock_guard<std::mutex> g(mu_);
                auto it = byFd_.find(fd);
                if (it != byFd_.end()) {
                    auto ct = conns_.find(it->second);
                    if (ct != conns_.end()) {
                        c = ct->second;
                    }
                }
            }
            if (!c) {
                continue;
            }
            if (evs[i].events & (EPOLLHUP | EPOLLERR)) {
                // Deliver what is still readable first so that a request followed by close is not lost.
                OnReadable(c);
                Drop(c);
                continue;
            }
            if (evs[i].events & EPOLLOUT) {
                Flush(c);
            }
            if (evs[i].events & EPOLLIN) {
                OnReadable(c);
            }
        }
        std::deque<LinkId> closing;
        {
            std::lock_guard<std::mutex> g(mu_);
            closing.swap(pendingClose_);
        }
        for (LinkId id : closing) {
            std::shared_ptr<Conn> c;
            {
                std::lock_guard<std::mutex> g(mu_);
                auto it = conns_.find(id);
                if (it != conns_.end()) {
                    c = it->second;
                }
            }
            if (c) {
                Drop(c);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------- client

RpcClient::RpcClient() = default;
RpcClient::~RpcClient() { Close(); }

void RpcClient::SetTls(std::shared_ptr<TlsContext> ctx) { tlsCtx_ = std::move(ctx); }

static bool ReadFull(int fd, void *buf, size_t len)
{
    char *p = (char *)buf;
    while (len > 0) {
        ssize_t n = ::recv(fd, p, len, 0);
        if (n > 0) {
            p += n;
            len -= (size_t)n;
        } else if (n < 0 && errno == EINTR) {
            continue;
        } else {
            return false;
        }
    }
    return true;
}

static bool WriteFull(int fd, const void *buf, size_t len)
{
    const char *p = (const char *)buf;
    while (len > 0) {
        ssize_t n = ::send(fd, p, len, MSG_NOSIGNAL);
        if (n > 0) {
            p += n;
            len -= (size_t)n;
        } else if (n < 0 && errno == EINTR) {
            continue;
        } else {
            return false;
        }
    }
    return true;
}

bool RpcClient::IoWrite(const void *p, size_t n)
{
    if (!tls_) {
        return WriteFull(fd_, p, n);
    }
    std::string wire;
    {
        std::lock_guard<std::mutex> g(tlsMu_);
        if (tls_->Encrypt(static_cast<const char *>(p), n, &wire) != 0) {
            return false;
        }
    }
    return WriteFull(fd_, wire.data(), wire.size());
}

bool RpcClient::IoRead(void *p, size_t n)
{
    if (!tls_) {
        return ReadFull(fd_, p, n);
    }
    char buf[65536];
    while (plainBuf_.size() - plainOff_ < n) {
        ssize_t r = ::recv(fd_, buf, sizeof(buf), 0);
        if (r < 0 && errno == EINTR) {
            continue;
        }
        if (r <= 0) {
            return false;
        }
        // Whatever the session wants to send in response (key updates, alerts) must leave in record order: take the send
        // lock first, as every writer does.
        std::lock_guard<std::mutex> gs(sendMu_);
        std::string wire;
        int rc;
        {
            std::lock_guard<std::mutex> g(tlsMu_);
            rc = tls_->Feed(buf, (size_t)r) ? tls_->Pump(&plainBuf_, &wire) : -1;
        }
        if (!wire.empty()) {
            WriteFull(fd_, wire.data(), wire.size());
        }
        if (rc < 0) {
            MF_WARN("rpc client: tls failure: " << tls_->LastError());
            return false;
        }
    }
    std::memcpy(p, plainBuf_.data() + plainOff_, n);
    plainOff_ += n;
    if (plainOff_ == plainBuf_.size()) {
        plainBuf_.clear();
        plainOff_ = 0;
    }
    return true;
}

bool RpcClient::TlsHandshake(int fd)
{
    tls_ = tlsCtx_->NewSession();
    if (!tls_) {
        return false;
    }
    plainBuf_.clear();
    plainOff_ = 0;
    char buf[16384];
    while (true) {
        std::string wire;
        if (tls_->Pump(&plainBuf_, &wire) < 0) {
            if (!wire.empty()) {
                WriteFull(fd, wire.data(), wire.size());
            }
            MF_WARN("rpc client: tls handshake failed: " << tls_->LastError());
            return false;
        }
        if (!wire.empty() && !WriteFull(fd, wire.data(), wire.size())) {
            return false;
        }
        if (tls_->HandshakeDone()) {
            return true;
        }
        ssize_t r = ::recv(fd, buf, sizeof(buf), 0);
        if (r < 0 && errno == EINTR) {
            continue;
        }
        if (r <= 0 || !tls_->Feed(buf, (size_t)r)) {
            return false;
        }
    }
}

int RpcClient::Connect(const Endpoint &ep, uint64_t peerId, int retries, int retryDelayMs)
{
    Close();
    closing_.store(false);
    goodbye_.store(false);
    sockaddr_storage ss{};
    socklen_t len = 0;
    if (Resolve(ep, &ss, &len, false) != 0) {
        MF_ERROR("rpc client: cannot resolve " << ep.host);
        return -1;
    }
    for (int attempt = 0; attempt < retries && !closing_.load(); attempt++) {
        int fd = ::socket(ss.ss_family, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (fd < 0) {
            return -1;
        }
        if (::connect(fd, (sockaddr *)&ss, len) == 0) {
            SetNoDelay(fd);
            // Handshake: hello → ack, done synchronously before the reader thread exists.
            HelloBody hb{kWireVersion, 0, 0, peerId};
            Frame hello;
            hello.type = MSG_HELLO;
            hello.body.assign((const char *)&hb, sizeof(hb));
            std::string bytes = Encode(hello);
            WireHeader h{};
            // The acknowledgement may take long when the server's process is stalled by the kernel (eight ranks pinning 8 GiB
            // of host memory each held a server's loop for ten seconds in one run): wait as long as the caller allowed for
            // connecting, at least 30 s.
            const long budgetMs = (long)retries * (long)retryDelayMs;
            timeval tv{std::max(30L, budgetMs / 1000), 0};
            setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
            fd_ = fd;
            tls_.reset();
            bool ok = tlsCtx_ == nullptr || TlsHandshake(fd);
            ok = ok && IoWrite(bytes.data(), bytes.size()) && IoRead(&h, sizeof(h)) && h.magic == kWireMagic && h.type == MSG_HELLO_ACK &&
                 h.bodyLen == 0 && h.result == RPC_OK;
            if (!ok) {
                fd_ = -1;
                tls_.reset();
            }
            if (ok) {
                tv = timeval{0, 0};
                setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
                connected_.store(true);
                reader_ = std::thread([this]() { ReaderLoop(); });
                return 0;
            }
            ::close(fd);
            MF_WARN("rpc client: handshake with " << ep.host << ":" << ep.port << " rejected");
            return -2;
        }
        ::close(fd);
        if (attempt + 1 < retries) {
            usleep((useconds_t)retryDelayMs * 1000);
        }
    }
    return -1;
}

void RpcClient::Close()
{
    closing_.store(true);
    if (fd_ >= 0) {
        ::shutdown(fd_, SHUT_RDWR);
    }
    if (reader_.joinable()) {
        if (reader_.get_id() == std::this_thread::get_id()) {
            reader_.detach();
        } else {
            reader_.join();
        }
    }
    if (fd_ >= 0) {
        ::close(fd_);
        fd_ = -1;
    }
    connected_.store(false);
    FailAll();
}

void RpcClient::FailAll()
{
    std::unordered_map<uint32_t, std::shared_ptr<Pending>> all;
    {
        std::lock_guard<std::mutex> g(mu_);
        all.swap(pending_);
    }
    for (auto &kv : all) {
        std::lock_guard<std::mutex> g(kv.second->mu);
        kv.second->failed = true;
        kv.second->done = true;
        kv.second->cv.notify_all();
    }
}

int RpcClient::SendFrame(uint16_t type, uint32_t seq, const std::string &body) { return SendParts(type, seq, body.data(), body.size(), nullptr, 0); }

int RpcClient::SendParts(uint16_t type, uint32_t seq, const void *head, size_t headLen, const void *payload, size_t payloadLen)
{
    if (headLen + payloadLen > kMaxBodyLen) {
        return -1;
    }
    WireHeader h{kWireMagic, type, 0, (uint32_t)(headLen + payloadLen), seq};
    std::lock_guard<std::mutex> g(sendMu_);
    if (!connected_.load() || fd_ < 0) {
        return -1;
    }
    if (tls_) {
        // The record layer needs one contiguous plaintext anyway.
        std::string bytes;
        bytes.reserve(sizeof(h) + headLen + payloadLen);
        bytes.append((const char *)&h, sizeof(h));
        bytes.append((const char *)head, headLen);
        bytes.append((const char *)payload, payloadLen);
        return IoWrite(bytes.data(), bytes.size()) ? 0 : -1;
    }
    // Plain TCP: wire header, head and payload leave from where they lie.
    iovec iov[3] = {{&h, sizeof(h)}, {const_cast<void *>(head), headLen}, {const_cast<void *>(payload), payloadLen}};
    size_t idx = 0, left = sizeof(h) + headLen + payloadLen;
    while (left > 0) {
        while (idx < 3 && iov[idx].iov_len == 0) {
            idx++;
        }
        msghdr mh{};
        mh.msg_iov = iov + idx;
        mh.msg_iovlen = 3 - idx;
        ssize_t n = ::sendmsg(fd_, &mh, MSG_NOSIGNAL);
        if (n < 0 && errno == EINTR) {
            continue;
        }
        if (n <= 0) {
            return -1;
        }
        left -= (size_t)n;
        size_t adv = (size_t)n;
        while (adv > 0 && idx < 3) {
            const size_t take = adv < iov[idx].iov_len ? adv : iov[idx].iov_len;
            iov[idx].iov_base = (char *)iov[idx].iov_base + take;
            iov[idx].iov_len -= take;
            adv -= take;
            if (iov[idx].iov_len == 0) {
                idx++;
            }
        }
    }
    return 0;
}

int RpcClient::Call(uint16_t type, const std::string &body, Frame *reply, int64_t timeoutMs)
{
    return CallGather(type, body.data(), body.size(), nullptr, 0, nullptr, 0, reply, timeoutMs);
}

int RpcClient::CallGather(uint16_t type, const void *head, size_t headLen, const void *payload, size_t payloadLen, void *sink, size_t sinkLen,
                          Frame *reply, int64_t timeoutMs)
{
    if (!connected_.load()) {
        return RPC_IO_ERROR;
    }
    uint32_t seq = nextSeq_.fetch_add(1);
    if (seq == 0) {
        seq = nextSeq_.fetch_add(1);
    }
    auto p = std::make_shared<Pending>();
    p->sink = sink;
    p->sinkLen = sinkLen;
    {
        std::lock_guard<std::mutex> g(mu_);
        pending_[seq] = p;
    }
    if (SendParts(type, seq, head, headLen, payload, payloadLen) != 0) {
        std::lock_guard<std::mutex> g(mu_);
        pending_.erase(seq);
        return RPC_IO_ERROR;
    }
    std::unique_lock<std::mutex> lk(p->mu);
    if (timeoutMs < 0) {
        p->cv.wait(lk, [&]() { return p->done; });
    } else if (!p->cv.wait_for(lk, std::chrono::milliseconds(timeoutMs), [&]() { return p->done; })) {
        p->abandoned = true;  // under p->mu: the reader fills a sink only while holding it, so it is not in the sink now
        lk.unlock();
        std::lock_guard<std::mutex> g(mu_);
        pending_.erase(seq);
        return RPC_TIMEOUT;
    }
    if (p->failed) {
        return RPC_IO_ERROR;
    }
    if (reply != nullptr) {
        *reply = std::move(p->reply);
    }
    return RPC_OK;
}

uint32_t RpcClient::CallPersistent(uint16_t type, const std::string &body, PersistCb cb)
{
    if (!connected_.load()) {
        return 0;
    }
    uint32_t seq = nextSeq_.fetch_add(1);
    if (seq == 0) {
        seq = nextSeq_.fetch_add(1);
    }
    auto p = std::make_shared<Pending>();
    p->persist = std::move(cb);
    {
        std::lock_guard<std::mutex> g(mu_);
        pending_[seq] = p;
    }
    if (SendFrame(type, seq, body) != 0) {
        std::lock_guard<std::mutex> g(mu_);
        pending_.erase(seq);
        return 0;
    }
    return seq;
}

void RpcClient::Cancel(uint32_t seq)
{
    std::lock_guard<std::mutex> g(mu_);
    pending_.erase(seq);
}

void RpcClient::ReaderLoop()
{
    while (!closing_.load()) {
        WireHeader h{};
        if (!IoRead(&h, sizeof(h)) || h.magic != kWireMagic || h.bodyLen > kMaxBodyLen) {
            break;
        }
        Frame f;
        f.type = h.type;
        f.result = h.result;
        f.seq = h.seq;
        // A caller that handed in a buffer of exactly the body's size gets the body read straight into it.
        std::shared_ptr<Pending> direct;
        if (h.bodyLen > 0 && h.result == 0 && h.type != MSG_GOODBYE) {
            std::lock_guard<std::mutex> g(mu_);
            auto it = pending_.find(h.seq);
            if (it != pending_.end() && it->second->sink != nullptr && it->second->sinkLen == h.bodyLen && !it->second->persist) {
                direct = it->second;
            }
        }
        bool filled = false;
        if (direct && !tls_) {
            // The caller's buffer is written only while the caller's mutex is held, and the mutex is held only while bytes
            // that have already arrived are copied out of the socket: a caller whose wait runs out is never kept waiting by a
            // peer that stalls in the middle of a body. If the caller has left, the rest goes to a scratch buffer.
            size_t got = 0;
            std::string scratch;
            bool broken = false;
            while (got < h.bodyLen && !broken) {
                pollfd pfd{fd_, POLLIN, 0};
                int pr = ::poll(&pfd, 1, 200);
                if (pr < 0 && errno != EINTR) {
                    broken = true;
                    break;
                }
                if (pr <= 0) {
                    if (closing_.load()) {
                        broken = true;
                    }
                    continue;
                }
                std::lock_guard<std::mutex> g(direct->mu);
                char *dstp = nullptr;
                if (!direct->abandoned && scratch.empty()) {
                    dstp = (char *)direct->sink + got;
                } else {
                    if (scratch.empty()) {
                        scratch.resize(h.bodyLen);  // what was already delivered in place is lost with the caller: nobody reads it
                    }
                    dstp = &scratch[got];
                }
                while (got < h.bodyLen) {  // take everything that has arrived; none of these calls blocks
                    ssize_t n = ::recv(fd_, dstp, h.bodyLen - got, MSG_DONTWAIT);
                    if (n > 0) {
                        got += (size_t)n;
                        dstp += n;
                    } else {
                        if (n == 0 || (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)) {
                            broken = true;
                        }
                        break;
                    }
                }
            }
            if (broken) {
                break;
            }
            filled = scratch.empty();
            if (!filled) {
                f.body.swap(scratch);
            }
        }
        if (!filled && f.body.size() != h.bodyLen) {
            f.body.resize(h.bodyLen);
            if (h.bodyLen > 0 && !IoRead(&f.body[0], h.bodyLen)) {
                break;
            }
        }
        if (f.type == MSG_GOODBYE) {
            goodbye_.store(true);  // the close that follows is the end of the job, not a failure
            continue;
        }
        std::shared_ptr<Pending> p;
        {
            std::lock_guard<std::mutex> g(mu_);
            auto it = pending_.find(f.seq);
            if (it == pending_.end()) {
                continue;  // late reply of a timed-out call
            }
            p = it->second;
            if (!p->persist) {
                pending_.erase(it);
            }
        }
        if (p->persist) {
            p->persist(f);
        } else {
            std::lock_guard<std::mutex> g(p->mu);
            p->reply = std::move(f);
            p->done = true;
            p->cv.notify_all();
        }
    }
    bool wasConnected = connected_.exchange(false);
    FailAll();
    if (wasConnected && !closing_.load() && onBroken_) {
        onBroken_();
    }
}

}  // namespace net
}  // namespace mf

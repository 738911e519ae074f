#include "mf_fd_channel.h"

#include <algorithm>
#include <cerrno>
#include <cstddef>
#include <cstring>
#include <fcntl.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include "../util/mf_log.h"
#include "../util/mf_retry.h"

namespace mf {
namespace hybm {

FdChannel &FdChannel::Instance()
{
    static FdChannel *c = new FdChannel();
    return *c;
}

static socklen_t FillAddr(sockaddr_un *addr, const std::string &name)
{
    std::memset(addr, 0, sizeof(*addr));
    addr->sun_family = AF_UNIX;
    // Abstract namespace: sun_path[0] == 0, no file-system entry, vanishes with the process.
    size_t n = std::min(name.size(), sizeof(addr->sun_path) - 2);
    std::memcpy(addr->sun_path + 1, name.data(), n);
    return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

int FdChannel::Start()
{
    if (listenFd_ >= 0) {
        return 0;
    }
    int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) {
        MF_ERROR("fd channel: socket failed: " << strerror(errno));
        return -1;
    }
    name_ = "mf_fd_" + std::to_string((int)getpid()) + "_" + std::to_string(NowNs() & 0xffffff);
    sockaddr_un addr;
    socklen_t len = FillAddr(&addr, name_);
    if (::bind(fd, (sockaddr *)&addr, len) != 0 || ::listen(fd, 128) != 0) {
        MF_ERROR("fd channel: bind/listen failed: " << strerror(errno));
        ::close(fd);
        return -1;
    }
    listenFd_ = fd;
    stop_.store(false);
    server_ = std::thread([this]() { Loop(); });
    return 0;
}

const std::string &FdChannel::Name()
{
    std::lock_guard<std::mutex> g(mu_);
    Start();
    return name_;
}

uint64_t FdChannel::Publish(int fd)
{
    std::lock_guard<std::mutex> g(mu_);
    if (Start() != 0) {
        return 0;
    }
    int copy = ::fcntl(fd, F_DUPFD_CLOEXEC, 0);
    if (copy < 0) {
        return 0;
    }
    uint64_t token = ((uint64_t)getpid() << 32) | nextToken_++;
    fds_[token] = copy;
    return token;
}

void FdChannel::Unpublish(uint64_t token)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = fds_.find(token);
    if (it != fds_.end()) {
        ::close(it->second);
        fds_.erase(it);
    }
}

static int SendFd(int sock, int fd)
{
    char data = fd >= 0 ? 'F' : 'N';
    iovec iov{&data, 1};
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char ctrl[CMSG_SPACE(sizeof(int))];
    if (fd >= 0) {
        std::memset(ctrl, 0, sizeof(ctrl));
        msg.msg_control = ctrl;
        msg.msg_controllen = sizeof(ctrl);
        cmsghdr *c = CMSG_FIRSTHDR(&msg);
        c->cmsg_level = SOL_SOCKET;
        c->cmsg_type = SCM_RIGHTS;
        c->cmsg_len = CMSG_LEN(sizeof(int));
        std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
    }
    return ::sendmsg(sock, &msg, MSG_NOSIGNAL) == 1 ? 0 : -1;
}

static int RecvFd(int sock)
{
    char data = 0;
    iovec iov{&data, 1};
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char ctrl[CMSG_SPACE(sizeof(int))];
    std::memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    if (::recvmsg(sock, &msg, MSG_CMSG_CLOEXEC) != 1 || data != 'F') {
        return -1;
    }
    for (cmsghdr *c = CMSG_FIRSTHDR(&msg); c != nullptr; c = CMSG_NXTHDR(&msg, c)) {
        if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
            int fd;
            std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
            return fd;
        }
    }
    return -1;
}

void FdChannel::Loop()
{
    while (!stop_.load()) {
        pollfd p{listenFd_, POLLIN, 0};
        int n = ::poll(&p, 1, 200);
        if (n <= 0) {
            continue;
        }
        int c = ::accept4(listenFd_, nullptr, nullptr, SOCK_CLOEXEC);
        if (c < 0) {
            continue;
        }
        timeval tv{2, 0};
        setsockopt(c, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
        uint64_t token = 0;
        if (::recv(c, &token, sizeof(token), MSG_WAITALL) == (ssize_t)sizeof(token)) {
            int fd = -1;
            {
                std::lock_guard<std::mutex> g(mu_);
                auto it = fds_.find(token);
                if (it != fds_.end()) {
                    fd = it->second;
                }
            }
            SendFd(c, fd);
        }
        ::close(c);
    }
}

int FdChannel::Fetch(const std::string &name, uint64_t token, int timeoutMs)
{
    uint64_t deadline = NowMs() + (uint64_t)timeoutMs;
    while (true) {
        int s = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (s < 0) {
            return -1;
        }
        sockaddr_un addr;
        socklen_t len = FillAddr(&addr, name);
        if (::connect(s, (sockaddr *)&addr, len) == 0) {
            timeval tv{5, 0};
            setsockopt(s, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
            int fd = -1;
            if (::send(s, &token, sizeof(token), MSG_NOSIGNAL) == (ssize_t)sizeof(token)) {
                fd = RecvFd(s);
            }
            ::close(s);
            if (fd < 0) {
                MF_ERROR("fd channel: peer " << name << " has no descriptor for token " << token);
            }
            return fd;
        }
        ::close(s);
        if (NowMs() > deadline) {
            MF_ERROR("fd channel: cannot connect to " << name << ": " << strerror(errno));
            return -1;
        }
        usleep(2000);
    }
}

int FdChannel::FetchWithRetry(const std::string &name, uint64_t token, int timeoutMsPerAttempt)
{
    int fd = -1;
    RetryWithBackoff(
        [&]() {
            fd = Fetch(name, token, timeoutMsPerAttempt);
            return fd >= 0;
        },
        [&](uint32_t failed) { MF_WARN("fd channel: fetching token " << token << " from " << name << " failed, attempt " << failed + 1); });
    return fd;
}

void FdChannel::Shutdown()
{
    stop_.store(true);
    if (server_.joinable()) {
        server_.join();
    }
    std::lock_guard<std::mutex> g(mu_);
    if (listenFd_ >= 0) {
        ::close(listenFd_);
        listenFd_ = -1;
    }
    for (auto &kv : fds_) {
        ::close(kv.second);
    }
    fds_.clear();
    name_.clear();
}

void FdChannel::ResetAfterFork()
{
    // The server thread does not exist in the child; the listening socket is shared with the parent and must not be
    // served twice. Descriptors published by the parent stay the parent's business.
    if (server_.joinable()) {
        server_.detach();
    }
    new (&mu_) std::mutex();
    if (listenFd_ >= 0) {
        ::close(listenFd_);
        listenFd_ = -1;
    }
    for (auto &kv : fds_) {
        ::close(kv.second);
    }
    fds_.clear();
    name_.clear();
    stop_.store(false);
}

}  // namespace hybm
}  // namespace mf

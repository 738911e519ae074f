// Framed TCP request/response transport used by the config store (control plane only).
//
// Role of the reference's acc_links library (src/acc_links/include/acc_tcp_server.h:64-168,
// acc_tcp_link.h:171-222, framing acc_def.h:72-90, handshake acc_def.h:45-56): a listener that accepts links
// after a hello/ack handshake, per-type message delivery, non-blocking queued sends, link-up / link-broken
// callbacks, and a client that matches replies to blocked callers by sequence number or routes them to a
// persistent context (used for watches). This implementation is one epoll thread per server and one reader
// thread per client; payloads are opaque strings.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>

namespace mf {
namespace net {

class TlsContext;
class TlsSession;

constexpr uint32_t kWireMagic = 0x4D464231u;  // "MFB1"
constexpr uint16_t kWireVersion = 1;
constexpr uint32_t kMaxBodyLen = 80u * 1024u * 1024u;  // a little above the 64 MiB value cap of the store

// Transport-level result codes placed in Frame::result by the transport itself (store codes share the field).
enum : int16_t { RPC_OK = 0, RPC_IO_ERROR = -602, RPC_TIMEOUT = -601 };
// MSG_GOODBYE: sent by a server that shuts down in good order, so that clients can tell an orderly end from a broken link.
enum : uint16_t { MSG_HELLO = 0xFFF0, MSG_HELLO_ACK = 0xFFF1, MSG_GOODBYE = 0xFFF2 };

#pragma pack(push, 1)
struct WireHeader {
    uint32_t magic;
    uint16_t type;
    int16_t result;
    uint32_t bodyLen;
    uint32_t seq;
};
struct HelloBody {
    uint16_t version;
    uint16_t reserved;
    uint32_t reserved2;
    uint64_t peerId;  // caller-defined identity; the store packs (worldSize << 32) | rankId
};
#pragma pack(pop)
static_assert(sizeof(WireHeader) == 16, "wire header is 16 bytes");

struct Frame {
    uint16_t type{0};
    int16_t result{0};
    uint32_t seq{0};
    std::string body;
};

using LinkId = uint64_t;

// host may be an IPv4 literal, an IPv6 literal (without brackets) or a name.
struct Endpoint {
    std::string host;
    uint16_t port{0};
    bool v6{false};
};
// Accepts tcp://ip:port, tcp://[v6]:port, tcp6://[v6]:port and bare ip:port. Returns false on a malformed URL.
bool ParseUrl(const std::string &url, Endpoint *out);
// Local address the kernel would use to reach `target` (UDP connect trick); empty string on failure.
std::string LocalIpToward(const Endpoint &target);
// All non-loopback IPv4 addresses of this host.
std::vector<std::string> LocalIpv4List();

class RpcServer {
public:
    using MsgHandler = std::function<void(LinkId, const Frame &)>;
    using LinkUpHandler = std::function<bool(LinkId, uint64_t peerId)>;  // false rejects the link
    using LinkDownHandler = std::function<void(LinkId)>;

    RpcServer();
    ~RpcServer();
    void SetHandlers(MsgHandler onMsg, LinkUpHandler onUp, LinkDownHandler onDown);
    // Every link accepted from now on speaks TLS 1.3 with this (server-role) context; nullptr = plain TCP. Call before Start.
    void SetTls(std::shared_ptr<TlsContext> ctx);
    // Binds and starts the I/O thread. port 0 picks a free port. Returns 0 or -errno; EADDRINUSE is reported as such.
    int Start(const Endpoint &ep);
    // Tells every link goodbye (so that the peers see an orderly end, not a failure), then closes them and the listener.
    void Stop();
    uint16_t Port() const { return port_; }
    bool Running() const { return running_.load(); }
    // Time (NowMs) of the event loop's latest pass: a supervisor that judges peers by what the loop has read from them must
    // first know that the loop itself has been running.
    uint64_t LoopBeatMs() const { return loopBeatMs_.load(std::memory_order_relaxed); }
    // Thread-safe. Returns 0 when queued/sent, -1 if the link is gone.
    int Send(LinkId link, const Frame &f);
    // A frame whose body is `payload` (f.body is ignored): on a plain link the bytes go to the socket from where they lie and
    // only what the socket does not take at once is copied into the queue. The payload must stay valid during the call only.
    int SendWithPayload(LinkId link, const Frame &f, const void *payload, size_t payloadLen);
    void CloseLink(LinkId link);
    size_t LinkCount();

private:
    struct Conn;
    void Loop();
    void Accept();
    void OnReadable(const std::shared_ptr<Conn> &c);
    void Flush(const std::shared_ptr<Conn> &c);
    void Drop(const std::shared_ptr<Conn> &c);
    void Wake();
    int SendBytesLocked(Conn &c, std::string bytes);

    MsgHandler onMsg_;
    LinkUpHandler onUp_;
    LinkDownHandler onDown_;
    int listenFd_{-1}, epfd_{-1}, wakeFd_{-1};
    uint16_t port_{0};
    std::atomic<bool> running_{false};
    std::atomic<uint64_t> loopBeatMs_{0};
    std::thread io_;
    std::mutex mu_;  // guards conns_ and every Conn::out queue
    std::unordered_map<LinkId, std::shared_ptr<Conn>> conns_;
    std::unordered_map<int, LinkId> byFd_;
    std::deque<LinkId> pendingClose_;
    LinkId nextLink_{1};
    std::shared_ptr<TlsContext> tls_;
};

class RpcClient {
public:
    using PersistCb = std::function<void(const Frame &)>;
    using BrokenCb = std::function<void()>;

    RpcClient();
    ~RpcClient();
    // Speak TLS 1.3 with this (client-role) context on the next Connect; nullptr = plain TCP.
    void SetTls(std::shared_ptr<TlsContext> ctx);
    // True if the server announced an orderly shutdown on the link that was open last.
    bool PeerSaidGoodbye() const { return goodbye_.load(); }
    // Tries up to `retries` times, sleeping retryDelayMs between attempts. 0 on success.
    int Connect(const Endpoint &ep, uint64_t peerId, int retries, int retryDelayMs);
    void Close();
    bool Connected() const { return connected_.load(); }
    void SetBrokenHandler(BrokenCb cb) { onBroken_ = std::move(cb); }
    // Blocking request. timeoutMs < 0 waits until the link breaks. Returns RPC_OK and fills reply, RPC_IO_ERROR or RPC_TIMEOUT.
    int Call(uint16_t type, const std::string &body, Frame *reply, int64_t timeoutMs);
    // The same request with its body given as two pieces that are sent from where they lie (no intermediate copy), and,
    // optionally, a buffer that receives the reply's body in place: if the reply carries exactly sinkLen bytes and result 0
    // they are read from the socket straight into `sink` and reply->body stays empty; any other reply arrives in reply->body.
    // Used by the bulk data path; `sink` must stay valid until the call returns. On TLS links the reply always arrives in
    // reply->body.
    int CallGather(uint16_t type, const void *head, size_t headLen, const void *payload, size_t payloadLen, void *sink, size_t sinkLen,
                   Frame *reply, int64_t timeoutMs);
    // Sends a request whose replies (possibly many) are delivered to cb on the reader thread until Cancel(seq).
    // Returns the sequence number, or 0 on failure.
    uint32_t CallPersistent(uint16_t type, const std::string &body, PersistCb cb);
    void Cancel(uint32_t seq);

private:
    struct Pending {
        std::mutex mu;
        std::condition_variable cv;
        bool done{false};
        bool failed{false};
        bool abandoned{false};  // the caller gave up: its sink must not be written any more
        void *sink{nullptr};
        size_t sinkLen{0};
        Frame reply;
        PersistCb persist;
    };
    int SendFrame(uint16_t type, uint32_t seq, const std::string &body);
    int SendParts(uint16_t type, uint32_t seq, const void *head, size_t headLen, const void *payload, size_t payloadLen);
    void ReaderLoop();
    void FailAll();
    bool IoWrite(const void *p, size_t n);  // caller holds sendMu_ (or is the only thread: during Connect)
    bool IoRead(void *p, size_t n);         // reader thread (or Connect)
    bool TlsHandshake(int fd);

    std::shared_ptr<TlsContext> tlsCtx_;
    std::unique_ptr<TlsSession> tls_;
    std::mutex tlsMu_;        // lock order: sendMu_ before tlsMu_
    std::string plainBuf_;    // decrypted bytes not yet consumed by the reader
    size_t plainOff_{0};
    std::atomic<bool> goodbye_{false};
    int fd_{-1};
    std::atomic<bool> connected_{false};
    std::atomic<bool> closing_{false};
    std::thread reader_;
    std::mutex sendMu_;
    std::mutex mu_;
    std::unordered_map<uint32_t, std::shared_ptr<Pending>> pending_;
    std::atomic<uint32_t> nextSeq_{1};
    BrokenCb onBroken_;
};

}  // namespace net
}  // namespace mf

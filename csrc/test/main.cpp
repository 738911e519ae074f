// Native test binary: exercises the C++ layers and the public C API directly (no Python), including a fork-based
// two-rank Big Memory run over a loopback config store — the shape of the reference's gtest suite
// (test/ut/testcase/smem/smem_bm_test.cpp:209-416, acc_config_store_test.cpp:68-462). Build: `make`; sanitised: `make asan`.
// Usage: mf_native_tests [filter-substring]. Exit code = number of failed cases.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <chrono>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <climits>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <string>
#include <thread>
#include <vector>

#include "group/mf_group.h"
#include "hybm/mf_range_pool.h"
#include "hybm/mf_va_manager.h"
#include "mf/mf.h"
#include "mf/mf_bm.h"
#include "mf/mf_hybm.h"
#include "store/mf_store_client.h"
#include "util/mf_file_util.h"
#include "util/mf_net_util.h"
#include "util/mf_str_util.h"
#include "util/mf_sync.h"

using namespace mf;

static int g_failed = 0;
#define EXPECT(cond)                                                          \
    do {                                                                      \
        if (!(cond)) {                                                        \
            printf("    EXPECT failed %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            ok = false;                                                       \
        }                                                                     \
    } while (0)

struct Case {
    const char *name;
    std::function<bool()> fn;
};

static uint16_t FreePort()
{
    net::RpcServer s;
    net::Endpoint ep{"127.0.0.1", 0, false};
    s.SetHandlers(nullptr, nullptr, nullptr);
    s.Start(ep);
    uint16_t p = s.Port();
    s.Stop();
    return p;
}

static bool TestCodec()
{
    bool ok = true;
    store::StoreMessage m, out;
    m.userDef = 42;
    m.keys = {"k"};
    m.values = {std::string("\0\1\2", 3), ""};
    std::string b = store::PackMessage(m);
    EXPECT(store::UnpackMessage(b, &out) && out.userDef == 42 && out.keys == m.keys && out.values == m.values);
    EXPECT(!store::UnpackMessage(b.substr(0, b.size() - 1), &out));
    EXPECT(!store::UnpackMessage(b + "x", &out));
    return ok;
}

static bool TestUtilLayer()
{
    bool ok = true;
    using namespace mf::util;
    // strings and numbers
    EXPECT(Trim("  a b\t\n") == "a b" && Trim(" \t") == "");
    EXPECT(Split("a,,b", ',').size() == 3 && Split("", ',').empty() && Split("x", ',').size() == 1);
    EXPECT(StartsWith("tcp://x", "tcp://") && !StartsWith("tc", "tcp://"));
    uint16_t u16 = 0;
    int32_t i32 = 0;
    EXPECT(ParseInt<uint16_t>("65535", &u16) && u16 == 65535 && !ParseInt<uint16_t>("65536", &u16));
    EXPECT(!ParseInt<uint16_t>("-1", &u16) && !ParseInt<uint16_t>(" 1", &u16) && !ParseInt<uint16_t>("1x", &u16) && !ParseInt<uint16_t>("", &u16));
    EXPECT(ParseInt<int32_t>("-2147483648", &i32) && i32 == INT32_MIN && !ParseInt<int32_t>("2147483648", &i32));
    EXPECT(WouldOverflow<uint32_t>(0xFFFFFFF0u, 0x20u, UINT32_MAX, '+') && !WouldOverflow<uint32_t>(1, 2, UINT32_MAX, '+'));
    EXPECT(WouldOverflow<uint64_t>(1ull << 40, 1ull << 30, UINT64_MAX, '*') && !WouldOverflow<uint64_t>(0, 5, 10, '*'));
    EXPECT(ExtractBits(0xABCD1234u, 8, 8) == 0x12 && ExtractBits(0xFFFFFFFFu, 0, 32) == 0xFFFFFFFFu && ExtractBits(1, 30, 4) == 0);
    // addresses
    EXPECT(IsValidIpv4("10.0.0.1") && IsValidIpv4("255.255.255.255") && !IsValidIpv4("256.1.1.1") && !IsValidIpv4("1.2.3"));
    EXPECT(!IsValidIpv4("01.2.3.4") && !IsValidIpv4("1.2.3.4.") && !IsValidIpv4("1..3.4") && !IsValidIpv4("a.b.c.d"));
    EXPECT(!IsValidIpv4("0.0.0.0") && IsValidIpv4("0.0.0.0", true) && !IsValidIpv4("1.2.3.4 "));
    EXPECT(IsValidIpv6("::1") && IsValidIpv6("fe80::1:2") && !IsValidIpv6("::g") && !IsValidIpv6(""));
    std::string ip, why;
    uint16_t port = 0;
    EXPECT(ParseIpv4Port("127.0.0.1:8570", 1025, &ip, &port, &why) && ip == "127.0.0.1" && port == 8570);
    EXPECT(!ParseIpv4Port("127.0.0.1:80", 1025, &ip, &port, &why) && !ParseIpv4Port("127.0.0.1", 0, &ip, &port, &why));
    EXPECT(!ParseIpv4Port("127.0.0.1:70000", 0, &ip, &port, &why) && !ParseIpv4Port("300.0.0.1:8000", 0, &ip, &port, &why));
    EXPECT(Ipv4InCidr("192.168.3.77", "192.168.0.0/16") && !Ipv4InCidr("192.169.0.1", "192.168.0.0/16") && Ipv4InCidr("8.8.8.8", "0.0.0.0/0"));
    EXPECT(!Ipv4InCidr("1.2.3.4", "1.2.3.0/33") && !Ipv4InCidr("1.2.3.4", "1.2.3.0"));
    NetAddr a4, a4b, a6;
    EXPECT(NetAddr::Parse("10.1.2.3", &a4) && NetAddr::Parse("10.1.2.3", &a4b) && NetAddr::Parse("::1", &a6) && !NetAddr::Parse("nope", &a4b));
    EXPECT(a4 == a4b && a4 != a6 && NetAddrHash()(a4) == NetAddrHash()(a4b) && a4.ToString() == "10.1.2.3" && a6.ToString() == "::1");
    // files
    char tmpl[] = "/tmp/mf_util_test_XXXXXX";
    const char *root = mkdtemp(tmpl);
    EXPECT(root != nullptr);
    if (root != nullptr) {
        std::string dir = std::string(root) + "/a/b/c";
        EXPECT(MakeDirs(dir, 0750) && IsDir(dir) && MakeDirs(dir, 0750));
        std::string file = dir + "/cert.pem", link = dir + "/link.pem", big = dir + "/big.bin";
        FILE *f = fopen(file.c_str(), "w");
        fputs("hello", f);
        fclose(f);
        EXPECT(symlink(file.c_str(), link.c_str()) == 0);
        f = fopen(big.c_str(), "w");
        for (int i = 0; i < 100; i++) {
            fputs("0123456789", f);
        }
        fclose(f);
        EXPECT(IsRegularFile(file) && !IsSymlink(file) && IsSymlink(link) && FileSize(file) == 5 && !IsEmptyFile(file));
        EXPECT(CheckConfigFile(file, 1024, false, &why));
        EXPECT(!CheckConfigFile(link, 1024, false, &why) && why.find("symbolic") != std::string::npos);
        EXPECT(CheckConfigFile(link, 1024, true, &why));
        EXPECT(!CheckConfigFile(big, 512, false, &why) && !CheckConfigFile(dir, 1024, false, &why));
        EXPECT(!CheckConfigFile(dir + "/absent", 1024, false, &why) && !CheckConfigFile("", 1024, false, &why));
        std::string content;
        EXPECT(ReadConfigFile(file, 1024, &content, &why) && content == "hello");
        std::string canon = dir + "/../c/cert.pem";
        EXPECT(Canonicalize(&canon) && canon.find("..") == std::string::npos);
        std::string lib;
        EXPECT(ResolveLibrary(dir, "cert.pem", &lib) && lib == canon);
        EXPECT(!ResolveLibrary(dir, "../c/cert.pem", &lib) && !ResolveLibrary(dir, "absent.so", &lib));
        std::string outer = std::string(root) + "/outer.so", escape = dir + "/escape.so";
        f = fopen(outer.c_str(), "w");
        fputs("x", f);
        fclose(f);
        EXPECT(symlink(outer.c_str(), escape.c_str()) == 0);
        EXPECT(!ResolveLibrary(dir, "escape.so", &lib));  // the link leads out of the directory
        EXPECT(RemoveFile(link) && IsRegularFile(file));                          // the link goes, its target stays
        EXPECT(!RemoveTree("/") && !RemoveTree("/tmp") && !RemoveTree("relative/path"));
        EXPECT(RemoveTree(root) && !Exists(root));
    }
    // locks: readers run together, a writer runs alone
    RwLock rw;
    SpinLock spin;
    std::atomic<int> readersInside{0}, maxReaders{0}, violations{0};
    long counter = 0, spinCounter = 0;
    std::vector<std::thread> th;
    for (int t = 0; t < 6; t++) {
        th.emplace_back([&, t]() {
            for (int i = 0; i < 2000; i++) {
                if (t < 2) {
                    WriteGuard g(rw);
                    if (readersInside.load() != 0) {
                        violations++;
                    }
                    counter++;
                } else {
                    ReadGuard g(rw);
                    int now = ++readersInside;
                    int prev = maxReaders.load();
                    while (now > prev && !maxReaders.compare_exchange_weak(prev, now)) {
                    }
                    --readersInside;
                }
                SpinGuard sg(spin);
                spinCounter++;
            }
        });
    }
    for (auto &t : th) {
        t.join();
    }
    EXPECT(violations.load() == 0 && counter == 4000 && spinCounter == 12000);
    EXPECT(rw.TryLockWrite());
    EXPECT(!rw.TryLockRead());
    rw.Unlock();
    return ok;
}

// A peer that answers a bulk read with the frame header and half of the body and then goes quiet: the caller's wait must end
// at its own limit (not when the peer feels like continuing), the half-filled buffer is simply abandoned, and when the rest
// arrives later it is swallowed without touching the caller's memory.
static bool TestStalledReplyBody()
{
    bool ok = true;
    int lfd = ::socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    EXPECT(::bind(lfd, (sockaddr *)&sa, sizeof(sa)) == 0 && ::listen(lfd, 1) == 0);
    socklen_t sl = sizeof(sa);
    getsockname(lfd, (sockaddr *)&sa, &sl);
    const uint16_t port = ntohs(sa.sin_port);
    constexpr uint32_t kBody = 1u << 20;
    std::atomic<int> phase{0};
    std::thread srv([&]() {
        int fd = ::accept(lfd, nullptr, nullptr);
        auto readn = [&](void *p, size_t n) {
            size_t got = 0;
            while (got < n) {
                ssize_t r = ::recv(fd, (char *)p + got, n - got, 0);
                if (r <= 0) {
                    return false;
                }
                got += (size_t)r;
            }
            return true;
        };
        net::WireHeader h{};
        char hello[sizeof(net::HelloBody)];
        if (!readn(&h, sizeof(h)) || !readn(hello, sizeof(hello))) {
            ::close(fd);
            return;
        }
        net::WireHeader ack{net::kWireMagic, net::MSG_HELLO_ACK, 0, 0, h.seq};
        ::send(fd, &ack, sizeof(ack), MSG_NOSIGNAL);
        // the request: header + 24-byte body
        char req[24];
        if (!readn(&h, sizeof(h)) || h.bodyLen != sizeof(req) || !readn(req, sizeof(req))) {
            ::close(fd);
            return;
        }
        std::string body(kBody, 'Z');
        net::WireHeader rh{net::kWireMagic, h.type, 0, kBody, h.seq};
        ::send(fd, &rh, sizeof(rh), MSG_NOSIGNAL);
        ::send(fd, body.data(), kBody / 2, MSG_NOSIGNAL);
        phase.store(1);
        while (phase.load() < 2) {
            usleep(10 * 1000);  // stalled
        }
        ::send(fd, body.data() + kBody / 2, kBody / 2, MSG_NOSIGNAL);
        phase.store(3);
        char dummy;
        ::recv(fd, &dummy, 1, 0);  // until the client closes
        ::close(fd);
    });
    {
        net::RpcClient c;
        net::Endpoint to{"127.0.0.1", port, false};
        EXPECT(c.Connect(to, 1, 3, 100) == 0);
        std::vector<char> sink(kBody, 'a');
        char head[24] = {0};
        net::Frame reply;
        auto t0 = std::chrono::steady_clock::now();
        int rc = c.CallGather(0x0201, head, sizeof(head), nullptr, 0, sink.data(), sink.size(), &reply, 400);
        double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        EXPECT(rc == net::RPC_TIMEOUT);
        EXPECT(ms >= 350 && ms < 2000);
        EXPECT(phase.load() == 1);
        std::fill(sink.begin(), sink.end(), 'b');  // the caller reuses its memory
        phase.store(2);
        while (phase.load() < 3) {
            usleep(10 * 1000);
        }
        usleep(300 * 1000);  // the late half has been read by now: into a scratch buffer, not into `sink`
        bool untouched = true;
        for (char ch : sink) {
            untouched = untouched && ch == 'b';
        }
        EXPECT(untouched);
        EXPECT(c.Connected());
        c.Close();
    }
    srv.join();
    ::close(lfd);
    return ok;
}

static bool TestVaAndPool()
{
    bool ok = true;
    auto &va = hybm::VaManager::Instance();
    va.Clear();
    uint64_t a = va.FindFreeWindow(1 << 20);
    EXPECT(a == hybm::GVA_WINDOW_BEGIN);
    EXPECT(va.AddReserved({a, hybm::GiB, 1, 1}) == 0);
    EXPECT(va.FindFreeWindow(1 << 20) == a + hybm::GiB);
    EXPECT(va.AddReserved({a + 4096, hybm::GiB, 1, 1}) != 0);
    va.Clear();
    hybm::RangePool pool(4096, 1 << 16);
    {
        hybm::PoolElement e1(&pool, 100), e2(&pool, 200);
        EXPECT((bool)e1 && (bool)e2 && e1.Address() != e2.Address() && pool.InUse() == 512);
    }
    EXPECT(pool.InUse() == 0 && pool.FreeBlocks() == 1);
    return ok;
}

static bool TestStoreAndGroup()
{
    bool ok = true;
    uint16_t port = FreePort();
    net::Endpoint ep{"127.0.0.1", port, false};
    store::StoreServer server;
    EXPECT(server.Start(ep) == 0);
    const int W = 4;
    std::vector<std::shared_ptr<store::TcpStore>> clients;
    for (int r = 0; r < W; r++) {
        clients.push_back(std::make_shared<store::TcpStore>(ep, false, W, r));
        EXPECT(clients.back()->Startup(5, 100) == 0);
    }
    int64_t v = 0;
    EXPECT(clients[0]->Add("n", 5, &v) == 0 && v == 5);
    std::string s;
    EXPECT(clients[1]->Get("n", &s, 0) == 0 && s == "5");
    EXPECT(clients[1]->Get("absent", &s, 50) == store::ST_TIMEOUT);
    std::vector<int> rcs(W, -1);
    std::vector<std::string> gathered(W);
    std::vector<std::thread> ts;
    for (int r = 0; r < W; r++) {
        ts.emplace_back([&, r]() {
            group::GroupOption o;
            o.rankSize = W;
            o.rank = r;
            o.timeoutMs = 10000;
            auto g = group::GroupEngine::Create(clients[r], o);
            int rc = g->GroupBarrier();
            uint32_t mine = 100 + r;
            std::string recv(4 * W, '\0');
            rc |= g->GroupAllGather(&mine, 4, &recv[0], (uint32_t)recv.size());
            rcs[r] = rc;
            gathered[r] = recv;
        });
    }
    for (auto &t : ts) {
        t.join();
    }
    for (int r = 0; r < W; r++) {
        EXPECT(rcs[r] == 0);
        for (int i = 0; i < W; i++) {
            uint32_t x;
            memcpy(&x, gathered[r].data() + 4 * i, 4);
            EXPECT(x == (uint32_t)(100 + i));
        }
    }
    for (auto &c : clients) {
        c->Shutdown();
    }
    server.Stop();
    return ok;
}

static bool TestHybmSingleRankHostPool()
{
    bool ok = true;
    EXPECT(mf_hybm_init(-1, 0) == 0);
    mf_hybm_options o;
    memset(&o, 0, sizeof(o));
    o.bmType = MF_HYBM_TYPE_HOST_INITIATE;
    o.memType = MF_HYBM_MEM_TYPE_HOST;
    o.bmDataOpType = MF_HYBM_DOP_HOST_RDMA;
    o.rankCount = 1;
    o.devId = -1;
    o.maxDRAMSize = 4 << 20;
    o.globalUniqueAddress = true;
    o.dramShmFd = -1;
    mf_hybm_entity_t e = mf_hybm_create_entity(300, &o, 0);
    EXPECT(e != nullptr);
    if (e == nullptr) {
        return false;
    }
    EXPECT(mf_hybm_reserve_mem_space(e, 0) == 0);
    mf_hybm_mem_slice_t sl = mf_hybm_alloc_local_memory(e, MF_HYBM_MEM_TYPE_HOST, 4 << 20, 0);
    EXPECT(sl != 0);
    char *base = (char *)mf_hybm_get_memory_ptr(e, MF_HYBM_MEM_TYPE_HOST);
    EXPECT(base != nullptr && mf_hybm_get_slice_va(e, sl) == base);
    mf_hybm_exchange_info info;
    EXPECT(mf_hybm_export(e, sl, 0, &info) == 0 && info.descLen > 0);
    size_t expSize = 0;
    EXPECT(mf_hybm_export_slice_size(e, &expSize) == 0 && expSize == info.descLen);
    EXPECT(mf_hybm_import(e, &info, 1, nullptr, 0) == 0 && mf_hybm_mmap(e, 0) == 0);  // importing oneself is a no-op
    std::vector<char> src(1 << 20), dst(1 << 20);
    for (size_t i = 0; i < src.size(); i++) {
        src[i] = (char)(i * 7);
    }
    mf_hybm_copy_params p{src.data(), base + 123, src.size()};
    EXPECT(mf_hybm_data_copy(e, &p, MF_HYBM_LH_TO_GH, nullptr, 0) == 0);
    mf_hybm_copy_params q{base + 123, dst.data(), dst.size()};
    EXPECT(mf_hybm_data_copy(e, &q, MF_HYBM_DIRECTION_AUTO, nullptr, 0) == 0);
    EXPECT(src == dst);
    mf_hybm_copy_params bad{src.data(), base + (4 << 20) - 10, 100};
    EXPECT(mf_hybm_data_copy(e, &bad, MF_HYBM_LH_TO_GH, nullptr, 0) != 0);  // leaves the pool
    void *srcs[2] = {src.data(), src.data() + 4096}, *dsts[2] = {base + (2 << 20), base + (2 << 20) + 4096};
    uint64_t sizes[2] = {4096, 4096};
    mf_hybm_batch_copy_params bp{srcs, dsts, sizes, 2};
    EXPECT(mf_hybm_data_batch_copy(e, &bp, MF_HYBM_LH_TO_GH, nullptr, 0) == 0);
    EXPECT(memcmp(base + (2 << 20), src.data(), 8192) == 0);
    uint32_t reach = 0;
    EXPECT(mf_hybm_entity_reach_types(e, 0, &reach, 0) == 0 && reach != 0);
    EXPECT(mf_hybm_entity_reach_types(e, 5, &reach, 0) != 0);
    EXPECT(mf_hybm_free_local_memory(e, sl, 0) == 0 && mf_hybm_free_local_memory(e, sl, 0) != 0);
    mf_hybm_destroy_entity(e, 0);
    EXPECT(mf_hybm_wait(e) != 0);  // stale handle is rejected, not dereferenced
    mf_hybm_uninit();
    return ok;
}

static int BmChild(int rank, uint16_t port)
{
    std::string url = "tcp://127.0.0.1:" + std::to_string(port);
    mf_bm_config_t cfg;
    mf_bm_config_init(&cfg);
    cfg.rankId = (uint16_t)rank;
    cfg.controlOperationTimeout = 30;
    if (mf_bm_init(url.c_str(), 2, (uint16_t)MF_INVALID_DEV_ID, &cfg) != 0) {
        return 1;
    }
    mf_bm_t h = mf_bm_create(0, 2, MF_BM_DATA_OP_HOST_RDMA, 8 << 20, 0, 0);
    if (h == nullptr) {
        return 2;
    }
    if (mf_bm_join(h, 0) != 0) {
        return 3;
    }
    for (int i = 0; i < 500 && mf_bm_get_joined_size(h) != 2; i++) {
        usleep(10000);
    }
    if (mf_bm_get_joined_size(h) != 2) {
        return 4;
    }
    char *peer = (char *)mf_bm_ptr_by_mem_type(h, MF_MEM_TYPE_HOST, (uint16_t)(1 - rank));
    char *mine = (char *)mf_bm_ptr_by_mem_type(h, MF_MEM_TYPE_HOST, (uint16_t)rank);
    std::vector<char> data(1 << 20, (char)('A' + rank));
    mf_copy_params p{data.data(), peer + 4096, data.size()};
    if (mf_bm_copy(h, &p, MF_BM_COPY_H2GH, 0) != 0) {
        return 5;
    }
    // flag word after the payload tells the peer the data is there
    char flag = 1;
    mf_copy_params f{&flag, peer, 1};
    if (mf_bm_copy(h, &f, MF_BM_COPY_H2GH, 0) != 0) {
        return 6;
    }
    for (int i = 0; i < 3000 && *(volatile char *)mine != 1; i++) {
        usleep(1000);
    }
    if (*(volatile char *)mine != 1) {
        return 7;
    }
    for (size_t i = 0; i < data.size(); i += 4097) {
        if (mine[4096 + i] != (char)('A' + 1 - rank)) {
            return 8;
        }
    }
    if (mf_bm_get_rank_id_by_gva(h, peer + 5) != (uint32_t)(1 - rank)) {
        return 9;
    }
    usleep(rank == 0 ? 300000 : 50000);  // the rank that hosts the store leaves last
    mf_bm_destroy(h);
    mf_bm_uninit(0);
    return 0;
}

static bool TestBmTwoRanksForked()
{
    bool ok = true;
    uint16_t port = FreePort();
    pid_t pids[2];
    for (int r = 0; r < 2; r++) {
        pids[r] = fork();
        if (pids[r] == 0) {
            _exit(BmChild(r, port));
        }
    }
    for (int r = 0; r < 2; r++) {
        int st = 0;
        waitpid(pids[r], &st, 0);
        if (!(WIFEXITED(st) && WEXITSTATUS(st) == 0)) {
            printf("    rank %d failed at step %d\n", r, WIFEXITED(st) ? WEXITSTATUS(st) : -1);
            ok = false;
        }
    }
    return ok;
}

int main(int argc, char **argv)
{
    mf_set_log_level(3);
    std::vector<Case> cases = {
        {"codec", TestCodec},
        {"util_layer", TestUtilLayer},
        {"rpc_stalled_reply_body", TestStalledReplyBody},
        {"va_manager_and_range_pool", TestVaAndPool},
        {"store_and_group_engine", TestStoreAndGroup},
        {"hybm_single_rank_host_pool", TestHybmSingleRankHostPool},
        {"bm_two_ranks_forked", TestBmTwoRanksForked},
    };
    const char *filter = argc > 1 ? argv[1] : "";
    for (auto &c : cases) {
        if (strstr(c.name, filter) == nullptr) {
            continue;
        }
        printf("[ RUN  ] %s\n", c.name);
        fflush(stdout);
        bool ok = c.fn();
        printf("[ %s ] %s\n", ok ? " OK " : "FAIL", c.name);
        g_failed += ok ? 0 : 1;
    }
    printf("%d failed\n", g_failed);
    return g_failed;
}

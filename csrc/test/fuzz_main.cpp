// Mutation fuzzer for every parser that reads bytes another process (or a user) produced: the store's message codec, URL and
// address parsing, the TLS option text, exchange blobs handed to an entity's import, number parsing, and the store server's
// request handler fed through a real loopback link. No external fuzzing engine: a seeded generator mutates a corpus of valid
// inputs (bit flips, truncation, splices, length-field edits, random bytes); the binary is meant to be built with
// AddressSanitizer + UBSan (`make fuzz`), so the oracle is "no crash, no sanitizer report, and accepted inputs round-trip".
// Role of the reference's fuzz build (script/run_fuzz.sh:22-75, which links its unit tests against a fuzzing library).
//
// usage: mf_fuzz [seconds=10] [seed=1] [target-substring]
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <random>
#include <string>
#include <vector>

#include "mf/mf.h"
#include "hybm/mf_entity.h"
#include "hybm/mf_segment.h"
#include "net/mf_rpc.h"
#include "net/mf_tls.h"
#include "store/mf_store.h"
#include "store/mf_store_client.h"
#include "store/mf_store_server.h"
#include "util/mf_log.h"
#include "util/mf_net_util.h"
#include "util/mf_str_util.h"

using namespace mf;

namespace {

std::mt19937_64 g_rng;

uint64_t Rnd(uint64_t n) { return n == 0 ? 0 : g_rng() % n; }

std::string Mutate(const std::vector<std::string> &corpus)
{
    std::string s = corpus[Rnd(corpus.size())];
    const int edits = 1 + (int)Rnd(4);
    for (int e = 0; e < edits; e++) {
        switch (Rnd(8)) {
            case 0:  // bit flip
                if (!s.empty()) {
                    s[Rnd(s.size())] ^= (char)(1u << Rnd(8));
                }
                break;
            case 1:  // truncate
                s.resize(Rnd(s.size() + 1));
                break;
            case 2: {  // insert random bytes
                std::string ins(1 + Rnd(16), '\0');
                for (auto &c : ins) {
                    c = (char)Rnd(256);
                }
                s.insert(Rnd(s.size() + 1), ins);
                break;
            }
            case 3: {  // splice with another corpus entry
                const std::string &o = corpus[Rnd(corpus.size())];
                s = s.substr(0, Rnd(s.size() + 1)) + o.substr(Rnd(o.size() + 1));
                break;
            }
            case 4:  // overwrite 4 bytes with an "interesting" integer (length fields)
                if (s.size() >= 4) {
                    static const uint32_t vals[] = {0, 1, 0x7F, 0x80, 0xFF, 0x100, 0xFFFF, 0x10000, 0x7FFFFFFF, 0x80000000u, 0xFFFFFFFFu, 0x04000001};
                    uint32_t v = vals[Rnd(sizeof(vals) / sizeof(vals[0]))];
                    std::memcpy(&s[Rnd(s.size() - 3)], &v, 4);
                }
                break;
            case 5:  // duplicate a chunk
                if (!s.empty()) {
                    size_t a = Rnd(s.size()), n = 1 + Rnd(s.size() - a);
                    s.insert(a, s.substr(a, n));
                }
                break;
            case 6:  // set a byte to a delimiter
                if (!s.empty()) {
                    static const char delims[] = {':', ';', ',', '/', '[', ']', '.', '\0', '\n', ' ', '-', '+'};
                    s[Rnd(s.size())] = delims[Rnd(sizeof(delims))];
                }
                break;
            default:  // fully random
                s.assign(Rnd(64), '\0');
                for (auto &c : s) {
                    c = (char)Rnd(256);
                }
                break;
        }
        if (s.size() > 4096) {
            s.resize(4096);
        }
    }
    return s;
}

struct Target {
    const char *name;
    std::vector<std::string> corpus;
    std::function<void(const std::string &)> run;
    uint64_t runs{0};
    uint64_t accepted{0};
};

[[noreturn]] void Fail(const char *target, const char *what, const std::string &input)
{
    std::fprintf(stderr, "FUZZ FAILURE in %s: %s\ninput (%zu bytes):", target, what, input.size());
    for (unsigned char c : input) {
        std::fprintf(stderr, " %02x", c);
    }
    std::fprintf(stderr, "\n");
    std::abort();
}

}  // namespace

int main(int argc, char **argv)
{
    const double seconds = argc > 1 ? std::atof(argv[1]) : 10.0;
    const uint64_t seed = argc > 2 ? std::strtoull(argv[2], nullptr, 10) : 1;
    const char *filter = argc > 3 ? argv[3] : "";
    g_rng.seed(seed);
    mf_set_log_level(5);  // the parsers complain about every bad input; that is not the signal here

    std::vector<Target> targets;

    // ---- store message codec: whatever unpacks must pack back to the same bytes
    {
        Target t;
        t.name = "store_message_codec";
        store::StoreMessage m;
        m.userDef = 1500;
        m.keys = {"MF_BM_0_12_BA", "k2"};
        m.values = {"value", std::string("\0\1\2", 3)};
        t.corpus = {store::PackMessage(m), store::PackMessage(store::StoreMessage{}), std::string(8, '\0')};
        m.keys.assign(store::MAX_KEYS_PER_MSG, std::string(100, 'k'));
        t.corpus.push_back(store::PackMessage(m));
        Target *self = nullptr;
        (void)self;
        t.run = [](const std::string &in) {
            store::StoreMessage out;
            if (store::UnpackMessage(in, &out)) {
                if (store::PackMessage(out) != in) {
                    Fail("store_message_codec", "accepted input does not round-trip", in);
                }
            }
        };
        targets.push_back(std::move(t));
    }
    // ---- URLs and addresses
    {
        Target t;
        t.name = "url_and_address_parsing";
        t.corpus = {"tcp://127.0.0.1:8570", "tcp6://[::1]:9000", "[fe80::1]:1", "10.0.0.300:80", "host.name:65535", "1.2.3.4/24", "0.0.0.0:0", "::ffff:1.2.3.4"};
        t.run = [](const std::string &in) {
            net::Endpoint ep;
            if (net::ParseUrl(in, &ep)) {
                if (ep.host.empty() || ep.port == 0) {
                    Fail("url_and_address_parsing", "accepted URL without host or port", in);
                }
            }
            std::string ip, why;
            uint16_t port = 0;
            if (util::ParseIpv4Port(in, 0, &ip, &port, &why) && !util::IsValidIpv4(ip, true)) {
                Fail("url_and_address_parsing", "ParseIpv4Port accepted what IsValidIpv4 refuses", in);
            }
            uint32_t a = 0, mk = 0;
            (void)util::ParseIpv4Cidr(in, &a, &mk);
            (void)util::Ipv4InCidr(in, "10.0.0.0/8");
            util::NetAddr na;
            if (util::NetAddr::Parse(in, &na)) {
                util::NetAddr back;
                if (!util::NetAddr::Parse(na.ToString(), &back) || back != na) {
                    Fail("url_and_address_parsing", "address does not survive ToString/Parse", in);
                }
            }
            (void)util::IsValidIpv6(in);
        };
        targets.push_back(std::move(t));
    }
    // ---- numbers and strings
    {
        Target t;
        t.name = "number_parsing";
        t.corpus = {"0", "65535", "-2147483648", "18446744073709551615", "+7", "0x10", "1e3", " 12", "12 ", ""};
        t.run = [](const std::string &in) {
            uint16_t u16 = 0;
            int32_t i32 = 0;
            uint64_t u64 = 0;
            if (util::ParseInt<uint16_t>(in, &u16) && std::to_string(u16) != in && in[0] != '0') {
                Fail("number_parsing", "uint16 does not print back", in);
            }
            (void)util::ParseInt<int32_t>(in, &i32);
            (void)util::ParseInt<uint64_t>(in, &u64);
            auto parts = util::Split(in, ',');
            size_t total = 0;
            for (auto &p : parts) {
                total += p.size();
            }
            if (!in.empty() && total + parts.size() - 1 != in.size()) {
                Fail("number_parsing", "Split loses bytes", in);
            }
            (void)util::Trim(in);
        };
        targets.push_back(std::move(t));
    }
    // ---- TLS option text
    {
        Target t;
        t.name = "tls_info_text";
        t.corpus = {"tlsCaPath: /etc/ssl/; tlsCaFile: a.pem,b.pem; tlsCert: /x/node.crt;", "tlsCert: c; tlsCaFile: a; tlsCrlPath: /crl/; tlsCrlFile: x.pem; packagePath: /opt/ssl",
                    "tlsCert:;tlsCaFile:", "unknownKey: 1; tlsCert: c; tlsCaFile: a"};
        t.run = [](const std::string &in) {
            net::TlsOptions o;
            std::string err;
            if (net::ParseTlsInfo(in, &o, &err)) {
                if (o.cert.empty() || o.caFiles.empty()) {
                    Fail("tls_info_text", "accepted options without certificate or CA", in);
                }
            } else if (err.empty()) {
                Fail("tls_info_text", "refused without saying why", in);
            }
        };
        targets.push_back(std::move(t));
    }
    // ---- exchange blobs into an entity's import (host-only entity: nothing is mapped for foreign hosts / bad windows)
    std::shared_ptr<hybm::MemEntity> entity;
    {
        hybm::HybmInit(-1, 0);
        hybm::Options opt;
        opt.memType = hybm::MEM_TYPE_HOST;
        opt.rankId = 0;
        opt.rankCount = 4;
        opt.devId = -1;
        opt.maxDRAMSize = 4u << 20;
        opt.maxHBMSize = 0;
        opt.dataOpType = hybm::OP_HOST_RDMA;
        int rc = 0;
        entity = hybm::EntityFactory::Instance().Create(7, opt, &rc);
        if (entity && entity->ReserveMemorySpace() == hybm::BM_OK) {
            Target t;
            t.name = "exchange_blob_import";
            uint64_t handle = 0;
            hybm::ExchangeInfo slice{}, ent{};
            if (entity->AllocLocalMemory(2u << 20, hybm::MEM_TYPE_HOST, 0, &handle) == hybm::BM_OK && entity->Export(handle, 0, &slice) == hybm::BM_OK &&
                entity->Export(0, hybm::FLAG_EXPORT_ENTITY, &ent) == hybm::BM_OK) {
                // a peer's view of the same blobs: other rank ids so that they are not skipped as "own"
                hybm::SliceExport se;
                std::memcpy(&se, slice.desc, sizeof(se));
                se.rank = 1;
                t.corpus.push_back(std::string((const char *)&se, sizeof(se)));
                se.rank = 2;
                std::strncpy(se.hostId, "another-host", sizeof(se.hostId) - 1);
                t.corpus.push_back(std::string((const char *)&se, sizeof(se)));
                hybm::EntityExport ee;
                std::memcpy(&ee, ent.desc, sizeof(ee));
                ee.rank = 3;
                t.corpus.push_back(std::string((const char *)&ee, sizeof(ee)));
                auto e = entity;
                t.run = [e](const std::string &in) {
                    hybm::ExchangeInfo x{};
                    x.descLen = (uint32_t)std::min<size_t>(in.size(), hybm::EXCHANGE_DESC_MAX);
                    std::memcpy(x.desc, in.data(), x.descLen);
                    if (g_rng() % 8 == 0) {
                        x.descLen = (uint32_t)(g_rng() % 1024);  // a length that lies
                    }
                    void *addr = nullptr;
                    (void)e->Import(&x, 1, &addr, 0);
                    if (g_rng() % 64 == 0) {
                        for (uint32_t r = 1; r < 4; r++) {
                            e->RemoveImported(r);
                        }
                    }
                };
                targets.push_back(std::move(t));
            }
        }
    }
    // ---- the store server's request handler behind a real link: raw frames of every type with mutated bodies
    store::StoreServer server;
    net::RpcClient client;
    {
        net::Endpoint ep{"127.0.0.1", 0, false};
        if (server.Start(ep) == 0) {
            net::Endpoint to{"127.0.0.1", server.Port(), false};
            if (client.Connect(to, (4ull << 32) | 1, 3, 100) == 0) {
                Target t;
                t.name = "store_server_requests";
                store::StoreMessage m;
                m.userDef = 0;
                m.keys = {"fuzz_key"};
                m.values = {"1"};
                t.corpus.push_back(store::PackMessage(m));
                m.values = {"a", "b"};
                t.corpus.push_back(store::PackMessage(m));
                m.keys = {"c", "w", "g1"};
                m.values = {"3"};
                t.corpus.push_back(store::PackMessage(m));
                m.values.clear();
                t.corpus.push_back(store::PackMessage(m));
                net::RpcClient *c = &client;
                t.run = [c](const std::string &in) {
                    net::Frame reply;
                    uint16_t type = (uint16_t)(g_rng() % 14);
                    if (type == store::OP_WATCH_RANK_STATE) {
                        type = store::OP_GET;  // a watch never answers; everything else must answer or time out quickly
                    }
                    int rc = c->Call(type, in, &reply, 200);
                    if (rc == net::RPC_IO_ERROR) {
                        Fail("store_server_requests", "the server dropped the link", in);
                    }
                };
                targets.push_back(std::move(t));
            }
        }
    }

    const auto t0 = std::chrono::steady_clock::now();
    uint64_t total = 0;
    while (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() < seconds) {
        for (auto &t : targets) {
            if (std::strstr(t.name, filter) == nullptr) {
                continue;
            }
            const int burst = std::strcmp(t.name, "store_server_requests") == 0 ? 20 : 200;
            for (int i = 0; i < burst; i++) {
                t.run(Mutate(t.corpus));
                t.runs++;
                total++;
            }
        }
    }
    for (auto &t : targets) {
        std::printf("%-28s %10llu inputs\n", t.name, (unsigned long long)t.runs);
    }
    std::printf("fuzz: %llu inputs in %.1f s, seed %llu, no failure\n", (unsigned long long)total, seconds, (unsigned long long)seed);
    client.Close();
    server.Stop();
    entity.reset();
    hybm::EntityFactory::Instance().DestroyAll();
    return 0;
}

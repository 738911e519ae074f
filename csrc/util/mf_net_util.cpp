#include "mf_net_util.h"

#include "mf_str_util.h"

namespace mf {
namespace util {

bool IsValidIpv4(const std::string &text, bool allowAny)
{
    if (text.size() < 7 || text.size() > 15) {
        return false;
    }
    auto fields = Split(text, '.');
    if (fields.size() != 4) {
        return false;
    }
    uint32_t sum = 0;
    for (const auto &f : fields) {
        if (f.empty() || f.size() > 3 || !IsDigits(f) || (f.size() > 1 && f[0] == '0')) {
            return false;
        }
        uint32_t v = 0;
        if (!ParseInt<uint32_t>(f, &v) || v > 255) {
            return false;
        }
        sum += v;
    }
    return allowAny || sum != 0;
}

bool IsValidIpv6(const std::string &text)
{
    if (text.empty() || text.size() > 45) {
        return false;
    }
    in6_addr a;
    return inet_pton(AF_INET6, text.c_str(), &a) == 1;
}

bool ParseIpv4Port(const std::string &text, uint16_t minPort, std::string *ip, uint16_t *port, std::string *why)
{
    auto fail = [&](const char *m) {
        if (why != nullptr) {
            *why = m;
        }
        return false;
    };
    auto parts = Split(text, ':');
    if (parts.size() != 2) {
        return fail("expected <ip>:<port>");
    }
    if (!IsValidIpv4(parts[0], true)) {
        return fail("ip is not a dotted quad of 0-255 fields");
    }
    uint32_t p = 0;
    if (!ParseInt<uint32_t>(parts[1], &p)) {
        return fail("port is not a number");
    }
    if (p > 65535 || p < minPort) {
        return fail("port out of range");
    }
    if (ip != nullptr) {
        *ip = parts[0];
    }
    if (port != nullptr) {
        *port = (uint16_t)p;
    }
    return true;
}

bool ParseIpv4Cidr(const std::string &text, uint32_t *addrBe, uint32_t *maskBe)
{
    auto parts = Split(text, '/');
    if (parts.size() != 2 || !IsValidIpv4(parts[0], true)) {
        return false;
    }
    uint32_t len = 0;
    if (!ParseInt<uint32_t>(parts[1], &len) || len > 32) {
        return false;
    }
    in_addr a;
    if (inet_pton(AF_INET, parts[0].c_str(), &a) != 1) {
        return false;
    }
    uint32_t mask = len == 0 ? 0u : 0xFFFFFFFFu << (32 - len);
    if (addrBe != nullptr) {
        *addrBe = a.s_addr;
    }
    if (maskBe != nullptr) {
        *maskBe = htonl(mask);
    }
    return true;
}

bool Ipv4InCidr(const std::string &ip, const std::string &cidr)
{
    uint32_t net = 0, mask = 0;
    in_addr a;
    if (!IsValidIpv4(ip, true) || !ParseIpv4Cidr(cidr, &net, &mask) || inet_pton(AF_INET, ip.c_str(), &a) != 1) {
        return false;
    }
    return (a.s_addr & mask) == (net & mask);
}

bool NetAddr::Parse(const std::string &text, NetAddr *out)
{
    if (out == nullptr) {
        return false;
    }
    if (IsValidIpv4(text, true)) {
        in_addr a;
        if (inet_pton(AF_INET, text.c_str(), &a) != 1) {
            return false;
        }
        *out = FromV4(a);
        return true;
    }
    in6_addr a6;
    if (text.size() <= 45 && inet_pton(AF_INET6, text.c_str(), &a6) == 1) {
        *out = FromV6(a6);
        return true;
    }
    return false;
}

std::string NetAddr::ToString() const
{
    char buf[INET6_ADDRSTRLEN] = {0};
    inet_ntop(v6 ? AF_INET6 : AF_INET, bytes.data(), buf, sizeof(buf));
    return buf;
}

}  // namespace util
}  // namespace mf

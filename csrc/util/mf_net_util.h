// Address validation and a family-agnostic address value (roles of src/util/csrc/mf_ipv4_validator.h:26-300 and
// src/util/csrc/mf_net.h:20-90 of the reference, plus the dotted-quad rule of src/smem/csrc/net/smem_net_common.cpp:48-64:
// four decimal fields 0-255 without leading zeros, at most 15 characters, and not the all-zero address).
#pragma once
#include <arpa/inet.h>
#include <array>
#include <cstdint>
#include <cstring>
#include <functional>
#include <string>

namespace mf {
namespace util {

// Strict dotted quad. "0.0.0.0" (any spelling of all zeros) is refused unless allowAny.
bool IsValidIpv4(const std::string &text, bool allowAny = false);
bool IsValidIpv6(const std::string &text);
// "<ipv4>:<port>" with port in [minPort, 65535]; fills ip/port. *why names the failing part.
bool ParseIpv4Port(const std::string &text, uint16_t minPort, std::string *ip, uint16_t *port, std::string *why);
// "<ipv4>/<prefix-length>" → network byte order address and mask.
bool ParseIpv4Cidr(const std::string &text, uint32_t *addrBe, uint32_t *maskBe);
// True if `ip` lies inside the CIDR block (used to pick the local interface that faces a configured network).
bool Ipv4InCidr(const std::string &ip, const std::string &cidr);

// One IPv4 or IPv6 address as a value that can key a hash map (per-peer link tables).
struct NetAddr {
    bool v6{false};
    std::array<uint8_t, 16> bytes{};  // IPv4 uses the first four bytes

    static NetAddr FromV4(const in_addr &a)
    {
        NetAddr n;
        std::memcpy(n.bytes.data(), &a, 4);
        return n;
    }
    static NetAddr FromV6(const in6_addr &a)
    {
        NetAddr n;
        n.v6 = true;
        std::memcpy(n.bytes.data(), &a, 16);
        return n;
    }
    // Parses either family; false on malformed text.
    static bool Parse(const std::string &text, NetAddr *out);
    std::string ToString() const;
    bool operator==(const NetAddr &o) const { return v6 == o.v6 && bytes == o.bytes; }
    bool operator!=(const NetAddr &o) const { return !(*this == o); }
};

struct NetAddrHash {
    size_t operator()(const NetAddr &a) const
    {
        size_t seed = std::hash<bool>()(a.v6);
        for (size_t i = 0; i < (a.v6 ? 16u : 4u); i++) {
            seed ^= std::hash<uint8_t>()(a.bytes[i]) + 0x9e3779b97f4a7c15ull + (seed << 6) + (seed >> 2);
        }
        return seed;
    }
};

}  // namespace util
}  // namespace mf

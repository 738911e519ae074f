// Small string and number helpers shared by the option parsers (roles of src/util/csrc/mf_str_util.h:26-36 and
// mf_num_util.h:21-60 of the reference): trimming, splitting, strictly checked text→integer conversion, overflow-checked
// arithmetic and bit-field extraction.
#pragma once
#include <cerrno>
#include <cstdint>
#include <cstdlib>
#include <limits>
#include <string>
#include <type_traits>
#include <vector>

namespace mf {
namespace util {

inline std::string Trim(const std::string &s)
{
    size_t b = 0, e = s.size();
    while (b < e && (s[b] == ' ' || s[b] == '\t' || s[b] == '\r' || s[b] == '\n')) {
        b++;
    }
    while (e > b && (s[e - 1] == ' ' || s[e - 1] == '\t' || s[e - 1] == '\r' || s[e - 1] == '\n')) {
        e--;
    }
    return s.substr(b, e - b);
}

// Splits on `sep`; empty fields are kept ("a,,b" → 3 fields), an empty string gives no field.
inline std::vector<std::string> Split(const std::string &s, char sep)
{
    std::vector<std::string> out;
    if (s.empty()) {
        return out;
    }
    size_t pos = 0;
    while (true) {
        size_t next = s.find(sep, pos);
        if (next == std::string::npos) {
            out.push_back(s.substr(pos));
            return out;
        }
        out.push_back(s.substr(pos, next - pos));
        pos = next + 1;
    }
}

inline bool StartsWith(const std::string &s, const std::string &prefix)
{
    return s.size() >= prefix.size() && s.compare(0, prefix.size(), prefix) == 0;
}

inline bool IsDigits(const std::string &s)
{
    if (s.empty()) {
        return false;
    }
    for (char c : s) {
        if (c < '0' || c > '9') {
            return false;
        }
    }
    return true;
}

// Whole-string decimal conversion: no leading blanks, no sign for unsigned types, no trailing text, range-checked.
template <typename T>
inline bool ParseInt(const std::string &s, T *out)
{
    static_assert(std::is_integral<T>::value, "integral types only");
    if (s.empty() || s.size() > 24 || out == nullptr) {
        return false;
    }
    size_t i = 0;
    bool neg = false;
    if (s[0] == '-' || s[0] == '+') {
        if (std::is_unsigned<T>::value) {
            return false;
        }
        neg = s[0] == '-';
        i = 1;
    }
    if (!IsDigits(s.substr(i))) {
        return false;
    }
    errno = 0;
    if (std::is_unsigned<T>::value) {
        unsigned long long v = std::strtoull(s.c_str(), nullptr, 10);
        if (errno != 0 || v > (unsigned long long)std::numeric_limits<T>::max()) {
            return false;
        }
        *out = (T)v;
    } else {
        long long v = std::strtoll(s.c_str(), nullptr, 10);
        if (errno != 0 || v > (long long)std::numeric_limits<T>::max() || v < (long long)std::numeric_limits<T>::min()) {
            return false;
        }
        (void)neg;
        *out = (T)v;
    }
    return true;
}

// True if a+b (op '+') or a*b (op '*') exceeds `max`. Unsigned types only.
template <typename T>
inline bool WouldOverflow(T a, T b, T max, char op)
{
    static_assert(std::is_unsigned<T>::value, "unsigned types only");
    if (op == '+') {
        return a > max || b > max - a;
    }
    if (op == '*') {
        return a != 0 && b > max / a;
    }
    return true;
}

// `len` bits of `flags` starting at bit `start` (0 = least significant); 0 for an out-of-range field.
inline uint32_t ExtractBits(uint32_t flags, uint8_t start, uint8_t len)
{
    if (len == 0 || start >= 32 || (uint32_t)start + len > 32) {
        return 0;
    }
    uint32_t mask = len == 32 ? 0xFFFFFFFFu : ((1u << len) - 1u);
    return (flags >> start) & mask;
}

}  // namespace util
}  // namespace mf

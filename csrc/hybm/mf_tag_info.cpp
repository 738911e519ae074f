#include "mf_tag_info.h"

#include <sstream>

#include "../util/mf_log.h"

namespace mf {
namespace hybm {

bool TagInfo::ValidTag(const std::string &tag)
{
    if (tag.empty() || tag.size() >= 32) {
        return false;
    }
    for (char c : tag) {
        if (!(std::isalnum((unsigned char)c) || c == '_' || c == '-')) {
            return false;
        }
    }
    return true;
}

uint32_t TagInfo::OpTypeFromName(const std::string &name)
{
    static const std::map<std::string, uint32_t> names = {
        {"DEVICE_MTE", OP_KERNEL_LDST}, {"KERNEL_LDST", OP_KERNEL_LDST},   {"DEVICE_SDMA", OP_COPY_ENGINE}, {"COPY_ENGINE", OP_COPY_ENGINE},
        {"DEVICE_RDMA", OP_DEVICE_RDMA}, {"NVLS", OP_DEVICE_RDMA},         {"HOST_RDMA", OP_HOST_RDMA},     {"HOST_TCP", OP_HOST_TCP},
        {"HOST_URMA", OP_HOST_URMA},
    };
    auto it = names.find(name);
    return it == names.end() ? 0 : it->second;
}

int TagInfo::Init(uint32_t localRank, const std::string &localTag, const std::string &tagOpInfo)
{
    std::lock_guard<std::mutex> g(mu_);
    rankTags_.clear();
    rules_.clear();
    if (localTag.empty() && tagOpInfo.empty()) {
        return BM_OK;
    }
    if (!localTag.empty()) {
        MF_CHECK_RET(ValidTag(localTag), BM_INVALID_PARAM, "tag info: invalid tag '" << localTag << "'");
        rankTags_[localRank] = localTag;
    }
    std::stringstream ss(tagOpInfo);
    std::string rule;
    while (std::getline(ss, rule, ',')) {
        if (rule.empty()) {
            continue;
        }
        size_t c1 = rule.find(':');
        size_t c2 = c1 == std::string::npos ? std::string::npos : rule.find(':', c1 + 1);
        MF_CHECK_RET(c2 != std::string::npos && rule.find(':', c2 + 1) == std::string::npos, BM_INVALID_PARAM,
                     "tag info: rule '" << rule << "' is not tagA:OPTYPE:tagB");
        std::string a = rule.substr(0, c1), op = rule.substr(c1 + 1, c2 - c1 - 1), b = rule.substr(c2 + 1);
        uint32_t bit = OpTypeFromName(op);
        MF_CHECK_RET(ValidTag(a) && ValidTag(b) && bit != 0, BM_INVALID_PARAM, "tag info: rule '" << rule << "' is invalid");
        rules_[{a, b}] |= bit;
        rules_[{b, a}] |= bit;
    }
    return BM_OK;
}

int TagInfo::AddRankTag(uint32_t rank, const std::string &tag)
{
    if (tag.empty()) {
        return BM_OK;
    }
    MF_CHECK_RET(ValidTag(tag), BM_INVALID_PARAM, "tag info: invalid tag '" << tag << "' for rank " << rank);
    std::lock_guard<std::mutex> g(mu_);
    rankTags_[rank] = tag;
    return BM_OK;
}

void TagInfo::RemoveRankTag(uint32_t rank)
{
    std::lock_guard<std::mutex> g(mu_);
    rankTags_.erase(rank);
}

std::string TagInfo::TagOf(uint32_t rank)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = rankTags_.find(rank);
    return it == rankTags_.end() ? "" : it->second;
}

uint32_t TagInfo::AllowedOps(uint32_t rankA, uint32_t rankB, uint32_t fallback)
{
    std::lock_guard<std::mutex> g(mu_);
    if (rules_.empty()) {
        return fallback;
    }
    auto a = rankTags_.find(rankA), b = rankTags_.find(rankB);
    if (a == rankTags_.end() || b == rankTags_.end()) {
        return fallback;
    }
    auto it = rules_.find({a->second, b->second});
    return it == rules_.end() ? fallback : it->second;
}

}  // namespace hybm
}  // namespace mf

// Per-rank tags and "tagA:OPTYPE:tagB" rules that restrict which data-operator kinds may serve a pair of ranks.
// Reference: HybmEntityTagInfo (src/hybm/csrc/entity/hybm_entity_tag_info.cpp:35-51 init, :53-85 rule parsing,
// :125-165 lookup, :176-188 op-type names). Rules are symmetric. Without any rule every configured engine is allowed.
#pragma once
#include <map>
#include <mutex>
#include <string>

#include "mf_hybm_types.h"

namespace mf {
namespace hybm {

class TagInfo {
public:
    // tagOpInfo: comma-separated rules, e.g. "prefill:DEVICE_SDMA:decode,prefill:HOST_RDMA:store".
    int Init(uint32_t localRank, const std::string &localTag, const std::string &tagOpInfo);
    int AddRankTag(uint32_t rank, const std::string &tag);
    void RemoveRankTag(uint32_t rank);
    std::string TagOf(uint32_t rank);
    // Bit mask of DataOpType allowed between the two ranks; `fallback` when no rule mentions their tags.
    uint32_t AllowedOps(uint32_t rankA, uint32_t rankB, uint32_t fallback);
    static bool ValidTag(const std::string &tag);
    // 0 if the name is unknown.
    static uint32_t OpTypeFromName(const std::string &name);

private:
    std::mutex mu_;
    std::map<uint32_t, std::string> rankTags_;
    std::map<std::pair<std::string, std::string>, uint32_t> rules_;
};

}  // namespace hybm
}  // namespace mf

#include "mf_va_manager.h"

#include <cstdio>
#include <sstream>

#include "../util/mf_log.h"

namespace mf {
namespace hybm {

static const char *kDirNames[] = {"LH_TO_GH", "LH_TO_GD", "LD_TO_GH", "LD_TO_GD", "GH_TO_LH", "GH_TO_LD", "GD_TO_LH",
                                  "GD_TO_LD", "GH_TO_GH", "GH_TO_GD", "GD_TO_GH", "GD_TO_GD", "AUTO",     "BUTT"};

const char *DirectionName(CopyDirection d) { return d <= DIR_BUTT ? kDirNames[d] : "?"; }

CopyDirection DirectionOf(PtrClass src, PtrClass dst)
{
    // rows: source class, columns: destination class (LH, LD, GH, GD)
    static const CopyDirection table[4][4] = {
        /* LH */ {DIR_BUTT, DIR_BUTT, DIR_LH_TO_GH, DIR_LH_TO_GD},
        /* LD */ {DIR_BUTT, DIR_BUTT, DIR_LD_TO_GH, DIR_LD_TO_GD},
        /* GH */ {DIR_GH_TO_LH, DIR_GH_TO_LD, DIR_GH_TO_GH, DIR_GH_TO_GD},
        /* GD */ {DIR_GD_TO_LH, DIR_GD_TO_LD, DIR_GD_TO_GH, DIR_GD_TO_GD},
    };
    if (src > PC_GLOBAL_DEVICE || dst > PC_GLOBAL_DEVICE) {
        return DIR_BUTT;
    }
    return table[src][dst];
}

VaManager &VaManager::Instance()
{
    static VaManager *m = new VaManager();
    return *m;
}

static uint64_t AlignUp(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

uint64_t VaManager::FindFreeWindow(uint64_t size, uint64_t hint)
{
    std::lock_guard<std::mutex> g(mu_);
    size = AlignUp(size, WINDOW_ALIGN);
    uint64_t cur = hint != 0 ? AlignUp(hint, WINDOW_ALIGN) : GVA_WINDOW_BEGIN;
    if (cur < GVA_WINDOW_BEGIN) {
        cur = GVA_WINDOW_BEGIN;
    }
    for (auto &kv : reserved_) {
        uint64_t b = kv.second.base, e = b + kv.second.size;
        if (e <= cur) {
            continue;
        }
        if (b >= cur + size) {
            break;
        }
        cur = AlignUp(e, WINDOW_ALIGN);
    }
    if (cur + size > GVA_WINDOW_END) {
        return 0;
    }
    return cur;
}

int VaManager::AddReserved(const ReservedRange &r)
{
    std::lock_guard<std::mutex> g(mu_);
    if (r.size == 0 || r.base % GRANULE != 0) {
        return BM_INVALID_PARAM;
    }
    auto it = reserved_.lower_bound(r.base);
    if (it != reserved_.end() && it->first < r.base + r.size) {
        return BM_INVALID_PARAM;
    }
    if (it != reserved_.begin()) {
        auto prev = std::prev(it);
        if (prev->second.base + prev->second.size > r.base) {
            return BM_INVALID_PARAM;
        }
    }
    reserved_[r.base] = r;
    return BM_OK;
}

int VaManager::RemoveReserved(uint64_t base)
{
    std::lock_guard<std::mutex> g(mu_);
    return reserved_.erase(base) ? BM_OK : BM_INVALID_PARAM;
}

bool VaManager::FindReserved(uint64_t addr, ReservedRange *out)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = reserved_.upper_bound(addr);
    if (it == reserved_.begin()) {
        return false;
    }
    --it;
    if (addr >= it->second.base + it->second.size) {
        return false;
    }
    if (out != nullptr) {
        *out = it->second;
    }
    return true;
}

int VaManager::AddAllocated(const AllocatedRange &r)
{
    std::lock_guard<std::mutex> g(mu_);
    if (r.size == 0) {
        return BM_INVALID_PARAM;
    }
    auto it = allocated_.lower_bound(r.gva);
    if (it != allocated_.end() && it->first < r.gva + r.size) {
        return BM_INVALID_PARAM;
    }
    if (it != allocated_.begin()) {
        auto prev = std::prev(it);
        if (prev->second.gva + prev->second.size > r.gva) {
            return BM_INVALID_PARAM;
        }
    }
    allocated_[r.gva] = r;
    return BM_OK;
}

int VaManager::RemoveAllocated(uint64_t gva)
{
    std::lock_guard<std::mutex> g(mu_);
    return allocated_.erase(gva) ? BM_OK : BM_INVALID_PARAM;
}

int VaManager::RemoveAllocatedOfRank(uint32_t entityId, uint32_t rank, bool importedOnly)
{
    std::lock_guard<std::mutex> g(mu_);
    int n = 0;
    for (auto it = allocated_.begin(); it != allocated_.end();) {
        const AllocatedRange &a = it->second;
        if (a.entityId == entityId && a.ownerRank == rank && (!importedOnly || a.imported)) {
            it = allocated_.erase(it);
            n++;
        } else {
            ++it;
        }
    }
    return n;
}

void VaManager::RemoveEntity(uint32_t entityId)
{
    std::lock_guard<std::mutex> g(mu_);
    for (auto it = allocated_.begin(); it != allocated_.end();) {
        it = it->second.entityId == entityId ? allocated_.erase(it) : std::next(it);
    }
    for (auto it = reserved_.begin(); it != reserved_.end();) {
        it = it->second.entityId == entityId ? reserved_.erase(it) : std::next(it);
    }
}

bool VaManager::FindAllocated(uint64_t addr, uint64_t len, AllocatedRange *out)
{
    std::lock_guard<std::mutex> g(mu_);
    if (allocated_.empty()) {
        return false;
    }
    if (len == 0) {
        len = 1;
    }
    auto it = allocated_.upper_bound(addr);
    if (it == allocated_.begin()) {
        return false;
    }
    --it;
    const AllocatedRange &a = it->second;
    if (addr < a.gva || addr + len > a.gva + a.size || addr + len < addr) {
        return false;
    }
    if (out != nullptr) {
        *out = a;
    }
    return true;
}

bool VaManager::IsGva(uint64_t addr) { return FindReserved(addr, nullptr); }

PtrClass VaManager::Classify(uint64_t addr)
{
    AllocatedRange a;
    if (!FindAllocated(addr, 1, &a)) {
        return PC_UNKNOWN;
    }
    return a.memType == MEM_TYPE_DEVICE ? PC_GLOBAL_DEVICE : PC_GLOBAL_HOST;
}

std::string VaManager::VaToInfo(uint64_t addr)
{
    AllocatedRange a;
    char buf[160];
    if (!FindAllocated(addr, 1, &a)) {
        snprintf(buf, sizeof(buf), "{0x%lx, not in pool}", (unsigned long)addr);
        return buf;
    }
    snprintf(buf, sizeof(buf), "{gva=0x%lx, %c%c(%u), off=0x%lx}", (unsigned long)addr, a.imported ? 'R' : 'L',
             a.memType == MEM_TYPE_DEVICE ? 'D' : 'H', a.ownerRank, (unsigned long)(addr - a.gva));
    return buf;
}

std::string VaManager::Dump()
{
    std::lock_guard<std::mutex> g(mu_);
    std::ostringstream oss;
    oss << "reserved(" << reserved_.size() << "):";
    char buf[192];
    for (auto &kv : reserved_) {
        snprintf(buf, sizeof(buf), " [0x%lx,+0x%lx e%u t%u]", (unsigned long)kv.second.base, (unsigned long)kv.second.size,
                 kv.second.entityId, kv.second.memType);
        oss << buf;
    }
    oss << " allocated(" << allocated_.size() << "):";
    for (auto &kv : allocated_) {
        const AllocatedRange &a = kv.second;
        snprintf(buf, sizeof(buf), " [0x%lx,+0x%lx %c%c r%u e%u%s]", (unsigned long)a.gva, (unsigned long)a.size,
                 a.imported ? 'R' : 'L', a.memType == MEM_TYPE_DEVICE ? 'D' : 'H', a.ownerRank, a.entityId,
                 a.registered ? " reg" : "");
        oss << buf;
    }
    return oss.str();
}

void VaManager::Clear()
{
    std::lock_guard<std::mutex> g(mu_);
    reserved_.clear();
    allocated_.clear();
}

}  // namespace hybm
}  // namespace mf

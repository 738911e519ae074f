// Process-wide registry of GVA ranges.
//
// Same job as the reference's HybmVaManager (src/hybm/csrc/mm/hybm_va_manager.h:56-264, .cpp:33-484): it hands out
// *reserved* windows first-fit inside the GVA search window, records every *allocated* range (local slices, imported
// peer slices, registered user memory) with its memory type and owner rank, answers "which kind of pointer is this"
// for AUTO direction inference, and can dump itself for debugging. It never touches the MMU; segments do.
#pragma once
#include <cstdint>
#include <map>
#include <mutex>
#include <string>

#include "mf_hybm_types.h"

namespace mf {
namespace hybm {

struct ReservedRange {
    uint64_t base{0};
    uint64_t size{0};
    uint32_t entityId{0};
    uint32_t memType{0};
};

struct AllocatedRange {
    uint64_t gva{0};
    uint64_t size{0};
    uint64_t lva{0};       // local alias if the range is reachable under another address (0 = same as gva)
    uint32_t memType{0};   // MEM_TYPE_DEVICE / MEM_TYPE_HOST
    uint32_t ownerRank{0};
    uint32_t entityId{0};
    bool imported{false};  // true: owned by a peer and mapped here
    bool registered{false};  // true: user memory registered into the pool
    bool remote{false};      // true: owned by a rank on another host; known here but NOT mapped, reached through the host transport
};

class VaManager {
public:
    static VaManager &Instance();

    // First-fit search for `size` bytes (GRANULE-aligned) starting at `hint` (0 = window begin). Does not record anything:
    // the caller confirms with AddReserved once the OS/driver accepted the address.
    uint64_t FindFreeWindow(uint64_t size, uint64_t hint = 0);
    int AddReserved(const ReservedRange &r);
    int RemoveReserved(uint64_t base);
    bool FindReserved(uint64_t addr, ReservedRange *out);

    int AddAllocated(const AllocatedRange &r);  // BM_INVALID_PARAM on overlap with an existing allocated range
    int RemoveAllocated(uint64_t gva);
    int RemoveAllocatedOfRank(uint32_t entityId, uint32_t rank, bool importedOnly);
    void RemoveEntity(uint32_t entityId);
    // Range containing [addr, addr+len). len 0 is treated as 1.
    bool FindAllocated(uint64_t addr, uint64_t len, AllocatedRange *out);
    bool IsGva(uint64_t addr);
    PtrClass Classify(uint64_t addr);  // PC_GLOBAL_* if inside an allocated range, PC_UNKNOWN otherwise
    std::string Dump();
    std::string VaToInfo(uint64_t addr);
    void Clear();

private:
    std::mutex mu_;
    std::map<uint64_t, ReservedRange> reserved_;
    std::map<uint64_t, AllocatedRange> allocated_;
};

// Opaque slice handle (reference: src/hybm/csrc/mm/hybm_mem_slice.h:20-36): 40-bit magic | 16-bit index | 4-bit memory
// type | 2-bit page-table kind, validated by re-encoding.
struct MemSlice {
    uint16_t index{0};
    uint32_t memType{0};
    uint32_t kind{0};
    uint64_t vAddress{0};
    uint64_t size{0};
    static constexpr uint64_t MAGIC = 0x4D46534C43ull;  // "MFSLC"
    uint64_t ToHandle() const { return (MAGIC << 24) | ((uint64_t)index << 8) | ((uint64_t)(memType & 0xF) << 4) | ((kind & 0x3) << 2) | 0x1; }
    static bool Decode(uint64_t h, uint16_t *index, uint32_t *memType)
    {
        if ((h >> 24) != MAGIC || (h & 0x1) != 1) {
            return false;
        }
        *index = (uint16_t)((h >> 8) & 0xFFFF);
        *memType = (uint32_t)((h >> 4) & 0xF);
        return true;
    }
};

}  // namespace hybm
}  // namespace mf

// Constants, enums and POD types of the memory-management core.
//
// Values track the reference where an API user can observe them: 2 MiB allocation granularity and 1024 ranks
// (src/hybm/csrc/common/hybm_define.h:24-70), the hybm result codes (src/hybm/csrc/common/hybm_types.h:22-35), the 12
// copy directions and the option bit masks (src/hybm/include/hybm_def.h:36-141), and the 512-byte exchange blob
// (hybm_def.h:78-81). The GVA search window differs: on x86-64 Linux the CUDA unified address space shares the 47-bit
// user VA with the process, so GVA windows are carved out of [32 TiB, 96 TiB), far from heap and mmap areas.
#pragma once
#include <cstddef>
#include <cstdint>

namespace mf {
namespace hybm {

constexpr uint64_t KiB = 1024ull, MiB = 1024ull * KiB, GiB = 1024ull * MiB, TiB = 1024ull * GiB;
constexpr uint64_t GRANULE = 2 * MiB;  // cuMemGetAllocationGranularity(recommended) on B200; also huge-page size
constexpr uint64_t WINDOW_ALIGN = GiB;  // start alignment and minimum length of a reserved GVA window
constexpr uint32_t RANK_MAX = 1024;
constexpr uint64_t GVA_WINDOW_BEGIN = 32 * TiB;
constexpr uint64_t GVA_WINDOW_END = 96 * TiB;
constexpr uint64_t GVA_HOST_BEGIN = 64 * TiB;  // host-DRAM windows are searched from here, HBM windows from the start
constexpr uint32_t ENTITY_MAX = 512;
constexpr uint32_t EXTRA_CONTEXT_MAX = 64 * 1024;
constexpr uint32_t EXCHANGE_DESC_MAX = 512;

enum BmCode : int {
    BM_OK = 0,
    BM_ERROR = -1,
    BM_INVALID_PARAM = -2,
    BM_MALLOC_FAILED = -3,
    BM_NEW_OBJECT_FAILED = -4,
    BM_FILE_NOT_ACCESS = -5,
    BM_DL_FUNCTION_FAILED = -6,
    BM_TIMEOUT = -7,
    BM_UNDER_API_UNLOAD = -8,
    BM_NOT_INITIALIZED = -9,
    BM_NOT_SUPPORTED = -100,
};

enum MemType : uint32_t { MEM_TYPE_DEVICE = 1u << 0, MEM_TYPE_HOST = 1u << 1 };
enum InitiateType : uint32_t { INIT_DEVICE_KERNEL = 0 /* reference: AI_CORE_INITIATE */, INIT_HOST = 1 };
enum Scene : uint32_t { SCENE_DEFAULT = 0, SCENE_TRANS = 1, SCENE_SHM = 2 };
enum Role : uint32_t { ROLE_PEER = 0, ROLE_SENDER = 1, ROLE_RECEIVER = 2 };

// Data-operator kinds (bit mask). Numeric values keep the reference's hybm_data_op_type layout so that option
// structs filled by existing callers select the analogous engine here:
//   MTE (in-kernel load/store) → LD/ST copy kernels over NVLink, SDMA → copy engine (cudaMemcpyAsync),
//   DEVICE_RDMA → NVLS/multimem-capable kernel path, HOST_RDMA/HOST_URMA → host shared-memory memcpy, HOST_TCP → same.
enum DataOpType : uint32_t {
    OP_KERNEL_LDST = 1u << 0,
    OP_COPY_ENGINE = 1u << 1,
    OP_DEVICE_RDMA = 1u << 2,
    OP_HOST_RDMA = 1u << 3,
    OP_HOST_TCP = 1u << 4,
    OP_HOST_URMA = 1u << 5,
};

// L = local (not in the pool), G = global (in the pool); H = host DRAM, D = device HBM.
enum CopyDirection : uint32_t {
    DIR_LH_TO_GH = 0,
    DIR_LH_TO_GD,
    DIR_LD_TO_GH,
    DIR_LD_TO_GD,
    DIR_GH_TO_LH,
    DIR_GH_TO_LD,
    DIR_GD_TO_LH,
    DIR_GD_TO_LD,
    DIR_GH_TO_GH,
    DIR_GH_TO_GD,
    DIR_GD_TO_GH,
    DIR_GD_TO_GD,
    DIR_AUTO,
    DIR_BUTT
};

enum PtrClass : uint32_t { PC_LOCAL_HOST = 0, PC_LOCAL_DEVICE = 1, PC_GLOBAL_HOST = 2, PC_GLOBAL_DEVICE = 3, PC_UNKNOWN = 4 };

// Direction from the classes of the two pointers; DIR_BUTT for local→local (not a pool operation).
CopyDirection DirectionOf(PtrClass src, PtrClass dst);
const char *DirectionName(CopyDirection d);
inline PtrClass SrcClassOf(CopyDirection d)
{
    static const PtrClass t[] = {PC_LOCAL_HOST,   PC_LOCAL_HOST,    PC_LOCAL_DEVICE, PC_LOCAL_DEVICE,  PC_GLOBAL_HOST,  PC_GLOBAL_HOST,
                                 PC_GLOBAL_DEVICE, PC_GLOBAL_DEVICE, PC_GLOBAL_HOST,  PC_GLOBAL_HOST,   PC_GLOBAL_DEVICE, PC_GLOBAL_DEVICE};
    return d < DIR_AUTO ? t[d] : PC_UNKNOWN;
}
inline PtrClass DstClassOf(CopyDirection d)
{
    static const PtrClass t[] = {PC_GLOBAL_HOST, PC_GLOBAL_DEVICE, PC_GLOBAL_HOST, PC_GLOBAL_DEVICE, PC_LOCAL_HOST,  PC_LOCAL_DEVICE,
                                 PC_LOCAL_HOST,  PC_LOCAL_DEVICE,  PC_GLOBAL_HOST, PC_GLOBAL_DEVICE, PC_GLOBAL_HOST, PC_GLOBAL_DEVICE};
    return d < DIR_AUTO ? t[d] : PC_UNKNOWN;
}

// Copy flags shared with the public API.
constexpr uint32_t FLAG_ASYNC_COPY = 1u << 0;
constexpr uint32_t FLAG_COPY_KERNEL = 1u << 1;  // reference: COPY_EXTEND_FLAG — force the kernel engine

// Create flags: bits 0-6 NUMA node (0x7F = follow the GPU's affinity), bit 7 performance mode, bit 8 user shm fd, bit 9 cross-host.
constexpr uint32_t FLAG_NUMA_MASK = 0x7F;
constexpr uint32_t FLAG_NUMA_AUTO = 0x7F;
constexpr uint32_t FLAG_PERFORMANCE_MODE = 1u << 7;
constexpr uint32_t FLAG_CREATE_WITH_SHM = 1u << 8;
// bit 9: also serve this rank's pool memory to ranks on OTHER hosts over the TCP host transport, and reach theirs the same way
// (the environment variable MF_CROSS_HOST=1 sets it for every entity of the process).
constexpr uint32_t FLAG_CROSS_HOST = 1u << 9;
constexpr uint64_t INIT_FLAG_DEVICE_META = 1ull << 63;
constexpr uint32_t FLAG_EXPORT_ENTITY = 1u << 0;

struct ExchangeInfo {
    uint8_t desc[EXCHANGE_DESC_MAX];
    uint32_t descLen;
};

struct Options {
    InitiateType bmType{INIT_HOST};
    uint32_t memType{MEM_TYPE_DEVICE};
    uint32_t dataOpType{OP_KERNEL_LDST | OP_COPY_ENGINE};
    Scene scene{SCENE_DEFAULT};
    Role role{ROLE_PEER};
    uint32_t rankCount{1};
    uint32_t rankId{0};
    int32_t devId{-1};  // -1: CPU-only process
    uint64_t maxHBMSize{0};
    uint64_t maxDRAMSize{0};
    uint64_t deviceVASpace{0};  // per-rank window size; 0 = max*Size
    uint64_t hostVASpace{0};
    bool globalUniqueAddress{true};
    uint32_t flags{0};
    char transUrl[64]{};
    char tag[32]{};
    char tagOpInfo[256]{};
    int dramShmFd{-1};
};

struct CopyParams {
    const void *src;
    void *dest;
    size_t dataSize;
};

struct BatchCopyParams {
    void **sources;
    void **destinations;
    const uint64_t *dataSizes;
    uint32_t batchSize;
};

// One 128-byte record per entity, readable from device code (reference: HybmDeviceMeta,
// src/hybm/csrc/common/hybm_define.h:36-47; writer src/hybm/csrc/entity/hybm_entity_default.cpp:870-902).
struct alignas(128) DeviceMeta {
    uint32_t entityId;
    uint32_t rankId;
    uint32_t rankCount;
    uint32_t extraContextSize;
    uint64_t symmetricSize;    // per-rank window size of the HBM pool
    uint64_t hbmBase;          // GVA of rank 0's HBM window
    uint64_t dramBase;         // GVA of rank 0's DRAM window (0 if none)
    uint64_t dramWindowSize;   // per-rank window size of the DRAM pool
    uint64_t signalBase;       // GVA offset-independent address of this entity's signal area on rank 0 (0 if none)
    uint64_t extraContextAddr; // device address of the ≤64 KiB user context
    uint64_t multicastBase;    // NVLS multicast mapping of the HBM window (0 if unavailable)
    uint64_t debugFlags;       // bit 0: kernels validate their heap arguments against this record before touching peers
    uint64_t reserved[6];
};
static_assert(sizeof(DeviceMeta) == 128, "device meta record is 128 bytes");

}  // namespace hybm
}  // namespace mf

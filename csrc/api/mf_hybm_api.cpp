// Core C API (include/mf/mf_hybm.h): parameter checks and thin calls into MemEntity / EntityFactory.
// Reference: src/hybm/csrc/hybm_entry.cpp:76-167, hybm_big_mem_entry.cpp:20-219, hybm_data_op_entry.cpp:24-131.
#include <cstring>

#include "../hybm/mf_entity.h"
#include "../util/mf_log.h"
#include "mf/mf_hybm.h"

using namespace mf;

static std::shared_ptr<hybm::MemEntity> Ent(mf_hybm_entity_t e)
{
    auto p = hybm::EntityFactory::Instance().FindByPtr(e);
    if (!p) {
        MF_ERROR("hybm: invalid entity handle");
    }
    return p;
}

static_assert(sizeof(mf_hybm_exchange_info) == sizeof(hybm::ExchangeInfo), "exchange blob layouts must agree");

extern "C" int32_t mf_hybm_init(int32_t deviceId, uint64_t flags) { return hybm::HybmInit(deviceId, flags); }
extern "C" void mf_hybm_uninit(void) { hybm::HybmUninit(); }
extern "C" int32_t mf_hybm_set_extern_logger(void (*logger)(int, const char *))
{
    Logger::Instance().SetExtern(logger);
    return MF_BM_OK;
}
extern "C" int32_t mf_hybm_set_log_level(int level)
{
    if (level < LOG_DEBUG || level > LOG_OFF) {
        return MF_BM_INVALID_PARAM;
    }
    Logger::Instance().SetLevel(level);
    return MF_BM_OK;
}
extern "C" const char *mf_hybm_get_error_string(int32_t c)
{
    switch (c) {
        case MF_BM_OK: return "success";
        case MF_BM_ERROR: return "error";
        case MF_BM_INVALID_PARAM: return "invalid parameter";
        case MF_BM_MALLOC_FAILED: return "memory allocation failed";
        case MF_BM_NEW_OBJECT_FAILED: return "object creation failed";
        case MF_BM_TIMEOUT: return "timed out";
        case MF_BM_NOT_INITIALIZED: return "not initialized";
        case MF_BM_NOT_SUPPORTED: return "not supported";
        default: return "unknown error";
    }
}

extern "C" mf_hybm_entity_t mf_hybm_create_entity(uint16_t id, const mf_hybm_options *o, uint32_t /*flags*/)
{
    if (o == nullptr) {
        MF_ERROR("hybm create_entity: null options");
        return nullptr;
    }
    if (!hybm::HybmInited()) {
        MF_ERROR("hybm create_entity: call mf_hybm_init first");
        return nullptr;
    }
    hybm::Options h;
    h.bmType = o->bmType == MF_HYBM_TYPE_KERNEL_INITIATE ? hybm::INIT_DEVICE_KERNEL : hybm::INIT_HOST;
    h.memType = o->memType;
    h.dataOpType = o->bmDataOpType;
    h.scene = (hybm::Scene)o->scene;
    h.role = (hybm::Role)o->role;
    h.rankCount = o->rankCount;
    h.rankId = o->rankId;
    h.devId = o->devId;
    h.maxHBMSize = o->maxHBMSize;
    h.maxDRAMSize = o->maxDRAMSize;
    h.deviceVASpace = o->deviceVASpace;
    h.hostVASpace = o->hostVASpace;
    h.globalUniqueAddress = o->globalUniqueAddress;
    h.flags = o->flags;
    h.dramShmFd = o->dramShmFd;
    std::memcpy(h.tag, o->tag, sizeof(h.tag));
    std::memcpy(h.tagOpInfo, o->tagOpInfo, sizeof(h.tagOpInfo));
    h.tag[sizeof(h.tag) - 1] = '\0';
    h.tagOpInfo[sizeof(h.tagOpInfo) - 1] = '\0';
    int rc = 0;
    auto e = hybm::EntityFactory::Instance().Create(id, h, &rc);
    return e ? e.get() : nullptr;
}

extern "C" void mf_hybm_destroy_entity(mf_hybm_entity_t e, uint32_t)
{
    auto p = Ent(e);
    if (p) {
        hybm::EntityFactory::Instance().Destroy(p->Id());
    }
}

extern "C" int32_t mf_hybm_reserve_mem_space(mf_hybm_entity_t e, uint32_t)
{
    auto p = Ent(e);
    return p ? p->ReserveMemorySpace(0, 0) : MF_BM_INVALID_PARAM;
}
extern "C" int32_t mf_hybm_reserve_mem_space_at(mf_hybm_entity_t e, uint64_t hbmHint, uint64_t dramHint)
{
    auto p = Ent(e);
    return p ? p->ReserveMemorySpace(hbmHint, dramHint) : MF_BM_INVALID_PARAM;
}
extern "C" int32_t mf_hybm_unreserve_mem_space(mf_hybm_entity_t e, uint32_t)
{
    auto p = Ent(e);
    return p ? p->UnreserveMemorySpace() : MF_BM_INVALID_PARAM;
}
extern "C" void *mf_hybm_get_memory_ptr(mf_hybm_entity_t e, mf_hybm_mem_type t)
{
    auto p = Ent(e);
    return p ? (void *)p->MemoryPtr((uint32_t)t) : nullptr;
}
extern "C" mf_hybm_mem_slice_t mf_hybm_alloc_local_memory(mf_hybm_entity_t e, mf_hybm_mem_type t, uint64_t size, uint32_t flags)
{
    auto p = Ent(e);
    uint64_t h = 0;
    if (!p || p->AllocLocalMemory(size, (uint32_t)t, flags, &h) != hybm::BM_OK) {
        return 0;
    }
    return h;
}
extern "C" int32_t mf_hybm_free_local_memory(mf_hybm_entity_t e, mf_hybm_mem_slice_t s, uint32_t)
{
    auto p = Ent(e);
    return p ? p->FreeLocalMemory(s) : MF_BM_INVALID_PARAM;
}
extern "C" void *mf_hybm_get_slice_va(mf_hybm_entity_t e, mf_hybm_mem_slice_t s)
{
    auto p = Ent(e);
    uint64_t va = 0;
    if (!p || p->SliceVa(s, &va, nullptr) != hybm::BM_OK) {
        return nullptr;
    }
    return (void *)va;
}
extern "C" mf_hybm_mem_slice_t mf_hybm_register_local_memory(mf_hybm_entity_t e, const void *ptr, uint64_t size, uint32_t flags)
{
    auto p = Ent(e);
    uint64_t h = 0;
    if (!p || ptr == nullptr || size == 0 || p->RegisterLocalMemory((uint64_t)ptr, size, flags, &h) != hybm::BM_OK) {
        return 0;
    }
    return h;
}
extern "C" int32_t mf_hybm_export(mf_hybm_entity_t e, mf_hybm_mem_slice_t s, uint32_t flags, mf_hybm_exchange_info *x)
{
    auto p = Ent(e);
    return p && x ? p->Export(s, flags, reinterpret_cast<hybm::ExchangeInfo *>(x)) : MF_BM_INVALID_PARAM;
}
extern "C" int32_t mf_hybm_export_slice_size(mf_hybm_entity_t e, size_t *size)
{
    auto p = Ent(e);
    if (!p || size == nullptr) {
        return MF_BM_INVALID_PARAM;
    }
    *size = sizeof(hybm::SliceExport);
    return MF_BM_OK;
}
extern "C" int32_t mf_hybm_import(mf_hybm_entity_t e, const mf_hybm_exchange_info all[], uint32_t count, void *addresses[], uint32_t flags)
{
    auto p = Ent(e);
    return p ? p->Import(reinterpret_cast<const hybm::ExchangeInfo *>(all), count, addresses, flags) : MF_BM_INVALID_PARAM;
}
extern "C" int32_t mf_hybm_mmap(mf_hybm_entity_t e, uint32_t)
{
    auto p = Ent(e);
    return p ? p->Mmap() : MF_BM_INVALID_PARAM;
}
extern "C" int32_t mf_hybm_unmap(mf_hybm_entity_t e, uint32_t)
{
    auto p = Ent(e);
    return p ? p->Unmap() : MF_BM_INVALID_PARAM;
}
extern "C" int32_t mf_hybm_remove_imported(mf_hybm_entity_t e, uint32_t rank, uint32_t)
{
    auto p = Ent(e);
    return p ? p->RemoveImported(rank) : MF_BM_INVALID_PARAM;
}
extern "C" int32_t mf_hybm_entity_reach_types(mf_hybm_entity_t e, uint32_t remoteRank, uint32_t *reach, uint32_t)
{
    auto p = Ent(e);
    if (!p || reach == nullptr || remoteRank >= p->Opt().rankCount) {
        return MF_BM_INVALID_PARAM;
    }
    *reach = p->ReachTypes(remoteRank);
    return MF_BM_OK;
}
extern "C" int32_t mf_hybm_set_extra_context(mf_hybm_entity_t e, const void *ctx, uint32_t size)
{
    auto p = Ent(e);
    return p ? p->SetExtraContext(ctx, size) : MF_BM_INVALID_PARAM;
}
extern "C" const void *mf_hybm_get_device_meta(mf_hybm_entity_t e)
{
    auto p = Ent(e);
    return p ? p->DeviceMetaPtr() : nullptr;
}

extern "C" int32_t mf_hybm_data_copy(mf_hybm_entity_t e, mf_hybm_copy_params *params, mf_hybm_copy_direction dir, void *stream, uint32_t flags)
{
    auto p = Ent(e);
    if (!p || params == nullptr || dir >= MF_HYBM_DIRECTION_BUTT) {
        return MF_BM_INVALID_PARAM;
    }
    hybm::CopyParams cp{params->src, params->dest, params->dataSize};
    return p->CopyData(cp, (hybm::CopyDirection)dir, stream, flags);
}
extern "C" int32_t mf_hybm_data_batch_copy(mf_hybm_entity_t e, mf_hybm_batch_copy_params *params, mf_hybm_copy_direction dir, void *stream,
                                           uint32_t flags)
{
    auto p = Ent(e);
    if (!p || params == nullptr || dir >= MF_HYBM_DIRECTION_BUTT) {
        return MF_BM_INVALID_PARAM;
    }
    hybm::BatchCopyParams bp{params->sources, params->destinations, params->dataSizes, params->batchSize};
    return p->BatchCopyData(bp, (hybm::CopyDirection)dir, stream, flags);
}
extern "C" int32_t mf_hybm_wait(mf_hybm_entity_t e)
{
    auto p = Ent(e);
    return p ? p->Wait() : MF_BM_INVALID_PARAM;
}

#include "mf_segment.h"

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <fstream>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include "../util/mf_log.h"
#include "mf_cuda.h"
#include "mf_fd_channel.h"

#ifndef MAP_FIXED_NOREPLACE
#define MAP_FIXED_NOREPLACE 0x100000
#endif
#ifndef MFD_CLOEXEC
#define MFD_CLOEXEC 0x0001U
#endif
#ifndef MFD_HUGETLB
#define MFD_HUGETLB 0x0004U
#endif

namespace mf {
namespace hybm {

static uint64_t AlignUp(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

std::string HostIdentity()
{
    static std::string id = []() {
        const char *forced = getenv("MF_HOST_IDENTITY");
        if (forced != nullptr && forced[0] != '\0') {
            return std::string(forced).substr(0, 39);
        }
        std::ifstream f("/proc/sys/kernel/random/boot_id");
        std::string s;
        if (f && std::getline(f, s) && !s.empty()) {
            return s;
        }
        char buf[64] = {0};
        gethostname(buf, sizeof(buf) - 1);
        return std::string(buf);
    }();
    return id;
}

bool MemSegment::FindSlice(uint16_t index, MemSlice *out)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = slices_.find(index);
    if (it == slices_.end()) {
        return false;
    }
    if (out != nullptr) {
        *out = it->second;
    }
    return true;
}

static void FillCommon(SliceExport *e, const SegmentOptions &opt, uint32_t memType)
{
    std::memset(e, 0, sizeof(*e));
    e->magic = SLICE_EXPORT_MAGIC;
    e->segType = opt.type;
    e->memType = memType;
    e->rank = opt.rankId;
    e->entityId = opt.entityId;
    e->pid = (uint32_t)getpid();
    e->devId = opt.devId;
    std::string host = HostIdentity();
    std::strncpy(e->hostId, host.c_str(), sizeof(e->hostId) - 1);
}

static bool ParseSlice(const std::string &blob, SliceExport *e)
{
    if (blob.size() != sizeof(SliceExport)) {
        return false;
    }
    std::memcpy(e, blob.data(), sizeof(*e));
    return e->magic == SLICE_EXPORT_MAGIC;
}

// =============================================================================================== DeviceVmmSegment

class DeviceVmmSegment : public MemSegment {
public:
    explicit DeviceVmmSegment(const SegmentOptions &opt) : MemSegment(opt) {}
    ~DeviceVmmSegment() override
    {
        Unmap();
        UnreserveMemorySpace();
    }

    int ReserveMemorySpace(uint64_t hint, uint64_t *base) override
    {
        const cu::DriverApi *d = cu::Driver();
        MF_CHECK_RET(d != nullptr, BM_NOT_SUPPORTED, "device segment: no CUDA driver VMM support in this process");
        MF_CHECK_RET(base_ == 0, BM_ERROR, "device segment: window already reserved");
        MF_CUDA_CHECK_RET(cudaSetDevice(opt_.devId), BM_ERROR);
        MF_CUDA_CHECK_RET(cudaFree(nullptr), BM_ERROR);  // make sure the primary context exists
        uint64_t total = ReservedBytes();
        uint64_t want = VaManager::Instance().FindFreeWindow(total, hint);
        MF_CHECK_RET(want != 0, BM_MALLOC_FAILED, "device segment: GVA window exhausted");
        CUdeviceptr got = 0;
        CUresult r = d->MemAddressReserve(&got, total, GRANULE, (CUdeviceptr)want, 0);
        if (r != CUDA_SUCCESS) {
            MF_WARN("device segment: cuMemAddressReserve(0x" << std::hex << want << std::dec << ") failed: " << cu::ErrStr(r));
            return BM_ERROR;
        }
        if ((uint64_t)got != want) {
            // The hint was not honoured: this address cannot be shared, give it back.
            d->MemAddressFree(got, total);
            MF_WARN("device segment: asked for 0x" << std::hex << want << " but the driver offered 0x" << (uint64_t)got << std::dec);
            return BM_ERROR;
        }
        base_ = want;
        VaManager::Instance().AddReserved(ReservedRange{base_, total, opt_.entityId, MEM_TYPE_DEVICE});
        *base = base_;
        return BM_OK;
    }

    int UnreserveMemorySpace() override
    {
        if (base_ == 0) {
            return BM_OK;
        }
        const cu::DriverApi *d = cu::Driver();
        if (d != nullptr) {
            d->MemAddressFree((CUdeviceptr)base_, ReservedBytes());
        }
        VaManager::Instance().RemoveReserved(base_);
        base_ = 0;
        return BM_OK;
    }

    int AllocLocalMemory(uint64_t size, uint32_t /*flags*/, MemSlice *out) override
    {
        const cu::DriverApi *d = cu::Driver();
        MF_CHECK_RET(d != nullptr && base_ != 0, BM_NOT_INITIALIZED, "device segment: reserve first");
        MF_CHECK_RET(size % GRANULE == 0, BM_INVALID_PARAM, "device segment: size must be a multiple of 2 MiB");
        std::lock_guard<std::mutex> g(mu_);
        MF_CHECK_RET(localUsed_ + size <= opt_.windowSize, BM_INVALID_PARAM, "device segment: window of rank exhausted");
        MemSlice s;
        s.index = nextSlice_++;
        s.memType = MEM_TYPE_DEVICE;
        s.vAddress = base_ + (uint64_t)opt_.rankId * opt_.windowSize + localUsed_;
        s.size = size;
        if (size > 0) {
            CUmemAllocationProp prop{};
            prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
            prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
            prop.location.id = opt_.devId;
            prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
            CUmemGenericAllocationHandle h = 0;
            uint64_t t0 = NowNs();
            MF_CU_CHECK_RET(d->MemCreate(&h, size, &prop, 0), BM_MALLOC_FAILED);
            CUresult r = d->MemMap((CUdeviceptr)s.vAddress, size, 0, h, 0);
            if (r != CUDA_SUCCESS) {
                d->MemRelease(h);
                MF_ERROR("device segment: cuMemMap failed: " << cu::ErrStr(r));
                return BM_ERROR;
            }
            CUmemAccessDesc acc{};
            acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
            acc.location.id = opt_.devId;
            acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
            r = d->MemSetAccess((CUdeviceptr)s.vAddress, size, &acc, 1);
            if (r != CUDA_SUCCESS) {
                d->MemUnmap((CUdeviceptr)s.vAddress, size);
                d->MemRelease(h);
                MF_ERROR("device segment: cuMemSetAccess failed: " << cu::ErrStr(r));
                return BM_ERROR;
            }
            MF_INFO("device segment: created " << (size >> 20) << " MiB of HBM in " << (NowNs() - t0) / 1000 << " us");
            handles_[s.index] = h;
            AllocatedRange a;
            a.gva = s.vAddress;
            a.size = size;
            a.memType = MEM_TYPE_DEVICE;
            a.ownerRank = opt_.rankId;
            a.entityId = opt_.entityId;
            VaManager::Instance().AddAllocated(a);
        }
        localUsed_ += size;
        slices_[s.index] = s;
        *out = s;
        return BM_OK;
    }

    int RegisterMemory(uint64_t, uint64_t, MemSlice *) override { return BM_NOT_SUPPORTED; }

    int ReleaseSlice(const MemSlice &slice) override
    {
        const cu::DriverApi *d = cu::Driver();
        std::lock_guard<std::mutex> g(mu_);
        auto it = slices_.find(slice.index);
        if (it == slices_.end()) {
            return BM_INVALID_PARAM;
        }
        auto h = handles_.find(slice.index);
        if (h != handles_.end() && d != nullptr) {
            d->MemUnmap((CUdeviceptr)it->second.vAddress, it->second.size);
            d->MemRelease(h->second);
            handles_.erase(h);
            VaManager::Instance().RemoveAllocated(it->second.vAddress);
        }
        auto t = tokens_.find(slice.index);
        if (t != tokens_.end()) {
            FdChannel::Instance().Unpublish(t->second);
            tokens_.erase(t);
        }
        slices_.erase(it);
        return BM_OK;
    }

    int Export(const MemSlice &slice, std::string *blob) override
    {
        const cu::DriverApi *d = cu::Driver();
        std::lock_guard<std::mutex> g(mu_);
        auto it = slices_.find(slice.index);
        MF_CHECK_RET(it != slices_.end(), BM_INVALID_PARAM, "device segment: unknown slice");
        SliceExport e;
        FillCommon(&e, opt_, MEM_TYPE_DEVICE);
        e.gva = it->second.vAddress;
        e.size = it->second.size;
        e.windowBase = base_;
        e.windowSize = opt_.windowSize;
        if (it->second.size > 0) {
            auto t = tokens_.find(slice.index);
            if (t == tokens_.end()) {
                int fd = -1;
                MF_CU_CHECK_RET(d->MemExportToShareableHandle(&fd, handles_[slice.index], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
                                BM_ERROR);
                uint64_t token = FdChannel::Instance().Publish(fd);
                ::close(fd);
                MF_CHECK_RET(token != 0, BM_ERROR, "device segment: cannot publish the allocation handle");
                t = tokens_.emplace(slice.index, token).first;
            }
            e.handleKind = HK_FD_CHANNEL;
            e.fdToken = t->second;
            std::strncpy(e.fdName, FdChannel::Instance().Name().c_str(), sizeof(e.fdName) - 1);
        }
        blob->assign((const char *)&e, sizeof(e));
        return BM_OK;
    }

    int Import(const std::vector<std::string> &blobs, std::vector<uint64_t> *localAddrs) override
    {
        std::lock_guard<std::mutex> g(mu_);
        for (auto &b : blobs) {
            SliceExport e;
            MF_CHECK_RET(ParseSlice(b, &e), BM_INVALID_PARAM, "device segment: malformed slice export");
            if (localAddrs != nullptr) {
                localAddrs->push_back(e.gva);
            }
            if (e.rank == opt_.rankId || e.size == 0) {
                continue;
            }
            MF_CHECK_RET(HostIdentity() == e.hostId, BM_NOT_SUPPORTED,
                         "device segment: rank " << e.rank << " is on another host; only one NVSwitch domain is supported");
            MF_CHECK_RET(e.windowBase == base_ && e.windowSize == opt_.windowSize, BM_ERROR,
                         "device segment: rank " << e.rank << " reserved its window at 0x" << std::hex << e.windowBase << ", ours is 0x"
                                                 << base_ << std::dec);
            MF_CHECK_RET(InWindow(e.gva, e.size) && RankOf(e.gva) == e.rank, BM_INVALID_PARAM, "device segment: slice outside its window");
            imported_[e.gva] = Imp{e, mapped_.count(e.gva) > 0};
        }
        return BM_OK;
    }

    int Mmap() override
    {
        const cu::DriverApi *d = cu::Driver();
        MF_CHECK_RET(d != nullptr, BM_NOT_SUPPORTED, "device segment: no driver");
        std::lock_guard<std::mutex> g(mu_);
        for (auto &kv : imported_) {
            Imp &imp = kv.second;
            if (imp.mapped) {
                continue;
            }
            const SliceExport &e = imp.info;
            int fd = FdChannel::FetchWithRetry(e.fdName, e.fdToken);
            MF_CHECK_RET(fd >= 0, BM_ERROR, "device segment: cannot fetch the handle of rank " << e.rank);
            CUmemGenericAllocationHandle h = 0;
            CUresult r = d->MemImportFromShareableHandle(&h, (void *)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            ::close(fd);
            if (r != CUDA_SUCCESS) {
                MF_ERROR("device segment: import of rank " << e.rank << " failed: " << cu::ErrStr(r));
                return BM_ERROR;
            }
            r = d->MemMap((CUdeviceptr)e.gva, e.size, 0, h, 0);
            if (r == CUDA_SUCCESS) {
                CUmemAccessDesc acc{};
                acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
                acc.location.id = opt_.devId;
                acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
                r = d->MemSetAccess((CUdeviceptr)e.gva, e.size, &acc, 1);
                if (r != CUDA_SUCCESS) {
                    d->MemUnmap((CUdeviceptr)e.gva, e.size);
                }
            }
            d->MemRelease(h);  // the mapping keeps the physical memory alive
            if (r != CUDA_SUCCESS) {
                MF_ERROR("device segment: mapping rank " << e.rank << " at 0x" << std::hex << e.gva << std::dec << " failed: " << cu::ErrStr(r));
                return BM_ERROR;
            }
            imp.mapped = true;
            mapped_[e.gva] = e.size;
            AllocatedRange a;
            a.gva = e.gva;
            a.size = e.size;
            a.memType = MEM_TYPE_DEVICE;
            a.ownerRank = e.rank;
            a.entityId = opt_.entityId;
            a.imported = true;
            VaManager::Instance().AddAllocated(a);
        }
        return BM_OK;
    }

    int RemoveImported(const std::vector<uint32_t> &ranks) override
    {
        const cu::DriverApi *d = cu::Driver();
        std::lock_guard<std::mutex> g(mu_);
        for (auto it = imported_.begin(); it != imported_.end();) {
            if (std::find(ranks.begin(), ranks.end(), it->second.info.rank) == ranks.end()) {
                ++it;
                continue;
            }
            if (it->second.mapped && d != nullptr) {
                cudaDeviceSynchronize();  // nothing of ours may still be reading the range
                d->MemUnmap((CUdeviceptr)it->first, it->second.info.size);
                mapped_.erase(it->first);
                VaManager::Instance().RemoveAllocated(it->first);
            }
            it = imported_.erase(it);
        }
        return BM_OK;
    }

    int Unmap() override
    {
        std::vector<uint32_t> all;
        {
            std::lock_guard<std::mutex> g(mu_);
            for (auto &kv : imported_) {
                all.push_back(kv.second.info.rank);
            }
        }
        RemoveImported(all);
        std::vector<MemSlice> mine;
        {
            std::lock_guard<std::mutex> g(mu_);
            for (auto &kv : slices_) {
                mine.push_back(kv.second);
            }
        }
        for (auto &s : mine) {
            ReleaseSlice(s);
        }
        localUsed_ = 0;
        return BM_OK;
    }

    uint32_t MemTypeBit() const override { return MEM_TYPE_DEVICE; }
    bool DeviceAccessible() const override { return true; }

private:
    struct Imp {
        SliceExport info;
        bool mapped;
    };
    std::map<uint16_t, CUmemGenericAllocationHandle> handles_;
    std::map<uint16_t, uint64_t> tokens_;
    std::map<uint64_t, Imp> imported_;
    std::map<uint64_t, uint64_t> mapped_;
};

// =============================================================================================== HostShmSegment

class HostShmSegment : public MemSegment {
public:
    explicit HostShmSegment(const SegmentOptions &opt) : MemSegment(opt) {}
    ~HostShmSegment() override
    {
        Unmap();
        UnreserveMemorySpace();
        if (fd_ >= 0 && ownFd_) {
            ::close(fd_);
        }
    }

    int ReserveMemorySpace(uint64_t hint, uint64_t *base) override
    {
        MF_CHECK_RET(base_ == 0, BM_ERROR, "host segment: window already reserved");
        uint64_t total = ReservedBytes();
        uint64_t want = VaManager::Instance().FindFreeWindow(total, hint != 0 ? hint : GVA_HOST_BEGIN);
        MF_CHECK_RET(want != 0, BM_MALLOC_FAILED, "host segment: GVA window exhausted");
        void *p = ::mmap((void *)want, total, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED_NOREPLACE, -1, 0);
        if (p == MAP_FAILED || (uint64_t)p != want) {
            if (p != MAP_FAILED) {
                ::munmap(p, total);  // kernels without MAP_FIXED_NOREPLACE treat the address as a hint
            }
            MF_WARN("host segment: cannot reserve 0x" << std::hex << want << std::dec << ": " << strerror(errno));
            return BM_ERROR;
        }
        base_ = want;
        VaManager::Instance().AddReserved(ReservedRange{base_, total, opt_.entityId, MEM_TYPE_HOST});
        *base = base_;
        return BM_OK;
    }

    int UnreserveMemorySpace() override
    {
        if (base_ == 0) {
            return BM_OK;
        }
        ::munmap((void *)base_, ReservedBytes());
        VaManager::Instance().RemoveReserved(base_);
        base_ = 0;
        return BM_OK;
    }

    int AllocLocalMemory(uint64_t size, uint32_t flags, MemSlice *out) override
    {
        MF_CHECK_RET(base_ != 0, BM_NOT_INITIALIZED, "host segment: reserve first");
        MF_CHECK_RET(size % GRANULE == 0, BM_INVALID_PARAM, "host segment: size must be a multiple of 2 MiB");
        std::lock_guard<std::mutex> g(mu_);
        MF_CHECK_RET(localUsed_ + size <= opt_.windowSize, BM_INVALID_PARAM, "host segment: window of rank exhausted");
        MemSlice s;
        s.index = nextSlice_++;
        s.memType = MEM_TYPE_HOST;
        s.vAddress = base_ + (uint64_t)opt_.rankId * opt_.windowSize + localUsed_;
        s.size = size;
        if (size > 0) {
            if (fd_ < 0) {
                if ((flags & FLAG_CREATE_WITH_SHM) && opt_.shmFd >= 0) {
                    fd_ = opt_.shmFd;  // contents survive this process if the fd owner keeps it
                    ownFd_ = false;
                } else {
                    fd_ = (int)syscall(SYS_memfd_create, "mf_dram_pool", MFD_CLOEXEC);
                    ownFd_ = true;
                }
                MF_CHECK_RET(fd_ >= 0, BM_MALLOC_FAILED, "host segment: memfd_create failed: " << strerror(errno));
            }
            uint64_t fileOff = localUsed_;
            struct stat st {};
            if (fstat(fd_, &st) != 0 || (uint64_t)st.st_size < fileOff + size) {
                MF_CHECK_RET(ftruncate(fd_, (off_t)(fileOff + size)) == 0, BM_MALLOC_FAILED,
                             "host segment: cannot size the backing file to " << (fileOff + size) << ": " << strerror(errno));
            }
            void *p = ::mmap((void *)s.vAddress, size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED | MAP_POPULATE, fd_, (off_t)fileOff);
            MF_CHECK_RET(p != MAP_FAILED, BM_MALLOC_FAILED, "host segment: mmap of the local slice failed: " << strerror(errno));
            BindNuma(s.vAddress, size, flags);
            Pin(s.vAddress, size);
            fileOffsets_[s.index] = fileOff;
            AllocatedRange a;
            a.gva = s.vAddress;
            a.size = size;
            a.memType = MEM_TYPE_HOST;
            a.ownerRank = opt_.rankId;
            a.entityId = opt_.entityId;
            VaManager::Instance().AddAllocated(a);
        }
        localUsed_ += size;
        slices_[s.index] = s;
        *out = s;
        return BM_OK;
    }

    int RegisterMemory(uint64_t, uint64_t, MemSlice *) override { return BM_NOT_SUPPORTED; }

    int ReleaseSlice(const MemSlice &slice) override
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = slices_.find(slice.index);
        if (it == slices_.end()) {
            return BM_INVALID_PARAM;
        }
        if (it->second.size > 0) {
            Unpin(it->second.vAddress);
            // Put the reservation back so that the range cannot be handed to anybody else.
            ::mmap((void *)it->second.vAddress, it->second.size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);
            VaManager::Instance().RemoveAllocated(it->second.vAddress);
        }
        slices_.erase(it);
        return BM_OK;
    }

    int Export(const MemSlice &slice, std::string *blob) override
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = slices_.find(slice.index);
        MF_CHECK_RET(it != slices_.end(), BM_INVALID_PARAM, "host segment: unknown slice");
        SliceExport e;
        FillCommon(&e, opt_, MEM_TYPE_HOST);
        e.gva = it->second.vAddress;
        e.size = it->second.size;
        e.windowBase = base_;
        e.windowSize = opt_.windowSize;
        if (it->second.size > 0) {
            if (token_ == 0) {
                token_ = FdChannel::Instance().Publish(fd_);
                MF_CHECK_RET(token_ != 0, BM_ERROR, "host segment: cannot publish the backing file");
            }
            e.handleKind = HK_FD_CHANNEL;
            e.fdToken = token_;
            e.fileOffset = fileOffsets_[slice.index];
            std::strncpy(e.fdName, FdChannel::Instance().Name().c_str(), sizeof(e.fdName) - 1);
        }
        blob->assign((const char *)&e, sizeof(e));
        return BM_OK;
    }

    int Import(const std::vector<std::string> &blobs, std::vector<uint64_t> *localAddrs) override
    {
        std::lock_guard<std::mutex> g(mu_);
        for (auto &b : blobs) {
            SliceExport e;
            MF_CHECK_RET(ParseSlice(b, &e), BM_INVALID_PARAM, "host segment: malformed slice export");
            if (localAddrs != nullptr) {
                localAddrs->push_back(e.gva);
            }
            if (e.rank == opt_.rankId || e.size == 0) {
                continue;
            }
            MF_CHECK_RET(HostIdentity() == e.hostId, BM_NOT_SUPPORTED, "host segment: rank " << e.rank << " is on another host");
            MF_CHECK_RET(e.windowBase == base_ && e.windowSize == opt_.windowSize, BM_ERROR,
                         "host segment: rank " << e.rank << " reserved its window at 0x" << std::hex << e.windowBase << ", ours is 0x" << base_
                                               << std::dec);
            MF_CHECK_RET(InWindow(e.gva, e.size) && RankOf(e.gva) == e.rank, BM_INVALID_PARAM, "host segment: slice outside its window");
            auto it = imported_.find(e.gva);
            bool mapped = it != imported_.end() && it->second.mapped;
            imported_[e.gva] = Imp{e, mapped};
        }
        return BM_OK;
    }

    int Mmap() override
    {
        std::lock_guard<std::mutex> g(mu_);
        for (auto &kv : imported_) {
            Imp &imp = kv.second;
            if (imp.mapped) {
                continue;
            }
            const SliceExport &e = imp.info;
            int fd = FdChannel::FetchWithRetry(e.fdName, e.fdToken);
            MF_CHECK_RET(fd >= 0, BM_ERROR, "host segment: cannot fetch the backing file of rank " << e.rank);
            void *p = ::mmap((void *)e.gva, e.size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fd, (off_t)e.fileOffset);
            int err = errno;
            ::close(fd);
            MF_CHECK_RET(p != MAP_FAILED, BM_ERROR, "host segment: mapping rank " << e.rank << " failed: " << strerror(err));
            Pin(e.gva, e.size);
            imp.mapped = true;
            AllocatedRange a;
            a.gva = e.gva;
            a.size = e.size;
            a.memType = MEM_TYPE_HOST;
            a.ownerRank = e.rank;
            a.entityId = opt_.entityId;
            a.imported = true;
            VaManager::Instance().AddAllocated(a);
        }
        return BM_OK;
    }

    int RemoveImported(const std::vector<uint32_t> &ranks) override
    {
        std::lock_guard<std::mutex> g(mu_);
        for (auto it = imported_.begin(); it != imported_.end();) {
            if (std::find(ranks.begin(), ranks.end(), it->second.info.rank) == ranks.end()) {
                ++it;
                continue;
            }
            if (it->second.mapped) {
                Unpin(it->first);
                ::mmap((void *)it->first, it->second.info.size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);
                VaManager::Instance().RemoveAllocated(it->first);
            }
            it = imported_.erase(it);
        }
        return BM_OK;
    }

    int Unmap() override
    {
        std::vector<uint32_t> all;
        {
            std::lock_guard<std::mutex> g(mu_);
            for (auto &kv : imported_) {
                all.push_back(kv.second.info.rank);
            }
        }
        RemoveImported(all);
        std::vector<MemSlice> mine;
        {
            std::lock_guard<std::mutex> g(mu_);
            for (auto &kv : slices_) {
                mine.push_back(kv.second);
            }
        }
        for (auto &s : mine) {
            ReleaseSlice(s);
        }
        if (token_ != 0) {
            FdChannel::Instance().Unpublish(token_);
            token_ = 0;
        }
        localUsed_ = 0;
        return BM_OK;
    }

    uint32_t MemTypeBit() const override { return MEM_TYPE_HOST; }
    bool DeviceAccessible() const override { return pinnedOk_; }

private:
    struct Imp {
        SliceExport info;
        bool mapped;
    };

    void BindNuma(uint64_t addr, uint64_t size, uint32_t flags)
    {
        uint32_t node = flags & FLAG_NUMA_MASK;
        if (node == FLAG_NUMA_AUTO) {
            if (opt_.devId < 0 || !cu::Available()) {
                return;
            }
            cu::DeviceCaps caps;
            if (cu::ProbeDevice(opt_.devId, &caps) != 0 || caps.numaNode < 0) {
                return;
            }
            node = (uint32_t)caps.numaNode;
        } else if ((flags & (FLAG_NUMA_MASK | FLAG_PERFORMANCE_MODE)) == 0) {
            return;  // flags == 0: leave placement to first touch
        }
        if (node >= 64) {
            return;
        }
        unsigned long mask = 1ul << node;
        // MPOL_PREFERRED = 1; MPOL_MF_MOVE = 2. Best effort: a container without the node simply keeps first-touch placement.
        long rc = syscall(SYS_mbind, (void *)addr, size, 1, &mask, sizeof(mask) * 8, 2);
        if (rc != 0) {
            MF_DEBUG("host segment: mbind to node " << node << " not applied: " << strerror(errno));
        }
    }

    void Pin(uint64_t addr, uint64_t size)
    {
        if (opt_.devId < 0 || !cu::Available()) {
            return;
        }
        cudaSetDevice(opt_.devId);
        cudaError_t e = cudaHostRegister((void *)addr, size, cudaHostRegisterPortable | cudaHostRegisterMapped);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            MF_WARN("host segment: cudaHostRegister of " << (size >> 20) << " MiB failed (" << cu::ErrStr(e)
                                                         << "); GPU copies from this range go through pageable staging");
            pinnedOk_ = false;
            return;
        }
        pinned_[addr] = size;
    }

    void Unpin(uint64_t addr)
    {
        auto it = pinned_.find(addr);
        if (it != pinned_.end()) {
            cudaHostUnregister((void *)addr);
            (void)cudaGetLastError();
            pinned_.erase(it);
        }
    }

    int fd_{-1};
    bool ownFd_{true};
    uint64_t token_{0};
    bool pinnedOk_{true};
    std::map<uint16_t, uint64_t> fileOffsets_;
    std::map<uint64_t, Imp> imported_;
    std::map<uint64_t, uint64_t> pinned_;
};

// =============================================================================================== UserMemSegment

// No pool and no common address: every registered buffer is exported as a CUDA IPC handle (cudaMalloc memory) and
// opened by peers wherever the driver places it. LocalAliasOf() translates (owner rank, owner address) to the local
// mapping; the owner's own buffers translate to themselves.
class UserMemSegment : public MemSegment {
public:
    explicit UserMemSegment(const SegmentOptions &opt) : MemSegment(opt) {}
    ~UserMemSegment() override { Unmap(); }

    int ReserveMemorySpace(uint64_t, uint64_t *base) override
    {
        *base = 0;
        return BM_OK;
    }
    int UnreserveMemorySpace() override { return BM_OK; }
    int AllocLocalMemory(uint64_t, uint32_t, MemSlice *) override { return BM_NOT_SUPPORTED; }

    int RegisterMemory(uint64_t addr, uint64_t size, MemSlice *out) override
    {
        MF_CHECK_RET(addr != 0 && size != 0, BM_INVALID_PARAM, "user segment: empty registration");
        std::lock_guard<std::mutex> g(mu_);
        for (auto &kv : slices_) {
            MF_CHECK_RET(addr + size <= kv.second.vAddress || addr >= kv.second.vAddress + kv.second.size, BM_INVALID_PARAM,
                         "user segment: range overlaps an earlier registration");
        }
        MemSlice s;
        s.index = nextSlice_++;
        s.vAddress = addr;
        s.size = size;
        cudaPointerAttributes attr{};
        bool isDevice = false;
        if (cu::Available() && cudaPointerGetAttributes(&attr, (void *)addr) == cudaSuccess) {
            isDevice = attr.type == cudaMemoryTypeDevice;
        } else {
            (void)cudaGetLastError();
        }
        s.memType = isDevice ? MEM_TYPE_DEVICE : MEM_TYPE_HOST;
        slices_[s.index] = s;
        AllocatedRange a;
        a.gva = addr;
        a.size = size;
        a.memType = s.memType;
        a.ownerRank = opt_.rankId;
        a.entityId = opt_.entityId;
        a.registered = true;
        VaManager::Instance().AddAllocated(a);
        *out = s;
        return BM_OK;
    }

    int ReleaseSlice(const MemSlice &slice) override
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = slices_.find(slice.index);
        if (it == slices_.end()) {
            return BM_INVALID_PARAM;
        }
        VaManager::Instance().RemoveAllocated(it->second.vAddress);
        slices_.erase(it);
        return BM_OK;
    }

    int Export(const MemSlice &slice, std::string *blob) override
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = slices_.find(slice.index);
        MF_CHECK_RET(it != slices_.end(), BM_INVALID_PARAM, "user segment: unknown slice");
        SliceExport e;
        FillCommon(&e, opt_, it->second.memType);
        e.gva = it->second.vAddress;
        e.size = it->second.size;
        if (it->second.memType == MEM_TYPE_DEVICE) {
            const cu::DriverApi *d = cu::Driver();
            MF_CHECK_RET(d != nullptr, BM_NOT_SUPPORTED, "user segment: no CUDA driver");
            CUdeviceptr allocBase = 0;
            size_t allocSize = 0;
            MF_CU_CHECK_RET(d->MemGetAddressRange(&allocBase, &allocSize, (CUdeviceptr)e.gva), BM_INVALID_PARAM);
            MF_CHECK_RET(e.gva + e.size <= (uint64_t)allocBase + allocSize, BM_INVALID_PARAM,
                         "user segment: registration crosses the end of its allocation");
            cudaIpcMemHandle_t h;
            cudaError_t ce = cudaIpcGetMemHandle(&h, (void *)allocBase);
            if (ce == cudaSuccess) {
                static_assert(sizeof(h) == 64, "CUDA IPC handle is 64 bytes");
                std::memcpy(e.ipcHandle, &h, sizeof(h));
                e.handleKind = HK_CUDA_IPC;
                e.fileOffset = e.gva - (uint64_t)allocBase;
            } else {
                (void)cudaGetLastError();
                // Memory created through the VMM API has no legacy IPC handle: share its allocation handle as an fd.
                CUmemGenericAllocationHandle gh = 0;
                MF_CU_CHECK_RET(d->MemRetainAllocationHandle(&gh, (void *)e.gva), BM_NOT_SUPPORTED);
                int fd = -1;
                CUresult r = d->MemExportToShareableHandle(&fd, gh, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
                d->MemRelease(gh);
                MF_CHECK_RET(r == CUDA_SUCCESS, BM_NOT_SUPPORTED, "user segment: this allocation cannot be shared: " << cu::ErrStr(r));
                uint64_t token = FdChannel::Instance().Publish(fd);
                ::close(fd);
                MF_CHECK_RET(token != 0, BM_ERROR, "user segment: cannot publish the allocation handle");
                e.handleKind = HK_FD_VMM_RETAINED;
                e.fdToken = token;
                e.fileOffset = e.gva - (uint64_t)allocBase;
                e.windowSize = allocSize;
                std::strncpy(e.fdName, FdChannel::Instance().Name().c_str(), sizeof(e.fdName) - 1);
            }
        } else {
            e.handleKind = HK_NONE;  // plain host memory of another process cannot be mapped; peers reach it through the owner
            for (auto &kv : hostBlocks_) {
                if (e.gva >= kv.first && e.gva + e.size <= kv.first + kv.second.size) {
                    e.handleKind = HK_FD_HOST;
                    e.fdToken = kv.second.token;
                    e.fileOffset = e.gva - kv.first;
                    e.windowSize = kv.second.size;
                    std::strncpy(e.fdName, FdChannel::Instance().Name().c_str(), sizeof(e.fdName) - 1);
                    break;
                }
            }
        }
        blob->assign((const char *)&e, sizeof(e));
        return BM_OK;
    }

    int Import(const std::vector<std::string> &blobs, std::vector<uint64_t> *localAddrs) override
    {
        for (auto &b : blobs) {
            SliceExport e;
            MF_CHECK_RET(ParseSlice(b, &e), BM_INVALID_PARAM, "user segment: malformed slice export");
            uint64_t local = 0;
            if (e.rank == opt_.rankId && e.pid == (uint32_t)getpid()) {
                local = e.gva;
            } else {
                int rc = Open(e, &local);
                if (rc != BM_OK) {
                    return rc;
                }
            }
            if (localAddrs != nullptr) {
                localAddrs->push_back(local);
            }
        }
        return BM_OK;
    }

    int Mmap() override { return BM_OK; }

    int AdoptHostBlock(uint64_t addr, uint64_t size, int fd) override
    {
        std::lock_guard<std::mutex> g(mu_);
        uint64_t token = FdChannel::Instance().Publish(fd);
        MF_CHECK_RET(token != 0, BM_ERROR, "user segment: cannot publish the host block");
        hostBlocks_[addr] = HostBlock{size, token};
        return BM_OK;
    }

    int DropHostBlock(uint64_t addr) override
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = hostBlocks_.find(addr);
        if (it == hostBlocks_.end()) {
            return BM_INVALID_PARAM;
        }
        FdChannel::Instance().Unpublish(it->second.token);
        hostBlocks_.erase(it);
        return BM_OK;
    }

    int RemoveImported(const std::vector<uint32_t> &ranks) override
    {
        std::lock_guard<std::mutex> g(mu_);
        for (auto it = opened_.begin(); it != opened_.end();) {
            if (std::find(ranks.begin(), ranks.end(), it->second.rank) == ranks.end()) {
                ++it;
                continue;
            }
            Close(it->second);
            it = opened_.erase(it);
        }
        return BM_OK;
    }

    int Unmap() override
    {
        std::lock_guard<std::mutex> g(mu_);
        for (auto &kv : opened_) {
            Close(kv.second);
        }
        opened_.clear();
        return BM_OK;
    }

    uint32_t MemTypeBit() const override { return MEM_TYPE_DEVICE; }
    bool DeviceAccessible() const override { return true; }

private:
    struct Opened {
        uint32_t rank;
        uint32_t kind;
        uint64_t mappedBase;  // start of the opened allocation
        uint64_t mappedSize;
        uint64_t local;       // alias of the registered range
        uint64_t size;
        uint64_t remoteBlock{0};  // owner-side start of the host block (HK_FD_HOST)
    };
    struct HostBlock {
        uint64_t size;
        uint64_t token;
    };
    std::map<uint64_t, HostBlock> hostBlocks_;

    int Open(const SliceExport &e, uint64_t *local)
    {
        std::lock_guard<std::mutex> g(mu_);
        auto key = std::make_pair(e.rank, e.gva);
        auto it = opened_.find(key);
        if (it != opened_.end()) {
            *local = it->second.local;
            return BM_OK;
        }
        MF_CHECK_RET(HostIdentity() == e.hostId, BM_NOT_SUPPORTED, "user segment: rank " << e.rank << " is on another host");
        Opened o{e.rank, e.handleKind, 0, 0, 0, e.size, 0};
        if (e.handleKind == HK_CUDA_IPC) {
            cudaSetDevice(opt_.devId);
            // An allocation may carry several registrations: open it once.
            for (auto &kv : opened_) {
                if (kv.second.rank == e.rank && kv.second.kind == HK_CUDA_IPC && std::memcmp(ipcOf_[kv.first].data(), e.ipcHandle, 64) == 0) {
                    o.mappedBase = kv.second.mappedBase;
                    break;
                }
            }
            if (o.mappedBase == 0) {
                cudaIpcMemHandle_t h;
                std::memcpy(&h, e.ipcHandle, sizeof(h));
                void *p = nullptr;
                MF_CUDA_CHECK_RET(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), BM_ERROR);
                o.mappedBase = (uint64_t)p;
            }
            ipcOf_[key] = std::string((const char *)e.ipcHandle, 64);
            o.local = o.mappedBase + e.fileOffset;
        } else if (e.handleKind == HK_FD_VMM_RETAINED) {
            const cu::DriverApi *d = cu::Driver();
            MF_CHECK_RET(d != nullptr, BM_NOT_SUPPORTED, "user segment: no CUDA driver");
            cudaSetDevice(opt_.devId);
            int fd = FdChannel::FetchWithRetry(e.fdName, e.fdToken);
            MF_CHECK_RET(fd >= 0, BM_ERROR, "user segment: cannot fetch the handle of rank " << e.rank);
            CUmemGenericAllocationHandle h = 0;
            CUresult r = d->MemImportFromShareableHandle(&h, (void *)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            ::close(fd);
            MF_CHECK_RET(r == CUDA_SUCCESS, BM_ERROR, "user segment: import failed: " << cu::ErrStr(r));
            CUdeviceptr va = 0;
            uint64_t sz = AlignUp(e.windowSize, GRANULE);
            r = d->MemAddressReserve(&va, sz, GRANULE, 0, 0);
            if (r == CUDA_SUCCESS) {
                r = d->MemMap(va, sz, 0, h, 0);
                if (r == CUDA_SUCCESS) {
                    CUmemAccessDesc acc{};
                    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
                    acc.location.id = opt_.devId;
                    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
                    r = d->MemSetAccess(va, sz, &acc, 1);
                }
            }
            d->MemRelease(h);
            MF_CHECK_RET(r == CUDA_SUCCESS, BM_ERROR, "user segment: mapping failed: " << cu::ErrStr(r));
            o.mappedBase = (uint64_t)va;
            o.mappedSize = sz;
            o.local = o.mappedBase + e.fileOffset;
        } else if (e.handleKind == HK_FD_HOST) {
            // One mapping per (rank, block): registrations inside the same block share it.
            const uint64_t blockBase = e.gva - e.fileOffset;
            for (auto &kv : opened_) {
                if (kv.second.rank == e.rank && kv.second.kind == HK_FD_HOST && kv.second.remoteBlock == blockBase) {
                    o.mappedBase = kv.second.mappedBase;
                    o.mappedSize = kv.second.mappedSize;
                    break;
                }
            }
            if (o.mappedBase == 0) {
                int fd = FdChannel::FetchWithRetry(e.fdName, e.fdToken);
                MF_CHECK_RET(fd >= 0, BM_ERROR, "user segment: cannot fetch the host block of rank " << e.rank);
                void *p = ::mmap(nullptr, e.windowSize, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
                int err = errno;
                ::close(fd);
                MF_CHECK_RET(p != MAP_FAILED, BM_ERROR, "user segment: mapping the host block failed: " << strerror(err));
                if (opt_.devId >= 0 && cu::Available()) {
                    cudaSetDevice(opt_.devId);
                    if (cudaHostRegister(p, e.windowSize, cudaHostRegisterPortable | cudaHostRegisterMapped) != cudaSuccess) {
                        (void)cudaGetLastError();
                    }
                }
                o.mappedBase = (uint64_t)p;
                o.mappedSize = e.windowSize;
            }
            o.remoteBlock = blockBase;
            o.local = o.mappedBase + e.fileOffset;
        } else {
            MF_ERROR("user segment: rank " << e.rank << " registered memory that cannot be mapped here (plain host memory)");
            return BM_NOT_SUPPORTED;
        }
        opened_[key] = o;
        *local = o.local;
        return BM_OK;
    }

    void Close(const Opened &o)
    {
        if (o.kind == HK_CUDA_IPC) {
            // Several registrations may share one opened allocation: close it with the last of them.
            int users = 0;
            for (auto &kv : opened_) {
                users += kv.second.kind == HK_CUDA_IPC && kv.second.mappedBase == o.mappedBase;
            }
            if (users <= 1) {
                cudaIpcCloseMemHandle((void *)o.mappedBase);
                (void)cudaGetLastError();
            }
        } else if (o.kind == HK_FD_VMM_RETAINED) {
            const cu::DriverApi *d = cu::Driver();
            if (d != nullptr) {
                d->MemUnmap((CUdeviceptr)o.mappedBase, o.mappedSize);
                d->MemAddressFree((CUdeviceptr)o.mappedBase, o.mappedSize);
            }
        } else if (o.kind == HK_FD_HOST) {
            int users = 0;
            for (auto &kv : opened_) {
                users += kv.second.kind == HK_FD_HOST && kv.second.mappedBase == o.mappedBase;
            }
            if (users <= 1) {
                if (cu::Available()) {
                    cudaHostUnregister((void *)o.mappedBase);
                    (void)cudaGetLastError();
                }
                ::munmap((void *)o.mappedBase, o.mappedSize);
            }
        }
    }

    std::map<std::pair<uint32_t, uint64_t>, Opened> opened_;
    std::map<std::pair<uint32_t, uint64_t>, std::string> ipcOf_;
};

std::shared_ptr<MemSegment> MemSegment::Create(const SegmentOptions &opt)
{
    if (opt.rankCount == 0 || opt.rankCount > RANK_MAX || opt.rankId >= opt.rankCount) {
        MF_ERROR("segment: invalid rank " << opt.rankId << "/" << opt.rankCount);
        return nullptr;
    }
    switch (opt.type) {
        case SEG_DEVICE_VMM:
            if (cu::Driver() == nullptr || opt.devId < 0) {
                MF_ERROR("segment: an HBM segment needs a GPU with virtual memory management");
                return nullptr;
            }
            if (opt.windowSize == 0 || opt.windowSize % GRANULE != 0) {
                MF_ERROR("segment: window size must be a non-zero multiple of 2 MiB");
                return nullptr;
            }
            return std::make_shared<DeviceVmmSegment>(opt);
        case SEG_HOST_SHM:
            if (opt.windowSize == 0 || opt.windowSize % GRANULE != 0) {
                MF_ERROR("segment: window size must be a non-zero multiple of 2 MiB");
                return nullptr;
            }
            return std::make_shared<HostShmSegment>(opt);
        case SEG_USER_MEM:
            return std::make_shared<UserMemSegment>(opt);
        default:
            return nullptr;
    }
}

}  // namespace hybm
}  // namespace mf

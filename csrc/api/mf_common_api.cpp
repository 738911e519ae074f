// Common part of the public C API (include/mf/mf.h). Reference: src/smem/csrc/smem.cpp:27-105.
#include <cstring>
#include <mutex>

#include "../net/mf_rpc.h"
#include "../store/mf_store_client.h"
#include "../net/mf_tls.h"
#include "../util/mf_log.h"
#include "../util/mf_tracer.h"
#include "mf/mf.h"
#include "mf_api_internal.h"

using namespace mf;

namespace mf {
namespace api {

int MapHybmCode(int rc)
{
    switch (rc) {
        case hybm::BM_OK:
            return MF_OK;
        case hybm::BM_INVALID_PARAM:
            return MF_INVALID_PARAM;
        case hybm::BM_MALLOC_FAILED:
            return MF_MALLOC_FAILED;
        case hybm::BM_NEW_OBJECT_FAILED:
            return MF_NEW_OBJECT_FAILED;
        case hybm::BM_TIMEOUT:
            return MF_TIMEOUT;
        case hybm::BM_NOT_INITIALIZED:
            return MF_NOT_INITIALIZED;
        default:
            return MF_ERROR;
    }
}

int MapGroupCode(int rc)
{
    switch (rc) {
        case group::GR_OK:
            return MF_OK;
        case group::GR_INVALID_PARAM:
            return MF_INVALID_PARAM;
        case group::GR_TIMEOUT:
            return MF_TIMEOUT;
        case group::GR_NOT_STARTED:
            return MF_NOT_STARTED;
        default:
            return MF_ERROR;
    }
}

store::StorePtr OpenStore(const std::string &url, bool tryServe, bool mustServe, uint32_t worldSize, int32_t rankId, uint32_t timeoutSec, int *rcOut)
{
    net::Endpoint ep;
    if (!net::ParseUrl(url, &ep)) {
        MF_ERROR("store url '" << url << "' is not tcp://ip:port");
        *rcOut = MF_INVALID_PARAM;
        return nullptr;
    }
    int retries = (int)std::max<uint32_t>(1, std::min<uint32_t>(timeoutSec, 600));
    if (tryServe) {
        auto st = store::StoreFactory::CreateStore(ep, true, worldSize, rankId, retries);
        if (st) {
            *rcOut = MF_OK;
            return st;
        }
        if (mustServe || store::StoreFactory::LastFailure() != -EADDRINUSE) {
            *rcOut = store::StoreFactory::LastFailure() == -EADDRINUSE ? MF_RESOURCE_IN_USE : MF_ERROR;
            if (mustServe) {
                MF_ERROR("cannot host the config store on " << url);
                return nullptr;
            }
        }
        // Somebody else already serves this address: be a client.
    }
    auto st = store::StoreFactory::CreateStore(ep, false, worldSize, rankId, retries);
    *rcOut = st ? MF_OK : MF_ERROR;
    return st;
}

bool UrlIsLocal(const std::string &url)
{
    net::Endpoint ep;
    if (!net::ParseUrl(url, &ep)) {
        return false;
    }
    if (ep.host == "127.0.0.1" || ep.host == "::1" || ep.host == "localhost" || ep.host == "0.0.0.0") {
        return true;
    }
    for (auto &ip : net::LocalIpv4List()) {
        if (ip == ep.host) {
            return true;
        }
    }
    return net::LocalIpToward(ep) == ep.host;
}

}  // namespace api
}  // namespace mf

static std::mutex g_mu;
static int g_inited = 0;

extern "C" int32_t mf_init(uint32_t /*flags*/)
{
    std::lock_guard<std::mutex> g(g_mu);
    g_inited++;
    return MF_OK;
}

extern "C" void mf_uninit(void)
{
    std::lock_guard<std::mutex> g(g_mu);
    if (g_inited > 0 && --g_inited == 0) {
        store::StoreFactory::DestroyAll();
    }
}

extern "C" int32_t mf_create_config_store(const char *storeUrl)
{
    if (storeUrl == nullptr) {
        MF_ERROR("create_config_store: null url");
        return MF_INVALID_PARAM;
    }
    net::Endpoint ep;
    if (!net::ParseUrl(storeUrl, &ep)) {
        MF_ERROR("create_config_store: '" << storeUrl << "' is not tcp://ip:port");
        return MF_INVALID_PARAM;
    }
    store::StoreServer *srv = nullptr;
    int rc = store::StoreFactory::CreateServer(ep, 0, &srv);
    if (rc == -EADDRINUSE) {
        MF_ERROR("create_config_store: " << storeUrl << " is already in use");
        return MF_RESOURCE_IN_USE;
    }
    if (rc != 0) {
        MF_ERROR("create_config_store: cannot listen on " << storeUrl);
        return MF_ERROR;
    }
    // The transfer engine's fault handler observes this server (see mf_trans_fault.cpp).
    mf::api::AttachTransFaultHandler(srv);
    return MF_OK;
}

extern "C" void mf_destroy_config_store(const char *storeUrl)
{
    net::Endpoint ep;
    if (storeUrl != nullptr && net::ParseUrl(storeUrl, &ep)) {
        store::StoreFactory::DestroyServer(ep.port);
    }
}

extern "C" int32_t mf_set_extern_logger(void (*func)(int, const char *))
{
    Logger::Instance().SetExtern(func);
    return MF_OK;
}

extern "C" int32_t mf_set_log_level(int level)
{
    if (level < LOG_DEBUG || level > LOG_OFF) {
        MF_ERROR("set_log_level: level " << level << " is out of range");
        return MF_INVALID_PARAM;
    }
    Logger::Instance().SetLevel(level);
    return MF_OK;
}

// TLS for every config-store link of this process (reference: smem_set_conf_store_tls / smem_set_config_store_tls_key,
// src/smem/include/host/smem.h; text form of doc/SECURITYNOTE.md:27-61). The options take effect for servers started and
// clients connected afterwards; both ends of a store must use the same setting.
extern "C" int32_t mf_set_conf_store_tls(bool enable, const char *tlsInfo, uint32_t tlsInfoLen)
{
    net::TlsOptions opt = net::GetStoreTlsOptions();
    if (!enable) {
        opt.enable = false;
        net::SetStoreTlsOptions(opt);
        return MF_OK;
    }
    if (tlsInfo == nullptr || tlsInfoLen == 0 || tlsInfoLen > 64 * 1024) {
        MF_ERROR("set_conf_store_tls: enabling TLS needs the option text (tlsCaPath, tlsCaFile, tlsCert, ...)");
        return MF_INVALID_PARAM;
    }
    net::TlsOptions parsed;
    parsed.pk = opt.pk;  // a key registered earlier stays
    parsed.pkPwd = opt.pkPwd;
    parsed.decrypt = opt.decrypt;
    std::string err;
    if (!net::ParseTlsInfo(std::string(tlsInfo, tlsInfoLen), &parsed, &err)) {
        MF_ERROR("set_conf_store_tls: " << err);
        return MF_INVALID_PARAM;
    }
    if (!net::TlsLibraryAvailable(parsed.packagePath, &err)) {
        MF_ERROR("set_conf_store_tls: " << err);
        return MF_ERROR;
    }
    parsed.enable = true;
    net::SetStoreTlsOptions(parsed);
    return MF_OK;
}

extern "C" int32_t mf_set_config_store_tls_key(const char *tlsPk, uint32_t tlsPkLen, const char *tlsPkPw, uint32_t tlsPkPwLen, mf_decrypt_handler h)
{
    if (tlsPk == nullptr || tlsPkLen == 0 || tlsPkLen > (1u << 20) || (tlsPkPw == nullptr && tlsPkPwLen != 0) || tlsPkPwLen > (10u << 20)) {
        MF_ERROR("set_config_store_tls_key: the private key (PEM text or file path) is required; the pass phrase is at most 10 MiB");
        return MF_INVALID_PARAM;
    }
    net::TlsOptions opt = net::GetStoreTlsOptions();
    opt.pk.assign(tlsPk, tlsPkLen);
    opt.pkPwd.assign(tlsPkPw != nullptr ? tlsPkPw : "", tlsPkPwLen);
    if (h != nullptr) {
        opt.decrypt = [h](const char *cipher, size_t cipherLen, char *plain, size_t &plainLen) { return h(cipher, cipherLen, plain, &plainLen); };
    } else {
        opt.decrypt = nullptr;
    }
    net::SetStoreTlsOptions(opt);
    return MF_OK;
}

extern "C" const char *mf_get_last_err_msg(void) { return LastError::Get(); }
extern "C" const char *mf_get_and_clear_last_err_msg(void) { return LastError::GetAndClear(); }
extern "C" const char *mf_version(void) { return "memfabric-b200 1.0.0 (sm_100a)"; }

extern "C" int32_t mf_trace_enable(const char *dumpDir)
{
    return Tracer::Instance().Init(dumpDir != nullptr ? dumpDir : "") == 0 ? MF_OK : MF_ERROR;
}
extern "C" void mf_trace_disable(void) { Tracer::Instance().Shutdown(); }
extern "C" size_t mf_trace_dump(char *buf, size_t len, bool reset)
{
    std::string s = Tracer::Instance().Dump(reset);
    if (buf != nullptr && len > 0) {
        size_t n = std::min(len - 1, s.size());
        std::memcpy(buf, s.data(), n);
        buf[n] = '\0';
    }
    return s.size();
}

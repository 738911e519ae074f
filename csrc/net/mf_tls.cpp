#include "mf_tls.h"

#include <dlfcn.h>
#include <openssl/err.h>
#include <openssl/pem.h>
#include <openssl/ssl.h>
#include <openssl/x509.h>
#include <openssl/x509_vfy.h>
#include <sys/stat.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <thread>

#include "../util/mf_file_util.h"
#include "../util/mf_log.h"

namespace mf {
namespace net {

namespace {

// Every OpenSSL entry point the module uses, resolved with dlsym. The headers supply the types and constants only; no
// OpenSSL function (and none of the header macros that expand to one) is called by name, so the library links without it.
#define MF_SSL_FUNCS(X)                                                                                                         \
    X(TLS_method) X(SSL_CTX_new) X(SSL_CTX_free) X(SSL_CTX_ctrl) X(SSL_CTX_set_verify) X(SSL_CTX_load_verify_locations)          \
    X(SSL_CTX_use_certificate_chain_file) X(SSL_CTX_use_PrivateKey) X(SSL_CTX_check_private_key) X(SSL_CTX_get_cert_store)      \
    X(SSL_new) X(SSL_free) X(SSL_set_bio) X(SSL_set_accept_state) X(SSL_set_connect_state) X(SSL_do_handshake) X(SSL_get_error) \
    X(SSL_read) X(SSL_write)
#define MF_CRYPTO_FUNCS(X)                                                                                                     \
    X(BIO_new) X(BIO_s_mem) X(BIO_write) X(BIO_read) X(BIO_ctrl) X(BIO_free) X(BIO_new_mem_buf) X(PEM_read_bio_PrivateKey)        \
    X(PEM_read_bio_X509) X(PEM_read_bio_X509_CRL) X(EVP_PKEY_free) X(X509_free) X(X509_CRL_free) X(X509_STORE_add_crl)          \
    X(X509_STORE_set_flags) X(X509_cmp_time) X(X509_get0_notAfter) X(X509_get0_notBefore) X(ERR_get_error) X(ERR_error_string_n) \
    X(ERR_clear_error)

struct Api {
    void *ssl{nullptr};
    void *crypto{nullptr};
#define X(name) decltype(&::name) name{nullptr};
    MF_SSL_FUNCS(X)
    MF_CRYPTO_FUNCS(X)
#undef X
};

std::mutex g_apiMu;
Api *g_api = nullptr;

Api *LoadApi(const std::string &packagePath, std::string *err)
{
    std::lock_guard<std::mutex> g(g_apiMu);
    if (g_api != nullptr) {
        return g_api;
    }
    auto open = [&](const char *name) -> void * {
        void *h = nullptr;
        if (!packagePath.empty()) {
            // Only a regular file that really lives in the configured directory is handed to dlopen.
            std::string real;
            if (util::ResolveLibrary(packagePath, name, &real)) {
                h = dlopen(real.c_str(), RTLD_NOW | RTLD_GLOBAL);
            }
        }
        return h != nullptr ? h : dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    };
    auto *a = new Api();
    a->crypto = open("libcrypto.so.3");
    a->ssl = open("libssl.so.3");
    if (a->crypto == nullptr || a->ssl == nullptr) {
        if (err != nullptr) {
            *err = std::string("cannot load OpenSSL 3 (libssl.so.3 / libcrypto.so.3): ") + (dlerror() ? dlerror() : "not found");
        }
        delete a;
        return nullptr;
    }
    bool ok = true;
    std::string missing;
#define X(name)                                                       \
    a->name = reinterpret_cast<decltype(a->name)>(dlsym(a->ssl, #name)); \
    if (a->name == nullptr) {                                         \
        ok = false;                                                   \
        missing = #name;                                              \
    }
    MF_SSL_FUNCS(X)
#undef X
#define X(name)                                                          \
    a->name = reinterpret_cast<decltype(a->name)>(dlsym(a->crypto, #name)); \
    if (a->name == nullptr) {                                            \
        ok = false;                                                      \
        missing = #name;                                                 \
    }
    MF_CRYPTO_FUNCS(X)
#undef X
    if (!ok) {
        if (err != nullptr) {
            *err = "OpenSSL library lacks " + missing;
        }
        delete a;
        return nullptr;
    }
    g_api = a;
    return g_api;
}

std::string SslErrors(Api *a)
{
    std::string out;
    unsigned long e;
    char buf[256];
    while ((e = a->ERR_get_error()) != 0) {
        a->ERR_error_string_n(e, buf, sizeof(buf));
        if (!out.empty()) {
            out += "; ";
        }
        out += buf;
    }
    return out.empty() ? "no detail" : out;
}

std::string Trim(const std::string &s)
{
    size_t b = s.find_first_not_of(" \t\r\n"), e = s.find_last_not_of(" \t\r\n");
    return b == std::string::npos ? "" : s.substr(b, e - b + 1);
}

std::vector<std::string> SplitList(const std::string &s, char sep)
{
    std::vector<std::string> out;
    size_t pos = 0;
    while (pos <= s.size()) {
        size_t next = s.find(sep, pos);
        std::string item = Trim(s.substr(pos, next == std::string::npos ? std::string::npos : next - pos));
        if (!item.empty()) {
            out.push_back(item);
        }
        if (next == std::string::npos) {
            break;
        }
        pos = next + 1;
    }
    return out;
}

// Certificates, keys, CRLs and pass-phrase files: regular files, leaf not a symbolic link, at most 10 MiB.
bool ReadFile(const std::string &path, std::string *out)
{
    std::string why;
    if (!util::ReadConfigFile(path, util::kMaxConfigFileBytes, out, &why)) {
        MF_WARN("tls: " << why);
        return false;
    }
    return true;
}

bool IsFile(const std::string &path)
{
    return util::IsRegularFile(path);
}

std::string Join(const std::string &dir, const std::string &file)
{
    if (file.empty() || file[0] == '/' || dir.empty()) {
        return file;
    }
    return dir.back() == '/' ? dir + file : dir + "/" + file;
}

int PasswordCb(char *buf, int size, int /*rwflag*/, void *u)
{
    const std::string *pw = static_cast<const std::string *>(u);
    if (pw == nullptr || (int)pw->size() > size) {
        return 0;
    }
    std::memcpy(buf, pw->data(), pw->size());
    return (int)pw->size();
}

void Wipe(std::string *s)
{
    volatile char *p = s->empty() ? nullptr : &(*s)[0];
    for (size_t i = 0; i < s->size(); i++) {
        p[i] = 0;
    }
    s->clear();
}

std::mutex g_optMu;
TlsOptions g_storeOpt;

// Periodic certificate check of one context (the reference's CheckCertExpiredTask).
class CertWatcher {
public:
    CertWatcher(std::vector<std::string> files, Api *a) : files_(std::move(files)), api_(a) {}
    ~CertWatcher() { Stop(); }
    void Start()
    {
        th_ = std::thread([this]() {
            int periodHours, aheadDays;
            CertCheckParams(&periodHours, &aheadDays);
            std::unique_lock<std::mutex> lk(mu_);
            while (!stop_) {
                cv_.wait_for(lk, std::chrono::hours(periodHours));
                if (stop_) {
                    break;
                }
                lk.unlock();
                Check(aheadDays, nullptr);
                lk.lock();
            }
        });
    }
    void Stop()
    {
        {
            std::lock_guard<std::mutex> g(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        if (th_.joinable()) {
            th_.join();
        }
    }
    int Check(int aheadDays, std::string *detail) const
    {
        int worst = 0;
        const time_t now = time(nullptr);
        time_t horizon = now + (time_t)aheadDays * 86400;
        for (const std::string &path : files_) {
            std::string pem;
            if (!ReadFile(path, &pem)) {
                MF_ERROR("tls: certificate check cannot read " << path);
                if (detail != nullptr) {
                    *detail = "unreadable: " + path;
                }
                return -1;
            }
            BIO *bio = api_->BIO_new_mem_buf(pem.data(), (int)pem.size());
            X509 *x = bio != nullptr ? api_->PEM_read_bio_X509(bio, nullptr, nullptr, nullptr) : nullptr;
            if (bio != nullptr) {
                api_->BIO_free(bio);
            }
            if (x == nullptr) {
                api_->ERR_clear_error();
                MF_ERROR("tls: certificate check cannot parse " << path);
                if (detail != nullptr) {
                    *detail = "unparsable: " + path;
                }
                return -1;
            }
            time_t t = now;
            const int afterNow = api_->X509_cmp_time(api_->X509_get0_notAfter(x), &t);
            t = now;
            const int beforeNow = api_->X509_cmp_time(api_->X509_get0_notBefore(x), &t);
            const int afterHorizon = api_->X509_cmp_time(api_->X509_get0_notAfter(x), &horizon);
            api_->X509_free(x);
            if (afterNow <= 0 || beforeNow > 0) {
                MF_ERROR("tls: certificate " << path << (afterNow <= 0 ? " has expired" : " is not valid yet"));
                if (detail != nullptr) {
                    *detail = (afterNow <= 0 ? "expired: " : "not valid yet: ") + path;
                }
                return -1;
            }
            if (afterHorizon <= 0) {
                MF_WARN("tls: certificate " << path << " expires within " << aheadDays << " days");
                if (detail != nullptr) {
                    *detail = "expires soon: " + path;
                }
                worst = 1;
            }
        }
        return worst;
    }

private:
    std::vector<std::string> files_;
    Api *api_;
    std::thread th_;
    std::mutex mu_;
    std::condition_variable cv_;
    bool stop_{false};
};

std::mutex g_watchMu;
std::vector<std::pair<void *, std::unique_ptr<CertWatcher>>> g_watchers;  // keyed by SSL_CTX

}  // namespace

bool TlsLibraryAvailable(const std::string &packagePath, std::string *err) { return LoadApi(packagePath, err) != nullptr; }

TlsDecryptFn LoadDecrypterLibrary(const std::string &path, std::string *err)
{
    auto fail = [&](const std::string &m) {
        if (err != nullptr) {
            *err = m;
        }
        return TlsDecryptFn();
    };
    std::string why;
    if (!util::CheckConfigFile(path, 256u << 20, false, &why)) {
        return fail("decrypter library: " + why);
    }
    std::string real = path;
    if (!util::Canonicalize(&real)) {
        return fail("decrypter library: cannot resolve " + path);
    }
    void *h = dlopen(real.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (h == nullptr) {
        const char *e = dlerror();
        return fail(std::string("decrypter library: dlopen failed: ") + (e ? e : "unknown"));
    }
    using RawFn = int (*)(const char *, size_t, char *, size_t);
    RawFn fn = (RawFn)dlsym(h, "DecryptPassword");
    if (fn == nullptr) {
        dlclose(h);
        return fail("decrypter library: symbol DecryptPassword not found in " + real);
    }
    return [fn](const char *cipher, size_t cipherLen, char *plain, size_t &plainLen) -> int {
        if (plain == nullptr || plainLen == 0) {
            return -1;
        }
        std::memset(plain, 0, plainLen);
        int rc = fn(cipher, cipherLen, plain, plainLen - 1);
        if (rc != 0) {
            return rc;
        }
        plainLen = strnlen(plain, plainLen - 1);
        return 0;
    };
}

bool TlsOptionsFromPaths(const TlsConfigPaths &in, TlsOptions *out, std::string *err)
{
    if (out == nullptr) {
        return false;
    }
    *out = TlsOptions();
    out->enable = in.enable;
    if (!in.enable) {
        return true;
    }
    if (in.caPath.empty() || in.certPath.empty() || in.keyPath.empty()) {
        if (err != nullptr) {
            *err = "tls config: caPath, certPath and keyPath are required";
        }
        return false;
    }
    out->caFiles = {in.caPath};
    if (!in.crlPath.empty()) {
        out->crlFiles = {in.crlPath};
    }
    out->cert = in.certPath;
    out->pk = in.keyPath;
    out->pkPwd = in.keyPassPath;
    out->packagePath = in.packagePath;
    if (!in.decrypterLibPath.empty()) {
        out->decrypt = LoadDecrypterLibrary(in.decrypterLibPath, err);
        if (!out->decrypt) {
            return false;
        }
    }
    return true;
}

void SetStoreTlsOptions(const TlsOptions &opt)
{
    std::lock_guard<std::mutex> g(g_optMu);
    g_storeOpt = opt;
}

TlsOptions GetStoreTlsOptions()
{
    std::lock_guard<std::mutex> g(g_optMu);
    return g_storeOpt;
}

void CertCheckParams(int *periodHours, int *aheadDays)
{
    auto envInt = [](const char *name) -> long {
        const char *v = getenv(name);
        if (v == nullptr || *v == 0) {
            return -1;
        }
        char *end = nullptr;
        long x = strtol(v, &end, 10);
        return (end == nullptr || *end != 0) ? -1 : x;
    };
    long p = envInt("ACCLINK_CHECK_PERIOD_HOURS");
    if (p < 24 || p > 24 * 30) {
        p = 7 * 24;
    }
    long d = envInt("ACCLINK_CERT_CHECK_AHEAD_DAYS");
    if (d < 7 || d > 180 || d * 24 < p) {
        d = 30;
    }
    *periodHours = (int)p;
    *aheadDays = (int)d;
}

bool ParseTlsInfo(const std::string &text, TlsOptions *out, std::string *err)
{
    for (const std::string &entry : SplitList(text, ';')) {
        size_t colon = entry.find(':');
        if (colon == std::string::npos) {
            if (err != nullptr) {
                *err = "tls info: '" + entry + "' is not 'key: value'";
            }
            return false;
        }
        const std::string key = Trim(entry.substr(0, colon)), val = Trim(entry.substr(colon + 1));
        if (key == "tlsCaPath") {
            out->caPath = val;
        } else if (key == "tlsCert") {
            out->cert = val;
        } else if (key == "tlsCrlPath") {
            out->crlPath = val;
        } else if (key == "tlsCrlFile") {
            out->crlFiles = SplitList(val, ',');
        } else if (key == "tlsCaFile") {
            out->caFiles = SplitList(val, ',');
        } else if (key == "packagePath") {
            out->packagePath = val;
        } else if (key == "tlsPk") {
            out->pk = val;
        } else if (key == "tlsPkPwd") {
            out->pkPwd = val;
        } else {
            if (err != nullptr) {
                *err = "tls info: unknown key '" + key + "'";
            }
            return false;
        }
    }
    if (out->cert.empty() || out->caFiles.empty()) {
        if (err != nullptr) {
            *err = "tls info: tlsCert and tlsCaFile are required";
        }
        return false;
    }
    return true;
}

// ------------------------------------------------------------------------------------------------ context

TlsContext::~TlsContext()
{
    {
        std::lock_guard<std::mutex> g(g_watchMu);
        for (auto it = g_watchers.begin(); it != g_watchers.end(); ++it) {
            if (it->first == ctx_) {
                g_watchers.erase(it);
                break;
            }
        }
    }
    if (ctx_ != nullptr && g_api != nullptr) {
        g_api->SSL_CTX_free(static_cast<SSL_CTX *>(ctx_));
    }
}

std::shared_ptr<TlsContext> TlsContext::Create(const TlsOptions &opt, bool server, std::string *err)
{
    std::string why;
    auto fail = [&](const std::string &m) -> std::shared_ptr<TlsContext> {
        MF_ERROR("tls: " << m);
        if (err != nullptr) {
            *err = m;
        }
        return nullptr;
    };
    Api *a = LoadApi(opt.packagePath, &why);
    if (a == nullptr) {
        return fail(why);
    }
    if (opt.cert.empty() || opt.caFiles.empty() || opt.pk.empty()) {
        return fail("certificate, CA file(s) and private key are all required");
    }
    SSL_CTX *ctx = a->SSL_CTX_new(a->TLS_method());
    if (ctx == nullptr) {
        return fail("SSL_CTX_new failed: " + SslErrors(a));
    }
    std::shared_ptr<TlsContext> out(new TlsContext());
    out->ctx_ = ctx;
    out->server_ = server;
    a->SSL_CTX_ctrl(ctx, SSL_CTRL_SET_MIN_PROTO_VERSION, TLS1_3_VERSION, nullptr);
    a->SSL_CTX_ctrl(ctx, SSL_CTRL_SET_MAX_PROTO_VERSION, TLS1_3_VERSION, nullptr);
    a->SSL_CTX_ctrl(ctx, SSL_CTRL_MODE, SSL_MODE_ENABLE_PARTIAL_WRITE | SSL_MODE_ACCEPT_MOVING_WRITE_BUFFER, nullptr);
    // Both ends present a certificate and verify the other's.
    a->SSL_CTX_set_verify(ctx, SSL_VERIFY_PEER | SSL_VERIFY_FAIL_IF_NO_PEER_CERT, nullptr);
    for (const std::string &f : opt.caFiles) {
        const std::string path = Join(opt.caPath, f);
        if (a->SSL_CTX_load_verify_locations(ctx, path.c_str(), nullptr) != 1) {
            return fail("cannot load CA file " + path + ": " + SslErrors(a));
        }
        out->certFiles_.push_back(path);
    }
    if (!opt.crlFiles.empty()) {
        X509_STORE *store = a->SSL_CTX_get_cert_store(ctx);
        for (const std::string &f : opt.crlFiles) {
            const std::string path = Join(opt.crlPath, f);
            std::string pem;
            if (!ReadFile(path, &pem)) {
                return fail("cannot read CRL file " + path);
            }
            BIO *bio = a->BIO_new_mem_buf(pem.data(), (int)pem.size());
            X509_CRL *crl = bio != nullptr ? a->PEM_read_bio_X509_CRL(bio, nullptr, nullptr, nullptr) : nullptr;
            if (bio != nullptr) {
                a->BIO_free(bio);
            }
            if (crl == nullptr || a->X509_STORE_add_crl(store, crl) != 1) {
                if (crl != nullptr) {
                    a->X509_CRL_free(crl);
                }
                return fail("cannot load CRL file " + path + ": " + SslErrors(a));
            }
            a->X509_CRL_free(crl);
        }
        a->X509_STORE_set_flags(store, X509_V_FLAG_CRL_CHECK);
    }
    if (a->SSL_CTX_use_certificate_chain_file(ctx, opt.cert.c_str()) != 1) {
        return fail("cannot load certificate " + opt.cert + ": " + SslErrors(a));
    }
    out->certFiles_.insert(out->certFiles_.begin(), opt.cert);
    // Private key: PEM text or a file; pass phrase: text or a file, run through the decrypter when one is registered.
    std::string pem = opt.pk;
    if (pem.find("-----BEGIN") == std::string::npos) {
        if (!ReadFile(opt.pk, &pem)) {
            return fail("cannot read private key file " + opt.pk);
        }
    }
    std::string pass = opt.pkPwd;
    if (IsFile(pass)) {
        std::string fromFile;
        if (ReadFile(pass, &fromFile)) {
            pass = Trim(fromFile);
        }
    }
    if (opt.decrypt && !pass.empty()) {
        std::string plain(pass.size() * 2 + 256, '\0');
        size_t n = plain.size();
        if (opt.decrypt(pass.data(), pass.size(), &plain[0], n) != 0 || n > plain.size()) {
            Wipe(&plain);
            return fail("the key pass phrase decrypter failed");
        }
        plain.resize(n);
        while (!plain.empty() && plain.back() == '\0') {
            plain.pop_back();
        }
        Wipe(&pass);
        pass = plain;
        Wipe(&plain);
    }
    BIO *kb = a->BIO_new_mem_buf(pem.data(), (int)pem.size());
    EVP_PKEY *key = kb != nullptr ? a->PEM_read_bio_PrivateKey(kb, nullptr, PasswordCb, &pass) : nullptr;
    if (kb != nullptr) {
        a->BIO_free(kb);
    }
    Wipe(&pass);
    Wipe(&pem);
    if (key == nullptr) {
        return fail("cannot parse the private key (wrong pass phrase?): " + SslErrors(a));
    }
    const bool keyOk = a->SSL_CTX_use_PrivateKey(ctx, key) == 1 && a->SSL_CTX_check_private_key(ctx) == 1;
    a->EVP_PKEY_free(key);
    if (!keyOk) {
        return fail("the private key does not match the certificate: " + SslErrors(a));
    }
    int periodHours, aheadDays;
    CertCheckParams(&periodHours, &aheadDays);
    std::string detail;
    if (out->CheckCertificates(aheadDays, &detail) < 0) {
        return fail("certificate check failed (" + detail + ")");
    }
    {
        std::lock_guard<std::mutex> g(g_watchMu);
        g_watchers.emplace_back(ctx, std::unique_ptr<CertWatcher>(new CertWatcher(out->certFiles_, a)));
        g_watchers.back().second->Start();
    }
    return out;
}

int TlsContext::CheckCertificates(int aheadDays, std::string *detail) const
{
    if (g_api == nullptr) {
        return -1;
    }
    CertWatcher once(certFiles_, g_api);
    return once.Check(aheadDays, detail);
}

std::unique_ptr<TlsSession> TlsContext::NewSession()
{
    Api *a = g_api;
    SSL *ssl = a->SSL_new(static_cast<SSL_CTX *>(ctx_));
    BIO *r = a->BIO_new(a->BIO_s_mem());
    BIO *w = a->BIO_new(a->BIO_s_mem());
    if (ssl == nullptr || r == nullptr || w == nullptr) {
        if (ssl != nullptr) {
            a->SSL_free(ssl);
        }
        if (r != nullptr) {
            a->BIO_free(r);
        }
        if (w != nullptr) {
            a->BIO_free(w);
        }
        return nullptr;
    }
    a->SSL_set_bio(ssl, r, w);  // the session owns both from here on
    if (server_) {
        a->SSL_set_accept_state(ssl);
    } else {
        a->SSL_set_connect_state(ssl);
    }
    std::unique_ptr<TlsSession> s(new TlsSession());
    s->ssl_ = ssl;
    s->rbio_ = r;
    s->wbio_ = w;
    return s;
}

// ------------------------------------------------------------------------------------------------ session

TlsSession::~TlsSession()
{
    if (ssl_ != nullptr && g_api != nullptr) {
        g_api->SSL_free(static_cast<SSL *>(ssl_));
    }
}

bool TlsSession::Feed(const char *data, size_t len)
{
    Api *a = g_api;
    size_t off = 0;
    while (off < len) {
        int n = a->BIO_write(static_cast<BIO *>(rbio_), data + off, (int)std::min<size_t>(len - off, 1u << 20));
        if (n <= 0) {
            return false;
        }
        off += (size_t)n;
    }
    return true;
}

void TlsSession::DrainWire(std::string *wire)
{
    Api *a = g_api;
    char buf[16384];
    while (a->BIO_ctrl(static_cast<BIO *>(wbio_), BIO_CTRL_PENDING, 0, nullptr) > 0) {
        int n = a->BIO_read(static_cast<BIO *>(wbio_), buf, sizeof(buf));
        if (n <= 0) {
            break;
        }
        wire->append(buf, (size_t)n);
    }
}

int TlsSession::Pump(std::string *plain, std::string *wire)
{
    Api *a = g_api;
    SSL *ssl = static_cast<SSL *>(ssl_);
    if (!done_) {
        a->ERR_clear_error();
        int r = a->SSL_do_handshake(ssl);
        if (r == 1) {
            done_ = true;
        } else {
            int e = a->SSL_get_error(ssl, r);
            if (e != SSL_ERROR_WANT_READ && e != SSL_ERROR_WANT_WRITE) {
                err_ = "handshake failed: " + SslErrors(a);
                DrainWire(wire);  // the alert that tells the peer why
                return -1;
            }
        }
        DrainWire(wire);
    }
    if (done_) {
        char buf[16384];
        while (true) {
            a->ERR_clear_error();
            int n = a->SSL_read(ssl, buf, sizeof(buf));
            if (n > 0) {
                plain->append(buf, (size_t)n);
                continue;
            }
            int e = a->SSL_get_error(ssl, n);
            if (e == SSL_ERROR_WANT_READ || e == SSL_ERROR_WANT_WRITE || e == SSL_ERROR_ZERO_RETURN) {
                break;
            }
            err_ = "read failed: " + SslErrors(a);
            DrainWire(wire);
            return -1;
        }
        DrainWire(wire);
    }
    return 0;
}

int TlsSession::Encrypt(const char *data, size_t len, std::string *wire)
{
    if (!done_) {
        err_ = "write before the handshake finished";
        return -1;
    }
    Api *a = g_api;
    SSL *ssl = static_cast<SSL *>(ssl_);
    size_t off = 0;
    while (off < len) {
        a->ERR_clear_error();
        int n = a->SSL_write(ssl, data + off, (int)std::min<size_t>(len - off, 1u << 20));
        if (n <= 0) {
            err_ = "write failed: " + SslErrors(a);
            return -1;
        }
        off += (size_t)n;
        DrainWire(wire);  // the memory BIO grows without bound otherwise
    }
    DrainWire(wire);
    return 0;
}

}  // namespace net
}  // namespace mf

// TLS 1.3 for the control-plane links (config store and everything built on it).
//
// Role of the reference's acc_links security layer (src/acc_links/csrc/security/acc_tcp_ssl_helper.cpp:1-610: OpenSSL loaded at
// run time, CA / CRL / certificate / encrypted private key, pluggable key-pass decrypter, periodic certificate-expiry check
// driven by ACCLINK_CHECK_PERIOD_HOURS and ACCLINK_CERT_CHECK_AHEAD_DAYS) and of the store's option mapping
// (src/smem/csrc/config_store/tcp_store/smem_tcp_config_store_ssl_helper.h). Design here: OpenSSL 3 is dlopen'ed (libssl.so.3,
// from `packagePath` when given) so the library still loads on hosts without it; a TlsSession runs the protocol over MEMORY
// BIOs, i.e. it turns received ciphertext into plaintext and plaintext into ciphertext without ever touching a socket, which
// lets the epoll server and the blocking client of mf_rpc keep their own I/O loops. Both sides authenticate (mutual TLS):
// the peer's certificate must chain to one of the configured CAs and must not be on a configured CRL.
#pragma once
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace mf {
namespace net {

// int handler(cipher, cipherLen, plainOut, plainLenInOut): 0 on success (mf_decrypt_handler of the public API).
using TlsDecryptFn = std::function<int(const char *cipher, size_t cipherLen, char *plain, size_t &plainLen)>;

struct TlsOptions {
    bool enable{false};
    std::string caPath;                // directory of the CA files (may be empty when caFiles are absolute)
    std::vector<std::string> caFiles;  // at least one
    std::string cert;                  // this side's certificate (PEM; a chain file is fine)
    std::string crlPath;
    std::vector<std::string> crlFiles;
    std::string packagePath;  // directory that holds libssl.so.3 / libcrypto.so.3 (default: the system's)
    std::string pk;           // private key: PEM text, or the path of a PEM file
    std::string pkPwd;        // key pass phrase: the text itself or the path of a file holding it; cipher text if `decrypt` is set
    TlsDecryptFn decrypt;
};

// Parses the reference's text form "tlsCaPath: /x/; tlsCert: /x/server.crt; tlsCaFile: a.pem,b.pem; tlsCrlPath: ...; tlsCrlFile: ...;
// packagePath: ..." (doc/SECURITYNOTE.md:27-61 of the reference). Unknown keys are an error. Returns false and fills *err.
bool ParseTlsInfo(const std::string &text, TlsOptions *out, std::string *err);

class TlsSession;

// One SSL_CTX (server or client role) built from TlsOptions. Thread-safe to share between links.
class TlsContext {
public:
    ~TlsContext();
    static std::shared_ptr<TlsContext> Create(const TlsOptions &opt, bool server, std::string *err);
    std::unique_ptr<TlsSession> NewSession();
    bool IsServer() const { return server_; }
    // 0: every configured certificate (own + CAs) is inside its validity period and stays so for `aheadDays` more days;
    // 1: valid now but one of them expires within `aheadDays` (a warning is logged); -1: one is expired or not yet valid, or
    // unreadable. The reference runs the same check at start-up and then every ACCLINK_CHECK_PERIOD_HOURS.
    int CheckCertificates(int aheadDays, std::string *detail) const;

private:
    TlsContext() = default;
    void *ctx_{nullptr};  // SSL_CTX
    bool server_{false};
    std::vector<std::string> certFiles_;
    friend class TlsSession;
};

// Period and warning horizon of the certificate check from the environment, with the reference's ranges and defaults:
// ACCLINK_CHECK_PERIOD_HOURS in [24, 720] else 168; ACCLINK_CERT_CHECK_AHEAD_DAYS in [7, 180] and >= the period else 30.
void CertCheckParams(int *periodHours, int *aheadDays);

// The protocol state of one link over memory BIOs. Not thread-safe: callers serialise access per session.
class TlsSession {
public:
    ~TlsSession();
    // Hands received ciphertext to the session.
    bool Feed(const char *data, size_t len);
    // Advances the handshake and decrypts what is available: plaintext is appended to *plain, ciphertext that must be sent to
    // the peer (handshake records, alerts, key updates) to *wire. Returns 0, or -1 on a fatal protocol error (close the link).
    int Pump(std::string *plain, std::string *wire);
    // Encrypts application data; the ciphertext is appended to *wire. Only valid once HandshakeDone(). Returns 0 or -1.
    int Encrypt(const char *data, size_t len, std::string *wire);
    bool HandshakeDone() const { return done_; }
    std::string LastError() const { return err_; }

private:
    friend class TlsContext;
    TlsSession() = default;
    void DrainWire(std::string *wire);
    void *ssl_{nullptr};   // SSL
    void *rbio_{nullptr};  // BIO the session reads ciphertext from (owned by ssl_)
    void *wbio_{nullptr};  // BIO the session writes ciphertext to (owned by ssl_)
    bool done_{false};
    std::string err_;
};

// The struct form of the options carried by the BM configuration (mf_tls_config: one CA file, one CRL file, certificate, key,
// pass-phrase file, OpenSSL directory, decrypter library). Fills *out; loads the decrypter library when one is named.
struct TlsConfigPaths {
    bool enable{false};
    std::string caPath, crlPath, certPath, keyPath, keyPassPath, packagePath, decrypterLibPath;
};
bool TlsOptionsFromPaths(const TlsConfigPaths &in, TlsOptions *out, std::string *err);
// Loads a key-pass decrypter from a shared object by path and returns it as a TlsDecryptFn (empty on failure, *err says
// why). The library must be a regular, non-symlinked file and export
//     int DecryptPassword(const char *cipherText, size_t cipherTextLen, char *plainText, size_t plainTextCapacity)
// which writes a NUL-terminated pass phrase (the reference's plug-in contract, src/util/csrc/mf_tls_util.h:32-48).
// The library stays loaded for the life of the process.
TlsDecryptFn LoadDecrypterLibrary(const std::string &path, std::string *err);

// Process-wide options for the config store's links, set through mf_set_conf_store_tls / mf_set_config_store_tls_key.
void SetStoreTlsOptions(const TlsOptions &opt);
TlsOptions GetStoreTlsOptions();
// True if the OpenSSL libraries could be loaded (from packagePath if non-empty).
bool TlsLibraryAvailable(const std::string &packagePath, std::string *err);

}  // namespace net
}  // namespace mf

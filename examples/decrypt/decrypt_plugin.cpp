// Example of a key-pass decrypter plug-in for TLS on the config-store links.
//
// Deployments rarely keep the pass phrase of a private key in clear text; they store it encrypted by a key-management
// service and hand the library a function that turns the stored form back into the pass phrase at the moment the key is
// loaded. This file builds into a small shared object that exports such a function, and main() below shows both ways to
// use it: link it and pass the function pointer to mf_set_config_store_tls_key, or dlopen it by path at run time.
// Counterpart of the reference's example/decrypt/decrypt_example.cpp (a toy that reverses the string); the toy here is
// hex decoding ("73336372" -> "s3cr"), which is just as insecure and just as easy to follow.
//
//   g++ -std=c++17 -shared -fPIC -DMF_DECRYPT_PLUGIN_ONLY -o libmf_decrypt_example.so decrypt_plugin.cpp
//   g++ -std=c++17 -I../../include -o decrypt_demo decrypt_plugin.cpp -L../../memfabric_hybrid_b200/lib -lmf_core -ldl
#include <cstddef>
#include <cstdio>
#include <cstring>

extern "C" int mf_example_decrypt(const char *cipherText, size_t cipherTextLen, char *plainText, size_t *plainTextLen)
{
    if (cipherText == nullptr || plainText == nullptr || plainTextLen == nullptr || cipherTextLen % 2 != 0 || cipherTextLen / 2 > *plainTextLen) {
        return -1;
    }
    auto nibble = [](char c) -> int {
        if (c >= '0' && c <= '9') return c - '0';
        if (c >= 'a' && c <= 'f') return c - 'a' + 10;
        if (c >= 'A' && c <= 'F') return c - 'A' + 10;
        return -1;
    };
    for (size_t i = 0; i < cipherTextLen; i += 2) {
        const int hi = nibble(cipherText[i]), lo = nibble(cipherText[i + 1]);
        if (hi < 0 || lo < 0) {
            return -1;
        }
        plainText[i / 2] = (char)(hi * 16 + lo);
    }
    *plainTextLen = cipherTextLen / 2;
    return 0;
}

// The by-path contract (mf_tls_config.decrypterLibPath of the BM configuration): capacity by value, NUL-terminated result.
extern "C" int DecryptPassword(const char *cipherText, size_t cipherTextLen, char *plainText, size_t plainTextCapacity)
{
    size_t n = plainTextCapacity;
    if (mf_example_decrypt(cipherText, cipherTextLen, plainText, &n) != 0 || n >= plainTextCapacity) {
        return -1;
    }
    plainText[n] = '\0';
    return 0;
}

#ifndef MF_DECRYPT_PLUGIN_ONLY
#include <dlfcn.h>

#include "mf/mf.h"

int main(int argc, char **argv)
{
    if (argc < 5) {
        std::printf("usage: %s <ca dir> <ca file> <certificate> <key file> <hex pass phrase> [plugin.so]\n", argv[0]);
        return 0;
    }
    mf_decrypt_handler handler = mf_example_decrypt;
    if (argc > 6) {  // the same function, found in a plug-in at run time
        void *lib = dlopen(argv[6], RTLD_NOW);
        handler = lib != nullptr ? reinterpret_cast<mf_decrypt_handler>(dlsym(lib, "mf_example_decrypt")) : nullptr;
        if (handler == nullptr) {
            std::printf("cannot load %s\n", argv[6]);
            return 1;
        }
    }
    char info[1024];
    std::snprintf(info, sizeof(info), "tlsCaPath: %s; tlsCaFile: %s; tlsCert: %s;", argv[1], argv[2], argv[3]);
    const char *pass = argc > 5 ? argv[5] : "";
    if (mf_set_config_store_tls_key(argv[4], (uint32_t)std::strlen(argv[4]), pass, (uint32_t)std::strlen(pass), handler) != 0 ||
        mf_set_conf_store_tls(true, info, (uint32_t)std::strlen(info)) != 0) {
        std::printf("TLS set-up failed: %s\n", mf_get_last_err_msg());
        return 1;
    }
    if (mf_create_config_store("tcp://127.0.0.1:29655") != 0) {
        std::printf("store start failed: %s\n", mf_get_last_err_msg());
        return 1;
    }
    std::printf("config store is serving TLS 1.3 on 127.0.0.1:29655\n");
    mf_destroy_config_store("tcp://127.0.0.1:29655");
    return 0;
}
#endif

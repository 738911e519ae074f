// Path and file checks used wherever the library opens something a user named: certificates and keys of the TLS layer, the
// decrypt plug-in and OpenSSL directories handed to dlopen, the tracer's dump directory. Same job as the reference's
// FileUtil (src/util/csrc/mf_file_util.h:28-133): canonical paths only, no symlinked leaves, regular files with a size cap.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace mf {
namespace util {

constexpr size_t kMaxConfigFileBytes = 10u * 1024 * 1024;  // cap for a certificate / key / CRL / pass-phrase file

// Longest path the library accepts (bounded by the platform's PATH_MAX and 4096).
size_t SafePathMax();
bool Exists(const std::string &path);
bool Readable(const std::string &path);
bool Writable(const std::string &path);
bool IsDir(const std::string &path);
bool IsRegularFile(const std::string &path);  // follows symlinks
bool IsSymlink(const std::string &path);      // the leaf itself is a link
// Size in bytes, or (size_t)-1 if the file cannot be inspected.
size_t FileSize(const std::string &path);
bool IsEmptyFile(const std::string &path);
// Replaces *path by its canonical absolute form. False if it does not exist, is too long or cannot be resolved.
bool Canonicalize(std::string *path);
bool MakeDir(const std::string &path, uint32_t mode);
bool MakeDirs(const std::string &path, uint32_t mode);  // like mkdir -p
bool RemoveFile(const std::string &path);
// Removes a directory tree. Refuses "/", relative paths and anything shallower than two components.
bool RemoveTree(const std::string &path);
// Canonical path of `name` inside `dir` if that is a regular file that really lives under `dir` (no "../" escapes, no
// symlink leading outside). Used before dlopen.
bool ResolveLibrary(const std::string &dir, const std::string &name, std::string *out);

// One-stop check for a file the user configured: non-empty path without NUL or newline, within SafePathMax, exists,
// regular, leaf not a symlink (unless allowSymlink), readable, at most maxBytes. On failure *why says which test failed.
bool CheckConfigFile(const std::string &path, size_t maxBytes, bool allowSymlink, std::string *why);
// Reads a whole checked file. False (and *why) if CheckConfigFile fails or the read is short.
bool ReadConfigFile(const std::string &path, size_t maxBytes, std::string *content, std::string *why);

}  // namespace util
}  // namespace mf

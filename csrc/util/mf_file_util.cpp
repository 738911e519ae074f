#include "mf_file_util.h"

#include <cerrno>
#include <climits>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <dirent.h>
#include <fstream>
#include <sstream>
#include <sys/stat.h>
#include <unistd.h>

namespace mf {
namespace util {

size_t SafePathMax()
{
#ifdef PATH_MAX
    return PATH_MAX < 4096 ? PATH_MAX : 4096;
#else
    return 4096;
#endif
}

static bool SanePathText(const std::string &path)
{
    return !path.empty() && path.size() < SafePathMax() && path.find('\0') == std::string::npos && path.find('\n') == std::string::npos;
}

bool Exists(const std::string &path) { return SanePathText(path) && ::access(path.c_str(), F_OK) == 0; }
bool Readable(const std::string &path) { return SanePathText(path) && ::access(path.c_str(), R_OK) == 0; }
bool Writable(const std::string &path) { return SanePathText(path) && ::access(path.c_str(), W_OK) == 0; }

bool IsDir(const std::string &path)
{
    struct stat st {};
    return SanePathText(path) && ::stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}

bool IsRegularFile(const std::string &path)
{
    struct stat st {};
    return SanePathText(path) && ::stat(path.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

bool IsSymlink(const std::string &path)
{
    struct stat st {};
    return SanePathText(path) && ::lstat(path.c_str(), &st) == 0 && S_ISLNK(st.st_mode);
}

size_t FileSize(const std::string &path)
{
    struct stat st {};
    if (!SanePathText(path) || ::stat(path.c_str(), &st) != 0 || !S_ISREG(st.st_mode)) {
        return (size_t)-1;
    }
    return (size_t)st.st_size;
}

bool IsEmptyFile(const std::string &path) { return FileSize(path) == 0; }

bool Canonicalize(std::string *path)
{
    if (path == nullptr || !SanePathText(*path)) {
        return false;
    }
    char buf[PATH_MAX + 1];
    if (::realpath(path->c_str(), buf) == nullptr) {
        return false;
    }
    std::string out(buf);
    if (out.size() >= SafePathMax()) {
        return false;
    }
    *path = std::move(out);
    return true;
}

bool MakeDir(const std::string &path, uint32_t mode)
{
    if (!SanePathText(path)) {
        return false;
    }
    if (::mkdir(path.c_str(), (mode_t)mode) == 0) {
        return true;
    }
    return errno == EEXIST && IsDir(path);
}

bool MakeDirs(const std::string &path, uint32_t mode)
{
    if (!SanePathText(path)) {
        return false;
    }
    std::string cur;
    size_t pos = 0;
    while (pos <= path.size()) {
        size_t slash = path.find('/', pos);
        if (slash == std::string::npos) {
            slash = path.size();
        }
        cur = path.substr(0, slash);
        if (!cur.empty() && cur != "." && !MakeDir(cur, mode)) {
            return false;
        }
        pos = slash + 1;
    }
    return IsDir(path);
}

bool RemoveFile(const std::string &path)
{
    std::string real = path;
    if (IsSymlink(path)) {
        return ::unlink(path.c_str()) == 0;  // drop the link, never its target
    }
    if (!Canonicalize(&real) || IsDir(real)) {
        return false;
    }
    return ::unlink(real.c_str()) == 0;
}

static bool RemoveTreeAt(const std::string &dir, int depth)
{
    if (depth > 64) {
        return false;
    }
    DIR *d = ::opendir(dir.c_str());
    if (d == nullptr) {
        return false;
    }
    bool ok = true;
    while (struct dirent *e = ::readdir(d)) {
        if (std::strcmp(e->d_name, ".") == 0 || std::strcmp(e->d_name, "..") == 0) {
            continue;
        }
        std::string child = dir + "/" + e->d_name;
        struct stat st {};
        if (::lstat(child.c_str(), &st) != 0) {
            ok = false;
            continue;
        }
        if (S_ISDIR(st.st_mode)) {
            ok = RemoveTreeAt(child, depth + 1) && ok;
        } else {
            ok = ::unlink(child.c_str()) == 0 && ok;  // links are unlinked, not followed
        }
    }
    ::closedir(d);
    return ::rmdir(dir.c_str()) == 0 && ok;
}

bool RemoveTree(const std::string &path)
{
    std::string real = path;
    if (path.empty() || path[0] != '/' || IsSymlink(path) || !Canonicalize(&real) || !IsDir(real)) {
        return false;
    }
    size_t components = 0;
    for (size_t i = 0; i < real.size(); i++) {
        if (real[i] == '/' && i + 1 < real.size()) {
            components++;
        }
    }
    if (components < 2) {
        return false;  // "/" or "/usr": never
    }
    return RemoveTreeAt(real, 0);
}

bool ResolveLibrary(const std::string &dir, const std::string &name, std::string *out)
{
    if (out == nullptr || name.empty() || name.find('/') != std::string::npos || name == "." || name == "..") {
        return false;
    }
    std::string base = dir;
    if (!Canonicalize(&base) || !IsDir(base)) {
        return false;
    }
    std::string full = base + "/" + name;
    if (!Canonicalize(&full) || !IsRegularFile(full)) {
        return false;
    }
    // The canonical file must still sit under the canonical directory (a link may have pointed elsewhere).
    const std::string prefix = base == "/" ? base : base + "/";
    if (full.compare(0, prefix.size(), prefix) != 0) {
        return false;
    }
    *out = std::move(full);
    return true;
}

bool CheckConfigFile(const std::string &path, size_t maxBytes, bool allowSymlink, std::string *why)
{
    auto fail = [&](const char *msg) {
        if (why != nullptr) {
            *why = std::string(msg) + ": " + (path.size() > 256 ? path.substr(0, 256) + "..." : path);
        }
        return false;
    };
    if (!SanePathText(path)) {
        return fail("empty, over-long or malformed path");
    }
    if (!Exists(path)) {
        return fail("no such file");
    }
    if (!allowSymlink && IsSymlink(path)) {
        return fail("symbolic link not accepted");
    }
    if (!IsRegularFile(path)) {
        return fail("not a regular file");
    }
    if (!Readable(path)) {
        return fail("not readable");
    }
    size_t sz = FileSize(path);
    if (sz == (size_t)-1 || sz > maxBytes) {
        return fail("file larger than the accepted maximum");
    }
    return true;
}

bool ReadConfigFile(const std::string &path, size_t maxBytes, std::string *content, std::string *why)
{
    if (content == nullptr || !CheckConfigFile(path, maxBytes, false, why)) {
        return false;
    }
    std::ifstream in(path, std::ios::binary);
    std::ostringstream ss;
    ss << in.rdbuf();
    if (!in.good() && !in.eof()) {
        if (why != nullptr) {
            *why = "read failed: " + path;
        }
        return false;
    }
    *content = ss.str();
    if (content->size() > maxBytes) {
        if (why != nullptr) {
            *why = "file grew past the accepted maximum while being read: " + path;
        }
        content->clear();
        return false;
    }
    return true;
}

}  // namespace util
}  // namespace mf

// Passing file descriptors between unrelated processes on one host.
//
// CUDA POSIX-fd shareable handles and memfd-backed host segments are identified by file descriptors, which the TCP
// config store cannot carry. Each process therefore runs one tiny server on an abstract unix-domain socket; an
// exporter registers (token → fd) and publishes "socket name + token" inside its exchange blob; an importer connects,
// sends the token and receives a duplicate of the descriptor through SCM_RIGHTS. The reference has no such component:
// its driver shares memory by name (IPC memory names / fabric handles, src/hybm/csrc/mm/hybm_vmm_based_segment.cpp:330-380).
#pragma once
#include <atomic>
#include <cstdint>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>

namespace mf {
namespace hybm {

class FdChannel {
public:
    static FdChannel &Instance();
    // Starts the server thread on first use. Returns the abstract socket name (without the leading NUL).
    const std::string &Name();
    // Registers a descriptor (dup'ed internally) and returns its token.
    uint64_t Publish(int fd);
    void Unpublish(uint64_t token);
    // Fetches a duplicate of the descriptor registered under `token` in the process serving `name`. -1 on failure.
    static int Fetch(const std::string &name, uint64_t token, int timeoutMs = 10000);
    // Fetch under the process-wide retry policy (three attempts, 1 s and 2 s apart by default): a peer that is restarting its
    // descriptor server gets the time to come back. -1 when every attempt failed.
    static int FetchWithRetry(const std::string &name, uint64_t token, int timeoutMsPerAttempt = 3000);
    void Shutdown();
    // After fork(): forget the parent's server thread and descriptors.
    void ResetAfterFork();

private:
    FdChannel() = default;
    int Start();
    void Loop();
    std::mutex mu_;
    std::string name_;
    int listenFd_{-1};
    std::thread server_;
    std::atomic<bool> stop_{false};
    std::unordered_map<uint64_t, int> fds_;
    uint64_t nextToken_{1};
};

}  // namespace hybm
}  // namespace mf

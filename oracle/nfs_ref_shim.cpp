// C entry points around the reference's own NFS-store space manager and file helpers
// (ucm/store/nfsstore/cc/domain/space/*.cc, ucm/store/infra/file/*.cc), compiled from the checkout
// where they lie.  Test infrastructure only: it pins the on-disk layout (paths, .act/.dat life
// cycle, file size) and the byte-level read/write of block slices that the CUDA-side store must match.
#include <cstring>
#include <string>
#include <vector>
#include "file/file.h"
#include "logger/logger.h"
#include "space/space_manager.h"

namespace UC::Logger {
// the reference links a spdlog-backed logger; the checker needs none
class NullLogger : public ILogger {
protected:
    void Log(Level&&, SourceLocation&&, std::string&&) override {}
};
ILogger* Make()
{
    static NullLogger logger;
    return &logger;
}
}  // namespace UC::Logger

namespace {
std::vector<std::string> split_backends(const char* s)
{
    std::vector<std::string> out;
    std::string cur;
    for (const char* p = s; *p; ++p) {
        if (*p == ':') {
            if (!cur.empty()) out.push_back(cur);
            cur.clear();
        } else {
            cur.push_back(*p);
        }
    }
    if (!cur.empty()) out.push_back(cur);
    return out;
}
}  // namespace

extern "C" {

void* nfsref_create(const char* backends, size_t block_size, int temp_dir, int* status)
{
    auto* mgr = new UC::SpaceManager();
    auto st = mgr->Setup(split_backends(backends), block_size, temp_dir != 0);
    *status = st.Underlying();
    if (st.Failure()) {
        delete mgr;
        return nullptr;
    }
    return mgr;
}

void nfsref_destroy(void* h) { delete static_cast<UC::SpaceManager*>(h); }

int nfsref_new_block(void* h, const char* id, size_t len)
{
    return static_cast<UC::SpaceManager*>(h)->NewBlock(std::string(id, len)).Underlying();
}

int nfsref_commit_block(void* h, const char* id, size_t len, int success)
{
    return static_cast<UC::SpaceManager*>(h)->CommitBlock(std::string(id, len), success != 0).Underlying();
}

int nfsref_lookup_block(void* h, const char* id, size_t len)
{
    return static_cast<UC::SpaceManager*>(h)->LookupBlock(std::string(id, len)) ? 1 : 0;
}

int nfsref_data_path(void* h, const char* id, size_t len, int activated, char* out, size_t cap)
{
    auto path = static_cast<UC::SpaceManager*>(h)->GetSpaceLayout()->DataFilePath(std::string(id, len), activated != 0);
    if (path.size() + 1 > cap) return -1;
    std::memcpy(out, path.c_str(), path.size() + 1);
    return (int)path.size();
}

int nfsref_write(const char* path, size_t offset, size_t length, const void* src, int direct)
{
    return UC::File::Write(path, offset, length, (uintptr_t)src, direct != 0).Underlying();
}

int nfsref_read(const char* path, size_t offset, size_t length, void* dst, int direct)
{
    return UC::File::Read(path, offset, length, (uintptr_t)dst, direct != 0).Underlying();
}

}  // extern "C"

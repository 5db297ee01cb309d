// File-per-block store data plane: the step after the pinned ring.  One file per KV block under
// <backend>/data/<first 8 id bytes as hex>/<next 8 id bytes as hex>.dat, written as ".act" until the
// block is committed (or under <backend>/temp/... when the temporary dump directory is enabled),
// created at the fixed block size; a task is a list of (block id, byte offset in the file, address,
// length) slices to dump or load.  The layout and life cycle follow the reference's NFS store
// (ucm/store/nfsstore/cc/domain/space/space_shard_layout.cc:51-126, space_shard_temp_layout.cc:29-54,
// space_manager.cc:40-139, task handling in ucm/store/task/task_manager.cc:28-104 and
// task_shard.h:88-114, the per-slice work in nfsstore/cc/domain/trans/posix_queue.cc:66-138).
//
// What differs is the device leg.  The reference copies one slice at a time (a blocking copy for
// dumps, one asynchronous copy per slice for loads) on 32 threads, each owning 128 MiB of pinned
// buffers.  Here every worker thread owns a small, double-buffered group of page-locked, device-mapped
// slots: a group of slices is read from disk into one half (O_DIRECT when the slice is 4 KiB
// aligned) while the previous half is still being pulled into HBM, and each group crosses PCIe in a
// single kernel launch that scatters all of its slices (ucmx_copy_batch), not one copy per slice.
// File descriptors are kept across consecutive slices of the same block (a block's 64 K/V layer
// slices share one file).
#include <fcntl.h>
#include <sys/stat.h>
#include <sys/types.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"

namespace {

constexpr size_t kIdBytes = 16;       // the part of a block id that names its file
constexpr size_t kDirectAlign = 4096;  // O_DIRECT granularity assumed by the reference as well

struct Slice {
    std::string block;
    size_t offset;
    uintptr_t address;
    size_t length;
};

struct TaskState {
    std::mutex mu;
    std::condition_variable cv;
    size_t remaining = 0;  // parts not yet finished
    std::atomic<bool> failed{false};
};

struct WorkItem {
    std::shared_ptr<TaskState> task;
    int type;      // UCMX_FSTORE_DUMP / UCMX_FSTORE_LOAD
    int location;  // UCMX_FSTORE_HOST / UCMX_FSTORE_DEVICE
    std::vector<Slice> slices;
};

struct Worker {
    std::thread thread;
    std::mutex mu;
    std::condition_variable cv;
    std::deque<WorkItem> queue;
    bool stop = false;
};

// one slice, or one io_size piece of a longer slice, staged in a slot
struct Piece {
    uintptr_t device;
    size_t file_offset;
    size_t length;
    int fd;
};

}  // namespace

struct ucmx_fstore {
    std::vector<std::string> backends;
    size_t block_size = 0;
    bool temp_dir = false;
    bool transfer = false;
    int device = -1;
    size_t io_size = 262144;
    size_t slots_per_worker = 16;
    size_t timeout_ms = 30000;
    std::vector<std::unique_ptr<Worker>> workers;
    std::mutex mu;  // tasks, next_worker
    std::map<size_t, std::shared_ptr<TaskState>> tasks;
    size_t next_worker = 0;
    std::atomic<int> worker_init_failures{0};

    // ------------------------------------------------------------------ layout
    std::string backend_of(const std::string& id) const
    {
        return backends[std::hash<std::string>{}(id) % backends.size()];
    }
    static void split_id(const std::string& id, uint64_t& front, uint64_t& back)
    {
        std::memcpy(&front, id.data(), 8);
        std::memcpy(&back, id.data() + 8, 8);
    }
    std::string parent(const std::string& id, bool activated) const
    {
        uint64_t front, back;
        split_id(id, front, back);
        char buf[40];
        snprintf(buf, sizeof(buf), "%s/%016llx", (activated && temp_dir) ? "temp" : "data", (unsigned long long)front);
        return backend_of(id) + buf;
    }
    std::string path(const std::string& id, bool activated) const
    {
        uint64_t front, back;
        split_id(id, front, back);
        char buf[40];
        snprintf(buf, sizeof(buf), "/%016llx.%s", (unsigned long long)back, (activated && !temp_dir) ? "act" : "dat");
        return parent(id, activated) + buf;
    }
};

namespace {

constexpr mode_t kDirMode = S_IRUSR | S_IWUSR | S_IXUSR | S_IRGRP | S_IROTH;
constexpr mode_t kFileMode = S_IRWXU | S_IRGRP | S_IXGRP | S_IROTH | S_IXOTH;

int32_t make_dir(const std::string& p)
{
    if (mkdir(p.c_str(), kDirMode) == 0) return UCMX_OK;
    return errno == EEXIST ? UCMX_EDUPLICATE : UCMX_EOSERROR;
}

bool aligned(size_t v) { return (v & (kDirectAlign - 1)) == 0; }

// open for slice I/O; direct I/O is tried when asked and quietly dropped where the file system
// refuses it (tmpfs, some overlay mounts)
int open_data(const std::string& p, bool write, bool direct)
{
    const int base = write ? O_WRONLY : O_RDONLY;
    if (direct) {
        const int fd = open(p.c_str(), base | O_DIRECT);
        if (fd >= 0 || errno != EINVAL) return fd;
    }
    return open(p.c_str(), base);
}

bool full_pread(int fd, void* buf, size_t n, size_t off)
{
    return pread(fd, buf, n, (off_t)off) == (ssize_t)n;   // a short read is a failure, as in the reference
}
bool full_pwrite(int fd, const void* buf, size_t n, size_t off)
{
    return pwrite(fd, buf, n, (off_t)off) == (ssize_t)n;
}

// keeps the last file open while consecutive slices name the same block
struct FdCache {
    std::string block;
    int fd = -1;
    bool direct = false;
    int get(const ucmx_fstore* s, const std::string& id, bool write, bool want_direct)
    {
        if (fd >= 0 && block == id && direct == want_direct) return fd;
        drop();
        fd = open_data(s->path(id, /*activated=*/write), write, want_direct);
        block = id;
        direct = want_direct;
        return fd;
    }
    void drop()
    {
        if (fd >= 0) close(fd);
        fd = -1;
    }
    ~FdCache() { drop(); }
};

// Per-thread staging: 2 halves of `half` slots each, io_size bytes per slot, plus pointer tables the
// copy kernel reads (all page-locked and mapped, so device and host use the same addresses).
struct Staging {
    unsigned char* slab = nullptr;
    void** dst_tab = nullptr;
    void** src_tab = nullptr;
    cudaStream_t stream = nullptr;
    cudaEvent_t done[2] = {nullptr, nullptr};
    bool busy[2] = {false, false};
    size_t half = 0, io = 0;
    bool init(int device, size_t slots, size_t io_size)
    {
        if (cudaSetDevice(device) != cudaSuccess) return false;
        half = std::max<size_t>(slots / 2, 1);
        io = io_size;
        if (cudaHostAlloc((void**)&slab, 2 * half * io, cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) return false;
        if (cudaHostAlloc((void**)&dst_tab, 2 * half * sizeof(void*), cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) return false;
        if (cudaHostAlloc((void**)&src_tab, 2 * half * sizeof(void*), cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) return false;
        if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) return false;
        for (auto& e : done)
            if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return false;
        return true;
    }
    unsigned char* slot(int h, size_t j) const { return slab + ((size_t)h * half + j) * io; }
    bool wait_half(int h)
    {
        if (!busy[h]) return true;
        busy[h] = false;
        return cudaEventSynchronize(done[h]) == cudaSuccess;
    }
    // move the staged pieces of half h between their slots and their device addresses: one launch per
    // run of equal lengths (normally the whole group); odd sizes fall back to single copies
    bool launch(int h, const std::vector<Piece>& pieces, bool to_device)
    {
        size_t i = 0;
        while (i < pieces.size()) {
            size_t j = i + 1;
            while (j < pieces.size() && pieces[j].length == pieces[i].length) ++j;
            const size_t len = pieces[i].length;
            bool batch = (len & 15) == 0;
            for (size_t k = i; k < j && batch; ++k) batch = (pieces[k].device & 15) == 0;
            if (batch) {
                for (size_t k = i; k < j; ++k) {
                    void* host = slot(h, k);
                    void* dev = (void*)pieces[k].device;
                    dst_tab[h * half + k] = to_device ? dev : host;
                    src_tab[h * half + k] = to_device ? host : dev;
                }
                if (ucmx_copy_batch(dst_tab + h * half + i, (const void* const*)(src_tab + h * half + i), (int32_t)(j - i),
                                    (int64_t)len, /*any_host_memory=*/1, stream) != UCMX_OK)
                    return false;
            } else {
                for (size_t k = i; k < j; ++k) {
                    void* host = slot(h, k);
                    void* dev = (void*)pieces[k].device;
                    if (cudaMemcpyAsync(to_device ? dev : host, to_device ? host : dev, len, cudaMemcpyDefault, stream) != cudaSuccess)
                        return false;
                }
            }
            i = j;
        }
        busy[h] = true;
        return cudaEventRecord(done[h], stream) == cudaSuccess;
    }
    void destroy()
    {
        if (stream) cudaStreamSynchronize(stream);
        for (auto& e : done)
            if (e) cudaEventDestroy(e);
        if (stream) cudaStreamDestroy(stream);
        if (slab) cudaFreeHost(slab);
        if (dst_tab) cudaFreeHost(dst_tab);
        if (src_tab) cudaFreeHost(src_tab);
    }
};

bool run_host(const ucmx_fstore* s, const WorkItem& w)
{
    FdCache files;
    const bool write = w.type == UCMX_FSTORE_DUMP;
    for (const Slice& sl : w.slices) {
        if (w.task->failed.load(std::memory_order_relaxed)) return false;
        const bool direct = aligned(sl.offset) && aligned(sl.length) && aligned((size_t)sl.address);
        const int fd = files.get(s, sl.block, write, direct);
        if (fd < 0) return false;
        const bool ok = write ? full_pwrite(fd, (const void*)sl.address, sl.length, sl.offset)
                              : full_pread(fd, (void*)sl.address, sl.length, sl.offset);
        if (!ok) return false;
    }
    return true;
}

bool run_device(const ucmx_fstore* s, const WorkItem& w, Staging& st)
{
    FdCache files;
    const bool dump = w.type == UCMX_FSTORE_DUMP;
    // cut slices into pieces of at most one slot
    std::vector<std::pair<size_t, Piece>> all;  // slice index, piece
    for (size_t i = 0; i < w.slices.size(); ++i) {
        const Slice& sl = w.slices[i];
        for (size_t done = 0; done < sl.length; done += st.io)
            all.push_back({i, Piece{sl.address + done, sl.offset + done, std::min(st.io, sl.length - done), -1}});
    }
    bool ok = true;
    int h = 0;
    std::vector<Piece> group[2];
    std::vector<size_t> owner[2];
    auto write_half = [&](int hh) {   // dump: the pieces of half hh have reached their slots; write them out
        if (!st.wait_half(hh)) return false;
        for (size_t k = 0; k < group[hh].size(); ++k) {
            const Piece& p = group[hh][k];
            const Slice& sl = w.slices[owner[hh][k]];
            const bool direct = aligned(p.file_offset) && aligned(p.length) && aligned((size_t)st.slot(hh, k));
            const int fd = files.get(s, sl.block, true, direct);
            if (fd < 0 || !full_pwrite(fd, st.slot(hh, k), p.length, p.file_offset)) return false;
        }
        group[hh].clear();
        owner[hh].clear();
        return true;
    };
    for (size_t pos = 0; pos < all.size() && ok; pos += st.half, h ^= 1) {
        if (w.task->failed.load(std::memory_order_relaxed)) {
            ok = false;
            break;
        }
        const size_t end = std::min(all.size(), pos + st.half);
        if (dump) {
            // start pulling this group out of HBM, then write the previous group while it flies
            if (!group[h].empty() && !write_half(h)) { ok = false; break; }
            for (size_t k = pos; k < end; ++k) {
                group[h].push_back(all[k].second);
                owner[h].push_back(all[k].first);
            }
            if (!st.launch(h, group[h], /*to_device=*/false)) { ok = false; break; }
            if (!group[h ^ 1].empty() && !write_half(h ^ 1)) { ok = false; break; }
        } else {
            // the slots of this half may still be feeding the previous launch that used them
            if (!st.wait_half(h)) { ok = false; break; }
            group[h].clear();
            for (size_t k = pos; k < end && ok; ++k) {
                const Piece& p = all[k].second;
                const Slice& sl = w.slices[all[k].first];
                const bool direct = aligned(p.file_offset) && aligned(p.length) && aligned((size_t)st.slot(h, k - pos));
                const int fd = files.get(s, sl.block, false, direct);
                ok = fd >= 0 && full_pread(fd, st.slot(h, k - pos), p.length, p.file_offset);
                group[h].push_back(p);
            }
            if (ok) ok = st.launch(h, group[h], /*to_device=*/true);
        }
    }
    if (dump) {
        for (int hh = 0; hh < 2; ++hh) {
            const int q = h ^ hh;  // older half first
            if (!group[q].empty()) {
                if (ok) ok = write_half(q);
                else st.wait_half(q);
            }
        }
    }
    // nothing of this part may still be in flight when it is reported finished
    if (!st.wait_half(0)) ok = false;
    if (!st.wait_half(1)) ok = false;
    return ok;
}

void finish_part(const WorkItem& w, bool ok)
{
    if (!ok) w.task->failed.store(true);
    std::lock_guard<std::mutex> lk(w.task->mu);
    if (--w.task->remaining == 0) w.task->cv.notify_all();
}

void worker_main(ucmx_fstore* s, Worker* me)
{
    Staging st;
    bool have_device = false;
    if (s->device >= 0) {
        have_device = st.init(s->device, s->slots_per_worker, s->io_size);
        if (!have_device) {
            cudaGetLastError();
            s->worker_init_failures.fetch_add(1);
        }
    }
    for (;;) {
        WorkItem w;
        {
            std::unique_lock<std::mutex> lk(me->mu);
            me->cv.wait(lk, [&] { return me->stop || !me->queue.empty(); });
            if (me->queue.empty()) break;  // stop requested and nothing left
            w = std::move(me->queue.front());
            me->queue.pop_front();
        }
        bool ok;
        if (w.task->failed.load()) ok = false;   // an earlier part failed or the task timed out: skip the work
        else if (w.location == UCMX_FSTORE_HOST) ok = run_host(s, w);
        else ok = have_device && run_device(s, w, st);
        finish_part(w, ok);
    }
    if (s->device >= 0) st.destroy();
}

std::vector<std::string> split_backends(const char* text)
{
    std::vector<std::string> out;
    std::string cur;
    for (const char* p = text; ; ++p) {
        if (*p == ':' || *p == 0) {
            if (!cur.empty()) {
                if (cur.back() != '/') cur.push_back('/');
                if (std::find(out.begin(), out.end(), cur) == out.end()) out.push_back(cur);
            }
            cur.clear();
            if (*p == 0) break;
        } else {
            cur.push_back(*p);
        }
    }
    return out;
}

std::atomic<size_t> g_next_task{1};  // 0 is the invalid task id, as in the reference

}  // namespace

extern "C" int32_t ucmx_fstore_create(const char* backends, size_t block_size, int32_t temp_dump_dir,
                                      int32_t transfer_enable, int32_t device_id, size_t io_size,
                                      size_t slots_per_worker, size_t worker_number, size_t timeout_ms,
                                      ucmx_fstore** out)
{
    if (!out || !backends || block_size == 0) return UCMX_EPARAM;
    auto list = split_backends(backends);
    if (list.empty()) return UCMX_EPARAM;
    auto s = std::unique_ptr<ucmx_fstore>(new (std::nothrow) ucmx_fstore());
    if (!s) return UCMX_EOOM;
    s->block_size = block_size;
    s->temp_dir = temp_dump_dir != 0;
    // the first backend gets its roots created; the others must already hold them (shared storage)
    std::vector<std::string> roots = {"data"};
    if (s->temp_dir) roots.push_back("temp");
    for (size_t i = 0; i < list.size(); ++i) {
        for (const auto& root : roots) {
            const std::string p = list[i] + root;
            if (i == 0) {
                const int32_t st = make_dir(p);
                if (st != UCMX_OK && st != UCMX_EDUPLICATE) {
                    ucmx::set_last_text(("cannot create " + p).c_str());
                    return st;
                }
            } else if (access(p.c_str(), R_OK | W_OK) != 0) {
                ucmx::set_last_text(("cannot access " + p).c_str());
                return UCMX_EPARAM;
            }
        }
        s->backends.push_back(list[i]);
    }
    s->transfer = transfer_enable != 0;
    if (s->transfer) {
        if (io_size == 0 || (io_size & 15)) return UCMX_EPARAM;
        s->device = device_id;
        s->io_size = io_size;
        s->slots_per_worker = std::max<size_t>(slots_per_worker ? slots_per_worker : 16, 2);
        s->timeout_ms = timeout_ms ? timeout_ms : 30000;
        const size_t n = worker_number ? worker_number : 8;
        for (size_t i = 0; i < n; ++i) {
            s->workers.emplace_back(new Worker());
            Worker* w = s->workers.back().get();
            w->thread = std::thread(worker_main, s.get(), w);
        }
    }
    *out = s.release();
    return UCMX_OK;
}

extern "C" int32_t ucmx_fstore_destroy(ucmx_fstore* s)
{
    if (!s) return UCMX_OK;
    for (auto& w : s->workers) {
        {
            std::lock_guard<std::mutex> lk(w->mu);
            w->stop = true;
        }
        w->cv.notify_all();
    }
    for (auto& w : s->workers)
        if (w->thread.joinable()) w->thread.join();
    delete s;
    return UCMX_OK;
}

extern "C" int32_t ucmx_fstore_path(const ucmx_fstore* s, const char* id, size_t id_len, int32_t activated,
                                    char* out, size_t capacity)
{
    if (!s || !id || id_len < kIdBytes || !out) return UCMX_EPARAM;
    const std::string p = s->path(std::string(id, id_len), activated != 0);
    if (p.size() + 1 > capacity) return UCMX_EPARAM;
    std::memcpy(out, p.c_str(), p.size() + 1);
    return UCMX_OK;
}

extern "C" int32_t ucmx_fstore_alloc(ucmx_fstore* s, const char* id, size_t id_len)
{
    if (!s || !id || id_len < kIdBytes) return UCMX_EPARAM;
    const std::string block(id, id_len);
    int32_t st = make_dir(s->parent(block, true));
    if (st != UCMX_OK && st != UCMX_EDUPLICATE) return st;
    if (access(s->path(block, false).c_str(), F_OK) == 0) return UCMX_EDUPLICATE;   // already committed
    const int fd = open(s->path(block, true).c_str(), O_CREAT | O_EXCL | O_RDWR, kFileMode);
    if (fd < 0) return errno == EEXIST ? UCMX_EDUPLICATE : UCMX_EOSERROR;          // someone else is writing it
    st = ftruncate(fd, (off_t)s->block_size) == 0 ? UCMX_OK : UCMX_EOSERROR;
    close(fd);
    return st;
}

extern "C" int32_t ucmx_fstore_lookup(const ucmx_fstore* s, const char* id, size_t id_len, int32_t* found)
{
    if (!s || !id || id_len < kIdBytes || !found) return UCMX_EPARAM;
    *found = access(s->path(std::string(id, id_len), false).c_str(), F_OK | R_OK | W_OK) == 0 ? 1 : 0;
    return UCMX_OK;
}

extern "C" int32_t ucmx_fstore_commit(ucmx_fstore* s, const char* id, size_t id_len, int32_t success)
{
    if (!s || !id || id_len < kIdBytes) return UCMX_EPARAM;
    const std::string block(id, id_len);
    const std::string act_parent = s->parent(block, true), act_file = s->path(block, true);
    const std::string dat_parent = s->parent(block, false);
    int32_t st = UCMX_OK;
    if (success) {
        if (dat_parent != act_parent) {
            st = make_dir(dat_parent);
            if (st == UCMX_EDUPLICATE) st = UCMX_OK;
        }
        if (st == UCMX_OK && rename(act_file.c_str(), s->path(block, false).c_str()) != 0)
            st = errno == ENOENT ? UCMX_ENOOBJ : UCMX_EOSERROR;
    }
    remove(act_file.c_str());   // a cancelled or half-renamed block leaves nothing behind
    if (!success || dat_parent != act_parent) rmdir(act_parent.c_str());   // fails harmlessly while siblings remain
    return st;
}

extern "C" int32_t ucmx_fstore_submit(ucmx_fstore* s, int32_t type, int32_t location, const char* const* ids,
                                      const size_t* id_lens, const size_t* offsets, const uintptr_t* addresses,
                                      const size_t* lengths, size_t n, size_t* task_id)
{
    if (task_id) *task_id = 0;
    if (!s || !task_id || !ids || !id_lens || !offsets || !addresses || !lengths || n == 0) return UCMX_EPARAM;
    if ((type != UCMX_FSTORE_DUMP && type != UCMX_FSTORE_LOAD) || (location != UCMX_FSTORE_HOST && location != UCMX_FSTORE_DEVICE))
        return UCMX_EPARAM;
    if (!s->transfer || s->workers.empty()) {
        ucmx::set_last_text("the store was created without transfer workers");
        return UCMX_EUNSUPPORTED;
    }
    if (location == UCMX_FSTORE_DEVICE && s->device < 0) return UCMX_EPARAM;
    for (size_t i = 0; i < n; ++i)
        if (!ids[i] || id_lens[i] < kIdBytes) return UCMX_EPARAM;
    auto task = std::make_shared<TaskState>();
    // contiguous runs of slices per worker, as even as possible (a block's slices stay together)
    const size_t parts = std::min(n, s->workers.size());
    task->remaining = parts;
    const size_t id = g_next_task.fetch_add(1, std::memory_order_relaxed);
    std::lock_guard<std::mutex> lk(s->mu);
    s->tasks.emplace(id, task);
    const size_t base = n / parts, rem = n % parts;
    size_t pos = 0;
    for (size_t p = 0; p < parts; ++p) {
        const size_t cnt = base + (p < rem ? 1 : 0);
        WorkItem w;
        w.task = task;
        w.type = type;
        w.location = location;
        w.slices.reserve(cnt);
        for (size_t i = pos; i < pos + cnt; ++i)
            w.slices.push_back(Slice{std::string(ids[i], id_lens[i]), offsets[i], addresses[i], lengths[i]});
        pos += cnt;
        Worker* wk = s->workers[s->next_worker].get();
        s->next_worker = (s->next_worker + 1) % s->workers.size();
        {
            std::lock_guard<std::mutex> wl(wk->mu);
            wk->queue.push_back(std::move(w));
        }
        wk->cv.notify_one();
    }
    *task_id = id;
    return UCMX_OK;
}

extern "C" int32_t ucmx_fstore_wait(ucmx_fstore* s, size_t task_id)
{
    if (!s) return UCMX_EPARAM;
    std::shared_ptr<TaskState> task;
    {
        std::lock_guard<std::mutex> lk(s->mu);
        auto it = s->tasks.find(task_id);
        if (it == s->tasks.end()) return UCMX_ENOOBJ;
        task = it->second;
        s->tasks.erase(it);
    }
    std::unique_lock<std::mutex> lk(task->mu);
    if (!task->cv.wait_for(lk, std::chrono::milliseconds(s->timeout_ms), [&] { return task->remaining == 0; })) {
        // too slow: mark it failed so that workers skip what is left, then let them drain - the caller's
        // buffers must not be touched after this returns
        task->failed.store(true);
        task->cv.wait(lk, [&] { return task->remaining == 0; });
    }
    return task->failed.load() ? UCMX_ERROR : UCMX_OK;
}

extern "C" int32_t ucmx_fstore_check(ucmx_fstore* s, size_t task_id, int32_t* finished)
{
    if (!s || !finished) return UCMX_EPARAM;
    std::shared_ptr<TaskState> task;
    {
        std::lock_guard<std::mutex> lk(s->mu);
        auto it = s->tasks.find(task_id);
        if (it == s->tasks.end()) return UCMX_ENOOBJ;
        task = it->second;
    }
    std::lock_guard<std::mutex> lk(task->mu);
    *finished = task->remaining == 0 ? 1 : 0;
    return UCMX_OK;
}

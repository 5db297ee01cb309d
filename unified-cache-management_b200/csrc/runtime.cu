// Host-side runtime above the kernels: the pinned host ring, event-backed transfer tasks and the
// device-resident retrieval back-end object.  These replace the reference's thread pools and
// condition variables (ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp, ucm/store/task/*,
// ucm/store/device/ibuffered_device.h) with CUDA streams and events: submitting work enqueues
// kernels, polling is an event query, waiting is a bounded event wait.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <mutex>
#include <new>
#include <thread>
#include <atomic>
#include <optional>
#include <unordered_map>
#include <vector>

#include "common.cuh"

// ------------------------------------------------------------------ pinned ring

struct ucmx_ring {
    unsigned char* base = nullptr;
    size_t slot_bytes = 0, n_slots = 0;
    std::mutex mu;
    std::vector<int32_t> free_list;
    std::vector<uint8_t> in_use;
};

extern "C" int32_t ucmx_ring_create(size_t slot_bytes, size_t n_slots, ucmx_ring** out)
{
    if (!out || slot_bytes == 0 || n_slots == 0 || (slot_bytes & 15) || n_slots > (1u << 30)) return UCMX_EPARAM;
    ucmx_ring* r = new (std::nothrow) ucmx_ring();
    if (!r) return UCMX_EOOM;
    void* p = nullptr;
    cudaError_t e = cudaHostAlloc(&p, slot_bytes * n_slots, cudaHostAllocPortable | cudaHostAllocMapped);
    if (e != cudaSuccess) {
        delete r;
        ucmx::cuda_status("cudaHostAlloc(ring)", e);
        return UCMX_EOOM;
    }
    r->base = (unsigned char*)p;
    r->slot_bytes = slot_bytes;
    r->n_slots = n_slots;
    r->in_use.assign(n_slots, 0);
    r->free_list.reserve(n_slots);
    for (size_t i = n_slots; i > 0; --i) r->free_list.push_back((int32_t)(i - 1));
    *out = r;
    return UCMX_OK;
}

extern "C" int32_t ucmx_ring_acquire(ucmx_ring* r, void** host_ptr, int32_t* slot_index)
{
    if (!r || !host_ptr || !slot_index) return UCMX_EPARAM;
    std::lock_guard<std::mutex> lk(r->mu);
    if (r->free_list.empty()) return UCMX_ENOOBJ;
    const int32_t idx = r->free_list.back();
    r->free_list.pop_back();
    r->in_use[idx] = 1;
    *host_ptr = r->base + (size_t)idx * r->slot_bytes;
    *slot_index = idx;
    return UCMX_OK;
}

extern "C" int32_t ucmx_ring_release(ucmx_ring* r, int32_t slot_index)
{
    if (!r || slot_index < 0 || (size_t)slot_index >= r->n_slots) return UCMX_EPARAM;
    std::lock_guard<std::mutex> lk(r->mu);
    if (!r->in_use[slot_index]) return UCMX_ENOOBJ;
    r->in_use[slot_index] = 0;
    r->free_list.push_back(slot_index);
    return UCMX_OK;
}

extern "C" int32_t ucmx_ring_base(ucmx_ring* r, void** host_ptr, size_t* slot_bytes, size_t* n_slots)
{
    if (!r) return UCMX_EPARAM;
    if (host_ptr) *host_ptr = r->base;
    if (slot_bytes) *slot_bytes = r->slot_bytes;
    if (n_slots) *n_slots = r->n_slots;
    return UCMX_OK;
}

extern "C" int32_t ucmx_ring_destroy(ucmx_ring* r)
{
    if (!r) return UCMX_EPARAM;
    if (r->base) cudaFreeHost(r->base);
    delete r;
    return UCMX_OK;
}

// ------------------------------------------------------------------ tasks

struct ucmx_task {
    cudaEvent_t ev = nullptr;
    bool recorded = false;
    bool failed = false;
};

extern "C" int32_t ucmx_task_create(ucmx_task** out)
{
    if (!out) return UCMX_EPARAM;
    ucmx_task* t = new (std::nothrow) ucmx_task();
    if (!t) return UCMX_EOOM;
    cudaError_t e = cudaEventCreateWithFlags(&t->ev, cudaEventDisableTiming);
    if (e != cudaSuccess) {
        delete t;
        return ucmx::cuda_status("cudaEventCreate", e);
    }
    *out = t;
    return UCMX_OK;
}

extern "C" int32_t ucmx_task_record(ucmx_task* t, ucmx_stream_t stream)
{
    if (!t) return UCMX_EPARAM;
    cudaError_t e = cudaEventRecord(t->ev, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        t->failed = true;
        return ucmx::cuda_status("cudaEventRecord", e);
    }
    t->recorded = true;
    return UCMX_OK;
}

extern "C" int32_t ucmx_task_check(ucmx_task* t, int32_t* finished)
{
    if (!t || !finished) return UCMX_EPARAM;
    *finished = 0;
    if (t->failed) {
        *finished = 1;
        return UCMX_ERROR;
    }
    if (!t->recorded) {
        *finished = 1;  // nothing was enqueued: trivially complete
        return UCMX_OK;
    }
    cudaError_t e = cudaEventQuery(t->ev);
    if (e == cudaSuccess) {
        *finished = 1;
        return UCMX_OK;
    }
    if (e == cudaErrorNotReady) {
        cudaGetLastError();
        return UCMX_OK;
    }
    t->failed = true;
    *finished = 1;
    ucmx::cuda_status("cudaEventQuery", e);
    return UCMX_ERROR;
}

extern "C" int32_t ucmx_task_wait(ucmx_task* t, int64_t timeout_ms)
{
    if (!t) return UCMX_EPARAM;
    if (t->failed) return UCMX_ERROR;
    if (!t->recorded) return UCMX_OK;
    if (timeout_ms < 0) {
        cudaError_t e = cudaEventSynchronize(t->ev);
        if (e != cudaSuccess) {
            t->failed = true;
            ucmx::cuda_status("cudaEventSynchronize", e);
            return UCMX_ERROR;
        }
        return UCMX_OK;
    }
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    int spins = 0;
    for (;;) {
        int32_t fin = 0;
        const int32_t rc = ucmx_task_check(t, &fin);
        if (rc != UCMX_OK) return UCMX_ERROR;
        if (fin) return UCMX_OK;
        if (std::chrono::steady_clock::now() >= deadline) return UCMX_ERROR;  // timed out; task stays pending
        if (++spins > 200) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

extern "C" int32_t ucmx_task_destroy(ucmx_task* t)
{
    if (!t) return UCMX_EPARAM;
    if (t->ev) cudaEventDestroy(t->ev);
    delete t;
    return UCMX_OK;
}

// ------------------------------------------------------------------ retrieval back-end

namespace ucmx {
namespace {

__global__ void f32_to_bf16_rows_kernel(const float* __restrict__ src, const int32_t* __restrict__ slots, int64_t n_rows,
                                        int32_t dim, uint16_t* __restrict__ dst_bf16, float* __restrict__ dst_f32)
{
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * dim) return;
    const int64_t row = idx / dim;
    const int32_t d = (int32_t)(idx - row * dim);
    const int64_t slot = slots ? (int64_t)slots[row] : row;
    if (slot < 0) return;
    const float v = src[idx];
    if (dst_bf16) dst_bf16[slot * dim + d] = (uint16_t)f32_to_bf16_bits(v);
    if (dst_f32) dst_f32[slot * dim + d] = v;
}

// Page-locked host memory that grows by doubling (contents kept).
struct PinnedBuf {
    unsigned char* p = nullptr;
    size_t size = 0, cap = 0;
    int32_t reserve(size_t want)
    {
        if (want <= cap) return UCMX_OK;
        size_t ncap = cap ? cap : (size_t)64 << 10;
        while (ncap < want) ncap *= 2;
        unsigned char* np = nullptr;
        UCMX_CUDA(cudaHostAlloc((void**)&np, ncap, cudaHostAllocPortable | cudaHostAllocMapped));   // (kernels of any device may write into it)
        if (p) {
            memcpy(np, p, size);
            cudaFreeHost(p);
        }
        p = np;
        cap = ncap;
        return UCMX_OK;
    }
    int32_t append(const void* src, size_t bytes)
    {
        const int32_t rc = reserve(size + bytes);
        if (rc != UCMX_OK) return rc;
        memcpy(p + size, src, bytes);
        size += bytes;
        return UCMX_OK;
    }
    void release()
    {
        if (p) cudaFreeHost(p);
        p = nullptr;
        size = cap = 0;
    }
};

// A batch is what goes to the GPU in one piece: the query rows and candidate lists of every submit that
// arrived since the last launch.  One ragged score + top-k serves them all.
struct Batch {
    PinnedBuf h_q, h_idx, h_out;
    std::vector<int32_t> off{0}, kk, ooff{0};   // CSR of candidates, k per row, CSR of outputs
    unsigned char* d_buf = nullptr;
    size_t d_cap = 0;
    cudaEvent_t done = nullptr;
    int32_t open = 0;          // requests whose result has not been collected yet
    int32_t kmax = 1;
    bool launched = false, failed = false;
    std::atomic<bool> finished{false};   // the batch's event has been seen complete: no more driver calls for its requests
    size_t o_counts = 0, o_idx = 0;   // byte offsets inside h_out once launched
    void reset()
    {
        h_q.size = h_idx.size = h_out.size = 0;
        off.assign(1, 0);
        kk.clear();
        ooff.assign(1, 0);
        open = 0;
        kmax = 1;
        launched = failed = false;
        finished.store(false, std::memory_order_relaxed);
    }
};

struct Request {
    Batch* batch = nullptr;
    int32_t row0 = 0, rows = 0, k = 0;
};

// The requests that have been submitted and not collected yet, by request id.  Ids are handed out in sequence and
// collected soon after, so a request lives in the slot its id's low bits name (no allocation per request, which is
// what a node-based map costs on each submit and each get_result); an id whose slot is still taken by a request
// from kLiveSlots ids ago goes to a map instead.
constexpr int32_t kLiveSlots = 1 << 14;
struct LiveTable {
    struct Slot {
        int32_t id = -1;
        Request rq;
    };
    std::vector<Slot> slots{(size_t)kLiveSlots};
    std::unordered_map<int32_t, Request> spill;

    Request* find(int32_t id)
    {
        if (id < 0) return nullptr;
        Slot& s = slots[(size_t)(id & (kLiveSlots - 1))];
        if (s.id == id) return &s.rq;
        if (spill.empty()) return nullptr;
        auto it = spill.find(id);
        return it == spill.end() ? nullptr : &it->second;
    }
    void insert(int32_t id, const Request& rq)
    {
        Slot& s = slots[(size_t)(id & (kLiveSlots - 1))];
        if (s.id < 0) {
            s.id = id;
            s.rq = rq;
        } else {
            spill[id] = rq;
        }
    }
    void erase(int32_t id)
    {
        Slot& s = slots[(size_t)(id & (kLiveSlots - 1))];
        if (s.id == id) s.id = -1;
        else spill.erase(id);
    }
    template <typename F>
    void for_each(F&& f)
    {
        for (Slot& s : slots)
            if (s.id >= 0) f(s.rq);
        for (auto& kv : spill) f(kv.second);
    }
};

}  // namespace
}  // namespace ucmx

struct ucmx_retrieval {
    int device = 0;
    int64_t n_items = 0;
    int32_t dim = 0;
    int32_t dtype = UCMX_DT_BF16;
    void* table = nullptr;
    cudaStream_t stream = nullptr;
    std::mutex mu;
    int32_t next_id = 0;
    int64_t launches = 0;
    ucmx::LiveTable live;
    ucmx::Batch* building = nullptr;
    std::vector<ucmx::Batch*> pool;
};

namespace ucmx {
namespace {

struct DeviceGuard {
    int prev = -1;
    bool ok = true, changed = false;
    explicit DeviceGuard(int dev)
    {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) {
            ok = cudaSetDevice(dev) == cudaSuccess;
            changed = ok;
        }
    }
    ~DeviceGuard()
    {
        if (changed && prev >= 0) cudaSetDevice(prev);   // (nothing to undo when the caller was on this device already)
    }
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

constexpr int32_t kFlushRows = 2048;               // a batch under construction is launched at this many query rows
constexpr size_t kFlushCandidates = (size_t)4 << 20;   // or this many candidates

void free_batch(Batch* b)
{
    if (!b) return;
    b->h_q.release();
    b->h_idx.release();
    b->h_out.release();
    if (b->d_buf) cudaFree(b->d_buf);
    if (b->done) cudaEventDestroy(b->done);
    delete b;
}

// Launches the batch under construction (caller holds the lock, the object's device is current).  A failure marks
// the batch: its requests then report the error from wait / get_result.
int32_t flush_locked(ucmx_retrieval* r)
{
    Batch* b = r->building;
    if (!b || b->kk.empty()) return UCMX_OK;
    r->building = nullptr;
    b->launched = true;
    const size_t rows = b->kk.size();
    const size_t total = (size_t)b->off.back();
    const size_t ksum = (size_t)b->ooff.back();
    const size_t s_q = align_up(b->h_q.size, 256), s_idx = align_up(total * 4, 256);
    const size_t m_off = align_up((rows + 1) * 4, 256), m_k = align_up(rows * 4, 256);
    const size_t s_meta = 2 * m_off + m_k;
    const size_t s_scores = align_up(total * 4, 256);
    b->o_counts = align_up(rows * 4, 256);
    b->o_idx = align_up((ksum ? ksum : 1) * 4, 256);
    const size_t out_bytes = b->o_counts + 2 * b->o_idx;
    const size_t dev_bytes = s_q + s_idx + s_meta + s_scores + out_bytes;
    auto fail = [&](int32_t rc) {
        b->failed = true;
        cudaStreamSynchronize(r->stream);      // nothing of this batch is in flight when its buffers are reused
        return rc;
    };
    if (b->d_cap < dev_bytes) {
        if (b->d_buf) cudaFree(b->d_buf);
        b->d_buf = nullptr;
        b->d_cap = 0;
        const cudaError_t e = cudaMalloc((void**)&b->d_buf, dev_bytes + dev_bytes / 2);
        if (e != cudaSuccess) return fail(cuda_status("cudaMalloc(batch)", e));
        b->d_cap = dev_bytes + dev_bytes / 2;
    }
    // One copy in instead of three: the candidate lists and the CSR arrays are laid behind the query rows in the same
    // page-locked buffer, in the order the device buffer has them (133 KB moved by the CPU costs less than two more DMAs).
    int32_t rc = b->h_out.reserve(out_bytes);
    if (rc == UCMX_OK) rc = b->h_q.reserve(s_q + s_idx + s_meta);
    if (rc != UCMX_OK) return fail(rc);
    if (!b->done) {
        const cudaError_t e = cudaEventCreateWithFlags(&b->done, cudaEventDisableTiming);
        if (e != cudaSuccess) return fail(cuda_status("cudaEventCreate", e));
    }
    memcpy(b->h_q.p + s_q, b->h_idx.p, total * 4);
    unsigned char* h_meta = b->h_q.p + s_q + s_idx;
    memcpy(h_meta, b->off.data(), (rows + 1) * 4);
    memcpy(h_meta + m_off, b->ooff.data(), (rows + 1) * 4);
    memcpy(h_meta + 2 * m_off, b->kk.data(), rows * 4);

    unsigned char* d = b->d_buf;
    float* d_q = (float*)d;
    int32_t* d_slots = (int32_t*)(d + s_q);
    int32_t* d_off = (int32_t*)(d + s_q + s_idx);
    int32_t* d_ooff = (int32_t*)((unsigned char*)d_off + m_off);
    int32_t* d_k = (int32_t*)((unsigned char*)d_off + 2 * m_off);
    float* d_scores = (float*)(d + s_q + s_idx + s_meta);
    // The selection goes straight into the pinned host buffer (mapped into every device's address space; with unified
    // addressing the host pointer is the device pointer): 8 bytes per winner, written once by the top-k kernel, and a
    // copy back - one more operation for the stream and for the host to wait for - is not needed.
    unsigned char* d_out = b->h_out.p;
    int32_t* d_counts = (int32_t*)d_out;
    int32_t* d_oidx = (int32_t*)(d_out + b->o_counts);
    float* d_osc = (float*)(d_out + b->o_counts + b->o_idx);

    cudaStream_t st = r->stream;
    cudaError_t e = cudaMemcpyAsync(d_q, b->h_q.p, s_q + s_idx + s_meta, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return fail(cuda_status("submit H2D", e));
    rc = ucmx_score_dot(r->table, r->dtype, r->n_items, 1, 1, r->dim, d_off, d_slots, d_q, (int32_t)rows, (int32_t)total,
                        1.0f, d_scores, nullptr, st);
    if (rc == UCMX_OK && ksum > 0)
        rc = ucmx_topk_ragged(d_scores, UCMX_DT_F32, d_off, d_k, (int32_t)rows, 0, 0, UCMX_WIN_NONE, UCMX_ORDER_SCORE_DESC,
                              d_slots, b->kmax, d_ooff, d_oidx, d_osc, d_counts, st);
    if (rc != UCMX_OK) return fail(rc);
    r->launches += ksum > 0 ? 2 : 1;
    if (ksum == 0) memset(d_counts, 0, rows * 4);          // (nothing was launched that writes there)
    e = cudaEventRecord(b->done, st);
    if (e != cudaSuccess) return fail(cuda_status("submit event", e));
    return UCMX_OK;
}

void retire_if_done(ucmx_retrieval* r, Batch* b)
{
    if (b->open > 0) return;
    b->reset();
    r->pool.push_back(b);
}

}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_retrieval_create(const float* host_data, int64_t n_items, int32_t dim, int32_t table_dtype,
                                         int32_t device, ucmx_retrieval** out)
{
    using namespace ucmx;
    if (!out || n_items <= 0 || dim <= 0 || (dim % 8)) return UCMX_EPARAM;
    if (table_dtype != UCMX_DT_BF16 && table_dtype != UCMX_DT_F32) return UCMX_EPARAM;
    DeviceGuard g(device);
    if (!g.ok) return UCMX_EPARAM;
    ucmx_retrieval* r = new (std::nothrow) ucmx_retrieval();
    if (!r) return UCMX_EOOM;
    r->device = device;
    r->n_items = n_items;
    r->dim = dim;
    r->dtype = table_dtype;
    const size_t esz = table_dtype == UCMX_DT_BF16 ? 2 : 4;
    cudaError_t e = cudaMalloc(&r->table, (size_t)n_items * dim * esz);
    if (e != cudaSuccess) {
        delete r;
        return cuda_status("cudaMalloc(table)", e);
    }
    e = cudaStreamCreateWithFlags(&r->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        cudaFree(r->table);
        delete r;
        return cuda_status("cudaStreamCreate", e);
    }
    if (host_data) {
        // upload in bounded pieces through a temporary device buffer
        const int64_t rows_per = std::max<int64_t>(1, (int64_t)(64 << 20) / ((int64_t)dim * 4));
        float* tmp = nullptr;
        e = cudaMalloc((void**)&tmp, (size_t)rows_per * dim * 4);
        if (e != cudaSuccess) {
            ucmx_retrieval_destroy(r);
            return cuda_status("cudaMalloc(tmp)", e);
        }
        for (int64_t r0 = 0; r0 < n_items && e == cudaSuccess; r0 += rows_per) {
            const int64_t nr = std::min(rows_per, n_items - r0);
            e = cudaMemcpyAsync(tmp, host_data + r0 * dim, (size_t)nr * dim * 4, cudaMemcpyHostToDevice, r->stream);
            if (e != cudaSuccess) break;
            const int64_t tot = nr * dim;
            f32_to_bf16_rows_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, r->stream>>>(
                tmp, nullptr, nr, dim,
                table_dtype == UCMX_DT_BF16 ? (uint16_t*)r->table + r0 * dim : nullptr,
                table_dtype == UCMX_DT_F32 ? (float*)r->table + r0 * dim : nullptr);
            e = cudaGetLastError();
            if (e == cudaSuccess) e = cudaStreamSynchronize(r->stream);
        }
        cudaFree(tmp);
        if (e != cudaSuccess) {
            ucmx_retrieval_destroy(r);
            return cuda_status("table upload", e);
        }
    }
    *out = r;
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_update_rows(ucmx_retrieval* r, const int32_t* host_slots, int32_t n,
                                              const float* host_rows)
{
    using namespace ucmx;
    if (!r || n < 0) return UCMX_EPARAM;
    if (n == 0) return UCMX_OK;
    if (!host_slots || !host_rows) return UCMX_EPARAM;
    for (int32_t i = 0; i < n; ++i)
        if (host_slots[i] < 0 || host_slots[i] >= r->n_items) return UCMX_EPARAM;
    DeviceGuard g(r->device);
    std::lock_guard<std::mutex> lk(r->mu);
    float* d_rows = nullptr;
    int32_t* d_slots = nullptr;
    UCMX_CUDA(cudaMalloc((void**)&d_rows, (size_t)n * r->dim * 4));
    cudaError_t e = cudaMalloc((void**)&d_slots, (size_t)n * 4);
    if (e != cudaSuccess) {
        cudaFree(d_rows);
        return cuda_status("cudaMalloc(slots)", e);
    }
    e = cudaMemcpyAsync(d_rows, host_rows, (size_t)n * r->dim * 4, cudaMemcpyHostToDevice, r->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_slots, host_slots, (size_t)n * 4, cudaMemcpyHostToDevice, r->stream);
    if (e == cudaSuccess) {
        const int64_t tot = (int64_t)n * r->dim;
        f32_to_bf16_rows_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, r->stream>>>(
            d_rows, d_slots, n, r->dim, r->dtype == UCMX_DT_BF16 ? (uint16_t*)r->table : nullptr,
            r->dtype == UCMX_DT_F32 ? (float*)r->table : nullptr);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(r->stream);
    cudaFree(d_rows);
    cudaFree(d_slots);
    if (e != cudaSuccess) return cuda_status("update_rows", e);
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_table(ucmx_retrieval* r, void** table, int32_t* table_dtype)
{
    if (!r) return UCMX_EPARAM;
    if (table) *table = r->table;
    if (table_dtype) *table_dtype = r->dtype;
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_submit(ucmx_retrieval* r, const float* host_query, int32_t batch, int32_t query_dim,
                                         int32_t topk, const int32_t* host_indexes, int32_t max_idx, int32_t* req_id)
{
    using namespace ucmx;
    if (!r || !host_query || !host_indexes || !req_id) return UCMX_EPARAM;
    if (query_dim != r->dim) {
        set_last_text("Query dim mismatch");
        return UCMX_EPARAM;
    }
    if (batch < 1 || max_idx < 1 || topk < 0) return UCMX_EPARAM;
    if ((int64_t)batch * max_idx > 0x3fffffffll) return UCMX_EUNSUPPORTED;
    const int32_t k = topk < max_idx ? topk : max_idx;
    if (k > 8192) return UCMX_EUNSUPPORTED;
    const size_t cand = (size_t)batch * max_idx;
    // The index lists are in host memory here, so a bad one is refused before anything reaches the GPU
    // (-1 pads a row; the reference bounds its loop by the table it owns, retrieval_backend.cpp:170-181).
    {
        // one pass without branches (it vectorises): v + 1 as unsigned must be at most n_items
        const uint32_t limit = (uint32_t)(r->n_items < 0x7fffffffll ? r->n_items : 0x7fffffffll);
        uint32_t bad = 0;
        for (size_t i = 0; i < cand; ++i) bad |= (uint32_t)((uint32_t)host_indexes[i] + 1u > limit);
        if (bad) {
            set_last_text("ucmx_retrieval_submit: an index is outside the table (allowed: -1 for padding, 0 .. n_items-1)");
            return UCMX_EPARAM;
        }
    }
    std::lock_guard<std::mutex> lk(r->mu);

    Batch* b = r->building;
    const bool full = b && ((int32_t)b->kk.size() + batch > kFlushRows || (size_t)b->off.back() + cand > kFlushCandidates);
    // (the object's device is made current only for a CUDA call: a launch, or pinned memory for a buffer that grows;
    // an ordinary submit is two memcpys into buffers that are there already)
    const bool grows = !b || full || b->h_q.size + (size_t)batch * r->dim * 4 > b->h_q.cap || b->h_idx.size + cand * 4 > b->h_idx.cap;
    std::optional<DeviceGuard> g;
    if (grows) {
        g.emplace(r->device);
        if (!g->ok) return UCMX_EPARAM;
    }
    if (full) {
        flush_locked(r);           // a failure is recorded in that batch and reported to its own requests
        b = nullptr;
    }
    if (!b) {
        if (!r->pool.empty()) {
            b = r->pool.back();
            r->pool.pop_back();
        } else {
            b = new (std::nothrow) Batch();
            if (!b) return UCMX_EOOM;
        }
        r->building = b;
    }
    const size_t q_size = b->h_q.size, idx_size = b->h_idx.size;
    int32_t rc = b->h_q.append(host_query, (size_t)batch * r->dim * 4);
    if (rc == UCMX_OK) rc = b->h_idx.append(host_indexes, cand * 4);
    if (rc != UCMX_OK) {
        b->h_q.size = q_size;
        b->h_idx.size = idx_size;
        return rc;
    }
    Request rq;
    rq.batch = b;
    rq.row0 = (int32_t)b->kk.size();
    rq.rows = batch;
    rq.k = k;
    for (int32_t i = 0; i < batch; ++i) {
        b->off.push_back(b->off.back() + max_idx);
        b->kk.push_back(k);
        b->ooff.push_back(b->ooff.back() + k);
    }
    if (k > b->kmax) b->kmax = k;
    b->open += 1;
    const int32_t id = r->next_id++;
    r->live.insert(id, rq);
    *req_id = id;
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_flush(ucmx_retrieval* r)
{
    using namespace ucmx;
    if (!r) return UCMX_EPARAM;
    DeviceGuard g(r->device);
    std::lock_guard<std::mutex> lk(r->mu);
    return flush_locked(r);
}

extern "C" int32_t ucmx_retrieval_launches(ucmx_retrieval* r, int64_t* kernels)
{
    if (!r || !kernels) return UCMX_EPARAM;
    std::lock_guard<std::mutex> lk(r->mu);
    *kernels = r->launches;
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_poll(ucmx_retrieval* r, int32_t req_id, int32_t* ready)
{
    using namespace ucmx;
    if (!r || !ready) return UCMX_EPARAM;
    DeviceGuard g(r->device);
    std::lock_guard<std::mutex> lk(r->mu);
    *ready = 0;
    Request* found = r->live.find(req_id);
    if (!found) return UCMX_OK;  // the reference's poll answers "not there" with false, not an error
    Batch* b = found->batch;
    if (!b->launched) flush_locked(r);
    if (b->failed) return UCMX_ERROR;
    const cudaError_t e = cudaEventQuery(b->done);
    if (e == cudaSuccess) {
        *ready = 1;
        return UCMX_OK;
    }
    if (e == cudaErrorNotReady) {
        cudaGetLastError();
        return UCMX_OK;
    }
    return cuda_status("cudaEventQuery", e);
}

extern "C" int32_t ucmx_retrieval_wait(ucmx_retrieval* r, int32_t req_id)
{
    using namespace ucmx;
    if (!r) return UCMX_EPARAM;
    cudaEvent_t ev = nullptr;
    Batch* b = nullptr;
    {
        std::lock_guard<std::mutex> lk(r->mu);
        Request* found = r->live.find(req_id);
        if (!found) return UCMX_ENOOBJ;  // "Bad req_id"
        b = found->batch;
        // ESA waits for every request of a layer in turn: all but the first find their batch already complete
        if (b->launched && !b->failed && b->finished.load(std::memory_order_acquire)) return UCMX_OK;
        if (!b->launched) {
            DeviceGuard g(r->device);
            flush_locked(r);
        }
        if (b->failed) return UCMX_ERROR;
        ev = b->done;
    }
    UCMX_CUDA(cudaEventSynchronize(ev));
    b->finished.store(true, std::memory_order_release);
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_result_shape(ucmx_retrieval* r, int32_t req_id, int32_t* batch, int32_t* topk)
{
    if (!r) return UCMX_EPARAM;
    std::lock_guard<std::mutex> lk(r->mu);
    ucmx::Request* found = r->live.find(req_id);
    if (!found) return UCMX_ENOOBJ;
    if (batch) *batch = found->rows;
    if (topk) *topk = found->k;
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_get_result(ucmx_retrieval* r, int32_t req_id, int32_t* host_indices, float* host_scores)
{
    using namespace ucmx;
    if (!r || !host_indices || !host_scores) return UCMX_EPARAM;
    std::lock_guard<std::mutex> lk(r->mu);
    Request* found = r->live.find(req_id);
    if (!found) return UCMX_ENOOBJ;
    const Request rq = *found;
    Batch* b = rq.batch;
    if (!b->launched) {
        DeviceGuard g(r->device);
        flush_locked(r);
    }
    if (b->failed) {
        r->live.erase(req_id);
        b->open -= 1;
        retire_if_done(r, b);
        return UCMX_ERROR;
    }
    if (!b->finished.load(std::memory_order_acquire)) {
        DeviceGuard g(r->device);
        const cudaError_t e = cudaEventQuery(b->done);
        if (e == cudaErrorNotReady) {
            cudaGetLastError();
            return UCMX_ENOOBJ;  // "Result not ready"
        }
        if (e != cudaSuccess) return cuda_status("cudaEventQuery", e);
        b->finished.store(true, std::memory_order_release);
    }
    const int32_t k = rq.k;
    const int32_t* counts = (const int32_t*)b->h_out.p;
    const int32_t* idx = (const int32_t*)(b->h_out.p + b->o_counts);
    const float* sc = (const float*)(b->h_out.p + b->o_counts + b->o_idx);
    for (int32_t i = 0; i < rq.rows; ++i) {
        const int32_t row = rq.row0 + i;
        const size_t o = (size_t)b->ooff[row];
        for (int32_t j = 0; j < k; ++j) {
            const bool valid = j < counts[row] && idx[o + j] >= 0;
            host_indices[(size_t)i * k + j] = valid ? idx[o + j] : -1;
            host_scores[(size_t)i * k + j] = valid ? sc[o + j] : -INFINITY;
        }
    }
    r->live.erase(req_id);
    b->open -= 1;
    retire_if_done(r, b);
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_destroy(ucmx_retrieval* r)
{
    using namespace ucmx;
    if (!r) return UCMX_EPARAM;
    DeviceGuard g(r->device);
    if (r->stream) cudaStreamSynchronize(r->stream);
    std::vector<Batch*> seen;
    r->live.for_each([&](Request& rq) {
        Batch* b = rq.batch;
        if (b != r->building && std::find(seen.begin(), seen.end(), b) == seen.end()) seen.push_back(b);
    });
    for (Batch* b : seen) free_batch(b);
    free_batch(r->building);
    for (Batch* b : r->pool) free_batch(b);
    if (r->table) cudaFree(r->table);
    if (r->stream) cudaStreamDestroy(r->stream);
    delete r;
    return UCMX_OK;
}

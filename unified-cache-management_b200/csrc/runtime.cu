// Host-side runtime above the kernels: the pinned host ring, event-backed transfer tasks and the
// device-resident retrieval back-end object.  These replace the reference's thread pools and
// condition variables (ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp, ucm/store/task/*,
// ucm/store/device/ibuffered_device.h) with CUDA streams and events: submitting work enqueues
// kernels, polling is an event query, waiting is a bounded event wait.
#include <chrono>
#include <cmath>
#include <cstring>
#include <mutex>
#include <new>
#include <thread>
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

__global__ void fill_regular_offsets_kernel(int32_t* offsets, int32_t* k_per_req, int32_t batch, int32_t max_idx,
                                            int32_t k)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= batch) offsets[i] = i * max_idx;
    if (i < batch) k_per_req[i] = k;
}

struct Request {
    int32_t id = -1;
    int32_t batch = 0, k = 0, topk = 0;
    // pinned host staging
    unsigned char* h_in = nullptr;
    size_t h_in_cap = 0;
    unsigned char* h_out = nullptr;
    size_t h_out_cap = 0;
    // device buffers
    unsigned char* d_buf = nullptr;
    size_t d_cap = 0;
    cudaEvent_t done = nullptr;
    bool in_flight = false;
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
    std::unordered_map<int32_t, ucmx::Request*> live;
    std::vector<ucmx::Request*> pool;
};

namespace ucmx {
namespace {

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev)
    {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard()
    {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int32_t ensure_caps(Request* rq, size_t in_bytes, size_t out_bytes, size_t dev_bytes)
{
    if (rq->h_in_cap < in_bytes) {
        if (rq->h_in) cudaFreeHost(rq->h_in);
        rq->h_in = nullptr;
        rq->h_in_cap = 0;
        UCMX_CUDA(cudaHostAlloc((void**)&rq->h_in, in_bytes, cudaHostAllocPortable));
        rq->h_in_cap = in_bytes;
    }
    if (rq->h_out_cap < out_bytes) {
        if (rq->h_out) cudaFreeHost(rq->h_out);
        rq->h_out = nullptr;
        rq->h_out_cap = 0;
        UCMX_CUDA(cudaHostAlloc((void**)&rq->h_out, out_bytes, cudaHostAllocPortable));
        rq->h_out_cap = out_bytes;
    }
    if (rq->d_cap < dev_bytes) {
        if (rq->d_buf) cudaFree(rq->d_buf);
        rq->d_buf = nullptr;
        rq->d_cap = 0;
        UCMX_CUDA(cudaMalloc((void**)&rq->d_buf, dev_bytes));
        rq->d_cap = dev_bytes;
    }
    if (!rq->done) UCMX_CUDA(cudaEventCreateWithFlags(&rq->done, cudaEventDisableTiming));
    return UCMX_OK;
}

void free_request(Request* rq)
{
    if (!rq) return;
    if (rq->h_in) cudaFreeHost(rq->h_in);
    if (rq->h_out) cudaFreeHost(rq->h_out);
    if (rq->d_buf) cudaFree(rq->d_buf);
    if (rq->done) cudaEventDestroy(rq->done);
    delete rq;
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
    if ((int64_t)batch * max_idx > 0x7fffffffll) return UCMX_EUNSUPPORTED;
    const int32_t k = topk < max_idx ? topk : max_idx;
    if (k > 8192) return UCMX_EUNSUPPORTED;
    const int32_t kcap = k > 0 ? k : 1;
    DeviceGuard g(r->device);
    std::lock_guard<std::mutex> lk(r->mu);

    Request* rq = nullptr;
    if (!r->pool.empty()) {
        rq = r->pool.back();
        r->pool.pop_back();
    } else {
        rq = new (std::nothrow) Request();
        if (!rq) return UCMX_EOOM;
    }
    const size_t total = (size_t)batch * max_idx;
    // host -> device block: [query fp32 b*dim | slot ids int32 total]
    const size_t in_q = align_up((size_t)batch * r->dim * 4, 256);
    const size_t in_idx = align_up(total * 4, 256);
    // device scratch behind it: [offsets b+1 | k_per_req b | scores total | counts b | out_idx b*k | out_scores b*k]
    const size_t s_off = align_up((size_t)(batch + 1) * 4, 256);
    const size_t s_k = align_up((size_t)batch * 4, 256);
    const size_t s_scores = align_up(total * 4, 256);
    const size_t o_counts = align_up((size_t)batch * 4, 256);
    const size_t o_idx = align_up((size_t)batch * kcap * 4, 256);
    const size_t o_sc = align_up((size_t)batch * kcap * 4, 256);
    const size_t out_bytes = o_counts + o_idx + o_sc;
    const size_t dev_bytes = in_q + in_idx + s_off + s_k + s_scores + out_bytes;
    int32_t rc = ensure_caps(rq, in_q + in_idx, out_bytes, dev_bytes);
    if (rc != UCMX_OK) {
        free_request(rq);
        return rc;
    }
    memcpy(rq->h_in, host_query, (size_t)batch * r->dim * 4);
    memcpy(rq->h_in + in_q, host_indexes, total * 4);

    unsigned char* d = rq->d_buf;
    float* d_q = (float*)d;
    int32_t* d_slots = (int32_t*)(d + in_q);
    int32_t* d_off = (int32_t*)(d + in_q + in_idx);
    int32_t* d_k = (int32_t*)((unsigned char*)d_off + s_off);
    float* d_scores = (float*)((unsigned char*)d_k + s_k);
    unsigned char* d_out = (unsigned char*)d_scores + s_scores;
    int32_t* d_counts = (int32_t*)d_out;
    int32_t* d_oidx = (int32_t*)(d_out + o_counts);
    float* d_osc = (float*)(d_out + o_counts + o_idx);

    cudaStream_t st = r->stream;
    cudaError_t e = cudaMemcpyAsync(d, rq->h_in, in_q + in_idx, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) {
        r->pool.push_back(rq);
        return cuda_status("submit H2D", e);
    }
    fill_regular_offsets_kernel<<<(batch + 256) / 256, 256, 0, st>>>(d_off, d_k, batch, max_idx, k);
    rc = ucmx_score_dot(r->table, r->dtype, 1, 1, r->dim, d_off, d_slots, d_q, batch, (int32_t)total, 1.0f, d_scores, st);
    if (rc == UCMX_OK && k > 0)
        rc = ucmx_topk_ragged(d_scores, UCMX_DT_F32, d_off, d_k, batch, 0, 0, UCMX_WIN_NONE, UCMX_ORDER_SCORE_DESC,
                              d_slots, kcap, nullptr, d_oidx, d_osc, d_counts, st);
    if (rc != UCMX_OK) {
        r->pool.push_back(rq);
        return rc;
    }
    e = cudaMemcpyAsync(rq->h_out, d_out, out_bytes, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaEventRecord(rq->done, st);
    if (e != cudaSuccess) {
        r->pool.push_back(rq);
        return cuda_status("submit D2H", e);
    }
    rq->id = r->next_id++;
    rq->batch = batch;
    rq->k = k;
    rq->topk = topk;
    rq->in_flight = true;
    r->live[rq->id] = rq;
    *req_id = rq->id;
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_poll(ucmx_retrieval* r, int32_t req_id, int32_t* ready)
{
    using namespace ucmx;
    if (!r || !ready) return UCMX_EPARAM;
    std::lock_guard<std::mutex> lk(r->mu);
    auto it = r->live.find(req_id);
    if (it == r->live.end()) {
        *ready = 0;
        return UCMX_OK;  // the reference's poll answers "not there" with false, not an error
    }
    cudaError_t e = cudaEventQuery(it->second->done);
    if (e == cudaSuccess) {
        *ready = 1;
        return UCMX_OK;
    }
    *ready = 0;
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
    {
        std::lock_guard<std::mutex> lk(r->mu);
        auto it = r->live.find(req_id);
        if (it == r->live.end()) return UCMX_ENOOBJ;  // "Bad req_id"
        ev = it->second->done;
    }
    UCMX_CUDA(cudaEventSynchronize(ev));
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_result_shape(ucmx_retrieval* r, int32_t req_id, int32_t* batch, int32_t* topk)
{
    if (!r) return UCMX_EPARAM;
    std::lock_guard<std::mutex> lk(r->mu);
    auto it = r->live.find(req_id);
    if (it == r->live.end()) return UCMX_ENOOBJ;
    if (batch) *batch = it->second->batch;
    if (topk) *topk = it->second->k;
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_get_result(ucmx_retrieval* r, int32_t req_id, int32_t* host_indices, float* host_scores)
{
    using namespace ucmx;
    if (!r || !host_indices || !host_scores) return UCMX_EPARAM;
    std::lock_guard<std::mutex> lk(r->mu);
    auto it = r->live.find(req_id);
    if (it == r->live.end()) return UCMX_ENOOBJ;
    Request* rq = it->second;
    cudaError_t e = cudaEventQuery(rq->done);
    if (e == cudaErrorNotReady) {
        cudaGetLastError();
        return UCMX_ENOOBJ;  // "Result not ready"
    }
    if (e != cudaSuccess) return cuda_status("cudaEventQuery", e);
    const int32_t b = rq->batch, k = rq->k, kcap = k > 0 ? k : 1;
    const size_t o_counts = align_up((size_t)b * 4, 256);
    const size_t o_idx = align_up((size_t)b * kcap * 4, 256);
    const int32_t* counts = (const int32_t*)rq->h_out;
    const int32_t* idx = (const int32_t*)(rq->h_out + o_counts);
    const float* sc = (const float*)(rq->h_out + o_counts + o_idx);
    for (int32_t i = 0; i < b; ++i) {
        for (int32_t j = 0; j < k; ++j) {
            const bool valid = j < counts[i] && idx[(size_t)i * kcap + j] >= 0;
            host_indices[(size_t)i * k + j] = valid ? idx[(size_t)i * kcap + j] : -1;
            host_scores[(size_t)i * k + j] = valid ? sc[(size_t)i * kcap + j] : -INFINITY;
        }
    }
    r->live.erase(it);
    rq->in_flight = false;
    r->pool.push_back(rq);
    return UCMX_OK;
}

extern "C" int32_t ucmx_retrieval_destroy(ucmx_retrieval* r)
{
    using namespace ucmx;
    if (!r) return UCMX_EPARAM;
    DeviceGuard g(r->device);
    if (r->stream) cudaStreamSynchronize(r->stream);
    for (auto& kv : r->live) free_request(kv.second);
    for (auto* rq : r->pool) free_request(rq);
    if (r->table) cudaFree(r->table);
    if (r->stream) cudaStreamDestroy(r->stream);
    delete r;
    return UCMX_OK;
}

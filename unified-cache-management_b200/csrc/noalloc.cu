// Allocation-free retrieval: score + top-k for callers that must not allocate device memory.
//
// Scoring followed by top-k needs room for one fp32 score per candidate between the two kernels.
// The other entry points leave that buffer to the caller (ucmx_score_dot / ucmx_topk_ragged) or
// take it from cudaMalloc (the retrieval back-end object).  Some callers can do neither: the
// attention hooks of a serving engine run in the middle of its forward pass, after the engine has
// handed almost all of HBM to its KV cache, so a cudaMalloc there may fail, and it synchronises the
// whole device even when it succeeds; such callers also often hold no allocator of their own to
// carve a scratch tensor from.  For them the score buffer below is part of the library image: a
// fixed array in device memory that every GPU loading the library holds until the process exits.
#include <mutex>

#include "common.cuh"

// One fp32 score per candidate; 2^20 candidates = 4 MiB per GPU.  At 128-token blocks that is
// 134 M tokens of context across the batch, thirty times the 64-request benchmark batch.
#define UCMX_NOALLOC_MAX_CANDIDATES (1 << 20)

static __device__ __align__(256) float g_noalloc_scores[UCMX_NOALLOC_MAX_CANDIDATES];

namespace ucmx {
namespace {

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices];  // device address of g_noalloc_scores, per device
std::mutex g_scratch_mu;

// In host code `g_noalloc_scores` is only a handle for the runtime, not an address a kernel can
// use; the device address has to be asked for, once per device, with that device current.
int32_t scratch_for_current_device(float** out)
{
    int dev = -1;
    UCMX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return UCMX_EUNSUPPORTED;
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scores);
        if (e != cudaSuccess) return cuda_status("cudaGetSymbolAddress(g_noalloc_scores)", e);
        if (!p) {
            set_last_text("cudaGetSymbolAddress returned a null address for the score scratch");
            return UCMX_EOSERROR;
        }
        g_scratch_addr[dev] = (float*)p;
    }
    *out = g_scratch_addr[dev];
    return UCMX_OK;
}

}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_retrieve_topk_noalloc(const void* reps, int32_t reps_dtype, int64_t n_slots,
                                              int32_t n_kv_heads, int32_t n_rep, int32_t head_dim,
                                              const int32_t* req_offsets,
                                              const int32_t* slot_ids, const float* q, int32_t n_req,
                                              int32_t total, float scale, const int32_t* k_per_req,
                                              int32_t start_win, int32_t end_win, int32_t window_mode,
                                              int32_t order, const int32_t* id_map, int32_t out_stride,
                                              const int32_t* out_offsets, int32_t* out_idx, float* out_scores,
                                              int32_t* out_counts, ucmx_stream_t stream)
{
    using namespace ucmx;
    if (n_req < 0 || total < 0) return UCMX_EPARAM;
    if (total > UCMX_NOALLOC_MAX_CANDIDATES) {
        set_last_text("ucmx_retrieve_topk_noalloc: more candidates than the built-in score scratch holds "
                      "(limit 1048576); use ucmx_score_dot + ucmx_topk_ragged with a caller-owned buffer");
        return UCMX_EUNSUPPORTED;
    }
    if (n_req == 0) return UCMX_OK;
    float* scratch = nullptr;
    int32_t rc = scratch_for_current_device(&scratch);
    if (rc != UCMX_OK) return rc;
    // Every score in [0, total) is written by the scoring kernel before the top-k kernel, next on the
    // same stream, reads it; nothing in the scratch has to start from zero.
    // (no error word on this path: the one ucmx_device_error reads is allocated on first use)
    rc = score_dot_impl(reps, reps_dtype, n_slots, n_kv_heads, n_rep, head_dim, req_offsets, slot_ids, q, n_req,
                        total, scale, scratch, nullptr, nullptr, (cudaStream_t)stream);
    if (rc != UCMX_OK) return rc;
    return ucmx_topk_ragged(scratch, UCMX_DT_F32, req_offsets, k_per_req, n_req, start_win, end_win, window_mode,
                            order, id_map, out_stride, out_offsets, out_idx, out_scores, out_counts, stream);
}

extern "C" int32_t ucmx_noalloc_max_candidates(void) { return UCMX_NOALLOC_MAX_CANDIDATES; }

// C entry point around the reference's KVStar retrieval kernel (KVStar::Execute,
// ucm/sparse/kvstar/retrieve/core/domain/retrieve_task/simd_compute_kernel.cpp), compiled from the
// checkout where it lies.  Test infrastructure only: it pins the multi-query softmax-vote block
// scores' consequence, the selected block set, for the CUDA path.
#include <cstdint>
#include <cstring>
#include <optional>
#include "retrieve_task/retrieve_task.h"
#include "retrieve_task/simd_compute_kernel.h"
#include "retrieve_task/task_result.h"

extern "C" int kvstar_ref_execute(const void* q_fp16, int64_t x, int64_t Hq, int64_t d_orig, const void* reps_fp16,
                                  int64_t n, int64_t M, int64_t h, int64_t d_pruned, const int64_t* pruned_index,
                                  int topk, int64_t* out_indices)
{
    KVStar::PlainTensor q, k;
    q.data = const_cast<void*>(q_fp16);
    q.shape = {x, Hq, d_orig};
    k.data = const_cast<void*>(reps_fp16);
    k.shape = {n, M, h, d_pruned};
    std::optional<KVStar::PlainTensor> idx;
    if (pruned_index) {
        KVStar::PlainTensor t;
        t.data = const_cast<int64_t*>(pruned_index);
        t.shape = {h, d_pruned};
        idx = t;
    }
    KVStar::RetrieveTask task(q, k, idx, topk, 0, KVStar::CPU);
    KVStar::TaskResult result;
    try {
        KVStar::Execute(task, result);
    } catch (const std::exception&) {
        return -1;
    }
    std::memcpy(out_indices, result.topkIndices.data(), result.topkIndices.size() * sizeof(int64_t));
    return (int)result.topkIndices.size();
}

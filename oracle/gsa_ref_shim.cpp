// C entry points over the reference's own GSA offload arithmetic
// (ucm/sparse/gsa/offload_ops: vec_product.cpp, k_repre.cpp, select_topk_block.cpp),
// which are compiled from the reference tree next to this file by oracle/Makefile.
// TEST INFRASTRUCTURE ONLY: used to pin oracle/ucm_oracle.c and as a CPU baseline.
#include <cstdint>
#include <vector>
#include "k_repre.h"
#include "select_topk_block.h"

extern "C" {

// KRepreComputer::ComputeKRepre over blocks laid out [kHead, blockSize, headSize] fp32.
void gsa_ref_k_repre(const float* k, int64_t block_elems, uint32_t num_block, uint32_t k_head,
                     uint32_t block_size, uint32_t head_size, float* out)
{
    KRepre::KRepreComputer c;
    std::vector<float*> in(num_block), o(num_block);
    for (uint32_t i = 0; i < num_block; ++i) {
        in[i] = const_cast<float*>(k) + (int64_t)i * block_elems;
        o[i] = out + (int64_t)i * k_head * head_size;
    }
    c.ComputeKRepre(in, num_block, k_head, block_size, head_size, o);
}

// TopkBlockSelector::SelectTopK for one request. q [qHead, headSize] is overwritten in place
// with the per-KV-head means, exactly as the reference does.
void gsa_ref_select_topk(float* q, const float* k_repre, uint32_t num_block, uint32_t k_head,
                         uint32_t q_head, uint32_t num_krepre, uint32_t head_size,
                         uint32_t start_window, uint32_t end_window, uint32_t topk,
                         int32_t* out)
{
    SelectTopkBlock::TopkBlockSelector s;
    s.SetWindowSize(start_window, end_window);
    s.SelectTopK(q, k_repre, num_block, k_head, q_head, num_krepre, head_size, topk, out);
}

// Scores only (ComputeKQDotScores) with q already reduced to [kHead, headSize].
void gsa_ref_scores(const float* q_mean, const float* k_repre, uint32_t num_block,
                    uint32_t k_head, uint32_t num_krepre, uint32_t head_size, float* out)
{
    SelectTopkBlock::TopkBlockSelector s;
    std::vector<float> v = s.ComputeKQDotScores(q_mean, k_repre, num_block, k_head, num_krepre,
                                                head_size);
    for (uint32_t i = 0; i < num_block; ++i) out[i] = v[i];
}

// ComputeQHeadMean in place.
void gsa_ref_q_head_mean(float* q, uint32_t k_head, uint32_t q_head, uint32_t head_size)
{
    SelectTopkBlock::TopkBlockSelector s;
    s.ComputeQHeadMean(q, k_head, q_head, head_size);
}

}  // extern "C"

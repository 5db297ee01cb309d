/*
 * CPU restatement of the UCM sparse-KV retrieval and block-transfer path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against.  Nothing in the shipped package imports, links or runs
 * it; only the test-suite, the smoke check and the benchmark's CPU-baseline
 * leg may.
 *
 * Every function names the reference lines (paths inside the UCM project)
 * whose arithmetic it restates.  Parity status of each function:
 *   - orc_score_dot_esa, orc_topk_esa : pinned against the compiled reference
 *     ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp (bit-exact scores).
 *   - orc_pool_blocks (fp32, unrounded), orc_score_dot_gsa, orc_topk_gsa :
 *     pinned against the compiled reference ucm/sparse/gsa/offload_ops/src.
 *   - orc_hash_encode, orc_unpack/hamming : pinned against vectors produced by
 *     importing ucm/sparse/kvcomp/hash_encoder.py on CPU (tests/golden).
 *   - torch expressions with no native twin (bf16-rounded mean, bf16 GQA query
 *     mean, KVComp top-k slicing): pinned against vectors produced by running
 *     those torch expressions on CPU (tests/golden); the reference ships no
 *     known-answer test for them.
 *
 * Build: see oracle/Makefile (plain C99, -ffp-contract=off so that a*b+c is
 * never fused and the summation matches the reference's x86-64 build).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ bf16 */

static inline float bf16_to_f32(uint16_t h)
{
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even, NaN kept quiet: what torch's .to(bfloat16) does */
static inline uint16_t f32_to_bf16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

float orc_bf16_round(float f) { return bf16_to_f32(f32_to_bf16(f)); }

/* ------------------------------------------------------------ stage 1: pool
 *
 * rep[b, h, :] = reduce over the block's tokens of K[block_ids[b], t, h, :].
 *
 * mode 0 mean, 1 max, 2 min, 3 sum.
 * Mean follows VectorMeanImpl (ucm/sparse/gsa/offload_ops/src/vec_product.cpp
 * :349-387): start from token 0, add tokens 1..T-1 in order, multiply by
 * 1.0f/T.  With round_bf16 != 0 the result is rounded to bf16 and widened
 * again, which is what ESA stores: `k_cache[ids].mean(1)` in bf16 followed by
 * `.to(float32)` (ucm/sparse/esa/esa.py:265-266, 363-364; GSA gsa.py:640-652).
 * max/min/sum are the chunk_repre_method variants of
 * ucm/sparse/kvcomp/kvcomp_config.py:56,116-120 (element-wise over tokens).
 *
 * k: bf16 paged cache; element (blk, t, h, d) at
 *    blk*block_stride + t*token_stride + h*head_dim + d.
 * out: fp32 [n, n_kv_heads*head_dim].
 */
void orc_pool_blocks(const uint16_t *k, int64_t block_stride, int64_t token_stride,
                     int32_t block_tokens, int32_t n_kv_heads, int32_t head_dim,
                     const int32_t *block_ids, int32_t n, int32_t mode, int32_t round_bf16,
                     float *out)
{
    const int64_t E = (int64_t)n_kv_heads * head_dim;
    const float inv = 1.0f / (float)block_tokens;
    for (int32_t b = 0; b < n; ++b) {
        const uint16_t *blk = k + (int64_t)block_ids[b] * block_stride;
        float *o = out + (int64_t)b * E;
        for (int64_t e = 0; e < E; ++e) o[e] = bf16_to_f32(blk[e]);
        for (int32_t t = 1; t < block_tokens; ++t) {
            const uint16_t *row = blk + (int64_t)t * token_stride;
            for (int64_t e = 0; e < E; ++e) {
                float v = bf16_to_f32(row[e]);
                if (mode == 1) o[e] = v > o[e] ? v : o[e];
                else if (mode == 2) o[e] = v < o[e] ? v : o[e];
                else o[e] += v;
            }
        }
        for (int64_t e = 0; e < E; ++e) {
            if (mode == 0) o[e] *= inv;
            if (round_bf16) o[e] = orc_bf16_round(o[e]);
        }
    }
}

/* ------------------------------------------------- stage 2 prologue: query
 *
 * qbar[t, h, :] = mean over the q-heads of KV group h.
 * ESA/KVComp take it in bf16 (esa.py:291-293, kvcomp.py:220-223): fp32 sum,
 * bf16 result, then cast to fp32 (retrieval_worker.py:16-18).  The GSA native
 * path keeps fp32 (ComputeQHeadMean, select_topk_block.cpp:101-114).
 * When n_q_heads < n_kv_heads the query head is repeated (esa.py:294-295).
 * q: bf16 [n_tok, n_q_heads, head_dim] with tok_stride elements per token.
 */
void orc_query_group_mean(const uint16_t *q, int32_t n_tok, int32_t n_q_heads,
                          int32_t n_kv_heads, int32_t head_dim, int64_t tok_stride,
                          int32_t round_bf16, float *out)
{
    for (int32_t t = 0; t < n_tok; ++t) {
        const uint16_t *qt = q + (int64_t)t * tok_stride;
        float *o = out + (int64_t)t * n_kv_heads * head_dim;
        if (n_q_heads >= n_kv_heads) {
            int32_t g = n_q_heads / n_kv_heads;
            float inv = 1.0f / (float)g;
            for (int32_t h = 0; h < n_kv_heads; ++h)
                for (int32_t d = 0; d < head_dim; ++d) {
                    float acc = bf16_to_f32(qt[(int64_t)(h * g) * head_dim + d]);
                    for (int32_t j = 1; j < g; ++j)
                        acc += bf16_to_f32(qt[(int64_t)(h * g + j) * head_dim + d]);
                    acc *= inv;
                    o[h * head_dim + d] = round_bf16 ? orc_bf16_round(acc) : acc;
                }
        } else {
            int32_t r = n_kv_heads / n_q_heads;
            for (int32_t h = 0; h < n_kv_heads; ++h)
                for (int32_t d = 0; d < head_dim; ++d)
                    o[h * head_dim + d] = bf16_to_f32(qt[(int64_t)(h / r) * head_dim + d]);
        }
    }
}

/* ------------------------------------------------------ stage 2: dot scores
 *
 * ESA (retrieval_backend.cpp:170-181): for each allowed slot,
 * score = sum over d of q[d]*data[slot*dim+d], accumulated left to right in
 * fp32 starting from 0.
 * Ragged batch: request r owns candidates [req_offsets[r], req_offsets[r+1]);
 * slot_ids may be NULL (slot = flat candidate index).
 */
void orc_score_dot_esa(const float *data, int32_t dim, const int32_t *req_offsets,
                       const int32_t *slot_ids, const float *q, int32_t n_req, float *out)
{
    for (int32_t r = 0; r < n_req; ++r) {
        const float *qr = q + (int64_t)r * dim;
        for (int32_t c = req_offsets[r]; c < req_offsets[r + 1]; ++c) {
            int64_t slot = slot_ids ? slot_ids[c] : c;
            const float *row = data + slot * dim;
            float s = 0.0f;
            for (int32_t d = 0; d < dim; ++d) s += qr[d] * row[d];
            out[c] = s;
        }
    }
}

/* GSA (select_topk_block.cpp:53-76): reps [slot, kvH, n_rep, D];
 * score = sum over kv heads of max over reps of dot(qbar_h, rep).
 * The dot is taken left to right here; the reference's SIMD variants use a
 * 16-lane (AVX-512) or 8-lane tree, so agreement is to rounding, not bits. */
void orc_score_dot_gsa(const float *reps, int32_t n_kv_heads, int32_t n_rep, int32_t head_dim,
                       const int32_t *req_offsets, const int32_t *slot_ids, const float *q,
                       int32_t n_req, float *out)
{
    const int64_t row = (int64_t)n_kv_heads * n_rep * head_dim;
    for (int32_t r = 0; r < n_req; ++r) {
        const float *qr = q + (int64_t)r * n_kv_heads * head_dim;
        for (int32_t c = req_offsets[r]; c < req_offsets[r + 1]; ++c) {
            int64_t slot = slot_ids ? slot_ids[c] : c;
            const float *blk = reps + slot * row;
            float total = 0.0f;
            for (int32_t h = 0; h < n_kv_heads; ++h) {
                float best = -3.402823466e+38f;
                for (int32_t j = 0; j < n_rep; ++j) {
                    const float *kv = blk + ((int64_t)h * n_rep + j) * head_dim;
                    float s = 0.0f;
                    for (int32_t d = 0; d < head_dim; ++d) s += qr[h * head_dim + d] * kv[d];
                    best = fmaxf(best, s);
                }
                total += best;
            }
            out[c] = total;
        }
    }
}

/* ------------------------------------------------------------ stage 3: top-k */

typedef struct { float s; int32_t i; } orc_pair;

static int cmp_desc_stable(const void *a, const void *b)
{
    const orc_pair *x = (const orc_pair *)a, *y = (const orc_pair *)b;
    if (x->s > y->s) return -1;
    if (x->s < y->s) return 1;
    return (x->i > y->i) - (x->i < y->i);
}

/* ESA (retrieval_backend.cpp:182-189): the k best of one request's candidates
 * in descending score order; returns min(k, n) entries.  std::partial_sort is
 * not stable, so equal scores may come out in any order there; this
 * restatement breaks ties by the lower candidate position.
 * out_idx holds id_map[position] when id_map is given (the reference returns
 * slot ids), else the position. Returns the count written. */
int32_t orc_topk_esa(const float *scores, int32_t n, int32_t k, const int32_t *id_map,
                     int32_t *out_idx, float *out_scores)
{
    orc_pair *p = (orc_pair *)malloc(sizeof(orc_pair) * (size_t)(n > 0 ? n : 1));
    for (int32_t i = 0; i < n; ++i) { p[i].s = scores[i]; p[i].i = i; }
    qsort(p, (size_t)n, sizeof(orc_pair), cmp_desc_stable);
    int32_t m = k < n ? k : n;
    if (m < 0) m = 0;
    for (int32_t j = 0; j < m; ++j) {
        out_idx[j] = id_map ? id_map[p[j].i] : p[j].i;
        if (out_scores) out_scores[j] = p[j].s;
    }
    free(p);
    return m;
}

static int cmp_int(const void *a, const void *b)
{
    int32_t x = *(const int32_t *)a, y = *(const int32_t *)b;
    return (x > y) - (x < y);
}

/* GSA (TopkBlockSelector::TopKImpl, select_topk_block.cpp:20-51): force the
 * first `start` and last `end` blocks, fill the rest of k from the middle by
 * descending score (stable: lower index wins ties), return ascending indices.
 * Degenerate inputs (start+end >= n, k >= n, k == 0) return the identity.
 * The reference writes n entries in the degenerate case even when its buffer
 * holds fewer; here at most `cap` entries are written.  Returns the count. */
int32_t orc_topk_gsa(const float *scores, int32_t n, int32_t k, int32_t start, int32_t end,
                     int32_t cap, int32_t *out_idx)
{
    int32_t cnt = 0;
    if (start + end >= n || k >= n || k == 0) {
        for (int32_t i = 0; i < n && cnt < cap; ++i) out_idx[cnt++] = i;
        return cnt;
    }
    int32_t mid = k - start - end;
    int32_t total = start + (mid > 0 ? mid : 0) + end;
    int32_t *tmp = (int32_t *)malloc(sizeof(int32_t) * (size_t)total);
    int32_t w = 0;
    for (int32_t i = 0; i < start; ++i) tmp[w++] = i;
    if (mid > 0) {
        int32_t m = n - start - end;
        orc_pair *p = (orc_pair *)malloc(sizeof(orc_pair) * (size_t)m);
        for (int32_t i = 0; i < m; ++i) { p[i].s = scores[start + i]; p[i].i = start + i; }
        qsort(p, (size_t)m, sizeof(orc_pair), cmp_desc_stable);
        for (int32_t j = 0; j < mid; ++j) tmp[w++] = p[j].i;
        free(p);
    }
    for (int32_t i = 0; i < end; ++i) tmp[w++] = n - end + i;
    qsort(tmp, (size_t)w, sizeof(int32_t), cmp_int);
    for (int32_t i = 0; i < w && cnt < cap; ++i) out_idx[cnt++] = tmp[i];
    free(tmp);
    return cnt;
}

/* KVComp (kvcomp.py:202-254): candidates are blocks [init, n-local+1); when
 * k >= n every one of them is returned; otherwise the k best of that range,
 * reported as ascending block ids.  torch.topk's tie order is unspecified;
 * ties go to the lower block here.  Scores are exact integers.  */
int32_t orc_topk_kvcomp(const int32_t *scores, int32_t n, int32_t k, int32_t init_win,
                        int32_t local_win, int32_t *out_idx)
{
    int32_t lo = init_win, hi = n - local_win + 1;
    int32_t cnt = 0;
    if (k >= n) {
        for (int32_t i = lo; i < hi; ++i) out_idx[cnt++] = i;
        return cnt;
    }
    int32_t m = hi - lo;
    if (m <= 0) return 0;
    orc_pair *p = (orc_pair *)malloc(sizeof(orc_pair) * (size_t)m);
    for (int32_t i = 0; i < m; ++i) { p[i].s = (float)scores[lo + i]; p[i].i = lo + i; }
    /* |score| <= 2^24 is exact in fp32 for the sizes used; guard anyway */
    qsort(p, (size_t)m, sizeof(orc_pair), cmp_desc_stable);
    int32_t take = k < m ? k : m;
    for (int32_t j = 0; j < take; ++j) out_idx[cnt++] = p[j].i;
    free(p);
    qsort(out_idx, (size_t)cnt, sizeof(int32_t), cmp_int);
    return cnt;
}

/* ------------------------------------------------------- stage 1: hash codes
 *
 * HashEncoder.compute_hash (ucm/sparse/kvcomp/hash_encoder.py:99-157):
 * bit j of a vector x is (sum_d x[d]*W[d,j] > 0); bits are packed LSB first,
 * 8 per byte (:139-149).  The reference takes the sum inside a library GEMM
 * whose accumulation order is unspecified; this restatement fixes it as the
 * fp32 fused multiply-add chain over d = 0..dim-1 starting from 0 (each bf16
 * product is exact in fp32, so only the order of additions is a choice).
 * x: bf16 [n_vec, dim]; w: bf16 [dim, bits]; out: uint8 [n_vec, bits/8].
 */
void orc_hash_encode(const uint16_t *x, int64_t n_vec, const uint16_t *w, int32_t dim,
                     int32_t bits, uint8_t *out)
{
    const int32_t nbytes = bits / 8;
    float *wf = (float *)malloc(sizeof(float) * (size_t)dim * bits);
    float *acc = (float *)malloc(sizeof(float) * (size_t)bits);
    for (int64_t i = 0; i < (int64_t)dim * bits; ++i) wf[i] = bf16_to_f32(w[i]);
    for (int64_t v = 0; v < n_vec; ++v) {
        const uint16_t *xv = x + v * dim;
        for (int32_t j = 0; j < bits; ++j) acc[j] = 0.0f;
        for (int32_t d = 0; d < dim; ++d) {
            float xd = bf16_to_f32(xv[d]);
            const float *wr = wf + (int64_t)d * bits;
            for (int32_t j = 0; j < bits; ++j) acc[j] = fmaf(xd, wr[j], acc[j]);
        }
        uint8_t *o = out + v * nbytes;
        for (int32_t b = 0; b < nbytes; ++b) {
            uint8_t byte = 0;
            for (int32_t i = 0; i < 8; ++i)
                if (acc[b * 8 + i] > 0.0f) byte |= (uint8_t)(1u << i);
            o[b] = byte;
        }
    }
    free(wf);
    free(acc);
}

/* The projection margins themselves, for tests that want to know how close to
 * zero a bit's pre-sign value was.  out: fp32 [n_vec, bits]. */
void orc_hash_project(const uint16_t *x, int64_t n_vec, const uint16_t *w, int32_t dim,
                      int32_t bits, float *out)
{
    for (int64_t v = 0; v < n_vec; ++v)
        for (int32_t j = 0; j < bits; ++j) {
            float a = 0.0f;
            for (int32_t d = 0; d < dim; ++d)
                a = fmaf(bf16_to_f32(x[v * dim + d]), bf16_to_f32(w[(int64_t)d * bits + j]), a);
            out[v * bits + j] = a;
        }
}

/* --------------------------------------------------- stage 2: Hamming scores
 *
 * kvcomp.py:233-247: codes are unpacked to +-1 (hash_encoder.py:159-219) and
 * contracted with einsum "tid,njsd->tijsn", then summed over t, i, j, s.  For
 * one query token that is
 *   score[n] = sum_i sum_j sum_s (bits - 2*popcount(q_i xor k_{n,j,s}))
 * over EVERY (query head i, key head j) pair when cross_head != 0.  With
 * cross_head == 0 only matching heads (i == j) are paired.
 * codes: uint8 [slot, n_kv_heads, block_tokens, bits/8]
 * q_codes: uint8 [n_req, n_q_heads, bits/8]; out: int32 per candidate.
 */
void orc_score_hamming(const uint8_t *codes, int32_t n_kv_heads, int32_t block_tokens,
                       int32_t bits, const int32_t *req_offsets, const int32_t *slot_ids,
                       const uint8_t *q_codes, int32_t n_q_heads, int32_t n_req,
                       int32_t cross_head, int32_t *out)
{
    const int32_t nb = bits / 8;
    const int64_t row = (int64_t)n_kv_heads * block_tokens * nb;
    for (int32_t r = 0; r < n_req; ++r) {
        const uint8_t *qr = q_codes + (int64_t)r * n_q_heads * nb;
        for (int32_t c = req_offsets[r]; c < req_offsets[r + 1]; ++c) {
            int64_t slot = slot_ids ? slot_ids[c] : c;
            const uint8_t *blk = codes + slot * row;
            int64_t total = 0;
            for (int32_t j = 0; j < n_kv_heads; ++j)
                for (int32_t s = 0; s < block_tokens; ++s) {
                    const uint8_t *kc = blk + ((int64_t)j * block_tokens + s) * nb;
                    for (int32_t i = 0; i < n_q_heads; ++i) {
                        if (!cross_head && i != j) continue;
                        const uint8_t *qc = qr + (int64_t)i * nb;
                        int32_t ham = 0;
                        for (int32_t b = 0; b < nb; ++b)
                            ham += __builtin_popcount((unsigned)(qc[b] ^ kc[b]));
                        total += bits - 2 * ham;
                    }
                }
            out[c] = (int32_t)total;
        }
    }
}

/* ------------------------------------------------ stage 4: gather / scatter
 *
 * What UcmDramStore.dump/load (ucm/store/dramstore/dramstore_connector.py
 * :112-166) and H2DKernel/D2HKernel (ucm/store/device/cuda/cuda_device.cu
 * :47-69) do per block: copy slice_bytes between block slot id*block_stride of
 * each plane (K, V) and a contiguous staging area laid out
 * [i][plane][slice_bytes].
 */
void orc_gather_blocks(const uint8_t *const *planes, int32_t n_planes, int64_t block_stride,
                       const int32_t *block_ids, int32_t n, int64_t slice_bytes, uint8_t *staging)
{
    for (int32_t i = 0; i < n; ++i)
        for (int32_t p = 0; p < n_planes; ++p)
            memcpy(staging + ((int64_t)i * n_planes + p) * slice_bytes,
                   planes[p] + (int64_t)block_ids[i] * block_stride, (size_t)slice_bytes);
}

void orc_scatter_blocks(uint8_t *const *planes, int32_t n_planes, int64_t block_stride,
                        const int32_t *block_ids, int32_t n, int64_t slice_bytes,
                        const uint8_t *staging)
{
    for (int32_t i = 0; i < n; ++i)
        for (int32_t p = 0; p < n_planes; ++p)
            memcpy(planes[p] + (int64_t)block_ids[i] * block_stride,
                   staging + ((int64_t)i * n_planes + p) * slice_bytes, (size_t)slice_bytes);
}

/* ---------------------------------------- stage 3 -> 4 glue: resident remap
 *
 * GSAPrefetchEngineC::GetHitAndMissBlock / RunPrefetchH2D / RunOneBsPrefetch /
 * LoadKVToHBM (ucm/sparse/gsa/prefetch/src/kvcache_pre.cpp:206-322), for one
 * (request, layer).  State: the request owns n_slots HBM blocks, slot s has
 * physical id slot_phys[s] (ascending, the iteration order of the reference's
 * std::map mBlocksMap) and holds logical block slot_logical[s] (-1 = nothing;
 * together mBlocksMap/mDocsTables); slot_free[s] != 0 marks the slots on the
 * free list the previous round left behind (mFreeBlock).
 * Round: every selected logical block that is resident is a hit and stays
 * (:216-227); the misses, in selection order, take the free-listed slots that
 * are not hits now, in list order (:249-265), and the maps are updated
 * (:313-322); the new free list is every slot that is neither hit nor newly
 * filled (:298-307).  `selected` must be ascending (TopKImpl sorts its output),
 * so that table[] is the block table in the reference's order (its
 * std::map hitBlocksIdx iterates by logical index, :291-296).
 * Outputs: table[j] = physical id serving selected[j] (-1 when no slot was
 * left), load_logical/load_phys = the (miss -> block) load list; returns the
 * number of loads.
 */
int32_t orc_remap_resident(int32_t *slot_logical, uint8_t *slot_free, const int32_t *slot_phys,
                           int32_t n_slots, const int32_t *selected, int32_t n_sel, int32_t *table,
                           int32_t *load_logical, int32_t *load_phys)
{
    uint8_t *hit = (uint8_t *)calloc((size_t)(n_slots > 0 ? n_slots : 1), 1);
    for (int32_t j = 0; j < n_sel; ++j) {
        table[j] = -1;
        if (selected[j] < 0) continue;
        for (int32_t s = 0; s < n_slots; ++s)
            if (slot_logical[s] == selected[j]) {
                table[j] = slot_phys[s];
                hit[s] = 1;
                break;
            }
    }
    int32_t n_load = 0, s = 0;
    for (int32_t j = 0; j < n_sel; ++j) {
        if (table[j] != -1 || selected[j] < 0) continue;
        while (s < n_slots && (!slot_free[s] || hit[s])) ++s;
        if (s >= n_slots) break;
        hit[s] = 1;
        slot_logical[s] = selected[j];
        table[j] = slot_phys[s];
        load_logical[n_load] = selected[j];
        load_phys[n_load] = slot_phys[s];
        ++n_load;
        ++s;
    }
    for (int32_t i = 0; i < n_slots; ++i) slot_free[i] = hit[i] ? 0 : 1;
    free(hit);
    return n_load;
}

/* Byte offset of one rank's K (or V) slice of one layer inside a stored block:
 * get_offset, ucm/sparse/esa/esa.py:124-135. */
int64_t orc_store_offset(int32_t block_tokens, int32_t heads_per_rank, int32_t head_dim,
                         int32_t rank, int32_t tp_size, int32_t elem_bytes, int32_t layer,
                         int32_t is_v, int32_t is_mla)
{
    int64_t k_sz = (int64_t)block_tokens * heads_per_rank * head_dim * elem_bytes;
    int64_t v_sz = is_mla ? 0 : k_sz;
    int64_t layer_sz = (k_sz + v_sz) * tp_size;
    int64_t k_off = is_mla ? layer_sz * layer : layer_sz * layer + layer_sz / tp_size * rank;
    return is_v ? k_off + k_sz : k_off;
}

/* ------------------------------------------------------------------------------------------
 * KVStar: multi-query softmax-vote retrieval.
 * ------------------------------------------------------------------------------------------ */

/* IEEE half -> float, every class of value (the reference's scalar path has the same table-free
 * conversion, ucm/sparse/kvstar/retrieve/core/domain/retrieve_task/simd_compute_kernel.cpp:773-813;
 * its AVX2 path uses vcvtph2ps, which is this function in hardware). */
static inline float f16_to_f32(uint16_t h)
{
    uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1fu, m = h & 0x3ffu, bits;
    if (e == 0) {
        if (m == 0) {
            bits = s;
        } else {
            int sh = 0;
            while (!(m & 0x400u)) { m <<= 1; ++sh; }
            bits = s | ((uint32_t)(127 - 15 - sh + 1) << 23) | ((m & 0x3ffu) << 13);
        }
    } else if (e == 31) {
        bits = s | 0x7f800000u | (m << 13);
    } else {
        bits = s | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* float -> IEEE half, round to nearest even (what torch's .to(float16) does) */
static inline uint16_t f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t s = (x >> 16) & 0x8000u, a = x & 0x7fffffffu;
    if (a >= 0x7f800000u) return (uint16_t)(s | 0x7c00u | ((a > 0x7f800000u) ? 0x200u : 0));
    if (a >= 0x477ff000u) return (uint16_t)(s | 0x7c00u);              /* rounds to infinity */
    if (a < 0x33000001u) return (uint16_t)s;                           /* below half the smallest subnormal */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7fffffu) | 0x800000u;
    int shift = e < -14 ? (13 + (-14 - e)) : 13;
    uint32_t half = m >> shift, rem = m & ((1u << shift) - 1u), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1u))) ++half;
    if (e < -14) return (uint16_t)(s | half);                         /* subnormal (may carry into the normal range) */
    return (uint16_t)(s | (((uint32_t)(e + 15) << 10) + (half - 0x400u)));
}

uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

/* Block representations (extract_block_repre, ucm/sparse/kvstar/multistep.py:279-316, and the cast
 * of :495-499): keep the d_pruned listed channels of every head, average each run of `merge`
 * consecutive tokens in the cache's dtype (fp32 sum in token order times the fp32 reciprocal, rounded
 * to bf16, which is how torch reduces a bf16 tensor on the GPU), then cast to half.
 * k: bf16 bits, element (block, token, head, d) at block*block_stride + token*token_stride + head*D + d.
 * out: half bits [n][T/merge][H][d_pruned].  pruned == NULL keeps all D channels (d_pruned == D). */
void orc_kvstar_block_repre(const uint16_t *k, int64_t block_stride, int64_t token_stride,
                            int32_t T, int32_t H, int32_t D, const int32_t *ids, int32_t n,
                            const int64_t *pruned, int32_t d_pruned, int32_t merge, uint16_t *out)
{
    const int32_t M = T / merge;
    const float inv = 1.0f / (float)merge;
    for (int32_t i = 0; i < n; ++i)
        for (int32_t m = 0; m < M; ++m)
            for (int32_t h = 0; h < H; ++h)
                for (int32_t dp = 0; dp < d_pruned; ++dp) {
                    const int64_t d = pruned ? pruned[(int64_t)h * d_pruned + dp] : dp;
                    float acc = 0.0f;
                    for (int32_t c = 0; c < merge; ++c)
                        acc += bf16_to_f32(k[(int64_t)ids[i] * block_stride + (int64_t)(m * merge + c) * token_stride + (int64_t)h * D + d]);
                    out[(((int64_t)i * M + m) * H + h) * d_pruned + dp] = f32_to_f16(bf16_to_f32(f32_to_bf16(acc * inv)));
                }
}

/* Vote scores of one request (the scalar path of KVStar::Execute, simd_compute_kernel.cpp:816-960,
 * stopping before its top-k): raw dot products of every query row (x tokens x Hq heads) with the
 * representations of its KV head over all S = n*M positions, a softmax over S per row, and per
 * block the sum of its M probabilities over all rows.  q: half [x][Hq][d_orig]; reps: half
 * [n][M][H][d_pruned]; pruned: [H][d_pruned] channel indices into d_orig or NULL; out: float [n].
 * scratch: x*Hq*n*M floats. */
void orc_kvstar_scores(const uint16_t *q, int32_t x, int32_t Hq, int32_t d_orig, const uint16_t *reps,
                       int32_t n, int32_t M, int32_t H, int32_t d_pruned, const int64_t *pruned,
                       float *scratch, float *out)
{
    const int32_t g = Hq / H;
    const int64_t S = (int64_t)n * M;
    for (int32_t t = 0; t < x; ++t)
        for (int32_t h = 0; h < H; ++h)
            for (int32_t gg = 0; gg < g; ++gg) {
                const int32_t head = h * g + gg;
                const uint16_t *qv = q + ((int64_t)t * Hq + head) * d_orig;
                float *row = scratch + ((int64_t)t * Hq + head) * S;
                for (int64_t s = 0; s < S; ++s) {
                    const uint16_t *kv = reps + (s * H + h) * d_pruned;
                    float score = 0.0f;
                    for (int32_t d = 0; d < d_pruned; ++d) {
                        const int64_t dq = pruned ? pruned[(int64_t)h * d_pruned + d] : d;
                        score += f16_to_f32(qv[dq]) * f16_to_f32(kv[d]);
                    }
                    row[s] = score;
                }
            }
    for (int64_t r = 0; r < (int64_t)x * Hq; ++r) {
        float *row = scratch + r * S;
        float mx = row[0], sum = 0.0f;
        for (int64_t s = 1; s < S; ++s)
            if (row[s] > mx) mx = row[s];
        for (int64_t s = 0; s < S; ++s) {
            row[s] = expf(row[s] - mx);
            sum += row[s];
        }
        if (sum > 1e-9f)
            for (int64_t s = 0; s < S; ++s) row[s] /= sum;
    }
    for (int32_t b = 0; b < n; ++b) out[b] = 0.0f;
    for (int64_t r = 0; r < (int64_t)x * Hq; ++r)
        for (int64_t s = 0; s < S; ++s) out[s / M] += scratch[r * S + s];
}

/* The k highest-voted blocks, best first; equal scores go to the lower index here (the reference's
 * heap and nth_element variants leave the order of ties, and of the result, unspecified:
 * simd_compute_kernel.cpp:748-755,962-979).  Returns the count written. */
int32_t orc_kvstar_topk(const float *scores, int32_t n, int32_t k, int64_t *out)
{
    if (k > n) k = n;
    if (k <= 0) return 0;
    orc_pair *p = (orc_pair *)malloc((size_t)n * sizeof(orc_pair));
    for (int32_t i = 0; i < n; ++i) { p[i].s = scores[i]; p[i].i = i; }
    qsort(p, (size_t)n, sizeof(orc_pair), cmp_desc_stable);
    for (int32_t i = 0; i < k; ++i) out[i] = p[i].i;
    free(p);
    return k;
}

/* GSA's on-device scoring variant (cal_topk, ucm/sparse/gsa/gsa.py:386-412): every query head is dotted
 * with the representatives of its KV head, the maximum over a block's n_rep representatives is taken
 * per QUERY head, and the block's weight is the mean over query heads; blocks flagged in include_mask
 * weigh +inf, those in exclude_mask -inf (exclude wins: it is applied last).  No softmax scale is applied
 * (the reference computes one and leaves it unused).  Computed in fp32 here; the reference's tensors are
 * in the model dtype, so its own result carries bf16 rounding on top.
 * q: bf16 bits [n_req][Hq][D]; reps: fp32 [n_slots][H][n_rep][D]; masks: one byte per candidate or NULL. */
void orc_score_dot_gsa_heads(const float *reps, int32_t n_kv_heads, int32_t n_rep, int32_t head_dim,
                             const int32_t *req_offsets, const int32_t *slot_ids, int32_t n_req,
                             const uint16_t *q, int32_t n_q_heads, const uint8_t *include_mask,
                             const uint8_t *exclude_mask, float *out)
{
    const int32_t g = n_q_heads / n_kv_heads;
    for (int32_t r = 0; r < n_req; ++r)
        for (int32_t c = req_offsets[r]; c < req_offsets[r + 1]; ++c) {
            const int32_t slot = slot_ids ? slot_ids[c] : c;
            float acc = 0.0f;
            if (slot < 0) {
                out[c] = -INFINITY;
                continue;
            }
            for (int32_t i = 0; i < n_q_heads; ++i) {
                const int32_t h = i / g;
                const uint16_t *qv = q + ((int64_t)r * n_q_heads + i) * head_dim;
                float best = -INFINITY;
                for (int32_t m = 0; m < n_rep; ++m) {
                    const float *kv = reps + (((int64_t)slot * n_kv_heads + h) * n_rep + m) * head_dim;
                    float dot = 0.0f;
                    for (int32_t d = 0; d < head_dim; ++d) dot += bf16_to_f32(qv[d]) * kv[d];
                    if (dot > best) best = dot;
                }
                acc += best;
            }
            float w = acc / (float)n_q_heads;
            if (include_mask && include_mask[c]) w = INFINITY;
            if (exclude_mask && exclude_mask[c]) w = -INFINITY;
            out[c] = w;
        }
}

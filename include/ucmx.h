/*
 * ucmx — C ABI of the B200 (sm_100a) sparse-KV retrieval and block-transfer library.
 *
 * Plain C: raw pointers, sizes and a CUDA stream handle; no C++ or framework types cross this
 * boundary.  Every function returns an int32 status and never throws or aborts:
 *     0        OK
 *    -1        generic failure (a CUDA launch or runtime call failed, a wait timed out)
 *    -50000    invalid parameter          -50001  out of memory
 *    -50002    OS / CUDA runtime error    -50005  object not found
 *    -50008    unsupported configuration
 * These are the values of UC::Status in the reference (ucm/store/infra/status/status.h:32-45).
 *
 * Unless a comment says "host", every pointer is a device pointer valid on the device that owns
 * `stream`.  All launches are asynchronous on `stream`; nothing here synchronises unless stated.
 * "Reference" paths are relative to the UCM project root.
 */
#ifndef UCMX_H
#define UCMX_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define UCMX_OK 0
#define UCMX_ERROR (-1)
#define UCMX_EPARAM (-50000)
#define UCMX_EOOM (-50001)
#define UCMX_EOSERROR (-50002)
#define UCMX_EDUPLICATE (-50003)
#define UCMX_ENOOBJ (-50005)
#define UCMX_EUNSUPPORTED (-50008)

typedef void* ucmx_stream_t; /* a cudaStream_t */

/* Layout of one layer's paged K (or V) cache of bf16 elements: element (block, token, head, d) is
 * at block*block_stride + token*token_stride + head*head_dim + d (strides in elements).  This is
 * vLLM's [num_blocks, block_size, num_kv_heads, head_size] cache, the tensor the reference indexes
 * as k_cache[ids] (ucm/sparse/esa/esa.py:265-266). */
typedef struct ucmx_kv_geometry {
    int64_t block_stride;
    int64_t token_stride;
    int32_t block_tokens;
    int32_t n_kv_heads;
    int32_t head_dim;
    int32_t reserved; /* number of blocks in the cache (required): a block id at or beyond it is dropped and reported
                         (ucmx_device_error code 3), never turned into an address; also sizes the tensor maps */
} ucmx_kv_geometry;

/* Library version and the SM architecture the kernels were compiled for (100 for sm_100a). */
int32_t ucmx_version(void);
int32_t ucmx_compiled_arch(void);
/* Text of the last CUDA error this thread's calls met ("" if none). Host. */
const char* ucmx_last_error(void);
/* Kernels never spin without limit: a wait on an asynchronous copy that does not complete gives
 * up and records a code here instead of hanging the device, and an id that points outside the
 * table or cache it indexes is skipped and recorded instead of dereferenced:
 *   1 = a bulk copy did not land, 2 = a misaligned pointer pair was skipped, 3 = a slot or block id
 *   was outside its table (the entry was treated as empty), 4 = a tensor-parallel peer never
 *   delivered its scores.  Reads the code (0 = none) and optionally clears it. */
int32_t ucmx_device_error(int32_t* code, int32_t clear);

/* ---------------------------------------------------------------------------------------------
 * Stage 1a — per-block key representatives by pooling.
 * Replaces: `k_cache[ids].mean(1)` (ucm/sparse/esa/esa.py:265-266), GSA `copy_k`
 * (ucm/sparse/gsa/gsa.py:640-652), KRepreComputer::ComputeKRepreBlock
 * (ucm/sparse/gsa/offload_ops/src/k_repre.cpp:15-35) with VectorMeanImpl
 * (.../vec_product.cpp:39-85), and the max/min/sum chunk_repre_method variants
 * (ucm/sparse/kvcomp/kvcomp_config.py:56,116-120).
 *
 * For i in [0,n): rep = reduce over the tokens of block block_ids[i]; written to row
 * out_slots[i] (or i when out_slots is NULL) of a table laid out [slot, n_kv_heads, n_rep, head_dim]
 * at representative index rep_index.  mode: 0 mean, 1 max, 2 min, 3 sum.  Tokens are accumulated in
 * fp32 in token order; the mean is sum*(1/block_tokens).  round_bf16 != 0 rounds the result to bf16
 * (nearest even) before it is stored, which is what the reference keeps; out_f32 then receives the
 * widened bf16 value.  Either of out_bf16 / out_f32 may be NULL.  n_out_slots is the number of rows
 * of the output table: a row index at or beyond it (like a block id beyond the cache) drops the entry
 * and is reported (code 3). */
#define UCMX_POOL_MEAN 0
#define UCMX_POOL_MAX 1
#define UCMX_POOL_MIN 2
#define UCMX_POOL_SUM 3
int32_t ucmx_pool_blocks(const void* k_cache, const ucmx_kv_geometry* geom /* host */,
                         const int32_t* block_ids, const int32_t* out_slots, int64_t n_out_slots, int32_t n, int32_t mode,
                         int32_t round_bf16, int32_t n_rep, int32_t rep_index, void* out_bf16,
                         float* out_f32, ucmx_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Stage 1b — KVComp sign-bit hash codes.
 * Replaces: HashEncoder.compute_hash (ucm/sparse/kvcomp/hash_encoder.py:99-157) and its use on key
 * blocks, extract_block_repre + transpose (ucm/sparse/kvcomp/kvcomp.py:314-318,342).
 *
 * Bit j of vector x is (sum_d x[d]*W[d][j] > 0), the sum taken as an fp32 fused-multiply-add chain
 * over d = 0..dim-1; bits are packed LSB first (bit 8b+i is bit i of byte b).
 * ucmx_hash_encode: x is bf16 [n_vec, dim] with row stride x_stride elements; out is
 *   uint8 [n_vec, bits/8].
 * ucmx_hash_encode_blocks: vectors are the (token, head) rows of paged blocks block_ids[i]; codes
 *   of block i go to row out_slots[i] (or i) of a table uint8 [slot, n_kv_heads, block_tokens,
 *   bits/8] when head_major != 0 (the layout KVComp keeps) or [slot, block_tokens, n_kv_heads,
 *   bits/8] when head_major == 0 (compute_hash's own output order).
 * w is bf16 [dim, bits] row major.  dim and bits must be multiples of 32; dim = head_dim.
 * n_out_slots: rows of the code table (bounds out_slots, as in ucmx_pool_blocks). */
int32_t ucmx_hash_encode(const void* x, int64_t n_vec, int64_t x_stride, const void* w, int32_t dim,
                         int32_t bits, uint8_t* out, ucmx_stream_t stream);
int32_t ucmx_hash_encode_blocks(const void* k_cache, const ucmx_kv_geometry* geom /* host */,
                                const int32_t* block_ids, const int32_t* out_slots, int64_t n_out_slots, int32_t n,
                                const void* w, int32_t bits, int32_t head_major, uint8_t* out,
                                ucmx_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Stage 2 prologue — per-KV-head query mean.
 * Replaces: `query.view(ntok, kvH, -1, D).mean(2)` + fp32 cast (ucm/sparse/esa/esa.py:291-296,
 * ucm/sparse/esa/retrieval/retrieval_worker.py:15-20) and TopkBlockSelector::ComputeQHeadMean
 * (ucm/sparse/gsa/offload_ops/src/select_topk_block.cpp:101-114).
 * q is bf16 [n_tok, n_q_heads, head_dim], tok_stride elements between tokens; out is fp32
 * [n_tok, n_kv_heads*head_dim].  round_bf16 != 0 rounds each mean to bf16 first (the ESA/KVComp
 * behaviour); 0 keeps fp32 (the GSA native behaviour).  If n_q_heads < n_kv_heads heads repeat. */
int32_t ucmx_query_group_mean(const void* q, int32_t n_tok, int32_t n_q_heads, int32_t n_kv_heads,
                              int32_t head_dim, int64_t tok_stride, int32_t round_bf16, float* out,
                              ucmx_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Stage 2a — query-to-block dot scores over a ragged batch.
 * Replaces: the scoring loop of RetrievalWorkerBackend::worker_loop
 * (ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp:170-181) and
 * TopkBlockSelector::ComputeBlockScore / ComputeKQDotScores
 * (ucm/sparse/gsa/offload_ops/src/select_topk_block.cpp:53-99).
 *
 * Request r owns candidates [req_offsets[r], req_offsets[r+1]) (req_offsets has n_req+1 entries,
 * total = req_offsets[n_req]).  Candidate c reads table row slot_ids[c] (or c if slot_ids is NULL);
 * a negative slot id scores -inf.  The table is [slot, n_kv_heads, n_rep, head_dim], bf16
 * (reps_dtype 0) or fp32 (reps_dtype 1).  q is fp32 [n_req, n_kv_heads*head_dim].
 * score = scale * sum_h max_r dot(q[r,h,:], rep[slot,h,r,:]); with n_rep == 1 that is the plain
 * dot product over n_kv_heads*head_dim the ESA backend takes. */
#define UCMX_DT_BF16 0
#define UCMX_DT_F32 1
#define UCMX_DT_I32 2
/* Tensor-parallel ranks pass `exchange` (host pointer; NULL on a single rank): the kernel then also
 * delivers its partial scores to every rank, see "Tensor-parallel retrieval" below; out_scores may
 * be NULL in that case.  n_slots is the number of rows of the table: a slot id at or beyond it is
 * treated as an empty entry (-inf) and reported through ucmx_device_error (code 3), never read. */
typedef struct ucmx_peer_exchange {
    void* const* bases; /* DEVICE array of `world` exchange-buffer addresses, in rank order */
    int32_t world;
    int32_t my_rank;
    int64_t n_scores;   /* scores a rank's part of the inbox holds (>= total of every call) */
} ucmx_peer_exchange;
int32_t ucmx_score_dot(const void* reps, int32_t reps_dtype, int64_t n_slots, int32_t n_kv_heads,
                       int32_t n_rep, int32_t head_dim, const int32_t* req_offsets,
                       const int32_t* slot_ids, const float* q, int32_t n_req, int32_t total,
                       float scale, float* out_scores, const ucmx_peer_exchange* exchange /* host */,
                       ucmx_stream_t stream);

/* Early start for the dot-scoring calls (ucmx_score_dot, ucmx_score_dot_query) the calling thread makes from now
 * on (on != 0) or no longer (on == 0); returns the previous setting.  With it a scoring kernel is launched so that
 * it may begin while the kernel ahead of it in the stream is still running (programmatic dependent launch, also
 * inside a stream capture): it reads the table, the slot list, the offsets and the queries right away and waits
 * for that kernel's end only before it stores its first score.  The caller promises that none of those four
 * inputs is written by the kernel ahead; out_scores may be (a top-k that still reads the previous scores is the
 * usual case).  Calls with an `exchange`, and shapes that do not take the row-ring kernel, are launched as ever. */
int32_t ucmx_set_early_start(int32_t on);

/* GSA's device-side weights (cal_topk, ucm/sparse/gsa/gsa.py:386-412): weight of a block = mean over the
 * QUERY heads of max over the block's n_rep representatives of dot(query head, representative of its KV
 * head); no softmax scale (the reference computes one and does not apply it).  query is raw bf16
 * [n_req, n_q_heads, head_dim], query_stride elements between requests; the table is bf16
 * [slot, n_kv_heads, n_rep, head_dim].  include_mask / exclude_mask: one byte per candidate (device), or
 * NULL; a set include byte gives +inf, a set exclude byte -inf (exclude wins), as masked_fill_ does there.
 * n_q_heads / n_kv_heads must be a power of two <= 32.  Computed in fp32. */
int32_t ucmx_score_dot_heads(const void* reps, int64_t n_slots, int32_t n_kv_heads, int32_t n_rep,
                             int32_t head_dim, const int32_t* req_offsets, const int32_t* slot_ids, const void* query,
                             int32_t n_q_heads, int64_t query_stride, int32_t n_req, int32_t total,
                             const uint8_t* include_mask, const uint8_t* exclude_mask,
                             float* out_scores, ucmx_stream_t stream);

/* Stages 2-prologue and 2a in one launch: `query` is the raw bf16 decode query [n_req, n_q_heads,
 * head_dim] (query_stride elements between requests); the per-KV-head mean of
 * ucmx_query_group_mean (same arithmetic, same round_bf16 switch) is taken inside the scoring
 * kernel.  n_rep is 1.  Returns UCMX_EUNSUPPORTED for shapes the single-pass kernel does not cover
 * (n_kv_heads*head_dim not a multiple of 256 for bf16 tables / 128 for fp32 tables, or above 2048);
 * use the two calls above then. */
int32_t ucmx_score_dot_query(const void* reps, int32_t reps_dtype, int64_t n_slots, int32_t n_kv_heads,
                             int32_t head_dim, const int32_t* req_offsets, const int32_t* slot_ids,
                             const void* query, int32_t n_q_heads, int64_t query_stride,
                             int32_t round_bf16, int32_t n_req, int32_t total, float scale,
                             float* out_scores, const ucmx_peer_exchange* exchange /* host */,
                             ucmx_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Stage 2b — Hamming-similarity scores on packed hash codes (integer exact).
 * Replaces: HashEncoder._unpack_hash + einsum("tid,njsd->tijsn") + sum
 * (ucm/sparse/kvcomp/hash_encoder.py:159-219, ucm/sparse/kvcomp/kvcomp.py:233-247).
 *
 * codes is uint8 [slot, n_kv_heads, block_tokens, bits/8]; q_codes is uint8 [n_req, n_q_heads,
 * bits/8].  score = sum over (i, j, s) of (bits - 2*popcount(q_i xor k_{j,s})) over every
 * (query head i, key head j) pair when cross_head != 0 (what the reference's einsum does), or over
 * matching heads only (i == j, needs n_q_heads == n_kv_heads) when cross_head == 0.
 * bits must be a multiple of 128.  Ragged batch, slot_ids and n_slots (rows of the code table) as in
 * ucmx_score_dot; a candidate without a valid slot scores INT32_MIN. */
int32_t ucmx_score_hamming(const uint8_t* codes, int64_t n_slots, int32_t n_kv_heads, int32_t block_tokens,
                           int32_t bits, const int32_t* req_offsets, const int32_t* slot_ids,
                           const uint8_t* q_codes, int32_t n_q_heads, int32_t n_req, int32_t total,
                           int32_t cross_head, int32_t* out_scores, ucmx_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Stage 3 — per-request top-k over a ragged batch (radix select, one thread block per request).
 * Replaces: std::partial_sort in RetrievalWorkerBackend::worker_loop (retrieval_backend.cpp:182-189),
 * TopkBlockSelector::TopKImpl (select_topk_block.cpp:20-51), and torch.topk + sort
 * (ucm/sparse/kvcomp/kvcomp.py:249-254).
 *
 * scores: fp32 (score_dtype UCMX_DT_F32) or int32 (UCMX_DT_I32), flat, ragged by req_offsets.
 * k_per_req[r]: how many to select for request r.
 * window_mode:
 *   UCMX_WIN_NONE    plain top-k of all candidates (ESA); returns min(k, n) entries.
 *   UCMX_WIN_FORCE   GSA TopKImpl: positions [0,start_win) and [n-end_win,n) are always selected
 *                    and count toward k; the other k-start-end come from the middle.  If
 *                    start+end >= n, k >= n or k == 0 every position is returned (identity).
 *   UCMX_WIN_EXCLUDE KVComp: candidates are positions [start_win, n-end_win); min(k, size) of them
 *                    are returned; if k >= n all of them are.  (KVComp's init_window_sz and
 *                    local_window_sz-1.)
 * order: UCMX_ORDER_SCORE_DESC (best first; needs k <= 8192) or UCMX_ORDER_INDEX_ASC.
 * Equal scores: the candidate with the lower position wins (the reference's stable_sort does the
 * same; partial_sort and torch.topk leave it unspecified).  -0.0 and +0.0 compare equal.
 * Output row r starts at r*out_stride and holds at most out_stride entries; or, when out_offsets
 * (n_req+1 entries) is given, it starts at out_offsets[r] and holds at most
 * out_offsets[r+1]-out_offsets[r] (<= out_stride) entries, which packs the rows back to back.
 * Entries beyond out_counts[r] are left untouched.  out_idx[j] is the candidate's position within
 * its request, or id_map[req_offsets[r]+position] when id_map is given.  out_scores (same dtype as
 * scores) may be NULL.
 * The kernel is launched with programmatic stream serialization and waits for the end of the kernel
 * ahead of it before it reads anything: stream order is what it always was, only the kernel's
 * placement on the SMs overlaps the tail of the scoring kernel in front of it. */
#define UCMX_WIN_NONE 0
#define UCMX_WIN_FORCE 1
#define UCMX_WIN_EXCLUDE 2
#define UCMX_ORDER_SCORE_DESC 0
#define UCMX_ORDER_INDEX_ASC 1
int32_t ucmx_topk_ragged(const void* scores, int32_t score_dtype, const int32_t* req_offsets,
                         const int32_t* k_per_req, int32_t n_req, int32_t start_win, int32_t end_win,
                         int32_t window_mode, int32_t order, const int32_t* id_map,
                         int32_t out_stride, const int32_t* out_offsets, int32_t* out_idx,
                         void* out_scores, int32_t* out_counts, ucmx_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Tensor-parallel retrieval: the all-reduce of partial block scores, fused into the scoring and
 * top-k kernels over peer memory.  (No counterpart in the reference, which has no cross-rank
 * exchange: under tensor parallelism its ranks select independently over their own KV heads,
 * ucm/sparse/esa/esa.py:196-198.)
 *
 * Every rank owns an exchange buffer of ucmx_peer_exchange_bytes(world, n_scores) bytes that all
 * ranks can address (peer-mapped, e.g. torch symmetric memory), zeroed once before its first use:
 * a 256-byte header (one flag per rank, this rank's arrival and round counters) and an inbox of
 * two halves x world parts of partial scores.  A round:
 *   1. ucmx_score_dot / ucmx_score_dot_query with `exchange` set: the rank scores its own KV heads
 *      and stores every score into inbox[round & 1][my_rank] of EVERY rank (plain peer stores); the
 *      kernel's last thread block then publishes the round number into flag[my_rank] of every rank
 *      (release at system scope: the scores stored before are visible to whoever sees the flag).
 *   2. ucmx_topk_ragged_peer_sum, next on the same stream: waits until all `world` flags of its own
 *      buffer have reached the round, adds the parts in rank order (local loads; the same order
 *      everywhere, so every rank gets bit-identical sums and selections), writes the sums to
 *      summed_scores and selects as ucmx_topk_ragged does.
 * The round number lives in the buffer and advances by itself, so the two launches can be captured
 * in a CUDA graph and replayed; the halves alternate, so a fast rank never overwrites scores a
 * slower peer may still be reading.  Every rank must run the same sequence of rounds.  The wait is
 * bounded: if a peer never delivers, code 4 is recorded (ucmx_device_error) and the kernel goes on
 * with what it has instead of hanging.  No multicast and no remote loads are involved. */
size_t ucmx_peer_exchange_bytes(int32_t world, int64_t n_scores);
int32_t ucmx_topk_ragged_peer_sum(const ucmx_peer_exchange* exchange /* host */, float* summed_scores,
                                  const int32_t* req_offsets, const int32_t* k_per_req, int32_t n_req,
                                  int32_t total, int32_t start_win, int32_t end_win, int32_t window_mode,
                                  int32_t order, const int32_t* id_map, int32_t out_stride,
                                  const int32_t* out_offsets, int32_t* out_idx, float* out_scores,
                                  int32_t* out_counts, ucmx_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Stage 3 -> 4 glue — resident-set remap (the "SparseKVManager block remap").
 * Replaces: GSAPrefetchEngineC::GetHitAndMissBlock / RunPrefetchH2D / RunOneBsPrefetch / LoadKVToHBM
 * (ucm/sparse/gsa/prefetch/src/kvcache_pre.cpp:206-322) and ESA's delta logic
 * (ucm/sparse/esa/esa.py:313-334).
 *
 * State, per request r (slots [slot_offsets[r], slot_offsets[r+1])): slot_phys[s] is the physical id
 * of the s-th HBM block the request owns (ascending; a negative id marks a slot that does not
 * exist, which lets requests with different numbers of blocks share one slot stride), slot_logical[s]
 * the logical block it holds (-1 = none), slot_free[s] != 0 marks slots the previous round left on
 * the free list.
 * Selection, per request (entries [sel_offsets[r], sel_offsets[r+1]), of which only the first
 * sel_counts[r] are used when sel_counts is given; a negative count leaves the request's state and
 * outputs untouched): ascending logical block ids (negative = skip).
 * One round: a selected block that is resident keeps its slot; the others, in selection order, take
 * the free-listed slots that are not hits now, in slot order; slot_logical is updated and the new
 * free list is every slot that is neither a hit nor newly filled.
 * Outputs, packed like sel: table[j] = physical id serving sel[j] (-1 if no slot was left);
 * load_logical / load_phys = the (block to load -> HBM block) list, load_counts[r] entries from
 * position sel_offsets[r]; the entries behind them, up to sel_offsets[r+1], are set to -1, so the
 * lists of all requests can go to ucmx_move_blocks as one array.  max_logical bounds the logical
 * ids, max_slots the slots of a request (both size the shared-memory lookup; (max_logical +
 * 2*max_slots)*4 bytes must stay under 200 KiB; a request with more slots than max_slots is
 * refused: nothing loaded, table -1, code 3 for ucmx_device_error).
 * moves (optional, host pointer): also write ONE list of block moves for all requests, ready for
 * ucmx_move_blocks, when the blocks' home is a paged pool in HBM: for every block to load,
 * move_src = src_map[src_map_offsets[r] + logical block] (e.g. the request's row of the block
 * table; src_map_offsets NULL: every request starts at 0) and move_dst = the HBM block it goes to.
 * Requests append their entries at move_count[0] (atomically, so the order of requests in the list
 * is arbitrary); move_count is two int32 in device memory, both 0 before the call -
 * ucmx_move_blocks(..., n_device = move_count, ...) consumes the list and zeroes them again. */
typedef struct ucmx_remap_moves {
    const int32_t* src_map;
    const int32_t* src_map_offsets;
    int32_t* move_src;
    int32_t* move_dst;
    int32_t* move_count;
} ucmx_remap_moves;
int32_t ucmx_remap_resident(int32_t* slot_logical, uint8_t* slot_free, const int32_t* slot_phys,
                            const int32_t* slot_offsets, const int32_t* sel, const int32_t* sel_offsets,
                            const int32_t* sel_counts, int32_t n_req, int32_t max_logical,
                            int32_t max_slots, int32_t* table, int32_t* load_logical, int32_t* load_phys,
                            int32_t* load_counts, const ucmx_remap_moves* moves /* host */,
                            ucmx_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Score + top-k without any allocation.  (No counterpart in the reference: its retrieval runs on
 * host threads with std::vector scratch.)
 *
 * Same arguments and results as ucmx_score_dot followed by ucmx_topk_ragged on fp32 scores, but the
 * per-candidate scores in between live in an array that is part of the library image instead of a
 * buffer the caller provides.  It is meant for callers that cannot allocate device memory at the
 * point of the call - hooks running inside a serving engine's forward pass after the engine has
 * given nearly all of HBM to its KV cache, where cudaMalloc may fail and in any case stalls the
 * device, and callers with no tensor allocator of their own.  This function calls neither
 * cudaMalloc/cudaFree nor any allocating library routine.
 * Limits and rules:
 *  - total must not exceed ucmx_noalloc_max_candidates() (1 048 576 candidates, a 4 MiB array that
 *    every GPU which loads the library holds until the process exits); larger batches are
 *    rejected with UCMX_EUNSUPPORTED and a message in ucmx_last_error().
 *  - Every call needs the device of `stream` to be the current device.  The first call on each
 *    device also looks up the array's device address; make that first call before starting any
 *    stream capture.
 *  - Out-of-range slot ids are skipped (scored -inf) as everywhere else, but not recorded for
 *    ucmx_device_error: the word that call reads is allocated on first use.
 *  - All calls on a device share the one array and it keeps the last call's scores.  Calls are
 *    safe back to back on one stream; two calls that may overlap on the GPU (different streams
 *    without an ordering between them) race on it and must be serialised by the caller.
 *  - Only out_idx / out_scores / out_counts are results; the scores of unselected candidates are
 *    not returned. */
int32_t ucmx_retrieve_topk_noalloc(const void* reps, int32_t reps_dtype, int64_t n_slots,
                                   int32_t n_kv_heads, int32_t n_rep, int32_t head_dim,
                                   const int32_t* req_offsets,
                                   const int32_t* slot_ids, const float* q, int32_t n_req,
                                   int32_t total, float scale, const int32_t* k_per_req,
                                   int32_t start_win, int32_t end_win, int32_t window_mode,
                                   int32_t order, const int32_t* id_map, int32_t out_stride,
                                   const int32_t* out_offsets, int32_t* out_idx, float* out_scores,
                                   int32_t* out_counts, ucmx_stream_t stream);
int32_t ucmx_noalloc_max_candidates(void);

/* ---------------------------------------------------------------------------------------------
 * Stage 4 — gather / scatter of paged KV block slices.
 * Replaces: the per-block copies of UcmDramStore.load/dump
 * (ucm/store/dramstore/dramstore_connector.py:112-166), PosixQueue::S2D/D2S's memcpy leg
 * (ucm/store/nfsstore/tsf_task/posix_queue.cc:98-124) and CudaDevice::H2DBatchSync/D2HBatchSync with
 * H2DKernel/D2HKernel (ucm/store/device/cuda/cuda_device.cu:47-81,180-211).
 *
 * planes: host array of n_planes (<= 8) base pointers (K cache, V cache, ... of one layer), each
 * holding n_blocks blocks.
 * For i in [0,n), p in [0,n_planes): slice_bytes bytes at planes[p] + block_ids[i]*block_stride_bytes
 * are copied to (gather) or from (scatter) staging + (i*n_planes + p)*slice_bytes.  block_ids is a
 * device array; negative ids are skipped, and so is an id at or beyond n_blocks, which is also
 * recorded for ucmx_device_error (code 3) - it is never turned into an address.  staging may be device memory or page-locked host memory
 * mapped into the device's address space (direct zero-copy transfer); pass staging_is_host != 0 in
 * the latter case so that plain loads/stores are used instead of bulk async copies.
 * slice_bytes, block_stride_bytes and all pointers must be multiples of 16. */
int32_t ucmx_gather_blocks(const void* const* planes /* host */, int32_t n_planes,
                           int64_t block_stride_bytes, int64_t n_blocks, const int32_t* block_ids,
                           int32_t n, int64_t slice_bytes, void* staging, int32_t staging_is_host,
                           ucmx_stream_t stream);
int32_t ucmx_scatter_blocks(void* const* planes /* host */, int32_t n_planes,
                            int64_t block_stride_bytes, int64_t n_blocks, const int32_t* block_ids,
                            int32_t n, int64_t slice_bytes, const void* staging,
                            int32_t staging_is_host, ucmx_stream_t stream);
/* Block to block inside device memory: for i in [0,n), p in [0,n_planes): the slice of block
 * src_ids[i] of src_planes[p] goes to block dst_ids[i] of dst_planes[p]; an entry with a negative
 * id on either side is skipped, an id beyond its cache is skipped and recorded (code 3).  This is
 * the delta load of a decode step (ESA wait_retrieval_and_start_load, ucm/sparse/esa/esa.py:313-338;
 * GSAPrefetchEngineC::RunPrefetchH2D, ucm/sparse/gsa/prefetch/src/kvcache_pre.cpp:240-272) when
 * the blocks' home is HBM: the move list of ucmx_remap_resident goes in as it is.
 * n_device (optional, device memory, two int32): when given, only the first min(n, n_device[0])
 * entries are moved - the length of a list that was built on the device - and the kernel sets both
 * words back to 0 when it is done (n_device[1] is its scratch; both must be 0 before the list is
 * built).  n then only bounds the launch. */
int32_t ucmx_move_blocks(const void* const* src_planes /* host */, void* const* dst_planes /* host */,
                         int32_t n_planes, int64_t src_block_stride_bytes, int64_t n_src_blocks,
                         const int32_t* src_ids, int64_t dst_block_stride_bytes, int64_t n_dst_blocks,
                         const int32_t* dst_ids, int32_t n, const int32_t* n_device, int64_t slice_bytes,
                         ucmx_stream_t stream);
/* Pointer-pair form, the signature of IDevice::H2DBatchSync / D2HBatchSync
 * (ucm/store/device/idevice.h:48-51) minus the blocking allocation: dst_ptrs/src_ptrs are DEVICE
 * arrays of `number` addresses, `count` bytes each (multiple of 16). Asynchronous on stream. */
int32_t ucmx_copy_batch(void* const* dst_ptrs, const void* const* src_ptrs, int32_t number,
                        int64_t count, int32_t any_host_memory, ucmx_stream_t stream);

/* One contiguous asynchronous copy in either direction (device or page-locked host memory on both
 * ends): CudaDevice::H2DAsync / D2HAsync (ucm/store/device/cuda/cuda_device.cu:152-159).  Paired
 * with a gather into (or scatter out of) a contiguous device staging area it moves a whole batch of
 * block slices over the host link with one DMA instead of one per slice. */
int32_t ucmx_memcpy_async(void* dst, const void* src, int64_t bytes, ucmx_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Pinned host ring — IBufferedDevice::GetBuffer (ucm/store/device/ibuffered_device.h:32-62):
 * one page-locked slab cut into n_slots slots of slot_bytes, handed out by index.
 * acquire returns UCMX_ENOOBJ when no slot is free (the reference falls back to a fresh
 * cudaMallocHost; callers here wait or split the batch instead). All host-side, thread safe. */
typedef struct ucmx_ring ucmx_ring;
int32_t ucmx_ring_create(size_t slot_bytes, size_t n_slots, ucmx_ring** out);
int32_t ucmx_ring_acquire(ucmx_ring* ring, void** host_ptr, int32_t* slot_index);
int32_t ucmx_ring_release(ucmx_ring* ring, int32_t slot_index);
int32_t ucmx_ring_base(ucmx_ring* ring, void** host_ptr, size_t* slot_bytes, size_t* n_slots);
int32_t ucmx_ring_destroy(ucmx_ring* ring);

/* ---------------------------------------------------------------------------------------------
 * Transfer tasks — TaskWaiter::Wait / TaskManager::Wait / Check
 * (ucm/store/task/task_waiter.h:41-55, ucm/store/task/task_manager.cc:57-96): a task completes when
 * the work recorded on its stream so far has run.  wait returns 0 on completion, -1 on timeout or
 * CUDA failure (timeout_ms < 0 waits without limit); check never blocks. */
typedef struct ucmx_task ucmx_task;
int32_t ucmx_task_create(ucmx_task** out);
int32_t ucmx_task_record(ucmx_task* task, ucmx_stream_t stream);
int32_t ucmx_task_check(ucmx_task* task, int32_t* finished);
int32_t ucmx_task_wait(ucmx_task* task, int64_t timeout_ms);
int32_t ucmx_task_destroy(ucmx_task* task);

/* ---------------------------------------------------------------------------------------------
 * Retrieval back-end object — RetrievalWorkerBackend
 * (ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp:17-225): a table of n_items representatives
 * of `dim` fp32 values; submit(query[b,dim], topk, indexes[b,max_idx] with -1 padding) -> request
 * id; poll / wait / get_result(indices int32[b,topk], scores fp32[b,topk]).
 * Here the table lives on the device (kept as bf16 when table_dtype == UCMX_DT_BF16, which is
 * lossless for bf16-rounded representatives, else fp32) and requests are served by a stream-ordered
 * score + top-k on a private stream instead of jobs for a thread pool.  Submits are coalesced: a
 * submit stores its query rows and index lists in page-locked memory and returns; everything
 * submitted since the last launch goes to the GPU as ONE ragged batch when any of those requests
 * is polled, waited for or collected, when ucmx_retrieval_flush is called, or when 2048 query rows
 * (or 4 Mi candidates) have piled up.  ESA's pattern - one submit per request of the decode batch,
 * then one wait per request (ucm/sparse/esa/esa.py:286-339) - thus costs one launch per layer.
 * submit refuses (UCMX_EPARAM) an index below -1 or at or beyond n_items.
 * Pointers named host_* are host memory; get_result copies min(topk, n_allowed) entries per row and
 * pads the rest of the row with -1 / -inf, then forgets the request (as the reference does). */
typedef struct ucmx_retrieval ucmx_retrieval;
int32_t ucmx_retrieval_create(const float* host_data, int64_t n_items, int32_t dim,
                              int32_t table_dtype, int32_t device, ucmx_retrieval** out);
/* Overwrite rows slots[i] of the table with host_rows[i] (fp32 [n, dim]); stream-ordered with
 * later submits. */
int32_t ucmx_retrieval_update_rows(ucmx_retrieval* r, const int32_t* host_slots, int32_t n,
                                   const float* host_rows);
/* Device pointer of the table, for kernels (e.g. ucmx_pool_blocks) that fill it in place. */
int32_t ucmx_retrieval_table(ucmx_retrieval* r, void** table, int32_t* table_dtype);
int32_t ucmx_retrieval_submit(ucmx_retrieval* r, const float* host_query, int32_t batch,
                              int32_t query_dim, int32_t topk, const int32_t* host_indexes,
                              int32_t max_idx, int32_t* req_id);
int32_t ucmx_retrieval_flush(ucmx_retrieval* r); /* launch what has been submitted so far */
int32_t ucmx_retrieval_launches(ucmx_retrieval* r, int64_t* kernels); /* kernels launched so far */
int32_t ucmx_retrieval_poll(ucmx_retrieval* r, int32_t req_id, int32_t* ready);
int32_t ucmx_retrieval_wait(ucmx_retrieval* r, int32_t req_id);
int32_t ucmx_retrieval_result_shape(ucmx_retrieval* r, int32_t req_id, int32_t* batch,
                                    int32_t* topk);
int32_t ucmx_retrieval_get_result(ucmx_retrieval* r, int32_t req_id, int32_t* host_indices,
                                  float* host_scores);
int32_t ucmx_retrieval_destroy(ucmx_retrieval* r);

/* ---------------------------------------------------------------- file-per-block store data plane
 * Replaces UC::NFSStore (ucm/store/nfsstore/cc/api/nfsstore.h:34-91) for block files and slice
 * transfer: SpaceManager::NewBlock/CommitBlock/LookupBlock (nfsstore/cc/domain/space/space_manager.cc:57-134),
 * the shard layout data/<first 8 id bytes, %016x>/<next 8 id bytes, %016x>.dat with ".act" (or temp/...)
 * until commit (space_shard_layout.cc:51-126, space_shard_temp_layout.cc:29-54), task submit/wait/check
 * (ucm/store/task/task_manager.cc:28-104) and PosixQueue::S2D/D2S/S2H/H2S (trans/posix_queue.cc:98-138).
 * Block ids are byte strings of at least 16 bytes; the first 16 name the file.  The storage backend of
 * a block is backends[std::hash<std::string>(id) % n], as in the reference (same C++ runtime).
 * Hotness tracking (utime touches on lookup) is not part of this data plane. */
typedef struct ucmx_fstore ucmx_fstore;
#define UCMX_FSTORE_DUMP 0
#define UCMX_FSTORE_LOAD 1
#define UCMX_FSTORE_HOST 0
#define UCMX_FSTORE_DEVICE 1
/* backends: ':'-separated directories (the first gets data/ [and temp/] created, the others must hold
 * them already).  transfer_enable = 0 builds a store that only manages block files (scheduler role).
 * device_id < 0: host-memory transfers only.  io_size: bytes per staging slot (262144 in the
 * reference); slots_per_worker (0 = 16) page-locked slots for each of worker_number (0 = 8) threads;
 * timeout_ms (0 = 30000) bounds ucmx_fstore_wait. */
int32_t ucmx_fstore_create(const char* backends, size_t block_size, int32_t temp_dump_dir,
                           int32_t transfer_enable, int32_t device_id, size_t io_size,
                           size_t slots_per_worker, size_t worker_number, size_t timeout_ms,
                           ucmx_fstore** out);
int32_t ucmx_fstore_destroy(ucmx_fstore* store);
/* path of the block's file: activated != 0 = while being written, 0 = committed */
int32_t ucmx_fstore_path(const ucmx_fstore* store, const char* id, size_t id_len, int32_t activated,
                         char* out, size_t capacity);
/* creates the block's file at block_size bytes; UCMX_EDUPLICATE if it exists committed or in progress */
int32_t ucmx_fstore_alloc(ucmx_fstore* store, const char* id, size_t id_len);
int32_t ucmx_fstore_lookup(const ucmx_fstore* store, const char* id, size_t id_len, int32_t* found);
/* success != 0: publish (rename to .dat), UCMX_ENOOBJ if nothing was in progress; 0: discard */
int32_t ucmx_fstore_commit(ucmx_fstore* store, const char* id, size_t id_len, int32_t success);
/* n slices: bytes [offsets[i], offsets[i]+lengths[i]) of block ids[i]'s file <-> addresses[i] (host
 * or device memory by `location`).  Dumps write the in-progress file, loads read the committed one.
 * Returns at once with a task id (> 0); the caller's buffers stay borrowed until wait returns. */
int32_t ucmx_fstore_submit(ucmx_fstore* store, int32_t type, int32_t location, const char* const* ids,
                           const size_t* id_lens, const size_t* offsets, const uintptr_t* addresses,
                           const size_t* lengths, size_t n, size_t* task_id);
/* 0 when every slice moved; UCMX_ERROR if any failed or the timeout passed (the call still returns
 * only after the workers have let go of the buffers); UCMX_ENOOBJ for an unknown or already waited id */
int32_t ucmx_fstore_wait(ucmx_fstore* store, size_t task_id);
int32_t ucmx_fstore_check(ucmx_fstore* store, size_t task_id, int32_t* finished);

/* ---------------------------------------------------------------- KVStar softmax-vote retrieval
 * Replaces kvstar_retrieve.AsyncRetrieveByCPU -> KVStar::Execute
 * (ucm/sparse/kvstar/retrieve/core/domain/retrieve_task/simd_compute_kernel.cpp:635-764, called from
 * ucm/sparse/kvstar/multistep.py:240-262) and extract_block_repre (multistep.py:279-316).
 *
 * ucmx_kvstar_block_repre: per block, keep d_pruned channels of every head (pruned_index: device int64
 * [H][d_pruned], or NULL to keep all) and average every `merge` consecutive tokens; result is IEEE half
 * [slot][T/merge][H][d_pruned] at out_slots[i] (or i).  The mean is rounded to bf16 first (the
 * reference averages in the cache's dtype), then converted to half.
 *
 * ucmx_kvstar_scores: for each request r, query rows q[q_offsets[r] .. q_offsets[r+1]) ([token][Hq][d_orig]
 * half, at most max_q_tokens tokens) vote on the request's candidate blocks (CSR req_offsets over slot_ids
 * into the representation table; slot_ids NULL = candidates are table rows 0..total-1):
 *   out[c] = sum over query rows of sum over the block's M positions of softmax_over_all_positions(q . k).
 * pruned_index: device int64 [n_req][H][d_pruned] (channels of d_orig), or NULL when d_pruned == d_orig.
 * Dot products are not scaled (as in the reference).  Follow with ucmx_topk_ragged on `out`.
 * workspace: device scratch of ucmx_kvstar_workspace_bytes(...) bytes, 16-byte aligned.
 * Shapes with H*d_pruned % 64 == 0, d_pruned % 16 == 0, M % 32 == 0, max_q_tokens*Hq/H <= 128 run on the
 * tensor cores (tcgen05); all others on a CUDA-core kernel with the same results to rounding. */
int32_t ucmx_kvstar_block_repre(const void* k_cache, const ucmx_kv_geometry* geom, const int32_t* block_ids,
                                const int32_t* out_slots, int64_t n_out_slots, int32_t n, const int64_t* pruned_index,
                                int32_t d_pruned, int32_t merge, void* reps_f16, ucmx_stream_t stream);
/* Which kernel ucmx_kvstar_scores runs for a shape: 0 = CUDA cores, 1 = tensor cores with one block per tile,
 * 2 = tensor cores with two blocks per instruction (host-side arithmetic only, nothing is launched). */
int32_t ucmx_kvstar_kernel_choice(int32_t n_slots, int32_t M, int32_t n_kv_heads, int32_t d_pruned,
                                  int32_t max_q_tokens, int32_t n_q_heads);
size_t ucmx_kvstar_workspace_bytes(int32_t total_blocks, int32_t n_req, int32_t max_q_tokens,
                                   int32_t n_q_heads, int32_t n_kv_heads);
int32_t ucmx_kvstar_scores(const void* reps_f16, int32_t n_slots, int32_t M, int32_t n_kv_heads,
                           int32_t d_pruned, const int32_t* req_offsets, const int32_t* slot_ids,
                           int32_t n_req, int32_t total, const void* q_f16, const int32_t* q_offsets,
                           int32_t max_q_tokens, int32_t n_q_heads, int32_t d_orig,
                           const int64_t* pruned_index, void* workspace, size_t workspace_bytes,
                           float* out_scores, ucmx_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* UCMX_H */

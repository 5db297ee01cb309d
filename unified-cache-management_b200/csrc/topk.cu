// Stage 3: per-request top-k over a ragged batch — one thread block per request.
//
// Selection is a most-significant-digit radix select (4 passes of 8 bits over order-preserving
// uint32 keys) that finds the k-th largest key exactly; an ordered compaction then emits every
// candidate above the threshold plus the first few equal to it, so ties always go to the lower
// position (what std::stable_sort gives in TopkBlockSelector::TopKImpl,
// ucm/sparse/gsa/offload_ops/src/select_topk_block.cpp:39-42).  Index-ascending output falls out of
// the compaction; score-descending output (RetrievalWorkerBackend's partial_sort order,
// ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp:182-189) adds a bitonic sort of the k winners
// in shared memory.  Scores were written by the scoring kernel a moment earlier and are re-read
// from L2, so the passes cost latency, not HBM traffic.
#include <cstdlib>

#include "common.cuh"

namespace ucmx {
namespace {

struct TopkParams {
    const uint32_t* scores;  // raw 32-bit words (fp32 or int32)
    int32_t is_float;
    const int32_t* offsets;
    const int32_t* k_per_req;
    int32_t start_win, end_win, window_mode, order;
    const int32_t* id_map;
    int32_t out_stride;
    const int32_t* out_offsets;
    int32_t* out_idx;
    uint32_t* out_scores;
    int32_t* out_counts;
    // tensor-parallel score exchange folded into the prologue (NULL / 0 on a single rank)
    const unsigned char* const* peer_bases;  // base of every rank's exchange buffer, peer-mapped
    int32_t world, my_rank;
    int64_t parts_offset;                    // byte offset of this round's partial scores inside a buffer
    uint32_t epoch;                          // value every rank's flag must have reached
    float* sum_out;                          // where the summed scores go (local), then read as `scores`
    int32_t* err;
};

constexpr uint32_t kPeerSpinLimit = 1u << 21;

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint32_t to_key(uint32_t bits, bool is_float)
{
    if (!is_float) return bits ^ 0x80000000u;
    if ((bits << 1) == 0) bits = 0;  // -0.0 == +0.0
    return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}
__device__ __forceinline__ uint32_t from_key(uint32_t key, bool is_float)
{
    if (!is_float) return key ^ 0x80000000u;
    return (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
}

// exclusive prefix sums of two small counts over the thread block, in thread order (one pass, two barriers);
// the block totals come back in tot_a / tot_b.  s_warp needs 64 ints.
__device__ __forceinline__ void block_excl_scan_pair(int a, int b, int* s_warp, int& before_a, int& before_b, int& tot_a, int& tot_b)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    int ia = a, ib = b;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int va = __shfl_up_sync(0xffffffffu, ia, o), vb = __shfl_up_sync(0xffffffffu, ib, o);
        if (lane >= o) {
            ia += va;
            ib += vb;
        }
    }
    if (lane == 31) {
        s_warp[warp] = ia;
        s_warp[32 + warp] = ib;
    }
    __syncthreads();
    int ba = 0, bb = 0, ta = 0, tb = 0;
    for (int w = 0; w < nwarp; ++w) {
        const int va = s_warp[w], vb = s_warp[32 + w];
        if (w < warp) {
            ba += va;
            bb += vb;
        }
        ta += va;
        tb += vb;
    }
    __syncthreads();
    before_a = ba + ia - a;
    before_b = bb + ib - b;
    tot_a = ta;
    tot_b = tb;
}

template <bool PEER>
__global__ void __launch_bounds__(1024) topk_ragged_kernel(TopkParams p)
{
    extern __shared__ __align__(16) unsigned long long s_sort[];  // score-descending order only
    __shared__ uint32_t s_hist[4][256];  // one histogram per radix pass, cleared once
    __shared__ int s_warp[64];
    __shared__ uint32_t s_prefix;
    __shared__ int s_krem;

    const int r = blockIdx.x;
    const int tid = threadIdx.x;
    const int base = __ldg(p.offsets + r);
    const int n = __ldg(p.offsets + r + 1) - base;
    const int k = __ldg(p.k_per_req + r);
    const bool is_float = p.is_float != 0;
    if (PEER) {
        // One-shot all-reduce fused into the selection: every rank scored its own KV heads into its
        // exchange buffer and then raised its flag on every peer; wait (bounded) for all flags, then
        // add the partial scores of this request straight out of the peers' memory, in rank order, so
        // that every rank computes bit-identical sums and therefore identical selections.
        if (tid < p.world) {
            const uint32_t* flag = reinterpret_cast<const uint32_t*>(p.peer_bases[p.my_rank]) + tid;
            bool ok = false;
            for (uint32_t it = 0; it < kPeerSpinLimit; ++it) {
                if ((int32_t)(ld_acquire_sys(flag) - p.epoch) >= 0) {
                    ok = true;
                    break;
                }
                __nanosleep(64);
            }
            if (!ok) {
                if (p.err) atomicExch(p.err, 4);   // a peer never signalled: sums below are incomplete
            }
        }
        __syncthreads();
        // The loads cross NVLink, so latency is what matters: up to eight ranks x eight elements per
        // thread are requested before the first one is used (L1 is bypassed: the data is a peer's).
        constexpr int kU = 4, kW = 8;
        for (int i0 = tid; i0 < n; i0 += blockDim.x * kU) {
            float acc[kU];
#pragma unroll
            for (int u = 0; u < kU; ++u) acc[u] = 0.0f;
            for (int r0 = 0; r0 < p.world; r0 += kW) {
                float v[kW][kU];
#pragma unroll
                for (int w = 0; w < kW; ++w) {
                    const bool live = r0 + w < p.world;
                    const float* part = reinterpret_cast<const float*>(p.peer_bases[live ? r0 + w : p.my_rank] + p.parts_offset);
#pragma unroll
                    for (int u = 0; u < kU; ++u) {
                        const int i = i0 + u * blockDim.x;
                        v[w][u] = (live && i < n) ? __ldcg(part + base + i) : 0.0f;
                    }
                }
#pragma unroll
                for (int w = 0; w < kW; ++w)
#pragma unroll
                    for (int u = 0; u < kU; ++u) acc[u] += v[w][u];   // rank order: the same sum on every rank
            }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int i = i0 + u * blockDim.x;
                if (i < n) p.sum_out[base + i] = acc[u];
            }
        }
        __syncthreads();
    }
    const uint32_t* sc = (PEER ? reinterpret_cast<const uint32_t*>(p.sum_out) : p.scores) + base;
    const int64_t orow = p.out_offsets ? (int64_t)__ldg(p.out_offsets + r) : (int64_t)r * p.out_stride;
    const int cap = p.out_offsets ? min(__ldg(p.out_offsets + r + 1) - (int)orow, p.out_stride) : p.out_stride;

    int lo = 0, hi = n, kk = 0, fstart = 0, fend = 0;
    bool identity = false;
    if (p.window_mode == UCMX_WIN_FORCE) {
        if (p.start_win + p.end_win >= n || k >= n || k == 0) {
            identity = true;
        } else {
            lo = p.start_win;
            hi = n - p.end_win;
            kk = max(k - p.start_win - p.end_win, 0);
            fstart = p.start_win;
            fend = p.end_win;
        }
    } else if (p.window_mode == UCMX_WIN_EXCLUDE) {
        lo = min(max(p.start_win, 0), n);
        hi = max(n - max(p.end_win, 0), lo);
        kk = (k >= n) ? (hi - lo) : min(max(k, 0), hi - lo);
    } else {
        kk = min(max(k, 0), n);
    }

    if (identity) {
        const int cnt = min(n, cap);
        for (int i = tid; i < cnt; i += blockDim.x) {
            p.out_idx[orow + i] = p.id_map ? __ldg(p.id_map + base + i) : i;
            if (p.out_scores) p.out_scores[orow + i] = sc[i];
        }
        if (tid == 0) p.out_counts[r] = cnt;
        return;
    }

    const int range = hi - lo;
    const bool all = kk >= range;  // everything in [lo, hi) is selected
    uint32_t T = 0;
    int need = 0;

    if (!all && kk > 0) {
        if (tid == 0) {
            s_prefix = 0;
            s_krem = kk;
        }
        for (int i = tid; i < 4 * 256; i += blockDim.x) (&s_hist[0][0])[i] = 0;
        __syncthreads();
        uint32_t mask = 0;
#pragma unroll 1
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            const uint32_t prefix = s_prefix;
            // (plain shared-memory adds: aggregating equal buckets within a warp by votes or match was measured slower)
            for (int i = lo + tid; i < hi; i += blockDim.x) {
                const uint32_t key = to_key(sc[i], is_float);
                if ((key & mask) == prefix) atomicAdd(&s_hist[pass][(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid < 32) {
                // lane l owns buckets 255-8l .. 248-8l, scanned from the largest digit down
                uint32_t h[8];
                uint32_t sum = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    h[j] = s_hist[pass][255 - 8 * tid - j];
                    sum += h[j];
                }
                uint32_t incl = sum;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
                    if (tid >= o) incl += v;
                }
                uint32_t before = incl - sum;
                const uint32_t krem = (uint32_t)s_krem;
                if (before < krem && krem <= incl) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (before < krem && krem <= before + h[j]) {
                            s_prefix = prefix | ((uint32_t)(255 - 8 * tid - j) << shift);
                            s_krem = (int)(krem - before);
                            before = 0xffffffffu;  // stop
                        } else if (before != 0xffffffffu) {
                            before += h[j];
                        }
                    }
                }
            }
            mask |= 0xffu << shift;
            __syncthreads();
        }
        T = s_prefix;
        need = s_krem;
    }

    // Ordered compaction over all positions.  Every thread owns a contiguous run of positions, counts what it will
    // surely take (forced windows, keys above the threshold) and its keys equal to the threshold; one scan of the two
    // counts over the block gives each run its first output place (ties go to the lowest positions: of the equal keys
    // before a run, the first `need` are taken), then the run is written out in order.
    const bool desc = p.order == UCMX_ORDER_SCORE_DESC;
    const int per = (n + (int)blockDim.x - 1) / (int)blockDim.x;
    const int i_begin = min(tid * per, n), i_end = min(i_begin + per, n);
    const bool ranged = kk > 0;
    int sure = 0, ties = 0;
    for (int i = i_begin; i < i_end; ++i) {
        const bool forced = (i < fstart) || (i >= n - fend);
        if (forced) {
            ++sure;
        } else if (ranged && i >= lo && i < hi) {
            if (all) {
                ++sure;
            } else {
                const uint32_t key = to_key(sc[i], is_float);
                sure += key > T;
                ties += key == T;
            }
        }
    }
    int sure_before, ties_before, sure_total, ties_total;
    block_excl_scan_pair(sure, ties, s_warp, sure_before, ties_before, sure_total, ties_total);
    int pos = sure_before + min(ties_before, need);
    int tie_rank = ties_before;
    for (int i = i_begin; i < i_end; ++i) {
        const bool forced = (i < fstart) || (i >= n - fend);
        const bool in_range = i >= lo && i < hi;
        if (!forced && !(ranged && in_range)) continue;
        const uint32_t key = to_key(sc[i], is_float);
        bool take = forced;
        if (!forced) {
            if (all) take = true;
            else if (key > T) take = true;
            else if (key == T) take = tie_rank++ < need;
        }
        if (take) {
            if (pos < cap) {
                if (desc) {
                    s_sort[pos] = ((unsigned long long)key << 32) | (unsigned long long)(~(uint32_t)i);
                } else {
                    p.out_idx[orow + pos] = p.id_map ? __ldg(p.id_map + base + i) : i;
                    if (p.out_scores) p.out_scores[orow + pos] = from_key(key, is_float);
                }
            }
            ++pos;
        }
    }
    const int out_base = sure_total + min(ties_total, need);
    const int cnt = min(out_base, cap);
    if (tid == 0) p.out_counts[r] = cnt;

    if (desc && cnt > 0 && cnt <= 256) {
        // few winners: every winner counts how many beat it (keys are unique), which is its place
        __syncthreads();
        unsigned long long mine = 0;
        int rank = 0;
        if (tid < cnt) {
            mine = s_sort[tid];
            for (int j = 0; j < cnt; ++j) rank += s_sort[j] > mine;
        }
        if (tid < cnt) {
            const int i = (int)(~(uint32_t)(mine & 0xffffffffull));
            p.out_idx[orow + rank] = p.id_map ? __ldg(p.id_map + base + i) : i;
            if (p.out_scores) p.out_scores[orow + rank] = from_key((uint32_t)(mine >> 32), is_float);
        }
    } else if (desc && cnt > 0) {
        int P = 1;
        while (P < cnt) P <<= 1;
        for (int i = cnt + tid; i < P; i += blockDim.x) s_sort[i] = 0ull;
        __syncthreads();
        // Bitonic network, one thread per compare-exchange: pair t of a stage with distance j is the elements
        // (t / j) * 2j + t % j and j further up.  For j <= 32 the 32 pairs of a warp lie in 64 consecutive elements
        // that no other warp touches, so between two such stages the warp alone has to meet; the block meets only
        // around the stages that reach further.
        for (int k2 = 2; k2 <= P; k2 <<= 1) {
            for (int j = k2 >> 1; j > 0; j >>= 1) {
                for (int t = tid; t < (P >> 1); t += blockDim.x) {
                    const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1)), ixj = i | j;
                    const unsigned long long a = s_sort[i], b = s_sort[ixj];
                    const bool up = (i & k2) == 0;  // descending overall
                    if (up ? (a < b) : (a > b)) {
                        s_sort[i] = b;
                        s_sort[ixj] = a;
                    }
                }
                const int j_next = j > 1 ? (j >> 1) : k2;          // first distance of the next merge is k2
                if (j > 32 || j_next > 32) __syncthreads();
                else __syncwarp();
            }
        }
        __syncthreads();
        for (int j = tid; j < cnt; j += blockDim.x) {
            const unsigned long long v = s_sort[j];
            const int i = (int)(~(uint32_t)(v & 0xffffffffull));
            p.out_idx[orow + j] = p.id_map ? __ldg(p.id_map + base + i) : i;
            if (p.out_scores) p.out_scores[orow + j] = from_key((uint32_t)(v >> 32), is_float);
        }
    }
}

}  // namespace
}  // namespace ucmx

namespace ucmx {
static int32_t topk_launch(const void* scores, int32_t score_dtype, const int32_t* req_offsets,
                                    const int32_t* k_per_req, int32_t n_req, int32_t start_win, int32_t end_win,
                                    int32_t window_mode, int32_t order, const int32_t* id_map, int32_t out_stride,
                                    const int32_t* out_offsets, int32_t* out_idx, void* out_scores,
                                    int32_t* out_counts, const unsigned char* const* peer_bases, int32_t world,
                                    int32_t my_rank, int64_t parts_offset, uint32_t epoch, float* sum_out,
                                    ucmx_stream_t stream)
{
    if (n_req < 0) return UCMX_EPARAM;
    if (n_req == 0) return UCMX_OK;
    if (!scores || !req_offsets || !k_per_req || !out_idx || !out_counts) return UCMX_EPARAM;
    if (score_dtype != UCMX_DT_F32 && score_dtype != UCMX_DT_I32) return UCMX_EPARAM;
    if (window_mode < 0 || window_mode > 2 || (order != 0 && order != 1)) return UCMX_EPARAM;
    if (start_win < 0 || end_win < 0 || out_stride < 1) return UCMX_EPARAM;
    size_t smem = 0;
    if (order == UCMX_ORDER_SCORE_DESC) {
        if (out_stride > 8192) return UCMX_EUNSUPPORTED;
        int P = 1;
        while (P < out_stride) P <<= 1;
        smem = (size_t)P * 8;
    }
    TopkParams p;
    p.scores = (const uint32_t*)scores;
    p.is_float = score_dtype == UCMX_DT_F32;
    p.offsets = req_offsets;
    p.k_per_req = k_per_req;
    p.start_win = start_win;
    p.end_win = end_win;
    p.window_mode = window_mode;
    p.order = order;
    p.id_map = id_map;
    p.out_stride = out_stride;
    p.out_offsets = out_offsets;
    p.out_idx = out_idx;
    p.out_scores = (uint32_t*)out_scores;
    p.out_counts = out_counts;
    p.peer_bases = peer_bases;
    p.world = world;
    p.my_rank = my_rank;
    p.parts_offset = parts_offset;
    p.epoch = epoch;
    p.sum_out = sum_out;
    p.err = peer_bases ? error_word() : nullptr;
    void (*kern)(TopkParams) = peer_bases ? topk_ragged_kernel<true> : topk_ragged_kernel<false>;
    if (smem > 48 * 1024) UCMX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // block size: enough threads for about two candidates each (the host does not know the ragged
    // sizes, only the output width, so k is the hint), never fewer than the rank sort needs
    int threads = 1024;
    if (out_stride <= 64) threads = 512;
    if (const char* e = getenv("UCMX_TOPK_THREADS")) {  // tuning knob
        const int v = atoi(e);
        if (v == 256 || v == 512 || v == 1024) threads = v;
    }
    kern<<<n_req, threads, smem, (cudaStream_t)stream>>>(p);
    UCMX_LAUNCH_CHECK("topk_ragged_kernel");
    return UCMX_OK;
}
}  // namespace ucmx

extern "C" int32_t ucmx_topk_ragged(const void* scores, int32_t score_dtype, const int32_t* req_offsets,
                                    const int32_t* k_per_req, int32_t n_req, int32_t start_win, int32_t end_win,
                                    int32_t window_mode, int32_t order, const int32_t* id_map, int32_t out_stride,
                                    const int32_t* out_offsets, int32_t* out_idx, void* out_scores,
                                    int32_t* out_counts, ucmx_stream_t stream)
{
    return ucmx::topk_launch(scores, score_dtype, req_offsets, k_per_req, n_req, start_win, end_win, window_mode, order,
                             id_map, out_stride, out_offsets, out_idx, out_scores, out_counts, nullptr, 1, 0, 0, 0, nullptr,
                             stream);
}

namespace ucmx {
namespace {
__global__ void peer_signal_kernel(unsigned char* const* peer_bases, int world, int my_rank, uint32_t epoch)
{
    // everything this rank wrote before (its partial scores) must be visible to a peer that sees the flag
    __threadfence_system();
    const int r = threadIdx.x;
    if (r < world) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(peer_bases[r]) + my_rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
    }
}
}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_peer_signal(void* const* peer_bases, int32_t world, int32_t my_rank, uint32_t epoch,
                                    ucmx_stream_t stream)
{
    if (!peer_bases || world < 1 || world > 32 || my_rank < 0 || my_rank >= world) return UCMX_EPARAM;
    ucmx::peer_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned char* const*)peer_bases, world, my_rank, epoch);
    UCMX_LAUNCH_CHECK("peer_signal_kernel");
    return UCMX_OK;
}

extern "C" int32_t ucmx_topk_ragged_peer_sum(void* const* peer_bases, int32_t world, int32_t my_rank,
                                             int64_t parts_offset_bytes, uint32_t epoch, float* summed_scores,
                                             const int32_t* req_offsets, const int32_t* k_per_req, int32_t n_req,
                                             int32_t start_win, int32_t end_win, int32_t window_mode, int32_t order,
                                             const int32_t* id_map, int32_t out_stride, const int32_t* out_offsets,
                                             int32_t* out_idx, float* out_scores, int32_t* out_counts,
                                             ucmx_stream_t stream)
{
    if (!peer_bases || !summed_scores || world < 1 || world > 32 || my_rank < 0 || my_rank >= world ||
        parts_offset_bytes < 128 || (parts_offset_bytes & 15))
        return UCMX_EPARAM;
    return ucmx::topk_launch(summed_scores, UCMX_DT_F32, req_offsets, k_per_req, n_req, start_win, end_win, window_mode,
                             order, id_map, out_stride, out_offsets, out_idx, out_scores, out_counts,
                             (const unsigned char* const*)peer_bases, world, my_rank, parts_offset_bytes, epoch,
                             summed_scores, stream);
}

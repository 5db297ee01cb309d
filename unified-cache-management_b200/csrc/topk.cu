// Stage 3: per-request top-k over a ragged batch — one thread block per request.
//
// Selection is a most-significant-digit radix select over order-preserving uint32 keys that finds
// the k-th largest key exactly.  Digits are 12, 12 and 8 bits wide: the leading digit of an fp32
// score then holds the sign, the exponent and three mantissa bits, which spreads scores of one
// magnitude over many buckets (with 8-bit digits nearly all of them land in two or three buckets
// and their shared-memory adds serialise).  A request of up to eight candidates per thread is read
// once and kept in registers for all passes.  An ordered compaction then emits every candidate
// above the threshold plus the first few equal to it, so ties always go to the lower position
// (what std::stable_sort gives in TopkBlockSelector::TopKImpl,
// ucm/sparse/gsa/offload_ops/src/select_topk_block.cpp:39-42).  Index-ascending output falls out of
// the compaction; score-descending output (RetrievalWorkerBackend's partial_sort order,
// ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp:182-189) adds a sort of the k winners in shared
// memory.  Scores were written by the scoring kernel a moment earlier and come from L2.
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
    // tensor-parallel score exchange folded into the prologue (px.world == 0 on a single rank)
    PeerPush px;
    float* sum_out;          // where the summed scores go (local); needed beyond 8 candidates per thread
    int32_t* err;
};

constexpr uint32_t kPeerSpinLimit = 1u << 21;
constexpr int kKeysPerThread = 8;          // candidates a thread keeps in registers
constexpr int kHistWords = 4096 + 4096 + 256;
constexpr int kListMax = 128;              // keys sharing the digits fixed so far that are ranked directly
constexpr int kSelectWords = kHistWords + 512 + 2 * kListMax;   // histograms, partial sums, the list (32-bit words)

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

// exclusive prefix sums of two counts over the thread block, in thread order (two barriers); the block totals
// come back in tot_a / tot_b.  Both counts travel in one 64-bit word.  s_warp needs 32 entries.
__device__ __forceinline__ void block_excl_scan_pair(int a, int b, unsigned long long* s_warp, int& before_a, int& before_b,
                                                     int& tot_a, int& tot_b)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    const unsigned long long mine = (unsigned long long)(uint32_t)a | ((unsigned long long)(uint32_t)b << 32);
    unsigned long long incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    // every warp scans the (at most 32) warp totals by itself
    const unsigned long long wt = lane < nwarp ? s_warp[lane] : 0ull;
    unsigned long long winc = wt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long v = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += v;
    }
    const unsigned long long total = __shfl_sync(0xffffffffu, winc, 31);
    const unsigned long long wbefore = __shfl_sync(0xffffffffu, winc - wt, warp);
    __syncthreads();
    const unsigned long long before = wbefore + incl - mine;
    before_a = (int)(uint32_t)before;
    before_b = (int)(before >> 32);
    tot_a = (int)(uint32_t)total;
    tot_b = (int)(total >> 32);
}

// Inclusive scan of one value per lane.
__device__ __forceinline__ uint32_t warp_incl_scan(uint32_t v)
{
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
    }
    return v;
}

// Which bucket holds the krem-th largest key of a histogram (digits counted from the top).  Called by the whole
// thread block: every thread adds up runs of eight buckets into s_part (buckets/8 partial sums), then warp 0
// narrows the search in three steps of one shuffle scan each - which 32nd of the partial sums, which partial sum,
// which bucket - and leaves the bucket, the keys above it and the keys in it in s_found[0..2].  Two barriers.
__device__ __forceinline__ void block_find_bucket(const uint32_t* hist, int buckets, int krem, uint32_t* s_part, int* s_found)
{
    const int tid = threadIdx.x, lane = tid & 31;
    const int parts = buckets >> 3;                         // 512 or 32
    for (int t = tid; t < parts; t += blockDim.x) {
        uint32_t sum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += hist[buckets - 1 - (t * 8 + ((j + t) & 7))];   // rotated: fewer bank conflicts
        s_part[t] = sum;
    }
    __syncthreads();
    if (tid < 32) {
        const int per_lane = parts >> 5;                    // 16 or 1
        uint32_t sum = 0;
        for (int j = 0; j < per_lane; ++j) sum += s_part[lane * per_lane + ((j + lane) % per_lane)];
        const uint32_t incl = warp_incl_scan(sum);
        const unsigned holds = __ballot_sync(0xffffffffu, incl - sum < (uint32_t)krem && (uint32_t)krem <= incl);
        const int owner = holds ? __ffs(holds) - 1 : 31;    // (krem never exceeds the histogram's total)
        uint32_t above = __shfl_sync(0xffffffffu, incl - sum, owner);
        // which partial sum of the owner's
        const uint32_t pv = lane < per_lane ? s_part[owner * per_lane + lane] : 0u;
        const uint32_t pincl = warp_incl_scan(pv);
        const unsigned ph = __ballot_sync(0xffffffffu, lane < per_lane && above + pincl - pv < (uint32_t)krem &&
                                                           (uint32_t)krem <= above + pincl);
        const int pl = ph ? __ffs(ph) - 1 : per_lane - 1;
        above += __shfl_sync(0xffffffffu, pincl - pv, pl);
        const int part = owner * per_lane + pl;
        // which of its eight buckets
        const uint32_t bv = lane < 8 ? hist[buckets - 1 - (part * 8 + lane)] : 0u;
        const uint32_t bincl = warp_incl_scan(bv);
        const unsigned bh = __ballot_sync(0xffffffffu, lane < 8 && above + bincl - bv < (uint32_t)krem &&
                                                           (uint32_t)krem <= above + bincl);
        const int bl = bh ? __ffs(bh) - 1 : 7;
        above += __shfl_sync(0xffffffffu, bincl - bv, bl);
        const uint32_t cnt = __shfl_sync(0xffffffffu, bv, bl);
        if (lane == 0) {
            s_found[0] = buckets - 1 - (part * 8 + bl);
            s_found[1] = (int)above;
            s_found[2] = (int)cnt;
        }
    }
    __syncthreads();
}

template <bool PEER>
__global__ void __launch_bounds__(1024) topk_ragged_kernel(TopkParams p)
{
    extern __shared__ __align__(16) unsigned char s_dyn[];
    uint32_t* s_hist = reinterpret_cast<uint32_t*>(s_dyn);                                    // three histograms
    unsigned long long* s_sort = reinterpret_cast<unsigned long long*>(s_dyn + kSelectWords * 4);  // score-descending order only
    __shared__ unsigned long long s_warp[32];
    __shared__ uint32_t s_prefix;
    __shared__ int s_krem, s_cnt, s_found[3];

    const int r = blockIdx.x;
    const int tid = threadIdx.x;
    // A scoring kernel launched for an early start behind this one may begin now: it stores nothing before this
    // kernel has ended.  (Not with a peer exchange: that scoring kernel is never launched early.)
    if (!PEER) early_start_allow();
    // This kernel itself is launched so that its thread blocks may be placed while the kernel ahead of it (the
    // scoring) is still running; everything it reads comes from that kernel, so it waits for its end right here.
    early_start_wait();
    const int base = __ldg(p.offsets + r);
    const int n = __ldg(p.offsets + r + 1) - base;
    const int k = __ldg(p.k_per_req + r);
    const bool is_float = p.is_float != 0;

    // every thread owns a contiguous run of positions; up to kKeysPerThread of them live in registers
    const int per = (n + (int)blockDim.x - 1) / (int)blockDim.x;
    const int i_begin = min(tid * per, n), i_end = min(i_begin + per, n);
    const bool in_regs = per <= kKeysPerThread;
    uint32_t kreg[kKeysPerThread];

    const uint32_t* sc = p.scores + base;
    if (PEER) {
        // The all-reduce of partial scores ends here: every rank's scoring kernel has stored its part into this
        // rank's inbox and raised its flag; wait (bounded) for all flags, then add the parts in rank order, so
        // that every rank forms bit-identical sums and therefore identical selections.
        const unsigned char* mine = p.px.bases[p.px.my_rank];
        const uint32_t round = *reinterpret_cast<const volatile uint32_t*>(mine + kPeerRoundOffset);
        if (tid < p.px.world) {
            const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine) + tid;
            bool ok = false;
            for (uint32_t it = 0; it < kPeerSpinLimit; ++it) {
                if ((int32_t)(ld_acquire_sys_u32(flag) - round) >= 0) {
                    ok = true;
                    break;
                }
                __nanosleep(64);
            }
            if (!ok && p.err) atomicExch(p.err, 4);   // a peer never delivered: the sums below are incomplete
        }
        __syncthreads();
        const float* inbox = reinterpret_cast<const float*>(mine + peer_inbox_offset(p.px, round, 0)) + base;
        const int64_t part = p.px.part_bytes / 4;
        if (in_regs) {
#pragma unroll
            for (int j = 0; j < kKeysPerThread; ++j) {
                const int i = i_begin + j;
                float acc = 0.0f;
                if (j < per && i < i_end) {
                    for (int t = 0; t < p.px.world; ++t) acc += __ldcg(inbox + (int64_t)t * part + i);
                    if (p.sum_out) p.sum_out[base + i] = acc;
                }
                kreg[j] = to_key(__float_as_uint(acc), true);
            }
        } else {
            for (int i = tid; i < n; i += blockDim.x) {
                float acc = 0.0f;
                for (int t = 0; t < p.px.world; ++t) acc += __ldcg(inbox + (int64_t)t * part + i);
                p.sum_out[base + i] = acc;
            }
            __syncthreads();
            sc = reinterpret_cast<const uint32_t*>(p.sum_out) + base;
        }
    } else if (in_regs) {
#pragma unroll
        for (int j = 0; j < kKeysPerThread; ++j) {
            const int i = i_begin + j;
            kreg[j] = (j < per && i < i_end) ? to_key(__ldg(sc + i), is_float) : 0u;
        }
    }
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

    // key of position i (inside this thread's run when the keys are in registers)
    auto key_of = [&](int i, int j) -> uint32_t { return in_regs ? kreg[j] : to_key(sc[i], is_float); };

    if (identity) {
        const int cnt = min(n, cap);
        if (in_regs) {
#pragma unroll
            for (int j = 0; j < kKeysPerThread; ++j) {
                const int i = i_begin + j;
                if (j < per && i < i_end && i < cnt) {
                    p.out_idx[orow + i] = p.id_map ? __ldg(p.id_map + base + i) : i;
                    if (p.out_scores) p.out_scores[orow + i] = from_key(kreg[j], is_float);
                }
            }
        } else {
            for (int i = tid; i < cnt; i += blockDim.x) {
                p.out_idx[orow + i] = p.id_map ? __ldg(p.id_map + base + i) : i;
                if (p.out_scores) p.out_scores[orow + i] = sc[i];
            }
        }
        if (tid == 0) p.out_counts[r] = cnt;
        return;
    }

    const int range = hi - lo;
    const bool all = kk >= range;  // everything in [lo, hi) is selected
    uint32_t T = 0;
    int need = 0;

    if (!all && kk > 0) {
        // Digit passes from the top (12, 12, 8 bits).  After a pass, if only a few keys share the digits fixed so
        // far (the usual case after the first pass), they are listed and ranked directly instead of histogrammed
        // again; a crowded digit (heavy ties, a narrow score range) takes the next pass.
        uint32_t* hist = s_hist;
        uint32_t* s_part = s_hist + kHistWords;                                               // 512 partial sums
        unsigned long long* s_list = reinterpret_cast<unsigned long long*>(s_part + 512);     // kListMax entries
        uint32_t mask = 0, prefix = 0;
        int krem = kk;
        bool done = false;
#pragma unroll 1
        for (int pass = 0; pass < 3 && !done; ++pass) {
            const int shift = pass == 0 ? 20 : (pass == 1 ? 8 : 0);
            const int buckets = pass == 2 ? 256 : 4096;
            for (int i = tid; i < buckets; i += blockDim.x) hist[i] = 0;
            if (tid == 0) s_cnt = 0;
            __syncthreads();
            if (in_regs) {
#pragma unroll
                for (int j = 0; j < kKeysPerThread; ++j) {
                    const int i = i_begin + j;
                    if (j < per && i < i_end && i >= lo && i < hi && (kreg[j] & mask) == prefix)
                        atomicAdd(&hist[(kreg[j] >> shift) & (uint32_t)(buckets - 1)], 1u);
                }
            } else {
                for (int i = lo + tid; i < hi; i += blockDim.x) {
                    const uint32_t key = to_key(sc[i], is_float);
                    if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & (uint32_t)(buckets - 1)], 1u);
                }
            }
            __syncthreads();
            block_find_bucket(hist, buckets, krem, s_part, s_found);
            prefix |= (uint32_t)s_found[0] << shift;
            krem -= s_found[1];
            const int in_bucket = s_found[2];
            mask |= (uint32_t)(buckets - 1) << shift;
            if (pass == 2) {
                T = prefix;
                need = krem;
                done = true;
            } else if (in_bucket <= kListMax) {
                // list the keys that share the digits so far; each warp takes listed keys in turn and its lanes
                // count together how many of the others beat it - the one beaten by exactly krem-1 is the threshold
                if (in_regs) {
#pragma unroll
                    for (int j = 0; j < kKeysPerThread; ++j) {
                        const int i = i_begin + j;
                        if (j < per && i < i_end && i >= lo && i < hi && (kreg[j] & mask) == prefix)
                            s_list[atomicAdd(&s_cnt, 1)] = ((unsigned long long)kreg[j] << 32) | (uint32_t)(~(uint32_t)i);
                    }
                } else {
                    for (int i = lo + tid; i < hi; i += blockDim.x) {
                        const uint32_t key = to_key(sc[i], is_float);
                        if ((key & mask) == prefix)
                            s_list[atomicAdd(&s_cnt, 1)] = ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)i);
                    }
                }
                __syncthreads();
                const int lane = tid & 31, warp = tid >> 5, nwarp = (int)blockDim.x >> 5;
                for (int e = warp; e < in_bucket; e += nwarp) {
                    const unsigned long long me = s_list[e];
                    int beaten_by = 0, greater_key = 0;
                    for (int j = lane; j < in_bucket; j += 32) {
                        const unsigned long long o = s_list[j];
                        beaten_by += o > me;                              // larger key, or equal key at a lower position
                        greater_key += (uint32_t)(o >> 32) > (uint32_t)(me >> 32);
                    }
                    beaten_by = warp_sum_i(beaten_by);
                    greater_key = warp_sum_i(greater_key);
                    if (lane == 0 && beaten_by == krem - 1) {
                        s_prefix = (uint32_t)(me >> 32);
                        s_krem = krem - greater_key;
                    }
                }
                __syncthreads();
                T = s_prefix;
                need = s_krem;
                done = true;
            }
            hist += buckets;
        }
    }

    // Ordered compaction over all positions.  Every thread owns a contiguous run of positions, counts what it will
    // surely take (forced windows, keys above the threshold) and its keys equal to the threshold; one scan of the two
    // counts over the block gives each run its first output place (ties go to the lowest positions: of the equal keys
    // before a run, the first `need` are taken), then the run is written out in order.
    const bool desc = p.order == UCMX_ORDER_SCORE_DESC;
    const bool ranged = kk > 0;
    int sure = 0, ties = 0;
    auto count_one = [&](int i, uint32_t key) {
        const bool forced = (i < fstart) || (i >= n - fend);
        if (forced) {
            ++sure;
        } else if (ranged && i >= lo && i < hi) {
            if (all) {
                ++sure;
            } else {
                sure += key > T;
                ties += key == T;
            }
        }
    };
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kKeysPerThread; ++j)
            if (j < per && i_begin + j < i_end) count_one(i_begin + j, kreg[j]);
    } else {
        for (int i = i_begin; i < i_end; ++i) count_one(i, to_key(sc[i], is_float));
    }
    int sure_before, ties_before, sure_total, ties_total;
    block_excl_scan_pair(sure, ties, s_warp, sure_before, ties_before, sure_total, ties_total);
    int pos = sure_before + min(ties_before, need);
    int tie_rank = ties_before;
    // take: is position i part of the output; advances the tie counter
    auto takes = [&](int i, uint32_t key) -> bool {
        const bool forced = (i < fstart) || (i >= n - fend);
        if (forced) return true;
        if (!(ranged && i >= lo && i < hi)) return false;
        if (all || key > T) return true;
        if (key == T) return tie_rank++ < need;
        return false;
    };
    if (in_regs) {
        // places first (registers only), then every id-map load of the run at once, then the stores
        int opos[kKeysPerThread];
#pragma unroll
        for (int j = 0; j < kKeysPerThread; ++j) {
            opos[j] = -1;
            if (j < per && i_begin + j < i_end && takes(i_begin + j, kreg[j])) {
                if (pos < cap) opos[j] = pos;
                ++pos;
            }
        }
        if (desc) {
#pragma unroll
            for (int j = 0; j < kKeysPerThread; ++j)
                if (opos[j] >= 0)
                    s_sort[opos[j]] = ((unsigned long long)kreg[j] << 32) | (unsigned long long)(~(uint32_t)(i_begin + j));
        } else {
            int ids[kKeysPerThread];
#pragma unroll
            for (int j = 0; j < kKeysPerThread; ++j)
                ids[j] = (opos[j] >= 0 && p.id_map) ? __ldg(p.id_map + base + i_begin + j) : i_begin + j;
#pragma unroll
            for (int j = 0; j < kKeysPerThread; ++j) {
                if (opos[j] >= 0) {
                    p.out_idx[orow + opos[j]] = ids[j];
                    if (p.out_scores) p.out_scores[orow + opos[j]] = from_key(kreg[j], is_float);
                }
            }
        }
    } else {
        for (int i = i_begin; i < i_end; ++i) {
            const uint32_t key = to_key(sc[i], is_float);
            if (!takes(i, key)) continue;
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
                           const int32_t* out_offsets, int32_t* out_idx, void* out_scores, int32_t* out_counts,
                           const PeerPush& px, float* sum_out, ucmx_stream_t stream)
{
    if (n_req < 0) return UCMX_EPARAM;
    if (n_req == 0) return UCMX_OK;
    if ((!scores && px.world == 0) || !req_offsets || !k_per_req || !out_idx || !out_counts) return UCMX_EPARAM;
    if (score_dtype != UCMX_DT_F32 && score_dtype != UCMX_DT_I32) return UCMX_EPARAM;
    if (window_mode < 0 || window_mode > 2 || (order != 0 && order != 1)) return UCMX_EPARAM;
    if (start_win < 0 || end_win < 0 || out_stride < 1) return UCMX_EPARAM;
    size_t smem = (size_t)kSelectWords * 4;
    if (order == UCMX_ORDER_SCORE_DESC) {
        if (out_stride > 8192) return UCMX_EUNSUPPORTED;
        int P = 1;
        while (P < out_stride) P <<= 1;
        smem += (size_t)P * 8;
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
    p.px = px;
    p.sum_out = sum_out;
    p.err = px.world > 0 ? error_word() : nullptr;
    void (*kern)(TopkParams) = px.world > 0 ? topk_ragged_kernel<true> : topk_ragged_kernel<false>;
    if (smem > 48 * 1024) UCMX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // block size: enough threads for a few candidates each (the host does not know the ragged sizes, only the
    // output width, so k is the hint), never fewer than the rank sort of up to 256 winners needs
    const int threads = out_stride <= 64 ? 512 : 1024;     // measured on 64 requests of ~520 candidates: 512 threads 6.9 us, 256 7.2, 128 8.3
    if (px.world == 0) {
        // (the launch latency of this small kernel is a fifth of its run time: let it overlap the tail of the scoring)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)n_req);
        cfg.blockDim = dim3((unsigned)threads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        UCMX_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    } else {
        kern<<<n_req, threads, smem, (cudaStream_t)stream>>>(p);
    }
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
    ucmx::PeerPush none{nullptr, 0, 0, 0};
    return ucmx::topk_launch(scores, score_dtype, req_offsets, k_per_req, n_req, start_win, end_win, window_mode, order,
                             id_map, out_stride, out_offsets, out_idx, out_scores, out_counts, none, nullptr, stream);
}

extern "C" size_t ucmx_peer_exchange_bytes(int32_t world, int64_t n_scores)
{
    if (world < 1 || n_scores < 0) return 0;
    return (size_t)ucmx::kPeerHeaderBytes + (size_t)2 * (size_t)world * (size_t)ucmx::peer_part_bytes(n_scores);
}

extern "C" int32_t ucmx_topk_ragged_peer_sum(const ucmx_peer_exchange* exchange, float* summed_scores,
                                             const int32_t* req_offsets, const int32_t* k_per_req, int32_t n_req,
                                             int32_t total, int32_t start_win, int32_t end_win, int32_t window_mode,
                                             int32_t order, const int32_t* id_map, int32_t out_stride,
                                             const int32_t* out_offsets, int32_t* out_idx, float* out_scores,
                                             int32_t* out_counts, ucmx_stream_t stream)
{
    using namespace ucmx;
    if (!exchange || !exchange->bases || exchange->world < 1 || exchange->world > 32 || exchange->my_rank < 0 ||
        exchange->my_rank >= exchange->world || total < 0 || exchange->n_scores < total || !summed_scores)
        return UCMX_EPARAM;
    PeerPush px{(unsigned char* const*)exchange->bases, exchange->world, exchange->my_rank,
                peer_part_bytes(exchange->n_scores)};
    return topk_launch(summed_scores, UCMX_DT_F32, req_offsets, k_per_req, n_req, start_win, end_win, window_mode, order,
                       id_map, out_stride, out_offsets, out_idx, out_scores, out_counts, px, summed_scores, stream);
}
